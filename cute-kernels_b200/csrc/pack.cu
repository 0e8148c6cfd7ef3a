// pack_sequence / unpack_sequence: rows of a padded batch [B, S, row] <-> the packed token list [total, row]
// described by cu_seqlens (B + 1 prefix sums of the sequence lengths), padding on the left or on the right.
// Pure row copies, HBM-bound: one warp per (sequence, position) of the padded layout, 128-bit accesses.
// Unpacking writes the padding rows as zeros in the same pass, so the output needs no separate zero-fill.
#include "common.cuh"

namespace fmab {

constexpr int kPackWarps = 8;

template <typename IndexT, bool kPack>
__global__ void __launch_bounds__(kPackWarps * 32)
pack_unpack_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, const IndexT* __restrict__ cu_seqlens,
                   int64_t B, int64_t S, int64_t total, int row_vecs, bool pad_left) {
    const int lane = threadIdx.x & 31;
    const int64_t pos = static_cast<int64_t>(blockIdx.x) * kPackWarps + (threadIdx.x >> 5);  // row of the padded layout
    if (pos >= B * S) return;
    const int64_t b = pos / S, s = pos - b * S;
    const int64_t start = static_cast<int64_t>(cu_seqlens[b]);
    int64_t len = static_cast<int64_t>(cu_seqlens[b + 1]) - start;
    len = len < 0 ? 0 : (len > S ? S : len);  // a malformed cu_seqlens never becomes a bad address
    const int64_t pad = S - len;
    const bool is_token = pad_left ? (s >= pad) : (s < len);
    const int64_t t = start + (pad_left ? s - pad : s);  // row of the packed layout
    const bool ok = is_token && t >= 0 && t < total;
    if (kPack) {
        if (!ok) return;
        const uint4* from = src + pos * row_vecs;
        uint4* to = dst + t * row_vecs;
        for (int i = lane; i < row_vecs; i += 32) to[i] = ld_stream_16(from + i);
    } else {
        uint4* to = dst + pos * row_vecs;
        if (ok) {
            const uint4* from = src + t * row_vecs;
            for (int i = lane; i < row_vecs; i += 32) to[i] = ld_stream_16(from + i);
        } else {
            for (int i = lane; i < row_vecs; i += 32) to[i] = make_uint4(0, 0, 0, 0);
        }
    }
}

static int launch_pack(const void* src, void* dst, const void* cu_seqlens, int32_t index_bytes, int64_t B, int64_t S,
                       int64_t total, int64_t row_bytes, int32_t pad_left, bool pack, cudaStream_t s) {
    FMAB_REQUIRE(B >= 0 && S >= 0 && total >= 0 && B * S < (1LL << 40), FMA_B200_ERR_BAD_ARG, "B=%lld S=%lld total=%lld",
                 (long long)B, (long long)S, (long long)total);
    FMAB_REQUIRE(row_bytes > 0 && row_bytes % 16 == 0 && row_bytes < (1LL << 31), FMA_B200_ERR_BAD_ARG,
                 "row of %lld bytes is not a positive multiple of 16", (long long)row_bytes);
    FMAB_REQUIRE(index_bytes == 4 || index_bytes == 8, FMA_B200_ERR_UNSUPPORTED, "cu_seqlens must hold 32- or 64-bit integers");
    if (B * S == 0) return FMA_B200_OK;
    FMAB_REQUIRE(cu_seqlens != nullptr && dst != nullptr && (src != nullptr || total == 0), FMA_B200_ERR_BAD_ARG, "NULL pointer");
    FMAB_REQUIRE(aligned16(src) && aligned16(dst), FMA_B200_ERR_BAD_ARG, "pointers not 16-byte aligned");
    const int64_t blocks = (B * S + kPackWarps - 1) / kPackWarps;
    FMAB_REQUIRE(blocks < (1LL << 31), FMA_B200_ERR_BAD_ARG, "grid too large");
    const unsigned grid = static_cast<unsigned>(blocks);
    const int row_vecs = static_cast<int>(row_bytes / 16);
    const uint4* from = static_cast<const uint4*>(src);
    uint4* to = static_cast<uint4*>(dst);
    const bool left = pad_left != 0;
#define FMAB_PACK(IndexT, kPack) \
    pack_unpack_kernel<IndexT, kPack><<<grid, kPackWarps * 32, 0, s>>>(from, to, static_cast<const IndexT*>(cu_seqlens), B, S, total, row_vecs, left)
    if (index_bytes == 4) {
        if (pack) FMAB_PACK(uint32_t, true); else FMAB_PACK(uint32_t, false);
    } else {
        if (pack) FMAB_PACK(int64_t, true); else FMAB_PACK(int64_t, false);
    }
#undef FMAB_PACK
    return check_launch(pack ? "pack_sequence" : "unpack_sequence");
}

}  // namespace fmab

extern "C" {

int fma_b200_pack_sequence(const void* padded, void* packed, const void* cu_seqlens, int32_t index_bytes, int64_t B,
                           int64_t S, int64_t total, int64_t row_bytes, int32_t pad_left, void* stream) {
    return fmab::launch_pack(padded, packed, cu_seqlens, index_bytes, B, S, total, row_bytes, pad_left, true,
                             static_cast<cudaStream_t>(stream));
}

int fma_b200_unpack_sequence(const void* packed, void* padded, const void* cu_seqlens, int32_t index_bytes, int64_t B,
                             int64_t S, int64_t total, int64_t row_bytes, int32_t pad_left, void* stream) {
    return fmab::launch_pack(packed, padded, cu_seqlens, index_bytes, B, S, total, row_bytes, pad_left, false,
                             static_cast<cudaStream_t>(stream));
}

}  // extern "C"
