// Row movers between the token order [T,H] and the expert-contiguous ("grouped") order
// [rows,H]: scatter and its backward, weighted combine and its backward.  All HBM-bound.
//
// Every kernel is token-major: one warp owns one token, reads that token's row ONCE with
// 128-bit accesses and touches its k grouped rows, so the algorithmic traffic
// (T+R)*H*s (scatter, combine) is also the DRAM traffic even when [T,H] exceeds L2.
// Sums over the k rows are taken in fp32 in ascending j, so results are run-to-run
// identical (the reference's atomic-add backward is not:
// fma/modules/moe/cuda_implementation/ungroup_kernel.py:59-69).
// Padding rows of the grouped layout are zero-filled by extra blocks of the same launch.
#include "common.cuh"

namespace fmab {

constexpr int kRowWarps = 8;
constexpr int kRowThreads = kRowWarps * 32;
constexpr int kMaxTopK = 32;

// Zero the padding rows [.. pad_offsets[E]) whose slot is -1; one warp per grouped row.
template <typename T>
__device__ __forceinline__ void zero_pad_row(int64_t row, const int32_t* slot_of_row, const int32_t* pad_offsets,
                                             int E, int H, T* grouped, int lane) {
    if (row >= pad_offsets[E]) return;
    if (slot_of_row[row] >= 0) return;
    constexpr int V = Elem<T>::kPerVec;
    uint4* dst = reinterpret_cast<uint4*>(grouped + row * H);
    for (int c = lane; c < H / V; c += 32) dst[c] = make_uint4(0, 0, 0, 0);
}

template <typename T>
__global__ void __launch_bounds__(kRowThreads)
scatter_kernel(const T* __restrict__ x, int64_t n_tok, int H, int k, const int32_t* __restrict__ row_of_slot,
               const int32_t* __restrict__ slot_of_row, const int32_t* __restrict__ pad_offsets, int E,
               int64_t tok_blocks, T* __restrict__ grouped) {
    constexpr int V = Elem<T>::kPerVec;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (blockIdx.x >= tok_blocks) {
        const int64_t row = (static_cast<int64_t>(blockIdx.x) - tok_blocks) * kRowWarps + warp;
        zero_pad_row<T>(row, slot_of_row, pad_offsets, E, H, grouped, lane);
        return;
    }
    const int64_t t = static_cast<int64_t>(blockIdx.x) * kRowWarps + warp;
    if (t >= n_tok) return;
    const uint4* src = reinterpret_cast<const uint4*>(x + t * H);
    const int n_vec = H / V;
    const int32_t* rows = row_of_slot + t * k;
    for (int c0 = 0; c0 < n_vec; c0 += 128) {
        uint4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int c = c0 + u * 32 + lane;
            if (c < n_vec) v[u] = ld_stream_16(src + c);
        }
        for (int j = 0; j < k; ++j) {
            if (rows[j] < 0) continue;  // slot without a row (its expert id was out of range)
            uint4* dst = reinterpret_cast<uint4*>(grouped + static_cast<int64_t>(rows[j]) * H);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int c = c0 + u * 32 + lane;
                if (c < n_vec) dst[c] = v[u];
            }
        }
    }
}

// out[t] = sum_j coeff[t,j] * grouped[row_j]   (coeff == nullptr -> plain sum)
template <typename T>
__global__ void __launch_bounds__(kRowThreads)
gather_sum_kernel(const T* __restrict__ grouped, const T* __restrict__ coeff, int64_t n_tok, int H, int k,
                  const int32_t* __restrict__ row_of_slot, T* __restrict__ out) {
    constexpr int V = Elem<T>::kPerVec;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t t = static_cast<int64_t>(blockIdx.x) * kRowWarps + warp;
    if (t >= n_tok) return;
    const int n_vec = H / V;
    // Lane j keeps the j-th row index and coefficient; broadcast by shuffle in the loop.
    int32_t my_row = 0;
    float my_w = 1.f;
    if (lane < k) {
        my_row = row_of_slot[t * k + lane];
        if (coeff != nullptr) {
            my_w = elem_to_float<T>(coeff[t * k + lane]);
        }
    }
    uint4* dst = reinterpret_cast<uint4*>(out + t * H);
    for (int c0 = 0; c0 < n_vec; c0 += 64) {
        float acc[2][V];
#pragma unroll
        for (int u = 0; u < 2; ++u)
#pragma unroll
            for (int i = 0; i < V; ++i) acc[u][i] = 0.f;
        for (int j = 0; j < k; ++j) {
            const int32_t row = __shfl_sync(0xffffffffu, my_row, j);
            const float w = __shfl_sync(0xffffffffu, my_w, j);
            if (row < 0) continue;  // slot without a row: contributes nothing
            const uint4* src = reinterpret_cast<const uint4*>(grouped + static_cast<int64_t>(row) * H);
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int c = c0 + u * 32 + lane;
                if (c < n_vec) {
                    float f[V];
                    Elem<T>::unpack(ld_stream_16(src + c), f);
#pragma unroll
                    for (int i = 0; i < V; ++i) acc[u][i] = fmaf(w, f[i], acc[u][i]);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int c = c0 + u * 32 + lane;
            if (c < n_vec) dst[c] = Elem<T>::pack(acc[u]);
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(kRowThreads)
combine_backward_kernel(const T* __restrict__ dy, const T* __restrict__ expert_out, const T* __restrict__ weights,
                        int64_t n_tok, int H, int k, const int32_t* __restrict__ row_of_slot,
                        const int32_t* __restrict__ slot_of_row, const int32_t* __restrict__ pad_offsets, int E,
                        int64_t tok_blocks, T* __restrict__ d_expert_out, T* __restrict__ d_weights) {
    constexpr int V = Elem<T>::kPerVec;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (blockIdx.x >= tok_blocks) {
        const int64_t row = (static_cast<int64_t>(blockIdx.x) - tok_blocks) * kRowWarps + warp;
        zero_pad_row<T>(row, slot_of_row, pad_offsets, E, H, d_expert_out, lane);
        return;
    }
    const int64_t t = static_cast<int64_t>(blockIdx.x) * kRowWarps + warp;
    if (t >= n_tok) return;
    const int n_vec = H / V;
    const uint4* g_src = reinterpret_cast<const uint4*>(dy + t * H);
    const bool want_dw = (d_weights != nullptr) && (expert_out != nullptr);
    for (int j = 0; j < k; ++j) {
        const int64_t row = row_of_slot[t * k + j];
        if (row < 0) {  // slot without a row: no gradient row to write, zero gradient for its weight
            if (want_dw && lane == 0) d_weights[t * k + j] = float_to_elem<T>(0.f);
            continue;
        }
        const float w = elem_to_float<T>(weights[t * k + j]);
        uint4* dst = reinterpret_cast<uint4*>(d_expert_out + row * H);
        const uint4* o_src = want_dw ? reinterpret_cast<const uint4*>(expert_out + row * H) : nullptr;
        float dot = 0.f;
        for (int c0 = 0; c0 < n_vec; c0 += 128) {
            // four independent 16-byte loads of dy (L1/L2 after the first j) and of expert_out in flight
            uint4 gv[4], ov[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int c = c0 + u * 32 + lane;
                if (c < n_vec) {
                    gv[u] = ld_global_16(g_src + c);
                    if (want_dw) ov[u] = ld_stream_16(o_src + c);
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int c = c0 + u * 32 + lane;
                if (c < n_vec) {
                    float g[V], o[V], r[V];
                    Elem<T>::unpack(gv[u], g);
#pragma unroll
                    for (int i = 0; i < V; ++i) r[i] = w * g[i];
                    dst[c] = Elem<T>::pack(r);
                    if (want_dw) {
                        Elem<T>::unpack(ov[u], o);
#pragma unroll
                        for (int i = 0; i < V; ++i) dot = fmaf(o[i], g[i], dot);
                    }
                }
            }
        }
        if (want_dw) {
            dot = warp_sum(dot);
            if (lane == 0) d_weights[t * k + j] = float_to_elem<T>(dot);
        }
    }
}

// grouped[p, :] += bias[e(p), :] on token rows (padding rows stay zero); one warp per grouped row.
template <typename T>
__global__ void __launch_bounds__(kRowThreads)
bias_add_kernel(T* __restrict__ grouped, const T* __restrict__ bias, int64_t rows_cap, int C,
                const int32_t* __restrict__ mtile_expert, const int32_t* __restrict__ slot_of_row) {
    constexpr int V = Elem<T>::kPerVec;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t row = static_cast<int64_t>(blockIdx.x) * kRowWarps + warp;
    if (row >= rows_cap) return;
    const int e = mtile_expert[row >> 7];
    if (e < 0 || slot_of_row[row] < 0) return;
    uint4* dst = reinterpret_cast<uint4*>(grouped + row * C);
    const uint4* b = reinterpret_cast<const uint4*>(bias + static_cast<int64_t>(e) * C);
    for (int c = lane; c < C / V; c += 32) {
        float x[V], y[V];
        Elem<T>::unpack(dst[c], x);
        Elem<T>::unpack(ld_global_16(b + c), y);
#pragma unroll
        for (int i = 0; i < V; ++i) x[i] += y[i];
        dst[c] = Elem<T>::pack(x);
    }
}

// d_bias[e, c] = sum over the rows of expert e of d_grouped[row, c] (padding rows are zero), fp32
// accumulation in row order: deterministic.  Block = (expert, 256 columns), thread = one column.
template <typename T>
__global__ void __launch_bounds__(256)
bias_grad_kernel(const T* __restrict__ d_grouped, int C, const int32_t* __restrict__ pad_offsets,
                 T* __restrict__ d_bias) {
    const int e = blockIdx.y;
    const int c = blockIdx.x * 256 + threadIdx.x;
    if (c >= C) return;
    const int64_t beg = pad_offsets[e], end = pad_offsets[e + 1];
    float acc = 0.f;
    int64_t r = beg;
    for (; r + 4 <= end; r += 4) {
        float v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            v[u] = elem_to_float<T>(d_grouped[(r + u) * C + c]);
        }
        acc += v[0];
        acc += v[1];
        acc += v[2];
        acc += v[3];
    }
    for (; r < end; ++r) {
        acc += elem_to_float<T>(d_grouped[r * C + c]);
    }
    d_bias[static_cast<int64_t>(e) * C + c] = float_to_elem<T>(acc);
}

static int check_rows_args(int32_t dtype, int64_t T, int32_t H, int32_t k) {
    FMAB_REQUIRE(known_dtype(dtype), FMA_B200_ERR_UNSUPPORTED, "dtype %d", dtype);
    FMAB_REQUIRE(T >= 0 && T < (1LL << 31), FMA_B200_ERR_BAD_ARG, "T=%lld", (long long)T);
    FMAB_REQUIRE(k >= 1 && k <= kMaxTopK, FMA_B200_ERR_BAD_ARG, "k=%d not in [1,%d]", k, kMaxTopK);
    const int per_vec = elems_per_16_bytes(dtype);
    FMAB_REQUIRE(H >= per_vec && H % per_vec == 0, FMA_B200_ERR_BAD_ARG, "H=%d is not a multiple of 16 bytes", H);
    return FMA_B200_OK;
}

}  // namespace fmab

namespace fmab {
// Zeroes the padding at the end of every segment: rows [seg_offsets[j] + counts[j], seg_offsets[j + 1]).
// gridDim.y blocks per segment (blockIdx.x = segment); 16-byte stores.
__global__ void __launch_bounds__(256) zero_padding_kernel(uint8_t* __restrict__ rows, int64_t row_bytes,
                                                           const int32_t* __restrict__ seg_offsets,
                                                           const int32_t* __restrict__ counts) {
    const int j = blockIdx.x;
    const int64_t first = static_cast<int64_t>(seg_offsets[j]) + counts[j];
    const int64_t end = seg_offsets[j + 1];
    if (end <= first) return;
    uint4* dst = reinterpret_cast<uint4*>(rows + first * row_bytes);
    const int64_t n = (end - first) * row_bytes / 16;
    for (int64_t i = blockIdx.y * blockDim.x + threadIdx.x; i < n; i += static_cast<int64_t>(gridDim.y) * blockDim.x)
        dst[i] = make_uint4(0, 0, 0, 0);
}
}  // namespace fmab

extern "C" {

int fma_b200_moe_scatter(const void* x, int32_t dtype, int64_t T, int32_t H, int32_t k, const int32_t* row_of_slot,
                         const int32_t* slot_of_row, const int32_t* pad_offsets, int32_t E, int64_t rows_cap,
                         void* grouped, void* stream) {
    using namespace fmab;
    if (int rc = check_rows_args(dtype, T, H, k)) return rc;
    FMAB_REQUIRE(row_of_slot && slot_of_row && pad_offsets && grouped, FMA_B200_ERR_BAD_ARG, "NULL pointer");
    FMAB_REQUIRE(T == 0 || x, FMA_B200_ERR_BAD_ARG, "x is NULL");
    FMAB_REQUIRE(aligned16(x) && aligned16(grouped), FMA_B200_ERR_BAD_ARG, "x/grouped not 16-byte aligned");
    FMAB_REQUIRE(rows_cap >= 0 && E >= 1, FMA_B200_ERR_BAD_ARG, "rows_cap=%lld E=%d", (long long)rows_cap, E);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int64_t tok_blocks = (T + kRowWarps - 1) / kRowWarps;
    const int64_t pad_blocks = (rows_cap + kRowWarps - 1) / kRowWarps;
    const int64_t grid = tok_blocks + pad_blocks;
    if (grid == 0) return FMA_B200_OK;
    FMAB_REQUIRE(grid < (1LL << 31), FMA_B200_ERR_BAD_ARG, "grid too large");
    dispatch_dtype(dtype, [&](auto tag) {
        using Elt = decltype(tag);
        scatter_kernel<Elt><<<(unsigned)grid, kRowThreads, 0, s>>>(static_cast<const Elt*>(x), T, H, k, row_of_slot, slot_of_row,
                                                                  pad_offsets, E, tok_blocks, static_cast<Elt*>(grouped));
    });
    return check_launch("moe_scatter");
}

static int launch_gather_sum(const void* grouped, const void* coeff, int32_t dtype, int64_t T, int32_t H, int32_t k,
                             const int32_t* row_of_slot, void* out, void* stream, const char* what) {
    using namespace fmab;
    if (int rc = check_rows_args(dtype, T, H, k)) return rc;
    if (T == 0) return FMA_B200_OK;
    FMAB_REQUIRE(grouped && row_of_slot && out, FMA_B200_ERR_BAD_ARG, "NULL pointer");
    FMAB_REQUIRE(aligned16(grouped) && aligned16(out), FMA_B200_ERR_BAD_ARG, "pointers not 16-byte aligned");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const unsigned grid = static_cast<unsigned>((T + kRowWarps - 1) / kRowWarps);
    dispatch_dtype(dtype, [&](auto tag) {
        using Elt = decltype(tag);
        gather_sum_kernel<Elt><<<grid, kRowThreads, 0, s>>>(static_cast<const Elt*>(grouped), static_cast<const Elt*>(coeff), T,
                                                           H, k, row_of_slot, static_cast<Elt*>(out));
    });
    return check_launch(what);
}

int fma_b200_moe_scatter_backward(const void* d_grouped, int32_t dtype, int64_t T, int32_t H, int32_t k,
                                  const int32_t* row_of_slot, void* dx, void* stream) {
    return launch_gather_sum(d_grouped, nullptr, dtype, T, H, k, row_of_slot, dx, stream, "moe_scatter_backward");
}

int fma_b200_moe_combine(const void* expert_out, const void* weights, int32_t dtype, int64_t T, int32_t H, int32_t k,
                         const int32_t* row_of_slot, void* y, void* stream) {
    using namespace fmab;
    FMAB_REQUIRE(T == 0 || weights, FMA_B200_ERR_BAD_ARG, "weights is NULL");
    return launch_gather_sum(expert_out, weights, dtype, T, H, k, row_of_slot, y, stream, "moe_combine");
}

int fma_b200_moe_combine_backward(const void* dy, const void* expert_out, const void* weights, int32_t dtype,
                                  int64_t T, int32_t H, int32_t k, const int32_t* row_of_slot,
                                  const int32_t* slot_of_row, const int32_t* pad_offsets, int32_t E,
                                  int64_t rows_cap, void* d_expert_out, void* d_weights, void* stream) {
    using namespace fmab;
    if (int rc = check_rows_args(dtype, T, H, k)) return rc;
    FMAB_REQUIRE(row_of_slot && slot_of_row && pad_offsets && d_expert_out, FMA_B200_ERR_BAD_ARG, "NULL pointer");
    FMAB_REQUIRE(T == 0 || (dy && weights), FMA_B200_ERR_BAD_ARG, "dy or weights is NULL");
    FMAB_REQUIRE(aligned16(dy) && aligned16(d_expert_out) && aligned16(expert_out), FMA_B200_ERR_BAD_ARG,
                 "pointers not 16-byte aligned");
    FMAB_REQUIRE(rows_cap >= 0 && E >= 1, FMA_B200_ERR_BAD_ARG, "rows_cap=%lld E=%d", (long long)rows_cap, E);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int64_t tok_blocks = (T + kRowWarps - 1) / kRowWarps;
    const int64_t pad_blocks = (rows_cap + kRowWarps - 1) / kRowWarps;
    const int64_t grid = tok_blocks + pad_blocks;
    if (grid == 0) return FMA_B200_OK;
    FMAB_REQUIRE(grid < (1LL << 31), FMA_B200_ERR_BAD_ARG, "grid too large");
    dispatch_dtype(dtype, [&](auto tag) {
        using Elt = decltype(tag);
        combine_backward_kernel<Elt><<<(unsigned)grid, kRowThreads, 0, s>>>(
            static_cast<const Elt*>(dy), static_cast<const Elt*>(expert_out), static_cast<const Elt*>(weights), T, H, k,
            row_of_slot, slot_of_row, pad_offsets, E, tok_blocks, static_cast<Elt*>(d_expert_out),
            static_cast<Elt*>(d_weights));
    });
    return check_launch("moe_combine_backward");
}

int fma_b200_moe_bias_add(void* grouped, const void* bias, int32_t dtype, int64_t rows_cap, int32_t C,
                          const int32_t* mtile_expert, const int32_t* slot_of_row, void* stream) {
    using namespace fmab;
    FMAB_REQUIRE(known_dtype(dtype), FMA_B200_ERR_UNSUPPORTED, "dtype %d", dtype);
    const int per_vec = elems_per_16_bytes(dtype);
    FMAB_REQUIRE(C >= per_vec && C % per_vec == 0, FMA_B200_ERR_BAD_ARG, "C=%d is not a multiple of 16 bytes", C);
    FMAB_REQUIRE(rows_cap >= 0 && rows_cap % 128 == 0, FMA_B200_ERR_BAD_ARG, "rows_cap=%lld", (long long)rows_cap);
    if (rows_cap == 0) return FMA_B200_OK;
    FMAB_REQUIRE(grouped && bias && mtile_expert && slot_of_row, FMA_B200_ERR_BAD_ARG, "NULL pointer");
    FMAB_REQUIRE(aligned16(grouped) && aligned16(bias), FMA_B200_ERR_BAD_ARG, "pointers not 16-byte aligned");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const unsigned grid = static_cast<unsigned>((rows_cap + kRowWarps - 1) / kRowWarps);
    dispatch_dtype(dtype, [&](auto tag) {
        using Elt = decltype(tag);
        bias_add_kernel<Elt><<<grid, kRowThreads, 0, s>>>(static_cast<Elt*>(grouped), static_cast<const Elt*>(bias), rows_cap,
                                                         C, mtile_expert, slot_of_row);
    });
    return check_launch("moe_bias_add");
}

int fma_b200_moe_bias_grad(const void* d_grouped, int32_t dtype, int32_t E, int32_t C, const int32_t* pad_offsets,
                           void* d_bias, void* stream) {
    using namespace fmab;
    FMAB_REQUIRE(known_dtype(dtype), FMA_B200_ERR_UNSUPPORTED, "dtype %d", dtype);
    FMAB_REQUIRE(E >= 1 && E <= 65535 && C >= 1, FMA_B200_ERR_BAD_ARG, "E=%d C=%d", E, C);
    FMAB_REQUIRE(d_grouped && pad_offsets && d_bias, FMA_B200_ERR_BAD_ARG, "NULL pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const dim3 grid((C + 255) / 256, E);
    dispatch_dtype(dtype, [&](auto tag) {
        using Elt = decltype(tag);
        bias_grad_kernel<Elt><<<grid, 256, 0, s>>>(static_cast<const Elt*>(d_grouped), C, pad_offsets, static_cast<Elt*>(d_bias));
    });
    return check_launch("moe_bias_grad");
}

int fma_b200_moe_zero_padding(void* rows, int64_t row_bytes, const int32_t* seg_offsets, const int32_t* counts,
                               int32_t n_segments, void* stream) {
    using namespace fmab;
    FMAB_REQUIRE(n_segments >= 0 && row_bytes > 0 && row_bytes % 16 == 0, FMA_B200_ERR_BAD_ARG,
                 "n_segments=%d row_bytes=%lld", n_segments, (long long)row_bytes);
    if (n_segments == 0) return FMA_B200_OK;
    FMAB_REQUIRE(rows && seg_offsets && counts, FMA_B200_ERR_BAD_ARG, "NULL pointer");
    FMAB_REQUIRE(aligned16(rows), FMA_B200_ERR_BAD_ARG, "rows are not 16-byte aligned");
    // enough blocks to fill the GPU whatever the number of segments (a segment's padding is at most a few MB)
    const int per_segment = n_segments >= 256 ? 1 : (n_segments >= 64 ? 4 : (n_segments >= 16 ? 16 : 32));
    zero_padding_kernel<<<dim3(n_segments, per_segment), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<uint8_t*>(rows), row_bytes, seg_offsets, counts);
    return check_launch("moe_zero_padding");
}

}  // extern "C"
