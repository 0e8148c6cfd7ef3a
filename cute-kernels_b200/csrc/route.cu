// Router post-processing and the expert sort.
//   * top-k + softmax over the selected logits (one warp per token row) and its backward;
//   * stable counting sort of the T*k selected expert ids, which also emits the row maps of
//     the expert-contiguous layout (expert segments padded to a multiple of row_align rows);
//   * row maps for rows received from other ranks under expert parallelism.
// All integer results are bit-exact functions of their inputs (no floating-point atomics,
// no order-dependent races): the sort equals torch.sort(stable=True).
#include <math.h>

#include "common.cuh"

namespace fmab {

// ---------------------------------------------------------------------------
// top-k + softmax
// ---------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ float load_as_float(const T* p);
template <>
__device__ __forceinline__ float load_as_float<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float load_as_float<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T>
__device__ __forceinline__ void store_from_float(T* p, float v);
template <>
__device__ __forceinline__ void store_from_float<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void store_from_float<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// (value, index) ordering of torch.topk made deterministic: larger value first, and
// among equal values the lower expert id first.
__device__ __forceinline__ bool better(float va, int ia, float vb, int ib) {
    return va > vb || (va == vb && ia < ib);
}

constexpr int kTopkWarps = 8;

template <typename T, int kPerLane>
__global__ void __launch_bounds__(kTopkWarps * 32)
topk_softmax_kernel(const T* __restrict__ logits, int64_t rows, int E, int k, T* __restrict__ weights,
                    int64_t* __restrict__ selected) {
    const int lane = threadIdx.x & 31;
    const int64_t row = static_cast<int64_t>(blockIdx.x) * kTopkWarps + (threadIdx.x >> 5);
    if (row >= rows) return;
    const T* src = logits + row * E;
    float v[kPerLane];
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
        const int c = lane + 32 * i;
        v[i] = (c < E) ? load_as_float(src + c) : -INFINITY;
    }
    uint32_t taken = 0;  // bit i set once v[i] has been selected
    float my_val = 0.f;  // lane r keeps the r-th selection
    int my_idx = 0;
    float top_val = 0.f;
    for (int r = 0; r < k; ++r) {
        float bv = -INFINITY;
        int bi = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < kPerLane; ++i) {
            const int c = lane + 32 * i;
            if (!((taken >> i) & 1u) && c < E && better(v[i], c, bv, bi)) {
                bv = v[i];
                bi = c;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (better(ov, oi, bv, bi)) {
                bv = ov;
                bi = oi;
            }
        }
        if (bi != 0x7fffffff && (bi & 31) == lane) taken |= 1u << (bi >> 5);
        if (r == 0) top_val = bv;
        if (lane == r) {
            my_val = bv;
            my_idx = bi;
        }
    }
    // softmax over the k selected values, fp32, then cast (MoE._compute_routing_weights).
    const float e = (lane < k) ? expf(my_val - top_val) : 0.f;
    const float denom = warp_sum(e);
    if (lane < k) {
        store_from_float(weights + row * k + lane, e / denom);
        selected[row * k + lane] = my_idx;
    }
}

template <typename T>
__global__ void __launch_bounds__(kTopkWarps * 32)
topk_softmax_backward_kernel(const T* __restrict__ weights, const T* __restrict__ d_weights,
                             const int64_t* __restrict__ selected, int64_t rows, int E, int k,
                             T* __restrict__ d_logits) {
    const int lane = threadIdx.x & 31;
    const int64_t row = static_cast<int64_t>(blockIdx.x) * kTopkWarps + (threadIdx.x >> 5);
    if (row >= rows) return;
    float w = 0.f, dw = 0.f;
    int idx = 0;
    if (lane < k) {
        w = load_as_float(weights + row * k + lane);
        dw = load_as_float(d_weights + row * k + lane);
        idx = static_cast<int>(selected[row * k + lane]);
    }
    const float dot = warp_sum(w * dw);
    const float d_tv = w * (dw - dot);
    T* dst = d_logits + row * E;
    for (int c = lane; c < E; c += 32) store_from_float(dst + c, 0.f);
    __syncwarp();
    if (lane < k) store_from_float(dst + idx, d_tv);
}

// ---------------------------------------------------------------------------
// stable counting sort
// ---------------------------------------------------------------------------
constexpr int kSortWarps = 8;
constexpr int kSortThreads = kSortWarps * 32;
constexpr int kMaxExperts = 1024;

// Elements handled by one warp ("piece"): a multiple of 32, chosen on the host.
struct SortPlan {
    int64_t piece;   // elements per warp
    int n_pieces;    // ceil(R / piece)
    int n_blocks;    // ceil(n_pieces / kSortWarps)
};

static SortPlan make_sort_plan(int64_t R, int E) {
    // Keep the piece table (n_pieces x E words) small: at most ~4096 pieces, at least 1024 ids per warp.
    int64_t piece = 1024;
    while ((R + piece - 1) / piece > 4096) piece *= 2;
    (void)E;
    SortPlan p;
    p.piece = piece;
    p.n_pieces = static_cast<int>((R + piece - 1) / piece);
    if (p.n_pieces < 1) p.n_pieces = 1;
    p.n_blocks = (p.n_pieces + kSortWarps - 1) / kSortWarps;
    return p;
}

// Pass 1: per-piece histograms.  piece_hist[piece][e].
__global__ void __launch_bounds__(kSortThreads)
sort_hist_kernel(const int64_t* __restrict__ ids, int64_t R, int E, int64_t piece, int n_pieces,
                 int32_t* __restrict__ piece_hist) {
    extern __shared__ int32_t sh[];  // [kSortWarps][E]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int32_t* mine = sh + warp * E;
    for (int e = lane; e < E; e += 32) mine[e] = 0;
    __syncwarp();
    const int p = blockIdx.x * kSortWarps + warp;
    if (p >= n_pieces) return;
    const int64_t beg = p * piece;
    const int64_t end = (beg + piece < R) ? beg + piece : R;
    for (int64_t i = beg + lane; i - lane < end; i += 32) {
        const bool ok = i < end;
        const int e = ok ? static_cast<int>(ids[i]) : -1;
        const unsigned active = __ballot_sync(0xffffffffu, ok);
        if (ok) {
            const unsigned same = __match_any_sync(active, e);
            if (lane == __ffs(same) - 1) mine[e] += __popc(same);
        }
        __syncwarp();
    }
    __syncwarp();
    for (int e = lane; e < E; e += 32) piece_hist[static_cast<int64_t>(p) * E + e] = mine[e];
}

// Pass 2 (one block): exclusive scan of every expert's column over the pieces (in place),
// expert totals, padded segment offsets, the tile -> expert table.
__global__ void __launch_bounds__(1024)
sort_scan_kernel(int32_t* __restrict__ piece_hist, int n_pieces, int E, int row_align, int64_t rows_cap,
                 uint32_t* __restrict__ expert_count, int32_t* __restrict__ pad_offsets,
                 int32_t* __restrict__ plain_offsets, int32_t* __restrict__ mtile_expert) {
    __shared__ int32_t s_count[kMaxExperts];
    __shared__ int32_t s_pad[kMaxExperts + 1];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int e = warp; e < E; e += 32) {
        int32_t running = 0;
        for (int base = 0; base < n_pieces; base += 32) {
            const int p = base + lane;
            const int32_t c = (p < n_pieces) ? piece_hist[static_cast<int64_t>(p) * E + e] : 0;
            int32_t incl = c;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int32_t t = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += t;
            }
            if (p < n_pieces) piece_hist[static_cast<int64_t>(p) * E + e] = running + incl - c;
            running += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (lane == 0) s_count[e] = running;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int32_t pad = 0, plain = 0;
        for (int e = 0; e < E; ++e) {
            s_pad[e] = pad;
            plain_offsets[e] = plain;
            const int32_t c = s_count[e];
            plain += c;
            pad += (row_align > 1) ? ((c + row_align - 1) / row_align) * row_align : c;
        }
        s_pad[E] = pad;
        plain_offsets[E] = plain;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) expert_count[e] = static_cast<uint32_t>(s_count[e]);
    for (int e = threadIdx.x; e <= E; e += blockDim.x) pad_offsets[e] = s_pad[e];
    if (mtile_expert != nullptr) {
        const int64_t n_tiles = rows_cap / 128;
        for (int64_t t = threadIdx.x; t < n_tiles; t += blockDim.x) {
            const int32_t row = static_cast<int32_t>(t * 128);
            int32_t owner = -1;
            if (row < s_pad[E]) {
                // Largest e with s_pad[e] <= row; empty experts share an offset with their
                // successor, so take the last one whose segment is non-empty.
                int lo = 0, hi = E;  // invariant: s_pad[lo] <= row < s_pad[hi]
                while (hi - lo > 1) {
                    const int mid = (lo + hi) >> 1;
                    if (s_pad[mid] <= row) lo = mid; else hi = mid;
                }
                owner = lo;
            }
            mtile_expert[t] = owner;
        }
    }
}

// Pass 3: place every id.  Within an expert, earlier flat indices get earlier rows.
__global__ void __launch_bounds__(kSortThreads)
sort_place_kernel(const int64_t* __restrict__ ids, int64_t R, int E, int64_t piece, int n_pieces,
                  const int32_t* __restrict__ piece_base, const int32_t* __restrict__ pad_offsets,
                  const int32_t* __restrict__ plain_offsets, int64_t* __restrict__ sorted_expert_idxs,
                  int64_t* __restrict__ sorted_scattered_idxs, int32_t* __restrict__ row_of_slot,
                  int32_t* __restrict__ slot_of_row) {
    extern __shared__ int32_t sh[];  // [kSortWarps][E] running ranks
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int p = blockIdx.x * kSortWarps + warp;
    if (p >= n_pieces) return;
    int32_t* running = sh + warp * E;
    for (int e = lane; e < E; e += 32) running[e] = piece_base[static_cast<int64_t>(p) * E + e];
    __syncwarp();
    const int64_t beg = p * piece;
    const int64_t end = (beg + piece < R) ? beg + piece : R;
    const unsigned lt_mask = (1u << lane) - 1u;
    for (int64_t i = beg + lane; i - lane < end; i += 32) {
        const bool ok = i < end;
        const int e = ok ? static_cast<int>(ids[i]) : -1;
        const unsigned active = __ballot_sync(0xffffffffu, ok);
        int32_t rank = 0;
        unsigned same = 0;
        if (ok) {
            same = __match_any_sync(active, e);
            rank = running[e] + __popc(same & lt_mask);
        }
        __syncwarp();
        if (ok && lane == __ffs(same) - 1) running[e] += __popc(same);
        __syncwarp();
        if (ok) {
            const int32_t row = pad_offsets[e] + rank;
            if (row_of_slot != nullptr) row_of_slot[i] = row;
            if (slot_of_row != nullptr) slot_of_row[row] = static_cast<int32_t>(i);
            const int64_t q = static_cast<int64_t>(plain_offsets[e]) + rank;
            if (sorted_expert_idxs != nullptr) sorted_expert_idxs[q] = e;
            if (sorted_scattered_idxs != nullptr) sorted_scattered_idxs[q] = i;
        }
    }
}

// ---------------------------------------------------------------------------
// expert-parallel receive maps (one block)
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(1024)
ep_recv_maps_kernel(const int32_t* __restrict__ counts, int n_src, int E_local, int row_align, int64_t rows_cap,
                    int32_t* __restrict__ seg_offsets, int32_t* __restrict__ mtile_expert) {
    extern __shared__ int32_t s_off[];  // [n_src*E_local + 1]
    const int n_seg = n_src * E_local;
    if (threadIdx.x == 0) {
        int32_t off = 0;
        for (int s = 0; s < n_seg; ++s) {
            s_off[s] = off;
            const int32_t c = counts[s];
            off += ((c + row_align - 1) / row_align) * row_align;
        }
        s_off[n_seg] = off;
    }
    __syncthreads();
    for (int s = threadIdx.x; s <= n_seg; s += blockDim.x) seg_offsets[s] = s_off[s];
    const int64_t n_tiles = rows_cap / 128;
    for (int64_t t = threadIdx.x; t < n_tiles; t += blockDim.x) {
        const int32_t row = static_cast<int32_t>(t * 128);
        int32_t owner = -1;
        if (row < s_off[n_seg]) {
            int lo = 0, hi = n_seg;
            while (hi - lo > 1) {
                const int mid = (lo + hi) >> 1;
                if (s_off[mid] <= row) lo = mid; else hi = mid;
            }
            owner = lo % E_local;
        }
        mtile_expert[t] = owner;
    }
}

template <typename T>
static int launch_topk(const void* logits, int64_t rows, int E, int k, void* weights, int64_t* selected,
                       cudaStream_t s) {
    const unsigned grid = static_cast<unsigned>((rows + kTopkWarps - 1) / kTopkWarps);
    const T* in = static_cast<const T*>(logits);
    T* w = static_cast<T*>(weights);
    const int per_lane = (E + 31) / 32;
    if (per_lane <= 1) topk_softmax_kernel<T, 1><<<grid, kTopkWarps * 32, 0, s>>>(in, rows, E, k, w, selected);
    else if (per_lane <= 2) topk_softmax_kernel<T, 2><<<grid, kTopkWarps * 32, 0, s>>>(in, rows, E, k, w, selected);
    else if (per_lane <= 4) topk_softmax_kernel<T, 4><<<grid, kTopkWarps * 32, 0, s>>>(in, rows, E, k, w, selected);
    else if (per_lane <= 8) topk_softmax_kernel<T, 8><<<grid, kTopkWarps * 32, 0, s>>>(in, rows, E, k, w, selected);
    else if (per_lane <= 16) topk_softmax_kernel<T, 16><<<grid, kTopkWarps * 32, 0, s>>>(in, rows, E, k, w, selected);
    else topk_softmax_kernel<T, 32><<<grid, kTopkWarps * 32, 0, s>>>(in, rows, E, k, w, selected);
    return check_launch("router_topk_softmax");
}

}  // namespace fmab

extern "C" {

int fma_b200_router_topk_softmax(const void* logits, int32_t dtype, int64_t T, int32_t E, int32_t k, void* weights,
                                 int64_t* selected, void* stream) {
    using namespace fmab;
    FMAB_REQUIRE(T >= 0 && T < (1LL << 31) * kTopkWarps, FMA_B200_ERR_BAD_ARG, "T=%lld out of range", (long long)T);
    FMAB_REQUIRE(E >= 1 && E <= kMaxExperts, FMA_B200_ERR_BAD_ARG, "E=%d not in [1,%d]", E, kMaxExperts);
    FMAB_REQUIRE(k >= 1 && k <= E && k <= 32, FMA_B200_ERR_BAD_ARG, "k=%d not in [1,min(E,32)]", k);
    if (T == 0) return FMA_B200_OK;
    FMAB_REQUIRE(logits && weights && selected, FMA_B200_ERR_BAD_ARG, "NULL pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == FMA_B200_F32) return launch_topk<float>(logits, T, E, k, weights, selected, s);
    if (dtype == FMA_B200_BF16) return launch_topk<__nv_bfloat16>(logits, T, E, k, weights, selected, s);
    return fail(FMA_B200_ERR_UNSUPPORTED, "router_topk_softmax: dtype %d", dtype);
}

int fma_b200_router_topk_softmax_backward(const void* weights, const void* d_weights, const int64_t* selected,
                                          int32_t dtype, int64_t T, int32_t E, int32_t k, void* d_logits,
                                          void* stream) {
    using namespace fmab;
    FMAB_REQUIRE(T >= 0, FMA_B200_ERR_BAD_ARG, "T=%lld", (long long)T);
    FMAB_REQUIRE(E >= 1 && E <= kMaxExperts && k >= 1 && k <= E && k <= 32, FMA_B200_ERR_BAD_ARG, "E=%d k=%d", E, k);
    if (T == 0) return FMA_B200_OK;
    FMAB_REQUIRE(weights && d_weights && selected && d_logits, FMA_B200_ERR_BAD_ARG, "NULL pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const unsigned grid = static_cast<unsigned>((T + kTopkWarps - 1) / kTopkWarps);
    if (dtype == FMA_B200_F32)
        topk_softmax_backward_kernel<float><<<grid, kTopkWarps * 32, 0, s>>>(
            static_cast<const float*>(weights), static_cast<const float*>(d_weights), selected, T, E, k,
            static_cast<float*>(d_logits));
    else if (dtype == FMA_B200_BF16)
        topk_softmax_backward_kernel<__nv_bfloat16><<<grid, kTopkWarps * 32, 0, s>>>(
            static_cast<const __nv_bfloat16*>(weights), static_cast<const __nv_bfloat16*>(d_weights), selected, T, E,
            k, static_cast<__nv_bfloat16*>(d_logits));
    else
        return fail(FMA_B200_ERR_UNSUPPORTED, "router_topk_softmax_backward: dtype %d", dtype);
    return check_launch("router_topk_softmax_backward");
}

int64_t fma_b200_moe_rows_cap(int64_t R, int32_t E, int32_t row_align) {
    if (R < 0 || E < 1 || row_align < 1) return 0;
    // Every expert wastes at most row_align-1 rows; round the total up to whole 128-row tiles.
    const int64_t worst = R + static_cast<int64_t>(E) * (row_align - 1);
    return ((worst + 127) / 128) * 128;
}

int64_t fma_b200_moe_sort_workspace_bytes(int64_t R, int32_t E) {
    if (R < 0 || E < 1) return 0;
    const fmab::SortPlan p = fmab::make_sort_plan(R, E);
    // piece table + unpadded offsets
    return (static_cast<int64_t>(p.n_pieces) * E + (E + 1)) * 4 + 256;
}

int fma_b200_moe_sort(const int64_t* selected, int64_t R, int32_t E, int32_t row_align, int64_t rows_cap,
                      int64_t* sorted_expert_idxs, int64_t* sorted_scattered_idxs, uint32_t* expert_count,
                      int32_t* pad_offsets, int32_t* row_of_slot, int32_t* slot_of_row, int32_t* mtile_expert,
                      void* workspace, int64_t workspace_bytes, void* stream) {
    using namespace fmab;
    FMAB_REQUIRE(R >= 0 && R < (1LL << 31) - 1024 * 128, FMA_B200_ERR_BAD_ARG, "R=%lld out of range", (long long)R);
    FMAB_REQUIRE(E >= 1 && E <= kMaxExperts, FMA_B200_ERR_BAD_ARG, "E=%d not in [1,%d]", E, kMaxExperts);
    FMAB_REQUIRE(row_align == 1 || row_align % 128 == 0, FMA_B200_ERR_BAD_ARG, "row_align=%d must be 1 or a multiple of 128", row_align);
    FMAB_REQUIRE(expert_count && pad_offsets && workspace, FMA_B200_ERR_BAD_ARG, "NULL pointer");
    FMAB_REQUIRE(R == 0 || selected, FMA_B200_ERR_BAD_ARG, "selected is NULL");
    FMAB_REQUIRE(rows_cap >= fma_b200_moe_rows_cap(R, E, row_align) || (!slot_of_row && !mtile_expert),
                 FMA_B200_ERR_BAD_ARG, "rows_cap=%lld < %lld", (long long)rows_cap,
                 (long long)fma_b200_moe_rows_cap(R, E, row_align));
    FMAB_REQUIRE(mtile_expert == nullptr || row_align % 128 == 0, FMA_B200_ERR_BAD_ARG,
                 "mtile_expert needs row_align %% 128 == 0");
    FMAB_REQUIRE(workspace_bytes >= fma_b200_moe_sort_workspace_bytes(R, E), FMA_B200_ERR_WORKSPACE,
                 "moe_sort workspace: %lld < %lld bytes", (long long)workspace_bytes,
                 (long long)fma_b200_moe_sort_workspace_bytes(R, E));
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const SortPlan plan = make_sort_plan(R, E);
    int32_t* piece_hist = static_cast<int32_t*>(workspace);
    int32_t* plain_offsets = piece_hist + static_cast<int64_t>(plan.n_pieces) * E;
    const size_t smem = static_cast<size_t>(kSortWarps) * E * 4;
    if (slot_of_row != nullptr) FMAB_CUDA(cudaMemsetAsync(slot_of_row, 0xff, static_cast<size_t>(rows_cap) * 4, s));
    sort_hist_kernel<<<plan.n_blocks, kSortThreads, smem, s>>>(selected, R, E, plan.piece, plan.n_pieces, piece_hist);
    if (int rc = check_launch("moe_sort/hist")) return rc;
    sort_scan_kernel<<<1, 1024, 0, s>>>(piece_hist, plan.n_pieces, E, row_align, rows_cap, expert_count,
                                        pad_offsets, plain_offsets, mtile_expert);
    if (int rc = check_launch("moe_sort/scan")) return rc;
    if (R > 0) {
        sort_place_kernel<<<plan.n_blocks, kSortThreads, smem, s>>>(
            selected, R, E, plan.piece, plan.n_pieces, piece_hist, pad_offsets, plain_offsets, sorted_expert_idxs,
            sorted_scattered_idxs, row_of_slot, slot_of_row);
        if (int rc = check_launch("moe_sort/place")) return rc;
    }
    return FMA_B200_OK;
}

int fma_b200_moe_ep_recv_maps(const int32_t* counts, int32_t n_src, int32_t E_local, int32_t row_align,
                              int64_t rows_cap, int32_t* seg_offsets, int32_t* mtile_expert, void* stream) {
    using namespace fmab;
    FMAB_REQUIRE(counts && seg_offsets && mtile_expert, FMA_B200_ERR_BAD_ARG, "NULL pointer");
    FMAB_REQUIRE(n_src >= 1 && E_local >= 1 && n_src * (int64_t)E_local <= 8192, FMA_B200_ERR_BAD_ARG,
                 "n_src=%d E_local=%d", n_src, E_local);
    FMAB_REQUIRE(row_align % 128 == 0 && row_align > 0, FMA_B200_ERR_BAD_ARG, "row_align=%d", row_align);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const size_t smem = (static_cast<size_t>(n_src) * E_local + 1) * 4;
    ep_recv_maps_kernel<<<1, 1024, smem, s>>>(counts, n_src, E_local, row_align, rows_cap, seg_offsets, mtile_expert);
    return check_launch("moe_ep_recv_maps");
}

}  // extern "C"
