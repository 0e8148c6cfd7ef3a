// Router post-processing and the expert sort.
//   * top-k + softmax over the selected logits (one warp per run of tokens) and its backward; the
//     same pass can also count the selected expert ids per warp (the sort's first pass) and sum
//     the full softmax of the logits per expert (what a load-balancing loss needs);
//   * stable counting sort of the T*k selected expert ids, which also emits the row maps of
//     the expert-contiguous layout (expert segments padded to a multiple of row_align rows);
//   * row maps for rows received from other ranks under expert parallelism.
// All integer results are bit-exact functions of their inputs (no floating-point atomics,
// no order-dependent races): the sort equals torch.sort(stable=True).
//
// Sort structure.  The flat ids are cut into `pieces` of consecutive ids, one warp each
// (make_plan: about 2048 pieces, fewer when E is large, so that the piece table stays small):
//   pass 1  histogram of every piece                       -> table[e][piece]   (or done by the top-k kernel)
//   pass 2  one warp per expert: exclusive scan of its row of the table (coalesced), expert totals
//   pass 3  every block derives the padded segment offsets from the totals, then each warp places
//           its piece in order (match.any gives the rank among equal ids of one 32-id step).
// Ids outside [0,E) are never used as an index: they are skipped (their row_of_slot is -1, which the
// row movers treat as "no row") and STATUS_BAD_EXPERT_ID is recorded in the device status word.
#include <math.h>

#include "common.cuh"

namespace fmab {

constexpr int32_t STATUS_BAD_EXPERT_ID = 0x7003;

// ---------------------------------------------------------------------------
// geometry shared by the top-k kernel and the sort
// ---------------------------------------------------------------------------
constexpr int kMaxExperts = 1024;
constexpr int kRouteWarps = 8;
constexpr int kRouteThreads = kRouteWarps * 32;

struct RoutePlan {
    int64_t tokens_per_piece;  // tokens (runs of k ids) handled by one warp
    int64_t piece;             // ids per piece = tokens_per_piece * k
    int n_pieces;
};

static int target_pieces(int E) {
    int t = (512 * 1024) / (E < 1 ? 1 : E);  // table of at most 512 Ki entries
    return t < 256 ? 256 : (t > 2048 ? 2048 : t);
}

// R ids that are T = R / k runs of k ids (k = 1 for a plain sort).
static RoutePlan make_plan(int64_t R, int E, int k) {
    if (k < 1) k = 1;
    const int64_t T = (R + k - 1) / k;
    const int64_t target = target_pieces(E);
    RoutePlan p;
    p.tokens_per_piece = (T + target - 1) / target;
    if (p.tokens_per_piece < 1) p.tokens_per_piece = 1;
    p.piece = p.tokens_per_piece * k;
    const int64_t n = (T + p.tokens_per_piece - 1) / p.tokens_per_piece;
    p.n_pieces = static_cast<int>(n < 1 ? 1 : n);
    return p;
}

// Workspace (32-bit words): [hist: target*E] [prob: target*E] [totals: E]; the tables are used with the
// pitch n_pieces of the actual plan.
struct RouteWorkspace {
    int32_t* hist;
    float* prob;
    int32_t* totals;
};
static int64_t route_workspace_bytes(int E) {
    return (2LL * target_pieces(E) * E + E + 64) * 4;
}
static RouteWorkspace carve_workspace(void* workspace, int E) {
    RouteWorkspace w;
    const int64_t table = static_cast<int64_t>(target_pieces(E)) * E;
    w.hist = static_cast<int32_t*>(workspace);
    w.prob = reinterpret_cast<float*>(w.hist + table);
    w.totals = w.hist + 2 * table;
    return w;
}

// ---------------------------------------------------------------------------
// top-k + softmax
// ---------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ float load_as_float(const T* p) { return elem_to_float<T>(*p); }
template <typename T>
__device__ __forceinline__ void store_from_float(T* p, float v) { *p = float_to_elem<T>(v); }

// Order-preserving map of a float to an unsigned key: a > b  <=>  key(a) > key(b).  NaN maps to the
// largest key, as torch.topk orders it; -0 and +0 share a key; every key of a real input is > 0.
__device__ __forceinline__ uint32_t order_key(float v) {
    if (v != v) return 0xffffffffu;
    if (v == 0.f) v = 0.f;
    const uint32_t u = __float_as_uint(v);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_value(uint32_t key) {
    if (key == 0xffffffffu) return __int_as_float(0x7fc00000);
    return __uint_as_float((key & 0x80000000u) ? (key ^ 0x80000000u) : ~key);
}

// One warp per piece (a run of tokens).  Per token: k rounds of "largest remaining key, lowest expert id
// among equals" (two warp reductions per round), softmax over the k values in fp32.
// Optional by-products, written as column `piece` of tables with n_pieces columns:
//   piece_hist[e][piece]  how often expert e was selected by the piece's tokens
//   prob_part[e][piece]   sum over the piece's tokens of softmax(logits[t, :])[e]   (all E logits)
template <typename T, int kPerLane>
__global__ void __launch_bounds__(kRouteThreads)
topk_softmax_kernel(const T* __restrict__ logits, int64_t rows, int E, int k, int64_t tokens_per_piece, int n_pieces,
                    T* __restrict__ weights, int64_t* __restrict__ selected, int32_t* __restrict__ piece_hist,
                    float* __restrict__ prob_part) {
    extern __shared__ int32_t sh_hist[];  // [kRouteWarps][E], only when piece_hist != nullptr
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int piece = blockIdx.x * kRouteWarps + warp;
    if (piece >= n_pieces) return;
    int32_t* hist = (piece_hist != nullptr) ? sh_hist + warp * E : nullptr;
    if (hist != nullptr) {
        for (int e = lane; e < E; e += 32) hist[e] = 0;
        __syncwarp();
    }
    float psum[kPerLane];
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) psum[i] = 0.f;

    const int64_t row0 = piece * tokens_per_piece;
    const int64_t row1 = (row0 + tokens_per_piece < rows) ? row0 + tokens_per_piece : rows;
    // The logits of the next token are in flight while the current one is processed (a warp walks its
    // tokens one after the other, so an unhidden load would cost a memory round trip per token).
    float nv[kPerLane];
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
        const int c = lane + 32 * i;
        nv[i] = (c < E && row0 < row1) ? load_as_float(logits + row0 * E + c) : 0.f;
    }
    for (int64_t row = row0; row < row1; ++row) {
        float v[kPerLane];
        uint32_t key[kPerLane];
#pragma unroll
        for (int i = 0; i < kPerLane; ++i) {
            const int c = lane + 32 * i;
            v[i] = nv[i];
            key[i] = (c < E) ? order_key(v[i]) : 0u;  // 0 = never selected
        }
        if (row + 1 < row1) {
            const T* nsrc = logits + (row + 1) * E;
#pragma unroll
            for (int i = 0; i < kPerLane; ++i) {
                const int c = lane + 32 * i;
                if (c < E) nv[i] = load_as_float(nsrc + c);
            }
        }
        uint32_t my_key = 0;  // lane r keeps the r-th selection
        int my_idx = 0;
        uint32_t top_key = 0;
        for (int r = 0; r < k; ++r) {
            uint32_t bk = 0;
            uint32_t bi = 0xffffffffu;
#pragma unroll
            for (int i = 0; i < kPerLane; ++i) {
                if (key[i] > bk) {  // ascending i = ascending expert id: the first of equal keys stays
                    bk = key[i];
                    bi = static_cast<uint32_t>(lane + 32 * i);
                }
            }
            const uint32_t m = __reduce_max_sync(0xffffffffu, bk);
            const uint32_t idx = __reduce_min_sync(0xffffffffu, (bk == m) ? bi : 0xffffffffu);
            // k <= E, so a real column is left in every round: m > 0 and idx < E
            if ((idx & 31u) == static_cast<uint32_t>(lane)) {
#pragma unroll
                for (int i = 0; i < kPerLane; ++i)
                    if (static_cast<uint32_t>(i) == (idx >> 5)) key[i] = 0u;
            }
            if (r == 0) top_key = m;
            if (lane == r) {
                my_key = m;
                my_idx = static_cast<int>(idx);
            }
        }
        // softmax over the k selected values, fp32, then cast (MoE._compute_routing_weights).
        const float top_val = key_value(top_key);
        const float e = (lane < k) ? expf(key_value(my_key) - top_val) : 0.f;
        const float denom = warp_sum(e);
        if (lane < k) {
            store_from_float(weights + row * k + lane, e / denom);
            selected[row * k + lane] = my_idx;
            if (hist != nullptr) hist[my_idx] += 1;  // the k ids of one token are distinct: no two lanes share a bin
        }
        if (prob_part != nullptr) {
            float pe[kPerLane];
            float z = 0.f;
#pragma unroll
            for (int i = 0; i < kPerLane; ++i) {
                pe[i] = (lane + 32 * i < E) ? expf(v[i] - top_val) : 0.f;
                z += pe[i];
            }
            z = warp_sum(z);
            const float inv = 1.f / z;
#pragma unroll
            for (int i = 0; i < kPerLane; ++i) psum[i] += pe[i] * inv;
        }
        __syncwarp();
    }
    if (hist != nullptr) {
        for (int e = lane; e < E; e += 32) piece_hist[static_cast<int64_t>(e) * n_pieces + piece] = hist[e];
    }
    if (prob_part != nullptr) {
#pragma unroll
        for (int i = 0; i < kPerLane; ++i) {
            const int c = lane + 32 * i;
            if (c < E) prob_part[static_cast<int64_t>(c) * n_pieces + piece] = psum[i];
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(kRouteThreads)
topk_softmax_backward_kernel(const T* __restrict__ weights, const T* __restrict__ d_weights,
                             const int64_t* __restrict__ selected, int64_t rows, int E, int k,
                             T* __restrict__ d_logits) {
    const int lane = threadIdx.x & 31;
    const int64_t row = static_cast<int64_t>(blockIdx.x) * kRouteWarps + (threadIdx.x >> 5);
    if (row >= rows) return;
    float w = 0.f, dw = 0.f;
    int idx = -1;
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
    if (lane < k && static_cast<unsigned>(idx) < static_cast<unsigned>(E)) store_from_float(dst + idx, d_tv);
}

// Backward of mean_prob[e] = (1/T) sum_t softmax(logits[t,:])[e]:
//   d_logits[t,c] = (1/T) * p[t,c] * (g[c] - sum_e g[e] p[t,e])     with g = d_mean_prob (fp32 [E]).
template <typename T, int kPerLane>
__global__ void __launch_bounds__(kRouteThreads)
router_prob_backward_kernel(const T* __restrict__ logits, const float* __restrict__ d_mean, int64_t rows, int E,
                            float inv_rows, T* __restrict__ d_logits) {
    const int lane = threadIdx.x & 31;
    const int64_t row = static_cast<int64_t>(blockIdx.x) * kRouteWarps + (threadIdx.x >> 5);
    if (row >= rows) return;
    const T* src = logits + row * E;
    float v[kPerLane], g[kPerLane];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
        const int c = lane + 32 * i;
        v[i] = (c < E) ? load_as_float(src + c) : -INFINITY;
        g[i] = (c < E) ? d_mean[c] : 0.f;
        mx = fmaxf(mx, v[i]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float z = 0.f;
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
        v[i] = (lane + 32 * i < E) ? expf(v[i] - mx) : 0.f;
        z += v[i];
    }
    z = warp_sum(z);
    const float inv = 1.f / z;
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
        v[i] *= inv;
        dot = fmaf(g[i], v[i], dot);
    }
    dot = warp_sum(dot);
    T* dst = d_logits + row * E;
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
        const int c = lane + 32 * i;
        if (c < E) store_from_float(dst + c, inv_rows * v[i] * (g[i] - dot));
    }
}

// ---------------------------------------------------------------------------
// stable counting sort
// ---------------------------------------------------------------------------
// Pass 1: histogram of every piece.  table[e][piece].
__global__ void __launch_bounds__(kRouteThreads)
sort_hist_kernel(const int64_t* __restrict__ ids, int64_t R, int E, int64_t piece_len, int n_pieces,
                 int32_t* __restrict__ table, int32_t* __restrict__ status) {
    extern __shared__ int32_t sh[];  // [kRouteWarps][E]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int p = blockIdx.x * kRouteWarps + warp;
    if (p >= n_pieces) return;
    int32_t* mine = sh + warp * E;
    for (int e = lane; e < E; e += 32) mine[e] = 0;
    __syncwarp();
    const int64_t beg = p * piece_len;
    const int64_t end = (beg + piece_len < R) ? beg + piece_len : R;
    bool bad = false;
    for (int64_t i0 = beg; i0 < end; i0 += 32) {
        const int64_t i = i0 + lane;
        const int64_t raw = (i < end) ? ids[i] : -1;
        const bool ok = static_cast<uint64_t>(raw) < static_cast<uint64_t>(E);
        bad |= (i < end) && !ok;
        const int e = ok ? static_cast<int>(raw) : -1;
        const unsigned active = __ballot_sync(0xffffffffu, ok);
        if (ok) {
            const unsigned same = __match_any_sync(active, e);
            if (lane == __ffs(same) - 1) mine[e] += __popc(same);
        }
        __syncwarp();
    }
    if (bad) atomicExch(status, STATUS_BAD_EXPERT_ID);
    for (int e = lane; e < E; e += 32) table[static_cast<int64_t>(e) * n_pieces + p] = mine[e];
}

// Pass 2: one warp per expert.  Exclusive scan of table[e][0..n_pieces) in place, totals[e]; and, when the
// router's probability sums are present, prob_mean[e] = (sum over pieces) / T in a fixed order.
__global__ void __launch_bounds__(kRouteThreads)
sort_scan_kernel(int32_t* __restrict__ table, int n_pieces, int E, int32_t* __restrict__ totals,
                 const float* __restrict__ prob_part, float inv_tokens, float* __restrict__ prob_mean) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int e = blockIdx.x * kRouteWarps + warp;
    if (e >= E) return;
    int32_t* row = table + static_cast<int64_t>(e) * n_pieces;
    int32_t running = 0;
    for (int base = 0; base < n_pieces; base += 32) {
        const int p = base + lane;
        const int32_t c = (p < n_pieces) ? row[p] : 0;
        int32_t incl = c;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int32_t t = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += t;
        }
        if (p < n_pieces) row[p] = running + incl - c;
        running += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) totals[e] = running;
    if (prob_part != nullptr && prob_mean != nullptr) {
        const float* pr = prob_part + static_cast<int64_t>(e) * n_pieces;
        float s = 0.f;
        for (int p = lane; p < n_pieces; p += 32) s += pr[p];
        s = warp_sum(s);
        if (lane == 0) prob_mean[e] = s * inv_tokens;
    }
}

// Pass 3: place every id.  Within an expert, earlier flat indices get earlier rows.
__global__ void __launch_bounds__(kRouteThreads)
sort_place_kernel(const int64_t* __restrict__ ids, int64_t R, int E, int64_t piece_len, int n_pieces,
                  const int32_t* __restrict__ table, const int32_t* __restrict__ totals, int row_align,
                  int64_t rows_cap, int64_t* __restrict__ sorted_expert_idxs,
                  int64_t* __restrict__ sorted_scattered_idxs, uint32_t* __restrict__ expert_count,
                  int32_t* __restrict__ pad_offsets, int32_t* __restrict__ row_of_slot,
                  int32_t* __restrict__ slot_of_row, int32_t* __restrict__ mtile_expert,
                  int32_t* __restrict__ status) {
    extern __shared__ int32_t sh[];  // [E+1] padded offsets, [E+1] plain offsets, [kRouteWarps][E] running ranks
    __shared__ int32_t warp_pad[kRouteWarps], warp_plain[kRouteWarps];
    int32_t* s_pad = sh;
    int32_t* s_plain = sh + (E + 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // Offsets of the expert segments from the totals: thread t owns experts [4t, 4t+4).
    {
        int32_t cnt[4], pad_sum = 0, plain_sum = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int e = threadIdx.x * 4 + j;
            cnt[j] = (e < E) ? totals[e] : 0;
            plain_sum += cnt[j];
            pad_sum += (row_align > 1) ? ((cnt[j] + row_align - 1) / row_align) * row_align : cnt[j];
        }
        int32_t pad_incl = pad_sum, plain_incl = plain_sum;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int32_t a = __shfl_up_sync(0xffffffffu, pad_incl, o);
            const int32_t b = __shfl_up_sync(0xffffffffu, plain_incl, o);
            if (lane >= o) {
                pad_incl += a;
                plain_incl += b;
            }
        }
        if (lane == 31) {
            warp_pad[warp] = pad_incl;
            warp_plain[warp] = plain_incl;
        }
        __syncthreads();
        int32_t pad = pad_incl - pad_sum, plain = plain_incl - plain_sum;
        for (int w = 0; w < warp; ++w) {
            pad += warp_pad[w];
            plain += warp_plain[w];
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int e = threadIdx.x * 4 + j;
            if (e < E) {
                s_pad[e] = pad;
                s_plain[e] = plain;
            }
            plain += cnt[j];
            pad += (row_align > 1) ? ((cnt[j] + row_align - 1) / row_align) * row_align : cnt[j];
            if (e == E - 1) {
                s_pad[E] = pad;
                s_plain[E] = plain;
            }
        }
        __syncthreads();
    }
    if (blockIdx.x == 0) {
        for (int e = threadIdx.x; e < E; e += kRouteThreads) expert_count[e] = static_cast<uint32_t>(totals[e]);
        for (int e = threadIdx.x; e <= E; e += kRouteThreads) pad_offsets[e] = s_pad[e];
    }
    if (mtile_expert != nullptr) {
        // every block fills its share of the tile -> expert table
        const int64_t n_tiles = rows_cap / 128;
        const int64_t per_block = (n_tiles + gridDim.x - 1) / gridDim.x;
        const int64_t t_end = min(n_tiles, (static_cast<int64_t>(blockIdx.x) + 1) * per_block);
        for (int64_t t = blockIdx.x * per_block + threadIdx.x; t < t_end; t += kRouteThreads) {
            const int32_t row = static_cast<int32_t>(t * 128);
            int32_t owner = -1;
            if (row < s_pad[E]) {
                // Largest e with s_pad[e] <= row; empty experts share an offset with their
                // successor, so this is the last of them, whose segment is non-empty.
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

    const int p = blockIdx.x * kRouteWarps + warp;
    if (p >= n_pieces) return;
    int32_t* running = sh + 2 * (E + 1) + warp * E;
    for (int e = lane; e < E; e += 32) running[e] = table[static_cast<int64_t>(e) * n_pieces + p];
    __syncwarp();
    const int64_t beg = p * piece_len;
    const int64_t end = (beg + piece_len < R) ? beg + piece_len : R;
    const unsigned lt_mask = (1u << lane) - 1u;
    bool bad = false;
    int64_t raw_next = (beg + lane < end) ? ids[beg + lane] : -1;
    for (int64_t i0 = beg; i0 < end; i0 += 32) {
        const int64_t i = i0 + lane;
        const int64_t raw = raw_next;
        raw_next = (i + 32 < end) ? ids[i + 32] : -1;  // the next step's id is in flight during this one
        const bool in_piece = i < end;
        const bool ok = static_cast<uint64_t>(raw) < static_cast<uint64_t>(E);
        const int e = ok ? static_cast<int>(raw) : -1;
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
            const int32_t row = s_pad[e] + rank;
            if (row_of_slot != nullptr) row_of_slot[i] = row;
            if (slot_of_row != nullptr) slot_of_row[row] = static_cast<int32_t>(i);
            const int64_t q = static_cast<int64_t>(s_plain[e]) + rank;
            if (sorted_expert_idxs != nullptr) sorted_expert_idxs[q] = e;
            if (sorted_scattered_idxs != nullptr) sorted_scattered_idxs[q] = i;
        } else if (in_piece) {
            bad = true;
            if (row_of_slot != nullptr) row_of_slot[i] = -1;  // "no row": skipped by the row movers
        }
    }
    if (bad) atomicExch(status, STATUS_BAD_EXPERT_ID);
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

// ---------------------------------------------------------------------------
// launches
// ---------------------------------------------------------------------------
template <typename T>
static int launch_topk(const void* logits, int64_t rows, int E, int k, void* weights, int64_t* selected,
                       const RoutePlan& plan, int32_t* piece_hist, float* prob_part, cudaStream_t s) {
    const unsigned grid = static_cast<unsigned>((plan.n_pieces + kRouteWarps - 1) / kRouteWarps);
    const T* in = static_cast<const T*>(logits);
    T* w = static_cast<T*>(weights);
    const size_t smem = (piece_hist != nullptr) ? static_cast<size_t>(kRouteWarps) * E * 4 : 0;
    const int per_lane = (E + 31) / 32;
#define FMAB_TOPK(N)                                                                                              \
    topk_softmax_kernel<T, N><<<grid, kRouteThreads, smem, s>>>(in, rows, E, k, plan.tokens_per_piece, plan.n_pieces, \
                                                                w, selected, piece_hist, prob_part)
    if (per_lane <= 1) FMAB_TOPK(1);
    else if (per_lane <= 2) FMAB_TOPK(2);
    else if (per_lane <= 4) FMAB_TOPK(4);
    else if (per_lane <= 8) FMAB_TOPK(8);
    else if (per_lane <= 16) FMAB_TOPK(16);
    else FMAB_TOPK(32);
#undef FMAB_TOPK
    return check_launch("router_topk_softmax");
}

template <typename T>
static int launch_prob_backward(const void* logits, const float* d_mean, int64_t rows, int E, void* d_logits,
                                cudaStream_t s) {
    const unsigned grid = static_cast<unsigned>((rows + kRouteWarps - 1) / kRouteWarps);
    const T* in = static_cast<const T*>(logits);
    T* out = static_cast<T*>(d_logits);
    const float inv = 1.f / static_cast<float>(rows);
    const int per_lane = (E + 31) / 32;
#define FMAB_PROB(N) router_prob_backward_kernel<T, N><<<grid, kRouteThreads, 0, s>>>(in, d_mean, rows, E, inv, out)
    if (per_lane <= 1) FMAB_PROB(1);
    else if (per_lane <= 2) FMAB_PROB(2);
    else if (per_lane <= 4) FMAB_PROB(4);
    else if (per_lane <= 8) FMAB_PROB(8);
    else if (per_lane <= 16) FMAB_PROB(16);
    else FMAB_PROB(32);
#undef FMAB_PROB
    return check_launch("router_mean_prob_backward");
}

static int check_topk_args(int64_t T, int32_t E, int32_t k) {
    FMAB_REQUIRE(T >= 0 && T < (1LL << 31), FMA_B200_ERR_BAD_ARG, "T=%lld out of range", (long long)T);
    FMAB_REQUIRE(E >= 1 && E <= kMaxExperts, FMA_B200_ERR_BAD_ARG, "E=%d not in [1,%d]", E, kMaxExperts);
    FMAB_REQUIRE(k >= 1 && k <= E && k <= 32, FMA_B200_ERR_BAD_ARG, "k=%d not in [1,min(E,32)]", k);
    return FMA_B200_OK;
}

// The sort proper.  hist_ready: pass 1 was done by the top-k kernel with the plan of (R, E, k).
static int run_sort(const int64_t* selected, int64_t R, int32_t k, int32_t E, int32_t row_align, int64_t rows_cap,
                    int64_t* sorted_expert_idxs, int64_t* sorted_scattered_idxs, uint32_t* expert_count,
                    int32_t* pad_offsets, int32_t* row_of_slot, int32_t* slot_of_row, int32_t* mtile_expert,
                    float* prob_mean, bool hist_ready, bool probs_ready, void* workspace, int64_t workspace_bytes,
                    cudaStream_t s) {
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
    FMAB_REQUIRE(workspace_bytes >= route_workspace_bytes(E), FMA_B200_ERR_WORKSPACE,
                 "moe_sort workspace: %lld < %lld bytes", (long long)workspace_bytes, (long long)route_workspace_bytes(E));
    FMAB_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 3u) == 0, FMA_B200_ERR_BAD_ARG, "workspace not 4-byte aligned");
    int32_t* status = device_status_ptr();
    FMAB_REQUIRE(status != nullptr, FMA_B200_ERR_LAUNCH, "no device status word");
    const RoutePlan plan = make_plan(R, E, k);
    const RouteWorkspace ws = carve_workspace(workspace, E);
    const unsigned piece_blocks = static_cast<unsigned>((plan.n_pieces + kRouteWarps - 1) / kRouteWarps);
    if (slot_of_row != nullptr) FMAB_CUDA(cudaMemsetAsync(slot_of_row, 0xff, static_cast<size_t>(rows_cap) * 4, s));
    if (!hist_ready || R == 0) {
        sort_hist_kernel<<<piece_blocks, kRouteThreads, static_cast<size_t>(kRouteWarps) * E * 4, s>>>(
            selected, R, E, plan.piece, plan.n_pieces, ws.hist, status);
        if (int rc = check_launch("moe_sort/hist")) return rc;
    }
    const bool probs = probs_ready && prob_mean != nullptr && R > 0;
    sort_scan_kernel<<<(E + kRouteWarps - 1) / kRouteWarps, kRouteThreads, 0, s>>>(
        ws.hist, plan.n_pieces, E, ws.totals, probs ? ws.prob : nullptr,
        probs ? 1.f / static_cast<float>(R / k) : 0.f, prob_mean);
    if (int rc = check_launch("moe_sort/scan")) return rc;
    const size_t place_smem = (2 * static_cast<size_t>(E + 1) + static_cast<size_t>(kRouteWarps) * E) * 4;
    sort_place_kernel<<<piece_blocks, kRouteThreads, place_smem, s>>>(
        selected, R, E, plan.piece, plan.n_pieces, ws.hist, ws.totals, row_align, rows_cap, sorted_expert_idxs,
        sorted_scattered_idxs, expert_count, pad_offsets, row_of_slot, slot_of_row, mtile_expert, status);
    return check_launch("moe_sort/place");
}

}  // namespace fmab

extern "C" {

int fma_b200_router_topk_softmax(const void* logits, int32_t dtype, int64_t T, int32_t E, int32_t k, void* weights,
                                 int64_t* selected, void* stream) {
    using namespace fmab;
    if (int rc = check_topk_args(T, E, k)) return rc;
    if (T == 0) return FMA_B200_OK;
    FMAB_REQUIRE(logits && weights && selected, FMA_B200_ERR_BAD_ARG, "NULL pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const RoutePlan plan = make_plan(T * k, E, k);
    int rc = FMA_B200_OK;
    if (!dispatch_dtype(dtype, [&](auto tag) {
            rc = launch_topk<decltype(tag)>(logits, T, E, k, weights, selected, plan, nullptr, nullptr, s);
        }))
        return fail(FMA_B200_ERR_UNSUPPORTED, "router_topk_softmax: dtype %d", dtype);
    return rc;
}

int fma_b200_router_topk_softmax_routed(const void* logits, int32_t dtype, int64_t T, int32_t E, int32_t k,
                                        void* weights, int64_t* selected, int32_t want_probs, void* sort_workspace,
                                        int64_t workspace_bytes, void* stream) {
    using namespace fmab;
    if (int rc = check_topk_args(T, E, k)) return rc;
    FMAB_REQUIRE(sort_workspace != nullptr && (reinterpret_cast<uintptr_t>(sort_workspace) & 3u) == 0,
                 FMA_B200_ERR_BAD_ARG, "sort_workspace NULL or not 4-byte aligned");
    FMAB_REQUIRE(workspace_bytes >= route_workspace_bytes(E), FMA_B200_ERR_WORKSPACE,
                 "router workspace: %lld < %lld bytes", (long long)workspace_bytes, (long long)route_workspace_bytes(E));
    if (T == 0) return FMA_B200_OK;
    FMAB_REQUIRE(logits && weights && selected, FMA_B200_ERR_BAD_ARG, "NULL pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const RoutePlan plan = make_plan(T * k, E, k);
    const RouteWorkspace ws = carve_workspace(sort_workspace, E);
    float* prob = want_probs ? ws.prob : nullptr;
    int rc = FMA_B200_OK;
    if (!dispatch_dtype(dtype, [&](auto tag) {
            rc = launch_topk<decltype(tag)>(logits, T, E, k, weights, selected, plan, ws.hist, prob, s);
        }))
        return fail(FMA_B200_ERR_UNSUPPORTED, "router_topk_softmax_routed: dtype %d", dtype);
    return rc;
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
    const unsigned grid = static_cast<unsigned>((T + kRouteWarps - 1) / kRouteWarps);
    if (!dispatch_dtype(dtype, [&](auto tag) {
            using Elt = decltype(tag);
            topk_softmax_backward_kernel<Elt><<<grid, kRouteThreads, 0, s>>>(
                static_cast<const Elt*>(weights), static_cast<const Elt*>(d_weights), selected, T, E, k,
                static_cast<Elt*>(d_logits));
        }))
        return fail(FMA_B200_ERR_UNSUPPORTED, "router_topk_softmax_backward: dtype %d", dtype);
    return check_launch("router_topk_softmax_backward");
}

int fma_b200_router_mean_prob_backward(const void* logits, const float* d_mean_prob, int32_t dtype, int64_t T,
                                       int32_t E, void* d_logits, void* stream) {
    using namespace fmab;
    FMAB_REQUIRE(T >= 0 && T < (1LL << 31), FMA_B200_ERR_BAD_ARG, "T=%lld out of range", (long long)T);
    FMAB_REQUIRE(E >= 1 && E <= kMaxExperts, FMA_B200_ERR_BAD_ARG, "E=%d not in [1,%d]", E, kMaxExperts);
    if (T == 0) return FMA_B200_OK;
    FMAB_REQUIRE(logits && d_mean_prob && d_logits, FMA_B200_ERR_BAD_ARG, "NULL pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int rc = FMA_B200_OK;
    if (!dispatch_dtype(dtype, [&](auto tag) {
            rc = launch_prob_backward<decltype(tag)>(logits, d_mean_prob, T, E, d_logits, s);
        }))
        return fail(FMA_B200_ERR_UNSUPPORTED, "router_mean_prob_backward: dtype %d", dtype);
    return rc;
}

int64_t fma_b200_moe_rows_cap(int64_t R, int32_t E, int32_t row_align) {
    if (R < 0 || E < 1 || row_align < 1) return 0;
    // Every expert wastes at most row_align-1 rows; round the total up to whole 128-row tiles.
    const int64_t worst = R + static_cast<int64_t>(E) * (row_align - 1);
    return ((worst + 127) / 128) * 128;
}

int64_t fma_b200_moe_sort_workspace_bytes(int64_t R, int32_t E) {
    if (R < 0 || E < 1 || E > fmab::kMaxExperts) return 0;
    return fmab::route_workspace_bytes(E);
}

int fma_b200_moe_sort(const int64_t* selected, int64_t R, int32_t E, int32_t row_align, int64_t rows_cap,
                      int64_t* sorted_expert_idxs, int64_t* sorted_scattered_idxs, uint32_t* expert_count,
                      int32_t* pad_offsets, int32_t* row_of_slot, int32_t* slot_of_row, int32_t* mtile_expert,
                      void* workspace, int64_t workspace_bytes, void* stream) {
    return fmab::run_sort(selected, R, 1, E, row_align, rows_cap, sorted_expert_idxs, sorted_scattered_idxs,
                          expert_count, pad_offsets, row_of_slot, slot_of_row, mtile_expert, nullptr, false, false,
                          workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

int fma_b200_moe_sort_routed(const int64_t* selected, int64_t T, int32_t k, int32_t E, int32_t row_align,
                             int64_t rows_cap, int64_t* sorted_expert_idxs, int64_t* sorted_scattered_idxs,
                             uint32_t* expert_count, int32_t* pad_offsets, int32_t* row_of_slot, int32_t* slot_of_row,
                             int32_t* mtile_expert, float* router_mean_prob, void* workspace, int64_t workspace_bytes,
                             void* stream) {
    using namespace fmab;
    FMAB_REQUIRE(T >= 0 && T < (1LL << 31), FMA_B200_ERR_BAD_ARG, "T=%lld out of range", (long long)T);
    FMAB_REQUIRE(k >= 1 && k <= 32, FMA_B200_ERR_BAD_ARG, "k=%d not in [1,32]", k);
    return run_sort(selected, T * k, k, E, row_align, rows_cap, sorted_expert_idxs, sorted_scattered_idxs, expert_count,
                    pad_offsets, row_of_slot, slot_of_row, mtile_expert, router_mean_prob, true,
                    router_mean_prob != nullptr, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
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
