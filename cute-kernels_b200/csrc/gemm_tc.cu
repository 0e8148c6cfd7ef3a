// bf16 grouped GEMM on the 5th-generation tensor cores (tcgen05) of sm_100a.
//
// One persistent CTA per SM, 320 threads, warp-specialised:
//   warp 0      TMA producer: cp.async.bulk.tensor loads of A/B k-blocks into a 4-stage
//               shared-memory ring (128-byte swizzle), signalled by mbarrier transaction counts;
//   warp 1      MMA issuer: one thread issues tcgen05.mma (M=128, N=256, K=16, bf16 in, fp32
//               accumulate in tensor memory); tcgen05.commit releases ring stages and publishes
//               finished accumulators;
//   warps 2-9   epilogue: tcgen05.ld of the accumulator (one TMEM lane = one output row per
//               thread; warps 2-5 take the first half of the tile's columns, warps 6-9 the second),
//               optional SwiGLU forward / backward math, bf16 rounding, 128-bit stores.
// Tensor memory holds two 128x256 fp32 accumulators (all 512 columns), so the epilogue of tile
// i overlaps the main loop of tile i+1.  Tiles are drawn from a global counter by the producer thread
// and published to the other warps through a small shared-memory ring, so CTAs that start late or
// draw long tiles take fewer of them.
//
// Operands may be K-major (the reduction index is contiguous in memory) or MN-major (the row /
// column index is contiguous); the latter is what dgrad (B = W[e], [K,N] row-major) and wgrad
// (A = dY^T, B = X, both [tokens, features] row-major) need, so no transposed copies are made.
// Every TMA load targets the issuing CTA's own shared memory; no thread-block clusters are used.
//
// Every mbarrier wait is bounded (about one second of %globaltimer); a wait that runs out sets
// the device status word, raises a CTA-wide abort flag that all other waits poll, and the CTA
// leaves its role loops, frees its tensor memory and exits; the host reads the status word.
#include <vector>

#include "gemm_tc.cuh"

namespace fmab {

// ---------------------------------------------------------------------------
// tile decode (identical in all three roles)
// ---------------------------------------------------------------------------
struct Tile {
    const CUtensorMap* map_a;
    const CUtensorMap* map_b;
    int32_t group;
    int32_t a_mn;        // A coordinate along M
    int32_t b_mn;        // B coordinate along N (of tile column 0)
    int32_t b_k_base;    // added to B's k coordinate (rows mode, MN-major stacked weights)
    int32_t n0;          // first D column of the tile
    int32_t n_valid;     // D columns to store
    int32_t rows_valid;  // D rows to store
    int64_t d_row;       // first D row (in units of ldd) ...
    int64_t d_base;      // ... plus element offset of the group's output (general mode)
    int64_t ldd;
};

// m-tile index of a linear tile id (SUPER_M m-tiles are walked together, n-tile by n-tile).
__device__ __forceinline__ int tile_to_mtile(const GemmParams& p, int tile, int& nt) {
    const int per_super = SUPER_M * p.n_ntiles;
    const int super = tile / per_super;
    const int m_first = super * SUPER_M;
    const int m_span = min(SUPER_M, p.n_mtiles - m_first);
    const int r = tile - super * per_super;
    nt = r / m_span;
    return m_first + (r - nt * m_span);
}
// Rows mode: the expert id of a tile, loaded early so that its latency hides behind the previous tile.
__device__ __forceinline__ int peek_expert(const GemmParams& p, int tile, int total_tiles) {
    if (p.mode != MODE_ROWS || tile >= total_tiles) return -1;
    int nt;
    return __ldg(p.mtile_expert + tile_to_mtile(p, tile, nt));
}

template <bool B_MN, int EPI>
__device__ __forceinline__ bool decode_tile(const GemmParams& p, int tile, int expert_hint, Tile& t) {
    int nt;
    const int mt = tile_to_mtile(p, tile, nt);
    constexpr int n_step = (EPI == EPI_SWIGLU_FWD) ? BN / 2 : BN;
    t.n0 = nt * n_step;
    t.map_a = &p.map_a;
    t.map_b = &p.map_b;
    t.b_k_base = 0;
    t.d_base = 0;
    t.ldd = p.ldd;
    if (p.mode == MODE_ROWS) {
        const int e = expert_hint;  // == mtile_expert[mt], fetched one tile ahead
        if (e < 0) return false;
        t.group = e;
        t.a_mn = mt * BM;
        t.d_row = static_cast<int64_t>(mt) * BM;
        t.rows_valid = BM;
        t.n_valid = min(n_step, p.n_cols - t.n0);
        if (B_MN) {
            t.b_mn = t.n0;
            t.b_k_base = e * p.b_group_stride;
        } else {
            t.b_mn = e * p.b_group_stride + t.n0;
        }
    } else if (p.mode == MODE_WGRAD) {
        const int e = mt / p.mtiles_per_group;
        const int m0 = (mt - e * p.mtiles_per_group) * BM;
        t.group = e;
        t.a_mn = m0;
        t.b_mn = t.n0;
        t.d_row = static_cast<int64_t>(e) * p.m_per_group + m0;
        t.rows_valid = min(BM, p.m_per_group - m0);
        t.n_valid = min(n_step, p.n_cols - t.n0);
    } else {
        const MTileRec rec = p.mtiles[mt];
        const GroupRec g = p.groups[rec.group];
        if (t.n0 >= g.n) return false;
        t.group = rec.group;
        t.map_a = p.group_maps + 2 * rec.group;
        t.map_b = p.group_maps + 2 * rec.group + 1;
        t.a_mn = rec.row0;
        t.b_mn = t.n0;
        t.d_row = rec.row0;
        t.d_base = g.d_offset;
        t.ldd = g.n;
        t.rows_valid = min(BM, g.m - rec.row0);
        t.n_valid = min(n_step, g.n - t.n0);
    }
    return true;
}

// k range of segment s of the tile's group: start coordinates in A and B, and length.
__device__ __forceinline__ void decode_segment(const GemmParams& p, const Tile& t, int s, int& a_k0, int& b_k0, int& len) {
    if (p.mode == MODE_ROWS) {
        a_k0 = 0;
        b_k0 = t.b_k_base;
        len = p.k_len;
    } else if (p.mode == MODE_WGRAD) {
        const int32_t* o = p.seg_offsets + s * p.n_groups + t.group;
        a_k0 = o[0];
        b_k0 = o[0];
        len = o[1] - o[0];
    } else {
        a_k0 = 0;
        b_k0 = 0;
        len = p.groups[t.group].k;
    }
}

// ---------------------------------------------------------------------------
// the kernel
// ---------------------------------------------------------------------------
template <bool A_MN, bool B_MN, int EPI, int EPI_WARPS>
__global__ void __launch_bounds__(64 + 32 * EPI_WARPS, 1) gemm_tc_kernel(const __grid_constant__ GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[STAGES];
    __shared__ __align__(8) uint64_t empty_bar[STAGES];
    __shared__ __align__(8) uint64_t acc_full_bar[2];
    __shared__ __align__(8) uint64_t acc_empty_bar[2];
    __shared__ __align__(8) uint64_t sched_full_bar[SCHED_SLOTS];
    __shared__ __align__(8) uint64_t sched_empty_bar[SCHED_SLOTS];
    __shared__ volatile int sched_tile[SCHED_SLOTS];
    __shared__ volatile int sched_expert[SCHED_SLOTS];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;  // swizzle atoms need 1024-byte alignment

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&acc_full_bar[b]), 1);
            mbar_init(smem_u32(&acc_empty_bar[b]), EPI_WARPS);  // one arrival per epilogue warp
        }
        for (int i = 0; i < SCHED_SLOTS; ++i) {
            mbar_init(smem_u32(&sched_full_bar[i]), 1);
            mbar_init(smem_u32(&sched_empty_bar[i]), 1 + EPI_WARPS);  // MMA thread + every epilogue warp
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)),
                     "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;
    volatile int* abort_ptr = &abort_flag;

    const int total_tiles = p.n_mtiles * p.n_ntiles;
    const int n_seg = (p.mode == MODE_WGRAD) ? p.n_seg : 1;

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool alive = true;
            // This thread is also the tile scheduler: tiles are handed out by a global counter (the first
            // one is blockIdx.x), so CTAs that start late or draw long tiles simply take fewer of them.
            int sslot = 0;
            uint32_t sphase = 0;
            int tile = blockIdx.x;
            int e_cur = peek_expert(p, tile, total_tiles);
            while (alive) {
                if (!mbar_wait(smem_u32(&sched_empty_bar[sslot]), sphase ^ 1u, abort_ptr, p.status)) {
                    alive = false;
                    break;
                }
                const bool end = tile >= total_tiles;
                sched_tile[sslot] = end ? -1 : tile;
                sched_expert[sslot] = e_cur;
                mbar_arrive(smem_u32(&sched_full_bar[sslot]));  // release: the two stores above are visible to waiters
                if (++sslot == SCHED_SLOTS) {
                    sslot = 0;
                    sphase ^= 1u;
                }
                if (end) break;
                // drawn now, needed only after this tile's loads have been issued
                const int next = p.dynamic_tiles ? static_cast<int>(atomicAdd(p.sched, 1u)) + static_cast<int>(gridDim.x)
                                                 : tile + static_cast<int>(gridDim.x);
                Tile t;
                if (decode_tile<B_MN, EPI>(p, tile, e_cur, t)) {
                    if (p.mode == MODE_GENERAL) {
                        tensormap_acquire(t.map_a);
                        tensormap_acquire(t.map_b);
                    }
                    for (int s = 0; s < n_seg && alive; ++s) {
                        int a_k0, b_k0, len;
                        decode_segment(p, t, s, a_k0, b_k0, len);
                        for (int k = 0; k < len; k += BK) {
                            if (!mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1u, abort_ptr, p.status)) {
                                alive = false;
                                break;
                            }
                            const uint32_t bar = smem_u32(&full_bar[stage]);
                            const uint32_t sa = ring + stage * STAGE_BYTES;
                            const uint32_t sb = sa + A_STAGE_BYTES;
                            mbar_arrive_expect_tx(bar, STAGE_BYTES);
                            if (A_MN) {
#pragma unroll
                                for (int j = 0; j < BM / 64; ++j)
                                    tma_load_2d(sa + j * (BK * 128), t.map_a, bar, t.a_mn + 64 * j, a_k0 + k);
                            } else {
                                tma_load_2d(sa, t.map_a, bar, a_k0 + k, t.a_mn);
                            }
                            if (B_MN) {
#pragma unroll
                                for (int j = 0; j < BN / 64; ++j)
                                    tma_load_2d(sb + j * (BK * 128), t.map_b, bar, t.b_mn + 64 * j, b_k0 + k);
                            } else if (EPI == EPI_SWIGLU_FWD) {
                                // up rows n0.. and gate rows I+n0.. of the same expert, 128 each
                                tma_load_2d(sb, t.map_b, bar, b_k0 + k, t.b_mn);
                                tma_load_2d(sb + (BN / 2) * (BK * 2), t.map_b, bar, b_k0 + k, t.b_mn + p.inter);
                            } else {
                                tma_load_2d(sb, t.map_b, bar, b_k0 + k, t.b_mn);
                            }
                            if (++stage == STAGES) {
                                stage = 0;
                                phase ^= 1u;
                            }
                        }
                    }
                }
                tile = next;
                e_cur = peek_expert(p, tile, total_tiles);
            }
            if (!alive) {
                // give copies that are still in flight time to land before the CTA retires
                for (int i = 0; i < 200; ++i) __nanosleep(1000);
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0) {
            const uint32_t idesc = with_operand_format(make_instr_desc<A_MN, B_MN>(), p.f16 != 0);
            int stage = 0;
            uint32_t phase = 0;
            int buf = 0;
            uint32_t acc_phase = 0;
            bool alive = true;
            int sslot = 0;
            uint32_t sphase = 0;
            while (alive) {
                if (!mbar_wait(smem_u32(&sched_full_bar[sslot]), sphase, abort_ptr, p.status)) break;
                const int tile = sched_tile[sslot];
                const int e_cur = sched_expert[sslot];
                mbar_arrive(smem_u32(&sched_empty_bar[sslot]));
                if (++sslot == SCHED_SLOTS) {
                    sslot = 0;
                    sphase ^= 1u;
                }
                if (tile < 0) break;
                Tile t;
                if (!decode_tile<B_MN, EPI>(p, tile, e_cur, t)) continue;
                if (!mbar_wait(smem_u32(&acc_empty_bar[buf]), acc_phase ^ 1u, abort_ptr, p.status)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * BN;
                uint32_t accumulate = 0;
                for (int s = 0; s < n_seg && alive; ++s) {
                    int a_k0, b_k0, len;
                    decode_segment(p, t, s, a_k0, b_k0, len);
                    for (int k = 0; k < len; k += BK) {
                        if (!mbar_wait(smem_u32(&full_bar[stage]), phase, abort_ptr, p.status)) {
                            alive = false;
                            break;
                        }
                        tc_fence_after();
                        const uint32_t sa = ring + stage * STAGE_BYTES;
                        const uint32_t sb = sa + A_STAGE_BYTES;
                        const uint64_t a_desc = make_smem_desc<A_MN>(sa);
                        const uint64_t b_desc = make_smem_desc<B_MN>(sb);
#pragma unroll
                        for (int ks = 0; ks < BK / UMMA_K; ++ks) {
                            tc_mma(d_tmem, a_desc + ((ks * desc_k_step<A_MN>()) >> 4),
                                   b_desc + ((ks * desc_k_step<B_MN>()) >> 4), idesc, accumulate);
                            accumulate = 1;
                        }
                        tc_commit(smem_u32(&empty_bar[stage]));  // stage is free once these MMAs have read it
                        if (++stage == STAGES) {
                            stage = 0;
                            phase ^= 1u;
                        }
                    }
                }
                if (!alive) break;
                if (accumulate) tc_commit(smem_u32(&acc_full_bar[buf]));
                else mbar_arrive(smem_u32(&acc_full_bar[buf]));  // empty reduction: the epilogue writes zeros
                if (++buf == 2) {
                    buf = 0;
                    acc_phase ^= 1u;
                }
            }
        }
    } else {
        // ------------------------------ epilogue ------------------------------
        const int quad = warp & 3;          // TMEM lanes [32*quad, 32*quad+32) are visible to this warp
        constexpr int kColSplit = EPI_WARPS / 4;  // 1: every warp stores all columns of its rows; 2: half each
        const int half = (warp - 2) >> 2;         // which part of the tile's columns this warp stores
        const int row_in_tile = quad * 32 + lane;
        const bool f16 = p.f16 != 0;
        int buf = 0;
        uint32_t acc_phase = 0;
        int sslot = 0;
        uint32_t sphase = 0;
        while (true) {
            if (!mbar_wait(smem_u32(&sched_full_bar[sslot]), sphase, abort_ptr, p.status)) break;
            const int tile = sched_tile[sslot];
            const int e_cur = sched_expert[sslot];
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&sched_empty_bar[sslot]));
            if (++sslot == SCHED_SLOTS) {
                sslot = 0;
                sphase ^= 1u;
            }
            if (tile < 0) break;
            Tile t;
            if (!decode_tile<B_MN, EPI>(p, tile, e_cur, t)) continue;
            // Does this tile have any reduction work?  (Same test as the MMA issuer's.)
            bool any_k = false;
            for (int s = 0; s < n_seg; ++s) {
                int a_k0, b_k0, len;
                decode_segment(p, t, s, a_k0, b_k0, len);
                any_k |= len > 0;
            }
            if (!mbar_wait(smem_u32(&acc_full_bar[buf]), acc_phase, abort_ptr, p.status)) break;
            tc_fence_after();
            const uint32_t taddr = tmem_base + buf * BN + (static_cast<uint32_t>(quad * 32) << 16);
            const bool row_ok = row_in_tile < t.rows_valid;
            const int64_t grow = t.d_row + row_in_tile;

            if (EPI == EPI_PLAIN) {
                __nv_bfloat16* drow = p.d + t.d_base + grow * t.ldd + t.n0;
                constexpr int kChunks = BN / 32 / kColSplit;
#pragma unroll 1
                for (int c = half * kChunks; c < (half + 1) * kChunks; ++c) {
                    const int cols_left = t.n_valid - c * 32;
                    if (cols_left <= 0) break;
                    float v[32];
                    if (any_k) {
                        tc_load_32(taddr + c * 32, v);
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = 0.f;
                    }
                    if (row_ok) store_row32(drow + c * 32, v, cols_left, f16);
                }
            } else if (EPI == EPI_SWIGLU_FWD) {
                // accumulator columns [0,128) = up, [128,256) = gate, for act columns n0..n0+127
                __nv_bfloat16* arow = p.d + grow * p.ldd + t.n0;
                __nv_bfloat16* prow = p.d2 ? p.d2 + grow * (2 * static_cast<int64_t>(p.inter)) + t.n0 : nullptr;
                constexpr int kChunks = BN / 64 / kColSplit;
#pragma unroll 1
                for (int c = half * kChunks; c < (half + 1) * kChunks; ++c) {
                    const int cols_left = t.n_valid - c * 32;
                    if (cols_left <= 0) break;
                    float u[32], g[32];
                    tc_load_32(taddr + c * 32, u);
                    tc_load_32(taddr + BN / 2 + c * 32, g);
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        u[i] = round16(u[i], f16);
                        g[i] = round16(g[i], f16);
                    }
                    if (row_ok && prow) {
                        store_row32(prow + c * 32, u, cols_left, f16);
                        store_row32(prow + p.inter + c * 32, g, cols_left, f16);
                    }
#pragma unroll
                    for (int i = 0; i < 32; ++i) u[i] = u[i] * g[i] * sigmoid_clamped_fast(g[i]);
                    if (row_ok) store_row32(arow + c * 32, u, cols_left, f16);
                }
            } else {
                // d_act tile -> d_up, d_gate using the saved pre-activations.  The up/gate values of the
                // next 32 columns are fetched while the current ones are processed.
                const __nv_bfloat16* prow = p.pre + grow * (2 * static_cast<int64_t>(p.inter)) + t.n0;
                __nv_bfloat16* drow = p.d + grow * (2 * static_cast<int64_t>(p.inter)) + t.n0;
                constexpr int kChunks = BN / 32 / kColSplit;
                const int c_begin = half * kChunks, c_end = (half + 1) * kChunks;
                uint4 nu[4], ng[4];
                auto fetch = [&](int c) {
                    const int cols_left = t.n_valid - c * 32;
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const bool ok = row_ok && q * 8 < cols_left;
                        nu[q] = ok ? ld_global_16(prow + c * 32 + q * 8) : make_uint4(0, 0, 0, 0);
                        ng[q] = ok ? ld_global_16(prow + p.inter + c * 32 + q * 8) : make_uint4(0, 0, 0, 0);
                    }
                };
                fetch(c_begin);
#pragma unroll 1
                for (int c = c_begin; c < c_end; ++c) {
                    const int cols_left = t.n_valid - c * 32;
                    if (cols_left <= 0) break;
                    float da[32], u[32], g[32];
                    tc_load_32(taddr + c * 32, da);
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        unpack8(nu[q], u + q * 8, f16);
                        unpack8(ng[q], g + q * 8, f16);
                    }
                    if (c + 1 < c_end) fetch(c + 1);
                    if (row_ok) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const float d = round16(da[i], f16);
                            const float s = sigmoid_clamped_fast(g[i]);
                            const float silu = g[i] * s;
                            da[i] = d * silu;                           // d_up
                            g[i] = d * u[i] * (s + silu * (1.f - s));   // d_gate
                        }
                        store_row32(drow + c * 32, da, cols_left, f16);
                        store_row32(drow + p.inter + c * 32, g, cols_left, f16);
                    }
                }
            }
            // all of this warp's TMEM reads are complete (tcgen05.wait::ld inside tc_load_32)
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&acc_empty_bar[buf]));
            if (++buf == 2) {
                buf = 0;
                acc_phase ^= 1u;
            }
        }
    }

    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
    if (threadIdx.x == 0) {
        // the last CTA to leave puts the scheduler words back to zero for the next launch that uses them
        __threadfence();
        if (atomicAdd(p.sched + 1, 1u) == gridDim.x - 1) {
            p.sched[0] = 0;
            p.sched[1] = 0;
            __threadfence();
        }
    }
}

// Epilogue width: 8 warps (two per TMEM lane quadrant) by default; FMA_B200_GEMM_EPI_WARPS=4 selects
// the narrower build (a tuning knob for measurements).
static int epilogue_warps() {
    static int cached = 0;
    if (cached == 0) {
        const char* env = getenv("FMA_B200_GEMM_EPI_WARPS");
        cached = (env != nullptr && atoi(env) == 4) ? 4 : 8;
    }
    return cached;
}

template <bool A_MN, bool B_MN, int EPI, int EPI_WARPS>
static int launch_gemm_w(const GemmParams& p_in, cudaStream_t s) {
    GemmParams p = p_in;
    if (int rc = next_sched_pair(&p.sched)) return rc;
    p.dynamic_tiles = dynamic_tiles_enabled();
    static bool configured[64] = {false};  // per device: the attribute applies to the current device only
    auto kernel = gemm_tc_kernel<A_MN, B_MN, EPI, EPI_WARPS>;
    const int dev = current_device_slot();
    FMAB_REQUIRE(dev >= 0, FMA_B200_ERR_LAUNCH, "no current CUDA device with an ordinal below 64");
    if (!configured[dev]) {
        FMAB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GEMM_SMEM_BYTES));
        configured[dev] = true;
    }
    const int64_t total = static_cast<int64_t>(p.n_mtiles) * p.n_ntiles;
    if (total <= 0) return FMA_B200_OK;
    FMAB_REQUIRE(total < (1LL << 31), FMA_B200_ERR_BAD_ARG, "too many tiles");
    const int grid = static_cast<int>(total < sm_count() ? total : sm_count());
    kernel<<<grid, 64 + 32 * EPI_WARPS, GEMM_SMEM_BYTES, s>>>(p);
    return check_launch("grouped GEMM (tcgen05)");
}

template <bool A_MN, bool B_MN, int EPI>
static int launch_gemm(const GemmParams& p, cudaStream_t s) {
    if (epilogue_warps() == 4) return launch_gemm_w<A_MN, B_MN, EPI, 4>(p, s);
    return launch_gemm_w<A_MN, B_MN, EPI, 8>(p, s);
}

static int fill_common(GemmParams& p) {
    memset(&p, 0, sizeof(p));
    p.status = device_status_ptr();
    FMAB_REQUIRE(p.status != nullptr, FMA_B200_ERR_LAUNCH, "no device status word");
    p.n_seg = 1;
    return FMA_B200_OK;
}

int tc_forward(const void* X, const void* W, void* Y, int64_t rows_cap, int E, int OUT, int IN,
               const int32_t* mtile_expert, bool f16, cudaStream_t s) {
    GemmParams p;
    if (int rc = fill_common(p)) return rc;
    p.f16 = f16 ? 1 : 0;
    if (int rc = encode_2d(&p.map_a, X, IN, rows_cap, IN, BK, BM, f16)) return rc;
    if (int rc = encode_2d(&p.map_b, W, IN, static_cast<uint64_t>(E) * OUT, IN, BK, BN, f16)) return rc;
    p.mode = MODE_ROWS;
    p.mtile_expert = mtile_expert;
    p.d = static_cast<__nv_bfloat16*>(Y);
    p.ldd = OUT;
    p.n_mtiles = static_cast<int>(rows_cap / BM);
    p.n_ntiles = (OUT + BN - 1) / BN;
    p.n_cols = OUT;
    p.k_len = IN;
    p.b_group_stride = OUT;
    p.n_groups = E;
    return launch_gemm<false, false, EPI_PLAIN>(p, s);
}

int tc_forward_swiglu(const void* X, const void* W, void* pre, void* act, int64_t rows_cap, int E, int I, int IN,
                      const int32_t* mtile_expert, bool f16, cudaStream_t s) {
    GemmParams p;
    if (int rc = fill_common(p)) return rc;
    p.f16 = f16 ? 1 : 0;
    if (int rc = encode_2d(&p.map_a, X, IN, rows_cap, IN, BK, BM, f16)) return rc;
    if (int rc = encode_2d(&p.map_b, W, IN, static_cast<uint64_t>(E) * 2 * I, IN, BK, BN / 2, f16)) return rc;
    p.mode = MODE_ROWS;
    p.mtile_expert = mtile_expert;
    p.d = static_cast<__nv_bfloat16*>(act);
    p.d2 = static_cast<__nv_bfloat16*>(pre);
    p.ldd = I;
    p.inter = I;
    p.n_mtiles = static_cast<int>(rows_cap / BM);
    p.n_ntiles = (I + BN / 2 - 1) / (BN / 2);
    p.n_cols = I;
    p.k_len = IN;
    p.b_group_stride = 2 * I;
    p.n_groups = E;
    return launch_gemm<false, false, EPI_SWIGLU_FWD>(p, s);
}

int tc_dgrad(const void* dY, const void* W, void* dX, const void* pre, int64_t rows_cap, int E, int OUT, int IN,
             const int32_t* mtile_expert, bool swiglu, bool f16, cudaStream_t s) {
    GemmParams p;
    if (int rc = fill_common(p)) return rc;
    p.f16 = f16 ? 1 : 0;
    if (int rc = encode_2d(&p.map_a, dY, OUT, rows_cap, OUT, BK, BM, f16)) return rc;
    // W[e] is [OUT, IN] row-major = the [K, N] operand with N contiguous: MN-major B, boxes of 64 columns x BK rows
    if (int rc = encode_2d(&p.map_b, W, IN, static_cast<uint64_t>(E) * OUT, IN, 64, BK, f16)) return rc;
    p.mode = MODE_ROWS;
    p.mtile_expert = mtile_expert;
    p.d = static_cast<__nv_bfloat16*>(dX);
    p.pre = static_cast<const __nv_bfloat16*>(pre);
    p.ldd = swiglu ? 2 * static_cast<int64_t>(IN) : IN;
    p.inter = IN;
    p.n_mtiles = static_cast<int>(rows_cap / BM);
    p.n_ntiles = (IN + BN - 1) / BN;
    p.n_cols = IN;
    p.k_len = OUT;
    p.b_group_stride = OUT;
    p.n_groups = E;
    if (swiglu) return launch_gemm<false, true, EPI_SWIGLU_BWD>(p, s);
    return launch_gemm<false, true, EPI_PLAIN>(p, s);
}

int tc_wgrad(const void* dY, const void* X, void* dW, int64_t rows_cap, int E, int OUT, int IN,
             const int32_t* seg_offsets, int n_seg, bool f16, cudaStream_t s) {
    GemmParams p;
    if (int rc = fill_common(p)) return rc;
    // both operands are [tokens, features] row-major: the token (reduction) index is the outer dimension
    if (int rc = encode_2d(&p.map_a, dY, OUT, rows_cap, OUT, 64, BK, f16)) return rc;
    if (int rc = encode_2d(&p.map_b, X, IN, rows_cap, IN, 64, BK, f16)) return rc;
    p.mode = MODE_WGRAD;
    p.seg_offsets = seg_offsets;
    p.n_seg = n_seg;
    p.d = static_cast<__nv_bfloat16*>(dW);
    p.ldd = IN;
    p.m_per_group = OUT;
    p.mtiles_per_group = (OUT + BM - 1) / BM;
    p.n_mtiles = E * p.mtiles_per_group;
    p.n_ntiles = (IN + BN - 1) / BN;
    p.n_cols = IN;
    p.n_groups = E;
    return launch_gemm<true, true, EPI_PLAIN>(p, s);
}

struct GeneralLayout {
    int64_t groups_off, mtiles_off, maps_off, total;
};
static GeneralLayout general_layout(int n_groups, int64_t total_mtiles) {
    GeneralLayout l;
    l.maps_off = 0;  // tensor maps first: they need 64-byte alignment (the workspace must be 128-byte aligned)
    l.groups_off = static_cast<int64_t>(n_groups) * 2 * sizeof(CUtensorMap);
    l.mtiles_off = l.groups_off + ((static_cast<int64_t>(n_groups) * sizeof(GroupRec) + 127) / 128) * 128;
    l.total = l.mtiles_off + ((total_mtiles * static_cast<int64_t>(sizeof(MTileRec)) + 127) / 128) * 128;
    return l;
}

int tc_general(const void* A, const void* B, void* D, const uint32_t* M, const uint32_t* N, const uint32_t* K,
               int n_groups, bool a_t, bool b_t, void* workspace, int64_t workspace_bytes, cudaStream_t s) {
    FMAB_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 127u) == 0, FMA_B200_ERR_BAD_ARG,
                 "grouped_gemm workspace must be 128-byte aligned");
    int64_t total_mtiles = 0;
    uint32_t max_n = 0;
    for (int g = 0; g < n_groups; ++g) {
        total_mtiles += (M[g] + BM - 1) / BM;
        if (N[g] > max_n) max_n = N[g];
    }
    const GeneralLayout lay = general_layout(n_groups, total_mtiles);
    FMAB_REQUIRE(workspace_bytes >= lay.total, FMA_B200_ERR_WORKSPACE, "grouped_gemm workspace: %lld < %lld bytes",
                 (long long)workspace_bytes, (long long)lay.total);
    if (total_mtiles == 0 || max_n == 0) return FMA_B200_OK;
    std::vector<uint8_t> host(static_cast<size_t>(lay.total), 0);
    CUtensorMap* maps = reinterpret_cast<CUtensorMap*>(host.data() + lay.maps_off);
    GroupRec* groups = reinterpret_cast<GroupRec*>(host.data() + lay.groups_off);
    MTileRec* mtiles = reinterpret_cast<MTileRec*>(host.data() + lay.mtiles_off);
    const __nv_bfloat16* a = static_cast<const __nv_bfloat16*>(A);
    const __nv_bfloat16* b = static_cast<const __nv_bfloat16*>(B);
    int64_t a_off = 0, b_off = 0, d_off = 0;
    int32_t mt = 0;
    for (int g = 0; g < n_groups; ++g) {
        const uint64_t m = M[g], n = N[g], k = K[g];
        FMAB_REQUIRE(m < (1u << 31) && n < (1u << 31) && k < (1u << 31), FMA_B200_ERR_BAD_ARG, "group %d too large", g);
        groups[g].m = (int32_t)m;
        groups[g].n = (int32_t)n;
        groups[g].k = (int32_t)k;
        groups[g].first_mtile = mt;
        groups[g].d_offset = d_off;
        FMAB_REQUIRE(n % 8 == 0, FMA_B200_ERR_BAD_ARG, "group %d: N=%llu must be a multiple of 8", g, (unsigned long long)n);
        if (m > 0 && n > 0 && k > 0) {
            int rc;
            if (a_t) rc = encode_2d(&maps[2 * g], a + a_off, m, k, m, 64, BK);       // [K, M], M contiguous
            else rc = encode_2d(&maps[2 * g], a + a_off, k, m, k, BK, BM);           // [M, K], K contiguous
            if (rc) return rc;
            if (b_t) rc = encode_2d(&maps[2 * g + 1], b + b_off, k, n, k, BK, BN);   // [N, K], K contiguous
            else rc = encode_2d(&maps[2 * g + 1], b + b_off, n, k, n, 64, BK);       // [K, N], N contiguous
            if (rc) return rc;
        }
        for (uint64_t r = 0; r < m; r += BM) {
            mtiles[mt].group = g;
            mtiles[mt].row0 = (int32_t)r;
            ++mt;
        }
        a_off += m * k;
        b_off += k * n;
        d_off += m * n;
    }
    FMAB_CUDA(cudaMemcpyAsync(workspace, host.data(), static_cast<size_t>(lay.total), cudaMemcpyHostToDevice, s));
    GemmParams p;
    if (int rc = fill_common(p)) return rc;
    uint8_t* ws = static_cast<uint8_t*>(workspace);
    p.mode = MODE_GENERAL;
    p.group_maps = reinterpret_cast<const CUtensorMap*>(ws + lay.maps_off);
    p.groups = reinterpret_cast<const GroupRec*>(ws + lay.groups_off);
    p.mtiles = reinterpret_cast<const MTileRec*>(ws + lay.mtiles_off);
    p.d = static_cast<__nv_bfloat16*>(D);
    p.n_mtiles = (int)total_mtiles;
    p.n_ntiles = (int)((max_n + BN - 1) / BN);
    p.n_groups = n_groups;
    if (!a_t && b_t) return launch_gemm<false, false, EPI_PLAIN>(p, s);
    if (!a_t && !b_t) return launch_gemm<false, true, EPI_PLAIN>(p, s);
    if (a_t && b_t) return launch_gemm<true, false, EPI_PLAIN>(p, s);
    return launch_gemm<true, true, EPI_PLAIN>(p, s);
}

int64_t tc_general_workspace_bytes(int n_groups, int64_t total_mtiles) {
    return general_layout(n_groups, total_mtiles).total;
}

}  // namespace fmab
