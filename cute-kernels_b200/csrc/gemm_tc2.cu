// bf16 grouped GEMM on CTA pairs: tcgen05.mma.cta_group::2, one 256x512 output tile per pair of SMs
//
// Why pairs: a 128x256x16 MMA issued by one CTA reads 12 KB of shared memory per 128 tensor-pipe
// cycles while TMA writes the next operands at the same rate, which together exceed what the
// shared-memory port delivers; the tensor pipe then idles about a third of the time.  With
// cta_group::2 the two CTAs of a cluster each hold their own 128 rows of A and HALF of the B tile
// (128 of the 256 columns); the pair's tensor cores use both halves, so every SM stages 32 KB per
// k-block instead of 48 KB and reads a third less per MMA.
//
// The kernels are bound by the bytes that cross from L2 to the SMs (measured ceiling ~9.2 TB/s), so a
// pair tile is 256 rows x 512 columns: per k-block each CTA loads its 128x64 slab of A ONCE and two
// 128-column slabs of B, and the leader issues two MMAs per k-step into the two 256-column halves of
// tensor memory.  That is 96 KB of loads per 16.8 MFLOP instead of 128 KB.  The halves have their own
// full/empty barriers, so the epilogue of half 0 overlaps the MMAs of half 1 and the next tile may
// start on half 0 while half 1 is still being stored.
//
// Structure (both CTAs run the same code; "leader" = cluster rank 0):
//   warp 0      TMA producer in each CTA: loads its A slab and its B slabs into a 4-stage ring.
//               All loads of a stage signal ONE mbarrier, the leader's (its address taken with
//               mapa); the leader arms it with the byte count of both CTAs.
//   warp 1      leader only: issues tcgen05.mma.cta_group::2 (M=256, N=256, K=16) and releases ring
//               stages / publishes accumulators with tcgen05.commit on both CTAs' barriers.
//   warps 2-9   epilogue in each CTA for its own 128 rows (tensor memory lanes), as in the
//               single-CTA kernel; they free an accumulator by arriving on the leader's barrier.
// Tiles are drawn from a global counter by the leader's producer thread, which publishes each tile id
// into a small ring in BOTH CTAs' shared memory (a remote store followed by a remote mbarrier arrive);
// every consumer of the id (the peer's producer, the MMA thread, all epilogue warps of both CTAs)
// arrives on the leader's "slot free" barrier.  Pairs that start late or draw long tiles therefore take
// fewer tiles (skewed expert loads, SMs shared with a collective).  Loads are the plain per-CTA cp.async.bulk.tensor form with the
// cta_group::2 qualifier; nothing in this file broadcasts a load to several CTAs.
// Token rows must be grouped with 256-row alignment so that both CTAs of a pair work for the same
// expert (forward / dgrad); wgrad pairs two 128-row slabs of one expert's weight gradient.
// Every mbarrier wait is bounded as in the single-CTA kernel; both CTAs always reach the final
// cluster barrier.
#include "gemm_tc.cuh"

namespace fmab {

constexpr int PAIR_B_ROWS = BN / 2;                                 // B rows staged per CTA and half (128)
constexpr int PAIR_B_BYTES = PAIR_B_ROWS * BK * 2;                  // 16 KB
constexpr int PAIR_THREADS = 320;
constexpr int PAIR_EPI_WARPS = 8;

// A pair tile is 256 rows x 512 columns: both 256-column halves of tensor memory belong to one tile, and every
// ring stage holds this CTA's A slab and its two B slabs.  (256x256 tiles whose halves belong to consecutive
// tiles were measured too: the whole epilogue then overlaps the next main loop, but A is staged twice as often,
// and they were slower at every benchmarked shape.)
constexpr int HALVES = 2;
constexpr int PAIR_STAGES = 4;
constexpr int PAIR_STAGE_BYTES = A_STAGE_BYTES + HALVES * PAIR_B_BYTES;  // 16 KB + 2 x 16 KB
constexpr size_t PAIR_RING_BYTES = static_cast<size_t>(PAIR_STAGES) * PAIR_STAGE_BYTES + 1024;
// Every epilogue passes its output through shared memory (a 4 KB patch per epilogue warp, behind the operand
// ring).  Tensor memory hands out an accumulator one row per lane; storing that straight from registers makes
// every store instruction touch 32 different 128-byte lines.  From the patch the output leaves
//   - as TMA stores issued by one lane (plain epilogue: 32 rows x 32 columns per store, the two halves of the
//     patch alternating), or
//   - in "line form": store instructions that each cover four whole 128-byte row segments (the peer-store
//     epilogue, whose destinations are arbitrary addresses, and the SwiGLU epilogues, which also do their
//     elementwise math in that form so that `pre` is read and written as whole lines too).
constexpr int PEER_PATCH_BYTES = 32 * 128;
constexpr size_t PEER_PATCH_TOTAL = static_cast<size_t>(PAIR_EPI_WARPS) * PEER_PATCH_BYTES;

// Address of the 16-byte piece (row, piece) of a per-warp staging patch: 32 rows x 128 bytes, pieces
// XOR-swizzled by the row.  Both ways the epilogues touch a patch are then free of bank conflicts:
//   row form   lane = row, one piece per access (how tensor memory hands out an accumulator: a row per lane);
//   line form  one access covers 4 rows x 8 pieces, i.e. four whole 128-byte rows (what global memory likes):
//              step `it` (0..7) gives lane the piece (row it*4 + lane/8, piece lane%8).
__device__ __forceinline__ uint32_t patch_addr(uint32_t patch, int row, int piece) {
    return patch + row * 128 + ((static_cast<uint32_t>(piece) ^ (static_cast<uint32_t>(row) & 7u)) << 4);
}

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// shared::cluster address of the same shared-memory offset in the CTA of rank `rank`
__device__ __forceinline__ uint32_t map_to_rank(uint32_t smem_addr, uint32_t rank) {
    uint32_t out;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(smem_addr), "r"(rank));
    return out;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// The same arrive without release semantics.  A releasing arrive at cluster scope has to wait until every
// global store the thread has issued is visible cluster-wide, i.e. until the epilogue's output has drained to
// L2 - a microsecond or two per tile during which the tensor memory it frees stays blocked.  What an epilogue
// warp hands back is tensor memory it has finished reading (tcgen05.wait::ld has returned and a
// tcgen05.fence::before_thread_sync precedes the arrive); its global stores need no ordering with the barrier.
__device__ __forceinline__ void mbar_arrive_cluster_relaxed(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void st_shared_cluster_u32(uint32_t cluster_addr, uint32_t v) {
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}
// Bounded wait with cluster-scope acquire, for barriers that a thread of the OTHER CTA arrives on after
// writing ordinary shared memory of this CTA.
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile int* abort_flag, int32_t* status) {
    const uint64_t t0 = global_timer();
    while (true) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.b32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(bar), "r"(parity)
            : "memory");
        if (ok) return true;
        if (*abort_flag) return false;
        if (global_timer() - t0 > 1000000000ull) {
            *abort_flag = 1;
            atomicExch(status, STATUS_GEMM_TIMEOUT);
            return false;
        }
    }
}
// TMA load into this CTA's shared memory whose completion bytes are counted on the LEADER's mbarrier.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t leader_bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(leader_bar), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void tc_mma_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrives (once the MMAs issued so far have completed) on the barrier at this offset in BOTH CTAs:
// one commit on the leader's own barrier, one on the peer's (its shared::cluster address).
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
    const uint32_t peer_bar = map_to_rank(bar, 1);
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(peer_bar) : "memory");
}
template <bool A_MN, bool B_MN>
__device__ __forceinline__ constexpr uint32_t make_instr_desc_pair() {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((A_MN ? 1u : 0u) << 15) | ((B_MN ? 1u : 0u) << 16) |
           (static_cast<uint32_t>(BN >> 3) << 17) | (static_cast<uint32_t>((2 * BM) >> 4) << 24);  // M = 256
}

// Work of one CTA for one pair tile.
struct PairTile {
    int32_t group;
    int32_t a_mn;      // this CTA's A coordinate along M
    int32_t b_mn;      // this CTA's B coordinate along N (its half of the tile's columns)
    int32_t b_k_base;
    int32_t n0;          // first D column of half 0
    int32_t n_step;      // D columns per half (256, or 128 act columns with the SwiGLU epilogue)
    int32_t halves;      // 1 or 2 halves carry columns
    int32_t rows_valid;
    int64_t d_row;
};

// tile -> (pair m-tile, n-tile) with SUPER_M/2 pair m-tiles walked together
template <bool B_MN, int EPI>
__device__ __forceinline__ bool decode_pair_tile(const GemmParams& p, int tile, int n_pair_mtiles, uint32_t rank, PairTile& t) {
    constexpr int kSuper = SUPER_M / 2;
    const int per_super = kSuper * p.n_ntiles;
    const int super = tile / per_super;
    const int m_first = super * kSuper;
    const int m_span = min(kSuper, n_pair_mtiles - m_first);
    const int r = tile - super * per_super;
    const int nt = r / m_span;
    const int pm = m_first + (r - nt * m_span);
    constexpr int n_step = (EPI == EPI_SWIGLU_FWD) ? BN / 2 : BN;
    t.n0 = nt * HALVES * n_step;
    t.n_step = n_step;
    t.halves = (t.n0 + n_step < p.n_cols) ? 2 : 1;
    t.b_k_base = 0;
    if (p.mode == MODE_ROWS) {
        const int e = __ldg(p.mtile_expert + 2 * pm);  // both 128-row tiles of the pair belong to this expert
        if (e < 0) return false;
        const int mt = 2 * pm + static_cast<int>(rank);
        t.group = e;
        t.a_mn = mt * BM;
        t.d_row = static_cast<int64_t>(mt) * BM;
        t.rows_valid = (mt < p.n_mtiles) ? BM : 0;
        if (EPI == EPI_SWIGLU_FWD) {
            // leader stages the 128 up rows, the peer the 128 gate rows of the same act columns
            t.b_mn = e * p.b_group_stride + t.n0 + static_cast<int>(rank) * p.inter;
        } else if (B_MN) {
            t.b_mn = t.n0 + static_cast<int>(rank) * PAIR_B_ROWS;
            t.b_k_base = e * p.b_group_stride;
        } else {
            t.b_mn = e * p.b_group_stride + t.n0 + static_cast<int>(rank) * PAIR_B_ROWS;
        }
    } else {  // MODE_WGRAD: pair m-tiles are counted per expert
        const int pairs_per_group = (p.mtiles_per_group + 1) / 2;
        const int slot = pm / pairs_per_group;
        // experts with the longest reductions first: a tile's time grows with its expert's row count, and a long
        // tile handed out last would run alone at the end of the launch
        const int e = (p.group_order != nullptr) ? __ldg(p.group_order + slot) : slot;
        const int m0 = ((pm - slot * pairs_per_group) * 2 + static_cast<int>(rank)) * BM;
        t.group = e;
        t.a_mn = m0;
        t.b_mn = t.n0 + static_cast<int>(rank) * PAIR_B_ROWS;
        t.d_row = static_cast<int64_t>(e) * p.m_per_group + m0;
        t.rows_valid = max(0, min(BM, p.m_per_group - m0));
    }
    return true;
}

__device__ __forceinline__ void decode_pair_segment(const GemmParams& p, const PairTile& t, int s, int& a_k0, int& b_k0, int& len) {
    if (p.mode == MODE_ROWS) {
        a_k0 = 0;
        b_k0 = t.b_k_base;
        len = p.k_len;
    } else {
        const int32_t* o = p.seg_offsets + s * p.n_groups + t.group;
        a_k0 = o[0];
        b_k0 = o[0];
        len = o[1] - o[0];
    }
}

template <bool A_MN, bool B_MN, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PAIR_THREADS, 1)
gemm_tc2_kernel(const __grid_constant__ GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[PAIR_STAGES];   // used in the leader only
    __shared__ __align__(8) uint64_t empty_bar[PAIR_STAGES];  // each CTA waits on its own copy
    __shared__ __align__(8) uint64_t acc_full_bar[2];         // each CTA waits on its own copy
    __shared__ __align__(8) uint64_t acc_empty_bar[2];        // used in the leader only
    __shared__ __align__(8) uint64_t sched_full_bar[SCHED_SLOTS];   // each CTA waits on its own copy
    __shared__ __align__(8) uint64_t sched_empty_bar[SCHED_SLOTS];  // used in the leader only
    __shared__ volatile int sched_tile[SCHED_SLOTS];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < PAIR_STAGES; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&acc_full_bar[b]), 1);
            mbar_init(smem_u32(&acc_empty_bar[b]), 2 * PAIR_EPI_WARPS);  // every epilogue warp of both CTAs
        }
        for (int i = 0; i < SCHED_SLOTS; ++i) {
            mbar_init(smem_u32(&sched_full_bar[i]), 1);
            // readers of a tile id: MMA thread + peer producer + the epilogue warps of both CTAs
            mbar_init(smem_u32(&sched_empty_bar[i]), 2 + 2 * PAIR_EPI_WARPS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {  // the same warp of both CTAs takes part in the paired allocation
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)),
                     "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // the peer's barriers exist before anything is signalled across CTAs
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;
    volatile int* abort_ptr = &abort_flag;

    const int n_pair_mtiles = (p.mode == MODE_ROWS) ? (p.n_mtiles + 1) / 2 : p.n_groups * ((p.mtiles_per_group + 1) / 2);
    const int total_tiles = n_pair_mtiles * p.n_ntiles;
    const int n_seg = (p.mode == MODE_WGRAD) ? p.n_seg : 1;
    const int pair_id = blockIdx.x >> 1;
    const int n_pairs = gridDim.x >> 1;

    if (warp == 0) {
        // ------------------------------ TMA producer (both CTAs) ------------------------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool alive = true;
            int sslot = 0;
            uint32_t sphase = 0;
            int tile = pair_id;
            while (alive) {
                int next = -1;
                if (leader) {
                    // publish the tile id (or the end marker) in both CTAs, then draw the next one
                    if (!mbar_wait_cluster(smem_u32(&sched_empty_bar[sslot]), sphase ^ 1u, abort_ptr, p.status)) {
                        alive = false;
                        break;
                    }
                    const int v = (tile < total_tiles) ? tile : -1;
                    sched_tile[sslot] = v;
                    st_shared_cluster_u32(map_to_rank(smem_u32(const_cast<int*>(&sched_tile[sslot])), 1), static_cast<uint32_t>(v));
                    mbar_arrive(smem_u32(&sched_full_bar[sslot]));
                    mbar_arrive_cluster(map_to_rank(smem_u32(&sched_full_bar[sslot]), 1));
                    if (v >= 0)
                        next = p.dynamic_tiles ? static_cast<int>(atomicAdd(p.sched, 1u)) + n_pairs : tile + n_pairs;
                } else {
                    if (!mbar_wait_cluster(smem_u32(&sched_full_bar[sslot]), sphase, abort_ptr, p.status)) {
                        alive = false;
                        break;
                    }
                    tile = sched_tile[sslot];
                    mbar_arrive_cluster(map_to_rank(smem_u32(&sched_empty_bar[sslot]), 0));
                    if (tile < 0) tile = total_tiles;  // end marker
                }
                if (++sslot == SCHED_SLOTS) {
                    sslot = 0;
                    sphase ^= 1u;
                }
                if (tile >= total_tiles) break;
                PairTile t;
                if (decode_pair_tile<B_MN, EPI>(p, tile, n_pair_mtiles, rank, t)) {
                for (int s = 0; s < n_seg && alive; ++s) {
                    int a_k0, b_k0, len;
                    decode_pair_segment(p, t, s, a_k0, b_k0, len);
                    for (int k = 0; k < len; k += BK) {
                        if (!mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1u, abort_ptr, p.status)) {
                            alive = false;
                            break;
                        }
                        const uint32_t leader_bar = map_to_rank(smem_u32(&full_bar[stage]), 0);
                        const uint32_t sa = ring + stage * PAIR_STAGE_BYTES;
                        const uint32_t sb = sa + A_STAGE_BYTES;
                        const uint32_t stage_bytes = A_STAGE_BYTES + t.halves * PAIR_B_BYTES;
                        if (leader) mbar_arrive_expect_tx(smem_u32(&full_bar[stage]), 2 * stage_bytes);
                        if (A_MN) {
#pragma unroll
                            for (int j = 0; j < BM / 64; ++j)
                                tma_load_2d_pair(sa + j * (BK * 128), &p.map_a, leader_bar, t.a_mn + 64 * j, a_k0 + k);
                        } else {
                            tma_load_2d_pair(sa, &p.map_a, leader_bar, a_k0 + k, t.a_mn);
                        }
                        for (int h = 0; h < t.halves; ++h) {
                            const uint32_t sbh = sb + h * PAIR_B_BYTES;
                            const int bn = t.b_mn + h * t.n_step;
                            if (B_MN) {
#pragma unroll
                                for (int j = 0; j < PAIR_B_ROWS / 64; ++j)
                                    tma_load_2d_pair(sbh + j * (BK * 128), &p.map_b, leader_bar, bn + 64 * j, b_k0 + k);
                            } else {
                                tma_load_2d_pair(sbh, &p.map_b, leader_bar, b_k0 + k, bn);
                            }
                        }
                        if (++stage == PAIR_STAGES) {
                            stage = 0;
                            phase ^= 1u;
                        }
                    }
                }
                }  // valid tile
                if (leader) tile = next;
            }
            if (!alive) {
                for (int i = 0; i < 200; ++i) __nanosleep(1000);  // let copies in flight land
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer (leader CTA only) ------------------------------
        if (leader && lane == 0) {
            const uint32_t idesc = with_operand_format(make_instr_desc_pair<A_MN, B_MN>(), p.f16 != 0);
            int stage = 0;
            uint32_t phase = 0;
            uint32_t acc_phase = 0;
            bool alive = true;
            int sslot = 0;
            uint32_t sphase = 0;
            while (alive) {
                if (!mbar_wait(smem_u32(&sched_full_bar[sslot]), sphase, abort_ptr, p.status)) break;
                const int tile = sched_tile[sslot];
                mbar_arrive(smem_u32(&sched_empty_bar[sslot]));
                if (++sslot == SCHED_SLOTS) {
                    sslot = 0;
                    sphase ^= 1u;
                }
                if (tile < 0) break;
                PairTile t;
                if (!decode_pair_tile<B_MN, EPI>(p, tile, n_pair_mtiles, rank, t)) continue;
                constexpr int h0 = 0;
                const uint32_t ph0 = acc_phase;
                // k-blocks of the tile (all segments); only their count matters to this warp
                int nkb = 0;
                for (int s = 0; s < n_seg; ++s) {
                    int a_k0, b_k0, len;
                    decode_pair_segment(p, t, s, a_k0, b_k0, len);
                    nkb += (len + BK - 1) / BK;
                }
                // Half 1 runs `skew` k-blocks behind half 0: at the end of a tile half 0 is published (and its
                // epilogue starts) while half 1 still has MMAs to run, and at the start of the next tile half
                // 0 can run while half 1 is still being stored.  A ring stage is released after BOTH halves
                // have read it, i.e. `skew` k-blocks later than without the skew.
                const int skew = (t.halves == 2) ? min(p.pair_skew, nkb) : 0;
                for (int step = 0; step < nkb + skew && alive; ++step) {
                    if (step < nkb) {  // half 0 on k-block `step`, which is the ring's current stage
                        if (!mbar_wait(smem_u32(&full_bar[stage]), phase, abort_ptr, p.status)) {
                            alive = false;
                            break;
                        }
                        tc_fence_after();
                        if (step == 0) {
                            if (!mbar_wait(smem_u32(&acc_empty_bar[h0]), ph0 ^ 1u, abort_ptr, p.status)) {
                                alive = false;
                                break;
                            }
                            tc_fence_after();
                        }
                        const uint32_t sa = ring + stage * PAIR_STAGE_BYTES;
                        const uint64_t a_desc = make_smem_desc<A_MN>(sa);
                        const uint64_t b_desc = make_smem_desc<B_MN>(sa + A_STAGE_BYTES);
#pragma unroll
                        for (int ks = 0; ks < BK / UMMA_K; ++ks)
                            tc_mma_pair(tmem_base + h0 * BN, a_desc + ((ks * desc_k_step<A_MN>()) >> 4),
                                        b_desc + ((ks * desc_k_step<B_MN>()) >> 4), idesc, (step | ks) ? 1u : 0u);
                        if (step == nkb - 1) tc_commit_pair(smem_u32(&acc_full_bar[h0]));
                    }
                    const int kb1 = step - skew;  // k-block of half 1 in this step
                    if (kb1 >= 0) {
                        // its stage is `skew` positions behind the ring's head (fewer once half 0 has finished)
                        const int behind = (step < nkb) ? skew : (nkb - kb1);  // the head already points past the last k-block
                        const int st1 = (stage + PAIR_STAGES - behind) % PAIR_STAGES;
                        if (t.halves == 2) {
                            if (kb1 == 0) {
                                if (!mbar_wait(smem_u32(&acc_empty_bar[1]), acc_phase ^ 1u, abort_ptr, p.status)) {
                                    alive = false;
                                    break;
                                }
                                tc_fence_after();
                            }
                            const uint32_t sa = ring + st1 * PAIR_STAGE_BYTES;
                            const uint64_t a_desc = make_smem_desc<A_MN>(sa);
                            const uint64_t b_desc = make_smem_desc<B_MN>(sa + A_STAGE_BYTES + PAIR_B_BYTES);
#pragma unroll
                            for (int ks = 0; ks < BK / UMMA_K; ++ks)
                                tc_mma_pair(tmem_base + BN, a_desc + ((ks * desc_k_step<A_MN>()) >> 4),
                                            b_desc + ((ks * desc_k_step<B_MN>()) >> 4), idesc, (kb1 | ks) ? 1u : 0u);
                        }
                        tc_commit_pair(smem_u32(&empty_bar[st1]));  // both halves are done with this stage
                    }
                    if (step < nkb) {
                        if (++stage == PAIR_STAGES) {
                            stage = 0;
                            phase ^= 1u;
                        }
                    }
                }
                if (!alive) break;
                if (nkb > 0) {
                    if (t.halves == 2) tc_commit_pair(smem_u32(&acc_full_bar[1]));
                } else {  // empty reduction: both epilogues write zeros
                    for (int h = 0; h < t.halves && alive; ++h) {
                        const int hb = h;
                        const uint32_t phb = acc_phase;
                        if (!mbar_wait(smem_u32(&acc_empty_bar[hb]), phb ^ 1u, abort_ptr, p.status)) {
                            alive = false;
                            break;
                        }
                        mbar_arrive(smem_u32(&acc_full_bar[hb]));
                        mbar_arrive_cluster(map_to_rank(smem_u32(&acc_full_bar[hb]), 1));
                    }
                    if (!alive) break;
                }
                if (t.halves == 1) {
                    // keep half 1's barriers in step with the tile count: pass its phase through unused
                    if (!mbar_wait(smem_u32(&acc_empty_bar[1]), acc_phase ^ 1u, abort_ptr, p.status)) break;
                    mbar_arrive(smem_u32(&acc_full_bar[1]));
                    mbar_arrive_cluster(map_to_rank(smem_u32(&acc_full_bar[1]), 1));
                }
                acc_phase ^= 1u;
            }
        }
    } else {
        // ------------------------------ epilogue (both CTAs, own 128 rows) ------------------------------
        const int quad = warp & 3;
        const int half = (warp - 2) >> 2;
        const bool f16 = p.f16 != 0;
        uint32_t acc_phase = 0;
        uint32_t store_seq = 0;  // TMA stores issued by this warp: picks the half of its patch
        int sslot = 0;
        uint32_t sphase = 0;
        while (true) {
            if (!mbar_wait_cluster(smem_u32(&sched_full_bar[sslot]), sphase, abort_ptr, p.status)) break;
            const int tile = sched_tile[sslot];
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_rank(smem_u32(&sched_empty_bar[sslot]), 0));
            if (++sslot == SCHED_SLOTS) {
                sslot = 0;
                sphase ^= 1u;
            }
            if (tile < 0) break;
            PairTile t;
            if (!decode_pair_tile<B_MN, EPI>(p, tile, n_pair_mtiles, rank, t)) continue;
            bool any_k = false;
            for (int s = 0; s < n_seg; ++s) {
                int a_k0, b_k0, len;
                decode_pair_segment(p, t, s, a_k0, b_k0, len);
                any_k |= len > 0;
            }
            const uint32_t patch = ring + PAIR_STAGES * PAIR_STAGE_BYTES + (warp - 2) * PEER_PATCH_BYTES;
            const int lr = lane >> 3, lp = lane & 7;  // line form: row within a 4-row step, 16-byte piece of the row
            constexpr int kGroups = BN / 64 / 2;       // 64-column groups per warp and accumulator half
            bool alive = true;

            // The SwiGLU epilogues run in two phases.  Phase 1 is the plain epilogue: the rounded accumulator leaves
            // through TMA stores (up / gate into `pre`; d_act into the d_up half of the output) and tensor memory is
            // handed back at once.  Phase 2 reads those values back in line form (they are in L2), does the
            // elementwise math and writes act, or d_up over d_act and d_gate, while the next tile's main loop is
            // already running.  Each warp reads back exactly the region it stored itself.
            const bool two_phase = (EPI == EPI_SWIGLU_BWD) || (EPI == EPI_SWIGLU_FWD && p.d2 != nullptr);
            const int64_t pre_pitch = 2 * static_cast<int64_t>(p.inter);

            for (int h = 0; h < HALVES; ++h) {
            const int hs = h;  // tensor-memory half
            const uint32_t phs = acc_phase;
            if (!mbar_wait(smem_u32(&acc_full_bar[hs]), phs, abort_ptr, p.status)) {
                alive = false;
                break;
            }
            tc_fence_after();
            const uint32_t taddr = tmem_base + hs * BN + (static_cast<uint32_t>(quad * 32) << 16);
            const int n0h = t.n0 + h * t.n_step;                 // first D column of this half
            const int n_valid = min(t.n_step, p.n_cols - n0h);   // <= 0: the half carries no columns
            bool released = false;  // tensor memory of this half already handed back

            if (EPI == EPI_PLAIN || two_phase) {
                // 32 rows x 32 columns at a time: accumulator -> bf16 -> one half of the warp's patch (64-byte
                // rows, 64-byte swizzle) -> ONE TMA store issued by lane 0.  The two halves of the patch
                // alternate, so a store drains while the next piece is converted and written.
                // A warp owns two 64-column pieces of the half: columns [half*128, +128) of the accumulator, or,
                // with the SwiGLU forward epilogue, the up and the gate columns of act columns [half*64, +64).
                const int row_c = ((p.mode == MODE_ROWS) ? static_cast<int>(t.d_row) : t.a_mn) + quad * 32;
                const int grp_c = (p.mode == MODE_ROWS) ? 0 : t.group;
                const bool rows_here = quad * 32 < t.rows_valid;
                // All of the warp's 128 accumulator columns are fetched and rounded first (64 packed registers per
                // lane) and tensor memory is handed back right then: the stores below no longer hold up the next
                // tile's first MMA.
                uint4 pk[16];
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const int acc_col = (EPI == EPI_SWIGLU_FWD) ? j * (BN / 2) + half * 64 : half * (BN / 2) + j * 64;
                    uint32_t ra[32], rb[32];
                    if (any_k) {  // both pieces of the pair are requested before either is awaited
                        tc_load_32_issue(taddr + acc_col, ra);
                        tc_load_32_issue(taddr + acc_col + 32, rb);
                        tc_load_wait();
                    }
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        float va[8], vb[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            va[i] = any_k ? __uint_as_float(ra[k * 8 + i]) : 0.f;
                            vb[i] = any_k ? __uint_as_float(rb[k * 8 + i]) : 0.f;
                        }
                        pk[j * 8 + k] = pack8(va, f16);
                        pk[j * 8 + 4 + k] = pack8(vb, f16);
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster_relaxed(map_to_rank(smem_u32(&acc_empty_bar[hs]), 0));  // the leader's barrier
                released = true;
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const int out_off = (EPI == EPI_SWIGLU_FWD) ? half * 64 : half * (BN / 2) + j * 64;  // within the half
                    const int cols_left = n_valid - out_off;
#pragma unroll
                    for (int q = 0; q < 2; ++q) {
                        if (cols_left <= q * 32) break;
                        const uint32_t sub = patch + (store_seq & 1u) * (PEER_PATCH_BYTES / 2);
                        ++store_seq;
                        if (lane == 0) bulk_wait_read_but_one();  // the store that last used this half has read it
                        __syncwarp();
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            st_shared_16(sub + lane * 64 + ((static_cast<uint32_t>(k) ^ ((lane >> 1) & 3u)) << 4),
                                         pk[j * 8 + q * 4 + k]);
                        fence_smem_to_async();
                        __syncwarp();
                        if (lane == 0 && rows_here) {
                            if (EPI == EPI_SWIGLU_FWD)
                                tma_store_3d(&p.map_d, sub, n0h + out_off + q * 32, j, row_c);  // {column, up | gate, row}
                            else
                                tma_store_3d(&p.map_d, sub, n0h + out_off + q * 32, row_c, grp_c);
                            bulk_commit();
                        }
                    }
                }
            } else if (EPI == EPI_PLAIN_PEER) {
                // 32 rows x 64 columns at a time: accumulator -> bf16 -> patch in row form -> read back in line
                // form -> eight store instructions of four whole 128-byte row segments each.  The 128 rows of
                // this CTA's tile go to the address from the per-tile table (possibly another GPU's memory), same
                // pitch; what crosses NVLink are whole 128-byte lines.
                uint8_t* dst_tile = reinterpret_cast<uint8_t*>(__ldg(p.mtile_dst + (t.d_row >> 7)));
#pragma unroll 1
                for (int g = half * kGroups; g < (half + 1) * kGroups; ++g) {
                    const int cols_left = n_valid - g * 64;
                    if (cols_left <= 0) break;
#pragma unroll
                    for (int q = 0; q < 2; ++q) {
                        float v[32];
                        if (any_k && cols_left > q * 32) {
                            tc_load_32(taddr + g * 64 + q * 32, v);
                        } else {
#pragma unroll
                            for (int i = 0; i < 32; ++i) v[i] = 0.f;
                        }
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            st_shared_16(patch_addr(patch, lane, q * 4 + k), pack8(v + k * 8, f16));
                    }
                    __syncwarp();
#pragma unroll
                    for (int it = 0; it < 8; ++it) {
                        const int r = it * 4 + lr;
                        const uint4 w = ld_shared_16(patch_addr(patch, r, lp));
                        const int row = quad * 32 + r;
                        if (row < t.rows_valid && lp * 8 < cols_left)
                            st_global_16(dst_tile + (static_cast<int64_t>(row) * p.ldd + n0h + g * 64 + lp * 8) * 2, w);
                    }
                    __syncwarp();
                }
            } else if (EPI == EPI_SWIGLU_FWD) {
                // (caller keeps no `pre`: one phase, nothing to read back)
                // This warp: 32 rows x 64 act columns of the half (up in accumulator columns [0,128), gate in
                // [128,256)).  up and gate are rounded to bf16 and go through the patch one after the other;
                // act = up * gate * sigmoid(gate) is computed from the rounded values in line form, and all three
                // leave as whole 128-byte row segments (up and gate into `pre`, act into its own matrix).
                const int col0 = half * 64;
                const int cols_left = n_valid - col0;
                if (cols_left > 0) {
                    uint4 pg[8];
#pragma unroll
                    for (int q = 0; q < 2; ++q) {
                        float u[32], g[32];
                        if (cols_left > q * 32) {
                            tc_load_32(taddr + col0 + q * 32, u);
                            tc_load_32(taddr + BN / 2 + col0 + q * 32, g);
                        } else {
#pragma unroll
                            for (int i = 0; i < 32; ++i) u[i] = g[i] = 0.f;
                        }
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            st_shared_16(patch_addr(patch, lane, q * 4 + k), pack8(u + k * 8, f16));
                            pg[q * 4 + k] = pack8(g + k * 8, f16);
                        }
                    }
                    __syncwarp();
                    uint4 lu[8];
#pragma unroll
                    for (int it = 0; it < 8; ++it) lu[it] = ld_shared_16(patch_addr(patch, it * 4 + lr, lp));
                    __syncwarp();
#pragma unroll
                    for (int j = 0; j < 8; ++j) st_shared_16(patch_addr(patch, lane, j), pg[j]);
                    __syncwarp();
#pragma unroll
                    for (int it = 0; it < 8; ++it) {
                        const int r = it * 4 + lr;
                        const uint4 lg = ld_shared_16(patch_addr(patch, r, lp));
                        const int row = quad * 32 + r;
                        float u[8], g[8];
                        unpack8(lu[it], u, f16);
                        unpack8(lg, g, f16);
                        swiglu_fwd8(u, g, u);
                        if (row < t.rows_valid && lp * 8 < cols_left) {
                            const int64_t grow = t.d_row + row;
                            const int col = n0h + col0 + lp * 8;
                            if (p.d2 != nullptr) {
                                st_global_16(p.d2 + grow * pre_pitch + col, lu[it]);
                                st_global_16(p.d2 + grow * pre_pitch + p.inter + col, lg);
                            }
                            st_global_16(p.d + grow * p.ldd + col, pack8(u, f16));
                        }
                    }
                    __syncwarp();
                }
            }
            if (!released) {
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster_relaxed(map_to_rank(smem_u32(&acc_empty_bar[hs]), 0));  // the leader's barrier
            }
            }  // halves
            if (!alive) break;
            acc_phase ^= 1u;
            if (two_phase) {
                if (lane == 0) {
                    bulk_wait_all();            // this warp's stores of the tile have been written ...
                    fence_async_to_generic();   // ... and are ordered before the ordinary loads below
                }
                __syncwarp();
                // The region is walked in batches of four accesses per lane.  As soon as an access has been unpacked
                // its registers are refilled with the same access of the next batch, so loads stay in flight while
                // the math and the stores of the current batch run.
                if (EPI == EPI_SWIGLU_FWD) {
                    // per half 32 rows x 64 act columns: an access covers four rows x 128 bytes; 2 x 2 batches
                    constexpr int kBatches = 2 * HALVES;
                    const int lr = lane >> 3, lp = lane & 7;
                    const int cw = half * 64 + lp * 8;
                    // row of the access and its column (the same in `pre`, pitch 2 I, and in `act`, pitch I)
                    auto at_of = [&](int b, int i, bool& ok, int& col) -> int64_t {
                        const int n0h = t.n0 + (b >> 1) * t.n_step;
                        const int row = quad * 32 + ((b & 1) * 4 + i) * 4 + lr;
                        ok = b < kBatches && cw < min(t.n_step, p.n_cols - n0h) && row < t.rows_valid;
                        col = n0h + cw;
                        return t.d_row + row;
                    };
                    uint4 vu[4], vg[4];
                    auto fetch = [&](int b, int i) {
                        bool ok;
                        int col;
                        const int64_t grow = at_of(b, i, ok, col);
                        vu[i] = ok ? ld_global_cg_16(p.d2 + grow * pre_pitch + col) : make_uint4(0, 0, 0, 0);
                        vg[i] = ok ? ld_global_cg_16(p.d2 + grow * pre_pitch + p.inter + col) : make_uint4(0, 0, 0, 0);
                    };
#pragma unroll
                    for (int i = 0; i < 4; ++i) fetch(0, i);
#pragma unroll 1
                    for (int b = 0; b < kBatches; ++b) {
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            bool ok;
                            int col;
                            const int64_t grow = at_of(b, i, ok, col);
                            float u[8], g[8];
                            unpack8(vu[i], u, f16);
                            unpack8(vg[i], g, f16);
                            fetch(b + 1, i);
                            swiglu_fwd8(u, g, u);
                            if (ok) st_global_16(p.d + grow * p.ldd + col, pack8(u, f16));
                        }
                    }
                } else {
                    // per half 32 rows x 128 columns: an access covers two rows x 256 bytes; 2 x 4 batches
                    constexpr int kBatches = 4 * HALVES;
                    const int lr = lane >> 4, lp = lane & 15;
                    const int cw = half * (BN / 2) + lp * 8;
                    auto at_of = [&](int b, int i, bool& ok) -> int64_t {
                        const int n0h = t.n0 + (b >> 2) * t.n_step;
                        const int row = quad * 32 + ((b & 3) * 4 + i) * 2 + lr;
                        ok = b < kBatches && cw < min(t.n_step, p.n_cols - n0h) && row < t.rows_valid;
                        return (t.d_row + row) * pre_pitch + n0h + cw;
                    };
                    uint4 vd[4], vu[4], vg[4];
                    auto fetch = [&](int b, int i) {
                        bool ok;
                        const int64_t at = at_of(b, i, ok);
                        vd[i] = ok ? ld_global_cg_16(p.d + at) : make_uint4(0, 0, 0, 0);
                        vu[i] = ok ? ld_global_16(p.pre + at) : make_uint4(0, 0, 0, 0);
                        vg[i] = ok ? ld_global_16(p.pre + at + p.inter) : make_uint4(0, 0, 0, 0);
                    };
#pragma unroll
                    for (int i = 0; i < 4; ++i) fetch(0, i);
#pragma unroll 1
                    for (int b = 0; b < kBatches; ++b) {
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            bool ok;
                            const int64_t at = at_of(b, i, ok);
                            float d[8], u[8], gt[8], du[8], dg[8];
                            unpack8(vd[i], d, f16);
                            unpack8(vu[i], u, f16);
                            unpack8(vg[i], gt, f16);
                            fetch(b + 1, i);
                            swiglu_bwd8(d, u, gt, du, dg);
                            if (ok) {
                                st_global_16(p.d + at, pack8(du, f16));
                                st_global_16(p.d + at + p.inter, pack8(dg, f16));
                            }
                        }
                    }
                }
            }
        }
        if (lane == 0) bulk_wait_all();  // TMA stores of this warp (if any) are complete before the CTA retires
    }

    __syncwarp();
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // neither CTA touches the pair's tensor memory or barriers after this point
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
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

// Experts sorted by their row count over all segments, largest first (ties: lower id first).  One block, one
// thread per expert.
constexpr int ORDER_MAX_GROUPS = 1024;
__global__ void __launch_bounds__(ORDER_MAX_GROUPS) group_order_kernel(const int32_t* __restrict__ seg_offsets,
                                                                       int n_seg, int n_groups, int32_t* __restrict__ order) {
    __shared__ int32_t rows[ORDER_MAX_GROUPS];
    const int e = threadIdx.x;
    int32_t mine = 0;
    if (e < n_groups) {
        for (int s = 0; s < n_seg; ++s) mine += seg_offsets[s * n_groups + e + 1] - seg_offsets[s * n_groups + e];
        rows[e] = mine;
    }
    __syncthreads();
    if (e < n_groups) {
        int rank = 0;
        for (int j = 0; j < n_groups; ++j) {
            const int32_t other = rows[j];
            rank += (other > mine || (other == mine && j < e)) ? 1 : 0;
        }
        order[rank] = e;
    }
}
// Scratch for the order: 64 slots per device handed out round-robin, like the scheduler words.
static __device__ int32_t g_group_order[64 * ORDER_MAX_GROUPS];

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
static int next_order_slot(int32_t** out) {
    static int32_t* base[64] = {nullptr};
    static unsigned int seq = 0;
    const int dev = current_device_slot();
    FMAB_REQUIRE(dev >= 0, FMA_B200_ERR_LAUNCH, "no current CUDA device with an ordinal below 64");
    if (base[dev] == nullptr) {
        void* ptr = nullptr;
        FMAB_CUDA(cudaGetSymbolAddress(&ptr, g_group_order));
        base[dev] = static_cast<int32_t*>(ptr);
    }
    *out = base[dev] + ORDER_MAX_GROUPS * (__atomic_fetch_add(&seq, 1u, __ATOMIC_RELAXED) % 64u);
    return FMA_B200_OK;
}

// k-blocks by which accumulator half 1 trails half 0 (0..2); FMA_B200_GEMM_SKEW overrides the default.
static int pair_skew() {
    static int v = -1;
    if (v < 0) {
        const char* env = getenv("FMA_B200_GEMM_SKEW");
        v = env ? atoi(env) : 1;  // 1 measured best with a 4-stage ring (2 starves the ring)
        if (v < 0 || v > 2) v = 1;
    }
    return v;
}

// Output map of a rows-mode GEMM with the plain epilogue: [rows_cap, n_cols] with row pitch `pitch` elements.
static int encode_rows_output(GemmParams& p, const void* D, int64_t rows_cap, int n_cols, int64_t pitch) {
    return encode_3d(&p.map_d, D, n_cols, rows_cap, 1, pitch, pitch, 32, 32, p.f16 != 0);
}

template <bool A_MN, bool B_MN, int EPI>
static int launch_pair(const GemmParams& p, int64_t total_tiles, cudaStream_t s) {
    static bool configured[64] = {false};  // per device: the attribute applies to the current device only
    auto kernel = gemm_tc2_kernel<A_MN, B_MN, EPI>;
    constexpr size_t PAIR_SMEM_BYTES = PAIR_RING_BYTES + PEER_PATCH_TOTAL;
    const int dev = current_device_slot();
    FMAB_REQUIRE(dev >= 0, FMA_B200_ERR_LAUNCH, "no current CUDA device with an ordinal below 64");
    if (!configured[dev]) {
        FMAB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PAIR_SMEM_BYTES));
        configured[dev] = true;
    }
    if (total_tiles <= 0) return FMA_B200_OK;
    FMAB_REQUIRE(total_tiles < (1LL << 31), FMA_B200_ERR_BAD_ARG, "too many tiles");
    const int64_t max_pairs = sm_count() / 2;
    const int pairs = static_cast<int>(total_tiles < max_pairs ? total_tiles : max_pairs);
    GemmParams q = p;
    if (int rc = next_sched_pair(&q.sched)) return rc;
    q.dynamic_tiles = dynamic_tiles_enabled();
    q.pair_skew = pair_skew();
    kernel<<<2 * pairs, PAIR_THREADS, PAIR_SMEM_BYTES, s>>>(q);
    return check_launch("grouped GEMM (tcgen05, CTA pairs)");
}

static int fill_pair_common(GemmParams& p) {
    memset(&p, 0, sizeof(p));
    p.status = device_status_ptr();
    FMAB_REQUIRE(p.status != nullptr, FMA_B200_ERR_LAUNCH, "no device status word");
    p.n_seg = 1;
    return FMA_B200_OK;
}

int tc2_forward(const void* X, const void* W, void* Y, int64_t rows_cap, int E, int OUT, int IN,
                const int32_t* mtile_expert, bool f16, cudaStream_t s) {
    GemmParams p;
    if (int rc = fill_pair_common(p)) return rc;
    p.f16 = f16 ? 1 : 0;
    if (int rc = encode_2d(&p.map_a, X, IN, rows_cap, IN, BK, BM, f16)) return rc;
    if (int rc = encode_2d(&p.map_b, W, IN, static_cast<uint64_t>(E) * OUT, IN, BK, PAIR_B_ROWS, f16)) return rc;
    p.mode = MODE_ROWS;
    p.mtile_expert = mtile_expert;
    p.d = static_cast<__nv_bfloat16*>(Y);
    p.ldd = OUT;
    p.n_mtiles = static_cast<int>(rows_cap / BM);
    const int tile_cols = 2 * BN;
    p.n_ntiles = (OUT + tile_cols - 1) / tile_cols;
    p.n_cols = OUT;
    p.k_len = IN;
    p.b_group_stride = OUT;
    p.n_groups = E;
    if (int rc = encode_rows_output(p, Y, rows_cap, OUT, OUT)) return rc;
    const int64_t total = static_cast<int64_t>((p.n_mtiles + 1) / 2) * p.n_ntiles;
    return launch_pair<false, false, EPI_PLAIN>(p, total, s);
}

int tc2_forward_swiglu(const void* X, const void* W, void* pre, void* act, int64_t rows_cap, int E, int I, int IN,
                       const int32_t* mtile_expert, bool f16, cudaStream_t s) {
    GemmParams p;
    if (int rc = fill_pair_common(p)) return rc;
    p.f16 = f16 ? 1 : 0;
    if (int rc = encode_2d(&p.map_a, X, IN, rows_cap, IN, BK, BM, f16)) return rc;
    if (int rc = encode_2d(&p.map_b, W, IN, static_cast<uint64_t>(E) * 2 * I, IN, BK, PAIR_B_ROWS, f16)) return rc;
    p.mode = MODE_ROWS;
    p.mtile_expert = mtile_expert;
    p.d = static_cast<__nv_bfloat16*>(act);
    p.d2 = static_cast<__nv_bfloat16*>(pre);
    p.ldd = I;
    p.inter = I;
    p.n_mtiles = static_cast<int>(rows_cap / BM);
    const int tile_cols = BN;  // 128 act columns per accumulator half
    p.n_ntiles = (I + tile_cols - 1) / tile_cols;
    p.n_cols = I;
    p.k_len = IN;
    p.b_group_stride = 2 * I;
    p.n_groups = E;
    if (pre != nullptr) {
        // `pre` as {I columns, up | gate, rows}: a store that overhangs the up columns is clipped, not written
        // into the gate columns
        if (int rc = encode_3d_box(&p.map_d, pre, I, 2, rows_cap, I, 2 * static_cast<uint64_t>(I), 32, 1, 32, f16)) return rc;
    }
    const int64_t total = static_cast<int64_t>((p.n_mtiles + 1) / 2) * p.n_ntiles;
    return launch_pair<false, false, EPI_SWIGLU_FWD>(p, total, s);
}

int tc2_dgrad(const void* dY, const void* W, void* dX, const void* pre, int64_t rows_cap, int E, int OUT, int IN,
              const int32_t* mtile_expert, bool swiglu, bool f16, cudaStream_t s) {
    GemmParams p;
    if (int rc = fill_pair_common(p)) return rc;
    p.f16 = f16 ? 1 : 0;
    if (int rc = encode_2d(&p.map_a, dY, OUT, rows_cap, OUT, BK, BM, f16)) return rc;
    if (int rc = encode_2d(&p.map_b, W, IN, static_cast<uint64_t>(E) * OUT, IN, 64, BK, f16)) return rc;
    p.mode = MODE_ROWS;
    p.mtile_expert = mtile_expert;
    p.d = static_cast<__nv_bfloat16*>(dX);
    p.pre = static_cast<const __nv_bfloat16*>(pre);
    p.ldd = swiglu ? 2 * static_cast<int64_t>(IN) : IN;
    p.inter = IN;
    p.n_mtiles = static_cast<int>(rows_cap / BM);
    const int tile_cols = 2 * BN;
    p.n_ntiles = (IN + tile_cols - 1) / tile_cols;
    p.n_cols = IN;
    p.k_len = OUT;
    p.b_group_stride = OUT;
    p.n_groups = E;
    // with SwiGLU backward the d_act tile is parked in the d_up columns of the [rows, 2 IN] output first
    if (int rc = encode_rows_output(p, dX, rows_cap, IN, swiglu ? 2 * static_cast<int64_t>(IN) : IN)) return rc;
    const int64_t total = static_cast<int64_t>((p.n_mtiles + 1) / 2) * p.n_ntiles;
    if (swiglu) return launch_pair<false, true, EPI_SWIGLU_BWD>(p, total, s);
    return launch_pair<false, true, EPI_PLAIN>(p, total, s);
}

// Forward / dgrad whose output tiles go to the addresses in dst_table (one per 128-row tile, row pitch = the
// output width): the epilogue of the expert-parallel layer that returns rows straight into the arenas of the
// ranks they came from.
int tc2_forward_peer(const void* X, const void* W, const uint64_t* dst_table, int64_t rows_cap, int E, int OUT, int IN,
                     const int32_t* mtile_expert, bool f16, cudaStream_t s) {
    GemmParams p;
    if (int rc = fill_pair_common(p)) return rc;
    p.f16 = f16 ? 1 : 0;
    if (int rc = encode_2d(&p.map_a, X, IN, rows_cap, IN, BK, BM, f16)) return rc;
    if (int rc = encode_2d(&p.map_b, W, IN, static_cast<uint64_t>(E) * OUT, IN, BK, PAIR_B_ROWS, f16)) return rc;
    p.mode = MODE_ROWS;
    p.mtile_expert = mtile_expert;
    p.mtile_dst = dst_table;
    p.ldd = OUT;
    p.n_mtiles = static_cast<int>(rows_cap / BM);
    p.n_ntiles = (OUT + 2 * BN - 1) / (2 * BN);
    p.n_cols = OUT;
    p.k_len = IN;
    p.b_group_stride = OUT;
    p.n_groups = E;
    return launch_pair<false, false, EPI_PLAIN_PEER>(p, static_cast<int64_t>((p.n_mtiles + 1) / 2) * p.n_ntiles, s);
}

int tc2_dgrad_peer(const void* dY, const void* W, const uint64_t* dst_table, int64_t rows_cap, int E, int OUT, int IN,
                   const int32_t* mtile_expert, bool f16, cudaStream_t s) {
    GemmParams p;
    if (int rc = fill_pair_common(p)) return rc;
    p.f16 = f16 ? 1 : 0;
    if (int rc = encode_2d(&p.map_a, dY, OUT, rows_cap, OUT, BK, BM, f16)) return rc;
    if (int rc = encode_2d(&p.map_b, W, IN, static_cast<uint64_t>(E) * OUT, IN, 64, BK, f16)) return rc;
    p.mode = MODE_ROWS;
    p.mtile_expert = mtile_expert;
    p.mtile_dst = dst_table;
    p.ldd = IN;
    p.inter = IN;
    p.n_mtiles = static_cast<int>(rows_cap / BM);
    p.n_ntiles = (IN + 2 * BN - 1) / (2 * BN);
    p.n_cols = IN;
    p.k_len = OUT;
    p.b_group_stride = OUT;
    p.n_groups = E;
    return launch_pair<false, true, EPI_PLAIN_PEER>(p, static_cast<int64_t>((p.n_mtiles + 1) / 2) * p.n_ntiles, s);
}

int tc2_wgrad(const void* dY, const void* X, void* dW, int64_t rows_cap, int E, int OUT, int IN,
              const int32_t* seg_offsets, int n_seg, bool f16, cudaStream_t s) {
    GemmParams p;
    if (int rc = fill_pair_common(p)) return rc;
    p.f16 = f16 ? 1 : 0;
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
    p.n_ntiles = (IN + 2 * BN - 1) / (2 * BN);
    p.n_cols = IN;
    p.n_groups = E;
    // dW as {IN, OUT, E}: rows of a tile beyond OUT are clipped, not written into the next expert
    if (int rc = encode_3d(&p.map_d, dW, IN, OUT, E, IN, static_cast<uint64_t>(OUT) * IN, 32, 32, f16)) return rc;
    const int64_t total = static_cast<int64_t>(E) * ((p.mtiles_per_group + 1) / 2) * p.n_ntiles;
    if (E > 1 && E <= ORDER_MAX_GROUPS && total > 0) {
        int32_t* order = nullptr;
        if (int rc = next_order_slot(&order)) return rc;
        group_order_kernel<<<1, ORDER_MAX_GROUPS, 0, s>>>(seg_offsets, n_seg, E, order);
        if (int rc = check_launch("grouped GEMM (expert order)")) return rc;
        p.group_order = order;
    }
    return launch_pair<true, true, EPI_PLAIN>(p, total, s);
}

}  // namespace fmab
