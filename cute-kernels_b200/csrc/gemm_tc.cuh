// Pieces shared by the two tensor-core grouped-GEMM kernels (one CTA per tile in gemm_tc.cu, CTA pairs
// with cta_group::2 in gemm_tc2.cu): tile constants, kernel parameters, PTX wrappers for mbarrier /
// TMA / tcgen05, shared-memory and instruction descriptors, epilogue row helpers, tensor-map encoding.
#pragma once

#include <cuda.h>
#include <stdlib.h>
#include <string.h>

#include "common.cuh"

namespace fmab {

// ---------------------------------------------------------------------------
// tile shape
// ---------------------------------------------------------------------------
constexpr int BM = 128;           // rows of D per tile = TMEM lanes
constexpr int BN = 256;           // columns of D per tile = TMEM columns per accumulator
constexpr int BK = 64;            // reduction elements per stage = one 128-byte swizzle row of bf16
constexpr int UMMA_K = 16;        // reduction elements per tcgen05.mma (bf16)
constexpr int STAGES = 4;
constexpr int A_STAGE_BYTES = BM * BK * 2;
constexpr int B_STAGE_BYTES = BN * BK * 2;
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int MAX_GEMM_THREADS = 320;  // 2 + 8 warps; the 4-epilogue-warp build uses 192
constexpr int TMEM_COLS = 512;
constexpr int SCHED_SLOTS = 4;    // tile ids published ahead by the producer warp
constexpr int SUPER_M = 16;       // m-tiles walked together so that concurrent CTAs share operand tiles in L2
constexpr size_t GEMM_SMEM_BYTES = static_cast<size_t>(STAGES) * STAGE_BYTES + 1024;

constexpr int EPI_PLAIN = 0;
constexpr int EPI_SWIGLU_FWD = 1;
constexpr int EPI_SWIGLU_BWD = 2;
constexpr int EPI_PLAIN_PEER = 3;  // CTA-pair kernel: plain epilogue whose 128-row tiles go to per-tile addresses

constexpr int MODE_ROWS = 0;     // ragged M: m-tile -> expert through mtile_expert (forward, dgrad)
constexpr int MODE_WGRAD = 1;    // ragged K: tile = (expert, m-tile, n-tile), k runs over the expert's rows
constexpr int MODE_GENERAL = 2;  // per-group tensor maps and host-built tables

constexpr int32_t STATUS_GEMM_TIMEOUT = 0x7001;

// Tables of the general mode (host-built, in the caller's workspace).
struct GroupRec {
    int32_t m, n, k;      // problem size of the group
    int32_t first_mtile;  // index of its first m-tile
    int64_t d_offset;     // element offset of D_g in the packed output
};
struct MTileRec {
    int32_t group;
    int32_t row0;  // first row of the tile inside the group
};

struct GemmParams {
    CUtensorMap map_a;
    CUtensorMap map_b;
    const CUtensorMap* group_maps;  // general mode: [2g] = A_g, [2g+1] = B_g
    const GroupRec* groups;
    const MTileRec* mtiles;
    const int32_t* mtile_expert;  // rows mode
    const int32_t* seg_offsets;   // wgrad mode: [n_seg][E] (+1)
    const int32_t* group_order;   // wgrad mode, CTA-pair kernel: experts in the order their tiles are handed out, or null
    __nv_bfloat16* d;             // output (act for SWIGLU_FWD, d_pre for SWIGLU_BWD)
    __nv_bfloat16* d2;            // SWIGLU_FWD: pre (may be null)
    const __nv_bfloat16* pre;     // SWIGLU_BWD: saved pre-activations
    int32_t* status;
    unsigned int* sched;          // [0] next-tile counter, [1] CTAs finished; both zero between launches
    int64_t ldd;                  // row pitch of d in elements
    int32_t mode;
    int32_t n_mtiles;             // m-tiles to walk
    int32_t n_ntiles;
    int32_t m_per_group;          // wgrad: rows of D per expert (OUT)
    int32_t mtiles_per_group;     // wgrad: ceil(OUT / 128)
    int32_t n_cols;               // columns of D (rows/wgrad modes)
    int32_t k_len;                // rows mode: reduction length
    int32_t b_group_stride;       // rows mode: B coordinate step per expert (rows of the stacked weight)
    int32_t n_groups;             // E
    int32_t n_seg;                // wgrad: segments per expert
    int32_t inter;                // SwiGLU: intermediate size I
    int32_t dynamic_tiles;        // 1: tiles drawn from the global counter; 0: tile = blockIdx.x + i * gridDim.x
    int32_t pair_skew;            // CTA-pair kernel: k-blocks by which accumulator half 1 trails half 0
    const uint64_t* mtile_dst;    // EPI_PLAIN_PEER: byte address of output row 0 of every 128-row tile (pitch ldd)
    // CTA-pair kernel, plain epilogue: output as a 3-D map {columns, rows, group} with boxes of 32 columns x
    // 32 rows for TMA stores; group coordinate 0 in rows mode.
    CUtensorMap map_d;
    int32_t f16;  // 1: operands and outputs are IEEE half instead of bfloat16 (same kernels, same 16-bit layouts)
};

// ---------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ uint64_t global_timer() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false if the wait was given up (here or by another thread of the CTA).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int32_t* status) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = global_timer();
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (global_timer() - t0 > 1000000000ull) {  // one second
            *abort_flag = 1;
            atomicExch(status, STATUS_GEMM_TIMEOUT);
            return false;
        }
    }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}
// TMA store of one box of a 3-D map from shared memory to coordinates {c0, c1, c2}.  Out-of-range parts of
// the box are not written.  Completion is tracked by the issuing thread's bulk async-groups: commit, then
// wait (".read": the source has been read and may be overwritten; "but one": all groups except the latest).
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, uint32_t src, int c0, int c1, int c2) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
                 ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(c0), "r"(c1), "r"(c2)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read_but_one() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// Orders this thread's completed bulk stores (async proxy) before its later ordinary accesses to the same memory.
__device__ __forceinline__ void fence_async_to_generic() { asm volatile("fence.proxy.async;" ::: "memory"); }
// 128-bit load that is served from L2: for data that this kernel itself wrote earlier.
__device__ __forceinline__ uint4 ld_global_cg_16(const void* p) {
    uint4 v;
    asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
// Makes this thread's shared-memory writes visible to the async proxy (TMA) before a store is issued.
__device__ __forceinline__ void fence_smem_to_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void st_shared_16(uint32_t addr, uint4 w) {
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w.x), "r"(w.y), "r"(w.z), "r"(w.w) : "memory");
}
__device__ __forceinline__ uint4 ld_shared_16(uint32_t addr) {
    uint4 w;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(w.x), "=r"(w.y), "=r"(w.z), "=r"(w.w) : "r"(addr) : "memory");
    return w;
}
__device__ __forceinline__ void tensormap_acquire(const CUtensorMap* map) {
    asm volatile("fence.proxy.tensormap::generic.acquire.gpu [%0], 128;" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// 32 lanes x 32 columns of 32-bit accumulators: thread i of the warp receives row (lane base + i).
__device__ __forceinline__ void tc_load_32(uint32_t taddr, float* v) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// The same load without the wait, so that several can be in flight; tc_load_wait() makes all of them valid.
__device__ __forceinline__ void tc_load_32_issue(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tc_load_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor for a 128-byte-swizzled operand tile.
//   K-major : rows of 64 bf16 (128 B); 8-row groups 1024 B apart (stride byte offset).
//   MN-major: rows of 64 MN elements (128 B) per k; 8-k groups 1024 B apart (stride byte offset);
//             the next 64 MN elements start BK*128 B further (leading byte offset).
template <bool MN_MAJOR>
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr) {
    constexpr uint64_t lbo = MN_MAJOR ? (BK * 128) >> 4 : 1;
    constexpr uint64_t sbo = 1024 >> 4;
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3ffff) >> 4);  // start address, bits [0,14)
    d |= lbo << 16;                                           // leading byte offset, bits [16,30)
    d |= sbo << 32;                                           // stride byte offset, bits [32,46)
    d |= 1ull << 46;                                          // descriptor version for sm_100
    d |= 2ull << 61;                                          // layout: 128-byte swizzle
    return d;
}
// Bytes to advance the start address for the next 16 reduction elements.
template <bool MN_MAJOR>
__device__ __forceinline__ constexpr uint32_t desc_k_step() { return MN_MAJOR ? UMMA_K * 128 : UMMA_K * 2; }

// A/B format field of the kind::f16 instruction descriptor: 1 = bfloat16, 0 = IEEE half.
__device__ __forceinline__ uint32_t with_operand_format(uint32_t idesc_bf16, bool f16) {
    return f16 ? (idesc_bf16 & ~((7u << 7) | (7u << 10))) : idesc_bf16;
}

template <bool A_MN, bool B_MN>
__device__ __forceinline__ constexpr uint32_t make_instr_desc() {
    return (1u << 4)                      // accumulator format: fp32
           | (1u << 7)                    // A format: bf16 (see with_operand_format)
           | (1u << 10)                   // B format: bf16
           | ((A_MN ? 1u : 0u) << 15)     // A major
           | ((B_MN ? 1u : 0u) << 16)     // B major
           | (static_cast<uint32_t>(BN >> 3) << 17)
           | (static_cast<uint32_t>(BM >> 4) << 24);
}


// ---------------------------------------------------------------------------
// epilogue helpers
// ---------------------------------------------------------------------------
// The kernels handle bfloat16 and IEEE half with the same code: both are 16-bit elements, the tensor cores
// take either (a field of the instruction descriptor), and only the conversions at the edges differ.  `f16` is
// a kernel parameter, uniform over the launch.
__device__ __forceinline__ uint4 pack8(const float* f, bool f16) {
    return f16 ? Elem<__half>::pack(f) : Elem<__nv_bfloat16>::pack(f);
}
__device__ __forceinline__ void unpack8(const uint4& v, float* f, bool f16) {
    if (f16) Elem<__half>::unpack(v, f); else Elem<__nv_bfloat16>::unpack(v, f);
}
__device__ __forceinline__ float round16(float x, bool f16) { return f16 ? Elem<__half>::round(x) : round_bf16(x); }

// sigmoid of two values, 1 / (1 + 2^(-x log2 e)), with the approximate exp2 and reciprocal instructions and packed
// fp32 arithmetic.  No clamp is needed: 2^(+large) is +inf, whose reciprocal is 0, and 2^(-large) is 0.
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float rcp_approx(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float2 sigmoid2_fast(float2 x) {
    const float2 t = __fmul2_rn(x, make_float2(-1.4426950408889634f, -1.4426950408889634f));
    const float2 d = __fadd2_rn(make_float2(ex2_approx(t.x), ex2_approx(t.y)), make_float2(1.f, 1.f));
    return make_float2(rcp_approx(d.x), rcp_approx(d.y));
}
// act = up * gate * sigmoid(gate) on 8 values (two at a time)
__device__ __forceinline__ void swiglu_fwd8(const float* u, const float* g, float* act) {
#pragma unroll
    for (int e = 0; e < 8; e += 2) {
        const float2 g2 = make_float2(g[e], g[e + 1]);
        const float2 r = __fmul2_rn(__fmul2_rn(make_float2(u[e], u[e + 1]), g2), sigmoid2_fast(g2));
        act[e] = r.x;
        act[e + 1] = r.y;
    }
}
// d_up = d * silu(gate);  d_gate = d * up * (s + silu(gate) * (1 - s)),  s = sigmoid(gate)
__device__ __forceinline__ void swiglu_bwd8(const float* d, const float* u, const float* g, float* du, float* dg) {
#pragma unroll
    for (int e = 0; e < 8; e += 2) {
        const float2 g2 = make_float2(g[e], g[e + 1]), d2 = make_float2(d[e], d[e + 1]);
        const float2 s = sigmoid2_fast(g2);
        const float2 silu = __fmul2_rn(g2, s);
        const float2 one_minus_s = __ffma2_rn(s, make_float2(-1.f, -1.f), make_float2(1.f, 1.f));
        const float2 w = __ffma2_rn(silu, one_minus_s, s);
        const float2 a = __fmul2_rn(d2, silu);
        const float2 b = __fmul2_rn(__fmul2_rn(d2, make_float2(u[e], u[e + 1])), w);
        du[e] = a.x;
        du[e + 1] = a.y;
        dg[e] = b.x;
        dg[e + 1] = b.y;
    }
}

// one thread owns one output row, 32 columns at a time
__device__ __forceinline__ void store_row32(__nv_bfloat16* dst, const float* v, int cols_left, bool f16) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        if (q * 8 < cols_left) st_global_16(dst + q * 8, pack8(v + q * 8, f16));
    }
}
__device__ __forceinline__ void load_row32(const __nv_bfloat16* src, float* v, int cols_left, bool f16) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        if (q * 8 < cols_left) {
            unpack8(ld_global_16(src + q * 8), v + q * 8, f16);
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[q * 8 + i] = 0.f;
        }
    }
}


// ---------------------------------------------------------------------------
// host side: tensor maps and launches
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}

// 2-D tensor of 16-bit elements [outer, inner] with row pitch `pitch` elements, box [box_outer, box_inner], 128-byte swizzle.
inline int encode_2d(CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer, uint64_t pitch,
                     uint32_t box_inner, uint32_t box_outer, bool f16 = false) {
    EncodeTiledFn fn = encode_fn();
    FMAB_REQUIRE(fn != nullptr, FMA_B200_ERR_LAUNCH, "cuTensorMapEncodeTiled is not available from the driver");
    FMAB_REQUIRE(aligned16(base), FMA_B200_ERR_BAD_ARG, "GEMM operand is not 16-byte aligned");
    FMAB_REQUIRE((pitch * 2) % 16 == 0, FMA_B200_ERR_BAD_ARG, "row pitch %llu elements is not a multiple of 8",
                 (unsigned long long)pitch);
    FMAB_REQUIRE(inner >= 1 && outer >= 1, FMA_B200_ERR_BAD_ARG, "empty tensor for a tensor map");
    const cuuint64_t dims[2] = {inner, outer};
    const cuuint64_t strides[1] = {pitch * 2};
    const cuuint32_t box[2] = {box_inner, box_outer};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(map, f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                          const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    FMAB_REQUIRE(r == CUDA_SUCCESS, FMA_B200_ERR_LAUNCH, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return FMA_B200_OK;
}

// 3-D tensor of 16-bit elements {d0 (contiguous), d1, d2} with pitches in elements, boxes of box0 x box1 x 1 whose rows are
// box0 * 2 = 64 bytes wide, 64-byte swizzle: the output map of the epilogue that stores with TMA.
inline int encode_3d_box(CUtensorMap* map, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t pitch1,
                         uint64_t pitch2, uint32_t box0, uint32_t box1, uint32_t box2, bool f16 = false) {
    EncodeTiledFn fn = encode_fn();
    FMAB_REQUIRE(fn != nullptr, FMA_B200_ERR_LAUNCH, "cuTensorMapEncodeTiled is not available from the driver");
    FMAB_REQUIRE(aligned16(base), FMA_B200_ERR_BAD_ARG, "GEMM output is not 16-byte aligned");
    FMAB_REQUIRE((pitch1 * 2) % 16 == 0 && (pitch2 * 2) % 16 == 0, FMA_B200_ERR_BAD_ARG,
                 "output pitches %llu / %llu elements are not multiples of 8", (unsigned long long)pitch1,
                 (unsigned long long)pitch2);
    FMAB_REQUIRE(d0 >= 1 && d1 >= 1 && d2 >= 1, FMA_B200_ERR_BAD_ARG, "empty tensor for a tensor map");
    const cuuint64_t dims[3] = {d0, d1, d2};
    const cuuint64_t strides[2] = {pitch1 * 2, pitch2 * 2};
    const cuuint32_t box[3] = {box0, box1, box2};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = fn(map, f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3,
                          const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    FMAB_REQUIRE(r == CUDA_SUCCESS, FMA_B200_ERR_LAUNCH, "cuTensorMapEncodeTiled (3-D) failed with CUresult %d", (int)r);
    return FMA_B200_OK;
}

inline int encode_3d(CUtensorMap* map, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t pitch1,
                     uint64_t pitch2, uint32_t box0, uint32_t box1, bool f16 = false) {
    return encode_3d_box(map, base, d0, d1, d2, pitch1, pitch2, box0, box1, 1, f16);
}

// Scheduler words of the dynamic tile scheduler: 64 pairs per device, handed out round-robin so that
// launches running concurrently on different streams do not share a pair.  Zero at load; every launch
// leaves its pair zero again.
// (one copy per translation unit that includes this header: each kernel file uses its own words)
static __device__ unsigned int g_sched_words[64 * 2];

static int next_sched_pair(unsigned int** out) {
    static unsigned int* base[64] = {nullptr};
    static unsigned int seq = 0;
    int dev = -1;
    FMAB_CUDA(cudaGetDevice(&dev));
    FMAB_REQUIRE(dev >= 0 && dev < 64, FMA_B200_ERR_BAD_ARG, "device ordinal %d is outside [0,64)", dev);
    if (base[dev] == nullptr) {
        void* ptr = nullptr;
        FMAB_CUDA(cudaGetSymbolAddress(&ptr, g_sched_words));
        base[dev] = static_cast<unsigned int*>(ptr);
    }
    *out = base[dev] + 2 * (__atomic_fetch_add(&seq, 1u, __ATOMIC_RELAXED) % 64u);
    return FMA_B200_OK;
}

// FMA_B200_GEMM_STATIC_TILES=1 switches the dynamic tile scheduler off (a measurement knob).
static int dynamic_tiles_enabled() {
    static int dynamic = -1;
    if (dynamic < 0) {
        const char* env = getenv("FMA_B200_GEMM_STATIC_TILES");
        dynamic = (env != nullptr && atoi(env) == 1) ? 0 : 1;
    }
    return dynamic;
}

}  // namespace fmab
