// continuous_count: integer histogram of ids in [0, size), HBM-bound.
//
// One launch, no zero-fill pass:
//   1. every block builds a histogram of its share of the ids in shared memory (128-bit streaming
//      loads, several in flight per thread);
//   2. it adds its non-zero bins to an accumulator in the caller's workspace (one global integer
//      atomic per bin and block; the accumulator is zero between calls) and takes a ticket;
//   3. the block that draws the last ticket moves the accumulator to `out` with atomicExch, which
//      also clears it, and resets the ticket: the workspace is ready for the next call.
// Integer atomics commute, so the result is exact and independent of block order.
//
// Three shared-memory schemes, selectable for measurement (fma_b200_continuous_count_variant):
//   variant 0 (default): up to 32 sub-histograms per block, one per lane, at a pitch that is 1 mod 32
//     words, updated with shared-memory atomics.  Lanes of a warp never hit the same address however
//     skewed the ids are, and equal ids in different lanes fall in different banks.  64 resident
//     warps per SM hide the memory latency.
//   variant 1: one histogram per block, equal ids of a warp merged with match.any before one atomic
//     per distinct id (warp-aggregated atomics).
//   variant 2 (size <= 1024): every lane of every warp owns a private column hist[warp][bin][lane];
//     increments are plain load / add / store, four in flight at a time; one block per SM.
// Measured on B200 (2^24 int32 ids, 128 bins, uniform and Zipf 1.1 alike): variant 0 20.5 us,
// variant 2 24.6 us, variant 1 85-121 us; at 2^28 ids variant 0 streams at 5.9 TB/s and variant 2 at
// 5.0 TB/s.  Variant 1 is limited by match.any; variant 2 by the latency of its read-modify-write
// chains at only 13 warps per SM.  About 12 us of every launch is size-independent (launch ramp and
// the accumulate / ticket / exchange tail).
#include "common.cuh"

namespace fmab {

constexpr int kCountThreads = 512;          // block size of the atomic variants
constexpr int kCountTicketWords = 32;       // the accumulator starts 128 bytes into the workspace
constexpr int kAccSlots = 8;                // copies of the accumulator; block b adds to copy b % 8 (8x fewer same-address atomics)
constexpr int kPrivateMaxBins = 1024;       // variant 2: (size+1)*128 B per warp must fit ~216 KB
constexpr int kPrivateLoads = 8;            // 16-byte vectors per buffer; two buffers per thread (one in flight)

template <typename IdT>
__device__ __forceinline__ bool id_in_range(IdT v, int size) {
    return static_cast<uint64_t>(v) < static_cast<uint64_t>(size);  // negative ids wrap to huge values
}
template <>
__device__ __forceinline__ bool id_in_range<int32_t>(int32_t v, int size) {
    return static_cast<uint32_t>(v) < static_cast<uint32_t>(size);
}

// Called by every thread of a block after it has added its bins to `acc`.
__device__ __forceinline__ void finish_in_last_block(int size, uint32_t* __restrict__ out, uint32_t* __restrict__ ticket,
                                                     uint32_t* __restrict__ acc) {
    __shared__ bool is_last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint32_t t = atomicAdd(ticket, 1u);
        is_last = (t == gridDim.x - 1);
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    for (int b = threadIdx.x; b < size; b += blockDim.x) {
        uint32_t s = 0;
#pragma unroll
        for (int c = 0; c < kAccSlots; ++c) s += atomicExch(&acc[c * size + b], 0u);  // read and clear
        out[b] = s;
    }
    if (threadIdx.x == 0) *ticket = 0;
}

// ---------------------------------------------------------------------------
// variant 2: lane-private 32-bit counters, no shared-memory atomics
// ---------------------------------------------------------------------------
// Shared memory of one warp: words [bin][lane]; row `size` is a sink for ids outside the range.
// The bank of every access is the lane id, so a warp-wide increment is two conflict-free
// shared-memory accesses (one load, one store) and three integer instructions.
__device__ __forceinline__ uint32_t clamp_bin(int32_t v, int size) {
    return min(static_cast<uint32_t>(v), static_cast<uint32_t>(size));  // negatives wrap above size
}
__device__ __forceinline__ uint32_t clamp_bin(int64_t v, int size) {
    return (static_cast<uint64_t>(v) < static_cast<uint64_t>(size)) ? static_cast<uint32_t>(v) : static_cast<uint32_t>(size);
}
// 128-bit streaming load that the compiler keeps ahead of the shared-memory work that follows it.
__device__ __forceinline__ uint4 ld_stream_16_early(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p)
                 : "memory");
    return v;
}

// Four increments with their four shared-memory loads in flight together (a read-modify-write chain
// costs ~120 cycles of latency, so issuing them one by one leaves a warp idle most of the time).
// Stores are issued in order and every value includes the earlier increments of the same bin, so
// repeated bins end up correct.
__device__ __forceinline__ void bump4(uint32_t* col, uint32_t b0, uint32_t b1, uint32_t b2, uint32_t b3) {
    uint32_t* p0 = col + b0 * 32;
    uint32_t* p1 = col + b1 * 32;
    uint32_t* p2 = col + b2 * 32;
    uint32_t* p3 = col + b3 * 32;
    const uint32_t x0 = *p0, x1 = *p1, x2 = *p2, x3 = *p3;
    const uint32_t v0 = x0 + 1;
    const uint32_t v1 = (b1 == b0) ? v0 + 1 : x1 + 1;
    const uint32_t v2 = (b2 == b1) ? v1 + 1 : (b2 == b0) ? v0 + 1 : x2 + 1;
    const uint32_t v3 = (b3 == b2) ? v2 + 1 : (b3 == b1) ? v1 + 1 : (b3 == b0) ? v0 + 1 : x3 + 1;
    *p0 = v0;
    *p1 = v1;
    *p2 = v2;
    *p3 = v3;
}

template <typename IdT>
__global__ void __launch_bounds__(512)
continuous_count_private_kernel(const IdT* __restrict__ ids, int64_t n, int size, uint32_t* __restrict__ out,
                                uint32_t* __restrict__ ticket, uint32_t* __restrict__ acc) {
    extern __shared__ uint32_t smem[];  // [size] block histogram, then [warps][size + 1][32] counters
    constexpr int kPerVec = 16 / sizeof(IdT);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int rows = size + 1;
    uint32_t* block_hist = smem;
    uint32_t* warp_hist = smem + ((size + 31) / 32) * 32 + warp * rows * 32;
    uint32_t* col = warp_hist + lane;

    const int64_t n_vec = n / kPerVec;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    const uint4* vec = reinterpret_cast<const uint4*>(ids);
    const uint4 filler = make_uint4(~0u, ~0u, ~0u, ~0u);  // decodes to out-of-range ids -> sink row
    int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;

    // the first loads are issued before the counters are cleared
    uint4 cur[kPrivateLoads], nxt[kPrivateLoads];
#pragma unroll
    for (int u = 0; u < kPrivateLoads; ++u)
        cur[u] = (i + u * stride < n_vec) ? ld_stream_16_early(vec + i + u * stride) : filler;
    for (int b = threadIdx.x; b < size; b += blockDim.x) block_hist[b] = 0;
    {
        uint4* z = reinterpret_cast<uint4*>(warp_hist);
        for (int w = lane; w < rows * 8; w += 32) z[w] = make_uint4(0, 0, 0, 0);
    }
    __syncthreads();
    while (i < n_vec) {
        // next buffer in flight while this one is counted
        const int64_t j = i + kPrivateLoads * stride;
#pragma unroll
        for (int u = 0; u < kPrivateLoads; ++u)
            nxt[u] = (j + u * stride < n_vec) ? ld_stream_16_early(vec + j + u * stride) : filler;
        {
            const IdT* e = reinterpret_cast<const IdT*>(&cur[0]);
#pragma unroll
            for (int q = 0; q < kPrivateLoads * kPerVec; q += 4)
                bump4(col, clamp_bin(e[q], size), clamp_bin(e[q + 1], size), clamp_bin(e[q + 2], size),
                      clamp_bin(e[q + 3], size));
        }
#pragma unroll
        for (int u = 0; u < kPrivateLoads; ++u) cur[u] = nxt[u];
        i = j;
    }
    // tail ids (n % kPerVec of them), one per lane of the first warp of block 0
    if (blockIdx.x == 0 && warp == 0) {
        const int64_t t = n_vec * kPerVec + lane;
        if (t < n) col[clamp_bin(ids[t], size) * 32] += 1;
    }
    __syncwarp();
    // fold this warp's columns: lane l sums row b0+l over the 32 lanes, rotated to stay conflict-free
    for (int b0 = 0; b0 < size; b0 += 32) {
        const int b = b0 + lane;
        if (b < size) {
            uint32_t s = 0;
#pragma unroll
            for (int j = 0; j < 32; ++j) s += warp_hist[b * 32 + ((j + lane) & 31)];
            if (s != 0) atomicAdd(&block_hist[b], s);
        }
    }
    __syncthreads();
    for (int b = threadIdx.x; b < size; b += blockDim.x) {
        const uint32_t s = block_hist[b];
        if (s != 0) atomicAdd(&acc[(blockIdx.x % kAccSlots) * size + b], s);
    }
    finish_in_last_block(size, out, ticket, acc);
}

// ---------------------------------------------------------------------------
// variants 0 and 1: shared-memory atomics
// ---------------------------------------------------------------------------
template <typename IdT, bool kAggregate>
__device__ __forceinline__ void count_one(IdT v, int size, uint32_t* hist_lane) {
    if constexpr (kAggregate) {
        const bool ok = id_in_range(v, size);
        const unsigned active = __ballot_sync(0xffffffffu, ok);
        if (ok) {
            const unsigned same = __match_any_sync(active, static_cast<int>(v));
            const int leader = __ffs(same) - 1;
            if ((threadIdx.x & 31) == leader) atomicAdd(&hist_lane[static_cast<int>(v)], __popc(same));
        }
    } else {
        if (id_in_range(v, size)) atomicAdd(&hist_lane[static_cast<int>(v)], 1u);
    }
}

template <typename IdT, bool kAggregate>
__global__ void __launch_bounds__(kCountThreads)
continuous_count_kernel(const IdT* __restrict__ ids, int64_t n, int size, int copies, int pitch,
                        uint32_t* __restrict__ out, uint32_t* __restrict__ ticket, uint32_t* __restrict__ acc) {
    extern __shared__ uint32_t hist[];
    constexpr int kPerVec = 16 / sizeof(IdT);

    for (int i = threadIdx.x; i < copies * pitch; i += kCountThreads) hist[i] = 0;
    __syncthreads();

    uint32_t* hist_lane = kAggregate ? hist : hist + (threadIdx.x & (copies - 1)) * pitch;

    // Body: whole 16-byte vectors, four independent loads in flight per thread.
    const int64_t n_vec = n / kPerVec;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * kCountThreads;
    int64_t i = static_cast<int64_t>(blockIdx.x) * kCountThreads + threadIdx.x;
    const uint4* vec = reinterpret_cast<const uint4*>(ids);
    // The aggregated variant uses warp-wide votes, so all lanes of a warp must take the
    // same trip count: iterate on the warp's first index and predicate each lane.
    const int64_t warp_first = i - (threadIdx.x & 31);
    for (int64_t base = warp_first; base < n_vec; base += 4 * stride, i += 4 * stride) {
        uint4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
            v[u] = ((i + u * stride) < n_vec) ? ld_stream_16(vec + i + u * stride) : make_uint4(~0u, ~0u, ~0u, ~0u);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            // Out-of-range filler (all ones = -1) is ignored by count_one.
            const IdT* e = reinterpret_cast<const IdT*>(&v[u]);
#pragma unroll
            for (int j = 0; j < kPerVec; ++j) count_one<IdT, kAggregate>(e[j], size, hist_lane);
        }
    }
    // Tail: the last n % kPerVec ids, taken by the first warp of block 0.
    if (blockIdx.x == 0 && threadIdx.x < 32) {
        const int64_t t = n_vec * kPerVec + threadIdx.x;
        const IdT v = (t < n) ? ids[t] : static_cast<IdT>(-1);
        count_one<IdT, kAggregate>(v, size, hist_lane);
    }
    __syncthreads();

    for (int b = threadIdx.x; b < size; b += kCountThreads) {
        uint32_t s = 0;
        if constexpr (kAggregate) {
            s = hist[b];
        } else {
            for (int c = 0; c < copies; ++c) s += hist[c * pitch + b];
        }
        if (s != 0) atomicAdd(&acc[(blockIdx.x % kAccSlots) * size + b], s);
    }
    finish_in_last_block(size, out, ticket, acc);
}

// ---------------------------------------------------------------------------
// launch: `scratch` = [ticket (32 words, word 0 used)] [kAccSlots accumulators of size words], all zero between calls
// ---------------------------------------------------------------------------
template <typename IdT>
static int launch_count(const void* ids, int64_t n, int size, uint32_t* out, uint32_t* scratch, int variant,
                        cudaStream_t stream) {
    constexpr int kPerVec = 16 / sizeof(IdT);
    uint32_t* ticket = scratch;
    uint32_t* acc = scratch + kCountTicketWords;
    const int64_t n_vec = n / kPerVec;
    if (variant == 2) {
        const int64_t per_warp = static_cast<int64_t>(size + 1) * 32 * 4;
        const int64_t block_hist = static_cast<int64_t>((size + 31) / 32) * 32 * 4;
        int warps = static_cast<int>((216 * 1024 - block_hist) / per_warp);
        warps = warps < 1 ? 1 : (warps > 16 ? 16 : warps);
        const int64_t smem = block_hist + warps * per_warp;
        static bool configured[2][64] = {{false}};  // per id width and device
        const int dev = current_device_slot();
        FMAB_REQUIRE(dev >= 0, FMA_B200_ERR_LAUNCH, "no current CUDA device with an ordinal below 64");
        bool& conf = configured[sizeof(IdT) == 4 ? 0 : 1][dev];
        if (!conf) {
            FMAB_CUDA(cudaFuncSetAttribute(continuous_count_private_kernel<IdT>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
            conf = true;
        }
        const int threads = warps * 32;
        const int64_t per_trip = static_cast<int64_t>(threads) * kPrivateLoads;
        const int64_t want = (n_vec + per_trip - 1) / per_trip;
        const int64_t cap = sm_count();  // one block per SM (its shared memory fills the SM)
        const int grid = static_cast<int>(want < 1 ? 1 : (want > cap ? cap : want));
        continuous_count_private_kernel<IdT><<<grid, threads, smem, stream>>>(static_cast<const IdT*>(ids), n, size,
                                                                             out, ticket, acc);
        return check_launch("continuous_count (lane-private)");
    }
    // Largest power-of-two number of sub-histograms that fits 48 KB of shared memory.
    const int pitch = ((size + 31) / 32) * 32 + 1;
    int copies = (variant == 1) ? 1 : 32;
    while (copies > 1 && static_cast<int64_t>(copies) * pitch * 4 > 48 * 1024) copies >>= 1;
    const int64_t smem = static_cast<int64_t>(copies) * pitch * 4;
    if (smem > 48 * 1024) {
        cudaError_t e;
        if (variant == 1)
            e = cudaFuncSetAttribute(continuous_count_kernel<IdT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        else
            e = cudaFuncSetAttribute(continuous_count_kernel<IdT, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail(FMA_B200_ERR_LAUNCH, "continuous_count smem opt-in: %s", cudaGetErrorString(e));
    }
    // Four vectors per thread per trip; a few resident blocks per SM.
    const int64_t want = (n_vec + 4LL * kCountThreads - 1) / (4LL * kCountThreads);
    const int64_t cap = static_cast<int64_t>(sm_count()) * ((smem > 24 * 1024) ? 2 : 4);
    const int grid = static_cast<int>(want < 1 ? 1 : (want > cap ? cap : want));
    if (variant == 1)
        continuous_count_kernel<IdT, true><<<grid, kCountThreads, smem, stream>>>(static_cast<const IdT*>(ids), n, size,
                                                                                copies, pitch, out, ticket, acc);
    else
        continuous_count_kernel<IdT, false><<<grid, kCountThreads, smem, stream>>>(static_cast<const IdT*>(ids), n, size,
                                                                                 copies, pitch, out, ticket, acc);
    return check_launch("continuous_count");
}

static int check_count_args(const void* ids, int32_t id_bytes, int64_t n, int32_t size, const uint32_t* out) {
    FMAB_REQUIRE(out != nullptr, FMA_B200_ERR_BAD_ARG, "out is NULL");
    FMAB_REQUIRE(n >= 0 && n < (1LL << 40), FMA_B200_ERR_BAD_ARG, "n=%lld out of range", (long long)n);
    FMAB_REQUIRE(n == 0 || ids != nullptr, FMA_B200_ERR_BAD_ARG, "ids is NULL");
    FMAB_REQUIRE(size >= 1, FMA_B200_ERR_BAD_ARG, "size=%d must be positive", size);
    FMAB_REQUIRE(id_bytes == 4 || id_bytes == 8, FMA_B200_ERR_UNSUPPORTED, "ids must be int32 or int64");
    FMAB_REQUIRE(aligned16(ids), FMA_B200_ERR_BAD_ARG, "ids not 16-byte aligned");
    return FMA_B200_OK;
}

// ---------------------------------------------------------------------------
// Variant for callers that cannot allocate device memory
// ---------------------------------------------------------------------------
// Some callers of this library have no way to obtain scratch memory at the point of the call:
// a plugin loaded into a host whose device heap is owned by someone else (an inference server's
// arena, another framework's caching allocator), code running inside a region where cudaMalloc
// would synchronise the device and break the host's stream ordering, or a small C program that
// links the library and wants a histogram without writing an allocator.  For them the ticket and
// the accumulator live in this file-scope array instead of a caller-provided workspace.  Every
// GPU that loads the library holds these 32 KiB + 128 B until the process exits.
constexpr int kStaticCountMaxBins = 1024;  // largest `size` the static variant accepts
static __device__ __align__(256) uint32_t g_static_count_scratch[kCountTicketWords + kAccSlots * kStaticCountMaxBins];

// In host code `g_static_count_scratch` is only a handle for the runtime, not a device address, so
// the address the kernel needs is looked up once per device (with that device current) and cached.
static int static_count_scratch(uint32_t** out) {
    static uint32_t* cached[64] = {nullptr};
    int dev = -1;
    FMAB_CUDA(cudaGetDevice(&dev));
    FMAB_REQUIRE(dev >= 0 && dev < 64, FMA_B200_ERR_BAD_ARG, "device ordinal %d is outside [0,64)", dev);
    if (cached[dev] == nullptr) {
        void* p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_static_count_scratch);
        if (e != cudaSuccess || p == nullptr)
            return fail(FMA_B200_ERR_LAUNCH, "cudaGetSymbolAddress(static count scratch): %s", cudaGetErrorString(e));
        cached[dev] = static_cast<uint32_t*>(p);
    }
    *out = cached[dev];
    return FMA_B200_OK;
}

}  // namespace fmab

extern "C" {

int64_t fma_b200_continuous_count_workspace_bytes(int32_t size) {
    if (size < 1) return 0;
    return (static_cast<int64_t>(fmab::kCountTicketWords) + static_cast<int64_t>(fmab::kAccSlots) * size) * 4;
}

int fma_b200_continuous_count_variant(const void* ids, int32_t id_bytes, int64_t n, int32_t size, uint32_t* out,
                                      void* workspace, int64_t workspace_bytes, int32_t variant, void* stream) {
    using namespace fmab;
    if (int rc = check_count_args(ids, id_bytes, n, size, out)) return rc;
    FMAB_REQUIRE(workspace != nullptr && aligned16(workspace), FMA_B200_ERR_BAD_ARG, "workspace NULL or not 16-byte aligned");
    FMAB_REQUIRE(size <= 16384, FMA_B200_ERR_BAD_ARG, "size=%d not in [1,16384]", size);
    FMAB_REQUIRE(variant >= 0 && variant <= 2, FMA_B200_ERR_BAD_ARG, "variant must be 0, 1 or 2");
    FMAB_REQUIRE(variant != 2 || size <= kPrivateMaxBins, FMA_B200_ERR_BAD_ARG, "variant 2 handles at most %d bins",
                 kPrivateMaxBins);
    FMAB_REQUIRE(workspace_bytes >= fma_b200_continuous_count_workspace_bytes(size), FMA_B200_ERR_WORKSPACE,
                 "continuous_count workspace: %lld < %lld bytes", (long long)workspace_bytes,
                 (long long)fma_b200_continuous_count_workspace_bytes(size));
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    uint32_t* scratch = static_cast<uint32_t*>(workspace);
    if (id_bytes == 4) return launch_count<int32_t>(ids, n, size, out, scratch, variant, s);
    return launch_count<int64_t>(ids, n, size, out, scratch, variant, s);
}

int fma_b200_continuous_count(const void* ids, int32_t id_bytes, int64_t n, int32_t size, uint32_t* out,
                              void* workspace, int64_t workspace_bytes, void* stream) {
    const int32_t variant = 0;  // measured fastest on B200 at every input size (see the header of this file)
    return fma_b200_continuous_count_variant(ids, id_bytes, n, size, out, workspace, workspace_bytes, variant, stream);
}

int fma_b200_continuous_count_static(const void* ids, int32_t id_bytes, int64_t n, int32_t size, uint32_t* out,
                                     void* stream) {
    using namespace fmab;
    if (int rc = check_count_args(ids, id_bytes, n, size, out)) return rc;
    FMAB_REQUIRE(size <= kStaticCountMaxBins, FMA_B200_ERR_BAD_ARG,
                 "size=%d exceeds the %d bins the built-in scratch array supports; use fma_b200_continuous_count "
                 "with a caller-provided workspace", size, kStaticCountMaxBins);
    uint32_t* scratch = nullptr;
    if (int rc = static_count_scratch(&scratch)) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // Same kernel choice as the workspace form.  The array is zero when the library is loaded and every
    // call leaves it zero again.
    const int variant = 0;
    if (id_bytes == 4) return launch_count<int32_t>(ids, n, size, out, scratch, variant, s);
    return launch_count<int64_t>(ids, n, size, out, scratch, variant, s);
}

}  // extern "C"
