// continuous_count: integer histogram of ids in [0, size), HBM-bound.
//
// One launch, no zero-fill pass and no global atomics on the result:
//   1. every block builds a histogram in shared memory from 128-bit streaming loads;
//   2. it writes its partial histogram to the workspace and takes a ticket;
//   3. the block that draws the last ticket sums the partials into `out` and
//      resets the ticket, so the workspace is ready for the next call.
// Shared-memory layout (variant 0): up to 32 sub-histograms, one per lane, at a
// pitch that is 1 mod 32 words.  Lanes of a warp therefore never hit the same address,
// however skewed the ids are, and equal ids in different lanes fall in different banks.
// Variant 1 keeps one histogram per block and merges equal ids of a warp with
// match.any before a single atomic per distinct id (warp-aggregated atomics).
#include "common.cuh"

namespace fmab {

constexpr int kCountThreads = 512;
constexpr int kCountMaxBlocks = 1024;
constexpr int kCountTicketBytes = 128;

template <typename IdT>
__device__ __forceinline__ bool id_in_range(IdT v, int size) {
    return static_cast<uint64_t>(v) < static_cast<uint64_t>(size);  // negative ids wrap to huge values
}
template <>
__device__ __forceinline__ bool id_in_range<int32_t>(int32_t v, int size) {
    return static_cast<uint32_t>(v) < static_cast<uint32_t>(size);
}

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
                        uint32_t* __restrict__ out, uint32_t* __restrict__ ticket, uint32_t* __restrict__ partials) {
    extern __shared__ uint32_t hist[];
    __shared__ bool is_last;
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
        bool live[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            live[u] = (i + u * stride) < n_vec;
            v[u] = live[u] ? ld_stream_16(vec + i + u * stride) : make_uint4(~0u, ~0u, ~0u, ~0u);
        }
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

    // Fold the sub-histograms and publish this block's partial.
    uint32_t* mine = partials + static_cast<int64_t>(blockIdx.x) * size;
    for (int b = threadIdx.x; b < size; b += kCountThreads) {
        uint32_t s = 0;
        if constexpr (kAggregate) {
            s = hist[b];
        } else {
            for (int c = 0; c < copies; ++c) s += hist[c * pitch + b];
        }
        mine[b] = s;
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint32_t t = atomicAdd(ticket, 1u);
        is_last = (t == gridDim.x - 1);
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    for (int b = threadIdx.x; b < size; b += kCountThreads) {
        uint32_t s = 0;
        for (unsigned g = 0; g < gridDim.x; ++g) s += __ldcg(partials + static_cast<int64_t>(g) * size + b);
        out[b] = s;
    }
    if (threadIdx.x == 0) *ticket = 0;
}

template <typename IdT>
static int launch_count(const void* ids, int64_t n, int size, uint32_t* out, void* workspace, int variant,
                        cudaStream_t stream) {
    constexpr int kPerVec = 16 / sizeof(IdT);
    // Largest power-of-two number of sub-histograms that fits 48 KB of shared memory.
    const int pitch = ((size + 31) / 32) * 32 + 1;
    int copies = 32;
    if (variant == 1) copies = 1;
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
    const int64_t n_vec = n / kPerVec;
    // Four vectors per thread per trip; cap the grid at a few resident blocks per SM.
    int64_t want = (n_vec + 4LL * kCountThreads - 1) / (4LL * kCountThreads);
    const int resident = (smem > 24 * 1024) ? 2 : 4;
    int64_t cap = static_cast<int64_t>(sm_count()) * resident;
    if (cap > kCountMaxBlocks) cap = kCountMaxBlocks;
    int grid = static_cast<int>(want < 1 ? 1 : (want > cap ? cap : want));
    uint32_t* ticket = static_cast<uint32_t*>(workspace);
    uint32_t* partials = reinterpret_cast<uint32_t*>(static_cast<char*>(workspace) + kCountTicketBytes);
    if (variant == 1)
        continuous_count_kernel<IdT, true><<<grid, kCountThreads, smem, stream>>>(
            static_cast<const IdT*>(ids), n, size, copies, pitch, out, ticket, partials);
    else
        continuous_count_kernel<IdT, false><<<grid, kCountThreads, smem, stream>>>(
            static_cast<const IdT*>(ids), n, size, copies, pitch, out, ticket, partials);
    return check_launch("continuous_count");
}

// ---------------------------------------------------------------------------
// Variant for callers that cannot allocate device memory
// ---------------------------------------------------------------------------
// Some callers of this library have no way to obtain scratch memory at the point of the call:
// a plugin loaded into a host whose device heap is owned by someone else (an inference server's
// arena, another framework's caching allocator), code running inside a region where cudaMalloc
// would synchronise the device and break the host's stream ordering, or a small C program that
// links the library and wants a histogram without writing an allocator.  For them the ticket and
// the block partials live in this file-scope array instead of a caller-provided workspace.  Every
// GPU that loads the library holds these 2 MiB + 256 B until the process exits.
constexpr int kStaticCountMaxBins = 1024;                 // largest `size` the static variant accepts
constexpr int kStaticCountPartialWords = 512 * 1024;      // grid * size never exceeds this
static __device__ __align__(256) uint32_t g_static_count_scratch[64 + kStaticCountPartialWords];

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

template <typename IdT>
static int launch_count_static(const void* ids, int64_t n, int size, uint32_t* out, uint32_t* scratch,
                               cudaStream_t stream) {
    constexpr int kPerVec = 16 / sizeof(IdT);
    const int pitch = ((size + 31) / 32) * 32 + 1;
    int copies = 32;
    while (copies > 1 && static_cast<int64_t>(copies) * pitch * 4 > 48 * 1024) copies >>= 1;
    const int64_t smem = static_cast<int64_t>(copies) * pitch * 4;  // <= 48 KB for size <= 1024: no opt-in needed
    const int64_t n_vec = n / kPerVec;
    int64_t want = (n_vec + 4LL * kCountThreads - 1) / (4LL * kCountThreads);
    int64_t cap = static_cast<int64_t>(sm_count()) * ((smem > 24 * 1024) ? 2 : 4);
    if (cap > kStaticCountPartialWords / size) cap = kStaticCountPartialWords / size;  // partials must fit the array
    const int grid = static_cast<int>(want < 1 ? 1 : (want > cap ? cap : want));
    // word 0 is the ticket (zero at load, reset to zero by the last block of every call);
    // the partials start 256 bytes in and are fully rewritten by each call before they are read
    continuous_count_kernel<IdT, false><<<grid, kCountThreads, smem, stream>>>(
        static_cast<const IdT*>(ids), n, size, copies, pitch, out, scratch, scratch + 64);
    return check_launch("continuous_count_static");
}

}  // namespace fmab

extern "C" {

int64_t fma_b200_continuous_count_workspace_bytes(int32_t size) {
    if (size < 1) return 0;
    return fmab::kCountTicketBytes + static_cast<int64_t>(fmab::kCountMaxBlocks) * size * 4;
}

int fma_b200_continuous_count_variant(const void* ids, int32_t id_bytes, int64_t n, int32_t size, uint32_t* out,
                                      void* workspace, int64_t workspace_bytes, int32_t variant, void* stream) {
    using namespace fmab;
    FMAB_REQUIRE(out != nullptr && workspace != nullptr, FMA_B200_ERR_BAD_ARG, "out or workspace is NULL");
    FMAB_REQUIRE(n >= 0 && n < (1LL << 40), FMA_B200_ERR_BAD_ARG, "n=%lld out of range", (long long)n);
    FMAB_REQUIRE(n == 0 || ids != nullptr, FMA_B200_ERR_BAD_ARG, "ids is NULL");
    FMAB_REQUIRE(size >= 1 && size <= 16384, FMA_B200_ERR_BAD_ARG, "size=%d not in [1,16384]", size);
    FMAB_REQUIRE(id_bytes == 4 || id_bytes == 8, FMA_B200_ERR_UNSUPPORTED, "ids must be int32 or int64");
    FMAB_REQUIRE(variant == 0 || variant == 1, FMA_B200_ERR_BAD_ARG, "variant must be 0 or 1");
    FMAB_REQUIRE(aligned16(ids) && aligned16(workspace), FMA_B200_ERR_BAD_ARG, "ids/workspace not 16-byte aligned");
    FMAB_REQUIRE(workspace_bytes >= fma_b200_continuous_count_workspace_bytes(size), FMA_B200_ERR_WORKSPACE,
                 "continuous_count workspace: %lld < %lld bytes", (long long)workspace_bytes,
                 (long long)fma_b200_continuous_count_workspace_bytes(size));
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (id_bytes == 4) return launch_count<int32_t>(ids, n, size, out, workspace, variant, s);
    return launch_count<int64_t>(ids, n, size, out, workspace, variant, s);
}

int fma_b200_continuous_count(const void* ids, int32_t id_bytes, int64_t n, int32_t size, uint32_t* out,
                              void* workspace, int64_t workspace_bytes, void* stream) {
    return fma_b200_continuous_count_variant(ids, id_bytes, n, size, out, workspace, workspace_bytes, 0, stream);
}

int fma_b200_continuous_count_static(const void* ids, int32_t id_bytes, int64_t n, int32_t size, uint32_t* out,
                                     void* stream) {
    using namespace fmab;
    FMAB_REQUIRE(out != nullptr, FMA_B200_ERR_BAD_ARG, "out is NULL");
    FMAB_REQUIRE(n >= 0 && n < (1LL << 40), FMA_B200_ERR_BAD_ARG, "n=%lld out of range", (long long)n);
    FMAB_REQUIRE(n == 0 || ids != nullptr, FMA_B200_ERR_BAD_ARG, "ids is NULL");
    FMAB_REQUIRE(size >= 1, FMA_B200_ERR_BAD_ARG, "size=%d must be positive", size);
    FMAB_REQUIRE(size <= kStaticCountMaxBins, FMA_B200_ERR_BAD_ARG,
                 "size=%d exceeds the %d bins the built-in scratch array supports; use fma_b200_continuous_count "
                 "with a caller-provided workspace", size, kStaticCountMaxBins);
    FMAB_REQUIRE(id_bytes == 4 || id_bytes == 8, FMA_B200_ERR_UNSUPPORTED, "ids must be int32 or int64");
    FMAB_REQUIRE(aligned16(ids), FMA_B200_ERR_BAD_ARG, "ids not 16-byte aligned");
    uint32_t* scratch = nullptr;
    if (int rc = static_count_scratch(&scratch)) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (id_bytes == 4) return launch_count_static<int32_t>(ids, n, size, out, scratch, s);
    return launch_count_static<int64_t>(ids, n, size, out, scratch, s);
}

}  // extern "C"
