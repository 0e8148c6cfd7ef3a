// Peer-memory transport of the expert-parallel MoE: buffers that every rank of a node can address
// (CUDA IPC), row-block pushes with the copy engines (no SM taken from the GEMMs that run at the same
// time), and sequence-numbered flags that tell the receiver a block has landed.
//
//   sender, side stream:    peer_copy(blocks -> the receivers' arenas);  peer_signal(flag on each receiver = seq)
//   receiver, main stream:  peer_wait(flags >= seq);  grouped GEMM on the rows that arrived
//
// Copies and the signal kernel are ordered by the stream, so a flag is written only after the rows it
// announces are in the receiver's memory.  peer_wait polls with a time limit: when it runs out the
// kernel records STATUS_PEER_TIMEOUT in the library's device status word and returns, so a missing
// peer ends in an error that the host reads, not in a hang.
#include <string.h>

#include "common.cuh"

namespace fmab {

constexpr int32_t STATUS_PEER_TIMEOUT = 0x7002;
constexpr int kMaxSignals = 64;

struct SignalArgs {
    int32_t* flag[kMaxSignals];
};

__global__ void peer_signal_kernel(SignalArgs args, int n, int32_t value) {
    const int i = threadIdx.x;
    if (i < n) {
        __threadfence_system();
        asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(args.flag[i]), "r"(value) : "memory");
    }
}

// Thread i waits until flags[i] has reached `value` (sequence numbers only grow; compared modulo 2^32).
__global__ void peer_wait_kernel(const int32_t* __restrict__ flags, int n, int32_t value, uint64_t timeout_ns,
                                 int32_t* __restrict__ status) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    // once any wait has run out the exchange is broken: later waits return at once, so the step ends
    // quickly and the host finds the status word
    if (*reinterpret_cast<volatile const int32_t*>(status) == STATUS_PEER_TIMEOUT) return;
    uint64_t t0;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    for (;;) {
        int32_t v;
        asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(flags + i) : "memory");
        if (v - value >= 0) return;
        uint64_t t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        if (t - t0 > timeout_ns) {
            atomicExch(status, STATUS_PEER_TIMEOUT);
            return;
        }
        __nanosleep(256);
    }
}

}  // namespace fmab

extern "C" {

int fma_b200_peer_buffer_create(int64_t bytes, void** ptr_out, uint8_t* handle_out) {
    using namespace fmab;
    static_assert(sizeof(cudaIpcMemHandle_t) == FMA_B200_PEER_HANDLE_BYTES, "handle size");
    FMAB_REQUIRE(bytes > 0 && ptr_out && handle_out, FMA_B200_ERR_BAD_ARG, "bytes=%lld or NULL output", (long long)bytes);
    void* p = nullptr;
    FMAB_CUDA(cudaMalloc(&p, static_cast<size_t>(bytes)));
    cudaError_t e = cudaMemset(p, 0, static_cast<size_t>(bytes));
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
        cudaFree(p);
        cudaGetLastError();
        return fail(FMA_B200_ERR_LAUNCH, "peer buffer of %lld bytes: %s", (long long)bytes, cudaGetErrorString(e));
    }
    memcpy(handle_out, &h, sizeof(h));
    *ptr_out = p;
    return FMA_B200_OK;
}

int fma_b200_peer_buffer_open(const uint8_t* handle, void** ptr_out) {
    using namespace fmab;
    FMAB_REQUIRE(handle && ptr_out, FMA_B200_ERR_BAD_ARG, "NULL argument");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    void* p = nullptr;
    FMAB_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    *ptr_out = p;
    return FMA_B200_OK;
}

int fma_b200_peer_buffer_close(void* ptr) {
    using namespace fmab;
    FMAB_REQUIRE(ptr != nullptr, FMA_B200_ERR_BAD_ARG, "NULL pointer");
    FMAB_CUDA(cudaIpcCloseMemHandle(ptr));
    return FMA_B200_OK;
}

int fma_b200_peer_buffer_destroy(void* ptr) {
    using namespace fmab;
    FMAB_REQUIRE(ptr != nullptr, FMA_B200_ERR_BAD_ARG, "NULL pointer");
    FMAB_CUDA(cudaFree(ptr));
    return FMA_B200_OK;
}

int fma_b200_peer_copy(int32_t n, const uint64_t* dst, const uint64_t* src, const int64_t* bytes, void* stream) {
    using namespace fmab;
    FMAB_REQUIRE(n >= 0, FMA_B200_ERR_BAD_ARG, "n=%d", n);
    if (n == 0) return FMA_B200_OK;
    FMAB_REQUIRE(dst && src && bytes, FMA_B200_ERR_BAD_ARG, "NULL array");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    for (int i = 0; i < n; ++i) {
        FMAB_REQUIRE(bytes[i] >= 0, FMA_B200_ERR_BAD_ARG, "bytes[%d]=%lld", i, (long long)bytes[i]);
        if (bytes[i] == 0) continue;
        FMAB_REQUIRE(dst[i] != 0 && src[i] != 0, FMA_B200_ERR_BAD_ARG, "copy %d has a NULL address", i);
        FMAB_CUDA(cudaMemcpyAsync(reinterpret_cast<void*>(dst[i]), reinterpret_cast<const void*>(src[i]),
                                  static_cast<size_t>(bytes[i]), cudaMemcpyDefault, s));
    }
    return FMA_B200_OK;
}

int fma_b200_peer_signal(int32_t n, const uint64_t* flag_addrs, int32_t value, void* stream) {
    using namespace fmab;
    FMAB_REQUIRE(n >= 1 && n <= kMaxSignals, FMA_B200_ERR_BAD_ARG, "n=%d (1..%d)", n, kMaxSignals);
    FMAB_REQUIRE(flag_addrs != nullptr, FMA_B200_ERR_BAD_ARG, "NULL array");
    SignalArgs args;
    for (int i = 0; i < n; ++i) {
        FMAB_REQUIRE(flag_addrs[i] != 0 && (flag_addrs[i] & 3u) == 0, FMA_B200_ERR_BAD_ARG, "flag %d address", i);
        args.flag[i] = reinterpret_cast<int32_t*>(flag_addrs[i]);
    }
    peer_signal_kernel<<<1, kMaxSignals, 0, static_cast<cudaStream_t>(stream)>>>(args, n, value);
    return check_launch("peer_signal");
}

int fma_b200_peer_wait(const int32_t* flags, int32_t n, int32_t value, int32_t timeout_ms, void* stream) {
    using namespace fmab;
    FMAB_REQUIRE(n >= 1 && n <= 65536, FMA_B200_ERR_BAD_ARG, "n=%d", n);
    FMAB_REQUIRE(flags != nullptr, FMA_B200_ERR_BAD_ARG, "NULL flags");
    FMAB_REQUIRE(timeout_ms >= 1 && timeout_ms <= 60000, FMA_B200_ERR_BAD_ARG, "timeout_ms=%d (1..60000)", timeout_ms);
    int32_t* status = device_status_ptr();
    FMAB_REQUIRE(status != nullptr, FMA_B200_ERR_LAUNCH, "no address for the device status word");
    const int threads = 128;
    peer_wait_kernel<<<(n + threads - 1) / threads, threads, 0, static_cast<cudaStream_t>(stream)>>>(
        flags, n, value, static_cast<uint64_t>(timeout_ms) * 1000000ull, status);
    return check_launch("peer_wait");
}

}  // extern "C"
