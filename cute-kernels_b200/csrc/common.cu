// Status reporting and per-device caches shared by every entry point.
#include <stdarg.h>
#include <string.h>

#include "common.cuh"

namespace fmab {

static thread_local char g_last_error[512] = {0};

// Written by kernels whose bounded waits run out; file scope so that no allocation is needed.
__device__ int32_t g_device_status = 0;

char* last_error_buffer() { return g_last_error; }

int fail(int status, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
    va_end(ap);
    return status;
}

static int g_sm_limit = 0;  // 0 = use every SM

void set_sm_limit(int n) { g_sm_limit = n < 0 ? 0 : n; }

int sm_count() {
    const int all = sm_count_physical();
    return (g_sm_limit > 0 && g_sm_limit < all) ? g_sm_limit : all;
}

int sm_count_physical() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

int32_t* device_status_ptr() {
    static int32_t* cached[64] = {nullptr};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (cached[dev] == nullptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_device_status) != cudaSuccess) return nullptr;
        cached[dev] = static_cast<int32_t*>(p);
    }
    return cached[dev];
}

}  // namespace fmab

extern "C" {

const char* fma_b200_status_string(int status) {
    switch (status) {
        case FMA_B200_OK: return "ok";
        case FMA_B200_ERR_BAD_ARG: return "bad argument";
        case FMA_B200_ERR_UNSUPPORTED: return "unsupported dtype or layout";
        case FMA_B200_ERR_LAUNCH: return "CUDA launch or copy failed";
        case FMA_B200_ERR_WORKSPACE: return "workspace too small";
        case FMA_B200_ERR_DEVICE: return "a kernel reported a device-side error";
        default: return "unknown status";
    }
}

const char* fma_b200_last_error(void) { return fmab::last_error_buffer(); }

int fma_b200_abi_version(void) { return 3; }

int fma_b200_set_sm_limit(int32_t sms) {
    fmab::set_sm_limit(sms);
    return FMA_B200_OK;
}

int fma_b200_device_status(int32_t* status_out, void* stream) {
    FMAB_REQUIRE(status_out != nullptr, FMA_B200_ERR_BAD_ARG, "status_out is NULL");
    int32_t* dptr = fmab::device_status_ptr();
    FMAB_REQUIRE(dptr != nullptr, FMA_B200_ERR_LAUNCH, "no address for the device status word");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    FMAB_CUDA(cudaMemcpyAsync(status_out, dptr, sizeof(int32_t), cudaMemcpyDeviceToHost, s));
    FMAB_CUDA(cudaMemsetAsync(dptr, 0, sizeof(int32_t), s));
    FMAB_CUDA(cudaStreamSynchronize(s));
    return FMA_B200_OK;
}

int fma_b200_device_status_peek(int32_t* device_out, void* stream) {
    FMAB_REQUIRE(device_out != nullptr, FMA_B200_ERR_BAD_ARG, "device_out is NULL");
    int32_t* dptr = fmab::device_status_ptr();
    FMAB_REQUIRE(dptr != nullptr, FMA_B200_ERR_LAUNCH, "no address for the device status word");
    FMAB_CUDA(cudaMemcpyAsync(device_out, dptr, sizeof(int32_t), cudaMemcpyDeviceToDevice,
                              static_cast<cudaStream_t>(stream)));
    return FMA_B200_OK;
}

}  // extern "C"
