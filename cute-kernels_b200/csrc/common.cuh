// Shared host/device helpers for the sm_100a MoE kernels: status reporting, 128-bit
// global accesses, dtype conversion and launch-size helpers.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/fma_b200.h"

namespace fmab {

// ---- host-side error reporting -------------------------------------------
// Thread-local text of the last failure; read through fma_b200_last_error().
char* last_error_buffer();
int fail(int status, const char* fmt, ...);

#define FMAB_REQUIRE(cond, status, ...)            \
    do {                                           \
        if (!(cond)) return ::fmab::fail((status), __VA_ARGS__); \
    } while (0)

#define FMAB_CUDA(expr)                                                                      \
    do {                                                                                     \
        cudaError_t _e = (expr);                                                             \
        if (_e != cudaSuccess)                                                               \
            return ::fmab::fail(FMA_B200_ERR_LAUNCH, "%s: %s", #expr, cudaGetErrorString(_e)); \
    } while (0)

// Launch errors are collected without clearing sticky state of other libraries' calls.
inline int check_launch(const char* what) {
    cudaError_t e = cudaPeekAtLastError();
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(FMA_B200_ERR_LAUNCH, "%s: %s", what, cudaGetErrorString(e));
    }
    return FMA_B200_OK;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// SMs that persistent kernels may occupy: the device's SM count, or the limit set with
// fma_b200_set_sm_limit when that is lower.
int sm_count();
int sm_count_physical();
void set_sm_limit(int n);

// Ordinal of the current device, or -1.  Used to key per-device caches (function attributes such as the
// dynamic shared-memory opt-in apply to the current device only).
inline int current_device_slot() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -1;
    return dev;
}

// Device status word shared by all kernels of this library (see fma_b200_device_status).
int32_t* device_status_ptr();

// ---- device helpers --------------------------------------------------------
__device__ __forceinline__ uint4 ld_global_16(const void* p) {
    return *reinterpret_cast<const uint4*>(p);
}
// Streaming 128-bit load for data read once (keeps it out of L1).
__device__ __forceinline__ uint4 ld_stream_16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ void st_global_16(void* p, uint4 v) { *reinterpret_cast<uint4*>(p) = v; }

__device__ __forceinline__ float bf16_lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// sigmoid with the input clamp the reference applies (fma/include/activations.h:14-22).
__device__ __forceinline__ float sigmoid_clamped(float x) {
    x = fminf(fmaxf(x, -88.3762626647949f), 88.3762626647949f);
    return 1.0f / (1.0f + expf(-x));
}

// Same with fast intrinsics, for results that are rounded to bf16 right away (GEMM epilogues).
__device__ __forceinline__ float sigmoid_clamped_fast(float x) {
    x = fminf(fmaxf(x, -88.3762626647949f), 88.3762626647949f);
    return __fdividef(1.0f, 1.0f + __expf(-x));
}

template <typename T>
struct Elem;
template <>
struct Elem<float> {
    static constexpr int kPerVec = 4;  // elements per 16 bytes
    __device__ static __forceinline__ void unpack(const uint4& v, float* f) {
        f[0] = __uint_as_float(v.x);
        f[1] = __uint_as_float(v.y);
        f[2] = __uint_as_float(v.z);
        f[3] = __uint_as_float(v.w);
    }
    __device__ static __forceinline__ uint4 pack(const float* f) {
        return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
    }
    __device__ static __forceinline__ float round(float x) { return x; }
};
template <>
struct Elem<__nv_bfloat16> {
    static constexpr int kPerVec = 8;
    __device__ static __forceinline__ void unpack(const uint4& v, float* f) {
        f[0] = bf16_lo(v.x); f[1] = bf16_hi(v.x);
        f[2] = bf16_lo(v.y); f[3] = bf16_hi(v.y);
        f[4] = bf16_lo(v.z); f[5] = bf16_hi(v.z);
        f[6] = bf16_lo(v.w); f[7] = bf16_hi(v.w);
    }
    __device__ static __forceinline__ uint4 pack(const float* f) {
        return make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
    }
    __device__ static __forceinline__ float round(float x) { return round_bf16(x); }
};

template <>
struct Elem<__half> {
    static constexpr int kPerVec = 8;
    __device__ static __forceinline__ void unpack(const uint4& v, float* f) {
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 p = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
            f[2 * i] = p.x;
            f[2 * i + 1] = p.y;
        }
    }
    __device__ static __forceinline__ uint4 pack(const float* f) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __half2 h = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
            w[i] = *reinterpret_cast<const uint32_t*>(&h);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
    __device__ static __forceinline__ float round(float x) { return __half2float(__float2half_rn(x)); }
};

// float <-> one element of the three supported types
template <typename T>
__device__ __forceinline__ float elem_to_float(T v);
template <>
__device__ __forceinline__ float elem_to_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float elem_to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float elem_to_float<__half>(__half v) { return __half2float(v); }
template <typename T>
__device__ __forceinline__ T float_to_elem(float v);
template <>
__device__ __forceinline__ float float_to_elem<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 float_to_elem<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ __half float_to_elem<__half>(float v) { return __float2half_rn(v); }

// Runs `body` (a generic lambda taking a value of the element type) for a dtype code; false for an unknown code.
template <typename F>
inline bool dispatch_dtype(int32_t dtype, F&& body) {
    if (dtype == FMA_B200_F32) body(float{});
    else if (dtype == FMA_B200_BF16) body(__nv_bfloat16{});
    else if (dtype == FMA_B200_F16) body(__half{});
    else return false;
    return true;
}
inline bool known_dtype(int32_t dtype) { return dtype == FMA_B200_F32 || dtype == FMA_B200_BF16 || dtype == FMA_B200_F16; }
inline int elems_per_16_bytes(int32_t dtype) { return dtype == FMA_B200_F32 ? 4 : 8; }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

}  // namespace fmab
