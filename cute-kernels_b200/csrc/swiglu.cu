// Stand-alone SwiGLU forward / backward (the op surface; inside the MoE layer the same math
// runs in the grouped-GEMM epilogues).  Elementwise, HBM-bound, 128-bit accesses, fp32 math.
#include "common.cuh"

namespace fmab {

constexpr int kSwigluThreads = 256;

template <typename T>
__global__ void __launch_bounds__(kSwigluThreads)
swiglu_forward_kernel(const T* __restrict__ gate, int64_t gate_pitch, const T* __restrict__ up, int64_t up_pitch,
                      T* __restrict__ out, int64_t out_pitch, int64_t rows, int64_t vec_per_row) {
    constexpr int V = Elem<T>::kPerVec;
    const int64_t total = rows * vec_per_row;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * kSwigluThreads + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * kSwigluThreads) {
        const int64_t r = i / vec_per_row, c = (i - r * vec_per_row) * V;
        float g[V], u[V], y[V];
        Elem<T>::unpack(ld_stream_16(gate + r * gate_pitch + c), g);
        Elem<T>::unpack(ld_stream_16(up + r * up_pitch + c), u);
#pragma unroll
        for (int j = 0; j < V; ++j) y[j] = u[j] * g[j] * sigmoid_clamped(g[j]);
        st_global_16(out + r * out_pitch + c, Elem<T>::pack(y));
    }
}

template <typename T>
__global__ void __launch_bounds__(kSwigluThreads)
swiglu_backward_kernel(const T* __restrict__ gate, int64_t gate_pitch, const T* __restrict__ up, int64_t up_pitch,
                       const T* __restrict__ dy, int64_t dy_pitch, T* __restrict__ gate_grad, int64_t gate_grad_pitch,
                       T* __restrict__ up_grad, int64_t up_grad_pitch, int64_t rows, int64_t vec_per_row) {
    constexpr int V = Elem<T>::kPerVec;
    const int64_t total = rows * vec_per_row;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * kSwigluThreads + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * kSwigluThreads) {
        const int64_t r = i / vec_per_row, c = (i - r * vec_per_row) * V;
        float g[V], u[V], d[V], dg[V], du[V];
        Elem<T>::unpack(ld_stream_16(gate + r * gate_pitch + c), g);
        Elem<T>::unpack(ld_stream_16(up + r * up_pitch + c), u);
        Elem<T>::unpack(ld_stream_16(dy + r * dy_pitch + c), d);
#pragma unroll
        for (int j = 0; j < V; ++j) {
            const float s = sigmoid_clamped(g[j]);
            const float silu = g[j] * s;
            dg[j] = d[j] * u[j] * (s + silu * (1.f - s));
            du[j] = d[j] * silu;
        }
        st_global_16(gate_grad + r * gate_grad_pitch + c, Elem<T>::pack(dg));
        st_global_16(up_grad + r * up_grad_pitch + c, Elem<T>::pack(du));
    }
}

static int swiglu_grid(int64_t total_vec) {
    int64_t want = (total_vec + kSwigluThreads - 1) / kSwigluThreads;
    const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
    return static_cast<int>(want < 1 ? 1 : (want > cap ? cap : want));
}

static int check_swiglu(int32_t dtype, int64_t rows, int64_t cols, const int64_t* pitches, int n_pitch,
                        const void* const* ptrs, int n_ptr) {
    FMAB_REQUIRE(known_dtype(dtype), FMA_B200_ERR_UNSUPPORTED, "dtype %d", dtype);
    FMAB_REQUIRE(rows >= 0 && cols >= 0, FMA_B200_ERR_BAD_ARG, "rows=%lld cols=%lld", (long long)rows, (long long)cols);
    const int per_vec = elems_per_16_bytes(dtype);
    FMAB_REQUIRE(cols % per_vec == 0, FMA_B200_ERR_BAD_ARG, "cols=%lld is not a multiple of 16 bytes", (long long)cols);
    for (int i = 0; i < n_pitch; ++i)
        FMAB_REQUIRE(pitches[i] >= cols && pitches[i] % per_vec == 0, FMA_B200_ERR_BAD_ARG, "pitch %d = %lld invalid", i,
                     (long long)pitches[i]);
    if (rows * cols == 0) return FMA_B200_OK;
    for (int i = 0; i < n_ptr; ++i)
        FMAB_REQUIRE(ptrs[i] != nullptr && aligned16(ptrs[i]), FMA_B200_ERR_BAD_ARG, "pointer %d NULL or not 16-byte aligned", i);
    return FMA_B200_OK;
}

}  // namespace fmab

extern "C" {

int fma_b200_swiglu_forward(const void* gate, int64_t gate_pitch, const void* up, int64_t up_pitch, void* out,
                            int64_t out_pitch, int32_t dtype, int64_t rows, int64_t cols, void* stream) {
    using namespace fmab;
    const int64_t pitches[3] = {gate_pitch, up_pitch, out_pitch};
    const void* ptrs[3] = {gate, up, out};
    if (int rc = check_swiglu(dtype, rows, cols, pitches, 3, ptrs, 3)) return rc;
    if (rows * cols == 0) return FMA_B200_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int64_t vpr = cols / elems_per_16_bytes(dtype);
    dispatch_dtype(dtype, [&](auto tag) {
        using Elt = decltype(tag);
        swiglu_forward_kernel<Elt><<<swiglu_grid(rows * vpr), kSwigluThreads, 0, s>>>(
            static_cast<const Elt*>(gate), gate_pitch, static_cast<const Elt*>(up), up_pitch, static_cast<Elt*>(out),
            out_pitch, rows, vpr);
    });
    return check_launch("swiglu_forward");
}

int fma_b200_swiglu_backward(const void* gate, int64_t gate_pitch, const void* up, int64_t up_pitch, const void* dy,
                             int64_t dy_pitch, void* gate_grad, int64_t gate_grad_pitch, void* up_grad,
                             int64_t up_grad_pitch, int32_t dtype, int64_t rows, int64_t cols, void* stream) {
    using namespace fmab;
    const int64_t pitches[5] = {gate_pitch, up_pitch, dy_pitch, gate_grad_pitch, up_grad_pitch};
    const void* ptrs[5] = {gate, up, dy, gate_grad, up_grad};
    if (int rc = check_swiglu(dtype, rows, cols, pitches, 5, ptrs, 5)) return rc;
    if (rows * cols == 0) return FMA_B200_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int64_t vpr = cols / elems_per_16_bytes(dtype);
    dispatch_dtype(dtype, [&](auto tag) {
        using Elt = decltype(tag);
        swiglu_backward_kernel<Elt><<<swiglu_grid(rows * vpr), kSwigluThreads, 0, s>>>(
            static_cast<const Elt*>(gate), gate_pitch, static_cast<const Elt*>(up), up_pitch, static_cast<const Elt*>(dy),
            dy_pitch, static_cast<Elt*>(gate_grad), gate_grad_pitch, static_cast<Elt*>(up_grad), up_grad_pitch, rows, vpr);
    });
    return check_launch("swiglu_backward");
}

}  // extern "C"
