// fp32 grouped GEMM on the FFMA pipe, for the layer's fp32 mode (results within 1e-5 of an fp32
// reference, which TF32 tensor-core products cannot give).  Same grouped layout and the same
// three products as the tensor-core kernel:
//   forward  Y[p,:]  = X[p,:] . W[e]^T     dgrad  dX[p,:] = dY[p,:] . W[e]     wgrad  dW[e] = dY_e^T . X_e
// 128x128 output tile per 256-thread block, 8x8 outputs per thread, k-blocks of 16 staged through
// shared memory with 128-bit global loads along whichever index is contiguous.
#include "common.cuh"

namespace fmab {

constexpr int SBM = 128, SBN = 128, SBK = 16;
constexpr int SIMT_THREADS = 256;

struct SimtParams {
    const float* a;
    const float* b;
    float* d;
    const int32_t* mtile_expert;  // rows mode
    const int32_t* seg_offsets;   // wgrad mode
    int64_t lda, ldb, ldd;        // row pitches in elements
    int32_t mode;                 // 0 forward, 1 dgrad, 2 wgrad
    int32_t n_cols;               // D columns
    int32_t k_len;                // forward/dgrad reduction length
    int32_t m_per_group;          // wgrad: OUT
    int32_t mtiles_per_group;
    int32_t group_rows;           // rows of W per expert (OUT)
    int32_t n_groups, n_seg;
};

// A element (m, k) and B element (k, n) of the current tile live at
//   a_base + m * a_sm + k * a_sk,   b_base + k * b_sk + n * b_sn
// with exactly one of the two strides of each operand equal to 1.
template <bool A_K_CONTIG, bool B_K_CONTIG>
__global__ void __launch_bounds__(SIMT_THREADS)
gemm_simt_kernel(const SimtParams p) {
    __shared__ __align__(16) float sa[SBK][SBM + 4];
    __shared__ __align__(16) float sb[SBK][SBN + 4];

    const int mt = blockIdx.y, nt = blockIdx.x;
    const int n0 = nt * SBN;
    int group, rows_valid;
    int64_t d_row;
    const float* a_base;
    const float* b_base;
    if (p.mode == 2) {
        group = mt / p.mtiles_per_group;
        const int m0 = (mt - group * p.mtiles_per_group) * SBM;
        rows_valid = min(SBM, p.m_per_group - m0);
        d_row = static_cast<int64_t>(group) * p.m_per_group + m0;
        a_base = p.a + m0;   // A(m,k) = dY[tok0 + k][m0 + m]
        b_base = p.b + n0;   // B(k,n) = X[tok0 + k][n0 + n]
    } else {
        group = p.mtile_expert[mt];
        if (group < 0) return;
        rows_valid = SBM;
        d_row = static_cast<int64_t>(mt) * SBM;
        a_base = p.a + d_row * p.lda;  // A(m,k) = X[row + m][k]
        if (p.mode == 0) b_base = p.b + (static_cast<int64_t>(group) * p.group_rows + n0) * p.ldb;  // B(k,n) = W[e][n0+n][k]
        else b_base = p.b + static_cast<int64_t>(group) * p.group_rows * p.ldb + n0;               // B(k,n) = W[e][k][n0+n]
    }
    const int cols_valid = min(SBN, p.n_cols - n0);

    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;  // 16 x 16 threads, 8x8 outputs each
    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

    const int n_seg = (p.mode == 2) ? p.n_seg : 1;
    for (int s = 0; s < n_seg; ++s) {
        int64_t k_begin = 0;
        int len = p.k_len;
        if (p.mode == 2) {
            const int32_t* o = p.seg_offsets + s * p.n_groups + group;
            k_begin = o[0];
            len = o[1] - o[0];
        }
        for (int k0 = 0; k0 < len; k0 += SBK) {
            // ---- stage A: SBM x SBK ----
#pragma unroll
            for (int it = 0; it < 2; ++it) {
                const int v = threadIdx.x + it * SIMT_THREADS;  // 512 float4 per operand tile
                if (A_K_CONTIG) {
                    const int m = v >> 2, kq = (v & 3) * 4;
                    float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (m < rows_valid && k0 + kq < len)
                        x = *reinterpret_cast<const float4*>(a_base + static_cast<int64_t>(m) * p.lda + k_begin + k0 + kq);
                    sa[kq + 0][m] = x.x; sa[kq + 1][m] = x.y; sa[kq + 2][m] = x.z; sa[kq + 3][m] = x.w;
                } else {
                    const int k = v >> 5, mq = (v & 31) * 4;
                    float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (k0 + k < len && mq < rows_valid)
                        x = *reinterpret_cast<const float4*>(a_base + (k_begin + k0 + k) * p.lda + mq);
                    *reinterpret_cast<float4*>(&sa[k][mq]) = x;
                }
            }
            // ---- stage B: SBK x SBN ----
#pragma unroll
            for (int it = 0; it < 2; ++it) {
                const int v = threadIdx.x + it * SIMT_THREADS;
                if (B_K_CONTIG) {
                    const int n = v >> 2, kq = (v & 3) * 4;
                    float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (n < cols_valid && k0 + kq < len)
                        x = *reinterpret_cast<const float4*>(b_base + static_cast<int64_t>(n) * p.ldb + k_begin + k0 + kq);
                    sb[kq + 0][n] = x.x; sb[kq + 1][n] = x.y; sb[kq + 2][n] = x.z; sb[kq + 3][n] = x.w;
                } else {
                    const int k = v >> 5, nq = (v & 31) * 4;
                    float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (k0 + k < len && nq < cols_valid)
                        x = *reinterpret_cast<const float4*>(b_base + (k_begin + k0 + k) * p.ldb + nq);
                    *reinterpret_cast<float4*>(&sb[k][nq]) = x;
                }
            }
            __syncthreads();
#pragma unroll
            for (int k = 0; k < SBK; ++k) {
                float av[8], bv[8];
                const float4 a0 = *reinterpret_cast<const float4*>(&sa[k][ty * 4]);
                const float4 a1 = *reinterpret_cast<const float4*>(&sa[k][64 + ty * 4]);
                const float4 b0 = *reinterpret_cast<const float4*>(&sb[k][tx * 4]);
                const float4 b1 = *reinterpret_cast<const float4*>(&sb[k][64 + tx * 4]);
                av[0] = a0.x; av[1] = a0.y; av[2] = a0.z; av[3] = a0.w; av[4] = a1.x; av[5] = a1.y; av[6] = a1.z; av[7] = a1.w;
                bv[0] = b0.x; bv[1] = b0.y; bv[2] = b0.z; bv[3] = b0.w; bv[4] = b1.x; bv[5] = b1.y; bv[6] = b1.z; bv[7] = b1.w;
#pragma unroll
                for (int i = 0; i < 8; ++i)
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
            }
            __syncthreads();
        }
    }
    // rows ty*4..+3 and 64+ty*4..+3; columns tx*4..+3 and 64+tx*4..+3
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int m = (i < 4) ? ty * 4 + i : 64 + ty * 4 + (i - 4);
        if (m >= rows_valid) continue;
        float* drow = p.d + (d_row + m) * p.ldd + n0;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int n = h * 64 + tx * 4;
            if (n < cols_valid)
                *reinterpret_cast<float4*>(drow + n) = make_float4(acc[i][h * 4 + 0], acc[i][h * 4 + 1], acc[i][h * 4 + 2], acc[i][h * 4 + 3]);
        }
    }
}

static int launch_simt(const SimtParams& p, int n_mtiles, cudaStream_t s) {
    const int n_ntiles = (p.n_cols + SBN - 1) / SBN;
    if (n_mtiles <= 0 || n_ntiles <= 0) return FMA_B200_OK;
    FMAB_REQUIRE(n_mtiles <= 65535, FMA_B200_ERR_BAD_ARG, "fp32 grouped GEMM: %d row tiles exceed the grid limit", n_mtiles);
    const dim3 grid(n_ntiles, n_mtiles);
    if (p.mode == 0) gemm_simt_kernel<true, true><<<grid, SIMT_THREADS, 0, s>>>(p);
    else if (p.mode == 1) gemm_simt_kernel<true, false><<<grid, SIMT_THREADS, 0, s>>>(p);
    else gemm_simt_kernel<false, false><<<grid, SIMT_THREADS, 0, s>>>(p);
    return check_launch("grouped GEMM (fp32)");
}

int simt_forward(const void* X, const void* W, void* Y, int64_t rows_cap, int E, int OUT, int IN,
                 const int32_t* mtile_expert, cudaStream_t s) {
    SimtParams p = {};
    p.a = static_cast<const float*>(X); p.b = static_cast<const float*>(W); p.d = static_cast<float*>(Y);
    p.mtile_expert = mtile_expert;
    p.lda = IN; p.ldb = IN; p.ldd = OUT;
    p.mode = 0; p.n_cols = OUT; p.k_len = IN; p.group_rows = OUT; p.n_groups = E; p.n_seg = 1;
    return launch_simt(p, static_cast<int>(rows_cap / SBM), s);
}

int simt_dgrad(const void* dY, const void* W, void* dX, int64_t rows_cap, int E, int OUT, int IN,
               const int32_t* mtile_expert, cudaStream_t s) {
    SimtParams p = {};
    p.a = static_cast<const float*>(dY); p.b = static_cast<const float*>(W); p.d = static_cast<float*>(dX);
    p.mtile_expert = mtile_expert;
    p.lda = OUT; p.ldb = IN; p.ldd = IN;
    p.mode = 1; p.n_cols = IN; p.k_len = OUT; p.group_rows = OUT; p.n_groups = E; p.n_seg = 1;
    return launch_simt(p, static_cast<int>(rows_cap / SBM), s);
}

int simt_wgrad(const void* dY, const void* X, void* dW, int64_t rows_cap, int E, int OUT, int IN,
               const int32_t* seg_offsets, int n_seg, cudaStream_t s) {
    (void)rows_cap;
    SimtParams p = {};
    p.a = static_cast<const float*>(dY); p.b = static_cast<const float*>(X); p.d = static_cast<float*>(dW);
    p.seg_offsets = seg_offsets;
    p.lda = OUT; p.ldb = IN; p.ldd = IN;
    p.mode = 2; p.n_cols = IN; p.m_per_group = OUT; p.mtiles_per_group = (OUT + SBM - 1) / SBM;
    p.n_groups = E; p.n_seg = n_seg;
    return launch_simt(p, E * p.mtiles_per_group, s);
}

}  // namespace fmab
