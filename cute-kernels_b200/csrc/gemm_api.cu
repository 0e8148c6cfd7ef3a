// C-ABI entry points of the grouped GEMMs: argument checks and dtype dispatch
// (bf16 -> tcgen05 kernel, f32 -> FFMA kernel).
#include <stdlib.h>

#include "common.cuh"

namespace fmab {
int tc_forward(const void* X, const void* W, void* Y, int64_t rows_cap, int E, int OUT, int IN,
               const int32_t* mtile_expert, bool f16, cudaStream_t s);
int tc_forward_swiglu(const void* X, const void* W, void* pre, void* act, int64_t rows_cap, int E, int I, int IN,
                      const int32_t* mtile_expert, bool f16, cudaStream_t s);
int tc_dgrad(const void* dY, const void* W, void* dX, const void* pre, int64_t rows_cap, int E, int OUT, int IN,
             const int32_t* mtile_expert, bool swiglu, bool f16, cudaStream_t s);
int tc_wgrad(const void* dY, const void* X, void* dW, int64_t rows_cap, int E, int OUT, int IN,
             const int32_t* seg_offsets, int n_seg, bool f16, cudaStream_t s);
int tc_general(const void* A, const void* B, void* D, const uint32_t* M, const uint32_t* N, const uint32_t* K,
               int n_groups, bool a_t, bool b_t, void* workspace, int64_t workspace_bytes, cudaStream_t s);
int64_t tc_general_workspace_bytes(int n_groups, int64_t total_mtiles);
int tc2_forward(const void* X, const void* W, void* Y, int64_t rows_cap, int E, int OUT, int IN,
                const int32_t* mtile_expert, bool f16, cudaStream_t s);
int tc2_forward_swiglu(const void* X, const void* W, void* pre, void* act, int64_t rows_cap, int E, int I, int IN,
                       const int32_t* mtile_expert, bool f16, cudaStream_t s);
int tc2_dgrad(const void* dY, const void* W, void* dX, const void* pre, int64_t rows_cap, int E, int OUT, int IN,
              const int32_t* mtile_expert, bool swiglu, bool f16, cudaStream_t s);
int tc2_wgrad(const void* dY, const void* X, void* dW, int64_t rows_cap, int E, int OUT, int IN,
              const int32_t* seg_offsets, int n_seg, bool f16, cudaStream_t s);
int tc2_forward_peer(const void* X, const void* W, const uint64_t* dst_table, int64_t rows_cap, int E, int OUT, int IN,
                     const int32_t* mtile_expert, bool f16, cudaStream_t s);
int tc2_dgrad_peer(const void* dY, const void* W, const uint64_t* dst_table, int64_t rows_cap, int E, int OUT, int IN,
                   const int32_t* mtile_expert, bool f16, cudaStream_t s);
int simt_forward(const void* X, const void* W, void* Y, int64_t rows_cap, int E, int OUT, int IN,
                 const int32_t* mtile_expert, cudaStream_t s);
int simt_dgrad(const void* dY, const void* W, void* dX, int64_t rows_cap, int E, int OUT, int IN,
               const int32_t* mtile_expert, cudaStream_t s);
int simt_wgrad(const void* dY, const void* X, void* dW, int64_t rows_cap, int E, int OUT, int IN,
               const int32_t* seg_offsets, int n_seg, cudaStream_t s);

// CTA-pair kernels (cta_group::2) are used when the grouped rows are aligned to 256.  Measurement knob
// FMA_B200_GEMM_PAIRS: 0 forces the single-CTA kernels everywhere, 1 keeps the two SwiGLU-epilogue GEMMs on
// the single-CTA kernel (its two accumulators belong to different tiles, so a long epilogue overlaps the next
// main loop), anything else (the default) runs all five layer GEMMs on pairs.
static int pairs_mode() {
    static int mode = -1;
    if (mode < 0) {
        const char* env = getenv("FMA_B200_GEMM_PAIRS");
        mode = (env == nullptr) ? 2 : atoi(env);
        if (mode < 0 || mode > 2) mode = 2;
    }
    return mode;
}
static bool use_pairs(int32_t row_align) { return pairs_mode() >= 1 && row_align > 0 && row_align % 256 == 0; }

static bool pairs_for_fused_epilogues() { return pairs_mode() == 2; }

static int check_layer_gemm(int32_t dtype, int64_t rows_cap, int32_t E, int32_t OUT, int32_t IN) {
    FMAB_REQUIRE(known_dtype(dtype), FMA_B200_ERR_UNSUPPORTED, "dtype %d", dtype);
    FMAB_REQUIRE(rows_cap >= 0 && rows_cap % 128 == 0 && rows_cap < (1LL << 31), FMA_B200_ERR_BAD_ARG,
                 "rows_cap=%lld must be a multiple of 128 below 2^31", (long long)rows_cap);
    FMAB_REQUIRE(E >= 1 && E <= 1024, FMA_B200_ERR_BAD_ARG, "E=%d not in [1,1024]", E);
    FMAB_REQUIRE(OUT >= 8 && IN >= 8 && OUT % 8 == 0 && IN % 8 == 0, FMA_B200_ERR_BAD_ARG,
                 "OUT=%d and IN=%d must be positive multiples of 8", OUT, IN);
    FMAB_REQUIRE(static_cast<int64_t>(E) * OUT < (1LL << 31), FMA_B200_ERR_BAD_ARG, "E*OUT overflows");
    return FMA_B200_OK;
}
}  // namespace fmab

extern "C" {

int fma_b200_moe_gemm_forward(const void* X, const void* W, void* Y, int32_t dtype, int64_t rows_cap, int32_t E,
                              int32_t OUT, int32_t IN, const int32_t* mtile_expert, int32_t row_align, void* stream) {
    using namespace fmab;
    if (int rc = check_layer_gemm(dtype, rows_cap, E, OUT, IN)) return rc;
    if (rows_cap == 0) return FMA_B200_OK;
    FMAB_REQUIRE(X && W && Y && mtile_expert, FMA_B200_ERR_BAD_ARG, "NULL pointer");
    FMAB_REQUIRE(aligned16(X) && aligned16(W) && aligned16(Y), FMA_B200_ERR_BAD_ARG, "pointers not 16-byte aligned");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool f16 = dtype == FMA_B200_F16;
    if (dtype != FMA_B200_F32 && use_pairs(row_align))
        return tc2_forward(X, W, Y, rows_cap, E, OUT, IN, mtile_expert, f16, s);
    if (dtype != FMA_B200_F32) return tc_forward(X, W, Y, rows_cap, E, OUT, IN, mtile_expert, f16, s);
    return simt_forward(X, W, Y, rows_cap, E, OUT, IN, mtile_expert, s);
}

int fma_b200_moe_gemm_dgrad(const void* dY, const void* W, void* dX, int32_t dtype, int64_t rows_cap, int32_t E,
                            int32_t OUT, int32_t IN, const int32_t* mtile_expert, int32_t row_align, void* stream) {
    using namespace fmab;
    if (int rc = check_layer_gemm(dtype, rows_cap, E, OUT, IN)) return rc;
    if (rows_cap == 0) return FMA_B200_OK;
    FMAB_REQUIRE(dY && W && dX && mtile_expert, FMA_B200_ERR_BAD_ARG, "NULL pointer");
    FMAB_REQUIRE(aligned16(dY) && aligned16(W) && aligned16(dX), FMA_B200_ERR_BAD_ARG, "pointers not 16-byte aligned");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool f16 = dtype == FMA_B200_F16;
    if (dtype != FMA_B200_F32 && use_pairs(row_align))
        return tc2_dgrad(dY, W, dX, nullptr, rows_cap, E, OUT, IN, mtile_expert, false, f16, s);
    if (dtype != FMA_B200_F32) return tc_dgrad(dY, W, dX, nullptr, rows_cap, E, OUT, IN, mtile_expert, false, f16, s);
    return simt_dgrad(dY, W, dX, rows_cap, E, OUT, IN, mtile_expert, s);
}

int fma_b200_moe_gemm_wgrad(const void* dY, const void* X, void* dW, int32_t dtype, int64_t rows_cap, int32_t E,
                            int32_t OUT, int32_t IN, const int32_t* seg_offsets, int32_t n_seg, void* stream) {
    using namespace fmab;
    if (int rc = check_layer_gemm(dtype, rows_cap, E, OUT, IN)) return rc;
    FMAB_REQUIRE(dW && seg_offsets, FMA_B200_ERR_BAD_ARG, "NULL pointer");
    FMAB_REQUIRE(n_seg >= 1 && n_seg <= 64, FMA_B200_ERR_BAD_ARG, "n_seg=%d not in [1,64]", n_seg);
    FMAB_REQUIRE(rows_cap > 0 && dY && X, FMA_B200_ERR_BAD_ARG, "wgrad needs non-empty dY and X buffers");
    FMAB_REQUIRE(aligned16(dY) && aligned16(X) && aligned16(dW), FMA_B200_ERR_BAD_ARG, "pointers not 16-byte aligned");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool f16 = dtype == FMA_B200_F16;
    if (dtype != FMA_B200_F32 && use_pairs(256)) return tc2_wgrad(dY, X, dW, rows_cap, E, OUT, IN, seg_offsets, n_seg, f16, s);
    if (dtype != FMA_B200_F32) return tc_wgrad(dY, X, dW, rows_cap, E, OUT, IN, seg_offsets, n_seg, f16, s);
    return simt_wgrad(dY, X, dW, rows_cap, E, OUT, IN, seg_offsets, n_seg, s);
}

int fma_b200_moe_gemm_forward_swiglu(const void* X, const void* W, void* pre, void* act, int32_t dtype,
                                     int64_t rows_cap, int32_t E, int32_t I, int32_t IN, const int32_t* mtile_expert,
                                     int32_t row_align, void* stream) {
    using namespace fmab;
    FMAB_REQUIRE(dtype == FMA_B200_BF16 || dtype == FMA_B200_F16, FMA_B200_ERR_UNSUPPORTED,
                 "the SwiGLU-fused up projection exists for the 16-bit types only; run forward + swiglu_forward for f32");
    const bool f16 = dtype == FMA_B200_F16;
    FMAB_REQUIRE(I >= 8 && I % 8 == 0 && I < (1 << 29), FMA_B200_ERR_BAD_ARG, "I=%d must be a positive multiple of 8", I);
    if (int rc = check_layer_gemm(dtype, rows_cap, E, 2 * I, IN)) return rc;
    if (rows_cap == 0) return FMA_B200_OK;
    FMAB_REQUIRE(X && W && act && mtile_expert, FMA_B200_ERR_BAD_ARG, "NULL pointer");
    FMAB_REQUIRE(aligned16(X) && aligned16(W) && aligned16(act) && aligned16(pre), FMA_B200_ERR_BAD_ARG,
                 "pointers not 16-byte aligned");
    if (use_pairs(row_align) && pairs_for_fused_epilogues())
        return tc2_forward_swiglu(X, W, pre, act, rows_cap, E, I, IN, mtile_expert, f16,
                                  static_cast<cudaStream_t>(stream));
    return tc_forward_swiglu(X, W, pre, act, rows_cap, E, I, IN, mtile_expert, f16, static_cast<cudaStream_t>(stream));
}

int fma_b200_moe_gemm_dgrad_swiglu(const void* dY, const void* W, const void* pre, void* d_pre, int32_t dtype,
                                   int64_t rows_cap, int32_t E, int32_t OUT, int32_t I, const int32_t* mtile_expert,
                                   int32_t row_align, void* stream) {
    using namespace fmab;
    FMAB_REQUIRE(dtype == FMA_B200_BF16 || dtype == FMA_B200_F16, FMA_B200_ERR_UNSUPPORTED,
                 "the SwiGLU-fused dgrad exists for the 16-bit types only; run dgrad + swiglu_backward for f32");
    const bool f16 = dtype == FMA_B200_F16;
    if (int rc = check_layer_gemm(dtype, rows_cap, E, OUT, I)) return rc;
    if (rows_cap == 0) return FMA_B200_OK;
    FMAB_REQUIRE(dY && W && pre && d_pre && mtile_expert, FMA_B200_ERR_BAD_ARG, "NULL pointer");
    FMAB_REQUIRE(aligned16(dY) && aligned16(W) && aligned16(pre) && aligned16(d_pre), FMA_B200_ERR_BAD_ARG,
                 "pointers not 16-byte aligned");
    if (use_pairs(row_align) && pairs_for_fused_epilogues())
        return tc2_dgrad(dY, W, d_pre, pre, rows_cap, E, OUT, I, mtile_expert, true, f16,
                         static_cast<cudaStream_t>(stream));
    return tc_dgrad(dY, W, d_pre, pre, rows_cap, E, OUT, I, mtile_expert, true, f16, static_cast<cudaStream_t>(stream));
}

static int check_peer_gemm(int32_t dtype, int64_t rows_cap, int32_t E, int32_t OUT, int32_t IN, int32_t row_align) {
    using namespace fmab;
    FMAB_REQUIRE(dtype == FMA_B200_BF16 || dtype == FMA_B200_F16, FMA_B200_ERR_UNSUPPORTED,
                 "the peer-store GEMMs exist for the 16-bit types only");
    FMAB_REQUIRE(row_align > 0 && row_align % 256 == 0, FMA_B200_ERR_UNSUPPORTED,
                 "the peer-store GEMMs run on CTA pairs: row_align=%d must be a multiple of 256", row_align);
    return check_layer_gemm(dtype, rows_cap, E, OUT, IN);
}

int fma_b200_moe_gemm_forward_peer(const void* X, const void* W, const uint64_t* dst_table, int32_t dtype,
                                   int64_t rows_cap, int32_t E, int32_t OUT, int32_t IN, const int32_t* mtile_expert,
                                   int32_t row_align, void* stream) {
    using namespace fmab;
    if (int rc = check_peer_gemm(dtype, rows_cap, E, OUT, IN, row_align)) return rc;
    if (rows_cap == 0) return FMA_B200_OK;
    FMAB_REQUIRE(X && W && dst_table && mtile_expert, FMA_B200_ERR_BAD_ARG, "NULL pointer");
    FMAB_REQUIRE(aligned16(X) && aligned16(W), FMA_B200_ERR_BAD_ARG, "pointers not 16-byte aligned");
    return tc2_forward_peer(X, W, dst_table, rows_cap, E, OUT, IN, mtile_expert, dtype == FMA_B200_F16,
                            static_cast<cudaStream_t>(stream));
}

int fma_b200_moe_gemm_dgrad_peer(const void* dY, const void* W, const uint64_t* dst_table, int32_t dtype,
                                 int64_t rows_cap, int32_t E, int32_t OUT, int32_t IN, const int32_t* mtile_expert,
                                 int32_t row_align, void* stream) {
    using namespace fmab;
    if (int rc = check_peer_gemm(dtype, rows_cap, E, OUT, IN, row_align)) return rc;
    if (rows_cap == 0) return FMA_B200_OK;
    FMAB_REQUIRE(dY && W && dst_table && mtile_expert, FMA_B200_ERR_BAD_ARG, "NULL pointer");
    FMAB_REQUIRE(aligned16(dY) && aligned16(W), FMA_B200_ERR_BAD_ARG, "pointers not 16-byte aligned");
    return tc2_dgrad_peer(dY, W, dst_table, rows_cap, E, OUT, IN, mtile_expert, dtype == FMA_B200_F16,
                          static_cast<cudaStream_t>(stream));
}

int64_t fma_b200_grouped_gemm_workspace_bytes(int32_t n_groups, int64_t total_mtiles) {
    if (n_groups < 0 || total_mtiles < 0) return 0;
    return fmab::tc_general_workspace_bytes(n_groups, total_mtiles);
}

int fma_b200_grouped_gemm(const void* A, const void* B, void* D, const uint32_t* M, const uint32_t* N,
                          const uint32_t* K, int32_t n_groups, int32_t a_transposed, int32_t b_transposed,
                          void* workspace, int64_t workspace_bytes, void* stream) {
    using namespace fmab;
    FMAB_REQUIRE(n_groups >= 0 && n_groups <= 1024, FMA_B200_ERR_BAD_ARG, "n_groups=%d not in [0,1024]", n_groups);
    if (n_groups == 0) return FMA_B200_OK;
    FMAB_REQUIRE(M && N && K && workspace, FMA_B200_ERR_BAD_ARG, "NULL pointer");
    FMAB_REQUIRE(A && B && D, FMA_B200_ERR_BAD_ARG, "NULL operand");
    FMAB_REQUIRE(aligned16(A) && aligned16(B) && aligned16(D), FMA_B200_ERR_BAD_ARG, "operands not 16-byte aligned");
    return tc_general(A, B, D, M, N, K, n_groups, a_transposed != 0, b_transposed != 0, workspace, workspace_bytes,
                      static_cast<cudaStream_t>(stream));
}

}  // extern "C"
