/*
 * fma_b200.h — C ABI of the B200 (sm_100a) MoE-layer kernels.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream handle
 * (passed as void* so that consumers need no CUDA headers) and returns an int
 * status: 0 on success, a FMA_B200_ERR_* code otherwise.  Nothing here throws,
 * aborts or calls exit().  Unless a comment says otherwise an entry point
 * allocates no memory: outputs and workspaces are owned by the caller.
 * All launches are asynchronous on `stream`.
 *
 * Each declaration cites the interface of the reference project
 * (open-lm-engine/cute-kernels, python package `fma`) that it stands in for,
 * as path:line inside that project.
 */
#ifndef FMA_B200_H
#define FMA_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes -------------------------------------------------------- */
#define FMA_B200_OK 0
#define FMA_B200_ERR_BAD_ARG 1     /* null pointer, negative size, misaligned pointer, unsupported shape */
#define FMA_B200_ERR_UNSUPPORTED 2 /* dtype / layout combination with no kernel */
#define FMA_B200_ERR_LAUNCH 3      /* the CUDA runtime refused a launch or a copy */
#define FMA_B200_ERR_WORKSPACE 4   /* workspace too small */
#define FMA_B200_ERR_DEVICE 5      /* a kernel recorded an error in the device status word */

/* ---- element types ------------------------------------------------------- */
#define FMA_B200_F32 0
#define FMA_B200_BF16 1
#define FMA_B200_F16 2 /* IEEE half: the reference's ops are dtype-generic (fma/include/dtypes/fp16.h) */

/* Text for a status code; never NULL. */
const char* fma_b200_status_string(int status);
/* Detail of the last failure on the calling thread (empty string if none). */
const char* fma_b200_last_error(void);
/* ABI version of this header; bumped when a signature changes. */
int fma_b200_abi_version(void);

/*
 * Upper bound on the SMs that the persistent kernels of this library occupy (grid size of the grouped
 * GEMMs); 0 restores "all SMs".  Process-wide.  The expert-parallel layer lowers it while NCCL
 * all-to-all kernels run next to the GEMMs so that the collective always finds free SMs.
 * No reference counterpart.
 */
int fma_b200_set_sm_limit(int32_t sms);

/*
 * Device status word.  Kernels that wait on barriers (the tensor-core grouped GEMM)
 * bound every wait; a wait that runs out records a non-zero code here and the
 * kernel returns after releasing what it holds.  This call copies the word of the
 * current device to *status_out and clears it.  It synchronises `stream`.
 * No reference counterpart (the reference does not check launches:
 * fma/ops/grouped_gemm/cuda_implementation/kernel.cu:327-333).
 */
int fma_b200_device_status(int32_t* status_out, void* stream);
/*
 * The same word without a host synchronisation: copies it (asynchronously, on `stream`) into the int32 at
 * device_out, a DEVICE address, and leaves it as it is.  For callers that already read some device data
 * back once per step and want the status to ride along.  Codes: 0x7001 a grouped-GEMM wait ran out,
 * 0x7002 a peer_wait ran out, 0x7003 the expert sort met an id outside [0,E).  No reference counterpart.
 */
int fma_b200_device_status_peek(int32_t* device_out, void* stream);

/* ======================================================================= */
/* continuous_count                                                         */
/* ======================================================================= */
/*
 * Histogram of ids in [0, size): out[v] = #{i : ids[i] == v}; ids outside the
 * range are ignored.  Replaces continuous_count_cuda
 * (fma/ops/continuous_count/cuda_implementation/forward.cu:115-167, called from
 * fma/ops/continuous_count/__init__.py:38-39).
 *   ids        int32 (id_bytes == 4) or int64 (id_bytes == 8), n elements, 16-byte aligned
 *   out        uint32[size], fully overwritten
 *   workspace  fma_b200_continuous_count_workspace_bytes(size) bytes (128 + 32*size), 16-byte
 *              aligned: a ticket and eight copies of an accumulator.  It must be zero-filled before the first
 *              call; every call leaves it zero-filled again, so one workspace can serve all
 *              later calls that do not overlap on the device.
 * size <= 16384, n < 2^40.
 */
int64_t fma_b200_continuous_count_workspace_bytes(int32_t size);
int fma_b200_continuous_count(const void* ids, int32_t id_bytes, int64_t n, int32_t size,
                              uint32_t* out, void* workspace, int64_t workspace_bytes, void* stream);
/*
 * Same, with the shared-memory scheme chosen by the caller (for measurement):
 * variant 0 = one sub-histogram per lane updated with shared-memory atomics (the default),
 * variant 1 = one histogram per block with warp-aggregated (match.any) atomics,
 * variant 2 = a private column per lane of every warp, plain load/add/store (size <= 1024).
 * fma_b200_continuous_count uses variant 0, the fastest measured on B200.
 */
int fma_b200_continuous_count_variant(const void* ids, int32_t id_bytes, int64_t n, int32_t size, uint32_t* out,
                                      void* workspace, int64_t workspace_bytes, int32_t variant, void* stream);

/*
 * continuous_count for callers that cannot allocate device memory (no counterpart in the
 * reference, which allocates its outputs and scratch through torch).  Think of a plugin running
 * inside a host process whose GPU memory pool belongs to that host, of code on a path where
 * cudaMalloc's implicit device synchronisation is not acceptable, or of a plain C program that
 * links this library without an allocator of its own.  The ticket and the accumulators live in a
 * 32 KiB + 128 B array that is part of the library image (every GPU that loads the library holds it until
 * the process exits); the caller passes only ids and out.
 *   - size <= 1024; larger sizes are refused with FMA_B200_ERR_BAD_ARG (use the workspace form).
 *   - Calls no cudaMalloc / cudaFree or any allocating routine.
 *   - The first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress, with that device current) and caches it; make that first call
 *     outside any stream capture.
 *   - All calls on a device share the one array: two calls whose kernels overlap on the GPU
 *     (different streams, no ordering between them) race.  Calls ordered on one stream are fine:
 *     the array is zero when the library is loaded and each call's last block clears it again.
 * Results are identical to fma_b200_continuous_count.
 */
int fma_b200_continuous_count_static(const void* ids, int32_t id_bytes, int64_t n, int32_t size, uint32_t* out,
                                     void* stream);

/* ======================================================================= */
/* router: top-k + softmax over the selected logits                         */
/* ======================================================================= */
/*
 * For each of T rows of logits[T,E]: the k largest values in descending order
 * (ties: lowest expert id first), softmax over those k values in fp32, cast to
 * `dtype`.  Replaces MoE._get_topk + the softmax of MoE._compute_routing_weights
 * (fma/modules/moe/__init__.py:191-204, :292-298).
 *   logits    [T,E] dtype, row-major      weights  [T,k] dtype
 *   selected  [T,k] int64                 E <= 1024, 1 <= k <= min(E, 32)
 */
int fma_b200_router_topk_softmax(const void* logits, int32_t dtype, int64_t T, int32_t E, int32_t k,
                                 void* weights, int64_t* selected, void* stream);
/*
 * NaN logits order as the largest value (what torch.topk does), lowest expert id first among them, so
 * `selected` always holds k distinct ids in [0,E); the weights of such a row are NaN, as the reference's
 * softmax makes them.
 *
 * The same pass with the by-products the next steps of the layer need, so that the logits and the selected
 * ids are not read again (same reference lines, plus continuous_count / sort in MoE._compute_experts,
 * fma/modules/moe/__init__.py:213-217, and the router_logits the caller turns into a load-balancing loss,
 * :189): the per-warp histograms of the selected ids, which are the first pass of the expert sort, and -
 * with want_probs != 0 - per-expert partial sums of softmax(logits[t,:]) over all E experts.  Both land in
 * `sort_workspace` (fma_b200_moe_sort_workspace_bytes(T*k, E) bytes); pass that workspace unchanged to
 * fma_b200_moe_sort_routed with the same T, k and E.
 */
int fma_b200_router_topk_softmax_routed(const void* logits, int32_t dtype, int64_t T, int32_t E, int32_t k,
                                        void* weights, int64_t* selected, int32_t want_probs, void* sort_workspace,
                                        int64_t workspace_bytes, void* stream);
/*
 * Backward of the above: d_logits[T,E] (fully written; zero outside the selected
 * columns) from d_weights[T,k]:  d_tv = w * (d_w - sum_j d_w*w) in fp32, scattered
 * to the selected columns.  Stands in for autograd through F.softmax/topk
 * (fma/modules/moe/__init__.py:201-202, :296).
 */
int fma_b200_router_topk_softmax_backward(const void* weights, const void* d_weights, const int64_t* selected,
                                          int32_t dtype, int64_t T, int32_t E, int32_t k, void* d_logits,
                                          void* stream);
/*
 * Backward of mean_prob[e] = (1/T) sum_t softmax(logits[t,:])[e] (the router statistic that
 * fma_b200_moe_sort_routed returns): d_logits[t,c] = p[t,c] * (g[c] - sum_e g[e]*p[t,e]) / T with
 * g = d_mean_prob (fp32 [E]); the softmax is recomputed from the logits.  Stands in for autograd through
 * the softmax a caller applies to the router_logits that MoE.forward returns
 * (fma/modules/moe/__init__.py:189) when it forms a load-balancing loss.  d_logits [T,E] dtype, fully written.
 */
int fma_b200_router_mean_prob_backward(const void* logits, const float* d_mean_prob, int32_t dtype, int64_t T,
                                       int32_t E, void* d_logits, void* stream);

/* ======================================================================= */
/* expert sort + row maps                                                   */
/* ======================================================================= */
/*
 * Stable counting sort of the R = T*k selected expert ids and the row maps of the
 * expert-contiguous ("grouped") layout.  Replaces selected_experts.flatten().sort()
 * and continuous_count in MoE._compute_experts (fma/modules/moe/__init__.py:213-217)
 * and the padding-offset helpers of the reference's cuda branch
 * (fma/modules/moe/cuda_implementation/__init__.py:83-104).
 *
 * Grouped layout: expert e owns rows [pad_offsets[e], pad_offsets[e+1]) where each
 * segment length is expert_count[e] rounded up to `row_align` (a multiple of 128 -
 * 256 lets the GEMMs use CTA pairs - or 1 for no padding); the first expert_count[e] rows of a segment hold its
 * tokens in ascending flat index (t*k+j), the rest are padding.
 *
 * Outputs (any may be NULL to skip, except expert_count and pad_offsets):
 *   sorted_expert_idxs     int64[R]   == sort(stable).values
 *   sorted_scattered_idxs  int64[R]   == sort(stable).indices
 *   expert_count           uint32[E]
 *   pad_offsets            int32[E+1]
 *   row_of_slot            int32[R]   grouped row of flat slot t*k+j
 *   slot_of_row            int32[rows_cap]  flat slot held by a grouped row, -1 for padding
 *                                     and for rows at or beyond pad_offsets[E]
 *   mtile_expert           int32[rows_cap/128]  expert that owns each 128-row tile, -1 beyond
 *                                     the last used tile (only when row_align % 128 == 0)
 * rows_cap must be >= fma_b200_moe_rows_cap(R, E, row_align).
 * workspace: fma_b200_moe_sort_workspace_bytes(R, E) bytes, 4-byte aligned, contents irrelevant.
 * `selected` values should lie in [0,E); E <= 1024.  An id outside the range is never used as an index:
 * it is left out of the counts and of the sorted outputs, its row_of_slot entry is -1 (the scatter /
 * combine kernels skip such slots) and code 0x7003 is recorded in the device status word.
 *
 * fma_b200_moe_sort_routed is the same sort for ids that fma_b200_router_topk_softmax_routed selected
 * (R = T*k): the histogram pass is skipped because that call left it in `workspace`.  If
 * router_mean_prob is not NULL (and the router call had want_probs != 0) it also receives
 * float32[E]: the mean over the T tokens of softmax(logits[t,:])[e], summed in a fixed order
 * (deterministic); together with expert_count these are the two factors of the usual load-balancing loss.
 */
int64_t fma_b200_moe_rows_cap(int64_t R, int32_t E, int32_t row_align);
int64_t fma_b200_moe_sort_workspace_bytes(int64_t R, int32_t E);
int fma_b200_moe_sort(const int64_t* selected, int64_t R, int32_t E, int32_t row_align, int64_t rows_cap,
                      int64_t* sorted_expert_idxs, int64_t* sorted_scattered_idxs, uint32_t* expert_count,
                      int32_t* pad_offsets, int32_t* row_of_slot, int32_t* slot_of_row, int32_t* mtile_expert,
                      void* workspace, int64_t workspace_bytes, void* stream);
int fma_b200_moe_sort_routed(const int64_t* selected, int64_t T, int32_t k, int32_t E, int32_t row_align,
                             int64_t rows_cap, int64_t* sorted_expert_idxs, int64_t* sorted_scattered_idxs,
                             uint32_t* expert_count, int32_t* pad_offsets, int32_t* row_of_slot, int32_t* slot_of_row,
                             int32_t* mtile_expert, float* router_mean_prob, void* workspace, int64_t workspace_bytes,
                             void* stream);

/*
 * Row maps for rows received from other ranks under expert parallelism: `counts` is
 * int32[n_src, E_local] (rows that source s holds for local expert e; each source sends
 * its segments padded to `row_align` back to back).  Writes, for the concatenated receive
 * buffer, mtile_expert int32[rows_cap/128] (local expert of each 128-row tile, -1 beyond
 * the end) and seg_offsets int32[n_src*E_local+1] (row offset of every (s,e) segment).
 * No reference counterpart (the reference has no expert parallelism).
 */
int fma_b200_moe_ep_recv_maps(const int32_t* counts, int32_t n_src, int32_t E_local, int32_t row_align,
                              int64_t rows_cap, int32_t* seg_offsets, int32_t* mtile_expert, void* stream);

/* ======================================================================= */
/* token scatter / weighted combine                                         */
/* ======================================================================= */
/*
 * grouped[row_of_slot[t*k+j], :] = x[t, :] for every token t and j < k (each token row is read
 * once), zeros for padding rows (slot_of_row == -1) below pad_offsets[E]; rows beyond are left
 * untouched.  Replaces
 * hidden_states[fan_in_index] (fma/modules/moe/__init__.py:269,275) and
 * group_with_padding (fma/modules/moe/cuda_implementation/__init__.py:107-157).
 * H*sizeof(dtype) must be a multiple of 16; pointers 16-byte aligned.
 */
int fma_b200_moe_scatter(const void* x, int32_t dtype, int64_t T, int32_t H, int32_t k,
                         const int32_t* row_of_slot, const int32_t* slot_of_row, const int32_t* pad_offsets,
                         int32_t E, int64_t rows_cap, void* grouped, void* stream);
/*
 * dx[t,:] = sum_j d_grouped[row_of_slot[t*k+j], :], accumulated in fp32 in ascending j
 * (deterministic).  Replaces the index backward of the gather and
 * _GroupWithPadding.backward (fma/modules/moe/cuda_implementation/__init__.py:161-183).
 */
int fma_b200_moe_scatter_backward(const void* d_grouped, int32_t dtype, int64_t T, int32_t H, int32_t k,
                                  const int32_t* row_of_slot, void* dx, void* stream);
/*
 * y[t,:] = sum_j w[t,j] * expert_out[row_of_slot[t*k+j], :] in fp32, cast to dtype.
 * Replaces batch_gates multiply + index_add (fma/modules/moe/__init__.py:272-273,
 * :284-286) and ungroup_with_padding + torch.bmm (:235-246).
 */
int fma_b200_moe_combine(const void* expert_out, const void* weights, int32_t dtype, int64_t T, int32_t H,
                         int32_t k, const int32_t* row_of_slot, void* y, void* stream);
/*
 * From dy[T,H]: d_expert_out[row,:] = w[t,j]*dy[t,:] on token rows and zeros on padding
 * rows below pad_offsets[E]; d_weights[t,j] = <expert_out[row,:], dy[t,:]> (fp32 sum,
 * cast to dtype; skipped when d_weights or expert_out is NULL).  Replaces autograd through
 * the combine (fma/modules/moe/__init__.py:284-286) and _UngroupWithPadding.backward
 * (fma/modules/moe/cuda_implementation/__init__.py:228-249); d_weights follows
 * fma/modules/moe/triton_implementation/__init__.py:82-87.
 */
int fma_b200_moe_combine_backward(const void* dy, const void* expert_out, const void* weights, int32_t dtype,
                                  int64_t T, int32_t H, int32_t k, const int32_t* row_of_slot,
                                  const int32_t* slot_of_row, const int32_t* pad_offsets, int32_t E,
                                  int64_t rows_cap, void* d_expert_out, void* d_weights, void* stream);

/*
 * Per-expert bias of `Experts` (add_bias=True): grouped[p,:] += bias[e(p),:] on token rows, padding rows
 * stay zero; and its gradient d_bias[e,:] = sum of d_grouped over the rows of expert e (fp32 sum in row
 * order).  Replaces the bias of F.linear in Experts.torch_forward (fma/modules/moe/__init__.py:102-105);
 * the reference's CUDA path drops the bias (:89-92).  C = bias width, a multiple of 16 bytes.
 */
int fma_b200_moe_bias_add(void* grouped, const void* bias, int32_t dtype, int64_t rows_cap, int32_t C,
                          const int32_t* mtile_expert, const int32_t* slot_of_row, void* stream);
int fma_b200_moe_bias_grad(const void* d_grouped, int32_t dtype, int32_t E, int32_t C, const int32_t* pad_offsets,
                           void* d_bias, void* stream);

/* Zeroes the padding rows at the end of every segment of a grouped layout that was filled by someone who writes
 * token rows only (the packed receive layout of the expert-parallel layer): rows
 * [seg_offsets[j] + counts[j], seg_offsets[j + 1]) for j < n_segments; seg_offsets has n_segments + 1 entries
 * relative to `rows`, row_bytes is a multiple of 16.  No reference counterpart (the reference zero-fills the whole
 * padded buffer, modules/moe/cuda_implementation/__init__.py:122-126). */
int fma_b200_moe_zero_padding(void* rows, int64_t row_bytes, const int32_t* seg_offsets, const int32_t* counts,
                               int32_t n_segments, void* stream);

/* ======================================================================= */
/* swiglu                                                                   */
/* ======================================================================= */
/*
 * out[r,c] = up[r,c] * gate[r,c] * sigmoid(gate[r,c]) computed in fp32, sigmoid input
 * clamped to +-88.3762626647949.  gate/up/out are [rows, cols] with row pitches in
 * elements (so the two halves of a packed [rows, 2*cols] tensor can be passed).
 * Replaces swiglu_forward_cuda (fma/ops/swiglu/cuda_implementation/forward.cu:59-94,
 * math :18-29, fma/include/activations.h:9-22).  cols and pitches multiples of 16 bytes.
 */
int fma_b200_swiglu_forward(const void* gate, int64_t gate_pitch, const void* up, int64_t up_pitch, void* out,
                            int64_t out_pitch, int32_t dtype, int64_t rows, int64_t cols, void* stream);
/*
 * gate_grad = dy*up*(s + g*s*(1-s)), up_grad = dy*g*s with s = sigmoid(g).  Replaces
 * swiglu_backward_cuda (fma/ops/swiglu/cuda_implementation/backward.cu:79-129, math :18-42).
 */
int fma_b200_swiglu_backward(const void* gate, int64_t gate_pitch, const void* up, int64_t up_pitch,
                             const void* dy, int64_t dy_pitch, void* gate_grad, int64_t gate_grad_pitch,
                             void* up_grad, int64_t up_grad_pitch, int32_t dtype, int64_t rows, int64_t cols,
                             void* stream);

/* ======================================================================= */
/* sequence packing (the op that hands packed tokens to the layer)          */
/* ======================================================================= */
/*
 * pack: packed[t, :] = padded[b, s, :] for every token of the padded batch [B, S, row]; unpack: the inverse,
 * with the padding rows of `padded` written as zeros (the output needs no zero-fill beforehand).  Sequence b
 * owns packed rows [cu_seqlens[b], cu_seqlens[b+1]) and sits at the end (pad_left != 0) or the start of its S
 * positions.  Rows are opaque: row_bytes = bytes of one token's data, a multiple of 16.  cu_seqlens: B+1
 * unsigned 32-bit or signed 64-bit integers on the device (index_bytes 4 or 8); total = rows of `packed`.
 * Lengths outside [0, S] and rows outside [0, total) are clamped / skipped, never dereferenced.
 * Replace pack_unpack_sequence_cuda (fma/ops/sequence_packing/cuda_implementation/kernel.cu:45-137) and the
 * torch.zeros that precedes its unpack call (fma/ops/sequence_packing/__init__.py:44).
 */
int fma_b200_pack_sequence(const void* padded, void* packed, const void* cu_seqlens, int32_t index_bytes, int64_t B,
                           int64_t S, int64_t total, int64_t row_bytes, int32_t pad_left, void* stream);
int fma_b200_unpack_sequence(const void* packed, void* padded, const void* cu_seqlens, int32_t index_bytes, int64_t B,
                             int64_t S, int64_t total, int64_t row_bytes, int32_t pad_left, void* stream);

/* ======================================================================= */
/* grouped GEMM                                                             */
/* ======================================================================= */
/*
 * Layer GEMMs over the grouped layout produced by fma_b200_moe_sort with
 * row_align % 128 == 0.  W is [E, OUT, IN] row-major (Experts.weight,
 * fma/modules/moe/__init__.py:22).  bf16 runs on tcgen05 tensor cores with fp32
 * accumulation in tensor memory; f32 runs on an fp32 FFMA kernel.  They replace the
 * three grouped_gemm calls of _GroupedGemmExperts
 * (fma/modules/moe/cuda_implementation/__init__.py:28-38 forward, :54-64 dgrad,
 * :68-78 wgrad) and grouped_gemm_cuda (fma/ops/grouped_gemm/cuda_implementation/kernel.cu:354-388).
 *
 *   forward  Y[p,:]  = X[p,:] . W[e(p)]^T                     X [rows_cap, IN]  -> Y  [rows_cap, OUT]
 *   dgrad    dX[p,:] = dY[p,:] . W[e(p)]                      dY [rows_cap, OUT] -> dX [rows_cap, IN]
 *   wgrad    dW[e]   = dY[seg e]^T . X[seg e]  (zeros for an empty expert)     -> dW [E, OUT, IN]
 *
 * Rows at or beyond pad_offsets[E] are neither read into results nor written.
 * mtile_expert / pad_offsets come from fma_b200_moe_sort or fma_b200_moe_ep_recv_maps.
 * For wgrad under expert parallelism an expert's rows may lie in n_seg segments:
 * seg_offsets is then int32[n_seg*E+1] laid out [segment s][expert e] and
 * pad_offsets is ignored; pass n_seg = 1 and seg_offsets = pad_offsets otherwise.
 * The 16-bit wgrad hands its tiles out expert by expert in the order of decreasing row count (a tile's reduction
 * length is its expert's row count; a one-block kernel writes the order into scratch inside the library first).
 * IN and OUT must be multiples of 8; all pointers 16-byte aligned.
 * row_align is the alignment the grouped rows were sorted with (fma_b200_moe_sort's row_align, or the
 * one given to fma_b200_moe_ep_recv_maps): with a multiple of 256 the bf16 kernels run on CTA pairs
 * (tcgen05 cta_group::2, one 256x512 tile per two SMs); with 128 on single CTAs (128x256 tiles).
 */
int fma_b200_moe_gemm_forward(const void* X, const void* W, void* Y, int32_t dtype, int64_t rows_cap, int32_t E,
                              int32_t OUT, int32_t IN, const int32_t* mtile_expert, int32_t row_align, void* stream);
int fma_b200_moe_gemm_dgrad(const void* dY, const void* W, void* dX, int32_t dtype, int64_t rows_cap, int32_t E,
                            int32_t OUT, int32_t IN, const int32_t* mtile_expert, int32_t row_align, void* stream);
int fma_b200_moe_gemm_wgrad(const void* dY, const void* X, void* dW, int32_t dtype, int64_t rows_cap, int32_t E,
                            int32_t OUT, int32_t IN, const int32_t* seg_offsets, int32_t n_seg, void* stream);
/*
 * Up projection with SwiGLU in the epilogue: W is [E, 2*I, IN] with rows 0..I-1 = up and
 * I..2I-1 = gate (the chunk order of swiglu_packed, fma/ops/swiglu/__init__.py:153).
 * Writes pre[p, 0:2I] = X.W^T rounded to dtype (kept for backward) and
 * act[p, 0:I] = swiglu(gate, up) computed from the rounded values, which is what
 * c_fc followed by self.act computes (fma/modules/moe/__init__.py:230-232).
 * pre may be NULL to skip storing it.  I % 8 == 0.
 */
int fma_b200_moe_gemm_forward_swiglu(const void* X, const void* W, void* pre, void* act, int32_t dtype,
                                     int64_t rows_cap, int32_t E, int32_t I, int32_t IN,
                                     const int32_t* mtile_expert, int32_t row_align, void* stream);
/*
 * Down-projection dgrad with the SwiGLU backward in the epilogue:
 * d_act = dY . W[e] ([rows, I], rounded to dtype), then with up/gate read from pre
 * [rows, 2I]:  d_pre[:, 0:I] = d_up, d_pre[:, I:2I] = d_gate.  Replaces the dgrad of c_proj
 * followed by the swiglu backward kernel
 * (fma/modules/moe/cuda_implementation/__init__.py:54-64; fma/ops/swiglu/__init__.py:41-59).
 */
int fma_b200_moe_gemm_dgrad_swiglu(const void* dY, const void* W, const void* pre, void* d_pre, int32_t dtype,
                                   int64_t rows_cap, int32_t E, int32_t OUT, int32_t I,
                                   const int32_t* mtile_expert, int32_t row_align, void* stream);

/*
 * General grouped GEMM with the reference's memory model: A, B and D are flat buffers of
 * per-group matrices packed back to back; group g multiplies [M_g,K_g] by [K_g,N_g].
 * A_g is row-major [M_g,K_g] ([K_g,M_g] if a_transposed), B_g row-major [K_g,N_g]
 * ([N_g,K_g] if b_transposed), D_g row-major [M_g,N_g].  bf16 only, alpha = 1, beta = 0.
 * Replaces grouped_gemm_cuda (fma/ops/grouped_gemm/cuda_implementation/kernel.cu:354-388).
 * M/N/K are HOST arrays of length n_groups (the python wrapper copies the reference's
 * device uint32 arrays to the host; the reference reads them on the device,
 * kernel.cu:50-92).  Every matrix row pitch must be a multiple of 8 elements.
 * workspace: device memory, fma_b200_grouped_gemm_workspace_bytes(n_groups, total_mtiles)
 * bytes where total_mtiles = sum_g ceil(M_g/128); the call fills it with
 * cudaMemcpyAsync from a pageable host buffer (which synchronises the host with that copy).
 */
int64_t fma_b200_grouped_gemm_workspace_bytes(int32_t n_groups, int64_t total_mtiles);
int fma_b200_grouped_gemm(const void* A, const void* B, void* D, const uint32_t* M, const uint32_t* N,
                          const uint32_t* K, int32_t n_groups, int32_t a_transposed, int32_t b_transposed,
                          void* workspace, int64_t workspace_bytes, void* stream);

/* ======================================================================= */
/* peer-memory transport of the expert-parallel layer                        */
/* ======================================================================= */
/*
 * No counterpart in the reference (it has no expert parallelism).  Buffers that every process of a
 * node can address (CUDA IPC), row-block copies into them with the copy engines, and sequence-numbered
 * flags: the sender's stream runs peer_copy then peer_signal, the receiver's stream runs peer_wait
 * before the kernels that read the rows.
 *
 * peer_buffer_create  cudaMalloc + zero fill + IPC handle (FMA_B200_PEER_HANDLE_BYTES bytes) of a
 *                     buffer on the current device.
 * peer_buffer_open    maps another process's buffer from its handle; *ptr_out is valid in this process
 *                     (copies and kernels of this library may write to it).  Not for one's own handle.
 * peer_buffer_close / peer_buffer_destroy   undo open / create.
 * peer_copy           n cudaMemcpyAsync calls dst[i] <- src[i], bytes[i] (device addresses in host
 *                     arrays), in order, on `stream`.
 * peer_signal         one small kernel: *flag_addrs[i] = value (release, system scope), n <= 64.
 * peer_wait           one small kernel: returns when flags[i] - value >= 0 for all i < n, or records
 *                     device status 0x7002 after timeout_ms (1..60000) and returns.
 */
/*
 * moe_gemm_forward_peer / moe_gemm_dgrad_peer: fma_b200_moe_gemm_forward / _dgrad (bf16, row_align a multiple
 * of 256) whose output is not one matrix: the 128 rows of m-tile i are stored at byte address dst_table[i]
 * (device array, rows_cap/128 entries; row pitch OUT resp. IN elements; addresses 16-byte aligned), which may
 * lie in a buffer opened with peer_buffer_open.  The expert-parallel layer uses them to return expert
 * outputs and input gradients straight into the arenas of the ranks the rows came from.  Entries of tiles
 * beyond the used rows (mtile_expert < 0) are not read.
 */
int fma_b200_moe_gemm_forward_peer(const void* X, const void* W, const uint64_t* dst_table, int32_t dtype,
                                   int64_t rows_cap, int32_t E, int32_t OUT, int32_t IN, const int32_t* mtile_expert,
                                   int32_t row_align, void* stream);
int fma_b200_moe_gemm_dgrad_peer(const void* dY, const void* W, const uint64_t* dst_table, int32_t dtype,
                                 int64_t rows_cap, int32_t E, int32_t OUT, int32_t IN, const int32_t* mtile_expert,
                                 int32_t row_align, void* stream);

#define FMA_B200_PEER_HANDLE_BYTES 64
int fma_b200_peer_buffer_create(int64_t bytes, void** ptr_out, uint8_t* handle_out);
int fma_b200_peer_buffer_open(const uint8_t* handle, void** ptr_out);
int fma_b200_peer_buffer_close(void* ptr);
int fma_b200_peer_buffer_destroy(void* ptr);
int fma_b200_peer_copy(int32_t n, const uint64_t* dst, const uint64_t* src, const int64_t* bytes, void* stream);
int fma_b200_peer_signal(int32_t n, const uint64_t* flag_addrs, int32_t value, void* stream);
int fma_b200_peer_wait(const int32_t* flags, int32_t n, int32_t value, int32_t timeout_ms, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FMA_B200_H */
