/*
 * b200_blockfp8 -- C ABI of the B200 (sm_100a) block-FP8 W8A8 linear + fused-MoE kernels.
 *
 * Conventions
 *  - Every pointer is a DEVICE pointer owned by the caller unless stated otherwise; the
 *    library borrows it for the duration of the call, allocates nothing, never
 *    synchronises and never creates a stream. Work is enqueued on `stream` (a
 *    cudaStream_t passed as void*).
 *  - Every entry point returns 0 on success or a negative B200_E_* code; nothing throws.
 *    b200_status_string() turns a code into text, b200_last_error_detail() gives the
 *    detail of the most recent failure on the calling thread.
 *  - dtype codes: B200_BF16 / B200_F16 / B200_F32 for floating tensors,
 *    B200_I32 / B200_I64 for index tensors.
 *
 * The reference has no C ABI for this path (its kernels are torch C++ ops); each entry
 * point cites the reference operator it replaces, by path inside the reference project.
 */
#ifndef B200_BLOCKFP8_H_
#define B200_BLOCKFP8_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  B200_OK = 0,
  B200_E_BAD_ARG = -1,       /* null pointer, negative size, unknown dtype / mode */
  B200_E_UNSUPPORTED = -2,   /* legal in the reference but not built here (stated per call) */
  B200_E_LAUNCH = -3,        /* CUDA reported an error at launch / descriptor encode */
  B200_E_WORKSPACE = -4,     /* workspace missing or smaller than *_workspace_bytes() */
  B200_E_TIMEOUT = -5        /* a bounded device-side wait ran out (see b200_read_device_status) */
};

enum { B200_BF16 = 0, B200_F16 = 1, B200_F32 = 2, B200_I32 = 3, B200_I64 = 4 };

/* quant arithmetic variants (all: amax = max(|x|, eps) over the group, fp32)
 *   0: s = amax / 448,     q = x / s        (reference torch-native + CUDA v1)
 *   1: s = amax / 448,     q = x * (1 / s)  (reference Triton row-major)
 *   2: s = amax * (1/448), q = x * (448 / amax)  (reference CUDA v2)
 *   3: variant 0 computed without a per-element division: r = 1/s correctly rounded,
 *      q0 = x * r, q = copysign(fma(fma(-q0, s, x), r, q0), x). For bf16 and f16 inputs with eps = 1e-10 the
 *      bytes and scales equal variant 0's for every (x, amax) pair that exists (both types have
 *      fewer than 2^31 such pairs; the GPU tests enumerate them all). Not claimed for f32 input. */
enum { B200_QUANT_DIV = 0, B200_QUANT_RECIP = 1, B200_QUANT_V2 = 2, B200_QUANT_DIV_CORRECTED = 3 };

const char* b200_status_string(int status);
const char* b200_last_error_detail(void);
int b200_abi_version(void);

/* Device-side status word. Kernels with bounded waits (the TMA / tcgen05 pipelines)
 * record a non-zero code there instead of trapping or spinning for ever.
 * b200_read_device_status synchronises `stream`, copies the word of the current device
 * to *out (host pointer) and clears it. 0 = no kernel reported a problem. */
int b200_read_device_status(int* out, void* stream);

/* Process-wide tuning knobs: how tests force one kernel path and tuning sweeps try a setting.
 * Product calls never read the environment; a knob left at -1 is decided automatically.
 * Names: "gemm_bn" (128 / 256), "gemm_skinny" (0 = never the decode kernel),
 * "gemm_skinny_max_m", "gemm_splitk" (> 0 forces the K split; size the workspace after setting
 * it), "gemm_2cta" (0 / 1), "gemm_ue8m0" (0 = packed power-of-two scales are unpacked and take the
 * fp32-scale kernels), "linear_decode_fused" (0 = never the one-launch decode linear), "moe_decode"
 * (1 = few-token swapped-operand MoE kernels; default off), "moe_down_splitk" (0 = never),
 * "moe_zero_pads" (0 / 1), "peer_wait_ms" (limit of a device-side wait for another GPU, 100 .. 60000).
 * No counterpart in the reference (its Triton launchers read tuned JSON configs instead,
 * python/sglang/srt/layers/moe/fused_moe_triton/fused_moe_triton_config.py). Not thread-safe
 * against concurrent launches: set knobs before the calls they affect. */
int b200_set_tuning(const char* name, long value);
int b200_get_tuning(const char* name, long* value);

/* ---------------------------------------------------------------------------------------
 * per_token_group_quant_fp8
 * replaces: python/sglang/srt/layers/quantization/fp8_kernel.py:498-565
 *           (torch.ops.sgl_kernel.sgl_per_token_group_quant_8bit[_v2],
 *            sgl-kernel/csrc/gemm/per_token_group_quant_8bit.cu:116-217)
 * x [M,K] contiguous (x_dtype bf16/f16/f32) -> q [M,K] FP8 E4M3 bytes, and one fp32 scale per
 * (row, group) stored at s[m*s_stride_m + g*s_stride_g] (row-major: (K/group,1);
 * column-major: (1,M); "TMA-aligned": (1, ceil4(M))). group in {16,32,64,128,256,512},
 * K % group == 0. q rows are 16-byte aligned when K % 16 == 0 (required).            */
int b200_per_token_group_quant_fp8(const void* x, int x_dtype, void* q, float* s,
                                   int64_t M, int64_t K, int group,
                                   int64_t s_stride_m, int64_t s_stride_g,
                                   float eps, int formula, void* stream);

/* Same quantisation with power-of-two ("UE8M0") scales packed for MN-major consumers
 * replaces: sglang_per_token_group_quant_fp8(..., column_major_scales=True, scale_tma_aligned=True,
 *           scale_ue8m0=True[, fuse_silu_and_mul=True[, masked_m=...]]) (fp8_kernel.py:498-565,
 *           :568-610) -> sgl-kernel/csrc/gemm/per_token_group_quant_8bit_v2.cu
 * x [M,K] (or [M,2K] = gate | up when fuse_silu_and_mul: the quantised value is T(silu(gate)) * up
 * in the input type); q [M,K] e4m3; s_packed: int32 words, the scale of (row t, group g) is the
 * biased exponent byte (g % 4) of word [g/4][t] of a [ceil(K/group/4)][aligned_mn] array
 * (aligned_mn >= rows, multiple of 4); bytes past the last group are written as 0.
 * amax is floored at 1e-10, e = ceil(log2(amax/448)), q = x * 2^-e, byte = e + 127.
 * masked_m != NULL: x is [num_experts][M/num_experts][..], rows t >= masked_m[expert] are skipped
 * and every expert has its own scale array (expert stride ceil(K/group/4) * aligned_mn words). */
int b200_per_token_group_quant_fp8_ue8m0(const void* x, int x_dtype, void* q, void* s_packed,
                                         int64_t M, int64_t K, int group, int64_t aligned_mn,
                                         int fuse_silu_and_mul, const int32_t* masked_m,
                                         int num_experts, void* stream);

/* ---------------------------------------------------------------------------------------
 * w8a8_block_fp8_matmul
 * replaces: python/sglang/srt/layers/quantization/fp8_kernel.py:1285-1300 (Triton kernel
 *           :780-869) and torch.ops.sgl_kernel.fp8_blockwise_scaled_mm
 *           (sgl-kernel/csrc/gemm/fp8_blockwise_gemm_kernel.cu:425-522)
 * C[m,n] = sum_kb (sum_{k in kb} A[m,k]*B[n,k]) * As[m,kb] * Bs[n/128,kb], block = [128,128].
 * A [M,K] e4m3 row-major, B [N,K] e4m3 row-major, As fp32 at As[m*as_stride_m+kb*as_stride_k],
 * Bs fp32 [ceil(N/128), ceil(K/128)] row-major, C [M,N] (c_dtype bf16/f16/f32) row-major.
 * Requirements: K % 16 == 0, N % 8 == 0, A, B and C 16-byte aligned.
 * workspace: b200_w8a8_block_fp8_gemm_workspace_bytes(M,N,K) bytes (may be 0 -> NULL ok). */
size_t b200_w8a8_block_fp8_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K);
int b200_w8a8_block_fp8_gemm(const void* A, const float* As, int64_t as_stride_m,
                             int64_t as_stride_k, const void* B, const float* Bs, void* C,
                             int c_dtype, int64_t M, int64_t N, int64_t K, void* workspace,
                             size_t workspace_bytes, void* stream);

/* ---------------------------------------------------------------------------------------
 * w8a8_block_fp8_matmul with power-of-two (UE8M0) scales applied inside the tensor core
 * replaces: the DeepGEMM path the reference takes on Blackwell for block-FP8 linears
 *           (python/sglang/srt/layers/quantization/fp8_utils.py:466-540 deepgemm_w8a8_block_fp8_linear_with_fallback,
 *            scales prepared by :1209-1334 requant_weight_ue8m0 / transform_scale_ue8m0 and the
 *            scale_ue8m0 form of per_token_group_quant_fp8, fp8_kernel.py:498-610)
 * C[m,n] = sum_k A[m,k] * B[n,k] * 2^(ea[m,k/128]-127) * 2^(eb[n,k/128]-127), fp32 accumulation over the whole
 * K in tensor memory (tcgen05.mma.kind::mxf8f6f4.block_scale): no per-K-block promotion.
 * A [M,K] e4m3 row-major, B [N,K] e4m3 row-major. sfa: int32 words, word [g*sfa_ld + m] holds the exponent
 * bytes of row m for the 128-K blocks 4g..4g+3 (byte kb%4; the packed MN-major layout of the reference,
 * sfa_ld = rows padded to a multiple of 4). sfb: the same for the rows of B (sfb_rows_per_word = 1) or for its
 * 128-row blocks (sfb_rows_per_word = 128). C [M,N] bf16/f16/f32. K % 16 == 0, N % 8 == 0; no workspace. */
int b200_w8a8_block_fp8_gemm_ue8m0(const void* A, const int32_t* sfa, int64_t sfa_ld, const void* B,
                                   const int32_t* sfb, int64_t sfb_ld, int sfb_rows_per_word, void* C,
                                   int c_dtype, int64_t M, int64_t N, int64_t K, void* stream);

/* ---------------------------------------------------------------------------------------
 * w8a8_block_fp8_linear at decode size: quantise + GEMM + split-K sum in ONE launch
 * replaces: the composition of python/sglang/srt/layers/quantization/fp8_utils.py:814-834
 *           (per_token_group_quant_fp8, then w8a8_block_fp8_matmul) for M <= 16 rows; the
 *           reference chains its quantiser and GEMM as programmatic dependents instead
 *           (sgl-kernel/csrc/gemm/per_token_group_quant_8bit_v2.cu:456-466)
 * out[m,n] = sum_kb (q(x)[m,kb] . B[n,kb]) * xs[m,kb] * Bs[n/128,kb] with q / xs the 1x128 group
 * quantisation of x (arithmetic variant 0, eps as given): the same bytes and scales the stand-alone
 * quantiser produces, so the result equals quantise-then-GEMM up to the fp32 summation order.
 * x [M,K] bf16/f16 row-major (M <= 16), B [N,K] e4m3, Bs fp32 [ceil(N/128), ceil(K/128)],
 * out [M,N] in the dtype of x. K % 16 == 0, N % 8 == 0, N <= 524288.
 * workspace: b200_w8a8_block_fp8_linear_decode_workspace_bytes(M,N,K) bytes (fp32 partials of the K
 * splits). tickets: 4096 uint32 that are ZERO before the first call and belong to one stream (every
 * call leaves them zero; calls that overlap on the GPU must not share them). Anything else:
 * B200_E_UNSUPPORTED (callers fall back to the two-step path). */
size_t b200_w8a8_block_fp8_linear_decode_workspace_bytes(int64_t M, int64_t N, int64_t K);
int b200_w8a8_block_fp8_linear_decode(const void* x, int x_dtype, const void* B, const float* Bs,
                                      void* out, int64_t M, int64_t N, int64_t K, float eps,
                                      void* workspace, size_t workspace_bytes, void* tickets,
                                      void* stream);

/* ---------------------------------------------------------------------------------------
 * moe_align_block_size
 * replaces: torch.ops.sgl_kernel.moe_align_block_size
 *           (sgl-kernel/csrc/moe/moe_align_kernel.cu:317-383; wrapper
 *            python/sglang/srt/layers/moe/moe_runner/triton_utils/moe_align_block_size.py:19-87)
 * topk_ids: numel ids (ids_dtype i32/i64) in [-1, num_buckets-1); bucket b holds id b-1.
 * Outputs: sorted_token_ids int32 [max_pad] (flat indices, ascending inside a bucket, `numel`
 * in pad slots; every one of the max_pad slots is written whatever pad_sorted says: a superset of
 * the reference's pad_sorted_token_ids=False, which leaves slots >= num_post_pad untouched),
 * expert_ids int32 [max_blocks] (bucket-1 per block, -1 past the last block),
 * num_post_pad int32 [1], cumsum int32 [num_buckets+1] (end of each bucket's real entries;
 * last = padded total). workspace: b200_moe_align_workspace_bytes(numel, num_buckets).     */
size_t b200_moe_align_workspace_bytes(int64_t numel, int num_buckets);
int b200_moe_align_block_size(const void* topk_ids, int ids_dtype, int64_t numel,
                              int num_buckets, int block_size, int32_t* sorted_token_ids,
                              int64_t max_pad, int32_t* expert_ids, int64_t max_blocks,
                              int32_t* num_post_pad, int32_t* cumsum, int pad_sorted,
                              void* workspace, size_t workspace_bytes, void* stream);

/* ---------------------------------------------------------------------------------------
 * moe_align_block_size without a workspace (no counterpart in the reference).
 * For callers that cannot allocate device memory at the point of the call -- a host that may
 * not call cudaMalloc (e.g. inside a region where the allocator is frozen, or an embedding
 * runtime that owns all device memory) and therefore has no workspace to hand over. Same
 * inputs, outputs and results as b200_moe_align_block_size; the scratch of the multi-block path
 * is a fixed array inside the library (about 129 KB of device memory held by every GPU that
 * loads the library, until the process exits). Limits: numel <= 131072 ids and
 * num_buckets <= 257; anything larger returns B200_E_UNSUPPORTED.
 * The first call on each device resolves the array's device address (one runtime query, no
 * allocation): make that first call before starting any stream capture. The call itself
 * allocates nothing. All calls on a device share the one array: two calls whose kernels can
 * overlap on the GPU (different streams) race on it -- keep them on one stream or order them
 * with events. The array needs no clearing between calls: every word a call reads, it wrote
 * earlier in the same call. */
int b200_moe_align_block_size_static(const void* topk_ids, int ids_dtype, int64_t numel,
                                     int num_buckets, int block_size, int32_t* sorted_token_ids,
                                     int64_t max_pad, int32_t* expert_ids, int64_t max_blocks,
                                     int32_t* num_post_pad, int32_t* cumsum, void* stream);

/* ---------------------------------------------------------------------------------------
 * fused_experts(use_fp8_w8a8=True, block_shape=[128,128])
 * replaces: python/sglang/srt/layers/moe/moe_runner/triton_utils/fused_moe.py:218-306
 *           (kernel sequence :401-785: align -> quant -> grouped GEMM -> silu_and_mul ->
 *            quant -> grouped GEMM * topk_weight -> sum over top-k)
 * hidden [T,H] (h_dtype bf16/f16); or, when hidden_scale != NULL, hidden is ALREADY quantised:
 * e4m3 bytes [T,H] with row-major fp32 scales hidden_scale [T,H/128] (what an expert-parallel
 * dispatch delivers, python/sglang/srt/layers/moe/token_dispatcher/deepep.py:507-567) and
 * h_dtype is the dtype of `out` only. w1 [E,2I,H] e4m3 (gate rows [0,I), up rows [I,2I)),
 * w2 [E,H,I] e4m3, w1_scale fp32 [E,2I/128,H/128], w2_scale fp32 [E,H/128,I/128],
 * topk_weights fp32 [T,topk], topk_ids int32 [T,topk] with values in [-1,E) (-1 = expert
 * not on this rank: contributes 0). out [T,H] (or [T,topk,H] when no_combine != 0), h_dtype;
 * out may alias a 16-bit hidden (the reference's inplace=True). H % 128 == 0, I % 128 == 0.
 * no_combine: B200_COMBINE_SUM (0) sums the slots; B200_COMBINE_NONE (1) returns [T,topk,H];
 * B200_COMBINE_SUM_SKIP_UNROUTED (2) sums the slots but leaves rows without any valid id unwritten
 * (the expert-parallel receive area, where most positions belong to other ranks).
 * routed_scaling_factor multiplies the combined output (pass 1.0f for none); it is ignored with
 * B200_COMBINE_NONE, as in the reference (the caller combines and scales).
 * workspace: b200_fused_experts_fp8_workspace_bytes(T, topk, E, H, I) bytes, 256-B aligned. */
enum { B200_COMBINE_SUM = 0, B200_COMBINE_NONE = 1, B200_COMBINE_SUM_SKIP_UNROUTED = 2 };
size_t b200_fused_experts_fp8_workspace_bytes(int64_t T, int topk, int E, int64_t H, int64_t I);
int b200_fused_experts_fp8(const void* hidden, const float* hidden_scale, int h_dtype,
                           const void* w1, const void* w2,
                           const float* w1_scale, const float* w2_scale,
                           const float* topk_weights, const int32_t* topk_ids, void* out,
                           int64_t T, int topk, int E, int64_t H, int64_t I, int no_combine,
                           int apply_router_weight_on_input, float routed_scaling_factor,
                           void* workspace, size_t workspace_bytes, void* stream);

/* ---------------------------------------------------------------------------------------
 * Experts over the masked (low-latency) layout: tokens already grouped by expert
 * replaces: python/sglang/srt/layers/moe/moe_runner/deep_gemm.py:362-494 (_run_masked_gemm:
 *           masked grouped GEMM -> SiLU*mul + 1x128 re-quant -> masked grouped GEMM) and the
 *           activation kernel python/sglang/srt/layers/moe/ep_moe/kernels.py:288-431
 * hidden_q [E,T_pad,H] e4m3 with row-major fp32 scales hidden_s [E,T_pad,H/128]; only the first
 * masked_m[e] rows of expert e are valid (int32 [E] on the device, clamped to [0,T_pad]).
 * w1 [E,2I,H] (gate rows then up rows), w2 [E,H,I] e4m3 with fp32 128x128 block scales as for
 * b200_fused_experts_fp8. out [E,T_pad,H] bf16/f16: rows t < masked_m[e] are written, the others
 * are left untouched. No router weights (the combine step of the caller applies them).
 * T_pad % 128 == 0, H % 128 == 0, I % 128 == 0. */
size_t b200_masked_experts_fp8_workspace_bytes(int E, int64_t T_pad, int64_t H, int64_t I);
int b200_masked_experts_fp8(const void* hidden_q, const float* hidden_s, const void* w1,
                            const void* w2, const float* w1_scale, const float* w2_scale,
                            const int32_t* masked_m, void* out, int out_dtype, int E, int64_t T_pad,
                            int64_t H, int64_t I, void* workspace, size_t workspace_bytes,
                            void* stream);

/* ---------------------------------------------------------------------------------------
 * Expert routing (the step before fused_experts): scores -> top-k weights and expert ids
 * replaces: python/sglang/srt/layers/moe/topk.py:550-588 (fused_topk_torch_native) and :640-700
 *           (fused_topk -> sgl-kernel topk_softmax / topk_sigmoid,
 *            sgl-kernel/csrc/moe/moe_topk_softmax_kernels.cu, moe_topk_sigmoid_kernels.cu);
 *           topk.py:703-764 (grouped_topk_gpu) and :923-992 (biased_grouped_topk_impl ->
 *            sgl-kernel/csrc/moe/moe_fused_gate.cu)
 * logits [T,E] f32/bf16/f16 row-major; correction_bias fp32 [E] or NULL.
 * scores = softmax(row) or sigmoid(element) in fp32; selection compares scores + bias;
 * n_group > 1: experts form n_group equal consecutive groups, a group's score is the maximum
 * (B200_GROUP_MAX) or the sum of the two largest (B200_GROUP_TOP2_SUM) of its selection values,
 * only the topk_group best groups stay eligible. Ties go to the lower index (the rule of the
 * reference's CUDA kernels, moe_topk_softmax_kernels.cu:545-546). Outputs, in descending order
 * of the selection value: topk_weights fp32 [T,topk] = unbiased scores of the chosen experts,
 * divided by their sum when renormalize != 0, then times output_scale (pass 1.0f for none);
 * topk_ids int32 [T,topk]. Rows t >= *num_token_non_padded (device scalar, may be NULL) get
 * id -1 (topk.py:999-1016). Limits: E <= 1024, topk <= 32, n_group <= 32. No workspace. */
enum { B200_SCORE_SOFTMAX = 0, B200_SCORE_SIGMOID = 1 };
enum { B200_GROUP_MAX = 0, B200_GROUP_TOP2_SUM = 1 };
int b200_route_topk(const void* logits, int logits_dtype, const float* correction_bias, int64_t T,
                    int E, int topk, int scoring, int n_group, int topk_group, int group_score,
                    int renormalize, float output_scale, const int32_t* num_token_non_padded,
                    float* topk_weights, int32_t* topk_ids, void* stream);

/* Softmax top-k over transformed logits
 * replaces: torch.ops.sgl_kernel.topk_softmax with moe_softcapping and / or correction_bias
 *           (sgl-kernel/csrc/moe/moe_topk_softmax_kernels.cu:85-115, 428-458, 720-816)
 * v = logits; softcap != 0: v = tanh(v / softcap) * softcap; logit_bias (fp32 [E], may be NULL): v += bias;
 * scores = softmax(v) per row; top-k of the scores (ties to the lower index), weights = those scores,
 * divided by their sum when renormalize != 0. Unlike b200_route_topk's correction_bias, which only
 * steers the selection, this bias is part of the scores. Same limits, no workspace. */
int b200_route_topk_softmax_capped(const void* logits, int logits_dtype, float softcap,
                                   const float* logit_bias, int64_t T, int E, int topk, int renormalize,
                                   float* topk_weights, int32_t* topk_ids, void* stream);

/* ---------------------------------------------------------------------------------------
 * Row-parallel linear with the tensor-parallel all-reduce done over peer memory
 * replaces: python/sglang/srt/layers/linear.py:1543-1558 (RowParallelLinear.forward: GEMM, then
 *           tensor_model_parallel_all_reduce), python/sglang/srt/distributed/communication_op.py:28-40,
 *           sgl-kernel/csrc/allreduce/custom_all_reduce.cuh:238-383 (one-/two-shot kernels) and the
 *           fused all-reduce + residual + RMSNorm of python/sglang/srt/layers/flashinfer_comm_fusion.py
 * b200_w8a8_block_fp8_gemm_fanout: the block-FP8 GEMM above, but every finished tile is stored
 * into the n_dest buffers dest[d] ([M,N] c_dtype, row-major, 16-byte aligned; `dest` is a HOST
 * array of device pointers, which may be peer GPUs' memory mapped into this process) while the
 * GEMM is still running. dest_by_tile != 0: the tile of 128-row block mt goes only to
 * dest[mt % n_dest] (reduce-scatter by row block). Workspace as for the plain GEMM, sized by
 * b200_w8a8_block_fp8_gemm_fanout_workspace_bytes.
 * b200_allreduce_finish: n_ranks slots of slot_stride elements each (LOCAL memory; slot r holds
 * the [M,N] partial written by rank r's fan-out GEMM; bf16/f16). Handshake with all ranks (flag arrays of 2*8 uint32, zero before the
 * first call, epoch strictly increasing by call and identical on all ranks; my_flags local,
 * peer_flags HOST array of every rank's flag array incl. this rank's), then
 * sum over ranks in fp32 (+ residual -> residual_out; then * rsqrt(mean(x^2)+eps) * rms_weight
 * when rms_weight != NULL) -> out[0]; by_tile != 0: only row blocks mt % n_ranks == rank are
 * reduced and the results are written to out[0..n_ranks) and residual_out[0..n_ranks) (every
 * rank's buffers; `out` and `residual_out` are HOST arrays of device pointers, NULL = none), followed
 * by a second handshake so that on return (in stream order) every rank's output is complete.
 * out_multicast / residual_out_multicast (by_tile only, may be NULL): an NVSwitch multicast address
 * that maps all ranks' output buffers; results are then written once with multimem.st and
 * replicated by the switch instead of being stored to every out[d].
 * epoch == 0 selects device-side epochs (a counter next to the flags, flags[16..18], advanced by
 * the kernels themselves): the identical call can then be replayed from a CUDA graph; a flag array
 * is driven either by host epochs or by device epochs, never both. The flag array is 32 uint32.
 * All waits are bounded (2 s; the "peer_wait_ms" tuning knob). On expiry the device status word
 * becomes 2, this rank's own result buffers (out, residual_out) are filled with NaN instead of a
 * stale sum, and the kernels return normally: callers that do not synchronise per call should poll
 * b200_read_device_status at a cadence of their choice (once per model step, say). */
size_t b200_w8a8_block_fp8_gemm_fanout_workspace_bytes(int64_t M, int64_t N, int64_t K);
int b200_w8a8_block_fp8_gemm_fanout(const void* A, const float* As, int64_t as_stride_m,
                                    int64_t as_stride_k, const void* B, const float* Bs,
                                    void* const* dest, int n_dest, int dest_by_tile, int c_dtype,
                                    int64_t M, int64_t N, int64_t K, void* workspace,
                                    size_t workspace_bytes, void* stream);
int b200_allreduce_finish(const void* slots, int64_t slot_stride, void* const* out, int dtype,
                          int64_t M, int64_t N,
                          int n_ranks, int rank, int by_tile, const void* residual,
                          void* const* residual_out, const void* rms_weight, float eps, void* my_flags,
                          void* const* peer_flags, uint32_t epoch, void* out_multicast,
                          void* residual_out_multicast, void* stream);

/* ---------------------------------------------------------------------------------------
 * Expert-parallel token exchange over peer memory (dispatch / combine around fused_experts)
 * replaces: python/sglang/srt/layers/moe/token_dispatcher/deepep.py:507-602 (normal dispatch and
 *           combine through DeepEP) and standard.py:172-210 (rebasing ids to the owning rank)
 * Rank r owns experts [r*E/p, (r+1)*E/p). Every rank has a receive area indexed by source rank
 * and source token position, four arrays of p*T_max positions: q [p][T_max][H] e4m3 bytes,
 * s [p][T_max][H/128] fp32, w [p][T_max][topk] fp32, ids [p][T_max][topk] int32 (ids rebased to
 * the owner, -1 = not for this rank or no token), and an output area out [p][T_max][H].
 * recv_q/recv_s/recv_w/recv_ids/peer_out are HOST arrays with one device pointer per rank
 * (that rank's area as mapped in this process; peer memory for other ranks).
 * b200_ep_dispatch: for each local token t < T (global topk_ids [T,topk], -1 allowed) store
 *   the row, scales, weights and rebased ids at position [rank][t] of every rank that owns one
 *   of its experts, and ids = -1 at every other rank and for positions T <= t < T_max.
 * b200_peer_handshake: epoch handshake with all ranks (flag arrays as for
 *   b200_allreduce_finish; phase 0 or 1 selects the flag row; epoch strictly increasing per
 *   phase, or 0 for device-side epochs as above). Bounded 2 s, then device status 2. After it returns (in stream order) everything the
 *   other ranks stored before THEIR handshake of the same epoch is visible.
 * (then: b200_fused_experts_fp8 over the p*T_max positions with hidden = q, hidden_scale = s,
 *  out = this rank's output area)
 * b200_ep_combine: out[t] = fp32 sum, in ascending owner rank, of peer_out[d][rank][t][:] over
 *   the ranks d that own an expert of token t; out [T,H] bf16/f16. When the device status word is
 *   already non-zero (a handshake before it gave up), out is filled with NaN instead: the owners'
 *   rows cannot be trusted. */
int b200_ep_dispatch(const void* x_q, const float* x_s, const float* topk_weights,
                     const int32_t* topk_ids, int64_t T, int64_t T_max, int topk, int64_t H, int E,
                     int n_ranks, int rank, void* const* recv_q, void* const* recv_s,
                     void* const* recv_w, void* const* recv_ids, void* stream);
int b200_peer_handshake(void* my_flags, void* const* peer_flags, int n_ranks, int rank, int phase,
                        uint32_t epoch, void* stream);
int b200_ep_combine(void* const* peer_out, const int32_t* topk_ids, void* out, int dtype, int64_t T,
                    int64_t T_max, int topk, int64_t H, int E, int n_ranks, int rank, void* stream);

/* Combine by push (the default of the Python layer): the owners' down GEMM sends every finished
 * (token, slot) row straight into the SOURCE rank's own area while the remaining tiles are still
 * being multiplied, so the combine traffic overlaps the GEMM instead of following it; after the
 * second handshake the source sums its slots locally.
 * replaces: the same DeepEP combine (deepep.py:560-602); in the reference the expert GEMMs and
 *           the combine all-to-all are separate steps.
 * b200_fused_experts_fp8_scatter: fused experts over T positions of quantised rows (hidden_q e4m3
 *   [T,H], hidden_scale fp32 [T,H/128], topk_ids local to this rank, -1 = not mine), router weight
 *   applied, no slot sum: the row of pair flat = t*topk + j goes to dests[flat / rows_per_dest] at
 *   row flat % rows_per_dest of a [rows_per_dest, H] bf16/f16 buffer (HOST array of device
 *   pointers, peer memory allowed; with the receive-area layout above rows_per_dest = T_max*topk and
 *   the destination is the source rank of the token). Rows of pairs that are not this rank's are
 *   not written. Workspace as b200_fused_experts_fp8.
 * b200_moe_sum_reduce: out[t,:] = scale * sum over the slots j with 0 <= topk_ids[t,j] < E of
 *   rows[t*topk + j, :], fp32 sum in slot order; rows without a valid id are zeroed, or left
 *   unwritten with skip_unrouted. poison_on_status != 0: when the device status word is non-zero
 *   (a handshake before it gave up) out is filled with NaN instead. The last step of
 *   fused_experts (moe_sum_reduce, python/sglang/srt/layers/moe/moe_runner/triton_utils/fused_moe.py:726-745)
 *   as an entry point of its own. */
int b200_fused_experts_fp8_scatter(const void* hidden_q, const float* hidden_scale, int out_dtype,
                                   const void* w1, const void* w2, const float* w1_scale,
                                   const float* w2_scale, const float* topk_weights,
                                   const int32_t* topk_ids, void* const* dests, int n_dest,
                                   int64_t rows_per_dest, int64_t T, int topk, int E, int64_t H,
                                   int64_t I, void* workspace, size_t workspace_bytes, void* stream);
int b200_moe_sum_reduce(const void* rows, const int32_t* topk_ids, void* out, int dtype, int64_t T,
                        int topk, int E, int64_t H, float scale, int skip_unrouted,
                        int poison_on_status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200_BLOCKFP8_H_ */
