/*
 * sglang_b200 — C ABI of the B200 (sm_100a) block-wise FP8 W8A8 kernels.
 *
 * Every entry point takes raw device pointers, sizes and a CUDA stream
 * (`cudaStream_t` passed as void*), enqueues work on that stream and returns
 * without synchronising.  No entry point allocates device memory unless its
 * comment says so.  Return value: 0 on success, a negative SGLB200_E_* code on
 * a rejected call (nothing was launched); sglb200_last_error() then holds a
 * message for the calling thread.
 *
 * Each declaration names the reference interface it stands in for (paths are
 * relative to the SGLang repository root).
 *
 * dtype codes for activations: 0 = bfloat16, 1 = float16, 2 = float32.
 */
#ifndef SGLANG_B200_H_
#define SGLANG_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SGLB200_OK 0
#define SGLB200_E_INVALID (-1)    /* bad shape / alignment / argument            */
#define SGLB200_E_UNSUPPORTED (-2) /* device is not sm_100, or unsupported dtype */
#define SGLB200_E_CUDA (-3)       /* a CUDA runtime / driver call failed         */
#define SGLB200_E_WORKSPACE (-4)  /* workspace missing or too small              */

/* Message describing the last non-zero return on this thread. */
const char* sglb200_last_error(void);

/* ABI version of this library (bumped on any signature change). */
int sglb200_abi_version(void);

/* 0 if `device` is a compute-capability 10.x GPU, SGLB200_E_UNSUPPORTED otherwise. */
int sglb200_check_device(int device);

/*
 * 1 x group_size activation quantizer: per group amax = max(|x|, eps),
 * scale = amax / fp8_max (IEEE division), code = e4m3(clamp(x / scale)) (IEEE division,
 * round-to-nearest-even, saturating).
 * Replaces: torch.ops.sgl_kernel.sgl_per_token_group_quant_8bit
 *   (sgl-kernel/csrc/gemm/per_token_group_quant_8bit.cu:116-217, schema
 *   sgl-kernel/csrc/common_extension.cc:138-141) and the Triton kernels behind
 *   per_token_group_quant_fp8 (python/sglang/srt/layers/quantization/fp8_kernel.py:125-216).
 * input  [num_tokens, hidden] contiguous, hidden % group_size == 0, group_size in {32,64,128,256}.
 * output_q [num_tokens, hidden] float8_e4m3fn.
 * output_s element (token t, group g) is written at output_s[t*s_stride_token + g*s_stride_group]
 *   (row-major: (hidden/group_size, 1); M-major "column_major_scales": (1, padded_tokens)).
 */
int sglb200_per_token_group_quant_fp8(const void* input, int in_dtype, void* output_q, float* output_s,
                                      int64_t num_tokens, int64_t hidden, int group_size, float eps, float fp8_min,
                                      float fp8_max, int64_t s_stride_token, int64_t s_stride_group, void* stream);

/*
 * out[r, i] = T( T(silu_f32(x[r, i])) * x[r, d + i] ),  x is [rows, 2d], T in {bf16, fp16}.
 * Replaces: torch.ops.sgl_kernel.silu_and_mul (sgl-kernel/csrc/elementwise/activation.cu:85-105,
 *   schema common_extension.cc:78-79).  d % 8 == 0.
 */
int sglb200_silu_and_mul(void* out, const void* input, int dtype, int64_t rows, int64_t d, void* stream);

/*
 * Fused silu_and_mul + 1x128 re-quantisation: h = silu_and_mul(x) kept in registers, then quantised
 * exactly as sglb200_per_token_group_quant_fp8 would quantise the bf16 tensor h.
 * Replaces the pair silu_and_mul + sglang_per_token_group_quant_fp8 inside fused_experts_impl
 *   (python/sglang/srt/layers/moe/fused_moe_triton/fused_moe.py:555-556 and
 *   fused_moe_triton_kernels.py:632-633); same fusion as
 *   sgl_per_token_group_quant_8bit_v2(fuse_silu_and_mul=True)
 *   (sgl-kernel/csrc/gemm/per_token_group_quant_8bit_v2.cu:336-341) and
 *   _silu_and_mul_post_quant_kernel (python/sglang/srt/layers/moe/ep_moe/kernels.py:287-361).
 * input [rows, 2d] (bf16/fp16), output_q [rows, d], output_s [rows, d/group_size] row-major.
 * If num_rows_dev != NULL it points to a device int32 holding the number of leading rows to process
 * (e.g. num_tokens_post_pad); rows beyond it are skipped.  `rows` is then the upper bound.
 */
int sglb200_silu_and_mul_quant_fp8(const void* input, int dtype, void* output_q, float* output_s, int64_t rows,
                                   int64_t d, int group_size, float eps, const int32_t* num_rows_dev, void* stream);

/*
 * The same fusion over the masked expert layout: input [num_experts, rows_per_expert, 2d] (bf16/fp16), of which only
 * the first masked_m[e] rows of expert e hold data (masked_m: device int32 [num_experts], values clamped to
 * [0, rows_per_expert]); output_q [num_experts, rows_per_expert, d], output_s [num_experts, rows_per_expert,
 * d/group_size] float32, both contiguous.  Rows beyond masked_m[e] are neither read nor written.
 * Replaces: silu_and_mul_masked_post_quant_fwd with scale_ue8m0=False
 *   (python/sglang/srt/layers/moe/ep_moe/kernels.py:287-420), the float32-scale form of the layout that
 *   sgl_per_token_group_quant_8bit_v2's MaskedLayoutScheduler walks
 *   (sgl-kernel/csrc/gemm/per_token_group_quant_8bit_v2.cu:194-238; that CUDA kernel is instantiated for UE8M0 scales
 *   only, :463-471, which this library does not produce).
 * At most 1024 experts per call.
 */
int sglb200_silu_and_mul_masked_quant_fp8(const void* input, int dtype, void* output_q, float* output_s,
                                          int num_experts, int64_t rows_per_expert, int64_t d, int group_size,
                                          float eps, const int32_t* masked_m, void* stream);

/*
 * Counting sort of flat topk_ids into block-padded expert segments; deterministic: within an expert,
 * entries keep ascending flat index.  Ids are shifted by +1 so that id -1 lands in bucket 0 and is
 * reported as expert -1; `num_experts` here is the bucket count, i.e. (model experts + 1), exactly
 * as the reference op is called.
 * Replaces: torch.ops.sgl_kernel.moe_align_block_size (sgl-kernel/csrc/moe/moe_align_kernel.cu:302-364,
 *   schema common_extension.cc:218-222; wrapper
 *   python/sglang/srt/layers/moe/fused_moe_triton/moe_align_block_size.py:17-82).
 * topk_ids [numel] int32; sorted_token_ids [numel + num_experts*(block_size-1)] int32;
 * expert_ids [ceil(that / block_size)] int32; num_tokens_post_pad [1] int32; cumsum_buffer [num_experts+1]
 * int32 (receives the padded exclusive prefix, as in the reference before its scatter).
 * workspace: device scratch of at least sglb200_moe_align_workspace_bytes(numel, num_experts) bytes, 4-byte
 * aligned (only 32-bit words are accessed); may be NULL when that function returns 0.  Contents need no
 * initialisation.
 * Entries of sorted_token_ids / expert_ids past num_tokens_post_pad are left untouched.
 */
int64_t sglb200_moe_align_workspace_bytes(int64_t numel, int num_experts);
int sglb200_moe_align_block_size(const int32_t* topk_ids, int64_t numel, int num_experts, int block_size,
                                 int32_t* sorted_token_ids, int32_t* expert_ids, int32_t* num_tokens_post_pad,
                                 int32_t* cumsum_buffer, int pad_sorted_token_ids, void* workspace,
                                 int64_t workspace_bytes, void* stream);

/*
 * Inputs of 2049 to 1 048 576 ids are sorted by ONE cooperative kernel (histogram, grid barrier, scatter).  Where
 * cooperative launches are not available (the device attribute is off, or the CTAs would not all be resident) the
 * same work runs as three ordinary launches; sglb200_moe_align_set_cooperative(0) forces that form, (1) restores
 * the default.  Process-wide; no counterpart in the reference, whose sort is always two launches
 * (sgl-kernel/csrc/moe/moe_align_kernel.cu:339-364).
 */
void sglb200_moe_align_set_cooperative(int on);

/*
 * moe_align_block_size for callers that cannot allocate device memory when they need the sort: code running
 * while a CUDA graph is being captured with the allocator frozen, a server whose memory pool is fully committed
 * to the KV cache, or a host program without torch's allocator.  No counterpart in the reference (its op always
 * receives a caller-allocated cumsum_buffer).  Same outputs as sglb200_moe_align_block_size; the scratch
 * (padded prefix + per-chunk histograms, about 0.5 MiB) is a fixed array inside the library image, resident on
 * every GPU that loads the library until the process exits.
 * Limits: num_experts (bucket count = experts + 1) <= 1024 and numel <= 1048576; larger calls are rejected with
 * SGLB200_E_INVALID and launch nothing.
 * The first call on each device resolves the array's device address (cudaGetSymbolAddress, with that device
 * current); make that first call before starting any stream capture.  All calls share the one array, which keeps
 * the previous call's contents (the kernels overwrite every word before reading it, so nothing needs clearing);
 * two calls that overlap on the GPU (different streams) race on it.  Calls cudaMalloc / cudaFree never.
 */
int sglb200_moe_align_block_size_noalloc(const int32_t* topk_ids, int64_t numel, int num_experts, int block_size,
                                         int32_t* sorted_token_ids, int32_t* expert_ids,
                                         int32_t* num_tokens_post_pad, int pad_sorted_token_ids, void* stream);

/*
 * Routing (the step before moe_align).  One row of `gating` [rows, num_experts] (dtype 0 bf16, 1 fp16, 2 fp32) per
 * token; outputs topk_weights [rows, topk] float32 and topk_ids [rows, topk] int32 in pick order (best first; equal
 * values: lower expert index first).  num_experts <= 1024.
 *
 * topk_softmax: v = x; if moe_softcapping != 0: v = tanh(v / cap) * cap; if correction_bias: v += bias[e];
 *   p = softmax(v); top-k of p; weights = p, divided by their sum when renormalize.
 *   Replaces torch.ops.sgl_kernel.topk_softmax (sgl-kernel/csrc/moe/moe_topk_softmax_kernels.cu:601-704,
 *   schema common_extension.cc:224-227).
 * topk_sigmoid: c = sigmoid(x) [+ bias[e]]; top-k of c; weights = c - bias[e] (as the reference reports them),
 *   divided by their sum when renormalize.  Replaces torch.ops.sgl_kernel.topk_sigmoid
 *   (sgl-kernel/csrc/moe/moe_topk_sigmoid_kernels.cu:60-170, schema common_extension.cc:229-232).
 * correction_bias: float32 [num_experts] or NULL.
 */
int sglb200_topk_softmax(const void* gating, int dtype, int64_t rows, int num_experts, int topk, int renormalize,
                         float moe_softcapping, const float* correction_bias, float* topk_weights, int32_t* topk_ids,
                         void* stream);
int sglb200_topk_sigmoid(const void* gating, int dtype, int64_t rows, int num_experts, int topk, int renormalize,
                         const float* correction_bias, float* topk_weights, int32_t* topk_ids, void* stream);

/*
 * DeepSeek-V3 grouped gate.  With T the dtype of `input` and `bias` (same dtype, bias [num_experts]):
 *   s = T(sigmoid(x)); b = T(s + bias); group score = T(sum of the group's two largest b); the topk_group groups with
 *   the largest score are kept (equal scores: lower group first); the (topk - num_fused_shared_experts) largest b of
 *   the kept groups are picked (equal: lower expert first); weights = s / sum(s of the picks), times
 *   routed_scaling_factor when apply_routed_scaling_factor_on_output.  Fused shared experts fill the last slots
 *   with ids num_experts, num_experts + 1, .. and weight 1 / routed_scaling_factor (times the factor when applied).
 * Replaces torch.ops.sgl_kernel.moe_fused_gate (sgl-kernel/csrc/moe/moe_fused_gate.cu:52-260, schema
 *   common_extension.cc:240-244).  Any group count <= 32 that divides num_experts (the reference wants powers of two
 *   and at most 32 experts per group).
 */
int sglb200_moe_fused_gate(const void* input, const void* bias, int dtype, int64_t rows, int num_experts,
                           int num_expert_group, int topk_group, int topk, int num_fused_shared_experts,
                           float routed_scaling_factor, int apply_routed_scaling_factor_on_output, float* topk_weights,
                           int32_t* topk_ids, void* stream);

/*
 * out[t, :] = bf16( scale * sum_k x[t, k, :] ), float32 accumulation in ascending k.
 * Replaces: torch.ops.sgl_kernel.moe_sum_reduce (sgl-kernel/csrc/moe/moe_sum_reduce.cu:56-116,
 *   schema common_extension.cc:234-235).  x [tokens, topk, hidden] contiguous, hidden % 8 == 0.
 */
int sglb200_moe_sum_reduce(const void* x, void* out, int dtype, int64_t tokens, int64_t topk, int64_t hidden,
                           float scale, void* stream);

/*
 * The same sum over the slots k with topk_ids[t, k] >= 0 only ([tokens, topk] int32, ids local to this rank): under
 * expert parallelism the slots of experts that live on other ranks are never written and are skipped here instead
 * of being zero-filled and read.  The reference reaches the same result by writing zeros for filtered experts
 * (python/sglang/srt/layers/moe/fused_moe_triton/fused_moe_triton_kernels.py:421-437) and summing every slot.
 */
int sglb200_moe_sum_reduce_masked(const void* x, const int32_t* topk_ids, void* out, int dtype, int64_t tokens,
                                  int64_t topk, int64_t hidden, float scale, void* stream);

/*
 * Removes the leading segment of filtered ids (bucket 0 = expert -1, the experts of other ranks) from the outputs of
 * sglb200_moe_align_block_size: sorted_out / expert_ids_out / post_out describe only the rows of local experts, in the
 * same order.  cumsum = the cumsum_buffer written by the sort (cumsum[1] is the padded length of bucket 0).  Outputs must
 * not alias inputs; max_rows bounds the entries of sorted_in.  The reference keeps the segment and lets its GEMM
 * kernel write zeros for it (fused_moe_triton_kernels.py:421-437); dropping it keeps every row of a foreign expert out
 * of the gather, both GEMMs and the activation kernel.
 */
int sglb200_moe_align_drop_filtered(const int32_t* sorted_in, const int32_t* expert_ids_in, const int32_t* cumsum,
                                    const int32_t* post_in, int32_t* sorted_out, int32_t* expert_ids_out,
                                    int32_t* post_out, int64_t max_rows, int block_size, void* stream);

/*
 * Combine step of the expert-parallel layer: out[t, :] = T( scale * sum_j src[slot[t, j], :] ), float32 accumulation in
 * ascending j; entries of `slot` [tokens, per_token] (int64) outside [0, src_rows) contribute nothing.  Replaces the
 * per-rank gather-and-add that follows `buffer.combine` in the reference's DeepEP dispatcher
 * (python/sglang/srt/layers/moe/token_dispatcher/deepep.py:502-509) for the NCCL all-to-all form used here.
 * src [src_rows, hidden], out [tokens, hidden], dtype 0 bf16 / 1 fp16, hidden % 8 == 0.
 */
int sglb200_gather_sum_rows(const void* src, const int64_t* slot, void* out, int dtype, int64_t tokens, int per_token,
                            int64_t src_rows, int64_t hidden, float scale, void* stream);

/*
 * output[t, :] = T( sum_j factors[t * topk + j] * input[permutation[t * topk + j], :] ), float32 accumulation in
 * ascending j; `factors` (same dtype as the data) may be NULL (= 1).  Replaces torch.ops.sgl_kernel.apply_shuffle_mul_sum
 * (sgl-kernel/csrc/moe/prepare_moe_input.cu:258-392, schema common_extension.cc:267-268), the combine of the
 * reference's CUTLASS MoE path (python/sglang/srt/layers/moe/cutlass_moe.py).  input [tokens * topk, hidden],
 * output [tokens, hidden], dtype 0 bf16 / 1 fp16, hidden % 8 == 0.
 */
int sglb200_shuffle_mul_sum(const void* input, void* output, const int32_t* permutation, const void* factors, int dtype,
                            int64_t tokens, int topk, int64_t hidden, void* stream);

/*
 * Row gather into expert-sorted order: for r < *num_rows_dev,
 *   src = sorted_token_ids[r]; if src < numel: dst_q[r,:] = src_q[src / topk, :], dst_s[r,:] = src_s[src / topk, :]
 *   else (padding) the row and its scales are zero-filled.
 * Replaces: torch.ops.sgl_kernel.shuffle_rows (sgl-kernel/csrc/moe/prepare_moe_input.cu:170-197) as used by
 *   cutlass_fused_experts_fp8 (python/sglang/srt/layers/moe/cutlass_moe.py:153-154), and the in-kernel row
 *   gather of fused_moe_kernel (fused_moe_triton_kernels.py:410-416,450-460).
 * src_q [tokens, hidden] 1-byte elements, hidden % 16 == 0; src_s [tokens, groups] float32.
 */
int sglb200_gather_rows_fp8(const void* src_q, const float* src_s, void* dst_q, float* dst_s,
                            const int32_t* sorted_token_ids, const int32_t* num_rows_dev, int64_t max_rows,
                            int64_t numel, int topk, int64_t hidden, int64_t groups, void* stream);

/*
 * Dense block-scaled GEMM:  C[m,n] = bf16( sum_kb a_s[m,kb] * b_s[n/128, kb] * sum_{k in kb} A[m,k] * B[n,k] ),
 * float32 accumulation, 1x128 activation scales, 128x128 weight-block scales.
 * Replaces: torch.ops.sgl_kernel.fp8_blockwise_scaled_mm
 *   (sgl-kernel/csrc/gemm/fp8_blockwise_gemm_kernel.cu:368-465, schema common_extension.cc:133-136) and
 *   w8a8_block_fp8_matmul (python/sglang/srt/layers/quantization/fp8_kernel.py:1072-1168, Triton kernel :695-777).
 * A [M,K] e4m3 row-major; B [N,K] e4m3 row-major (the checkpoint layout of `weight`);
 * a_s element (m,kb) at a_s[m*as_stride_m + kb*as_stride_k]; b_s [ceil(N/128), ceil(K/128)] row-major;
 * C [M,N] row-major, out_dtype 0 = bf16, 1 = fp16.  K % 16 == 0, K <= 65536, N % 8 == 0; A, B, C 16-byte aligned.
 * bias (optional, may be NULL): [N] of out_dtype, added in float32 before the final rounding.
 * workspace: only used for the split-K path chosen for small M; at least
 * sglb200_gemm_workspace_bytes(M,N,K) bytes (0 means none needed).
 */
int64_t sglb200_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K);
int sglb200_fp8_blockwise_scaled_mm(const void* A, const void* B, const float* a_s, const float* b_s, void* C,
                                    const void* bias, int64_t M, int64_t N, int64_t K, int64_t as_stride_m,
                                    int64_t as_stride_k, int out_dtype, void* workspace, int64_t workspace_bytes,
                                    void* stream);

/*
 * Grouped (MoE) block-scaled GEMM over expert-sorted rows.  For every 128-row block b < *num_rows_dev / 128,
 * e = expert_ids[b]:  acc[r, n] = blockscaled( A[r, :], B[e, n, :] ) for the block's rows r.
 *   e == -1  -> the block contributes zeros.
 * Output modes:
 *   scatter == 0: C[r, n] = bf16(acc)                       (C is [max_rows, N], expert-sorted order)
 *   scatter == 1: id = sorted_token_ids[r]; if id < numel:
 *                 C[id, n] = bf16( acc * (row_weights ? row_weights[id] : 1) )   (C is [numel, N], token-major)
 * Replaces: fused_moe_kernel via invoke_fused_moe_kernel
 *   (python/sglang/srt/layers/moe/fused_moe_triton/fused_moe_triton_kernels.py:307-583, 586-790) and
 *   torch.ops.sgl_kernel.fp8_blockwise_scaled_grouped_mm (sgl-kernel/csrc/moe/fp8_blockwise_moe_kernel.cu:650-810).
 * A [max_rows, K] e4m3 (rows already in sorted order), a_s [max_rows, K/128] row-major,
 * B [E, N, K] e4m3, b_s [E, ceil(N/128), ceil(K/128)], block size of the sort must be 128.  K % 16 == 0, K <= 65536,
 * N % 8 == 0.
 */
int sglb200_fp8_blockwise_grouped_mm(const void* A, const float* a_s, const void* B, const float* b_s, void* C,
                                     const int32_t* sorted_token_ids, const int32_t* expert_ids,
                                     const int32_t* num_rows_dev, const float* row_weights, int64_t max_rows,
                                     int64_t numel, int num_experts, int64_t N, int64_t K, int scatter, int out_dtype,
                                     void* stream);

/*
 * Health of the GEMM pipelines: 0, or 1 if a bounded mbarrier wait inside a GEMM kernel expired since the
 * library was loaded (the kernel then unwinds, frees its tensor memory and leaves its output incomplete).
 * Synchronises the device.  Stands in for the C++ exception a failed CUTLASS launch raises in
 * sgl-kernel/csrc/gemm/fp8_blockwise_gemm_kernel.cu:164-171.
 */
int sglb200_gemm_status(void);
/* Sets the status word back to 0 on the current device (after the failure has been handled).  Synchronises. */
int sglb200_gemm_status_clear(void);

/*
 * Diagnostic knob of the GEMM kernels' pipeline waits (each a bounded run of barrier probes, seconds at most):
 * UINT32_MAX makes every wait give up at once, so that a healthy GEMM gives up before it has loaded anything, which
 * exercises the give-up path (status word, drain, tensor-memory release) without any fault; any other value
 * restores the normal limit.  Applies to GEMMs launched afterwards by this process.  No counterpart in the
 * reference.
 */
void sglb200_gemm_set_wait_probes(uint32_t probes);

/*
 * Health of the streaming kernels (the quantizer and the fused silu_and_mul + quantizer stage their input
 * through shared memory with bulk copies that complete on mbarriers): 0, or 1 if a bounded wait for a staged
 * tile expired since the library was loaded (the CTA then returns and leaves its output incomplete).
 * Synchronises the device.  Stands in for the CUDA error a failed run of the reference's quantizer launcher
 * (sgl-kernel/csrc/gemm/per_token_group_quant_8bit.cu:116-217) would surface at the next synchronisation.
 */
int sglb200_stream_status(void);
int sglb200_stream_status_clear(void); /* back to 0 on the current device; synchronises */

/*
 * Number of barrier probes (a few microseconds each) after which a streaming kernel gives up waiting for a staged
 * tile; 0 restores the default (seconds); UINT32_MAX makes every wait give up at once.  A diagnostic knob like
 * sglb200_gemm_set_wait_probes: with UINT32_MAX a healthy call gives up before its first tile has landed, sets the
 * status word and returns after its copies in flight have landed.  No counterpart in the reference.
 */
void sglb200_stream_set_wait_probes(uint32_t probes);

/*
 * Fused row-parallel all-reduce (tensor-parallel o_proj / down): the sum over ranks of a row-parallel layer as a
 * two-shot all-reduce whose reduce-scatter is folded into the GEMM epilogue.
 * Replaces, for RowParallelLinear.forward (python/sglang/srt/layers/linear.py:1365-1393): the block GEMM followed
 * by tensor_model_parallel_all_reduce (python/sglang/srt/distributed/parallel_state.py:544-623), i.e. the
 * reference's NCCL / custom all-reduce (sgl-kernel/csrc/allreduce/custom_all_reduce.cuh) after the matmul.
 *
 * Peer buffers are plain device allocations shared with CUDA IPC handles (one process per GPU, one node):
 *   sglb200_comm_alloc       zero-filled device memory for a buffer peers will touch (set-up time; synchronises)
 *   sglb200_comm_ipc_export  64-byte handle of such a buffer, to be sent to the other ranks by any host channel
 *   sglb200_comm_ipc_open    maps a peer's buffer into this process; sglb200_comm_ipc_close unmaps it
 *   sglb200_comm_flag_bytes  size of the flag buffer each rank must provide (zero-filled once)
 *
 * Output rows are owned in blocks of rpo = sglb200_push_rows_per_owner(M, world) rows (M / world rounded up to whole
 * 128-row tiles): rank d owns rows [d * rpo, min((d + 1) * rpo, M)), possibly none for the last ranks.
 * sglb200_fp8_blockwise_scaled_mm_push: the dense block GEMM of this rank's K slice; output tile rows [m0, m0+128) go
 *   to rank m0 / rpo's staging buffer, block `rank`, instead of to a local C.  stage_ptrs: HOST array of `world`
 *   device pointers, entry d = rank d's staging buffer [world][rpo][N] of out_dtype as mapped in THIS process.  The
 *   first call for a given set of buffers and shape allocates and fills a small device table (do it before any
 *   stream capture).
 * sglb200_reduce_gather: after the push GEMM on the same stream.  Waits (bounded) until every rank's GEMM has
 *   finished, sums the `world` blocks of this rank's staging buffer in rank order in float32 into
 *   reduced_ptrs[rank] ([rpo][N]) and `out`, waits for the other ranks, then copies their reduced rows from
 *   reduced_ptrs[peer] into `out` [M][N] (private memory of this rank).  flag_ptrs[d] = rank d's flag buffer.
 *   The call's epoch (the value the flag words are compared with) is counted on the device, per block, in this
 *   rank's own flag buffer, so a CUDA graph that replays the call sees a new epoch at every replay.  Every rank must
 *   make the same sequence of calls (with the same `max_blocks`).  sglb200_comm_status() is 1 after a wait
 *   for a peer expired (the kernel then returns without touching peer data; the output is incomplete; the next
 *   well-formed call works again).
 *   Pipelining over row chunks: `sm_margin` SMs are left free by the push GEMM and `max_blocks` (> 0; the same on
 *   every rank) caps the CTAs of sglb200_reduce_gather, so that the reduce-and-gather of chunk c (issued on a second
 *   stream, on its own slices of the buffers) runs beside the GEMM of chunk c + 1.  0 / 0 = no pipelining.
 * sglb200_comm_set_wait_probes: probes (about 0.25 us each) after which a wait for a peer's flag gives up; 0 restores
 *   the default (about a second).  A diagnostic knob: with a small limit and a peer that never arrives the kernel
 *   returns within milliseconds with the status word set.
 */
int sglb200_comm_alloc(int64_t bytes, void** out);
int sglb200_comm_free(void* p);
int sglb200_comm_ipc_export(void* p, void* handle64);
int sglb200_comm_ipc_open(const void* handle64, void** out);
int sglb200_comm_ipc_close(void* p);
int64_t sglb200_comm_flag_bytes(void);
int sglb200_comm_status(void);
int sglb200_comm_status_clear(void); /* back to 0 on the current device; synchronises */
void sglb200_comm_set_wait_probes(uint32_t probes);
int64_t sglb200_push_rows_per_owner(int64_t M, int world);
/* Builds (and keeps) the device table of tensor maps that sglb200_fp8_blockwise_scaled_mm_push needs for outputs of
 * M x N through these staging buffers: the small allocation and synchronous copy of a shape's first push call, done
 * at set-up time instead.  No counterpart in the reference. */
int sglb200_push_prepare(void* const* stage_ptrs, int world, int64_t M, int64_t N, int out_dtype);
int sglb200_fp8_blockwise_scaled_mm_push(const void* A, const void* B, const float* a_s, const float* b_s,
                                         void* const* stage_ptrs, int world, int rank, int64_t M, int64_t N, int64_t K,
                                         int64_t as_stride_m, int64_t as_stride_k, int out_dtype, int sm_margin,
                                         void* stream);
int sglb200_reduce_gather(const void* stage, void* const* reduced_ptrs, void* const* flag_ptrs, void* out, int world,
                          int rank, int64_t M, int64_t N, int dtype, int max_blocks, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SGLANG_B200_H_ */
