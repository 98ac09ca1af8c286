/* C ABI of the sm_100a CUDA backend (libbaremetal_b200.so).
 *
 * This is the layer that sits where the reference has src/backend/backend.h + its Metal shaders:
 * the C11 host code (trainer, model, optimizer state) calls these entry points and nothing else
 * to reach the GPU. Where the reference dispatches a kernel *by name* with a buffer list and
 * Metal grid sizes (backend_encode_dispatch, src/backend/backend.h:55-62), this ABI has one typed
 * entry point per operation: plain device pointers, explicit shapes and leading dimensions,
 * an int status. Launch geometry is chosen inside the backend.
 *
 * Conventions
 *  - every pointer argument named d_* is DEVICE memory obtained from bmc_alloc();
 *  - `dtype` is the activation storage type (BMC_F32 or BMC_BF16); arithmetic is fp32 either way.
 *    With BMC_BF16 the matmul entry points run on the tcgen05 tensor cores and expect bf16
 *    weights; with BMC_F32 they run fp32 FFMA and expect fp32 weights;
 *  - all work is enqueued on the context's compute stream; nothing blocks except bmc_sync(),
 *    bmc_download() and bmc_status();
 *  - return value 0 = enqueued, <0 = rejected (bad shape/alignment, missing device). There is no
 *    CPU fallback: without a usable CUDA device bmc_create() returns NULL.
 */
#ifndef BM_CUDA_BACKEND_H
#define BM_CUDA_BACKEND_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct bmc_ctx_s bmc_ctx_t;

enum { BMC_F32 = 0, BMC_BF16 = 1 };

/* ---- context, memory, transfers (replace backend_create/destroy, backend_buffer_alloc/free/map/unmap,
 *      backend_encode_wait: src/backend/backend.h:17-18,40-44,65-66) ---- */
bmc_ctx_t* bmc_create(int device_ordinal);
void       bmc_destroy(bmc_ctx_t* ctx);
void*      bmc_alloc(bmc_ctx_t* ctx, size_t bytes);            /* NULL when bytes == 0 or out of memory */
void       bmc_free(bmc_ctx_t* ctx, void* d_ptr);
size_t     bmc_allocated_bytes(bmc_ctx_t* ctx);               /* backend_get_allocated_memory, backend.h:19 */
size_t     bmc_peak_allocated_bytes(bmc_ctx_t* ctx);          /* backend_get_peak_allocated_memory, backend.h:20 */
int        bmc_upload(bmc_ctx_t* ctx, void* d_dst, const void* h_src, size_t bytes);    /* async H2D on the compute stream */
int        bmc_download(bmc_ctx_t* ctx, void* h_dst, const void* d_src, size_t bytes);  /* D2H, returns after the copy */
int        bmc_memset(bmc_ctx_t* ctx, void* d_ptr, int byte_value, size_t bytes);
/* Second stream of the context. Calls between bmc_side_begin and bmc_side_end are enqueued on it, ordered after everything the main
 * stream holds at bmc_side_begin, and may run concurrently with later main-stream work (the trainer puts weight-gradient GEMMs there
 * so that they overlap the memory-bound kernels of the backward chain). bmc_side_end returns a ticket (0..15, reused round-robin: at
 * most 16 may be outstanding) or a negative code; bmc_side_wait makes later main-stream work wait for the side work up to the ticket.
 * bmc_sync waits for both streams. No reference counterpart: the reference encodes one command buffer at a time. */
int        bmc_side_begin(bmc_ctx_t* ctx);
int        bmc_side_end(bmc_ctx_t* ctx);
int        bmc_side_wait(bmc_ctx_t* ctx, int ticket);
int        bmc_copy(bmc_ctx_t* ctx, void* d_dst, const void* d_src, size_t bytes);
int        bmc_sync(bmc_ctx_t* ctx);                          /* waits for the compute stream; returns bmc_status() */
/* Non-zero when a kernel reported a failed bounded wait or a CUDA call failed since the last call. */
int        bmc_status(bmc_ctx_t* ctx);
/* Self-test of the bounded waits: enqueues a one-CTA kernel that waits (2 ms limit) on a barrier nothing arrives at. The kernel gives
 * up, leaves code 1999 in the error word and returns; the next bmc_status() / bmc_sync() reports 1999 once and the context stays
 * usable. No counterpart in the reference (its Metal kernels have no device-side waits). */
int        bmc_selftest_bounded_wait(bmc_ctx_t* ctx);
void*      bmc_stream(bmc_ctx_t* ctx);                        /* the cudaStream_t work is enqueued on */
/* Kernel launches issued through this context since creation (all entry points). */
long       bmc_launch_count(bmc_ctx_t* ctx);
/* Pinned host memory for staging step inputs. */
void*      bmc_host_alloc(size_t bytes);
/* A value the host needs before the stream has drained (the loss of a training step, known after the forward pass): _readback
 * enqueues a copy of *d_value and of the error word to pinned memory plus an event behind them (capturable: inside a CUDA graph the
 * event is an external event node); _wait blocks until that point of the stream has been reached. */
int        bmc_early_readback(bmc_ctx_t* ctx, const float* d_value);
int        bmc_early_wait(bmc_ctx_t* ctx, float* value_out, int* status_out);
void       bmc_host_free(void* p);
/* GPU-side phase timing (replaces backend_encode_wait_timed / backend_get_gpu_busy_ms, backend.h:32-37):
 * bmc_timer_begin/end bracket work on the compute stream with events; end returns elapsed ms (blocking). */
int        bmc_timer_begin(bmc_ctx_t* ctx, int slot);
float      bmc_timer_end(bmc_ctx_t* ctx, int slot);

/* Per-launch timing of the tensor-core GEMM kernel: while enabled every launch is bracketed by CUDA events on the
 * compute stream. collect() waits for the stream and returns out[0] = launches, out[1] = summed kernel time in ms,
 * out[2] = summed algorithmic FLOPs (2*M*N*K) since enable/collect. (The reference accumulates whole-command-buffer
 * GPU time instead: backend_get_gpu_busy_ms, src/backend/backend.h:32-34.) */
int        bmc_gemm_timing(bmc_ctx_t* ctx, int enable);
int        bmc_gemm_timing_collect(bmc_ctx_t* ctx, double* out3);

/* ---- embedding (embed_lookup src/baremetal/trainer.c:275-298; embedding_backward src/kernels/backward.metal:636) ---- */
/* V = rows of the table. A token id outside [0, V) is never used as an index: the gathered row is zero, the scatter skips it, and
 * bmc_status() reports 2001 afterwards. */
int bmc_embedding_forward(bmc_ctx_t* ctx, int dtype, void* d_out, const float* d_table_f32, const int* d_tokens, int n_tok, int D, int V);
int bmc_embedding_backward(bmc_ctx_t* ctx, int dtype, float* d_gwte_f32, const void* d_gout, const int* d_tokens, int n_tok, int D, int V);

/* ---- RMSNorm (rmsnorm_forward forward.metal:993; rmsnorm_backward_x / _w backward.metal:340,379) ----
 * forward also stores 1/rms per row in d_rstd (may be NULL).
 * backward: d_gx += dL/dx (accumulates, like the reference kernel); d_gw_f32[j] (+)= sum over rows
 * [w_row0, w_row1) of gout*x*rstd — the row window lets a caller reproduce the reference's
 * "last sequence only" weight gradient (backward.metal:400 overwrites per sequence) or the full sum. */
int bmc_rmsnorm_forward(bmc_ctx_t* ctx, int dtype, void* d_out, float* d_rstd, const void* d_x, const float* d_w, int N, int C, float eps);
int bmc_rmsnorm_backward(bmc_ctx_t* ctx, int dtype, void* d_gx, float* d_gw_f32, int gw_accumulate, const void* d_gout, const void* d_x,
                         const float* d_w, const float* d_rstd, int N, int C, int w_row0, int w_row1);

/* RMSNorm backward without any allocation — no counterpart in the reference (its backend allocates buffers freely and
 * has no such variant). Same arithmetic and arguments as bmc_rmsnorm_backward, but it takes the raw cudaStream_t to
 * enqueue on instead of a context, and its partial-sum scratch is a fixed array inside the library (about 2.3 MiB per
 * GPU, held until exit). For hosts that own all device memory themselves or must never hit the implicit device
 * synchronisation of cudaMalloc/cudaFree in steady state. C must be <= BMC_STATIC_RMS_MAX_C, otherwise
 * BMC_ERR_STATIC_TOO_LARGE is returned and nothing is enqueued. All calls on a GPU share the scratch: do not let two of
 * them overlap on the device. The first call on a device resolves the scratch address; make it before any stream capture. */
#define BMC_STATIC_RMS_MAX_C 1024
#define BMC_ERR_STATIC_TOO_LARGE (-60)
int bmc_rmsnorm_backward_static(void* cuda_stream, int dtype, void* d_gx, float* d_gw_f32, int gw_accumulate, const void* d_gout,
                                const void* d_x, const float* d_w, const float* d_rstd, int N, int C, int w_row0, int w_row1);

/* ---- linear layers (matmul_forward_* forward.metal:176,449; matmul_backward_inp_* backward.metal:122,174;
 *      matmul_backward_w_tiled backward.metal:277). Weight is row-major [OC, C] in the activation dtype.
 *   forward : out[BT,OC] = inp[BT,C] * W^T (+ residual[BT,OC] when d_residual != NULL)
 *   backward_inp : ginp[BT,C] = gout[BT,OC] * W         (overwrites; pass accumulate=1 for the reference's +=)
 *   backward_w   : gw_f32[OC,C] += gout^T * inp          (always accumulates, fp32, like the reference) ---- */
int bmc_matmul_forward(bmc_ctx_t* ctx, int dtype, void* d_out, int ldo, const void* d_inp, int ldi, const void* d_weight,
                       const void* d_residual, int ldr, int BT, int C, int OC);
int bmc_matmul_backward_inp(bmc_ctx_t* ctx, int dtype, void* d_ginp, int ldgi, int accumulate, const void* d_gout, int ldgo,
                            const void* d_weight, int BT, int C, int OC);
int bmc_matmul_backward_w(bmc_ctx_t* ctx, int dtype, float* d_gw_f32, const void* d_gout, int ldgo, const void* d_inp, int ldi,
                          int BT, int C, int OC);

/* ---- linear layers that absorb the memory-bound kernel next to them (bf16 / tensor-core path). Each returns BMC_ERR_UNFUSED
 *      without enqueuing anything when the dtype or the shape has no fused form; the caller then uses the separate entry points.
 *   swiglu_forward      : [gate | up][BT, 2H] = inp[BT,C] * [W_gate; W_up]^T  and  act[BT,H] = silu(gate) * up in the same launch
 *                         (matmul_forward_* followed by swiglu_forward, forward.metal:1179). d_w_gate_up: [2H, C], gate rows first.
 *                         H % 128 == 0.
 *   backward_inp_swiglu : [dgate | dup][BT, 2H] from gout[BT,OC] * W_down[OC,H] and the saved [gate | up]; the intermediate
 *                         dact[BT,H] is never stored (matmul_backward_inp_* followed by swiglu_backward, backward.metal:505).
 *   backward_inp_rowdot : ginp[BT,C] = gout[BT,OC] * W[OC,C]  and  rowdot[b][h][s] = sum over the 64 columns of head h of
 *                         ginp[row,:] * other[row,:], row = b*S + s — the per-row sums attention backward subtracts from dP
 *                         when ginp is the gradient of the attention output and `other` that output. C == NH * 64. ---- */
#define BMC_ERR_UNFUSED (-70)
int bmc_matmul_swiglu_forward(bmc_ctx_t* ctx, int dtype, void* d_gate_up, int ldgu, void* d_act, int ldact, const void* d_inp, int ldi,
                              const void* d_w_gate_up, int BT, int C, int H);
int bmc_matmul_backward_inp_swiglu(bmc_ctx_t* ctx, int dtype, void* d_dgate_dup, int lddgu, const void* d_gout, int ldgo,
                                   const void* d_w_down, const void* d_gate_up, int ldgu, int BT, int H, int OC);
int bmc_matmul_backward_inp_rowdot(bmc_ctx_t* ctx, int dtype, void* d_ginp, int ldgi, float* d_rowdot, const void* d_gout, int ldgo,
                                   const void* d_weight, const void* d_other, int ldother, int BT, int C, int OC, int S, int NH);

/* ---- RoPE (rope_forward_seq forward.metal:2225; rope_backward_seq backward.metal:980), in place.
 * d_cs_table: float[S][HD/2][2] = (cos, sin)(pos * inv_freq), built by the host with the reference's formula
 * (rope_inv_freq forward.metal:1260-1279). rows = B*S, position = row % S. dir: +1 forward, -1 backward. ---- */
int bmc_rope(bmc_ctx_t* ctx, int dtype, void* d_q, int ldq, void* d_k, int ldk, const float* d_cs_table, int rows, int S, int NH,
             int NKV, int HD, int dir);

/* ---- causal GQA attention (attention_forward_seq / _train_tiled forward.metal:1811,2122;
 *      attention_backward / _tiled backward.metal:665,820). Q[row,h,:] at d_q + row*ldq + h*HD, K and V
 *      likewise with NKV heads and pitch ldkv; row = b*S + s. d_lse: float[B][NH][S] log-sum-exp saved
 *      by forward for backward. d_mask (uint8[B*S], may be NULL): 0 excludes that position as key and query.
 *      backward overwrites d_gq and d_gk/d_gv (all in the activation dtype, same pitches as q / kv). ---- */
int bmc_attention_forward(bmc_ctx_t* ctx, int dtype, void* d_out, int ldo, float* d_lse, const void* d_q, int ldq, const void* d_k,
                          const void* d_v, int ldkv, const uint8_t* d_mask, int B, int S, int NH, int NKV, int HD, float scale);
int bmc_attention_backward(bmc_ctx_t* ctx, int dtype, void* d_gq, int ldgq, void* d_gk, void* d_gv, int ldgkv, const void* d_gout,
                           int ldo, const void* d_out, const float* d_lse, const void* d_q, int ldq, const void* d_k, const void* d_v,
                           int ldkv, const uint8_t* d_mask, int B, int S, int NH, int NKV, int HD, float scale);
/* Same, with the two passes that surround it in the training step folded in (both optional, NULL = off):
 *   d_delta   float[B][NH][S] = rowsum(gout * out) computed elsewhere (bmc_matmul_backward_inp_rowdot), so it is not recomputed;
 *   d_rope_cs the rotation table of bmc_rope: d_gq and d_gk leave with RoPE backward (rope_backward_seq, backward.metal:980)
 *             already applied, which saves a read-modify-write pass over both. */
int bmc_attention_backward_fused(bmc_ctx_t* ctx, int dtype, void* d_gq, int ldgq, void* d_gk, void* d_gv, int ldgkv, const void* d_gout,
                                 int ldo, const void* d_out, const float* d_lse, const void* d_q, int ldq, const void* d_k, const void* d_v,
                                 int ldkv, const uint8_t* d_mask, const float* d_delta, const float* d_rope_cs, int B, int S, int NH, int NKV,
                                 int HD, float scale);

/* ---- SwiGLU (swiglu_forward forward.metal:1179; swiglu_backward backward.metal:505) ---- */
int bmc_swiglu_forward(bmc_ctx_t* ctx, int dtype, void* d_out, int ldo, const void* d_gate, const void* d_up, int ldgu, int rows, int H);
int bmc_swiglu_backward(bmc_ctx_t* ctx, int dtype, void* d_ggate, void* d_gup, int ldg, const void* d_gate, const void* d_up, int ldgu,
                        const void* d_gout, int ldo, int rows, int H);
/* residual add (add_forward forward.metal:1332) */
int bmc_add_forward(bmc_ctx_t* ctx, int dtype, void* d_out, const void* d_a, const void* d_b, size_t n);

/* ---- loss (host loss loop src/baremetal/scheduler.c:1622-1634 + xent_backward backward.metal:567, masked :597).
 * Overwrites logits with (softmax - onehot) * grad_scale, writes per-row losses, then reduces them to
 * *d_loss = mean over B sequences of the per-sequence mean (src/baremetal/trainer.c:528). ---- */
/* d_row_weight (float[B*S], may be NULL) selects the completion-only form: the weight of a row is 1 / (unmasked rows of its
 * sequence) or 0 for a masked row, and replaces grad_scale; the loss is then the batch mean of the per-sequence weighted sums. */
int bmc_xent(bmc_ctx_t* ctx, int dtype, void* d_logits, int ldv, float* d_row_loss, float* d_loss, const int* d_targets,
             const float* d_row_weight, int B, int S, int V, float grad_scale);

/* ---- AdamW over a flat parameter range (adamw_step src/anneal/adamw.metal:26 + the host recast loop
 *      src/baremetal/trainer.c:373-396). hp (HOST pointer, 8 floats) = {lr, b1, b2, eps, wd, 1-b1^t, 1-b2^t, grad_scale}.
 *      grad_dtype: BMC_F32 or BMC_BF16. d_w_bf16 (may be NULL) receives the bf16 working copy. ---- */
int bmc_adamw(bmc_ctx_t* ctx, float* d_w, void* d_w_bf16, const void* d_g, int grad_dtype, float* d_m, float* d_v, size_t n,
              const float* h_hp);
int bmc_cast_f32_to_bf16(bmc_ctx_t* ctx, void* d_out_bf16, const float* d_in, size_t n);
int bmc_cast_bf16_to_f32(bmc_ctx_t* ctx, float* d_out, const void* d_in_bf16, size_t n);
/* x[b] <- carry + x[0] + .. + x[b] over the B sequences of a batch (per_seq elements each), carry <- last sum.
 * Reference-compatibility helper: the reference's layer-0 input gradient is never cleared between the sequences
 * of an optimizer window (src/baremetal/scheduler.c:263-266, src/baremetal/trainer.c:459-470). */
int bmc_seq_prefix_accumulate(bmc_ctx_t* ctx, int dtype, void* d_x, float* d_carry_f32, int B, size_t per_seq);
/* greedy sampler: lowest index among the maxima (bm_sample argmax branch src/baremetal/sampler.c:36-40) */
int bmc_argmax(bmc_ctx_t* ctx, int* d_index, const float* d_logits, int V);

/* ---- token-by-token inference (decode walk src/baremetal/scheduler.c:712-996; kernels matmul_forward_q8_vec forward.metal:575,
 *      rmsnorm_forward_v2 :1019, rope_forward :1284, kv_store :1317, attention_forward :1362, swiglu_forward :1179), batched over
 *      NB independent sequences that share one position counter. Activations are fp32; the KV cache holds fp32 elements
 *      (cache_dtype BMC_F32: what the reference keeps, scheduler.c kv buffers) or, on request, bf16 (BMC_BF16, head_dim 64).
 *      Weight types: BMC_W_Q8 = int8 q[OC][C] + float scale[OC][C/32] (the values of the reference's 36-byte blocks,
 *      src/baremetal/quant.h:19-22, stored as two arrays), BMC_W_BF16, BMC_W_F32, BMC_W_Q4 = uint8 qs[OC][C/2] + float
 *      scale[OC][C/32] (the reference's 20-byte blocks, quant.h:39-42, as two arrays: element 2j of a row in the low and 2j+1 in
 *      the high nibble of byte j, two's-complement codes in [-8, 7]). Any other value is refused (-1).
 *      d_pos is a DEVICE int holding the position of the token being processed (so a captured step can be replayed).
 *      KV cache layout: element[L][2][NB][MS][KV]; rope table float[MS][HD/2][2]. ---- */
enum { BMC_W_Q8 = 0, BMC_W_BF16 = 1, BMC_W_F32 = 2, BMC_W_Q4 = 3 };
int bmc_decode_gemv(bmc_ctx_t* ctx, float* d_out, int ldo, const float* d_x, int ldx, int wtype, const void* d_w, const float* d_scales,
                    const float* d_residual, int ldr, int NB, int C, int OC);
/* The same product with a prologue folded into the operand load (single-sequence kernel, C <= 3072):
 *   prologue 1: RMSNorm(x) * d_norm_weight (rmsnorm_forward_v2 followed by the matmul, as the reference's fused
 *               rmsnorm_matmul_forward does for the classifier, src/kernels/forward.metal);
 *   prologue 2: d_x rows are [gate | up] (2C wide) and the operand is silu(gate) * up (swiglu_forward, forward.metal:1179). */
int bmc_decode_gemv_fused(bmc_ctx_t* ctx, float* d_out, int ldo, const float* d_x, int ldx, int wtype, const void* d_w, const float* d_scales,
                          const float* d_residual, int ldr, int prologue, const float* d_norm_weight, float eps, int NB, int C, int OC);
int bmc_decode_rmsnorm(bmc_ctx_t* ctx, float* d_out, const float* d_x, const float* d_w, int NB, int C, float eps);
int bmc_decode_rope_kv(bmc_ctx_t* ctx, float* d_qkv, void* d_cache, int cache_dtype, const float* d_cs_table, const int* d_pos, int layer, int NB, int MS,
                       int NH, int NKV, int HD);
/* d_scratch: NULL (one block per sequence and KV head walks every position) or a buffer of bmc_decode_attention_scratch_bytes(),
 * zeroed once by the caller, which lets the positions be split over several blocks that merge their softmax partials. */
size_t bmc_decode_attention_scratch_bytes(int NB, int MS, int NH, int NKV, int HD);
int bmc_decode_attention(bmc_ctx_t* ctx, float* d_out, const float* d_qkv, const void* d_cache, int cache_dtype, const int* d_pos, void* d_scratch, int layer,
                         int NB, int MS, int NH, int NKV, int HD, float scale);
/* rope_forward + kv_store + attention_forward in one kernel: d_qkv holds the raw projections and is left untouched */
int bmc_decode_attention_fused(bmc_ctx_t* ctx, float* d_out, const float* d_qkv, void* d_cache, int cache_dtype, const float* d_cs_table, const int* d_pos,
                               void* d_scratch, int layer, int NB, int MS, int NH, int NKV, int HD, float scale);
/* Tensor-core products with fp32-accurate results, for many rows (batched decode, prefill). bmc_decode_prep splits the fp32 operand
 * rows (mode 0 = x, 1 = RMSNorm(x) * weight, 2 = silu(gate) * up of [gate | up] rows) into bf16 [hi | lo] (parts 2) or [hi | lo | hi]
 * (parts 3) and sets the fp32 output rows to d_init_src rows or zero; bmc_decode_gemm accumulates a x w^T into them, where w holds
 * [w | w] (parts 2: weights exactly representable in bf16) or [w_hi | w_hi | w_lo] (parts 3) per output row. Same arithmetic
 * as matmul_forward_q8 / _bf16 / _naive (src/kernels/forward.metal:625,52,23) to ~2^-17 relative. */
int bmc_decode_prep(bmc_ctx_t* ctx, void* d_a, int parts, const float* d_x, int ldx, int mode, const float* d_norm_weight, float eps,
                    float* d_init_out, int ldo, const float* d_init_src, int ldr, int n_out, int rows, int C);
int bmc_decode_gemm(bmc_ctx_t* ctx, float* d_out, int ldo, const void* d_a, const void* d_w, int parts, int rows, int C, int OC);
/* prefill (bmt_scheduler_copy_prefill_kv, src/baremetal/session.c:136): K | V columns of prompt row b * T + t into cache[layer][0|1][b][t] */
int bmc_decode_kv_scatter(bmc_ctx_t* ctx, void* d_cache, int cache_dtype, const float* d_qkv, int ldqkv, int layer, int NB, int T, int MS, int QD, int KV);
/* attention_forward_prefill_tiled (src/kernels/forward.metal:2024): causal attention over the T prompt rows of each of NB sequences,
 * fp32 in and out, fp32-accurate on the tensor pipe (operands split into bf16 hi + lo, three tcgen05 products per product);
 * head_dim 64 (-1 otherwise: use bmc_attention_forward with BMC_F32) */
int bmc_prefill_attention(bmc_ctx_t* ctx, float* d_out, int ldo, const float* d_q, int ldq, const float* d_k, const float* d_v, int ldkv, int NB,
                          int T, int NH, int NKV, int HD, float scale);
int bmc_decode_swiglu(bmc_ctx_t* ctx, float* d_out, const float* d_gate_up, int NB, int H);
int bmc_decode_embed(bmc_ctx_t* ctx, float* d_out, int table_type, const void* d_table, const int* d_tokens, int NB, int D);
int bmc_decode_argmax(bmc_ctx_t* ctx, int* d_out, const float* d_logits, int NB, int V);
/* argmax per sequence, then the position counter + 1 (last kernel of a step) */
int bmc_decode_argmax_advance(bmc_ctx_t* ctx, int* d_out, const float* d_logits, int NB, int V, int* d_pos);
int bmc_decode_advance(bmc_ctx_t* ctx, int* d_pos);
/* Record everything enqueued between begin and end into a CUDA graph and replay it with launch (one graph per context). */
/* two graph slots per context (0 = default, used by the inference session; 1 = used by the trainer); begin/end/launch act on the
 * selected slot */
int bmc_graph_select(bmc_ctx_t* ctx, int slot);
int bmc_gemm_timing_enabled(bmc_ctx_t* ctx);
int bmc_graph_begin(bmc_ctx_t* ctx);
int bmc_graph_end(bmc_ctx_t* ctx);
int bmc_graph_launch(bmc_ctx_t* ctx);

#ifdef __cplusplus
}
#endif
#endif /* BM_CUDA_BACKEND_H */
