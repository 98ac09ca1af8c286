/* Additions beside the reference's public API. Nothing here changes a signature of include/baremetal.h.
 *
 *  - introspection of the trainer's per-tensor state, which the reference exposes only through its
 *    internal structs (bm_trainer_s::opt_states src/baremetal/trainer.h:13-22,33 and
 *    bmt_scheduler_get_grad_buffer src/baremetal/scheduler.h:50) and which its tests reach by
 *    including those headers;
 *  - a step variant whose inputs already live in device memory (the reference always stages tokens
 *    from the host, src/baremetal/trainer.c:473-516);
 *  - data-parallel set-up: the reference is single-device (one MTLDevice, src/backend/metal/device.m:20),
 *    so rank/world size and the NCCL id arrive through an added call and bm_train_step keeps its signature.
 */
#ifndef BAREMETAL_EXT_H
#define BAREMETAL_EXT_H

#include <stddef.h>
#include <stdint.h>
#include "baremetal.h"

#ifdef __cplusplus
extern "C" {
#endif

enum { BMX_WEIGHT = 0, BMX_GRAD = 1, BMX_ADAM_M = 2, BMX_ADAM_V = 3 };

/* tensors in trainer-state order: per layer ln1w, qw, kw, vw, ow, ln2w, gate, up, down; lnfw; tied embedding */
int    bmx_trainer_num_tensors(bm_trainer_t* t);
size_t bmx_trainer_tensor_size(bm_trainer_t* t, int i);
/* copies tensor i of the chosen kind (fp32) to host_out; returns 0 or -1 */
int    bmx_trainer_read(bm_trainer_t* t, int what, int i, float* host_out);
/* Reference-compatibility options (value 1 = behave like the reference, 0 = default, the mathematically
 * intended result). They exist so that parity with the reference can be shown on batches of more than one
 * sequence and over several fp32 steps, where the reference deviates from the exact gradient:
 *   "ref_norm_grad"        RMSNorm weight gradients keep only the last sequence of the batch
 *                          (rmsnorm_backward_w overwrites, src/kernels/backward.metal:400);
 *   "ref_input_grad_carry" the embedding scatter of sequence b adds the input gradients of all earlier
 *                          sequences of the optimizer window as well (the layer-0 input gradient buffer is
 *                          never cleared in between, src/baremetal/scheduler.c:263-266, trainer.c:459-470);
 *   "ref_stale_embedding"  in fp32 mode the embedding gather keeps reading the initial table after updates
 *                          (embed_lookup falls back to the host copy, src/baremetal/trainer.c:287-293);
 *   "ref_quirks"           all of the above.
 * Set before the first step. Also enabled for every trainer by the environment variable BM_REF_QUIRKS=1. */
int    bmx_trainer_set_option(bm_trainer_t* t, const char* key, int value);
/* Copies the trained fp32 master weights from the device back into the bm_model_t the trainer was created from, so that
 * bm_save_weights(model, path) exports them (a safetensors directory, or the legacy file when path ends in ".bin"). The reference
 * has no counterpart: its bm_save_weights is unimplemented (src/baremetal/checkpoint.c:84-88). 0 on success. */
int    bmx_trainer_sync_model(bm_trainer_t* t);
long   bmx_trainer_launch_count(bm_trainer_t* t);
size_t bmx_trainer_device_bytes(bm_trainer_t* t);

/* One optimizer micro-step with inputs/targets already in device memory (int32[B*T] each). Enqueues the
 * whole step and returns without waiting; 0 on success. bmx_train_last_loss() waits and returns the loss. */
int    bmx_train_step_resident(bm_trainer_t* t, const int* d_inputs, const int* d_targets, int B, int T);
float  bmx_train_last_loss(bm_trainer_t* t);
/* device allocation helpers for callers that keep inputs resident */
void*  bmx_device_alloc(bm_context_t* ctx, size_t bytes);
void   bmx_device_free(bm_context_t* ctx, void* d_ptr);
int    bmx_device_upload(bm_context_t* ctx, void* d_dst, const void* h_src, size_t bytes);
int    bmx_device_sync(bm_context_t* ctx);
/* GPU time of work enqueued between begin and end on the context's stream, in ms (end blocks). */
int    bmx_timer_begin(bm_context_t* ctx, int slot);
float  bmx_timer_end(bm_context_t* ctx, int slot);

/* Host weight buffer of a model (fp32, the flat order of the legacy .bin payload): lets a caller fill in
 * weights without going through a file. *n_out receives the element count. */
float* bmx_model_weight_buffer(bm_model_t* model, size_t* n_out);
int    bmx_model_vocab_size(const bm_model_t* model);
/* One field of the model's bm_arch_t by name ("dim", "n_layers", "rope_theta", "rope_scaling", "rope_factor", ...), -1 for an unknown
 * name: what a loader made of a checkpoint's own description (config.json or the .bin header). */
double bmx_model_arch_field(const bm_model_t* model, const char* name);
/* per-launch timing of the tensor-core GEMM (see bmc_gemm_timing in bm_cuda_backend.h) */
int    bmx_gemm_timing(bm_context_t* ctx, int enable);
int    bmx_gemm_timing_collect(bm_context_t* ctx, double* out3);

/* ---- inference ----
 * Q8 / Q4 selection: the reference sets bm_model_s::quant_bits from its CLI (tools/cli.c:886); here through a call. bits = 0, 4 or 8.
 * A 4-bit session holds two codes per byte plus one fp32 scale per 32 weights (0.625 bytes per weight), the reference's Q4 block content. */
int    bmx_model_set_quant(bm_model_t* model, int bits);
/* The reference's Q8 block quantiser (bmt_quantize_q8, src/baremetal/quant.c:10-29,54-60) with the int8 values and the scales
 * in two arrays: q[n], scales[n/32]. Returns the number of blocks, 0 when n is not a positive multiple of 32. */
size_t bmx_quantize_q8(const float* src, int8_t* q, float* scales, size_t n);
/* The reference's Q4 block quantiser (bmt_quantize_q4, src/baremetal/quant.c:31-52, 73-79) with the codes unpacked: q[n] in [-8, 7]
 * (the reference packs code 2j into the low and 2j+1 into the high nibble of byte j), scales[n/32] = amax / 7. */
size_t bmx_quantize_q4(const float* src, int8_t* q, float* scales, size_t n);
/* A session that advances n_sequences independent sequences in lock step (the reference API is single-sequence:
 * bm_create_session == n_sequences 1). max_positions = KV cache length per sequence (0: the model's max_seq_len). */
bm_session_t* bmx_create_session_batched(bm_context_t* ctx, bm_model_t* model, int n_sequences, int max_positions);
/* the same with the element type of the KV cache chosen: 0 = fp32 (the reference's, and the default; env BM_KV_BF16=1 flips the
 * default), 1 = bf16 (half the attention bytes of a decode step; head_dim 64) */
bm_session_t* bmx_create_session_kv(bm_context_t* ctx, bm_model_t* model, int n_sequences, int max_positions, int kv_bf16);
int    bmx_session_kv_bytes_per_element(bm_session_t* s);
/* prompt: int[n_sequences][n_prompt]; out: int[n_sequences][n_new] greedy continuations (lowest index among maxima). */
int    bmx_session_generate_greedy(bm_session_t* s, const int* prompt, int n_prompt, int n_new, int* out);
const float* bmx_session_logits(bm_session_t* s);
int    bmx_session_position(bm_session_t* s);
/* Weight bytes per decode step: what the session actually streams (the tensor-core path of >= 8 sequences reads bf16 expansions of
 * the Q8 values), and the algorithmic minimum in the model's own precision (Q8 = 1.125 bytes per weight, as bench/bench.c:339-348
 * of the reference counts). Roofline fractions are quoted on the second. */
size_t bmx_session_weight_bytes(bm_session_t* s);
size_t bmx_session_algorithmic_weight_bytes(bm_session_t* s);

/* Data parallel: every rank holds a full replica and calls bm_train_step with its own B sequences;
 * gradients are summed across ranks (bf16 buckets over NCCL, overlapped with backward) before AdamW and the
 * returned loss is the mean over all ranks. `nccl_id` is the 128-byte ncclUniqueId created on rank 0 with
 * bmx_dp_unique_id() and handed to the other ranks by the launcher. */
#define BMX_DP_ID_BYTES 128
/* The gradient bucket plan as pure host logic (no GPU needed): see the definition for the meaning of the arrays. */
int    bmx_dp_plan_buckets(int n_layers, const size_t* layer_begin, size_t n_params_total, int layers_per_bucket, size_t* begin,
                           size_t* end, int* ready_at, int cap);
int    bmx_dp_unique_id(void* out_id);
int    bmx_trainer_dp_init(bm_trainer_t* t, int rank, int world, const void* nccl_id);

#ifdef __cplusplus
}
#endif
#endif
