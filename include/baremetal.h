/* Public C API of the engine. Same types, enumerator values, struct layouts and function
 * signatures as the reference's include/baremetal.h (enums :18-51, bm_arch_t :54-87,
 * bm_train_config_t :91-107, functions :120-206), so a program written against the reference links
 * against libbaremetal_b200.so unchanged. One enumerator is appended: BM_DEVICE_CUDA.
 *
 * All calls are synchronous from the caller's point of view and a context is used from one host
 * thread. Failures are reported as NULL / -1 / -1.0f plus a line on stderr.
 *
 * Scope of this build: the training path (bm_create .. bm_create_trainer, bm_train_step*, state
 * save/load, profiling), the inference session (bm_create_session, bm_forward, bm_step; fp32 / bf16 /
 * Q8 / Q4 weights) and the greedy sampler run on the GPU backend; weight export (bm_save_weights) and
 * adapter loading (bm_load_adapter merges the low-rank updates into the host weights) are host code.
 * Entry points of the reference outside those paths (tokenizer, adapter training and bm_save_adapter,
 * the sampled-generation driver) are exported so that the header is complete, and return the failure
 * value of their signature.
 */
#ifndef BAREMETAL_H
#define BAREMETAL_H

#ifdef __cplusplus
extern "C" {
#endif

#include <stdint.h>
#include "baremetal/types.h"

/* ------------------------------------------------------------------ enums (values are ABI) */
typedef enum { BM_NORM_LAYERNORM, BM_NORM_RMSNORM } bm_norm_t;
typedef enum { BM_ACT_GELU, BM_ACT_SWIGLU } bm_act_t;
typedef enum { BM_POS_LEARNED, BM_POS_ROPE } bm_pos_t;
typedef enum { BM_ATTN_MHA, BM_ATTN_GQA } bm_attn_t;
typedef enum { BM_ROPE_NONE = 0, BM_ROPE_LLAMA3 = 1 } bm_rope_scaling_t;
typedef enum { BM_PRECISION_FP32, BM_PRECISION_FP16, BM_PRECISION_BF16 } bm_precision_t;
typedef enum {
    BM_DEVICE_CPU,   /* accepted by the reference's enum only; no engine implements it */
    BM_DEVICE_METAL, /* "the accelerator": existing callers pass this and get the CUDA backend here */
    BM_DEVICE_CUDA   /* explicit name for the same backend */
} bm_device_t;

/* ------------------------------------------------------------------ architecture descriptor */
typedef struct {
    int dim, hidden_dim, n_layers, n_heads, n_kv_heads, vocab_size, padded_vocab_size, max_seq_len;
    bm_norm_t norm;
    bm_act_t activation;
    bm_pos_t pos_enc;
    bm_attn_t attention;
    bm_precision_t precision;
    int bias, weight_tie, has_qk_norm, has_ffn_post_norm, head_dim, gated_mlp, gemma_norm, embed_scale, weight_layout;
    float rope_theta;
    bm_rope_scaling_t rope_scaling;
    float rope_factor, rope_low_freq_factor, rope_high_freq_factor, rope_original_max;
} bm_arch_t;

/* ------------------------------------------------------------------ training configuration
 * Honoured: learning_rate, beta1, beta2, epsilon, weight_decay, grad_accum_steps, seq_len.
 * Carried but not read, exactly like the reference: grad_clip, warmup_steps, max_steps,
 * use_master_weights. lora_* must be 0 (training of adapters is outside this build). */
typedef struct {
    float learning_rate, beta1, beta2, epsilon, weight_decay, grad_clip;
    int grad_accum_steps, warmup_steps, max_steps, use_master_weights, seq_len, lora_rank;
    float lora_alpha;
    int lora_targets, lora_seed;
} bm_train_config_t;

typedef struct bm_context_s bm_context_t;
typedef struct bm_model_s bm_model_t;
typedef struct bm_session_s bm_session_t;
typedef struct bm_trainer_s bm_trainer_t;
typedef struct bm_sampler_s bm_sampler_t;
typedef struct bm_tokenizer_s bm_tokenizer_t;

/* ------------------------------------------------------------------ lifecycle */
bm_context_t* bm_create(bm_device_t device); /* NULL when no sm_100 GPU is usable: there is no CPU fallback */
void bm_destroy(bm_context_t* ctx);
bm_precision_t bm_get_supported_precision(bm_context_t* ctx);

/* ------------------------------------------------------------------ model */
bm_model_t* bm_create_model(bm_context_t* ctx, const bm_arch_t* arch);
void bm_load_weights(bm_model_t* model, const char* path); /* legacy .bin file, or a directory with config.json + *.safetensors */
void bm_save_weights(bm_model_t* model, const char* path);
void bm_destroy_model(bm_model_t* model);
void bm_compile(bm_model_t* model);
void bm_autotune(bm_model_t* model, int warmup, int iterations);

/* ------------------------------------------------------------------ inference */
/* Adds scale * B * A of every entry of an adapter file to the model's host weights (call it before creating a
 * session or trainer). 0 on success; -1 for an unreadable file, a header of another architecture or an entry
 * whose target or shape does not fit the model. */
int bm_load_adapter(bm_model_t* model, const char* path);
bm_session_t* bm_create_session(bm_context_t* ctx, bm_model_t* model);
float* bm_forward(bm_session_t* sess, const int* tokens, int n_tokens);
float* bm_step(bm_session_t* sess, int token);
void bm_reset_session(bm_session_t* sess);
void bm_destroy_session(bm_session_t* sess);
void bm_profile_begin(bm_session_t* sess);
void bm_profile_end(bm_session_t* sess, double* attention_ms, double* mlp_ms, double* other_ms);
typedef int (*bm_token_cb_t)(int token_id, void* user_data);
int bm_run_tokens(bm_context_t* ctx, bm_model_t* model, const int* prompt_ids, int n_prompt, int steps, float temperature,
                  int top_k, float top_p, uint64_t seed, bm_token_cb_t callback, void* user_data);

/* ------------------------------------------------------------------ sampler */
bm_sampler_t* bm_create_sampler(int vocab_size, float temp, float topp, uint64_t seed);
int bm_sample(bm_sampler_t* sampler, const float* logits); /* temp <= 0: lowest index among the maxima */
void bm_destroy_sampler(bm_sampler_t* sampler);

/* ------------------------------------------------------------------ tokenizer (outside this build) */
bm_tokenizer_t* bm_create_tokenizer(const char* path);
int* bm_encode(bm_tokenizer_t* tok, const char* text, int* n_tokens);
char* bm_decode(bm_tokenizer_t* tok, int prev_token, int token);
void bm_destroy_tokenizer(bm_tokenizer_t* tok);

/* ------------------------------------------------------------------ training */
#ifdef BAREMETAL_TRAIN
bm_trainer_t* bm_create_trainer(bm_context_t* ctx, bm_model_t* model, const bm_train_config_t* cfg);
/* inputs/targets: host int32[B*T], row-major; T must equal the trainer's sequence length.
 * Returns the mean over the B sequences of the per-sequence mean loss, or -1.0f. */
float bm_train_step(bm_trainer_t* trainer, const int* inputs, const int* targets, int B, int T);
float bm_train_step_masked(bm_trainer_t* trainer, const int* inputs, const int* targets, const uint8_t* attn_mask,
                           const uint8_t* loss_mask, int B, int T);
float bm_train_eval_masked(bm_trainer_t* trainer, const int* inputs, const int* targets, const uint8_t* attn_mask,
                           const uint8_t* loss_mask, int B, int T);
void bm_load_state(bm_trainer_t* trainer, const char* path);
void bm_save_state(bm_trainer_t* trainer, const char* path);
void bm_train_flush(bm_trainer_t* trainer);
int bm_save_adapter(bm_trainer_t* trainer, const char* path);
void bm_train_profile_begin(bm_trainer_t* trainer);
void bm_train_profile_end(bm_trainer_t* trainer, double* forward_ms, double* loss_ms, double* backward_ms, double* optimizer_ms);
void bm_destroy_trainer(bm_trainer_t* trainer);
#endif /* BAREMETAL_TRAIN */

/* ------------------------------------------------------------------ utility */
int bm_get_num_parameters(const bm_model_t* model);
const char* bm_get_arch_name(const bm_model_t* model);
void bm_print_model_info(const bm_model_t* model);

#ifdef __cplusplus
}
#endif
#endif /* BAREMETAL_H */
