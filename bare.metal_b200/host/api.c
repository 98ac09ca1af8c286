/* Public API glue: context and model lifecycle, the sampler, and the reference entry points that lie
 * outside this build (they keep their signatures and return the failure value).
 * Counterpart of the reference's src/baremetal/api.c:20-194 and context.c:10-34. */
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "bm_internal.h"

/* ---- lifecycle ------------------------------------------------------------------------------------ */
bm_context_t* bm_create(bm_device_t device) {
    if (device != BM_DEVICE_METAL && device != BM_DEVICE_CUDA) {
        /* BM_DEVICE_CPU exists in the enum only; the reference builds no backend for it either (context.c:16-22). */
        BM_LOG_ERROR("bm_create: device %d has no backend (this engine runs on the CUDA backend only)", (int)device);
        return NULL;
    }
    bm_context_t* ctx = (bm_context_t*)calloc(1, sizeof *ctx);
    if (!ctx) return NULL;
    ctx->device_type = device;
    int ordinal = 0;
    const char* lr = getenv("LOCAL_RANK");
    const char* dv = getenv("BM_CUDA_DEVICE");
    if (dv && dv[0]) ordinal = atoi(dv);
    else if (lr && lr[0]) ordinal = atoi(lr);
    ctx->be = bmc_create(ordinal);
    if (!ctx->be) {
        BM_LOG_ERROR("bm_create: CUDA backend unavailable (no sm_100 device %d); there is no CPU fallback", ordinal);
        free(ctx);
        return NULL;
    }
    BM_LOG_INFO("Context created (device=%d, cuda ordinal %d)", (int)device, ordinal);
    return ctx;
}

void bm_destroy(bm_context_t* ctx) {
    if (!ctx) return;
    bmc_destroy(ctx->be);
    free(ctx);
}

bm_precision_t bm_get_supported_precision(bm_context_t* ctx) {
    if (!ctx || !ctx->be) return BM_PRECISION_FP32;
    return BM_PRECISION_BF16;
}

/* ---- model ---------------------------------------------------------------------------------------- */
bm_model_t* bm_create_model(bm_context_t* ctx, const bm_arch_t* arch) {
    (void)ctx;
    if (!arch) return NULL;
    bm_model_t* m = (bm_model_t*)calloc(1, sizeof *m);
    if (!m) return NULL;
    if (bm_model_alloc(m, arch) != 0) {
        free(m);
        return NULL;
    }
    return m;
}

void bm_load_weights(bm_model_t* model, const char* path) {
    if (!model || !path) return;
    const bm_precision_t keep = model->precision;
    if (bm_load_bin(model, path) == 0 || bm_load_safetensors_dir(model, path) == 0) {
        /* a precision chosen by the caller before loading wins over the file's header field */
        if (keep != BM_PRECISION_FP32) model->precision = keep;
        return;
    }
    BM_LOG_ERROR("Failed to load weights from %s", path);
}

/* Writes the model's host weights: a Hugging Face safetensors directory, or the legacy .bin file when the path ends in ".bin"
 * (host/safetensors.c). The reference declares this function and leaves it unimplemented (src/baremetal/checkpoint.c:84-88).
 * Weights a trainer has updated live on the device: bmx_trainer_sync_model() brings them back into the model first. */
void bm_save_weights(bm_model_t* model, const char* path) {
    if (bm_save_weights_to(model, path) != 0) BM_LOG_ERROR("bm_save_weights: could not write %s", path ? path : "(null)");
}

void bm_destroy_model(bm_model_t* model) {
    if (!model) return;
    bm_model_release(model);
    free(model);
}

void bm_compile(bm_model_t* model) { (void)model; }
void bm_autotune(bm_model_t* model, int warmup, int iterations) { (void)model; (void)warmup; (void)iterations; }

/* ---- outside this build (tokenizer, adapter training, sampled generation driver): same signatures, failure values --------------------------------------
 * bm_load_adapter() is in host/adapter.c. */
int bm_run_tokens(bm_context_t* ctx, bm_model_t* model, const int* prompt_ids, int n_prompt, int steps, float temperature, int top_k,
                  float top_p, uint64_t seed, bm_token_cb_t callback, void* user_data) {
    (void)ctx; (void)model; (void)prompt_ids; (void)n_prompt; (void)steps; (void)temperature; (void)top_k; (void)top_p; (void)seed;
    (void)callback; (void)user_data;
    return -1;
}
bm_tokenizer_t* bm_create_tokenizer(const char* path) { (void)path; return NULL; }
int* bm_encode(bm_tokenizer_t* tok, const char* text, int* n_tokens) {
    (void)tok; (void)text;
    if (n_tokens) *n_tokens = 0;
    return NULL;
}
char* bm_decode(bm_tokenizer_t* tok, int prev_token, int token) { (void)tok; (void)prev_token; (void)token; return NULL; }
void bm_destroy_tokenizer(bm_tokenizer_t* tok) { (void)tok; }
int bm_save_adapter(bm_trainer_t* trainer, const char* path) { (void)trainer; (void)path; return -1; }

/* ---- sampler ---------------------------------------------------------------------------------------- */
struct bm_sampler_s {
    int vocab_size;
    float temperature, topp;
    unsigned int rng_state;
    float* probs;
};

bm_sampler_t* bm_create_sampler(int vocab_size, float temp, float topp, uint64_t seed) {
    if (vocab_size <= 0) return NULL;
    bm_sampler_t* s = (bm_sampler_t*)calloc(1, sizeof *s);
    if (!s) return NULL;
    s->vocab_size = vocab_size;
    s->temperature = temp;
    s->topp = topp;
    s->rng_state = seed ? (unsigned int)seed : 0x9E3779B9u;
    s->probs = (float*)malloc((size_t)vocab_size * sizeof(float));
    if (!s->probs) { free(s); return NULL; }
    return s;
}

/* Greedy branch: first index of the maximum, strict '>' scan from index 0 (src/baremetal/sampler.c:36-40).
 * With temperature > 0 the draw is a plain temperature softmax + inverse-CDF sample; the reference's
 * top-k / nucleus filtering is outside this build. */
int bm_sample(bm_sampler_t* s, const float* logits) {
    if (!s || !logits) return 0;
    const int n = s->vocab_size;
    if (s->temperature <= 0.0f) {
        int best = 0;
        for (int i = 1; i < n; ++i)
            if (logits[i] > logits[best]) best = i;
        return best;
    }
    float mx = logits[0];
    for (int i = 1; i < n; ++i) if (logits[i] > mx) mx = logits[i];
    float sum = 0.0f;
    for (int i = 0; i < n; ++i) { s->probs[i] = expf((logits[i] - mx) / s->temperature); sum += s->probs[i]; }
    unsigned int r = s->rng_state * 1664525u + 1013904223u;
    s->rng_state = r;
    const float target = ((float)(r >> 8) / (float)0x1000000) * sum;
    float c = 0.0f;
    for (int i = 0; i < n; ++i) { c += s->probs[i]; if (c >= target) return i; }
    return n - 1;
}

void bm_destroy_sampler(bm_sampler_t* s) {
    if (!s) return;
    free(s->probs);
    free(s);
}

/* ---- utility ---------------------------------------------------------------------------------------- */
int bm_get_num_parameters(const bm_model_t* model) { return model ? (int)model->n_parameters : 0; }

const char* bm_get_arch_name(const bm_model_t* model) {
    if (!model) return "none";
    return model->arch.attention == BM_ATTN_GQA ? "Llama3-GQA" : "Llama2-MQA";
}

void bm_print_model_info(const bm_model_t* model) {
    if (!model) return;
    const bm_arch_t* a = &model->arch;
    printf("=== %s Model ===\n", bm_get_arch_name(model));
    printf("  dim:         %d\n  hidden_dim:  %d\n  n_layers:    %d\n  n_heads:     %d\n  n_kv_heads:  %d\n", a->dim, a->hidden_dim,
           a->n_layers, a->n_heads, a->n_kv_heads);
    printf("  vocab_size:  %d\n  max_seq_len: %d\n  weight_tie:  %s\n", a->vocab_size, a->max_seq_len, a->weight_tie ? "yes" : "no");
    printf("  precision:   %s\n", model->precision == BM_PRECISION_BF16 ? "bf16" : model->precision == BM_PRECISION_FP16 ? "fp16" : "fp32");
    printf("  parameters:  %zu\n", model->n_parameters);
}

/* ---- device helpers of baremetal_ext.h --------------------------------------------------------------- */
void* bmx_device_alloc(bm_context_t* ctx, size_t bytes) { return ctx ? bmc_alloc(ctx->be, bytes) : NULL; }
void bmx_device_free(bm_context_t* ctx, void* p) { if (ctx) bmc_free(ctx->be, p); }
int bmx_device_upload(bm_context_t* ctx, void* d, const void* h, size_t bytes) { return ctx ? bmc_upload(ctx->be, d, h, bytes) : -1; }
int bmx_device_sync(bm_context_t* ctx) { return ctx ? bmc_sync(ctx->be) : -1; }
int bmx_timer_begin(bm_context_t* ctx, int slot) { return ctx ? bmc_timer_begin(ctx->be, slot) : -1; }
float bmx_timer_end(bm_context_t* ctx, int slot) { return ctx ? bmc_timer_end(ctx->be, slot) : -1.0f; }
float* bmx_model_weight_buffer(bm_model_t* model, size_t* n_out) {
    if (!model) return NULL;
    if (n_out) *n_out = model->n_parameters;
    return model->weight_buffer;
}
int bmx_gemm_timing(bm_context_t* ctx, int enable) { return ctx ? bmc_gemm_timing(ctx->be, enable) : -1; }
int bmx_gemm_timing_collect(bm_context_t* ctx, double* out3) { return ctx ? bmc_gemm_timing_collect(ctx->be, out3) : -1; }
int bmx_model_vocab_size(const bm_model_t* model) { return model ? model->arch.vocab_size : 0; }
double bmx_model_arch_field(const bm_model_t* model, const char* name) {
    if (!model || !name) return -1.0;
    const bm_arch_t* a = &model->arch;
#define F(n) if (strcmp(name, #n) == 0) return (double)a->n
    F(dim); F(hidden_dim); F(n_layers); F(n_heads); F(n_kv_heads); F(vocab_size); F(max_seq_len); F(head_dim); F(weight_tie);
    F(rope_theta); F(rope_scaling); F(rope_factor); F(rope_low_freq_factor); F(rope_high_freq_factor); F(rope_original_max);
#undef F
    return -1.0;
}
int bmx_model_set_quant(bm_model_t* model, int bits) {
    if (!model || (bits != 0 && bits != 4 && bits != 8)) return -1;
    model->quant_bits = bits;
    return 0;
}
