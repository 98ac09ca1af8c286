/* Internal structures of the C11 host layer. The host layer owns model weights on the host,
 * the trainer's device buffers and the step schedule; every GPU operation goes through the
 * C ABI in include/bm_cuda_backend.h. */
#ifndef BM_INTERNAL_H
#define BM_INTERNAL_H

#ifndef BAREMETAL_TRAIN
#define BAREMETAL_TRAIN
#endif
#include <stddef.h>
#include <stdint.h>

#include "../../include/baremetal.h"
#include "../../include/baremetal_ext.h"
#include "../../include/bm_cuda_backend.h"

#define BM_LOG_ERROR(...) do { fprintf(stderr, "[ERROR] " __VA_ARGS__); fputc('\n', stderr); } while (0)
#define BM_LOG_INFO(...)  do { if (bm_log_verbose()) { fprintf(stderr, "[INFO] " __VA_ARGS__); fputc('\n', stderr); } } while (0)
int bm_log_verbose(void);

struct bm_context_s {
    bm_device_t device_type;
    bmc_ctx_t* be;
};

/* Host copy of the weights: one flat fp32 buffer in the reference's model order
 * (src/baremetal/model.c:140-172): embed, ln1w[L], qw[L], kw[L], vw[L], ow[L], ln2w[L], gate[L],
 * up[L], down[L], lnfw. The tied LM head aliases `embed`. */
struct bm_model_s {
    bm_arch_t arch;
    bm_precision_t precision;
    size_t n_parameters;
    int head_size, kv_dim, kv_mul;
    int quant_bits; /* 0 = weights as stored, 8 = Q8 layer matrices for inference sessions */
    float* weight_buffer;
    float *embed, *ln1w, *qw, *kw, *vw, *ow, *ln2w, *gate, *up, *down, *lnfw;
};

#define BM_CHECKPOINT_MAGIC 20250718 /* src/baremetal/checkpoint.h:11 */
int bm_model_alloc(bm_model_t* m, const bm_arch_t* arch);
void bm_model_release(bm_model_t* m);
int bm_arch_supported(const bm_arch_t* arch);
float* bm_build_rope_table(float theta, int scaling, float factor, float low, float high, float orig, int S, int HD);
float* bm_build_rope_table_arch(const bm_arch_t* a, int S, int HD);
int bm_load_bin(bm_model_t* m, const char* path);
int bm_load_safetensors_dir(bm_model_t* m, const char* dir);
int bm_save_weights_to(const bm_model_t* m, const char* path);

/* One entry per trainable tensor, in trainer-state order (per layer ln1w, qw, kw, vw, ow, ln2w, gate,
 * up, down; then lnfw; then the tied embedding — src/baremetal/graph.c:288-369, trainer.c:86-111).
 * `off` is the tensor's element offset inside the flat device arrays, which use the same order. */
typedef struct {
    size_t off, n;
    float* host_src; /* where the tensor lives in bm_model_s.weight_buffer */
} bm_param_t;

typedef struct {
    void *x, *n1, *qkv, *attn, *x1, *n2, *gu, *act;
    float *rstd1, *rstd2, *lse;
} bm_layer_act_t;

struct bm_trainer_s {
    bm_context_t* ctx;
    bm_model_t* model;
    bm_train_config_t cfg;
    int S, B_cap, dtype, esize;
    /* reference-compatibility switches (all off by default; see bmx_trainer_set_option) */
    int side_stream;          /* weight-gradient GEMMs on the backend's side stream (default on; env BM_NO_SIDE_STREAM) */
    int graph_mode;           /* forward + backward of the plain step replayed as a CUDA graph: 0 off, 1 on (env BM_NO_TRAIN_GRAPH) */
    int graph_B;              /* batch the captured graph is for (0 = none) */
    int graph_eager_steps;    /* plain steps run eagerly with the current settings (the first ones size scratch buffers) */
    int loss_is_early;        /* the step just enqueued was a graph replay: its loss is read back right after the forward pass */
    int graph_seen_B;         /* batch of those eager steps: a different batch starts the count again */
    int ref_norm_grad;        /* RMSNorm weight gradient = last sequence of the batch only */
    int ref_input_grad_carry; /* embedding scatter of sequence b uses the running sum of input gradients */
    float* d_gx_carry;        /* [S, D] running sum for the switch above */
    float* d_embed_frozen;    /* initial embedding table, read by the fp32 gather when "ref_stale_embedding" is on */

    size_t P; /* total trainable elements */
    bm_param_t* params;
    int n_params;
    float *d_master, *d_grad, *d_m, *d_v;
    void* d_wlow; /* bf16 working copy of every parameter (mixed precision only) */
    float* d_rope_cs;

    /* activations kept for backward, sized for B_cap * S rows */
    bm_layer_act_t* act;
    void *x_last, *nf, *logits;
    float *rstdf, *row_loss, *d_loss;
    /* backward temporaries */
    void *dres, *dn, *dact, *dgu, *dattn, *dqkv;
    float* d_delta;           /* [B, NH, S] rowsum(dattn * attn), written by the O-projection input-gradient GEMM */
    int fuse;                 /* fused GEMM epilogues / attention helpers (default on; option "fused_epilogues", env BM_NO_FUSE) */
    int *d_tokens, *d_targets;
    uint8_t* d_attn_mask;
    float* d_row_weight; /* per-row loss weights of a masked step */
    int* h_stage;        /* pinned: tokens, targets, row weights, attention mask */

    int step, accum_count, window_microsteps;
    int profile;
    double prof_forward_ms, prof_loss_ms, prof_backward_ms, prof_opt_ms;

    /* data parallel (bm_dp.c); world == 1 when unused */
    struct bm_dp_s* dp;
};

/* data-parallel gradient exchange, implemented over NCCL in csrc/dp_nccl.cu */
struct bm_dp_s;

#endif
