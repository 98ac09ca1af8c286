/* Training step driver: forward, loss, backward and AdamW for the Llama-family decoder, batched over
 * all B sequences of a step ([B*S, .] activations) and issued as one asynchronous stream of backend
 * calls. Counterpart of the reference's trainer + training scheduler walk
 * (src/baremetal/trainer.c:30-123,349-533, src/baremetal/scheduler.c:1015-1332,1364-1617,
 * graph src/baremetal/graph.c:273-381), which loops over the sequences one by one with four
 * command-buffer waits each.
 *
 * Differences in form, not in result:
 *  - Q, K and V projections are one GEMM over the row-concatenated weight [qw; kw; vw] (they are adjacent in
 *    the parameter order), likewise gate and up; attention, RoPE and SwiGLU address the packed rows through
 *    leading dimensions;
 *  - the two residual adds per layer are GEMM epilogues; their backward is the identity on the residual
 *    gradient, which lives in one buffer that RMSNorm backward accumulates into (the reference's `+=`,
 *    src/kernels/backward.metal:372);
 *  - parameters, gradients and AdamW moments are flat arrays in trainer-state order, so AdamW is one launch.
 */
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

#include "bm_internal.h"
#include "dp.h"

#define RMS_EPS 1e-5f /* fixed by the reference's graph builder, src/baremetal/graph.c:283 */

static size_t esz(const bm_trainer_t* t) { return (size_t)t->esize; }

static void free_activations(bm_trainer_t* t) {
    bmc_ctx_t* be = t->ctx->be;
    if (t->act) {
        for (int l = 0; l < t->model->arch.n_layers; ++l) {
            bm_layer_act_t* a = &t->act[l];
            bmc_free(be, a->x); bmc_free(be, a->n1); bmc_free(be, a->qkv); bmc_free(be, a->attn); bmc_free(be, a->x1);
            bmc_free(be, a->n2); bmc_free(be, a->gu); bmc_free(be, a->act); bmc_free(be, a->rstd1); bmc_free(be, a->rstd2);
            bmc_free(be, a->lse);
        }
        free(t->act);
        t->act = NULL;
    }
    bmc_free(be, t->x_last); bmc_free(be, t->nf); bmc_free(be, t->logits); bmc_free(be, t->rstdf); bmc_free(be, t->row_loss);
    bmc_free(be, t->dres); bmc_free(be, t->dn); bmc_free(be, t->dact); bmc_free(be, t->dgu); bmc_free(be, t->dattn); bmc_free(be, t->dqkv);
    bmc_free(be, t->d_delta);
    t->d_delta = NULL;
    bmc_free(be, t->d_tokens); bmc_free(be, t->d_targets); bmc_free(be, t->d_attn_mask); bmc_free(be, t->d_row_weight);
    t->x_last = t->nf = t->logits = NULL;
    t->rstdf = t->row_loss = NULL;
    t->dres = t->dn = t->dact = t->dgu = t->dattn = t->dqkv = NULL;
    t->d_tokens = t->d_targets = NULL;
    t->d_attn_mask = NULL;
    t->d_row_weight = NULL;
    if (t->h_stage) { bmc_host_free(t->h_stage); t->h_stage = NULL; }
    t->B_cap = 0;
}

/* (Re)allocate everything whose size depends on the batch. */
static int ensure_batch(bm_trainer_t* t, int B) {
    if (B <= t->B_cap) return 0;
    t->graph_B = 0; /* every activation buffer moves: a captured step is stale */
    t->graph_eager_steps = 0;
    free_activations(t);
    bmc_ctx_t* be = t->ctx->be;
    const bm_arch_t* a = &t->model->arch;
    const size_t M = (size_t)B * t->S, D = a->dim, H = a->hidden_dim, V = a->vocab_size;
    const size_t QD = (size_t)a->n_heads * t->model->head_size, KV = t->model->kv_dim, QKVD = QD + 2 * KV;
    const size_t e = esz(t);
    int ok = 1;
#define ALLOC(p, bytes) do { (p) = bmc_alloc(be, (bytes)); if (!(p)) ok = 0; } while (0)
    t->act = (bm_layer_act_t*)calloc(a->n_layers, sizeof(bm_layer_act_t));
    if (!t->act) return -1;
    for (int l = 0; l < a->n_layers && ok; ++l) {
        bm_layer_act_t* c = &t->act[l];
        ALLOC(c->x, M * D * e); ALLOC(c->n1, M * D * e); ALLOC(c->qkv, M * QKVD * e); ALLOC(c->attn, M * QD * e);
        ALLOC(c->x1, M * D * e); ALLOC(c->n2, M * D * e); ALLOC(c->gu, M * 2 * H * e); ALLOC(c->act, M * H * e);
        ALLOC(c->rstd1, M * sizeof(float)); ALLOC(c->rstd2, M * sizeof(float));
        ALLOC(c->lse, (size_t)B * a->n_heads * t->S * sizeof(float));
    }
    ALLOC(t->x_last, M * D * e); ALLOC(t->nf, M * D * e); ALLOC(t->logits, M * V * e);
    ALLOC(t->rstdf, M * sizeof(float)); ALLOC(t->row_loss, M * sizeof(float));
    ALLOC(t->dres, M * D * e); ALLOC(t->dn, M * D * e); ALLOC(t->dact, M * H * e); ALLOC(t->dgu, M * 2 * H * e);
    ALLOC(t->dattn, M * QD * e); ALLOC(t->dqkv, M * QKVD * e);
    ALLOC(t->d_delta, (size_t)B * a->n_heads * t->S * sizeof(float));
    ALLOC(t->d_tokens, M * sizeof(int)); ALLOC(t->d_targets, M * sizeof(int));
    ALLOC(t->d_attn_mask, M); ALLOC(t->d_row_weight, M * sizeof(float));
#undef ALLOC
    t->h_stage = (int*)bmc_host_alloc(3 * M * sizeof(int) + M);
    if (!ok || !t->h_stage) {
        BM_LOG_ERROR("bm_train_step: out of device memory for B=%d, S=%d", B, t->S);
        free_activations(t);
        return -1;
    }
    t->B_cap = B;
    return 0;
}

bm_trainer_t* bm_create_trainer(bm_context_t* ctx, bm_model_t* model, const bm_train_config_t* cfg) {
    if (!ctx || !ctx->be || !model || !model->weight_buffer || !cfg) return NULL;
    if (cfg->lora_rank > 0) {
        BM_LOG_ERROR("bm_create_trainer: LoRA adapters are outside this build (lora_rank must be 0)");
        return NULL;
    }
    const bm_arch_t* a = &model->arch;
    bm_precision_t prec = model->precision;
    const char* pe = getenv("BM_PRECISION");
    if (pe && pe[0]) prec = strcmp(pe, "bf16") == 0 ? BM_PRECISION_BF16 : strcmp(pe, "fp16") == 0 ? BM_PRECISION_FP16 : BM_PRECISION_FP32;
    if (prec == BM_PRECISION_FP16) {
        BM_LOG_ERROR("bm_create_trainer: fp16 weights are not supported by this backend (use bf16 or fp32)");
        return NULL;
    }
    const int HD = model->head_size;
    if ((a->dim % 8) || (a->hidden_dim % 8) || (HD % 2) || ((a->n_heads * HD) % 8) || (model->kv_dim % 8) || (a->vocab_size % 8)) {
        BM_LOG_ERROR("bm_create_trainer: dim, hidden_dim, head widths and vocab_size must be multiples of 8");
        return NULL;
    }
    bm_trainer_t* t = (bm_trainer_t*)calloc(1, sizeof *t);
    if (!t) return NULL;
    t->ctx = ctx;
    t->model = model;
    t->cfg = *cfg;
    t->S = cfg->seq_len > 0 ? cfg->seq_len : 64; /* default as bm_create_trainer, src/baremetal/api.c:191 */
    t->dtype = prec == BM_PRECISION_BF16 ? BMC_BF16 : BMC_F32;
    t->esize = t->dtype == BMC_BF16 ? 2 : 4;

    const int L = a->n_layers;
    const size_t D = a->dim, H = a->hidden_dim, V = a->vocab_size, QD = (size_t)a->n_heads * HD, KV = model->kv_dim;
    t->n_params = 9 * L + 2;
    t->params = (bm_param_t*)calloc(t->n_params, sizeof(bm_param_t));
    size_t off = 0;
    int k = 0;
#define ADD(ptr, n_) do { t->params[k].off = off; t->params[k].n = (n_); t->params[k].host_src = (ptr); off += (n_); ++k; } while (0)
    for (int l = 0; l < L; ++l) {
        ADD(model->ln1w + (size_t)l * D, D);
        ADD(model->qw + (size_t)l * QD * D, QD * D);
        ADD(model->kw + (size_t)l * KV * D, KV * D);
        ADD(model->vw + (size_t)l * KV * D, KV * D);
        ADD(model->ow + (size_t)l * D * QD, D * QD);
        ADD(model->ln2w + (size_t)l * D, D);
        ADD(model->gate + (size_t)l * H * D, H * D);
        ADD(model->up + (size_t)l * H * D, H * D);
        ADD(model->down + (size_t)l * D * H, D * H);
    }
    ADD(model->lnfw, D);
    ADD(model->embed, V * D);
#undef ADD
    t->P = off;

    bmc_ctx_t* be = ctx->be;
    t->d_master = (float*)bmc_alloc(be, t->P * sizeof(float));
    t->d_grad = (float*)bmc_alloc(be, t->P * sizeof(float));
    t->d_m = (float*)bmc_alloc(be, t->P * sizeof(float));
    t->d_v = (float*)bmc_alloc(be, t->P * sizeof(float));
    t->d_loss = (float*)bmc_alloc(be, 16);
    if (t->dtype == BMC_BF16) t->d_wlow = bmc_alloc(be, t->P * 2);
    float* cs = bm_build_rope_table_arch(a, t->S, HD);
    t->d_rope_cs = (float*)bmc_alloc(be, (size_t)t->S * (HD / 2) * 2 * sizeof(float));
    if (!t->d_master || !t->d_grad || !t->d_m || !t->d_v || !t->d_loss || !t->d_rope_cs || !cs || (t->dtype == BMC_BF16 && !t->d_wlow)) {
        BM_LOG_ERROR("bm_create_trainer: out of memory");
        free(cs);
        bm_destroy_trainer(t);
        return NULL;
    }
    for (int i = 0; i < t->n_params; ++i)
        bmc_upload(be, t->d_master + t->params[i].off, t->params[i].host_src, t->params[i].n * sizeof(float));
    bmc_upload(be, t->d_rope_cs, cs, (size_t)t->S * (HD / 2) * 2 * sizeof(float));
    bmc_memset(be, t->d_m, 0, t->P * sizeof(float));
    bmc_memset(be, t->d_v, 0, t->P * sizeof(float));
    bmc_memset(be, t->d_grad, 0, t->P * sizeof(float));
    if (t->d_wlow) bmc_cast_f32_to_bf16(be, t->d_wlow, t->d_master, t->P);
    const int rc = bmc_sync(be);
    free(cs);
    if (rc) {
        BM_LOG_ERROR("bm_create_trainer: device set-up failed (%d)", rc);
        bm_destroy_trainer(t);
        return NULL;
    }
    t->side_stream = getenv("BM_NO_SIDE_STREAM") ? 0 : 1;
    t->fuse = getenv("BM_NO_FUSE") ? 0 : 1;
    t->graph_mode = getenv("BM_NO_TRAIN_GRAPH") ? 0 : 1;
    t->graph_B = 0;
    t->graph_eager_steps = 0;
    t->graph_seen_B = 0;
    const char* rq = getenv("BM_REF_QUIRKS");
    if (rq && rq[0] == '1') bmx_trainer_set_option(t, "ref_quirks", 1);
    BM_LOG_INFO("Trainer created: %d weight tensors, S=%d, D=%d", t->n_params, t->S, a->dim);
    return t;
}

void bm_destroy_trainer(bm_trainer_t* t) {
    if (!t) return;
    bmc_ctx_t* be = t->ctx->be;
    bmc_sync(be);
    if (t->dp) bm_dp_destroy(t->dp);
    free_activations(t);
    bmc_free(be, t->d_master); bmc_free(be, t->d_grad); bmc_free(be, t->d_m); bmc_free(be, t->d_v); bmc_free(be, t->d_wlow);
    bmc_free(be, t->d_rope_cs); bmc_free(be, t->d_loss); bmc_free(be, t->d_gx_carry); bmc_free(be, t->d_embed_frozen);
    free(t->params);
    free(t);
}

/* weight pointer for the GEMMs: bf16 working copy in mixed precision, the fp32 master otherwise */
static const void* wptr(const bm_trainer_t* t, int param_index) {
    const size_t off = t->params[param_index].off;
    return t->dtype == BMC_BF16 ? (const void*)((const uint16_t*)t->d_wlow + off) : (const void*)(t->d_master + off);
}
static const float* wf32(const bm_trainer_t* t, int param_index) { return t->d_master + t->params[param_index].off; }
static float* gptr(const bm_trainer_t* t, int param_index) { return t->d_grad + t->params[param_index].off; }
static void* at(void* base, size_t elems, const bm_trainer_t* t) { return (char*)base + elems * esz(t); }

enum { P_LN1 = 0, P_Q, P_K, P_V, P_O, P_LN2, P_GATE, P_UP, P_DOWN };

#define TRY(call) do { int rc__ = (call); if (rc__) { BM_LOG_ERROR("train step: %s failed (%d)", #call, rc__); return rc__; } } while (0)

/* forward + loss. Tokens, targets (and masks) are already in t->d_tokens / t->d_targets. */
static int forward_and_loss(bm_trainer_t* t, int B, const uint8_t* d_attn_mask, const float* d_row_weight, int with_grad) {
    bmc_ctx_t* be = t->ctx->be;
    const bm_arch_t* a = &t->model->arch;
    const int L = a->n_layers, D = a->dim, H = a->hidden_dim, V = a->vocab_size, S = t->S;
    const int NH = a->n_heads, NKV = a->n_kv_heads, HD = t->model->head_size;
    const int QD = NH * HD, KV = NKV * HD, QKVD = QD + 2 * KV, M = B * S, dt = t->dtype;
    const float scale = 1.0f / sqrtf((float)HD);
    const int p_lnf = 9 * L, p_emb = 9 * L + 1;

    /* embedding rows come from the fp32 master (embed_lookup, src/baremetal/trainer.c:275-298); with the
     * "ref_stale_embedding" option, fp32 mode reads the initial table instead, as the reference does there. */
    TRY(bmc_embedding_forward(be, dt, t->act[0].x, (t->d_embed_frozen && dt == BMC_F32) ? t->d_embed_frozen : wf32(t, p_emb),
                              t->d_tokens, M, D, V));
    for (int l = 0; l < L; ++l) {
        bm_layer_act_t* c = &t->act[l];
        const int pb = 9 * l;
        void* x_next = l + 1 < L ? t->act[l + 1].x : t->x_last;
        TRY(bmc_rmsnorm_forward(be, dt, c->n1, c->rstd1, c->x, wf32(t, pb + P_LN1), M, D, RMS_EPS));
        TRY(bmc_matmul_forward(be, dt, c->qkv, QKVD, c->n1, D, wptr(t, pb + P_Q), NULL, 0, M, D, QKVD));
        TRY(bmc_rope(be, dt, c->qkv, QKVD, at(c->qkv, QD, t), QKVD, t->d_rope_cs, M, S, NH, NKV, HD, +1));
        TRY(bmc_attention_forward(be, dt, c->attn, QD, c->lse, c->qkv, QKVD, at(c->qkv, QD, t), at(c->qkv, QD + KV, t), QKVD,
                                  d_attn_mask, B, S, NH, NKV, HD, scale));
        TRY(bmc_matmul_forward(be, dt, c->x1, D, c->attn, QD, wptr(t, pb + P_O), c->x, D, M, QD, D));
        TRY(bmc_rmsnorm_forward(be, dt, c->n2, c->rstd2, c->x1, wf32(t, pb + P_LN2), M, D, RMS_EPS));
        /* gate and up in one GEMM whose epilogue also writes act = silu(gate) * up; shapes without that form take two launches */
        int frc = t->fuse ? bmc_matmul_swiglu_forward(be, dt, c->gu, 2 * H, c->act, H, c->n2, D, wptr(t, pb + P_GATE), M, D, H) : BMC_ERR_UNFUSED;
        if (frc == BMC_ERR_UNFUSED) {
            TRY(bmc_matmul_forward(be, dt, c->gu, 2 * H, c->n2, D, wptr(t, pb + P_GATE), NULL, 0, M, D, 2 * H));
            TRY(bmc_swiglu_forward(be, dt, c->act, H, c->gu, at(c->gu, H, t), 2 * H, M, H));
        } else {
            TRY(frc);
        }
        TRY(bmc_matmul_forward(be, dt, x_next, D, c->act, H, wptr(t, pb + P_DOWN), c->x1, D, M, H, D));
    }
    TRY(bmc_rmsnorm_forward(be, dt, t->nf, t->rstdf, t->x_last, wf32(t, p_lnf), M, D, RMS_EPS));
    TRY(bmc_matmul_forward(be, dt, t->logits, V, t->nf, D, wptr(t, p_emb), NULL, 0, M, D, V));
    if (t->profile) bmc_timer_begin(be, 3);   /* the loss phase is timed by itself, as src/baremetal/trainer.c:400-423 does */
    /* gradient of the per-sequence mean loss: (softmax - onehot) / S (xent_backward, src/kernels/backward.metal:585);
     * the 1 / (number of sequences) factor is applied by AdamW (src/anneal/adamw.metal:38). */
    (void)with_grad;
    TRY(bmc_xent(be, dt, t->logits, V, t->row_loss, t->d_loss, t->d_targets, d_row_weight, B, S, V, 1.0f / (float)S));
    if (t->profile) {
        const double loss_ms = bmc_timer_end(be, 3);
        t->prof_loss_ms += loss_ms;
        t->prof_forward_ms -= loss_ms;   /* the caller's forward bracket spans the loss kernels too */
    }
    return 0;
}

static int backward(bm_trainer_t* t, int B, const uint8_t* d_attn_mask) {
    bmc_ctx_t* be = t->ctx->be;
    const bm_arch_t* a = &t->model->arch;
    const int L = a->n_layers, D = a->dim, H = a->hidden_dim, V = a->vocab_size, S = t->S;
    const int NH = a->n_heads, NKV = a->n_kv_heads, HD = t->model->head_size;
    const int QD = NH * HD, KV = NKV * HD, QKVD = QD + 2 * KV, M = B * S, dt = t->dtype;
    const float scale = 1.0f / sqrtf((float)HD);
    const int p_lnf = 9 * L, p_emb = 9 * L + 1;
    /* RMSNorm weight gradient: full sum over the batch, accumulated across micro-steps — or the reference's
     * behaviour (last sequence only, overwriting), selected by the "ref_norm_grad" option. */
    const int nw_acc = t->ref_norm_grad ? 0 : 1;
    const int nw_r0 = t->ref_norm_grad ? (B - 1) * S : 0, nw_r1 = M;

    /* Weight-gradient GEMMs go to the context's side stream: each is enqueued right after the input-gradient GEMM that shares
     * its operand, so it runs while the main stream executes the memory-bound kernel that follows (SwiGLU / RMSNorm backward,
     * attention helpers). A ticket is waited for before a buffer the side GEMM reads is overwritten. */
    const int side = t->side_stream;
    int tk_head = -1, tk_down = -1, tk_gu = -1, tk_o = -1, tk_q = -1, frc;
#define SIDE_WGRAD(ticket, call) do { if (side) { TRY(bmc_side_begin(be)); } TRY(call); if (side) { (ticket) = bmc_side_end(be); if ((ticket) < 0) return -1; } } while (0)
#define SIDE_WAIT(ticket) do { if (side && (ticket) >= 0) { TRY(bmc_side_wait(be, (ticket))); (ticket) = -1; } } while (0)

    /* LM head: logits buffer now holds dL/dlogits */
    TRY(bmc_matmul_backward_inp(be, dt, t->dn, D, 0, t->logits, V, wptr(t, p_emb), M, D, V));
    SIDE_WGRAD(tk_head, bmc_matmul_backward_w(be, dt, gptr(t, p_emb), t->logits, V, t->nf, D, M, D, V));
    TRY(bmc_memset(be, t->dres, 0, (size_t)M * D * esz(t)));
    TRY(bmc_rmsnorm_backward(be, dt, t->dres, gptr(t, p_lnf), nw_acc, t->dn, t->x_last, wf32(t, p_lnf), t->rstdf, M, D, nw_r0, nw_r1));
    if (t->dp) TRY(bm_dp_bucket_ready(t->dp, L));

    for (int l = L - 1; l >= 0; --l) {
        bm_layer_act_t* c = &t->act[l];
        const int pb = 9 * l;
        /* MLP: dres is dL/d(x_{l+1}); the residual add routes it unchanged to both of its inputs */
        SIDE_WAIT(tk_gu); /* the previous layer's gate/up weight gradient still reads dgu */
        /* down-projection input gradient whose epilogue applies SwiGLU backward (dact is never stored) */
        frc = t->fuse ? bmc_matmul_backward_inp_swiglu(be, dt, t->dgu, 2 * H, t->dres, D, wptr(t, pb + P_DOWN), c->gu, 2 * H, M, H, D) : BMC_ERR_UNFUSED;
        if (frc == BMC_ERR_UNFUSED) {
            TRY(bmc_matmul_backward_inp(be, dt, t->dact, H, 0, t->dres, D, wptr(t, pb + P_DOWN), M, H, D));
            TRY(bmc_swiglu_backward(be, dt, t->dgu, at(t->dgu, H, t), 2 * H, c->gu, at(c->gu, H, t), 2 * H, t->dact, H, M, H));
        } else {
            TRY(frc);
        }
        SIDE_WGRAD(tk_down, bmc_matmul_backward_w(be, dt, gptr(t, pb + P_DOWN), t->dres, D, c->act, H, M, H, D));
        TRY(bmc_matmul_backward_inp(be, dt, t->dn, D, 0, t->dgu, 2 * H, wptr(t, pb + P_GATE), M, D, 2 * H));
        SIDE_WGRAD(tk_gu, bmc_matmul_backward_w(be, dt, gptr(t, pb + P_GATE), t->dgu, 2 * H, c->n2, D, M, D, 2 * H));
        SIDE_WAIT(tk_down); /* reads dres, which the norm backward accumulates into */
        TRY(bmc_rmsnorm_backward(be, dt, t->dres, gptr(t, pb + P_LN2), nw_acc, t->dn, c->x1, wf32(t, pb + P_LN2), c->rstd2, M, D, nw_r0, nw_r1));
        /* attention block: dres is now dL/d(x1) */
        /* O-projection input gradient; its epilogue also leaves rowsum(dattn * attn) per (row, head) for attention backward */
        const float* delta = NULL;
        frc = (t->fuse && HD == 64)
                  ? bmc_matmul_backward_inp_rowdot(be, dt, t->dattn, QD, t->d_delta, t->dres, D, wptr(t, pb + P_O), c->attn, QD, M, QD, D, S, NH)
                  : BMC_ERR_UNFUSED;
        if (frc == BMC_ERR_UNFUSED) TRY(bmc_matmul_backward_inp(be, dt, t->dattn, QD, 0, t->dres, D, wptr(t, pb + P_O), M, QD, D));
        else { TRY(frc); delta = t->d_delta; }
        SIDE_WGRAD(tk_o, bmc_matmul_backward_w(be, dt, gptr(t, pb + P_O), t->dres, D, c->attn, QD, M, QD, D));
        SIDE_WAIT(tk_q); /* the previous layer's QKV weight gradient still reads dqkv */
        /* dQ and dK leave already rotated backwards (RoPE backward folded into the kernel's output pass) */
        TRY(bmc_attention_backward_fused(be, dt, t->dqkv, QKVD, at(t->dqkv, QD, t), at(t->dqkv, QD + KV, t), QKVD, t->dattn, QD, c->attn,
                                         c->lse, c->qkv, QKVD, at(c->qkv, QD, t), at(c->qkv, QD + KV, t), QKVD, d_attn_mask, delta,
                                         t->d_rope_cs, B, S, NH, NKV, HD, scale));
        TRY(bmc_matmul_backward_inp(be, dt, t->dn, D, 0, t->dqkv, QKVD, wptr(t, pb + P_Q), M, D, QKVD));
        SIDE_WGRAD(tk_q, bmc_matmul_backward_w(be, dt, gptr(t, pb + P_Q), t->dqkv, QKVD, c->n1, D, M, D, QKVD));
        SIDE_WAIT(tk_o);
        TRY(bmc_rmsnorm_backward(be, dt, t->dres, gptr(t, pb + P_LN1), nw_acc, t->dn, c->x, wf32(t, pb + P_LN1), c->rstd1, M, D, nw_r0, nw_r1));
        if (t->dp) {
            /* a gradient bucket may close here: every weight gradient of this layer must be behind the main stream */
            SIDE_WAIT(tk_gu);
            SIDE_WAIT(tk_q);
            TRY(bm_dp_bucket_ready(t->dp, l));
        }
    }
    SIDE_WAIT(tk_gu);
    SIDE_WAIT(tk_q);
    SIDE_WAIT(tk_head); /* the embedding scatter adds into the buffer the LM-head weight gradient accumulated into */
#undef SIDE_WGRAD
#undef SIDE_WAIT
    /* tied embedding: scatter dL/dx_0 on top of the LM-head wgrad already in the same buffer
     * (embed_backward, src/baremetal/trainer.c:302-346) */
    if (t->ref_input_grad_carry) TRY(bmc_seq_prefix_accumulate(be, dt, t->dres, t->d_gx_carry, B, (size_t)S * D));
    TRY(bmc_embedding_backward(be, dt, gptr(t, p_emb), t->dres, t->d_tokens, M, D, V));
    if (t->dp) TRY(bm_dp_bucket_ready(t->dp, -1));
    return 0;
}

/* AdamW over every parameter (adamw_apply, src/baremetal/trainer.c:349-398). */
static int adamw_apply(bm_trainer_t* t) {
    t->step++;
    const float b1 = t->cfg.beta1, b2 = t->cfg.beta2;
    const float bias1 = 1.0f - powf(b1, (float)t->step), bias2 = 1.0f - powf(b2, (float)t->step);
    int n_micro = t->window_microsteps > 0 ? t->window_microsteps : 1;
    if (t->dp) n_micro *= bm_dp_world(t->dp);
    const float hp[8] = {t->cfg.learning_rate, b1, b2, t->cfg.epsilon, t->cfg.weight_decay, bias1, bias2, 1.0f / (float)n_micro};
    int rc;
    if (t->dp) rc = bm_dp_adamw(t->dp, t, hp);
    else rc = bmc_adamw(t->ctx->be, t->d_master, t->d_wlow, t->d_grad, BMC_F32, t->d_m, t->d_v, t->P, hp);
    t->window_microsteps = 0;
    return rc;
}

/* Everything after the inputs are on the device; asynchronous. */
static int step_enqueue(bm_trainer_t* t, int B, const uint8_t* d_attn_mask, const float* d_row_weight, int train) {
    bmc_ctx_t* be = t->ctx->be;
    const int accum = t->cfg.grad_accum_steps > 0 ? t->cfg.grad_accum_steps : 1;
    t->loss_is_early = 0;
    if (train && t->accum_count == 0) {
        /* gradients accumulate over the B sequences and over micro-steps; cleared at the start of a window
         * (src/baremetal/trainer.c:459-470) */
        TRY(bmc_memset(be, t->d_grad, 0, t->P * sizeof(float)));
        if (t->ref_input_grad_carry) TRY(bmc_memset(be, t->d_gx_carry, 0, (size_t)t->S * t->model->arch.dim * sizeof(float)));
        if (t->dp) bm_dp_begin_window(t->dp);
    }
    /* The plain training step (no masks, one GPU, no profiling) replays its forward + backward as one CUDA graph from the third
     * step on: about 850 launches become one, which matters to the synchronous bm_train_step, where the host cannot run
     * ahead of the device. AdamW stays outside: its bias corrections change every step and travel as kernel arguments. */
    const int graphable = t->graph_mode && train && !d_attn_mask && !d_row_weight && !t->dp && !t->profile && !bmc_gemm_timing_enabled(be);
    if (graphable) {
        int replayed = 0;
        bmc_graph_select(be, 1);
        if (t->graph_seen_B != B) { /* scratch buffers are sized by eager steps of THIS batch before anything is captured */
            t->graph_seen_B = B;
            t->graph_eager_steps = 0;
            t->graph_B = 0;
        }
        if (t->graph_B == B) {
            if (bmc_graph_launch(be) == 0) replayed = 1;
            else t->graph_B = 0;
        } else if (t->graph_eager_steps >= 2) {
            int rc = bmc_graph_begin(be);
            if (rc == 0) {
                rc = forward_and_loss(t, B, NULL, NULL, 1);
                /* the loss is final here: hand it to the host now, so that bm_train_step can return (and its caller prepare the
                 * next batch) while backward and AdamW are still running */
                if (rc == 0) rc = bmc_early_readback(be, t->d_loss);
                if (rc == 0) rc = backward(t, B, NULL);
                const int rc2 = bmc_graph_end(be);
                if (rc == 0 && rc2 == 0 && bmc_graph_launch(be) == 0) {
                    t->graph_B = B;
                    replayed = 1;
                } else {
                    BM_LOG_ERROR("train step: CUDA graph capture failed (%d, %d); continuing without a graph", rc, rc2);
                    t->graph_mode = 0;
                }
            } else {
                t->graph_mode = 0;
            }
        }
        t->loss_is_early = replayed;
        if (replayed) {
            t->window_microsteps += B;
            t->accum_count++;
            if (t->accum_count >= accum) {
                TRY(adamw_apply(t));
                t->accum_count = 0;
            }
            return 0;
        }
        t->graph_eager_steps++;
    }
    if (t->profile) bmc_timer_begin(be, 0);
    TRY(forward_and_loss(t, B, d_attn_mask, d_row_weight, train));
    if (t->profile) {
        /* the loss kernels are the tail of forward_and_loss; attribute them separately by bracketing again */
        t->prof_forward_ms += bmc_timer_end(be, 0);
    }
    if (!train) return 0;
    if (t->profile) bmc_timer_begin(be, 1);
    if (t->dp) bm_dp_set_last_microstep(t->dp, t->accum_count + 1 >= accum);
    TRY(backward(t, B, d_attn_mask));
    if (t->profile) t->prof_backward_ms += bmc_timer_end(be, 1);
    t->window_microsteps += B;
    t->accum_count++;
    if (t->accum_count >= accum) {
        if (t->profile) bmc_timer_begin(be, 2);
        TRY(adamw_apply(t));
        if (t->profile) t->prof_opt_ms += bmc_timer_end(be, 2);
        t->accum_count = 0;
    }
    return 0;
}

static float read_loss(bm_trainer_t* t) {
    float loss = -1.0f;
    if (t->loss_is_early) {
        /* graph-replayed step: the loss and the error word were copied out right after the forward pass. Returning now leaves
         * backward and AdamW running; every later call goes through the same stream and so stays ordered behind them. An error raised
         * by backward shows in the error word of the NEXT step (or of any call that synchronises). */
        int st = 0;
        t->loss_is_early = 0;
        if (bmc_early_wait(t->ctx->be, &loss, &st) != 0) return -1.0f;
        if (st == 0) return loss;
        /* something failed: take the slow path below, which synchronises, reports and clears */
    }
    if (bmc_download(t->ctx->be, &loss, t->d_loss, sizeof(float)) != 0) return -1.0f;
    const int st = bmc_status(t->ctx->be);
    if (st) {
        BM_LOG_ERROR("train step: backend reported status %d", st);
        return -1.0f;
    }
    if (t->dp) loss = bm_dp_mean_loss(t->dp, loss);
    return loss;
}

static float step_host(bm_trainer_t* t, const int* inputs, const int* targets, const uint8_t* attn_mask, const uint8_t* loss_mask,
                       int B, int T, int train) {
    if (!t || !inputs || !targets || B <= 0) return -1.0f;
    if (T != t->S) {
        BM_LOG_ERROR("bm_train_step: S=%d != trainer S=%d (rebuild trainer for new S)", T, t->S);
        return -1.0f;
    }
    /* Ids index device memory (embedding gather and scatter, the target logit): a value outside [0, vocab_size) is refused here,
     * before anything is uploaded or enqueued. A target on a row that the loss mask excludes is never read (as in
     * xent_backward_masked, src/kernels/backward.metal:609-612), so ignore markers such as -100 are fine there. */
    {
        const int V = t->model->arch.vocab_size;
        const size_t n = (size_t)B * T;
        for (size_t i = 0; i < n; ++i) {
            if ((unsigned)inputs[i] >= (unsigned)V) {
                BM_LOG_ERROR("bm_train_step: input id %d at position %zu is outside the vocabulary [0, %d)", inputs[i], i, V);
                return -1.0f;
            }
            if ((!loss_mask || loss_mask[i]) && (unsigned)targets[i] >= (unsigned)V) {
                BM_LOG_ERROR("bm_train_step: target id %d at position %zu is outside the vocabulary [0, %d)", targets[i], i, V);
                return -1.0f;
            }
        }
    }
    if (ensure_batch(t, B) != 0) return -1.0f;
    bmc_ctx_t* be = t->ctx->be;
    const size_t M = (size_t)B * T;
    /* stage through pinned memory so the copies are truly asynchronous */
    memcpy(t->h_stage, inputs, M * sizeof(int));
    memcpy(t->h_stage + M, targets, M * sizeof(int));
    float* hw = (float*)(t->h_stage + 2 * M);
    uint8_t* hm = (uint8_t*)(t->h_stage + 3 * M);
    if (attn_mask) memcpy(hm, attn_mask, M);
    if (loss_mask) {
        /* completion-only loss: every unmasked row of sequence b weighs 1 / count_b (the reference divides by the number of
         * unmasked rows, src/baremetal/scheduler.c:1661-1676, src/kernels/backward.metal:620); a sequence without any unmasked
         * row contributes zero loss and zero gradient (scheduler.c:1679-1684) */
        for (int b = 0; b < B; ++b) {
            int count = 0;
            for (int s = 0; s < T; ++s) count += loss_mask[(size_t)b * T + s] ? 1 : 0;
            const float w = count > 0 ? 1.0f / (float)count : 0.0f;
            for (int s = 0; s < T; ++s) hw[(size_t)b * T + s] = loss_mask[(size_t)b * T + s] ? w : 0.0f;
        }
    }
    bmc_upload(be, t->d_tokens, t->h_stage, M * sizeof(int));
    bmc_upload(be, t->d_targets, t->h_stage + M, M * sizeof(int));
    if (attn_mask) bmc_upload(be, t->d_attn_mask, hm, M);
    if (loss_mask) bmc_upload(be, t->d_row_weight, hw, M * sizeof(float));
    if (step_enqueue(t, B, attn_mask ? t->d_attn_mask : NULL, loss_mask ? t->d_row_weight : NULL, train) != 0) return -1.0f;
    return read_loss(t);
}

float bm_train_step_masked(bm_trainer_t* t, const int* inputs, const int* targets, const uint8_t* attn_mask, const uint8_t* loss_mask,
                           int B, int T) {
    return step_host(t, inputs, targets, attn_mask, loss_mask, B, T, 1);
}
float bm_train_step(bm_trainer_t* t, const int* inputs, const int* targets, int B, int T) {
    return step_host(t, inputs, targets, NULL, NULL, B, T, 1);
}
/* forward + loss only (bm_train_eval_masked, src/baremetal/trainer.c:425-445) */
float bm_train_eval_masked(bm_trainer_t* t, const int* inputs, const int* targets, const uint8_t* attn_mask, const uint8_t* loss_mask,
                           int B, int T) {
    return step_host(t, inputs, targets, attn_mask, loss_mask, B, T, 0);
}

/* Applies the gradients of a window that has not reached grad_accum_steps micro-steps (bm_train_flush, src/baremetal/trainer.c:535-543).
 * Under data parallel this is a collective call: the micro-steps so far never exchanged their gradients (only a window's last
 * micro-step does), so every rank all-reduces the whole gradient here before AdamW. */
void bm_train_flush(bm_trainer_t* t) {
    if (!t) return;
    if (t->accum_count > 0) {
        if (t->dp && bm_dp_reduce_all(t->dp) != 0) {
            BM_LOG_ERROR("bm_train_flush: gradient exchange failed; the partial window is dropped");
            t->accum_count = 0;
            t->window_microsteps = 0;
            return;
        }
        adamw_apply(t);
        t->accum_count = 0;
        bmc_sync(t->ctx->be);
    }
}

int bmx_train_step_resident(bm_trainer_t* t, const int* d_inputs, const int* d_targets, int B, int T) {
    if (!t || !d_inputs || !d_targets || B <= 0 || T != t->S) return -1;
    if (ensure_batch(t, B) != 0) return -1;
    const size_t M = (size_t)B * T;
    bmc_copy(t->ctx->be, t->d_tokens, d_inputs, M * sizeof(int));
    bmc_copy(t->ctx->be, t->d_targets, d_targets, M * sizeof(int));
    return step_enqueue(t, B, NULL, NULL, 1);
}
float bmx_train_last_loss(bm_trainer_t* t) { return t ? read_loss(t) : -1.0f; }

/* ---- profiling (bm_train_profile_begin/end, src/baremetal/trainer.c:406-423): GPU time per phase ------ */
void bm_train_profile_begin(bm_trainer_t* t) {
    if (!t) return;
    t->profile = 1;
    t->prof_forward_ms = t->prof_loss_ms = t->prof_backward_ms = t->prof_opt_ms = 0.0;
}
void bm_train_profile_end(bm_trainer_t* t, double* forward_ms, double* loss_ms, double* backward_ms, double* optimizer_ms) {
    if (!t) return;
    if (forward_ms) *forward_ms = t->prof_forward_ms;
    if (loss_ms) *loss_ms = t->prof_loss_ms;
    if (backward_ms) *backward_ms = t->prof_backward_ms;
    if (optimizer_ms) *optimizer_ms = t->prof_opt_ms;
    t->profile = 0;
}

/* ---- trainer state file (bm_save_state / bm_load_state, src/baremetal/trainer.c:144-262) ----------------
 * int32 step; int32 n_states; n_states x { size_t n; float w[n]; float m[n]; float v[n] }, native endianness. */
void bm_save_state(bm_trainer_t* t, const char* path) {
    if (!t || !path) return;
    FILE* f = fopen(path, "wb");
    if (!f) {
        BM_LOG_ERROR("bm_save_state: cannot open %s", path);
        return;
    }
    bmc_ctx_t* be = t->ctx->be;
    const int step = t->step, n_states = t->n_params;
    fwrite(&step, sizeof(int), 1, f);
    fwrite(&n_states, sizeof(int), 1, f);
    size_t max_n = 0;
    for (int i = 0; i < n_states; ++i) if (t->params[i].n > max_n) max_n = t->params[i].n;
    float* buf = (float*)malloc(max_n * sizeof(float));
    int ok = buf != NULL;
    for (int i = 0; i < n_states && ok; ++i) {
        const size_t n = t->params[i].n, off = t->params[i].off;
        fwrite(&n, sizeof(size_t), 1, f);
        const float* srcs[3] = {t->d_master + off, t->d_m + off, t->d_v + off};
        for (int k = 0; k < 3 && ok; ++k) {
            if (bmc_download(be, buf, srcs[k], n * sizeof(float)) != 0 || fwrite(buf, sizeof(float), n, f) != n) ok = 0;
        }
    }
    free(buf);
    fclose(f);
    if (!ok) BM_LOG_ERROR("bm_save_state: write to %s failed", path);
    else BM_LOG_INFO("bm_save_state: saved step=%d, %d weight tensors to %s", step, n_states, path);
}

void bm_load_state(bm_trainer_t* t, const char* path) {
    if (!t || !path) return;
    FILE* f = fopen(path, "rb");
    if (!f) {
        BM_LOG_ERROR("bm_load_state: cannot open %s", path);
        return;
    }
    int step, n_states;
    if (fread(&step, sizeof(int), 1, f) != 1 || fread(&n_states, sizeof(int), 1, f) != 1) {
        BM_LOG_ERROR("bm_load_state: failed to read header");
        fclose(f);
        return;
    }
    if (n_states != t->n_params) {
        BM_LOG_ERROR("bm_load_state: state has %d tensors, trainer has %d", n_states, t->n_params);
        fclose(f);
        return;
    }
    bmc_ctx_t* be = t->ctx->be;
    size_t max_n = 0;
    for (int i = 0; i < n_states; ++i) if (t->params[i].n > max_n) max_n = t->params[i].n;
    float* buf = (float*)malloc(max_n * sizeof(float));
    if (!buf) { fclose(f); return; }
    t->step = step;
    for (int i = 0; i < n_states; ++i) {
        size_t n;
        if (fread(&n, sizeof(size_t), 1, f) != 1 || n != t->params[i].n) {
            BM_LOG_ERROR("bm_load_state: tensor %d size mismatch", i);
            break;
        }
        const size_t off = t->params[i].off;
        float* dsts[3] = {t->d_master + off, t->d_m + off, t->d_v + off};
        int bad = 0;
        for (int k = 0; k < 3; ++k) {
            if (fread(buf, sizeof(float), n, f) != n) { bad = 1; break; }
            bmc_upload(be, dsts[k], buf, n * sizeof(float));
            bmc_sync(be); /* buf is pageable and reused */
        }
        if (bad) {
            BM_LOG_ERROR("bm_load_state: failed to read tensor %d data", i);
            break;
        }
    }
    if (t->d_wlow) bmc_cast_f32_to_bf16(be, t->d_wlow, t->d_master, t->P);
    bmc_sync(be);
    free(buf);
    fclose(f);
    BM_LOG_INFO("bm_load_state: loaded step=%d, %d weight tensors from %s", step, n_states, path);
}

/* ---- introspection (include/baremetal_ext.h) ----------------------------------------------------------- */
int bmx_trainer_num_tensors(bm_trainer_t* t) { return t ? t->n_params : 0; }
size_t bmx_trainer_tensor_size(bm_trainer_t* t, int i) { return (t && i >= 0 && i < t->n_params) ? t->params[i].n : 0; }
int bmx_trainer_read(bm_trainer_t* t, int what, int i, float* host_out) {
    if (!t || i < 0 || i >= t->n_params || !host_out) return -1;
    const float* base = what == BMX_WEIGHT ? t->d_master : what == BMX_GRAD ? t->d_grad : what == BMX_ADAM_M ? t->d_m : what == BMX_ADAM_V ? t->d_v : NULL;
    if (!base) return -1;
    return bmc_download(t->ctx->be, host_out, base + t->params[i].off, t->params[i].n * sizeof(float));
}
int bmx_trainer_set_option(bm_trainer_t* t, const char* key, int value) {
    if (!t || !key) return -1;
    bmc_ctx_t* be = t->ctx->be;
    const int all = strcmp(key, "ref_quirks") == 0;
    int known = 0;
    /* any switch changes what a step enqueues: a captured graph is dropped and re-made after two eager steps */
    t->graph_B = 0;
    t->graph_eager_steps = 0;
    if (strcmp(key, "side_stream") == 0) { t->side_stream = value ? 1 : 0; return 0; }
    if (strcmp(key, "train_graph") == 0) { t->graph_mode = value ? 1 : 0; return 0; }
    if (strcmp(key, "fused_epilogues") == 0) { t->fuse = value ? 1 : 0; return 0; }
    if (all || strcmp(key, "ref_norm_grad") == 0) { t->ref_norm_grad = value ? 1 : 0; known = 1; }
    if (all || strcmp(key, "ref_input_grad_carry") == 0) {
        known = 1;
        t->ref_input_grad_carry = value ? 1 : 0;
        if (value && !t->d_gx_carry) {
            const size_t n = (size_t)t->S * t->model->arch.dim;
            t->d_gx_carry = (float*)bmc_alloc(be, n * sizeof(float));
            if (!t->d_gx_carry) return -1;
            bmc_memset(be, t->d_gx_carry, 0, n * sizeof(float));
        }
    }
    if (all || strcmp(key, "ref_stale_embedding") == 0) {
        known = 1;
        if (value && !t->d_embed_frozen && t->dtype == BMC_F32) {
            const bm_param_t* pe = &t->params[t->n_params - 1];
            t->d_embed_frozen = (float*)bmc_alloc(be, pe->n * sizeof(float));
            if (!t->d_embed_frozen) return -1;
            bmc_copy(be, t->d_embed_frozen, t->d_master + pe->off, pe->n * sizeof(float));
        } else if (!value && t->d_embed_frozen) {
            bmc_free(be, t->d_embed_frozen);
            t->d_embed_frozen = NULL;
        }
    }
    return known ? 0 : -1;
}
/* Copies the fp32 master weights from the device back into the model the trainer was created from, so that bm_save_weights
 * exports the trained weights. */
int bmx_trainer_sync_model(bm_trainer_t* t) {
    if (!t) return -1;
    for (int i = 0; i < t->n_params; ++i)
        if (bmc_download(t->ctx->be, t->params[i].host_src, t->d_master + t->params[i].off, t->params[i].n * sizeof(float)) != 0) return -2;
    return 0;
}
long bmx_trainer_launch_count(bm_trainer_t* t) { return t ? bmc_launch_count(t->ctx->be) : 0; }
size_t bmx_trainer_device_bytes(bm_trainer_t* t) { return t ? bmc_allocated_bytes(t->ctx->be) : 0; }
