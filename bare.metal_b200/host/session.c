/* Inference session: prefill and token-by-token decode with a KV cache, Q8 / bf16 / fp32 weights and fp32 activations.
 * Counterpart of the reference's session + decode scheduler walk (src/baremetal/session.c:34-185,
 * src/baremetal/scheduler.c:712-996, decode graph src/baremetal/graph.c:109-240):
 *   per layer  RMSNorm -> Q,K,V GEMV -> RoPE at the current position -> K,V into the cache -> attention over the cache ->
 *              O GEMV + residual -> RMSNorm -> gate,up GEMV -> SwiGLU -> down GEMV + residual;
 *   then       final RMSNorm -> LM-head GEMV (never quantised, src/baremetal/graph.c:228-239) -> logits.
 * Q8 quantisation is the reference's (bmt_quantize_q8, src/baremetal/quant.c:10-29,54-60): per 32 weights of a row,
 * scale = amax / 127, q = lroundf(w / scale) clamped to [-128, 127]; applied to every 2-D layer matrix.
 * Q4 (bmt_quantize_q4, src/baremetal/quant.c:31-52) is the same scheme with scale = amax / 7 and q clamped to [-8, 7]. The
 * reference multiplies x * ((float)q * scale) for both widths (matmul_forward_q8 / matmul_forward_q4, src/kernels/forward.metal:
 * 575-650, 830-858). On the device a Q4 matrix is the reference's block content as two arrays: two codes per byte (element 2j of a
 * row in the low, 2j+1 in the high nibble of byte j) and the scales, 0.625 bytes per weight.
 * The whole step is enqueued without host synchronisation and, after the first token, replayed as a CUDA graph; the
 * position lives in device memory. bm_forward with several tokens runs the same step per token, which the reference
 * establishes as equivalent to its sequence prefill (test/prefill_test.c).
 * The public API drives one sequence; bmx_create_session_batched runs NB independent sequences in lock step. */
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "bm_internal.h"

typedef struct {
    void* w;       /* int8 q[OC][C] (Q8), uint8 [OC][C/2] (Q4, two codes per byte), or bf16 / fp32 [OC][C] */
    float* scales; /* Q8 and Q4: [OC][C/32] */
    void* wx;      /* tensor-core path only: bf16 [OC][parts * C], [w | w] or [w_hi | w_hi | w_lo] of the SAME weight values */
    int parts;
    int OC, C;
} bm_mat_t;

#define BM_TC_MIN_SEQUENCES 8 /* from this many sequences on, the products run as tensor-core GEMMs */

typedef struct {
    float *ln1, *ln2;
    bm_mat_t qkv, o, gu, down;
} bm_dec_layer_t;

struct bm_session_s {
    bm_context_t* ctx;
    bm_model_t* model;
    int NB, MS, pos, wtype, head_type;
    bm_dec_layer_t* layers;
    float* lnf;
    void* head;   /* [V, D] bf16 or fp32: LM head */
    float* embed; /* [V, D] fp32 embedding table as loaded (src/baremetal/session.c:114-123); aliases head in fp32 mode */
    void* cache;   /* [L][2][NB][MS][KV], fp32 (the reference's layout) or bf16 (bmx_create_session_kv) */
    int kv_dtype;  /* BMC_F32 or BMC_BF16 */
    float *cs, *x, *xn, *qkv, *att, *x1, *gu, *act, *logits;
    int *d_pos, *d_tokens, *d_next, *d_gen;
    void* att_scratch;
    void* a_op; /* tensor-core path: bf16 split operand rows */
    void* pf_buf; /* prefill scratch, grows to the largest prompt seen */
    size_t pf_bytes;
    void* head_wx;
    int head_parts, tc, tc_weights;
    int gen_cap;
    float* h_logits;
    int graph_ready;
};

/* reference quantiser, one 32-wide block (src/baremetal/quant.c:10-29) */
static void quantize_q8_block(const float* p, float* scale_out, int8_t* q) {
    float amax = 0.0f;
    for (int i = 0; i < 32; i++) {
        const float a = fabsf(p[i]);
        if (a > amax) amax = a;
    }
    const float scale = amax / 127.0f;
    *scale_out = scale;
    if (scale == 0.0f) {
        memset(q, 0, 32);
        return;
    }
    const float inv = 1.0f / scale;
    for (int i = 0; i < 32; i++) {
        long v = lroundf(p[i] * inv);
        if (v > 127) v = 127;
        if (v < -128) v = -128;
        q[i] = (int8_t)v;
    }
}
/* exported for tests: quantise n floats (n % 32 == 0) into q[n] and scales[n/32] */
size_t bmx_quantize_q8(const float* src, int8_t* q, float* scales, size_t n) {
    if (n == 0 || (n % 32) != 0) return 0;
    for (size_t b = 0; b < n / 32; b++) quantize_q8_block(src + b * 32, &scales[b], q + b * 32);
    return n / 32;
}

/* one 32-wide block of the reference's 4-bit quantiser (src/baremetal/quant.c:31-52), codes left unpacked: the reference stores
 * code 2j in the low and code 2j+1 in the high nibble of byte j and sign-extends them again in its kernels */
static void quantize_q4_block(const float* p, float* scale_out, int8_t* q) {
    float amax = 0.0f;
    for (int i = 0; i < 32; i++) {
        const float a = fabsf(p[i]);
        if (a > amax) amax = a;
    }
    const float scale = amax / 7.0f;
    *scale_out = scale;
    if (scale == 0.0f) {
        memset(q, 0, 32);
        return;
    }
    const float inv = 1.0f / scale;
    for (int i = 0; i < 32; i++) {
        long v = lroundf(p[i] * inv);
        if (v > 7) v = 7;
        if (v < -8) v = -8;
        q[i] = (int8_t)v;
    }
}
/* exported for tests: as bmx_quantize_q8, with codes in [-8, 7] */
size_t bmx_quantize_q4(const float* src, int8_t* q, float* scales, size_t n) {
    if (n == 0 || (n % 32) != 0) return 0;
    for (size_t b = 0; b < n / 32; b++) quantize_q4_block(src + b * 32, &scales[b], q + b * 32);
    return n / 32;
}
static size_t quantize_blocks(int bits, const float* src, int8_t* q, float* scales, size_t n) {
    return bits == 4 ? bmx_quantize_q4(src, q, scales, n) : bmx_quantize_q8(src, q, scales, n);
}

/* upload `rows` (OC x C fp32, given as up to three row blocks that are concatenated) in the session's weight type */
static int upload_matrix(bm_session_t* s, bm_mat_t* m, int wtype, const float* const* parts, const int* part_rows, int n_parts, int C) {
    bmc_ctx_t* be = s->ctx->be;
    int OC = 0;
    for (int i = 0; i < n_parts; i++) OC += part_rows[i];
    m->OC = OC;
    m->C = C;
    const size_t n = (size_t)OC * C;
    float* host = (float*)malloc(n * sizeof(float));
    if (!host) return -1;
    size_t off = 0;
    for (int i = 0; i < n_parts; i++) {
        memcpy(host + off, parts[i], (size_t)part_rows[i] * C * sizeof(float));
        off += (size_t)part_rows[i] * C;
    }
    int rc = 0;
    if (wtype == BMC_W_Q8 || wtype == BMC_W_Q4) {
        /* quantised from the loaded values; a bf16 checkpoint was widened exactly, so this equals the reference's
         * bmt_quantize_q8_bf16 / _q4_bf16 for bf16 sources and bmt_quantize_q8 / _q4 for fp32 ones (src/baremetal/scheduler.c:378-392) */
        int8_t* q = (int8_t*)malloc(n);
        float* sc = (float*)malloc(n / 32 * sizeof(float));
        quantize_blocks(wtype == BMC_W_Q4 ? 4 : 8, host, q, sc, n);
        size_t wbytes = n;
        if (wtype == BMC_W_Q4) {
            /* the reference's nibble order (src/baremetal/quant.c:44-50); C is even, so a byte never straddles two rows */
            uint8_t* pk = (uint8_t*)q;
            for (size_t j = 0; j < n / 2; j++) pk[j] = (uint8_t)(((uint8_t)q[2 * j] & 0x0F) | (((uint8_t)q[2 * j + 1] & 0x0F) << 4));
            wbytes = n / 2;
        }
        m->w = bmc_alloc(be, wbytes);
        m->scales = (float*)bmc_alloc(be, n / 32 * sizeof(float));
        if (!m->w || !m->scales) rc = -1;
        else { bmc_upload(be, m->w, q, wbytes); bmc_upload(be, m->scales, sc, n / 32 * sizeof(float)); bmc_sync(be); }
        free(q);
        free(sc);
    } else if (wtype == BMC_W_BF16) {
        uint16_t* h = (uint16_t*)malloc(n * 2);
        bm_f32_to_bf16_array(host, h, n);
        m->w = bmc_alloc(be, n * 2);
        if (!m->w) rc = -1;
        else { bmc_upload(be, m->w, h, n * 2); bmc_sync(be); }
        free(h);
    } else {
        m->w = bmc_alloc(be, n * sizeof(float));
        if (!m->w) rc = -1;
        else { bmc_upload(be, m->w, host, n * sizeof(float)); bmc_sync(be); }
    }
    if (rc == 0 && s->tc_weights) {
        /* the values the GEMV path would multiply with, split into bf16 hi + lo (lo is zero for bf16 weights) */
        const int parts = wtype == BMC_W_BF16 ? 2 : 3;
        float* eff = (float*)malloc(n * sizeof(float));
        uint16_t* hi = (uint16_t*)malloc(n * 2);
        uint16_t* lo = (uint16_t*)malloc(n * 2);
        uint16_t* wx = (uint16_t*)malloc(n * 2 * parts);
        if (wtype == BMC_W_Q8 || wtype == BMC_W_Q4) {
            int8_t* q = (int8_t*)malloc(n);
            float* sc = (float*)malloc(n / 32 * sizeof(float));
            quantize_blocks(wtype == BMC_W_Q4 ? 4 : 8, host, q, sc, n);
            for (size_t i = 0; i < n; i++) eff[i] = (float)q[i] * sc[i / 32];
            free(q);
            free(sc);
        } else {
            memcpy(eff, host, n * sizeof(float));
        }
        bm_f32_to_bf16_array(eff, hi, n);
        bm_bf16_to_f32_array(hi, host, n);
        for (size_t i = 0; i < n; i++) eff[i] -= host[i];
        bm_f32_to_bf16_array(eff, lo, n);
        for (int r = 0; r < OC; r++) {
            uint16_t* d = wx + (size_t)r * parts * C;
            memcpy(d, hi + (size_t)r * C, (size_t)C * 2);
            memcpy(d + C, hi + (size_t)r * C, (size_t)C * 2);
            if (parts == 3) memcpy(d + 2 * (size_t)C, lo + (size_t)r * C, (size_t)C * 2);
        }
        m->parts = parts;
        m->wx = bmc_alloc(be, n * 2 * parts);
        if (!m->wx) rc = -1;
        else { bmc_upload(be, m->wx, wx, n * 2 * parts); bmc_sync(be); }
        free(eff); free(hi); free(lo); free(wx);
    }
    free(host);
    return rc;
}

static float* upload_f32(bm_session_t* s, const float* src, size_t n) {
    float* d = (float*)bmc_alloc(s->ctx->be, n * sizeof(float));
    if (d) bmc_upload(s->ctx->be, d, src, n * sizeof(float));
    return d;
}

bm_session_t* bmx_create_session_batched(bm_context_t* ctx, bm_model_t* model, int n_sequences, int max_positions) {
    return bmx_create_session_kv(ctx, model, n_sequences, max_positions, getenv("BM_KV_BF16") ? 1 : 0);
}

/* kv_bf16 = 0: fp32 KV cache, the reference's (its kv buffers are fp32 whatever the weight precision) and what every parity test
 * runs. kv_bf16 = 1: keys and values are rounded to bf16 when they enter the cache, which halves the bytes the attention of a
 * decode step reads — the one memory-bound part of batched decode. head_dim 64 only. */
bm_session_t* bmx_create_session_kv(bm_context_t* ctx, bm_model_t* model, int n_sequences, int max_positions, int kv_bf16) {
    if (!ctx || !ctx->be || !model || !model->weight_buffer || n_sequences < 1) return NULL;
    if (kv_bf16 && model->head_size != 64) {
        BM_LOG_ERROR("bm_create_session: a bf16 KV cache needs head_dim 64");
        return NULL;
    }
    const bm_arch_t* a = &model->arch;
    if (model->precision == BM_PRECISION_FP16) {
        BM_LOG_ERROR("bm_create_session: fp16 weights are not supported by this backend");
        return NULL;
    }
    if ((a->dim % 32) || (a->hidden_dim % 32) || ((a->n_heads * model->head_size) % 32)) {
        BM_LOG_ERROR("bm_create_session: layer widths must be multiples of 32");
        return NULL;
    }
    bm_session_t* s = (bm_session_t*)calloc(1, sizeof *s);
    if (!s) return NULL;
    s->ctx = ctx;
    s->model = model;
    s->NB = n_sequences;
    s->kv_dtype = kv_bf16 ? BMC_BF16 : BMC_F32;
    s->tc_weights = !getenv("BM_NO_TC_DECODE"); /* split-bf16 copies: prefill of any session, decode of batched ones */
    s->tc = s->tc_weights && n_sequences >= BM_TC_MIN_SEQUENCES;
    s->MS = max_positions > 0 ? max_positions : (a->max_seq_len > 0 ? a->max_seq_len : 2048);
    const int lowp = model->precision == BM_PRECISION_BF16;
    s->wtype = model->quant_bits == 8 ? BMC_W_Q8 : model->quant_bits == 4 ? BMC_W_Q4 : (lowp ? BMC_W_BF16 : BMC_W_F32);
    s->head_type = lowp ? BMC_W_BF16 : BMC_W_F32;
    bmc_ctx_t* be = ctx->be;
    const int L = a->n_layers, D = a->dim, H = a->hidden_dim, V = a->vocab_size, HD = model->head_size;
    const int QD = a->n_heads * HD, KV = model->kv_dim, NB = s->NB, MS = s->MS;
    s->layers = (bm_dec_layer_t*)calloc(L, sizeof(bm_dec_layer_t));
    int ok = s->layers != NULL;
    for (int l = 0; l < L && ok; l++) {
        bm_dec_layer_t* y = &s->layers[l];
        y->ln1 = upload_f32(s, model->ln1w + (size_t)l * D, D);
        y->ln2 = upload_f32(s, model->ln2w + (size_t)l * D, D);
        const float* p3[3] = {model->qw + (size_t)l * QD * D, model->kw + (size_t)l * KV * D, model->vw + (size_t)l * KV * D};
        const int r3[3] = {QD, KV, KV};
        const float* po[1] = {model->ow + (size_t)l * D * QD};
        const int ro[1] = {D};
        const float* pg[2] = {model->gate + (size_t)l * H * D, model->up + (size_t)l * H * D};
        const int rg[2] = {H, H};
        const float* pd[1] = {model->down + (size_t)l * D * H};
        const int rd[1] = {D};
        ok = y->ln1 && y->ln2 && upload_matrix(s, &y->qkv, s->wtype, p3, r3, 3, D) == 0 && upload_matrix(s, &y->o, s->wtype, po, ro, 1, QD) == 0 &&
             upload_matrix(s, &y->gu, s->wtype, pg, rg, 2, D) == 0 && upload_matrix(s, &y->down, s->wtype, pd, rd, 1, H) == 0;
    }
    if (ok) {
        s->lnf = upload_f32(s, model->lnfw, D);
        bm_mat_t head = {0};
        const float* ph[1] = {model->embed};
        const int rh[1] = {V};
        ok = s->lnf && upload_matrix(s, &head, s->head_type, ph, rh, 1, D) == 0;
        s->head = head.w;
        s->head_wx = head.wx;
        s->head_parts = head.parts;
        if (ok && s->head_type == BMC_W_F32) s->embed = (float*)s->head;
        else if (ok) { s->embed = upload_f32(s, model->embed, (size_t)V * D); ok = s->embed != NULL; }
    }
    /* RoPE table with the reference's fp32 formula (rope_inv_freq, src/kernels/forward.metal:1260-1279) */
    if (ok) {
        const int hd2 = HD / 2;
        float* cs = bm_build_rope_table_arch(a, MS, HD);   /* the same builder as the trainer: frequency scaling included */
        s->cs = cs ? upload_f32(s, cs, (size_t)MS * hd2 * 2) : NULL;
        if (!s->cs) ok = 0;
        bmc_sync(be);
        free(cs);
    }
#define DALLOC(p, n) do { (p) = bmc_alloc(be, (size_t)(n)); if (!(p)) ok = 0; } while (0)
    if (ok) {
        DALLOC(s->cache, (size_t)L * 2 * NB * MS * KV * (kv_bf16 ? 2 : sizeof(float)));
        DALLOC(s->x, (size_t)NB * D * 4); DALLOC(s->xn, (size_t)NB * D * 4); DALLOC(s->qkv, (size_t)NB * (QD + 2 * KV) * 4);
        DALLOC(s->att, (size_t)NB * QD * 4); DALLOC(s->x1, (size_t)NB * D * 4); DALLOC(s->gu, (size_t)NB * 2 * H * 4);
        DALLOC(s->act, (size_t)NB * H * 4); DALLOC(s->logits, (size_t)NB * V * 4);
        const size_t asb = bmc_decode_attention_scratch_bytes(NB, MS, a->n_heads, a->n_kv_heads, HD);
        DALLOC(s->att_scratch, asb);
        if (s->att_scratch) bmc_memset(be, s->att_scratch, 0, asb);
        if (s->tc) {
            int cmax = D > H ? D : H;
            if (QD > cmax) cmax = QD;
            DALLOC(s->a_op, (size_t)NB * 3 * cmax * 2);
        }
        DALLOC(s->d_pos, 16); DALLOC(s->d_tokens, (size_t)NB * 4); DALLOC(s->d_next, (size_t)NB * 4);
    }
#undef DALLOC
    s->h_logits = (float*)malloc((size_t)NB * V * sizeof(float));
    if (!ok || !s->cs || !s->h_logits) {
        BM_LOG_ERROR("bm_create_session: out of memory");
        bm_destroy_session(s);
        return NULL;
    }
    bmc_memset(be, s->d_pos, 0, 16);
    bmc_sync(be);
    return s;
}

bm_session_t* bm_create_session(bm_context_t* ctx, bm_model_t* model) { return bmx_create_session_batched(ctx, model, 1, 0); }

void bm_destroy_session(bm_session_t* s) {
    if (!s) return;
    bmc_ctx_t* be = s->ctx->be;
    bmc_sync(be);
    if (s->layers) {
        for (int l = 0; l < s->model->arch.n_layers; l++) {
            bm_dec_layer_t* y = &s->layers[l];
            bmc_free(be, y->ln1); bmc_free(be, y->ln2);
            bm_mat_t* ms[4] = {&y->qkv, &y->o, &y->gu, &y->down};
            for (int i = 0; i < 4; i++) { bmc_free(be, ms[i]->w); bmc_free(be, ms[i]->scales); bmc_free(be, ms[i]->wx); }
        }
        free(s->layers);
    }
    bmc_free(be, s->lnf); if ((void*)s->embed != s->head) bmc_free(be, s->embed); bmc_free(be, s->head); bmc_free(be, s->cache); bmc_free(be, s->cs); bmc_free(be, s->x); bmc_free(be, s->xn);
    bmc_free(be, s->qkv); bmc_free(be, s->att); bmc_free(be, s->x1); bmc_free(be, s->gu); bmc_free(be, s->act); bmc_free(be, s->logits);
    bmc_free(be, s->att_scratch); bmc_free(be, s->pf_buf); bmc_free(be, s->a_op); bmc_free(be, s->head_wx); bmc_free(be, s->d_pos); bmc_free(be, s->d_tokens); bmc_free(be, s->d_next); bmc_free(be, s->d_gen);
    free(s->h_logits);
    free(s);
}

void bm_reset_session(bm_session_t* s) {
    if (!s) return;
    s->pos = 0;
    bmc_memset(s->ctx->be, s->d_pos, 0, 4);
}

#define TRYS(call) do { int rc__ = (call); if (rc__) { BM_LOG_ERROR("decode step: %s failed (%d)", #call, rc__); return rc__; } } while (0)

/* one token for every sequence: tokens are in d_tokens, the position in d_pos; leaves logits, the greedy choice in d_next,
 * and advances the device position */
static int enqueue_step(bm_session_t* s) {
    bmc_ctx_t* be = s->ctx->be;
    const bm_arch_t* a = &s->model->arch;
    const int L = a->n_layers, D = a->dim, H = a->hidden_dim, V = a->vocab_size, HD = s->model->head_size, NH = a->n_heads, NKV = a->n_kv_heads;
    const int QD = NH * HD, KV = NKV * HD, NB = s->NB, MS = s->MS;
    const float scale = 1.0f / sqrtf((float)HD), eps = 1e-5f;
    TRYS(bmc_decode_embed(be, s->x, BMC_W_F32, s->embed, s->d_tokens, NB, D));
    /* few sequences: five kernels per layer, norms / RoPE / cache store / SwiGLU folded into their consumers */
    const int fused = NB < 4 && D <= 3072 && H <= 3072 && QD <= 3072;
    for (int l = 0; l < L; l++) {
        const bm_dec_layer_t* y = &s->layers[l];
        if (s->tc) {
            TRYS(bmc_decode_prep(be, s->a_op, y->qkv.parts, s->x, D, 1, y->ln1, eps, s->qkv, QD + 2 * KV, NULL, 0, QD + 2 * KV, NB, D));
            TRYS(bmc_decode_gemm(be, s->qkv, QD + 2 * KV, s->a_op, y->qkv.wx, y->qkv.parts, NB, D, QD + 2 * KV));
            TRYS(bmc_decode_attention_fused(be, s->att, s->qkv, s->cache, s->kv_dtype, s->cs, s->d_pos, s->att_scratch, l, NB, MS, NH, NKV, HD, scale));
            TRYS(bmc_decode_prep(be, s->a_op, y->o.parts, s->att, QD, 0, NULL, 0.0f, s->x1, D, s->x, D, D, NB, QD));
            TRYS(bmc_decode_gemm(be, s->x1, D, s->a_op, y->o.wx, y->o.parts, NB, QD, D));
            TRYS(bmc_decode_prep(be, s->a_op, y->gu.parts, s->x1, D, 1, y->ln2, eps, s->gu, 2 * H, NULL, 0, 2 * H, NB, D));
            TRYS(bmc_decode_gemm(be, s->gu, 2 * H, s->a_op, y->gu.wx, y->gu.parts, NB, D, 2 * H));
            TRYS(bmc_decode_prep(be, s->a_op, y->down.parts, s->gu, 2 * H, 2, NULL, 0.0f, s->x, D, s->x1, D, D, NB, H));
            TRYS(bmc_decode_gemm(be, s->x, D, s->a_op, y->down.wx, y->down.parts, NB, H, D));
            continue;
        }
        if (fused) {
            TRYS(bmc_decode_gemv_fused(be, s->qkv, QD + 2 * KV, s->x, D, s->wtype, y->qkv.w, y->qkv.scales, NULL, 0, 1, y->ln1, eps, NB, D, QD + 2 * KV));
            TRYS(bmc_decode_attention_fused(be, s->att, s->qkv, s->cache, s->kv_dtype, s->cs, s->d_pos, s->att_scratch, l, NB, MS, NH, NKV, HD, scale));
            TRYS(bmc_decode_gemv(be, s->x1, D, s->att, QD, s->wtype, y->o.w, y->o.scales, s->x, D, NB, QD, D));
            TRYS(bmc_decode_gemv_fused(be, s->gu, 2 * H, s->x1, D, s->wtype, y->gu.w, y->gu.scales, NULL, 0, 1, y->ln2, eps, NB, D, 2 * H));
            TRYS(bmc_decode_gemv_fused(be, s->x, D, s->gu, 2 * H, s->wtype, y->down.w, y->down.scales, s->x1, D, 2, NULL, 0.0f, NB, H, D));
            continue;
        }
        TRYS(bmc_decode_rmsnorm(be, s->xn, s->x, y->ln1, NB, D, eps));
        TRYS(bmc_decode_gemv(be, s->qkv, QD + 2 * KV, s->xn, D, s->wtype, y->qkv.w, y->qkv.scales, NULL, 0, NB, D, QD + 2 * KV));
        TRYS(bmc_decode_rope_kv(be, s->qkv, s->cache, s->kv_dtype, s->cs, s->d_pos, l, NB, MS, NH, NKV, HD));
        TRYS(bmc_decode_attention(be, s->att, s->qkv, s->cache, s->kv_dtype, s->d_pos, s->att_scratch, l, NB, MS, NH, NKV, HD, scale));
        TRYS(bmc_decode_gemv(be, s->x1, D, s->att, QD, s->wtype, y->o.w, y->o.scales, s->x, D, NB, QD, D));
        TRYS(bmc_decode_rmsnorm(be, s->xn, s->x1, y->ln2, NB, D, eps));
        TRYS(bmc_decode_gemv(be, s->gu, 2 * H, s->xn, D, s->wtype, y->gu.w, y->gu.scales, NULL, 0, NB, D, 2 * H));
        TRYS(bmc_decode_swiglu(be, s->act, s->gu, NB, H));
        TRYS(bmc_decode_gemv(be, s->x, D, s->act, H, s->wtype, y->down.w, y->down.scales, s->x1, D, NB, H, D));
    }
    if (s->tc) {
        TRYS(bmc_decode_prep(be, s->a_op, s->head_parts, s->x, D, 1, s->lnf, eps, s->logits, V, NULL, 0, V, NB, D));
        TRYS(bmc_decode_gemm(be, s->logits, V, s->a_op, s->head_wx, s->head_parts, NB, D, V));
    } else if (fused) {
        TRYS(bmc_decode_gemv_fused(be, s->logits, V, s->x, D, s->head_type, s->head, NULL, NULL, 0, 1, s->lnf, eps, NB, D, V));
    } else {
        TRYS(bmc_decode_rmsnorm(be, s->xn, s->x, s->lnf, NB, D, eps));
        TRYS(bmc_decode_gemv(be, s->logits, V, s->xn, D, s->head_type, s->head, NULL, NULL, 0, NB, D, V));
    }
    TRYS(bmc_decode_argmax_advance(be, s->d_next, s->logits, NB, V, s->d_pos));
    return 0;
}

/* the first step runs eagerly (it also sizes every kernel attribute); it is then captured once and replayed */
static int run_step(bm_session_t* s) {
    bmc_ctx_t* be = s->ctx->be;
    if (s->pos >= s->MS) {
        BM_LOG_ERROR("decode step: position %d exceeds the KV cache (%d)", s->pos, s->MS);
        return -1;
    }
    int rc;
    bmc_graph_select(be, 0);
    if (s->graph_ready == 2) {
        rc = bmc_graph_launch(be);
    } else if (s->graph_ready == 1) {
        rc = bmc_graph_begin(be);
        if (!rc) rc = enqueue_step(s);
        if (!rc) rc = bmc_graph_end(be);
        if (!rc) { s->graph_ready = 2; rc = bmc_graph_launch(be); }
        else { BM_LOG_ERROR("decode step: graph capture failed (%d), continuing without a graph", rc); s->graph_ready = -1; rc = enqueue_step(s); }
    } else {
        rc = enqueue_step(s);
        if (s->graph_ready == 0) s->graph_ready = getenv("BM_NO_GRAPH") ? -1 : 1;
    }
    if (!rc) s->pos++;
    return rc;
}

#define BM_PREFILL_MIN_TOKENS 8

/* Prompt pass from position 0 for every sequence at once (bm_prefill, src/baremetal/session.c:86-139): all T prompt rows go
 * through each layer together, products on the tensor cores, causal attention over the prompt, K and V copied into the cache.
 * tokens: NB x T (host). Leaves the last row's logits, the greedy choice in d_next and the position at T. */
static int prefill(bm_session_t* s, const int* tokens, int T) {
    bmc_ctx_t* be = s->ctx->be;
    const bm_arch_t* a = &s->model->arch;
    const int L = a->n_layers, D = a->dim, H = a->hidden_dim, V = a->vocab_size, HD = s->model->head_size, NH = a->n_heads, NKV = a->n_kv_heads;
    const int QD = NH * HD, KV = NKV * HD, NB = s->NB, MS = s->MS, W = QD + 2 * KV;
    const size_t R = (size_t)NB * T;
    const float scale = 1.0f / sqrtf((float)HD), eps = 1e-5f;
    int cmax = D > H ? D : H;
    if (QD > cmax) cmax = QD;
    /* one grow-only scratch allocation, carved into 256-byte aligned pieces */
    size_t sizes[8] = {R * D * 4, R * D * 4, R * W * 4, R * QD * 4, R * 2 * H * 4, (size_t)NB * NH * T * 4, R * 3 * cmax * 2, R * sizeof(int)};
    size_t offs[8], total = 0;
    for (int i = 0; i < 8; i++) { offs[i] = total; total += (sizes[i] + 255) / 256 * 256; }
    int rc = -1;
    if (total > s->pf_bytes) {
        bmc_sync(be);
        bmc_free(be, s->pf_buf);
        s->pf_buf = bmc_alloc(be, total);
        s->pf_bytes = s->pf_buf ? total : 0;
        if (!s->pf_buf) { BM_LOG_ERROR("prefill: out of memory (%zu bytes)", total); return -1; }
    }
    char* base = (char*)s->pf_buf;
    float *x = (float*)(base + offs[0]), *x1 = (float*)(base + offs[1]), *qkv = (float*)(base + offs[2]), *att = (float*)(base + offs[3]);
    float *gu = (float*)(base + offs[4]), *lse = (float*)(base + offs[5]);
    void* aop = base + offs[6];
    int* dtok = (int*)(base + offs[7]);
#define TRYP(call) do { rc = (call); if (rc) { BM_LOG_ERROR("prefill: %s failed (%d)", #call, rc); goto done; } } while (0)
    TRYP(bmc_upload(be, dtok, tokens, R * sizeof(int)));
    TRYP(bmc_decode_embed(be, x, BMC_W_F32, s->embed, dtok, (int)R, D));
    for (int l = 0; l < L; l++) {
        const bm_dec_layer_t* y = &s->layers[l];
        TRYP(bmc_decode_prep(be, aop, y->qkv.parts, x, D, 1, y->ln1, eps, qkv, W, NULL, 0, W, (int)R, D));
        TRYP(bmc_decode_gemm(be, qkv, W, aop, y->qkv.wx, y->qkv.parts, (int)R, D, W));
        TRYP(bmc_rope(be, BMC_F32, qkv, W, qkv + QD, W, s->cs, (int)R, T, NH, NKV, HD, 1));
        TRYP(bmc_decode_kv_scatter(be, s->cache, s->kv_dtype, qkv, W, l, NB, T, MS, QD, KV));
        if (HD == 64) TRYP(bmc_prefill_attention(be, att, QD, qkv, W, qkv + QD, qkv + QD + KV, W, NB, T, NH, NKV, HD, scale));
        else TRYP(bmc_attention_forward(be, BMC_F32, att, QD, lse, qkv, W, qkv + QD, qkv + QD + KV, W, NULL, NB, T, NH, NKV, HD, scale));
        TRYP(bmc_decode_prep(be, aop, y->o.parts, att, QD, 0, NULL, 0.0f, x1, D, x, D, D, (int)R, QD));
        TRYP(bmc_decode_gemm(be, x1, D, aop, y->o.wx, y->o.parts, (int)R, QD, D));
        TRYP(bmc_decode_prep(be, aop, y->gu.parts, x1, D, 1, y->ln2, eps, gu, 2 * H, NULL, 0, 2 * H, (int)R, D));
        TRYP(bmc_decode_gemm(be, gu, 2 * H, aop, y->gu.wx, y->gu.parts, (int)R, D, 2 * H));
        TRYP(bmc_decode_prep(be, aop, y->down.parts, gu, 2 * H, 2, NULL, 0.0f, x, D, x1, D, D, (int)R, H));
        TRYP(bmc_decode_gemm(be, x, D, aop, y->down.wx, y->down.parts, (int)R, H, D));
    }
    /* only the last row of each sequence feeds the classifier */
    TRYP(bmc_decode_prep(be, aop, s->head_parts, x + (size_t)(T - 1) * D, T * D, 1, s->lnf, eps, s->logits, V, NULL, 0, V, NB, D));
    TRYP(bmc_decode_gemm(be, s->logits, V, aop, s->head_wx, s->head_parts, NB, D, V));
    TRYP(bmc_decode_argmax(be, s->d_next, s->logits, NB, V));
    TRYP(bmc_upload(be, s->d_pos, &T, sizeof(int)));
    TRYP(bmc_sync(be));
    s->pos = T;
#undef TRYP
done:
    return rc;
}
static int can_prefill(const bm_session_t* s, int T) {
    return s->tc_weights && s->pos == 0 && T >= BM_PREFILL_MIN_TOKENS && T <= s->MS && !getenv("BM_NO_PREFILL");
}

float* bm_step(bm_session_t* s, int token) {
    if (!s || s->NB != 1) return NULL;
    bmc_ctx_t* be = s->ctx->be;
    if (token < 0 || token >= s->model->arch.vocab_size) return NULL;
    if (bmc_upload(be, s->d_tokens, &token, sizeof(int)) != 0 || bmc_sync(be) != 0) return NULL; /* `token` is a stack variable */
    if (run_step(s) != 0) return NULL;
    if (bmc_download(be, s->h_logits, s->logits, (size_t)s->model->arch.vocab_size * sizeof(float)) != 0) return NULL;
    return s->h_logits;
}

/* n tokens from the current position; returns the logits after the last one (bm_forward, src/baremetal/session.c:86-149) */
float* bm_forward(bm_session_t* s, const int* tokens, int n_tokens) {
    if (!s || s->NB != 1 || !tokens || n_tokens < 1) return NULL;
    bmc_ctx_t* be = s->ctx->be;
    for (int i = 0; i < n_tokens; i++)
        if (tokens[i] < 0 || tokens[i] >= s->model->arch.vocab_size) return NULL;
    if (can_prefill(s, n_tokens)) {
        if (prefill(s, tokens, n_tokens) != 0) return NULL;
    } else {
        for (int i = 0; i < n_tokens; i++) {
            if (bmc_upload(be, s->d_tokens, &tokens[i], sizeof(int)) != 0) return NULL;
            if (run_step(s) != 0) return NULL;
        }
    }
    if (bmc_download(be, s->h_logits, s->logits, (size_t)s->model->arch.vocab_size * sizeof(float)) != 0) return NULL;
    return s->h_logits;
}

void bm_profile_begin(bm_session_t* s) { (void)s; }
void bm_profile_end(bm_session_t* s, double* attention_ms, double* mlp_ms, double* other_ms) {
    (void)s;
    if (attention_ms) *attention_ms = 0.0;
    if (mlp_ms) *mlp_ms = 0.0;
    if (other_ms) *other_ms = 0.0;
}

/* ---- batched greedy generation (include/baremetal_ext.h) ---------------------------------------------------------------- */
/* Feeds prompt[b][0..n_prompt) to every sequence b, then generates n_new tokens greedily. out[b][0..n_new) receives the ids.
 * The loop never returns to the host between tokens: the chosen ids are copied device-to-device into the next step's input. */
int bmx_session_generate_greedy(bm_session_t* s, const int* prompt, int n_prompt, int n_new, int* out) {
    if (!s || !prompt || n_prompt < 1 || n_new < 1 || !out) return -1;
    bmc_ctx_t* be = s->ctx->be;
    const int NB = s->NB;
    if (s->pos + n_prompt + n_new - 1 > s->MS) return -2; /* n_prompt + n_new - 1 steps are taken */
    if (s->gen_cap < n_new) {
        bmc_free(be, s->d_gen);
        s->d_gen = (int*)bmc_alloc(be, (size_t)n_new * NB * sizeof(int));
        if (!s->d_gen) return -3;
        s->gen_cap = n_new;
    }
    for (size_t i = 0; i < (size_t)NB * n_prompt; i++)
        if (prompt[i] < 0 || prompt[i] >= s->model->arch.vocab_size) return -4;
    if (can_prefill(s, n_prompt)) {
        int rc0 = prefill(s, prompt, n_prompt);
        if (rc0) return rc0;
        n_prompt = 0; /* the loop below then starts from the prompt's greedy choice */
    }
    int* col = (int*)malloc(((size_t)NB * n_prompt + 1) * sizeof(int));
    for (int i = 0; i < n_prompt; i++)
        for (int b = 0; b < NB; b++) col[(size_t)i * NB + b] = prompt[(size_t)b * n_prompt + i];
    int* d_prompt = (int*)bmc_alloc(be, ((size_t)NB * n_prompt + 1) * sizeof(int));
    if (!d_prompt) { free(col); return -3; }
    if (n_prompt > 0) bmc_upload(be, d_prompt, col, (size_t)NB * n_prompt * sizeof(int));
    bmc_sync(be);
    free(col);
    int rc = 0;
    for (int i = 0; i < n_prompt && !rc; i++) {
        bmc_copy(be, s->d_tokens, d_prompt + (size_t)i * NB, (size_t)NB * sizeof(int));
        rc = run_step(s);
    }
    for (int i = 0; i < n_new && !rc; i++) {
        bmc_copy(be, s->d_gen + (size_t)i * NB, s->d_next, (size_t)NB * sizeof(int));
        if (i + 1 < n_new) {
            bmc_copy(be, s->d_tokens, s->d_next, (size_t)NB * sizeof(int));
            rc = run_step(s);
        }
    }
    if (!rc) {
        int* h = (int*)malloc((size_t)n_new * NB * sizeof(int));
        rc = bmc_download(be, h, s->d_gen, (size_t)n_new * NB * sizeof(int));
        for (int i = 0; i < n_new; i++)
            for (int b = 0; b < NB; b++) out[(size_t)b * n_new + i] = h[(size_t)i * NB + b];
        free(h);
        if (!rc) rc = bmc_status(be);
    }
    bmc_free(be, d_prompt);
    return rc;
}
/* logits of every sequence after the most recent step (NB x V floats, host pointer valid until the next call) */
const float* bmx_session_logits(bm_session_t* s) {
    if (!s) return NULL;
    if (bmc_download(s->ctx->be, s->h_logits, s->logits, (size_t)s->NB * s->model->arch.vocab_size * sizeof(float)) != 0) return NULL;
    return s->h_logits;
}
int bmx_session_position(bm_session_t* s) { return s ? s->pos : -1; }
/* Bytes of weights one step must read at the least: the matrices in the precision the model asks for (Q8: int8 blocks of 32 with one
 * fp32 scale = 1.125 bytes per weight, Q4: 0.625, as the reference counts them, bench/bench.c:339-348), whatever layout the session
 * streams. */
size_t bmx_session_algorithmic_weight_bytes(bm_session_t* s) {
    if (!s) return 0;
    size_t n = 0;
    for (int l = 0; l < s->model->arch.n_layers; l++) {
        const bm_mat_t* ms[4] = {&s->layers[l].qkv, &s->layers[l].o, &s->layers[l].gu, &s->layers[l].down};
        for (int i = 0; i < 4; i++) {
            const size_t e = (size_t)ms[i]->OC * ms[i]->C;
            n += s->wtype == BMC_W_Q8 ? e + e / 32 * 4 : s->wtype == BMC_W_Q4 ? e / 2 + e / 32 * 4 : s->wtype == BMC_W_BF16 ? e * 2 : e * 4;
        }
    }
    n += (size_t)s->model->arch.vocab_size * s->model->arch.dim * (s->head_type == BMC_W_BF16 ? 2 : 4);
    return n;
}
int bmx_session_kv_bytes_per_element(bm_session_t* s) { return s ? (s->kv_dtype == BMC_BF16 ? 2 : 4) : 0; }
/* Bytes of weights the session actually streams per step (the tensor-core path of >= 8 sequences reads bf16 expansions). */
size_t bmx_session_weight_bytes(bm_session_t* s) {
    if (!s) return 0;
    size_t n = 0;
    for (int l = 0; l < s->model->arch.n_layers; l++) {
        const bm_mat_t* ms[4] = {&s->layers[l].qkv, &s->layers[l].o, &s->layers[l].gu, &s->layers[l].down};
        for (int i = 0; i < 4; i++) {
            const size_t e = (size_t)ms[i]->OC * ms[i]->C;
            n += s->tc ? e * 2 * ms[i]->parts : s->wtype == BMC_W_Q8 ? e + e / 32 * 4 : s->wtype == BMC_W_Q4 ? e / 2 + e / 32 * 4 : s->wtype == BMC_W_BF16 ? e * 2 : e * 4;
        }
    }
    n += (size_t)s->model->arch.vocab_size * s->model->arch.dim * (s->tc ? 2 * s->head_parts : s->head_type == BMC_W_BF16 ? 2 : 4);
    return n;
}
