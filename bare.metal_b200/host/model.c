/* Host-side model storage and weight loading.
 * Layout and file formats follow the reference: flat fp32 buffer in a fixed tensor order
 * (src/baremetal/model.c:41-178), legacy .bin checkpoint = 256 x int32 header + that buffer
 * (src/baremetal/checkpoint.c:12-88). */
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "bm_internal.h"


int bm_log_verbose(void) {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("BM_LOG");
        v = (e && e[0] && e[0] != '0') ? 1 : 0;
    }
    return v;
}

/* The training path serves the Llama family the reference supports (src/baremetal/config.c:33-76):
 * RMSNorm, SwiGLU gated MLP, RoPE, tied embeddings, no biases / qk-norm / post-norms
 * (bmt_arch_validate, src/baremetal/model.c:14-40). */
int bm_arch_supported(const bm_arch_t* a) {
    if (a->bias || a->has_qk_norm || a->has_ffn_post_norm || a->gemma_norm || a->embed_scale) {
        BM_LOG_ERROR("Unsupported architecture feature (bias/qk_norm/post_ffn_norm/gemma_norm/embed_scale)");
        return 0;
    }
    if (a->norm != BM_NORM_RMSNORM || a->activation != BM_ACT_SWIGLU || a->pos_enc != BM_POS_ROPE || !a->gated_mlp) {
        BM_LOG_ERROR("Unsupported architecture: this build serves RMSNorm + SwiGLU + RoPE decoders");
        return 0;
    }
    if (!a->weight_tie) {
        BM_LOG_ERROR("Unsupported architecture: untied LM head");
        return 0;
    }
    if (a->dim <= 0 || a->n_layers <= 0 || a->n_heads <= 0 || a->n_kv_heads <= 0 || a->n_heads % a->n_kv_heads ||
        a->vocab_size <= 0 || a->hidden_dim <= 0)
        return 0;
    return 1;
}

int bm_model_alloc(bm_model_t* m, const bm_arch_t* arch) {
    memset(m, 0, sizeof(*m));
    if (!bm_arch_supported(arch)) return -1;
    m->arch = *arch;
    m->precision = arch->precision;
    m->head_size = arch->head_dim > 0 ? arch->head_dim : arch->dim / arch->n_heads;
    m->kv_dim = m->head_size * arch->n_kv_heads;
    m->kv_mul = arch->n_heads / arch->n_kv_heads;
    const size_t V = (size_t)(arch->padded_vocab_size > 0 ? arch->padded_vocab_size : arch->vocab_size);
    const size_t L = (size_t)arch->n_layers, D = (size_t)arch->dim, H = (size_t)arch->hidden_dim;
    const size_t QD = (size_t)arch->n_heads * m->head_size, KV = (size_t)m->kv_dim;
    const size_t total = V * D + L * D + L * QD * D + 2 * L * KV * D + L * D * QD + L * D + 2 * L * H * D + L * D * H + D;
    m->n_parameters = total;
    m->weight_buffer = (float*)calloc(total, sizeof(float));
    if (!m->weight_buffer) {
        BM_LOG_ERROR("Failed to allocate weight buffer (%zu bytes)", total * sizeof(float));
        return -1;
    }
    float* w = m->weight_buffer;
    m->embed = w; w += V * D;
    m->ln1w = w;  w += L * D;
    m->qw = w;    w += L * QD * D;
    m->kw = w;    w += L * KV * D;
    m->vw = w;    w += L * KV * D;
    m->ow = w;    w += L * D * QD;
    m->ln2w = w;  w += L * D;
    m->gate = w;  w += L * H * D;
    m->up = w;    w += L * H * D;
    m->down = w;  w += L * D * H;
    m->lnfw = w;
    return 0;
}

void bm_model_release(bm_model_t* m) {
    if (!m) return;
    free(m->weight_buffer);
    m->weight_buffer = NULL;
}

int bm_load_bin(bm_model_t* m, const char* path) {
    FILE* f = fopen(path, "rb");
    if (!f) return -1;
    int32_t h[256];
    if (fread(h, sizeof(int32_t), 256, f) != 256 || h[0] != BM_CHECKPOINT_MAGIC) {
        fclose(f);
        return -1;
    }
    bm_arch_t a;
    memset(&a, 0, sizeof a);
    a.precision = (bm_precision_t)h[2];
    a.dim = h[3]; a.hidden_dim = h[4]; a.n_layers = h[5]; a.n_heads = h[6]; a.n_kv_heads = h[7];
    a.vocab_size = h[8]; a.max_seq_len = h[9];
    a.norm = (bm_norm_t)h[10]; a.activation = (bm_act_t)h[11]; a.pos_enc = (bm_pos_t)h[12]; a.attention = (bm_attn_t)h[13];
    a.bias = h[14]; a.weight_tie = h[15]; a.has_qk_norm = h[16]; a.has_ffn_post_norm = h[17]; a.head_dim = h[18];
    a.gated_mlp = h[19]; a.embed_scale = h[20]; a.weight_layout = h[21]; a.gemma_norm = h[22];
    a.rope_theta = (float)h[23];
    if (a.rope_theta <= 0.0f) a.rope_theta = 10000.0f;
    a.padded_vocab_size = a.vocab_size;
    const bm_precision_t keep = m->precision;
    bm_model_release(m);
    if (bm_model_alloc(m, &a) != 0) {
        fclose(f);
        return -1;
    }
    (void)keep;
    const size_t got = fread(m->weight_buffer, sizeof(float), m->n_parameters, f);
    fclose(f);
    if (got != m->n_parameters) {
        BM_LOG_ERROR("Read %zu floats, expected %zu", got, m->n_parameters);
        bm_model_release(m);
        return -1;
    }
    BM_LOG_INFO("Loaded checkpoint: %s (%zu params)", path, m->n_parameters);
    return 0;
}

/* cos/sin table [S][HD/2][cos, sin] with the reference's fp32 arithmetic (rope_inv_freq incl. the llama3 frequency rule,
 * src/kernels/forward.metal:1260-1279; angle = float(pos) * inv_freq, rope_forward_seq forward.metal:2241-2243), evaluated with
 * the host libm. One builder for the trainer, the inference session and the kernel-name backend, so that all three rotate by
 * bit-identical angles. Caller frees. */
float* bm_build_rope_table(float theta, int scaling, float factor, float low, float high, float orig, int S, int HD) {
    const int hd2 = HD / 2;
    float* cs = (float*)malloc((size_t)S * hd2 * 2 * sizeof(float));
    if (!cs) return NULL;
    for (int i = 0; i < hd2; ++i) {
        float inv = 1.0f / powf(theta, (float)(2 * i) / (float)HD);
        if (scaling == BM_ROPE_LLAMA3) {
            const float pi = 3.14159265358979323846f;
            const float wavelen = 2.0f * pi / inv;
            const float low_w = orig / low, high_w = orig / high;
            if (wavelen > low_w) inv /= factor;
            if (wavelen >= high_w && wavelen <= low_w) {
                const float smooth = (orig / wavelen - low) / (high - low);
                inv = (1.0f - smooth) * inv / factor + smooth * inv;
            }
        }
        for (int s = 0; s < S; ++s) {
            const float ang = (float)s * inv;
            cs[((size_t)s * hd2 + i) * 2] = cosf(ang);
            cs[((size_t)s * hd2 + i) * 2 + 1] = sinf(ang);
        }
    }
    return cs;
}
float* bm_build_rope_table_arch(const bm_arch_t* a, int S, int HD) {
    return bm_build_rope_table(a->rope_theta, a->rope_scaling, a->rope_factor, a->rope_low_freq_factor, a->rope_high_freq_factor,
                               a->rope_original_max, S, HD);
}
