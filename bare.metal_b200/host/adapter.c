/* Adapter files: low-rank updates merged into the host weights of a model.
 *
 * bm_load_adapter() follows the reference's loader (src/baremetal/adapter.c:151-212): it does not keep the adapter beside the
 * model, it adds scale * B * A to the projection the entry names, in the model's fp32 host buffer. Sessions and trainers created
 * afterwards upload the merged matrices, so nothing on the device knows about adapters.
 *
 * File layout (little endian, src/baremetal/adapter.c:20-40):
 *   header  { u32 magic 0x424D4C52, u32 version 1, i32 dim, layers, n_heads, n_kv_heads, vocab, head_size, rank, f32 alpha,
 *             i32 n_adapters }
 *   entry[] { i32 layer, target, r, c, oc } followed by A[r][c] and B[oc][r] as fp32
 * `target` is one bit of the reference's target set (src/baremetal/lora.h:13-21). The merge of one entry is
 *   W[row][col] += (alpha / rank) * sum_k B[row][k] * A[k][col]        (W is [oc][c], the row-major projection weight)
 * with the sum taken in fp32 in increasing k, as the reference does, so that the merged weights are the same floats.
 *
 * Unlike the reference, an entry whose layer index is outside the model is refused instead of written through. */
#include "bm_internal.h"

#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#define ADAPTER_MAGIC 0x424D4C52u
#define ADAPTER_VERSION 1u

enum { TGT_Q = 1 << 0, TGT_K = 1 << 1, TGT_V = 1 << 2, TGT_O = 1 << 3, TGT_GATE = 1 << 4, TGT_UP = 1 << 5, TGT_DOWN = 1 << 6 };

typedef struct {
    uint32_t magic, version;
    int32_t dim, layers, n_heads, n_kv_heads, vocab, head_size, rank;
    float alpha;
    int32_t n_adapters;
} adapter_header_t;

typedef struct {
    int32_t layer, target, r, c, oc;
} adapter_entry_t;

/* The [oc][c] projection an entry addresses (src/baremetal/adapter.c:42-78). This build's models are gated
 * (bm_arch_supported), so "up" is the third MLP matrix. */
static float* projection_of(bm_model_t* m, int layer, int target, int* c, int* oc) {
    const size_t D = (size_t)m->arch.dim, H = (size_t)m->arch.hidden_dim, Q = (size_t)m->arch.n_heads * (size_t)m->head_size,
                 KV = (size_t)m->kv_dim, l = (size_t)layer;
    switch (target) {
        case TGT_Q: *c = (int)D; *oc = (int)Q; return m->qw + l * Q * D;
        case TGT_K: *c = (int)D; *oc = (int)KV; return m->kw + l * KV * D;
        case TGT_V: *c = (int)D; *oc = (int)KV; return m->vw + l * KV * D;
        case TGT_O: *c = (int)Q; *oc = (int)D; return m->ow + l * D * Q;
        case TGT_GATE: *c = (int)D; *oc = (int)H; return m->gate + l * H * D;
        case TGT_UP: *c = (int)D; *oc = (int)H; return m->up + l * H * D;
        case TGT_DOWN: *c = (int)H; *oc = (int)D; return m->down + l * D * H;
        default: return NULL;
    }
}

static void merge_entry(float* w, const float* a, const float* b, int r, int c, int oc, float scale) {
    for (int row = 0; row < oc; row++) {
        const float* brow = b + (size_t)row * r;
        float* wrow = w + (size_t)row * c;
        for (int col = 0; col < c; col++) {
            float sum = 0.0f;
            for (int k = 0; k < r; k++) sum += brow[k] * a[(size_t)k * c + col];
            wrow[col] += scale * sum;
        }
    }
}

int bm_load_adapter(bm_model_t* model, const char* path) {
    if (!model || !path || !model->weight_buffer) return -1;
    FILE* f = fopen(path, "rb");
    if (!f) {
        BM_LOG_ERROR("bm_load_adapter: cannot open %s", path);
        return -1;
    }
    int rc = -1;
    float *a = NULL, *b = NULL;
    adapter_header_t h;
    if (fread(&h, sizeof h, 1, f) != 1 || h.magic != ADAPTER_MAGIC || h.version != ADAPTER_VERSION) {
        BM_LOG_ERROR("bm_load_adapter: bad header");
        goto done;
    }
    if (h.dim != model->arch.dim || h.layers != model->arch.n_layers || h.n_heads != model->arch.n_heads ||
        h.n_kv_heads != model->arch.n_kv_heads || h.vocab != model->arch.vocab_size || h.head_size != model->head_size ||
        h.rank <= 0 || h.n_adapters <= 0) {
        BM_LOG_ERROR("bm_load_adapter: architecture mismatch");
        goto done;
    }
    const float scale = h.alpha / (float)h.rank;
    for (int i = 0; i < h.n_adapters; i++) {
        adapter_entry_t e;
        if (fread(&e, sizeof e, 1, f) != 1 || e.r != h.rank || e.c <= 0 || e.oc <= 0 || e.layer < 0 ||
            e.layer >= model->arch.n_layers) {
            BM_LOG_ERROR("bm_load_adapter: bad entry");
            goto done;
        }
        int c = 0, oc = 0;
        float* w = projection_of(model, e.layer, e.target, &c, &oc);
        if (!w || c != e.c || oc != e.oc) {
            BM_LOG_ERROR("bm_load_adapter: target mismatch");
            goto done;
        }
        const size_t an = (size_t)e.r * (size_t)e.c, bn = (size_t)e.oc * (size_t)e.r;
        a = (float*)malloc(an * sizeof(float));
        b = (float*)malloc(bn * sizeof(float));
        if (!a || !b || fread(a, sizeof(float), an, f) != an || fread(b, sizeof(float), bn, f) != bn) {
            BM_LOG_ERROR("bm_load_adapter: short read");
            goto done;
        }
        merge_entry(w, a, b, e.r, e.c, e.oc, scale);
        free(a);
        free(b);
        a = b = NULL;
    }
    rc = 0;
done:
    free(a);
    free(b);
    fclose(f);
    return rc;
}
