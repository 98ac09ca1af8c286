/* Weights from a Hugging Face style directory: config.json + model.safetensors (F32 or BF16 tensors, Llama tensor
 * names), into the flat fp32 model buffer. Counterpart of the reference's directory loader
 * (src/baremetal/checkpoint_st.c:430-671, name table src/baremetal/config.c:14-31) for the one model family this build
 * serves. Sharded checkpoints (model.safetensors.index.json) are read shard by shard.
 *
 * safetensors layout: u64 little-endian header length N, N bytes of JSON mapping tensor name ->
 * {"dtype", "shape", "data_offsets": [begin, end]} (offsets relative to the end of the header), then the raw data. */
#include <ctype.h>
#include <math.h>
#include <errno.h>
#include <stdio.h>
#include <sys/stat.h>
#include <stdlib.h>
#include <string.h>

#include "bm_internal.h"

static char* read_file(const char* path, size_t* len_out) {
    FILE* f = fopen(path, "rb");
    if (!f) return NULL;
    fseek(f, 0, SEEK_END);
    const long n = ftell(f);
    fseek(f, 0, SEEK_SET);
    char* buf = (char*)malloc((size_t)n + 1);
    if (!buf || fread(buf, 1, (size_t)n, f) != (size_t)n) {
        free(buf);
        fclose(f);
        return NULL;
    }
    buf[n] = 0;
    fclose(f);
    if (len_out) *len_out = (size_t)n;
    return buf;
}

/* value text following "key": in a flat JSON object (first occurrence); NULL when absent */
/* Value of member `key` of the JSON object that starts at the first '{' of `json`. Only that object's own members are
 * looked at: a key of the same name inside a nested object or array, or text inside a string, never matches. */
static const char* json_value(const char* json, const char* key) {
    const char* p = strchr(json, '{');
    if (!p) return NULL;
    const size_t klen = strlen(key);
    int depth = 0;
    for (; *p; ++p) {
        if (*p == '"') {
            const char* start = p + 1;
            for (++p; *p && *p != '"'; ++p)
                if (*p == '\\' && p[1]) ++p;
            if (!*p) return NULL;
            if (depth == 1 && (size_t)(p - start) == klen && strncmp(start, key, klen) == 0) {
                const char* q = p + 1;
                while (*q && isspace((unsigned char)*q)) ++q;
                if (*q == ':') {   /* a member name, not a string value */
                    ++q;
                    while (*q && isspace((unsigned char)*q)) ++q;
                    return q;
                }
            }
        } else if (*p == '{' || *p == '[') {
            ++depth;
        } else if (*p == '}' || *p == ']') {
            if (--depth <= 0) return NULL;
        }
    }
    return NULL;
}
static int json_int(const char* json, const char* key, int dflt) {
    const char* v = json_value(json, key);
    return (v && (isdigit((unsigned char)*v) || *v == '-')) ? atoi(v) : dflt;
}
static double json_num(const char* json, const char* key, double dflt) {
    const char* v = json_value(json, key);
    return (v && (isdigit((unsigned char)*v) || *v == '-' || *v == '.')) ? atof(v) : dflt;
}
static int json_bool(const char* json, const char* key, int dflt) {
    const char* v = json_value(json, key);
    if (!v) return dflt;
    return strncmp(v, "true", 4) == 0 ? 1 : strncmp(v, "false", 5) == 0 ? 0 : dflt;
}

typedef struct {
    FILE* f;
    char* header;
    size_t data_start;
} st_file_t;

static int st_open(st_file_t* s, const char* path) {
    memset(s, 0, sizeof *s);
    s->f = fopen(path, "rb");
    if (!s->f) return -1;
    uint64_t n = 0;
    if (fread(&n, 8, 1, s->f) != 1 || n == 0 || n > ((uint64_t)1 << 30)) { fclose(s->f); s->f = NULL; return -1; }
    s->header = (char*)malloc((size_t)n + 1);
    if (!s->header || fread(s->header, 1, (size_t)n, s->f) != (size_t)n) { free(s->header); fclose(s->f); s->f = NULL; return -1; }
    s->header[n] = 0;
    s->data_start = 8 + (size_t)n;
    return 0;
}
static void st_close(st_file_t* s) {
    if (s->f) fclose(s->f);
    free(s->header);
    memset(s, 0, sizeof *s);
}
/* 0 = copied, 1 = tensor not in this file, -1 = error */
static int st_read_tensor(st_file_t* s, const char* name, float* dst, size_t n_expected) {
    char pat[256];
    snprintf(pat, sizeof pat, "\"%s\"", name);
    const char* p = strstr(s->header, pat);
    if (!p) return 1;
    const char* end = strchr(p, '}');
    if (!end) return -1;
    const char* dt = strstr(p, "\"dtype\"");
    const char* off = strstr(p, "\"data_offsets\"");
    if (!dt || !off || dt > end || off > end) return -1;
    dt = strchr(dt + 7, ':');
    dt = strchr(dt, '"') + 1;
    const int is_bf16 = strncmp(dt, "BF16", 4) == 0, is_f32 = strncmp(dt, "F32", 3) == 0;
    if (!is_bf16 && !is_f32) {
        BM_LOG_ERROR("safetensors: tensor %s has unsupported dtype (need F32 or BF16)", name);
        return -1;
    }
    off = strchr(off, '[') + 1;
    const unsigned long long b = strtoull(off, (char**)&off, 10);
    off = strchr(off, ',') + 1;
    const unsigned long long e = strtoull(off, NULL, 10);
    const size_t esz = is_bf16 ? 2 : 4;
    if ((e - b) != n_expected * esz) {
        BM_LOG_ERROR("safetensors: tensor %s has %llu bytes, expected %zu", name, e - b, n_expected * esz);
        return -1;
    }
    if (fseek(s->f, (long)(s->data_start + b), SEEK_SET) != 0) return -1;
    if (is_f32) return fread(dst, 4, n_expected, s->f) == n_expected ? 0 : -1;
    uint16_t* tmp = (uint16_t*)malloc(n_expected * 2);
    if (!tmp || fread(tmp, 2, n_expected, s->f) != n_expected) { free(tmp); return -1; }
    bm_bf16_to_f32_array(tmp, dst, n_expected);
    free(tmp);
    return 0;
}

int bm_load_safetensors_dir(bm_model_t* m, const char* dir) {
    char path[4096];
    if (strlen(dir) > 3000) return -1;
    snprintf(path, sizeof path, "%s/config.json", dir);
    char* cfg = read_file(path, NULL);
    if (!cfg) return -1;
    bm_arch_t a;
    memset(&a, 0, sizeof a);
    a.dim = json_int(cfg, "hidden_size", 0);
    a.hidden_dim = json_int(cfg, "intermediate_size", 0);
    a.n_layers = json_int(cfg, "num_hidden_layers", 0);
    a.n_heads = json_int(cfg, "num_attention_heads", 0);
    a.n_kv_heads = json_int(cfg, "num_key_value_heads", a.n_heads);
    a.vocab_size = json_int(cfg, "vocab_size", 0);
    a.padded_vocab_size = a.vocab_size;
    a.max_seq_len = json_int(cfg, "max_position_embeddings", 2048);
    a.head_dim = json_int(cfg, "head_dim", a.n_heads > 0 ? a.dim / a.n_heads : 0);
    a.rope_theta = (float)json_num(cfg, "rope_theta", 10000.0);
    /* "rope_scaling": null, or an object; only the llama3 rule exists in the engine (src/baremetal/config.c:192-211,289-294).
     * Any other rule would train and decode with the wrong frequencies, so it is refused instead of ignored. */
    {
        const char* rs = json_value(cfg, "rope_scaling");
        if (rs && *rs == '{') {
            const char* ty = json_value(rs, "rope_type");
            if (!ty) ty = json_value(rs, "type");
            if (!ty || strncmp(ty, "\"llama3\"", 8) != 0) {
                BM_LOG_ERROR("config.json: rope_scaling type %.16s is not supported (only \"llama3\")", ty ? ty : "(none)");
                free(cfg);
                return -1;
            }
            a.rope_scaling = BM_ROPE_LLAMA3;
            a.rope_factor = (float)json_num(rs, "factor", 1.0);
            a.rope_low_freq_factor = (float)json_num(rs, "low_freq_factor", 1.0);
            a.rope_high_freq_factor = (float)json_num(rs, "high_freq_factor", 4.0);
            a.rope_original_max = (float)json_num(rs, "original_max_position_embeddings", 0.0);
            if (a.rope_factor <= 0.0f) a.rope_factor = 1.0f;
            if (a.rope_low_freq_factor <= 0.0f) a.rope_low_freq_factor = 1.0f;
            if (a.rope_high_freq_factor <= 0.0f) a.rope_high_freq_factor = 4.0f;
            if (a.rope_original_max <= 0.0f) a.rope_original_max = a.max_seq_len > 0 ? (float)a.max_seq_len : 8192.0f;
        }
    }
    a.weight_tie = json_bool(cfg, "tie_word_embeddings", 1);
    a.bias = json_bool(cfg, "attention_bias", 0);
    a.norm = BM_NORM_RMSNORM;
    a.activation = BM_ACT_SWIGLU;
    a.pos_enc = BM_POS_ROPE;
    a.attention = a.n_kv_heads != a.n_heads ? BM_ATTN_GQA : BM_ATTN_MHA;
    a.gated_mlp = 1;
    a.precision = m->precision;
    const double eps = json_num(cfg, "rms_norm_eps", 1e-5);
    if (fabs(eps - 1e-5) > 1e-9)
        fprintf(stderr, "[WARN] config.json rms_norm_eps=%g is ignored: the engine uses 1e-5 (as the reference, src/baremetal/graph.c:283)\n", eps);
    free(cfg);
    if (a.dim <= 0 || a.n_layers <= 0 || a.vocab_size <= 0) return -1;
    const bm_precision_t keep = m->precision;
    bm_model_release(m);
    if (bm_model_alloc(m, &a) != 0) return -1;
    m->precision = keep;

    /* shard list: a single model.safetensors, or every "*.safetensors" named in the index */
    static char shard_names[64][256];
    int n_shards = 0;
    snprintf(path, sizeof path, "%s/model.safetensors.index.json", dir);
    char* idx = read_file(path, NULL);
    if (idx) {
        const char* p = idx;
        while ((p = strstr(p, ".safetensors\"")) != NULL && n_shards < 64) {
            const char* q = p;
            while (q > idx && q[-1] != '"') --q;
            char nm[256];
            const size_t len = (size_t)(p + 12 - q);
            if (len < sizeof nm) {
                memcpy(nm, q, len);
                nm[len] = 0;
                int seen = 0;
                for (int i = 0; i < n_shards; ++i) seen |= strcmp(shard_names[i], nm) == 0;
                if (!seen) strcpy(shard_names[n_shards++], nm);
            }
            p += 12;
        }
        free(idx);
    }
    if (n_shards == 0) strcpy(shard_names[n_shards++], "model.safetensors");

    const size_t D = a.dim, H = a.hidden_dim, V = a.vocab_size, QD = (size_t)a.n_heads * m->head_size, KV = m->kv_dim;
    struct { const char* suffix; float* base; size_t n; } per_layer[9] = {
        {"input_layernorm.weight", m->ln1w, D},          {"self_attn.q_proj.weight", m->qw, QD * D},
        {"self_attn.k_proj.weight", m->kw, KV * D},      {"self_attn.v_proj.weight", m->vw, KV * D},
        {"self_attn.o_proj.weight", m->ow, D * QD},      {"post_attention_layernorm.weight", m->ln2w, D},
        {"mlp.gate_proj.weight", m->gate, H * D},        {"mlp.up_proj.weight", m->up, H * D},
        {"mlp.down_proj.weight", m->down, D * H}};
    const int n_needed = 9 * a.n_layers + 2;
    int n_found = 0;
    for (int s = 0; s < n_shards; ++s) {
        st_file_t st;
        snprintf(path, sizeof path, "%.3000s/%.255s", dir, shard_names[s]);
        if (st_open(&st, path) != 0) {
            BM_LOG_ERROR("cannot read %s", path);
            bm_model_release(m);
            return -1;
        }
        int rc = st_read_tensor(&st, "model.embed_tokens.weight", m->embed, V * D);
        if (rc < 0) goto fail;
        n_found += rc == 0;
        rc = st_read_tensor(&st, "model.norm.weight", m->lnfw, D);
        if (rc < 0) goto fail;
        n_found += rc == 0;
        for (int l = 0; l < a.n_layers; ++l)
            for (int k = 0; k < 9; ++k) {
                char nm[256];
                snprintf(nm, sizeof nm, "model.layers.%d.%s", l, per_layer[k].suffix);
                rc = st_read_tensor(&st, nm, per_layer[k].base + (size_t)l * per_layer[k].n, per_layer[k].n);
                if (rc < 0) goto fail;
                n_found += rc == 0;
            }
        st_close(&st);
        continue;
    fail:
        st_close(&st);
        bm_model_release(m);
        return -1;
    }
    if (n_found != n_needed) {
        BM_LOG_ERROR("safetensors: found %d of %d tensors in %s", n_found, n_needed, dir);
        bm_model_release(m);
        return -1;
    }
    BM_LOG_INFO("Loaded safetensors directory %s (%zu params)", dir, m->n_parameters);
    return 0;
}

/* ---- export -----------------------------------------------------------------------------------------------------------------
 * bm_save_weights (include/baremetal.h; declared but left unimplemented by the reference, src/baremetal/checkpoint.c:84-88).
 * A path ending in ".bin" gets the legacy single-file layout (256 x int32 header, then the flat fp32 payload,
 * src/baremetal/checkpoint.c:19-72); any other path is created as a directory holding config.json and model.safetensors with
 * the Hugging Face Llama tensor names (src/baremetal/config.c:14-31), F32, tied embedding stored once — what
 * bm_load_safetensors_dir above and the reference's loader (src/baremetal/checkpoint_st.c:541-637) read back. */
static int save_bin(const bm_model_t* m, const char* path) {
    const bm_arch_t* a = &m->arch;
    int32_t h[256];
    memset(h, 0, sizeof h);
    h[0] = BM_CHECKPOINT_MAGIC; h[1] = 1; h[2] = (int32_t)a->precision;
    h[3] = a->dim; h[4] = a->hidden_dim; h[5] = a->n_layers; h[6] = a->n_heads; h[7] = a->n_kv_heads; h[8] = a->vocab_size;
    h[9] = a->max_seq_len; h[10] = (int32_t)a->norm; h[11] = (int32_t)a->activation; h[12] = (int32_t)a->pos_enc;
    h[13] = (int32_t)a->attention; h[14] = a->bias; h[15] = a->weight_tie; h[16] = a->has_qk_norm; h[17] = a->has_ffn_post_norm;
    h[18] = a->head_dim; h[19] = a->gated_mlp; h[20] = a->embed_scale; h[21] = a->weight_layout; h[22] = a->gemma_norm;
    h[23] = (int32_t)a->rope_theta;
    FILE* f = fopen(path, "wb");
    if (!f) return -1;
    const int ok = fwrite(h, sizeof(int32_t), 256, f) == 256 && fwrite(m->weight_buffer, sizeof(float), m->n_parameters, f) == m->n_parameters;
    return (fclose(f) == 0 && ok) ? 0 : -1;
}

int bm_save_weights_to(const bm_model_t* m, const char* path) {
    if (!m || !m->weight_buffer || !path) return -1;
    const size_t plen = strlen(path);
    if (plen > 4 && strcmp(path + plen - 4, ".bin") == 0) return save_bin(m, path);
    if (plen > 3000) return -1;
    if (mkdir(path, 0777) != 0 && errno != EEXIST) {
        BM_LOG_ERROR("bm_save_weights: cannot create directory %s", path);
        return -1;
    }
    const bm_arch_t* a = &m->arch;
    char file[4096];
    snprintf(file, sizeof file, "%s/config.json", path);
    FILE* f = fopen(file, "w");
    if (!f) return -1;
    fprintf(f, "{\n  \"architectures\": [\"LlamaForCausalLM\"],\n  \"model_type\": \"llama\",\n  \"hidden_size\": %d,\n"
               "  \"intermediate_size\": %d,\n  \"num_hidden_layers\": %d,\n  \"num_attention_heads\": %d,\n"
               "  \"num_key_value_heads\": %d,\n  \"head_dim\": %d,\n  \"vocab_size\": %d,\n  \"max_position_embeddings\": %d,\n"
               "  \"rms_norm_eps\": 1e-05,\n  \"rope_theta\": %.9g,\n  \"hidden_act\": \"silu\",\n  \"attention_bias\": false,\n"
               "  \"mlp_bias\": false,\n  \"tie_word_embeddings\": true,\n  \"torch_dtype\": \"float32\",\n",
            a->dim, a->hidden_dim, a->n_layers, a->n_heads, a->n_kv_heads, m->head_size, a->vocab_size, a->max_seq_len, (double)a->rope_theta);
    if (a->rope_scaling == BM_ROPE_LLAMA3)
        fprintf(f, "  \"rope_scaling\": {\"rope_type\": \"llama3\", \"factor\": %.9g, \"low_freq_factor\": %.9g, \"high_freq_factor\": %.9g, "
                   "\"original_max_position_embeddings\": %d}\n}\n",
                (double)a->rope_factor, (double)a->rope_low_freq_factor, (double)a->rope_high_freq_factor, (int)a->rope_original_max);
    else
        fprintf(f, "  \"rope_scaling\": null\n}\n");
    if (fclose(f) != 0) return -1;

    /* header: one entry per tensor in file order, offsets relative to the start of the data section */
    const size_t D = a->dim, H = a->hidden_dim, V = a->vocab_size, QD = (size_t)a->n_heads * m->head_size, KV = m->kv_dim;
    struct { const char* suffix; const float* base; size_t rows, cols; } per_layer[9] = {
        {"input_layernorm.weight", m->ln1w, D, 0},          {"self_attn.q_proj.weight", m->qw, QD, D},
        {"self_attn.k_proj.weight", m->kw, KV, D},          {"self_attn.v_proj.weight", m->vw, KV, D},
        {"self_attn.o_proj.weight", m->ow, D, QD},          {"post_attention_layernorm.weight", m->ln2w, D, 0},
        {"mlp.gate_proj.weight", m->gate, H, D},            {"mlp.up_proj.weight", m->up, H, D},
        {"mlp.down_proj.weight", m->down, D, H}};
    const size_t cap = 512 + (size_t)(9 * a->n_layers + 2) * 200;
    char* hdr = (char*)malloc(cap);
    if (!hdr) return -1;
    size_t hl = 0, off = 0;
    hl += (size_t)snprintf(hdr + hl, cap - hl, "{\"__metadata__\":{\"format\":\"pt\"}");
#define ENTRY(name_fmt, name_arg, rows_, cols_) do { \
        const size_t n__ = (cols_) ? (size_t)(rows_) * (cols_) : (size_t)(rows_); \
        hl += (size_t)snprintf(hdr + hl, cap - hl, ",\"" name_fmt "\":{\"dtype\":\"F32\",\"shape\":[", name_arg); \
        if (cols_) hl += (size_t)snprintf(hdr + hl, cap - hl, "%zu,%zu", (size_t)(rows_), (size_t)(cols_)); \
        else hl += (size_t)snprintf(hdr + hl, cap - hl, "%zu", (size_t)(rows_)); \
        hl += (size_t)snprintf(hdr + hl, cap - hl, "],\"data_offsets\":[%zu,%zu]}", off, off + n__ * 4); \
        off += n__ * 4; \
    } while (0)
    ENTRY("%s", "model.embed_tokens.weight", V, D);
    for (int l = 0; l < a->n_layers; ++l)
        for (int k = 0; k < 9; ++k) {
            char nm[128];
            snprintf(nm, sizeof nm, "model.layers.%d.%s", l, per_layer[k].suffix);
            ENTRY("%s", nm, per_layer[k].rows, per_layer[k].cols);
        }
    ENTRY("%s", "model.norm.weight", D, 0);
#undef ENTRY
    hl += (size_t)snprintf(hdr + hl, cap - hl, "}");
    while (hl % 8) hdr[hl++] = ' ';   /* the data section starts 8-byte aligned */
    snprintf(file, sizeof file, "%s/model.safetensors", path);
    f = fopen(file, "wb");
    if (!f) { free(hdr); return -1; }
    const uint64_t hlen = (uint64_t)hl;
    int ok = fwrite(&hlen, 8, 1, f) == 1 && fwrite(hdr, 1, hl, f) == hl;
    free(hdr);
    ok = ok && fwrite(m->embed, 4, V * D, f) == V * D;
    for (int l = 0; l < a->n_layers && ok; ++l)
        for (int k = 0; k < 9 && ok; ++k) {
            const size_t n = per_layer[k].cols ? per_layer[k].rows * per_layer[k].cols : per_layer[k].rows;
            ok = fwrite(per_layer[k].base + (size_t)l * n, 4, n, f) == n;
        }
    ok = ok && fwrite(m->lnfw, 4, D, f) == D;
    if (fclose(f) != 0 || !ok) {
        BM_LOG_ERROR("bm_save_weights: write to %s failed", file);
        return -1;
    }
    BM_LOG_INFO("Saved %zu parameters to %s (config.json + model.safetensors)", m->n_parameters, path);
    return 0;
}
