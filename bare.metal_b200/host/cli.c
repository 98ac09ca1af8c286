/* baremetal-train: the `train` sub-command of the reference CLI (tools/cli.c:634-805) on the CUDA backend.
 * Same positional arguments, flags, per-step line and final average line.
 *
 * The tokenizer lies outside this build, so <data_file> is one of
 *   - a file of raw little-endian int32 token ids (any name ending in .bin, .tok or .tokens), or
 *   - the literal lcg:<seed> for the reference's synthetic token stream (bench/train_bench.c:286-290),
 * instead of a text file. Windows are contiguous: sequence b of step k continues where the previous one ended and the
 * target of a position is the next token of the stream (tools/cli.c:762-768).
 *
 * Data parallel: started once per GPU with RANK / WORLD_SIZE / LOCAL_RANK in the environment (as torchrun exports them), every
 * process trains a replica on its own sequences of the global batch — rank r takes sequences r*B .. r*B+B-1 of the world*B
 * sequences of a step — and gradients are all-reduced over NCCL. The 128-byte NCCL id travels through a file in <output_dir>;
 * rank 0 prints the step lines (the loss is the mean over all ranks) and writes the checkpoints. */
#ifndef BAREMETAL_TRAIN
#define BAREMETAL_TRAIN
#endif
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/stat.h>
#include <time.h>
#include <unistd.h>

#include "../../include/baremetal.h"
#include "../../include/baremetal_ext.h"

static double now_ms(void) {
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return ts.tv_sec * 1e3 + ts.tv_nsec / 1e6;
}
static size_t rss_mb(void) { /* tools/cli.c:47-54 uses Mach task_info; Linux: resident pages from /proc/self/statm */
    FILE* f = fopen("/proc/self/statm", "r");
    if (!f) return 0;
    long total = 0, res = 0;
    if (fscanf(f, "%ld %ld", &total, &res) != 2) res = 0;
    fclose(f);
    return (size_t)res * 4096 / (1024 * 1024);
}
static int ends_with(const char* s, const char* suf) {
    const size_t a = strlen(s), b = strlen(suf);
    return a >= b && strcmp(s + a - b, suf) == 0;
}

static int env_int(const char* name, int dflt) {
    const char* v = getenv(name);
    return (v && v[0]) ? atoi(v) : dflt;
}
/* Rank 0 creates the NCCL id and leaves it in <dir>/.bm_nccl_id.<port>; the other ranks wait for a file that is not older than
 * this process (a file left behind by an earlier run on the same port is ignored). Returns 0 on success. */
static int exchange_nccl_id(const char* dir, int rank, unsigned char id[128], char* path, size_t path_len) {
    const char* port = getenv("MASTER_PORT");
    snprintf(path, path_len, "%s/.bm_nccl_id.%s", dir, (port && port[0]) ? port : "0");
    if (rank == 0) {
        char tmp[600];
        snprintf(tmp, sizeof tmp, "%s.tmp", path);
        if (bmx_dp_unique_id(id) != 0) return -1;
        FILE* f = fopen(tmp, "wb");
        if (!f) return -1;
        const int ok = fwrite(id, 1, 128, f) == 128;
        fclose(f);
        return (ok && rename(tmp, path) == 0) ? 0 : -1;
    }
    const time_t started = time(NULL);
    for (int tries = 0; tries < 6000; ++tries) {   /* up to ten minutes: rank 0 may still be loading the model */
        struct stat st;
        if (stat(path, &st) == 0 && st.st_size == 128 && st.st_mtime >= started - 30) {
            FILE* f = fopen(path, "rb");
            if (f) {
                const int ok = fread(id, 1, 128, f) == 128;
                fclose(f);
                if (ok) return 0;
            }
        }
        usleep(100000);
    }
    return -1;
}

/* ---- `parity`: the reference's architecture parity harness (test/parity/parity.c), fixture format "baremetal.parity/v1" ----
 * A fixture is a JSON object {format, model, precision, prompt_token_ids[], generated_token_ids[], vocab_size, logits_file}
 * next to a raw little-endian float32 file with the full-vocabulary logits after the prompt (test/parity/make_fixture.py).
 * Checks, thresholds and output lines are the reference's: cosine of the prefill logits (0.9999 fp32, 0.999 otherwise), their
 * argmax, and the greedy continuation token by token. */
static char* read_text_file(const char* path) {
    FILE* f = fopen(path, "rb");
    if (!f) return NULL;
    fseek(f, 0, SEEK_END);
    const long n = ftell(f);
    fseek(f, 0, SEEK_SET);
    char* buf = (char*)malloc((size_t)n + 1);
    if (!buf || fread(buf, 1, (size_t)n, f) != (size_t)n) { free(buf); fclose(f); return NULL; }
    buf[n] = 0;
    fclose(f);
    return buf;
}
/* value text of member `key` of the top-level object (keys inside nested values or strings never match) */
static const char* fx_value(const char* json, const char* key) {
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
                while (*q == ' ' || *q == '\t' || *q == '\n' || *q == '\r') ++q;
                if (*q == ':') {
                    ++q;
                    while (*q == ' ' || *q == '\t' || *q == '\n' || *q == '\r') ++q;
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
static int* fx_int_array(const char* json, const char* key, int* n_out) {
    const char* v = fx_value(json, key);
    *n_out = 0;
    if (!v || *v != '[') return NULL;
    int cap = 64, n = 0;
    int* out = (int*)malloc((size_t)cap * sizeof(int));
    for (const char* p = v + 1; out && *p && *p != ']';) {
        if (*p == '-' || (*p >= '0' && *p <= '9')) {
            char* end = NULL;
            const long x = strtol(p, &end, 10);
            if (n == cap) { cap *= 2; out = (int*)realloc(out, (size_t)cap * sizeof(int)); if (!out) break; }
            out[n++] = (int)x;
            p = end;
        } else {
            ++p;
        }
    }
    *n_out = n;
    return out;
}
static int fx_string(const char* json, const char* key, char* out, size_t cap) {
    const char* v = fx_value(json, key);
    if (!v || *v != '"') return -1;
    size_t n = 0;
    for (++v; *v && *v != '"' && n + 1 < cap; ++v) out[n++] = *v;
    out[n] = 0;
    return 0;
}
static int argmax_first(const float* x, int n) {   /* first index of the maximum (strict >), as the reference's sampler */
    int b = 0;
    for (int i = 1; i < n; i++)
        if (x[i] > x[b]) b = i;
    return b;
}
static int parity_main(int argc, char** argv) {
    const char *model_dir = NULL, *fixture_path = NULL, *prec_arg = NULL;
    int max_gen = 0, max_seq = 0;
    for (int i = 2; i < argc; i++) {
        if (strcmp(argv[i], "--model") == 0 && i + 1 < argc) model_dir = argv[++i];
        else if (strcmp(argv[i], "--fixture") == 0 && i + 1 < argc) fixture_path = argv[++i];
        else if (strcmp(argv[i], "--precision") == 0 && i + 1 < argc) prec_arg = argv[++i];
        else if (strcmp(argv[i], "--gen") == 0 && i + 1 < argc) max_gen = atoi(argv[++i]);
        else if (strcmp(argv[i], "--max-seq") == 0 && i + 1 < argc) max_seq = atoi(argv[++i]);
        else model_dir = fixture_path = NULL;
    }
    if (!model_dir || !fixture_path) {
        fprintf(stderr, "usage: %s parity --model DIR --fixture FILE [--precision fp32|bf16] [--gen N] [--max-seq N]\n", argv[0]);
        return 2;
    }
    char* fx = read_text_file(fixture_path);
    if (!fx) { fprintf(stderr, "cannot read fixture: %s\n", fixture_path); return 1; }
    char prec_name[32] = "fp32", model_name[128] = "", logits_file[512] = "";
    fx_string(fx, "precision", prec_name, sizeof prec_name);
    if (prec_arg) snprintf(prec_name, sizeof prec_name, "%s", prec_arg);
    fx_string(fx, "model", model_name, sizeof model_name);
    int np = 0, ng = 0;
    int* prompt = fx_int_array(fx, "prompt_token_ids", &np);
    int* golden_gen = fx_int_array(fx, "generated_token_ids", &ng);
    if (!prompt || !golden_gen || np < 1 || ng < 1) { fprintf(stderr, "fixture missing prompt_token_ids or generated_token_ids\n"); return 1; }
    if (max_gen > 0 && max_gen < ng) ng = max_gen;
    const char* vv = fx_value(fx, "vocab_size");
    const int vocab = vv ? atoi(vv) : 0;
    if (vocab <= 0 || fx_string(fx, "logits_file", logits_file, sizeof logits_file)) { fprintf(stderr, "fixture missing vocab_size or logits_file\n"); return 1; }
    char logits_path[2048];
    const char* slash = strrchr(fixture_path, '/');
    if (slash) snprintf(logits_path, sizeof logits_path, "%.*s/%s", (int)(slash - fixture_path), fixture_path, logits_file);
    else snprintf(logits_path, sizeof logits_path, "%s", logits_file);
    float* golden_logits = (float*)malloc((size_t)vocab * sizeof(float));
    FILE* lf = fopen(logits_path, "rb");
    if (!lf || !golden_logits || fread(golden_logits, sizeof(float), (size_t)vocab, lf) != (size_t)vocab) {
        fprintf(stderr, "cannot read %d logits from %s\n", vocab, logits_path);
        return 1;
    }
    fclose(lf);
    if (strcmp(prec_name, "fp16") == 0) { fprintf(stderr, "fp16 weights are not supported by this backend (use bf16 or fp32)\n"); return 1; }
    const int is_fp32 = strcmp(prec_name, "bf16") != 0;
    printf("parity: %s (%s)\n", model_name[0] ? model_name : model_dir, prec_name);
    printf("  prompt: %d tokens, gen: %d\n", np, ng);

    bm_context_t* ctx = bm_create(BM_DEVICE_CUDA);
    if (!ctx) { fprintf(stderr, "bm_create failed\n"); return 1; }
    bm_arch_t a;
    memset(&a, 0, sizeof a);   /* placeholder: bm_load_weights takes the architecture from the checkpoint */
    a.dim = 64; a.hidden_dim = 64; a.n_layers = 1; a.n_heads = 1; a.n_kv_heads = 1; a.vocab_size = 8; a.padded_vocab_size = 8;
    a.max_seq_len = 64; a.head_dim = 64; a.norm = BM_NORM_RMSNORM; a.activation = BM_ACT_SWIGLU; a.pos_enc = BM_POS_ROPE;
    a.attention = BM_ATTN_GQA; a.weight_tie = 1; a.gated_mlp = 1; a.rope_theta = 10000.0f;
    a.precision = is_fp32 ? BM_PRECISION_FP32 : BM_PRECISION_BF16;
    bm_model_t* m = bm_create_model(ctx, &a);
    if (!m) return 1;
    bm_load_weights(m, model_dir);
    if (bm_get_num_parameters(m) <= 64 * 64 * 8) { fprintf(stderr, "failed to load weights from %s\n", model_dir); return 1; }
    if (vocab != bmx_model_vocab_size(m)) { fprintf(stderr, "vocab mismatch: fixture %d, model %d\n", vocab, bmx_model_vocab_size(m)); return 1; }
    bm_compile(m);
    const int need = np + ng + 1;
    bm_session_t* sess = bmx_create_session_batched(ctx, m, 1, max_seq > need ? max_seq : need);
    if (!sess) { fprintf(stderr, "session creation failed\n"); return 1; }
    bm_reset_session(sess);
    float* logits = bm_forward(sess, prompt, np);
    if (!logits) { fprintf(stderr, "forward failed\n"); return 1; }
    double dot = 0.0, na = 0.0, nb = 0.0, max_diff = 0.0;
    for (int i = 0; i < vocab; i++) {
        dot += (double)logits[i] * golden_logits[i];
        na += (double)logits[i] * logits[i];
        nb += (double)golden_logits[i] * golden_logits[i];
        const double d = fabs((double)logits[i] - (double)golden_logits[i]);
        if (d > max_diff) max_diff = d;
    }
    const double cosv = (na > 0 && nb > 0) ? dot / (sqrt(na) * sqrt(nb)) : 0.0;
    const double threshold = is_fp32 ? 0.9999 : 0.999;
    int failures = 0;
    printf("  logits cos: %.7f (min %.4f)  max|diff|: %.3e\n", cosv, threshold, max_diff);
    if (cosv < threshold) { printf("FAIL: logits cosine below threshold\n"); failures++; }
    const int got_argmax = argmax_first(logits, vocab), want_argmax = argmax_first(golden_logits, vocab);
    printf("  argmax: got %d, want %d\n", got_argmax, want_argmax);
    if (got_argmax != want_argmax) { printf("FAIL: argmax mismatch\n"); failures++; }
    int* gen = (int*)malloc((size_t)ng * sizeof(int));
    if (!gen) return 1;
    gen[0] = got_argmax;
    int n_done = 1;
    for (int i = 1; i < ng; i++, n_done++) {
        logits = bm_step(sess, gen[i - 1]);
        if (!logits) { printf("FAIL: step %d returned NULL\n", i); failures++; break; }
        gen[i] = argmax_first(logits, vocab);
    }
    int first_bad = -1;
    for (int i = 0; i < n_done; i++)
        if (gen[i] != golden_gen[i]) { first_bad = i; break; }
    if (first_bad < 0 && n_done == ng) printf("  tokens: match (%d/%d)\n", ng, ng);
    else if (first_bad >= 0) { printf("FAIL: token mismatch at %d: got %d, want %d\n", first_bad, gen[first_bad], golden_gen[first_bad]); failures++; }
    free(gen); free(golden_logits); free(golden_gen); free(prompt); free(fx);
    bm_destroy_session(sess);
    bm_destroy_model(m);
    bm_destroy(ctx);
    if (failures) { printf("PARITY FAIL\n"); return 1; }
    printf("PARITY PASS\n");
    return 0;
}

static int usage(const char* argv0) {
    fprintf(stderr, "Usage: %s train <model_dir|model.bin> <data_file> <output_dir> [options]\n", argv0);
    fprintf(stderr, "       %s parity --model DIR --fixture FILE [--precision fp32|bf16] [--gen N] [--max-seq N]\n", argv0);
    fprintf(stderr, "  <data_file>         int32 token ids (*.bin, *.tok, *.tokens) or lcg:<seed> for the synthetic stream\n");
    fprintf(stderr, "  --steps <int>       Max training steps (default: 100)\n");
    fprintf(stderr, "  --seq-len <int>     Sequence length S (default: 64)\n");
    fprintf(stderr, "  --batch-size <int>  Batch size B (default: 1)\n");
    fprintf(stderr, "  --grad-accum <int>  Micro-steps per optimizer step (default: 1)\n");
    fprintf(stderr, "  --lr <float>        Learning rate (default: 3e-4)\n");
    fprintf(stderr, "  --weight-decay <f>  AdamW weight decay (default: 0)\n");
    fprintf(stderr, "  --save-every <int>  Save checkpoint every N steps (default: 0 = no save)\n");
    fprintf(stderr, "  --resume <path>     Resume from checkpoint\n");
    fprintf(stderr, "  --precision <bf16|fp32>  Weight precision (default: bf16)\n");
    fprintf(stderr, "  --save-weights <p>  After training, export the weights: a safetensors directory, or a legacy file if <p> ends in .bin\n");
    fprintf(stderr, "  --lora-rank <int>   must be 0: adapters are outside this build\n");
    return 1;
}

int main(int argc, char** argv) {
    if (argc >= 2 && strcmp(argv[1], "parity") == 0) return parity_main(argc, argv);
    if (argc < 2 || strcmp(argv[1], "train") != 0 || argc < 5) return usage(argv[0]);
    const char *model_path = argv[2], *data_file = argv[3], *output_dir = argv[4];
    int max_steps = 100, seq_len = 64, batch_size = 1, grad_accum = 1, save_every = 0, lora_rank = 0;
    float lr = 3e-4f, wd = 0.0f;
    const char *resume_path = NULL, *prec_str = NULL, *save_weights = NULL;
    for (int i = 5; i < argc; i++) {
        if (strcmp(argv[i], "--steps") == 0 && i + 1 < argc) max_steps = atoi(argv[++i]);
        else if (strcmp(argv[i], "--seq-len") == 0 && i + 1 < argc) seq_len = atoi(argv[++i]);
        else if (strcmp(argv[i], "--batch-size") == 0 && i + 1 < argc) batch_size = atoi(argv[++i]);
        else if (strcmp(argv[i], "--grad-accum") == 0 && i + 1 < argc) grad_accum = atoi(argv[++i]);
        else if (strcmp(argv[i], "--lr") == 0 && i + 1 < argc) lr = (float)atof(argv[++i]);
        else if (strcmp(argv[i], "--weight-decay") == 0 && i + 1 < argc) wd = (float)atof(argv[++i]);
        else if (strcmp(argv[i], "--save-every") == 0 && i + 1 < argc) save_every = atoi(argv[++i]);
        else if (strcmp(argv[i], "--resume") == 0 && i + 1 < argc) resume_path = argv[++i];
        else if (strcmp(argv[i], "--precision") == 0 && i + 1 < argc) prec_str = argv[++i];
        else if (strcmp(argv[i], "--save-weights") == 0 && i + 1 < argc) save_weights = argv[++i];
        else if (strcmp(argv[i], "--lora-rank") == 0 && i + 1 < argc) lora_rank = atoi(argv[++i]);
    }
    if (batch_size < 1) {
        fprintf(stderr, "Error: batch-size must be >= 1\n");
        return 1;
    }
    if (lora_rank != 0) {
        fprintf(stderr, "Error: LoRA adapters are outside this build (--lora-rank must be 0)\n");
        return 1;
    }
    const int rank = env_int("RANK", 0), world = env_int("WORLD_SIZE", 1);
    if (world < 1 || rank < 0 || rank >= world) {
        fprintf(stderr, "Error: RANK=%d is outside WORLD_SIZE=%d\n", rank, world);
        return 1;
    }
    bm_context_t* ctx = bm_create(BM_DEVICE_CUDA);   /* device: BM_CUDA_DEVICE, else LOCAL_RANK, else 0 */
    if (!ctx) {
        fprintf(stderr, "No CUDA (sm_100) device available; this engine has no CPU fallback\n");
        return 1;
    }
    bm_arch_t seed_arch;
    memset(&seed_arch, 0, sizeof seed_arch);
    /* a placeholder architecture: bm_load_weights re-creates the buffers from the checkpoint's own description */
    seed_arch.dim = 64; seed_arch.hidden_dim = 64; seed_arch.n_layers = 1; seed_arch.n_heads = 1; seed_arch.n_kv_heads = 1;
    seed_arch.vocab_size = 8; seed_arch.padded_vocab_size = 8; seed_arch.max_seq_len = 64; seed_arch.head_dim = 64;
    seed_arch.norm = BM_NORM_RMSNORM; seed_arch.activation = BM_ACT_SWIGLU; seed_arch.pos_enc = BM_POS_ROPE;
    seed_arch.attention = BM_ATTN_GQA; seed_arch.weight_tie = 1; seed_arch.gated_mlp = 1; seed_arch.rope_theta = 10000.0f;
    seed_arch.precision = (prec_str && strcmp(prec_str, "fp32") == 0) ? BM_PRECISION_FP32 : BM_PRECISION_BF16;
    if (prec_str && strcmp(prec_str, "fp16") == 0) {
        fprintf(stderr, "Error: fp16 weights are not supported by this backend (use bf16 or fp32)\n");
        return 1;
    }
    bm_model_t* model = bm_create_model(ctx, &seed_arch);
    if (!model) return 1;
    bm_load_weights(model, model_path);
    if (bm_get_num_parameters(model) <= 64 * 64 * 8) {
        fprintf(stderr, "Failed to load model from %s\n", model_path);
        return 1;
    }
    bm_print_model_info(model);

    /* token stream */
    int* tokens = NULL;
    long n_tokens = 0;
    if (strncmp(data_file, "lcg:", 4) == 0) {
        size_t np = 0;
        (void)bmx_model_weight_buffer(model, &np);
        n_tokens = (long)max_steps * world * batch_size * seq_len + 1;
        tokens = (int*)malloc((size_t)n_tokens * sizeof(int));
        /* vocabulary size: the embedding is the first tensor of the buffer; ask the model info instead of guessing */
        unsigned s = (unsigned)atoi(data_file + 4);
        const int V = bmx_model_vocab_size(model);
        for (long i = 0; i < n_tokens; i++) {
            s = s * 1664525u + 1013904223u;
            tokens[i] = (int)(s % (unsigned)V);
        }
    } else if (ends_with(data_file, ".bin") || ends_with(data_file, ".tok") || ends_with(data_file, ".tokens")) {
        FILE* f = fopen(data_file, "rb");
        if (!f) {
            fprintf(stderr, "Cannot open data file: %s\n", data_file);
            return 1;
        }
        fseek(f, 0, SEEK_END);
        n_tokens = ftell(f) / (long)sizeof(int);
        fseek(f, 0, SEEK_SET);
        tokens = (int*)malloc((size_t)n_tokens * sizeof(int));
        if (fread(tokens, sizeof(int), (size_t)n_tokens, f) != (size_t)n_tokens) n_tokens = 0;
        fclose(f);
    } else {
        fprintf(stderr, "Text data needs the tokenizer, which is outside this build: pass int32 token ids (*.bin) or lcg:<seed>\n");
        return 1;
    }
    if (n_tokens < 2) {
        fprintf(stderr, "No tokens in %s\n", data_file);
        return 1;
    }
    fprintf(stderr, "[train] loaded %ld tokens from %s\n", n_tokens, data_file);

    bm_train_config_t cfg;
    memset(&cfg, 0, sizeof cfg);
    cfg.learning_rate = lr; cfg.beta1 = 0.9f; cfg.beta2 = 0.95f; cfg.epsilon = 1e-8f; cfg.weight_decay = wd;
    cfg.grad_clip = 1.0f; cfg.grad_accum_steps = grad_accum > 0 ? grad_accum : 1; cfg.warmup_steps = 10;
    cfg.max_steps = max_steps; cfg.seq_len = seq_len;
    bm_trainer_t* trainer = bm_create_trainer(ctx, model, &cfg);
    if (!trainer) {
        fprintf(stderr, "Failed to create trainer\n");
        return 1;
    }
    if (resume_path) {
        bm_load_state(trainer, resume_path);
        fprintf(stderr, "[train] resumed from %s\n", resume_path);
    }
    char id_path[512] = "";
    if (world > 1) {
        unsigned char id[128];
        if (exchange_nccl_id(output_dir, rank, id, id_path, sizeof id_path) != 0 || bmx_trainer_dp_init(trainer, rank, world, id) != 0) {
            fprintf(stderr, "[train] rank %d: data-parallel set-up failed (NCCL id file %s)\n", rank, id_path);
            return 1;
        }
        fprintf(stderr, "[train] rank %d of %d: data parallel, %d sequences per rank per step\n", rank, world, batch_size);
    }
    const int batch_tokens = batch_size * seq_len;
    int* inputs = (int*)malloc((size_t)batch_tokens * sizeof(int));
    int* targets = (int*)malloc((size_t)batch_tokens * sizeof(int));
    long pos = 0;
    double total_step_time = 0.0;
    for (int step = 0; step < max_steps; step++) {
        /* this rank's sequences of the step's global batch: r*B .. r*B+B-1 of world*B contiguous windows */
        pos = ((long)step * world + rank) * batch_tokens;
        for (int b = 0; b < batch_size; b++)
            for (int i = 0; i < seq_len; i++) {
                inputs[b * seq_len + i] = tokens[pos % n_tokens];
                targets[b * seq_len + i] = tokens[(pos + 1) % n_tokens];
                pos++;
            }
        const double t0 = now_ms();
        const float loss = bm_train_step(trainer, inputs, targets, batch_size, seq_len);
        const double step_ms = now_ms() - t0;
        total_step_time += step_ms;
        if (loss < 0.0f) {
            fprintf(stderr, "[train] rank %d: step %d failed\n", rank, step + 1);
            return 1;
        }
        if (rank != 0) continue;   /* replicas are identical: one rank reports and saves (tools/cli.c:777-786) */
        printf("step %d/%d: loss=%.4f  step_ms=%.0f  gpu_mem=%.1fMB  rss=%zuMB\n", step + 1, max_steps, loss, step_ms,
               (double)(bmx_trainer_device_bytes(trainer) / (1024 * 1024)), rss_mb());
        if (save_every > 0 && (step + 1) % save_every == 0) {
            char path[512];
            snprintf(path, sizeof path, "%s/checkpoint_%d.bin", output_dir, step + 1);
            bm_save_state(trainer, path);
            fprintf(stderr, "[train] saved checkpoint to %s\n", path);
        }
    }
    bm_train_flush(trainer);   /* collective under data parallel: every rank reaches it after the same number of steps */
    if (rank == 0) {
        if (save_weights && bmx_trainer_sync_model(trainer) == 0) {
            bm_save_weights(model, save_weights);
            fprintf(stderr, "[train] exported weights to %s\n", save_weights);
        }
        printf("Avg step time: %.1fms\n", total_step_time / max_steps);
        if (id_path[0]) unlink(id_path);
    }
    free(inputs); free(targets); free(tokens);
    bm_destroy_trainer(trainer);
    bm_destroy_model(model);
    bm_destroy(ctx);
    return 0;
}
