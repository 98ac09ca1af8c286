/* TEST INFRASTRUCTURE — a CPU restatement of the reference's training step, used only as a checker
 * (tests/, smoke(), the cpu_baseline leg of bench.py). It is never linked into or called by the product.
 *
 * Plain C, fp32 arithmetic, one function per reference kernel, each citing the reference lines it restates.
 * Parity pin: tests/test_oracle_pins.py checks this file against (a) the committed golden vectors under
 * tests/golden/ that were produced by the reference's own PyTorch golden generators (test/grad/gen_*.py) and by the
 * reference's C11 host code + Metal kernel sources executed on CPU, and (b) that reference-on-CPU build itself
 * (oracle/_ref/libbm_ref.so) wherever it is present.
 *
 * The step driver mirrors the reference's control flow — sequences of a batch processed one after another with
 * gradients accumulating (bm_train_step_masked, src/baremetal/trainer.c:447-533) — including three behaviours of the
 * reference that differ from the exact batch gradient. Each can be switched off with a flag to obtain the intended
 * mathematics:
 *   ORC_Q_NORM_GRAD   RMSNorm weight gradient overwritten per sequence (src/kernels/backward.metal:400);
 *   ORC_Q_GX_CARRY    the layer-0 input gradient is not cleared between the sequences of a window
 *                     (src/baremetal/scheduler.c:263-266, src/baremetal/trainer.c:459-470);
 *   ORC_Q_STALE_EMBED fp32 mode gathers embeddings from the initial table (src/baremetal/trainer.c:287-293).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_Q_NORM_GRAD 1
#define ORC_Q_GX_CARRY 2
#define ORC_Q_STALE_EMBED 4

typedef struct {
    int D, H, L, NH, NKV, V, HD, S;
    int precision; /* 0 = fp32, 2 = bf16 weights (2-D tensors rounded to bf16 for the matmuls, fp32 everywhere else) */
    int quirks;
    float lr, b1, b2, eps, wd, rope_theta;
    int accum_steps;
    /* flat arrays in trainer-state order: per layer ln1w,qw,kw,vw,ow,ln2w,gate,up,down; lnfw; embed */
    size_t P;
    int n_tensors;
    size_t *off, *cnt;
    float *w, *wq /* bf16-rounded copy of w (precision 2) */, *g, *m, *v, *embed_init;
    float* gx_carry; /* [S, D] */
    int step, accum_count, window_seqs;
} orc_t;

/* round-to-nearest-even bf16, as include/baremetal/types.h:22-29 */
static float bf16_round(float x) {
    uint32_t u;
    memcpy(&u, &x, 4);
    u += 0x7FFFu + ((u >> 16) & 1u);
    u &= 0xFFFF0000u;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* ---- kernels ------------------------------------------------------------------------------------------- */

/* out[bt,oc] = sum_i inp[bt,i] * w[oc,i]   (matmul_forward_naive, src/kernels/forward.metal:23-47) */
static void matmul_forward(float* out, const float* inp, const float* w, int BT, int C, int OC) {
#pragma omp parallel for collapse(2) schedule(static)
    for (int bt = 0; bt < BT; bt++)
        for (int oc = 0; oc < OC; oc++) {
            const float* x = inp + (size_t)bt * C;
            const float* wr = w + (size_t)oc * C;
            float acc = 0.0f;
            for (int i = 0; i < C; i++) acc += x[i] * wr[i];
            out[(size_t)bt * OC + oc] = acc;
        }
}
/* ginp[bt,i] += sum_oc gout[bt,oc] * w[oc,i]   (matmul_backward_inp, src/kernels/backward.metal:26-41) */
static void matmul_backward_inp(float* ginp, const float* gout, const float* w, int BT, int C, int OC) {
#pragma omp parallel for collapse(2) schedule(static)
    for (int bt = 0; bt < BT; bt++)
        for (int i = 0; i < C; i++) {
            float acc = 0.0f;
            for (int oc = 0; oc < OC; oc++) acc += gout[(size_t)bt * OC + oc] * w[(size_t)oc * C + i];
            ginp[(size_t)bt * C + i] += acc;
        }
}
/* gw[oc,i] += sum_bt gout[bt,oc] * inp[bt,i]   (matmul_backward_w, src/kernels/backward.metal:94-110) */
static void matmul_backward_w(float* gw, const float* gout, const float* inp, int BT, int C, int OC) {
#pragma omp parallel for collapse(2) schedule(static)
    for (int oc = 0; oc < OC; oc++)
        for (int i = 0; i < C; i++) {
            float acc = 0.0f;
            for (int bt = 0; bt < BT; bt++) acc += gout[(size_t)bt * OC + oc] * inp[(size_t)bt * C + i];
            gw[(size_t)oc * C + i] += acc;
        }
}
/* rmsnorm_forward, src/kernels/forward.metal:993-1014 */
static void rmsnorm_forward(float* out, const float* inp, const float* w, int N, int C, float eps) {
#pragma omp parallel for schedule(static)
    for (int r = 0; r < N; r++) {
        const float* x = inp + (size_t)r * C;
        float ss = 0.0f;
        for (int j = 0; j < C; j++) ss += x[j] * x[j];
        ss /= (float)C;
        const float inv = 1.0f / sqrtf(ss + eps);
        for (int j = 0; j < C; j++) out[(size_t)r * C + j] = x[j] * inv * w[j];
    }
}
/* rmsnorm_backward_x (gx +=), src/kernels/backward.metal:340-372 */
static void rmsnorm_backward_x(float* gx, const float* gout, const float* w, const float* x, int N, int C, float eps) {
#pragma omp parallel for schedule(static)
    for (int r = 0; r < N; r++) {
        const float* xr = x + (size_t)r * C;
        const float* gr = gout + (size_t)r * C;
        float ss = 0.0f;
        for (int j = 0; j < C; j++) ss += xr[j] * xr[j];
        ss /= (float)C;
        const float inv = 1.0f / sqrtf(ss + eps);
        float c1 = 0.0f;
        for (int j = 0; j < C; j++) c1 += gr[j] * xr[j] * inv * w[j];
        c1 /= (float)C;
        for (int j = 0; j < C; j++) {
            const float n = xr[j] * inv;
            gx[(size_t)r * C + j] += inv * (gr[j] * w[j] - n * c1);
        }
    }
}
/* rmsnorm_backward_w, src/kernels/backward.metal:379-401: gw[j] = sum_rows gout*n  (overwrites; `accumulate`
 * selects the intended += instead) */
static void rmsnorm_backward_w(float* gw, const float* gout, const float* x, int N, int C, float eps, int accumulate) {
    float* inv = (float*)malloc((size_t)N * sizeof(float));
    for (int r = 0; r < N; r++) {
        const float* xr = x + (size_t)r * C;
        float ss = 0.0f;
        for (int k = 0; k < C; k++) ss += xr[k] * xr[k];
        ss /= (float)C;
        inv[r] = 1.0f / sqrtf(ss + eps);
    }
#pragma omp parallel for schedule(static)
    for (int j = 0; j < C; j++) {
        float acc = 0.0f;
        for (int r = 0; r < N; r++) acc += gout[(size_t)r * C + j] * (x[(size_t)r * C + j] * inv[r]);
        gw[j] = accumulate ? gw[j] + acc : acc;
    }
    free(inv);
}
/* rope_forward_seq / rope_backward_seq (dir = +1 / -1), src/kernels/forward.metal:2225-2256,
 * src/kernels/backward.metal:980-1012; inverse frequency rope_inv_freq forward.metal:1260-1279 without scaling */
static void rope_seq(float* q, float* k, int S, int NH, int NKV, int HD, float theta, int dir) {
    const int hd2 = HD / 2;
#pragma omp parallel for schedule(static)
    for (int s = 0; s < S; s++)
        for (int h = 0; h < NH + NKV; h++) {
            float* p = h < NH ? q + ((size_t)s * NH + h) * HD : k + ((size_t)s * NKV + (h - NH)) * HD;
            for (int i = 0; i < hd2; i++) {
                const float freq = 1.0f / powf(theta, (float)(2 * i) / (float)HD);
                const float c = cosf((float)s * freq), sn = sinf((float)s * freq) * (float)dir;
                const float x0 = p[i], x1 = p[i + hd2];
                p[i] = x0 * c - x1 * sn;
                p[i + hd2] = x0 * sn + x1 * c;
            }
        }
}
/* attention_forward_seq, src/kernels/forward.metal:1811-1846 */
static void attention_forward(float* out, const float* Q, const float* K, const float* V, int S, int NH, int NKV, int HD, float scale) {
    const int mul = NH / NKV;
#pragma omp parallel for collapse(2) schedule(dynamic, 4)
    for (int h = 0; h < NH; h++)
        for (int i = 0; i < S; i++) {
            const int kh = h / mul, n = i + 1;
            const float* qi = Q + ((size_t)i * NH + h) * HD;
            float* sc = (float*)malloc((size_t)n * sizeof(float));
            float mx = -INFINITY;
            for (int j = 0; j < n; j++) {
                const float* kj = K + ((size_t)j * NKV + kh) * HD;
                float s = 0.0f;
                for (int d = 0; d < HD; d++) s += qi[d] * kj[d];
                sc[j] = s * scale;
                if (sc[j] > mx) mx = sc[j];
            }
            float sum = 0.0f;
            for (int j = 0; j < n; j++) { sc[j] = expf(sc[j] - mx); sum += sc[j]; }
            const float inv = 1.0f / sum;
            for (int j = 0; j < n; j++) sc[j] *= inv;
            float* oi = out + ((size_t)i * NH + h) * HD;
            for (int d = 0; d < HD; d++) {
                float acc = 0.0f;
                for (int j = 0; j < n; j++) acc += sc[j] * V[((size_t)j * NKV + kh) * HD + d];
                oi[d] = acc;
            }
            free(sc);
        }
}
/* attention_backward, src/kernels/backward.metal:665-733. gK/gV accumulate (zeroed by the caller). The reference adds
 * into gK/gV with float atomics in an unspecified order; here the order is fixed (heads, then queries). */
static void attention_backward(float* gQ, float* gK, float* gV, const float* gout, const float* Q, const float* K, const float* V,
                               int S, int NH, int NKV, int HD, float scale) {
    const int mul = NH / NKV;
#pragma omp parallel for schedule(dynamic, 1)
    for (int kh = 0; kh < NKV; kh++)
        for (int h = kh * mul; h < (kh + 1) * mul; h++)
            for (int i = 0; i < S; i++) {
                const int n = i + 1;
                const float* qi = Q + ((size_t)i * NH + h) * HD;
                const float* gi = gout + ((size_t)i * NH + h) * HD;
                float* pr = (float*)malloc((size_t)n * 3 * sizeof(float));
                float* gp = pr + n;
                float* gs = gp + n;
                float mx = -INFINITY;
                for (int j = 0; j < n; j++) {
                    const float* kj = K + ((size_t)j * NKV + kh) * HD;
                    float s = 0.0f;
                    for (int d = 0; d < HD; d++) s += qi[d] * kj[d];
                    s *= scale;
                    pr[j] = s;
                    if (s > mx) mx = s;
                }
                float sum = 0.0f;
                for (int j = 0; j < n; j++) { pr[j] = expf(pr[j] - mx); sum += pr[j]; }
                const float inv = 1.0f / sum;
                for (int j = 0; j < n; j++) pr[j] *= inv;
                float dot = 0.0f;
                for (int j = 0; j < n; j++) {
                    const float* vj = V + ((size_t)j * NKV + kh) * HD;
                    float dp = 0.0f;
                    for (int d = 0; d < HD; d++) dp += gi[d] * vj[d];
                    gp[j] = dp;
                    dot += pr[j] * dp;
                }
                for (int j = 0; j < n; j++) gs[j] = pr[j] * (gp[j] - dot);
                float* gqi = gQ + ((size_t)i * NH + h) * HD;
                for (int d = 0; d < HD; d++) {
                    float acc = 0.0f;
                    for (int j = 0; j < n; j++) acc += gs[j] * K[((size_t)j * NKV + kh) * HD + d];
                    gqi[d] = acc * scale;
                }
                for (int j = 0; j < n; j++)
                    for (int d = 0; d < HD; d++) {
                        gK[((size_t)j * NKV + kh) * HD + d] += scale * gs[j] * qi[d];
                        gV[((size_t)j * NKV + kh) * HD + d] += pr[j] * gi[d];
                    }
                free(pr);
            }
}
/* swiglu_forward src/kernels/forward.metal:1179-1190; swiglu_backward src/kernels/backward.metal:505-521 */
static void swiglu_forward(float* out, const float* gate, const float* up, size_t n) {
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; i++) {
        const float x = gate[i];
        out[i] = x / (1.0f + expf(-x)) * up[i];
    }
}
static void swiglu_backward(float* ggate, float* gup, const float* gate, const float* up, const float* gout, size_t n) {
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; i++) {
        const float x = gate[i], u = up[i], g = gout[i];
        const float s = 1.0f / (1.0f + expf(-x));
        ggate[i] = g * u * s * (1.0f + x * (1.0f - s));
        gup[i] = g * (x * s);
    }
}
/* loss: host loop of bmt_scheduler_xent_backward src/baremetal/scheduler.c:1622-1634; gradient: xent_backward
 * src/kernels/backward.metal:567-591 */
static float xent(float* glogits, const float* logits, const int* targets, int N, int V) {
    float loss = 0.0f;
    for (int s = 0; s < N; s++) {
        const float* lr = logits + (size_t)s * V;
        float mx = lr[0];
        for (int j = 1; j < V; j++) if (lr[j] > mx) mx = lr[j];
        float sum = 0.0f;
        for (int j = 0; j < V; j++) sum += expf(lr[j] - mx);
        loss += -(lr[targets[s]] - mx - logf(sum));
    }
    loss /= (float)N;
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; n++) {
        const float* lr = logits + (size_t)n * V;
        float* gr = glogits + (size_t)n * V;
        float mx = -INFINITY;
        for (int j = 0; j < V; j++) if (lr[j] > mx) mx = lr[j];
        float sum = 0.0f;
        for (int j = 0; j < V; j++) { const float e = expf(lr[j] - mx); gr[j] = e; sum += e; }
        const float inv = 1.0f / sum, invN = 1.0f / (float)N;
        const int tgt = targets[n];
        for (int j = 0; j < V; j++) gr[j] = (gr[j] * inv - (j == tgt ? 1.0f : 0.0f)) * invN;
    }
    return loss;
}
/* adamw_step, src/anneal/adamw.metal:26-46 */
static void adamw(float* w, const float* g, float* m, float* v, size_t n, const float* hp) {
    const float lr = hp[0], b1 = hp[1], b2 = hp[2], eps = hp[3], wd = hp[4], bias1 = hp[5], bias2 = hp[6];
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; i++) {
        const float gi = g[i] * hp[7];
        const float mn = b1 * m[i] + (1.0f - b1) * gi;
        const float vn = b2 * v[i] + (1.0f - b2) * gi * gi;
        m[i] = mn;
        v[i] = vn;
        const float mh = mn / bias1, vh = vn / bias2;
        w[i] = w[i] * (1.0f - lr * wd) - lr * mh / (sqrtf(vh) + eps);
    }
}

/* ---- exported single-kernel entry points (for the golden-vector pins) ------------------------------------- */
void orc_matmul_forward(float* out, const float* inp, const float* w, int BT, int C, int OC) { matmul_forward(out, inp, w, BT, C, OC); }
void orc_matmul_backward_inp(float* ginp, const float* gout, const float* w, int BT, int C, int OC) { matmul_backward_inp(ginp, gout, w, BT, C, OC); }
void orc_matmul_backward_w(float* gw, const float* gout, const float* inp, int BT, int C, int OC) { matmul_backward_w(gw, gout, inp, BT, C, OC); }
void orc_rmsnorm_forward(float* out, const float* inp, const float* w, int N, int C, float eps) { rmsnorm_forward(out, inp, w, N, C, eps); }
void orc_rmsnorm_backward_x(float* gx, const float* gout, const float* w, const float* x, int N, int C, float eps) { rmsnorm_backward_x(gx, gout, w, x, N, C, eps); }
void orc_rmsnorm_backward_w(float* gw, const float* gout, const float* x, int N, int C, float eps) { rmsnorm_backward_w(gw, gout, x, N, C, eps, 0); }
void orc_rope_seq(float* q, float* k, int S, int NH, int NKV, int HD, float theta, int dir) { rope_seq(q, k, S, NH, NKV, HD, theta, dir); }
void orc_attention_forward(float* out, const float* Q, const float* K, const float* V, int S, int NH, int NKV, int HD, float scale) { attention_forward(out, Q, K, V, S, NH, NKV, HD, scale); }
void orc_attention_backward(float* gQ, float* gK, float* gV, const float* gout, const float* Q, const float* K, const float* V, int S, int NH, int NKV, int HD, float scale) { attention_backward(gQ, gK, gV, gout, Q, K, V, S, NH, NKV, HD, scale); }
void orc_swiglu_forward(float* out, const float* gate, const float* up, size_t n) { swiglu_forward(out, gate, up, n); }
void orc_swiglu_backward(float* ggate, float* gup, const float* gate, const float* up, const float* gout, size_t n) { swiglu_backward(ggate, gup, gate, up, gout, n); }
float orc_xent(float* glogits, const float* logits, const int* targets, int N, int V) { return xent(glogits, logits, targets, N, V); }
void orc_adamw(float* w, const float* g, float* m, float* v, size_t n, const float* hp8) { adamw(w, g, m, v, n, hp8); }
/* embedding_backward, src/kernels/backward.metal:636-647 */
void orc_embedding_backward(float* gwte, const float* gout, const int* tokens, int T, int D) {
    for (int t = 0; t < T; t++)
        for (int d = 0; d < D; d++) gwte[(size_t)tokens[t] * D + d] += gout[(size_t)t * D + d];
}
/* argmax branch of bm_sample, src/baremetal/sampler.c:36-40 */
int orc_argmax(const float* logits, int n) {
    int best = 0;
    for (int i = 1; i < n; i++) if (logits[i] > logits[best]) best = i;
    return best;
}

/* ---- trainer ------------------------------------------------------------------------------------------------ */
enum { T_LN1 = 0, T_Q, T_K, T_V, T_O, T_LN2, T_GATE, T_UP, T_DOWN };

/* weights arrive in the reference's model-buffer order (src/baremetal/model.c:140-172): embed, ln1w[L], qw[L], kw[L],
 * vw[L], ow[L], ln2w[L], gate[L], up[L], down[L], lnfw */
orc_t* orc_create(int D, int H, int L, int NH, int NKV, int V, int HD, int S, int precision, int quirks, float lr, float b1, float b2,
                  float eps, float wd, float rope_theta, int accum_steps, const float* model_weights) {
    orc_t* o = (orc_t*)calloc(1, sizeof *o);
    o->D = D; o->H = H; o->L = L; o->NH = NH; o->NKV = NKV; o->V = V; o->HD = HD; o->S = S;
    o->precision = precision; o->quirks = quirks;
    o->lr = lr; o->b1 = b1; o->b2 = b2; o->eps = eps; o->wd = wd; o->rope_theta = rope_theta;
    o->accum_steps = accum_steps > 0 ? accum_steps : 1;
    const size_t QD = (size_t)NH * HD, KV = (size_t)NKV * HD;
    o->n_tensors = 9 * L + 2;
    o->off = (size_t*)calloc(o->n_tensors, sizeof(size_t));
    o->cnt = (size_t*)calloc(o->n_tensors, sizeof(size_t));
    const size_t sizes[9] = {(size_t)D, QD * D, KV * D, KV * D, (size_t)D * QD, (size_t)D, (size_t)H * D, (size_t)H * D, (size_t)D * H};
    size_t off = 0;
    for (int l = 0; l < L; l++)
        for (int k = 0; k < 9; k++) { o->off[9 * l + k] = off; o->cnt[9 * l + k] = sizes[k]; off += sizes[k]; }
    o->off[9 * L] = off; o->cnt[9 * L] = D; off += D;
    o->off[9 * L + 1] = off; o->cnt[9 * L + 1] = (size_t)V * D; off += (size_t)V * D;
    o->P = off;
    o->w = (float*)malloc(off * sizeof(float));
    o->g = (float*)calloc(off, sizeof(float));
    o->m = (float*)calloc(off, sizeof(float));
    o->v = (float*)calloc(off, sizeof(float));
    o->gx_carry = (float*)calloc((size_t)S * D, sizeof(float));
    /* scatter from model order into state order */
    const float* src = model_weights;
    const float* embed = src; src += (size_t)V * D;
    const float* bases[9];
    const int order[9] = {T_LN1, T_Q, T_K, T_V, T_O, T_LN2, T_GATE, T_UP, T_DOWN};
    for (int k = 0; k < 9; k++) { bases[order[k]] = src; src += sizes[order[k]] * L; }
    const float* lnf = src;
    for (int l = 0; l < L; l++)
        for (int k = 0; k < 9; k++) memcpy(o->w + o->off[9 * l + k], bases[k] + sizes[k] * l, sizes[k] * sizeof(float));
    memcpy(o->w + o->off[9 * L], lnf, (size_t)D * sizeof(float));
    memcpy(o->w + o->off[9 * L + 1], embed, (size_t)V * D * sizeof(float));
    o->embed_init = (float*)malloc((size_t)V * D * sizeof(float));
    memcpy(o->embed_init, embed, (size_t)V * D * sizeof(float));
    if (precision == 2) {
        o->wq = (float*)malloc(off * sizeof(float));
        for (size_t i = 0; i < off; i++) o->wq[i] = bf16_round(o->w[i]);
    }
    return o;
}
void orc_destroy(orc_t* o) {
    if (!o) return;
    free(o->off); free(o->cnt); free(o->w); free(o->wq); free(o->g); free(o->m); free(o->v); free(o->embed_init); free(o->gx_carry);
    free(o);
}
int orc_num_tensors(orc_t* o) { return o->n_tensors; }
size_t orc_tensor_size(orc_t* o, int i) { return o->cnt[i]; }
/* what: 0 weight (fp32 master), 1 grad, 2 m, 3 v */
void orc_read(orc_t* o, int what, int i, float* out) {
    const float* base = what == 0 ? o->w : what == 1 ? o->g : what == 2 ? o->m : o->v;
    memcpy(out, base + o->off[i], o->cnt[i] * sizeof(float));
}

/* matmul weight: bf16-rounded copy in bf16 mode (the reference stores 2-D weights as bf16 on the device,
 * src/baremetal/scheduler.c:369-402), fp32 otherwise. 1-D norm weights are always fp32. */
static const float* mw(const orc_t* o, int idx) { return (o->precision == 2 ? o->wq : o->w) + o->off[idx]; }

static float one_sequence(orc_t* o, const int* tokens, const int* targets) {
    const int D = o->D, H = o->H, L = o->L, NH = o->NH, NKV = o->NKV, V = o->V, HD = o->HD, S = o->S;
    const int QD = NH * HD, KV = NKV * HD;
    const float eps = 1e-5f, scale = 1.0f / sqrtf((float)HD);
    const int p_lnf = 9 * L, p_emb = 9 * L + 1;
    typedef struct { float *x, *n1, *q, *k, *v, *att, *x1, *n2, *gate, *up, *act; } lay_t;
    lay_t* a = (lay_t*)calloc(L, sizeof(lay_t));
#define NEW(n) ((float*)calloc((size_t)(n), sizeof(float)))
    float* x = NEW((size_t)S * D);
    /* embed_lookup, src/baremetal/trainer.c:275-298: fp32 master in mixed precision; the initial host table in fp32 mode */
    const float* table = (o->precision == 0 && (o->quirks & ORC_Q_STALE_EMBED)) ? o->embed_init : o->w + o->off[p_emb];
    for (int s = 0; s < S; s++) memcpy(x + (size_t)s * D, table + (size_t)tokens[s] * D, (size_t)D * sizeof(float));
    float* cur = x;
    for (int l = 0; l < L; l++) {
        lay_t* c = &a[l];
        const int pb = 9 * l;
        c->x = cur;
        c->n1 = NEW((size_t)S * D); c->q = NEW((size_t)S * QD); c->k = NEW((size_t)S * KV); c->v = NEW((size_t)S * KV);
        c->att = NEW((size_t)S * QD); c->x1 = NEW((size_t)S * D); c->n2 = NEW((size_t)S * D);
        c->gate = NEW((size_t)S * H); c->up = NEW((size_t)S * H); c->act = NEW((size_t)S * H);
        rmsnorm_forward(c->n1, c->x, o->w + o->off[pb + T_LN1], S, D, eps);
        matmul_forward(c->q, c->n1, mw(o, pb + T_Q), S, D, QD);
        matmul_forward(c->k, c->n1, mw(o, pb + T_K), S, D, KV);
        matmul_forward(c->v, c->n1, mw(o, pb + T_V), S, D, KV);
        rope_seq(c->q, c->k, S, NH, NKV, HD, o->rope_theta, +1);
        attention_forward(c->att, c->q, c->k, c->v, S, NH, NKV, HD, scale);
        float* proj = NEW((size_t)S * D);
        matmul_forward(proj, c->att, mw(o, pb + T_O), S, QD, D);
        for (size_t i = 0; i < (size_t)S * D; i++) c->x1[i] = c->x[i] + proj[i]; /* add_forward, forward.metal:1332 */
        rmsnorm_forward(c->n2, c->x1, o->w + o->off[pb + T_LN2], S, D, eps);
        matmul_forward(c->gate, c->n2, mw(o, pb + T_GATE), S, D, H);
        matmul_forward(c->up, c->n2, mw(o, pb + T_UP), S, D, H);
        swiglu_forward(c->act, c->gate, c->up, (size_t)S * H);
        matmul_forward(proj, c->act, mw(o, pb + T_DOWN), S, H, D);
        float* nx = NEW((size_t)S * D);
        for (size_t i = 0; i < (size_t)S * D; i++) nx[i] = c->x1[i] + proj[i];
        free(proj);
        cur = nx;
    }
    float* nf = NEW((size_t)S * D);
    rmsnorm_forward(nf, cur, o->w + o->off[p_lnf], S, D, eps);
    float* logits = NEW((size_t)S * V);
    matmul_forward(logits, nf, mw(o, p_emb), S, D, V);
    float* glogits = NEW((size_t)S * V);
    const float loss = xent(glogits, logits, targets, S, V);
    free(logits);

    /* backward (bmt_scheduler_backward, src/baremetal/scheduler.c:1364-1617) */
    const int acc_norm = (o->quirks & ORC_Q_NORM_GRAD) ? 0 : 1;
    float* gres = NEW((size_t)S * D);
    float* gn = NEW((size_t)S * D);
    matmul_backward_inp(gn, glogits, mw(o, p_emb), S, D, V);
    matmul_backward_w(o->g + o->off[p_emb], glogits, nf, S, D, V);
    free(glogits);
    rmsnorm_backward_x(gres, gn, o->w + o->off[p_lnf], cur, S, D, eps);
    rmsnorm_backward_w(o->g + o->off[p_lnf], gn, cur, S, D, eps, acc_norm);
    for (int l = L - 1; l >= 0; l--) {
        lay_t* c = &a[l];
        const int pb = 9 * l;
        /* gres = dL/d(x_{l+1}); add_backward routes it to both inputs of the residual add (backward.metal:530) */
        float* gact = NEW((size_t)S * H);
        matmul_backward_inp(gact, gres, mw(o, pb + T_DOWN), S, H, D);
        matmul_backward_w(o->g + o->off[pb + T_DOWN], gres, c->act, S, H, D);
        float* ggate = NEW((size_t)S * H);
        float* gup = NEW((size_t)S * H);
        swiglu_backward(ggate, gup, c->gate, c->up, gact, (size_t)S * H);
        free(gact);
        memset(gn, 0, (size_t)S * D * sizeof(float));
        matmul_backward_inp(gn, ggate, mw(o, pb + T_GATE), S, D, H);
        matmul_backward_w(o->g + o->off[pb + T_GATE], ggate, c->n2, S, D, H);
        matmul_backward_inp(gn, gup, mw(o, pb + T_UP), S, D, H);
        matmul_backward_w(o->g + o->off[pb + T_UP], gup, c->n2, S, D, H);
        free(ggate); free(gup);
        rmsnorm_backward_x(gres, gn, o->w + o->off[pb + T_LN2], c->x1, S, D, eps);
        rmsnorm_backward_w(o->g + o->off[pb + T_LN2], gn, c->x1, S, D, eps, acc_norm);
        /* attention block: gres = dL/d(x1) */
        float* gatt = NEW((size_t)S * QD);
        matmul_backward_inp(gatt, gres, mw(o, pb + T_O), S, QD, D);
        matmul_backward_w(o->g + o->off[pb + T_O], gres, c->att, S, QD, D);
        float* gq = NEW((size_t)S * QD);
        float* gk = NEW((size_t)S * KV);
        float* gv = NEW((size_t)S * KV);
        attention_backward(gq, gk, gv, gatt, c->q, c->k, c->v, S, NH, NKV, HD, scale);
        free(gatt);
        rope_seq(gq, gk, S, NH, NKV, HD, o->rope_theta, -1);
        memset(gn, 0, (size_t)S * D * sizeof(float));
        matmul_backward_inp(gn, gq, mw(o, pb + T_Q), S, D, QD);
        matmul_backward_w(o->g + o->off[pb + T_Q], gq, c->n1, S, D, QD);
        matmul_backward_inp(gn, gk, mw(o, pb + T_K), S, D, KV);
        matmul_backward_w(o->g + o->off[pb + T_K], gk, c->n1, S, D, KV);
        matmul_backward_inp(gn, gv, mw(o, pb + T_V), S, D, KV);
        matmul_backward_w(o->g + o->off[pb + T_V], gv, c->n1, S, D, KV);
        free(gq); free(gk); free(gv);
        rmsnorm_backward_x(gres, gn, o->w + o->off[pb + T_LN1], c->x, S, D, eps);
        rmsnorm_backward_w(o->g + o->off[pb + T_LN1], gn, c->x, S, D, eps, acc_norm);
    }
    /* embed_backward (src/baremetal/trainer.c:302-346): scatter the layer-0 input gradient into the tied table's gradient */
    if (o->quirks & ORC_Q_GX_CARRY) {
        for (size_t i = 0; i < (size_t)S * D; i++) { o->gx_carry[i] += gres[i]; gres[i] = o->gx_carry[i]; }
    }
    orc_embedding_backward(o->g + o->off[p_emb], gres, tokens, S, D);
    /* release */
    free(gres); free(gn); free(nf);
    free(cur);
    for (int l = 0; l < L; l++) {
        lay_t* c = &a[l];
        if (l == 0) free(c->x); /* x of layer l > 0 is the output buffer of layer l-1, released in the loop below */
        free(c->n1); free(c->q); free(c->k); free(c->v); free(c->att); free(c->x1); free(c->n2); free(c->gate); free(c->up); free(c->act);
    }
    for (int l = 1; l < L; l++) free(a[l].x);
    free(a);
#undef NEW
    return loss;
}

/* bm_train_step, src/baremetal/trainer.c:447-533 */
float orc_step(orc_t* o, const int* inputs, const int* targets, int B) {
    if (o->accum_count == 0) {
        memset(o->g, 0, o->P * sizeof(float));
        memset(o->gx_carry, 0, (size_t)o->S * o->D * sizeof(float));
    }
    float total = 0.0f;
    for (int b = 0; b < B; b++) total += one_sequence(o, inputs + (size_t)b * o->S, targets + (size_t)b * o->S);
    o->window_seqs += B;
    o->accum_count++;
    if (o->accum_count >= o->accum_steps) {
        /* adamw_apply, src/baremetal/trainer.c:349-398 */
        o->step++;
        const float bias1 = 1.0f - powf(o->b1, (float)o->step), bias2 = 1.0f - powf(o->b2, (float)o->step);
        const float hp[8] = {o->lr, o->b1, o->b2, o->eps, o->wd, bias1, bias2, 1.0f / (float)(o->window_seqs > 0 ? o->window_seqs : 1)};
        adamw(o->w, o->g, o->m, o->v, o->P, hp);
        if (o->wq) {
            /* only 2-D tensors are re-rounded; norm weights stay fp32 (src/baremetal/trainer.c:373-396) */
            for (size_t i = 0; i < o->P; i++) o->wq[i] = bf16_round(o->w[i]);
        }
        o->accum_count = 0;
        o->window_seqs = 0;
    }
    return total / (float)B;
}

/* ======================= inference: prefill / decode with a KV cache, Q8 or plain weights =========================
 * Restates the reference's decode walk (src/baremetal/scheduler.c:712-996 over the graph of src/baremetal/graph.c:109-240):
 * fp32 activations, fp32 KV cache, layer matrices optionally Q8 or Q4 (src/baremetal/quant.c:10-52), LM head never quantised
 * (graph.c:228-239). Matmul with Q8 weights: val += x[i] * ((float)q[i] * scale) (matmul_forward_q8,
 * src/kernels/forward.metal:625-648). */
size_t orc_quantize_q8(const float* src, int8_t* q, float* scales, size_t n) {
    if (n == 0 || (n % 32) != 0) return 0;
    for (size_t b = 0; b < n / 32; b++) {
        const float* p = src + b * 32;
        float amax = 0.0f;
        for (int i = 0; i < 32; i++) { const float a = fabsf(p[i]); if (a > amax) amax = a; }
        const float scale = amax / 127.0f;
        scales[b] = scale;
        if (scale == 0.0f) { memset(q + b * 32, 0, 32); continue; }
        const float inv = 1.0f / scale;
        for (int i = 0; i < 32; i++) {
            long v = lroundf(p[i] * inv);
            if (v > 127) v = 127;
            if (v < -128) v = -128;
            q[b * 32 + i] = (int8_t)v;
        }
    }
    return n / 32;
}

/* Q4 (src/baremetal/quant.c:31-52): scale = amax / 7, codes clamped to [-8, 7]. The reference packs code 2j into the low and
 * code 2j+1 into the high nibble of byte j and its kernels sign-extend them again (matmul_forward_q4,
 * src/kernels/forward.metal:830-858: val += x[2j] * ((float)lo * s); val += x[2j+1] * ((float)hi * s), the Q8 arithmetic on the
 * narrower codes); here the codes stay one per byte. */
size_t orc_quantize_q4(const float* src, int8_t* q, float* scales, size_t n) {
    if (n == 0 || (n % 32) != 0) return 0;
    for (size_t b = 0; b < n / 32; b++) {
        const float* p = src + b * 32;
        float amax = 0.0f;
        for (int i = 0; i < 32; i++) { const float a = fabsf(p[i]); if (a > amax) amax = a; }
        const float scale = amax / 7.0f;
        scales[b] = scale;
        if (scale == 0.0f) { memset(q + b * 32, 0, 32); continue; }
        const float inv = 1.0f / scale;
        for (int i = 0; i < 32; i++) {
            long v = lroundf(p[i] * inv);
            if (v > 7) v = 7;
            if (v < -8) v = -8;
            q[b * 32 + i] = (int8_t)v;
        }
    }
    return n / 32;
}

typedef struct { float* w; int8_t* q; float* sc; int OC, C; } orc_mat_t;
typedef struct {
    int D, H, L, NH, NKV, V, HD, MS, pos, quant;
    float theta;
    float *ln1, *ln2, *lnf, *head, *embed;   /* ln1/ln2: [L][D]; head: [V][D] (bf16-rounded in bf16 mode); embed: [V][D] as loaded */
    orc_mat_t *q, *k, *v, *o, *gate, *up, *down;   /* [L] */
    float* cache;                    /* [L][2][MS][KV] */
    float* logits;
} orc_dec_t;

static void mat_init(orc_mat_t* m, const float* src, int OC, int C, int quant, int round_bf16) {
    m->OC = OC; m->C = C; m->w = NULL; m->q = NULL; m->sc = NULL;
    const size_t n = (size_t)OC * C;
    if (quant == 8 || quant == 4) {
        /* from the loaded fp32 values (src/baremetal/scheduler.c:378-392; a bf16 source widens exactly) */
        m->q = (int8_t*)malloc(n);
        m->sc = (float*)malloc(n / 32 * sizeof(float));
        if (quant == 8) orc_quantize_q8(src, m->q, m->sc, n);
        else orc_quantize_q4(src, m->q, m->sc, n);
    } else {
        m->w = (float*)malloc(n * sizeof(float));
        for (size_t i = 0; i < n; i++) m->w[i] = round_bf16 ? bf16_round(src[i]) : src[i];
    }
}
static void mat_free(orc_mat_t* m) { free(m->w); free(m->q); free(m->sc); }
static void mat_vec(float* out, const orc_mat_t* m, const float* x) {
#pragma omp parallel for schedule(static)
    for (int oc = 0; oc < m->OC; oc++) {
        float val = 0.0f;
        if (m->q) {
            const int nb = m->C / 32;
            for (int b = 0; b < nb; b++) {
                const float s = m->sc[(size_t)oc * nb + b];
                const int8_t* qb = m->q + (size_t)oc * m->C + b * 32;
                const float* xb = x + b * 32;
                for (int i = 0; i < 32; i++) val += xb[i] * ((float)qb[i] * s);
            }
        } else {
            const float* wr = m->w + (size_t)oc * m->C;
            for (int i = 0; i < m->C; i++) val += x[i] * wr[i];
        }
        out[oc] = val;
    }
}

orc_dec_t* orc_dec_create(int D, int H, int L, int NH, int NKV, int V, int HD, int MS, int quant, int lowp_bf16, float theta,
                          const float* model_weights) {
    orc_dec_t* o = (orc_dec_t*)calloc(1, sizeof *o);
    o->D = D; o->H = H; o->L = L; o->NH = NH; o->NKV = NKV; o->V = V; o->HD = HD; o->MS = MS; o->quant = quant; o->theta = theta;
    const size_t QD = (size_t)NH * HD, KV = (size_t)NKV * HD;
    const float* src = model_weights;   /* model order: embed, ln1w[L], qw[L], kw[L], vw[L], ow[L], ln2w[L], gate[L], up[L], down[L], lnfw */
    const float* embed = src; src += (size_t)V * D;
    const float* ln1 = src; src += (size_t)L * D;
    const float* qw = src; src += L * QD * D;
    const float* kw = src; src += L * KV * D;
    const float* vw = src; src += L * KV * D;
    const float* ow = src; src += L * D * QD;
    const float* ln2 = src; src += (size_t)L * D;
    const float* gw = src; src += (size_t)L * H * D;
    const float* uw = src; src += (size_t)L * H * D;
    const float* dw = src; src += (size_t)L * D * H;
    const float* lnf = src;
    o->ln1 = (float*)malloc((size_t)L * D * 4); memcpy(o->ln1, ln1, (size_t)L * D * 4);
    o->ln2 = (float*)malloc((size_t)L * D * 4); memcpy(o->ln2, ln2, (size_t)L * D * 4);
    o->lnf = (float*)malloc((size_t)D * 4); memcpy(o->lnf, lnf, (size_t)D * 4);
    o->head = (float*)malloc((size_t)V * D * 4);
    o->embed = (float*)malloc((size_t)V * D * 4);
    memcpy(o->embed, embed, (size_t)V * D * 4);   /* the host gathers rows of the loaded table (src/baremetal/session.c:114-123) */
    for (size_t i = 0; i < (size_t)V * D; i++) o->head[i] = lowp_bf16 ? bf16_round(embed[i]) : embed[i];
    orc_mat_t** arrs[7] = {&o->q, &o->k, &o->v, &o->o, &o->gate, &o->up, &o->down};
    for (int i = 0; i < 7; i++) *arrs[i] = (orc_mat_t*)calloc(L, sizeof(orc_mat_t));
    const int plain_bf16 = lowp_bf16;
    for (int l = 0; l < L; l++) {
        mat_init(&o->q[l], qw + l * QD * D, (int)QD, D, quant, plain_bf16);
        mat_init(&o->k[l], kw + l * KV * D, (int)KV, D, quant, plain_bf16);
        mat_init(&o->v[l], vw + l * KV * D, (int)KV, D, quant, plain_bf16);
        mat_init(&o->o[l], ow + l * D * QD, D, (int)QD, quant, plain_bf16);
        mat_init(&o->gate[l], gw + (size_t)l * H * D, H, D, quant, plain_bf16);
        mat_init(&o->up[l], uw + (size_t)l * H * D, H, D, quant, plain_bf16);
        mat_init(&o->down[l], dw + (size_t)l * D * H, D, H, quant, plain_bf16);
    }
    o->cache = (float*)calloc((size_t)L * 2 * MS * KV, sizeof(float));
    o->logits = (float*)malloc((size_t)V * sizeof(float));
    return o;
}
void orc_dec_destroy(orc_dec_t* o) {
    if (!o) return;
    orc_mat_t* arrs[7] = {o->q, o->k, o->v, o->o, o->gate, o->up, o->down};
    for (int i = 0; i < 7; i++) { for (int l = 0; l < o->L; l++) mat_free(&arrs[i][l]); free(arrs[i]); }
    free(o->ln1); free(o->ln2); free(o->lnf); free(o->head); free(o->embed); free(o->cache); free(o->logits);
    free(o);
}
void orc_dec_reset(orc_dec_t* o) { o->pos = 0; }

/* bm_step, src/baremetal/session.c:151-185 */
float* orc_dec_step(orc_dec_t* o, int token) {
    const int D = o->D, H = o->H, NH = o->NH, NKV = o->NKV, HD = o->HD, MS = o->MS, pos = o->pos;
    const int QD = NH * HD, KV = NKV * HD, mul = NH / NKV, hd2 = HD / 2;
    const float eps = 1e-5f, scale = 1.0f / sqrtf((float)HD);
    float *x = (float*)malloc(D * 4), *xn = (float*)malloc(D * 4), *q = (float*)malloc(QD * 4), *k = (float*)malloc(KV * 4),
          *v = (float*)malloc(KV * 4), *att = (float*)malloc(QD * 4), *t = (float*)malloc(D * 4), *g = (float*)malloc(H * 4),
          *u = (float*)malloc(H * 4), *sc = (float*)malloc((size_t)(pos + 1) * 4);
    memcpy(x, o->embed + (size_t)token * D, D * 4);
    for (int l = 0; l < o->L; l++) {
        rmsnorm_forward(xn, x, o->ln1 + (size_t)l * D, 1, D, eps);
        mat_vec(q, &o->q[l], xn); mat_vec(k, &o->k[l], xn); mat_vec(v, &o->v[l], xn);
        /* rope_forward at this position, src/kernels/forward.metal:1284-1314 */
        for (int h = 0; h < NH + NKV; h++) {
            float* p = h < NH ? q + h * HD : k + (h - NH) * HD;
            for (int i = 0; i < hd2; i++) {
                const float freq = 1.0f / powf(o->theta, (float)(2 * i) / (float)HD);
                const float c = cosf((float)pos * freq), s = sinf((float)pos * freq);
                const float x0 = p[i], x1 = p[i + hd2];
                p[i] = x0 * c - x1 * s;
                p[i + hd2] = x0 * s + x1 * c;
            }
        }
        float* kc = o->cache + ((size_t)l * 2 + 0) * MS * KV;
        float* vc = o->cache + ((size_t)l * 2 + 1) * MS * KV;
        memcpy(kc + (size_t)pos * KV, k, KV * 4);   /* kv_store, forward.metal:1317 */
        memcpy(vc + (size_t)pos * KV, v, KV * 4);
        /* attention_forward, forward.metal:1362-1460: softmax over positions 0..pos */
        for (int h = 0; h < NH; h++) {
            const int kh = h / mul;
            float mx = -INFINITY;
            for (int tt = 0; tt <= pos; tt++) {
                float s = 0.0f;
                for (int i = 0; i < HD; i++) s += q[h * HD + i] * kc[(size_t)tt * KV + kh * HD + i];
                sc[tt] = s * scale;
                if (sc[tt] > mx) mx = sc[tt];
            }
            float sum = 0.0f;
            for (int tt = 0; tt <= pos; tt++) { sc[tt] = expf(sc[tt] - mx); sum += sc[tt]; }
            for (int d = 0; d < HD; d++) {
                float acc = 0.0f;
                for (int tt = 0; tt <= pos; tt++) acc += sc[tt] * vc[(size_t)tt * KV + kh * HD + d];
                att[h * HD + d] = acc / sum;
            }
        }
        mat_vec(t, &o->o[l], att);
        for (int i = 0; i < D; i++) x[i] += t[i];
        rmsnorm_forward(xn, x, o->ln2 + (size_t)l * D, 1, D, eps);
        mat_vec(g, &o->gate[l], xn); mat_vec(u, &o->up[l], xn);
        for (int i = 0; i < H; i++) g[i] = g[i] / (1.0f + expf(-g[i])) * u[i];
        mat_vec(t, &o->down[l], g);
        for (int i = 0; i < D; i++) x[i] += t[i];
    }
    rmsnorm_forward(xn, x, o->lnf, 1, D, eps);
    orc_mat_t head = {o->head, NULL, NULL, o->V, D};
    mat_vec(o->logits, &head, xn);
    o->pos++;
    free(x); free(xn); free(q); free(k); free(v); free(att); free(t); free(g); free(u); free(sc);
    return o->logits;
}
