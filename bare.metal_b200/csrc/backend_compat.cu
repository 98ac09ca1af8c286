// The reference's internal backend ABI (src/backend/backend.h:17-67) on CUDA: context, host-visible buffers, kernels looked up by
// NAME, blocking dispatch and command encoders. It exists so that the reference's own C11 host code (graph, scheduler, trainer)
// and its kernel tests can run against this library unchanged; the training step of this library does not use it (it calls the
// typed bmc_* entry points of bm_cuda_backend.h, which fuse and batch what this ABI dispatches one kernel at a time).
//
// What the ABI promises its callers, and how it is kept here:
//   * backend_buffer_map() returns a host pointer that stays valid for the buffer's life, shows every GPU write completed before
//     the last wait, and whose host writes are seen by the next dispatch; unmap may be omitted (tools/cli.c:115-121). Buffers are
//     CUDA managed allocations: one address for host and device, pages migrate on demand, and map() waits for the stream.
//   * Dispatches of one encoder run in order with full memory visibility between them (a Metal serial encoder): every dispatch is
//     enqueued on one stream at encode time.
//   * Scalar parameters arrive as buffers (`constant int*`, `constant float&`) in a fixed slot order per kernel name; they are read
//     on the host when the dispatch is encoded. offsets[] are byte offsets (the scheduler uses them for zero_buffer only,
//     src/baremetal/scheduler.c:1378-1381).
//   * The grid is Metal's (total threads); launch geometry here comes from the parameter values instead. embedding_backward is the
//     one kernel whose token count exists only in the grid (grid = T * D).
//   * backend_kernel_create() returns NULL for a name this backend does not serve; the reference degrades to a sibling kernel
//     (src/baremetal/scheduler.c:1117-1146, 1430-1456).
// Activations are fp32 through this ABI, as everywhere in the reference; bf16 weight matrices are widened to fp32 before the GEMM,
// which is the reference's arithmetic for its bf16 mode (matmul_forward_bf16, src/kernels/forward.metal:52).
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <map>
#include <string>
#include <vector>

#include "../../include/backend.h"
#include "kernels.cuh"

extern "C" float* bm_build_rope_table(float theta, int scaling, float factor, float low, float high, float orig, int S, int HD);

using namespace bmb;

namespace {

struct Compat;

struct Launch {
    void** b;       // slot pointers (buffer base + byte offset)
    size_t* bytes;  // bytes from the slot pointer to the end of its buffer
    int nb;
    long grid;      // total threads the caller asked for
    cudaStream_t st;
    Compat* cx;
};
typedef int (*KernelFn)(const Launch&);
struct KernelEntry { KernelFn fn; int min_slots; };

// The public handle is the first member, so a backend_ctx_t* is also a Compat*.
struct Compat {
    backend_ctx_s pub;
    cudaStream_t st;
    int* d_err;
    void* scratch[6];
    size_t scratch_bytes[6];
    std::map<std::string, float*> rope_tables;  // device tables keyed by their parameters
};

void* scratch(Compat* cx, int slot, size_t bytes) {
    if (cx->scratch_bytes[slot] >= bytes) return cx->scratch[slot];
    if (cx->scratch[slot]) {
        cudaStreamSynchronize(cx->st);
        cudaFree(cx->scratch[slot]);
        cx->scratch[slot] = nullptr;
        cx->scratch_bytes[slot] = 0;
    }
    if (cudaMalloc(&cx->scratch[slot], bytes) != cudaSuccess) return nullptr;
    cx->scratch_bytes[slot] = bytes;
    return cx->scratch[slot];
}

const int* ip(const Launch& l, int slot) { return (const int*)l.b[slot]; }
const float* fp(const Launch& l, int slot) { return (const float*)l.b[slot]; }
float* fpw(const Launch& l, int slot) { return (float*)l.b[slot]; }

__global__ void fill_kernel(float* p, float v, size_t n) {
    const size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if (i < n) p[i] = v;
}
// row weights of the masked cross-entropy: 1 / count for a row that counts, 0 for a masked one (xent_backward_masked,
// src/kernels/backward.metal:597-624)
__global__ void mask_weights_kernel(float* w, const unsigned char* mask, int n, float inv_count) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) w[i] = mask[i] ? inv_count : 0.f;
}

// Element-granular forms for shapes the 16-byte-vector kernels of the training step do not take (a vocabulary or a width that is
// not a multiple of 4, as in the reference's small kernel tests): same results, one element per thread.
__global__ void embedding_backward_any_kernel(float* gwte, const float* gout, const int* tokens, int T, int D, int V, int* err) {
    const long i = blockIdx.x * (long)blockDim.x + threadIdx.x;
    if (i >= (long)T * D) return;
    const int t = (int)(i / D), d = (int)(i - (long)t * D), tok = tokens[t];
    if ((unsigned)tok >= (unsigned)V) {
        if (d == 0 && err) atomicExch(err, BMB_ERR_BAD_TOKEN);
        return;
    }
    atomicAdd(gwte + (size_t)tok * D + d, gout[i]);
}
// one block per row: (softmax - onehot) * row scale; a row of weight 0 gets a zero gradient
__global__ void xent_any_kernel(float* glogits, const float* logits, const int* targets, const float* row_weight, int V, float scale,
                                int* err) {
    __shared__ float red[32];
    const int row = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float* lr = logits + (size_t)row * V;
    float* gr = glogits + (size_t)row * V;
    if (row_weight) scale = row_weight[row];
    if (row_weight && scale == 0.f) {
        for (int j = threadIdx.x; j < V; j += blockDim.x) gr[j] = 0.f;
        return;
    }
    float mx = -INFINITY;
    for (int j = threadIdx.x; j < V; j += blockDim.x) mx = fmaxf(mx, lr[j]);
    mx = warp_max(mx);
    if (lane == 0) red[warp] = mx;
    __syncthreads();
    mx = red[0];
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w) mx = fmaxf(mx, red[w]);
    __syncthreads();
    float sum = 0.f;
    for (int j = threadIdx.x; j < V; j += blockDim.x) sum += expf(lr[j] - mx);
    sum = warp_sum(sum);
    if (lane == 0) red[warp] = sum;
    __syncthreads();
    sum = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) sum += red[w];
    const int tgt = targets[row];
    if ((unsigned)tgt >= (unsigned)V && threadIdx.x == 0 && err) atomicExch(err, BMB_ERR_BAD_TARGET);
    const float inv = 1.0f / sum;
    for (int j = threadIdx.x; j < V; j += blockDim.x) gr[j] = (expf(lr[j] - mx) * inv - (j == tgt ? 1.0f : 0.0f)) * scale;
}
__global__ void swiglu_forward_any_kernel(float* out, const float* gate, const float* up, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = gate[i] / (1.0f + expf(-gate[i])) * up[i];
}
__global__ void swiglu_backward_any_kernel(float* gg, float* gu, const float* gate, const float* up, const float* gout, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float x = gate[i], s = 1.0f / (1.0f + expf(-x));
    gg[i] = gout[i] * up[i] * s * (1.0f + x * (1.0f - s));
    gu[i] = gout[i] * (x * s);
}
__global__ void adamw_any_kernel(float* w, const float* g, float* m, float* v, int n, float lr, float b1, float b2, float eps, float wd,
                                 float bias1, float bias2, float gs) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float gi = g[i] * gs;
    const float mn = b1 * m[i] + (1.0f - b1) * gi, vn = b2 * v[i] + (1.0f - b2) * gi * gi;
    m[i] = mn;
    v[i] = vn;
    w[i] = w[i] * (1.0f - lr * wd) - lr * (mn / bias1) / (sqrtf(vn / bias2) + eps);
}

// ---- linear layers: slots 0 inp [BT,C], 1 weight [OC,C], 2 bias, 3 out [BT,OC], 4 params {BT, C, OC, has_bias} ----------------------
int mm_forward(const Launch& l, bool w_bf16) {
    const int *p = ip(l, 4), BT = p[0], C = p[1], OC = p[2];
    if (p[3]) return -1;  // the reference never enables the bias (src/baremetal/scheduler.c:1154)
    const float* w = fp(l, 1);
    if (w_bf16) {
        float* wf = (float*)scratch(l.cx, 0, (size_t)OC * C * sizeof(float));
        if (!wf || cast_bf16_to_f32(wf, (const bf16*)l.b[1], (size_t)OC * C, l.st)) return -1;
        w = wf;
    }
    return gemm_f32_simt(fpw(l, 3), OC, 0, fp(l, 0), C, 1, w, C, 1, nullptr, 0, BT, OC, C, l.st);
}
int k_mm_forward_f32(const Launch& l) { return mm_forward(l, false); }
int k_mm_forward_bf16(const Launch& l) { return mm_forward(l, true); }
// slots 0 gout [BT,OC], 1 w [OC,C], 2 ginp [BT,C] (+=), 3 params {BT, C, OC}
int mm_backward_inp(const Launch& l, bool w_bf16) {
    const int *p = ip(l, 3), BT = p[0], C = p[1], OC = p[2];
    const float* w = fp(l, 1);
    if (w_bf16) {
        float* wf = (float*)scratch(l.cx, 0, (size_t)OC * C * sizeof(float));
        if (!wf || cast_bf16_to_f32(wf, (const bf16*)l.b[1], (size_t)OC * C, l.st)) return -1;
        w = wf;
    }
    return gemm_f32_simt(fpw(l, 2), C, 1, fp(l, 0), OC, 1, w, 1, C, nullptr, 0, BT, C, OC, l.st);
}
int k_mm_backward_inp_f32(const Launch& l) { return mm_backward_inp(l, false); }
int k_mm_backward_inp_bf16(const Launch& l) { return mm_backward_inp(l, true); }
// slots 0 gout [BT,OC], 1 inp [BT,C], 2 gw [OC,C] (+=), 3 params {BT, C, OC}
int k_mm_backward_w(const Launch& l) {
    const int *p = ip(l, 3), BT = p[0], C = p[1], OC = p[2];
    return gemm_f32_simt(fpw(l, 2), C, 1, fp(l, 0), 1, OC, fp(l, 1), 1, C, nullptr, 0, OC, C, BT, l.st);
}

// ---- RMSNorm ----------------------------------------------------------------------------------------------------------------
// slots 0 inp [N,C], 1 weight [C], 2 out, 3 params {N, C}, 4 eps
int k_rmsnorm_forward(const Launch& l) {
    const int *p = ip(l, 3), N = p[0], C = p[1];
    float* rstd = (float*)scratch(l.cx, 1, (size_t)N * sizeof(float));
    if (!rstd) return -1;
    return rmsnorm_forward<float>(fpw(l, 2), rstd, fp(l, 0), fp(l, 1), N, C, *fp(l, 4), l.st);
}
// 1 / rms per row of x, by a forward pass whose output is discarded
float* row_rstd(const Launch& l, const float* x, int N, int C, float eps) {
    float* rstd = (float*)scratch(l.cx, 1, (size_t)N * sizeof(float));
    float* out = (float*)scratch(l.cx, 2, (size_t)N * C * sizeof(float));
    float* ones = (float*)scratch(l.cx, 3, (size_t)C * sizeof(float));
    if (!rstd || !out || !ones) return nullptr;
    fill_kernel<<<(C + 255) / 256, 256, 0, l.st>>>(ones, 1.0f, (size_t)C);
    if (rmsnorm_forward<float>(out, rstd, x, ones, N, C, eps, l.st)) return nullptr;
    return rstd;
}
// slots 0 gout, 1 w, 2 x, 3 gx (+=), 4 params {N, C}, 5 eps
int k_rmsnorm_backward_x(const Launch& l) {
    const int *p = ip(l, 4), N = p[0], C = p[1];
    const float* rstd = row_rstd(l, fp(l, 2), N, C, *fp(l, 5));
    float* gw_unused = (float*)scratch(l.cx, 4, (size_t)C * sizeof(float));
    float* part = (float*)scratch(l.cx, 5, rmsnorm_backward_scratch_floats(C) * sizeof(float));
    if (!rstd || !gw_unused || !part) return -1;
    return rmsnorm_backward<float>(fpw(l, 3), gw_unused, 0, fp(l, 0), fp(l, 2), fp(l, 1), rstd, N, C, 0, 0, part, l.st);
}
// slots 0 gout, 1 x, 2 gw [C] (overwritten: src/kernels/backward.metal:400), 3 params {N, C}, 4 eps
int k_rmsnorm_backward_w(const Launch& l) {
    const int *p = ip(l, 3), N = p[0], C = p[1];
    const float* rstd = row_rstd(l, fp(l, 1), N, C, *fp(l, 4));
    float* gx_unused = (float*)scratch(l.cx, 2, (size_t)N * C * sizeof(float));  // the discarded forward output is done with
    float* ones = (float*)scratch(l.cx, 3, (size_t)C * sizeof(float));
    float* part = (float*)scratch(l.cx, 5, rmsnorm_backward_scratch_floats(C) * sizeof(float));
    if (!rstd || !gx_unused || !ones || !part) return -1;
    return rmsnorm_backward<float>(gx_unused, fpw(l, 2), 0, fp(l, 0), fp(l, 1), ones, rstd, N, C, 0, N, part, l.st);
}

// ---- RoPE: params {HD, NKV, S, NH}; rope {theta, factor, low, high, orig_max, llama3_flag} (src/baremetal/graph.c:99-107) ------------
const float* rope_table(const Launch& l, const int* p, const float* r) {
    const int HD = p[0], S = p[2];
    char key[160];
    snprintf(key, sizeof key, "%d/%d/%a/%a/%a/%a/%a/%a", HD, S, r[0], r[1], r[2], r[3], r[4], r[5]);
    auto it = l.cx->rope_tables.find(key);
    if (it != l.cx->rope_tables.end()) return it->second;
    float* h = bm_build_rope_table(r[0], r[5] != 0.f ? 1 : 0, r[1], r[2], r[3], r[4], S, HD);
    float* d = nullptr;
    const size_t bytes = (size_t)S * (HD / 2) * 2 * sizeof(float);
    if (!h || cudaMalloc(&d, bytes) != cudaSuccess) { free(h); return nullptr; }
    cudaMemcpyAsync(d, h, bytes, cudaMemcpyHostToDevice, l.st);
    cudaStreamSynchronize(l.st);
    free(h);
    l.cx->rope_tables[key] = d;
    return d;
}
// slots 0 q [S,NH,HD], 1 k [S,NKV,HD], 2 params, 3 rope; in place
int k_rope_forward_seq(const Launch& l) {
    const int *p = ip(l, 2), HD = p[0], NKV = p[1], S = p[2], NH = p[3];
    const float* t = rope_table(l, p, fp(l, 3));
    if (!t) return -1;
    return rope_apply<float>(fpw(l, 0), NH * HD, fpw(l, 1), NKV * HD, t, S, S, NH, NKV, HD, +1, l.st);
}
// slots 0 gout_q, 1 gout_k, 2 gq, 3 gk, 4 params, 5 rope (the scheduler binds 0 == 2 and 1 == 3, src/baremetal/scheduler.c:1567-1571)
int k_rope_backward_seq(const Launch& l) {
    const int *p = ip(l, 4), HD = p[0], NKV = p[1], S = p[2], NH = p[3];
    const float* t = rope_table(l, p, fp(l, 5));
    if (!t) return -1;
    if (l.b[2] != l.b[0]) cudaMemcpyAsync(l.b[2], l.b[0], (size_t)S * NH * HD * sizeof(float), cudaMemcpyDeviceToDevice, l.st);
    if (l.b[3] != l.b[1]) cudaMemcpyAsync(l.b[3], l.b[1], (size_t)S * NKV * HD * sizeof(float), cudaMemcpyDeviceToDevice, l.st);
    return rope_apply<float>(fpw(l, 2), NH * HD, fpw(l, 3), NKV * HD, t, S, S, NH, NKV, HD, -1, l.st);
}

// ---- attention: params {NH, S, HD, NKV, kv_mul, masked}; one sequence per dispatch ---------------------------------------------
// slots 0 Q, 1 K, 2 V, 3 out, 4 params, 5 scale, 6 mask uchar[S]
int k_attention_forward(const Launch& l) {
    const int *p = ip(l, 4), NH = p[0], S = p[1], HD = p[2], NKV = p[3];
    const uint8_t* mask = (p[5] && l.nb > 6) ? (const uint8_t*)l.b[6] : nullptr;
    float* lse = (float*)scratch(l.cx, 1, (size_t)NH * S * sizeof(float));
    if (!lse) return -1;
    return attention_forward_simt<float>(fpw(l, 3), NH * HD, lse, fp(l, 0), NH * HD, fp(l, 1), fp(l, 2), NKV * HD, mask, 1, S, NH, NKV, HD,
                                         *fp(l, 5), l.st);
}
// slots 0 gout, 1 Q, 2 K, 3 V, 4 gQ (=), 5 gK (+=, atomics), 6 gV (+=), 7 params, 8 scale, 9 mask. The reference recomputes the
// probabilities from Q and K; the kernel here wants the forward's output and log-sum-exp, so a forward pass into scratch comes first.
int k_attention_backward(const Launch& l) {
    const int *p = ip(l, 7), NH = p[0], S = p[1], HD = p[2], NKV = p[3];
    const uint8_t* mask = (p[5] && l.nb > 9) ? (const uint8_t*)l.b[9] : nullptr;
    float* lse = (float*)scratch(l.cx, 1, (size_t)NH * S * sizeof(float));
    float* out = (float*)scratch(l.cx, 2, (size_t)S * NH * HD * sizeof(float));
    if (!lse || !out) return -1;
    const float scale = *fp(l, 8);
    int rc = attention_forward_simt<float>(out, NH * HD, lse, fp(l, 1), NH * HD, fp(l, 2), fp(l, 3), NKV * HD, mask, 1, S, NH, NKV, HD, scale, l.st);
    if (rc) return rc;
    return attention_backward_simt<float>(fpw(l, 4), NH * HD, fpw(l, 5), fpw(l, 6), NKV * HD, fp(l, 0), NH * HD, out, lse, fp(l, 1), NH * HD,
                                          fp(l, 2), fp(l, 3), NKV * HD, mask, 1, S, NH, NKV, HD, scale, l.st);
}

// ---- element-wise -------------------------------------------------------------------------------------------------------------
int k_add_forward(const Launch& l) { return add_forward<float>(fpw(l, 2), fp(l, 0), fp(l, 1), (size_t)*ip(l, 3), l.st); }
// slots 0 gout, 1 gx (+=), 2 gy (+=), 3 N
int k_add_backward(const Launch& l) {
    const size_t n = (size_t)*ip(l, 3);
    int rc = add_forward<float>(fpw(l, 1), fp(l, 1), fp(l, 0), n, l.st);
    if (!rc) rc = add_forward<float>(fpw(l, 2), fp(l, 2), fp(l, 0), n, l.st);
    return rc;
}
// slots 0 gate, 1 up, 2 out, 3 N
int k_swiglu_forward(const Launch& l) {
    const int n = *ip(l, 3);
    if (swiglu_forward<float>(fpw(l, 2), n, fp(l, 0), fp(l, 1), n, 1, n, l.st) == 0) return 0;
    swiglu_forward_any_kernel<<<(n + 255) / 256, 256, 0, l.st>>>(fpw(l, 2), fp(l, 0), fp(l, 1), n);
    return 0;
}
// slots 0 gate, 1 up, 2 gout, 3 ggate (=), 4 gup (=), 5 N
int k_swiglu_backward(const Launch& l) {
    const int n = *ip(l, 5);
    if (swiglu_backward<float>(fpw(l, 3), fpw(l, 4), n, fp(l, 0), fp(l, 1), n, fp(l, 2), n, 1, n, l.st) == 0) return 0;
    swiglu_backward_any_kernel<<<(n + 255) / 256, 256, 0, l.st>>>(fpw(l, 3), fpw(l, 4), fp(l, 0), fp(l, 1), fp(l, 2), n);
    return 0;
}
// slots 0 p (bound with a byte offset), 1 n
int k_zero_buffer(const Launch& l) {
    const size_t n = (size_t)*ip(l, 1);
    if (n * sizeof(float) > l.bytes[0]) return -1;
    return cudaMemsetAsync(l.b[0], 0, n * sizeof(float), l.st) == cudaSuccess ? 0 : -1;
}

// ---- loss, embedding, optimizer -------------------------------------------------------------------------------------------------
// slots 0 logits [N,V], 1 targets, 2 glogits (=), 3 params {N, V}: (softmax - onehot) / N
int k_xent_backward(const Launch& l) {
    const int *p = ip(l, 3), N = p[0], V = p[1];
    float* row_loss = (float*)scratch(l.cx, 1, (size_t)N * sizeof(float));
    if (!row_loss) return -1;
    if (V % 4) {
        xent_any_kernel<<<N, 128, 0, l.st>>>(fpw(l, 2), fp(l, 0), ip(l, 1), nullptr, V, 1.0f / (float)N, l.cx->d_err);
        return 0;
    }
    if (l.b[2] != l.b[0]) cudaMemcpyAsync(l.b[2], l.b[0], (size_t)N * V * sizeof(float), cudaMemcpyDeviceToDevice, l.st);
    return xent_forward_backward<float>(fpw(l, 2), row_loss, ip(l, 1), nullptr, N, V, V, 1.0f / (float)N, l.cx->d_err, l.st);
}
// slots 0 logits, 1 targets, 2 glogits, 3 mask uchar[N], 4 params {N, V, count}: masked rows get a zero gradient, the others / count
int k_xent_backward_masked(const Launch& l) {
    const int *p = ip(l, 4), N = p[0], V = p[1], count = p[2];
    float* row_loss = (float*)scratch(l.cx, 1, (size_t)N * sizeof(float));
    float* weights = (float*)scratch(l.cx, 4, (size_t)N * sizeof(float));
    if (!row_loss || !weights) return -1;
    mask_weights_kernel<<<(N + 255) / 256, 256, 0, l.st>>>(weights, (const unsigned char*)l.b[3], N, count > 0 ? 1.0f / (float)count : 0.f);
    if (V % 4) {
        xent_any_kernel<<<N, 128, 0, l.st>>>(fpw(l, 2), fp(l, 0), ip(l, 1), weights, V, 0.f, l.cx->d_err);
        return 0;
    }
    if (l.b[2] != l.b[0]) cudaMemcpyAsync(l.b[2], l.b[0], (size_t)N * V * sizeof(float), cudaMemcpyDeviceToDevice, l.st);
    return xent_forward_backward<float>(fpw(l, 2), row_loss, ip(l, 1), weights, N, V, V, 0.f, l.cx->d_err, l.st);
}
// slots 0 tokens [T], 1 gout [T,D], 2 gwte [V,D] (+=, atomics), 3 D; grid = T * D
int k_embedding_backward(const Launch& l) {
    const int D = *ip(l, 3);
    if (D <= 0 || l.grid % D) return -1;
    const int T = (int)(l.grid / D), V = (int)(l.bytes[2] / ((size_t)D * sizeof(float)));
    if (embedding_backward_f32(fpw(l, 2), fp(l, 1), ip(l, 0), T, D, V, l.cx->d_err, l.st) == 0) return 0;
    embedding_backward_any_kernel<<<(int)((l.grid + 255) / 256), 256, 0, l.st>>>(fpw(l, 2), fp(l, 1), ip(l, 0), T, D, V, l.cx->d_err);
    return 0;
}
// slots 0 w, 1 g, 2 m, 3 v, 4 N, 5 hp {lr, b1, b2, eps, wd, 1-b1^t, 1-b2^t, 1/n_micro}
int k_adamw_step(const Launch& l) {
    const int n = *ip(l, 4);
    const float* hp = fp(l, 5);
    if (adamw_f32grad(fpw(l, 0), nullptr, fp(l, 1), fpw(l, 2), fpw(l, 3), (size_t)n, hp, l.st) == 0) return 0;
    adamw_any_kernel<<<(n + 255) / 256, 256, 0, l.st>>>(fpw(l, 0), fp(l, 1), fpw(l, 2), fpw(l, 3), n, hp[0], hp[1], hp[2], hp[3], hp[4], hp[5], hp[6],
                                                        hp[7]);
    return 0;
}

const std::map<std::string, KernelEntry>& kernel_table() {
    static const std::map<std::string, KernelEntry> t = {
        {"matmul_forward_naive", {k_mm_forward_f32, 5}},          {"matmul_forward_fp32_tiled", {k_mm_forward_f32, 5}},
        {"matmul_forward_bf16", {k_mm_forward_bf16, 5}},          {"matmul_forward_bf16_tiled", {k_mm_forward_bf16, 5}},
        {"matmul_forward_bf16_tiled64", {k_mm_forward_bf16, 5}},  {"matmul_backward_inp", {k_mm_backward_inp_f32, 4}},
        {"matmul_backward_inp_fp32_tiled", {k_mm_backward_inp_f32, 4}}, {"matmul_backward_inp_bf16", {k_mm_backward_inp_bf16, 4}},
        {"matmul_backward_inp_bf16_tiled", {k_mm_backward_inp_bf16, 4}}, {"matmul_backward_w", {k_mm_backward_w, 4}},
        {"matmul_backward_w_tiled", {k_mm_backward_w, 4}},        {"rmsnorm_forward", {k_rmsnorm_forward, 5}},
        {"rmsnorm_backward_x", {k_rmsnorm_backward_x, 6}},        {"rmsnorm_backward_w", {k_rmsnorm_backward_w, 5}},
        {"rope_forward_seq", {k_rope_forward_seq, 4}},            {"rope_backward_seq", {k_rope_backward_seq, 6}},
        {"attention_forward_seq", {k_attention_forward, 6}},      {"attention_forward_seq_masked", {k_attention_forward, 7}},
        {"attention_forward_train_tiled", {k_attention_forward, 6}}, {"attention_backward", {k_attention_backward, 9}},
        {"attention_backward_masked", {k_attention_backward, 10}}, {"attention_backward_tiled", {k_attention_backward, 9}},
        {"add_forward", {k_add_forward, 4}},                      {"add_backward", {k_add_backward, 4}},
        {"swiglu_forward", {k_swiglu_forward, 4}},                {"swiglu_backward", {k_swiglu_backward, 6}},
        {"zero_buffer", {k_zero_buffer, 2}},                      {"xent_backward", {k_xent_backward, 4}},
        {"xent_backward_masked", {k_xent_backward_masked, 5}},    {"embedding_backward", {k_embedding_backward, 4}},
        {"adamw_step", {k_adamw_step, 6}},
    };
    return t;
}

int enqueue(Compat* cx, backend_kernel_t* k, backend_buffer_t* buffers[], size_t offsets[], int nb, long grid) {
    if (!cx || !k || !k->pipeline_state || !buffers || nb < 0 || nb > 16) return -1;
    const KernelEntry* e = (const KernelEntry*)k->pipeline_state;
    if (nb < e->min_slots) return -1;
    void* ptrs[16] = {nullptr};
    size_t bytes[16] = {0};
    for (int i = 0; i < nb; ++i) {
        if (!buffers[i]) continue;
        const size_t off = offsets ? offsets[i] : 0;
        if (off > buffers[i]->size) return -1;
        ptrs[i] = (char*)buffers[i]->buffer + off;
        bytes[i] = buffers[i]->size - off;
    }
    for (int i = 0; i < e->min_slots; ++i)
        if (!ptrs[i] && !(i == 2 && e->fn == k_mm_forward_f32) && !(i == 2 && e->fn == k_mm_forward_bf16)) return -1;  // the bias slot may be empty
    Launch l{ptrs, bytes, nb, grid, cx->st, cx};
    const int rc = e->fn(l);
    if (rc) return -1;
    return cudaPeekAtLastError() == cudaSuccess ? 0 : -1;
}

struct EncoderState { cudaEvent_t t0, t1; int committed; };

}  // namespace

extern "C" {

backend_ctx_t* backend_create(void) {
    int n = 0, dev = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n <= 0) {
        fprintf(stderr, "backend_create: no CUDA device; this backend has no CPU fallback\n");
        return nullptr;
    }
    const char* e = getenv("BM_DEVICE_ORDINAL");
    if (e && e[0]) dev = atoi(e);
    if (dev < 0 || dev >= n || cudaSetDevice(dev) != cudaSuccess) return nullptr;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) return nullptr;
    Compat* cx = new Compat();
    memset(&cx->pub, 0, sizeof cx->pub);
    for (int i = 0; i < 6; ++i) { cx->scratch[i] = nullptr; cx->scratch_bytes[i] = 0; }
    if (cudaStreamCreateWithFlags(&cx->st, cudaStreamNonBlocking) != cudaSuccess || cudaMalloc(&cx->d_err, sizeof(int)) != cudaSuccess) {
        delete cx;
        return nullptr;
    }
    cudaMemset(cx->d_err, 0, sizeof(int));
    cx->pub.device = cx;
    cx->pub.supports_bf16 = 1;
    cx->pub.dev_max_threads_per_tg = prop.maxThreadsPerBlock;
    cx->pub.dev_max_threadgroup_mem = prop.sharedMemPerBlockOptin;
    cx->pub.dev_max_buffer_bytes = prop.totalGlobalMem;
    cx->pub.dev_recommended_working_set = prop.totalGlobalMem;
    cx->pub.dev_has_unified_memory = 0;
    return &cx->pub;
}
void backend_destroy(backend_ctx_t* ctx) {
    if (!ctx) return;
    Compat* cx = (Compat*)ctx;
    cudaStreamSynchronize(cx->st);
    for (int i = 0; i < 6; ++i) cudaFree(cx->scratch[i]);
    for (auto& kv : cx->rope_tables) cudaFree(kv.second);
    cudaFree(cx->d_err);
    cudaStreamDestroy(cx->st);
    delete cx;
}
size_t backend_get_allocated_memory(backend_ctx_t* ctx) { return ctx ? ctx->allocated_bytes : 0; }
size_t backend_get_peak_allocated_memory(backend_ctx_t* ctx) { return ctx ? ctx->peak_allocated_bytes : 0; }
void backend_get_device_info(backend_ctx_t* ctx, backend_device_info_t* out) {
    if (!ctx || !out) return;
    out->max_threads_per_threadgroup = ctx->dev_max_threads_per_tg;
    out->max_threadgroup_memory = ctx->dev_max_threadgroup_mem;
    out->max_buffer_bytes = ctx->dev_max_buffer_bytes;
    out->recommended_max_working_set = ctx->dev_recommended_working_set;
    out->has_unified_memory = ctx->dev_has_unified_memory;
}
double backend_get_gpu_busy_ms(backend_ctx_t* ctx) { return ctx ? ctx->gpu_busy_ms : 0.0; }
uint64_t backend_get_command_buffers(backend_ctx_t* ctx) { return ctx ? ctx->cmd_buffers : 0; }
void backend_reset_gpu_timing(backend_ctx_t* ctx) {
    if (ctx) { ctx->gpu_busy_ms = 0.0; ctx->cmd_buffers = 0; }
}

backend_buffer_t* backend_buffer_alloc(backend_ctx_t* ctx, size_t size) {
    if (!ctx || size == 0) return nullptr;   // size 0 -> NULL, as src/backend/metal/device.m:117
    backend_buffer_t* b = (backend_buffer_t*)calloc(1, sizeof *b);
    if (!b) return nullptr;
    if (cudaMallocManaged(&b->buffer, size, cudaMemAttachGlobal) != cudaSuccess) {
        cudaGetLastError();
        free(b);
        return nullptr;
    }
    memset(b->buffer, 0, size);   // fresh shared-storage buffers read as zero
    b->size = size;
    b->ctx = ctx;
    ctx->allocated_bytes += size;
    if (ctx->allocated_bytes > ctx->peak_allocated_bytes) ctx->peak_allocated_bytes = ctx->allocated_bytes;
    return b;
}
void backend_buffer_free(backend_buffer_t* b) {
    if (!b) return;
    if (b->ctx) {
        cudaStreamSynchronize(((Compat*)b->ctx)->st);
        b->ctx->allocated_bytes -= b->size;
    }
    cudaFree(b->buffer);
    free(b);
}
void* backend_buffer_map(backend_buffer_t* b) {
    if (!b) return nullptr;
    if (b->ctx) cudaStreamSynchronize(((Compat*)b->ctx)->st);   // everything enqueued so far is visible to the host
    return b->buffer;
}
void backend_buffer_unmap(backend_buffer_t*) {}
size_t backend_buffer_size(backend_buffer_t* b) { return b ? b->size : 0; }

backend_kernel_t* backend_kernel_create(backend_ctx_t* ctx, const char* name) {
    if (!ctx || !name) return nullptr;
    auto it = kernel_table().find(name);
    if (it == kernel_table().end()) return nullptr;
    backend_kernel_t* k = (backend_kernel_t*)calloc(1, sizeof *k);
    if (k) k->pipeline_state = (void*)&it->second;
    return k;
}
void backend_kernel_destroy(backend_kernel_t* k) { free(k); }

int backend_kernel_dispatch(backend_ctx_t* ctx, backend_kernel_t* k, backend_buffer_t* buffers[], size_t offsets[], int nb, int gx, int gy,
                            int gz, int, int, int) {
    if (!ctx) return -1;
    Compat* cx = (Compat*)ctx;
    cudaEvent_t t0, t1;
    cudaEventCreate(&t0);
    cudaEventCreate(&t1);
    cudaEventRecord(t0, cx->st);
    const int rc = enqueue(cx, k, buffers, offsets, nb, (long)gx * gy * gz);
    cudaEventRecord(t1, cx->st);
    const cudaError_t se = cudaStreamSynchronize(cx->st);   // blocking, like the reference's one-kernel command buffer
    float ms = 0.f;
    cudaEventElapsedTime(&ms, t0, t1);
    cudaEventDestroy(t0);
    cudaEventDestroy(t1);
    ctx->gpu_busy_ms += ms;
    ctx->cmd_buffers += 1;
    return (rc == 0 && se == cudaSuccess) ? 0 : -1;
}
void backend_synchronize(backend_ctx_t* ctx) {
    if (ctx) cudaStreamSynchronize(((Compat*)ctx)->st);
}

backend_encoder_t* backend_encode_begin(backend_ctx_t* ctx) {
    if (!ctx) return nullptr;
    backend_encoder_t* enc = (backend_encoder_t*)calloc(1, sizeof *enc);
    EncoderState* s = (EncoderState*)calloc(1, sizeof *s);
    if (!enc || !s) { free(enc); free(s); return nullptr; }
    cudaEventCreate(&s->t0);
    cudaEventCreate(&s->t1);
    cudaEventRecord(s->t0, ((Compat*)ctx)->st);
    enc->command_buffer = s;
    enc->ctx = ctx;
    return enc;
}
int backend_encode_dispatch(backend_encoder_t* enc, backend_kernel_t* k, backend_buffer_t* buffers[], size_t offsets[], int nb, int gx,
                            int gy, int gz, int, int, int) {
    if (!enc) return -1;
    return enqueue((Compat*)enc->ctx, k, buffers, offsets, nb, (long)gx * gy * gz);
}
void backend_encode_commit(backend_encoder_t* enc) {
    if (!enc) return;
    EncoderState* s = (EncoderState*)enc->command_buffer;
    if (!s->committed) cudaEventRecord(s->t1, ((Compat*)enc->ctx)->st);
    s->committed = 1;
}
double backend_encode_wait_timed(backend_encoder_t* enc) {
    if (!enc) return 0.0;
    EncoderState* s = (EncoderState*)enc->command_buffer;
    Compat* cx = (Compat*)enc->ctx;
    if (!s->committed) cudaEventRecord(s->t1, cx->st);   // a wait without a commit still ends the encoder
    cudaStreamSynchronize(cx->st);
    float ms = 0.f;
    cudaEventElapsedTime(&ms, s->t0, s->t1);
    enc->ctx->gpu_busy_ms += ms;
    enc->ctx->cmd_buffers += 1;
    cudaEventDestroy(s->t0);
    cudaEventDestroy(s->t1);
    free(s);
    free(enc);
    return ms;
}
void backend_encode_wait(backend_encoder_t* enc) { (void)backend_encode_wait_timed(enc); }

}  // extern "C"
