// C++ launchers of the hand-written kernels behind the C ABI (include/bm_cuda_backend.h).
// T is the activation type: float (fp32 parity mode) or bf16 (mixed-precision mode).
// Every launcher enqueues on `st` and returns 0 or a negative code for an unsupported shape.
#pragma once
#include "common.cuh"

namespace bmb {

// ---- memory-bound kernels (kernels_mem.cu) ---------------------------------------------------
// Codes a kernel leaves in the context's error word (read by bmc_status) instead of using an id that is out of range as an index.
constexpr int BMB_ERR_BAD_TOKEN = 2001;   // embedding gather / scatter met a token id outside [0, V)
constexpr int BMB_ERR_BAD_TARGET = 2002;  // cross-entropy met a target id outside [0, V) on a row that counts
template <typename T> int embedding_forward(T* out, const float* table, const int* tokens, int n_tok, int D, int V, int* err, cudaStream_t st);
int embedding_backward_f32(float* gwte, const float* gout, const int* tokens, int n_tok, int D, int V, int* err, cudaStream_t st);
int embedding_backward_bf16(float* gwte, const bf16* gout, const int* tokens, int n_tok, int D, int V, int* err, cudaStream_t st);

template <typename T> int rmsnorm_forward(T* out, float* rstd, const T* x, const float* w, int N, int C, float eps, cudaStream_t st);
// gx += d(rmsnorm)/dx ; gw (+)= sum over rows [w_row0, w_row1) of gout * x * rstd.
// `scratch` holds rmsnorm_backward_scratch_floats(C) floats.
size_t rmsnorm_backward_scratch_floats(int C);
template <typename T> int rmsnorm_backward(T* gx, float* gw, int gw_accumulate, const T* gout, const T* x, const float* w,
                                           const float* rstd, int N, int C, int w_row0, int w_row1, float* scratch,
                                           cudaStream_t st);

// cs_table: [S][HD/2][2] = (cos, sin) of pos * inv_freq. dir = +1 forward, -1 backward. In place.
template <typename T> int rope_apply(T* q, int ldq, T* k, int ldk, const float* cs_table, int rows, int S, int NH, int NKV,
                                     int HD, int dir, cudaStream_t st);

template <typename T> int swiglu_forward(T* out, int ldo, const T* gate, const T* up, int ldgu, int rows, int H, cudaStream_t st);
template <typename T> int swiglu_backward(T* ggate, T* gup, int ldg, const T* gate, const T* up, int ldgu, const T* gout, int ldo,
                                          int rows, int H, cudaStream_t st);
template <typename T> int add_forward(T* out, const T* a, const T* b, size_t n, cudaStream_t st);

// logits -> (softmax - onehot) * grad_scale in place; row_loss[n] = -log softmax[target].
// row_weight (may be null): per-row gradient scale replacing grad_scale; 0 = masked row (zero gradient, zero loss). With
// row weights the stored row loss is already weighted.
template <typename T> int xent_forward_backward(T* logits, float* row_loss, const int* targets, const float* row_weight, int N, int V,
                                                int ldv, float grad_scale, int* err, cudaStream_t st);
// loss = (1/B) sum_b (1/S) sum_s row_loss   (weighted != 0: the rows are already weighted, so no 1/S)
int loss_reduce(float* out, const float* row_loss, int B, int S, int weighted, cudaStream_t st);

// hp (HOST pointer) = {lr, b1, b2, eps, wd, 1-b1^t, 1-b2^t, grad_scale}
int adamw_f32grad(float* w, bf16* w_bf16, const float* g, float* m, float* v, size_t n, const float* hp, cudaStream_t st);
int adamw_bf16grad(float* w, bf16* w_bf16, const bf16* g, float* m, float* v, size_t n, const float* hp, cudaStream_t st);
int cast_f32_to_bf16(bf16* out, const float* in, size_t n, cudaStream_t st);
int cast_bf16_to_f32(float* out, const bf16* in, size_t n, cudaStream_t st);
template <typename T> int seq_prefix_accumulate(T* x, float* carry, int B, size_t per_seq, cudaStream_t st);
int argmax_first(int* out_index, const float* logits, int V, cudaStream_t st);

// ---- fp32-accumulating SIMT GEMM for the fp32 parity mode (gemm_simt.cu) -------------------------
// C[m,n] (+)= sum_k A(m,k) B(n,k) [+ R[m,n]],  A(m,k) at A[m*sam + k*sak], B(n,k) at B[n*sbn + k*sbk].
int gemm_f32_simt(float* C, int ldc, int accumulate, const float* A, long sam, long sak, const float* B, long sbn, long sbk,
                  const float* R, int ldr, int M, int N, int K, cudaStream_t st);

// ---- attention (attention_simt.cu: exact-softmax fp32 math, masks, any head_dim; the bf16 tensor-core kernels are in attention_umma.cuh) ----
// Layout as the reference: Q[row, h, :] at q + row*ldq + h*HD (row = b*S + s), K/V with NKV heads, causal, GQA.
template <typename T> int attention_forward_simt(T* out, int ldo, float* lse, const T* q, int ldq, const T* k, const T* v, int ldkv,
                                                 const uint8_t* mask, int B, int S, int NH, int NKV, int HD, float scale,
                                                 cudaStream_t st);
// gk/gv must be zero on entry (fp32 accumulators, row pitch ldgkv); gq is overwritten.
template <typename T> int attention_backward_simt(float* gq, int ldgq, float* gk, float* gv, int ldgkv, const T* gout, int ldo,
                                                  const T* out, const float* lse, const T* q, int ldq, const T* k, const T* v,
                                                  int ldkv, const uint8_t* mask, int B, int S, int NH, int NKV, int HD,
                                                  float scale, cudaStream_t st);

}  // namespace bmb
