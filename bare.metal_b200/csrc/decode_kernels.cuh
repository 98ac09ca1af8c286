// Launchers of the inference (decode) kernels, see decode_kernels.cu.
#pragma once
#include "common.cuh"

namespace bmb {
// wtype: 0 = Q8 (w = int8 q[OC][C], scales = float[OC][C/32]), 1 = bf16, 2 = fp32. out[b, oc] = x[b,:] . w[oc,:] (+ res[b, oc])
int decode_gemv(float* out, int ldo, const float* x, int ldx, int wtype, const void* w, const float* scales, const float* res, int ldr,
                int NB, int C, int OC, cudaStream_t st);
int decode_rmsnorm(float* out, const float* x, const float* w, int NB, int C, float eps, cudaStream_t st);
int decode_rope_kv(float* qkv, float* cache, const float* cs, const int* pos, int layer, int NB, int MS, int NH, int NKV, int HD,
                   cudaStream_t st);
int decode_attention(float* out, const float* qkv, const float* cache, const int* pos, int layer, int NB, int MS, int NH, int NKV, int HD,
                     float scale, cudaStream_t st);
int decode_swiglu(float* out, const float* gu, int NB, int H, cudaStream_t st);
int decode_embed(float* out, int ttype, const void* table, const int* tokens, int NB, int D, cudaStream_t st);
int decode_argmax(int* out, const float* logits, int NB, int V, cudaStream_t st);
int decode_advance(int* pos, cudaStream_t st);
}  // namespace bmb
