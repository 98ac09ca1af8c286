// Launchers of the inference (decode) kernels, see decode_kernels.cu.
#pragma once
#include "common.cuh"

namespace bmb {
// wtype: 0 = Q8 (w = int8 q[OC][C], scales = float[OC][C/32]), 1 = bf16, 2 = fp32, 3 = Q4 (w = uint8 [OC][C/2], element 2j in the low
// and 2j+1 in the high nibble of byte j, scales as Q8). out[b, oc] = x[b,:] . w[oc,:] (+ res[b, oc])
// prologue: 0 = none, 1 = RMSNorm(x) * lnw folded in, 2 = x is [gate | up] (2C wide) and the operand is silu(gate) * up
int decode_gemv(float* out, int ldo, const float* x, int ldx, int wtype, const void* w, const float* scales, const float* res, int ldr,
                int prologue, const float* lnw, float eps, int NB, int C, int OC, cudaStream_t st);
int decode_rmsnorm(float* out, const float* x, const float* w, int NB, int C, float eps, cudaStream_t st);
int decode_rope_kv(float* qkv, void* cache, int cache_bf16, const float* cs, const int* pos, int layer, int NB, int MS, int NH, int NKV, int HD,
                   cudaStream_t st);
// cs != null: q and k are rotated and k, v stored into the cache inside the kernel (qkv holds the raw projections).
// The cache holds fp32 (cache_bf16 = 0, the reference's layout) or bf16 elements (head_dim 64 only).
// scratch: null (one block walks all positions) or a zero-initialised buffer of decode_attention_scratch_bytes() + 16 bytes, which
// lets the positions be split over several blocks per (sequence, KV head)
size_t decode_attention_scratch_bytes(int NB, int MS, int NH, int NKV, int HD);
int decode_attention(float* out, const float* qkv, void* cache, int cache_bf16, const float* cs, const int* pos, void* scratch, int layer, int NB, int MS,
                     int NH, int NKV, int HD, float scale, cudaStream_t st);
// Tensor-core path operand: a[row] = [hi | lo] (parts 2) or [hi | lo | hi] (parts 3) bf16 split of the fp32 operand row
// (mode 0 = x, 1 = RMSNorm(x) * lnw, 2 = silu(gate) * up of a [gate | up] row); init_out rows (n_out wide) are set to
// init_src rows, or zero.
int decode_prep(bf16* a, int parts, const float* x, int ldx, int mode, const float* lnw, float eps, float* init_out, int ldo,
                const float* init_src, int ldr, int n_out, int rows, int C, cudaStream_t st);
// prefill: cache[layer][0|1][b][t][:] = k | v columns of row b * T + t of the packed [q | k | v] matrix
int decode_kv_scatter(void* cache, int cache_bf16, const float* qkv, int ldqkv, int layer, int NB, int T, int MS, int QD, int KV, cudaStream_t st);
int decode_swiglu(float* out, const float* gu, int NB, int H, cudaStream_t st);
int decode_embed(float* out, int ttype, const void* table, const int* tokens, int NB, int D, cudaStream_t st);
int decode_argmax(int* out, const float* logits, int NB, int V, int* pos_to_advance, cudaStream_t st);
int decode_advance(int* pos, cudaStream_t st);
}  // namespace bmb
