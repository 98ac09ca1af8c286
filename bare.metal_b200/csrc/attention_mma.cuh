// bf16 causal GQA flash attention, forward and backward, head_dim 64.
#pragma once
#include "common.cuh"

namespace bmb {

bool flash_attention_supported(int HD, int NH, int NKV, bool has_mask);

// out[row, h, :] = softmax(scale * Q K^T, causal) V ; lse[b, h, s] = log sum exp of the scaled scores.
int flash_attention_forward(bf16* out, int ldo, float* lse, const bf16* q, int ldq, const bf16* k, const bf16* v, int ldkv, int B, int S,
                            int NH, int NKV, int HD, float scale, cudaStream_t st);

// Same contract, tcgen05/TMEM/TMA implementation (attention_umma.cu). err_flag (device int, may be null) receives a
// non-zero code if a bounded wait inside the kernel ran out.
int flash_attention_forward_umma(bf16* out, int ldo, float* lse, const bf16* q, int ldq, const bf16* k, const bf16* v, int ldkv, int B,
                                 int S, int NH, int NKV, int HD, float scale, int* err_flag, cudaStream_t st);

// Scratch: fp32 dQ accumulators [B*S, NH*HD] followed by delta[B, NH, S].
size_t flash_attention_backward_scratch_bytes(int B, int S, int NH, int HD);
int flash_attention_backward(bf16* gq, int ldgq, bf16* gk, bf16* gv, int ldgkv, const bf16* gout, int ldo, const bf16* out,
                             const float* lse, const bf16* q, int ldq, const bf16* k, const bf16* v, int ldkv, int B, int S, int NH,
                             int NKV, int HD, float scale, void* scratch, cudaStream_t st);

// tcgen05/TMEM/TMA implementation of the backward (attention_umma.cu); same scratch layout as flash_attention_backward.
int flash_attention_backward_umma(bf16* gq, int ldgq, bf16* gk, bf16* gv, int ldgkv, const bf16* gout, int ldo, const bf16* out,
                                  const float* lse, const bf16* q, int ldq, const bf16* k, const bf16* v, int ldkv, int B, int S, int NH,
                                  int NKV, int HD, float scale, void* scratch, int* err_flag, cudaStream_t st);

// out[r, 0:cols] (bf16, pitch ldo) = in[r, 0:cols] (fp32, pitch ldi)
int cast_rows_f32_to_bf16(bf16* out, int ldo, const float* in, int ldi, int rows, int cols, cudaStream_t st);

}  // namespace bmb
