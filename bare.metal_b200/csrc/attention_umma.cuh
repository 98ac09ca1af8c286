// bf16 causal GQA flash attention on the tcgen05 tensor cores, forward and backward, head_dim 64 (attention_umma.cu).
#pragma once
#include "common.cuh"

namespace bmb {

// Shapes the tensor-core kernels take: head_dim 64, query heads a multiple of the KV heads.
bool flash_attention_supported(int HD, int NH, int NKV);

// out[row, h, :] = softmax(scale * Q K^T, causal) V ; lse[b, h, s] = log sum exp of the scaled scores.
// err_flag (device int, may be null) receives a non-zero code if a bounded wait inside the kernel ran out.
// keymask (may be null): padding mask as bits, [B][ceil(S / 32)] words from flash_attention_pack_mask: a position whose bit is 0 is
// neither key nor query (zero output row, +infinity log-sum-exp).
size_t flash_attention_mask_bits_bytes(int B, int S);
int flash_attention_pack_mask(uint32_t* bits, const uint8_t* mask, int B, int S, cudaStream_t st);
int flash_attention_forward_umma(bf16* out, int ldo, float* lse, const bf16* q, int ldq, const bf16* k, const bf16* v, int ldkv,
                                 const uint32_t* keymask, int B, int S, int NH, int NKV, int HD, float scale, int* err_flag, cudaStream_t st);

// Scratch: fp32 dQ accumulators [B*S, NH*HD] followed by delta[B, NH, S].
size_t flash_attention_backward_scratch_bytes(int B, int S, int NH, int HD);
// delta_in (may be null): precomputed rowsum(gout * out) as [B, NH, S]; null = computed here into the scratch.
// rope_cs (may be null): [S][HD/2][cos, sin]; when given, gq and gk leave with RoPE backward already applied.
int flash_attention_backward_umma(bf16* gq, int ldgq, bf16* gk, bf16* gv, int ldgkv, const bf16* gout, int ldo, const bf16* out,
                                  const float* lse, const bf16* q, int ldq, const bf16* k, const bf16* v, int ldkv, int B, int S, int NH,
                                  int NKV, int HD, float scale, void* scratch, const float* delta_in, const float* rope_cs,
                                  const uint32_t* keymask, int* err_flag, cudaStream_t st);

// Causal GQA attention for the inference session's prefill: fp32 in, fp32 out, fp32-accurate on the tensor pipe (each fp32 operand
// is split into bf16 hi + lo and each product is three tcgen05 products). Replaces attention_forward_prefill_tiled
// (src/kernels/forward.metal:2024). q [NB*T, ldq], k / v [NB*T, ldkv], out [NB*T, ldo]; head_dim 64.
size_t prefill_attention_umma_scratch_bytes(long rows, int NH, int NKV);
int prefill_attention_umma(float* out, int ldo, const float* q, int ldq, const float* k, const float* v, int ldkv, int NB, int T, int NH, int NKV,
                           int HD, float scale, void* scratch, int* err_flag, cudaStream_t st);

// out[r, 0:cols] (bf16, pitch ldo) = in[r, 0:cols] (fp32, pitch ldi)
int cast_rows_f32_to_bf16(bf16* out, int ldo, const float* in, int ldi, int rows, int cols, cudaStream_t st);

}  // namespace bmb
