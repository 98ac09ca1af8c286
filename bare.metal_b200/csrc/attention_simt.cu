// Causal GQA attention with exact fp32 softmax arithmetic on the CUDA cores: the fp32 parity mode's
// attention, and the on-device cross-check for the tensor-core flash kernels. One warp per
// (batch, head, query); lanes stride over the keys with a private online softmax that is merged
// across the warp at the end, which equals the reference's whole-row softmax
// (attention_forward_seq src/kernels/forward.metal:1811, attention_backward src/kernels/backward.metal:665,
// masked variants forward.metal:1853 / backward.metal:738) up to fp32 rounding.
// Layout as the reference: Q[row, h, :], K/V[row, kh, :] with row = b*S + s and kh = h / (NH/NKV).
#include "kernels.cuh"

namespace bmb {

namespace {
constexpr int AW = 4;  // warps per block

template <typename T, int HD>
__global__ void __launch_bounds__(AW * 32)
attn_fwd_simt_kernel(T* __restrict__ out, int ldo, float* __restrict__ lse, const T* __restrict__ q, int ldq, const T* __restrict__ k,
                     const T* __restrict__ v, int ldkv, const uint8_t* __restrict__ mask, int B, int S, int NH, int NKV, float scale) {
    __shared__ float sq[AW][HD];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long wid = (long)blockIdx.x * AW + warp;
    if (wid >= (long)B * NH * S) return;
    const int i = (int)(wid % S);
    const int h = (int)((wid / S) % NH);
    const int b = (int)(wid / ((long)S * NH));
    const int kh = h / (NH / NKV);
    const size_t row_i = (size_t)b * S + i;
    const T* qi = q + row_i * ldq + (size_t)h * HD;
    for (int d = lane; d < HD; d += 32) sq[warp][d] = to_f32(qi[d]);
    __syncwarp();

    float m = -INFINITY, l = 0.f, acc[HD];
#pragma unroll
    for (int d = 0; d < HD; ++d) acc[d] = 0.f;
    const bool q_on = !mask || mask[row_i];
    if (q_on) {
        for (int j = lane; j <= i; j += 32) {
            const size_t row_j = (size_t)b * S + j;
            if (mask && !mask[row_j]) continue;
            const T* kj = k + row_j * ldkv + (size_t)kh * HD;
            const T* vj = v + row_j * ldkv + (size_t)kh * HD;
            float s = 0.f;
#pragma unroll
            for (int d = 0; d < HD; ++d) s += sq[warp][d] * to_f32(kj[d]);
            s *= scale;
            const float mn = fmaxf(m, s);
            const float corr = expf(m - mn), p = expf(s - mn);
            l = l * corr + p;
#pragma unroll
            for (int d = 0; d < HD; ++d) acc[d] = acc[d] * corr + p * to_f32(vj[d]);
            m = mn;
        }
    }
    const float mall = warp_max(m);
    const float w = (m == -INFINITY) ? 0.f : expf(m - mall);
    const float lall = warp_sum(l * w);
    const float inv = lall > 0.f ? 1.0f / lall : 0.f;
    T* oi = out + row_i * ldo + (size_t)h * HD;
#pragma unroll
    for (int d = 0; d < HD; ++d) {
        const float o = warp_sum(acc[d] * w) * inv;
        if (lane == (d & 31)) oi[d] = from_f32<T>(o);
    }
    if (lane == 0 && lse) lse[((size_t)b * NH + h) * S + i] = lall > 0.f ? mall + logf(lall) : -INFINITY;
}

template <typename T, int HD>
__global__ void __launch_bounds__(AW * 32)
attn_bwd_simt_kernel(float* __restrict__ gq, int ldgq, float* __restrict__ gk, float* __restrict__ gv, int ldgkv,
                     const T* __restrict__ gout, int ldo, const T* __restrict__ out, const float* __restrict__ lse,
                     const T* __restrict__ q, int ldq, const T* __restrict__ k, const T* __restrict__ v, int ldkv,
                     const uint8_t* __restrict__ mask, int B, int S, int NH, int NKV, float scale) {
    __shared__ float sq[AW][HD];
    __shared__ float sg[AW][HD];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long wid = (long)blockIdx.x * AW + warp;
    if (wid >= (long)B * NH * S) return;
    const int i = (int)(wid % S);
    const int h = (int)((wid / S) % NH);
    const int b = (int)(wid / ((long)S * NH));
    const int kh = h / (NH / NKV);
    const size_t row_i = (size_t)b * S + i;
    const T* qi = q + row_i * ldq + (size_t)h * HD;
    const T* gi = gout + row_i * ldo + (size_t)h * HD;
    const T* oi = out + row_i * ldo + (size_t)h * HD;
    float dpart = 0.f;
    for (int d = lane; d < HD; d += 32) {
        sq[warp][d] = to_f32(qi[d]);
        sg[warp][d] = to_f32(gi[d]);
        dpart += to_f32(gi[d]) * to_f32(oi[d]);
    }
    const float delta = warp_sum(dpart);  // = sum_j p_j (gout . V_j)
    __syncwarp();
    const float L = lse[((size_t)b * NH + h) * S + i];
    float gqa[HD];
#pragma unroll
    for (int d = 0; d < HD; ++d) gqa[d] = 0.f;
    const bool q_on = (!mask || mask[row_i]) && L != -INFINITY;
    if (q_on) {
        for (int j = lane; j <= i; j += 32) {
            const size_t row_j = (size_t)b * S + j;
            if (mask && !mask[row_j]) continue;
            const T* kj = k + row_j * ldkv + (size_t)kh * HD;
            const T* vj = v + row_j * ldkv + (size_t)kh * HD;
            float s = 0.f, gp = 0.f;
#pragma unroll
            for (int d = 0; d < HD; ++d) {
                s += sq[warp][d] * to_f32(kj[d]);
                gp += sg[warp][d] * to_f32(vj[d]);
            }
            const float p = expf(s * scale - L);
            const float gs = p * (gp - delta);
            float* gkj = gk + row_j * ldgkv + (size_t)kh * HD;
            float* gvj = gv + row_j * ldgkv + (size_t)kh * HD;
#pragma unroll
            for (int d = 0; d < HD; ++d) {
                gqa[d] += gs * to_f32(kj[d]);
                atomicAdd(gkj + d, scale * gs * sq[warp][d]);
                atomicAdd(gvj + d, p * sg[warp][d]);
            }
        }
    }
    float* gqi = gq + row_i * ldgq + (size_t)h * HD;
#pragma unroll
    for (int d = 0; d < HD; ++d) {
        const float t = warp_sum(gqa[d]) * scale;
        if (lane == (d & 31)) gqi[d] = t;
    }
}

}  // namespace

template <typename T>
int attention_forward_simt(T* out, int ldo, float* lse, const T* q, int ldq, const T* k, const T* v, int ldkv, const uint8_t* mask,
                           int B, int S, int NH, int NKV, int HD, float scale, cudaStream_t st) {
    if (NKV <= 0 || NH % NKV) return -1;
    const long warps = (long)B * NH * S;
    const int grid = (int)((warps + AW - 1) / AW);
#define BMB_CASE(H) \
    case H: attn_fwd_simt_kernel<T, H><<<grid, AW * 32, 0, st>>>(out, ldo, lse, q, ldq, k, v, ldkv, mask, B, S, NH, NKV, scale); return 0;
    switch (HD) {
        BMB_CASE(4) BMB_CASE(8) BMB_CASE(16) BMB_CASE(32) BMB_CASE(64) BMB_CASE(128)
    }
#undef BMB_CASE
    return -2;
}
template <typename T>
int attention_backward_simt(float* gq, int ldgq, float* gk, float* gv, int ldgkv, const T* gout, int ldo, const T* out,
                            const float* lse, const T* q, int ldq, const T* k, const T* v, int ldkv, const uint8_t* mask, int B,
                            int S, int NH, int NKV, int HD, float scale, cudaStream_t st) {
    if (NKV <= 0 || NH % NKV) return -1;
    const long warps = (long)B * NH * S;
    const int grid = (int)((warps + AW - 1) / AW);
#define BMB_CASE(H)                                                                                                          \
    case H:                                                                                                                  \
        attn_bwd_simt_kernel<T, H><<<grid, AW * 32, 0, st>>>(gq, ldgq, gk, gv, ldgkv, gout, ldo, out, lse, q, ldq, k, v, ldkv, \
                                                              mask, B, S, NH, NKV, scale);                                   \
        return 0;
    switch (HD) {
        BMB_CASE(4) BMB_CASE(8) BMB_CASE(16) BMB_CASE(32) BMB_CASE(64) BMB_CASE(128)
    }
#undef BMB_CASE
    return -2;
}
template int attention_forward_simt<float>(float*, int, float*, const float*, int, const float*, const float*, int, const uint8_t*,
                                           int, int, int, int, int, float, cudaStream_t);
template int attention_forward_simt<bf16>(bf16*, int, float*, const bf16*, int, const bf16*, const bf16*, int, const uint8_t*, int,
                                          int, int, int, int, float, cudaStream_t);
template int attention_backward_simt<float>(float*, int, float*, float*, int, const float*, int, const float*, const float*,
                                            const float*, int, const float*, const float*, int, const uint8_t*, int, int, int, int,
                                            int, float, cudaStream_t);
template int attention_backward_simt<bf16>(float*, int, float*, float*, int, const bf16*, int, const bf16*, const float*,
                                           const bf16*, int, const bf16*, const bf16*, int, const uint8_t*, int, int, int, int, int,
                                           float, cudaStream_t);

}  // namespace bmb
