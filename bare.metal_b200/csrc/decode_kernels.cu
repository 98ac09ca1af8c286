// Kernels of the token-by-token inference path (Q8 / bf16 / fp32 weights, fp32 activations, fp32 KV cache), batched over
// independent sequences. Arithmetic follows the reference's decode kernels; every launcher enqueues on the given stream.
//   decode_gemv      matmul_forward_q8_vec / _bf16_vec / naive (src/kernels/forward.metal:575,52,23) — out = x W^T (+ residual)
//   decode_rmsnorm   rmsnorm_forward_v2 (forward.metal:1019)
//   decode_rope_kv   rope_forward (forward.metal:1284) + kv_store (forward.metal:1317)
//   decode_attention attention_forward (forward.metal:1362): one query against the cache, softmax over positions 0..pos
//   decode_swiglu    swiglu_forward (forward.metal:1179)
//   decode_embed     the host-side row gather of bm_step (src/baremetal/session.c:151-185)
//   decode_argmax    bm_sample's greedy branch (src/baremetal/sampler.c:36-40), one row per sequence
// Q8 weights keep the reference's values (int8 q, fp32 scale per 32, src/baremetal/quant.h:19-22) but are stored as two
// arrays — q[OC][C] and scale[OC][C/32] — so rows can be read with aligned 16-byte loads.
#include "decode_kernels.cuh"

namespace bmb {

namespace {

constexpr int GEMV_WARPS = 8;
constexpr int GEMV_TB = 8;    // sequences per pass in the batched kernel
constexpr int GEMV_ROWS = 8;  // output rows per warp in the batched kernel

__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// four int8 -> (float)q * scale, exactly as the reference's dequantisation (forward.metal:610), without the
// conversion unit: the byte, biased by 128, is placed in the mantissa of 2^23 and the bias subtracted again.
__device__ __forceinline__ void dequant4(uint32_t pk, float s, float* w) {
    const uint32_t u = pk ^ 0x80808080u;
    w[0] = (__uint_as_float(__byte_perm(u, 0x4B000000u, 0x7540)) - 8388736.0f) * s;
    w[1] = (__uint_as_float(__byte_perm(u, 0x4B000000u, 0x7541)) - 8388736.0f) * s;
    w[2] = (__uint_as_float(__byte_perm(u, 0x4B000000u, 0x7542)) - 8388736.0f) * s;
    w[3] = (__uint_as_float(__byte_perm(u, 0x4B000000u, 0x7543)) - 8388736.0f) * s;
}

// WT: 0 = Q8 (q + scales), 1 = bf16, 2 = fp32. Elements one lane reads with one 16-byte load:
template <int WT> struct Epl { static constexpr int v = WT == 0 ? 16 : (WT == 1 ? 8 : 4); };

template <int WT>
__device__ __forceinline__ void load_weights16(const void* w, const float* scales, size_t row, int C, int c, float* wv) {
    if (WT == 0) {
        const uint4 pk = *reinterpret_cast<const uint4*>((const int8_t*)w + row * C + c);
        const float s = scales[row * (C / 32) + (c >> 5)];
        dequant4(pk.x, s, wv); dequant4(pk.y, s, wv + 4); dequant4(pk.z, s, wv + 8); dequant4(pk.w, s, wv + 12);
    } else if (WT == 1) {
        const uint4 pk = *reinterpret_cast<const uint4*>((const bf16*)w + row * C + c);
        wv[0] = __uint_as_float(pk.x << 16); wv[1] = __uint_as_float(pk.x & 0xffff0000u);
        wv[2] = __uint_as_float(pk.y << 16); wv[3] = __uint_as_float(pk.y & 0xffff0000u);
        wv[4] = __uint_as_float(pk.z << 16); wv[5] = __uint_as_float(pk.z & 0xffff0000u);
        wv[6] = __uint_as_float(pk.w << 16); wv[7] = __uint_as_float(pk.w & 0xffff0000u);
    } else {
        const float4 v = *reinterpret_cast<const float4*>((const float*)w + row * C + c);
        wv[0] = v.x; wv[1] = v.y; wv[2] = v.z; wv[3] = v.w;
    }
}

// Single sequence (or a few, one after the other): one warp per output row; the activation row lives in registers
// (CH chunks of 32 lanes x EPL columns), so the loop touches only the weight stream. Two rows are in flight per warp.
template <int WT, int CH>
__global__ void __launch_bounds__(GEMV_WARPS * 32)
decode_gemv1_kernel(float* __restrict__ out, int ldo, const float* __restrict__ x, int ldx, const void* __restrict__ w,
                    const float* __restrict__ scales, const float* __restrict__ res, int ldr, int C, int OC) {
    constexpr int EPL = Epl<WT>::v;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b = blockIdx.y;
    float xr[CH * EPL];
#pragma unroll
    for (int j = 0; j < CH; ++j) {
        const int c = (j * 32 + lane) * EPL;
#pragma unroll
        for (int i = 0; i < EPL; i += 4) {
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (c < C) v = *reinterpret_cast<const float4*>(x + (size_t)b * ldx + c + i);
            xr[j * EPL + i] = v.x; xr[j * EPL + i + 1] = v.y; xr[j * EPL + i + 2] = v.z; xr[j * EPL + i + 3] = v.w;
        }
    }
    const int stride = gridDim.x * GEMV_WARPS;
    for (int oc = blockIdx.x * GEMV_WARPS + warp; oc < OC; oc += 2 * stride) {
        const int oc1 = oc + stride;
        const bool two = oc1 < OC;
        float a0 = 0.f, a1 = 0.f;
#pragma unroll
        for (int j = 0; j < CH; ++j) {
            const int c = (j * 32 + lane) * EPL;
            if (c < C) {
                float w0[EPL], w1[EPL];
                load_weights16<WT>(w, scales, (size_t)oc, C, c, w0);
                load_weights16<WT>(w, scales, (size_t)(two ? oc1 : oc), C, c, w1);
#pragma unroll
                for (int i = 0; i < EPL; ++i) {
                    a0 = fmaf(xr[j * EPL + i], w0[i], a0);
                    a1 = fmaf(xr[j * EPL + i], w1[i], a1);
                }
            }
        }
        a0 = warp_sum_f(a0);
        a1 = warp_sum_f(a1);
        if (lane == 0) {
            out[(size_t)b * ldo + oc] = a0 + (res ? res[(size_t)b * ldr + oc] : 0.f);
            if (two) out[(size_t)b * ldo + oc1] = a1 + (res ? res[(size_t)b * ldr + oc1] : 0.f);
        }
    }
}

// Several sequences: a warp owns GEMV_ROWS output rows and GEMV_TB sequences; a lane owns 4 columns of every
// 128-column chunk. Activations of the batch tile sit in shared memory and are read as consecutive float4 (no bank
// conflicts); each weight is dequantised once and used GEMV_TB times.
template <int WT>
__global__ void __launch_bounds__(GEMV_WARPS * 32)
decode_gemvb_kernel(float* __restrict__ out, int ldo, const float* __restrict__ x, int ldx, const void* __restrict__ w,
                    const float* __restrict__ scales, const float* __restrict__ res, int ldr, int NB, int C, int OC) {
    extern __shared__ float sx[];  // [GEMV_TB][C]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b0 = blockIdx.y * GEMV_TB;
    const int nb = min(GEMV_TB, NB - b0);
    for (int i = threadIdx.x * 4; i < GEMV_TB * C; i += blockDim.x * 4) {
        const int b = i / C, c = i - b * C;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (b < nb) v = *reinterpret_cast<const float4*>(x + (size_t)(b0 + b) * ldx + c);
        *reinterpret_cast<float4*>(sx + i) = v;
    }
    __syncthreads();
    for (int r0 = (blockIdx.x * GEMV_WARPS + warp) * GEMV_ROWS; r0 < OC; r0 += gridDim.x * GEMV_WARPS * GEMV_ROWS) {
        float acc[GEMV_ROWS][GEMV_TB];
#pragma unroll
        for (int r = 0; r < GEMV_ROWS; ++r)
#pragma unroll
            for (int b = 0; b < GEMV_TB; ++b) acc[r][b] = 0.f;
        for (int c = lane * 4; c < C; c += 128) {
            float wv[GEMV_ROWS][4];
#pragma unroll
            for (int r = 0; r < GEMV_ROWS; ++r) {
                const size_t row = (size_t)min(r0 + r, OC - 1);
                if (WT == 0) {
                    const uint32_t pk = *reinterpret_cast<const uint32_t*>((const int8_t*)w + row * C + c);
                    dequant4(pk, scales[row * (C / 32) + (c >> 5)], wv[r]);
                } else if (WT == 1) {
                    const uint2 pk = *reinterpret_cast<const uint2*>((const bf16*)w + row * C + c);
                    wv[r][0] = __uint_as_float(pk.x << 16); wv[r][1] = __uint_as_float(pk.x & 0xffff0000u);
                    wv[r][2] = __uint_as_float(pk.y << 16); wv[r][3] = __uint_as_float(pk.y & 0xffff0000u);
                } else {
                    const float4 v = *reinterpret_cast<const float4*>((const float*)w + row * C + c);
                    wv[r][0] = v.x; wv[r][1] = v.y; wv[r][2] = v.z; wv[r][3] = v.w;
                }
            }
#pragma unroll
            for (int b = 0; b < GEMV_TB; ++b) {
                const float4 xv = *reinterpret_cast<const float4*>(sx + b * C + c);
#pragma unroll
                for (int r = 0; r < GEMV_ROWS; ++r) {
                    acc[r][b] = fmaf(xv.x, wv[r][0], acc[r][b]);
                    acc[r][b] = fmaf(xv.y, wv[r][1], acc[r][b]);
                    acc[r][b] = fmaf(xv.z, wv[r][2], acc[r][b]);
                    acc[r][b] = fmaf(xv.w, wv[r][3], acc[r][b]);
                }
            }
        }
#pragma unroll
        for (int r = 0; r < GEMV_ROWS; ++r)
#pragma unroll
            for (int b = 0; b < GEMV_TB; ++b) {
                const float t = warp_sum_f(acc[r][b]);
                if (lane == 0 && b < nb && r0 + r < OC) {
                    const int oc = r0 + r;
                    out[(size_t)(b0 + b) * ldo + oc] = t + (res ? res[(size_t)(b0 + b) * ldr + oc] : 0.f);
                }
            }
    }
}

__global__ void decode_rmsnorm_kernel(float* __restrict__ out, const float* __restrict__ x, const float* __restrict__ w, int C, float eps) {
    __shared__ float red[32];
    const float* xr = x + (size_t)blockIdx.x * C;
    float ss = 0.f;
    for (int i = threadIdx.x; i < C; i += blockDim.x) ss += xr[i] * xr[i];
    ss = warp_sum_f(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x < 32) {
        float t = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
        t = warp_sum_f(t);
        if (threadIdx.x == 0) red[0] = t;
    }
    __syncthreads();
    const float inv = 1.0f / sqrtf(red[0] / (float)C + eps);
    for (int i = threadIdx.x; i < C; i += blockDim.x) out[(size_t)blockIdx.x * C + i] = xr[i] * inv * w[i];
}

// RoPE on this token's q and k at position *pos, then k and v into the cache. qkv: [NB][QD + 2 KV].
// cache: [L][2][NB][MS][KV] fp32. cs: [MS][HD/2][2].
__global__ void decode_rope_kv_kernel(float* __restrict__ qkv, float* __restrict__ cache, const float* __restrict__ cs,
                                      const int* __restrict__ pos_ptr, int layer, int NB, int MS, int NH, int NKV, int HD) {
    const int b = blockIdx.x;
    const int pos = *pos_ptr;
    const int QD = NH * HD, KV = NKV * HD, hd2 = HD / 2;
    float* row = qkv + (size_t)b * (QD + 2 * KV);
    for (int i = threadIdx.x; i < (NH + NKV) * hd2; i += blockDim.x) {
        const int h = i / hd2, p = i - h * hd2;
        float* base = row + h * HD;  // q heads then k heads are contiguous in the packed row
        const float c = cs[((size_t)pos * hd2 + p) * 2], s = cs[((size_t)pos * hd2 + p) * 2 + 1];
        const float x0 = base[p], x1 = base[p + hd2];
        base[p] = x0 * c - x1 * s;
        base[p + hd2] = x0 * s + x1 * c;
    }
    __syncthreads();
    float* kc = cache + (((size_t)layer * 2 + 0) * NB + b) * (size_t)MS * KV + (size_t)pos * KV;
    float* vc = cache + (((size_t)layer * 2 + 1) * NB + b) * (size_t)MS * KV + (size_t)pos * KV;
    for (int i = threadIdx.x; i < KV; i += blockDim.x) {
        kc[i] = row[QD + i];
        vc[i] = row[QD + KV + i];
    }
}

// One block (256 threads) per (KV head, sequence); it serves the MUL query heads that share the KV head, so every cache
// row is read once. Phase 1: 8 lanes per position read one K row (coalesced) and form the MUL scaled scores.
// Phase 2: softmax statistics per head over positions 0..pos. Phase 3: 16 (HD 64) position groups accumulate p * V with
// float4 reads of the V rows; the groups are then summed through shared memory.
constexpr int ATT_THREADS = 256;
template <int HD, int MUL>
__global__ void __launch_bounds__(ATT_THREADS)
decode_attention_kernel(float* __restrict__ out, const float* __restrict__ qkv, const float* __restrict__ cache,
                        const int* __restrict__ pos_ptr, int layer, int NB, int MS, int NH, int NKV, float scale) {
    extern __shared__ float sm[];
    constexpr int EPL = HD / 8;             // K floats per lane in phase 1
    constexpr int D4 = HD / 4;              // float4 per V row
    constexpr int GROUPS = ATT_THREADS / D4;
    const int kh = blockIdx.x, b = blockIdx.y, tid = threadIdx.x;
    const int n = *pos_ptr + 1;
    const int QD = NH * HD, KV = NKV * HD;
    float* sc = sm;                                    // [MUL][MS]
    float* red = sm + (size_t)MUL * MS;                // [MUL][GROUPS][HD] (phase 3) / [MUL][8] (phase 2)
    const float* kc = cache + (((size_t)layer * 2 + 0) * NB + b) * (size_t)MS * KV + (size_t)kh * HD;
    const float* vc = cache + (((size_t)layer * 2 + 1) * NB + b) * (size_t)MS * KV + (size_t)kh * HD;
    const float* qrow = qkv + (size_t)b * (QD + 2 * KV) + (size_t)kh * MUL * HD;

    // phase 1
    const int sub = tid & 7, slot = tid >> 3;          // 32 positions per block iteration
    float qr[MUL][EPL];
#pragma unroll
    for (int h = 0; h < MUL; ++h)
#pragma unroll
        for (int i = 0; i < EPL; i += 4) {
            const float4 v = *reinterpret_cast<const float4*>(qrow + h * HD + sub * EPL + i);
            qr[h][i] = v.x; qr[h][i + 1] = v.y; qr[h][i + 2] = v.z; qr[h][i + 3] = v.w;
        }
    float mx[MUL];
#pragma unroll
    for (int h = 0; h < MUL; ++h) mx[h] = -INFINITY;
    for (int t0 = 0; t0 < n; t0 += ATT_THREADS / 8) {
        const int t = t0 + slot;
        float s[MUL];
#pragma unroll
        for (int h = 0; h < MUL; ++h) s[h] = 0.f;
        if (t < n) {
            const float* kt = kc + (size_t)t * KV + sub * EPL;
#pragma unroll
            for (int i = 0; i < EPL; i += 4) {
                const float4 kv = *reinterpret_cast<const float4*>(kt + i);
#pragma unroll
                for (int h = 0; h < MUL; ++h)
                    s[h] = fmaf(qr[h][i], kv.x, fmaf(qr[h][i + 1], kv.y, fmaf(qr[h][i + 2], kv.z, fmaf(qr[h][i + 3], kv.w, s[h]))));
            }
        }
#pragma unroll
        for (int h = 0; h < MUL; ++h) {
            float v = s[h];
            v += __shfl_xor_sync(0xffffffffu, v, 1);
            v += __shfl_xor_sync(0xffffffffu, v, 2);
            v += __shfl_xor_sync(0xffffffffu, v, 4);
            v *= scale;
            if (t < n) {
                if (sub == 0) sc[(size_t)h * MS + t] = v;
                mx[h] = fmaxf(mx[h], v);
            }
        }
    }
    // phase 2
#pragma unroll
    for (int h = 0; h < MUL; ++h) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], o));
        if ((tid & 31) == 0) red[h * 8 + (tid >> 5)] = mx[h];
    }
    __syncthreads();
    float inv[MUL];
#pragma unroll
    for (int h = 0; h < MUL; ++h) {
        float m = red[h * 8];
#pragma unroll
        for (int i = 1; i < 8; ++i) m = fmaxf(m, red[h * 8 + i]);
        mx[h] = m;
    }
    __syncthreads();
#pragma unroll
    for (int h = 0; h < MUL; ++h) {
        float sum = 0.f;
        for (int t = tid; t < n; t += ATT_THREADS) {
            const float e = expf(sc[(size_t)h * MS + t] - mx[h]);
            sc[(size_t)h * MS + t] = e;
            sum += e;
        }
        sum = warp_sum_f(sum);
        if ((tid & 31) == 0) red[h * 8 + (tid >> 5)] = sum;
    }
    __syncthreads();
#pragma unroll
    for (int h = 0; h < MUL; ++h) {
        float t = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) t += red[h * 8 + i];
        inv[h] = 1.0f / t;
    }
    __syncthreads();
    // phase 3
    const int d4 = tid % D4, grp = tid / D4;
    float4 acc[MUL];
#pragma unroll
    for (int h = 0; h < MUL; ++h) acc[h] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int t = grp; t < n; t += GROUPS) {
        const float4 v = *reinterpret_cast<const float4*>(vc + (size_t)t * KV + d4 * 4);
#pragma unroll
        for (int h = 0; h < MUL; ++h) {
            const float p = sc[(size_t)h * MS + t];
            acc[h].x = fmaf(p, v.x, acc[h].x); acc[h].y = fmaf(p, v.y, acc[h].y);
            acc[h].z = fmaf(p, v.z, acc[h].z); acc[h].w = fmaf(p, v.w, acc[h].w);
        }
    }
#pragma unroll
    for (int h = 0; h < MUL; ++h) *reinterpret_cast<float4*>(red + ((size_t)h * GROUPS + grp) * HD + d4 * 4) = acc[h];
    __syncthreads();
    for (int i = tid; i < MUL * HD; i += ATT_THREADS) {
        const int h = i / HD, d = i - h * HD;
        float t = 0.f;
#pragma unroll
        for (int g = 0; g < GROUPS; ++g) t += red[((size_t)h * GROUPS + g) * HD + d];
        float iv = inv[0];
#pragma unroll
        for (int hh = 1; hh < MUL; ++hh) iv = (h == hh) ? inv[hh] : iv;
        out[(size_t)b * QD + (size_t)(kh * MUL + h) * HD + d] = t * iv;
    }
}

__global__ void decode_swiglu_kernel(float* __restrict__ out, const float* __restrict__ gu, int H, int NB) {
    const long i = blockIdx.x * (long)blockDim.x + threadIdx.x;
    if (i >= (long)NB * H) return;
    const int b = (int)(i / H), c = (int)(i - (long)b * H);
    const float g = gu[(size_t)b * 2 * H + c], u = gu[(size_t)b * 2 * H + H + c];
    out[i] = g / (1.0f + expf(-g)) * u;
}

template <typename TT>
__global__ void decode_embed_kernel(float* __restrict__ out, const TT* __restrict__ table, const int* __restrict__ tokens, int D, int NB) {
    const long i = blockIdx.x * (long)blockDim.x + threadIdx.x;
    if (i >= (long)NB * D) return;
    const int b = (int)(i / D), c = (int)(i - (long)b * D);
    out[i] = to_f32(table[(size_t)tokens[b] * D + c]);
}

__global__ void decode_argmax_kernel(int* __restrict__ out, const float* __restrict__ logits, int V) {
    __shared__ float sv[32];
    __shared__ int si[32];
    const float* lr = logits + (size_t)blockIdx.x * V;
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float x = lr[i];
        if (x > best || (x == best && i < bi)) { best = x; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x < 32) {
        best = threadIdx.x < (blockDim.x >> 5) ? sv[threadIdx.x] : -INFINITY;
        bi = threadIdx.x < (blockDim.x >> 5) ? si[threadIdx.x] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
        }
        if (threadIdx.x == 0) out[blockIdx.x] = bi == 0x7fffffff ? 0 : bi;
    }
}

__global__ void decode_advance_kernel(int* pos) { *pos += 1; }

}  // namespace

template <int WT, int CH>
static void launch_gemv1(float* out, int ldo, const float* x, int ldx, const void* w, const float* scales, const float* res, int ldr,
                         int NB, int C, int OC, cudaStream_t st) {
    int gx = (OC + GEMV_WARPS - 1) / GEMV_WARPS;
    if (gx > 148 * 4) gx = 148 * 4;
    decode_gemv1_kernel<WT, CH><<<dim3(gx, NB), GEMV_WARPS * 32, 0, st>>>(out, ldo, x, ldx, w, scales, res, ldr, C, OC);
}
template <int WT>
static int gemv_dispatch(float* out, int ldo, const float* x, int ldx, const void* w, const float* scales, const float* res, int ldr,
                         int NB, int C, int OC, cudaStream_t st) {
    constexpr int EPL = Epl<WT>::v;
    const int chunks = (C + 32 * EPL - 1) / (32 * EPL);
    const int max_regs_chunks = 96 / EPL;  // at most 96 activation registers per lane
    if (NB < 4 && chunks <= max_regs_chunks) {
        if (chunks * EPL <= 32) launch_gemv1<WT, 32 / EPL>(out, ldo, x, ldx, w, scales, res, ldr, NB, C, OC, st);
        else if (chunks * EPL <= 48) launch_gemv1<WT, 48 / EPL>(out, ldo, x, ldx, w, scales, res, ldr, NB, C, OC, st);
        else if (chunks * EPL <= 80) launch_gemv1<WT, 80 / EPL>(out, ldo, x, ldx, w, scales, res, ldr, NB, C, OC, st);
        else launch_gemv1<WT, 96 / EPL>(out, ldo, x, ldx, w, scales, res, ldr, NB, C, OC, st);
        return 0;
    }
    const size_t smem = (size_t)GEMV_TB * C * sizeof(float);
    if (smem > 200 * 1024) return -2;
    static bool attr_done = false;
    if (!attr_done) {
        cudaFuncSetAttribute(decode_gemvb_kernel<WT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        attr_done = true;
    }
    const int rows_per_block = GEMV_WARPS * GEMV_ROWS;
    int gx = (OC + rows_per_block - 1) / rows_per_block;
    if (gx > 148 * 4) gx = 148 * 4;
    decode_gemvb_kernel<WT><<<dim3(gx, (NB + GEMV_TB - 1) / GEMV_TB), GEMV_WARPS * 32, smem, st>>>(out, ldo, x, ldx, w, scales, res, ldr, NB, C, OC);
    return 0;
}

// x rows must be 16-byte aligned (ldx % 4 == 0); C % 32 == 0.
int decode_gemv(float* out, int ldo, const float* x, int ldx, int wtype, const void* w, const float* scales, const float* res, int ldr,
                int NB, int C, int OC, cudaStream_t st) {
    if (C % 32 || NB <= 0 || (ldx & 3)) return -1;
    if (wtype == 0) return gemv_dispatch<0>(out, ldo, x, ldx, w, scales, res, ldr, NB, C, OC, st);
    if (wtype == 1) return gemv_dispatch<1>(out, ldo, x, ldx, w, scales, res, ldr, NB, C, OC, st);
    return gemv_dispatch<2>(out, ldo, x, ldx, w, scales, res, ldr, NB, C, OC, st);
}
int decode_rmsnorm(float* out, const float* x, const float* w, int NB, int C, float eps, cudaStream_t st) {
    decode_rmsnorm_kernel<<<NB, 256, 0, st>>>(out, x, w, C, eps);
    return 0;
}
int decode_rope_kv(float* qkv, float* cache, const float* cs, const int* pos, int layer, int NB, int MS, int NH, int NKV, int HD,
                   cudaStream_t st) {
    decode_rope_kv_kernel<<<NB, 256, 0, st>>>(qkv, cache, cs, pos, layer, NB, MS, NH, NKV, HD);
    return 0;
}
template <int HD, int MUL>
static int launch_attention(float* out, const float* qkv, const float* cache, const int* pos, int layer, int NB, int MS, int NH, int NKV,
                            float scale, cudaStream_t st) {
    const size_t smem = ((size_t)MUL * MS + (size_t)MUL * (ATT_THREADS / (HD / 4)) * HD) * sizeof(float);
    static size_t attr_smem = 48 * 1024;
    if (smem > attr_smem) {
        if (smem > 220 * 1024) return -2;
        cudaFuncSetAttribute(decode_attention_kernel<HD, MUL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        attr_smem = smem;
    }
    decode_attention_kernel<HD, MUL><<<dim3(NKV, NB), ATT_THREADS, smem, st>>>(out, qkv, cache, pos, layer, NB, MS, NH, NKV, scale);
    return 0;
}
// head_dim 64 or 128; 1, 2, 3, 4 or 8 query heads per KV head
int decode_attention(float* out, const float* qkv, const float* cache, const int* pos, int layer, int NB, int MS, int NH, int NKV, int HD,
                     float scale, cudaStream_t st) {
    if (NKV <= 0 || NH % NKV) return -1;
    const int mul = NH / NKV;
#define BM_ATT_CASE(hd, m) if (HD == hd && mul == m) return launch_attention<hd, m>(out, qkv, cache, pos, layer, NB, MS, NH, NKV, scale, st);
    BM_ATT_CASE(64, 1) BM_ATT_CASE(64, 2) BM_ATT_CASE(64, 3) BM_ATT_CASE(64, 4) BM_ATT_CASE(64, 8)
    BM_ATT_CASE(128, 1) BM_ATT_CASE(128, 2) BM_ATT_CASE(128, 4) BM_ATT_CASE(128, 8)
#undef BM_ATT_CASE
    return -3;
}
int decode_swiglu(float* out, const float* gu, int NB, int H, cudaStream_t st) {
    const long n = (long)NB * H;
    decode_swiglu_kernel<<<(int)((n + 255) / 256), 256, 0, st>>>(out, gu, H, NB);
    return 0;
}
int decode_embed(float* out, int ttype, const void* table, const int* tokens, int NB, int D, cudaStream_t st) {
    const long n = (long)NB * D;
    if (ttype == 1) decode_embed_kernel<bf16><<<(int)((n + 255) / 256), 256, 0, st>>>(out, (const bf16*)table, tokens, D, NB);
    else decode_embed_kernel<float><<<(int)((n + 255) / 256), 256, 0, st>>>(out, (const float*)table, tokens, D, NB);
    return 0;
}
int decode_argmax(int* out, const float* logits, int NB, int V, cudaStream_t st) {
    decode_argmax_kernel<<<NB, 1024, 0, st>>>(out, logits, V);
    return 0;
}
int decode_advance(int* pos, cudaStream_t st) {
    decode_advance_kernel<<<1, 1, 0, st>>>(pos);
    return 0;
}

}  // namespace bmb
