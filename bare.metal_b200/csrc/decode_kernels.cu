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

#include <cstdlib>

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

// Programmatic dependent launch: a kernel launched with the stream-serialisation attribute may start while its
// predecessor is still running; pdl_wait() blocks until the predecessor has completed and its writes are visible.
// Everything before pdl_wait() may only touch memory no kernel of the step writes (weights, earlier cache rows).
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// four int8 -> (float)q * scale, exactly as the reference's dequantisation (forward.metal:610), without the
// conversion unit: the byte, biased by 128, is placed in the mantissa of 2^23 and the bias subtracted again.
__device__ __forceinline__ void dequant4(uint32_t pk, float s, float* w) {
    const uint32_t u = pk ^ 0x80808080u;
    w[0] = (__uint_as_float(__byte_perm(u, 0x4B000000u, 0x7540)) - 8388736.0f) * s;
    w[1] = (__uint_as_float(__byte_perm(u, 0x4B000000u, 0x7541)) - 8388736.0f) * s;
    w[2] = (__uint_as_float(__byte_perm(u, 0x4B000000u, 0x7542)) - 8388736.0f) * s;
    w[3] = (__uint_as_float(__byte_perm(u, 0x4B000000u, 0x7543)) - 8388736.0f) * s;
}

// eight 4-bit codes of one 32-bit word -> (float)q * scale, q = the nibble read as a two's-complement number in [-8, 7]
// (matmul_forward_q4, src/kernels/forward.metal:849-854: element 2j is the low and 2j+1 the high nibble of byte j, so
// element i of a little-endian word is bits [4i, 4i+4)). nibble ^ 8 = q + 8, placed in the mantissa of 2^23.
__device__ __forceinline__ void dequant8_nibbles(uint32_t pk, float s, float* w) {
#pragma unroll
    for (int i = 0; i < 8; ++i) w[i] = (__uint_as_float(((pk >> (4 * i)) & 0xFu) ^ 0x4B000008u) - 8388616.0f) * s;
}

// WT: 0 = Q8 (q + scales), 1 = bf16, 2 = fp32, 3 = Q4 (two codes per byte + scales). Elements one lane reads with one load
// (16 bytes; 8 bytes for Q4):
template <int WT> struct Epl { static constexpr int v = (WT == 0 || WT == 3) ? 16 : (WT == 1 ? 8 : 4); };

// raw 16-byte weight chunk of one lane (+ its block scale for Q8), loaded before the data it multiplies is known
struct RawW { uint4 v; float s; };
template <int WT>
__device__ __forceinline__ RawW load_raw(const void* w, const float* scales, size_t row, int C, int c) {
    RawW r;
    r.s = 0.f;
    if (WT == 0) {
        r.v = *reinterpret_cast<const uint4*>((const int8_t*)w + row * C + c);
        r.s = scales[row * (C / 32) + (c >> 5)];
    } else if (WT == 1) {
        r.v = *reinterpret_cast<const uint4*>((const bf16*)w + row * C + c);
    } else if (WT == 3) {
        const uint2 h = *reinterpret_cast<const uint2*>((const uint8_t*)w + ((row * C + c) >> 1));
        r.v = make_uint4(h.x, h.y, 0u, 0u);
        r.s = scales[row * (C / 32) + (c >> 5)];
    } else {
        r.v = *reinterpret_cast<const uint4*>((const float*)w + row * C + c);
    }
    return r;
}
template <int WT>
__device__ __forceinline__ void expand_raw(const RawW& r, float* wv) {
    if (WT == 0) {
        dequant4(r.v.x, r.s, wv); dequant4(r.v.y, r.s, wv + 4); dequant4(r.v.z, r.s, wv + 8); dequant4(r.v.w, r.s, wv + 12);
    } else if (WT == 1) {
        wv[0] = __uint_as_float(r.v.x << 16); wv[1] = __uint_as_float(r.v.x & 0xffff0000u);
        wv[2] = __uint_as_float(r.v.y << 16); wv[3] = __uint_as_float(r.v.y & 0xffff0000u);
        wv[4] = __uint_as_float(r.v.z << 16); wv[5] = __uint_as_float(r.v.z & 0xffff0000u);
        wv[6] = __uint_as_float(r.v.w << 16); wv[7] = __uint_as_float(r.v.w & 0xffff0000u);
    } else if (WT == 3) {
        dequant8_nibbles(r.v.x, r.s, wv); dequant8_nibbles(r.v.y, r.s, wv + 8);
    } else {
        wv[0] = __uint_as_float(r.v.x); wv[1] = __uint_as_float(r.v.y); wv[2] = __uint_as_float(r.v.z); wv[3] = __uint_as_float(r.v.w);
    }
}

// Single sequence (or a few, blockIdx.y): one warp per output row; the activation row lives in registers (CH chunks of
// 32 lanes x EPL columns), so the loop touches only the weight stream. Two rows are in flight per warp, and the first
// two rows' weights are requested before the kernel waits for its predecessor.
// PRO: 0 = x as given; 1 = RMSNorm(x) * lnw (rmsnorm_forward, src/kernels/forward.metal:988-1017) folded in;
//      2 = x is [gate | up] of width 2C and the operand is silu(gate) * up (swiglu_forward, forward.metal:1179).
template <int WT, int CH, int PRO>
__global__ void __launch_bounds__(GEMV_WARPS * 32)
decode_gemv1_kernel(float* __restrict__ out, int ldo, const float* __restrict__ x, int ldx, const void* __restrict__ w,
                    const float* __restrict__ scales, const float* __restrict__ res, int ldr, const float* __restrict__ lnw, float eps,
                    int C, int OC) {
    constexpr int EPL = Epl<WT>::v;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b = blockIdx.y;
    const int stride = gridDim.x * GEMV_WARPS;
    int oc = blockIdx.x * GEMV_WARPS + warp;
    RawW r0[CH], r1[CH];
    if (oc < OC) {
        const int o1 = oc + stride < OC ? oc + stride : oc;
#pragma unroll
        for (int j = 0; j < CH; ++j) {
            const int c = (j * 32 + lane) * EPL;
            if (c < C) { r0[j] = load_raw<WT>(w, scales, (size_t)oc, C, c); r1[j] = load_raw<WT>(w, scales, (size_t)o1, C, c); }
        }
    }
    // norm gains of the float4 pieces this thread will transform: weights, so they can be requested before the wait as well
    constexpr int NPIECE = (CH * 32 * (EPL / 4) + GEMV_WARPS * 32 - 1) / (GEMV_WARPS * 32);
    float4 gain[PRO == 1 ? NPIECE : 1];
    if (PRO == 1) {
#pragma unroll
        for (int k = 0; k < NPIECE; ++k) {
            const int f = threadIdx.x + k * GEMV_WARPS * 32;
            gain[k] = f < C / 4 ? *reinterpret_cast<const float4*>(lnw + 4 * f) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    pdl_launch_dependents();
    pdl_wait();
    // the residual of this warp's first two rows: requested now, needed only after the reduction
    float res0 = 0.f, res1 = 0.f;
    if (res && lane == 0 && oc < OC) {
        res0 = res[(size_t)b * ldr + oc];
        if (oc + stride < OC) res1 = res[(size_t)b * ldr + oc + stride];
    }
    // The operand row is fetched ONCE per block (every warp needs all of it), transformed, and parked in shared memory in
    // the order the lanes consume it: float4 number f of the row belongs to chunk f / (32 * E4), lane (f / E4) % 32, piece
    // f % E4, and is stored at chunk * 32 * E4 + piece * 32 + lane, so a warp reads 32 consecutive float4 per piece.
    extern __shared__ float4 sx4[];
    __shared__ float s_red[GEMV_WARPS];
    constexpr int E4 = EPL / 4;
    const int nvec = C / 4;
    const float* xrow = x + (size_t)b * ldx;
    float ss = 0.f;
    for (int f = threadIdx.x; f < CH * 32 * E4; f += GEMV_WARPS * 32) {
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (f < nvec) {
            v = *reinterpret_cast<const float4*>(xrow + 4 * f);
            if (PRO == 1) {
                ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
            } else if (PRO == 2) {
                const float4 u = *reinterpret_cast<const float4*>(xrow + C + 4 * f);
                v.x = v.x / (1.0f + expf(-v.x)) * u.x; v.y = v.y / (1.0f + expf(-v.y)) * u.y;
                v.z = v.z / (1.0f + expf(-v.z)) * u.z; v.w = v.w / (1.0f + expf(-v.w)) * u.w;
            }
        }
        const int within = f % (32 * E4);
        sx4[(f / (32 * E4)) * (32 * E4) + (within % E4) * 32 + within / E4] = v;
    }
    if (PRO == 1) {
        ss = warp_sum_f(ss);
        if (lane == 0) s_red[warp] = ss;
        __syncthreads();
        float t = 0.f;
#pragma unroll
        for (int i = 0; i < GEMV_WARPS; ++i) t += s_red[i];
        const float inv = 1.0f / sqrtf(t / (float)C + eps);
#pragma unroll
        for (int k = 0; k < NPIECE; ++k) {   // each thread rescales the pieces it wrote itself
            const int f = threadIdx.x + k * GEMV_WARPS * 32;
            if (f >= nvec) break;
            const int within = f % (32 * E4);
            const int idx = (f / (32 * E4)) * (32 * E4) + (within % E4) * 32 + within / E4;
            const float4 g = gain[PRO == 1 ? k : 0];
            float4 v = sx4[idx];
            v.x = v.x * inv * g.x; v.y = v.y * inv * g.y; v.z = v.z * inv * g.z; v.w = v.w * inv * g.w;
            sx4[idx] = v;
        }
    }
    __syncthreads();
    float xr[CH * EPL];
#pragma unroll
    for (int j = 0; j < CH; ++j)
#pragma unroll
        for (int i4 = 0; i4 < E4; ++i4) {
            const float4 v = sx4[j * (32 * E4) + i4 * 32 + lane];
            xr[j * EPL + 4 * i4] = v.x; xr[j * EPL + 4 * i4 + 1] = v.y; xr[j * EPL + 4 * i4 + 2] = v.z; xr[j * EPL + 4 * i4 + 3] = v.w;
        }
    bool first = true;
    for (; oc < OC; oc += 2 * stride) {
        const int oc1 = oc + stride;
        const bool two = oc1 < OC;
        float a0 = 0.f, a1 = 0.f;
#pragma unroll
        for (int j = 0; j < CH; ++j) {
            const int c = (j * 32 + lane) * EPL;
            if (c < C) {
                if (!first) { r0[j] = load_raw<WT>(w, scales, (size_t)oc, C, c); r1[j] = load_raw<WT>(w, scales, (size_t)(two ? oc1 : oc), C, c); }
                float w0[EPL], w1[EPL];
                expand_raw<WT>(r0[j], w0);
                expand_raw<WT>(r1[j], w1);
#pragma unroll
                for (int i = 0; i < EPL; ++i) {
                    a0 = fmaf(xr[j * EPL + i], w0[i], a0);
                    a1 = fmaf(xr[j * EPL + i], w1[i], a1);
                }
            }
        }
        first = false;
        a0 = warp_sum_f(a0);
        a1 = warp_sum_f(a1);
        if (lane == 0) {
            out[(size_t)b * ldo + oc] = a0 + res0;
            if (two) out[(size_t)b * ldo + oc1] = a1 + res1;
            // residuals of the next pair of rows (only the LM head has more than one pair per warp)
            const int n0 = oc + 2 * stride, n1 = n0 + stride;
            res0 = (res && n0 < OC) ? res[(size_t)b * ldr + n0] : 0.f;
            res1 = (res && n1 < OC) ? res[(size_t)b * ldr + n1] : 0.f;
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
    pdl_launch_dependents();
    pdl_wait();
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
                } else if (WT == 3) {
                    const uint32_t pk = *reinterpret_cast<const uint16_t*>((const uint8_t*)w + ((row * C + c) >> 1));
                    const float sc = scales[row * (C / 32) + (c >> 5)];
#pragma unroll
                    for (int i = 0; i < 4; ++i) wv[r][i] = (__uint_as_float(((pk >> (4 * i)) & 0xFu) ^ 0x4B000008u) - 8388616.0f) * sc;
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
    pdl_wait();
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

// Element type of the KV cache: fp32 as the reference keeps it (the default, and what every parity test runs), or bf16 on request
// (half the bytes of the one memory-bound part of batched decode; values are rounded when a row is stored).
template <typename CT> struct KvT;
template <> struct KvT<float> {
    static __device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
    static __device__ __forceinline__ void st1(float* p, float v) { *p = v; }
    static __device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct KvT<bf16> {
    static __device__ __forceinline__ float4 ld4(const bf16* p) {
        const uint2 r = *reinterpret_cast<const uint2*>(p);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.x)), b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.y));
        return make_float4(a.x, a.y, b.x, b.y);
    }
    static __device__ __forceinline__ void st1(bf16* p, float v) { *p = __float2bfloat16_rn(v); }
    static __device__ __forceinline__ void st4(bf16* p, float4 v) {
        const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 r;
        r.x = *reinterpret_cast<const uint32_t*>(&a);
        r.y = *reinterpret_cast<const uint32_t*>(&b);
        *reinterpret_cast<uint2*>(p) = r;
    }
};

// RoPE on this token's q and k at position *pos, then k and v into the cache. qkv: [NB][QD + 2 KV].
// cache: [L][2][NB][MS][KV] fp32 or bf16. cs: [MS][HD/2][2].
template <typename CT>
__global__ void decode_rope_kv_kernel(float* __restrict__ qkv, CT* __restrict__ cache, const float* __restrict__ cs,
                                      const int* __restrict__ pos_ptr, int layer, int NB, int MS, int NH, int NKV, int HD) {
    const int b = blockIdx.x;
    pdl_wait();
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
    CT* kc = cache + (((size_t)layer * 2 + 0) * NB + b) * (size_t)MS * KV + (size_t)pos * KV;
    CT* vc = cache + (((size_t)layer * 2 + 1) * NB + b) * (size_t)MS * KV + (size_t)pos * KV;
    for (int i = threadIdx.x; i < KV; i += blockDim.x) {
        KvT<CT>::st1(kc + i, row[QD + i]);
        KvT<CT>::st1(vc + i, row[QD + KV + i]);
    }
}

// One block (256 threads) per (KV head, sequence, slice of positions); it serves the MUL query heads that share the KV
// head, so every cache row is read once. Phase 1: 8 lanes per position read one K row (coalesced) and form the MUL scaled
// scores. Phase 2: softmax statistics per head over the slice. Phase 3: position groups accumulate p * V with float4
// reads of the V rows and are summed through shared memory. With more than one slice the (max, sum, accumulator)
// triples go to scratch and the block that finishes last (an atomic ticket, no waiting) merges them.
// ROPE: the kernel first rotates this token's q (in registers) and k by the position's angles (rope_forward,
// forward.metal:1284) and stores k, v into the cache row of the position (kv_store, forward.metal:1317); qkv then holds the
// un-rotated projections and stays untouched.
constexpr int ATT_THREADS = 256;
// VPRE (grids of a few blocks per SM, where latency, not occupancy, decides): the first K and V rows of the slice are requested
// before the dependency wait, together.
template <int HD, int MUL, bool ROPE, bool VPRE, typename CT>
__global__ void __launch_bounds__(ATT_THREADS)
decode_attention_kernel(float* __restrict__ out, const float* __restrict__ qkv, CT* cache, const float* __restrict__ cs,
                        const int* __restrict__ pos_ptr, float* part, unsigned* tickets, int layer, int NB, int MS, int NH, int NKV,
                        int chunk, float scale) {
    extern __shared__ float sm[];
    constexpr int EPL = HD / 8;             // K floats per lane in phase 1
    constexpr int D4 = HD / 4;              // float4 per V row
    constexpr int GROUPS = ATT_THREADS / D4;
    constexpr int PW = HD + 2;              // partial record: acc[HD], max, sum
    const int kh = blockIdx.x, b = blockIdx.y, z = blockIdx.z, nz = gridDim.z, tid = threadIdx.x;
    // Before the dependency wait: everything that was written by EARLIER steps — the position counter (advanced by the last
    // kernel of the previous step), the cache rows below the current position, the rotation table. Only the row of the
    // current position is produced inside this step; whoever loaded it early reloads it after the wait.
    const int n = *pos_ptr + 1;
    const int t_begin = z * chunk, t_end = min(n, t_begin + chunk), len = max(t_end - t_begin, 0);
    const int QD = NH * HD, KV = NKV * HD;
    constexpr int PU = 4;   // positions in flight per 8-lane group: the K rows of all four are requested before any is used
    constexpr int VU = 8;   // V rows in flight per thread
    const int sub = tid & 7, slot = tid >> 3;          // phase 1: 8 lanes per position, 32 positions per block iteration
    const int d4 = tid % D4, grp = tid / D4;           // phase 3: one float4 of a V row per thread, GROUPS rows per block iteration
    const int tn = n - 1 - t_begin;                    // the current position inside this slice (if 0 <= tn < len)
    const CT* kc = cache + (((size_t)layer * 2 + 0) * NB + b) * (size_t)MS * KV + (size_t)kh * HD;
    const CT* vc = cache + (((size_t)layer * 2 + 1) * NB + b) * (size_t)MS * KV + (size_t)kh * HD;
    float4 kpre[VPRE ? PU : 1][EPL / 4];
    if (VPRE) {
#pragma unroll
        for (int u = 0; u < PU; ++u) {
            const int t = slot + u * (ATT_THREADS / 8);
#pragma unroll
            for (int i = 0; i < EPL / 4; ++i)
                kpre[u][i] = t < len ? KvT<CT>::ld4(kc + (size_t)(t_begin + t) * KV + sub * EPL + i * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    float4 vpre[VPRE ? VU : 1];
    if (VPRE) {
#pragma unroll
        for (int u = 0; u < VU; ++u) {
            const int t = grp + u * GROUPS;
            vpre[u] = t < len ? KvT<CT>::ld4(vc + (size_t)(t_begin + t) * KV + d4 * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    float rc[ROPE ? EPL : 1], rs[ROPE ? EPL : 1];      // rotation of this lane's query elements
    if (ROPE) {
#pragma unroll
        for (int i = 0; i < EPL; ++i) {
            const int p = (sub & 3) * EPL + i;
            rc[i] = cs[((size_t)(n - 1) * (HD / 2) + p) * 2];
            rs[i] = cs[((size_t)(n - 1) * (HD / 2) + p) * 2 + 1];
        }
    }
    pdl_launch_dependents();
    pdl_wait();
    float* sc = sm;                                    // [MUL][chunk]
    float* red = sm + (size_t)MUL * chunk;             // [MUL][GROUPS][HD] (phase 3) / [MUL][8] (phase 2)
    __shared__ float s_stat[2 * MUL];
    __shared__ unsigned s_ticket;
    if (ROPE && n - 1 >= t_begin && n - 1 < t_begin + chunk) {  // block-uniform: the slice that owns the new position
        constexpr int hd2 = HD / 2;
        const float* krow = qkv + (size_t)b * (QD + 2 * KV) + QD + (size_t)kh * HD;
        CT* kdst = cache + (((size_t)layer * 2 + 0) * NB + b) * (size_t)MS * KV + (size_t)(n - 1) * KV + (size_t)kh * HD;
        CT* vdst = cache + (((size_t)layer * 2 + 1) * NB + b) * (size_t)MS * KV + (size_t)(n - 1) * KV + (size_t)kh * HD;
        if (tid < hd2) {
            const float c = cs[((size_t)(n - 1) * hd2 + tid) * 2], s = cs[((size_t)(n - 1) * hd2 + tid) * 2 + 1];
            const float x0 = krow[tid], x1 = krow[tid + hd2];
            KvT<CT>::st1(kdst + tid, x0 * c - x1 * s);
            KvT<CT>::st1(kdst + tid + hd2, x0 * s + x1 * c);
        } else if (tid >= 128 && tid < 128 + HD) {
            KvT<CT>::st1(vdst + tid - 128, krow[KV + tid - 128]);
        }
        __syncthreads();  // the rows just written are read back below by other threads of this block
    }
    // the row of the current position was (re)written inside this step: fetch it again where it was requested early
    if (VPRE && tn >= 0 && tn < len) {
#pragma unroll
        for (int u = 0; u < PU; ++u)
            if (slot + u * (ATT_THREADS / 8) == tn)
#pragma unroll
                for (int i = 0; i < EPL / 4; ++i) kpre[VPRE ? u : 0][i] = KvT<CT>::ld4(kc + (size_t)(n - 1) * KV + sub * EPL + i * 4);
        {
#pragma unroll
            for (int u = 0; u < VU; ++u)
                if (grp + u * GROUPS == tn) vpre[u] = KvT<CT>::ld4(vc + (size_t)(n - 1) * KV + d4 * 4);
        }
    }
    const float* qrow = qkv + (size_t)b * (QD + 2 * KV) + (size_t)kh * MUL * HD;

    // phase 1
    float qr[MUL][EPL];
#pragma unroll
    for (int h = 0; h < MUL; ++h)
#pragma unroll
        for (int i = 0; i < EPL; i += 4) {
            const float4 v = *reinterpret_cast<const float4*>(qrow + h * HD + sub * EPL + i);
            qr[h][i] = v.x; qr[h][i + 1] = v.y; qr[h][i + 2] = v.z; qr[h][i + 3] = v.w;
        }
    if (ROPE) {
        // lanes sub 0..3 hold the first half of the head, sub 4..7 the second: the rotation partner sits 4 lanes away
#pragma unroll
        for (int i = 0; i < EPL; ++i) {
            const float c = rc[ROPE ? i : 0], s = rs[ROPE ? i : 0];
#pragma unroll
            for (int h = 0; h < MUL; ++h) {
                const float mine = qr[h][i];
                const float other = __shfl_xor_sync(0xffffffffu, mine, 4);
                qr[h][i] = sub < 4 ? mine * c - other * s : other * s + mine * c;
            }
        }
    }
    float mx[MUL];
#pragma unroll
    for (int h = 0; h < MUL; ++h) mx[h] = -INFINITY;
    for (int t0 = 0; t0 < len; t0 += PU * (ATT_THREADS / 8)) {
        float4 kv[PU][EPL / 4];
#pragma unroll
        for (int u = 0; u < PU; ++u) {
            const int t = t0 + slot + u * (ATT_THREADS / 8);
            if (VPRE && t0 == 0) {
#pragma unroll
                for (int i = 0; i < EPL / 4; ++i) kv[u][i] = kpre[VPRE ? u : 0][i];
            } else if (t < len) {
                const CT* kt = kc + (size_t)(t_begin + t) * KV + sub * EPL;
#pragma unroll
                for (int i = 0; i < EPL / 4; ++i) kv[u][i] = KvT<CT>::ld4(kt + i * 4);
            } else {
#pragma unroll
                for (int i = 0; i < EPL / 4; ++i) kv[u][i] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
#pragma unroll
        for (int u = 0; u < PU; ++u) {
            const int t = t0 + slot + u * (ATT_THREADS / 8);
#pragma unroll
            for (int h = 0; h < MUL; ++h) {
                float v = 0.f;
#pragma unroll
                for (int i = 0; i < EPL / 4; ++i)
                    v = fmaf(qr[h][i * 4], kv[u][i].x, fmaf(qr[h][i * 4 + 1], kv[u][i].y, fmaf(qr[h][i * 4 + 2], kv[u][i].z, fmaf(qr[h][i * 4 + 3], kv[u][i].w, v))));
                v += __shfl_xor_sync(0xffffffffu, v, 1);
                v += __shfl_xor_sync(0xffffffffu, v, 2);
                v += __shfl_xor_sync(0xffffffffu, v, 4);
                v *= scale;
                if (t < len) {
                    if (sub == 0) sc[(size_t)h * chunk + t] = v;
                    mx[h] = fmaxf(mx[h], v);
                }
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
        for (int t = tid; t < len; t += ATT_THREADS) {
            const float e = expf(sc[(size_t)h * chunk + t] - mx[h]);
            sc[(size_t)h * chunk + t] = e;
            sum += e;
        }
        sum = warp_sum_f(sum);
        if ((tid & 31) == 0) red[h * 8 + (tid >> 5)] = sum;
    }
    __syncthreads();
    if (tid < MUL) {
        float t = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) t += red[tid * 8 + i];
        s_stat[tid] = t;  // sum of exp over the slice
    }
    __syncthreads();
    // phase 3
    float4 acc[MUL];
#pragma unroll
    for (int h = 0; h < MUL; ++h) acc[h] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int t0 = grp; t0 < len; t0 += VU * GROUPS) {
        float4 v[VU];
#pragma unroll
        for (int u = 0; u < VU; ++u) {
            const int t = t0 + u * GROUPS;
            if (VPRE && t0 == grp) v[u] = vpre[VPRE ? u : 0];
            else v[u] = t < len ? KvT<CT>::ld4(vc + (size_t)(t_begin + t) * KV + d4 * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int u = 0; u < VU; ++u) {
            const int t = t0 + u * GROUPS;
            if (t < len) {
#pragma unroll
                for (int h = 0; h < MUL; ++h) {
                    const float p = sc[(size_t)h * chunk + t];
                    acc[h].x = fmaf(p, v[u].x, acc[h].x); acc[h].y = fmaf(p, v[u].y, acc[h].y);
                    acc[h].z = fmaf(p, v[u].z, acc[h].z); acc[h].w = fmaf(p, v[u].w, acc[h].w);
                }
            }
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
        if (nz == 1) {
            out[(size_t)b * QD + (size_t)(kh * MUL + h) * HD + d] = t / s_stat[h];
        } else {
            float mh = mx[0];
#pragma unroll
            for (int hh = 1; hh < MUL; ++hh) mh = (h == hh) ? mx[hh] : mh;
            float* rec = part + ((((size_t)b * NKV + kh) * MUL + h) * nz + z) * PW;
            rec[d] = t;
            if (d == 0) { rec[HD] = mh; rec[HD + 1] = s_stat[h]; }
        }
    }
    if (nz == 1) return;
    // merge: the block that draws the last ticket of this (sequence, KV head) combines all slices
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const unsigned tk = atomicAdd(&tickets[(size_t)b * NKV + kh], 1u);
        s_ticket = tk;
        if (tk == (unsigned)nz - 1) tickets[(size_t)b * NKV + kh] = 0;  // ready for the next launch
    }
    __syncthreads();
    if (s_ticket != (unsigned)nz - 1) return;
    __threadfence();
    for (int i = tid; i < MUL * HD; i += ATT_THREADS) {
        const int h = i / HD, d = i - h * HD;
        const float* rec = part + ((((size_t)b * NKV + kh) * MUL + h) * nz) * PW;
        float M = -INFINITY;
        for (int zz = 0; zz < nz; ++zz) M = fmaxf(M, __ldcg(rec + (size_t)zz * PW + HD));
        float Lsum = 0.f, a = 0.f;
        for (int zz = 0; zz < nz; ++zz) {
            const float mz = __ldcg(rec + (size_t)zz * PW + HD);
            const float wgt = mz == -INFINITY ? 0.f : expf(mz - M);
            Lsum = fmaf(__ldcg(rec + (size_t)zz * PW + HD + 1), wgt, Lsum);
            a = fmaf(__ldcg(rec + (size_t)zz * PW + d), wgt, a);
        }
        out[(size_t)b * QD + (size_t)(kh * MUL + h) * HD + d] = a / Lsum;
    }
}

// Operand preparation for the tensor-core path: one block per row. The fp32 operand row (optionally RMSNorm(x) * lnw, or
// silu(gate) * up of a [gate | up] row) is split into bf16 hi = rn(v) and lo = rn(v - hi) and written as [hi | lo] (parts 2)
// or [hi | lo | hi] (parts 3), to be multiplied with weights laid out as [w | w] or [w_hi | w_hi | w_lo]: one bf16 GEMM over the
// concatenated reduction axis then equals the fp32 product to about 2^-17 relative. The same launch initialises the fp32
// output row the GEMM accumulates into (with the residual, or zero).
template <int MODE>
__global__ void __launch_bounds__(256)
decode_prep_kernel(bf16* __restrict__ a, int parts, const float* __restrict__ x, int ldx, const float* __restrict__ lnw, float eps,
                   float* __restrict__ init_out, int ldo, const float* __restrict__ init_src, int ldr, int n_out, int C) {
    __shared__ float red[8];
    const size_t row = blockIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    const float* xr = x + row * ldx;
    float inv = 1.f;
    if (MODE == 1) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < C; i += 256) ss += xr[i] * xr[i];
        ss = warp_sum_f(ss);
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
        __syncthreads();
        float t = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) t += red[i];
        inv = 1.0f / sqrtf(t / (float)C + eps);
    }
    bf16* ar = a + row * (size_t)parts * C;
    const int step = gridDim.y * 256;
    for (int c = blockIdx.y * 256 + threadIdx.x; c < C; c += step) {
        float v = xr[c];
        if (MODE == 1) v = v * inv * lnw[c];
        if (MODE == 2) v = v / (1.0f + expf(-v)) * xr[C + c];
        const bf16 hi = __float2bfloat16_rn(v);
        const bf16 lo = __float2bfloat16_rn(v - __bfloat162float(hi));
        ar[c] = hi;
        ar[C + c] = lo;
        if (parts == 3) ar[2 * C + c] = hi;
    }
    if (init_out)
        for (int j = blockIdx.y * 256 + threadIdx.x; j < n_out; j += step) init_out[row * ldo + j] = init_src ? init_src[row * ldr + j] : 0.f;
}

// Prefill: K and V of every prompt row (row = b * T + t of a packed [q | k | v] matrix, k already rotated) into the cache.
template <typename CT>
__global__ void decode_kv_scatter_kernel(CT* __restrict__ cache, const float* __restrict__ qkv, int ldqkv, int layer, int NB, int T, int MS,
                                         int QD, int KV) {
    pdl_wait();
    const long i = blockIdx.x * (long)blockDim.x + threadIdx.x;  // float4 index over [NB*T][2][KV/4]
    const int kv4 = KV / 4;
    if (i >= (long)NB * T * 2 * kv4) return;
    const int c = (int)(i % kv4);
    const int which = (int)((i / kv4) & 1);
    const long row = i / (2 * kv4);
    const int b = (int)(row / T), t = (int)(row - (long)b * T);
    const float4 v = *reinterpret_cast<const float4*>(qkv + row * ldqkv + QD + which * KV + c * 4);
    KvT<CT>::st4(cache + ((((size_t)layer * 2 + which) * NB + b) * (size_t)MS + t) * KV + c * 4, v);
}

__global__ void decode_swiglu_kernel(float* __restrict__ out, const float* __restrict__ gu, int H, int NB) {
    pdl_wait();
    const long i = blockIdx.x * (long)blockDim.x + threadIdx.x;
    if (i >= (long)NB * H) return;
    const int b = (int)(i / H), c = (int)(i - (long)b * H);
    const float g = gu[(size_t)b * 2 * H + c], u = gu[(size_t)b * 2 * H + H + c];
    out[i] = g / (1.0f + expf(-g)) * u;
}

template <typename TT>
__global__ void decode_embed_kernel(float* __restrict__ out, const TT* __restrict__ table, const int* __restrict__ tokens, int D, int NB) {
    pdl_wait();
    const long i = blockIdx.x * (long)blockDim.x + threadIdx.x;
    if (i >= (long)NB * D) return;
    const int b = (int)(i / D), c = (int)(i - (long)b * D);
    out[i] = to_f32(table[(size_t)tokens[b] * D + c]);
}

// pos (may be null): the step's position counter, advanced by one once every row is done with it
__global__ void decode_argmax_kernel(int* __restrict__ out, const float* __restrict__ logits, int V, int* pos) {
    __shared__ float sv[32];
    __shared__ int si[32];
    pdl_wait();
    const float* lr = logits + (size_t)blockIdx.x * V;
    float best = -INFINITY;
    int bi = 0x7fffffff;
    if ((V & 3) == 0 && ((((size_t)blockIdx.x * V) & 3) == 0)) {
        // 8 float4 per thread are requested before the first comparison: one memory round trip per 32768 logits
        const int nv = V >> 2;
        for (int base = 0; base < nv; base += 8 * (int)blockDim.x) {
            float4 v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int f = base + u * (int)blockDim.x + (int)threadIdx.x;
                v[u] = f < nv ? reinterpret_cast<const float4*>(lr)[f] : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int i = 4 * (base + u * (int)blockDim.x + (int)threadIdx.x);   // ascending in u: ties keep the lowest index
                if (v[u].x > best) { best = v[u].x; bi = i; }
                if (v[u].y > best) { best = v[u].y; bi = i + 1; }
                if (v[u].z > best) { best = v[u].z; bi = i + 2; }
                if (v[u].w > best) { best = v[u].w; bi = i + 3; }
            }
        }
    } else {
        for (int i = threadIdx.x; i < V; i += blockDim.x) {
            const float x = lr[i];
            if (x > best || (x == best && i < bi)) { best = x; bi = i; }
        }
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
        if (threadIdx.x == 0) {
            out[blockIdx.x] = bi == 0x7fffffff ? 0 : bi;
            if (pos && blockIdx.x == 0) *pos += 1;  // no block of this kernel reads the counter
        }
    }
}

__global__ void decode_advance_kernel(int* pos) {
    pdl_wait();
    *pos += 1;
}

}  // namespace

// Launch with the programmatic-stream-serialisation attribute (every kernel of this file waits with pdl_wait()).
static bool pdl_enabled() {
    static int v = -1;
    if (v < 0) v = getenv("BM_NO_PDL") ? 0 : 1;
    return v == 1;
}
template <typename... KArgs, typename... Args>
static int launch_k(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...) == cudaSuccess ? 0 : -9;
}

template <int WT, int CH, int PRO>
static int launch_gemv1(float* out, int ldo, const float* x, int ldx, const void* w, const float* scales, const float* res, int ldr,
                        const float* lnw, float eps, int NB, int C, int OC, cudaStream_t st) {
    int gx = (OC + GEMV_WARPS - 1) / GEMV_WARPS;
    if (gx > 148 * 4) gx = 148 * 4;
    constexpr size_t smem = (size_t)CH * 32 * Epl<WT>::v * sizeof(float);  // the operand row, at most 12 KB
    return launch_k(decode_gemv1_kernel<WT, CH, PRO>, dim3(gx, NB), dim3(GEMV_WARPS * 32), smem, st, out, ldo, x, ldx, w, scales, res, ldr, lnw,
                    eps, C, OC);
}
template <int WT, int PRO>
static int gemv1_dispatch(float* out, int ldo, const float* x, int ldx, const void* w, const float* scales, const float* res, int ldr,
                          const float* lnw, float eps, int NB, int C, int OC, cudaStream_t st) {
    constexpr int EPL = Epl<WT>::v;
    const int regs = (C + 32 * EPL - 1) / (32 * EPL) * EPL;  // activation registers per lane
#define BM_GEMV1(r) return launch_gemv1<WT, r / EPL, PRO>(out, ldo, x, ldx, w, scales, res, ldr, lnw, eps, NB, C, OC, st)
    if (regs <= 32) BM_GEMV1(32);
    if (regs <= 48) BM_GEMV1(48);
    if (regs <= 80) BM_GEMV1(80);
    if (regs <= 96) BM_GEMV1(96);
#undef BM_GEMV1
    return -4;
}
template <int WT>
static int gemv_dispatch(float* out, int ldo, const float* x, int ldx, const void* w, const float* scales, const float* res, int ldr,
                         int prologue, const float* lnw, float eps, int NB, int C, int OC, cudaStream_t st) {
    constexpr int EPL = Epl<WT>::v;
    const bool fits = (C + 32 * EPL - 1) / (32 * EPL) * EPL <= 96;
    if (prologue != 0 || (NB < 4 && fits)) {
        if (!fits) return -4;
        if (prologue == 1) return gemv1_dispatch<WT, 1>(out, ldo, x, ldx, w, scales, res, ldr, lnw, eps, NB, C, OC, st);
        if (prologue == 2) return gemv1_dispatch<WT, 2>(out, ldo, x, ldx, w, scales, res, ldr, lnw, eps, NB, C, OC, st);
        return gemv1_dispatch<WT, 0>(out, ldo, x, ldx, w, scales, res, ldr, lnw, eps, NB, C, OC, st);
    }
    const size_t smem = (size_t)GEMV_TB * C * sizeof(float);
    if (smem > 200 * 1024) return -2;
    static std::atomic<unsigned long long> attr_done{0};
    if (first_use_on_current_device(attr_done))
        cudaFuncSetAttribute(decode_gemvb_kernel<WT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    const int rows_per_block = GEMV_WARPS * GEMV_ROWS;
    int gx = (OC + rows_per_block - 1) / rows_per_block;
    if (gx > 148 * 4) gx = 148 * 4;
    return launch_k(decode_gemvb_kernel<WT>, dim3(gx, (NB + GEMV_TB - 1) / GEMV_TB), dim3(GEMV_WARPS * 32), smem, st, out, ldo, x, ldx, w, scales,
                    res, ldr, NB, C, OC);
}

// x rows must be 16-byte aligned (ldx % 4 == 0); C % 32 == 0. prologue: 0 = none, 1 = RMSNorm(x) * lnw, 2 = x is [gate | up] and
// the operand is silu(gate) * up (both only with the register-resident kernel: C <= 96 * 32 columns).
int decode_gemv(float* out, int ldo, const float* x, int ldx, int wtype, const void* w, const float* scales, const float* res, int ldr,
                int prologue, const float* lnw, float eps, int NB, int C, int OC, cudaStream_t st) {
    if (C % 32 || NB <= 0 || (ldx & 3) || prologue < 0 || prologue > 2 || (prologue == 1 && !lnw)) return -1;
    if (wtype == 0) return gemv_dispatch<0>(out, ldo, x, ldx, w, scales, res, ldr, prologue, lnw, eps, NB, C, OC, st);
    if (wtype == 1) return gemv_dispatch<1>(out, ldo, x, ldx, w, scales, res, ldr, prologue, lnw, eps, NB, C, OC, st);
    if (wtype == 2) return gemv_dispatch<2>(out, ldo, x, ldx, w, scales, res, ldr, prologue, lnw, eps, NB, C, OC, st);
    if (wtype == 3) return gemv_dispatch<3>(out, ldo, x, ldx, w, scales, res, ldr, prologue, lnw, eps, NB, C, OC, st);
    return -1;
}
int decode_rmsnorm(float* out, const float* x, const float* w, int NB, int C, float eps, cudaStream_t st) {
    return launch_k(decode_rmsnorm_kernel, dim3(NB), dim3(256), 0, st, out, x, w, C, eps);
}
int decode_rope_kv(float* qkv, void* cache, int cache_bf16, const float* cs, const int* pos, int layer, int NB, int MS, int NH, int NKV, int HD,
                   cudaStream_t st) {
    if (cache_bf16) return launch_k(decode_rope_kv_kernel<bf16>, dim3(NB), dim3(256), 0, st, qkv, (bf16*)cache, cs, pos, layer, NB, MS, NH, NKV, HD);
    return launch_k(decode_rope_kv_kernel<float>, dim3(NB), dim3(256), 0, st, qkv, (float*)cache, cs, pos, layer, NB, MS, NH, NKV, HD);
}
// Number of position slices for a cache of MS rows: enough blocks to fill the GPU about four times over.
static void attention_split(int NB, int NKV, int MS, int* chunk, int* splits) {
    int want = (592 + NKV * NB - 1) / (NKV * NB);
    if (want < 1) want = 1;
    if (want > 16) want = 16;
    int c = ((MS + want - 1) / want + 31) / 32 * 32;
    if (c < 32) c = 32;
    *chunk = c;
    *splits = (MS + c - 1) / c;
}
size_t decode_attention_scratch_bytes(int NB, int MS, int NH, int NKV, int HD) {
    int chunk, splits;
    attention_split(NB, NKV, MS, &chunk, &splits);
    return (size_t)NB * NH * splits * (HD + 2) * sizeof(float) + (size_t)NB * NKV * sizeof(unsigned);
}
template <int HD, int MUL, bool ROPE, typename CT>
static int launch_attention(float* out, const float* qkv, CT* cache, const float* cs, const int* pos, void* scratch, int layer, int NB,
                            int MS, int NH, int NKV, float scale, cudaStream_t st) {
    int chunk, splits;
    attention_split(NB, NKV, MS, &chunk, &splits);
    if (splits > 1 && !scratch) { chunk = (MS + 31) / 32 * 32; splits = 1; }
    const size_t smem = ((size_t)MUL * chunk + (size_t)MUL * (ATT_THREADS / (HD / 4)) * HD) * sizeof(float);
    // the largest dynamic shared memory size this instantiation has been granted, per device (kernel attributes are per device)
    static size_t attr_smem[64];
    int dev = 0;
    cudaGetDevice(&dev);
    size_t& granted = attr_smem[dev & 63];
    if (smem > 48 * 1024 && smem > granted) {
        if (smem > 220 * 1024) return -2;
        cudaFuncSetAttribute(decode_attention_kernel<HD, MUL, ROPE, true, CT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        cudaFuncSetAttribute(decode_attention_kernel<HD, MUL, ROPE, false, CT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        granted = smem;
    }
    // scratch: tickets first (zeroed once by the owner; every launch leaves them zero), then the partial records
    unsigned* tickets = (unsigned*)scratch;
    float* part = scratch ? (float*)((char*)scratch + (((size_t)NB * NKV * sizeof(unsigned) + 15) / 16) * 16) : nullptr;
    if ((long)NKV * NB * splits <= 2 * 148)
        return launch_k(decode_attention_kernel<HD, MUL, ROPE, true, CT>, dim3(NKV, NB, splits), dim3(ATT_THREADS), smem, st, out, qkv, cache, cs, pos,
                        part, tickets, layer, NB, MS, NH, NKV, chunk, scale);
    return launch_k(decode_attention_kernel<HD, MUL, ROPE, false, CT>, dim3(NKV, NB, splits), dim3(ATT_THREADS), smem, st, out, qkv, cache, cs, pos,
                    part, tickets, layer, NB, MS, NH, NKV, chunk, scale);
}
// head_dim 64 or 128; 1, 2, 3, 4 or 8 query heads per KV head. cs != null: RoPE and the cache store happen inside.
// scratch (may be null: one slice per block): decode_attention_scratch_bytes() + 16 bytes, zero-initialised once.
int decode_attention(float* out, const float* qkv, void* cache, int cache_bf16, const float* cs, const int* pos, void* scratch, int layer, int NB,
                     int MS, int NH, int NKV, int HD, float scale, cudaStream_t st) {
    if (NKV <= 0 || NH % NKV) return -1;
    const int mul = NH / NKV;
#define BM_ATT_CASE_T(hd, m, CT)                                                                                                      \
    if (HD == hd && mul == m)                                                                                                         \
        return cs ? launch_attention<hd, m, true, CT>(out, qkv, (CT*)cache, cs, pos, scratch, layer, NB, MS, NH, NKV, scale, st)      \
                  : launch_attention<hd, m, false, CT>(out, qkv, (CT*)cache, cs, pos, scratch, layer, NB, MS, NH, NKV, scale, st);
#define BM_ATT_CASE(hd, m) BM_ATT_CASE_T(hd, m, float)
    if (cache_bf16) {   // bf16 cache: head_dim 64 only
        BM_ATT_CASE_T(64, 1, bf16) BM_ATT_CASE_T(64, 2, bf16) BM_ATT_CASE_T(64, 3, bf16) BM_ATT_CASE_T(64, 4, bf16) BM_ATT_CASE_T(64, 8, bf16)
        return -3;
    }
    BM_ATT_CASE(64, 1) BM_ATT_CASE(64, 2) BM_ATT_CASE(64, 3) BM_ATT_CASE(64, 4) BM_ATT_CASE(64, 8)
    BM_ATT_CASE(128, 1) BM_ATT_CASE(128, 2) BM_ATT_CASE(128, 4) BM_ATT_CASE(128, 8)
#undef BM_ATT_CASE_T
#undef BM_ATT_CASE
    return -3;
}
int decode_prep(bf16* a, int parts, const float* x, int ldx, int mode, const float* lnw, float eps, float* init_out, int ldo,
                const float* init_src, int ldr, int n_out, int rows, int C, cudaStream_t st) {
    if (rows <= 0 || C <= 0 || (parts != 2 && parts != 3) || mode < 0 || mode > 2 || (mode == 1 && !lnw)) return -1;
    // the norm needs the whole row in one block; the other modes spread a row over several blocks when there are few rows
    int ny = 1;
    if (rows < 592) {
        const int widest = C > n_out ? C : n_out;
        ny = (widest + 511) / 512;
        if (ny > 16) ny = 16;
        if (ny < 1) ny = 1;
    }
    if (mode == 1) return launch_k(decode_prep_kernel<1>, dim3(rows, ny), dim3(256), 0, st, a, parts, x, ldx, lnw, eps, init_out, ldo, init_src, ldr, n_out, C);
    if (mode == 2) return launch_k(decode_prep_kernel<2>, dim3(rows, ny), dim3(256), 0, st, a, parts, x, ldx, lnw, eps, init_out, ldo, init_src, ldr, n_out, C);
    return launch_k(decode_prep_kernel<0>, dim3(rows, ny), dim3(256), 0, st, a, parts, x, ldx, lnw, eps, init_out, ldo, init_src, ldr, n_out, C);
}
int decode_kv_scatter(void* cache, int cache_bf16, const float* qkv, int ldqkv, int layer, int NB, int T, int MS, int QD, int KV, cudaStream_t st) {
    if ((KV & 3) || (QD & 3) || (ldqkv & 3) || T > MS) return -1;
    const long n = (long)NB * T * 2 * (KV / 4);
    if (cache_bf16)
        return launch_k(decode_kv_scatter_kernel<bf16>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, (bf16*)cache, qkv, ldqkv, layer, NB, T, MS, QD, KV);
    return launch_k(decode_kv_scatter_kernel<float>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, (float*)cache, qkv, ldqkv, layer, NB, T, MS, QD, KV);
}
// head_dim 64 only (returns -3 otherwise); all pitches multiples of 4 floats
int decode_swiglu(float* out, const float* gu, int NB, int H, cudaStream_t st) {
    const long n = (long)NB * H;
    return launch_k(decode_swiglu_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, out, gu, H, NB);
}
int decode_embed(float* out, int ttype, const void* table, const int* tokens, int NB, int D, cudaStream_t st) {
    const long n = (long)NB * D;
    // first kernel of a step: launched without the attribute, so it fully serialises behind whatever precedes the step
    if (ttype == 1) decode_embed_kernel<bf16><<<(int)((n + 255) / 256), 256, 0, st>>>(out, (const bf16*)table, tokens, D, NB);
    else decode_embed_kernel<float><<<(int)((n + 255) / 256), 256, 0, st>>>(out, (const float*)table, tokens, D, NB);
    return 0;
}
int decode_argmax(int* out, const float* logits, int NB, int V, int* pos_to_advance, cudaStream_t st) {
    return launch_k(decode_argmax_kernel, dim3(NB), dim3(1024), 0, st, out, logits, V, pos_to_advance);
}
int decode_advance(int* pos, cudaStream_t st) {
    return launch_k(decode_advance_kernel, dim3(1), dim3(1), 0, st, pos);
}

}  // namespace bmb
