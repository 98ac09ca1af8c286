// HBM-bound kernels of the training step: embedding gather / scatter-add, RMSNorm forward and
// backward, RoPE, SwiGLU, softmax cross-entropy with its gradient, AdamW, casts, argmax.
// All are coalesced, 128-bit vectorised and warp-reduced; arithmetic is fp32 whatever the storage
// type. Each kernel cites the reference kernel whose result it reproduces.
#include "kernels.cuh"

namespace bmb {

namespace {
constexpr int WARPS_PER_BLOCK = 8;
constexpr int BLOCK = WARPS_PER_BLOCK * 32;
inline int ceil_div(long a, long b) { return (int)((a + b - 1) / b); }
inline bool aligned16(const void* p) { return (((uintptr_t)p) & 15) == 0; }
}  // namespace

// ------------------------------------------------------------------------------------------------
// Embedding gather: out[t,:] = table[tokens[t],:]  (reference: embed_lookup, src/baremetal/trainer.c:275-298,
// which reads the fp32 master table). One thread per 4 elements.
// An id outside [0, V) never indexes the table: the row becomes zero and the error word is set (BMB_ERR_BAD_TOKEN).
template <typename T>
__global__ void embedding_forward_kernel(T* __restrict__ out, const float* __restrict__ table, const int* __restrict__ tokens,
                                         int n_tok, int D4, int V, int* __restrict__ err) {
    const long i = blockIdx.x * (long)blockDim.x + threadIdx.x;
    if (i >= (long)n_tok * D4) return;
    const int t = (int)(i / D4), d4 = (int)(i - (long)t * D4);
    const int tok = tokens[t];
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if ((unsigned)tok < (unsigned)V) v = reinterpret_cast<const float4*>(table + (size_t)tok * D4 * 4)[d4];
    else if (d4 == 0 && err) atomicExch(err, BMB_ERR_BAD_TOKEN);
    T* o = out + (size_t)t * D4 * 4 + d4 * 4;
    o[0] = from_f32<T>(v.x); o[1] = from_f32<T>(v.y); o[2] = from_f32<T>(v.z); o[3] = from_f32<T>(v.w);
}
template <typename T> int embedding_forward(T* out, const float* table, const int* tokens, int n_tok, int D, int V, int* err, cudaStream_t st) {
    if (D % 4) return -1;
    const long n = (long)n_tok * (D / 4);
    embedding_forward_kernel<T><<<ceil_div(n, 256), 256, 0, st>>>(out, table, tokens, n_tok, D / 4, V, err);
    return 0;
}
template int embedding_forward<float>(float*, const float*, const int*, int, int, int, int*, cudaStream_t);
template int embedding_forward<bf16>(bf16*, const float*, const int*, int, int, int, int*, cudaStream_t);

// Embedding scatter-add: gwte[tokens[t],:] += gout[t,:] with float atomics, on top of whatever the
// buffer already holds (the tied LM-head wgrad) — reference: embedding_backward, src/kernels/backward.metal:636.
template <typename T>
__global__ void embedding_backward_kernel(float* __restrict__ gwte, const T* __restrict__ gout, const int* __restrict__ tokens,
                                          int n_tok, int D4, int V, int* __restrict__ err) {
    const long i = blockIdx.x * (long)blockDim.x + threadIdx.x;
    if (i >= (long)n_tok * D4) return;
    const int t = (int)(i / D4), d4 = (int)(i - (long)t * D4);
    const int tok = tokens[t];
    if ((unsigned)tok >= (unsigned)V) {  // never scatter outside the table
        if (d4 == 0 && err) atomicExch(err, BMB_ERR_BAD_TOKEN);
        return;
    }
    const T* g = gout + (size_t)t * D4 * 4 + d4 * 4;
    float* dst = gwte + (size_t)tok * D4 * 4 + d4 * 4;
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(to_f32(g[0])), "f"(to_f32(g[1])),
                 "f"(to_f32(g[2])), "f"(to_f32(g[3]))
                 : "memory");
}
int embedding_backward_f32(float* gwte, const float* gout, const int* tokens, int n_tok, int D, int V, int* err, cudaStream_t st) {
    if (D % 4 || !aligned16(gwte)) return -1;
    const long n = (long)n_tok * (D / 4);
    embedding_backward_kernel<float><<<ceil_div(n, 256), 256, 0, st>>>(gwte, gout, tokens, n_tok, D / 4, V, err);
    return 0;
}
int embedding_backward_bf16(float* gwte, const bf16* gout, const int* tokens, int n_tok, int D, int V, int* err, cudaStream_t st) {
    if (D % 4 || !aligned16(gwte)) return -1;
    const long n = (long)n_tok * (D / 4);
    embedding_backward_kernel<bf16><<<ceil_div(n, 256), 256, 0, st>>>(gwte, gout, tokens, n_tok, D / 4, V, err);
    return 0;
}

// ------------------------------------------------------------------------------------------------
// RMSNorm forward: out = x * rsqrt(mean(x^2) + eps) * w (reference: rmsnorm_forward, src/kernels/forward.metal:993).
// One warp per row; the row stays in registers between the sum of squares and the scaling (NV 16-byte vectors per lane),
// so it is read from memory once. Rows wider than 8 vectors per lane take the two-sweep form.
template <typename T, int NV>
__global__ void rmsnorm_forward_kernel(T* __restrict__ out, float* __restrict__ rstd, const T* __restrict__ x,
                                       const float* __restrict__ w, int N, int C, float eps) {
    constexpr int V = Vec<T>::N;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nvec = C / V;
    // the gains of this lane's columns stay in registers for every row the warp handles
    float wr[NV][V];
#pragma unroll
    for (int a = 0; a < NV; ++a) {
        const int v = lane + a * 32;
#pragma unroll
        for (int i = 0; i < V; i += 4) {
            float4 g = make_float4(0.f, 0.f, 0.f, 0.f);
            if (v < nvec) g = *reinterpret_cast<const float4*>(w + v * V + i);
            wr[a][i] = g.x; wr[a][i + 1] = g.y; wr[a][i + 2] = g.z; wr[a][i + 3] = g.w;
        }
    }
    for (int row = blockIdx.x * WARPS_PER_BLOCK + warp; row < N; row += gridDim.x * WARPS_PER_BLOCK) {
        const T* xr = x + (size_t)row * C;
        T* orow = out + (size_t)row * C;
        typename Vec<T>::Raw raw[NV];
#pragma unroll
        for (int a = 0; a < NV; ++a) {
            const int v = lane + a * 32;
            if (v < nvec) raw[a] = Vec<T>::load_raw(xr + v * V);
        }
        float ss = 0.f;
#pragma unroll
        for (int a = 0; a < NV; ++a) {
            const int v = lane + a * 32;
            if (v < nvec) {
                float f[V];
                Vec<T>::unpack(raw[a], f);
#pragma unroll
                for (int i = 0; i < V; ++i) ss += f[i] * f[i];
            }
        }
        ss = warp_sum(ss) / (float)C;
        const float r = 1.0f / sqrtf(ss + eps);
        if (lane == 0 && rstd) rstd[row] = r;
#pragma unroll
        for (int a = 0; a < NV; ++a) {
            const int v = lane + a * 32;
            if (v < nvec) {
                float f[V], o[V];
                Vec<T>::unpack(raw[a], f);
#pragma unroll
                for (int i = 0; i < V; ++i) o[i] = f[i] * r * wr[a][i];
                Vec<T>::store(orow + v * V, o);
            }
        }
    }
}
template <typename T>
__global__ void rmsnorm_forward_wide_kernel(T* __restrict__ out, float* __restrict__ rstd, const T* __restrict__ x,
                                            const float* __restrict__ w, int N, int C, float eps) {
    constexpr int V = Vec<T>::N;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x * WARPS_PER_BLOCK + warp;
    if (row >= N) return;
    const T* xr = x + (size_t)row * C;
    T* orow = out + (size_t)row * C;
    const int nvec = C / V;
    float ss = 0.f;
    for (int v = lane; v < nvec; v += 32) {
        float f[V];
        Vec<T>::load(xr + v * V, f);
#pragma unroll
        for (int i = 0; i < V; ++i) ss += f[i] * f[i];
    }
    ss = warp_sum(ss) / (float)C;
    const float r = 1.0f / sqrtf(ss + eps);
    if (lane == 0 && rstd) rstd[row] = r;
    for (int v = lane; v < nvec; v += 32) {
        float f[V], o[V];
        Vec<T>::load(xr + v * V, f);
#pragma unroll
        for (int i = 0; i < V; ++i) o[i] = f[i] * r * w[v * V + i];
        Vec<T>::store(orow + v * V, o);
    }
}
template <typename T> int rmsnorm_forward(T* out, float* rstd, const T* x, const float* w, int N, int C, float eps, cudaStream_t st) {
    if (C % Vec<T>::N) return -1;
    const int nv = ceil_div(C / Vec<T>::N, 32);
    const int full = ceil_div(N, WARPS_PER_BLOCK);
    const int grid = full < 148 * 8 ? full : 148 * 8;  // persistent over rows (the register-resident kernels loop)
    if (nv <= 1) rmsnorm_forward_kernel<T, 1><<<grid, BLOCK, 0, st>>>(out, rstd, x, w, N, C, eps);
    else if (nv <= 2) rmsnorm_forward_kernel<T, 2><<<grid, BLOCK, 0, st>>>(out, rstd, x, w, N, C, eps);
    else if (nv <= 4) rmsnorm_forward_kernel<T, 4><<<grid, BLOCK, 0, st>>>(out, rstd, x, w, N, C, eps);
    else if (nv <= 8) rmsnorm_forward_kernel<T, 8><<<grid, BLOCK, 0, st>>>(out, rstd, x, w, N, C, eps);
    else rmsnorm_forward_wide_kernel<T><<<full, BLOCK, 0, st>>>(out, rstd, x, w, N, C, eps);
    return 0;
}
template int rmsnorm_forward<float>(float*, float*, const float*, const float*, int, int, float, cudaStream_t);
template int rmsnorm_forward<bf16>(bf16*, float*, const bf16*, const float*, int, int, float, cudaStream_t);

// RMSNorm backward, input and weight gradient in one sweep
// (reference: rmsnorm_backward_x / rmsnorm_backward_w, src/kernels/backward.metal:340,379):
//   c1 = mean_j(g_j w_j x_j r);  gx_j += r (g_j w_j - x_j r c1);  gw_j = sum_rows g_j x_j r.
// A lane always owns the same columns, so it carries its gw partial in registers across all rows
// of its warp; warps are combined through shared memory into one partial row per block in `scratch`,
// and a second kernel folds the per-block partials in a fixed order (no atomics, deterministic).
constexpr int RMS_BWD_MAX_BLOCKS = 592;  // 4 CTAs per SM on 148 SMs

template <typename T, int NV>
__global__ void rmsnorm_backward_kernel(T* __restrict__ gx, float* __restrict__ scratch, const T* __restrict__ gout,
                                        const T* __restrict__ x, const float* __restrict__ w, const float* __restrict__ rstd,
                                        int N, int C, int w_row0, int w_row1) {
    constexpr int V = Vec<T>::N;
    extern __shared__ float s_gw[];  // [WARPS_PER_BLOCK][C], then the gains as float4 [NV][V/4][32 lanes]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nvec = C / V;
    // The gains are read for every row. Straight from global memory a lane's 8 values sit 32 bytes from its neighbour's, so one
    // scalar load costs 8 L1 wavefronts and the L1 data pipe, not HBM, bounds the kernel; parked in shared memory in lane order
    // a float4 read is 4 conflict-free wavefronts.
    float4* s_w4 = reinterpret_cast<float4*>(s_gw + (size_t)WARPS_PER_BLOCK * C);
    for (int idx = threadIdx.x; idx < NV * (V / 4) * 32; idx += blockDim.x) {
        const int l = idx & 31, ai = idx >> 5, a = ai / (V / 4), i4 = ai % (V / 4);
        const int v = l + a * 32;
        s_w4[idx] = v < nvec ? *reinterpret_cast<const float4*>(w + v * V + i4 * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    __syncthreads();
    float gw_acc[NV][V];
#pragma unroll
    for (int a = 0; a < NV; ++a)
#pragma unroll
        for (int i = 0; i < V; ++i) gw_acc[a][i] = 0.f;

    for (int row = blockIdx.x * WARPS_PER_BLOCK + warp; row < N; row += gridDim.x * WARPS_PER_BLOCK) {
        const T* xr = x + (size_t)row * C;
        const T* gr = gout + (size_t)row * C;
        T* gxr = gx + (size_t)row * C;
        const float r = rstd[row];
        const bool in_w = row >= w_row0 && row < w_row1;
        typename Vec<T>::Raw xraw[NV], graw[NV], oraw[NV];
        float c1 = 0.f;
        // all three operand streams of the row are requested before anything is consumed; they stay packed until used
#pragma unroll
        for (int a = 0; a < NV; ++a) {
            const int v = lane + a * 32;
            if (v < nvec) {
                xraw[a] = Vec<T>::load_raw(xr + v * V);
                graw[a] = Vec<T>::load_raw(gr + v * V);
                oraw[a] = Vec<T>::load_raw(gxr + v * V);
            }
        }
#pragma unroll
        for (int a = 0; a < NV; ++a) {
            const int v = lane + a * 32;
            if (v < nvec) {
                float xs[V], gs[V], ws[V];
                Vec<T>::unpack(xraw[a], xs);
                Vec<T>::unpack(graw[a], gs);
#pragma unroll
                for (int i4 = 0; i4 < V / 4; ++i4) {
                    const float4 g4 = s_w4[(a * (V / 4) + i4) * 32 + lane];
                    ws[4 * i4] = g4.x; ws[4 * i4 + 1] = g4.y; ws[4 * i4 + 2] = g4.z; ws[4 * i4 + 3] = g4.w;
                }
#pragma unroll
                for (int i = 0; i < V; ++i) {
                    const float n = xs[i] * r;
                    if (in_w) gw_acc[a][i] += gs[i] * n;
                    c1 += gs[i] * ws[i] * n;
                }
            }
        }
        c1 = warp_sum(c1) / (float)C;
#pragma unroll
        for (int a = 0; a < NV; ++a) {
            const int v = lane + a * 32;
            if (v < nvec) {
                float xs[V], gs[V], os[V], ws[V];
                Vec<T>::unpack(xraw[a], xs);
                Vec<T>::unpack(graw[a], gs);
                Vec<T>::unpack(oraw[a], os);
#pragma unroll
                for (int i4 = 0; i4 < V / 4; ++i4) {
                    const float4 g4 = s_w4[(a * (V / 4) + i4) * 32 + lane];
                    ws[4 * i4] = g4.x; ws[4 * i4 + 1] = g4.y; ws[4 * i4 + 2] = g4.z; ws[4 * i4 + 3] = g4.w;
                }
#pragma unroll
                for (int i = 0; i < V; ++i) os[i] += r * (gs[i] * ws[i] - xs[i] * r * c1);
                Vec<T>::store(gxr + v * V, os);
            }
        }
    }
#pragma unroll
    for (int a = 0; a < NV; ++a) {
        const int v = lane + a * 32;
        if (v < nvec)
#pragma unroll
            for (int i = 0; i < V; ++i) s_gw[warp * C + v * V + i] = gw_acc[a][i];
    }
    __syncthreads();
    for (int j = threadIdx.x; j < C; j += blockDim.x) {
        float s = 0.f;
#pragma unroll
        for (int wv = 0; wv < WARPS_PER_BLOCK; ++wv) s += s_gw[wv * C + j];
        scratch[(size_t)blockIdx.x * C + j] = s;
    }
}
// 32 columns x 32 row-groups per block: each thread folds every 32nd partial row in a fixed order, then the 32
// row-groups are combined through shared memory in a fixed order.
__global__ void rmsnorm_backward_reduce_kernel(float* __restrict__ gw, const float* __restrict__ scratch, int nblocks, int C,
                                               int accumulate) {
    __shared__ float part[32][33];
    const int j = blockIdx.x * 32 + threadIdx.x;
    float s = 0.f;
    if (j < C)
        for (int b = threadIdx.y; b < nblocks; b += 32) s += scratch[(size_t)b * C + j];
    part[threadIdx.y][threadIdx.x] = s;
    __syncthreads();
    if (threadIdx.y == 0 && j < C) {
        float t = 0.f;
#pragma unroll
        for (int r = 0; r < 32; ++r) t += part[r][threadIdx.x];
        gw[j] = accumulate ? gw[j] + t : t;
    }
}
size_t rmsnorm_backward_scratch_floats(int C) { return (size_t)RMS_BWD_MAX_BLOCKS * C; }

template <typename T, int NV>
static int rmsnorm_backward_launch(T* gx, float* gw, int gw_accumulate, const T* gout, const T* x, const float* w, const float* rstd,
                                   int N, int C, int w_row0, int w_row1, float* scratch, cudaStream_t st) {
    int nblocks = ceil_div(N, WARPS_PER_BLOCK);
    if (nblocks > RMS_BWD_MAX_BLOCKS) nblocks = RMS_BWD_MAX_BLOCKS;
    const size_t smem = (size_t)WARPS_PER_BLOCK * C * sizeof(float) + (size_t)NV * Vec<T>::N * 32 * sizeof(float);
    static std::atomic<unsigned long long> attr_done{0};
    if (first_use_on_current_device(attr_done))
        cudaFuncSetAttribute(rmsnorm_backward_kernel<T, NV>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
    if (smem > 64 * 1024) return -2;
    rmsnorm_backward_kernel<T, NV><<<nblocks, BLOCK, smem, st>>>(gx, scratch, gout, x, w, rstd, N, C, w_row0, w_row1);
    rmsnorm_backward_reduce_kernel<<<ceil_div(C, 32), dim3(32, 32), 0, st>>>(gw, scratch, nblocks, C, gw_accumulate);
    return 0;
}
template <typename T>
int rmsnorm_backward(T* gx, float* gw, int gw_accumulate, const T* gout, const T* x, const float* w, const float* rstd, int N,
                     int C, int w_row0, int w_row1, float* scratch, cudaStream_t st) {
    constexpr int V = Vec<T>::N;
    if (C % V) return -1;
    const int nv = ceil_div(C / V, 32);
#define BMB_RMS_CASE(NVV) \
    return rmsnorm_backward_launch<T, NVV>(gx, gw, gw_accumulate, gout, x, w, rstd, N, C, w_row0, w_row1, scratch, st)
    if (nv <= 1) BMB_RMS_CASE(1);
    if (nv <= 2) BMB_RMS_CASE(2);
    if (nv <= 4) BMB_RMS_CASE(4);
    if (nv <= 8) BMB_RMS_CASE(8);
#undef BMB_RMS_CASE
    return -3;  // C > 2048 (bf16) / 1024 (fp32) is outside the model family this path serves
}
template int rmsnorm_backward<float>(float*, float*, int, const float*, const float*, const float*, const float*, int, int, int,
                                     int, float*, cudaStream_t);
template int rmsnorm_backward<bf16>(bf16*, float*, int, const bf16*, const bf16*, const float*, const float*, int, int, int, int,
                                    float*, cudaStream_t);

// ------------------------------------------------------------------------------------------------
// RoPE, rotate-half pairing (i, i+HD/2), in place on Q and K
// (reference: rope_forward_seq src/kernels/forward.metal:2225, rope_backward_seq src/kernels/backward.metal:980).
// cos/sin come from a table built on the host with the reference's fp32 formula, so every
// implementation rotates by identical angles. One thread per (row, head, pair).
template <typename T>
__global__ void rope_kernel(T* __restrict__ q, int ldq, T* __restrict__ k, int ldk, const float* __restrict__ cs, int rows, int S,
                            int NH, int NKV, int HD, float dir) {
    const int hd2 = HD >> 1;
    const long i = blockIdx.x * (long)blockDim.x + threadIdx.x;
    const long total = (long)rows * (NH + NKV) * hd2;
    if (i >= total) return;
    const int p = (int)(i % hd2);
    const long rh = i / hd2;
    const int h = (int)(rh % (NH + NKV));
    const int row = (int)(rh / (NH + NKV));
    const int pos = row % S;
    T* base = h < NH ? q + (size_t)row * ldq + (size_t)h * HD : k + (size_t)row * ldk + (size_t)(h - NH) * HD;
    const float c = cs[((size_t)pos * hd2 + p) * 2], s = cs[((size_t)pos * hd2 + p) * 2 + 1] * dir;
    const float x0 = to_f32(base[p]), x1 = to_f32(base[p + hd2]);
    base[p] = from_f32<T>(x0 * c - x1 * s);
    base[p + hd2] = from_f32<T>(x0 * s + x1 * c);
}
// Vector form: one thread rotates Vec<T>::N adjacent pairs (two 16-byte loads, two 16-byte stores).
template <typename T>
__global__ void rope_vec_kernel(T* __restrict__ q, int ldq, T* __restrict__ k, int ldk, const float* __restrict__ cs, int rows, int S,
                                int NH, int NKV, int HD, float dir) {
    constexpr int V = Vec<T>::N;
    const int hd2 = HD >> 1, vph = hd2 / V;  // vectors per half head
    const long i = blockIdx.x * (long)blockDim.x + threadIdx.x;
    const long total = (long)rows * (NH + NKV) * vph;
    if (i >= total) return;
    const int pv = (int)(i % vph);
    const long rh = i / vph;
    const int h = (int)(rh % (NH + NKV));
    const int row = (int)(rh / (NH + NKV));
    const int pos = row % S;
    T* base = (h < NH ? q + (size_t)row * ldq + (size_t)h * HD : k + (size_t)row * ldk + (size_t)(h - NH) * HD) + pv * V;
    const float* t = cs + ((size_t)pos * hd2 + pv * V) * 2;
    float x0[V], x1[V], o0[V], o1[V];
    Vec<T>::load(base, x0);
    Vec<T>::load(base + hd2, x1);
#pragma unroll
    for (int j = 0; j < V; j += 2) {
        const float4 c4 = *reinterpret_cast<const float4*>(t + 2 * j);  // cos_j, sin_j, cos_j+1, sin_j+1
        const float s0 = c4.y * dir, s1 = c4.w * dir;
        o0[j] = x0[j] * c4.x - x1[j] * s0;
        o1[j] = x0[j] * s0 + x1[j] * c4.x;
        o0[j + 1] = x0[j + 1] * c4.z - x1[j + 1] * s1;
        o1[j + 1] = x0[j + 1] * s1 + x1[j + 1] * c4.z;
    }
    Vec<T>::store(base, o0);
    Vec<T>::store(base + hd2, o1);
}
template <typename T>
int rope_apply(T* q, int ldq, T* k, int ldk, const float* cs_table, int rows, int S, int NH, int NKV, int HD, int dir, cudaStream_t st) {
    if (HD % 2) return -1;
    constexpr int V = Vec<T>::N;
    const float d = dir >= 0 ? 1.f : -1.f;
    if ((HD / 2) % V == 0 && ldq % V == 0 && ldk % V == 0 && aligned16(q) && aligned16(k) && aligned16(cs_table)) {
        const long total = (long)rows * (NH + NKV) * (HD / 2 / V);
        rope_vec_kernel<T><<<ceil_div(total, 256), 256, 0, st>>>(q, ldq, k, ldk, cs_table, rows, S, NH, NKV, HD, d);
        return 0;
    }
    const long total = (long)rows * (NH + NKV) * (HD / 2);
    rope_kernel<T><<<ceil_div(total, 256), 256, 0, st>>>(q, ldq, k, ldk, cs_table, rows, S, NH, NKV, HD, d);
    return 0;
}
template int rope_apply<float>(float*, int, float*, int, const float*, int, int, int, int, int, int, cudaStream_t);
template int rope_apply<bf16>(bf16*, int, bf16*, int, const float*, int, int, int, int, int, int, cudaStream_t);

// ------------------------------------------------------------------------------------------------
// SwiGLU: out = gate / (1 + exp(-gate)) * up (reference: swiglu_forward src/kernels/forward.metal:1179,
// swiglu_backward src/kernels/backward.metal:505). gate/up may be the two halves of one packed row.
template <typename T>
__global__ void swiglu_forward_kernel(T* __restrict__ out, int ldo, const T* __restrict__ gate, const T* __restrict__ up, int ldgu,
                                      int rows, int HV) {
    constexpr int V = Vec<T>::N;
    constexpr int U = 2;  // vectors per thread, both requested before either is used
    const long total = (long)rows * HV;
    const long i0 = (blockIdx.x * (long)blockDim.x) * U + threadIdx.x;
    float g[U][V], u[U][V];
    int r[U], c[U];
#pragma unroll
    for (int k = 0; k < U; ++k) {
        const long i = i0 + (long)k * blockDim.x;
        if (i < total) {
            r[k] = (int)(i / HV);
            c[k] = (int)(i - (long)r[k] * HV) * V;
            Vec<T>::load(gate + (size_t)r[k] * ldgu + c[k], g[k]);
            Vec<T>::load(up + (size_t)r[k] * ldgu + c[k], u[k]);
        }
    }
#pragma unroll
    for (int k = 0; k < U; ++k) {
        const long i = i0 + (long)k * blockDim.x;
        if (i < total) {
            float o[V];
#pragma unroll
            for (int j = 0; j < V; ++j) {
                // bf16 output carries 8 mantissa bits: the fast exponential and division are far inside its rounding; the fp32
                // path keeps the exact forms the parity tests compare against
                if (sizeof(T) == 2) o[j] = __fdividef(g[k][j], 1.0f + __expf(-g[k][j])) * u[k][j];
                else o[j] = g[k][j] / (1.0f + expf(-g[k][j])) * u[k][j];
            }
            Vec<T>::store(out + (size_t)r[k] * ldo + c[k], o);
        }
    }
}
template <typename T>
__global__ void swiglu_backward_kernel(T* __restrict__ ggate, T* __restrict__ gup, int ldg, const T* __restrict__ gate,
                                       const T* __restrict__ up, int ldgu, const T* __restrict__ gout, int ldo, int rows, int HV) {
    constexpr int V = Vec<T>::N;
    const long i = blockIdx.x * (long)blockDim.x + threadIdx.x;
    if (i >= (long)rows * HV) return;
    const int r = (int)(i / HV), c = (int)(i - (long)r * HV) * V;
    float x[V], u[V], g[V], dg[V], du[V];
    Vec<T>::load(gate + (size_t)r * ldgu + c, x);
    Vec<T>::load(up + (size_t)r * ldgu + c, u);
    Vec<T>::load(gout + (size_t)r * ldo + c, g);
#pragma unroll
    for (int j = 0; j < V; ++j) {
        const float s = 1.0f / (1.0f + expf(-x[j]));
        dg[j] = g[j] * u[j] * s * (1.0f + x[j] * (1.0f - s));
        du[j] = g[j] * (x[j] * s);
    }
    Vec<T>::store(ggate + (size_t)r * ldg + c, dg);
    Vec<T>::store(gup + (size_t)r * ldg + c, du);
}
template <typename T> int swiglu_forward(T* out, int ldo, const T* gate, const T* up, int ldgu, int rows, int H, cudaStream_t st) {
    constexpr int V = Vec<T>::N;
    if (H % V || ldo % V || ldgu % V || !aligned16(gate) || !aligned16(up) || !aligned16(out)) return -1;
    const long n = (long)rows * (H / V);
    swiglu_forward_kernel<T><<<ceil_div(n, 512), 256, 0, st>>>(out, ldo, gate, up, ldgu, rows, H / V);
    return 0;
}
template <typename T>
int swiglu_backward(T* ggate, T* gup, int ldg, const T* gate, const T* up, int ldgu, const T* gout, int ldo, int rows, int H,
                    cudaStream_t st) {
    constexpr int V = Vec<T>::N;
    if (H % V || ldo % V || ldgu % V || ldg % V || !aligned16(gate) || !aligned16(up) || !aligned16(gout) || !aligned16(ggate) ||
        !aligned16(gup))
        return -1;
    const long n = (long)rows * (H / V);
    swiglu_backward_kernel<T><<<ceil_div(n, 256), 256, 0, st>>>(ggate, gup, ldg, gate, up, ldgu, gout, ldo, rows, H / V);
    return 0;
}
template int swiglu_forward<float>(float*, int, const float*, const float*, int, int, int, cudaStream_t);
template int swiglu_forward<bf16>(bf16*, int, const bf16*, const bf16*, int, int, int, cudaStream_t);
template int swiglu_backward<float>(float*, float*, int, const float*, const float*, int, const float*, int, int, int, cudaStream_t);
template int swiglu_backward<bf16>(bf16*, bf16*, int, const bf16*, const bf16*, int, const bf16*, int, int, int, cudaStream_t);

// Residual add (reference: add_forward src/kernels/forward.metal:1332). The training step fuses the add
// into the GEMM epilogue; this standalone form serves the kernel-name ABI.
template <typename T> __global__ void add_forward_kernel(T* __restrict__ out, const T* __restrict__ a, const T* __restrict__ b, size_t n) {
    const size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if (i < n) out[i] = from_f32<T>(to_f32(a[i]) + to_f32(b[i]));
}
template <typename T> int add_forward(T* out, const T* a, const T* b, size_t n, cudaStream_t st) {
    add_forward_kernel<T><<<ceil_div((long)n, 256), 256, 0, st>>>(out, a, b, n);
    return 0;
}
template int add_forward<float>(float*, const float*, const float*, size_t, cudaStream_t);
template int add_forward<bf16>(bf16*, const bf16*, const bf16*, size_t, cudaStream_t);

// ------------------------------------------------------------------------------------------------
// Softmax cross-entropy, loss and gradient in one kernel, gradient written over the logits
// (reference: host loss loop src/baremetal/scheduler.c:1622-1634 + xent_backward src/kernels/backward.metal:567,
// masked variant :597). One CTA per row: max, then sum exp(x - max), then (p - onehot) * grad_scale.
// The row is read from DRAM once; the later sweeps hit L2.
constexpr int XENT_THREADS = 512;
template <typename T>
__global__ void __launch_bounds__(XENT_THREADS)
xent_kernel(T* __restrict__ logits, float* __restrict__ row_loss, const int* __restrict__ targets, const float* __restrict__ row_weight,
            int V, int ldv, float grad_scale, int* __restrict__ err) {
    constexpr int VN = Vec<T>::N;
    __shared__ float red[XENT_THREADS / 32];
    __shared__ float bcast;
    const int row = blockIdx.x;
    T* lr = logits + (size_t)row * ldv;
    const int nvec = V / VN;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // completion-only loss (xent_backward_masked, src/kernels/backward.metal:597): a row's weight is 1 / (number of unmasked
    // rows of its sequence), or 0 for a masked row (no loss, zero gradient); it replaces the uniform grad_scale.
    if (row_weight) grad_scale = row_weight[row];
    if (row_weight && grad_scale == 0.f) {
        float z[VN];
#pragma unroll
        for (int i = 0; i < VN; ++i) z[i] = 0.f;
        for (int v = threadIdx.x; v < nvec; v += XENT_THREADS) Vec<T>::store(lr + v * VN, z);
        if (threadIdx.x == 0) row_loss[row] = 0.f;
        return;
    }
    float mx = -INFINITY;
    for (int v = threadIdx.x; v < nvec; v += XENT_THREADS) {
        float f[VN];
        Vec<T>::load(lr + v * VN, f);
#pragma unroll
        for (int i = 0; i < VN; ++i) mx = fmaxf(mx, f[i]);
    }
    mx = warp_max(mx);
    if (lane == 0) red[warp] = mx;
    __syncthreads();
    if (warp == 0) {
        float t = lane < XENT_THREADS / 32 ? red[lane] : -INFINITY;
        t = warp_max(t);
        if (lane == 0) bcast = t;
    }
    __syncthreads();
    mx = bcast;
    float sum = 0.f;
    for (int v = threadIdx.x; v < nvec; v += XENT_THREADS) {
        float f[VN];
        Vec<T>::load(lr + v * VN, f);
#pragma unroll
        for (int i = 0; i < VN; ++i) sum += expf(f[i] - mx);
    }
    sum = warp_sum(sum);
    __syncthreads();
    if (lane == 0) red[warp] = sum;
    __syncthreads();
    if (warp == 0) {
        float t = lane < XENT_THREADS / 32 ? red[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) bcast = t;
    }
    __syncthreads();
    sum = bcast;
    const float inv = 1.0f / sum;
    // A target outside [0, V) on a row that counts is never used as an index: the row's loss is 0, its gradient is the plain
    // softmax, and the error word is set (BMB_ERR_BAD_TARGET). Rows with weight 0 never read their target.
    const int tgt = targets[row];
    const bool tgt_ok = (unsigned)tgt < (unsigned)V;
    if (threadIdx.x == 0) {
        const float nll = tgt_ok ? -(to_f32(lr[tgt]) - mx - logf(sum)) : 0.f;
        row_loss[row] = row_weight ? nll * grad_scale : nll;
        if (!tgt_ok && err) atomicExch(err, BMB_ERR_BAD_TARGET);
    }
    __syncthreads();  // the target logit is read before any thread overwrites it
    for (int v = threadIdx.x; v < nvec; v += XENT_THREADS) {
        float f[VN], o[VN];
        Vec<T>::load(lr + v * VN, f);
#pragma unroll
        for (int i = 0; i < VN; ++i) {
            const float p = expf(f[i] - mx) * inv;
            o[i] = (p - ((v * VN + i) == tgt ? 1.0f : 0.0f)) * grad_scale;
        }
        Vec<T>::store(lr + v * VN, o);
    }
}
// bf16 rows of up to 49152 logits are parked in shared memory (96 KB) by the first sweep, so the row is read from memory once and
// written once (the general kernel above reads it three times, twice from L2), and two CTAs share an SM: while one waits for its
// row to arrive the other does its arithmetic. (A variant that kept the row in registers, one CTA per SM, ran at the general
// kernel's speed: load, arithmetic and store phases of the one resident row do not overlap.)
constexpr int XENT_SMEM_MAX_V = 49152;
__device__ __forceinline__ float exp2_fast(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__global__ void __launch_bounds__(XENT_THREADS, 2)
xent_rowsmem_kernel(bf16* __restrict__ logits, float* __restrict__ row_loss, const int* __restrict__ targets,
                    const float* __restrict__ row_weight, int V, int ldv, float grad_scale, int* __restrict__ err) {
    extern __shared__ uint4 xent_row[];   // V / 8 vectors of eight bf16
    __shared__ float red[XENT_THREADS / 32];
    __shared__ float bcast;
    const int row = blockIdx.x;
    bf16* lr = logits + (size_t)row * ldv;
    const int nvec = V / 8;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (row_weight) grad_scale = row_weight[row];
    if (row_weight && grad_scale == 0.f) {   // masked row: zero gradient, zero loss
        for (int v = threadIdx.x; v < nvec; v += XENT_THREADS) *reinterpret_cast<uint4*>(lr + v * 8) = make_uint4(0u, 0u, 0u, 0u);
        if (threadIdx.x == 0) row_loss[row] = 0.f;
        return;
    }
    float mx = -INFINITY;
    for (int v0 = threadIdx.x; v0 < nvec; v0 += 4 * XENT_THREADS) {   // four loads in flight per thread
        uint4 r[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int v = v0 + k * XENT_THREADS;
            if (v < nvec) r[k] = *reinterpret_cast<const uint4*>(lr + v * 8);
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int v = v0 + k * XENT_THREADS;
            if (v < nvec) {
                xent_row[v] = r[k];
                float f[8];
                Vec<bf16>::unpack(r[k], f);
#pragma unroll
                for (int i = 0; i < 8; ++i) mx = fmaxf(mx, f[i]);
            }
        }
    }
    mx = warp_max(mx);
    if (lane == 0) red[warp] = mx;
    __syncthreads();
    if (warp == 0) {
        float t = lane < XENT_THREADS / 32 ? red[lane] : -INFINITY;
        t = warp_max(t);
        if (lane == 0) bcast = t;
    }
    __syncthreads();
    mx = bcast;
    float sum = 0.f;
    // exp(x - max) = 2^(x * log2(e) - max * log2(e)): one FMA and one ex2.approx (relative error 2^-22, far below the bf16 rounding of
    // the gradient) instead of libm's expf, whose two evaluations per element made the kernel arithmetic-bound (1.7 ms for 1.0 ms
    // of memory traffic)
    constexpr float L2E = 1.4426950408889634f;
    const float mxl = -mx * L2E;
    for (int v = threadIdx.x; v < nvec; v += XENT_THREADS) {   // a thread re-reads the vectors it stored itself
        float f[8];
        Vec<bf16>::unpack(xent_row[v], f);
#pragma unroll
        for (int i = 0; i < 8; ++i) sum += exp2_fast(fmaf(f[i], L2E, mxl));
    }
    sum = warp_sum(sum);
    __syncthreads();
    if (lane == 0) red[warp] = sum;
    __syncthreads();
    if (warp == 0) {
        float t = lane < XENT_THREADS / 32 ? red[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) bcast = t;
    }
    __syncthreads();
    sum = bcast;
    const float inv = 1.0f / sum;
    // A target outside [0, V) on a row that counts is never used as an index: the row's loss is 0, its gradient is the plain
    // softmax, and the error word is set.
    const int tgt = targets[row];
    const bool tgt_ok = (unsigned)tgt < (unsigned)V;
    if (threadIdx.x == 0) {
        float nll = 0.f;
        if (tgt_ok) nll = -(__bfloat162float(reinterpret_cast<const bf16*>(xent_row)[tgt]) - mx - logf(sum));
        row_loss[row] = row_weight ? nll * grad_scale : nll;
        if (!tgt_ok && err) atomicExch(err, BMB_ERR_BAD_TARGET);
    }
    const float ps = inv * grad_scale;
    const int tv = tgt_ok ? (tgt >> 3) : -1;
    for (int v = threadIdx.x; v < nvec; v += XENT_THREADS) {
        float f[8], g[8];
        Vec<bf16>::unpack(xent_row[v], f);
#pragma unroll
        for (int i = 0; i < 8; ++i) g[i] = exp2_fast(fmaf(f[i], L2E, mxl)) * ps;
        if (v == tv) g[tgt & 7] -= grad_scale;   // (p - 1) * scale for the target's element
        uint4 o;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int i = 0; i < 8; i += 2) h[i >> 1] = __floats2bfloat162_rn(g[i], g[i + 1]);
        *reinterpret_cast<uint4*>(lr + v * 8) = o;
    }
}

template <typename T>
int xent_forward_backward(T* logits, float* row_loss, const int* targets, const float* row_weight, int N, int V, int ldv, float grad_scale,
                          int* err, cudaStream_t st) {
    if (V % Vec<T>::N || ldv % Vec<T>::N || !aligned16(logits)) return -1;
    if constexpr (sizeof(T) == 2) {
        if (V <= XENT_SMEM_MAX_V) {
            static std::atomic<unsigned long long> attr_done{0};
            if (first_use_on_current_device(attr_done) &&
                cudaFuncSetAttribute(xent_rowsmem_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, XENT_SMEM_MAX_V * 2) != cudaSuccess)
                return -5;
            xent_rowsmem_kernel<<<N, XENT_THREADS, (size_t)V * 2, st>>>(logits, row_loss, targets, row_weight, V, ldv, grad_scale, err);
            return 0;
        }
    }
    xent_kernel<T><<<N, XENT_THREADS, 0, st>>>(logits, row_loss, targets, row_weight, V, ldv, grad_scale, err);
    return 0;
}
template int xent_forward_backward<float>(float*, float*, const int*, const float*, int, int, int, float, int*, cudaStream_t);
template int xent_forward_backward<bf16>(bf16*, float*, const int*, const float*, int, int, int, float, int*, cudaStream_t);

// loss = (1/B) sum_b (1/S) sum_s row_loss[b,s], summed in a fixed order
// (reference: per-sequence mean scheduler.c:1634, batch mean trainer.c:528).
__global__ void loss_reduce_kernel(float* __restrict__ out, const float* __restrict__ row_loss, int B, int S, int weighted) {
    __shared__ float red[32];
    float total = 0.f;
    for (int b = 0; b < B; ++b) {
        float s = 0.f;
        for (int i = threadIdx.x; i < S; i += blockDim.x) s += row_loss[(size_t)b * S + i];
        s = warp_sum(s);
        __syncthreads();
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
        __syncthreads();
        if (threadIdx.x < 32) {
            float t = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
            t = warp_sum(t);
            if (threadIdx.x == 0) total += weighted ? t : t / (float)S;
        }
    }
    if (threadIdx.x == 0) out[0] = total / (float)B;
}
int loss_reduce(float* out, const float* row_loss, int B, int S, int weighted, cudaStream_t st) {
    loss_reduce_kernel<<<1, 1024, 0, st>>>(out, row_loss, B, S, weighted);
    return 0;
}

// ------------------------------------------------------------------------------------------------
// AdamW over one flat parameter range (reference: adamw_step src/anneal/adamw.metal:26 launched per tensor by
// adamw_apply src/baremetal/trainer.c:349-398, followed by a host loop recasting fp32 masters to bf16).
// Every tensor shares the same hyper-parameters — decay included — so the whole model is one launch, and
// the bf16 working copy is written in the same pass.
struct AdamHP { float v[8]; };
template <typename GT>
__global__ void adamw_kernel(float* __restrict__ w, bf16* __restrict__ wb, const GT* __restrict__ g, float* __restrict__ m,
                             float* __restrict__ v, size_t n4, const AdamHP hpv) {
    const float* hp = hpv.v;
    const float lr = hp[0], b1 = hp[1], b2 = hp[2], eps = hp[3], wd = hp[4], bias1 = hp[5], bias2 = hp[6], gs = hp[7];
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
        float4 wv = reinterpret_cast<float4*>(w)[i];
        float4 mv = reinterpret_cast<float4*>(m)[i];
        float4 vv = reinterpret_cast<float4*>(v)[i];
        float gg[4];
        if constexpr (sizeof(GT) == 4) {
            const float4 t = reinterpret_cast<const float4*>(g)[i];
            gg[0] = t.x; gg[1] = t.y; gg[2] = t.z; gg[3] = t.w;
        } else {
            const uint2 t = reinterpret_cast<const uint2*>(g)[i];
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&t);
            const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
            gg[0] = a.x; gg[1] = a.y; gg[2] = b.x; gg[3] = b.y;
        }
        float* wp = &wv.x; float* mp = &mv.x; float* vp = &vv.x;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float gi = gg[j] * gs;
            const float mn = b1 * mp[j] + (1.0f - b1) * gi;
            const float vn = b2 * vp[j] + (1.0f - b2) * gi * gi;
            mp[j] = mn;
            vp[j] = vn;
            const float mh = mn / bias1, vh = vn / bias2;
            wp[j] = wp[j] * (1.0f - lr * wd) - lr * mh / (sqrtf(vh) + eps);
        }
        reinterpret_cast<float4*>(w)[i] = wv;
        reinterpret_cast<float4*>(m)[i] = mv;
        reinterpret_cast<float4*>(v)[i] = vv;
        if (wb) {
            uint2 o;
            __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&o);
            h[0] = __floats2bfloat162_rn(wv.x, wv.y);
            h[1] = __floats2bfloat162_rn(wv.z, wv.w);
            reinterpret_cast<uint2*>(wb)[i] = o;
        }
    }
}
template <typename GT> static int adamw_launch(float* w, bf16* wb, const GT* g, float* m, float* v, size_t n, const float* hp, cudaStream_t st) {
    if (n % 4 || !aligned16(w) || !aligned16(m) || !aligned16(v) || (((uintptr_t)g) & (sizeof(GT) * 4 - 1)) || (((uintptr_t)wb) & 7))
        return -1;
    const size_t n4 = n / 4;
    long blocks = (long)((n4 + 255) / 256);
    if (blocks > 148 * 16) blocks = 148 * 16;
    AdamHP hpv;
    for (int i = 0; i < 8; ++i) hpv.v[i] = hp[i];  // hp is a HOST pointer; the values travel as kernel arguments
    adamw_kernel<GT><<<(int)blocks, 256, 0, st>>>(w, wb, g, m, v, n4, hpv);
    return 0;
}
int adamw_f32grad(float* w, bf16* wb, const float* g, float* m, float* v, size_t n, const float* hp, cudaStream_t st) {
    return adamw_launch<float>(w, wb, g, m, v, n, hp, st);
}
int adamw_bf16grad(float* w, bf16* wb, const bf16* g, float* m, float* v, size_t n, const float* hp, cudaStream_t st) {
    return adamw_launch<bf16>(w, wb, g, m, v, n, hp, st);
}

// ------------------------------------------------------------------------------------------------
__global__ void cast_f32_bf16_kernel(bf16* __restrict__ out, const float* __restrict__ in, size_t n) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        out[i] = __float2bfloat16_rn(in[i]);
}
__global__ void cast_bf16_f32_kernel(float* __restrict__ out, const bf16* __restrict__ in, size_t n) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        out[i] = __bfloat162float(in[i]);
}
int cast_f32_to_bf16(bf16* out, const float* in, size_t n, cudaStream_t st) {
    long blocks = (long)((n + 255) / 256);
    if (blocks > 148 * 32) blocks = 148 * 32;
    if (blocks > 0) cast_f32_bf16_kernel<<<(int)blocks, 256, 0, st>>>(out, in, n);
    return 0;
}
int cast_bf16_to_f32(float* out, const bf16* in, size_t n, cudaStream_t st) {
    long blocks = (long)((n + 255) / 256);
    if (blocks > 148 * 32) blocks = 148 * 32;
    if (blocks > 0) cast_bf16_f32_kernel<<<(int)blocks, 256, 0, st>>>(out, in, n);
    return 0;
}

// Running sum over the sequences of a batch: x[b] <- carry + x[0] + ... + x[b], carry <- x[B-1] (new value).
// Reproduces what the reference's layer-0 input gradient holds when its embedding scatter runs for
// sequence b: that gradient buffer is excluded from slot pooling (src/baremetal/scheduler.c:263-266) and is
// cleared only at the start of an optimizer window (src/baremetal/trainer.c:459-470), so it still contains the
// sum over the window's earlier sequences.
template <typename T>
__global__ void seq_prefix_accumulate_kernel(T* __restrict__ x, float* __restrict__ carry, int B, size_t per_seq) {
    const size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if (i >= per_seq) return;
    float c = carry[i];
    for (int b = 0; b < B; ++b) {
        c += to_f32(x[(size_t)b * per_seq + i]);
        x[(size_t)b * per_seq + i] = from_f32<T>(c);
    }
    carry[i] = c;
}
template <typename T> int seq_prefix_accumulate(T* x, float* carry, int B, size_t per_seq, cudaStream_t st) {
    seq_prefix_accumulate_kernel<T><<<ceil_div((long)per_seq, 256), 256, 0, st>>>(x, carry, B, per_seq);
    return 0;
}
template int seq_prefix_accumulate<float>(float*, float*, int, size_t, cudaStream_t);
template int seq_prefix_accumulate<bf16>(bf16*, float*, int, size_t, cudaStream_t);

// Greedy sampler: lowest index among the maxima (reference: bm_sample argmax branch, src/baremetal/sampler.c:36-40).
__global__ void argmax_first_kernel(int* __restrict__ out, const float* __restrict__ logits, int V) {
    __shared__ float sv[32];
    __shared__ int si[32];
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float x = logits[i];
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
        if (threadIdx.x == 0) out[0] = bi == 0x7fffffff ? 0 : bi;
    }
}
int argmax_first(int* out_index, const float* logits, int V, cudaStream_t st) {
    argmax_first_kernel<<<1, 1024, 0, st>>>(out_index, logits, V);
    return 0;
}

}  // namespace bmb
