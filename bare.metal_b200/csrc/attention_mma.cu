// bf16 causal GQA flash attention on the warp-level tensor-core path (mma.sync m16n8k16, ldmatrix,
// cp.async double buffering), head_dim 64. It replaces the reference's tiled training attention
// (attention_forward_train_tiled src/kernels/forward.metal:2122, attention_backward_tiled
// src/kernels/backward.metal:820): same online-softmax recurrence, scores never leave the SM.
//
// Layout: Q[row, h, :] at q + row*ldq + h*64, K/V[row, kh, :] with pitch ldkv, row = b*S + s,
// kh = h / (NH/NKV). Tiles are 64 queries x 64 keys; shared-memory tiles are [64][64] bf16 with the
// 16-byte chunk index XOR-swizzled by (row & 7) so ldmatrix is bank-conflict free.
//
// Backward is organised by key/value block: one CTA owns 64 keys of one KV head, keeps dK and dV in
// registers while it sweeps every query block at or after it of every query head that shares the
// KV head, and writes them once (no atomics, deterministic). dQ contributions are accumulated in an
// fp32 scratch with vector reductions and cast to bf16 afterwards.
#include "attention_mma.cuh"

namespace bmb {

namespace {

constexpr int HD64 = 64;
constexpr int BQ = 64;   // queries per tile
constexpr int BKV = 64;  // keys per tile
constexpr int TILE_BYTES = 64 * 128;
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ uint32_t swz(int r, int c) { return (uint32_t)(r * 128 + ((c ^ (r & 7)) << 4)); }
__device__ __forceinline__ uint32_t s_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(uint32_t saddr, const void* g, bool pred) {
    const int n = pred ? 16 : 0;  // src-size 0 -> the 16 destination bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(saddr), "l"(g), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldsm4(uint32_t (&r)[4], uint32_t saddr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(saddr));
}
__device__ __forceinline__ void ldsm4t(uint32_t (&r)[4], uint32_t saddr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(saddr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

// Copy a [64][64] bf16 tile (rows row0.. of a matrix with pitch ld) into swizzled shared memory.
// Rows at or beyond `rows_valid` are zero-filled.
__device__ __forceinline__ void load_tile_async(uint8_t* smem, const bf16* g, int ld, int rows_valid, int tid, int nthreads) {
    const uint32_t base = s_u32(smem);
    for (int i = tid; i < 64 * 8; i += nthreads) {
        const int r = i >> 3, c = i & 7;
        const bool ok = r < rows_valid;
        cp_async16(base + swz(r, c), g + (size_t)(ok ? r : 0) * ld + c * 8, ok);
    }
}

// ================================ forward ===================================================
__global__ void __launch_bounds__(128)
flash_fwd_kernel(bf16* __restrict__ out, int ldo, float* __restrict__ lse, const bf16* __restrict__ q, int ldq,
                 const bf16* __restrict__ k, const bf16* __restrict__ v, int ldkv, int S, int NH, int NKV, float scale) {
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* Qs = smem;                   // 8 KB
    uint8_t* Ks = smem + TILE_BYTES;      // 2 x 8 KB
    uint8_t* Vs = smem + 3 * TILE_BYTES;  // 2 x 8 KB
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    // heaviest (latest) query blocks first
    const int mblk = (int)gridDim.x - 1 - (int)blockIdx.x;
    const int h = blockIdx.y, b = blockIdx.z;
    const int kh = h / (NH / NKV);
    const int q0 = mblk * BQ;
    const size_t row_base = (size_t)b * S;
    const bf16* qg = q + (row_base + q0) * ldq + (size_t)h * HD64;
    const bf16* kg = k + row_base * ldkv + (size_t)kh * HD64;
    const bf16* vg = v + row_base * ldkv + (size_t)kh * HD64;

    load_tile_async(Qs, qg, ldq, S - q0, tid, 128);
    load_tile_async(Ks, kg, ldkv, S, tid, 128);
    load_tile_async(Vs, vg, ldkv, S, tid, 128);
    cp_async_commit();

    const float sl2 = scale * LOG2E;
    float o[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) o[i][j] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    uint32_t qf[4][4];

    const int nblk = mblk + 1;  // causal: key blocks 0..mblk
    for (int n = 0; n < nblk; ++n) {
        const int buf = n & 1;
        if (n + 1 < nblk) {
            const int k0n = (n + 1) * BKV;
            load_tile_async(Ks + (buf ^ 1) * TILE_BYTES, kg + (size_t)k0n * ldkv, ldkv, S - k0n, tid, 128);
            load_tile_async(Vs + (buf ^ 1) * TILE_BYTES, vg + (size_t)k0n * ldkv, ldkv, S - k0n, tid, 128);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if (n == 0) {
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) ldsm4(qf[ks], s_u32(Qs) + swz(16 * warp + (lane & 15), 2 * ks + (lane >> 4)));
        }
        const uint32_t ksb = s_u32(Ks + buf * TILE_BYTES), vsb = s_u32(Vs + buf * TILE_BYTES);
        float s[8][4];
#pragma unroll
        for (int nb = 0; nb < 8; ++nb) {
#pragma unroll
            for (int j = 0; j < 4; ++j) s[nb][j] = 0.f;
#pragma unroll
            for (int kp = 0; kp < 2; ++kp) {
                uint32_t kf[4];
                ldsm4(kf, ksb + swz(8 * nb + (lane & 7), 4 * kp + (lane >> 3)));
                mma16816(s[nb], qf[2 * kp], kf[0], kf[1]);
                mma16816(s[nb], qf[2 * kp + 1], kf[2], kf[3]);
            }
        }
        const int k0 = n * BKV;
        const bool need_mask = (n == mblk) || (k0 + BKV > S);
        if (need_mask) {
#pragma unroll
            for (int nb = 0; nb < 8; ++nb)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int qi = q0 + 16 * warp + g + ((j >> 1) << 3);
                    const int kj = k0 + 8 * nb + 2 * t + (j & 1);
                    if (kj > qi || kj >= S) s[nb][j] = -INFINITY;
                }
        }
        float mx[2] = {m_run[0], m_run[1]};
#pragma unroll
        for (int nb = 0; nb < 8; ++nb) {
            mx[0] = fmaxf(mx[0], fmaxf(s[nb][0], s[nb][1]));
            mx[1] = fmaxf(mx[1], fmaxf(s[nb][2], s[nb][3]));
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        }
        float corr[2], mb[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mb[r] = (mx[r] == -INFINITY) ? 0.f : mx[r] * sl2;
            corr[r] = (m_run[r] == -INFINITY) ? 0.f : exp2f(m_run[r] * sl2 - mb[r]);
            m_run[r] = mx[r];
            l_run[r] *= corr[r];
        }
#pragma unroll
        for (int nb = 0; nb < 8; ++nb) {
            o[nb][0] *= corr[0]; o[nb][1] *= corr[0];
            o[nb][2] *= corr[1]; o[nb][3] *= corr[1];
        }
        uint32_t pa[4][4];
#pragma unroll
        for (int nb = 0; nb < 8; ++nb) {
            const float p0 = exp2f(s[nb][0] * sl2 - mb[0]), p1 = exp2f(s[nb][1] * sl2 - mb[0]);
            const float p2 = exp2f(s[nb][2] * sl2 - mb[1]), p3 = exp2f(s[nb][3] * sl2 - mb[1]);
            l_run[0] += p0 + p1;
            l_run[1] += p2 + p3;
            pa[nb >> 1][(nb & 1) * 2] = pack_bf16(p0, p1);
            pa[nb >> 1][(nb & 1) * 2 + 1] = pack_bf16(p2, p3);
        }
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
            for (int dp = 0; dp < 4; ++dp) {
                uint32_t vf[4];
                ldsm4t(vf, vsb + swz(16 * kk + (lane & 7) + ((lane >> 3) & 1) * 8, 2 * dp + (lane >> 4)));
                mma16816(o[2 * dp], pa[kk], vf[0], vf[1]);
                mma16816(o[2 * dp + 1], pa[kk], vf[2], vf[3]);
            }
        }
        __syncthreads();  // everyone is done with this K/V buffer before it is refilled
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int qi = q0 + 16 * warp + g + 8 * r;
        if (qi >= S) continue;
        const float inv = l_run[r] > 0.f ? 1.0f / l_run[r] : 0.f;
        bf16* orow = out + (row_base + qi) * ldo + (size_t)h * HD64;
#pragma unroll
        for (int nb = 0; nb < 8; ++nb)
            *reinterpret_cast<uint32_t*>(orow + 8 * nb + 2 * t) = pack_bf16(o[nb][2 * r] * inv, o[nb][2 * r + 1] * inv);
        if (t == 0) lse[((size_t)b * NH + h) * S + qi] = l_run[r] > 0.f ? m_run[r] * scale + logf(l_run[r]) : -INFINITY;
    }
}

// ================================ backward ==================================================
// delta[b, h, s] = sum_d gout * out. One warp per (row, head).
__global__ void flash_delta_kernel(float* __restrict__ delta, const bf16* __restrict__ gout, const bf16* __restrict__ out, int ldo,
                                   int B, int S, int NH) {
    const long wid = (blockIdx.x * (long)blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (wid >= (long)B * S * NH) return;
    const int h = (int)(wid % NH);
    const long row = wid / NH;
    const bf16* gr = gout + row * ldo + (size_t)h * HD64;
    const bf16* orr = out + row * ldo + (size_t)h * HD64;
    const __nv_bfloat162 a = reinterpret_cast<const __nv_bfloat162*>(gr)[lane];
    const __nv_bfloat162 c = reinterpret_cast<const __nv_bfloat162*>(orr)[lane];
    const float2 fa = __bfloat1622float2(a), fc = __bfloat1622float2(c);
    const float d = warp_sum(fa.x * fc.x + fa.y * fc.y);
    if (lane == 0) {
        const int b = (int)(row / S), s = (int)(row % S);
        delta[((size_t)b * NH + h) * S + s] = d;
    }
}

__global__ void __launch_bounds__(128)
flash_bwd_kernel(float* __restrict__ dq_acc, bf16* __restrict__ gk, bf16* __restrict__ gv, int ldgkv, const bf16* __restrict__ gout,
                 int ldo, const float* __restrict__ lse, const float* __restrict__ delta, const bf16* __restrict__ q, int ldq,
                 const bf16* __restrict__ k, const bf16* __restrict__ v, int ldkv, int S, int NH, int NKV, float scale) {
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* Ks = smem;
    uint8_t* Vs = smem + TILE_BYTES;
    uint8_t* Qs = smem + 2 * TILE_BYTES;   // 2 stages
    uint8_t* Gs = smem + 4 * TILE_BYTES;   // 2 stages (gout tiles)
    uint8_t* Ds = smem + 6 * TILE_BYTES;   // dS^T tile [key][query]
    float* s_lse = reinterpret_cast<float*>(smem + 7 * TILE_BYTES);  // [2][64], already multiplied by log2(e)
    float* s_delta = s_lse + 128;                                    // [2][64]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int nblk = blockIdx.x, kh = blockIdx.y, b = blockIdx.z;
    const int mul = NH / NKV;
    const int QD = NH * HD64;
    const int n0 = nblk * BKV;
    const int nqb = (S + BQ - 1) / BQ;
    const size_t row_base = (size_t)b * S;
    const float sl2 = scale * LOG2E;

    load_tile_async(Ks, k + (row_base + n0) * ldkv + (size_t)kh * HD64, ldkv, S - n0, tid, 128);
    load_tile_async(Vs, v + (row_base + n0) * ldkv + (size_t)kh * HD64, ldkv, S - n0, tid, 128);
    cp_async_commit();

    const int per_head = nqb - nblk;  // query blocks nblk .. nqb-1
    const int total = mul * per_head;
    auto issue = [&](int it) {
        const int hl = it / per_head, mb = nblk + (it - hl * per_head);
        const int h = kh * mul + hl, q0 = mb * BQ, buf = it & 1;
        load_tile_async(Qs + buf * TILE_BYTES, q + (row_base + q0) * ldq + (size_t)h * HD64, ldq, S - q0, tid, 128);
        load_tile_async(Gs + buf * TILE_BYTES, gout + (row_base + q0) * ldo + (size_t)h * HD64, ldo, S - q0, tid, 128);
        if (tid < 64) {
            const int qi = q0 + tid;
            const size_t idx = ((size_t)b * NH + h) * S + qi;
            // rows past the end get lse = +inf so that their probabilities vanish
            s_lse[buf * 64 + tid] = qi < S ? lse[idx] * LOG2E : INFINITY;
            s_delta[buf * 64 + tid] = qi < S ? delta[idx] : 0.f;
        }
        cp_async_commit();
    };
    if (total > 0) issue(0);

    float dk[8][4], dv[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) { dk[i][j] = 0.f; dv[i][j] = 0.f; }
    uint32_t kfa[4][4], vfa[4][4];

    for (int it = 0; it < total; ++it) {
        const int buf = it & 1;
        if (it + 1 < total) { issue(it + 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
        __syncthreads();
        if (it == 0) {
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                ldsm4(kfa[ks], s_u32(Ks) + swz(16 * warp + (lane & 15), 2 * ks + (lane >> 4)));
                ldsm4(vfa[ks], s_u32(Vs) + swz(16 * warp + (lane & 15), 2 * ks + (lane >> 4)));
            }
        }
        const int hl = it / per_head, mb = nblk + (it - hl * per_head);
        const int h = kh * mul + hl, q0 = mb * BQ;
        const uint32_t qsb = s_u32(Qs + buf * TILE_BYTES), gsb = s_u32(Gs + buf * TILE_BYTES);
        const float* lse_s = s_lse + buf * 64;
        const float* delta_s = s_delta + buf * 64;

        // S^T = K_w Q^T  and  dP^T = V_w dO^T : [16 keys of this warp] x [64 queries]
        float st[8][4], dpt[8][4];
#pragma unroll
        for (int nb = 0; nb < 8; ++nb) {
#pragma unroll
            for (int j = 0; j < 4; ++j) { st[nb][j] = 0.f; dpt[nb][j] = 0.f; }
#pragma unroll
            for (int kp = 0; kp < 2; ++kp) {
                uint32_t f[4];
                ldsm4(f, qsb + swz(8 * nb + (lane & 7), 4 * kp + (lane >> 3)));
                mma16816(st[nb], kfa[2 * kp], f[0], f[1]);
                mma16816(st[nb], kfa[2 * kp + 1], f[2], f[3]);
                ldsm4(f, gsb + swz(8 * nb + (lane & 7), 4 * kp + (lane >> 3)));
                mma16816(dpt[nb], vfa[2 * kp], f[0], f[1]);
                mma16816(dpt[nb], vfa[2 * kp + 1], f[2], f[3]);
            }
        }
        // P^T = exp(scale*S^T - lse[q]);  dS^T = P^T * (dP^T - delta[q]) * scale
        uint32_t pa[4][4], dsa[4][4];
        const bool diag = (mb == nblk);
#pragma unroll
        for (int nb = 0; nb < 8; ++nb) {
            float p[4], ds[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int kl = 16 * warp + g + ((j >> 1) << 3);  // key within the tile
                const int ql = 8 * nb + 2 * t + (j & 1);         // query within the tile
                float pj = exp2f(st[nb][j] * sl2 - lse_s[ql]);
                if ((diag && kl > ql) || (n0 + kl >= S)) pj = 0.f;
                p[j] = pj;
                ds[j] = pj * (dpt[nb][j] - delta_s[ql]) * scale;
            }
            pa[nb >> 1][(nb & 1) * 2] = pack_bf16(p[0], p[1]);
            pa[nb >> 1][(nb & 1) * 2 + 1] = pack_bf16(p[2], p[3]);
            const uint32_t d01 = pack_bf16(ds[0], ds[1]), d23 = pack_bf16(ds[2], ds[3]);
            dsa[nb >> 1][(nb & 1) * 2] = d01;
            dsa[nb >> 1][(nb & 1) * 2 + 1] = d23;
            // dS^T to shared memory as [key][query] for the dQ product below
            *reinterpret_cast<uint32_t*>(Ds + swz(16 * warp + g, nb) + 4 * t) = d01;
            *reinterpret_cast<uint32_t*>(Ds + swz(16 * warp + g + 8, nb) + 4 * t) = d23;
        }
        // dV += P^T dO ; dK += dS^T Q   (reduction over the 64 queries)
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
            for (int dp = 0; dp < 4; ++dp) {
                uint32_t f[4];
                const uint32_t off = swz(16 * kk + (lane & 7) + ((lane >> 3) & 1) * 8, 2 * dp + (lane >> 4));
                ldsm4t(f, gsb + off);
                mma16816(dv[2 * dp], pa[kk], f[0], f[1]);
                mma16816(dv[2 * dp + 1], pa[kk], f[2], f[3]);
                ldsm4t(f, qsb + off);
                mma16816(dk[2 * dp], dsa[kk], f[0], f[1]);
                mma16816(dk[2 * dp + 1], dsa[kk], f[2], f[3]);
            }
        }
        __syncthreads();  // dS^T tile complete
        // dQ[16 queries of this warp] += dS[q, keys] K[keys, :]
        float dq[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) dq[i][j] = 0.f;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
            uint32_t a[4];
            ldsm4t(a, s_u32(Ds) + swz(16 * ks + (lane & 7) + (lane >> 4) * 8, 2 * warp + ((lane >> 3) & 1)));
#pragma unroll
            for (int dp = 0; dp < 4; ++dp) {
                uint32_t f[4];
                ldsm4t(f, s_u32(Ks) + swz(16 * ks + (lane & 7) + ((lane >> 3) & 1) * 8, 2 * dp + (lane >> 4)));
                mma16816(dq[2 * dp], a, f[0], f[1]);
                mma16816(dq[2 * dp + 1], a, f[2], f[3]);
            }
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int qi = q0 + 16 * warp + g + 8 * r;
            if (qi < S) {
                float* dst = dq_acc + (row_base + qi) * QD + (size_t)h * HD64 + 2 * t;
#pragma unroll
                for (int nb = 0; nb < 8; ++nb)
                    asm volatile("red.global.add.v2.f32 [%0], {%1, %2};" ::"l"(dst + 8 * nb), "f"(dq[nb][2 * r]), "f"(dq[nb][2 * r + 1])
                                 : "memory");
            }
        }
        __syncthreads();  // Ds and this Q/dO stage may be overwritten next
    }
    if (total == 0) { cp_async_wait<0>(); }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int kj = n0 + 16 * warp + g + 8 * r;
        if (kj >= S) continue;
        bf16* gkr = gk + (row_base + kj) * ldgkv + (size_t)kh * HD64;
        bf16* gvr = gv + (row_base + kj) * ldgkv + (size_t)kh * HD64;
#pragma unroll
        for (int nb = 0; nb < 8; ++nb) {
            *reinterpret_cast<uint32_t*>(gkr + 8 * nb + 2 * t) = pack_bf16(dk[nb][2 * r], dk[nb][2 * r + 1]);
            *reinterpret_cast<uint32_t*>(gvr + 8 * nb + 2 * t) = pack_bf16(dv[nb][2 * r], dv[nb][2 * r + 1]);
        }
    }
}

__global__ void cast_rows_kernel(bf16* __restrict__ out, int ldo, const float* __restrict__ in, int ldi, int rows, int cols4) {
    const long i = blockIdx.x * (long)blockDim.x + threadIdx.x;
    if (i >= (long)rows * cols4) return;
    const int r = (int)(i / cols4), c = (int)(i - (long)r * cols4) * 4;
    const float4 v = *reinterpret_cast<const float4*>(in + (size_t)r * ldi + c);
    uint2 o;
    o.x = pack_bf16(v.x, v.y);
    o.y = pack_bf16(v.z, v.w);
    *reinterpret_cast<uint2*>(out + (size_t)r * ldo + c) = o;
}

constexpr int FWD_SMEM = 5 * TILE_BYTES;
constexpr int BWD_SMEM = 7 * TILE_BYTES + 4 * 64 * (int)sizeof(float);

bool aligned_for_tiles(const void* p, int ld) { return ((((uintptr_t)p) & 15) == 0) && (ld % 8 == 0); }

}  // namespace

bool flash_attention_supported(int HD, int NH, int NKV, bool has_mask) {
    return HD == 64 && !has_mask && NKV > 0 && NH % NKV == 0;
}

int flash_attention_forward(bf16* out, int ldo, float* lse, const bf16* q, int ldq, const bf16* k, const bf16* v, int ldkv, int B, int S,
                            int NH, int NKV, int HD, float scale, cudaStream_t st) {
    if (!flash_attention_supported(HD, NH, NKV, false)) return -1;
    if (!aligned_for_tiles(q, ldq) || !aligned_for_tiles(k, ldkv) || !aligned_for_tiles(v, ldkv) || (ldo % 2) || (((uintptr_t)out) & 3))
        return -2;
    static bool attr_done = false;
    if (!attr_done) {
        cudaFuncSetAttribute(flash_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FWD_SMEM);
        attr_done = true;
    }
    dim3 grid((S + BQ - 1) / BQ, NH, B);
    flash_fwd_kernel<<<grid, 128, FWD_SMEM, st>>>(out, ldo, lse, q, ldq, k, v, ldkv, S, NH, NKV, scale);
    return 0;
}

size_t flash_attention_backward_scratch_bytes(int B, int S, int NH, int HD) {
    return (size_t)B * S * NH * HD * sizeof(float) + (size_t)B * NH * S * sizeof(float);
}

int flash_attention_backward(bf16* gq, int ldgq, bf16* gk, bf16* gv, int ldgkv, const bf16* gout, int ldo, const bf16* out,
                             const float* lse, const bf16* q, int ldq, const bf16* k, const bf16* v, int ldkv, int B, int S, int NH,
                             int NKV, int HD, float scale, void* scratch, cudaStream_t st) {
    if (!flash_attention_supported(HD, NH, NKV, false)) return -1;
    if (!aligned_for_tiles(q, ldq) || !aligned_for_tiles(k, ldkv) || !aligned_for_tiles(v, ldkv) || !aligned_for_tiles(gout, ldo) ||
        (ldgkv % 2) || (ldgq % 4) || (((uintptr_t)gq) & 7) || (((uintptr_t)gk) & 3) || (((uintptr_t)gv) & 3) || (((uintptr_t)out) & 3))
        return -2;
    static bool attr_done = false;
    if (!attr_done) {
        cudaFuncSetAttribute(flash_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BWD_SMEM);
        attr_done = true;
    }
    const size_t rows = (size_t)B * S;
    const int QD = NH * HD;
    float* dq_acc = (float*)scratch;
    float* delta = dq_acc + rows * QD;
    cudaMemsetAsync(dq_acc, 0, rows * QD * sizeof(float), st);
    const long warps = (long)rows * NH;
    flash_delta_kernel<<<(int)((warps * 32 + 255) / 256), 256, 0, st>>>(delta, gout, out, ldo, B, S, NH);
    dim3 grid((S + BKV - 1) / BKV, NKV, B);
    flash_bwd_kernel<<<grid, 128, BWD_SMEM, st>>>(dq_acc, gk, gv, ldgkv, gout, ldo, lse, delta, q, ldq, k, v, ldkv, S, NH, NKV, scale);
    return cast_rows_f32_to_bf16(gq, ldgq, dq_acc, QD, (int)rows, QD, st);
}

int cast_rows_f32_to_bf16(bf16* out, int ldo, const float* in, int ldi, int rows, int cols, cudaStream_t st) {
    if (cols % 4 || ldi % 4 || ldo % 4 || (((uintptr_t)out) & 7) || (((uintptr_t)in) & 15)) return -1;
    const long n = (long)rows * (cols / 4);
    cast_rows_kernel<<<(int)((n + 255) / 256), 256, 0, st>>>(out, ldo, in, ldi, rows, cols / 4);
    return 0;
}

}  // namespace bmb
