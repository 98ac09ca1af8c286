// bf16 causal GQA flash attention on the sm_100a tensor cores (tcgen05.mma with TMEM accumulators, TMA-fed
// operand tiles), head_dim 64. Forward pass.
//
// One CTA = 256 consecutive queries of one head, handled as two tiles X = A, B of 128 queries that share every K/V
// tile. For each tile of 128 keys up to the diagonal and each X:
//   S_X = Q_X K^T        UMMA 128x128x64, A = Q_X (K-major smem), B = K tile (K-major smem), accumulator in TMEM
//   softmax              one warpgroup per X, one thread per query row: the S row is pulled into registers,
//                        running max / sum in the log2 domain, P written back to TMEM as packed bf16 pairs
//                        (tcgen05.st, 64 columns per tile: P never touches shared memory);
//                        O_X in TMEM is rescaled only when the row maximum grew by more than 2^8 since the value the
//                        accumulator is referenced to (the stale reference cancels in the final division)
//   O_X += P_X V         UMMA 128x64x128, A = P_X read from TMEM (lane = query row, column = key pair), B = V tile
//                        (MN-major smem: the reduction index, the key, is the row of V), accumulator in TMEM
// The single UMMA-issuing thread interleaves the two tiles (PV_A(j), QK_A(j+1), PV_B(j), QK_B(j+1), ...) so that
// the tensor core works on one tile while the other tile's warpgroup does its softmax. K/V tiles are
// in a four-stage ring filled by a TMA producer warp. 12 warps: TMA, UMMA, two idle (they complete the control warpgroup), 4 + 4 softmax.
// Reference: attention_forward_train_tiled, src/kernels/forward.metal:2122: out = softmax(scale * Q K^T, causal) V and
// lse = log-sum-exp of the scaled scores.
#include <cuda.h>
#include <stdio.h>
#include <stdlib.h>

#include "attention_umma.cuh"
#include "ptx_sm100.cuh"

namespace bmb {

namespace {

constexpr int FQ = 128;   // queries per tile (two tiles per CTA)
constexpr int FK = 128;   // keys per tile
constexpr int FHD = 64;
constexpr int Q_BYTES = FQ * FHD * 2;        // 16 KB per Q tile
constexpr int KV_TILE_BYTES = FK * FHD * 2;  // 16 KB each for K and V
constexpr int P_BYTES = FQ * FK * 2;         // 32 KB per P tile
// K/V stages: a stage is refilled only after every UMMA that read it has completed, and the refill (32 KB from L2) takes over a
// thousand clocks, so with two stages S of key tile j+2 waited for the load that P V of tile j had just released. Four
// stages put the load two tiles ahead of its use.
constexpr int FWD_KV_STAGES = 4;
constexpr int FWD_DYN_SMEM = 2 * Q_BYTES + FWD_KV_STAGES * 2 * KV_TILE_BYTES + 1024;  // Q x 2 tiles, K and V stages; P lives in tensor memory
constexpr int FWD_THREADS = 384;  // warpgroup 0: TMA warp, UMMA warp, two idle warps; warpgroups 1 and 2: softmax of tile A and tile B
// Register budget: 3 warps per scheduler cap the kernel at 168 registers per thread. The control warpgroup hands most of
// its share back (setmaxnreg.dec) and the two softmax warpgroups, which hold a 128-column score row per thread, take it
// (setmaxnreg.inc): 128 x 72 + 256 x 216 = 384 x 168.
constexpr int FWD_REGS_CONTROL = 72, FWD_REGS_SOFTMAX = 216;
constexpr uint32_t FWD_TMEM_COLS = 512;  // S_A [0,128) S_B [128,256) O_A [256,320) O_B [320,384) P_A [384,448) P_B [448,512)
constexpr uint32_t FWD_TMEM_P = 2 * FK + 2 * FHD;  // P as packed bf16 pairs: 128 keys = 64 columns per query tile
constexpr float LOG2E_F = 1.4426950408889634f;
constexpr float RESCALE_THRESHOLD = 8.0f;  // log2 units

struct __align__(8) FwdBars {
    uint64_t q_full, kv_full[FWD_KV_STAGES], kv_empty[FWD_KV_STAGES], s_full[2], s_free[2], p_ready[2], pv_done[2];
    uint32_t tmem_base;
    int abort_flag;
};

__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
        "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
        "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]),
        "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// Blackwell's three-input max and packed two-wide fp32 arithmetic: half the issue slots of the scalar forms.
__device__ __forceinline__ float max3_f(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
// (d0, d1) = (a0, a1) * b + c
__device__ __forceinline__ void fma2_f(float& d0, float& d1, float a0, float a1, float b, float c) {
    asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %4};\n\tmov.b64 rc, {%5, %5};\n\t"
        "fma.rn.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(d0), "=f"(d1)
        : "f"(a0), "f"(a1), "f"(b), "f"(c));
}
// (d0, d1) += (a0, a1)
__device__ __forceinline__ void add2_f(float& d0, float& d1, float a0, float a1) {
    asm("{\n\t.reg .b64 ra, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rd, {%0, %1};\n\tadd.rn.f32x2 rd, rd, ra;\n\tmov.b64 {%0, %1}, rd;\n\t}"
        : "+f"(d0), "+f"(d1)
        : "f"(a0), "f"(a1));
}
// (d0, d1) = (a0, a1) * (b0, b1)
__device__ __forceinline__ void mul2_f(float& d0, float& d1, float a0, float a1, float b0, float b1) {
    asm("{\n\t.reg .b64 ra, rb, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tmul.rn.f32x2 rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(d0), "=f"(d1)
        : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
}
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

struct FwdArgs {
    bf16* out;
    int ldo;
    float* lse;
    const uint32_t* keymask;   // [B][ceil(S / 32)] bit i of word w = position 32 * w + i takes part (null: every position does)
    int S, NH, NKV;
    float scale;
    int* err;
};


// MASKED = false: no padding mask (the plain training step); the mask words, their loads and the per-element tests are compiled out
template <bool MASKED>
__global__ void __launch_bounds__(FWD_THREADS, 1)
flash_fwd_umma_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV, const FwdArgs p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ FwdBars bars;
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* sQ = smem;                          // 2 tiles
    uint8_t* sK = sQ + 2 * Q_BYTES;              // FWD_KV_STAGES stages
    uint8_t* sV = sK + FWD_KV_STAGES * KV_TILE_BYTES;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int qb = (int)gridDim.x - 1 - (int)blockIdx.x;  // latest (longest) query blocks first
    const int h = blockIdx.y, b = blockIdx.z;
    const int kh = h / (p.NH / p.NKV);
    const int q0 = qb * 2 * FQ;        // first query of tile A; tile B starts FQ later
    const int row0 = b * p.S;          // first row of this sequence in the [B*S, .] matrices
    // causal, FQ == FK: tile X attends key tiles 0 .. 2*qb + X; a tile that starts past the sequence is inactive
    const int n_a = 2 * qb + 1, n_b = (q0 + FQ < p.S) ? 2 * qb + 2 : 0;
    const int n_tiles = max(n_a, n_b);

    if (threadIdx.x == 0) {
        mbar_init(&bars.q_full, 1);
        for (int i = 0; i < FWD_KV_STAGES; ++i) {
            mbar_init(&bars.kv_full[i], 1);
            mbar_init(&bars.kv_empty[i], n_b > 0 ? 2 : 1);   // one arrival per issuing thread
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&bars.s_full[i], 1);
            mbar_init(&bars.s_free[i], 4);
            mbar_init(&bars.p_ready[i], 4);
            mbar_init(&bars.pv_done[i], 1);
        }
        bars.abort_flag = 0;
        mbar_fence_init();
        fence_proxy_async_smem();
    }
    if (warp == 1) {
        tmem_alloc(&bars.tmem_base, FWD_TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = bars.tmem_base;
    volatile int* abort_flag = &bars.abort_flag;

    if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(FWD_REGS_CONTROL));
    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
            mbar_expect_tx(&bars.q_full, 2 * Q_BYTES);
            tma_load_2d(sQ, &tmQ, &bars.q_full, h * FHD, row0 + q0);
            tma_load_2d(sQ + Q_BYTES, &tmQ, &bars.q_full, h * FHD, row0 + q0 + FQ);
            for (int j = 0; j < n_tiles; ++j) {
                const int st = j % FWD_KV_STAGES;
                if (!mbar_wait(&bars.kv_empty[st], ((j / FWD_KV_STAGES) & 1) ^ 1, abort_flag)) break;
                mbar_expect_tx(&bars.kv_full[st], 2 * KV_TILE_BYTES);
                tma_load_2d(sK + st * KV_TILE_BYTES, &tmK, &bars.kv_full[st], kh * FHD, row0 + j * FK);
                tma_load_2d(sV + st * KV_TILE_BYTES, &tmV, &bars.kv_full[st], kh * FHD, row0 + j * FK);
            }
        }
    } else if (warp == 1 || warp == 2) {
        // ------------------------------ UMMA issuers: warp 1 for query tile A, warp 2 for tile B ------------------
        // One thread per query tile: a thread that issues for both tiles meets their barriers in a fixed order (five waits per key
        // tile at ~160 cycles each, 24 issues at ~53) and makes one tile wait behind the other's.
        const int x = warp - 1;
        const int n_this = x ? n_b : n_a;
        if (lane == 0 && n_this > 0) {
            const uint32_t idesc_s = umma_idesc_bf16_f32(FQ, FK, 0, 0);    // S = Q K^T : both operands K-major
            const uint32_t idesc_o = umma_idesc_bf16_f32(FQ, FHD, 0, 1);   // O += P V  : P K-major, V MN-major
            // Descriptors differ only in their 14-bit start-address field (address >> 4), so each is built once and
            // stepped by plain integer adds: +2 per 32 B (one K-step inside a 128-byte row), +128 per 2048 B
            // (16 rows of an MN-major tile), +1024 per 16 KB (tile stage / key half).
            const uint64_t qd = umma_smem_desc_sw128(smem_u32(sQ), 16, 1024) + (uint64_t)(x * (Q_BYTES >> 4));
            const uint64_t kd0 = umma_smem_desc_sw128(smem_u32(sK), 16, 1024);
            const uint64_t vd0 = umma_smem_desc_sw128(smem_u32(sV), FK * 128, 1024);
            auto issue_qk = [&](int j) {
                const uint64_t kd = kd0 + (uint64_t)((j % FWD_KV_STAGES) * (KV_TILE_BYTES >> 4));
#pragma unroll
                for (int k = 0; k < FHD / 16; ++k) umma_bf16_ss(tmem + x * FK, qd + 2 * k, kd + 2 * k, idesc_s, k > 0 ? 1u : 0u);
                umma_commit(&bars.s_full[x]);
            };
            auto issue_pv = [&](int j) {
                const uint64_t vd = vd0 + (uint64_t)((j % FWD_KV_STAGES) * (KV_TILE_BYTES >> 4));
#pragma unroll
                for (int k = 0; k < FK / 16; ++k)
                    // P comes from tensor memory (16 keys = 8 columns of bf16 pairs); V: 16 keys = 2048 B
                    umma_bf16_ts(tmem + 2 * FK + x * FHD, tmem + FWD_TMEM_P + x * (FK / 2) + 8 * k, vd + 128 * k, idesc_o,
                                 (j > 0 || k > 0) ? 1u : 0u);
                umma_commit(&bars.pv_done[x]);
            };
            bool ok = mbar_wait(&bars.q_full, 0, abort_flag) && mbar_wait(&bars.kv_full[0], 0, abort_flag);
            if (ok) {
                tc_fence_after_sync();
                issue_qk(0);
            }
            for (int j = 0; j < n_tiles && ok; ++j) {
                // S of the NEXT key tile is issued as soon as the softmax warps have read this tile's S out of TMEM (s_free),
                // i.e. before P V of this tile: the scores of tile j+1 are ready when the softmax of tile j ends, and the
                // softmax of tile j+1 runs while the tensor core does P V of tile j.
                if (j + 1 < n_this) {
                    if (!mbar_wait(&bars.s_free[x], j & 1, abort_flag)) { ok = false; break; }
                    if (!mbar_wait(&bars.kv_full[(j + 1) % FWD_KV_STAGES], ((j + 1) / FWD_KV_STAGES) & 1, abort_flag)) { ok = false; break; }
                    tc_fence_after_sync();
                    issue_qk(j + 1);
                }
                if (j < n_this) {
                    if (!mbar_wait(&bars.p_ready[x], j & 1, abort_flag)) { ok = false; break; }
                    tc_fence_after_sync();
                    issue_pv(j);
                    umma_commit(&bars.kv_empty[j % FWD_KV_STAGES]);  // every UMMA of this query tile that reads the stage has been issued
                } else {
                    mbar_arrive(&bars.kv_empty[j % FWD_KV_STAGES]);  // a key tile this query tile does not attend
                }
            }
        }
    }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(FWD_REGS_SOFTMAX));
        // ------------------------------ softmax / epilogue: warps 4-7 = tile A, 8-11 = tile B ------------
        const int x = (warp - 4) >> 2;
        const int quarter = warp & 3;              // TMEM lane quarter this warp may access
        const int r = quarter * 32 + lane;         // query row inside the tile
        const int qi = q0 + x * FQ + r;            // query position in the sequence
        const uint32_t lane_addr = tmem + ((uint32_t)(quarter * 32) << 16);
        const uint32_t s_addr = lane_addr + x * FK, o_addr = lane_addr + 2 * FK + x * FHD;
        const uint32_t p_addr = lane_addr + FWD_TMEM_P + x * (FK / 2);
        const float sl2 = p.scale * LOG2E_F;
        const int n_mine = x ? n_b : n_a;
        float m_ref = -INFINITY;   // the maximum O and l are currently referenced to (log2 domain)
        float l_run = 0.f;
        bool ok = true;
        for (int j = 0; j < n_mine; ++j) {
            ok = mbar_wait(&bars.s_full[x], j & 1, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after_sync();
            uint32_t v[4][32];
#pragma unroll
            for (int ch = 0; ch < 4; ++ch) tmem_ld_32x32(s_addr + ch * 32, v[ch]);
            tmem_ld_wait();
            // the scores are in registers: their TMEM columns may receive the next key tile
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars.s_free[x]);
            const int k0 = j * FK;
            // padding mask (attention_forward_seq_masked, src/kernels/forward.metal:1853): one word of key bits per 32 columns
            uint32_t mw[4] = {0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu};
            bool tile_masked = false;
            if (MASKED && p.keymask) {
                const int W = (p.S + 31) >> 5;
#pragma unroll
                for (int ch = 0; ch < 4; ++ch) {
                    const int wi = (k0 >> 5) + ch;
                    mw[ch] = wi < W ? p.keymask[(size_t)b * W + wi] : 0u;
                    tile_masked |= mw[ch] != 0xffffffffu;
                }
            }
            if (j == n_mine - 1 || k0 + FK > p.S || tile_masked) {  // diagonal tile, ragged end or masked keys
#pragma unroll
                for (int ch = 0; ch < 4; ++ch)
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int kj = k0 + ch * 32 + i;
                        if (kj > qi || kj >= p.S || (MASKED && !((mw[ch] >> i) & 1u))) v[ch][i] = __float_as_uint(-INFINITY);
                    }
            }
            // eight independent max chains (a single chain of 128 dependent FMNMX would be latency-bound)
            float mxp[8];
#pragma unroll
            for (int t = 0; t < 8; ++t) mxp[t] = -INFINITY;
#pragma unroll
            for (int ch = 0; ch < 4; ++ch)
#pragma unroll
                for (int i = 0; i < 32; i += 2) mxp[(i >> 1) & 7] = max3_f(mxp[(i >> 1) & 7], __uint_as_float(v[ch][i]), __uint_as_float(v[ch][i + 1]));
            float mx = fmaxf(fmaxf(fmaxf(mxp[0], mxp[1]), fmaxf(mxp[2], mxp[3])), fmaxf(fmaxf(mxp[4], mxp[5]), fmaxf(mxp[6], mxp[7])));
            mx *= sl2;
            // lazy rescale: keep the old reference unless the maximum grew by more than the threshold
            float corr = 1.0f;
            bool need = false;
            if (m_ref == -INFINITY) {
                if (mx != -INFINITY) m_ref = mx;  // first finite maximum: O and l are still zero, nothing to rescale
            } else if (mx > m_ref + RESCALE_THRESHOLD) {
                corr = ex2_approx(m_ref - mx);
                m_ref = mx;
                need = true;
            }
            const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;
            // probabilities, packed to bf16 pairs (keys 2c, 2c+1 -> column c of the P block in tensor memory); four independent sum chains
            uint32_t pk[2][32];
            float ls[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int ch = 0; ch < 4; ++ch)
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    float p0, p1;
                    fma2_f(p0, p1, __uint_as_float(v[ch][i]), __uint_as_float(v[ch][i + 1]), sl2, -m_use);
                    p0 = ex2_approx(p0);
                    p1 = ex2_approx(p1);
                    add2_f(ls[2 * ((i >> 1) & 3)], ls[2 * ((i >> 1) & 3) + 1], p0, p1);
                    __nv_bfloat162 hh = __floats2bfloat162_rn(p0, p1);
                    pk[ch >> 1][(ch & 1) * 16 + (i >> 1)] = *reinterpret_cast<uint32_t*>(&hh);
                }
            const float lsum = ((ls[0] + ls[1]) + (ls[2] + ls[3])) + ((ls[4] + ls[5]) + (ls[6] + ls[7]));
            l_run = l_run * corr + lsum;
            if (j > 0) {
                // P_X(j-1) must have been consumed (and O_X updated) before P is overwritten / O rescaled
                ok = mbar_wait(&bars.pv_done[x], (j - 1) & 1, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after_sync();
                if (__any_sync(0xffffffffu, need)) {
#pragma unroll
                    for (int ch = 0; ch < FHD / 32; ++ch) {
                        uint32_t o[32];
                        tmem_ld_32x32(o_addr + ch * 32, o);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * corr);
                        tmem_st_32x32(o_addr + ch * 32, o);
                    }
                }
            }
            // P row -> tensor memory, where P V reads it as its A operand (this thread's TMEM lane = its query row)
            tmem_st_32x32(p_addr, pk[0]);
            tmem_st_32x32(p_addr + 32, pk[1]);
            tmem_st_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars.p_ready[x]);
        }
        if (ok && n_mine > 0) {
            ok = mbar_wait(&bars.pv_done[x], (n_mine - 1) & 1, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
        }
        if (ok && n_mine > 0) {
            tc_fence_after_sync();
            // a masked position is no query either: its output row is zero, and its log-sum-exp +infinity makes every probability
            // the backward recomputes for it zero (no gradient to or from the row)
            const bool q_on = !MASKED || !p.keymask || (qi < p.S && ((p.keymask[(size_t)b * ((p.S + 31) >> 5) + (qi >> 5)] >> (qi & 31)) & 1u));
            const float inv = (l_run > 0.f && q_on) ? 1.0f / l_run : 0.f;
            bf16* orow = p.out + (size_t)(row0 + qi) * p.ldo + (size_t)h * FHD;
#pragma unroll
            for (int ch = 0; ch < FHD / 32; ++ch) {
                uint32_t o[32];
                tmem_ld_32x32(o_addr + ch * 32, o);
                tmem_ld_wait();
                if (qi < p.S) {
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        uint4 w;
                        __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&w);
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            ob[i] = __floats2bfloat162_rn(__uint_as_float(o[c * 8 + 2 * i]) * inv, __uint_as_float(o[c * 8 + 2 * i + 1]) * inv);
                        *reinterpret_cast<uint4*>(orow + ch * 32 + c * 8) = w;
                    }
                }
            }
            if (qi < p.S)
                p.lse[((size_t)b * p.NH + h) * p.S + qi] = !q_on ? INFINITY : l_run > 0.f ? (m_ref + log2f(l_run)) * (1.0f / LOG2E_F) : -INFINITY;
            tc_fence_before_sync();
        }
    }

    // ------------------------------ teardown ---------------------------------------
    __syncwarp();
    if (*abort_flag) {
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 2000000ull) __nanosleep(1000);
        if (threadIdx.x == 0 && p.err) atomicExch(p.err, 2000 + (int)blockIdx.x);
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    if (warp == 1) tmem_dealloc(tmem, FWD_TMEM_COLS);
}

// ================================ backward =====================================================================
// One CTA owns 128 keys of one KV head (K and V tiles stay in shared memory, dK and dV stay in TMEM) and sweeps every
// 128-query tile at or after it of every query head that shares the KV head. Per query tile:
//   S  = Q K^T, dP = dO V^T          two UMMA 128x128x64 into TMEM                       (both operands K-major)
//   P  = exp2(S*scale*log2e - lse*log2e),  dS = P * (dP - delta) * scale
//                                     16 warps: warp w handles TMEM lane quarter w%4 and 32 of the 128 key columns;
//                                     no row maximum is needed because lse is known, so columns split freely.
//                                     P and dS go to shared memory as bf16 rows [query][key] (128B-swizzled halves).
//   dV += P^T dO, dK += dS^T Q        UMMA 128x64x128: A = the P / dS tile read MN-major (the reduction index, the query,
//                                     is the row), B = dO / Q tile read MN-major
//   dQ  = dS K                        UMMA 128x64x128: A = dS tile read K-major, B = K tile read MN-major
// dQ tiles are added into an fp32 scratch with red.global.add.v4.f32 (another key block adds to the same rows);
// dK and dV are written once at the end, so they need no atomics and are deterministic.
// Reference: attention_backward_tiled, src/kernels/backward.metal:820 (same two-level loop, float atomics for dK/dV there).
constexpr int BWD_THREADS = 608;  // TMA warp, UMMA warp (S, dP), 16 compute warps, second UMMA warp (dV, dK, dQ)
constexpr int BWD_DYN_SMEM = 2 * KV_TILE_BYTES + 2 * 2 * Q_BYTES + 4 * P_BYTES + 1024;  // K,V + 2 stages of (Q,dO) + 2 x (P + dS) = 224 KB
constexpr uint32_t BT_S = 0, BT_DP = 128, BT_DV = 256, BT_DK = 320, BT_DQ = 384;  // dQ: two buffers of 64 columns (384, 448)

struct __align__(8) BwdBars {
    uint64_t kv_full, q_full[2], q_empty[2], g_full[2], g_empty[2], sdp_full, sdp_free, pds_ready[2], dq_full[2];
    uint32_t tmem_base;
    int abort_flag;
};

struct BwdArgs {
    float* dq_acc;   // [B*S, NH*64] fp32, zero on entry
    bf16 *gk, *gv;
    int ldgkv;
    const float *lse, *delta;
    const float* rope_cs;   // [S][32][cos, sin] or null; when set, dK leaves rotated backwards (the transposed rotation of RoPE)
    const uint32_t* keymask;   // as in the forward; masked queries need nothing here: the forward stored +infinity as their log-sum-exp
    int S, NH, NKV;
    float scale;
    int* err;
};

__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

__global__ void __launch_bounds__(BWD_THREADS, 1)
flash_bwd_umma_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmG, const BwdArgs p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ BwdBars bars;
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* sK = smem;
    uint8_t* sV = sK + KV_TILE_BYTES;
    uint8_t* sQ = sV + KV_TILE_BYTES;       // 2 stages
    uint8_t* sG = sQ + 2 * Q_BYTES;         // 2 stages (dO tiles)
    uint8_t* sP = sG + 2 * Q_BYTES;         // 2 buffers x [2 key halves][128 query rows][128 B]
    uint8_t* sD = sP + 2 * P_BYTES;         // dS, same layout, 2 buffers

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nblk = blockIdx.x, kh = blockIdx.y, b = blockIdx.z;   // key block 0 has the most work and starts first
    const int mul = p.NH / p.NKV;
    const int QD = p.NH * FHD;
    const int n0 = nblk * FK;
    const int nqb = (p.S + FQ - 1) / FQ;
    const int row0 = b * p.S;
    const int per_head = nqb - nblk;        // query tiles nblk .. nqb-1
    const int total = mul * per_head;

    if (threadIdx.x == 0) {
        mbar_init(&bars.kv_full, 1);
        for (int i = 0; i < 2; ++i) { mbar_init(&bars.q_full[i], 1); mbar_init(&bars.q_empty[i], 1); mbar_init(&bars.g_full[i], 1); mbar_init(&bars.g_empty[i], 1); }
        mbar_init(&bars.sdp_full, 1);
        mbar_init(&bars.sdp_free, 16);
        for (int i = 0; i < 2; ++i) { mbar_init(&bars.pds_ready[i], 16); mbar_init(&bars.dq_full[i], 1); }
        bars.abort_flag = 0;
        mbar_fence_init();
        fence_proxy_async_smem();
    }
    if (warp == 1) {
        tmem_alloc(&bars.tmem_base, 512);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = bars.tmem_base;
    volatile int* abort_flag = &bars.abort_flag;

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV); tma_prefetch_desc(&tmG);
            mbar_expect_tx(&bars.kv_full, 2 * KV_TILE_BYTES);
            tma_load_2d(sK, &tmK, &bars.kv_full, kh * FHD, row0 + n0);
            tma_load_2d(sV, &tmV, &bars.kv_full, kh * FHD, row0 + n0);
            for (int it = 0; it < total; ++it) {
                const int st = it & 1;
                const int hl = it / per_head, mb = nblk + (it - hl * per_head);
                const int h = kh * mul + hl;
                // Q and dO have a barrier pair each: the Q half of a stage is released after dK (issued first), the dO half after dV
                if (!mbar_wait(&bars.q_empty[st], ((it >> 1) & 1) ^ 1, abort_flag)) break;
                mbar_expect_tx(&bars.q_full[st], Q_BYTES);
                tma_load_2d(sQ + st * Q_BYTES, &tmQ, &bars.q_full[st], h * FHD, row0 + mb * FQ);
                if (!mbar_wait(&bars.g_empty[st], ((it >> 1) & 1) ^ 1, abort_flag)) break;
                mbar_expect_tx(&bars.g_full[st], Q_BYTES);
                tma_load_2d(sG + st * Q_BYTES, &tmG, &bars.g_full[st], h * FHD, row0 + mb * FQ);
            }
        }
    } else if (warp == 1) {
        // ------------------------------ UMMA issuer --------------------------------
        if (lane == 0) {
            const uint32_t id_s = umma_idesc_bf16_f32(FQ, FK, 0, 0);     // S, dP: A K-major, B K-major, N = 128
            // descriptor bases; K-major tiles step +2 (32 B) per UMMA
            const uint64_t k_km = umma_smem_desc_sw128(smem_u32(sK), 16, 1024);
            const uint64_t v_km = umma_smem_desc_sw128(smem_u32(sV), 16, 1024);
            const uint64_t q_km0 = umma_smem_desc_sw128(smem_u32(sQ), 16, 1024);
            const uint64_t g_km0 = umma_smem_desc_sw128(smem_u32(sG), 16, 1024);
            // Software pipeline: S and dP of tile it+1 are issued as soon as the compute warps have read tile it's out of TMEM
            // (sdp_free), i.e. BEFORE the dV/dK/dQ UMMAs of tile it, so the exponentials of tile it+1 run while the tensor
            // core works through the second stage of tile it.
            bool ok = mbar_wait(&bars.kv_full, 0, abort_flag);
            if (ok && total > 0) {
                ok = mbar_wait(&bars.q_full[0], 0, abort_flag) && mbar_wait(&bars.g_full[0], 0, abort_flag);
                if (ok) {
                    tc_fence_after_sync();
#pragma unroll
                    for (int k = 0; k < FHD / 16; ++k) umma_bf16_ss(tmem + BT_S, q_km0 + 2 * k, k_km + 2 * k, id_s, k > 0 ? 1u : 0u);
#pragma unroll
                    for (int k = 0; k < FHD / 16; ++k) umma_bf16_ss(tmem + BT_DP, g_km0 + 2 * k, v_km + 2 * k, id_s, k > 0 ? 1u : 0u);
                    umma_commit(&bars.sdp_full);
                }
            }
            for (int it = 0; it + 1 < total && ok; ++it) {
                const int nx = (it + 1) & 1;
                const uint64_t sn = (uint64_t)(nx * (Q_BYTES >> 4));
                if (!mbar_wait(&bars.sdp_free, it & 1, abort_flag)) { ok = false; break; }
                if (!mbar_wait(&bars.q_full[nx], ((it + 1) >> 1) & 1, abort_flag)) { ok = false; break; }
                tc_fence_after_sync();
#pragma unroll
                for (int k = 0; k < FHD / 16; ++k) umma_bf16_ss(tmem + BT_S, q_km0 + sn + 2 * k, k_km + 2 * k, id_s, k > 0 ? 1u : 0u);
                if (!mbar_wait(&bars.g_full[nx], ((it + 1) >> 1) & 1, abort_flag)) { ok = false; break; }
                tc_fence_after_sync();
#pragma unroll
                for (int k = 0; k < FHD / 16; ++k) umma_bf16_ss(tmem + BT_DP, g_km0 + sn + 2 * k, v_km + 2 * k, id_s, k > 0 ? 1u : 0u);
                umma_commit(&bars.sdp_full);
            }
        }
    } else if (warp == 18) {
        // ------------------------------ second UMMA issuer: dV, dK, dQ ----------------
        // A thread's UMMAs are accepted one at a time; with the first-stage and second-stage products issued by two threads
        // the tensor core's queue is fed from both while the compute warps work on the tile in between.
        if (lane == 0) {
            const uint32_t id_kv = umma_idesc_bf16_f32(FK, FHD, 1, 1);   // dV, dK: A MN-major, B MN-major, N = 64
            const uint32_t id_q = umma_idesc_bf16_f32(FQ, FHD, 0, 1);    // dQ: A K-major, B MN-major, N = 64
            // MN-major tiles step +128 (2048 B = 16 rows) per UMMA
            const uint64_t k_mn = umma_smem_desc_sw128(smem_u32(sK), FK * 128, 1024);        // N = 64: a single MN group
            const uint64_t q_mn0 = umma_smem_desc_sw128(smem_u32(sQ), FQ * 128, 1024);
            const uint64_t g_mn0 = umma_smem_desc_sw128(smem_u32(sG), FQ * 128, 1024);
            const uint64_t p_mn = umma_smem_desc_sw128(smem_u32(sP), FQ * 128, 1024);        // M = 128 keys: LBO = next key half (16 KB)
            const uint64_t d_mn = umma_smem_desc_sw128(smem_u32(sD), FQ * 128, 1024);
            const uint64_t d_km = umma_smem_desc_sw128(smem_u32(sD), 16, 1024);
            bool ok = mbar_wait(&bars.kv_full, 0, abort_flag);
            for (int it = 0; it < total && ok; ++it) {
                const int st = it & 1;
                const uint64_t so = (uint64_t)(st * (Q_BYTES >> 4));
                if (!mbar_wait(&bars.q_full[st], (it >> 1) & 1, abort_flag)) { ok = false; break; }
                if (!mbar_wait(&bars.g_full[st], (it >> 1) & 1, abort_flag)) { ok = false; break; }
                // P and dS of this tile are in shared-memory buffer it & 1; the dQ columns of that parity were read out two tiles ago
                const int pb = it & 1;
                const uint64_t po = (uint64_t)(pb * (P_BYTES >> 4));
                if (!mbar_wait(&bars.pds_ready[pb], (it >> 1) & 1, abort_flag)) { ok = false; break; }
                tc_fence_after_sync();
                // The refill of a stage (over a thousand clocks) is what S / dP of the tile after next wait for, so each half is
                // released as early as its last reader allows: Q after dK, dO after dV; dQ reads neither.
#pragma unroll
                for (int k = 0; k < FQ / 16; ++k) umma_bf16_ss(tmem + BT_DK, d_mn + po + 128 * k, q_mn0 + so + 128 * k, id_kv, (it > 0 || k > 0) ? 1u : 0u);
                umma_commit(&bars.q_empty[st]);
#pragma unroll
                for (int k = 0; k < FQ / 16; ++k) umma_bf16_ss(tmem + BT_DV, p_mn + po + 128 * k, g_mn0 + so + 128 * k, id_kv, (it > 0 || k > 0) ? 1u : 0u);
                umma_commit(&bars.g_empty[st]);
#pragma unroll
                for (int k = 0; k < FK / 16; ++k)
                    umma_bf16_ss(tmem + BT_DQ + pb * FHD, d_km + po + (uint64_t)((k >> 2) * ((FQ * 128) >> 4) + (k & 3) * 2), k_mn + 128 * k, id_q,
                                 k > 0 ? 1u : 0u);
                umma_commit(&bars.dq_full[pb]);
            }
        }
    } else {
        // ------------------------------ 16 compute warps ----------------------------
        const int cw = warp - 2;
        const int quarter = warp & 3;           // TMEM lanes this warp may touch: 32*quarter .. +31
        const int cg = cw >> 2;                 // column group: S/dP columns [32*cg, +32), dQ/dK/dV columns [16*cg, +16)
        const int r = quarter * 32 + lane;      // row inside the tile (query for S/dP/dQ, key for dK/dV)
        const uint32_t lane_addr = tmem + ((uint32_t)(quarter * 32) << 16);
        const float sl2 = p.scale * LOG2E_F;
        bool ok = true;
        uint32_t dq_regs[16];
        int prev_h = 0, prev_q0 = 0;
        // dQ of a finished tile (this thread: 16 fp32 of query row r) is added into the fp32 scratch. One red per row piece
        // straight from the registers would touch 32 different lines per instruction, so the warp first transposes through
        // shared memory: a thread parks its 64 bytes in the half row of the P buffer `buf` that holds its own P piece (free
        // once that tile's second-stage UMMAs are done, and next written by this same thread), slots rotated by the row so
        // that a quarter warp hits eight different 16-byte slots; then four lanes cover one row and an instruction adds
        // eight 64-byte row pieces.
        auto flush_dq = [&](int buf) {
            const uint32_t base = smem_u32(sP + buf * P_BYTES + (cg >> 1) * (FQ * 128) + quarter * 32 * 128);
            const uint32_t mine = base + lane * 128 + (((cg & 1) ^ ((lane >> 2) & 1)) * 64);
#pragma unroll
            for (int c = 0; c < 4; ++c)
                st_shared_v4(mine + ((c ^ (lane & 3)) * 16), dq_regs[4 * c], dq_regs[4 * c + 1], dq_regs[4 * c + 2], dq_regs[4 * c + 3]);
            __syncwarp();
            const int c = lane & 3;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int rr = 8 * i + (lane >> 3) + 4 * ((lane >> 2) & 1);   // row inside the warp's 32 rows
                const uint32_t src = base + rr * 128 + (((cg & 1) ^ ((rr >> 2) & 1)) * 64) + ((c ^ (rr & 3)) * 16);
                float4 v;
                asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(src) : "memory");
                const int pq = prev_q0 + quarter * 32 + rr;
                if (pq < p.S) {
                    float* dst = p.dq_acc + (size_t)(row0 + pq) * QD + (size_t)prev_h * FHD + cg * 16 + c * 4;
                    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
                }
            }
            __syncwarp();
        };
        // per-row statistics of tile `t` (rows past the end: lse = +inf makes every probability zero); fetched one tile ahead
        auto load_stats = [&](int t, float& lse_out, float& dlt_out) {
            lse_out = INFINITY;
            dlt_out = 0.f;
            if (t < total) {
                const int thl = t / per_head, tmb = nblk + (t - thl * per_head);
                const int tq = tmb * FQ + r;
                if (tq < p.S) {
                    const size_t idx = ((size_t)b * p.NH + kh * mul + thl) * p.S + tq;
                    lse_out = p.lse[idx];
                    dlt_out = p.delta[idx];
                }
            }
        };
        // this warp's 32 key columns of the padding mask (all ones without a mask)
        uint32_t kw = 0xffffffffu;
        if (p.keymask) {
            const int W = (p.S + 31) >> 5, wi = (n0 >> 5) + cg;
            kw = wi < W ? p.keymask[(size_t)b * W + wi] : 0u;
        }
        float lse_next, dlt_next;
        load_stats(0, lse_next, dlt_next);
        for (int it = 0; it < total; ++it) {
            const int hl = it / per_head, mb = nblk + (it - hl * per_head);
            const int h = kh * mul + hl, q0 = mb * FQ;
            const float lse2 = lse_next * LOG2E_F, dlt = dlt_next;
            load_stats(it + 1, lse_next, dlt_next);
            ok = mbar_wait(&bars.sdp_full, it & 1, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after_sync();
            uint32_t sv[32], dv[32];
            tmem_ld_32x32(lane_addr + BT_S + cg * 32, sv);
            tmem_ld_32x32(lane_addr + BT_DP + cg * 32, dv);
            tmem_ld_wait();
            // S and dP are in registers: their TMEM columns may receive the next tile
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars.sdp_free);
            const bool diag = (mb == nblk) || (n0 + FK > p.S) || kw != 0xffffffffu;
            const float dlt_s = -dlt * p.scale;
            uint32_t pp[16], dd[16];
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
                float p0, p1, d0, d1;
                fma2_f(p0, p1, __uint_as_float(sv[i]), __uint_as_float(sv[i + 1]), sl2, -lse2);
                fma2_f(d0, d1, __uint_as_float(dv[i]), __uint_as_float(dv[i + 1]), p.scale, dlt_s);   // scale * (dP - delta)
                p0 = ex2_approx(p0);
                p1 = ex2_approx(p1);
                if (diag) {
                    const int kl = cg * 32 + i;   // key inside the tile; on the diagonal tile n0 == q0
                    if ((mb == nblk && kl > r) || n0 + kl >= p.S || !((kw >> i) & 1u)) p0 = 0.f;
                    if ((mb == nblk && kl + 1 > r) || n0 + kl + 1 >= p.S || !((kw >> (i + 1)) & 1u)) p1 = 0.f;
                }
                mul2_f(d0, d1, d0, d1, p0, p1);
                __nv_bfloat162 hp = __floats2bfloat162_rn(p0, p1), hd = __floats2bfloat162_rn(d0, d1);
                pp[i >> 1] = *reinterpret_cast<uint32_t*>(&hp);
                dd[i >> 1] = *reinterpret_cast<uint32_t*>(&hd);
            }
            const int pb = it & 1;
            if (it >= 2) {
                // the second-stage UMMAs of tile it-2 have read this P/dS buffer
                ok = mbar_wait(&bars.dq_full[pb], ((it - 2) >> 1) & 1, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
            }
            // rows of P and dS: key half = cg / 2, 16-byte chunks (cg & 1) * 4 .. +3 of the 128-byte row
            {
                const uint32_t prow = smem_u32(sP + pb * P_BYTES + (cg >> 1) * (FQ * 128) + r * 128);
                const uint32_t drow = smem_u32(sD + pb * P_BYTES + (cg >> 1) * (FQ * 128) + r * 128);
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const int cc = ((cg & 1) * 4 + c) ^ (r & 7);
                    st_shared_v4(prow + cc * 16, pp[4 * c], pp[4 * c + 1], pp[4 * c + 2], pp[4 * c + 3]);
                    st_shared_v4(drow + cc * 16, dd[4 * c], dd[4 * c + 1], dd[4 * c + 2], dd[4 * c + 3]);
                }
            }
            tc_fence_before_sync();
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars.pds_ready[pb]);
            if (it > 0) {
                // the previous tile's dQ (the other TMEM buffer) goes into the fp32 scratch while the tensor core works on this tile
                ok = mbar_wait(&bars.dq_full[pb ^ 1], ((it - 1) >> 1) & 1, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after_sync();
                tmem_ld_32x16(lane_addr + BT_DQ + (pb ^ 1) * FHD + cg * 16, dq_regs);
                tmem_ld_wait();
                flush_dq(pb ^ 1);
            }
            prev_h = h;
            prev_q0 = q0;
        }
        if (ok && total > 0) {
            ok = mbar_wait(&bars.dq_full[(total - 1) & 1], ((total - 1) >> 1) & 1, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
        }
        if (ok) {
            tc_fence_after_sync();
            if (total > 0) {
                tmem_ld_32x16(lane_addr + BT_DQ + ((total - 1) & 1) * FHD + cg * 16, dq_regs);
                tmem_ld_wait();
                flush_dq((total - 1) & 1);
            }
            // dK, dV: row = key, this warp's 16 columns
            const int kj = n0 + r;
            uint32_t a[16], c2[16];
            if (total > 0) {
                tmem_ld_32x16(lane_addr + BT_DK + cg * 16, a);
                tmem_ld_32x16(lane_addr + BT_DV + cg * 16, c2);
                tmem_ld_wait();
                if (p.rope_cs) {   // uniform over the warp: the tensor-memory load below is a warp-collective instruction
                    // RoPE backward on dK (rope_backward_seq, src/kernels/backward.metal:980): column i of the first half pairs with
                    // column i + 32, which another warp of this lane quarter owns; every warp of a quarter can read all columns
                    // of its lanes, so the partner's 16 values are fetched as well.
                    uint32_t o[16];
                    tmem_ld_32x16(lane_addr + BT_DK + (cg ^ 2) * 16, o);
                    tmem_ld_wait();
                    if (kj < p.S) {   // rows past the end of the sequence have no table entry (and are not stored)
                        const float4* cs4 = reinterpret_cast<const float4*>(p.rope_cs + ((size_t)kj * (FHD / 2) + (cg & 1) * 16) * 2);
#pragma unroll
                        for (int i = 0; i < 16; i += 2) {
                            const float4 t = cs4[i >> 1];   // cos_i, sin_i, cos_i+1, sin_i+1
                            const float m0 = __uint_as_float(a[i]), m1 = __uint_as_float(a[i + 1]);
                            const float o0 = __uint_as_float(o[i]), o1 = __uint_as_float(o[i + 1]);
                            // first half: g0 * cos + g1 * sin; second half: g1 * cos - g0 * sin  (g0 = first-half value, g1 = its partner)
                            a[i] = __float_as_uint(cg < 2 ? m0 * t.x + o0 * t.y : m0 * t.x - o0 * t.y);
                            a[i + 1] = __float_as_uint(cg < 2 ? m1 * t.z + o1 * t.w : m1 * t.z - o1 * t.w);
                        }
                    }
                }
            } else {
#pragma unroll
                for (int i = 0; i < 16; ++i) { a[i] = 0u; c2[i] = 0u; }
            }
            if (kj < p.S) {
                bf16* gkr = p.gk + (size_t)(row0 + kj) * p.ldgkv + (size_t)kh * FHD + cg * 16;
                bf16* gvr = p.gv + (size_t)(row0 + kj) * p.ldgkv + (size_t)kh * FHD + cg * 16;
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    uint4 wk, wv;
                    __nv_bfloat162* bk = reinterpret_cast<__nv_bfloat162*>(&wk);
                    __nv_bfloat162* bv = reinterpret_cast<__nv_bfloat162*>(&wv);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        bk[i] = __floats2bfloat162_rn(__uint_as_float(a[c * 8 + 2 * i]), __uint_as_float(a[c * 8 + 2 * i + 1]));
                        bv[i] = __floats2bfloat162_rn(__uint_as_float(c2[c * 8 + 2 * i]), __uint_as_float(c2[c * 8 + 2 * i + 1]));
                    }
                    *reinterpret_cast<uint4*>(gkr + c * 8) = wk;
                    *reinterpret_cast<uint4*>(gvr + c * 8) = wv;
                }
            }
            tc_fence_before_sync();
        }
    }

    // ------------------------------ teardown ---------------------------------------
    __syncwarp();
    if (*abort_flag) {
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 2000000ull) __nanosleep(1000);
        if (threadIdx.x == 0 && p.err) atomicExch(p.err, 3000 + (int)blockIdx.x);
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    if (warp == 1) tmem_dealloc(tmem, 512);
}

// delta[b, h, s] = sum_d gout * out. Eight lanes per (row, head): one 16-byte load of each operand per lane.
__global__ void flash_delta_umma_kernel(float* __restrict__ delta, const bf16* __restrict__ gout, const bf16* __restrict__ out, int ldo,
                                        int B, int S, int NH) {
    const long gid = (blockIdx.x * (long)blockDim.x + threadIdx.x) >> 3;   // (row, head) index
    const int sub = threadIdx.x & 7;
    const long total = (long)B * S * NH;
    float d = 0.f;
    long row = 0;
    int h = 0;
    if (gid < total) {
        h = (int)(gid % NH);
        row = gid / NH;
        const uint4 a = *reinterpret_cast<const uint4*>(gout + row * ldo + (size_t)h * FHD + sub * 8);
        const uint4 c = *reinterpret_cast<const uint4*>(out + row * ldo + (size_t)h * FHD + sub * 8);
        const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&a);
        const __nv_bfloat162* pc = reinterpret_cast<const __nv_bfloat162*>(&c);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 fa = __bfloat1622float2(pa[i]), fc = __bfloat1622float2(pc[i]);
            d = fmaf(fa.x, fc.x, fmaf(fa.y, fc.y, d));
        }
    }
    d += __shfl_xor_sync(0xffffffffu, d, 1);
    d += __shfl_xor_sync(0xffffffffu, d, 2);
    d += __shfl_xor_sync(0xffffffffu, d, 4);
    if (sub == 0 && gid < total) delta[((size_t)(row / S) * NH + h) * S + (row % S)] = d;
}

// dQ leaves the backward as fp32 sums in a scratch buffer (several key blocks add to the same rows); this pass turns them into
// the bf16 gradient and, when a rotation table is given, applies RoPE backward on the way (rope_backward_seq,
// src/kernels/backward.metal:980) so that no separate rotation pass reads and rewrites the tensor. One thread: four adjacent
// columns of the first half of a head and their partners 32 columns further on.
__global__ void dq_finish_kernel(bf16* __restrict__ gq, int ldgq, const float* __restrict__ acc, int rows, int NH, int S,
                                 const float* __restrict__ cs) {
    const long i = blockIdx.x * (long)blockDim.x + threadIdx.x;
    if (i >= (long)rows * NH * 8) return;
    const int c = (int)(i & 7) * 4;
    const long rh = i >> 3;
    const int h = (int)(rh % NH);
    const long row = rh / NH;
    const float* src = acc + ((size_t)row * NH + h) * FHD + c;
    float4 x0 = *reinterpret_cast<const float4*>(src), x1 = *reinterpret_cast<const float4*>(src + 32);
    if (cs) {
        const float4* t = reinterpret_cast<const float4*>(cs + ((size_t)(row % S) * (FHD / 2) + c) * 2);
        const float4 t0 = t[0], t1 = t[1];   // cos, sin of pairs c, c+1 | c+2, c+3
        const float4 a = x0, b = x1;
        x0.x = a.x * t0.x + b.x * t0.y; x1.x = b.x * t0.x - a.x * t0.y;
        x0.y = a.y * t0.z + b.y * t0.w; x1.y = b.y * t0.z - a.y * t0.w;
        x0.z = a.z * t1.x + b.z * t1.y; x1.z = b.z * t1.x - a.z * t1.y;
        x0.w = a.w * t1.z + b.w * t1.w; x1.w = b.w * t1.z - a.w * t1.w;
    }
    bf16* dst = gq + (size_t)row * ldgq + (size_t)h * FHD + c;
    __nv_bfloat162 lo0 = __floats2bfloat162_rn(x0.x, x0.y), lo1 = __floats2bfloat162_rn(x0.z, x0.w);
    __nv_bfloat162 hi0 = __floats2bfloat162_rn(x1.x, x1.y), hi1 = __floats2bfloat162_rn(x1.z, x1.w);
    uint2 w0, w1;
    w0.x = *reinterpret_cast<uint32_t*>(&lo0); w0.y = *reinterpret_cast<uint32_t*>(&lo1);
    w1.x = *reinterpret_cast<uint32_t*>(&hi0); w1.y = *reinterpret_cast<uint32_t*>(&hi1);
    *reinterpret_cast<uint2*>(dst) = w0;
    *reinterpret_cast<uint2*>(dst + 32) = w1;
}


// ================================ prefill: fp32-accurate attention on the tensor pipe ==========================================
// The inference session keeps fp32 activations (the reference's attention_forward_prefill_tiled, src/kernels/forward.metal:2024,
// is fp32 arithmetic), so bf16 operands would miss its accuracy by two orders of magnitude. Every fp32 operand x is therefore
// split into bf16 hi = rn(x) and lo = rn(x - hi), and each product is the sum of three tensor-core products:
//   S = Qh Kh^T + Ql Kh^T + Qh Kl^T          O += Ph Vh + Pl Vh + Ph Vl
// (the lo x lo terms are below 2^-17 of the result). Accumulation is fp32 in tensor memory, the softmax fp32 in registers.
// One CTA = 128 queries of one head: warp 0 TMA, warp 1 UMMA issuer, warps 4-7 softmax (one query row per thread).
// Tensor memory: S0 [0,128) S1 [128,256) O [256,320) Ph [320,384) Pl [384,448) (P as packed bf16 pairs, the A operand of P V).
// Shared memory: Q hi|lo 32 KB, two stages of K hi|lo and V hi|lo (64 KB each).
constexpr int PF_THREADS = 256;
constexpr int PF_KV_STAGES = 2;
constexpr int PF_DYN_SMEM = 2 * Q_BYTES + PF_KV_STAGES * 4 * KV_TILE_BYTES + 1024;
constexpr uint32_t PF_T_O = 2 * FK, PF_T_PH = 2 * FK + FHD, PF_T_PL = 2 * FK + FHD + FK / 2;

struct PfBars {
    uint64_t q_full, kv_full[PF_KV_STAGES], kv_empty[PF_KV_STAGES], s_full[2], p_ready, pv_done;
    uint32_t tmem_base;
    int abort_flag;
};
struct PfArgs {
    float* out;
    int ldo;
    int T, NH, NKV;
    float scale;
    int* err;
};

__device__ __forceinline__ void tmem_st_32x16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
        "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}

// fp32 rows -> [hi 64 | lo 64] bf16 per head; one thread per four values. Columns [0, QD) of a row are Q, the K and V rows come
// from their own pointers (the packed QKV rows of the session).
__global__ void prefill_split_kernel(bf16* __restrict__ qs, bf16* __restrict__ ks, bf16* __restrict__ vs, const float* __restrict__ q, int ldq,
                                     const float* __restrict__ k, const float* __restrict__ v, int ldkv, long rows, int NH, int NKV) {
    const int per_row = (NH + 2 * NKV) * (FHD / 4);
    const long i = blockIdx.x * (long)blockDim.x + threadIdx.x;
    if (i >= rows * per_row) return;
    const long r = i / per_row;
    int c = (int)(i - r * per_row);
    int head = c / (FHD / 4);
    const int d = (c - head * (FHD / 4)) * 4;
    const float* src;
    bf16* dst;
    if (head < NH) {
        src = q + (size_t)r * ldq + head * FHD + d;
        dst = qs + ((size_t)r * NH + head) * (2 * FHD) + d;
    } else if (head < NH + NKV) {
        head -= NH;
        src = k + (size_t)r * ldkv + head * FHD + d;
        dst = ks + ((size_t)r * NKV + head) * (2 * FHD) + d;
    } else {
        head -= NH + NKV;
        src = v + (size_t)r * ldkv + head * FHD + d;
        dst = vs + ((size_t)r * NKV + head) * (2 * FHD) + d;
    }
    const float4 x = *reinterpret_cast<const float4*>(src);
    const __nv_bfloat162 h0 = __floats2bfloat162_rn(x.x, x.y), h1 = __floats2bfloat162_rn(x.z, x.w);
    const float2 f0 = __bfloat1622float2(h0), f1 = __bfloat1622float2(h1);
    const __nv_bfloat162 l0 = __floats2bfloat162_rn(x.x - f0.x, x.y - f0.y), l1 = __floats2bfloat162_rn(x.z - f1.x, x.w - f1.y);
    uint2 hv, lv;
    hv.x = *reinterpret_cast<const uint32_t*>(&h0); hv.y = *reinterpret_cast<const uint32_t*>(&h1);
    lv.x = *reinterpret_cast<const uint32_t*>(&l0); lv.y = *reinterpret_cast<const uint32_t*>(&l1);
    *reinterpret_cast<uint2*>(dst) = hv;
    *reinterpret_cast<uint2*>(dst + FHD) = lv;
}

__global__ void __launch_bounds__(PF_THREADS, 1)
prefill_attention_umma_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                              const __grid_constant__ CUtensorMap tmV, const PfArgs p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ PfBars bars;
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* sQ = smem;                                   // hi box, lo box
    uint8_t* sK = sQ + 2 * Q_BYTES;                       // per stage: hi box, lo box
    uint8_t* sV = sK + PF_KV_STAGES * 2 * KV_TILE_BYTES;  // per stage: hi box, lo box

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int qb = (int)gridDim.x - 1 - (int)blockIdx.x;  // longest query blocks first
    const int h = blockIdx.y, b = blockIdx.z;
    const int kh = h / (p.NH / p.NKV);
    const int q0 = qb * FQ;
    const int row0 = b * p.T;
    const int n_tiles = qb + 1;   // causal, FQ == FK

    if (threadIdx.x == 0) {
        mbar_init(&bars.q_full, 1);
        for (int i = 0; i < PF_KV_STAGES; ++i) {
            mbar_init(&bars.kv_full[i], 1);
            mbar_init(&bars.kv_empty[i], 1);
        }
        mbar_init(&bars.s_full[0], 1);
        mbar_init(&bars.s_full[1], 1);
        mbar_init(&bars.p_ready, 4);
        mbar_init(&bars.pv_done, 1);
        bars.abort_flag = 0;
        mbar_fence_init();
        fence_proxy_async_smem();
    }
    if (warp == 1) {
        tmem_alloc(&bars.tmem_base, 512);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = bars.tmem_base;
    volatile int* abort_flag = &bars.abort_flag;

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
            mbar_expect_tx(&bars.q_full, 2 * Q_BYTES);
            tma_load_2d(sQ, &tmQ, &bars.q_full, h * 2 * FHD, row0 + q0);
            tma_load_2d(sQ + Q_BYTES, &tmQ, &bars.q_full, h * 2 * FHD + FHD, row0 + q0);
            for (int j = 0; j < n_tiles; ++j) {
                const int st = j % PF_KV_STAGES;
                if (!mbar_wait(&bars.kv_empty[st], ((j / PF_KV_STAGES) & 1) ^ 1, abort_flag)) break;
                mbar_expect_tx(&bars.kv_full[st], 4 * KV_TILE_BYTES);
                uint8_t* kd = sK + st * 2 * KV_TILE_BYTES;
                uint8_t* vd = sV + st * 2 * KV_TILE_BYTES;
                tma_load_2d(kd, &tmK, &bars.kv_full[st], kh * 2 * FHD, row0 + j * FK);
                tma_load_2d(kd + KV_TILE_BYTES, &tmK, &bars.kv_full[st], kh * 2 * FHD + FHD, row0 + j * FK);
                tma_load_2d(vd, &tmV, &bars.kv_full[st], kh * 2 * FHD, row0 + j * FK);
                tma_load_2d(vd + KV_TILE_BYTES, &tmV, &bars.kv_full[st], kh * 2 * FHD + FHD, row0 + j * FK);
            }
        }
    } else if (warp == 1) {
        // ------------------------------ UMMA issuer --------------------------------
        if (lane == 0) {
            const uint32_t idesc_s = umma_idesc_bf16_f32(FQ, FK, 0, 0);    // S = Q K^T : both operands K-major
            const uint32_t idesc_o = umma_idesc_bf16_f32(FQ, FHD, 0, 1);   // O += P V  : P from tensor memory, V MN-major
            const uint64_t qh = umma_smem_desc_sw128(smem_u32(sQ), 16, 1024), ql = qh + (uint64_t)(Q_BYTES >> 4);
            const uint64_t kd0 = umma_smem_desc_sw128(smem_u32(sK), 16, 1024);
            const uint64_t vd0 = umma_smem_desc_sw128(smem_u32(sV), FK * 128, 1024);
            auto issue_qk = [&](int j) {
                const uint64_t kh_d = kd0 + (uint64_t)((j % PF_KV_STAGES) * ((2 * KV_TILE_BYTES) >> 4)), kl_d = kh_d + (uint64_t)(KV_TILE_BYTES >> 4);
                const uint32_t ts = tmem + (uint32_t)(j & 1) * FK;
#pragma unroll
                for (int k = 0; k < FHD / 16; ++k) umma_bf16_ss(ts, qh + 2 * k, kh_d + 2 * k, idesc_s, k > 0 ? 1u : 0u);
#pragma unroll
                for (int k = 0; k < FHD / 16; ++k) umma_bf16_ss(ts, ql + 2 * k, kh_d + 2 * k, idesc_s, 1u);
#pragma unroll
                for (int k = 0; k < FHD / 16; ++k) umma_bf16_ss(ts, qh + 2 * k, kl_d + 2 * k, idesc_s, 1u);
                umma_commit(&bars.s_full[j & 1]);
            };
            auto issue_pv = [&](int j) {
                const uint64_t vh_d = vd0 + (uint64_t)((j % PF_KV_STAGES) * ((2 * KV_TILE_BYTES) >> 4)), vl_d = vh_d + (uint64_t)(KV_TILE_BYTES >> 4);
#pragma unroll
                for (int k = 0; k < FK / 16; ++k) umma_bf16_ts(tmem + PF_T_O, tmem + PF_T_PH + 8 * k, vh_d + 128 * k, idesc_o, (j > 0 || k > 0) ? 1u : 0u);
#pragma unroll
                for (int k = 0; k < FK / 16; ++k) umma_bf16_ts(tmem + PF_T_O, tmem + PF_T_PL + 8 * k, vh_d + 128 * k, idesc_o, 1u);
#pragma unroll
                for (int k = 0; k < FK / 16; ++k) umma_bf16_ts(tmem + PF_T_O, tmem + PF_T_PH + 8 * k, vl_d + 128 * k, idesc_o, 1u);
                umma_commit(&bars.pv_done);
                umma_commit(&bars.kv_empty[j % PF_KV_STAGES]);
            };
            bool ok = mbar_wait(&bars.q_full, 0, abort_flag) && mbar_wait(&bars.kv_full[0], 0, abort_flag);
            if (ok) {
                tc_fence_after_sync();
                issue_qk(0);
            }
            for (int j = 0; j < n_tiles && ok; ++j) {
                if (j + 1 < n_tiles) {
                    // S of the next key tile goes to the other S buffer (its previous scores were consumed before p_ready(j-1))
                    if (!mbar_wait(&bars.kv_full[(j + 1) % PF_KV_STAGES], ((j + 1) / PF_KV_STAGES) & 1, abort_flag)) { ok = false; break; }
                    tc_fence_after_sync();
                    issue_qk(j + 1);
                }
                if (!mbar_wait(&bars.p_ready, j & 1, abort_flag)) { ok = false; break; }
                tc_fence_after_sync();
                issue_pv(j);
            }
        }
    } else if (warp >= 4) {
        // ------------------------------ softmax / epilogue -------------------------
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;
        const int qi = q0 + r;
        const uint32_t lane_addr = tmem + ((uint32_t)(quarter * 32) << 16);
        const float sl2 = p.scale * LOG2E_F;
        float m_ref = -INFINITY, l_run = 0.f;
        bool ok = true;
        for (int j = 0; j < n_tiles; ++j) {
            ok = mbar_wait(&bars.s_full[j & 1], (j >> 1) & 1, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after_sync();
            uint32_t v[4][32];
#pragma unroll
            for (int ch = 0; ch < 4; ++ch) tmem_ld_32x32(lane_addr + (uint32_t)(j & 1) * FK + ch * 32, v[ch]);
            tmem_ld_wait();
            const int k0 = j * FK;
            if (j == n_tiles - 1) {   // diagonal tile (also the ragged end: a key past the sequence is past every valid query)
#pragma unroll
                for (int ch = 0; ch < 4; ++ch)
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (k0 + ch * 32 + i > qi) v[ch][i] = __float_as_uint(-INFINITY);
            }
            float mxp[8];
#pragma unroll
            for (int t = 0; t < 8; ++t) mxp[t] = -INFINITY;
#pragma unroll
            for (int ch = 0; ch < 4; ++ch)
#pragma unroll
                for (int i = 0; i < 32; i += 2) mxp[(i >> 1) & 7] = max3_f(mxp[(i >> 1) & 7], __uint_as_float(v[ch][i]), __uint_as_float(v[ch][i + 1]));
            float mx = fmaxf(fmaxf(fmaxf(mxp[0], mxp[1]), fmaxf(mxp[2], mxp[3])), fmaxf(fmaxf(mxp[4], mxp[5]), fmaxf(mxp[6], mxp[7])));
            mx *= sl2;
            float corr = 1.0f;
            bool need = false;
            if (mx > m_ref) {   // every valid row sees key 0, so mx is finite from the first tile on
                if (m_ref != -INFINITY) { corr = ex2_approx(m_ref - mx); need = true; }
                m_ref = mx;
            }
            const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;
            if (j > 0) {
                // P V of the previous tile has read P and updated O: P may be overwritten and O rescaled
                ok = mbar_wait(&bars.pv_done, (j - 1) & 1, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after_sync();
                if (__any_sync(0xffffffffu, need)) {
#pragma unroll
                    for (int ch = 0; ch < FHD / 32; ++ch) {
                        uint32_t o[32];
                        tmem_ld_32x32(lane_addr + PF_T_O + ch * 32, o);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * corr);
                        tmem_st_32x32(lane_addr + PF_T_O + ch * 32, o);
                    }
                }
            }
            float ls[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int ch = 0; ch < 4; ++ch) {
                uint32_t ph[16], pl[16];   // 32 keys = 16 columns of bf16 pairs
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    float p0, p1;
                    fma2_f(p0, p1, __uint_as_float(v[ch][i]), __uint_as_float(v[ch][i + 1]), sl2, -m_use);
                    p0 = ex2_approx(p0);
                    p1 = ex2_approx(p1);
                    add2_f(ls[(i >> 1) & 1 ? 2 : 0], ls[(i >> 1) & 1 ? 3 : 1], p0, p1);
                    const __nv_bfloat162 hh = __floats2bfloat162_rn(p0, p1);
                    const float2 hf = __bfloat1622float2(hh);
                    const __nv_bfloat162 ll = __floats2bfloat162_rn(p0 - hf.x, p1 - hf.y);
                    ph[i >> 1] = *reinterpret_cast<const uint32_t*>(&hh);
                    pl[i >> 1] = *reinterpret_cast<const uint32_t*>(&ll);
                }
                tmem_st_32x16(lane_addr + PF_T_PH + ch * 16, ph);
                tmem_st_32x16(lane_addr + PF_T_PL + ch * 16, pl);
            }
            l_run = l_run * corr + ((ls[0] + ls[1]) + (ls[2] + ls[3]));
            tmem_st_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars.p_ready);
        }
        if (ok) {
            ok = mbar_wait(&bars.pv_done, (n_tiles - 1) & 1, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
        }
        if (ok) {
            tc_fence_after_sync();
            const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
            float* orow = p.out + (size_t)(row0 + qi) * p.ldo + (size_t)h * FHD;
#pragma unroll
            for (int ch = 0; ch < FHD / 32; ++ch) {
                uint32_t o[32];
                tmem_ld_32x32(lane_addr + PF_T_O + ch * 32, o);
                tmem_ld_wait();
                if (qi < p.T) {
#pragma unroll
                    for (int c = 0; c < 8; ++c)
                        *reinterpret_cast<float4*>(orow + ch * 32 + c * 4) =
                            make_float4(__uint_as_float(o[c * 4]) * inv, __uint_as_float(o[c * 4 + 1]) * inv, __uint_as_float(o[c * 4 + 2]) * inv,
                                        __uint_as_float(o[c * 4 + 3]) * inv);
                }
            }
            tc_fence_before_sync();
        }
    }

    // ------------------------------ teardown ---------------------------------------
    __syncwarp();
    if (*abort_flag) {
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 2000000ull) __nanosleep(1000);
        if (threadIdx.x == 0 && p.err) atomicExch(p.err, 2500 + (int)blockIdx.x);
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    if (warp == 1) tmem_dealloc(tmem, 512);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)ptr;
    }
    return fn;
}
// [rows, width] bf16 matrix with row pitch ld (elements); box = 64 columns x box_rows rows, 128B swizzle.
int make_rows_map(CUtensorMap* tm, const void* base, uint64_t width, uint64_t rows, uint64_t ld, uint32_t box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return -10;
    cuuint64_t dims[2] = {width, rows};
    cuuint64_t strides[1] = {ld * 2};
    cuuint32_t box[2] = {64, box_rows};
    cuuint32_t estr[2] = {1, 1};
    return fn(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void*)base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS
               ? 0
               : -11;
}

// uint8 mask [B, S] -> one bit per position, [B][ceil(S / 32)] words
__global__ void pack_mask_kernel(uint32_t* __restrict__ bits, const uint8_t* __restrict__ mask, int B, int S) {
    const int W = (S + 31) >> 5;
    const long gw = (blockIdx.x * (long)blockDim.x + threadIdx.x) >> 5;   // one warp per word
    if (gw >= (long)B * W) return;
    const int bb = (int)(gw / W), w = (int)(gw - (long)bb * W), pos = w * 32 + (threadIdx.x & 31);
    const unsigned vote = __ballot_sync(0xffffffffu, pos < S && mask[(size_t)bb * S + pos] != 0);
    if ((threadIdx.x & 31) == 0) bits[gw] = vote;
}

__global__ void cast_rows_kernel(bf16* __restrict__ out, int ldo, const float* __restrict__ in, int ldi, int rows, int cols4) {
    const long i = blockIdx.x * (long)blockDim.x + threadIdx.x;
    if (i >= (long)rows * cols4) return;
    const int r = (int)(i / cols4), c = (int)(i - (long)r * cols4) * 4;
    const float4 v = *reinterpret_cast<const float4*>(in + (size_t)r * ldi + c);
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 o;
    o.x = *reinterpret_cast<uint32_t*>(&lo);
    o.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(out + (size_t)r * ldo + c) = o;
}

}  // namespace

bool flash_attention_supported(int HD, int NH, int NKV) { return HD == FHD && NKV > 0 && NH % NKV == 0; }

size_t flash_attention_backward_scratch_bytes(int B, int S, int NH, int HD) {
    return (size_t)B * S * NH * HD * sizeof(float) + (size_t)B * NH * S * sizeof(float);
}

int cast_rows_f32_to_bf16(bf16* out, int ldo, const float* in, int ldi, int rows, int cols, cudaStream_t st) {
    if (cols % 4 || ldi % 4 || ldo % 4 || (((uintptr_t)out) & 7) || (((uintptr_t)in) & 15)) return -1;
    const long n = (long)rows * (cols / 4);
    cast_rows_kernel<<<(int)((n + 255) / 256), 256, 0, st>>>(out, ldo, in, ldi, rows, cols / 4);
    return 0;
}

size_t flash_attention_mask_bits_bytes(int B, int S) { return (size_t)B * ((S + 31) / 32) * sizeof(uint32_t); }
int flash_attention_pack_mask(uint32_t* bits, const uint8_t* mask, int B, int S, cudaStream_t st) {
    const long threads = (long)B * ((S + 31) / 32) * 32;
    pack_mask_kernel<<<(int)((threads + 255) / 256), 256, 0, st>>>(bits, mask, B, S);
    return 0;
}

int flash_attention_forward_umma(bf16* out, int ldo, float* lse, const bf16* q, int ldq, const bf16* k, const bf16* v, int ldkv,
                                 const uint32_t* keymask, int B, int S, int NH, int NKV, int HD, float scale, int* err_flag, cudaStream_t st) {
    if (HD != FHD || NKV <= 0 || NH % NKV) return -1;
    if ((ldq % 8) || (ldkv % 8) || (ldo % 8) || (((uintptr_t)q) & 15) || (((uintptr_t)k) & 15) || (((uintptr_t)v) & 15) ||
        (((uintptr_t)out) & 15))
        return -2;
    static std::atomic<unsigned long long> attr_done{0};
    if (first_use_on_current_device(attr_done) &&
        (cudaFuncSetAttribute(flash_fwd_umma_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, FWD_DYN_SMEM) != cudaSuccess ||
         cudaFuncSetAttribute(flash_fwd_umma_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, FWD_DYN_SMEM) != cudaSuccess))
        return -5;
    CUtensorMap tq, tk, tv;
    const uint64_t rows = (uint64_t)B * S;
    int rc = make_rows_map(&tq, q, (uint64_t)NH * HD, rows, ldq, FQ);
    if (!rc) rc = make_rows_map(&tk, k, (uint64_t)NKV * HD, rows, ldkv, FK);
    if (!rc) rc = make_rows_map(&tv, v, (uint64_t)NKV * HD, rows, ldkv, FK);
    if (rc) return rc;
    FwdArgs a{out, ldo, lse, keymask, S, NH, NKV, scale, err_flag};
    dim3 grid((S + 2 * FQ - 1) / (2 * FQ), NH, B);
    if (keymask) flash_fwd_umma_kernel<true><<<grid, FWD_THREADS, FWD_DYN_SMEM, st>>>(tq, tk, tv, a);
    else flash_fwd_umma_kernel<false><<<grid, FWD_THREADS, FWD_DYN_SMEM, st>>>(tq, tk, tv, a);
    const cudaError_t le = cudaGetLastError();
    if (le != cudaSuccess) {
        fprintf(stderr, "flash_attention_forward_umma: launch failed: %s\n", cudaGetErrorString(le));
        return -7;
    }
    return 0;
}

int flash_attention_backward_umma(bf16* gq, int ldgq, bf16* gk, bf16* gv, int ldgkv, const bf16* gout, int ldo, const bf16* out,
                                  const float* lse, const bf16* q, int ldq, const bf16* k, const bf16* v, int ldkv, int B, int S, int NH,
                                  int NKV, int HD, float scale, void* scratch, const float* delta_in, const float* rope_cs,
                                  const uint32_t* keymask, int* err_flag, cudaStream_t st) {
    if (HD != FHD || NKV <= 0 || NH % NKV) return -1;
    if ((ldq % 8) || (ldkv % 8) || (ldo % 8) || (ldgkv % 8) || (ldgq % 4) || (((uintptr_t)q) & 15) || (((uintptr_t)k) & 15) ||
        (((uintptr_t)v) & 15) || (((uintptr_t)gout) & 15) || (((uintptr_t)gk) & 15) || (((uintptr_t)gv) & 15) || (((uintptr_t)gq) & 7) ||
        (((uintptr_t)out) & 15))
        return -2;
    static std::atomic<unsigned long long> attr_done{0};
    if (first_use_on_current_device(attr_done) &&
        cudaFuncSetAttribute(flash_bwd_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BWD_DYN_SMEM) != cudaSuccess)
        return -5;
    const uint64_t rows = (uint64_t)B * S;
    const int QD = NH * HD;
    float* dq_acc = (float*)scratch;
    float* delta_own = dq_acc + rows * QD;
    const float* delta = delta_in ? delta_in : delta_own;
    CUtensorMap tq, tk, tv, tg;
    int rc = make_rows_map(&tq, q, (uint64_t)NH * HD, rows, ldq, FQ);
    if (!rc) rc = make_rows_map(&tk, k, (uint64_t)NKV * HD, rows, ldkv, FK);
    if (!rc) rc = make_rows_map(&tv, v, (uint64_t)NKV * HD, rows, ldkv, FK);
    if (!rc) rc = make_rows_map(&tg, gout, (uint64_t)NH * HD, rows, ldo, FQ);
    if (rc) return rc;
    if (!delta_in) {
        const long groups = (long)rows * NH;   // eight lanes each
        flash_delta_umma_kernel<<<(int)((groups * 8 + 255) / 256), 256, 0, st>>>(delta_own, gout, out, ldo, B, S, NH);
    }
    cudaMemsetAsync(dq_acc, 0, rows * QD * sizeof(float), st);
    BwdArgs a{dq_acc, gk, gv, ldgkv, lse, delta, rope_cs, keymask, S, NH, NKV, scale, err_flag};
    dim3 grid((S + FK - 1) / FK, NKV, B);
    flash_bwd_umma_kernel<<<grid, BWD_THREADS, BWD_DYN_SMEM, st>>>(tq, tk, tv, tg, a);
    const cudaError_t le = cudaGetLastError();
    if (le != cudaSuccess) {
        fprintf(stderr, "flash_attention_backward_umma: launch failed: %s\n", cudaGetErrorString(le));
        return -7;
    }
    const long n = (long)rows * NH * 8;
    dq_finish_kernel<<<(int)((n + 255) / 256), 256, 0, st>>>(gq, ldgq, dq_acc, (int)rows, NH, S, rope_cs);
    return 0;
}

size_t prefill_attention_umma_scratch_bytes(long rows, int NH, int NKV) { return (size_t)rows * (NH + 2 * NKV) * 2 * FHD * sizeof(bf16); }

// fp32 in, fp32 out; q [rows, ldq], k / v [rows, ldkv] (rows = NB * T, sequence b owns rows b*T ..), out [rows, ldo]. `scratch` holds the
// split operands (prefill_attention_umma_scratch_bytes).
int prefill_attention_umma(float* out, int ldo, const float* q, int ldq, const float* k, const float* v, int ldkv, int NB, int T, int NH, int NKV,
                           int HD, float scale, void* scratch, int* err_flag, cudaStream_t st) {
    if (HD != FHD || NKV <= 0 || NH % NKV || NB <= 0 || T <= 0) return -1;
    if ((ldq % 4) || (ldkv % 4) || (ldo % 4) || (((uintptr_t)q) & 15) || (((uintptr_t)k) & 15) || (((uintptr_t)v) & 15) || (((uintptr_t)out) & 15) ||
        (((uintptr_t)scratch) & 15))
        return -2;
    static std::atomic<unsigned long long> attr_done{0};
    if (first_use_on_current_device(attr_done) &&
        cudaFuncSetAttribute(prefill_attention_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PF_DYN_SMEM) != cudaSuccess)
        return -5;
    const long rows = (long)NB * T;
    bf16* qs = (bf16*)scratch;
    bf16* ks = qs + (size_t)rows * NH * 2 * FHD;
    bf16* vs = ks + (size_t)rows * NKV * 2 * FHD;
    const long n = rows * (NH + 2 * NKV) * (FHD / 4);
    prefill_split_kernel<<<(int)((n + 255) / 256), 256, 0, st>>>(qs, ks, vs, q, ldq, k, v, ldkv, rows, NH, NKV);
    CUtensorMap tq, tk, tv;
    int rc = make_rows_map(&tq, qs, (uint64_t)NH * 2 * FHD, (uint64_t)rows, (uint64_t)NH * 2 * FHD, FQ);
    if (!rc) rc = make_rows_map(&tk, ks, (uint64_t)NKV * 2 * FHD, (uint64_t)rows, (uint64_t)NKV * 2 * FHD, FK);
    if (!rc) rc = make_rows_map(&tv, vs, (uint64_t)NKV * 2 * FHD, (uint64_t)rows, (uint64_t)NKV * 2 * FHD, FK);
    if (rc) return rc;
    PfArgs a{out, ldo, T, NH, NKV, scale, err_flag};
    dim3 grid((T + FQ - 1) / FQ, NH, NB);
    prefill_attention_umma_kernel<<<grid, PF_THREADS, PF_DYN_SMEM, st>>>(tq, tk, tv, a);
    const cudaError_t le = cudaGetLastError();
    if (le != cudaSuccess) {
        fprintf(stderr, "prefill_attention_umma: launch failed: %s\n", cudaGetErrorString(le));
        return -7;
    }
    return 0;
}

}  // namespace bmb
