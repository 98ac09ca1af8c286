// Persistent, warp-specialised tcgen05 GEMM. See gemm_umma.cuh for the operand convention.
//
// CTA = 192 threads: warp 0 = TMA producer, warp 1 = TMEM owner + UMMA issuer,
// warps 2..5 = epilogue (warp w reads TMEM lanes 32*(w&3) .. +31).
// Tile = 128 (M) x tile_n (N, <= 256) x 64 (K per stage), 4-stage shared-memory ring,
// two TMEM accumulator buffers of 256 fp32 columns so the epilogue of tile i overlaps the
// main loop of tile i+1. One CTA per SM; work units (tile, k-split) are dealt round-robin.
#include "gemm_umma.cuh"

#include <cuda.h>
#include <stdio.h>
#include <stdlib.h>

#include <atomic>

#include "common.cuh"
#include "ptx_sm100.cuh"

namespace bmb {

namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int STAGES = 4;         // one CTA per tile: 4 x (16 KB of A + 32 KB of B)
constexpr int STAGES_PAIR = 6;    // CTA pair per tile: 6 x (16 KB of A + 16 KB = this CTA's half of B)
constexpr int MAX_BN = 256;
constexpr int A_STAGE_BYTES = BM * BK * 2;      // 16 KB
constexpr int B_STAGE_BYTES = MAX_BN * BK * 2;  // 32 KB
constexpr int B_HALF_STAGE_BYTES = B_STAGE_BYTES / 2;
constexpr int MN_BOX_BYTES = 64 * BK * 2;       // one 64(mn) x 64(k) box of an MN-major operand
constexpr int NUM_THREADS = 192;
// Epilogue staging: each of the 4 epilogue warps owns 32 rows x 128 payload bytes (64 bf16 or 32 fp32 columns) at a
// 144-byte pitch, which makes both the row-per-thread accesses and the 8-lanes-per-row accesses bank-conflict free.
constexpr int STG_PITCH = 144;
constexpr int STG_WARP_BYTES = 32 * STG_PITCH;
constexpr int SMEM_DYN_BYTES = STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + 4 * STG_WARP_BYTES + 1024;
constexpr uint32_t TMEM_COLS = 512;

struct KArgs {
    int M, N, K;
    int BN;
    int a_mn, b_mn;
    int tiles_m, tiles_n, splits, kb_total, kb_per_split;
    int tile_rows;  // rows of C per work unit: 128, or 256 when a CTA pair shares the unit
    void* C;
    int ldc;
    int out_mode;
    const __nv_bfloat16* R;
    int ldr;
    int* err;
};

struct __align__(8) Barriers {
    uint64_t full[STAGES_PAIR];
    uint64_t empty[STAGES_PAIR];
    uint64_t acc_full[2];
    uint64_t acc_empty[2];
    uint32_t tmem_base;
    int abort_flag;
};

__device__ __forceinline__ void decode_unit(const KArgs& p, int u, int& m0, int& n0, int& kb0, int& kb1) {
    const int ntiles = p.tiles_m * p.tiles_n;
    const int split = u / ntiles;
    const int tile = u - split * ntiles;
    const int tm = tile / p.tiles_n;
    const int tn = tile - tm * p.tiles_n;
    m0 = tm * p.tile_rows;
    n0 = tn * p.BN;
    kb0 = split * p.kb_per_split;
    kb1 = min(p.kb_total, kb0 + p.kb_per_split);
}

// CTAS = 1: one CTA computes a 128 x BN tile. CTAS = 2: the kernel is launched in clusters of two CTAs on neighbouring SMs; the
// pair computes a 256 x BN tile with tcgen05.mma.cta_group::2 — each CTA holds its 128 rows of A and HALF of the B tile, the
// leader (cluster rank 0) issues the UMMAs, each CTA's TMEM receives its 128 rows of the accumulator and each CTA runs its own
// epilogue. B is read from shared memory once per pair instead of once per CTA.
template <int CTAS>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_bf16_umma_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                      const KArgs p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ Barriers bars;

    // 1024-byte alignment: the 128B swizzle pattern is a function of address bits [7,10).
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    constexpr int NST = CTAS == 2 ? STAGES_PAIR : STAGES;
    constexpr int BST = CTAS == 2 ? B_HALF_STAGE_BYTES : B_STAGE_BYTES;
    uint8_t* sA = smem;
    uint8_t* sB = smem + NST * A_STAGE_BYTES;
    const uint32_t rank = CTAS == 2 ? cluster_ctarank() : 0u;   // 0 = leader of the pair
    const int worker = CTAS == 2 ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
    const int nworkers = CTAS == 2 ? (int)(gridDim.x >> 1) : (int)gridDim.x;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int units = p.tiles_m * p.tiles_n * p.splits;

    if (threadIdx.x == 0) {
        for (int s = 0; s < NST; ++s) {
            mbar_init(&bars.full[s], 1);   // pair: only the leader's is used; both CTAs' copies count bytes on it
            mbar_init(&bars.empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&bars.acc_full[b], 1);
            mbar_init(&bars.acc_empty[b], 4 * CTAS);  // pair: the leader's collects the epilogue warps of both CTAs
        }
        bars.abort_flag = 0;
        mbar_fence_init();
        fence_proxy_async_smem();
    }
    if (warp == 1) {
        if (CTAS == 2) { tmem_alloc_pair(&bars.tmem_base, TMEM_COLS); tmem_relinquish_pair(); }
        else { tmem_alloc(&bars.tmem_base, TMEM_COLS); tmem_relinquish(); }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (CTAS == 2) cluster_sync_all();  // the peer's barriers exist before anything is signalled across the pair
    tc_fence_after_sync();
    // Launched with programmatic stream serialisation, the set-up above overlaps the tail of the preceding kernel; nothing
    // before this point touches global memory. Without the launch attribute both instructions are no-ops.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t tmem_base = bars.tmem_base;
    volatile int* abort_flag = &bars.abort_flag;

    // bytes one stage receives: this CTA's A tile and B tile — for a pair, both CTAs' (A tile + half B tile) on the leader's barrier
    const uint32_t stage_tx_bytes = CTAS == 2 ? (uint32_t)(2 * (BM * BK * 2 + (p.BN / 2) * BK * 2)) : (uint32_t)(BM * BK * 2 + p.BN * BK * 2);
    const int bn_local = CTAS == 2 ? p.BN / 2 : p.BN;  // B rows held by this CTA

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            tma_prefetch_desc(&tmA);
            tma_prefetch_desc(&tmB);
            uint32_t c = 0;  // k-block counter across all of this CTA's units
            bool ok = true;
            for (int u = worker; u < units && ok; u += nworkers) {
                int m0, n0, kb0, kb1;
                decode_unit(p, u, m0, n0, kb0, kb1);
                m0 += (int)rank * BM;        // this CTA's rows of the tile
                n0 += (int)rank * bn_local;  // this CTA's part of the B tile
                for (int kb = kb0; kb < kb1; ++kb, ++c) {
                    const int s = c % NST;
                    const uint32_t ph = (c / NST) & 1;
                    if (!mbar_wait(&bars.empty[s], ph ^ 1, abort_flag)) { ok = false; break; }
                    uint8_t* a_dst = sA + s * A_STAGE_BYTES;
                    uint8_t* b_dst = sB + s * BST;
                    const int k0 = kb * BK;
                    if (CTAS == 2) {
                        const uint32_t full_leader = mapa_shared(&bars.full[s], 0);
                        if (rank == 0) mbar_expect_tx(&bars.full[s], stage_tx_bytes);
                        if (!p.a_mn) {
                            tma_load_2d_pair(a_dst, &tmA, full_leader, k0, m0);
                        } else {
                            tma_load_2d_pair(a_dst, &tmA, full_leader, m0, k0);
                            tma_load_2d_pair(a_dst + MN_BOX_BYTES, &tmA, full_leader, m0 + 64, k0);
                        }
                        if (!p.b_mn) {
                            tma_load_2d_pair(b_dst, &tmB, full_leader, k0, n0);
                        } else {
                            for (int j = 0; j < bn_local / 64; ++j)
                                tma_load_2d_pair(b_dst + j * MN_BOX_BYTES, &tmB, full_leader, n0 + 64 * j, k0);
                        }
                        continue;
                    }
                    mbar_expect_tx(&bars.full[s], stage_tx_bytes);
                    if (!p.a_mn) {
                        tma_load_2d(a_dst, &tmA, &bars.full[s], k0, m0);
                    } else {
                        tma_load_2d(a_dst, &tmA, &bars.full[s], m0, k0);
                        tma_load_2d(a_dst + MN_BOX_BYTES, &tmA, &bars.full[s], m0 + 64, k0);
                    }
                    if (!p.b_mn) {
                        tma_load_2d(b_dst, &tmB, &bars.full[s], k0, n0);
                    } else {
                        for (int j = 0; j < p.BN / 64; ++j)
                            tma_load_2d(b_dst + j * MN_BOX_BYTES, &tmB, &bars.full[s], n0 + 64 * j, k0);
                    }
                }
            }
            // Tail: do not let the CTA retire while UMMA commits may still arrive on `empty`.
            for (int i = 0; i < NST && ok; ++i, ++c) {
                const int s = c % NST;
                const uint32_t ph = (c / NST) & 1;
                if (!mbar_wait(&bars.empty[s], ph ^ 1, abort_flag)) ok = false;
            }
        }
    } else if (warp == 1) {
        // ------------------------------ UMMA issuer --------------------------------
        if (lane == 0 && rank == 0) {
            const uint32_t idesc = umma_idesc_bf16_f32(BM * CTAS, p.BN, p.a_mn, p.b_mn);
            // K-major operand: rows of 128 B, 8-row swizzle atoms 1024 B apart; one UMMA (K=16) = 32 B along the row.
            // MN-major operand: 64(mn) x 64(k) boxes of 8 KB; 8-deep k groups 1024 B apart inside a box,
            // 64-wide mn groups one box apart; one UMMA (K=16) = two k groups = 2048 B.
            const uint32_t a_lbo = p.a_mn ? MN_BOX_BYTES : 16, a_sbo = 1024, a_kstep = p.a_mn ? 2048 : 32;
            const uint32_t b_lbo = p.b_mn ? MN_BOX_BYTES : 16, b_sbo = 1024, b_kstep = p.b_mn ? 2048 : 32;
            uint32_t c = 0;
            int it = 0;
            bool ok = true;
            for (int u = worker; u < units && ok; u += nworkers, ++it) {
                int m0, n0, kb0, kb1;
                decode_unit(p, u, m0, n0, kb0, kb1);
                const int buf = it & 1;
                const uint32_t acc_ph = (it >> 1) & 1;
                if (!mbar_wait(&bars.acc_empty[buf], acc_ph ^ 1, abort_flag)) { ok = false; break; }
                tc_fence_after_sync();
                const uint32_t tmem_acc = tmem_base + (uint32_t)buf * MAX_BN;
                for (int kb = kb0; kb < kb1; ++kb, ++c) {
                    const int s = c % NST;
                    const uint32_t ph = (c / NST) & 1;
                    if (!mbar_wait(&bars.full[s], ph, abort_flag)) { ok = false; break; }
                    tc_fence_after_sync();
                    const uint32_t a_addr = smem_u32(sA + s * A_STAGE_BYTES);
                    const uint32_t b_addr = smem_u32(sB + s * BST);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) {
                        const uint64_t ad = umma_smem_desc_sw128(a_addr + k * a_kstep, a_lbo, a_sbo);
                        const uint64_t bd = umma_smem_desc_sw128(b_addr + k * b_kstep, b_lbo, b_sbo);
                        if (CTAS == 2) umma_bf16_ss_pair(tmem_acc, ad, bd, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
                        else umma_bf16_ss(tmem_acc, ad, bd, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
                    }
                    // releases the stage (in both CTAs of a pair) once these UMMAs have read it
                    if (CTAS == 2) umma_commit_pair(&bars.empty[s], 3);
                    else umma_commit(&bars.empty[s]);
                }
                if (ok) {
                    if (CTAS == 2) umma_commit_pair(&bars.acc_full[buf], 3);
                    else umma_commit(&bars.acc_full[buf]);
                }
            }
        }
    } else {
        // ------------------------------ epilogue -----------------------------------
        const int q = warp & 3;
        int it = 0;
        bool ok = true;
        for (int u = worker; u < units && ok; u += nworkers, ++it) {
            int m0, n0, kb0, kb1;
            decode_unit(p, u, m0, n0, kb0, kb1);
            m0 += (int)rank * BM;
            const int buf = it & 1;
            const uint32_t acc_ph = (it >> 1) & 1;
            const int sub = lane & 7, rgrp = lane >> 3;
            const int row_base = m0 + q * 32;
            const bool c_al = (((uintptr_t)p.C) & 15) == 0;
            const bool bf16_fast = p.out_mode == GEMM_OUT_BF16 && c_al && (p.ldc % 8) == 0 && (n0 % 8) == 0 &&
                                   (!p.R || ((((uintptr_t)p.R) & 15) == 0 && (p.ldr % 8) == 0));
            const bool f32_fast = p.out_mode != GEMM_OUT_BF16 && c_al && (p.ldc % 4) == 0 && (n0 % 4) == 0;
            // The residual does not depend on the accumulator: the first chunk's rows are requested before the wait for the
            // UMMAs, every later chunk's while the previous chunk is converted and stored (a global load issued only when its
            // chunk comes up costs a full memory latency per chunk, which made the short-K projections epilogue-bound).
            uint4 rpre[8];
            bool rpre_valid = false;
            if (bf16_fast && p.R && 64 <= p.BN && n0 + 64 <= p.N) {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int grow = row_base + rgrp + 4 * i;
                    rpre[i] = grow < p.M ? *(const uint4*)(p.R + (size_t)grow * p.ldr + n0 + sub * 8) : make_uint4(0u, 0u, 0u, 0u);
                }
                rpre_valid = true;
            }
            ok = mbar_wait(&bars.acc_full[buf], acc_ph, abort_flag);
            ok = __all_sync(0xffffffffu, ok);  // tcgen05.ld is warp-collective: leave together or not at all
            if (!ok) break;
            tc_fence_after_sync();
            const int row = m0 + q * 32 + lane;
            const uint32_t taddr0 = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)buf * MAX_BN;
            // Accumulator rows live one per thread (TMEM lane = output row), but a warp-wide store of one 16-byte piece per
            // row would touch 32 different 128-byte lines. So full chunks go through the warp's staging rows and leave (and
            // the residual arrives) as whole 128-byte row segments, 4 rows per instruction.
            uint8_t* stg = smem + NST * (A_STAGE_BYTES + BST) + q * STG_WARP_BYTES;
            uint8_t* my_row = stg + lane * STG_PITCH;
            for (int c0 = 0; c0 < p.BN;) {
                const int col0 = n0 + c0;
                if (col0 >= p.N) break;
                if (bf16_fast && c0 + 64 <= p.BN && col0 + 64 <= p.N) {
                    uint32_t ra[32], rb2[32];
                    tmem_ld_32x32(taddr0 + c0, ra);
                    tmem_ld_32x32(taddr0 + c0 + 32, rb2);
                    if (p.R) {
                        if (!rpre_valid) {
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                const int grow = row_base + rgrp + 4 * i;
                                rpre[i] = grow < p.M ? *(const uint4*)(p.R + (size_t)grow * p.ldr + col0 + sub * 8) : make_uint4(0u, 0u, 0u, 0u);
                            }
                        }
#pragma unroll
                        for (int i = 0; i < 8; ++i) *(uint4*)(stg + (rgrp + 4 * i) * STG_PITCH + sub * 16) = rpre[i];
                        __syncwarp();
                        // the next 64-column chunk's residual, if there is one
                        rpre_valid = c0 + 128 <= p.BN && col0 + 128 <= p.N;
                        if (rpre_valid) {
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                const int grow = row_base + rgrp + 4 * i;
                                rpre[i] = grow < p.M ? *(const uint4*)(p.R + (size_t)grow * p.ldr + col0 + 64 + sub * 8) : make_uint4(0u, 0u, 0u, 0u);
                            }
                        }
                    }
                    tmem_ld_wait();
#pragma unroll
                    for (int v = 0; v < 8; ++v) {
                        float f[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(v < 4 ? ra[(v & 3) * 8 + i] : rb2[(v & 3) * 8 + i]);
                        if (p.R) {
                            const uint4 rv = *(const uint4*)(my_row + v * 16);
                            const __nv_bfloat162* rb = (const __nv_bfloat162*)&rv;
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const float2 t = __bfloat1622float2(rb[i]);
                                f[2 * i] += t.x;
                                f[2 * i + 1] += t.y;
                            }
                        }
                        uint4 o;
                        __nv_bfloat162* ob = (__nv_bfloat162*)&o;
#pragma unroll
                        for (int i = 0; i < 4; ++i) ob[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
                        *(uint4*)(my_row + v * 16) = o;  // a thread reads and rewrites only its own staging row
                    }
                    __syncwarp();
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int rr = rgrp + 4 * i, grow = row_base + rr;
                        if (grow < p.M)
                            *(uint4*)((__nv_bfloat16*)p.C + (size_t)grow * p.ldc + col0 + sub * 8) = *(const uint4*)(stg + rr * STG_PITCH + sub * 16);
                    }
                    __syncwarp();
                    c0 += 64;
                    continue;
                }
                if (bf16_fast && col0 + 32 <= p.N) {
                    // 32-column remainder of a tile whose width is not a multiple of 64 (e.g. 160): same staging, 64 payload bytes
                    // per row, 4 lanes per row and 8 rows per instruction on the way out
                    uint32_t r[32];
                    tmem_ld_32x32(taddr0 + c0, r);
                    const int sub4 = lane & 3, rgrp8 = lane >> 2;
                    if (p.R) {
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int rr = rgrp8 + 8 * i, grow = row_base + rr;
                            uint4 v = make_uint4(0u, 0u, 0u, 0u);
                            if (grow < p.M) v = *(const uint4*)(p.R + (size_t)grow * p.ldr + col0 + sub4 * 8);
                            *(uint4*)(stg + rr * STG_PITCH + sub4 * 16) = v;
                        }
                        __syncwarp();
                    }
                    tmem_ld_wait();
#pragma unroll
                    for (int v = 0; v < 4; ++v) {
                        float f[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(r[v * 8 + i]);
                        if (p.R) {
                            const uint4 rv = *(const uint4*)(my_row + v * 16);
                            const __nv_bfloat162* rb = (const __nv_bfloat162*)&rv;
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const float2 t = __bfloat1622float2(rb[i]);
                                f[2 * i] += t.x;
                                f[2 * i + 1] += t.y;
                            }
                        }
                        uint4 o;
                        __nv_bfloat162* ob = (__nv_bfloat162*)&o;
#pragma unroll
                        for (int i = 0; i < 4; ++i) ob[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
                        *(uint4*)(my_row + v * 16) = o;
                    }
                    __syncwarp();
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int rr = rgrp8 + 8 * i, grow = row_base + rr;
                        if (grow < p.M)
                            *(uint4*)((__nv_bfloat16*)p.C + (size_t)grow * p.ldc + col0 + sub4 * 8) = *(const uint4*)(stg + rr * STG_PITCH + sub4 * 16);
                    }
                    __syncwarp();
                    c0 += 32;
                    continue;
                }
                if (f32_fast && col0 + 32 <= p.N) {
                    uint32_t r[32];
                    tmem_ld_32x32(taddr0 + c0, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int v = 0; v < 8; ++v) *(uint4*)(my_row + v * 16) = make_uint4(r[v * 4], r[v * 4 + 1], r[v * 4 + 2], r[v * 4 + 3]);
                    __syncwarp();
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int rr = rgrp + 4 * i, grow = row_base + rr;
                        if (grow < p.M) {
                            const uint4 v = *(const uint4*)(stg + rr * STG_PITCH + sub * 16);
                            float* dst = (float*)p.C + (size_t)grow * p.ldc + col0 + sub * 4;
                            if (p.out_mode == GEMM_OUT_F32) {
                                *(uint4*)dst = v;
                            } else {
                                asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(__uint_as_float(v.x)),
                                             "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
                                             : "memory");
                            }
                        }
                    }
                    __syncwarp();
                    c0 += 32;
                    continue;
                }
                // ragged or unaligned chunk: one row per thread, element by element where needed
                uint32_t r[32];
                tmem_ld_32x32(taddr0 + c0, r);
                tmem_ld_wait();
                c0 += 32;
                if (row < p.M) {
                    const int ncols = min(32, p.N - col0);
                    if (p.out_mode == GEMM_OUT_BF16) {
                        __nv_bfloat16* crow = (__nv_bfloat16*)p.C + (size_t)row * p.ldc + col0;
                        const __nv_bfloat16* rrow = p.R ? p.R + (size_t)row * p.ldr + col0 : nullptr;
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            if (i < ncols) {
                                float f = __uint_as_float(r[i]);
                                if (rrow) f += __bfloat162float(rrow[i]);
                                crow[i] = __float2bfloat16_rn(f);
                            }
                        }
                    } else if (p.out_mode == GEMM_OUT_F32) {
                        float* crow = (float*)p.C + (size_t)row * p.ldc + col0;
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (i < ncols) crow[i] = __uint_as_float(r[i]);
                    } else {
                        float* crow = (float*)p.C + (size_t)row * p.ldc + col0;
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (i < ncols) atomicAdd(crow + i, __uint_as_float(r[i]));
                    }
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                if (CTAS == 2 && rank != 0) mbar_arrive_cluster(mapa_shared(&bars.acc_empty[buf], 0));
                else mbar_arrive(&bars.acc_empty[buf]);
            }
        }
    }

    // ------------------------------ teardown ---------------------------------------
    __syncwarp();
    if (*abort_flag) {
        // A wait ran out: give copies and UMMAs still in flight time to land before the
        // shared memory and TMEM they target are released.
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 2000000ull) __nanosleep(1000);
        if (threadIdx.x == 0 && p.err) atomicExch(p.err, 1000 + (int)blockIdx.x);
    }
    tc_fence_before_sync();
    __syncthreads();
    if (CTAS == 2) cluster_sync_all();  // no signal of the peer may still be on its way to this CTA's barriers
    tc_fence_after_sync();
    if (warp == 1) {
        if (CTAS == 2) tmem_dealloc_pair(tmem_base, TMEM_COLS);
        else tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ---------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

// 2-D bf16 tensor map with 128B swizzle. inner/outer extents in elements, row pitch `ld` in elements.
int make_map(CUtensorMap* tm, const void* base, uint64_t inner, uint64_t outer, uint64_t ld, uint32_t box_inner,
             uint32_t box_outer) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return -10;
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {ld * 2};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void*)base, dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : -11;
}

// pair: B is split over the two CTAs, so an MN-major B tile must be two whole 64-wide boxes per CTA
int choose_tile_n(int N, int b_mn, int ctas) {
    const int step = b_mn ? 64 * ctas : 32;
    int best = 64;
    double best_cost = 1e30;
    for (int bn = (step > 64 ? step : 64); bn <= MAX_BN; bn += step) {
        const double padded = (double)((N + bn - 1) / bn) * bn;
        const double cost = padded * (1.0 + 24.0 / bn);
        if (cost < best_cost - 1e-9 || (cost < best_cost + 1e-9 && bn > best)) {
            best_cost = cost;
            best = bn;
        }
    }
    return best;
}

std::atomic<long> g_launches{0};

}  // namespace

long gemm_bf16_umma_launch_count() { return g_launches.load(); }

int gemm_bf16_umma(const GemmProblem& g, int* err_flag, cudaStream_t stream) {
    if (g.M <= 0 || g.N <= 0 || g.K <= 0) return -1;
    if ((g.lda % 8) || (g.ldb % 8)) return -2;  // TMA: row pitch must be a multiple of 16 bytes
    if ((((uintptr_t)g.A) & 15) || (((uintptr_t)g.B) & 15)) return -3;
    if (g.splits > 1 && g.out_mode != GEMM_OUT_F32_ATOMIC) return -4;

    static std::atomic<unsigned long long> attr_done{0};
    static const bool pair_off = getenv("BM_GEMM_1CTA") != nullptr;
    if (first_use_on_current_device(attr_done)) {
        cudaError_t e = cudaFuncSetAttribute(gemm_bf16_umma_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_DYN_BYTES);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_bf16_umma_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_DYN_BYTES);
        if (e != cudaSuccess) return -5;
    }
    const int g_num_sms = sm_count_current_device();

    // CTA pairs (256-row tiles) whenever there are at least 256 rows and the caller did not fix a narrow tile
    const int ctas = (!pair_off && g.M >= 2 * BM && g.tile_n == 0) ? 2 : 1;
    KArgs p;
    p.M = g.M; p.N = g.N; p.K = g.K;
    p.BN = g.tile_n > 0 ? g.tile_n : choose_tile_n(g.N, g.b_mn_major, ctas);
    if (p.BN < 32 || p.BN > MAX_BN || (p.BN % 32) || (g.b_mn_major && (p.BN % (64 * ctas)))) return -6;
    p.tile_rows = BM * ctas;
    p.a_mn = g.a_mn_major ? 1 : 0;
    p.b_mn = g.b_mn_major ? 1 : 0;
    p.tiles_m = (g.M + p.tile_rows - 1) / p.tile_rows;
    p.tiles_n = (g.N + p.BN - 1) / p.BN;
    p.kb_total = (g.K + BK - 1) / BK;
    int splits = g.splits > 0 ? g.splits : 1;
    if (g.splits <= 0 && g.out_mode == GEMM_OUT_F32_ATOMIC) {
        // Split the reduction axis so that the waves of work units fill the machine: minimise
        // waves x (k-blocks per unit + a fixed cost per unit for pipeline fill and the accumulator drain).
        const long workers = ctas == 2 ? g_num_sms / 2 : g_num_sms;
        const long tiles = (long)p.tiles_m * p.tiles_n;
        long best = -1;
        const int max_s = p.kb_total / 4 > 16 ? 16 : (p.kb_total / 4 > 1 ? p.kb_total / 4 : 1);
        for (int sp = 1; sp <= max_s; ++sp) {
            const long waves = (tiles * sp + workers - 1) / workers;
            const long cost = waves * ((p.kb_total + sp - 1) / sp + 8);
            if (best < 0 || cost < best) { best = cost; splits = sp; }
        }
    }
    if (splits > p.kb_total) splits = p.kb_total;
    p.kb_per_split = (p.kb_total + splits - 1) / splits;
    p.splits = (p.kb_total + p.kb_per_split - 1) / p.kb_per_split;
    p.C = g.C; p.ldc = g.ldc; p.out_mode = g.out_mode;
    p.R = g.R; p.ldr = g.ldr;
    p.err = err_flag;

    CUtensorMap tmA, tmB;
    int rc;
    if (!p.a_mn) rc = make_map(&tmA, g.A, (uint64_t)g.K, (uint64_t)g.M, (uint64_t)g.lda, BK, BM);
    else         rc = make_map(&tmA, g.A, (uint64_t)g.M, (uint64_t)g.K, (uint64_t)g.lda, 64, BK);
    if (rc) return rc;
    if (!p.b_mn) rc = make_map(&tmB, g.B, (uint64_t)g.K, (uint64_t)g.N, (uint64_t)g.ldb, BK, (uint32_t)(p.BN / ctas));
    else         rc = make_map(&tmB, g.B, (uint64_t)g.N, (uint64_t)g.K, (uint64_t)g.ldb, 64, BK);
    if (rc) return rc;

    const long units = (long)p.tiles_m * p.tiles_n * p.splits;
    g_launches.fetch_add(1);
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(NUM_THREADS);
    cfg.dynamicSmemBytes = SMEM_DYN_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute at[2];
    int na = 0;
    if (g.pdl) {
        at[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    if (ctas == 2) {
        at[na].id = cudaLaunchAttributeClusterDimension;
        at[na].val.clusterDim.x = 2;
        at[na].val.clusterDim.y = 1;
        at[na].val.clusterDim.z = 1;
        ++na;
        const int pairs = g_num_sms / 2;
        cfg.gridDim = dim3((unsigned)(2 * (units < pairs ? units : pairs)));
        cfg.attrs = at;
        cfg.numAttrs = na;
        return cudaLaunchKernelEx(&cfg, gemm_bf16_umma_kernel<2>, tmA, tmB, p) == cudaSuccess ? 0 : -7;
    }
    cfg.gridDim = dim3((unsigned)(units < g_num_sms ? units : g_num_sms));
    cfg.attrs = at;
    cfg.numAttrs = na;
    return cudaLaunchKernelEx(&cfg, gemm_bf16_umma_kernel<1>, tmA, tmB, p) == cudaSuccess ? 0 : -7;
}

}  // namespace bmb
