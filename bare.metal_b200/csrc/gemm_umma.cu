// Persistent, warp-specialised tcgen05 GEMM. See gemm_umma.cuh for the operand convention.
//
// CTA = 192 threads: warp 0 = TMA producer, warp 1 = TMEM owner + UMMA issuer, warps 2..5 = epilogue (warp w reads TMEM lanes 32*(w&3) .. +31; the two warps of a lane quarter split the columns).
// Tile = 128 (M) x tile_n (N, <= 256) x 64 (K per stage), shared-memory ring of as many stages as fit (3 to 8),
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
constexpr int KPS = 2;            // 64-deep k-blocks per ring stage. A stage costs its issuing thread one barrier wait and one commit
                                  // (about 250 cycles together, more than the 53 an instruction issue costs), so with one k-block
                                  // per stage the thread needed ~520 cycles for the 512 the tensor pipe takes at 256 columns and
                                  // could never run ahead of it; two k-blocks per stage halve that share.
constexpr int MAX_STAGES = 8;     // ring stages: as many KPS x (16 KB of A + this CTA's rows of B) as fit, see ring_stages()
constexpr int MAX_BN = 256;
constexpr int A_STAGE_BYTES = BM * BK * 2;      // 16 KB
constexpr int MN_BOX_BYTES = 64 * BK * 2;       // one 64(mn) x 64(k) box of an MN-major operand
constexpr int EPI_WARPS = 4;      // one epilogue warp per TMEM lane quarter (eight, two per quarter splitting the columns, measured slower:
                                  // every GEMM of the step lost 5-14 % while only the heaviest epilogue gained)
constexpr int NUM_THREADS = 64 + 32 * EPI_WARPS;
// Epilogue staging: each of the 4 epilogue warps owns 32 rows x 128 payload bytes (64 bf16 or 32 fp32 columns) at a
// 144-byte pitch, which makes both the row-per-thread accesses and the 8-lanes-per-row accesses bank-conflict free.
constexpr int STG_PITCH = 144;
constexpr int STG_WARP_BYTES = 32 * STG_PITCH;
constexpr int RING_BYTES = 192 * 1024;  // what the operand ring may use: 227 KB less the staging rows and the alignment slack
constexpr int SMEM_DYN_BYTES = RING_BYTES + EPI_WARPS * STG_WARP_BYTES + 1024;
static_assert(SMEM_DYN_BYTES <= 227 * 1024, "shared memory budget");
// stages of KPS x (A tile + bn_local rows of B, 128 bytes each) that fit in the ring
__host__ __device__ inline int ring_stages(int bn_local) {
    const int n = RING_BYTES / (KPS * (A_STAGE_BYTES + bn_local * BK * 2));
    return n > MAX_STAGES ? MAX_STAGES : n;
}
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
    void* C2;
    int ldc2;
    float* aux;
    int aux_S, aux_NH;
};

struct __align__(8) Barriers {
    uint64_t full[MAX_STAGES];
    uint64_t empty[MAX_STAGES];
    uint64_t acc_full[2];
    uint64_t acc_empty[2];
    uint32_t tmem_base;
    int abort_flag;
};

// Work unit -> tile. Tiles run row-tile-major (all column tiles of a row tile are neighbours, so one wave of CTAs shares its A
// rows) inside column groups of RASTER_GN tiles: with more column tiles than that (the LM head has 192) a wave would otherwise
// sweep tens of MB of B per row tile and, with C streaming through L2 beside it, fetch B from DRAM once per row tile (measured:
// 1.7 GB of DRAM reads for 110 MB of operands at 8192 rows). Inside a group B's slice stays in L2 for every row tile.
constexpr int RASTER_GN = 32;
__device__ __forceinline__ void decode_unit(const KArgs& p, int u, int& m0, int& n0, int& kb0, int& kb1) {
    const int ntiles = p.tiles_m * p.tiles_n;
    const int split = u / ntiles;
    const int tile = u - split * ntiles;
    int tm, tn;
    if (p.tiles_n <= RASTER_GN) {
        tm = tile / p.tiles_n;
        tn = tile - tm * p.tiles_n;
    } else {
        const int per_group = RASTER_GN * p.tiles_m;
        const int g = tile / per_group;
        const int idx = tile - g * per_group;
        const int w = min(RASTER_GN, p.tiles_n - g * RASTER_GN);   // the last group may be narrower
        tm = idx / w;
        tn = g * RASTER_GN + (idx - tm * w);
    }
    m0 = tm * p.tile_rows;
    n0 = tn * p.BN;
    kb0 = split * p.kb_per_split;
    kb1 = min(p.kb_total, kb0 + p.kb_per_split);
}

// CTAS = 1: one CTA computes a 128 x BN tile. CTAS = 2: the kernel is launched in clusters of two CTAs on neighbouring SMs; the
// pair computes a 256 x BN tile with tcgen05.mma.cta_group::2 — each CTA holds its 128 rows of A and HALF of the B tile, the
// leader (cluster rank 0) issues the UMMAs, each CTA's TMEM receives its 128 rows of the accumulator and each CTA runs its own
// epilogue. B is read from shared memory once per pair instead of once per CTA.
template <int CTAS, int EPI>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_bf16_umma_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                      const KArgs p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ Barriers bars;

    // 1024-byte alignment: the 128B swizzle pattern is a function of address bits [7,10).
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int bn_local = CTAS == 2 ? p.BN / 2 : p.BN;  // B rows held by this CTA
    const int BST = bn_local * BK * 2;
    const int NST = ring_stages(bn_local);
    uint8_t* sA = smem;                              // stage s: KPS A tiles at sA + s * KPS * A_STAGE_BYTES
    uint8_t* sB = smem + NST * KPS * A_STAGE_BYTES;  // stage s: KPS B tiles at sB + s * KPS * BST
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
            mbar_init(&bars.acc_empty[b], EPI_WARPS * CTAS);  // pair: the leader's collects the epilogue warps of both CTAs
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


    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            tma_prefetch_desc(&tmA);
            tma_prefetch_desc(&tmB);
            int s = 0;        // ring stage and its phase, advanced per k-block across all of this CTA's units
            uint32_t ph = 0;
            bool ok = true;
            for (int u = worker; u < units && ok; u += nworkers) {
                int m0, n0, kb0, kb1;
                decode_unit(p, u, m0, n0, kb0, kb1);
                m0 += (int)rank * BM;        // this CTA's rows of the tile
                // gated forward: the tile's first half comes from the gate rows h0.., its second half from the up rows H + h0..
                const int n_second = EPI == GEMM_EPI_SWIGLU_FWD ? p.N / 2 + (n0 / p.BN) * (p.BN / 2) : 0;
                if (EPI == GEMM_EPI_SWIGLU_FWD) n0 = CTAS == 2 ? (rank ? n_second : (n0 / p.BN) * (p.BN / 2)) : (n0 / p.BN) * (p.BN / 2);
                else n0 += (int)rank * bn_local;  // this CTA's part of the B tile
                for (int kb = kb0; kb < kb1; kb += KPS, s = (s + 1 == NST ? 0 : s + 1), ph ^= (s == 0)) {
                    if (!mbar_wait(&bars.empty[s], ph ^ 1, abort_flag)) { ok = false; break; }
                    const int g = min(KPS, kb1 - kb);   // k-blocks in this stage (the last stage of a unit may hold fewer)
                    uint8_t* a_stage = sA + s * KPS * A_STAGE_BYTES;
                    uint8_t* b_stage = sB + s * KPS * BST;
                    const int k0 = kb * BK;
                    // A K-major operand arrives one k-block per copy (a 128-byte swizzled row cannot be wider than 64 elements).
                    // An MN-major operand arrives one 64-wide group of rows per copy, KPS k-blocks deep: a copy costs the issuing
                    // thread as much as a UMMA costs its thread, and the weight-gradient GEMMs (both operands MN-major, four
                    // copies per k-block) were bound by this thread. Such a box always holds KPS k-blocks, also when the unit ends
                    // after the first (what lies beyond K is zero-filled; what lies beyond the unit's split is not used).
                    const uint32_t tx = (uint32_t)((p.a_mn ? KPS : g) * A_STAGE_BYTES + (p.b_mn ? KPS : g) * BST) * (CTAS == 2 ? 2u : 1u);
                    if (CTAS == 2) {
                        const uint32_t full_leader = mapa_shared(&bars.full[s], 0);
                        if (rank == 0) mbar_expect_tx(&bars.full[s], tx);
                        if (!p.a_mn) {
                            for (int j = 0; j < g; ++j) tma_load_2d_pair(a_stage + j * A_STAGE_BYTES, &tmA, full_leader, k0 + j * BK, m0);
                        } else {
                            tma_load_2d_pair(a_stage, &tmA, full_leader, m0, k0);
                            tma_load_2d_pair(a_stage + KPS * MN_BOX_BYTES, &tmA, full_leader, m0 + 64, k0);
                        }
                        if (!p.b_mn) {
                            for (int j = 0; j < g; ++j) tma_load_2d_pair(b_stage + j * BST, &tmB, full_leader, k0 + j * BK, n0);
                        } else {
                            for (int jb = 0; jb < bn_local / 64; ++jb)
                                tma_load_2d_pair(b_stage + jb * KPS * MN_BOX_BYTES, &tmB, full_leader, n0 + 64 * jb, k0);
                        }
                        continue;
                    }
                    mbar_expect_tx(&bars.full[s], tx);
                    if (!p.a_mn) {
                        for (int j = 0; j < g; ++j) tma_load_2d(a_stage + j * A_STAGE_BYTES, &tmA, &bars.full[s], k0 + j * BK, m0);
                    } else {
                        tma_load_2d(a_stage, &tmA, &bars.full[s], m0, k0);
                        tma_load_2d(a_stage + KPS * MN_BOX_BYTES, &tmA, &bars.full[s], m0 + 64, k0);
                    }
                    if (EPI == GEMM_EPI_SWIGLU_FWD) {
                        for (int j = 0; j < g; ++j) {
                            tma_load_2d(b_stage + j * BST, &tmB, &bars.full[s], k0 + j * BK, n0);
                            tma_load_2d(b_stage + j * BST + (p.BN / 2) * BK * 2, &tmB, &bars.full[s], k0 + j * BK, n_second);
                        }
                    } else if (!p.b_mn) {
                        for (int j = 0; j < g; ++j) tma_load_2d(b_stage + j * BST, &tmB, &bars.full[s], k0 + j * BK, n0);
                    } else {
                        for (int jb = 0; jb < p.BN / 64; ++jb)
                            tma_load_2d(b_stage + jb * KPS * MN_BOX_BYTES, &tmB, &bars.full[s], n0 + 64 * jb, k0);
                    }
                }
            }
            // Tail: do not let the CTA retire while UMMA commits may still arrive on `empty`.
            for (int i = 0; i < NST && ok; ++i, s = (s + 1 == NST ? 0 : s + 1), ph ^= (s == 0)) {
                if (!mbar_wait(&bars.empty[s], ph ^ 1, abort_flag)) ok = false;
            }
        }
    } else if (warp == 1) {
        // ------------------------------ UMMA issuer --------------------------------
        if (lane == 0 && rank == 0) {
            const uint32_t idesc = umma_idesc_bf16_f32(BM * CTAS, p.BN, p.a_mn, p.b_mn);
            // K-major operand: rows of 128 B, 8-row swizzle atoms 1024 B apart; one UMMA (K=16) = 32 B along the row.
            // MN-major operand: per 64-wide mn group one box of 64(mn) x KPS*64(k), KPS * 8 KB; 8-deep k groups 1024 B apart inside
            // a box, mn groups one box apart; one UMMA (K=16) = two k groups = 2048 B; a k-block = 8 KB further into every box.
            const uint32_t a_lbo = p.a_mn ? KPS * MN_BOX_BYTES : 16, a_sbo = 1024, a_kstep = p.a_mn ? 2048 : 32;
            const uint32_t b_lbo = p.b_mn ? KPS * MN_BOX_BYTES : 16, b_sbo = 1024, b_kstep = p.b_mn ? 2048 : 32;
            // One thread issues every UMMA, so the instructions between two of them are on the critical path whenever a UMMA
            // is shorter than they are (tiles narrower than 256 columns). The descriptors of stage 0 are built once; a stage or a
            // k step only moves the 14-bit start-address field (units of 16 bytes; shared memory ends below 256 KB, so the
            // field never carries into its neighbour).
            const uint64_t adesc0 = umma_smem_desc_sw128(smem_u32(sA), a_lbo, a_sbo);
            const uint64_t bdesc0 = umma_smem_desc_sw128(smem_u32(sB), b_lbo, b_sbo);
            const uint32_t a_kb16 = (p.a_mn ? MN_BOX_BYTES : A_STAGE_BYTES) >> 4;             // one k-block inside a stage
            const uint32_t b_kb16 = (uint32_t)(p.b_mn ? MN_BOX_BYTES : BST) >> 4;
            const uint32_t a_st16 = KPS * (A_STAGE_BYTES >> 4), b_st16 = KPS * ((uint32_t)BST >> 4), a_k16 = a_kstep >> 4, b_k16 = b_kstep >> 4;
            int s = 0;
            uint32_t ph = 0, a_off = 0, b_off = 0;   // stage s starts a_off / b_off sixteen-byte units into its ring
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
                uint32_t acc = 0u;   // the tile's first UMMA overwrites the accumulator
                for (int kb = kb0; kb < kb1; kb += KPS) {
                    if (!mbar_wait(&bars.full[s], ph, abort_flag)) { ok = false; break; }
                    tc_fence_after_sync();
                    const int g = min(KPS, kb1 - kb);
                    uint32_t ja = a_off, jb = b_off;
                    for (int j = 0; j < g; ++j, ja += a_kb16, jb += b_kb16) {
                        uint64_t ad = adesc0 + ja, bd = bdesc0 + jb;
#pragma unroll
                        for (int k = 0; k < BK / 16; ++k) {
                            if (CTAS == 2) umma_bf16_ss_pair(tmem_acc, ad, bd, idesc, acc);
                            else umma_bf16_ss(tmem_acc, ad, bd, idesc, acc);
                            acc = 1u;
                            ad += a_k16;
                            bd += b_k16;
                        }
                    }
                    // releases the stage (in both CTAs of a pair) once these UMMAs have read it
                    if (CTAS == 2) umma_commit_pair(&bars.empty[s], 3);
                    else umma_commit(&bars.empty[s]);
                    if (++s == NST) { s = 0; ph ^= 1u; a_off = 0; b_off = 0; }
                    else { a_off += a_st16; b_off += b_st16; }
                }
                if (ok) {
                    if (CTAS == 2) umma_commit_pair(&bars.acc_full[buf], 3);
                    else umma_commit(&bars.acc_full[buf]);
                }
            }
        }
    } else {
        // ------------------------------ epilogue -----------------------------------
        // Warp w may touch TMEM lanes 32 * (w % 4) .. +31 (a hardware rule). With more than one warp per lane quarter the warps
        // of a quarter split the tile's columns: [0, cmid) and [cmid, BN), cmid a multiple of 64.
        const int q = warp & 3;
        const int ew = warp - 2, hsel = ew >> 2;
        const int cmid = EPI_WARPS > 4 ? min(p.BN, ((p.BN / 32 + 3) / 4) * 64) : p.BN;
        const int c_lo = hsel ? cmid : 0, c_hi = hsel ? p.BN : cmid;
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
            if constexpr (EPI == GEMM_EPI_SWIGLU_FWD || EPI == GEMM_EPI_SWIGLU_BWD) {
                // Both gated-MLP epilogues move rows as [first 32 columns | second 32 columns] = 2 x 64 bytes through the warp's
                // staging rows: lanes 0-3 of a row carry the piece that belongs at column h, lanes 4-7 the piece at column H + h.
                uint8_t* stg = smem + NST * KPS * (A_STAGE_BYTES + BST) + ew * STG_WARP_BYTES;
                uint8_t* my_row = stg + lane * STG_PITCH;
                const uint32_t taddr0 = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)buf * MAX_BN;
                const int piece = sub & 3, second = sub >> 2;
                if constexpr (EPI == GEMM_EPI_SWIGLU_FWD) {
                    const int half = p.BN / 2, H = p.N / 2;
                    const int h0 = (n0 / p.BN) * half;
                    __nv_bfloat16* Cgu = (__nv_bfloat16*)p.C;
                    __nv_bfloat16* Cact = (__nv_bfloat16*)p.C2;
                    ok = mbar_wait(&bars.acc_full[buf], acc_ph, abort_flag);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    tc_fence_after_sync();
                    for (int c0 = c_lo / 2; c0 < c_hi / 2 && h0 + c0 < H; c0 += 64) {
                        uint32_t pa[32];  // act of 64 hidden units, packed bf16 pairs
#pragma unroll
                        for (int sc = 0; sc < 2; ++sc) {
                            uint32_t g[32], u[32];
                            tmem_ld_32x32(taddr0 + c0 + sc * 32, g);
                            tmem_ld_32x32(taddr0 + half + c0 + sc * 32, u);
                            tmem_ld_wait();
                            uint32_t pg[16], pu[16];
#pragma unroll
                            for (int i = 0; i < 16; ++i) {
                                // act is computed from the stored (bf16-rounded) gate and up, which is what the backward differentiates
                                const __nv_bfloat162 gb = __floats2bfloat162_rn(__uint_as_float(g[2 * i]), __uint_as_float(g[2 * i + 1]));
                                const __nv_bfloat162 ub = __floats2bfloat162_rn(__uint_as_float(u[2 * i]), __uint_as_float(u[2 * i + 1]));
                                const float2 gf = __bfloat1622float2(gb), uf = __bfloat1622float2(ub);
                                const float2 a2 = f2_mul(f2_mul(gf, sigmoid2_approx(gf)), uf);   // silu(gate) * up
                                const __nv_bfloat162 ab = __floats2bfloat162_rn(a2.x, a2.y);
                                pg[i] = *(const uint32_t*)&gb;
                                pu[i] = *(const uint32_t*)&ub;
                                pa[sc * 16 + i] = *(const uint32_t*)&ab;
                            }
#pragma unroll
                            for (int v = 0; v < 4; ++v) {
                                *(uint4*)(my_row + v * 16) = make_uint4(pg[4 * v], pg[4 * v + 1], pg[4 * v + 2], pg[4 * v + 3]);
                                *(uint4*)(my_row + 64 + v * 16) = make_uint4(pu[4 * v], pu[4 * v + 1], pu[4 * v + 2], pu[4 * v + 3]);
                            }
                            __syncwarp();
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                const int rr = rgrp + 4 * i, grow = row_base + rr;
                                if (grow < p.M)
                                    *(uint4*)(Cgu + (size_t)grow * p.ldc + (second ? H : 0) + h0 + c0 + sc * 32 + piece * 8) =
                                        *(const uint4*)(stg + rr * STG_PITCH + sub * 16);
                            }
                            __syncwarp();
                        }
#pragma unroll
                        for (int v = 0; v < 8; ++v) *(uint4*)(my_row + v * 16) = make_uint4(pa[4 * v], pa[4 * v + 1], pa[4 * v + 2], pa[4 * v + 3]);
                        __syncwarp();
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const int rr = rgrp + 4 * i, grow = row_base + rr;
                            if (grow < p.M)
                                *(uint4*)(Cact + (size_t)grow * p.ldc2 + h0 + c0 + sub * 8) = *(const uint4*)(stg + rr * STG_PITCH + sub * 16);
                        }
                        __syncwarp();
                    }
                } else {
                    const int H = p.N;
                    __nv_bfloat16* Cd = (__nv_bfloat16*)p.C;
                    // saved gate | up of the first 32 columns are requested before the wait for the accumulator, every later
                    // group while the previous one is being worked on
                    // Two register buffers keep the saved gate | up rows two 32-column groups ahead of their use (the first two are
                    // requested before the wait for the accumulator), and the rows of the NEXT tile are pulled into L2 a whole tile
                    // ahead: with one warp per scheduler nothing else hides the memory latency.
                    uint4 preA[8], preB[8];
                    auto fetch = [&](uint4 (&pre)[8], int c0) {
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const int grow = row_base + rgrp + 4 * i;
                            pre[i] = (grow < p.M && n0 + c0 < H) ? *(const uint4*)(p.R + (size_t)grow * p.ldr + (second ? H : 0) + n0 + c0 + piece * 8)
                                                               : make_uint4(0u, 0u, 0u, 0u);
                        }
                    };
                    fetch(preA, c_lo);
                    fetch(preB, c_lo + 32);
                    if (u + nworkers < units) {
                        int m1, n1, ka, kb;
                        decode_unit(p, u + nworkers, m1, n1, ka, kb);
                        const int prow = m1 + (int)rank * BM + q * 32 + lane;
                        if (prow < p.M) {
                            const __nv_bfloat16* g0 = p.R + (size_t)prow * p.ldr + n1;
                            for (int b = c_lo * 2; b < c_hi * 2 && n1 + b / 2 < H; b += 128) {
                                prefetch_l2((const uint8_t*)g0 + b);
                                prefetch_l2((const uint8_t*)(g0 + H) + b);
                            }
                        }
                    }
                    ok = mbar_wait(&bars.acc_full[buf], acc_ph, abort_flag);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    tc_fence_after_sync();
                    auto process = [&](uint4 (&pre)[8], int c0) {
                        uint32_t d[32];
                        tmem_ld_32x32(taddr0 + c0, d);
#pragma unroll
                        for (int i = 0; i < 8; ++i) *(uint4*)(stg + (rgrp + 4 * i) * STG_PITCH + sub * 16) = pre[i];
                        __syncwarp();
                        if (c0 + 64 < c_hi) fetch(pre, c0 + 64);
                        tmem_ld_wait();
#pragma unroll
                        for (int v = 0; v < 4; ++v) {
                            const uint4 gv = *(const uint4*)(my_row + v * 16), uv = *(const uint4*)(my_row + 64 + v * 16);
                            const __nv_bfloat162* gb = (const __nv_bfloat162*)&gv;
                            const __nv_bfloat162* ub = (const __nv_bfloat162*)&uv;
                            uint4 og, ou;
                            __nv_bfloat162* ogb = (__nv_bfloat162*)&og;
                            __nv_bfloat162* oub = (__nv_bfloat162*)&ou;
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                // dgate = dact * up * s * (1 + x * (1 - s)), dup = dact * x * s, s = sigmoid(x)
                                const float2 x = __bfloat1622float2(gb[i]), uu = __bfloat1622float2(ub[i]);
                                const float2 dd = make_float2(__uint_as_float(d[v * 8 + 2 * i]), __uint_as_float(d[v * 8 + 2 * i + 1]));
                                const float2 sg = sigmoid2_approx(x);
                                const float2 xs = f2_mul(x, sg);
                                const float2 oms = f2_fma(sg, make_float2(-1.f, -1.f), make_float2(1.f, 1.f));
                                const float2 w = f2_fma(x, oms, make_float2(1.f, 1.f));
                                const float2 dg = f2_mul(f2_mul(dd, uu), f2_mul(sg, w));
                                const float2 du = f2_mul(dd, xs);
                                ogb[i] = __floats2bfloat162_rn(dg.x, dg.y);
                                oub[i] = __floats2bfloat162_rn(du.x, du.y);
                            }
                            *(uint4*)(my_row + v * 16) = og;
                            *(uint4*)(my_row + 64 + v * 16) = ou;
                        }
                        __syncwarp();
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const int rr = rgrp + 4 * i, grow = row_base + rr;
                            if (grow < p.M)
                                *(uint4*)(Cd + (size_t)grow * p.ldc + (second ? H : 0) + n0 + c0 + piece * 8) = *(const uint4*)(stg + rr * STG_PITCH + sub * 16);
                        }
                        __syncwarp();
                    };
                    for (int c0 = c_lo; c0 < c_hi && n0 + c0 < H; c0 += 64) {
                        process(preA, c0);
                        if (n0 + c0 + 32 < H) process(preB, c0 + 32);
                    }
                }
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) {
                    if (CTAS == 2 && rank != 0) mbar_arrive_cluster(mapa_shared(&bars.acc_empty[buf], 0));
                    else mbar_arrive(&bars.acc_empty[buf]);
                }
                continue;
            }
            const bool c_al = (((uintptr_t)p.C) & 15) == 0;
            const bool bf16_fast = p.out_mode == GEMM_OUT_BF16 && c_al && (p.ldc % 8) == 0 && (n0 % 8) == 0 &&
                                   (!p.R || ((((uintptr_t)p.R) & 15) == 0 && (p.ldr % 8) == 0));
            const bool f32_fast = p.out_mode != GEMM_OUT_BF16 && c_al && (p.ldc % 4) == 0 && (n0 % 4) == 0;
            // The residual does not depend on the accumulator: the first chunk's rows are requested before the wait for the
            // UMMAs, every later chunk's while the previous chunk is converted and stored (a global load issued only when its
            // chunk comes up costs a full memory latency per chunk, which made the short-K projections epilogue-bound).
            if (p.R && u + nworkers < units) {   // the next tile's rows of R are pulled into L2 a whole tile ahead of their use
                int m1, n1, ka, kb;
                decode_unit(p, u + nworkers, m1, n1, ka, kb);
                const int prow = m1 + (int)rank * BM + q * 32 + lane;
                if (prow < p.M && bf16_fast)
                    for (int b = c_lo * 2; b < c_hi * 2 && n1 + b / 2 < p.N; b += 128) prefetch_l2((const uint8_t*)(p.R + (size_t)prow * p.ldr + n1) + b);
            }
            uint4 rpre[8];
            bool rpre_valid = false;
            if (bf16_fast && p.R && c_lo + 64 <= c_hi && n0 + c_lo + 64 <= p.N) {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int grow = row_base + rgrp + 4 * i;
                    rpre[i] = grow < p.M ? *(const uint4*)(p.R + (size_t)grow * p.ldr + n0 + c_lo + sub * 8) : make_uint4(0u, 0u, 0u, 0u);
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
            uint8_t* stg = smem + NST * KPS * (A_STAGE_BYTES + BST) + ew * STG_WARP_BYTES;
            uint8_t* my_row = stg + lane * STG_PITCH;
            for (int c0 = c_lo; c0 < c_hi;) {
                const int col0 = n0 + c0;
                if (col0 >= p.N) break;
                if (bf16_fast && c0 + 64 <= c_hi && col0 + 64 <= p.N) {
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
                        rpre_valid = c0 + 128 <= c_hi && col0 + 128 <= p.N;
                        if (rpre_valid) {
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                const int grow = row_base + rgrp + 4 * i;
                                rpre[i] = grow < p.M ? *(const uint4*)(p.R + (size_t)grow * p.ldr + col0 + 64 + sub * 8) : make_uint4(0u, 0u, 0u, 0u);
                            }
                        }
                    }
                    tmem_ld_wait();
                    float rowdot = 0.f;
#pragma unroll
                    for (int v = 0; v < 8; ++v) {
                        float f[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(v < 4 ? ra[(v & 3) * 8 + i] : rb2[(v & 3) * 8 + i]);
                        uint4 o;
                        __nv_bfloat162* ob = (__nv_bfloat162*)&o;
                        if constexpr (EPI == GEMM_EPI_ROWDOT) {
                            // the products use the values as stored (rounded to bf16): the consumer of C reads those
                            const uint4 rv = *(const uint4*)(my_row + v * 16);
                            const __nv_bfloat162* rb = (const __nv_bfloat162*)&rv;
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                ob[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
                                const float2 t = __bfloat1622float2(rb[i]), c2 = __bfloat1622float2(ob[i]);
                                rowdot = fmaf(c2.x, t.x, fmaf(c2.y, t.y, rowdot));
                            }
                        } else {
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
#pragma unroll
                            for (int i = 0; i < 4; ++i) ob[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
                        }
                        *(uint4*)(my_row + v * 16) = o;  // a thread reads and rewrites only its own staging row
                    }
                    if constexpr (EPI == GEMM_EPI_ROWDOT) {
                        if (row < p.M) p.aux[((size_t)(row / p.aux_S) * p.aux_NH + (col0 >> 6)) * p.aux_S + (row % p.aux_S)] = rowdot;
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

// pair: B is split over the two CTAs, so an MN-major B tile must be two whole 64-wide boxes per CTA.
// The thread that issues the UMMAs spends about 520 cycles per 64-deep k-block whatever the tile's width (barrier wait, four
// instruction issues, commit: measured with an issue loop of its own), while the four UMMAs of a k-block take 2 * bn cycles.
// So below 256 columns a tile costs as much time as a 256-wide one: take the fewest tiles, and among equals the narrowest.
int choose_tile_n(int N, int b_mn, int ctas) {
    const int step = b_mn ? 64 * ctas : 32;
    int best = 64;
    long best_cost = -1;
    for (int bn = (step > 64 ? step : 64); bn <= MAX_BN; bn += step) {
        const long tiles = (N + bn - 1) / bn;
        const long cost = tiles * (2 * bn > 520 ? 2 * bn : 520);
        if (best_cost < 0 || cost < best_cost) {
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
        cudaError_t e = cudaSuccess;
#define BMB_GEMM_ATTR(CT, EP) \
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_bf16_umma_kernel<CT, EP>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_DYN_BYTES)
        BMB_GEMM_ATTR(1, GEMM_EPI_NONE); BMB_GEMM_ATTR(2, GEMM_EPI_NONE);
        BMB_GEMM_ATTR(1, GEMM_EPI_SWIGLU_FWD); BMB_GEMM_ATTR(2, GEMM_EPI_SWIGLU_FWD);
        BMB_GEMM_ATTR(1, GEMM_EPI_SWIGLU_BWD); BMB_GEMM_ATTR(2, GEMM_EPI_SWIGLU_BWD);
        BMB_GEMM_ATTR(1, GEMM_EPI_ROWDOT); BMB_GEMM_ATTR(2, GEMM_EPI_ROWDOT);
#undef BMB_GEMM_ATTR
        if (e != cudaSuccess) return -5;
    }
    const int g_num_sms = sm_count_current_device();
    // Fused epilogues: bf16 output through the staged 128-byte row path only, so every pitch and pointer must be 16-byte aligned
    // and the column counts whole 64- (or 128-) column groups; anything else is the caller's cue to use the unfused kernels.
    if (g.epi != GEMM_EPI_NONE) {
        if (g.out_mode != GEMM_OUT_BF16 || g.splits > 1 || (((uintptr_t)g.C) & 15) || (g.ldc % 8)) return -8;
        if (g.epi == GEMM_EPI_SWIGLU_FWD) {
            if (g.b_mn_major || (g.N % 256) || !g.C2 || (((uintptr_t)g.C2) & 15) || (g.ldc2 % 8) || (g.tile_n && g.tile_n != 256)) return -8;
        } else if (g.epi == GEMM_EPI_SWIGLU_BWD) {
            if ((g.N % 128) || !g.R || (((uintptr_t)g.R) & 15) || (g.ldr % 8) || (g.tile_n && (g.tile_n % 128))) return -8;
        } else if (g.epi == GEMM_EPI_ROWDOT) {
            if ((g.N % 64) || !g.R || (((uintptr_t)g.R) & 15) || (g.ldr % 8) || !g.aux || g.aux_S <= 0 || g.aux_NH * 64 != g.N ||
                (g.M % g.aux_S) || (g.tile_n && (g.tile_n % 64)))
                return -8;
        } else {
            return -8;
        }
    }

    // CTA pairs (256-row tiles) whenever there are at least 256 rows and the caller did not fix a narrow tile
    const int ctas = (!pair_off && g.M >= 2 * BM && g.tile_n == 0) ? 2 : 1;
    KArgs p;
    p.M = g.M; p.N = g.N; p.K = g.K;
    p.BN = g.tile_n > 0 ? g.tile_n : choose_tile_n(g.N, g.b_mn_major, ctas);
    if (g.epi == GEMM_EPI_SWIGLU_FWD) p.BN = 256;                                   // 128 gate + 128 up columns of the same hidden units
    else if (g.epi == GEMM_EPI_SWIGLU_BWD && (p.BN % 128)) p.BN = 256;
    else if (g.epi == GEMM_EPI_ROWDOT && (p.BN % 64)) p.BN = 256;                   // whole heads per tile
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
    if (splits > 1) p.kb_per_split = (p.kb_per_split + KPS - 1) / KPS * KPS;   // whole ring stages per split: only the end of K may leave one half empty
    p.splits = (p.kb_total + p.kb_per_split - 1) / p.kb_per_split;
    p.C = g.C; p.ldc = g.ldc; p.out_mode = g.out_mode;
    p.R = g.R; p.ldr = g.ldr;
    p.err = err_flag;
    p.C2 = g.C2; p.ldc2 = g.ldc2;
    p.aux = g.aux; p.aux_S = g.aux_S; p.aux_NH = g.aux_NH;

    CUtensorMap tmA, tmB;
    int rc;
    if (!p.a_mn) rc = make_map(&tmA, g.A, (uint64_t)g.K, (uint64_t)g.M, (uint64_t)g.lda, BK, BM);
    else         rc = make_map(&tmA, g.A, (uint64_t)g.M, (uint64_t)g.K, (uint64_t)g.lda, 64, KPS * BK);
    if (rc) return rc;
    if (!p.b_mn) rc = make_map(&tmB, g.B, (uint64_t)g.K, (uint64_t)g.N, (uint64_t)g.ldb, BK,
                               (uint32_t)(g.epi == GEMM_EPI_SWIGLU_FWD ? p.BN / 2 : p.BN / ctas));
    else         rc = make_map(&tmB, g.B, (uint64_t)g.N, (uint64_t)g.K, (uint64_t)g.ldb, 64, KPS * BK);
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
        cudaError_t le;
        switch (g.epi) {
            case GEMM_EPI_SWIGLU_FWD: le = cudaLaunchKernelEx(&cfg, gemm_bf16_umma_kernel<2, GEMM_EPI_SWIGLU_FWD>, tmA, tmB, p); break;
            case GEMM_EPI_SWIGLU_BWD: le = cudaLaunchKernelEx(&cfg, gemm_bf16_umma_kernel<2, GEMM_EPI_SWIGLU_BWD>, tmA, tmB, p); break;
            case GEMM_EPI_ROWDOT: le = cudaLaunchKernelEx(&cfg, gemm_bf16_umma_kernel<2, GEMM_EPI_ROWDOT>, tmA, tmB, p); break;
            default: le = cudaLaunchKernelEx(&cfg, gemm_bf16_umma_kernel<2, GEMM_EPI_NONE>, tmA, tmB, p); break;
        }
        return le == cudaSuccess ? 0 : -7;
    }
    cfg.gridDim = dim3((unsigned)(units < g_num_sms ? units : g_num_sms));
    cfg.attrs = at;
    cfg.numAttrs = na;
    cudaError_t le;
    switch (g.epi) {
        case GEMM_EPI_SWIGLU_FWD: le = cudaLaunchKernelEx(&cfg, gemm_bf16_umma_kernel<1, GEMM_EPI_SWIGLU_FWD>, tmA, tmB, p); break;
        case GEMM_EPI_SWIGLU_BWD: le = cudaLaunchKernelEx(&cfg, gemm_bf16_umma_kernel<1, GEMM_EPI_SWIGLU_BWD>, tmA, tmB, p); break;
        case GEMM_EPI_ROWDOT: le = cudaLaunchKernelEx(&cfg, gemm_bf16_umma_kernel<1, GEMM_EPI_ROWDOT>, tmA, tmB, p); break;
        default: le = cudaLaunchKernelEx(&cfg, gemm_bf16_umma_kernel<1, GEMM_EPI_NONE>, tmA, tmB, p); break;
    }
    return le == cudaSuccess ? 0 : -7;
}

}  // namespace bmb
