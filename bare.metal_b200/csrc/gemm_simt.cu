// fp32 GEMM on the CUDA cores, for the fp32 parity mode only (the mixed-precision path uses
// gemm_umma.cu). Pure FFMA with fp32 accumulation — no TF32 — so results track the reference's fp32
// kernels (matmul_forward_fp32_tiled src/kernels/forward.metal:449, matmul_backward_inp_fp32_tiled and
// matmul_backward_w_tiled src/kernels/backward.metal:122,277) to summation-order rounding.
//
//   C[m,n] (+)= sum_k A(m,k) * B(n,k) [+ R[m,n]]
// with arbitrary element strides for A and B, so forward, dgrad and wgrad are the same kernel.
// 64x64 tile, 256 threads, 4x4 outputs per thread, K staged 16 at a time through shared memory.
#include "kernels.cuh"

namespace bmb {

namespace {
constexpr int TM = 64, TN = 64, TK = 16;

__global__ void __launch_bounds__(256)
gemm_f32_simt_kernel(float* __restrict__ C, int ldc, int accumulate, const float* __restrict__ A, long sam, long sak,
                     const float* __restrict__ B, long sbn, long sbk, const float* __restrict__ R, int ldr, int M, int N, int K) {
    __shared__ float As[TK][TM + 4];
    __shared__ float Bs[TK][TN + 4];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += TK) {
        // 64x16 elements per operand, 256 threads -> 4 each. Index so the unit-stride dimension of
        // the source varies fastest across threads.
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            const int e = threadIdx.x + t * 256;
            int mm, kk;
            if (sak == 1) { kk = e & 15; mm = e >> 4; } else { mm = e & 63; kk = e >> 6; }
            const int m = m0 + mm, k = k0 + kk;
            As[kk][mm] = (m < M && k < K) ? A[m * sam + k * sak] : 0.f;
            int nn, kb;
            if (sbk == 1) { kb = e & 15; nn = e >> 4; } else { nn = e & 63; kb = e >> 6; }
            const int n = n0 + nn, k2 = k0 + kb;
            Bs[kb][nn] = (n < N && k2 < K) ? B[n * sbn + k2 * sbk] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < TK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (R) v += R[(size_t)m * ldr + n];
            float* c = C + (size_t)m * ldc + n;
            *c = accumulate ? *c + v : v;
        }
    }
}
}  // namespace

int gemm_f32_simt(float* C, int ldc, int accumulate, const float* A, long sam, long sak, const float* B, long sbn, long sbk,
                  const float* R, int ldr, int M, int N, int K, cudaStream_t st) {
    if (M <= 0 || N <= 0 || K <= 0) return -1;
    dim3 grid((N + TN - 1) / TN, (M + TM - 1) / TM);
    gemm_f32_simt_kernel<<<grid, 256, 0, st>>>(C, ldc, accumulate, A, sam, sak, B, sbn, sbk, R, ldr, M, N, K);
    return 0;
}

}  // namespace bmb
