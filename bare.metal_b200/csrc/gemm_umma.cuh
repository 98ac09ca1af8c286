// bf16 x bf16 -> fp32 GEMM on the sm_100a tensor cores (tcgen05.mma, accumulators in TMEM,
// operands staged by TMA into a 128B-swizzled shared-memory ring).
//
//   C[m, n] (+)= sum_k A(m, k) * B(n, k)
//
// Each operand is described by where its reduction index k lives in memory:
//   K-major  : A(m,k) at A[m*lda + k]   (activations X[M,K], weights W[N,K])
//   MN-major : A(m,k) at A[k*lda + m]   (the transposed view needed by wgrad and dgrad)
// so the three GEMMs of a linear layer (reference: matmul_forward_*, matmul_backward_inp_*,
// matmul_backward_w_* in src/kernels/forward.metal:449, backward.metal:122,277) are one kernel:
//   forward  Y  = X  W^T : A=X  (K-major),  B=W  (K-major)
//   dgrad    dX = dY W   : A=dY (K-major),  B=W  (MN-major, reduction over W's rows)
//   wgrad    dW += dY^T X: A=dY (MN-major), B=X  (MN-major), split over the token dimension
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace bmb {

enum GemmOut : int {
    GEMM_OUT_BF16 = 0,        // C (bf16) = acc [+ R]
    GEMM_OUT_F32 = 1,         // C (fp32) = acc
    GEMM_OUT_F32_ATOMIC = 2,  // C (fp32) += acc via red.global.add (split-K safe; C must hold the running sum)
};

// What the epilogue does with the accumulator tile besides storing it (GEMM_OUT_BF16 only). Each replaces a memory-bound kernel
// of the training step and the round trip of its operand through HBM.
enum GemmEpilogue : int {
    GEMM_EPI_NONE = 0,
    // Gated MLP, forward. B is the row-concatenated [gate; up] weight [2H, K]; N = 2H. A tile covers 128 hidden units: its first
    // half is the gate projection and its second half the up projection of the SAME units (the two halves of B are fetched from
    // rows h0 and H + h0). Stores gate and up (bf16) into C[:, h] and C[:, H + h] and act = silu(gate) * up into C2[:, h]
    // (swiglu_forward, src/kernels/forward.metal:1179). H % 128 == 0.
    GEMM_EPI_SWIGLU_FWD = 1,
    // Gated MLP, backward: the accumulator is dact[M, N = H]; R holds the saved gate at R[:, h] and up at R[:, H + h]; stores
    // dgate into C[:, h] and dup into C[:, H + h] (swiglu_backward, src/kernels/backward.metal:505). dact is never stored.
    GEMM_EPI_SWIGLU_BWD = 2,
    // Attention output gradient: stores C = acc (bf16) and aux[(b * NH + h) * S + s] = sum over the 64 columns of head h of
    // C[row, :] * R[row, :], row = b * S + s: the row sums flash attention backward subtracts from dP. N % 64 == 0.
    GEMM_EPI_ROWDOT = 3,
};

struct GemmProblem {
    int M, N, K;
    const __nv_bfloat16* A;
    int lda;
    int a_mn_major;
    const __nv_bfloat16* B;
    int ldb;
    int b_mn_major;
    void* C;
    int ldc;
    int out_mode;
    const __nv_bfloat16* R;  // optional residual added in the epilogue (GEMM_OUT_BF16 only), same shape as C
    int ldr;
    int splits;  // >1 only with GEMM_OUT_F32_ATOMIC; 0 = choose (fills the machine with whole waves of work units)
    int tile_n;  // 0 = choose
    int pdl;     // 1 = launch with programmatic stream serialisation (the predecessor must be a kernel of the same stream)
    int epi = GEMM_EPI_NONE;
    void* C2 = nullptr;  // GEMM_EPI_SWIGLU_FWD: act [M, H] bf16
    int ldc2 = 0;
    float* aux = nullptr;  // GEMM_EPI_ROWDOT: [M / aux_S, aux_NH, aux_S] fp32
    int aux_S = 0, aux_NH = 0;
};

// Launches on `stream`. Returns 0, or a negative code for an invalid problem / failed launch.
// `err_flag` (device int, may be null) receives a non-zero code if a bounded wait inside the
// kernel ran out.
int gemm_bf16_umma(const GemmProblem& p, int* err_flag, cudaStream_t stream);

// Number of UMMA GEMM kernel launches since process start (for launch accounting).
long gemm_bf16_umma_launch_count();

}  // namespace bmb
