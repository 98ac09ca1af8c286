// extern "C" surface of the CUDA backend (include/bm_cuda_backend.h): context, memory, and one
// typed entry point per operation of the training step. Each entry point validates its
// arguments, picks the kernel for the activation dtype and enqueues it on the context's stream.
#include "../../include/bm_cuda_backend.h"

#include <stdio.h>
#include <stdlib.h>

#include <map>
#include <utility>
#include <mutex>
#include <vector>

#include "attention_umma.cuh"
#include "decode_kernels.cuh"
#include "gemm_umma.cuh"
#include "kernels.cuh"

using namespace bmb;
namespace bmb { int wait_probe_launch(int* err, cudaStream_t st); }

struct bmc_ctx_s {
    int device;
    cudaStream_t stream;
    int* d_err;  // set by kernels whose bounded waits ran out
    int sticky_status;
    size_t allocated, peak;
    std::map<void*, size_t> allocs;
    std::mutex mu;
    long launches, launches_at_capture;
    int num_sms;
    // scratch owned by the context
    float* rms_scratch;
    size_t rms_scratch_floats;
    void* attn_scratch;
    size_t attn_scratch_bytes;
    void* mask_bits;  // padding mask of the attention kernels, one bit per position
    size_t mask_bits_bytes;
    cudaEvent_t ev0[8], ev1[8];
    // optional per-launch timing of the tensor-core GEMM (bmc_gemm_timing)
    bool gemm_timing;
    std::vector<cudaEvent_t> gt_events;  // pairs (begin, end)
    std::vector<double> gt_flops;
    size_t gt_used;
    cudaGraph_t graphs[2];
    cudaGraphExec_t graph_execs[2];
    long graph_kernels[2];  // kernel nodes of each captured graph: what one replay adds to `launches`
    // early read-back (bmc_early_readback / bmc_early_wait): a pinned pair {loss, error word} and the event that says it has landed
    float* h_early;
    cudaEvent_t early_ev;
    int graph_slot;  // slot 0: inference session, slot 1: trainer
    // side stream (bmc_side_begin / _end / _wait): work that may overlap the main stream
    cudaStream_t side_stream;
    cudaEvent_t side_fork, side_done[16];
    int side_next, in_side;
};

namespace {

#define BMC_CHECK_CTX(ctx) \
    if (!(ctx)) return -100;

int note(bmc_ctx_t* ctx, int rc, int nlaunch = 1) {
    if (rc == 0) {
        ctx->launches += nlaunch;
        cudaError_t e = cudaPeekAtLastError();
        if (e != cudaSuccess) {
            ctx->sticky_status = -200 - (int)e;
            return ctx->sticky_status;
        }
    }
    return rc;
}

void* scratch_get(bmc_ctx_t* ctx, void** slot, size_t* cap, size_t bytes) {
    if (*cap >= bytes) return *slot;
    if (*slot) {
        cudaStreamSynchronize(ctx->stream);
        cudaFree(*slot);
        *slot = nullptr;
        *cap = 0;
    }
    if (cudaMalloc(slot, bytes) != cudaSuccess) return nullptr;
    cudaMemsetAsync(*slot, 0, bytes, ctx->stream);   // nothing a kernel reads may depend on what a previous owner left in the memory
    *cap = bytes;
    return *slot;
}

// tensor-core GEMM launch, bracketed by events when per-launch timing is on
int run_umma(bmc_ctx_t* ctx, const GemmProblem& g) {
    if (!ctx->gemm_timing) return gemm_bf16_umma(g, ctx->d_err, ctx->stream);
    if (ctx->gt_used * 2 + 2 > ctx->gt_events.size()) {
        for (int i = 0; i < 2; ++i) {
            cudaEvent_t e;
            cudaEventCreate(&e);
            ctx->gt_events.push_back(e);
        }
    }
    cudaEventRecord(ctx->gt_events[ctx->gt_used * 2], ctx->stream);
    const int rc = gemm_bf16_umma(g, ctx->d_err, ctx->stream);
    cudaEventRecord(ctx->gt_events[ctx->gt_used * 2 + 1], ctx->stream);
    if (ctx->gt_flops.size() <= ctx->gt_used) ctx->gt_flops.resize(ctx->gt_used + 1);
    ctx->gt_flops[ctx->gt_used] = 2.0 * g.M * g.N * g.K;
    ctx->gt_used++;
    return rc;
}

}  // namespace

extern "C" {

int bmc_gemm_timing(bmc_ctx_t* ctx, int enable) {
    BMC_CHECK_CTX(ctx);
    ctx->gemm_timing = enable != 0;
    ctx->gt_used = 0;
    return 0;
}
// out[0] = launches, out[1] = summed duration in ms, out[2] = summed algorithmic FLOPs. Blocks until the stream is idle.
int bmc_gemm_timing_collect(bmc_ctx_t* ctx, double* out) {
    BMC_CHECK_CTX(ctx);
    cudaStreamSynchronize(ctx->stream);
    double ms = 0, fl = 0;
    for (size_t i = 0; i < ctx->gt_used; ++i) {
        float t = 0.f;
        cudaEventElapsedTime(&t, ctx->gt_events[2 * i], ctx->gt_events[2 * i + 1]);
        ms += t;
        fl += ctx->gt_flops[i];
    }
    out[0] = (double)ctx->gt_used;
    out[1] = ms;
    out[2] = fl;
    ctx->gt_used = 0;
    return 0;
}

bmc_ctx_t* bmc_create(int device_ordinal) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n <= 0 || device_ordinal < 0 || device_ordinal >= n) {
        fprintf(stderr, "bmc_create: no usable CUDA device (count=%d, requested=%d); this backend has no CPU fallback\n", n,
                device_ordinal);
        return nullptr;
    }
    if (cudaSetDevice(device_ordinal) != cudaSuccess) return nullptr;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device_ordinal) != cudaSuccess) return nullptr;
    if (prop.major != 10) {
        fprintf(stderr, "bmc_create: device %d is sm_%d%d; this backend is built for sm_100a only\n", device_ordinal, prop.major,
                prop.minor);
        return nullptr;
    }
    bmc_ctx_t* ctx = new bmc_ctx_s();
    ctx->device = device_ordinal;
    ctx->num_sms = prop.multiProcessorCount;
    ctx->sticky_status = 0;
    ctx->allocated = ctx->peak = 0;
    ctx->launches = 0;
    ctx->rms_scratch = nullptr;
    ctx->rms_scratch_floats = 0;
    ctx->attn_scratch = nullptr;
    ctx->attn_scratch_bytes = 0;
    ctx->mask_bits = nullptr;
    ctx->mask_bits_bytes = 0;
    ctx->gemm_timing = false;
    ctx->gt_used = 0;
    for (int i = 0; i < 2; ++i) { ctx->graphs[i] = nullptr; ctx->graph_execs[i] = nullptr; }
    ctx->graph_slot = 0;
    if (cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking) != cudaSuccess) { delete ctx; return nullptr; }
    if (cudaMalloc(&ctx->d_err, sizeof(int)) != cudaSuccess) { delete ctx; return nullptr; }
    cudaMemset(ctx->d_err, 0, sizeof(int));
    for (int i = 0; i < 8; ++i) {
        cudaEventCreate(&ctx->ev0[i]);
        cudaEventCreate(&ctx->ev1[i]);
    }
    if (cudaStreamCreateWithFlags(&ctx->side_stream, cudaStreamNonBlocking) != cudaSuccess) { delete ctx; return nullptr; }
    cudaEventCreateWithFlags(&ctx->side_fork, cudaEventDisableTiming);
    for (int i = 0; i < 16; ++i) cudaEventCreateWithFlags(&ctx->side_done[i], cudaEventDisableTiming);
    ctx->side_next = 0;
    ctx->in_side = 0;
    return ctx;
}

void bmc_destroy(bmc_ctx_t* ctx) {
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    if (ctx->in_side) std::swap(ctx->stream, ctx->side_stream);
    cudaStreamSynchronize(ctx->side_stream);
    cudaStreamSynchronize(ctx->stream);
    cudaStreamDestroy(ctx->side_stream);
    cudaEventDestroy(ctx->side_fork);
    for (int i = 0; i < 16; ++i) cudaEventDestroy(ctx->side_done[i]);
    for (auto& kv : ctx->allocs) cudaFree(kv.first);
    if (ctx->rms_scratch) cudaFree(ctx->rms_scratch);
    if (ctx->attn_scratch) cudaFree(ctx->attn_scratch);
    if (ctx->mask_bits) cudaFree(ctx->mask_bits);
    cudaFree(ctx->d_err);
    for (int i = 0; i < 8; ++i) {
        cudaEventDestroy(ctx->ev0[i]);
        cudaEventDestroy(ctx->ev1[i]);
    }
    for (auto e : ctx->gt_events) cudaEventDestroy(e);
    for (int i = 0; i < 2; ++i) {
        if (ctx->graph_execs[i]) cudaGraphExecDestroy(ctx->graph_execs[i]);
        if (i == 0 && ctx->h_early) { cudaEventDestroy(ctx->early_ev); cudaFreeHost(ctx->h_early); ctx->h_early = nullptr; }
        if (ctx->graphs[i]) cudaGraphDestroy(ctx->graphs[i]);
    }
    cudaStreamDestroy(ctx->stream);
    delete ctx;
}

void* bmc_alloc(bmc_ctx_t* ctx, size_t bytes) {
    if (!ctx || bytes == 0) return nullptr;
    void* p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    // Zero-filled: cudaMalloc hands back whatever the previous owner left, and padding rows or a scratch row that a launch of a
    // smaller shape never writes must not make results depend on the process's allocation history. Creation-time cost only.
    cudaMemsetAsync(p, 0, bytes, ctx->stream);
    std::lock_guard<std::mutex> lk(ctx->mu);
    ctx->allocs[p] = bytes;
    ctx->allocated += bytes;
    if (ctx->allocated > ctx->peak) ctx->peak = ctx->allocated;
    return p;
}
void bmc_free(bmc_ctx_t* ctx, void* p) {
    if (!ctx || !p) return;
    std::lock_guard<std::mutex> lk(ctx->mu);
    auto it = ctx->allocs.find(p);
    if (it == ctx->allocs.end()) return;
    ctx->allocated -= it->second;
    ctx->allocs.erase(it);
    cudaStreamSynchronize(ctx->stream);
    cudaFree(p);
}
size_t bmc_allocated_bytes(bmc_ctx_t* ctx) { return ctx ? ctx->allocated : 0; }
size_t bmc_peak_allocated_bytes(bmc_ctx_t* ctx) { return ctx ? ctx->peak : 0; }

int bmc_upload(bmc_ctx_t* ctx, void* d_dst, const void* h_src, size_t bytes) {
    BMC_CHECK_CTX(ctx);
    return cudaMemcpyAsync(d_dst, h_src, bytes, cudaMemcpyHostToDevice, ctx->stream) == cudaSuccess ? 0 : -1;
}
int bmc_download(bmc_ctx_t* ctx, void* h_dst, const void* d_src, size_t bytes) {
    BMC_CHECK_CTX(ctx);
    if (cudaMemcpyAsync(h_dst, d_src, bytes, cudaMemcpyDeviceToHost, ctx->stream) != cudaSuccess) return -1;
    return cudaStreamSynchronize(ctx->stream) == cudaSuccess ? 0 : -2;
}
int bmc_memset(bmc_ctx_t* ctx, void* d_ptr, int byte_value, size_t bytes) {
    BMC_CHECK_CTX(ctx);
    return cudaMemsetAsync(d_ptr, byte_value, bytes, ctx->stream) == cudaSuccess ? 0 : -1;
}
int bmc_copy(bmc_ctx_t* ctx, void* d_dst, const void* d_src, size_t bytes) {
    BMC_CHECK_CTX(ctx);
    return cudaMemcpyAsync(d_dst, d_src, bytes, cudaMemcpyDeviceToDevice, ctx->stream) == cudaSuccess ? 0 : -1;
}
int bmc_status(bmc_ctx_t* ctx) {
    BMC_CHECK_CTX(ctx);
    if (ctx->sticky_status) return ctx->sticky_status;
    int h = 0;
    if (cudaMemcpyAsync(&h, ctx->d_err, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream) != cudaSuccess) return -3;
    cudaError_t e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) {
        ctx->sticky_status = -200 - (int)e;
        return ctx->sticky_status;
    }
    if (h) {
        cudaMemsetAsync(ctx->d_err, 0, sizeof(int), ctx->stream);
        return h;
    }
    return 0;
}
int bmc_sync(bmc_ctx_t* ctx) {
    BMC_CHECK_CTX(ctx);
    cudaError_t e = cudaStreamSynchronize(ctx->side_stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) {
        ctx->sticky_status = -200 - (int)e;
        return ctx->sticky_status;
    }
    return bmc_status(ctx);
}
void* bmc_stream(bmc_ctx_t* ctx) { return ctx ? (void*)ctx->stream : nullptr; }
// Side stream: everything enqueued between bmc_side_begin and bmc_side_end runs on a second stream, ordered after all work
// enqueued on the main stream so far, and may overlap what the main stream does next. bmc_side_end returns a ticket;
// bmc_side_wait(ticket) orders later main-stream work after the side work up to that ticket. Host calls are single-threaded.
int bmc_side_begin(bmc_ctx_t* ctx) {
    BMC_CHECK_CTX(ctx);
    if (ctx->in_side) return -1;
    if (cudaEventRecord(ctx->side_fork, ctx->stream) != cudaSuccess) return -2;
    if (cudaStreamWaitEvent(ctx->side_stream, ctx->side_fork, 0) != cudaSuccess) return -2;
    std::swap(ctx->stream, ctx->side_stream);
    ctx->in_side = 1;
    return 0;
}
int bmc_side_end(bmc_ctx_t* ctx) {
    BMC_CHECK_CTX(ctx);
    if (!ctx->in_side) return -1;
    const int ticket = ctx->side_next;
    ctx->side_next = (ctx->side_next + 1) % 16;
    const cudaError_t e = cudaEventRecord(ctx->side_done[ticket], ctx->stream);
    std::swap(ctx->stream, ctx->side_stream);
    ctx->in_side = 0;
    return e == cudaSuccess ? ticket : -2;
}
int bmc_side_wait(bmc_ctx_t* ctx, int ticket) {
    BMC_CHECK_CTX(ctx);
    if (ticket < 0 || ticket >= 16 || ctx->in_side) return -1;
    return cudaStreamWaitEvent(ctx->stream, ctx->side_done[ticket], 0) == cudaSuccess ? 0 : -2;
}
long bmc_launch_count(bmc_ctx_t* ctx) { return ctx ? ctx->launches : 0; }
void* bmc_host_alloc(size_t bytes) {
    void* p = nullptr;
    if (cudaMallocHost(&p, bytes) != cudaSuccess) return nullptr;
    return p;
}
void bmc_host_free(void* p) {
    if (p) cudaFreeHost(p);
}
int bmc_timer_begin(bmc_ctx_t* ctx, int slot) {
    BMC_CHECK_CTX(ctx);
    if (slot < 0 || slot >= 8) return -1;
    return cudaEventRecord(ctx->ev0[slot], ctx->stream) == cudaSuccess ? 0 : -2;
}
float bmc_timer_end(bmc_ctx_t* ctx, int slot) {
    if (!ctx || slot < 0 || slot >= 8) return -1.f;
    cudaEventRecord(ctx->ev1[slot], ctx->stream);
    cudaEventSynchronize(ctx->ev1[slot]);
    float ms = 0.f;
    cudaEventElapsedTime(&ms, ctx->ev0[slot], ctx->ev1[slot]);
    return ms;
}

// ---- embedding ---------------------------------------------------------------------------------------
int bmc_embedding_forward(bmc_ctx_t* ctx, int dtype, void* d_out, const float* d_table, const int* d_tokens, int n_tok, int D, int V) {
    BMC_CHECK_CTX(ctx);
    if (dtype == BMC_F32) return note(ctx, embedding_forward<float>((float*)d_out, d_table, d_tokens, n_tok, D, V, ctx->d_err, ctx->stream));
    return note(ctx, embedding_forward<bf16>((bf16*)d_out, d_table, d_tokens, n_tok, D, V, ctx->d_err, ctx->stream));
}
int bmc_embedding_backward(bmc_ctx_t* ctx, int dtype, float* d_gwte, const void* d_gout, const int* d_tokens, int n_tok, int D, int V) {
    BMC_CHECK_CTX(ctx);
    if (dtype == BMC_F32) return note(ctx, embedding_backward_f32(d_gwte, (const float*)d_gout, d_tokens, n_tok, D, V, ctx->d_err, ctx->stream));
    return note(ctx, embedding_backward_bf16(d_gwte, (const bf16*)d_gout, d_tokens, n_tok, D, V, ctx->d_err, ctx->stream));
}

// ---- RMSNorm -----------------------------------------------------------------------------------------
int bmc_rmsnorm_forward(bmc_ctx_t* ctx, int dtype, void* d_out, float* d_rstd, const void* d_x, const float* d_w, int N, int C, float eps) {
    BMC_CHECK_CTX(ctx);
    if (dtype == BMC_F32) return note(ctx, rmsnorm_forward<float>((float*)d_out, d_rstd, (const float*)d_x, d_w, N, C, eps, ctx->stream));
    return note(ctx, rmsnorm_forward<bf16>((bf16*)d_out, d_rstd, (const bf16*)d_x, d_w, N, C, eps, ctx->stream));
}
int bmc_rmsnorm_backward(bmc_ctx_t* ctx, int dtype, void* d_gx, float* d_gw, int gw_accumulate, const void* d_gout, const void* d_x,
                         const float* d_w, const float* d_rstd, int N, int C, int w_row0, int w_row1) {
    BMC_CHECK_CTX(ctx);
    const size_t need = rmsnorm_backward_scratch_floats(C);
    size_t cap_bytes = ctx->rms_scratch_floats * sizeof(float);
    float* scratch = (float*)scratch_get(ctx, (void**)&ctx->rms_scratch, &cap_bytes, need * sizeof(float));
    ctx->rms_scratch_floats = cap_bytes / sizeof(float);
    if (!scratch) return -50;
    if (dtype == BMC_F32)
        return note(ctx, rmsnorm_backward<float>((float*)d_gx, d_gw, gw_accumulate, (const float*)d_gout, (const float*)d_x, d_w, d_rstd, N,
                                                 C, w_row0, w_row1, scratch, ctx->stream), 2);
    return note(ctx, rmsnorm_backward<bf16>((bf16*)d_gx, d_gw, gw_accumulate, (const bf16*)d_gout, (const bf16*)d_x, d_w, d_rstd, N, C,
                                            w_row0, w_row1, scratch, ctx->stream), 2);
}

// ---- linear layers -----------------------------------------------------------------------------------
int bmc_matmul_forward(bmc_ctx_t* ctx, int dtype, void* d_out, int ldo, const void* d_inp, int ldi, const void* d_weight,
                       const void* d_residual, int ldr, int BT, int C, int OC) {
    BMC_CHECK_CTX(ctx);
    if (dtype == BMC_F32)
        return note(ctx, gemm_f32_simt((float*)d_out, ldo, 0, (const float*)d_inp, ldi, 1, (const float*)d_weight, C, 1,
                                       (const float*)d_residual, ldr, BT, OC, C, ctx->stream));
    GemmProblem g{BT, OC, C, (const bf16*)d_inp, ldi, 0, (const bf16*)d_weight, C, 0, d_out, ldo, GEMM_OUT_BF16,
                  (const bf16*)d_residual, ldr, 1, 0};
    return note(ctx, run_umma(ctx, g));
}
int bmc_matmul_backward_inp(bmc_ctx_t* ctx, int dtype, void* d_ginp, int ldgi, int accumulate, const void* d_gout, int ldgo,
                            const void* d_weight, int BT, int C, int OC) {
    BMC_CHECK_CTX(ctx);
    if (dtype == BMC_F32)
        return note(ctx, gemm_f32_simt((float*)d_ginp, ldgi, accumulate, (const float*)d_gout, ldgo, 1, (const float*)d_weight, 1, C,
                                       nullptr, 0, BT, C, OC, ctx->stream));
    // ginp[BT, C] = gout[BT, OC] (K-major, reduction over OC) x W[OC, C] (MN-major: reduction index is W's row)
    GemmProblem g{BT, C, OC, (const bf16*)d_gout, ldgo, 0, (const bf16*)d_weight, C, 1, d_ginp, ldgi, GEMM_OUT_BF16,
                  accumulate ? (const bf16*)d_ginp : nullptr, ldgi, 1, 0};
    return note(ctx, run_umma(ctx, g));
}
int bmc_matmul_backward_w(bmc_ctx_t* ctx, int dtype, float* d_gw, const void* d_gout, int ldgo, const void* d_inp, int ldi, int BT,
                          int C, int OC) {
    BMC_CHECK_CTX(ctx);
    if (dtype == BMC_F32)
        return note(ctx, gemm_f32_simt(d_gw, C, 1, (const float*)d_gout, 1, ldgo, (const float*)d_inp, 1, ldi, nullptr, 0, OC, C, BT,
                                       ctx->stream));
    // gw[OC, C] += gout^T[OC, BT] x inp[BT, C]: both operands MN-major, reduction over the tokens, split (by the GEMM) so that
    // whole waves of work units exist even when OC x C is only a few dozen tiles.
    const int splits = 0;
    GemmProblem g{OC, C, BT, (const bf16*)d_gout, ldgo, 1, (const bf16*)d_inp, ldi, 1, d_gw, C, GEMM_OUT_F32_ATOMIC, nullptr, 0, splits, 0};
    return note(ctx, run_umma(ctx, g));
}

// ---- linear layers with a fused neighbour (bf16 tensor-core path only; BMC_ERR_UNFUSED otherwise) ----
int bmc_matmul_swiglu_forward(bmc_ctx_t* ctx, int dtype, void* d_gu, int ldgu, void* d_act, int ldact, const void* d_inp, int ldi,
                              const void* d_w_gate_up, int BT, int C, int H) {
    BMC_CHECK_CTX(ctx);
    if (dtype != BMC_BF16 || (H % 128)) return BMC_ERR_UNFUSED;
    GemmProblem g{BT, 2 * H, C, (const bf16*)d_inp, ldi, 0, (const bf16*)d_w_gate_up, C, 0, d_gu, ldgu, GEMM_OUT_BF16, nullptr, 0, 1, 0, 0};
    g.epi = GEMM_EPI_SWIGLU_FWD;
    g.C2 = d_act;
    g.ldc2 = ldact;
    const int rc = run_umma(ctx, g);
    return rc == -8 ? BMC_ERR_UNFUSED : note(ctx, rc);
}
int bmc_matmul_backward_inp_swiglu(bmc_ctx_t* ctx, int dtype, void* d_dgu, int lddgu, const void* d_gout, int ldgo, const void* d_w_down,
                                   const void* d_gu, int ldgu, int BT, int H, int OC) {
    BMC_CHECK_CTX(ctx);
    if (dtype != BMC_BF16 || (H % 128)) return BMC_ERR_UNFUSED;
    // dact[BT, H] = gout[BT, OC] x W_down[OC, H] (MN-major B), never stored: the epilogue turns it into dgate | dup
    GemmProblem g{BT, H, OC, (const bf16*)d_gout, ldgo, 0, (const bf16*)d_w_down, H, 1, d_dgu, lddgu, GEMM_OUT_BF16, (const bf16*)d_gu, ldgu, 1, 0, 0};
    g.epi = GEMM_EPI_SWIGLU_BWD;
    const int rc = run_umma(ctx, g);
    return rc == -8 ? BMC_ERR_UNFUSED : note(ctx, rc);
}
int bmc_matmul_backward_inp_rowdot(bmc_ctx_t* ctx, int dtype, void* d_ginp, int ldgi, float* d_rowdot, const void* d_gout, int ldgo,
                                   const void* d_weight, const void* d_other, int ldother, int BT, int C, int OC, int S, int NH) {
    BMC_CHECK_CTX(ctx);
    if (dtype != BMC_BF16 || NH * 64 != C || S <= 0 || (BT % S)) return BMC_ERR_UNFUSED;
    GemmProblem g{BT, C, OC, (const bf16*)d_gout, ldgo, 0, (const bf16*)d_weight, C, 1, d_ginp, ldgi, GEMM_OUT_BF16, (const bf16*)d_other, ldother, 1, 0, 0};
    g.epi = GEMM_EPI_ROWDOT;
    g.aux = d_rowdot;
    g.aux_S = S;
    g.aux_NH = NH;
    const int rc = run_umma(ctx, g);
    return rc == -8 ? BMC_ERR_UNFUSED : note(ctx, rc);
}

// ---- RoPE --------------------------------------------------------------------------------------------
int bmc_rope(bmc_ctx_t* ctx, int dtype, void* d_q, int ldq, void* d_k, int ldk, const float* d_cs_table, int rows, int S, int NH, int NKV,
             int HD, int dir) {
    BMC_CHECK_CTX(ctx);
    if (dtype == BMC_F32) return note(ctx, rope_apply<float>((float*)d_q, ldq, (float*)d_k, ldk, d_cs_table, rows, S, NH, NKV, HD, dir, ctx->stream));
    return note(ctx, rope_apply<bf16>((bf16*)d_q, ldq, (bf16*)d_k, ldk, d_cs_table, rows, S, NH, NKV, HD, dir, ctx->stream));
}

// ---- attention ---------------------------------------------------------------------------------------
int bmc_attention_forward(bmc_ctx_t* ctx, int dtype, void* d_out, int ldo, float* d_lse, const void* d_q, int ldq, const void* d_k,
                          const void* d_v, int ldkv, const uint8_t* d_mask, int B, int S, int NH, int NKV, int HD, float scale) {
    BMC_CHECK_CTX(ctx);
    if (dtype == BMC_F32)
        return note(ctx, attention_forward_simt<float>((float*)d_out, ldo, d_lse, (const float*)d_q, ldq, (const float*)d_k,
                                                       (const float*)d_v, ldkv, d_mask, B, S, NH, NKV, HD, scale, ctx->stream));
    if (flash_attention_supported(HD, NH, NKV) && (ldo % 8) == 0) {
        const uint32_t* bits = nullptr;
        if (d_mask) {   // the tensor-core kernels take the padding mask as bits
            bits = (const uint32_t*)scratch_get(ctx, &ctx->mask_bits, &ctx->mask_bits_bytes, flash_attention_mask_bits_bytes(B, S));
            if (!bits || flash_attention_pack_mask((uint32_t*)bits, d_mask, B, S, ctx->stream)) return -50;
        }
        return note(ctx, flash_attention_forward_umma((bf16*)d_out, ldo, d_lse, (const bf16*)d_q, ldq, (const bf16*)d_k, (const bf16*)d_v,
                                                      ldkv, bits, B, S, NH, NKV, HD, scale, ctx->d_err, ctx->stream), d_mask ? 2 : 1);
    }
    return note(ctx, attention_forward_simt<bf16>((bf16*)d_out, ldo, d_lse, (const bf16*)d_q, ldq, (const bf16*)d_k, (const bf16*)d_v,
                                                  ldkv, d_mask, B, S, NH, NKV, HD, scale, ctx->stream));
}
// Attention backward; with d_delta / d_rope_cs the two neighbouring passes of the training step are folded in (see the header).
int bmc_attention_backward_fused(bmc_ctx_t* ctx, int dtype, void* d_gq, int ldgq, void* d_gk, void* d_gv, int ldgkv, const void* d_gout,
                                 int ldo, const void* d_out, const float* d_lse, const void* d_q, int ldq, const void* d_k, const void* d_v,
                                 int ldkv, const uint8_t* d_mask, const float* d_delta, const float* d_rope_cs, int B, int S, int NH, int NKV,
                                 int HD, float scale) {
    BMC_CHECK_CTX(ctx);
    const size_t rows = (size_t)B * S;
    if (dtype == BMC_BF16 && flash_attention_supported(HD, NH, NKV) && (ldgkv % 8) == 0 && (ldo % 8) == 0) {
        const size_t need = flash_attention_backward_scratch_bytes(B, S, NH, HD);
        void* scratch = scratch_get(ctx, &ctx->attn_scratch, &ctx->attn_scratch_bytes, need);
        if (!scratch) return -50;
        const uint32_t* bits = nullptr;
        if (d_mask) {
            bits = (const uint32_t*)scratch_get(ctx, &ctx->mask_bits, &ctx->mask_bits_bytes, flash_attention_mask_bits_bytes(B, S));
            if (!bits || flash_attention_pack_mask((uint32_t*)bits, d_mask, B, S, ctx->stream)) return -50;
        }
        return note(ctx, flash_attention_backward_umma((bf16*)d_gq, ldgq, (bf16*)d_gk, (bf16*)d_gv, ldgkv, (const bf16*)d_gout, ldo,
                                                       (const bf16*)d_out, d_lse, (const bf16*)d_q, ldq, (const bf16*)d_k, (const bf16*)d_v,
                                                       ldkv, B, S, NH, NKV, HD, scale, scratch, d_delta, d_rope_cs, bits, ctx->d_err,
                                                       ctx->stream),
                    d_delta ? 3 : 4);
    }
    int rc;
    if (dtype == BMC_F32) {
        // gK/gV accumulate through atomics and must start from zero (reference: zero_buffer before attention_backward,
        // src/baremetal/scheduler.c:1372-1383). K and V rows may be interleaved with other columns, so clear row by row.
        cudaMemset2DAsync(d_gk, (size_t)ldgkv * 4, 0, (size_t)NKV * HD * 4, rows, ctx->stream);
        cudaMemset2DAsync(d_gv, (size_t)ldgkv * 4, 0, (size_t)NKV * HD * 4, rows, ctx->stream);
        rc = attention_backward_simt<float>((float*)d_gq, ldgq, (float*)d_gk, (float*)d_gv, ldgkv, (const float*)d_gout, ldo,
                                            (const float*)d_out, d_lse, (const float*)d_q, ldq, (const float*)d_k, (const float*)d_v, ldkv,
                                            d_mask, B, S, NH, NKV, HD, scale, ctx->stream);
        if (rc == 0 && d_rope_cs)
            rc = rope_apply<float>((float*)d_gq, ldgq, (float*)d_gk, ldgkv, d_rope_cs, (int)rows, S, NH, NKV, HD, -1, ctx->stream);
        return note(ctx, rc, d_rope_cs ? 2 : 1);
    }
    // General bf16 shapes (head_dim != 64, masks): exact fp32 kernel into fp32 scratch, then one cast per output.
    const int QD = NH * HD, KVD = NKV * HD;
    const size_t need = rows * (size_t)(QD + 2 * KVD) * sizeof(float);
    float* scratch = (float*)scratch_get(ctx, &ctx->attn_scratch, &ctx->attn_scratch_bytes, need);
    if (!scratch) return -50;
    float* sgq = scratch;
    float* sgk = sgq + rows * QD;
    float* sgv = sgk + rows * KVD;
    cudaMemsetAsync(sgk, 0, rows * 2 * KVD * sizeof(float), ctx->stream);
    rc = attention_backward_simt<bf16>(sgq, QD, sgk, sgv, KVD, (const bf16*)d_gout, ldo, (const bf16*)d_out, d_lse, (const bf16*)d_q,
                                       ldq, (const bf16*)d_k, (const bf16*)d_v, ldkv, d_mask, B, S, NH, NKV, HD, scale, ctx->stream);
    if (rc) return rc;
    if (d_rope_cs) rc = rope_apply<float>(sgq, QD, sgk, KVD, d_rope_cs, (int)rows, S, NH, NKV, HD, -1, ctx->stream);
    if (!rc) rc = cast_rows_f32_to_bf16((bf16*)d_gq, ldgq, sgq, QD, (int)rows, QD, ctx->stream);
    if (!rc) rc = cast_rows_f32_to_bf16((bf16*)d_gk, ldgkv, sgk, KVD, (int)rows, KVD, ctx->stream);
    if (!rc) rc = cast_rows_f32_to_bf16((bf16*)d_gv, ldgkv, sgv, KVD, (int)rows, KVD, ctx->stream);
    return note(ctx, rc, d_rope_cs ? 5 : 4);
}
int bmc_attention_backward(bmc_ctx_t* ctx, int dtype, void* d_gq, int ldgq, void* d_gk, void* d_gv, int ldgkv, const void* d_gout,
                           int ldo, const void* d_out, const float* d_lse, const void* d_q, int ldq, const void* d_k, const void* d_v,
                           int ldkv, const uint8_t* d_mask, int B, int S, int NH, int NKV, int HD, float scale) {
    return bmc_attention_backward_fused(ctx, dtype, d_gq, ldgq, d_gk, d_gv, ldgkv, d_gout, ldo, d_out, d_lse, d_q, ldq, d_k, d_v, ldkv, d_mask,
                                        nullptr, nullptr, B, S, NH, NKV, HD, scale);
}

// ---- SwiGLU / add ------------------------------------------------------------------------------------
int bmc_swiglu_forward(bmc_ctx_t* ctx, int dtype, void* d_out, int ldo, const void* d_gate, const void* d_up, int ldgu, int rows, int H) {
    BMC_CHECK_CTX(ctx);
    if (dtype == BMC_F32) return note(ctx, swiglu_forward<float>((float*)d_out, ldo, (const float*)d_gate, (const float*)d_up, ldgu, rows, H, ctx->stream));
    return note(ctx, swiglu_forward<bf16>((bf16*)d_out, ldo, (const bf16*)d_gate, (const bf16*)d_up, ldgu, rows, H, ctx->stream));
}
int bmc_swiglu_backward(bmc_ctx_t* ctx, int dtype, void* d_ggate, void* d_gup, int ldg, const void* d_gate, const void* d_up, int ldgu,
                        const void* d_gout, int ldo, int rows, int H) {
    BMC_CHECK_CTX(ctx);
    if (dtype == BMC_F32)
        return note(ctx, swiglu_backward<float>((float*)d_ggate, (float*)d_gup, ldg, (const float*)d_gate, (const float*)d_up, ldgu,
                                                (const float*)d_gout, ldo, rows, H, ctx->stream));
    return note(ctx, swiglu_backward<bf16>((bf16*)d_ggate, (bf16*)d_gup, ldg, (const bf16*)d_gate, (const bf16*)d_up, ldgu,
                                           (const bf16*)d_gout, ldo, rows, H, ctx->stream));
}
int bmc_add_forward(bmc_ctx_t* ctx, int dtype, void* d_out, const void* d_a, const void* d_b, size_t n) {
    BMC_CHECK_CTX(ctx);
    if (dtype == BMC_F32) return note(ctx, add_forward<float>((float*)d_out, (const float*)d_a, (const float*)d_b, n, ctx->stream));
    return note(ctx, add_forward<bf16>((bf16*)d_out, (const bf16*)d_a, (const bf16*)d_b, n, ctx->stream));
}

// ---- loss --------------------------------------------------------------------------------------------
int bmc_xent(bmc_ctx_t* ctx, int dtype, void* d_logits, int ldv, float* d_row_loss, float* d_loss, const int* d_targets,
             const float* d_row_weight, int B, int S, int V, float grad_scale) {
    BMC_CHECK_CTX(ctx);
    int rc;
    if (dtype == BMC_F32)
        rc = xent_forward_backward<float>((float*)d_logits, d_row_loss, d_targets, d_row_weight, B * S, V, ldv, grad_scale, ctx->d_err, ctx->stream);
    else
        rc = xent_forward_backward<bf16>((bf16*)d_logits, d_row_loss, d_targets, d_row_weight, B * S, V, ldv, grad_scale, ctx->d_err, ctx->stream);
    if (rc) return rc;
    if (d_loss) rc = loss_reduce(d_loss, d_row_loss, B, S, d_row_weight != nullptr, ctx->stream);
    return note(ctx, rc, d_loss ? 2 : 1);
}

// ---- optimizer / casts / sampler ---------------------------------------------------------------------
int bmc_adamw(bmc_ctx_t* ctx, float* d_w, void* d_w_bf16, const void* d_g, int grad_dtype, float* d_m, float* d_v, size_t n,
              const float* h_hp) {
    BMC_CHECK_CTX(ctx);
    if (grad_dtype == BMC_F32) return note(ctx, adamw_f32grad(d_w, (bf16*)d_w_bf16, (const float*)d_g, d_m, d_v, n, h_hp, ctx->stream));
    return note(ctx, adamw_bf16grad(d_w, (bf16*)d_w_bf16, (const bf16*)d_g, d_m, d_v, n, h_hp, ctx->stream));
}
int bmc_cast_f32_to_bf16(bmc_ctx_t* ctx, void* d_out, const float* d_in, size_t n) {
    BMC_CHECK_CTX(ctx);
    return note(ctx, cast_f32_to_bf16((bf16*)d_out, d_in, n, ctx->stream));
}
int bmc_cast_bf16_to_f32(bmc_ctx_t* ctx, float* d_out, const void* d_in, size_t n) {
    BMC_CHECK_CTX(ctx);
    return note(ctx, cast_bf16_to_f32(d_out, (const bf16*)d_in, n, ctx->stream));
}
int bmc_seq_prefix_accumulate(bmc_ctx_t* ctx, int dtype, void* d_x, float* d_carry_f32, int B, size_t per_seq) {
    BMC_CHECK_CTX(ctx);
    if (dtype == BMC_F32) return note(ctx, seq_prefix_accumulate<float>((float*)d_x, d_carry_f32, B, per_seq, ctx->stream));
    return note(ctx, seq_prefix_accumulate<bf16>((bf16*)d_x, d_carry_f32, B, per_seq, ctx->stream));
}
int bmc_argmax(bmc_ctx_t* ctx, int* d_index, const float* d_logits, int V) {
    BMC_CHECK_CTX(ctx);
    return note(ctx, argmax_first(d_index, d_logits, V, ctx->stream));
}

// ---- inference (decode) ------------------------------------------------------------------------------
int bmc_decode_gemv(bmc_ctx_t* ctx, float* d_out, int ldo, const float* d_x, int ldx, int wtype, const void* d_w, const float* d_scales,
                    const float* d_residual, int ldr, int NB, int C, int OC) {
    BMC_CHECK_CTX(ctx);
    return note(ctx, decode_gemv(d_out, ldo, d_x, ldx, wtype, d_w, d_scales, d_residual, ldr, 0, nullptr, 0.f, NB, C, OC, ctx->stream));
}
int bmc_decode_gemv_fused(bmc_ctx_t* ctx, float* d_out, int ldo, const float* d_x, int ldx, int wtype, const void* d_w, const float* d_scales,
                          const float* d_residual, int ldr, int prologue, const float* d_norm_weight, float eps, int NB, int C, int OC) {
    BMC_CHECK_CTX(ctx);
    return note(ctx, decode_gemv(d_out, ldo, d_x, ldx, wtype, d_w, d_scales, d_residual, ldr, prologue, d_norm_weight, eps, NB, C, OC, ctx->stream));
}
int bmc_decode_rmsnorm(bmc_ctx_t* ctx, float* d_out, const float* d_x, const float* d_w, int NB, int C, float eps) {
    BMC_CHECK_CTX(ctx);
    return note(ctx, decode_rmsnorm(d_out, d_x, d_w, NB, C, eps, ctx->stream));
}
int bmc_decode_rope_kv(bmc_ctx_t* ctx, float* d_qkv, void* d_cache, int cache_dtype, const float* d_cs_table, const int* d_pos, int layer, int NB, int MS,
                       int NH, int NKV, int HD) {
    BMC_CHECK_CTX(ctx);
    return note(ctx, decode_rope_kv(d_qkv, d_cache, cache_dtype == BMC_BF16, d_cs_table, d_pos, layer, NB, MS, NH, NKV, HD, ctx->stream));
}
size_t bmc_decode_attention_scratch_bytes(int NB, int MS, int NH, int NKV, int HD) {
    return decode_attention_scratch_bytes(NB, MS, NH, NKV, HD) + 16;
}
int bmc_decode_attention(bmc_ctx_t* ctx, float* d_out, const float* d_qkv, const void* d_cache, int cache_dtype, const int* d_pos, void* d_scratch, int layer,
                         int NB, int MS, int NH, int NKV, int HD, float scale) {
    BMC_CHECK_CTX(ctx);
    return note(ctx, decode_attention(d_out, d_qkv, const_cast<void*>(d_cache), cache_dtype == BMC_BF16, nullptr, d_pos, d_scratch, layer, NB, MS, NH, NKV, HD, scale,
                                      ctx->stream));
}
int bmc_decode_attention_fused(bmc_ctx_t* ctx, float* d_out, const float* d_qkv, void* d_cache, int cache_dtype, const float* d_cs_table, const int* d_pos,
                               void* d_scratch, int layer, int NB, int MS, int NH, int NKV, int HD, float scale) {
    BMC_CHECK_CTX(ctx);
    if (!d_cs_table) return note(ctx, -1);
    return note(ctx, decode_attention(d_out, d_qkv, d_cache, cache_dtype == BMC_BF16, d_cs_table, d_pos, d_scratch, layer, NB, MS, NH, NKV, HD, scale, ctx->stream));
}
int bmc_decode_prep(bmc_ctx_t* ctx, void* d_a, int parts, const float* d_x, int ldx, int mode, const float* d_norm_weight, float eps,
                    float* d_init_out, int ldo, const float* d_init_src, int ldr, int n_out, int rows, int C) {
    BMC_CHECK_CTX(ctx);
    return note(ctx, decode_prep((bf16*)d_a, parts, d_x, ldx, mode, d_norm_weight, eps, d_init_out, ldo, d_init_src, ldr, n_out, rows, C, ctx->stream));
}
// out[rows, OC] (fp32, holds the running sum) += a[rows, parts*C] x w[OC, parts*C]^T on the tensor cores
int bmc_decode_gemm(bmc_ctx_t* ctx, float* d_out, int ldo, const void* d_a, const void* d_w, int parts, int rows, int C, int OC) {
    BMC_CHECK_CTX(ctx);
    const int K = parts * C;
    const int tiles_m = (rows + 127) / 128;
    int tile_n = 0, splits = 1;
    if (tiles_m * ((OC + 255) / 256) < ctx->num_sms) {  // few row tiles: narrow column tiles and a split reduction axis fill the GPU
        tile_n = 64;
        const int units = tiles_m * ((OC + 63) / 64);
        splits = (2 * ctx->num_sms + units - 1) / units;
        const int kb = (K + 63) / 64;
        if (splits > kb / 2) splits = kb / 2 > 0 ? kb / 2 : 1;
    }
    GemmProblem g{rows, OC, K, (const bf16*)d_a, K, 0, (const bf16*)d_w, K, 0, d_out, ldo, GEMM_OUT_F32_ATOMIC, nullptr, 0, splits, tile_n,
                  getenv("BM_NO_PDL") ? 0 : 1};
    return note(ctx, run_umma(ctx, g));
}
int bmc_decode_kv_scatter(bmc_ctx_t* ctx, void* d_cache, int cache_dtype, const float* d_qkv, int ldqkv, int layer, int NB, int T, int MS, int QD, int KV) {
    BMC_CHECK_CTX(ctx);
    return note(ctx, decode_kv_scatter(d_cache, cache_dtype == BMC_BF16, d_qkv, ldqkv, layer, NB, T, MS, QD, KV, ctx->stream));
}
int bmc_prefill_attention(bmc_ctx_t* ctx, float* d_out, int ldo, const float* d_q, int ldq, const float* d_k, const float* d_v, int ldkv, int NB,
                          int T, int NH, int NKV, int HD, float scale) {
    BMC_CHECK_CTX(ctx);
    // tcgen05 kernel on split bf16 operands (fp32-accurate); the split copies of Q, K and V live in the attention scratch
    void* scratch = scratch_get(ctx, &ctx->attn_scratch, &ctx->attn_scratch_bytes, prefill_attention_umma_scratch_bytes((long)NB * T, NH, NKV));
    if (!scratch) return -4;
    return note(ctx, prefill_attention_umma(d_out, ldo, d_q, ldq, d_k, d_v, ldkv, NB, T, NH, NKV, HD, scale, scratch, ctx->d_err, ctx->stream), 2);
}
int bmc_decode_swiglu(bmc_ctx_t* ctx, float* d_out, const float* d_gate_up, int NB, int H) {
    BMC_CHECK_CTX(ctx);
    return note(ctx, decode_swiglu(d_out, d_gate_up, NB, H, ctx->stream));
}
int bmc_decode_embed(bmc_ctx_t* ctx, float* d_out, int table_type, const void* d_table, const int* d_tokens, int NB, int D) {
    BMC_CHECK_CTX(ctx);
    return note(ctx, decode_embed(d_out, table_type, d_table, d_tokens, NB, D, ctx->stream));
}
int bmc_decode_argmax(bmc_ctx_t* ctx, int* d_out, const float* d_logits, int NB, int V) {
    BMC_CHECK_CTX(ctx);
    return note(ctx, decode_argmax(d_out, d_logits, NB, V, nullptr, ctx->stream));
}
int bmc_decode_argmax_advance(bmc_ctx_t* ctx, int* d_out, const float* d_logits, int NB, int V, int* d_pos) {
    BMC_CHECK_CTX(ctx);
    return note(ctx, decode_argmax(d_out, d_logits, NB, V, d_pos, ctx->stream));
}
int bmc_decode_advance(bmc_ctx_t* ctx, int* d_pos) {
    BMC_CHECK_CTX(ctx);
    return note(ctx, decode_advance(d_pos, ctx->stream));
}
int bmc_graph_select(bmc_ctx_t* ctx, int slot) {
    BMC_CHECK_CTX(ctx);
    if (slot < 0 || slot > 1) return -1;
    ctx->graph_slot = slot;
    return 0;
}
int bmc_graph_begin(bmc_ctx_t* ctx) {
    BMC_CHECK_CTX(ctx);
    const int k = ctx->graph_slot;
    if (ctx->graph_execs[k]) { cudaGraphExecDestroy(ctx->graph_execs[k]); ctx->graph_execs[k] = nullptr; }
    if (ctx->graphs[k]) { cudaGraphDestroy(ctx->graphs[k]); ctx->graphs[k] = nullptr; }
    ctx->launches_at_capture = ctx->launches;
    return cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal) == cudaSuccess ? 0 : -1;
}
int bmc_graph_end(bmc_ctx_t* ctx) {
    BMC_CHECK_CTX(ctx);
    const int k = ctx->graph_slot;
    if (cudaStreamEndCapture(ctx->stream, &ctx->graphs[k]) != cudaSuccess || !ctx->graphs[k]) {
        cudaGetLastError();  // a failed capture must not poison the status of later launches
        ctx->graphs[k] = nullptr;
        return -1;
    }
    if (cudaGraphInstantiate(&ctx->graph_execs[k], ctx->graphs[k], 0) != cudaSuccess) {
        cudaGetLastError();
        ctx->graph_execs[k] = nullptr;
        return -2;
    }
    // the capture itself went through note(), which counted launches that did not run: take them back, and count the graph's
    // kernel nodes once per replay instead
    size_t n_nodes = 0;
    ctx->graph_kernels[k] = 0;
    if (cudaGraphGetNodes(ctx->graphs[k], nullptr, &n_nodes) == cudaSuccess && n_nodes) {
        std::vector<cudaGraphNode_t> nodes(n_nodes);
        if (cudaGraphGetNodes(ctx->graphs[k], nodes.data(), &n_nodes) == cudaSuccess)
            for (size_t i = 0; i < n_nodes; ++i) {
                cudaGraphNodeType ty;
                if (cudaGraphNodeGetType(nodes[i], &ty) == cudaSuccess && ty == cudaGraphNodeTypeKernel) ++ctx->graph_kernels[k];
            }
    }
    ctx->launches = ctx->launches_at_capture;
    return 0;
}
int bmc_graph_launch(bmc_ctx_t* ctx) {
    BMC_CHECK_CTX(ctx);
    const int k = ctx->graph_slot;
    if (!ctx->graph_execs[k]) return -1;
    if (cudaGraphLaunch(ctx->graph_execs[k], ctx->stream) != cudaSuccess) return -2;
    ctx->launches += ctx->graph_kernels[k];
    return 0;
}
int bmc_gemm_timing_enabled(bmc_ctx_t* ctx) { return ctx && ctx->gemm_timing ? 1 : 0; }
// Copies *d_value and the error word to pinned host memory and records an event behind the copies, all on the context's stream and
// all capturable: inside a stream capture the event becomes an external event node, so the host can wait for THIS point of a
// replayed graph (bmc_early_wait) while the rest of the graph is still running.
int bmc_early_readback(bmc_ctx_t* ctx, const float* d_value) {
    BMC_CHECK_CTX(ctx);
    if (!ctx->h_early) {
        if (cudaMallocHost((void**)&ctx->h_early, 2 * sizeof(float)) != cudaSuccess) { ctx->h_early = nullptr; return -1; }
        if (cudaEventCreateWithFlags(&ctx->early_ev, cudaEventDisableTiming) != cudaSuccess) { cudaFreeHost(ctx->h_early); ctx->h_early = nullptr; return -1; }
    }
    if (cudaMemcpyAsync(ctx->h_early, d_value, sizeof(float), cudaMemcpyDeviceToHost, ctx->stream) != cudaSuccess) return -2;
    if (cudaMemcpyAsync(ctx->h_early + 1, ctx->d_err, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream) != cudaSuccess) return -2;
    return cudaEventRecordWithFlags(ctx->early_ev, ctx->stream, cudaEventRecordExternal) == cudaSuccess ? 0 : -3;
}
// Waits for the most recent bmc_early_readback to land. *status_out is the error word as it stood at that point of the stream.
int bmc_early_wait(bmc_ctx_t* ctx, float* value_out, int* status_out) {
    BMC_CHECK_CTX(ctx);
    if (!ctx->h_early) return -1;
    const cudaError_t e = cudaEventSynchronize(ctx->early_ev);
    if (e != cudaSuccess) {
        ctx->sticky_status = -200 - (int)e;
        return ctx->sticky_status;
    }
    if (value_out) *value_out = ctx->h_early[0];
    if (status_out) memcpy(status_out, ctx->h_early + 1, sizeof(int));
    return ctx->sticky_status;
}
int bmc_selftest_bounded_wait(bmc_ctx_t* ctx) {
    BMC_CHECK_CTX(ctx);
    return note(ctx, wait_probe_launch(ctx->d_err, ctx->stream));
}

}  // extern "C"
