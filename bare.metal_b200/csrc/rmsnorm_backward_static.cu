// RMSNorm backward for callers that must not allocate device memory.
//
// bmc_rmsnorm_backward() keeps its per-block partial sums in a buffer the context obtains from cudaMalloc the
// first time it is needed (and again whenever a wider row arrives). Some embedders cannot tolerate that:
//   * a host application that reserves the whole GPU for its own arena or caching pool at start-up, after which a
//     late cudaMalloc from a library either fails or fragments the pool's address space;
//   * a latency-critical training or serving loop that has been written so that no call in steady state can block
//     the device: cudaMalloc and cudaFree synchronise the whole device implicitly;
//   * plug-in style hosts whose contract with extensions is "bring your own memory, never call the CUDA allocator".
// For them this file offers the same computation with the partial-sum buffer living in a fixed, file-scope device
// array. The entry point takes a raw stream instead of a backend context and performs no allocation of any kind.
//
// Limits and sharing rules
//   * Row width C <= BMC_STATIC_RMS_MAX_C (1024 floats wide: covers SmolLM2-135M/360M, D = 576 / 960). Wider rows
//     are rejected with BMC_ERR_STATIC_TOO_LARGE and a message on stderr; use bmc_rmsnorm_backward() for those.
//   * The array is 592 x 1024 floats = 2.3 MiB and is part of the library image: every GPU on which the library is
//     loaded carries it until the process exits, whether or not this entry point is ever called.
//   * All calls on one GPU share the one array. A call first writes every word it will later read, so whatever an
//     earlier call left behind is harmless and nothing has to be cleared. Two calls whose kernels overlap on the GPU
//     (different streams, or the same stream from two host threads without ordering) would race on it: serialise them.
//   * The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that device
//     current). Make that first call during start-up, before any stream capture begins.
#include <stdio.h>

#include <mutex>

#include "../../include/bm_cuda_backend.h"
#include "kernels.cuh"

namespace {

constexpr int kMaxDevices = 64;
constexpr size_t kScratchFloats = (size_t)592 * BMC_STATIC_RMS_MAX_C;

// In host code this name is only a handle for the runtime's symbol table, not a device address:
// it must be translated with cudaGetSymbolAddress before a kernel can be given the pointer.
static __device__ __align__(256) float g_rms_static_scratch[kScratchFloats];

float* g_scratch_addr[kMaxDevices];
std::mutex g_mu;

// Device address of the scratch array on the CURRENT device; resolved once per device.
int scratch_on_current_device(float** out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return -61;
    std::lock_guard<std::mutex> lk(g_mu);
    if (!g_scratch_addr[dev]) {
        float* ptr = nullptr;
        const cudaError_t e = cudaGetSymbolAddress((void**)&ptr, g_rms_static_scratch);
        if (e != cudaSuccess || !ptr) {
            fprintf(stderr, "bmc_rmsnorm_backward_static: cudaGetSymbolAddress failed on device %d: %s\n", dev, cudaGetErrorString(e));
            return -62;
        }
        g_scratch_addr[dev] = ptr;
    }
    *out = g_scratch_addr[dev];
    return 0;
}

}  // namespace

extern "C" int bmc_rmsnorm_backward_static(void* cuda_stream, int dtype, void* d_gx, float* d_gw_f32, int gw_accumulate,
                                           const void* d_gout, const void* d_x, const float* d_w, const float* d_rstd, int N, int C,
                                           int w_row0, int w_row1) {
    if (N <= 0 || C <= 0) return -1;
    if (C > BMC_STATIC_RMS_MAX_C || bmb::rmsnorm_backward_scratch_floats(C) > kScratchFloats) {
        fprintf(stderr,
                "bmc_rmsnorm_backward_static: row width C=%d exceeds the built-in scratch (max C = %d); "
                "use bmc_rmsnorm_backward(), which sizes its scratch on demand\n",
                C, BMC_STATIC_RMS_MAX_C);
        return BMC_ERR_STATIC_TOO_LARGE;
    }
    float* scratch = nullptr;
    const int rc = scratch_on_current_device(&scratch);
    if (rc) return rc;
    cudaStream_t st = (cudaStream_t)cuda_stream;
    int lrc;
    if (dtype == BMC_F32)
        lrc = bmb::rmsnorm_backward<float>((float*)d_gx, d_gw_f32, gw_accumulate, (const float*)d_gout, (const float*)d_x, d_w, d_rstd, N,
                                           C, w_row0, w_row1, scratch, st);
    else if (dtype == BMC_BF16)
        lrc = bmb::rmsnorm_backward<bmb::bf16>((bmb::bf16*)d_gx, d_gw_f32, gw_accumulate, (const bmb::bf16*)d_gout, (const bmb::bf16*)d_x,
                                               d_w, d_rstd, N, C, w_row0, w_row1, scratch, st);
    else
        return -2;
    if (lrc) return lrc;
    // A launch that the runtime refused (a stream of another device, a first call made during stream capture, ...) is an
    // error of this call, reported the way the context-based entry points report it: -200 - cudaError.
    const cudaError_t le = cudaPeekAtLastError();
    if (le != cudaSuccess) {
        fprintf(stderr, "bmc_rmsnorm_backward_static: launch failed: %s\n", cudaGetErrorString(le));
        return -200 - (int)le;
    }
    return 0;
}
