// TEST INFRASTRUCTURE — not part of the product, never linked into it.
//
// A CPU implementation of the reference's internal backend ABI (src/backend/backend.h:17-67)
// whose "kernels" are the reference's own Metal shader sources, compiled as C++ through
// oracle/metal_stub/metal_stdlib and executed thread by thread by a grid loop (OpenMP across
// the grid). Linked with the reference's unmodified C11 host code it yields oracle/_ref/libbm_ref.so:
// the reference's training step (graph, scheduler, trainer, AdamW, state files) running on host
// cores. That library is the parity oracle "kind: reference" and the timed CPU baseline.
//
// Only kernels without threadgroup barriers or cross-lane operations are registered. For every
// other name backend_kernel_create() returns NULL, which the reference scheduler answers by
// falling back to the barrier-free kernel of the same op (scheduler.c:1117-1146, 1430-1456);
// the reference's own tests establish that the variants agree (test/train_attn_tiled_test.c:105,125,
// test/matmul_prefill_test.c:92).
//
// Buffers are plain host allocations: map() returns the allocation itself, exactly like the
// shared-storage MTLBuffers of the reference (src/backend/metal/device.m:116-189).
#include <stdio.h>
#include <time.h>

#include <functional>
#include <map>
#include <string>
#include <tuple>
#include <utility>

// The stub defines the MSL address-space keywords as macros; keep every other header above it
// and drop the macros again once the shader sources have been read.
#include <metal_stdlib>

namespace fwd {
#include BM_REF_FORWARD_METAL
}
namespace bwd {
#include BM_REF_BACKWARD_METAL
}
namespace opt {
#include BM_REF_ADAMW_METAL
}
#undef kernel
#undef device
#undef thread
#undef constant
#undef threadgroup

extern "C" {
#include "backend/backend.h"
#include "backend/metal/device.h"
}

// ---- generic adapter: buffer list + thread id -> kernel function call ---------------------
namespace {

struct Gid { unsigned x, y, z; };

template <class T> struct BindBuf {  // pointer parameter: the buffer itself
    static T get(void* p) { return (T)p; }
};
template <class T> struct BindBuf<const T&> {  // `constant T&` parameter: first element of the buffer
    static const T& get(void* p) { return *(const T*)p; }
};
template <class T> struct BindGid;
template <> struct BindGid<metal::uint> { static metal::uint get(Gid g) { return g.x; } };
template <> struct BindGid<metal::uint2> { static metal::uint2 get(Gid g) { return metal::uint2{g.x, g.y}; } };
template <> struct BindGid<metal::uint3> { static metal::uint3 get(Gid g) { return metal::uint3{g.x, g.y, g.z}; } };

using Thunk = std::function<void(void** bufs, Gid gid)>;

template <class... A, size_t... I>
Thunk make_thunk_impl(void (*fn)(A...), std::index_sequence<I...>) {
    using Tup = std::tuple<A...>;
    constexpr size_t NB = sizeof...(A) - 1;
    return [fn](void** bufs, Gid gid) {
        fn(BindBuf<std::tuple_element_t<I, Tup>>::get(bufs[I])..., BindGid<std::tuple_element_t<NB, Tup>>::get(gid));
    };
}
template <class... A> std::pair<Thunk, int> make_thunk(void (*fn)(A...)) {
    return {make_thunk_impl(fn, std::make_index_sequence<sizeof...(A) - 1>{}), (int)sizeof...(A) - 1};
}

// `regrid` (optional) derives the launch grid from the kernel's own parameter buffer instead of the
// grid the caller passed; used when a tiled kernel name is served by its barrier-free sibling.
struct KernelEntry { Thunk call; int n_bufs; std::function<void(void** bufs, int* g)> regrid; };

const std::map<std::string, KernelEntry>& kernel_table() {
    static std::map<std::string, KernelEntry> t;
    if (!t.empty()) return t;
#define REG(ns, name) { auto pr = make_thunk(&ns::name); t[#name] = KernelEntry{pr.first, pr.second, nullptr}; }
    // forward (src/kernels/forward.metal)
    REG(fwd, matmul_forward_naive)
    REG(fwd, matmul_forward_bf16)
    REG(fwd, matmul_forward_q8)
    REG(fwd, matmul_forward_q4)
    REG(fwd, rmsnorm_forward)
    REG(fwd, swiglu_forward)
    REG(fwd, add_forward)
    REG(fwd, rope_forward_seq)
    REG(fwd, rope_forward)
    REG(fwd, kv_store)
    REG(fwd, attention_forward_seq)
    REG(fwd, attention_forward_seq_masked)
    REG(fwd, attention_forward_prefill)
    // backward (src/kernels/backward.metal)
    REG(bwd, zero_buffer)
    REG(bwd, matmul_backward_inp)
    REG(bwd, matmul_backward_inp_bf16)
    REG(bwd, matmul_backward_w)
    REG(bwd, rmsnorm_backward_x)
    REG(bwd, rmsnorm_backward_w)
    REG(bwd, swiglu_backward)
    REG(bwd, add_backward)
    REG(bwd, rope_backward_seq)
    REG(bwd, attention_backward)
    REG(bwd, attention_backward_masked)
    REG(bwd, xent_backward)
    REG(bwd, xent_backward_masked)
    REG(bwd, embedding_backward)
    // optimizer (src/anneal/adamw.metal)
    REG(opt, adamw_step)
#undef REG
    // The reference scheduler has no barrier-free fallback for the bf16 input-gradient GEMM when BT > 1: with
    // the tiled kernel missing it would run the fp32 kernel on bf16 weight bytes (src/baremetal/scheduler.c:1430-1441).
    // Serve the tiled name with the per-thread bf16 kernel of the same arithmetic
    // (matmul_backward_inp_bf16, src/kernels/backward.metal:49-66; params {BT, C, OC} in slot 3; one thread per (i, bt)).
    {
        KernelEntry e = t["matmul_backward_inp_bf16"];
        e.regrid = [](void** bufs, int* g) {
            const int* p = (const int*)bufs[3];
            g[0] = p[1]; g[1] = p[0]; g[2] = 1;
        };
        t["matmul_backward_inp_bf16_tiled"] = e;
    }
    return t;
}

double now_ms() {
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return ts.tv_sec * 1e3 + ts.tv_nsec / 1e6;
}

}  // namespace

// The handle structs are the reference's own (src/backend/metal/device.h:9-44): its api.c reads
// backend_ctx_s::supports_bf16 directly (src/baremetal/api.c:29), so the layout is part of the ABI.
// Field use here: backend_buffer_s::buffer = host allocation, backend_kernel_s::pipeline_state =
// KernelEntry*, backend_encoder_s::command_buffer = heap double accumulating the encoder's run time.
extern "C" {

backend_ctx_t* backend_create(void) {
    backend_ctx_t* c = (backend_ctx_t*)calloc(1, sizeof(backend_ctx_t));
    if (c) c->supports_bf16 = 1;
    return c;
}
void backend_destroy(backend_ctx_t* ctx) { free(ctx); }
size_t backend_get_allocated_memory(backend_ctx_t* ctx) { return ctx ? ctx->allocated_bytes : 0; }
size_t backend_get_peak_allocated_memory(backend_ctx_t* ctx) { return ctx ? ctx->peak_allocated_bytes : 0; }

void backend_get_device_info(backend_ctx_t*, backend_device_info_t* out) {
    if (!out) return;
    out->max_threads_per_threadgroup = 1024;
    out->max_threadgroup_memory = 32768;
    out->max_buffer_bytes = (size_t)1 << 40;
    out->recommended_max_working_set = (size_t)1 << 40;
    out->has_unified_memory = 1;
}
double backend_get_gpu_busy_ms(backend_ctx_t* ctx) { return ctx ? ctx->gpu_busy_ms : 0.0; }
uint64_t backend_get_command_buffers(backend_ctx_t* ctx) { return ctx ? ctx->cmd_buffers : 0; }
void backend_reset_gpu_timing(backend_ctx_t* ctx) {
    if (ctx) { ctx->gpu_busy_ms = 0; ctx->cmd_buffers = 0; }
}

backend_buffer_t* backend_buffer_alloc(backend_ctx_t* ctx, size_t size) {
    if (!ctx || size == 0) return NULL;
    backend_buffer_t* b = (backend_buffer_t*)calloc(1, sizeof(*b));
    b->buffer = calloc(1, size);  // fresh shared-storage MTLBuffers read as zero
    if (!b->buffer) { free(b); return NULL; }
    b->ctx = ctx;
    b->size = size;
    ctx->allocated_bytes += size;
    if (ctx->allocated_bytes > ctx->peak_allocated_bytes) ctx->peak_allocated_bytes = ctx->allocated_bytes;
    return b;
}
void backend_buffer_free(backend_buffer_t* b) {
    if (!b) return;
    if (b->ctx) b->ctx->allocated_bytes -= b->size;
    free(b->buffer);
    free(b);
}
void* backend_buffer_map(backend_buffer_t* b) { return b ? b->buffer : NULL; }
void backend_buffer_unmap(backend_buffer_t*) {}
size_t backend_buffer_size(backend_buffer_t* b) { return b ? b->size : 0; }

backend_kernel_t* backend_kernel_create(backend_ctx_t* ctx, const char* name) {
    if (!ctx || !name) return NULL;
    auto it = kernel_table().find(name);
    if (it == kernel_table().end()) return NULL;
    backend_kernel_t* k = (backend_kernel_t*)calloc(1, sizeof(*k));
    k->pipeline_state = (void*)&it->second;
    return k;
}
void backend_kernel_destroy(backend_kernel_t* k) { free(k); }

static int run_grid(backend_kernel_t* k, backend_buffer_t* buffers[], size_t offsets[], int nb, int gx, int gy, int gz) {
    if (!k || !buffers) return -1;
    void* ptrs[32] = {0};
    if (nb > 32) return -1;
    for (int i = 0; i < nb; i++)
        ptrs[i] = buffers[i] ? (char*)buffers[i]->buffer + (offsets ? offsets[i] : 0) : NULL;
    const KernelEntry* e = (const KernelEntry*)k->pipeline_state;
    if (e->regrid) {
        int g[3];
        e->regrid(ptrs, g);
        gx = g[0]; gy = g[1]; gz = g[2];
    }
    const long total = (long)gx * gy * gz;
#pragma omp parallel for schedule(dynamic, 16) if (total >= 64)
    for (long t = 0; t < total; t++) {
        Gid g;
        g.x = (unsigned)(t % gx);
        g.y = (unsigned)((t / gx) % gy);
        g.z = (unsigned)(t / ((long)gx * gy));
        e->call(ptrs, g);
    }
    return 0;
}

int backend_kernel_dispatch(backend_ctx_t* ctx, backend_kernel_t* k, backend_buffer_t* buffers[], size_t offsets[], int nb,
                            int gx, int gy, int gz, int, int, int) {
    if (!ctx) return -1;
    double t0 = now_ms();
    int rc = run_grid(k, buffers, offsets, nb, gx, gy, gz);
    ctx->gpu_busy_ms += now_ms() - t0;
    ctx->cmd_buffers += 1;
    return rc;
}
void backend_synchronize(backend_ctx_t*) {}

backend_encoder_t* backend_encode_begin(backend_ctx_t* ctx) {
    if (!ctx) return NULL;
    backend_encoder_t* e = (backend_encoder_t*)calloc(1, sizeof(*e));
    e->ctx = ctx;
    e->command_buffer = calloc(1, sizeof(double));
    return e;
}
// Dispatches run at encode time: host memory is the device memory, and a Metal compute encoder
// executes its dispatches serially in order, so eager execution is observationally the same.
int backend_encode_dispatch(backend_encoder_t* enc, backend_kernel_t* k, backend_buffer_t* buffers[], size_t offsets[], int nb,
                            int gx, int gy, int gz, int, int, int) {
    if (!enc) return -1;
    double t0 = now_ms();
    int rc = run_grid(k, buffers, offsets, nb, gx, gy, gz);
    *(double*)enc->command_buffer += now_ms() - t0;
    return rc;
}
void backend_encode_commit(backend_encoder_t*) {}
double backend_encode_wait_timed(backend_encoder_t* enc) {
    if (!enc) return 0.0;
    double ms = *(double*)enc->command_buffer;
    enc->ctx->gpu_busy_ms += ms;
    enc->ctx->cmd_buffers += 1;
    free(enc->command_buffer);
    free(enc);
    return ms;
}
void backend_encode_wait(backend_encoder_t* enc) { (void)backend_encode_wait_timed(enc); }

}  // extern "C"
