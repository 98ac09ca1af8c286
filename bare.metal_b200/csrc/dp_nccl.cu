// Data-parallel gradient all-reduce over NCCL (NVLink 5 / NVSwitch), overlapped with backward.
//
// Gradients are produced in fp32 in one flat array (trainer-state order: layer 0 .. layer L-1, final norm,
// tied embedding). Layers are grouped into buckets; as soon as backward has finished the lowest layer of a
// bucket, the compute stream records an event, and the communication stream (a) casts that fp32 range to
// bf16 into a flat bf16 gradient array, (b) all-reduces it in place (sum) — a trainer in fp32 mode skips the cast and all-reduces
// the fp32 range itself, so that its 1e-4 parity bound also holds across ranks. Backward runs from the last layer
// to the first, so buckets complete from the end of the array towards the start and their reductions overlap
// the remaining backward work; the final-norm + embedding bucket completes last. AdamW then reads the reduced
// bf16 gradients with grad_scale = 1 / (sequences per rank * world).
//
// NCCL is bound at run time with dlopen("libnccl.so.2"), so a single-GPU process never needs the library and
// a process that already loaded NCCL (e.g. through torch) shares that copy.
#include <dlfcn.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

#include <vector>

#include "../host/dp.h"
#include "kernels.cuh"

namespace {

typedef struct ncclComm* ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
enum { ncclSuccess = 0 };
enum { ncclFloat32 = 7, ncclBfloat16 = 9 };
enum { ncclSum = 0 };

struct NcclApi {
    void* lib;
    int (*GetUniqueId)(ncclUniqueId*);
    int (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int);
    int (*CommDestroy)(ncclComm_t);
    int (*AllReduce)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t);
    const char* (*GetErrorString)(int);
    int (*CommGetAsyncError)(ncclComm_t, int*);  // optional
    int (*CommAbort)(ncclComm_t);                // optional
};

NcclApi* nccl() {
    static NcclApi api;
    static int state = 0;  // 0 = untried, 1 = ok, -1 = failed
    if (state == 0) {
        state = -1;
        api.lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!api.lib) api.lib = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (api.lib) {
            api.GetUniqueId = (int (*)(ncclUniqueId*))dlsym(api.lib, "ncclGetUniqueId");
            api.CommInitRank = (int (*)(ncclComm_t*, int, ncclUniqueId, int))dlsym(api.lib, "ncclCommInitRank");
            api.CommDestroy = (int (*)(ncclComm_t))dlsym(api.lib, "ncclCommDestroy");
            api.AllReduce = (int (*)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t))dlsym(api.lib, "ncclAllReduce");
            api.GetErrorString = (const char* (*)(int))dlsym(api.lib, "ncclGetErrorString");
            api.CommGetAsyncError = (int (*)(ncclComm_t, int*))dlsym(api.lib, "ncclCommGetAsyncError");
            api.CommAbort = (int (*)(ncclComm_t))dlsym(api.lib, "ncclCommAbort");
            if (api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.AllReduce) state = 1;
        }
        if (state != 1) fprintf(stderr, "[ERROR] data parallel: cannot load NCCL (libnccl.so.2): %s\n", dlerror());
    }
    return state == 1 ? &api : nullptr;
}

struct Bucket {
    size_t begin, end;  // element range in the flat parameter order
    int ready_at;       // bm_dp_bucket_ready(layer) value that completes the bucket
};

}  // namespace

struct bm_dp_s {
    bmc_ctx_t* be;
    int rank, world;
    ncclComm_t comm;
    cudaStream_t comm_stream;
    std::vector<Bucket> buckets;
    std::vector<cudaEvent_t> ready_ev;
    cudaEvent_t done_ev;
    float* d_grad_f32;
    bmb::bf16* d_grad_bf16;
    float* d_loss_buf;
    size_t P;
    int last_microstep;
    int f32;          // gradients travel as fp32 (trainer in fp32 mode)
    int failed;       // a wait ran out or NCCL reported an asynchronous error: the communicator has been aborted
    double timeout_s; // host-side bound on every wait for the communication stream (env BM_DP_TIMEOUT_S, default 600)
    // BM_DP_PROFILE=1: CUDA events around every bucket's exchange and at the end of backward; rank 0 prints the averages when
    // the exchange is destroyed. The step is synchronised after AdamW has been enqueued, so profiled steps are slower.
    int profile;
    long prof_steps;
    std::vector<cudaEvent_t> t0_ev, t1_ev;
    cudaEvent_t bwd_done_ev, all_done_ev;
    std::vector<double> prof_start_ms, prof_dur_ms;   // per bucket: start after the first bucket became ready, duration
    double prof_tail_ms;                              // end of the last exchange minus end of backward: what AdamW waited for
};

namespace {
// Host-side wait for the communication stream with a deadline: polls the stream (and NCCL's asynchronous error state where
// the library offers it) instead of blocking, so that a peer that exited or never joined ends this rank's step with an error
// instead of hanging it behind a spinning NCCL kernel. On expiry or error the communicator is aborted (ncclCommAbort frees the
// stream) and every later exchange fails fast.
int wait_comm(bm_dp_s* dp) {
    if (dp->failed) return -1;
    NcclApi* api = nccl();
    struct timespec t0, t;
    clock_gettime(CLOCK_MONOTONIC, &t0);
    for (long it = 0;; ++it) {
        const cudaError_t q = cudaStreamQuery(dp->comm_stream);
        if (q == cudaSuccess) return 0;
        int async_err = 0;
        bool bad = q != cudaErrorNotReady;
        if (!bad && api && api->CommGetAsyncError && (it & 63) == 0 && api->CommGetAsyncError(dp->comm, &async_err) == ncclSuccess && async_err != ncclSuccess)
            bad = true;
        clock_gettime(CLOCK_MONOTONIC, &t);
        const double el = (double)(t.tv_sec - t0.tv_sec) + 1e-9 * (double)(t.tv_nsec - t0.tv_nsec);
        if (bad || el > dp->timeout_s) {
            fprintf(stderr, "[ERROR] data parallel: %s after %.1f s on rank %d; aborting the communicator\n",
                    bad ? "communication error" : "gradient exchange timed out", el, dp->rank);
            if (api && api->CommAbort && dp->comm) { api->CommAbort(dp->comm); dp->comm = nullptr; }
            dp->failed = 1;
            return -1;
        }
        if (it > 1000) {   // after the first microseconds of spinning, yield the core between polls
            struct timespec ns = {0, 50000};
            nanosleep(&ns, nullptr);
        }
    }
}
}  // namespace

extern "C" {

// Bucket plan (pure host logic): groups of `layers_per_bucket` layers, highest layers first — the order in which
// backward completes them —, layer 0 in a bucket of its own, then one tail bucket holding the final norm and the tied
// embedding, which the embedding scatter completes last. Whatever is exchanged after backward has ended is exposed (nothing is
// left to hide it behind), so the last two buckets are kept small: one layer and the embedding. Bucket i covers elements
// [begin[i], end[i]) of the flat parameter order and is complete when backward reports ready_at[i] (a layer index, or -1 for
// the tail). Returns the bucket count; fills the arrays when cap is large enough.
int bmx_dp_plan_buckets(int n_layers, const size_t* layer_begin, size_t n_params_total, int layers_per_bucket, size_t* begin,
                        size_t* end, int* ready_at, int cap) {
    if (layers_per_bucket < 1) layers_per_bucket = 1;
    int n = 0;
    const int first_grouped = n_layers > 1 ? 1 : 0;   // layers [first_grouped, n_layers) are grouped from the top
    for (int hi = n_layers; hi > first_grouped; hi -= layers_per_bucket) {
        const int lo = hi - layers_per_bucket > first_grouped ? hi - layers_per_bucket : first_grouped;
        if (n < cap && begin) { begin[n] = layer_begin[lo]; end[n] = layer_begin[hi]; ready_at[n] = lo; }
        ++n;
    }
    if (first_grouped) {
        if (n < cap && begin) { begin[n] = layer_begin[0]; end[n] = layer_begin[1]; ready_at[n] = 0; }
        ++n;
    }
    if (n < cap && begin) { begin[n] = layer_begin[n_layers]; end[n] = n_params_total; ready_at[n] = -1; }
    ++n;
    return n;
}

int bmx_dp_unique_id(void* out_id) {
    NcclApi* api = nccl();
    if (!api || !out_id) return -1;
    ncclUniqueId id;
    if (api->GetUniqueId(&id) != ncclSuccess) return -2;
    memcpy(out_id, &id, sizeof id);
    return 0;
}

struct bm_dp_s* bm_dp_create(bmc_ctx_t* be, int rank, int world, const void* nccl_id, size_t P, int n_layers, const size_t* layer_begin,
                             float* d_grad_f32, int grads_f32) {
    NcclApi* api = nccl();
    if (!api || !be || !nccl_id || world < 1 || rank < 0 || rank >= world) return nullptr;
    bm_dp_s* dp = new bm_dp_s();
    dp->be = be;
    dp->rank = rank;
    dp->world = world;
    dp->P = P;
    dp->d_grad_f32 = d_grad_f32;
    dp->last_microstep = 1;
    dp->f32 = grads_f32 ? 1 : 0;
    dp->failed = 0;
    dp->timeout_s = 600.0;
    if (const char* te = getenv("BM_DP_TIMEOUT_S")) if (atof(te) > 0) dp->timeout_s = atof(te);
    dp->d_grad_bf16 = nullptr;
    ncclUniqueId id;
    memcpy(&id, nccl_id, sizeof id);
    int rc = api->CommInitRank(&dp->comm, world, id, rank);
    if (rc != ncclSuccess) {
        fprintf(stderr, "[ERROR] ncclCommInitRank failed: %s\n", api->GetErrorString ? api->GetErrorString(rc) : "?");
        delete dp;
        return nullptr;
    }
    cudaStreamCreateWithFlags(&dp->comm_stream, cudaStreamNonBlocking);
    cudaEventCreateWithFlags(&dp->done_ev, cudaEventDisableTiming);
    if ((!dp->f32 && cudaMalloc(&dp->d_grad_bf16, P * sizeof(bmb::bf16)) != cudaSuccess) || cudaMalloc(&dp->d_loss_buf, 16) != cudaSuccess) {
        fprintf(stderr, "[ERROR] data parallel: out of device memory\n");
        delete dp;
        return nullptr;
    }
    int per = 4;
    const char* e = getenv("BM_DP_LAYERS_PER_BUCKET");
    if (e && atoi(e) > 0) per = atoi(e);
    const int nb = bmx_dp_plan_buckets(n_layers, layer_begin, P, per, nullptr, nullptr, nullptr, 0);
    std::vector<size_t> bb(nb), be_(nb);
    std::vector<int> br(nb);
    bmx_dp_plan_buckets(n_layers, layer_begin, P, per, bb.data(), be_.data(), br.data(), nb);
    for (int i = 0; i < nb; ++i) dp->buckets.push_back(Bucket{bb[i], be_[i], br[i]});
    dp->ready_ev.resize(dp->buckets.size());
    dp->profile = getenv("BM_DP_PROFILE") != nullptr;
    for (auto& ev : dp->ready_ev) cudaEventCreateWithFlags(&ev, dp->profile ? cudaEventDefault : cudaEventDisableTiming);
    dp->prof_steps = 0;
    dp->prof_tail_ms = 0.0;
    if (dp->profile) {
        dp->t0_ev.resize(dp->buckets.size());
        dp->t1_ev.resize(dp->buckets.size());
        for (auto& ev : dp->t0_ev) cudaEventCreate(&ev);
        for (auto& ev : dp->t1_ev) cudaEventCreate(&ev);
        cudaEventCreate(&dp->bwd_done_ev);
        cudaEventCreate(&dp->all_done_ev);
        dp->prof_start_ms.assign(dp->buckets.size(), 0.0);
        dp->prof_dur_ms.assign(dp->buckets.size(), 0.0);
    }
    return dp;
}

void bm_dp_destroy(struct bm_dp_s* dp) {
    if (!dp) return;
    if (!dp->failed) wait_comm(dp);
    if (dp->profile && dp->rank == 0 && dp->prof_steps > 0) {
        const double n = (double)dp->prof_steps, esz = dp->f32 ? 4.0 : 2.0;
        fprintf(stderr, "[dp profile] %ld steps, %d ranks, %s gradients; times in ms, averages per step\n", dp->prof_steps, dp->world,
                dp->f32 ? "fp32" : "bf16");
        for (size_t i = 0; i < dp->buckets.size(); ++i) {
            const double mb = (double)(dp->buckets[i].end - dp->buckets[i].begin) * esz / 1e6, dur = dp->prof_dur_ms[i] / n;
            fprintf(stderr, "[dp profile] bucket %zu (ready at layer %d): %.1f MB, starts %.2f after the first bucket, takes %.3f (bus %.0f GB/s)\n", i,
                    dp->buckets[i].ready_at, mb, dp->prof_start_ms[i] / n, dur, dur > 0 ? mb / dur * 2.0 * (dp->world - 1) / dp->world : 0.0);
        }
        fprintf(stderr, "[dp profile] last exchange ends %.3f after backward ends (what AdamW waits for)\n", dp->prof_tail_ms / n);
    }
    for (auto& ev : dp->t0_ev) cudaEventDestroy(ev);
    for (auto& ev : dp->t1_ev) cudaEventDestroy(ev);
    if (dp->profile) { cudaEventDestroy(dp->bwd_done_ev); cudaEventDestroy(dp->all_done_ev); }
    NcclApi* api = nccl();
    if (api && dp->comm) api->CommDestroy(dp->comm);
    for (auto& ev : dp->ready_ev) cudaEventDestroy(ev);
    cudaEventDestroy(dp->done_ev);
    cudaFree(dp->d_grad_bf16);
    cudaFree(dp->d_loss_buf);
    cudaStreamDestroy(dp->comm_stream);
    delete dp;
}

int bm_dp_world(struct bm_dp_s* dp) { return dp ? dp->world : 1; }
void bm_dp_begin_window(struct bm_dp_s*) {}
void bm_dp_set_last_microstep(struct bm_dp_s* dp, int is_last) { if (dp) dp->last_microstep = is_last; }

// cast (bf16 mode) + all-reduce of one bucket on the communication stream, behind an event recorded now on the compute stream
static int reduce_bucket(struct bm_dp_s* dp, size_t i) {
    NcclApi* api = nccl();
    if (!api || dp->failed) return -3;
    cudaStream_t compute = (cudaStream_t)bmc_stream(dp->be);
    const Bucket& b = dp->buckets[i];
    cudaEventRecord(dp->ready_ev[i], compute);
    cudaStreamWaitEvent(dp->comm_stream, dp->ready_ev[i], 0);
    if (dp->profile) cudaEventRecord(dp->t0_ev[i], dp->comm_stream);
    const size_t n = b.end - b.begin;
    int rc;
    if (dp->f32) {
        rc = api->AllReduce(dp->d_grad_f32 + b.begin, dp->d_grad_f32 + b.begin, n, ncclFloat32, ncclSum, dp->comm, dp->comm_stream);
    } else {
        if (bmb::cast_f32_to_bf16(dp->d_grad_bf16 + b.begin, dp->d_grad_f32 + b.begin, n, dp->comm_stream)) return -1;
        rc = api->AllReduce(dp->d_grad_bf16 + b.begin, dp->d_grad_bf16 + b.begin, n, ncclBfloat16, ncclSum, dp->comm, dp->comm_stream);
    }
    if (rc != ncclSuccess) {
        fprintf(stderr, "[ERROR] ncclAllReduce failed: %s\n", api->GetErrorString ? api->GetErrorString(rc) : "?");
        return -2;
    }
    if (dp->profile) cudaEventRecord(dp->t1_ev[i], dp->comm_stream);
    return 0;
}

int bm_dp_bucket_ready(struct bm_dp_s* dp, int layer) {
    if (!dp || !dp->last_microstep) return 0;
    for (size_t i = 0; i < dp->buckets.size(); ++i) {
        if (dp->buckets[i].ready_at != layer) continue;
        const int rc = reduce_bucket(dp, i);
        if (rc) return rc;
    }
    return 0;
}

// Every bucket at once: for a window that ends before its last micro-step (bm_train_flush), whose gradients were never exchanged.
// A collective call: every rank must make it.
int bm_dp_reduce_all(struct bm_dp_s* dp) {
    if (!dp) return 0;
    for (size_t i = 0; i < dp->buckets.size(); ++i) {
        const int rc = reduce_bucket(dp, i);
        if (rc) return rc;
    }
    return 0;
}

int bm_dp_adamw(struct bm_dp_s* dp, bm_trainer_t* t, const float* hp) {
    if (dp->failed) return -3;
    cudaStream_t compute = (cudaStream_t)bmc_stream(dp->be);
    if (dp->profile) {
        cudaEventRecord(dp->bwd_done_ev, compute);
        cudaEventRecord(dp->all_done_ev, dp->comm_stream);
    }
    cudaEventRecord(dp->done_ev, dp->comm_stream);
    cudaStreamWaitEvent(compute, dp->done_ev, 0);
    const int rc = dp->f32 ? bmc_adamw(dp->be, t->d_master, t->d_wlow, dp->d_grad_f32, BMC_F32, t->d_m, t->d_v, t->P, hp)
                           : bmc_adamw(dp->be, t->d_master, t->d_wlow, dp->d_grad_bf16, BMC_BF16, t->d_m, t->d_v, t->P, hp);
    if (dp->profile && rc == 0 && wait_comm(dp) == 0 && cudaEventSynchronize(dp->bwd_done_ev) == cudaSuccess) {
        float ms = 0.f;
        bool ok = true;
        for (size_t i = 0; i < dp->buckets.size() && ok; ++i) {
            ok = cudaEventElapsedTime(&ms, dp->ready_ev[0], dp->t0_ev[i]) == cudaSuccess;
            if (ok) dp->prof_start_ms[i] += ms;
            ok = ok && cudaEventElapsedTime(&ms, dp->t0_ev[i], dp->t1_ev[i]) == cudaSuccess;
            if (ok) dp->prof_dur_ms[i] += ms;
        }
        if (ok && cudaEventElapsedTime(&ms, dp->bwd_done_ev, dp->all_done_ev) == cudaSuccess) {
            dp->prof_tail_ms += ms;
            ++dp->prof_steps;
        }
        cudaGetLastError();   // a bucket that was not exchanged this step leaves its events unrecorded: not an error of the step
    }
    return rc;
}

float bm_dp_mean_loss(struct bm_dp_s* dp, float local_loss) {
    NcclApi* api = nccl();
    if (!dp || !api) return local_loss;
    if (dp->failed) return -1.0f;
    cudaMemcpyAsync(dp->d_loss_buf, &local_loss, sizeof(float), cudaMemcpyHostToDevice, dp->comm_stream);
    if (api->AllReduce(dp->d_loss_buf, dp->d_loss_buf, 1, ncclFloat32, ncclSum, dp->comm, dp->comm_stream) != ncclSuccess) return -1.0f;
    float sum = 0.f;
    cudaMemcpyAsync(&sum, dp->d_loss_buf, sizeof(float), cudaMemcpyDeviceToHost, dp->comm_stream);
    if (wait_comm(dp) != 0) return -1.0f;   // bounded: a peer that left ends the step with an error, not a hang
    return sum / (float)dp->world;
}

int bmx_trainer_dp_init(bm_trainer_t* t, int rank, int world, const void* nccl_id) {
    if (!t || t->dp) return -1;
    if (world <= 1) return 0;
    const int L = t->model->arch.n_layers;
    std::vector<size_t> layer_begin(L + 1);
    for (int l = 0; l < L; ++l) layer_begin[l] = t->params[9 * l].off;
    layer_begin[L] = t->params[9 * L].off;
    t->dp = bm_dp_create(t->ctx->be, rank, world, nccl_id, t->P, L, layer_begin.data(), t->d_grad, t->dtype == BMC_F32);
    // Three streams (compute, weight-gradient side stream, communication) have only been exercised on one GPU; with the
    // exchange active the weight gradients stay on the compute stream unless BM_DP_SIDE_STREAM=1 asks otherwise.
    if (t->dp && !getenv("BM_DP_SIDE_STREAM")) t->side_stream = 0;
    return t->dp ? 0 : -2;
}

}  // extern "C"
