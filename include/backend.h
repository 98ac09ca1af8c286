/* The reference's internal backend ABI, served by the CUDA backend of this library.
 *
 * Same 22 functions, argument meaning and failure values as the reference's src/backend/backend.h:17-67, so that its C11 host code
 * (src/baremetal/scheduler.c, trainer.c, session.c), its CLI self-tests (tools/cli.c:93-257) and its kernel tests (test/ *_test.c)
 * link against libbaremetal_b200.so in place of the Metal backend. The handle structs repeat the field order of the reference's
 * src/backend/metal/device.h:9-44, because its api.c reads backend_ctx_s::supports_bf16 directly (src/baremetal/api.c:29).
 *
 * Contract kept (details in bare.metal_b200/csrc/backend_compat.cu):
 *   - buffers are host-visible: map() returns a pointer that is valid for the buffer's life and reflects all GPU work enqueued
 *     before the call; host writes are seen by the next dispatch; unmap() is optional;
 *   - dispatches of an encoder execute in order; backend_kernel_dispatch() blocks;
 *   - scalar parameters are buffers in the per-kernel slot order of the reference's shaders; offsets[] are byte offsets;
 *   - the grid is accepted and ignored (embedding_backward alone derives its token count from it: grid = T * D);
 *   - backend_kernel_create() returns NULL for a name that is not served.
 * Names served (the training path): matmul_forward_naive / _fp32_tiled / _bf16 / _bf16_tiled / _bf16_tiled64,
 * matmul_backward_inp / _fp32_tiled / _bf16 / _bf16_tiled, matmul_backward_w / _w_tiled, rmsnorm_forward, rmsnorm_backward_x / _w,
 * rope_forward_seq, rope_backward_seq, attention_forward_seq / _seq_masked / _train_tiled, attention_backward / _masked / _tiled,
 * add_forward, add_backward, swiglu_forward, swiglu_backward, zero_buffer, xent_backward / _masked, embedding_backward, adamw_step.
 */
#ifndef BM_B200_BACKEND_H
#define BM_B200_BACKEND_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct backend_ctx_s backend_ctx_t;
typedef struct backend_buffer_s backend_buffer_t;
typedef struct backend_kernel_s backend_kernel_t;
typedef struct backend_encoder_s backend_encoder_t;

/* field order = src/backend/metal/device.h:9-44 of the reference */
struct backend_ctx_s {
    void* device;   /* here: the backend's own state */
    void* queue;
    void* library;
    int supports_bf16;
    size_t allocated_bytes, peak_allocated_bytes;
    int dev_max_threads_per_tg;
    size_t dev_max_threadgroup_mem, dev_max_buffer_bytes, dev_recommended_working_set;
    int dev_has_unified_memory;
    double gpu_busy_ms;
    uint64_t cmd_buffers;
};
struct backend_buffer_s {
    void* buffer;   /* host pointer == device pointer (managed memory) */
    size_t size;
    struct backend_ctx_s* ctx;
};
struct backend_kernel_s {
    void* pipeline_state;
};
struct backend_encoder_s {
    void* command_buffer;
    void* encoder;
    struct backend_ctx_s* ctx;
};

typedef struct {
    int max_threads_per_threadgroup;
    size_t max_threadgroup_memory;
    size_t max_buffer_bytes;
    size_t recommended_max_working_set;
    int has_unified_memory;
} backend_device_info_t;

/* context (backend.h:17-20, 30, 32-34) */
backend_ctx_t* backend_create(void);
void backend_destroy(backend_ctx_t* ctx);
size_t backend_get_allocated_memory(backend_ctx_t* ctx);
size_t backend_get_peak_allocated_memory(backend_ctx_t* ctx);
void backend_get_device_info(backend_ctx_t* ctx, backend_device_info_t* out);
double backend_get_gpu_busy_ms(backend_ctx_t* ctx);
uint64_t backend_get_command_buffers(backend_ctx_t* ctx);
void backend_reset_gpu_timing(backend_ctx_t* ctx);

/* buffers (backend.h:40-44): alloc(size 0) returns NULL */
backend_buffer_t* backend_buffer_alloc(backend_ctx_t* ctx, size_t size);
void backend_buffer_free(backend_buffer_t* buf);
void* backend_buffer_map(backend_buffer_t* buf);
void backend_buffer_unmap(backend_buffer_t* buf);
size_t backend_buffer_size(backend_buffer_t* buf);

/* kernels by name (backend.h:46-47) and the blocking single dispatch (backend.h:49-56); 0 / -1 */
backend_kernel_t* backend_kernel_create(backend_ctx_t* ctx, const char* name);
void backend_kernel_destroy(backend_kernel_t* kernel);
int backend_kernel_dispatch(backend_ctx_t* ctx, backend_kernel_t* kernel, backend_buffer_t* buffers[], size_t offsets[], int num_buffers,
                            int grid_x, int grid_y, int grid_z, int tg_x, int tg_y, int tg_z);
void backend_synchronize(backend_ctx_t* ctx);

/* encoders (backend.h:36-38, 58-67): wait and wait_timed consume the encoder; wait_timed returns its GPU time in ms */
backend_encoder_t* backend_encode_begin(backend_ctx_t* ctx);
int backend_encode_dispatch(backend_encoder_t* enc, backend_kernel_t* kernel, backend_buffer_t* buffers[], size_t offsets[],
                            int num_buffers, int grid_x, int grid_y, int grid_z, int tg_x, int tg_y, int tg_z);
void backend_encode_commit(backend_encoder_t* enc);
void backend_encode_wait(backend_encoder_t* enc);
double backend_encode_wait_timed(backend_encoder_t* enc);

#ifdef __cplusplus
}
#endif
#endif
