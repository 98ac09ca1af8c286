/* Data-parallel gradient exchange used by the trainer (implemented in csrc/dp_nccl.cu).
 * The reference has no counterpart: it drives one device (src/backend/metal/device.m:20). */
#ifndef BM_DP_H
#define BM_DP_H
#include "bm_internal.h"

#ifdef __cplusplus
extern "C" {
#endif

struct bm_dp_s;
/* bucket boundaries are given as element offsets into the flat parameter order */
struct bm_dp_s* bm_dp_create(bmc_ctx_t* be, int rank, int world, const void* nccl_id, size_t n_params_total, int n_layers,
                             const size_t* layer_begin /* [n_layers + 1] */, float* d_grad_f32, int grads_f32);
void bm_dp_destroy(struct bm_dp_s* dp);
int  bm_dp_world(struct bm_dp_s* dp);
void bm_dp_begin_window(struct bm_dp_s* dp);
void bm_dp_set_last_microstep(struct bm_dp_s* dp, int is_last);
/* layer == n_layers: final norm gradient done; 0 <= layer < n_layers: that layer's gradients done;
 * layer == -1: embedding gradient done (everything is). On the last micro-step of a window this launches the
 * bf16 cast + all-reduce of every bucket that has become complete, on the communication stream. */
int  bm_dp_bucket_ready(struct bm_dp_s* dp, int layer);
/* all buckets now (a window cut short by bm_train_flush); collective: every rank calls it */
int  bm_dp_reduce_all(struct bm_dp_s* dp);
/* waits (on the device) for all buckets, then runs AdamW from the reduced gradients (bf16, or fp32 for an fp32 trainer) */
int  bm_dp_adamw(struct bm_dp_s* dp, bm_trainer_t* t, const float* hp);
float bm_dp_mean_loss(struct bm_dp_s* dp, float local_loss);

#ifdef __cplusplus
}
#endif
#endif
