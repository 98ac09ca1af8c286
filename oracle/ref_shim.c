/* TEST INFRASTRUCTURE — compiled only into oracle/_ref/libbm_ref.so.
 *
 * A few accessors over the reference's internal structs (src/baremetal/model.h:12-60,
 * src/baremetal/trainer.h:13-52) so a test can select the weight precision the way the reference
 * CLI does (tools/cli.c:737-741 writes model->precision directly) and read back per-tensor
 * gradients, weights, optimizer moments and logits after bm_train_step. */
#include "baremetal.h"
#include "baremetal/model.h"
#include "baremetal/trainer.h"
#include "baremetal/scheduler.h"
#include "backend/backend.h"

void bmref_set_precision(bm_model_t* m, int precision) { m->precision = (bm_precision_t)precision; }
void bmref_set_quant(bm_model_t* m, int bits) { m->quant_bits = bits; }
int bmref_n_states(bm_trainer_t* t) { return t->n_opt_states; }
size_t bmref_state_size(bm_trainer_t* t, int i) { return t->opt_states[i].n_params; }
float* bmref_grad(bm_trainer_t* t, int i) {
    backend_buffer_t* b = bmt_scheduler_get_grad_buffer(t->sched, t->opt_states[i].grad_tensor_id);
    return b ? (float*)backend_buffer_map(b) : 0;
}
/* fp32 master when the trainer keeps one, else the fp32 working buffer (as bm_save_state does,
 * src/baremetal/trainer.c:166-168). */
float* bmref_weight(bm_trainer_t* t, int i) {
    bmt_adamw_state_t* st = &t->opt_states[i];
    backend_buffer_t* b = st->master_w ? st->master_w : bmt_scheduler_get_buffer(t->sched, st->grad_tensor_id);
    return b ? (float*)backend_buffer_map(b) : 0;
}
float* bmref_m(bm_trainer_t* t, int i) { return (float*)backend_buffer_map(t->opt_states[i].m); }
float* bmref_v(bm_trainer_t* t, int i) { return (float*)backend_buffer_map(t->opt_states[i].v); }
float* bmref_logits(bm_trainer_t* t) {
    backend_buffer_t* b = bmt_scheduler_get_buffer(t->sched, t->t_logits_id);
    return b ? (float*)backend_buffer_map(b) : 0;
}
float* bmref_activation(bm_trainer_t* t, int tensor_id) {
    backend_buffer_t* b = bmt_scheduler_get_buffer(t->sched, tensor_id);
    return b ? (float*)backend_buffer_map(b) : 0;
}
