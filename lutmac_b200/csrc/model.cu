// placeholder until the decode step lands
#include "common.cuh"
extern "C" {
#define STUB { lmb::set_last_error("not implemented yet"); return LMB_ERR_STATE; }
int lmb_model_create(lmb_ctx *, const lmb_model_config *, lmb_model **) STUB
int lmb_model_destroy(lmb_model *) STUB
int lmb_model_set_weight(lmb_model *, int, int, int, int, const void *, size_t, size_t) STUB
int lmb_model_set_vector(lmb_model *, int, int, const float *, size_t) STUB
int lmb_model_forward(lmb_model *, const int *, const size_t *, size_t, float *) STUB
int lmb_model_logits_dev(lmb_model *, const float **) STUB
int lmb_model_reset(lmb_model *) STUB
int lmb_model_kv_export(lmb_model *, size_t, float *) STUB
int lmb_model_kv_import(lmb_model *, size_t, const float *) STUB
int lmb_model_step_bytes(lmb_model *, size_t, uint64_t *) STUB
int lmb_tp_unique_id(void *) STUB
int lmb_tp_init(lmb_ctx *, const void *, int, int) STUB
int lmb_tp_destroy(lmb_ctx *) STUB
int lmb_allreduce_sum(lmb_ctx *, float *, size_t) STUB
int lmb_allgather(lmb_ctx *, const float *, float *, size_t) STUB
}
