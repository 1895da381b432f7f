// Tensor-core attention (placeholder plan object until the tcgen05 kernel lands).
#include "common.cuh"

struct AttnTcPlan { int unused; };
bool attention_tc_supported(const fe2o3_flash_attention_v1_args *) { return false; }
int32_t attention_tc_plan(fe2o3_ctx *, const fe2o3_flash_attention_v1_args *, AttnTcPlan **) { return FE2O3_ERR_UNSUPPORTED_SHAPE; }
int32_t attention_tc_launch(const AttnTcPlan *, cudaStream_t) { return FE2O3_ERR_UNSUPPORTED_SHAPE; }
void attention_tc_geometry(const AttnTcPlan *, fe2o3_geometry *) {}
void attention_tc_free(AttnTcPlan *) {}
