// placeholder, replaced below in this session
#include "common.h"
namespace tf {
int tc_matmul(const float*, bool, const float*, bool, float*, int64_t, int64_t, int64_t, cudaStream_t, int*) { return 0; }
int tc_conv_fwd(ConvPlan*, const float*, const float*, float*, cudaStream_t, int*) { return 0; }
int tc_conv_dgrad(ConvPlan*, const float*, const float*, float*, cudaStream_t, int*) { return 0; }
int tc_conv_wgrad(ConvPlan*, const float*, const float*, float*, cudaStream_t, int*) { return 0; }
}
