// placeholder, replaced below in this session
#include "common.h"
namespace tf { int dp_sgd_update(float*, const float*, int64_t, float, cudaStream_t) { return 0; } }
extern "C" {
int TfDpInit(int, int, const char*) { return -1; }
int TfDpFlush(void**) { return 0; }
int TfDpShutdown(void) { return 0; }
}
