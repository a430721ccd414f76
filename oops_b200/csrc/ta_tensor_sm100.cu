// placeholder until the tcgen05 kernels land
#include "ta_internal.h"
namespace oops_ta {
bool tensor_forward_applies(const oops_ta_problem&) { return false; }
bool tensor_backward_applies(const oops_ta_problem&, const oops_ta_grads*) { return false; }
uint64_t tensor_forward_workspace(const oops_ta_problem&) { return 0; }
uint64_t tensor_backward_workspace(const oops_ta_problem&, const oops_ta_grads&) { return 0; }
int tensor_forward(const oops_ta_problem&, const oops_ta_pair&, float*, cudaStream_t) { return OOPS_TA_UNSUPPORTED_LAYOUT; }
int tensor_backward(const oops_ta_problem&, const oops_ta_pair&, const oops_ta_pair&, const float*, const oops_ta_grads&, cudaStream_t) { return OOPS_TA_UNSUPPORTED_LAYOUT; }
}
