// placeholder: tcgen05 kernels
#include "faws_internal.cuh"
namespace faws {
bool tc_fwd_supported(const FwdParams&, int) { return false; }
cudaError_t launch_tc_fwd(const FwdParams&, int, cudaStream_t) { return cudaErrorNotSupported; }
bool tc_colsoftmax_supported(const ColSoftmaxParams&, int) { return false; }
cudaError_t launch_tc_colsoftmax(const ColSoftmaxParams&, int, cudaStream_t) { return cudaErrorNotSupported; }
}
