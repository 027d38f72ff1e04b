// tcgen05 backward kernels of attention() (sm_100a).
#include "faws_internal.cuh"
#include "faws_tc_host.cuh"
#include "faws_tc_ptx.cuh"

namespace faws {

bool tc_bwd_supported(const BwdParams& p, int dtype) {
  (void)p;
  (void)dtype;
  return false;
}

cudaError_t launch_tc_bwd(const BwdParams& p, int dtype, cudaStream_t s) {
  (void)p;
  (void)dtype;
  (void)s;
  return cudaErrorNotSupported;
}

}  // namespace faws
