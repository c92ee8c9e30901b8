// placeholder until the tcgen05 kernel lands
#include "uq_common.cuh"
bool uq_verify_tc_serves(const UQParams&, const UQLaunch&) { return false; }
int uq_verify_tc_splits(const UQParams&, const UQLaunch&) { return 1; }
cudaError_t uq_verify_tc_dispatch(const UQParams&, const UQLaunch&, cudaStream_t) { return cudaErrorInvalidValue; }
