// placeholder until the tcgen05 kernel lands
#include "vb_common.cuh"
namespace vb {
bool gemm_tc_supported(int, const float *, const float *, long long, long long, long long, const Epilogue &) { return false; }
cudaError_t launch_gemm_tc(int, const float *, const float *, long long, long long, long long, const Epilogue &,
                           unsigned int *, cudaStream_t) { return cudaErrorNotSupported; }
}  // namespace vb
