// tcgen05 / TMEM chunked scan path (placeholder until the kernels land).
#include "common.cuh"

namespace sl {
bool scan_tc_supported(const ScanDims&, int) { return false; }
size_t scan_tc_fwd_workspace(const ScanDims&) { return 0; }
size_t scan_tc_bwd_workspace(const ScanDims&) { return 0; }
int scan_tc_fwd(const void*, const float*, const float*, const void*, const void*, const float*,
                const void*, const void*, void*, float*, const ScanDims&, int, int, void*,
                size_t, cudaStream_t) {
  return SL_ERR_UNSUPPORTED;
}
int scan_tc_bwd(const void*, const float*, const float*, const void*, const void*, const float*,
                const void*, const void*, const void*, const float*, void*, float*, float*,
                void*, void*, float*, void*, void*, const ScanDims&, int, int, void*, size_t,
                cudaStream_t) {
  return SL_ERR_UNSUPPORTED;
}
}  // namespace sl
