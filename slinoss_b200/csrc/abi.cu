// C-ABI entry points of the scan (argument validation and path selection).
#include <atomic>

#include "common.cuh"

namespace sl {

static std::atomic<unsigned long long> g_launches{0};
void note_launches(int n) { g_launches.fetch_add((unsigned long long)n, std::memory_order_relaxed); }
static std::atomic<int> g_cuda_error{0};
void note_cuda_error(int code) { g_cuda_error.store(code, std::memory_order_relaxed); }

// Implemented in scan_tc.cu (tcgen05 / TMEM chunked path).
bool scan_tc_supported(const ScanDims& d, int io_dtype);
size_t scan_tc_fwd_workspace(const ScanDims& d);
size_t scan_tc_bwd_workspace(const ScanDims& d);
size_t scan_tc_states_bytes(const ScanDims& d);
int scan_tc_fwd(const void* U, const float* M, const float* K, const void* B, const void* C,
                const float* z0, const void* Bprev, const void* Uprev, void* Y, float* zfinal,
                void* states_out, const ScanDims& d, int io_dtype, int y_dtype, void* ws,
                size_t ws_bytes, cudaStream_t st);
int scan_tc_bwd(const void* U, const float* M, const float* K, const void* B, const void* C,
                const float* z0, const void* Bprev, const void* Uprev, const void* states_in,
                const float* zfinal_in, const void* dY,
                const float* dfinal, void* dU, float* dM, float* dK, void* dB, void* dC,
                float* dinit, void* dBprev, void* dUprev, const ScanDims& d, int io_dtype,
                int dy_dtype, void* ws, size_t ws_bytes, cudaStream_t st);

int scan_tc_device_status(bool reset);

namespace {

int check_scan(const void* U, const float* M, const float* K, const void* B, const void* C,
               const void* Bprev, const void* Uprev, const ScanDims& d, int io_dtype) {
  if (!U || !M || !K || !B || !C) return SL_ERR_NULL_POINTER;
  if ((Bprev == nullptr) != (Uprev == nullptr)) return SL_ERR_NULL_POINTER;
  if (d.batch < 1 || d.heads < 1 || d.groups < 1 || d.heads % d.groups || d.T < 1 || d.P < 1 ||
      d.N < 1 || d.chunk < 1)
    return SL_ERR_BAD_SHAPE;
  if (!dtype_ok(io_dtype)) return SL_ERR_UNSUPPORTED;
  if (!aligned(M, 8) || !aligned(K, 16) || !aligned(U, 16) || !aligned(B, 16) || !aligned(C, 16))
    return SL_ERR_BAD_ALIGNMENT;
  return SL_OK;
}

bool use_tc(int path, const ScanDims& d, int io_dtype) {
  if (path == SL_PATH_SIMT) return false;
  return scan_tc_supported(d, io_dtype);
}

}  // namespace
}  // namespace sl

extern "C" int sl_version(void) { return 100; }

extern "C" unsigned long long sl_kernel_launches(void) {
  return sl::g_launches.load(std::memory_order_relaxed);
}

extern "C" int sl_device_status(void) {
  return sl::scan_tc_device_status(false) != 0 ? SL_ERR_DEVICE_TIMEOUT : SL_OK;
}

extern "C" int sl_device_status_reset(void) { return sl::scan_tc_device_status(true); }

extern "C" const char* sl_last_cuda_error(void) {
  return cudaGetErrorString((cudaError_t)sl::g_cuda_error.load(std::memory_order_relaxed));
}

extern "C" const char* sl_status_string(int status) {
  switch (status) {
    case SL_OK: return "ok";
    case SL_ERR_NULL_POINTER: return "a required pointer is NULL (or only one of a pair was given)";
    case SL_ERR_BAD_SHAPE: return "bad shape";
    case SL_ERR_BAD_ALIGNMENT: return "pointer not aligned as required";
    case SL_ERR_UNSUPPORTED: return "unsupported dtype, size or path for this kernel";
    case SL_ERR_WORKSPACE_TOO_SMALL: return "workspace missing or too small";
    case SL_ERR_LAUNCH_FAILED: return "CUDA launch failed";
    case SL_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait gave up";
    case SL_ERR_STATIC_SCRATCH_EXCEEDED:
      return "problem needs more scratch than the built-in static array holds";
    default: return "unknown status";
  }
}

extern "C" size_t sl_workspace_bytes(int kind, int batch, int heads, int groups, int T, int P,
                                     int N, int chunk, int io_dtype, int path) {
  using namespace sl;
  const ScanDims d{batch, heads, groups, T, P, N, chunk};
  if (batch < 1 || heads < 1 || groups < 1 || T < 1 || P < 1 || N < 1) return 0;
  switch (kind) {
    case SL_WS_SCAN_FWD:
      return use_tc(path, d, io_dtype) ? scan_tc_fwd_workspace(d) : 0;
    case SL_WS_SCAN_BWD:
      return use_tc(path, d, io_dtype) ? scan_tc_bwd_workspace(d) : scan_simt_bwd_workspace(d);
    case SL_WS_SCAN_STATES:
      return use_tc(path, d, io_dtype) ? scan_tc_states_bytes(d) : 0;
    default:
      return 0;
  }
}

extern "C" int sl_v2x2ssd_fwd(const void* U, const float* M, const float* K, const void* B,
                              const void* C, const float* initial_states, const void* B_prev,
                              const void* U_prev, void* Y, float* final_state,
                              void* chunk_states, int batch, int heads, int groups, int T, int P,
                              int N, int chunk, int io_dtype, int y_dtype, int path,
                              void* workspace, size_t workspace_bytes, void* stream) {
  using namespace sl;
  const ScanDims d{batch, heads, groups, T, P, N, chunk};
  if (int e = check_scan(U, M, K, B, C, B_prev, U_prev, d, io_dtype)) return e;
  if (!Y) return SL_ERR_NULL_POINTER;
  if (!dtype_ok(y_dtype)) return SL_ERR_UNSUPPORTED;
  if (!aligned(Y, 16) || (chunk_states && !aligned(chunk_states, 16))) return SL_ERR_BAD_ALIGNMENT;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (path == SL_PATH_TC && !scan_tc_supported(d, io_dtype)) return SL_ERR_UNSUPPORTED;
  if (use_tc(path, d, io_dtype))
    return scan_tc_fwd(U, M, K, B, C, initial_states, B_prev, U_prev, Y, final_state,
                       final_state ? chunk_states : nullptr, d, io_dtype, y_dtype, workspace,
                       workspace_bytes, st);
  return scan_simt_fwd(U, M, K, B, C, initial_states, B_prev, U_prev, Y, final_state, d,
                       io_dtype, y_dtype, st);
}

extern "C" int sl_v2x2ssd_bwd(const void* U, const float* M, const float* K, const void* B,
                              const void* C, const float* initial_states, const void* B_prev,
                              const void* U_prev, const void* chunk_states,
                              const float* final_state, const void* dY,
                              const float* d_final_state, void* dU, float* dM, float* dK,
                              void* dB, void* dC,
                              float* d_initial, void* dB_prev, void* dU_prev, int batch,
                              int heads, int groups, int T, int P, int N, int chunk,
                              int io_dtype, int dy_dtype, int path, void* workspace,
                              size_t workspace_bytes, void* stream) {
  using namespace sl;
  const ScanDims d{batch, heads, groups, T, P, N, chunk};
  if (int e = check_scan(U, M, K, B, C, B_prev, U_prev, d, io_dtype)) return e;
  if (!dU || !dM || !dK || !dB || !dC) return SL_ERR_NULL_POINTER;
  if (!aligned(dU, 16) || !aligned(dB, 16) || !aligned(dC, 16) || (dY && !aligned(dY, 16)))
    return SL_ERR_BAD_ALIGNMENT;
  if (!dtype_ok(dy_dtype)) return SL_ERR_UNSUPPORTED;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (path == SL_PATH_TC && !scan_tc_supported(d, io_dtype)) return SL_ERR_UNSUPPORTED;
  if (use_tc(path, d, io_dtype))
    return scan_tc_bwd(U, M, K, B, C, initial_states, B_prev, U_prev,
                       final_state ? chunk_states : nullptr, chunk_states ? final_state : nullptr, dY,
                       d_final_state, dU, dM,
                       dK, dB, dC, d_initial, dB_prev, dU_prev, d, io_dtype, dy_dtype, workspace,
                       workspace_bytes, st);
  return scan_simt_bwd(U, M, K, B, C, initial_states, B_prev, U_prev, dY, d_final_state, dU, dM,
                       dK, dB, dC, d_initial, dB_prev, dU_prev, d, io_dtype, dy_dtype, workspace,
                       workspace_bytes, st);
}
