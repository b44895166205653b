// Scan backward for callers that must not allocate device memory.
//
// Some hosts of this library cannot hand it a scratch buffer: an inference server
// that has already given the whole GPU to its own memory pool, a real-time loop that
// forbids allocator calls on its hot path, or code running between
// cudaStreamBeginCapture / EndCapture where cudaMalloc is illegal.  For them this
// file offers the exact float32 (SIMT) backward of the scan with its scratch held in
// a fixed array that is part of the library image.
//
// Consequences the caller has to know:
//  * the array (SL_STATIC_SCRATCH_BYTES) is resident on every GPU that loads the
//    library, from load until the process exits;
//  * problems whose scratch need exceeds it are refused with
//    SL_ERR_STATIC_SCRATCH_EXCEEDED - nothing is launched;
//  * all calls share the one array: two calls whose kernels overlap on the GPU
//    (different streams, different host threads) race on it.  Serialise them;
//  * the array keeps whatever the previous call left.  Everything a call reads from it
//    is written by that same call first, and the part that is accumulated into is
//    cleared by the call itself, so stale contents never leak into a result;
//  * the first call on each device resolves the array's device address (a one-time
//    host-side set-up).  Make that first call outside of any stream capture.
#include <mutex>

#include "common.cuh"

namespace {

// File-scope device array.  In host code this name is only a handle for the runtime's
// symbol table, never a device address: it must go through cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char g_static_scratch[SL_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
void* g_scratch_ptr[kMaxDevices] = {};
std::mutex g_setup_mutex;

// Device address of the array on the current device (resolved once per device).
int scratch_address(void** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return SL_ERR_LAUNCH_FAILED;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess || p == nullptr) {   // e.g. the module's 64 MiB array could not be placed on this device
      cudaGetLastError();
      sl::note_cuda_error(e != cudaSuccess ? (int)e : (int)cudaErrorInvalidSymbol);   // for sl_last_cuda_error()
      return SL_ERR_LAUNCH_FAILED;
    }
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  return SL_OK;
}

}  // namespace

extern "C" size_t sl_static_scratch_bytes(void) { return SL_STATIC_SCRATCH_BYTES; }

extern "C" int sl_v2x2ssd_bwd_static(const void* U, const float* M, const float* K, const void* B,
                                     const void* C, const float* initial_states,
                                     const void* B_prev, const void* U_prev, const void* dY,
                                     const float* d_final_state, void* dU, float* dM, float* dK,
                                     void* dB, void* dC, float* d_initial, void* dB_prev,
                                     void* dU_prev, int batch, int heads, int groups, int T,
                                     int P, int N, int io_dtype, int dy_dtype, void* stream) {
  using namespace sl;
  if (!U || !M || !K || !B || !C || !dU || !dM || !dK || !dB || !dC) return SL_ERR_NULL_POINTER;
  if ((B_prev == nullptr) != (U_prev == nullptr)) return SL_ERR_NULL_POINTER;
  if (batch < 1 || heads < 1 || groups < 1 || heads % groups || T < 1 || P < 1 || N < 1)
    return SL_ERR_BAD_SHAPE;
  if (!dtype_ok(io_dtype) || !dtype_ok(dy_dtype)) return SL_ERR_UNSUPPORTED;
  if (!aligned(M, 8) || !aligned(K, 16)) return SL_ERR_BAD_ALIGNMENT;
  const ScanDims d{batch, heads, groups, T, P, N, 64};
  if (!scan_simt_supported(d)) return SL_ERR_UNSUPPORTED;
  const size_t need = scan_simt_bwd_workspace(d);
  if (need > (size_t)SL_STATIC_SCRATCH_BYTES) return SL_ERR_STATIC_SCRATCH_EXCEEDED;
  void* scratch = nullptr;
  if (int e = scratch_address(&scratch)) return e;
  return scan_simt_bwd(U, M, K, B, C, initial_states, B_prev, U_prev, dY, d_final_state, dU, dM,
                       dK, dB, dC, d_initial, dB_prev, dU_prev, d, io_dtype, dy_dtype, scratch,
                       SL_STATIC_SCRATCH_BYTES, reinterpret_cast<cudaStream_t>(stream));
}
