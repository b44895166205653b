// Shared device/host helpers for the slinoss_b200 kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/slinoss_b200.h"

namespace sl {

// ---- element access in float32 -------------------------------------------------
__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}
template <> __device__ __forceinline__ __half from_f32<__half>(float v) {
  // saturate to the finite range like the reference's output cast
  v = fminf(fmaxf(v, -65504.f), 65504.f);
  return __float2half_rn(v);
}

// Pairs: packed conversions (one F2FP instruction on the ALU pipe) instead of two scalar ones,
// which run on the much narrower XU pipe.
template <typename T> __device__ __forceinline__ uint32_t pack_pair(float a, float b);
template <> __device__ __forceinline__ uint32_t pack_pair<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <> __device__ __forceinline__ uint32_t pack_pair<__half>(float a, float b) {
  a = fminf(fmaxf(a, -65504.f), 65504.f); b = fminf(fmaxf(b, -65504.f), 65504.f);   // saturate like from_f32
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <typename T> __device__ __forceinline__ float2 unpack_pair(uint32_t v);
template <> __device__ __forceinline__ float2 unpack_pair<__nv_bfloat16>(uint32_t v) {
  return make_float2(__uint_as_float(v << 16), __uint_as_float(v & 0xffff0000u));
}
template <> __device__ __forceinline__ float2 unpack_pair<__half>(uint32_t v) {
  return __half22float2(*reinterpret_cast<__half2*>(&v));
}
// a, b rounded to the io dtype and back (the roundings the reference makes between its steps)
template <typename T> __device__ __forceinline__ void round_pair(float& a, float& b) {
  if constexpr (sizeof(T) == 2) {
    const float2 r = unpack_pair<T>(pack_pair<T>(a, b));
    a = r.x; b = r.y;
  }
}

// 16-byte vectors of io elements: 4 floats or 8 16-bit values, handled as floats
template <typename T> struct Vec16 { static constexpr int N = 16 / (int)sizeof(T); };
template <typename T>
__device__ __forceinline__ void unpack16(const uint4& r, float (&v)[Vec16<T>::N]);
template <typename T>
__device__ __forceinline__ void load16(const T* p, float (&v)[Vec16<T>::N]) {
  unpack16<T>(*reinterpret_cast<const uint4*>(p), v);
}
template <typename T>
__device__ __forceinline__ void unpack16(const uint4& r, float (&v)[Vec16<T>::N]) {
  if constexpr (sizeof(T) == 2) {
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = unpack_pair<T>(w[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
  } else {
    v[0] = __uint_as_float(r.x); v[1] = __uint_as_float(r.y); v[2] = __uint_as_float(r.z); v[3] = __uint_as_float(r.w);
  }
}
template <typename T>
__device__ __forceinline__ void store16(T* p, const float (&v)[Vec16<T>::N]) {
  if constexpr (sizeof(T) == 2) {
    *reinterpret_cast<uint4*>(p) = make_uint4(pack_pair<T>(v[0], v[1]), pack_pair<T>(v[2], v[3]),
                                              pack_pair<T>(v[4], v[5]), pack_pair<T>(v[6], v[7]));
  } else {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
}

struct cf {  // complex float
  float re, im;
};
__device__ __forceinline__ cf cmul(cf a, cf b) {
  return {a.re * b.re - a.im * b.im, a.re * b.im + a.im * b.re};
}
__device__ __forceinline__ cf cmul_conj_a(cf a, cf b) {  // conj(a) * b
  return {a.re * b.re + a.im * b.im, a.re * b.im - a.im * b.re};
}
__device__ __forceinline__ cf cadd(cf a, cf b) { return {a.re + b.re, a.im + b.im}; }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// (__fdividef: 2 ulp, and 0 for a denominator beyond 2^126, which is the right limit here)
__device__ __forceinline__ float silu_f(float x) { return __fdividef(x, 1.f + __expf(-x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return __fdividef(1.f, 1.f + __expf(-x)); }

// ---- host side -----------------------------------------------------------------
inline size_t dtype_size(int dt) { return dt == SL_F32 ? 4 : 2; }
inline bool dtype_ok(int dt) { return dt == SL_F32 || dt == SL_BF16 || dt == SL_F16; }
inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }
inline size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// process-wide count of kernels this library has launched (see sl_kernel_launches)
void note_launches(int n);

// remembers the CUDA error behind the last SL_ERR_LAUNCH_FAILED (see sl_last_cuda_error)
void note_cuda_error(int code);

inline int launch_status() {
  const cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) return SL_OK;
  note_cuda_error((int)e);
  return SL_ERR_LAUNCH_FAILED;
}

// Dispatch a callable templated on the io element type.
#define SL_DISPATCH_DTYPE(dt, T, ...)                         \
  do {                                                        \
    if ((dt) == SL_F32) {                                     \
      using T = float;                                        \
      __VA_ARGS__;                                            \
    } else if ((dt) == SL_BF16) {                             \
      using T = __nv_bfloat16;                                \
      __VA_ARGS__;                                            \
    } else {                                                  \
      using T = __half;                                       \
      __VA_ARGS__;                                            \
    }                                                         \
  } while (0)

// ---- internal entry points implemented in the other translation units ----------
struct ScanDims {
  int batch, heads, groups, T, P, N, chunk;
};

int scan_simt_fwd(const void* U, const float* M, const float* K, const void* B, const void* C,
                  const float* z0, const void* Bprev, const void* Uprev, void* Y, float* zfinal,
                  const ScanDims& d, int io_dtype, int y_dtype, cudaStream_t st);
size_t scan_simt_bwd_workspace(const ScanDims& d);
int scan_simt_bwd(const void* U, const float* M, const float* K, const void* B, const void* C,
                  const float* z0, const void* Bprev, const void* Uprev, const void* dY,
                  const float* dfinal, void* dU, float* dM, float* dK, void* dB, void* dC,
                  float* dinit, void* dBprev, void* dUprev, const ScanDims& d, int io_dtype,
                  int dy_dtype, void* ws, size_t ws_bytes, cudaStream_t st);
bool scan_simt_supported(const ScanDims& d);

}  // namespace sl
