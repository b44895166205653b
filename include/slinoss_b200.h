/*
 * slinoss_b200 - C ABI of the B200 (sm_100a) v2x2ssd scan and its mixer hot path.
 *
 * Every entry point
 *   - is `extern "C"`, takes plain device pointers, sizes, a dtype code and a
 *     CUDA stream handle (`cudaStream_t` passed as `void*`), and returns an
 *     `int` status (SL_OK == 0); no exception crosses the boundary;
 *   - launches on the given stream and returns without synchronising;
 *   - allocates nothing: scratch memory is supplied by the caller
 *     (`sl_workspace_bytes` gives the size), so calls are CUDA-graph friendly;
 *   - validates shapes / alignment on the host before any launch.
 *
 * Tensor layouts are the reference's canonical ones
 * (slinoss/ops/v2x2ssd/reference.py:11-28):
 *   U, Y      (batch, heads, T, P)
 *   M         (batch, heads, T, 2)        packed complex (re, im), float32
 *   K         (batch, heads, T, 2, 2)     tap 0 = prev, tap 1 = curr, float32
 *   B, C      (batch, groups, T, 2N)      interleaved (re, im); groups | heads
 *   state     (batch, heads, P, 2N)       float32
 *   B_prev    (batch, groups, 2N),  U_prev (batch, heads, P)
 * All tensors are dense (contiguous) unless a stride argument says otherwise.
 */
#ifndef SLINOSS_B200_H_
#define SLINOSS_B200_H_

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define SL_API __attribute__((visibility("default")))
#else
#define SL_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* status codes */
enum {
  SL_OK = 0,
  SL_ERR_NULL_POINTER = 1,
  SL_ERR_BAD_SHAPE = 2,
  SL_ERR_BAD_ALIGNMENT = 3,
  SL_ERR_UNSUPPORTED = 4,
  SL_ERR_WORKSPACE_TOO_SMALL = 5,
  SL_ERR_LAUNCH_FAILED = 6,
  SL_ERR_DEVICE_TIMEOUT = 7,
  SL_ERR_STATIC_SCRATCH_EXCEEDED = 8
};

/* element types of the "io" tensors (U, B, C, Y, their gradients, gate, ...) */
enum { SL_F32 = 0, SL_BF16 = 1, SL_F16 = 2 };

/* kernel family selector for the scan */
enum {
  SL_PATH_AUTO = 0, /* tensor-core path when the shape allows, else SIMT */
  SL_PATH_SIMT = 1, /* exact float32 sequential recurrence (any dtype in)     */
  SL_PATH_TC = 2    /* tcgen05/TMEM chunked path: bf16 / fp16 operands, P = 64, N = 64 or 128
                       (N = 128 runs as two passes over the column blocks of B and C and needs the
                       SL_WS_SCAN_FWD workspace in the forward pass too)       */
};

/* workspace kinds for sl_workspace_bytes */
enum {
  SL_WS_SCAN_FWD = 0,
  SL_WS_SCAN_BWD = 1,
  SL_WS_SCANPREP_BWD = 2,
  SL_WS_TAIL_BWD = 3,
  SL_WS_SCAN_STATES = 4 /* optional chunk-state buffer handed from forward to backward */
};

/* Library version, major*10000 + minor*100 + patch. */
SL_API int sl_version(void);

/* Number of CUDA kernels this library has launched in this process so far
 * (monotonic; used by benchmarks to report their launch count). */
SL_API unsigned long long sl_kernel_launches(void);

/* SL_OK, or SL_ERR_DEVICE_TIMEOUT when a kernel of this library on the current device gave up a
 * bounded device-side wait since load (or since the last sl_device_status_reset).  Such a kernel
 * returns early, after draining what it had in flight, and leaves its outputs incomplete; the
 * entry points are asynchronous, so the condition surfaces here, not in their return value.
 * Check it where the host synchronises anyway (end of a step, before results are trusted).
 * Synchronises with the device.  The limit is about a second of SM clocks; the environment
 * variable SLINOSS_B200_WAIT_CLOCKS, read at every launch, overrides it (diagnostics only).
 * No reference counterpart (the reference's kernels have no device-side waits). */
SL_API int sl_device_status(void);

/* Returns the site code of the first expired wait (0 = none; it identifies the wait in the kernel
 * source) and clears the record, so that one expiry does not mark every later query.
 * Synchronises with the device. */
SL_API int sl_device_status_reset(void);

/* Static, human readable text of a status code. */
SL_API const char* sl_status_string(int status);

/* The CUDA runtime's text for the error behind the most recent SL_ERR_LAUNCH_FAILED of this
 * process ("no error" if there was none).  Diagnostics only; no reference counterpart. */
SL_API const char* sl_last_cuda_error(void);

/* Scratch bytes a call of the given kind needs for these dimensions
 * (0 when none).  `path` is one of SL_PATH_*.  For SL_WS_SCANPREP_BWD and
 * SL_WS_TAIL_BWD only batch, heads, groups, T, P, N are read. */
SL_API size_t sl_workspace_bytes(int kind, int batch, int heads, int groups, int T, int P, int N,
                          int chunk, int io_dtype, int path);

/*
 * Scan forward.  Replaces slinoss.ops.v2x2ssd.v2x2ssd_cute
 * (slinoss/ops/v2x2ssd/cute/api.py:53-200; semantics = v2x2ssd,
 * slinoss/ops/v2x2ssd/reference.py:1267-1347).
 *   U, B, C, B_prev, U_prev : io_dtype;  Y : y_dtype;  M, K, states : float32.
 *   initial_states, B_prev, U_prev, final_state may be NULL (B_prev and U_prev
 *   together).  T must be >= 1 (T == 0 is answered by the host wrapper).
 *   Precondition of the tensor-core path: every transition is non-zero (|m_t| > 0; the kernels form
 *   log|m| and kp/m and do not check: a zero gives NaN/Inf).  The reference rejects it in its chunked
 *   paths (slinoss/ops/v2x2ssd/reference.py:509-517); SL_PATH_SIMT computes through it.  With bfloat16
 *   operands dM (= S / conj(m)) keeps the 16-bit tolerance down to |m| of about 0.3.
 *   chunk_states (optional, sl_workspace_bytes(SL_WS_SCAN_STATES, ...) bytes): when given
 *   together with final_state, the tensor-core path stores the state at the start of every
 *   64-token chunk there; handing both to sl_v2x2ssd_bwd saves its state pre-sweep.  The
 *   reference recomputes instead (it saves only the inputs); passing NULL does the same.
 */
SL_API int sl_v2x2ssd_fwd(const void* U, const float* M, const float* K, const void* B, const void* C,
                   const float* initial_states, const void* B_prev, const void* U_prev,
                   void* Y, float* final_state, void* chunk_states, int batch, int heads,
                   int groups, int T, int P, int N, int chunk, int io_dtype, int y_dtype, int path,
                   void* workspace, size_t workspace_bytes, void* stream);

/*
 * Scan backward.  Replaces _V2x2SSDCuTeTrainingFn.backward
 * (slinoss/ops/v2x2ssd/cute/autograd.py:148-296).
 *   dY : dy_dtype (NULL = zero);  d_final_state : float32 or NULL.
 *   dU, dB, dC, dB_prev, dU_prev : io_dtype;  dM, dK, d_initial : float32.
 *   d_initial, dB_prev, dU_prev may be NULL.  Grouped dB/dC/dB_prev are summed
 *   over the heads of a group in float32 before the cast.
 *   chunk_states / final_state: both as filled by sl_v2x2ssd_fwd for the same inputs,
 *   or both NULL (then the backward recomputes them).
 */
SL_API int sl_v2x2ssd_bwd(const void* U, const float* M, const float* K, const void* B, const void* C,
                   const float* initial_states, const void* B_prev, const void* U_prev,
                   const void* chunk_states, const float* final_state,
                   const void* dY, const float* d_final_state, void* dU, float* dM, float* dK,
                   void* dB, void* dC, float* d_initial, void* dB_prev, void* dU_prev,
                   int batch, int heads, int groups, int T, int P, int N, int chunk,
                   int io_dtype, int dy_dtype, int path, void* workspace,
                   size_t workspace_bytes, void* stream);

/*
 * Scan backward that allocates nothing and needs no scratch from the caller.
 * (No counterpart in the reference: it exists for hosts of this library that cannot
 * call cudaMalloc - the GPU already belongs to their own memory pool, their hot loop
 * bans allocator calls, or they are inside a stream capture.)
 *
 * Same arguments and results as sl_v2x2ssd_bwd on the exact float32 (SIMT) path,
 * minus chunk / path / workspace.  The scratch is a fixed array of
 * SL_STATIC_SCRATCH_BYTES inside the library image, resident on every GPU that loads
 * the library until the process exits.  Limits and rules:
 *   - a problem needing more scratch (about batch*heads*T*(24*N+8) bytes) is refused
 *     with SL_ERR_STATIC_SCRATCH_EXCEEDED and nothing is launched;
 *   - every call shares the array, so calls whose kernels can overlap on the GPU
 *     race: keep them on one stream or otherwise serialised;
 *   - the array keeps the previous call's contents; each call itself clears the
 *     part it accumulates into, so results never depend on them;
 *   - the first call on each device looks up the array's device address on the host;
 *     issue that first call before starting any stream capture;
 *   - the array used is the CURRENT device's (cudaGetDevice at the time of the call): the stream
 *     passed in must belong to that device;
 *   - if the address lookup fails, the call returns SL_ERR_LAUNCH_FAILED and sl_last_cuda_error()
 *     gives the runtime's reason.
 */
#define SL_STATIC_SCRATCH_BYTES (64u << 20)
SL_API size_t sl_static_scratch_bytes(void);
SL_API int sl_v2x2ssd_bwd_static(const void* U, const float* M, const float* K, const void* B,
                                 const void* C, const float* initial_states, const void* B_prev,
                                 const void* U_prev, const void* dY, const float* d_final_state,
                                 void* dU, float* dM, float* dK, void* dB, void* dC,
                                 float* d_initial, void* dB_prev, void* dU_prev, int batch,
                                 int heads, int groups, int T, int P, int N, int io_dtype,
                                 int dy_dtype, void* stream);

/*
 * One-token decode of the scan (T = 1) over the carried float32 state.
 * Replaces the v2x2ssm(T=1) call of run_reference_decode_step
 * (slinoss/ops/mixer/step.py:201-258) and the scan part of
 * mixer_decode_step_cute (slinoss/ops/v2x2ssd/cute/step.py:224-627).
 *   U (batch,heads,P), B,C (batch,groups,2N), B_prev (batch,groups,2N),
 *   U_prev (batch,heads,P) : io_dtype;  M (batch,heads,2), K (batch,heads,2,2),
 *   state_in/state_out (batch,heads,P,2N) : float32;  Y (batch,heads,P) : y_dtype.
 *   state_out may alias state_in (in-place update).  B_prev/U_prev may be NULL
 *   (zeros).  The caller carries B -> B_prev and U -> U_prev itself.
 */
SL_API int sl_v2x2ssd_decode(const void* U, const float* M, const float* K, const void* B,
                      const void* C, const float* state_in, const void* B_prev,
                      const void* U_prev, void* Y, float* state_out, int batch, int heads,
                      int groups, int P, int N, int io_dtype, int y_dtype, void* stream);

/* Scalar configuration of scan preparation (slinoss/layers/scanprep.py:41-58). */
typedef struct {
  float dt_min, dt_max;
  float alpha_min, alpha_max;
  float theta_init_min, theta_init_max, theta_mod_scale;
  float r_min, r_max;
  float eps;
} sl_scanprep_config;

/*
 * Fused causal depthwise conv1d + bias + SiLU + scan preparation, forward.
 * Replaces cconv1d_fwd (csrc/causal_conv1d/causal_conv1d.cpp:559, through
 * slinoss/ops/mixer/convolution.py:104-173) followed by scanprep_cute
 * (slinoss/ops/scanprep/cute/api.py:88; math of slinoss/layers/scanprep.py:237-283
 * and slinoss/ops/scanprep/parameterization.py:60-107).
 *   value  (batch, T, heads*P), row stride `value_row_stride` elements
 *   conv_weight (heads*P, d_conv), conv_bias (heads*P) : io_dtype; d_conv in 1..4;
 *          conv_weight == NULL skips the convolution (value is only re-laid out)
 *   conv_state_in  (batch, heads*P, d_conv-1) or NULL (zeros) : io_dtype
 *   conv_state_out (batch, heads*P, d_conv-1) or NULL
 *   params (batch, T, heads*3) : io_dtype;  bc (batch, T, groups, 4, N) : io_dtype
 *   dt_bias, alpha_bias, theta_mod_bias, theta_bias, theta_sign (heads) : float32
 *   U out: element (b,h,t,p) at b*u_stride_b + h*u_stride_h + t*u_stride_t + p
 *          ((batch,heads,T,P) dense, or (batch,T,heads*P) for a conv-only call)
 *   M (batch,heads,T,2), K (batch,heads,T,2,2) : float32;  Bo, Co (batch,groups,T,2N).
 *   Any of {params,M,K} / {bc,Bo,Co} / {value,U} may be NULL as a set to skip it.
 */
SL_API int sl_scanprep_conv_fwd(const void* value, int64_t value_row_stride, const void* conv_weight,
                         const void* conv_bias, const void* conv_state_in,
                         void* conv_state_out, int d_conv, const void* params, const void* bc,
                         const float* dt_bias, const float* alpha_bias,
                         const float* theta_mod_bias, const float* theta_bias,
                         const float* theta_sign, const sl_scanprep_config* cfg, void* U,
                         int64_t u_stride_b, int64_t u_stride_h, int64_t u_stride_t, float* M,
                         float* K, void* Bo, void* Co, int batch, int heads, int groups, int T,
                         int P, int N, int io_dtype, void* stream);

/*
 * Backward of sl_scanprep_conv_fwd.  Replaces cconv1d_bwd
 * (csrc/causal_conv1d/causal_conv1d.cpp:560) and the scanprep backward kernels
 * (slinoss/ops/scanprep/cute/kernels/bwd.py:79-915).
 *   dU laid out by the same u_stride_* as U; dM, dK float32; dBo, dCo io_dtype.
 *   Outputs: d_value (batch,T,heads*P) dense io_dtype; d_conv_weight
 *   (heads*P,d_conv), d_conv_bias (heads*P), d_conv_state (batch,heads*P,d_conv-1
 *   or NULL), d_params (batch,T,3*heads), d_bc like bc : io_dtype except the
 *   float32 accumulators d_conv_weight/d_conv_bias/d_*_bias (heads), which this
 *   call ACCUMULATES into (caller zeroes them).
 */
SL_API int sl_scanprep_conv_bwd(const void* value, int64_t value_row_stride, const void* conv_weight,
                         const void* conv_bias, const void* conv_state_in, int d_conv,
                         const void* params, const void* bc, const float* dt_bias,
                         const float* alpha_bias, const float* theta_mod_bias,
                         const float* theta_bias, const float* theta_sign,
                         const sl_scanprep_config* cfg, const void* dU, int64_t u_stride_b,
                         int64_t u_stride_h, int64_t u_stride_t, const float* dM,
                         const float* dK, const void* dBo, const void* dCo, void* d_value,
                         float* d_conv_weight, float* d_conv_bias, void* d_conv_state,
                         void* d_params, void* d_bc, float* d_dt_bias, float* d_alpha_bias,
                         float* d_theta_mod_bias, float* d_theta_bias, int batch, int heads,
                         int groups, int T, int P, int N, int io_dtype, void* stream);

/*
 * Mixer tail, row-wise part: normed = RMSNorm((Y + d_skip*U) * SiLU(gate)) * w.
 * Replaces MixerTailRowwiseFwdFused (slinoss/ops/mixer/cute/fwd.py:64-205; math of
 * slinoss/ops/mixer/tail.py:63-142).  out_proj stays a library GEMM in the caller.
 *   Y, skip (batch,heads,T,P) : io_dtype (skip/d_skip may be NULL together)
 *   gate (batch,T,heads*P) with row stride `gate_row_stride` elements : io_dtype
 *   d_skip (heads) float32;  norm_weight (heads*P) : io_dtype
 *   normed (batch,T,heads*P) dense : io_dtype
 */
SL_API int sl_mixer_tail_fwd(const void* Y, const void* gate, int64_t gate_row_stride,
                      const void* skip, const float* d_skip, const void* norm_weight,
                      float eps, void* normed, int batch, int heads, int T, int P,
                      int io_dtype, void* stream);

/*
 * Backward of sl_mixer_tail_fwd.  Replaces MixerTailRowwiseBwdFused
 * (slinoss/ops/mixer/cute/bwd.py:73-260).
 *   d_normed (batch,T,heads*P) dense.  Outputs dY, d_skip_input (batch,heads,T,P),
 *   d_gate (batch,T,heads*P) dense : io_dtype;  d_d_skip (heads) and
 *   d_norm_weight (heads*P) float32, ACCUMULATED into (caller zeroes them).
 */
SL_API int sl_mixer_tail_bwd(const void* Y, const void* gate, int64_t gate_row_stride,
                      const void* skip, const float* d_skip, const void* norm_weight,
                      float eps, const void* d_normed, void* dY, void* d_gate,
                      void* d_skip_input, float* d_d_skip, float* d_norm_weight, int batch,
                      int heads, int T, int P, int io_dtype, void* stream);

/*
 * One decode token of the whole mixer between in_proj and out_proj, in one launch: causal conv
 * update + bias + SiLU, scan preparation of the token, state update and read-out, skip, gate and
 * RMSNorm.  Replaces the per-token path of SLinOSSMixer.step: run_reference_decode_step
 * (slinoss/ops/mixer/step.py:201-258, 323-429; a chain of torch ops) and mixer_decode_step_cute
 * (slinoss/ops/v2x2ssd/cute/step.py:224-627; fused, but unreachable for mixers with d_skip).
 *   gate, value (batch, heads*P) : io_dtype, row strides in elements (column slices of the in_proj
 *          output are passed where they lie)
 *   params (batch, 3*heads), bc (batch, groups, 4, N) : io_dtype, dense
 *   conv_weight (heads*P, d_conv), conv_bias (heads*P) : io_dtype; conv_weight == NULL skips the conv
 *   conv_state (batch, heads*P, d_conv-1) : io_dtype, the carried inputs, UPDATED IN PLACE
 *   dt_bias ... theta_sign, d_skip (heads) float32 (d_skip may be NULL);  norm_weight (heads*P) io_dtype
 *   state (batch, heads, P, 2N) float32, UPDATED IN PLACE
 *   b_prev_in (batch, groups, 2N) io_dtype or NULL (zeros): the previous token's b
 *   b_prev_out (batch, groups, 2N): this token's b; must not alias b_prev_in (the heads of a group
 *          read one while one of them writes the other)
 *   u_prev (batch, heads, P) : io_dtype, the previous token's u, UPDATED IN PLACE
 *   normed (batch, heads*P) : io_dtype, dense - the input of out_proj
 *   workspace: sl_mixer_decode_step_workspace_bytes(batch, heads, P) bytes that are ZERO before the
 *          first call; every call leaves them zero again (calls on one workspace must not overlap).
 */
SL_API size_t sl_mixer_decode_step_workspace_bytes(int batch, int heads, int P);
SL_API int sl_mixer_decode_step(const void* gate, int64_t gate_row_stride, const void* value,
                                int64_t value_row_stride, const void* params, const void* bc,
                                const void* conv_weight, const void* conv_bias, void* conv_state,
                                int d_conv, const float* dt_bias, const float* alpha_bias,
                                const float* theta_mod_bias, const float* theta_bias,
                                const float* theta_sign, const sl_scanprep_config* cfg,
                                const float* d_skip, const void* norm_weight, float norm_eps,
                                float* state, const void* b_prev_in, void* b_prev_out, void* u_prev,
                                void* normed, void* workspace, size_t workspace_bytes, int batch,
                                int heads, int groups, int P, int N, int io_dtype, void* stream);

/*
 * Row-wise kernels of the block's FFN branch (the two GEMMs stay library calls): RMSNorm and the
 * activation, forward and backward.  With them the branch is rematerialised in the backward pass
 * from its input alone.  They replace FFNRmsNormFwdFused / FFNRmsNormBwdFused
 * (slinoss/ops/block/cute/norm.py:85,173) and FFNActivationFwdFused / FFNActivationBwdFused
 * (slinoss/ops/block/cute/activation.py:78,153) as block_ffn_residual calls them
 * (slinoss/ops/block/training.py:193-354).
 *   x, out, d_out, d_x (rows, C) dense : io_dtype;  weight (C) : io_dtype;  d_weight (C) float32,
 *   ACCUMULATED into (caller zeroes it).  C a multiple of 8 (4 for float32), at most 2048 (1024).
 *   kind 0 = GELU (tanh form): projected, hidden, d_* (rows, hidden_dim);
 *   kind 1 = SwiGLU: projected, d_projected (rows, 2*hidden_dim) = [value | gate], hidden = value*silu(gate).
 */
SL_API int sl_rmsnorm_fwd(const void* x, const void* weight, float eps, void* out, long long rows, int C,
                          int io_dtype, void* stream);
SL_API int sl_rmsnorm_bwd(const void* x, const void* weight, float eps, const void* d_out, void* d_x,
                          float* d_weight, long long rows, int C, int io_dtype, void* stream);
SL_API int sl_ffn_activation_fwd(const void* projected, void* hidden, long long rows, int hidden_dim,
                                 int kind, int io_dtype, void* stream);
SL_API int sl_ffn_activation_bwd(const void* projected, const void* d_hidden, void* d_projected,
                                 long long rows, int hidden_dim, int kind, int io_dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SLINOSS_B200_H_ */
