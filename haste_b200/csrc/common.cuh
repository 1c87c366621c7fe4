// Shared device/host helpers for the haste_b200 kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/haste_b200.h"

namespace hb {

// ---------------------------------------------------------------------------
// Status handling: every CUDA call is checked and turned into a C-ABI status.
// ---------------------------------------------------------------------------
void set_last_error(const char* fmt, ...);

#define HB_CUDA_OK(expr)                                                          \
  do {                                                                            \
    cudaError_t _e = (expr);                                                      \
    if (_e != cudaSuccess) {                                                      \
      ::hb::set_last_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), \
                           __FILE__, __LINE__);                                   \
      return HASTE_B200_ERR_CUDA;                                                 \
    }                                                                             \
  } while (0)

#define HB_LAUNCH_OK()                                                           \
  do {                                                                           \
    cudaError_t _e = cudaGetLastError();                                         \
    if (_e != cudaSuccess) {                                                     \
      ::hb::set_last_error("kernel launch failed: %s (%s:%d)",                   \
                           cudaGetErrorString(_e), __FILE__, __LINE__);          \
      return HASTE_B200_ERR_CUDA;                                                \
    }                                                                            \
  } while (0)

#define HB_REQUIRE(cond, msg)                                        \
  do {                                                               \
    if (!(cond)) {                                                   \
      ::hb::set_last_error("invalid argument: %s (%s)", msg, #cond); \
      return HASTE_B200_ERR_INVALID;                                 \
    }                                                                \
  } while (0)

#define HB_TRY(expr)                          \
  do {                                        \
    int _s = (expr);                          \
    if (_s != HASTE_B200_OK) return _s;       \
  } while (0)

// ---------------------------------------------------------------------------
// Storage types: fp32, or bf16 storage with all arithmetic in fp32.
// ---------------------------------------------------------------------------
template <typename T> struct is_bf16 { static constexpr bool value = false; };
template <> struct is_bf16<__nv_bfloat16> { static constexpr bool value = true; };

__device__ __forceinline__ float ld(const float* p) { return *p; }
__device__ __forceinline__ float ld(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ float ld(const __half* p) { return __half2float(*p); }
__device__ __forceinline__ void st(float* p, float v) { *p = v; }
__device__ __forceinline__ void st(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
__device__ __forceinline__ void st(__half* p, float v) { *p = __float2half_rn(v); }

// The value as the storage type will hold it (what a later load returns).
template <typename T> __device__ __forceinline__ float round_to_storage(float v) { return v; }
template <> __device__ __forceinline__ float round_to_storage<__nv_bfloat16>(float v) {
  return __bfloat162float(__float2bfloat16_rn(v));
}
template <> __device__ __forceinline__ float round_to_storage<__half>(float v) {
  return __half2float(__float2half_rn(v));
}

// ---------------------------------------------------------------------------
// Gate math (accurate expf/tanhf: the fp32 parity bar is 1e-4 over long chains).
// Derivatives are taken from the activation outputs, as in the reference
// (lib/inline_ops.h:20-42).
// ---------------------------------------------------------------------------
__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float d_sigmoid(float s) { return s * (1.0f - s); }
__device__ __forceinline__ float d_tanh(float t) { return 1.0f - t * t; }

// Zoneout on the new state (lib/lstm_forward_gpu.cu.cc:77-83).
//   training : h' = (h' - h) * mask + h
//   inference: h' = p * h + (1 - p) * h'
template <bool Training>
__device__ __forceinline__ float zoneout(float h_new, float h_prev, float prob, float mask) {
  if (Training) return (h_new - h_prev) * mask + h_prev;
  return prob * h_prev + (1.0f - prob) * h_new;
}

constexpr float kLnEps = 1e-5f;  // lib/layer_norm_forward_gpu.cu.cc:77

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

static inline int ceil_div(long long a, long long b) { return (int)((a + b - 1) / b); }

// ---------------------------------------------------------------------------
// Dense contraction used by every cell:
//   C[m, n] (+)= sum_k A(m, k) * B(k, n)
// with A(m,k) at a[m*a_rs + k*a_cs], B(k,n) at b[k*b_rs + n*b_cs] and C row-major
// with leading dimension ldc.  accumulate != 0 adds into C.  Arithmetic is fp32.
// The dispatcher picks the tcgen05/TMA kernel when the operand layout allows it
// and the generic SIMT kernel otherwise.
// ---------------------------------------------------------------------------
struct GemmDesc {
  int dtype;    // storage of A and B: HASTE_B200_F32 / HASTE_B200_BF16
  int dtype_c;  // storage of C (fp32 C with bf16 operands is used for carries)
  int M, N, K;
  const void* a; long long a_rs, a_cs;
  const void* b; long long b_rs, b_cs;
  void* c; long long ldc;
  int accumulate;
  // fp32 storage only: split operands into three bf16 planes (six products) instead of two
  // (three products); the result is then accurate to fp32 rounding.  The LayerNorm cells
  // ask for it because normalisation amplifies the input projection's error.
  int precise = 0;
  // fp32 storage only: operand already available as two bf16 planes (hi at *_pl, lo
  // *_pl_stride elements later), same orientation as the operand, leading dimension *_pl_ld.
  // The recurrence kernels write gate gradients in this form so that they are split once.
  const void* a_pl = nullptr; long long a_pl_ld = 0, a_pl_stride = 0;
  const void* b_pl = nullptr; long long b_pl_ld = 0, b_pl_stride = 0;
};
int gemm(const GemmDesc& g, cudaStream_t stream);
int gemm_simt(const GemmDesc& g, cudaStream_t stream);
// fp32 [rows, cols] -> two bf16 planes (hi, lo), the a_pl / b_pl form, for an operand that
// more than one contraction reads (gemm_sm100.cu).
int gemm_split_planes(const float* src, long long ld_src, int rows, int cols,
                      __nv_bfloat16* dst, long long ld_dst, long long plane_stride,
                      cudaStream_t stream);

// Row LayerNorm launchers (layer_norm.cu); see include/haste_b200.h for semantics.
// `cache` is [rows,2] (mean, invstd) in `dtype`.  In the backward, dgamma/dbeta
// (dbeta may be null) are accumulated in `acc_dtype`, and `scratch` must hold
// layer_norm_backward_scratch_floats(rows, width) floats.  dx may alias dy.
int layer_norm_forward(int dtype, int rows, int width, const void* gamma, const void* beta,
                       const void* x, void* y, void* cache, cudaStream_t stream);
// Same, with the input stored as `in_dtype` (fp32 input with bf16 everything else is
// allowed) and an optional copy of the input, converted to `dtype`, written to x_copy.
int layer_norm_forward_from(int in_dtype, int dtype, int rows, int width, const void* gamma,
                            const void* beta, const void* x, void* y, void* cache, void* x_copy,
                            cudaStream_t stream);
size_t layer_norm_backward_scratch_floats(int rows, int width);
// dx_planes (fp32 storage only, width a multiple of 8): dx is also written as two bf16 planes
// (hi, then lo plane_stride elements later), the form GemmDesc::a_pl / b_pl takes.
int layer_norm_backward(int dtype, int rows, int width, const void* gamma, const void* x,
                        const void* dy, void* dx, int acc_dtype, void* dgamma, void* dbeta,
                        const void* cache, float* scratch, cudaStream_t stream,
                        __nv_bfloat16* dx_planes = nullptr, long long plane_stride = 0);

}  // namespace hb
