// Row LayerNorm, forward and backward.
//
// Same arithmetic as the reference's kernels (two-pass mean, biased variance,
// eps 1e-5 inside the rsqrt, cache of (mean, invstd) per row:
// lib/layer_norm_forward_gpu.cu.cc:22-88; gradient formula
// lib/layer_norm_backward_gpu.cu.cc:44-91), but reductions use warp shuffles and
// the parameter gradients are a deterministic two-stage column reduction instead
// of per-element atomics.
#include <mutex>

#include "common.cuh"
#include "util.cuh"

namespace hb {
namespace {

constexpr int LN_THREADS = 128;

// Sum over the block; every thread gets the result.  `red` holds one float per warp.
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();  // protect `red` from the previous use
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float s = 0.f;
#pragma unroll
  for (int w = 0; w < LN_THREADS / 32; ++w) s += red[w];
  return s;
}

// TI is the storage type of the input (fp32 input with bf16 parameters/outputs is used
// inside the bf16 LayerNorm cells so that a value is rounded once, when it is saved).
// x_copy, if not null, receives the input converted to T.
template <typename T, typename TI>
__global__ void __launch_bounds__(LN_THREADS)
ln_forward_kernel(int width, const T* __restrict__ gamma, const T* __restrict__ beta,
                  const TI* __restrict__ x, T* __restrict__ y, T* __restrict__ cache,
                  T* __restrict__ x_copy) {
  __shared__ float red[LN_THREADS / 32];
  const long long row = blockIdx.x;
  const TI* xr = x + row * width;
  T* yr = y + row * width;
  if (x_copy)
    for (int i = threadIdx.x; i < width; i += LN_THREADS) st(x_copy + row * width + i, ld(xr + i));
  float s = 0.f;
  for (int i = threadIdx.x; i < width; i += LN_THREADS) s += ld(xr + i);
  const float mean = block_sum(s, red) / width;
  float q = 0.f;
  for (int i = threadIdx.x; i < width; i += LN_THREADS) {
    const float d = ld(xr + i) - mean;
    q += d * d;
  }
  const float invstd = rsqrtf(block_sum(q, red) / width + kLnEps);
  for (int i = threadIdx.x; i < width; i += LN_THREADS) {
    float v = (ld(xr + i) - mean) * invstd * ld(gamma + i);
    if (beta) v += ld(beta + i);
    st(yr + i, v);
  }
  if (threadIdx.x == 0) {
    st(cache + row * 2 + 0, mean);
    st(cache + row * 2 + 1, invstd);
  }
}

// Stage 1 of the parameter gradients: partial column sums of z*dy and dy over a
// chunk of rows.  One thread per column, consecutive threads on consecutive columns.
constexpr int PG_COLS = 128;
constexpr int PG_CHUNKS = 64;
inline int pg_chunks(int rows) { return rows < PG_CHUNKS ? (rows > 0 ? rows : 1) : PG_CHUNKS; }

template <typename T>
__global__ void ln_param_grad_stage1(int rows, int width, int chunks, const T* __restrict__ x,
                                     const T* __restrict__ dy, const T* __restrict__ cache,
                                     float* __restrict__ part_g, float* __restrict__ part_b) {
  const int j = blockIdx.x * PG_COLS + threadIdx.x;
  if (j >= width) return;
  const int c = blockIdx.y;
  const int per = (rows + chunks - 1) / chunks;
  const int r0 = c * per, r1 = min(rows, r0 + per);
  float g = 0.f, b = 0.f;
  for (int r = r0; r < r1; ++r) {
    const float mean = ld(cache + (long long)r * 2), invstd = ld(cache + (long long)r * 2 + 1);
    const float d = ld(dy + (long long)r * width + j);
    g += (ld(x + (long long)r * width + j) - mean) * invstd * d;
    b += d;
  }
  part_g[(long long)c * width + j] = g;
  part_b[(long long)c * width + j] = b;
}

template <typename TA>
__global__ void ln_param_grad_stage2(int width, int chunks, const float* __restrict__ part_g,
                                     const float* __restrict__ part_b, TA* __restrict__ dgamma,
                                     TA* __restrict__ dbeta) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= width) return;
  float g = 0.f, b = 0.f;
  for (int c = 0; c < chunks; ++c) {
    g += part_g[(long long)c * width + j];
    b += part_b[(long long)c * width + j];
  }
  st(dgamma + j, ld(dgamma + j) + g);
  if (dbeta) st(dbeta + j, ld(dbeta + j) + b);
}

template <typename T>
__global__ void __launch_bounds__(LN_THREADS)
ln_backward_dx_kernel(int width, const T* __restrict__ gamma, const T* __restrict__ x,
                      const T* dy, T* dx, const T* __restrict__ cache) {
  __shared__ float red[LN_THREADS / 32];
  const long long row = blockIdx.x;
  const T* xr = x + row * width;
  const T* dyr = dy + row * width;
  T* dxr = dx + row * width;
  const float mean = ld(cache + row * 2), invstd = ld(cache + row * 2 + 1);
  float s_sigma = 0.f, s_mu1 = 0.f, s_mu2 = 0.f;
  for (int i = threadIdx.x; i < width; i += LN_THREADS) {
    const float cx = ld(xr + i) - mean;
    const float db = ld(gamma + i) * ld(dyr + i);
    s_sigma += cx * db;
    s_mu1 += cx;
    s_mu2 += db;
  }
  s_sigma = block_sum(s_sigma, red);
  s_mu1 = block_sum(s_mu1, red);
  s_mu2 = block_sum(s_mu2, red);
  const float dsigma = -0.5f * s_sigma * invstd * invstd * invstd;
  const float dmu = (-2.0f * s_mu1 * dsigma / width) - (s_mu2 * invstd);
  // dx may alias dy: each element is read before it is written by the same thread.
  for (int i = threadIdx.x; i < width; i += LN_THREADS) {
    const float cx = ld(xr + i) - mean;
    const float db = ld(gamma + i) * ld(dyr + i);
    st(dxr + i, (2.0f * cx * dsigma / width) + (invstd * db) + (dmu / width));
  }
}

}  // namespace

int layer_norm_forward(int dtype, int rows, int width, const void* gamma, const void* beta,
                       const void* x, void* y, void* cache, cudaStream_t stream) {
  return layer_norm_forward_from(dtype, dtype, rows, width, gamma, beta, x, y, cache, nullptr,
                                 stream);
}

int layer_norm_forward_from(int in_dtype, int dtype, int rows, int width, const void* gamma,
                            const void* beta, const void* x, void* y, void* cache, void* x_copy,
                            cudaStream_t stream) {
  if (rows <= 0) return HASTE_B200_OK;
  using bf = __nv_bfloat16;
  if (dtype == HASTE_B200_F32 && in_dtype == HASTE_B200_F32)
    ln_forward_kernel<float, float><<<rows, LN_THREADS, 0, stream>>>(
        width, (const float*)gamma, (const float*)beta, (const float*)x, (float*)y, (float*)cache,
        (float*)x_copy);
  else if (dtype == HASTE_B200_BF16 && in_dtype == HASTE_B200_BF16)
    ln_forward_kernel<bf, bf><<<rows, LN_THREADS, 0, stream>>>(
        width, (const bf*)gamma, (const bf*)beta, (const bf*)x, (bf*)y, (bf*)cache, (bf*)x_copy);
  else if (dtype == HASTE_B200_BF16 && in_dtype == HASTE_B200_F32)
    ln_forward_kernel<bf, float><<<rows, LN_THREADS, 0, stream>>>(
        width, (const bf*)gamma, (const bf*)beta, (const float*)x, (bf*)y, (bf*)cache, (bf*)x_copy);
  else {
    set_last_error("layer_norm_forward: unsupported dtype combination %d -> %d", in_dtype, dtype);
    return HASTE_B200_ERR_INVALID;
  }
  HB_LAUNCH_OK();
  count_launch(1);
  return HASTE_B200_OK;
}

size_t layer_norm_backward_scratch_floats(int rows, int width) {
  return 2 * (size_t)pg_chunks(rows) * width;
}

int layer_norm_backward(int dtype, int rows, int width, const void* gamma, const void* x,
                        const void* dy, void* dx, int acc_dtype, void* dgamma, void* dbeta,
                        const void* cache, float* scratch, cudaStream_t stream) {
  if (rows <= 0) return HASTE_B200_OK;
  const int chunks = pg_chunks(rows);
  float* part_g = scratch;
  float* part_b = scratch + (size_t)chunks * width;
  dim3 g1(ceil_div(width, PG_COLS), chunks);
  if (dtype == HASTE_B200_F32)
    ln_param_grad_stage1<float><<<g1, PG_COLS, 0, stream>>>(
        rows, width, chunks, (const float*)x, (const float*)dy, (const float*)cache, part_g, part_b);
  else
    ln_param_grad_stage1<__nv_bfloat16><<<g1, PG_COLS, 0, stream>>>(
        rows, width, chunks, (const __nv_bfloat16*)x, (const __nv_bfloat16*)dy,
        (const __nv_bfloat16*)cache, part_g, part_b);
  HB_LAUNCH_OK();
  if (acc_dtype == HASTE_B200_F32)
    ln_param_grad_stage2<float><<<ceil_div(width, 128), 128, 0, stream>>>(
        width, chunks, part_g, part_b, (float*)dgamma, (float*)dbeta);
  else
    ln_param_grad_stage2<__nv_bfloat16><<<ceil_div(width, 128), 128, 0, stream>>>(
        width, chunks, part_g, part_b, (__nv_bfloat16*)dgamma, (__nv_bfloat16*)dbeta);
  HB_LAUNCH_OK();
  if (dtype == HASTE_B200_F32)
    ln_backward_dx_kernel<float><<<rows, LN_THREADS, 0, stream>>>(
        width, (const float*)gamma, (const float*)x, (const float*)dy, (float*)dx,
        (const float*)cache);
  else
    ln_backward_dx_kernel<__nv_bfloat16><<<rows, LN_THREADS, 0, stream>>>(
        width, (const __nv_bfloat16*)gamma, (const __nv_bfloat16*)x, (const __nv_bfloat16*)dy,
        (__nv_bfloat16*)dx, (const __nv_bfloat16*)cache);
  HB_LAUNCH_OK();
  count_launch(3);
  return HASTE_B200_OK;
}

}  // namespace hb

// ---------------------------------------------------------------------------------------
// LayerNorm backward for callers that must not allocate.
//
// haste_b200_layer_norm_backward takes its reduction scratch (the per-chunk partial sums of
// dgamma/dbeta) from the library's grow-only pool, which calls cudaMalloc the first time and
// whenever a larger problem arrives.  Some callers cannot afford that: a serving or audio
// loop that has handed every byte of device memory to its own arena (cudaMalloc then fails
// or fragments it), code between cudaStreamBeginCapture and EndCapture (allocation is
// illegal there), and latency-critical loops in which cudaMalloc's implicit device-wide
// synchronisation would stall every other stream.  For them this entry point keeps the
// scratch in a fixed array inside the library image: 2 * 64 chunks * 4096 columns of fp32
// = 2 MiB per GPU that loads the library, held until the process exits.
// ---------------------------------------------------------------------------------------
namespace hb {
namespace {

constexpr int NOALLOC_MAX_WIDTH = 4096;
static __device__ __align__(256) float g_ln_noalloc_scratch[2 * PG_CHUNKS * NOALLOC_MAX_WIDTH];

// g_ln_noalloc_scratch names a host-side handle here, not device memory: the address a
// kernel can use is looked up once per device (with that device current) and remembered.
constexpr int NOALLOC_MAX_DEVICES = 64;
float* g_noalloc_ptr[NOALLOC_MAX_DEVICES] = {};
std::mutex g_noalloc_mu;

int noalloc_scratch(float** out) {
  int dev = 0;
  HB_CUDA_OK(cudaGetDevice(&dev));
  HB_REQUIRE(dev >= 0 && dev < NOALLOC_MAX_DEVICES, "device ordinal out of range");
  std::lock_guard<std::mutex> lk(g_noalloc_mu);
  if (!g_noalloc_ptr[dev]) {
    float* p = nullptr;
    HB_CUDA_OK(cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_ln_noalloc_scratch));
    g_noalloc_ptr[dev] = p;
  }
  *out = g_noalloc_ptr[dev];
  return HASTE_B200_OK;
}

}  // namespace
}  // namespace hb

extern "C" int haste_b200_layer_norm_backward_noalloc(int dtype, int rows, int width,
                                                      const void* gamma, const void* x,
                                                      const void* dy, void* dx, void* dgamma,
                                                      void* dbeta, const void* cache,
                                                      void* stream) {
  using namespace hb;
  HB_REQUIRE(dtype == HASTE_B200_F32 || dtype == HASTE_B200_BF16, "dtype");
  HB_REQUIRE(rows >= 0 && width > 0, "rows,width");
  if (width > NOALLOC_MAX_WIDTH) {
    set_last_error("layer_norm_backward_noalloc: width %d exceeds the built-in scratch (max %d "
                   "columns); use haste_b200_layer_norm_backward", width, NOALLOC_MAX_WIDTH);
    return HASTE_B200_ERR_UNSUPPORTED;
  }
  HB_REQUIRE(gamma && x && dy && dx && dgamma && cache, "null pointer");
  if (rows == 0) return HASTE_B200_OK;
  float* scratch = nullptr;
  HB_TRY(noalloc_scratch(&scratch));
  // Stage 1 writes every partial that stage 2 reads, so nothing in the array has to start
  // at zero; what the previous call left behind is simply overwritten.
  return layer_norm_backward(dtype, rows, width, gamma, x, dy, dx, dtype, dgamma, dbeta, cache,
                             scratch, (cudaStream_t)stream);
}
