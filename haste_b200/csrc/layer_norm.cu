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

// Three sums at once (one pair of barriers).
__device__ __forceinline__ void block_sum3(float& a, float& b, float& c, float (*red)[3]) {
  a = warp_sum(a); b = warp_sum(b); c = warp_sum(c);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) { red[warp][0] = a; red[warp][1] = b; red[warp][2] = c; }
  __syncthreads();
  a = b = c = 0.f;
#pragma unroll
  for (int w = 0; w < LN_THREADS / 32; ++w) { a += red[w][0]; b += red[w][1]; c += red[w][2]; }
}

// Four consecutive elements, 16-byte (fp32) or 8-byte (bf16) accesses.
__device__ __forceinline__ void ld4(const float* p, float (&v)[4]) {
  const float4 f = *reinterpret_cast<const float4*>(p);
  v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
}
__device__ __forceinline__ void ld4(const __nv_bfloat16* p, float (&v)[4]) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  v[0] = __uint_as_float(u.x << 16); v[1] = __uint_as_float(u.x & 0xFFFF0000u);
  v[2] = __uint_as_float(u.y << 16); v[3] = __uint_as_float(u.y & 0xFFFF0000u);
}
__device__ __forceinline__ void st4(float* p, const float (&v)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void st4(__nv_bfloat16* p, const float (&v)[4]) {
  const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
  uint2 u;
  u.x = *reinterpret_cast<const uint32_t*>(&a);
  u.y = *reinterpret_cast<const uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = u;
}

// Rows of up to LN_THREADS * 4 * LN_MAXV elements (a multiple of 4, vector-aligned) are read
// from memory once and kept in registers between the passes of the two-pass algorithm; the
// kernels are instantiated for 1, 2, 4 and 8 groups of four elements per thread, so that a
// narrow row does not pay the registers (and the occupancy) of a wide one.
constexpr int LN_MAXV = 8;
inline int ln_groups(int width) {
  const int per = ((width >> 2) + LN_THREADS - 1) / LN_THREADS;
  return per <= 1 ? 1 : (per <= 2 ? 2 : (per <= 4 ? 4 : 8));
}
inline bool ln_vec_ok(int width, const void* a, const void* b, const void* c, const void* d,
                      size_t elem) {
  const uintptr_t m = elem * 4 - 1;
  auto al = [&](const void* p) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) & m) == 0; };
  return (width % 4) == 0 && width <= LN_THREADS * 4 * LN_MAXV && al(a) && al(b) && al(c) && al(d);
}

template <typename T, typename TI, int MAXV>
__global__ void __launch_bounds__(LN_THREADS)
ln_forward_vec_kernel(int width, const T* __restrict__ gamma, const T* __restrict__ beta,
                      const TI* __restrict__ x, T* __restrict__ y, T* __restrict__ cache,
                      T* __restrict__ x_copy) {
  __shared__ float red[LN_THREADS / 32];
  const long long row = blockIdx.x;
  const TI* xr = x + row * width;
  const int nvec = width >> 2;
  float v[MAXV][4];
  float s = 0.f;
#pragma unroll
  for (int k = 0; k < MAXV; ++k) {
    const int i = k * LN_THREADS + threadIdx.x;
    if (i < nvec) {
      ld4(xr + i * 4, v[k]);
      s += (v[k][0] + v[k][1]) + (v[k][2] + v[k][3]);
    }
  }
  const float mean = block_sum(s, red) / width;
  float q = 0.f;
#pragma unroll
  for (int k = 0; k < MAXV; ++k) {
    const int i = k * LN_THREADS + threadIdx.x;
    if (i < nvec) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float d = v[k][e] - mean;
        q += d * d;
      }
    }
  }
  const float invstd = rsqrtf(block_sum(q, red) / width + kLnEps);
#pragma unroll
  for (int k = 0; k < MAXV; ++k) {
    const int i = k * LN_THREADS + threadIdx.x;
    if (i < nvec) {
      float g[4], o[4];
      ld4(gamma + i * 4, g);
#pragma unroll
      for (int e = 0; e < 4; ++e) o[e] = (v[k][e] - mean) * invstd * g[e];
      if (beta) {
        float b[4];
        ld4(beta + i * 4, b);
#pragma unroll
        for (int e = 0; e < 4; ++e) o[e] += b[e];
      }
      st4(y + row * width + i * 4, o);
      if (x_copy) st4(x_copy + row * width + i * 4, v[k]);
    }
  }
  if (threadIdx.x == 0) {
    st(cache + row * 2 + 0, mean);
    st(cache + row * 2 + 1, invstd);
  }
}

// Planes (fp32 only): dx is also written as two bf16 planes (hi, lo) of the same shape, the lo
// plane `plane_stride` elements after the hi plane - the form the contractions read fp32
// operands in.
template <typename T, bool Planes, int MAXV>
__global__ void __launch_bounds__(LN_THREADS)
ln_backward_dx_vec_kernel(int width, const T* __restrict__ gamma, const T* __restrict__ x,
                          const T* dy, T* dx, const T* __restrict__ cache,
                          __nv_bfloat16* __restrict__ planes, long long plane_stride) {
  __shared__ float red[LN_THREADS / 32][3];
  const long long row = blockIdx.x;
  const int nvec = width >> 2;
  const float mean = ld(cache + row * 2), invstd = ld(cache + row * 2 + 1);
  float cx[MAXV][4], db[MAXV][4];
  float s_sigma = 0.f, s_mu1 = 0.f, s_mu2 = 0.f;
#pragma unroll
  for (int k = 0; k < MAXV; ++k) {
    const int i = k * LN_THREADS + threadIdx.x;
    if (i < nvec) {
      float g[4];
      ld4(x + row * width + i * 4, cx[k]);
      ld4(dy + row * width + i * 4, db[k]);
      ld4(gamma + i * 4, g);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        cx[k][e] -= mean;
        db[k][e] *= g[e];
        s_sigma += cx[k][e] * db[k][e];
        s_mu1 += cx[k][e];
        s_mu2 += db[k][e];
      }
    }
  }
  block_sum3(s_sigma, s_mu1, s_mu2, red);
  const float dsigma = -0.5f * s_sigma * invstd * invstd * invstd;
  const float dmu = (-2.0f * s_mu1 * dsigma / width) - (s_mu2 * invstd);
  // dx may alias dy: the row is in registers before anything is written
#pragma unroll
  for (int k = 0; k < MAXV; ++k) {
    const int i = k * LN_THREADS + threadIdx.x;
    if (i < nvec) {
      float o[4];
#pragma unroll
      for (int e = 0; e < 4; ++e)
        o[e] = (2.0f * cx[k][e] * dsigma / width) + (invstd * db[k][e]) + (dmu / width);
      st4(dx + row * width + i * 4, o);
      if (Planes) {
        float hi[4], lo[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          hi[e] = __bfloat162float(__float2bfloat16_rn(o[e]));
          lo[e] = o[e] - hi[e];
        }
        st4(planes + row * width + i * 4, hi);
        st4(planes + plane_stride + row * width + i * 4, lo);
      }
    }
  }
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
  // four independent partial sums (rows r, r+1, r+2, r+3 in turn): the loads of four rows are
  // in flight together; the order of the sums is fixed, so the result is deterministic
  float g[4] = {0.f, 0.f, 0.f, 0.f}, b[4] = {0.f, 0.f, 0.f, 0.f};
  int r = r0;
  for (; r + 4 <= r1; r += 4) {
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const long long rr = r + u;
      const float mean = ld(cache + rr * 2), invstd = ld(cache + rr * 2 + 1);
      const float d = ld(dy + rr * width + j);
      g[u] += (ld(x + rr * width + j) - mean) * invstd * d;
      b[u] += d;
    }
  }
  for (; r < r1; ++r) {
    const float mean = ld(cache + (long long)r * 2), invstd = ld(cache + (long long)r * 2 + 1);
    const float d = ld(dy + (long long)r * width + j);
    g[0] += (ld(x + (long long)r * width + j) - mean) * invstd * d;
    b[0] += d;
  }
  part_g[(long long)c * width + j] = (g[0] + g[1]) + (g[2] + g[3]);
  part_b[(long long)c * width + j] = (b[0] + b[1]) + (b[2] + b[3]);
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
  const size_t es_in = in_dtype == HASTE_B200_F32 ? 4 : 2, es = dtype == HASTE_B200_F32 ? 4 : 2;
  const bool vec = ln_vec_ok(width, x, nullptr, nullptr, nullptr, es_in) &&
                   ln_vec_ok(width, gamma, beta, y, x_copy, es);
#define HB_LN_FWD_V(T_, TI_, V_)                                                               \
  ln_forward_vec_kernel<T_, TI_, V_><<<rows, LN_THREADS, 0, stream>>>(                          \
      width, (const T_*)gamma, (const T_*)beta, (const TI_*)x, (T_*)y, (T_*)cache, (T_*)x_copy)
#define HB_LN_FWD(T_, TI_)                                                                     \
  do {                                                                                         \
    switch (ln_groups(width)) {                                                                \
      case 1: HB_LN_FWD_V(T_, TI_, 1); break;                                                  \
      case 2: HB_LN_FWD_V(T_, TI_, 2); break;                                                  \
      case 4: HB_LN_FWD_V(T_, TI_, 4); break;                                                  \
      default: HB_LN_FWD_V(T_, TI_, 8); break;                                                 \
    }                                                                                          \
  } while (0)
  if (vec && dtype == HASTE_B200_F32 && in_dtype == HASTE_B200_F32)
    HB_LN_FWD(float, float);
  else if (vec && dtype == HASTE_B200_BF16 && in_dtype == HASTE_B200_BF16)
    HB_LN_FWD(bf, bf);
  else if (vec && dtype == HASTE_B200_BF16 && in_dtype == HASTE_B200_F32)
    HB_LN_FWD(bf, float);
  else if (dtype == HASTE_B200_F32 && in_dtype == HASTE_B200_F32)
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
#undef HB_LN_FWD
#undef HB_LN_FWD_V
  HB_LAUNCH_OK();
  count_launch(1);
  return HASTE_B200_OK;
}

size_t layer_norm_backward_scratch_floats(int rows, int width) {
  return 2 * (size_t)pg_chunks(rows) * width;
}

int layer_norm_backward(int dtype, int rows, int width, const void* gamma, const void* x,
                        const void* dy, void* dx, int acc_dtype, void* dgamma, void* dbeta,
                        const void* cache, float* scratch, cudaStream_t stream,
                        __nv_bfloat16* dx_planes, long long plane_stride) {
  if (rows <= 0) return HASTE_B200_OK;
  if (dx_planes && (dtype != HASTE_B200_F32 || (width % 8) != 0)) {
    set_last_error("layer_norm_backward: planes need fp32 storage and a width that is a multiple of 8");
    return HASTE_B200_ERR_INVALID;
  }
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
  const bool vec = ln_vec_ok(width, gamma, x, dy, dx, dtype == HASTE_B200_F32 ? 4 : 2);
  if (dtype == HASTE_B200_F32) {
#define HB_LN_BWD_V(T_, P_, V_)                                                                \
  ln_backward_dx_vec_kernel<T_, P_, V_><<<rows, LN_THREADS, 0, stream>>>(                       \
      width, (const T_*)gamma, (const T_*)x, (const T_*)dy, (T_*)dx, (const T_*)cache,          \
      P_ ? dx_planes : nullptr, plane_stride)
#define HB_LN_BWD(T_, P_)                                                                      \
  do {                                                                                         \
    switch (ln_groups(width)) {                                                                \
      case 1: HB_LN_BWD_V(T_, P_, 1); break;                                                   \
      case 2: HB_LN_BWD_V(T_, P_, 2); break;                                                   \
      case 4: HB_LN_BWD_V(T_, P_, 4); break;                                                   \
      default: HB_LN_BWD_V(T_, P_, 8); break;                                                  \
    }                                                                                          \
  } while (0)
    if (vec && dx_planes)
      HB_LN_BWD(float, true);
    else if (vec)
      HB_LN_BWD(float, false);
    else
      ln_backward_dx_kernel<float><<<rows, LN_THREADS, 0, stream>>>(
          width, (const float*)gamma, (const float*)x, (const float*)dy, (float*)dx,
          (const float*)cache);
    if (!vec && dx_planes) {
      HB_LAUNCH_OK();
      HB_TRY(gemm_split_planes(static_cast<const float*>(dx), width, rows, width, dx_planes, width,
                               plane_stride, stream));
    }
  } else {
    using bf = __nv_bfloat16;
    if (vec)
      HB_LN_BWD(bf, false);
    else
      ln_backward_dx_kernel<bf><<<rows, LN_THREADS, 0, stream>>>(
          width, (const bf*)gamma, (const bf*)x, (const bf*)dy, (bf*)dx, (const bf*)cache);
  }
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
