// Generic strided contraction on CUDA cores.
//
// This is the shape-agnostic path of hb::gemm: any M, N, K, any operand strides
// (so every transpose the cells need is expressed without a copy), fp32 or bf16
// storage, fp32 arithmetic.  The tcgen05/TMA kernel (gemm_sm100.cu) takes over
// whenever the operand layout satisfies TMA's alignment rules; this kernel is
// what remains for ragged shapes and is the in-library cross-check for it.
//
// Replaces the cuBLAS calls of the reference (lib/blas.h:48-61).
#include "common.cuh"
#include "util.cuh"

namespace hb {
namespace {

constexpr int TM = 64, TN = 64, TK = 16, THREADS = 256;

template <typename T, typename TC>
__global__ void __launch_bounds__(THREADS)
gemm_simt_kernel(int M, int N, int K, const T* __restrict__ A, long long a_rs, long long a_cs,
                 const T* __restrict__ B, long long b_rs, long long b_cs, TC* __restrict__ C,
                 long long ldc, int accumulate) {
  __shared__ float As[TK][TM + 4];
  __shared__ float Bs[TK][TN + 4];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
  const int tx = tid % 16, ty = tid / 16;  // 16 x 16 threads, 4 x 4 outputs each
  float acc[4][4] = {};

  // Loader mapping: choose the thread->element order so that the unit-stride
  // operand axis is walked by consecutive threads.
  const bool a_k_fast = (a_cs == 1);
  const bool b_n_fast = (b_cs == 1);

  for (int k0 = 0; k0 < K; k0 += TK) {
#pragma unroll
    for (int i = 0; i < (TM * TK) / THREADS; ++i) {
      const int e = tid + i * THREADS;
      int mm, kk;
      if (a_k_fast) { kk = e % TK; mm = e / TK; } else { mm = e % TM; kk = e / TM; }
      const int m = m0 + mm, k = k0 + kk;
      As[kk][mm] = (m < M && k < K) ? ld(A + (long long)m * a_rs + (long long)k * a_cs) : 0.0f;
    }
#pragma unroll
    for (int i = 0; i < (TN * TK) / THREADS; ++i) {
      const int e = tid + i * THREADS;
      int nn, kk;
      if (b_n_fast) { nn = e % TN; kk = e / TN; } else { kk = e % TK; nn = e / TK; }
      const int n = n0 + nn, k = k0 + kk;
      Bs[kk][nn] = (n < N && k < K) ? ld(B + (long long)k * b_rs + (long long)n * b_cs) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      TC* p = C + (long long)m * ldc + n;
      float v = acc[i][j];
      if (accumulate) v += ld(p);
      st(p, v);
    }
  }
}

}  // namespace



int gemm_simt(const GemmDesc& g, cudaStream_t stream) {
  if (g.M <= 0 || g.N <= 0) return HASTE_B200_OK;
  dim3 grid(ceil_div(g.N, TN), ceil_div(g.M, TM));
#define HB_SIMT_LAUNCH(TA, TC_)                                                              \
  gemm_simt_kernel<TA, TC_><<<grid, THREADS, 0, stream>>>(                                   \
      g.M, g.N, g.K, (const TA*)g.a, g.a_rs, g.a_cs, (const TA*)g.b, g.b_rs, g.b_cs,          \
      (TC_*)g.c, g.ldc, g.accumulate)
  if (g.dtype == HASTE_B200_F32 && g.dtype_c == HASTE_B200_F32) {
    HB_SIMT_LAUNCH(float, float);
  } else if (g.dtype == HASTE_B200_BF16 && g.dtype_c == HASTE_B200_BF16) {
    HB_SIMT_LAUNCH(__nv_bfloat16, __nv_bfloat16);
  } else if (g.dtype == HASTE_B200_BF16 && g.dtype_c == HASTE_B200_F32) {
    HB_SIMT_LAUNCH(__nv_bfloat16, float);
  } else if (g.dtype == HASTE_B200_F16 && g.dtype_c == HASTE_B200_F16) {
    HB_SIMT_LAUNCH(__half, __half);
  } else if (g.dtype == HASTE_B200_F16 && g.dtype_c == HASTE_B200_F32) {
    HB_SIMT_LAUNCH(__half, float);
  } else {
    set_last_error("gemm: unsupported dtype combination %d/%d", g.dtype, g.dtype_c);
    return HASTE_B200_ERR_INVALID;
  }
#undef HB_SIMT_LAUNCH
  count_launch(1);
  HB_LAUNCH_OK();
  return HASTE_B200_OK;
}

}  // namespace hb
