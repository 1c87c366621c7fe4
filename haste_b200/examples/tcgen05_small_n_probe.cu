// Measurement aid: what does one tcgen05.mma cost at the shape a recurrence step has?
//
// A recurrence step multiplies the CTA's resident slice of the recurrent matrix (as the M side,
// held in tensor memory: the "TS" form of tcgen05.mma) by the 16 batch rows the CTA owns (N = 16,
// from shared memory, K-major, 128-byte swizzle written by hand).  The program checks the
// result against the host (which also validates the tensor-memory operand layout: row = lane,
// two consecutive K elements per 32-bit column) and times 32 and 64 instructions of
// M=128, N=16, K=16 with 1, 2, 4 and 8 independent accumulators, issue loop fully unrolled.
//
// Measured on B200: 32 instructions 1760 cycles, 64 instructions 3670 cycles (commit, mbarrier
// wait, tcgen05.ld and CTA barrier included), i.e. ~60 cycles per instruction whatever the number
// of accumulators - 3700 cycles for the 64 instructions a step of the fp32 LSTM needs, against
// ~2000 cycles for the 768 mma.sync m16n8k16 the persistent kernels issue.  At N = 16 the tensor-memory path runs at an eighth of
// its peak, which is why the recurrence stays on mma.sync.
//
//   nvcc -std=c++17 -gencode arch=compute_100a,code=sm_100a -O3 tcgen05_small_n_probe.cu -o probe
//   ./probe            (one CTA, every wait bounded, a few milliseconds)
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <vector>
#include <cmath>

constexpr int K = 512, NB = 16;          // K elements, N (batch rows)
constexpr long long LIMIT = 2000000000LL;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((lbo >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo >> 4) & 0x3FFFu) << 32;
  d |= 1ull << 46;
  d |= 2ull << 61;
  return d;
}
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t desc_b, uint32_t idesc, uint32_t acc) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t}"
               :: "r"(d_tmem), "r"(a_tmem), "l"(desc_b), "r"(idesc), "r"(acc), "r"(0u) : "memory");
}

// A: [128][K] bf16 row-major (global), B: [NB][K] bf16 row-major (global), D: [128][NB] float
template <int NSLAB, int NACC>
__global__ void __launch_bounds__(128, 1) probe(const __nv_bfloat16* A, const __nv_bfloat16* B, float* D,
                                               long long* cycles, int iters, int* err) {
  constexpr int nacc = NACC;
  extern __shared__ __align__(1024) uint8_t smem[];
  __shared__ uint32_t tmem_slot;
  __shared__ __align__(8) uint64_t bar;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  uint8_t* bs = smem;  // B slabs: [K/64][16 rows][128 B], 128B swizzle
  // ---- B -> smem, swizzled by hand
  for (int e = tid; e < NB * (K / 8); e += 128) {       // one 16-byte chunk (8 elements) each
    const int r = e / (K / 8), c8 = e % (K / 8);         // row, chunk index along K
    const int slab = c8 / 8, c = c8 % 8;
    const uint4 v = *reinterpret_cast<const uint4*>(B + (size_t)r * K + c8 * 8);
    *reinterpret_cast<uint4*>(bs + slab * (NB * 128) + r * 128 + ((c ^ (r & 7)) * 16)) = v;
  }
  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&bar)));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = tmem_slot;
  // ---- A -> TMEM: lane = row, column c holds K elements 2c (low half), 2c+1 (high half)
  {
    const int m = warp * 32 + lane;
    const uint32_t taddr = tmem + ((uint32_t)(warp * 32) << 16);
    for (int c0 = 0; c0 < K / 2; c0 += 8) {
      uint32_t r[8];
      const uint4 v0 = *reinterpret_cast<const uint4*>(A + (size_t)m * K + c0 * 2);
      const uint4 v1 = *reinterpret_cast<const uint4*>(A + (size_t)m * K + c0 * 2 + 8);
      r[0] = v0.x; r[1] = v0.y; r[2] = v0.z; r[3] = v0.w; r[4] = v1.x; r[5] = v1.y; r[6] = v1.z; r[7] = v1.w;
      asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                   :: "r"(taddr + c0), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]) : "memory");
    }
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic smem writes -> async proxy
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

  const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(NB >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
  const uint32_t d_tmem = tmem + 256;   // accumulator columns 256..271
  uint32_t parity = 0;
  bool ok = true;
  long long t0 = clock64();
  for (int it = 0; it < iters && ok; ++it) {
    if (tid == 0) {
      const uint64_t db0 = smem_desc(smem_u32(bs), 16, 1024);
#pragma unroll
      for (int i = 0; i < NSLAB * 4; ++i) {
        const int slab = (i / 4) % (K / 64), ks = i % 4;
        // the start-address field counts 16-byte units: a plain add moves the descriptor
        mma_ts(d_tmem + (i % NACC) * 16, tmem + (slab * 4 + ks) * 8,
               db0 + (uint64_t)((slab * (NB * 128) + ks * 32) >> 4), idesc, i < NACC ? 0u : 1u);
      }
      asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&bar)) : "memory");
    }
    // all threads wait (bounded)
    const long long w0 = clock64();
    while (!mbar_try_wait(smem_u32(&bar), parity)) {
      if (clock64() - w0 > LIMIT) { ok = false; *err = 1; break; }
    }
    parity ^= 1u;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    float r[16];
    for (int j = 0; j < 16; ++j) r[j] = 0.f;
    for (int a = 0; a < nacc; ++a) {
      uint32_t q[16];
      asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                   : "=r"(q[0]), "=r"(q[1]), "=r"(q[2]), "=r"(q[3]), "=r"(q[4]), "=r"(q[5]), "=r"(q[6]), "=r"(q[7]),
                     "=r"(q[8]), "=r"(q[9]), "=r"(q[10]), "=r"(q[11]), "=r"(q[12]), "=r"(q[13]), "=r"(q[14]), "=r"(q[15])
                   : "r"(d_tmem + a * 16 + ((uint32_t)(warp * 32) << 16)));
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      for (int j = 0; j < 16; ++j) r[j] += __uint_as_float(q[j]);
    }
    if (it == iters - 1) {
      for (int j = 0; j < 16; ++j) D[(size_t)(warp * 32 + lane) * NB + j] = r[j];
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();   // D consumed before the next iteration overwrites it
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  }
  if (tid == 0) *cycles = clock64() - t0;
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
}

int main() {
  std::vector<__nv_bfloat16> hA(128 * K), hB(NB * K);
  std::vector<float> fA(128 * K), fB(NB * K);
  for (int i = 0; i < 128 * K; ++i) { float v = (float)((i * 7 + i / K) % 13 - 6) / 8.0f; hA[i] = __float2bfloat16(v); fA[i] = __bfloat162float(hA[i]); }
  for (int i = 0; i < NB * K; ++i) { float v = (float)((i * 5 + 3 * (i / K)) % 11 - 5) / 4.0f; hB[i] = __float2bfloat16(v); fB[i] = __bfloat162float(hB[i]); }
  __nv_bfloat16 *dA, *dB; float* dD; long long* dc; int* derr;
  cudaMalloc(&dA, hA.size() * 2); cudaMalloc(&dB, hB.size() * 2); cudaMalloc(&dD, 128 * NB * 4); cudaMalloc(&dc, 8); cudaMalloc(&derr, 4);
  cudaMemcpy(dA, hA.data(), hA.size() * 2, cudaMemcpyHostToDevice);
  cudaMemcpy(dB, hB.data(), hB.size() * 2, cudaMemcpyHostToDevice);
  cudaMemset(derr, 0, 4);
  const int smem = (K / 64) * NB * 128 + 1024;
  for (int cfg = 0; cfg < 9; ++cfg) {
    const int iters = 1000;
    int nacc = 1, nslab = 8;
    switch (cfg) {
      case 0: cudaFuncSetAttribute(probe<8, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); probe<8, 1><<<1, 128, smem>>>(dA, dB, dD, dc, iters, derr); nacc = 1; nslab = 8; break;
      case 1: cudaFuncSetAttribute(probe<8, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); probe<8, 1><<<1, 128, smem>>>(dA, dB, dD, dc, iters, derr); nacc = 1; nslab = 8; break;
      case 2: cudaFuncSetAttribute(probe<16, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); probe<16, 1><<<1, 128, smem>>>(dA, dB, dD, dc, iters, derr); nacc = 1; nslab = 16; break;
      case 3: cudaFuncSetAttribute(probe<8, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); probe<8, 2><<<1, 128, smem>>>(dA, dB, dD, dc, iters, derr); nacc = 2; nslab = 8; break;
      case 4: cudaFuncSetAttribute(probe<16, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); probe<16, 2><<<1, 128, smem>>>(dA, dB, dD, dc, iters, derr); nacc = 2; nslab = 16; break;
      case 5: cudaFuncSetAttribute(probe<8, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); probe<8, 4><<<1, 128, smem>>>(dA, dB, dD, dc, iters, derr); nacc = 4; nslab = 8; break;
      case 6: cudaFuncSetAttribute(probe<16, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); probe<16, 4><<<1, 128, smem>>>(dA, dB, dD, dc, iters, derr); nacc = 4; nslab = 16; break;
      case 7: cudaFuncSetAttribute(probe<8, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); probe<8, 8><<<1, 128, smem>>>(dA, dB, dD, dc, iters, derr); nacc = 8; nslab = 8; break;
      case 8: cudaFuncSetAttribute(probe<16, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); probe<16, 8><<<1, 128, smem>>>(dA, dB, dD, dc, iters, derr); nacc = 8; nslab = 16; break;
    }
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) { printf("CUDA error: %s\n", cudaGetErrorString(e)); return 1; }
    long long cyc; int err; std::vector<float> hD(128 * NB);
    cudaMemcpy(&cyc, dc, 8, cudaMemcpyDeviceToHost); cudaMemcpy(&err, derr, 4, cudaMemcpyDeviceToHost);
    cudaMemcpy(hD.data(), dD, hD.size() * 4, cudaMemcpyDeviceToHost);
    double maxerr = 0; 
    for (int m = 0; m < 128; ++m) for (int n = 0; n < NB; ++n) {
      double s = 0; for (int k = 0; k < K; ++k) s += (double)fA[m * K + k] * fB[n * K + k];
      maxerr = std::fmax(maxerr, std::fabs(s - hD[m * NB + n]));
    }
    printf("nacc %d mmas %3d: err flag %d, max |D - ref| = %g, cycles/iter = %.1f\n", nacc, nslab * 4, err, maxerr, (double)cyc / iters);
  }
  return 0;
}
