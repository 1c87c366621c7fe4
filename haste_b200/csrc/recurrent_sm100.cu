// Persistent recurrence kernels for LSTM and GRU (forward and backward).
//
// One cooperative launch covers all T steps of a layer pass; nothing is launched per
// time step.  The grid is (hidden slices) x (batch slices).  A CTA owns U = 16 hidden
// units (all G gates of them) for up to 64 batch rows and keeps its slice of the
// recurrent matrix R in REGISTERS, as ready-made mma.sync B-fragments, for the whole
// kernel: R is read from HBM exactly once per pass.
//
//   forward : gates[rows, G*U] = h_{t-1}[rows, :] . R[:, slice]       (K = H)
//             The K range is split over the 8 warps (each warp owns H/8 of K for all of
//             the CTA's columns), so the CTA's copy of h_{t-1} is read from shared memory
//             once, not once per warp; the 8 partial tiles are summed by the pointwise
//             stage, which also adds x.W + b, applies the nonlinearities, zoneout and the
//             c/h update, and writes h_t, c_t and the gate cache.
//   backward: dh_{t-1}[rows, :] += dG_t[rows, slice] . R[:, slice]^T   (K = G*U)
//             Each CTA turns its own gate gradients into a partial dh for ALL hidden units
//             (output columns split over the warps); partials are exchanged through a
//             double-buffered scratch area and summed, in a fixed order, by the CTA that
//             owns the unit.  dh/dc carries live in registers.
//
// fp32 storage: operands are split on the fly into bf16 (hi, lo) pairs and three
// products (hi.hi, hi.lo, lo.hi) are accumulated in fp32, which keeps the step product
// within ~1e-5 of fp32 arithmetic.  bf16 storage: one product.
//
// Steps are ordered by one monotonically increasing counter per batch-slice group
// (release/acquire through L2); CTAs of different batch slices never wait on each other.
// Every wait is bounded: when the limit runs out the CTA raises the abort flag and the
// process error word, every CTA leaves its loop, and the host reports
// HASTE_B200_ERR_TIMEOUT.  The launch is cooperative, so all CTAs are co-resident.
//
// Replaces the per-step cuBLAS call + pointwise kernel of the reference
// (lib/lstm_forward_gpu.cu.cc:210-310, lib/lstm_backward_gpu.cu.cc:246-316,
//  lib/gru_forward_gpu.cu.cc:214-308, lib/gru_backward_gpu.cu.cc:252-320).
#include <cstdlib>
#include <mutex>

#include "cells.cuh"

namespace hb {
namespace {

constexpr int U = 16;          // hidden units per CTA
constexpr int WARPS = 8;
constexpr int THREADS = WARPS * 32;
constexpr int MAX_MT = 4;      // up to 4 m-tiles of 16 batch rows per CTA
constexpr long long SPIN_LIMIT_CYCLES = 4000000000LL;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo_elem, float hi_elem) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo_elem, hi_elem);  // .x = first (lower address)
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ void split_bf16(float x, float& hi, float& lo) {
  hi = __bfloat162float(__float2bfloat16_rn(x));
  lo = x - hi;
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t (&a)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3])
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned int ld_acquire(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float ldcg(const float* p) { return __ldcg(p); }
__device__ __forceinline__ float ldcg(const __nv_bfloat16* p) {
  return __bfloat162float(__ldcg(p));
}

struct Sync {
  unsigned int* ctr;  // one counter per batch slice, 32 words apart
  int* abort_flag;    // device-global
  int* err;           // process error word (pinned host memory)
};

// Thread 0 waits until the group's counter reaches `target`; everyone learns the result.
// Returns false when the kernel must stop.
__device__ __forceinline__ bool wait_group(const Sync& s, int bs, unsigned int target,
                                           int* smem_flag) {
  if (threadIdx.x == 0) {
    int ok = 1;
    const unsigned int* c = s.ctr + bs * 32;
    if (ld_acquire(c) < target) {
      const long long t0 = clock64();
      unsigned int it = 0;
      while (ld_acquire(c) < target) {
        if ((++it & 63u) == 0) {
          if (*reinterpret_cast<volatile int*>(s.abort_flag)) { ok = 0; break; }
          if (clock64() - t0 > SPIN_LIMIT_CYCLES) {
            *reinterpret_cast<volatile int*>(s.abort_flag) = 1;
            *reinterpret_cast<volatile int*>(s.err) = 16;
            __threadfence_system();
            ok = 0;
            break;
          }
        }
      }
    }
    *smem_flag = ok;
  }
  __syncthreads();
  return *smem_flag != 0;
}

// All threads have issued their global writes for this step; publish them.
__device__ __forceinline__ void signal_group(const Sync& s, int bs) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    atomicAdd(s.ctr + bs * 32, 1u);
  }
}

// ---------------------------------------------------------------------------------------
// Forward
// ---------------------------------------------------------------------------------------
struct FwdParams {
  int T, N, H, nHS, MT, training, has_zoneout;
  float zoneout_prob;
  const void* R;     // [H, G*H]
  const void* b;     // LSTM: b [4H];  GRU: bx [3H]
  const void* b2;    // GRU: br [3H]
  const void* Wx;    // [T, N, G*H] input projection (LSTM: aliases v)
  void* h;           // [T+1, N, H]
  void* c;           // LSTM only
  void* v;           // gate cache [T, N, 4H] (may be null when not training, GRU)
  const void* mask;  // [T, N, H]
  Sync sync;
  int dbg;           // timing experiments only (wrong results): 1 no waits, 2 no MMA, 4 no h load
};

template <int G, int KSW, int SPLIT, typename T>
__global__ void __launch_bounds__(THREADS, 1) rec_fwd_kernel(const FwdParams p) {
  constexpr int COLS = G * U;            // gate columns owned by the CTA
  constexpr int NT = COLS / 8;           // n-tiles
  constexpr int KPAD = WARPS * KSW * 16; // padded K
  constexpr int AROW = KPAD + 8;         // bf16 elements per smem row (16 B pad: no conflicts)
  constexpr int PROW = COLS + 8;         // floats per partial row
  extern __shared__ __align__(16) uint8_t smem[];
  const int BNR = p.MT * 16;
  __nv_bfloat16* a_hi = reinterpret_cast<__nv_bfloat16*>(smem);
  __nv_bfloat16* a_lo = a_hi + (SPLIT == 2 ? (size_t)BNR * AROW : 0);
  float* part = reinterpret_cast<float*>(smem + (size_t)SPLIT * BNR * AROW * 2);
  __shared__ int s_flag;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int gq = lane >> 2, q = lane & 3;
  const int hs = blockIdx.x % p.nHS, bs = blockIdx.x / p.nHS;
  const int u0 = hs * U, n0 = bs * BNR;
  const int H = p.H, N = p.N;
  const long long NH = (long long)N * H;
  const int GH = G * H;

  // ---- recurrent weights -> registers (B fragments), once
  uint32_t rf[SPLIT][NT][KSW][2];
  {
    const T* R = reinterpret_cast<const T*>(p.R);
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const int cl = nt * 8 + gq;              // local column, ordered unit-major: cl = u*G + gate
      const int u = cl / G, gate = cl % G;
      const bool col_ok = (u0 + u) < H;
      const long long col = (long long)gate * H + u0 + u;
#pragma unroll
      for (int ks = 0; ks < KSW; ++ks) {
        const int kb = (warp * KSW + ks) * 16 + 2 * q;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          float x0 = 0.f, x1 = 0.f;
          const int k = kb + half * 8;
          if (col_ok && k < H) x0 = ld(R + (long long)k * GH + col);
          if (col_ok && k + 1 < H) x1 = ld(R + (long long)(k + 1) * GH + col);
          if (SPLIT == 2) {
            float h0, l0, h1, l1;
            split_bf16(x0, h0, l0);
            split_bf16(x1, h1, l1);
            rf[0][nt][ks][half] = pack_bf16(h0, h1);
            rf[SPLIT - 1][nt][ks][half] = pack_bf16(l0, l1);
          } else {
            rf[0][nt][ks][half] = pack_bf16(x0, x1);
          }
        }
      }
    }
  }

  // ---- pointwise ownership: thread -> (row nl of each m-tile, unit ul)
  const int nl = tid >> 4, ul = tid & 15;
  const bool unit_ok = (u0 + ul) < H;
  T* hbuf = reinterpret_cast<T*>(p.h);
  T* cbuf = reinterpret_cast<T*>(p.c);
  T* vbuf = reinterpret_cast<T*>(p.v);
  const T* wx = reinterpret_cast<const T*>(p.Wx);
  const T* mask = reinterpret_cast<const T*>(p.mask);
  float bias[G], bias2[G];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    bias[g] = unit_ok ? ld(reinterpret_cast<const T*>(p.b) + g * H + u0 + ul) : 0.f;
    bias2[g] = (G == 3 && unit_ok) ? ld(reinterpret_cast<const T*>(p.b2) + g * H + u0 + ul) : 0.f;
  }
  float c_reg[MAX_MT], h_reg[MAX_MT];
#pragma unroll
  for (int mt = 0; mt < MAX_MT; ++mt) {
    const int n = n0 + mt * 16 + nl;
    const bool ok = mt < p.MT && n < N && unit_ok;
    h_reg[mt] = ok ? ld(hbuf + (long long)n * H + u0 + ul) : 0.f;
    c_reg[mt] = (G == 4 && ok) ? ld(cbuf + (long long)n * H + u0 + ul) : 0.f;
  }

  for (int t = 0; t < p.T; ++t) {
    // ---- loads that do not depend on the recurrence: x.W (+ zoneout mask)
    float wxr[MAX_MT][G], mk[MAX_MT];
#pragma unroll
    for (int mt = 0; mt < MAX_MT; ++mt) {
      const int n = n0 + mt * 16 + nl;
      const bool ok = mt < p.MT && n < N && unit_ok;
#pragma unroll
      for (int g = 0; g < G; ++g)
        wxr[mt][g] = ok ? ld(wx + ((long long)t * N + n) * GH + g * H + u0 + ul) : 0.f;
      mk[mt] = (ok && p.has_zoneout && p.training)
                   ? ld(mask + (long long)t * NH + (long long)n * H + u0 + ul) : 0.f;
    }

    // ---- wait until every CTA of this batch slice has published h_t
    if (t > 0 && !(p.dbg & 1)) {
      if (!wait_group(p.sync, bs, (unsigned int)p.nHS * t, &s_flag)) break;
    }

    // ---- h_t rows of this batch slice -> shared memory (bf16 planes).  All loads of an
    // m-tile are issued before any is consumed, so their L2 latencies overlap.
    if (!(p.dbg & 4)) {
      const T* hsrc = hbuf + (long long)t * NH;
      constexpr int CPR = KPAD / 4;           // 4-element chunks per row
      constexpr int CPT = 16 * CPR / THREADS; // chunks per thread per m-tile
      const bool vec_ok = (H & 3) == 0;
      for (int mt = 0; mt < p.MT; ++mt) {
        float x[CPT][4];
#pragma unroll
        for (int i = 0; i < CPT; ++i) {
          const int e = tid + i * THREADS;
          const int r = mt * 16 + e / CPR, kc = (e % CPR) * 4;
          const int n = n0 + r;
          x[i][0] = x[i][1] = x[i][2] = x[i][3] = 0.f;
          if (n < N && kc < H) {
            const T* src = hsrc + (long long)n * H + kc;
            if (vec_ok) {
              if (sizeof(T) == 4) {
                const float4 f = __ldcg(reinterpret_cast<const float4*>(src));
                x[i][0] = f.x; x[i][1] = f.y; x[i][2] = f.z; x[i][3] = f.w;
              } else {
                const uint2 w2 = __ldcg(reinterpret_cast<const uint2*>(src));
                const __nv_bfloat162 p0 = *reinterpret_cast<const __nv_bfloat162*>(&w2.x);
                const __nv_bfloat162 p1 = *reinterpret_cast<const __nv_bfloat162*>(&w2.y);
                x[i][0] = __low2float(p0); x[i][1] = __high2float(p0);
                x[i][2] = __low2float(p1); x[i][3] = __high2float(p1);
              }
            } else {
#pragma unroll
              for (int j = 0; j < 4; ++j)
                if (kc + j < H) x[i][j] = ldcg(src + j);
            }
          }
        }
#pragma unroll
        for (int i = 0; i < CPT; ++i) {
          const int e = tid + i * THREADS;
          const int r = mt * 16 + e / CPR, kc = (e % CPR) * 4;
          uint2 hi2;
          if (SPLIT == 2) {
            float hi[4], lo[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) split_bf16(x[i][j], hi[j], lo[j]);
            hi2 = make_uint2(pack_bf16(hi[0], hi[1]), pack_bf16(hi[2], hi[3]));
            *reinterpret_cast<uint2*>(a_lo + (size_t)r * AROW + kc) =
                make_uint2(pack_bf16(lo[0], lo[1]), pack_bf16(lo[2], lo[3]));
          } else {
            hi2 = make_uint2(pack_bf16(x[i][0], x[i][1]), pack_bf16(x[i][2], x[i][3]));
          }
          *reinterpret_cast<uint2*>(a_hi + (size_t)r * AROW + kc) = hi2;
        }
      }
    }
    __syncthreads();

    for (int mt = 0; mt < p.MT; ++mt) {
      // ---- this warp's K range of the step product
      float acc[NT][4];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
      if (!(p.dbg & 2))
#pragma unroll
      for (int ks = 0; ks < KSW; ++ks) {
        const int row = mt * 16 + (lane & 15);
        const int kcol = (warp * KSW + ks) * 16 + (lane >> 4) * 8;
        uint32_t ah[4], al[4];
        ldmatrix_x4(smem_u32(a_hi + (size_t)row * AROW + kcol), ah);
        if (SPLIT == 2) ldmatrix_x4(smem_u32(a_lo + (size_t)row * AROW + kcol), al);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          mma_bf16(acc[nt], ah, rf[0][nt][ks][0], rf[0][nt][ks][1]);
          if (SPLIT == 2) {
            mma_bf16(acc[nt], ah, rf[SPLIT - 1][nt][ks][0], rf[SPLIT - 1][nt][ks][1]);
            mma_bf16(acc[nt], al, rf[0][nt][ks][0], rf[0][nt][ks][1]);
          }
        }
      }
      float* pw = part + (size_t)warp * 16 * PROW;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        *reinterpret_cast<float2*>(pw + gq * PROW + nt * 8 + 2 * q) =
            make_float2(acc[nt][0], acc[nt][1]);
        *reinterpret_cast<float2*>(pw + (gq + 8) * PROW + nt * 8 + 2 * q) =
            make_float2(acc[nt][2], acc[nt][3]);
      }
      __syncthreads();

      // ---- pointwise stage for (row nl of m-tile mt, unit ul)
      {
        float rh[G];
#pragma unroll
        for (int g = 0; g < G; ++g) rh[g] = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
          const float* src = part + ((size_t)w * 16 + nl) * PROW + ul * G;
          if (G == 4) {
            const float4 f = *reinterpret_cast<const float4*>(src);
            rh[0] += f.x; rh[1] += f.y; rh[2] += f.z; rh[G - 1] += f.w;
          } else {
#pragma unroll
            for (int g = 0; g < G; ++g) rh[g] += src[g];
          }
        }
        const int n = n0 + mt * 16 + nl;
        if (n < N && unit_ok) {
          // select this m-tile's registers without dynamic indexing
          float hp = 0.f, cp = 0.f, m = 0.f, wv[G];
#pragma unroll
          for (int k = 0; k < MAX_MT; ++k)
            if (k == mt) {
              hp = h_reg[k]; cp = c_reg[k]; m = mk[k];
#pragma unroll
              for (int g = 0; g < G; ++g) wv[g] = wxr[k][g];
            }
          const long long o0 = (long long)n * H + u0 + ul;
          float h_new, c_new = 0.f;
          if (G == 4) {
            const float i = sigmoidf_(wv[0] + rh[0] + bias[0]);
            const float g = tanhf(wv[1] + rh[1] + bias[1]);
            const float f = sigmoidf_(wv[2] + rh[2] + bias[2]);
            const float o = sigmoidf_(wv[G - 1] + rh[G - 1] + bias[G - 1]);
            if (p.training) {
              T* vt = vbuf + ((long long)t * N + n) * GH + u0 + ul;
              st(vt, i); st(vt + H, g); st(vt + 2 * H, f); st(vt + 3 * H, o);
            }
            c_new = f * cp + i * g;
            h_new = o * tanhf(c_new);
            st(cbuf + (long long)(t + 1) * NH + o0, c_new);
          } else {
            const float z = sigmoidf_(wv[0] + rh[0] + bias[0] + bias2[0]);
            const float r = sigmoidf_(wv[1] + rh[1] + bias[1] + bias2[1]);
            const float qg = rh[2] + bias2[2];
            const float g = tanhf(wv[2] + r * qg + bias[2]);
            if (p.training && vbuf) {
              T* vt = vbuf + ((long long)t * N + n) * 4 * H + u0 + ul;
              st(vt, z); st(vt + H, r); st(vt + 2 * H, g); st(vt + 3 * H, qg);
            }
            h_new = z * hp + (1.0f - z) * g;
          }
          if (p.has_zoneout) {
            h_new = p.training ? zoneout<true>(h_new, hp, p.zoneout_prob, m)
                               : zoneout<false>(h_new, hp, p.zoneout_prob, m);
          }
          st(hbuf + (long long)(t + 1) * NH + o0, h_new);
          // carry what the next step will actually read back (bf16 storage rounds h)
          if (is_bf16<T>::value) h_new = __bfloat162float(__float2bfloat16_rn(h_new));
#pragma unroll
          for (int k = 0; k < MAX_MT; ++k)
            if (k == mt) { h_reg[k] = h_new; c_reg[k] = c_new; }
        }
      }
      __syncthreads();  // `part` is reused by the next m-tile / step
    }
    if (t + 1 < p.T && !(p.dbg & 1)) signal_group(p.sync, bs);
  }
}

// ---------------------------------------------------------------------------------------
// Backward
// ---------------------------------------------------------------------------------------
struct BwdParams {
  int T, N, H, nHS, MT, has_zoneout, r_transposed;
  const void* R;        // [H, G*H], or R_t [G*H, H] when r_transposed
  const void* h;        // [T+1, N, H]
  const void* c;        // LSTM
  void* v;              // LSTM: gate cache in, gate gradients out.  GRU: cache in
  const void* dh_new;   // [T+1, N, H]
  const void* dc_new;   // LSTM
  void* dp;             // GRU out [T, N, 3H]
  void* dq;             // GRU out [T, N, 3H]
  const void* mask;
  float* dh_carry;      // [N, H] in/out
  float* dc_carry;      // LSTM
  float* exch;          // [2][nBS][nHS(dest)][nHS(src)][16*MT rows][U] partial dh
  Sync sync;
};

template <int G, int NTW, int SPLIT, typename T>
__global__ void __launch_bounds__(THREADS, 1) rec_bwd_kernel(const BwdParams p) {
  constexpr int COLS = G * U;                 // K of the step product
  constexpr int KS = (COLS + 15) / 16;        // k-steps (LSTM 4, GRU 3)
  constexpr int KPAD = KS * 16;
  constexpr int AROW = KPAD + 8;
  extern __shared__ __align__(16) uint8_t smem[];
  const int BNR = p.MT * 16;
  __nv_bfloat16* a_hi = reinterpret_cast<__nv_bfloat16*>(smem);
  __nv_bfloat16* a_lo = a_hi + (SPLIT == 2 ? (size_t)BNR * AROW : 0);
  __shared__ int s_flag;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int gq = lane >> 2, q = lane & 3;
  const int hs = blockIdx.x % p.nHS, bs = blockIdx.x / p.nHS;
  const int nBS = gridDim.x / p.nHS;
  const int u0 = hs * U, n0 = bs * BNR;
  const int H = p.H, N = p.N;
  const long long NH = (long long)N * H;
  const int GH = G * H;

  // ---- R[:, slice]^T as B fragments: B(k = local gate column, n = output unit j)
  // Output units j in [warp*NTW*8, (warp+1)*NTW*8).
  uint32_t rf[SPLIT][NTW][KS][2];
  {
    const T* R = reinterpret_cast<const T*>(p.R);
#pragma unroll
    for (int nt = 0; nt < NTW; ++nt) {
      const int j = (warp * NTW + nt) * 8 + gq;
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          float x[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int cl = ks * 16 + half * 8 + 2 * q + e;  // local gate column = u*G + gate
            const int u = cl / G, gate = cl % G;
            float val = 0.f;
            if (cl < COLS && j < H && (u0 + u) < H) {
              const long long col = (long long)gate * H + u0 + u;
              val = p.r_transposed ? ld(R + col * H + j) : ld(R + (long long)j * GH + col);
            }
            x[e] = val;
          }
          if (SPLIT == 2) {
            float h0, l0, h1, l1;
            split_bf16(x[0], h0, l0);
            split_bf16(x[1], h1, l1);
            rf[0][nt][ks][half] = pack_bf16(h0, h1);
            rf[SPLIT - 1][nt][ks][half] = pack_bf16(l0, l1);
          } else {
            rf[0][nt][ks][half] = pack_bf16(x[0], x[1]);
          }
        }
      }
    }
  }

  const int nl = tid >> 4, ul = tid & 15;
  const bool unit_ok = (u0 + ul) < H;
  const T* hbuf = reinterpret_cast<const T*>(p.h);
  const T* cbuf = reinterpret_cast<const T*>(p.c);
  T* vbuf = reinterpret_cast<T*>(p.v);
  const T* dhn = reinterpret_cast<const T*>(p.dh_new);
  const T* dcn = reinterpret_cast<const T*>(p.dc_new);
  const T* mask = reinterpret_cast<const T*>(p.mask);
  T* dpb = reinterpret_cast<T*>(p.dp);
  T* dqb = reinterpret_cast<T*>(p.dq);

  float dh_c[MAX_MT], dc_c[MAX_MT];
#pragma unroll
  for (int mt = 0; mt < MAX_MT; ++mt) {
    const int n = n0 + mt * 16 + nl;
    const bool ok = mt < p.MT && n < N && unit_ok;
    dh_c[mt] = ok ? p.dh_carry[(long long)n * H + u0 + ul] : 0.f;
    dc_c[mt] = (G == 4 && ok) ? p.dc_carry[(long long)n * H + u0 + ul] : 0.f;
  }
  const size_t blk = (size_t)BNR * U;  // floats per (dest, src) exchange block
  bool alive = true;

  for (int t = p.T - 1; t >= 0; --t) {
    // ---- loads independent of the carried gradient
    float gv[MAX_MT][4], cprev[MAX_MT], cnew[MAX_MT], dhv[MAX_MT], dcv[MAX_MT], mk[MAX_MT],
        hprev[MAX_MT];
#pragma unroll
    for (int mt = 0; mt < MAX_MT; ++mt) {
      const int n = n0 + mt * 16 + nl;
      const bool ok = mt < p.MT && n < N && unit_ok;
      const long long o0 = (long long)n * H + u0 + ul;
      const T* vt = vbuf + ((long long)t * N + n) * 4 * H + u0 + ul;
#pragma unroll
      for (int g = 0; g < 4; ++g) gv[mt][g] = ok ? ld(vt + g * H) : 0.f;
      dhv[mt] = ok ? ld(dhn + (long long)(t + 1) * NH + o0) : 0.f;
      mk[mt] = (ok && p.has_zoneout) ? ld(mask + (long long)t * NH + o0) : 1.f;
      if (G == 4) {
        cprev[mt] = ok ? ld(cbuf + (long long)t * NH + o0) : 0.f;
        cnew[mt] = ok ? ld(cbuf + (long long)(t + 1) * NH + o0) : 0.f;
        dcv[mt] = ok ? ld(dcn + (long long)(t + 1) * NH + o0) : 0.f;
        hprev[mt] = 0.f;
      } else {
        hprev[mt] = ok ? ld(hbuf + (long long)t * NH + o0) : 0.f;
        cprev[mt] = cnew[mt] = dcv[mt] = 0.f;
      }
    }

    // ---- recurrent part of dh_t: sum of the partials published at step t+1
    if (t < p.T - 1) {
      if (!wait_group(p.sync, bs, (unsigned int)p.nHS * (p.T - 1 - t), &s_flag)) {
        alive = false;
        break;
      }
      const int par = (t + 1) & 1;
      const float* src = p.exch + (((size_t)par * nBS + bs) * p.nHS + hs) * p.nHS * blk;
#pragma unroll
      for (int mt = 0; mt < MAX_MT; ++mt) {
        if (mt < p.MT) {
          float s = 0.f;
          const float* q0 = src + (size_t)(mt * 16 + nl) * U + ul;
          // 8 loads in flight per pass; the summation order is fixed by this code
          for (int s0 = 0; s0 < p.nHS; s0 += 8) {
            float a[8];
#pragma unroll
            for (int k = 0; k < 8; ++k)
              a[k] = (s0 + k < p.nHS) ? __ldcg(q0 + (size_t)(s0 + k) * blk) : 0.f;
            s += ((a[0] + a[1]) + (a[2] + a[3])) + ((a[4] + a[5]) + (a[6] + a[7]));
          }
          dh_c[mt] += s;
        }
      }
    }

    // ---- pointwise gradients; gate gradients -> global and -> smem (A operand)
#pragma unroll
    for (int mt = 0; mt < MAX_MT; ++mt) {
      if (mt < p.MT) {
        const int n = n0 + mt * 16 + nl;
        const bool ok = n < N && unit_ok;
        float dgate[G];
        float dh_total = dhv[mt] + dh_c[mt];
        float keep = 0.f;
        if (p.has_zoneout) {
          keep = (1.0f - mk[mt]) * dh_total;
          dh_total = mk[mt] * dh_total;
        }
        if (G == 4) {
          const float i = gv[mt][0], g = gv[mt][1], f = gv[mt][2], o = gv[mt][3];
          const float c_tanh = tanhf(cnew[mt]);
          float dc_total = dcv[mt] + dc_c[mt];
          const float d_o = c_tanh * dh_total;
          dc_total += d_tanh(c_tanh) * (o * dh_total);
          dgate[0] = d_sigmoid(i) * (g * dc_total);
          dgate[1] = d_tanh(g) * (i * dc_total);
          dgate[2] = d_sigmoid(f) * (cprev[mt] * dc_total);
          dgate[G - 1] = d_sigmoid(o) * d_o;
          dc_c[mt] = f * dc_total;
          dh_c[mt] = keep;
          if (ok) {
            T* vt = vbuf + ((long long)t * N + n) * 4 * H + u0 + ul;
#pragma unroll
            for (int g4 = 0; g4 < 4; ++g4) st(vt + g4 * H, dgate[g4 % G]);
          }
        } else {
          const float z = gv[mt][0], r = gv[mt][1], g = gv[mt][2], qg = gv[mt][3];
          const float dg = (1.0f - z) * dh_total;
          const float dz = (hprev[mt] - g) * dh_total;
          const float dp_g = d_tanh(g) * dg;
          const float dp_r = d_sigmoid(r) * (dp_g * qg);
          const float dp_z = d_sigmoid(z) * dz;
          dgate[0] = dp_z;
          dgate[1] = dp_r;
          dgate[2] = dp_g * r;  // dq
          dh_c[mt] = keep + z * dh_total;
          if (ok) {
            const long long w0 = ((long long)t * N + n) * 3 * H + u0 + ul;
            st(dpb + w0, dp_z); st(dpb + w0 + H, dp_r); st(dpb + w0 + 2 * H, dp_g);
            st(dqb + w0, dp_z); st(dqb + w0 + H, dp_r); st(dqb + w0 + 2 * H, dgate[2]);
          }
        }
        // A operand row (mt*16+nl), columns ul*G .. ul*G+G-1
        __nv_bfloat16* rowh = a_hi + (size_t)(mt * 16 + nl) * AROW + ul * G;
        __nv_bfloat16* rowl = a_lo + (size_t)(mt * 16 + nl) * AROW + ul * G;
#pragma unroll
        for (int g = 0; g < G; ++g) {
          const float x = ok ? dgate[g] : 0.f;
          if (SPLIT == 2) {
            float hi, lo;
            split_bf16(x, hi, lo);
            rowh[g] = __float2bfloat16_rn(hi);
            rowl[g] = __float2bfloat16_rn(lo);
          } else {
            rowh[g] = __float2bfloat16_rn(x);
          }
        }
      }
    }
    if (t == 0) break;  // nobody consumes partials of the last step
    __syncthreads();

    // ---- partial dh_{t-1}[rows, all units] = dG . R[:, slice]^T, warp owns NTW*8 units
    {
      const int par = t & 1;
      float* dstbase = p.exch + ((size_t)par * nBS + bs) * p.nHS * p.nHS * blk;
      for (int mt = 0; mt < p.MT; ++mt) {
        float acc[NTW][4];
#pragma unroll
        for (int nt = 0; nt < NTW; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
          const int row = mt * 16 + (lane & 15);
          const int kcol = ks * 16 + (lane >> 4) * 8;
          uint32_t ah[4], al[4];
          ldmatrix_x4(smem_u32(a_hi + (size_t)row * AROW + kcol), ah);
          if (SPLIT == 2) ldmatrix_x4(smem_u32(a_lo + (size_t)row * AROW + kcol), al);
#pragma unroll
          for (int nt = 0; nt < NTW; ++nt) {
            mma_bf16(acc[nt], ah, rf[0][nt][ks][0], rf[0][nt][ks][1]);
            if (SPLIT == 2) {
              mma_bf16(acc[nt], ah, rf[SPLIT - 1][nt][ks][0], rf[SPLIT - 1][nt][ks][1]);
              mma_bf16(acc[nt], al, rf[0][nt][ks][0], rf[0][nt][ks][1]);
            }
          }
        }
#pragma unroll
        for (int nt = 0; nt < NTW; ++nt) {
          const int j = (warp * NTW + nt) * 8 + 2 * q;  // output unit of acc[.][0]
          if (j < H) {
            const int dest = j / U, uj = j % U;
            float* d = dstbase + ((size_t)dest * p.nHS + hs) * blk + (size_t)(mt * 16) * U + uj;
            __stcg(reinterpret_cast<float2*>(d + (size_t)gq * U), make_float2(acc[nt][0], acc[nt][1]));
            __stcg(reinterpret_cast<float2*>(d + (size_t)(gq + 8) * U),
                   make_float2(acc[nt][2], acc[nt][3]));
          }
        }
      }
    }
    signal_group(p.sync, bs);  // includes the __syncthreads that protects the A planes
  }

  // ---- carries out.  After the last step dh_c holds only the zoneout / GRU direct part
  // of dh_0; the recurrent part of that step is added by the host-issued contraction.
  if (alive) {
#pragma unroll
    for (int mt = 0; mt < MAX_MT; ++mt) {
      const int n = n0 + mt * 16 + nl;
      if (mt < p.MT && n < N && unit_ok) {
        p.dh_carry[(long long)n * H + u0 + ul] = dh_c[mt];
        if (G == 4) p.dc_carry[(long long)n * H + u0 + ul] = dc_c[mt];
      }
    }
  }
}

// ---------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------
struct Geometry {
  int nHS, nBS, MT;
};

int sm_count() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

// Picks the batch tiling: as many CTAs as fit on the GPU at once (one CTA per SM).
bool pick_geometry(int N, int H, Geometry* g) {
  const int nHS = ceil_div(H, U);
  const int sms = sm_count();
  for (int mt = 1; mt <= MAX_MT; ++mt) {
    const int nBS = ceil_div(N, 16 * mt);
    if ((long long)nHS * nBS <= sms) {
      g->nHS = nHS; g->nBS = nBS; g->MT = mt;
      return true;
    }
  }
  return false;
}

template <typename K>
int launch_coop(K kernel, int grid, size_t smem, void* params, cudaStream_t s) {
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return HASTE_B200_ERR_UNSUPPORTED;
  }
  int per_sm = 0;
  e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, THREADS, smem);
  if (e != cudaSuccess || per_sm * sm_count() < grid) {
    cudaGetLastError();
    return HASTE_B200_ERR_UNSUPPORTED;
  }
  void* args[] = {params};
  e = cudaLaunchCooperativeKernel((const void*)kernel, dim3(grid), dim3(THREADS), args, smem, s);
  if (e != cudaSuccess) {
    set_last_error("cooperative launch failed: %s", cudaGetErrorString(e));
    cudaGetLastError();
    return HASTE_B200_ERR_CUDA;
  }
  count_launch(1);
  return HASTE_B200_OK;
}

// Scratch for the step counters, the abort flag and the backward exchange buffers.
struct SyncMem {
  Sync sync;
  float* exch;
};
int make_sync(const Geometry& g, size_t exch_floats, SyncMem* out, cudaStream_t s) {
  Arena ws;
  const size_t ctr_bytes = Arena::pad((size_t)(g.nBS * 32 + 32) * 4);
  HB_TRY(make_arena(&ws, s, ctr_bytes + Arena::pad(exch_floats * 4) + 512, /*slot=*/2));
  unsigned int* ctr = ws.take<unsigned int>(g.nBS * 32 + 32);
  float* exch = ws.take<float>(exch_floats);
  HB_REQUIRE(ctr && (exch || !exch_floats), "scratch arena");
  HB_CUDA_OK(cudaMemsetAsync(ctr, 0, ctr_bytes, s));
  out->sync.ctr = ctr;
  out->sync.abort_flag = reinterpret_cast<int*>(ctr + g.nBS * 32);
  out->sync.err = device_error_word();
  HB_REQUIRE(out->sync.err, "error word");
  out->exch = exch;
  return HASTE_B200_OK;
}

template <int G, int SPLIT, typename T>
int run_fwd(FwdParams& p, const Geometry& g, cudaStream_t s) {
  const int H = p.H;
  const int ksteps = ceil_div(H, 16);
  const int ksw = ceil_div(ksteps, WARPS);
  auto smem_for = [&](int KSW) {
    const size_t arow = (size_t)WARPS * KSW * 16 + 8;
    return (size_t)SPLIT * g.MT * 16 * arow * 2 + (size_t)WARPS * 16 * (G * U + 8) * 4;
  };
  const int grid = g.nHS * g.nBS;
#define HB_FWD(KSW)                                                                       \
  if (ksw <= KSW) {                                                                       \
    if (smem_for(KSW) > 220 * 1024) return HASTE_B200_ERR_UNSUPPORTED;                    \
    return launch_coop(rec_fwd_kernel<G, KSW, SPLIT, T>, grid, smem_for(KSW), &p, s);     \
  }
  HB_FWD(1)
  HB_FWD(2)
  HB_FWD(4)
  if constexpr (SPLIT == 1) { HB_FWD(8) }
#undef HB_FWD
  return HASTE_B200_ERR_UNSUPPORTED;
}

template <int G, int SPLIT, typename T>
int run_bwd(BwdParams& p, const Geometry& g, cudaStream_t s) {
  const int ntw = ceil_div(ceil_div(p.H, 8), WARPS);  // n-tiles per warp
  const size_t arow = (size_t)((G * U + 15) / 16) * 16 + 8;
  const size_t smem = (size_t)SPLIT * g.MT * 16 * arow * 2;
  const int grid = g.nHS * g.nBS;
#define HB_BWD(NTW) \
  if (ntw <= NTW) return launch_coop(rec_bwd_kernel<G, NTW, SPLIT, T>, grid, smem, &p, s);
  HB_BWD(1)
  HB_BWD(2)
  HB_BWD(4)
  HB_BWD(8)
  if constexpr (SPLIT == 1) { HB_BWD(16) }
#undef HB_BWD
  return HASTE_B200_ERR_UNSUPPORTED;
}

bool path_allowed() { return recurrence_path() != HASTE_B200_PATH_STEPWISE; }

int debug_skip() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("HASTE_B200_DEBUG_SKIP");
    v = e ? atoi(e) : 0;
  }
  return v;
}

}  // namespace

int lstm_forward_persistent(const LstmFwd& a, cudaStream_t s) {
  Geometry g;
  if (!path_allowed() || !pick_geometry(a.N, a.H, &g)) return HASTE_B200_ERR_UNSUPPORTED;
  if (a.dtype == HASTE_B200_F32 && a.H > 512) return HASTE_B200_ERR_UNSUPPORTED;
  if (a.dtype == HASTE_B200_BF16 && a.H > 1024) return HASTE_B200_ERR_UNSUPPORTED;
  SyncMem sm;
  HB_TRY(make_sync(g, 0, &sm, s));
  const bool zo = a.zoneout_prob != 0.0f && a.zoneout_mask != nullptr;
  FwdParams p{a.T, a.N, a.H, g.nHS, g.MT, a.training, zo ? 1 : 0, a.zoneout_prob, a.R, a.b,
              nullptr, a.v, a.h, a.c, a.v, a.zoneout_mask, sm.sync, debug_skip()};
  if (a.dtype == HASTE_B200_F32) return run_fwd<4, 2, float>(p, g, s);
  return run_fwd<4, 1, __nv_bfloat16>(p, g, s);
}

int gru_forward_persistent(const GruFwd& a, cudaStream_t s) {
  Geometry g;
  if (!path_allowed() || !pick_geometry(a.N, a.H, &g)) return HASTE_B200_ERR_UNSUPPORTED;
  if (a.dtype == HASTE_B200_F32 && a.H > 512) return HASTE_B200_ERR_UNSUPPORTED;
  if (a.dtype == HASTE_B200_BF16 && a.H > 1024) return HASTE_B200_ERR_UNSUPPORTED;
  SyncMem sm;
  HB_TRY(make_sync(g, 0, &sm, s));
  const bool zo = a.zoneout_prob != 0.0f && a.zoneout_mask != nullptr;
  FwdParams p{a.T, a.N, a.H, g.nHS, g.MT, a.training, zo ? 1 : 0, a.zoneout_prob, a.R, a.bx,
              a.br, a.tmp_Wx, a.h, nullptr, a.v, a.zoneout_mask, sm.sync, debug_skip()};
  if (a.dtype == HASTE_B200_F32) return run_fwd<3, 2, float>(p, g, s);
  return run_fwd<3, 1, __nv_bfloat16>(p, g, s);
}

// The persistent backward kernels leave the recurrent contribution of the very last
// processed step (t = 0) out of dh (nothing inside the kernel consumes it); it is added
// here with one small contraction: dh += dG_0 . R^T.
int lstm_backward_persistent(const LstmBwd& a, float* dh_carry, float* dc_carry, cudaStream_t s) {
  Geometry g;
  if (!path_allowed() || !pick_geometry(a.N, a.H, &g)) return HASTE_B200_ERR_UNSUPPORTED;
  if (a.dtype == HASTE_B200_F32 && a.H > 512) return HASTE_B200_ERR_UNSUPPORTED;
  if (a.dtype == HASTE_B200_BF16 && a.H > 1024) return HASTE_B200_ERR_UNSUPPORTED;
  SyncMem sm;
  const size_t exch = (size_t)2 * g.nBS * g.nHS * g.nHS * g.MT * 16 * U;
  HB_TRY(make_sync(g, exch, &sm, s));
  BwdParams p{a.T, a.N, a.H, g.nHS, g.MT, a.zoneout_mask ? 1 : 0, a.transposed_inputs, a.R, a.h,
              a.c, a.v, a.dh_new, a.dc_new, nullptr, nullptr, a.zoneout_mask, dh_carry, dc_carry,
              sm.exch, sm.sync};
  int st_ = (a.dtype == HASTE_B200_F32) ? run_bwd<4, 2, float>(p, g, s)
                                        : run_bwd<4, 1, __nv_bfloat16>(p, g, s);
  if (st_ != HASTE_B200_OK) return st_;
  const int H = a.H;
  GemmDesc gd{a.dtype, HASTE_B200_F32, a.N, H, 4 * H, a.v, 4LL * H, 1, a.R,
              a.transposed_inputs ? H : 1, a.transposed_inputs ? 1 : 4LL * H, dh_carry, H, 1};
  return gemm_small(gd, s);
}

int gru_backward_persistent(const GruBwd& a, float* dh_carry, cudaStream_t s) {
  Geometry g;
  if (!path_allowed() || !pick_geometry(a.N, a.H, &g)) return HASTE_B200_ERR_UNSUPPORTED;
  if (a.dtype == HASTE_B200_F32 && a.H > 512) return HASTE_B200_ERR_UNSUPPORTED;
  if (a.dtype == HASTE_B200_BF16 && a.H > 1024) return HASTE_B200_ERR_UNSUPPORTED;
  SyncMem sm;
  const size_t exch = (size_t)2 * g.nBS * g.nHS * g.nHS * g.MT * 16 * U;
  HB_TRY(make_sync(g, exch, &sm, s));
  BwdParams p{a.T, a.N, a.H, g.nHS, g.MT, a.zoneout_mask ? 1 : 0, a.transposed_inputs, a.R, a.h,
              nullptr, const_cast<void*>(a.v), a.dh_new, nullptr, a.dp, a.dq, a.zoneout_mask,
              dh_carry, nullptr, sm.exch, sm.sync};
  int st_ = (a.dtype == HASTE_B200_F32) ? run_bwd<3, 2, float>(p, g, s)
                                        : run_bwd<3, 1, __nv_bfloat16>(p, g, s);
  if (st_ != HASTE_B200_OK) return st_;
  const int H = a.H;
  GemmDesc gd{a.dtype, HASTE_B200_F32, a.N, H, 3 * H, a.dq, 3LL * H, 1, a.R,
              a.transposed_inputs ? H : 1, a.transposed_inputs ? 1 : 3LL * H, dh_carry, H, 1};
  return gemm_small(gd, s);
}

}  // namespace hb
