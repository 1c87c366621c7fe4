// Persistent recurrence kernels for LSTM and GRU (forward and backward), sm_100a.
//
// One cooperative launch covers all T steps of a layer pass; nothing is launched per
// time step.  The grid is (hidden slices) x (batch slices).  A CTA owns U = 16 hidden
// units (all G gates of them) for up to 64 batch rows and keeps its slice of the
// recurrent matrix R in REGISTERS, as ready-made mma.sync B-fragments, for the whole
// kernel: R is read from HBM exactly once per pass.
//
//   forward : gates[rows, G*U] = h_{t-1}[rows, :] . R[:, slice]       (K = H)
//             The K range is split over the 8 warps: a warp fetches only its own K range
//             of h_{t-1}, multiplies it against all of the CTA's columns and leaves a
//             partial tile in shared memory; the pointwise stage sums the 8 partials, adds
//             x.W + b, applies the nonlinearities, zoneout and the c/h update, and writes
//             h_t, c_t and the gate cache.
//   backward: dh_{t-1}[rows, :] += dG_t[rows, slice] . R[:, slice]^T   (K = G*U)
//             Each CTA turns its own gate gradients into a partial dh for ALL hidden units
//             (output columns split over the warps); partials travel through a
//             double-buffered exchange area and are summed, in a fixed order, by the CTA
//             that owns the unit.  dh/dc carries live in registers.
//
// fp32 storage: operands are split into bf16 (hi, lo) pairs and three products
// (hi.hi, hi.lo, lo.hi) are accumulated in fp32, which keeps the step product within
// ~1e-5 of fp32 arithmetic.  bf16 storage: one product.
//
// Step-to-step data flow carries its own readiness: everything a CTA hands to another
// CTA is written as 32-bit words that hold the value and a tag that alternates every time
// a buffer is reused.  h_t (forward) travels as a bf16 (hi, lo) pair - the consumer copies the
// halves straight into its operand planes - with the tag in bit 14 of the lo half, always
// zero for a genuine lo, whose magnitude is below 2^-8 of the value; partial dh (backward)
// travels as fp32 with the tag in the lowest mantissa bit.  A consumer simply re-reads a word until the
// tag is the one it expects.  There is no counter, no fence and no grid-wide barrier on
// the critical path, and 32-bit stores cannot tear.  CTAs of different batch slices never
// touch each other's data.
//
// Every wait is bounded: when the limit runs out the warp raises the CTA's and the
// grid's abort flags and the process error word; all CTAs leave their loops and the host
// reports HASTE_B200_ERR_TIMEOUT.  The launch is cooperative, so all CTAs are co-resident.
//
// Replaces the per-step cuBLAS call + pointwise kernel of the reference
// (lib/lstm_forward_gpu.cu.cc:210-310, lib/lstm_backward_gpu.cu.cc:246-316,
//  lib/gru_forward_gpu.cu.cc:214-308, lib/gru_backward_gpu.cu.cc:252-320).
#pragma once

#include "cells.cuh"

namespace hb {
namespace rec {

constexpr int U = 16;          // hidden units per CTA
constexpr int WARPS = 8;
constexpr int THREADS = WARPS * 32;
constexpr long long SPIN_LIMIT_CYCLES = 4000000000LL;

// Timing experiments (attributing step time to waits, contraction, prefetch) are compiled in
// only with -DHASTE_B200_TIMING_EXPERIMENTS; the shipped kernels carry none of their branches.
#ifdef HASTE_B200_TIMING_EXPERIMENTS
#define HB_DBG(p, bit) (((p).dbg & (bit)) != 0)
#else
#define HB_DBG(p, bit) false
#endif

struct Sync {
  int* abort_flag;  // device-global
  int* err;         // process error word (pinned host memory)
};

struct FwdParams {
  int T, N, H, Hx, nHS, MT, training, has_zoneout;
  float zoneout_prob;
  const void* R;     // [H, G*H]
  const void* b;     // LSTM: b [4H];  GRU: bx [3H]
  const void* b2;    // GRU: br [3H]
  const void* Wx;    // [T, N, G*H] input projection (LSTM: aliases v)
  void* h;           // [T+1, N, H]
  void* c;           // LSTM only
  void* v;           // gate cache [T, N, 4H] (may be null when not training, GRU)
  const void* mask;  // [T, N, H]
  uint32_t* xbuf;    // [2][N][Hx] tagged exchange words, zeroed before launch
  Sync sync;
  int dbg;           // read only in timing-experiment builds (see HB_DBG): 1 no waits, 2 no MMA
};

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
  uint32_t* exch;       // [2][nBS][nHS(dest)][nHS(src)][16*MT rows][U] tagged partial dh
  Sync sync;
  int dbg;
  // fp32 storage, optional: the gate gradients also as bf16 (hi, lo) planes, hi at gpl and lo
  // gpl_stride elements later, laid out like v / dp (gpl) and dq (gpl2), so that the
  // contractions that follow do not have to split them again.
  __nv_bfloat16* gpl;
  __nv_bfloat16* gpl2;
  long long gpl_stride;
  // Bias gradients: every thread sums its gate gradients over all steps in registers and leaves
  // them here as [nBS*16 rows][4H] partials - LSTM (di, dg, df, do); GRU (dp_z, dp_r, dp_g,
  // dq_g) - which the host reduces over 16*nBS rows instead of over T*N rows of the gradients.
  float* db_part;
};

// ---------------------------------------------------------------------------------------
// device helpers
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo_elem, float hi_elem) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo_elem, hi_elem);  // .x = lower address
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
__device__ __forceinline__ float ldcg_f(const float* p) { return __ldcg(p); }
__device__ __forceinline__ float ldcg_f(const __nv_bfloat16* p) {
  return __bfloat162float(__ldcg(p));
}

// Polling loads: relaxed, gpu scope, so that every poll is served by L2.
__device__ __forceinline__ uint32_t ld_relaxed_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_relaxed_u32x4(const uint32_t* p) {
  uint4 v;
  asm volatile("ld.relaxed.gpu.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

__device__ __forceinline__ void prefetch_l2(const void* p) {
  asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
}

// Publishing stores of the exchange: `volatile` with a memory clobber, so that the compiler
// issues them exactly where they are written - ahead of the bulky activation stores of the same
// stage, never behind them.  .cg: the word goes to L2, where the consumers poll.
__device__ __forceinline__ void publish_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.global.cg.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void publish_u32x2(uint32_t* p, uint32_t a, uint32_t b) {
  asm volatile("st.global.cg.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(a), "r"(b) : "memory");
}

// Exchange word: bits 0-15 hi (bf16), bits 16-31 lo (bf16) with bit 30 replaced by `tag`.
__device__ __forceinline__ uint32_t xword_encode(float x, uint32_t tag) {
  float hi, lo;
  split_bf16(x, hi, lo);
  if (!(fabsf(lo) < 1.0f)) lo = 0.0f;  // NaN/Inf/huge values travel in hi alone
  return (pack_bf16(hi, lo) & 0xBFFFFFFFu) | (tag << 30);
}
__device__ __forceinline__ float xword_value(uint32_t w) {
  return __uint_as_float(w << 16) + __uint_as_float(w & 0xBFFF0000u);
}
__device__ __forceinline__ bool xword_ready(uint32_t w, uint32_t tag) {
  return ((w >> 30) & 1u) == tag;
}

// Tagged fp32 word: the value with its lowest mantissa bit replaced by the tag (22 explicit
// mantissa bits survive).  One logic instruction to encode or decode; used wherever the
// consumer wants the number itself rather than ready-made bf16 planes.
__device__ __forceinline__ uint32_t fword_encode(float x, uint32_t tag) {
  return (__float_as_uint(x) & ~1u) | tag;
}
__device__ __forceinline__ float fword_value(uint32_t w) { return __uint_as_float(w & ~1u); }
__device__ __forceinline__ bool fword_ready(uint32_t w, uint32_t tag) { return (w & 1u) == tag; }

// Fast gate functions (ex2.approx based): error ~1e-6 absolute, far inside the parity bar.
__device__ __forceinline__ float sigmoid_fast(float x) {
  return __fdividef(1.0f, 1.0f + __expf(-x));
}
__device__ __forceinline__ float tanh_fast(float x) {
  // 1 - 2/(1+e^{2x}); clamp keeps e^{2x} finite
  const float e = __expf(2.0f * fminf(fmaxf(x, -15.0f), 15.0f));
  return 1.0f - __fdividef(2.0f, 1.0f + e);
}

// Marks the grid as failed; the first reporter also leaves four words of detail.
__device__ __forceinline__ void raise_abort(const Sync& s, int* s_abort, int code, int d0 = 0,
                                            int d1 = 0, int d2 = 0, int d3 = 0) {
  *reinterpret_cast<volatile int*>(s_abort) = 1;
  if (atomicExch(s.abort_flag, 1) == 0) {
    volatile int* e = reinterpret_cast<volatile int*>(s.err);
    e[1] = d0; e[2] = d1; e[3] = d2; e[4] = d3;
    __threadfence_system();
    e[0] = code;
  }
  __threadfence_system();
}

// ---------------------------------------------------------------------------------------
// Forward
// ---------------------------------------------------------------------------------------
template <int G, int KSW, int SPLIT, int MTMAX, typename T>
__global__ void __launch_bounds__(THREADS, 1) rec_fwd_kernel(const FwdParams p) {
  constexpr int COLS = G * U;             // gate columns owned by the CTA
  constexpr int NT = COLS / 8;            // n-tiles
  constexpr int KW = KSW * 16;            // K elements per warp
  constexpr int KPAD = WARPS * KW;        // padded K
  constexpr int AROW = KPAD + 8;          // bf16 elements per smem row (16 B pad: no conflicts)
  constexpr int PROW = COLS + 8;          // floats per partial row
  extern __shared__ __align__(16) uint8_t smem[];
  const int BNR = p.MT * 16;
  // A planes hold ONE m-tile (16 rows): a warp only ever reads its own K range of them, so it
  // restages them per m-tile without any CTA-wide synchronisation.
  __nv_bfloat16* a_hi = reinterpret_cast<__nv_bfloat16*>(smem);
  __nv_bfloat16* a_lo = a_hi + (SPLIT == 2 ? (size_t)16 * AROW : 0);
  float* part = reinterpret_cast<float*>(smem + (size_t)SPLIT * 16 * AROW * 2);  // [2][8][16][PROW]
  __shared__ int s_abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int gq = lane >> 2, q = lane & 3;
  const int hs = blockIdx.x % p.nHS, bs = blockIdx.x / p.nHS;
  const int u0 = hs * U, n0 = bs * BNR;
  const int H = p.H, N = p.N, Hx = p.Hx;
  const long long NH = (long long)N * H;
  const int GH = G * H;
  if (tid == 0) s_abort = 0;

  // ---- recurrent weights -> registers (B fragments), once
  uint32_t rf[SPLIT][NT][KSW][2];
  {
    const T* R = reinterpret_cast<const T*>(p.R);
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const int cl = nt * 8 + gq;              // local column, unit-major: cl = u*G + gate
      const int u = cl / G, gate = cl % G;
      const bool col_ok = (u0 + u) < H;
      const long long col = (long long)gate * H + u0 + u;
#pragma unroll
      for (int ks = 0; ks < KSW; ++ks) {
        const int kb = warp * KW + ks * 16 + 2 * q;
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
  const bool unit_pad = !unit_ok && (u0 + ul) < Hx;  // padding word the consumers still read
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
  float c_reg[MTMAX], h_reg[MTMAX];
#pragma unroll
  for (int mt = 0; mt < MTMAX; ++mt) {
    const int n = n0 + mt * 16 + nl;
    const bool ok = mt < p.MT && n < N && unit_ok;
    h_reg[mt] = ok ? ld(hbuf + (long long)n * H + u0 + ul) : 0.f;
    c_reg[mt] = (G == 4 && ok) ? ld(cbuf + (long long)n * H + u0 + ul) : 0.f;
  }

  __syncthreads();

  bool alive = true;
  int pbuf = 0;
  for (int t = 0; t < p.T && alive; ++t) {
    // ---- loads that do not depend on the recurrence: x.W (+ zoneout mask)
    float wxr[MTMAX][G], mk[MTMAX];
#pragma unroll
    for (int mt = 0; mt < MTMAX; ++mt) {
      const int n = n0 + mt * 16 + nl;
      const bool ok = mt < p.MT && n < N && unit_ok;
#pragma unroll
      for (int g = 0; g < G; ++g)
        wxr[mt][g] = ok ? ld(wx + ((long long)t * N + n) * GH + g * H + u0 + ul) : 0.f;
      mk[mt] = (ok && p.has_zoneout && p.training)
                   ? ld(mask + (long long)t * NH + (long long)n * H + u0 + ul) : 0.f;
      if (MTMAX == 1 && ok && t + 1 < p.T && !HB_DBG(p, 512)) {  // next step inputs: into L2 now
#pragma unroll
        for (int g = 0; g < G; ++g)
          prefetch_l2(wx + ((long long)(t + 1) * N + n) * GH + g * H + u0 + ul);
        if (p.has_zoneout && p.training)
          prefetch_l2(mask + (long long)(t + 1) * NH + (long long)n * H + u0 + ul);
      }
    }

    for (int mt = 0; mt < p.MT; ++mt) {
      // ---- this warp's K range of h_t for the rows of m-tile mt -> the A planes.  At t = 0
      // the caller's initial state; afterwards the tagged words the producers wrote.  Staging
      // per m-tile lets the wait for one m-tile hide behind the work on the others.
      {
        constexpr int CPR = KW / 4;         // 4-element chunks per row in this warp's range
        constexpr int CPL = 16 * CPR / 32;  // chunks per lane
        __syncwarp();                       // the previous m-tile's fragment loads are done
        if (t == 0) {
#pragma unroll
          for (int i = 0; i < CPL; ++i) {
            const int e = lane + i * 32;
            const int r = e / CPR, k = warp * KW + (e % CPR) * 4;
            const int n = n0 + mt * 16 + r;
            float x[4], lo[4];
#pragma unroll
            for (int j4 = 0; j4 < 4; ++j4) {
              x[j4] = (n < N && k + j4 < H) ? ld(hbuf + (long long)n * H + k + j4) : 0.f;
              lo[j4] = 0.f;
              if (SPLIT == 2) split_bf16(x[j4], x[j4], lo[j4]);
            }
            *reinterpret_cast<uint2*>(a_hi + (size_t)r * AROW + k) =
                make_uint2(pack_bf16(x[0], x[1]), pack_bf16(x[2], x[3]));
            if (SPLIT == 2)
              *reinterpret_cast<uint2*>(a_lo + (size_t)r * AROW + k) =
                  make_uint2(pack_bf16(lo[0], lo[1]), pack_bf16(lo[2], lo[3]));
          }
        } else if (alive && !HB_DBG(p, 1)) {
          const uint32_t want = (((uint32_t)(t - 1) >> 1) & 1u) ^ 1u;
          const uint32_t wtag = want << 30;
          const uint32_t* xsrc = p.xbuf + (size_t)((t - 1) & 1) * N * Hx;
          uint4 w[CPL];
          const long long t0 = clock64();
          unsigned int spins = 0;
          for (;;) {
            // issue every load before looking at any of them, so their latencies overlap
#pragma unroll
            for (int i = 0; i < CPL; ++i) {
              const int e = lane + i * 32;
              const int r = e / CPR, k = warp * KW + (e % CPR) * 4;
              const int n = n0 + mt * 16 + r;
              if (n < N && k < Hx) w[i] = ld_relaxed_u32x4(xsrc + (size_t)n * Hx + k);
              else w[i] = make_uint4(wtag, wtag, wtag, wtag);
            }
            // one logic instruction per word: bit 30 of `bad` ends up set if any tag is stale
            uint32_t bad = 0;
#pragma unroll
            for (int i = 0; i < CPL; ++i)
              bad |= (w[i].x ^ wtag) | (w[i].y ^ wtag) | (w[i].z ^ wtag) | (w[i].w ^ wtag);
            const bool ok = (bad & 0x40000000u) == 0;
            if (__all_sync(0xffffffffu, ok)) break;
            if ((++spins & 63u) == 0) {
              bool stop = *reinterpret_cast<volatile int*>(p.sync.abort_flag) != 0;
              if (!stop && clock64() - t0 > SPIN_LIMIT_CYCLES) {
                raise_abort(p.sync, &s_abort, 16);
                stop = true;
              }
              if (__any_sync(0xffffffffu, stop)) { alive = false; break; }
            }
          }
          if (!alive) *reinterpret_cast<volatile int*>(&s_abort) = 1;  // the barrier below sees it
#pragma unroll
          for (int i = 0; i < CPL; ++i) {
            const int e = lane + i * 32;
            const int r = e / CPR, k = warp * KW + (e % CPR) * 4;
            *reinterpret_cast<uint2*>(a_hi + (size_t)r * AROW + k) =
                make_uint2(__byte_perm(w[i].x, w[i].y, 0x5410), __byte_perm(w[i].z, w[i].w, 0x5410));
            if (SPLIT == 2)
              *reinterpret_cast<uint2*>(a_lo + (size_t)r * AROW + k) =
                  make_uint2(__byte_perm(w[i].x, w[i].y, 0x7632) & 0xBFFFBFFFu,
                             __byte_perm(w[i].z, w[i].w, 0x7632) & 0xBFFFBFFFu);
          }
        }
        __syncwarp();
      }
      // ---- this warp's K range of the step product
      float acc[NT][4];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
      if (!HB_DBG(p, 2)) {
#pragma unroll
        for (int ks = 0; ks < KSW; ++ks) {
          const int row = lane & 15;
          const int kcol = warp * KW + ks * 16 + (lane >> 4) * 8;
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
      }
      float* pb = part + (size_t)pbuf * WARPS * 16 * PROW;
      float* pw = pb + (size_t)warp * 16 * PROW;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        *reinterpret_cast<float2*>(pw + gq * PROW + nt * 8 + 2 * q) =
            make_float2(acc[nt][0], acc[nt][1]);
        *reinterpret_cast<float2*>(pw + (gq + 8) * PROW + nt * 8 + 2 * q) =
            make_float2(acc[nt][2], acc[nt][3]);
      }
      // the only CTA-wide barrier per m-tile (partials are double-buffered); the OR makes the
      // decision to stop the same for every thread
      if (__syncthreads_or(*reinterpret_cast<volatile int*>(&s_abort))) { alive = false; break; }

      // ---- pointwise stage for (row nl of m-tile mt, unit ul)
      float rh[G];
#pragma unroll
      for (int g = 0; g < G; ++g) rh[g] = 0.f;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) {
        const float* src = pb + ((size_t)w * 16 + nl) * PROW + ul * G;
        if (G == 4) {
          const float4 f = *reinterpret_cast<const float4*>(src);
          rh[0] += f.x; rh[1] += f.y; rh[2] += f.z; rh[G - 1] += f.w;
        } else {
#pragma unroll
          for (int g = 0; g < G; ++g) rh[g] += src[g];
        }
      }
      pbuf ^= 1;
      const int n = n0 + mt * 16 + nl;
      const uint32_t tag = (((uint32_t)t >> 1) & 1u) ^ 1u;
      uint32_t* xdst = p.xbuf + (size_t)(t & 1) * N * Hx + (size_t)n * Hx + u0 + ul;
      if (n < N && unit_ok) {
        float hp = 0.f, cp = 0.f, m = 0.f, wv[G];
#pragma unroll
        for (int k = 0; k < MTMAX; ++k)
          if (k == mt) {
            hp = h_reg[k]; cp = c_reg[k]; m = mk[k];
#pragma unroll
            for (int g = 0; g < G; ++g) wv[g] = wxr[k][g];
          }
        const long long o0 = (long long)n * H + u0 + ul;
        float h_new, c_new = 0.f;
        if (G == 4) {
          const float i = sigmoid_fast(wv[0] + rh[0] + bias[0]);
          const float g = tanh_fast(wv[1] + rh[1] + bias[1]);
          const float f = sigmoid_fast(wv[2] + rh[2] + bias[2]);
          const float o = sigmoid_fast(wv[G - 1] + rh[G - 1] + bias[G - 1]);
          c_new = f * cp + i * g;
          h_new = o * tanh_fast(c_new);
          if (p.has_zoneout)
            h_new = p.training ? zoneout<true>(h_new, hp, p.zoneout_prob, m)
                               : zoneout<false>(h_new, hp, p.zoneout_prob, m);
          h_new = round_to_storage<T>(h_new);  // exchange exactly what a later load of h returns
          if (t + 1 < p.T) publish_u32(xdst, xword_encode(h_new, tag));  // first: it is on the critical path
          st(hbuf + (long long)(t + 1) * NH + o0, h_new);
          st(cbuf + (long long)(t + 1) * NH + o0, c_new);
          if (p.training) {
            T* vt = vbuf + ((long long)t * N + n) * GH + u0 + ul;
            st(vt, i); st(vt + H, g); st(vt + 2 * H, f); st(vt + 3 * H, o);
          }
        } else {
          const float z = sigmoid_fast(wv[0] + rh[0] + bias[0] + bias2[0]);
          const float r = sigmoid_fast(wv[1] + rh[1] + bias[1] + bias2[1]);
          const float qg = rh[2] + bias2[2];
          const float g = tanh_fast(wv[2] + r * qg + bias[2]);
          h_new = z * hp + (1.0f - z) * g;
          if (p.has_zoneout)
            h_new = p.training ? zoneout<true>(h_new, hp, p.zoneout_prob, m)
                               : zoneout<false>(h_new, hp, p.zoneout_prob, m);
          h_new = round_to_storage<T>(h_new);  // exchange exactly what a later load of h returns
          if (t + 1 < p.T) publish_u32(xdst, xword_encode(h_new, tag));
          st(hbuf + (long long)(t + 1) * NH + o0, h_new);
          if (p.training && vbuf) {
            T* vt = vbuf + ((long long)t * N + n) * 4 * H + u0 + ul;
            st(vt, z); st(vt + H, r); st(vt + 2 * H, g); st(vt + 3 * H, qg);
          }
        }
#pragma unroll
        for (int k = 0; k < MTMAX; ++k)
          if (k == mt) { h_reg[k] = h_new; c_reg[k] = c_new; }
      } else if (n < N && unit_pad && t + 1 < p.T) {
        publish_u32(xdst, xword_encode(0.0f, tag));
      }
    }
  }
}

// ---------------------------------------------------------------------------------------
// Backward
// ---------------------------------------------------------------------------------------
// Gate gradients of one (row, unit) to global memory: the fp32/bf16 tensors the reference
// defines (LSTM: v; GRU: dp, dq) and, for fp32 storage, their bf16 planes for the
// time-parallel contractions.  dg: LSTM d(i,g,f,o); GRU dp_z, dp_r, dp_g, dq_g.
template <int G, int SPLIT, typename T>
__device__ __forceinline__ void store_gate_grads(const BwdParams& p, int t, int n, int unit, int N,
                                                 int H, bool unit_ok, const float (&dg)[4]) {
  if (!(n < N && unit_ok)) return;
  if (G == 4) {
    T* vt = reinterpret_cast<T*>(p.v) + ((long long)t * N + n) * 4 * H + unit;
#pragma unroll
    for (int g4 = 0; g4 < 4; ++g4) st(vt + g4 * H, dg[g4]);
    if (SPLIT == 2 && p.gpl) {
      __nv_bfloat16* ph = p.gpl + ((long long)t * N + n) * 4 * H + unit;
#pragma unroll
      for (int g4 = 0; g4 < 4; ++g4) {
        float hi, lo;
        split_bf16(dg[g4], hi, lo);
        ph[g4 * H] = __float2bfloat16_rn(hi);
        ph[p.gpl_stride + g4 * H] = __float2bfloat16_rn(lo);
      }
    }
  } else {
    T* dpb = reinterpret_cast<T*>(p.dp);
    T* dqb = reinterpret_cast<T*>(p.dq);
    const float dp_z = dg[0], dp_r = dg[1], dp_g = dg[2], dq_g = dg[3];
    const long long w0 = ((long long)t * N + n) * 3 * H + unit;
    st(dpb + w0, dp_z); st(dpb + w0 + H, dp_r); st(dpb + w0 + 2 * H, dp_g);
    st(dqb + w0, dp_z); st(dqb + w0 + H, dp_r); st(dqb + w0 + 2 * H, dq_g);
    if (SPLIT == 2 && p.gpl) {
      const float pv[3] = {dp_z, dp_r, dp_g};
#pragma unroll
      for (int g3 = 0; g3 < 3; ++g3) {
        float hi, lo;
        split_bf16(pv[g3], hi, lo);
        p.gpl[w0 + g3 * H] = __float2bfloat16_rn(hi);
        p.gpl[p.gpl_stride + w0 + g3 * H] = __float2bfloat16_rn(lo);
        split_bf16(g3 == 2 ? dq_g : pv[g3], hi, lo);
        p.gpl2[w0 + g3 * H] = __float2bfloat16_rn(hi);
        p.gpl2[p.gpl_stride + w0 + g3 * H] = __float2bfloat16_rn(lo);
      }
    }
  }
}

template <int G, int NTW, int SPLIT, int MTMAX, typename T>
__global__ void __launch_bounds__(THREADS, 1) rec_bwd_kernel(const BwdParams p) {
  constexpr int COLS = G * U;                 // K of the step product
  constexpr int KS = (COLS + 15) / 16;        // k-steps (LSTM 4, GRU 3)
  constexpr int KPAD = KS * 16;
  constexpr int AROW = KPAD + 8;
  extern __shared__ __align__(16) uint8_t smem[];
  const int BNR = p.MT * 16;
  // A planes, double-buffered by step parity: [2][SPLIT][BNR][AROW]
  __nv_bfloat16* a_base = reinterpret_cast<__nv_bfloat16*>(smem);
  const size_t a_plane = (size_t)BNR * AROW;
  __shared__ int s_abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int gq = lane >> 2, q = lane & 3;
  const int hs = blockIdx.x % p.nHS, bs = blockIdx.x / p.nHS;
  const int nBS = gridDim.x / p.nHS;
  const int u0 = hs * U, n0 = bs * BNR;
  const int H = p.H, N = p.N;
  const long long NH = (long long)N * H;
  const int GH = G * H;
  if (tid == 0) s_abort = 0;
  // zero the A planes once: padding columns (GRU: 48..63 never exist; KPAD == COLS) and
  // rows of masked units stay zero
  for (int e = tid; e < 2 * SPLIT * (int)a_plane; e += THREADS) a_base[e] = __float2bfloat16_rn(0.f);

  // ---- R[:, slice]^T as B fragments: B(k = local gate column, n = output unit j);
  // output units j in [warp*NTW*8, (warp+1)*NTW*8).
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

  float dh_c[MTMAX], dc_c[MTMAX];
#pragma unroll
  for (int mt = 0; mt < MTMAX; ++mt) {
    const int n = n0 + mt * 16 + nl;
    const bool ok = mt < p.MT && n < N && unit_ok;
    dh_c[mt] = ok ? p.dh_carry[(long long)n * H + u0 + ul] : 0.f;
    dc_c[mt] = (G == 4 && ok) ? p.dc_carry[(long long)n * H + u0 + ul] : 0.f;
  }
  const size_t blk = (size_t)BNR * U;  // words per (dest, src) exchange block
  float acc_b[4] = {0.f, 0.f, 0.f, 0.f};  // bias-gradient sums of this thread's (rows, unit)
  bool alive = true;
  __syncthreads();

  for (int t = p.T - 1; t >= 0 && alive; --t) {
    const int ti = p.T - 1 - t;  // production index of this step
    // ---- loads independent of the carried gradient
    float gv[MTMAX][4], cprev[MTMAX], cnew[MTMAX], dhv[MTMAX], dcv[MTMAX], mk[MTMAX],
        hprev[MTMAX];
#pragma unroll
    for (int mt = 0; mt < MTMAX; ++mt) {
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
      // Ask L2 for the next step's inputs now, so that their loads return from L2 and do not
      // occupy the SM's miss queue for an HBM round trip while the exchange polls need it.
      if (MTMAX == 1 && ok && t > 0 && !HB_DBG(p, 512)) {
#pragma unroll
        for (int g = 0; g < 4; ++g) prefetch_l2(vt - (long long)N * 4 * H + g * H);
        prefetch_l2(dhn + (long long)t * NH + o0);
        if (p.has_zoneout) prefetch_l2(mask + (long long)(t - 1) * NH + o0);
        if (G == 4) {
          prefetch_l2(cbuf + (long long)(t - 1) * NH + o0);
          prefetch_l2(dcn + (long long)t * NH + o0);
        } else {
          prefetch_l2(hbuf + (long long)(t - 1) * NH + o0);
        }
      }
    }

    // ---- recurrent part of dh_t: the partials published at the previous step (ti-1)
    if (ti > 0 && !HB_DBG(p, 1)) {
      const uint32_t want = (((uint32_t)(ti - 1) >> 1) & 1u) ^ 1u;
      const uint32_t* src =
          p.exch + ((((size_t)((ti - 1) & 1) * nBS + bs) * p.nHS + hs) * p.nHS) * blk;
      // Thread (row nl, unit ul) sits in a group of 4 adjacent lanes that share
      // (row, unit quad); lane sg = ul & 3 of the group fetches 16-byte pieces (4 units) from
      // sources sg*8 .. sg*8+7 of each pass of 32 sources, all loads in flight together,
      // and a two-step butterfly adds the four lanes.  The summation order is fixed.
      const int sg = ul & 3, quad = ul >> 2;
#pragma unroll
      for (int mt = 0; mt < MTMAX; ++mt) {
        if (mt < p.MT) {  // uniform: the shuffles below are executed by whole warps
          float s4[4] = {0.f, 0.f, 0.f, 0.f};
          const uint32_t* q0 = src + (size_t)(mt * 16 + nl) * U + quad * 4;
          for (int s0 = 0; s0 < p.nHS && alive; s0 += 32) {
            uint4 a[8];
            const long long t0 = clock64();
            unsigned int spins = 0;
            const uint32_t rdy = want;
            for (;;) {
#pragma unroll
              for (int k = 0; k < 8; ++k) {
                const int sidx = s0 + sg * 8 + k;
                a[k] = (sidx < p.nHS) ? ld_relaxed_u32x4(q0 + (size_t)sidx * blk)
                                      : make_uint4(rdy, rdy, rdy, rdy);
              }
              uint32_t bad = 0;  // bit 0 ends up set if any tag is stale
#pragma unroll
              for (int k = 0; k < 8; ++k)
                bad |= (a[k].x ^ want) | (a[k].y ^ want) | (a[k].z ^ want) | (a[k].w ^ want);
              if ((bad & 1u) == 0) break;
              if ((++spins & 63u) == 0) {
                if (*reinterpret_cast<volatile int*>(p.sync.abort_flag) != 0) { alive = false; break; }
                if (clock64() - t0 > SPIN_LIMIT_CYCLES) {
                  raise_abort(p.sync, &s_abort, 17, blockIdx.x * 1000 + tid, ti * 100 + s0);
                  alive = false;
                  break;
                }
              }
            }
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              s4[0] += fword_value(a[k].x);
              s4[1] += fword_value(a[k].y);
              s4[2] += fword_value(a[k].z);
              s4[3] += fword_value(a[k].w);
            }
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            s4[j] += __shfl_xor_sync(0xffffffffu, s4[j], 1);
            s4[j] += __shfl_xor_sync(0xffffffffu, s4[j], 2);
          }
          dh_c[mt] += sg == 0 ? s4[0] : (sg == 1 ? s4[1] : (sg == 2 ? s4[2] : s4[3]));
        }
      }
    }
    if (!alive) *reinterpret_cast<volatile int*>(&s_abort) = 1;

    // Deferred stores where they measured faster (N=64, fp32: LSTM H=512 3.76 -> 3.45, H=256
    // 2.55 -> 2.51, GRU H=512 3.43 -> 3.32 us per step); the GRU with narrower slices measured
    // slower with them (H=256: 2.35 -> 2.45) and keeps the immediate stores.
    constexpr bool DEFER = MTMAX == 1 && (G == 4 || NTW >= 8);
    __nv_bfloat16* a_hi = a_base + (size_t)(ti & 1) * SPLIT * a_plane;
    __nv_bfloat16* a_lo = a_hi + (SPLIT == 2 ? a_plane : 0);
    float dg4[4];  // LSTM: d(i,g,f,o); GRU: dp_z, dp_r, dp_g, dq_g (one m-tile only)
    // (With several m-tiles the body is empty and the closure captures nothing.  How this is
    // written matters more than it should: the same stores issued through a direct call
    // instead of this closure measured 0.5 us per step slower at N=64, and a closure that
    // captures in the multi-tile instantiation measured 0.9 us per step slower at N=128.)
    auto store_gates = [&]() {
      if constexpr (DEFER) store_gate_grads<G, SPLIT, T>(p, t, n0 + nl, u0 + ul, N, H, unit_ok, dg4);
    };
    if constexpr (!DEFER) {
      // ---- pointwise gradients; gate gradients -> global and -> smem (A operand)
#pragma unroll
      for (int mt = 0; mt < MTMAX; ++mt) {
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
            const float c_tanh = tanh_fast(cnew[mt]);
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
#pragma unroll
              for (int g4 = 0; g4 < 4; ++g4) acc_b[g4] += dgate[g4 % G];
              T* vt = vbuf + ((long long)t * N + n) * 4 * H + u0 + ul;
#pragma unroll
              for (int g4 = 0; g4 < 4; ++g4) st(vt + g4 * H, dgate[g4 % G]);
              if (SPLIT == 2 && p.gpl) {
                __nv_bfloat16* ph = p.gpl + ((long long)t * N + n) * 4 * H + u0 + ul;
#pragma unroll
                for (int g4 = 0; g4 < 4; ++g4) {
                  float hi, lo;
                  split_bf16(dgate[g4 % G], hi, lo);
                  ph[g4 * H] = __float2bfloat16_rn(hi);
                  ph[p.gpl_stride + g4 * H] = __float2bfloat16_rn(lo);
                }
              }
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
              acc_b[0] += dp_z; acc_b[1] += dp_r; acc_b[2] += dp_g; acc_b[3] += dgate[2];
              const long long w0 = ((long long)t * N + n) * 3 * H + u0 + ul;
              st(dpb + w0, dp_z); st(dpb + w0 + H, dp_r); st(dpb + w0 + 2 * H, dp_g);
              st(dqb + w0, dp_z); st(dqb + w0 + H, dp_r); st(dqb + w0 + 2 * H, dgate[2]);
              if (SPLIT == 2 && p.gpl) {
                const float pv[3] = {dp_z, dp_r, dp_g};
#pragma unroll
                for (int g3 = 0; g3 < 3; ++g3) {
                  float hi, lo;
                  split_bf16(pv[g3], hi, lo);
                  p.gpl[w0 + g3 * H] = __float2bfloat16_rn(hi);
                  p.gpl[p.gpl_stride + w0 + g3 * H] = __float2bfloat16_rn(lo);
                  split_bf16(g3 == 2 ? dgate[2] : pv[g3], hi, lo);
                  p.gpl2[w0 + g3 * H] = __float2bfloat16_rn(hi);
                  p.gpl2[p.gpl_stride + w0 + g3 * H] = __float2bfloat16_rn(lo);
                }
              }
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
    } else {
      // ---- pointwise gradients; gate gradients -> smem (A operand) and -> global.
      // With one m-tile the global stores are issued after the partials have been published
      // (the values stay in registers), which takes them off the step-to-step chain: measured
      // 3.76 -> 3.43 us per step (LSTM, N=64, H=512, fp32).  With several m-tiles the values
      // of all tiles would have to stay live; there the stores go out at once, before the
      // shared-memory rows (the other order measured 0.8 us per step slower at N=128).
#pragma unroll
      for (int mt = 0; mt < MTMAX; ++mt) {
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
            const float c_tanh = tanh_fast(cnew[mt]);
            float dc_total = dcv[mt] + dc_c[mt];
            const float d_o = c_tanh * dh_total;
            dc_total += d_tanh(c_tanh) * (o * dh_total);
            dgate[0] = d_sigmoid(i) * (g * dc_total);
            dgate[1] = d_tanh(g) * (i * dc_total);
            dgate[2] = d_sigmoid(f) * (cprev[mt] * dc_total);
            dgate[G - 1] = d_sigmoid(o) * d_o;
            dc_c[mt] = f * dc_total;
            dh_c[mt] = keep;
#pragma unroll
            for (int g4 = 0; g4 < 4; ++g4) dg4[g4] = dgate[g4 % G];
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
            dg4[0] = dp_z; dg4[1] = dp_r; dg4[2] = dp_g; dg4[3] = dgate[2];
          }
          if (ok) {
#pragma unroll
            for (int g4 = 0; g4 < 4; ++g4) acc_b[g4] += dg4[g4];
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
      if (t == 0) store_gates();
    }
    if (t == 0) break;  // nobody consumes partials of the last step
    __syncthreads();    // the only CTA-wide barrier of the step (A planes are double-buffered)
    if (*reinterpret_cast<volatile int*>(&s_abort)) {
      alive = false;
      break;
    }

    // ---- partial dh_{t-1}[rows, all units] = dG . R[:, slice]^T, warp owns NTW*8 units
    {
      const uint32_t tag = (((uint32_t)ti >> 1) & 1u) ^ 1u;
      uint32_t* dstbase = p.exch + ((size_t)(ti & 1) * nBS + bs) * p.nHS * p.nHS * blk;
      for (int mt = 0; mt < p.MT; ++mt) {
        float acc[NTW][4];
#pragma unroll
        for (int nt = 0; nt < NTW; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
        if (!HB_DBG(p, 2)) {
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
        }
#pragma unroll
        for (int nt = 0; nt < NTW; ++nt) {
          const int j = (warp * NTW + nt) * 8 + 2 * q;  // output unit of acc[.][0]
          if (j < p.nHS * U) {
            const int dest = j / U, uj = j % U;
            uint32_t* d = dstbase + ((size_t)dest * p.nHS + hs) * blk + (size_t)(mt * 16) * U + uj;
            publish_u32x2(d + (size_t)gq * U, fword_encode(acc[nt][0], tag),
                          fword_encode(acc[nt][1], tag));
            publish_u32x2(d + (size_t)(gq + 8) * U, fword_encode(acc[nt][2], tag),
                          fword_encode(acc[nt][3], tag));
          }
        }
      }
    }
    store_gates();
  }

  if (p.db_part && unit_ok) {
    float* dst = p.db_part + ((size_t)bs * 16 + nl) * 4 * H + u0 + ul;
#pragma unroll
    for (int g4 = 0; g4 < 4; ++g4) dst[(size_t)g4 * H] = acc_b[g4];
  }
  // ---- carries out.  After the last step dh_c holds only the zoneout / GRU direct part
  // of dh_0; the recurrent part of that step is added by the host-issued contraction.
  if (alive) {
#pragma unroll
    for (int mt = 0; mt < MTMAX; ++mt) {
      const int n = n0 + mt * 16 + nl;
      if (mt < p.MT && n < N && unit_ok) {
        p.dh_carry[(long long)n * H + u0 + ul] = dh_c[mt];
        if (G == 4) p.dc_carry[(long long)n * H + u0 + ul] = dc_c[mt];
      }
    }
  }
}

// ---------------------------------------------------------------------------------------
// Host-side launch helpers shared by the instantiation files
// ---------------------------------------------------------------------------------------
struct Geometry {
  int nHS, nBS, MT;
};

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

template <int G, int SPLIT, typename T>
int run_fwd(FwdParams& p, const Geometry& g, cudaStream_t s) {
  const int ksteps = ceil_div(p.H, 16);
  const int ksw = ceil_div(ksteps, WARPS);
  auto smem_for = [&](int KSW) {
    const size_t arow = (size_t)WARPS * KSW * 16 + 8;
    return (size_t)SPLIT * 16 * arow * 2 + (size_t)2 * WARPS * 16 * (G * U + 8) * 4;
  };
  const int grid = g.nHS * g.nBS;
#define HB_FWD(KSW)                                                                          \
  if (ksw <= KSW) {                                                                          \
    if (smem_for(KSW) > 220 * 1024) return HASTE_B200_ERR_UNSUPPORTED;                       \
    if (g.MT == 1)                                                                           \
      return launch_coop(rec_fwd_kernel<G, KSW, SPLIT, 1, T>, grid, smem_for(KSW), &p, s);   \
    return launch_coop(rec_fwd_kernel<G, KSW, SPLIT, 4, T>, grid, smem_for(KSW), &p, s);     \
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
  const size_t smem = (size_t)2 * SPLIT * g.MT * 16 * arow * 2;
  const int grid = g.nHS * g.nBS;
#define HB_BWD(NTW)                                                                   \
  if (ntw <= NTW) {                                                                   \
    if (g.MT == 1)                                                                    \
      return launch_coop(rec_bwd_kernel<G, NTW, SPLIT, 1, T>, grid, smem, &p, s);     \
    return launch_coop(rec_bwd_kernel<G, NTW, SPLIT, 4, T>, grid, smem, &p, s);       \
  }
  HB_BWD(1)
  HB_BWD(2)
  HB_BWD(4)
  HB_BWD(8)
  if constexpr (SPLIT == 1) { HB_BWD(16) }
#undef HB_BWD
  return HASTE_B200_ERR_UNSUPPORTED;
}

// Defined one per translation unit so the kernels compile in parallel.
int run_fwd_lstm_f32(FwdParams& p, const Geometry& g, cudaStream_t s);
int run_fwd_lstm_bf16(FwdParams& p, const Geometry& g, cudaStream_t s);
int run_fwd_gru_f32(FwdParams& p, const Geometry& g, cudaStream_t s);
int run_fwd_gru_bf16(FwdParams& p, const Geometry& g, cudaStream_t s);
int run_bwd_lstm_f32(BwdParams& p, const Geometry& g, cudaStream_t s);
int run_bwd_lstm_bf16(BwdParams& p, const Geometry& g, cudaStream_t s);
int run_bwd_gru_f32(BwdParams& p, const Geometry& g, cudaStream_t s);
int run_bwd_gru_bf16(BwdParams& p, const Geometry& g, cudaStream_t s);
int run_fwd_gru_f16(FwdParams& p, const Geometry& g, cudaStream_t s);
int run_bwd_gru_f16(BwdParams& p, const Geometry& g, cudaStream_t s);

}  // namespace rec
}  // namespace hb
