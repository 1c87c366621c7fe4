// Persistent LayerNormLSTM recurrence kernels (forward and backward), sm_100a.
//
// Same skeleton as recurrent_kernels.cuh - cooperative grid of (hidden slices) x (batch
// slices), the CTA's slice of R resident in registers as mma.sync fragments, self-validating
// tagged words for every inter-CTA hand-off, bounded waits - plus what LayerNorm adds: a
// normalisation runs over a whole row (all 4H gate columns of h.R, all H units of c'), while a
// CTA only holds 64 / 16 of those columns.  Each row statistic is therefore built in two
// levels: the 16 threads that own a row inside a CTA reduce with shuffles, the CTAs of the
// batch slice then exchange one (a, b) pair per row through a small tagged buffer and every
// CTA combines the nHS pairs in a fixed order.  Forward: (mean, M2) pairs combined with
// Chan's formula (no E[x^2]-mean^2 cancellation); backward: the two row sums of the
// LayerNorm gradient.  Per step that is three exchange rounds forward (h.R statistics, c'
// statistics, h) and three backward (partial dh, LN(c') sums, LN(h.R) sums).
//
// All LayerNorm inputs stay in fp32 registers between the stages of a step (with bf16 storage
// too: a value is rounded only when it is saved for the backward pass).
//
// Math and saved tensors follow the reference (lib/layer_norm_lstm_forward_gpu.cu.cc:26-109,
// 191-273; lib/layer_norm_lstm_backward_gpu.cu.cc:27-118,207-252; LayerNorm gradient
// lib/layer_norm_backward_gpu.cu.cc:44-91).  One deliberate difference: the reference's
// LayerNorm gradient carries a term proportional to sum(x - mean), which is zero in exact
// arithmetic; it is left out here.
#pragma once

#include "recurrent_kernels.cuh"

namespace hb {
namespace rec {

struct LnFwdParams {
  int T, N, H, Hx, nHS, MT, training, has_zoneout;
  float zoneout_prob;
  const void* R;        // [H, 4H]
  const void* b;        // LSTM: b [4H];  GRU: bx [3H]
  const void* b2;       // GRU: br [3H]
  const void* Wx;       // LN(x.W) [T,N,G*H] (LSTM: aliases v)
  const void* gamma_Rh; // [G*H]
  const void* gamma_h;  // [H]
  const void* beta_h;   // [H]
  void* v;              // LSTM: act_Wx_norm [T,N,4H], LN(x.W) in, gate activations out
                        // GRU: cache [T,N,4H] = (z, r, g, LN(h.R)_g + br_g), may be null in inference
  void* act_Rh;         // [T,N,G*H] pre-norm h.R (saved)
  void* cache_Rh;       // [T,N,2]
  void* act_c_norm;     // [T,N,H]
  void* cache_c;        // [T,N,2]
  void* h;              // [T+1,N,H]
  void* c;              // [T+1,N,H] un-normalised cell state
  const void* mask;
  uint32_t* xbuf;       // [2][N][Hx] tagged h words
  uint32_t* sbuf;       // [2 stats][2 parity][nBS][rows][nHS][2] tagged statistic pairs
  Sync sync;
  int dbg = 0;          // read only in timing-experiment builds (HB_DBG): 1 no h wait, 2 no MMA, 4 no statistic waits
};

struct LnBwdParams {
  int T, N, H, nHS, MT, has_zoneout, r_transposed;
  const void* R;
  const void* gamma_Rh;
  const void* gamma_h;
  const void* c;          // LSTM [T+1,N,H]
  const void* h;          // GRU [T+1,N,H]
  void* dp;               // GRU out [T,N,3H]: gradient w.r.t. LN(x.W)+bx
  void* dq;               // GRU out [T,N,3H]: gradient w.r.t. LN(h.R)+br
  void* v;                // LSTM: act_Wx_norm, gate activations in, gate gradients out.
                          // GRU: cache [T,N,4H] in (untouched)
  void* act_Rh;           // pre-norm h.R in, d(h.R) out
  const void* cache_Rh;
  void* act_c_norm;       // LN(c') in (left untouched)
  const void* cache_c;
  const void* dh_new;
  const void* dc_new;
  const void* mask;
  float* dh_carry;        // [N,H] in/out
  float* dc_carry;        // [N,H] in/out
  float* dgRh_part;       // [N,4H] per-row partial sums of dgamma_Rh (reduced by the host)
  float* dgh_part;        // [N,H]  per-row partial sums of dgamma_h
  float* dbh_part;        // [N,H]  per-row partial sums of dbeta_h
  uint32_t* exch;         // tagged partial dh, as in rec_bwd_kernel
  uint32_t* sbuf;         // [2 stats][2 parity][nBS][rows][nHS][2]
  Sync sync;
  __nv_bfloat16* gpl;     // optional bf16 planes of d(x.W-side gate gradient) (dv)
  __nv_bfloat16* gpl2;    // optional bf16 planes of d(h.R)
  long long gpl_stride;
  int dbg = 0;            // read only in timing-experiment builds (HB_DBG): 1 no dh wait, 2 no MMA, 4 no statistic waits
};

// Statistics, partial gradients and (with fp32 storage) h travel as tagged fp32 words
// (fword_* of recurrent_kernels.cuh): LayerNorm amplifies a relative error of the exchanged
// value roughly tenfold, so the 17 bits of the (hi, lo) bf16 pair are not enough here.
// h words: tagged fp32 with fp32 storage, the (hi, lo) bf16 pair with bf16 storage.
template <int SPLIT> __device__ __forceinline__ uint32_t hword_encode(float x, uint32_t tag) {
  return SPLIT == 2 ? fword_encode(x, tag) : xword_encode(x, tag);
}
template <int SPLIT> __device__ __forceinline__ bool hword_ready(uint32_t w, uint32_t tag) {
  return SPLIT == 2 ? fword_ready(w, tag) : xword_ready(w, tag);
}
// Gate functions of the LayerNorm cells.  With fp32 storage the accurate expf / tanhf: three
// normalisations per step amplify a relative error of 1e-6 (the ex2.approx-based fast forms)
// a hundredfold over a few dozen steps, which is most of the distance between these kernels
// and the reference's float32 path on the 3-layer bidirectional configuration.  bf16 storage
// keeps the fast forms (its bar is 2e-2).
template <int SPLIT> __device__ __forceinline__ float ln_sigmoid(float x) {
  return SPLIT == 2 ? 1.0f / (1.0f + expf(-x)) : sigmoid_fast(x);
}
template <int SPLIT> __device__ __forceinline__ float ln_tanh(float x) {
  if (SPLIT != 2) return tanh_fast(x);
  // 1 - 2 / (1 + e^{2x}) with the accurate expf and a true division: absolute error ~1e-7
  const float e = expf(2.0f * fminf(fmaxf(x, -15.0f), 15.0f));
  return 1.0f - 2.0f / (1.0f + e);
}

// x = p[0] + p[1] + p[2], each the bf16 rounding of what the previous ones left.
__device__ __forceinline__ void split3_bf16(float x, float (&p)[3]) {
  p[0] = __bfloat162float(__float2bfloat16_rn(x));
  const float r1 = x - p[0];
  p[1] = __bfloat162float(__float2bfloat16_rn(r1));
  p[2] = __bfloat162float(__float2bfloat16_rn(r1 - p[1]));
}

// Sum over the 16 consecutive lanes that own one batch row.
__device__ __forceinline__ float row16_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  v += __shfl_xor_sync(0xffffffffu, v, 2);
  v += __shfl_xor_sync(0xffffffffu, v, 4);
  v += __shfl_xor_sync(0xffffffffu, v, 8);
  return v;
}

// One exchange round of per-row pairs among the CTAs of a batch slice, in two halves.
//   area : this exchange's buffer, laid out [rows][nHS][2] tagged words
// stat_publish: lane ul == 0 of the row's 16-thread group stores this CTA's pair (a, b).
__device__ __forceinline__ void stat_publish(uint32_t* area, int row, int hs, int nHS,
                                             uint32_t tag, float a, float b) {
  publish_u32x2(area + ((size_t)row * nHS + hs) * 2, fword_encode(a, tag), fword_encode(b, tag));
}
// stat_collect: thread ul of the group fetches the pairs of sources ul, ul+16, ul+32, ul+48
// (zero where there is no such source, or when `active` is false); the caller combines them
// and finishes with row16_sum.  Returns false if the wait was abandoned.
__device__ __forceinline__ bool stat_collect(const uint32_t* area, int row, int nHS, int ul,
                                             uint32_t tag, bool active, float (&out_a)[4],
                                             float (&out_b)[4], const Sync& sync, int* s_abort,
                                             int code) {
  const uint32_t* rowp = area + (size_t)row * nHS * 2;
  uint2 w[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) w[k] = make_uint2(tag, tag);
  bool alive = true;
  if (active) {
    const long long t0 = clock64();
    unsigned int spins = 0;
    for (;;) {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int s = ul + 16 * k;
        if (s < nHS) {
          const uint32_t* q = rowp + s * 2;
          asm volatile("ld.relaxed.gpu.global.v2.u32 {%0,%1}, [%2];"
                       : "=r"(w[k].x), "=r"(w[k].y) : "l"(q) : "memory");
        }
      }
      bool ok = true;
#pragma unroll
      for (int k = 0; k < 4; ++k) ok = ok && fword_ready(w[k].x, tag) && fword_ready(w[k].y, tag);
      if (ok) break;
      if ((++spins & 63u) == 0) {
        if (*reinterpret_cast<volatile int*>(sync.abort_flag) != 0) { alive = false; break; }
        if (clock64() - t0 > SPIN_LIMIT_CYCLES) {
          raise_abort(sync, s_abort, code, blockIdx.x * 1000 + threadIdx.x, row);
          alive = false;
          break;
        }
      }
    }
  }
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const bool have = active && alive && (ul + 16 * k) < nHS;
    out_a[k] = have ? fword_value(w[k].x) : 0.f;
    out_b[k] = have ? fword_value(w[k].y) : 0.f;
  }
  return alive;
}

// Combines (mean, M2) pairs of nHS column slices (slice s holds cnt(s) values) into the row's
// mean and 1/sqrt(var + eps).  Executed by all 16 lanes of the row group.
__device__ __forceinline__ void chan_combine(const float (&m)[4], const float (&m2)[4], int ul,
                                             int nHS, int width, int per_slice, float& mean,
                                             float& invstd) {
  float cnt[4], s = 0.f;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int src = ul + 16 * k;
    const int c = src < nHS ? min(per_slice, width - src * per_slice) : 0;
    cnt[k] = (float)c;
    s += cnt[k] * m[k];
  }
  mean = row16_sum(s) / (float)width;
  float q = 0.f;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float d = m[k] - mean;
    q += m2[k] + cnt[k] * d * d;
  }
  invstd = rsqrtf(row16_sum(q) / (float)width + kLnEps);
}

// ---------------------------------------------------------------------------------------
// Forward
// ---------------------------------------------------------------------------------------
template <int G, int KSW, int SPLIT, int MTMAX, typename T>
__global__ void __launch_bounds__(THREADS, 1) ln_fwd_kernel(const LnFwdParams p) {
  static_assert(G == 4 || G == 3, "G = 4: LayerNormLSTM, G = 3: LayerNormGRU");
  constexpr int COLS = G * U;
  constexpr int NT = COLS / 8;
  constexpr int KW = KSW * 16;
  constexpr int KPAD = WARPS * KW;
  constexpr int AROW = KPAD + 8;
  constexpr int PROW = COLS + 8;
  extern __shared__ __align__(16) uint8_t smem[];
  const int BNR = p.MT * 16;
  // fp32 storage: h in three bf16 planes (a0 + a1 + a2 carries 24 mantissa bits)
  constexpr int PA = SPLIT == 2 ? 3 : 1;
  __nv_bfloat16* a_hi = reinterpret_cast<__nv_bfloat16*>(smem);
  const size_t a_plane = (size_t)16 * AROW;  // one m-tile; each warp only touches its own K range
  float* part = reinterpret_cast<float*>(smem + (size_t)PA * a_plane * 2);  // [2][8][16][PROW]
  // fp32 storage: third plane of R as ready-made B fragments, [warp][nt][ks][half][lane]
  uint32_t* b2f = reinterpret_cast<uint32_t*>(part + (size_t)2 * WARPS * 16 * PROW);
  __shared__ int s_abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int gq = lane >> 2, q = lane & 3;
  const int hs = blockIdx.x % p.nHS, bs = blockIdx.x / p.nHS;
  const int nBS = gridDim.x / p.nHS;
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
      const int cl = nt * 8 + gq;  // local column, unit-major: cl = u*G + gate
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
            float p0[3], p1[3];
            split3_bf16(x0, p0);
            split3_bf16(x1, p1);
            rf[0][nt][ks][half] = pack_bf16(p0[0], p1[0]);
            rf[SPLIT - 1][nt][ks][half] = pack_bf16(p0[1], p1[1]);
            b2f[((((size_t)warp * NT + nt) * KSW + ks) * 2 + half) * 32 + lane] =
                pack_bf16(p0[2], p1[2]);
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
  const bool unit_pad = !unit_ok && (u0 + ul) < Hx;
  const float cnt_units = (float)min(U, H - u0);  // valid units of this CTA
  T* hbuf = reinterpret_cast<T*>(p.h);
  T* cbuf = reinterpret_cast<T*>(p.c);
  T* vbuf = reinterpret_cast<T*>(p.v);
  T* rhbuf = reinterpret_cast<T*>(p.act_Rh);
  T* cnbuf = reinterpret_cast<T*>(p.act_c_norm);
  T* cache1 = reinterpret_cast<T*>(p.cache_Rh);
  T* cache3 = reinterpret_cast<T*>(p.cache_c);
  const T* mask = reinterpret_cast<const T*>(p.mask);
  const T* wx = reinterpret_cast<const T*>(p.Wx);
  float bias[G], bias2[G], g1[G];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    bias[g] = unit_ok ? ld(reinterpret_cast<const T*>(p.b) + g * H + u0 + ul) : 0.f;
    bias2[g] = (G == 3 && unit_ok) ? ld(reinterpret_cast<const T*>(p.b2) + g * H + u0 + ul) : 0.f;
    g1[g] = unit_ok ? ld(reinterpret_cast<const T*>(p.gamma_Rh) + g * H + u0 + ul) : 0.f;
  }
  const float gh = (G == 4 && unit_ok) ? ld(reinterpret_cast<const T*>(p.gamma_h) + u0 + ul) : 0.f;
  const float bh = (G == 4 && unit_ok) ? ld(reinterpret_cast<const T*>(p.beta_h) + u0 + ul) : 0.f;
  float c_reg[MTMAX], h_reg[MTMAX];
  (void)gh; (void)bh; (void)cbuf; (void)cnbuf; (void)cache3; (void)cnt_units;
#pragma unroll
  for (int mt = 0; mt < MTMAX; ++mt) {
    const int n = n0 + mt * 16 + nl;
    const bool ok = mt < p.MT && n < N && unit_ok;
    h_reg[mt] = ok ? ld(hbuf + (long long)n * H + u0 + ul) : 0.f;
    c_reg[mt] = (G == 4 && ok) ? ld(cbuf + (long long)n * H + u0 + ul) : 0.f;
  }

  __syncthreads();

  const size_t sarea = (size_t)BNR * p.nHS * 2;  // words of one (statistic, parity, slice) area
  bool alive = true;
  int pbuf = 0;
  for (int t = 0; t < p.T && alive; ++t) {
    const uint32_t tag = (((uint32_t)t >> 1) & 1u) ^ 1u;
    uint32_t* area1 = p.sbuf + (((size_t)0 * 2 + (t & 1)) * nBS + bs) * sarea;
    uint32_t* area3 = p.sbuf + (((size_t)1 * 2 + (t & 1)) * nBS + bs) * sarea;
    // ---- loads that do not depend on the recurrence: LN(x.W) (+ zoneout mask)
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

    // ---- stage A: step product, pre-norm h.R saved, its row statistics published
    float rh[MTMAX][G];
    bool stop = false;  // CTA-uniform: taken from a barrier-wide OR of the abort flag
#pragma unroll
    for (int mt = 0; mt < MTMAX; ++mt) {
#pragma unroll
      for (int g = 0; g < G; ++g) rh[mt][g] = 0.f;
      if (mt < p.MT && !stop) {
        // ---- this warp's K range of h_t for the rows of m-tile mt -> the A planes.  At t = 0
        // the caller's initial state; afterwards the tagged words the producers wrote.
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
              float x[4];
#pragma unroll
              for (int j4 = 0; j4 < 4; ++j4)
                x[j4] = (n < N && k + j4 < H) ? ld(hbuf + (long long)n * H + k + j4) : 0.f;
              if (SPLIT == 2) {
                float px[3], py[3], pz[3], pw[3];
                split3_bf16(x[0], px); split3_bf16(x[1], py);
                split3_bf16(x[2], pz); split3_bf16(x[3], pw);
#pragma unroll
                for (int k3 = 0; k3 < PA; ++k3)
                  *reinterpret_cast<uint2*>(a_hi + k3 * a_plane + (size_t)r * AROW + k) = make_uint2(
                      pack_bf16(px[k3 % 3], py[k3 % 3]), pack_bf16(pz[k3 % 3], pw[k3 % 3]));
              } else {
                *reinterpret_cast<uint2*>(a_hi + (size_t)r * AROW + k) =
                    make_uint2(pack_bf16(x[0], x[1]), pack_bf16(x[2], x[3]));
              }
            }
          } else if (alive && !HB_DBG(p, 1)) {
            const uint32_t want = (((uint32_t)(t - 1) >> 1) & 1u) ^ 1u;
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
                else w[i] = SPLIT == 2 ? make_uint4(want, want, want, want)
                                       : make_uint4(want << 30, want << 30, want << 30, want << 30);
              }
              // one logic instruction per word: the tag bit of `bad` ends up set if any is stale
              uint32_t bad = 0;
              const uint32_t wtag = SPLIT == 2 ? want : want << 30;
#pragma unroll
              for (int i = 0; i < CPL; ++i)
                bad |= (w[i].x ^ wtag) | (w[i].y ^ wtag) | (w[i].z ^ wtag) | (w[i].w ^ wtag);
              const bool ok = (bad & (SPLIT == 2 ? 1u : 0x40000000u)) == 0;
              if (__all_sync(0xffffffffu, ok)) break;
              if ((++spins & 63u) == 0) {
                bool quit = *reinterpret_cast<volatile int*>(p.sync.abort_flag) != 0;
                if (!quit && clock64() - t0 > SPIN_LIMIT_CYCLES) {
                  raise_abort(p.sync, &s_abort, 26, blockIdx.x, t);
                  quit = true;
                }
                if (__any_sync(0xffffffffu, quit)) { alive = false; break; }
              }
            }
            if (!alive) *reinterpret_cast<volatile int*>(&s_abort) = 1;  // the barrier below sees it
#pragma unroll
            for (int i = 0; i < CPL; ++i) {
              const int e = lane + i * 32;
              const int r = e / CPR, k = warp * KW + (e % CPR) * 4;
              if (SPLIT == 2) {
                float px[3], py[3], pz[3], pw[3];
                split3_bf16(fword_value(w[i].x), px);
                split3_bf16(fword_value(w[i].y), py);
                split3_bf16(fword_value(w[i].z), pz);
                split3_bf16(fword_value(w[i].w), pw);
#pragma unroll
                for (int k3 = 0; k3 < PA; ++k3)
                  *reinterpret_cast<uint2*>(a_hi + k3 * a_plane + (size_t)r * AROW + k) = make_uint2(
                      pack_bf16(px[k3 % 3], py[k3 % 3]), pack_bf16(pz[k3 % 3], pw[k3 % 3]));
              } else {
                *reinterpret_cast<uint2*>(a_hi + (size_t)r * AROW + k) = make_uint2(
                    __byte_perm(w[i].x, w[i].y, 0x5410), __byte_perm(w[i].z, w[i].w, 0x5410));
              }
            }
          }
          __syncwarp();
        }
        float acc[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
        // fp32 storage, six products in three passes over the K range, smallest terms first.
        // The tensor core adds each product into the fp32 accumulator with truncation (about
        // half an ulp of the accumulator, always the same way); with the passes ordered like
        // this only the last pass's KSW accumulations happen at the full magnitude of the
        // result, instead of all 6 * KSW of them.
        if (SPLIT == 2) {
#pragma unroll
          for (int pass = 0; pass < (HB_DBG(p, 2) ? 0 : 3); ++pass) {
#pragma unroll
            for (int ks = 0; ks < KSW; ++ks) {
              const int row = lane & 15;
              const int kcol = warp * KW + ks * 16 + (lane >> 4) * 8;
              uint32_t a0[4], a1[4], a2[4];
              ldmatrix_x4(smem_u32(a_hi + (size_t)row * AROW + kcol), a0);
              if (pass < 2) ldmatrix_x4(smem_u32(a_hi + a_plane + (size_t)row * AROW + kcol), a1);
              if (pass == 0)
                ldmatrix_x4(smem_u32(a_hi + (PA - 1) * a_plane + (size_t)row * AROW + kcol), a2);
#pragma unroll
              for (int nt = 0; nt < NT; ++nt) {
                if (pass == 0) {  // terms of relative size 2^-16
                  const uint32_t* bq = b2f + ((((size_t)warp * NT + nt) * KSW + ks) * 2) * 32 + lane;
                  mma_bf16(acc[nt], a0, bq[0], bq[32]);
                  mma_bf16(acc[nt], a2, rf[0][nt][ks][0], rf[0][nt][ks][1]);
                  mma_bf16(acc[nt], a1, rf[SPLIT - 1][nt][ks][0], rf[SPLIT - 1][nt][ks][1]);
                } else if (pass == 1) {  // 2^-8
                  mma_bf16(acc[nt], a0, rf[SPLIT - 1][nt][ks][0], rf[SPLIT - 1][nt][ks][1]);
                  mma_bf16(acc[nt], a1, rf[0][nt][ks][0], rf[0][nt][ks][1]);
                } else {
                  mma_bf16(acc[nt], a0, rf[0][nt][ks][0], rf[0][nt][ks][1]);
                }
              }
            }
          }
        } else {
#pragma unroll
          for (int ks = 0; ks < (HB_DBG(p, 2) ? 0 : KSW); ++ks) {
            const int row = lane & 15;
            const int kcol = warp * KW + ks * 16 + (lane >> 4) * 8;
            uint32_t a0[4];
            ldmatrix_x4(smem_u32(a_hi + (size_t)row * AROW + kcol), a0);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) mma_bf16(acc[nt], a0, rf[0][nt][ks][0], rf[0][nt][ks][1]);
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
        stop = __syncthreads_or(*reinterpret_cast<volatile int*>(&s_abort)) != 0;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
          const float* src = pb + ((size_t)w * 16 + nl) * PROW + ul * G;
          if (G == 4) {
            const float4 f = *reinterpret_cast<const float4*>(src);
            rh[mt][0] += f.x; rh[mt][1] += f.y; rh[mt][2] += f.z; rh[mt][G - 1] += f.w;
          } else {
#pragma unroll
            for (int g = 0; g < G; ++g) rh[mt][g] += src[g];
          }
        }
        pbuf ^= 1;
        const int n = n0 + mt * 16 + nl;
        const bool ok = n < N && unit_ok;
        if (ok) {
          T* rt = rhbuf + ((long long)t * N + n) * GH + u0 + ul;
#pragma unroll
          for (int g = 0; g < G; ++g) st(rt + g * H, rh[mt][g]);
        }
        float s = 0.f;
        if (ok) {
#pragma unroll
          for (int g = 0; g < G; ++g) s += rh[mt][g];
        }
        const float m_loc = row16_sum(s) / (G * cnt_units);
        float dd = 0.f;
        if (ok) {
#pragma unroll
          for (int g = 0; g < G; ++g) dd += (rh[mt][g] - m_loc) * (rh[mt][g] - m_loc);
        }
        dd = row16_sum(dd);
        if (ul == 0 && n < N) stat_publish(area1, mt * 16 + nl, hs, p.nHS, tag, m_loc, dd);
      }
    }
    if (stop) break;

    if constexpr (G == 4) {
      // ---- stage B: LayerNorm of h.R, gates, new cell state, its row statistics published
      float og[MTMAX], cnew[MTMAX];
  #pragma unroll
      for (int mt = 0; mt < MTMAX; ++mt) {
        og[mt] = cnew[mt] = 0.f;
        if (mt < p.MT) {
          const int n = n0 + mt * 16 + nl;
          const bool ok = n < N && unit_ok;
          float sa[4], sb[4], mean1, inv1;
          if (!stat_collect(area1, mt * 16 + nl, p.nHS, ul, tag, n < N && !HB_DBG(p, 4), sa, sb, p.sync, &s_abort, 27))
            *reinterpret_cast<volatile int*>(&s_abort) = 1;
          chan_combine(sa, sb, ul, p.nHS, GH, COLS, mean1, inv1);
          float pre[G];
  #pragma unroll
          for (int g = 0; g < G; ++g)
            pre[g] = (rh[mt][g] - mean1) * inv1 * g1[g] + wxr[mt][g] + bias[g];
          const float i = ln_sigmoid<SPLIT>(pre[0]);
          const float gg = ln_tanh<SPLIT>(pre[1]);
          const float f = ln_sigmoid<SPLIT>(pre[2]);
          const float o = ln_sigmoid<SPLIT>(pre[G - 1]);
          const float c_new = f * c_reg[mt] + i * gg;
          og[mt] = o;
          cnew[mt] = c_new;
          const float s = row16_sum(ok ? c_new : 0.f);
          const float m_loc = s / cnt_units;
          const float dd = row16_sum(ok ? (c_new - m_loc) * (c_new - m_loc) : 0.f);
          if (ul == 0 && n < N) stat_publish(area3, mt * 16 + nl, hs, p.nHS, tag, m_loc, dd);
          if (ok) {
            st(cbuf + (long long)(t + 1) * NH + (long long)n * H + u0 + ul, c_new);
            if (p.training) {
              T* vt = vbuf + ((long long)t * N + n) * GH + u0 + ul;
              st(vt, i); st(vt + H, gg); st(vt + 2 * H, f); st(vt + 3 * H, o);
            }
          }
          if (hs == 0 && ul == 0 && n < N) {
            st(cache1 + ((long long)t * N + n) * 2, mean1);
            st(cache1 + ((long long)t * N + n) * 2 + 1, inv1);
          }
        }
      }

      // ---- stage C: LayerNorm of the cell state, output, h_t published
  #pragma unroll
      for (int mt = 0; mt < MTMAX; ++mt) {
        if (mt < p.MT) {
          const int n = n0 + mt * 16 + nl;
          const bool ok = n < N && unit_ok;
          float sa[4], sb[4], mean3, inv3;
          if (!stat_collect(area3, mt * 16 + nl, p.nHS, ul, tag, n < N && !HB_DBG(p, 4), sa, sb, p.sync, &s_abort, 28))
            *reinterpret_cast<volatile int*>(&s_abort) = 1;
          chan_combine(sa, sb, ul, p.nHS, H, U, mean3, inv3);
          const float c_norm = (cnew[mt] - mean3) * inv3 * gh + bh;
          float h_new = og[mt] * ln_tanh<SPLIT>(c_norm);
          if (p.has_zoneout)
            h_new = p.training ? zoneout<true>(h_new, h_reg[mt], p.zoneout_prob, mk[mt])
                               : zoneout<false>(h_new, h_reg[mt], p.zoneout_prob, mk[mt]);
          h_new = round_to_storage<T>(h_new);
          uint32_t* xdst = p.xbuf + (size_t)(t & 1) * N * Hx + (size_t)n * Hx + u0 + ul;
          if (ok) {
            if (t + 1 < p.T) publish_u32(xdst, hword_encode<SPLIT>(h_new, tag));
            const long long o0 = (long long)n * H + u0 + ul;
            st(hbuf + (long long)(t + 1) * NH + o0, h_new);
            st(cnbuf + (long long)t * NH + o0, c_norm);
            h_reg[mt] = h_new;
            c_reg[mt] = cnew[mt];
          } else if (n < N && unit_pad && t + 1 < p.T) {
            publish_u32(xdst, hword_encode<SPLIT>(0.0f, tag));
          }
          if (hs == 0 && ul == 0 && n < N) {
            st(cache3 + ((long long)t * N + n) * 2, mean3);
            st(cache3 + ((long long)t * N + n) * 2 + 1, inv3);
          }
        }
      }
    } else {
      // ---- stage B: LayerNorm of h.R, gates, output, h_t published
  #pragma unroll
      for (int mt = 0; mt < MTMAX; ++mt) {
        if (mt < p.MT) {
          const int n = n0 + mt * 16 + nl;
          const bool ok = n < N && unit_ok;
          float sa[4], sb[4], mean1, inv1;
          if (!stat_collect(area1, mt * 16 + nl, p.nHS, ul, tag, n < N && !HB_DBG(p, 4), sa, sb, p.sync, &s_abort, 27))
            *reinterpret_cast<volatile int*>(&s_abort) = 1;
          chan_combine(sa, sb, ul, p.nHS, GH, COLS, mean1, inv1);
          float rn[G];
  #pragma unroll
          for (int g = 0; g < G; ++g) rn[g] = (rh[mt][g] - mean1) * inv1 * g1[g] + bias2[g];
          const float z = ln_sigmoid<SPLIT>(wxr[mt][0] + bias[0] + rn[0]);
          const float r = ln_sigmoid<SPLIT>(wxr[mt][1] + bias[1] + rn[1]);
          const float qg = rn[2];
          const float gg = ln_tanh<SPLIT>(wxr[mt][2] + bias[2] + r * qg);
          float h_new = z * h_reg[mt] + (1.0f - z) * gg;
          if (p.has_zoneout)
            h_new = p.training ? zoneout<true>(h_new, h_reg[mt], p.zoneout_prob, mk[mt])
                               : zoneout<false>(h_new, h_reg[mt], p.zoneout_prob, mk[mt]);
          h_new = round_to_storage<T>(h_new);
          uint32_t* xdst = p.xbuf + (size_t)(t & 1) * N * Hx + (size_t)n * Hx + u0 + ul;
          if (ok) {
            if (t + 1 < p.T) publish_u32(xdst, hword_encode<SPLIT>(h_new, tag));
            st(hbuf + (long long)(t + 1) * NH + (long long)n * H + u0 + ul, h_new);
            if (p.training && vbuf) {
              T* vt = vbuf + ((long long)t * N + n) * 4 * H + u0 + ul;
              st(vt, z); st(vt + H, r); st(vt + 2 * H, gg); st(vt + 3 * H, qg);
            }
            h_reg[mt] = h_new;
          } else if (n < N && unit_pad && t + 1 < p.T) {
            publish_u32(xdst, hword_encode<SPLIT>(0.0f, tag));
          }
          if (hs == 0 && ul == 0 && n < N) {
            st(cache1 + ((long long)t * N + n) * 2, mean1);
            st(cache1 + ((long long)t * N + n) * 2 + 1, inv1);
          }
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------------------
// Backward
// ---------------------------------------------------------------------------------------
template <int G, int NTW, int SPLIT, int MTMAX, typename T>
__global__ void __launch_bounds__(THREADS, 1) ln_bwd_kernel(const LnBwdParams p) {
  static_assert(G == 4 || G == 3, "G = 4: LayerNormLSTM, G = 3: LayerNormGRU");
  constexpr int COLS = G * U;
  constexpr int KS = COLS / 16;  // 64 or 48 gate columns: no padding
  constexpr int AROW = COLS + 8;
  extern __shared__ __align__(16) uint8_t smem[];
  const int BNR = p.MT * 16;
  constexpr int PA = SPLIT == 2 ? 3 : 1;  // fp32 storage: three bf16 planes per operand
  __nv_bfloat16* a_base = reinterpret_cast<__nv_bfloat16*>(smem);  // [2][PA][BNR][AROW]
  const size_t a_plane = (size_t)BNR * AROW;
  // fp32 storage: third plane of R^T as B fragments, [warp][nt][ks][half][lane]
  uint32_t* b2f = reinterpret_cast<uint32_t*>(smem + (size_t)2 * PA * a_plane * 2);
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
  for (int e = tid; e < 2 * PA * (int)a_plane; e += THREADS) a_base[e] = __float2bfloat16_rn(0.f);

  // ---- R[:, slice]^T as B fragments (k = local gate column u*G+gate, n = output unit j)
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
            const int cl = ks * 16 + half * 8 + 2 * q + e;
            const int u = cl / G, gate = cl % G;
            float val = 0.f;
            if (j < H && (u0 + u) < H) {
              const long long col = (long long)gate * H + u0 + u;
              val = p.r_transposed ? ld(R + col * H + j) : ld(R + (long long)j * GH + col);
            }
            x[e] = val;
          }
          if (SPLIT == 2) {
            float p0[3], p1[3];
            split3_bf16(x[0], p0);
            split3_bf16(x[1], p1);
            rf[0][nt][ks][half] = pack_bf16(p0[0], p1[0]);
            rf[SPLIT - 1][nt][ks][half] = pack_bf16(p0[1], p1[1]);
            b2f[((((size_t)warp * NTW + nt) * KS + ks) * 2 + half) * 32 + lane] =
                pack_bf16(p0[2], p1[2]);
          } else {
            rf[0][nt][ks][half] = pack_bf16(x[0], x[1]);
          }
        }
      }
    }
  }

  const int nl = tid >> 4, ul = tid & 15;
  const bool unit_ok = (u0 + ul) < H;
  const T* cbuf = reinterpret_cast<const T*>(p.c);
  const T* hbuf = reinterpret_cast<const T*>(p.h);
  T* dpb = reinterpret_cast<T*>(p.dp);
  T* dqb = reinterpret_cast<T*>(p.dq);
  T* vbuf = reinterpret_cast<T*>(p.v);
  T* rhbuf = reinterpret_cast<T*>(p.act_Rh);
  const T* cnbuf = reinterpret_cast<const T*>(p.act_c_norm);
  const T* cache1 = reinterpret_cast<const T*>(p.cache_Rh);
  const T* cache3 = reinterpret_cast<const T*>(p.cache_c);
  const T* dhn = reinterpret_cast<const T*>(p.dh_new);
  const T* dcn = reinterpret_cast<const T*>(p.dc_new);
  const T* mask = reinterpret_cast<const T*>(p.mask);
  float g1[G];
#pragma unroll
  for (int g = 0; g < G; ++g)
    g1[g] = unit_ok ? ld(reinterpret_cast<const T*>(p.gamma_Rh) + g * H + u0 + ul) : 0.f;
  const float gh = (G == 4 && unit_ok) ? ld(reinterpret_cast<const T*>(p.gamma_h) + u0 + ul) : 0.f;
  (void)gh; (void)cbuf; (void)hbuf; (void)dpb; (void)dqb; (void)cnbuf; (void)cache3; (void)dcn;
  const float inv_H = 1.0f / (float)H, inv_GH = 1.0f / (float)GH;

  float dh_c[MTMAX], dc_c[MTMAX];
#pragma unroll
  for (int mt = 0; mt < MTMAX; ++mt) {
    const int n = n0 + mt * 16 + nl;
    const bool ok = mt < p.MT && n < N && unit_ok;
    dh_c[mt] = ok ? p.dh_carry[(long long)n * H + u0 + ul] : 0.f;
    dc_c[mt] = (G == 4 && ok) ? p.dc_carry[(long long)n * H + u0 + ul] : 0.f;
  }
  float acc_g1[G], acc_gh = 0.f, acc_bh = 0.f;  // parameter gradients
#pragma unroll
  for (int g = 0; g < G; ++g) acc_g1[g] = 0.f;
  const size_t blk = (size_t)BNR * U;
  const size_t sarea = (size_t)BNR * p.nHS * 2;
  bool alive = true;
  __syncthreads();

  for (int t = p.T - 1; t >= 0 && alive; --t) {
    const int ti = p.T - 1 - t;
    const uint32_t tag = (((uint32_t)ti >> 1) & 1u) ^ 1u;
    uint32_t* area3 = p.sbuf + (((size_t)0 * 2 + (ti & 1)) * nBS + bs) * sarea;
    uint32_t* area1 = p.sbuf + (((size_t)1 * 2 + (ti & 1)) * nBS + bs) * sarea;
    // ---- loads independent of the carried gradient
    // gv: saved activations (LSTM i,g,f,o; GRU z,r,g,q); rhv: pre-norm h.R
    float gv[MTMAX][4], rhv[MTMAX][G], cprev[MTMAX], cx3[MTMAX], cnv[MTMAX], dhv[MTMAX],
        dcv[MTMAX], mk[MTMAX], mean1[MTMAX], inv1[MTMAX], inv3[MTMAX], hprev[MTMAX];
#pragma unroll
    for (int mt = 0; mt < MTMAX; ++mt) {
      const int n = n0 + mt * 16 + nl;
      const bool rok = mt < p.MT && n < N;
      const bool ok = rok && unit_ok;
      const long long o0 = (long long)n * H + u0 + ul;
      const long long w0 = ((long long)t * N + n) * GH + u0 + ul;
      const long long v0 = ((long long)t * N + n) * 4 * H + u0 + ul;
#pragma unroll
      for (int g = 0; g < 4; ++g) gv[mt][g] = ok ? ld(vbuf + v0 + g * H) : 0.f;
#pragma unroll
      for (int g = 0; g < G; ++g) rhv[mt][g] = ok ? ld(rhbuf + w0 + g * H) : 0.f;
      dhv[mt] = ok ? ld(dhn + (long long)(t + 1) * NH + o0) : 0.f;
      mk[mt] = (ok && p.has_zoneout) ? ld(mask + (long long)t * NH + o0) : 1.f;
      mean1[mt] = rok ? ld(cache1 + ((long long)t * N + n) * 2) : 0.f;
      inv1[mt] = rok ? ld(cache1 + ((long long)t * N + n) * 2 + 1) : 0.f;
      cprev[mt] = cx3[mt] = cnv[mt] = dcv[mt] = inv3[mt] = hprev[mt] = 0.f;
      if constexpr (G == 4) {
        dcv[mt] = ok ? ld(dcn + (long long)(t + 1) * NH + o0) : 0.f;
        cprev[mt] = ok ? ld(cbuf + (long long)t * NH + o0) : 0.f;
        cnv[mt] = ok ? ld(cnbuf + (long long)t * NH + o0) : 0.f;
        const float mean3 = rok ? ld(cache3 + ((long long)t * N + n) * 2) : 0.f;
        inv3[mt] = rok ? ld(cache3 + ((long long)t * N + n) * 2 + 1) : 0.f;
        cx3[mt] = ok ? ld(cbuf + (long long)(t + 1) * NH + o0) - mean3 : 0.f;
      } else {
        hprev[mt] = ok ? ld(hbuf + (long long)t * NH + o0) : 0.f;
      }
      // Ask L2 for the next step's inputs now: when that step loads them they come back from
      // L2 in a fraction of the HBM latency and do not sit in the SM's miss queue while the
      // polling loads of the exchange need it.
      if (MTMAX == 1 && ok && t > 0 && !HB_DBG(p, 512)) {
        const long long w1 = w0 - (long long)N * GH, v1 = v0 - (long long)N * 4 * H;
#pragma unroll
        for (int g = 0; g < 4; ++g) prefetch_l2(vbuf + v1 + g * H);
#pragma unroll
        for (int g = 0; g < G; ++g) prefetch_l2(rhbuf + w1 + g * H);
        prefetch_l2(dhn + (long long)t * NH + o0);
        if (p.has_zoneout) prefetch_l2(mask + (long long)(t - 1) * NH + o0);
        if constexpr (G == 4) {
          prefetch_l2(dcn + (long long)t * NH + o0);
          prefetch_l2(cbuf + (long long)(t - 1) * NH + o0);
          prefetch_l2(cnbuf + (long long)(t - 1) * NH + o0);
        } else {
          prefetch_l2(hbuf + (long long)(t - 1) * NH + o0);
        }
      }
    }

    // ---- recurrent part of dh_t: the partials published at the previous step
    if (ti > 0 && !HB_DBG(p, 1)) {
      const uint32_t want = (((uint32_t)(ti - 1) >> 1) & 1u) ^ 1u;
      const uint32_t* src =
          p.exch + ((((size_t)((ti - 1) & 1) * nBS + bs) * p.nHS + hs) * p.nHS) * blk;
      const int sg = ul & 3, quad = ul >> 2;
#pragma unroll
      for (int mt = 0; mt < MTMAX; ++mt) {
        if (mt < p.MT) {
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
                  raise_abort(p.sync, &s_abort, 37, blockIdx.x * 1000 + tid, ti * 100 + s0);
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
    alive = true;  // from here on failures only mark s_abort; the barriers below decide
    // All warps leave the wait above together.  Without this barrier the warps that are still
    // polling (32 KB of loads per round and CTA) keep the SM's load/store path full, and the
    // small statistic stores and loads of the warps that are already through queue up behind
    // them: measured 12.5 -> 9.8 us per step.
    if (__syncthreads_or(*reinterpret_cast<volatile int*>(&s_abort))) { alive = false; break; }

    float dgate[MTMAX][G];
    if constexpr (G == 4) {
      // ---- stage A: output gate and LayerNorm(c') input gradients; LN(c') row sums published
      float d_o[MTMAX], db3[MTMAX];
  #pragma unroll
      for (int mt = 0; mt < MTMAX; ++mt) {
        d_o[mt] = db3[mt] = 0.f;
        if (mt < p.MT) {
          const int n = n0 + mt * 16 + nl;
          float dh_total = dhv[mt] + dh_c[mt];
          float keep = 0.f;
          if (p.has_zoneout) {
            keep = (1.0f - mk[mt]) * dh_total;
            dh_total = mk[mt] * dh_total;
          }
          dh_c[mt] = keep;
          const float o = gv[mt][3];
          const float c_tanh = ln_tanh<SPLIT>(cnv[mt]);
          d_o[mt] = d_sigmoid(o) * (c_tanh * dh_total);
          const float dcn_ = d_tanh(c_tanh) * (o * dh_total);  // gradient w.r.t. LayerNorm(c')
          acc_gh += cx3[mt] * inv3[mt] * dcn_;
          acc_bh += dcn_;
          db3[mt] = gh * dcn_;
          const float s1 = row16_sum(cx3[mt] * db3[mt]);
          const float s2 = row16_sum(db3[mt]);
          if (ul == 0 && n < N) stat_publish(area3, mt * 16 + nl, hs, p.nHS, tag, s1, s2);
        }
      }

      // ---- stage B: gate gradients; LN(h.R) row sums published
  #pragma unroll
      for (int mt = 0; mt < MTMAX; ++mt) {
  #pragma unroll
        for (int g = 0; g < G; ++g) dgate[mt][g] = 0.f;
        if (mt < p.MT) {
          const int n = n0 + mt * 16 + nl;
          const bool ok = n < N && unit_ok;
          float sa[4], sb[4];
          if (!stat_collect(area3, mt * 16 + nl, p.nHS, ul, tag, n < N && !HB_DBG(p, 4), sa, sb, p.sync, &s_abort, 38))
            *reinterpret_cast<volatile int*>(&s_abort) = 1;
          const float S1 = row16_sum((sa[0] + sa[1]) + (sa[2] + sa[3]));
          const float S2 = row16_sum((sb[0] + sb[1]) + (sb[2] + sb[3]));
          const float r = inv3[mt];
          const float dsigma = -0.5f * S1 * r * r * r;
          const float dmu = -S2 * r;
          const float dcl = 2.0f * cx3[mt] * dsigma * inv_H + r * db3[mt] + dmu * inv_H;
          const float i = gv[mt][0], gg = gv[mt][1], f = gv[mt][2];
          const float dc_total = ok ? dcv[mt] + dc_c[mt] + dcl : 0.f;
          dgate[mt][0] = d_sigmoid(i) * (gg * dc_total);
          dgate[mt][1] = d_tanh(gg) * (i * dc_total);
          dgate[mt][2] = d_sigmoid(f) * (cprev[mt] * dc_total);
          dgate[mt][G - 1] = d_o[mt];
          dc_c[mt] = f * dc_total;
          float s1 = 0.f, s2 = 0.f;
  #pragma unroll
          for (int g = 0; g < G; ++g) {
            const float cx = rhv[mt][g] - mean1[mt];
            const float db = g1[g] * dgate[mt][g];
            if (ok) {
              s1 += cx * db;
              s2 += db;
              acc_g1[g] += cx * inv1[mt] * dgate[mt][g];
            }
          }
          s1 = row16_sum(s1);
          s2 = row16_sum(s2);
          if (ul == 0 && n < N) stat_publish(area1, mt * 16 + nl, hs, p.nHS, tag, s1, s2);
          if (ok) {
            const long long w0 = ((long long)t * N + n) * GH + u0 + ul;
  #pragma unroll
            for (int g = 0; g < G; ++g) st(vbuf + w0 + g * H, dgate[mt][g]);
            if (SPLIT == 2 && p.gpl) {
  #pragma unroll
              for (int g = 0; g < G; ++g) {
                float hi, lo;
                split_bf16(dgate[mt][g], hi, lo);
                p.gpl[w0 + g * H] = __float2bfloat16_rn(hi);
                p.gpl[p.gpl_stride + w0 + g * H] = __float2bfloat16_rn(lo);
              }
            }
          }
        }
      }

    } else {
      // ---- stage A: gate gradients (dp: w.r.t. LN(x.W)+bx, dq: w.r.t. LN(h.R)+br); LN(h.R)
      // row sums published
  #pragma unroll
      for (int mt = 0; mt < MTMAX; ++mt) {
  #pragma unroll
        for (int g = 0; g < G; ++g) dgate[mt][g] = 0.f;
        if (mt < p.MT) {
          const int n = n0 + mt * 16 + nl;
          const bool ok = n < N && unit_ok;
          float dh_total = dhv[mt] + dh_c[mt];
          float keep = 0.f;
          if (p.has_zoneout) {
            keep = (1.0f - mk[mt]) * dh_total;
            dh_total = mk[mt] * dh_total;
          }
          const float z = gv[mt][0], r = gv[mt][1], gg = gv[mt][2], qg = gv[mt][3];
          const float dg = (1.0f - z) * dh_total;
          const float dz = (hprev[mt] - gg) * dh_total;
          const float dp_g = d_tanh(gg) * dg;
          const float dp_r = d_sigmoid(r) * (dp_g * qg);
          const float dp_z = d_sigmoid(z) * dz;
          dgate[mt][0] = dp_z;
          dgate[mt][1] = dp_r;
          dgate[mt][2] = dp_g * r;
          dh_c[mt] = keep + z * dh_total;
          float s1 = 0.f, s2 = 0.f;
  #pragma unroll
          for (int g = 0; g < G; ++g) {
            const float cx = rhv[mt][g] - mean1[mt];
            const float db = g1[g] * dgate[mt][g];
            if (ok) {
              s1 += cx * db;
              s2 += db;
              acc_g1[g] += cx * inv1[mt] * dgate[mt][g];
            }
          }
          s1 = row16_sum(s1);
          s2 = row16_sum(s2);
          if (ul == 0 && n < N) stat_publish(area1, mt * 16 + nl, hs, p.nHS, tag, s1, s2);
          if (ok) {
            const long long w0 = ((long long)t * N + n) * GH + u0 + ul;
            st(dpb + w0, dp_z); st(dpb + w0 + H, dp_r); st(dpb + w0 + 2 * H, dp_g);
            st(dqb + w0, dp_z); st(dqb + w0 + H, dp_r); st(dqb + w0 + 2 * H, dgate[mt][2]);
          }
        }
      }

    }
    // ---- stage C: gradient w.r.t. the pre-norm h.R -> global and -> smem (A operand)
    __nv_bfloat16* a_hi = a_base + (size_t)(ti & 1) * PA * a_plane;
#pragma unroll
    for (int mt = 0; mt < MTMAX; ++mt) {
      if (mt < p.MT) {
        const int n = n0 + mt * 16 + nl;
        const bool ok = n < N && unit_ok;
        float sa[4], sb[4];
        if (!stat_collect(area1, mt * 16 + nl, p.nHS, ul, tag, n < N && !HB_DBG(p, 4), sa, sb, p.sync, &s_abort, 39))
          *reinterpret_cast<volatile int*>(&s_abort) = 1;
        const float S1 = row16_sum((sa[0] + sa[1]) + (sa[2] + sa[3]));
        const float S2 = row16_sum((sb[0] + sb[1]) + (sb[2] + sb[3]));
        const float r = inv1[mt];
        const float dsigma = -0.5f * S1 * r * r * r;
        const float dmu = -S2 * r;
        __nv_bfloat16* rowh = a_hi + (size_t)(mt * 16 + nl) * AROW + ul * G;
        const long long w0 = ((long long)t * N + n) * GH + u0 + ul;
#pragma unroll
        for (int g = 0; g < G; ++g) {
          const float cx = rhv[mt][g] - mean1[mt];
          const float x = ok ? 2.0f * cx * dsigma * inv_GH + r * (g1[g] * dgate[mt][g]) + dmu * inv_GH
                             : 0.f;
          float pl[3] = {x, 0.f, 0.f};
          if (SPLIT == 2) split3_bf16(x, pl);
#pragma unroll
          for (int k3 = 0; k3 < PA; ++k3) rowh[k3 * a_plane + g] = __float2bfloat16_rn(pl[k3 % 3]);
          if (ok) {
            st(rhbuf + w0 + g * H, x);
            if (SPLIT == 2 && p.gpl2) {
              p.gpl2[w0 + g * H] = __float2bfloat16_rn(pl[0]);
              p.gpl2[p.gpl_stride + w0 + g * H] = __float2bfloat16_rn(pl[1]);
            }
          }
        }
      }
    }
    if (t == 0) break;
    if (__syncthreads_or(*reinterpret_cast<volatile int*>(&s_abort))) { alive = false; break; }

    // ---- partial dh_{t-1}[rows, all units] = d(h.R) . R[:, slice]^T
    {
      uint32_t* dstbase = p.exch + ((size_t)(ti & 1) * nBS + bs) * p.nHS * p.nHS * blk;
      for (int mt = 0; mt < p.MT; ++mt) {
        float acc[NTW][4];
#pragma unroll
        for (int nt = 0; nt < NTW; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
        if (SPLIT == 2) {
          // three passes, smallest terms first (see the forward kernel)
#pragma unroll
          for (int pass = (HB_DBG(p, 8) ? 1 : 0); pass < (HB_DBG(p, 2) ? 0 : 3); ++pass) {
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
              const int row = mt * 16 + (lane & 15);
              const int kcol = ks * 16 + (lane >> 4) * 8;
              uint32_t a0[4], a1[4], a2[4];
              ldmatrix_x4(smem_u32(a_hi + (size_t)row * AROW + kcol), a0);
              if (pass < 2) ldmatrix_x4(smem_u32(a_hi + a_plane + (size_t)row * AROW + kcol), a1);
              if (pass == 0)
                ldmatrix_x4(smem_u32(a_hi + (PA - 1) * a_plane + (size_t)row * AROW + kcol), a2);
#pragma unroll
              for (int nt = 0; nt < NTW; ++nt) {
                if (pass == 0) {
                  const uint32_t* bq = b2f + ((((size_t)warp * NTW + nt) * KS + ks) * 2) * 32 + lane;
                  mma_bf16(acc[nt], a0, bq[0], bq[32]);
                  mma_bf16(acc[nt], a2, rf[0][nt][ks][0], rf[0][nt][ks][1]);
                  mma_bf16(acc[nt], a1, rf[SPLIT - 1][nt][ks][0], rf[SPLIT - 1][nt][ks][1]);
                } else if (pass == 1) {
                  mma_bf16(acc[nt], a0, rf[SPLIT - 1][nt][ks][0], rf[SPLIT - 1][nt][ks][1]);
                  mma_bf16(acc[nt], a1, rf[0][nt][ks][0], rf[0][nt][ks][1]);
                } else {
                  mma_bf16(acc[nt], a0, rf[0][nt][ks][0], rf[0][nt][ks][1]);
                }
              }
            }
          }
        } else {
#pragma unroll
          for (int ks = 0; ks < (HB_DBG(p, 2) ? 0 : KS); ++ks) {
            const int row = mt * 16 + (lane & 15);
            const int kcol = ks * 16 + (lane >> 4) * 8;
            uint32_t a0[4];
            ldmatrix_x4(smem_u32(a_hi + (size_t)row * AROW + kcol), a0);
#pragma unroll
            for (int nt = 0; nt < NTW; ++nt) mma_bf16(acc[nt], a0, rf[0][nt][ks][0], rf[0][nt][ks][1]);
          }
        }
#pragma unroll
        for (int nt = 0; nt < NTW; ++nt) {
          const int j = (warp * NTW + nt) * 8 + 2 * q;
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
  }

  // ---- carries and per-row-group parameter-gradient partials out
  if (alive && !*reinterpret_cast<volatile int*>(&s_abort)) {
#pragma unroll
    for (int mt = 0; mt < MTMAX; ++mt) {
      const int n = n0 + mt * 16 + nl;
      if (mt < p.MT && n < N && unit_ok) {
        p.dh_carry[(long long)n * H + u0 + ul] = dh_c[mt];
        if (G == 4) p.dc_carry[(long long)n * H + u0 + ul] = dc_c[mt];
      }
    }
  }
  if (unit_ok) {
    const long long r = (long long)bs * 16 + nl;
#pragma unroll
    for (int g = 0; g < G; ++g) p.dgRh_part[r * GH + g * H + u0 + ul] = acc_g1[g];
    if (G == 4) {
      p.dgh_part[r * H + u0 + ul] = acc_gh;
      p.dbh_part[r * H + u0 + ul] = acc_bh;
    }
  }
}

// ---------------------------------------------------------------------------------------
// Host-side dispatch (instantiated one storage type per translation unit)
// ---------------------------------------------------------------------------------------
template <int G, int SPLIT, typename T>
int run_ln_fwd(LnFwdParams& p, const Geometry& g, cudaStream_t s) {
  const int ksw = ceil_div(ceil_div(p.H, 16), WARPS);
  auto smem_for = [&](int KSW) {
    const size_t arow = (size_t)WARPS * KSW * 16 + 8;
    return (size_t)(SPLIT == 2 ? 3 : 1) * 16 * arow * 2 +
           (size_t)2 * WARPS * 16 * (G * U + 8) * 4 +
           (SPLIT == 2 ? (size_t)KSW * WARPS * (G * U / 8) * 256 : 0);
  };
  const int grid = g.nHS * g.nBS;
#define HB_FWD(KSW)                                                                       \
  if (ksw <= KSW) {                                                                       \
    if (smem_for(KSW) > 220 * 1024) return HASTE_B200_ERR_UNSUPPORTED;                    \
    if (g.MT == 1)                                                                        \
      return launch_coop(ln_fwd_kernel<G, KSW, SPLIT, 1, T>, grid, smem_for(KSW), &p, s);    \
    return launch_coop(ln_fwd_kernel<G, KSW, SPLIT, 4, T>, grid, smem_for(KSW), &p, s);      \
  }
  HB_FWD(1)
  HB_FWD(2)
  HB_FWD(4)
  if constexpr (SPLIT == 1) { HB_FWD(8) }
#undef HB_FWD
  return HASTE_B200_ERR_UNSUPPORTED;
}

inline int ntw_pad(int ntw) { return ntw <= 1 ? 1 : ntw <= 2 ? 2 : ntw <= 4 ? 4 : ntw <= 8 ? 8 : 16; }

template <int G, int SPLIT, typename T>
int run_ln_bwd(LnBwdParams& p, const Geometry& g, cudaStream_t s) {
  const int ntw = ceil_div(ceil_div(p.H, 8), WARPS);
  const size_t smem = (size_t)2 * (SPLIT == 2 ? 3 : 1) * g.MT * 16 * (G * U + 8) * 2 +
                      (SPLIT == 2 ? (size_t)ntw_pad(ntw) * WARPS * (G * U / 16) * 256 : 0);  // + third plane of R^T
  const int grid = g.nHS * g.nBS;
#define HB_BWD(NTW)                                                                \
  if (ntw <= NTW) {                                                                \
    if (g.MT == 1)                                                                 \
      return launch_coop(ln_bwd_kernel<G, NTW, SPLIT, 1, T>, grid, smem, &p, s);      \
    return launch_coop(ln_bwd_kernel<G, NTW, SPLIT, 4, T>, grid, smem, &p, s);        \
  }
  HB_BWD(1)
  HB_BWD(2)
  HB_BWD(4)
  HB_BWD(8)
  if constexpr (SPLIT == 1) { HB_BWD(16) }
#undef HB_BWD
  return HASTE_B200_ERR_UNSUPPORTED;
}

int run_ln_fwd_f32(LnFwdParams& p, const Geometry& g, cudaStream_t s);
int run_ln_fwd_bf16(LnFwdParams& p, const Geometry& g, cudaStream_t s);
int run_ln_bwd_f32(LnBwdParams& p, const Geometry& g, cudaStream_t s);
int run_ln_bwd_bf16(LnBwdParams& p, const Geometry& g, cudaStream_t s);
int run_lngru_fwd_f32(LnFwdParams& p, const Geometry& g, cudaStream_t s);
int run_lngru_fwd_bf16(LnFwdParams& p, const Geometry& g, cudaStream_t s);
int run_lngru_bwd_f32(LnBwdParams& p, const Geometry& g, cudaStream_t s);
int run_lngru_bwd_bf16(LnBwdParams& p, const Geometry& g, cudaStream_t s);

}  // namespace rec
}  // namespace hb
