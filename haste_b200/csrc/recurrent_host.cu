// Host side of the persistent recurrence kernels (recurrent_kernels.cuh): tiling choice,
// exchange-buffer scratch, and the four entry points the cell drivers call.
#include <cstdio>
#include <cstdlib>

#include "recurrent_ln_kernels.cuh"

namespace hb {
namespace rec {


namespace {

constexpr int MAX_MT = 4;

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

bool supported(int dtype, int N, int H, Geometry* g) {
  if (recurrence_path() == HASTE_B200_PATH_STEPWISE) return false;
  // R slice must fit the register file (two bf16 planes for fp32 and fp16 storage, one for bf16)
  if (dtype != HASTE_B200_BF16 && H > 512) return false;
  if (dtype == HASTE_B200_BF16 && H > 1024) return false;
  return pick_geometry(N, H, g);
}

// Timing-experiment builds only (-DHASTE_B200_TIMING_EXPERIMENTS): the environment variable
// HASTE_B200_TIMING_EXPERIMENT=<bits> switches parts of the persistent kernels off to attribute
// step time to them; results of such a run are wrong by construction and the library says so
// on stderr.  The shipped library reads no environment variable and compiles the switches out.
int debug_skip() {
#ifdef HASTE_B200_TIMING_EXPERIMENTS
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("HASTE_B200_TIMING_EXPERIMENT");
    v = e ? atoi(e) : 0;
    if (v != 0)
      fprintf(stderr, "haste_b200: HASTE_B200_TIMING_EXPERIMENT=%d - parts of the recurrence "
                      "kernels are switched off, results are wrong\n", v);
  }
  return v;
#else
  return 0;
#endif
}

// Zeroed scratch: abort flag followed by `words` exchange words.
int make_scratch(size_t words, Sync* sync, uint32_t** xwords, cudaStream_t s) {
  Arena ws;
  const size_t bytes = Arena::pad(4096) + Arena::pad(words * 4);
  HB_TRY(make_arena(&ws, s, bytes + 512, /*slot=*/2));
  int* flag = ws.take<int>(1024);
  uint32_t* x = ws.take<uint32_t>(words);
  HB_REQUIRE(flag && x, "scratch arena");
  HB_CUDA_OK(cudaMemsetAsync(flag, 0, bytes, s));
  sync->abort_flag = flag;
  sync->err = device_error_word();
  HB_REQUIRE(sync->err, "error word");
  *xwords = x;
  return HASTE_B200_OK;
}

}  // namespace
}  // namespace rec

// ---- exchange-only probe ---------------------------------------------------------------
// The hand-off of the forward recurrence with everything else taken out: per step every CTA
// publishes its 16 x 16 tagged words and every warp waits for its K range of all rows, then
// the CTA meets at its barrier.  No contraction, no gate math, no activation traffic.  Its
// time per step is the part of a recurrence step that no amount of arithmetic tuning removes
// (store -> L2 -> polling load, plus the CTA barrier); benchmarks quote it beside the measured
// step time.  No reference counterpart.
namespace rec {
namespace {

template <int KSW>
__global__ void __launch_bounds__(THREADS, 1)
exchange_probe_kernel(int T, int N, int Hx, int nHS, uint32_t* xbuf, Sync sync) {
  constexpr int KW = KSW * 16, CPR = KW / 4, CPL = 16 * CPR / 32;
  __shared__ int s_abort;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int hs = blockIdx.x % nHS, bs = blockIdx.x / nHS;
  const int nl = tid >> 4, ul = tid & 15;
  const int u0 = hs * U, n0 = bs * 16;
  if (tid == 0) s_abort = 0;
  __syncthreads();
  float carry = 0.f;
  for (int t = 0; t < T; ++t) {
    const uint32_t tag = (((uint32_t)t >> 1) & 1u) ^ 1u;
    const int n = n0 + nl;
    if (n < N && u0 + ul < Hx)
      publish_u32(xbuf + (size_t)(t & 1) * N * Hx + (size_t)n * Hx + u0 + ul,
                  xword_encode(carry * 0.5f + 0.25f, tag));
    const uint32_t wtag = tag << 30;
    const uint32_t* xsrc = xbuf + (size_t)(t & 1) * N * Hx;
    uint4 w[CPL];
    const long long t0 = clock64();
    unsigned int spins = 0;
    bool alive = true;
    for (;;) {
#pragma unroll
      for (int i = 0; i < CPL; ++i) {
        const int e = lane + i * 32;
        const int r = e / CPR, k = warp * KW + (e % CPR) * 4;
        if (n0 + r < N && k < Hx) w[i] = ld_relaxed_u32x4(xsrc + (size_t)(n0 + r) * Hx + k);
        else w[i] = make_uint4(wtag, wtag, wtag, wtag);
      }
      uint32_t bad = 0;
#pragma unroll
      for (int i = 0; i < CPL; ++i)
        bad |= (w[i].x ^ wtag) | (w[i].y ^ wtag) | (w[i].z ^ wtag) | (w[i].w ^ wtag);
      if (__all_sync(0xffffffffu, (bad & 0x40000000u) == 0)) break;
      if ((++spins & 63u) == 0) {
        bool stop = *reinterpret_cast<volatile int*>(sync.abort_flag) != 0;
        if (!stop && clock64() - t0 > SPIN_LIMIT_CYCLES) {
          raise_abort(sync, &s_abort, 46, blockIdx.x, t);
          stop = true;
        }
        if (__any_sync(0xffffffffu, stop)) { alive = false; break; }
      }
    }
    if (!alive) *reinterpret_cast<volatile int*>(&s_abort) = 1;
    carry = xword_value(w[0].x);  // the next word depends on a received one, as h does
    if (__syncthreads_or(*reinterpret_cast<volatile int*>(&s_abort))) break;
  }
}

}  // namespace
}  // namespace rec

// Runs the probe for `steps` steps with the tiling the recurrence would use for (N, H) and
// returns the device time per step in microseconds.
int exchange_probe(int N, int H, int steps, float* us_per_step, cudaStream_t s) {
  using namespace rec;
  HB_REQUIRE(N > 0 && H > 0 && steps > 0 && us_per_step, "arguments");
  const int nHS = ceil_div(H, U), nBS = ceil_div(N, 16);
  HB_REQUIRE((long long)nHS * nBS <= sm_count(), "does not fit one CTA per SM");
  const int Hx = nHS * U;
  const int ksw = ceil_div(nHS, WARPS);
  HB_REQUIRE(ksw <= 8, "H too large for the probe");
  Sync sync;
  uint32_t* xbuf = nullptr;
  HB_TRY(make_scratch((size_t)2 * N * Hx, &sync, &xbuf, s));
  cudaEvent_t e0, e1;
  HB_CUDA_OK(cudaEventCreate(&e0));
  HB_CUDA_OK(cudaEventCreate(&e1));
  int T = steps, Nn = N, Hxx = Hx, nhs = nHS;
  void* args[] = {&T, &Nn, &Hxx, &nhs, &xbuf, &sync};
  const void* fn = ksw <= 1   ? (const void*)exchange_probe_kernel<1>
                   : ksw <= 2 ? (const void*)exchange_probe_kernel<2>
                   : ksw <= 4 ? (const void*)exchange_probe_kernel<4>
                              : (const void*)exchange_probe_kernel<8>;
  HB_CUDA_OK(cudaEventRecord(e0, s));
  cudaError_t e = cudaLaunchCooperativeKernel(fn, dim3(nHS * nBS), dim3(THREADS), args, 0, s);
  if (e != cudaSuccess) {
    set_last_error("cooperative launch failed: %s", cudaGetErrorString(e));
    cudaGetLastError();
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    return HASTE_B200_ERR_CUDA;
  }
  count_launch(1);
  HB_CUDA_OK(cudaEventRecord(e1, s));
  HB_CUDA_OK(cudaEventSynchronize(e1));
  float ms = 0.f;
  HB_CUDA_OK(cudaEventElapsedTime(&ms, e0, e1));
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  *us_per_step = ms * 1e3f / steps;
  return HASTE_B200_OK;
}

using namespace rec;

int lstm_forward_persistent(const LstmFwd& a, cudaStream_t s) {
  Geometry g;
  if (!supported(a.dtype, a.N, a.H, &g)) return HASTE_B200_ERR_UNSUPPORTED;
  const int Hx = (a.H + 3) & ~3;
  Sync sync;
  uint32_t* xbuf = nullptr;
  HB_TRY(make_scratch((size_t)2 * a.N * Hx, &sync, &xbuf, s));
  const bool zo = a.zoneout_prob != 0.0f && a.zoneout_mask != nullptr;
  FwdParams p{a.T, a.N, a.H, Hx, g.nHS, g.MT, a.training, zo ? 1 : 0, a.zoneout_prob, a.R, a.b,
              nullptr, a.v, a.h, a.c, a.v, a.zoneout_mask, xbuf, sync, debug_skip()};
  return a.dtype == HASTE_B200_F32 ? run_fwd_lstm_f32(p, g, s) : run_fwd_lstm_bf16(p, g, s);
}

int gru_forward_persistent(const GruFwd& a, cudaStream_t s) {
  Geometry g;
  if (!supported(a.dtype, a.N, a.H, &g)) return HASTE_B200_ERR_UNSUPPORTED;
  const int Hx = (a.H + 3) & ~3;
  Sync sync;
  uint32_t* xbuf = nullptr;
  HB_TRY(make_scratch((size_t)2 * a.N * Hx, &sync, &xbuf, s));
  const bool zo = a.zoneout_prob != 0.0f && a.zoneout_mask != nullptr;
  FwdParams p{a.T, a.N, a.H, Hx, g.nHS, g.MT, a.training, zo ? 1 : 0, a.zoneout_prob, a.R, a.bx,
              a.br, a.tmp_Wx, a.h, nullptr, a.v, a.zoneout_mask, xbuf, sync, debug_skip()};
  if (a.dtype == HASTE_B200_F16) return run_fwd_gru_f16(p, g, s);
  return a.dtype == HASTE_B200_F32 ? run_fwd_gru_f32(p, g, s) : run_fwd_gru_bf16(p, g, s);
}

// The persistent backward kernels leave the recurrent contribution of the very last
// processed step (t = 0) out of dh (nothing inside the kernel consumes it); it is added
// here with one small contraction: dh += dG_0 . R^T.
int lstm_backward_persistent(const LstmBwd& a, float* dh_carry, float* dc_carry,
                             const GradPlanes& planes, cudaStream_t s) {
  Geometry g;
  if (!supported(a.dtype, a.N, a.H, &g)) return HASTE_B200_ERR_UNSUPPORTED;
  Sync sync;
  uint32_t* exch = nullptr;
  const int H = a.H;
  const size_t ewords = ((size_t)2 * g.nBS * g.nHS * g.nHS * g.MT * 16 * U + 63) & ~size_t(63);
  const int prow = g.nBS * 16;
  const size_t pwords = (size_t)prow * 4 * H;
  HB_TRY(make_scratch(ewords + pwords + colsum_scratch_floats(prow, 4 * H) + 64, &sync, &exch, s));
  float* part = reinterpret_cast<float*>(exch + ewords);
  BwdParams p{a.T, a.N, a.H, g.nHS, g.MT, a.zoneout_mask ? 1 : 0, a.transposed_inputs, a.R, a.h,
              a.c, a.v, a.dh_new, a.dc_new, nullptr, nullptr, a.zoneout_mask, dh_carry, dc_carry,
              exch, sync, debug_skip(), planes.p, planes.p2, planes.stride, part};
  int st_ = a.dtype == HASTE_B200_F32 ? run_bwd_lstm_f32(p, g, s) : run_bwd_lstm_bf16(p, g, s);
  if (st_ != HASTE_B200_OK) return st_;
  // db += column sums of the kernel's per-row-group partials
  HB_TRY(colsum(HASTE_B200_F32, part, 4LL * H, prow, 4 * H, a.dtype, a.db, 1, part + pwords, s));
  GemmDesc gd{a.dtype, HASTE_B200_F32, a.N, H, 4 * H, a.v, 4LL * H, 1, a.R,
              a.transposed_inputs ? H : 1, a.transposed_inputs ? 1 : 4LL * H, dh_carry, H, 1};
  return gemm_small(gd, s);
}

int gru_backward_persistent(const GruBwd& a, float* dh_carry, const GradPlanes& planes,
                            cudaStream_t s) {
  Geometry g;
  if (!supported(a.dtype, a.N, a.H, &g)) return HASTE_B200_ERR_UNSUPPORTED;
  Sync sync;
  uint32_t* exch = nullptr;
  const int H = a.H;
  const size_t ewords = ((size_t)2 * g.nBS * g.nHS * g.nHS * g.MT * 16 * U + 63) & ~size_t(63);
  const int prow = g.nBS * 16;
  const size_t pwords = (size_t)prow * 4 * H;
  HB_TRY(make_scratch(ewords + pwords + colsum_scratch_floats(prow, 3 * H) + 64, &sync, &exch, s));
  float* part = reinterpret_cast<float*>(exch + ewords);
  BwdParams p{a.T, a.N, a.H, g.nHS, g.MT, a.zoneout_mask ? 1 : 0, a.transposed_inputs, a.R, a.h,
              nullptr, const_cast<void*>(a.v), a.dh_new, nullptr, a.dp, a.dq, a.zoneout_mask,
              dh_carry, nullptr, exch, sync, debug_skip(), planes.p, planes.p2, planes.stride, part};
  int st_ = a.dtype == HASTE_B200_F16   ? run_bwd_gru_f16(p, g, s)
            : a.dtype == HASTE_B200_F32 ? run_bwd_gru_f32(p, g, s)
                                        : run_bwd_gru_bf16(p, g, s);
  if (st_ != HASTE_B200_OK) return st_;
  {
    // partial columns: dp_z, dp_r, dp_g, dq_g.  dbx += sums of (dp_z, dp_r, dp_g);
    // dbr += sums of (dp_z, dp_r, dq_g)
    float* cs = part + pwords;
    const size_t es = dtype_size(a.dtype);
    char* dbr = static_cast<char*>(a.dbr);
    HB_TRY(colsum(HASTE_B200_F32, part, 4LL * H, prow, 3 * H, a.dtype, a.dbx, 1, cs, s));
    HB_TRY(colsum(HASTE_B200_F32, part, 4LL * H, prow, 2 * H, a.dtype, dbr, 1, cs, s));
    HB_TRY(colsum(HASTE_B200_F32, part + 3 * H, 4LL * H, prow, H, a.dtype, dbr + (size_t)2 * H * es,
                  1, cs, s));
  }
  GemmDesc gd{a.dtype, HASTE_B200_F32, a.N, H, 3 * H, a.dq, 3LL * H, 1, a.R,
              a.transposed_inputs ? H : 1, a.transposed_inputs ? 1 : 3LL * H, dh_carry, H, 1};
  return gemm_small(gd, s);
}

// ---- LayerNormLSTM (recurrent_ln_kernels.cuh) ------------------------------------------
// Forward: LN(x.W) is already in a.act_Wx_norm.  Four source slices per thread in the
// statistic exchange limit the kernels to 64 hidden slices, which `supported` guarantees.
int layer_norm_lstm_forward_persistent(const LnLstmFwd& a, cudaStream_t s) {
  Geometry g;
  if (!supported(a.dtype, a.N, a.H, &g) || g.nHS > 64) return HASTE_B200_ERR_UNSUPPORTED;
  const int Hx = (a.H + 3) & ~3;
  const size_t xwords = (size_t)2 * a.N * Hx;
  const size_t swords = (size_t)2 * 2 * g.nBS * g.MT * 16 * g.nHS * 2;
  Sync sync;
  uint32_t* words = nullptr;
  HB_TRY(make_scratch(xwords + swords + 64, &sync, &words, s));
  const bool zo = a.zoneout_prob != 0.0f && a.zoneout_mask != nullptr;
  LnFwdParams p{a.T, a.N, a.H, Hx, g.nHS, g.MT, a.training, zo ? 1 : 0, a.zoneout_prob, a.R, a.b,
                nullptr, a.act_Wx_norm, a.gamma_Rh, a.gamma_h, a.beta_h, a.act_Wx_norm, a.act_Rh, a.cache_Rh,
                a.act_c_norm, a.cache_c, a.h, a.c, a.zoneout_mask, words,
                words + ((xwords + 63) & ~size_t(63)), sync, debug_skip()};
  return a.dtype == HASTE_B200_F32 ? run_ln_fwd_f32(p, g, s) : run_ln_fwd_bf16(p, g, s);
}

// Backward.  `acc` holds fp32 accumulators [dgamma_Rh 4H | dgamma_h H | dbeta_h H] that the
// per-row-group partial sums of the kernel are added into (fixed order).  As for the plain
// LSTM, the recurrent contribution of step 0 to dh is added here by one small contraction.
int layer_norm_lstm_backward_persistent(const LnLstmBwd& a, float* dh_carry, float* dc_carry,
                                        float* acc, const GradPlanes& planes, cudaStream_t s) {
  Geometry g;
  if (!supported(a.dtype, a.N, a.H, &g) || g.nHS > 64) return HASTE_B200_ERR_UNSUPPORTED;
  const int H = a.H;
  const size_t ewords = ((size_t)2 * g.nBS * g.nHS * g.nHS * g.MT * 16 * U + 63) & ~size_t(63);
  const size_t swords = ((size_t)2 * 2 * g.nBS * g.MT * 16 * g.nHS * 2 + 63) & ~size_t(63);
  const int prow = g.nBS * 16;
  const size_t pwords = (size_t)prow * 6 * H;
  const size_t cwords = colsum_scratch_floats(prow, 4 * H);
  Sync sync;
  uint32_t* words = nullptr;
  HB_TRY(make_scratch(ewords + swords + pwords + cwords + 64, &sync, &words, s));
  float* part = reinterpret_cast<float*>(words + ewords + swords);
  float* cs = part + pwords;
  LnBwdParams p{a.T, a.N, H, g.nHS, g.MT, a.zoneout_mask ? 1 : 0, a.transposed_inputs, a.R,
                a.gamma_Rh, a.gamma_h, a.c, nullptr, nullptr, nullptr, a.act_Wx_norm, a.act_Rh,
                a.cache_Rh, a.act_c_norm,
                a.cache_c, a.dh_new, a.dc_new, a.zoneout_mask, dh_carry, dc_carry, part,
                part + (size_t)prow * 4 * H, part + (size_t)prow * 5 * H, words, words + ewords,
                sync, planes.p, planes.p2, planes.stride, debug_skip()};
  int st_ = a.dtype == HASTE_B200_F32 ? run_ln_bwd_f32(p, g, s) : run_ln_bwd_bf16(p, g, s);
  if (st_ != HASTE_B200_OK) return st_;
  HB_TRY(colsum(HASTE_B200_F32, part, 4LL * H, prow, 4 * H, HASTE_B200_F32, acc, 1, cs, s));
  HB_TRY(colsum(HASTE_B200_F32, part + (size_t)prow * 4 * H, H, prow, H, HASTE_B200_F32,
                acc + 4 * H, 1, cs, s));
  HB_TRY(colsum(HASTE_B200_F32, part + (size_t)prow * 5 * H, H, prow, H, HASTE_B200_F32,
                acc + 5 * H, 1, cs, s));
  GemmDesc gd{a.dtype, HASTE_B200_F32, a.N, H, 4 * H, a.act_Rh, 4LL * H, 1, a.R,
              a.transposed_inputs ? H : 1, a.transposed_inputs ? 1 : 4LL * H, dh_carry, H, 1};
  gd.precise = 1;
  return gemm_small(gd, s);
}

// ---- LayerNormGRU (the G = 3 instantiation of the same kernels) ---------------------------
// Forward: LN(x.W) is already in a.tmp_Wx_norm.
int layer_norm_gru_forward_persistent(const LnGruFwd& a, cudaStream_t s) {
  Geometry g;
  if (!supported(a.dtype, a.N, a.H, &g) || g.nHS > 64) return HASTE_B200_ERR_UNSUPPORTED;
  const int Hx = (a.H + 3) & ~3;
  const size_t xwords = (size_t)2 * a.N * Hx;
  const size_t swords = (size_t)2 * 2 * g.nBS * g.MT * 16 * g.nHS * 2;
  Sync sync;
  uint32_t* words = nullptr;
  HB_TRY(make_scratch(xwords + swords + 64, &sync, &words, s));
  const bool zo = a.zoneout_prob != 0.0f && a.zoneout_mask != nullptr;
  LnFwdParams p{a.T, a.N, a.H, Hx, g.nHS, g.MT, a.training, zo ? 1 : 0, a.zoneout_prob, a.R, a.bx,
                a.br, a.tmp_Wx_norm, a.gamma_Rh, nullptr, nullptr, a.v, a.act_Rh, a.cache_Rh,
                nullptr, nullptr, a.h, nullptr, a.zoneout_mask, words,
                words + ((xwords + 63) & ~size_t(63)), sync};
  return a.dtype == HASTE_B200_F32 ? run_lngru_fwd_f32(p, g, s) : run_lngru_fwd_bf16(p, g, s);
}

// Backward.  `acc` is the fp32 accumulator [3H] for dgamma_Rh.  a.act_Rh is overwritten with
// d(h.R); a.dp / a.dq receive the gradients w.r.t. the normalised projections (+ biases).
int layer_norm_gru_backward_persistent(const LnGruBwd& a, float* dh_carry, float* acc,
                                       const GradPlanes& planes, cudaStream_t s) {
  Geometry g;
  if (!supported(a.dtype, a.N, a.H, &g) || g.nHS > 64) return HASTE_B200_ERR_UNSUPPORTED;
  const int H = a.H;
  const size_t ewords = ((size_t)2 * g.nBS * g.nHS * g.nHS * g.MT * 16 * U + 63) & ~size_t(63);
  const size_t swords = ((size_t)2 * 2 * g.nBS * g.MT * 16 * g.nHS * 2 + 63) & ~size_t(63);
  const int prow = g.nBS * 16;
  const size_t pwords = (size_t)prow * 3 * H;
  const size_t cwords = colsum_scratch_floats(prow, 3 * H);
  Sync sync;
  uint32_t* words = nullptr;
  HB_TRY(make_scratch(ewords + swords + pwords + cwords + 64, &sync, &words, s));
  float* part = reinterpret_cast<float*>(words + ewords + swords);
  float* cs = part + pwords;
  LnBwdParams p{a.T, a.N, H, g.nHS, g.MT, a.zoneout_mask ? 1 : 0, a.transposed_inputs, a.R,
                a.gamma_Rh, nullptr, nullptr, a.h, a.dp, a.dq, const_cast<void*>(a.v), a.act_Rh,
                a.cache_Rh, nullptr, nullptr, a.dh_new, nullptr, a.zoneout_mask, dh_carry, nullptr,
                part, nullptr, nullptr, words, words + ewords, sync, planes.p, planes.p2,
                planes.stride};
  int st_ = a.dtype == HASTE_B200_F32 ? run_lngru_bwd_f32(p, g, s) : run_lngru_bwd_bf16(p, g, s);
  if (st_ != HASTE_B200_OK) return st_;
  HB_TRY(colsum(HASTE_B200_F32, part, 3LL * H, prow, 3 * H, HASTE_B200_F32, acc, 1, cs, s));
  GemmDesc gd{a.dtype, HASTE_B200_F32, a.N, H, 3 * H, a.act_Rh, 3LL * H, 1, a.R,
              a.transposed_inputs ? H : 1, a.transposed_inputs ? 1 : 3LL * H, dh_carry, H, 1};
  gd.precise = 1;
  return gemm_small(gd, s);
}

}  // namespace hb
