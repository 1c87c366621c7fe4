// One time step of LSTM / GRU in ONE launch: x.W + h.R, biases, gate functions, state update
// and zoneout fused, for the reference's per-step Iterate API (lib/haste/lstm.h:73-86,
// lib/haste/gru.h:72-84; lib/lstm_forward_gpu.cu.cc:141-208, lib/gru_forward_gpu.cu.cc:160-212),
// which the reference runs as two cuBLAS calls and a pointwise kernel.
//
// Autoregressive use means a small batch and one step at a time, so the step is bound by
// launches and by reading W and R (which stay in L2 from call to call), not by arithmetic:
// the products run on the CUDA cores in fp32 (exact for fp32 storage, no operand planes to
// prepare per call).  A CTA owns four hidden units = 16 accumulator columns (the unit's four
// gate pre-activations; for the GRU: z, r, the x part of g and the h part of g, which the
// reset gate multiplies).  Its threads form K-groups; a group's threads hold 4 rows x 4 gates
// of one unit in registers and walk their share of K = C + H in 32-wide chunks staged through
// shared memory; the groups' partial sums meet in shared memory and the same launch applies
// the cell.
#include <algorithm>

#include "cells.cuh"

namespace hb {
namespace {

constexpr int IT_THREADS = 256;
constexpr int IT_UNITS = 4;      // hidden units per CTA
constexpr int IT_KC = 32;        // k per staged chunk
constexpr int IT_MAXN = 64;      // batch rows (the whole batch lives in one CTA's tiles)
constexpr int IT_MAXG = 8;       // K-groups per CTA

struct StepParams {
  int N, C, H;
  const void *W, *R, *b0, *b1, *x, *h_prev, *c_prev;
  void *h_out, *c_out, *v;
  float zoneout_prob;
  const void* mask;
};

// RT: row tiles of 4 rows (1, 2, 4, 8 or 16: the batch rounded up).  Threads per K-group = 4 * RT,
// groups = min(8, 256 / (4 * RT)).  Each round stages one 32-wide k-chunk per group; the next
// round's operands are fetched into registers before the current round's arithmetic, so the
// global-memory latency of a round is paid under the previous round's work.
template <typename T, bool GRU, bool Training, int RT>
__global__ void __launch_bounds__(IT_THREADS) step_fused_kernel(const StepParams p) {
  constexpr int ROWS = 4 * RT;                                       // padded batch rows
  constexpr int TPG = 4 * RT;                                        // threads per K-group
  constexpr int GROUPS = (IT_THREADS / TPG) < IT_MAXG ? (IT_THREADS / TPG) : IT_MAXG;
  constexpr int WARPS = IT_THREADS / 32;
  constexpr int A_PER_G = (ROWS + WARPS - 1) / WARPS;                // rows a warp stages per group
  constexpr int W_PER_T = GROUPS * IT_KC * 16 / IT_THREADS;          // weights a thread stages
  constexpr int A_STRIDE = IT_KC + 1;
  // staging: As[g][row][IT_KC + 1] and Ws[g][kk][unit][4 gates]; the A area is reused for the
  // groups' partial sums red[g][row][unit][4]
  extern __shared__ float smem[];
  float* As = smem;
  float* Ws = smem + GROUPS * ROWS * A_STRIDE;
  const int N = p.N, C = p.C, H = p.H;
  constexpr int G = GRU ? 3 : 4;  // gate blocks in a row of W / R
  const int j0 = blockIdx.x * IT_UNITS;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = tid / TPG, rt = (tid % TPG) >> 2, u = tid & 3;
  const bool active = g < GROUPS;
  const T* W = static_cast<const T*>(p.W);
  const T* R = static_cast<const T*>(p.R);
  const T* x = static_cast<const T*>(p.x);
  const T* hp = static_cast<const T*>(p.h_prev);

  float acc[4][4];
#pragma unroll
  for (int r = 0; r < 4; ++r)
#pragma unroll
    for (int q = 0; q < 4; ++q) acc[r][q] = 0.f;

  const int chunks_x = (C + IT_KC - 1) / IT_KC, chunks_h = (H + IT_KC - 1) / IT_KC;
  const int chunks = chunks_x + chunks_h;

  float areg[GROUPS][A_PER_G], wreg[W_PER_T];
  // fetch one round (chunks c0 .. c0 + GROUPS - 1) into registers; every load is issued before
  // any is used
  auto fetch = [&](int c0) {
#pragma unroll
    for (int gg = 0; gg < GROUPS; ++gg) {
      const int q = c0 + gg;
      const bool xp = q < chunks_x;
      const int k = (xp ? q : q - chunks_x) * IT_KC + lane;
      const bool k_ok = q < chunks && k < (xp ? C : H);
      const T* src = xp ? x + k : hp + k;
      const long long ld_src = xp ? C : H;
#pragma unroll
      for (int rr = 0; rr < A_PER_G; ++rr) {
        const int row = warp + rr * WARPS;
        areg[gg][rr] = (k_ok && row < N) ? ld(src + row * ld_src) : 0.f;
      }
    }
#pragma unroll
    for (int e = 0; e < W_PER_T; ++e) {
      const int i = tid + e * IT_THREADS;
      const int uu = i & 3, gate = (i >> 2) & 3, kk = (i >> 4) & (IT_KC - 1), gg = i >> 9;
      const int q = c0 + gg;
      const bool xp = q < chunks_x;
      const int k = (xp ? q : q - chunks_x) * IT_KC + kk;
      // column block of W / R this accumulator takes its weights from (-1: none)
      int blk = gate;
      if (GRU) blk = gate < 2 ? gate : (gate == 2 ? (xp ? 2 : -1) : (xp ? -1 : 2));
      const bool ok = q < chunks && j0 + uu < H && k < (xp ? C : H) && blk >= 0;
      wreg[e] = ok ? ld((xp ? W : R) + (long long)k * G * H + (long long)blk * H + j0 + uu) : 0.f;
    }
  };
  auto stage = [&]() {
#pragma unroll
    for (int gg = 0; gg < GROUPS; ++gg)
#pragma unroll
      for (int rr = 0; rr < A_PER_G; ++rr) {
        const int row = warp + rr * WARPS;
        if (row < ROWS) As[(gg * ROWS + row) * A_STRIDE + lane] = areg[gg][rr];
      }
#pragma unroll
    for (int e = 0; e < W_PER_T; ++e) {
      const int i = tid + e * IT_THREADS;
      const int uu = i & 3, gate = (i >> 2) & 3, kk = (i >> 4) & (IT_KC - 1), gg = i >> 9;
      Ws[((gg * IT_KC + kk) * IT_UNITS + uu) * 4 + gate] = wreg[e];
    }
  };

  fetch(0);
  for (int c0 = 0; c0 < chunks; c0 += GROUPS) {
    stage();
    __syncthreads();
    if (c0 + GROUPS < chunks) fetch(c0 + GROUPS);
    // ---- 4 rows x 4 gates of one unit per thread
    if (active && c0 + g < chunks) {
      const float* a0 = As + (g * ROWS + rt * 4) * A_STRIDE;
      const float* w0 = Ws + g * IT_KC * 16 + u * 4;
#pragma unroll 8
      for (int kk = 0; kk < IT_KC; ++kk) {
        const float4 w = *reinterpret_cast<const float4*>(w0 + kk * 16);
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const float a = a0[r * A_STRIDE + kk];
          acc[r][0] += a * w.x;
          acc[r][1] += a * w.y;
          acc[r][2] += a * w.z;
          acc[r][3] += a * w.w;
        }
      }
    }
    __syncthreads();
  }

  // ---- the groups' partial sums meet: red[g][row][unit][gate]
  float* red = smem;
  if (active) {
#pragma unroll
    for (int r = 0; r < 4; ++r)
      *reinterpret_cast<float4*>(red + ((g * ROWS + rt * 4 + r) * IT_UNITS + u) * 4) =
          make_float4(acc[r][0], acc[r][1], acc[r][2], acc[r][3]);
  }
  __syncthreads();

  // ---- the cell: one thread per (row, unit)
  const T* b0 = static_cast<const T*>(p.b0);
  const T* b1 = static_cast<const T*>(p.b1);
  const T* cp = static_cast<const T*>(p.c_prev);
  const T* mask = static_cast<const T*>(p.mask);
  T* h_out = static_cast<T*>(p.h_out);
  T* c_out = static_cast<T*>(p.c_out);
  T* v = static_cast<T*>(p.v);
  for (int i = tid; i < N * IT_UNITS; i += IT_THREADS) {
    const int n = i >> 2, uu = i & 3, j = j0 + uu;
    if (j >= H) continue;
    float s[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int gg = 0; gg < GROUPS; ++gg) {
      const float4 t = *reinterpret_cast<const float4*>(red + ((gg * ROWS + n) * IT_UNITS + uu) * 4);
      s[0] += t.x; s[1] += t.y; s[2] += t.z; s[3] += t.w;
    }
    const long long o0 = (long long)n * H + j;
    const float hprev = ld(hp + o0);
    float h_new;
    if (GRU) {
      const float z = sigmoidf_(s[0] + ld(b0 + j) + ld(b1 + j));
      const float r = sigmoidf_(s[1] + ld(b0 + j + H) + ld(b1 + j + H));
      const float q_g = s[3] + ld(b1 + j + 2 * H);
      const float gv = tanhf(s[2] + r * q_g + ld(b0 + j + 2 * H));
      if (Training && v) {
        const long long v0 = (long long)n * 4 * H + j;
        st(v + v0, z);
        st(v + v0 + H, r);
        st(v + v0 + 2 * H, gv);
        st(v + v0 + 3 * H, q_g);
      }
      h_new = z * hprev + (1.0f - z) * gv;
    } else {
      const float iv = sigmoidf_(s[0] + ld(b0 + j));
      const float gv = tanhf(s[1] + ld(b0 + j + H));
      const float fv = sigmoidf_(s[2] + ld(b0 + j + 2 * H));
      const float ov = sigmoidf_(s[3] + ld(b0 + j + 3 * H));
      if (Training && v) {
        const long long v0 = (long long)n * 4 * H + j;
        st(v + v0, iv);
        st(v + v0 + H, gv);
        st(v + v0 + 2 * H, fv);
        st(v + v0 + 3 * H, ov);
      }
      const float c_new = fv * ld(cp + o0) + iv * gv;
      st(c_out + o0, c_new);
      h_new = ov * tanhf(c_new);
    }
    if (mask)  // zoneout is on only with a probability and a mask (the host passes neither otherwise)
      h_new = zoneout<Training>(h_new, hprev, p.zoneout_prob, Training ? ld(mask + o0) : 0.f);
    st(h_out + o0, h_new);
  }
}

template <typename T, bool GRU, bool Training, int RT>
int launch_step_rt(const StepParams& p, cudaStream_t s) {
  constexpr int ROWS = 4 * RT, TPG = 4 * RT;
  constexpr int GROUPS = (IT_THREADS / TPG) < IT_MAXG ? (IT_THREADS / TPG) : IT_MAXG;
  constexpr size_t SMEM = (size_t)(GROUPS * ROWS * (IT_KC + 1) + GROUPS * IT_KC * 16) * sizeof(float);
  static_assert((GROUPS * ROWS * (IT_KC + 1)) % 4 == 0, "the weight area must stay 16-byte aligned");
  auto k = step_fused_kernel<T, GRU, Training, RT>;
  if (SMEM > 48 * 1024)
    HB_CUDA_OK(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM));
  k<<<ceil_div(p.H, IT_UNITS), IT_THREADS, SMEM, s>>>(p);
  HB_LAUNCH_OK();
  count_launch(1);
  return HASTE_B200_OK;
}

template <typename T, bool GRU, bool Training>
int launch_step_t(const StepParams& p, cudaStream_t s) {
  const int rt = (p.N + 3) / 4;
  if (rt <= 1) return launch_step_rt<T, GRU, Training, 1>(p, s);
  if (rt <= 2) return launch_step_rt<T, GRU, Training, 2>(p, s);
  if (rt <= 4) return launch_step_rt<T, GRU, Training, 4>(p, s);
  if (rt <= 8) return launch_step_rt<T, GRU, Training, 8>(p, s);
  return launch_step_rt<T, GRU, Training, 16>(p, s);
}

template <bool GRU>
int launch_step(int dtype, bool training, StepParams& p, cudaStream_t s) {
  if (p.N > IT_MAXN || p.N < 1 || p.H < 1 || p.C < 1) return HASTE_B200_ERR_UNSUPPORTED;
  // Measured per call (fp32, fused / general path): 1 row, H=512: 10 / 79 us; 16 rows: 12 / 81;
  // 64 rows: 23 / 45; 1 row, H=1024: 23 / 151; 64 rows, H=1024: 64 / 53.  Beyond the work of
  // the 64-row H=512 step the tensor-core contractions of the general path win.
  if ((long long)p.N * (p.C + p.H) * p.H > 64LL * 1024 * 512) return HASTE_B200_ERR_UNSUPPORTED;
  if (dtype == HASTE_B200_F32)
    return training ? launch_step_t<float, GRU, true>(p, s) : launch_step_t<float, GRU, false>(p, s);
  if (dtype == HASTE_B200_BF16)
    return training ? launch_step_t<__nv_bfloat16, GRU, true>(p, s)
                    : launch_step_t<__nv_bfloat16, GRU, false>(p, s);
  return HASTE_B200_ERR_UNSUPPORTED;
}

}  // namespace

// The single-step (Iterate) forward of the LSTM in one launch.  HASTE_B200_ERR_UNSUPPORTED
// (more than 64 rows, other storage types) sends the caller to the general path.
int lstm_forward_step_fused(const LstmFwd& a, cudaStream_t s) {
  // (a new state written over the old one would race with the CTAs still reading it)
  if (a.T != 1 || !a.h_out || !a.c_out || a.h_out == a.h) return HASTE_B200_ERR_UNSUPPORTED;
  StepParams p{};
  p.N = a.N; p.C = a.C; p.H = a.H;
  p.W = a.W; p.R = a.R; p.b0 = a.b; p.b1 = nullptr; p.x = a.x; p.h_prev = a.h; p.c_prev = a.c;
  p.h_out = a.h_out; p.c_out = a.c_out; p.v = a.v;
  const bool zo = a.zoneout_prob != 0.0f && a.zoneout_mask != nullptr;
  p.zoneout_prob = zo ? a.zoneout_prob : 0.0f;
  p.mask = zo ? a.zoneout_mask : nullptr;
  return launch_step<false>(a.dtype, a.training != 0, p, s);
}

int gru_forward_step_fused(const GruFwd& a, cudaStream_t s) {
  if (a.T != 1 || !a.h_out || a.h_out == a.h) return HASTE_B200_ERR_UNSUPPORTED;
  StepParams p{};
  p.N = a.N; p.C = a.C; p.H = a.H;
  p.W = a.W; p.R = a.R; p.b0 = a.bx; p.b1 = a.br; p.x = a.x; p.h_prev = a.h; p.c_prev = nullptr;
  p.h_out = a.h_out; p.c_out = nullptr; p.v = a.v;
  const bool zo = a.zoneout_prob != 0.0f && a.zoneout_mask != nullptr;
  p.zoneout_prob = zo ? a.zoneout_prob : 0.0f;
  p.mask = zo ? a.zoneout_mask : nullptr;
  return launch_step<true>(a.dtype, a.training != 0, p, s);
}

}  // namespace hb
