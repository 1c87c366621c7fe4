// IndRNN and LayerNormIndRNN: h_t = tanh(Wx_t + u * h_{t-1} + b), with zoneout.
//
// The recurrence is elementwise, so one thread owns one (batch, unit) pair for
// all T steps and the kernels are pure HBM streams; loads that do not depend on
// the carried state are issued several steps ahead.  The parameter gradients
// du/db are per-thread sums reduced over the batch by a deterministic column sum.
// Math follows lib/indrnn_forward_gpu.cu.cc:25-63 and
// lib/indrnn_backward_gpu.cu.cc:25-74 (LayerNorm variant:
// lib/layer_norm_indrnn_{forward,backward}_gpu.cu.cc).
#include "cells.cuh"

namespace hb {
namespace {

constexpr int AHEAD = 8;  // independent loads in flight per thread

template <typename T, bool Training, bool Zoneout>
__global__ void indrnn_scan_fwd(int T_, long long NH, int H, const T* __restrict__ Wx,
                                const T* __restrict__ u, const T* __restrict__ b,
                                T* __restrict__ h, float zoneout_prob,
                                const T* __restrict__ mask) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= NH) return;
  const int j = (int)(idx % H);
  const float uj = ld(u + j), bj = ld(b + j);
  float hp = ld(h + idx);
  for (int t0 = 0; t0 < T_; t0 += AHEAD) {
    float wx[AHEAD], m[AHEAD];
#pragma unroll
    for (int k = 0; k < AHEAD; ++k) {
      const int t = t0 + k;
      wx[k] = (t < T_) ? ld(Wx + t * NH + idx) : 0.f;
      m[k] = (Zoneout && Training && t < T_) ? ld(mask + t * NH + idx) : 0.f;
    }
#pragma unroll
    for (int k = 0; k < AHEAD; ++k) {
      const int t = t0 + k;
      if (t < T_) {
        float hn = tanhf(wx[k] + uj * hp + bj);
        if (Zoneout) hn = zoneout<Training>(hn, hp, zoneout_prob, m[k]);
        st(h + (t + 1) * NH + idx, hn);
        hp = hn;  // the carried state stays fp32 whatever the storage type
      }
    }
  }
}

// Planes: dk is also written as two bf16 planes (hi, lo; `dk_planes`, the lo plane
// `plane_stride` elements later) - the form the two contractions that read it take their
// fp32 operands in, so that neither splits it again.
template <typename T, bool Zoneout, bool Planes>
__global__ void indrnn_scan_bwd(int T_, long long NH, int H, const T* __restrict__ u,
                                const T* __restrict__ h, const T* __restrict__ dh_new,
                                float* __restrict__ du_part, float* __restrict__ db_part,
                                float* __restrict__ dh_carry, T* __restrict__ dk_out,
                                const T* __restrict__ mask,
                                __nv_bfloat16* __restrict__ dk_planes, long long plane_stride) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= NH) return;
  const int j = (int)(idx % H);
  const float uj = ld(u + j);
  float carry = dh_carry[idx];
  float du = 0.f, db = 0.f;
  for (int t0 = T_ - 1; t0 >= 0; t0 -= AHEAD) {
    float hn[AHEAD], hpv[AHEAD], dn[AHEAD], m[AHEAD];
#pragma unroll
    for (int k = 0; k < AHEAD; ++k) {
      const int t = t0 - k;
      const bool ok = t >= 0;
      hn[k] = ok ? ld(h + (t + 1) * NH + idx) : 0.f;
      hpv[k] = ok ? ld(h + t * NH + idx) : 0.f;
      dn[k] = ok ? ld(dh_new + (t + 1) * NH + idx) : 0.f;
      m[k] = (Zoneout && ok) ? ld(mask + t * NH + idx) : 0.f;
    }
#pragma unroll
    for (int k = 0; k < AHEAD; ++k) {
      const int t = t0 - k;
      if (t >= 0) {
        float dh_total = dn[k] + carry;
        float keep = 0.f;
        if (Zoneout) {
          keep = (1.0f - m[k]) * dh_total;
          dh_total = m[k] * dh_total;
        }
        const float dk = d_tanh(hn[k]) * dh_total;
        st(dk_out + t * NH + idx, dk);
        if (Planes) {
          const __nv_bfloat16 hi = __float2bfloat16_rn(dk);
          dk_planes[t * NH + idx] = hi;
          dk_planes[plane_stride + t * NH + idx] = __float2bfloat16_rn(dk - __bfloat162float(hi));
        }
        carry = keep + uj * dk;
        du += hpv[k] * dk;
        db += dk;
      }
    }
  }
  dh_carry[idx] = carry;
  du_part[idx] = du;
  db_part[idx] = db;
}

template <typename T>
int scan_fwd(const IndrnnFwd& a, const void* Wx, cudaStream_t s) {
  const long long NH = (long long)a.N * a.H;
  const T* mask = (const T*)a.zoneout_mask;
  const bool zo = a.zoneout_prob != 0.0f && mask != nullptr;
  const int blocks = ceil_div(NH, 128);
#define HB_ARGS a.T, NH, a.H, (const T*)Wx, (const T*)a.u, (const T*)a.b, (T*)a.h, \
                a.zoneout_prob, zo ? mask : nullptr
  if (a.training) {
    if (zo) indrnn_scan_fwd<T, true, true><<<blocks, 128, 0, s>>>(HB_ARGS);
    else    indrnn_scan_fwd<T, true, false><<<blocks, 128, 0, s>>>(HB_ARGS);
  } else {
    if (zo) indrnn_scan_fwd<T, false, true><<<blocks, 128, 0, s>>>(HB_ARGS);
    else    indrnn_scan_fwd<T, false, false><<<blocks, 128, 0, s>>>(HB_ARGS);
  }
#undef HB_ARGS
  HB_LAUNCH_OK();
  count_launch(1);
  return HASTE_B200_OK;
}

template <typename T>
int scan_bwd(const IndrnnBwd& a, float* du_part, float* db_part, float* dh_carry,
             __nv_bfloat16* planes, long long plane_stride, cudaStream_t s) {
  const long long NH = (long long)a.N * a.H;
  const int blocks = ceil_div(NH, 128);
#define HB_ARGS a.T, NH, a.H, (const T*)a.u, (const T*)a.h, (const T*)a.dh_new, du_part, db_part, \
                dh_carry, (T*)a.workspace, (const T*)a.zoneout_mask, planes, plane_stride
  if (planes) {
    if (a.zoneout_mask) indrnn_scan_bwd<T, true, true><<<blocks, 128, 0, s>>>(HB_ARGS);
    else                indrnn_scan_bwd<T, false, true><<<blocks, 128, 0, s>>>(HB_ARGS);
  } else {
    if (a.zoneout_mask) indrnn_scan_bwd<T, true, false><<<blocks, 128, 0, s>>>(HB_ARGS);
    else                indrnn_scan_bwd<T, false, false><<<blocks, 128, 0, s>>>(HB_ARGS);
  }
#undef HB_ARGS
  HB_LAUNCH_OK();
  count_launch(1);
  return HASTE_B200_OK;
}

}  // namespace

int indrnn_forward(const IndrnnFwd& a, cudaStream_t s) {
  HB_REQUIRE(a.dtype == HASTE_B200_F32 || a.dtype == HASTE_B200_BF16, "dtype");
  HB_REQUIRE(a.T >= 0 && a.N > 0 && a.C > 0 && a.H > 0, "T,N,C,H");
  HB_REQUIRE(a.W && a.u && a.b && a.h && a.workspace, "null pointer");
  HB_REQUIRE(!a.gamma || (a.act_Wx && a.cache_Wx), "act_Wx/cache_Wx required with gamma");
  if (a.T == 0) return HASTE_B200_OK;
  HB_REQUIRE(a.x, "x is null");
  const long long TN = (long long)a.T * a.N;
  HB_REQUIRE(TN < (1LL << 31), "T*N too large");
  void* proj = a.gamma ? a.act_Wx : a.workspace;
  GemmDesc g{a.dtype, a.dtype, (int)TN, a.H, a.C, a.x, a.C, 1, a.W, a.H, 1, proj, a.H, 0};
  // The projection feeds a recurrence whose gain u * (1 - h^2) is close to one for u near 1:
  // an error of x.W is carried along the whole sequence and on through the layers of a stack
  // (measured: two-plane products leave 1.6e-4 on the output of six layers, three planes
  // 1.5e-5), so the forward projection always uses the fp32-accurate product.
  g.precise = 1;
  {
    ProfScope p(PH_PROJ, s);
    HB_TRY(gemm(g, s));
  }
  if (a.gamma) {
    ProfScope p(PH_OTHER, s);
    HB_TRY(layer_norm_forward(a.dtype, (int)TN, a.H, a.gamma, nullptr, a.act_Wx, a.workspace,
                              a.cache_Wx, s));
  }
  ProfScope p(PH_REC_FWD, s);
  if (a.dtype == HASTE_B200_F32) return scan_fwd<float>(a, a.workspace, s);
  return scan_fwd<__nv_bfloat16>(a, a.workspace, s);
}

int indrnn_backward(const IndrnnBwd& a, cudaStream_t s) {
  HB_REQUIRE(a.dtype == HASTE_B200_F32 || a.dtype == HASTE_B200_BF16, "dtype");
  HB_REQUIRE(a.T >= 0 && a.N > 0 && a.C > 0 && a.H > 0, "T,N,C,H");
  HB_REQUIRE(a.W && a.u && a.h && a.dh_new && a.dW && a.du && a.db && a.dh && a.workspace,
             "null pointer");
  HB_REQUIRE(!a.gamma || (a.dgamma && a.act_Wx && a.cache_Wx), "LayerNorm buffers");
  const int N = a.N, H = a.H, C = a.C;
  const long long TN = (long long)a.T * N;
  HB_REQUIRE(TN < (1LL << 31), "T*N too large");
  if (a.T == 0) return HASTE_B200_OK;
  HB_REQUIRE(a.x && a.dx, "x/dx is null");
  const size_t NH = (size_t)N * H;
  const size_t csf = colsum_scratch_floats(N, H);
  const size_t lnf = a.gamma ? layer_norm_backward_scratch_floats((int)TN, H) : 0;
  Arena ws;
  HB_TRY(make_arena(&ws, s, 3 * Arena::pad(NH * 4) + Arena::pad(csf * 4) + Arena::pad(lnf * 4) + 1024));
  float* dh_carry = ws.take<float>(NH);
  float* du_part = ws.take<float>(NH);
  float* db_part = ws.take<float>(NH);
  float* cs = ws.take<float>(csf);
  float* lns = ws.take<float>(lnf);
  HB_REQUIRE(dh_carry && du_part && db_part && cs && (lns || !lnf), "scratch arena");
  HB_TRY(to_float(a.dtype, a.dh, dh_carry, NH, s));
  // fp32: dk = d/d(x.W) is read by both contractions below as two bf16 planes.  Without
  // LayerNorm the scan writes them next to the fp32 values; with LayerNorm its backward pass
  // does.  (Grow-only library scratch; without it the contractions split for themselves.)
  __nv_bfloat16* planes = nullptr;
  long long plane_stride = 0;
  if (a.dtype == HASTE_B200_F32 && (H % 8) == 0) {
    const size_t pe = Arena::pad((size_t)TN * H * 2) / 2;  // elements per plane
    planes = static_cast<__nv_bfloat16*>(workspace(s, 2 * pe * 2 + 256, /*slot=*/3));
    plane_stride = (long long)pe;
  }
  {
    ProfScope p(PH_REC_BWD, s);
    __nv_bfloat16* sp = a.gamma ? nullptr : planes;
    if (a.dtype == HASTE_B200_F32) HB_TRY(scan_bwd<float>(a, du_part, db_part, dh_carry, sp, plane_stride, s));
    else HB_TRY(scan_bwd<__nv_bfloat16>(a, du_part, db_part, dh_carry, nullptr, 0, s));
  }
  HB_TRY(from_float(a.dtype, dh_carry, a.dh, NH, s));
  HB_TRY(colsum(HASTE_B200_F32, du_part, H, N, H, a.dtype, a.du, 1, cs, s));
  HB_TRY(colsum(HASTE_B200_F32, db_part, H, N, H, a.dtype, a.db, 1, cs, s));
  if (a.gamma) {
    ProfScope p(PH_OTHER, s);
    // workspace holds dk = d/d(LN(x.W)); turn it into d/d(x.W) in place.
    HB_TRY(layer_norm_backward(a.dtype, (int)TN, H, a.gamma, a.act_Wx, a.workspace, a.workspace,
                               a.dtype, a.dgamma, nullptr, a.cache_Wx, lns, s, planes,
                               plane_stride));
  }
  const bool tr = a.transposed_inputs != 0;
  // dW[C,H] = x^T . dk   (assigned, as in the reference)
  GemmDesc gw{a.dtype, a.dtype, C, H, (int)TN, a.x, tr ? TN : 1, tr ? 1 : C, a.workspace, H, 1,
              a.dW, H, 0};
  // the backward contractions feed no recurrence: the three-product form is enough also for
  // the LayerNorm variant (six products measured the same 2.6e-5 on a six-layer stack)
  if (planes) { gw.b_pl = planes; gw.b_pl_ld = H; gw.b_pl_stride = plane_stride; }
  {
    ProfScope p(PH_WGRAD, s);
    HB_TRY(gemm(gw, s));
  }
  GemmDesc gx{a.dtype, a.dtype, (int)TN, C, H, a.workspace, H, 1, a.W, tr ? C : 1, tr ? 1 : H,
              a.dx, C, 0};
  if (planes) { gx.a_pl = planes; gx.a_pl_ld = H; gx.a_pl_stride = plane_stride; }
  {
    ProfScope p(PH_DGRAD, s);
    HB_TRY(gemm(gx, s));
  }
  return HASTE_B200_OK;
}

}  // namespace hb
