// Tensor-core GRU recurrence for large batches (bf16 storage), sm_100a.
//
// The register-resident kernels of recurrent_kernels.cuh are built for small batches: a CTA
// multiplies 16..64 batch rows with mma.sync and every row of h reaches it as tagged words.
// From about a hundred rows per GPU the step product is a real tile for the 5th-generation
// tensor cores, and this file runs it there:
//
//   forward   gates[rows, 3*16] = h_{t-1}[rows, 0:H] . R[0:H, slice]            K = H
//   backward  dh_rec[rows, 16]  = dq_{t+1}[rows, 0:3H] . R[slice, 0:3H]^T       K = 3H
//
// * Grid = (H / 16 hidden slices) x (row groups), one cooperative launch per layer pass; a
//   CTA owns 16 hidden units for MT tiles of RB (64 or 128) batch rows.
// * The CTA's slice of R lives in SHARED MEMORY for the whole pass, written once in the
//   128-byte-swizzled K-major layout that tcgen05.mma reads (96 KB at H = 1024): R is read
//   from HBM once per pass.
// * The other operand is streamed every step by TMA (cp.async.bulk.tensor, no multicast)
//   straight out of the tensor the step before wrote - h itself in the forward pass, the
//   gate-gradient tensor dq in the backward pass - through an mbarrier ring; nothing is
//   packed into a separate exchange buffer.
// * The accumulator lives in tensor memory (two buffers, so the tile that follows starts
//   while this one is drained); four epilogue warps read it with tcgen05.ld, one batch row
//   per thread, and do the whole gate math, zoneout and the stores for their 16 units.
// * Steps synchronise through one arrival counter per row tile: an epilogue warp that has
//   stored its part of step t adds one (release); the TMA warp of every CTA of the row group
//   waits for all of them (acquire) before it loads step t's operand.  CTAs of different row
//   groups never wait for each other, and with several tiles per CTA the wait for one tile
//   hides behind the contraction of the others.
// * Every wait - counter or mbarrier - is bounded; on expiry the grid's abort flag and the
//   process error word are set, all roles leave their loops, tensor memory is released and
//   the host reports HASTE_B200_ERR_TIMEOUT.
//
// Warp roles (192 threads): warp 0 TMA producer, warp 1 MMA issuer, warps 2-5 epilogue.
// Replaces the per-step cuBLAS call + pointwise kernel of the reference
// (lib/gru_forward_gpu.cu.cc:214-308,345-363, lib/gru_backward_gpu.cu.cc:252-320) for
// bf16 batches of about a hundred rows and more; math as in lib/gru_forward_gpu.cu.cc:27-85
// and lib/gru_backward_gpu.cu.cc:26-96.
#include "recurrent_kernels.cuh"
#include "tcgen05.cuh"

namespace hb {
namespace {

using namespace tc;
using rec::sigmoid_fast;
using rec::tanh_fast;
typedef __nv_bfloat16 bf16;

constexpr int UC = 16;                 // hidden units per CTA
constexpr int BK = 64;                 // K elements per TMA box / swizzle row (128 bytes)
constexpr int A_STAGE = 128 * BK * 2;  // one streamed stage: 128 rows x 128 bytes
constexpr int TC_THREADS = 192;
constexpr int MAX_SMEM = 227 * 1024;

struct TcParams {
  int T, N, H, nHS, MT, RB, training, has_zoneout, r_transposed;
  int stage_bytes;     // RB * 128: one stage of the ring holds one k-block of RB rows
  int ring_bytes;      // stages * stage_bytes, plus padding up to a whole 128-row tile
  float zoneout_prob;
  const bf16* R;       // forward: [H,3H]; backward: [H,3H] or R_t [3H,H]
  const bf16* bx;      // forward
  const bf16* br;
  const bf16* Wx;      // forward: x.W [T,N,3H]
  const bf16* mask;    // [T,N,H] or null
  bf16* h;             // [T+1,N,H] (backward: read only)
  bf16* v;             // [T,N,4H] gate cache (forward: out or null; backward: in)
  const bf16* dh_new;  // backward [T+1,N,H]
  bf16* dp;            // backward out [T,N,3H]
  bf16* dq;            // backward out [T,N,3H], also the streamed operand
  float* dh_carry;     // backward [N,H] fp32 in/out
  unsigned int* cnt;   // [row tiles] arrival counters, zeroed before launch
  int* abort_flag;     // device-global, zeroed before launch
  int* err;            // process error word
};

__device__ __forceinline__ unsigned int ld_acquire_u32(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_add(unsigned int* p, unsigned int v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_all() {
  asm volatile("fence.proxy.async;" ::: "memory");
}

// Waits until *c >= target.  False when the limit ran out or the grid was aborted.
__device__ __forceinline__ bool wait_count(const unsigned int* c, unsigned int target,
                                           volatile int* s_abort, const TcParams& p, int code,
                                           int d0, int d1) {
  if (ld_acquire_u32(c) >= target) return true;
  const long long t0 = clock64();
  unsigned int it = 0;
  while (ld_acquire_u32(c) < target) {
    if ((++it & 63u) == 0) {
      if (*s_abort || *reinterpret_cast<volatile int*>(p.abort_flag)) {
        *s_abort = 1;
        return false;
      }
      if (clock64() - t0 > SPIN_LIMIT_CYCLES) {
        *s_abort = 1;
        if (atomicExch(p.abort_flag, 1) == 0) {
          volatile int* e = reinterpret_cast<volatile int*>(p.err);
          e[1] = blockIdx.x; e[2] = d0; e[3] = d1; e[4] = (int)target;
          __threadfence_system();
          e[0] = code;
        }
        __threadfence_system();
        return false;
      }
    }
  }
  return true;
}

// 16 consecutive bf16 (32 bytes, 16-byte aligned) <-> floats
__device__ __forceinline__ void ld16(const bf16* p, float (&x)[16]) {
  const uint4 a = *reinterpret_cast<const uint4*>(p);
  const uint4 b = *reinterpret_cast<const uint4*>(p + 8);
  const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    x[2 * i] = __uint_as_float(w[i] << 16);
    x[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}
__device__ __forceinline__ void st16(bf16* p, const float (&x)[16]) {
  uint32_t w[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    __nv_bfloat162 t2 = __floats2bfloat162_rn(x[2 * i], x[2 * i + 1]);
    w[i] = *reinterpret_cast<uint32_t*>(&t2);
  }
  *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
  *reinterpret_cast<uint4*>(p + 8) = make_uint4(w[4], w[5], w[6], w[7]);
}

// Byte offset of element (row n, k) inside one K-major, 128-byte-swizzled k-block tile
// (rows of 64 bf16 = 128 bytes; 16-byte chunk c of row n sits at chunk c ^ (n & 7)).
__device__ __forceinline__ uint32_t swz_off(int n, int kk) {
  return (uint32_t)((n >> 3) * 1024 + (n & 7) * 128 + ((((kk >> 3) ^ (n & 7)) & 7) << 4) + (kk & 7) * 2);
}

template <int NB, bool FWD>
__global__ void __launch_bounds__(TC_THREADS, 1)
gru_tc_kernel(const __grid_constant__ CUtensorMap map_a, const TcParams p, const int stages) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* aligned = smem_raw + (base - smem_u32(smem_raw));
  const int H = p.H, N = p.N;
  const int K = FWD ? H : 3 * H;
  const int KB = K / BK;
  constexpr int R_TILE = NB * 128;  // bytes of the resident operand per k-block
  const uint32_t r_bytes = (uint32_t)KB * R_TILE;
  const uint32_t ring = base + r_bytes;  // r_bytes is a multiple of 1024
  uint8_t* ring_ptr = aligned + r_bytes;
  // (a 64-row stage is read by the 128-row MMA together with the stage behind it - rows whose
  // results nobody uses - so the ring is padded by half a tile at its end)
  uint64_t* bars = reinterpret_cast<uint64_t*>(ring_ptr + p.ring_bytes);
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (stages + s); };
  auto accf_bar = [&](int a) { return bar0 + 8u * (2 * stages + a); };
  auto acce_bar = [&](int a) { return bar0 + 8u * (2 * stages + 2 + a); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * stages + 4);
  volatile int* s_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* s_bias = reinterpret_cast<float*>(tmem_slot + 4);  // forward: [2][48] bx, br

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hs = blockIdx.x % p.nHS, rg = blockIdx.x / p.nHS;
  const int u0 = hs * UC;
  constexpr int ACC_COLS = NB <= 32 ? 32 : 64;   // tensor-memory columns per accumulator
  constexpr uint32_t TMEM_COLS = 2 * ACC_COLS;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(accf_bar(a), 1);
      mbar_init(acce_bar(a), 128);
    }
    *s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_slot)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  // ---- streamed-operand ring: zero once, so that rows a 64-row box never writes are zeros
  for (int i = threadIdx.x; i < p.ring_bytes / 16; i += TC_THREADS)
    reinterpret_cast<uint4*>(ring_ptr)[i] = make_uint4(0u, 0u, 0u, 0u);
  // ---- resident operand: this CTA's slice of R, K-major and swizzled
  if (FWD) {
    // B^T[n = gate*16 + u][k] = R[k][gate*H + u0 + u]
    for (int item = threadIdx.x; item < K * 3; item += TC_THREADS) {
      const int k = item / 3, gate = item % 3;
      float x[16];
      ld16(p.R + (size_t)k * 3 * H + (size_t)gate * H + u0, x);
      uint8_t* tile = aligned + (size_t)(k / BK) * R_TILE;
#pragma unroll
      for (int u = 0; u < 16; ++u)
        *reinterpret_cast<bf16*>(tile + swz_off(gate * 16 + u, k % BK)) = __float2bfloat16_rn(x[u]);
    }
    for (int i = threadIdx.x; i < 96; i += TC_THREADS) {
      const int which = i / 48, c = i % 48, gate = c / 16, u = c % 16;
      s_bias[i] = __bfloat162float((which ? p.br : p.bx)[gate * H + u0 + u]);
    }
  } else {
    // B^T[n = unit j][k = gate column c] = R[u0 + j][c]   (R_t[c][u0 + j] when transposed)
    if (!p.r_transposed) {
      for (int item = threadIdx.x; item < 16 * (K / 8); item += TC_THREADS) {
        const int j = item / (K / 8), c8 = (item % (K / 8)) * 8;
        const uint4 w = *reinterpret_cast<const uint4*>(p.R + (size_t)(u0 + j) * K + c8);
        uint8_t* tile = aligned + (size_t)(c8 / BK) * R_TILE;
        *reinterpret_cast<uint4*>(tile + swz_off(j, c8 % BK)) = w;  // one whole 16-byte chunk
      }
    } else {
      for (int c = threadIdx.x; c < K; c += TC_THREADS) {
        float x[16];
        ld16(p.R + (size_t)c * H + u0, x);
        uint8_t* tile = aligned + (size_t)(c / BK) * R_TILE;
#pragma unroll
        for (int j = 0; j < 16; ++j)
          *reinterpret_cast<bf16*>(tile + swz_off(j, c % BK)) = __float2bfloat16_rn(x[j]);
      }
    }
  }
  // the tensor core reads shared memory through the async proxy
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int tiles_total = (N + p.RB - 1) / p.RB;
  const unsigned int arrivals = (unsigned int)p.nHS * 4u;  // per step: four epilogue warps per CTA

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      const uint32_t box_bytes = (uint32_t)p.RB * 128u;
      for (int it = 0; it < p.T && ok; ++it) {
        if (!FWD && it == 0) continue;  // the first backward step has no recurrent part
        for (int mt = 0; mt < p.MT && ok; ++mt) {
          const int tile = rg * p.MT + mt;
          if (tile >= tiles_total) break;
          // forward step it reads h_it (published it times); backward iteration it reads the
          // dq of iteration it-1 (published it times as well)
          if (it > 0 && !wait_count(p.cnt + tile, arrivals * (unsigned int)it, s_abort, p, 51,
                                    it, tile)) { ok = false; break; }
          fence_proxy_async_all();
          const int trow = FWD ? it : (p.T - it);  // time slot of the streamed tensor
          const int row = trow * N + tile * p.RB;
          for (int kb = 0; kb < KB; ++kb) {
            if (!mbar_wait(empty_bar(stage), phase ^ 1u, s_abort, p.err, 52)) { ok = false; break; }
            mbar_expect_tx(full_bar(stage), box_bytes);
            tma_load_3d(ring + stage * p.stage_bytes, &map_a, full_bar(stage), kb * BK, row, 0);
            if (++stage == (uint32_t)stages) { stage = 0; phase ^= 1u; }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(NB >> 3) << 17) |
                             ((uint32_t)(128 >> 4) << 24);
      uint32_t stage = 0, phase = 0;
      uint32_t acc_phase[2] = {0, 0};
      int n_acc = 0;
      bool ok = true;
      const uint64_t a_desc0 = smem_desc(ring, 16, 1024);
      const uint64_t b_desc0 = smem_desc(base, 16, 1024);
      const uint64_t a_stage_inc = (uint64_t)(p.stage_bytes >> 4);
      for (int it = 0; it < p.T && ok; ++it) {
        if (!FWD && it == 0) continue;
        for (int mt = 0; mt < p.MT && ok; ++mt) {
          if (rg * p.MT + mt >= tiles_total) break;
          const int acc = n_acc & 1;
          ++n_acc;
          if (!mbar_wait(acce_bar(acc), acc_phase[acc] ^ 1u, s_abort, p.err, 53)) { ok = false; break; }
          acc_phase[acc] ^= 1u;
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + acc * ACC_COLS;
          // Descriptors differ only in their 14-bit start-address field (bytes >> 4): one add
          // per MMA instead of rebuilding them - with N = 16 or 48 an instruction is a few
          // dozen cycles of tensor work, so the issuing thread's own instruction count is
          // what bounds the k-loop.
          uint64_t bd = b_desc0;
#pragma unroll 1
          for (int kb = 0; kb < KB; ++kb) {
            if (!mbar_wait(full_bar(stage), phase, s_abort, p.err, 54)) { ok = false; break; }
            tc_fence_after();
            const uint64_t ad = a_desc0 + (uint64_t)stage * a_stage_inc;
            tc_mma_bf16(d_tmem, ad, bd, idesc, kb ? 1u : 0u);
            tc_mma_bf16(d_tmem, ad + 2, bd + 2, idesc, 1u);
            tc_mma_bf16(d_tmem, ad + 4, bd + 4, idesc, 1u);
            tc_mma_bf16(d_tmem, ad + 6, bd + 6, idesc, 1u);
            tc_commit(empty_bar(stage));
            bd += R_TILE >> 4;
            if (++stage == (uint32_t)stages) { stage = 0; phase ^= 1u; }
          }
          if (ok) tc_commit(accf_bar(acc));
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    const int quad = warp & 3;
    const int r = quad * 32 + lane;  // row of the tile = tensor-memory lane
    uint32_t acc_phase[2] = {0, 0};
    int n_acc = 0;
    bool ok = true;
    const long long NH = (long long)N * H;
    for (int it = 0; it < p.T && ok; ++it) {
      const int t = FWD ? it : (p.T - 1 - it);
      for (int mt = 0; mt < p.MT && ok; ++mt) {
        const int tile = rg * p.MT + mt;
        if (tile >= tiles_total) break;
        const int n = tile * p.RB + r;
        const bool valid = r < p.RB && n < N;
        const bool have_acc = FWD || it > 0;
        const long long o0 = (long long)n * H + u0;
        // ---- inputs that do not depend on the recurrence
        float in0[16], in1[16], in2[16], in3[16], hp[16], mk[16], dhn[16], carry[16];
        if (valid) {
          if (FWD) {
            const bf16* wx = p.Wx + ((long long)t * N + n) * 3 * H + u0;
            ld16(wx, in0);
            ld16(wx + H, in1);
            ld16(wx + 2 * H, in2);
            ld16(p.h + (long long)t * NH + o0, hp);
            if (p.has_zoneout && p.training) ld16(p.mask + (long long)t * NH + o0, mk);
          } else {
            const bf16* vt = p.v + ((long long)t * N + n) * 4 * H + u0;
            ld16(vt, in0);
            ld16(vt + H, in1);
            ld16(vt + 2 * H, in2);
            ld16(vt + 3 * H, in3);
            ld16(p.h + (long long)t * NH + o0, hp);
            ld16(p.dh_new + (long long)(t + 1) * NH + o0, dhn);
            if (p.has_zoneout) ld16(p.mask + (long long)t * NH + o0, mk);
            const float4* cp = reinterpret_cast<const float4*>(p.dh_carry + o0);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float4 f = cp[i];
              carry[4 * i] = f.x; carry[4 * i + 1] = f.y; carry[4 * i + 2] = f.z; carry[4 * i + 3] = f.w;
            }
          }
        }
        // ---- the step product from tensor memory
        uint32_t a0[16], a1[16], a2[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) a0[i] = a1[i] = a2[i] = 0u;
        if (have_acc) {
          const int acc = n_acc & 1;
          ++n_acc;
          bool got = mbar_wait(accf_bar(acc), acc_phase[acc], s_abort, p.err, 55);
          got = __all_sync(0xffffffffu, got);
          if (!got) { ok = false; break; }
          acc_phase[acc] ^= 1u;
          tc_fence_after();
          const uint32_t taddr = tmem_base + acc * ACC_COLS + ((uint32_t)(quad * 32) << 16);
          tc_ld16(taddr, a0);
          if (FWD) {
            tc_ld16(taddr + 16, a1);
            tc_ld16(taddr + 32, a2);
          }
          tc_wait_ld();
          tc_fence_before();
          mbar_arrive(acce_bar(acc));
        }
        // ---- gate math; first the stores the next step streams (h / dq), then the publish,
        // then the stores nothing on the chain waits for (gate cache, dp, carry)
        float o0v[16], o1v[16], o2v[16], o3v[16];  // fwd: z, r, g, q   bwd: dp_z, dp_r, dp_g, dq_g
        if (valid) {
          if (FWD) {
            float hn[16];
#pragma unroll
            for (int u = 0; u < 16; ++u) {
              const float z = sigmoid_fast(in0[u] + __uint_as_float(a0[u]) + s_bias[u] + s_bias[48 + u]);
              const float rr = sigmoid_fast(in1[u] + __uint_as_float(a1[u]) + s_bias[16 + u] + s_bias[64 + u]);
              const float qg = __uint_as_float(a2[u]) + s_bias[80 + u];
              const float g = tanh_fast(in2[u] + rr * qg + s_bias[32 + u]);
              float x = z * hp[u] + (1.0f - z) * g;
              if (p.has_zoneout)
                x = p.training ? zoneout<true>(x, hp[u], p.zoneout_prob, mk[u])
                               : zoneout<false>(x, hp[u], p.zoneout_prob, 0.f);
              hn[u] = x; o0v[u] = z; o1v[u] = rr; o2v[u] = g; o3v[u] = qg;
            }
            st16(p.h + (long long)(t + 1) * NH + o0, hn);
          } else {
#pragma unroll
            for (int u = 0; u < 16; ++u) {
              const float z = in0[u], rr = in1[u], g = in2[u], qg = in3[u];
              float dh_total = dhn[u] + carry[u] + __uint_as_float(a0[u]);
              float keep = 0.f;
              if (p.has_zoneout) {
                keep = (1.0f - mk[u]) * dh_total;
                dh_total = mk[u] * dh_total;
              }
              const float dg = (1.0f - z) * dh_total;
              const float dz = (hp[u] - g) * dh_total;
              const float dp_g = d_tanh(g) * dg;
              o0v[u] = d_sigmoid(z) * dz;
              o1v[u] = d_sigmoid(rr) * (dp_g * qg);
              o2v[u] = dp_g;
              o3v[u] = dp_g * rr;
              carry[u] = keep + z * dh_total;
            }
            const long long w0 = ((long long)t * N + n) * 3 * H + u0;
            st16(p.dq + w0, o0v); st16(p.dq + w0 + H, o1v); st16(p.dq + w0 + 2 * H, o3v);
          }
        }
        // publish: the stores above become visible to the other CTAs' TMA loads, then the
        // warp's arrival is counted (rows beyond the batch store nothing but still arrive)
        fence_proxy_async_all();
        __threadfence();
        __syncwarp();
        if (lane == 0) red_release_add(p.cnt + tile, 1u);
        if (valid) {
          if (FWD) {
            if (p.training && p.v) {
              bf16* vt = p.v + ((long long)t * N + n) * 4 * H + u0;
              st16(vt, o0v); st16(vt + H, o1v); st16(vt + 2 * H, o2v); st16(vt + 3 * H, o3v);
            }
          } else {
            const long long w0 = ((long long)t * N + n) * 3 * H + u0;
            st16(p.dp + w0, o0v); st16(p.dp + w0 + H, o1v); st16(p.dp + w0 + 2 * H, o2v);
            float4* cp = reinterpret_cast<float4*>(p.dh_carry + o0);
#pragma unroll
            for (int i = 0; i < 4; ++i)
              cp[i] = make_float4(carry[4 * i], carry[4 * i + 1], carry[4 * i + 2], carry[4 * i + 3]);
          }
        }
      }
    }
  }

  // Drain: every role arrives here, also after a time-out, so tensor memory is released.
  tc_fence_before();
  __syncthreads();
  if (*s_abort) atomicExch(p.abort_flag, 1);
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(TMEM_COLS)
                 : "memory");
  }
}

// ---- host side ---------------------------------------------------------------------------
struct TcGeometry {
  int nHS, nRG, MT, RB, stages;
  size_t ring, smem;
};

// Shapes this path takes: bf16, H a multiple of 64 up to 1024 (the resident slice of R and a
// useful ring must fit shared memory), at least 96 batch rows (below that the register
// kernels are faster) and at most two row tiles per CTA: every CTA of a row group streams
// the group's whole h (or dq), H / 16 copies of it per step out of L2, which is what bounds
// the step from a few hundred rows per GPU on - there the per-step contraction + pointwise
// launches of the step-wise path, with their full-size tiles, are faster (measured at
// H = 1024: forward 9.4 / 10.3 / 11.8 us per step at 128 / 256 / 512 rows against 9.3
// (register kernel) / 18.4 / 20.5 us; backward 20.6 / 22.4 / 30.4 against 16.4 / 18.6 / 24.6).
// `half` asks for the geometry under the SM budget (concurrent directions); without it, or
// when the budget would need more than two tiles per CTA, the whole GPU is used.
bool tc_geometry_for(int N, int H, bool fwd, int sms, TcGeometry* g) {
  const int K = fwd ? H : 3 * H;
  const size_t r_bytes = (size_t)(K / BK) * (fwd ? 48 : 16) * 128;
  const size_t fixed = 1024 /*alignment*/ + r_bytes + 1024 /*barriers, bias*/;
  if (fixed + 2 * (size_t)A_STAGE > (size_t)MAX_SMEM) return false;
  g->nHS = H / UC;
  const int groups_max = sms / g->nHS;
  if (groups_max < 1) return false;
  // 64-row tiles when that still gives one tile per CTA (more CTAs, less to stream per CTA)
  for (int rb = 64; rb <= 128; rb *= 2) {
    const int tiles = ceil_div(N, rb);
    const int mt = ceil_div(tiles, groups_max);
    if (rb == 64 && mt > 1) continue;
    if (mt > 2) return false;
    g->RB = rb;
    g->MT = mt;
    g->nRG = ceil_div(tiles, mt);
    // ring: as many stages of one k-block (rb rows x 128 bytes) as shared memory holds, up
    // to 16; bytes in flight are what the streaming rate of a step is made of
    const size_t stage = (size_t)rb * 128, pad = A_STAGE - stage;
    int stages = (int)(((size_t)MAX_SMEM - fixed - pad) / stage);
    if (stages > 16) stages = 16;
    g->stages = stages;
    g->ring = stages * stage + pad;
    g->smem = fixed + g->ring;
    return true;
  }
  return false;
}

// `budgeted` reports whether the geometry honours the SM budget (then the two directions of a
// bidirectional layer are co-resident).
bool tc_geometry(int N, int H, bool fwd, TcGeometry* g, bool* budgeted) {
  *budgeted = false;
  if (H % 64 != 0 || H < 64 || H > 1024 || N < 96) return false;
  const int budget = sm_budget();
  if (budget > 0 && budget < sm_count() && tc_geometry_for(N, H, fwd, budget, g)) {
    *budgeted = true;
    return true;
  }
  return tc_geometry_for(N, H, fwd, sm_count(), g);
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <int NB, bool FWD>
int launch_tc(const CUtensorMap& map, TcParams& p, const TcGeometry& g, cudaStream_t s) {
  auto kernel = gru_tc_kernel<NB, FWD>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)g.smem);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return HASTE_B200_ERR_UNSUPPORTED;
  }
  int per_sm = 0;
  e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, TC_THREADS, g.smem);
  const int grid = g.nHS * g.nRG;
  if (e != cudaSuccess || per_sm * sm_count() < grid) {
    cudaGetLastError();
    return HASTE_B200_ERR_UNSUPPORTED;
  }
  int stages = g.stages;
  void* args[] = {const_cast<CUtensorMap*>(&map), &p, &stages};
  e = cudaLaunchCooperativeKernel((const void*)kernel, dim3(grid), dim3(TC_THREADS), args, g.smem, s);
  if (e != cudaSuccess) {
    set_last_error("cooperative launch failed: %s", cudaGetErrorString(e));
    cudaGetLastError();
    return HASTE_B200_ERR_CUDA;
  }
  count_launch(1);
  return HASTE_B200_OK;
}

// Zeroed scratch: abort flag + one arrival counter per row tile.
int tc_scratch(int tiles, TcParams* p, cudaStream_t s) {
  const size_t bytes = Arena::pad(4096) + Arena::pad((size_t)tiles * 4);
  Arena ws;
  HB_TRY(make_arena(&ws, s, bytes + 512, /*slot=*/2));
  int* flag = ws.take<int>(1024);
  unsigned int* cnt = ws.take<unsigned int>(tiles);
  HB_REQUIRE(flag && cnt, "scratch arena");
  HB_CUDA_OK(cudaMemsetAsync(flag, 0, bytes, s));
  p->abort_flag = flag;
  p->cnt = cnt;
  p->err = device_error_word();
  HB_REQUIRE(p->err, "error word");
  return HASTE_B200_OK;
}

}  // namespace

// Forward: x.W is already in a.tmp_Wx.  HASTE_B200_ERR_UNSUPPORTED (nothing touched) when the
// shape is not this path's.
int gru_forward_tc(const GruFwd& a, cudaStream_t s) {
  TcGeometry g;
  bool budgeted = false;
  if (a.dtype != HASTE_B200_BF16 || recurrence_path() == HASTE_B200_PATH_STEPWISE ||
      recurrence_path() == HASTE_B200_PATH_NO_TENSOR_CORE || a.h_out ||
      !encode_fn() || !tc_geometry(a.N, a.H, true, &g, &budgeted))
    return HASTE_B200_ERR_UNSUPPORTED;
  if (!aligned16(a.R) || !aligned16(a.tmp_Wx) || !aligned16(a.h) || !aligned16(a.v) ||
      !aligned16(a.zoneout_mask) || !aligned16(a.bx) || !aligned16(a.br))
    return HASTE_B200_ERR_UNSUPPORTED;
  CUtensorMap map;
  if (!make_map(&map, a.h, a.H, (long long)(a.T + 1) * a.N, a.H, 0, 1, BK, g.RB))
    return HASTE_B200_ERR_UNSUPPORTED;
  const bool zo = a.zoneout_prob != 0.0f && a.zoneout_mask != nullptr;
  TcParams p{};
  p.T = a.T; p.N = a.N; p.H = a.H; p.nHS = g.nHS; p.MT = g.MT; p.RB = g.RB;
  p.stage_bytes = g.RB * 128; p.ring_bytes = (int)g.ring;
  p.training = a.training; p.has_zoneout = zo ? 1 : 0; p.zoneout_prob = a.zoneout_prob;
  p.R = (const bf16*)a.R; p.bx = (const bf16*)a.bx; p.br = (const bf16*)a.br;
  p.Wx = (const bf16*)a.tmp_Wx; p.mask = (const bf16*)a.zoneout_mask;
  p.h = (bf16*)a.h; p.v = (bf16*)a.v;
  HB_TRY(tc_scratch(ceil_div(a.N, g.RB), &p, s));
  return launch_tc<48, true>(map, p, g, s);
}

// Backward: dh_carry (fp32 [N,H]) holds the incoming gradient of the final state and receives
// the carry after the last processed step, without the recurrent contribution of that step
// (the caller adds dq_0 . R^T).  Bias gradients are NOT summed here.
int gru_backward_tc(const GruBwd& a, float* dh_carry, cudaStream_t s) {
  TcGeometry g;
  bool budgeted = false;
  if (a.dtype != HASTE_B200_BF16 || recurrence_path() == HASTE_B200_PATH_STEPWISE ||
      recurrence_path() == HASTE_B200_PATH_NO_TENSOR_CORE || a.iterate ||
      !encode_fn() || !tc_geometry(a.N, a.H, false, &g, &budgeted))
    return HASTE_B200_ERR_UNSUPPORTED;
  // On its own this kernel is slower than the register kernel / the step-wise path (see
  // tc_geometry_for); it pays when it lets the two directions of a layer run at the same time,
  // or when the caller asks for the persistent path explicitly.
  if (!budgeted && recurrence_path() != HASTE_B200_PATH_PERSISTENT)
    return HASTE_B200_ERR_UNSUPPORTED;
  if (!aligned16(a.R) || !aligned16(a.h) || !aligned16(a.v) || !aligned16(a.dh_new) ||
      !aligned16(a.dp) || !aligned16(a.dq) || !aligned16(a.zoneout_mask) || !aligned16(dh_carry))
    return HASTE_B200_ERR_UNSUPPORTED;
  CUtensorMap map;
  if (!make_map(&map, a.dq, 3LL * a.H, (long long)a.T * a.N, 3LL * a.H, 0, 1, BK, g.RB))
    return HASTE_B200_ERR_UNSUPPORTED;
  TcParams p{};
  p.T = a.T; p.N = a.N; p.H = a.H; p.nHS = g.nHS; p.MT = g.MT; p.RB = g.RB;
  p.stage_bytes = g.RB * 128; p.ring_bytes = (int)g.ring;
  p.has_zoneout = a.zoneout_mask ? 1 : 0; p.r_transposed = a.transposed_inputs;
  p.R = (const bf16*)a.R; p.mask = (const bf16*)a.zoneout_mask;
  p.h = (bf16*)const_cast<void*>(a.h); p.v = (bf16*)const_cast<void*>(a.v);
  p.dh_new = (const bf16*)a.dh_new; p.dp = (bf16*)a.dp; p.dq = (bf16*)a.dq;
  p.dh_carry = dh_carry;
  HB_TRY(tc_scratch(ceil_div(a.N, g.RB), &p, s));
  return launch_tc<16, false>(map, p, g, s);
}

}  // namespace hb
