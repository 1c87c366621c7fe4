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
// * The other operand is streamed every step by TMA (cp.async.bulk.tensor; every CTA fetches
//   its own copy) straight out of the tensor the step before wrote - h itself in the forward
//   pass, the gate-gradient tensor dq in the backward pass - through an mbarrier ring; nothing
//   is packed into a separate exchange buffer.
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
// Warp roles: warp 0 TMA producer (four lanes issue), warps 1..NI MMA issuers (a tcgen05.mma
// of this shape occupies its issuing thread for ~65 cycles, 2-3x its tensor-pipe time, so NI
// threads issue the k-blocks in turn, each into its own accumulator), then four epilogue warps.
// Replaces the per-step cuBLAS call + pointwise kernel of the reference
// (lib/gru_forward_gpu.cu.cc:214-308,345-363, lib/gru_backward_gpu.cu.cc:252-320) for
// bf16 batches of about a hundred rows and more; math as in lib/gru_forward_gpu.cu.cc:27-85
// and lib/gru_backward_gpu.cu.cc:26-96.
#include "recurrent_kernels.cuh"
#include "tcgen05.cuh"

namespace hb {
namespace {

using namespace tc;
typedef __nv_bfloat16 bf16;

// Gate functions of this bf16-only path: one MUFU.TANH each (relative error 2^-11, a
// fraction of a bf16 ulp; the parity bar of bf16 storage is 2e-2).
__device__ __forceinline__ float tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float sigmoid_fast(float x) { return fmaf(0.5f, tanh_fast(0.5f * x), 0.5f); }

constexpr int UC = 16;                 // hidden units per CTA
constexpr int BK = 64;                 // K elements per TMA box / swizzle row (128 bytes)
constexpr int A_STAGE = 128 * BK * 2;  // one streamed stage: 128 rows x 128 bytes
#ifndef HB_TC_NI
#define HB_TC_NI 4
#endif
constexpr int NI = HB_TC_NI;           // MMA-issuing warps (k-blocks go to them in turn)
constexpr int TC_THREADS = 32 * (1 + NI + 4);  // warp 0 TMA, warps 1..NI MMA, then 4 epilogue warps
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
#ifdef HASTE_B200_TIMING_EXPERIMENTS
  long long* stamps;   // [T][16] clock64 stamps of CTA 0, tile 0 (timing-experiment builds only)
#endif
};

#ifdef HASTE_B200_TIMING_EXPERIMENTS
#define HB_STAMP(p, it, mt, slot)                                            \
  do {                                                                       \
    if ((p).stamps && blockIdx.x == 0 && (mt) == 0)                          \
      (p).stamps[(size_t)(it) * 16 + (slot)] = clock64();                     \
  } while (0)
#else
#define HB_STAMP(p, it, mt, slot) do {} while (0)
#endif

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
  // (polling with relaxed loads and one acquire fence at the end measured 0.2 us per step slower)
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

// 8 consecutive bf16 as one 16-byte load, and element u of such a group as a float
__device__ __forceinline__ uint4 ldq(const bf16* p) { return *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ float bfq(const uint4& q, int u) {
  const uint32_t w = (u >> 1) == 0 ? q.x : ((u >> 1) == 1 ? q.y : ((u >> 1) == 2 ? q.z : q.w));
  return (u & 1) ? __uint_as_float(w & 0xFFFF0000u) : __uint_as_float(w << 16);
}

// 8 consecutive bf16 (16 bytes, 16-byte aligned) <-> floats
__device__ __forceinline__ void ld8(const bf16* p, float (&x)[8]) {
  const uint4 a = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    x[2 * i] = __uint_as_float(w[i] << 16);
    x[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}
__device__ __forceinline__ void st8(bf16* p, const float (&x)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __nv_bfloat162 t2 = __floats2bfloat162_rn(x[2 * i], x[2 * i + 1]);
    w[i] = *reinterpret_cast<uint32_t*>(&t2);
  }
  *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
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
  constexpr uint32_t TMEM_COLS = 2 * NI * ACC_COLS;  // two buffers x one accumulator per issuer

  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_a)) : "memory");
    for (int s = 0; s < stages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(accf_bar(a), NI);
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
    // PL lanes issue the k-blocks of a tile in turn (lane l takes k-blocks l, l + PL, ...): a
    // cp.async.bulk.tensor holds its issuing thread for about 0.1 us, which would otherwise
    // be the rate of the whole ring.
    constexpr int PL = 4;
    constexpr unsigned PMASK = (1u << PL) - 1u;
    if (lane < PL) {
      uint32_t g0 = 0;  // k-blocks issued before this tile (the same in every lane)
      bool ok = true;
      const uint32_t box_bytes = (uint32_t)p.RB * 128u;
      for (int it = 0; it < p.T && ok; ++it) {
        if (!FWD && it == 0) continue;  // the first backward step has no recurrent part
        for (int mt = 0; mt < p.MT && ok; ++mt) {
          const int tile = rg * p.MT + mt;
          if (tile >= tiles_total) break;
          // forward step it reads h_it (published it times); backward iteration it reads the
          // dq of iteration it-1 (published it times as well)
          if (it > 0 && lane == 0)
            ok = wait_count(p.cnt + tile, arrivals * (unsigned int)it, s_abort, p, 51, it, tile);
          __syncwarp(PMASK);  // lane 0's acquire is ordered before the other lanes' loads
          HB_STAMP(p, it, mt, 0);  // the step's operand is published
          fence_proxy_async_all();
          const int trow = FWD ? it : (p.T - it);  // time slot of the streamed tensor
          const int row = trow * N + tile * p.RB;
          for (int kb = lane; kb < KB && ok; kb += PL) {
            const uint32_t g = g0 + (uint32_t)kb;
            const uint32_t stage = g % (uint32_t)stages, phase = (g / (uint32_t)stages) & 1u;
            if (!mbar_wait(empty_bar(stage), phase ^ 1u, s_abort, p.err, 52)) { ok = false; break; }
            mbar_expect_tx(full_bar(stage), box_bytes);
            tma_load_3d(ring + stage * p.stage_bytes, &map_a, full_bar(stage), kb * BK, row, 0);
          }
          g0 += (uint32_t)KB;
          ok = __all_sync(PMASK, ok);  // all producer lanes leave together
          HB_STAMP(p, it, mt, 1);  // all TMA loads of the tile issued
        }
      }
    }
  } else if (warp <= NI) {
    // ------------------------------------------------------------------ MMA issuers
    if (lane == 0) {
      const int iss = warp - 1;  // this issuer takes k-blocks iss, iss + NI, ...
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(NB >> 3) << 17) |
                             ((uint32_t)(128 >> 4) << 24);
      uint32_t g0 = 0;  // k-blocks consumed before this tile
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
          const uint32_t d_tmem = tmem_base + (acc * NI + iss) * ACC_COLS;
          // Descriptors differ only in their 14-bit start-address field (bytes >> 4): one add
          // per MMA instead of rebuilding them.
#pragma unroll 1
          for (int kb = iss; kb < KB; kb += NI) {
            const uint32_t g = g0 + (uint32_t)kb;
            const uint32_t stage = g % (uint32_t)stages, phase = (g / (uint32_t)stages) & 1u;
            if (!mbar_wait(full_bar(stage), phase, s_abort, p.err, 54)) { ok = false; break; }
            tc_fence_after();
            if (kb == 0) HB_STAMP(p, it, mt, 2);  // first k-block has landed
            const uint64_t ad = a_desc0 + (uint64_t)stage * a_stage_inc;
            const uint64_t bd = b_desc0 + (uint64_t)kb * (R_TILE >> 4);
            tc_mma_bf16(d_tmem, ad, bd, idesc, kb >= NI ? 1u : 0u);
            tc_mma_bf16(d_tmem, ad + 2, bd + 2, idesc, 1u);
            tc_mma_bf16(d_tmem, ad + 4, bd + 4, idesc, 1u);
            tc_mma_bf16(d_tmem, ad + 6, bd + 6, idesc, 1u);
            tc_commit(empty_bar(stage));
          }
          g0 += (uint32_t)KB;
          if (iss == 0) HB_STAMP(p, it, mt, 3);  // last MMA issued
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
        // The 16 units are handled in two halves of 8 and the step inputs stay packed (bf16
        // pairs) until they are used, so that the live state of a thread stays within its
        // share of the register file (nine warps per CTA).
        // ---- inputs that do not depend on the recurrence: issued before the wait below
        uint4 in0[2], in1[2], in2[2], in3[2], hp[2], mk[2], dhn[2];
        float carry[2][8];
        if (valid) {
#pragma unroll
          for (int hf = 0; hf < 2; ++hf) {
            const int uo = hf * 8;
            if (FWD) {
              const bf16* wx = p.Wx + ((long long)t * N + n) * 3 * H + u0 + uo;
              in0[hf] = ldq(wx);
              in1[hf] = ldq(wx + H);
              in2[hf] = ldq(wx + 2 * H);
              hp[hf] = ldq(p.h + (long long)t * NH + o0 + uo);
              if (p.has_zoneout && p.training) mk[hf] = ldq(p.mask + (long long)t * NH + o0 + uo);
            } else {
              const bf16* vt = p.v + ((long long)t * N + n) * 4 * H + u0 + uo;
              in0[hf] = ldq(vt);
              in1[hf] = ldq(vt + H);
              in2[hf] = ldq(vt + 2 * H);
              in3[hf] = ldq(vt + 3 * H);
              hp[hf] = ldq(p.h + (long long)t * NH + o0 + uo);
              dhn[hf] = ldq(p.dh_new + (long long)(t + 1) * NH + o0 + uo);
              if (p.has_zoneout) mk[hf] = ldq(p.mask + (long long)t * NH + o0 + uo);
              const float4* cp = reinterpret_cast<const float4*>(p.dh_carry + o0 + uo);
              const float4 f0 = cp[0], f1 = cp[1];
              carry[hf][0] = f0.x; carry[hf][1] = f0.y; carry[hf][2] = f0.z; carry[hf][3] = f0.w;
              carry[hf][4] = f1.x; carry[hf][5] = f1.y; carry[hf][6] = f1.z; carry[hf][7] = f1.w;
            }
          }
        }
        // ---- wait for the step product
        int acc = 0;
        if (have_acc) {
          acc = n_acc & 1;
          ++n_acc;
          bool got = mbar_wait(accf_bar(acc), acc_phase[acc], s_abort, p.err, 55);
          got = __all_sync(0xffffffffu, got);
          if (!got) { ok = false; break; }
          acc_phase[acc] ^= 1u;
          tc_fence_after();
          if (warp == NI + 1 && lane == 0) HB_STAMP(p, it, mt, 4);  // accumulator complete
        }
        const uint32_t taddr = tmem_base + acc * NI * ACC_COLS + ((uint32_t)(quad * 32) << 16);
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          const int uo = hf * 8;
          // this half's columns of the accumulators (one per issuer), summed
          float s0[8], s1[8], s2[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) s0[i] = s1[i] = s2[i] = 0.f;
          if (have_acc) {
            // the issuers' accumulators, GRP of them per wait (all loads of a group in flight)
            constexpr int GRP = FWD ? 2 : NI;
#pragma unroll
            for (int g0 = 0; g0 < NI; g0 += GRP) {
              uint32_t b0[GRP][8], b1[GRP][8], b2[GRP][8];
#pragma unroll
              for (int k = 0; k < GRP; ++k) {
                const int i2 = g0 + k;
                if (i2 < NI && KB > i2) {
                  tc_ld8(taddr + i2 * ACC_COLS + uo, b0[k]);
                  if (FWD) {
                    tc_ld8(taddr + i2 * ACC_COLS + 16 + uo, b1[k]);
                    tc_ld8(taddr + i2 * ACC_COLS + 32 + uo, b2[k]);
                  }
                }
              }
              tc_wait_ld();
#pragma unroll
              for (int k = 0; k < GRP; ++k) {
                const int i2 = g0 + k;
                if (i2 < NI && KB > i2) {
#pragma unroll
                  for (int i = 0; i < 8; ++i) {
                    s0[i] += __uint_as_float(b0[k][i]);
                    if (FWD) {
                      s1[i] += __uint_as_float(b1[k][i]);
                      s2[i] += __uint_as_float(b2[k][i]);
                    }
                  }
                }
              }
            }
            if (hf == 1) {  // both halves are in registers: the accumulator buffer is free
              tc_fence_before();
              mbar_arrive(acce_bar(acc));
              if (warp == NI + 1 && lane == 0) HB_STAMP(p, it, mt, 5);
            }
          }
          if (valid) {
            if (FWD) {
              float hn[8], vz[8], vr[8], vg[8], vq[8];
#pragma unroll
              for (int u = 0; u < 8; ++u) {
                const float hprev = bfq(hp[hf], u);
                const float z = sigmoid_fast(bfq(in0[hf], u) + s0[u] + s_bias[uo + u] + s_bias[48 + uo + u]);
                const float rr = sigmoid_fast(bfq(in1[hf], u) + s1[u] + s_bias[16 + uo + u] + s_bias[64 + uo + u]);
                const float qg = s2[u] + s_bias[80 + uo + u];
                const float g = tanh_fast(bfq(in2[hf], u) + rr * qg + s_bias[32 + uo + u]);
                float x = z * hprev + (1.0f - z) * g;
                if (p.has_zoneout)
                  x = p.training ? zoneout<true>(x, hprev, p.zoneout_prob, bfq(mk[hf], u))
                                 : zoneout<false>(x, hprev, p.zoneout_prob, 0.f);
                hn[u] = x; vz[u] = z; vr[u] = rr; vg[u] = g; vq[u] = qg;
              }
              st8(p.h + (long long)(t + 1) * NH + o0 + uo, hn);  // the next step streams it
              if (p.training && p.v) {
                bf16* vt = p.v + ((long long)t * N + n) * 4 * H + u0 + uo;
                st8(vt, vz); st8(vt + H, vr); st8(vt + 2 * H, vg); st8(vt + 3 * H, vq);
              }
            } else {
              float dpz[8], dpr[8], dpg[8], dqg[8];
#pragma unroll
              for (int u = 0; u < 8; ++u) {
                const float z = bfq(in0[hf], u), rr = bfq(in1[hf], u), g = bfq(in2[hf], u),
                            qg = bfq(in3[hf], u);
                float dh_total = bfq(dhn[hf], u) + carry[hf][u] + s0[u];
                float keep = 0.f;
                if (p.has_zoneout) {
                  const float m = bfq(mk[hf], u);
                  keep = (1.0f - m) * dh_total;
                  dh_total = m * dh_total;
                }
                const float dg = (1.0f - z) * dh_total;
                const float dz = (bfq(hp[hf], u) - g) * dh_total;
                const float dp_g = d_tanh(g) * dg;
                dpz[u] = d_sigmoid(z) * dz;
                dpr[u] = d_sigmoid(rr) * (dp_g * qg);
                dpg[u] = dp_g;
                dqg[u] = dp_g * rr;
                carry[hf][u] = keep + z * dh_total;
              }
              const long long w0 = ((long long)t * N + n) * 3 * H + u0 + uo;
              st8(p.dq + w0, dpz); st8(p.dq + w0 + H, dpr); st8(p.dq + w0 + 2 * H, dqg);  // streamed next
              st8(p.dp + w0, dpz); st8(p.dp + w0 + H, dpr); st8(p.dp + w0 + 2 * H, dpg);
              float4* cp = reinterpret_cast<float4*>(p.dh_carry + o0 + uo);
              cp[0] = make_float4(carry[hf][0], carry[hf][1], carry[hf][2], carry[hf][3]);
              cp[1] = make_float4(carry[hf][4], carry[hf][5], carry[hf][6], carry[hf][7]);
            }
          }
        }
        if (warp == NI + 1 && lane == 0) HB_STAMP(p, it, mt, 6);  // gate math done, h / dq stored
        // ---- publish.  The warp barrier orders every lane's stores before lane 0's release,
        // and a release at GPU scope is cumulative: it makes visible what happened before it
        // in any thread it synchronised with, so the one red.release counts the warp's arrival
        // and publishes all 32 lanes' stores.  (A __threadfence() in front of it cost another
        // 0.5 us per step and changed nothing.)  Only lane 0 waits; the other lanes go on to
        // the next step's loads.  Rows beyond the batch store nothing but still arrive.
        __syncwarp();
        if (lane == 0) red_release_add(p.cnt + tile, 1u);
        if (warp == NI + 1 && lane == 0) HB_STAMP(p, it, mt, 7);  // published
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

#ifdef HASTE_B200_TIMING_EXPERIMENTS
long long* g_stamps = nullptr;
int g_stamp_steps = 0;
#endif

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
#ifdef HASTE_B200_TIMING_EXPERIMENTS
  if (!g_stamps) cudaMalloc(&g_stamps, (size_t)4096 * 16 * sizeof(long long));
  cudaMemsetAsync(g_stamps, 0, (size_t)4096 * 16 * sizeof(long long), s);
  p->stamps = p->T <= 4096 ? g_stamps : nullptr;
  g_stamp_steps = p->T;
#endif
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

#ifdef HASTE_B200_TIMING_EXPERIMENTS
// Timing-experiment builds only: the clock64 stamps the last tensor-core recurrence launch
// left (CTA 0, tile 0; eight per step), copied to host memory.
extern "C" int haste_b200_debug_read_stamps(long long* out, int max_steps) {
  if (!g_stamps) return 0;
  const int n = g_stamp_steps < max_steps ? g_stamp_steps : max_steps;
  cudaDeviceSynchronize();
  cudaMemcpy(out, g_stamps, (size_t)n * 16 * sizeof(long long), cudaMemcpyDeviceToHost);
  return n;
}
#endif

}  // namespace hb
