// Dense contraction on the 5th-generation tensor cores (sm_100a):
//   TMA (cp.async.bulk.tensor, 128-byte swizzle) -> shared memory -> tcgen05.mma with
//   the fp32 accumulator in tensor memory -> tcgen05.ld epilogue.
//
//   C[M,N] (+)= sum over products p of A_p[M,K] . B_p[K,N]        (bf16 operands)
//
// * bf16 storage: one product, operands read in place.
// * fp32 storage: every operand is first split into two bf16 planes, x = hi + lo with
//   hi = bf16(x), lo = bf16(x - hi), and three products are accumulated
//   (hi.hi + hi.lo + lo.hi).  The dropped lo.lo term and the plane rounding leave a
//   relative error near 2^-17 per product, far inside the 1e-4 parity bar, at 3/16 of
//   the fp32 CUDA-core cost.
// * Either operand may be K-major or MN-major (every transpose the cells need), chosen
//   from its strides; no data is ever transposed in memory.
// * Persistent kernel: one CTA per SM walks (tile, k-split) work items.  Warp 0 issues
//   TMA, warp 1 issues MMA, warps 2-5 drain the accumulator; two accumulators in tensor
//   memory let the epilogue of one tile overlap the main loop of the next.
// * Long-K, small-output contractions (the weight gradients, K = T*N) are split along K;
//   partial tiles go to scratch and a second kernel sums them in a fixed order.
// * Every wait on an mbarrier is bounded; on expiry the kernel raises an error word,
//   all roles drain and exit, tensor memory is released and the host returns
//   HASTE_B200_ERR_TIMEOUT.
//
// Replaces the cuBLAS calls of the reference (lib/blas.h:48-61 and the call sites in
// lib/*_gpu.cu.cc).
#include <atomic>

#include "cells.cuh"
#include "tcgen05.cuh"

namespace hb {
namespace {

using namespace tc;

constexpr int BM = 128, BN = 128, BK = 64;   // CTA tile; BK bf16 = one 128-byte swizzle row
constexpr int UK = 16;                       // K of one tcgen05.mma (bf16)
constexpr int TILE_BYTES = BM * BK * 2;      // one operand plane of one stage (A or B): 16 KiB
constexpr int THREADS = 192;                 // warp 0 TMA, warp 1 MMA, warps 2..5 epilogue
constexpr int NACC = 4;                      // fp32 accumulators of BN columns in tensor memory
constexpr int TMEM_COLS = NACC * BN;         // (all 512 columns: one CTA per SM)

struct Params {
  int M, N, K;
  int a_mn_major, b_mn_major;  // 0: K contiguous, 1: M/N contiguous
  int tiles_m, tiles_n, splits, kb_per_split, kb_total;
  int c_is_bf16, accumulate;   // direct epilogue only; c_is_bf16: 0 fp32, 1 bf16, 2 fp16 output
  void* c;
  long long ldc;
  float* partial;              // non-null: write fp32 partial tiles [split][M][N]
  int* err;
};

template <int NPROD>
struct Cfg {
  // 1 product: bf16 operands as they are.  3 products: (hi, lo) planes.  6 products:
  // (hi, mid, lo) planes, accurate to fp32 rounding (used where LayerNorm amplifies error).
  static constexpr int PLANES = NPROD == 1 ? 1 : (NPROD == 3 ? 2 : 3);
  static constexpr int STAGE_BYTES = 2 * PLANES * TILE_BYTES;
  static constexpr int STAGES = NPROD == 1 ? 6 : (NPROD == 3 ? 3 : 2);
  static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;
  // fp32 storage: the tensor core adds every MMA result into the fp32 accumulator with
  // truncation, a bias of about half an ulp per accumulation that always points the same way;
  // over the few hundred accumulations of a long K it reaches 1e-5 of the result (measured:
  // 1.2e-5 at K = 1024 with six products, where the operand planes themselves are exact to
  // 2^-25).  The accumulator is therefore handed over every CHUNK k-blocks: the epilogue warps
  // add it into fp32 registers with round-to-nearest while the MMA warp continues in the
  // other accumulator.  0: one hand-over per tile (bf16 storage, where 2e-2 is the bar).
  // Four accumulators take turns, so the MMA warp runs up to three chunks ahead of the
  // epilogue; a chunk is about 1.6 us of MMA work either way.
  // (Twice these chunk lengths fails the fp32 parity test of the three-layer LayerNormLSTM stack.)
  static constexpr int CHUNK = NPROD == 1 ? 0 : (NPROD == 3 ? 4 : 2);
};

// Stores 32 consecutive columns (starting at nb) of row m of the result: r holds the fp32 bit
// patterns.  Partial tile of a K split, or the final C in fp32 / bf16 / fp16, optionally
// accumulating into what C holds.
__device__ __forceinline__ void store_chunk(const Params& p, int sp, int m, int nb,
                                      const uint32_t (&r)[32]) {
  if (m < p.M && nb < p.N) {
    if (p.partial) {
      float* dst = p.partial + ((long long)sp * p.M + m) * p.N + nb;
      if (nb + 32 <= p.N && (p.N & 3) == 0) {
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          *reinterpret_cast<float4*>(dst + j) =
              make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]),
                          __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
      } else {
        for (int j = 0; j < 32 && nb + j < p.N; ++j) dst[j] = __uint_as_float(r[j]);
      }
    } else if (p.c_is_bf16) {
      __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.c) + (long long)m * p.ldc + nb;
      if (nb + 32 <= p.N && (p.ldc & 7) == 0 &&
          (reinterpret_cast<uintptr_t>(p.c) & 15) == 0) {
        // 16-byte stores: eight bf16 per store, four per 32-column chunk
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          float v[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) v[e] = __uint_as_float(r[j + e]);
          if (p.accumulate) {
            const uint4 old = *reinterpret_cast<const uint4*>(dst + j);
            const uint32_t ow[4] = {old.x, old.y, old.z, old.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              if (p.c_is_bf16 == 2) {
                const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&ow[e]));
                v[2 * e] += f.x;
                v[2 * e + 1] += f.y;
              } else {
                v[2 * e] += __uint_as_float(ow[e] << 16);
                v[2 * e + 1] += __uint_as_float(ow[e] & 0xFFFF0000u);
              }
            }
          }
          uint32_t w[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            if (p.c_is_bf16 == 2) {
              __half2 t2 = __floats2half2_rn(v[2 * e], v[2 * e + 1]);
              w[e] = *reinterpret_cast<uint32_t*>(&t2);
            } else {
              __nv_bfloat162 t2 = __floats2bfloat162_rn(v[2 * e], v[2 * e + 1]);
              w[e] = *reinterpret_cast<uint32_t*>(&t2);
            }
          }
          *reinterpret_cast<uint4*>(dst + j) = make_uint4(w[0], w[1], w[2], w[3]);
        }
      } else {
        for (int j = 0; j < 32 && nb + j < p.N; ++j) {
          float v = __uint_as_float(r[j]);
          if (p.c_is_bf16 == 2) {
            __half* hd = reinterpret_cast<__half*>(dst);
            if (p.accumulate) v += __half2float(hd[j]);
            hd[j] = __float2half_rn(v);
          } else {
            if (p.accumulate) v += __bfloat162float(dst[j]);
            dst[j] = __float2bfloat16_rn(v);
          }
        }
      }
    } else {
      float* dst = reinterpret_cast<float*>(p.c) + (long long)m * p.ldc + nb;
      if (nb + 32 <= p.N && (p.ldc & 3) == 0 &&
          (reinterpret_cast<uintptr_t>(p.c) & 15) == 0) {
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          float4 o = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]),
                                 __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
          if (p.accumulate) {
            const float4 c0 = *reinterpret_cast<const float4*>(dst + j);
            o.x += c0.x; o.y += c0.y; o.z += c0.z; o.w += c0.w;
          }
          *reinterpret_cast<float4*>(dst + j) = o;
        }
      } else {
        for (int j = 0; j < 32 && nb + j < p.N; ++j) {
          float v = __uint_as_float(r[j]);
          if (p.accumulate) v += dst[j];
          dst[j] = v;
        }
      }
    }
  }
}

template <int NPROD>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a,
                    const __grid_constant__ CUtensorMap map_b, const Params p) {
  using C = Cfg<NPROD>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* aligned = smem_raw + (base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(aligned + C::STAGES * C::STAGE_BYTES);
  // barrier slots: full[STAGES], empty[STAGES], acc_full[NACC], acc_empty[NACC]
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (C::STAGES + s); };
  auto accf_bar = [&](int a) { return bar0 + 8u * (2 * C::STAGES + a); };
  auto acce_bar = [&](int a) { return bar0 + 8u * (2 * C::STAGES + NACC + a); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * C::STAGES + 2 * NACC);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < NACC; ++a) {
      mbar_init(accf_bar(a), 1);
      mbar_init(acce_bar(a), 128);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_slot)),
                 "r"((uint32_t)TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int total_items = p.tiles_m * p.tiles_n * p.splits;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
        const int tn = item % p.tiles_n;
        const int tm = (item / p.tiles_n) % p.tiles_m;
        const int sp = item / (p.tiles_n * p.tiles_m);
        const int kb0 = sp * p.kb_per_split;
        const int kb1 = min(p.kb_total, kb0 + p.kb_per_split);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.err, 1)) { ok = false; break; }
          mbar_expect_tx(full_bar(stage), C::STAGE_BYTES);
          const uint32_t sa = base + stage * C::STAGE_BYTES;
          const uint32_t sb = sa + C::PLANES * TILE_BYTES;
          const int k0 = kb * BK, m0 = tm * BM, n0 = tn * BN;
#pragma unroll
          for (int pl = 0; pl < C::PLANES; ++pl) {
            const CUtensorMap* ma = &map_a;
            const CUtensorMap* mb = &map_b;
            const uint32_t da = sa + pl * TILE_BYTES, db = sb + pl * TILE_BYTES;
            if (p.a_mn_major) {  // two boxes of 64 (m) x 64 (k)
              tma_load_3d(da, ma, full_bar(stage), m0, k0, pl);
              tma_load_3d(da + TILE_BYTES / 2, ma, full_bar(stage), m0 + 64, k0, pl);
            } else {             // one box of 64 (k) x 128 (m)
              tma_load_3d(da, ma, full_bar(stage), k0, m0, pl);
            }
            if (p.b_mn_major) {
              tma_load_3d(db, mb, full_bar(stage), n0, k0, pl);
              tma_load_3d(db + TILE_BYTES / 2, mb, full_bar(stage), n0 + 64, k0, pl);
            } else {
              tma_load_3d(db, mb, full_bar(stage), k0, n0, pl);
            }
          }
          if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) |
                             ((uint32_t)p.a_mn_major << 15) | ((uint32_t)p.b_mn_major << 16) |
                             ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
      // K-major: 8-row groups 1024 B apart, a K step of 16 elements is 32 B along the row.
      // MN-major: 8-k-row groups 1024 B apart, 64-element MN chunks one box (8192 B) apart,
      //           a K step of 16 rows is 2048 B.
      const uint32_t a_lbo = p.a_mn_major ? TILE_BYTES / 2 : 16, a_kstep = p.a_mn_major ? 2048 : 32;
      const uint32_t b_lbo = p.b_mn_major ? TILE_BYTES / 2 : 16, b_kstep = p.b_mn_major ? 2048 : 32;
      uint32_t stage = 0, phase = 0;
      uint32_t acc_phase = 0;  // one parity bit per accumulator
      int cidx = 0;  // accumulator hand-overs so far: they alternate between the two buffers
      bool ok = true;
      for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
        const int sp = item / (p.tiles_n * p.tiles_m);
        const int kb0 = sp * p.kb_per_split;
        const int kb1 = min(p.kb_total, kb0 + p.kb_per_split);
        int kb = kb0;
        while (kb < kb1 && ok) {
          const int acc = cidx % NACC;
          ++cidx;
          if (!mbar_wait(acce_bar(acc), ((acc_phase >> acc) & 1u) ^ 1u, abort_flag, p.err, 2)) { ok = false; break; }
          acc_phase ^= 1u << acc;
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + acc * BN;
          const int kend = C::CHUNK ? min(kb1, kb + C::CHUNK) : kb1;
          uint32_t first = 1;
          for (; kb < kend; ++kb) {
            if (!mbar_wait(full_bar(stage), phase, abort_flag, p.err, 3)) { ok = false; break; }
            tc_fence_after();
            const uint32_t sa = base + stage * C::STAGE_BYTES;
            const uint32_t sb = sa + C::PLANES * TILE_BYTES;
#pragma unroll
            for (int pr = 0; pr < NPROD; ++pr) {
              // plane pairs, most significant first:
              //   (0,0) (0,1) (1,0) | (1,1) (0,2) (2,0)      0 = hi, 1 = mid/lo, 2 = lo
              const int ia = pr == 2 ? 1 : (pr == 3 ? 1 : (pr == 5 ? 2 : 0));
              const int ib = pr == 1 ? 1 : (pr == 3 ? 1 : (pr == 4 ? 2 : 0));
              const uint32_t pa = sa + ia * TILE_BYTES;
              const uint32_t pb = sb + ib * TILE_BYTES;
#pragma unroll
              for (int ks = 0; ks < BK / UK; ++ks) {
                const uint64_t da = smem_desc(pa + ks * a_kstep, a_lbo, 1024);
                const uint64_t db = smem_desc(pb + ks * b_kstep, b_lbo, 1024);
                tc_mma_bf16(d_tmem, da, db, idesc, first ? 0u : 1u);
                first = 0;
              }
            }
            tc_commit(empty_bar(stage));  // frees the stage once these MMAs have read it
            if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
          }
          if (ok) tc_commit(accf_bar(acc));  // this chunk of the accumulation is complete
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    const int quad = warp & 3;  // tensor-memory lane quadrant this warp may read
    uint32_t acc_phase = 0;  // one parity bit per accumulator
    int cidx = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < total_items; item += gridDim.x) {
      const int tn = item % p.tiles_n;
      const int tm = (item / p.tiles_n) % p.tiles_m;
      const int sp = item / (p.tiles_n * p.tiles_m);
      const int kb0 = sp * p.kb_per_split;
      const int kb1 = min(p.kb_total, kb0 + p.kb_per_split);
      const int nchunks = C::CHUNK ? (kb1 - kb0 + C::CHUNK - 1) / C::CHUNK : 1;
      const int m = tm * BM + quad * 32 + lane;
      const int n0 = tn * BN;
      // running sums of this thread's row of the tile (only with chunked hand-over)
      float sum[C::CHUNK ? BN : 1];
#pragma unroll
      for (int j = 0; j < (C::CHUNK ? BN : 1); ++j) sum[j] = 0.f;
      for (int c = 0; c < nchunks; ++c) {
        const int acc = cidx % NACC;
        ++cidx;
        if (ok) ok = mbar_wait(accf_bar(acc), (acc_phase >> acc) & 1u, abort_flag, p.err, 4);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        acc_phase ^= 1u << acc;
        tc_fence_after();
        const uint32_t taddr = tmem_base + acc * BN + ((uint32_t)(quad * 32) << 16);
        if (C::CHUNK) {
#pragma unroll
          for (int ch = 0; ch < BN / 32; ++ch) {
            uint32_t r[32];
            tc_ld32(taddr + ch * 32, r);
            tc_wait_ld();
#pragma unroll
            for (int j = 0; j < 32; ++j) sum[(C::CHUNK ? ch * 32 : 0) + j] += __uint_as_float(r[j]);
          }
        } else {
#pragma unroll 1
          for (int ch = 0; ch < BN / 32; ++ch) {
            uint32_t r[32];
            tc_ld32(taddr + ch * 32, r);
            tc_wait_ld();
            store_chunk(p, sp, m, n0 + ch * 32, r);
          }
        }
        tc_fence_before();
        mbar_arrive(acce_bar(acc));
      }
      if (!ok) break;
      if (C::CHUNK) {
#pragma unroll
        for (int ch = 0; ch < BN / 32; ++ch) {
          uint32_t r[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(sum[(C::CHUNK ? ch * 32 : 0) + j]);
          store_chunk(p, sp, m, n0 + ch * 32, r);
        }
      }
    }
  }

  // Drain: every role arrives here, also after a time-out, so tensor memory is released.
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"((uint32_t)TMEM_COLS)
                 : "memory");
  }
}

// ---- the same contraction on CTA pairs ------------------------------------------------------
// The single-CTA kernel above runs at (shared-memory ring bytes) / (load latency): a 128 x 128
// tile needs 32 KB of operands per 64-wide k-block and product, about twice what the ring can
// have in flight per unit of tensor-pipe time.  Here two CTAs of a cluster share a 256 x 256
// tile (tcgen05.mma.cta_group::2, M = 256): each CTA loads its own 128 rows of A and its own
// 128-column half of B - the same two 16 KB boxes per plane as above - and the tensor cores of
// both SMs read both halves of B, so every loaded byte feeds twice the arithmetic.  Each CTA's
// tensor memory holds its 128 rows x 256 columns of the accumulator (two accumulators of 256
// columns).  CTA 0 of the pair issues all MMAs; its full barriers count the bytes of both
// CTAs' loads (the loads name the barrier through cta_group::2; every CTA fetches its own
// tiles), its commits arrive on the empty and accumulator-full barriers of both CTAs, and both
// CTAs' epilogue warps (eight per CTA: four lane quadrants x two column halves) arrive on its
// accumulator-empty barriers.
constexpr int PAIR_THREADS = 320;        // warp 0 TMA, warp 1 MMA / tensor memory, warps 2..9 epilogue
constexpr int PBN = 256;                 // columns of the pair's tile and of one accumulator
constexpr int PBM = 256;                 // rows of the pair's tile (128 per CTA)
constexpr int PAIR_NACC = 2;
constexpr int PAIR_EPI_WARPS = 8;

// (Ten warps put three on two of the SM's four sub-partitions, 16384 registers each, so 168
// registers per thread is the most a 320-thread CTA can have; the epilogue therefore drains the
// accumulator 16 columns at a time.)
template <int NPROD>
__global__ void __launch_bounds__(PAIR_THREADS, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_a,
                         const __grid_constant__ CUtensorMap map_b, const Params p) {
  using C = Cfg<NPROD>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* aligned = smem_raw + (base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(aligned + C::STAGES * C::STAGE_BYTES);
  // barrier slots: full[STAGES], empty[STAGES], acc_full[2], acc_empty[2]
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (C::STAGES + s); };
  auto accf_bar = [&](int a) { return bar0 + 8u * (2 * C::STAGES + a); };
  auto acce_bar = [&](int a) { return bar0 + 8u * (2 * C::STAGES + PAIR_NACC + a); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * C::STAGES + 2 * PAIR_NACC);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 issues the MMAs
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(full_bar(s), 1);   // CTA 0's producer; the bytes of both CTAs' loads
      mbar_init(empty_bar(s), 1);  // one commit
    }
    for (int a = 0; a < PAIR_NACC; ++a) {
      mbar_init(accf_bar(a), 1);
      mbar_init(acce_bar(a), 2 * PAIR_EPI_WARPS);  // one arrival per epilogue warp of both CTAs
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    // collective over the pair: the same warp of both CTAs, the same shared-memory slot
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_slot)),
                 "r"((uint32_t)(PAIR_NACC * PBN))
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers are initialised before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int total_items = p.tiles_m * p.tiles_n * p.splits;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int item = pair; item < total_items && ok; item += npairs) {
        const int tn = item % p.tiles_n;
        const int tm = (item / p.tiles_n) % p.tiles_m;
        const int sp = item / (p.tiles_n * p.tiles_m);
        const int kb0 = sp * p.kb_per_split;
        const int kb1 = min(p.kb_total, kb0 + p.kb_per_split);
        const int m0 = tm * PBM + (int)rank * BM, n0 = tn * PBN + (int)rank * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.err, 11)) { ok = false; break; }
          if (rank == 0) mbar_expect_tx(full_bar(stage), 2 * C::STAGE_BYTES);
          const uint32_t fb = mapa_u32(full_bar(stage), 0);
          const uint32_t sa = base + stage * C::STAGE_BYTES;
          const uint32_t sb = sa + C::PLANES * TILE_BYTES;
          const int k0 = kb * BK;
#pragma unroll
          for (int pl = 0; pl < C::PLANES; ++pl) {
            const uint32_t da = sa + pl * TILE_BYTES, db = sb + pl * TILE_BYTES;
            if (p.a_mn_major) {  // two boxes of 64 (m) x 64 (k)
              tma_load_3d_pair(da, &map_a, fb, m0, k0, pl);
              tma_load_3d_pair(da + TILE_BYTES / 2, &map_a, fb, m0 + 64, k0, pl);
            } else {             // one box of 64 (k) x 128 (m)
              tma_load_3d_pair(da, &map_a, fb, k0, m0, pl);
            }
            if (p.b_mn_major) {
              tma_load_3d_pair(db, &map_b, fb, n0, k0, pl);
              tma_load_3d_pair(db + TILE_BYTES / 2, &map_b, fb, n0 + 64, k0, pl);
            } else {
              tma_load_3d_pair(db, &map_b, fb, k0, n0, pl);
            }
          }
          if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (CTA 0 only)
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) |
                             ((uint32_t)p.a_mn_major << 15) | ((uint32_t)p.b_mn_major << 16) |
                             ((uint32_t)(PBN >> 3) << 17) | ((uint32_t)(PBM >> 4) << 24);
      const uint32_t a_lbo = p.a_mn_major ? TILE_BYTES / 2 : 16, a_kstep = p.a_mn_major ? 2048 : 32;
      const uint32_t b_lbo = p.b_mn_major ? TILE_BYTES / 2 : 16, b_kstep = p.b_mn_major ? 2048 : 32;
      uint32_t stage = 0, phase = 0;
      uint32_t acc_phase = 0;  // one parity bit per accumulator
      int cidx = 0;
      bool ok = true;
      for (int item = pair; item < total_items && ok; item += npairs) {
        const int sp = item / (p.tiles_n * p.tiles_m);
        const int kb0 = sp * p.kb_per_split;
        const int kb1 = min(p.kb_total, kb0 + p.kb_per_split);
        int kb = kb0;
        while (kb < kb1 && ok) {
          const int acc = cidx % PAIR_NACC;
          ++cidx;
          if (!mbar_wait_cluster(acce_bar(acc), ((acc_phase >> acc) & 1u) ^ 1u, abort_flag, p.err, 12)) { ok = false; break; }
          acc_phase ^= 1u << acc;
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + acc * PBN;
          const int kend = C::CHUNK ? min(kb1, kb + C::CHUNK) : kb1;
          uint32_t first = 1;
          for (; kb < kend; ++kb) {
            if (!mbar_wait_cluster(full_bar(stage), phase, abort_flag, p.err, 13)) { ok = false; break; }
            tc_fence_after();
            const uint32_t sa = base + stage * C::STAGE_BYTES;
            const uint32_t sb = sa + C::PLANES * TILE_BYTES;
#pragma unroll
            for (int pr = 0; pr < NPROD; ++pr) {
              const int ia = pr == 2 ? 1 : (pr == 3 ? 1 : (pr == 5 ? 2 : 0));
              const int ib = pr == 1 ? 1 : (pr == 3 ? 1 : (pr == 4 ? 2 : 0));
              const uint32_t pa = sa + ia * TILE_BYTES;
              const uint32_t pb = sb + ib * TILE_BYTES;
#pragma unroll
              for (int ks = 0; ks < BK / UK; ++ks) {
                const uint64_t da = smem_desc(pa + ks * a_kstep, a_lbo, 1024);
                const uint64_t db = smem_desc(pb + ks * b_kstep, b_lbo, 1024);
                tc_mma_bf16_pair(d_tmem, da, db, idesc, first ? 0u : 1u);
                first = 0;
              }
            }
            tc_commit_pair(empty_bar(stage), 3);  // frees the stage in both CTAs
            if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
          }
          if (ok) tc_commit_pair(accf_bar(acc), 3);  // this chunk is complete in both CTAs
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (both CTAs)
    const int quad = warp & 3;         // tensor-memory lane quadrant this warp may read
    const int half = (warp - 2) >> 2;  // which 128 columns of the accumulator
    uint32_t acc_phase = 0;  // one parity bit per accumulator
    int cidx = 0;
    bool ok = true;
    for (int item = pair; item < total_items; item += npairs) {
      const int tn = item % p.tiles_n;
      const int tm = (item / p.tiles_n) % p.tiles_m;
      const int sp = item / (p.tiles_n * p.tiles_m);
      const int kb0 = sp * p.kb_per_split;
      const int kb1 = min(p.kb_total, kb0 + p.kb_per_split);
      const int nchunks = C::CHUNK ? (kb1 - kb0 + C::CHUNK - 1) / C::CHUNK : 1;
      const int m = tm * PBM + (int)rank * BM + quad * 32 + lane;
      const int n0 = tn * PBN + half * BN;
      float sum[C::CHUNK ? BN : 1];
#pragma unroll
      for (int j = 0; j < (C::CHUNK ? BN : 1); ++j) sum[j] = 0.f;
      for (int c = 0; c < nchunks; ++c) {
        const int acc = cidx % PAIR_NACC;
        ++cidx;
        if (ok) ok = mbar_wait(accf_bar(acc), (acc_phase >> acc) & 1u, abort_flag, p.err, 14);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        acc_phase ^= 1u << acc;
        tc_fence_after();
        const uint32_t taddr = tmem_base + acc * PBN + half * BN + ((uint32_t)(quad * 32) << 16);
        if (C::CHUNK) {
#pragma unroll
          for (int ch = 0; ch < BN / 16; ++ch) {
            uint32_t r[16];
            tc_ld16(taddr + ch * 16, r);
            tc_wait_ld();
#pragma unroll
            for (int j = 0; j < 16; ++j) sum[(C::CHUNK ? ch * 16 : 0) + j] += __uint_as_float(r[j]);
          }
        } else {
#pragma unroll 1
          for (int ch = 0; ch < BN / 32; ++ch) {
            uint32_t r[32];
            tc_ld32(taddr + ch * 32, r);
            tc_wait_ld();
            store_chunk(p, sp, m, n0 + ch * 32, r);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(mapa_u32(acce_bar(acc), 0));
      }
      if (!ok) break;
      if (C::CHUNK) {
#pragma unroll
        for (int ch = 0; ch < BN / 32; ++ch) {
          uint32_t r[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(sum[(C::CHUNK ? ch * 32 : 0) + j]);
          store_chunk(p, sp, m, n0 + ch * 32, r);
        }
      }
    }
  }

  // Drain: every role of both CTAs arrives here, also after a time-out.  Neither CTA may leave
  // while the other's MMAs can still read its shared memory or signal its barriers.
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"((uint32_t)(PAIR_NACC * PBN))
                 : "memory");
  }
}

// x -> `planes` bf16 planes (x = p0 + p1 (+ p2), each the bf16 rounding of what is left),
// same orientation as the source, leading dimension ld_dst (a multiple of 8), planes
// `plane_stride` elements apart.  One thread converts 4 consecutive elements of a row:
// a 16-byte load and one 8-byte store per plane when the source allows it.
template <int PLANES, typename TS>
__global__ void split_planes_kernel(const TS* __restrict__ src, long long ld_src, int rows,
                                    int cols, __nv_bfloat16* __restrict__ dst, long long ld_dst,
                                    long long plane_stride, int vec_ok) {
  const int quads = (int)(ld_dst / 4);
  const long long total = (long long)rows * quads;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / quads;
    const int c = (int)(i - r * quads) * 4;
    float x[4] = {0.f, 0.f, 0.f, 0.f};
    const TS* sp = src + r * ld_src + c;
    if (vec_ok && c + 3 < cols) {
      if constexpr (sizeof(TS) == 4) {
        const float4 f = *reinterpret_cast<const float4*>(sp);
        x[0] = f.x; x[1] = f.y; x[2] = f.z; x[3] = f.w;
      } else {
        const uint2 u = *reinterpret_cast<const uint2*>(sp);
        const __half2 h0 = *reinterpret_cast<const __half2*>(&u.x);
        const __half2 h1 = *reinterpret_cast<const __half2*>(&u.y);
        x[0] = __low2float(h0); x[1] = __high2float(h0);
        x[2] = __low2float(h1); x[3] = __high2float(h1);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (c + j < cols) x[j] = ld(sp + j);
    }
    __nv_bfloat16* dp = dst + r * ld_dst + c;
#pragma unroll
    for (int pl = 0; pl < PLANES; ++pl) {
      __nv_bfloat162 a = __floats2bfloat162_rn(x[0], x[1]);
      __nv_bfloat162 b = __floats2bfloat162_rn(x[2], x[3]);
      uint2 w;
      w.x = *reinterpret_cast<uint32_t*>(&a);
      w.y = *reinterpret_cast<uint32_t*>(&b);
      *reinterpret_cast<uint2*>(dp + pl * plane_stride) = w;
      x[0] -= __low2float(a); x[1] -= __high2float(a);
      x[2] -= __low2float(b); x[3] -= __high2float(b);
    }
  }
}

// `half_src`: the source is __half (its 11 significant bits split exactly into two planes).
int launch_split(const void* src, bool half_src, long long ld_src, int rows, int cols,
                 __nv_bfloat16* dst, long long ld_dst, long long plane_stride, int planes,
                 int blocks, cudaStream_t stream) {
  const int vec_ok = ((ld_src & 3) == 0) &&
                     ((reinterpret_cast<uintptr_t>(src) & (half_src ? 7 : 15)) == 0);
  if (half_src) {
    const __half* hs = static_cast<const __half*>(src);
    if (planes == 3)
      split_planes_kernel<3, __half><<<blocks, 256, 0, stream>>>(hs, ld_src, rows, cols, dst, ld_dst,
                                                                 plane_stride, vec_ok);
    else
      split_planes_kernel<2, __half><<<blocks, 256, 0, stream>>>(hs, ld_src, rows, cols, dst, ld_dst,
                                                                 plane_stride, vec_ok);
  } else if (planes == 3)
    split_planes_kernel<3, float><<<blocks, 256, 0, stream>>>(static_cast<const float*>(src), ld_src,
                                                              rows, cols, dst, ld_dst, plane_stride,
                                                              vec_ok);
  else
    split_planes_kernel<2, float><<<blocks, 256, 0, stream>>>(static_cast<const float*>(src), ld_src,
                                                              rows, cols, dst, ld_dst, plane_stride,
                                                              vec_ok);
  HB_LAUNCH_OK();
  count_launch(1);
  return HASTE_B200_OK;
}

template <typename TC>
__global__ void splitk_reduce_kernel(const float* __restrict__ part, int splits, long long MN,
                                     int N, TC* __restrict__ c, long long ldc, int accumulate) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < MN;
       i += (long long)gridDim.x * blockDim.x) {
    float s = 0.f;
    for (int k = 0; k < splits; ++k) s += part[k * MN + i];
    const long long m = i / N;
    TC* dst = c + m * ldc + (i - m * N);
    if (accumulate) s += ld(dst);
    st(dst, s);
  }
}

// ----------------------------------------------------------------------------
// Host side
// ----------------------------------------------------------------------------
struct Operand {
  bool mn_major;          // contiguous along M (A) or N (B)
  long long ld;           // elements between consecutive outer indices
  long long plane_stride; // elements between planes
  const void* base;
};

// The opt-in to more than 48 KB of dynamic shared memory is a per-device (per-context)
// function attribute: one flag per device ordinal, so that a process driving several GPUs
// opts in on each of them.
constexpr int kMaxDevices = 64;
std::atomic<bool> g_attr_set[kMaxDevices];
std::atomic<int> g_max_pairs[kMaxDevices];  // 0: not asked yet, -1: no clusters, else the count

int set_kernel_attributes() {
  int dev = 0;
  HB_CUDA_OK(cudaGetDevice(&dev));
  if (dev >= 0 && dev < kMaxDevices && g_attr_set[dev].load(std::memory_order_acquire))
    return HASTE_B200_OK;
  const auto attr = cudaFuncAttributeMaxDynamicSharedMemorySize;
  HB_CUDA_OK(cudaFuncSetAttribute(gemm_tcgen05_kernel<1>, attr, Cfg<1>::SMEM));
  HB_CUDA_OK(cudaFuncSetAttribute(gemm_tcgen05_kernel<3>, attr, Cfg<3>::SMEM));
  HB_CUDA_OK(cudaFuncSetAttribute(gemm_tcgen05_kernel<6>, attr, Cfg<6>::SMEM));
  HB_CUDA_OK(cudaFuncSetAttribute(gemm_tcgen05_pair_kernel<1>, attr, Cfg<1>::SMEM));
  HB_CUDA_OK(cudaFuncSetAttribute(gemm_tcgen05_pair_kernel<3>, attr, Cfg<3>::SMEM));
  HB_CUDA_OK(cudaFuncSetAttribute(gemm_tcgen05_pair_kernel<6>, attr, Cfg<6>::SMEM));
  if (dev >= 0 && dev < kMaxDevices) g_attr_set[dev].store(true, std::memory_order_release);
  return HASTE_B200_OK;
}

// How many clusters of two CTAs of the pair kernel the device holds at once (its persistent
// grid); 0 when cluster launch is not available.
int max_pairs() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 0;
  int n = g_max_pairs[dev].load(std::memory_order_acquire);
  if (n == 0) {
    n = -1;
    if (set_kernel_attributes() == HASTE_B200_OK) {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(2 * sm_count());
      cfg.blockDim = dim3(PAIR_THREADS);
      cfg.dynamicSmemBytes = Cfg<6>::SMEM;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = 2;
      attr[0].val.clusterDim.y = 1;
      attr[0].val.clusterDim.z = 1;
      cfg.attrs = attr;
      cfg.numAttrs = 1;
      int clusters = 0;
      if (cudaOccupancyMaxActiveClusters(&clusters, gemm_tcgen05_pair_kernel<6>, &cfg) ==
              cudaSuccess && clusters > 0)
        n = min(clusters, sm_count() / 2);
      cudaGetLastError();
    }
    g_max_pairs[dev].store(n, std::memory_order_release);
  }
  return n > 0 ? n : 0;
}

}  // namespace

// fp32 [rows, cols] (leading dimension ld_src) -> two bf16 planes of leading dimension ld_dst,
// plane_stride elements apart: the form GemmDesc::a_pl / b_pl takes, for an operand that
// several contractions read.
int gemm_split_planes(const float* src, long long ld_src, int rows, int cols,
                      __nv_bfloat16* dst, long long ld_dst, long long plane_stride,
                      cudaStream_t stream) {
  return launch_split(src, false, ld_src, rows, cols, dst, ld_dst, plane_stride, 2,
                      8 * sm_count(), stream);
}

int gemm_sm100(const GemmDesc& g, cudaStream_t stream) {
  auto unsupported = [](const char* why) {
    set_last_error("gemm_sm100: %s", why);
    return HASTE_B200_ERR_UNSUPPORTED;
  };
  if (!encode_fn()) return unsupported("cuTensorMapEncodeTiled not available");
  if (g.M <= 0 || g.N <= 0) return HASTE_B200_OK;
  if (g.K <= 0) return unsupported("K == 0");
  // Small problems are launch-bound either way; keep them on the generic kernel.
  if ((long long)g.M * g.N * g.K < (1LL << 21) || g.M < 32 || g.N < 32)
    return unsupported("problem too small for the tensor-core path");
  // __half storage takes the split path too: a half splits exactly into two bf16 planes
  const bool half_src = g.dtype == HASTE_B200_F16;
  const bool f32 = g.dtype == HASTE_B200_F32 || half_src;
  const bool a_k = g.a_cs == 1, a_m = g.a_rs == 1 && !a_k;
  const bool b_k = g.b_rs == 1, b_n = g.b_cs == 1 && !b_k;
  if (!(a_k || a_m) || !(b_k || b_n)) return unsupported("operand has no unit stride");

  const int M = g.M, N = g.N, K = g.K;
  Operand A, B;
  A.mn_major = !a_k;
  B.mn_major = !b_k;
  // extents in (outer rows, inner contiguous) form
  const long long a_rows = a_k ? M : K, a_cols = a_k ? K : M;
  const long long b_rows = b_k ? N : K, b_cols = b_k ? K : N;
  const long long a_ld_src = a_k ? g.a_rs : g.a_cs;
  const long long b_ld_src = b_k ? g.b_cs : g.b_rs;

  // scratch: planes for fp32 operands, partial tiles for split-K
  const int sms = sm_count();
  // CTA pairs on 256 x 256 tiles where the output is wide enough to fill them
  const int pairs = (gemm_path() == HASTE_B200_GEMM_TCGEN05_SINGLE || M < 192 || N < 192)
                        ? 0 : max_pairs();
  const bool pair = pairs > 0;
  const int units = pair ? pairs : sms;
  const int tiles_m = ceil_div(M, pair ? PBM : BM), tiles_n = ceil_div(N, pair ? PBN : BN);
  const int kb_total = ceil_div(K, BK);
  int splits = 1;
  if (tiles_m * tiles_n < units && kb_total >= 8) {
    // Split K so that the work items fill whole waves of the persistent grid: pick the split
    // count with the smallest estimated time = (waves / splits) x K blocks x time per K block
    // + the traffic of the partial tiles (written once, read once by the reduction).
    const int tiles = tiles_m * tiles_n;
    const int max_splits = min(kb_total / 4, 64);
    const double products = g.dtype == HASTE_B200_BF16 ? 1.0 : (g.precise ? 6.0 : 3.0);
    // us per K block and work unit (measured: the single-CTA kernel is bound by its operand
    // loads, the pair kernel by the tensor pipe)
    const double t_kb = pair ? 0.27 * products : (products == 1.0 ? 0.27 : 0.17 * products);
    const double t_part = 2.0 * (double)M * N * 4.0 / 6.0e6;          // us per split (HBM)
    double best = 1e30;
    for (int sp = 1; sp <= max_splits; ++sp) {
      const int per = ceil_div(kb_total, sp);
      const int real = ceil_div(kb_total, per);
      if (real != sp) continue;  // the same blocks per split as a smaller count: skip
      const double t = (double)ceil_div(tiles * sp, units) * per * t_kb + (sp > 1 ? sp * t_part : 0.0);
      if (t < best) { best = t; splits = sp; }
    }
  }
  int kb_per_split = ceil_div(kb_total, splits);
  splits = ceil_div(kb_total, kb_per_split);

  auto planes_usable = [&](const void* p, long long ld) {
    return f32 && !g.precise && p && (ld % 8) == 0 && (reinterpret_cast<uintptr_t>(p) & 15) == 0;
  };
  const bool a_pre = planes_usable(g.a_pl, g.a_pl_ld) && (g.a_pl_stride % 8) == 0;
  const bool b_pre = planes_usable(g.b_pl, g.b_pl_ld) && (g.b_pl_stride % 8) == 0;
  const long long a_ld = a_pre ? g.a_pl_ld : (f32 ? ((a_cols + 7) & ~7LL) : a_ld_src);
  const long long b_ld = b_pre ? g.b_pl_ld : (f32 ? ((b_cols + 7) & ~7LL) : b_ld_src);
  if (!f32) {
    if ((a_ld % 8) || (b_ld % 8) || ((uintptr_t)g.a & 15) || ((uintptr_t)g.b & 15))
      return unsupported("bf16 operand not 16-byte aligned for TMA");
  }
  const int planes = f32 ? (g.precise ? 3 : 2) : 1;
  const size_t a_plane = (f32 && !a_pre) ? Arena::pad((size_t)a_rows * a_ld * 2) : 0;
  const size_t b_plane = (f32 && !b_pre) ? Arena::pad((size_t)b_rows * b_ld * 2) : 0;
  const size_t part_bytes = splits > 1 ? Arena::pad((size_t)splits * M * N * 4) : 0;
  const size_t bytes = planes * (a_plane + b_plane) + part_bytes + 1024;
  Arena ws;
  HB_TRY(make_arena(&ws, stream, bytes, /*slot=*/1));
  int* err = device_error_word();
  if (!err) return unsupported("error word allocation failed");
  if (f32) {
    __nv_bfloat16* ap = ws.take<__nv_bfloat16>(planes * a_plane / 2);
    __nv_bfloat16* bp = ws.take<__nv_bfloat16>(planes * b_plane / 2);
    if (!ap || !bp) return unsupported("scratch arena");
    const int blocks = 8 * sms;
    if (!a_pre)
      HB_TRY(launch_split(g.a, half_src, a_ld_src, (int)a_rows, (int)a_cols, ap, a_ld,
                          a_plane / 2, planes, blocks, stream));
    if (!b_pre)
      HB_TRY(launch_split(g.b, half_src, b_ld_src, (int)b_rows, (int)b_cols, bp, b_ld,
                          b_plane / 2, planes, blocks, stream));
    A.base = ap; A.plane_stride = a_plane / 2;
    B.base = bp; B.plane_stride = b_plane / 2;
    if (a_pre) { A.base = g.a_pl; A.plane_stride = g.a_pl_stride; }
    if (b_pre) { B.base = g.b_pl; B.plane_stride = g.b_pl_stride; }
  } else {
    A.base = g.a; A.plane_stride = 0;
    B.base = g.b; B.plane_stride = 0;
  }
  A.ld = a_ld;
  B.ld = b_ld;
  float* partial = nullptr;
  if (splits > 1) {
    partial = ws.take<float>(part_bytes / 4);
    if (!partial) return unsupported("scratch arena");
  }

  CUtensorMap m_a, m_b;
  bool ok = true;
  // K-major: inner = K, box 64 (k) x 128 rows.  MN-major: inner = M/N, box 64 x 64 (k).
  ok &= make_map(&m_a, A.base, a_cols, a_rows, A.ld, A.plane_stride, planes, 64,
                 A.mn_major ? 64 : BM);
  ok &= make_map(&m_b, B.base, b_cols, b_rows, B.ld, B.plane_stride, planes, 64,
                 B.mn_major ? 64 : BN);
  if (!ok) return unsupported("tensor map encoding rejected the operand");

  Params p;
  p.M = M; p.N = N; p.K = K;
  p.a_mn_major = A.mn_major; p.b_mn_major = B.mn_major;
  p.tiles_m = tiles_m; p.tiles_n = tiles_n; p.splits = splits;
  p.kb_per_split = kb_per_split; p.kb_total = kb_total;
  p.c_is_bf16 = g.dtype_c == HASTE_B200_BF16 ? 1 : (g.dtype_c == HASTE_B200_F16 ? 2 : 0);
  p.accumulate = g.accumulate;
  p.c = g.c; p.ldc = g.ldc;
  p.partial = partial;
  p.err = err;

  HB_TRY(set_kernel_attributes());
  if (pair) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * min(pairs, tiles_m * tiles_n * splits));
    cfg.blockDim = dim3(PAIR_THREADS);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (planes == 3) {
      cfg.dynamicSmemBytes = Cfg<6>::SMEM;
      HB_CUDA_OK(cudaLaunchKernelEx(&cfg, gemm_tcgen05_pair_kernel<6>, m_a, m_b, p));
    } else if (planes == 2) {
      cfg.dynamicSmemBytes = Cfg<3>::SMEM;
      HB_CUDA_OK(cudaLaunchKernelEx(&cfg, gemm_tcgen05_pair_kernel<3>, m_a, m_b, p));
    } else {
      cfg.dynamicSmemBytes = Cfg<1>::SMEM;
      HB_CUDA_OK(cudaLaunchKernelEx(&cfg, gemm_tcgen05_pair_kernel<1>, m_a, m_b, p));
    }
  } else {
    const int grid = min(sms, tiles_m * tiles_n * splits);
    if (planes == 3)
      gemm_tcgen05_kernel<6><<<grid, THREADS, Cfg<6>::SMEM, stream>>>(m_a, m_b, p);
    else if (planes == 2)
      gemm_tcgen05_kernel<3><<<grid, THREADS, Cfg<3>::SMEM, stream>>>(m_a, m_b, p);
    else
      gemm_tcgen05_kernel<1><<<grid, THREADS, Cfg<1>::SMEM, stream>>>(m_a, m_b, p);
  }
  HB_LAUNCH_OK();
  count_launch(1);
  if (splits > 1) {
    const long long MN = (long long)M * N;
    const int blocks = min(ceil_div(MN, 256), 8 * sms);
    if (g.dtype_c == HASTE_B200_BF16)
      splitk_reduce_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(
          partial, splits, MN, N, (__nv_bfloat16*)g.c, g.ldc, g.accumulate);
    else if (g.dtype_c == HASTE_B200_F16)
      splitk_reduce_kernel<__half><<<blocks, 256, 0, stream>>>(partial, splits, MN, N,
                                                                (__half*)g.c, g.ldc, g.accumulate);
    else
      splitk_reduce_kernel<float><<<blocks, 256, 0, stream>>>(partial, splits, MN, N, (float*)g.c,
                                                              g.ldc, g.accumulate);
    HB_LAUNCH_OK();
    count_launch(1);
  }
  return HASTE_B200_OK;
}

}  // namespace hb
