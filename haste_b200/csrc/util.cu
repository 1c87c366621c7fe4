#include "util.cuh"

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <map>
#include <mutex>
#include <tuple>
#include <utility>
#include <vector>

namespace hb {

// ---------------------------------------------------------------------------
// Error text (thread-local) and launch counter.
// ---------------------------------------------------------------------------
static thread_local char g_err[512] = "";

void set_last_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}
const char* last_error() { return g_err; }

static std::atomic<long long> g_launches{0};
void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
long long launch_count() { return g_launches.load(std::memory_order_relaxed); }

int sm_count() {
  static std::atomic<int> cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    cudaGetLastError();
    return 148;
  }
  if (dev >= 0 && dev < 64) {
    const int c = cached[dev].load(std::memory_order_relaxed);
    if (c > 0) return c;
  }
  int n = 0;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
    cudaGetLastError();
    n = 148;
  }
  if (dev >= 0 && dev < 64) cached[dev].store(n, std::memory_order_relaxed);
  return n;
}

// ---------------------------------------------------------------------------
// Error word shared with the kernels.
// ---------------------------------------------------------------------------
namespace {
std::once_flag g_errw_once;
int* g_errw = nullptr;
}  // namespace

int* device_error_word() {
  std::call_once(g_errw_once, [] {
    void* p = nullptr;
    if (cudaHostAlloc(&p, 64, cudaHostAllocPortable | cudaHostAllocMapped) == cudaSuccess) {
      g_errw = static_cast<int*>(p);
      *g_errw = 0;
    } else {
      cudaGetLastError();
    }
  });
  return g_errw;  // unified addressing: the host pointer is valid on every device
}

int take_error_word(int* detail) {
  if (!g_errw) return 0;
  volatile int* w = g_errw;
  const int v = *w;
  if (v) {
    if (detail)
      for (int i = 0; i < 4; ++i) detail[i] = w[1 + i];
    *w = 0;
  }
  return v;
}

// ---------------------------------------------------------------------------
// Per-phase timing.
// ---------------------------------------------------------------------------
namespace {
struct ProfRec { int phase; cudaEvent_t a, b; bool closed; };
std::mutex g_prof_mu;
std::vector<ProfRec> g_prof;
std::atomic<bool> g_prof_on{false};
}  // namespace

void profile_enable(bool on) { g_prof_on.store(on); }
bool profile_enabled() { return g_prof_on.load(std::memory_order_relaxed); }

void profile_mark(int phase, bool begin, cudaStream_t s) {
  std::lock_guard<std::mutex> lk(g_prof_mu);
  if (begin) {
    ProfRec r{phase, nullptr, nullptr, false};
    cudaEventCreate(&r.a);
    cudaEventCreate(&r.b);
    cudaEventRecord(r.a, s);
    g_prof.push_back(r);
  } else {
    for (auto it = g_prof.rbegin(); it != g_prof.rend(); ++it)
      if (it->phase == phase && !it->closed) {
        cudaEventRecord(it->b, s);
        it->closed = true;
        break;
      }
  }
}

void profile_read(float* ms, int n) {
  std::lock_guard<std::mutex> lk(g_prof_mu);
  for (int i = 0; i < n; ++i) ms[i] = 0.f;
  for (auto& r : g_prof) {
    if (r.closed) {
      cudaEventSynchronize(r.b);
      float t = 0.f;
      if (cudaEventElapsedTime(&t, r.a, r.b) == cudaSuccess && r.phase < n) ms[r.phase] += t;
    }
    cudaEventDestroy(r.a);
    cudaEventDestroy(r.b);
  }
  g_prof.clear();
}

// ---------------------------------------------------------------------------
// Scratch pool.
// ---------------------------------------------------------------------------
namespace {
struct Block { void* p = nullptr; size_t n = 0; };
std::mutex g_ws_mu;
std::map<std::tuple<int, cudaStream_t, int>, Block> g_ws;
}  // namespace

void* workspace(cudaStream_t stream, size_t bytes, int slot) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    set_last_error("cudaGetDevice failed");
    return nullptr;
  }
  std::lock_guard<std::mutex> lk(g_ws_mu);
  Block& b = g_ws[std::make_tuple(dev, stream, slot)];
  if (b.n >= bytes && b.p) return b.p;
  if (b.p) {
    // Work already queued on this stream may still read the old block.
    cudaStreamSynchronize(stream);
    cudaFree(b.p);
    b.p = nullptr;
    b.n = 0;
  }
  size_t want = bytes + bytes / 4 + (1 << 20);
  cudaError_t e = cudaMalloc(&b.p, want);
  if (e != cudaSuccess) {
    want = bytes;
    e = cudaMalloc(&b.p, want);
  }
  if (e != cudaSuccess) {
    cudaGetLastError();
    b.p = nullptr;
    set_last_error("scratch allocation of %zu bytes failed: %s", bytes, cudaGetErrorString(e));
    return nullptr;
  }
  b.n = want;
  return b.p;
}

int make_arena(Arena* a, cudaStream_t stream, size_t bytes, int slot) {
  a->base = static_cast<char*>(workspace(stream, bytes, slot));
  a->cap = bytes;
  a->off = 0;
  return a->base ? HASTE_B200_OK : HASTE_B200_ERR_CUDA;
}

// ---------------------------------------------------------------------------
// Column sums.
// ---------------------------------------------------------------------------
namespace {

constexpr int CS_COLS = 128;   // columns per block (one per thread)
constexpr int CS_CHUNKS = 64;  // row chunks (partials per column)

inline int cs_chunks(int rows) { return rows < CS_CHUNKS ? (rows > 0 ? rows : 1) : CS_CHUNKS; }

template <typename T>
__global__ void colsum_stage1(const T* __restrict__ in, long long lda, int rows, int width,
                              int chunks, float* __restrict__ part) {
  const int j = blockIdx.x * CS_COLS + threadIdx.x;
  if (j >= width) return;
  const int c = blockIdx.y;
  const int per = (rows + chunks - 1) / chunks;
  const int r0 = c * per, r1 = min(rows, r0 + per);
  // four independent chains keep loads in flight; the combination order is fixed
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  int r = r0;
  for (; r + 3 < r1; r += 4) {
    s0 += ld(in + (long long)(r + 0) * lda + j);
    s1 += ld(in + (long long)(r + 1) * lda + j);
    s2 += ld(in + (long long)(r + 2) * lda + j);
    s3 += ld(in + (long long)(r + 3) * lda + j);
  }
  for (; r < r1; ++r) s0 += ld(in + (long long)r * lda + j);
  part[(long long)c * width + j] = (s0 + s1) + (s2 + s3);
}

template <typename T>
__global__ void colsum_stage2(const float* __restrict__ part, int width, int chunks,
                              T* __restrict__ out, int accumulate) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= width) return;
  float s = 0.f;
  for (int c = 0; c < chunks; ++c) s += part[(long long)c * width + j];
  if (accumulate) s += ld(out + j);
  st(out + j, s);
}

template <typename T>
__global__ void to_float_kernel(const T* __restrict__ src, float* __restrict__ dst, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = ld(src + i);
}
template <typename T>
__global__ void from_float_kernel(const float* __restrict__ src, T* __restrict__ dst, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) st(dst + i, src[i]);
}

template <typename T>
__global__ void add_float_into_kernel(const float* __restrict__ src, T* __restrict__ dst, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) st(dst + i, ld(dst + i) + src[i]);
}

}  // namespace

int add_float_into(int dtype, const float* src, void* dst, size_t n, cudaStream_t stream) {
  if (n == 0) return HASTE_B200_OK;
  const int blocks = ceil_div((long long)n, 256);
  if (dtype == HASTE_B200_F32)
    add_float_into_kernel<float><<<blocks, 256, 0, stream>>>(src, (float*)dst, n);
  else if (dtype == HASTE_B200_F16)
    add_float_into_kernel<__half><<<blocks, 256, 0, stream>>>(src, (__half*)dst, n);
  else
    add_float_into_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(src, (__nv_bfloat16*)dst, n);
  HB_LAUNCH_OK();
  count_launch(1);
  return HASTE_B200_OK;
}

size_t colsum_scratch_floats(int rows, int width) { return (size_t)cs_chunks(rows) * width; }

int colsum(int in_dtype, const void* in, long long ld_, int rows, int width, int out_dtype,
           void* out, int accumulate, float* scratch, cudaStream_t stream) {
  if (width <= 0) return HASTE_B200_OK;
  const int chunks = cs_chunks(rows);
  dim3 g1(ceil_div(width, CS_COLS), chunks);
  if (in_dtype == HASTE_B200_F32)
    colsum_stage1<float><<<g1, CS_COLS, 0, stream>>>((const float*)in, ld_, rows, width, chunks,
                                                      scratch);
  else if (in_dtype == HASTE_B200_F16)
    colsum_stage1<__half><<<g1, CS_COLS, 0, stream>>>((const __half*)in, ld_, rows, width, chunks,
                                                       scratch);
  else
    colsum_stage1<__nv_bfloat16><<<g1, CS_COLS, 0, stream>>>((const __nv_bfloat16*)in, ld_, rows,
                                                              width, chunks, scratch);
  HB_LAUNCH_OK();
  if (out_dtype == HASTE_B200_F32)
    colsum_stage2<float><<<ceil_div(width, 128), 128, 0, stream>>>(scratch, width, chunks,
                                                                    (float*)out, accumulate);
  else if (out_dtype == HASTE_B200_F16)
    colsum_stage2<__half><<<ceil_div(width, 128), 128, 0, stream>>>(scratch, width, chunks,
                                                                     (__half*)out, accumulate);
  else
    colsum_stage2<__nv_bfloat16><<<ceil_div(width, 128), 128, 0, stream>>>(
        scratch, width, chunks, (__nv_bfloat16*)out, accumulate);
  HB_LAUNCH_OK();
  count_launch(2);
  return HASTE_B200_OK;
}

int to_float(int dtype, const void* src, float* dst, size_t n, cudaStream_t stream) {
  if (n == 0) return HASTE_B200_OK;
  const int blocks = ceil_div((long long)n, 256);
  if (dtype == HASTE_B200_F32)
    to_float_kernel<float><<<blocks, 256, 0, stream>>>((const float*)src, dst, n);
  else if (dtype == HASTE_B200_F16)
    to_float_kernel<__half><<<blocks, 256, 0, stream>>>((const __half*)src, dst, n);
  else
    to_float_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)src, dst, n);
  HB_LAUNCH_OK();
  count_launch(1);
  return HASTE_B200_OK;
}

int from_float(int dtype, const float* src, void* dst, size_t n, cudaStream_t stream) {
  if (n == 0) return HASTE_B200_OK;
  const int blocks = ceil_div((long long)n, 256);
  if (dtype == HASTE_B200_F32)
    from_float_kernel<float><<<blocks, 256, 0, stream>>>(src, (float*)dst, n);
  else if (dtype == HASTE_B200_F16)
    from_float_kernel<__half><<<blocks, 256, 0, stream>>>(src, (__half*)dst, n);
  else
    from_float_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(src, (__nv_bfloat16*)dst, n);
  HB_LAUNCH_OK();
  count_launch(1);
  return HASTE_B200_OK;
}

}  // namespace hb
