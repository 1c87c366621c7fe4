// Host-side utilities shared by the cell drivers: per-(device, stream) scratch,
// deterministic column sums, dtype conversion helpers and the launch counter.
#pragma once

#include "common.cuh"

namespace hb {

// SM count of the current device (cached per device ordinal).
int sm_count();

// Counts kernels launched by this library (reported through the C ABI).
void count_launch(int n);

// One process-wide error word in pinned, device-visible host memory.  Kernels that give
// up on a bounded wait store a non-zero code there; the host reads it without having to
// copy anything back.  device_error_word() is the pointer kernels get;
// take_error_word() returns the current value and clears it.
int* device_error_word();
int take_error_word(int* detail = nullptr);  // detail: 4 ints of kernel-specific context

// Library-owned scratch.  One grow-only buffer per (device, stream, slot), so
// calls issued on different streams never share scratch.  The pointer stays
// valid until the next larger request on the same stream.  Returns nullptr
// (and sets the last error) if the allocation fails.
void* workspace(cudaStream_t stream, size_t bytes, int slot = 0);

// Bump allocator over one workspace() block; every sub-buffer is 256-byte aligned.
struct Arena {
  char* base = nullptr;
  size_t cap = 0, off = 0;
  static size_t pad(size_t b) { return (b + 255) & ~size_t(255); }
  template <typename T> T* take(size_t n) {
    size_t b = pad(n * sizeof(T));
    if (off + b > cap) return nullptr;
    T* p = reinterpret_cast<T*>(base + off);
    off += b;
    return p;
  }
};
int make_arena(Arena* a, cudaStream_t stream, size_t bytes, int slot = 0);

// out[j] (+)= sum_r in[r*ld + j], r < rows, j < width.  Deterministic: a fixed
// two-stage tree whatever the launch timing.  `in_dtype`/`out_dtype` are
// HASTE_B200_F32 / HASTE_B200_BF16.  `scratch` needs colsum_scratch_floats().
size_t colsum_scratch_floats(int rows, int width);
int colsum(int in_dtype, const void* in, long long ld, int rows, int width, int out_dtype,
           void* out, int accumulate, float* scratch, cudaStream_t stream);

// dst[i] = (float)src[i] and back, n elements.
int to_float(int dtype, const void* src, float* dst, size_t n, cudaStream_t stream);
int from_float(int dtype, const float* src, void* dst, size_t n, cudaStream_t stream);

// dst[i] += src[i] (dst in `dtype`), n elements.
int add_float_into(int dtype, const float* src, void* dst, size_t n, cudaStream_t stream);

// Optional per-phase device timing (CUDA events on the call's stream), switched on
// through the C ABI; used by the benchmark to attribute time to kernels.
enum Phase { PH_PROJ = 0, PH_REC_FWD = 1, PH_REC_BWD = 2, PH_WGRAD = 3, PH_DGRAD = 4, PH_OTHER = 5,
             PH_COUNT = 6 };
void profile_enable(bool on);
bool profile_enabled();
void profile_mark(int phase, bool begin, cudaStream_t s);
// Sums elapsed ms per phase since the last read (synchronises the recorded events).
void profile_read(float* ms, int n);
struct ProfScope {
  int phase; cudaStream_t s; bool on;
  ProfScope(int phase_, cudaStream_t s_) : phase(phase_), s(s_), on(profile_enabled()) {
    if (on) profile_mark(phase, true, s);
  }
  ~ProfScope() { if (on) profile_mark(phase, false, s); }
};

inline size_t dtype_size(int dtype) { return dtype == HASTE_B200_F32 ? 4 : 2; }

}  // namespace hb
