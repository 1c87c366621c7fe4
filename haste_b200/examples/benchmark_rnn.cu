// Benchmark driver in C++ against the drop-in header, in the form of the reference's own
// harness (benchmarks/benchmark_lstm.cc:43-44,522-555 and benchmark_gru.cc:523-548): a grid of
// batch size N, hidden size H and input size C, `time_steps` steps per sequence, the mean of
// `sample_size` timed runs by CUDA events, one CSV line "batch_size,hidden_size,input_size,time_ms"
// per point.  No Eigen and no cuDNN: buffers are plain device allocations filled with a fixed
// pattern (the reference times uninitialised buffers).
//
//   nvcc -std=c++17 -gencode arch=compute_100a,code=sm_100a -I include \
//        haste_b200/examples/benchmark_rnn.cu -o benchmark_rnn -L haste_b200 -lhaste_b200
//   ./benchmark_rnn [--cell lstm|gru] [--inference] [--sample_size 10] [--time_steps 50]
//                   [--point N,H,C]      (one point instead of the grid)
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <string>
#include <vector>

#include "haste_b200/haste.hpp"

using namespace haste::v0;

static float* device_buffer(size_t n, float scale) {
  std::vector<float> host(n);
  for (size_t i = 0; i < n; ++i) host[i] = scale * std::sin(0.37f * (float)(i % 4099) + 0.1f);
  float* p = nullptr;
  if (cudaMalloc(&p, n * sizeof(float)) != cudaSuccess) {
    std::fprintf(stderr, "cudaMalloc of %zu floats failed\n", n);
    std::exit(2);
  }
  cudaMemcpy(p, host.data(), n * sizeof(float), cudaMemcpyHostToDevice);
  return p;
}

static float time_loop(const std::function<void()>& fn, int iterations) {
  cudaEvent_t start, stop;
  cudaEventCreate(&start);
  cudaEventCreate(&stop);
  fn();  // warm-up, not timed
  cudaEventRecord(start);
  for (int i = 0; i < iterations; ++i) fn();
  cudaEventRecord(stop);
  cudaEventSynchronize(stop);
  float ms = 0.f;
  cudaEventElapsedTime(&ms, start, stop);
  cudaEventDestroy(start);
  cudaEventDestroy(stop);
  return ms / iterations;
}

static float bench_point(bool lstm, bool inference, int sample_size, int T, int N, int H, int C) {
  const int G = lstm ? 4 : 3;
  const size_t TN = (size_t)T * N;
  float* W = device_buffer((size_t)C * G * H, 1.0f / std::sqrt((float)C));
  float* R = device_buffer((size_t)H * G * H, 1.0f / std::sqrt((float)H));
  float* b = device_buffer((size_t)G * H, 0.1f);
  float* b2 = device_buffer((size_t)G * H, 0.1f);
  float* x = device_buffer(TN * C, 1.0f);
  float* h = device_buffer((size_t)(T + 1) * N * H, 0.0f);
  float* c = device_buffer((size_t)(T + 1) * N * H, 0.0f);
  float* v = device_buffer(TN * 4 * H, 0.0f);
  float* tmp_Wx = device_buffer(TN * G * H, 0.0f);
  float* tmp_Rh = device_buffer((size_t)N * G * H, 0.0f);
  float ms;
  if (inference) {
    ms = time_loop([&] {
      if (lstm) {
        lstm::ForwardPass<float> fw(false, N, C, H, nullptr, 0);
        fw.Run(T, W, R, b, x, h, c, v, tmp_Rh, 0.0f, nullptr);
      } else {
        gru::ForwardPass<float> fw(false, N, C, H, nullptr, 0);
        fw.Run(T, W, R, b, b2, x, h, nullptr, tmp_Wx, tmp_Rh, 0.0f, nullptr);
      }
    }, sample_size);
  } else {
    // the reference's backward takes pre-transposed W, R and x; as its harness does, the
    // transposes are not part of the timed region (benchmark_lstm.cc passes them ready-made)
    float* W_t = device_buffer((size_t)C * G * H, 1.0f / std::sqrt((float)C));
    float* R_t = device_buffer((size_t)H * G * H, 1.0f / std::sqrt((float)H));
    float* x_t = device_buffer(TN * C, 1.0f);
    float* dh_new = device_buffer((size_t)(T + 1) * N * H, 0.01f);
    float* dc_new = device_buffer((size_t)(T + 1) * N * H, 0.01f);
    float* dx = device_buffer(TN * C, 0.0f);
    float* dW = device_buffer((size_t)C * G * H, 0.0f);
    float* dR = device_buffer((size_t)H * G * H, 0.0f);
    float* db = device_buffer((size_t)G * H, 0.0f);
    float* db2 = device_buffer((size_t)G * H, 0.0f);
    float* dh = device_buffer((size_t)N * H, 0.0f);
    float* dc = device_buffer((size_t)N * H, 0.0f);
    float* dp = device_buffer(TN * 3 * H, 0.0f);
    float* dq = device_buffer(TN * 3 * H, 0.0f);
    ms = time_loop([&] {
      if (lstm) {
        lstm::ForwardPass<float> fw(true, N, C, H, nullptr, 0);
        fw.Run(T, W, R, b, x, h, c, v, tmp_Rh, 0.0f, nullptr);
        lstm::BackwardPass<float> bw(N, C, H, nullptr, 0);
        bw.Run(T, W_t, R_t, b, x_t, h, c, dh_new, dc_new, dx, dW, dR, db, dh, dc, v, nullptr);
      } else {
        gru::ForwardPass<float> fw(true, N, C, H, nullptr, 0);
        fw.Run(T, W, R, b, b2, x, h, v, tmp_Wx, tmp_Rh, 0.0f, nullptr);
        gru::BackwardPass<float> bw(N, C, H, nullptr, 0);
        bw.Run(T, W_t, R_t, b, b2, x_t, h, v, dh_new, dx, dW, dR, db, db2, dh, dp, dq, nullptr);
      }
    }, sample_size);
    for (float* p : {W_t, R_t, x_t, dh_new, dc_new, dx, dW, dR, db, db2, dh, dc, dp, dq}) cudaFree(p);
  }
  for (float* p : {W, R, b, b2, x, h, c, v, tmp_Wx, tmp_Rh}) cudaFree(p);
  return ms;
}

int main(int argc, char** argv) {
  bool lstm = true, inference = false;
  int sample_size = 10, time_steps = 50;
  int pn = 0, ph = 0, pc = 0;
  for (int i = 1; i < argc; ++i) {
    const std::string a = argv[i];
    auto next = [&]() -> const char* { return i + 1 < argc ? argv[++i] : ""; };
    if (a == "--cell") lstm = std::string(next()) != "gru";
    else if (a == "--inference") inference = true;
    else if (a == "--sample_size") sample_size = std::atoi(next());
    else if (a == "--time_steps") time_steps = std::atoi(next());
    else if (a == "--point") std::sscanf(next(), "%d,%d,%d", &pn, &ph, &pc);
    else { std::fprintf(stderr, "unknown argument %s\n", a.c_str()); return 2; }
  }
  std::printf("# Benchmark configuration:\n");
  std::printf("#   Cell: %s\n", lstm ? "LSTM" : "GRU");
  std::printf("#   Mode: %s\n", inference ? "inference" : "training");
  std::printf("#   Implementation: haste_b200\n");
  std::printf("#   Sample size: %d\n", sample_size);
  std::printf("#   Time steps: %d\n", time_steps);
  std::printf("#\n# batch_size,hidden_size,input_size,time_ms\n");
  try {
    if (pn > 0) {
      std::printf("%d,%d,%d,%f\n", pn, ph, pc,
                  bench_point(lstm, inference, sample_size, time_steps, pn, ph, pc));
      return 0;
    }
    for (const int N : {1, 16, 32, 64, 128})
      for (const int H : {128, 256, 512, 768, 1024, 1536, 2048, 3072, 4096})
        for (const int C : {64, 128, 256, 512}) {
          std::printf("%d,%d,%d,%f\n", N, H, C,
                      bench_point(lstm, inference, sample_size, time_steps, N, H, C));
          std::fflush(stdout);
        }
  } catch (const std::exception& e) {
    std::fprintf(stderr, "error: %s\n", e.what());
    return 1;
  }
  return 0;
}
