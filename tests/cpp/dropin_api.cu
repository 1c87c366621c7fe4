// Compile-and-run check of the drop-in C++ API: runs one LSTM forward+backward through
// haste::v0::lstm::{ForwardPass,BackwardPass}<float> with the reference's calling convention
// (pre-transposed x_t/W_t/R_t) and prints a checksum that the Python test compares with the
// same computation done through the Python ops.  Also instantiates every other class so that
// signature drift is a compile error.
#include <cstdio>
#include <cstdlib>
#include <cmath>
#include <stdexcept>
#include <vector>

#include "haste_b200/haste.hpp"

using namespace haste::v0;

template <typename T>
void instantiate_all() {
  layer_norm::ForwardPass<T> lf(1, 1, nullptr, nullptr, nullptr);
  layer_norm::BackwardPass<T> lb(1, 1, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr);
  (void)sizeof(gru::ForwardPass<T>);
  (void)sizeof(gru::BackwardPass<T>);
  (void)sizeof(indrnn::ForwardPass<T>);
  (void)sizeof(indrnn::BackwardPass<T>);
  auto f1 = &layer_norm_lstm::ForwardPass<T>::Run;
  auto f2 = &layer_norm_lstm::BackwardPass<T>::Run;
  auto f3 = &layer_norm_gru::ForwardPass<T>::Run;
  auto f4 = &layer_norm_gru::BackwardPass<T>::Run;
  auto f5 = &layer_norm_indrnn::ForwardPass<T>::Run;
  auto f6 = &layer_norm_indrnn::BackwardPass<T>::Run;
  auto f7 = &gru::ForwardPass<T>::Run;
  auto f8 = &gru::BackwardPass<T>::Run;
  auto f9 = &indrnn::ForwardPass<T>::Run;
  auto f10 = &indrnn::BackwardPass<T>::Run;
  auto i1 = &lstm::ForwardPass<T>::Iterate;
  auto i2 = &lstm::BackwardPass<T>::Iterate;
  auto i3 = &gru::ForwardPass<T>::Iterate;
  auto i4 = &gru::BackwardPass<T>::Iterate;
  (void)i1; (void)i2; (void)i3; (void)i4;
  (void)f1; (void)f2; (void)f3; (void)f4; (void)f5; (void)f6; (void)f7; (void)f8; (void)f9; (void)f10;
  (void)lf; (void)lb;
}

static float* dev(const std::vector<float>& v) {
  float* p = nullptr;
  cudaMalloc(&p, v.size() * sizeof(float));
  cudaMemcpy(p, v.data(), v.size() * sizeof(float), cudaMemcpyHostToDevice);
  return p;
}
static float* dev_zero(size_t n) {
  float* p = nullptr;
  cudaMalloc(&p, n * sizeof(float));
  cudaMemset(p, 0, n * sizeof(float));
  return p;
}
static double checksum(const float* d, size_t n) {
  std::vector<float> h(n);
  cudaMemcpy(h.data(), d, n * sizeof(float), cudaMemcpyDeviceToHost);
  double s = 0;
  for (size_t i = 0; i < n; ++i) s += (double)h[i] * (double)((i % 7) + 1);
  return s;
}

int main() {
  instantiate_all<float>();
  instantiate_all<__nv_bfloat16>();
  const int T = 6, N = 5, C = 7, H = 12;
  // deterministic pseudo-random fill shared with the Python side: x_k = sin(0.37 k + phase)
  auto fill = [](size_t n, double phase, double scale) {
    std::vector<float> v(n);
    for (size_t i = 0; i < n; ++i) v[i] = (float)(scale * std::sin(0.37 * (double)i + phase));
    return v;
  };
  std::vector<float> x = fill((size_t)T * N * C, 0.1, 1.0), W = fill((size_t)C * 4 * H, 0.2, 0.4),
                     R = fill((size_t)H * 4 * H, 0.3, 0.3), b = fill(4 * H, 0.4, 0.1),
                     dh_new = fill((size_t)(T + 1) * N * H, 0.5, 1.0),
                     dc_new = fill((size_t)(T + 1) * N * H, 0.6, 1.0);
  // reference convention: transposed copies for the backward pass
  std::vector<float> x_t((size_t)C * T * N), W_t((size_t)4 * H * C), R_t((size_t)4 * H * H);
  for (int t = 0; t < T * N; ++t)
    for (int c = 0; c < C; ++c) x_t[(size_t)c * T * N + t] = x[(size_t)t * C + c];
  for (int c = 0; c < C; ++c)
    for (int j = 0; j < 4 * H; ++j) W_t[(size_t)j * C + c] = W[(size_t)c * 4 * H + j];
  for (int k = 0; k < H; ++k)
    for (int j = 0; j < 4 * H; ++j) R_t[(size_t)j * H + k] = R[(size_t)k * 4 * H + j];

  float *dx_ = dev(x), *dW_ = dev(W), *dR_ = dev(R), *db_ = dev(b);
  float *h = dev_zero((size_t)(T + 1) * N * H), *c = dev_zero((size_t)(T + 1) * N * H);
  float *v = dev_zero((size_t)T * N * 4 * H), *tmp = dev_zero((size_t)N * 4 * H);
  cudaStream_t stream = 0;
  try {
    lstm::ForwardPass<float> fw(true, N, C, H, nullptr, stream);
    fw.Run(T, dW_, dR_, db_, dx_, h, c, v, tmp, 0.0f, nullptr);
    float *gx = dev_zero((size_t)T * N * C), *gW = dev_zero((size_t)C * 4 * H),
          *gR = dev_zero((size_t)H * 4 * H), *gb = dev_zero(4 * H), *gh = dev_zero((size_t)N * H),
          *gc = dev_zero((size_t)N * H);
    float *xt = dev(x_t), *Wt = dev(W_t), *Rt = dev(R_t), *dhn = dev(dh_new), *dcn = dev(dc_new);
    lstm::BackwardPass<float> bw(N, C, H, nullptr, stream);
    bw.Run(T, Wt, Rt, db_, xt, h, c, dhn, dcn, gx, gW, gR, gb, gh, gc, v, nullptr);
    if (haste_b200_sync_check(stream) != HASTE_B200_OK) throw std::runtime_error(haste_b200_last_error());
    std::printf("h %.9e\ndx %.9e\ndW %.9e\ndR %.9e\ndb %.9e\ndh %.9e\ndc %.9e\n",
                checksum(h, (size_t)(T + 1) * N * H), checksum(gx, (size_t)T * N * C),
                checksum(gW, (size_t)C * 4 * H), checksum(gR, (size_t)H * 4 * H), checksum(gb, 4 * H),
                checksum(gh, (size_t)N * H), checksum(gc, (size_t)N * H));
  } catch (const std::exception& e) {
    std::fprintf(stderr, "FAILED: %s\n", e.what());
    return 1;
  }
  return 0;
}
