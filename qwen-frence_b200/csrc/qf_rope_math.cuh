// RoPE frequencies shared by the kernels that rotate Q / K: the table is evaluated once on
// the host in fp32 and handed to a kernel by value, so every kernel rotates with the same
// bits.  inv_freq[i] = expf(i * (-(float)log(base) / half)): the formula of the reference's
// fused kernels (custom_kernels/rope_kv_write.py:190-191).
#pragma once

#include <cmath>

namespace qf {

constexpr int kMaxHalf = 128;  // head_dim <= 256

struct InvFreqTable {
  float v[kMaxHalf];
};

inline InvFreqTable make_inv_freq(double base, int half) {
  InvFreqTable freq{};
  const float log_theta = static_cast<float>(std::log(base));
  const float step = -log_theta / static_cast<float>(half);
  for (int i = 0; i < half && i < kMaxHalf; ++i) freq.v[i] = expf(static_cast<float>(i) * step);
  return freq;
}

}  // namespace qf
