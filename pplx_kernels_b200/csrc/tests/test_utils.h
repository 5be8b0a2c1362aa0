// Helpers for the C++ test and benchmark executables: deterministic synthetic
// routing data and small host-side conveniences.
//
// Role parity: csrc/all_to_all/test_utils.h:18-146 of the reference.
#pragma once

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <numeric>
#include <random>
#include <vector>

#include <cuda_bf16.h>

#include "../core/buffer.h"
#include "../core/utils.h"

namespace pplx {
namespace testing {

inline float to_float(float v) { return v; }
inline float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T>
T from_float(float v);
template <>
inline float from_float<float>(float v) { return v; }
template <>
inline __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16(v); }

// Tokens, routing and weights of one DP group.
template <typename T>
struct RankData {
  int num_tokens = 0;
  int hidden = 0;
  int topk = 0;
  std::vector<T> x;             // [num_tokens][hidden]
  std::vector<uint32_t> indices;  // [num_tokens][topk], distinct per token
  std::vector<float> weights;     // [num_tokens][topk]

  RankData(std::mt19937& rng, int max_tokens, int num_experts, int topk_, int hidden_,
           bool use_max_tokens)
      : hidden(hidden_), topk(topk_) {
    num_tokens = use_max_tokens
                     ? max_tokens
                     : std::uniform_int_distribution<int>(1, max_tokens)(rng);
    std::normal_distribution<float> normal(0.f, 1.f);
    std::uniform_real_distribution<float> uniform(0.f, 1.f);
    x.resize(static_cast<size_t>(num_tokens) * hidden);
    for (auto& v : x) v = from_float<T>(normal(rng));
    indices.resize(static_cast<size_t>(num_tokens) * topk);
    weights.resize(static_cast<size_t>(num_tokens) * topk);
    std::vector<uint32_t> experts(num_experts);
    for (int i = 0; i < num_tokens; ++i) {
      std::iota(experts.begin(), experts.end(), 0u);
      std::shuffle(experts.begin(), experts.end(), rng);
      for (int k = 0; k < topk; ++k) {
        indices[static_cast<size_t>(i) * topk + k] = experts[k];
        weights[static_cast<size_t>(i) * topk + k] = uniform(rng);
      }
    }
  }
};

template <typename T>
DeviceBuffer<T> to_device(const std::vector<T>& v) {
  DeviceBuffer<T> d(std::max<size_t>(v.size(), 1), false);
  if (!v.empty()) d.copy_from_host(v);
  return d;
}

struct Stats {
  double mean = 0, stddev = 0, p50 = 0;
};

inline Stats stats(std::vector<float> v) {
  Stats s;
  if (v.empty()) return s;
  s.mean = std::accumulate(v.begin(), v.end(), 0.0) / v.size();
  double var = 0;
  for (float x : v) var += (x - s.mean) * (x - s.mean);
  s.stddev = std::sqrt(var / v.size());
  std::sort(v.begin(), v.end());
  s.p50 = v[v.size() / 2];
  return s;
}

}  // namespace testing
}  // namespace pplx
