// C++ test of the host classes without Python, MPI or torch: a world of four
// ranks with two DP groups runs on ONE device as cooperative group launches.
//
// Role parity: csrc/all_to_all/test_all_to_all.cpp:46-394 of the reference
// (testDispatchCombine<T, Kernel>: 8 experts, top-3, hidden 16, at most 10
// tokens, dp 2; float and bf16 payloads; checks of per-expert counts, of the
// received rows as a set, and of the combined result).  The reference needs
// `mpirun -np 4` and four GPUs; this needs one GPU.
#include <cstdio>
#include <cstdlib>
#include <map>
#include <set>
#include <string>

#include "../runtime/all_to_all.h"
#include "test_utils.h"

using namespace pplx;
using namespace pplx::testing;

namespace {

template <typename T>
DType dtype_of();
template <>
DType dtype_of<float>() { return DType::kF32; }
template <>
DType dtype_of<__nv_bfloat16>() { return DType::kBF16; }

#define EXPECT(cond, ...)                                   \
  do {                                                      \
    if (!(cond)) {                                          \
      std::fprintf(stderr, "FAILED %s:%d: ", __FILE__, __LINE__); \
      std::fprintf(stderr, __VA_ARGS__);                    \
      std::fprintf(stderr, "\n");                           \
      return false;                                         \
    }                                                       \
  } while (0)

template <typename T>
bool test_dispatch_combine(int world, int dp_size, bool split) {
  constexpr int kExperts = 8, kTopk = 3, kHidden = 16, kMaxTokens = 10;
  const int groups = world / dp_size;
  const int nle = kExperts / world;
  const int cap = kMaxTokens * groups;

  A2AConfig cfg;
  cfg.max_num_tokens = kMaxTokens;
  cfg.num_experts = kExperts;
  cfg.experts_per_token = kTopk;
  cfg.world_size = world;
  cfg.dp_size = dp_size;
  cfg.hidden_dim = kHidden;
  cfg.hidden_dim_bytes = kHidden * static_cast<int>(sizeof(T));
  cfg.hidden_dim_scale_bytes = 0;
  auto ranks = AllToAll::create_local_world(cfg);
  std::vector<AllToAll*> raw;
  for (auto& r : ranks) {
    r->set_debug_checks(true);
    r->set_timeout_ms(3000);
    raw.push_back(r.get());
  }

  std::mt19937 rng(0xdeadbeef);
  std::vector<RankData<T>> data;
  for (int g = 0; g < groups; ++g) data.emplace_back(rng, kMaxTokens, kExperts, kTopk, kHidden, false);

  struct Buffers {
    DeviceBuffer<T> x, expert_x, expert_y;
    DeviceBuffer<uint32_t> indices, bound_m;
    DeviceBuffer<float> weights;
    DeviceBuffer<int32_t> counts;
    DeviceBuffer<__nv_bfloat16> out;
  };
  std::vector<Buffers> bufs(world);
  std::vector<DispatchCall> dcalls(world);
  std::vector<CombineCall> ccalls(world);
  for (int r = 0; r < world; ++r) {
    const RankData<T>& d = data[r / dp_size];
    Buffers& b = bufs[r];
    b.x = to_device(d.x);
    b.indices = to_device(d.indices);
    b.weights = to_device(d.weights);
    b.bound_m = to_device(std::vector<uint32_t>{static_cast<uint32_t>(d.num_tokens)});
    b.counts = DeviceBuffer<int32_t>(nle);
    b.expert_x = DeviceBuffer<T>(static_cast<size_t>(nle) * cap * kHidden);
    b.expert_y = DeviceBuffer<T>(static_cast<size_t>(nle) * cap * kHidden);
    b.out = DeviceBuffer<__nv_bfloat16>(static_cast<size_t>(kMaxTokens) * kHidden);

    DispatchCall& dc = dcalls[r];
    dc.out_num_tokens = b.counts.get();
    dc.out_x.data = reinterpret_cast<uint8_t*>(b.expert_x.get());
    dc.out_x.stride_outer = static_cast<int64_t>(cap) * kHidden * sizeof(T);
    dc.out_x.stride_row = kHidden * sizeof(T);
    dc.out_rows = cap;
    dc.x.data = reinterpret_cast<const uint8_t*>(b.x.get());
    dc.x.stride_row = kHidden * sizeof(T);
    dc.indices = b.indices.get();
    dc.bound_m = b.bound_m.get();
    dc.num_tokens = d.num_tokens;

    CombineCall& cc = ccalls[r];
    cc.out_tokens = b.out.get();
    cc.out_stride_row = kHidden;
    cc.weights = b.weights.get();
    cc.w_stride_row = kTopk;
    cc.expert_y = b.expert_y.get();
    cc.y_stride_e = static_cast<int64_t>(cap) * kHidden;
    cc.y_stride_row = kHidden;
    cc.bound_m = b.bound_m.get();
    cc.num_tokens = d.num_tokens;
    cc.in = dtype_of<T>();
    cc.out = DType::kBF16;
  }

  cudaStream_t stream = nullptr;
  for (int iteration = 0; iteration < 3; ++iteration) {
    if (split) {
      AllToAll::dispatch_group(raw, dcalls, SplitMode::kSend, stream);
      AllToAll::dispatch_group(raw, dcalls, SplitMode::kRecv, stream);
    } else {
      AllToAll::dispatch_group(raw, dcalls, SplitMode::kNone, stream);
    }
    CUDA_CHECK(cudaDeviceSynchronize());

    // Expected rows per expert: (group, token) pairs, each sent by one rank of the group.
    std::map<int, std::multiset<std::vector<float>>> expected;
    for (int g = 0; g < groups; ++g) {
      const RankData<T>& d = data[g];
      for (int i = 0; i < d.num_tokens; ++i) {
        for (int k = 0; k < kTopk; ++k) {
          std::vector<float> row(kHidden);
          for (int j = 0; j < kHidden; ++j) row[j] = to_float(d.x[static_cast<size_t>(i) * kHidden + j]);
          expected[static_cast<int>(d.indices[static_cast<size_t>(i) * kTopk + k])].insert(row);
        }
      }
    }
    for (int r = 0; r < world; ++r) {
      raw[r]->check_status();
      const std::vector<int32_t> counts = bufs[r].counts.to_host();
      const std::vector<T> ex = bufs[r].expert_x.to_host();
      for (int le = 0; le < nle; ++le) {
        const int e = r * nle + le;
        EXPECT(counts[le] == static_cast<int>(expected[e].size()),
               "rank %d expert %d: %d rows, expected %zu", r, e, counts[le], expected[e].size());
        std::multiset<std::vector<float>> got;
        for (int row = 0; row < counts[le]; ++row) {
          std::vector<float> v(kHidden);
          for (int j = 0; j < kHidden; ++j)
            v[j] = to_float(ex[(static_cast<size_t>(le) * cap + row) * kHidden + j]);
          got.insert(v);
        }
        EXPECT(got == expected[e], "rank %d expert %d: received rows differ", r, e);
      }
      // Identity experts: y = x.
      CUDA_CHECK(cudaMemcpy(bufs[r].expert_y.get(), bufs[r].expert_x.get(), bufs[r].expert_x.bytes(),
                            cudaMemcpyDeviceToDevice));
    }

    if (split) {
      AllToAll::combine_group(raw, ccalls, SplitMode::kSend, stream);
      AllToAll::combine_group(raw, ccalls, SplitMode::kRecv, stream);
    } else {
      AllToAll::combine_group(raw, ccalls, SplitMode::kNone, stream);
    }
    CUDA_CHECK(cudaDeviceSynchronize());
    for (int r = 0; r < world; ++r) {
      raw[r]->check_status();
      const RankData<T>& d = data[r / dp_size];
      const std::vector<__nv_bfloat16> out = bufs[r].out.to_host();
      for (int i = 0; i < d.num_tokens; ++i) {
        float wsum = 0.f;
        for (int k = 0; k < kTopk; ++k) wsum += d.weights[static_cast<size_t>(i) * kTopk + k];
        for (int j = 0; j < kHidden; ++j) {
          const float want = to_float(d.x[static_cast<size_t>(i) * kHidden + j]) * wsum;
          const float got = to_float(out[static_cast<size_t>(i) * kHidden + j]);
          EXPECT(std::fabs(got - want) <= 0.05f + 0.02f * std::fabs(want),
                 "rank %d token %d col %d: %f, expected %f", r, i, j, got, want);
        }
      }
    }
  }
  return true;
}

bool test_timeout_is_reported() {
  A2AConfig cfg;
  cfg.max_num_tokens = 4;
  cfg.num_experts = 4;
  cfg.experts_per_token = 2;
  cfg.world_size = 2;
  cfg.dp_size = 1;
  cfg.hidden_dim = 16;
  cfg.hidden_dim_bytes = 32;
  auto ranks = AllToAll::create_local_world(cfg);
  ranks[0]->set_timeout_ms(50);
  std::mt19937 rng(1);
  RankData<__nv_bfloat16> d(rng, 4, 4, 2, 16, true);
  auto x = to_device(d.x);
  auto idx = to_device(d.indices);
  DeviceBuffer<int32_t> counts(2);
  DeviceBuffer<__nv_bfloat16> ex(2 * 8 * 16);
  DispatchCall dc;
  dc.out_num_tokens = counts.get();
  dc.out_x.data = reinterpret_cast<uint8_t*>(ex.get());
  dc.out_x.stride_outer = 8 * 32;
  dc.out_x.stride_row = 32;
  dc.out_rows = 8;
  dc.x.data = reinterpret_cast<const uint8_t*>(x.get());
  dc.x.stride_row = 32;
  dc.indices = idx.get();
  dc.num_tokens = 4;
  // Only rank 0 takes part: its wait for rank 1's counts must run out and be reported.
  AllToAll::dispatch_group({ranks[0].get()}, {dc}, SplitMode::kNone, nullptr);
  CUDA_CHECK(cudaDeviceSynchronize());
  const Status s = ranks[0]->read_status();
  EXPECT(s.code == kTimeout && s.phase == kPhaseDispatchCounts && s.peer == 1,
         "status %u phase %u peer %u", s.code, s.phase, s.peer);
  bool threw = false;
  try {
    ranks[0]->check_status();
  } catch (const Error&) {
    threw = true;
  }
  EXPECT(threw, "check_status did not throw");
  return true;
}

}  // namespace

int main() {
  int failures = 0;
  auto run = [&](const char* name, bool ok) {
    std::printf("[%s] %s\n", ok ? " OK " : "FAIL", name);
    if (!ok) ++failures;
  };
  try {
    CUDA_CHECK(cudaSetDevice(0));
    run("dispatch/combine float  world 4 dp 2", test_dispatch_combine<float>(4, 2, false));
    run("dispatch/combine bf16   world 4 dp 2", test_dispatch_combine<__nv_bfloat16>(4, 2, false));
    run("dispatch/combine bf16   world 4 dp 2 split", test_dispatch_combine<__nv_bfloat16>(4, 2, true));
    run("dispatch/combine float  world 2 dp 1", test_dispatch_combine<float>(2, 1, false));
    run("dispatch/combine bf16   world 1 dp 1", test_dispatch_combine<__nv_bfloat16>(1, 1, false));
    run("dispatch/combine bf16   world 8 dp 4", test_dispatch_combine<__nv_bfloat16>(8, 4, false));
    run("missing peer times out and is reported", test_timeout_is_reported());
  } catch (const std::exception& e) {
    std::fprintf(stderr, "exception: %s\n", e.what());
    return 2;
  }
  std::printf("%d failure(s)\n", failures);
  return failures == 0 ? 0 : 1;
}
