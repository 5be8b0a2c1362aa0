// C++ benchmark of dispatch and combine without Python or MPI.
//
//   bench_all_to_all                       one rank on GPU 0
//   bench_all_to_all --world 8 --rank R --uid-file /tmp/uid      (one process per GPU;
//       rank 0 writes the rendezvous id to the file, the others read it)
//
// Role parity: csrc/all_to_all/bench_all_to_all.cpp:63-364 of the reference.  Like
// it, every sample times six things with CUDA events: dispatch and combine fused,
// then dispatch send / recv and combine send / recv separately, with a 100 us sleep
// kernel and a barrier between a send and its recv so that the recv measures only
// the receive work.  Reported per configuration: mean +- std and p50 in
// microseconds, maximum over ranks of the per-rank means, and GB/s of payload.
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <string>
#include <thread>

#include <cuda_profiler_api.h>

#include "../kernels/collectives.h"
#include "../runtime/all_to_all.h"
#include "../runtime/bootstrap.h"
#include "test_utils.h"

using namespace pplx;
using namespace pplx::testing;

namespace {

struct Options {
  int world = 1, rank = 0;
  std::string uid_file;
  int experts = 256, topk = 8, hidden = 7168;
  bool fp8 = true;
  int warmup = 10, repeat = 10, samples = 10;
  std::vector<int> tokens = {1, 4, 8, 16, 32, 64, 128};
};

Options parse(int argc, char** argv) {
  Options o;
  for (int i = 1; i < argc; ++i) {
    const std::string a = argv[i];
    auto next = [&]() -> const char* {
      PPLX_CHECK(i + 1 < argc, "missing value after " << a);
      return argv[++i];
    };
    if (a == "--world") o.world = std::atoi(next());
    else if (a == "--rank") o.rank = std::atoi(next());
    else if (a == "--uid-file") o.uid_file = next();
    else if (a == "--experts") o.experts = std::atoi(next());
    else if (a == "--topk") o.topk = std::atoi(next());
    else if (a == "--hidden") o.hidden = std::atoi(next());
    else if (a == "--bf16") o.fp8 = false;
    else if (a == "--fp8") o.fp8 = true;
    else if (a == "--repeat") o.repeat = std::atoi(next());
    else if (a == "--samples") o.samples = std::atoi(next());
    else if (a == "--tokens") {
      o.tokens.clear();
      std::string list = next();
      size_t pos = 0;
      while (pos < list.size()) {
        const size_t comma = list.find(',', pos);
        o.tokens.push_back(std::atoi(list.substr(pos, comma - pos).c_str()));
        if (comma == std::string::npos) break;
        pos = comma + 1;
      }
    } else {
      PPLX_CHECK(false, "unknown option " << a);
    }
  }
  return o;
}

std::shared_ptr<Bootstrap> make_bootstrap(const Options& o) {
  if (o.world == 1) return std::make_shared<SingleBootstrap>();
  PPLX_CHECK(!o.uid_file.empty(), "--uid-file is required for more than one rank");
  UniqueId id{};
  if (o.rank == 0) {
    id = create_unique_id();
    std::ofstream f(o.uid_file + ".tmp", std::ios::binary);
    f.write(reinterpret_cast<const char*>(id.bytes), kUniqueIdBytes);
    f.close();
    std::rename((o.uid_file + ".tmp").c_str(), o.uid_file.c_str());
  } else {
    for (int tries = 0;; ++tries) {
      std::ifstream f(o.uid_file, std::ios::binary);
      if (f.good() && f.read(reinterpret_cast<char*>(id.bytes), kUniqueIdBytes)) break;
      PPLX_CHECK(tries < 3000, "no unique id appeared in " << o.uid_file);
      std::this_thread::sleep_for(std::chrono::milliseconds(10));
    }
  }
  return std::make_shared<SocketBootstrap>(id, o.rank, o.world);
}

enum Slot { kDispatch, kCombine, kDispatchSend, kDispatchRecv, kCombineSend, kCombineRecv, kSlots };
const char* kSlotNames[kSlots] = {"dispatch", "combine", "dispatch send", "dispatch recv",
                                  "combine send", "combine recv"};

void bench_config(const Options& o, Bootstrap& bs, StreamBarrier& barrier, int tokens) {
  A2AConfig cfg;
  cfg.max_num_tokens = tokens;
  cfg.num_experts = o.experts;
  cfg.experts_per_token = o.topk;
  cfg.rank = o.rank;
  cfg.world_size = o.world;
  cfg.dp_size = 1;
  cfg.hidden_dim = o.hidden;
  cfg.hidden_dim_bytes = o.fp8 ? o.hidden : o.hidden * 2;
  cfg.hidden_dim_scale_bytes = o.fp8 ? ceil_div(o.hidden, 128) * 4 : 0;
  auto ata = AllToAll::create(cfg, bs);
  const int nle = o.experts / o.world;
  const int cap = tokens * o.world;
  const int nscale = cfg.hidden_dim_scale_bytes / 4;

  std::mt19937 rng(1234 + o.rank);
  RankData<__nv_bfloat16> d(rng, tokens, o.experts, o.topk, 8, true);  // routing + weights only
  DeviceBuffer<uint8_t> x(static_cast<size_t>(tokens) * cfg.hidden_dim_bytes);
  DeviceBuffer<float> x_scale(static_cast<size_t>(tokens) * std::max(nscale, 1));
  DeviceBuffer<uint8_t> expert_x(static_cast<size_t>(nle) * cap * cfg.hidden_dim_bytes);
  DeviceBuffer<float> expert_scale(static_cast<size_t>(nle) * cap * std::max(nscale, 1));
  DeviceBuffer<__nv_bfloat16> expert_y(static_cast<size_t>(nle) * cap * o.hidden);
  DeviceBuffer<__nv_bfloat16> out(static_cast<size_t>(tokens) * o.hidden);
  DeviceBuffer<int32_t> counts(nle);
  auto indices = to_device(d.indices);
  auto weights = to_device(d.weights);
  auto bound_m = to_device(std::vector<uint32_t>{static_cast<uint32_t>(tokens)});

  DispatchCall dc;
  dc.out_num_tokens = counts.get();
  dc.out_x.data = expert_x.get();
  dc.out_x.stride_outer = static_cast<int64_t>(cap) * cfg.hidden_dim_bytes;
  dc.out_x.stride_row = cfg.hidden_dim_bytes;
  dc.out_rows = cap;
  dc.x.data = x.get();
  dc.x.stride_row = cfg.hidden_dim_bytes;
  if (o.fp8) {
    dc.out_scale.data = expert_scale.get();
    dc.out_scale.stride_outer = static_cast<int64_t>(cap) * nscale;
    dc.out_scale.stride_row = nscale;
    dc.out_scale.stride_col = 1;
    dc.x_scale.data = x_scale.get();
    dc.x_scale.stride_row = nscale;
    dc.x_scale.stride_col = 1;
  }
  dc.indices = indices.get();
  dc.bound_m = bound_m.get();
  dc.num_tokens = tokens;
  CombineCall cc;
  cc.out_tokens = out.get();
  cc.out_stride_row = o.hidden;
  cc.weights = weights.get();
  cc.w_stride_row = o.topk;
  cc.expert_y = expert_y.get();
  cc.y_stride_e = static_cast<int64_t>(cap) * o.hidden;
  cc.y_stride_row = o.hidden;
  cc.bound_m = bound_m.get();
  cc.num_tokens = tokens;
  cc.in = DType::kBF16;
  cc.out = DType::kBF16;

  cudaStream_t stream;
  CUDA_CHECK(cudaStreamCreate(&stream));
  const int n_events = kSlots + 1 + 4;  // see the sequence below
  std::vector<cudaEvent_t> ev(static_cast<size_t>(o.samples) * n_events);
  for (auto& e : ev) CUDA_CHECK(cudaEventCreate(&e));
  const uint64_t nap_ns = 100000;

  std::vector<std::vector<float>> times(kSlots);
  for (int rep = 0; rep < o.warmup + o.repeat; ++rep) {
    for (int s = 0; s < o.samples; ++s) {
      cudaEvent_t* e = &ev[static_cast<size_t>(s) * n_events];
      barrier.run(stream);
      CUDA_CHECK(cudaEventRecord(e[0], stream));
      ata->dispatch(dc, SplitMode::kNone, stream);
      CUDA_CHECK(cudaEventRecord(e[1], stream));
      ata->combine(cc, SplitMode::kNone, stream);
      CUDA_CHECK(cudaEventRecord(e[2], stream));
      barrier.run(stream);
      CUDA_CHECK(cudaEventRecord(e[3], stream));
      ata->dispatch(dc, SplitMode::kSend, stream);
      CUDA_CHECK(cudaEventRecord(e[4], stream));
      CUDA_CHECK(launch_sleep(nap_ns, stream));
      barrier.run(stream);
      CUDA_CHECK(cudaEventRecord(e[5], stream));
      ata->dispatch(dc, SplitMode::kRecv, stream);
      CUDA_CHECK(cudaEventRecord(e[6], stream));
      barrier.run(stream);
      CUDA_CHECK(cudaEventRecord(e[7], stream));
      ata->combine(cc, SplitMode::kSend, stream);
      CUDA_CHECK(cudaEventRecord(e[8], stream));
      CUDA_CHECK(launch_sleep(nap_ns, stream));
      barrier.run(stream);
      CUDA_CHECK(cudaEventRecord(e[9], stream));
      ata->combine(cc, SplitMode::kRecv, stream);
      CUDA_CHECK(cudaEventRecord(e[10], stream));
    }
    CUDA_CHECK(cudaStreamSynchronize(stream));
    if (rep < o.warmup) continue;
    const int pairs[kSlots][2] = {{0, 1}, {1, 2}, {3, 4}, {5, 6}, {7, 8}, {9, 10}};
    for (int s = 0; s < o.samples; ++s) {
      cudaEvent_t* e = &ev[static_cast<size_t>(s) * n_events];
      for (int k = 0; k < kSlots; ++k) {
        float ms = 0;
        CUDA_CHECK(cudaEventElapsedTime(&ms, e[pairs[k][0]], e[pairs[k][1]]));
        times[k].push_back(ms * 1e3f);
      }
    }
  }
  ata->check_status();

  // Per-rank summary -> maximum over ranks.
  double mine[kSlots * 3];
  for (int k = 0; k < kSlots; ++k) {
    const Stats st = stats(times[k]);
    mine[3 * k] = st.mean;
    mine[3 * k + 1] = st.stddev;
    mine[3 * k + 2] = st.p50;
  }
  std::vector<double> all(static_cast<size_t>(o.world) * kSlots * 3);
  bs.all_gather(mine, all.data(), sizeof(mine));
  if (o.rank == 0) {
    const double dispatch_bytes =
        static_cast<double>(tokens) * o.topk * (cfg.hidden_dim_bytes + cfg.hidden_dim_scale_bytes);
    const double combine_bytes = static_cast<double>(tokens) * o.topk * o.hidden * 2;
    std::printf("E=%d top-%d hidden=%d %s tokens/rank=%d EP=%d\n", o.experts, o.topk, o.hidden,
                o.fp8 ? "fp8+scales" : "bf16", tokens, o.world);
    for (int k = 0; k < kSlots; ++k) {
      double worst_mean = 0, worst_p50 = 0;
      for (int r = 0; r < o.world; ++r) {
        worst_mean = std::max(worst_mean, all[(static_cast<size_t>(r) * kSlots + k) * 3]);
        worst_p50 = std::max(worst_p50, all[(static_cast<size_t>(r) * kSlots + k) * 3 + 2]);
      }
      const double bytes = (k == kCombine || k == kCombineSend || k == kCombineRecv)
                               ? combine_bytes
                               : dispatch_bytes;
      std::printf("  %-14s rank0 %7.1f us +- %5.1f   max over ranks: mean %7.1f us  p50 %7.1f us"
                  "  %8.2f GB/s\n",
                  kSlotNames[k], mine[3 * k], mine[3 * k + 1], worst_mean, worst_p50,
                  bytes / worst_mean / 1e3);
    }
    std::fflush(stdout);
  }
  for (auto& e : ev) cudaEventDestroy(e);
  cudaStreamDestroy(stream);
  bs.barrier();
}

}  // namespace

int main(int argc, char** argv) {
  try {
    const Options o = parse(argc, argv);
    int devices = 0;
    CUDA_CHECK(cudaGetDeviceCount(&devices));
    PPLX_CHECK(devices > 0, "no CUDA device");
    CUDA_CHECK(cudaSetDevice(o.rank % devices));
    auto bs = make_bootstrap(o);
    StreamBarrier barrier(*bs);
    cudaProfilerStart();
    for (int tokens : o.tokens) {
      if (o.experts % o.world != 0) continue;
      bench_config(o, *bs, barrier, tokens);
    }
    cudaProfilerStop();
    bs->barrier();
  } catch (const std::exception& e) {
    std::fprintf(stderr, "bench_all_to_all: %s\n", e.what());
    return 1;
  }
  return 0;
}
