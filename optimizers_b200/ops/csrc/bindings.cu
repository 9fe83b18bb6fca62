// Python bindings of the sm_100a kernels.  Host-side work here is plan construction: TMA tensor
// maps, problem tables and tile lists are encoded once (when a parameter group is set up or its
// gradient selector changes) and uploaded; each step then only launches kernels.
#include <torch/extension.h>

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda.h>
#include <cuda_runtime.h>
#include <nvtx3/nvToolsExt.h>

#include <algorithm>
#include <array>
#include <map>
#include <memory>
#include <cstdlib>
#include <cstring>
#include <optional>
#include <string>
#include <vector>

#include "block_kernels.cuh"
#include "eig_kernels.cuh"
#include "flat_kernels.cuh"
#include "grouped_gemm.cuh"
#include "two_sided_apply.h"

namespace py = pybind11;
using namespace ob200;

namespace ob200 {
void register_model_ops(pybind11::module_& m);  // model_kernels.cu
}

namespace {

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn get_encode_fn() {
  static EncodeFn fn = nullptr;
  if (fn == nullptr) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t err = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres);
    TORCH_CHECK(err == cudaSuccess && sym != nullptr, "cuTensorMapEncodeTiled is not available from the driver");
    fn = reinterpret_cast<EncodeFn>(sym);
  }
  return fn;
}

// Tensor map of a K-major fp32 operand: `t` is a 2-D view [rows, K] whose last stride is 1.
CUtensorMap encode_operand(const torch::Tensor& t, int box_rows) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == torch::kFloat32 && t.dim() == 2, "operand must be a 2-D fp32 CUDA tensor");
  TORCH_CHECK(t.stride(1) == 1, "operand must be contiguous along K");
  TORCH_CHECK((t.stride(0) * 4) % 16 == 0, "operand row pitch must be a multiple of 16 bytes, got ", t.stride(0), " elements");
  TORCH_CHECK(reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 == 0, "operand base must be 16-byte aligned");
  CUtensorMap map;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(t.size(1)), static_cast<cuuint64_t>(t.size(0))};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(t.stride(0)) * 4};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(kBK), static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t elem_strides[2] = {1, 1};
  CUresult res = get_encode_fn()(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, t.data_ptr(), dims, strides, box,
                                 elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                 CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  TORCH_CHECK(res == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with code ", static_cast<int>(res));
  return map;
}

float* fptr(const std::optional<torch::Tensor>& t) {
  if (!t.has_value()) return nullptr;
  TORCH_CHECK(t->is_cuda() && t->scalar_type() == torch::kFloat32, "expected an fp32 CUDA tensor");
  return t->data_ptr<float>();
}

// Tracing of the native launches.  Bit 0 of the mode wraps every binding that launches kernels in
// an NVTX range named after it (visible to Nsight Systems / Nsight Compute range filters); bit 1
// brackets it with CUDA events on the current stream and accumulates the device time per name,
// read (after a synchronisation of the pending events) with launch_timings().  Both are off by
// default and cost one branch per call.
int g_trace_mode = 0;
constexpr int kTraceNvtx = 1, kTraceTiming = 2;

struct LaunchStat {
  int64_t count = 0;
  double ms = 0.0;
  std::vector<std::pair<cudaEvent_t, cudaEvent_t>> pending;
};
std::map<std::string, LaunchStat>& launch_stats() {
  static std::map<std::string, LaunchStat> stats;
  return stats;
}

void drain(LaunchStat& st) {
  for (auto& [begin, end] : st.pending) {
    float ms = 0.f;
    if (cudaEventSynchronize(end) == cudaSuccess && cudaEventElapsedTime(&ms, begin, end) == cudaSuccess) st.ms += ms;
    cudaEventDestroy(begin);
    cudaEventDestroy(end);
  }
  st.pending.clear();
}

class LaunchScope {
 public:
  explicit LaunchScope(const char* name) : name_(name), mode_(g_trace_mode) {
    if (mode_ == 0) return;
    if (mode_ & kTraceNvtx) nvtxRangePushA(name_);
    if (mode_ & kTraceTiming) {
      cudaEventCreate(&begin_);
      cudaEventCreate(&end_);
      cudaEventRecord(begin_, at::cuda::getCurrentCUDAStream());
    }
  }
  ~LaunchScope() {
    if (mode_ == 0) return;
    if (mode_ & kTraceTiming) {
      cudaEventRecord(end_, at::cuda::getCurrentCUDAStream());
      LaunchStat& st = launch_stats()[name_];
      st.count += 1;
      st.pending.emplace_back(begin_, end_);
      if (st.pending.size() >= 4096) drain(st);
    }
    if (mode_ & kTraceNvtx) nvtxRangePop();
  }
  LaunchScope(const LaunchScope&) = delete;
  LaunchScope& operator=(const LaunchScope&) = delete;

 private:
  const char* name_;
  int mode_;
  cudaEvent_t begin_ = nullptr, end_ = nullptr;
};

void set_launch_tracing(bool nvtx, bool timing) {
  g_trace_mode = (nvtx ? kTraceNvtx : 0) | (timing ? kTraceTiming : 0);
}

// name -> (calls, device milliseconds) since the last reset.
std::map<std::string, std::pair<int64_t, double>> launch_timings(bool reset) {
  std::map<std::string, std::pair<int64_t, double>> out;
  for (auto& [name, st] : launch_stats()) {
    drain(st);
    out[name] = {st.count, st.ms};
  }
  if (reset) launch_stats().clear();
  return out;
}

// Host table -> device, asynchronously on the current stream: the staging buffer is pinned and
// torch's host allocator keeps it alive until the copy has run, so building a launch table never
// drains the stream.
torch::Tensor upload_bytes(const void* src, size_t bytes, const torch::Device& device) {
  auto host = torch::empty({static_cast<int64_t>(std::max<size_t>(bytes, 1))}, torch::dtype(torch::kUInt8).pinned_memory(true));
  std::memcpy(host.data_ptr(), src, bytes);
  return host.to(device, /*non_blocking=*/true);
}

// Host-side assembly of grouped-GEMM launch tables.  Problems of any number of launches go into
// one device buffer laid out as [problem table][tensor maps]; a tensor map is encoded once per
// distinct array (pointer, extents, pitch) however many problems view it.  Each launch owns a
// contiguous range of the common tile list.
class PlanBuilder {
 public:
  struct Operand {
    const torch::Tensor* hi = nullptr;
    const torch::Tensor* lo = nullptr;  // may be null (single-product mode)
    int row0 = 0, k0 = 0;
  };
  struct Problem {
    Operand a, b;
    float* c = nullptr;
    float* d_hi = nullptr;
    float* d_lo = nullptr;
    float* sumsq = nullptr;
    int M = 0, N = 0, K = 0, ldc = 0, ldd = 0, flags = 0;
    long long push_offset = 0;
    bool upper_tiles_only = false;
  };

  void begin_launch() { launch_begin_ = static_cast<int>(problems_.size()); }

  void add(const Problem& q) {
    GemmProblem p;
    std::memset(&p, 0, sizeof(p));
    TORCH_CHECK(q.M > 0 && q.N > 0 && q.K > 0, "empty GEMM problem");
    for (const Operand* op : {&q.a, &q.b}) {
      const int64_t array_k = op->hi->size(1);
      TORCH_CHECK(op->k0 % 4 == 0 && op->k0 >= 0 && op->k0 + q.K <= array_k, "operand view exceeds its array along K");
      TORCH_CHECK(op->k0 + q.K == array_k || q.K % kBK == 0,
                  "an operand view that ends before its array along K needs K to be a multiple of ", kBK);
      TORCH_CHECK(op->row0 >= 0, "negative row origin");
    }
    TORCH_CHECK(q.a.row0 + q.M <= q.a.hi->size(0) && q.b.row0 + q.N <= q.b.hi->size(0), "operand view exceeds its array");
    device_ = q.a.hi->device();
    index_.push_back({map_of(*q.a.hi, kBM), q.a.lo != nullptr ? map_of(*q.a.lo, kBM) : -1, map_of(*q.b.hi, kBN),
                      q.b.lo != nullptr ? map_of(*q.b.lo, kBN) : -1});
    p.a_row0 = q.a.row0;
    p.a_k0 = q.a.k0;
    p.b_row0 = q.b.row0;
    p.b_k0 = q.b.k0;
    p.c = q.c;
    p.d_hi = q.d_hi;
    p.d_lo = q.d_lo;
    p.sumsq = q.sumsq;
    p.M = q.M;
    p.N = q.N;
    p.K = q.K;
    p.ldc = q.ldc;
    p.ldd = q.ldd;
    p.flags = q.flags;
    p.push_offset = q.push_offset;
    if (p.flags & kFlagPackedC) TORCH_CHECK(p.M == p.N && q.upper_tiles_only, "packed output needs a square upper-tile problem");
    if (p.flags & kFlagMirror) {
      TORCH_CHECK(p.M == p.N && q.upper_tiles_only && !(p.flags & kFlagPackedC),
                  "mirrored output needs a square, unpacked upper-tile problem");
    }
    if (!(p.flags & kFlagNoC)) TORCH_CHECK(p.c != nullptr, "C is required unless kFlagNoC is set");
    if (p.flags & kFlagSplitOut) TORCH_CHECK(p.d_hi != nullptr && p.d_lo != nullptr, "split output needs d_hi and d_lo");
    if (p.flags & (kFlagSumSq | kFlagTrace)) TORCH_CHECK(p.sumsq != nullptr, "sumsq output missing");
    problems_.push_back(p);
    upper_.push_back(q.upper_tiles_only);
  }

  // Closes the current launch: its tiles are appended to the tile list, longest K loops first so
  // that the persistent CTAs finish together.  Returns (first tile, number of tiles).
  std::pair<int64_t, int64_t> end_launch() {
    struct Order {
      int problem;
      int K;
    };
    std::vector<Order> order;
    for (int i = launch_begin_; i < static_cast<int>(problems_.size()); ++i) order.push_back({i, problems_[i].K});
    std::stable_sort(order.begin(), order.end(), [](const Order& x, const Order& y) { return x.K > y.K; });
    const int64_t first = static_cast<int64_t>(tiles_.size());
    // Tiles are issued in bands of kBandRows tile rows, column by column inside a band, so that
    // the tiles in flight together touch about 2 * sqrt(#SMs) operand panels instead of a
    // whole row of them: for K = 4096 a (hi, lo) panel is 4 MB and a full tile row of B panels
    // alone would exceed the L2.
    static const int kBandRows = [] {
      const char* env = std::getenv("OB200_GEMM_BAND_ROWS");  // tuning knob; 1 = plain row-major order
      const int v = env != nullptr ? std::atoi(env) : 12;
      return v > 0 ? v : 12;
    }();
    for (const Order& o : order) {
      const GemmProblem& p = problems_[o.problem];
      const bool upper = upper_[o.problem];
      for (int band = 0; band < p.M; band += kBandRows * kBM) {
        const int band_end = std::min(p.M, band + kBandRows * kBM);
        for (int n0 = upper ? band : 0; n0 < p.N; n0 += kBN) {
          for (int m0 = band; m0 < band_end; m0 += kBM) {
            if (upper && n0 < m0) continue;
            tiles_.push_back({o.problem, m0, n0, 0});
          }
        }
      }
    }
    launch_begin_ = static_cast<int>(problems_.size());
    return {first, static_cast<int64_t>(tiles_.size()) - first};
  }

  bool empty() const { return problems_.empty(); }

  // Uploads everything; returns (problem table + tensor maps, tile list).
  std::pair<torch::Tensor, torch::Tensor> finalize() {
    TORCH_CHECK(!problems_.empty(), "empty GEMM plan");
    const size_t table_bytes = problems_.size() * sizeof(GemmProblem);
    const size_t map_bytes = maps_.size() * sizeof(CUtensorMap);
    auto buffer = torch::empty({static_cast<int64_t>(table_bytes + map_bytes)}, torch::dtype(torch::kUInt8).device(device_));
    const auto base = reinterpret_cast<uintptr_t>(buffer.data_ptr());
    TORCH_CHECK(base % 128 == 0, "problem table must be 128-byte aligned");
    const auto* dev_maps = reinterpret_cast<const CUtensorMap*>(base + table_bytes);
    for (size_t i = 0; i < problems_.size(); ++i) {
      const auto& ix = index_[i];
      GemmProblem& p = problems_[i];
      p.a_hi = dev_maps + ix[0];
      p.a_lo = dev_maps + (ix[1] >= 0 ? ix[1] : ix[0]);
      p.b_hi = dev_maps + ix[2];
      p.b_lo = dev_maps + (ix[3] >= 0 ? ix[3] : ix[2]);
    }
    auto host = torch::empty({static_cast<int64_t>(table_bytes + map_bytes)}, torch::dtype(torch::kUInt8).pinned_memory(true));
    std::memcpy(host.data_ptr(), problems_.data(), table_bytes);
    std::memcpy(static_cast<uint8_t*>(host.data_ptr()) + table_bytes, maps_.data(), map_bytes);
    buffer.copy_(host, /*non_blocking=*/true);
    auto d_tiles = upload_bytes(tiles_.data(), tiles_.size() * sizeof(GemmTile), device_);
    return {buffer, d_tiles};
  }

 private:
  int map_of(const torch::Tensor& t, int box_rows) {
    const std::array<int64_t, 5> key = {reinterpret_cast<int64_t>(t.data_ptr()), t.size(0), t.size(1), t.stride(0), box_rows};
    auto it = cache_.find(key);
    if (it != cache_.end()) return it->second;
    maps_.push_back(encode_operand(t, box_rows));
    const int idx = static_cast<int>(maps_.size()) - 1;
    cache_.emplace(key, idx);
    return idx;
  }

  std::vector<GemmProblem> problems_;
  std::vector<std::array<int, 4>> index_;
  std::vector<bool> upper_;
  std::vector<GemmTile> tiles_;
  std::vector<CUtensorMap> maps_;
  std::map<std::array<int64_t, 5>, int> cache_;
  torch::Device device_{torch::kCPU};
  int launch_begin_ = 0;
};

// Holds the tensors of one Python GEMM spec alive while the builder refers to them.
struct SpecTensors {
  torch::Tensor a_hi, b_hi;
  std::optional<torch::Tensor> a_lo, b_lo, c, d_hi, d_lo, sumsq;
};

// Spec fields: (a_hi, a_lo | None, b_hi, b_lo | None, c | None, d_hi | None, d_lo | None, sumsq | None,
//               ldc, ldd, flags, upper_tiles_only [, push_offset [, (a_row0, a_k0, b_row0, b_k0, M, N, K)]])
// With the last field the operands are views, of the given origin and extent, of the arrays passed.
void add_spec(PlanBuilder& builder, const py::tuple& s, std::vector<std::unique_ptr<SpecTensors>>& keep) {
  TORCH_CHECK(s.size() >= 12 && s.size() <= 14, "GEMM spec must have 12 to 14 fields");
  keep.push_back(std::make_unique<SpecTensors>());
  SpecTensors& g = *keep.back();
  g.a_hi = s[0].cast<torch::Tensor>();
  g.a_lo = s[1].cast<std::optional<torch::Tensor>>();
  g.b_hi = s[2].cast<torch::Tensor>();
  g.b_lo = s[3].cast<std::optional<torch::Tensor>>();
  g.c = s[4].cast<std::optional<torch::Tensor>>();
  g.d_hi = s[5].cast<std::optional<torch::Tensor>>();
  g.d_lo = s[6].cast<std::optional<torch::Tensor>>();
  g.sumsq = s[7].cast<std::optional<torch::Tensor>>();
  PlanBuilder::Problem q;
  q.a.hi = &g.a_hi;
  q.a.lo = g.a_lo.has_value() ? &*g.a_lo : nullptr;
  q.b.hi = &g.b_hi;
  q.b.lo = g.b_lo.has_value() ? &*g.b_lo : nullptr;
  q.c = fptr(g.c);
  q.d_hi = fptr(g.d_hi);
  q.d_lo = fptr(g.d_lo);
  q.sumsq = fptr(g.sumsq);
  q.ldc = static_cast<int>(s[8].cast<int64_t>());
  q.ldd = static_cast<int>(s[9].cast<int64_t>());
  q.flags = static_cast<int>(s[10].cast<int64_t>());
  q.upper_tiles_only = s[11].cast<bool>();
  q.push_offset = s.size() >= 13 && !s[12].is_none() ? s[12].cast<int64_t>() : 0;
  if (q.flags & kFlagPeerPush) TORCH_CHECK(s.size() >= 13 && !s[12].is_none(), "a pushing problem needs its slot offset");
  if (q.flags & kFlagTrace) TORCH_CHECK(g.sumsq.has_value() && g.sumsq->numel() >= 2, "trace output needs a two-element sumsq");
  if (s.size() == 14 && !s[13].is_none()) {
    const auto view = s[13].cast<std::vector<int64_t>>();
    TORCH_CHECK(view.size() == 7, "operand view must be (a_row0, a_k0, b_row0, b_k0, M, N, K)");
    q.a.row0 = static_cast<int>(view[0]);
    q.a.k0 = static_cast<int>(view[1]);
    q.b.row0 = static_cast<int>(view[2]);
    q.b.k0 = static_cast<int>(view[3]);
    q.M = static_cast<int>(view[4]);
    q.N = static_cast<int>(view[5]);
    q.K = static_cast<int>(view[6]);
  } else {
    q.M = static_cast<int>(g.a_hi.size(0));
    q.N = static_cast<int>(g.b_hi.size(0));
    q.K = static_cast<int>(g.a_hi.size(1));
    TORCH_CHECK(g.b_hi.size(1) == q.K, "A and B must agree on K");
  }
  builder.add(q);
}

// Returns (problem table bytes, tile list bytes, number of tiles), the first two on the device.
std::tuple<torch::Tensor, torch::Tensor, int64_t> build_gemm_plan(const std::vector<py::tuple>& specs) {
  TORCH_CHECK(!specs.empty(), "empty GEMM plan");
  PlanBuilder builder;
  std::vector<std::unique_ptr<SpecTensors>> keep;
  builder.begin_launch();
  for (const py::tuple& s : specs) add_spec(builder, s, keep);
  const auto range = builder.end_launch();
  auto [table, tiles] = builder.finalize();
  return {table, tiles, range.second};
}

// Several launches in one table and one upload.  Returns (table, tiles, [(first tile, tiles), ...]);
// launch i runs with run_gemm_plan_range(table, tiles, first_i, count_i, ...).
std::tuple<torch::Tensor, torch::Tensor, std::vector<std::pair<int64_t, int64_t>>> build_gemm_plans(
    const std::vector<std::vector<py::tuple>>& launches) {
  PlanBuilder builder;
  std::vector<std::unique_ptr<SpecTensors>> keep;
  std::vector<std::pair<int64_t, int64_t>> ranges;
  for (const auto& specs : launches) {
    builder.begin_launch();
    for (const py::tuple& s : specs) add_spec(builder, s, keep);
    ranges.push_back(builder.end_launch());
  }
  auto [table, tiles] = builder.finalize();
  return {table, tiles, ranges};
}

void run_gemm_range(const torch::Tensor& problems, const torch::Tensor& tiles, int64_t first_tile, int64_t num_tiles,
                    double alpha, double beta, bool split, torch::Tensor status, double gamma) {
  LaunchScope scope("ob200::grouped_gemm");
  if (num_tiles <= 0) return;
  c10::cuda::CUDAGuard guard(problems.device());
  const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  launch_grouped_gemm(reinterpret_cast<const GemmProblem*>(problems.data_ptr()),
                      reinterpret_cast<const GemmTile*>(tiles.data_ptr()) + first_tile, static_cast<int>(num_tiles),
                      static_cast<float>(alpha), static_cast<float>(beta), split, status.data_ptr<int>(), sms,
                      at::cuda::getCurrentCUDAStream(), nullptr, static_cast<float>(gamma));
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

void run_gemm_plan(const torch::Tensor& problems, const torch::Tensor& tiles, int64_t num_tiles, double alpha,
                   double beta, bool split, torch::Tensor status, double gamma) {
  LaunchScope scope("ob200::grouped_gemm");
  c10::cuda::CUDAGuard guard(problems.device());
  const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  launch_grouped_gemm(reinterpret_cast<const GemmProblem*>(problems.data_ptr()),
                      reinterpret_cast<const GemmTile*>(tiles.data_ptr()), static_cast<int>(num_tiles),
                      static_cast<float>(alpha), static_cast<float>(beta), split, status.data_ptr<int>(), sms,
                      at::cuda::getCurrentCUDAStream(), nullptr, static_cast<float>(gamma));
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

// run_gemm_plan with the kFlagPeerPush problems storing into the gather buffers at `peer_bases`.
void run_gemm_plan_push(const torch::Tensor& problems, const torch::Tensor& tiles, int64_t num_tiles, double alpha,
                        double beta, bool split, torch::Tensor status, const std::vector<int64_t>& peer_bases,
                        int64_t send_dtype) {
  LaunchScope scope("ob200::grouped_gemm_push");
  c10::cuda::CUDAGuard guard(problems.device());
  TORCH_CHECK(peer_bases.size() <= 8, "at most 8 peers");
  PeerPush push{};
  push.num_peers = static_cast<int>(peer_bases.size());
  push.dtype = static_cast<int>(send_dtype);
  for (size_t r = 0; r < peer_bases.size(); ++r) push.base[r] = static_cast<unsigned long long>(peer_bases[r]);
  const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  launch_grouped_gemm(reinterpret_cast<const GemmProblem*>(problems.data_ptr()),
                      reinterpret_cast<const GemmTile*>(tiles.data_ptr()), static_cast<int>(num_tiles),
                      static_cast<float>(alpha), static_cast<float>(beta), split, status.data_ptr<int>(), sms,
                      at::cuda::getCurrentCUDAStream(), &push);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

// Block table.  Each spec: (param_view, grad_offset, grad_slot, m, n, n_pad, m_pad, m1, v, mom, z,
//                           g_hi, g_lo, gt_hi, gt_lo, f_hi, f_lo, p, norms, send_ptr, slot_offset, ev)
std::tuple<torch::Tensor, torch::Tensor, int64_t> build_block_table(const std::vector<py::tuple>& specs) {
  std::vector<BlockDesc> blocks(specs.size());
  std::vector<TileRef> tiles;
  torch::Device device(torch::kCPU);
  for (size_t i = 0; i < specs.size(); ++i) {
    const py::tuple& s = specs[i];
    TORCH_CHECK(s.size() == 23, "block spec must have 23 fields");
    BlockDesc& b = blocks[i];
    std::memset(&b, 0, sizeof(b));
    auto param = s[0].cast<torch::Tensor>();
    TORCH_CHECK(param.is_cuda() && param.scalar_type() == torch::kFloat32, "parameter blocks must be fp32 CUDA tensors");
    device = param.device();
    b.param = param.data_ptr<float>();
    b.grad_offset = s[1].cast<int64_t>();
    b.grad_slot = s[2].cast<int>();
    b.m = s[3].cast<int>();
    b.n = s[4].cast<int>();
    b.n_pad = s[5].cast<int>();
    b.m_pad = s[6].cast<int>();
    if (param.dim() == 2) {
      TORCH_CHECK(param.stride(1) == 1, "parameter block must be contiguous along its last dim");
      b.param_pitch = param.stride(0);
    } else {
      TORCH_CHECK(param.dim() == 1 && param.stride(0) == 1 && b.m == 1, "1-D blocks are presented as 1 x n");
      b.param_pitch = b.n;
    }
    auto opt = [&](int k) { return fptr(s[k].cast<std::optional<torch::Tensor>>()); };
    b.m1 = opt(7);
    b.v = opt(8);
    b.mom = opt(9);
    b.z = opt(10);
    b.g_hi = opt(11);
    b.g_lo = opt(12);
    b.gt_hi = opt(13);
    b.gt_lo = opt(14);
    b.f_hi = opt(15);
    b.f_lo = opt(16);
    b.p = opt(17);
    b.norms = opt(18);
    b.send = reinterpret_cast<void*>(s[19].cast<int64_t>());
    b.slot_offset = s[20].cast<int64_t>();
    b.ev = opt(21);
    b.aux = s[22].cast<int>();
  }
  // Tiles of 32 rows x 128 columns.
  for (size_t i = 0; i < specs.size(); ++i) {
    const BlockDesc& b = blocks[i];
    const int tm = (b.m + 31) / 32, tn = (b.n + 127) / 128;
    for (int ti = 0; ti < tm; ++ti)
      for (int tj = 0; tj < tn; ++tj) tiles.push_back({static_cast<int>(i), ti, tj, 0});
  }
  auto d_blocks = upload_bytes(blocks.data(), blocks.size() * sizeof(BlockDesc), device);
  auto d_tiles = upload_bytes(tiles.data(), tiles.size() * sizeof(TileRef), device);
  return {d_blocks, d_tiles, static_cast<int64_t>(tiles.size())};
}

inline const TileRef* tile_ptr(const torch::Tensor& tiles) { return reinterpret_cast<const TileRef*>(tiles.data_ptr()); }

void grad_prologue(const torch::Tensor& blocks, const torch::Tensor& tiles, int64_t num_tiles,
                   const torch::Tensor& grad_ptrs, double l2_weight_decay, double beta1, double beta3,
                   double bias_correction1, int64_t graft_kind, double graft_beta2, double graft_weight,
                   double graft_bc2, double graft_eps, bool write_split, torch::Tensor status,
                   int64_t num_grad_peers, double grad_scale) {
  LaunchScope scope("ob200::grad_prologue");
  c10::cuda::CUDAGuard guard(blocks.device());
  PrologueArgs a;
  a.blocks = reinterpret_cast<const BlockDesc*>(blocks.data_ptr());
  a.tiles = tile_ptr(tiles);
  a.num_tiles = static_cast<int>(num_tiles);
  a.grad_ptrs = reinterpret_cast<const float* const*>(grad_ptrs.data_ptr<int64_t>());
  a.l2_weight_decay = static_cast<float>(l2_weight_decay);
  a.beta1 = static_cast<float>(beta1);
  a.beta3 = static_cast<float>(beta3);
  a.bias_correction1 = static_cast<float>(bias_correction1);
  a.graft_kind = static_cast<int>(graft_kind);
  a.graft_beta2 = static_cast<float>(graft_beta2);
  a.graft_weight = static_cast<float>(graft_weight);
  a.graft_bias_correction2 = static_cast<float>(graft_bc2);
  a.graft_epsilon = static_cast<float>(graft_eps);
  a.write_split = write_split ? 1 : 0;
  a.status = status.data_ptr<int>();
  a.num_grad_peers = static_cast<int>(num_grad_peers);
  a.grad_scale = static_cast<float>(grad_scale);
  launch_grad_prologue(a, at::cuda::getCurrentCUDAStream());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

void direction_epilogue(const torch::Tensor& blocks, const torch::Tensor& tiles, int64_t num_tiles,
                        const torch::Tensor& lr, bool graft_only, int64_t graft_kind, double graft_bc2,
                        double graft_eps, double wd_alpha, bool primal_averaging, const torch::Tensor& mu_y,
                        const torch::Tensor& mu_x, bool classic_momentum, double momentum, double dampening,
                        bool nesterov, int64_t send_dtype, bool split_input, const std::vector<int64_t>& peer_bases,
                        bool send_params) {
  LaunchScope scope("ob200::direction_epilogue");
  c10::cuda::CUDAGuard guard(blocks.device());
  EpilogueArgs a;
  a.blocks = reinterpret_cast<const BlockDesc*>(blocks.data_ptr());
  a.tiles = tile_ptr(tiles);
  a.num_tiles = static_cast<int>(num_tiles);
  a.lr = lr.data_ptr<float>();
  a.send_params = send_params ? 1 : 0;
  a.graft_only = graft_only ? 1 : 0;
  a.graft_kind = static_cast<int>(graft_kind);
  a.graft_bias_correction2 = static_cast<float>(graft_bc2);
  a.graft_epsilon = static_cast<float>(graft_eps);
  a.wd_alpha = static_cast<float>(wd_alpha);
  a.primal_averaging = primal_averaging ? 1 : 0;
  a.mu_y = mu_y.data_ptr<float>();
  a.mu_x = mu_x.data_ptr<float>();
  a.classic_momentum = classic_momentum ? 1 : 0;
  a.momentum = static_cast<float>(momentum);
  a.dampening = static_cast<float>(dampening);
  a.nesterov = nesterov ? 1 : 0;
  a.send_dtype = static_cast<int>(send_dtype);
  a.split_input = split_input ? 1 : 0;
  TORCH_CHECK(peer_bases.size() <= 8, "at most 8 peers");
  a.num_push_peers = static_cast<int>(peer_bases.size());
  for (size_t r = 0; r < 8; ++r) a.peer_base[r] = r < peer_bases.size() ? static_cast<unsigned long long>(peer_bases[r]) : 0ull;
  launch_direction_epilogue(a, at::cuda::getCurrentCUDAStream());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

void gathered_apply(const torch::Tensor& blocks, const torch::Tensor& tiles, int64_t num_tiles, int64_t dtype,
                    bool copy_params, const std::optional<torch::Tensor>& status) {
  LaunchScope scope("ob200::gathered_apply");
  c10::cuda::CUDAGuard guard(blocks.device());
  launch_gathered_apply(reinterpret_cast<const BlockDesc*>(blocks.data_ptr()), tile_ptr(tiles),
                        static_cast<int>(num_tiles), static_cast<int>(dtype), nullptr, 0.f, copy_params,
                        status.has_value() ? status->data_ptr<int>() : nullptr, at::cuda::getCurrentCUDAStream());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

// The slots hold unscaled Shampoo directions P (pushed from the GEMM epilogue); BlockDesc::norms
// points at the block's grafting scale: W <- W - lr (scale P + wd_alpha W).
void gathered_apply_scaled(const torch::Tensor& blocks, const torch::Tensor& tiles, int64_t num_tiles, int64_t dtype,
                           const torch::Tensor& lr, double wd_alpha, const std::optional<torch::Tensor>& status) {
  LaunchScope scope("ob200::gathered_apply_scaled");
  c10::cuda::CUDAGuard guard(blocks.device());
  launch_gathered_apply(reinterpret_cast<const BlockDesc*>(blocks.data_ptr()), tile_ptr(tiles),
                        static_cast<int>(num_tiles), static_cast<int>(dtype), lr.data_ptr<float>(),
                        static_cast<float>(wd_alpha), false, status.has_value() ? status->data_ptr<int>() : nullptr,
                        at::cuda::getCurrentCUDAStream());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

void eig_scale(const torch::Tensor& blocks, const torch::Tensor& tiles, int64_t num_tiles, double bc2, double inv_root,
               double eps, bool write_split) {
  LaunchScope scope("ob200::eig_scale");
  c10::cuda::CUDAGuard guard(blocks.device());
  launch_eig_scale(reinterpret_cast<const BlockDesc*>(blocks.data_ptr()), tile_ptr(tiles),
                   static_cast<int>(num_tiles), static_cast<float>(bc2), static_cast<float>(inv_root),
                   static_cast<float>(eps), write_split ? 1 : 0, at::cuda::getCurrentCUDAStream());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

void mode_switch(const torch::Tensor& blocks, const torch::Tensor& tiles, int64_t num_tiles, double coeff, int64_t send_dtype) {
  LaunchScope scope("ob200::mode_switch");
  c10::cuda::CUDAGuard guard(blocks.device());
  launch_mode_switch(reinterpret_cast<const BlockDesc*>(blocks.data_ptr()), tile_ptr(tiles),
                     static_cast<int>(num_tiles), static_cast<float>(coeff), static_cast<int>(send_dtype),
                     at::cuda::getCurrentCUDAStream());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

void peer_barrier(torch::Tensor local_flags, const torch::Tensor& peer_flag_bases, int64_t my_rank, int64_t world,
                  int64_t seq, torch::Tensor status) {
  LaunchScope scope("ob200::peer_barrier");
  c10::cuda::CUDAGuard guard(local_flags.device());
  TORCH_CHECK(world <= 32, "peer barrier supports up to 32 ranks");
  launch_peer_barrier(local_flags.data_ptr<int>(),
                      reinterpret_cast<const unsigned long long*>(peer_flag_bases.data_ptr<int64_t>()),
                      static_cast<int>(my_rank), static_cast<int>(world), static_cast<int>(seq),
                      status.data_ptr<int>(), at::cuda::getCurrentCUDAStream());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

// Table for the grouped square-matrix passes.  Each spec: (src, dst_hi | None, dst_lo | None, err | None).
std::tuple<torch::Tensor, torch::Tensor, int64_t> build_mat_table(const std::vector<py::tuple>& specs) {
  std::vector<MatOp> ops(specs.size());
  std::vector<int2> chunks;
  torch::Device device(torch::kCPU);
  for (size_t i = 0; i < specs.size(); ++i) {
    const py::tuple& s = specs[i];
    auto src = s[0].cast<torch::Tensor>();
    TORCH_CHECK(src.is_cuda() && src.scalar_type() == torch::kFloat32 && src.dim() == 2 && src.stride(1) == 1 && src.size(0) == src.size(1));
    device = src.device();
    MatOp& op = ops[i];
    std::memset(&op, 0, sizeof(op));
    op.src = src.data_ptr<float>();
    op.d = static_cast<int>(src.size(0));
    op.ld_src = static_cast<int>(src.stride(0));
    auto hi = s[1].cast<std::optional<torch::Tensor>>();
    auto lo = s[2].cast<std::optional<torch::Tensor>>();
    if (hi.has_value()) {
      TORCH_CHECK(hi->dim() == 2 && hi->stride(1) == 1);
      op.dst_hi = hi->data_ptr<float>();
      op.ld_dst = static_cast<int>(hi->stride(0));
    }
    if (lo.has_value()) {
      TORCH_CHECK(hi.has_value() && lo->stride(0) == hi->stride(0));
      op.dst_lo = lo->data_ptr<float>();
    }
    op.err = fptr(s[3].cast<std::optional<torch::Tensor>>());
    for (int r = 0; r < (op.d + kMatRowsPerChunk - 1) / kMatRowsPerChunk; ++r) chunks.push_back(make_int2(static_cast<int>(i), r));
  }
  auto d_ops = upload_bytes(ops.data(), ops.size() * sizeof(MatOp), device);
  auto d_chunks = upload_bytes(chunks.data(), chunks.size() * sizeof(int2), device);
  return {d_ops, d_chunks, static_cast<int64_t>(chunks.size())};
}

void affine_identity_split(const torch::Tensor& ops, const torch::Tensor& chunks, int64_t num_chunks, double a, double b) {
  LaunchScope scope("ob200::affine_identity_split");
  c10::cuda::CUDAGuard guard(ops.device());
  launch_affine_identity_split(reinterpret_cast<const MatOp*>(ops.data_ptr()), reinterpret_cast<const int2*>(chunks.data_ptr()),
                               static_cast<int>(num_chunks), static_cast<float>(a), static_cast<float>(b),
                               at::cuda::getCurrentCUDAStream());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

void identity_error(const torch::Tensor& ops, const torch::Tensor& chunks, int64_t num_chunks) {
  LaunchScope scope("ob200::identity_error");
  c10::cuda::CUDAGuard guard(ops.device());
  launch_identity_error(reinterpret_cast<const MatOp*>(ops.data_ptr()), reinterpret_cast<const int2*>(chunks.data_ptr()),
                        static_cast<int>(num_chunks), at::cuda::getCurrentCUDAStream());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

// Exact-fp32 P = L G R for one block; the m x n intermediate comes from torch's allocator.
torch::Tensor two_sided_apply(const torch::Tensor& L, const torch::Tensor& G, const torch::Tensor& R) {
  LaunchScope scope("ob200::two_sided_apply");
  TORCH_CHECK(L.is_cuda() && G.is_cuda() && R.is_cuda(), "operands must be CUDA tensors");
  TORCH_CHECK(L.scalar_type() == torch::kFloat32 && G.scalar_type() == torch::kFloat32 && R.scalar_type() == torch::kFloat32);
  TORCH_CHECK(L.is_contiguous() && G.is_contiguous() && R.is_contiguous() && G.dim() == 2);
  const int m = static_cast<int>(G.size(0)), n = static_cast<int>(G.size(1));
  TORCH_CHECK(L.size(0) == m && L.size(1) == m && R.size(0) == n && R.size(1) == n, "shape mismatch");
  c10::cuda::CUDAGuard guard(G.device());
  auto scratch = torch::empty_like(G);
  auto P = torch::empty_like(G);
  launch_two_sided_apply(L.data_ptr<float>(), G.data_ptr<float>(), R.data_ptr<float>(), P.data_ptr<float>(),
                         scratch.data_ptr<float>(), m, n, at::cuda::getCurrentCUDAStream());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return P;
}

void tf32_split(const torch::Tensor& src, torch::Tensor hi, torch::Tensor lo) {
  LaunchScope scope("ob200::tf32_split");
  TORCH_CHECK(src.is_cuda() && src.scalar_type() == torch::kFloat32 && src.dim() == 2 && src.stride(1) == 1);
  TORCH_CHECK(hi.dim() == 2 && lo.dim() == 2 && hi.stride(1) == 1 && lo.stride(1) == 1);
  c10::cuda::CUDAGuard guard(src.device());
  launch_tf32_split(src.data_ptr<float>(), src.stride(0), hi.data_ptr<float>(), lo.data_ptr<float>(), hi.stride(0),
                    static_cast<int>(src.size(0)), static_cast<int>(src.size(1)), at::cuda::getCurrentCUDAStream());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

void gpa_adamw_step(const torch::Tensor& table, int64_t total_chunks, const torch::Tensor& chunk_map, double lr,
                    double beta1, double beta2, double eps, double bias_correction1, double bias_correction2,
                    double weight_decay, bool wd_on_y, double avg_coeff, double train_interp_coeff) {
  LaunchScope scope("ob200::gpa_adamw_step");
  c10::cuda::CUDAGuard guard(table.device());
  launch_gpa_adamw(reinterpret_cast<const GpaTensorDesc*>(table.data_ptr()),
                   reinterpret_cast<const int2*>(chunk_map.data_ptr()), static_cast<int>(total_chunks),
                   static_cast<float>(lr), static_cast<float>(beta1), static_cast<float>(beta2), static_cast<float>(eps),
                   static_cast<float>(bias_correction1), static_cast<float>(bias_correction2),
                   static_cast<float>(weight_decay), wd_on_y, static_cast<float>(avg_coeff),
                   static_cast<float>(train_interp_coeff), at::cuda::getCurrentCUDAStream());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

void gpa_lerp(const torch::Tensor& table, int64_t total_chunks, const torch::Tensor& chunk_map, double weight) {
  LaunchScope scope("ob200::gpa_lerp");
  c10::cuda::CUDAGuard guard(table.device());
  launch_gpa_lerp(reinterpret_cast<const GpaTensorDesc*>(table.data_ptr()), reinterpret_cast<const int2*>(chunk_map.data_ptr()),
                  static_cast<int>(total_chunks), static_cast<float>(weight), at::cuda::getCurrentCUDAStream());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

// Table for the GPA-AdamW kernels.  Each spec: (param, grad, z, exp_avg, exp_avg_sq); params may be
// fp32, bf16 or fp16 (grad of the same dtype); state is fp32.
std::tuple<torch::Tensor, torch::Tensor, int64_t> build_gpa_table(const std::vector<py::tuple>& specs) {
  std::vector<GpaTensorDesc> descs(specs.size());
  std::vector<int2> chunks;
  torch::Device device(torch::kCPU);
  for (size_t i = 0; i < specs.size(); ++i) {
    const py::tuple& s = specs[i];
    auto p = s[0].cast<torch::Tensor>();
    auto g = s[1].cast<std::optional<torch::Tensor>>();
    auto z = s[2].cast<torch::Tensor>();
    auto m = s[3].cast<torch::Tensor>();
    auto v = s[4].cast<torch::Tensor>();
    TORCH_CHECK(p.is_cuda() && p.is_contiguous() && z.is_contiguous() && m.is_contiguous() && v.is_contiguous());
    device = p.device();
    GpaTensorDesc& d = descs[i];
    d.param = p.data_ptr();
    d.grad = g.has_value() ? g->data_ptr() : nullptr;
    if (g.has_value()) TORCH_CHECK(g->is_contiguous() && g->scalar_type() == p.scalar_type());
    d.z = z.data_ptr<float>();
    d.m = m.data_ptr<float>();
    d.v = v.data_ptr<float>();
    d.numel = p.numel();
    d.dtype = p.scalar_type() == torch::kFloat32 ? 0 : (p.scalar_type() == torch::kBFloat16 ? 1 : 2);
    TORCH_CHECK(p.scalar_type() == torch::kFloat32 || p.scalar_type() == torch::kBFloat16 || p.scalar_type() == torch::kFloat16);
    const int64_t n_chunks = (d.numel + kGpaChunk - 1) / kGpaChunk;
    for (int64_t c = 0; c < n_chunks; ++c) chunks.push_back(make_int2(static_cast<int>(i), static_cast<int>(c)));
  }
  auto d_descs = upload_bytes(descs.data(), descs.size() * sizeof(GpaTensorDesc), device);
  auto d_chunks = upload_bytes(chunks.data(), chunks.size() * sizeof(int2), device);
  return {d_descs, d_chunks, static_cast<int64_t>(chunks.size())};
}

// specs: (source address, destination address, bytes); addresses may belong to peer GPUs.
std::tuple<torch::Tensor, torch::Tensor, int64_t> build_copy_table(const std::vector<std::tuple<int64_t, int64_t, int64_t>>& specs,
                                                                   int64_t device_index) {
  std::vector<CopyDesc> descs;
  std::vector<int2> chunks;
  for (const auto& [src, dst, bytes] : specs) {
    TORCH_CHECK(bytes >= 0 && bytes % 4 == 0 && (src % 4) == 0 && (dst % 4) == 0, "peer_copy: 4-byte granularity");
    if (bytes == 0) continue;
    const int idx = static_cast<int>(descs.size());
    descs.push_back({reinterpret_cast<const void*>(src), reinterpret_cast<void*>(dst), bytes});
    const int64_t n_chunks = (bytes + kCopyChunkBytes - 1) / kCopyChunkBytes;
    for (int64_t c = 0; c < n_chunks; ++c) chunks.push_back(make_int2(idx, static_cast<int>(c)));
  }
  torch::Device device(torch::kCUDA, static_cast<c10::DeviceIndex>(device_index));
  auto d_descs = upload_bytes(descs.data(), descs.size() * sizeof(CopyDesc), device);
  auto d_chunks = upload_bytes(chunks.data(), chunks.size() * sizeof(int2), device);
  return {d_descs, d_chunks, static_cast<int64_t>(chunks.size())};
}

// Eigendecomposition of a list of small symmetric fp32 matrices (n <= 128) in one launch.
// Returns (eigenvalue tensors, eigenvector tensors, sweeps used per matrix as a device int tensor).
std::tuple<std::vector<torch::Tensor>, std::vector<torch::Tensor>, torch::Tensor> jacobi_eigh(
    const std::vector<torch::Tensor>& mats, int64_t max_sweeps, double tol) {
  LaunchScope scope("ob200::jacobi_eigh");
  TORCH_CHECK(!mats.empty(), "jacobi_eigh: empty batch");
  const auto device = mats[0].device();
  c10::cuda::CUDAGuard guard(device);
  std::vector<JacobiDesc> descs(mats.size());
  std::vector<torch::Tensor> lams, qs;
  for (size_t i = 0; i < mats.size(); ++i) {
    const auto& a = mats[i];
    TORCH_CHECK(a.is_cuda() && a.scalar_type() == torch::kFloat32 && a.dim() == 2 && a.size(0) == a.size(1) &&
                    a.stride(1) == 1 && a.size(0) <= kJacobiMaxN && a.size(0) >= 1,
                "jacobi_eigh: square fp32 CUDA matrices of size <= ", kJacobiMaxN);
    const int64_t n = a.size(0);
    lams.push_back(torch::empty({n}, a.options()));
    qs.push_back(torch::empty({n, n}, a.options()));
    descs[i] = {a.data_ptr<float>(), qs.back().data_ptr<float>(), lams.back().data_ptr<float>(), static_cast<int>(n),
                static_cast<int>(a.stride(0)), static_cast<int>(n), 0, 0.f, 0};
  }
  auto d_descs = upload_bytes(descs.data(), descs.size() * sizeof(JacobiDesc), device);
  auto sweeps = torch::zeros({static_cast<int64_t>(mats.size())}, torch::dtype(torch::kInt32).device(device));
  launch_jacobi_eigh(reinterpret_cast<const JacobiDesc*>(d_descs.data_ptr()), static_cast<int>(mats.size()),
                     static_cast<int>(max_sweeps), static_cast<float>(tol), sweeps.data_ptr<int>(),
                     at::cuda::getCurrentCUDAStream());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {lams, qs, sweeps};
}

// jacobi_eigh writing into caller-provided storage: qs[i] is an n x n view (any row pitch) that
// receives the eigenvectors as columns (or as rows with `transposed`), lams[i] an n-vector.
// `shift_scale` > 0 (JacobiDesc::shift_scale) makes the kernel robust on singular and indefinite
// matrices at the price of absolute instead of relative accuracy of the small eigenvalues.
torch::Tensor jacobi_eigh_into(const std::vector<torch::Tensor>& mats, const std::vector<torch::Tensor>& qs,
                               const std::vector<torch::Tensor>& lams, bool transposed, int64_t max_sweeps, double tol,
                               double shift_scale) {
  LaunchScope scope("ob200::jacobi_eigh_into");
  TORCH_CHECK(!mats.empty() && mats.size() == qs.size() && mats.size() == lams.size(), "jacobi_eigh_into: list sizes");
  const auto device = mats[0].device();
  c10::cuda::CUDAGuard guard(device);
  std::vector<JacobiDesc> descs(mats.size());
  for (size_t i = 0; i < mats.size(); ++i) {
    const auto& a = mats[i];
    const auto& q = qs[i];
    const auto& l = lams[i];
    TORCH_CHECK(a.is_cuda() && a.scalar_type() == torch::kFloat32 && a.dim() == 2 && a.size(0) == a.size(1) &&
                    a.stride(1) == 1 && a.size(0) <= kJacobiMaxN && a.size(0) >= 1,
                "jacobi_eigh_into: square fp32 CUDA matrices of size <= ", kJacobiMaxN);
    const int64_t n = a.size(0);
    TORCH_CHECK(q.scalar_type() == torch::kFloat32 && q.dim() == 2 && q.size(0) == n && q.size(1) == n && q.stride(1) == 1);
    TORCH_CHECK(l.scalar_type() == torch::kFloat32 && l.dim() == 1 && l.size(0) == n && l.stride(0) == 1);
    descs[i] = {a.data_ptr<float>(), q.data_ptr<float>(), l.data_ptr<float>(), static_cast<int>(n),
                static_cast<int>(a.stride(0)), static_cast<int>(q.stride(0)), transposed ? 1 : 0,
                static_cast<float>(shift_scale), 0};
  }
  auto d_descs = upload_bytes(descs.data(), descs.size() * sizeof(JacobiDesc), device);
  auto sweeps = torch::zeros({static_cast<int64_t>(mats.size())}, torch::dtype(torch::kInt32).device(device));
  launch_jacobi_eigh(reinterpret_cast<const JacobiDesc*>(d_descs.data_ptr()), static_cast<int>(mats.size()),
                     static_cast<int>(max_sweeps), static_cast<float>(tol), sweeps.data_ptr<int>(),
                     at::cuda::getCurrentCUDAStream());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return sweeps;
}

// Panels of the blocked Householder QR, for driving the panel kernel on its own.
// Each spec: (ct, n, c0, c1, vt, ttv, tv) with vt / ttv / tv of shape [QR_PANEL, n - c0] and one pitch.
torch::Tensor build_qr_panel_table(const std::vector<py::tuple>& specs) {
  std::vector<QrPanelDesc> descs(specs.size());
  torch::Device device(torch::kCPU);
  for (size_t i = 0; i < specs.size(); ++i) {
    const py::tuple& s = specs[i];
    TORCH_CHECK(s.size() == 7, "QR panel spec must have 7 fields");
    auto ct = s[0].cast<torch::Tensor>();
    TORCH_CHECK(ct.is_cuda() && ct.scalar_type() == torch::kFloat32 && ct.dim() == 2 && ct.stride(1) == 1);
    device = ct.device();
    QrPanelDesc& d = descs[i];
    std::memset(&d, 0, sizeof(d));
    d.ct = ct.data_ptr<float>();
    d.ld = static_cast<int>(ct.stride(0));
    d.n = s[1].cast<int>();
    d.c0 = s[2].cast<int>();
    d.c1 = s[3].cast<int>();
    TORCH_CHECK(d.c0 >= 0 && d.c1 > d.c0 && d.c1 - d.c0 <= kQrPanel && d.c1 <= d.n && d.c1 <= ct.size(0) && d.n <= ct.size(1),
                "QR panel bounds");
    const int L = d.n - d.c0;
    auto get = [&](int k) {
      auto t = s[k].cast<torch::Tensor>();
      TORCH_CHECK(t.is_cuda() && t.scalar_type() == torch::kFloat32 && t.dim() == 2 && t.stride(1) == 1 &&
                      t.size(0) >= kQrPanel && t.size(1) >= L,
                  "QR panel operand ", k, " too small");
      return t;
    };
    auto vt = get(4), ttv = get(5), tv = get(6);
    d.ldw = static_cast<int>(vt.stride(0));
    TORCH_CHECK(ttv.stride(0) == d.ldw && tv.stride(0) == d.ldw, "common pitch");
    d.vt = vt.data_ptr<float>();
    d.ttv = ttv.data_ptr<float>();
    d.tv = tv.data_ptr<float>();
  }
  return upload_bytes(descs.data(), descs.size() * sizeof(QrPanelDesc), device);
}

void householder_panel(const torch::Tensor& table, int64_t count) {
  LaunchScope scope("ob200::householder_panel");
  c10::cuda::CUDAGuard guard(table.device());
  launch_householder_panel(reinterpret_cast<const QrPanelDesc*>(table.data_ptr()), static_cast<int>(count),
                           at::cuda::getCurrentCUDAStream());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

// Blocked Householder QR of a batch of matrices, entirely on the device and without host
// synchronisation: for every panel of kQrPanel columns one launch of the panel kernel over all
// matrices that still have such a panel, then one launch of the block-reflector kernel that
// applies it to the remaining columns (C <- C - (C V T) V^T in the transposed storage); one more
// launch then accumulates Q^T of every matrix, each CTA carrying a tile of rows of the identity
// through all panels' reflectors in shared memory.  All launch tables are assembled here and
// uploaded once.
//
// Each spec: (ct, n, k, zt, zt_hi, zt_lo)
//   ct                [>= k, n] view (row pitch a multiple of 4): row c is column c of the n x k matrix
//                     to factor; overwritten (R and reflectors, LAPACK geqrf layout transposed)
//   zt, zt_hi, zt_lo  [n, n] views of one pitch: receive Q^T of the full n x n orthogonal factor, plain
//                     and as a tf32 (hi, lo) pair; its first k rows span the columns of the matrix, the
//                     others their complement
// Replaces torch.linalg.qr (cuSOLVER geqrf + orgqr) of the reference's QR iteration
// (distributed_shampoo/preconditioner/matrix_functions.py:843).
void householder_qr(const std::vector<py::tuple>& specs) {
  LaunchScope scope("ob200::householder_qr");
  TORCH_CHECK(!specs.empty(), "householder_qr: empty batch");
  struct Item {
    torch::Tensor ct, zt, zt_hi, zt_lo, vt, ttv, tv;
    int n = 0, k = 0, npan = 0, q_rows = 0;
  };
  std::vector<Item> items(specs.size());
  int max_pan = 0;
  torch::Device device(torch::kCPU);
  for (size_t i = 0; i < specs.size(); ++i) {
    const py::tuple& s = specs[i];
    TORCH_CHECK(s.size() == 6 || s.size() == 7, "householder_qr spec must have 6 or 7 fields");
    Item& it = items[i];
    it.ct = s[0].cast<torch::Tensor>();
    it.n = s[1].cast<int>();
    it.k = s[2].cast<int>();
    it.zt = s[3].cast<torch::Tensor>();
    it.zt_hi = s[4].cast<torch::Tensor>();
    it.zt_lo = s[5].cast<torch::Tensor>();
    TORCH_CHECK(it.k >= 1 && it.k <= it.n, "householder_qr: need 1 <= k <= n");
    // Optional 7th field: only the first q_rows rows of Q^T (the first q_rows columns of Q) are wanted.
    it.q_rows = s.size() == 7 ? s[6].cast<int>() : it.n;
    TORCH_CHECK(it.q_rows >= 1 && it.q_rows <= it.n, "householder_qr: need 1 <= q_rows <= n");
    TORCH_CHECK(it.n <= kReflectSmemFloats, "householder_qr: n too large for the row-tile kernel");
    TORCH_CHECK(it.ct.is_cuda() && it.ct.scalar_type() == torch::kFloat32 && it.ct.dim() == 2 && it.ct.stride(1) == 1 &&
                    it.ct.size(0) >= it.k && it.ct.size(1) == it.n,
                "householder_qr: ct must be a [>= k, n] fp32 view");
    for (const torch::Tensor* t : {&it.zt, &it.zt_hi, &it.zt_lo}) {
      TORCH_CHECK(t->is_cuda() && t->scalar_type() == torch::kFloat32 && t->dim() == 2 && t->stride(1) == 1 &&
                      t->size(0) >= it.q_rows && t->size(1) == it.n && t->stride(0) == it.zt.stride(0),
                  "householder_qr: zt arrays must be [>= q_rows, n] fp32 views with one pitch");
    }
    device = it.ct.device();
    it.npan = (it.k + kQrPanel - 1) / kQrPanel;
    max_pan = std::max(max_pan, it.npan);
    // kReflectChunk columns of slack per row: the reflector kernel copies whole chunks
    const int64_t k16 = static_cast<int64_t>(it.npan) * kQrPanel, ldw = (it.n + 3) / 4 * 4 + kReflectChunk;
    it.vt = torch::empty({k16, ldw}, it.ct.options());
    it.ttv = torch::empty({k16, ldw}, it.ct.options());
    it.tv = torch::empty({k16, ldw}, it.ct.options());
  }
  c10::cuda::CUDAGuard guard(device);
  auto stream = at::cuda::getCurrentCUDAStream();

  // Launch tables, panel-major: panel descriptors, then the reflector applications of the forward
  // with their row tiles.
  std::vector<QrPanelDesc> panels;
  std::vector<ReflectDesc> reflect;
  std::vector<int2> tiles;
  struct Range {
    int first = 0, count = 0;
  };
  std::vector<Range> panel_range(max_pan), fwd_range(max_pan);
  auto add_reflect = [&](float* x, float* x_hi, float* x_lo, int ldx, int rows, int L, const float* w, const float* vt,
                         int ldw) {
    ReflectDesc r;
    std::memset(&r, 0, sizeof(r));
    r.x = x;
    r.x_hi = x_hi;
    r.x_lo = x_lo;
    r.w = w;
    r.vt = vt;
    r.ldx = ldx;
    r.ldw = ldw;
    r.rows = rows;
    r.L = L;
    r.rows_per_tile = std::max(1, std::min(kReflectMaxRows, kReflectSmemFloats / L));
    const int idx = static_cast<int>(reflect.size());
    reflect.push_back(r);
    for (int row0 = 0; row0 < rows; row0 += r.rows_per_tile) tiles.push_back(make_int2(idx, row0));
  };
  for (int j = 0; j < max_pan; ++j) {
    const int panel_first = static_cast<int>(panels.size());
    const int tile_first = static_cast<int>(tiles.size());
    for (const Item& it : items) {
      if (j >= it.npan) continue;
      const int c0 = j * kQrPanel, c1 = std::min(it.k, c0 + kQrPanel), L = it.n - c0;
      const int ldw = static_cast<int>(it.vt.stride(0));
      const int64_t w_off = static_cast<int64_t>(c0) * ldw + c0;  // panel row 0, column c0
      QrPanelDesc d;
      std::memset(&d, 0, sizeof(d));
      d.ct = it.ct.data_ptr<float>();
      d.ld = static_cast<int>(it.ct.stride(0));
      d.n = it.n;
      d.c0 = c0;
      d.c1 = c1;
      d.ldw = ldw;
      d.vt = it.vt.data_ptr<float>() + w_off;
      d.ttv = it.ttv.data_ptr<float>() + w_off;
      d.tv = it.tv.data_ptr<float>() + w_off;
      panels.push_back(d);
      if (it.k > c1) {
        const int64_t ld = it.ct.stride(0);
        add_reflect(it.ct.data_ptr<float>() + c1 * ld + c0, nullptr, nullptr, static_cast<int>(ld), it.k - c1, L,
                    it.ttv.data_ptr<float>() + w_off, it.vt.data_ptr<float>() + w_off, ldw);
      }
    }
    panel_range[j] = {panel_first, static_cast<int>(panels.size()) - panel_first};
    fwd_range[j] = {tile_first, static_cast<int>(tiles.size()) - tile_first};
  }
  // Accumulation of Q^T: one descriptor per matrix, tiles of whole rows.
  std::vector<AccumulateDesc> accumulate;
  std::vector<int2> acc_tiles;
  for (const Item& it : items) {
    AccumulateDesc a;
    std::memset(&a, 0, sizeof(a));
    a.zt = it.zt.data_ptr<float>();
    a.zt_hi = it.zt_hi.data_ptr<float>();
    a.zt_lo = it.zt_lo.data_ptr<float>();
    a.vt = it.vt.data_ptr<float>();
    a.tv = it.tv.data_ptr<float>();
    a.ldz = static_cast<int>(it.zt.stride(0));
    a.ldw = static_cast<int>(it.vt.stride(0));
    a.n = it.n;
    a.npan = it.npan;
    a.rows_per_tile = std::max(1, std::min(kReflectMaxRows, kReflectSmemFloats / it.n));
    a.q_rows = it.q_rows;
    const int idx = static_cast<int>(accumulate.size());
    accumulate.push_back(a);
    for (int row0 = 0; row0 < it.q_rows; row0 += a.rows_per_tile) acc_tiles.push_back(make_int2(idx, row0));
  }
  auto d_panels = upload_bytes(panels.data(), panels.size() * sizeof(QrPanelDesc), device);
  auto d_reflect = upload_bytes(reflect.data(), reflect.size() * sizeof(ReflectDesc), device);
  auto d_tiles = upload_bytes(tiles.data(), tiles.size() * sizeof(int2), device);
  const auto* panel_table = reinterpret_cast<const QrPanelDesc*>(d_panels.data_ptr());
  const auto* reflect_table = reinterpret_cast<const ReflectDesc*>(d_reflect.data_ptr());
  const auto* tile_table = reinterpret_cast<const int2*>(d_tiles.data_ptr());

  auto d_accumulate = upload_bytes(accumulate.data(), accumulate.size() * sizeof(AccumulateDesc), device);
  auto d_acc_tiles = upload_bytes(acc_tiles.data(), acc_tiles.size() * sizeof(int2), device);

  for (int j = 0; j < max_pan; ++j) {
    launch_householder_panel(panel_table + panel_range[j].first, panel_range[j].count, stream);
    launch_apply_block_reflector(reflect_table, tile_table + fwd_range[j].first, fwd_range[j].count, stream);
  }
  launch_accumulate_q(reinterpret_cast<const AccumulateDesc*>(d_accumulate.data_ptr()),
                      reinterpret_cast<const int2*>(d_acc_tiles.data_ptr()), static_cast<int>(acc_tiles.size()), stream);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  // The launch tables and the workspace are referenced by kernels still in flight: torch's caching
  // allocator only reuses their memory for work queued later on this same stream.
}

// One allocation for a batch of matrices in padded storage: matrix i is rows[i] x cols[i] with row
// pitch pad4(cols[i]), as its plain array and / or its tf32 (hi, lo) pair, every array starting on a
// 16-byte boundary.  Returns (plain | None, hi | None, lo | None) per matrix.  The eigensolver
// creates tens of thousands of such scratch matrices per refresh; making the views here instead of
// one allocation and three as_strided calls per matrix in Python removes most of that host time.
std::vector<std::tuple<std::optional<torch::Tensor>, std::optional<torch::Tensor>, std::optional<torch::Tensor>>>
alloc_mat_batch(const std::vector<int64_t>& rows, const std::vector<int64_t>& cols, bool plain, bool pair,
                const torch::Device& device) {
  TORCH_CHECK(rows.size() == cols.size(), "alloc_mat_batch: rows and cols differ in length");
  TORCH_CHECK(plain || pair, "alloc_mat_batch: nothing to allocate");
  const int count = (plain ? 1 : 0) + (pair ? 2 : 0);
  int64_t total = 0;
  for (size_t i = 0; i < rows.size(); ++i) total += count * rows[i] * ((cols[i] + 3) / 4 * 4);
  auto block = torch::empty({std::max<int64_t>(total, 1)}, torch::TensorOptions().dtype(torch::kFloat32).device(device));
  std::vector<std::tuple<std::optional<torch::Tensor>, std::optional<torch::Tensor>, std::optional<torch::Tensor>>> out;
  out.reserve(rows.size());
  int64_t offset = 0;
  for (size_t i = 0; i < rows.size(); ++i) {
    const int64_t r = rows[i], c = cols[i], ld = (c + 3) / 4 * 4;
    std::optional<torch::Tensor> views[3];
    for (int k = 0; k < 3; ++k) {
      const bool want = k == 0 ? plain : pair;
      if (!want) continue;
      views[k] = block.as_strided({r, c}, {ld, 1}, offset);
      offset += r * ld;
    }
    out.emplace_back(std::move(views[0]), std::move(views[1]), std::move(views[2]));
  }
  return out;
}

// Table for the per-matrix passes of the eigensolver.  Each spec: (src, dst_hi | None, dst_lo | None,
// stats | None, a, b).
std::tuple<torch::Tensor, torch::Tensor, int64_t> build_sym_table(const std::vector<py::tuple>& specs) {
  std::vector<SymOp> ops(specs.size());
  std::vector<int2> chunks;
  torch::Device device(torch::kCPU);
  for (size_t i = 0; i < specs.size(); ++i) {
    const py::tuple& s = specs[i];
    TORCH_CHECK(s.size() == 6, "sym spec must have 6 fields");
    auto src = s[0].cast<torch::Tensor>();
    TORCH_CHECK(src.is_cuda() && src.scalar_type() == torch::kFloat32 && src.dim() == 2 && src.stride(1) == 1 && src.size(0) == src.size(1));
    device = src.device();
    SymOp& op = ops[i];
    std::memset(&op, 0, sizeof(op));
    op.src = src.data_ptr<float>();
    op.n = static_cast<int>(src.size(0));
    op.ld_src = static_cast<int>(src.stride(0));
    auto hi = s[1].cast<std::optional<torch::Tensor>>();
    auto lo = s[2].cast<std::optional<torch::Tensor>>();
    if (hi.has_value()) {
      TORCH_CHECK(hi->dim() == 2 && hi->stride(1) == 1 && hi->size(0) >= op.n && hi->size(1) >= op.n);
      op.dst_hi = hi->data_ptr<float>();
      op.ld_dst = static_cast<int>(hi->stride(0));
    }
    if (lo.has_value()) {
      TORCH_CHECK(hi.has_value() && lo->stride(0) == hi->stride(0));
      op.dst_lo = lo->data_ptr<float>();
    }
    auto stats = s[3].cast<std::optional<torch::Tensor>>();
    if (stats.has_value()) {
      TORCH_CHECK(stats->numel() >= 2 && stats->is_contiguous());
      op.stats = fptr(stats);
    }
    op.a = s[4].cast<float>();
    op.b = s[5].cast<float>();
    for (int r = 0; r < (op.n + kSymRowsPerChunk - 1) / kSymRowsPerChunk; ++r) chunks.push_back(make_int2(static_cast<int>(i), r));
  }
  auto d_ops = upload_bytes(ops.data(), ops.size() * sizeof(SymOp), device);
  auto d_chunks = upload_bytes(chunks.data(), chunks.size() * sizeof(int2), device);
  return {d_ops, d_chunks, static_cast<int64_t>(chunks.size())};
}

void sym_measure(const torch::Tensor& ops, int64_t count) {
  LaunchScope scope("ob200::sym_measure");
  c10::cuda::CUDAGuard guard(ops.device());
  launch_sym_measure(reinterpret_cast<const SymOp*>(ops.data_ptr()), static_cast<int>(count), at::cuda::getCurrentCUDAStream());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

void sq_offdiag(const torch::Tensor& ops, int64_t count) {
  LaunchScope scope("ob200::sq_offdiag");
  c10::cuda::CUDAGuard guard(ops.device());
  launch_sq_offdiag(reinterpret_cast<const SymOp*>(ops.data_ptr()), static_cast<int>(count), at::cuda::getCurrentCUDAStream());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

void shift_scale_split(const torch::Tensor& ops, const torch::Tensor& chunks, int64_t num_chunks) {
  LaunchScope scope("ob200::shift_scale_split");
  c10::cuda::CUDAGuard guard(ops.device());
  launch_shift_scale_split(reinterpret_cast<const SymOp*>(ops.data_ptr()), reinterpret_cast<const int2*>(chunks.data_ptr()),
                           static_cast<int>(num_chunks), at::cuda::getCurrentCUDAStream());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

// Each spec: (src, d, dst_hi, dst_lo | None): src is the packed upper triangle (1-D, d (d + 1) / 2
// elements) or the full d x d matrix (2-D) of a symmetric matrix; dst_* are d x d views.
std::tuple<torch::Tensor, torch::Tensor, int64_t> build_unpack_table(const std::vector<py::tuple>& specs) {
  std::vector<UnpackOp> ops(specs.size());
  std::vector<int2> chunks;
  torch::Device device(torch::kCPU);
  for (size_t i = 0; i < specs.size(); ++i) {
    const py::tuple& s = specs[i];
    TORCH_CHECK(s.size() == 4, "unpack spec must have 4 fields");
    auto src = s[0].cast<torch::Tensor>();
    TORCH_CHECK(src.is_cuda() && src.scalar_type() == torch::kFloat32, "unpack source must be an fp32 CUDA tensor");
    device = src.device();
    UnpackOp& op = ops[i];
    std::memset(&op, 0, sizeof(op));
    op.src = src.data_ptr<float>();
    op.d = s[1].cast<int>();
    if (src.dim() == 1) {
      TORCH_CHECK(src.is_contiguous() && src.numel() == static_cast<int64_t>(op.d) * (op.d + 1) / 2, "packed source size");
      op.packed = 1;
    } else {
      TORCH_CHECK(src.dim() == 2 && src.stride(1) == 1 && src.size(0) == op.d && src.size(1) == op.d, "full source shape");
      op.ld_src = static_cast<int>(src.stride(0));
    }
    auto hi = s[2].cast<torch::Tensor>();
    auto lo = s[3].cast<std::optional<torch::Tensor>>();
    TORCH_CHECK(hi.dim() == 2 && hi.stride(1) == 1 && hi.size(0) >= op.d && hi.size(1) >= op.d, "unpack destination shape");
    op.dst_hi = hi.data_ptr<float>();
    op.ld_dst = static_cast<int>(hi.stride(0));
    if (lo.has_value()) {
      TORCH_CHECK(lo->stride(0) == hi.stride(0), "dst_hi and dst_lo share one pitch");
      op.dst_lo = lo->data_ptr<float>();
    }
    for (int r = 0; r < (op.d + kSymRowsPerChunk - 1) / kSymRowsPerChunk; ++r) chunks.push_back(make_int2(static_cast<int>(i), r));
  }
  auto d_ops = upload_bytes(ops.data(), ops.size() * sizeof(UnpackOp), device);
  auto d_chunks = upload_bytes(chunks.data(), chunks.size() * sizeof(int2), device);
  return {d_ops, d_chunks, static_cast<int64_t>(chunks.size())};
}

// Each spec: (src [d, d], dst): dst is 1-D (the packed upper triangle) or a [d, d] view.
std::tuple<torch::Tensor, torch::Tensor, int64_t> build_pack_table(const std::vector<py::tuple>& specs) {
  std::vector<UnpackOp> ops(specs.size());
  std::vector<int2> chunks;
  torch::Device device(torch::kCPU);
  for (size_t i = 0; i < specs.size(); ++i) {
    const py::tuple& s = specs[i];
    TORCH_CHECK(s.size() == 2, "pack spec must have 2 fields");
    auto src = s[0].cast<torch::Tensor>();
    auto dst = s[1].cast<torch::Tensor>();
    TORCH_CHECK(src.is_cuda() && src.scalar_type() == torch::kFloat32 && src.dim() == 2 && src.stride(1) == 1 &&
                    src.size(0) == src.size(1) && dst.scalar_type() == torch::kFloat32,
                "pack source must be a square fp32 CUDA matrix");
    device = src.device();
    UnpackOp& op = ops[i];
    std::memset(&op, 0, sizeof(op));
    op.src = src.data_ptr<float>();
    op.d = static_cast<int>(src.size(0));
    op.ld_src = static_cast<int>(src.stride(0));
    op.dst_hi = dst.data_ptr<float>();
    if (dst.dim() == 1) {
      TORCH_CHECK(dst.is_contiguous() && dst.numel() == static_cast<int64_t>(op.d) * (op.d + 1) / 2, "packed destination size");
      op.packed = 1;
    } else {
      TORCH_CHECK(dst.dim() == 2 && dst.stride(1) == 1 && dst.size(0) == op.d && dst.size(1) == op.d, "full destination shape");
      op.ld_dst = static_cast<int>(dst.stride(0));
    }
    for (int r = 0; r < (op.d + kSymRowsPerChunk - 1) / kSymRowsPerChunk; ++r) chunks.push_back(make_int2(static_cast<int>(i), r));
  }
  auto d_ops = upload_bytes(ops.data(), ops.size() * sizeof(UnpackOp), device);
  auto d_chunks = upload_bytes(chunks.data(), chunks.size() * sizeof(int2), device);
  return {d_ops, d_chunks, static_cast<int64_t>(chunks.size())};
}

void pack_upper(const torch::Tensor& ops, const torch::Tensor& chunks, int64_t num_chunks) {
  LaunchScope scope("ob200::pack_upper");
  c10::cuda::CUDAGuard guard(ops.device());
  launch_pack_upper(reinterpret_cast<const UnpackOp*>(ops.data_ptr()), reinterpret_cast<const int2*>(chunks.data_ptr()),
                    static_cast<int>(num_chunks), at::cuda::getCurrentCUDAStream());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

void unpack_split(const torch::Tensor& ops, const torch::Tensor& chunks, int64_t num_chunks) {
  LaunchScope scope("ob200::unpack_split");
  c10::cuda::CUDAGuard guard(ops.device());
  launch_unpack_split(reinterpret_cast<const UnpackOp*>(ops.data_ptr()), reinterpret_cast<const int2*>(chunks.data_ptr()),
                      static_cast<int>(num_chunks), at::cuda::getCurrentCUDAStream());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

// Each spec: (src [rows, cols], dst | None, dst_hi | None, dst_lo | None); destinations are [cols, rows].
std::tuple<torch::Tensor, torch::Tensor, int64_t> build_transpose_table(const std::vector<py::tuple>& specs) {
  std::vector<TransposeOp> ops(specs.size());
  std::vector<int4> tiles;
  torch::Device device(torch::kCPU);
  for (size_t i = 0; i < specs.size(); ++i) {
    const py::tuple& s = specs[i];
    TORCH_CHECK(s.size() == 4, "transpose spec must have 4 fields");
    auto src = s[0].cast<torch::Tensor>();
    TORCH_CHECK(src.is_cuda() && src.scalar_type() == torch::kFloat32 && src.dim() == 2 && src.stride(1) == 1);
    device = src.device();
    TransposeOp& op = ops[i];
    std::memset(&op, 0, sizeof(op));
    op.src = src.data_ptr<float>();
    op.rows = static_cast<int>(src.size(0));
    op.cols = static_cast<int>(src.size(1));
    op.ld_src = static_cast<int>(src.stride(0));
    int64_t ld = -1;
    auto take = [&](int k) -> float* {
      auto t = s[k].cast<std::optional<torch::Tensor>>();
      if (!t.has_value()) return nullptr;
      TORCH_CHECK(t->is_cuda() && t->scalar_type() == torch::kFloat32 && t->dim() == 2 && t->stride(1) == 1 &&
                      t->size(0) >= op.cols && t->size(1) >= op.rows,
                  "transpose destination too small");
      TORCH_CHECK(ld < 0 || ld == t->stride(0), "transpose destinations must share one pitch");
      ld = t->stride(0);
      return t->data_ptr<float>();
    };
    op.dst = take(1);
    op.dst_hi = take(2);
    op.dst_lo = take(3);
    TORCH_CHECK((op.dst_hi == nullptr) == (op.dst_lo == nullptr), "dst_hi and dst_lo come together");
    TORCH_CHECK(ld > 0, "no destination");
    op.ld_dst = static_cast<int>(ld);
    for (int r = 0; r < (op.rows + 31) / 32; ++r)
      for (int c = 0; c < (op.cols + 31) / 32; ++c) tiles.push_back(make_int4(static_cast<int>(i), r, c, 0));
  }
  auto d_ops = upload_bytes(ops.data(), ops.size() * sizeof(TransposeOp), device);
  auto d_tiles = upload_bytes(tiles.data(), tiles.size() * sizeof(int4), device);
  return {d_ops, d_tiles, static_cast<int64_t>(tiles.size())};
}

void transpose_split(const torch::Tensor& ops, const torch::Tensor& tiles, int64_t num_tiles) {
  LaunchScope scope("ob200::transpose_split");
  c10::cuda::CUDAGuard guard(ops.device());
  launch_transpose_split(reinterpret_cast<const TransposeOp*>(ops.data_ptr()), reinterpret_cast<const int4*>(tiles.data_ptr()),
                         static_cast<int>(num_tiles), at::cuda::getCurrentCUDAStream());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

void peer_copy(const torch::Tensor& table, const torch::Tensor& chunks, int64_t num_chunks) {
  LaunchScope scope("ob200::peer_copy");
  if (num_chunks == 0) return;
  c10::cuda::CUDAGuard guard(table.device());
  launch_peer_copy(reinterpret_cast<const CopyDesc*>(table.data_ptr()), reinterpret_cast<const int2*>(chunks.data_ptr()),
                   static_cast<int>(num_chunks), at::cuda::getCurrentCUDAStream());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.attr("FLAG_PACKED_C") = kFlagPackedC;
  m.attr("FLAG_SPLIT_OUT") = kFlagSplitOut;
  m.attr("FLAG_SUMSQ") = kFlagSumSq;
  m.attr("FLAG_NO_C") = kFlagNoC;
  m.def("set_launch_tracing", &set_launch_tracing, py::arg("nvtx"), py::arg("timing"));
  m.def("launch_timings", &launch_timings, py::arg("reset") = false);
  m.def("build_gemm_plan", &build_gemm_plan);
  m.def("run_gemm_plan", &run_gemm_plan, py::arg("problems"), py::arg("tiles"), py::arg("num_tiles"), py::arg("alpha"),
        py::arg("beta"), py::arg("split"), py::arg("status"), py::arg("gamma") = 0.0);
  m.def("build_gemm_plans", &build_gemm_plans);
  m.def("run_gemm_plan_range", &run_gemm_range, py::arg("problems"), py::arg("tiles"), py::arg("first_tile"),
        py::arg("num_tiles"), py::arg("alpha"), py::arg("beta"), py::arg("split"), py::arg("status"), py::arg("gamma") = 0.0);
  m.attr("FLAG_MIRROR") = kFlagMirror;
  m.attr("FLAG_ADD_DIAG") = kFlagAddDiag;
  m.attr("FLAG_TRACE") = kFlagTrace;
  m.def("build_qr_panel_table", &build_qr_panel_table);
  m.def("householder_panel", &householder_panel);
  m.def("householder_qr", &householder_qr);
  m.attr("QR_PANEL") = kQrPanel;
  m.def("alloc_mat_batch", &alloc_mat_batch);
  m.def("build_sym_table", &build_sym_table);
  m.def("sym_measure", &sym_measure);
  m.def("sq_offdiag", &sq_offdiag);
  m.def("shift_scale_split", &shift_scale_split);
  m.def("build_unpack_table", &build_unpack_table);
  m.def("unpack_split", &unpack_split);
  m.def("build_pack_table", &build_pack_table);
  m.def("pack_upper", &pack_upper);
  m.def("build_transpose_table", &build_transpose_table);
  m.def("transpose_split", &transpose_split);
  m.def("jacobi_eigh_into", &jacobi_eigh_into);
  m.def("run_gemm_plan_push", &run_gemm_plan_push);
  m.attr("FLAG_PEER_PUSH") = kFlagPeerPush;
  m.def("gathered_apply_scaled", &gathered_apply_scaled);
  m.def("build_block_table", &build_block_table);
  m.def("grad_prologue", &grad_prologue);
  m.def("direction_epilogue", &direction_epilogue);
  m.def("gathered_apply", &gathered_apply);
  m.def("peer_barrier", &peer_barrier);
  m.def("eig_scale", &eig_scale);
  m.def("mode_switch", &mode_switch);
  m.attr("FLAG_SQUARE_ACC") = kFlagSquareAcc;
  m.def("build_mat_table", &build_mat_table);
  m.def("affine_identity_split", &affine_identity_split);
  m.def("identity_error", &identity_error);
  m.def("two_sided_apply", &two_sided_apply);
  m.def("tf32_split", &tf32_split);
  m.def("build_gpa_table", &build_gpa_table);
  m.def("gpa_adamw_step", &gpa_adamw_step);
  m.def("gpa_lerp", &gpa_lerp);
  m.def("jacobi_eigh", &jacobi_eigh);
  m.attr("JACOBI_MAX_N") = kJacobiMaxN;
  m.def("build_copy_table", &build_copy_table);
  m.def("peer_copy", &peer_copy);
  ob200::register_model_ops(m);
}
