// Native model runtime: the C ABI a compiled model exposes, implemented as a plan executor.
//
// The reference generates C++ per model (python/aitemplate/backend/main_templates.py:21-403) and links it
// with static/csrc/model_container.cpp + static/include/model.h into one .so per model. Here every model
// shares this library: compile_model() writes a *plan* (tensors, dynamic dims, memory offsets, op list)
// and AITemplateModelContainerCreateFromPlan() turns it into a ModelContainer with the same behaviour:
//   * a pool of `num_runtimes` executors, each with its own activation blob, handed out under a
//     mutex + condition variable (static/include/model_container.h:122-153, model_container.cpp:792-832)
//   * input/output count, dtype, null-pointer and dynamic-dim range checks before every run
//     (model_container.cpp:757-790, static/include/model.h:281-305)
//   * constants in a container-owned slab with a second buffer for SetDoubleBufferConstant /
//     SwapConstants (model_container.cpp:366-681)
//   * optional CUDA-graph replay of the op sequence (static/include/model.h:219-252)
//   * every exception converted to AITemplateError at the C boundary (static/csrc/model_interface.cpp:25-41)
// No device memory is allocated during Run.
#include <cuda_runtime.h>

#include <algorithm>
#include <chrono>
#include <condition_variable>
#include <cstring>
#include <deque>
#include <fstream>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <shared_mutex>
#include <sstream>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

#include "common.h"
#include "model_interface.h"

// per-op entry points of this library (include/b200ait.h)
extern "C" {
int b200ait_gemm_rcr(const void*, const void*, const void*, const void*, const void*, void*, int64_t, int64_t, int64_t,
                     int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int, int, float,
                     int, int64_t, int64_t, int64_t, int, void*, int64_t, int, cudaStream_t);
int b200ait_gemm_rcr_workspace_bytes(int64_t, int64_t, int64_t, int64_t, int, int, int64_t*);
int b200ait_bmm_permute0213(const void*, const void*, void*, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t,
                            int64_t, int, int, float, int, cudaStream_t);
int b200ait_gemm_rrr(const void*, const void*, const void*, const void*, const void*, void*, int64_t, int64_t, int64_t,
                     int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int, int, float, int,
                     void*, int64_t, int, cudaStream_t);
int b200ait_mem_eff_attention(void*, const void*, const void*, const void*, int64_t, int64_t, int64_t, int, int, int,
                              float, int, const int32_t*, const int32_t*, int, cudaStream_t);
int b200ait_mem_eff_attention_strided(void*, const void*, const void*, const void*, int64_t, int64_t, int64_t, int, int,
                                      int, const int64_t*, const int64_t*, const int64_t*, float, int, int, cudaStream_t);
int b200ait_flash_attention(void*, const void*, const int*, float*, float*, int, int, int, int, float, float, int, int,
                            int64_t, int, cudaStream_t);
int b200ait_layernorm(void*, const void*, const void*, const void*, int64_t, int64_t, float, int64_t, int64_t, int,
                      cudaStream_t);
int b200ait_softmax(const void*, void*, int64_t, int64_t, int64_t, int, cudaStream_t);
int b200ait_concatenate(void*, int64_t*, const void* const*, const int64_t* const*, const uint8_t*, int64_t, int64_t,
                        int64_t, int64_t, cudaStream_t);
int b200ait_split(void* const*, const uint8_t*, const void*, const int64_t*, int64_t, const int64_t*, int64_t, int64_t,
                  int64_t, cudaStream_t);
int b200ait_permute(const void*, void*, const int64_t*, const int64_t*, int64_t, int64_t, cudaStream_t);
int b200ait_elementwise(void*, const int64_t*, int64_t, const void* const*, const int64_t* const*, int64_t, const int*,
                        const int*, const float*, int64_t, int, cudaStream_t);
int b200ait_device_status(int*);
}

namespace b200ait {

// -------------------------------------------------------------------------------------- allocators
struct DefaultAllocator : public AITemplateAllocator {
  void* Allocate(size_t nbytes) override {
    void* p = nullptr;
    B200AIT_CUDA_CHECK(cudaMalloc(&p, nbytes ? nbytes : 1));
    return p;
  }
  void Free(void* ptr) override { cudaFree(ptr); }
};
struct TrackingAllocator : public DefaultAllocator {
  void* Allocate(size_t nbytes) override {
    num_bytes_ += nbytes;
    return DefaultAllocator::Allocate(nbytes);
  }
  size_t NumBytesAllocated() const { return num_bytes_; }
  size_t num_bytes_ = 0;
};

static size_t dtype_size(int dtype) {
  switch (dtype) {
    case 1: case 6: return 2;
    case 2: case 3: return 4;
    case 4: return 8;
    case 5: return 1;
    default: throw Error("dtype handling is not implemented!");
  }
}

// -------------------------------------------------------------------------------------------- plan
struct DimTok {
  bool is_static;
  int64_t v;  // value, or index into the dynamic-dim table
};
enum TensorKind { kInput = 0, kOutput = 1, kConstant = 2, kBlob = 3, kView = 4 };
struct TensorInfo {
  std::string name;
  int dtype = 1;
  int kind = kBlob;
  int slot = -1;
  int64_t offset = 0;
  int base = -1;
  std::vector<DimTok> dims;
};
struct DimInfo {
  std::string name;
  int64_t lo = 0, hi = 0;
};
struct OpInfo {
  std::string kernel, name;
  std::vector<int> operands, outputs;
  std::vector<int64_t> ints;
  std::vector<double> floats;
};
struct ConstantInfo {
  std::string name, original_name;
  int tensor = -1;
  int64_t offset = 0, nbytes = 0;
  bool bound = false;
  int64_t file_offset = 0;
};
struct Plan {
  std::string name;
  int64_t blob_bytes = 0, constants_bytes = 0;
  std::vector<DimInfo> dims;
  std::vector<TensorInfo> tensors;
  std::vector<OpInfo> ops;
  std::vector<ConstantInfo> constants;
  std::vector<int> inputs, outputs;  // tensor index per input / output slot
  std::string constants_file;
};

static Plan parse_plan(const std::string& path) {
  std::ifstream f(path);
  if (!f) throw Error("cannot open plan file " + path);
  Plan p;
  std::string tok;
  auto expect = [&](const char* w) {
    if (!(f >> tok) || tok != w) throw Error(std::string("plan parse error: expected '") + w + "', got '" + tok + "'");
  };
  expect("B200AIT_PLAN");
  int version = 0;
  f >> version;
  if (version != 1) throw Error("unsupported plan version");
  expect("name");
  f >> p.name;
  expect("blob_bytes");
  f >> p.blob_bytes;
  expect("constants_bytes");
  f >> p.constants_bytes;
  expect("constants_file");
  f >> p.constants_file;
  if (p.constants_file == "-") p.constants_file.clear();
  size_t n = 0;
  expect("num_dims");
  f >> n;
  p.dims.resize(n);
  for (size_t i = 0; i < n; ++i) {
    expect("dim");
    f >> p.dims[i].name >> p.dims[i].lo >> p.dims[i].hi;
  }
  expect("num_tensors");
  f >> n;
  p.tensors.resize(n);
  for (size_t i = 0; i < n; ++i) {
    expect("tensor");
    TensorInfo& t = p.tensors[i];
    size_t rank = 0;
    f >> t.name >> t.dtype >> t.kind >> t.slot >> t.offset >> t.base >> rank;
    t.dims.resize(rank);
    for (size_t d = 0; d < rank; ++d) {
      f >> tok;
      if (tok.size() < 2 || (tok[0] != 's' && tok[0] != 'd')) throw Error("plan parse error: bad dim token " + tok);
      t.dims[d].is_static = tok[0] == 's';
      t.dims[d].v = std::stoll(tok.substr(1));
      if (!t.dims[d].is_static && (t.dims[d].v < 0 || t.dims[d].v >= static_cast<int64_t>(p.dims.size())))
        throw Error("plan parse error: dim index out of range");
    }
  }
  expect("num_ops");
  f >> n;
  p.ops.resize(n);
  for (size_t i = 0; i < n; ++i) {
    expect("op");
    OpInfo& o = p.ops[i];
    size_t k = 0;
    f >> o.kernel >> o.name >> k;
    o.operands.resize(k);
    for (auto& x : o.operands) f >> x;
    f >> k;
    o.outputs.resize(k);
    for (auto& x : o.outputs) f >> x;
    f >> k;
    o.ints.resize(k);
    for (auto& x : o.ints) f >> x;
    f >> k;
    o.floats.resize(k);
    for (auto& x : o.floats) f >> x;
    for (int x : o.operands)
      if (x < -1 || x >= static_cast<int>(p.tensors.size())) throw Error("plan parse error: operand index");
    for (int x : o.outputs)
      if (x < 0 || x >= static_cast<int>(p.tensors.size())) throw Error("plan parse error: output index");
  }
  expect("num_constants");
  f >> n;
  p.constants.resize(n);
  for (size_t i = 0; i < n; ++i) {
    expect("constant");
    ConstantInfo& c = p.constants[i];
    int bound = 0;
    f >> c.name >> c.original_name >> c.tensor >> c.offset >> c.nbytes >> bound >> c.file_offset;
    c.bound = bound != 0;
  }
  expect("num_inputs");
  f >> n;
  p.inputs.assign(n, -1);
  for (size_t i = 0; i < n; ++i) {
    expect("input");
    size_t slot = 0;
    int t = -1;
    f >> slot >> t;
    if (slot >= n || t < 0 || t >= static_cast<int>(p.tensors.size())) throw Error("plan parse error: input entry");
    p.inputs[slot] = t;
  }
  expect("num_outputs");
  f >> n;
  p.outputs.assign(n, -1);
  for (size_t i = 0; i < n; ++i) {
    expect("output");
    size_t slot = 0;
    int t = -1;
    f >> slot >> t;
    if (slot >= n || t < 0 || t >= static_cast<int>(p.tensors.size())) throw Error("plan parse error: output entry");
    p.outputs[slot] = t;
  }
  if (!f) throw Error("plan parse error: truncated file");
  for (int t : p.inputs)
    if (t < 0) throw Error("plan parse error: missing input slot");
  for (int t : p.outputs)
    if (t < 0) throw Error("plan parse error: missing output slot");
  for (size_t i = 0; i < p.tensors.size(); ++i) {
    const TensorInfo& t = p.tensors[i];
    if (t.kind == kView && (t.base < 0 || t.base >= static_cast<int>(i)))
      throw Error("plan parse error: a view must come after its base tensor");
    if (t.kind == kInput && (t.slot < 0 || t.slot >= static_cast<int>(p.inputs.size())))
      throw Error("plan parse error: input slot out of range");
    if (t.kind == kOutput && (t.slot < 0 || t.slot >= static_cast<int>(p.outputs.size())))
      throw Error("plan parse error: output slot out of range");
  }
  return p;
}

// ---------------------------------------------------------------------------------------- executor
struct RunState {
  std::vector<int64_t> dims;      // current value of each dynamic dim
  std::vector<uint8_t> dim_set;
  std::vector<void*> input_ptrs, output_ptrs;
};

class ModelContainer;

class Executor {
 public:
  Executor(const Plan& plan, AITemplateAllocator& alloc) : plan_(plan), alloc_(alloc) {
    blob_ = alloc_.Allocate(static_cast<size_t>(plan.blob_bytes));
    // one split-K scratch area shared by every GEMM of the plan, sized for the hungriest of them at the
    // lower and upper bound of its dynamic dims (reference: global workspace = max over ops,
    // python/aitemplate/compiler/transform/memory_planning.py:141-195)
    for (const OpInfo& op : plan.ops) {
      if (op.kernel != "gemm_rcr") continue;
      const TensorInfo& a = plan.tensors[op.operands[0]];
      const TensorInfo& b = plan.tensors[op.operands[1]];
      if (a.dims.empty() || b.dims.size() != 2 || !b.dims[0].is_static || !a.dims.back().is_static) continue;
      // Split-K demand is not monotonic in M (none once the tiles fill the SMs, little at M = 1, most
      // around M = 128..512), so a dynamic M is sampled: both bounds, then every multiple of 128 up to 2048
      // and powers of two above, inside [lo, hi].
      int64_t m_lo = 1, m_hi = 1;
      for (size_t i = 0; i + 1 < a.dims.size(); ++i) {
        m_lo *= a.dims[i].is_static ? a.dims[i].v : plan.dims[a.dims[i].v].lo;
        m_hi *= a.dims[i].is_static ? a.dims[i].v : plan.dims[a.dims[i].v].hi;
      }
      std::vector<int64_t> ms{m_lo, m_hi};
      for (int64_t m = 128; m < m_hi && m <= 2048; m += 128)
        if (m > m_lo) ms.push_back(m);
      for (int64_t m = 4096; m < m_hi; m *= 2)
        if (m > m_lo) ms.push_back(m);
      // ints[7], ints[8]: tile width and split-K chosen by the compile-time profiler (0 = library decides)
      const int tile_hint = op.ints.size() > 8 ? static_cast<int>(op.ints[7]) : 0;
      const int split_hint = op.ints.size() > 8 ? static_cast<int>(op.ints[8]) : 0;
      for (int64_t m : ms) {
        int64_t bytes = 0;
        if (b200ait_gemm_rcr_workspace_bytes(1, m, b.dims[0].v, a.dims.back().v, tile_hint, split_hint, &bytes) == 0)
          workspace_bytes_ = std::max(workspace_bytes_, bytes);
      }
    }
    workspace_bytes_ = std::min<int64_t>(workspace_bytes_, 256ll << 20);
    if (workspace_bytes_ > 0) workspace_ = alloc_.Allocate(static_cast<size_t>(workspace_bytes_));
    B200AIT_CUDA_CHECK(cudaEventCreateWithFlags(&run_finished_, cudaEventDisableTiming));
    B200AIT_CUDA_CHECK(cudaStreamCreateWithFlags(&graph_stream_, cudaStreamNonBlocking));
    st_.dims.assign(plan.dims.size(), 0);
    st_.dim_set.assign(plan.dims.size(), 0);
    ptrs_.assign(plan.tensors.size(), nullptr);
  }
  ~Executor() {
    for (auto& entry : graph_cache_)
      if (entry.exec) cudaGraphExecDestroy(entry.exec);
    if (graph_stream_) cudaStreamDestroy(graph_stream_);
    if (run_finished_) cudaEventDestroy(run_finished_);
    if (blob_) alloc_.Free(blob_);
    if (workspace_) alloc_.Free(workspace_);
  }

  RunState& state() { return st_; }

  int64_t dim_value(const DimTok& d) const {
    if (d.is_static) return d.v;
    if (!st_.dim_set[d.v]) throw Error("dynamic dim '" + plan_.dims[d.v].name + "' used before it was bound");
    return st_.dims[d.v];
  }
  std::vector<int64_t> shape_of(int t) const {
    std::vector<int64_t> s;
    for (auto& d : plan_.tensors[t].dims) s.push_back(dim_value(d));
    return s;
  }
  int64_t numel_of(int t) const {
    int64_t n = 1;
    for (auto& d : plan_.tensors[t].dims) n *= dim_value(d);
    return n;
  }
  // binds (or verifies) the dims of tensor t to `shape`
  void bind_shape(int t, const std::vector<int64_t>& shape, const char* what) {
    const TensorInfo& ti = plan_.tensors[t];
    if (shape.size() != ti.dims.size())
      throw Error(std::string(what) + " '" + ti.name + "': rank mismatch");
    for (size_t i = 0; i < shape.size(); ++i) {
      const DimTok& d = ti.dims[i];
      if (d.is_static) {
        if (d.v != shape[i])
          throw Error(std::string(what) + " '" + ti.name + "': dim " + std::to_string(i) + " is " +
                      std::to_string(shape[i]) + ", expected " + std::to_string(d.v));
      } else {
        const DimInfo& di = plan_.dims[d.v];
        if (shape[i] < di.lo || shape[i] > di.hi)
          throw std::out_of_range("dynamic dim '" + di.name + "' of " + what + " '" + ti.name + "' is " +
                                  std::to_string(shape[i]) + ", outside [" + std::to_string(di.lo) + ", " +
                                  std::to_string(di.hi) + "]");
        if (st_.dim_set[d.v] && st_.dims[d.v] != shape[i])
          throw Error("dynamic dim '" + di.name + "' bound to both " + std::to_string(st_.dims[d.v]) + " and " +
                      std::to_string(shape[i]));
        st_.dims[d.v] = shape[i];
        st_.dim_set[d.v] = 1;
      }
    }
  }

  void* ptr_of(int t) const { return t < 0 ? nullptr : ptrs_[t]; }

  void resolve_pointers(uint8_t* constants) {
    for (size_t i = 0; i < plan_.tensors.size(); ++i) {
      const TensorInfo& t = plan_.tensors[i];
      switch (t.kind) {
        case kInput: ptrs_[i] = st_.input_ptrs[t.slot]; break;
        case kOutput: ptrs_[i] = st_.output_ptrs[t.slot]; break;
        case kConstant: ptrs_[i] = constants + t.offset; break;
        case kBlob: ptrs_[i] = static_cast<uint8_t*>(blob_) + t.offset; break;
        case kView: ptrs_[i] = static_cast<uint8_t*>(ptrs_[t.base]) + t.offset; break;  // bases precede views
      }
    }
  }

  void run_ops(cudaStream_t stream, bool launch);
  void run(cudaStream_t stream, bool graph_mode, uint8_t* constants);
  void profile(cudaStream_t stream, size_t iters, const std::string& filename, uint8_t* constants);

  cudaEvent_t run_finished() const { return run_finished_; }
  // Orders a new run on `stream` after this executor's previous run (which may still be in flight on
  // another stream and owns the same blob and workspace) without blocking the host.
  void order_after_previous_run(cudaStream_t stream) {
    if (has_run_ && stream != last_stream_) B200AIT_CUDA_CHECK(cudaStreamWaitEvent(stream, run_finished_, 0));
    last_stream_ = stream;
    has_run_ = true;
  }
  // Marks the end of whatever an aborted run managed to enqueue, so that the next run of this
  // executor is still ordered after those kernels.
  void mark_run_finished(cudaStream_t stream) noexcept {
    if (cudaEventRecord(run_finished_, stream) != cudaSuccess) cudaGetLastError();
  }

 private:
  void check(int code, const OpInfo& op) {
    if (code != 0) throw Error("op '" + op.name + "' (" + op.kernel + ") failed: " + last_error());
  }
  void run_one(const OpInfo& op, cudaStream_t stream, bool launch);

  const Plan& plan_;
  AITemplateAllocator& alloc_;
  void* blob_ = nullptr;
  void* workspace_ = nullptr;
  int64_t workspace_bytes_ = 0;
  RunState st_;
  std::vector<void*> ptrs_;
  cudaEvent_t run_finished_ = nullptr;
  cudaStream_t last_stream_ = nullptr;
  bool has_run_ = false;
  cudaStream_t graph_stream_ = nullptr;
  struct GraphEntry {
    std::vector<int64_t> key;
    cudaGraphExec_t exec = nullptr;
    uint64_t last_use = 0;
  };
  static constexpr size_t kGraphCacheSize = 8;
  std::vector<GraphEntry> graph_cache_;
  uint64_t graph_clock_ = 0;
  bool graph_ok_ = true;
  bool warmed_ = false;
};

// Evaluates the op's output shapes (always) and launches its kernel (when `launch`).
void Executor::run_one(const OpInfo& op, cudaStream_t stream, bool launch) {
  const auto& T = plan_.tensors;
  auto in = [&](size_t i) { return i < op.operands.size() ? op.operands[i] : -1; };
  const int out0 = op.outputs.empty() ? -1 : op.outputs[0];
  if (op.kernel == "view") {
    // reshape / flatten / squeeze / unsqueeze: same bytes, new shape; at most one unbound dim is inferred
    const int64_t numel = numel_of(in(0));
    const TensorInfo& o = T[out0];
    int64_t known = 1;
    int unknown = -1;
    for (size_t i = 0; i < o.dims.size(); ++i) {
      const DimTok& d = o.dims[i];
      if (d.is_static || st_.dim_set[d.v]) {
        known *= d.is_static ? d.v : st_.dims[d.v];
      } else {
        if (unknown >= 0 && o.dims[unknown].v != d.v) throw Error("view '" + op.name + "': more than one unknown dim");
        unknown = static_cast<int>(i);
      }
    }
    if (unknown >= 0) {
      if (known == 0 || numel % known != 0) throw Error("view '" + op.name + "': cannot infer the unknown dim");
      std::vector<int64_t> shape;
      for (size_t i = 0; i < o.dims.size(); ++i)
        shape.push_back(static_cast<int>(i) == unknown ? numel / known : dim_value(o.dims[i]));
      bind_shape(out0, shape, "view output");
    } else if (known != numel) {
      throw Error("view '" + op.name + "': element count changes from " + std::to_string(numel) + " to " +
                  std::to_string(known));
    }
    return;
  }
  if (op.kernel == "gemm_rcr") {
    const int a = in(0), b = in(1), bias = in(2), d0 = in(3), d1 = in(4);
    const auto as = shape_of(a);
    const auto bs = shape_of(b);
    const int64_t k = as.back(), n = bs[0];
    int64_t m = 1;
    for (size_t i = 0; i + 1 < as.size(); ++i) m *= as[i];
    if (bs[1] != k) throw Error("gemm '" + op.name + "': K mismatch");
    std::vector<int64_t> os(as.begin(), as.end() - 1);
    os.push_back(n);
    bind_shape(out0, os, "gemm output");
    if (!launch) return;
    const int64_t out_off = op.ints[5], out_stride = op.ints[6];
    const int tile_hint = op.ints.size() > 8 ? static_cast<int>(op.ints[7]) : 0;
    const int split_hint = op.ints.size() > 8 ? static_cast<int>(op.ints[8]) : 0;
    uint8_t* c = static_cast<uint8_t*>(ptr_of(out0)) + out_off * dtype_size(T[out0].dtype);
    // ints[9]: row stride of A when it is a column block of a wider buffer (a split read in place); 0 = K
    const int64_t lda = op.ints.size() > 9 && op.ints[9] > 0 ? op.ints[9] : k;
    const int64_t ldb = op.ints.size() > 10 && op.ints[10] > 0 ? op.ints[10] : k;  // ints[10]: the same for B
    check(b200ait_gemm_rcr(ptr_of(a), ptr_of(b), ptr_of(bias), ptr_of(d0), ptr_of(d1), c, 1, m, n, k, lda, ldb,
                           out_stride, n, 0, 0, 0, 0, static_cast<int>(op.ints[0]), T[a].dtype,
                           static_cast<float>(op.floats[0]), static_cast<int>(op.ints[1]), op.ints[2], op.ints[3],
                           op.ints[4], tile_hint, workspace_, workspace_bytes_, split_hint, stream),
          op);
    return;
  }
  if (op.kernel == "gemm_rrr") {  // B stored [K, N]
    const int a = in(0), b = in(1), bias = in(2), d0 = in(3), d1 = in(4);
    const auto as = shape_of(a);
    const auto bs = shape_of(b);
    const int64_t k = as.back(), n = bs[1];
    int64_t m = 1;
    for (size_t i = 0; i + 1 < as.size(); ++i) m *= as[i];
    if (bs[0] != k) throw Error("gemm '" + op.name + "': K mismatch");
    std::vector<int64_t> os(as.begin(), as.end() - 1);
    os.push_back(n);
    bind_shape(out0, os, "gemm output");
    if (!launch) return;
    const int64_t out_off = op.ints[5], out_stride = op.ints[6];
    uint8_t* c = static_cast<uint8_t*>(ptr_of(out0)) + out_off * dtype_size(T[out0].dtype);
    const int64_t lda = op.ints.size() > 9 && op.ints[9] > 0 ? op.ints[9] : k;
    check(b200ait_gemm_rrr(ptr_of(a), ptr_of(b), ptr_of(bias), ptr_of(d0), ptr_of(d1), c, 1, m, n, k, lda, n, out_stride,
                           n, 0, 0, 0, 0, static_cast<int>(op.ints[0]), T[a].dtype, static_cast<float>(op.floats[0]),
                           static_cast<int>(op.ints[7]), workspace_, workspace_bytes_, static_cast<int>(op.ints[8]),
                           stream),
          op);
    return;
  }
  if (op.kernel == "bmm_rrr") {
    const int a = in(0), b = in(1);
    auto as = shape_of(a), bs = shape_of(b);
    if (as.size() == 2) as.insert(as.begin(), 1);
    if (bs.size() == 2) bs.insert(bs.begin(), 1);
    const int64_t ba = as[0], bb = bs[0], m = as[1], k = as[2], n = bs[2];
    if (bs[1] != k) throw Error("bmm '" + op.name + "': K mismatch");
    if (!(ba == bb || ba == 1 || bb == 1)) throw Error("bmm '" + op.name + "': batch sizes are not broadcastable");
    const int64_t batch = std::max(ba, bb);
    bind_shape(out0, {batch, m, n}, "bmm output");
    if (!launch) return;
    // ints: [d1, lda, ldb, out offset, ldc]. d1 > 0: the "0213" permuted store of bmm_rrr_permute
    // ([B / d1, M, d1, N]). lda / ldb: row strides of operands that are column blocks of a wider buffer (a split
    // read in place). out offset / ldc: the output is a column block of a concatenate's buffer. 0 = contiguous.
    const auto opt = [&](size_t i) { return op.ints.size() > i ? op.ints[i] : 0; };
    const int64_t lda = opt(1) > 0 ? opt(1) : k, ldb = opt(2) > 0 ? opt(2) : n, ldc = opt(4) > 0 ? opt(4) : n;
    const int64_t a_bs = (ba == 1 && batch > 1) ? 0 : m * lda, b_bs = (bb == 1 && batch > 1) ? 0 : k * ldb;
    if (opt(0) > 0) {
      if (opt(1) > 0 || opt(2) > 0 || opt(4) > 0) throw Error("bmm '" + op.name + "': permuted store with strided operands");
      check(b200ait_bmm_permute0213(ptr_of(a), ptr_of(b), ptr_of(out0), batch, m, n, k, a_bs, b_bs, opt(0), 1,
                                    T[a].dtype, static_cast<float>(op.floats[0]), 0, stream),
            op);
      return;
    }
    uint8_t* c = static_cast<uint8_t*>(ptr_of(out0)) + opt(3) * dtype_size(T[out0].dtype);
    check(b200ait_gemm_rrr(ptr_of(a), ptr_of(b), nullptr, nullptr, nullptr, c, batch, m, n, k, lda, ldb, ldc, n,
                           a_bs, b_bs, m * ldc, m * n, 0, T[a].dtype, static_cast<float>(op.floats[0]), 0, nullptr, 0,
                           1, stream),
          op);
    return;
  }
  if (op.kernel == "bmm_rcr") {
    const int a = in(0), b = in(1);
    auto as = shape_of(a), bs = shape_of(b);
    if (as.size() == 2) as.insert(as.begin(), 1);
    if (bs.size() == 2) bs.insert(bs.begin(), 1);
    const int64_t ba = as[0], bb = bs[0], m = as[1], k = as[2], n = bs[1];
    if (bs[2] != k) throw Error("bmm '" + op.name + "': K mismatch");
    if (!(ba == bb || ba == 1 || bb == 1)) throw Error("bmm '" + op.name + "': batch sizes are not broadcastable");
    const int64_t batch = std::max(ba, bb);
    bind_shape(out0, {batch, m, n}, "bmm output");
    if (!launch) return;
    // ints: [d1, lda, ldb, out offset, ldc], as for bmm_rrr above
    const auto opt = [&](size_t i) { return op.ints.size() > i ? op.ints[i] : 0; };
    const int64_t lda = opt(1) > 0 ? opt(1) : k, ldb = opt(2) > 0 ? opt(2) : k, ldc = opt(4) > 0 ? opt(4) : n;
    const int64_t a_bs = (ba == 1 && batch > 1) ? 0 : m * lda, b_bs = (bb == 1 && batch > 1) ? 0 : n * ldb;
    if (opt(0) > 0) {
      if (opt(1) > 0 || opt(2) > 0 || opt(4) > 0) throw Error("bmm '" + op.name + "': permuted store with strided operands");
      check(b200ait_bmm_permute0213(ptr_of(a), ptr_of(b), ptr_of(out0), batch, m, n, k, a_bs, b_bs, opt(0), 0,
                                    T[a].dtype, static_cast<float>(op.floats[0]), 0, stream),
            op);
      return;
    }
    uint8_t* c = static_cast<uint8_t*>(ptr_of(out0)) + opt(3) * dtype_size(T[out0].dtype);
    check(b200ait_gemm_rcr(ptr_of(a), ptr_of(b), nullptr, nullptr, nullptr, c, batch, m, n, k, lda, ldb, ldc, n,
                           a_bs, b_bs, m * ldc, m * n, 0, T[a].dtype, static_cast<float>(op.floats[0]), 0, 1, 1, 1, 0,
                           nullptr, 0, 1, stream),
          op);
    return;
  }
  if (op.kernel == "mem_eff_attention") {
    // ints: causal, then one flag per operand: 1 = the operand is stored [B, S, H, D] (a permute (0, 2, 1, 3) that the
    // compiler folded into this op) and is read in place through strides
    const int q = in(0), k = in(1), v = in(2);
    const bool qt = op.ints.size() > 1 && op.ints[1], kt = op.ints.size() > 2 && op.ints[2],
               vt = op.ints.size() > 3 && op.ints[3];
    auto bhsd = [&](int t, bool stored_bshd) {  // logical [B, H, S, D] dims of an operand
      auto s = shape_of(t);
      if (stored_bshd) std::swap(s[1], s[2]);
      return s;
    };
    const auto qs = bhsd(q, qt), ks = bhsd(k, kt), vs = bhsd(v, vt);
    bind_shape(out0, {qs[0], qs[2], qs[1], vs[3]}, "attention output");
    // ints[4], ints[5]: an int32 lengths_kv / lengths_q operand (one value per batch) follows q, k, v
    int next = 3;
    const int lkv = op.ints.size() > 4 && op.ints[4] ? in(next++) : -1;
    const int lq = op.ints.size() > 5 && op.ints[5] ? in(next++) : -1;
    for (int t : {lkv, lq}) {
      if (t < 0) continue;
      int64_t count = 1;
      for (int64_t d : shape_of(t)) count *= d;
      if (T[t].dtype != kDTypeInt || count != qs[0])
        throw Error("attention '" + op.name + "': a lengths operand must hold one int32 per batch");
    }
    if (!launch) return;
    if (!qt && !kt && !vt) {
      check(b200ait_mem_eff_attention(ptr_of(out0), ptr_of(q), ptr_of(k), ptr_of(v), qs[0], ks[2], qs[2],
                                      static_cast<int>(qs[1]), static_cast<int>(qs[3]), static_cast<int>(vs[3]),
                                      static_cast<float>(op.floats[0]), static_cast<int>(op.ints[0]),
                                      lkv >= 0 ? static_cast<const int32_t*>(ptr_of(lkv)) : nullptr,
                                      lq >= 0 ? static_cast<const int32_t*>(ptr_of(lq)) : nullptr, T[q].dtype, stream),
            op);
      return;
    }
    if (lkv >= 0 || lq >= 0) throw Error("attention '" + op.name + "': lengths with operands read through strides");
    auto strides = [](const std::vector<int64_t>& s, bool stored_bshd, int64_t* out) {
      const int64_t h = s[1], rows = s[2], d = s[3];
      if (stored_bshd) {
        out[0] = h * d, out[1] = d, out[2] = rows * h * d;
      } else {
        out[0] = d, out[1] = rows * d, out[2] = h * rows * d;
      }
    };
    int64_t sq[3], sk[3], sv[3];
    strides(qs, qt, sq), strides(ks, kt, sk), strides(vs, vt, sv);
    check(b200ait_mem_eff_attention_strided(ptr_of(out0), ptr_of(q), ptr_of(k), ptr_of(v), qs[0], ks[2], qs[2],
                                            static_cast<int>(qs[1]), static_cast<int>(qs[3]), static_cast<int>(vs[3]),
                                            sq, sk, sv, static_cast<float>(op.floats[0]), static_cast<int>(op.ints[0]),
                                            T[q].dtype, stream),
          op);
    return;
  }
  if (op.kernel == "flash_attention") {  // ints: causal, batch_size, max_seq_len; floats: scale
    const int x = in(0), cu = in(1);
    const auto xs = shape_of(x);  // [total, 3, H, D]
    bind_shape(out0, {xs[0], xs[2], xs[3]}, "flash_attention output");
    if (!launch) return;
    check(b200ait_flash_attention(ptr_of(out0), ptr_of(x), static_cast<const int*>(ptr_of(cu)), nullptr, nullptr,
                                  static_cast<int>(op.ints[1]), static_cast<int>(op.ints[2]),
                                  static_cast<int>(xs[2]), static_cast<int>(xs[3]), 0.f,
                                  static_cast<float>(op.floats[0]), static_cast<int>(op.ints[0]), 0, xs[0], T[x].dtype,
                                  stream),
          op);
    return;
  }
  if (op.kernel == "layernorm") {
    const int x = in(0);
    const auto xs = shape_of(x);
    bind_shape(out0, xs, "layernorm output");
    if (!launch) return;
    const int64_t n = op.ints[0];
    int64_t numel = 1;
    for (auto d : xs) numel *= d;
    const int64_t m = n ? numel / n : 0;
    // ints[1], ints[2]: element offset and row stride of the output when it is a column block of a wider
    // buffer (a layernorm fused into a concatenate); 0 stride = contiguous rows
    const int64_t out_off = op.ints.size() > 2 ? op.ints[1] : 0, out_stride = op.ints.size() > 2 ? op.ints[2] : 0;
    // ints[3]: row stride of the input when it is a column block of a wider buffer (a split read in place)
    const int64_t in_stride = op.ints.size() > 3 ? op.ints[3] : 0;
    uint8_t* y = static_cast<uint8_t*>(ptr_of(out0)) + out_off * dtype_size(T[out0].dtype);
    check(b200ait_layernorm(y, ptr_of(x), ptr_of(in(1)), ptr_of(in(2)), m, n, static_cast<float>(op.floats[0]),
                            in_stride, out_stride, T[x].dtype, stream),
          op);
    return;
  }
  if (op.kernel == "softmax") {
    const int x = in(0);
    const auto xs = shape_of(x);
    bind_shape(out0, xs, "softmax output");
    if (!launch) return;
    const int64_t dim = op.ints[0];
    int64_t outer = 1, inner = 1;
    for (int64_t i = 0; i < dim; ++i) outer *= xs[i];
    for (size_t i = dim + 1; i < xs.size(); ++i) inner *= xs[i];
    check(b200ait_softmax(ptr_of(x), ptr_of(out0), outer, xs[dim], inner, T[x].dtype, stream), op);
    return;
  }
  if (op.kernel == "concatenate") {
    const int64_t dim = op.ints[0];
    const size_t n = op.operands.size();
    std::vector<std::vector<int64_t>> shapes(n);
    std::vector<const int64_t*> shape_ptrs(n);
    std::vector<const void*> ptrs(n);
    std::vector<uint8_t> masks(n);
    int rank = 0;
    for (size_t i = 0; i < n; ++i) {
      shapes[i] = shape_of(op.operands[i]);
      rank = std::max<int>(rank, static_cast<int>(shapes[i].size()));
    }
    for (size_t i = 0; i < n; ++i) {
      if (static_cast<int>(shapes[i].size()) != rank) {  // an empty rank-1 tensor stands for "no rows"
        shapes[i] = shapes[n - 1].size() == static_cast<size_t>(rank) ? shapes[n - 1] : shapes[0];
        for (size_t j = 0; j < n; ++j)
          if (static_cast<int>(shape_of(op.operands[j]).size()) == rank) shapes[i] = shape_of(op.operands[j]);
        shapes[i][dim] = 0;
      }
      shape_ptrs[i] = shapes[i].data();
      ptrs[i] = ptr_of(op.operands[i]);
      masks[i] = static_cast<uint8_t>(op.ints[2 + i]);
    }
    std::vector<int64_t> os = shapes[0];
    os[dim] = 0;
    for (size_t i = 0; i < n; ++i) os[dim] += shapes[i][dim];
    bind_shape(out0, os, "concatenate output");
    if (!launch) return;
    check(b200ait_concatenate(ptr_of(out0), nullptr, ptrs.data(), shape_ptrs.data(), masks.data(), dim, rank,
                              static_cast<int64_t>(n), static_cast<int64_t>(dtype_size(T[out0].dtype)), stream),
          op);
    return;
  }
  if (op.kernel == "split") {
    const int x = in(0);
    const auto xs = shape_of(x);
    const int64_t dim = op.ints[0], n = op.ints[1];
    std::vector<int64_t> sizes(op.ints.begin() + 2, op.ints.begin() + 2 + n);
    std::vector<uint8_t> masks(n);
    std::vector<void*> outs(n);
    for (int64_t i = 0; i < n; ++i) {
      masks[i] = static_cast<uint8_t>(op.ints[2 + n + i]);
      auto os = xs;
      os[dim] = sizes[i];
      bind_shape(op.outputs[i], os, "split output");
      outs[i] = ptr_of(op.outputs[i]);
    }
    if (!launch) return;
    check(b200ait_split(outs.data(), masks.data(), ptr_of(x), xs.data(), n, sizes.data(), dim,
                        static_cast<int64_t>(xs.size()), static_cast<int64_t>(dtype_size(T[x].dtype)), stream),
          op);
    return;
  }
  if (op.kernel == "permute") {
    const int x = in(0);
    const auto xs = shape_of(x);
    const int64_t rank = op.ints[0];
    std::vector<int64_t> dims(op.ints.begin() + 1, op.ints.begin() + 1 + rank), os(rank);
    for (int64_t i = 0; i < rank; ++i) os[i] = xs[dims[i]];
    bind_shape(out0, os, "permute output");
    if (!launch) return;
    check(b200ait_permute(ptr_of(x), ptr_of(out0), xs.data(), dims.data(), rank,
                          static_cast<int64_t>(dtype_size(T[x].dtype)), stream),
          op);
    return;
  }
  if (op.kernel == "elementwise") {
    const size_t n = op.operands.size();
    std::vector<std::vector<int64_t>> shapes(n);
    size_t rank = 0;
    for (size_t i = 0; i < n; ++i) {
      shapes[i] = shape_of(op.operands[i]);
      rank = std::max(rank, shapes[i].size());
    }
    std::vector<int64_t> os(rank, 1);
    std::vector<const int64_t*> shape_ptrs(n);
    std::vector<const void*> ptrs(n);
    for (size_t i = 0; i < n; ++i) {
      shapes[i].insert(shapes[i].begin(), rank - shapes[i].size(), 1);
      for (size_t d = 0; d < rank; ++d) {
        if (shapes[i][d] != 1) {
          if (os[d] != 1 && os[d] != shapes[i][d]) throw Error("elementwise '" + op.name + "': shapes do not broadcast");
          os[d] = shapes[i][d];
        }
      }
      shape_ptrs[i] = shapes[i].data();
      ptrs[i] = ptr_of(op.operands[i]);
    }
    bind_shape(out0, os, "elementwise output");
    if (!launch) return;
    const int64_t steps = op.ints[0];
    std::vector<int> codes(steps), operands(steps);
    std::vector<float> consts(steps);
    for (int64_t s = 0; s < steps; ++s) {
      codes[s] = static_cast<int>(op.ints[1 + 2 * s]);
      operands[s] = static_cast<int>(op.ints[2 + 2 * s]);
      consts[s] = static_cast<float>(op.floats[s]);
    }
    check(b200ait_elementwise(ptr_of(out0), os.data(), static_cast<int64_t>(rank), ptrs.data(), shape_ptrs.data(),
                              static_cast<int64_t>(n), codes.data(), operands.data(), consts.data(), steps,
                              T[out0].dtype, stream),
          op);
    return;
  }
  if (op.kernel == "copy") {
    // an output that aliases an input, a constant or another output is materialised by a device copy
    // (static/include/model_container.h:127-130)
    const int x = in(0);
    const auto xs = shape_of(x);
    bind_shape(out0, xs, "copy output");
    if (!launch) return;
    int64_t numel = 1;
    for (auto d : xs) numel *= d;
    if (numel > 0)
      B200AIT_CUDA_CHECK(cudaMemcpyAsync(ptr_of(out0), ptr_of(x), static_cast<size_t>(numel) * dtype_size(T[x].dtype),
                                         cudaMemcpyDeviceToDevice, stream));
    return;
  }
  throw Error("plan names an unknown kernel '" + op.kernel + "'");
}

void Executor::run_ops(cudaStream_t stream, bool launch) {
  for (const OpInfo& op : plan_.ops) run_one(op, stream, launch);
}

void Executor::run(cudaStream_t stream, bool graph_mode, uint8_t* constants) {
  resolve_pointers(constants);
  // The first run always goes eagerly so that one-time set-up (kernel attributes, the status word)
  // never happens inside a stream capture.
  if (!graph_mode || !graph_ok_ || !warmed_) {
    run_ops(stream, true);
    warmed_ = true;
    B200AIT_CUDA_CHECK(cudaEventRecord(run_finished_, stream));
    return;
  }
  run_ops(nullptr, false);  // host-only pass: binds every dynamic dim, validates shapes
  // graph key: every pointer and every dim; a key seen before replays its instantiated graph
  std::vector<int64_t> key;
  key.reserve(ptrs_.size() + st_.dims.size());
  for (void* p : ptrs_) key.push_back(reinterpret_cast<int64_t>(p));
  for (size_t i = 0; i < st_.dims.size(); ++i) key.push_back(st_.dim_set[i] ? st_.dims[i] : -1);
  cudaGraphExec_t exec = nullptr;
  for (auto& entry : graph_cache_) {
    if (entry.key == key) {
      exec = entry.exec;
      entry.last_use = ++graph_clock_;
      break;
    }
  }
  if (exec == nullptr) {
    B200AIT_CUDA_CHECK(cudaStreamBeginCapture(graph_stream_, cudaStreamCaptureModeThreadLocal));
    cudaGraph_t graph = nullptr;
    try {
      run_ops(graph_stream_, true);
    } catch (...) {
      cudaStreamEndCapture(graph_stream_, &graph);
      if (graph) cudaGraphDestroy(graph);
      throw;
    }
    if (cudaStreamEndCapture(graph_stream_, &graph) != cudaSuccess) {
      // reference behaviour: a capture that cannot be ended disables graph mode (static/include/model.h:205-217)
      graph_ok_ = false;
      cudaGetLastError();
      run_ops(stream, true);
      B200AIT_CUDA_CHECK(cudaEventRecord(run_finished_, stream));
      return;
    }
    // a full cache recycles its least recently used executable graph through cudaGraphExecUpdate
    GraphEntry* slot = nullptr;
    if (graph_cache_.size() >= kGraphCacheSize) {
      slot = &graph_cache_[0];
      for (auto& entry : graph_cache_)
        if (entry.last_use < slot->last_use) slot = &entry;
      cudaGraphExecUpdateResultInfo info;
      if (cudaGraphExecUpdate(slot->exec, graph, &info) != cudaSuccess) {
        cudaGetLastError();
        cudaGraphExecDestroy(slot->exec);
        slot->exec = nullptr;
      }
    } else {
      graph_cache_.push_back(GraphEntry{});
      slot = &graph_cache_.back();
    }
    if (slot->exec == nullptr) {
      const cudaError_t ie = cudaGraphInstantiate(&slot->exec, graph, 0);
      if (ie != cudaSuccess) {
        cudaGraphDestroy(graph);
        slot->exec = nullptr;
        slot->key.clear();
        throw Error(std::string("cudaGraphInstantiate failed: ") + cudaGetErrorString(ie));
      }
    }
    cudaGraphDestroy(graph);
    slot->key = std::move(key);
    slot->last_use = ++graph_clock_;
    exec = slot->exec;
  }
  B200AIT_CUDA_CHECK(cudaGraphLaunch(exec, stream));
  B200AIT_CUDA_CHECK(cudaEventRecord(run_finished_, stream));
}


void Executor::profile(cudaStream_t stream, size_t iters, const std::string& filename, uint8_t* constants) {
  // Per-op timing with an L2 flush between iterations, written as JSON
  // (python/aitemplate/backend/main_templates.py:229-293).
  resolve_pointers(constants);
  run_ops(stream, true);  // warm-up, binds every dim
  cudaEvent_t e0, e1;
  B200AIT_CUDA_CHECK(cudaEventCreate(&e0));
  B200AIT_CUDA_CHECK(cudaEventCreate(&e1));
  const size_t flush_bytes = 256u << 20;
  void* flush = alloc_.Allocate(flush_bytes);
  std::ostringstream js;
  js << "{\n";
  bool first = true;
  try {
    for (const OpInfo& op : plan_.ops) {
      if (op.kernel == "view") continue;
      float total = 0.f;
      for (size_t it = 0; it < iters; ++it) {
        B200AIT_CUDA_CHECK(cudaMemsetAsync(flush, static_cast<int>(it), flush_bytes, stream));
        B200AIT_CUDA_CHECK(cudaEventRecord(e0, stream));
        run_one(op, stream, true);
        B200AIT_CUDA_CHECK(cudaEventRecord(e1, stream));
        B200AIT_CUDA_CHECK(cudaEventSynchronize(e1));
        float ms = 0.f;
        B200AIT_CUDA_CHECK(cudaEventElapsedTime(&ms, e0, e1));
        total += ms;
      }
      const float per = iters ? total / static_cast<float>(iters) : 0.f;
      auto sizes = [&](const std::vector<int>& ts) {
        std::ostringstream o;
        o << "[";
        bool f1 = true;
        for (int t : ts) {
          if (t < 0) continue;
          if (!f1) o << ", ";
          f1 = false;
          o << "[";
          const auto sh = shape_of(t);
          for (size_t d = 0; d < sh.size(); ++d) o << (d ? ", " : "") << "\"" << sh[d] << "\"";
          o << "]";
        }
        o << "]";
        return o.str();
      };
      if (!first) js << ",\n";
      first = false;
      js << "  \"" << op.name << "\": { \"ms_per_iter\": " << per << ", \"qps\": " << (per > 0 ? 1000.f / per : 0.f)
         << ", \"input_sizes\": " << sizes(op.operands) << ", \"output_sizes\": " << sizes(op.outputs) << " }";
    }
  } catch (...) {
    alloc_.Free(flush);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    throw;
  }
  js << "\n}\n";
  alloc_.Free(flush);
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  std::ofstream out(filename);
  if (!out) throw Error("cannot write profile file " + filename);
  out << js.str();
}

// --------------------------------------------------------------------------------------- container
class ModelContainer {
 public:
  ModelContainer(const std::string& plan_path, size_t num_runtimes, AITemplateAllocator* allocator)
      : plan_(parse_plan(plan_path)), alloc_(allocator ? *allocator : default_alloc_) {
    if (num_runtimes == 0) throw Error("num_runtimes must be positive!");
    B200AIT_CUDA_CHECK(cudaGetDevice(&device_));
    device_status_word();  // allocate before any stream capture can be active
    sm_count();
    const size_t cbytes = static_cast<size_t>(std::max<int64_t>(plan_.constants_bytes, 1));
    constants_[0] = static_cast<uint8_t*>(alloc_.Allocate(cbytes));
    constants_[1] = nullptr;  // second buffer is created on first double-buffer use
    for (size_t i = 0; i < plan_.constants.size(); ++i) {
      constant_index_[plan_.constants[i].name] = i;
      constant_set_[0].push_back(false);
      constant_set_[1].push_back(false);
    }
    load_bound_constants(plan_path);
    for (size_t i = 0; i < num_runtimes; ++i) {
      executors_.push_back(std::make_unique<Executor>(plan_, alloc_));
      available_.push_back(executors_.back().get());
    }
    max_in_shapes_.resize(plan_.inputs.size());
    for (size_t i = 0; i < plan_.inputs.size(); ++i) max_in_shapes_[i] = max_shape(plan_.inputs[i]);
    max_out_shapes_.resize(plan_.outputs.size());
    for (size_t i = 0; i < plan_.outputs.size(); ++i) max_out_shapes_[i] = max_shape(plan_.outputs[i]);
  }

  ~ModelContainer() {
    // wait for in-flight runs before their buffers disappear
    for (auto& e : executors_) cudaEventSynchronize(e->run_finished());
    executors_.clear();
    for (auto* c : constants_)
      if (c) alloc_.Free(c);
  }

  size_t num_inputs() const { return plan_.inputs.size(); }
  size_t num_outputs() const { return plan_.outputs.size(); }
  size_t num_runtimes() const { return executors_.size(); }
  const TensorInfo& input(size_t i) const {
    if (i >= plan_.inputs.size()) throw std::out_of_range("input index out of range");
    return plan_.tensors[plan_.inputs[i]];
  }
  const TensorInfo& output(size_t i) const {
    if (i >= plan_.outputs.size()) throw std::out_of_range("output index out of range");
    return plan_.tensors[plan_.outputs[i]];
  }
  const std::vector<int64_t>& max_input_shape(size_t i) const { return max_in_shapes_.at(i); }
  const std::vector<int64_t>& max_output_shape(size_t i) const { return max_out_shapes_.at(i); }

  // ------------------------------------------------------------------ constants
  size_t num_constants(bool unbound_only, bool folding_inputs_only) const {
    if (folding_inputs_only) return 0;  // plans carry no constant-folding sub-graph
    size_t n = 0;
    for (auto& c : plan_.constants) n += (!unbound_only || !c.bound) ? 1 : 0;
    return n;
  }
  void constant_names(bool unbound_only, bool folding_inputs_only, const char** out) const {
    if (folding_inputs_only) return;
    size_t k = 0;
    for (auto& c : plan_.constants)
      if (!unbound_only || !c.bound) out[k++] = c.name.c_str();
  }
  const ConstantInfo& constant(const char* name) const {
    if (!name) throw Error("constant name is null");
    auto it = constant_index_.find(name);
    if (it == constant_index_.end()) throw std::out_of_range(std::string("Could not find constant ") + name);
    return plan_.constants[it->second];
  }
  int constant_dtype(const char* name) const { return plan_.tensors[constant(name).tensor].dtype; }
  void set_constant(const char* name, const AITData* tensor, bool double_buffer, cudaStream_t stream) {
    if (!tensor) throw Error("tensor is null");
    const ConstantInfo& c = constant(name);
    const TensorInfo& t = plan_.tensors[c.tensor];
    if (static_cast<int>(tensor->dtype) != t.dtype)
      throw Error(std::string("constant ") + name + ": dtype does not match the model's");
    size_t numel = 1;
    for (size_t i = 0; i < tensor->shape.size; ++i) numel *= static_cast<size_t>(tensor->shape.shape_data[i]);
    if (numel * dtype_size(t.dtype) != static_cast<size_t>(c.nbytes))
      throw Error(std::string("constant ") + name + ": expected " + std::to_string(c.nbytes) + " bytes, got " +
                  std::to_string(numel * dtype_size(t.dtype)));
    if (c.nbytes > 0 && !tensor->ptr) throw Error(std::string("constant ") + name + ": null data pointer");
    std::unique_lock<std::shared_mutex> lock(constants_mutex_);
    const int buf = double_buffer ? 1 - active_ : active_;
    if (!double_buffer) wait_for_all_runs();  // in-flight runs read the active buffer
    ensure_buffer(buf);
    if (c.nbytes > 0) {
      cudaPointerAttributes attr{};
      cudaMemcpyKind kind = cudaMemcpyDefault;
      if (cudaPointerGetAttributes(&attr, tensor->ptr) != cudaSuccess) cudaGetLastError();
      B200AIT_CUDA_CHECK(cudaMemcpyAsync(constants_[buf] + c.offset, tensor->ptr, static_cast<size_t>(c.nbytes), kind, stream));
      B200AIT_CUDA_CHECK(cudaStreamSynchronize(stream));
    }
    constant_set_[buf][constant_index_.at(name)] = true;
  }
  void swap_constants() {
    std::unique_lock<std::shared_mutex> lock(constants_mutex_);
    wait_for_all_runs();
    ensure_buffer(1 - active_);
    // constants that were never written to the inactive buffer keep their current value
    for (size_t i = 0; i < plan_.constants.size(); ++i) {
      if (!constant_set_[1 - active_][i] && constant_set_[active_][i] && plan_.constants[i].nbytes > 0) {
        const ConstantInfo& c = plan_.constants[i];
        B200AIT_CUDA_CHECK(cudaMemcpy(constants_[1 - active_] + c.offset, constants_[active_] + c.offset,
                                      static_cast<size_t>(c.nbytes), cudaMemcpyDeviceToDevice));
        constant_set_[1 - active_][i] = true;
      }
    }
    active_ = 1 - active_;
  }
  void fold_constants(cudaStream_t stream, bool sync, bool double_buffer) {
    // Plans carry no constant-only sub-graph (constants are consumed as given), so folding is a no-op
    // that only honours the synchronisation contract.
    (void)double_buffer;
    if (sync) B200AIT_CUDA_CHECK(cudaStreamSynchronize(stream));
  }

  // ------------------------------------------------------------------------ run
  void run(const AITData* inputs, size_t num_in, AITData* outputs, size_t num_out, cudaStream_t stream, bool sync,
           bool graph_mode, int64_t** output_shapes_out) {
    std::shared_lock<std::shared_mutex> clock(constants_mutex_);
    check_constants_ready();
    Executor* ex = acquire(stream);
    try {
      prepare(*ex, inputs, num_in, outputs, num_out);
      ex->run(stream, graph_mode, constants_[active_]);
      write_output_shapes(*ex, output_shapes_out);
    } catch (...) {
      ex->mark_run_finished(stream);  // an op that threw mid-plan leaves earlier kernels queued
      release(ex);
      throw;
    }
    release(ex);
    if (sync) {
      B200AIT_CUDA_CHECK(cudaStreamSynchronize(stream));
      int status = 0;
      B200AIT_CUDA_CHECK(cudaMemcpy(&status, device_status_word(), sizeof(int), cudaMemcpyDeviceToHost));
      if (status != 0) {
        B200AIT_CUDA_CHECK(cudaMemset(device_status_word(), 0, sizeof(int)));
        throw Error("a kernel gave up waiting (device status " + std::to_string(status) + "); outputs are invalid");
      }
    }
  }

  void run_with_outputs_on_host(const AITData* inputs, size_t num_in, AITData* outputs, size_t num_out,
                                cudaStream_t stream, bool graph_mode, int64_t** output_shapes_out) {
    // device staging buffers sized for the maximum output shapes, then D2H (model_container.cpp:156-206)
    if (num_out != plan_.outputs.size()) throw Error("wrong number of outputs");
    if (!outputs) throw Error("outputs is null");
    std::vector<void*> staging(num_out, nullptr);
    std::vector<AITData> dev(outputs, outputs + num_out);
    std::vector<std::vector<int64_t>> shapes(num_out);
    std::vector<int64_t*> shape_ptrs(num_out);
    try {
      for (size_t i = 0; i < num_out; ++i) {
        size_t bytes = dtype_size(output(i).dtype);
        for (auto d : max_out_shapes_[i]) bytes *= static_cast<size_t>(d);
        staging[i] = alloc_.Allocate(bytes);
        dev[i].ptr = staging[i];
        shapes[i].assign(max_out_shapes_[i].size(), 0);
        shape_ptrs[i] = output_shapes_out ? output_shapes_out[i] : shapes[i].data();
      }
      run(inputs, num_in, dev.data(), num_out, stream, true, graph_mode, shape_ptrs.data());
      for (size_t i = 0; i < num_out; ++i) {
        size_t bytes = dtype_size(output(i).dtype);
        for (size_t d = 0; d < max_out_shapes_[i].size(); ++d) bytes *= static_cast<size_t>(shape_ptrs[i][d]);
        if (bytes) B200AIT_CUDA_CHECK(cudaMemcpy(outputs[i].ptr, staging[i], bytes, cudaMemcpyDeviceToHost));
      }
    } catch (...) {
      for (void* p : staging)
        if (p) alloc_.Free(p);
      throw;
    }
    for (void* p : staging)
      if (p) alloc_.Free(p);
  }

  void profile(const AITData* inputs, size_t num_in, AITData* outputs, size_t num_out, cudaStream_t stream,
               size_t iters, const char* filename) {
    if (!filename) throw Error("filename is null");
    std::shared_lock<std::shared_mutex> clock(constants_mutex_);
    check_constants_ready();
    Executor* ex = acquire(stream);
    try {
      prepare(*ex, inputs, num_in, outputs, num_out);
      ex->profile(stream, iters, filename, constants_[active_]);
    } catch (...) {
      ex->mark_run_finished(stream);
      release(ex);
      throw;
    }
    release(ex);
  }

  float benchmark(const AITData* inputs, size_t num_in, AITData* outputs, size_t num_out, cudaStream_t stream,
                  bool graph_mode, size_t count, size_t num_threads, bool unique_streams, int64_t** output_shapes_out) {
    if (count == 0) throw Error("count must be positive!");
    if (num_threads == 0) num_threads = std::thread::hardware_concurrency();
    if (num_threads <= 1) return benchmark_one(inputs, num_in, outputs, num_out, stream, graph_mode, count, output_shapes_out);
    // multi-threaded: every thread runs `count` inferences into its own copy of the outputs
    // (model_container.cpp:264-363); the time is wall clock over all threads divided by the total runs
    std::vector<std::vector<void*>> outs(num_threads, std::vector<void*>(num_out, nullptr));
    std::vector<std::vector<AITData>> out_data(num_threads, std::vector<AITData>(outputs, outputs + num_out));
    std::vector<cudaStream_t> streams(num_threads, stream);
    std::vector<std::string> errors(num_threads);
    for (size_t t = 1; t < num_threads; ++t) {
      for (size_t i = 0; i < num_out; ++i) {
        size_t bytes = dtype_size(output(i).dtype);
        for (auto d : max_out_shapes_[i]) bytes *= static_cast<size_t>(d);
        outs[t][i] = alloc_.Allocate(bytes);
        out_data[t][i].ptr = outs[t][i];
      }
      if (unique_streams) B200AIT_CUDA_CHECK(cudaStreamCreateWithFlags(&streams[t], cudaStreamNonBlocking));
    }
    run(inputs, num_in, outputs, num_out, stream, true, graph_mode, output_shapes_out);  // warm-up
    const int device = device_;
    auto t0 = std::chrono::steady_clock::now();
    std::vector<std::thread> threads;
    for (size_t t = 0; t < num_threads; ++t) {
      threads.emplace_back([&, t] {
        try {
          cudaSetDevice(device);
          for (size_t i = 0; i < count; ++i)
            run(inputs, num_in, out_data[t].data(), num_out, streams[t], false, graph_mode, nullptr);
          cudaStreamSynchronize(streams[t]);
        } catch (const std::exception& e) {
          errors[t] = e.what();
        }
      });
    }
    for (auto& th : threads) th.join();
    auto t1 = std::chrono::steady_clock::now();
    for (size_t t = 1; t < num_threads; ++t) {
      for (void* p : outs[t])
        if (p) alloc_.Free(p);
      if (unique_streams && streams[t] != stream) cudaStreamDestroy(streams[t]);
    }
    for (auto& e : errors)
      if (!e.empty()) throw Error("benchmark thread failed: " + e);
    const double ms = std::chrono::duration<double, std::milli>(t1 - t0).count();
    return static_cast<float>(ms / static_cast<double>(count * num_threads));
  }

 private:
  float benchmark_one(const AITData* inputs, size_t num_in, AITData* outputs, size_t num_out, cudaStream_t stream,
                      bool graph_mode, size_t count, int64_t** output_shapes_out) {
    // CUDA events around `count` back-to-back runs (model_container.cpp:856-901)
    run(inputs, num_in, outputs, num_out, stream, true, graph_mode, output_shapes_out);  // warm-up
    if (graph_mode) run(inputs, num_in, outputs, num_out, stream, true, graph_mode, output_shapes_out);
    cudaEvent_t e0, e1;
    B200AIT_CUDA_CHECK(cudaEventCreate(&e0));
    B200AIT_CUDA_CHECK(cudaEventCreate(&e1));
    float ms = 0.f;
    try {
      B200AIT_CUDA_CHECK(cudaEventRecord(e0, stream));
      for (size_t i = 0; i < count; ++i) run(inputs, num_in, outputs, num_out, stream, false, graph_mode, nullptr);
      B200AIT_CUDA_CHECK(cudaEventRecord(e1, stream));
      B200AIT_CUDA_CHECK(cudaEventSynchronize(e1));
      B200AIT_CUDA_CHECK(cudaEventElapsedTime(&ms, e0, e1));
    } catch (...) {
      cudaEventDestroy(e0);
      cudaEventDestroy(e1);
      throw;
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    return ms / static_cast<float>(count);
  }

  std::vector<int64_t> max_shape(int t) const {
    std::vector<int64_t> s;
    for (auto& d : plan_.tensors[t].dims) s.push_back(d.is_static ? d.v : plan_.dims[d.v].hi);
    return s;
  }

  void load_bound_constants(const std::string& plan_path) {
    bool any = false;
    for (auto& c : plan_.constants) any = any || (c.bound && c.nbytes > 0);
    if (!any) {
      for (size_t i = 0; i < plan_.constants.size(); ++i)
        if (plan_.constants[i].bound) constant_set_[0][i] = true;
      return;
    }
    if (plan_.constants_file.empty()) throw Error("plan has bound constants but names no constants file");
    std::string path = plan_.constants_file;
    if (path[0] != '/') {
      const size_t slash = plan_path.find_last_of('/');
      path = (slash == std::string::npos ? std::string(".") : plan_path.substr(0, slash)) + "/" + path;
    }
    std::ifstream f(path, std::ios::binary);
    if (!f) throw Error("cannot open constants file " + path);
    std::vector<char> buf;
    for (size_t i = 0; i < plan_.constants.size(); ++i) {
      const ConstantInfo& c = plan_.constants[i];
      if (!c.bound) continue;
      if (c.nbytes > 0) {
        buf.resize(static_cast<size_t>(c.nbytes));
        f.seekg(c.file_offset);
        f.read(buf.data(), c.nbytes);
        if (!f) throw Error("constants file is truncated at constant " + c.name);
        B200AIT_CUDA_CHECK(cudaMemcpy(constants_[0] + c.offset, buf.data(), buf.size(), cudaMemcpyHostToDevice));
      }
      constant_set_[0][i] = true;
    }
  }

  void ensure_buffer(int buf) {
    if (constants_[buf]) return;
    constants_[buf] = static_cast<uint8_t*>(alloc_.Allocate(static_cast<size_t>(std::max<int64_t>(plan_.constants_bytes, 1))));
  }

  void check_constants_ready() const {
    for (size_t i = 0; i < plan_.constants.size(); ++i)
      if (!constant_set_[active_][i])
        throw Error("constant '" + plan_.constants[i].name + "' was never set; call SetConstant before Run");
  }

  void wait_for_all_runs() {
    std::unique_lock<std::mutex> lock(pool_mutex_);
    pool_cv_.wait(lock, [&] { return available_.size() == executors_.size(); });
    for (auto& e : executors_) B200AIT_CUDA_CHECK(cudaEventSynchronize(e->run_finished()));
  }

  // An executor is held only while a run is being ENQUEUED (its host state is the per-run shapes and
  // pointers); reuse of its blob by the next run is ordered on the device, so the host can queue any
  // number of runs ahead of the GPU.
  Executor* acquire(cudaStream_t stream) {
    std::unique_lock<std::mutex> lock(pool_mutex_);
    pool_cv_.wait(lock, [&] { return !available_.empty(); });
    Executor* ex = available_.front();
    available_.pop_front();
    lock.unlock();
    try {
      ex->order_after_previous_run(stream);
    } catch (...) {
      release(ex);
      throw;
    }
    return ex;
  }
  void release(Executor* ex) {
    {
      std::lock_guard<std::mutex> lock(pool_mutex_);
      available_.push_back(ex);
    }
    pool_cv_.notify_all();
  }

  void prepare(Executor& ex, const AITData* inputs, size_t num_in, AITData* outputs, size_t num_out) {
    if (num_in != plan_.inputs.size())
      throw Error("Got wrong number of inputs; expected " + std::to_string(plan_.inputs.size()) + ", got " +
                  std::to_string(num_in));
    if (num_out != plan_.outputs.size())
      throw Error("Got wrong number of outputs; expected " + std::to_string(plan_.outputs.size()) + ", got " +
                  std::to_string(num_out));
    if (num_in > 0 && !inputs) throw Error("inputs cannot be null");
    if (num_out > 0 && !outputs) throw Error("outputs cannot be null");
    RunState& st = ex.state();
    std::fill(st.dim_set.begin(), st.dim_set.end(), 0);
    st.input_ptrs.assign(num_in, nullptr);
    st.output_ptrs.assign(num_out, nullptr);
    for (size_t i = 0; i < num_in; ++i) {
      const TensorInfo& t = input(i);
      if (static_cast<int>(inputs[i].dtype) != t.dtype)
        throw Error("Got wrong dtype for input " + std::to_string(i) + " ('" + t.name + "')");
      if (inputs[i].shape.size > 0 && !inputs[i].shape.shape_data) throw Error("input shape data is null");
      std::vector<int64_t> shape(inputs[i].shape.shape_data, inputs[i].shape.shape_data + inputs[i].shape.size);
      ex.bind_shape(plan_.inputs[i], shape, "input");
      int64_t numel = 1;
      for (auto d : shape) numel *= d;
      if (numel > 0 && !inputs[i].ptr) throw Error("input " + std::to_string(i) + " ('" + t.name + "') has a null pointer");
      st.input_ptrs[i] = inputs[i].ptr;
    }
    for (size_t i = 0; i < num_out; ++i) {
      const TensorInfo& t = output(i);
      if (static_cast<int>(outputs[i].dtype) != t.dtype)
        throw Error("Got wrong dtype for output " + std::to_string(i) + " ('" + t.name + "')");
      int64_t max_numel = 1;
      for (auto d : max_out_shapes_[i]) max_numel *= d;
      if (max_numel > 0 && !outputs[i].ptr)
        throw Error("output " + std::to_string(i) + " ('" + t.name + "') has a null pointer");
      st.output_ptrs[i] = outputs[i].ptr;
    }
  }

  void write_output_shapes(const Executor& ex, int64_t** out) const {
    if (!out) return;
    for (size_t i = 0; i < plan_.outputs.size(); ++i) {
      if (!out[i]) continue;
      const auto s = ex.shape_of(plan_.outputs[i]);
      for (size_t d = 0; d < s.size(); ++d) out[i][d] = s[d];
    }
  }

  Plan plan_;
  DefaultAllocator default_alloc_;
  AITemplateAllocator& alloc_;
  int device_ = 0;
  uint8_t* constants_[2] = {nullptr, nullptr};
  int active_ = 0;
  std::vector<bool> constant_set_[2];
  std::unordered_map<std::string, size_t> constant_index_;
  std::shared_mutex constants_mutex_;
  std::vector<std::unique_ptr<Executor>> executors_;
  std::deque<Executor*> available_;
  std::mutex pool_mutex_;
  std::condition_variable pool_cv_;
  std::vector<std::vector<int64_t>> max_in_shapes_, max_out_shapes_;
};

}  // namespace b200ait

// ------------------------------------------------------------------------------------------- C ABI
using namespace b200ait;

namespace {
template <class F>
AITemplateError convert(const char* where, F&& fn) {
  return guarded(where, std::forward<F>(fn)) == 0 ? AITemplateError::AITemplateSuccess
                                                  : AITemplateError::AITemplateFailure;
}
ModelContainer* as_container(AITemplateModelHandle h) {
  if (!h) throw Error("model handle is null (was the model closed?)");
  return reinterpret_cast<ModelContainer*>(h);
}
cudaStream_t as_stream(AITemplateStreamHandle s) { return reinterpret_cast<cudaStream_t>(s); }
}  // namespace

extern "C" {

AITemplateError AITemplateModelContainerCreateFromPlan(AITemplateModelHandle* ret, const char* plan_path,
                                                       size_t num_runtimes, AITemplateAllocator* allocator) {
  return convert("AITemplateModelContainerCreateFromPlan", [&] {
    if (!ret) throw Error("ret is null");
    if (!plan_path) throw Error("plan_path is null");
    *ret = reinterpret_cast<AITemplateModelHandle>(new ModelContainer(plan_path, num_runtimes, allocator));
  });
}
AITemplateError AITemplateModelContainerCreate(AITemplateModelHandle* ret, size_t num_runtimes,
                                               AITemplateAllocator* allocator) {
  return convert("AITemplateModelContainerCreate", [&] {
    if (!ret) throw Error("ret is null");
    const char* plan = getenv("B200AIT_PLAN");
    if (!plan) throw Error("this library serves every model: set B200AIT_PLAN or call AITemplateModelContainerCreateFromPlan");
    *ret = reinterpret_cast<AITemplateModelHandle>(new ModelContainer(plan, num_runtimes, allocator));
  });
}
AITemplateError AITemplateModelContainerDelete(AITemplateModelHandle handle) {
  return convert("AITemplateModelContainerDelete", [&] {
    if (handle) delete reinterpret_cast<ModelContainer*>(handle);
  });
}
AITemplateError AITemplateModelContainerSetConstant(AITemplateModelHandle handle, const char* name,
                                                    const AITData* tensor) {
  return convert("AITemplateModelContainerSetConstant", [&] { as_container(handle)->set_constant(name, tensor, false, nullptr); });
}
AITemplateError AITemplateModelContainerSetManyConstants(AITemplateModelHandle handle, const char** names,
                                                         const AITData* tensors, size_t num_tensors) {
  return convert("AITemplateModelContainerSetManyConstants", [&] {
    auto* m = as_container(handle);
    if (num_tensors && (!names || !tensors)) throw Error("names / tensors is null");
    for (size_t i = 0; i < num_tensors; ++i) m->set_constant(names[i], &tensors[i], false, nullptr);
  });
}
AITemplateError AITemplateModelContainerSetDoubleBufferConstant(AITemplateModelHandle handle,
                                                                AITemplateStreamHandle stream_handle,
                                                                const char* name, const AITData* tensor) {
  return convert("AITemplateModelContainerSetDoubleBufferConstant",
                 [&] { as_container(handle)->set_constant(name, tensor, true, as_stream(stream_handle)); });
}
AITemplateError AITemplateModelContainerSetManyDoubleBufferConstants(AITemplateModelHandle handle,
                                                                     AITemplateStreamHandle stream_handle,
                                                                     const char** names, const AITData* tensors,
                                                                     size_t num_tensors) {
  return convert("AITemplateModelContainerSetManyDoubleBufferConstants", [&] {
    auto* m = as_container(handle);
    if (num_tensors && (!names || !tensors)) throw Error("names / tensors is null");
    for (size_t i = 0; i < num_tensors; ++i) m->set_constant(names[i], &tensors[i], true, as_stream(stream_handle));
  });
}
AITemplateError AITemplateModelContainerGetNumConstants(AITemplateModelHandle handle, bool unbound_constants_only,
                                                        bool constant_folding_inputs_only,
                                                        size_t* num_constants_out) {
  return convert("AITemplateModelContainerGetNumConstants", [&] {
    if (!num_constants_out) throw Error("num_constants_out is null");
    *num_constants_out = as_container(handle)->num_constants(unbound_constants_only, constant_folding_inputs_only);
  });
}
AITemplateError AITemplateModelContainerGetConstantNames(AITemplateModelHandle handle, bool unbound_constants_only,
                                                         bool constant_folding_inputs_only,
                                                         const char** constant_names_out) {
  return convert("AITemplateModelContainerGetConstantNames", [&] {
    auto* m = as_container(handle);
    if (!constant_names_out && m->num_constants(unbound_constants_only, constant_folding_inputs_only) > 0)
      throw Error("constant_names_out is null");
    m->constant_names(unbound_constants_only, constant_folding_inputs_only, constant_names_out);
  });
}
AITemplateError AITemplateModelContainerGetConstantDtype(AITemplateModelHandle handle, const char* name,
                                                         AITemplateDtype* dtype) {
  return convert("AITemplateModelContainerGetConstantDtype", [&] {
    if (!dtype) throw Error("dtype is null");
    auto* m = as_container(handle);
    *dtype = static_cast<AITemplateDtype>(m->constant_dtype(name));
  });
}
AITemplateError AITemplateModelContainerGetConstantOriginalName(AITemplateModelHandle handle, const char* name,
                                                                const char** original_name_out) {
  return convert("AITemplateModelContainerGetConstantOriginalName", [&] {
    if (!original_name_out) throw Error("original_name_out is null");
    *original_name_out = as_container(handle)->constant(name).original_name.c_str();
  });
}
AITemplateError AITemplateModelContainerRun(AITemplateModelHandle handle, const AITData* inputs, size_t num_inputs,
                                            AITData* outputs, size_t num_outputs,
                                            AITemplateStreamHandle stream_handle, bool sync, bool graph_mode,
                                            int64_t** output_shapes_out) {
  return convert("AITemplateModelContainerRun", [&] {
    as_container(handle)->run(inputs, num_inputs, outputs, num_outputs, as_stream(stream_handle), sync, graph_mode,
                              output_shapes_out);
  });
}
AITemplateError AITemplateModelContainerRunWithOutputsOnHost(AITemplateModelHandle handle, const AITData* inputs,
                                                             size_t num_inputs, AITData* outputs, size_t num_outputs,
                                                             AITemplateStreamHandle stream_handle, bool graph_mode,
                                                             int64_t** output_shapes_out) {
  return convert("AITemplateModelContainerRunWithOutputsOnHost", [&] {
    as_container(handle)->run_with_outputs_on_host(inputs, num_inputs, outputs, num_outputs, as_stream(stream_handle),
                                                   graph_mode, output_shapes_out);
  });
}
AITemplateError AITemplateModelContainerProfile(AITemplateModelHandle handle, const AITData* inputs,
                                                size_t num_inputs, AITData* outputs, size_t num_outputs,
                                                AITemplateStreamHandle stream_handle, size_t num_iters,
                                                const char* filename) {
  return convert("AITemplateModelContainerProfile", [&] {
    as_container(handle)->profile(inputs, num_inputs, outputs, num_outputs, as_stream(stream_handle), num_iters,
                                  filename);
  });
}
AITemplateError AITemplateModelContainerBenchmark(AITemplateModelHandle handle, const AITData* inputs,
                                                  size_t num_inputs, AITData* outputs, size_t num_outputs,
                                                  AITemplateStreamHandle stream_handle, bool graph_mode, size_t count,
                                                  size_t num_threads, bool use_unique_stream_per_thread,
                                                  float* runtime_ms, int64_t** output_shapes_out) {
  return convert("AITemplateModelContainerBenchmark", [&] {
    if (!runtime_ms) throw Error("runtime_ms is null");
    *runtime_ms = as_container(handle)->benchmark(inputs, num_inputs, outputs, num_outputs, as_stream(stream_handle),
                                                  graph_mode, count, num_threads, use_unique_stream_per_thread,
                                                  output_shapes_out);
  });
}
AITemplateError AITemplateModelContainerGetNumInputs(AITemplateModelHandle handle, size_t* num_inputs_out) {
  return convert("AITemplateModelContainerGetNumInputs", [&] {
    if (!num_inputs_out) throw Error("num_inputs_out is null");
    *num_inputs_out = as_container(handle)->num_inputs();
  });
}
AITemplateError AITemplateModelContainerGetInputName(AITemplateModelHandle handle, size_t input_idx,
                                                     const char** input_name_out) {
  return convert("AITemplateModelContainerGetInputName", [&] {
    if (!input_name_out) throw Error("input_name_out is null");
    *input_name_out = as_container(handle)->input(input_idx).name.c_str();
  });
}
AITemplateError AITemplateModelContainerGetMaximumInputShape(AITemplateModelHandle handle, size_t input_idx,
                                                             AITemplateParamShape* shape) {
  return convert("AITemplateModelContainerGetMaximumInputShape", [&] {
    if (!shape) throw Error("shape is null");
    const auto& s = as_container(handle)->max_input_shape(input_idx);
    *shape = AITemplateParamShape(s.data(), s.size());
  });
}
AITemplateError AITemplateModelContainerGetInputDtype(AITemplateModelHandle handle, size_t input_idx,
                                                      AITemplateDtype* input_dtype) {
  return convert("AITemplateModelContainerGetInputDtype", [&] {
    if (!input_dtype) throw Error("input_dtype is null");
    *input_dtype = static_cast<AITemplateDtype>(as_container(handle)->input(input_idx).dtype);
  });
}
AITemplateError AITemplateModelContainerGetNumOutputs(AITemplateModelHandle handle, size_t* num_outputs_out) {
  return convert("AITemplateModelContainerGetNumOutputs", [&] {
    if (!num_outputs_out) throw Error("num_outputs_out is null");
    *num_outputs_out = as_container(handle)->num_outputs();
  });
}
AITemplateError AITemplateModelContainerGetOutputName(AITemplateModelHandle handle, size_t output_idx,
                                                      const char** output_name_out) {
  return convert("AITemplateModelContainerGetOutputName", [&] {
    if (!output_name_out) throw Error("output_name_out is null");
    *output_name_out = as_container(handle)->output(output_idx).name.c_str();
  });
}
AITemplateError AITemplateModelContainerGetMaximumOutputShape(AITemplateModelHandle handle, size_t output_idx,
                                                              AITemplateParamShape* shape_out) {
  return convert("AITemplateModelContainerGetMaximumOutputShape", [&] {
    if (!shape_out) throw Error("shape_out is null");
    const auto& s = as_container(handle)->max_output_shape(output_idx);
    *shape_out = AITemplateParamShape(s.data(), s.size());
  });
}
AITemplateError AITemplateModelContainerGetOutputDtype(AITemplateModelHandle handle, size_t output_idx,
                                                       AITemplateDtype* out) {
  return convert("AITemplateModelContainerGetOutputDtype", [&] {
    if (!out) throw Error("out is null");
    *out = static_cast<AITemplateDtype>(as_container(handle)->output(output_idx).dtype);
  });
}
AITemplateError AITemplateModelContainerGetNumRuntimes(AITemplateModelHandle handle, size_t* num_runtimes_out) {
  return convert("AITemplateModelContainerGetNumRuntimes", [&] {
    if (!num_runtimes_out) throw Error("num_runtimes_out is null");
    *num_runtimes_out = as_container(handle)->num_runtimes();
  });
}
AITemplateError AITemplateModelContainerFoldConstants(AITemplateModelHandle handle,
                                                      AITemplateStreamHandle stream_handle, bool sync) {
  return convert("AITemplateModelContainerFoldConstants",
                 [&] { as_container(handle)->fold_constants(as_stream(stream_handle), sync, false); });
}
AITemplateError AITemplateModelContainerFoldConstantsInDoubleBuffer(AITemplateModelHandle handle,
                                                                    AITemplateStreamHandle stream_handle, bool sync) {
  return convert("AITemplateModelContainerFoldConstantsInDoubleBuffer",
                 [&] { as_container(handle)->fold_constants(as_stream(stream_handle), sync, true); });
}
AITemplateError AITemplateModelContainerSwapConstants(AITemplateModelHandle handle) {
  return convert("AITemplateModelContainerSwapConstants", [&] { as_container(handle)->swap_constants(); });
}
AITemplateError AITemplateAllocatorCreate(AITemplateAllocator** allocator_out, AITemplateAllocatorType allocator_type) {
  return convert("AITemplateAllocatorCreate", [&] {
    if (!allocator_out) throw Error("allocator_out is null");
    switch (allocator_type) {
      case AITemplateAllocatorType::kDefault: *allocator_out = new DefaultAllocator(); break;
      case AITemplateAllocatorType::kTracking: *allocator_out = new TrackingAllocator(); break;
      default: throw Error("Unrecognized allocator type");
    }
  });
}
AITemplateError AITemplateAllocatorDelete(AITemplateAllocator* allocator) {
  return convert("AITemplateAllocatorDelete", [&] { delete allocator; });
}
AITemplateError AITemplateTrackingAllocatorGetNumBytes(AITemplateAllocator* allocator, size_t* num_bytes_out) {
  return convert("AITemplateTrackingAllocatorGetNumBytes", [&] {
    if (!allocator || !num_bytes_out) throw Error("allocator / num_bytes_out is null");
    auto* t = dynamic_cast<TrackingAllocator*>(allocator);
    if (!t) throw Error("Allocator was not a tracking allocator!");
    *num_bytes_out = t->NumBytesAllocated();
  });
}
AITemplateError AITemplateDeviceMalloc(void** ptr_out, size_t size, AITemplateStreamHandle stream_handle, bool sync) {
  return convert("AITemplateDeviceMalloc", [&] {
    if (!ptr_out) throw Error("ptr_out is null");
    B200AIT_CUDA_CHECK(cudaMallocAsync(ptr_out, size, as_stream(stream_handle)));
    if (sync) B200AIT_CUDA_CHECK(cudaStreamSynchronize(as_stream(stream_handle)));
  });
}
AITemplateError AITemplateDeviceFree(void* ptr, AITemplateStreamHandle stream_handle, bool sync) {
  return convert("AITemplateDeviceFree", [&] {
    B200AIT_CUDA_CHECK(cudaFreeAsync(ptr, as_stream(stream_handle)));
    if (sync) B200AIT_CUDA_CHECK(cudaStreamSynchronize(as_stream(stream_handle)));
  });
}
AITemplateError AITemplateMemcpy(void* dst, const void* src, size_t count, AITemplateMemcpyKind kind,
                                 AITemplateStreamHandle stream_handle, bool sync) {
  return convert("AITemplateMemcpy", [&] {
    cudaMemcpyKind k;
    switch (kind) {
      case AITemplateMemcpyKind::HostToDevice: k = cudaMemcpyHostToDevice; break;
      case AITemplateMemcpyKind::DeviceToHost: k = cudaMemcpyDeviceToHost; break;
      case AITemplateMemcpyKind::DeviceToDevice: k = cudaMemcpyDeviceToDevice; break;
      default: throw Error("unknown memcpy kind");
    }
    B200AIT_CUDA_CHECK(cudaMemcpyAsync(dst, src, count, k, as_stream(stream_handle)));
    if (sync) B200AIT_CUDA_CHECK(cudaStreamSynchronize(as_stream(stream_handle)));
  });
}

}  // extern "C"
