// Host layer behind the C ABI of include/qfg.h: attribute validation, per-call shape and type
// checks, segment tables, launch planning and error reporting.  It plays the part of the
// reference's Ort::CustomOpBase kernel-state structs (src/fused_gemm/fused_gemm.cu:468-593 for
// SkinnyGemm, :731-779 for ArgmaxRows, :842-954 for DequantWeightBf16) with ORT's tensor and
// attribute accessors replaced by plain arguments.  Nothing here synchronises, and the compute
// entry points neither allocate nor copy, so they are legal inside a stream capture.
#include <cuda_runtime.h>

#include <chrono>

#include <climits>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <stdexcept>
#include <string>
#include <vector>

#include "qfg_internal.h"

namespace {

thread_local std::string g_last_error;

int Fail(int code, const std::string& msg) {
  g_last_error = msg;
  return code;
}

struct InvalidArgument : std::runtime_error {
  using std::runtime_error::runtime_error;
};

int Alignment(const void* base, long long pitch) {
  const uintptr_t a = reinterpret_cast<uintptr_t>(base);
  for (int v = 16; v >= 4; v >>= 1) {
    if (a % v == 0 && pitch % v == 0) return v;
  }
  return 0;
}

float* UploadScales(const float* host, size_t n, const char* op) {
  if (host == nullptr || n == 0) return nullptr;
  float* dev = nullptr;
  if (cudaMalloc(&dev, n * sizeof(float)) != cudaSuccess ||
      cudaMemcpy(dev, host, n * sizeof(float), cudaMemcpyHostToDevice) != cudaSuccess) {
    cudaFree(dev);
    cudaGetLastError();
    throw std::runtime_error(std::string(op) + ": failed to upload w_scale");
  }
  return dev;
}

// Optional `trigger` attribute; SKINNY_TRIGGER_FORCE=<n> overrides a non-zero value.
int ResolveTrigger(int attr) {
  const char* e = std::getenv("SKINNY_TRIGGER_FORCE");
  return (attr != 0 && e != nullptr) ? std::atoi(e) : attr;
}

int EnvInt(const char* name, int dflt) {
  const char* e = std::getenv(name);
  return e != nullptr ? std::atoi(e) : dflt;
}

}  // namespace

struct qfg_skinny_gemm {
  std::vector<int> seg_outs;
  std::vector<int> widths;
  int trigger = 0;
  float* d_w_scale = nullptr;
  size_t w_scale_len = 0;
  int pdl_wait = 0;
  int force_slow = 0;
  int exchange_spin = qfg::kExchangeSpin;  // sharded LM head: bound of the wait for a peer's keys (iterations)
  int dense_rows = -1;  // calls with more rows take the dequantise + library GEMM branch; -1 = qfg::DenseRowsDefault(mode), 0 = never
  unsigned long long phase_times = 0;  // device address given through set_option("phase_times", ...)
  std::string plan_spec;
  // plans already computed for this node, keyed by the shape of the call
  mutable std::mutex plan_mu;
  mutable std::map<std::string, qfg::Plan> plans;
  // the shape of the last call and its plan: a decode loop repeats one shape, and comparing a few integers is
  // cheaper than building the map's key
  mutable bool last_valid = false;
  mutable qfg::PlanInput last_in;
  mutable std::string last_spec;
  mutable qfg::Plan last_plan;
  qfg_skinny_gemm() = default;
  qfg_skinny_gemm(const qfg_skinny_gemm& o)
      : seg_outs(o.seg_outs), widths(o.widths), trigger(o.trigger), d_w_scale(o.d_w_scale), w_scale_len(o.w_scale_len),
        pdl_wait(o.pdl_wait), force_slow(o.force_slow), exchange_spin(o.exchange_spin), dense_rows(o.dense_rows), phase_times(o.phase_times),
        plan_spec(o.plan_spec) {}
};

struct qfg_dequant {
  int64_t n_cols = 0;
  int64_t col_offset = 0;
  std::vector<int> widths;
  float* d_w_scale = nullptr;
  size_t w_scale_len = 0;
};

struct qfg_lmhead {
  qfg_skinny_gemm gemm;
};

struct qfg_shared_expert_down {
  qfg_skinny_gemm gemm;
};

struct qfg_untile_hc {
  int kind = 0;
  float* d_w_scale = nullptr;
  size_t w_scale_len = 0;
};

namespace {

struct Prepared {
  qfg::GemmParams params;
  qfg::PlanInput plan_in;
  int mode = 0;
};

// Shape / type checks and segment tables of one call (fused_gemm.cu:512-572).  `outs` may be
// null when only the plan is wanted.
Prepared Prepare(const qfg_skinny_gemm& op, const void* x, int64_t m, int64_t k, const qfg_tensor2d* weights,
                 int n_weights, void* const* outs, int n_outs, bool need_outs, int64_t single_width = 0) {
  const int nseg = static_cast<int>(op.seg_outs.size());
  if (n_weights != nseg) throw InvalidArgument("SkinnyGemm: input count");
  if (m < 1) throw InvalidArgument("SkinnyGemm: M must be >= 1");
  if (k < 1 || k > INT_MAX) throw InvalidArgument("SkinnyGemm: bad K");
  if (k % 2 != 0) throw InvalidArgument("SkinnyGemm: K must be even");
  if (need_outs && n_outs != static_cast<int>(op.widths.size())) throw InvalidArgument("SkinnyGemm: output count");
  if (need_outs && (x == nullptr || reinterpret_cast<uintptr_t>(x) % 4 != 0))
    throw InvalidArgument("SkinnyGemm: x must be a 4-byte aligned device pointer");

  Prepared pr;
  qfg::GemmParams& p = pr.params;
  p.x = static_cast<const uint16_t*>(x);
  p.K = static_cast<int>(k);
  p.nseg = nseg;
  p.trigger = op.trigger;
  p.pdl_wait = op.pdl_wait;
  p.force_slow = op.force_slow;
  p.phase_times = reinterpret_cast<unsigned long long*>(static_cast<uintptr_t>(op.phase_times));
  int o = 0;
  size_t scale_off = 0;
  int row_align = 16;
  for (int s = 0; s < nseg; ++s) {
    const qfg_tensor2d& w = weights[s];
    if (w.rows != k) throw InvalidArgument("SkinnyGemm: weight shape");
    qfg::Segment& sg = p.seg[s];
    sg.out_begin = o;
    long long begin = 0;
    for (int i = 0; i < op.seg_outs[s]; ++i, ++o) {
      // the fused LM head passes the shard width per call instead of as an attribute
      const int64_t width = single_width > 0 ? single_width : op.widths[o];
      if (width < 1 || width > INT_MAX) throw InvalidArgument("SkinnyGemm: widths must be positive");
      p.out[o] = need_outs ? static_cast<uint16_t*>(outs[o]) : nullptr;
      if (need_outs && outs[o] == nullptr) throw InvalidArgument("SkinnyGemm: null output");
      p.col_begin[o] = static_cast<int>(begin);
      p.width[o] = static_cast<int>(width);
      begin += width;
    }
    sg.out_end = o;
    if (begin > INT_MAX) throw InvalidArgument("SkinnyGemm: N too large");
    sg.n = static_cast<int>(begin);
    int mode;
    if (w.dtype == QFG_BFLOAT16) {
      if (w.cols != begin) throw InvalidArgument("SkinnyGemm: widths do not add up to N");
      mode = qfg::kBf16;
      sg.pitch = 2 * begin;
    } else if (w.dtype == QFG_FLOAT8E4M3FN) {
      if (w.cols != begin) throw InvalidArgument("SkinnyGemm: FP8 widths do not add up to N");
      mode = qfg::kFp8;
      sg.pitch = begin;
    } else if (w.dtype == QFG_UINT8) {
      if (begin % 16 != 0 || w.cols != (begin * 9) / 16)
        throw InvalidArgument("SkinnyGemm: NVFP4 packed width must equal N * 9 / 16");
      if (begin % 64 != 0) throw InvalidArgument("SkinnyGemm: NVFP4 needs N % 64 == 0 (4-byte aligned rows)");
      mode = qfg::kNvfp4;
      sg.pitch = (begin * 9) / 16;
    } else {
      throw InvalidArgument("SkinnyGemm: unsupported weight element type");
    }
    if (mode != qfg::kBf16 && op.d_w_scale != nullptr && scale_off + static_cast<size_t>(begin) <= op.w_scale_len) {
      sg.w_scale = op.d_w_scale + scale_off;
      scale_off += static_cast<size_t>(begin);
    }
    if (sg.n % 4 != 0) throw InvalidArgument("SkinnyGemm: N must be a multiple of 4");
    if (s == 0) {
      pr.mode = mode;
    } else if (mode != pr.mode) {
      throw InvalidArgument("SkinnyGemm: all weights of one call must share one element type");
    }
    sg.w = static_cast<const uint8_t*>(w.data);
    sg.total_bytes = sg.pitch * k;
    if (need_outs) {
      if (w.data == nullptr) throw InvalidArgument("SkinnyGemm: null weight");
      int a = Alignment(w.data, sg.pitch);
      if (a == 0) throw InvalidArgument("SkinnyGemm: weight rows must be 4-byte aligned");
      // the streaming kernel copies aligned 16-byte pieces: it needs a 16-byte aligned base even
      // where the pitch is only a multiple of 8
      if (a == 8 && reinterpret_cast<uintptr_t>(w.data) % 16 != 0) a = 4;
      row_align = std::min(row_align, a);
    } else {
      row_align = std::min(row_align, Alignment(nullptr, sg.pitch) == 0 ? 4 : Alignment(nullptr, sg.pitch));
    }
    pr.plan_in.n[s] = sg.n;
  }
  for (int s = 0; s < nseg; ++s) {
    p.seg[s].vec = row_align;
    p.seg[s].svec = row_align;
  }
  pr.plan_in.K = p.K;
  pr.plan_in.nseg = nseg;
  pr.plan_in.mode = pr.mode;
  pr.plan_in.row_align = row_align;
  pr.plan_in.sm_count = qfg::DeviceSmCount();
  pr.plan_in.max_clusters = need_outs ? &qfg::QueryMaxActiveClusters : nullptr;
  return pr;
}

qfg::Plan ComputePlan(const qfg_skinny_gemm& op, const qfg::PlanInput& in);

bool SamePlanInput(const qfg::PlanInput& a, const qfg::PlanInput& b) {
  if (a.K != b.K || a.nseg != b.nseg || a.mode != b.mode || a.row_align != b.row_align || a.sm_count != b.sm_count ||
      a.max_rows != b.max_rows || a.max_clusters != b.max_clusters || a.allow_tail != b.allow_tail) {
    return false;
  }
  for (int s = 0; s < a.nseg; ++s) {
    if (a.n[s] != b.n[s]) return false;
  }
  return true;
}

qfg::Plan PlanFor(const qfg_skinny_gemm& op, qfg::PlanInput in, int rows) {
  in.max_rows = rows;
  {
    std::lock_guard<std::mutex> lock(op.plan_mu);
    if (op.last_valid && SamePlanInput(op.last_in, in) && op.last_spec == op.plan_spec) return op.last_plan;
  }
  auto remember = [&](const qfg::Plan& plan) {  // caller holds plan_mu
    op.last_in = in;
    op.last_spec = op.plan_spec;
    op.last_plan = plan;
    op.last_valid = true;
  };
  std::string key = std::to_string(in.K) + "/" + std::to_string(in.mode) + "/" + std::to_string(in.row_align) + "/" +
                    std::to_string(rows) + "/" + (in.max_clusters != nullptr ? "d" : "h") + (in.allow_tail ? "t" : "");
  for (int s = 0; s < in.nseg; ++s) key += "/" + std::to_string(in.n[s]);
  {
    std::lock_guard<std::mutex> lock(op.plan_mu);
    auto it = op.plans.find(key + "|" + op.plan_spec);
    if (it != op.plans.end()) {
      remember(it->second);
      return it->second;
    }
  }
  qfg::Plan plan = ComputePlan(op, in);
  std::lock_guard<std::mutex> lock(op.plan_mu);
  op.plans[key + "|" + op.plan_spec] = plan;
  remember(plan);
  return plan;
}

qfg::Plan ComputePlan(const qfg_skinny_gemm& op, const qfg::PlanInput& in) {
  qfg::Plan plan = qfg::ChoosePlan(in);
  std::string spec = op.plan_spec;
  if (spec.empty()) {
    const char* e = std::getenv("QFG_PLAN");
    if (e != nullptr) spec = e;
  }
  if (!spec.empty() && !qfg::ApplyPlanOverrides(spec, in, &plan)) throw InvalidArgument("SkinnyGemm: bad plan override");
  qfg::FinishPlan(in, spec, &plan);
  return plan;
}

// Launches row blocks of at most eight rows; only the last block may release PDL dependents
// (skinny_gemm.cuh:661-676 does the same with blocks of four).
void Run(const qfg_skinny_gemm& op, Prepared& pr, int64_t m, cudaStream_t stream, const char* name) {
  const int dense_rows = op.dense_rows < 0 ? qfg::DenseRowsDefault(pr.mode) : op.dense_rows;
  if (dense_rows > 0 && m > dense_rows && qfg::DenseEligible(pr.params)) {
    qfg::LaunchDenseGemm(pr.mode, pr.params, m, stream);
    return;
  }
  const qfg::Plan plan = PlanFor(op, pr.plan_in, static_cast<int>(std::min<int64_t>(m, qfg::kMaxRows)));
  qfg::GemmParams base = pr.params;
  int64_t done = 0;
  while (done < m) {
    const int chunk = static_cast<int>(std::min<int64_t>(m - done, qfg::kMaxRows));
    qfg::GemmParams q = base;
    q.M = chunk;
    q.x = base.x + static_cast<size_t>(done) * base.K;
    if (base.fuse) {
      q.x2 = base.x2 + static_cast<size_t>(done) * base.K;
      q.gx = base.gx + static_cast<size_t>(done) * base.gk;
      if (base.routed != nullptr) q.routed = base.routed + static_cast<size_t>(done) * base.seg[0].n;
    }
    if (done + chunk < m) q.trigger = 0;
    const int n_out = base.seg[base.nseg - 1].out_end;
    for (int o = 0; o < n_out; ++o) {
      if (base.out[o] != nullptr) q.out[o] = base.out[o] + static_cast<size_t>(done) * base.width[o];
    }
    if (q.lm) {
      if (m > qfg::kMaxRows) throw InvalidArgument(std::string(name) + ": at most 8 rows per call");
    }
    cudaError_t err = qfg::LaunchSkinnyGemm(pr.mode, q, plan, stream);
    if (err == cudaSuccess) err = cudaGetLastError();
    if (err != cudaSuccess) throw std::runtime_error(std::string(name) + ": " + cudaGetErrorString(err));
    done += chunk;
  }
}

void InitGemmOp(qfg_skinny_gemm* op, const int64_t* seg_outs, int n_seg, const int64_t* widths, int n_widths,
                const float* w_scale, size_t n_w_scale, int trigger, const char* name) {
  if (n_seg < 0 || n_widths < 0 || (n_seg > 0 && seg_outs == nullptr) || (n_widths > 0 && widths == nullptr))
    throw InvalidArgument(std::string(name) + ": bad seg_outs/widths");
  long long total = 0;
  for (int i = 0; i < n_seg; ++i) {
    if (seg_outs[i] < 1 || seg_outs[i] > qfg::kMaxOut) throw InvalidArgument(std::string(name) + ": bad seg_outs/widths");
    op->seg_outs.push_back(static_cast<int>(seg_outs[i]));
    total += seg_outs[i];
  }
  for (int i = 0; i < n_widths; ++i) {
    if (widths[i] < 1 || widths[i] > INT_MAX) throw InvalidArgument(std::string(name) + ": bad seg_outs/widths");
    op->widths.push_back(static_cast<int>(widths[i]));
  }
  if (op->seg_outs.empty() || op->seg_outs.size() > static_cast<size_t>(qfg::kMaxSeg) || total != n_widths ||
      total > qfg::kMaxOut) {
    throw InvalidArgument(std::string(name) + ": bad seg_outs/widths");
  }
  op->trigger = ResolveTrigger(trigger);
  op->pdl_wait = EnvInt("QFG_PDL_WAIT", 0);
  const cudaError_t err = qfg::ConfigureSkinnyGemmKernels();
  if (err != cudaSuccess) throw std::runtime_error(std::string(name) + ": " + cudaGetErrorString(err));
  op->d_w_scale = UploadScales(w_scale, n_w_scale, name);
  op->w_scale_len = op->d_w_scale != nullptr ? n_w_scale : 0;
}

int SetGemmOption(qfg_skinny_gemm* op, const char* key, const char* value) {
  if (op == nullptr || key == nullptr || value == nullptr) return Fail(QFG_INVALID_ARGUMENT, "set_option: null argument");
  const std::string k = key;
  if (k == "pdl_wait") op->pdl_wait = std::atoi(value);
  else if (k == "force_slow") op->force_slow = std::atoi(value);
  else if (k == "dense_rows") op->dense_rows = std::atoi(value);
  else if (k == "exchange_spin") op->exchange_spin = std::max(0, std::atoi(value));
#ifdef QFG_PHASE_TIMES
  else if (k == "phase_times") op->phase_times = std::strtoull(value, nullptr, 10);  // measurement builds only
#endif
  else if (k == "plan") op->plan_spec = value;
  else if (k == "trigger") op->trigger = std::atoi(value);
  else return Fail(QFG_INVALID_ARGUMENT, "set_option: unknown key " + k);
  return QFG_OK;
}

}  // namespace

namespace qfg {

int SetLastError(int code, const char* message) { return Fail(code, message); }

// The fused LM head on a caller-chosen scratch area (see qfg_lmhead_compute).
int LmheadComputeWithWorkspace(const qfg_lmhead* op, const void* x, int64_t m, int64_t k, const qfg_tensor2d* weight,
                       int64_t n, int64_t col_offset, void* workspace, size_t workspace_bytes, int64_t* idx, float* val,
                       uint64_t* key, void* logits, void* stream, const qfg_lmhead_exchange* exchange,
                       unsigned int* status_out) {
  if (op == nullptr || weight == nullptr) return Fail(QFG_FAIL, "LmHead: null argument");
  try {
    if (workspace == nullptr || reinterpret_cast<uintptr_t>(workspace) % 8 != 0)
      throw InvalidArgument("LmHead: workspace must be an 8-byte aligned device pointer");
    if (n < 1 || n > INT_MAX || col_offset < 0 || col_offset + n > 0xFFFFFFFELL)
      throw InvalidArgument("LmHead: bad vocabulary range");
    if (m < 1 || m > qfg::kMaxRows) throw InvalidArgument("LmHead: 1 <= rows <= 8");
    const qfg_skinny_gemm& call = op->gemm;
    void* outs[1] = {logits};
    Prepared pr = Prepare(call, x, m, k, weight, 1, outs, 1, false, n);
    if (x == nullptr || reinterpret_cast<uintptr_t>(x) % 4 != 0 || weight->data == nullptr)
      throw InvalidArgument("LmHead: null or misaligned input");
    int a = Alignment(weight->data, pr.params.seg[0].pitch);
    if (a == 0) throw InvalidArgument("LmHead: weight rows must be 4-byte aligned");
    if (a == 8 && reinterpret_cast<uintptr_t>(weight->data) % 16 != 0) a = 4;
    pr.params.seg[0].vec = pr.params.seg[0].svec = a;
    pr.plan_in.row_align = a;
    pr.plan_in.max_clusters = &qfg::QueryMaxActiveClusters;
    pr.plan_in.allow_tail = workspace_bytes >= qfg::kLmHeaderBytes + qfg::kLmTailBytes;
    if (pr.plan_in.allow_tail) pr.params.lm_tail = reinterpret_cast<float*>(static_cast<char*>(workspace) + qfg::kLmHeaderBytes);
    pr.params.out[0] = static_cast<uint16_t*>(logits);
    pr.params.lm = 1;
    pr.params.lm_keys = static_cast<unsigned long long*>(workspace);
    pr.params.lm_count = reinterpret_cast<unsigned int*>(static_cast<unsigned long long*>(workspace) + qfg::kMaxRows);
    pr.params.lm_idx = reinterpret_cast<long long*>(idx);
    pr.params.lm_val = val;
    pr.params.lm_key_out = reinterpret_cast<unsigned long long*>(key);
    pr.params.lm_col_offset = col_offset;
    if (exchange != nullptr && exchange->world > 1) {
      if (exchange->world > QFG_MAX_RANKS || exchange->rank < 0 || exchange->rank >= exchange->world)
        throw InvalidArgument("LmHead: bad exchange (1 <= world <= 8, 0 <= rank < world)");
      pr.params.xworld = exchange->world;
      pr.params.xrank = exchange->rank;
      pr.params.xspin = call.exchange_spin;
      pr.params.lm_status_out = status_out;
      for (int r = 0; r < exchange->world; ++r) {
        if (exchange->peers[r] == nullptr || reinterpret_cast<uintptr_t>(exchange->peers[r]) % 8 != 0)
          throw InvalidArgument("LmHead: exchange buffers must be 8-byte aligned device pointers");
        pr.params.xpeer[r] = static_cast<qfg::LmExchange*>(exchange->peers[r]);
      }
    }
    Run(call, pr, m, static_cast<cudaStream_t>(stream), "LmHead");
    return QFG_OK;
  } catch (const InvalidArgument& e) {
    return Fail(QFG_INVALID_ARGUMENT, e.what());
  } catch (const std::exception& e) {
    return Fail(QFG_FAIL, e.what());
  }
}

}  // namespace qfg

namespace {

// The input copy of the host step as a kernel, so that the fused kernel can be its programmatic dependent:
// it releases the dependent at once, and the dependent streams its first weight tiles while these few
// kilobytes cross the host link, waiting (griddepcontrol.wait) only before it reads x.  `src` is pinned host
// memory addressed by the device.
template <typename V>
__global__ void __launch_bounds__(256) HostRowsToDeviceKernel(const V* __restrict__ src, V* __restrict__ dst, size_t n) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += static_cast<size_t>(gridDim.x) * blockDim.x)
    dst[i] = src[i];
}

cudaError_t LaunchHostRowsToDevice(const void* src, void* dst, size_t bytes, cudaStream_t stream) {
  const bool v16 = bytes % 16 == 0 && reinterpret_cast<uintptr_t>(src) % 16 == 0 && reinterpret_cast<uintptr_t>(dst) % 16 == 0;
  const size_t n = v16 ? bytes / 16 : bytes / 4;
  const unsigned blocks = static_cast<unsigned>(std::min<size_t>(16, (n + 255) / 256));
  if (v16) {
    HostRowsToDeviceKernel<uint4><<<blocks, 256, 0, stream>>>(static_cast<const uint4*>(src), static_cast<uint4*>(dst), n);
  } else {
    HostRowsToDeviceKernel<uint32_t><<<blocks, 256, 0, stream>>>(static_cast<const uint32_t*>(src), static_cast<uint32_t*>(dst), n);
  }
  return cudaGetLastError();
}

}  // namespace

extern "C" {

const char* qfg_last_error(void) { return g_last_error.c_str(); }
const char* qfg_version(void) { return "qfg-b200 0.1 sm_100a"; }

int qfg_skinny_gemm_create(const int64_t* seg_outs, int n_seg, const int64_t* widths, int n_widths,
                           const float* w_scale, size_t n_w_scale, int trigger, qfg_skinny_gemm** out) {
  if (out == nullptr) return Fail(QFG_INVALID_ARGUMENT, "SkinnyGemm: null handle pointer");
  *out = nullptr;
  qfg_skinny_gemm* op = new qfg_skinny_gemm();
  try {
    InitGemmOp(op, seg_outs, n_seg, widths, n_widths, w_scale, n_w_scale, trigger, "SkinnyGemm");
  } catch (const std::exception& e) {
    delete op;
    return Fail(QFG_INVALID_ARGUMENT, e.what());
  }
  *out = op;
  return QFG_OK;
}

int qfg_skinny_gemm_compute(const qfg_skinny_gemm* op, const void* x, int64_t m, int64_t k,
                            const qfg_tensor2d* weights, int n_weights, void* const* outs, int n_outs,
                            void* stream) {
  if (op == nullptr || weights == nullptr || outs == nullptr) return Fail(QFG_FAIL, "SkinnyGemm: null argument");
  try {
    Prepared pr = Prepare(*op, x, m, k, weights, n_weights, outs, n_outs, true);
    Run(*op, pr, m, static_cast<cudaStream_t>(stream), "SkinnyGemm");
    return QFG_OK;
  } catch (const InvalidArgument& e) {
    return Fail(QFG_INVALID_ARGUMENT, e.what());
  } catch (const std::exception& e) {
    return Fail(QFG_FAIL, e.what());
  }
}

int qfg_skinny_gemm_set_option(qfg_skinny_gemm* op, const char* key, const char* value) {
  return SetGemmOption(op, key, value);
}

int qfg_skinny_gemm_describe(const qfg_skinny_gemm* op, int64_t k, const qfg_tensor2d* weights, int n_weights,
                             char* buf, size_t buf_len) {
  if (op == nullptr || weights == nullptr || buf == nullptr || buf_len == 0)
    return Fail(QFG_INVALID_ARGUMENT, "describe: null argument");
  try {
    Prepared pr = Prepare(*op, nullptr, 1, k, weights, n_weights, nullptr, 0, false);
    const qfg::Plan plan = PlanFor(*op, pr.plan_in, qfg::kMaxRows);
    const std::string d = qfg::DescribePlan(plan, pr.plan_in) + ",trigger=" + std::to_string(op->trigger);
    std::snprintf(buf, buf_len, "%s", d.c_str());
    return QFG_OK;
  } catch (const std::exception& e) {
    return Fail(QFG_INVALID_ARGUMENT, e.what());
  }
}

int qfg_plan_describe(int dtype, int64_t k, const int64_t* n, int nseg, int row_align, int sm_count,
                      const char* spec, char* buf, size_t buf_len) {
  if (n == nullptr || buf == nullptr || buf_len == 0 || nseg < 1 || nseg > qfg::kMaxSeg || k < 1 || k > INT_MAX ||
      (row_align != 16 && row_align != 8 && row_align != 4) || sm_count < 1) {
    return Fail(QFG_INVALID_ARGUMENT, "plan_describe: bad argument");
  }
  qfg::PlanInput in;
  in.K = static_cast<int>(k);
  in.nseg = nseg;
  in.mode = dtype == QFG_BFLOAT16 ? qfg::kBf16 : dtype == QFG_FLOAT8E4M3FN ? qfg::kFp8 : qfg::kNvfp4;
  if (dtype != QFG_BFLOAT16 && dtype != QFG_FLOAT8E4M3FN && dtype != QFG_UINT8)
    return Fail(QFG_INVALID_ARGUMENT, "plan_describe: unsupported weight element type");
  for (int s = 0; s < nseg; ++s) {
    if (n[s] < 1 || n[s] > INT_MAX) return Fail(QFG_INVALID_ARGUMENT, "plan_describe: bad width");
    in.n[s] = static_cast<int>(n[s]);
  }
  in.row_align = row_align;
  in.sm_count = sm_count;
  // a spec that starts with "lmhead" (optionally followed by ",key=value...") describes the fused LM head,
  // whose workspace allows the shared tail
  std::string overrides = spec != nullptr ? spec : "";
  if (overrides.rfind("lmhead", 0) == 0) {
    in.allow_tail = true;
    overrides = overrides.size() > 7 ? overrides.substr(7) : "";
  }
  qfg::Plan plan = qfg::ChoosePlan(in);
  if (!overrides.empty() && !qfg::ApplyPlanOverrides(overrides, in, &plan))
    return Fail(QFG_INVALID_ARGUMENT, "plan_describe: bad plan override");
  qfg::FinishPlan(in, overrides, &plan);
  std::string d = qfg::DescribePlan(plan, in);
  d += ",seg_tiles=";
  for (int s = 0; s < nseg; ++s) d += (s ? "/" : "") + std::to_string(plan.tiles[s]);
  std::snprintf(buf, buf_len, "%s", d.c_str());
  return QFG_OK;
}

void qfg_skinny_gemm_destroy(qfg_skinny_gemm* op) {
  if (op == nullptr) return;
  cudaFree(op->d_w_scale);
  delete op;
}

int qfg_argmax_rows(int dtype, const void* x, int64_t rows, int64_t vocab, int64_t* idx, float* val, void* stream) {
  if (dtype != QFG_BFLOAT16 && dtype != QFG_FLOAT16 && dtype != QFG_FLOAT)
    return Fail(QFG_INVALID_ARGUMENT, "ArgmaxRows: logits must be BF16/FP16/FP32");
  if (vocab < 1 || rows < 0) return Fail(QFG_INVALID_ARGUMENT, "ArgmaxRows: bad shape");
  if (rows == 0) return QFG_OK;
  if (x == nullptr || idx == nullptr) return Fail(QFG_INVALID_ARGUMENT, "ArgmaxRows: null argument");
  if (vocab >= INT_MAX) return Fail(QFG_FAIL, std::string("ArgmaxRows: ") + cudaGetErrorString(cudaErrorInvalidValue));
  const size_t elem = dtype == QFG_FLOAT ? 4 : 2;
  if (reinterpret_cast<uintptr_t>(x) % elem != 0) return Fail(QFG_INVALID_ARGUMENT, "ArgmaxRows: misaligned logits");
  // the grid's y extent caps one launch at 65535 rows
  for (int64_t r0 = 0; r0 < rows; r0 += 65535) {
    const int64_t n = std::min<int64_t>(65535, rows - r0);
    cudaError_t err = qfg::LaunchArgmaxRows(dtype, static_cast<const uint8_t*>(x) + static_cast<size_t>(r0) * vocab * elem,
                                            n, vocab, idx + r0, val != nullptr ? val + r0 : nullptr,
                                            static_cast<cudaStream_t>(stream));
    if (err == cudaSuccess) err = cudaGetLastError();
    if (err != cudaSuccess) return Fail(QFG_FAIL, std::string("ArgmaxRows: ") + cudaGetErrorString(err));
  }
  return QFG_OK;
}

int qfg_shared_expert_down_create(const float* w_scale, size_t n_w_scale, int trigger, qfg_shared_expert_down** out) {
  if (out == nullptr) return Fail(QFG_INVALID_ARGUMENT, "SharedExpertDown: null handle pointer");
  *out = nullptr;
  qfg_shared_expert_down* op = new qfg_shared_expert_down();
  const int64_t one = 1;
  try {
    InitGemmOp(&op->gemm, &one, 1, &one, 1, w_scale, n_w_scale, trigger, "SharedExpertDown");
  } catch (const std::exception& e) {
    delete op;
    return Fail(QFG_INVALID_ARGUMENT, e.what());
  }
  *out = op;
  return QFG_OK;
}

int qfg_shared_expert_down_compute(const qfg_shared_expert_down* op, const void* g, const void* u, int64_t m, int64_t k,
                                   const qfg_tensor2d* weight, const void* gx, int64_t gk, const void* gw,
                                   const void* routed, int64_t n, void* out, void* stream) {
  if (op == nullptr || weight == nullptr) return Fail(QFG_INVALID_ARGUMENT, "SharedExpertDown: null argument");
  try {
    if (m < 1 || n < 1 || n > INT_MAX || n % 8 != 0 || gk < 0 || gk > INT_MAX || gk % 2 != 0)
      throw InvalidArgument("SharedExpertDown: shape mismatch");
    if (g == nullptr || u == nullptr || gx == nullptr || gw == nullptr || out == nullptr ||
        reinterpret_cast<uintptr_t>(u) % 4 != 0 || reinterpret_cast<uintptr_t>(gx) % 2 != 0 ||
        reinterpret_cast<uintptr_t>(gw) % 2 != 0 || reinterpret_cast<uintptr_t>(routed) % 2 != 0) {
      throw InvalidArgument("SharedExpertDown: null or misaligned input");
    }
    void* outs[1] = {out};
    Prepared pr = Prepare(op->gemm, g, m, k, weight, 1, outs, 1, true, n);
    pr.params.fuse = 1;
    pr.params.x2 = static_cast<const uint16_t*>(u);
    pr.params.gx = static_cast<const uint16_t*>(gx);
    pr.params.gw = static_cast<const uint16_t*>(gw);
    pr.params.routed = static_cast<const uint16_t*>(routed);
    pr.params.gk = static_cast<int>(gk);
    Run(op->gemm, pr, m, static_cast<cudaStream_t>(stream), "SharedExpertDown");
    return QFG_OK;
  } catch (const InvalidArgument& e) {
    return Fail(QFG_INVALID_ARGUMENT, e.what());
  } catch (const std::exception& e) {
    return Fail(QFG_FAIL, e.what());
  }
}

int qfg_shared_expert_down_set_option(qfg_shared_expert_down* op, const char* key, const char* value) {
  if (op == nullptr) return Fail(QFG_INVALID_ARGUMENT, "SharedExpertDown: null node");
  return SetGemmOption(&op->gemm, key, value);
}

void qfg_shared_expert_down_destroy(qfg_shared_expert_down* op) {
  if (op == nullptr) return;
  cudaFree(op->gemm.d_w_scale);
  delete op;
}

int qfg_untile_hc_create(int kind, const float* w_scale, size_t n_w_scale, qfg_untile_hc** out) {
  if (out == nullptr) return Fail(QFG_INVALID_ARGUMENT, "UntileHcBf16: null handle pointer");
  *out = nullptr;
  if (kind != 0 && kind != 1) return Fail(QFG_INVALID_ARGUMENT, "UntileHcBf16: kind must be 0 or 1");
  qfg_untile_hc* op = new qfg_untile_hc();
  try {
    op->kind = kind;
    op->d_w_scale = UploadScales(w_scale, n_w_scale, "UntileHcBf16");
    op->w_scale_len = op->d_w_scale != nullptr ? n_w_scale : 0;
  } catch (const std::exception& e) {
    delete op;
    return Fail(QFG_INVALID_ARGUMENT, e.what());
  }
  *out = op;
  return QFG_OK;
}

int qfg_untile_hc_compute(const qfg_untile_hc* op, const qfg_tensor2d* w, void* out, void* stream) {
  if (op == nullptr || w == nullptr) return Fail(QFG_FAIL, "UntileHcBf16: null argument");
  if (w->rows != 160 || w->cols != 20480) return Fail(QFG_FAIL, "UntileHcBf16: expected [160, 20480]");
  if (w->dtype != QFG_BFLOAT16 && w->dtype != QFG_FLOAT8E4M3FN) return Fail(QFG_FAIL, "UntileHcBf16: unsupported input element type");
  if (w->data == nullptr || out == nullptr || reinterpret_cast<uintptr_t>(w->data) % 16 != 0 ||
      reinterpret_cast<uintptr_t>(out) % 16 != 0) {
    return Fail(QFG_FAIL, "UntileHcBf16: null or misaligned tensor");
  }
  const bool fp8 = w->dtype == QFG_FLOAT8E4M3FN;
  const size_t need = op->kind == 0 ? 320 : 10240;
  if (fp8 && op->d_w_scale != nullptr && op->w_scale_len < need) return Fail(QFG_FAIL, "UntileHcBf16: w_scale shorter than the output width");
  const cudaError_t err = qfg::LaunchUntileHc(fp8, w->data, out, op->d_w_scale, op->kind, static_cast<cudaStream_t>(stream));
  if (err != cudaSuccess) return Fail(QFG_FAIL, (std::string("UntileHcBf16: ") + cudaGetErrorString(err)).c_str());
  return QFG_OK;
}

void qfg_untile_hc_destroy(qfg_untile_hc* op) {
  if (op == nullptr) return;
  cudaFree(op->d_w_scale);
  delete op;
}

int qfg_dequant_create(int64_t n_cols, int64_t col_offset, const int64_t* widths, int n_widths,
                       const float* w_scale, size_t n_w_scale, qfg_dequant** out) {
  if (out == nullptr) return Fail(QFG_INVALID_ARGUMENT, "DequantWeightBf16: null handle pointer");
  *out = nullptr;
  qfg_dequant* op = new qfg_dequant();
  try {
    op->n_cols = n_cols;
    op->col_offset = col_offset;
    for (int i = 0; i < n_widths; ++i) {
      if (widths[i] > INT_MAX) throw InvalidArgument("DequantWeightBf16: invalid widths or col_offset");
      op->widths.push_back(static_cast<int>(widths[i]));
    }
    if (op->widths.empty()) op->widths.push_back(static_cast<int>(n_cols));
    long long sum_w = 0;
    for (int v : op->widths) {
      if (v <= 0 || v % 8 != 0)
        throw InvalidArgument("DequantWeightBf16: each width must be a positive multiple of 8");
      sum_w += v;
    }
    if (sum_w != n_cols || op->widths.size() > static_cast<size_t>(qfg::kMaxOut) || col_offset < 0 || col_offset % 8 != 0)
      throw InvalidArgument("DequantWeightBf16: invalid widths or col_offset");
    op->d_w_scale = UploadScales(w_scale, n_w_scale, "DequantWeightBf16");
    op->w_scale_len = op->d_w_scale != nullptr ? n_w_scale : 0;
  } catch (const std::exception& e) {
    delete op;
    return Fail(QFG_INVALID_ARGUMENT, e.what());
  }
  *out = op;
  return QFG_OK;
}

int qfg_dequant_compute(const qfg_dequant* op, const qfg_tensor2d* w, void* const* outs, int n_outs, void* stream) {
  if (op == nullptr || w == nullptr || outs == nullptr) return Fail(QFG_FAIL, "DequantWeightBf16: null argument");
  try {
    const int64_t N = op->n_cols;
    if (N <= 0 || N % 8 != 0 || w->rows < 0 || w->rows > INT_MAX || N > INT_MAX)
      throw InvalidArgument("DequantWeightBf16: invalid shape");
    if (n_outs != static_cast<int>(op->widths.size())) throw InvalidArgument("DequantWeightBf16: output count");
    if (op->d_w_scale != nullptr && op->w_scale_len < static_cast<size_t>(N))
      throw InvalidArgument("DequantWeightBf16: w_scale shorter than n_cols");
    qfg::DequantParams p;
    const int64_t co = op->col_offset;
    if (w->dtype == QFG_BFLOAT16 && w->cols >= co + N) {
      p.mode = qfg::kBf16;
      p.row_stride = static_cast<int>(w->cols);
      p.aligned = reinterpret_cast<uintptr_t>(w->data) % 16 == 0 && w->cols % 8 == 0;
    } else if (w->dtype == QFG_FLOAT8E4M3FN && w->cols >= co + N) {
      p.mode = qfg::kFp8;
      p.row_stride = static_cast<int>(w->cols);
      p.aligned = reinterpret_cast<uintptr_t>(w->data) % 8 == 0 && w->cols % 8 == 0;
    } else if (w->dtype == QFG_UINT8 && N % 16 == 0 && co % 16 == 0 && w->cols * 16 >= (co + N) * 9 &&
               (w->cols * 16) % 9 == 0) {
      p.mode = qfg::kNvfp4;
      p.row_stride = static_cast<int>((w->cols * 16) / 9);
      p.aligned = reinterpret_cast<uintptr_t>(w->data) % 4 == 0 && w->cols % 4 == 0;
    } else {
      throw InvalidArgument("DequantWeightBf16: unsupported input type/shape");
    }
    if (w->data == nullptr && w->rows > 0) throw InvalidArgument("DequantWeightBf16: null weight");
    p.w = static_cast<const uint8_t*>(w->data);
    p.w_scale = op->d_w_scale;
    p.K = static_cast<int>(w->rows);
    p.N = static_cast<int>(N);
    p.col_offset = static_cast<int>(co);
    p.num_outs = static_cast<int>(op->widths.size());
    int col_off = 0;
    for (int i = 0; i < p.num_outs; ++i) {
      if (outs[i] == nullptr || reinterpret_cast<uintptr_t>(outs[i]) % 16 != 0)
        throw InvalidArgument("DequantWeightBf16: outputs must be 16-byte aligned");
      p.out[i] = static_cast<uint16_t*>(outs[i]);
      p.col_begin[i] = col_off;
      p.width[i] = op->widths[i];
      col_off += op->widths[i];
    }
    cudaError_t err = qfg::LaunchDequant(p, static_cast<cudaStream_t>(stream));
    if (err != cudaSuccess) throw std::runtime_error(std::string("DequantWeightBf16: ") + cudaGetErrorString(err));
    return QFG_OK;
  } catch (const InvalidArgument& e) {
    return Fail(QFG_INVALID_ARGUMENT, e.what());
  } catch (const std::exception& e) {
    return Fail(QFG_FAIL, e.what());
  }
}

void qfg_dequant_destroy(qfg_dequant* op) {
  if (op == nullptr) return;
  cudaFree(op->d_w_scale);
  delete op;
}

size_t qfg_lmhead_exchange_bytes(void) { return (sizeof(qfg::LmExchange) + 255) & ~static_cast<size_t>(255); }

int qfg_lmhead_compute_sharded(const qfg_lmhead* op, const void* x, int64_t m, int64_t k, const qfg_tensor2d* weight,
                               int64_t n, int64_t col_offset, void* workspace, const qfg_lmhead_exchange* exchange,
                               int64_t* idx, float* val, void* logits, void* stream) {
  if (exchange == nullptr) return Fail(QFG_INVALID_ARGUMENT, "LmHead: null exchange");
  return qfg::LmheadComputeWithWorkspace(op, x, m, k, weight, n, col_offset, workspace, qfg_lmhead_workspace_bytes(), idx, val,
                                         nullptr, logits, stream, exchange);
}

int qfg_lmhead_exchange_status(const void* own_buffer, int* status) {
  if (own_buffer == nullptr || status == nullptr) return Fail(QFG_INVALID_ARGUMENT, "LmHead: null argument");
  unsigned int s = 0;
  const cudaError_t err = cudaMemcpy(&s, &static_cast<const qfg::LmExchange*>(own_buffer)->status, sizeof(s), cudaMemcpyDeviceToHost);
  if (err != cudaSuccess) return Fail(QFG_FAIL, (std::string("LmHead: ") + cudaGetErrorString(err)).c_str());
  *status = static_cast<int>(s);
  return QFG_OK;
}

int qfg_lmhead_exchange_times(const void* own_buffer, uint64_t out[3]) {
  if (own_buffer == nullptr || out == nullptr) return Fail(QFG_INVALID_ARGUMENT, "LmHead: null argument");
  const qfg::LmExchange* e = static_cast<const qfg::LmExchange*>(own_buffer);
  unsigned long long t[3] = {0, 0, 0};
  const cudaError_t err = cudaMemcpy(t, &e->t_ready, sizeof(t), cudaMemcpyDeviceToHost);
  if (err != cudaSuccess) return Fail(QFG_FAIL, (std::string("LmHead: ") + cudaGetErrorString(err)).c_str());
  for (int i = 0; i < 3; ++i) out[i] = t[i];
  return QFG_OK;
}

struct qfg_lmhead_host {
  cudaStream_t stream = nullptr;
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
  qfg_lmhead op;  // the caller's node with pdl_wait set (shares, and does not own, its w_scale)
  unsigned int* status_host = nullptr;  // pinned, device-addressable: 1 if the step's wait for a peer ran out
  // where the kernel stores the step's results (pinned host memory): polled by qfg_lmhead_host_run
  int64_t rows = 0;
  volatile int64_t* idx_host = nullptr;
  volatile uint32_t* val_host = nullptr;
};

// Values the kernel never stores: an index of -1, and a float whose low 16 bits are set (the maximum is a BF16
// logit widened to FP32, or the canonical NaN, so its low half is zero); the status word is 0 or 1.
constexpr int64_t kIdxSentinel = -1;
constexpr uint32_t kValSentinel = 0xFFC0DEADu;
constexpr unsigned int kStatusSentinel = 0xFFFFFFFFu;


int qfg_lmhead_host_create(const qfg_lmhead* op, int64_t m, int64_t k, const qfg_tensor2d* weight, int64_t n,
                           int64_t col_offset, void* workspace, const qfg_lmhead_exchange* exchange, const void* x_host,
                           void* x_dev, int64_t* idx_host, float* val_host, qfg_lmhead_host** out) {
  if (out == nullptr) return Fail(QFG_INVALID_ARGUMENT, "LmHead: null handle pointer");
  *out = nullptr;
  if (op == nullptr || weight == nullptr || x_host == nullptr || x_dev == nullptr || idx_host == nullptr || m < 1 || k < 1)
    return Fail(QFG_INVALID_ARGUMENT, "LmHead: null or bad host-step argument");
  if (k % 2 != 0 || reinterpret_cast<uintptr_t>(x_host) % 4 != 0 || reinterpret_cast<uintptr_t>(x_dev) % 4 != 0)
    return Fail(QFG_INVALID_ARGUMENT, "LmHead: x must be 4-byte aligned with an even K");
  qfg_lmhead_host* h = new qfg_lmhead_host{nullptr, nullptr, nullptr, *op, nullptr};
  h->op.gemm.pdl_wait = 1;
  h->rows = m;
  h->idx_host = idx_host;
  h->val_host = reinterpret_cast<volatile uint32_t*>(val_host);
  if (exchange != nullptr && exchange->world > 1) {
    // the sharded step reports a wait that ran out through one word of pinned memory, read after the synchronise
    if (cudaHostAlloc(reinterpret_cast<void**>(&h->status_host), sizeof(unsigned int), cudaHostAllocMapped) != cudaSuccess) {
      cudaGetLastError();
      delete h;
      return Fail(QFG_FAIL, "LmHead: cannot allocate the pinned status word");
    }
    *h->status_host = 0;
  }
  const size_t x_bytes = static_cast<size_t>(m) * static_cast<size_t>(k) * 2;
  // one step: input copy, then the fused kernel as its programmatic dependent, results addressed to host memory
  auto enqueue = [&]() -> int {
    const cudaError_t err = LaunchHostRowsToDevice(x_host, x_dev, x_bytes, h->stream);
    if (err != cudaSuccess) return Fail(QFG_FAIL, std::string("LmHead: ") + cudaGetErrorString(err));
    return qfg::LmheadComputeWithWorkspace(&h->op, x_dev, m, k, weight, n, col_offset, workspace, qfg_lmhead_workspace_bytes(),
                                           idx_host, val_host, nullptr, nullptr, h->stream, exchange, h->status_host);
  };
  int rc = QFG_OK;
  cudaError_t err = cudaStreamCreateWithFlags(&h->stream, cudaStreamNonBlocking);
  if (err == cudaSuccess) {
    // eagerly once: plans and kernel attributes are settled outside the capture
    rc = enqueue();
    if (rc == QFG_OK) err = cudaStreamSynchronize(h->stream);
  }
  if (rc == QFG_OK && err == cudaSuccess) {
    err = cudaStreamBeginCapture(h->stream, cudaStreamCaptureModeThreadLocal);
    if (err == cudaSuccess) {
      rc = enqueue();
      const cudaError_t end = cudaStreamEndCapture(h->stream, &h->graph);  // always ends the capture
      if (rc == QFG_OK) err = end;
    }
  }
  if (rc == QFG_OK && err == cudaSuccess) err = cudaGraphInstantiate(&h->exec, h->graph, 0);
  if (rc != QFG_OK || err != cudaSuccess) {
    if (rc == QFG_OK) rc = Fail(QFG_FAIL, std::string("LmHead: ") + cudaGetErrorString(err));
    qfg_lmhead_host_destroy(h);
    return rc;
  }
  *out = h;
  return QFG_OK;
}

int qfg_lmhead_host_run(qfg_lmhead_host* h) {
  if (h == nullptr || h->exec == nullptr) return Fail(QFG_INVALID_ARGUMENT, "LmHead: null host-step handle");
  // The kernel's last CTA stores the results straight into pinned host memory.  The host marks every result
  // word with a value the kernel never stores, launches, and reads the words until all have changed: the call
  // returns when the results are there, not when the stream has drained and the synchronising thread has been
  // woken (5-8 us later).  The wait is bounded; past the bound, and on any error, the stream is synchronised.
  for (int64_t i = 0; i < h->rows; ++i) {
    h->idx_host[i] = kIdxSentinel;
    if (h->val_host != nullptr) h->val_host[i] = kValSentinel;
  }
  volatile unsigned int* status = h->status_host;
  if (status != nullptr) *status = kStatusSentinel;
  cudaError_t err = cudaGraphLaunch(h->exec, h->stream);
  if (err != cudaSuccess) return Fail(QFG_FAIL, std::string("LmHead: ") + cudaGetErrorString(err));
  bool there = false;
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(20);
  for (unsigned spin = 0; !there; ++spin) {
    there = status == nullptr || *status != kStatusSentinel;
    for (int64_t i = 0; there && i < h->rows; ++i) {
      there = h->idx_host[i] != kIdxSentinel && (h->val_host == nullptr || h->val_host[i] != kValSentinel);
    }
    if (!there && (spin & 1023u) == 1023u && std::chrono::steady_clock::now() > deadline) break;
  }
  if (!there) {
    err = cudaStreamSynchronize(h->stream);
    if (err != cudaSuccess) return Fail(QFG_FAIL, std::string("LmHead: ") + cudaGetErrorString(err));
  }
  if (status != nullptr && *status != 0)
    return Fail(QFG_FAIL, "LmHead: the wait for a peer's keys ran out; the result lacks that peer");
  return QFG_OK;
}

void qfg_lmhead_host_destroy(qfg_lmhead_host* h) {
  if (h == nullptr) return;
  if (h->stream != nullptr) cudaStreamSynchronize(h->stream);  // a step may have returned before the stream drained
  if (h->status_host != nullptr) cudaFreeHost(h->status_host);
  if (h->exec != nullptr) cudaGraphExecDestroy(h->exec);
  if (h->graph != nullptr) cudaGraphDestroy(h->graph);
  if (h->stream != nullptr) cudaStreamDestroy(h->stream);
  delete h;
}

int qfg_peer_alloc(size_t bytes, void** ptr, unsigned char handle[64]) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  if (ptr == nullptr || handle == nullptr || bytes == 0) return Fail(QFG_INVALID_ARGUMENT, "peer_alloc: bad argument");
  void* p = nullptr;
  cudaError_t err = cudaMalloc(&p, bytes);
  if (err == cudaSuccess) err = cudaMemset(p, 0, bytes);
  cudaIpcMemHandle_t h;
  if (err == cudaSuccess) err = cudaIpcGetMemHandle(&h, p);
  if (err == cudaSuccess) err = cudaDeviceSynchronize();
  if (err != cudaSuccess) {
    if (p != nullptr) cudaFree(p);
    return Fail(QFG_FAIL, (std::string("peer_alloc: ") + cudaGetErrorString(err)).c_str());
  }
  std::memcpy(handle, &h, 64);
  *ptr = p;
  return QFG_OK;
}

int qfg_peer_open(const unsigned char handle[64], void** ptr) {
  if (ptr == nullptr || handle == nullptr) return Fail(QFG_INVALID_ARGUMENT, "peer_open: bad argument");
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle, 64);
  const cudaError_t err = cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
  if (err != cudaSuccess) return Fail(QFG_FAIL, (std::string("peer_open: ") + cudaGetErrorString(err)).c_str());
  return QFG_OK;
}

int qfg_peer_close(void* ptr) {
  const cudaError_t err = cudaIpcCloseMemHandle(ptr);
  return err == cudaSuccess ? QFG_OK : Fail(QFG_FAIL, (std::string("peer_close: ") + cudaGetErrorString(err)).c_str());
}

int qfg_peer_free(void* ptr) {
  const cudaError_t err = cudaFree(ptr);
  return err == cudaSuccess ? QFG_OK : Fail(QFG_FAIL, (std::string("peer_free: ") + cudaGetErrorString(err)).c_str());
}

size_t qfg_lmhead_workspace_bytes(void) { return qfg::kLmHeaderBytes + qfg::kLmTailBytes; }

int qfg_lmhead_create(const float* w_scale, size_t n_w_scale, int trigger, qfg_lmhead** out) {
  if (out == nullptr) return Fail(QFG_INVALID_ARGUMENT, "LmHead: null handle pointer");
  *out = nullptr;
  qfg_lmhead* op = new qfg_lmhead();
  try {
    // geometry is per call (the vocabulary shard width is an argument), so the attribute lists
    // hold a placeholder of one weight with one output
    const int64_t one = 1;
    InitGemmOp(&op->gemm, &one, 1, &one, 1, w_scale, n_w_scale, trigger, "LmHead");
  } catch (const std::exception& e) {
    delete op;
    return Fail(QFG_INVALID_ARGUMENT, e.what());
  }
  *out = op;
  return QFG_OK;
}

int qfg_lmhead_compute(const qfg_lmhead* op, const void* x, int64_t m, int64_t k, const qfg_tensor2d* weight,
                       int64_t n, int64_t col_offset, void* workspace, int64_t* idx, float* val, uint64_t* key,
                       void* logits, void* stream) {
  return qfg::LmheadComputeWithWorkspace(op, x, m, k, weight, n, col_offset, workspace, qfg_lmhead_workspace_bytes(), idx, val,
                                         key, logits, stream);
}

int qfg_lmhead_set_option(qfg_lmhead* op, const char* key, const char* value) {
  return SetGemmOption(op != nullptr ? &op->gemm : nullptr, key, value);
}

void qfg_lmhead_destroy(qfg_lmhead* op) {
  if (op == nullptr) return;
  cudaFree(op->gemm.d_w_scale);
  delete op;
}

int qfg_lmhead_combine(const uint64_t* keys, int ranks, int64_t m, int64_t* idx, float* val, void* stream) {
  if (keys == nullptr || ranks < 1 || m < 1) return Fail(QFG_INVALID_ARGUMENT, "LmHead: bad combine arguments");
  cudaError_t err = qfg::LaunchLmheadCombine(keys, ranks, m, idx, val, static_cast<cudaStream_t>(stream));
  if (err != cudaSuccess) return Fail(QFG_FAIL, std::string("LmHead: ") + cudaGetErrorString(err));
  return QFG_OK;
}

}  // extern "C"
