// ONNX Runtime custom-op shim: builds the drop-in libqwen_fused_gemm_r5.so on top of the C ABI of
// include/qfg.h.  Same entry point (RegisterCustomOps), op domain (qwen.fused_gemm), op names,
// attributes, input/output signatures, execution provider and status behaviour as the reference
// library (src/fused_gemm/fused_gemm.cu:781-840, :956-977, :1093-1117 of the reference project).
// This is the only translation unit that includes ONNX Runtime headers; it compiles only where
// ORT_INCLUDE_DIR points at genuine headers (make ORT_INCLUDE_DIR=... in qwen38_flash_ops_b200/csrc).
//
// Registered ops: SkinnyGemm, SharedExpertDown, ArgmaxRows, DequantWeightBf16, UntileHcBf16 - the five
// names of the reference library.  SharedExpertDown runs without the reference's deferred-merge hook
// (QMoESharedExpertBridge, an ORT-internal peer): `routed` is always added by this op.
#ifndef ORT_API_MANUAL_INIT
#define ORT_API_MANUAL_INIT
#endif
#include "onnxruntime_cxx_api.h"

#include <cstdint>
#include <mutex>
#include <stdexcept>
#include <string>
#include <vector>

#include "qfg.h"

namespace {

void* ComputeStream(const OrtApi& api, OrtKernelContext* context) {
  void* raw = nullptr;
  Ort::ThrowOnError(api.KernelContext_GetGPUComputeStream(context, &raw));
  return raw;
}

int ToQfgType(ONNXTensorElementDataType t) {
  switch (t) {
    case ONNX_TENSOR_ELEMENT_DATA_TYPE_BFLOAT16: return QFG_BFLOAT16;
    case ONNX_TENSOR_ELEMENT_DATA_TYPE_FLOAT8E4M3FN: return QFG_FLOAT8E4M3FN;
    case ONNX_TENSOR_ELEMENT_DATA_TYPE_UINT8: return QFG_UINT8;
    case ONNX_TENSOR_ELEMENT_DATA_TYPE_FLOAT16: return QFG_FLOAT16;
    case ONNX_TENSOR_ELEMENT_DATA_TYPE_FLOAT: return QFG_FLOAT;
    default: return -1;
  }
}

qfg_tensor2d Tensor2d(const Ort::ConstValue& v, const char* what) {
  auto info = v.GetTensorTypeAndShapeInfo();
  auto shape = info.GetShape();
  if (shape.size() != 2) throw std::invalid_argument(std::string(what) + ": weight shape");
  qfg_tensor2d t;
  t.data = v.GetTensorRawData();
  t.dtype = ToQfgType(info.GetElementType());
  t.rows = shape[0];
  t.cols = shape[1];
  return t;
}

template <typename T>
std::vector<T> OptionalAttributes(const Ort::ConstKernelInfo& k, const char* name) {
  try {
    return k.GetAttributes<T>(name);
  } catch (const std::exception&) {
    return {};
  }
}

int64_t OptionalAttribute(const Ort::ConstKernelInfo& k, const char* name, int64_t dflt) {
  try {
    return k.GetAttribute<int64_t>(name);
  } catch (const std::exception&) {
    return dflt;
  }
}

// qfg status of a compute call -> OrtStatus.  Every compute-time error of the reference's ComputeV2 is ORT_FAIL
// (fused_gemm.cu:589-591, :723-725, :775-777, :950-952, :1065-1067), whatever went wrong; the library's finer
// code (QFG_INVALID_ARGUMENT / QFG_FAIL) stays in the message's source, qfg_last_error().  Errors of kernel
// creation are ORT_INVALID_ARGUMENT, as in the reference's CreateKernelV2.
OrtStatus* ToStatus(const OrtApi& api, int code) {
  if (code == QFG_OK) return nullptr;
  return api.CreateStatus(ORT_FAIL, qfg_last_error());
}

struct SkinnyGemmState {
  const OrtApi& api;
  qfg_skinny_gemm* op = nullptr;
  size_t n_seg = 0;
  std::vector<int64_t> widths;

  SkinnyGemmState(const OrtApi& a, const OrtKernelInfo* info) : api(a) {
    Ort::ConstKernelInfo k(info);
    const std::vector<int64_t> seg_outs = k.GetAttributes<int64_t>("seg_outs");
    widths = k.GetAttributes<int64_t>("widths");
    const std::vector<float> w_scale = OptionalAttributes<float>(k, "w_scale");
    const int trigger = static_cast<int>(OptionalAttribute(k, "trigger", 0));
    n_seg = seg_outs.size();
    if (qfg_skinny_gemm_create(seg_outs.data(), static_cast<int>(seg_outs.size()), widths.data(),
                               static_cast<int>(widths.size()), w_scale.empty() ? nullptr : w_scale.data(),
                               w_scale.size(), trigger, &op) != QFG_OK) {
      throw std::invalid_argument(qfg_last_error());
    }
  }
  ~SkinnyGemmState() { qfg_skinny_gemm_destroy(op); }

  OrtStatus* ComputeV2(OrtKernelContext* raw) noexcept {
    try {
      Ort::KernelContext c(raw);
      if (c.GetInputCount() != n_seg + 1) throw std::invalid_argument("SkinnyGemm: input count");
      auto x = c.GetInput(0);
      auto xshape = x.GetTensorTypeAndShapeInfo().GetShape();
      if (xshape.empty()) throw std::invalid_argument("SkinnyGemm: x needs a last dimension K");
      const int64_t K = xshape.back();
      int64_t m = 1;
      for (size_t i = 0; i + 1 < xshape.size(); ++i) m *= xshape[i];
      if (m < 1) throw std::invalid_argument("SkinnyGemm: M must be >= 1");
      std::vector<qfg_tensor2d> weights;
      for (size_t s = 0; s < n_seg; ++s) weights.push_back(Tensor2d(c.GetInput(1 + s), "SkinnyGemm"));
      std::vector<void*> outs;
      for (size_t o = 0; o < widths.size(); ++o) {
        std::vector<int64_t> shape(xshape.begin(), xshape.end() - 1);
        shape.push_back(widths[o]);
        auto out = c.GetOutput(o, shape);
        outs.push_back(out.GetTensorMutableRawData());
      }
      return ToStatus(api, qfg_skinny_gemm_compute(op, x.GetTensorRawData(), m, K, weights.data(),
                                                   static_cast<int>(weights.size()), outs.data(),
                                                   static_cast<int>(outs.size()), ComputeStream(api, raw)));
    } catch (const std::exception& e) {
      return api.CreateStatus(ORT_FAIL, e.what());
    }
  }
};

struct ArgmaxRowsState {
  const OrtApi& api;
  explicit ArgmaxRowsState(const OrtApi& a) : api(a) {}

  OrtStatus* ComputeV2(OrtKernelContext* raw) noexcept {
    try {
      Ort::KernelContext c(raw);
      if (c.GetInputCount() != 1 || c.GetOutputCount() < 1 || c.GetOutputCount() > 2) {
        throw std::invalid_argument("ArgmaxRows: 1 input, 1 or 2 outputs");
      }
      auto x = c.GetInput(0);
      auto info = x.GetTensorTypeAndShapeInfo();
      auto shape = info.GetShape();
      if (shape.empty() || shape.back() < 1) throw std::invalid_argument("ArgmaxRows: bad shape");
      const int dtype = ToQfgType(info.GetElementType());
      if (dtype != QFG_BFLOAT16 && dtype != QFG_FLOAT16 && dtype != QFG_FLOAT)
        throw std::invalid_argument("ArgmaxRows: logits must be BF16/FP16/FP32");
      const int64_t V = shape.back();
      std::vector<int64_t> oshape(shape.begin(), shape.end() - 1);
      int64_t rows = 1;
      for (auto d : oshape) rows *= d;
      auto idx = c.GetOutput(0, oshape);
      float* val = nullptr;
      if (c.GetOutputCount() == 2) val = c.GetOutput(1, oshape).GetTensorMutableData<float>();
      if (rows == 0) return nullptr;
      return ToStatus(api, qfg_argmax_rows(dtype, x.GetTensorRawData(), rows, V, idx.GetTensorMutableData<int64_t>(),
                                           val, ComputeStream(api, raw)));
    } catch (const std::exception& e) {
      return api.CreateStatus(ORT_FAIL, e.what());
    }
  }
};

struct DequantWeightBf16State {
  const OrtApi& api;
  qfg_dequant* op = nullptr;
  std::vector<int64_t> widths;

  DequantWeightBf16State(const OrtApi& a, const OrtKernelInfo* info) : api(a) {
    Ort::ConstKernelInfo k(info);
    const int64_t n_cols = k.GetAttribute<int64_t>("n_cols");
    const int64_t col_offset = OptionalAttribute(k, "col_offset", 0);
    widths = OptionalAttributes<int64_t>(k, "widths");
    const std::vector<float> w_scale = OptionalAttributes<float>(k, "w_scale");
    if (qfg_dequant_create(n_cols, col_offset, widths.empty() ? nullptr : widths.data(),
                           static_cast<int>(widths.size()), w_scale.empty() ? nullptr : w_scale.data(),
                           w_scale.size(), &op) != QFG_OK) {
      throw std::invalid_argument(qfg_last_error());
    }
    if (widths.empty()) widths.push_back(n_cols);
  }
  ~DequantWeightBf16State() { qfg_dequant_destroy(op); }

  OrtStatus* ComputeV2(OrtKernelContext* raw) noexcept {
    try {
      Ort::KernelContext c(raw);
      const qfg_tensor2d w = Tensor2d(c.GetInput(0), "DequantWeightBf16");
      std::vector<void*> outs;
      for (size_t i = 0; i < widths.size(); ++i) {
        auto out = c.GetOutput(i, {w.rows, widths[i]});
        outs.push_back(out.GetTensorMutableRawData());
      }
      return ToStatus(api, qfg_dequant_compute(op, &w, outs.data(), static_cast<int>(outs.size()),
                                               ComputeStream(api, raw)));
    } catch (const std::exception& e) {
      return api.CreateStatus(ORT_FAIL, e.what());
    }
  }
};

struct SkinnyGemmOp : Ort::CustomOpBase<SkinnyGemmOp, SkinnyGemmState, true> {
  const char* GetName() const { return "SkinnyGemm"; }
  const char* GetExecutionProviderType() const { return "CUDAExecutionProvider"; }
  size_t GetInputTypeCount() const { return 2; }
  ONNXTensorElementDataType GetInputType(size_t i) const {
    return i == 0 ? ONNX_TENSOR_ELEMENT_DATA_TYPE_BFLOAT16 : ONNX_TENSOR_ELEMENT_DATA_TYPE_UNDEFINED;
  }
  OrtCustomOpInputOutputCharacteristic GetInputCharacteristic(size_t i) const {
    return i == 0 ? INPUT_OUTPUT_REQUIRED : INPUT_OUTPUT_VARIADIC;
  }
  bool GetVariadicInputHomogeneity() const { return false; }
  size_t GetOutputTypeCount() const { return 1; }
  ONNXTensorElementDataType GetOutputType(size_t) const { return ONNX_TENSOR_ELEMENT_DATA_TYPE_BFLOAT16; }
  OrtCustomOpInputOutputCharacteristic GetOutputCharacteristic(size_t) const { return INPUT_OUTPUT_VARIADIC; }
  OrtStatus* CreateKernelV2(const OrtApi& api, const OrtKernelInfo* info, void** kernel) const noexcept {
    try {
      *kernel = new SkinnyGemmState(api, info);
      return nullptr;
    } catch (const std::exception& e) {
      return api.CreateStatus(ORT_INVALID_ARGUMENT, e.what());
    }
  }
};

struct ArgmaxRowsOp : Ort::CustomOpBase<ArgmaxRowsOp, ArgmaxRowsState, true> {
  const char* GetName() const { return "ArgmaxRows"; }
  const char* GetExecutionProviderType() const { return "CUDAExecutionProvider"; }
  size_t GetInputTypeCount() const { return 1; }
  ONNXTensorElementDataType GetInputType(size_t) const { return ONNX_TENSOR_ELEMENT_DATA_TYPE_UNDEFINED; }
  size_t GetOutputTypeCount() const { return 2; }
  ONNXTensorElementDataType GetOutputType(size_t i) const {
    return i == 0 ? ONNX_TENSOR_ELEMENT_DATA_TYPE_INT64 : ONNX_TENSOR_ELEMENT_DATA_TYPE_FLOAT;
  }
  OrtCustomOpInputOutputCharacteristic GetOutputCharacteristic(size_t i) const {
    return i == 0 ? INPUT_OUTPUT_REQUIRED : INPUT_OUTPUT_OPTIONAL;
  }
  OrtStatus* CreateKernelV2(const OrtApi& api, const OrtKernelInfo*, void** kernel) const noexcept {
    *kernel = new ArgmaxRowsState(api);
    return nullptr;
  }
};

struct DequantWeightBf16Op : Ort::CustomOpBase<DequantWeightBf16Op, DequantWeightBf16State, true> {
  const char* GetName() const { return "DequantWeightBf16"; }
  const char* GetExecutionProviderType() const { return "CUDAExecutionProvider"; }
  size_t GetInputTypeCount() const { return 2; }
  ONNXTensorElementDataType GetInputType(size_t) const { return ONNX_TENSOR_ELEMENT_DATA_TYPE_UNDEFINED; }
  OrtCustomOpInputOutputCharacteristic GetInputCharacteristic(size_t i) const {
    return i == 0 ? INPUT_OUTPUT_REQUIRED : INPUT_OUTPUT_OPTIONAL;
  }
  size_t GetOutputTypeCount() const { return QFG_MAX_OUTPUTS; }
  ONNXTensorElementDataType GetOutputType(size_t) const { return ONNX_TENSOR_ELEMENT_DATA_TYPE_BFLOAT16; }
  OrtCustomOpInputOutputCharacteristic GetOutputCharacteristic(size_t i) const {
    return i == 0 ? INPUT_OUTPUT_REQUIRED : INPUT_OUTPUT_OPTIONAL;
  }
  OrtStatus* CreateKernelV2(const OrtApi& api, const OrtKernelInfo* info, void** kernel) const noexcept {
    try {
      *kernel = new DequantWeightBf16State(api, info);
      return nullptr;
    } catch (const std::exception& e) {
      return api.CreateStatus(ORT_INVALID_ARGUMENT, e.what());
    }
  }
};

int64_t ElementCount(const Ort::ConstValue& v) {
  int64_t n = 1;
  for (int64_t d : v.GetTensorTypeAndShapeInfo().GetShape()) n *= d;
  return n;
}

// Six inputs g, u, w, gx, gw, routed -> one output shaped like routed (src/fused_gemm/fused_gemm.cu:630-727, :799-816).
struct SharedExpertDownState {
  const OrtApi& api;
  qfg_shared_expert_down* op = nullptr;

  SharedExpertDownState(const OrtApi& a, const OrtKernelInfo* info) : api(a) {
    Ort::ConstKernelInfo k(info);
    const std::vector<float> w_scale = OptionalAttributes<float>(k, "w_scale");
    const int trigger = static_cast<int>(OptionalAttribute(k, "trigger", 0));
    if (qfg_shared_expert_down_create(w_scale.empty() ? nullptr : w_scale.data(), w_scale.size(), trigger, &op) != QFG_OK)
      throw std::invalid_argument(qfg_last_error());
  }
  ~SharedExpertDownState() { qfg_shared_expert_down_destroy(op); }

  OrtStatus* ComputeV2(OrtKernelContext* raw) noexcept {
    try {
      Ort::KernelContext c(raw);
      if (c.GetInputCount() != 6) throw std::invalid_argument("SharedExpertDown: needs 6 inputs");
      const qfg_tensor2d w = Tensor2d(c.GetInput(2), "SharedExpertDown");
      const auto routed_shape = c.GetInput(5).GetTensorTypeAndShapeInfo().GetShape();
      const int64_t K = w.rows, N = routed_shape.empty() ? 0 : routed_shape.back();
      const int64_t M = K > 0 ? ElementCount(c.GetInput(0)) / K : 0;
      const int64_t gk = ElementCount(c.GetInput(4));
      const auto gw_shape = c.GetInput(4).GetTensorTypeAndShapeInfo().GetShape();
      if (M < 1 || ElementCount(c.GetInput(0)) != M * K || ElementCount(c.GetInput(1)) != M * K ||
          ElementCount(c.GetInput(5)) != M * N || ElementCount(c.GetInput(3)) != M * gk || gw_shape.empty() ||
          gw_shape.back() != 1) {
        throw std::invalid_argument("SharedExpertDown: shape mismatch");
      }
      if (w.dtype == QFG_UINT8 ? (N % 16 != 0 || w.cols != N * 9 / 16) : w.cols != N)
        throw std::invalid_argument("SharedExpertDown: weight N mismatch");
      auto out = c.GetOutput(0, routed_shape);
      return ToStatus(api, qfg_shared_expert_down_compute(op, c.GetInput(0).GetTensorRawData(), c.GetInput(1).GetTensorRawData(),
                                                          M, K, &w, c.GetInput(3).GetTensorRawData(), gk,
                                                          c.GetInput(4).GetTensorRawData(), c.GetInput(5).GetTensorRawData(), N,
                                                          out.GetTensorMutableRawData(), ComputeStream(api, raw)));
    } catch (const std::exception& e) {
      return api.CreateStatus(ORT_FAIL, e.what());
    }
  }
};

struct SharedExpertDownOp : Ort::CustomOpBase<SharedExpertDownOp, SharedExpertDownState, true> {
  const char* GetName() const { return "SharedExpertDown"; }
  const char* GetExecutionProviderType() const { return "CUDAExecutionProvider"; }
  size_t GetInputTypeCount() const { return 6; }
  ONNXTensorElementDataType GetInputType(size_t i) const {
    return i == 2 ? ONNX_TENSOR_ELEMENT_DATA_TYPE_UNDEFINED : ONNX_TENSOR_ELEMENT_DATA_TYPE_BFLOAT16;
  }
  size_t GetOutputTypeCount() const { return 1; }
  ONNXTensorElementDataType GetOutputType(size_t) const { return ONNX_TENSOR_ELEMENT_DATA_TYPE_BFLOAT16; }
  OrtStatus* CreateKernelV2(const OrtApi& api, const OrtKernelInfo* info, void** kernel) const noexcept {
    try {
      *kernel = new SharedExpertDownState(api, info);
      return nullptr;
    } catch (const std::exception& e) {
      return api.CreateStatus(ORT_INVALID_ARGUMENT, e.what());
    }
  }
};

// [160, 20480] -> [10240, 320] (kind 0) or [320, 10240] (kind 1) (src/fused_gemm/fused_gemm.cu:1013-1089).
struct UntileHcBf16State {
  const OrtApi& api;
  qfg_untile_hc* op = nullptr;
  int kind = 0;

  UntileHcBf16State(const OrtApi& a, const OrtKernelInfo* info) : api(a) {
    Ort::ConstKernelInfo k(info);
    kind = static_cast<int>(k.GetAttribute<int64_t>("kind"));
    const std::vector<float> w_scale = OptionalAttributes<float>(k, "w_scale");
    if (qfg_untile_hc_create(kind, w_scale.empty() ? nullptr : w_scale.data(), w_scale.size(), &op) != QFG_OK)
      throw std::invalid_argument(qfg_last_error());
  }
  ~UntileHcBf16State() { qfg_untile_hc_destroy(op); }

  OrtStatus* ComputeV2(OrtKernelContext* raw) noexcept {
    try {
      Ort::KernelContext c(raw);
      const qfg_tensor2d w = Tensor2d(c.GetInput(0), "UntileHcBf16");
      if (w.rows != 160 || w.cols != 20480) throw std::invalid_argument("UntileHcBf16: expected [160, 20480]");
      auto out = kind == 0 ? c.GetOutput(0, {10240, 320}) : c.GetOutput(0, {320, 10240});
      return ToStatus(api, qfg_untile_hc_compute(op, &w, out.GetTensorMutableRawData(), ComputeStream(api, raw)));
    } catch (const std::exception& e) {
      return api.CreateStatus(ORT_FAIL, e.what());
    }
  }
};

struct UntileHcBf16Op : Ort::CustomOpBase<UntileHcBf16Op, UntileHcBf16State, true> {
  const char* GetName() const { return "UntileHcBf16"; }
  const char* GetExecutionProviderType() const { return "CUDAExecutionProvider"; }
  size_t GetInputTypeCount() const { return 2; }
  ONNXTensorElementDataType GetInputType(size_t) const { return ONNX_TENSOR_ELEMENT_DATA_TYPE_UNDEFINED; }
  OrtCustomOpInputOutputCharacteristic GetInputCharacteristic(size_t i) const {
    return i == 0 ? INPUT_OUTPUT_REQUIRED : INPUT_OUTPUT_OPTIONAL;
  }
  size_t GetOutputTypeCount() const { return 1; }
  ONNXTensorElementDataType GetOutputType(size_t) const { return ONNX_TENSOR_ELEMENT_DATA_TYPE_BFLOAT16; }
  OrtStatus* CreateKernelV2(const OrtApi& api, const OrtKernelInfo* info, void** kernel) const noexcept {
    try {
      *kernel = new UntileHcBf16State(api, info);
      return nullptr;
    } catch (const std::exception& e) {
      return api.CreateStatus(ORT_INVALID_ARGUMENT, e.what());
    }
  }
};

}  // namespace

extern "C" __attribute__((visibility("default"))) OrtStatus* ORT_API_CALL RegisterCustomOps(
    OrtSessionOptions* options, const OrtApiBase* api_base) {
  const OrtApi* api = api_base->GetApi(ORT_API_VERSION);
  if (api == nullptr) return api_base->GetApi(1)->CreateStatus(ORT_FAIL, "Unsupported ORT API");
  Ort::InitApi(api);
  try {
    static SkinnyGemmOp skinny_gemm;
    static SharedExpertDownOp shared_down;
    static ArgmaxRowsOp argmax_rows;
    static DequantWeightBf16Op dequant;
    static UntileHcBf16Op untile;
    static Ort::CustomOpDomain domain("qwen.fused_gemm");
    static std::once_flag registered;
    std::call_once(registered, [&]() {
      domain.Add(&skinny_gemm);
      domain.Add(&shared_down);
      domain.Add(&argmax_rows);
      domain.Add(&dequant);
      domain.Add(&untile);
    });
    Ort::UnownedSessionOptions(options).Add(domain);
    return nullptr;
  } catch (const std::exception& e) {
    return api->CreateStatus(ORT_FAIL, e.what());
  }
}
