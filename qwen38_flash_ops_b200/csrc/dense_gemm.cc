// Prefill-shaped SkinnyGemm calls: many rows of x against the same weights.
//
// The streaming kernels read the weights once per eight rows, which is the right trade for decode and the
// wrong one for hundreds of rows.  Past a row threshold the call is served the way the reference serves its
// M > 8 calls (fused_gemm.cu:292-428, dispatch at :578-583): quantised weights (and BF16 weights with a
// w_scale) are dequantised in column tiles into a cached BF16 buffer, w_scale folded in before the rounding,
// and a library GEMM with FP32 accumulation produces each output slice.  cuBLAS is a plain library call here,
// as it is in the reference; it is looked up at run time so that the decode library carries no link-time
// dependency on it.  This branch allocates (handle, buffer) on first use and is not graph-capturable, like
// the reference's.
#include <cublas_v2.h>
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <algorithm>
#include <cstdlib>
#include <map>
#include <mutex>
#include <stdexcept>
#include <string>
#include <utility>

#include "qfg_internal.h"

namespace qfg {
namespace {

// Columns dequantised per GEMM call.  QFG_DENSE_TILE overrides it (a multiple of 16).
int DenseTileCols() {
  static const int cols = [] {
    const char* e = std::getenv("QFG_DENSE_TILE");
    const int v = e != nullptr ? std::atoi(e) : 0;
    return v >= 16 && v % 16 == 0 ? v : 16384;
  }();
  return cols;
}

using GemmExFn = cublasStatus_t (*)(cublasHandle_t, cublasOperation_t, cublasOperation_t, int, int, int, const void*,
                                    const void*, cudaDataType, int, const void*, cudaDataType, int, const void*, void*,
                                    cudaDataType, int, cublasComputeType_t, cublasGemmAlgo_t);

struct CublasApi {
  cublasStatus_t (*create)(cublasHandle_t*) = nullptr;
  cublasStatus_t (*set_stream)(cublasHandle_t, cudaStream_t) = nullptr;
  GemmExFn gemm_ex = nullptr;
  std::string error;
};

const CublasApi& Cublas() {
  static const CublasApi api = [] {
    CublasApi a;
    void* lib = nullptr;
    for (const char* name : {"libcublas.so.12", "libcublas.so"}) {
      lib = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
      if (lib != nullptr) break;
    }
    if (lib == nullptr) {
      a.error = "cuBLAS could not be loaded (libcublas.so.12)";
      return a;
    }
    a.create = reinterpret_cast<decltype(a.create)>(dlsym(lib, "cublasCreate_v2"));
    a.set_stream = reinterpret_cast<decltype(a.set_stream)>(dlsym(lib, "cublasSetStream_v2"));
    a.gemm_ex = reinterpret_cast<decltype(a.gemm_ex)>(dlsym(lib, "cublasGemmEx"));
    if (a.create == nullptr || a.set_stream == nullptr || a.gemm_ex == nullptr) a.error = "cuBLAS lacks an expected symbol";
    return a;
  }();
  return api;
}

// One handle and one dequantisation buffer per (device, stream): two streams never share a buffer, so calls
// on different streams cannot overwrite each other's weights while a GEMM still reads them.
struct DenseContext {
  cublasHandle_t handle = nullptr;
  uint16_t* buf = nullptr;
  size_t cap = 0;  // elements
};

std::mutex g_mu;
std::map<std::pair<int, cudaStream_t>, DenseContext> g_ctx;

uint16_t* EnsureBuffer(DenseContext& c, size_t elems, cudaStream_t stream) {
  if (elems <= c.cap) return c.buf;
  if (c.buf != nullptr) {
    // Work queued earlier on this stream may still read the old buffer.
    if (cudaStreamSynchronize(stream) != cudaSuccess) throw std::runtime_error("SkinnyGemm(dense): stream synchronize failed");
    cudaFree(c.buf);
    c.buf = nullptr;
    c.cap = 0;
  }
  void* p = nullptr;
  if (cudaMalloc(&p, elems * sizeof(uint16_t)) != cudaSuccess) {
    cudaGetLastError();
    throw std::runtime_error("SkinnyGemm(dense): cannot allocate the dequantisation buffer");
  }
  c.buf = static_cast<uint16_t*>(p);
  c.cap = elems;
  return c.buf;
}

}  // namespace

bool DenseEligible(const GemmParams& p) {
  if (p.lm || p.fuse) return false;
  const int n_out = p.seg[p.nseg - 1].out_end;
  for (int o = 0; o < n_out; ++o) {
    if (p.width[o] % 8 != 0) return false;  // the dequantisation kernel writes eight columns per thread
  }
  return true;
}

void LaunchDenseGemm(int mode, const GemmParams& p, int64_t m, cudaStream_t stream) {
  const CublasApi& api = Cublas();
  if (!api.error.empty()) throw std::runtime_error("SkinnyGemm(dense): " + api.error);
  if (m > INT_MAX) throw std::runtime_error("SkinnyGemm(dense): too many rows");
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess) throw std::runtime_error("SkinnyGemm(dense): no current device");

  std::lock_guard<std::mutex> lock(g_mu);
  DenseContext& ctx = g_ctx[{device, stream}];
  if (ctx.handle == nullptr) {
    if (api.create(&ctx.handle) != CUBLAS_STATUS_SUCCESS) throw std::runtime_error("SkinnyGemm(dense): cublasCreate failed");
    if (api.set_stream(ctx.handle, stream) != CUBLAS_STATUS_SUCCESS)
      throw std::runtime_error("SkinnyGemm(dense): cublasSetStream failed");
  }
  const float alpha = 1.f, beta = 0.f;
  const int kDenseTileCols = DenseTileCols();
  const int K = p.K;
  const int M = static_cast<int>(m);
  size_t need = 0;
  for (int s = 0; s < p.nseg; ++s) {
    if (mode == kBf16 && p.seg[s].w_scale == nullptr) continue;
    for (int o = p.seg[s].out_begin; o < p.seg[s].out_end; ++o) {
      if (p.out[o] != nullptr) need = std::max(need, static_cast<size_t>(K) * std::min(kDenseTileCols, p.width[o]));
    }
  }
  uint16_t* const buf = need > 0 ? EnsureBuffer(ctx, need, stream) : nullptr;
  for (int s = 0; s < p.nseg; ++s) {
    const Segment& sg = p.seg[s];
    const bool direct = mode == kBf16 && sg.w_scale == nullptr;
    // Logical columns of a stored row, which may be wider than the columns this call uses.
    const long long stored_cols = mode == kBf16 ? sg.pitch / 2 : mode == kFp8 ? sg.pitch : sg.pitch * 16 / 9;
    for (int o = sg.out_begin; o < sg.out_end; ++o) {
      if (p.out[o] == nullptr) continue;
      const int cb = p.col_begin[o];
      const int width = p.width[o];
      for (int t = 0; t < width; t += kDenseTileCols) {
        const int cur = std::min(kDenseTileCols, width - t);
        const void* a = nullptr;
        int lda = 0;
        if (direct) {
          a = reinterpret_cast<const uint16_t*>(sg.w) + cb + t;
          lda = static_cast<int>(stored_cols);
        } else {
          DequantParams d;
          d.w = sg.w;
          d.w_scale = sg.w_scale != nullptr ? sg.w_scale + cb + t : nullptr;
          d.mode = mode;
          d.K = K;
          d.N = cur;
          d.row_stride = static_cast<int>(stored_cols);
          d.col_offset = cb + t;
          d.num_outs = 1;
          d.out[0] = buf;
          d.col_begin[0] = 0;
          d.width[0] = cur;
          const uintptr_t addr = reinterpret_cast<uintptr_t>(sg.w);
          d.aligned = mode == kBf16  ? addr % 16 == 0 && sg.pitch % 16 == 0
                      : mode == kFp8 ? addr % 8 == 0 && sg.pitch % 8 == 0
                                     : addr % 4 == 0 && sg.pitch % 4 == 0;
          const cudaError_t err = LaunchDequant(d, stream);
          if (err != cudaSuccess) throw std::runtime_error(std::string("SkinnyGemm(dense): ") + cudaGetErrorString(err));
          a = buf;
          lda = cur;
        }
        // Row-major out[M, width] = x[M, K] @ W[K, cur] is the column-major product W^T-as-stored x x^T-as-stored.
        const cublasStatus_t st =
            api.gemm_ex(ctx.handle, CUBLAS_OP_N, CUBLAS_OP_N, cur, M, K, &alpha, a, CUDA_R_16BF, lda, p.x, CUDA_R_16BF, K,
                        &beta, p.out[o] + t, CUDA_R_16BF, width, CUBLAS_COMPUTE_32F, CUBLAS_GEMM_DEFAULT_TENSOR_OP);
        if (st != CUBLAS_STATUS_SUCCESS)
          throw std::runtime_error("SkinnyGemm(dense): cublasGemmEx failed with status " + std::to_string(static_cast<int>(st)));
      }
    }
  }
}

}  // namespace qfg
