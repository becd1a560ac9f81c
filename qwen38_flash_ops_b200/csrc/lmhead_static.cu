// The fused LM head for callers that cannot allocate device memory.
//
// Some hosts of this library have no way to hand it scratch memory: a plugin whose compute hook
// runs after the host application has frozen its memory pools, an inference server that forbids
// cudaMalloc once serving has started, or a custom-op hook that only receives its inputs and
// outputs.  qfg_lmhead_compute_static is qfg_lmhead_compute without the `workspace` argument:
// the keys and the arrival counter that the fused kernel folds its per-CTA (max, index) pairs
// into live in the file-scope device array below instead of in caller memory.
//
// Consequences of a fixed array:
//   * its size is fixed (kStaticScratchBytes, enough for the eight rows one call may have), and
//     every GPU that loads this library holds it until the process exits;
//   * all calls on a device share it, so two calls that overlap on the GPU (different streams)
//     race; calls on one stream are ordered and safe;
//   * it keeps what the last call left in it.  The kernel leaves the keys and the counter at
//     zero when it finishes, and the first call on a device clears the array before use.
// The first call on each device does that set-up: the address look-up, a clear, and a device-wide
// synchronisation so that the clear has finished before any kernel - on whatever stream, blocking or
// not - can touch the array.  That first call therefore belongs before any stream capture begins.
// No call allocates or frees anything.
//
// Without a caller workspace there is no room for the partial sums of the "shared tail" launch shape
// that qfg_lmhead_compute uses for vocabularies whose 128-column groups do not divide by the SM count,
// so this entry point runs the plain launch shape: about a tenth slower on such vocabularies, and the
// columns the shared tail would cover are summed over K in the plain kernel's order (their logits can
// differ from qfg_lmhead_compute's by one BF16 unit; each entry point's argmax is exact on its own logits).
#include <cuda_runtime.h>

#include <mutex>
#include <string>

#include "qfg_internal.h"

namespace {

constexpr size_t kStaticScratchBytes = 256;  // 8 keys of 8 bytes, one 4-byte counter, padding
constexpr int kMaxDevices = 64;

static __device__ __align__(256) unsigned char g_lmhead_static_scratch[kStaticScratchBytes];

std::mutex g_setup_mu;
void* g_scratch_ptr[kMaxDevices] = {};

// The array's name is only a host-side handle here; its device address has to be looked up, per
// device, with that device current.  Returns nullptr and sets the error message on failure.
void* ScratchForCurrentDevice() {
  int dev = -1;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    qfg::SetLastError(QFG_FAIL, "LmHead(static): cannot identify the current device");
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_setup_mu);
  if (g_scratch_ptr[dev] != nullptr) return g_scratch_ptr[dev];
  void* ptr = nullptr;
  err = cudaGetSymbolAddress(&ptr, g_lmhead_static_scratch);
  if (err == cudaSuccess) err = cudaMemset(ptr, 0, kStaticScratchBytes);
  // the clear runs on the legacy stream, which non-blocking streams do not wait for: finish it here
  if (err == cudaSuccess) err = cudaDeviceSynchronize();
  if (err != cudaSuccess || ptr == nullptr) {
    const std::string msg = std::string("LmHead(static): scratch set-up failed: ") + cudaGetErrorString(err);
    qfg::SetLastError(QFG_FAIL, msg.c_str());
    return nullptr;
  }
  g_scratch_ptr[dev] = ptr;
  return ptr;
}

}  // namespace

extern "C" QFG_API size_t qfg_lmhead_static_max_rows(void) { return qfg::kMaxRows; }

extern "C" QFG_API int qfg_lmhead_compute_static(const qfg_lmhead* op, const void* x, int64_t m, int64_t k,
                                                 const qfg_tensor2d* weight, int64_t n, int64_t col_offset, int64_t* idx,
                                                 float* val, uint64_t* key, void* logits, void* stream) {
  if (m < 1 || static_cast<size_t>(m) > qfg_lmhead_static_max_rows()) {
    return qfg::SetLastError(QFG_INVALID_ARGUMENT,
                             "LmHead(static): the built-in scratch holds at most 8 rows per call; split the batch");
  }
  static_assert(kStaticScratchBytes >= qfg::kMaxRows * 8 + 4, "scratch too small for the keys and the counter");
  void* scratch = ScratchForCurrentDevice();
  if (scratch == nullptr) return QFG_FAIL;
  return qfg::LmheadComputeWithWorkspace(op, x, m, k, weight, n, col_offset, scratch, kStaticScratchBytes, idx, val, key, logits,
                                         stream);
}
