// TEST INFRASTRUCTURE.  A thin extern "C" wrapper around the reference project's own kernel
// headers (src/fused_gemm/skinny_gemm.cuh and argmax_rows.cuh), which are compiled where they lie
// in the reference checkout - nothing of them is copied here.  The resulting library
// (oracle/_ref/libref_kernels.so, never committed) is the reference's GPU implementation
// recompiled for sm_100a: the tests use it as a second oracle and the benchmark's reference arm
// reports its speed beside the CPU baseline.
//
// The launch configuration is the reference's generic fallback (src/fused_gemm/fused_gemm.cu:167-174:
// tx = 8, 256 threads, unroll 4, cluster chosen from the 64-column tile count), which is what its
// planner returns for every shape that is not in its H200 tuning table.  Only that configuration
// is instantiated, to keep the build short.
#include <cuda_runtime.h>

#include <cstdint>

#include "argmax_rows.cuh"
#include "skinny_gemm.cuh"

namespace {

template <int M>
cudaError_t LaunchCluster(const skinny::Params& p, int cluster, cudaStream_t s) {
  switch (cluster) {
    case 1: return skinny::LaunchT<M, 8, 256, 1, 4>(p, s);
    case 2: return skinny::LaunchT<M, 8, 256, 2, 4>(p, s);
    case 4: return skinny::LaunchT<M, 8, 256, 4, 4>(p, s);
    case 8: return skinny::LaunchT<M, 8, 256, 8, 4>(p, s);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace

extern "C" {

// One SkinnyGemm call of at most four rows.  Arrays are indexed by weight (nseg <= 4) or by
// output (n_outs <= 8) exactly like skinny::Params.  Returns a cudaError_t.
__attribute__((visibility("default"))) int ref_skinny_gemm(
    const void* x, int m, int k, int nseg, const void* const* w, const int* w_mode, const int* n,
    const float* const* w_scale, const int* seg_outs, void* const* outs, const int* widths, int trigger,
    int cluster_override, void* stream) {
  if (m < 1 || m > 4 || nseg < 1 || nseg > skinny::kMaxSeg) return static_cast<int>(cudaErrorInvalidValue);
  skinny::Params p = {};
  p.x = static_cast<const skinny::bf16*>(x);
  p.K = k;
  p.nseg = nseg;
  p.trigger = trigger;
  int o = 0, total = 0;
  for (int s = 0; s < nseg; ++s) {
    p.out_begin[s] = o;
    int begin = 0;
    for (int i = 0; i < seg_outs[s]; ++i, ++o) {
      p.out[o] = static_cast<skinny::bf16*>(outs[o]);
      p.col_begin[o] = begin;
      p.width[o] = widths[o];
      begin += widths[o];
    }
    if (begin != n[s]) return static_cast<int>(cudaErrorInvalidValue);
    p.n[s] = n[s];
    p.w_mode[s] = w_mode[s];
    if (w_mode[s] == 0) {
      p.w[s] = static_cast<const skinny::bf16*>(w[s]);
    } else {
      p.w_q[s] = static_cast<const uint8_t*>(w[s]);
    }
    p.w_scale[s] = w_scale[s];
    total += n[s];
  }
  p.out_begin[nseg] = o;
  const long tiles = (total + 63) / 64;
  int cluster = tiles >= 256 ? 1 : tiles >= 128 ? 2 : tiles >= 64 ? 4 : 8;
  if (cluster_override > 0) cluster = cluster_override;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t err;
  switch (m) {
    case 1: err = LaunchCluster<1>(p, cluster, s); break;
    case 2: err = LaunchCluster<2>(p, cluster, s); break;
    case 3: err = LaunchCluster<3>(p, cluster, s); break;
    default: err = LaunchCluster<4>(p, cluster, s); break;
  }
  if (err == cudaSuccess) err = cudaGetLastError();
  return static_cast<int>(err);
}

// SharedExpertDown of at most four rows with the launch configuration the reference operator uses
// (src/fused_gemm/fused_gemm.cu:680-689: 512 threads, no cluster, unroll 8, tx = 8 for FP8 and 4 otherwise).
// Only m = 1, 2 and 4 are instantiated, to keep the build short.
__attribute__((visibility("default"))) int ref_shared_expert_down(
    const void* g, const void* u, int m, int k, const void* w, int w_mode, int n, const float* w_scale, const void* gx,
    int gk, const void* gw, const void* routed, void* out, int trigger, void* stream) {
  skinny::Params p = {};
  p.trigger = trigger;
  p.x = static_cast<const skinny::bf16*>(g);
  p.x2 = static_cast<const skinny::bf16*>(u);
  p.K = k;
  p.nseg = 1;
  p.n[0] = n;
  p.w_mode[0] = w_mode;
  if (w_mode == 0) {
    p.w[0] = static_cast<const skinny::bf16*>(w);
  } else {
    p.w_q[0] = static_cast<const uint8_t*>(w);
    p.w_scale[0] = w_scale;
  }
  p.out_begin[0] = 0;
  p.out_begin[1] = 1;
  p.out[0] = static_cast<skinny::bf16*>(out);
  p.col_begin[0] = 0;
  p.width[0] = n;
  p.gx = static_cast<const skinny::bf16*>(gx);
  p.gw = static_cast<const skinny::bf16*>(gw);
  p.routed = static_cast<const skinny::bf16*>(routed);
  p.gk = gk;
  if (k > skinny::kFuseMaxK) return static_cast<int>(cudaErrorInvalidValue);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t err = cudaErrorInvalidValue;
  if (w_mode == 1) {
    if (m == 1) err = skinny::LaunchT<1, 8, 512, 1, 8, true>(p, s);
    if (m == 2) err = skinny::LaunchT<2, 8, 512, 1, 8, true>(p, s);
    if (m == 4) err = skinny::LaunchT<4, 8, 512, 1, 8, true>(p, s);
  } else {
    if (m == 1) err = skinny::LaunchT<1, 4, 512, 1, 8, true>(p, s);
    if (m == 2) err = skinny::LaunchT<2, 4, 512, 1, 8, true>(p, s);
    if (m == 4) err = skinny::LaunchT<4, 4, 512, 1, 8, true>(p, s);
  }
  if (err == cudaSuccess) err = cudaGetLastError();
  return static_cast<int>(err);
}

// type: 0 = BF16, 1 = FP16, 2 = FP32 (skinny::LogitType).
__attribute__((visibility("default"))) int ref_argmax_rows(int type, const void* x, long long rows, long long vocab,
                                                           long long* idx, float* val, void* stream) {
  cudaError_t err = skinny::LaunchArgmaxRows(static_cast<skinny::LogitType>(type), x, rows, vocab,
                                             reinterpret_cast<int64_t*>(idx), val, static_cast<cudaStream_t>(stream));
  if (err == cudaSuccess) err = cudaGetLastError();
  return static_cast<int>(err);
}

}  // extern "C"
