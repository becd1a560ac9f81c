// ArgmaxRows for B200: idx[r] = argmax_v x[r, v] with numpy semantics (lowest index on ties, the
// first NaN wins over everything, -0 == +0), optionally with the maximum as FP32.
//
// One thread-block cluster per row.  Each CTA scans a contiguous range of the row with 16-byte
// loads (a scalar head and tail absorb any misalignment, so odd vocabulary sizes and unaligned
// rows still take the vector body), six to ten loads in flight per thread; (value, index) pairs are
// reduced with the same total order at every level - lanes, warps, then the CTAs of the cluster
// through distributed shared memory - so the result does not depend on the launch geometry.
// No workspace, no atomics.
#include <cooperative_groups.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <climits>

#include "qfg_internal.h"

namespace qfg {
namespace {

namespace cg = cooperative_groups;

constexpr int kThreads = 512;  // 1024 threads per CTA measured slower at every row count (5.7 us against 4.8 for one row)
constexpr int kNone = INT_MAX;

__device__ __forceinline__ bool Better(float av, int ai, float bv, int bi) {
  if (av != av) return (bv == bv) || ai < bi;
  if (bv != bv) return false;
  return av > bv || (av == bv && ai < bi);
}

__device__ __forceinline__ float ToFloat(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float ToFloat(__half v) { return __half2float(v); }
__device__ __forceinline__ float ToFloat(float v) { return v; }

// Order-independent update: keeps the best pair under `Better`.
__device__ __forceinline__ void Consider(float& bv, int& bi, float v, int idx) {
  if (bi == kNone || Better(v, idx, bv, bi)) {
    bv = v;
    bi = idx;
  }
}

// The same update for a candidate whose index exceeds every index seen so far by this thread: a strict
// comparison keeps the lowest index of equal values, and a NaN is never replaced.
__device__ __forceinline__ void ConsiderInOrder(float& bv, int& bi, float v, int idx) {
  if (bi == kNone || v > bv || (v != v && bv == bv)) {
    bv = v;
    bi = idx;
  }
}

__device__ __forceinline__ void WarpReduce(float& v, int& i) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, off);
    const int oi = __shfl_xor_sync(0xffffffffu, i, off);
    if (oi != kNone && (i == kNone || Better(ov, oi, v, i))) {
      v = ov;
      i = oi;
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads) ArgmaxRowsKernel(const T* __restrict__ x, long long V,
                                                             long long* __restrict__ idx_out,
                                                             float* __restrict__ val_out) {
  constexpr int kVecElems = 16 / sizeof(T);
  constexpr int kWarps = kThreads / 32;
  __shared__ float s_wv[kWarps];
  __shared__ int s_wi[kWarps];
  __shared__ float s_cv;
  __shared__ int s_ci;

  const int C = static_cast<int>(gridDim.x);
  const int c = static_cast<int>(blockIdx.x);
  const long long row = blockIdx.y;
  const T* xr = x + row * V;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  // Row layout: `head` scalar elements up to the first 16-byte boundary, `nvec` vectors, a scalar tail.
  const uintptr_t addr = reinterpret_cast<uintptr_t>(xr);
  long long head = ((16 - (addr & 15)) & 15) / sizeof(T);
  if (head > V) head = V;
  const long long nvec = (V - head) / kVecElems;
  const long long tail_begin = head + nvec * kVecElems;

  float bv = 0.f;
  int bi = kNone;

  // vectors are split evenly over the CTAs of the cluster
  const long long per = (nvec + C - 1) / C;
  const long long vbeg = min(nvec, per * c);
  const long long vend = min(nvec, vbeg + per);
  const uint4* xv = reinterpret_cast<const uint4*>(xr + head);
  // 8 CTAs x 512 threads x 6 (10 for FP32) loads cover a 151936-column row in one round trip to L2: the
  // kernel is a few microseconds of latency and a second, mostly empty trip through the loop adds one more.
  constexpr int kInFlight = sizeof(T) == 4 ? 10 : 6;
  for (long long v0 = vbeg + tid; v0 < vend; v0 += static_cast<long long>(kThreads) * kInFlight) {
    uint4 q[kInFlight];
#pragma unroll
    for (int i = 0; i < kInFlight; ++i) {
      const long long v = v0 + static_cast<long long>(i) * kThreads;
      q[i] = v < vend ? __ldg(xv + v) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int i = 0; i < kInFlight; ++i) {
      const long long v = v0 + static_cast<long long>(i) * kThreads;
      if (v < vend) {
        const T* e = reinterpret_cast<const T*>(&q[i]);
#pragma unroll
        for (int j = 0; j < kVecElems; ++j) {
          ConsiderInOrder(bv, bi, ToFloat(e[j]), static_cast<int>(head + v * kVecElems + j));
        }
      }
    }
  }
  // head goes to the first CTA, tail to the last
  if (c == 0) {
    for (long long i = tid; i < head; i += kThreads) Consider(bv, bi, ToFloat(xr[i]), static_cast<int>(i));
  }
  if (c == C - 1) {
    for (long long i = tail_begin + tid; i < V; i += kThreads) Consider(bv, bi, ToFloat(xr[i]), static_cast<int>(i));
  }

  WarpReduce(bv, bi);
  if (lane == 0) {
    s_wv[warp] = bv;
    s_wi[warp] = bi;
  }
  __syncthreads();
  if (warp == 0) {
    float v = lane < kWarps ? s_wv[lane] : 0.f;
    int i = lane < kWarps ? s_wi[lane] : kNone;
    WarpReduce(v, i);
    if (lane == 0) {
      s_cv = v;
      s_ci = i;
    }
  }
  cg::cluster_group cluster = cg::this_cluster();
  cluster.sync();
  if (c == 0 && warp == 0) {
    float v = 0.f;
    int i = kNone;
    if (lane < C) {
      v = *cluster.map_shared_rank(&s_cv, lane);
      i = *cluster.map_shared_rank(&s_ci, lane);
    }
    WarpReduce(v, i);
    if (lane == 0) {
      idx_out[row] = i;
      if (val_out != nullptr) val_out[row] = v;
    }
  }
  cluster.sync();
}

template <typename T>
cudaError_t LaunchT(const T* x, int64_t rows, int64_t V, int64_t* idx, float* val, cudaStream_t s) {
  // enough CTAs per row that each thread sees a few vectors; at most the portable cluster size
  const long long vecs = V / (16 / static_cast<long long>(sizeof(T)));
  int cluster = 1;
  while (cluster < 8 && vecs > static_cast<long long>(cluster) * kThreads * 2) cluster *= 2;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(cluster), static_cast<unsigned>(rows), 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = static_cast<unsigned>(cluster);
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, ArgmaxRowsKernel<T>, x, static_cast<long long>(V),
                            reinterpret_cast<long long*>(idx), val);
}

// Folds gathered (value, index) keys: the unsigned maximum of the 64-bit words of a row.
__global__ void LmheadCombineKernel(const unsigned long long* __restrict__ keys, int ranks, int m,
                                    long long* __restrict__ idx, float* __restrict__ val) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= m) return;
  unsigned long long best = 0;
  for (int r = 0; r < ranks; ++r) {
    const unsigned long long k = keys[static_cast<size_t>(r) * m + row];
    best = k > best ? k : best;
  }
  const uint32_t ord = static_cast<uint32_t>(best >> 32);
  const uint32_t bits = (ord == 0xFFFFFFFFu) ? 0x7FC00000u : ((ord & 0x80000000u) ? (ord & 0x7FFFFFFFu) : ~ord);
  if (idx != nullptr) idx[row] = static_cast<long long>(0xFFFFFFFFu - static_cast<uint32_t>(best));
  if (val != nullptr) val[row] = __uint_as_float(bits);
}

}  // namespace

cudaError_t LaunchArgmaxRows(int dtype, const void* x, int64_t rows, int64_t vocab, int64_t* idx, float* val,
                             cudaStream_t stream) {
  if (rows < 1 || vocab < 1 || vocab >= INT_MAX || rows > 65535) return cudaErrorInvalidValue;
  switch (dtype) {
    case QFG_BFLOAT16: return LaunchT(static_cast<const __nv_bfloat16*>(x), rows, vocab, idx, val, stream);
    case QFG_FLOAT16: return LaunchT(static_cast<const __half*>(x), rows, vocab, idx, val, stream);
    case QFG_FLOAT: return LaunchT(static_cast<const float*>(x), rows, vocab, idx, val, stream);
    default: return cudaErrorInvalidValue;
  }
}

cudaError_t LaunchLmheadCombine(const uint64_t* keys, int ranks, int64_t m, int64_t* idx, float* val,
                                cudaStream_t stream) {
  if (ranks < 1 || m < 1) return cudaErrorInvalidValue;
  const int threads = 64;
  const int blocks = static_cast<int>((m + threads - 1) / threads);
  LmheadCombineKernel<<<blocks, threads, 0, stream>>>(reinterpret_cast<const unsigned long long*>(keys), ranks,
                                                      static_cast<int>(m), reinterpret_cast<long long*>(idx), val);
  return cudaGetLastError();
}

}  // namespace qfg
