// ArgmaxRows for B200: idx[r] = argmax_v x[r, v] with numpy semantics (lowest index on ties, the
// first NaN wins over everything, -0 == +0), optionally with the maximum as FP32.
//
// At decode row counts the op is latency, not bandwidth: a row of 151936 BF16 logits is 304 KB that is
// already in L2.  The kernel is built around that.
//   * One cluster of up to eight CTAs per row; a CTA issues all the 16-byte loads of its share of the row at
//     once (a scalar head and tail keep the vector body for odd vocabularies and unaligned rows), so a row
//     costs one round trip to L2.
//   * Candidates travel as 64-bit keys whose unsigned maximum is the winner (argmax_key.cuh): a thread packs
//     its best pair once, a warp needs two redux.sync.max, warps meet in one shared-memory atomicMax.
//   * The CTAs of a cluster do not meet at a barrier at the end.  CTA 0 owns one mbarrier and one key slot
//     per peer; a peer stores its key into CTA 0's shared memory, arrives on the barrier with release
//     semantics at cluster scope, and exits; CTA 0 alone waits (bounded), folds and writes.  The one cluster
//     barrier that must precede a remote arrival (the mbarrier has to exist) is split: every CTA arrives
//     right after it has issued its loads and waits only when its own result is ready, so the barrier's
//     latency lies under the memory latency.
// No workspace, no global atomics; the result does not depend on the launch geometry.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <climits>

#include "argmax_key.cuh"
#include "qfg_internal.h"

namespace qfg {
namespace {

constexpr int kThreads = 512;   // 1024 threads per CTA measured slower at every row count
constexpr int kMaxCluster = 8;
constexpr int kPeerSpin = 1 << 24;  // bound of CTA 0's wait for its peers (iterations of about 30 ns)

__device__ __forceinline__ float ToFloat(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float ToFloat(__half v) { return __half2float(v); }
__device__ __forceinline__ float ToFloat(float v) { return v; }

__device__ __forceinline__ uint32_t SharedAddr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

// A thread's running best.  `InOrder`: the candidate's index exceeds every index this thread has seen, so a
// strict comparison keeps the lowest index of equal values and a NaN is never replaced; `Any`: full order.
struct Best {
  float v = 0.f;
  long long i = -1;
  __device__ __forceinline__ void InOrder(float c, long long idx) {
    if (i < 0 || c > v || (c != c && v == v)) {
      v = c;
      i = idx;
    }
  }
  __device__ __forceinline__ void Any(float c, long long idx) {
    const bool c_nan = c != c, v_nan = v != v;
    const bool better = c_nan ? (!v_nan || idx < i) : (!v_nan && (c > v || (c == v && idx < i)));
    if (i < 0 || better) {
      v = c;
      i = idx;
    }
  }
  __device__ __forceinline__ unsigned long long Key() const { return i < 0 ? 0ull : PackKey(v, i); }
};

template <typename T>
__global__ void __launch_bounds__(kThreads) ArgmaxRowsKernel(const T* __restrict__ x, long long V,
                                                             long long* __restrict__ idx_out,
                                                             float* __restrict__ val_out) {
  constexpr int kVecElems = 16 / sizeof(T);
  constexpr int kInFlight = sizeof(T) == 4 ? 10 : 6;  // 8 CTAs x 512 threads x 6 (10) loads cover 151936 columns
  __shared__ unsigned long long s_best;               // this CTA's best key
  __shared__ unsigned long long s_slot[kMaxCluster];  // CTA 0: the peers' keys
  __shared__ unsigned long long s_bar;                // CTA 0: mbarrier, one arrival per peer

  const int C = static_cast<int>(gridDim.x);  // the cluster spans the grid's x extent
  const int c = static_cast<int>(blockIdx.x);
  const long long row = blockIdx.y;
  const T* xr = x + row * V;
  const int tid = threadIdx.x, lane = tid & 31;

  // Row layout: `head` scalar elements up to the first 16-byte boundary, `nvec` vectors, a scalar tail;
  // the vectors are split evenly over the CTAs of the cluster.
  const uintptr_t addr = reinterpret_cast<uintptr_t>(xr);
  long long head = ((16 - (addr & 15)) & 15) / sizeof(T);
  if (head > V) head = V;
  const long long nvec = (V - head) / kVecElems;
  const long long per = (nvec + C - 1) / C;
  const long long vbeg = min(nvec, per * c), vend = min(nvec, vbeg + per);
  const uint4* xv = reinterpret_cast<const uint4*>(xr + head);

  // ---- the first batch of loads goes out before anything else
  uint4 q[kInFlight];
  long long v0 = vbeg + tid;
#pragma unroll
  for (int k = 0; k < kInFlight; ++k) {
    const long long v = v0 + static_cast<long long>(k) * kThreads;
    q[k] = v < vend ? __ldg(xv + v) : make_uint4(0, 0, 0, 0);
  }
  if (tid == 0) {
    s_best = 0ull;
    if (c == 0 && C > 1) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(SharedAddr(&s_bar)), "r"(C - 1) : "memory");
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
  }
  __syncthreads();
  if (C > 1) asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");

  Best best;
  for (;;) {
#pragma unroll
    for (int k = 0; k < kInFlight; ++k) {
      const long long v = v0 + static_cast<long long>(k) * kThreads;
      if (v < vend) {
        const T* e = reinterpret_cast<const T*>(&q[k]);
#pragma unroll
        for (int j = 0; j < kVecElems; ++j) best.InOrder(ToFloat(e[j]), head + v * kVecElems + j);
      }
    }
    v0 += static_cast<long long>(kThreads) * kInFlight;
    if (v0 >= vend) break;  // rows longer than one batch per thread take further round trips
#pragma unroll
    for (int k = 0; k < kInFlight; ++k) {
      const long long v = v0 + static_cast<long long>(k) * kThreads;
      q[k] = v < vend ? __ldg(xv + v) : make_uint4(0, 0, 0, 0);
    }
  }
  // head goes to the first CTA, tail to the last
  if (c == 0) {
    for (long long i = tid; i < head; i += kThreads) best.Any(ToFloat(xr[i]), i);
  }
  if (c == C - 1) {
    for (long long i = head + nvec * kVecElems + tid; i < V; i += kThreads) best.Any(ToFloat(xr[i]), i);
  }

  const unsigned long long wkey = WarpMaxKey(best.Key());
  if (lane == 0 && wkey != 0ull) atomicMax(&s_best, wkey);
  __syncthreads();

  // the key of a NaN carries no payload: a NaN winner's value is read back from the row, bit for bit
  auto write_out = [&](unsigned long long key, bool ok) {
    const long long i = KeyIndex(key);
    idx_out[row] = ok ? i : -1;
    if (val_out != nullptr) val_out[row] = (ok && (key >> 32) == 0xFFFFFFFFull) ? ToFloat(xr[i]) : KeyValue(key);
  };
  if (C == 1) {
    if (tid == 0) write_out(s_best, true);
    return;
  }
  // every CTA of the cluster has started (so CTA 0's mbarrier exists) before anybody arrives on it
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
  if (c != 0) {
    if (tid == 0) {
      uint32_t slot, bar;
      asm volatile("mapa.shared::cluster.u32 %0, %1, 0;" : "=r"(slot) : "r"(SharedAddr(&s_slot[c])));
      asm volatile("mapa.shared::cluster.u32 %0, %1, 0;" : "=r"(bar) : "r"(SharedAddr(&s_bar)));
      asm volatile("st.shared::cluster.u64 [%0], %1;" ::"r"(slot), "l"(s_best) : "memory");
      asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
    }
    return;  // nobody reads this CTA's shared memory: it may leave
  }
  if (tid < 32) {
    uint32_t done = 0;
    for (int spin = 0; spin < kPeerSpin && !done; ++spin) {
      asm volatile("{ .reg .pred p;\n mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], 0;\n selp.u32 %0, 1, 0, p;\n}"
                   : "=r"(done)
                   : "r"(SharedAddr(&s_bar))
                   : "memory");
    }
    unsigned long long key = 0ull;
    if (done) key = lane == 0 ? s_best : (lane < C ? s_slot[lane] : 0ull);
    key = WarpMaxKey(key);
    if (lane == 0) write_out(key, done != 0);  // a wait that ran out (a peer CTA never arrived) leaves an index no row can have
  }
}

template <typename T>
cudaError_t LaunchT(const T* x, int64_t rows, int64_t V, int64_t* idx, float* val, cudaStream_t s) {
  // enough CTAs per row that each thread sees a few vectors; at most the portable cluster size
  const long long vecs = V / (16 / static_cast<long long>(sizeof(T)));
  int cluster = 1;
  while (cluster < kMaxCluster && vecs > static_cast<long long>(cluster) * kThreads * 2) cluster *= 2;
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
  if (idx != nullptr) idx[row] = KeyIndex(best);
  if (val != nullptr) val[row] = KeyValue(best);
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
