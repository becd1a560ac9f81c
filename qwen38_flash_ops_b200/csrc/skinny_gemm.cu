// SkinnyGemm for B200 (sm_100a): y[M, N] = x[M, K] @ W[K, N] for M <= 8 rows, streaming W once.
//
// Structure of one CTA (wn x wk warps):
//   * it owns one column tile of one weight and one 1/cluster slice of K;
//   * all threads feed a multi-stage shared-memory ring with cp.async (16-byte pieces where the
//     rows allow it, 8- or 4-byte pieces otherwise), so the bytes in flight per SM are set by the
//     ring depth and not by registers;
//   * each warp consumes 16 weight rows x (64 or 128) columns per k-step: a thread reads four
//     rows of its 8/16 columns from the ring, turns them into k-paired 16-bit operands
//     (BF16: byte permute; FP8: byte permute + cvt.e4m3x2; NVFP4: nibble interleave +
//     cvt.e2m1x2 + one packed multiply by the E4M3 block scale) and issues m16n8k16 MMAs with
//     the weights as the 16-row operand and x (padded to 8 rows) as the 8-column operand.
//     Every weight and every product is exact; accumulation is FP32;
//   * partial sums are combined in a fixed order: across the wk warps through shared memory,
//     then across the CTAs of the cluster through distributed shared memory, then scaled by the
//     per-column w_scale, rounded once to BF16 and routed to the output that owns the column.
//
// The quantised modes run the MMA in FP16 (the only type cvt.e2m1x2 / cvt.e4m3x2 produce).  x is
// BF16, so each CTA rescales its K slice of every x row by a power of two that puts the row
// maximum in [2^14, 2^15) and converts it to FP16; if any element is not exactly representable
// (dynamic range above 2^28 inside one slice, infinities, NaNs) the CTA takes the BF16 path
// instead, which converts the dequantised weights to BF16 and multiplies by the unscaled x.
// Both paths feed the tensor core exact operands.
#include <cooperative_groups.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <climits>
#include <mutex>

#include "qfg_internal.h"

namespace qfg {
namespace {

namespace cg = cooperative_groups;

constexpr int kMaxThreads = 256;

// ------------------------------------------------------------------------------ PTX helpers
__device__ __forceinline__ uint32_t SmemAddr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void CpAsync16(uint32_t dst, const void* src, int bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void CpAsync8(uint32_t dst, const void* src, int bytes) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void CpAsync4(uint32_t dst, const void* src, int bytes) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void CpAsyncCommit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void CpAsyncWait(int pending) {
  switch (pending) {
    case 0: asm volatile("cp.async.wait_group 0;" ::: "memory"); break;
    case 1: asm volatile("cp.async.wait_group 1;" ::: "memory"); break;
    case 2: asm volatile("cp.async.wait_group 2;" ::: "memory"); break;
    case 3: asm volatile("cp.async.wait_group 3;" ::: "memory"); break;
    case 4: asm volatile("cp.async.wait_group 4;" ::: "memory"); break;
    case 5: asm volatile("cp.async.wait_group 5;" ::: "memory"); break;
    case 6: asm volatile("cp.async.wait_group 6;" ::: "memory"); break;
    default: asm volatile("cp.async.wait_group 7;" ::: "memory"); break;
  }
}
__device__ __forceinline__ uint4 Lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint2 Lds64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint32_t Lds8(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint32_t Prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}
// Four E2M1 pairs (one per byte, low nibble -> low half) to four f16x2 registers.
__device__ __forceinline__ void CvtE2m1x8(uint32_t c, uint32_t (&r)[4]) {
  asm("{ .reg .b8 b0, b1, b2, b3;\n"
      " mov.b32 {b0, b1, b2, b3}, %4;\n"
      " cvt.rn.f16x2.e2m1x2 %0, b0;\n"
      " cvt.rn.f16x2.e2m1x2 %1, b1;\n"
      " cvt.rn.f16x2.e2m1x2 %2, b2;\n"
      " cvt.rn.f16x2.e2m1x2 %3, b3;\n}"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
      : "r"(c));
}
// Two E4M3 pairs (low 16 bits, high 16 bits) to two f16x2 registers.
__device__ __forceinline__ void CvtE4m3x4(uint32_t c, uint32_t& lo, uint32_t& hi) {
  asm("{ .reg .b16 h0, h1;\n"
      " mov.b32 {h0, h1}, %2;\n"
      " cvt.rn.f16x2.e4m3x2 %0, h0;\n"
      " cvt.rn.f16x2.e4m3x2 %1, h1;\n}"
      : "=r"(lo), "=r"(hi)
      : "r"(c));
}
__device__ __forceinline__ uint32_t CvtE4m3x2(uint32_t pair16) {
  uint32_t r;
  asm("{ .reg .b16 h0;\n cvt.u16.u32 h0, %1;\n cvt.rn.f16x2.e4m3x2 %0, h0;\n}" : "=r"(r) : "r"(pair16));
  return r;
}
__device__ __forceinline__ uint32_t Hmul2(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
// An exact f16x2 value as bf16x2 (the values here have at most 6 significant bits).
__device__ __forceinline__ uint32_t HalfPairToBf16Pair(uint32_t h) {
  const __half2 hv = *reinterpret_cast<const __half2*>(&h);
  const float2 f = __half22float2(hv);
  const __nv_bfloat162 b = __floats2bfloat162_rn(f.x, f.y);
  return *reinterpret_cast<const uint32_t*>(&b);
}
template <bool BF16>
__device__ __forceinline__ void Mma(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                    uint32_t b1) {
  if constexpr (BF16) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  } else {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
}
__device__ __forceinline__ void GridLaunchDependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void GridDependencyWait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ int CeilLog2(int v) { return v <= 1 ? 0 : 32 - __clz(v - 1); }

// (value, index) order of ArgmaxRows: NaN beats non-NaN, then larger value, then lower index.
__device__ __forceinline__ bool Better(float av, long long ai, float bv, long long bi) {
  if (av != av) return (bv == bv) || ai < bi;
  if (bv != bv) return false;
  return av > bv || (av == bv && ai < bi);
}
// A 64-bit word whose unsigned order is the Better order; every real candidate maps above 0.
__device__ __forceinline__ unsigned long long PackKey(float v, long long idx) {
  uint32_t ord;
  if (v != v) {
    ord = 0xFFFFFFFFu;
  } else {
    const uint32_t b = (v == 0.f) ? 0u : __float_as_uint(v);
    ord = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
  }
  return (static_cast<unsigned long long>(ord) << 32) | (0xFFFFFFFFu - static_cast<uint32_t>(idx));
}

template <int MODE>
struct Geom;
template <>
struct Geom<kBf16> {
  static constexpr int kColsPerThread = 8, kBytesPerThread = 16, kMmas = 4;
};
template <>
struct Geom<kFp8> {
  static constexpr int kColsPerThread = 16, kBytesPerThread = 16, kMmas = 8;
};
template <>
struct Geom<kNvfp4> {
  static constexpr int kColsPerThread = 16, kBytesPerThread = 8, kMmas = 8;
};

// One k-step of one warp: 16 weight rows x the warp's columns.  `w_addr` is the shared-memory
// address of this thread's bytes in row t of the step (rows t+4, t+8, t+12 follow at
// 4 * row_bytes), `s_addr` the address of its NVFP4 scale byte in row t.
template <int MODE, bool SLOW>
__device__ __forceinline__ void KStep(float (&acc)[Geom<MODE>::kMmas][4], uint32_t w_addr, uint32_t row4_bytes,
                                      uint32_t s_addr, uint32_t srow4_bytes, uint32_t b0, uint32_t b1) {
  constexpr bool kBf16Mma = (MODE == kBf16) || SLOW;
  if constexpr (MODE == kBf16) {
    const uint4 ra = Lds128(w_addr), rb = Lds128(w_addr + row4_bytes), rc = Lds128(w_addr + 2 * row4_bytes),
                rd = Lds128(w_addr + 3 * row4_bytes);
    const uint32_t a[4] = {ra.x, ra.y, ra.z, ra.w}, b[4] = {rb.x, rb.y, rb.z, rb.w};
    const uint32_t c[4] = {rc.x, rc.y, rc.z, rc.w}, d[4] = {rd.x, rd.y, rd.z, rd.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      Mma<true>(acc[i], Prmt(a[i], b[i], 0x5410u), Prmt(a[i], b[i], 0x7632u), Prmt(c[i], d[i], 0x5410u),
                Prmt(c[i], d[i], 0x7632u), b0, b1);
    }
  } else if constexpr (MODE == kFp8) {
    const uint4 ra = Lds128(w_addr), rb = Lds128(w_addr + row4_bytes), rc = Lds128(w_addr + 2 * row4_bytes),
                rd = Lds128(w_addr + 3 * row4_bytes);
    const uint32_t a[4] = {ra.x, ra.y, ra.z, ra.w}, b[4] = {rb.x, rb.y, rb.z, rb.w};
    const uint32_t c[4] = {rc.x, rc.y, rc.z, rc.w}, d[4] = {rd.x, rd.y, rd.z, rd.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint32_t p[4], q[4];
      CvtE4m3x4(Prmt(a[i], b[i], 0x5140u), p[0], p[1]);
      CvtE4m3x4(Prmt(a[i], b[i], 0x7362u), p[2], p[3]);
      CvtE4m3x4(Prmt(c[i], d[i], 0x5140u), q[0], q[1]);
      CvtE4m3x4(Prmt(c[i], d[i], 0x7362u), q[2], q[3]);
      if constexpr (SLOW) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          p[e] = HalfPairToBf16Pair(p[e]);
          q[e] = HalfPairToBf16Pair(q[e]);
        }
      }
      Mma<kBf16Mma>(acc[2 * i], p[0], p[1], q[0], q[1], b0, b1);
      Mma<kBf16Mma>(acc[2 * i + 1], p[2], p[3], q[2], q[3], b0, b1);
    }
  } else {
    const uint2 ra = Lds64(w_addr), rb = Lds64(w_addr + row4_bytes), rc = Lds64(w_addr + 2 * row4_bytes),
                rd = Lds64(w_addr + 3 * row4_bytes);
    const uint32_t sa = Lds8(s_addr), sb = Lds8(s_addr + srow4_bytes), sc = Lds8(s_addr + 2 * srow4_bytes),
                   sd = Lds8(s_addr + 3 * srow4_bytes);
    const uint32_t s_ab = CvtE4m3x2(sa | (sb << 8)), s_cd = CvtE4m3x2(sc | (sd << 8));
    const uint32_t a[2] = {ra.x, ra.y}, b[2] = {rb.x, rb.y}, c[2] = {rc.x, rc.y}, d[2] = {rd.x, rd.y};
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      // byte q of `even`: (row A nibble, row B nibble) of column 8i + 2q; of `odd`: column 8i + 2q + 1
      uint32_t e_ab[4], o_ab[4], e_cd[4], o_cd[4];
      CvtE2m1x8((a[i] & 0x0F0F0F0Fu) | ((b[i] << 4) & 0xF0F0F0F0u), e_ab);
      CvtE2m1x8(((a[i] >> 4) & 0x0F0F0F0Fu) | (b[i] & 0xF0F0F0F0u), o_ab);
      CvtE2m1x8((c[i] & 0x0F0F0F0Fu) | ((d[i] << 4) & 0xF0F0F0F0u), e_cd);
      CvtE2m1x8(((c[i] >> 4) & 0x0F0F0F0Fu) | (d[i] & 0xF0F0F0F0u), o_cd);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint32_t a0 = Hmul2(e_ab[q], s_ab), a1 = Hmul2(o_ab[q], s_ab);
        uint32_t a2 = Hmul2(e_cd[q], s_cd), a3 = Hmul2(o_cd[q], s_cd);
        if constexpr (SLOW) {
          a0 = HalfPairToBf16Pair(a0);
          a1 = HalfPairToBf16Pair(a1);
          a2 = HalfPairToBf16Pair(a2);
          a3 = HalfPairToBf16Pair(a3);
        }
        Mma<kBf16Mma>(acc[4 * i + q], a0, a1, a2, a3, b0, b1);
      }
    }
  }
}

template <int MODE>
__global__ void __launch_bounds__(kMaxThreads, 2) SkinnyGemmKernel(const GemmParams p) {
  using G = Geom<MODE>;
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ float s_inv_scale[kMaxRows];
  __shared__ uint32_t s_amax[kMaxThreads / 32][kMaxRows];
  __shared__ float s_best_v[kMaxThreads / 32][kMaxRows];
  __shared__ long long s_best_i[kMaxThreads / 32][kMaxRows];
  __shared__ int s_last;

  if (p.trigger == 1) GridLaunchDependents();

  const int tid = threadIdx.x;
  const int nthreads = blockDim.x;
  const int warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int wn = warp % p.wn, wk = warp / p.wn;
  const int M = p.M;

  // ---- which tile of which weight
  int s = 0;
#pragma unroll
  for (int i = 1; i < kMaxSeg; ++i) s += (i < p.nseg && static_cast<int>(blockIdx.x) >= p.seg[i].tile_begin) ? 1 : 0;
  const Segment& sg = p.seg[s];
  const int N = sg.n;
  const int tl = static_cast<int>(blockIdx.x) - sg.tile_begin;
  const int n0 = static_cast<int>(static_cast<long long>(tl) * sg.granules / sg.tiles) * p.gran;
  const int n1 = min(N, static_cast<int>(static_cast<long long>(tl + 1) * sg.granules / sg.tiles) * p.gran);
  const long long pitch = sg.pitch;

  // ---- which slice of K
  const int C = static_cast<int>(gridDim.y);
  const int crank = static_cast<int>(blockIdx.y);
  const int ksteps_total = (p.K + 15) >> 4;
  const int kbeg = static_cast<int>(static_cast<long long>(crank) * ksteps_total / C) * 16;
  const int kend = min(p.K, static_cast<int>(static_cast<long long>(crank + 1) * ksteps_total / C) * 16);
  const int kslice = max(0, kend - kbeg);
  const int R = 16 * p.wk * p.ks;
  const int nst = (kslice + R - 1) / R;

  const int TB = p.tile_row_bytes;
  const int SRB = p.scale_row_bytes;
  const uint32_t ring = SmemAddr(smem);
  const uint32_t swz_mask = static_cast<uint32_t>((TB / 16 - 1) & 6);

  // ---- producer geometry: weight bytes
  const int vec = sg.vec;
  const int ppr = TB / vec;
  const int lgp = CeilLog2(ppr);
  const int valid_row_bytes = (MODE == kBf16) ? (n1 - n0) * 2 : (MODE == kFp8) ? (n1 - n0) : (n1 - n0) / 2;
  const long long col_byte0 = (MODE == kBf16) ? static_cast<long long>(n0) * 2 : (MODE == kFp8) ? n0 : n0 / 2;
  const uint8_t* wbase = sg.w + col_byte0;
  // ---- producer geometry: NVFP4 scale bytes (an aligned superset of the tile's scale bytes)
  int svec = 4, sphase = 0, spps = 0, lgs = 0;
  long long srow_off = 0;
  if constexpr (MODE == kNvfp4) {
    svec = sg.svec;
    const long long soff = (N >> 1) + (n0 >> 4);
    srow_off = soff / svec * svec;
    sphase = static_cast<int>(soff - srow_off);
    spps = (sphase + ((n1 - n0) >> 4) + svec - 1) / svec;
    lgs = CeilLog2(spps);
  }

  auto issue_stage = [&](int stage) {
    const uint32_t slot = ring + static_cast<uint32_t>(stage % p.stages) * p.stage_bytes;
    const int row_base = kbeg + stage * R;
    {
      const int total = R << lgp;
      for (int i = tid; i < total; i += nthreads) {
        const int row = i >> lgp;
        const int c = i & ((1 << lgp) - 1);
        if (c >= ppr) continue;
        const int bo = c * vec;
        int bytes = min(vec, max(0, valid_row_bytes - bo));
        const int krow = row_base + row;
        if (krow >= kend) bytes = 0;
        const uint8_t* src = bytes > 0 ? wbase + static_cast<long long>(krow) * pitch + bo : sg.w;
        const uint32_t dst = slot + row * TB + ((((bo >> 4) ^ ((row & 3) << 1 & swz_mask)) << 4) | (bo & 15));
        if (vec == 16) {
          CpAsync16(dst, src, bytes);
        } else if (vec == 8) {
          CpAsync8(dst, src, bytes);
        } else {
          CpAsync4(dst, src, bytes);
        }
      }
    }
    if constexpr (MODE == kNvfp4) {
      const uint32_t sslot = slot + R * TB;
      const int total = R << lgs;
      for (int i = tid; i < total; i += nthreads) {
        const int row = i >> lgs;
        const int c = i & ((1 << lgs) - 1);
        if (c >= spps) continue;
        const int krow = row_base + row;
        const long long pos = static_cast<long long>(krow) * pitch + srow_off + c * svec;
        int bytes = krow < kend ? static_cast<int>(min(static_cast<long long>(svec), sg.total_bytes - pos)) : 0;
        bytes = max(bytes, 0);
        const uint8_t* src = bytes > 0 ? sg.w + pos : sg.w;
        const uint32_t dst = sslot + row * SRB + c * svec;
        if (svec == 16) {
          CpAsync16(dst, src, bytes);
        } else if (svec == 8) {
          CpAsync8(dst, src, bytes);
        } else {
          CpAsync4(dst, src, bytes);
        }
      }
    }
  };

  // ---- prologue: fill the ring, then stage x while the first weights are in flight
  for (int st = 0; st < p.stages - 1; ++st) {
    if (st < nst) issue_stage(st);
    CpAsyncCommit();
  }
  if (p.pdl_wait) GridDependencyWait();

  const int kpad = (kslice + 15) & ~15;
  uint16_t* xs = reinterpret_cast<uint16_t*>(smem + p.ring_bytes);
  const int xpitch = p.xpitch;
  bool slow = false;
  {
    // Raw BF16 copy in the k-permuted order the B fragments read: position 4t+i of a 16-block
    // holds row t+4i.  K is even and slices start on multiples of 16, so pairs never straddle.
    uint32_t amax[kMaxRows];
#pragma unroll
    for (int m = 0; m < kMaxRows; ++m) amax[m] = 0;
    const int npairs = kpad >> 1;
#pragma unroll
    for (int m = 0; m < kMaxRows; ++m) {
      if (m < M) {
        const uint32_t* xr = reinterpret_cast<const uint32_t*>(p.x + static_cast<size_t>(m) * p.K + kbeg);
        for (int pp = tid; pp < npairs; pp += nthreads) {
          const int kk = pp * 2;
          const uint32_t v2 = kk < kslice ? __ldg(xr + pp) : 0u;
          const uint32_t lo = v2 & 0xFFFFu, hi = v2 >> 16;
          const int r16 = kk & 15;
          const int base = m * xpitch + (kk & ~15);
          xs[base + ((r16 & 3) << 2) + (r16 >> 2)] = static_cast<uint16_t>(lo);
          xs[base + (((r16 + 1) & 3) << 2) + ((r16 + 1) >> 2)] = static_cast<uint16_t>(hi);
          amax[m] = max(amax[m], max(lo & 0x7FFFu, hi & 0x7FFFu));
        }
      }
    }
    if constexpr (MODE == kBf16) {
      if (tid < kMaxRows) s_inv_scale[tid] = 1.f;
      __syncthreads();
    } else {
#pragma unroll
      for (int m = 0; m < kMaxRows; ++m) {
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) amax[m] = max(amax[m], __shfl_xor_sync(0xffffffffu, amax[m], off));
        if (lane == 0) s_amax[warp][m] = amax[m];
      }
      __syncthreads();
      // Power-of-two scale per row that puts the slice maximum in [2^14, 2^15); then convert in place.
      bool ok = !p.force_slow;
      const int nwarps = nthreads >> 5;
      float inv_scale[kMaxRows];
#pragma unroll
      for (int m = 0; m < kMaxRows; ++m) {
        inv_scale[m] = 1.f;
        if (m < M) {
          uint32_t a = 0;
          for (int w = 0; w < nwarps; ++w) a = max(a, s_amax[w][m]);
          const int e = static_cast<int>(a >> 7);  // BF16 exponent field of the row maximum
          float sc = 1.f;
          if (a != 0) {
            if (e < 32 || e >= 255) {
              ok = false;
            } else {
              sc = __uint_as_float(static_cast<uint32_t>(268 - e) << 23);
            }
          }
          const float inv = 1.f / sc;
          inv_scale[m] = inv;
          for (int kk = tid; kk < kpad; kk += nthreads) {
            uint16_t* px = &xs[m * xpitch + kk];
            const float xf = __uint_as_float(static_cast<uint32_t>(*px) << 16);
            const float v = xf * sc;
            const __half h = __float2half_rn(v);
            ok = ok && (__half2float(h) == v) && (v == 0.f || fabsf(v) >= 6.103515625e-05f) && (v * inv == xf);
            *px = __half_as_ushort(h);
          }
        }
      }
      slow = !__syncthreads_and(ok ? 1 : 0);
      if (slow) {
        // Not exactly representable: put the BF16 values back and use the BF16 MMA.
#pragma unroll
        for (int m = 0; m < kMaxRows; ++m) {
          if (m < M) {
            const uint32_t* xr = reinterpret_cast<const uint32_t*>(p.x + static_cast<size_t>(m) * p.K + kbeg);
            for (int pp = tid; pp < npairs; pp += nthreads) {
              const int kk = pp * 2;
              const uint32_t v2 = kk < kslice ? __ldg(xr + pp) : 0u;
              const int r16 = kk & 15;
              const int base = m * xpitch + (kk & ~15);
              xs[base + ((r16 & 3) << 2) + (r16 >> 2)] = static_cast<uint16_t>(v2 & 0xFFFFu);
              xs[base + (((r16 + 1) & 3) << 2) + ((r16 + 1) >> 2)] = static_cast<uint16_t>(v2 >> 16);
            }
          }
        }
      }
      if (tid == 0) {
#pragma unroll
        for (int m = 0; m < kMaxRows; ++m) s_inv_scale[m] = slow ? 1.f : inv_scale[m];
      }
      __syncthreads();
    }
  }

  // ---- consumer geometry
  constexpr int NM = G::kMmas;
  float acc[NM][4];
#pragma unroll
  for (int j = 0; j < NM; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[j][e] = 0.f;

  const int cols_per_warp = 8 * G::kColsPerThread;
  const bool warp_has_cols = n0 + wn * cols_per_warp < n1;
  uint32_t w_off, s_off = 0;
  if constexpr (MODE == kNvfp4) {
    const uint32_t chunk = static_cast<uint32_t>(wn * 4 + (g >> 1));
    w_off = t * TB + (((chunk ^ ((t << 1) & swz_mask)) << 4) | ((g & 1) << 3));
    s_off = static_cast<uint32_t>(R * TB + t * SRB + sphase + wn * 8 + g);
  } else {
    const uint32_t chunk = static_cast<uint32_t>(wn * 8 + g);
    w_off = t * TB + ((chunk ^ ((t << 1) & swz_mask)) << 4);
  }
  const uint32_t xs_addr = SmemAddr(xs) + static_cast<uint32_t>((g * xpitch + 4 * t) * 2);
  const bool has_row = g < M;

  for (int it = 0; it < nst; ++it) {
    CpAsyncWait(p.stages - 2);
    __syncthreads();
    const int nxt = it + p.stages - 1;
    if (nxt < nst) issue_stage(nxt);
    CpAsyncCommit();
    if (warp_has_cols) {
      const uint32_t slot = ring + static_cast<uint32_t>(it % p.stages) * p.stage_bytes;
      for (int q = 0; q < p.ks; ++q) {
        const int step_in_stage = q * p.wk + wk;
        const int kstep = it * (p.wk * p.ks) + step_in_stage;
        if (kstep * 16 >= kslice) break;
        uint32_t b0 = 0, b1 = 0;
        if (has_row) {
          const uint2 xv = Lds64(xs_addr + static_cast<uint32_t>(kstep) * 32u);
          b0 = xv.x;
          b1 = xv.y;
        }
        const uint32_t wa = slot + static_cast<uint32_t>(step_in_stage * 16) * TB + w_off;
        const uint32_t sa = slot + static_cast<uint32_t>(step_in_stage * 16) * SRB + s_off;
        if constexpr (MODE == kBf16) {
          KStep<MODE, false>(acc, wa, 4u * TB, sa, 4u * SRB, b0, b1);
        } else {
          if (slow) {
            KStep<MODE, true>(acc, wa, 4u * TB, sa, 4u * SRB, b0, b1);
          } else {
            KStep<MODE, false>(acc, wa, 4u * TB, sa, 4u * SRB, b0, b1);
          }
        }
      }
    }
  }
  CpAsyncWait(0);
  if (p.trigger == 2) GridLaunchDependents();
  __syncthreads();

  // ---- reduction across the wk warps (fixed order), rows scaled back by 2^e
  const int TNc = p.wn * cols_per_warp;
  float* red = reinterpret_cast<float*>(smem);
  float* part = red + static_cast<size_t>(p.wk) * M * TNc;
  if (warp_has_cols) {
#pragma unroll
    for (int j = 0; j < NM; ++j) {
      const int cl = wn * cols_per_warp + g * G::kColsPerThread + 2 * j;
      const int m0 = 2 * t, m1 = 2 * t + 1;
      if (m0 < M) *reinterpret_cast<float2*>(&red[(wk * M + m0) * TNc + cl]) = make_float2(acc[j][0], acc[j][2]);
      if (m1 < M) *reinterpret_cast<float2*>(&red[(wk * M + m1) * TNc + cl]) = make_float2(acc[j][1], acc[j][3]);
    }
  } else {
    // warps beyond the tile's last column contribute zeros
    for (int m = 0; m < M; ++m)
      for (int c = lane; c < cols_per_warp; c += 32) red[(wk * M + m) * TNc + wn * cols_per_warp + c] = 0.f;
  }
  __syncthreads();

  const int ncols = n1 - n0;  // valid columns of the tile (<= TNc)
  float best_v[kMaxRows];
  long long best_i[kMaxRows];
#pragma unroll
  for (int m = 0; m < kMaxRows; ++m) {
    best_v[m] = 0.f;
    best_i[m] = -1;
  }
  auto finalize = [&](int m, int c, float v) {
    const int n = n0 + c;
    if (sg.w_scale != nullptr) v *= sg.w_scale[n];
    const __nv_bfloat16 b = __float2bfloat16(v);
    if (!p.lm || p.out[sg.out_begin] != nullptr) {
      int j = sg.out_begin;
      for (int i = j + 1; i < sg.out_end; ++i) {
        if (n >= p.col_begin[i]) j = i;
      }
      p.out[j][static_cast<size_t>(m) * p.width[j] + (n - p.col_begin[j])] = __bfloat16_as_ushort(b);
    }
    if (p.lm) {
      const float f = __bfloat162float(b);
#pragma unroll
      for (int r = 0; r < kMaxRows; ++r) {
        if (r == m && (best_i[r] < 0 || f > best_v[r] || (f != f && best_v[r] == best_v[r]))) {
          best_v[r] = f;
          best_i[r] = p.lm_col_offset + n;
        }
      }
    }
  };

  if (C == 1) {
    for (int m = 0; m < M; ++m) {
      const float inv = s_inv_scale[m];
      for (int c = tid; c < ncols; c += nthreads) {
        float sum = 0.f;
        for (int w = 0; w < p.wk; ++w) sum += red[(w * M + m) * TNc + c];
        finalize(m, c, sum * inv);
      }
    }
  } else {
    for (int m = 0; m < M; ++m) {
      const float inv = s_inv_scale[m];
      for (int c = tid; c < TNc; c += nthreads) {
        float sum = 0.f;
        for (int w = 0; w < p.wk; ++w) sum += red[(w * M + m) * TNc + c];
        part[m * TNc + c] = sum * inv;
      }
    }
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();
    const int cper = TNc / C;  // TNc is a multiple of 64 and C <= 8
    const int cb = crank * cper;
    for (int m = 0; m < M; ++m) {
      for (int cc = tid; cc < cper; cc += nthreads) {
        const int c = cb + cc;
        if (c >= ncols) break;
        float sum = 0.f;
        for (int r = 0; r < C; ++r) sum += cluster.map_shared_rank(part, r)[m * TNc + c];
        finalize(m, c, sum);
      }
    }
    cluster.sync();
  }

  if (p.lm) {
    // CTA-level (max, index) per row, folded into the workspace keys with a 64-bit atomic max.
    __syncthreads();
#pragma unroll
    for (int m = 0; m < kMaxRows; ++m) {
      if (m < M) {
        float v = best_i[m] < 0 ? -INFINITY : best_v[m];
        long long i = best_i[m] < 0 ? LLONG_MAX : best_i[m];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
          const float ov = __shfl_xor_sync(0xffffffffu, v, off);
          const long long oi = __shfl_xor_sync(0xffffffffu, i, off);
          if (Better(ov, oi, v, i)) {
            v = ov;
            i = oi;
          }
        }
        if (lane == 0) {
          s_best_v[warp][m] = v;
          s_best_i[warp][m] = i;
        }
      }
    }
    __syncthreads();
    if (tid < M) {
      float v = s_best_v[0][tid];
      long long i = s_best_i[0][tid];
      for (int w = 1; w < (nthreads >> 5); ++w) {
        if (Better(s_best_v[w][tid], s_best_i[w][tid], v, i)) {
          v = s_best_v[w][tid];
          i = s_best_i[w][tid];
        }
      }
      if (i != LLONG_MAX) atomicMax(p.lm_keys + tid, PackKey(v, i));
      __threadfence();
    }
    __syncthreads();
    if (tid == 0) {
      const unsigned int total = gridDim.x * gridDim.y;
      const unsigned int prev = atomicAdd(p.lm_count, 1u);
      s_last = (prev == total - 1) ? 1 : 0;
      __threadfence();
    }
    __syncthreads();
    if (s_last) {
      if (tid < M) {
        const unsigned long long key = atomicExch(p.lm_keys + tid, 0ull);
        const uint32_t ord = static_cast<uint32_t>(key >> 32);
        const uint32_t bits = (ord == 0xFFFFFFFFu) ? 0x7FC00000u : ((ord & 0x80000000u) ? (ord & 0x7FFFFFFFu) : ~ord);
        if (p.lm_idx != nullptr) p.lm_idx[tid] = static_cast<long long>(0xFFFFFFFFu - static_cast<uint32_t>(key));
        if (p.lm_val != nullptr) p.lm_val[tid] = __uint_as_float(bits);
        if (p.lm_key_out != nullptr) p.lm_key_out[tid] = key;
      }
      if (tid == 0) *p.lm_count = 0u;
    }
  }
}

// Largest dynamic shared-memory request any of the kernels accepts: the opt-in limit of the
// device minus the kernel's static shared memory.
int g_max_dynamic_smem = 0;

template <int MODE>
cudaError_t ConfigureKernel() {
  int dev = 0, optin = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return err;
  err = cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
  if (err != cudaSuccess) return err;
  cudaFuncAttributes fa;
  err = cudaFuncGetAttributes(&fa, SkinnyGemmKernel<MODE>);
  if (err != cudaSuccess) return err;
  const int dyn = optin - static_cast<int>(fa.sharedSizeBytes);
  if (g_max_dynamic_smem == 0 || dyn < g_max_dynamic_smem) g_max_dynamic_smem = dyn;
  return cudaFuncSetAttribute(SkinnyGemmKernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, dyn);
}

template <int MODE>
cudaError_t LaunchMode(const GemmParams& p, const Plan& plan, size_t smem, cudaStream_t stream) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(p.seg[p.nseg - 1].tile_begin + p.seg[p.nseg - 1].tiles),
                     static_cast<unsigned>(plan.cluster), 1);
  cfg.blockDim = dim3(static_cast<unsigned>(plan.threads()), 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n_attr = 0;
  if (plan.cluster > 1) {
    attr[n_attr].id = cudaLaunchAttributeClusterDimension;
    attr[n_attr].val.clusterDim.x = 1;
    attr[n_attr].val.clusterDim.y = static_cast<unsigned>(plan.cluster);
    attr[n_attr].val.clusterDim.z = 1;
    ++n_attr;
  }
  if (p.pdl_wait) {
    attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
    ++n_attr;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n_attr;
  return cudaLaunchKernelEx(&cfg, SkinnyGemmKernel<MODE>, p);
}

}  // namespace

int DeviceSmCount() {
  static int count = [] {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) return 148;
    return n;
  }();
  return count;
}

// Raises the dynamic shared-memory limit of the three kernels once per process.  Called from the
// *_create entry points, i.e. outside any stream capture.
cudaError_t ConfigureSkinnyGemmKernels() {
  static std::once_flag once;
  static cudaError_t status = cudaSuccess;
  std::call_once(once, [] {
    status = ConfigureKernel<kBf16>();
    if (status == cudaSuccess) status = ConfigureKernel<kFp8>();
    if (status == cudaSuccess) status = ConfigureKernel<kNvfp4>();
  });
  return status;
}

cudaError_t LaunchSkinnyGemm(int mode, GemmParams& p, const Plan& plan, cudaStream_t stream) {
  const ModeGeom geom = GeomOf(mode);
  p.wn = plan.wn;
  p.wk = plan.wk;
  p.ks = plan.ks;
  p.stages = plan.stages;
  p.cluster = plan.cluster;
  p.gran = plan.gran;
  p.tile_row_bytes = plan.wn * geom.bytes_per_warp;
  p.scale_row_bytes = mode == kNvfp4 ? plan.wn * 8 + 16 : 0;
  const int R = plan.rows_per_stage();
  p.stage_bytes = (R * (p.tile_row_bytes + p.scale_row_bytes) + 127) & ~127;
  const int TNc = plan.wn * geom.cols_per_warp;
  const int red_bytes = (plan.wk + (plan.cluster > 1 ? 1 : 0)) * p.M * TNc * 4;
  p.ring_bytes = (std::max(plan.stages * p.stage_bytes, red_bytes) + 127) & ~127;
  const int ksteps = (p.K + 15) / 16;
  const int kslice_max = ((ksteps + plan.cluster - 1) / plan.cluster) * 16;
  p.xpitch = ((kslice_max + 63) & ~63) + 16;  // 32 bytes off a 128-byte multiple: rows land in distinct banks
  const size_t smem = static_cast<size_t>(p.ring_bytes) + static_cast<size_t>(p.M) * p.xpitch * 2;
  if (g_max_dynamic_smem > 0 && smem > static_cast<size_t>(g_max_dynamic_smem)) return cudaErrorInvalidConfiguration;
  int tiles = 0;
  for (int s = 0; s < p.nseg; ++s) {
    p.seg[s].tile_begin = tiles;
    p.seg[s].tiles = plan.tiles[s];
    p.seg[s].granules = (p.seg[s].n + plan.gran - 1) / plan.gran;
    tiles += plan.tiles[s];
  }
  switch (mode) {
    case kBf16: return LaunchMode<kBf16>(p, plan, smem, stream);
    case kFp8: return LaunchMode<kFp8>(p, plan, smem, stream);
    case kNvfp4: return LaunchMode<kNvfp4>(p, plan, smem, stream);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace qfg
