// SkinnyGemm for B200 (sm_100a): y[M, N] = x[M, K] @ W[K, N] for M <= 8 rows, streaming W once.
//
// A CTA of wn x wk warps owns one column tile of one weight and one 1/cluster slice of K.  A warp
// consumes 16 weight rows x (64 or 128) columns per k-step: a thread holds four rows of its 8/16
// columns, turns them into k-paired 16-bit operands (BF16: byte permute; FP8: byte permute +
// cvt.e4m3x2; NVFP4: nibble interleave + cvt.e2m1x2 + one packed multiply by the E4M3 block
// scales) and issues m16n8k16 MMAs with the weights as the 16-row operand and x (padded to 8 rows)
// as the 8-column operand.  Every weight and every product is exact; accumulation is FP32.
//
// Two kernels share that arithmetic and differ in how the weight bytes reach the registers:
//   * SkinnyGemmDirectKernel (the fast path): every warp streams its own rows from HBM into a
//     warp-private shared-memory ring with lane-private cp.async copies, `depth` k-steps ahead of
//     the MMAs.  No CTA barrier in the K loop; the bytes in flight per SM are warps x depth x
//     1-2 KiB, bounded by shared memory rather than registers (a B200 needs well over 100 KiB in
//     flight per SM to stream at HBM speed).  Needs 16-byte aligned rows (8 for NVFP4) and whole
//     thread chunks.
//   * SkinnyGemmRingKernel (any 4-byte aligned layout, ragged column tails): all threads feed a
//     multi-stage shared-memory ring with cp.async pieces of 16, 8 or 4 bytes with zero fill.
//
// Partial sums are combined in a fixed order: across the wk warps through shared memory, then
// across the CTAs of the cluster through distributed shared memory, then scaled by the per-column
// w_scale, rounded once to BF16 and routed to the output that owns the column.  With `lm` set the
// epilogue also folds the BF16-rounded values into a per-row (max, index) key (fused LM head).
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
#include <map>
#include <mutex>
#include <tuple>
#include <type_traits>
#include <utility>

#include "argmax_key.cuh"
#include "qfg_internal.h"

namespace qfg {
namespace {

namespace cg = cooperative_groups;

constexpr int kMaxThreads = 32 * kMaxWarps;  // warp-ring and tcgen05 kernels (20 warps: at most 102 registers per thread)
constexpr int kRingThreads = 256;  // ring kernel: up to 8 warps

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
// shared-memory loads at a register address plus a compile-time offset (folded into the instruction)
template <int OFF>
__device__ __forceinline__ uint4 Lds128At(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4+%5];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr), "n"(OFF));
  return v;
}
template <int OFF>
__device__ __forceinline__ uint2 Lds64At(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2+%3];" : "=r"(v.x), "=r"(v.y) : "r"(addr), "n"(OFF));
  return v;
}
template <int OFF>
__device__ __forceinline__ uint32_t Lds8At(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u8 %0, [%1+%2];" : "=r"(v) : "r"(addr), "n"(OFF));
  return v;
}
// 16 bytes from `base + off` to shared memory at `dst + OFF`; CACHED keeps the line in L1 (.ca) for neighbours
template <int OFF, bool CACHED>
__device__ __forceinline__ void CpAsync16At(uint32_t dst, const uint8_t* base, uint32_t off) {
  if constexpr (CACHED) {
    asm volatile("{ .reg .u64 a;\n mad.wide.u32 a, %2, 1, %1;\n cp.async.ca.shared.global [%0+%3], [a], 16;\n}" ::"r"(dst), "l"(base),
                 "r"(off), "n"(OFF)
                 : "memory");
  } else {
    asm volatile("{ .reg .u64 a;\n mad.wide.u32 a, %2, 1, %1;\n cp.async.cg.shared.global [%0+%3], [a], 16;\n}" ::"r"(dst), "l"(base),
                 "r"(off), "n"(OFF)
                 : "memory");
  }
}
__device__ __forceinline__ uint4 Ldg128(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint2 Ldg64(const void* p) {
  uint2 v;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t Ldg8(const void* p) {
  uint32_t v;
  asm volatile("ld.global.nc.u8 %0, [%1];" : "=r"(v) : "l"(p));
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
// (a & mask) | (b & ~mask) in one instruction
__device__ __forceinline__ uint32_t BitSelect(uint32_t a, uint32_t b, uint32_t mask) {
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0xE4;" : "=r"(r) : "r"(a), "r"(b), "r"(mask));
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
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  } else {
    asm(
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
// W: 16-column groups a thread of the NVFP4 direct kernel owns.  With W = 2 a warp covers 256
// columns and thread group g owns groups g and g + 8 of them, i.e. two 8-byte runs 64 bytes
// apart in every row: fewer partly used sectors and less loop overhead per weight, and the
// 8-byte shared-memory reads stay aligned on rows that start 8 bytes off a 16-byte boundary.
template <int MODE, int W = 1>
struct Geom;
template <>
struct Geom<kBf16, 1> {
  static constexpr int kColsPerThread = 8, kBytesPerThread = 16, kMmas = 4;
};
template <>
struct Geom<kFp8, 1> {
  static constexpr int kColsPerThread = 16, kBytesPerThread = 16, kMmas = 8;
};
template <int W>
struct Geom<kNvfp4, W> {
  static constexpr int kColsPerThread = 16, kBytesPerThread = 8, kMmas = 8 * W;
};

// The raw bytes of one k-step of one thread: four consecutive weight rows (4t .. 4t+3 of the
// step) of its columns, plus the NVFP4 block-scale bytes of those rows (one byte per 16-column
// group).  The B fragment of the same thread is x[4t .. 4t+3] of the step: the k index of an MMA
// is a free permutation.
template <int MODE, int W = 1>
struct Raw {
  uint4 r[4];
};
template <int W>
struct Raw<kNvfp4, W> {
  uint2 r[W][4];
  uint32_t s[W][4];
};

// One k-step of one warp from registers: dequantise to k-paired operands and run the MMAs.
template <int MODE, bool SLOW, int W = 1>
__device__ __forceinline__ void ComputeStep(float (&acc)[Geom<MODE, W>::kMmas][4], const Raw<MODE, W>& w, uint32_t b0,
                                            uint32_t b1) {
  constexpr bool kBf16Mma = (MODE == kBf16) || SLOW;
  if constexpr (MODE == kBf16) {
    const uint32_t a[4] = {w.r[0].x, w.r[0].y, w.r[0].z, w.r[0].w}, b[4] = {w.r[1].x, w.r[1].y, w.r[1].z, w.r[1].w};
    const uint32_t c[4] = {w.r[2].x, w.r[2].y, w.r[2].z, w.r[2].w}, d[4] = {w.r[3].x, w.r[3].y, w.r[3].z, w.r[3].w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      Mma<true>(acc[i], Prmt(a[i], b[i], 0x5410u), Prmt(a[i], b[i], 0x7632u), Prmt(c[i], d[i], 0x5410u),
                Prmt(c[i], d[i], 0x7632u), b0, b1);
    }
  } else if constexpr (MODE == kFp8) {
    const uint32_t a[4] = {w.r[0].x, w.r[0].y, w.r[0].z, w.r[0].w}, b[4] = {w.r[1].x, w.r[1].y, w.r[1].z, w.r[1].w};
    const uint32_t c[4] = {w.r[2].x, w.r[2].y, w.r[2].z, w.r[2].w}, d[4] = {w.r[3].x, w.r[3].y, w.r[3].z, w.r[3].w};
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
#pragma unroll
    for (int h = 0; h < W; ++h) {
      const uint32_t s_ab = CvtE4m3x2(Prmt(w.s[h][0], w.s[h][1], 0x0040u));
      const uint32_t s_cd = CvtE4m3x2(Prmt(w.s[h][2], w.s[h][3], 0x0040u));
      const uint32_t a[2] = {w.r[h][0].x, w.r[h][0].y}, b[2] = {w.r[h][1].x, w.r[h][1].y};
      const uint32_t c[2] = {w.r[h][2].x, w.r[h][2].y}, d[2] = {w.r[h][3].x, w.r[h][3].y};
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        // byte q of `e_*`: (row A nibble, row B nibble) of column 8i + 2q; of `o_*`: column 8i + 2q + 1
        uint32_t e_ab[4], o_ab[4], e_cd[4], o_cd[4];
        CvtE2m1x8(BitSelect(a[i], b[i] << 4, 0x0F0F0F0Fu), e_ab);
        CvtE2m1x8(BitSelect(a[i] >> 4, b[i], 0x0F0F0F0Fu), o_ab);
        CvtE2m1x8(BitSelect(c[i], d[i] << 4, 0x0F0F0F0Fu), e_cd);
        CvtE2m1x8(BitSelect(c[i] >> 4, d[i], 0x0F0F0F0Fu), o_cd);
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
          Mma<kBf16Mma>(acc[8 * h + 4 * i + q], a0, a1, a2, a3, b0, b1);
        }
      }
    }
  }
}

// What a CTA works on: a column tile of one weight and a slice of K.
struct Tile {
  int seg, n0, n1, kbeg, kend, kslice, crank, C;
};

__device__ __forceinline__ Tile LocateTile(const GemmParams& p) {
  Tile tl;
  int s = 0;
#pragma unroll
  for (int i = 1; i < kMaxSeg; ++i) s += (i < p.nseg && static_cast<int>(blockIdx.x) >= p.seg[i].tile_begin) ? 1 : 0;
  tl.seg = s;
  const Segment& sg = p.seg[s];
  // tile t covers granules [t G / T, (t + 1) G / T): in 32 bits, from G = quot T + rem (a 64-bit division is
  // a hundred instructions, and this is the first thing every CTA does)
  const unsigned t = blockIdx.x - static_cast<unsigned>(sg.tile_begin), T = static_cast<unsigned>(sg.tiles);
  const unsigned g0 = t * sg.gran_quot + t * sg.gran_rem / T, g1 = (t + 1) * sg.gran_quot + (t + 1) * sg.gran_rem / T;
  tl.n0 = static_cast<int>(g0) * p.gran;
  tl.n1 = min(sg.n - sg.tail_cols, static_cast<int>(g1) * p.gran);
  tl.C = static_cast<int>(gridDim.y);
  tl.crank = static_cast<int>(blockIdx.y);
  tl.kbeg = 0;
  tl.kend = p.K;
  if (tl.C > 1) {
    const unsigned ksteps_total = static_cast<unsigned>(p.K + 15) >> 4, C = gridDim.y, r = blockIdx.y;
    tl.kbeg = static_cast<int>(r * ksteps_total / C) * 16;
    tl.kend = min(p.K, static_cast<int>((r + 1) * ksteps_total / C) * 16);
  }
  tl.kslice = max(0, tl.kend - tl.kbeg);
  return tl;
}

struct SharedScratch {
  float inv_scale[kMaxRows];
  float scale[kMaxRows];
  uint32_t rmax[kMaxRows];  // largest BF16 magnitude bits of the row's K slice
  uint32_t rmin[kMaxRows];  // smallest non-zero BF16 magnitude bits (0x7FFF if the slice is all zero)
  float best_v[kMaxThreads / 32][kMaxRows];
  long long best_i[kMaxThreads / 32][kMaxRows];
  float gate[kMaxRows];  // SharedExpertDown: the BF16 sigmoid gate of every row (best_v holds its partial sums first)
  int last;
  int xfail;  // sharded LM head: a wait for a peer's keys ran out in this call
  unsigned long long rowkey[kMaxRows];  // fused LM head: the CTA's best key of every row (atomicMax of the warps' bests)
};

// The BF16 arithmetic of SharedExpertDown (src/common/sigmoid_acc.cuh:12-21, skinny_gemm.cuh:73-80): sigmoid
// in FP32 from exp(-|a|), rounded once to BF16; Swish = bf16(x * bf16(sigmoid(x))); swish_mul = bf16(Swish(g) * u).
__device__ __forceinline__ float RoundBf16(float v) { return __bfloat162float(__float2bfloat16(v)); }
__device__ __forceinline__ float SigmoidBf16(float a) {
  const float e = expf(-fabsf(a));
  return RoundBf16(a > 0.0f ? 1.0f / (1.0f + e) : e / (1.0f + e));
}
__device__ __forceinline__ uint32_t SwishMulBits(uint32_t g_bits, uint32_t u_bits) {  // one BF16 each, in the low 16 bits
  const float g = __uint_as_float(g_bits << 16), u = __uint_as_float(u_bits << 16);
  const float swish = RoundBf16(g * SigmoidBf16(g));
  return static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16(swish * u)));
}
__device__ __forceinline__ uint32_t SwishMulWord(uint32_t g2, uint32_t u2) {  // two BF16 per word
  return SwishMulBits(g2 & 0xFFFFu, u2 & 0xFFFFu) | (SwishMulBits(g2 >> 16, u2 >> 16) << 16);
}

// max / min-nonzero of the two BF16 magnitudes packed in a word
// Measurement aid, compiled in only with -DQFG_PHASE_TIMES: thread 0 of every CTA records the global timer
// at the phase boundaries into GemmParams::phase_times ([CTA][16]).
#ifdef QFG_PHASE_TIMES
__device__ __forceinline__ void Stamp(const GemmParams& p, int slot) {
  if (p.phase_times != nullptr && threadIdx.x == 0) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    p.phase_times[(static_cast<size_t>(blockIdx.y) * gridDim.x + blockIdx.x) * 16 + slot] = t;
  }
}
#else
__device__ __forceinline__ void Stamp(const GemmParams&, int) {}
#endif
__device__ __forceinline__ void TrackWord(uint32_t w, uint32_t& mx, uint32_t& mn) {
  const uint32_t lo = w & 0x7FFFu, hi = (w >> 16) & 0x7FFFu;
  mx = max(mx, max(lo, hi));
  mn = min(mn, min(lo != 0 ? lo : 0x7FFFu, hi != 0 ? hi : 0x7FFFu));
}

// two BF16 values times a power of two, as an FP16 pair (exact when the caller checked the range)
__device__ __forceinline__ uint32_t ScaleToHalf2(uint32_t w, float sc) {
  const float lo = __uint_as_float(w << 16) * sc, hi = __uint_as_float(w & 0xFFFF0000u) * sc;
  const __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// Copies the CTA's K slice of x into shared memory and, for the quantised modes, rescales every
// row by a power of two and converts it to FP16.  WORDS = 4: 16-byte chunks (x 16-byte aligned,
// K % 8 == 0); WORDS = 1: 4-byte pairs (K is even and slices start on multiples of 16, so a pair
// never straddles a slice).  Returns true if the CTA must take the BF16 path.
// Position (in 16-bit elements) of element k of row m of the staged x.  TC = false: rows of `xpitch`
// elements.  TC = true: the K-major no-swizzle operand layout of tcgen05.mma - per k-step 256 bytes,
// two 8-row x 16-byte core matrices (k 0..7, then k 8..15), row m at 16 m bytes inside each.
template <bool TC>
__device__ __forceinline__ int XsIndex(int m, int k, int xpitch) {
  if constexpr (TC) {
    return (k >> 4) * 128 + ((k >> 3) & 1) * 64 + m * 8 + (k & 7);
  } else {
    return m * xpitch + k;
  }
}

// WALK = false keeps the per-item divisions: the register-streaming kernel holds its prefetched weights in
// registers across the staging, and with the walk's state added the compiler's schedule of its K loop lost
// 5 us on the 52 MB BF16 projection (measured), so that kernel stays on the form it was tuned with.
template <int MODE, int WORDS, bool TC = false, bool FUSE = false, bool WALK = true>
__device__ __forceinline__ bool StageXImpl(const GemmParams& p, const Tile& tl, uint16_t* xs, SharedScratch& sh) {
  constexpr int kElems = 2 * WORDS;
  constexpr int kBatch = 4;  // loads in flight per thread (eight measured slower: twice the cold code for one round trip less)
  // a CTA whose K slice is empty (more cluster ranks than k-steps) stages nothing and adds nothing
  if (tl.kslice <= 0) return false;
  const int tid = threadIdx.x, nthreads = blockDim.x, lane = tid & 31;
  const int M = p.M, xpitch = p.xpitch;
  const int kpad = (tl.kslice + 15) & ~15;
  const int chunks = kpad / kElems;
  const int total = M * chunks;
  uint32_t* xw = reinterpret_cast<uint32_t*>(xs);
  // Item idx is chunk (idx % chunks) of row (idx / chunks).  A thread's items are nthreads apart, so it walks
  // (row, k) by a fixed step instead of dividing per item: the staging is a few hundred dependent
  // instructions per warp, and the divisions were a third of them.
  const int step_m = nthreads / chunks, step_k = (nthreads - step_m * chunks) * kElems;
  const int first_m = tid / chunks, first_k = (tid - first_m * chunks) * kElems;
  auto advance = [&](int& m, int& kk) {
    m += step_m;
    kk += step_k;
    if (kk >= kpad) {
      kk -= kpad;
      ++m;
    }
  };

  // pass 1: global -> shared (raw BF16).  All loads of a batch are issued before the first is
  // consumed, so a batch costs one L2 round trip.
  int next_m = first_m, next_k = first_k;
  for (int base0 = 0; base0 < total; base0 += nthreads * kBatch) {  // warp-uniform trip count
    uint32_t v[kBatch][WORDS];
    int st_m = next_m, st_k = next_k;  // the store phase below walks the batch again (cheaper than keeping 2 x kBatch indices)
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      int m, kk;
      if constexpr (WALK) {
        m = next_m;
        kk = next_k;
        advance(next_m, next_k);
      } else {
        const int idx = base0 + tid + j * nthreads;
        m = idx < total ? idx / chunks : M;
        kk = (idx - m * chunks) * kElems;
      }
#pragma unroll
      for (int e = 0; e < WORDS; ++e) v[j][e] = 0;
      if (m < M) {
        if (kk < tl.kslice) {
          const uint16_t* src = p.x + static_cast<size_t>(m) * p.K + tl.kbeg + kk;
          if constexpr (WORDS == 4) {
            const uint4 q = __ldg(reinterpret_cast<const uint4*>(src));
            v[j][0] = q.x, v[j][1] = q.y, v[j][2] = q.z, v[j][3] = q.w;
          } else {
            v[j][0] = __ldg(reinterpret_cast<const uint32_t*>(src));
          }
          if constexpr (FUSE) {  // SharedExpertDown: the row of x is swish_mul(g, u)
            const uint16_t* src2 = p.x2 + static_cast<size_t>(m) * p.K + tl.kbeg + kk;
#pragma unroll
            for (int e = 0; e < WORDS; ++e) v[j][e] = SwishMulWord(v[j][e], __ldg(reinterpret_cast<const uint32_t*>(src2) + e));
          }
        }
      }
    }
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      bool live;
      int m, kk;
      if constexpr (WALK) {
        live = st_m < M;
        m = live ? st_m : 0;
        kk = st_k;
        advance(st_m, st_k);
      } else {
        const int idx = base0 + tid + j * nthreads;
        live = idx < total;
        m = live ? idx / chunks : 0;
        kk = (idx - m * chunks) * kElems;
      }
      if (live) {
        uint32_t* dst = xw + (XsIndex<TC>(m, kk, xpitch) >> 1);
        if constexpr (WORDS == 4) {
          *reinterpret_cast<uint4*>(dst) = make_uint4(v[j][0], v[j][1], v[j][2], v[j][3]);
        } else {
          *dst = v[j][0];
        }
      }
      if constexpr (MODE != kBf16) {
        uint32_t mx = 0, mn = 0x7FFFu;
#pragma unroll
        for (int e = 0; e < WORDS; ++e) TrackWord(v[j][e], mx, mn);
        // lanes of a warp almost always work on the same row: one pair of atomics per warp
        const int m0 = __shfl_sync(0xffffffffu, m, 0);
        if (__all_sync(0xffffffffu, m == m0)) {
          mx = __reduce_max_sync(0xffffffffu, mx);
          mn = __reduce_min_sync(0xffffffffu, mn);
          if (lane == 0) {
            atomicMax(&sh.rmax[m0], mx);
            atomicMin(&sh.rmin[m0], mn);
          }
        } else if (live) {
          atomicMax(&sh.rmax[m], mx);
          atomicMin(&sh.rmin[m], mn);
        }
      }
    }
  }
  if constexpr (MODE == kBf16) {
    __syncthreads();
    return false;
  } else {
    __syncthreads();
    // Power-of-two scale per row that puts the slice maximum in [2^14, 2^15).  Every non-zero
    // element must land in the normal FP16 range: exponent no more than 28 below the maximum's.
    bool ok = !p.force_slow;
#pragma unroll
    for (int m = 0; m < kMaxRows; ++m) {
      if (m < M) {
        const uint32_t a = sh.rmax[m];
        const int e = static_cast<int>(a >> 7);  // BF16 exponent field of the row maximum
        if (a != 0 && (e < 32 || e >= 255 || static_cast<int>(sh.rmin[m] >> 7) < e - 28)) ok = false;
      }
    }
    const bool slow = !ok;
    if (tid < kMaxRows) {
      float sc = 1.f;
      if (!slow && tid < M && sh.rmax[tid] != 0) sc = __uint_as_float((268u - (sh.rmax[tid] >> 7)) << 23);
      sh.scale[tid] = sc;
      sh.inv_scale[tid] = 1.f / sc;
    }
    __syncthreads();
    if (!slow) {
      // pass 2: in place, BF16 -> scaled FP16
      for (int m = first_m, kk = first_k; m < M; advance(m, kk)) {
        const float sc = sh.scale[m];
        uint32_t* px = xw + (XsIndex<TC>(m, kk, xpitch) >> 1);
        if constexpr (WORDS == 4) {
          uint4 q = *reinterpret_cast<uint4*>(px);
          q.x = ScaleToHalf2(q.x, sc);
          q.y = ScaleToHalf2(q.y, sc);
          q.z = ScaleToHalf2(q.z, sc);
          q.w = ScaleToHalf2(q.w, sc);
          *reinterpret_cast<uint4*>(px) = q;
        } else {
          *px = ScaleToHalf2(*px, sc);
        }
      }
      __syncthreads();
    }
    return slow;
  }
}

// Asynchronous staging of x for the warp-ring kernel.  The x loads of the staging above are issued after the
// ring prologue and queue behind its weight copies (50 - 130 KB per SM, one to three microseconds of the SM's
// share of the bandwidth) while every warp waits for them.  Here the CTA's K slice of x is copied raw into its
// place in shared memory with 16-byte cp.async BEFORE the weight copies are issued - the copy group is the
// oldest, so `cp.async.wait_group <weight groups>` completes it - and converted in place afterwards, while the
// weights are in flight.  Needs 16-byte rows of x (x 16-byte aligned, K % 8 == 0).
__device__ __forceinline__ bool XRowsAre16ByteAligned(const GemmParams& p) {
  return (reinterpret_cast<uintptr_t>(p.x) % 16 == 0) && (p.K % 8 == 0);
}
// Which 16-byte items of the staged x a thread handles.  A warp works on one row at a time (warp w on row
// w mod M, the warps of a row sharing its items; with fewer warps than rows, on rows w, w + warps, ...), so a
// row's maximum is reduced once per warp, and nothing here divides per item.  f(live, kk): elements kk .. kk + 7
// of the row, `live` false past the row's end (the trip count is warp-uniform); row_done(m) after each row.
template <class F, class G>
__device__ __forceinline__ void ForMyXItems(const GemmParams& p, const Tile& tl, F&& f, G&& row_done) {
  const unsigned warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5, M = static_cast<unsigned>(p.M);
  const int chunks = ((tl.kslice + 15) & ~15) >> 3;
  const unsigned part = warp / M, row0 = warp - part * M;
  const unsigned cnt = nwarps > M ? (nwarps - row0 + M - 1) / M : 1u;  // warps that share row0
#pragma unroll 1
  for (unsigned m = row0; m < M; m += nwarps) {
#pragma unroll 1
    for (int c0 = static_cast<int>(32u * part); c0 < chunks; c0 += static_cast<int>(32u * cnt)) {
      const int c = c0 + static_cast<int>(lane);
      f(c < chunks, static_cast<int>(m), c * 8);
    }
    row_done(static_cast<int>(m));
  }
}
__device__ __forceinline__ void XCopyIssue(const GemmParams& p, const Tile& tl, uint16_t* xs) {
  if (tl.kslice <= 0) return;
  const uint32_t base = SmemAddr(xs);
  ForMyXItems(
      p, tl,
      [&](bool live, int m, int kk) {
        if (!live) return;
        const bool in = kk < tl.kslice;  // the slice is padded to whole k-steps with zeros
        const uint16_t* src = p.x + static_cast<size_t>(m) * p.K + tl.kbeg + kk;
        CpAsync16(base + static_cast<uint32_t>(m * p.xpitch + kk) * 2u, in ? src : p.x, in ? 16 : 0);
      },
      [](int) {});
}
// Second half: every thread's copies have completed (cp.async.wait_group).  Must be called by every thread of
// the CTA.  Returns true if the CTA must take the BF16 path.
template <int MODE>
__device__ __forceinline__ bool StageXConvert(const GemmParams& p, const Tile& tl, uint16_t* xs, SharedScratch& sh) {
  const int tid = threadIdx.x, lane = tid & 31, M = p.M;
  if (tid < kMaxRows) {
    sh.rmax[tid] = 0;
    sh.rmin[tid] = 0x7FFFu;
    sh.inv_scale[tid] = 1.f;
  }
  __syncthreads();  // the raw rows are visible to every thread
  if constexpr (MODE == kBf16) {
    return false;
  } else {
    if (tl.kslice <= 0) return false;
    uint32_t* xw = reinterpret_cast<uint32_t*>(xs);
    uint32_t mx = 0, mn = 0x7FFFu;
    ForMyXItems(
        p, tl,
        [&](bool live, int m, int kk) {
          if (live) {
            const uint4 q = *reinterpret_cast<const uint4*>(xw + ((m * p.xpitch + kk) >> 1));
            TrackWord(q.x, mx, mn);
            TrackWord(q.y, mx, mn);
            TrackWord(q.z, mx, mn);
            TrackWord(q.w, mx, mn);
          }
        },
        [&](int m) {
          mx = __reduce_max_sync(0xffffffffu, mx);
          mn = __reduce_min_sync(0xffffffffu, mn);
          if (lane == 0) {
            atomicMax(&sh.rmax[m], mx);
            atomicMin(&sh.rmin[m], mn);
          }
          mx = 0;
          mn = 0x7FFFu;
        });
    __syncthreads();
    // Power-of-two scale per row that puts the slice maximum in [2^14, 2^15).  Every non-zero element must
    // land in the normal FP16 range: exponent no more than 28 below the maximum's.
    bool ok = !p.force_slow;
#pragma unroll 1
    for (int m = 0; m < M; ++m) {
      const uint32_t a = sh.rmax[m];
      const int e = static_cast<int>(a >> 7);  // BF16 exponent field of the row maximum
      if (a != 0 && (e < 32 || e >= 255 || static_cast<int>(sh.rmin[m] >> 7) < e - 28)) ok = false;
    }
    const bool slow = !ok;
    auto scale_of = [&](int m) {
      const uint32_t a = sh.rmax[m];
      return (!slow && a != 0) ? __uint_as_float((268u - (a >> 7)) << 23) : 1.f;
    };
    if (tid < M) {  // for the epilogue, which runs behind further barriers
      const float sc = scale_of(tid);
      sh.scale[tid] = sc;
      sh.inv_scale[tid] = 1.f / sc;
    }
    if (!slow) {
      float sc = 1.f;
      int sc_row = -1;
      ForMyXItems(
          p, tl,
          [&](bool live, int m, int kk) {
            if (!live) return;
            if (m != sc_row) {
              sc = scale_of(m);
              sc_row = m;
            }
            uint4* px = reinterpret_cast<uint4*>(xw + ((m * p.xpitch + kk) >> 1));
            uint4 q = *px;
            q.x = ScaleToHalf2(q.x, sc);
            q.y = ScaleToHalf2(q.y, sc);
            q.z = ScaleToHalf2(q.z, sc);
            q.w = ScaleToHalf2(q.w, sc);
            *px = q;
          },
          [](int) {});
    }
    __syncthreads();
    return slow;
  }
}

// SharedExpertDown's staging: the gate of every row, then x = swish_mul(g, u) staged like a plain x.  Kept
// out of line: the streaming kernels were measured to slow down by several percent whenever code was added
// to their inlined body, executed or not, so everything this op adds to them is one call on a cold branch.
template <int MODE, bool TC>
__device__ __noinline__ bool StageXFused(const GemmParams& p, const Tile& tl, uint16_t* xs, SharedScratch& sh) {
  // gate logit of every row: thread-strided partial sums, warps in order, then bf16 -> sigmoid -> bf16.  All rows
  // at once - a thread reads a 16-byte chunk of gw and the same chunk of every row of gx before it adds anything -
  // so the gate costs one round trip to L2, not one per row (one row at a time took 1.7 us per row).
  const int tid = threadIdx.x, nthreads = blockDim.x, warp = tid >> 5, lane = tid & 31;
  const int M = p.M;
  float part[kMaxRows];
#pragma unroll
  for (int m = 0; m < kMaxRows; ++m) part[m] = 0.f;
  const bool gvec = (reinterpret_cast<uintptr_t>(p.gx) % 16 == 0) && (reinterpret_cast<uintptr_t>(p.gw) % 16 == 0) && (p.gk % 8 == 0);
  if (gvec) {
    const int chunks = p.gk >> 3;
    const uint4* gw4 = reinterpret_cast<const uint4*>(p.gw);
#pragma unroll 1
    for (int c = tid; c < chunks; c += nthreads) {
      const uint4 w = __ldg(gw4 + c);
      uint4 xv[kMaxRows];
#pragma unroll
      for (int m = 0; m < kMaxRows; ++m) {
        if (m < M) xv[m] = __ldg(reinterpret_cast<const uint4*>(p.gx + static_cast<size_t>(m) * p.gk) + c);
      }
      const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
      for (int m = 0; m < kMaxRows; ++m) {
        if (m < M) {
          const uint32_t xx[4] = {xv[m].x, xv[m].y, xv[m].z, xv[m].w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {  // elements in index order
            part[m] += __uint_as_float(xx[e] << 16) * __uint_as_float(ww[e] << 16);
            part[m] += __uint_as_float(xx[e] & 0xFFFF0000u) * __uint_as_float(ww[e] & 0xFFFF0000u);
          }
        }
      }
    }
  } else {
    for (int m = 0; m < M; ++m) {
      float acc = 0.f;
      const uint16_t* gxm = p.gx + static_cast<size_t>(m) * p.gk;
      for (int i = tid; i < p.gk; i += nthreads)
        acc += __uint_as_float(static_cast<uint32_t>(gxm[i]) << 16) * __uint_as_float(static_cast<uint32_t>(p.gw[i]) << 16);
      part[m] = acc;
    }
  }
#pragma unroll
  for (int m = 0; m < kMaxRows; ++m) {
    if (m < M) {  // warp-uniform
      float v = part[m];
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
      if (lane == 0) sh.best_v[warp][m] = v;
    }
  }
  __syncthreads();
  if (tid < kMaxRows) {
    float logit = 0.f;
    if (tid < p.M)
      for (int w = 0; w < (nthreads >> 5); ++w) logit += sh.best_v[w][tid];
    sh.gate[tid] = SigmoidBf16(RoundBf16(logit));
  }
  __syncthreads();
  // swish_mul reads x2 with the same vector width as x
  const bool vec8 = (reinterpret_cast<uintptr_t>(p.x) % 16 == 0) && (p.K % 8 == 0) && (reinterpret_cast<uintptr_t>(p.x2) % 16 == 0);
  if (vec8) return StageXImpl<MODE, 4, TC, true>(p, tl, xs, sh);
  return StageXImpl<MODE, 1, TC, true>(p, tl, xs, sh);
}

// Must be called by every thread of the CTA; sh.rmax / sh.rmin are initialised here.
template <int MODE, bool TC = false, bool WALK = true, bool FUSE = false>
__device__ __forceinline__ bool StageX(const GemmParams& p, const Tile& tl, uint16_t* xs, SharedScratch& sh) {
  if (threadIdx.x < kMaxRows) {
    sh.rmax[threadIdx.x] = 0;
    sh.rmin[threadIdx.x] = 0x7FFFu;
    sh.inv_scale[threadIdx.x] = 1.f;
  }
  __syncthreads();
  if constexpr (FUSE) return StageXFused<MODE, TC>(p, tl, xs, sh);
  const bool vec8 = (reinterpret_cast<uintptr_t>(p.x) % 16 == 0) && (p.K % 8 == 0);
  if (vec8) return StageXImpl<MODE, 4, TC, false, WALK>(p, tl, xs, sh);
  return StageXImpl<MODE, 1, TC, false, WALK>(p, tl, xs, sh);
}

// Position of column c of row m inside a row of the partial-sum array.  An MMA accumulator fragment puts the
// lanes of a warp 16 (or 8) columns apart in rows 2t and 2t + 1, and a row is a multiple of 32 floats long, so
// plain indexing made the 8-byte stores of a warp collide 8- to 16-way.  The exclusive-or moves column bits
// 5-6 and row bits 1-2 into the bank bits (1-4) and stays inside the aligned group of 32 columns.
__device__ __forceinline__ int RedCol(int c, int m) { return c ^ ((((c >> 5) & 3) << 1) ^ (((m >> 1) & 3) << 3)); }

// The part of the epilogue that starts from the partial sums in shared memory: `red` holds
// [nparts][M][TNc] floats (part w = the sum over the k-steps of K-group w), the cluster partials
// follow it.  Every thread of the CTA must call this after a __syncthreads() that follows the
// last write to `red`.
template <int MODE, bool FUSE = false>
__device__ __forceinline__ void EpilogueTail(const GemmParams& p, const Tile& tl, uint8_t* smem, SharedScratch& sh,
                                             int nparts, int TNc) {
  const int tid = threadIdx.x, nthreads = blockDim.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int M = p.M, C = tl.C, n0 = tl.n0, n1 = tl.n1;
  const Segment& sg = p.seg[tl.seg];
  float* red = reinterpret_cast<float*>(smem);
  float* part = red + static_cast<size_t>(nparts) * M * TNc;
  const int ncols = n1 - n0;  // valid columns of the tile (<= TNc)
  // Fused argmax: rows are finished one at a time, so a thread carries the best (value, index) of the row in
  // hand only, and flush_row leaves the warp's best of that row in shared memory.  One copy of this code
  // serves every row: the epilogue runs once, from a cold instruction cache, and an eight-way unrolled form
  // of it was measured at 1.7 us per row.
  float cur_v = 0.f;
  long long cur_i = -1;
  // what every element needs from the parameter block, read once
  const float* const w_scale = sg.w_scale;
  const bool lm = p.lm != 0;
  const int out_begin = sg.out_begin, out_end = sg.out_end;
  const bool store = !lm || p.out[out_begin] != nullptr;
  const long long col_offset = p.lm_col_offset;
  auto finalize = [&](int m, int c, float v) {
    const int n = n0 + c;
    if (w_scale != nullptr) v *= w_scale[n];
    if constexpr (FUSE) {
      // SharedExpertDown: routed + bf16(bf16(sum) * gate), every step rounded to BF16 (skinny_gemm.cuh:226-240)
      const float shared = RoundBf16(RoundBf16(v) * sh.gate[m]);
      v = p.routed != nullptr ? __uint_as_float(static_cast<uint32_t>(p.routed[static_cast<size_t>(m) * sg.n + n]) << 16) + shared
                              : shared;
    }
    const __nv_bfloat16 b = __float2bfloat16(v);
    if (store) {
      int j = out_begin;
      for (int i = j + 1; i < out_end; ++i) {
        if (n >= p.col_begin[i]) j = i;
      }
      p.out[j][static_cast<size_t>(m) * p.width[j] + (n - p.col_begin[j])] = __bfloat16_as_ushort(b);
    }
    if (lm) {
      // a thread meets the columns of a row in increasing order: strict comparison, a NaN is never replaced
      const float f = __bfloat162float(b);
      if (cur_i < 0 || f > cur_v || (f != f && cur_v == cur_v)) {
        cur_v = f;
        cur_i = col_offset + n;
      }
    }
  };
  // The warp's best of row m joins the CTA's best of that row: keys (argmax_key.cuh), two redux per warp, one
  // shared-memory atomicMax.
  auto flush_row = [&](int m) {
    if (!lm) return;
    const unsigned long long key = WarpMaxKey(cur_i < 0 ? 0ull : PackKey(cur_v, cur_i));
    if (lane == 0 && key != 0ull) atomicMax(&sh.rowkey[m], key);
    cur_v = 0.f;
    cur_i = -1;
  };
  if (tid < kMaxRows) sh.rowkey[tid] = 0ull;
  __syncthreads();

  // All rows are finished side by side: a warp works on one row at a time - wpr warps per row, every lane on
  // columns 32 wpr apart in increasing order - so the rows' shared-memory (or cluster) round trips overlap
  // instead of following one another, and a warp reduces its candidates once per row it touches.
  const int nwarps = nthreads >> 5;
  const int wpr = max(1, nwarps / M), rows_per_pass = max(1, nwarps / wpr);
  const int my_row = warp / wpr, my_part = warp - my_row * wpr;
  auto for_my_columns = [&](int share, auto&& value) {  // value(m, j): column j of this CTA's share, 0 <= j < share
    for (int m0 = 0; m0 < M; m0 += rows_per_pass) {
      const int m = m0 + my_row;
      if (my_row < rows_per_pass && m < M) {
        for (int j = my_part * 32 + lane; j < share; j += wpr * 32) value(m, j);
        flush_row(m);
      }
    }
  };

  if (C == 1) {
    for_my_columns(ncols, [&](int m, int c) {
      float sum = 0.f;
      for (int w = 0; w < nparts; ++w) sum += red[(w * M + m) * TNc + RedCol(c, m)];
      finalize(m, c, sum * sh.inv_scale[m]);
    });
  } else {
    for (int m = 0; m < M; ++m) {
      const float inv = sh.inv_scale[m];
      for (int c = tid; c < TNc; c += nthreads) {
        float sum = 0.f;
        for (int w = 0; w < nparts; ++w) sum += red[(w * M + m) * TNc + RedCol(c, m)];
        part[m * TNc + c] = sum * inv;
      }
    }
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();
    const int cper = (TNc + C - 1) / C;  // the last rank's share may be short (any C <= 8)
    const int cb = tl.crank * cper;
    const int share = max(0, min(cper, ncols - cb));
    // The C partial sums of an output come from C CTAs' shared memory: all eight possible loads are issued
    // before the first is used (one round trip through the cluster network instead of C), then added in rank order.
    for_my_columns(share, [&](int m, int j) {
      const int idx = m * TNc + cb + j;
      float v[8];
#pragma unroll
      for (int r = 0; r < 8; ++r) v[r] = r < C ? cluster.map_shared_rank(part, r)[idx] : 0.f;
      float sum = 0.f;
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        if (r < C) sum += v[r];
      }
      finalize(m, cb + j, sum);
    });
    cluster.sync();
  }

  if (p.lm) {
    // The warps' bests of every row (flush_row) folded into the workspace keys with a 64-bit atomic max.
    auto fold_into_keys = [&]() {
      __syncthreads();
      if (tid < M) {
        const unsigned long long best = sh.rowkey[tid];
        sh.rowkey[tid] = 0ull;
        if (best != 0ull) atomicMax(p.lm_keys + tid, best);
        __threadfence();
      }
      __syncthreads();
    };
    fold_into_keys();
    if (tid == 0) {
      const unsigned int total = gridDim.x * gridDim.y;
      const unsigned int prev = atomicAdd(p.lm_count, 1u);
      sh.last = (prev == total - 1) ? 1 : 0;
      __threadfence();
    }
    __syncthreads();
    if (sh.last) {
      unsigned long long tail_best = 0ull;  // thread m < M: best key of row m among the shared columns
      if (p.tail_groups > 0) {
        // the partial sums of the shared columns were stored before their CTAs counted themselves in:
        // add the K slices up in order, finish those columns and fold their best into the keys
        __threadfence();
        const int n_main = sg.n - p.tail_groups * 128;
        const int tcols = p.tail_groups * 128;
        // This runs after every other CTA has finished, so it is all on the critical path.  One output (row,
        // shared column) per thread and pass: all its slices are loaded before the first is added (one round
        // trip to L2), still in slice order.  A group is 128 columns wide, so the 32 outputs of a warp belong
        // to one row, which flush_row needs.
        const int outs = M * tcols;
        for (int o = tid; o < outs; o += nthreads) {
          const int m = o / tcols, j = o - m * tcols;
          const float* src = p.lm_tail + (static_cast<size_t>(j >> 7) * p.tail_split * kMaxRows + m) * 128 + (j & 127);
          float part[kMaxTailSplit];
#pragma unroll
          for (int c = 0; c < kMaxTailSplit; ++c) part[c] = c < p.tail_split ? __ldcg(src + static_cast<size_t>(c) * kMaxRows * 128) : 0.f;
          float sum = 0.f;
#pragma unroll
          for (int c = 0; c < kMaxTailSplit; ++c) sum += part[c];
          finalize(m, n_main + j - n0, sum * sh.inv_scale[m]);
          flush_row(m);
        }
        // no other CTA is left to see these keys: they join the global ones in registers below
        __syncthreads();
        if (tid < M) tail_best = sh.rowkey[tid];
      }
      unsigned long long key = 0ull;  // thread m < M: the winning key of row m
      if (p.xworld > 1) {
        // Sharded head: this rank's keys go straight into every rank's exchange buffer (peer memory) as
        // self-validating words - (upper or lower half of the key) << 32 | call count - so that one round of
        // 8-byte stores carries both the data and the signal that it has arrived: no fence, no separate flag.
        // Slots alternate with the parity of the call count: a rank that is one call ahead writes the other
        // slot.  Every rank then awaits - bounded - the words of all ranks in its own buffer and folds them;
        // the maximum of the order-preserving keys is the Better order, so every rank ends with the same
        // winner.  A wait that runs out sets the buffer's status and the row is folded without that peer.
        LmExchange* own = p.xpeer[p.xrank];
        const unsigned int epoch = own->epoch + 1;  // every thread reads it before thread 0 advances it below
        const int par = static_cast<int>(epoch & 1u);
        if (tid < M) {
          unsigned long long mine = atomicExch(p.lm_keys + tid, 0ull);
          sh.best_i[0][tid] = static_cast<long long>(tail_best > mine ? tail_best : mine);
        }
        if (tid == 0) sh.xfail = 0;
        __syncthreads();
        unsigned long long t_ready = 0, t_sent = 0;
        if (tid == 0) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_ready));
        const int nwords = 2 * M * p.xworld;
        for (int w = tid; w < nwords; w += nthreads) {
          const int r = w / (2 * M), rem = w - r * 2 * M, row = rem >> 1, half = rem & 1;
          const unsigned long long k = static_cast<unsigned long long>(sh.best_i[0][row]);
          const unsigned long long payload = half ? (k & 0xFFFFFFFFull) : (k >> 32);
          *reinterpret_cast<volatile unsigned long long*>(&p.xpeer[r]->words[par][p.xrank][row][half]) = (payload << 32) | epoch;
        }
        if (tid == 0) {
          own->epoch = epoch;
          asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_sent));
        }
        for (int w = tid; w < nwords; w += nthreads) {
          const int r = w / (2 * M), rem = w - r * 2 * M, row = rem >> 1, half = rem & 1;
          const volatile unsigned long long* word = &own->words[par][r][row][half];
          int spin = 0;
          while (static_cast<unsigned int>(*word) != epoch && spin < p.xspin) {
            ++spin;
            __nanosleep(32);
          }
          if (static_cast<unsigned int>(*word) != epoch) {
            own->status = 1;
            sh.xfail = 1;
          }
        }
        __syncthreads();
        if (tid < M) {
          for (int r = 0; r < p.xworld; ++r) {
            const unsigned long long w0 = *reinterpret_cast<const volatile unsigned long long*>(&own->words[par][r][tid][0]);
            const unsigned long long w1 = *reinterpret_cast<const volatile unsigned long long*>(&own->words[par][r][tid][1]);
            const bool arrived = static_cast<unsigned int>(w0) == epoch && static_cast<unsigned int>(w1) == epoch;
            const unsigned long long k = (w0 & 0xFFFFFFFF00000000ull) | (w1 >> 32);
            if (arrived && k > key) key = k;
          }
        }
        if (tid == 0) {
          // telemetry of the owner's last call: keys ready, stores issued, all words seen (or given up on)
          unsigned long long t_done;
          asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_done));
          own->t_ready = t_ready;
          own->t_sent = t_sent;
          own->t_done = t_done;
          if (p.lm_status_out != nullptr) *p.lm_status_out = static_cast<unsigned int>(sh.xfail);
        }
      } else if (tid < M) {
        key = atomicExch(p.lm_keys + tid, 0ull);
        key = tail_best > key ? tail_best : key;
      }
      if (tid < M) {
        if (p.lm_idx != nullptr) p.lm_idx[tid] = KeyIndex(key);
        if (p.lm_val != nullptr) p.lm_val[tid] = KeyValue(key);
        if (p.lm_key_out != nullptr) p.lm_key_out[tid] = key;
      }
      if (tid == 0) *p.lm_count = 0u;
    }
  }
}

// Reduction of the accumulators (wk warps, then the cluster), scaling, rounding, stores, and the
// fused argmax.  `smem` is reused for the partial sums; every thread of the CTA must call this
// after a __syncthreads() that ends all use of the shared memory by the main loop.
template <int MODE, int W = 1, bool FUSE = false>
__device__ __forceinline__ void Epilogue(const GemmParams& p, const Tile& tl, float (&acc)[Geom<MODE, W>::kMmas][4],
                                         uint8_t* smem, SharedScratch& sh, bool warp_has_cols) {
  using G = Geom<MODE, W>;
  constexpr int NM = G::kMmas;
  const int tid = threadIdx.x, nthreads = blockDim.x;
  const int warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int wn = warp % p.wn, wk = warp / p.wn;
  const int M = p.M, C = tl.C, n0 = tl.n0, n1 = tl.n1;
  const Segment& sg = p.seg[tl.seg];
  const int cols_per_warp = 8 * G::kColsPerThread * W;
  const int TNc = p.wn * cols_per_warp;
  float* red = reinterpret_cast<float*>(smem);
  float* part = red + static_cast<size_t>(p.wk) * M * TNc;
  if (warp_has_cols) {
#pragma unroll
    for (int j = 0; j < NM; ++j) {
      // MMA j covers columns 2 (j % 8), +1 of the thread's (j / 8)-th column group (128 columns apart)
      const int per_group = G::kMmas / W;
      const int cl = wn * cols_per_warp + (j / per_group) * 8 * G::kColsPerThread + g * G::kColsPerThread + 2 * (j % per_group);
      const int m0 = 2 * t, m1 = 2 * t + 1;
      if (m0 < M) *reinterpret_cast<float2*>(&red[(wk * M + m0) * TNc + RedCol(cl, m0)]) = make_float2(acc[j][0], acc[j][2]);
      if (m1 < M) *reinterpret_cast<float2*>(&red[(wk * M + m1) * TNc + RedCol(cl, m1)]) = make_float2(acc[j][1], acc[j][3]);
    }
  } else {
    for (int m = 0; m < M; ++m)
      for (int c = lane; c < cols_per_warp; c += 32) red[(wk * M + m) * TNc + wn * cols_per_warp + c] = 0.f;
  }
  __syncthreads();
  EpilogueTail<MODE, FUSE>(p, tl, smem, sh, p.wk, TNc);
}

// ------------------------------------------------------------------------------ direct kernel
// Every warp streams its own weight rows into a warp-private shared-memory ring with 16-byte
// cp.async.cg copies (L1 bypass), DEPTH k-steps ahead of the MMAs.  There is no CTA barrier in
// the K loop, and the bytes in flight per SM (warps x DEPTH x 2-3 KiB) are bounded by shared
// memory, not by registers.  Measured on B200: this copy pattern streams at over 6 TB/s with 16
// warps per SM, where 8-byte copies through L1 or register loads at the same occupancy stay
// below 4 TB/s.
//
// Ring slot of one warp.
//   BF16 / FP8: [4 rows][32 lanes][16 bytes]; every lane copies exactly the bytes it consumes.
//   NVFP4: the warp's 64 W nibble bytes of each of the 16 rows, copied as aligned 16-byte pieces
//     (a chunk that starts 8 bytes off a 16-byte boundary - odd rows of a weight whose packed
//     pitch is 8 mod 16, like the 151936-column LM head, or a tile whose first column is 16 mod
//     32 - takes one piece more and is read back at an offset of 8), then the one or two aligned
//     pieces around the warp's 8 W block-scale bytes of each row.  Rows 8..15 of the nibble area
//     and every fourth row of the scale area are displaced by 32 bytes, which puts the four row
//     groups a warp-wide shared-memory load touches into distinct banks.
// A lane owns up to kPieces pieces; their sources are one 64-bit base, advanced by a k-step
// stride per step, plus a 32-bit offset each.
template <typename T>
__device__ __forceinline__ void Pin(T& v) {
  asm volatile("" : "+r"(v));  // keeps a loop invariant in its register instead of being recomputed
}
__device__ __forceinline__ void CpAsync16If(uint32_t pred, uint32_t dst, const uint8_t* base, uint32_t off) {
  asm volatile(
      "{ .reg .pred p; .reg .u64 a;\n"
      " setp.ne.b32 p, %0, 0;\n"
      " mad.wide.u32 a, %3, 1, %2;\n"
      " @p cp.async.cg.shared.global [%1], [a], 16;\n}" ::"r"(pred), "r"(dst), "l"(base), "r"(off)
      : "memory");
}

template <int MODE, int W>
struct DirectSlot {
  using G = Geom<MODE, W>;
  static constexpr int kNibPitch = 64 * W + 16;                 // NVFP4: bytes per nibble row of a warp
  static constexpr int kNibBytes = MODE == kNvfp4 ? 16 * kNibPitch + 32 : 4 * 32 * G::kBytesPerThread;
  static constexpr int kSclPitch = 32;
  static constexpr int kSclBytes = MODE == kNvfp4 ? 16 * kSclPitch + 96 : 0;
  static constexpr int kBytes = kNibBytes + kSclBytes;
  static constexpr int kPiecesPerRow = 4 * W + 3;               // NVFP4: 4W+1 nibble pieces, 2 scale pieces
  static constexpr int kPieces = MODE == kNvfp4 ? (16 * kPiecesPerRow + 31) / 32 : 4;
  __device__ static constexpr int NibRow(int r) { return r * kNibPitch + ((r >> 3) & 1) * 32; }
  __device__ static constexpr int SclRow(int r) { return kNibBytes + r * kSclPitch + (r >> 2) * 32; }
};

// One warp's NVFP4 stream (128 columns): copy plan, ring and read offsets of the direct kernel, W = 1.
template <int DEPTH>
struct Nvfp4Stream {
  using S = DirectSlot<kNvfp4, 1>;
  static constexpr int NP = S::kPieces;
  const uint8_t* gbase;
  long long step_stride;
  uint32_t off[NP], dst[NP], pmask, rd_w[2], rd_s[2], ring;
  int nsteps, careful_step, row0, lane, kstride;

  // k-steps wk, wk + p.wk, ... of the CTA's K slice
  __device__ __forceinline__ void Setup(const GemmParams& p, const Tile& tl, const Segment& sg, int colwarp, int wk,
                                        uint32_t ring_addr, bool active) {
    const int ksteps = (tl.kslice + 15) >> 4;
    SetupRange(tl, sg, colwarp, wk, (active && ksteps > wk) ? (ksteps - wk + p.wk - 1) / p.wk : 0, p.wk, ring_addr);
  }

  // k-steps k_first, k_first + k_stride, ... (k_count of them) of the CTA's K slice; colwarp is a column of the weight
  __device__ __forceinline__ void SetupRange(const Tile& tl, const Segment& sg, int colwarp, int k_first, int k_count,
                                             int k_stride, uint32_t ring_addr) {
    lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const long long pitch = sg.pitch;
    const int ksteps = (tl.kslice + 15) >> 4;
    nsteps = k_count;
    kstride = k_stride;
    // the slice's last k-step is copied by the careful path
    careful_step = (k_count > 0 && ksteps - 1 >= k_first && (ksteps - 1 - k_first) % k_stride == 0 &&
                    (ksteps - 1 - k_first) / k_stride < k_count)
                       ? (ksteps - 1 - k_first) / k_stride
                       : -1;
    row0 = tl.kbeg + k_first * 16;
    step_stride = static_cast<long long>(k_stride) * 16 * pitch;
    ring = ring_addr;
    const long long warp_col_byte = colwarp / 2;
    gbase = sg.w + static_cast<long long>(row0) * pitch + warp_col_byte - 16;
    const int mis = static_cast<int>(pitch & 8);
    const int cshift = static_cast<int>(warp_col_byte & 8);
    const long long sabs = static_cast<long long>(sg.n >> 1) + (colwarp >> 4);
    const int so_even = static_cast<int>(sabs & 15), so_odd = static_cast<int>((sabs + mis) & 15);
    const int sh_even = cshift, sh_odd = (mis + cshift) & 15;
    pmask = 0;
#pragma unroll
    for (int j = 0; j < NP; ++j) {
      const int slot = lane + 32 * j;
      const int r = slot / S::kPiecesPerRow, c = slot - r * S::kPiecesPerRow;
      off[j] = 0;
      dst[j] = 0;
      if (r < 16) {
        if (c < 5) {
          const int shift = (r & 1) ? sh_odd : sh_even;
          if (c < 4 || shift != 0) pmask |= 1u << j;
          off[j] = static_cast<uint32_t>(static_cast<long long>(r) * pitch + (c * 16 - shift) + 16);
          dst[j] = static_cast<uint32_t>(S::NibRow(r) + c * 16);
        } else {
          const int c2 = c - 5;
          const int o = (r & 1) ? so_odd : so_even;
          if (c2 == 0 || o + 8 > 16) pmask |= 1u << j;
          off[j] = static_cast<uint32_t>(static_cast<long long>(r) * pitch + (sabs - o + c2 * 16 - warp_col_byte) + 16);
          dst[j] = static_cast<uint32_t>(S::SclRow(r) + c2 * 16);
        }
      }
    }
    const int rbase = S::NibRow(4 * t) + g * 8, sbase = S::SclRow(4 * t) + g;
    rd_w[0] = static_cast<uint32_t>(rbase + sh_even);
    rd_w[1] = static_cast<uint32_t>(rbase + sh_odd);
    rd_s[0] = static_cast<uint32_t>(sbase + so_even);
    rd_s[1] = static_cast<uint32_t>(sbase + so_odd);
#pragma unroll
    for (int j = 0; j < NP; ++j) {
      Pin(off[j]);
      Pin(dst[j]);
    }
    Pin(pmask);
    Pin(rd_w[0]);
    Pin(rd_w[1]);
    Pin(rd_s[0]);
    Pin(rd_s[1]);
  }

  __device__ __forceinline__ void Issue(const GemmParams& p, const Tile& tl, const Segment& sg, int s, uint32_t slot_addr) {
    if (s != careful_step) {
#pragma unroll
      for (int j = 0; j < NP; ++j) CpAsync16If(pmask & (1u << j), slot_addr + dst[j], gbase, off[j]);
    } else {
      const int r0 = row0 + s * kstride * 16;
#pragma unroll
      for (int j = 0; j < NP; ++j) {
        if (pmask & (1u << j)) {
          const int r = (lane + 32 * j) / S::kPiecesPerRow;
          const uint8_t* src = gbase + off[j];
          const long long room = sg.total_bytes - (src - sg.w);
          const int bytes = (r0 + r >= tl.kend) ? 0 : room >= 16 ? 16 : room > 0 ? static_cast<int>(room) : 0;
          CpAsync16(slot_addr + dst[j], bytes > 0 ? src : sg.w, bytes);
        }
      }
    }
    gbase += step_stride;
  }

  __device__ __forceinline__ void Prologue(const GemmParams& p, const Tile& tl, const Segment& sg) {
#pragma unroll
    for (int d = 0; d < DEPTH - 1; ++d) {
      if (d < nsteps) Issue(p, tl, sg, d, ring + d * S::kBytes);
      CpAsyncCommit();
    }
  }

  // consume(raw, s) for every local step s, DEPTH - 1 steps behind the copies
  template <class F>
  __device__ __forceinline__ void Run(const GemmParams& p, const Tile& tl, const Segment& sg, F&& consume) {
    const uint32_t ring_end = ring + DEPTH * S::kBytes;
    uint32_t rd_slot = ring, wr_slot = ring + (DEPTH - 1) * S::kBytes;
    for (int s = 0; s < nsteps; ++s) {
      __syncwarp();
      if (s + DEPTH - 1 < nsteps) Issue(p, tl, sg, s + DEPTH - 1, wr_slot);
      CpAsyncCommit();
      asm volatile("cp.async.wait_group %0;" ::"n"(DEPTH - 1) : "memory");
      __syncwarp();
      Raw<kNvfp4, 1> raw;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        raw.r[0][i] = Lds64(rd_slot + rd_w[i & 1] + i * S::kNibPitch);
        raw.s[0][i] = Lds8(rd_slot + rd_s[i & 1] + i * S::kSclPitch);
      }
      wr_slot = rd_slot;
      rd_slot += S::kBytes;
      if (rd_slot == ring_end) rd_slot = ring;
      consume(raw, s);
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
  }
};

// One warp's stream through its shared-memory ring: copy plan, read offsets and the K loop.
//
// A loop iteration handles a PAIR of the warp's k-steps (2 x 16 weight rows): one cp.async wait, one warp
// barrier, the copies of the pair DEPTH - 1 pairs ahead, then all shared-memory loads of both steps and
// their dequantisation and MMAs, which the compiler interleaves.  The body is not unrolled over the ring -
// the ring position is one register added to the few per-lane address registers - because the K loop runs
// out of the instruction cache of an SM sub-partition: a body over about 8 KB was measured 5-25 % slower.
//
// Slot of one k-step (RingSlot).  NVFP4 (column tiles start on multiples of 128 columns): 16 rows of
// 5 aligned 16-byte pieces around the row's 64 nibble bytes - the fifth is needed only where the chunk
// starts 8 bytes off a 16-byte boundary (odd rows of a weight whose packed pitch is 8 mod 16, like the
// 151936-column LM head) - then 16 rows of the one aligned piece that holds the row's 8 scale bytes.  The
// 160 nibble pieces of a pair are five copy instructions (piece index lane + 32 j), its 32 scale pieces a
// sixth, which keeps its lines in L1 (.ca): the four column warps whose scale bytes share a 32-byte sector
// then fetch it from L2 once, and the stream is bound by the sectors that cross from L2 to the SM (measured:
// 9.4 TB/s of sector traffic at 2.07 sector bytes per payload byte without this, 4.5 TB/s of weights).
// A lane whose index names an unneeded piece repeats piece 0 of that row (same source, same destination), so
// no copy is predicated.  Rows 8..15 of both areas are displaced (32 / 16 bytes), which puts the four rows a
// warp-wide load touches into distinct banks.  BF16 / FP8: [4 rows][32 lanes][16 bytes] per step, a lane
// copies exactly the bytes it consumes.  The last k-step of a K slice is copied by a careful path (rows past
// K read as zero, pieces clamped to the end of the tensor); a pair that contains it, or has no second step,
// takes that path for both steps.
template <int MODE>
struct RingSlot {
  static constexpr int kNibPitch = 80;
  static constexpr int kNibBytes = MODE == kNvfp4 ? 16 * kNibPitch + 32 : 4 * 32 * 16;
  static constexpr int kSclPitch = 16;
  static constexpr int kSclBytes = MODE == kNvfp4 ? 16 * kSclPitch + 16 : 0;
  static constexpr int kBytes = kNibBytes + kSclBytes;
  static constexpr int NP = MODE == kNvfp4 ? 6 : 8;  // copy instructions per pair of k-steps
  __device__ static constexpr int NibRow(int r) { return r * kNibPitch + ((r >> 3) & 1) * 32; }
  __device__ static constexpr int SclRow(int r) { return kNibBytes + r * kSclPitch + ((r >> 3) & 1) * 16; }
};
static_assert(RingSlot<kNvfp4>::kBytes == 1584 && RingSlot<kBf16>::kBytes == 2048, "keep RingSlotBytes() in step");

// The pieces of a lane within a pair of k-steps: source offset from the pair's base, destination offset in the
// ring, and (careful path) the row within the pair, 5 bits each.
template <int NP>
struct CopyPieces {
  uint32_t off[NP], dst[NP];
};
// Copies the pieces of a pair that belong to existing steps, with clamped sizes.
template <int NP>
__device__ __noinline__ void IssueCareful(const uint8_t* w, long long total_bytes, const uint8_t* gbase, int kend, int row0,
                                          int row_step, unsigned long long rows, CopyPieces<NP> pc, uint32_t slot_off, int steps) {
#pragma unroll
  for (int j = 0; j < NP; ++j) {
    const int rr = static_cast<int>((rows >> (5 * j)) & 31u);  // step of the pair (bit 4) and row within it
    const int e = rr >> 4, r = rr & 15;
    if (e < steps) {
      const uint8_t* src = gbase + pc.off[j];
      const long long room = total_bytes - (src - w);
      const int bytes = (row0 + e * row_step + r >= kend) ? 0 : room >= 16 ? 16 : room > 0 ? static_cast<int>(room) : 0;
      CpAsync16(pc.dst[j] + slot_off, bytes > 0 ? src : w, bytes);
    }
  }
}

template <int MODE, int DEPTH>
struct WarpRing {
  using S = RingSlot<MODE>;
  static constexpr int NP = S::NP;
  static constexpr int kPairBytes = 2 * S::kBytes;
  static_assert(DEPTH >= 2 && DEPTH <= 4, "ring depth in pairs of k-steps");

  const uint8_t* gbase;  // next pair to copy, less 16 bytes (piece offsets are unsigned)
  long long step_stride;
  CopyPieces<NP> pc;     // dst includes the ring's address
  uint32_t rd_w[2], rd_s[2];
  unsigned long long rows;
  int nsteps, nfast, row_next, row_step;
  bool scales_l1;  // NVFP4: keep the scale pieces' lines in L1 (pays only while the CTA leaves L1 room beside its shared memory)

  // Local step s is k-step k_first + s * k_stride of the CTA's K slice, k_count steps in all.  `colwarp`:
  // first column of the warp; `lane_cols_ok`: the lane's own columns exist (BF16 / FP8 lanes past the
  // tile's last column copy the warp's first chunk instead; their sums are never stored).
  __device__ __forceinline__ void Setup(const Tile& tl, const Segment& sg, int colwarp, bool lane_cols_ok, int k_first,
                                        int k_count, int k_stride, uint32_t ring) {
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const long long pitch = sg.pitch;
    const int ksteps = (tl.kslice + 15) >> 4;
    nsteps = k_count;
    const int last = ksteps - 1 - k_first;
    const bool has_last = k_count > 0 && last >= 0 && last % k_stride == 0 && last / k_stride < k_count;
    nfast = has_last ? last / k_stride : nsteps;
    row_next = tl.kbeg + k_first * 16;
    row_step = k_stride * 16;
    step_stride = static_cast<long long>(k_stride) * 16 * pitch;
    rows = 0;
    scales_l1 = false;
    if constexpr (MODE == kNvfp4) {
      const long long warp_col_byte = colwarp / 2;  // a multiple of 64
      gbase = sg.w + static_cast<long long>(row_next) * pitch + warp_col_byte - 16;
      const int mis = static_cast<int>(pitch & 8);  // odd rows start 8 bytes off a 16-byte boundary
      const long long sabs = static_cast<long long>(sg.n >> 1) + (colwarp >> 4);  // scale bytes within the row: 0 or 8 mod 16
      const int so_even = static_cast<int>(sabs & 15), so_odd = static_cast<int>((sabs + mis) & 15);
#pragma unroll
      for (int j = 0; j < NP; ++j) {
        int e, r;
        long long src;
        uint32_t dst;
        if (j < 5) {  // nibble piece lane + 32 j of the pair's 2 x 16 x 5
          const int q = lane + 32 * j;
          e = q / 80;
          const int qq = q - e * 80;
          r = qq / 5;
          int c = qq - r * 5;
          const int shift = (r & 1) ? mis : 0;
          if (c == 4 && shift == 0) c = 0;
          src = c * 16 - shift;
          dst = static_cast<uint32_t>(S::NibRow(r) + c * 16);
        } else {      // scale piece of row lane % 16 of step lane / 16
          e = lane >> 4;
          r = lane & 15;
          const int o = (r & 1) ? so_odd : so_even;
          src = sabs - o - warp_col_byte;
          dst = static_cast<uint32_t>(S::SclRow(r));
        }
        pc.off[j] = static_cast<uint32_t>(static_cast<long long>(e) * step_stride + static_cast<long long>(r) * pitch + src + 16);
        pc.dst[j] = ring + dst + static_cast<uint32_t>(e * S::kBytes);
        rows |= static_cast<unsigned long long>(e * 16 + r) << (5 * j);
      }
      const int rbase = S::NibRow(4 * t) + g * 8, sbase = S::SclRow(4 * t) + g;
      rd_w[0] = ring + static_cast<uint32_t>(rbase);
      rd_w[1] = ring + static_cast<uint32_t>(rbase + mis);
      rd_s[0] = ring + static_cast<uint32_t>(sbase + so_even);
      rd_s[1] = ring + static_cast<uint32_t>(sbase + so_odd);
    } else {
      const long long warp_col_byte = MODE == kBf16 ? static_cast<long long>(colwarp) * 2 : colwarp;
      gbase = sg.w + static_cast<long long>(row_next) * pitch + warp_col_byte - 16;
      const int gsrc = lane_cols_ok ? g : 0;
#pragma unroll
      for (int j = 0; j < NP; ++j) {
        const int e = j >> 2, i = j & 3;
        pc.off[j] = static_cast<uint32_t>(static_cast<long long>(e) * step_stride + static_cast<long long>(4 * t + i) * pitch + gsrc * 16 + 16);
        pc.dst[j] = ring + static_cast<uint32_t>(e * S::kBytes + i * 512 + lane * 16);
        rows |= static_cast<unsigned long long>(e * 16 + 4 * t + i) << (5 * j);
      }
      rd_w[0] = rd_w[1] = ring + static_cast<uint32_t>(lane * 16);
      rd_s[0] = rd_s[1] = 0;
    }
  }

  // copies the pair of local steps (s0, s0 + 1) - the next ones in order - into the slots at `slot_off`
  __device__ __forceinline__ void IssuePair(const Tile& tl, const Segment& sg, int s0, uint32_t slot_off) {
    if (s0 + 1 < nfast) {
#pragma unroll
      for (int j = 0; j < NP; ++j) {
        if (MODE == kNvfp4 && j == NP - 1 && scales_l1) {
          CpAsync16At<0, true>(pc.dst[j] + slot_off, gbase, pc.off[j]);
        } else {
          CpAsync16At<0, false>(pc.dst[j] + slot_off, gbase, pc.off[j]);
        }
      }
    } else if (s0 < nsteps) {
      IssueCareful<NP>(sg.w, sg.total_bytes, gbase, tl.kend, row_next, row_step, rows, pc, slot_off, nsteps - s0);
    }
    gbase += 2 * step_stride;
    row_next += 2 * row_step;
  }

  // the first DEPTH - 1 pairs in flight
  __device__ __forceinline__ void Prologue(const Tile& tl, const Segment& sg) {
#pragma unroll
    for (int d = 0; d < DEPTH - 1; ++d) {
      IssuePair(tl, sg, 2 * d, static_cast<uint32_t>(d * kPairBytes));
      CpAsyncCommit();
    }
  }

  template <int OFF>
  __device__ __forceinline__ void LoadStep(Raw<MODE, 1>& raw, uint32_t w0, uint32_t w1, uint32_t s0, uint32_t s1) const {
    if constexpr (MODE == kNvfp4) {
      raw.r[0][0] = Lds64At<OFF>(w0);
      raw.r[0][1] = Lds64At<OFF + S::kNibPitch>(w1);
      raw.r[0][2] = Lds64At<OFF + 2 * S::kNibPitch>(w0);
      raw.r[0][3] = Lds64At<OFF + 3 * S::kNibPitch>(w1);
      raw.s[0][0] = Lds8At<OFF>(s0);
      raw.s[0][1] = Lds8At<OFF + S::kSclPitch>(s1);
      raw.s[0][2] = Lds8At<OFF + 2 * S::kSclPitch>(s0);
      raw.s[0][3] = Lds8At<OFF + 3 * S::kSclPitch>(s1);
    } else {
      raw.r[0] = Lds128At<OFF>(w0);
      raw.r[1] = Lds128At<OFF + 512>(w0);
      raw.r[2] = Lds128At<OFF + 1024>(w0);
      raw.r[3] = Lds128At<OFF + 1536>(w0);
    }
  }

  // consume(raw_a, raw_b, has_b) for every pair of local steps in order, DEPTH - 1 pairs behind the copies
  template <class F>
  __device__ __forceinline__ void Run(const Tile& tl, const Segment& sg, F&& consume) {
    const int npairs = (nsteps + 1) >> 1;
    uint32_t rd_off = 0, wr_off = static_cast<uint32_t>((DEPTH - 1) * kPairBytes);
    for (int i = 0; i < npairs; ++i) {
      asm volatile("cp.async.wait_group %0;" ::"n"(DEPTH - 2) : "memory");
      __syncwarp();  // every lane's copies of this pair are visible, and every lane is done reading the previous pair
      IssuePair(tl, sg, 2 * (i + DEPTH - 1), wr_off);
      CpAsyncCommit();
      Raw<MODE, 1> raw_a, raw_b;
      const uint32_t w0 = rd_w[0] + rd_off, w1 = rd_w[1] + rd_off, s0 = rd_s[0] + rd_off, s1 = rd_s[1] + rd_off;
      LoadStep<0>(raw_a, w0, w1, s0, s1);
      LoadStep<S::kBytes>(raw_b, w0, w1, s0, s1);
      consume(raw_a, raw_b, 2 * i + 1 < nsteps);
      wr_off = rd_off;
      rd_off += kPairBytes;
      if (rd_off == static_cast<uint32_t>(DEPTH * kPairBytes)) rd_off = 0;
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
  }
};

// DEPTH: pairs of k-steps in every warp's ring (2, 3 or 4)
// FUSE: the SharedExpertDown form (x = swish_mul(g, u) and the gate while x is staged, the gated rounding chain
// in the epilogue).  A kernel of its own, so that the plain kernels carry none of that code: they were measured
// to lose 2-3 % whenever it changed, run or not.
template <int MODE, int DEPTH, bool FUSE = false>
__global__ void __launch_bounds__(kMaxThreads, 1) SkinnyGemmDirectKernel(const __grid_constant__ GemmParams p) {
  using G = Geom<MODE, 1>;
  using S = RingSlot<MODE>;
  constexpr int NM = G::kMmas;
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ SharedScratch sh;

  if (p.trigger == 1) GridLaunchDependents();
  Stamp(p, 0);
  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int wn = warp % p.wn, wk = warp / p.wn;
  const Tile tl = LocateTile(p);
  const Segment& sg = p.seg[tl.seg];

  // this thread's columns and this warp's k-steps (local step s is k-step wk + s * p.wk of the slice)
  constexpr int cols_per_warp = 8 * G::kColsPerThread;
  const int colwarp = tl.n0 + wn * cols_per_warp;
  const bool warp_has_cols = colwarp < tl.n1;
  const bool cvalid = colwarp + g * G::kColsPerThread < tl.n1;
  const int ksteps = (tl.kslice + 15) >> 4;
  const uint32_t ring_addr = SmemAddr(smem) + static_cast<uint32_t>(warp) * (DEPTH * 2 * S::kBytes);

  // Shared tail of the fused LM head: a warp without columns of the tile (the last warp column of the CTA)
  // streams one K slice of one left-over column group through the same loop and stores FP32 partial sums.
  bool tail_worker = false;
  int tail_index = 0, first_step = wk, step_stride = p.wk, step_count = (warp_has_cols && ksteps > wk) ? (ksteps - wk + p.wk - 1) / p.wk : 0;
  int stream_col = colwarp;
  if constexpr (MODE == kNvfp4) {
    if (p.tail_groups > 0 && !warp_has_cols && wn == p.wn - 1) {
      // one (group, K slice) per idle warp: spread over the CTAs, or in order where the CTAs are few
      bool mine = true;
      if (p.tail_stride > 0) {
        tail_index = static_cast<int>(blockIdx.x) / p.tail_stride;
        mine = tail_index * p.tail_stride == static_cast<int>(blockIdx.x) && wk == tail_index % p.wk;
      } else {
        tail_index = static_cast<int>(blockIdx.x) * p.wk + wk;
      }
      if (mine && tail_index < p.tail_groups * p.tail_split) {
        tail_worker = true;
        const int tg = tail_index / p.tail_split, slice = tail_index - tg * p.tail_split;
        const unsigned split = static_cast<unsigned>(p.tail_split);
        first_step = static_cast<int>(static_cast<unsigned>(slice) * ksteps / split);
        step_count = static_cast<int>(static_cast<unsigned>(slice + 1) * ksteps / split) - first_step;
        step_stride = 1;
        stream_col = sg.n - p.tail_groups * 128 + tg * 128;
      }
    }
  }

  // x first (unless it is still the predecessor kernel's to write): its copies then do not queue behind the weights
  uint16_t* xs = reinterpret_cast<uint16_t*>(smem + p.ring_bytes);
  const bool x_async = !FUSE && XRowsAre16ByteAligned(p);
  if (x_async && !p.pdl_wait) {
    XCopyIssue(p, tl, xs);
    CpAsyncCommit();
  }
  // weights do not depend on the predecessor kernel: get the first k-steps in flight, then wait
  WarpRing<MODE, DEPTH> ring;
  ring.Setup(tl, sg, stream_col, cvalid, first_step, step_count, step_stride, ring_addr);
  ring.scales_l1 = p.scales_l1 != 0;
  ring.Prologue(tl, sg);
  if (p.pdl_wait) GridDependencyWait();
  Stamp(p, 1);

  bool slow;
  if (x_async) {
    if (p.pdl_wait) {  // x belongs to the predecessor until now
      XCopyIssue(p, tl, xs);
      CpAsyncCommit();
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group %0;" ::"n"(DEPTH - 1) : "memory");
    }
    slow = StageXConvert<MODE>(p, tl, xs, sh);
  } else {
    slow = StageX<MODE, false, true, FUSE>(p, tl, xs, sh);
  }
  Stamp(p, 2);

  float acc[NM][4];
#pragma unroll
  for (int j = 0; j < NM; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[j][e] = 0.f;

  // lanes whose x row does not exist read row 0; their accumulators are never stored
  uint32_t x_rd = SmemAddr(xs) + static_cast<uint32_t>(((g < p.M ? g : 0) * p.xpitch + 4 * t + first_step * 16) * 2);
  const uint32_t x_step = static_cast<uint32_t>(step_stride) * 32u;
  // One copy of the loop per operand path: the loop body then holds a single dequantisation.
  auto k_loop = [&](auto slow_tag) {
    constexpr bool kSlow = decltype(slow_tag)::value;
    ring.Run(tl, sg, [&](const Raw<MODE, 1>& raw_a, const Raw<MODE, 1>& raw_b, bool has_b) {
      const uint2 xa = Lds64(x_rd);
      ComputeStep<MODE, kSlow, 1>(acc, raw_a, xa.x, xa.y);
      if (has_b) {  // warp-uniform
        const uint2 xb = Lds64(x_rd + x_step);
        ComputeStep<MODE, kSlow, 1>(acc, raw_b, xb.x, xb.y);
      }
      x_rd += 2 * x_step;
    });
  };
  if constexpr (MODE == kBf16) {
    k_loop(std::false_type{});
  } else {
    if (slow) {
      k_loop(std::true_type{});
    } else {
      k_loop(std::false_type{});
    }
  }
  if constexpr (MODE == kNvfp4) {
    if (tail_worker) {
      float* dstp = p.lm_tail + static_cast<size_t>(tail_index) * kMaxRows * 128;
#pragma unroll
      for (int j = 0; j < NM; ++j) {
        const int cl = g * 16 + 2 * j;
        const int m0 = 2 * t, m1 = 2 * t + 1;
        if (m0 < p.M) *reinterpret_cast<float2*>(&dstp[m0 * 128 + cl]) = make_float2(acc[j][0], acc[j][2]);
        if (m1 < p.M) *reinterpret_cast<float2*>(&dstp[m1 * 128 + cl]) = make_float2(acc[j][1], acc[j][3]);
      }
      __threadfence();
    }
  }
  Stamp(p, 3);
  if (p.trigger == 2) GridLaunchDependents();
  __syncthreads();
  Stamp(p, 4);
  Epilogue<MODE, 1, FUSE>(p, tl, acc, smem, sh, warp_has_cols);
  Stamp(p, 5);
}


// ------------------------------------------------------------------------------ register-streaming kernel
// BF16 / FP8 only.  Every warp loads its rows straight into registers with 128-bit non-allocating
// loads, D k-steps ahead of the MMAs: no shared-memory ring, no cp.async, nothing to fill before the
// first MMA.  On the 50 MB decode projections (a dozen k-steps per warp) that start-up matters more
// than the deeper prefetch of the warp rings; on long streams the rings win.
constexpr int kRegThreads = 512;

template <int MODE, bool FUSE = false>
__global__ void __launch_bounds__(kRegThreads, 1) SkinnyGemmRegKernel(const __grid_constant__ GemmParams p) {
  using G = Geom<MODE>;
  constexpr int NM = G::kMmas;
  constexpr int D = MODE == kBf16 ? 4 : 3;  // k-steps in flight per warp (16 registers each)
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ SharedScratch sh;

  if (p.trigger == 1) GridLaunchDependents();
  Stamp(p, 0);
  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int wn = warp % p.wn, wk = warp / p.wn;
  const Tile tl = LocateTile(p);
  const Segment& sg = p.seg[tl.seg];
  const long long pitch = sg.pitch;

  // this thread's columns and this warp's k-steps (local step s is k-step wk + s * p.wk of the slice)
  const int cols_per_warp = 8 * G::kColsPerThread;
  const int colbase = tl.n0 + wn * cols_per_warp + g * G::kColsPerThread;
  const bool warp_has_cols = tl.n0 + wn * cols_per_warp < tl.n1;
  // threads past the tile's last column load nothing; their pointer is parked on the tile's first chunk
  const bool cvalid = colbase < tl.n1;
  const int colload = cvalid ? colbase : tl.n0;
  const int ksteps = (tl.kslice + 15) >> 4;
  const int nsteps = ksteps > wk ? (ksteps - wk + p.wk - 1) / p.wk : 0;
  // only the last k-step of the slice can be partial (K not a multiple of 16)
  const bool tail_here = (tl.kslice & 15) != 0 && ((ksteps - 1) % p.wk) == wk;
  const long long col_byte = (MODE == kBf16) ? static_cast<long long>(colload) * 2 : (MODE == kFp8) ? colload : colload / 2;
  // a thread owns rows 4t .. 4t+3 of a k-step (the k index of an MMA is a free permutation)
  const uint8_t* wq = sg.w + static_cast<long long>(tl.kbeg + wk * 16 + 4 * t) * pitch + col_byte;  // next step to load
  const long long scale_delta = static_cast<long long>(sg.n >> 1) + (colload >> 4) - col_byte;
  const long long step_stride = static_cast<long long>(p.wk) * 16 * pitch;
  const long long pitch2 = 2 * pitch, pitch3 = 3 * pitch;

  // loads local step s (steps are loaded in increasing order, so a running pointer suffices)
  auto load_step = [&](Raw<MODE>& raw, int s) {
    const uint8_t* q0 = wq;
    wq += step_stride;
    if (tail_here && s == nsteps - 1) {
      const int r = tl.kbeg + (wk + s * p.wk) * 16 + 4 * t;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const bool ok = cvalid && r + i < tl.kend;
        if constexpr (MODE == kNvfp4) {
          raw.r[i] = ok ? Ldg64(q0 + i * pitch) : make_uint2(0, 0);
          raw.s[i] = ok ? Ldg8(q0 + i * pitch + scale_delta) : 0u;
        } else {
          raw.r[i] = ok ? Ldg128(q0 + i * pitch) : make_uint4(0, 0, 0, 0);
        }
      }
      return;
    }
    const uint8_t* q1 = q0 + pitch;
    const uint8_t* q2 = q0 + pitch2;
    const uint8_t* q3 = q0 + pitch3;
    if (!cvalid) {  // columns past the tile: nothing to stream, the sums are never stored
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if constexpr (MODE == kNvfp4) {
          raw.r[i] = make_uint2(0, 0);
          raw.s[i] = 0u;
        } else {
          raw.r[i] = make_uint4(0, 0, 0, 0);
        }
      }
      return;
    }
    if constexpr (MODE == kNvfp4) {
      raw.r[0] = Ldg64(q0);
      raw.r[1] = Ldg64(q1);
      raw.r[2] = Ldg64(q2);
      raw.r[3] = Ldg64(q3);
      raw.s[0] = Ldg8(q0 + scale_delta);
      raw.s[1] = Ldg8(q1 + scale_delta);
      raw.s[2] = Ldg8(q2 + scale_delta);
      raw.s[3] = Ldg8(q3 + scale_delta);
    } else {
      raw.r[0] = Ldg128(q0);
      raw.r[1] = Ldg128(q1);
      raw.r[2] = Ldg128(q2);
      raw.r[3] = Ldg128(q3);
    }
  };

  // x first (unless it is still the predecessor kernel's to write): its copies then do not queue behind the weights
  uint16_t* xs = reinterpret_cast<uint16_t*>(smem + p.ring_bytes);
  const bool x_async = !FUSE && XRowsAre16ByteAligned(p);
  if (x_async && !p.pdl_wait) {
    XCopyIssue(p, tl, xs);
    CpAsyncCommit();
  }
  // weights do not depend on the predecessor kernel: get the first k-steps in flight, then wait
  Raw<MODE> buf[D];
#pragma unroll
  for (int d = 0; d < D; ++d) {
    if (warp_has_cols && d < nsteps) load_step(buf[d], d);
  }
  Stamp(p, 1);
  if (p.pdl_wait) GridDependencyWait();

  bool slow;
  if (x_async) {
    if (p.pdl_wait) {
      XCopyIssue(p, tl, xs);
      CpAsyncCommit();
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    slow = StageXConvert<MODE>(p, tl, xs, sh);
  } else {
    slow = StageX<MODE, false, false, FUSE>(p, tl, xs, sh);
  }
  Stamp(p, 2);

  float acc[NM][4];
#pragma unroll
  for (int j = 0; j < NM; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[j][e] = 0.f;

  const uint32_t xs_addr = SmemAddr(xs) + static_cast<uint32_t>((g * p.xpitch + 4 * t) * 2);
  const bool has_row = g < p.M;
  if (warp_has_cols) {
    for (int base = 0; base < nsteps; base += D) {
#pragma unroll
      for (int d = 0; d < D; ++d) {
        const int s = base + d;
        if (s < nsteps) {
          uint32_t b0 = 0, b1 = 0;
          if (has_row) {
            const uint2 xv = Lds64(xs_addr + static_cast<uint32_t>(wk + s * p.wk) * 32u);
            b0 = xv.x;
            b1 = xv.y;
          }
          if constexpr (MODE == kBf16) {
            ComputeStep<MODE, false>(acc, buf[d], b0, b1);
          } else {
            if (slow) {
              ComputeStep<MODE, true>(acc, buf[d], b0, b1);
            } else {
              ComputeStep<MODE, false>(acc, buf[d], b0, b1);
            }
          }
          if (s + D < nsteps) load_step(buf[d], s + D);
        }
      }
    }
  }
  Stamp(p, 3);
  if (p.trigger == 2) GridLaunchDependents();
  __syncthreads();
  Stamp(p, 4);
  Epilogue<MODE, 1, FUSE>(p, tl, acc, smem, sh, warp_has_cols);
  Stamp(p, 5);
}

// ------------------------------------------------------------------------------ tcgen05 kernel
// NVFP4 only.  The warp rings, the dequantisation and the epilogue are those of the direct kernel;
// the MMAs move from the legacy mma.sync pipe (measured: busy 62 % of all cycles and the first
// limiter of the direct kernel) to tcgen05.mma with the accumulators in tensor memory:
//   * warps come in groups of four side by side in N (a warpgroup, 512 columns); warp q of a group
//     can only touch TMEM lanes [32 q, 32 q + 32), so the four warps together fill the 128 lanes of
//     an A tile.  Per k-step a warp stores its eight 16-column x 16-row fragments with two
//     tcgen05.st.16x256b.x4 - that shape has exactly the register layout of the mma.sync A
//     fragment - into four A tiles (fragment j goes to tile j / 2, lanes 16 (j % 2) + ...).
//   * x is staged as the K-major no-swizzle B operand (8 rows x 16 k per step; rows 8..15 of the
//     N = 16 instruction alias the next step's bytes and land in accumulator columns nobody reads).
//   * one extra warp issues, in increasing k order, four M128 N16 K16 MMAs per warpgroup k-step and
//     commits them to the mbarrier that frees the A buffer (three buffers per warpgroup).  All K
//     groups of a column group accumulate into the same TMEM tile, so the sum over K runs in
//     k order whatever wk is.
//   * tile columns past wn x 128 (at most 128 more) are handled by wk extra warps on the mma.sync
//     path, so that a tile does not have to be a multiple of 512 columns.
// Every wait on an mbarrier is bounded.
constexpr int kTcBuffers = 3;
constexpr int kTcSpin = 1 << 22;
constexpr int kTcMaxGroups = 8;  // warpgroups per CTA (TMEM: groups x buffers x 32 + 64 per column group <= 512)

__device__ __forceinline__ void MbarInit(uint32_t addr, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(addr), "r"(count) : "memory");
}
__device__ __forceinline__ void MbarArrive(uint32_t addr) {
  asm volatile("{ .reg .b64 st; mbarrier.arrive.shared::cta.b64 st, [%0]; }" ::"r"(addr) : "memory");
}
// false if the phase did not complete within the spin limit (the caller carries on; results are then wrong
// but nothing hangs)
__device__ __forceinline__ bool MbarWait(uint32_t addr, uint32_t parity) {
  uint32_t done = 0;
  for (int spin = 0; spin < kTcSpin && !done; ++spin) {
    asm volatile("{ .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(done)
                 : "r"(addr), "r"(parity)
                 : "memory");
  }
  return done != 0;
}
__device__ __forceinline__ void TcFenceBefore() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void TcFenceAfter() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

struct TcShared {
  unsigned long long full[kTcMaxGroups][kTcBuffers];   // 4 arrivals: the warps of the group stored their fragments
  unsigned long long empty[kTcMaxGroups][kTcBuffers];  // 1 arrival: the MMAs that read the buffer completed
  unsigned long long done;                             // 1 arrival: every MMA of the CTA completed
  uint32_t tmem_base;
  uint32_t fault;
};

// The A operand registers of the eight 16-column MMAs of one k-step (fr[j] = {a0, a1, a2, a3} of MMA j as
// ComputeStep would pass them to mma.sync).
template <bool SLOW>
__device__ __forceinline__ void Nvfp4Fragments(const Raw<kNvfp4, 1>& w, uint32_t (&fr)[8][4]) {
  const uint32_t s_ab = CvtE4m3x2(Prmt(w.s[0][0], w.s[0][1], 0x0040u));
  const uint32_t s_cd = CvtE4m3x2(Prmt(w.s[0][2], w.s[0][3], 0x0040u));
  const uint32_t a[2] = {w.r[0][0].x, w.r[0][0].y}, b[2] = {w.r[0][1].x, w.r[0][1].y};
  const uint32_t c[2] = {w.r[0][2].x, w.r[0][2].y}, d[2] = {w.r[0][3].x, w.r[0][3].y};
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    uint32_t e_ab[4], o_ab[4], e_cd[4], o_cd[4];
    CvtE2m1x8(BitSelect(a[i], b[i] << 4, 0x0F0F0F0Fu), e_ab);
    CvtE2m1x8(BitSelect(a[i] >> 4, b[i], 0x0F0F0F0Fu), o_ab);
    CvtE2m1x8(BitSelect(c[i], d[i] << 4, 0x0F0F0F0Fu), e_cd);
    CvtE2m1x8(BitSelect(c[i] >> 4, d[i], 0x0F0F0F0Fu), o_cd);
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
      fr[4 * i + q][0] = a0;
      fr[4 * i + q][1] = a1;
      fr[4 * i + q][2] = a2;
      fr[4 * i + q][3] = a3;
    }
  }
}

// Fragments `half`, `half` + 2, `half` + 4, `half` + 6 of a k-step into lanes [lane_base, lane_base + 16) of the
// four A tiles of a buffer (32 TMEM columns from `taddr`).  A 16x256b store takes, per 8-column tile,
// (row g: k 4t..4t+1), (row g: k 4t+2..4t+3), (row g + 8: ...), (row g + 8: ...) = a0, a2, a1, a3.
__device__ __forceinline__ void TcStoreHalf(uint32_t taddr, const uint32_t (&fr)[8][4], int half) {
  const uint32_t(&f0)[4] = fr[half], (&f1)[4] = fr[half + 2], (&f2)[4] = fr[half + 4], (&f3)[4] = fr[half + 6];
  asm volatile(
      "tcgen05.st.sync.aligned.16x256b.x4.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(
          taddr),
      "r"(f0[0]), "r"(f0[2]), "r"(f0[1]), "r"(f0[3]), "r"(f1[0]), "r"(f1[2]), "r"(f1[1]), "r"(f1[3]), "r"(f2[0]), "r"(f2[2]),
      "r"(f2[1]), "r"(f2[3]), "r"(f3[0]), "r"(f3[2]), "r"(f3[1]), "r"(f3[3])
      : "memory");
}

template <int DEPTH>
__global__ void __launch_bounds__(kMaxThreads, 1) SkinnyGemmTcKernel(const __grid_constant__ GemmParams p) {
  using S = DirectSlot<kNvfp4, 1>;
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ SharedScratch sh;
  __shared__ __align__(8) TcShared tc;

  if (p.trigger == 1) GridLaunchDependents();
  Stamp(p, 0);
  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int nd = p.wn * p.wk;        // dequantising warps feeding tcgen05
  const int ngroups = p.wn >> 2;     // column groups of 512
  const bool is_tc = warp < nd, is_issuer = warp == nd, is_legacy = warp > nd;
  const int wn = is_tc ? warp % p.wn : p.wn;                       // legacy warps own the column warp after the last
  const int wk = is_tc ? warp / p.wn : (is_legacy ? warp - nd - 1 : 0);
  const int q = wn & 3, ng = wn >> 2;                              // quadrant and column group of a TC warp
  const int unit = wk * ngroups + ng;                              // warpgroup index
  const Tile tl = LocateTile(p);
  const Segment& sg = p.seg[tl.seg];
  const int colwarp = tl.n0 + wn * 128;
  const bool warp_has_cols = !is_issuer && colwarp < tl.n1;
  const int ksteps = (tl.kslice + 15) >> 4;
  const int TNc = (p.wn + 1) * 128;

  if (tid == 0) {
    for (int u = 0; u < p.wk * ngroups; ++u)
      for (int b = 0; b < kTcBuffers; ++b) {
        MbarInit(SmemAddr(&tc.full[u][b]), 4);
        MbarInit(SmemAddr(&tc.empty[u][b]), 1);
      }
    MbarInit(SmemAddr(&tc.done), 1);
    tc.fault = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  const int d_cols = ngroups * 64;
  const int need_cols = d_cols + p.wk * ngroups * kTcBuffers * 32;
  const int alloc_cols = need_cols <= 32 ? 32 : need_cols <= 64 ? 64 : need_cols <= 128 ? 128 : need_cols <= 256 ? 256 : 512;
  if (is_issuer) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(SmemAddr(&tc.tmem_base)), "r"(alloc_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }

  Nvfp4Stream<DEPTH> st;
  st.Setup(p, tl, sg, colwarp, wk, SmemAddr(smem) + static_cast<uint32_t>(is_legacy ? nd + wk : warp) * (DEPTH * S::kBytes),
           warp_has_cols);
  // a TC warp without columns still takes part in the barrier protocol of its group
  const int proto_steps = (is_tc && ksteps > wk) ? (ksteps - wk + p.wk - 1) / p.wk : 0;
  if (!is_issuer) st.Prologue(p, tl, sg);
  if (p.pdl_wait) GridDependencyWait();
  Stamp(p, 1);

  uint16_t* xs = reinterpret_cast<uint16_t*>(smem + p.ring_bytes);
  const bool slow = p.fuse ? StageX<kNvfp4, true, true, true>(p, tl, xs, sh) : StageX<kNvfp4, true>(p, tl, xs, sh);
  TcFenceBefore();
  __syncthreads();
  TcFenceAfter();
  Stamp(p, 2);
  const uint32_t tmem = tc.tmem_base;

  float acc[8][4];  // legacy warps only
#pragma unroll
  for (int j = 0; j < 8; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[j][e] = 0.f;

  if (is_tc) {
    const uint32_t a_base = tmem + static_cast<uint32_t>(d_cols + unit * kTcBuffers * 32) + (static_cast<uint32_t>(32 * q) << 16);
    const uint32_t full0 = SmemAddr(&tc.full[unit][0]), empty0 = SmemAddr(&tc.empty[unit][0]);
    int b = 0, round = 0;  // buffer of step s and how many times the buffers were cycled
    auto publish = [&](const Raw<kNvfp4, 1>* raw) {
      uint32_t fr[8][4];
      if (raw != nullptr) {
        if (slow) {
          Nvfp4Fragments<true>(*raw, fr);
        } else {
          Nvfp4Fragments<false>(*raw, fr);
        }
      }
      if (round > 0 && !MbarWait(empty0 + b * 8, static_cast<uint32_t>((round - 1) & 1))) tc.fault = 1;
      if (raw != nullptr) {
        TcFenceAfter();
        const uint32_t ta = a_base + static_cast<uint32_t>(b * 32);
        TcStoreHalf(ta, fr, 0);
        TcStoreHalf(ta + (16u << 16), fr, 1);
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        TcFenceBefore();
      }
      __syncwarp();
      if (lane == 0) MbarArrive(full0 + b * 8);
      if (++b == kTcBuffers) {
        b = 0;
        ++round;
      }
    };
    if (warp_has_cols) {
      st.Run(p, tl, sg, [&](const Raw<kNvfp4, 1>& raw, int) { publish(&raw); });
    } else {
      for (int s = 0; s < proto_steps; ++s) publish(nullptr);
    }
  } else if (is_issuer) {
    if (lane == 0) {
      const uint32_t idesc = 0x10u | (2u << 17) | (8u << 24) | (slow ? ((1u << 7) | (1u << 10)) : 0u);
      const uint32_t xa = SmemAddr(xs);
      const int max_steps = (ksteps + p.wk - 1) / p.wk;
      int b = 0, round = 0;
      for (int s = 0; s < max_steps; ++s) {
        for (int wkI = 0; wkI < p.wk; ++wkI) {
          const int kk = wkI + s * p.wk;
          if (kk >= ksteps) break;
          // x tile of k-step kk: 256 bytes; K chunks 128 bytes apart; rows 8..15 alias the next 256 bytes
          const unsigned long long desc = static_cast<unsigned long long>(((xa + static_cast<uint32_t>(kk) * 256u) >> 4) & 0x3FFF) |
                                          (static_cast<unsigned long long>(128 >> 4) << 16) |
                                          (static_cast<unsigned long long>(256 >> 4) << 32) | (1ull << 46);
          for (int gi = 0; gi < ngroups; ++gi) {
            const int u = wkI * ngroups + gi;
            if (!MbarWait(SmemAddr(&tc.full[u][b]), static_cast<uint32_t>(round & 1))) tc.fault = 1;
            TcFenceAfter();
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const uint32_t d_t = tmem + static_cast<uint32_t>(gi * 64 + i * 16);
              const uint32_t a_t = tmem + static_cast<uint32_t>(d_cols + (u * kTcBuffers + b) * 32 + i * 8);
              asm volatile(
                  "{ .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                  " tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n}" ::"r"(d_t),
                  "r"(a_t), "l"(desc), "r"(idesc), "r"(kk > 0 ? 1 : 0), "r"(0)
                  : "memory");
            }
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                             SmemAddr(&tc.empty[u][b]))
                         : "memory");
          }
        }
        if (++b == kTcBuffers) {
          b = 0;
          ++round;
        }
      }
      asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(SmemAddr(&tc.done))
                   : "memory");
    }
    __syncwarp();
  } else {
    // mma.sync path for the tile's columns past the warpgroups
    const int x_row = g < p.M ? g : 0;
    uint32_t x_rd = SmemAddr(xs) + static_cast<uint32_t>(wk * 256 + (t >> 1) * 128 + x_row * 16 + (t & 1) * 8);
    const uint32_t x_step = static_cast<uint32_t>(p.wk) * 256u;
    st.Run(p, tl, sg, [&](const Raw<kNvfp4, 1>& raw, int) {
      const uint2 xv = Lds64(x_rd);
      x_rd += x_step;
      if (slow) {
        ComputeStep<kNvfp4, true, 1>(acc, raw, xv.x, xv.y);
      } else {
        ComputeStep<kNvfp4, false, 1>(acc, raw, xv.x, xv.y);
      }
    });
  }
  Stamp(p, 3);
  if (p.trigger == 2) GridLaunchDependents();
  // all MMAs done before anybody reads the accumulators or reuses the ring as `red`
  if (!MbarWait(SmemAddr(&tc.done), 0)) tc.fault = 1;
  TcFenceAfter();
  __syncthreads();
  Stamp(p, 4);

  float* red = reinterpret_cast<float*>(smem);
  const int M = p.M;
  if (is_tc) {
    if (wk == 0) {
      // accumulators of this warp's 128 columns: TMEM lane 32 q + L of the group's four tiles, column n = x row
      uint32_t d[4][8];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint32_t ta = tmem + static_cast<uint32_t>(ng * 64 + i * 16) + (static_cast<uint32_t>(32 * q) << 16);
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                     : "=r"(d[i][0]), "=r"(d[i][1]), "=r"(d[i][2]), "=r"(d[i][3]), "=r"(d[i][4]), "=r"(d[i][5]), "=r"(d[i][6]),
                       "=r"(d[i][7])
                     : "r"(ta));
      }
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      const int half = lane >> 4, l = lane & 15;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int j = 2 * i + half;  // fragment = MMA index of the direct kernel: columns 16 g' + 2 j (+ 1)
        const int c = wn * 128 + (l < 8 ? 16 * l + 2 * j : 16 * (l - 8) + 2 * j + 1);
#pragma unroll
        for (int m = 0; m < kMaxRows; ++m)
          if (m < M) red[m * TNc + RedCol(c, m)] = __uint_as_float(d[i][m]);
      }
    } else {
      for (int m = 0; m < M; ++m)
        for (int c = lane; c < 128; c += 32) red[(wk * M + m) * TNc + wn * 128 + c] = 0.f;
    }
  } else if (is_legacy) {
    if (warp_has_cols) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int cl = wn * 128 + g * 16 + 2 * j;
        const int m0 = 2 * t, m1 = 2 * t + 1;
        if (m0 < M) *reinterpret_cast<float2*>(&red[(wk * M + m0) * TNc + RedCol(cl, m0)]) = make_float2(acc[j][0], acc[j][2]);
        if (m1 < M) *reinterpret_cast<float2*>(&red[(wk * M + m1) * TNc + RedCol(cl, m1)]) = make_float2(acc[j][1], acc[j][3]);
      }
    } else {
      for (int m = 0; m < M; ++m)
        for (int c = lane; c < 128; c += 32) red[(wk * M + m) * TNc + wn * 128 + c] = 0.f;
    }
  }
  TcFenceBefore();
  __syncthreads();
  if (is_issuer) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(alloc_cols) : "memory");
  }
  if (p.fuse) {
    EpilogueTail<kNvfp4, true>(p, tl, smem, sh, p.wk, TNc);
  } else {
    EpilogueTail<kNvfp4>(p, tl, smem, sh, p.wk, TNc);
  }
  Stamp(p, 5);
}

// ------------------------------------------------------------------------------ ring kernel
template <int MODE>
__global__ void __launch_bounds__(kRingThreads, 2) SkinnyGemmRingKernel(const __grid_constant__ GemmParams p) {
  using G = Geom<MODE>;
  constexpr int NM = G::kMmas;
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ SharedScratch sh;

  if (p.trigger == 1) GridLaunchDependents();

  const int tid = threadIdx.x;
  const int nthreads = blockDim.x;
  const int warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int wn = warp % p.wn, wk = warp / p.wn;
  const Tile tl = LocateTile(p);
  const Segment& sg = p.seg[tl.seg];
  const int N = sg.n, n0 = tl.n0, n1 = tl.n1, kbeg = tl.kbeg, kend = tl.kend, kslice = tl.kslice;
  const long long pitch = sg.pitch;
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
        const uint32_t dst = slot + row * TB + ((((bo >> 4) ^ (((row >> 2) & 3) << 1 & swz_mask)) << 4) | (bo & 15));
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

  uint16_t* xs = reinterpret_cast<uint16_t*>(smem + p.ring_bytes);
  const bool slow = p.fuse ? StageX<MODE, false, true, true>(p, tl, xs, sh) : StageX<MODE>(p, tl, xs, sh);

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
    w_off = 4 * t * TB + (((chunk ^ ((t << 1) & swz_mask)) << 4) | ((g & 1) << 3));
    s_off = static_cast<uint32_t>(R * TB + 4 * t * SRB + sphase + wn * 8 + g);
  } else {
    const uint32_t chunk = static_cast<uint32_t>(wn * 8 + g);
    w_off = 4 * t * TB + ((chunk ^ ((t << 1) & swz_mask)) << 4);
  }
  const uint32_t xs_addr = SmemAddr(xs) + static_cast<uint32_t>((g * p.xpitch + 4 * t) * 2);
  const bool has_row = g < p.M;

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
        Raw<MODE> raw;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          if constexpr (MODE == kNvfp4) {
            raw.r[0][i] = Lds64(wa + static_cast<uint32_t>(i) * TB);
          } else {
            raw.r[i] = Lds128(wa + static_cast<uint32_t>(i) * TB);
          }
        }
        if constexpr (MODE == kNvfp4) {
          const uint32_t sa = slot + static_cast<uint32_t>(step_in_stage * 16) * SRB + s_off;
#pragma unroll
          for (int i = 0; i < 4; ++i) raw.s[0][i] = Lds8(sa + static_cast<uint32_t>(i) * SRB);
        }
        if constexpr (MODE == kBf16) {
          ComputeStep<MODE, false>(acc, raw, b0, b1);
        } else {
          if (slow) {
            ComputeStep<MODE, true>(acc, raw, b0, b1);
          } else {
            ComputeStep<MODE, false>(acc, raw, b0, b1);
          }
        }
      }
    }
  }
  CpAsyncWait(0);
  if (p.trigger == 2) GridLaunchDependents();
  __syncthreads();
  if (p.fuse) {
    Epilogue<MODE, 1, true>(p, tl, acc, smem, sh, warp_has_cols);
  } else {
    Epilogue<MODE>(p, tl, acc, smem, sh, warp_has_cols);
  }
}

// Largest dynamic shared-memory request any of the kernels accepts: the opt-in limit of the
// device minus the kernels' static shared memory.
int g_max_dynamic_smem = 0;

template <typename K>
cudaError_t ConfigureKernel(K kernel) {
  int dev = 0, optin = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return err;
  err = cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
  if (err != cudaSuccess) return err;
  cudaFuncAttributes fa;
  err = cudaFuncGetAttributes(&fa, kernel);
  if (err != cudaSuccess) return err;
  const int dyn = optin - static_cast<int>(fa.sharedSizeBytes);
  if (g_max_dynamic_smem == 0 || dyn < g_max_dynamic_smem) g_max_dynamic_smem = dyn;
  return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, dyn);
}

template <int MODE>
cudaError_t ConfigureDirect() {
  cudaError_t err = ConfigureKernel(SkinnyGemmDirectKernel<MODE, 2>);
  if (err == cudaSuccess) err = ConfigureKernel(SkinnyGemmDirectKernel<MODE, 3>);
  if (err == cudaSuccess) err = ConfigureKernel(SkinnyGemmDirectKernel<MODE, 4>);
  if (err == cudaSuccess) err = ConfigureKernel(SkinnyGemmDirectKernel<MODE, 2, true>);
  if (err == cudaSuccess) err = ConfigureKernel(SkinnyGemmDirectKernel<MODE, 3, true>);
  if (err == cudaSuccess) err = ConfigureKernel(SkinnyGemmDirectKernel<MODE, 4, true>);
  return err;
}

// the direct kernel is compiled for rings of 4, 6 and 8 k-steps (2, 3, 4 pairs)
template <int MODE>
cudaError_t LaunchDirect(const cudaLaunchConfig_t* cfg, int stages, const GemmParams& p) {
  if (p.fuse) {
    switch (stages) {
      case 4: return cudaLaunchKernelEx(cfg, SkinnyGemmDirectKernel<MODE, 2, true>, p);
      case 6: return cudaLaunchKernelEx(cfg, SkinnyGemmDirectKernel<MODE, 3, true>, p);
      case 8: return cudaLaunchKernelEx(cfg, SkinnyGemmDirectKernel<MODE, 4, true>, p);
      default: return cudaErrorInvalidValue;
    }
  }
  switch (stages) {
    case 4: return cudaLaunchKernelEx(cfg, SkinnyGemmDirectKernel<MODE, 2>, p);
    case 6: return cudaLaunchKernelEx(cfg, SkinnyGemmDirectKernel<MODE, 3>, p);
    case 8: return cudaLaunchKernelEx(cfg, SkinnyGemmDirectKernel<MODE, 4>, p);
    default: return cudaErrorInvalidValue;
  }
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
  if constexpr (MODE != kNvfp4) {
    if (plan.direct == 2) {
      return p.fuse ? cudaLaunchKernelEx(&cfg, SkinnyGemmRegKernel<MODE, true>, p) : cudaLaunchKernelEx(&cfg, SkinnyGemmRegKernel<MODE>, p);
    }
  }
  if (plan.direct) {
    if constexpr (MODE == kNvfp4) {
      if (plan.tc) {
        switch (plan.stages) {
          case 3: return cudaLaunchKernelEx(&cfg, SkinnyGemmTcKernel<3>, p);
          case 4: return cudaLaunchKernelEx(&cfg, SkinnyGemmTcKernel<4>, p);
          case 6: return cudaLaunchKernelEx(&cfg, SkinnyGemmTcKernel<6>, p);
          default: return cudaErrorInvalidValue;
        }
      }
    }
    return LaunchDirect<MODE>(&cfg, plan.stages, p);
  }
  return cudaLaunchKernelEx(&cfg, SkinnyGemmRingKernel<MODE>, p);
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

// Co-resident clusters (CTAs for cluster == 1) of one launch shape on the current device; cached.
int QueryMaxActiveClusters(int mode, int direct, int threads, size_t smem, int cluster) {
  static std::mutex mu;
  static std::map<std::tuple<int, int, int, size_t, int>, int> cache;
  const size_t smem_key = (smem + 4095) & ~static_cast<size_t>(4095);
  const auto key = std::make_tuple(mode, direct, threads, smem_key, cluster);
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it != cache.end()) return it->second;
  const void* fn = nullptr;
  switch (mode) {
    case kBf16:
      fn = direct == 4 ? (const void*)SkinnyGemmRegKernel<kBf16>
           : direct    ? (const void*)SkinnyGemmDirectKernel<kBf16, 2>
                       : (const void*)SkinnyGemmRingKernel<kBf16>;
      break;
    case kFp8:
      fn = direct == 4 ? (const void*)SkinnyGemmRegKernel<kFp8>
           : direct    ? (const void*)SkinnyGemmDirectKernel<kFp8, 2>
                       : (const void*)SkinnyGemmRingKernel<kFp8>;
      break;
    default:
      fn = direct == 3   ? (const void*)SkinnyGemmTcKernel<4>
           : direct >= 1 ? (const void*)SkinnyGemmDirectKernel<kNvfp4, 2>
                         : (const void*)SkinnyGemmRingKernel<kNvfp4>;
      break;
  }
  int result = 0;
  if (g_max_dynamic_smem > 0 && smem_key > static_cast<size_t>(g_max_dynamic_smem)) {
    result = 0;
  } else if (cluster <= 1) {
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fn, threads, smem_key) == cudaSuccess) {
      result = per_sm * DeviceSmCount();
    }
  } else {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1, static_cast<unsigned>(cluster), 1);
    cfg.blockDim = dim3(static_cast<unsigned>(threads), 1, 1);
    cfg.dynamicSmemBytes = smem_key;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = static_cast<unsigned>(cluster);
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, fn, &cfg) == cudaSuccess) result = n;
  }
  cudaGetLastError();
  cache[key] = result;
  return result;
}

// Raises the dynamic shared-memory limit of the kernels once per process.  Called from the
// *_create entry points, i.e. outside any stream capture.
int g_configured_device = -1;

cudaError_t ConfigureSkinnyGemmKernels() {
  static std::once_flag once;
  static cudaError_t status = cudaSuccess;
  std::call_once(once, [] {
    status = cudaGetDevice(&g_configured_device);
    if (status == cudaSuccess) status = ConfigureDirect<kBf16>();
    if (status == cudaSuccess) status = ConfigureDirect<kFp8>();
    if (status == cudaSuccess) status = ConfigureDirect<kNvfp4>();
    if (status == cudaSuccess) status = ConfigureKernel(SkinnyGemmRegKernel<kBf16>);
    if (status == cudaSuccess) status = ConfigureKernel(SkinnyGemmRegKernel<kFp8>);
    if (status == cudaSuccess) status = ConfigureKernel(SkinnyGemmRegKernel<kBf16, true>);
    if (status == cudaSuccess) status = ConfigureKernel(SkinnyGemmRegKernel<kFp8, true>);
    if (status == cudaSuccess) status = ConfigureKernel(SkinnyGemmTcKernel<3>);
    if (status == cudaSuccess) status = ConfigureKernel(SkinnyGemmTcKernel<4>);
    if (status == cudaSuccess) status = ConfigureKernel(SkinnyGemmTcKernel<6>);
    if (status == cudaSuccess) status = ConfigureKernel(SkinnyGemmRingKernel<kBf16>);
    if (status == cudaSuccess) status = ConfigureKernel(SkinnyGemmRingKernel<kFp8>);
    if (status == cudaSuccess) status = ConfigureKernel(SkinnyGemmRingKernel<kNvfp4>);
  });
  return status;
}

cudaError_t LaunchSkinnyGemm(int mode, GemmParams& p, const Plan& plan, cudaStream_t stream) {
  // The kernels' attributes (shared-memory limits, co-resident cluster counts, SM count) were set up for one
  // device: one process drives one GPU, and a call with another device current is refused rather than launched
  // with the wrong limits.
  int dev = -1;
  if (g_configured_device >= 0 && (cudaGetDevice(&dev) != cudaSuccess || dev != g_configured_device)) return cudaErrorInvalidDevice;
  const ModeGeom geom = GeomOf(mode, plan.direct ? plan.wide : 1);
  p.wn = plan.wn;
  p.wk = plan.wk;
  p.ks = plan.ks;
  p.stages = plan.stages;
  p.cluster = plan.cluster;
  p.gran = plan.gran;
  p.tile_row_bytes = plan.wn * geom.bytes_per_warp;
  p.scale_row_bytes = mode == kNvfp4 ? (plan.wn * 8 + 16 + 15) & ~15 : 0;
  const int R = plan.rows_per_stage();
  p.stage_bytes = (R * (p.tile_row_bytes + p.scale_row_bytes) + 127) & ~127;
  const int TNc = PlanMaxCols(plan, mode);
  const int red_bytes = (plan.wk + (plan.cluster > 1 ? 1 : 0)) * p.M * TNc * 4;
  const int direct_slot = plan.tc ? DirectSlotBytes(mode, 1) : RingSlotBytes(mode);
  const int ring_warps = plan.tc ? plan.wn * plan.wk + plan.wk : plan.wn * plan.wk;
  const int ring = plan.direct == 2 ? 0 : plan.direct ? ring_warps * plan.stages * direct_slot : plan.stages * p.stage_bytes;
  p.ring_bytes = (std::max(ring, red_bytes) + 127) & ~127;
  const int ksteps = (p.K + 15) / 16;
  const int kslice_max = ((ksteps + plan.cluster - 1) / plan.cluster) * 16;
  p.xpitch = ((kslice_max + 63) & ~63) + 16;  // 32 bytes off a 128-byte multiple: rows land in distinct banks
  size_t smem = static_cast<size_t>(p.ring_bytes) + static_cast<size_t>(p.M) * p.xpitch * 2;
  if (plan.tc) {
    // x as the MMA operand: 256 bytes per k-step plus one spare step; at least 120 KB so that two CTAs,
    // each allocating up to all of tensor memory, can never share an SM
    smem = static_cast<size_t>(p.ring_bytes) + static_cast<size_t>(kslice_max / 16 + 1) * 256;
    if (smem < 120 * 1024) smem = 120 * 1024;
  }
  if (g_max_dynamic_smem > 0 && smem > static_cast<size_t>(g_max_dynamic_smem)) return cudaErrorInvalidConfiguration;
  p.scales_l1 = smem <= kL1UsableSmem ? 1 : 0;
  p.tail_groups = plan.tail;
  // K slices per shared group: at most kMaxTailSplit, one per CTA where there are enough CTAs, else one per idle warp
  p.tail_split = 1;
  p.tail_stride = 0;
  if (plan.tail > 0) {
    const int ctas = plan.tiles[0];
    if (ctas >= 2 * plan.tail) {
      p.tail_split = std::min(kMaxTailSplit, ctas / plan.tail);
      p.tail_stride = ctas / (plan.tail * p.tail_split);
    } else {
      p.tail_split = std::max(1, std::min(kMaxTailSplit, ctas * plan.wk / plan.tail));
    }
  }
  if (plan.tail > 0 && (!p.lm || p.lm_tail == nullptr || p.nseg != 1 || plan.cluster != 1)) return cudaErrorInvalidValue;
  int tiles = 0;
  for (int s = 0; s < p.nseg; ++s) {
    p.seg[s].tile_begin = tiles;
    p.seg[s].tiles = plan.tiles[s];
    p.seg[s].tail_cols = (s == 0) ? plan.tail * 128 : 0;
    p.seg[s].granules = (p.seg[s].n - p.seg[s].tail_cols + plan.gran - 1) / plan.gran;
    if (plan.tiles[s] < 1 || plan.tiles[s] > 65535) return cudaErrorInvalidValue;
    p.seg[s].gran_quot = p.seg[s].granules / plan.tiles[s];
    p.seg[s].gran_rem = p.seg[s].granules % plan.tiles[s];
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
