// UntileHcBf16: the pre-tiled hyper-connection weight [160, 20480] back to row-major BF16,
// [10240, 320] (kind 0) or [320, 10240] (kind 1), dequantising FP8 E4M3FN with a per-output-column
// scale on the way.  Follows UntileHcBf16Kernel of the reference (src/fused_gemm/fused_gemm.cu:979-1011).
//
// The tensor is 204800 groups of 16 consecutive elements; the op is a permutation of groups:
//   kind 0: out[(s*10 + i)*128 + r][16 j + e] = in[s*20 + j][(i*128 + r)*16 + e]     s<8, j<20, i<10, r<128
//   kind 1: out[i*32 + r][(c*160 + h)*16 + e] = in[h][((i*32 + r)*4 + c)*16 + e]     h<160, i<10, r<32, c<4
// (the layout the reference's test builds with view(8,10,128,20,2,8).permute(0,3,1,2,4,5),
// tests/test_load.py:404-409).  6.5 MB in, 6.5 MB out: one thread per output group so that the 32-byte
// stores of a warp are contiguous; bound by HBM and far too small to matter next to the GEMMs.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "qfg_internal.h"

namespace qfg {
namespace {

constexpr int kGroups = 204800;

__device__ __forceinline__ int SourceGroup(int og, int kind) {
  if (kind == 0) {
    const int j = og % 20, row = og / 20;
    const int r = row & 127, t = row >> 7;
    const int i = t % 10, s = t / 10;
    return ((s * 20 + j) * 10 + i) * 128 + r;
  }
  const int cg = og % 640, row = og / 640;
  const int c = cg / 160, h = cg % 160;
  return (h * 320 + row) * 4 + c;
}

// eight E4M3 bytes (two words) times the scales of their columns, rounded once to BF16
__device__ __forceinline__ uint4 DequantEight(uint32_t lo, uint32_t hi, const float* scale, int col) {
  uint32_t out[4];
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    const uint32_t pair = ((p < 2 ? lo : hi) >> (16 * (p & 1))) & 0xFFFFu;
    uint32_t h2;
    asm("{ .reg .b16 h;\n cvt.u16.u32 h, %1;\n cvt.rn.f16x2.e4m3x2 %0, h;\n}" : "=r"(h2) : "r"(pair));
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h2));
    const float s0 = scale != nullptr ? scale[col + 2 * p] : 1.f, s1 = scale != nullptr ? scale[col + 2 * p + 1] : 1.f;
    const __nv_bfloat162 b = __floats2bfloat162_rn(f.x * s0, f.y * s1);
    out[p] = *reinterpret_cast<const uint32_t*>(&b);
  }
  return make_uint4(out[0], out[1], out[2], out[3]);
}

template <bool FP8>
__global__ void __launch_bounds__(256) UntileHcKernel(const uint4* __restrict__ src, uint4* __restrict__ dst,
                                                      const float* __restrict__ scale, int kind) {
  const int og = blockIdx.x * blockDim.x + threadIdx.x;
  if (og >= kGroups) return;
  const int sg = SourceGroup(og, kind);
  if constexpr (!FP8) {
    dst[2 * og] = __ldg(src + 2 * sg);
    dst[2 * og + 1] = __ldg(src + 2 * sg + 1);
  } else {
    const int col = (kind == 0 ? og % 20 : og % 640) * 16;
    const uint4 raw = __ldg(src + sg);
    dst[2 * og] = DequantEight(raw.x, raw.y, scale, col);
    dst[2 * og + 1] = DequantEight(raw.z, raw.w, scale, col + 8);
  }
}

}  // namespace

cudaError_t LaunchUntileHc(bool fp8, const void* w, void* out, const float* scale, int kind, cudaStream_t stream) {
  const int blocks = (kGroups + 255) / 256;
  if (fp8) {
    UntileHcKernel<true><<<blocks, 256, 0, stream>>>(static_cast<const uint4*>(w), static_cast<uint4*>(out), scale, kind);
  } else {
    UntileHcKernel<false><<<blocks, 256, 0, stream>>>(static_cast<const uint4*>(w), static_cast<uint4*>(out), nullptr, kind);
  }
  return cudaGetLastError();
}

}  // namespace qfg
