// DequantWeightBf16 for B200: a column slice of a BF16 / FP8 E4M3FN / block-16 NVFP4 weight as
// BF16, optionally multiplied by a per-output-column FP32 scale, split over up to eight outputs.
// FP8: bf16_rn(float(q) * s[col]).  NVFP4: bf16_rn(e2m1 * e4m3_block_scale * s[col]) where the
// first product is exact.  BF16: copy.  Each thread produces 8 consecutive columns of one row
// (one 16-byte store); the grid is sized in multiples of the SM count and strides over the rest.
// A write-bound stream: 2 bytes out per weight against 2, 1 or 0.5625 bytes in.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include <algorithm>

#include "qfg_internal.h"

namespace qfg {
namespace {

__device__ __forceinline__ uint32_t PackBf16(float a, float b) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&v);
}

__device__ __forceinline__ float E4m3ToFloat(uint32_t byte) {
  const __half_raw hr = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(byte), __NV_E4M3);
  return __half2float(*reinterpret_cast<const __half*>(&hr));
}

// 2 * |e2m1| as a float times half the block scale, sign from nibble bit 3 (so 0x8 is -0).
__device__ __forceinline__ float E2m1Scaled(uint32_t nib, float s_half) {
  const uint32_t mag2 = (0xC8643210u >> ((nib & 7u) * 4u)) & 0xFu;
  const float f = static_cast<float>(mag2) * s_half;
  return __uint_as_float(__float_as_uint(f) ^ ((nib & 8u) << 28));
}

template <int MODE, bool ALIGNED>
__global__ void __launch_bounds__(256) DequantKernel(const DequantParams p) {
  const int chunks_per_row = p.N / 8;
  const long long total = static_cast<long long>(p.K) * chunks_per_row;
  for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int r = static_cast<int>(idx / chunks_per_row);
    const int col = static_cast<int>(idx % chunks_per_row) * 8;
    const int src_col = p.col_offset + col;
    float sc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) sc[i] = p.w_scale != nullptr ? __ldg(p.w_scale + col + i) : 1.f;
    uint4 o;
    if constexpr (MODE == kBf16) {
      const uint16_t* src = reinterpret_cast<const uint16_t*>(p.w) + static_cast<size_t>(r) * p.row_stride + src_col;
      if constexpr (ALIGNED) {
        o = __ldg(reinterpret_cast<const uint4*>(src));
      } else {
        uint16_t e[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) e[i] = __ldg(src + i);
        o = make_uint4(e[0] | (e[1] << 16), e[2] | (e[3] << 16), e[4] | (e[5] << 16), e[6] | (e[7] << 16));
      }
    } else if constexpr (MODE == kFp8) {
      const uint8_t* src = p.w + static_cast<size_t>(r) * p.row_stride + src_col;
      uint8_t q[8];
      if constexpr (ALIGNED) {
        const uint2 raw = __ldg(reinterpret_cast<const uint2*>(src));
        *reinterpret_cast<uint2*>(q) = raw;
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) q[i] = __ldg(src + i);
      }
      float f[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = E4m3ToFloat(q[i]) * sc[i];
      o = make_uint4(PackBf16(f[0], f[1]), PackBf16(f[2], f[3]), PackBf16(f[4], f[5]), PackBf16(f[6], f[7]));
    } else {
      const size_t row_bytes = static_cast<size_t>(p.row_stride) * 9 / 16;
      const uint8_t* row_p = p.w + static_cast<size_t>(r) * row_bytes;
      uint32_t pack8;
      if constexpr (ALIGNED) {
        pack8 = __ldg(reinterpret_cast<const uint32_t*>(row_p + (src_col >> 1)));
      } else {
        const uint8_t* s = row_p + (src_col >> 1);
        pack8 = __ldg(s) | (__ldg(s + 1) << 8) | (__ldg(s + 2) << 16) | (static_cast<uint32_t>(__ldg(s + 3)) << 24);
      }
      const float s_half = E4m3ToFloat(__ldg(row_p + (p.row_stride >> 1) + (src_col >> 4))) * 0.5f;
      float f[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = E2m1Scaled((pack8 >> (4 * i)) & 0xFu, s_half) * sc[i];
      o = make_uint4(PackBf16(f[0], f[1]), PackBf16(f[2], f[3]), PackBf16(f[4], f[5]), PackBf16(f[6], f[7]));
    }
    int j = 0;
#pragma unroll
    for (int i = 1; i < kMaxOut; ++i) {
      if (i < p.num_outs && col >= p.col_begin[i]) j = i;
    }
    *reinterpret_cast<uint4*>(p.out[j] + static_cast<size_t>(r) * p.width[j] + (col - p.col_begin[j])) = o;
  }
}

template <int MODE>
void LaunchMode(const DequantParams& p, int blocks, cudaStream_t stream) {
  if (p.aligned) {
    DequantKernel<MODE, true><<<blocks, 256, 0, stream>>>(p);
  } else {
    DequantKernel<MODE, false><<<blocks, 256, 0, stream>>>(p);
  }
}

}  // namespace

cudaError_t LaunchDequant(const DequantParams& p, cudaStream_t stream) {
  const long long total = static_cast<long long>(p.K) * (p.N / 8);
  if (total <= 0) return cudaSuccess;
  const int sms = DeviceSmCount();
  const long long want = (total + 255) / 256;
  const int blocks = static_cast<int>(std::min<long long>(want, static_cast<long long>(sms) * 32));
  switch (p.mode) {
    case kBf16: LaunchMode<kBf16>(p, blocks, stream); break;
    case kFp8: LaunchMode<kFp8>(p, blocks, stream); break;
    case kNvfp4: LaunchMode<kNvfp4>(p, blocks, stream); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

}  // namespace qfg
