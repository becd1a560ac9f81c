// DequantWeightBf16 for B200: a column slice of a BF16 / FP8 E4M3FN / block-16 NVFP4 weight as
// BF16, optionally multiplied by a per-output-column FP32 scale, split over up to eight outputs.
// FP8: bf16_rn(float(q) * s[col]).  NVFP4: bf16_rn(e2m1 * e4m3_block_scale * s[col]) where the
// first product is exact.  BF16: copy.  Each thread produces 8 consecutive columns of four consecutive rows
// (16-byte stores); the grid is sized in multiples of the SM count and strides over the rest.
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

// The bytes of one 8-column chunk of one row as stored: 16 (BF16), 8 (FP8) or 4 + the block's scale byte (NVFP4).
struct RawChunk {
  uint4 v;
  uint32_t s;
};

template <int MODE, bool ALIGNED>
__device__ __forceinline__ RawChunk LoadChunk(const DequantParams& p, int r, int src_col) {
  RawChunk raw;
  raw.v = make_uint4(0, 0, 0, 0);
  raw.s = 0;
  if constexpr (MODE == kBf16) {
    const uint16_t* src = reinterpret_cast<const uint16_t*>(p.w) + static_cast<size_t>(r) * p.row_stride + src_col;
    if constexpr (ALIGNED) {
      raw.v = __ldg(reinterpret_cast<const uint4*>(src));
    } else {
      uint32_t e[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) e[i] = __ldg(src + i);
      raw.v = make_uint4(e[0] | (e[1] << 16), e[2] | (e[3] << 16), e[4] | (e[5] << 16), e[6] | (e[7] << 16));
    }
  } else if constexpr (MODE == kFp8) {
    const uint8_t* src = p.w + static_cast<size_t>(r) * p.row_stride + src_col;
    if constexpr (ALIGNED) {
      const uint2 q = __ldg(reinterpret_cast<const uint2*>(src));
      raw.v.x = q.x;
      raw.v.y = q.y;
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        raw.v.x |= static_cast<uint32_t>(__ldg(src + i)) << (8 * i);
        raw.v.y |= static_cast<uint32_t>(__ldg(src + 4 + i)) << (8 * i);
      }
    }
  } else {
    const size_t row_bytes = static_cast<size_t>(p.row_stride) * 9 / 16;
    const uint8_t* row_p = p.w + static_cast<size_t>(r) * row_bytes;
    const uint8_t* q = row_p + (src_col >> 1);
    if constexpr (ALIGNED) {
      raw.v.x = __ldg(reinterpret_cast<const uint32_t*>(q));
    } else {
      raw.v.x = __ldg(q) | (__ldg(q + 1) << 8) | (__ldg(q + 2) << 16) | (static_cast<uint32_t>(__ldg(q + 3)) << 24);
    }
    raw.s = __ldg(row_p + (p.row_stride >> 1) + (src_col >> 4));
  }
  return raw;
}

template <int MODE>
__device__ __forceinline__ uint4 ConvertChunk(const RawChunk& raw, const float (&sc)[8]) {
  if constexpr (MODE == kBf16) {
    return raw.v;
  } else {
    float f[8];
    if constexpr (MODE == kFp8) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        f[i] = E4m3ToFloat((raw.v.x >> (8 * i)) & 0xFFu) * sc[i];
        f[4 + i] = E4m3ToFloat((raw.v.y >> (8 * i)) & 0xFFu) * sc[4 + i];
      }
    } else {
      // byte q holds columns 2q (low nibble) and 2q + 1; E2M1 is exact in FP16 and its product with the
      // E4M3 block scale is exact in FP32 (4 + 4 significant bits): the value of the
      // reference's scaled look-up (skinny_gemm.cuh:161, used at fused_gemm.cu:232-233), -0 for nibble 0x8 included
      uint32_t h[4];
      CvtE2m1x8(raw.v.x, h);
      const float s = E4m3ToFloat(raw.s);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 v = __half22float2(*reinterpret_cast<const __half2*>(&h[q]));
        f[2 * q] = (v.x * s) * sc[2 * q];
        f[2 * q + 1] = (v.y * s) * sc[2 * q + 1];
      }
    }
    return make_uint4(PackBf16(f[0], f[1]), PackBf16(f[2], f[3]), PackBf16(f[4], f[5]), PackBf16(f[6], f[7]));
  }
}

// A thread owns one 8-column chunk of kDequantRows consecutive rows: all of their loads are issued before the
// first conversion, which keeps four times the bytes of the one-row form in flight (the kernel is a pure
// stream and was latency-bound with one 4-byte load per thread), and w_scale is read once for the rows.
constexpr int kDequantRows = 4;

template <int MODE, bool ALIGNED>
__global__ void __launch_bounds__(256) DequantKernel(const DequantParams p) {
  const int chunks_per_row = p.N / 8;
  const int row_groups = (p.K + kDequantRows - 1) / kDequantRows;
  const long long total = static_cast<long long>(row_groups) * chunks_per_row;
  for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int rg = static_cast<int>(idx / chunks_per_row);
    const int col = static_cast<int>(idx - static_cast<long long>(rg) * chunks_per_row) * 8;
    const int r0 = rg * kDequantRows;
    const int src_col = p.col_offset + col;
    RawChunk raw[kDequantRows];
#pragma unroll
    for (int i = 0; i < kDequantRows; ++i) {
      if (r0 + i < p.K) raw[i] = LoadChunk<MODE, ALIGNED>(p, r0 + i, src_col);
    }
    float sc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) sc[i] = 1.f;
    if constexpr (MODE != kBf16) {
      if (p.w_scale != nullptr) {
        if (p.scale_vec) {  // col is a multiple of 8: two aligned 16-byte loads
          const float4 a = __ldg(reinterpret_cast<const float4*>(p.w_scale + col));
          const float4 b = __ldg(reinterpret_cast<const float4*>(p.w_scale + col + 4));
          sc[0] = a.x, sc[1] = a.y, sc[2] = a.z, sc[3] = a.w, sc[4] = b.x, sc[5] = b.y, sc[6] = b.z, sc[7] = b.w;
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) sc[i] = __ldg(p.w_scale + col + i);
        }
      }
    }
    int j = 0;
#pragma unroll
    for (int i = 1; i < kMaxOut; ++i) {
      if (i < p.num_outs && col >= p.col_begin[i]) j = i;
    }
    uint16_t* dst = p.out[j] + static_cast<size_t>(r0) * p.width[j] + (col - p.col_begin[j]);
#pragma unroll
    for (int i = 0; i < kDequantRows; ++i) {
      if (r0 + i < p.K) *reinterpret_cast<uint4*>(dst + static_cast<size_t>(i) * p.width[j]) = ConvertChunk<MODE>(raw[i], sc);
    }
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

cudaError_t LaunchDequant(const DequantParams& params, cudaStream_t stream) {
  DequantParams p = params;
  p.scale_vec = p.w_scale != nullptr && reinterpret_cast<uintptr_t>(p.w_scale) % 16 == 0;
  const long long total = static_cast<long long>((p.K + kDequantRows - 1) / kDequantRows) * (p.N / 8);
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
