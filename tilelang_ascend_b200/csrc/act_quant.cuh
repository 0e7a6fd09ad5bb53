// Per-token activation quantiser for sm_100a: bf16/f16 [M, N] -> int8 [M, N] + fp32 scale [M].
//
// The step in front of the W8A8 GEMM: it produces exactly that GEMM's A operand and scale_a.  Arithmetic
// follows the reference golden act_quant_torch (examples/deepseek_v4/act_quant.py:112-142) operation by
// operation in fp32, so that results are bit-identical to it:
//   amax  = max(max_j |x[i,j]|, 1e-4)
//   scale = amax / 127                      (IEEE division; round_scale: 2^ceil(log2(amax / 127)))
//   y     = int8( rint( clamp(x / scale, -127, 127) ) )      (IEEE division, round half to even)
// The device kernel it replaces is act_quant_kernel_int8_optimized (act_quant.py:33-92).
//
// HBM bound: every element is read once (2 bytes) and written once (1 byte).  A row is held in registers
// between the abs-max pass and the quantise pass: 4 or 8 16-byte chunks per thread; rows longer than
// 256 * AQ_MAX_CHUNKS * 8 elements are read a second time (from L2).  The host picks how many
// threads share a row (32, 64, 128 or 256) so that short rows do not leave most of a block idle.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace qg {

constexpr int AQ_THREADS = 256;
// Blocks per SM the 4-chunk variants are compiled for (caps registers at 32 per thread): measured 4 - 20 %
// faster than the compiler's own choice of 44 registers / 5 blocks on the shapes timed.
#ifndef AQ_MIN_BLOCKS
#define AQ_MIN_BLOCKS 7
#endif
constexpr int AQ_MAX_CHUNKS = 8;  // most 16-byte chunks (8 elements each) a thread keeps in registers

struct ActQuantParams {
  const uint4* X;   // [M, N] bf16 or f16
  int8_t* Y;        // [M, N]
  float* S;         // [M]
  long long M;
  int N;            // multiple of 8
  int is_bf16;
  int round_scale;
};

__device__ __forceinline__ void aq_unpack8(const uint4& v, bool bf16, float (&f)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (bf16) {
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    } else {
      const __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
      f[2 * i] = __low2float(h);
      f[2 * i + 1] = __high2float(h);
    }
  }
}

// Running abs-max of a row piece, kept as a packed pair in the input's own 16-bit format (the maximum of
// absolute values is exact in any format): one abs + one max per two elements.
__device__ __forceinline__ uint32_t aq_absmax8(const uint4& v, bool bf16, uint32_t m2) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (bf16) {
      const __nv_bfloat162 a = __habs2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
      const __nv_bfloat162 r = __hmax2(a, *reinterpret_cast<const __nv_bfloat162*>(&m2));
      m2 = *reinterpret_cast<const uint32_t*>(&r);
    } else {
      const __half2 a = __habs2(*reinterpret_cast<const __half2*>(&w[i]));
      const __half2 r = __hmax2(a, *reinterpret_cast<const __half2*>(&m2));
      m2 = *reinterpret_cast<const uint32_t*>(&r);
    }
  }
  return m2;
}

__device__ __forceinline__ float aq_pair_max(uint32_t m2, bool bf16) {
  if (bf16) return fmaxf(__uint_as_float(m2 << 16), __uint_as_float(m2 & 0xffff0000u));
  const __half2 h = *reinterpret_cast<const __half2*>(&m2);
  return fmaxf(__low2float(h), __high2float(h));
}

// x / scale rounded to the nearest integer (ties to even), eight values packed into two words.
//
// The quotient must round as IEEE fp32 division followed by rint does.  With y = RN(1 / scale) hoisted per
// row (__frcp_rn), q0 = x * y is within 1.5 ulp of x / scale; one residual correction
// q1 = fma(fma(-q0, scale, x), y, q0) makes it faithful (the residual is exact in the FMA), and a second
// one, q2 = fma(fma(-q1, scale, x), y, q1), is then the correctly rounded quotient RN(x / scale)
// (Markstein's theorem: a faithful quotient corrected once with the correctly rounded reciprocal and the
// exact residual rounds correctly).  Five FMA-class instructions, no branch, against the IEEE division
// routine's slow path per element.  Adding 1.5 * 2^23 rounds to an integer, ties to even, and leaves it in the
// low mantissa bits (two's complement), so no float-to-int conversion is needed.  |x / scale| <= 127 by
// construction (|x| <= amax <= 127 * scale), which makes the golden's clamp to [-127, 127] a no-op for
// finite inputs.
__device__ __forceinline__ uint32_t aq_pack4(const float* v) {
  return __byte_perm(__byte_perm(__float_as_uint(v[0]), __float_as_uint(v[1]), 0x0040),
                     __byte_perm(__float_as_uint(v[2]), __float_as_uint(v[3]), 0x0040), 0x5410);
}

__device__ __forceinline__ uint2 aq_quant8(const uint4& v, bool bf16, float scale, float rcp) {
  const float MAGIC = 12582912.0f;  // 1.5 * 2^23
  float f[8];
  aq_unpack8(v, bf16, f);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float q0 = f[i] * rcp;
    const float q1 = fmaf(fmaf(-q0, scale, f[i]), rcp, q0);
    const float q2 = fmaf(fmaf(-q1, scale, f[i]), rcp, q1);
    f[i] = q2 + MAGIC;
  }
  return make_uint2(aq_pack4(f), aq_pack4(f + 4));
}

// 2^ceil(log2(x)) for a positive normal fp32 x, from its bits (act_quant.py:95-109 does the same).
__device__ __forceinline__ float aq_pow2_ceil(float x) {
  const uint32_t bits = __float_as_uint(x);
  const int e = (int)((bits >> 23) & 0xffu) + ((bits & 0x7fffffu) ? 1 : 0);
  return __uint_as_float((uint32_t)e << 23);
}

// TPR threads share one row; a block holds AQ_THREADS / TPR rows; KEEP chunks per thread stay in registers.
template <int TPR, int KEEP>
__global__ void __launch_bounds__(AQ_THREADS, KEEP == 4 ? AQ_MIN_BLOCKS : 1) act_quant_kernel(const ActQuantParams p) {
  constexpr int ROWS = AQ_THREADS / TPR;
  constexpr int WPR = TPR / 32;  // warps per row
  __shared__ float red[AQ_THREADS / 32];
  const int t = threadIdx.x % TPR;
  const int r = threadIdx.x / TPR;
  const int warp = threadIdx.x >> 5;
  const long long row = (long long)blockIdx.x * ROWS + r;
  const bool live = row < p.M;
  const int chunks = p.N >> 3;
  const bool bf16 = p.is_bf16 != 0;
  const uint4* x = p.X + (live ? row : 0) * chunks;

  uint4 keep[KEEP];
  uint32_t m2 = 0u;  // (+0, +0) in either format
  if (live) {
#pragma unroll
    for (int i = 0; i < KEEP; ++i) {
      const int c = t + i * TPR;
      if (c < chunks) {
        keep[i] = __ldcs(x + c);
        m2 = aq_absmax8(keep[i], bf16, m2);
      }
    }
    for (int c = t + KEEP * TPR; c < chunks; c += TPR) m2 = aq_absmax8(__ldg(x + c), bf16, m2);
  }
  float m = aq_pair_max(m2, bf16);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if (WPR > 1) {
    if ((threadIdx.x & 31) == 0) red[warp] = m;
    __syncthreads();
#pragma unroll
    for (int w = 0; w < WPR; ++w) m = fmaxf(m, red[r * WPR + w]);
  }
  if (!live) return;

  const float amax = fmaxf(m, 1e-4f);
  float scale = __fdiv_rn(amax, 127.0f);
  if (p.round_scale) scale = aq_pow2_ceil(scale);
  if (t == 0) p.S[row] = scale;
  const float rcp = __frcp_rn(scale);

  uint2* y = reinterpret_cast<uint2*>(p.Y) + row * chunks;
#pragma unroll
  for (int i = 0; i < KEEP; ++i) {
    const int c = t + i * TPR;
    if (c < chunks) __stcs(y + c, aq_quant8(keep[i], bf16, scale, rcp));
  }
  for (int c = t + KEEP * TPR; c < chunks; c += TPR) __stcs(y + c, aq_quant8(__ldg(x + c), bf16, scale, rcp));
}

}  // namespace qg
