// The per-block NVFP4 arithmetic (16 values -> 8 bytes of E2M1 codes + one E4M3 scale byte),
// shared by the stand-alone quantizer kernels and by the kernels that quantize what they
// have just produced (the GEMM epilogue, the norm + quantize row kernel): one definition,
// so a fused producer writes the bytes the separate quantizer would have written.
#pragma once

#include "common.cuh"

__device__ __forceinline__ float amax16(const float* v) {
  float m[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) m[i] = fmaxf(fabsf(v[i]), fabsf(v[i + 8]));
  float a01 = fmaxf(fmaxf(m[0], m[1]), fmaxf(m[2], m[3]));
  float a23 = fmaxf(fmaxf(m[4], m[5]), fmaxf(m[6], m[7]));
  return fmaxf(a01, a23);
}

// The divide recipe in two steps, so that a block spread over two threads (eight values
// each) runs the same arithmetic as a block held by one: the scale byte and the divisor
// from the block's amax, then eight codes from eight values.
__device__ __forceinline__ float quant_divisor_scaled(float bamax, float s2, uint32_t& sbyte) {
  float t = __fdiv_rn(bamax, 6.0f);
  if (s2 != 1.0f) t = __fdiv_rn(t, s2);            // x / 1 is x: the unit global costs no divide
  sbyte = mb_e4m3_from_f32(fminf(t, 448.0f));
  return __fmul_rn(mb_e4m3_to_f32(sbyte), s2);
}
__device__ __forceinline__ uint32_t quant_codes8_div(const float* v, float d, float bamax) {
  if (!(d > 0.0f)) return 0u;
  // x / d, correctly rounded. Fast form: with r = RN(1/d) and q0 = RN(x r), the residual
  // x - q0 d is exact in one fma and RN(q0 + residual r) is the correctly rounded quotient
  // (Markstein), as long as d's significand is not all ones, nothing leaves the normal
  // range and the block holds no infinity; otherwise the divide instruction itself.
  const uint32_t db = __float_as_uint(d);
  const bool fast = (db & 0x7FFFFFu) != 0x7FFFFFu && d >= 5.4210108624275222e-20f && d <= 1.8446744073709552e19f &&
                    bamax <= 3.4028234663852886e38f;
  float q[8];
  if (fast) {
    const float r = __frcp_rn(d);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float q0 = __fmul_rn(v[i], r);
      const float rem = __fmaf_rn(-q0, d, v[i]);
      q[i] = __fmaf_rn(rem, r, q0);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) q[i] = __fdiv_rn(v[i], d);
  }
  return mb_cvt_e2m1x8(q);
}

// One block under second-level scale `s2` with true divides: the weight recipe
// and the mary::nn activation recipe.
__device__ __forceinline__ void quant_block_scaled(const float* v, float s2, uint32_t& sbyte, uint2& codes) {
  const float bamax = amax16(v);
  const float d = quant_divisor_scaled(bamax, s2, sbyte);
  codes.x = quant_codes8_div(v, d, bamax);
  codes.y = quant_codes8_div(v + 8, d, bamax);
}

// One block, no second level, hoisted reciprocal: the Inkling activation recipe.
__device__ __forceinline__ void quant_block_recip(const float* v, uint32_t& sbyte, uint2& codes) {
  float amax = amax16(v);
  float sf = fminf(__fdiv_rn(amax, 6.0f), 448.0f);
  sbyte = mb_e4m3_from_f32(sf);
  float s = mb_e4m3_to_f32(sbyte);
  float r = 0.0f;
  if (s > 0.0f) r = __fdiv_rn(1.0f, s);
  float q[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) q[i] = __fmul_rn(v[i], r);
  codes.x = mb_cvt_e2m1x8(q);
  codes.y = mb_cvt_e2m1x8(q + 8);
}

