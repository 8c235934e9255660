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

// Eight quotients v[i] / d by the packed two-lane f32 instructions of sm_100 (each lane is an
// IEEE round-to-nearest op, so the results are those of the scalar forms): q0 = v r,
// residual = v - q0 d in one fma, q = q0 + residual r. `r` = RN(1/d), `dneg` = -d.
__device__ __forceinline__ void mb_markstein8(const float* v, float r, float dneg, float* q) {
  asm("{\n\t.reg .b64 x0, x1, x2, x3, q0, q1, q2, q3, m0, m1, m2, m3, rr, dd;\n\t"
      "mov.b64 rr, {%16, %16};\n\tmov.b64 dd, {%17, %17};\n\t"
      "mov.b64 x0, {%8, %9};\n\tmov.b64 x1, {%10, %11};\n\tmov.b64 x2, {%12, %13};\n\tmov.b64 x3, {%14, %15};\n\t"
      "mul.rn.f32x2 q0, x0, rr;\n\tmul.rn.f32x2 q1, x1, rr;\n\tmul.rn.f32x2 q2, x2, rr;\n\tmul.rn.f32x2 q3, x3, rr;\n\t"
      "fma.rn.f32x2 m0, q0, dd, x0;\n\tfma.rn.f32x2 m1, q1, dd, x1;\n\t"
      "fma.rn.f32x2 m2, q2, dd, x2;\n\tfma.rn.f32x2 m3, q3, dd, x3;\n\t"
      "fma.rn.f32x2 q0, m0, rr, q0;\n\tfma.rn.f32x2 q1, m1, rr, q1;\n\t"
      "fma.rn.f32x2 q2, m2, rr, q2;\n\tfma.rn.f32x2 q3, m3, rr, q3;\n\t"
      "mov.b64 {%0, %1}, q0;\n\tmov.b64 {%2, %3}, q1;\n\tmov.b64 {%4, %5}, q2;\n\tmov.b64 {%6, %7}, q3;\n\t}"
      : "=f"(q[0]), "=f"(q[1]), "=f"(q[2]), "=f"(q[3]), "=f"(q[4]), "=f"(q[5]), "=f"(q[6]), "=f"(q[7])
      : "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7]), "f"(r), "f"(dneg));
  // The quotient carries the sign of the dividend (d > 0), also when it is zero: x / d of x = -0.0 is -0.0 and
  // its code keeps the sign bit (src/nvfp4.rs:117-126), but the refinement's last sum (+0 residual term plus a -0
  // first estimate) rounds to +0. One bit-select per value puts the dividend's sign back.
#pragma unroll
  for (int i = 0; i < 8; ++i)
    q[i] = __uint_as_float((__float_as_uint(q[i]) & 0x7FFFFFFFu) | (__float_as_uint(v[i]) & 0x80000000u));
}
// Eight products v[i] * r the same way.
__device__ __forceinline__ void mb_mul8(const float* v, float r, float* q) {
  asm("{\n\t.reg .b64 x0, x1, x2, x3, rr;\n\t"
      "mov.b64 rr, {%16, %16};\n\t"
      "mov.b64 x0, {%8, %9};\n\tmov.b64 x1, {%10, %11};\n\tmov.b64 x2, {%12, %13};\n\tmov.b64 x3, {%14, %15};\n\t"
      "mul.rn.f32x2 x0, x0, rr;\n\tmul.rn.f32x2 x1, x1, rr;\n\tmul.rn.f32x2 x2, x2, rr;\n\tmul.rn.f32x2 x3, x3, rr;\n\t"
      "mov.b64 {%0, %1}, x0;\n\tmov.b64 {%2, %3}, x1;\n\tmov.b64 {%4, %5}, x2;\n\tmov.b64 {%6, %7}, x3;\n\t}"
      : "=f"(q[0]), "=f"(q[1]), "=f"(q[2]), "=f"(q[3]), "=f"(q[4]), "=f"(q[5]), "=f"(q[6]), "=f"(q[7])
      : "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7]), "f"(r));
}

// The divide recipe in two steps, so that a block spread over two threads (eight values
// each) runs the same arithmetic as a block held by one: the scale byte and the divisor
// from the block's amax, then eight codes from eight values.
__device__ __forceinline__ float quant_divisor_scaled(float bamax, float s2, uint32_t& sbyte) {
  float t = mb_div6(bamax);
  if (s2 != 1.0f) t = __fdiv_rn(t, s2);            // x / 1 is x: the unit global costs no divide
  sbyte = mb_e4m3_encode(fminf(t, 448.0f));        // fminf drops a NaN operand: an all-NaN block takes 448
  const float s = mb_e4m3_decode(sbyte);
  return s2 != 1.0f ? __fmul_rn(s, s2) : s;
}
// x / d for eight values, correctly rounded. Fast form: with r = RN(1/d) and q0 = RN(x r), the
// residual x - q0 d is exact in one fma and RN(q0 + residual r) is the correctly rounded
// quotient (Markstein), as long as d's significand is not all ones, nothing leaves the normal
// range and the block holds no infinity; otherwise the divide instruction itself.
__device__ __forceinline__ bool quant_div_is_fast(float d, float bamax) {
  const uint32_t db = __float_as_uint(d);
  return (db & 0x7FFFFFu) != 0x7FFFFFu && d >= 5.4210108624275222e-20f && d <= 1.8446744073709552e19f &&
         bamax <= 3.4028234663852886e38f;
}
__device__ __forceinline__ uint32_t quant_codes8_div(const float* v, float d, float bamax) {
  if (!(d > 0.0f)) return 0u;
  float q[8];
  if (quant_div_is_fast(d, bamax)) {
    mb_markstein8(v, __frcp_rn(d), -d, q);
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) q[i] = __fdiv_rn(v[i], d);
  }
  return mb_cvt_e2m1x8(q);
}

// One block under second-level scale `s2` with true divides: the weight recipe
// and the mary::nn activation recipe. One branch separates the ordinary block from the rest.
__device__ __forceinline__ void quant_block_scaled(const float* v, float s2, uint32_t& sbyte, uint2& codes) {
  const float bamax = amax16(v);
  const float d = quant_divisor_scaled(bamax, s2, sbyte);
  if (quant_div_is_fast(d, bamax)) {
    const float r = __frcp_rn(d);
    float q[16];
    mb_markstein8(v, r, -d, q);
    mb_markstein8(v + 8, r, -d, q + 8);
    codes.x = mb_cvt_e2m1x8(q);
    codes.y = mb_cvt_e2m1x8(q + 8);
  } else {
    codes.x = quant_codes8_div(v, d, bamax);
    codes.y = quant_codes8_div(v + 8, d, bamax);
  }
}

// One block, no second level, hoisted reciprocal: the Inkling activation recipe.
__device__ __forceinline__ void quant_block_recip(const float* v, uint32_t& sbyte, uint2& codes) {
  float amax = amax16(v);
  float sf = fminf(mb_div6(amax), 448.0f);
  sbyte = mb_e4m3_encode(sf);
  float s = mb_e4m3_decode(sbyte);
  float r = 0.0f;
  if (s > 0.0f) r = __frcp_rn(s);                  // correctly rounded, as 1 / s is
  float q[16];
  mb_mul8(v, r, q);
  mb_mul8(v + 8, r, q + 8);
  codes.x = mb_cvt_e2m1x8(q);
  codes.y = mb_cvt_e2m1x8(q + 8);
}

