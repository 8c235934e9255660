// CPU oracle: a plain C++17 restatement of the reference's arithmetic for the
// quantized-inference hot path. TEST INFRASTRUCTURE ONLY. Nothing in the product
// library links, imports or calls this file; it exists so that the CUDA kernels
// can be checked against the reference's own rules on identical seeded bytes, and
// so that a CPU baseline can be timed beside the GPU numbers.
//
// Every function cites the reference file:line it follows (paths are relative to
// the reference project root). Build: see oracle/Makefile (g++ -O2
// -ffp-contract=off so that no multiply-add is fused behind the code's back).
//
// Parity pin: the codec and planner functions are checked by tests/ against the
// known-answer tests the reference keeps in-source (src/nvfp4.rs:333-462,
// src/nn/nvfp4_gemv.rs:753-767, src/models/inkling/moegroup.rs:1947-2007,
// src/models/inkling/flash.rs:1989-2016, src/models/inkling/tp.rs:761-793,
// src/models/k3/router.rs:518-572). The BF16xBF16 GEMM has no numeric pin in the
// reference beyond "f32 accumulation of bf16 products": parity unpinned for it.

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <numeric>
#include <vector>

#if defined(_OPENMP)
#include <omp.h>
#endif

#define ORC_API extern "C" __attribute__((visibility("default")))

namespace {

constexpr int BLOCK = 16;             // src/nvfp4.rs:40
constexpr float E2M1_MAX = 6.0f;      // src/nvfp4.rs:44
constexpr float E4M3_MAX = 448.0f;    // src/nvfp4.rs:46
constexpr uint8_t E4M3_MAX_BYTE = 0x7E;  // src/nvfp4.rs:48
const float E2M1[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};  // src/nvfp4.rs:42

inline uint32_t f32_bits(float v) { uint32_t b; std::memcpy(&b, &v, 4); return b; }
inline float bits_f32(uint32_t b) { float v; std::memcpy(&v, &b, 4); return v; }

// bf16 <-> f32. Widening is a shift (src/models/k3/router.rs:492-497); narrowing
// is round-to-nearest-even with NaN kept quiet, the rule of the `half` crate and
// of the hardware cvt.rn.bf16.f32.
inline float bf16_to_f32(uint16_t b) { return bits_f32(uint32_t(b) << 16); }
inline uint16_t f32_to_bf16(float v) {
  uint32_t x = f32_bits(v);
  if ((x & 0x7FFFFFFFu) > 0x7F800000u) return uint16_t((x >> 16) | 0x0040u);
  uint32_t lsb = (x >> 16) & 1u;
  x += 0x7FFFu + lsb;
  return uint16_t(x >> 16);
}
inline float round_bf16(float v) { return bf16_to_f32(f32_to_bf16(v)); }

// src/nvfp4.rs:52-64
inline float e4m3_to_f32(uint8_t b) {
  float sign = (b & 0x80) ? -1.0f : 1.0f;
  int exp = (b >> 3) & 0xF;
  float man = float(b & 7);
  float mag;
  if (exp == 0) {
    mag = man * std::ldexp(1.0f, -9);
  } else if (exp == 15 && man == 7.0f) {
    mag = std::numeric_limits<float>::quiet_NaN();
  } else {
    mag = (1.0f + man / 8.0f) * std::ldexp(1.0f, exp - 7);
  }
  return sign * mag;
}

// src/nvfp4.rs:73-92
inline uint8_t e4m3_from_f32(float v) {
  if (!(v > 0.0f)) return 0;
  if (v >= E4M3_MAX) return E4M3_MAX_BYTE;
  int e = std::max(int((f32_bits(v) >> 23) & 0xFF) - 127, -6);
  float scaled = v * std::ldexp(1.0f, 3 - e);
  uint32_t steps = uint32_t(std::nearbyintf(scaled));  // default mode: ties to even
  uint32_t byte;
  if (e == -6 && steps < 8) {
    byte = steps;
  } else {
    int ee = e;
    uint32_t m;
    if (steps == 16) { ee = e + 1; m = 0; } else { m = steps - 8; }
    byte = (uint32_t(ee + 7) << 3) | m;
  }
  return uint8_t(std::min<uint32_t>(byte, E4M3_MAX_BYTE));
}

// src/nvfp4.rs:96-111
inline uint8_t e2m1_code(float m) {
  static const float MID[7] = {0.25f, 0.75f, 1.25f, 1.75f, 2.5f, 3.5f, 5.0f};
  if (std::isnan(m)) return 7;
  uint8_t code = 0;
  for (int i = 0; i < 7; ++i) {
    if (m > MID[i] || (m == MID[i] && (i + 1) % 2 == 0)) code = uint8_t(i + 1);
  }
  return code;
}

// src/nvfp4.rs:117-126
inline uint8_t code_of(float v, float unit) {
  if (!(unit > 0.0f)) return 0;
  uint8_t sign = std::signbit(v) ? 8 : 0;
  if (v == 0.0f || std::isnan(v)) return sign;
  return uint8_t(e2m1_code(std::fabs(v) / unit) | sign);
}

// src/nvfp4.rs:129-132
inline float decode_code(uint8_t code) {
  float m = E2M1[code & 7];
  return (code & 8) ? -m : m;
}

// `cvt.rn.satfinite.e2m1x2.f32` of one already-divided quotient, as the device
// quantizers apply it: sign kept on a zero result, NaN saturates to magnitude 6
// (src/models/inkling/fp4quant.rs:28-55; host twin src/nn/nvfp4_gemv.rs:669-679).
inline uint8_t cvt_e2m1(float q) {
  uint8_t sign = std::signbit(q) ? 8 : 0;
  if (std::isnan(q)) return uint8_t(7 | sign);
  return uint8_t(e2m1_code(std::fabs(q)) | sign);
}

inline float block_amax(const float* b) {
  float m = 0.0f;
  for (int i = 0; i < BLOCK; ++i) m = std::max(m, std::fabs(b[i]));  // fmax drops NaN like the device max
  return m;
}

// One 16-block under a given second-level scale: the single definition of
// src/nn/nvfp4_gemv.rs:140-172 (`quantize_block`) == src/nvfp4.rs:146-150 + :287-293.
inline void quantize_block(const float* w, float scale2, uint8_t* codes8, uint8_t* scale_byte) {
  float bamax = block_amax(w);
  float t = (bamax / E2M1_MAX) / scale2;          // two correctly rounded divides, in this order
  uint8_t se = e4m3_from_f32(std::fmin(t, E4M3_MAX));  // f32::min / fminf: a NaN operand is dropped
  *scale_byte = se;
  float d = e4m3_to_f32(se) * scale2;
  for (int i = 0; i < BLOCK / 2; ++i) {
    uint8_t lo = 0, hi = 0;
    if (d > 0.0f) {
      lo = cvt_e2m1(w[2 * i] / d);
      hi = cvt_e2m1(w[2 * i + 1] / d);
    }
    codes8[i] = uint8_t(lo | (hi << 4));
  }
}

struct SplitMix {  // src/nn/nvfp4_gemv.rs:610-627
  uint64_t s;
  uint64_t next() {
    s += 0x9E3779B97F4A7C15ull;
    uint64_t z = s;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
  }
  double unit() { return double(next() >> 11) / double(1ull << 53); }
  double normal() {
    double u = std::max(unit(), 1e-300);
    double r = std::sqrt(-2.0 * std::log(u));
    return r * std::cos(6.283185307179586476925286766559 * unit());
  }
};

}  // namespace

// ---------------------------------------------------------------------------
// Scalar codec (src/nvfp4.rs:52-150)
// ---------------------------------------------------------------------------
ORC_API float orc_e4m3_to_f32(uint8_t b) { return e4m3_to_f32(b); }
ORC_API uint8_t orc_e4m3_from_f32(float v) { return e4m3_from_f32(v); }
ORC_API uint8_t orc_e2m1_code(float m) { return e2m1_code(m); }
ORC_API uint8_t orc_code_of(float v, float unit) { return code_of(v, unit); }
ORC_API float orc_decode_code(uint8_t c) { return decode_code(c); }
ORC_API uint8_t orc_cvt_e2m1(float q) { return cvt_e2m1(q); }
ORC_API uint16_t orc_f32_to_bf16(float v) { return f32_to_bf16(v); }
ORC_API float orc_bf16_to_f32(uint16_t b) { return bf16_to_f32(b); }

// src/nvfp4.rs:136-143
ORC_API float orc_global_scale(const float* w, size_t len) {
  float absmax = 0.0f;
  for (size_t i = 0; i < len; ++i) absmax = std::max(absmax, std::fabs(w[i]));
  if (absmax > 0.0f && std::isfinite(absmax)) return absmax / (E2M1_MAX * E4M3_MAX);
  return 1.0f;
}

// src/nn/nvfp4_gemv.rs:92-118 + :583-600: NaN-carrying amax, then scale2_of.
// Returns 0 and writes scale2, or -1 when the tensor holds a non-finite value
// (the reference refuses such a weight).
ORC_API int orc_scale2_of_tensor(const float* w, size_t len, float* scale2) {
  float amax = 0.0f;
  bool nan = false;
  for (size_t i = 0; i < len; ++i) {
    float a = std::fabs(w[i]);
    if (a != a) nan = true;
    amax = std::max(amax, a);
  }
  if (nan || !std::isfinite(amax)) return -1;
  *scale2 = amax > 0.0f ? amax / (6.0f * 448.0f) : 1.0f;
  return 0;
}

// src/nvfp4.rs:146-150
ORC_API void orc_block_unit(const float* block, float scale2, uint8_t* byte, float* unit) {
  float bmax = block_amax(block);
  uint8_t b = e4m3_from_f32(std::fmin((bmax / E2M1_MAX) / scale2, E4M3_MAX));
  *byte = b;
  *unit = e4m3_to_f32(b) * scale2;
}

// src/nvfp4.rs:268-305 (`pack_nearest`): row-major [rows, cols] f32 -> codes
// [rows*cols/2] (lower index in the LOW nibble), scales [rows*cols/16], scale2.
ORC_API int orc_pack_nearest(const float* w, size_t rows, size_t cols, uint8_t* codes,
                             uint8_t* scales, float* scale2_out) {
  if (cols == 0 || cols % BLOCK != 0) return -1;
  size_t len = rows * cols;
  float scale2 = orc_global_scale(w, len);
  *scale2_out = scale2;
  size_t blocks = len / BLOCK;
#pragma omp parallel for schedule(static)
  for (long long blk = 0; blk < (long long)blocks; ++blk) {
    const float* b = w + blk * BLOCK;
    uint8_t byte;
    float unit;
    orc_block_unit(b, scale2, &byte, &unit);
    scales[blk] = byte;
    for (int i = 0; i < BLOCK / 2; ++i) {
      codes[blk * (BLOCK / 2) + i] = uint8_t(code_of(b[2 * i], unit) | (code_of(b[2 * i + 1], unit) << 4));
    }
  }
  return 0;
}

// Payload = codes || scales || scale2 (little-endian f32): src/nvfp4.rs:153-167, :203-210.
ORC_API size_t orc_payload_len(size_t elems) { return (elems + 1) / 2 + (elems + BLOCK - 1) / BLOCK + 4; }

// src/nvfp4.rs:170-182 (`decode_payload`): unit formed first, then code * unit.
ORC_API int orc_decode_payload(const uint8_t* payload, size_t payload_len, size_t elems, float* out) {
  if (payload_len != orc_payload_len(elems)) return -1;
  size_t codes_len = (elems + 1) / 2, scales_len = (elems + BLOCK - 1) / BLOCK;
  const uint8_t* codes = payload;
  const uint8_t* scales = payload + codes_len;
  float scale2;
  std::memcpy(&scale2, payload + codes_len + scales_len, 4);
#pragma omp parallel for schedule(static)
  for (long long blk = 0; blk < (long long)scales_len; ++blk) {
    float unit = e4m3_to_f32(scales[blk]) * scale2;
    for (int i = 0; i < BLOCK; ++i) {
      size_t e = size_t(blk) * BLOCK + i;
      if (e >= elems) break;
      uint8_t code = (codes[e / 2] >> (4 * (e % 2))) & 0xF;
      out[e] = decode_code(code) * unit;
    }
  }
  return 0;
}

// Planes apart (codes, scales, scale2) -> dense f32; scale2 == 1 gives the
// activation planes' values (src/models/inkling/fp4quant.rs:437-459).
ORC_API void orc_dequantize(const uint8_t* codes, const uint8_t* scales, float scale2, size_t elems, float* out) {
  size_t blocks = elems / BLOCK;
#pragma omp parallel for schedule(static)
  for (long long blk = 0; blk < (long long)blocks; ++blk) {
    float unit = e4m3_to_f32(scales[blk]) * scale2;
    for (int i = 0; i < BLOCK; ++i) {
      size_t e = size_t(blk) * BLOCK + i;
      uint8_t code = (codes[e / 2] >> (4 * (e % 2))) & 0xF;
      out[e] = decode_code(code) * unit;
    }
  }
}

// ---------------------------------------------------------------------------
// Device quantizer recipes
// ---------------------------------------------------------------------------

// Weight quantizer from bf16 bits: src/nn/nvfp4_gemv.rs:284-351 (K1 amax + K2
// quantize_block). Bit-identical to pack_nearest of the widened values
// (`pack_matching`, :468-501). Returns -1 for a non-finite weight.
ORC_API int orc_quantize_weight_bf16(const uint16_t* w, size_t n, size_t k, uint8_t* codes, uint8_t* scales,
                                     float* scale2_out) {
  size_t len = n * k;
  std::vector<float> f(len);
  for (size_t i = 0; i < len; ++i) f[i] = bf16_to_f32(w[i]);
  float scale2;
  if (orc_scale2_of_tensor(f.data(), len, &scale2) != 0) return -1;
  *scale2_out = scale2;
  size_t blocks = len / BLOCK;
#pragma omp parallel for schedule(static)
  for (long long blk = 0; blk < (long long)blocks; ++blk)
    quantize_block(f.data() + blk * BLOCK, scale2, codes + blk * 8, scales + blk);
  return 0;
}

// Activation quantizer of the `mary::nn` W4A4 lane: quantize_block with the
// operation's `input_scale` as the second-level scale (src/nn/nvfp4_gemm.rs:644-669).
ORC_API void orc_quantize_act_scaled(const float* x, size_t rows, size_t k, float input_scale, uint8_t* codes,
                                     uint8_t* scales) {
  size_t blocks = rows * k / BLOCK;
#pragma omp parallel for schedule(static)
  for (long long blk = 0; blk < (long long)blocks; ++blk)
    quantize_block(x + blk * BLOCK, input_scale, codes + blk * 8, scales + blk);
}

// Per-row second-level scale: src/nn/nvfp4_gemm.rs:757-813 (`row_scale_kernel`,
// `quantize_rows_kernel`). rowscale = amax/2688, 1.0 for a zero row, NaN for a NaN row.
ORC_API void orc_quantize_act_rows(const float* x, size_t rows, size_t k, float* rowscale, uint8_t* codes,
                                   uint8_t* scales) {
  for (size_t r = 0; r < rows; ++r) {
    float a = 0.0f;
    bool nan = false;
    for (size_t j = 0; j < k; ++j) {
      float v = std::fabs(x[r * k + j]);
      if (v != v) nan = true;
      a = std::max(a, v);
    }
    float s = a > 0.0f ? a / 2688.0f : 1.0f;
    if (nan) s = std::numeric_limits<float>::quiet_NaN();
    rowscale[r] = s;
  }
  size_t row_blocks = k / BLOCK;
  size_t blocks = rows * row_blocks;
#pragma omp parallel for schedule(static)
  for (long long blk = 0; blk < (long long)blocks; ++blk)
    quantize_block(x + blk * BLOCK, rowscale[blk / row_blocks], codes + blk * 8, scales + blk);
}

// Inkling activation quantizer, no second level, hoisted reciprocal:
// src/models/inkling/fp4quant.rs:199-238.
ORC_API void orc_quantize_act_recip(const float* x, size_t rows, size_t k, uint8_t* codes, uint8_t* scales) {
  size_t blocks = rows * k / BLOCK;
#pragma omp parallel for schedule(static)
  for (long long blk = 0; blk < (long long)blocks; ++blk) {
    const float* b = x + blk * BLOCK;
    float amax = block_amax(b);
    float sf = std::min(amax / 6.0f, 448.0f);
    uint8_t se = e4m3_from_f32(sf);
    float s = e4m3_to_f32(se);
    scales[blk] = se;
    float r = 0.0f;
    if (s > 0.0f) r = 1.0f / s;
    for (int i = 0; i < 8; ++i) {
      uint8_t lo = cvt_e2m1(b[2 * i] * r);
      uint8_t hi = cvt_e2m1(b[2 * i + 1] * r);
      codes[blk * 8 + i] = uint8_t(lo | (hi << 4));
    }
  }
}

// ---------------------------------------------------------------------------
// Linear layers (oracle accumulation in f64 of the dequantised operands)
// ---------------------------------------------------------------------------

// W4A16: y[m,n] = (sum_k x[m,k] * E2M1[code]*e4m3(scale))*scale2, x bf16.
// The order "block partial x E4M3, carried, x scale2 once" is src/nn/nvfp4_gemv.rs:41-50,
// :202-250; the reference CPU lane decodes to dense f32 first (src/leaf.rs:184-191,
// src/nvfp4.rs:170-182) and multiplies. out_f64 is the unrounded sum; the bf16
// rounding is the caller's single final cast.
ORC_API void orc_linear_w4a16(const uint16_t* x, const uint8_t* codes, const uint8_t* scales, float scale2,
                              size_t M, size_t N, size_t K, double* out) {
  std::vector<float> xf(M * K);
  for (size_t i = 0; i < M * K; ++i) xf[i] = bf16_to_f32(x[i]);
#pragma omp parallel for schedule(static)
  for (long long n = 0; n < (long long)N; ++n) {
    std::vector<float> wrow(K);
    for (size_t kb = 0; kb < K / BLOCK; ++kb) {
      float s = e4m3_to_f32(scales[n * (K / BLOCK) + kb]);
      for (int i = 0; i < BLOCK; ++i) {
        size_t e = size_t(n) * K + kb * BLOCK + i;
        uint8_t code = (codes[e / 2] >> (4 * (e % 2))) & 0xF;
        wrow[kb * BLOCK + i] = decode_code(code) * s;  // exact in f32
      }
    }
    for (size_t m = 0; m < M; ++m) {
      double acc = 0.0;
      const float* xr = xf.data() + m * K;
      for (size_t k = 0; k < K; ++k) acc += double(xr[k]) * double(wrow[k]);
      out[m * N + n] = acc * double(scale2);
    }
  }
}

// The reference's CPU lane for config 0, as it runs: dense f32 decode
// (decode_payload) then an f32 matmul x.W^T with f32 accumulation
// (src/models/inkling/burn.rs:49-54 on the ndarray backend), bf16 result.
ORC_API void orc_linear_cpu_lane(const uint16_t* x, const float* w_dense, size_t M, size_t N, size_t K,
                                 uint16_t* out) {
  std::vector<float> xf(M * K);
  for (size_t i = 0; i < M * K; ++i) xf[i] = bf16_to_f32(x[i]);
#pragma omp parallel for schedule(static)
  for (long long n = 0; n < (long long)N; ++n) {
    const float* wr = w_dense + size_t(n) * K;
    for (size_t m = 0; m < M; ++m) {
      const float* xr = xf.data() + m * K;
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (size_t k = 0; k < K; k += 8)
        for (int j = 0; j < 8; ++j) acc[j] += xr[k + j] * wr[k + j];
      float s = ((acc[0] + acc[1]) + (acc[2] + acc[3])) + ((acc[4] + acc[5]) + (acc[6] + acc[7]));
      out[m * N + n] = f32_to_bf16(s);
    }
  }
}

// W4A4: both operands NVFP4 planes without their global scales; the epilogue
// multiplies by alpha (= f32(scale2*input_scale), src/nn/nvfp4_gemm.rs:688) and,
// when rowscale != null, by rowscale[m] first (src/nn/nvfp4_gemm.rs:814-816:
// acc * (rowscale[r] * scale)). out is f32 (unrounded to bf16).
ORC_API void orc_linear_w4a4(const uint8_t* a_codes, const uint8_t* a_scales, const uint8_t* b_codes,
                             const uint8_t* b_scales, const float* rowscale, float alpha, size_t M, size_t N,
                             size_t K, float* out) {
  std::vector<float> af(M * K), bf(N * K);
  orc_dequantize(a_codes, a_scales, 1.0f, M * K, af.data());
  orc_dequantize(b_codes, b_scales, 1.0f, N * K, bf.data());
#pragma omp parallel for schedule(static)
  for (long long n = 0; n < (long long)N; ++n) {
    const float* br = bf.data() + size_t(n) * K;
    for (size_t m = 0; m < M; ++m) {
      const float* ar = af.data() + m * K;
      double acc = 0.0;
      for (size_t k = 0; k < K; ++k) acc += double(ar[k]) * double(br[k]);
      float scale = rowscale ? rowscale[m] * alpha : alpha;
      out[m * N + n] = float(acc) * scale;
    }
  }
}

// Decode-time grouped experts (src/nn/nvfp4_gemm.rs:293-313, 320-432, 462-523): group g's row (the shared row
// when x_per_group == 0) is quantized with input_scale[ids[g]] as the second-level scale and multiplied with
// expert ids[g] of the bank, epilogue alpha[ids[g]]: "per group exactly project_w4a4_scaled on one row".
// x bf16 bits; bank planes [experts, n, k/2], [experts, n, k/16]. out f32 [groups, n] (the caller rounds to bf16);
// a_codes / a_scales (may be null) receive the activation planes.
ORC_API void orc_w4a4_grouped(const uint16_t* x, int x_per_group, const uint32_t* ids, size_t groups,
                              const float* input_scale, const float* alpha, const uint8_t* bank_codes,
                              const uint8_t* bank_scales, size_t n, size_t k, uint8_t* a_codes, uint8_t* a_scales,
                              float* out) {
  std::vector<float> row(k);
  std::vector<uint8_t> c(k / 2), sc(k / 16);
  for (size_t g = 0; g < groups; ++g) {
    const uint16_t* xr = x + (x_per_group ? g * k : 0);
    for (size_t i = 0; i < k; ++i) row[i] = bf16_to_f32(xr[i]);
    const size_t e = ids[g];
    orc_quantize_act_scaled(row.data(), 1, k, input_scale[e], c.data(), sc.data());
    if (a_codes) std::memcpy(a_codes + g * k / 2, c.data(), k / 2);
    if (a_scales) std::memcpy(a_scales + g * k / 16, sc.data(), k / 16);
    orc_linear_w4a4(c.data(), sc.data(), bank_codes + e * n * k / 2, bank_scales + e * n * k / 16, nullptr, alpha[e], 1,
                    n, k, out + g * n);
  }
}

// BF16 x BF16 -> f32 (src/models/inkling/bf16gemm.rs:64-152): f64 accumulation of
// the identical bf16 operands. Parity unpinned in the reference (no numeric pin).
ORC_API void orc_linear_bf16(const uint16_t* x, const uint16_t* w, size_t M, size_t N, size_t K, float* out) {
  std::vector<float> xf(M * K), wf(N * K);
  for (size_t i = 0; i < M * K; ++i) xf[i] = bf16_to_f32(x[i]);
  for (size_t i = 0; i < N * K; ++i) wf[i] = bf16_to_f32(w[i]);
#pragma omp parallel for schedule(static)
  for (long long n = 0; n < (long long)N; ++n)
    for (size_t m = 0; m < M; ++m) {
      double acc = 0.0;
      for (size_t k = 0; k < K; ++k) acc += double(xf[m * K + k]) * double(wf[size_t(n) * K + k]);
      out[m * N + n] = float(acc);
    }
}

// ---------------------------------------------------------------------------
// MXFP4 -> NVFP4 relabelling (src/nn/mxfp4.rs:141-400). An E8M0 scale byte b is 2^(b - 127)
// (0xFF = NaN); E4M3 holds the powers of two 2^-9 .. 2^8 exactly. With g = e_max - 8 as the
// global exponent every block scale becomes 2^(e - g), written twice (one 32-block = two
// 16-blocks); the codes are not touched.
// ---------------------------------------------------------------------------
static int e4m3_from_pow2(int e) {                    // mxfp4.rs:169-177; -1 outside the window
  if (e == -9) return 0x01;
  if (e == -8) return 0x02;
  if (e == -7) return 0x04;
  if (e >= -6 && e <= 8) return (e + 7) << 3;
  return -1;
}
ORC_API int orc_e4m3_from_pow2(int e) { return e4m3_from_pow2(e); }

// Returns 0; 1 = NaN scale (info[0] = index); 2 = span too wide (info = e_min, e_max, octaves);
// 3 = global scale 2^g not a normal f32 (info[0] = g). On success info[0] = g, info[1] = 1 when a
// block scale is an E4M3 subnormal. block_scale: 2 * n bytes.
ORC_API int orc_mxfp4_transcode(const uint8_t* scale, size_t n, uint8_t* block_scale, long long* info) {
  int e_min = INT32_MAX, e_max = INT32_MIN;
  for (size_t i = 0; i < n; ++i) {
    if (scale[i] == 0xFF) { info[0] = (long long)i; return 1; }
    int e = int(scale[i]) - 127;
    e_min = std::min(e_min, e);
    e_max = std::max(e_max, e);
  }
  const int g = e_max - 8;
  if (e_min - g < -9) { info[0] = e_min; info[1] = e_max; info[2] = e_max - e_min + 1; return 2; }
  if (g < -126 || g > 127) { info[0] = g; return 3; }
  bool sub = false;
  for (size_t i = 0; i < n; ++i) {
    int e = int(scale[i]) - 127 - g;
    sub |= e < -6;
    uint8_t b = uint8_t(e4m3_from_pow2(e));
    block_scale[2 * i] = b;
    block_scale[2 * i + 1] = b;
  }
  info[0] = g;
  info[1] = sub ? 1 : 0;
  return 0;
}

// decode_mxfp4 (mxfp4.rs:265-300): value = E2M1[code] * 2^(b - 127), low nibble first, blocks of 32 along a row.
ORC_API void orc_mxfp4_decode(const uint8_t* packed, const uint8_t* scale, size_t rows, size_t cols, float* out) {
  static const float E2M1[16] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f,
                                 -0.0f, -0.5f, -1.0f, -1.5f, -2.0f, -3.0f, -4.0f, -6.0f};
  for (size_t i = 0; i < rows * cols; ++i) {
    uint8_t b = scale[i / 32];
    float s;
    if (b == 0xFF) s = std::numeric_limits<float>::quiet_NaN();
    else if (b == 0) { uint32_t bits = 1u << 22; std::memcpy(&s, &bits, 4); }
    else { uint32_t bits = uint32_t(b) << 23; std::memcpy(&s, &bits, 4); }
    uint8_t code = (packed[i / 2] >> ((i & 1) * 4)) & 15;
    out[i] = E2M1[code] * s;
  }
}

// ---------------------------------------------------------------------------
// Router (src/models/k3/router.rs:343-488, softmax branch; equals
// src/models/gemma/gemma4/layers.rs:288-325 without per_expert_scale)
// ---------------------------------------------------------------------------

// Softmax scores: f64 exp, f32 store, then f32(f64(v)/s) (router.rs:352-368).
ORC_API void orc_router_scores_softmax(const float* logits, size_t tokens, size_t n, float* v) {
  for (size_t t = 0; t < tokens; ++t) {
    const float* row = logits + t * n;
    double m = -std::numeric_limits<double>::infinity();
    for (size_t i = 0; i < n; ++i) m = std::max(m, double(row[i]));
    double s = 0.0;
    for (size_t i = 0; i < n; ++i) {
      double e = std::exp(double(row[i]) - m);
      v[t * n + i] = float(e);
      s += e;
    }
    for (size_t i = 0; i < n; ++i) v[t * n + i] = float(double(v[t * n + i]) / s);
  }
}

// Sigmoid scores, each expert alone: f32(1 / (1 + exp(-f64(x)))) (router.rs:347-350).
ORC_API void orc_router_scores_sigmoid(const float* logits, size_t tokens, size_t n, float* v) {
  for (size_t i = 0; i < tokens * n; ++i) v[i] = float(1.0 / (1.0 + std::exp(-double(logits[i]))));
}

// Selection (router.rs:399-425): descending score, ties ascending index; gather
// (router.rs:431-446); normalise w/(sum+1e-20)*scale (router.rs:451-471).
// Returns -1 on a non-finite score (the reference panics).
ORC_API int orc_router_select(const float* scores, const float* bias, size_t tokens, size_t n, size_t k,
                              int renormalize, float scaling, uint32_t* idx, float* weight) {
  std::vector<uint32_t> order(n);
  std::vector<float> sfc(n);
  for (size_t t = 0; t < tokens; ++t) {
    const float* row = scores + t * n;
    for (size_t e = 0; e < n; ++e) {
      sfc[e] = bias ? row[e] + bias[e] : row[e];
      if (!std::isfinite(sfc[e])) return -1;
    }
    std::iota(order.begin(), order.end(), 0u);
    std::sort(order.begin(), order.end(), [&](uint32_t a, uint32_t b) {
      if (sfc[a] != sfc[b]) return sfc[a] > sfc[b];
      return a < b;
    });
    for (size_t j = 0; j < k; ++j) {
      idx[t * k + j] = order[j];
      weight[t * k + j] = row[order[j]];
    }
    if (k > 1 && renormalize) {
      float s = 0.0f;
      for (size_t j = 0; j < k; ++j) s += weight[t * k + j];
      float d = s + 1e-20f;
      for (size_t j = 0; j < k; ++j) weight[t * k + j] /= d;
    }
    if (scaling != 1.0f)
      for (size_t j = 0; j < k; ++j) weight[t * k + j] *= scaling;
  }
  return 0;
}

// The Inkling router with shared-expert sinks (src/models/inkling/block.rs:176-258, host twin of
// src/models/inkling/routetopk.rs): selection among the n_routed experts by sigmoid(logit) + bias
// (f32, descending, ties to the lower index); the weights are a softmax over log_sigmoid of the
// chosen routed logits followed by the n_shared sink logits, times route_scale, times global_scale.
// All arithmetic in f32 with the host's expf/logf, sums in index order. logits [tokens, n_routed +
// n_shared]. Returns 0, or 1 with the first non-finite (token, row) in bad[0..1] (the reference panics).
static float orc_sigmoid32(float x) {                     // block.rs:260-267
  if (x >= 0.0f) return 1.0f / (1.0f + std::exp(-x));
  float e = std::exp(x);
  return e / (1.0f + e);
}
static float orc_log_sigmoid32(float x) {                 // block.rs:20-26
  if (x >= 0.0f) return -std::log(1.0f + std::exp(-x));
  return x - std::log(1.0f + std::exp(x));
}
ORC_API int orc_router_sinks(const float* logits, const float* bias, float global_scale, float route_scale,
                             size_t tokens, size_t n_routed, size_t n_shared, size_t k, uint32_t* idx,
                             float* weight, float* gammas, size_t* bad) {
  const size_t rows = n_routed + n_shared;
  std::vector<uint32_t> order(n_routed);
  std::vector<float> score(n_routed), lp(k + n_shared);
  for (size_t t = 0; t < tokens; ++t) {
    const float* row = logits + t * rows;
    for (size_t r = 0; r < rows; ++r)
      if (!std::isfinite(row[r])) { bad[0] = t; bad[1] = r; return 1; }
    for (size_t e = 0; e < n_routed; ++e) score[e] = orc_sigmoid32(row[e]) + bias[e];
    std::iota(order.begin(), order.end(), 0u);
    std::sort(order.begin(), order.end(), [&](uint32_t a, uint32_t b) {
      if (score[a] != score[b]) return score[a] > score[b];
      return a < b;
    });
    for (size_t j = 0; j < k; ++j) { idx[t * k + j] = order[j]; lp[j] = orc_log_sigmoid32(row[order[j]]); }
    for (size_t j = 0; j < n_shared; ++j) lp[k + j] = orc_log_sigmoid32(row[n_routed + j]);
    float m = -std::numeric_limits<float>::infinity();
    for (float v : lp) m = std::max(m, v);
    float sum = 0.0f;
    for (float v : lp) sum += std::exp(v - m);
    const float lse = m + std::log(sum);
    for (size_t j = 0; j < k; ++j) weight[t * k + j] = std::exp(lp[j] - lse) * route_scale * global_scale;
    for (size_t j = 0; j < n_shared; ++j) gammas[t * n_shared + j] = std::exp(lp[k + j] - lse) * route_scale * global_scale;
  }
  return 0;
}

// Router logits from bf16 hidden states and a bf16 gate: f32 = sum in f64
// (router.rs:310-339, Accum::F64) of the widened operands.
ORC_API void orc_router_logits(const uint16_t* h, const uint16_t* gate, size_t tokens, size_t hid, size_t n,
                               float* logits) {
#pragma omp parallel for schedule(static)
  for (long long t = 0; t < (long long)tokens; ++t)
    for (size_t e = 0; e < n; ++e) {
      double s = 0.0;
      for (size_t j = 0; j < hid; ++j) s += double(bf16_to_f32(h[t * hid + j])) * double(bf16_to_f32(gate[e * hid + j]));
      logits[t * n + e] = float(s);
    }
}

// ---------------------------------------------------------------------------
// MoE row plan (src/models/inkling/assembly.rs:2865-2880 builds by_expert in token
// order; src/models/inkling/moegroup.rs:1850-1909 `RowPlan::build` stacks it)
// ---------------------------------------------------------------------------
// Experts ascending (BTreeMap order); only experts with at least one token get a
// slot. Each expert's rows are padded to `mtile`. Outputs sized by the caller:
// row_tok/row_wgt [m_cap], slot_expert/slot_row0/slot_rows [n_experts], tok_rows
// [tokens*k], tok_cnt [tokens]. Returns m_total (padded rows) or -1 if m_cap is
// too small. kmax_out = max(1, max tok_cnt); tok_rows is written [tokens, k] with
// the row stride k (the caller compacts to kmax when it wants the reference's shape).
ORC_API long long orc_row_plan(const uint32_t* idx, const float* weight, size_t tokens, size_t k,
                               size_t n_experts, size_t mtile, size_t m_cap, int32_t* row_tok, float* row_wgt,
                               uint32_t* slot_expert, uint32_t* slot_row0, uint32_t* slot_rows,
                               uint32_t* n_slots_out, uint32_t* tok_rows, uint32_t* tok_cnt, uint32_t* kmax_out) {
  std::vector<std::vector<std::pair<uint32_t, float>>> by_expert(n_experts);
  for (size_t t = 0; t < tokens; ++t)
    for (size_t j = 0; j < k; ++j) by_expert[idx[t * k + j]].push_back({uint32_t(t), weight[t * k + j]});
  for (size_t t = 0; t < tokens; ++t) tok_cnt[t] = 0;
  size_t row = 0, slot = 0;
  for (size_t e = 0; e < n_experts; ++e) {
    auto& toks = by_expert[e];
    if (toks.empty()) continue;
    size_t m = toks.size();
    size_t m_pad = (m + mtile - 1) / mtile * mtile;
    if (row + m_pad > m_cap) return -1;
    slot_expert[slot] = uint32_t(e);
    slot_row0[slot] = uint32_t(row);
    slot_rows[slot] = uint32_t(m);
    for (auto& tw : toks) {
      tok_rows[size_t(tw.first) * k + tok_cnt[tw.first]++] = uint32_t(row);
      row_tok[row] = int32_t(tw.first);
      row_wgt[row] = tw.second;
      ++row;
    }
    for (size_t p = m; p < m_pad; ++p) {
      row_tok[row] = -1;
      row_wgt[row] = 0.0f;
      ++row;
    }
    ++slot;
  }
  *n_slots_out = uint32_t(slot);
  uint32_t kmax = 1;
  for (size_t t = 0; t < tokens; ++t) kmax = std::max(kmax, tok_cnt[t]);
  *kmax_out = kmax;
  return (long long)row;
}

// src/models/inkling/moegroup.rs:313-331 (`gather_grouped_kernel`): idx<0 -> zero row.
ORC_API void orc_gather_rows_bf16(const uint16_t* src, const int32_t* row_tok, size_t m_total, size_t h,
                                  uint16_t* out) {
  for (size_t r = 0; r < m_total; ++r)
    for (size_t c = 0; c < h; ++c) out[r * h + c] = row_tok[r] < 0 ? 0 : src[size_t(row_tok[r]) * h + c];
}

// src/models/inkling/fp4gemm.rs:472-507 (`gate_up_silu`), f32 math; halved=0 is the
// interleaved g0,u0,g1,u1 reading. Output optionally rounded to bf16 (narrow lane).
ORC_API void orc_gate_up_silu(const float* both, size_t rows, size_t inter, int halved, int round_bf16_out,
                              float* act) {
  for (size_t r = 0; r < rows; ++r)
    for (size_t i = 0; i < inter; ++i) {
      float g, u;
      if (halved) {
        g = both[r * 2 * inter + i];
        u = both[r * 2 * inter + inter + i];
      } else {
        g = both[r * 2 * inter + 2 * i];
        u = both[r * 2 * inter + 2 * i + 1];
      }
      float a = (g / (1.0f + std::exp(-g))) * u;
      act[r * inter + i] = round_bf16_out ? round_bf16(a) : a;
    }
}

// src/models/inkling/moegroup.rs:1690-1716 (`scatter_weighted_kernel`): ascending
// rows, the multiply-add contracts to one fma per term.
ORC_API void orc_scatter_weighted(const float* y, const float* row_wgt, const uint32_t* tok_rows,
                                  const uint32_t* tok_cnt, size_t tokens, size_t k_stride, size_t h, float* out) {
#pragma omp parallel for schedule(static)
  for (long long t = 0; t < (long long)tokens; ++t)
    for (size_t c = 0; c < h; ++c) {
      float sum = 0.0f;
      for (uint32_t j = 0; j < tok_cnt[t]; ++j) {
        size_t r = tok_rows[size_t(t) * k_stride + j];
        sum = std::fmaf(y[r * h + c], row_wgt[r], sum);
      }
      out[size_t(t) * h + c] = sum;
    }
}

// The whole expert block of one MoE layer on the narrow (bf16-intermediate) lane:
// src/models/inkling/assembly.rs:3048-3075 (algorithm), :3429-3588 (launch order):
// gather -> quantize (fp4quant recipe) -> grouped GEMM w13 (x per-expert scale2,
// bf16) -> de-interleave + silu*up (bf16) -> quantize -> grouped GEMM w2 (bf16) ->
// ordered weighted sum (f32). Expert e's planes start at e*n13*h/2 (codes) etc.
ORC_API int orc_moe_experts(const uint16_t* x, size_t tokens, size_t h, size_t inter, size_t n_experts,
                            const uint32_t* idx, const float* weight, size_t k, const uint8_t* w13_codes,
                            const uint8_t* w13_scales, const float* w13_scale2, const uint8_t* w2_codes,
                            const uint8_t* w2_scales, const float* w2_scale2, int halved, float* out) {
  size_t m_cap = tokens * k;  // mtile = 1: padding-free
  std::vector<int32_t> row_tok(m_cap);
  std::vector<float> row_wgt(m_cap);
  std::vector<uint32_t> slot_e(n_experts), slot_r0(n_experts), slot_n(n_experts), tok_rows(tokens * k), tok_cnt(tokens);
  uint32_t n_slots = 0, kmax = 0;
  long long m_total = orc_row_plan(idx, weight, tokens, k, n_experts, 1, m_cap, row_tok.data(), row_wgt.data(),
                                   slot_e.data(), slot_r0.data(), slot_n.data(), &n_slots, tok_rows.data(),
                                   tok_cnt.data(), &kmax);
  if (m_total < 0) return -1;
  size_t M = size_t(m_total);
  std::vector<uint16_t> xg(M * h);
  orc_gather_rows_bf16(x, row_tok.data(), M, h, xg.data());
  std::vector<float> xf(M * h);
  for (size_t i = 0; i < M * h; ++i) xf[i] = bf16_to_f32(xg[i]);
  std::vector<uint8_t> a_codes(M * h / 2), a_scales(M * h / 16);
  orc_quantize_act_recip(xf.data(), M, h, a_codes.data(), a_scales.data());
  size_t n13 = 2 * inter;
  std::vector<float> both(M * n13);
  for (uint32_t s = 0; s < n_slots; ++s) {
    size_t e = slot_e[s], r0 = slot_r0[s], rows = slot_n[s];
    orc_linear_w4a4(a_codes.data() + r0 * h / 2, a_scales.data() + r0 * h / 16, w13_codes + e * n13 * h / 2,
                    w13_scales + e * n13 * h / 16, nullptr, w13_scale2[e], rows, n13, h, both.data() + r0 * n13);
  }
  for (auto& v : both) v = round_bf16(v);
  std::vector<float> act(M * inter);
  orc_gate_up_silu(both.data(), M, inter, halved, 1, act.data());
  std::vector<uint8_t> c2(M * inter / 2), s2(M * inter / 16);
  orc_quantize_act_recip(act.data(), M, inter, c2.data(), s2.data());
  std::vector<float> y(M * h);
  for (uint32_t s = 0; s < n_slots; ++s) {
    size_t e = slot_e[s], r0 = slot_r0[s], rows = slot_n[s];
    orc_linear_w4a4(c2.data() + r0 * inter / 2, s2.data() + r0 * inter / 16, w2_codes + e * h * inter / 2,
                    w2_scales + e * h * inter / 16, nullptr, w2_scale2[e], rows, h, inter, y.data() + r0 * h);
  }
  for (auto& v : y) v = round_bf16(v);
  orc_scatter_weighted(y.data(), row_wgt.data(), tok_rows.data(), tok_cnt.data(), tokens, k, h, out);
  return 0;
}

// ---------------------------------------------------------------------------
// Attention (src/models/inkling/flash.rs:1937-1987 `cpu_attention`, generalised to
// a `scale` argument; GQA kv_h = h / groups)
// ---------------------------------------------------------------------------
// q [nq, heads*D], k/v [keys, kv_heads*D] token-major f32. Query i sits at
// absolute position q0+i; key j at key_pos[j] (null -> j). window <= 0: none.
// rel (null -> none): [nq, heads, eff] f32, added to the scaled score of a visible key at
// distance dist = q_abs - k_abs < eff (flash.rs:1966-1972).
ORC_API int orc_attention_rel(const float* q, const float* k, const float* v, size_t nq, size_t keys, size_t heads,
                              size_t kv_heads, size_t D, size_t q0, const int64_t* key_pos, float scale,
                              long long window, const float* rel, size_t eff, double* out) {
  size_t q_row = heads * D, kv_row = kv_heads * D;
  int bad = 0;
#pragma omp parallel for schedule(dynamic, 4)
  for (long long qi = 0; qi < (long long)nq; ++qi) {
    size_t q_abs = q0 + size_t(qi);
    std::vector<std::pair<size_t, double>> scores;
    for (size_t h = 0; h < heads; ++h) {
      size_t qoff = size_t(qi) * q_row + h * D;
      size_t kvh = h / (heads / kv_heads);
      scores.clear();
      for (size_t ki = 0; ki < keys; ++ki) {
        size_t k_abs = key_pos ? size_t(key_pos[ki]) : ki;
        if (k_abs > q_abs || (window > 0 && q_abs - k_abs >= size_t(window))) continue;
        size_t koff = ki * kv_row + kvh * D;
        double dot = 0.0;
        for (size_t d = 0; d < D; ++d) dot += double(q[qoff + d]) * double(k[koff + d]);
        const size_t dist = q_abs - k_abs;
        const double bias = (rel && dist < eff) ? double(rel[(size_t(qi) * heads + h) * eff + dist]) : 0.0;
        scores.push_back({koff, dot * double(scale) + bias});
      }
      for (size_t d = 0; d < D; ++d) out[qoff + d] = 0.0;
      if (scores.empty()) { bad = 1; continue; }
      double mx = -std::numeric_limits<double>::infinity();
      for (auto& s : scores) mx = std::max(mx, s.second);
      double denom = 0.0;
      for (auto& s : scores) denom += std::exp(s.second - mx);
      for (auto& s : scores) {
        double p = std::exp(s.second - mx) / denom;
        for (size_t d = 0; d < D; ++d) out[qoff + d] += p * double(v[s.first + d]);
      }
    }
  }
  return bad ? -1 : 0;
}

ORC_API int orc_attention(const float* q, const float* k, const float* v, size_t nq, size_t keys, size_t heads,
                          size_t kv_heads, size_t D, size_t q0, const int64_t* key_pos, float scale,
                          long long window, double* out) {
  return orc_attention_rel(q, k, v, nq, keys, heads, kv_heads, D, q0, key_pos, scale, window, nullptr, 0, out);
}

// ---------------------------------------------------------------------------
// Decoder-layer glue with the reference's bf16 rounding points
// ---------------------------------------------------------------------------

// src/models/breeze/cuda_ops.rs:88-117 (`norm_kernel`, gemma=false): f32 sum of
// squares in index order, inv = 1/sqrt(mean+eps), bf16(x*inv) then bf16(.*gain).
ORC_API void orc_rmsnorm_breeze(const uint16_t* x, const uint16_t* w, size_t rows, size_t width, float eps,
                                uint16_t* y) {
  for (size_t r = 0; r < rows; ++r) {
    float sum = 0.0f;
    for (size_t j = 0; j < width; ++j) {
      float v = bf16_to_f32(x[r * width + j]);
      sum += v * v;
    }
    float inv = 1.0f / std::sqrt(sum / float(width) + eps);
    for (size_t j = 0; j < width; ++j) {
      float value = bf16_to_f32(x[r * width + j]) * inv;
      float normalized = round_bf16(value);
      y[r * width + j] = f32_to_bf16(normalized * bf16_to_f32(w[j]));
    }
  }
}

// src/models/inkling/resid.rs:272-322 (`rms_norm_kernel`), the Inkling convention: every element widened to f32,
// `units` = min(256, next power of two of h) partial sums (unit u adds elements u, u + units, ... in turn), a
// halving tree over the partials, denom = sqrt(red[0] / h + eps), out = O(v / denom * gain[j]) with an f32 gain:
// one rounding. The reference's kernel source reaches the GPU through a run-time compiler that contracts
// `acc += v * v` into a fused multiply-add, stated here explicitly (this file is built with contraction off).
// x: bf16 bits (x_bf16) or f32 (x_f32), exactly one non-null; out_bf16 or out_f32 likewise.
ORC_API void orc_rmsnorm_inkling(const uint16_t* x_bf16, const float* x_f32, const float* gain, size_t rows, size_t h,
                                 float eps, uint16_t* out_bf16, float* out_f32) {
  size_t units = 1;
  while (units < h && units < 256) units *= 2;
  std::vector<float> v(h), red(units);
  for (size_t r = 0; r < rows; ++r) {
    for (size_t j = 0; j < h; ++j) v[j] = x_bf16 ? bf16_to_f32(x_bf16[r * h + j]) : x_f32[r * h + j];
    for (size_t u = 0; u < units; ++u) {
      float acc = 0.0f;
      for (size_t i = u; i < h; i += units) acc = std::fmaf(v[i], v[i], acc);
      red[u] = acc;
    }
    for (size_t step = units / 2; step > 0; step /= 2)
      for (size_t u = 0; u < step; ++u) red[u] += red[u + step];
    const float denom = std::sqrt(red[0] / float(h) + eps);
    for (size_t j = 0; j < h; ++j) {
      const float o = v[j] / denom * gain[j];
      if (out_bf16) out_bf16[r * h + j] = f32_to_bf16(o); else out_f32[r * h + j] = o;
    }
  }
}

// src/models/breeze/cuda_ops.rs:230-255 mode 0 (add) and mode 2 (swiglu).
ORC_API void orc_add_bf16(const uint16_t* a, const uint16_t* b, size_t n, uint16_t* out) {
  for (size_t i = 0; i < n; ++i) out[i] = f32_to_bf16(bf16_to_f32(a[i]) + bf16_to_f32(b[i]));
}
ORC_API void orc_swiglu_bf16(const uint16_t* gate, const uint16_t* up, size_t n, uint16_t* out) {
  for (size_t i = 0; i < n; ++i) {
    float x = bf16_to_f32(gate[i]);
    float activated = round_bf16(x / (1.0f + std::exp(-x)));
    out[i] = f32_to_bf16(activated * bf16_to_f32(up[i]));
  }
}

// src/models/breeze/cuda_ops.rs:286-320 (`rope_kernel`): half-split rotation,
// cos/sin rounded to bf16, each product rounded to bf16. x is [rows*heads, d]
// with position = past + row/heads. inv_freq[f] = theta^(-2f/d) as f32.
ORC_API void orc_rope_bf16(const uint16_t* x, size_t tokens, size_t heads, size_t d, size_t past,
                           const float* inv_freq, uint16_t* out) {
  size_t half = d / 2;
  for (size_t row = 0; row < tokens * heads; ++row) {
    size_t position = past + row / heads;
    for (size_t j = 0; j < d; ++j) {
      size_t f = j % half;
      float angle = float(position) * inv_freq[f];
      float c = round_bf16(std::cos(angle));
      float s = round_bf16(std::sin(angle));
      float low = bf16_to_f32(x[row * d + f]);
      float high = bf16_to_f32(x[row * d + half + f]);
      if (j < half)
        out[row * d + j] = f32_to_bf16(round_bf16(low * c) - round_bf16(high * s));
      else
        out[row * d + j] = f32_to_bf16(round_bf16(high * c) + round_bf16(low * s));
    }
  }
}

// ---------------------------------------------------------------------------
// Tensor-parallel shard arithmetic (src/models/inkling/tp.rs:540-555 `shard`)
// ---------------------------------------------------------------------------
ORC_API int orc_tp_shard(size_t rank, size_t world, size_t extent, size_t* lo, size_t* hi) {
  if (world == 0 || rank >= world || extent % world != 0) return -1;
  size_t per = extent / world;
  *lo = rank * per;
  *hi = (rank + 1) * per;
  return 0;
}

// ---------------------------------------------------------------------------
// Fixture generator: splitmix64 + Box-Muller (src/nn/nvfp4_gemv.rs:610-636)
// ---------------------------------------------------------------------------
ORC_API void orc_rng_normal_f32(uint64_t seed, size_t n, double sigma, float* out) {
  SplitMix r{seed};
  for (size_t i = 0; i < n; ++i) out[i] = float(r.normal() * sigma);
}
ORC_API void orc_rng_normal_bf16(uint64_t seed, size_t n, double sigma, uint16_t* out) {
  SplitMix r{seed};
  for (size_t i = 0; i < n; ++i) out[i] = f32_to_bf16(float(r.normal() * sigma));
}

// The deterministic sign-mixed sample of src/nvfp4.rs:385-394.
ORC_API void orc_sample(size_t rows, size_t cols, float* out) {
  for (size_t i = 0; i < rows * cols; ++i) {
    float r = float(i / cols) + 1.0f;
    float x = float((i * 7919) % 1000) / 1000.0f - 0.5f;
    out[i] = x * r * 0.37f;
  }
}

ORC_API int orc_threads() {
#if defined(_OPENMP)
  return omp_get_max_threads();
#else
  return 1;
#endif
}
ORC_API void orc_set_threads(int n) {
#if defined(_OPENMP)
  omp_set_num_threads(n);
#else
  (void)n;
#endif
}
