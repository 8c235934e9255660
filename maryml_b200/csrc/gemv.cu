// W4A16 GEMV over resident NVFP4 planes: [rows <= 8, k] x [n, k]^T.
//
// HBM-bound weight streaming: 0.5625 bytes per weight, read once. One warp per
// output row; a lane takes 32 consecutive weights per step (one 16-byte code load,
// two scale bytes) so a warp's code loads are contiguous 512-byte lines; the K loop
// is unrolled so several loads are in flight per lane. Products accumulate in f32
// per 16-block, are scaled by the block's E4M3 once, carried across K in f32, summed
// across the warp, multiplied by scale2 once and cast once.
#include "common.cuh"

#include <cuda_fp16.h>

namespace {

constexpr int GEMV_WARPS = 4;
constexpr int MAX_ROWS = 8;

// Two E2M1 codes of one byte -> two f32, through the hardware's e2m1x2 -> f16x2 convert.
__device__ __forceinline__ float2 e2m1x2_to_f32(uint32_t byte) {
  uint32_t h2;
  asm("{ .reg .b8 t; cvt.u8.u32 t, %1; cvt.rn.f16x2.e2m1x2 %0, t; }" : "=r"(h2) : "r"(byte));
  __half2 h = *reinterpret_cast<__half2*>(&h2);
  return __half22float2(h);
}

// sum_i x[i] * E2M1[nibble i of word] over the eight nibbles of one word.
__device__ __forceinline__ float dot8(uint32_t word, const uint4& xv) {
  const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
  float acc = 0.0f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 w = e2m1x2_to_f32((word >> (8 * i)) & 0xFFu);
    acc = fmaf(__uint_as_float(xw[i] << 16), w.x, acc);
    acc = fmaf(__uint_as_float(xw[i] & 0xFFFF0000u), w.y, acc);
  }
  return acc;
}

template <int ROWS, typename O>
__global__ void __launch_bounds__(32 * GEMV_WARPS)
gemv_w4a16_kernel(const uint4* __restrict__ x, const uint4* __restrict__ codes, const uint8_t* __restrict__ scales,
                  O* __restrict__ out, uint32_t n, uint32_t k, float scale2) {
  const uint32_t lane = threadIdx.x & 31;
  const uint32_t row = blockIdx.x * GEMV_WARPS + (threadIdx.x >> 5);
  if (row >= n) return;   // uniform per warp
  const uint32_t chunks = k / 32;
  float acc[ROWS];
#pragma unroll
  for (int r = 0; r < ROWS; ++r) acc[r] = 0.0f;
  const uint4* crow = codes + size_t(row) * chunks;
  const uint16_t* srow = reinterpret_cast<const uint16_t*>(scales + size_t(row) * (k / 16));
#pragma unroll 4
  for (uint32_t c = lane; c < chunks; c += 32) {
    const uint4 words = __ldg(crow + c);
    const uint32_t s01 = __ldg(srow + c);
    // both scale bytes through one e4m3x2 -> f16x2 convert (f16 holds every E4M3 value exactly)
    uint32_t sh2;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(sh2) : "h"(uint16_t(s01)));
    const float2 s01f = __half22float2(*reinterpret_cast<__half2*>(&sh2));
    const float s0 = s01f.x, s1 = s01f.y;
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      const uint4* xr = x + (size_t(r) * k + size_t(c) * 32) / 8;
      float b0 = dot8(words.x, __ldg(xr)) + dot8(words.y, __ldg(xr + 1));
      float b1 = dot8(words.z, __ldg(xr + 2)) + dot8(words.w, __ldg(xr + 3));
      acc[r] += b0 * s0 + b1 * s1;
    }
  }
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    float t = acc[r];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xFFFFFFFFu, t, o);
    if (lane == 0) out[size_t(r) * n + row] = O(t * scale2);
  }
}

template <typename O>
int launch_rows(cudaStream_t stream, size_t rows, const void* x, const uint8_t* codes, const uint8_t* scales, O* out,
                uint32_t n, uint32_t k, float scale2) {
  dim3 grid((n + GEMV_WARPS - 1) / GEMV_WARPS), block(32 * GEMV_WARPS);
  const uint4* xv = static_cast<const uint4*>(x);
  const uint4* cv = reinterpret_cast<const uint4*>(codes);
  switch (rows) {
#define CASE(R) case R: gemv_w4a16_kernel<R, O><<<grid, block, 0, stream>>>(xv, cv, scales, out, n, k, scale2); break;
    CASE(1) CASE(2) CASE(3) CASE(4) CASE(5) CASE(6) CASE(7) CASE(8)
#undef CASE
    default: return -1;
  }
  return 0;
}

}  // namespace

MB_API int mb_nvfp4_gemv_w4a16(mb_ctx* ctx, mb_stream stream_, const void* x_bf16, size_t rows, const uint8_t* codes,
                               const uint8_t* scales, float scale2, size_t n, size_t k, void* out, int out_dtype) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  MB_REQUIRE(ctx, ctx && x_bf16 && codes && scales && out, "gemv: null argument");
  MB_REQUIRE(ctx, rows >= 1 && rows <= MAX_ROWS, "NVFP4 GEMV takes 1..=%d rows", MAX_ROWS);
  MB_REQUIRE(ctx, n > 0 && k > 0 && k % 32 == 0, "NVFP4 weight [%zu, %zu] needs k a multiple of 32", n, k);
  MB_REQUIRE(ctx, n * k <= 0xFFFFFFFFull, "NVFP4 weight exceeds u32 indexing");
  MB_REQUIRE(ctx, scale2 == scale2 && scale2 > 0.0f && scale2 <= 3.4e38f,
             "NVFP4 global scale %g is not a positive finite number", double(scale2));
  MB_REQUIRE(ctx, mb_aligned(x_bf16, 16), "NVFP4 GEMV needs a 16-byte aligned activation");
  MB_REQUIRE(ctx, mb_aligned(codes, 16) && mb_aligned(scales, 2), "NVFP4 GEMV needs 16-byte aligned code rows");
  int rc;
  if (out_dtype == MB_DT_BF16)
    rc = launch_rows(stream, rows, x_bf16, codes, scales, static_cast<__nv_bfloat16*>(out), uint32_t(n), uint32_t(k), scale2);
  else if (out_dtype == MB_DT_F32)
    rc = launch_rows(stream, rows, x_bf16, codes, scales, static_cast<float*>(out), uint32_t(n), uint32_t(k), scale2);
  else
    return mb_fail(ctx, MB_ERR_INVALID, "gemv: output is bf16 or f32");
  if (rc) return mb_fail(ctx, MB_ERR_INVALID, "gemv: unsupported row count");
  MB_LAUNCH_OK(ctx);
  return MB_OK;
}
