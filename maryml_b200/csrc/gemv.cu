// W4A16 GEMV over resident NVFP4 planes: [rows <= 8, k] x [n, k]^T.
//
// HBM-bound weight streaming: 0.5625 bytes per weight, read once. The dot products run on the
// tensor cores (mma.sync m16n8k16, bf16 x bf16 -> f32): 16 weight rows are the M side, the up to
// eight activation rows the N side, so one to eight rows cost the same. A decoded weight times
// its block scale has at most 7 significant bits (E2M1 x E4M3), so w * s is exact in f16 and in
// bf16 and every product x * (w s) is exact in f32; only the order of the f32 sums differs from
// a scalar loop. Decode per pair of weights: cvt.e2m1x2 -> f16x2, one f16x2 multiply by the
// scale, f16 -> f32 -> bf16x2 (all exact).
//
// A block of eight warps owns 16 weight rows; warp w takes every eighth 128-value slice of K
// (split-K inside the block keeps ~14 warps per SM busy and many loads in flight), the eight
// partial tiles are summed in warp order through shared memory. Inside a slice lane (g, t)
// loads 32 consecutive weights of rows g and g + 8 (one 16-byte load each) and the matching 32
// activations of row g; the instruction's K slots are a permutation of those 128 values that
// is the same for both operands, which is all the product needs.
#include "common.cuh"

#include <cuda_fp16.h>

namespace {

constexpr int GEMV_WARPS = 8;
constexpr int MAX_ROWS = 8;

// Four weights (two bytes of codes) times their block scale -> two bf16x2 registers.
__device__ __forceinline__ void decode4(uint32_t two_bytes, __half2 s, uint32_t& lo, uint32_t& hi) {
  uint32_t h0, h1;
  asm("{ .reg .b8 b0, b1, b2, b3; mov.b32 {b0, b1, b2, b3}, %2;\n\t"
      "cvt.rn.f16x2.e2m1x2 %0, b0;\n\tcvt.rn.f16x2.e2m1x2 %1, b1; }"
      : "=r"(h0), "=r"(h1) : "r"(two_bytes));
  const float2 f0 = __half22float2(__hmul2(*reinterpret_cast<__half2*>(&h0), s));
  const float2 f1 = __half22float2(__hmul2(*reinterpret_cast<__half2*>(&h1), s));
  __nv_bfloat162 p0 = __floats2bfloat162_rn(f0.x, f0.y), p1 = __floats2bfloat162_rn(f1.x, f1.y);
  lo = *reinterpret_cast<uint32_t*>(&p0);
  hi = *reinterpret_cast<uint32_t*>(&p1);
}

__device__ __forceinline__ void mma_bf16(float* d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
               "{%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <typename O>
__global__ void __launch_bounds__(32 * GEMV_WARPS)
gemv_w4a16_kernel(const uint4* __restrict__ x, const uint4* __restrict__ codes, const uint8_t* __restrict__ scales,
                  O* __restrict__ out, uint32_t rows, uint32_t n, uint32_t k, float scale2) {
  __shared__ float part[GEMV_WARPS][16][8];
  const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t g = lane >> 2, t = lane & 3;
  const uint32_t row_base = blockIdx.x * 16;
  const uint32_t r0 = min(row_base + g, n - 1), r1 = min(row_base + g + 8, n - 1);   // loads stay inside the planes
  const uint32_t slices = (k + 127) / 128;
  const uint4* c0 = codes + size_t(r0) * (k / 32);
  const uint4* c1 = codes + size_t(r1) * (k / 32);
  const uint16_t* s0p = reinterpret_cast<const uint16_t*>(scales + size_t(r0) * (k / 16));
  const uint16_t* s1p = reinterpret_cast<const uint16_t*>(scales + size_t(r1) * (k / 16));
  const uint4* xr = x + size_t(g) * (k / 8);
  const bool x_live = g < rows;
  float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  constexpr int U = 4;                                   // slices whose weight loads are in flight together
  for (uint32_t sl0 = warp; sl0 < slices; sl0 += GEMV_WARPS * U) {
    uint4 wa[U], wb[U];
    uint32_t sa[U], sb[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint32_t k0 = (sl0 + u * GEMV_WARPS) * 128 + t * 32;    // this lane's 32 values of the slice
      const bool live = k0 < k;                            // k is a multiple of 32: a group is whole or absent
      wa[u] = live ? __ldg(c0 + k0 / 32) : make_uint4(0u, 0u, 0u, 0u);
      wb[u] = live ? __ldg(c1 + k0 / 32) : make_uint4(0u, 0u, 0u, 0u);
      sa[u] = live ? uint32_t(__ldg(s0p + k0 / 32)) : 0u;
      sb[u] = live ? uint32_t(__ldg(s1p + k0 / 32)) : 0u;
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint32_t k0 = (sl0 + u * GEMV_WARPS) * 128 + t * 32;
      if (sl0 + u * GEMV_WARPS >= slices) break;           // warp-uniform: the MMAs below need the whole warp
      const bool live = x_live && k0 < k;                  // a lane beyond k in the last slice holds zero weights
      uint4 xv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) xv[i] = live ? __ldg(xr + k0 / 8 + i) : make_uint4(0u, 0u, 0u, 0u);
      // both scale bytes of a row through one e4m3x2 -> f16x2 convert (f16 holds every E4M3 value exactly)
      uint32_t sah, sbh;
      asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(sah) : "h"(uint16_t(sa[u])));
      asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(sbh) : "h"(uint16_t(sb[u])));
      const __half2 sa2 = *reinterpret_cast<__half2*>(&sah), sb2 = *reinterpret_cast<__half2*>(&sbh);
      const __half2 sa_lo = __low2half2(sa2), sa_hi = __high2half2(sa2);
      const __half2 sb_lo = __low2half2(sb2), sb_hi = __high2half2(sb2);
      const uint32_t wwa[4] = {wa[u].x, wa[u].y, wa[u].z, wa[u].w}, wwb[4] = {wb[u].x, wb[u].y, wb[u].z, wb[u].w};
#pragma unroll
      for (int i = 0; i < 8; ++i) {                      // instruction i takes values 4 i .. 4 i + 3 of the 32
        const uint32_t ba = (wwa[i >> 1] >> ((i & 1) * 16)) & 0xFFFFu, bb = (wwb[i >> 1] >> ((i & 1) * 16)) & 0xFFFFu;
        uint32_t a0, a1, a2, a3;
        decode4(ba, i < 4 ? sa_lo : sa_hi, a0, a2);      // row g:     slots (2t, 2t+1) and (2t+8, 2t+9)
        decode4(bb, i < 4 ? sb_lo : sb_hi, a1, a3);      // row g + 8
        const uint4& xq = xv[i >> 1];
        const uint32_t b0 = (i & 1) ? xq.z : xq.x, b1 = (i & 1) ? xq.w : xq.y;
        mma_bf16(acc, a0, a1, a2, a3, b0, b1);
      }
    }
  }
  // acc[0], acc[1]: weight row g, activation rows 2t, 2t+1; acc[2], acc[3]: weight row g + 8
  part[warp][g][2 * t] = acc[0];
  part[warp][g][2 * t + 1] = acc[1];
  part[warp][g + 8][2 * t] = acc[2];
  part[warp][g + 8][2 * t + 1] = acc[3];
  __syncthreads();
  if (threadIdx.x < 128) {
    const uint32_t wr = threadIdx.x >> 3, ar = threadIdx.x & 7;
    float sum = 0.0f;
#pragma unroll
    for (int w = 0; w < GEMV_WARPS; ++w) sum += part[w][wr][ar];
    if (ar < rows && row_base + wr < n) out[size_t(ar) * n + row_base + wr] = O(sum * scale2);
  }
}

template <typename O>
int launch_rows(cudaStream_t stream, size_t rows, const void* x, const uint8_t* codes, const uint8_t* scales, O* out,
                uint32_t n, uint32_t k, float scale2) {
  dim3 grid((n + 15) / 16), block(32 * GEMV_WARPS);
  gemv_w4a16_kernel<O><<<grid, block, 0, stream>>>(static_cast<const uint4*>(x), reinterpret_cast<const uint4*>(codes),
                                                   scales, out, uint32_t(rows), n, k, scale2);
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
