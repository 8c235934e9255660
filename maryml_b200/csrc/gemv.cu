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
#include "quant_block.cuh"

#include <cuda_fp16.h>

namespace {

constexpr int GEMV_WARPS = 8;
constexpr int MAX_ROWS = 8;

// A block scale (an E4M3 value held as f16) as the bf16x2 multiplier of decode4: scale * 2^112 in both halves
// (four significant bits and at most 448 * 2^112: exact and finite in bf16).
__device__ __forceinline__ __nv_bfloat162 scale_bf16x2(__half2 s_both) {
  return __float2bfloat162_rn(__low2float(s_both) * 5.192296858534828e33f);
}

// Four weights (two bytes of codes) times their block scale -> two bf16x2 registers, without leaving 16-bit
// registers: an E2M1 value as f16 is zero or a normal number, and its f16 pattern shifted three places to the right
// (sign kept in place) is the bf16 pattern of the value times 2^-112; one packed bf16 multiply by scale * 2^112
// gives value * scale, exact (at most six significant bits, no intermediate below the normal range).
__device__ __forceinline__ void decode4(uint32_t two_bytes, __nv_bfloat162 s, uint32_t& lo, uint32_t& hi) {
  uint32_t h0, h1;
  asm("{ .reg .b8 b0, b1, b2, b3; mov.b32 {b0, b1, b2, b3}, %2;\n\t"
      "cvt.rn.f16x2.e2m1x2 %0, b0;\n\tcvt.rn.f16x2.e2m1x2 %1, b1; }"
      : "=r"(h0), "=r"(h1) : "r"(two_bytes));
  h0 = ((h0 >> 3) & 0x0FFF0FFFu) | (h0 & 0x80008000u);
  h1 = ((h1 >> 3) & 0x0FFF0FFFu) | (h1 & 0x80008000u);
  const __nv_bfloat162 p0 = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&h0), s);
  const __nv_bfloat162 p1 = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&h1), s);
  lo = *reinterpret_cast<const uint32_t*>(&p0);
  hi = *reinterpret_cast<const uint32_t*>(&p1);
}

__device__ __forceinline__ void mma_bf16(float* d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
               "{%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Four weights (two bytes of codes) times their block scale -> two f16x2 registers (exact, no further conversion).
__device__ __forceinline__ void decode4_f16(uint32_t two_bytes, __half2 s, uint32_t& lo, uint32_t& hi) {
  uint32_t h0, h1;
  asm("{ .reg .b8 b0, b1, b2, b3; mov.b32 {b0, b1, b2, b3}, %2;\n\t"
      "cvt.rn.f16x2.e2m1x2 %0, b0;\n\tcvt.rn.f16x2.e2m1x2 %1, b1; }"
      : "=r"(h0), "=r"(h1) : "r"(two_bytes));
  const __half2 p0 = __hmul2(*reinterpret_cast<__half2*>(&h0), s), p1 = __hmul2(*reinterpret_cast<__half2*>(&h1), s);
  lo = *reinterpret_cast<const uint32_t*>(&p0);
  hi = *reinterpret_cast<const uint32_t*>(&p1);
}
__device__ __forceinline__ void mma_f16_acc(float* d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                            uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
               "{%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// The body of the GEMV for one block of 16 weight rows. F16 = false: activations are the caller's bf16 rows and the
// decoded weights go f16 -> f32 -> bf16 for the bf16 product. F16 = true: activations are an f16 copy of the rows
// (exact: the conversion pass refuses values f16 cannot hold), the decoded weights stay f16, and the expansion costs
// five instructions per four weights instead of eleven, which is what separates an instruction-bound kernel from
// one that streams weights at the HBM rate.
// K slices (128 values each) may be cut into `ksplit` ranges over blockIdx.y, so that a weight with few rows and a
// long K still puts several blocks on every SM: each range's sums go to `partials` and the block that arrives last
// at the row block's counter adds them in range order (deterministic) and stores the result.
struct GemvSplit {
  uint32_t ksplit;          // 1: no split, the fields below are unused
  float* partials;          // [ksplit][row blocks][16 weight rows x 8 activation rows]
  int* counters;            // one per row block, zero between calls
  int cluster;              // the ranges of a row block are the CTAs of one cluster (1, ksplit, 1) and meet in shared memory
};

// Thread-block cluster primitives of the K-split that needs no workspace.
__device__ __forceinline__ void gemv_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release;\n\tbarrier.cluster.wait.acquire;" ::: "memory");
}
__device__ __forceinline__ float gemv_ld_cluster(const float* own, uint32_t rank) {
  uint32_t a = uint32_t(__cvta_generic_to_shared(own)), r;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(r) : "memory");
  return v;
}

// The warps' sums of one row block meet in shared memory; with a K split the ranges' sums meet in the workspace.
template <typename O>
__device__ __forceinline__ void gemv_finish(const float* acc, O* __restrict__ out, uint32_t rows, uint32_t n, float scale2,
                                            float (*part)[16][8], const GemvSplit& sp) {
  const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t g = lane >> 2, t = lane & 3;
  const uint32_t row_base = blockIdx.x * 16;
  // acc[0], acc[1]: weight row g, activation rows 2t, 2t+1; acc[2], acc[3]: weight row g + 8
  part[warp][g][2 * t] = acc[0];
  part[warp][g][2 * t + 1] = acc[1];
  part[warp][g + 8][2 * t] = acc[2];
  part[warp][g + 8][2 * t + 1] = acc[3];
  __syncthreads();
  const uint32_t wr = (threadIdx.x >> 3) & 15, ar = threadIdx.x & 7;
  float sum = 0.0f;
  if (threadIdx.x < 128) {
#pragma unroll
    for (int w = 0; w < GEMV_WARPS; ++w) sum += part[w][wr][ar];
  }
  if (sp.ksplit > 1 && sp.cluster) {
    // every CTA of the cluster parks its range's sums; the first one adds them in range order
    __shared__ float s_range[128];
    if (threadIdx.x < 128) s_range[threadIdx.x] = sum;
    gemv_cluster_sync();
    if (blockIdx.y == 0 && threadIdx.x < 128) {
      sum = 0.0f;
      for (uint32_t y = 0; y < sp.ksplit; ++y) sum += gemv_ld_cluster(s_range + threadIdx.x, y);
      if (ar < rows && row_base + wr < n) out[size_t(ar) * n + row_base + wr] = O(sum * scale2);
    }
    gemv_cluster_sync();               // no CTA leaves while the first may still read its sums
    return;
  }
  if (sp.ksplit > 1) {
    __shared__ int s_last;
    const size_t stride = size_t(gridDim.x) * 128;
    if (threadIdx.x < 128) sp.partials[blockIdx.y * stride + size_t(blockIdx.x) * 128 + threadIdx.x] = sum;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_last = atomicAdd(sp.counters + blockIdx.x, 1) == int(sp.ksplit) - 1;
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    if (threadIdx.x == 0) sp.counters[blockIdx.x] = 0;                 // ready for the next call
    sum = 0.0f;
    if (threadIdx.x < 128)
      for (uint32_t y = 0; y < sp.ksplit; ++y) sum += __ldcg(sp.partials + y * stride + size_t(blockIdx.x) * 128 + threadIdx.x);
  }
  if (threadIdx.x < 128 && ar < rows && row_base + wr < n) out[size_t(ar) * n + row_base + wr] = O(sum * scale2);
}

template <bool F16, typename O>
__device__ __forceinline__ void gemv_body(const uint4* __restrict__ x, const uint4* __restrict__ codes,
                                          const uint8_t* __restrict__ scales, O* __restrict__ out, uint32_t rows, uint32_t n,
                                          uint32_t k, float scale2, float (*part)[16][8], const GemvSplit& sp) {
  const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t g = lane >> 2, t = lane & 3;
  const uint32_t row_base = blockIdx.x * 16;
  const uint32_t r0 = min(row_base + g, n - 1), r1 = min(row_base + g + 8, n - 1);   // loads stay inside the planes
  const uint32_t all_slices = (k + 127) / 128;
  const uint32_t per_split = (all_slices + sp.ksplit - 1) / sp.ksplit;
  const uint32_t sl_begin = blockIdx.y * per_split, slices = min(all_slices, sl_begin + per_split);
  const uint4* c0 = codes + size_t(r0) * (k / 32);
  const uint4* c1 = codes + size_t(r1) * (k / 32);
  const uint16_t* s0p = reinterpret_cast<const uint16_t*>(scales + size_t(r0) * (k / 16));
  const uint16_t* s1p = reinterpret_cast<const uint16_t*>(scales + size_t(r1) * (k / 16));
  const uint4* xr = x + size_t(g) * (k / 8);
  const bool x_live = g < rows;
  float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  constexpr int U = 4;                                   // slices whose weight loads are in flight together
  for (uint32_t sl0 = sl_begin + warp; sl0 < slices; sl0 += GEMV_WARPS * U) {
    uint4 wa[U], wb[U];
    uint32_t sa[U], sb[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint32_t k0 = (sl0 + u * GEMV_WARPS) * 128 + t * 32;    // this lane's 32 values of the slice
      const bool live = sl0 + u * GEMV_WARPS < slices && k0 < k;   // k is a multiple of 32: a group is whole or absent
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
      __nv_bfloat162 qa_lo, qa_hi, qb_lo, qb_hi;
      if (!F16) { qa_lo = scale_bf16x2(sa_lo); qa_hi = scale_bf16x2(sa_hi); qb_lo = scale_bf16x2(sb_lo); qb_hi = scale_bf16x2(sb_hi); }
      const uint32_t wwa[4] = {wa[u].x, wa[u].y, wa[u].z, wa[u].w}, wwb[4] = {wb[u].x, wb[u].y, wb[u].z, wb[u].w};
#pragma unroll
      for (int i = 0; i < 8; ++i) {                      // instruction i takes values 4 i .. 4 i + 3 of the 32
        const uint32_t ba = (wwa[i >> 1] >> ((i & 1) * 16)) & 0xFFFFu, bb = (wwb[i >> 1] >> ((i & 1) * 16)) & 0xFFFFu;
        uint32_t a0, a1, a2, a3;
        const uint4& xq = xv[i >> 1];
        const uint32_t b0 = (i & 1) ? xq.z : xq.x, b1 = (i & 1) ? xq.w : xq.y;
        if (F16) {
          decode4_f16(ba, i < 4 ? sa_lo : sa_hi, a0, a2);
          decode4_f16(bb, i < 4 ? sb_lo : sb_hi, a1, a3);
          mma_f16_acc(acc, a0, a1, a2, a3, b0, b1);
        } else {
          decode4(ba, i < 4 ? qa_lo : qa_hi, a0, a2);    // row g:     slots (2t, 2t+1) and (2t+8, 2t+9)
          decode4(bb, i < 4 ? qb_lo : qb_hi, a1, a3);    // row g + 8
          mma_bf16(acc, a0, a1, a2, a3, b0, b1);
        }
      }
    }
  }
  gemv_finish(acc, out, rows, n, scale2, part, sp);
}

// The same product with the weight bytes streamed through a ring of cp.async copies per warp (k % 128 == 0).
// In the body above a warp holds four slices of loads in registers, computes, and only then asks for more; two
// blocks fit an SM, so about 64 KB per SM are in flight, with gaps. Here every warp keeps GEMV_RING slices (16
// weight rows x 64 code bytes + 16 x 8 scale bytes each) in flight in shared memory all the time, three blocks fit
// an SM, and the next slice's activation chunk is loaded while the current one is multiplied. A lane copies the two
// 16-byte code chunks it will itself read; lanes 0-15 copy one row's eight scale bytes, which other lanes read, so
// a __syncwarp stands on both sides of a slot's use.
constexpr int GEMV_RING = 5;
constexpr int GEMV_SLICE_BYTES = 16 * 64 + 16 * 8;
constexpr int GEMV_RING_SMEM = GEMV_WARPS * GEMV_RING * GEMV_SLICE_BYTES;

template <bool F16, typename O>
__device__ __forceinline__ void gemv_body_ring(const uint4* __restrict__ x, const uint4* __restrict__ codes,
                                               const uint8_t* __restrict__ scales, O* __restrict__ out, uint32_t rows,
                                               uint32_t n, uint32_t k, float scale2, float (*part)[16][8],
                                               const GemvSplit& sp, uint8_t* ring_all) {
  const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t g = lane >> 2, t = lane & 3;
  const uint32_t row_base = blockIdx.x * 16;
  const uint32_t r0 = min(row_base + g, n - 1), r1 = min(row_base + g + 8, n - 1);   // loads stay inside the planes
  const uint32_t all_slices = k / 128;
  const uint32_t per_split = (all_slices + sp.ksplit - 1) / sp.ksplit;
  const uint32_t sl_begin = blockIdx.y * per_split, sl_end = min(all_slices, sl_begin + per_split);
  // this warp's slices: sl_begin + warp, + GEMV_WARPS, ...
  const uint32_t first = sl_begin + warp;
  const uint32_t mine = first < sl_end ? (sl_end - first + GEMV_WARPS - 1) / GEMV_WARPS : 0u;
  uint8_t* ring = ring_all + warp * (GEMV_RING * GEMV_SLICE_BYTES);
  const uint32_t ring_s = uint32_t(__cvta_generic_to_shared(ring));
  const uint8_t* c0 = reinterpret_cast<const uint8_t*>(codes) + size_t(r0) * (k / 2) + t * 16;
  const uint8_t* c1 = reinterpret_cast<const uint8_t*>(codes) + size_t(r1) * (k / 2) + t * 16;
  const uint8_t* sc = scales + size_t(min(row_base + (lane & 15u), n - 1)) * (k / 16);
  auto issue = [&](uint32_t j) {                       // j-th slice of this warp; an empty group keeps the count uniform
    if (j < mine) {
      const uint32_t sl = first + j * GEMV_WARPS;
      const uint32_t dst = ring_s + (j % GEMV_RING) * GEMV_SLICE_BYTES;
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + g * 64 + t * 16), "l"(c0 + size_t(sl) * 64) : "memory");
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + (g + 8) * 64 + t * 16), "l"(c1 + size_t(sl) * 64) : "memory");
      if (lane < 16)
        asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst + 1024 + lane * 8), "l"(sc + size_t(sl) * 8) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  const uint4* xr = x + size_t(g) * (k / 8) + t * 4;
  const bool x_live = g < rows;
  auto load_x = [&](uint32_t j, uint4* xv) {
    const bool live = x_live && j < mine;
    const uint4* src = xr + size_t(first + j * GEMV_WARPS) * 16;
#pragma unroll
    for (int i = 0; i < 4; ++i) xv[i] = live ? __ldg(src + i) : make_uint4(0u, 0u, 0u, 0u);
  };
#pragma unroll
  for (int j = 0; j < GEMV_RING; ++j) issue(uint32_t(j));
  float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  uint4 xv[4], xn[4];
  load_x(0, xv);
  for (uint32_t j = 0; j < mine; ++j) {
    load_x(j + 1, xn);
    asm volatile("cp.async.wait_group %0;" ::"n"(GEMV_RING - 1) : "memory");
    __syncwarp();
    const uint8_t* slot = ring + (j % GEMV_RING) * GEMV_SLICE_BYTES;
    const uint4 wa = *reinterpret_cast<const uint4*>(slot + g * 64 + t * 16);
    const uint4 wb = *reinterpret_cast<const uint4*>(slot + (g + 8) * 64 + t * 16);
    const uint32_t sa = *reinterpret_cast<const uint16_t*>(slot + 1024 + g * 8 + t * 2);
    const uint32_t sb = *reinterpret_cast<const uint16_t*>(slot + 1024 + (g + 8) * 8 + t * 2);
    __syncwarp();                                        // every lane has taken its bytes: the slot may be refilled
    issue(j + GEMV_RING);
    uint32_t sah, sbh;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(sah) : "h"(uint16_t(sa)));
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(sbh) : "h"(uint16_t(sb)));
    const __half2 sa2 = *reinterpret_cast<__half2*>(&sah), sb2 = *reinterpret_cast<__half2*>(&sbh);
    const __half2 sa_lo = __low2half2(sa2), sa_hi = __high2half2(sa2);
    const __half2 sb_lo = __low2half2(sb2), sb_hi = __high2half2(sb2);
    __nv_bfloat162 qa_lo, qa_hi, qb_lo, qb_hi;
    if (!F16) { qa_lo = scale_bf16x2(sa_lo); qa_hi = scale_bf16x2(sa_hi); qb_lo = scale_bf16x2(sb_lo); qb_hi = scale_bf16x2(sb_hi); }
    const uint32_t wwa[4] = {wa.x, wa.y, wa.z, wa.w}, wwb[4] = {wb.x, wb.y, wb.z, wb.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) {                        // instruction i takes values 4 i .. 4 i + 3 of the lane's 32
      const uint32_t ba = (wwa[i >> 1] >> ((i & 1) * 16)) & 0xFFFFu, bb = (wwb[i >> 1] >> ((i & 1) * 16)) & 0xFFFFu;
      uint32_t a0, a1, a2, a3;
      const uint4& xq = xv[i >> 1];
      const uint32_t b0 = (i & 1) ? xq.z : xq.x, b1 = (i & 1) ? xq.w : xq.y;
      if (F16) {
        decode4_f16(ba, i < 4 ? sa_lo : sa_hi, a0, a2);
        decode4_f16(bb, i < 4 ? sb_lo : sb_hi, a1, a3);
        mma_f16_acc(acc, a0, a1, a2, a3, b0, b1);
      } else {
        decode4(ba, i < 4 ? qa_lo : qa_hi, a0, a2);
        decode4(bb, i < 4 ? qb_lo : qb_hi, a1, a3);
        mma_bf16(acc, a0, a1, a2, a3, b0, b1);
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) xv[i] = xn[i];
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");   // nothing of this warp's is in flight when the block ends
  gemv_finish(acc, out, rows, n, scale2, part, sp);
}

template <typename O>
__global__ void __launch_bounds__(32 * GEMV_WARPS, 4)
gemv_w4a16_kernel(const uint4* __restrict__ x, const uint4* __restrict__ codes, const uint8_t* __restrict__ scales,
                  O* __restrict__ out, uint32_t rows, uint32_t n, uint32_t k, float scale2, uint32_t ksplit) {
  __shared__ float part[GEMV_WARPS][16][8];
  extern __shared__ __align__(16) uint8_t gemv_ring[];      // GEMV_RING_SMEM bytes when k % 128 == 0, else none
  mb_grid_dependency_sync();                 // the rows may come from the kernel before this one
  const GemvSplit sp{ksplit, nullptr, nullptr, 1};
  if (k % 128 == 0) gemv_body_ring<false, O>(x, codes, scales, out, rows, n, k, scale2, part, sp, gemv_ring);
  else gemv_body<false, O>(x, codes, scales, out, rows, n, k, scale2, part, sp);
}

// The same with the f16 copy of the activations when every row converted exactly (flags all zero), else with the
// caller's bf16 rows; the choice is uniform over the grid.
template <typename O>
__global__ void __launch_bounds__(32 * GEMV_WARPS, 3)
gemv_w4a16_dual_kernel(const uint4* __restrict__ x, const uint4* __restrict__ x_f16, const int* __restrict__ inexact,
                       const uint4* __restrict__ codes, const uint8_t* __restrict__ scales, O* __restrict__ out,
                       uint32_t rows, uint32_t n, uint32_t k, float scale2, const GemvSplit sp) {
  __shared__ float part[GEMV_WARPS][16][8];
  mb_grid_dependency_sync();                 // the conversion pass before this kernel wrote x_f16 and the flags
  extern __shared__ __align__(16) uint8_t gemv_ring[];      // GEMV_RING_SMEM bytes when k % 128 == 0, else none
  int any = 0;
  for (uint32_t r = 0; r < rows; ++r) any |= __ldg(inexact + r);
  if (k % 128 == 0) {
    if (any) gemv_body_ring<false, O>(x, codes, scales, out, rows, n, k, scale2, part, sp, gemv_ring);
    else gemv_body_ring<true, O>(x_f16, codes, scales, out, rows, n, k, scale2, part, sp, gemv_ring);
  } else {
    if (any) gemv_body<false, O>(x, codes, scales, out, rows, n, k, scale2, part, sp);
    else gemv_body<true, O>(x_f16, codes, scales, out, rows, n, k, scale2, part, sp);
  }
}

// One block per activation row: bf16 -> f16, exact when the value is zero, infinite, NaN or a normal f16 (bf16 has
// 8 significant bits, f16 has 11); a finite value outside f16's normal range raises the row's flag.
__global__ void __launch_bounds__(256)
gemv_x_to_f16_kernel(const uint4* __restrict__ x, uint4* __restrict__ x_f16, int* __restrict__ inexact, uint32_t k8,
                     int* __restrict__ counters, uint32_t n_counters) {
  __shared__ int s_bad;
  if (threadIdx.x == 0) s_bad = 0;
  __syncthreads();
  mb_grid_dependency_sync();                 // the rows come from the kernel before this one
  const uint32_t row = blockIdx.x;
  // the K-split counters of the product that follows (a workspace arrives with any content)
  if (row == 0)
    for (uint32_t i = threadIdx.x; i < n_counters; i += 256) counters[i] = 0;
  int bad = 0;
  for (uint32_t i = threadIdx.x; i < k8; i += 256) {
    const uint4 v = __ldg(x + size_t(row) * k8 + i);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t h[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float lo = __uint_as_float(w[j] << 16), hi = __uint_as_float(w[j] & 0xFFFF0000u);
      const float alo = fabsf(lo), ahi = fabsf(hi);
      bad |= (alo != 0.0f && alo < 6.103515625e-05f) || (alo > 65504.0f && alo < __int_as_float(0x7F800000));
      bad |= (ahi != 0.0f && ahi < 6.103515625e-05f) || (ahi > 65504.0f && ahi < __int_as_float(0x7F800000));
      __half2 p = __floats2half2_rn(lo, hi);
      h[j] = *reinterpret_cast<uint32_t*>(&p);
    }
    x_f16[size_t(row) * k8 + i] = make_uint4(h[0], h[1], h[2], h[3]);
  }
  if (bad) s_bad = 1;
  __syncthreads();
  if (threadIdx.x == 0) inexact[row] = s_bad;
}

// ---------------------------------------------------------------------------------
// Decode-time grouped experts: one activation row per group against expert ids[g] of a bank.
//
// Two launches, as the reference's lane (src/nn/nvfp4_gemm.rs:293-523). The quantizer is the
// divide recipe with the expert's own second-level scale input_scale[ids[g]]. The product is the
// GEMV above with both operands four bits: a decoded code times its block scale is exact in f16
// (at most 7 significant bits, magnitudes in [2^-10, 2688]) for the weights AND for the quantized
// activation, so the row is expanded to f16 once in shared memory, the weights of sixteen rows per
// block stream through registers, and the products (exact in f32) are summed by the warp-level
// tensor cores in f32. Per group that is project_w4a4_scaled on one row up to the order of the
// f32 sums. HBM-bound: each chosen expert's planes (0.5625 B per weight) are read once.
// ---------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
quantize_grouped_kernel(const __nv_bfloat16* __restrict__ x, const int32_t* __restrict__ ids,
                        const float* __restrict__ input_scale, uint32_t group_blocks, uint32_t total_blocks,
                        uint32_t x_group_blocks, uint32_t experts, uint2* __restrict__ codes,
                        uint8_t* __restrict__ scales, int* __restrict__ flag) {
  const uint32_t blk = blockIdx.x * 256 + threadIdx.x;
  if (blk >= total_blocks) return;
  const uint32_t g = blk / group_blocks, within = blk - g * group_blocks;
  int32_t e = __ldg(ids + g);
  if (e < 0 || uint32_t(e) >= experts) {      // a bad expert id: flagged, quantized with a unit scale
    atomicCAS(flag, 0, int(g) + 1);
    e = -1;
  }
  const float s2 = e < 0 ? 1.0f : __ldg(input_scale + e);
  const uint4* p = reinterpret_cast<const uint4*>(x + (size_t(g) * x_group_blocks + within) * 16);
  const uint4 a = __ldg(p), b = __ldg(p + 1);
  const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
  float v[16];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
  uint32_t sbyte;
  uint2 c;
  quant_block_scaled(v, s2, sbyte, c);
  codes[blk] = c;
  scales[blk] = uint8_t(sbyte);
}

// Four codes (two bytes) times their block scale -> two f16x2 registers (exact).
__device__ __forceinline__ void decode4h(uint32_t two_bytes, __half2 s, uint32_t& lo, uint32_t& hi) {
  uint32_t h0, h1;
  asm("{ .reg .b8 b0, b1, b2, b3; mov.b32 {b0, b1, b2, b3}, %2;\n\t"
      "cvt.rn.f16x2.e2m1x2 %0, b0;\n\tcvt.rn.f16x2.e2m1x2 %1, b1; }"
      : "=r"(h0), "=r"(h1) : "r"(two_bytes));
  const __half2 p0 = __hmul2(*reinterpret_cast<__half2*>(&h0), s), p1 = __hmul2(*reinterpret_cast<__half2*>(&h1), s);
  lo = *reinterpret_cast<const uint32_t*>(&p0);
  hi = *reinterpret_cast<const uint32_t*>(&p1);
}
__device__ __forceinline__ void mma_f16(float* d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                        uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
               "{%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// grid (n / 16, groups); dynamic shared memory: the group's activation row as k f16 values.
template <typename O>
__global__ void __launch_bounds__(32 * GEMV_WARPS)
gemv_w4a4_grouped_kernel(const uint2* __restrict__ a_codes, const uint8_t* __restrict__ a_scales,
                         const uint4* __restrict__ bank_codes, const uint8_t* __restrict__ bank_scales,
                         const int32_t* __restrict__ ids, const float* __restrict__ alpha, O* __restrict__ out,
                         uint32_t n, uint32_t k, uint32_t experts) {
  extern __shared__ __align__(16) uint8_t xs_raw[];
  uint4* xs = reinterpret_cast<uint4*>(xs_raw);                 // k / 8 units of eight f16 values
  __shared__ float part[GEMV_WARPS][16];
  const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t g = lane >> 2, t = lane & 3;
  const uint32_t grp = blockIdx.y;
  const int32_t e_raw = __ldg(ids + grp);
  const bool bad = e_raw < 0 || uint32_t(e_raw) >= experts;     // flagged by the quantizer; the row comes out as zeros
  const uint32_t e = bad ? 0u : uint32_t(e_raw);
  // the activation row: one 16-block per thread and step -> sixteen f16 values
  for (uint32_t kb = threadIdx.x; kb < k / 16; kb += 32 * GEMV_WARPS) {
    const uint2 c = __ldg(a_codes + size_t(grp) * (k / 16) + kb);
    uint32_t sh;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(sh) : "h"(uint16_t(__ldg(a_scales + size_t(grp) * (k / 16) + kb))));
    const __half2 s = __low2half2(*reinterpret_cast<__half2*>(&sh));
    uint32_t h[8];
    decode4h(c.x & 0xFFFFu, s, h[0], h[1]);
    decode4h(c.x >> 16, s, h[2], h[3]);
    decode4h(c.y & 0xFFFFu, s, h[4], h[5]);
    decode4h(c.y >> 16, s, h[6], h[7]);
    xs[kb * 2] = make_uint4(h[0], h[1], h[2], h[3]);
    xs[kb * 2 + 1] = make_uint4(h[4], h[5], h[6], h[7]);
  }
  __syncthreads();
  const uint32_t row_base = blockIdx.x * 16;
  const uint32_t r0 = min(row_base + g, n - 1), r1 = min(row_base + g + 8, n - 1);
  const uint32_t slices = (k + 127) / 128;
  const uint4* c0 = bank_codes + (size_t(e) * n + r0) * (k / 32);
  const uint4* c1 = bank_codes + (size_t(e) * n + r1) * (k / 32);
  const uint16_t* s0p = reinterpret_cast<const uint16_t*>(bank_scales + (size_t(e) * n + r0) * (k / 16));
  const uint16_t* s1p = reinterpret_cast<const uint16_t*>(bank_scales + (size_t(e) * n + r1) * (k / 16));
  float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  constexpr int U = 4;
  for (uint32_t sl0 = warp; sl0 < slices; sl0 += GEMV_WARPS * U) {
    uint4 wa[U], wb[U];
    uint32_t sa[U], sb[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint32_t k0 = (sl0 + u * GEMV_WARPS) * 128 + t * 32;
      const bool live = k0 < k;
      wa[u] = live ? __ldg(c0 + k0 / 32) : make_uint4(0u, 0u, 0u, 0u);
      wb[u] = live ? __ldg(c1 + k0 / 32) : make_uint4(0u, 0u, 0u, 0u);
      sa[u] = live ? uint32_t(__ldg(s0p + k0 / 32)) : 0u;
      sb[u] = live ? uint32_t(__ldg(s1p + k0 / 32)) : 0u;
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint32_t k0 = (sl0 + u * GEMV_WARPS) * 128 + t * 32;
      if (sl0 + u * GEMV_WARPS >= slices) break;           // warp-uniform
      // the one activation row is column 0 of the instruction's N side: lanes with g == 0 supply it
      const bool live = g == 0 && k0 < k;
      uint4 xv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) xv[i] = live ? xs[k0 / 8 + i] : make_uint4(0u, 0u, 0u, 0u);
      uint32_t sah, sbh;
      asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(sah) : "h"(uint16_t(sa[u])));
      asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(sbh) : "h"(uint16_t(sb[u])));
      const __half2 sa2 = *reinterpret_cast<__half2*>(&sah), sb2 = *reinterpret_cast<__half2*>(&sbh);
      const __half2 sa_lo = __low2half2(sa2), sa_hi = __high2half2(sa2);
      const __half2 sb_lo = __low2half2(sb2), sb_hi = __high2half2(sb2);
      const uint32_t wwa[4] = {wa[u].x, wa[u].y, wa[u].z, wa[u].w}, wwb[4] = {wb[u].x, wb[u].y, wb[u].z, wb[u].w};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const uint32_t ba = (wwa[i >> 1] >> ((i & 1) * 16)) & 0xFFFFu, bb = (wwb[i >> 1] >> ((i & 1) * 16)) & 0xFFFFu;
        uint32_t a0, a1, a2, a3;
        decode4h(ba, i < 4 ? sa_lo : sa_hi, a0, a2);
        decode4h(bb, i < 4 ? sb_lo : sb_hi, a1, a3);
        const uint4& xq = xv[i >> 1];
        const uint32_t b0 = (i & 1) ? xq.z : xq.x, b1 = (i & 1) ? xq.w : xq.y;
        mma_f16(acc, a0, a1, a2, a3, b0, b1);
      }
    }
  }
  // column 0 of the accumulator tile: lanes with t == 0 hold weight rows g (acc[0]) and g + 8 (acc[2])
  if (t == 0) {
    part[warp][g] = acc[0];
    part[warp][g + 8] = acc[2];
  }
  __syncthreads();
  if (threadIdx.x < 16 && row_base + threadIdx.x < n) {
    float sum = 0.0f;
#pragma unroll
    for (int w = 0; w < GEMV_WARPS; ++w) sum += part[w][threadIdx.x];
    out[size_t(grp) * n + row_base + threadIdx.x] = O(bad ? 0.0f : sum * __ldg(alpha + e));
  }
}

// The ring of the k % 128 == 0 bodies needs more than the default 48 KB of dynamic shared memory.
int gemv_set_attributes(mb_ctx* ctx) {
  if (!mb_once(ctx, MB_ONCE_GEMV_RING)) {
    MB_CUDA_OK(ctx, cudaFuncSetAttribute(gemv_w4a16_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMV_RING_SMEM));
    MB_CUDA_OK(ctx, cudaFuncSetAttribute(gemv_w4a16_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMV_RING_SMEM));
    MB_CUDA_OK(ctx, cudaFuncSetAttribute(gemv_w4a16_dual_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMV_RING_SMEM));
    MB_CUDA_OK(ctx, cudaFuncSetAttribute(gemv_w4a16_dual_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMV_RING_SMEM));
    mb_once_done(ctx, MB_ONCE_GEMV_RING);
  }
  return MB_OK;
}

// Ranges of K slices per row block: doubled while the grid would leave fewer than four blocks per SM and every
// warp of a range still has a slice of its own.
uint32_t gemv_ksplit(size_t n, size_t k) {
  const size_t blocks = (n + 15) / 16, slices = (k + 127) / 128;
  uint32_t s = 1;
  while (blocks * s < 592 && s < 8 && slices / (2 * s) >= size_t(GEMV_WARPS)) s *= 2;
  return s;
}

// K ranges of the one-kernel form: doubled while the whole grid still fits the device at once (four blocks per
// SM; a grid a little over one wave costs two) and every warp of a range keeps a slice of its own.
uint32_t gemv_ksplit_one_wave(int sm_count, size_t n, size_t k) {
  const size_t blocks = (n + 15) / 16, slices = (k + 127) / 128, slots = size_t(sm_count) * 4;
  uint32_t s = 1;
  while (blocks * 2 * s <= slots && s < 8 && slices / (2 * s) >= size_t(GEMV_WARPS)) s *= 2;
  return s;
}

// One kernel: the caller's bf16 rows as they are, the K ranges of a row block as one cluster (1, ksplit, 1).
template <typename O>
cudaError_t launch_rows(int sm_count, cudaStream_t stream, size_t rows, const void* x, const uint8_t* codes,
                        const uint8_t* scales, O* out, uint32_t n, uint32_t k, float scale2) {
  const uint32_t ksplit = gemv_ksplit_one_wave(sm_count, n, k);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((n + 15) / 16, ksplit);
  cfg.blockDim = dim3(32 * GEMV_WARPS);
  cfg.dynamicSmemBytes = k % 128 == 0 ? GEMV_RING_SMEM : 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  unsigned na = 0;
  if (ksplit > 1) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = 1; attr[na].val.clusterDim.y = ksplit; attr[na].val.clusterDim.z = 1;
    ++na;
  }
  if (mb_pdl_enabled()) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  return cudaLaunchKernelEx(&cfg, gemv_w4a16_kernel<O>, static_cast<const uint4*>(x), reinterpret_cast<const uint4*>(codes),
                            scales, out, uint32_t(rows), n, k, scale2, ksplit);
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
  MB_REQUIRE(ctx, mb_aligned(codes, 16) && mb_aligned(scales, k % 128 == 0 ? 8 : 2),
             "NVFP4 GEMV needs 16-byte aligned code rows (and 8-byte aligned scale rows when k is a multiple of 128)");
  int rc = gemv_set_attributes(ctx);
  if (rc) return rc;
  if (out_dtype == MB_DT_BF16)
    MB_CUDA_OK(ctx, launch_rows(ctx->sm_count, stream, rows, x_bf16, codes, scales, static_cast<__nv_bfloat16*>(out), uint32_t(n), uint32_t(k), scale2));
  else if (out_dtype == MB_DT_F32)
    MB_CUDA_OK(ctx, launch_rows(ctx->sm_count, stream, rows, x_bf16, codes, scales, static_cast<float*>(out), uint32_t(n), uint32_t(k), scale2));
  else
    return mb_fail(ctx, MB_ERR_INVALID, "gemv: output is bf16 or f32");
  MB_LAUNCH_OK(ctx);
  return MB_OK;
}

namespace {

struct GemvWorkspace {
  size_t counters_off, partials_off, x16_off, bytes;
  uint32_t ksplit, row_blocks;
};

GemvWorkspace gemv_workspace_plan(size_t rows, size_t n, size_t k) {
  GemvWorkspace w;
  w.ksplit = gemv_ksplit(n, k);
  w.row_blocks = uint32_t((n + 15) / 16);
  w.counters_off = 256;                                                     // the rows' flags come first
  w.partials_off = w.counters_off + ((size_t(w.row_blocks) * 4 + 255) & ~size_t(255));
  const size_t partials = w.ksplit > 1 ? size_t(w.ksplit) * w.row_blocks * 128 * sizeof(float) : 0;
  w.x16_off = w.partials_off + ((partials + 255) & ~size_t(255));
  w.bytes = w.x16_off + rows * k * 2;
  return w;
}

}  // namespace

MB_API size_t mb_nvfp4_gemv_workspace(size_t rows, size_t n, size_t k) {
  if (rows == 0 || rows > MAX_ROWS || n == 0 || k == 0 || k % 32 != 0) return 0;
  return gemv_workspace_plan(rows, n, k).bytes;
}

MB_API int mb_nvfp4_gemv_w4a16_ws(mb_ctx* ctx, mb_stream stream_, const void* x_bf16, size_t rows, const uint8_t* codes,
                                  const uint8_t* scales, float scale2, size_t n, size_t k, void* out, int out_dtype,
                                  void* workspace, size_t workspace_bytes) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const size_t need = mb_nvfp4_gemv_workspace(rows, n, k);
  // The one-kernel form (bf16 rows as they are, K ranges meeting inside a cluster) needs no workspace. The form with
  // an f16 copy of the rows, two kernels and K ranges meeting in the workspace serves tall weights (below);
  // MB_GEMV_TWO_PASS=1 / 0 in the environment forces one or the other.
  // Weights of more 16-row blocks than the device holds at once (four per SM) are bound by instruction issue, and
  // there the f16 form's shorter decode is worth its second launch.
  const char* env = getenv("MB_GEMV_TWO_PASS");      // read per call: the tests run both forms in one process
  const int forced = !env ? -1 : (env[0] == '1' ? 1 : 0);
  const bool two_pass = forced >= 0 ? forced == 1 : (ctx && (n + 15) / 16 > size_t(ctx->sm_count) * 4);
  if (!two_pass || !workspace || need == 0 || workspace_bytes < need)
    return mb_nvfp4_gemv_w4a16(ctx, stream_, x_bf16, rows, codes, scales, scale2, n, k, out, out_dtype);
  MB_REQUIRE(ctx, ctx && x_bf16 && codes && scales && out, "gemv: null argument");
  MB_REQUIRE(ctx, n * k <= 0xFFFFFFFFull, "NVFP4 weight exceeds u32 indexing");
  MB_REQUIRE(ctx, scale2 == scale2 && scale2 > 0.0f && scale2 <= 3.4e38f,
             "NVFP4 global scale %g is not a positive finite number", double(scale2));
  MB_REQUIRE(ctx, mb_aligned(x_bf16, 16) && mb_aligned(workspace, 256), "NVFP4 GEMV needs a 16-byte aligned activation and a 256-byte aligned workspace");
  MB_REQUIRE(ctx, mb_aligned(codes, 16) && mb_aligned(scales, k % 128 == 0 ? 8 : 2),
             "NVFP4 GEMV needs 16-byte aligned code rows (and 8-byte aligned scale rows when k is a multiple of 128)");
  MB_REQUIRE(ctx, out_dtype == MB_DT_BF16 || out_dtype == MB_DT_F32, "gemv: output is bf16 or f32");
  {
    int rc = gemv_set_attributes(ctx);
    if (rc) return rc;
  }
  const size_t ring_smem = k % 128 == 0 ? size_t(GEMV_RING_SMEM) : 0;
  const GemvWorkspace w = gemv_workspace_plan(rows, n, k);
  uint8_t* base = static_cast<uint8_t*>(workspace);
  int* flags = reinterpret_cast<int*>(base);
  int* counters = reinterpret_cast<int*>(base + w.counters_off);
  uint4* x16 = reinterpret_cast<uint4*>(base + w.x16_off);
  const GemvSplit sp{w.ksplit, reinterpret_cast<float*>(base + w.partials_off), counters, 0};
  MB_CUDA_OK(ctx, mb_launch_pdl(gemv_x_to_f16_kernel, dim3(unsigned(rows)), dim3(256), 0, stream,
                                static_cast<const uint4*>(x_bf16), x16, flags, uint32_t(k / 8), counters, w.row_blocks));
  const dim3 grid(w.row_blocks, w.ksplit), block(32 * GEMV_WARPS);
  if (out_dtype == MB_DT_BF16)
    MB_CUDA_OK(ctx, mb_launch_pdl(gemv_w4a16_dual_kernel<__nv_bfloat16>, grid, block, ring_smem, stream,
                                  static_cast<const uint4*>(x_bf16), static_cast<const uint4*>(x16), static_cast<const int*>(flags),
                                  reinterpret_cast<const uint4*>(codes), scales, static_cast<__nv_bfloat16*>(out),
                                  uint32_t(rows), uint32_t(n), uint32_t(k), scale2, sp));
  else
    MB_CUDA_OK(ctx, mb_launch_pdl(gemv_w4a16_dual_kernel<float>, grid, block, ring_smem, stream, static_cast<const uint4*>(x_bf16),
                                  static_cast<const uint4*>(x16), static_cast<const int*>(flags),
                                  reinterpret_cast<const uint4*>(codes), scales, static_cast<float*>(out), uint32_t(rows),
                                  uint32_t(n), uint32_t(k), scale2, sp));
  MB_LAUNCH_OK(ctx);
  return MB_OK;
}

MB_API int mb_nvfp4_quantize_grouped(mb_ctx* ctx, mb_stream stream_, const void* x_bf16, int x_per_group,
                                     const int32_t* ids, size_t groups, const float* input_scale, size_t experts,
                                     size_t k, uint8_t* codes, uint8_t* scales_rowmajor) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  MB_REQUIRE(ctx, ctx && x_bf16 && ids && input_scale && codes && scales_rowmajor, "quantize_grouped: null argument");
  MB_REQUIRE(ctx, k > 0 && k % 64 == 0 && groups > 0 && groups <= 65535 && experts > 0,
             "grouped W4A4 geometry [%zu groups, k %zu]", groups, k);
  MB_REQUIRE(ctx, groups * (k / 16) <= 0xFFFFFF00ull, "quantize_grouped: exceeds u32 block indexing");
  MB_REQUIRE(ctx, mb_aligned(x_bf16, 16) && mb_aligned(codes, 8), "quantize_grouped: 16/8-byte alignment");
  const uint32_t group_blocks = uint32_t(k / 16), total = uint32_t(groups * (k / 16));
  quantize_grouped_kernel<<<(total + 255) / 256, 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(x_bf16), ids, input_scale, group_blocks, total, x_per_group ? group_blocks : 0u,
      uint32_t(experts), reinterpret_cast<uint2*>(codes), scales_rowmajor, ctx->flags_dev + MB_FLAG_PLAN_FAULT);
  MB_LAUNCH_OK(ctx);
  return MB_OK;
}

MB_API int mb_nvfp4_gemv_w4a4_grouped(mb_ctx* ctx, mb_stream stream_, const uint8_t* a_codes,
                                      const uint8_t* a_scales_rowmajor, const uint8_t* bank_codes,
                                      const uint8_t* bank_scales_rowmajor, const float* alpha, const int32_t* ids,
                                      size_t groups, size_t experts, size_t n, size_t k, void* out, int out_dtype) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  MB_REQUIRE(ctx, ctx && a_codes && a_scales_rowmajor && bank_codes && bank_scales_rowmajor && alpha && ids && out,
             "gemv_w4a4_grouped: null argument");
  MB_REQUIRE(ctx, k > 0 && k % 64 == 0 && n > 0 && n % 8 == 0 && groups > 0 && groups <= 65535 && experts > 0,
             "grouped W4A4 geometry [%zu x %zu, %zu]", groups, n, k);
  MB_REQUIRE(ctx, n * k <= 0xFFFFFFFFull && k <= 24576, "gemv_w4a4_grouped: [%zu, %zu] exceeds u32 indexing or k > 24576", n, k);
  MB_REQUIRE(ctx, mb_aligned(a_codes, 8) && mb_aligned(bank_codes, 16) && mb_aligned(bank_scales_rowmajor, 2),
             "gemv_w4a4_grouped: planes need 8/16/2-byte alignment");
  MB_REQUIRE(ctx, out_dtype == MB_DT_BF16 || out_dtype == MB_DT_F32, "gemv_w4a4_grouped: output is bf16 or f32");
  const dim3 grid(unsigned((n + 15) / 16), unsigned(groups)), block(32 * GEMV_WARPS);
  const size_t smem = k * 2;
  if (out_dtype == MB_DT_BF16)
    gemv_w4a4_grouped_kernel<__nv_bfloat16><<<grid, block, smem, stream>>>(
        reinterpret_cast<const uint2*>(a_codes), a_scales_rowmajor, reinterpret_cast<const uint4*>(bank_codes),
        bank_scales_rowmajor, ids, alpha, static_cast<__nv_bfloat16*>(out), uint32_t(n), uint32_t(k), uint32_t(experts));
  else
    gemv_w4a4_grouped_kernel<float><<<grid, block, smem, stream>>>(
        reinterpret_cast<const uint2*>(a_codes), a_scales_rowmajor, reinterpret_cast<const uint4*>(bank_codes),
        bank_scales_rowmajor, ids, alpha, static_cast<float*>(out), uint32_t(n), uint32_t(k), uint32_t(experts));
  MB_LAUNCH_OK(ctx);
  return MB_OK;
}
