// GQA flash attention, bf16 in / bf16 out, head_dim 128: softmax(scale * Q K^T + causal) V.
//
// Two kernels share one tile format. K and V tiles of 64 keys x 128 dims arrive by
// TMA (4-D tensor maps over [batch, keys, kv_heads, D]) as two 64-dim halves, each a
// 128-byte-row tile under the 128-byte swizzle, so that ldmatrix reads them without
// bank conflicts; a dedicated producer warp keeps a ring of tiles in flight.
//
//  * decode  (nq * group <= 16): one CTA per (key split, kv head, sequence). All
//    query heads of the kv head ride in one 16-row MMA tile, so every K/V byte is
//    read once from HBM and shared by the whole group. The four compute warps take
//    16 keys of each 64-key tile; partial (o, m, l) of the warps and of the key
//    splits are merged at the end (flash-decoding). HBM-bound: algorithmic bytes =
//    2 * keys * kv_heads * D * 2 per sequence.
//  * prefill runs on tcgen05 (attention_tc5.cu). The warp-level prefill kernel below
//    (one CTA per 128-query tile, eight compute warps of 16 rows) is kept as the
//    comparison arm, selected with MB_ATTN_PREFILL=legacy in the environment.
//
// Decode (and the comparison prefill) use warp-level mma.sync m16n8k16 (bf16, f32
// accumulate): with 4 valid rows per 16-row tile the product is HBM-bound, not
// tensor-bound. Every mbarrier wait is bounded.
#include "common.cuh"
#include "tc5.cuh"
#include "attention.cuh"

#include <cuda_fp16.h>

namespace {

using namespace tc5;

constexpr int D = 128;            // head dim
constexpr int BC = 64;            // keys per tile
constexpr int TILE_HALF_BYTES = BC * 128;       // one 64-dim half of a K or V tile
constexpr int KV_STAGE_BYTES = 4 * TILE_HALF_BYTES;   // K lo, K hi, V lo, V hi = 32 KB

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_f16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
               "{%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack2h(float lo, float hi) {
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Byte offset of (row, 16-byte chunk c of 16 chunks = 128 dims) in a [rows x 128 dims]
// tile stored as two swizzled 64-dim halves of `half_bytes` each.
__device__ __forceinline__ uint32_t tile_off(uint32_t row, uint32_t c, uint32_t half_bytes) {
  return (c >> 3) * half_bytes + row * 128u + (((c & 7u) ^ (row & 7u)) << 4);
}

// Four E2M1 codes (two bytes, low nibble first) times their block scale -> two f16x2 registers.
// code x scale has at most 7 significant bits and lies in [2^-10, 2688]: exact in f16.
__device__ __forceinline__ void fp4_decode4(uint32_t two_bytes, __half2 s, uint32_t& lo, uint32_t& hi) {
  uint32_t h0, h1;
  asm("{ .reg .b8 b0, b1, b2, b3; mov.b32 {b0, b1, b2, b3}, %2;\n\t"
      "cvt.rn.f16x2.e2m1x2 %0, b0;\n\tcvt.rn.f16x2.e2m1x2 %1, b1; }"
      : "=r"(h0), "=r"(h1) : "r"(two_bytes));
  const __half2 p0 = __hmul2(*reinterpret_cast<__half2*>(&h0), s), p1 = __hmul2(*reinterpret_cast<__half2*>(&h1), s);
  lo = *reinterpret_cast<const uint32_t*>(&p0);
  hi = *reinterpret_cast<const uint32_t*>(&p1);
}

// A warp's slot of packed bytes: 16 key rows of K codes [16][64], V codes [16][64] at +1024,
// K scales [16][8] at +2048, V scales [16][8] at +2176.
//
// S[16 x 16] = Q K^T straight from the codes. Lane (g, t4) takes keys g and g + 8 and the 32
// values d = 32 t4 .. 32 t4 + 31 of each (one 16-byte load, two scale bytes); step ks multiplies
// d = 32 t4 + 4 ks + 0..3, the same permutation of d the Q fragments were loaded in.
__device__ __forceinline__ void fp4_qk(float (*s)[4], const uint32_t (*qf)[4], const uint8_t* raw, uint32_t lane) {
  const uint32_t g = lane >> 2, t4 = lane & 3u;
#pragma unroll
  for (int jn = 0; jn < 2; ++jn) {
    s[jn][0] = s[jn][1] = s[jn][2] = s[jn][3] = 0.0f;
    const uint32_t key = 8u * jn + g;
    const uint4 w = *reinterpret_cast<const uint4*>(raw + (key * 4u + t4) * 16u);
    uint32_t sh;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(sh) : "h"(*reinterpret_cast<const uint16_t*>(raw + 2048u + key * 8u + t4 * 2u)));
    const __half2 s2 = *reinterpret_cast<__half2*>(&sh);
    const __half2 s_lo = __low2half2(s2), s_hi = __high2half2(s2);
    const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      uint32_t b0, b1;
      fp4_decode4((ww[ks >> 1] >> (16 * (ks & 1))) & 0xFFFFu, ks < 4 ? s_lo : s_hi, b0, b1);
      mma_f16(s[jn], qf[ks], b0, b1);
    }
  }
}

// O[16 x 128] += P[16 x 16] V straight from the codes. Lane (g, t4) takes the 16-value block
// d = 16 g .. 16 g + 15 (eight code bytes, one scale byte) of keys 2 t4, 2 t4 + 1, 2 t4 + 8 and
// 2 t4 + 9; output tile n, column g is d = 16 g + n (the caller stores the columns accordingly).
__device__ __forceinline__ void fp4_pv(float (*o)[4], const float (*pfrag)[4], const uint8_t* raw, uint32_t lane) {
  const uint32_t g = lane >> 2, t4 = lane & 3u;
  uint32_t a[4];
  a[0] = pack2h(pfrag[0][0], pfrag[0][1]);
  a[1] = pack2h(pfrag[0][2], pfrag[0][3]);
  a[2] = pack2h(pfrag[1][0], pfrag[1][1]);
  a[3] = pack2h(pfrag[1][2], pfrag[1][3]);
  uint2 c[4];
  __half2 sc[4];
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const uint32_t key = 2u * t4 + (q & 1u) + 8u * (q >> 1);
    c[q] = *reinterpret_cast<const uint2*>(raw + 1024u + key * 64u + g * 8u);
    uint32_t sh;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(sh) : "h"(uint16_t(raw[2176u + key * 8u + g])));
    sc[q] = __low2half2(*reinterpret_cast<__half2*>(&sh));
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {                      // code bytes 2 j, 2 j + 1 of each key: values 4 j .. 4 j + 3
    uint32_t h[4][2];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const uint32_t word = (j < 2) ? c[q].x : c[q].y;
      fp4_decode4((word >> (16 * (j & 1))) & 0xFFFFu, sc[q], h[q][0], h[q][1]);
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {                    // output tile n = 4 j + e: value e of the four
      const uint32_t sel = (e & 1) ? 0x7632u : 0x5410u;
      const uint32_t b0 = __byte_perm(h[0][e >> 1], h[1][e >> 1], sel);
      const uint32_t b1 = __byte_perm(h[2][e >> 1], h[3][e >> 1], sel);
      mma_f16(o[4 * j + e], a, b0, b1);
    }
  }
}

// S[16 x 8*NT] = Q[16 x 128] K^T for keys key0.. of a tile; Q fragments come from qf (8 k-steps x 4 regs).
template <int NT, bool F16 = false>
__device__ __forceinline__ void qk_tile(float (*s)[4], const uint32_t (*qf)[4], uint32_t k_base, uint32_t key0,
                                        uint32_t lane) {
#pragma unroll
  for (int j = 0; j < NT; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f; }
  const uint32_t mi = lane >> 3, l8 = lane & 7;
#pragma unroll
  for (int ks = 0; ks < 8; ++ks) {
#pragma unroll
    for (int jp = 0; jp < NT / 2; ++jp) {
      uint32_t b0, b1, b2, b3;
      const uint32_t row = key0 + jp * 16 + (mi >> 1) * 8 + l8;
      ldsm_x4(k_base + tile_off(row, ks * 2 + (mi & 1), TILE_HALF_BYTES), b0, b1, b2, b3);
      if (F16) { mma_f16(s[2 * jp], qf[ks], b0, b1); mma_f16(s[2 * jp + 1], qf[ks], b2, b3); }
      else { mma_bf16(s[2 * jp], qf[ks], b0, b1); mma_bf16(s[2 * jp + 1], qf[ks], b2, b3); }
    }
  }
}

// O[16 x 128] += P[16 x 16*KT] V for keys key0.. of a tile; P in C-fragment layout (bf16-rounded here).
template <int KT, bool F16 = false>
__device__ __forceinline__ void pv_tile(float (*o)[4], const float (*pfrag)[4], uint32_t v_base, uint32_t key0,
                                        uint32_t lane) {
  const uint32_t mi = lane >> 3, l8 = lane & 7;
#pragma unroll
  for (int kt = 0; kt < KT; ++kt) {
    uint32_t a[4];
    if (F16) {
      a[0] = pack2h(pfrag[2 * kt][0], pfrag[2 * kt][1]);
      a[1] = pack2h(pfrag[2 * kt][2], pfrag[2 * kt][3]);
      a[2] = pack2h(pfrag[2 * kt + 1][0], pfrag[2 * kt + 1][1]);
      a[3] = pack2h(pfrag[2 * kt + 1][2], pfrag[2 * kt + 1][3]);
    } else {
      a[0] = pack2(pfrag[2 * kt][0], pfrag[2 * kt][1]);
      a[1] = pack2(pfrag[2 * kt][2], pfrag[2 * kt][3]);
      a[2] = pack2(pfrag[2 * kt + 1][0], pfrag[2 * kt + 1][1]);
      a[3] = pack2(pfrag[2 * kt + 1][2], pfrag[2 * kt + 1][3]);
    }
    const uint32_t row = key0 + kt * 16 + (mi & 1) * 8 + l8;
#pragma unroll
    for (int np = 0; np < 8; ++np) {
      uint32_t b0, b1, b2, b3;
      ldsm_x4_trans(v_base + tile_off(row, np * 2 + (mi >> 1), TILE_HALF_BYTES), b0, b1, b2, b3);
      if (F16) { mma_f16(o[2 * np], a, b0, b1); mma_f16(o[2 * np + 1], a, b2, b3); }
      else { mma_bf16(o[2 * np], a, b0, b1); mma_bf16(o[2 * np + 1], a, b2, b3); }
    }
  }
}

// One online-softmax step over NT key tiles of 8: masks, updates (m, l), rescales o, leaves p in s.
// Rows g (regs 0, 1) and g + 8 (regs 2, 3); mask_lo/hi = number of visible keys from `kbase` for those rows.
// HI = false when rows 8..15 of the tile are all padding (at most eight query rows): their half of the
// work is left out and their probabilities are zero.
template <int NT, bool HI = true>
__device__ __forceinline__ void softmax_step(float (*s)[4], float (*o)[4], float* m, float* l, float scale_log2,
                                             int vis_lo, int vis_hi, uint32_t lane, int first_lo = 0, int first_hi = 0) {
  const int t2 = (lane & 3) * 2;
  constexpr int E = HI ? 4 : 2, H = HI ? 2 : 1;
  float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int j = 0; j < NT; ++j) {
#pragma unroll
    for (int e = 0; e < E; ++e) {
      const int key = j * 8 + t2 + (e & 1);
      const int vis = e < 2 ? vis_lo : vis_hi, first = e < 2 ? first_lo : first_hi;   // first: keys below the window
      s[j][e] = (key < vis && key >= first) ? s[j][e] * scale_log2 : -INFINITY;
      mx[e >> 1] = fmaxf(mx[e >> 1], s[j][e]);
    }
  }
#pragma unroll
  for (int h = 0; h < H; ++h) {
    mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xFFFFFFFFu, mx[h], 1));
    mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xFFFFFFFFu, mx[h], 2));
  }
  float corr[2] = {1.0f, 1.0f}, sum[2] = {0.0f, 0.0f}, mnew[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int h = 0; h < H; ++h) {
    mnew[h] = fmaxf(m[h], mx[h]);
    // a fully masked row keeps m = -inf; exp2(-inf - (-inf)) is avoided by the guard
    corr[h] = mnew[h] == -INFINITY ? 1.0f : exp2f(m[h] - mnew[h]);
    m[h] = mnew[h];
  }
#pragma unroll
  for (int j = 0; j < NT; ++j) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      if (e >= E) { s[j][e] = 0.0f; continue; }
      const float mm = mnew[e >> 1];
      const float pv = mm == -INFINITY ? 0.0f : exp2f(s[j][e] - mm);
      s[j][e] = pv;
      sum[e >> 1] += pv;
    }
  }
#pragma unroll
  for (int h = 0; h < H; ++h) l[h] = l[h] * corr[h] + sum[h];   // per-thread partial; quad-reduced at the end
#pragma unroll
  for (int n = 0; n < 16; ++n) {
    o[n][0] *= corr[0]; o[n][1] *= corr[0];
    if (HI) { o[n][2] *= corr[1]; o[n][3] *= corr[1]; }
  }
}

// ---------------------------------------------------------------------------------
// Decode: grid (splits, kv_heads, batch), 4 compute warps + 1 producer warp.
// ---------------------------------------------------------------------------------
constexpr int DEC_STAGES = 3;
constexpr int DEC_THREADS = 160;
// NVFP4 rows: no producer warp and no shared ring. Each compute warp brings in the packed bytes of
// the 16 key rows it multiplies (K and V) through a cp.async ring of its own.
constexpr int DEC_THREADS_FP4 = 128;
constexpr int FP4_STAGES = 3;                     // tiles of packed bytes in flight per warp (cp.async groups)
constexpr int FP4_RAW_WARP = 2 * 16 * (D / 2) + 2 * 16 * (D / 16);   // 16 key rows: K, V codes + K, V scales = 2304 B
constexpr int DEC_TILE_FP4 = 36 * 1024;           // room for the merge patch (33.3 KB) at the end of the kernel
constexpr int DEC_RING_FP4 = DEC_TILE_FP4 + 4 * FP4_STAGES * FP4_RAW_WARP;
constexpr int DEC_SMEM_FP4 = DEC_RING_FP4 + 16 * D * 2 + 1024 + 128;
constexpr int DEC_SMEM = DEC_STAGES * KV_STAGE_BYTES + 16 * D * 2 /*Q*/ + 1024 + 128;
static_assert(4 * 16 * (D + 2) * 4 <= DEC_STAGES * KV_STAGE_BYTES, "the merge patch reuses the tile ring");

// EXT: the instantiation with the relative bias and the eviction gaps (positions instead of rows in the masks)
template <bool FP4, bool EXT = false>
__global__ void __launch_bounds__(FP4 ? DEC_THREADS_FP4 : DEC_THREADS, FP4 ? 3 : 2)
attn_decode_kernel(const __grid_constant__ AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
  constexpr uint32_t RING = FP4 ? DEC_RING_FP4 : DEC_STAGES * KV_STAGE_BYTES;
  const uint32_t q_smem = base + RING;            // [16][128] bf16, swizzled halves of 16 rows
  float* merge = reinterpret_cast<float*>(gen);   // reuses the tile ring once every compute warp is done with it
  const uint32_t bar_base = base + RING + 16 * D * 2;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (DEC_STAGES + s); };
  volatile int* abort_smem = reinterpret_cast<volatile int*>(gen + (bar_base - base) + 8 * 2 * DEC_STAGES);
  int* tflag = p.flags ? p.flags + MB_FLAG_WAIT_TIMEOUT : nullptr;

  const int warp = __shfl_sync(0xFFFFFFFFu, int(threadIdx.x >> 5), 0);
  const uint32_t lane = threadIdx.x & 31;
  const uint32_t split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const uint32_t group = p.heads / p.kv_heads;
  const uint32_t rows = p.nq * group;                      // <= 16
  // keys this query block can see at all, and this CTA's slice of them
  const uint32_t visible = p.causal ? min(p.keys, p.q0 + p.nq) : p.keys;
  const uint32_t k_begin = p.k_lo + split * p.keys_per_split;
  const uint32_t k_end = min(visible, k_begin + p.keys_per_split);
  const uint32_t n_tiles = k_end > k_begin ? (k_end - k_begin + BC - 1) / BC : 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < DEC_STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 4); }
    *abort_smem = 0;
    fence_barrier_init();
    if (!FP4) {
      tma_prefetch_desc(&p.tmap_k);
      tma_prefetch_desc(&p.tmap_v);
    }
  }
  mb_grid_dependency_sync();      // shared-memory set-up above; Q, K and V are read from here on
  // Q rows r = qi * group + hg, zero beyond `rows`; 16 chunks of 16 bytes per row.
  for (uint32_t i = threadIdx.x; i < 16 * 16; i += blockDim.x) {
    const uint32_t r = i >> 4, c = i & 15;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < rows) {
      const uint32_t qi = r / group, hg = r % group;
      const size_t qoff = ((size_t(b) * p.nq + qi) * p.heads + kvh * group + hg) * D + c * 8;
      if (p.q_f32) {
        const float4 f0 = *reinterpret_cast<const float4*>(p.q_f32 + qoff), f1 = *reinterpret_cast<const float4*>(p.q_f32 + qoff + 4);
        v = make_uint4(pack2(f0.x, f0.y), pack2(f0.z, f0.w), pack2(f1.x, f1.y), pack2(f1.z, f1.w));
      } else {
        v = *reinterpret_cast<const uint4*>(p.q + qoff);
      }
      if (FP4) {
        // the packed rows expand to f16, so the products run as f16 x f16: Q goes to f16 (exact for
        // magnitudes in [2^-14, 65504], which bf16's 8 significant bits fit; larger ones saturate)
        uint32_t* w = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float lo = fminf(fmaxf(__uint_as_float(w[i] << 16), -65504.0f), 65504.0f);
          const float hi = fminf(fmaxf(__uint_as_float(w[i] & 0xFFFF0000u), -65504.0f), 65504.0f);
          w[i] = pack2h(lo, hi);
        }
      }
    }
    *reinterpret_cast<uint4*>(gen + (q_smem - base) + tile_off(r, c, 16 * 128)) = v;
  }
  __syncthreads();

  if (!FP4 && warp == 4) {
    // producer
    int stage = 0;
    uint32_t phase = 0;
    for (uint32_t t = 0; t < n_tiles; ++t) {
      if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_smem, tflag, 11)) break;
      if (elect_one()) {
        const uint32_t s0 = base + stage * KV_STAGE_BYTES;
        const int key0 = int(k_begin + t * BC);
        mbar_arrive_expect_tx(full_bar(stage), KV_STAGE_BYTES);
        tma_load_4d(s0, &p.tmap_k, 0, int(kvh), key0, int(b), full_bar(stage));
        tma_load_4d(s0 + TILE_HALF_BYTES, &p.tmap_k, 64, int(kvh), key0, int(b), full_bar(stage));
        tma_load_4d(s0 + 2 * TILE_HALF_BYTES, &p.tmap_v, 0, int(kvh), key0, int(b), full_bar(stage));
        tma_load_4d(s0 + 3 * TILE_HALF_BYTES, &p.tmap_v, 64, int(kvh), key0, int(b), full_bar(stage));
      }
      __syncwarp();
      if (++stage == DEC_STAGES) { stage = 0; phase ^= 1u; }
    }
  } else {
    // compute warp w takes keys [16 w, 16 w + 16) of every tile
    uint32_t qf[8][4];
    if (FP4) {
      // the packed products sum over d in a permuted order: lane (g, t4) holds d = 32 t4 + 4 ks + 0..3 in
      // step ks, the 32 consecutive values one 16-byte load of codes gives it for a key
      const uint8_t* qs = gen + (q_smem - base);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const uint32_t d0 = 32u * (lane & 3u) + 4u * ks;
        const uint2 lo = *reinterpret_cast<const uint2*>(qs + tile_off(lane >> 2, d0 >> 3, 16 * 128) + (d0 & 7u) * 2u);
        const uint2 hi = *reinterpret_cast<const uint2*>(qs + tile_off((lane >> 2) + 8u, d0 >> 3, 16 * 128) + (d0 & 7u) * 2u);
        qf[ks][0] = lo.x; qf[ks][1] = hi.x; qf[ks][2] = lo.y; qf[ks][3] = hi.y;
      }
    } else {
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)
        ldsm_x4(q_smem + tile_off(lane & 15, ks * 2 + (lane >> 4), 16 * 128), qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
    }
    float o[16][4];
#pragma unroll
    for (int n = 0; n < 16; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};
    const uint32_t g = lane >> 2;
    // query position of rows g and g + 8 (rows >= `rows` are padding; they see what row 0 sees)
    const uint32_t qpos_lo = p.q0 + (g < rows ? g / group : 0);
    const uint32_t qpos_hi = p.q0 + (g + 8 < rows ? (g + 8) / group : 0);
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    // NVFP4 rows. The warp keeps FP4_STAGES tiles of its 16 key rows' packed bytes in flight as
    // cp.async groups into a ring of its own (nobody else reads it, so a __syncwarp is all the
    // hand-over needs); both products take their fragments straight from those bytes.
    uint8_t* raw_ring = gen + DEC_TILE_FP4 + uint32_t(warp) * FP4_STAGES * FP4_RAW_WARP;
    const size_t stride_c = size_t(p.kv_heads) * (D / 2), stride_s = size_t(p.kv_heads) * (D / 16);
    const uint8_t* kc0 = p.k_codes + (size_t(b) * p.cap * p.kv_heads + kvh) * (D / 2);
    const uint8_t* vc0 = p.v_codes + (size_t(b) * p.cap * p.kv_heads + kvh) * (D / 2);
    const uint8_t* ks0 = p.k_scales + (size_t(b) * p.cap * p.kv_heads + kvh) * (D / 16);
    const uint8_t* vs0 = p.v_scales + (size_t(b) * p.cap * p.kv_heads + kvh) * (D / 16);
    // lane's sources for tile 0, advanced by 64 rows per tile: two 16-byte chunks of K and of V codes
    // (chunk i = lane + 32 u of 64: key row i >> 2, part i & 3) and one row's eight scale bytes
    // (lanes 0-15 K, 16-31 V). Rows past the slice are masked: zero fill keeps P V finite, and their
    // (unread) source is the slice's first row.
    const uint32_t key_c = k_begin + uint32_t(warp) * 16u + (lane >> 2), key_s = k_begin + uint32_t(warp) * 16u + (lane & 15u);
    const uint8_t* kc_first = kc0 + size_t(k_begin) * stride_c;
    const uint8_t* sc_first = (lane < 16 ? ks0 : vs0) + size_t(k_begin) * stride_s;
    const ptrdiff_t v_minus_k = vc0 - kc0;
    const uint8_t* kc_p = kc0 + size_t(key_c) * stride_c + (lane & 3u) * 16u;
    const uint8_t* sc_p = (lane < 16 ? ks0 : vs0) + size_t(key_s) * stride_s;
    uint32_t issued = 0;                                 // tiles issued so far: issue() is called for t = 0, 1, 2, ...
    auto issue = [&](uint32_t t) {
      if (t < n_tiles) {
        const uint32_t dst = smem_u32(raw_ring + (t % FP4_STAGES) * FP4_RAW_WARP);
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const bool live = key_c + issued * BC + 8u * u < k_end;
          const uint8_t* src = live ? kc_p + size_t(8u * u) * stride_c : kc_first;
          const uint32_t n = live ? 16u : 0u, i = lane + 32u * u;
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst + i * 16u), "l"(src), "r"(n) : "memory");
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst + 1024u + i * 16u), "l"(src + v_minus_k), "r"(n) : "memory");
        }
        {
          const bool live = key_s + issued * BC < k_end;
          asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"(dst + 2048u + lane * 8u),
                       "l"(live ? sc_p : sc_first), "r"(live ? 8u : 0u) : "memory");
        }
        kc_p += size_t(BC) * stride_c;
        sc_p += size_t(BC) * stride_s;
        ++issued;
      }
      asm volatile("cp.async.commit_group;" ::: "memory");   // an empty group keeps the count uniform
    };
    if (FP4) {
#pragma unroll
      for (int s2 = 0; s2 < FP4_STAGES; ++s2) issue(uint32_t(s2));
    }
    for (uint32_t t = 0; t < n_tiles; ++t) {
      const uint8_t* raw = raw_ring + (t % FP4_STAGES) * FP4_RAW_WARP;
      if (FP4) {
        asm volatile("cp.async.wait_group %0;" ::"n"(FP4_STAGES - 1) : "memory");
        __syncwarp();                              // every lane's copies of tile t have landed
      } else if (!mbar_wait(full_bar(stage), phase, abort_smem, tflag, 12)) { ok = false; break; }
      const uint32_t s0 = base + stage * KV_STAGE_BYTES;
      const uint32_t key0 = warp * 16;
      const int kabs = int(k_begin + t * BC + key0);       // absolute index of this warp's first key
      float s[2][4];
      if (FP4) fp4_qk(s, qf, raw, lane);
      else {
        qk_tile<2>(s, qf, s0, key0, lane);
        if (t > 0) {
          __syncwarp();
          if (lane == 0) mbar_arrive(empty_bar(stage == 0 ? DEC_STAGES - 1 : stage - 1));   // the tile before this one
        }
      }
      int vis_lo = int(k_end) - kabs, vis_hi = vis_lo;
      if (p.causal) {
        vis_lo = min(vis_lo, int(qpos_lo) + 1 - kabs);
        vis_hi = min(vis_hi, int(qpos_hi) + 1 - kabs);
      }
      int first_lo = 0, first_hi = 0;
      if (p.window) {
        first_lo = int(qpos_lo) + 1 - int(p.window) - kabs;
        first_hi = int(qpos_hi) + 1 - int(p.window) - kabs;
      }
      if (EXT) {
        // positions instead of rows: each score is masked and biased on its own, then the step runs unmasked
#pragma unroll
        for (int j = 0; j < 2; ++j) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const uint32_t r = g + 8u * (e >> 1);
            const uint32_t qi = r < rows ? r / group : 0u, hg = r < rows ? r % group : 0u;
            const uint32_t krow = uint32_t(kabs) + j * 8 + (lane & 3) * 2 + (e & 1);
            uint32_t pos = p.pos0 + krow;
            for (uint32_t gi = 0; gi < p.ngaps; ++gi)
              if (__ldg(p.gap_rows + gi) <= p.row0 + krow) pos = p.pos0 + krow + __ldg(p.gap_cums + gi);
            const uint32_t qpos = p.q0_abs + qi;
            bool vis = krow < k_end && pos <= qpos;
            if (vis && p.window && qpos - pos >= p.window) vis = false;
            float val = s[j][e] * p.scale_log2;
            if (vis && p.rel && qpos - pos < p.eff)
              val += __ldg(p.rel + ((size_t(b) * p.nq + qi) * p.heads + kvh * group + hg) * p.eff + (qpos - pos)) *
                     1.4426950408889634f;
            s[j][e] = vis ? val : -INFINITY;
          }
        }
        softmax_step<2, true>(s, o, m, l, 1.0f, 16, 16, lane, 0, 0);
      } else if (rows <= 8) softmax_step<2, false>(s, o, m, l, p.scale_log2, vis_lo, vis_hi, lane, first_lo, first_hi);
      else softmax_step<2, true>(s, o, m, l, p.scale_log2, vis_lo, vis_hi, lane, first_lo, first_hi);
      if (FP4) {
        fp4_pv(o, s, raw, lane);
        __syncwarp();                              // the warp is done with the ring slot
        issue(t + FP4_STAGES);
      } else {
        pv_tile<1>(o, s, s0 + 2 * TILE_HALF_BYTES, key0, lane);
        // This tile's stage goes back to the producer only after the NEXT tile's scores (see the top of the loop):
        // handing it back right here let the refill overtake the last ldmatrix reads of V on rare occasions, when
        // the refill was a tile past the end of the keys (zero fill, no trip to memory) and the machine code had
        // the arrive ahead of those reads. A whole QK^T pass between the last read and the arrive leaves no window.
        if (++stage == DEC_STAGES) { stage = 0; phase ^= 1u; }
      }
    }
    (void)ok;
    // quad-reduce l, then publish this warp's partial (o, m, l) for rows g and g + 8
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      l[h] += __shfl_xor_sync(0xFFFFFFFFu, l[h], 1);
      l[h] += __shfl_xor_sync(0xFFFFFFFFu, l[h], 2);
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");   // all four compute warps have read their last tile
    float* mine = merge + warp * 16 * (D + 2);
    const uint32_t t2 = (lane & 3) * 2;
#pragma unroll
    for (int n = 0; n < 16; ++n) {
      // column c of output tile n is d = 8 n + c, or d = 16 c + n where the packed product permuted them
      const uint32_t d0 = FP4 ? 16u * t2 + n : n * 8 + t2, d1 = FP4 ? 16u * (t2 + 1) + n : n * 8 + t2 + 1;
      mine[g * (D + 2) + d0] = o[n][0];
      mine[g * (D + 2) + d1] = o[n][1];
      mine[(g + 8) * (D + 2) + d0] = o[n][2];
      mine[(g + 8) * (D + 2) + d1] = o[n][3];
    }
    if ((lane & 3) == 0) {
      mine[g * (D + 2) + D] = m[0];
      mine[g * (D + 2) + D + 1] = l[0];
      mine[(g + 8) * (D + 2) + D] = m[1];
      mine[(g + 8) * (D + 2) + D + 1] = l[1];
    }
  }
  __syncthreads();
  // merge the four warps: thread (r, d-group) handles row r, dims d..d+... ; 128 threads x 16 rows
  if (threadIdx.x < 128) {
    const uint32_t d = threadIdx.x;
    for (uint32_t r = 0; r < rows; ++r) {
      float mm = -INFINITY;
      for (int w = 0; w < 4; ++w) mm = fmaxf(mm, merge[(w * 16 + r) * (D + 2) + D]);
      float acc = 0.0f, ll = 0.0f;
      for (int w = 0; w < 4; ++w) {
        const float mw = merge[(w * 16 + r) * (D + 2) + D];
        const float f = mw == -INFINITY ? 0.0f : exp2f(mw - mm);
        acc += merge[(w * 16 + r) * (D + 2) + d] * f;
        ll += merge[(w * 16 + r) * (D + 2) + D + 1] * f;
      }
      const uint32_t qi = r / group, hg = r % group;
      if (p.slots == 1) {
        const float v = ll > 0.0f ? acc / ll : 0.0f;
        const size_t o = ((size_t(b) * p.nq + qi) * p.heads + kvh * group + hg) * D + d;
        if (p.out_f32) p.out_f32[o] = v; else p.out[o] = __float2bfloat16_rn(v);
      } else {
        float* dst = p.part + (((size_t(b) * p.kv_heads + kvh) * p.slots + p.slot0 + split) * 16 + r) * (D + 2);
        dst[d] = acc;
        if (d == 0) { dst[D] = mm; dst[D + 1] = ll; }
      }
    }
  }
}

// Merge the key splits: out = sum_s o_s 2^(m_s - M) / sum_s l_s 2^(m_s - M).
__global__ void __launch_bounds__(128)
attn_combine_kernel(const float* __restrict__ part, __nv_bfloat16* __restrict__ out, float* __restrict__ out_f32,
                    uint32_t nq, uint32_t heads, uint32_t kv_heads, uint32_t splits) {
  mb_grid_dependency_sync();
  const uint32_t h = blockIdx.x % heads, qi = (blockIdx.x / heads) % nq, b = blockIdx.x / (heads * nq);
  const uint32_t group = heads / kv_heads, kvh = h / group, r = qi * group + h % group, d = threadIdx.x;
  const float* src = part + ((size_t(b) * kv_heads + kvh) * splits * 16 + r) * (D + 2);
  const size_t split_stride = size_t(16) * (D + 2);
  float mm = -INFINITY;
  for (uint32_t s = 0; s < splits; ++s) mm = fmaxf(mm, src[s * split_stride + D]);
  float acc = 0.0f, ll = 0.0f;
  for (uint32_t s = 0; s < splits; ++s) {
    const float ms = src[s * split_stride + D];
    const float f = ms == -INFINITY ? 0.0f : exp2f(ms - mm);
    acc += src[s * split_stride + d] * f;
    ll += src[s * split_stride + D + 1] * f;
  }
  const float res = ll > 0.0f ? acc / ll : 0.0f;
  const size_t o = ((size_t(b) * nq + qi) * heads + h) * D + d;
  if (out_f32) out_f32[o] = res; else out[o] = __float2bfloat16_rn(res);
}

// ---------------------------------------------------------------------------------
// Prefill: grid (q tiles, heads, batch), 8 compute warps + 1 producer warp.
// ---------------------------------------------------------------------------------
constexpr int PRE_STAGES = 3;
constexpr int PRE_THREADS = 288;
constexpr int BR = 128;
constexpr int PRE_SMEM = PRE_STAGES * KV_STAGE_BYTES + BR * D * 2 + 1024 + 128;

// EXT: the instantiation with the relative bias and the eviction gaps for prompt-shaped blocks (positions instead of
// rows in the masks, as in the decode kernel's). It is the route of prompt shapes that carry either; the tcgen05
// kernel serves the rest.
template <bool EXT>
__global__ void __launch_bounds__(PRE_THREADS, 1)
attn_prefill_kernel(const __grid_constant__ AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t q_smem = base + PRE_STAGES * KV_STAGE_BYTES;      // two halves of [128][64]
  const uint32_t bar_base = q_smem + BR * D * 2;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (PRE_STAGES + s); };
  const uint32_t q_bar = bar_base + 8u * 2 * PRE_STAGES;
  volatile int* abort_smem = reinterpret_cast<volatile int*>(gen + (bar_base - base) + 8 * (2 * PRE_STAGES + 1));
  int* tflag = p.flags ? p.flags + MB_FLAG_WAIT_TIMEOUT : nullptr;

  const int warp = __shfl_sync(0xFFFFFFFFu, int(threadIdx.x >> 5), 0);
  const uint32_t lane = threadIdx.x & 31;
  // heavy (late) query tiles first
  const uint32_t qt = gridDim.x - 1 - blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const uint32_t kvh = h / (p.heads / p.kv_heads);
  const uint32_t q_row0 = qt * BR;
  const uint32_t q_rows = min(uint32_t(BR), p.nq - q_row0);
  const uint32_t last_q = p.q0 + q_row0 + q_rows - 1;
  const uint32_t k_end = p.causal ? min(p.keys, last_q + 1) : p.keys;
  const uint32_t n_tiles = (k_end + BC - 1) / BC;

  if (threadIdx.x == 0) {
    for (int s = 0; s < PRE_STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 8); }
    mbar_init(q_bar, 1);
    *abort_smem = 0;
    fence_barrier_init();
    tma_prefetch_desc(&p.tmap_q);
    tma_prefetch_desc(&p.tmap_k);
    tma_prefetch_desc(&p.tmap_v);
  }
  __syncthreads();

  if (warp == 8) {
    if (elect_one()) {
      mbar_arrive_expect_tx(q_bar, BR * D * 2);
      tma_load_4d(q_smem, &p.tmap_q, 0, int(h), int(q_row0), int(b), q_bar);
      tma_load_4d(q_smem + BR * 128, &p.tmap_q, 64, int(h), int(q_row0), int(b), q_bar);
    }
    __syncwarp();
    int stage = 0;
    uint32_t phase = 0;
    for (uint32_t t = 0; t < n_tiles; ++t) {
      if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_smem, tflag, 13)) break;
      if (elect_one()) {
        const uint32_t s0 = base + stage * KV_STAGE_BYTES;
        const int key0 = int(t * BC);
        mbar_arrive_expect_tx(full_bar(stage), KV_STAGE_BYTES);
        tma_load_4d(s0, &p.tmap_k, 0, int(kvh), key0, int(b), full_bar(stage));
        tma_load_4d(s0 + TILE_HALF_BYTES, &p.tmap_k, 64, int(kvh), key0, int(b), full_bar(stage));
        tma_load_4d(s0 + 2 * TILE_HALF_BYTES, &p.tmap_v, 0, int(kvh), key0, int(b), full_bar(stage));
        tma_load_4d(s0 + 3 * TILE_HALF_BYTES, &p.tmap_v, 64, int(kvh), key0, int(b), full_bar(stage));
      }
      __syncwarp();
      if (++stage == PRE_STAGES) { stage = 0; phase ^= 1u; }
    }
  } else {
    bool ok = mbar_wait(q_bar, 0u, abort_smem, tflag, 14);
    uint32_t qf[8][4];
    const uint32_t qr = warp * 16 + (lane & 15);
#pragma unroll
    for (int ks = 0; ks < 8; ++ks)
      ldsm_x4(q_smem + tile_off(qr, ks * 2 + (lane >> 4), BR * 128), qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
    float o[16][4];
#pragma unroll
    for (int n = 0; n < 16; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};
    const uint32_t g = lane >> 2;
    const int qpos_lo = int(p.q0 + q_row0 + warp * 16 + g), qpos_hi = qpos_lo + 8;
    int stage = 0;
    uint32_t phase = 0;
    for (uint32_t t = 0; ok && t < n_tiles; ++t) {
      if (!mbar_wait(full_bar(stage), phase, abort_smem, tflag, 15)) { ok = false; break; }
      const uint32_t s0 = base + stage * KV_STAGE_BYTES;
      const int kabs = int(t * BC);
      // a warp whose rows all lie before this tile (causal) has nothing to add
      const bool live = !p.causal || kabs <= qpos_lo + 8 + 7 - int(g);   // uniform: uses the warp's last row
      float s[8][4];
      if (live) qk_tile<8>(s, qf, s0, 0, lane);
      // the stage of the tile BEFORE this one goes back to the producer here, a scores pass after its last read
      // (the decode kernel says why)
      if (t > 0) {
        __syncwarp();
        if (lane == 0) mbar_arrive(empty_bar(stage == 0 ? PRE_STAGES - 1 : stage - 1));
      }
      if (live && EXT) {
        // every score is masked and biased on its own by position, then the step runs unmasked
        const uint32_t h_abs = h;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const uint32_t qi = q_row0 + warp * 16 + g + 8u * (e >> 1);          // query row of the block
            const uint32_t krow = uint32_t(kabs) + j * 8 + (lane & 3) * 2 + (e & 1);
            uint32_t pos = p.pos0 + krow;
            for (uint32_t gi = 0; gi < p.ngaps; ++gi)
              if (__ldg(p.gap_rows + gi) <= p.row0 + krow) pos = p.pos0 + krow + __ldg(p.gap_cums + gi);
            const uint32_t qpos = p.q0_abs + qi;
            bool vis = qi < p.nq && krow < p.keys && pos <= qpos;
            if (vis && p.window && qpos - pos >= p.window) vis = false;
            float val = s[j][e] * p.scale_log2;
            if (vis && p.rel && qpos - pos < p.eff)
              val += __ldg(p.rel + ((size_t(b) * p.nq + qi) * p.heads + h_abs) * p.eff + (qpos - pos)) * 1.4426950408889634f;
            s[j][e] = vis ? val : -INFINITY;
          }
        }
        softmax_step<8>(s, o, m, l, 1.0f, BC, BC, lane);
        pv_tile<4>(o, s, s0 + 2 * TILE_HALF_BYTES, 0, lane);
      } else if (live) {
        int vis_lo = int(p.keys) - kabs, vis_hi = vis_lo;
        if (p.causal) {
          vis_lo = min(vis_lo, qpos_lo + 1 - kabs);
          vis_hi = min(vis_hi, qpos_hi + 1 - kabs);
        }
        softmax_step<8>(s, o, m, l, p.scale_log2, vis_lo, vis_hi, lane);
        pv_tile<4>(o, s, s0 + 2 * TILE_HALF_BYTES, 0, lane);
      }
      if (++stage == PRE_STAGES) { stage = 0; phase ^= 1u; }
    }
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      l[hh] += __shfl_xor_sync(0xFFFFFFFFu, l[hh], 1);
      l[hh] += __shfl_xor_sync(0xFFFFFFFFu, l[hh], 2);
    }
    const float inv0 = l[0] > 0.0f ? 1.0f / l[0] : 0.0f, inv1 = l[1] > 0.0f ? 1.0f / l[1] : 0.0f;
    const uint32_t r_lo = warp * 16 + g, r_hi = r_lo + 8;
    const uint32_t t2 = (lane & 3) * 2;
#pragma unroll
    for (int n = 0; n < 16; ++n) {
      if (r_lo < q_rows)
        *reinterpret_cast<uint32_t*>(p.out + ((size_t(b) * p.nq + q_row0 + r_lo) * p.heads + h) * D + n * 8 + t2) =
            pack2(o[n][0] * inv0, o[n][1] * inv0);
      if (r_hi < q_rows)
        *reinterpret_cast<uint32_t*>(p.out + ((size_t(b) * p.nq + q_row0 + r_hi) * p.heads + h) * D + n * 8 + t2) =
            pack2(o[n][2] * inv1, o[n][3] * inv1);
    }
  }
}

// ---------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// [batch, rows, hh, D] bf16 rows of which `rows` are live per sequence; consecutive sequences are `cap_rows`
// rows apart (a cache allocated longer than its live keys is read in place: rows past `rows` are out of the
// map's bounds and arrive as zeros, whatever the memory behind them holds).
int make_tmap_4d(mb_ctx* ctx, CUtensorMap* tm, const void* basep, uint64_t batch, uint64_t rows, uint64_t cap_rows,
                 uint64_t hh, uint32_t box_rows) {
  if (!ctx->encode_tiled) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    MB_CUDA_OK(ctx, cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q));
    if (!sym || q != cudaDriverEntryPointSuccess)
      return mb_fail(ctx, MB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    ctx->encode_tiled = sym;
  }
  EncodeTiledFn enc = reinterpret_cast<EncodeTiledFn>(ctx->encode_tiled);
  cuuint64_t dims[4] = {uint64_t(D), hh, rows, batch};
  cuuint64_t strides[3] = {uint64_t(D) * 2, hh * D * 2, cap_rows * hh * D * 2};
  cuuint32_t box[4] = {64, 1, box_rows, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(basep), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return mb_fail(ctx, MB_ERR_CUDA, "cuTensorMapEncodeTiled (attention) failed with %d", int(r));
  return MB_OK;
}

uint32_t decode_splits(size_t batch, size_t kv_heads, size_t keys) {
  // Fill a 148-SM part about eight CTAs deep; never split below 256 keys. The CTAs of a launch all
  // take about the same time, so among a few more splits than that the count whose last wave of
  // 148 x 2 resident CTAs is fullest wins (5 splits of 256 (sequence, head) pairs leave the fifth wave
  // a third full, 8 fill seven waves).
  size_t base = batch * kv_heads;
  size_t want = (size_t(148) * 8 + base - 1) / base;
  size_t max_splits = (keys + 255) / 256;
  if (max_splits > 64) max_splits = 64;
  if (want < 1) want = 1;
  if (want >= max_splits) return uint32_t(max_splits ? max_splits : 1);
  const size_t slots = size_t(148) * 2;
  size_t best = want;
  double best_eff = 0.0;
  for (size_t s = want; s <= want + 6 && s <= max_splits; ++s) {
    const size_t total = base * s, waves = (total + slots - 1) / slots;
    const double eff = double(total) / double(waves * slots);
    if (eff > best_eff + 0.02) { best_eff = eff; best = s; }
  }
  return uint32_t(best);
}

// [batch, live rows, elems] out of [batch, cap rows, elems] f32 -> contiguous bf16 (elems a multiple of 4)
__global__ void __launch_bounds__(256)
f32_rows_to_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, size_t live_elems,
                        size_t cap_elems, size_t total4) {
  const size_t i = size_t(blockIdx.x) * 256 + threadIdx.x;
  if (i >= total4) return;
  const size_t e = i * 4, b = e / live_elems, r = e - b * live_elems;
  const float4 v = *reinterpret_cast<const float4*>(src + b * cap_elems + r);
  *reinterpret_cast<uint2*>(dst + e) = make_uint2(pack2(v.x, v.y), pack2(v.z, v.w));
}
__global__ void __launch_bounds__(256)
bf16_to_f32_kernel(const __nv_bfloat16* __restrict__ src, float* __restrict__ dst, size_t total4) {
  const size_t i = size_t(blockIdx.x) * 256 + threadIdx.x;
  if (i >= total4) return;
  const uint2 v = *reinterpret_cast<const uint2*>(src + i * 4);
  *reinterpret_cast<float4*>(dst + i * 4) = make_float4(__uint_as_float(v.x << 16), __uint_as_float(v.x & 0xFFFF0000u),
                                                        __uint_as_float(v.y << 16), __uint_as_float(v.y & 0xFFFF0000u));
}

// NVFP4 rows -> contiguous bf16 [batch, live rows, elems] (exact: a code times its block scale has six significant
// bits). One 16-value block per thread; the source keeps `cap` rows per sequence, of which `live` are copied.
__global__ void __launch_bounds__(256)
fp4_rows_to_bf16_kernel(const uint2* __restrict__ codes, const uint8_t* __restrict__ scales, uint4* __restrict__ dst,
                        size_t live_blocks, size_t cap_blocks, size_t total_blocks) {
  const size_t i = size_t(blockIdx.x) * 256 + threadIdx.x;
  if (i >= total_blocks) return;
  const size_t b = i / live_blocks, r = i - b * live_blocks, src = b * cap_blocks + r;
  const uint2 c = __ldg(codes + src);
  uint32_t sh;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(sh) : "h"(uint16_t(__ldg(scales + src))));
  const __half2 sc = __low2half2(*reinterpret_cast<__half2*>(&sh));
  uint32_t h[8];
  fp4_decode4(c.x & 0xFFFFu, sc, h[0], h[1]);
  fp4_decode4(c.x >> 16, sc, h[2], h[3]);
  fp4_decode4(c.y & 0xFFFFu, sc, h[4], h[5]);
  fp4_decode4(c.y >> 16, sc, h[6], h[7]);
  uint32_t w[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float2 f = __half22float2(*reinterpret_cast<__half2*>(&h[j]));
    w[j] = pack2(f.x, f.y);
  }
  dst[i * 2] = make_uint4(w[0], w[1], w[2], w[3]);
  dst[i * 2 + 1] = make_uint4(w[4], w[5], w[6], w[7]);
}

struct AttnExt {
  const float* rel = nullptr;
  size_t eff = 0;
  const uint32_t* gap_rows = nullptr;
  const uint32_t* gap_cums = nullptr;
  size_t ngaps = 0;
};

// One run of key/value rows as a launch sees it: its live rows only.
struct RunView {
  const void* k = nullptr;          // first live row: bf16 values, or NVFP4 code bytes
  const void* v = nullptr;
  const uint8_t* k_scales = nullptr;
  const uint8_t* v_scales = nullptr;
  size_t live = 0;                  // live rows
  size_t cap = 0;                   // rows per sequence of the buffer (the batch stride)
  size_t pos0 = 0;                  // absolute position of the first live row (gaps aside)
  size_t row0 = 0;                  // logical row of the first live row (the gap table's index)
};

// The rows of a run some query of the block can see, [first, end) in live-row numbering, and the split count
// each run gets: the call's total follows decode_splits over all visible rows, a run takes its share by span
// (src/models/inkling/flash.rs `key_run_splits`), at least one, never below 256 keys per split.
struct RunPlan {
  size_t first = 0, end = 0;
  uint32_t splits = 0, slot0 = 0;
};

size_t plan_runs(const RunView* runs, size_t n_runs, size_t batch, size_t kv_heads, size_t nq, size_t q0, int causal,
                 size_t window, bool gapped, RunPlan* plan) {
  size_t total = 0;
  for (size_t i = 0; i < n_runs; ++i) {
    const RunView& r = runs[i];
    size_t end = r.live, first = 0;
    if (causal) {
      // a key at position pos0 + row (or later, with gaps) is visible to the last query when pos <= q0 + nq - 1
      end = q0 + nq > r.pos0 ? std::min(r.live, q0 + nq - r.pos0) : 0;
    }
    if (window && !gapped && q0 + 1 > window + r.pos0) first = std::min(end, (q0 + 1 - window - r.pos0) / BC * BC);
    plan[i].first = first;
    plan[i].end = end;
    total += end - first;
  }
  const size_t want = decode_splits(batch, kv_heads, total ? total : 1);
  uint32_t slots = 0;
  for (size_t i = 0; i < n_runs; ++i) {
    const size_t span = plan[i].end - plan[i].first;
    uint32_t s = 0;
    if (span) {
      const size_t by_span = (want * span + total - 1) / total;
      const size_t cap = std::min<size_t>((span + 255) / 256, 64);
      s = uint32_t(std::max<size_t>(1, std::min(by_span, cap)));
    }
    plan[i].splits = s;
    plan[i].slot0 = slots;
    slots += s;
  }
  return slots;
}

int decode_set_attributes(mb_ctx* ctx) {
  if (!mb_once(ctx, MB_ONCE_ATTN_DECODE)) {
    MB_CUDA_OK(ctx, cudaFuncSetAttribute(attn_decode_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, DEC_SMEM));
    MB_CUDA_OK(ctx, cudaFuncSetAttribute(attn_decode_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, DEC_SMEM));
    MB_CUDA_OK(ctx, cudaFuncSetAttribute(attn_decode_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, DEC_SMEM_FP4));
    MB_CUDA_OK(ctx, cudaFuncSetAttribute(attn_decode_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, DEC_SMEM_FP4));
    mb_once_done(ctx, MB_ONCE_ATTN_DECODE);
  }
  return MB_OK;
}

constexpr size_t MAX_RUNS = 64;

// Attention of one query block over key runs. q/out bf16 (q, out) or f32 (q_f32, out_f32).
int attention_core(mb_ctx* ctx, cudaStream_t stream, const void* q, const float* q_f32, const RunView* runs,
                   size_t n_runs, bool fp4, size_t batch, size_t nq, size_t heads, size_t kv_heads, size_t d, size_t q0,
                   float scale, int causal, size_t window, const AttnExt* ext, void* out, float* out_f32,
                   void* workspace, size_t workspace_bytes) {
  MB_REQUIRE(ctx, ctx != nullptr, "attention: null context");
  MB_REQUIRE(ctx, window == 0 || causal, "attention: a sliding window is a causal window");
  MB_REQUIRE(ctx, window < (1ull << 31), "attention: bad window");
  MB_REQUIRE(ctx, (q || q_f32) && (out || out_f32) && runs && n_runs > 0, "attention: null argument");
  MB_REQUIRE(ctx, n_runs <= MAX_RUNS, "attention: at most %zu key runs per call, got %zu", MAX_RUNS, n_runs);
  MB_REQUIRE(ctx, d == D, "attention: head_dim must be 128, got %zu", d);
  MB_REQUIRE(ctx, batch > 0 && nq > 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0,
             "attention: bad extents (batch %zu, nq %zu, heads %zu, kv_heads %zu)", batch, nq, heads, kv_heads);
  MB_REQUIRE(ctx, scale == scale && scale > 0.0f, "attention: scale must be positive");
  MB_REQUIRE(ctx, mb_aligned(q, 16) && mb_aligned(q_f32, 16) && mb_aligned(out, 16) && mb_aligned(out_f32, 16),
             "attention: 16-byte alignment");
  MB_REQUIRE(ctx, batch <= 65535 && heads <= 65535 && kv_heads <= 65535 && nq < (1ull << 31) && q0 < (1ull << 31),
             "attention: extent overflow");
  MB_REQUIRE_DEVICE(ctx, "attention");
  const bool has_ext = ext && (ext->rel || ext->ngaps);
  const size_t group = heads / kv_heads;
  const bool decode = nq * group <= 16;
  size_t total_live = 0;
  for (size_t i = 0; i < n_runs; ++i) {
    const RunView& r = runs[i];
    MB_REQUIRE(ctx, r.k && r.v && (!fp4 || (r.k_scales && r.v_scales)), "attention: key run %zu has a null plane", i);
    MB_REQUIRE(ctx, r.live <= r.cap && r.cap < (1ull << 31) && r.pos0 < (1ull << 31) && r.row0 < (1ull << 31),
               "attention: key run %zu: %zu live rows of %zu, position %zu", i, r.live, r.cap, r.pos0);
    if (fp4)
      MB_REQUIRE(ctx, mb_aligned(r.k, 16) && mb_aligned(r.v, 16) && mb_aligned(r.k_scales, 8) && mb_aligned(r.v_scales, 8),
                 "attention: NVFP4 rows need 16-byte aligned codes and 8-byte aligned scales");
    else
      MB_REQUIRE(ctx, mb_aligned(r.k, 16) && mb_aligned(r.v, 16), "attention: 16-byte alignment");
    total_live += r.live;
  }
  MB_REQUIRE(ctx, total_live > 0, "attention: no live key in any run");
  if (fp4)
    MB_REQUIRE(ctx, decode, "attention: NVFP4 rows are read by the decode kernel only (nq * heads / kv_heads <= 16)");
  if (has_ext) {
    MB_REQUIRE(ctx, causal, "attention: relative bias and eviction gaps belong to causal attention");
    MB_REQUIRE(ctx, !ext->rel || ext->eff > 0, "attention: a relative bias table needs eff > 0");
    MB_REQUIRE(ctx, ext->ngaps <= 64 && (ext->ngaps == 0 || (ext->gap_rows && ext->gap_cums)), "attention: bad gap list");
    MB_REQUIRE(ctx, ext->eff < (1ull << 31), "attention: bad eff");
  }
  const bool gapped = has_ext && ext->ngaps > 0;

  AttnParams p;
  memset(&p, 0, sizeof p);
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.q_f32 = q_f32;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.out_f32 = out_f32;
  p.flags = ctx->flags_dev;
  p.batch = uint32_t(batch); p.nq = uint32_t(nq); p.heads = uint32_t(heads);
  p.kv_heads = uint32_t(kv_heads); p.causal = causal;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.window = uint32_t(window);
  p.q0_abs = uint32_t(q0);
  if (has_ext) {
    p.rel = ext->rel; p.eff = uint32_t(ext->rel ? ext->eff : 0);
    p.gap_rows = ext->gap_rows; p.gap_cums = ext->gap_cums; p.ngaps = uint32_t(ext->ngaps);
  }

  if (decode) {
    RunPlan plan[MAX_RUNS];
    const size_t slots = plan_runs(runs, n_runs, batch, kv_heads, nq, q0, causal, window, gapped, plan);
    if (slots == 0) {
      // no query of the block sees any key: the reference's combine writes zeros there
      if (out_f32) MB_CUDA_OK(ctx, cudaMemsetAsync(out_f32, 0, batch * nq * heads * D * sizeof(float), stream));
      else MB_CUDA_OK(ctx, cudaMemsetAsync(out, 0, batch * nq * heads * D * 2, stream));
      return MB_OK;
    }
    const size_t need = batch * kv_heads * slots * 16 * (D + 2) * sizeof(float);
    if (slots > 1) {
      MB_REQUIRE(ctx, workspace && workspace_bytes >= need, "attention: decode needs %zu workspace bytes", need);
      MB_REQUIRE(ctx, mb_aligned(workspace, 16), "attention: workspace needs 16-byte alignment");
    }
    int rc = decode_set_attributes(ctx);
    if (rc) return rc;
    p.slots = uint32_t(slots);
    p.part = static_cast<float*>(workspace);
    for (size_t i = 0; i < n_runs; ++i) {
      if (!plan[i].splits) continue;
      const RunView& r = runs[i];
      p.keys = uint32_t(plan[i].end);
      p.k_lo = uint32_t(plan[i].first);
      p.q0 = uint32_t(int64_t(q0) - int64_t(r.pos0));       // relative to the run's first live row; may be negative
      p.pos0 = uint32_t(r.pos0); p.row0 = uint32_t(r.row0);
      p.cap = uint32_t(r.cap);
      p.splits = plan[i].splits; p.slot0 = plan[i].slot0;
      const size_t span = plan[i].end - plan[i].first;
      p.keys_per_split = uint32_t(((span + p.splits - 1) / p.splits + BC - 1) / BC * BC);
      if (fp4) {
        p.k_codes = static_cast<const uint8_t*>(r.k); p.v_codes = static_cast<const uint8_t*>(r.v);
        p.k_scales = r.k_scales; p.v_scales = r.v_scales;
      } else {
        rc = make_tmap_4d(ctx, &p.tmap_k, r.k, batch, plan[i].end, r.cap, kv_heads, BC);
        if (rc) return rc;
        rc = make_tmap_4d(ctx, &p.tmap_v, r.v, batch, plan[i].end, r.cap, kv_heads, BC);
        if (rc) return rc;
      }
      dim3 grid(p.splits, unsigned(kv_heads), unsigned(batch));
      if (fp4 && has_ext)
        MB_CUDA_OK(ctx, mb_launch_pdl(attn_decode_kernel<true, true>, grid, dim3(DEC_THREADS_FP4), DEC_SMEM_FP4, stream, p));
      else if (fp4)
        MB_CUDA_OK(ctx, mb_launch_pdl(attn_decode_kernel<true, false>, grid, dim3(DEC_THREADS_FP4), DEC_SMEM_FP4, stream, p));
      else if (has_ext)
        MB_CUDA_OK(ctx, mb_launch_pdl(attn_decode_kernel<false, true>, grid, dim3(DEC_THREADS), DEC_SMEM, stream, p));
      else
        MB_CUDA_OK(ctx, mb_launch_pdl(attn_decode_kernel<false, false>, grid, dim3(DEC_THREADS), DEC_SMEM, stream, p));
      MB_LAUNCH_OK(ctx);
    }
    if (slots > 1) {
      MB_CUDA_OK(ctx, mb_launch_pdl(attn_combine_kernel, dim3(unsigned(batch * nq * heads)), dim3(128), 0, stream, p.part, p.out,
                                    p.out_f32, p.nq, p.heads, p.kv_heads, uint32_t(slots)));
      MB_LAUNCH_OK(ctx);
    }
    return MB_OK;
  }

  // prompt shapes: one run (the freshly projected keys and values, or one cache the prompt was appended to)
  const RunView* one = nullptr;
  for (size_t i = 0; i < n_runs; ++i) {
    if (!runs[i].live) continue;
    MB_REQUIRE(ctx, one == nullptr, "attention: prompt shapes (nq * heads / kv_heads > 16) take one key run, not %zu", n_runs);
    one = &runs[i];
  }
  MB_REQUIRE(ctx, q != nullptr && out != nullptr, "attention: prompt shapes take bf16 queries and write bf16");
  MB_REQUIRE(ctx, q0 >= one->pos0, "attention: the first query (position %zu) stands before the run's first key (%zu)",
             q0, one->pos0);
  MB_REQUIRE(ctx, one->live < (1ull << 31), "attention: extent overflow");
  MB_REQUIRE(ctx, window == 0 || gapped || one->live >= q0 - one->pos0 + nq,
             "attention: with a window every query needs its own key in the cache");
  p.keys = uint32_t(one->live);
  p.q0 = uint32_t(q0 - one->pos0);
  p.splits = 1; p.slots = 1;
  int rc = make_tmap_4d(ctx, &p.tmap_k, one->k, batch, one->live, one->cap, kv_heads, BC);
  if (rc) return rc;
  rc = make_tmap_4d(ctx, &p.tmap_v, one->v, batch, one->live, one->cap, kv_heads, BC);
  if (rc) return rc;
  if (!has_ext && !mb_attention_prefill_legacy()) {
    rc = make_tmap_4d(ctx, &p.tmap_q, q, batch, nq, nq, heads, 128);
    if (rc) return rc;
    return mb_attention_prefill_tc5(ctx, stream, p);
  }
  // The warp-level (mma.sync) kernel: the route of prompt-shaped blocks with a relative bias or eviction gaps
  // (its EXT instantiation masks and biases by position, window included), and the comparison arm of the rest.
  MB_REQUIRE(ctx, has_ext || window == 0, "attention: the comparison (mma.sync) prefill kernel has no sliding window");
  p.pos0 = uint32_t(one->pos0); p.row0 = uint32_t(one->row0);
  rc = make_tmap_4d(ctx, &p.tmap_q, q, batch, nq, nq, heads, BR);
  if (rc) return rc;
  if (!mb_once(ctx, MB_ONCE_ATTN_PREFILL_LEGACY)) {
    MB_CUDA_OK(ctx, cudaFuncSetAttribute(attn_prefill_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, PRE_SMEM));
    MB_CUDA_OK(ctx, cudaFuncSetAttribute(attn_prefill_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, PRE_SMEM));
    mb_once_done(ctx, MB_ONCE_ATTN_PREFILL_LEGACY);
  }
  dim3 grid(unsigned((nq + BR - 1) / BR), unsigned(heads), unsigned(batch));
  if (has_ext) attn_prefill_kernel<true><<<grid, PRE_THREADS, PRE_SMEM, stream>>>(p);
  else attn_prefill_kernel<false><<<grid, PRE_THREADS, PRE_SMEM, stream>>>(p);
  MB_LAUNCH_OK(ctx);
  return MB_OK;
}

// The single-buffer entry points: one run of `keys` live rows at position 0 in a buffer of `keys` rows.
int attention_common(mb_ctx* ctx, mb_stream stream_, const void* q, const void* k, const void* v, size_t batch,
                     size_t nq, size_t keys, size_t heads, size_t kv_heads, size_t d, size_t q0, float scale,
                     int causal, size_t window, void* out, void* workspace, size_t workspace_bytes,
                     const uint8_t* const* fp4 = nullptr, const AttnExt* ext = nullptr) {
  MB_REQUIRE(ctx, keys > 0 && keys < (1ull << 31), "attention: bad key count %zu", keys);
  MB_REQUIRE(ctx, window == 0 || (ext && ext->ngaps) || keys >= q0 + nq,
             "attention: with a window every query needs its own key in the cache");
  RunView r;
  if (fp4) { r.k = fp4[0]; r.k_scales = fp4[1]; r.v = fp4[2]; r.v_scales = fp4[3]; }
  else { r.k = k; r.v = v; }
  r.live = keys; r.cap = keys;
  return attention_core(ctx, static_cast<cudaStream_t>(stream_), q, nullptr, &r, 1, fp4 != nullptr, batch, nq, heads,
                        kv_heads, d, q0, scale, causal, window, ext, out, nullptr, workspace, workspace_bytes);
}

}  // namespace

MB_API size_t mb_attention_workspace(size_t batch, size_t nq, size_t keys, size_t heads, size_t kv_heads, size_t d) {
  (void)d;
  if (kv_heads == 0 || heads % kv_heads != 0) return 0;
  if (nq * (heads / kv_heads) > 16) return 0;   // prefill needs none
  return batch * kv_heads * size_t(decode_splits(batch, kv_heads, keys)) * 16 * (D + 2) * sizeof(float);
}

MB_API int mb_attention(mb_ctx* ctx, mb_stream stream, const void* q, const void* k, const void* v, size_t batch,
                        size_t nq, size_t keys, size_t heads, size_t kv_heads, size_t d, size_t q0, float scale,
                        int causal, void* out, void* workspace, size_t workspace_bytes) {
  return attention_common(ctx, stream, q, k, v, batch, nq, keys, heads, kv_heads, d, q0, scale, causal, 0, out, workspace,
                          workspace_bytes);
}

MB_API int mb_attention_window(mb_ctx* ctx, mb_stream stream, const void* q, const void* k, const void* v, size_t batch,
                               size_t nq, size_t keys, size_t heads, size_t kv_heads, size_t d, size_t q0, float scale,
                               size_t window, void* out, void* workspace, size_t workspace_bytes) {
  return attention_common(ctx, stream, q, k, v, batch, nq, keys, heads, kv_heads, d, q0, scale, 1, window, out, workspace,
                          workspace_bytes);
}

MB_API int mb_attention_fp4kv(mb_ctx* ctx, mb_stream stream, const void* q, const uint8_t* k_codes,
                              const uint8_t* k_scales, const uint8_t* v_codes, const uint8_t* v_scales, size_t batch,
                              size_t nq, size_t keys, size_t heads, size_t kv_heads, size_t d, size_t q0, float scale,
                              int causal, size_t window, void* out, void* workspace, size_t workspace_bytes) {
  const uint8_t* planes[4] = {k_codes, k_scales, v_codes, v_scales};
  MB_REQUIRE(ctx, k_codes && k_scales && v_codes && v_scales, "attention: null argument");
  return attention_common(ctx, stream, q, nullptr, nullptr, batch, nq, keys, heads, kv_heads, d, q0, scale, causal,
                          window, out, workspace, workspace_bytes, planes);
}

MB_API int mb_attention_decode_ext(mb_ctx* ctx, mb_stream stream, const void* q, const void* k, const void* v,
                                   size_t batch, size_t nq, size_t keys, size_t heads, size_t kv_heads, size_t d,
                                   size_t q0, float scale, size_t window, const float* rel, size_t eff,
                                   const uint32_t* gap_rows, const uint32_t* gap_cums, size_t ngaps, void* out,
                                   void* workspace, size_t workspace_bytes) {
  AttnExt ext;
  ext.rel = rel; ext.eff = eff; ext.gap_rows = gap_rows; ext.gap_cums = gap_cums; ext.ngaps = ngaps;
  return attention_common(ctx, stream, q, k, v, batch, nq, keys, heads, kv_heads, d, q0, scale, 1, window, out,
                          workspace, workspace_bytes, nullptr, &ext);
}

// ---------------------------------------------------------------------------------
// flash_attention_launch over key runs (one run per page of a paged cache).
// ---------------------------------------------------------------------------------
namespace {

size_t align256(size_t n) { return (n + 255) / 256 * 256; }

// Live-row views of the caller's runs. For an f32 cache `converted` (when given) is where the bf16 copy of the
// live rows of K then V of each run goes; the views then point there.
// `expand`: the rows are read through a bf16 copy of the live rows in the workspace (always for f32 rows; for NVFP4
// rows when the query block is prompt-shaped, which the tensor-core kernel serves from bf16 tiles).
int view_runs(mb_ctx* ctx, const mb_key_run* runs, size_t n_runs, int kv_elem, bool expand, size_t batch, size_t kv_heads,
              uint8_t* converted, RunView* views, size_t* converted_bytes) {
  const size_t row_bytes = kv_heads * D * (kv_elem == MB_KV_F32 ? 4 : kv_elem == MB_KV_BF16 ? 2 : 0);
  size_t off = 0;
  for (size_t i = 0; i < n_runs; ++i) {
    const mb_key_run& r = runs[i];
    MB_REQUIRE(ctx, r.lo <= r.hi && r.hi <= r.rows, "attention_runs: run %zu: live range %zu..%zu is not inside its %zu rows",
               i, r.lo, r.hi, r.rows);
    MB_REQUIRE(ctx, r.k && r.v, "attention_runs: run %zu has a null plane", i);
    MB_REQUIRE(ctx, (kv_elem == MB_KV_NVFP4) == (r.k_scales != nullptr && r.v_scales != nullptr),
               "attention_runs: NVFP4 needs both block-scale planes and no other element type may carry them");
    RunView& v = views[i];
    v = RunView();
    v.live = r.hi - r.lo; v.cap = r.rows; v.pos0 = r.base + r.lo; v.row0 = r.row0 + r.lo;
    if (kv_elem == MB_KV_NVFP4 && !expand) {
      v.k = static_cast<const uint8_t*>(r.k) + r.lo * kv_heads * (D / 2);
      v.v = static_cast<const uint8_t*>(r.v) + r.lo * kv_heads * (D / 2);
      v.k_scales = static_cast<const uint8_t*>(r.k_scales) + r.lo * kv_heads * (D / 16);
      v.v_scales = static_cast<const uint8_t*>(r.v_scales) + r.lo * kv_heads * (D / 16);
    } else if (kv_elem == MB_KV_BF16) {
      v.k = static_cast<const uint8_t*>(r.k) + r.lo * row_bytes;
      v.v = static_cast<const uint8_t*>(r.v) + r.lo * row_bytes;
    } else {
      const size_t plane = align256(batch * v.live * kv_heads * D * 2);
      if (converted) { v.k = converted + off; v.v = converted + off + plane; }
      else { v.k = r.k; v.v = r.v; }       // sizing pass: any non-null pointer
      v.cap = v.live;
      off += 2 * plane;
    }
  }
  *converted_bytes = off;
  return MB_OK;
}

}  // namespace

MB_API size_t mb_attention_runs_workspace(const mb_key_run* runs, size_t n_runs, int kv_elem, size_t batch, size_t nq,
                                          size_t q0, size_t heads, size_t kv_heads, size_t d, size_t window, size_t ngaps,
                                          int q_dtype, int out_dtype) {
  (void)d;
  if (!runs || n_runs == 0 || n_runs > MAX_RUNS || kv_heads == 0 || heads % kv_heads != 0) return 0;
  RunView views[MAX_RUNS];
  size_t conv = 0;
  const bool prompt = nq * (heads / kv_heads) > 16;
  if (view_runs(nullptr, runs, n_runs, kv_elem, kv_elem == MB_KV_F32 || prompt, batch, kv_heads, nullptr, views, &conv) != MB_OK)
    return 0;
  size_t need = conv;
  if (nq * (heads / kv_heads) <= 16) {
    RunPlan plan[MAX_RUNS];
    const size_t slots = plan_runs(views, n_runs, batch, kv_heads, nq, q0, 1, window, ngaps > 0, plan);
    if (slots > 1) need += align256(batch * kv_heads * slots * 16 * (D + 2) * sizeof(float));
  } else {
    if (q_dtype == MB_DT_F32) need += align256(batch * nq * heads * D * 2);
    if (out_dtype == MB_DT_F32) need += align256(batch * nq * heads * D * 2);
  }
  return need;
}

MB_API int mb_attention_runs(mb_ctx* ctx, mb_stream stream_, const void* q, int q_dtype, const mb_key_run* runs,
                             size_t n_runs, int kv_elem, const float* rel, size_t eff, const uint32_t* gap_rows,
                             const uint32_t* gap_cums, size_t ngaps, size_t batch, size_t nq, size_t q0, size_t heads,
                             size_t kv_heads, size_t d, size_t window, float scale, void* out, int out_dtype,
                             void* workspace, size_t workspace_bytes) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  MB_REQUIRE(ctx, ctx && q && out && runs, "attention_runs: null argument");
  MB_REQUIRE(ctx, n_runs > 0 && n_runs <= MAX_RUNS, "attention_runs: 1..%zu key runs, got %zu", MAX_RUNS, n_runs);
  MB_REQUIRE(ctx, kv_elem == MB_KV_F32 || kv_elem == MB_KV_BF16 || kv_elem == MB_KV_NVFP4, "attention_runs: unknown key/value element type %d", kv_elem);
  MB_REQUIRE(ctx, (q_dtype == MB_DT_BF16 || q_dtype == MB_DT_F32) && (out_dtype == MB_DT_BF16 || out_dtype == MB_DT_F32),
             "attention_runs: queries and output are bf16 or f32");
  MB_REQUIRE(ctx, d == D && kv_heads > 0 && heads > 0 && heads % kv_heads == 0 && batch > 0 && nq > 0,
             "attention_runs: bad extents (head_dim %zu, heads %zu, kv_heads %zu, batch %zu, nq %zu)", d, heads, kv_heads, batch, nq);
  MB_REQUIRE(ctx, workspace == nullptr || mb_aligned(workspace, 256), "attention_runs: workspace needs 256-byte alignment");
  const size_t need = mb_attention_runs_workspace(runs, n_runs, kv_elem, batch, nq, q0, heads, kv_heads, d, window, ngaps,
                                                  q_dtype, out_dtype);
  MB_REQUIRE(ctx, need == 0 || (workspace && workspace_bytes >= need), "attention_runs: needs %zu workspace bytes", need);
  MB_REQUIRE_DEVICE(ctx, "attention_runs");
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  RunView views[MAX_RUNS];
  size_t conv = 0;
  const bool decode = nq * (heads / kv_heads) <= 16;
  const bool expand_fp4 = kv_elem == MB_KV_NVFP4 && !decode;
  int rc = view_runs(ctx, runs, n_runs, kv_elem, kv_elem == MB_KV_F32 || expand_fp4, batch, kv_heads, ws, views, &conv);
  if (rc) return rc;
  if (expand_fp4) {
    // prompt-shaped reads of packed rows: the reference's dequantizing reader (src/models/inkling/flash.rs:520-540);
    // the live rows are expanded to bf16 once (exactly) and the tensor-core kernel reads those
    for (size_t i = 0; i < n_runs; ++i) {
      const size_t live = views[i].live;
      if (!live) continue;
      MB_REQUIRE(ctx, mb_aligned(runs[i].k, 8) && mb_aligned(runs[i].v, 8), "attention_runs: NVFP4 rows need 8-byte aligned codes");
      const size_t row_blocks = kv_heads * (D / 16), total = batch * live * row_blocks;
      const unsigned grid = unsigned((total + 255) / 256);
      const uint8_t* kc = static_cast<const uint8_t*>(runs[i].k) + runs[i].lo * row_blocks * 8;
      const uint8_t* vc = static_cast<const uint8_t*>(runs[i].v) + runs[i].lo * row_blocks * 8;
      const uint8_t* ksc = static_cast<const uint8_t*>(runs[i].k_scales) + runs[i].lo * row_blocks;
      const uint8_t* vsc = static_cast<const uint8_t*>(runs[i].v_scales) + runs[i].lo * row_blocks;
      fp4_rows_to_bf16_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<const uint2*>(kc), ksc,
                                                        static_cast<uint4*>(const_cast<void*>(views[i].k)), live * row_blocks,
                                                        runs[i].rows * row_blocks, total);
      fp4_rows_to_bf16_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<const uint2*>(vc), vsc,
                                                        static_cast<uint4*>(const_cast<void*>(views[i].v)), live * row_blocks,
                                                        runs[i].rows * row_blocks, total);
      MB_LAUNCH_OK(ctx);
    }
  }
  if (kv_elem == MB_KV_F32) {
    // f32 rows go through a bf16 copy of the live rows (both products multiply bf16)
    for (size_t i = 0; i < n_runs; ++i) {
      const size_t live = views[i].live;
      if (!live) continue;
      MB_REQUIRE(ctx, mb_aligned(runs[i].k, 16) && mb_aligned(runs[i].v, 16), "attention_runs: 16-byte alignment");
      const size_t row = kv_heads * D, total4 = batch * live * row / 4;
      const float* ksrc = static_cast<const float*>(runs[i].k) + runs[i].lo * row;
      const float* vsrc = static_cast<const float*>(runs[i].v) + runs[i].lo * row;
      const unsigned grid = unsigned((total4 + 255) / 256);
      f32_rows_to_bf16_kernel<<<grid, 256, 0, stream>>>(ksrc, static_cast<__nv_bfloat16*>(const_cast<void*>(views[i].k)),
                                                        live * row, runs[i].rows * row, total4);
      f32_rows_to_bf16_kernel<<<grid, 256, 0, stream>>>(vsrc, static_cast<__nv_bfloat16*>(const_cast<void*>(views[i].v)),
                                                        live * row, runs[i].rows * row, total4);
      MB_LAUNCH_OK(ctx);
    }
  }
  ws += conv;
  AttnExt ext;
  ext.rel = rel; ext.eff = eff; ext.gap_rows = gap_rows; ext.gap_cums = gap_cums; ext.ngaps = ngaps;
  if (decode) {
    return attention_core(ctx, stream, q_dtype == MB_DT_BF16 ? q : nullptr,
                          q_dtype == MB_DT_F32 ? static_cast<const float*>(q) : nullptr, views, n_runs,
                          kv_elem == MB_KV_NVFP4, batch, nq, heads, kv_heads, d, q0, scale, 1, window, &ext,
                          out_dtype == MB_DT_BF16 ? out : nullptr, out_dtype == MB_DT_F32 ? static_cast<float*>(out) : nullptr,
                          ws, workspace_bytes - conv);
  }
  // prompt shapes run on the tcgen05 kernel, which reads and writes bf16: f32 queries and output pass through
  // bf16 staging areas of the workspace
  const size_t qo4 = batch * nq * heads * D / 4;
  const void* q16 = q;
  if (q_dtype == MB_DT_F32) {
    MB_REQUIRE(ctx, mb_aligned(q, 16), "attention_runs: 16-byte alignment");
    f32_rows_to_bf16_kernel<<<unsigned((qo4 + 255) / 256), 256, 0, stream>>>(static_cast<const float*>(q),
                                                                             reinterpret_cast<__nv_bfloat16*>(ws), qo4 * 4, qo4 * 4, qo4);
    MB_LAUNCH_OK(ctx);
    q16 = ws;
    ws += align256(qo4 * 8);
  }
  void* out16 = out_dtype == MB_DT_F32 ? static_cast<void*>(ws) : out;
  rc = attention_core(ctx, stream, q16, nullptr, views, n_runs, false, batch, nq, heads, kv_heads, d, q0, scale, 1, window,
                      &ext, out16, nullptr, nullptr, 0);
  if (rc) return rc;
  if (out_dtype == MB_DT_F32) {
    MB_REQUIRE(ctx, mb_aligned(out, 16), "attention_runs: 16-byte alignment");
    bf16_to_f32_kernel<<<unsigned((qo4 + 255) / 256), 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(out16),
                                                                        static_cast<float*>(out), qo4);
    MB_LAUNCH_OK(ctx);
  }
  return MB_OK;
}

// ---------------------------------------------------------------------------------
// Decode attention for hosts that must not allocate.
//
// Some hosts of this library hand their whole device-memory budget to an arena of
// their own when they start (the compute client a Rust serving process keeps is one)
// and, from then on, treat any driver allocation as a fault: it would synchronise the
// device in the middle of a token step and can fail outright when the arena has left
// nothing. Such a host can pass inputs and outputs it already owns, but it has nowhere
// to get the scratch the key-split partials need. This entry point keeps that scratch
// in a fixed array inside the library image instead.
//
// The array, like any module-scope device data, comes into being when the driver loads
// this part of the library, which by default it puts off until first use. So that this
// does not happen in the middle of serving either, mb_ctx_create runs the set-up below
// (mb_attention_decode_static_warm): it resolves the array's address, sets the kernels'
// attributes and launches both kernels once on a tiny problem laid out inside the array
// itself. A host should create its contexts before it sizes its arena.
// ---------------------------------------------------------------------------------
constexpr size_t STATIC_SCRATCH_BYTES = size_t(16) << 20;   // 16 MiB, held by every GPU that loads the library
static __device__ __align__(256) unsigned char g_decode_scratch[STATIC_SCRATCH_BYTES];

// Device address of the array, resolved once per device. In host code the array's
// name is only a handle for the runtime; the kernel needs the address looked up here.
constexpr int STATIC_MAX_DEVICES = 64;
static float* g_decode_scratch_ptr[STATIC_MAX_DEVICES] = {};
static std::mutex g_decode_scratch_mu;

static int decode_static_launch(mb_ctx* ctx, cudaStream_t stream, const void* q, const void* k, const void* v,
                                size_t batch, size_t nq, size_t keys, size_t heads, size_t kv_heads, size_t q0,
                                float scale, int causal, void* out, float* scratch, uint32_t splits) {
  AttnParams p;
  memset(&p, 0, sizeof p);
  int rc = make_tmap_4d(ctx, &p.tmap_k, k, batch, keys, keys, kv_heads, BC);
  if (rc) return rc;
  rc = make_tmap_4d(ctx, &p.tmap_v, v, batch, keys, keys, kv_heads, BC);
  if (rc) return rc;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.flags = ctx->flags_dev;
  p.batch = uint32_t(batch); p.nq = uint32_t(nq); p.keys = uint32_t(keys); p.heads = uint32_t(heads);
  p.kv_heads = uint32_t(kv_heads); p.q0 = uint32_t(q0); p.q0_abs = uint32_t(q0); p.causal = causal;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.splits = splits; p.slots = splits; p.cap = uint32_t(keys);
  p.keys_per_split = uint32_t(((keys + splits - 1) / splits + BC - 1) / BC * BC);
  p.part = scratch;
  dim3 grid(splits, unsigned(kv_heads), unsigned(batch));
  MB_CUDA_OK(ctx, mb_launch_pdl(attn_decode_kernel<false, false>, grid, dim3(DEC_THREADS), DEC_SMEM, stream, p));
  MB_LAUNCH_OK(ctx);
  if (splits > 1) {
    MB_CUDA_OK(ctx, mb_launch_pdl(attn_combine_kernel, dim3(unsigned(batch * nq * heads)), dim3(128), 0, stream, p.part, p.out,
                                  static_cast<float*>(nullptr), p.nq, p.heads, p.kv_heads, splits));
    MB_LAUNCH_OK(ctx);
  }
  return MB_OK;
}

MB_API int mb_attention_decode_static_warm(mb_ctx* ctx) {
  MB_REQUIRE(ctx, ctx != nullptr, "attention_decode_static_warm: null context");
  if (mb_once(ctx, MB_ONCE_ATTN_STATIC)) return MB_OK;
  MB_REQUIRE_DEVICE(ctx, "attention_decode_static_warm");
  MB_REQUIRE(ctx, ctx->device < STATIC_MAX_DEVICES, "attention_decode_static_warm: device index %d is beyond %d", ctx->device,
             STATIC_MAX_DEVICES);
  float* base = nullptr;
  {
    std::lock_guard<std::mutex> g(g_decode_scratch_mu);
    if (!g_decode_scratch_ptr[ctx->device]) {
      void* ptr = nullptr;
      MB_CUDA_OK(ctx, cudaGetSymbolAddress(&ptr, g_decode_scratch));
      g_decode_scratch_ptr[ctx->device] = static_cast<float*>(ptr);
    }
    base = g_decode_scratch_ptr[ctx->device];
  }
  int rc = decode_set_attributes(ctx);
  if (rc) return rc;
  // One launch of the decode kernel and of the combine kernel, so that the driver has their code resident before
  // the host's first token step: one sequence, one head, 512 zero keys in two splits, every operand carved out of
  // the array itself (the array starts zeroed; the launch leaves partials and a zero output row in it).
  uint8_t* a = reinterpret_cast<uint8_t*>(base);
  const size_t kv_bytes = 512 * D * 2;
  rc = decode_static_launch(ctx, nullptr, a + (1 << 20), a + (2 << 20), a + (2 << 20) + kv_bytes, 1, 1, 512, 1, 1, 511,
                            0.088388347648f, 1, a + (1 << 20) + 4096, base, 2);
  if (rc) return rc;
  MB_CUDA_OK(ctx, cudaStreamSynchronize(nullptr));
  mb_once_done(ctx, MB_ONCE_ATTN_STATIC);
  return MB_OK;
}

MB_API int mb_attention_decode_static(mb_ctx* ctx, mb_stream stream_, const void* q, const void* k, const void* v,
                                      size_t batch, size_t nq, size_t keys, size_t heads, size_t kv_heads, size_t d,
                                      size_t q0, float scale, int causal, void* out) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  MB_REQUIRE(ctx, ctx && q && k && v && out, "attention_decode_static: null argument");
  MB_REQUIRE(ctx, d == D, "attention_decode_static: head_dim must be 128, got %zu", d);
  MB_REQUIRE(ctx, batch > 0 && nq > 0 && keys > 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0,
             "attention_decode_static: bad extents");
  MB_REQUIRE(ctx, nq * (heads / kv_heads) <= 16,
             "attention_decode_static: takes decode shapes only (nq * heads/kv_heads <= 16)");
  MB_REQUIRE(ctx, scale == scale && scale > 0.0f, "attention_decode_static: scale must be positive");
  MB_REQUIRE(ctx, mb_aligned(q, 16) && mb_aligned(k, 16) && mb_aligned(v, 16) && mb_aligned(out, 16),
             "attention_decode_static: 16-byte alignment");
  MB_REQUIRE(ctx, batch <= 65535 && heads <= 65535 && kv_heads <= 65535 && keys < (1ull << 31) && q0 < (1ull << 31),
             "attention_decode_static: extent overflow");
  // fewer key splits than the heuristic's when its choice would not fit the built-in array. The array's size is
  // also the entry point's stated limit: a shape whose partials would not fit it at one split is refused, although
  // an unsplit launch writes the output itself and would not touch the array (one limit, known in advance,
  // instead of one that depends on the split heuristic).
  uint32_t splits = decode_splits(batch, kv_heads, keys);
  const size_t per_split = batch * kv_heads * size_t(16) * (D + 2) * sizeof(float);
  while (splits > 1 && per_split * splits > STATIC_SCRATCH_BYTES) --splits;
  MB_REQUIRE(ctx, per_split * splits <= STATIC_SCRATCH_BYTES,
             "attention_decode_static: batch x kv_heads = %zu is beyond the entry point's limit: one split's partials take "
             "%zu bytes, the built-in array holds %zu; use mb_attention with a caller workspace",
             batch * kv_heads, per_split, STATIC_SCRATCH_BYTES);
  MB_REQUIRE_DEVICE(ctx, "attention_decode_static");
  int rc = mb_attention_decode_static_warm(ctx);      // a no-op after mb_ctx_create
  if (rc) return rc;
  return decode_static_launch(ctx, stream, q, k, v, batch, nq, keys, heads, kv_heads, q0, scale, causal, out,
                              g_decode_scratch_ptr[ctx->device], splits);
}
