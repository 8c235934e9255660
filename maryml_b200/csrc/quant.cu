// NVFP4 quantizers, dequantizer and scale-plane re-layout.
//
// All of these are HBM-bound byte kernels: one thread owns one or two 16-element blocks
// (32 B of bf16 or 64 B of f32 in, 8 B of codes + 1 scale byte out per block), loads are
// 128-bit, neighbouring lanes merge their scale bytes into one 32-bit store.
// Algorithmic traffic per element: 2 (bf16) or 4 (f32) bytes read + 0.5625 written.
#include "common.cuh"
#include "quant_block.cuh"

namespace {

constexpr int QUANT_THREADS = 256;
#ifndef QUANT_MIN_BLOCKS
#define QUANT_MIN_BLOCKS 5   // blocks per SM the two-block kernel is compiled for (register cap 48)
#endif

__device__ __forceinline__ void load16(const __nv_bfloat16* p, float* v) {
  const uint4* q = reinterpret_cast<const uint4*>(p);
  uint4 a = __ldg(q), b = __ldg(q + 1);
  uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}
__device__ __forceinline__ void load16(const float* p, float* v) {
  const float4* q = reinterpret_cast<const float4*>(p);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float4 a = __ldg(q + i);
    v[4 * i] = a.x; v[4 * i + 1] = a.y; v[4 * i + 2] = a.z; v[4 * i + 3] = a.w;
  }
}
// Scalar fallback for sources that are only element-aligned.
template <typename T>
__device__ __forceinline__ void load16_scalar(const T* p, float* v) {
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = float(p[i]);
}

// One thread per 16-value block. The kernel is bound by instruction issue, not by memory,
// unless the per-block instruction count stays near a hundred: the recipe is a template
// parameter, the block index splits into (row, k-block) by a multiply-high, the scale byte
// goes through the hardware E4M3 converters, amax / 6 is a three-instruction exact quotient.
template <typename T, int RECIPE>
__global__ void __launch_bounds__(QUANT_THREADS)
quantize_kernel(const T* __restrict__ x, uint32_t blocks, uint32_t k, mb_fastdiv rb, float input_scale,
                const float* __restrict__ rowscale, const int32_t* __restrict__ gather, uint2* __restrict__ codes,
                uint8_t* __restrict__ scales, int tiled, uint32_t kchunks, int vec_ok) {
  const uint32_t blk = blockIdx.x * QUANT_THREADS + threadIdx.x;
  const bool live = blk < blocks;
  const uint32_t row = mb_fastdiv_q(live ? blk : 0u, rb);
  const uint32_t kb = (live ? blk : 0u) - row * rb.d;
  uint32_t sbyte = 0;
  if (live) {
    float v[16];
    const int32_t src = gather ? gather[row] : int32_t(row);
    if (src < 0) {
#pragma unroll
      for (int i = 0; i < 16; ++i) v[i] = 0.0f;
    } else {
      const T* p = x + size_t(uint32_t(src)) * k + kb * 16u;
      if (vec_ok) load16(p, v); else load16_scalar(p, v);
    }
    uint2 c;
    if (RECIPE == MB_QUANT_RECIP) {
      quant_block_recip(v, sbyte, c);
    } else {
      const float s2 = RECIPE == MB_QUANT_ROWS ? rowscale[row] : input_scale;
      quant_block_scaled(v, s2, sbyte, c);
    }
    codes[blk] = c;
  }
  // Four neighbouring lanes (same row, kb%4 = 0..3) merge their scale bytes.
  if ((rb.d & 3u) == 0) {
    uint32_t w = sbyte;
    w |= __shfl_down_sync(0xFFFFFFFFu, sbyte, 1) << 8;
    w |= __shfl_down_sync(0xFFFFFFFFu, sbyte, 2) << 16;
    w |= __shfl_down_sync(0xFFFFFFFFu, sbyte, 3) << 24;
    if (live && (threadIdx.x & 3) == 0) {
      const size_t off = tiled ? mb_sf_offset(row, kb, kchunks) : blk;
      *reinterpret_cast<uint32_t*>(scales + off) = w;
    }
  } else if (live) {
    const size_t off = tiled ? mb_sf_offset(row, kb, kchunks) : blk;
    scales[off] = uint8_t(sbyte);
  }
}

// The same with two neighbouring blocks of a row per thread (k a multiple of 32): the index
// arithmetic, the parameter loads and the control flow are paid once per 32 values, the codes
// leave as one 128-bit store and two lanes fill a 32-bit word of scale bytes.
template <typename T, int RECIPE>
__global__ void __launch_bounds__(QUANT_THREADS, QUANT_MIN_BLOCKS)
quantize2_kernel(const T* __restrict__ x, uint32_t pairs, uint32_t k, mb_fastdiv rbp, float input_scale,
                 const float* __restrict__ rowscale, const int32_t* __restrict__ gather, uint4* __restrict__ codes,
                 uint8_t* __restrict__ scales, int tiled, uint32_t kchunks, int vec_ok) {
  mb_grid_dependency_sync();
  const uint32_t pr = blockIdx.x * QUANT_THREADS + threadIdx.x;
  const bool live = pr < pairs;
  const uint32_t row = mb_fastdiv_q(live ? pr : 0u, rbp);
  const uint32_t kb = ((live ? pr : 0u) - row * rbp.d) * 2u;
  uint32_t s0 = 0, s1 = 0;
  if (live) {
    const int32_t src = gather ? gather[row] : int32_t(row);
    if (src < 0) {
      // a pad row of a gathered plan: zero codes and zero scales, which is what zeros quantize to
      codes[pr] = make_uint4(0u, 0u, 0u, 0u);
    } else {
      float v[32];
      const T* p = x + size_t(uint32_t(src)) * k + kb * 16u;
      if (vec_ok) { load16(p, v); load16(p + 16, v + 16); }
      else { load16_scalar(p, v); load16_scalar(p + 16, v + 16); }
      uint2 c0, c1;
      if (RECIPE == MB_QUANT_RECIP) {
        quant_block_recip(v, s0, c0);
        quant_block_recip(v + 16, s1, c1);
      } else {
        const float s2 = RECIPE == MB_QUANT_ROWS ? rowscale[row] : input_scale;
        quant_block_scaled(v, s2, s0, c0);
        quant_block_scaled(v + 16, s2, s1, c1);
      }
      codes[pr] = make_uint4(c0.x, c0.y, c1.x, c1.y);
    }
  }
  const uint32_t w2 = s0 | (s1 << 8);
  if ((rbp.d & 1u) == 0) {
    // k-blocks per row a multiple of four: lanes (2j, 2j+1) hold kb % 4 = 0 and 2 of one word
    const uint32_t w = w2 | (__shfl_down_sync(0xFFFFFFFFu, w2, 1) << 16);
    if (live && (threadIdx.x & 1) == 0) {
      const size_t off = tiled ? mb_sf_offset(row, kb, kchunks) : size_t(pr) * 2;
      *reinterpret_cast<uint32_t*>(scales + off) = w;
    }
  } else if (live) {
    const size_t off = tiled ? mb_sf_offset(row, kb, kchunks) : size_t(pr) * 2;
    *reinterpret_cast<uint16_t*>(scales + off) = uint16_t(w2);
  }
}

template <typename T>
static void launch_quantize(cudaStream_t stream, int recipe, const T* x, size_t rows, size_t k, float input_scale,
                            const float* rowscale, const int32_t* gather, uint8_t* codes, uint8_t* scales, int tiled,
                            int vec_ok) {
  const uint32_t kc = uint32_t(mb_sf_kchunks(k));
  if (k % 32 == 0 && mb_aligned(codes, 16)) {
    const uint32_t pairs = uint32_t(rows * (k / 32));
    const unsigned grid2 = (pairs + QUANT_THREADS - 1) / QUANT_THREADS;
    const mb_fastdiv rbp = mb_fastdiv_make(uint32_t(k / 32));
    uint4* c4 = reinterpret_cast<uint4*>(codes);
    if (recipe == MB_QUANT_RECIP)
      mb_launch_pdl(quantize2_kernel<T, MB_QUANT_RECIP>, dim3(grid2), dim3(QUANT_THREADS), 0, stream, x, pairs, uint32_t(k), rbp,
                    input_scale, rowscale, gather, c4, scales, tiled, kc, vec_ok);
    else if (recipe == MB_QUANT_ROWS)
      mb_launch_pdl(quantize2_kernel<T, MB_QUANT_ROWS>, dim3(grid2), dim3(QUANT_THREADS), 0, stream, x, pairs, uint32_t(k), rbp,
                    input_scale, rowscale, gather, c4, scales, tiled, kc, vec_ok);
    else
      mb_launch_pdl(quantize2_kernel<T, MB_QUANT_SCALED>, dim3(grid2), dim3(QUANT_THREADS), 0, stream, x, pairs, uint32_t(k), rbp,
                    input_scale, rowscale, gather, c4, scales, tiled, kc, vec_ok);
    return;
  }
  const uint32_t blocks = uint32_t(rows * (k / 16));
  const unsigned grid = (blocks + QUANT_THREADS - 1) / QUANT_THREADS;
  const mb_fastdiv rb = mb_fastdiv_make(uint32_t(k / 16));
  uint2* c = reinterpret_cast<uint2*>(codes);
  if (recipe == MB_QUANT_RECIP)
    quantize_kernel<T, MB_QUANT_RECIP><<<grid, QUANT_THREADS, 0, stream>>>(x, blocks, uint32_t(k), rb, input_scale,
                                                                           rowscale, gather, c, scales, tiled, kc, vec_ok);
  else if (recipe == MB_QUANT_ROWS)
    quantize_kernel<T, MB_QUANT_ROWS><<<grid, QUANT_THREADS, 0, stream>>>(x, blocks, uint32_t(k), rb, input_scale,
                                                                          rowscale, gather, c, scales, tiled, kc, vec_ok);
  else
    quantize_kernel<T, MB_QUANT_SCALED><<<grid, QUANT_THREADS, 0, stream>>>(x, blocks, uint32_t(k), rb, input_scale,
                                                                            rowscale, gather, c, scales, tiled, kc, vec_ok);
}

// amax over a tensor with a separate NaN/Inf witness: max drops a NaN operand,
// so non-finite values are recorded apart and the host refuses the tensor.
__global__ void __launch_bounds__(256)
amax_kernel(const __nv_bfloat16* __restrict__ w, size_t len, uint32_t* __restrict__ out2) {
  float m = 0.0f;
  uint32_t bad = 0;
  size_t stride = size_t(gridDim.x) * blockDim.x;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < len; i += stride) {
    float a = fabsf(__bfloat162float(w[i]));
    if (!(a <= 3.4028234663852886e38f)) bad = 1;  // NaN or Inf
    m = fmaxf(m, a);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
    bad |= __shfl_xor_sync(0xFFFFFFFFu, bad, o);
  }
  if ((threadIdx.x & 31) == 0) {
    atomicMax(out2, __float_as_uint(m));  // non-negative floats order as their bit patterns
    if (bad) atomicOr(out2 + 1, 1u);
  }
}

// rowscale[r] = amax(|x[r,:]|)/2688, 1.0 for an all-zero row, NaN for a NaN row.
template <typename T>
__global__ void __launch_bounds__(256)
row_scale_kernel(const T* __restrict__ x, size_t k, const int32_t* __restrict__ gather, float* __restrict__ rowscale,
                 int vec_ok) {
  size_t r = blockIdx.x;
  long long src = gather ? (long long)gather[r] : (long long)r;
  float m = 0.0f;
  uint32_t nan = 0;
  if (src >= 0) {
    // sixteen values (two 128-bit loads) per thread and step; k is a multiple of 16
    for (size_t j = size_t(threadIdx.x) * 16; j < k; j += size_t(blockDim.x) * 16) {
      float v[16];
      const T* p = x + size_t(src) * k + j;
      if (vec_ok) load16(p, v); else load16_scalar(p, v);
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float a = fabsf(v[i]);
        if (a != a) nan = 1;
        m = fmaxf(m, a);
      }
    }
  }
  __shared__ float sm[8];
  __shared__ uint32_t sn[8];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
    nan |= __shfl_xor_sync(0xFFFFFFFFu, nan, o);
  }
  if ((threadIdx.x & 31) == 0) { sm[threadIdx.x >> 5] = m; sn[threadIdx.x >> 5] = nan; }
  __syncthreads();
  if (threadIdx.x == 0) {
    float a = 0.0f;
    uint32_t seen = 0;
    for (int i = 0; i < 8; ++i) { a = fmaxf(a, sm[i]); seen |= sn[i]; }
    float s = 1.0f;
    if (a > 0.0f) s = __fdiv_rn(a, 2688.0f);
    if (seen) s = __int_as_float(0x7FC00000);
    rowscale[r] = s;
  }
}

template <typename O>
__global__ void __launch_bounds__(256)
dequantize_kernel(const uint2* __restrict__ codes, const uint8_t* __restrict__ scales, float scale2, size_t blocks,
                  O* __restrict__ out) {
  size_t blk = size_t(blockIdx.x) * 256 + threadIdx.x;
  if (blk >= blocks) return;
  uint2 c = codes[blk];
  float unit = __fmul_rn(mb_e4m3_to_f32(scales[blk]), scale2);
  float v[16];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    v[i] = __fmul_rn(mb_e2m1_to_f32(c.x >> (4 * i)), unit);
    v[8 + i] = __fmul_rn(mb_e2m1_to_f32(c.y >> (4 * i)), unit);
  }
  // a block's sixteen values leave as 16-byte stores: consecutive threads write consecutive 32 (bf16) or 64 (f32)
  // byte pieces of the plane (out + blk * 16 is 32-byte aligned when `out` is)
  if (sizeof(O) == 2) {
    uint32_t w[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      __nv_bfloat162 p2 = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&p2);
    }
    uint4* o = reinterpret_cast<uint4*>(out + blk * 16);
    o[0] = make_uint4(w[0], w[1], w[2], w[3]);
    o[1] = make_uint4(w[4], w[5], w[6], w[7]);
  } else {
    float4* o = reinterpret_cast<float4*>(out + blk * 16);
#pragma unroll
    for (int i = 0; i < 4; ++i) o[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
  }
}

__global__ void __launch_bounds__(256)
tile_scales_kernel(const uint8_t* __restrict__ in, size_t rows, size_t row_blocks, size_t kchunks,
                   uint8_t* __restrict__ out, int inverse) {
  size_t i = size_t(blockIdx.x) * 256 + threadIdx.x;
  if (i >= rows * row_blocks) return;
  size_t row = i / row_blocks, kb = i % row_blocks;
  size_t off = mb_sf_offset(row, kb, kchunks);
  if (inverse) out[i] = in[off]; else out[off] = in[i];
}

// Row gather of quantized activation planes. A block owns one 128-row tile of the output:
// the source rows go to shared memory once; each warp then copies eight code rows with all
// eight 16-byte loads of a lane in flight before the stores; the tile's scale atoms (512 bytes
// = 128 rows x 4 scales, one word per row) are written whole, thread by consecutive word, from
// the scattered words of the source plane. Pad rows and the K padding of the plane get zeros,
// so the kernel writes every byte of both output planes. A negative source is a zero row.
constexpr int GATHER_THREADS = 128;
constexpr int GATHER_SPLIT = 4;      // blocks per 128-row tile: 32 code rows and every fourth scale atom each

// Four small blocks per tile rather than one large one: a plan of a few hundred tiles then spreads evenly over
// the SMs (with one block per tile some SMs held three tiles and others two).
__global__ void __launch_bounds__(GATHER_THREADS)
gather_planes_kernel(const uint4* __restrict__ codes, const uint8_t* __restrict__ sf, const int32_t* __restrict__ gather,
                     uint32_t rows, uint32_t src_rows, uint32_t code_vecs, uint32_t sf_words, uint32_t kchunks,
                     uint4* __restrict__ out_codes, uint8_t* __restrict__ out_sf, int* __restrict__ flag) {
  __shared__ int32_t s_src[128];
  mb_grid_dependency_sync();
  const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t tile = blockIdx.x / GATHER_SPLIT, sub = blockIdx.x % GATHER_SPLIT;
  const uint32_t row0 = tile * 128;
  {
    const uint32_t row = row0 + threadIdx.x;
    int32_t src = row < rows ? __ldg(gather + row) : -1;
    if (src >= int32_t(src_rows)) {
      atomicCAS(flag, 0, int(row) + 1);
      src = -1;
    }
    s_src[threadIdx.x] = src;
  }
  __syncthreads();
  // codes: warp w copies rows 32 sub + 8 w .. + 7 of the tile
  const uint32_t r0 = sub * 32 + warp * 8;
  int32_t src[8];
#pragma unroll
  for (int r = 0; r < 8; ++r) src[r] = s_src[r0 + r];
  for (uint32_t i = lane; i < code_vecs; i += 32) {
    uint4 v[8];
#pragma unroll
    for (int r = 0; r < 8; ++r)
      v[r] = src[r] < 0 ? make_uint4(0u, 0u, 0u, 0u) : __ldg(codes + size_t(uint32_t(src[r])) * code_vecs + i);
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      const uint32_t row = row0 + r0 + r;
      if (row < rows) out_codes[size_t(row) * code_vecs + i] = v[r];
    }
  }
  // scales: word t of atom kc belongs to tile row (t >> 2) + 32 (t & 3); this block rebuilds atoms sub, sub + 4, ...
  uint32_t* dst = reinterpret_cast<uint32_t*>(out_sf + size_t(tile) * kchunks * 512);
  const uint32_t t = threadIdx.x;
  const int32_t s = s_src[(t >> 2) + 32 * (t & 3)];
  for (uint32_t kc0 = sub; kc0 < kchunks; kc0 += GATHER_SPLIT * 8) {
    uint32_t v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const uint32_t kc = kc0 + u * GATHER_SPLIT;
      v[u] = (kc < sf_words && s >= 0)
                 ? __ldg(reinterpret_cast<const uint32_t*>(sf + mb_sf_offset(uint32_t(s), 4 * kc, kchunks)))
                 : 0u;
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const uint32_t kc = kc0 + u * GATHER_SPLIT;
      if (kc < kchunks) dst[kc * 128 + t] = v[u];
    }
  }
}

}  // namespace

MB_API int mb_nvfp4_gather_rows(mb_ctx* ctx, mb_stream stream_, const uint8_t* codes, const uint8_t* sf_tiled,
                                size_t src_rows, size_t k, const int32_t* gather, size_t rows, uint8_t* out_codes,
                                uint8_t* out_sf_tiled) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  MB_REQUIRE(ctx, ctx && codes && sf_tiled && gather && out_codes && out_sf_tiled, "gather_rows: null argument");
  MB_REQUIRE(ctx, rows > 0 && src_rows > 0 && k > 0 && k % 64 == 0,
             "gather_rows: [%zu <- %zu, %zu] needs k a positive multiple of 64", rows, src_rows, k);
  MB_REQUIRE(ctx, rows <= 0x7FFFFFFFull && src_rows <= 0x7FFFFFFFull && rows * (k / 16) <= 0xFFFFFF00ull,
             "gather_rows: exceeds u32 block indexing");
  MB_REQUIRE(ctx, mb_aligned(codes, 16) && mb_aligned(out_codes, 16) && mb_aligned(sf_tiled, 4) &&
                      mb_aligned(out_sf_tiled, 4), "gather_rows: planes need 16/4-byte alignment");
  const unsigned grid = unsigned((rows + 127) / 128) * GATHER_SPLIT;
  mb_launch_pdl(gather_planes_kernel, dim3(grid), dim3(GATHER_THREADS), 0, stream,
                reinterpret_cast<const uint4*>(codes), sf_tiled, gather, uint32_t(rows), uint32_t(src_rows),
                uint32_t(k / 32), uint32_t(k / 64), uint32_t(mb_sf_kchunks(k)), reinterpret_cast<uint4*>(out_codes),
                out_sf_tiled, ctx->flags_dev + MB_FLAG_PLAN_FAULT);
  MB_LAUNCH_OK(ctx);
  return MB_OK;
}

MB_API size_t mb_nvfp4_sf_bytes(size_t rows, size_t k) { return mb_sf_plane_bytes(rows, k); }

MB_API int mb_nvfp4_quantize_act(mb_ctx* ctx, mb_stream stream_, const void* x, int x_dtype, size_t rows, size_t k,
                                 int recipe, float input_scale, const int32_t* gather, size_t src_rows,
                                 uint8_t* codes, uint8_t* scales, int sf_layout, float* rowscale) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  MB_REQUIRE(ctx, ctx && x && codes && scales, "quantize_act: null argument");
  MB_REQUIRE(ctx, rows > 0 && k > 0 && k % 16 == 0, "quantize_act: [%zu, %zu] needs k a positive multiple of 16", rows, k);
  MB_REQUIRE(ctx, x_dtype == MB_DT_BF16 || x_dtype == MB_DT_F32, "quantize_act: activations are bf16 or f32");
  MB_REQUIRE(ctx, recipe >= MB_QUANT_SCALED && recipe <= MB_QUANT_ROWS, "quantize_act: unknown recipe %d", recipe);
  MB_REQUIRE(ctx, sf_layout == MB_SF_ROWMAJOR || sf_layout == MB_SF_TILED, "quantize_act: unknown scale layout");
  MB_REQUIRE(ctx, rows * (k / 16) <= 0xFFFFFF00ull, "quantize_act: exceeds u32 block indexing");
  MB_REQUIRE(ctx, mb_aligned(codes, 8) && mb_aligned(scales, 4), "quantize_act: outputs need 8/4-byte alignment");
  size_t esz = x_dtype == MB_DT_BF16 ? 2 : 4;
  MB_REQUIRE(ctx, mb_aligned(x, esz == 2 ? 4 : 4), "quantize_act: activation needs 4-byte alignment");
  if (recipe == MB_QUANT_SCALED)
    MB_REQUIRE(ctx, input_scale > 0.0f && input_scale <= 3.4e38f, "quantize_act: input_scale must be finite positive");
  if (recipe == MB_QUANT_ROWS) MB_REQUIRE(ctx, rowscale != nullptr, "quantize_act: the rows recipe writes rowscale");
  if (gather) MB_REQUIRE(ctx, src_rows > 0, "quantize_act: gather needs the source row count");
  int vec_ok = mb_aligned(x, 16) && (k * esz) % 16 == 0;
  if (sf_layout == MB_SF_TILED && (rows % 128 != 0 || k % 256 != 0)) {
    // Scale bytes of the K padding are read by the product that consumes the plane and must decode
    // to a finite value; the bytes of pad rows only make the plane deterministic (their outputs
    // are never stored). A plane without padding is written whole by the kernel.
    MB_CUDA_OK(ctx, cudaMemsetAsync(scales, 0, mb_sf_plane_bytes(rows, k), stream));
  }
  if (recipe == MB_QUANT_ROWS) {
    if (x_dtype == MB_DT_BF16)
      row_scale_kernel<<<unsigned(rows), 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), k, gather, rowscale,
                                                           vec_ok);
    else
      row_scale_kernel<<<unsigned(rows), 256, 0, stream>>>(static_cast<const float*>(x), k, gather, rowscale, vec_ok);
    MB_LAUNCH_OK(ctx);
  }
  if (x_dtype == MB_DT_BF16)
    launch_quantize(stream, recipe, static_cast<const __nv_bfloat16*>(x), rows, k, input_scale, rowscale, gather, codes,
                    scales, sf_layout == MB_SF_TILED, vec_ok);
  else
    launch_quantize(stream, recipe, static_cast<const float*>(x), rows, k, input_scale, rowscale, gather, codes, scales,
                    sf_layout == MB_SF_TILED, vec_ok);
  MB_LAUNCH_OK(ctx);
  return MB_OK;
}

MB_API int mb_nvfp4_quantize_weight(mb_ctx* ctx, mb_stream stream_, const void* w_bf16, size_t n, size_t k,
                                    uint8_t* codes, uint8_t* scales, float* scale2_host_out) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  MB_REQUIRE(ctx, ctx && w_bf16 && codes && scales && scale2_host_out, "quantize_weight: null argument");
  MB_REQUIRE(ctx, n > 0 && k > 0 && k % 32 == 0, "NVFP4 needs contiguous [n, k] with k a multiple of 32, got [%zu, %zu]", n, k);
  MB_REQUIRE(ctx, n * k <= 0xFFFFFFFFull, "NVFP4 weight exceeds u32 indexing");
  uint32_t host[2];
  {
  std::lock_guard<std::mutex> scratch_lock(ctx->scratch_mu);   // the spare words are shared by the context's streams
  uint32_t* scratch = reinterpret_cast<uint32_t*>(ctx->flags_dev + MB_FLAG_COUNT);  // two spare words
  MB_CUDA_OK(ctx, cudaMemsetAsync(scratch, 0, 8, stream));
  size_t len = n * k;
  unsigned grid = unsigned(std::min<size_t>((len + 255) / 256, size_t(ctx->sm_count) * 8));
  amax_kernel<<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(w_bf16), len, scratch);
  MB_LAUNCH_OK(ctx);
  MB_CUDA_OK(ctx, cudaMemcpyAsync(host, scratch, 8, cudaMemcpyDeviceToHost, stream));
  MB_CUDA_OK(ctx, cudaStreamSynchronize(stream));
  }
  if (host[1]) return mb_fail(ctx, MB_ERR_NONFINITE, "NVFP4 source has a non-finite weight");
  float amax;
  memcpy(&amax, &host[0], 4);
  float scale2 = amax > 0.0f ? amax / (6.0f * 448.0f) : 1.0f;
  *scale2_host_out = scale2;
  return mb_nvfp4_quantize_act(ctx, stream_, w_bf16, MB_DT_BF16, n, k, MB_QUANT_SCALED, scale2, nullptr, 0, codes,
                               scales, MB_SF_ROWMAJOR, nullptr);
}

// MXFP4 -> NVFP4 scale relabelling: an E8M0 byte is the power of two 2^(b - 127); E4M3 holds
// 2^-9 .. 2^8 exactly; with the global exponent g = e_max - 8 each block scale is 2^(e - g),
// written for both 16-blocks of the 32-block. Pass 1 finds the byte range and the first NaN.
namespace {

__global__ void __launch_bounds__(256)
e8m0_range_kernel(const uint8_t* __restrict__ scale, size_t n, uint32_t* __restrict__ out3) {
  uint32_t hi = 0, lo_inv = 0, nan_inv = 0;
  const size_t stride = size_t(gridDim.x) * blockDim.x;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    const uint32_t b = scale[i];
    if (b == 0xFFu) nan_inv = max(nan_inv, 0xFFFFFFFFu - uint32_t(i));   // the largest of these is the first index
    else { hi = max(hi, b + 1u); lo_inv = max(lo_inv, 256u - b); }
  }
  hi = __reduce_max_sync(0xFFFFFFFFu, hi);
  lo_inv = __reduce_max_sync(0xFFFFFFFFu, lo_inv);
  nan_inv = __reduce_max_sync(0xFFFFFFFFu, nan_inv);
  if ((threadIdx.x & 31) == 0) {
    atomicMax(out3, hi);
    atomicMax(out3 + 1, lo_inv);
    if (nan_inv) atomicMax(out3 + 2, nan_inv);
  }
}

__global__ void __launch_bounds__(256)
e8m0_relabel_kernel(const uint8_t* __restrict__ scale, size_t n, int g, uint16_t* __restrict__ out) {
  const size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int e = int(scale[i]) - 127 - g;                        // -9 .. 8 by the range check
  const uint32_t b = e >= -6 ? uint32_t(e + 7) << 3 : (1u << (e + 9));   // subnormals 2^-9, 2^-8, 2^-7 = mantissa 1, 2, 4
  out[i] = uint16_t(b | (b << 8));
}

}  // namespace

MB_API int mb_mxfp4_to_nvfp4_scales(mb_ctx* ctx, mb_stream stream_, const uint8_t* e8m0, size_t n,
                                    uint8_t* block_scales, float* global_scale_host_out, int* global_exp_host_out) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  MB_REQUIRE(ctx, ctx && e8m0 && block_scales && global_scale_host_out, "mxfp4 transcode: null argument");
  MB_REQUIRE(ctx, n > 0 && n < 0xFFFFFFFFull, "mxfp4 transcode: empty or oversized scale plane");
  MB_REQUIRE(ctx, mb_aligned(block_scales, 2), "mxfp4 transcode: the NVFP4 scale plane needs 2-byte alignment");
  uint32_t host[3];
  {
  std::lock_guard<std::mutex> scratch_lock(ctx->scratch_mu);   // the spare words are shared by the context's streams
  uint32_t* scratch = reinterpret_cast<uint32_t*>(ctx->flags_dev + MB_FLAG_COUNT);   // spare words
  MB_CUDA_OK(ctx, cudaMemsetAsync(scratch, 0, 12, stream));
  const unsigned grid = unsigned(std::min<size_t>((n + 255) / 256, size_t(ctx->sm_count) * 8));
  e8m0_range_kernel<<<grid, 256, 0, stream>>>(e8m0, n, scratch);
  MB_LAUNCH_OK(ctx);
  MB_CUDA_OK(ctx, cudaMemcpyAsync(host, scratch, 12, cudaMemcpyDeviceToHost, stream));
  MB_CUDA_OK(ctx, cudaStreamSynchronize(stream));
  }
  if (host[2]) return mb_fail(ctx, MB_ERR_NONFINITE, "E8M0 scale[%u] is NaN (0xFF)", 0xFFFFFFFFu - host[2]);
  const int e_max = int(host[0]) - 1 - 127, e_min = 256 - int(host[1]) - 127;
  const int g = e_max - 8;
  if (e_min - g < -9)
    return mb_fail(ctx, MB_ERR_INVALID, "E8M0 exponents span %d octaves (%d..%d); E4M3 holds 18 exactly",
                   e_max - e_min + 1, e_min, e_max);
  if (g < -126 || g > 127) return mb_fail(ctx, MB_ERR_INVALID, "global scale 2^%d is not a normal f32", g);
  e8m0_relabel_kernel<<<unsigned((n + 255) / 256), 256, 0, stream>>>(e8m0, n, g, reinterpret_cast<uint16_t*>(block_scales));
  MB_LAUNCH_OK(ctx);
  const uint32_t bits = uint32_t(g + 127) << 23;
  memcpy(global_scale_host_out, &bits, 4);
  if (global_exp_host_out) *global_exp_host_out = g;
  return MB_OK;
}

MB_API int mb_nvfp4_dequantize(mb_ctx* ctx, mb_stream stream_, const uint8_t* codes, const uint8_t* scales,
                               float scale2, size_t rows, size_t k, void* out, int out_dtype) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  MB_REQUIRE(ctx, ctx && codes && scales && out, "dequantize: null argument");
  MB_REQUIRE(ctx, rows > 0 && k > 0 && k % 16 == 0, "dequantize: k must be a positive multiple of 16");
  MB_REQUIRE(ctx, mb_aligned(codes, 8) && mb_aligned(out, 16), "dequantize: codes need 8-byte and the output 16-byte alignment");
  size_t blocks = rows * k / 16;
  unsigned grid = unsigned((blocks + 255) / 256);
  if (out_dtype == MB_DT_F32)
    dequantize_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<const uint2*>(codes), scales, scale2, blocks,
                                                static_cast<float*>(out));
  else if (out_dtype == MB_DT_BF16)
    dequantize_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<const uint2*>(codes), scales, scale2, blocks,
                                                static_cast<__nv_bfloat16*>(out));
  else
    return mb_fail(ctx, MB_ERR_INVALID, "dequantize: output is bf16 or f32");
  MB_LAUNCH_OK(ctx);
  return MB_OK;
}

static int tile_scales(mb_ctx* ctx, mb_stream stream_, const uint8_t* in, size_t rows, size_t k, uint8_t* out,
                       int inverse) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  MB_REQUIRE(ctx, ctx && in && out, "tile_scales: null argument");
  MB_REQUIRE(ctx, rows > 0 && k > 0 && k % 16 == 0, "tile_scales: k must be a positive multiple of 16");
  if (!inverse) MB_CUDA_OK(ctx, cudaMemsetAsync(out, 0, mb_sf_plane_bytes(rows, k), stream));
  size_t total = rows * (k / 16);
  tile_scales_kernel<<<unsigned((total + 255) / 256), 256, 0, stream>>>(in, rows, k / 16, mb_sf_kchunks(k), out,
                                                                        inverse);
  MB_LAUNCH_OK(ctx);
  return MB_OK;
}

MB_API int mb_nvfp4_tile_scales(mb_ctx* ctx, mb_stream stream, const uint8_t* scales_rowmajor, size_t rows, size_t k,
                                uint8_t* scales_tiled) {
  return tile_scales(ctx, stream, scales_rowmajor, rows, k, scales_tiled, 0);
}
MB_API int mb_nvfp4_untile_scales(mb_ctx* ctx, mb_stream stream, const uint8_t* scales_tiled, size_t rows, size_t k,
                                  uint8_t* scales_rowmajor) {
  return tile_scales(ctx, stream, scales_tiled, rows, k, scales_rowmajor, 1);
}
