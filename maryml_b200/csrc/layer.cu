// Decoder-layer glue with the reference's bf16 rounding points: RMSNorm, residual
// add, SwiGLU, RoPE. HBM-bound elementwise kernels with 128-bit accesses; the norm
// keeps a row in registers between the sum-of-squares pass and the scaling pass.
#include "common.cuh"
#include "quant_block.cuh"

namespace {

__device__ __forceinline__ float bf16r(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
__device__ __forceinline__ void unpack8(const uint4& q, float* v) {
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}
__device__ __forceinline__ uint4 pack8(const float* v) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __nv_bfloat162 t = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    w[i] = *reinterpret_cast<uint32_t*>(&t);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// One CTA of 256 threads per row; width <= 256 * 8 * VEC elements held in registers.
// inv = 1/sqrt(mean(x^2) + eps); y = bf16(bf16(x * inv) * gain).
template <int VEC>
__global__ void __launch_bounds__(256)
rmsnorm_kernel(const uint4* __restrict__ x, const uint4* __restrict__ gain, uint4* __restrict__ y, uint32_t width,
               float eps) {
  const uint32_t row = blockIdx.x, chunks = width / 8;
  const uint4* xr = x + size_t(row) * chunks;
  float v[VEC][8];
  float sum = 0.0f;
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    const uint32_t c = threadIdx.x + i * 256;
    if (c < chunks) {
      unpack8(__ldg(xr + c), v[i]);
#pragma unroll
      for (int j = 0; j < 8; ++j) sum += v[i][j] * v[i][j];
    }
  }
  __shared__ float red[8];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sum;
  __syncthreads();
  float total = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) total += red[i];
  const float inv = 1.0f / sqrtf(total / float(width) + eps);
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    const uint32_t c = threadIdx.x + i * 256;
    if (c < chunks) {
      float g[8], o[8];
      unpack8(__ldg(gain + c), g);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = bf16r(v[i][j] * inv) * g[j];
      y[size_t(row) * chunks + c] = pack8(o);
    }
  }
}

// mode 0: a + b; mode 2: bf16(silu(a)) * b. n8 = elements / 8.
template <int MODE>
__global__ void __launch_bounds__(256)
element_kernel(const uint4* __restrict__ a, const uint4* __restrict__ b, uint4* __restrict__ out, size_t n8) {
  size_t i = size_t(blockIdx.x) * 256 + threadIdx.x;
  if (i >= n8) return;
  float x[8], y[8], o[8];
  unpack8(__ldg(a + i), x);
  unpack8(__ldg(b + i), y);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    if (MODE == 0) o[j] = x[j] + y[j];
    else o[j] = bf16r(__fdiv_rn(x[j], 1.0f + expf(-x[j]))) * y[j];
  }
  out[i] = pack8(o);
}

// out = bf16(a + bf16(b)) with b an f32 partial sum.
__global__ void __launch_bounds__(256)
add_f32_kernel(const uint4* __restrict__ a, const float4* __restrict__ b, uint4* __restrict__ out, size_t n8) {
  mb_grid_dependency_sync();
  size_t i = size_t(blockIdx.x) * 256 + threadIdx.x;
  if (i >= n8) return;
  float x[8], o[8];
  unpack8(__ldg(a + i), x);
  float4 p0 = __ldg(b + 2 * i), p1 = __ldg(b + 2 * i + 1);
  const float y[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
#pragma unroll
  for (int j = 0; j < 8; ++j) o[j] = x[j] + bf16r(y[j]);
  out[i] = pack8(o);
}

// Half-split rotation; cos/sin rounded to bf16, each product rounded to bf16.
// One thread per (row, f) pair: reads x[row, f] and x[row, half + f], writes both.
__global__ void __launch_bounds__(256)
rope_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out, size_t rows, uint32_t heads,
            uint32_t d, uint32_t past, const float* __restrict__ inv_freq) {
  const uint32_t half = d / 2;
  size_t i = size_t(blockIdx.x) * 256 + threadIdx.x;
  if (i >= rows * half) return;
  const size_t row = i / half;
  const uint32_t f = uint32_t(i % half);
  const uint32_t position = past + uint32_t(row / heads);
  const float angle = float(position) * inv_freq[f];
  const float c = bf16r(cosf(angle)), s = bf16r(sinf(angle));
  const float low = __bfloat162float(x[row * d + f]), high = __bfloat162float(x[row * d + half + f]);
  out[row * d + f] = __float2bfloat16_rn(bf16r(low * c) - bf16r(high * s));
  out[row * d + half + f] = __float2bfloat16_rn(bf16r(high * c) + bf16r(low * s));
}

// Residual add, RMSNorm and the W4A4 activation quantizer in one pass over a row:
//   r = bf16(resid + bf16(partial))          (only with a partial; r is stored)
//   y = bf16(bf16(r * inv) * gain)           (the rmsnorm kernel's arithmetic and summation order)
//   codes, scale bytes = divide recipe with a unit global on y.
// Same chunk-to-thread assignment as rmsnorm_kernel, so the bytes equal those of the three
// separate kernels. A 16-value block is two neighbouring threads; four blocks (eight lanes)
// merge their scale bytes into one store of the tiled plane. width % 64 == 0.
template <int VEC>
__global__ void __launch_bounds__(256)
residual_norm_quantize_kernel(const uint4* __restrict__ resid, const float4* __restrict__ partial,
                              const uint4* __restrict__ gain, uint4* __restrict__ resid_out, uint32_t* __restrict__ codes,
                              uint8_t* __restrict__ scales, uint32_t width, float eps, uint32_t kchunks) {
  mb_grid_dependency_sync();
  const uint32_t row = blockIdx.x, chunks = width / 8;
  const uint4* xr = resid + size_t(row) * chunks;
  float v[VEC][8];
  float sum = 0.0f;
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    const uint32_t c = threadIdx.x + i * 256;
    if (c < chunks) {
      unpack8(__ldg(xr + c), v[i]);
      if (partial) {
        const float4* pr = partial + (size_t(row) * chunks + c) * 2;
        const float4 p0 = __ldg(pr), p1 = __ldg(pr + 1);
        const float y[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) v[i][j] = bf16r(v[i][j] + bf16r(y[j]));
        resid_out[size_t(row) * chunks + c] = pack8(v[i]);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) sum += v[i][j] * v[i][j];
    }
  }
  __shared__ float red[8];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sum;
  __syncthreads();
  float total = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) total += red[i];
  const float inv = 1.0f / sqrtf(total / float(width) + eps);
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    const uint32_t c = threadIdx.x + i * 256;
    const bool live = c < chunks;          // uniform over each aligned group of eight lanes
    float o[8];
    float amax = 0.0f;
    if (live) {
      float g[8];
      unpack8(__ldg(gain + c), g);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        o[j] = bf16r(bf16r(v[i][j] * inv) * g[j]);
        amax = fmaxf(amax, fabsf(o[j]));
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = 0.0f;
    }
    const float bamax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
    uint32_t sbyte;
    const float d = quant_divisor_scaled(bamax, 1.0f, sbyte);
    const uint32_t mine = quant_codes8_div(o, d, bamax);
    // scale bytes of the four blocks of this group of eight lanes -> lane 0 of the group
    uint32_t w = sbyte;
    w |= __shfl_down_sync(0xFFFFFFFFu, sbyte, 2) << 8;
    w |= __shfl_down_sync(0xFFFFFFFFu, sbyte, 4) << 16;
    w |= __shfl_down_sync(0xFFFFFFFFu, sbyte, 6) << 24;
    if (live) {
      codes[size_t(row) * chunks + c] = mine;
      if ((threadIdx.x & 7) == 0)
        *reinterpret_cast<uint32_t*>(scales + mb_sf_offset(row, c >> 1, kchunks)) = w;
    }
  }
}

// Rotation of the q and k heads of a stacked [tokens, (hq + 2 hkv) d] projection and the
// cache append in one pass: q goes out contiguous, rotated k and plain v land in the caches
// [batch, capacity, hkv, d] at position past + i of their sequence. The per-element
// arithmetic is rope_kernel's. One thread per eight (f, f + d/2) pairs of ROPE_HEADS heads of a token: the sixteen
// sines and cosines depend on the position and the pair only, so at prompt sizes they are taken once for eight heads
// (the pass was bound by them: 71 us for 8192 tokens x 48 heads against 31 us of memory traffic); at decode sizes
// one head per thread keeps the grid wide and the thread's chain short.
template <uint32_t ROPE_HEADS>
__global__ void __launch_bounds__(256)
rope_append_kernel(const uint4* __restrict__ qkv, uint4* __restrict__ q_out, uint4* __restrict__ k_cache,
                   uint4* __restrict__ v_cache, uint32_t batch, uint32_t t, uint32_t hq, uint32_t hkv, uint32_t d,
                   uint32_t past, uint32_t capacity, const float* __restrict__ inv_freq) {
  mb_grid_dependency_sync();
  const uint32_t groups = d / 16;                      // eight-pair groups per head
  const uint32_t heads = hq + 2 * hkv;
  const uint32_t hgroups = (heads + ROPE_HEADS - 1) / ROPE_HEADS;
  const size_t total = size_t(batch) * t * hgroups * groups;
  const size_t idx = size_t(blockIdx.x) * 256 + threadIdx.x;
  if (idx >= total) return;
  const uint32_t g = uint32_t(idx % groups);
  const uint32_t head0 = uint32_t((idx / groups) % hgroups) * ROPE_HEADS;
  const size_t tok = idx / (size_t(groups) * hgroups);   // b * t + i
  const uint32_t i = uint32_t(tok % t), b = uint32_t(tok / t);
  const uint32_t d8 = d / 8, half8 = d8 / 2;
  const uint32_t n_here = min(ROPE_HEADS, heads - head0);
  // all loads of this thread's heads first
  uint4 lo_q[ROPE_HEADS], hi_q[ROPE_HEADS];
#pragma unroll
  for (uint32_t hh = 0; hh < ROPE_HEADS; ++hh) {
    if (hh < n_here) {
      const uint4* src = qkv + (tok * heads + head0 + hh) * d8;
      lo_q[hh] = __ldg(src + g);
      hi_q[hh] = __ldg(src + half8 + g);
    }
  }
  float c[8], s[8];
  if (head0 < hq + hkv) {                              // at least one rotated head among them
    const float position = float(past + i);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float angle = position * inv_freq[g * 8 + j];
      c[j] = bf16r(cosf(angle));
      s[j] = bf16r(sinf(angle));
    }
  }
#pragma unroll
  for (uint32_t hh = 0; hh < ROPE_HEADS; ++hh) {
    if (hh >= n_here) break;
    const uint32_t head = head0 + hh;
    uint4* dst;
    if (head < hq) dst = q_out + (tok * hq + head) * d8;
    else if (head < hq + hkv) dst = k_cache + ((size_t(b) * capacity + past + i) * hkv + (head - hq)) * d8;
    else dst = v_cache + ((size_t(b) * capacity + past + i) * hkv + (head - hq - hkv)) * d8;
    if (head >= hq + hkv) {
      dst[g] = lo_q[hh];
      dst[half8 + g] = hi_q[hh];
      continue;
    }
    float low[8], high[8], ol[8], oh[8];
    unpack8(lo_q[hh], low);
    unpack8(hi_q[hh], high);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      ol[j] = bf16r(low[j] * c[j]) - bf16r(high[j] * s[j]);
      oh[j] = bf16r(high[j] * c[j]) + bf16r(low[j] * s[j]);
    }
    dst[g] = pack8(ol);
    dst[half8 + g] = pack8(oh);
  }
}


// The Inkling convention (src/models/inkling/resid.rs:272-322): everything in f32 and ONE rounding at the end,
// out = O(x / sqrt(mean(x^2) + eps) * gain) with an f32 gain. The sum of squares follows the reference kernel's
// order exactly: `units` = min(256, next power of two of the width) partial sums, unit u adding elements u,
// u + units, ... in turn (a * a + acc as one fused multiply-add, which is what the run-time compiler the
// reference goes through makes of that expression), then a shared-memory tree that halves the partials. The
// row is staged in shared memory as f32 so that the global loads stay 128-bit while the sums keep that order.
template <typename I, typename O>
__global__ void __launch_bounds__(256)
rmsnorm_inkling_kernel(const I* __restrict__ x, const float* __restrict__ gain, O* __restrict__ out, uint32_t h,
                       float eps, uint32_t units) {
  extern __shared__ float srow[];
  __shared__ float red[256];
  mb_grid_dependency_sync();
  const uint32_t u = threadIdx.x;
  const size_t base = size_t(blockIdx.x) * h;
  if (sizeof(I) == 2) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + base);
    for (uint32_t c = u; c < h / 8; c += 256) unpack8(__ldg(xr + c), srow + c * 8);
  } else {
    const float4* xr = reinterpret_cast<const float4*>(x + base);
    for (uint32_t c = u; c < h / 4; c += 256) *reinterpret_cast<float4*>(srow + c * 4) = __ldg(xr + c);
  }
  __syncthreads();
  float acc = 0.0f;
  if (u < units)
    for (uint32_t i = u; i < h; i += units) acc = __fmaf_rn(srow[i], srow[i], acc);
  red[u] = acc;
  __syncthreads();
  for (uint32_t step = units / 2; step > 0; step /= 2) {
    if (u < step) red[u] = __fadd_rn(red[u], red[u + step]);
    __syncthreads();
  }
  const float denom = __fsqrt_rn(__fadd_rn(__fdiv_rn(red[0], float(h)), eps));
  for (uint32_t j = u; j < h; j += 256) {
    const float r = __fmul_rn(__fdiv_rn(srow[j], denom), __ldg(gain + j));
    if (sizeof(O) == 2) reinterpret_cast<__nv_bfloat16*>(out)[base + j] = __float2bfloat16_rn(r);
    else reinterpret_cast<float*>(out)[base + j] = r;
  }
}


// gate_up_silu (src/models/inkling/fp4gemm.rs:472-507) as the stand-alone pass the reference runs after its
// fused gate/up product: act[r, i] = O(silu(g) * u) in f32, with (g, u) = both[r, 2i], both[r, 2i + 1]
// (interleaved rows of w13) or both[r, i], both[r, inter + i] (halved). Four outputs per thread.
template <typename I, typename O>
__global__ void __launch_bounds__(256)
gate_up_silu_kernel(const I* __restrict__ both, O* __restrict__ act, size_t total4, uint32_t inter, int halved) {
  const size_t q = size_t(blockIdx.x) * 256 + threadIdx.x;
  if (q >= total4) return;
  const size_t idx = q * 4, r = idx / inter;
  const uint32_t i = uint32_t(idx - r * inter);
  const I* row = both + r * 2 * size_t(inter);
  float g[4], u[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    g[j] = float(halved ? row[i + j] : row[2 * (i + j)]);
    u[j] = float(halved ? row[inter + i + j] : row[2 * (i + j) + 1]);
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) act[idx + j] = O(__fmul_rn(__fdiv_rn(g[j], __fadd_rn(1.0f, expf(-g[j]))), u[j]));
}

}  // namespace

MB_API int mb_gate_up_silu(mb_ctx* ctx, mb_stream stream_, const void* both, int in_dtype, size_t rows, size_t inter,
                           int halved, void* act, int out_dtype) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  MB_REQUIRE(ctx, ctx && both && act, "gate_up_silu: null argument");
  MB_REQUIRE(ctx, rows > 0 && inter > 0 && inter % 4 == 0 && inter < (1ull << 30), "gate_up_silu: inter must be a positive multiple of 4, got %zu", inter);
  MB_REQUIRE(ctx, (in_dtype == MB_DT_BF16 || in_dtype == MB_DT_F32) && (out_dtype == MB_DT_BF16 || out_dtype == MB_DT_F32),
             "gate_up_silu: input and output are bf16 or f32");
  const size_t total4 = rows * inter / 4;
  const unsigned grid = unsigned((total4 + 255) / 256);
  const uint32_t it = uint32_t(inter);
  if (in_dtype == MB_DT_F32 && out_dtype == MB_DT_F32)
    gate_up_silu_kernel<<<grid, 256, 0, stream>>>(static_cast<const float*>(both), static_cast<float*>(act), total4, it, halved);
  else if (in_dtype == MB_DT_F32)
    gate_up_silu_kernel<<<grid, 256, 0, stream>>>(static_cast<const float*>(both), static_cast<__nv_bfloat16*>(act), total4, it, halved);
  else if (out_dtype == MB_DT_F32)
    gate_up_silu_kernel<<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(both), static_cast<float*>(act), total4, it, halved);
  else
    gate_up_silu_kernel<<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(both), static_cast<__nv_bfloat16*>(act), total4, it, halved);
  MB_LAUNCH_OK(ctx);
  return MB_OK;
}

MB_API int mb_rmsnorm_inkling(mb_ctx* ctx, mb_stream stream_, const void* x, int x_dtype, const float* gain_f32,
                              size_t rows, size_t width, float eps, void* out, int out_dtype) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  MB_REQUIRE(ctx, ctx && x && gain_f32 && out, "rmsnorm_inkling: null argument");
  MB_REQUIRE(ctx, rows > 0 && rows < (1ull << 31) && width > 0 && width % 8 == 0 && width <= 8192,
             "rmsnorm_inkling: width must be a multiple of 8 up to 8192, got %zu", width);
  MB_REQUIRE(ctx, (x_dtype == MB_DT_BF16 || x_dtype == MB_DT_F32) && (out_dtype == MB_DT_BF16 || out_dtype == MB_DT_F32),
             "rmsnorm_inkling: input and output are bf16 or f32");
  MB_REQUIRE(ctx, mb_aligned(x, 16) && mb_aligned(gain_f32, 4) && mb_aligned(out, 4), "rmsnorm_inkling: alignment");
  uint32_t units = 1;
  while (units < width && units < 256) units *= 2;     // min(256, next power of two)
  const size_t smem = width * sizeof(float);
  const uint32_t h = uint32_t(width);
  const dim3 grid(static_cast<unsigned>(rows));
  if (x_dtype == MB_DT_BF16 && out_dtype == MB_DT_BF16)
    rmsnorm_inkling_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, 256, smem, stream>>>(
        static_cast<const __nv_bfloat16*>(x), gain_f32, static_cast<__nv_bfloat16*>(out), h, eps, units);
  else if (x_dtype == MB_DT_BF16)
    rmsnorm_inkling_kernel<__nv_bfloat16, float><<<grid, 256, smem, stream>>>(
        static_cast<const __nv_bfloat16*>(x), gain_f32, static_cast<float*>(out), h, eps, units);
  else if (out_dtype == MB_DT_BF16)
    rmsnorm_inkling_kernel<float, __nv_bfloat16><<<grid, 256, smem, stream>>>(
        static_cast<const float*>(x), gain_f32, static_cast<__nv_bfloat16*>(out), h, eps, units);
  else
    rmsnorm_inkling_kernel<float, float><<<grid, 256, smem, stream>>>(static_cast<const float*>(x), gain_f32,
                                                                      static_cast<float*>(out), h, eps, units);
  MB_LAUNCH_OK(ctx);
  return MB_OK;
}

MB_API int mb_rmsnorm(mb_ctx* ctx, mb_stream stream_, const void* x, const void* gain, size_t rows, size_t width,
                      float eps, void* out) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  MB_REQUIRE(ctx, ctx && x && gain && out, "rmsnorm: null argument");
  MB_REQUIRE(ctx, rows > 0 && width > 0 && width % 8 == 0 && width <= 256 * 8 * 4,
             "rmsnorm: width must be a multiple of 8 up to 8192, got %zu", width);
  MB_REQUIRE(ctx, mb_aligned(x, 16) && mb_aligned(gain, 16) && mb_aligned(out, 16), "rmsnorm: 16-byte alignment");
  const uint4* xv = static_cast<const uint4*>(x);
  const uint4* gv = static_cast<const uint4*>(gain);
  uint4* ov = static_cast<uint4*>(out);
  if (width <= 2048) rmsnorm_kernel<1><<<unsigned(rows), 256, 0, stream>>>(xv, gv, ov, uint32_t(width), eps);
  else if (width <= 4096) rmsnorm_kernel<2><<<unsigned(rows), 256, 0, stream>>>(xv, gv, ov, uint32_t(width), eps);
  else rmsnorm_kernel<4><<<unsigned(rows), 256, 0, stream>>>(xv, gv, ov, uint32_t(width), eps);
  MB_LAUNCH_OK(ctx);
  return MB_OK;
}

static int element(mb_ctx* ctx, mb_stream stream_, const void* a, const void* b, size_t n, void* out, int mode) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  MB_REQUIRE(ctx, ctx && a && b && out, "element: null argument");
  MB_REQUIRE(ctx, n > 0 && n % 8 == 0, "element: the element count must be a positive multiple of 8");
  MB_REQUIRE(ctx, mb_aligned(a, 16) && mb_aligned(b, 16) && mb_aligned(out, 16), "element: 16-byte alignment");
  size_t n8 = n / 8;
  unsigned grid = unsigned((n8 + 255) / 256);
  if (mode == 0)
    element_kernel<0><<<grid, 256, 0, stream>>>(static_cast<const uint4*>(a), static_cast<const uint4*>(b),
                                                static_cast<uint4*>(out), n8);
  else
    element_kernel<2><<<grid, 256, 0, stream>>>(static_cast<const uint4*>(a), static_cast<const uint4*>(b),
                                                static_cast<uint4*>(out), n8);
  MB_LAUNCH_OK(ctx);
  return MB_OK;
}

MB_API int mb_add(mb_ctx* ctx, mb_stream stream, const void* a, const void* b, size_t n, void* out) {
  return element(ctx, stream, a, b, n, out, 0);
}
MB_API int mb_add_f32(mb_ctx* ctx, mb_stream stream_, const void* a, const float* b, size_t n, void* out) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  MB_REQUIRE(ctx, ctx && a && b && out, "add_f32: null argument");
  MB_REQUIRE(ctx, n > 0 && n % 8 == 0, "add_f32: the element count must be a positive multiple of 8");
  MB_REQUIRE(ctx, mb_aligned(a, 16) && mb_aligned(b, 16) && mb_aligned(out, 16), "add_f32: 16-byte alignment");
  size_t n8 = n / 8;
  MB_CUDA_OK(ctx, mb_launch_pdl(add_f32_kernel, dim3(unsigned((n8 + 255) / 256)), dim3(256), 0, stream,
                                static_cast<const uint4*>(a), reinterpret_cast<const float4*>(b),
                                static_cast<uint4*>(out), n8));
  MB_LAUNCH_OK(ctx);
  return MB_OK;
}
MB_API int mb_swiglu(mb_ctx* ctx, mb_stream stream, const void* gate, const void* up, size_t n, void* out) {
  return element(ctx, stream, gate, up, n, out, 2);
}

MB_API int mb_rope(mb_ctx* ctx, mb_stream stream_, const void* x, size_t tokens, size_t heads, size_t d, size_t past,
                   const float* inv_freq, void* out) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  MB_REQUIRE(ctx, ctx && x && inv_freq && out, "rope: null argument");
  MB_REQUIRE(ctx, tokens > 0 && heads > 0 && d > 0 && d % 2 == 0, "rope: d must be even");
  size_t rows = tokens * heads;
  size_t total = rows * (d / 2);
  rope_kernel<<<unsigned((total + 255) / 256), 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x),
                                                                 static_cast<__nv_bfloat16*>(out), rows,
                                                                 uint32_t(heads), uint32_t(d), uint32_t(past), inv_freq);
  MB_LAUNCH_OK(ctx);
  return MB_OK;
}

MB_API int mb_residual_norm_quantize(mb_ctx* ctx, mb_stream stream_, const void* resid, const float* partial,
                                     const void* gain, size_t rows, size_t width, float eps, void* resid_out,
                                     uint8_t* codes, uint8_t* sf_tiled) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  MB_REQUIRE(ctx, ctx && resid && gain && codes && sf_tiled, "residual_norm_quantize: null argument");
  MB_REQUIRE(ctx, !partial || resid_out, "residual_norm_quantize: a partial sum needs somewhere to put the new residual");
  MB_REQUIRE(ctx, rows > 0 && width > 0 && width % 64 == 0 && width <= 256 * 8 * 4,
             "residual_norm_quantize: width must be a multiple of 64 up to 8192, got %zu", width);
  MB_REQUIRE(ctx, mb_aligned(resid, 16) && mb_aligned(gain, 16) && mb_aligned(partial, 16) && mb_aligned(resid_out, 16) &&
                      mb_aligned(codes, 4) && mb_aligned(sf_tiled, 4),
             "residual_norm_quantize: alignment");
  const uint4* xv = static_cast<const uint4*>(resid);
  const float4* pv = reinterpret_cast<const float4*>(partial);
  const uint4* gv = static_cast<const uint4*>(gain);
  uint4* rv = static_cast<uint4*>(resid_out);
  uint32_t* cv = reinterpret_cast<uint32_t*>(codes);
  const uint32_t kc = uint32_t(mb_sf_kchunks(width));
  const unsigned grid = unsigned(rows);
  // scale bytes of the K padding must decode to a finite value for the product that reads the plane
  if (width % 256 != 0) MB_CUDA_OK(ctx, cudaMemsetAsync(sf_tiled, 0, mb_sf_plane_bytes(rows, width), stream));
  auto kern = width <= 2048 ? residual_norm_quantize_kernel<1>
              : width <= 4096 ? residual_norm_quantize_kernel<2> : residual_norm_quantize_kernel<4>;
  MB_CUDA_OK(ctx, mb_launch_pdl(kern, dim3(grid), dim3(256), 0, stream, xv, pv, gv, rv, cv, sf_tiled, uint32_t(width), eps, kc));
  MB_LAUNCH_OK(ctx);
  return MB_OK;
}

MB_API int mb_rope_append(mb_ctx* ctx, mb_stream stream_, const void* qkv, size_t batch, size_t t, size_t hq,
                          size_t hkv, size_t d, size_t past, const float* inv_freq, void* q_out, void* k_cache,
                          void* v_cache, size_t capacity) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  MB_REQUIRE(ctx, ctx && qkv && inv_freq && q_out && k_cache && v_cache, "rope_append: null argument");
  MB_REQUIRE(ctx, batch > 0 && t > 0 && hq > 0 && hkv > 0 && d > 0 && d % 16 == 0, "rope_append: d must be a multiple of 16");
  MB_REQUIRE(ctx, past + t <= capacity, "rope_append: positions [%zu, %zu) exceed the cache capacity %zu", past, past + t,
             capacity);
  MB_REQUIRE(ctx, mb_aligned(qkv, 16) && mb_aligned(q_out, 16) && mb_aligned(k_cache, 16) && mb_aligned(v_cache, 16),
             "rope_append: 16-byte alignment");
  const bool prompt = batch * t >= 1024;           // enough tokens to fill the device with eight heads per thread
  const size_t hpt = prompt ? 8 : 1;
  const size_t total = batch * t * ((hq + 2 * hkv + hpt - 1) / hpt) * (d / 16);
  MB_REQUIRE(ctx, total < (1ull << 40) && batch * capacity < (1ull << 32) && past + t < (1ull << 31),
             "rope_append: extent too large");
  auto kern = prompt ? rope_append_kernel<8> : rope_append_kernel<1>;
  MB_CUDA_OK(ctx, mb_launch_pdl(kern, dim3(unsigned((total + 255) / 256)), dim3(256), 0, stream,
                                static_cast<const uint4*>(qkv), static_cast<uint4*>(q_out), static_cast<uint4*>(k_cache),
                                static_cast<uint4*>(v_cache), uint32_t(batch), uint32_t(t), uint32_t(hq), uint32_t(hkv),
                                uint32_t(d), uint32_t(past), uint32_t(capacity), inv_freq));
  MB_LAUNCH_OK(ctx);
  return MB_OK;
}
