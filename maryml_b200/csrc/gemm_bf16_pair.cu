// BF16 x BF16 prompt product on CTA pairs for sm_100a: out[m, n] = (sum_k a[m, k] * b[n, k]) * alpha, f32
// accumulation (bf16_gemm_launch, src/models/inkling/bf16gemm.rs). The single-CTA kernel of gemm_tc5.cu moves 128
// rows of A and 256 rows of B into every SM per 64-element K step; here a pair of CTAs (cta_group::2, cluster of 2)
// owns a 256 x 256 tile, each CTA loads its own 128 rows of A and its own half of the B tile (128 rows), and the
// leader issues one 256 x 256 x 16 tcgen05.mma per 32 bytes of K for both tensor cores: 32 KB per SM and K step
// instead of 48 KB, and a shared-memory port that carries 48 KB of operand reads per 512-cycle K step.
//
//   warp 0      producer (both CTAs): TMA tiles into a 6-stage ring of 32 KB; the bytes of both CTAs are counted
//               on the leader's barrier (cp.async.bulk.tensor ... cta_group::2). No load is multicast.
//   warp 1      MMA issuer (leader only): four MMAs per stage, tcgen05.commit (multicast to both CTAs' barriers)
//               frees the stage; two full 256-column accumulators in TMEM (512 columns, none shared: there are
//               no scale columns), so the next tile's MMAs start while the epilogue drains the other buffer.
//   warps 2-17  epilogue (both CTAs): four warps per TMEM lane quadrant, two 32-column chunks each;
//               tcgen05.ld, times alpha, one cast, coalesced stores through a shared-memory patch.
//
// Tile order: row-pair groups as in the NVFP4 pair kernel (a group's A rows stay in L2 while every column tile
// passes). Every mbarrier wait is bounded. Taken by mb_bf16_gemm for n % 256 == 0, k % 64 == 0 and at least 74 tiles.
#include "common.cuh"
#include "tc5.cuh"

namespace {

using namespace tc5;

constexpr int EPI_WARPS = 16;
constexpr int THREADS = 32 * (2 + EPI_WARPS);
constexpr int BN = 256;
constexpr int A_BYTES = 128 * 128;
constexpr int B_BYTES = 128 * 128;                   // this CTA's half of the B tile
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int STAGES = 6;
constexpr int BAR_BYTES = 256;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + BAR_BYTES + EPI_WARPS * 512;
constexpr int TMEM_COLS = 512;

struct PairParams {
  CUtensorMap tmap_a;        // [m, k] bf16, box 64 x 128, 128-byte swizzle
  CUtensorMap tmap_b;        // [n, k] bf16, box 64 x 128
  void* out;
  int* flags;
  float alpha;
  uint32_t m, n, k_steps, m_pairs, n_tiles, raster_group;
  int out_dtype;
};

// Row pairs in groups of `group`: inside a group the row pair runs fastest and the column tile slowest.
__device__ __forceinline__ void pair_tile(uint32_t tile, uint32_t m_pairs, uint32_t n_tiles, uint32_t group, uint32_t& mp,
                                          uint32_t& nt) {
  const uint32_t per_group = group * n_tiles;
  const uint32_t g = tile / per_group, r = tile - g * per_group;
  const uint32_t g0 = g * group;
  const uint32_t gsz = min(group, m_pairs - g0);
  nt = r / gsz;
  mp = g0 + (r - nt * gsz);
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// 256 x N x 16 MMA over a CTA pair: each CTA supplies 128 rows of A and N / 2 rows of B.
__device__ __forceinline__ void mma_f16_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// bf16 x bf16 -> f32, both operands K-major, M = 256 over the pair.
__host__ __device__ constexpr uint32_t idesc_bf16_pair(uint32_t n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((256u >> 4) << 24);
}

// Warp-level transpose through a 512-byte shared-memory patch so that global stores are coalesced: lane l holds
// two 16-byte units of ITS row (32 rows x 32 bytes); each half of the warp parks its 16 rows in the patch and the
// whole warp stores them, one instruction writing 16 rows x 32 contiguous bytes.
__device__ __forceinline__ void store_rows(uint8_t* patch, uint32_t lane, const uint4& u0, const uint4& u1, uint8_t* gbase,
                                           size_t row_stride_bytes, uint32_t rows_valid) {
  const uint32_t lr = lane & 15u, swz_w = (lr >> 2) & 1u;
  const uint32_t rr = lane >> 1, u = lane & 1u, swz_r = (rr >> 2) & 1u;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    if ((lane >> 4) == uint32_t(i)) {
      *reinterpret_cast<uint4*>(patch + lr * 32 + ((0u ^ swz_w) * 16)) = u0;
      *reinterpret_cast<uint4*>(patch + lr * 32 + ((1u ^ swz_w) * 16)) = u1;
    }
    __syncwarp();
    const uint4 v = *reinterpret_cast<const uint4*>(patch + rr * 32 + ((u ^ swz_r) * 16));
    const uint32_t r = i * 16 + rr;
    if (r < rows_valid) *reinterpret_cast<uint4*>(gbase + size_t(r) * row_stride_bytes + u * 16) = v;
    __syncwarp();
  }
}

// 32 accumulator columns of this lane's row -> alpha, cast, stores.
__device__ __forceinline__ void store_chunk(const PairParams& p, const uint32_t* r, uint32_t col0, uint32_t row0,
                                            uint32_t rows_valid, uint8_t* patch, uint32_t lane) {
  float v[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * p.alpha;
  if (p.out_dtype == MB_DT_BF16) {
    uint4 units[4];
#pragma unroll
    for (int g = 0; g < 4; ++g)
      units[g] = make_uint4(pack_bf16x2(v[8 * g], v[8 * g + 1]), pack_bf16x2(v[8 * g + 2], v[8 * g + 3]),
                            pack_bf16x2(v[8 * g + 4], v[8 * g + 5]), pack_bf16x2(v[8 * g + 6], v[8 * g + 7]));
    uint8_t* g8 = static_cast<uint8_t*>(p.out) + (size_t(row0) * p.n + col0) * 2;
    store_rows(patch, lane, units[0], units[1], g8, size_t(p.n) * 2, rows_valid);
    store_rows(patch, lane, units[2], units[3], g8 + 32, size_t(p.n) * 2, rows_valid);
  } else {
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      uint4 units[4];
#pragma unroll
      for (int g = 0; g < 4; ++g)
        units[g] = make_uint4(__float_as_uint(v[16 * hh + 4 * g]), __float_as_uint(v[16 * hh + 4 * g + 1]),
                              __float_as_uint(v[16 * hh + 4 * g + 2]), __float_as_uint(v[16 * hh + 4 * g + 3]));
      uint8_t* g8 = static_cast<uint8_t*>(p.out) + (size_t(row0) * p.n + col0 + 16 * hh) * 4;
      store_rows(patch, lane, units[0], units[1], g8, size_t(p.n) * 4, rows_valid);
      store_rows(patch, lane, units[2], units[3], g8 + 32, size_t(p.n) * 4, rows_valid);
    }
  }
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
gemm_bf16_pair_kernel(const __grid_constant__ PairParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + STAGES * STAGE_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto acc_full_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + b); };
  auto acc_free_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + 2 + b); };   // used on the leader only
  const uint32_t drain_bar = bar_base + 8u * (2 * STAGES + 4);
  constexpr int N_BARS = 2 * STAGES + 5;
  static_assert(8 * N_BARS + 8 <= BAR_BYTES, "barrier area");
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(smem_gen + STAGES * STAGE_BYTES + 8 * N_BARS);
  volatile int* abort_smem = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);

  const int warp = __shfl_sync(0xFFFFFFFFu, int(threadIdx.x >> 5), 0);
  const uint32_t lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  int* tflag = p.flags ? p.flags + MB_FLAG_WAIT_TIMEOUT : nullptr;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full_bar(b), 1);
      mbar_init(acc_free_bar(b), 2 * EPI_WARPS);       // one arrival per epilogue warp of both CTAs
    }
    mbar_init(drain_bar, 1);
    *abort_smem = 0;
    fence_barrier_init();
    tma_prefetch_desc(&p.tmap_a);
    tma_prefetch_desc(&p.tmap_b);
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_ptr_smem), TMEM_COLS);
    tmem_relinquish_pair();
  }
  fence_before_sync();
  __syncthreads();
  cluster_sync_all();                  // the peer's barriers exist before anything is signalled on them
  fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr_smem;

  const uint32_t total_tiles = p.m_pairs * p.n_tiles;
  const uint32_t pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;

  if (warp == 0) {
    // ------------------------------ producer (both CTAs) --------------------------
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (uint32_t tile = pair; ok && tile < total_tiles; tile += n_pairs) {
      uint32_t mp, nt;
      pair_tile(tile, p.m_pairs, p.n_tiles, p.raster_group, mp, nt);
      const uint32_t mt = mp * 2 + rank;                         // this CTA's 128-row tile of A
      for (uint32_t ks = 0; ks < p.k_steps; ++ks) {
        if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_smem, tflag, 41)) { ok = false; break; }
        const uint32_t sa = smem_base + stage * STAGE_BYTES;
        if (elect_one()) {
          // all bytes of both CTAs are counted on the leader's barrier
          const uint32_t fb = map_to_cta(full_bar(stage), 0);
          if (leader) mbar_arrive_expect_tx(full_bar(stage), 2 * STAGE_BYTES);
          tma_load_2d_pair(sa, &p.tmap_a, int(ks * 64), int(mt * 128), fb);
          tma_load_2d_pair(sa + A_BYTES, &p.tmap_b, int(ks * 64), int(nt * BN + rank * 128), fb);
        }
        __syncwarp();
        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader CTA only) ------------------
    if (leader) {
      int stage = 0;
      uint32_t phase = 0;
      const uint32_t idesc = idesc_bf16_pair(BN);
      uint32_t it = 0;
      bool ok = true;
      for (uint32_t tile = pair; ok && tile < total_tiles; tile += n_pairs, ++it) {
        const uint32_t buf = it & 1u;
        // the epilogue warps of both CTAs have read the tile before last out of this buffer
        if (!mbar_wait_cluster(acc_free_bar(buf), ((it >> 1) & 1u) ^ 1u, abort_smem, tflag, 42)) { ok = false; break; }
        fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (uint32_t ks = 0; ks < p.k_steps; ++ks) {
          if (!mbar_wait_cluster(full_bar(stage), phase, abort_smem, tflag, 43)) { ok = false; break; }
          fence_after_sync();
          const uint32_t sa = smem_base + stage * STAGE_BYTES;
          if (elect_one()) {
            const uint64_t adesc = make_kmajor_sw128_desc(sa), bdesc = make_kmajor_sw128_desc(sa + A_BYTES);
#pragma unroll
            for (int j = 0; j < 4; ++j) mma_f16_pair(d_tmem, adesc + 2 * j, bdesc + 2 * j, idesc, (ks | uint32_t(j)) != 0u);
            umma_commit_pair(empty_bar(stage), 3);                 // frees the stage in both CTAs
            if (ks + 1 == p.k_steps) umma_commit_pair(acc_full_bar(buf), 3);
          }
          __syncwarp();
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        if (elect_one()) umma_commit(drain_bar);
        __syncwarp();
        const long long t0 = clock64();
        while (!mbar_try_wait(drain_bar, 0u) && clock64() - t0 < WAIT_LIMIT_CYCLES) {}
      }
    }
  } else {
    // ------------------------------ epilogue (both CTAs) --------------------------
    const uint32_t quad = uint32_t(warp) & 3u;
    const uint32_t ew = uint32_t(warp) - 2u, part = ew >> 2;        // part 0..3: chunks 2 part, 2 part + 1 of eight
    uint8_t* patch = smem_gen + STAGES * STAGE_BYTES + BAR_BYTES + ew * 512;
    uint32_t it = 0;
    for (uint32_t tile = pair; tile < total_tiles; tile += n_pairs, ++it) {
      uint32_t mp, nt;
      pair_tile(tile, p.m_pairs, p.n_tiles, p.raster_group, mp, nt);
      const uint32_t buf = it & 1u;
      const uint32_t row0 = (mp * 2 + rank) * 128 + quad * 32u;
      const uint32_t rows_valid = row0 < p.m ? min(32u, p.m - row0) : 0u;
      if (!mbar_wait_cluster(acc_full_bar(buf), (it >> 1) & 1u, abort_smem, tflag, 44)) break;
      fence_after_sync();
      const uint32_t t_acc = tmem_base + ((quad * 32u) << 16) + buf * BN + part * 64;
      uint32_t r0[32], r1[32];
      tmem_ld_x32(t_acc, r0);
      tmem_ld_x32(t_acc + 32, r1);
      tmem_ld_wait();
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(acc_free_bar(buf), 0));   // this warp is done with the buffer
      store_chunk(p, r0, nt * BN + part * 64, row0, rows_valid, patch, lane);
      store_chunk(p, r1, nt * BN + part * 64 + 32, row0, rows_valid, patch, lane);
    }
  }

  // ------------------------------ teardown ----------------------------------------
  fence_before_sync();
  __syncthreads();
  cluster_sync_all();                  // neither CTA leaves while the peer may still touch it
  if (warp == 1) {
    fence_after_sync();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int encode_rows(mb_ctx* ctx, CUtensorMap* tm, const void* base, size_t rows, size_t k) {
  if (!ctx->encode_tiled) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    MB_CUDA_OK(ctx, cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q));
    if (!sym || q != cudaDriverEntryPointSuccess)
      return mb_fail(ctx, MB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    ctx->encode_tiled = sym;
  }
  EncodeTiledFn enc = reinterpret_cast<EncodeTiledFn>(ctx->encode_tiled);
  cuuint64_t dims[2] = {k, rows};
  cuuint64_t strides[1] = {k * 2};
  cuuint32_t box[2] = {64u, 128u}, estr[2] = {1, 1};
  CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return mb_fail(ctx, MB_ERR_CUDA, "cuTensorMapEncodeTiled (bf16 pair product) failed with %d", int(r));
  return MB_OK;
}

}  // namespace

// Whether the pair kernel takes this product (mb_bf16_gemm asks).
// Products with fewer 256 x 256 tiles than the device has CTA pairs stay on the single-CTA kernel, whose 128-row
// tiles fill more SMs.
bool mb_bf16_pair_takes(size_t m, size_t n, size_t k) {
  return m >= 256 && n % 256 == 0 && k % 64 == 0 && ((m + 255) / 256) * (n / 256) >= 74;
}

int mb_bf16_pair_launch(mb_ctx* ctx, cudaStream_t stream, const void* a, const void* b, float alpha, size_t m, size_t n,
                        size_t k, void* out, int out_dtype) {
  PairParams p;
  memset(&p, 0, sizeof p);
  int rc = encode_rows(ctx, &p.tmap_a, a, m, k);
  if (rc) return rc;
  rc = encode_rows(ctx, &p.tmap_b, b, n, k);
  if (rc) return rc;
  p.out = out; p.flags = ctx->flags_dev; p.alpha = alpha;
  p.m = uint32_t(m); p.n = uint32_t(n); p.k_steps = uint32_t(k / 64);
  p.m_pairs = uint32_t((m + 255) / 256); p.n_tiles = uint32_t(n / BN);
  p.out_dtype = out_dtype;
  // a group's A rows (256 x k x 2 bytes per row pair) stay within about half of L2 while all column tiles pass: the
  // weights are read once per group, so larger groups mean fewer passes over them
  const double a_pair = 256.0 * double(k) * 2.0;
  const uint32_t gmax = std::max<uint32_t>(1u, uint32_t(64e6 / a_pair));
  const uint32_t ngroups = (p.m_pairs + gmax - 1) / gmax;
  p.raster_group = (p.m_pairs + ngroups - 1) / ngroups;
  if (!mb_once(ctx, MB_ONCE_GEMM_BF16_PAIR)) {
    MB_CUDA_OK(ctx, cudaFuncSetAttribute(gemm_bf16_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    mb_once_done(ctx, MB_ONCE_GEMM_BF16_PAIR);
  }
  // as many pairs as the device holds at once (the NVFP4 pair kernel asked the driver; one CTA per SM either way)
  uint32_t pairs = ctx->pair_clusters > 0 ? uint32_t(ctx->pair_clusters) : uint32_t(ctx->sm_count / 2);
  if (ctx->sm_limit > 0) pairs = std::min<uint32_t>(pairs, uint32_t(std::max(1, ctx->sm_limit / 2)));
  pairs = std::min<uint32_t>(pairs, p.m_pairs * p.n_tiles);
  gemm_bf16_pair_kernel<<<pairs * 2, THREADS, SMEM_BYTES, stream>>>(p);
  MB_LAUNCH_OK(ctx);
  return MB_OK;
}
