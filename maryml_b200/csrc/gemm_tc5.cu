// Tensor-core GEMMs for sm_100a: out[m, n] = sum_k a[m, k] * b[n, k] (both operands
// K-major), as one persistent, warp-specialised kernel:
//
//   warp 0   TMA producer: per 128-byte K step, the A tile (128 rows) and the B tile
//            (BN rows) land in 128B-swizzled shared memory; for NVFP4 the tiled
//            scale atoms of both operands come with them (plain bulk copies).
//   warp 1   MMA issuer: tcgen05.mma (kind::mxf4nvf4 block-scaled, or kind::f16)
//            with the accumulator in tensor memory; scale atoms are copied
//            shared -> TMEM by tcgen05.cp right before the MMAs that read them.
//   warps 2-17 epilogue: tcgen05.ld the finished accumulator, scale, convert, store;
//            four warps per TMEM lane quadrant, each taking a quarter of the columns.
//
// Two accumulators alternate so that the epilogue of tile i overlaps the MMAs of
// tile i+1. TMEM has 512 columns; the NVFP4 kernel also keeps scale factors there,
// so with BN = 256 the two accumulators share 64 columns: the epilogue drains those
// first and releases them to the next tile's MMAs.
//
// NVFP4 algorithmic work per tile: 2*128*BN*K flop; bytes from L2: (128+BN)*K*(1/2+1/16).
// Every mbarrier wait is bounded (tc5::mbar_wait).
#include "common.cuh"
#include "quant_block.cuh"
#include "tc5.cuh"

namespace {

using namespace tc5;

enum { KIND_NVF4 = 0, KIND_BF16 = 1 };

struct GemmParams {
  CUtensorMap tmap_a;
  CUtensorMap tmap_b;
  const uint8_t* sfa;         // tiled scale plane of A (NVFP4)
  const uint8_t* sfb;         // tiled scale plane(s) of B
  void* out;
  const float* rowscale;      // [m] or null
  const float* alpha_vec;     // [experts] or null
  const int32_t* tile_expert; // grouped: expert of each 128-row tile
  const int32_t* n_mtiles_dev;// grouped: tiles in use (device word)
  const int32_t* row_tok;     // grouped, optional: token of each stacked row, negative = pad row (not stored)
  int* flags;
  float alpha;
  uint32_t m, n, k_steps;     // k_steps: 128-byte K steps
  uint32_t m_tiles, n_tiles;
  uint32_t sf_kchunks;        // scale atoms along K per 128-row tile
  uint32_t b_rows_per_expert; // grouped: n
  uint64_t sfb_expert_stride; // grouped: bytes of one expert's tiled scale plane
  uint32_t ldo;               // output row stride in elements
  int out_dtype;
  int epilogue;
  // MB_EPI_SCATTER: f32 partial tiles go straight into the owning rank's exchange memory.
  float* scatter_base[8];     // recv area (this step's half) of every rank, peer-mapped
  uint32_t scatter_world, scatter_rank, scatter_nw;   // nw = n / world columns per owner
  uint32_t scatter_tmax;      // rows of one source slot
  // split-K (few output tiles, long K): tile index carries a K slice; partial sums go to a workspace
  uint32_t splits, ks_per_split;
  // tile order: 0 = row tiles fastest (dense), 1 = column tiles fastest (grouped: the CTAs that run together share a
  // row tile of activations and the column tiles of one expert, so both operands come from DRAM once)
  uint32_t n_fastest;
  // stacked projections / fused output quantization
  const float* colscale;      // [n] per-column factor or null
  uint8_t* out_sf;            // tiled scale plane of the quantized output
  uint32_t out_sf_kchunks;
  int silu_rounded;           // SwiGLU epilogue: round silu(gate) to bf16 before the product
  int quant;                  // SwiGLU epilogue: 0 bf16 out, 1 NVFP4 (reciprocal recipe), 2 NVFP4 (divide recipe, unit global)
  int cluster_splitk;         // the `splits` K slices of a tile run as one cluster and meet in distributed shared memory
};

constexpr int MB_EPI_SCATTER = 2;   // internal: used by mb_nvfp4_gemm_w4a4_scatter only

constexpr int EPI_WARPS_ = 16;      // four epilogue warps per TMEM lane quadrant

template <int KIND, int BN>
struct Cfg {
  static constexpr int BM = 128;
  static constexpr int A_BYTES = BM * 128;
  static constexpr int B_BYTES = BN * 128;
  static constexpr int SFA_BYTES = KIND == KIND_NVF4 ? 2048 : 0;
  static constexpr int SFB_BYTES = KIND == KIND_NVF4 ? (BN / 128) * 2048 : 0;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES;
  static constexpr int STAGES = (KIND == KIND_NVF4) ? (BN == 256 ? 4 : 6) : (BN == 256 ? 4 : 6);
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment*/ + 256 /*barriers*/ + EPI_WARPS_ * 512 /*store patches*/;
  // TMEM columns
  static constexpr bool OVERLAP = (KIND == KIND_NVF4 && BN == 256);
  static constexpr int ACC0 = 0;
  static constexpr int ACC1 = OVERLAP ? 192 : BN;
  static constexpr int SFA_COL = OVERLAP ? 448 : 2 * BN;   // 16 columns
  static constexpr int SFB_COL = SFA_COL + 16;             // 4 * BN/32 columns
  static constexpr int TMEM_COLS = 512;
  static_assert(KIND == KIND_BF16 || SFB_COL + 4 * (BN / 32) <= 512, "TMEM budget");
  static_assert(KIND == KIND_NVF4 || 2 * BN <= 512, "TMEM budget");
};

// Development aid, compiled in only with -DMB_GEMM_PROFILE: cycles each role of the single-CTA kernel spends
// waiting, per CTA. Slots: 0 producer on a free stage, 1 MMA on a free accumulator, 2 MMA on loaded operands,
// 3 first epilogue warp on a finished accumulator, 4 that warp's work, 5 whole kernel, 6 tiles.
#ifdef MB_GEMM_PROFILE
__device__ unsigned long long g_gemm_prof[160 * 8];
__device__ int g_gemm_dbg;
#define PROF_T0() const long long prof_t0_ = clock64()
#define PROF_ADD(slot) do { if ((threadIdx.x & 31) == 0) atomicAdd(&g_gemm_prof[blockIdx.x * 8 + (slot)], (unsigned long long)(clock64() - prof_t0_)); } while (0)
#else
#define PROF_T0() do {} while (0)
#define PROF_ADD(slot) do {} while (0)
#endif

// Producer warp, MMA warp, sixteen epilogue warps. The epilogue is a chain of dependent conversions,
// special-function ops and shared-memory round trips; four warps per scheduler hide those latencies where two
// left the issue slots three quarters empty (measured: the epilogue, not the tensor pipe, bounded short-K tiles).
constexpr int EPI_WARPS = EPI_WARPS_;
constexpr int NUM_THREADS = 64 + 32 * EPI_WARPS;
constexpr int EPI_THREADS = 32 * EPI_WARPS;

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}


// Warp-level transpose through a 512-byte shared-memory patch so that global stores are
// coalesced: on entry lane l holds two 16-byte units of ITS row (32 rows x 32 bytes); each
// half of the warp in turn parks its 16 rows in the patch and the whole warp stores them,
// one instruction writing 16 rows x 32 contiguous bytes (whole sectors). The XOR on the unit
// index keeps the 128-bit shared stores and loads conflict free.
__device__ __forceinline__ void stage_and_store(uint8_t* patch, uint32_t lane, const uint4& u0, const uint4& u1,
                                                uint8_t* gbase, size_t row_stride_bytes, uint32_t rows_valid,
                                                uint32_t units_valid) {
#ifdef MB_GEMM_PROFILE
  const int dbg = g_gemm_dbg;
  if (dbg & 2) { if ((u0.x ^ u1.y) == 0x12345678u && rows_valid == 77u) *reinterpret_cast<uint4*>(gbase) = u0; return; }
#endif
  const uint32_t lr = lane & 15u;
  const uint32_t swz_w = (lr >> 2) & 1u;
  const uint32_t rr = lane >> 1, u = lane & 1u;          // the row (of 16) and unit this lane stores
  const uint32_t swz_r = (rr >> 2) & 1u;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    if ((lane >> 4) == uint32_t(i)) {
      *reinterpret_cast<uint4*>(patch + lr * 32 + ((0u ^ swz_w) * 16)) = u0;
      *reinterpret_cast<uint4*>(patch + lr * 32 + ((1u ^ swz_w) * 16)) = u1;
    }
    __syncwarp();
    const uint4 v = *reinterpret_cast<const uint4*>(patch + rr * 32 + ((u ^ swz_r) * 16));
    const uint32_t r = i * 16 + rr;
#ifdef MB_GEMM_PROFILE
    if (dbg & 1) { if (v.x == 0x12345678u && rows_valid == 77u) *reinterpret_cast<uint4*>(gbase) = v; __syncwarp(); continue; }
#endif
    if (r < rows_valid && u < units_valid)
      *reinterpret_cast<uint4*>(gbase + size_t(r) * row_stride_bytes + u * 16) = v;
    __syncwarp();
  }
}

// One 32-column chunk of one warp's 32 accumulator rows: scale, convert, transpose, store.
__device__ __forceinline__ void epilogue_chunk(const GemmParams& p, const uint32_t* r, uint32_t col0, uint32_t row0,
                                               uint32_t rows_valid, float scale, uint8_t* patch, uint32_t lane) {
      if (col0 >= p.n) return;       // warp-uniform
      // acc * alpha [* rowscale], and for stacked projections * the column's own global scale
      // (the entry point keeps alpha at 1 there, so the product is rounded once)
      float v[32];
      if (p.colscale) {
        const float4* cs = reinterpret_cast<const float4*>(p.colscale + col0);
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          const float4 c = __ldg(cs + g);
          v[4 * g + 0] = __uint_as_float(r[4 * g + 0]) * scale * c.x;
          v[4 * g + 1] = __uint_as_float(r[4 * g + 1]) * scale * c.y;
          v[4 * g + 2] = __uint_as_float(r[4 * g + 2]) * scale * c.z;
          v[4 * g + 3] = __uint_as_float(r[4 * g + 3]) * scale * c.w;
        }
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * scale;
      }
      if (p.epilogue == MB_EPI_SCATTER) {
        // Reduce-scatter by peer stores: the 32 columns belong to one owner rank; this rank's
        // f32 partial lands in slot [rank] of the owner's receive area while the next tile's
        // MMAs run. Two passes of 16 columns through the patch, as for any f32 output.
        const uint32_t owner = col0 / p.scatter_nw, c_in = col0 - owner * p.scatter_nw;
        float* dst = p.scatter_base[owner] + (size_t(p.scatter_rank) * p.scatter_tmax + row0) * p.scatter_nw + c_in;
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          uint4 units[4];
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            units[g].x = __float_as_uint(v[16 * hh + 4 * g + 0]);
            units[g].y = __float_as_uint(v[16 * hh + 4 * g + 1]);
            units[g].z = __float_as_uint(v[16 * hh + 4 * g + 2]);
            units[g].w = __float_as_uint(v[16 * hh + 4 * g + 3]);
          }
          uint8_t* g8 = reinterpret_cast<uint8_t*>(dst + 16 * hh);
          stage_and_store(patch, lane, units[0], units[1], g8, size_t(p.scatter_nw) * 4, rows_valid, 2u);
          stage_and_store(patch, lane, units[2], units[3], g8 + 32, size_t(p.scatter_nw) * 4, rows_valid, 2u);
        }
        return;
      }
      if (p.epilogue == MB_EPI_SWIGLU_INTERLEAVED) {
        // (gate, up) pairs -> bf16(silu(bf16 gate) * bf16 up); 16 outputs per row = one NVFP4 block.
        float o[16];
#pragma unroll
        for (int i = 0; i < 16; i += 2) {
          // packed conversions (one instruction per pair) instead of scalar ones, which share the
          // special-function unit with the exponential and the reciprocal
          const uint32_t gu0 = pack_bf16x2(v[2 * i], v[2 * i + 1]), gu1 = pack_bf16x2(v[2 * i + 2], v[2 * i + 3]);
          const float g0 = __uint_as_float(gu0 << 16), u0 = __uint_as_float(gu0 & 0xFFFF0000u);
          const float g1 = __uint_as_float(gu1 << 16), u1 = __uint_as_float(gu1 & 0xFFFF0000u);
          float t0, t1;
          if (p.silu_rounded) {   // the dense layer's order: silu rounded to bf16, then the product
            const uint32_t s01 = pack_bf16x2(__fdiv_rn(g0, 1.0f + expf(-g0)), __fdiv_rn(g1, 1.0f + expf(-g1)));
            t0 = __uint_as_float(s01 << 16) * u0;
            t1 = __uint_as_float(s01 & 0xFFFF0000u) * u1;
          } else {                // fast exp/divide: a bf16 result hides their last bits
            t0 = __fdividef(g0, 1.0f + __expf(-g0)) * u0;
            t1 = __fdividef(g1, 1.0f + __expf(-g1)) * u1;
          }
          const uint32_t o01 = pack_bf16x2(t0, t1);
          o[i] = __uint_as_float(o01 << 16);
          o[i + 1] = __uint_as_float(o01 & 0xFFFF0000u);
        }
        if (p.quant) {
          // The block goes out as NVFP4 for the next projection: 8 bytes of codes and one byte of
          // the tiled scale plane per row, the bytes the stand-alone quantizer would write.
          uint32_t sbyte;
          uint2 codes;
          if (p.quant == 1) quant_block_recip(o, sbyte, codes);
          else quant_block_scaled(o, 1.0f, sbyte, codes);
          if (lane < rows_valid) {
            const uint32_t row = row0 + lane, kb = col0 >> 5;
            *reinterpret_cast<uint2*>(static_cast<uint8_t*>(p.out) + size_t(row) * (p.n >> 2) + size_t(kb) * 8) = codes;
            p.out_sf[mb_sf_offset(row, kb, p.out_sf_kchunks)] = uint8_t(sbyte);
          }
          return;
        }
        uint32_t w[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) w[i] = pack_bf16x2(o[2 * i], o[2 * i + 1]);
        uint8_t* g = static_cast<uint8_t*>(p.out) + (size_t(row0) * p.ldo + col0 / 2) * 2;
        stage_and_store(patch, lane, make_uint4(w[0], w[1], w[2], w[3]), make_uint4(w[4], w[5], w[6], w[7]), g,
                        size_t(p.ldo) * 2, rows_valid, min(2u, (p.n - col0) / 16));
      } else if (p.out_dtype == MB_DT_BF16) {
        uint4 units[4];
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          units[g].x = pack_bf16x2(v[8 * g + 0], v[8 * g + 1]);
          units[g].y = pack_bf16x2(v[8 * g + 2], v[8 * g + 3]);
          units[g].z = pack_bf16x2(v[8 * g + 4], v[8 * g + 5]);
          units[g].w = pack_bf16x2(v[8 * g + 6], v[8 * g + 7]);
        }
        uint8_t* g = static_cast<uint8_t*>(p.out) + (size_t(row0) * p.ldo + col0) * 2;
        const uint32_t uv = (p.n - col0) / 8;
        stage_and_store(patch, lane, units[0], units[1], g, size_t(p.ldo) * 2, rows_valid, min(2u, uv));
        if (uv > 2) stage_and_store(patch, lane, units[2], units[3], g + 32, size_t(p.ldo) * 2, rows_valid, min(2u, uv - 2));
      } else {
        // f32: 32 columns = 128 bytes per row, in two passes of 16 columns through the patch
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          uint4 units[4];
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            units[g].x = __float_as_uint(v[16 * hh + 4 * g + 0]);
            units[g].y = __float_as_uint(v[16 * hh + 4 * g + 1]);
            units[g].z = __float_as_uint(v[16 * hh + 4 * g + 2]);
            units[g].w = __float_as_uint(v[16 * hh + 4 * g + 3]);
          }
          const uint32_t c0 = col0 + 16 * hh;
          if (c0 < p.n) {
            uint8_t* g = static_cast<uint8_t*>(p.out) + (size_t(row0) * p.ldo + c0) * 4;
            const uint32_t uv = (p.n - c0) / 4;
            stage_and_store(patch, lane, units[0], units[1], g, size_t(p.ldo) * 4, rows_valid, min(2u, uv));
            if (uv > 2) stage_and_store(patch, lane, units[2], units[3], g + 32, size_t(p.ldo) * 4, rows_valid, min(2u, uv - 2));
          }
        }
      }
}

template <int KIND, int BN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tc5_kernel(const __grid_constant__ GemmParams p) {
  using C = Cfg<KIND, BN>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;   // swizzle atoms need 1024-byte alignment
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + C::STAGES * C::STAGE_BYTES;
  // barrier words: full[STAGES], empty[STAGES], acc_full[2], acc_empty[2], ovl_free, drain, then tmem ptr + abort
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (C::STAGES + s); };
  auto acc_full_bar = [&](int b) { return bar_base + 8u * (2 * C::STAGES + b); };
  auto acc_empty_bar = [&](int b) { return bar_base + 8u * (2 * C::STAGES + 2 + b); };
  const uint32_t ovl_free_bar = bar_base + 8u * (2 * C::STAGES + 4);
  const uint32_t drain_bar = bar_base + 8u * (2 * C::STAGES + 5);   // only used when a wait ran out
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(smem_gen + C::STAGES * C::STAGE_BYTES + 8 * (2 * C::STAGES + 6));
  volatile int* abort_smem = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);

  const int warp = __shfl_sync(0xFFFFFFFFu, int(threadIdx.x >> 5), 0);   // warp-uniform by construction
  const int lane = threadIdx.x & 31;
  int* tflag = p.flags ? p.flags + MB_FLAG_WAIT_TIMEOUT : nullptr;
#ifdef MB_GEMM_PROFILE
  const long long prof_k0 = clock64();
#endif

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(acc_full_bar(b), 1); mbar_init(acc_empty_bar(b), EPI_THREADS); }
    mbar_init(ovl_free_bar, EPI_THREADS);
    mbar_init(drain_bar, 1);
    *abort_smem = 0;
    fence_barrier_init();
    tma_prefetch_desc(&p.tmap_a);
    tma_prefetch_desc(&p.tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_ptr_smem), C::TMEM_COLS);
    tmem_relinquish();
  }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr_smem;
  // everything above touched only this CTA's own shared and tensor memory; global memory from here on
  mb_grid_dependency_sync();

  const uint32_t m_tiles = p.n_mtiles_dev ? uint32_t(*p.n_mtiles_dev) : p.m_tiles;
  const uint32_t total_tiles = m_tiles * p.n_tiles * p.splits;

  // The two issuing roles run with all 32 lanes converged; every asynchronous
  // instruction (TMA, tcgen05.cp/mma/commit) sits under elect_one() so that the
  // compiler sees a single active thread with warp-uniform operands.
  if (warp == 0) {
    // ------------------------------ producer ------------------------------------
    int stage = 0;
    uint32_t phase = 0;
    uint32_t armed = 0;   // bit s: stage s armed at least once; parity of its last arming in armed_par
    uint32_t armed_par = 0;
    bool ok = true;
    // Grouped products: the expert of a tile comes from device memory; it is fetched one tile
    // ahead so that its latency never sits between two tiles' loads.
    int e_next = 0;
    auto row_tile = [&](uint32_t tl) { return p.n_fastest ? tl / p.n_tiles : tl % m_tiles; };   // splits is 1 when grouped
    if (p.tile_expert && blockIdx.x < total_tiles) e_next = p.tile_expert[row_tile(blockIdx.x)];
    for (uint32_t tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
      const uint32_t sp = tile % p.splits, rest = tile / p.splits;
      const uint32_t mt = p.n_fastest ? rest / p.n_tiles : rest % m_tiles;
      const uint32_t nt = p.n_fastest ? rest % p.n_tiles : rest / m_tiles;
      const uint32_t ks0 = sp * p.ks_per_split, ks1 = min(p.k_steps, ks0 + p.ks_per_split);
      uint32_t brow = nt * BN;
      const uint8_t* sfb = p.sfb;
      if (p.tile_expert) {
        int e = e_next;
        const uint32_t nxt = tile + gridDim.x;
        if (nxt < total_tiles) e_next = p.tile_expert[row_tile(nxt)];
        if (e < 0) e = 0;
        brow += uint32_t(e) * p.b_rows_per_expert;
        sfb += uint64_t(e) * p.sfb_expert_stride;
      }
      for (uint32_t ks = ks0; ks < ks1; ++ks) {
        { PROF_T0();
        if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_smem, tflag, 1)) { ok = false; break; }
        PROF_ADD(0); }
        const uint32_t sa = smem_base + stage * C::STAGE_BYTES;
        const uint32_t sb = sa + C::A_BYTES;
        armed |= 1u << stage;
        armed_par = (armed_par & ~(1u << stage)) | (phase << stage);
        if (elect_one()) {
          mbar_arrive_expect_tx(full_bar(stage), C::STAGE_BYTES);
          const int x = KIND == KIND_NVF4 ? int(ks * 128) : int(ks * 64);   // element coordinate (bytes / bf16)
          tma_load_2d(sa, &p.tmap_a, x, int(mt * C::BM), full_bar(stage));
          tma_load_2d(sb, &p.tmap_b, x, int(brow), full_bar(stage));
          if (KIND == KIND_NVF4) {
            const uint32_t ssfa = sb + C::B_BYTES;
            const uint32_t ssfb = ssfa + C::SFA_BYTES;
            bulk_load(ssfa, p.sfa + (uint64_t(mt) * p.sf_kchunks + ks * 4u) * 512u, 2048u, full_bar(stage));
#pragma unroll
            for (int rt = 0; rt < BN / 128; ++rt)
              bulk_load(ssfb + rt * 2048u,
                        sfb + (uint64_t(nt * (BN / 128) + rt) * p.sf_kchunks + ks * 4u) * 512u, 2048u,
                        full_bar(stage));
          }
        }
        __syncwarp();
        if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
      }
    }
    if (!ok) {
      // Leave no copy in flight: wait (bounded) for every stage this warp armed.
      for (int s = 0; s < C::STAGES; ++s)
        if (armed & (1u << s)) {
          long long t0 = clock64();
          while (!mbar_try_wait(full_bar(s), (armed_par >> s) & 1u) && clock64() - t0 < WAIT_LIMIT_CYCLES) {}
        }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ----------------------------------
    int stage = 0;
    uint32_t phase = 0;
    const uint32_t idesc = KIND == KIND_NVF4 ? idesc_nvf4(BN) : idesc_bf16(BN);
    uint32_t it = 0;
    bool ok = true;
    for (uint32_t tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++it) {
      const uint32_t buf = it & 1u;
      if (C::OVERLAP) {
        // The previous tile's epilogue has drained the 64 shared columns.
        PROF_T0();
        if (it > 0 && !mbar_wait(ovl_free_bar, (it - 1u) & 1u, abort_smem, tflag, 2)) { ok = false; break; }
        PROF_ADD(1);
      } else {
        PROF_T0();
        if (!mbar_wait(acc_empty_bar(buf), ((it >> 1) & 1u) ^ 1u, abort_smem, tflag, 2)) { ok = false; break; }
        PROF_ADD(1);
      }
      fence_after_sync();
      const uint32_t d_tmem = tmem_base + (buf ? C::ACC1 : C::ACC0);
      const uint32_t sp = tile % p.splits;
      const uint32_t ks0 = sp * p.ks_per_split, ks1 = min(p.k_steps, ks0 + p.ks_per_split);
      for (uint32_t ks = ks0; ks < ks1; ++ks) {
        { PROF_T0();
        if (!mbar_wait(full_bar(stage), phase, abort_smem, tflag, 3)) { ok = false; break; }
        PROF_ADD(2); }
        fence_after_sync();
        const uint32_t sa = smem_base + stage * C::STAGE_BYTES;
        const uint32_t sb = sa + C::A_BYTES;
        if (elect_one()) {
          if (KIND == KIND_NVF4) {
            const uint32_t ssfa = sb + C::B_BYTES;
            const uint32_t ssfb = ssfa + C::SFA_BYTES;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              utccp_32x128b_warpx4(tmem_base + C::SFA_COL + 4 * j, make_sf_desc(ssfa + 512 * j));
#pragma unroll
              for (int rt = 0; rt < BN / 128; ++rt)
                utccp_32x128b_warpx4(tmem_base + C::SFB_COL + j * (BN / 32) + rt * 4,
                                     make_sf_desc(ssfb + rt * 2048 + 512 * j));
            }
          }
          const uint64_t adesc = make_kmajor_sw128_desc(sa);
          const uint64_t bdesc = make_kmajor_sw128_desc(sb);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t acc = ((ks - ks0) | uint32_t(j)) != 0u;
            // 32 bytes of K per instruction: the descriptor start address advances by 2 (16-byte units).
            if (KIND == KIND_NVF4)
              mma_nvf4(d_tmem, adesc + 2 * j, bdesc + 2 * j, idesc, tmem_base + C::SFA_COL + 4 * j,
                       tmem_base + C::SFB_COL + j * (BN / 32), acc);
            else
              mma_f16(d_tmem, adesc + 2 * j, bdesc + 2 * j, idesc, acc);
          }
          umma_commit(empty_bar(stage));   // the stage is free once these MMAs have read it
          if (ks + 1 == ks1) umma_commit(acc_full_bar(buf));
        }
        __syncwarp();
        if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
      }
    }
    if (!ok) {
      // Let the issued MMAs retire before TMEM is freed: one more commit, bounded wait.
      if (elect_one()) umma_commit(drain_bar);
      __syncwarp();
      long long t0 = clock64();
      while (!mbar_try_wait(drain_bar, 0u) && clock64() - t0 < WAIT_LIMIT_CYCLES) {}
    }
  } else {
    // ------------------------------ epilogue ------------------------------------
    const uint32_t quad = warp & 3u;                  // TMEM lane quadrant this warp may read
    const uint32_t ew = uint32_t(warp) - 2u, part = ew >> 2;   // four warps per quadrant split the columns
    uint8_t* patch = smem_gen + C::STAGES * C::STAGE_BYTES + 256 + ew * 512;
    uint32_t it = 0;
    bool ok = true;
    for (uint32_t tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++it) {
      const uint32_t sp = tile % p.splits, rest = tile / p.splits;
      const uint32_t mt = p.n_fastest ? rest / p.n_tiles : rest % m_tiles;
      const uint32_t nt = p.n_fastest ? rest % p.n_tiles : rest / m_tiles;
      const uint32_t buf = it & 1u;
      float alpha = p.alpha;
      if (p.tile_expert) {
        int e = p.tile_expert[mt];
        alpha = e >= 0 ? p.alpha_vec[e] : 0.0f;
      }
      const uint32_t row0 = mt * C::BM + quad * 32u;       // first row of this warp's 32
      const uint32_t row = row0 + lane;
      uint32_t rows_valid = row0 < p.m ? min(32u, p.m - row0) : 0u;
      // pad rows close an expert's last tile, so the live rows of a warp are a prefix
      if (p.row_tok) rows_valid = __popc(__ballot_sync(0xFFFFFFFFu, row < p.m && __ldg(p.row_tok + row) >= 0));
      float scale = alpha;
      if (p.rowscale && row < p.m) scale = p.rowscale[row] * alpha;
#ifdef MB_GEMM_PROFILE
      const long long prof_e0 = clock64();
#endif
      if (!mbar_wait(acc_full_bar(buf), (it >> 1) & 1u, abort_smem, tflag, 4)) { ok = false; break; }
#ifdef MB_GEMM_PROFILE
      const long long prof_e1 = clock64();
#endif
      fence_after_sync();
      const uint32_t t_acc = tmem_base + ((quad * 32u) << 16) + (buf ? C::ACC1 : C::ACC0);
      constexpr int CHUNKS = BN / 32;
      if (p.cluster_splitk) {
        // This CTA's K slice of the tile: the raw f32 sums are parked in the operand stages (idle now: one tile per
        // CTA, every MMA has retired) as [128 rows][BN] with the 16-byte units of a row XOR-ed by the row, so that
        // the 32 rows of a warp store, and the readers of the other CTAs load, without bank conflicts.
        constexpr int PERW = CHUNKS / (EPI_WARPS / 4);
        const uint32_t trow = quad * 32u + uint32_t(lane);
        uint8_t* rowp = smem_gen + trow * (BN * 4);
#pragma unroll 1
        for (int ci = 0; ci < PERW; ++ci) {
          const int c = int(part) * PERW + ci;
          uint32_t r[32];
          tmem_ld_x32(t_acc + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const uint32_t unit = uint32_t(c) * 8u + uint32_t(u);
            *reinterpret_cast<uint4*>(rowp + ((unit ^ (trow & 7u)) * 16u)) =
                make_uint4(r[4 * u], r[4 * u + 1], r[4 * u + 2], r[4 * u + 3]);
          }
        }
        continue;
      }
      // split-K: slice sp of the K sum lands in plane sp of the f32 workspace (p.out, p.m rows per plane)
      const uint32_t row0_store = row0 + sp * p.m;
      auto process = [&](int c, const uint32_t* r) {
        epilogue_chunk(p, r, nt * BN + c * 32, row0_store, rows_valid, scale, patch, lane);
      };
      constexpr int PER = CHUNKS / (EPI_WARPS / 4);     // chunks per warp: 2 (BN 256) or 1 (BN 128)
      if (C::OVERLAP) {
        // The 64 columns shared with the other accumulator come out first (one chunk each for the
        // first two warps of the quadrant), before any store work, so that the next tile's MMAs are
        // released at once; the other six chunks follow: one more for those two warps, two each
        // for the other two.
        const int shared0 = buf == 0 ? CHUNKS - 2 : 0, rest0 = buf == 0 ? 0 : 2;
        const int c0 = part < 2 ? shared0 + int(part) : rest0 + 2 * int(part) - 2;
        const int c1 = part < 2 ? rest0 + int(part) : rest0 + 2 * int(part) - 1;
        uint32_t ra[32];
        { PROF_T0();
        tmem_ld_x32(t_acc + c0 * 32, ra);
        tmem_ld_wait();
        if (warp == 2) PROF_ADD(7); }
        fence_before_sync();
        mbar_arrive(ovl_free_bar);
        process(c0, ra);
        uint32_t r[32];
        tmem_ld_x32(t_acc + c1 * 32, r);
        tmem_ld_wait();
        process(c1, r);
      } else {
#pragma unroll 1
        for (int ci = 0; ci < PER; ++ci) {
          const int c = int(part) * PER + ci;
          uint32_t r[32];
          tmem_ld_x32(t_acc + c * 32, r);
          tmem_ld_wait();
          process(c, r);
        }
      }
      fence_before_sync();
      mbar_arrive(acc_empty_bar(buf));
#ifdef MB_GEMM_PROFILE
      if (warp == 2 && lane == 0) {
        atomicAdd(&g_gemm_prof[blockIdx.x * 8 + 3], (unsigned long long)(prof_e1 - prof_e0));
        atomicAdd(&g_gemm_prof[blockIdx.x * 8 + 4], (unsigned long long)(clock64() - prof_e1));
        atomicAdd(&g_gemm_prof[blockIdx.x * 8 + 6], 1ull);
      }
#endif
    }
  }

  if (p.cluster_splitk) {
    // ------------------------------ K slices meet ------------------------------------
    // Every thread of every CTA of the cluster comes here, also after a wait that ran out (the flag word tells the
    // host; the sums are then wrong but every load below still finds its shared memory in place). CTA r sums the
    // 32-column chunks r, r + splits, ... over the slices in slice order, the order of the stand-alone sum of
    // planes, so both paths give the same bits.
    cluster_sync_unaligned();
    if (warp >= 2 && *abort_smem == 0) {
      const uint32_t ew = uint32_t(warp) - 2u, rank = cluster_ctarank();
      const uint32_t rest = blockIdx.x / p.splits;
      const uint32_t mt = p.n_fastest ? rest / p.n_tiles : rest % m_tiles;
      const uint32_t nt = p.n_fastest ? rest % p.n_tiles : rest / m_tiles;
      const uint32_t m_valid = min(128u, p.m - mt * 128u);
      const uint32_t tile_s = smem_u32(smem_gen);
      for (uint32_t c = rank; c < uint32_t(BN / 32); c += p.splits) {
        const uint32_t col = nt * BN + c * 32u + (uint32_t(lane) & 7u) * 4u;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const uint32_t row = ew * 8u + uint32_t(h) * 4u + (uint32_t(lane) >> 3);
          if (row >= m_valid || col >= p.n) continue;
          const uint32_t unit = c * 8u + (uint32_t(lane) & 7u);
          const uint32_t addr = tile_s + row * (BN * 4) + ((unit ^ (row & 7u)) * 16u);
          float4 v[8];
#pragma unroll
          for (uint32_t sl = 0; sl < 8; ++sl)
            if (sl < p.splits) v[sl] = ld_cluster_f32x4(map_to_cta(addr, sl));
          float4 acc = v[0];
#pragma unroll
          for (uint32_t sl = 1; sl < 8; ++sl)
            if (sl < p.splits) { acc.x += v[sl].x; acc.y += v[sl].y; acc.z += v[sl].z; acc.w += v[sl].w; }
          const size_t grow = size_t(mt) * 128u + row;
          const float scale = p.rowscale ? p.rowscale[grow] * p.alpha : p.alpha;
          float4 o;
          if (p.colscale) {
            const float4 cs = __ldg(reinterpret_cast<const float4*>(p.colscale + col));
            o = make_float4(acc.x * scale * cs.x, acc.y * scale * cs.y, acc.z * scale * cs.z, acc.w * scale * cs.w);
          } else {
            o = make_float4(acc.x * scale, acc.y * scale, acc.z * scale, acc.w * scale);
          }
          if (p.out_dtype == MB_DT_F32)
            *reinterpret_cast<float4*>(static_cast<float*>(p.out) + grow * p.ldo + col) = o;
          else
            *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(p.out) + grow * p.ldo + col) =
                make_uint2(pack_bf16x2(o.x, o.y), pack_bf16x2(o.z, o.w));
        }
      }
    }
    cluster_sync_unaligned();          // no CTA leaves while another may still read its sums
  }

  // ------------------------------ teardown ----------------------------------------
  fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    fence_after_sync();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
#ifdef MB_GEMM_PROFILE
  if (threadIdx.x == 0) atomicAdd(&g_gemm_prof[blockIdx.x * 8 + 5], (unsigned long long)(clock64() - prof_k0));
#endif
}


// ---------------------------------------------------------------------------------
// CTA-pair variant (cta_group::2): one 256 x 256 output tile per pair of CTAs.
//
// Each CTA of the pair loads its own 128 rows of A, its own half (128 rows) of the B
// tile, its own A scales and the B scales of all 256 columns; the leader CTA issues
// one 256 x 256 x 64 MMA per K block for both tensor cores, so that per SM only
// 128 + 128 operand rows cross L2 -> shared memory per K step instead of 128 + 256.
// No load is multicast: every CTA fetches what lands in its own shared memory; only
// the completion counts (leader's barrier) and tcgen05.commit cross the pair.
// ---------------------------------------------------------------------------------
struct Cfg2 {
  static constexpr int BN = 256;
  static constexpr int A_BYTES = 128 * 128;
  static constexpr int B_BYTES = 128 * 128;          // this CTA's half of the B tile
  static constexpr int SFA_BYTES = 2048;
  static constexpr int SFB_BYTES = 4096;             // scales of all 256 columns
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES;   // 38 KB
  static constexpr int STAGES = 5;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256 + EPI_WARPS_ * 512;
  static constexpr int ACC0 = 0, ACC1 = 192, SFA_COL = 448, SFB_COL = 464, TMEM_COLS = 512;
};

struct Gemm2Params {
  GemmParams g;
  CUtensorMap tmap_sfa;   // tiled scale planes as [atoms, 128 x int32], box 4 atoms
  CUtensorMap tmap_sfb;
  uint32_t m_pairs;
  uint32_t raster_group;  // row pairs per group of the tile order (see pair_tile)
};

// Tile order of the pair kernel. The pairs that run together take consecutive tile numbers, so the order
// decides what they share in L2. Row pairs are taken in groups of `group`: inside a group the row pair runs
// fastest and the column tile slowest, then the next group starts. The concurrent tiles then cover `group`
// row pairs x (pairs / group) column tiles, a near-square patch whose operands are a few tens of MB, and
// the A rows of a group stay in L2 while the group walks every column tile: A comes from DRAM once, B once
// per group. With the row pair fastest over ALL rows (group = m_pairs) a K = 14336 activation (66 MB with its
// scales) was pulled from DRAM again for every wave of column tiles (366 MB read for 99 MB of operands); with
// small groups the weights are read once per group instead (K = 4096, N = 14336: 143 MB against 52 MB at
// 8 pairs per group). The host picks the group size from K (see launch).
__device__ __forceinline__ void pair_tile(uint32_t tile, uint32_t m_pairs, uint32_t n_tiles, uint32_t group,
                                          uint32_t& mp, uint32_t& nt) {
  const uint32_t per_group = group * n_tiles;
  const uint32_t g = tile / per_group, r = tile - g * per_group;
  const uint32_t g0 = g * group;
  const uint32_t gsz = min(group, m_pairs - g0);
  nt = r / gsz;
  mp = g0 + (r - nt * gsz);
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
gemm_tc5_pair_kernel(const __grid_constant__ Gemm2Params pp) {
  using C = Cfg2;
  const GemmParams& p = pp.g;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + C::STAGES * C::STAGE_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (C::STAGES + s); };
  auto acc_full_bar = [&](int b) { return bar_base + 8u * (2 * C::STAGES + b); };
  const uint32_t ovl_free_bar = bar_base + 8u * (2 * C::STAGES + 2);
  const uint32_t drain_bar = bar_base + 8u * (2 * C::STAGES + 3);
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(smem_gen + C::STAGES * C::STAGE_BYTES + 8 * (2 * C::STAGES + 4));
  volatile int* abort_smem = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);

  const int warp = __shfl_sync(0xFFFFFFFFu, int(threadIdx.x >> 5), 0);
  const uint32_t lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  int* tflag = p.flags ? p.flags + MB_FLAG_WAIT_TIMEOUT : nullptr;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int b = 0; b < 2; ++b) mbar_init(acc_full_bar(b), 1);
    mbar_init(ovl_free_bar, 2 * EPI_WARPS);       // one arrival per epilogue warp of both CTAs
    mbar_init(drain_bar, 1);
    *abort_smem = 0;
    fence_barrier_init();
    tma_prefetch_desc(&p.tmap_a);
    tma_prefetch_desc(&p.tmap_b);
    tma_prefetch_desc(&pp.tmap_sfa);
    tma_prefetch_desc(&pp.tmap_sfb);
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_ptr_smem), C::TMEM_COLS);
    tmem_relinquish_pair();
  }
  fence_before_sync();
  __syncthreads();
  cluster_sync_all();                  // the peer's barriers exist before anything is signalled on them
  fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr_smem;

  const uint32_t total_tiles = pp.m_pairs * p.n_tiles;
  const uint32_t pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;

  if (warp == 0) {
    // ------------------------------ producer (both CTAs) --------------------------
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (uint32_t tile = pair; ok && tile < total_tiles; tile += n_pairs) {
      uint32_t mp, nt;
      pair_tile(tile, pp.m_pairs, p.n_tiles, pp.raster_group, mp, nt);
      const uint32_t mt = mp * 2 + rank;                         // this CTA's 128-row tile of A
      for (uint32_t ks = 0; ks < p.k_steps; ++ks) {
        if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_smem, tflag, 21)) { ok = false; break; }
        const uint32_t sa = smem_base + stage * C::STAGE_BYTES;
        const uint32_t sb = sa + C::A_BYTES;
        const uint32_t ssfa = sb + C::B_BYTES;
        const uint32_t ssfb = ssfa + C::SFA_BYTES;
        if (elect_one()) {
          // all bytes of both CTAs are counted on the leader's barrier
          const uint32_t fb = map_to_cta(full_bar(stage), 0);
          if (leader) mbar_arrive_expect_tx(full_bar(stage), 2 * C::STAGE_BYTES);
          tma_load_2d_pair(sa, &p.tmap_a, int(ks * 128), int(mt * 128), fb);
          tma_load_2d_pair(sb, &p.tmap_b, int(ks * 128), int(nt * C::BN + rank * 128), fb);
          tma_load_2d_pair(ssfa, &pp.tmap_sfa, 0, int(mt * p.sf_kchunks + ks * 4u), fb);
          tma_load_2d_pair(ssfb, &pp.tmap_sfb, 0, int((nt * 2) * p.sf_kchunks + ks * 4u), fb);
          tma_load_2d_pair(ssfb + 2048, &pp.tmap_sfb, 0, int((nt * 2 + 1) * p.sf_kchunks + ks * 4u), fb);
        }
        __syncwarp();
        if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader CTA only) ------------------
    if (leader) {
      int stage = 0;
      uint32_t phase = 0;
      const uint32_t idesc = idesc_nvf4(C::BN, 256);
      uint32_t it = 0;
      bool ok = true;
      for (uint32_t tile = pair; ok && tile < total_tiles; tile += n_pairs, ++it) {
        const uint32_t buf = it & 1u;
        if (it > 0 && !mbar_wait_cluster(ovl_free_bar, (it - 1u) & 1u, abort_smem, tflag, 22)) { ok = false; break; }
        fence_after_sync();
        const uint32_t d_tmem = tmem_base + (buf ? C::ACC1 : C::ACC0);
        for (uint32_t ks = 0; ks < p.k_steps; ++ks) {
          if (!mbar_wait_cluster(full_bar(stage), phase, abort_smem, tflag, 23)) { ok = false; break; }
          fence_after_sync();
          const uint32_t sa = smem_base + stage * C::STAGE_BYTES;
          const uint32_t sb = sa + C::A_BYTES;
          const uint32_t ssfa = sb + C::B_BYTES;
          const uint32_t ssfb = ssfa + C::SFA_BYTES;
          if (elect_one()) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              utccp_32x128b_warpx4_pair(tmem_base + C::SFA_COL + 4 * j, make_sf_desc(ssfa + 512 * j));
              utccp_32x128b_warpx4_pair(tmem_base + C::SFB_COL + j * 8, make_sf_desc(ssfb + 512 * j));
              utccp_32x128b_warpx4_pair(tmem_base + C::SFB_COL + j * 8 + 4, make_sf_desc(ssfb + 2048 + 512 * j));
            }
            const uint64_t adesc = make_kmajor_sw128_desc(sa);
            const uint64_t bdesc = make_kmajor_sw128_desc(sb);
#pragma unroll
            for (int j = 0; j < 4; ++j)
              mma_nvf4_pair(d_tmem, adesc + 2 * j, bdesc + 2 * j, idesc, tmem_base + C::SFA_COL + 4 * j,
                            tmem_base + C::SFB_COL + j * 8, (ks | uint32_t(j)) != 0u);
            umma_commit_pair(empty_bar(stage), 3);                 // frees the stage in both CTAs
            if (ks + 1 == p.k_steps) umma_commit_pair(acc_full_bar(buf), 3);
          }
          __syncwarp();
          if (++stage == C::STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        if (elect_one()) umma_commit(drain_bar);
        __syncwarp();
        long long t0 = clock64();
        while (!mbar_try_wait(drain_bar, 0u) && clock64() - t0 < WAIT_LIMIT_CYCLES) {}
      }
    }
  } else {
    // ------------------------------ epilogue (both CTAs) --------------------------
    const uint32_t quad = warp & 3u;
    const uint32_t ew = uint32_t(warp) - 2u, part = ew >> 2;
    uint8_t* patch = smem_gen + C::STAGES * C::STAGE_BYTES + 256 + ew * 512;
    const uint32_t ovl_remote = map_to_cta(ovl_free_bar, 0);
    uint32_t it = 0;
    bool ok = true;
    for (uint32_t tile = pair; ok && tile < total_tiles; tile += n_pairs, ++it) {
      uint32_t mp, nt;
      pair_tile(tile, pp.m_pairs, p.n_tiles, pp.raster_group, mp, nt);
      const uint32_t buf = it & 1u;
      const uint32_t row0 = (mp * 2 + rank) * 128 + quad * 32u;
      const uint32_t row = row0 + lane;
      const uint32_t rows_valid = row0 < p.m ? min(32u, p.m - row0) : 0u;
      float scale = p.alpha;
      if (p.rowscale && row < p.m) scale = p.rowscale[row] * p.alpha;
      if (!mbar_wait_cluster(acc_full_bar(buf), (it >> 1) & 1u, abort_smem, tflag, 24)) { ok = false; break; }
      fence_after_sync();
      const uint32_t t_acc = tmem_base + ((quad * 32u) << 16) + (buf ? C::ACC1 : C::ACC0);
      constexpr int CHUNKS = C::BN / 32;
      const int shared0 = buf == 0 ? CHUNKS - 2 : 0, rest0 = buf == 0 ? 0 : 2;
      const int c0 = part < 2 ? shared0 + int(part) : rest0 + 2 * int(part) - 2;
      const int c1 = part < 2 ? rest0 + int(part) : rest0 + 2 * int(part) - 1;
      uint32_t ra[32];
      tmem_ld_x32(t_acc + c0 * 32, ra);
      tmem_ld_wait();
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(ovl_remote);              // this warp is past the shared columns
      epilogue_chunk(p, ra, nt * C::BN + c0 * 32, row0, rows_valid, scale, patch, lane);
      uint32_t r[32];
      tmem_ld_x32(t_acc + c1 * 32, r);
      tmem_ld_wait();
      epilogue_chunk(p, r, nt * C::BN + c1 * 32, row0, rows_valid, scale, patch, lane);
    }
  }

  // ------------------------------ teardown ----------------------------------------
  fence_before_sync();
  __syncthreads();
  cluster_sync_all();                  // neither CTA leaves while the peer may still touch it
  if (warp == 1) {
    fence_after_sync();
    tmem_dealloc_pair(tmem_base, C::TMEM_COLS);
  }
}

// Sum of the split-K planes in plane order, times the epilogue scale, one cast.
template <typename O>
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(const float4* __restrict__ partial, uint32_t splits, size_t plane4, uint32_t n4,
                     const float* __restrict__ rowscale, const float4* __restrict__ colscale, float alpha,
                     O* __restrict__ out) {
  mb_grid_dependency_sync();
  size_t i = size_t(blockIdx.x) * 256 + threadIdx.x;
  if (i >= plane4) return;
  float4 acc = partial[i];
  for (uint32_t s = 1; s < splits; ++s) {
    const float4 v = partial[size_t(s) * plane4 + i];
    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
  }
  const float scale = rowscale ? rowscale[i / n4] * alpha : alpha;
  float4 c = make_float4(1.0f, 1.0f, 1.0f, 1.0f);
  if (colscale) c = __ldg(colscale + i % n4);
  const float4 r = colscale ? make_float4(acc.x * scale * c.x, acc.y * scale * c.y, acc.z * scale * c.z, acc.w * scale * c.w)
                            : make_float4(acc.x * scale, acc.y * scale, acc.z * scale, acc.w * scale);
  if (sizeof(O) == 4) {
    reinterpret_cast<float4*>(out)[i] = r;
  } else {
    reinterpret_cast<uint2*>(out)[i] = make_uint2(pack_bf16x2(r.x, r.y), pack_bf16x2(r.z, r.w));
  }
}

// How many K slices a product with few output tiles is cut into (1 = no split).
uint32_t splitk_factor(int sm_count, size_t m, size_t n, size_t k) {
  if (m > 128 || n % 4 != 0) return 1;
  const uint32_t bn = n % 256 == 0 ? 256 : 128;
  const uint32_t tiles = uint32_t((n + bn - 1) / bn);
  const uint32_t k_steps = uint32_t((k + 255) / 256);
  if (tiles * 2 > uint32_t(sm_count) || k_steps < 4) return 1;
  uint32_t want = uint32_t(sm_count) / tiles;             // one wave: tiles x slices <= SMs
  want = std::min<uint32_t>(want, k_steps);
  want = std::min<uint32_t>(want, 32);
  if (want < 2) return 1;
  const uint32_t per = (k_steps + want - 1) / want;
  return (k_steps + per - 1) / per;
}

// ---------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int get_encoder(mb_ctx* ctx, EncodeTiledFn* fn) {
  if (!ctx->encode_tiled) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    MB_CUDA_OK(ctx, cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q));
    if (!sym || q != cudaDriverEntryPointSuccess)
      return mb_fail(ctx, MB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    ctx->encode_tiled = sym;
  }
  *fn = reinterpret_cast<EncodeTiledFn>(ctx->encode_tiled);
  return MB_OK;
}

// Row-major [rows, row_bytes] matrix, box of 128 bytes x box_rows, 128-byte swizzle.
int make_tmap(mb_ctx* ctx, CUtensorMap* tm, const void* base, bool bf16, uint64_t rows, uint64_t row_bytes,
              uint32_t box_rows) {
  EncodeTiledFn enc;
  int rc = get_encoder(ctx, &enc);
  if (rc) return rc;
  cuuint64_t dims[2] = {bf16 ? row_bytes / 2 : row_bytes, rows};
  cuuint64_t strides[1] = {row_bytes};
  cuuint32_t box[2] = {bf16 ? 64u : 128u, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(tm, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 2,
                   const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return mb_fail(ctx, MB_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d", int(r));
  return MB_OK;
}

template <int KIND, int BN>
int launch(mb_ctx* ctx, cudaStream_t stream, const GemmParams& p, uint32_t max_tiles) {
  using C = Cfg<KIND, BN>;
  constexpr uint32_t once_bit = KIND == KIND_NVF4 ? (BN == 256 ? MB_ONCE_GEMM_NVF4_256 : MB_ONCE_GEMM_NVF4_128)
                                                  : (BN == 256 ? MB_ONCE_GEMM_BF16_256 : MB_ONCE_GEMM_BF16_128);
  auto kern = gemm_tc5_kernel<KIND, BN>;
  if (!mb_once(ctx, once_bit)) {
    MB_CUDA_OK(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
    mb_once_done(ctx, once_bit);
  }
  const int sms = ctx->sm_limit > 0 ? std::min(ctx->sm_limit, ctx->sm_count) : ctx->sm_count;
  unsigned grid = std::min<uint32_t>(max_tiles, uint32_t(sms));
  if (grid == 0) return MB_OK;
  MB_CUDA_OK(ctx, mb_launch_pdl(kern, dim3(grid), dim3(NUM_THREADS), C::SMEM_BYTES, stream, p));
  MB_LAUNCH_OK(ctx);
  return MB_OK;
}


// Split-K as clusters: the K slices of an output tile are the CTAs of one cluster (consecutive block indices),
// one tile per CTA, and meet in distributed shared memory instead of f32 planes in global memory and a second
// kernel. A cluster must sit inside one GPC, so the device holds fewer CTAs of them than of single CTAs (B200,
// one CTA per SM: 74 clusters of two, 33 of four, 22 of six, 15 of eight); the slice count is the largest one, up
// to the count the plane path would use and at most eight, for which all tiles' clusters are resident at once.
// MB_SPLITK_CLUSTER=0 in the environment switches the form off (comparison runs and tests; read per call).
template <int KIND, int BN>
int splitk_clusters_held(mb_ctx* ctx, uint32_t cluster) {
  using C = Cfg<KIND, BN>;
  int& held = ctx->splitk_clusters[(KIND == KIND_NVF4 ? 0 : 2) + (BN == 256 ? 0 : 1)][cluster];
  if (held == 0) {
    constexpr uint32_t once_bit = KIND == KIND_NVF4 ? (BN == 256 ? MB_ONCE_GEMM_NVF4_256 : MB_ONCE_GEMM_NVF4_128)
                                                    : (BN == 256 ? MB_ONCE_GEMM_BF16_256 : MB_ONCE_GEMM_BF16_128);
    auto kern = gemm_tc5_kernel<KIND, BN>;
    if (!mb_once(ctx, once_bit)) {
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES) != cudaSuccess) {
        (void)cudaGetLastError();
        return 0;
      }
      mb_once_done(ctx, once_bit);
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(cluster);
    cfg.blockDim = dim3(NUM_THREADS);
    cfg.dynamicSmemBytes = C::SMEM_BYTES;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = cluster; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) { (void)cudaGetLastError(); n = 0; }
    held = n >= 1 ? n : -1;
  }
  return held > 0 ? held : 0;
}

// The cluster form for a product the plane path would cut into `sk` slices: which tile width and how many slices
// put the most CTAs on the device with every tile's cluster resident at once. A 128-column tile doubles the tiles
// and so allows smaller clusters, of which the device holds more (a [64, 4096] output: 32 tiles x 4 slices = 128
// CTAs, where 16 tiles x 8 slices do not fit as clusters). slices = 0: the form does not apply, or would leave more
// than a third of the plane path's CTAs unused. min_steps: fewest K steps per slice.
struct SplitkCluster { uint32_t slices; bool wide; };

int splitk_held(mb_ctx* ctx, int kind, bool wide, uint32_t cluster) {
  if (kind == KIND_NVF4) return wide ? splitk_clusters_held<KIND_NVF4, 256>(ctx, cluster) : splitk_clusters_held<KIND_NVF4, 128>(ctx, cluster);
  return wide ? splitk_clusters_held<KIND_BF16, 256>(ctx, cluster) : splitk_clusters_held<KIND_BF16, 128>(ctx, cluster);
}

SplitkCluster splitk_cluster_plan(mb_ctx* ctx, int kind, size_t m, size_t n, uint32_t k_steps, uint32_t sk,
                                  uint32_t min_steps) {
  SplitkCluster best = {0u, n % 256 == 0};
  const char* env = getenv("MB_SPLITK_CLUSTER");
  if ((env && env[0] == '0') || sk < 2) return best;
  const uint32_t sms = uint32_t(ctx->sm_limit > 0 ? std::min(ctx->sm_limit, ctx->sm_count) : ctx->sm_count);
  const uint32_t m_tiles = uint32_t((m + 127) / 128);
  const uint32_t plane_ctas = m_tiles * uint32_t((n + (best.wide ? 255 : 127)) / (best.wide ? 256 : 128)) * sk;
  uint32_t best_ctas = 0;
  for (int w = best.wide ? 1 : 0; w >= 0; --w) {
    const uint32_t bn = w ? 256u : 128u;
    const uint32_t tiles = m_tiles * uint32_t((n + bn - 1) / bn);
    if (tiles == 0 || tiles * 2 > sms) continue;
    uint32_t want = std::min<uint32_t>(std::min<uint32_t>(8u, sms / tiles), k_steps / std::max(1u, min_steps));
    for (; want >= 2; --want) {
      const uint32_t per = (k_steps + want - 1) / want;
      const uint32_t slices = (k_steps + per - 1) / per;
      if (slices < 2) break;
      if (tiles * slices > sms || tiles > uint32_t(splitk_held(ctx, kind, w != 0, slices))) continue;
      if (tiles * slices > best_ctas) { best_ctas = tiles * slices; best.slices = slices; best.wide = w != 0; }
      break;
    }
  }
  if (best_ctas * 100 < plane_ctas * 65) best.slices = 0;
  return best;
}

template <int KIND, int BN>
int launch_splitk_cluster(mb_ctx* ctx, cudaStream_t stream, const GemmParams& p, uint32_t tiles) {
  using C = Cfg<KIND, BN>;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(tiles * p.splits);
  cfg.blockDim = dim3(NUM_THREADS);
  cfg.dynamicSmemBytes = C::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = p.splits; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = mb_pdl_enabled() ? 2 : 1;
  MB_CUDA_OK(ctx, cudaLaunchKernelEx(&cfg, gemm_tc5_kernel<KIND, BN>, p));
  MB_LAUNCH_OK(ctx);
  return MB_OK;
}

// A tiled scale plane seen as [atoms, 512 bytes]: 128 int32 per atom, box of 4 atoms (one K step).
int make_sf_tmap(mb_ctx* ctx, CUtensorMap* tm, const void* base, uint64_t atoms) {
  EncodeTiledFn enc;
  int rc = get_encoder(ctx, &enc);
  if (rc) return rc;
  cuuint64_t dims[2] = {128, atoms};
  cuuint64_t strides[1] = {512};
  cuuint32_t box[2] = {128, 4};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_INT32, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return mb_fail(ctx, MB_ERR_CUDA, "cuTensorMapEncodeTiled (scales) failed with %d", int(r));
  return MB_OK;
}

// Launch of the CTA-pair kernel: as many clusters as the device can hold at once, persistent.
int launch_pair(mb_ctx* ctx, cudaStream_t stream, Gemm2Params& pp) {
  if (!ctx->pair_clusters) {
    MB_CUDA_OK(ctx, cudaFuncSetAttribute(gemm_tc5_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg2::SMEM_BYTES));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(unsigned(ctx->sm_count) & ~1u);
    cfg.blockDim = dim3(NUM_THREADS);
    cfg.dynamicSmemBytes = Cfg2::SMEM_BYTES;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    MB_CUDA_OK(ctx, cudaOccupancyMaxActiveClusters(&n, gemm_tc5_pair_kernel, &cfg));
    if (n < 1) return mb_fail(ctx, MB_ERR_CUDA, "no CTA pair of the GEMM kernel fits on this device");
    ctx->pair_clusters = n;
  }
  const uint32_t tiles = pp.m_pairs * pp.g.n_tiles;
  uint32_t pairs = uint32_t(ctx->pair_clusters);
  if (ctx->sm_limit > 0) pairs = std::min<uint32_t>(pairs, std::max(1, ctx->sm_limit / 2));
  const unsigned grid = 2u * std::min<uint32_t>(tiles, pairs);
  gemm_tc5_pair_kernel<<<grid, NUM_THREADS, Cfg2::SMEM_BYTES, stream>>>(pp);
  MB_LAUNCH_OK(ctx);
  return MB_OK;
}

// What the plain product does not need: the fused exchange, the split-K workspace, per-column
// scales of stacked projections, the quantized output of a SwiGLU epilogue.
struct GemmExtra {
  const mb_symm* symm = nullptr;
  int step = 0;
  void* workspace = nullptr;
  size_t workspace_bytes = 0;
  const float* colscale = nullptr;
  void* out_sf = nullptr;
  const int32_t* row_tok = nullptr;
};

int gemm_w4a4_common(mb_ctx* ctx, cudaStream_t stream, const uint8_t* a_codes, const uint8_t* a_sf,
                     const uint8_t* b_codes, const uint8_t* b_sf, const float* rowscale, float alpha,
                     const float* alpha_vec, const int32_t* tile_expert, const int32_t* n_tiles_dev, size_t m,
                     size_t experts, size_t n, size_t k, void* out, int out_dtype, int epilogue_word,
                     const GemmExtra& ex = GemmExtra()) {
  const mb_symm* symm = ex.symm;
  const int step = ex.step;
  void* workspace = ex.workspace;
  const size_t workspace_bytes = ex.workspace_bytes;
  // epilogue word: kind in the low byte, output quantization in the flag bits
  const int kind = epilogue_word & 0xFF;
  const int quant = (epilogue_word & MB_EPI_QUANT_RECIP) ? 1 : (epilogue_word & MB_EPI_QUANT_SCALED) ? 2 : 0;
  const bool swiglu = kind == MB_EPI_SWIGLU_INTERLEAVED || kind == MB_EPI_SWIGLU_ROUNDED;
  const int epilogue = swiglu ? MB_EPI_SWIGLU_INTERLEAVED : kind;
  MB_REQUIRE(ctx, (epilogue_word & ~(0xFF | MB_EPI_QUANT_RECIP | MB_EPI_QUANT_SCALED)) == 0 &&
                      (epilogue_word & (MB_EPI_QUANT_RECIP | MB_EPI_QUANT_SCALED)) !=
                          (MB_EPI_QUANT_RECIP | MB_EPI_QUANT_SCALED),
             "gemm_w4a4: unknown epilogue word 0x%x", epilogue_word);
  MB_REQUIRE(ctx, !quant || (swiglu && ex.out_sf && n % 32 == 0 && mb_aligned(ex.out_sf, 16)),
             "gemm_w4a4: a quantized output needs a SwiGLU epilogue, n a multiple of 32 and a scale plane");
  MB_REQUIRE(ctx, !swiglu || n % 32 == 0,
             "gemm_w4a4: a SwiGLU epilogue pairs 32 accumulator columns into 16 results; n must be a multiple of 32, got %zu", n);
  MB_REQUIRE(ctx, !ex.colscale || (n % 32 == 0 && mb_aligned(ex.colscale, 16)),
             "gemm_w4a4: column scales need n a multiple of 32 and 16-byte alignment");
  MB_REQUIRE(ctx, ctx && a_codes && a_sf && b_codes && b_sf && out, "gemm_w4a4: null argument");
  MB_REQUIRE(ctx, m > 0 && n > 0 && k > 0, "gemm_w4a4: empty extent");
  MB_REQUIRE(ctx, k % 64 == 0, "W4A4 needs k a multiple of 64, got %zu", k);
  MB_REQUIRE(ctx, n % 8 == 0, "NVFP4 prompt projection needs n a multiple of 8, got %zu", n);
  MB_REQUIRE(ctx, m * k <= 0xFFFFFFFFull && n * k <= 0xFFFFFFFFull && experts * n < (1ull << 31),
             "gemm_w4a4: exceeds u32 indexing");
  MB_REQUIRE(ctx, out_dtype == MB_DT_BF16 || out_dtype == MB_DT_F32, "gemm_w4a4: output is bf16 or f32");
  MB_REQUIRE(ctx, epilogue == MB_EPI_PLAIN || epilogue == MB_EPI_SCATTER ||
                      (epilogue == MB_EPI_SWIGLU_INTERLEAVED && out_dtype == MB_DT_BF16),
             "gemm_w4a4: the SwiGLU epilogue writes bf16 (or NVFP4 planes)");
  MB_REQUIRE(ctx, mb_aligned(a_codes, 16) && mb_aligned(b_codes, 16) && mb_aligned(a_sf, 16) && mb_aligned(b_sf, 16) &&
                      mb_aligned(out, 16),
             "gemm_w4a4: operands and output need 16-byte alignment");
  if (tile_expert) MB_REQUIRE(ctx, n % 128 == 0 && m % 128 == 0, "grouped gemm: n and the stacked rows are multiples of 128");
  GemmParams p;
  memset(&p, 0, sizeof p);
  bool wide = (n % 256 == 0);
  // decode-sized plain products: the K slices of a tile as one cluster when the device holds enough of them
  SplitkCluster sc = {0u, wide};
  uint32_t sk = 1;
  if (epilogue == MB_EPI_PLAIN && !tile_expert) {
    sk = splitk_factor(ctx->sm_count, m, n, k);
    sc = splitk_cluster_plan(ctx, KIND_NVF4, m, n, uint32_t((k + 255) / 256), sk, 2);
    if (sc.slices) wide = sc.wide;
  }
  int rc = make_tmap(ctx, &p.tmap_a, a_codes, false, m, k / 2, 128);
  if (rc) return rc;
  rc = make_tmap(ctx, &p.tmap_b, b_codes, false, experts * n, k / 2, wide ? 256 : 128);
  if (rc) return rc;
  p.sfa = a_sf; p.sfb = b_sf; p.out = out; p.rowscale = rowscale; p.alpha_vec = alpha_vec;
  p.tile_expert = tile_expert; p.n_mtiles_dev = n_tiles_dev; p.row_tok = quant ? nullptr : ex.row_tok; p.flags = ctx->flags_dev; p.alpha = alpha;
  p.m = uint32_t(m); p.n = uint32_t(n); p.k_steps = uint32_t((k + 255) / 256);
  p.m_tiles = uint32_t((m + 127) / 128);
  p.n_tiles = uint32_t((n + (wide ? 255 : 127)) / (wide ? 256 : 128));
  p.sf_kchunks = uint32_t(mb_sf_kchunks(k));
  p.b_rows_per_expert = uint32_t(n);
  p.sfb_expert_stride = mb_sf_plane_bytes(n, k);
  p.ldo = uint32_t(epilogue == MB_EPI_SWIGLU_INTERLEAVED ? n / 2 : n);
  p.out_dtype = out_dtype; p.epilogue = epilogue;
  p.colscale = ex.colscale; p.silu_rounded = kind == MB_EPI_SWIGLU_ROUNDED; p.quant = quant;
  p.out_sf = static_cast<uint8_t*>(ex.out_sf); p.out_sf_kchunks = uint32_t(mb_sf_kchunks(n / 2));
  // Scale bytes of the K padding (up to the next 256 values) are read by the product that consumes the
  // plane and must decode to a finite value; the epilogue writes live blocks only.
  if (quant && (n / 2) % 256 != 0) MB_CUDA_OK(ctx, cudaMemsetAsync(ex.out_sf, 0, mb_sf_plane_bytes(m, n / 2), stream));
  if (epilogue == MB_EPI_SCATTER) {
    p.scatter_world = uint32_t(symm->world); p.scatter_rank = uint32_t(symm->rank);
    p.scatter_nw = uint32_t(n / symm->world); p.scatter_tmax = uint32_t(symm->t_max);
    const size_t half = symm->t_max * symm->n;     // floats in one step's half of a receive area
    for (int r = 0; r < symm->world; ++r)
      p.scatter_base[r] = reinterpret_cast<float*>(static_cast<uint8_t*>(symm->peer[r]) + mb_symm_flags_bytes()) +
                          size_t(step & 1) * half;
  }
  p.splits = 1; p.ks_per_split = p.k_steps;
  p.n_fastest = tile_expert ? 1u : 0u;
  if (epilogue == MB_EPI_PLAIN && !tile_expert) {
    if (sc.slices) {
      // summed in shared memory: no planes, no second kernel, no workspace
      GemmParams pc = p;
      pc.ks_per_split = (p.k_steps + sc.slices - 1) / sc.slices;
      pc.splits = sc.slices;
      pc.cluster_splitk = 1;
      return wide ? launch_splitk_cluster<KIND_NVF4, 256>(ctx, stream, pc, pc.m_tiles * pc.n_tiles)
                  : launch_splitk_cluster<KIND_NVF4, 128>(ctx, stream, pc, pc.m_tiles * pc.n_tiles);
    }
    if (workspace && sk > 1 && workspace_bytes >= size_t(sk) * m * n * sizeof(float)) {
      // K slices into f32 planes of the workspace, then one ordered sum with the epilogue scale
      p.ks_per_split = (p.k_steps + sk - 1) / sk;
      p.splits = (p.k_steps + p.ks_per_split - 1) / p.ks_per_split;
      GemmParams ps = p;
      ps.out = workspace; ps.out_dtype = MB_DT_F32; ps.ldo = uint32_t(n); ps.alpha = 1.0f; ps.rowscale = nullptr;
      ps.colscale = nullptr;
      rc = wide ? launch<KIND_NVF4, 256>(ctx, stream, ps, ps.m_tiles * ps.n_tiles * ps.splits)
                : launch<KIND_NVF4, 128>(ctx, stream, ps, ps.m_tiles * ps.n_tiles * ps.splits);
      if (rc) return rc;
      const size_t plane4 = m * n / 4;
      const unsigned grid = unsigned((plane4 + 255) / 256);
      if (out_dtype == MB_DT_F32)
        MB_CUDA_OK(ctx, mb_launch_pdl(splitk_reduce_kernel<float>, dim3(grid), dim3(256), 0, stream,
                                      static_cast<const float4*>(workspace), p.splits, plane4, uint32_t(n / 4), rowscale,
                                      reinterpret_cast<const float4*>(ex.colscale), alpha, static_cast<float*>(out)));
      else
        MB_CUDA_OK(ctx, mb_launch_pdl(splitk_reduce_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, stream,
                                      static_cast<const float4*>(workspace), p.splits, plane4, uint32_t(n / 4), rowscale,
                                      reinterpret_cast<const float4*>(ex.colscale), alpha,
                                      static_cast<__nv_bfloat16*>(out)));
      MB_LAUNCH_OK(ctx);
      return MB_OK;
    }
  }
  uint32_t tiles = p.m_tiles * p.n_tiles;
  // Dense products with at least one full pair of row tiles go to the CTA-pair kernel
  // (MB_GEMM_CTA_GROUP=1 in the environment keeps the single-CTA kernel, for comparison runs).
  static const bool single_only = [] { const char* e = getenv("MB_GEMM_CTA_GROUP"); return e && e[0] == '1'; }();
  if (wide && !tile_expert && m > 128 && !single_only) {
    Gemm2Params pp;
    memset(&pp, 0, sizeof pp);
    pp.g = p;
    rc = make_tmap(ctx, &pp.g.tmap_b, b_codes, false, n, k / 2, 128);   // each CTA loads half of the B tile
    if (rc) return rc;
    rc = make_sf_tmap(ctx, &pp.tmap_sfa, a_sf, uint64_t(p.m_tiles) * p.sf_kchunks);
    if (rc) return rc;
    rc = make_sf_tmap(ctx, &pp.tmap_sfb, b_sf, uint64_t((n + 127) / 128) * p.sf_kchunks);
    if (rc) return rc;
    pp.m_pairs = (p.m_tiles + 1) / 2;
    // MB_GEMM_RASTER=<row pairs per group> in the environment overrides the group size (measurement runs)
    static const uint32_t raster_env = [] { const char* e = getenv("MB_GEMM_RASTER"); return e ? uint32_t(atoi(e)) : 0u; }();
    // As many row pairs per group as keep the group's A rows (256 rows of codes and scales per pair) within about
    // 36 MB of the 126 MB L2, the output stream passing through the same cache; groups of equal size. K = 14336:
    // 16 pairs (two groups at 8192 rows), K = 4096: all of them (one group, B read once).
    const double a_pair = 256.0 * double(k) * 0.5625;
    const uint32_t gmax = std::max<uint32_t>(1u, uint32_t(36.0e6 / a_pair));
    const uint32_t ngroups = (pp.m_pairs + gmax - 1) / gmax;
    const uint32_t gauto = (pp.m_pairs + ngroups - 1) / ngroups;
    pp.raster_group = std::max<uint32_t>(1u, std::min<uint32_t>(pp.m_pairs, raster_env ? raster_env : gauto));
    return launch_pair(ctx, stream, pp);
  }
  return wide ? launch<KIND_NVF4, 256>(ctx, stream, p, tiles) : launch<KIND_NVF4, 128>(ctx, stream, p, tiles);
}

}  // namespace

#ifdef MB_GEMM_PROFILE
MB_API int mb_debug_gemm_dbg(int v) { cudaMemcpyToSymbol(g_gemm_dbg, &v, sizeof v); return 0; }
MB_API int mb_debug_gemm_profile(unsigned long long* host_out, int reset) {
  if (host_out) cudaMemcpyFromSymbol(host_out, g_gemm_prof, sizeof g_gemm_prof);
  if (reset) { static unsigned long long z[160 * 8]; cudaMemcpyToSymbol(g_gemm_prof, z, sizeof z); }
  return 0;
}
#endif

MB_API int mb_nvfp4_gemm_w4a4(mb_ctx* ctx, mb_stream stream, const uint8_t* a_codes, const uint8_t* a_sf_tiled,
                              const uint8_t* b_codes, const uint8_t* b_sf_tiled, const float* rowscale, float alpha,
                              size_t m, size_t n, size_t k, void* out, int out_dtype, int epilogue) {
  MB_REQUIRE(ctx, alpha == alpha && alpha > 0.0f && alpha <= 3.4e38f,
             "W4A4 calibrated globals/product must be finite positive");
  return gemm_w4a4_common(ctx, static_cast<cudaStream_t>(stream), a_codes, a_sf_tiled, b_codes, b_sf_tiled, rowscale,
                          alpha, nullptr, nullptr, nullptr, m, 1, n, k, out, out_dtype, epilogue);
}

MB_API size_t mb_nvfp4_gemm_splitk_workspace(size_t m, size_t n, size_t k) {
  const uint32_t sk = splitk_factor(148, m, n, k);
  return sk > 1 ? size_t(sk) * m * n * sizeof(float) : 0;
}

MB_API int mb_nvfp4_gemm_w4a4_splitk(mb_ctx* ctx, mb_stream stream, const uint8_t* a_codes, const uint8_t* a_sf_tiled,
                                     const uint8_t* b_codes, const uint8_t* b_sf_tiled, const float* rowscale,
                                     float alpha, size_t m, size_t n, size_t k, void* out, int out_dtype,
                                     void* workspace, size_t workspace_bytes) {
  MB_REQUIRE(ctx, alpha == alpha && alpha > 0.0f && alpha <= 3.4e38f,
             "W4A4 calibrated globals/product must be finite positive");
  MB_REQUIRE(ctx, workspace == nullptr || mb_aligned(workspace, 16), "gemm_w4a4_splitk: workspace needs 16-byte alignment");
  GemmExtra ex;
  ex.workspace = workspace; ex.workspace_bytes = workspace_bytes;
  return gemm_w4a4_common(ctx, static_cast<cudaStream_t>(stream), a_codes, a_sf_tiled, b_codes, b_sf_tiled, rowscale,
                          alpha, nullptr, nullptr, nullptr, m, 1, n, k, out, out_dtype, MB_EPI_PLAIN, ex);
}

MB_API int mb_nvfp4_gemm_w4a4_stacked(mb_ctx* ctx, mb_stream stream, const uint8_t* a_codes, const uint8_t* a_sf_tiled,
                                      const uint8_t* b_codes, const uint8_t* b_sf_tiled, const float* colscale,
                                      size_t m, size_t n, size_t k, void* out, int out_dtype, int epilogue, void* out_sf,
                                      void* workspace, size_t workspace_bytes) {
  MB_REQUIRE(ctx, colscale != nullptr, "gemm_w4a4_stacked: the column scales carry the weights' globals");
  MB_REQUIRE(ctx, workspace == nullptr || mb_aligned(workspace, 16), "gemm_w4a4_stacked: workspace needs 16-byte alignment");
  GemmExtra ex;
  ex.colscale = colscale; ex.out_sf = out_sf; ex.workspace = workspace; ex.workspace_bytes = workspace_bytes;
  return gemm_w4a4_common(ctx, static_cast<cudaStream_t>(stream), a_codes, a_sf_tiled, b_codes, b_sf_tiled, nullptr,
                          1.0f, nullptr, nullptr, nullptr, m, 1, n, k, out, out_dtype, epilogue, ex);
}

MB_API int mb_nvfp4_gemm_w4a4_scatter(mb_ctx* ctx, mb_stream stream, const uint8_t* a_codes,
                                      const uint8_t* a_sf_tiled, const uint8_t* b_codes, const uint8_t* b_sf_tiled,
                                      float alpha, size_t m, size_t n, size_t k, int step) {
  MB_REQUIRE(ctx, ctx && ctx->symm, "gemm_w4a4_scatter: no exchange memory attached (mb_tp_symm_attach)");
  const mb_symm* sy = ctx->symm;
  MB_REQUIRE(ctx, n == sy->n && m <= sy->t_max, "gemm_w4a4_scatter: [%zu, %zu] does not fit the exchange memory [%zu, %zu]",
             m, n, sy->t_max, sy->n);
  MB_REQUIRE(ctx, (n / sy->world) % 32 == 0 && n % sy->world == 0, "gemm_w4a4_scatter: n / world must be a multiple of 32");
  MB_REQUIRE(ctx, alpha == alpha && alpha > 0.0f && alpha <= 3.4e38f, "W4A4 calibrated globals/product must be finite positive");
  GemmExtra ex;
  ex.symm = sy; ex.step = step;
  return gemm_w4a4_common(ctx, static_cast<cudaStream_t>(stream), a_codes, a_sf_tiled, b_codes, b_sf_tiled, nullptr,
                          alpha, nullptr, nullptr, nullptr, m, 1, n, k, sy->local, MB_DT_F32, MB_EPI_SCATTER, ex);
}

MB_API int mb_nvfp4_gemm_w4a4_grouped(mb_ctx* ctx, mb_stream stream, const uint8_t* a_codes,
                                      const uint8_t* a_sf_tiled, const uint8_t* bank_codes,
                                      const uint8_t* bank_sf_tiled, const float* alpha, const int32_t* tile_expert,
                                      const int32_t* n_tiles_dev, size_t m_cap, size_t experts, size_t n, size_t k,
                                      void* out, int out_dtype, int epilogue, void* out_sf,
                                      const int32_t* row_tok) {
  MB_REQUIRE(ctx, alpha && tile_expert && n_tiles_dev && experts > 0, "grouped gemm: null argument");
  GemmExtra ex;
  ex.out_sf = out_sf;
  ex.row_tok = row_tok;
  return gemm_w4a4_common(ctx, static_cast<cudaStream_t>(stream), a_codes, a_sf_tiled, bank_codes, bank_sf_tiled,
                          nullptr, 1.0f, alpha, tile_expert, n_tiles_dev, m_cap, experts, n, k, out, out_dtype,
                          epilogue, ex);
}

// K slices of a bf16 product with few output tiles (the MoE router projection: 32 tiles of a [4096, 128] output).
static uint32_t bf16_splitk_factor(int sm_count, size_t m, size_t n, size_t k) {
  const uint32_t bn = n % 256 == 0 ? 256 : 128;
  const uint32_t tiles = uint32_t((m + 127) / 128) * uint32_t((n + bn - 1) / bn);
  const uint32_t k_steps = uint32_t((k + 63) / 64);
  if (tiles * 2 > uint32_t(sm_count) || k_steps < 8 || n % 4 != 0) return 1;
  uint32_t want = std::min<uint32_t>(uint32_t(sm_count) / tiles, k_steps / 4);   // at least four K steps per slice
  if (want < 2) return 1;
  const uint32_t per = (k_steps + want - 1) / want;
  return (k_steps + per - 1) / per;
}

// The CTA-pair kernel for prompt-sized products (gemm_bf16_pair.cu).
bool mb_bf16_pair_takes(size_t m, size_t n, size_t k);
int mb_bf16_pair_launch(mb_ctx* ctx, cudaStream_t stream, const void* a, const void* b, float alpha, size_t m, size_t n,
                        size_t k, void* out, int out_dtype);

static int bf16_gemm_common(mb_ctx* ctx, cudaStream_t stream, const void* a, const void* b, float alpha, size_t m,
                            size_t n, size_t k, void* out, int out_dtype, void* workspace, size_t workspace_bytes) {
  MB_REQUIRE(ctx, ctx && a && b && out, "bf16_gemm: null argument");
  MB_REQUIRE(ctx, m > 0 && n > 0 && k > 0 && k % 8 == 0 && n % 8 == 0, "bf16_gemm: k and n must be positive multiples of 8");
  MB_REQUIRE(ctx, m * k <= 0xFFFFFFFFull && n * k <= 0xFFFFFFFFull, "bf16_gemm: exceeds u32 indexing");
  MB_REQUIRE(ctx, out_dtype == MB_DT_BF16 || out_dtype == MB_DT_F32, "bf16_gemm: output is bf16 or f32");
  MB_REQUIRE(ctx, mb_aligned(a, 16) && mb_aligned(b, 16) && mb_aligned(out, 16) && mb_aligned(workspace, 16),
             "bf16_gemm: 16-byte alignment");
  MB_REQUIRE_DEVICE(ctx, "bf16_gemm");
  {
    static const bool pair_off = [] { const char* e = getenv("MB_BF16_PAIR"); return e && e[0] == '0'; }();
    if (!pair_off && mb_bf16_pair_takes(m, n, k)) return mb_bf16_pair_launch(ctx, stream, a, b, alpha, m, n, k, out, out_dtype);
  }
  GemmParams p;
  memset(&p, 0, sizeof p);
  bool wide = (n % 256 == 0);
  const uint32_t sk = bf16_splitk_factor(ctx->sm_count, m, n, k);
  const SplitkCluster sc = splitk_cluster_plan(ctx, KIND_BF16, m, n, uint32_t((k + 63) / 64), sk, 4);
  if (sc.slices) wide = sc.wide;
  int rc = make_tmap(ctx, &p.tmap_a, a, true, m, k * 2, 128);
  if (rc) return rc;
  rc = make_tmap(ctx, &p.tmap_b, b, true, n, k * 2, wide ? 256 : 128);
  if (rc) return rc;
  p.out = out; p.flags = ctx->flags_dev; p.alpha = alpha;
  p.m = uint32_t(m); p.n = uint32_t(n); p.k_steps = uint32_t((k + 63) / 64);
  p.m_tiles = uint32_t((m + 127) / 128);
  p.n_tiles = uint32_t((n + (wide ? 255 : 127)) / (wide ? 256 : 128));
  p.ldo = uint32_t(n); p.out_dtype = out_dtype; p.epilogue = MB_EPI_PLAIN;
  p.splits = 1; p.ks_per_split = p.k_steps;
  uint32_t tiles = p.m_tiles * p.n_tiles;
  if (sc.slices) {
    // the K slices of a tile as one cluster, summed in shared memory
    GemmParams pc = p;
    pc.ks_per_split = (p.k_steps + sc.slices - 1) / sc.slices;
    pc.splits = sc.slices;
    pc.cluster_splitk = 1;
    return wide ? launch_splitk_cluster<KIND_BF16, 256>(ctx, stream, pc, tiles)
                : launch_splitk_cluster<KIND_BF16, 128>(ctx, stream, pc, tiles);
  }
  if (workspace && sk > 1 && workspace_bytes >= size_t(sk) * m * n * sizeof(float)) {
    // K slices into f32 planes, then one ordered sum with alpha (deterministic)
    p.ks_per_split = (p.k_steps + sk - 1) / sk;
    p.splits = (p.k_steps + p.ks_per_split - 1) / p.ks_per_split;
    p.out = workspace; p.out_dtype = MB_DT_F32; p.alpha = 1.0f;
    tiles *= p.splits;
    rc = wide ? launch<KIND_BF16, 256>(ctx, stream, p, tiles) : launch<KIND_BF16, 128>(ctx, stream, p, tiles);
    if (rc) return rc;
    const size_t plane4 = m * n / 4;
    const unsigned grid = unsigned((plane4 + 255) / 256);
    if (out_dtype == MB_DT_F32)
      MB_CUDA_OK(ctx, mb_launch_pdl(splitk_reduce_kernel<float>, dim3(grid), dim3(256), 0, stream,
                                    static_cast<const float4*>(workspace), p.splits, plane4, uint32_t(n / 4),
                                    static_cast<const float*>(nullptr), static_cast<const float4*>(nullptr), alpha,
                                    static_cast<float*>(out)));
    else
      MB_CUDA_OK(ctx, mb_launch_pdl(splitk_reduce_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, stream,
                                    static_cast<const float4*>(workspace), p.splits, plane4, uint32_t(n / 4),
                                    static_cast<const float*>(nullptr), static_cast<const float4*>(nullptr), alpha,
                                    static_cast<__nv_bfloat16*>(out)));
    return MB_OK;
  }
  return wide ? launch<KIND_BF16, 256>(ctx, stream, p, tiles) : launch<KIND_BF16, 128>(ctx, stream, p, tiles);
}

MB_API int mb_bf16_gemm(mb_ctx* ctx, mb_stream stream, const void* a, const void* b, float alpha, size_t m, size_t n,
                        size_t k, void* out, int out_dtype) {
  return bf16_gemm_common(ctx, static_cast<cudaStream_t>(stream), a, b, alpha, m, n, k, out, out_dtype, nullptr, 0);
}

MB_API int mb_gemm_splitk_plan(mb_ctx* ctx, int operands, size_t m, size_t n, size_t k, int* cluster_slices,
                               int* plane_slices) {
  MB_REQUIRE(ctx, ctx && cluster_slices && plane_slices, "gemm_splitk_plan: null argument");
  MB_REQUIRE(ctx, (operands == 0 || operands == 1) && m > 0 && n > 0 && k > 0, "gemm_splitk_plan: operands 0 or 1, sizes > 0");
  uint32_t sk, cs;
  if (operands == 0) {
    sk = splitk_factor(ctx->sm_count, m, n, k);
    cs = splitk_cluster_plan(ctx, KIND_NVF4, m, n, uint32_t((k + 255) / 256), sk, 2).slices;
  } else {
    sk = bf16_splitk_factor(ctx->sm_count, m, n, k);
    cs = splitk_cluster_plan(ctx, KIND_BF16, m, n, uint32_t((k + 63) / 64), sk, 4).slices;
  }
  *cluster_slices = int(cs);
  *plane_slices = int(sk);
  return MB_OK;
}

MB_API size_t mb_bf16_gemm_splitk_workspace(size_t m, size_t n, size_t k) {
  const uint32_t sk = bf16_splitk_factor(148, m, n, k);
  return sk > 1 ? size_t(sk) * m * n * sizeof(float) : 0;
}

MB_API int mb_bf16_gemm_splitk(mb_ctx* ctx, mb_stream stream, const void* a, const void* b, float alpha, size_t m,
                               size_t n, size_t k, void* out, int out_dtype, void* workspace, size_t workspace_bytes) {
  return bf16_gemm_common(ctx, static_cast<cudaStream_t>(stream), a, b, alpha, m, n, k, out, out_dtype, workspace,
                          workspace_bytes);
}
