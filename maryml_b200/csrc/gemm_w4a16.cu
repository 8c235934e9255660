// W4A16 prompt projection for sm_100a: out[m, n] = (sum_k x[m, k] * w[n, k]) * scale2 with bf16 activations
// and NVFP4 weights that stay four bits in HBM. The reference's W4A16 kernel decodes the weight inside the
// product and keeps no 16-bit copy of it (src/nn/nvfp4_gemm.rs:93-197; src/nvfp4.rs:245-254); here the decode
// sits between the TMA stage and the tensor core:
//
//   warp 0      producer: per 64-element K step, the A tile (128 rows of bf16) by TMA into 128B-swizzled shared
//               memory, and the B tile's CODE bytes (BN rows x 32 bytes) by TMA into a raw ring that runs a few
//               steps ahead.
//   warps 6-21  converters: a thread owns half (or a quarter) of one weight row of the step: its code bytes and
//               block scales (read from global memory one step ahead) become bf16 values, E2M1[code] *
//               e4m3(scale) exactly (at most 6 significant bits), written into the swizzled K-major B operand
//               tile the tensor core reads; fence.proxy.async, one arrival per warp. The hardware converts a
//               code pair to f16x2 in one instruction; the f16 bit pattern of an E2M1 value shifted three places
//               down IS the bf16 pattern of that value times 2^-112 (zero stays zero), so one packed bf16
//               multiply by (scale * 2^112) finishes the pair with no trip through f32.
//   warp 1      MMA issuer: tcgen05.mma kind::f16 on two bf16 operands (one instruction descriptor cannot mix a
//               bf16 and an f16 operand: the hardware refuses it as an illegal instruction), f32 accumulation
//               in TMEM, two accumulators in turn.
//   warps 2-5   epilogue: tcgen05.ld, times scale2 (applied once to the accumulator, as the reference does),
//               one cast, coalesced stores through a shared-memory patch.
//
// A product with few output tiles and a long K is cut into K slices (more CTAs streaming weights); the slices land
// in f32 planes of a caller workspace and are summed in slice order.
//
// Algorithmic bytes: n * k * 0.5625 (weights, once) + 2 m k + out. Every mbarrier wait is bounded.
#include "common.cuh"
#include "tc5.cuh"

#include <cuda_fp16.h>

namespace {

using namespace tc5;

constexpr int BM = 128;
constexpr int BK = 64;                        // K elements per step: one 128-byte row of bf16
constexpr int CONV_WARPS = 16;
constexpr int EPI_WARPS = 4;
constexpr int THREADS = 32 * (2 + EPI_WARPS + CONV_WARPS);
// The code bytes are the only operand that comes from HBM (the activation tile is shared by every CTA and stays in
// L2), so their ring is what has to cover the memory latency: 64 KB per CTA, filled RAW_AHEAD steps ahead of the A
// stream. The ring is deeper than that by three, so the producer's wait for a free raw stage asks for a step the
// converters finished long ago and never holds back the next A tile.
constexpr int RAW_RING_BYTES = 64 * 1024;
constexpr int SCALE_AHEAD = 4;                // block-scale words a converter thread holds ahead of its step

template <int BN>
struct Cfg {
  static constexpr int A_BYTES = BM * 128;
  static constexpr int B_BYTES = BN * 128;
  static constexpr int OP_BYTES = A_BYTES + B_BYTES;
  static constexpr int OP_STAGES = BN == 256 ? 3 : 4;
  static constexpr int RAW_BYTES = BN * 32;
  static constexpr int RAW_STAGES = RAW_RING_BYTES / RAW_BYTES;     // 16 or 8
  static constexpr int RAW_AHEAD = RAW_STAGES - 3;
  static constexpr int BAR_BYTES = 512;
  static constexpr int SMEM_BYTES = OP_STAGES * OP_BYTES + RAW_STAGES * RAW_BYTES + 1024 + BAR_BYTES + EPI_WARPS * 512;
  static constexpr int TMEM_COLS = 2 * BN;   // 512 or 256: two accumulators
  static constexpr int TPR = 32 * CONV_WARPS / BN;   // converter threads per weight row: 2 or 4
};

struct W4a16Params {
  CUtensorMap tmap_a;        // [m, k] bf16, box 64 x 128, 128-byte swizzle
  CUtensorMap tmap_codes;    // [n, k / 2] bytes, box 32 x BN, no swizzle
  const uint8_t* scales;     // [n, k / 16] E4M3, row-major
  void* out;
  int* flags;
  float alpha;
  uint32_t m, n, k_steps, m_tiles, n_tiles, sc_stride;   // sc_stride = k / 16
  // split-K (few output tiles, long K): a tile index carries a K slice of ks_per_split steps (k_steps is a multiple
  // of it); slice sp of the sum lands unscaled in plane sp of an f32 workspace [splits, m, n]
  uint32_t splits, ks_per_split;
  float* planes;
  int out_dtype;
  int cluster_splitk;        // the `splits` K slices of a tile are the CTAs of one cluster (consecutive blocks, one
                             // item per CTA) and meet in distributed shared memory: no planes, no second kernel
};

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Four codes (two bytes, low nibble first) times their block scale -> two bf16x2 words (exact). `s112` holds the
// block scale times 2^112 in both halves.
__device__ __forceinline__ void decode4(uint32_t two_bytes, __nv_bfloat162 s112, uint32_t& lo, uint32_t& hi) {
  uint32_t h0, h1;
  asm("{ .reg .b8 b0, b1, b2, b3; mov.b32 {b0, b1, b2, b3}, %2;\n\t"
      "cvt.rn.f16x2.e2m1x2 %0, b0;\n\tcvt.rn.f16x2.e2m1x2 %1, b1; }"
      : "=r"(h0), "=r"(h1) : "r"(two_bytes));
  // f16 s.eeeee.mmmmmmmmmm -> bf16 s.000eeeee.mmmmmmm: the value times 2^(15 - 127); the three mantissa bits that
  // fall off are zero for every E2M1 value
  uint32_t t0 = ((h0 >> 3) & 0x0FFF0FFFu) | (h0 & 0x80008000u);
  uint32_t t1 = ((h1 >> 3) & 0x0FFF0FFFu) | (h1 & 0x80008000u);
  const __nv_bfloat162 p0 = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&t0), s112);
  const __nv_bfloat162 p1 = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&t1), s112);
  lo = *reinterpret_cast<const uint32_t*>(&p0);
  hi = *reinterpret_cast<const uint32_t*>(&p1);
}

// Sixteen codes (eight bytes) and their scale byte -> two 16-byte chunks of eight bf16 values each.
__device__ __forceinline__ void decode_block(uint2 codes, uint32_t scale_byte, uint4& c0, uint4& c1) {
  uint32_t sh;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(sh) : "h"(uint16_t(scale_byte)));
  // 2^112 * scale <= 2^121 is a bf16 value with the scale's four significant bits
  const float sf = __half2float(__low2half(*reinterpret_cast<__half2*>(&sh))) * 5192296858534827628530496329220096.0f;
  const __nv_bfloat162 s = __float2bfloat162_rn(sf);
  decode4(codes.x & 0xFFFFu, s, c0.x, c0.y);
  decode4(codes.x >> 16, s, c0.z, c0.w);
  decode4(codes.y & 0xFFFFu, s, c1.x, c1.y);
  decode4(codes.y >> 16, s, c1.z, c1.w);
}

// Warp-level transpose through a 512-byte shared-memory patch so that global stores are coalesced: lane l holds
// two 16-byte units of ITS row (32 rows x 32 bytes); each half of the warp parks its 16 rows in the patch and
// the whole warp stores them, one instruction writing 16 rows x 32 contiguous bytes.
__device__ __forceinline__ void store_rows(uint8_t* patch, uint32_t lane, const uint4& u0, const uint4& u1, uint8_t* gbase,
                                           size_t row_stride_bytes, uint32_t rows_valid, uint32_t units_valid) {
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
    if (r < rows_valid && u < units_valid)
      *reinterpret_cast<uint4*>(gbase + size_t(r) * row_stride_bytes + u * 16) = v;
    __syncwarp();
  }
}

template <int BN>
__global__ void __launch_bounds__(THREADS, 1)
gemm_w4a16_kernel(const __grid_constant__ W4a16Params p) {
  using C = Cfg<BN>;
  constexpr int RAW_STAGES = C::RAW_STAGES, RAW_AHEAD = C::RAW_AHEAD;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t raw_base = smem_base + C::OP_STAGES * C::OP_BYTES;
  const uint32_t bar_base = raw_base + RAW_STAGES * C::RAW_BYTES;
  auto op_full = [&](int s) { return bar_base + 8u * s; };
  auto op_empty = [&](int s) { return bar_base + 8u * (C::OP_STAGES + s); };
  auto raw_full = [&](int s) { return bar_base + 8u * (2 * C::OP_STAGES + s); };
  auto raw_empty = [&](int s) { return bar_base + 8u * (2 * C::OP_STAGES + RAW_STAGES + s); };
  auto acc_full = [&](int b) { return bar_base + 8u * (2 * C::OP_STAGES + 2 * RAW_STAGES + b); };
  auto acc_empty = [&](int b) { return bar_base + 8u * (2 * C::OP_STAGES + 2 * RAW_STAGES + 2 + b); };
  const uint32_t drain_bar = bar_base + 8u * (2 * C::OP_STAGES + 2 * RAW_STAGES + 4);
  constexpr int N_BARS = 2 * C::OP_STAGES + 2 * RAW_STAGES + 5;
  static_assert(8 * N_BARS + 8 <= C::BAR_BYTES, "barrier area");
  uint8_t* bar_gen = smem_gen + (bar_base - smem_base);
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(bar_gen + 8 * N_BARS);
  volatile int* abort_smem = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);
  uint8_t* patches = bar_gen + C::BAR_BYTES;

  const int warp = __shfl_sync(0xFFFFFFFFu, int(threadIdx.x >> 5), 0);
  const uint32_t lane = threadIdx.x & 31;
  int* tflag = p.flags ? p.flags + MB_FLAG_WAIT_TIMEOUT : nullptr;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::OP_STAGES; ++s) { mbar_init(op_full(s), 1 + CONV_WARPS); mbar_init(op_empty(s), 1); }
    for (int s = 0; s < RAW_STAGES; ++s) { mbar_init(raw_full(s), 1); mbar_init(raw_empty(s), CONV_WARPS); }
    for (int b = 0; b < 2; ++b) { mbar_init(acc_full(b), 1); mbar_init(acc_empty(b), 32 * EPI_WARPS); }
    mbar_init(drain_bar, 1);
    *abort_smem = 0;
    fence_barrier_init();
    tma_prefetch_desc(&p.tmap_a);
    tma_prefetch_desc(&p.tmap_codes);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_ptr_smem), C::TMEM_COLS);
    tmem_relinquish();
  }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr_smem;
  mb_grid_dependency_sync();

  // Work items: (K slice, row tile, column tile) with the row tile fastest, so that the CTAs running together share a
  // column tile's weights in L2; every item has ks_per_split K steps.
  const uint32_t mn_tiles = p.m_tiles * p.n_tiles;
  const uint32_t total_tiles = mn_tiles * p.splits;
  const uint32_t my_tiles = blockIdx.x < total_tiles ? (total_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0u;
  const uint32_t kps = p.ks_per_split;
  const uint32_t total_steps = my_tiles * kps;          // this CTA's K steps over all its items, in order
  // item number -> (row tile, column tile, first K step)
  auto item = [&](uint32_t it, uint32_t& mt, uint32_t& nt, uint32_t& ks0) {
    const uint32_t tile = blockIdx.x + it * gridDim.x;
    uint32_t sp, mn;
    if (p.cluster_splitk) { mn = tile / p.splits; sp = tile - mn * p.splits; }      // slices of a tile side by side
    else { sp = tile / mn_tiles; mn = tile - sp * mn_tiles; }
    nt = mn / p.m_tiles;
    mt = mn - nt * p.m_tiles;
    ks0 = sp * kps;
  };

  // A cursor over this CTA's K steps in order: the divisions of item() run once per work item, not per step.
  struct Cursor {
    uint32_t it, ks, mt, nt, ks0;     // item number, step inside it, and the item's coordinates
  };
  auto cursor_at0 = [&]() {
    Cursor c{0u, 0u, 0u, 0u, 0u};
    if (my_tiles) item(0u, c.mt, c.nt, c.ks0);
    return c;
  };
  auto cursor_next = [&](Cursor& c) {
    if (++c.ks == kps) {
      c.ks = 0;
      if (++c.it < my_tiles) item(c.it, c.mt, c.nt, c.ks0);
    }
  };

  if (warp == 0) {
    // ------------------------------ producer ------------------------------------
    uint32_t op_armed = 0, op_par = 0, raw_armed = 0, raw_par = 0;
    bool ok = true;
    // the code-byte stream: step j of this CTA belongs to tile blockIdx.x + (j / k_steps) * gridDim.x
    Cursor rc = cursor_at0(), ac = rc;              // the code-byte stream's position and the A stream's
    uint32_t rj = 0, rs = 0, rph = 0;               // raw steps issued, their ring stage and phase
    auto issue_raw = [&]() -> bool {
      if (!mbar_wait(raw_empty(rs), rph ^ 1u, abort_smem, tflag, 31)) return false;
      raw_armed |= 1u << rs;
      raw_par = (raw_par & ~(1u << rs)) | (rph << rs);
      if (elect_one()) {
        mbar_arrive_expect_tx(raw_full(rs), C::RAW_BYTES);
        tma_load_2d(raw_base + rs * C::RAW_BYTES, &p.tmap_codes, int((rc.ks0 + rc.ks) * 32), int(rc.nt * BN), raw_full(rs));
      }
      __syncwarp();
      cursor_next(rc);
      ++rj;
      if (++rs == uint32_t(RAW_STAGES)) { rs = 0; rph ^= 1u; }
      return true;
    };
    while (ok && rj < uint32_t(RAW_AHEAD) && rj < total_steps) ok = issue_raw();
    uint32_t os = 0, ph = 0;
    for (uint32_t i = 0; ok && i < total_steps; ++i) {
      if (!mbar_wait(op_empty(os), ph ^ 1u, abort_smem, tflag, 32)) { ok = false; break; }
      op_armed |= 1u << os;
      op_par = (op_par & ~(1u << os)) | (ph << os);
      if (elect_one()) {
        mbar_arrive_expect_tx(op_full(os), C::A_BYTES);
        tma_load_2d(smem_base + os * C::OP_BYTES, &p.tmap_a, int((ac.ks0 + ac.ks) * BK), int(ac.mt * BM), op_full(os));
      }
      __syncwarp();
      cursor_next(ac);
      if (++os == uint32_t(C::OP_STAGES)) { os = 0; ph ^= 1u; }
      if (rj < total_steps && !issue_raw()) { ok = false; break; }
    }
    if (!ok) {
      // leave no copy in flight: a bounded wait for every raw stage this warp armed (the operand stages'
      // barriers also need the converters, which have left; their A copies land within the same bound)
      for (int s = 0; s < RAW_STAGES; ++s)
        if (raw_armed & (1u << s)) {
          const long long t0 = clock64();
          while (!mbar_try_wait(raw_full(s), (raw_par >> s) & 1u) && clock64() - t0 < WAIT_LIMIT_CYCLES) {}
        }
      const long long t0 = clock64();
      while (clock64() - t0 < 2000000LL) {}      // about a millisecond: TMA copies of 16 KB issued before the abort
      (void)op_armed; (void)op_par;
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ----------------------------------
    const uint32_t idesc = idesc_bf16(BN);
    bool ok = true;
    uint32_t i = 0;
    for (uint32_t it = 0; ok && it < my_tiles; ++it) {
      const uint32_t buf = it & 1u;
      if (!mbar_wait(acc_empty(buf), ((it >> 1) & 1u) ^ 1u, abort_smem, tflag, 33)) { ok = false; break; }
      fence_after_sync();
      const uint32_t d_tmem = tmem_base + buf * BN;
      for (uint32_t ks = 0; ks < kps; ++ks, ++i) {
        const uint32_t os = i % C::OP_STAGES, ph = (i / C::OP_STAGES) & 1u;
        if (!mbar_wait(op_full(os), ph, abort_smem, tflag, 34)) { ok = false; break; }
        fence_after_sync();
        const uint32_t sa = smem_base + os * C::OP_BYTES, sb = sa + C::A_BYTES;
        if (elect_one()) {
          const uint64_t adesc = make_kmajor_sw128_desc(sa), bdesc = make_kmajor_sw128_desc(sb);
#pragma unroll
          for (int j = 0; j < 4; ++j) mma_f16(d_tmem, adesc + 2 * j, bdesc + 2 * j, idesc, (ks | uint32_t(j)) != 0u);
          umma_commit(op_empty(os));
          if (ks + 1 == kps) umma_commit(acc_full(buf));
        }
        __syncwarp();
      }
    }
    if (!ok) {
      if (elect_one()) umma_commit(drain_bar);
      __syncwarp();
      const long long t0 = clock64();
      while (!mbar_try_wait(drain_bar, 0u) && clock64() - t0 < WAIT_LIMIT_CYCLES) {}
    }
  } else if (warp < 2 + EPI_WARPS) {
    // ------------------------------ epilogue ------------------------------------
    const uint32_t quad = uint32_t(warp) & 3u;
    uint8_t* patch = patches + (uint32_t(warp) - 2u) * 512;
    for (uint32_t it = 0; it < my_tiles; ++it) {
      uint32_t mt, nt, ks0;
      item(it, mt, nt, ks0);
      const uint32_t buf = it & 1u, sp = ks0 / kps;
      if (!mbar_wait(acc_full(buf), (it >> 1) & 1u, abort_smem, tflag, 35)) break;
      fence_after_sync();
      const uint32_t row0 = mt * BM + quad * 32u;
      const uint32_t rows_valid = row0 < p.m ? min(32u, p.m - row0) : 0u;
      const uint32_t t_acc = tmem_base + ((quad * 32u) << 16) + buf * BN;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const uint32_t col0 = nt * BN + c * 32;
        if (col0 >= p.n) break;                       // warp-uniform
        uint32_t r[32];
        tmem_ld_x32(t_acc + c * 32, r);
        tmem_ld_wait();
        if (p.cluster_splitk) {
          // This CTA's K slice: the raw sums are parked in the operand stages (idle: one item per CTA, every MMA has
          // retired) as [128 rows][BN] f32, the 16-byte units of a row XOR-ed by the row (no bank conflicts for the
          // 32 rows of a warp here, nor for the readers of the other CTAs below).
          const uint32_t trow = quad * 32u + lane;
          uint8_t* rowp = smem_gen + trow * (BN * 4);
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const uint32_t unit = uint32_t(c) * 8u + uint32_t(u);
            *reinterpret_cast<uint4*>(rowp + ((unit ^ (trow & 7u)) * 16u)) = make_uint4(r[4 * u], r[4 * u + 1], r[4 * u + 2], r[4 * u + 3]);
          }
          continue;
        }
        float v[32];
        const bool to_plane = p.splits > 1;           // a K slice: the unscaled partial sum, f32, into its plane
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = to_plane ? __uint_as_float(r[i]) : __uint_as_float(r[i]) * p.alpha;
        uint8_t* obase = to_plane ? reinterpret_cast<uint8_t*>(p.planes + size_t(sp) * p.m * p.n) : static_cast<uint8_t*>(p.out);
        if (!to_plane && p.out_dtype == MB_DT_BF16) {
          uint4 units[4];
#pragma unroll
          for (int g = 0; g < 4; ++g)
            units[g] = make_uint4(pack_bf16x2(v[8 * g], v[8 * g + 1]), pack_bf16x2(v[8 * g + 2], v[8 * g + 3]),
                                  pack_bf16x2(v[8 * g + 4], v[8 * g + 5]), pack_bf16x2(v[8 * g + 6], v[8 * g + 7]));
          uint8_t* g8 = obase + (size_t(row0) * p.n + col0) * 2;
          const uint32_t uv = (p.n - col0) / 8;
          store_rows(patch, lane, units[0], units[1], g8, size_t(p.n) * 2, rows_valid, min(2u, uv));
          if (uv > 2) store_rows(patch, lane, units[2], units[3], g8 + 32, size_t(p.n) * 2, rows_valid, min(2u, uv - 2));
        } else {
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            const uint32_t c0 = col0 + 16 * hh;
            if (c0 >= p.n) break;
            uint4 units[4];
#pragma unroll
            for (int g = 0; g < 4; ++g)
              units[g] = make_uint4(__float_as_uint(v[16 * hh + 4 * g]), __float_as_uint(v[16 * hh + 4 * g + 1]),
                                    __float_as_uint(v[16 * hh + 4 * g + 2]), __float_as_uint(v[16 * hh + 4 * g + 3]));
            uint8_t* g8 = obase + (size_t(row0) * p.n + c0) * 4;
            const uint32_t uv = (p.n - c0) / 4;
            store_rows(patch, lane, units[0], units[1], g8, size_t(p.n) * 4, rows_valid, min(2u, uv));
            if (uv > 2) store_rows(patch, lane, units[2], units[3], g8 + 32, size_t(p.n) * 4, rows_valid, min(2u, uv - 2));
          }
        }
      }
      fence_before_sync();
      mbar_arrive(acc_empty(buf));
    }
  } else {
    // ------------------------------ converters ----------------------------------
    const uint32_t ct = threadIdx.x - 32u * (2 + EPI_WARPS);          // 0 .. 511
    const uint32_t r = ct / C::TPR, part = ct % C::TPR;               // weight row of the tile, part of the row
    constexpr int BLOCKS = 4 / C::TPR;                                // 16-value blocks per thread and step: 2 or 1
    // the four scale bytes of a step come from global memory (one word per row and step); a short queue in
    // registers keeps the loads SCALE_AHEAD steps ahead of their use
    Cursor sc_cur = cursor_at0();
    uint32_t sc_j = 0;                               // steps whose scale word has been asked for
    auto scale_word = [&]() -> uint32_t {
      uint32_t w = 0u;
      if (sc_j < total_steps) {
        const uint32_t row = sc_cur.nt * BN + r;
        if (row < p.n)
          w = __ldg(reinterpret_cast<const uint32_t*>(p.scales + size_t(row) * p.sc_stride) + sc_cur.ks0 + sc_cur.ks);
        cursor_next(sc_cur);
      }
      ++sc_j;
      return w;
    };
    uint32_t sq[SCALE_AHEAD];
#pragma unroll
    for (int j = 0; j < SCALE_AHEAD; ++j) sq[j] = scale_word();
    uint32_t rs = 0, rph = 0, os = 0, oph = 0;
    for (uint32_t i = 0; i < total_steps; ++i) {
      const uint32_t sc = sq[0];
#pragma unroll
      for (int j = 0; j + 1 < SCALE_AHEAD; ++j) sq[j] = sq[j + 1];
      sq[SCALE_AHEAD - 1] = scale_word();
      if (!mbar_wait(raw_full(rs), rph, abort_smem, tflag, 36)) break;
      if (!mbar_wait(op_empty(os), oph ^ 1u, abort_smem, tflag, 37)) break;
      const uint8_t* raw = smem_gen + (raw_base - smem_base) + rs * C::RAW_BYTES + r * 32 + part * (32 / C::TPR);
      uint8_t* brow = smem_gen + os * C::OP_BYTES + C::A_BYTES + r * 128;
      uint2 codes[BLOCKS];
      if (BLOCKS == 2) {
        const uint4 lo = *reinterpret_cast<const uint4*>(raw);
        codes[0] = make_uint2(lo.x, lo.y); codes[BLOCKS - 1] = make_uint2(lo.z, lo.w);
      } else {
        codes[0] = *reinterpret_cast<const uint2*>(raw);
      }
#pragma unroll
      for (int b = 0; b < BLOCKS; ++b) {
        const uint32_t blk = part * BLOCKS + b;                         // 16-value block of the step: 0 .. 3
        uint4 c0, c1;
        decode_block(codes[b], (sc >> (8 * blk)) & 0xFFu, c0, c1);
        *reinterpret_cast<uint4*>(brow + (((2 * blk) ^ (r & 7u)) << 4)) = c0;
        *reinterpret_cast<uint4*>(brow + (((2 * blk + 1) ^ (r & 7u)) << 4)) = c1;
      }
      fence_proxy_async();          // the tensor core reads these bytes through the asynchronous proxy
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(op_full(os));
        mbar_arrive(raw_empty(rs));
      }
      if (++rs == uint32_t(RAW_STAGES)) { rs = 0; rph ^= 1u; }
      if (++os == uint32_t(C::OP_STAGES)) { os = 0; oph ^= 1u; }
    }
  }

  if (p.cluster_splitk) {
    // ------------------------------ K slices meet ------------------------------------
    // Every thread of every CTA of the cluster comes here, also after a wait that ran out. CTA r adds the 32-column
    // chunks r, r + splits, ... over the slices in slice order (the order of the stand-alone sum of planes: the same
    // bits), times alpha, one cast.
    cluster_sync_unaligned();
    if (warp >= 2 && warp < 2 + EPI_WARPS && *abort_smem == 0 && blockIdx.x < total_tiles) {
      const uint32_t e = (uint32_t(warp) - 2u) * 32u + lane, rank = cluster_ctarank();
      uint32_t mt, nt, ks0;
      item(0u, mt, nt, ks0);
      const uint32_t m_valid = min(uint32_t(BM), p.m - mt * BM);
      const uint32_t tile_s = smem_u32(smem_gen);
      for (uint32_t c = rank; c < uint32_t(BN / 32); c += p.splits) {
        const uint32_t col = nt * BN + c * 32u + (e & 7u) * 4u;
        if (col >= p.n) continue;
        for (uint32_t row = e >> 3; row < m_valid; row += 32u * EPI_WARPS / 8u) {
          const uint32_t unit = c * 8u + (e & 7u);
          const uint32_t addr = tile_s + row * (BN * 4) + ((unit ^ (row & 7u)) * 16u);
          float4 v[8];
#pragma unroll
          for (uint32_t sl = 0; sl < 8; ++sl)
            if (sl < p.splits) v[sl] = ld_cluster_f32x4(map_to_cta(addr, sl));
          float4 acc = v[0];
#pragma unroll
          for (uint32_t sl = 1; sl < 8; ++sl)
            if (sl < p.splits) { acc.x += v[sl].x; acc.y += v[sl].y; acc.z += v[sl].z; acc.w += v[sl].w; }
          const size_t o = (size_t(mt) * BM + row) * p.n + col;
          if (p.out_dtype == MB_DT_F32)
            *reinterpret_cast<float4*>(static_cast<float*>(p.out) + o) =
                make_float4(acc.x * p.alpha, acc.y * p.alpha, acc.z * p.alpha, acc.w * p.alpha);
          else
            *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(p.out) + o) =
                make_uint2(pack_bf16x2(acc.x * p.alpha, acc.y * p.alpha), pack_bf16x2(acc.z * p.alpha, acc.w * p.alpha));
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
}

// Sum of the K-slice planes in slice order (deterministic), times scale2, one cast.
template <typename O>
__global__ void __launch_bounds__(256)
w4a16_splitk_reduce_kernel(const float4* __restrict__ planes, uint32_t splits, size_t plane4, float alpha, O* __restrict__ out) {
  mb_grid_dependency_sync();
  const size_t i = size_t(blockIdx.x) * 256 + threadIdx.x;
  if (i >= plane4) return;
  float4 acc = planes[i];
  for (uint32_t s = 1; s < splits; ++s) {
    const float4 v = planes[size_t(s) * plane4 + i];
    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
  }
  if (sizeof(O) == 4) reinterpret_cast<float4*>(out)[i] = make_float4(acc.x * alpha, acc.y * alpha, acc.z * alpha, acc.w * alpha);
  else reinterpret_cast<uint2*>(out)[i] = make_uint2(pack_bf16x2(acc.x * alpha, acc.y * alpha), pack_bf16x2(acc.z * alpha, acc.w * alpha));
}

// K slices for a product whose output tiles would leave most SMs idle while the weights stream: the largest
// divisor of the K steps that keeps tiles x slices within the SMs and at least eight steps per slice (1 = no split).
uint32_t w4a16_splits(int sm_count, size_t m, size_t n, size_t k) {
  if (n % 4 != 0) return 1;
  const uint32_t tiles = uint32_t((m + BM - 1) / BM) * uint32_t((n + 127) / 128);
  const uint32_t k_steps = uint32_t(k / BK);
  if (tiles * 2 > uint32_t(sm_count) || k_steps < 16) return 1;
  const uint32_t want = std::min<uint32_t>(uint32_t(sm_count) / tiles, k_steps / 8);
  uint32_t best = 1;
  for (uint32_t s = 2; s <= want; ++s)
    if (k_steps % s == 0) best = s;
  return best;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int encoder(mb_ctx* ctx, EncodeTiledFn* fn) {
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

template <int BN>
int launch(mb_ctx* ctx, cudaStream_t stream, const W4a16Params& p) {
  using C = Cfg<BN>;
  constexpr uint32_t bit = BN == 256 ? MB_ONCE_GEMM_W4A16_256 : MB_ONCE_GEMM_W4A16_128;
  if (!mb_once(ctx, bit)) {
    MB_CUDA_OK(ctx, cudaFuncSetAttribute(gemm_w4a16_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
    mb_once_done(ctx, bit);
  }
  const int sms = ctx->sm_limit > 0 ? std::min(ctx->sm_limit, ctx->sm_count) : ctx->sm_count;
  const unsigned grid = std::min<uint32_t>(p.m_tiles * p.n_tiles * p.splits, uint32_t(sms));
  MB_CUDA_OK(ctx, mb_launch_pdl(gemm_w4a16_kernel<BN>, dim3(grid), dim3(THREADS), C::SMEM_BYTES, stream, p));
  MB_LAUNCH_OK(ctx);
  return MB_OK;
}

}  // namespace

MB_API size_t mb_nvfp4_gemm_w4a16_workspace(size_t m, size_t n, size_t k) {
  if (k == 0 || k % 64 != 0) return 0;
  const uint32_t sp = w4a16_splits(148, m, n, k);
  return sp > 1 ? size_t(sp) * m * n * sizeof(float) : 0;
}

MB_API int mb_nvfp4_gemm_w4a16(mb_ctx* ctx, mb_stream stream_, const void* x_bf16, const uint8_t* codes,
                               const uint8_t* scales_rowmajor, float scale2, size_t m, size_t n, size_t k, void* out,
                               int out_dtype, void* workspace, size_t workspace_bytes) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  MB_REQUIRE(ctx, ctx && x_bf16 && codes && scales_rowmajor && out, "gemm_w4a16: null argument");
  MB_REQUIRE(ctx, m > 0 && n > 0 && k > 0, "gemm_w4a16: empty extent");
  MB_REQUIRE(ctx, k % 64 == 0, "W4A16 prompt projection needs k a multiple of 64, got %zu", k);
  MB_REQUIRE(ctx, n % 8 == 0, "NVFP4 prompt projection needs n a multiple of 8, got %zu", n);
  MB_REQUIRE(ctx, m * k <= 0xFFFFFFFFull && n * k <= 0xFFFFFFFFull, "gemm_w4a16: exceeds u32 indexing");
  MB_REQUIRE(ctx, out_dtype == MB_DT_BF16 || out_dtype == MB_DT_F32, "gemm_w4a16: output is bf16 or f32");
  MB_REQUIRE(ctx, scale2 == scale2 && scale2 > 0.0f && scale2 <= 3.4e38f,
             "NVFP4 global scale %g is not a positive finite number", double(scale2));
  MB_REQUIRE(ctx, mb_aligned(x_bf16, 16) && mb_aligned(codes, 16) && mb_aligned(scales_rowmajor, 4) && mb_aligned(out, 16),
             "gemm_w4a16: activation, codes and output need 16-byte alignment, scales 4-byte");
  MB_REQUIRE_DEVICE(ctx, "gemm_w4a16");
  EncodeTiledFn enc;
  int rc = encoder(ctx, &enc);
  if (rc) return rc;
  W4a16Params p;
  memset(&p, 0, sizeof p);
  // few row tiles leave column tiles as the only parallelism: narrower column tiles then fill more SMs
  const size_t m_tiles = (m + BM - 1) / BM;
  const bool wide = n % 256 == 0 && m_tiles * (n / 256) >= size_t(ctx->sm_count);
  const uint32_t bn = wide ? 256u : 128u;
  {
    cuuint64_t dims[2] = {k, m};
    cuuint64_t strides[1] = {k * 2};
    cuuint32_t box[2] = {64u, uint32_t(BM)}, estr[2] = {1, 1};
    CUresult r = enc(&p.tmap_a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(x_bf16), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return mb_fail(ctx, MB_ERR_CUDA, "cuTensorMapEncodeTiled (activation) failed with %d", int(r));
  }
  {
    cuuint64_t dims[2] = {k / 2, n};
    cuuint64_t strides[1] = {k / 2};
    cuuint32_t box[2] = {32u, bn}, estr[2] = {1, 1};
    CUresult r = enc(&p.tmap_codes, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(codes), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return mb_fail(ctx, MB_ERR_CUDA, "cuTensorMapEncodeTiled (codes) failed with %d", int(r));
  }
  p.scales = scales_rowmajor; p.out = out; p.flags = ctx->flags_dev; p.alpha = scale2;
  p.m = uint32_t(m); p.n = uint32_t(n); p.k_steps = uint32_t(k / BK);
  p.m_tiles = uint32_t(m_tiles); p.n_tiles = uint32_t((n + bn - 1) / bn);
  p.sc_stride = uint32_t(k / 16);
  p.out_dtype = out_dtype;
  p.splits = 1; p.ks_per_split = p.k_steps;
  const uint32_t sp = wide ? 1u : w4a16_splits(ctx->sm_count, m, n, k);
  if (sp > 1 && sp <= 8) {
    // the K slices of a tile as one cluster, summed in shared memory, when every tile's cluster is resident at once
    // (MB_SPLITK_CLUSTER=0 in the environment keeps the planes below; read per call)
    const char* env = getenv("MB_SPLITK_CLUSTER");
    const uint32_t tiles = p.m_tiles * p.n_tiles;
    const int sms = ctx->sm_limit > 0 ? std::min(ctx->sm_limit, ctx->sm_count) : ctx->sm_count;
    if (!(env && env[0] == '0') && tiles * sp <= uint32_t(sms)) {
      if (!mb_once(ctx, MB_ONCE_GEMM_W4A16_128)) {
        MB_CUDA_OK(ctx, cudaFuncSetAttribute(gemm_w4a16_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<128>::SMEM_BYTES));
        mb_once_done(ctx, MB_ONCE_GEMM_W4A16_128);
      }
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(tiles * sp);
      cfg.blockDim = dim3(THREADS);
      cfg.dynamicSmemBytes = Cfg<128>::SMEM_BYTES;
      cfg.stream = stream;
      cudaLaunchAttribute attr[2];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = sp; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
      attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attr[1].val.programmaticStreamSerializationAllowed = 1;
      cfg.attrs = attr;
      int& held = ctx->w4a16_clusters[sp];
      if (held == 0) {
        cfg.numAttrs = 1;
        int nc = 0;
        if (cudaOccupancyMaxActiveClusters(&nc, gemm_w4a16_kernel<128>, &cfg) != cudaSuccess) { (void)cudaGetLastError(); nc = 0; }
        held = nc >= 1 ? nc : -1;
      }
      if (held > 0 && tiles <= uint32_t(held)) {
        p.splits = sp; p.ks_per_split = p.k_steps / sp; p.cluster_splitk = 1;
        cfg.numAttrs = mb_pdl_enabled() ? 2 : 1;
        MB_CUDA_OK(ctx, cudaLaunchKernelEx(&cfg, gemm_w4a16_kernel<128>, p));
        MB_LAUNCH_OK(ctx);
        return MB_OK;
      }
    }
  }
  if (sp > 1 && workspace && workspace_bytes >= size_t(sp) * m * n * sizeof(float)) {
    MB_REQUIRE(ctx, mb_aligned(workspace, 16), "gemm_w4a16: workspace needs 16-byte alignment");
    p.splits = sp; p.ks_per_split = p.k_steps / sp;
    p.planes = static_cast<float*>(workspace);
    rc = launch<128>(ctx, stream, p);
    if (rc) return rc;
    const size_t plane4 = m * n / 4;
    const unsigned grid = unsigned((plane4 + 255) / 256);
    if (out_dtype == MB_DT_F32)
      MB_CUDA_OK(ctx, mb_launch_pdl(w4a16_splitk_reduce_kernel<float>, dim3(grid), dim3(256), 0, stream,
                                    static_cast<const float4*>(workspace), sp, plane4, scale2, static_cast<float*>(out)));
    else
      MB_CUDA_OK(ctx, mb_launch_pdl(w4a16_splitk_reduce_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, stream,
                                    static_cast<const float4*>(workspace), sp, plane4, scale2,
                                    static_cast<__nv_bfloat16*>(out)));
    MB_LAUNCH_OK(ctx);
    return MB_OK;
  }
  return wide ? launch<256>(ctx, stream, p) : launch<128>(ctx, stream, p);
}
