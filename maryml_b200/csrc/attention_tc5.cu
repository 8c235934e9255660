// Causal GQA prefill attention on the sm_100a tensor cores (tcgen05 + TMEM), head_dim 128.
//
// One CTA owns 256 query rows of one head as two 128-row tiles. Per 128-key tile:
//
//   S_t  = Q_t K^T      tcgen05.mma kind::f16, 128 x 128 x 128, accumulator in TMEM
//   P_t  = 2^(S_t*c - m) one softmax thread per query row reads its row of S_t from
//                        TMEM (no cross-thread reduction) and writes bf16 P_t back over
//                        the first 64 columns of the same score buffer (tcgen05.st)
//   O_t += P_t V         tcgen05.mma with the A operand in TMEM, 128 x 128 x 128, V read
//                        MN-major straight from the TMA tile; O_t stays in TMEM over the
//                        whole key loop
//
// Why these shapes. Per-phase cycle counters of the 64-key version showed the MMA warp busy
// issuing 1.7 k of the 2.1 k cycles a tile took: a 128 x 64 score instruction occupies the tensor
// pipe as long as a 128 x 128 one, so the score products ran at half rate; 128-key tiles make
// every instruction 128 x 128. P lives in tensor memory because shared-memory bandwidth is
// the next limit (a P tile in shared memory is written once and read once per tile, on top of
// the Q re-read of every score product, the V read and the TMA fill).
//
// TMEM: S0, S1 (128 columns each), PV0, PV1 (128 each) = 512. One score buffer per query tile:
// the issuer sends PV(t, j) and then S(t, j + 1) as soon as group t publishes P(t, j), and the
// tensor core works for the other group while group t exponentiates (the two groups alternate).
//
// The running maximum a row subtracts may lag the true one: a probability of 2^40 is as exact in bf16 P and in the
// f32 sums as one of 1 (P, O_t and l scale together; O_t / l is exact either way). After the first tile no maximum
// is tracked at all; the sum of a row's probabilities tells when a score has outgrown the subtracted maximum by 2^40
// or more, and only then are the tile's maxima found and O_t in TMEM rescaled (tcgen05.ld, multiply, tcgen05.st).
//
// Warp roles: 0 = TMA producer (Q once, a ring of two K tiles and a ring of two V tiles),
// 1 = MMA issuer, 2-9 and 10-17 = the two softmax groups (one per query tile). A row of 128 scores is shared by
// two threads (warps w and w + 4 of a group take columns 0-63 and 64-127 of the same TMEM lanes): the chain
// load -> exponentials -> store of one thread per row was the longest link of the pipeline, and two warps
// per scheduler and group hide each other's latencies. The pair swaps its maxima through shared memory.
// Algorithmic work: 4 * nq * keys * 128 flop per head, half under the mask.
// Every mbarrier wait is bounded.
#include "attention.cuh"

namespace {

using namespace tc5;

constexpr int D = 128;
constexpr int BC = 128;                        // keys per tile
constexpr int BOX = 64;                        // key rows of one TMA box (the tensor maps are shared with the decode kernel)
constexpr int QT = 128;                        // query rows per tile (two tiles per CTA)
constexpr int HALF = BC * 128;                 // one 64-dim half of a K or V tile: 16 KB
constexpr int TILE = 2 * HALF;                 // a K tile or a V tile: 32 KB
constexpr int KSTAGES = 2, VSTAGES = 2;
constexpr int Q_BYTES = 2 * QT * D * 2;        // 64 KB: [tile][half][128 rows][64 dims]
constexpr int XCHG_BYTES = 2 * 2 * 2 * 128 * 4; // row maxima (later row sums) the two threads of a row swap: [phase parity][tile][part][row]
constexpr int SMEM = (KSTAGES + VSTAGES) * TILE + Q_BYTES + XCHG_BYTES + 1024 + 256;
constexpr int THREADS = 576;                   // producer, issuer, two softmax groups of eight warps
constexpr int S_COL0 = 0, S_COL1 = 128, PV_COL0 = 256, PV_COL1 = 384, TMEM_COLS = 512;

// Development aid (-DMB_ATTN_PROFILE): cycles per phase, summed over CTAs. Slots: 12 / 13 / 14 issuer waits for the first
// K tile / a V tile / the next K tile (issuing time in between lands in the slot after it), 1 issuer waits
// P of tile 0, 2 issuer waits P of tile 1, 3 whole kernel, 4 key tiles; first warp of softmax group 0: 5 waits scores,
// 6 score load + maximum, 8 exponentials, 9 P store, 10 waits PV, 11 rescales taken.
#ifdef MB_ATTN_PROFILE
__device__ unsigned long long g_attn_prof[16];
#define APROF_T0() long long aprof_t0_ = clock64()
#define APROF_LAP(slot) do { const long long n_ = clock64(); if ((threadIdx.x & 31) == 0) atomicAdd(&g_attn_prof[slot], (unsigned long long)(n_ - aprof_t0_)); aprof_t0_ = n_; } while (0)
#define APROF_COUNT(slot) do { if ((threadIdx.x & 31) == 0) atomicAdd(&g_attn_prof[slot], 1ull); } while (0)
#else
#define APROF_T0() do {} while (0)
#define APROF_LAP(slot) do {} while (0)
#define APROF_COUNT(slot) do {} while (0)
#endif

// bf16 A and B, f32 accumulate, M = 128; B either K-major (0) or MN-major (1).
__host__ __device__ constexpr uint32_t idesc(uint32_t n, uint32_t b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn_major << 16) | ((n >> 3) << 17) | ((128u >> 4) << 24);
}
// V tile [64 keys][128 dims] as two 64-dim halves of 128-byte rows: MN-major operand with
// 8 KB between the 64-element MN blocks (leading offset) and 1 KB between 8-key groups.
__device__ __forceinline__ uint64_t make_v_desc(uint32_t saddr) {
  return make_smem_desc(saddr, HALF, 1024, LAYOUT_SWIZZLE_128B);
}

__device__ __forceinline__ float ex2(float x) {
#ifdef MB_ATTN_NOEXP   // timing experiment only: what the kernel costs without the special-function unit (wrong results)
  return x * 0.001f + 0.01f;
#else
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
#endif
}
// Two-lane f32 arithmetic of sm_100 (each lane an IEEE round-to-nearest op): half the issue slots of the scalar forms.
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 f2_pack(float a, float b) {
  f32x2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ void f2_unpack(f32x2 v, float& a, float& b) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ f32x2 f2_fma(f32x2 a, f32x2 b, f32x2 c) {
  f32x2 r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ f32x2 f2_add(f32x2 a, f32x2 b) {
  f32x2 r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__global__ void __launch_bounds__(THREADS, 1)
attn_prefill_tc5_kernel(const __grid_constant__ AttnParams p) {
#ifdef MB_ATTN_PROFILE
  const long long aprof_k0 = clock64();
#endif
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t k_smem = base, v_smem = base + KSTAGES * TILE;
  const uint32_t q_smem = v_smem + VSTAGES * TILE;
  float* xchg = reinterpret_cast<float*>(gen + (q_smem - base) + Q_BYTES);
  const uint32_t bar_base = q_smem + Q_BYTES + XCHG_BYTES;
  // barriers: k_full[2], k_empty[2], v_full[2], v_empty[2], q_full, s_full[2], p_full[2], pv_done[2], drain, pair[2][4]
  auto k_full = [&](int s) { return bar_base + 8u * s; };
  auto k_empty = [&](int s) { return bar_base + 8u * (KSTAGES + s); };
  auto v_full = [&](int s) { return bar_base + 8u * (2 * KSTAGES + s); };
  auto v_empty = [&](int s) { return bar_base + 8u * (2 * KSTAGES + VSTAGES + s); };
  constexpr int NB = 2 * KSTAGES + 2 * VSTAGES;
  const uint32_t q_full = bar_base + 8u * NB;
  auto s_full = [&](int t) { return bar_base + 8u * (NB + 1 + t); };
  auto p_full = [&](int t) { return bar_base + 8u * (NB + 3 + t); };
  auto pv_done = [&](int t) { return bar_base + 8u * (NB + 5 + t); };
  const uint32_t drain_bar = bar_base + 8u * (NB + 7);
  auto pair_bar = [&](int t, uint32_t quad) { return bar_base + 8u * (NB + 8 + 4 * t + quad); };   // the two warps of a row set
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(gen + (bar_base - base) + 8 * (NB + 16));
  volatile int* abort_smem = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);
  int* tflag = p.flags ? p.flags + MB_FLAG_WAIT_TIMEOUT : nullptr;

  const int warp = __shfl_sync(0xFFFFFFFFu, int(threadIdx.x >> 5), 0);
  const uint32_t lane = threadIdx.x & 31;
  // Blocks start in the order of their linear index. Within a sequence the heaviest (latest) query blocks of ALL
  // heads go first and the lightest last, so that the kernel's tail is made of blocks of a tile or two instead of a
  // late head's 64-tile block; heads run fastest (the four query heads of a KV head side by side), and a sequence's
  // K and V (33 MB at 8192 keys) stay in L2 while all its heads pass over them. MB_ATTN_ORDER=0: head-major.
#ifndef MB_ATTN_ORDER
#define MB_ATTN_ORDER 1
#endif
#if MB_ATTN_ORDER
  const uint32_t lin = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
  const uint32_t per_seq = gridDim.x * gridDim.y, in_seq = lin % per_seq;
  const uint32_t qb = gridDim.x - 1 - in_seq / gridDim.y, h = in_seq % gridDim.y, b = lin / per_seq;
#else
  const uint32_t qb = gridDim.x - 1 - blockIdx.x, h = blockIdx.y, b = blockIdx.z;
#endif
  const uint32_t kvh = h / (p.heads / p.kv_heads);
  const uint32_t q_row0 = qb * 2 * QT;
  const uint32_t q_rows = min(uint32_t(2 * QT), p.nq - q_row0);
  const uint32_t last_q = p.q0 + q_row0 + q_rows - 1;
  const uint32_t k_end = p.causal ? min(p.keys, last_q + 1) : p.keys;
  // with a sliding window the block's first query row bounds the keys from below: whole tiles under it are skipped
  const uint32_t first_q = p.q0 + q_row0;
  const uint32_t j_start = (p.window && first_q + 1 > p.window) ? (first_q + 1 - p.window) / BC : 0u;
  const uint32_t n_tiles = (k_end + BC - 1) / BC - j_start;   // >= 1: the window holds at least the row's own key

  if (threadIdx.x == 0) {
    for (int s = 0; s < KSTAGES; ++s) { mbar_init(k_full(s), 1); mbar_init(k_empty(s), 1); }
    for (int s = 0; s < VSTAGES; ++s) { mbar_init(v_full(s), 1); mbar_init(v_empty(s), 1); }
    mbar_init(q_full, 1);
    for (int t = 0; t < 2; ++t) {
      mbar_init(s_full(t), 1);
      mbar_init(p_full(t), 256);
      mbar_init(pv_done(t), 1);
      for (uint32_t q = 0; q < 4; ++q) mbar_init(pair_bar(t, q), 64);
    }
    mbar_init(drain_bar, 1);
    *abort_smem = 0;
    fence_barrier_init();
    tma_prefetch_desc(&p.tmap_q);
    tma_prefetch_desc(&p.tmap_k);
    tma_prefetch_desc(&p.tmap_v);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_ptr_smem), TMEM_COLS);
    tmem_relinquish();
  }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr_smem;

  if (warp == 0) {
    // ------------------------------ producer ------------------------------------
    if (elect_one()) {
      mbar_arrive_expect_tx(q_full, Q_BYTES);
#pragma unroll
      for (int t = 0; t < 2; ++t)
#pragma unroll
        for (int hf = 0; hf < 2; ++hf)
          tma_load_4d(q_smem + (t * 2 + hf) * (QT * 128), &p.tmap_q, hf * 64, int(h), int(q_row0 + t * QT), int(b), q_full);
    }
    __syncwarp();
    // A tile of 128 keys is four boxes: [64-dim half][64-key box]; K(0), then V(j) and K(j + 1) alternate.
    auto load_tile = [&](const CUtensorMap* tm, uint32_t dst, uint32_t j, uint32_t bar) {
      if (elect_one()) {
        mbar_arrive_expect_tx(bar, TILE);
#pragma unroll
        for (int hf = 0; hf < 2; ++hf)
#pragma unroll
          for (int bx = 0; bx < 2; ++bx)
            tma_load_4d(dst + hf * HALF + bx * (BOX * 128), tm, hf * 64, int(kvh), int((j + j_start) * BC + bx * BOX), int(b), bar);
      }
      __syncwarp();
    };
    bool ok = true;
    for (uint32_t i = 0; ok && i <= n_tiles; ++i) {
      if (i < n_tiles) {                                   // K(i)
        const int st = int(i % KSTAGES);
        if (!mbar_wait(k_empty(st), ((i / KSTAGES) & 1u) ^ 1u, abort_smem, tflag, 31)) {
          if (tflag && lane == 0) atomicCAS(tflag + 7, 0, int(i | n_tiles << 10 | (p.q0 >> 6) << 20));
          ok = false;
          break;
        }
        load_tile(&p.tmap_k, k_smem + st * TILE, i, k_full(st));
      }
      if (i > 0) {                                         // V(i - 1)
        const uint32_t j = i - 1;
        const int st = int(j % VSTAGES);
        if (!mbar_wait(v_empty(st), ((j / VSTAGES) & 1u) ^ 1u, abort_smem, tflag, 30)) { ok = false; break; }
        load_tile(&p.tmap_v, v_smem + st * TILE, j, v_full(st));
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ----------------------------------
    // S(0, 0), S(1, 0); then per key tile and query tile: wait for P(t, j), issue O_t += P V(j) and at once
    // S(t, j + 1) into the same score buffer (the tensor core runs its instructions in issue order, so the
    // scores overwrite P only after the PV product has read it).
    bool ok = mbar_wait(q_full, 0u, abort_smem, tflag, 32);
    const uint32_t id_s = idesc(BC, 0), id_pv = idesc(D, 1);
    uint32_t mma_where = 0, mma_j = 0;     // the wait the issuer was in, for the status block of a run-out wait
    auto issue_s = [&](int t, uint32_t j) {                // K(j) is resident
      if (elect_one()) {
        const uint32_t k0 = k_smem + (j % KSTAGES) * TILE;
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          const uint64_t adesc = make_kmajor_sw128_desc(q_smem + (t * 2 + hf) * (QT * 128));
          const uint64_t bdesc = make_kmajor_sw128_desc(k0 + hf * HALF);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            mma_f16(tmem_base + (t ? S_COL1 : S_COL0), adesc + 2 * kk, bdesc + 2 * kk, id_s, (hf | kk) != 0);
        }
        umma_commit(s_full(t));
        if (t == 1) umma_commit(k_empty(int(j % KSTAGES)));   // both query tiles have their scores of K(j)
      }
      __syncwarp();
    };
    if (ok) {
      mma_where = 33;
      APROF_T0();
      ok = mbar_wait(k_full(0), 0u, abort_smem, tflag, 33);
      APROF_LAP(12);
      if (ok) {
        fence_after_sync();
        issue_s(0, 0);
        issue_s(1, 0);
      }
    }
    for (uint32_t j = 0; ok && j < n_tiles; ++j) {
      mma_j = j;
      APROF_COUNT(4);
      const int vst = int(j % VSTAGES);
      for (int t = 0; t < 2 && ok; ++t) {
        mma_where = 34 + 64 * t;
        APROF_T0();
        if (!mbar_wait(p_full(t), j & 1u, abort_smem, tflag, 34)) { ok = false; break; }
        APROF_LAP(1 + t);
        if (t == 0) {
          mma_where = 35;
          if (!mbar_wait(v_full(vst), (j / VSTAGES) & 1u, abort_smem, tflag, 35)) { ok = false; break; }
          APROF_LAP(13);
        }
        fence_after_sync();
        if (elect_one()) {
          const uint32_t a_tmem = tmem_base + (t ? S_COL1 : S_COL0);      // P_t(j): 64 columns of bf16 pairs
          const uint64_t bdesc = make_v_desc(v_smem + vst * TILE);
#pragma unroll
          for (int kk = 0; kk < BC / 16; ++kk)            // 16 keys per instruction: 8 columns of P, 16 rows of V
            mma_f16_ts(tmem_base + (t ? PV_COL1 : PV_COL0), a_tmem + 8 * kk, bdesc + 128 * kk, id_pv, (j | uint32_t(kk)) != 0u);
          umma_commit(pv_done(t));
          if (t == 1) umma_commit(v_empty(vst));          // both query tiles are done with V(j)
        }
        __syncwarp();
        if (j + 1 < n_tiles) {
          if (t == 0) {
            mma_where = 33;
            if (!mbar_wait(k_full(int((j + 1) % KSTAGES)), ((j + 1) / KSTAGES) & 1u, abort_smem, tflag, 33)) { ok = false; break; }
            APROF_LAP(14);
            fence_after_sync();
          }
          issue_s(t, j + 1);
        }
      }
    }
    if (!ok) {
      if (tflag && lane == 0) atomicCAS(tflag + 5, 0, int(1u << 30 | mma_where << 20 | mma_j));
      if (elect_one()) umma_commit(drain_bar);
      __syncwarp();
      long long t0 = clock64();
      while (!mbar_try_wait(drain_bar, 0u) && clock64() - t0 < WAIT_LIMIT_CYCLES) {}
    }
  } else {
    // ------------------------------ softmax groups -------------------------------
    const int t = (warp - 2) >> 3;                        // query tile of this group
    const uint32_t part = uint32_t(warp - 2) >> 2 & 1u;   // which 64 of the row's 128 scores this thread takes
    const uint32_t quad = warp & 3u;                      // TMEM lane quadrant of this warp
    const uint32_t r = quad * 32u + lane;                 // row within the tile
    const uint32_t row = q_row0 + t * QT + r;             // row within the sequence's queries
    const int qpos = int(p.q0 + row);
    const uint32_t lane_addr = (quad * 32u) << 16;
    const uint32_t t_s = tmem_base + lane_addr + (t ? S_COL1 : S_COL0) + part * 64;     // this thread's scores
    const uint32_t t_p = tmem_base + lane_addr + (t ? S_COL1 : S_COL0) + part * 32;     // and where its P goes
    const uint32_t t_pv = tmem_base + lane_addr + (t ? PV_COL1 : PV_COL0) + part * 64;  // its half of the output columns
    float* x_mine = xchg + (t * 2 + part) * 128 + r;
    const float* x_other = xchg + (t * 2 + (part ^ 1u)) * 128 + r;
    float m = -INFINITY, l = 0.0f;       // m: the maximum this row currently subtracts (may lag, see header); l: this thread's part of the row sum
    uint32_t xph = 0;                    // phase of the pair barrier
    bool ok = true;
    uint32_t sm_where = 0, sm_j = 0;
    // the pair's hand-shake: both threads of a row have published a value and finished their score loads
    // (two slots by phase parity: a slot is rewritten only after the partner has arrived for the phase in between,
    // which it does after reading)
    auto swap = [&](float mine) -> float {
      const uint32_t slot = (xph & 1u) * (2 * 2 * 128);
      x_mine[slot] = mine;
      mbar_arrive(pair_bar(t, quad));
      sm_where = 42;
      if (!mbar_wait(pair_bar(t, quad), xph & 1u, abort_smem, tflag, 42)) { ok = false; return mine; }
      ++xph;
      return x_other[slot];
    };
    for (uint32_t j = 0; ok && j < n_tiles; ++j) {
      sm_j = j;
      const int kabs = int((j + j_start) * BC + part * 64);
      int vis = int(p.keys) - kabs;
      if (p.causal) vis = min(vis, qpos + 1 - kabs);
      const int first = p.window ? qpos + 1 - int(p.window) - kabs : 0;   // keys [first, vis) of this thread's 64 are visible
      bool pv_waited = j == 0;           // whether PV(j-1) is known to be complete
      const bool full_tile = __all_sync(0xFFFFFFFFu, vis >= 64 && first <= 0);   // no mask work away from the band's edges
      sm_where = 37;
#ifdef MB_ATTN_PROFILE
      long long aprof_t0_ = clock64();
      const bool aprof_on = warp == 2;
#define SPROF(slot) do { if (aprof_on) APROF_LAP(slot); } while (0)
#else
#define SPROF(slot) do {} while (0)
#endif
      if (!mbar_wait(s_full(t), j & 1u, abort_smem, tflag, 37)) { ok = false; break; }
      SPROF(5);
      fence_after_sync();
      // One pass in the common case: the probabilities are taken against the maximum the row already
      // subtracts (it may lag the true one, see the header); P stays in registers until the pair knows from the
      // sums that the maximum is within reach.
      uint32_t w[32];
      float sum = 0.0f;
      auto probabilities = [&]() {
        const float neg_m = m == -INFINITY ? -INFINITY : -m;      // a row with nothing visible so far gives p = 0
        const f32x2 c2 = f2_pack(p.scale_log2, p.scale_log2), nm2 = f2_pack(neg_m, neg_m);
        f32x2 acc0 = f2_pack(0.0f, 0.0f), acc1 = acc0;           // two running pairs of partial row sums
        auto half = [&](const uint32_t* s, int q) {
          if (full_tile) {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const float s0 = __uint_as_float(s[2 * i]), s1 = __uint_as_float(s[2 * i + 1]);
              float x0, x1;
              f2_unpack(f2_fma(f2_pack(s0, s1), c2, nm2), x0, x1);
              const float p0 = ex2(x0), p1 = ex2(x1);
              if (i & 1) acc1 = f2_add(acc1, f2_pack(p0, p1)); else acc0 = f2_add(acc0, f2_pack(p0, p1));
              w[q * 16 + i] = pack2(p0, p1);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const float s0 = __uint_as_float(s[2 * i]), s1 = __uint_as_float(s[2 * i + 1]);
              const int i0 = q * 32 + 2 * i, i1 = i0 + 1;
              const bool v0 = i0 < vis && i0 >= first, v1 = i1 < vis && i1 >= first;
              const float p0 = v0 ? ex2(fmaf(s0, p.scale_log2, neg_m)) : 0.0f;
              const float p1 = v1 ? ex2(fmaf(s1, p.scale_log2, neg_m)) : 0.0f;
              acc0 = f2_add(acc0, f2_pack(p0, p1));
              w[q * 16 + i] = pack2(p0, p1);
            }
          }
        };
        uint32_t sa[32], sb[32];
        tmem_ld_x32(t_s, sa);
        tmem_ld_x32(t_s + 32, sb);
        tmem_ld_wait();
        half(sa, 0);
        half(sb, 1);
        float a0, a1, b0, b1;
        f2_unpack(acc0, a0, a1);
        f2_unpack(acc1, b0, b1);
        sum = (a0 + a1) + (b0 + b1);
      };
      auto row_maximum = [&]() -> float {      // over this thread's visible scores of the tile
        float mx = -INFINITY;
        uint32_t sa[32], sb[32];
        tmem_ld_x32(t_s, sa);
        tmem_ld_x32(t_s + 32, sb);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          if (full_tile || (i < vis && i >= first)) mx = fmaxf(mx, __uint_as_float(sa[i]));
          if (full_tile || (32 + i < vis && 32 + i >= first)) mx = fmaxf(mx, __uint_as_float(sb[i]));
        }
        return mx;
      };
      if (j == 0) {
        // first tile: the row maximum first (this thread's 64 scores, then the partner's), then the probabilities
        const float mx = row_maximum();
        const float other = swap(mx);
        if (!ok) break;
        m = fmaxf(mx, other) * p.scale_log2;
        SPROF(6);
        probabilities();
        // the partner may store its P over columns this thread has just read a second time: one more hand-shake
        (void)swap(0.0f);
        if (!ok) break;
      } else {
        // No maximum is tracked here: the probabilities are taken against the maximum the row already subtracts,
        // and their sum tells whether that is still good. A score more than 2^40 above the maximum (in the exponent's
        // units) makes the pair's sums exceed 2^40, or not a number; such a row, and a row that has seen no key yet,
        // looks for its maximum in a second pass (rare: after its first tiles a row's maximum hardly moves, and
        // anything up to 2^40 is as exact in bf16 P and f32 O, l as 1 is, since all three scale together).
        probabilities();
        const float other = swap(sum);        // also: both threads are past their score loads
        if (!ok) break;
        const bool grown = !(fmaxf(sum, other) <= 1099511627776.0f) || m == -INFINITY;
        if (__any_sync(0xFFFFFFFFu, grown)) {
#ifdef MB_ATTN_PROFILE
          if (aprof_on) APROF_COUNT(11);
#endif
          // some row of this warp pair outgrew its maximum (both warps see the same sums and decide alike):
          // find the tile's maxima, bring this thread's half of O_t, and l, to the new maxima and take the
          // probabilities again (the scores are still in place: no P has been stored yet)
          const float mx = row_maximum();
          const float omx = swap(mx);
          if (!ok) break;
          const float mt = fmaxf(mx, omx) * p.scale_log2;
          sm_where = 38;
          if (!mbar_wait(pv_done(t), (j - 1u) & 1u, abort_smem, tflag, 38)) { ok = false; break; }
          pv_waited = true;
          fence_after_sync();
          const float m_new = fmaxf(m, mt);
          const float f = (m == -INFINITY || m_new == -INFINITY) ? 0.0f : ex2(m - m_new);
#pragma unroll 1
          for (int c = 0; c < 2; ++c) {
            uint32_t v[32];
            tmem_ld_x32(t_pv + c * 32, v);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * f);
            tmem_st_x32(t_pv + c * 32, v);
          }
          tmem_st_wait();
          l *= f;
          m = m_new;
          probabilities();
          (void)swap(0.0f);                   // both threads are past their second read of the scores
          if (!ok) break;
        }
      }
      // bf16 P (two keys per 32-bit column): this thread's 64 keys take 32 columns of the first half of the score buffer
      tmem_st_x32(t_p, w);
      SPROF(8);
      tmem_st_wait();
      SPROF(9);
      l += sum;
      // PV(j-1) must be complete before P(j) is published (never a stall in practice: it was issued a
      // whole softmax pass ago). The order matters: a parity wait tells apart only two neighbouring
      // phases, so this group may not complete phase j of p_full before the issuer has consumed phase
      // j-1 (it has, once PV(j-1) is committed), nor may the issuer commit PV(j) before this group has
      // consumed pv_done of j-1. With the arrive first, an issuer held up between its two query tiles
      // found p_full two phases ahead and waited for ever.
      sm_where = 39;
      if (!pv_waited && !mbar_wait(pv_done(t), (j - 1u) & 1u, abort_smem, tflag, 39)) { ok = false; break; }
      SPROF(10);
      fence_before_sync();                                 // P in tensor memory, and any O_t rescale, before the PV product
      mbar_arrive(p_full(t));
    }
    if (!ok && tflag && r == 0 && t == 0 && part == 0) atomicCAS(tflag + 6, 0, int(1u << 30 | sm_where << 20 | sm_j));
    if (ok && n_tiles > 0) ok = mbar_wait(pv_done(t), (n_tiles - 1u) & 1u, abort_smem, tflag, 40);
    fence_after_sync();
    // the row sum is the pair's
    float l_row = l;
    if (ok) l_row += swap(l);
    const float inv = l_row > 0.0f ? 1.0f / l_row : 0.0f;
    __nv_bfloat16* dst_row = p.out + ((size_t(b) * p.nq + row) * p.heads + h) * D + part * 64;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      uint32_t v[32];
      tmem_ld_x32(t_pv + c * 32, v);
      tmem_ld_wait();
      if (ok && row < p.nq) {
        uint4* dst = reinterpret_cast<uint4*>(dst_row + c * 32);
#pragma unroll
        for (int g = 0; g < 4; ++g)
          dst[g] = make_uint4(pack2(__uint_as_float(v[8 * g]) * inv, __uint_as_float(v[8 * g + 1]) * inv),
                              pack2(__uint_as_float(v[8 * g + 2]) * inv, __uint_as_float(v[8 * g + 3]) * inv),
                              pack2(__uint_as_float(v[8 * g + 4]) * inv, __uint_as_float(v[8 * g + 5]) * inv),
                              pack2(__uint_as_float(v[8 * g + 6]) * inv, __uint_as_float(v[8 * g + 7]) * inv));
      }
    }
  }

  fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
#ifdef MB_ATTN_PROFILE
  if (threadIdx.x == 0) atomicAdd(&g_attn_prof[3], (unsigned long long)(clock64() - aprof_k0));
#endif
}

}  // namespace

#ifdef MB_ATTN_PROFILE
MB_API int mb_debug_attn_profile(unsigned long long* host_out, int reset) {
  if (host_out) cudaMemcpyFromSymbol(host_out, g_attn_prof, sizeof g_attn_prof);
  if (reset) { static unsigned long long z[16]; cudaMemcpyToSymbol(g_attn_prof, z, sizeof z); }
  return 0;
}
#endif

int mb_attention_prefill_tc5(mb_ctx* ctx, cudaStream_t stream, const AttnParams& p) {
  if (!mb_once(ctx, MB_ONCE_ATTN_PREFILL_TC5)) {
    MB_CUDA_OK(ctx, cudaFuncSetAttribute(attn_prefill_tc5_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
    mb_once_done(ctx, MB_ONCE_ATTN_PREFILL_TC5);
  }
  dim3 grid(unsigned((p.nq + 2 * QT - 1) / (2 * QT)), p.heads, p.batch);
  attn_prefill_tc5_kernel<<<grid, THREADS, SMEM, stream>>>(p);
  MB_LAUNCH_OK(ctx);
  return MB_OK;
}
