// MoE routing: softmax top-k router, the stacked-row plan (token permutation) and
// the ordered weighted un-permute. All HBM/latency-bound integer and f32 work:
// warp-shuffle reductions, 128-bit accesses, no atomics on the data path (the
// row order is deterministic: expert-ascending, then token-ascending).
#include "common.cuh"

namespace {

// ---------------------------------------------------------------------------------
// Router. A block routes 32 tokens, one per warp (four per warp beyond 128 experts, where the
// registers of a 1024-thread block run short); expert e of a token lives in lane e % 32,
// slot e / 32 of the token's warp.
// Scores follow the CPU rule exactly: m = max logit; e_i = exp(f64(x_i) - m);
// v_i = f32(e_i); s = sum of e_i in index order (f64); score_i = f32(f64(v_i) / s).
// The index-order sum is a chain of dependent f64 adds: the block parks its e_i in shared
// memory and one warp walks the 32 chains side by side, lane t summing token t.
// The sigmoid form scores each expert alone: f32(1 / (1 + exp(-f64(x)))). With a bias the
// selection runs on score + bias (one f32 add) while the weights stay the unbiased scores.
// Selection: descending score, ties to the lower index: per round every lane offers its best
// free slot as an order-preserving integer key; a warp max on the keys and a warp min on the
// indices that hold it find the pick (two redux instructions), one shuffle fetches its score.
// Weights: gathered scores, w / (sum + 1e-20) in selection order, times the scaling factor.
// ---------------------------------------------------------------------------------
constexpr int ROUTER_TOKENS = 32;    // tokens per block

// f32 -> u32 whose unsigned order is the float order (-0 was folded into +0 by the caller).
__device__ __forceinline__ uint32_t router_key(float c) {
  const uint32_t u = __float_as_uint(c);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

template <int EPL, bool SIGMOID, int ROUTER_WARPS>
__global__ void __launch_bounds__(32 * ROUTER_WARPS)
router_topk_kernel(const float* __restrict__ logits, const float* __restrict__ bias, uint32_t tokens,
                   uint32_t n_experts, uint32_t k, int renormalize, float scaling, int32_t* __restrict__ idx,
                   float* __restrict__ weight, int* __restrict__ flag) {
  extern __shared__ double s_router[];
  mb_grid_dependency_sync();
  constexpr uint32_t ROW = 32 * EPL + 1;             // odd stride in doubles: the column walk below meets no bank twice
  double* s_e = s_router;                            // [ROUTER_TOKENS][ROW]
  double* s_sum = s_router + ROUTER_TOKENS * ROW;    // [ROUTER_TOKENS]
  const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  constexpr uint32_t PER = ROUTER_TOKENS / ROUTER_WARPS;
  const uint32_t t0 = blockIdx.x * ROUTER_TOKENS;
  float bs[EPL];
#pragma unroll
  for (int j = 0; j < EPL; ++j) bs[j] = bias ? __ldg(bias + lane + 32 * j) : 0.0f;

  // phase 1: logits -> e_i (softmax) or the finished score (sigmoid), parked in shared memory
#pragma unroll 1
  for (uint32_t q = 0; q < PER; ++q) {
    const uint32_t tl = warp * PER + q, t = t0 + tl;
    if (t >= tokens) break;                          // warp-uniform
    const float* row = logits + size_t(t) * n_experts;
    float x[EPL];
    bool bad = false;
    double m = -INFINITY;
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
      x[j] = __ldg(row + lane + 32 * j);
      if (!(fabsf(x[j]) <= 3.4028234663852886e38f)) bad = true;
      m = fmax(m, double(x[j]));
    }
    if (!SIGMOID) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) m = fmax(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
    }
    if (__any_sync(0xFFFFFFFFu, bad)) {
      if (lane == 0) atomicCAS(flag, 0, int(t) + 1);
    }
#pragma unroll
    for (int j = 0; j < EPL; ++j)
      s_e[tl * ROW + lane + 32 * j] = SIGMOID ? 1.0 / (1.0 + exp(-double(x[j]))) : exp(double(x[j]) - m);
  }
  if (!SIGMOID) {
    __syncthreads();
    // phase 2: lane t of warp 0 sums token t's e_i in expert order
    if (warp == 0) {
      const double* col = s_e + lane * ROW;
      double s = 0.0;
#pragma unroll 8
      for (uint32_t i = 0; i < 32 * EPL; ++i) s += col[i];
      s_sum[lane] = s;
    }
    __syncthreads();
  } else {
    __syncwarp();
  }

  // phase 3: scores, k rounds of arg-max on (score desc, index asc), weights
#pragma unroll 1
  for (uint32_t q = 0; q < PER; ++q) {
    const uint32_t tl = warp * PER + q, t = t0 + tl;
    if (t >= tokens) break;
    float v[EPL];
    uint32_t key[EPL];
    bool bad = false;
    const double s = SIGMOID ? 1.0 : s_sum[tl];
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
      const float e32 = float(s_e[tl * ROW + lane + 32 * j]);
      v[j] = SIGMOID ? e32 : float(double(e32) / s);
      const float c = (bias ? v[j] + bs[j] : v[j]) + 0.0f;       // what the selection compares; -0 -> +0
      if (!(fabsf(c) <= 3.4028234663852886e38f)) bad = true;
      key[j] = router_key(c);
    }
    if (__any_sync(0xFFFFFFFFu, bad)) {
      if (lane == 0) atomicCAS(flag, 0, int(t) + 1);
    }
    uint32_t taken = 0;   // bit j: slot j of this lane already selected
    float wsum = 0.0f;
    float my_w = 0.0f;    // lane r keeps the weight of pick r (k <= 32)
    int my_i = 0;
    for (uint32_t r = 0; r < k; ++r) {
      uint32_t bk = 0, bi = 0xFFFFFFFFu;
      float bv = 0.0f;
#pragma unroll
      for (int j = 0; j < EPL; ++j) {
        const bool free_slot = !((taken >> j) & 1u);
        if (free_slot && (bi == 0xFFFFFFFFu || key[j] > bk)) {   // ascending j: a tie keeps the lower index
          bk = key[j];
          bi = lane + 32 * j;
          bv = v[j];
        }
      }
      const uint32_t mk = __reduce_max_sync(0xFFFFFFFFu, bk);
      const uint32_t best_i = __reduce_min_sync(0xFFFFFFFFu, bk == mk ? bi : 0xFFFFFFFFu);
      const float best_v = __shfl_sync(0xFFFFFFFFu, bv, best_i & 31u);
      if ((best_i & 31u) == lane) taken |= 1u << (best_i >> 5);
      wsum += best_v;   // selection order, as the CPU rule sums; the unbiased score
      if (lane == r) { my_w = best_v; my_i = int(best_i); }
    }
    if (k > 1 && renormalize) my_w = __fdiv_rn(my_w, wsum + 1e-20f);
    if (scaling != 1.0f) my_w *= scaling;
    if (lane < k) {
      idx[size_t(t) * k + lane] = my_i;
      weight[size_t(t) * k + lane] = my_w;
    }
  }
}

// ---------------------------------------------------------------------------------
// Router with shared-expert sinks. One warp per token; logits [tokens, n_routed + n_shared].
// Selection among the routed experts by sigmoid(x) + bias in f32 (descending, ties to the lower
// index), as the rounds above. The k chosen logits (lane r keeps pick r) and the n_shared sink
// logits (lane r keeps sink r) then share one softmax over log_sigmoid, summed in index order,
// chosen first; weights are exp(lp - lse) * route_scale * global_scale. Every f32 exp / log of the
// CPU rule is taken here as the f64 function rounded to f32: the correctly rounded value, which is
// what a good libm returns in all but a vanishing share of arguments.
// ---------------------------------------------------------------------------------
__device__ __forceinline__ float exp32(float x) { return float(exp(double(x))); }
__device__ __forceinline__ float log32(float x) { return float(log(double(x))); }
__device__ __forceinline__ float sigmoid32(float x) {
  if (x >= 0.0f) return __fdiv_rn(1.0f, __fadd_rn(1.0f, exp32(-x)));
  const float e = exp32(x);
  return __fdiv_rn(e, __fadd_rn(1.0f, e));
}
__device__ __forceinline__ float log_sigmoid32(float x) {
  if (x >= 0.0f) return -log32(__fadd_rn(1.0f, exp32(-x)));
  return __fsub_rn(x, log32(__fadd_rn(1.0f, exp32(x))));
}

template <int EPL>
__global__ void __launch_bounds__(128)
router_sinks_kernel(const float* __restrict__ logits, const float* __restrict__ bias, float global_scale,
                    float route_scale, uint32_t tokens, uint32_t n_routed, uint32_t n_shared, uint32_t k,
                    int32_t* __restrict__ idx, float* __restrict__ weight, float* __restrict__ gammas,
                    int* __restrict__ flag) {
  const uint32_t lane = threadIdx.x & 31;
  const uint32_t t = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (t >= tokens) return;
  const float* row = logits + size_t(t) * (n_routed + n_shared);
  float x[EPL];
  uint32_t key[EPL];
  bool bad = false;
#pragma unroll
  for (int j = 0; j < EPL; ++j) {
    x[j] = __ldg(row + lane + 32 * j);
    if (!(fabsf(x[j]) <= 3.4028234663852886e38f)) bad = true;
    const float c = __fadd_rn(sigmoid32(x[j]), __ldg(bias + lane + 32 * j)) + 0.0f;   // -0 -> +0
    if (!(fabsf(c) <= 3.4028234663852886e38f)) bad = true;
    key[j] = router_key(c);
  }
  const float xs = lane < n_shared ? __ldg(row + n_routed + lane) : 0.0f;
  if (!(fabsf(xs) <= 3.4028234663852886e38f)) bad = true;
  if (__any_sync(0xFFFFFFFFu, bad)) {
    if (lane == 0) atomicCAS(flag, 0, int(t) + 1);
  }
  uint32_t taken = 0;
  float my_x = 0.0f;    // lane r keeps the logit of pick r
  int my_i = 0;
  for (uint32_t r = 0; r < k; ++r) {
    uint32_t bk = 0, bi = 0xFFFFFFFFu;
    float bx = 0.0f;
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
      const bool free_slot = !((taken >> j) & 1u);
      if (free_slot && (bi == 0xFFFFFFFFu || key[j] > bk)) {
        bk = key[j];
        bi = lane + 32 * j;
        bx = x[j];
      }
    }
    const uint32_t mk = __reduce_max_sync(0xFFFFFFFFu, bk);
    const uint32_t best_i = __reduce_min_sync(0xFFFFFFFFu, bk == mk ? bi : 0xFFFFFFFFu);
    const float best_x = __shfl_sync(0xFFFFFFFFu, bx, best_i & 31u);
    if ((best_i & 31u) == lane) taken |= 1u << (best_i >> 5);
    if (lane == r) { my_x = best_x; my_i = int(best_i); }
  }
  const float lp_sel = lane < k ? log_sigmoid32(my_x) : -INFINITY;
  const float lp_sh = lane < n_shared ? log_sigmoid32(xs) : -INFINITY;
  float m = fmaxf(lp_sel, lp_sh);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
  const float e_sel = lane < k ? exp32(__fsub_rn(lp_sel, m)) : 0.0f;
  const float e_sh = lane < n_shared ? exp32(__fsub_rn(lp_sh, m)) : 0.0f;
  float sum = 0.0f;     // index order: the chosen experts, then the sinks
  for (uint32_t r = 0; r < k; ++r) sum = __fadd_rn(sum, __shfl_sync(0xFFFFFFFFu, e_sel, r));
  for (uint32_t r = 0; r < n_shared; ++r) sum = __fadd_rn(sum, __shfl_sync(0xFFFFFFFFu, e_sh, r));
  const float lse = __fadd_rn(m, log32(sum));
  if (lane < k) {
    idx[size_t(t) * k + lane] = my_i;
    weight[size_t(t) * k + lane] = __fmul_rn(__fmul_rn(exp32(__fsub_rn(lp_sel, lse)), route_scale), global_scale);
  }
  if (lane < n_shared)
    gammas[size_t(t) * n_shared + lane] = __fmul_rn(__fmul_rn(exp32(__fsub_rn(lp_sh, lse)), route_scale), global_scale);
}

// ---------------------------------------------------------------------------------
// Row plan
// ---------------------------------------------------------------------------------
constexpr int PLAN_PAD = 128;   // rows per GEMM tile: each expert's rows are padded to this

constexpr int PLAN_CHUNK = 256;   // tokens per block of the count and place passes

// A pick (t, j) takes a row unless its expert is out of range or repeats an earlier pick of the token.
__device__ __forceinline__ bool plan_pick_ok(const int32_t* p, uint32_t j, uint32_t n_experts) {
  const int32_t e = p[j];
  bool ok = e >= 0 && uint32_t(e) < n_experts;
  for (uint32_t i = 0; ok && i < j; ++i) ok = p[i] != e;
  return ok;
}

// Pass 1, one block per 256 tokens: picks per expert within the chunk (a shared-memory
// histogram; the sums do not depend on the order of the adds) -> chunk_counts[chunk][expert].
// The same launch puts the row arrays in their empty state (-1, weight 0).
__global__ void __launch_bounds__(PLAN_CHUNK)
plan_count_kernel(const int32_t* __restrict__ idx, uint32_t tokens, uint32_t k, uint32_t n_experts,
                  int32_t* __restrict__ chunk_counts, int32_t* __restrict__ row_tok, float* __restrict__ row_wgt,
                  uint32_t m_cap, int* __restrict__ flag) {
  extern __shared__ int32_t s_hist[];
  for (uint32_t e = threadIdx.x; e < n_experts; e += PLAN_CHUNK) s_hist[e] = 0;
  mb_grid_dependency_sync();
  for (uint32_t i = blockIdx.x * PLAN_CHUNK + threadIdx.x; i < m_cap; i += gridDim.x * PLAN_CHUNK) {
    row_tok[i] = -1;
    row_wgt[i] = 0.0f;
  }
  __syncthreads();
  const uint32_t t = blockIdx.x * PLAN_CHUNK + threadIdx.x;
  if (t < tokens) {
    const int32_t* p = idx + size_t(t) * k;
    for (uint32_t j = 0; j < k; ++j) {
      if (plan_pick_ok(p, j, n_experts)) atomicAdd(&s_hist[p[j]], 1);
      else atomicCAS(flag, 0, int(t) + 1);
    }
  }
  __syncthreads();
  for (uint32_t e = threadIdx.x; e < n_experts; e += PLAN_CHUNK)
    chunk_counts[size_t(blockIdx.x) * n_experts + e] = s_hist[e];
}

// Pass 2, one block, thread e = expert e: the chunk counts become exclusive prefixes over
// the chunks (rows of expert e that earlier chunks take); the totals, padded to 128, give the
// first stacked row of each expert, the expert of each tile and the number of tiles in use.
__global__ void __launch_bounds__(1024)
plan_scan_kernel(const int32_t* __restrict__ chunk_counts, int32_t* __restrict__ chunk_base, uint32_t chunks,
                 uint32_t n_experts, int32_t* __restrict__ expert_rows, int32_t* __restrict__ expert_row0,
                 int32_t* __restrict__ tile_expert, uint32_t tile_cap, int32_t* __restrict__ n_tiles) {
  __shared__ int32_t s_pad[1024];
  __shared__ int32_t s_off[1024];
  __shared__ int32_t s_total;
  mb_grid_dependency_sync();
  const uint32_t e = threadIdx.x;
  int32_t c = 0;
  if (e < n_experts) {
    // counts and prefixes live in separate arrays so that the loads of a batch are independent
    for (uint32_t ch0 = 0; ch0 < chunks; ch0 += 8) {
      int32_t here[8];
#pragma unroll
      for (uint32_t i = 0; i < 8; ++i) here[i] = ch0 + i < chunks ? __ldg(chunk_counts + size_t(ch0 + i) * n_experts + e) : 0;
#pragma unroll
      for (uint32_t i = 0; i < 8; ++i) {
        if (ch0 + i < chunks) chunk_base[size_t(ch0 + i) * n_experts + e] = c;
        c += here[i];
      }
    }
  }
  const int32_t pad = (c + PLAN_PAD - 1) / PLAN_PAD;   // tiles of this expert (0 beyond n_experts)
  s_pad[e] = pad;
  // exclusive prefix of the tile counts over the experts: warp scans, then a scan of the 32 warp totals
  __shared__ int32_t s_warp[32];
  const uint32_t lane = e & 31, wp = e >> 5;
  int32_t inc = pad;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int32_t up = __shfl_up_sync(0xFFFFFFFFu, inc, o);
    if (lane >= uint32_t(o)) inc += up;
  }
  if (lane == 31) s_warp[wp] = inc;
  __syncthreads();
  if (wp == 0) {
    const int32_t tot = s_warp[lane];
    int32_t winc = tot;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int32_t up = __shfl_up_sync(0xFFFFFFFFu, winc, o);
      if (lane >= uint32_t(o)) winc += up;
    }
    s_warp[lane] = winc - tot;
    if (lane == 31) { *n_tiles = winc; s_total = winc; }
  }
  __syncthreads();
  s_off[e] = s_warp[wp] + inc - pad;
  __syncthreads();
  if (e < n_experts) {
    expert_rows[e] = c;
    expert_row0[e] = s_off[e] * PLAN_PAD;
    for (int32_t i = 0; i < s_pad[e]; ++i)
      if (uint32_t(s_off[e] + i) < tile_cap) tile_expert[s_off[e] + i] = int32_t(e);
  }
  for (uint32_t i = uint32_t(s_total) + e; i < tile_cap; i += 1024) tile_expert[i] = -1;
}

// Pass 3, one block per 256 tokens, thread = token. A bit mask per expert records which
// tokens of the chunk picked it; a pick's row is the expert's first row + the rows earlier
// chunks take + the number of earlier tokens of this chunk in the mask. Deterministic:
// expert-ascending, token-ascending. The token's k rows are then sorted and stored.
__global__ void __launch_bounds__(PLAN_CHUNK)
plan_place_kernel(const int32_t* __restrict__ idx, const float* __restrict__ weight, uint32_t tokens, uint32_t k,
                  uint32_t n_experts, const int32_t* __restrict__ chunk_base, const int32_t* __restrict__ expert_row0,
                  int32_t* __restrict__ row_tok, float* __restrict__ row_wgt, int32_t* __restrict__ tok_rows) {
  extern __shared__ uint32_t s_mask[];   // [n_experts][8]
  for (uint32_t i = threadIdx.x; i < n_experts * 8; i += PLAN_CHUNK) s_mask[i] = 0u;
  mb_grid_dependency_sync();
  __syncthreads();
  const uint32_t t = blockIdx.x * PLAN_CHUNK + threadIdx.x;
  const uint32_t word = threadIdx.x >> 5, bit = threadIdx.x & 31;
  const int32_t* p = idx + size_t(t) * k;
  uint32_t ok_bits = 0;
  if (t < tokens) {
    for (uint32_t j = 0; j < k; ++j) {
      if (plan_pick_ok(p, j, n_experts)) {
        ok_bits |= 1u << j;
        atomicOr(&s_mask[uint32_t(p[j]) * 8 + word], 1u << bit);
      }
    }
  }
  __syncthreads();
  if (t >= tokens) return;
  int32_t rows[32];
  for (uint32_t j = 0; j < k; ++j) {
    int32_t row = -1;
    if (ok_bits >> j & 1u) {
      const uint32_t e = uint32_t(p[j]);
      const uint32_t* m = s_mask + e * 8;
      int32_t rank = __popc(m[word] & ((1u << bit) - 1u));
      for (uint32_t w = 0; w < word; ++w) rank += __popc(m[w]);
      row = expert_row0[e] + chunk_base[size_t(blockIdx.x) * n_experts + e] + rank;
      row_tok[row] = int32_t(t);
      row_wgt[row] = weight[size_t(t) * k + j];
    }
    // insertion into the ascending list (a pick without a row, -1, sorts first)
    int i = int(j) - 1;
    while (i >= 0 && rows[i] > row) { rows[i + 1] = rows[i]; --i; }
    rows[i + 1] = row;
  }
  for (uint32_t j = 0; j < k; ++j) tok_rows[size_t(t) * k + j] = rows[j];
}

// out[t, c..c+7] = sum_j fma(y[row_j, c..c+7], wgt[row_j], acc), rows ascending.
template <typename Y>
__global__ void __launch_bounds__(256)
scatter_weighted_kernel(const Y* __restrict__ y, const float* __restrict__ row_wgt,
                        const int32_t* __restrict__ tok_rows, uint32_t tokens, uint32_t k, uint32_t h,
                        float* __restrict__ out) {
  const uint32_t per_tok = h / 8;
  mb_grid_dependency_sync();
  size_t gid = size_t(blockIdx.x) * 256 + threadIdx.x;
  if (gid >= size_t(tokens) * per_tok) return;
  uint32_t t = uint32_t(gid / per_tok), c = uint32_t(gid % per_tok) * 8;
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (uint32_t j = 0; j < k; ++j) {
    int32_t r = tok_rows[size_t(t) * k + j];
    if (r < 0) continue;
    float w = row_wgt[r];
    float v[8];
    if (sizeof(Y) == 2) {
      uint4 q = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(y) + size_t(r) * h + c));
      uint32_t ww[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        v[2 * i] = __uint_as_float(ww[i] << 16);
        v[2 * i + 1] = __uint_as_float(ww[i] & 0xFFFF0000u);
      }
    } else {
      const float4* q = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(y) + size_t(r) * h + c);
      float4 a = __ldg(q), b = __ldg(q + 1);
      v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = fmaf(v[i], w, acc[i]);
  }
  float4* o = reinterpret_cast<float4*>(out + size_t(t) * h + c);
  o[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
  o[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
}

// The same pass for k <= 8 with a token's picks in registers: its picks and weights, then the two
// bases of every pick, are loaded together instead of as one dependent pair of loads per pick,
// and the rows are sorted by a fixed exchange network.
__global__ void __launch_bounds__(PLAN_CHUNK)
plan_place8_kernel(const int32_t* __restrict__ idx, const float* __restrict__ weight, uint32_t tokens, uint32_t k,
                   uint32_t n_experts, const int32_t* __restrict__ chunk_base, const int32_t* __restrict__ expert_row0,
                   int32_t* __restrict__ row_tok, float* __restrict__ row_wgt, int32_t* __restrict__ tok_rows) {
  extern __shared__ uint32_t s_mask[];   // [n_experts][8]
  for (uint32_t i = threadIdx.x; i < n_experts * 8; i += PLAN_CHUNK) s_mask[i] = 0u;
  mb_grid_dependency_sync();
  const uint32_t t = blockIdx.x * PLAN_CHUNK + threadIdx.x;
  const uint32_t word = threadIdx.x >> 5, bit = threadIdx.x & 31;
  const bool live = t < tokens;
  int32_t e[8];
  float w[8];
#pragma unroll
  for (uint32_t j = 0; j < 8; ++j) {
    const bool have = live && j < k;
    e[j] = have ? __ldg(idx + size_t(t) * k + j) : -1;
    w[j] = have ? __ldg(weight + size_t(t) * k + j) : 0.0f;
  }
  __syncthreads();
  uint32_t ok_bits = 0;
#pragma unroll
  for (uint32_t j = 0; j < 8; ++j) {
    bool ok = live && j < k && e[j] >= 0 && uint32_t(e[j]) < n_experts;
#pragma unroll
    for (uint32_t i = 0; i < j; ++i) ok = ok && e[i] != e[j];
    if (ok) {
      ok_bits |= 1u << j;
      atomicOr(&s_mask[uint32_t(e[j]) * 8 + word], 1u << bit);
    }
  }
  __syncthreads();
  if (!live) return;
  int32_t base[8];
#pragma unroll
  for (uint32_t j = 0; j < 8; ++j)
    base[j] = (ok_bits >> j & 1u)
                  ? __ldg(expert_row0 + e[j]) + __ldg(chunk_base + size_t(blockIdx.x) * n_experts + uint32_t(e[j]))
                  : 0;
  int32_t rows[8];
#pragma unroll
  for (uint32_t j = 0; j < 8; ++j) {
    int32_t row = j < k ? -1 : 0x7FFFFFFF;          // a pick without a row sorts first, an absent pick last
    if (ok_bits >> j & 1u) {
      const uint32_t* m = s_mask + uint32_t(e[j]) * 8;
      int32_t rank = __popc(m[word] & ((1u << bit) - 1u));
      for (uint32_t ww = 0; ww < word; ++ww) rank += __popc(m[ww]);
      row = base[j] + rank;
      row_tok[row] = int32_t(t);
      row_wgt[row] = w[j];
    }
    rows[j] = row;
  }
#pragma unroll
  for (int pass = 0; pass < 8; ++pass) {
#pragma unroll
    for (int i = pass & 1; i + 1 < 8; i += 2) {
      const int32_t lo = min(rows[i], rows[i + 1]), hi = max(rows[i], rows[i + 1]);
      rows[i] = lo;
      rows[i + 1] = hi;
    }
  }
#pragma unroll
  for (uint32_t j = 0; j < 8; ++j)
    if (j < k) tok_rows[size_t(t) * k + j] = rows[j];
}

// The three passes as one kernel for plans of up to 16 chunks (4096 tokens) and k <= 8: the chunks' CTAs are one
// thread-block cluster, a chunk's histogram stays in its CTA's shared memory, and after a cluster barrier every CTA
// reads the histograms of all chunks through distributed shared memory: the sums over the earlier chunks are its
// bases, the sums over all chunks give every expert's rows, tiles and first row (each CTA scans them for itself; the
// first CTA also writes them out). The same values as the three kernels, without their two round trips through
// global memory and two launches.
constexpr int PLAN_CLUSTER_MAX = 16;

__device__ __forceinline__ void plan_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release;\n\tbarrier.cluster.wait.acquire;" ::: "memory");
}
__device__ __forceinline__ int32_t plan_ld_cluster(const int32_t* own, uint32_t rank) {
  uint32_t a = uint32_t(__cvta_generic_to_shared(own)), r;
  int32_t v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(rank));
  asm volatile("ld.shared::cluster.b32 %0, [%1];" : "=r"(v) : "r"(r) : "memory");
  return v;
}

__global__ void __launch_bounds__(PLAN_CHUNK)
plan_cluster8_kernel(const int32_t* __restrict__ idx, const float* __restrict__ weight, uint32_t tokens, uint32_t k,
                     uint32_t n_experts, int32_t* __restrict__ row_tok, float* __restrict__ row_wgt,
                     int32_t* __restrict__ tok_rows, int32_t* __restrict__ expert_rows, int32_t* __restrict__ expert_row0,
                     int32_t* __restrict__ tile_expert, uint32_t tile_cap, int32_t* __restrict__ n_tiles, uint32_t m_cap,
                     int* __restrict__ flag) {
  extern __shared__ int32_t s_plan[];          // hist | base | row0 | pad  [n_experts] each, then mask [n_experts][8]
  int32_t* s_hist = s_plan;
  int32_t* s_base = s_hist + n_experts;
  int32_t* s_row0 = s_base + n_experts;
  int32_t* s_pad = s_row0 + n_experts;
  uint32_t* s_mask = reinterpret_cast<uint32_t*>(s_pad + n_experts);
  __shared__ int32_t s_warp[PLAN_CHUNK / 32];
  __shared__ int32_t s_total;
  for (uint32_t e = threadIdx.x; e < n_experts; e += PLAN_CHUNK) s_hist[e] = 0;
  for (uint32_t i = threadIdx.x; i < n_experts * 8; i += PLAN_CHUNK) s_mask[i] = 0u;
  mb_grid_dependency_sync();
  for (uint32_t i = blockIdx.x * PLAN_CHUNK + threadIdx.x; i < m_cap; i += gridDim.x * PLAN_CHUNK) {
    row_tok[i] = -1;
    row_wgt[i] = 0.0f;
  }
  const uint32_t t = blockIdx.x * PLAN_CHUNK + threadIdx.x;
  const uint32_t word = threadIdx.x >> 5, bit = threadIdx.x & 31, lane = bit;
  const bool live = t < tokens;
  int32_t e[8];
  float w[8];
#pragma unroll
  for (uint32_t j = 0; j < 8; ++j) {
    const bool have = live && j < k;
    e[j] = have ? __ldg(idx + size_t(t) * k + j) : -1;
    w[j] = have ? __ldg(weight + size_t(t) * k + j) : 0.0f;
  }
  __syncthreads();
  uint32_t ok_bits = 0;
#pragma unroll
  for (uint32_t j = 0; j < 8; ++j) {
    bool ok = live && j < k && e[j] >= 0 && uint32_t(e[j]) < n_experts;
#pragma unroll
    for (uint32_t i = 0; i < j; ++i) ok = ok && e[i] != e[j];
    if (ok) {
      ok_bits |= 1u << j;
      atomicAdd(&s_hist[e[j]], 1);
      atomicOr(&s_mask[uint32_t(e[j]) * 8 + word], 1u << bit);
    } else if (live && j < k) {
      atomicCAS(flag, 0, int(t) + 1);
    }
  }
  __syncthreads();
  plan_cluster_sync();                         // every chunk's histogram is in place; the rows' empty state is written
  // this thread's experts: a contiguous run, so that the prefix over the experts is a scan over the threads
  const uint32_t per = (n_experts + PLAN_CHUNK - 1) / PLAN_CHUNK;       // <= 4
  const uint32_t e0 = threadIdx.x * per, rank = blockIdx.x, ranks = gridDim.x;
  int32_t tot[4] = {0, 0, 0, 0}, pads = 0;
  for (uint32_t i = 0; i < per; ++i) {
    const uint32_t ex = e0 + i;
    if (ex >= n_experts) break;
    int32_t base = 0, total = 0;
    for (uint32_t r = 0; r < ranks; ++r) {
      const int32_t c = plan_ld_cluster(s_hist + ex, r);
      if (r < rank) base += c;
      total += c;
    }
    s_base[ex] = base;
    tot[i] = total;
    const int32_t pad = (total + PLAN_PAD - 1) / PLAN_PAD;
    s_pad[ex] = pad;
    pads += pad;
  }
  int32_t inc = pads;                          // inclusive prefix of the tile counts over the threads
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int32_t up = __shfl_up_sync(0xFFFFFFFFu, inc, o);
    if (lane >= uint32_t(o)) inc += up;
  }
  if (lane == 31) s_warp[word] = inc;
  __syncthreads();
  if (word == 0) {
    const int32_t v = lane < PLAN_CHUNK / 32 ? s_warp[lane] : 0;
    int32_t winc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int32_t up = __shfl_up_sync(0xFFFFFFFFu, winc, o);
      if (lane >= uint32_t(o)) winc += up;
    }
    if (lane < PLAN_CHUNK / 32) s_warp[lane] = winc - v;
    if (lane == 31) s_total = winc;
  }
  __syncthreads();
  int32_t off = s_warp[word] + inc - pads;     // tiles before this thread's first expert
  for (uint32_t i = 0; i < per; ++i) {
    const uint32_t ex = e0 + i;
    if (ex >= n_experts) break;
    s_row0[ex] = off * PLAN_PAD;
    if (rank == 0) {
      expert_rows[ex] = tot[i];
      expert_row0[ex] = off * PLAN_PAD;
      for (int32_t q = 0; q < s_pad[ex]; ++q)
        if (uint32_t(off + q) < tile_cap) tile_expert[off + q] = int32_t(ex);
    }
    off += s_pad[ex];
  }
  if (rank == 0) {
    if (threadIdx.x == 0) *n_tiles = s_total;
    for (uint32_t i = uint32_t(s_total) + threadIdx.x; i < tile_cap; i += PLAN_CHUNK) tile_expert[i] = -1;
  }
  __syncthreads();
  plan_cluster_sync();                         // no CTA leaves (or reuses nothing) while another reads its histogram
  if (!live) return;
  int32_t rows[8];
#pragma unroll
  for (uint32_t j = 0; j < 8; ++j) {
    int32_t row = j < k ? -1 : 0x7FFFFFFF;          // a pick without a row sorts first, an absent pick last
    if (ok_bits >> j & 1u) {
      const uint32_t ex = uint32_t(e[j]);
      const uint32_t* m = s_mask + ex * 8;
      int32_t pos = __popc(m[word] & ((1u << bit) - 1u));
      for (uint32_t ww = 0; ww < word; ++ww) pos += __popc(m[ww]);
      row = s_row0[ex] + s_base[ex] + pos;
      row_tok[row] = int32_t(t);
      row_wgt[row] = w[j];
    }
    rows[j] = row;
  }
#pragma unroll
  for (int pass = 0; pass < 8; ++pass) {
#pragma unroll
    for (int i = pass & 1; i + 1 < 8; i += 2) {
      const int32_t lo = min(rows[i], rows[i + 1]), hi = max(rows[i], rows[i + 1]);
      rows[i] = lo;
      rows[i + 1] = hi;
    }
  }
#pragma unroll
  for (uint32_t j = 0; j < 8; ++j)
    if (j < k) tok_rows[size_t(t) * k + j] = rows[j];
}

}  // namespace

MB_API int mb_router_topk(mb_ctx* ctx, mb_stream stream_, const float* logits, const float* bias, int activation,
                          size_t tokens, size_t n_experts, size_t k, int renormalize, float scaling, int32_t* idx,
                          float* weight) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  MB_REQUIRE(ctx, ctx && logits && idx && weight, "router: null argument");
  MB_REQUIRE(ctx, activation == MB_ROUTER_SOFTMAX || activation == MB_ROUTER_SIGMOID,
             "router: activation %d is neither softmax nor sigmoid", activation);
  MB_REQUIRE(ctx, tokens > 0, "router: select() on zero tokens");
  MB_REQUIRE(ctx, n_experts >= 32 && n_experts % 32 == 0 && n_experts <= 512,
             "router: n_experts must be a multiple of 32 up to 512, got %zu", n_experts);
  MB_REQUIRE(ctx, k >= 1 && k <= 32 && k <= n_experts, "router: top_k must be 1..32, got %zu", k);
  const unsigned grid = unsigned((tokens + ROUTER_TOKENS - 1) / ROUTER_TOKENS);
  int* flag = ctx->flags_dev + MB_FLAG_ROUTER_NONFINITE;
  const bool sigmoid = activation == MB_ROUTER_SIGMOID;
  const size_t smem = (size_t(ROUTER_TOKENS) * (n_experts + 1) + ROUTER_TOKENS) * sizeof(double);
#define ROUTE1(EPL, SIG)                                                                                        \
  do {                                                                                                          \
    constexpr int WARPS = EPL <= 4 ? 32 : 8;                                                                    \
    auto kern = router_topk_kernel<EPL, SIG, WARPS>;                                                            \
    if (smem > 48 * 1024)                                                                                       \
      MB_CUDA_OK(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));      \
    mb_launch_pdl(kern, dim3(grid), dim3(32 * WARPS), smem, stream, logits, bias, uint32_t(tokens),             \
                  uint32_t(n_experts), uint32_t(k), renormalize, scaling, idx, weight, flag);                   \
  } while (0)
#define ROUTE(EPL) do { if (sigmoid) ROUTE1(EPL, true); else ROUTE1(EPL, false); } while (0)
  switch (n_experts / 32) {
    case 1: ROUTE(1); break;
    case 2: ROUTE(2); break;
    case 3: ROUTE(3); break;
    case 4: ROUTE(4); break;
    case 6: ROUTE(6); break;
    case 8: ROUTE(8); break;
    case 12: ROUTE(12); break;
    case 16: ROUTE(16); break;
    default: return mb_fail(ctx, MB_ERR_INVALID, "router: unsupported expert count %zu", n_experts);
  }
#undef ROUTE1
#undef ROUTE
  MB_LAUNCH_OK(ctx);
  return MB_OK;
}

MB_API int mb_router_topk_softmax(mb_ctx* ctx, mb_stream stream, const float* logits, size_t tokens,
                                  size_t n_experts, size_t k, int renormalize, float scaling, int32_t* idx,
                                  float* weight) {
  return mb_router_topk(ctx, stream, logits, nullptr, MB_ROUTER_SOFTMAX, tokens, n_experts, k, renormalize, scaling,
                        idx, weight);
}

MB_API int mb_router_topk_sinks(mb_ctx* ctx, mb_stream stream_, const float* logits, const float* bias,
                                float global_scale, float route_scale, size_t tokens, size_t n_routed, size_t n_shared,
                                size_t k, int32_t* idx, float* weight, float* shared_gammas) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  MB_REQUIRE(ctx, ctx && logits && bias && idx && weight && (n_shared == 0 || shared_gammas), "router: null argument");
  MB_REQUIRE(ctx, tokens > 0, "router: route() on zero tokens");
  MB_REQUIRE(ctx, n_routed >= 32 && n_routed % 32 == 0 && n_routed <= 512,
             "router: n_routed must be a multiple of 32 up to 512, got %zu", n_routed);
  MB_REQUIRE(ctx, n_shared <= 32, "router: at most 32 shared experts, got %zu", n_shared);
  MB_REQUIRE(ctx, k >= 1 && k <= 32 && k <= n_routed, "router: top_k must be 1..32, got %zu", k);
  const unsigned grid = unsigned((tokens + 3) / 4);
  int* flag = ctx->flags_dev + MB_FLAG_ROUTER_NONFINITE;
#define ROUTE(EPL)                                                                                               \
  router_sinks_kernel<EPL><<<grid, 128, 0, stream>>>(logits, bias, global_scale, route_scale, uint32_t(tokens),  \
                                                     uint32_t(n_routed), uint32_t(n_shared), uint32_t(k), idx,   \
                                                     weight, shared_gammas, flag)
  switch (n_routed / 32) {
    case 1: ROUTE(1); break;
    case 2: ROUTE(2); break;
    case 3: ROUTE(3); break;
    case 4: ROUTE(4); break;
    case 6: ROUTE(6); break;
    case 8: ROUTE(8); break;
    case 12: ROUTE(12); break;
    case 16: ROUTE(16); break;
    default: return mb_fail(ctx, MB_ERR_INVALID, "router: unsupported expert count %zu", n_routed);
  }
#undef ROUTE
  MB_LAUNCH_OK(ctx);
  return MB_OK;
}

MB_API size_t mb_moe_plan_rows(size_t tokens, size_t k, size_t n_experts) {
  size_t active = n_experts < tokens * k ? n_experts : tokens * k;
  size_t worst = tokens * k + active * (PLAN_PAD - 1);
  return (worst + PLAN_PAD - 1) / PLAN_PAD * PLAN_PAD;
}

MB_API size_t mb_moe_plan_workspace(size_t tokens, size_t k, size_t n_experts) {
  (void)k;
  // picks per (chunk of 256 tokens, expert) and their exclusive prefixes over the chunks
  return 2 * ((tokens + PLAN_CHUNK - 1) / PLAN_CHUNK) * n_experts * sizeof(int32_t);
}

MB_API int mb_moe_plan(mb_ctx* ctx, mb_stream stream_, const int32_t* idx, const float* weight, size_t tokens,
                       size_t k, size_t n_experts, int32_t* row_tok, float* row_wgt, int32_t* tok_rows,
                       int32_t* expert_rows, int32_t* expert_row0, int32_t* tile_expert, int32_t* n_tiles,
                       void* workspace, size_t workspace_bytes) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  MB_REQUIRE(ctx, ctx && idx && weight && row_tok && row_wgt && tok_rows && expert_rows && expert_row0 && tile_expert &&
                      n_tiles && workspace,
             "moe_plan: null argument");
  MB_REQUIRE(ctx, tokens > 0 && k >= 1 && k <= 32 && n_experts >= 1 && n_experts <= 1024,
             "moe_plan: tokens > 0, 1 <= k <= 32, experts <= 1024");
  MB_REQUIRE(ctx, workspace_bytes >= mb_moe_plan_workspace(tokens, k, n_experts), "moe_plan: workspace too small");
  MB_REQUIRE(ctx, tokens * k < (1ull << 31), "moe_plan: exceeds i32 indexing");
  size_t m_cap = mb_moe_plan_rows(tokens, k, n_experts);
  int32_t* chunk_counts = static_cast<int32_t*>(workspace);
  const unsigned chunks = unsigned((tokens + PLAN_CHUNK - 1) / PLAN_CHUNK);
  int* flag = ctx->flags_dev + MB_FLAG_PLAN_FAULT;
  {
    // one kernel, the chunks as one cluster, where the plan is small enough (MB_MOE_PLAN_CLUSTER=0: the three passes)
    const char* env = getenv("MB_MOE_PLAN_CLUSTER");
    const size_t smem = n_experts * (4 * sizeof(int32_t) + 32);
    if (!(env && env[0] == '0') && k <= 8 && chunks <= unsigned(PLAN_CLUSTER_MAX) && smem <= 48 * 1024) {
      if (!mb_once(ctx, MB_ONCE_MOE_PLAN_CLUSTER)) {
        MB_CUDA_OK(ctx, cudaFuncSetAttribute(plan_cluster8_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
        mb_once_done(ctx, MB_ONCE_MOE_PLAN_CLUSTER);
      }
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(chunks);
      cfg.blockDim = dim3(PLAN_CHUNK);
      cfg.dynamicSmemBytes = smem;
      cfg.stream = stream;
      cudaLaunchAttribute attr[2];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = chunks; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
      attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attr[1].val.programmaticStreamSerializationAllowed = 1;
      cfg.attrs = attr;
      cfg.numAttrs = mb_pdl_enabled() ? 2 : 1;
      int& fits = ctx->plan_clusters[chunks];
      if (fits == 0) {
        int held = 0;
        if (cudaOccupancyMaxActiveClusters(&held, plan_cluster8_kernel, &cfg) != cudaSuccess) { (void)cudaGetLastError(); held = 0; }
        fits = held >= 1 ? 1 : -1;
      }
      if (fits > 0) {
        MB_CUDA_OK(ctx, cudaLaunchKernelEx(&cfg, plan_cluster8_kernel, idx, weight, uint32_t(tokens), uint32_t(k),
                                           uint32_t(n_experts), row_tok, row_wgt, tok_rows, expert_rows, expert_row0,
                                           tile_expert, uint32_t(m_cap / PLAN_PAD), n_tiles, uint32_t(m_cap), flag));
        MB_LAUNCH_OK(ctx);
        return MB_OK;
      }
    }
  }
  mb_launch_pdl(plan_count_kernel, dim3(chunks), dim3(PLAN_CHUNK), n_experts * sizeof(int32_t), stream, idx,
                uint32_t(tokens), uint32_t(k), uint32_t(n_experts), chunk_counts, row_tok, row_wgt, uint32_t(m_cap), flag);
  MB_LAUNCH_OK(ctx);
  int32_t* chunk_base = chunk_counts + size_t(chunks) * n_experts;
  mb_launch_pdl(plan_scan_kernel, dim3(1), dim3(1024), 0, stream, chunk_counts, chunk_base, uint32_t(chunks),
                uint32_t(n_experts), expert_rows, expert_row0, tile_expert, uint32_t(m_cap / PLAN_PAD), n_tiles);
  MB_LAUNCH_OK(ctx);
  if (k <= 8)
    mb_launch_pdl(plan_place8_kernel, dim3(chunks), dim3(PLAN_CHUNK), n_experts * 32, stream, idx, weight,
                  uint32_t(tokens), uint32_t(k), uint32_t(n_experts), chunk_base, expert_row0, row_tok, row_wgt,
                  tok_rows);
  else
    mb_launch_pdl(plan_place_kernel, dim3(chunks), dim3(PLAN_CHUNK), n_experts * 32, stream, idx, weight,
                  uint32_t(tokens), uint32_t(k), uint32_t(n_experts), chunk_base, expert_row0, row_tok, row_wgt,
                  tok_rows);
  MB_LAUNCH_OK(ctx);
  return MB_OK;
}

MB_API int mb_moe_scatter_weighted(mb_ctx* ctx, mb_stream stream_, const void* y, int y_dtype, const float* row_wgt,
                                   const int32_t* tok_rows, size_t tokens, size_t k, size_t h, float* out) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  MB_REQUIRE(ctx, ctx && y && row_wgt && tok_rows && out, "scatter_weighted: null argument");
  MB_REQUIRE(ctx, tokens > 0 && k >= 1 && h > 0 && h % 8 == 0, "scatter_weighted: h must be a positive multiple of 8");
  MB_REQUIRE(ctx, mb_aligned(y, 16) && mb_aligned(out, 16), "scatter_weighted: 16-byte alignment");
  size_t total = tokens * (h / 8);
  unsigned grid = unsigned((total + 255) / 256);
  if (y_dtype == MB_DT_BF16)
    mb_launch_pdl(scatter_weighted_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, stream,
                  static_cast<const __nv_bfloat16*>(y), row_wgt, tok_rows, uint32_t(tokens), uint32_t(k), uint32_t(h), out);
  else if (y_dtype == MB_DT_F32)
    mb_launch_pdl(scatter_weighted_kernel<float>, dim3(grid), dim3(256), 0, stream, static_cast<const float*>(y),
                  row_wgt, tok_rows, uint32_t(tokens), uint32_t(k), uint32_t(h), out);
  else
    return mb_fail(ctx, MB_ERR_INVALID, "scatter_weighted: y is bf16 or f32");
  MB_LAUNCH_OK(ctx);
  return MB_OK;
}
