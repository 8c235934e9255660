// Shared definitions of the library: the context object behind the C ABI, error
// reporting, and the small device helpers every kernel file uses.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <atomic>
#include <cstring>
#include <mutex>
#include <string>

#include "../../include/mary_b200.h"

#define MB_API extern "C" __attribute__((visibility("default")))

// Device-side status words of a context (one int each, in one small allocation).
enum : int {
  MB_FLAG_WAIT_TIMEOUT = 0,   // a bounded mbarrier wait ran out inside a kernel
  MB_FLAG_ROUTER_NONFINITE,   // a router logit was NaN/Inf (token index + 1)
  MB_FLAG_PLAN_FAULT,         // a routing plan held an out-of-range or duplicate expert
  MB_FLAG_COUNT = 8
};

// One-time per-context set-up steps (function attributes and the like), one bit each.
enum : uint32_t {
  MB_ONCE_GEMM_NVF4_256 = 1u << 0,
  MB_ONCE_GEMM_NVF4_128 = 1u << 1,
  MB_ONCE_GEMM_BF16_256 = 1u << 2,
  MB_ONCE_GEMM_BF16_128 = 1u << 3,
  MB_ONCE_ATTN_DECODE = 1u << 4,
  MB_ONCE_ATTN_PREFILL_LEGACY = 1u << 5,
  MB_ONCE_ATTN_PREFILL_TC5 = 1u << 6,
  MB_ONCE_ATTN_STATIC = 1u << 7,
  MB_ONCE_GEMM_W4A16_256 = 1u << 8,
  MB_ONCE_GEMM_W4A16_128 = 1u << 9,
  MB_ONCE_GEMV_RING = 1u << 10,
  MB_ONCE_GEMM_BF16_PAIR = 1u << 11,
  MB_ONCE_MOE_PLAN_CLUSTER = 1u << 12,
};

struct mb_ctx {
  int device = 0;
  int sm_count = 148;
  int sm_limit = 0;                  // persistent kernels use at most this many SMs (0 = all): room for a collective
  int* flags_dev = nullptr;          // MB_FLAG_COUNT ints, then 8 spare words (see scratch_mu)
  std::string last_error;
  std::mutex mu;
  // The spare words behind the status words are scratch of the entry points that read a reduction back
  // (weight amax, E8M0 range, the warm-up sum): those hold this lock from their memset to their readback.
  std::mutex scratch_mu;
  // which one-time set-up steps this context has done (a context belongs to one device)
  std::atomic<uint32_t> once{0};
  int pair_clusters = 0;             // CTA pairs of the pair GEMM the device holds at once (0 = not asked yet)
  // clusters of 2..8 CTAs of the single-CTA GEMM kernels (split-K through distributed shared memory) the device
  // holds at once, per kernel variant (NVFP4 / bf16 x column width): 0 = not asked yet, -1 = none
  int splitk_clusters[4][9] = {};
  int w4a16_clusters[9] = {};        // the same for the W4A16 prompt kernel (128-column tiles)
  int plan_clusters[17] = {};        // whether a cluster of this many CTAs of the MoE plan kernel fits (1 yes, -1 no)
  // budget of the waits on peers in the fused exchange (tp.cu), microseconds of wall time
  uint32_t wait_limit_us = 1000000;
  // Lazily resolved driver entry point for tensor-map encoding.
  void* encode_tiled = nullptr;
  // Tensor-parallel state (tp.cu).
  void* nccl_lib = nullptr;
  void* nccl_comm = nullptr;
  int tp_rank = 0, tp_world = 1;
  // Peer-mapped exchange memory of the fused row-parallel path (tp.cu).
  struct mb_symm* symm = nullptr;
  // Peer-mapped region of the prompt-sized exchanges (tp_bulk.cu).
  struct mb_bulk* bulk = nullptr;
};

// A region of device memory every rank of the group maps (CUDA IPC): a 4 KB header of flags, then the callers'
// receive areas and gathered buffers at offsets of their choosing.
struct mb_bulk {
  void* local = nullptr;            // this rank's allocation
  void* peer[8] = {};               // every rank's allocation as seen from here (peer[rank] == local)
  void** peer_dev = nullptr;        // the same table in device memory
  size_t bytes = 0;
  int world = 0, rank = 0;          // world 0: not attached yet
  bool ipc = true;
  int* counters = nullptr;          // device words of the exchange kernels (CTAs that finished pushing)
};

// Exchange memory of one rank, mapped into every rank of the group (CUDA IPC). Layout:
//   flags   2 x 64 ints    [0..63]: "my GEMM of step s has landed", [64..127]: "my slice of step s has landed"
//   recv    2 x world x t_max x (n / world) f32   partial tiles pushed here by every rank's GEMM epilogue
//   out     2 x t_max x n bf16                     reduced + residual-added activations, gathered from all ranks
struct mb_symm {
  void* local = nullptr;            // this rank's allocation
  void* peer[8] = {};               // every rank's allocation as seen from here (peer[rank] == local)
  void** peer_dev = nullptr;        // the same table in device memory
  size_t t_max = 0, n = 0, bytes = 0;
  int world = 1, rank = 0;
  bool ipc = true;                  // peers opened through CUDA IPC (closed at destroy) or handed in as pointers
  int* done_counter = nullptr;      // two device counters of the reduce kernel's finished CTAs, one per step parity
};
__host__ __device__ inline size_t mb_symm_flags_bytes() { return 2 * 64 * sizeof(int); }
__host__ __device__ inline size_t mb_symm_recv_bytes(size_t t_max, size_t n) { return 2 * t_max * n * sizeof(float); }
__host__ __device__ inline size_t mb_symm_out_bytes(size_t t_max, size_t n) { return 2 * t_max * n * 2; }

inline int mb_fail(mb_ctx* ctx, int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  if (ctx) {
    std::lock_guard<std::mutex> g(ctx->mu);
    ctx->last_error = buf;
  }
  return code;
}

#define MB_CUDA_OK(ctx, expr)                                                                      \
  do {                                                                                             \
    cudaError_t e__ = (expr);                                                                      \
    if (e__ != cudaSuccess)                                                                        \
      return mb_fail(ctx, MB_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e__),    \
                     __FILE__, __LINE__);                                                          \
  } while (0)

#define MB_REQUIRE(ctx, cond, ...)                                   \
  do {                                                               \
    if (!(cond)) return mb_fail(ctx, MB_ERR_INVALID, __VA_ARGS__);   \
  } while (0)

#define MB_LAUNCH_OK(ctx) MB_CUDA_OK(ctx, cudaGetLastError())

inline bool mb_aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

// True when the step was already done for this context; otherwise the caller does it and calls mb_once_done.
inline bool mb_once(mb_ctx* ctx, uint32_t bit) { return (ctx->once.load(std::memory_order_acquire) & bit) != 0; }
inline void mb_once_done(mb_ctx* ctx, uint32_t bit) { ctx->once.fetch_or(bit, std::memory_order_release); }

// The context's device must be the calling thread's current device: launches and function attributes go to
// the current device, tensor maps and pointers belong to the context's.
#define MB_REQUIRE_DEVICE(ctx, what)                                                                      \
  do {                                                                                                    \
    int cur__ = -1;                                                                                       \
    MB_CUDA_OK(ctx, cudaGetDevice(&cur__));                                                               \
    MB_REQUIRE(ctx, cur__ == (ctx)->device, "%s: device %d must be current (it is %d)", what, (ctx)->device, cur__); \
  } while (0)

// ---------------------------------------------------------------------------
// Device helpers
// ---------------------------------------------------------------------------
#if defined(__CUDACC__)

// Programmatic dependent launch. A kernel launched through mb_launch_pdl may be set up on the
// SMs (block scheduling, parameter and barrier set-up, TMEM allocation) while the kernel before
// it in the stream is still draining; it calls mb_grid_dependency_sync() before its first access
// to global memory, which waits until that kernel has completed and its writes are visible. The
// same call lets the NEXT kernel start its own set-up. Between short kernels of a decode step
// this hides most of the launch gap. MB_PDL=0 in the environment launches everything serialized.
__device__ __forceinline__ void mb_grid_dependency_sync() {
  asm volatile("griddepcontrol.launch_dependents;\n\tgriddepcontrol.wait;" ::: "memory");
}
inline bool mb_pdl_enabled() {
  static const bool on = [] { const char* e = getenv("MB_PDL"); return !(e && e[0] == '0'); }();
  return on;
}
template <typename... KArgs, typename... Args>
inline cudaError_t mb_launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                 Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = mb_pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

__device__ __forceinline__ float mb_bf16_to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

// E4M3 byte -> f32 (finite patterns; 0x7F/0xFF decode to NaN as the format says).
__device__ __forceinline__ float mb_e4m3_to_f32(uint32_t b) {
  uint32_t exp = (b >> 3) & 0xF, man = b & 7;
  float mag;
  if (exp == 0) {
    mag = float(man) * 0.001953125f;  // 2^-9
  } else if (exp == 15 && man == 7) {
    mag = __int_as_float(0x7FC00000);
  } else {
    mag = __int_as_float(((exp + 120u) << 23) | (man << 20));
  }
  return (b & 0x80) ? -mag : mag;
}

// The E2M1 value of the low nibble of `code` by bit construction: for a
// magnitude code m >= 2 the f32 bits are (m << 22) + bits(0.5); codes 0 and 1
// are the subnormal pair; the sign bit moves to bit 31 (so code 8 is -0.0).
__device__ __forceinline__ float mb_e2m1_to_f32(uint32_t code) {
  uint32_t m = code & 7u;
  uint32_t low = (m & 1u) * 0x3F000000u;
  uint32_t high = (m << 22) + 0x3F000000u;
  return __int_as_float((m >= 2u ? high : low) | ((code & 8u) << 28));
}

// f32 -> E4M3 byte for a non-negative finite value already clamped to [0, 448]:
// round to nearest, ties to even significand. Arithmetic form: scaling by a
// power of two is exact, so one rint is the conversion.
__device__ __forceinline__ uint32_t mb_e4m3_from_f32(float v) {
  if (!(v > 0.0f)) return 0;
  if (v >= 448.0f) return 0x7E;
  int e = int((__float_as_uint(v) >> 23) & 0xFF) - 127;
  e = e < -6 ? -6 : e;
  float scaled = v * __int_as_float(uint32_t(127 + 3 - e) << 23);
  uint32_t steps = uint32_t(__float2int_rn(scaled));
  uint32_t byte;
  if (e == -6 && steps < 8) {
    byte = steps;
  } else {
    uint32_t m;
    if (steps == 16) { e += 1; m = 0; } else { m = steps - 8; }
    byte = (uint32_t(e + 7) << 3) | m;
  }
  return byte > 0x7E ? 0x7E : byte;
}

// The same two conversions by the hardware converters (one instruction each way instead of a
// dozen): cvt.rn.satfinite.e4m3x2.f32 rounds to nearest even and saturates at 448; the decode
// goes through f16, which holds every E4M3 value exactly. Callers clamp to [0, 448] first, so
// the NaN and negative cases of the arithmetic form above never reach them.
__device__ __forceinline__ uint32_t mb_e4m3_encode(float v) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(0.0f), "f"(v));
  return uint32_t(r) & 0xFFu;
}
__device__ __forceinline__ float mb_e4m3_decode(uint32_t b) {
  uint32_t h2;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(uint16_t(b)));
  float f;
  asm("{ .reg .b16 lo, hi; mov.b32 {lo, hi}, %1; cvt.f32.f16 %0, lo; }" : "=f"(f) : "r"(h2));
  return f;
}

// RN(a / 6) without the divide subroutine: q = RN(a c), c = RN(1/6); the residual a - 6 q is
// exact in one fma and RN(q + residual c) is the correctly rounded quotient (Markstein; 6's
// significand is not all ones). Tiny, infinite and NaN operands take the divide itself.
__device__ __forceinline__ float mb_div6(float a) {
  const float c = 0.16666667163372040f;   // 0x3E2AAAAB
  if (a >= 1.0e-30f && a <= 3.0e38f) {
    const float q = __fmul_rn(a, c);
    return __fmaf_rn(__fmaf_rn(-q, 6.0f, a), c, q);
  }
  return __fdiv_rn(a, 6.0f);
}

// n / d and n % d for a divisor fixed at launch (Granlund-Montgomery, exact for every 32-bit n).
struct mb_fastdiv {
  uint32_t d, mul, sh1, sh2;
};
inline mb_fastdiv mb_fastdiv_make(uint32_t d) {
  mb_fastdiv f;
  f.d = d;
  uint32_t l = 0;
  while ((1ull << l) < d) ++l;
  f.mul = uint32_t(((1ull << 32) * ((1ull << l) - d)) / d + 1);
  f.sh1 = l < 1 ? l : 1;
  f.sh2 = l - f.sh1;
  return f;
}
__device__ __forceinline__ uint32_t mb_fastdiv_q(uint32_t n, const mb_fastdiv& f) {
  const uint32_t t = __umulhi(f.mul, n);
  return (t + ((n - t) >> f.sh1)) >> f.sh2;
}

// Two f32 -> one byte of E2M1 codes, `lo` in the LOW nibble: the hardware
// cvt.rn.satfinite.e2m1x2.f32 (ties to the even code, saturating at 6, sign kept
// on a zero result). PTX puts its first source operand in the HIGH nibble.
__device__ __forceinline__ uint32_t mb_cvt_e2m1x2(float lo, float hi) {
  uint16_t r;
  asm volatile("{ .reg .b8 t; cvt.rn.satfinite.e2m1x2.f32 t, %1, %2; cvt.u16.u8 %0, t; }"
               : "=h"(r) : "f"(hi), "f"(lo));
  return uint32_t(r) & 0xFFu;
}

// Eight f32 -> one u32 of eight codes, element i at bits 4*i: four e2m1x2 converts
// packed by one byte-vector move.
__device__ __forceinline__ uint32_t mb_cvt_e2m1x8(const float* v) {
  uint32_t r;
  asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n\t"
      "mov.b32 %0, {b0, b1, b2, b3};\n\t}"
      : "=r"(r)
      : "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7]));
  return r;
}

// Byte offset of scale (row, kb) [kb = index of the 16-element block along K] in
// the tiled scale-factor plane the tensor-core GEMM consumes: 512-byte atoms of
// 128 rows x 4 scales, atom-internal offset (row%32)*16 + (row/32%4)*4 + kb%4,
// atoms ordered [row/128][kb/4]. `kchunks` = atoms along K (padded to 4).
__device__ __host__ __forceinline__ size_t mb_sf_offset(size_t row, size_t kb, size_t kchunks) {
  return ((row >> 7) * kchunks + (kb >> 2)) * 512 + (row & 31) * 16 + ((row >> 5) & 3) * 4 + (kb & 3);
}

#endif  // __CUDACC__

// Atoms along K of the tiled scale plane for a given K (4 per 256-element stage).
inline size_t mb_sf_kchunks(size_t k) { return ((k + 255) / 256) * 4; }
inline size_t mb_sf_plane_bytes(size_t rows, size_t k) { return ((rows + 127) / 128) * mb_sf_kchunks(k) * 512; }
