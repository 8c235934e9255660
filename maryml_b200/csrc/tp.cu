// Tensor-parallel plumbing: shard arithmetic and the SUM all-reduce over NCCL
// (NVLink 5 / NVSwitch on a B200 node). NCCL is loaded at run time from the
// process (the library torch already brought in) so that the kernels' shared
// object has no link-time dependency on it.
#include "common.cuh"

#include <dlfcn.h>

#include <algorithm>

namespace {

typedef struct { char internal[128]; } NcclUniqueId;
typedef void* NcclComm;
enum { NCCL_SUM = 0, NCCL_UINT8 = 1, NCCL_FLOAT32 = 7, NCCL_BFLOAT16 = 9 };

struct NcclApi {
  int (*GetUniqueId)(NcclUniqueId*);
  int (*CommInitRank)(NcclComm*, int, NcclUniqueId, int);
  int (*CommDestroy)(NcclComm);
  int (*CommAbort)(NcclComm);
  int (*AllReduce)(const void*, void*, size_t, int, int, NcclComm, cudaStream_t);
  int (*ReduceScatter)(const void*, void*, size_t, int, int, NcclComm, cudaStream_t);
  int (*AllGather)(const void*, void*, size_t, int, NcclComm, cudaStream_t);
  const char* (*GetErrorString)(int);
};
NcclApi g_nccl;

int load_nccl(mb_ctx* ctx) {
  if (ctx->nccl_lib) return MB_OK;
  void* lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
  if (!lib) lib = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
  if (!lib) return mb_fail(ctx, MB_ERR_UNAVAILABLE, "NCCL could not be loaded: %s", dlerror());
#define SYM(field, name)                                                     \
  *reinterpret_cast<void**>(&g_nccl.field) = dlsym(lib, name);               \
  if (!g_nccl.field) return mb_fail(ctx, MB_ERR_UNAVAILABLE, "NCCL lacks %s", name);
  SYM(GetUniqueId, "ncclGetUniqueId")
  SYM(CommInitRank, "ncclCommInitRank")
  SYM(CommDestroy, "ncclCommDestroy")
  SYM(CommAbort, "ncclCommAbort")
  SYM(AllReduce, "ncclAllReduce")
  SYM(ReduceScatter, "ncclReduceScatter")
  SYM(AllGather, "ncclAllGather")
  SYM(GetErrorString, "ncclGetErrorString")
#undef SYM
  ctx->nccl_lib = lib;
  return MB_OK;
}

#define MB_NCCL_OK(ctx, expr)                                                                        \
  do {                                                                                               \
    int r__ = (expr);                                                                                \
    if (r__ != 0) return mb_fail(ctx, MB_ERR_CUDA, "%s failed: %s", #expr, g_nccl.GetErrorString(r__)); \
  } while (0)

}  // namespace

MB_API int mb_tp_shard(size_t rank, size_t world, size_t extent, size_t* lo, size_t* hi) {
  if (!lo || !hi || world == 0 || rank >= world || extent % world != 0) return MB_ERR_INVALID;
  size_t per = extent / world;
  *lo = rank * per;
  *hi = (rank + 1) * per;
  return MB_OK;
}

MB_API int mb_tp_unique_id(mb_ctx* ctx, uint8_t id_out[128]) {
  MB_REQUIRE(ctx, ctx && id_out, "tp_unique_id: null argument");
  int rc = load_nccl(ctx);
  if (rc) return rc;
  NcclUniqueId id;
  MB_NCCL_OK(ctx, g_nccl.GetUniqueId(&id));
  memcpy(id_out, id.internal, 128);
  return MB_OK;
}

MB_API int mb_tp_form(mb_ctx* ctx, const uint8_t id[128], int rank, int world) {
  MB_REQUIRE(ctx, ctx && id, "tp_form: null argument");
  MB_REQUIRE(ctx, world >= 1 && rank >= 0 && rank < world, "tp_form: rank %d of %d", rank, world);
  MB_REQUIRE(ctx, ctx->nccl_comm == nullptr, "tp_form: this context already holds a group");
  int rc = load_nccl(ctx);
  if (rc) return rc;
  MB_CUDA_OK(ctx, cudaSetDevice(ctx->device));
  NcclUniqueId uid;
  memcpy(uid.internal, id, 128);
  NcclComm comm = nullptr;
  MB_NCCL_OK(ctx, g_nccl.CommInitRank(&comm, world, uid, rank));
  ctx->nccl_comm = comm;
  ctx->tp_rank = rank;
  ctx->tp_world = world;
  return MB_OK;
}

MB_API int mb_tp_all_reduce(mb_ctx* ctx, mb_stream stream, void* buf, size_t count, int dtype) {
  MB_REQUIRE(ctx, ctx && buf, "tp_all_reduce: null argument");
  MB_REQUIRE(ctx, dtype == MB_DT_F32 || dtype == MB_DT_BF16, "tp_all_reduce: f32 or bf16");
  if (ctx->tp_world == 1 && !ctx->nccl_comm) return MB_OK;   // the identity world shards nothing
  MB_REQUIRE(ctx, ctx->nccl_comm != nullptr, "tp_all_reduce: no group formed");
  MB_NCCL_OK(ctx, g_nccl.AllReduce(buf, buf, count, dtype == MB_DT_F32 ? NCCL_FLOAT32 : NCCL_BFLOAT16, NCCL_SUM,
                                   ctx->nccl_comm, static_cast<cudaStream_t>(stream)));
  return MB_OK;
}

// The two halves of the all-reduce, for the prompt path that works on its own rows between them: SUM
// reduce-scatter of f32 ([world x count] in, this rank's [count] out) and all-gather of raw bytes ([bytes] in
// at recv + rank * bytes or elsewhere, [world x bytes] out; in place when send == recv + rank * bytes).
MB_API int mb_tp_reduce_scatter_f32(mb_ctx* ctx, mb_stream stream, const float* send, float* recv, size_t recv_count) {
  MB_REQUIRE(ctx, ctx && send && recv && recv_count > 0, "tp_reduce_scatter_f32: null or empty argument");
  if (ctx->tp_world == 1 && !ctx->nccl_comm) {
    if (send != recv)
      MB_CUDA_OK(ctx, cudaMemcpyAsync(recv, send, recv_count * sizeof(float), cudaMemcpyDeviceToDevice,
                                      static_cast<cudaStream_t>(stream)));
    return MB_OK;
  }
  MB_REQUIRE(ctx, ctx->nccl_comm != nullptr, "tp_reduce_scatter_f32: no group formed");
  MB_NCCL_OK(ctx, g_nccl.ReduceScatter(send, recv, recv_count, NCCL_FLOAT32, NCCL_SUM, ctx->nccl_comm,
                                       static_cast<cudaStream_t>(stream)));
  return MB_OK;
}

MB_API int mb_tp_all_gather(mb_ctx* ctx, mb_stream stream, const void* send, void* recv, size_t send_bytes) {
  MB_REQUIRE(ctx, ctx && send && recv && send_bytes > 0, "tp_all_gather: null or empty argument");
  if (ctx->tp_world == 1 && !ctx->nccl_comm) {
    if (send != recv)
      MB_CUDA_OK(ctx, cudaMemcpyAsync(recv, send, send_bytes, cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(stream)));
    return MB_OK;
  }
  MB_REQUIRE(ctx, ctx->nccl_comm != nullptr, "tp_all_gather: no group formed");
  MB_NCCL_OK(ctx, g_nccl.AllGather(send, recv, send_bytes, NCCL_UINT8, ctx->nccl_comm, static_cast<cudaStream_t>(stream)));
  return MB_OK;
}

// One all-reduce of ones; the sum must equal the world size on every rank.
MB_API int mb_tp_warm(mb_ctx* ctx, mb_stream stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  MB_REQUIRE(ctx, ctx != nullptr, "tp_warm: null context");
  std::lock_guard<std::mutex> scratch(ctx->scratch_mu);
  float* probe = reinterpret_cast<float*>(ctx->flags_dev + MB_FLAG_COUNT + 4);
  float one = 1.0f, got = 0.0f;
  MB_CUDA_OK(ctx, cudaMemcpyAsync(probe, &one, 4, cudaMemcpyHostToDevice, stream));
  int rc = mb_tp_all_reduce(ctx, stream_, probe, 1, MB_DT_F32);
  if (rc) return rc;
  MB_CUDA_OK(ctx, cudaMemcpyAsync(&got, probe, 4, cudaMemcpyDeviceToHost, stream));
  MB_CUDA_OK(ctx, cudaStreamSynchronize(stream));
  if (got != float(ctx->tp_world))
    return mb_fail(ctx, MB_ERR_CUDA, "tp_warm: the sum of ones is %g in a world of %d", double(got), ctx->tp_world);
  return MB_OK;
}

MB_API int mb_tp_close(mb_ctx* ctx) {
  if (!ctx) return MB_ERR_INVALID;
  if (ctx->nccl_comm) {
    g_nccl.CommDestroy(ctx->nccl_comm);
    ctx->nccl_comm = nullptr;
  }
  ctx->tp_rank = 0;
  ctx->tp_world = 1;
  return MB_OK;
}

// ---------------------------------------------------------------------------------
// Fused row-parallel path over peer memory.
//
// The row-parallel GEMM (o, down) pushes its f32 partial tiles from its epilogue straight
// into the owning rank's receive area (reduce-scatter by peer stores, overlapped with the
// MMAs of the next tile: mb_nvfp4_gemm_w4a4_scatter). The kernel below then, on every rank:
//   A  tells every peer "my partials of step s have landed" and waits for theirs,
//   B  sums its column slice over the source slots in rank order (deterministic), rounds
//      to bf16, adds the residual, and stores the result into EVERY rank's output buffer
//      (all-gather by peer stores),
//   C  tells every peer "my slice of step s has landed" once all its CTAs are done,
//   D  waits for every peer's slice before it ends, so that the next kernel on the stream
//      may read the whole output.
// Plain peer loads/stores only (no multicast). Every wait is bounded; a wait that runs out
// raises the context's timeout word and the kernel ends without reducing or publishing anything;
// the exchange is still counted, so the following exchange finds its counters in order. The grid
// never exceeds the SM count, so CTAs waiting in A or D cannot keep the others from running.
// ---------------------------------------------------------------------------------
namespace {

struct ReduceParams {
  void* const* peer;          // device table of every rank's exchange memory
  const __nv_bfloat16* resid; // [t, n] replicated residual stream
  int* done_counter;          // two counters, one per step parity, then the exchange counter (word 2)
  int* flags;                 // the context's status words
  unsigned long long wait_ns; // budget of one wait on the peers
  uint32_t t, n, nw, t_max, world, rank;
  int step;
};

__device__ __forceinline__ int* symm_flags(void* base) { return static_cast<int*>(base); }
__device__ __forceinline__ unsigned long long wall_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Waits until every rank's flag has reached `step`, for at most `wait_ns` of wall time. A wait that runs out
// puts `code` into the context's timeout word; the first one of the context also leaves the time waited
// (microseconds) in word 3 and the rank it was waiting for in word 4.
__device__ bool wait_flags(volatile int* flags, uint32_t world, int step, int* status, unsigned long long wait_ns,
                           int code) {
  const unsigned long long t0 = wall_ns();
  for (uint32_t r = 0; r < world; ++r) {
    while (flags[r] < step) {
      const unsigned long long waited = wall_ns() - t0;
      if (waited > wait_ns) {
        if (status && atomicCAS(status + MB_FLAG_WAIT_TIMEOUT, 0, code) == 0) {
          status[3] = int(waited / 1000ull);
          status[4] = int(r);
        }
        return false;
      }
    }
  }
  return true;
}

__global__ void __launch_bounds__(256)
tp_reduce_gather_kernel(const ReduceParams p_in) {
  __shared__ int s_ok;
  // The number of this exchange comes from a counter in device memory (the exchanges completed so far, plus one),
  // not from the launch parameters, so that a captured graph of the layer can be replayed: every replay then waits
  // for, and publishes, flag values of its own. The host's number only has to agree in parity (it chose the halves
  // of the exchange memory by it); a disagreement raises status code 53 and the kernel ends.
  ReduceParams p = p_in;
  p.step = p_in.done_counter[2] + 1;
  if ((p.step ^ p_in.step) & 1) {
    if (threadIdx.x == 0 && p.flags) atomicCAS(p.flags + MB_FLAG_WAIT_TIMEOUT, 0, 53);
    return;
  }
  void* const local = p.peer[p.rank];
  // ---- A: my partials have landed everywhere (the GEMM kernel before this one is complete)
  if (blockIdx.x == 0 && threadIdx.x < p.world) {
    __threadfence_system();
    volatile int* f = symm_flags(p.peer[threadIdx.x]);
    f[p.rank] = p.step;
  }
  // The counter of the other step parity is cleared here for the next step: the kernel that used it has ended
  // (stream order), also when it gave up in a wait and left its count unfinished.
  if (blockIdx.x == 0 && threadIdx.x == 0) p.done_counter[(p.step + 1) & 1] = 0;
  if (threadIdx.x == 0) s_ok = wait_flags(symm_flags(local), p.world, p.step, p.flags, p.wait_ns, 51) ? 1 : 0;
  __syncthreads();
  const bool ok = s_ok != 0;       // a wait that ran out: nothing is reduced or published, but the exchange is still counted
  __threadfence_system();
  // ---- B: reduce my slice, add the residual, store it into every rank's output
  const size_t half_recv = size_t(p.t_max) * p.n;                    // floats per step parity
  const float* recv = reinterpret_cast<const float*>(static_cast<uint8_t*>(local) + mb_symm_flags_bytes()) +
                      size_t(p.step & 1) * half_recv;
  const size_t out_off = mb_symm_flags_bytes() + mb_symm_recv_bytes(p.t_max, p.n) +
                         size_t(p.step & 1) * size_t(p.t_max) * p.n * 2;
  const uint32_t groups_per_row = p.nw / 8;
  const size_t total = size_t(p.t) * groups_per_row;
  for (size_t g = size_t(blockIdx.x) * 256 + threadIdx.x; ok && g < total; g += size_t(gridDim.x) * 256) {
    const uint32_t row = uint32_t(g / groups_per_row), c = uint32_t(g % groups_per_row) * 8;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (uint32_t r = 0; r < p.world; ++r) {
      const float4* src = reinterpret_cast<const float4*>(recv + (size_t(r) * p.t_max + row) * p.nw + c);
      const float4 a = src[0], b = src[1];
      acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
      acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
    }
    const uint32_t col = p.rank * p.nw + c;
    const uint4 rv = *reinterpret_cast<const uint4*>(p.resid + size_t(row) * p.n + col);
    const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
    uint32_t ow[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      // out = bf16(resid + bf16(sum)): the rounding points of add(x, linear(..))
      const float s0 = __bfloat162float(__float2bfloat16_rn(acc[2 * i]));
      const float s1 = __bfloat162float(__float2bfloat16_rn(acc[2 * i + 1]));
      __nv_bfloat162 o = __floats2bfloat162_rn(__uint_as_float(rw[i] << 16) + s0,
                                               __uint_as_float(rw[i] & 0xFFFF0000u) + s1);
      ow[i] = *reinterpret_cast<uint32_t*>(&o);
    }
    const uint4 ov = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    for (uint32_t r = 0; r < p.world; ++r) {
      __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(static_cast<uint8_t*>(p.peer[r]) + out_off);
      *reinterpret_cast<uint4*>(dst + size_t(row) * p.n + col) = ov;
    }
  }
  // ---- C: the last CTA of this rank tells every peer that the slice has landed
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int done = atomicAdd(p.done_counter + (p.step & 1), 1);
    if (done == int(gridDim.x) - 1) {
      p.done_counter[2] = p.step;          // every CTA of this exchange has read the counter: the exchange is counted
      __threadfence_system();
      for (uint32_t r = 0; ok && r < p.world; ++r) {
        volatile int* f = symm_flags(p.peer[r]) + 64;
        f[p.rank] = p.step;
      }
    }
    // ---- D: every rank's slice is in my output before this kernel ends
    if (ok) wait_flags(symm_flags(local) + 64, p.world, p.step, p.flags, p.wait_ns, 52);
    __threadfence_system();
  }
}

}  // namespace

MB_API size_t mb_tp_symm_bytes(size_t t_max, size_t n) {
  return mb_symm_flags_bytes() + mb_symm_recv_bytes(t_max, n) + mb_symm_out_bytes(t_max, n);
}

MB_API int mb_tp_symm_create(mb_ctx* ctx, size_t t_max, size_t n, uint8_t handle_out[64]) {
  MB_REQUIRE(ctx, ctx && handle_out && t_max > 0 && n > 0 && n % 8 == 0, "tp_symm_create: bad arguments");
  MB_REQUIRE(ctx, ctx->symm == nullptr, "tp_symm_create: this context already holds exchange memory");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  MB_CUDA_OK(ctx, cudaSetDevice(ctx->device));
  mb_symm* sy = new mb_symm();
  sy->t_max = t_max; sy->n = n; sy->bytes = mb_tp_symm_bytes(t_max, n);
  MB_CUDA_OK(ctx, cudaMalloc(&sy->local, sy->bytes));
  MB_CUDA_OK(ctx, cudaMemset(sy->local, 0, sy->bytes));
  MB_CUDA_OK(ctx, cudaMalloc(&sy->peer_dev, 8 * sizeof(void*)));
  MB_CUDA_OK(ctx, cudaMalloc(&sy->done_counter, 4 * sizeof(int)));
  MB_CUDA_OK(ctx, cudaMemset(sy->done_counter, 0, 4 * sizeof(int)));
  cudaIpcMemHandle_t h;
  MB_CUDA_OK(ctx, cudaIpcGetMemHandle(&h, sy->local));
  memcpy(handle_out, &h, 64);
  ctx->symm = sy;
  return MB_OK;
}

MB_API int mb_tp_symm_attach(mb_ctx* ctx, const uint8_t* handles, int rank, int world) {
  MB_REQUIRE(ctx, ctx && ctx->symm && handles, "tp_symm_attach: create the exchange memory first");
  MB_REQUIRE(ctx, world >= 1 && world <= 8 && rank >= 0 && rank < world, "tp_symm_attach: rank %d of %d", rank, world);
  mb_symm* sy = ctx->symm;
  MB_REQUIRE(ctx, sy->n % size_t(world) == 0 && (sy->n / world) % 32 == 0, "tp_symm_attach: n / world must be a multiple of 32");
  MB_CUDA_OK(ctx, cudaSetDevice(ctx->device));
  sy->world = world; sy->rank = rank; sy->ipc = true;
  for (int r = 0; r < world; ++r) {
    if (r == rank) { sy->peer[r] = sy->local; continue; }
    cudaIpcMemHandle_t h;
    memcpy(&h, handles + 64 * r, 64);
    MB_CUDA_OK(ctx, cudaIpcOpenMemHandle(&sy->peer[r], h, cudaIpcMemLazyEnablePeerAccess));
  }
  MB_CUDA_OK(ctx, cudaMemcpy(sy->peer_dev, sy->peer, 8 * sizeof(void*), cudaMemcpyHostToDevice));
  return MB_OK;
}

MB_API int mb_tp_symm_local(mb_ctx* ctx, void** local_out) {
  MB_REQUIRE(ctx, ctx && ctx->symm && local_out, "tp_symm_local: create the exchange memory first");
  *local_out = ctx->symm->local;
  return MB_OK;
}

MB_API int mb_tp_symm_attach_ptrs(mb_ctx* ctx, void* const* peers, int rank, int world) {
  MB_REQUIRE(ctx, ctx && ctx->symm && peers, "tp_symm_attach_ptrs: create the exchange memory first");
  MB_REQUIRE(ctx, world >= 1 && world <= 8 && rank >= 0 && rank < world, "tp_symm_attach_ptrs: rank %d of %d", rank, world);
  mb_symm* sy = ctx->symm;
  MB_REQUIRE(ctx, sy->n % size_t(world) == 0 && (sy->n / world) % 32 == 0, "tp_symm_attach_ptrs: n / world must be a multiple of 32");
  for (int r = 0; r < world; ++r)
    MB_REQUIRE(ctx, r == rank || (peers[r] != nullptr && mb_aligned(peers[r], 256)), "tp_symm_attach_ptrs: peer %d is null or unaligned", r);
  MB_CUDA_OK(ctx, cudaSetDevice(ctx->device));
  sy->world = world; sy->rank = rank; sy->ipc = false;
  for (int r = 0; r < world; ++r) sy->peer[r] = r == rank ? sy->local : peers[r];
  MB_CUDA_OK(ctx, cudaMemcpy(sy->peer_dev, sy->peer, 8 * sizeof(void*), cudaMemcpyHostToDevice));
  return MB_OK;
}

MB_API int mb_tp_reduce_residual(mb_ctx* ctx, mb_stream stream_, const void* resid_bf16, size_t t, size_t n, int step,
                                 void** out_dev) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  MB_REQUIRE(ctx, ctx && ctx->symm && resid_bf16 && out_dev, "tp_reduce_residual: null argument");
  mb_symm* sy = ctx->symm;
  MB_REQUIRE(ctx, n == sy->n && t > 0 && t <= sy->t_max, "tp_reduce_residual: [%zu, %zu] does not fit the exchange memory", t, n);
  MB_REQUIRE(ctx, step > 0, "tp_reduce_residual: steps count from 1");
  MB_REQUIRE(ctx, mb_aligned(resid_bf16, 16), "tp_reduce_residual: 16-byte alignment");
  ReduceParams p;
  p.peer = sy->peer_dev; p.resid = static_cast<const __nv_bfloat16*>(resid_bf16); p.done_counter = sy->done_counter;
  p.flags = ctx->flags_dev;
  p.wait_ns = uint64_t(ctx->wait_limit_us) * 1000ull;
  p.t = uint32_t(t); p.n = uint32_t(n); p.nw = uint32_t(n / sy->world); p.t_max = uint32_t(sy->t_max);
  p.world = uint32_t(sy->world); p.rank = uint32_t(sy->rank); p.step = step;
  const size_t total = t * (p.nw / 8);
  unsigned grid = unsigned(std::min<size_t>((total + 255) / 256, size_t(ctx->sm_count)));
  tp_reduce_gather_kernel<<<grid, 256, 0, stream>>>(p);
  MB_LAUNCH_OK(ctx);
  *out_dev = static_cast<uint8_t*>(sy->local) + mb_symm_flags_bytes() + mb_symm_recv_bytes(sy->t_max, sy->n) +
             size_t(step & 1) * sy->t_max * sy->n * 2;
  return MB_OK;
}

MB_API int mb_tp_symm_destroy(mb_ctx* ctx) {
  if (!ctx || !ctx->symm) return MB_OK;
  mb_symm* sy = ctx->symm;
  cudaDeviceSynchronize();
  for (int r = 0; r < sy->world; ++r)
    if (sy->ipc && r != sy->rank && sy->peer[r]) cudaIpcCloseMemHandle(sy->peer[r]);
  cudaFree(sy->local);
  cudaFree(sy->peer_dev);
  cudaFree(sy->done_counter);
  delete sy;
  ctx->symm = nullptr;
  return MB_OK;
}
