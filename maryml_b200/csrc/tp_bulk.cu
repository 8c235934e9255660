// Prompt-sized exchanges of the sharded layer over peer memory (NVLink 5 / NVSwitch), one process per GPU.
//
// The two halves of the layer's all-reduce (tp_reduce, src/models/inkling/tpcomm.rs:1453-1467) for a prompt whose
// rows stay sharded between them: a SUM reduce-scatter of the f32 partial by rows and an all-gather of whatever
// the next product reads. Both are kernels of this library over a region of device memory that every rank maps
// (CUDA IPC), with plain peer loads and stores and flags, no multicast:
//
//   reduce-scatter  every rank's row-parallel product writes its f32 partial into its own part of the region; a
//                   rank tells the peers that its partial is complete, waits for theirs, and reads ITS rows out of
//                   every rank's partial with 16-byte peer loads, adding in rank order (deterministic) into local
//                   memory: what crosses the links is the rows a rank owns, once, with no staging copy;
//   all-gather      every rank has written its slice at its place in its own copy of the buffer; it pushes that
//                   slice to the same place in every peer's copy, tells them, and waits until all slices are in.
//
// A partial or a gathered buffer may be written again two exchanges of the same kind later (the callers alternate
// between two of each): a rank reaches that point only after waits that every peer answers after it has finished
// reading. Every wait is bounded by wall
// time (the context's wait limit); one that runs out raises status 54 (reduce-scatter) or 55 (all-gather), the
// kernel skips what depended on it and ends, and the context stays usable.
#include "common.cuh"

namespace {

constexpr size_t BULK_HEADER = 4096;        // flags: ints [0, 8) reduce-scatter steps by source rank, [32, 40) all-gather
constexpr int RS_FLAGS = 0, AG_FLAGS = 32;

struct BulkCommon {
  void* const* peer;          // device table of every rank's region
  int* counters;              // [0]: CTAs of the running kernel that finished pushing
  int* flags;                 // the context's status words
  unsigned long long wait_ns;
  uint32_t world, rank;
  int step;
};

__device__ __forceinline__ unsigned long long wall_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ bool wait_steps(volatile int* f, uint32_t world, int step, int* status, unsigned long long wait_ns, int code) {
  const unsigned long long t0 = wall_ns();
  for (uint32_t r = 0; r < world; ++r) {
    while (f[r] < step) {
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

// Every CTA calls this after its own peer stores: the last one to arrive tells every peer that this rank's bytes
// of `step` have landed (flag word `base + rank` in the peer's header).
__device__ void publish_when_all_ctas_done(const BulkCommon& c, int base) {
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int done = atomicAdd(c.counters, 1);
    if (done == int(gridDim.x) - 1) {
      c.counters[0] = 0;                        // the next kernel of this context starts from zero (stream order)
      __threadfence_system();
      for (uint32_t q = 0; q < c.world; ++q) {
        volatile int* f = static_cast<int*>(c.peer[q]);
        f[base + c.rank] = c.step;
      }
      __threadfence_system();
    }
  }
}

struct RsParams {
  BulkCommon c;
  float4* out;                // [rows / world, n] f32, local
  size_t part_off;            // byte offset (region's user part) of every rank's [rows, n] f32 partial
  size_t slice4;              // float4 units of one rank's rows = (rows / world) * n / 4
};

// 16 bytes from a peer's memory, fetched anew (no cached copy of that line is trusted).
__device__ __forceinline__ float4 peer_load(const float4* p) {
  float4 v;
  asm volatile("ld.volatile.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
  return v;
}

// Every rank's partial lies in its own part of the region (its row-parallel product wrote it there). A rank tells
// the peers that its partial is complete, waits for theirs, and then reads ITS rows out of every rank's partial
// with peer loads (the local one included), adding in rank order: what crosses the links is exactly the rows this
// rank owns, once, and nothing is staged in between.
__global__ void __launch_bounds__(512)
bulk_reduce_scatter_kernel(const RsParams p) {
  __shared__ int s_ok;
  const BulkCommon& c = p.c;
  if (blockIdx.x == 0 && threadIdx.x < c.world) {
    __threadfence_system();                    // the product before this kernel is complete: make it visible to the peers
    volatile int* f = static_cast<int*>(c.peer[threadIdx.x]);
    f[RS_FLAGS + c.rank] = c.step;
  }
  if (threadIdx.x == 0)
    s_ok = wait_steps(static_cast<int*>(c.peer[c.rank]) + RS_FLAGS, c.world, c.step, c.flags, c.wait_ns, 54) ? 1 : 0;
  __syncthreads();
  if (!s_ok) return;
  __threadfence_system();
  const size_t per = p.slice4;
  const size_t stride = size_t(gridDim.x) * blockDim.x;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < per; i += 2 * stride) {
    const size_t j = i + stride;
    const bool two = j < per;
    // all loads of both units first (up to sixteen 16-byte peer loads in flight per thread), then the sums
    float4 a[8], b[8];
#pragma unroll
    for (uint32_t r = 0; r < 8; ++r) {
      if (r < c.world) {
        const float4* src = reinterpret_cast<const float4*>(static_cast<const uint8_t*>(c.peer[r]) + BULK_HEADER + p.part_off) +
                            size_t(c.rank) * per;
        a[r] = peer_load(src + i);
        if (two) b[r] = peer_load(src + j);
      }
    }
    float4 sa = a[0], sb = two ? b[0] : a[0];
#pragma unroll
    for (uint32_t r = 1; r < 8; ++r) {
      if (r < c.world) {
        sa.x += a[r].x; sa.y += a[r].y; sa.z += a[r].z; sa.w += a[r].w;
        if (two) { sb.x += b[r].x; sb.y += b[r].y; sb.z += b[r].z; sb.w += b[r].w; }
      }
    }
    p.out[i] = sa;
    if (two) p.out[j] = sb;
  }
}

struct AgParams {
  BulkCommon c;
  size_t off[2];              // byte offsets (region's user part) of up to two gathered buffers
  size_t part4[2];            // uint4 units of one rank's slice of each (0: unused)
};

__global__ void __launch_bounds__(512)
bulk_all_gather_kernel(const AgParams p) {
  const BulkCommon& c = p.c;
  uint8_t* mine = static_cast<uint8_t*>(c.peer[c.rank]) + BULK_HEADER;
  for (int b = 0; b < 2; ++b) {
    const size_t per = p.part4[b];
    if (!per) continue;
    const uint4* src = reinterpret_cast<const uint4*>(mine + p.off[b]) + size_t(c.rank) * per;
    // a unit of the slice is loaded once and stored to every peer
    const size_t stride = size_t(gridDim.x) * blockDim.x;
    for (size_t e = size_t(blockIdx.x) * blockDim.x + threadIdx.x; e < per; e += 2 * stride) {
      const bool two = e + stride < per;
      const uint4 v0 = __ldcg(src + e);
      uint4 v1 = v0;
      if (two) v1 = __ldcg(src + e + stride);
      for (uint32_t hop = 0; hop + 1 < c.world; ++hop) {
        const uint32_t q = (c.rank + 1 + hop) % c.world;
        uint4* dst = reinterpret_cast<uint4*>(static_cast<uint8_t*>(c.peer[q]) + BULK_HEADER + p.off[b]) + size_t(c.rank) * per;
        dst[e] = v0;
        if (two) dst[e + stride] = v1;
      }
    }

  }
  publish_when_all_ctas_done(c, AG_FLAGS);
  // the kernel ends (and the next one on the stream may read the whole buffers) once every slice is in
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    wait_steps(static_cast<int*>(c.peer[c.rank]) + AG_FLAGS, c.world, c.step, c.flags, c.wait_ns, 55);
    __threadfence_system();
  }
}

int fill_common(mb_ctx* ctx, BulkCommon* c, int step, const char* what) {
  MB_REQUIRE(ctx, ctx && ctx->bulk && ctx->bulk->world > 0, "%s: create and attach the bulk exchange memory first", what);
  MB_REQUIRE(ctx, step > 0, "%s: steps count from 1", what);
  const mb_bulk* bk = ctx->bulk;
  c->peer = bk->peer_dev; c->counters = bk->counters; c->flags = ctx->flags_dev;
  c->wait_ns = uint64_t(ctx->wait_limit_us) * 1000ull;
  c->world = uint32_t(bk->world); c->rank = uint32_t(bk->rank); c->step = step;
  return MB_OK;
}

}  // namespace

MB_API size_t mb_tp_bulk_header_bytes(void) { return BULK_HEADER; }

MB_API int mb_tp_bulk_create(mb_ctx* ctx, size_t user_bytes, uint8_t handle_out[64]) {
  MB_REQUIRE(ctx, ctx && handle_out && user_bytes > 0 && user_bytes % 256 == 0, "tp_bulk_create: bad arguments");
  MB_REQUIRE(ctx, ctx->bulk == nullptr, "tp_bulk_create: this context already holds bulk exchange memory");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  MB_CUDA_OK(ctx, cudaSetDevice(ctx->device));
  mb_bulk* bk = new mb_bulk();
  bk->bytes = BULK_HEADER + user_bytes;
  cudaError_t e = cudaMalloc(&bk->local, bk->bytes);
  if (e != cudaSuccess) {
    delete bk;
    return mb_fail(ctx, MB_ERR_CUDA, "tp_bulk_create: cudaMalloc of %zu bytes failed: %s", BULK_HEADER + user_bytes, cudaGetErrorString(e));
  }
  MB_CUDA_OK(ctx, cudaMemset(bk->local, 0, BULK_HEADER));
  MB_CUDA_OK(ctx, cudaMalloc(&bk->peer_dev, 8 * sizeof(void*)));
  MB_CUDA_OK(ctx, cudaMalloc(&bk->counters, 4 * sizeof(int)));
  MB_CUDA_OK(ctx, cudaMemset(bk->counters, 0, 4 * sizeof(int)));
  cudaIpcMemHandle_t h;
  MB_CUDA_OK(ctx, cudaIpcGetMemHandle(&h, bk->local));
  memcpy(handle_out, &h, 64);
  ctx->bulk = bk;
  return MB_OK;
}

MB_API int mb_tp_bulk_attach(mb_ctx* ctx, const uint8_t* handles, int rank, int world) {
  MB_REQUIRE(ctx, ctx && ctx->bulk && handles, "tp_bulk_attach: create the bulk exchange memory first");
  MB_REQUIRE(ctx, world >= 1 && world <= 8 && rank >= 0 && rank < world, "tp_bulk_attach: rank %d of %d", rank, world);
  mb_bulk* bk = ctx->bulk;
  MB_CUDA_OK(ctx, cudaSetDevice(ctx->device));
  for (int r = 0; r < world; ++r) {
    if (r == rank) { bk->peer[r] = bk->local; continue; }
    cudaIpcMemHandle_t h;
    memcpy(&h, handles + 64 * r, 64);
    MB_CUDA_OK(ctx, cudaIpcOpenMemHandle(&bk->peer[r], h, cudaIpcMemLazyEnablePeerAccess));
  }
  bk->world = world; bk->rank = rank; bk->ipc = true;
  MB_CUDA_OK(ctx, cudaMemcpy(bk->peer_dev, bk->peer, 8 * sizeof(void*), cudaMemcpyHostToDevice));
  return MB_OK;
}

MB_API int mb_tp_bulk_attach_ptrs(mb_ctx* ctx, void* const* peers, int rank, int world) {
  MB_REQUIRE(ctx, ctx && ctx->bulk && peers, "tp_bulk_attach_ptrs: create the bulk exchange memory first");
  MB_REQUIRE(ctx, world >= 1 && world <= 8 && rank >= 0 && rank < world, "tp_bulk_attach_ptrs: rank %d of %d", rank, world);
  mb_bulk* bk = ctx->bulk;
  for (int r = 0; r < world; ++r)
    MB_REQUIRE(ctx, r == rank || (peers[r] != nullptr && mb_aligned(peers[r], 256)), "tp_bulk_attach_ptrs: peer %d is null or unaligned", r);
  MB_CUDA_OK(ctx, cudaSetDevice(ctx->device));
  for (int r = 0; r < world; ++r) bk->peer[r] = r == rank ? bk->local : peers[r];
  bk->world = world; bk->rank = rank; bk->ipc = false;
  MB_CUDA_OK(ctx, cudaMemcpy(bk->peer_dev, bk->peer, 8 * sizeof(void*), cudaMemcpyHostToDevice));
  return MB_OK;
}

MB_API int mb_tp_bulk_local(mb_ctx* ctx, void** region_out, void** user_out) {
  MB_REQUIRE(ctx, ctx && ctx->bulk && (region_out || user_out), "tp_bulk_local: create the bulk exchange memory first");
  if (region_out) *region_out = ctx->bulk->local;
  if (user_out) *user_out = static_cast<uint8_t*>(ctx->bulk->local) + BULK_HEADER;
  return MB_OK;
}

MB_API int mb_tp_bulk_reduce_scatter_f32(mb_ctx* ctx, mb_stream stream_, size_t partial_off, size_t rows, size_t n,
                                         float* out, int step) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  RsParams p;
  memset(&p, 0, sizeof p);
  int rc = fill_common(ctx, &p.c, step, "tp_bulk_reduce_scatter_f32");
  if (rc) return rc;
  const mb_bulk* bk = ctx->bulk;
  MB_REQUIRE(ctx, out && rows > 0 && n > 0, "tp_bulk_reduce_scatter_f32: null or empty argument");
  MB_REQUIRE(ctx, rows % size_t(bk->world) == 0 && n % 4 == 0, "tp_bulk_reduce_scatter_f32: rows must divide by the world and n by 4");
  MB_REQUIRE(ctx, mb_aligned(out, 16) && partial_off % 256 == 0, "tp_bulk_reduce_scatter_f32: alignment");
  MB_REQUIRE(ctx, BULK_HEADER + partial_off + rows * n * sizeof(float) <= bk->bytes,
             "tp_bulk_reduce_scatter_f32: the partial [%zu, +%zu) does not fit the region", partial_off, rows * n * sizeof(float));
  p.out = reinterpret_cast<float4*>(out);
  p.part_off = partial_off;
  p.slice4 = rows / size_t(bk->world) * n / 4;
  // never more CTAs than SMs: every CTA waits for the peers at its start and must be resident
  const int sms = ctx->sm_limit > 0 ? std::min(ctx->sm_limit, ctx->sm_count) : ctx->sm_count;
  const unsigned grid = unsigned(std::max<size_t>(1, std::min<size_t>(size_t(sms), (p.slice4 + 1023) / 1024)));
  bulk_reduce_scatter_kernel<<<grid, 512, 0, stream>>>(p);
  MB_LAUNCH_OK(ctx);
  return MB_OK;
}

MB_API int mb_tp_bulk_all_gather(mb_ctx* ctx, mb_stream stream_, size_t off0, size_t part_bytes0, size_t off1,
                                 size_t part_bytes1, int step) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  AgParams p;
  memset(&p, 0, sizeof p);
  int rc = fill_common(ctx, &p.c, step, "tp_bulk_all_gather");
  if (rc) return rc;
  const mb_bulk* bk = ctx->bulk;
  MB_REQUIRE(ctx, part_bytes0 > 0 && part_bytes0 % 16 == 0 && part_bytes1 % 16 == 0 && off0 % 256 == 0 && off1 % 256 == 0,
             "tp_bulk_all_gather: slices are multiples of 16 bytes at 256-byte aligned offsets");
  MB_REQUIRE(ctx, BULK_HEADER + off0 + part_bytes0 * bk->world <= bk->bytes &&
                      (part_bytes1 == 0 || BULK_HEADER + off1 + part_bytes1 * bk->world <= bk->bytes),
             "tp_bulk_all_gather: a gathered buffer does not fit the region");
  p.off[0] = off0; p.part4[0] = part_bytes0 / 16;
  p.off[1] = off1; p.part4[1] = part_bytes1 / 16;
  const int sms = ctx->sm_limit > 0 ? std::min(ctx->sm_limit, ctx->sm_count) : ctx->sm_count;
  const size_t units = p.part4[0] + p.part4[1];
  const unsigned grid = unsigned(std::max<size_t>(1, std::min<size_t>(size_t(sms), (units + 1023) / 1024)));
  bulk_all_gather_kernel<<<grid, 512, 0, stream>>>(p);
  MB_LAUNCH_OK(ctx);
  return MB_OK;
}

MB_API int mb_tp_bulk_destroy(mb_ctx* ctx) {
  if (!ctx || !ctx->bulk) return MB_OK;
  mb_bulk* bk = ctx->bulk;
  cudaDeviceSynchronize();
  for (int r = 0; r < bk->world; ++r)
    if (bk->ipc && r != bk->rank && bk->peer[r]) cudaIpcCloseMemHandle(bk->peer[r]);
  cudaFree(bk->local);
  cudaFree(bk->peer_dev);
  cudaFree(bk->counters);
  delete bk;
  ctx->bulk = nullptr;
  return MB_OK;
}
