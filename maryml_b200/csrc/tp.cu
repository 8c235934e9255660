// Tensor-parallel plumbing: shard arithmetic and the SUM all-reduce over NCCL
// (NVLink 5 / NVSwitch on a B200 node). NCCL is loaded at run time from the
// process (the library torch already brought in) so that the kernels' shared
// object has no link-time dependency on it.
#include "common.cuh"

#include <dlfcn.h>

namespace {

typedef struct { char internal[128]; } NcclUniqueId;
typedef void* NcclComm;
enum { NCCL_SUM = 0, NCCL_FLOAT32 = 7, NCCL_BFLOAT16 = 9 };

struct NcclApi {
  int (*GetUniqueId)(NcclUniqueId*);
  int (*CommInitRank)(NcclComm*, int, NcclUniqueId, int);
  int (*CommDestroy)(NcclComm);
  int (*CommAbort)(NcclComm);
  int (*AllReduce)(const void*, void*, size_t, int, int, NcclComm, cudaStream_t);
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

// One all-reduce of ones; the sum must equal the world size on every rank.
MB_API int mb_tp_warm(mb_ctx* ctx, mb_stream stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  MB_REQUIRE(ctx, ctx != nullptr, "tp_warm: null context");
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
