// Context object and error reporting of the C ABI.
#include "common.cuh"

MB_API const char* mb_version(void) { return "mary-b200 0.1 (sm_100a)"; }

MB_API int mb_ctx_create(int device, mb_ctx** out) {
  if (!out) return MB_ERR_INVALID;
  *out = nullptr;
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || device < 0 || device >= count) return MB_ERR_CUDA;
  if (cudaSetDevice(device) != cudaSuccess) return MB_ERR_CUDA;
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return MB_ERR_CUDA;
  if (prop.major != 10) return MB_ERR_UNAVAILABLE;  // the kernels are sm_100a only; there is no fallback
  mb_ctx* ctx = new mb_ctx();
  ctx->device = device;
  ctx->sm_count = prop.multiProcessorCount;
  if (cudaMalloc(&ctx->flags_dev, (MB_FLAG_COUNT + 8) * sizeof(int)) != cudaSuccess ||
      cudaMemset(ctx->flags_dev, 0, (MB_FLAG_COUNT + 8) * sizeof(int)) != cudaSuccess) {
    delete ctx;
    return MB_ERR_CUDA;
  }
  // The allocation-free decode entry point's array and kernels are made resident now, while the host may still
  // allocate, not at its first call (which may come after the host's arena has taken the device's memory).
  if (mb_attention_decode_static_warm(ctx) != MB_OK) {
    cudaFree(ctx->flags_dev);
    delete ctx;
    return MB_ERR_CUDA;
  }
  *out = ctx;
  return MB_OK;
}

MB_API void mb_ctx_destroy(mb_ctx* ctx) {
  if (!ctx) return;
  mb_tp_symm_destroy(ctx);
  mb_tp_bulk_destroy(ctx);
  mb_tp_close(ctx);
  if (ctx->flags_dev) cudaFree(ctx->flags_dev);
  delete ctx;
}

MB_API int mb_ctx_set_sm_limit(mb_ctx* ctx, int sms) {
  MB_REQUIRE(ctx, ctx != nullptr, "set_sm_limit: null context");
  MB_REQUIRE(ctx, sms >= 0 && sms <= ctx->sm_count, "set_sm_limit: 0 (all) .. %d SMs, got %d", ctx->sm_count, sms);
  ctx->sm_limit = sms;
  return MB_OK;
}

MB_API int mb_ctx_set_wait_limit_us(mb_ctx* ctx, uint32_t microseconds) {
  MB_REQUIRE(ctx, ctx != nullptr, "set_wait_limit_us: null context");
  MB_REQUIRE(ctx, microseconds >= 100 && microseconds <= 60000000u, "set_wait_limit_us: 100 us .. 60 s, got %u", microseconds);
  ctx->wait_limit_us = microseconds;
  return MB_OK;
}

MB_API const char* mb_last_error(mb_ctx* ctx) {
  if (!ctx) return "no context";
  std::lock_guard<std::mutex> g(ctx->mu);
  return ctx->last_error.c_str();
}

MB_API int mb_check_flags(mb_ctx* ctx, mb_stream stream_, int32_t* flags_out8) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  MB_REQUIRE(ctx, ctx != nullptr, "check_flags: null context");
  int32_t host[MB_FLAG_COUNT];
  MB_CUDA_OK(ctx, cudaMemcpyAsync(host, ctx->flags_dev, sizeof host, cudaMemcpyDeviceToHost, stream));
  MB_CUDA_OK(ctx, cudaMemsetAsync(ctx->flags_dev, 0, sizeof host, stream));
  MB_CUDA_OK(ctx, cudaStreamSynchronize(stream));
  bool any = false;
  for (int i = 0; i < MB_FLAG_COUNT; ++i) {
    if (flags_out8) flags_out8[i] = host[i];
    any |= host[i] != 0;
  }
  if (any)
    return mb_fail(ctx, MB_ERR_DEVICE_FLAG, "device status: wait_timeout=%d router_nonfinite=%d plan_fault=%d",
                   host[MB_FLAG_WAIT_TIMEOUT], host[MB_FLAG_ROUTER_NONFINITE], host[MB_FLAG_PLAN_FAULT]);
  return MB_OK;
}
