// Lifecycle, memory and timing entry points of the C ABI.
#include <stdlib.h>
#include "common.cuh"
#include <string.h>

thread_local std::string g_vn_thread_error;

extern "C" {

int32_t vn_version(void) { return 100; }

int32_t vn_ctx_create(int32_t device, vn_ctx** out) {
  if (!out) return vn_fail(nullptr, VN_ERR_INVALID, "out is null");
  *out = nullptr;
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess || n == 0)
    return vn_fail(nullptr, VN_ERR_CUDA, "no CUDA device: %s", cudaGetErrorString(e));
  if (device < 0 || device >= n) return vn_fail(nullptr, VN_ERR_INVALID, "device %d out of range (%d)", device, n);
  vn_ctx* ctx = new vn_ctx();
  ctx->device = device;
  e = cudaSetDevice(device);
  if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking);
  if (e != cudaSuccess) {
    delete ctx;
    return vn_fail(nullptr, VN_ERR_CUDA, "context setup: %s", cudaGetErrorString(e));
  }
  cudaDeviceGetAttribute(&ctx->sm_count, cudaDevAttrMultiProcessorCount, device);
  if (const char* e = getenv("VN_PDL")) ctx->pdl = atoi(e);
  *out = ctx;
  return VN_OK;
}

int32_t vn_ctx_destroy(vn_ctx* ctx) {
  if (!ctx) return VN_OK;
  cudaSetDevice(ctx->device);
  cudaStreamSynchronize(ctx->stream);
  if (ctx->ws) cudaFree(ctx->ws);
  if (ctx->flush) cudaFree(ctx->flush);
  if (ctx->tickets) cudaFree(ctx->tickets);
  cudaStreamDestroy(ctx->stream);
  delete ctx;
  return VN_OK;
}

const char* vn_last_error(vn_ctx* ctx) { return ctx ? ctx->err.c_str() : g_vn_thread_error.c_str(); }

int32_t vn_sync(vn_ctx* ctx) {
  VN_CHECK_CTX(ctx);
  VN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return VN_OK;
}

int32_t vn_launch_count(vn_ctx* ctx, uint64_t* out) {
  if (!ctx || !out) return vn_fail(ctx, VN_ERR_INVALID, "null argument");
  *out = ctx->launches;
  return VN_OK;
}

int32_t vn_stream(vn_ctx* ctx, void** out) {
  if (!ctx || !out) return vn_fail(ctx, VN_ERR_INVALID, "null argument");
  *out = (void*)ctx->stream;
  return VN_OK;
}

int32_t vn_alloc(vn_ctx* ctx, size_t bytes, void** out_dev) {
  VN_CHECK_CTX(ctx);
  VN_REQUIRE(ctx, out_dev, "out_dev is null");
  *out_dev = nullptr;
  if (bytes == 0) bytes = 16;
  VN_CUDA(ctx, cudaMalloc(out_dev, bytes));
  return VN_OK;
}

int32_t vn_free(vn_ctx* ctx, void* dev) {
  VN_CHECK_CTX(ctx);
  if (!dev) return VN_OK;
  VN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  VN_CUDA(ctx, cudaFree(dev));
  return VN_OK;
}

int32_t vn_memset(vn_ctx* ctx, void* dev, int32_t byte, size_t bytes) {
  VN_CHECK_CTX(ctx);
  VN_CUDA(ctx, cudaMemsetAsync(dev, byte, bytes, ctx->stream));
  return VN_OK;
}

int32_t vn_h2d(vn_ctx* ctx, void* dst_dev, const void* src, size_t bytes) {
  VN_CHECK_CTX(ctx);
  if (bytes == 0) return VN_OK;
  VN_REQUIRE(ctx, dst_dev && src, "null pointer");
  VN_CUDA(ctx, cudaMemcpyAsync(dst_dev, src, bytes, cudaMemcpyHostToDevice, ctx->stream));
  VN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return VN_OK;
}

int32_t vn_d2h(vn_ctx* ctx, void* dst, const void* src_dev, size_t bytes) {
  VN_CHECK_CTX(ctx);
  if (bytes == 0) return VN_OK;
  VN_REQUIRE(ctx, dst && src_dev, "null pointer");
  VN_CUDA(ctx, cudaMemcpyAsync(dst, src_dev, bytes, cudaMemcpyDeviceToHost, ctx->stream));
  VN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return VN_OK;
}

int32_t vn_d2d(vn_ctx* ctx, void* dst_dev, const void* src_dev, size_t bytes) {
  VN_CHECK_CTX(ctx);
  if (bytes == 0) return VN_OK;
  VN_CUDA(ctx, cudaMemcpyAsync(dst_dev, src_dev, bytes, cudaMemcpyDeviceToDevice, ctx->stream));
  return VN_OK;
}

int32_t vn_copy_2d(vn_ctx* ctx, void* dst_dev, size_t dst_pitch, const void* src_dev, size_t src_pitch, size_t width_bytes,
                   size_t rows) {
  VN_CHECK_CTX(ctx);
  VN_REQUIRE(ctx, dst_pitch >= width_bytes && src_pitch >= width_bytes, "pitch below the row width");
  if (width_bytes == 0 || rows == 0) return VN_OK;
  VN_CUDA(ctx, cudaMemcpy2DAsync(dst_dev, dst_pitch, src_dev, src_pitch, width_bytes, rows, cudaMemcpyDeviceToDevice,
                                 ctx->stream));
  return VN_OK;
}

int32_t vn_host_alloc(vn_ctx* ctx, size_t bytes, void** out) {
  VN_CHECK_CTX(ctx);
  VN_REQUIRE(ctx, out, "out is null");
  VN_CUDA(ctx, cudaMallocHost(out, bytes ? bytes : 16));
  return VN_OK;
}

int32_t vn_host_free(vn_ctx* ctx, void* p) {
  VN_CHECK_CTX(ctx);
  if (p) VN_CUDA(ctx, cudaFreeHost(p));
  return VN_OK;
}

int32_t vn_h2d_async(vn_ctx* ctx, void* dst_dev, const void* src_pinned, size_t bytes) {
  VN_CHECK_CTX(ctx);
  if (bytes == 0) return VN_OK;
  VN_CUDA(ctx, cudaMemcpyAsync(dst_dev, src_pinned, bytes, cudaMemcpyHostToDevice, ctx->stream));
  return VN_OK;
}

int32_t vn_d2h_async(vn_ctx* ctx, void* dst_pinned, const void* src_dev, size_t bytes) {
  VN_CHECK_CTX(ctx);
  if (bytes == 0) return VN_OK;
  VN_CUDA(ctx, cudaMemcpyAsync(dst_pinned, src_dev, bytes, cudaMemcpyDeviceToHost, ctx->stream));
  return VN_OK;
}

int32_t vn_mem_info(vn_ctx* ctx, size_t* free_bytes, size_t* total_bytes) {
  VN_CHECK_CTX(ctx);
  VN_CUDA(ctx, cudaMemGetInfo(free_bytes, total_bytes));
  return VN_OK;
}

int32_t vn_event_create(vn_ctx* ctx, void** out_event) {
  VN_CHECK_CTX(ctx);
  cudaEvent_t ev;
  VN_CUDA(ctx, cudaEventCreate(&ev));
  *out_event = (void*)ev;
  return VN_OK;
}

int32_t vn_event_destroy(vn_ctx* ctx, void* event) {
  VN_CHECK_CTX(ctx);
  if (event) VN_CUDA(ctx, cudaEventDestroy((cudaEvent_t)event));
  return VN_OK;
}

int32_t vn_event_record(vn_ctx* ctx, void* event) {
  VN_CHECK_CTX(ctx);
  VN_CUDA(ctx, cudaEventRecord((cudaEvent_t)event, ctx->stream));
  return VN_OK;
}

int32_t vn_event_elapsed_ms(vn_ctx* ctx, void* start, void* stop, float* out_ms) {
  VN_CHECK_CTX(ctx);
  VN_CUDA(ctx, cudaEventSynchronize((cudaEvent_t)stop));
  VN_CUDA(ctx, cudaEventElapsedTime(out_ms, (cudaEvent_t)start, (cudaEvent_t)stop));
  return VN_OK;
}

int32_t vn_flush_l2(vn_ctx* ctx) {
  VN_CHECK_CTX(ctx);
  const size_t bytes = 256u << 20;  // twice the 126 MB L2
  if (!ctx->flush) {
    VN_CUDA(ctx, cudaMalloc(&ctx->flush, bytes));
    ctx->flush_bytes = bytes;
  }
  VN_CUDA(ctx, cudaMemsetAsync(ctx->flush, 0, ctx->flush_bytes, ctx->stream));
  return VN_OK;
}

int32_t vn_profile(vn_ctx* ctx, int32_t enable) {
  VN_CHECK_CTX(ctx);
  VN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  for (auto& r : ctx->prof) { cudaEventDestroy(r.a); cudaEventDestroy(r.b); }
  ctx->prof.clear();
  ctx->profiling = enable != 0;
  return VN_OK;
}

int32_t vn_profile_report(vn_ctx* ctx, char* buf, size_t buf_bytes) {
  VN_CHECK_CTX(ctx);
  VN_REQUIRE(ctx, buf && buf_bytes > 2, "buffer missing");
  VN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  std::map<std::string, std::pair<uint64_t, double>> agg;
  for (auto& r : ctx->prof) {
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, r.a, r.b) == cudaSuccess) {
      auto& e = agg[r.name];
      e.first++;
      e.second += ms;
    }
  }
  std::string out = "{";
  bool first = true;
  for (auto& kv : agg) {
    char line[384];
    snprintf(line, sizeof line, "%s\"%s\": {\"launches\": %llu, \"ms\": %.6f}", first ? "" : ", ",
             kv.first.c_str(), (unsigned long long)kv.second.first, kv.second.second);
    out += line;
    first = false;
  }
  out += "}";
  VN_REQUIRE(ctx, out.size() + 1 <= buf_bytes, "report needs %zu bytes", out.size() + 1);
  memcpy(buf, out.c_str(), out.size() + 1);
  return VN_OK;
}

}  // extern "C"

void vn_prof_begin(vn_ctx* ctx, const char* name) {
  vn_ctx::ProfRec r;
  r.name = name;
  if (cudaEventCreate(&r.a) != cudaSuccess || cudaEventCreate(&r.b) != cudaSuccess) return;
  cudaEventRecord(r.a, ctx->stream);
  ctx->prof.push_back(r);
}

void vn_prof_end(vn_ctx* ctx) {
  if (!ctx->prof.empty()) cudaEventRecord(ctx->prof.back().b, ctx->stream);
}

int32_t vn_tickets(vn_ctx* ctx, int** out) {
  if (!ctx->tickets) {
    VN_CUDA(ctx, cudaMalloc((void**)&ctx->tickets, sizeof(int) * VN_TICKETS));
    VN_CUDA(ctx, cudaMemsetAsync(ctx->tickets, 0, sizeof(int) * VN_TICKETS, ctx->stream));
  }
  *out = ctx->tickets;
  return VN_OK;
}

int32_t vn_workspace(vn_ctx* ctx, size_t bytes, void** out) {
  if (bytes > ctx->ws_bytes) {
    VN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (ctx->ws) VN_CUDA(ctx, cudaFree(ctx->ws));
    ctx->ws = nullptr;
    ctx->ws_bytes = 0;
    size_t want = bytes + (bytes >> 2);
    VN_CUDA(ctx, cudaMalloc(&ctx->ws, want));
    ctx->ws_bytes = want;
  }
  *out = ctx->ws;
  return VN_OK;
}
