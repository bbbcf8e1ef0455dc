// Shared host-side plumbing of the library: context, error reporting, launch accounting.
#pragma once
#include <stdlib.h>

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>
#include <string>
#include <vector>
#include <map>
#include <mutex>

#include "../../include/vn_b200.h"

struct vn_ctx {
  int device = 0;
  cudaStream_t stream = nullptr;
  std::string err;
  uint64_t launches = 0;
  // scratch owned by the context, grown on demand (never shrinks)
  void* ws = nullptr;
  size_t ws_bytes = 0;
  void* flush = nullptr;
  size_t flush_bytes = 0;
  // arrival counters for kernels whose last CTA finishes a row's work (VN_TICKETS ints, zero between kernels:
  // whoever takes the last ticket sets the counter back)
  int* tickets = nullptr;
  int sm_count = 148;
  // when set, every Philox offset of the acceptance / sampling kernels is incremented by *offset_src
  // (a round counter that lives on the device, so that a captured graph draws fresh numbers on every replay)
  const unsigned* offset_src = nullptr;
  // optional per-kernel timing: CUDA events around every launch, summed per kernel name
  bool profiling = false;
  // programmatic dependent launch: kernels launched through VN_LAUNCH_PDL may start while their predecessor
  // in the stream drains; each of them waits (pdl_wait) before it touches anything a predecessor wrote.
  // Level 0 (VN_PDL=0): plain stream order.  1 (default): only the weight-streaming GEMMs, which prefetch
  // weight tiles before they wait (+4 % rounds per second on B200).  2: every kernel that supports it (measured
  // no better than 0: waiting CTAs of the small kernels only take up SM slots).
  int pdl = 1;
  struct ProfRec { const char* name; cudaEvent_t a, b; };
  std::vector<ProfRec> prof;
};

constexpr int VN_TICKETS = 1 << 16;
int32_t vn_tickets(vn_ctx* ctx, int** out);
void vn_prof_begin(vn_ctx* ctx, const char* name);
void vn_prof_end(vn_ctx* ctx);

extern thread_local std::string g_vn_thread_error;

inline int32_t vn_fail(vn_ctx* ctx, int32_t code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  g_vn_thread_error = buf;
  if (ctx) ctx->err = buf;
  return code;
}

#define VN_CUDA(ctx, expr)                                                            \
  do {                                                                                \
    cudaError_t _e = (expr);                                                          \
    if (_e != cudaSuccess)                                                            \
      return vn_fail((ctx), _e == cudaErrorMemoryAllocation ? VN_ERR_OOM : VN_ERR_CUDA, \
                     "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, __LINE__); \
  } while (0)

#define VN_CHECK_CTX(ctx)                                             \
  do {                                                                \
    if (!(ctx)) return vn_fail(nullptr, VN_ERR_INVALID, "null context"); \
    cudaError_t _e = cudaSetDevice((ctx)->device);                    \
    if (_e != cudaSuccess) return vn_fail((ctx), VN_ERR_CUDA, "cudaSetDevice: %s", cudaGetErrorString(_e)); \
  } while (0)

#define VN_REQUIRE(ctx, cond, ...)                                  \
  do {                                                              \
    if (!(cond)) return vn_fail((ctx), VN_ERR_INVALID, __VA_ARGS__); \
  } while (0)

// every kernel launch goes through this so that the context can report how many ran
#define VN_LAUNCH(ctx, kernel, grid, block, smem, ...)                                  \
  do {                                                                                  \
    if ((ctx)->profiling) vn_prof_begin((ctx), #kernel);                                \
    kernel<<<(grid), (block), (smem), (ctx)->stream>>>(__VA_ARGS__);                    \
    if ((ctx)->profiling) vn_prof_end((ctx));                                           \
    (ctx)->launches++;                                                                  \
    cudaError_t _e = cudaGetLastError();                                                \
    if (_e != cudaSuccess)                                                              \
      return vn_fail((ctx), VN_ERR_CUDA, "launch of %s failed: %s", #kernel, cudaGetErrorString(_e)); \
  } while (0)

// same, with an explicit name for the per-kernel timing report (call sites of one kernel told apart)
#define VN_LAUNCH_NAMED(ctx, name, kernel, grid, block, smem, ...)                      \
  do {                                                                                  \
    if ((ctx)->profiling) vn_prof_begin((ctx), (name));                                 \
    kernel<<<(grid), (block), (smem), (ctx)->stream>>>(__VA_ARGS__);                    \
    if ((ctx)->profiling) vn_prof_end((ctx));                                           \
    (ctx)->launches++;                                                                  \
    cudaError_t _e = cudaGetLastError();                                                \
    if (_e != cudaSuccess)                                                              \
      return vn_fail((ctx), VN_ERR_CUDA, "launch of %s failed: %s", (name), cudaGetErrorString(_e)); \
  } while (0)

// ---- programmatic dependent launch --------------------------------------------------------------------
// Device side.  A kernel launched through VN_LAUNCH_PDL calls pdl_trigger() first (its successor may then be
// scheduled onto free SM resources) and pdl_wait() before its first access to memory that an earlier kernel
// of the stream wrote, and before its own first global write; pdl_wait returns when the predecessor grid has
// completed and its writes are visible.  Both are no-ops in a kernel that was launched the plain way.
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
#endif

template <typename... KArgs, typename... Args>
inline cudaError_t vn_launch_cluster(vn_ctx* ctx, int level, int cluster_y, void (*kernel)(KArgs...), dim3 grid,
                                     dim3 block, size_t smem, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = ctx->stream;
  cudaLaunchAttribute at[2];
  int n = 0;
  if (cluster_y > 1) {     // thread-block cluster along y (grid.y must be a multiple of it)
    at[n].id = cudaLaunchAttributeClusterDimension;
    at[n].val.clusterDim.x = 1; at[n].val.clusterDim.y = (unsigned)cluster_y; at[n].val.clusterDim.z = 1;
    ++n;
  }
  if (ctx->pdl >= level && !ctx->profiling) {
    at[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = at;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
template <typename... KArgs, typename... Args>
inline cudaError_t vn_launch_pdl(vn_ctx* ctx, int level, void (*kernel)(KArgs...), dim3 grid, dim3 block,
                                 size_t smem, Args&&... args) {
  return vn_launch_cluster(ctx, level, 1, kernel, grid, block, smem, static_cast<Args&&>(args)...);
}

// only for kernels that call pdl_wait() as described above
#define VN_LAUNCH_PDL_LEVEL(ctx, level, name, kernel, grid, block, smem, ...)           \
  do {                                                                                  \
    if ((ctx)->profiling) vn_prof_begin((ctx), (name));                                 \
    cudaError_t _e = vn_launch_pdl((ctx), (level), kernel, dim3(grid), dim3(block), (smem), __VA_ARGS__); \
    if ((ctx)->profiling) vn_prof_end((ctx));                                           \
    (ctx)->launches++;                                                                  \
    if (_e == cudaSuccess) _e = cudaGetLastError();                                     \
    if (_e != cudaSuccess)                                                              \
      return vn_fail((ctx), VN_ERR_CUDA, "launch of %s failed: %s", (name), cudaGetErrorString(_e)); \
  } while (0)
// the same with a thread-block cluster of cluster_y CTAs along y
#define VN_LAUNCH_CLUSTER(ctx, level, cluster_y, name, kernel, grid, block, smem, ...)  \
  do {                                                                                  \
    if ((ctx)->profiling) vn_prof_begin((ctx), (name));                                 \
    cudaError_t _e = vn_launch_cluster((ctx), (level), (cluster_y), kernel, dim3(grid), dim3(block), (smem), __VA_ARGS__); \
    if ((ctx)->profiling) vn_prof_end((ctx));                                           \
    (ctx)->launches++;                                                                  \
    if (_e == cudaSuccess) _e = cudaGetLastError();                                     \
    if (_e != cudaSuccess)                                                              \
      return vn_fail((ctx), VN_ERR_CUDA, "launch of %s failed: %s", (name), cudaGetErrorString(_e)); \
  } while (0)
#define VN_LAUNCH_PDL_NAMED(ctx, name, kernel, grid, block, smem, ...) \
  VN_LAUNCH_PDL_LEVEL(ctx, 2, name, kernel, grid, block, smem, __VA_ARGS__)
#define VN_LAUNCH_PDL(ctx, kernel, grid, block, smem, ...) \
  VN_LAUNCH_PDL_LEVEL(ctx, 2, #kernel, kernel, grid, block, smem, __VA_ARGS__)
// Kernel families that join the default level one by one: VN_PDL_MASK in the environment, a sum of
// 1 attention, 2 q|k|v finalize, 4 split-K add + norm, 8 split-K SwiGLU, 16 routing / dispatch / combine,
// 32 RMSNorm / embedding, 64 top-k select, 128 top-k merge, 256 top-k decisions.
// Default 12: measured on B200 (config-4 round, 2.425 ms with none) 1 -> 2.423, 2 -> 2.424, 4 -> 2.398, 16 -> 2.425,
// all of 1..16 -> 2.418; with the two-pairs-per-thread SwiGLU finalize 4 -> 2.387, 4+8 -> 2.382, and adding 32, 64,
// 128 or 256 to 4 stays within +-0.002 ms: the small grids that directly follow a GEMM are the ones that pay.
inline int vn_pdl_mask() {
  static const int m = [] { const char* e = getenv("VN_PDL_MASK"); return e ? atoi(e) : 12; }();
  return m;
}
#define VN_LAUNCH_PDL_BIT(ctx, bit, kernel, grid, block, smem, ...) \
  VN_LAUNCH_PDL_LEVEL(ctx, (vn_pdl_mask() & (bit)) ? 1 : 2, #kernel, kernel, grid, block, smem, __VA_ARGS__)

int32_t vn_workspace(vn_ctx* ctx, size_t bytes, void** out);

template <typename T>
static inline T ceil_div(T a, T b) { return (a + b - 1) / b; }
