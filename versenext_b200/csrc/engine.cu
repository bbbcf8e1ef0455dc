// Device-side bookkeeping of a speculative-decoding round, so that a round needs no host synchronisation:
// assembling the verify input from the draft's proposals, and folding the acceptance result into the running
// state (last two committed tokens, per-request output history, number of cache entries to keep).
#include "common.cuh"

namespace {

// step_tokens [k, B] (token proposed at draft step i for request b) and pair [B, 2] (the last two committed
// tokens) -> draft [B, k] and the target's verify input [B, n_verify] = (last committed, d_0, d_1, ...)
__global__ void spec_gather_kernel(const long long* __restrict__ step_tokens, const long long* __restrict__ pair, int B,
                                   int k, int n_verify, long long* __restrict__ draft, long long* __restrict__ verify) {
  pdl_trigger();
  pdl_wait();
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  verify[(long long)b * n_verify] = pair[b * 2 + 1];
  for (int i = 0; i < k; ++i) {
    const long long t = step_tokens[(long long)i * B + b];
    draft[(long long)b * k + i] = t;
    if (i + 1 < n_verify) verify[(long long)b * n_verify + i + 1] = t;
  }
}

// out_tokens [B, k+1] (committed tokens of this round, -1 padded) -> history, counts, pair, n_commit
__global__ void spec_advance_kernel(const long long* __restrict__ out_tokens, int B, int k, long long* __restrict__ pair,
                                    long long* __restrict__ history, int cap, int* __restrict__ count,
                                    int* __restrict__ n_commit, unsigned* __restrict__ round_counter) {
  pdl_trigger();
  pdl_wait();
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b == 0 && round_counter) *round_counter += 1u;   // read by this round's kernels earlier in the stream
  if (b >= B) return;
  long long prev = pair[b * 2], last = pair[b * 2 + 1];
  int c = count[b], n = 0;
  for (int i = 0; i <= k; ++i) {
    const long long t = out_tokens[(long long)b * (k + 1) + i];
    if (t < 0) break;
    if (c < cap) history[(long long)b * cap + c] = t;
    ++c; ++n;
    prev = last; last = t;
  }
  pair[b * 2] = prev; pair[b * 2 + 1] = last;
  count[b] = c;
  n_commit[b] = n;
}

}  // namespace

extern "C" {

int32_t vn_spec_gather(vn_ctx* ctx, const int64_t* step_tokens_dev, const int64_t* pair_dev, int32_t B, int32_t k,
                       int32_t n_verify, int64_t* draft_dev, int64_t* verify_dev) {
  VN_CHECK_CTX(ctx);
  VN_REQUIRE(ctx, step_tokens_dev && pair_dev && draft_dev && verify_dev && B >= 1 && k >= 1 && n_verify >= 1 &&
             n_verify <= k + 1, "bad arguments");
  VN_LAUNCH_PDL(ctx, spec_gather_kernel, ceil_div(B, 128), 128, 0, (const long long*)step_tokens_dev,
            (const long long*)pair_dev, B, k, n_verify, (long long*)draft_dev, (long long*)verify_dev);
  return VN_OK;
}

int32_t vn_spec_advance(vn_ctx* ctx, const int64_t* out_tokens_dev, int32_t B, int32_t k, int64_t* pair_dev,
                        int64_t* history_dev, int32_t cap, int32_t* count_dev, int32_t* n_commit_dev) {
  VN_CHECK_CTX(ctx);
  VN_REQUIRE(ctx, out_tokens_dev && pair_dev && history_dev && count_dev && n_commit_dev && B >= 1 && k >= 0 && cap >= 0,
             "bad arguments");
  VN_LAUNCH_PDL(ctx, spec_advance_kernel, ceil_div(B, 128), 128, 0, (const long long*)out_tokens_dev, B, k,
            (long long*)pair_dev, (long long*)history_dev, cap, count_dev, n_commit_dev,
            const_cast<unsigned*>(ctx->offset_src));
  return VN_OK;
}

int32_t vn_set_offset_source(vn_ctx* ctx, const uint32_t* counter_dev) {
  VN_CHECK_CTX(ctx);
  ctx->offset_src = counter_dev;
  return VN_OK;
}

int32_t vn_graph_begin(vn_ctx* ctx) {
  VN_CHECK_CTX(ctx);
  VN_REQUIRE(ctx, !ctx->profiling, "per-kernel timing and graph capture exclude each other");
  VN_CUDA(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeRelaxed));
  return VN_OK;
}

struct vn_graph_exec {
  cudaGraphExec_t exec;
  uint64_t kernels;   // kernel nodes in the graph: added to the context's launch count on every replay
};

int32_t vn_graph_end(vn_ctx* ctx, void** out_exec) {
  VN_CHECK_CTX(ctx);
  VN_REQUIRE(ctx, out_exec, "out_exec is null");
  *out_exec = nullptr;
  cudaGraph_t graph = nullptr;
  VN_CUDA(ctx, cudaStreamEndCapture(ctx->stream, &graph));
  size_t n_nodes = 0;
  uint64_t kernels = 0;
  if (cudaGraphGetNodes(graph, nullptr, &n_nodes) == cudaSuccess && n_nodes) {
    std::vector<cudaGraphNode_t> nodes(n_nodes);
    if (cudaGraphGetNodes(graph, nodes.data(), &n_nodes) == cudaSuccess)
      for (size_t i = 0; i < n_nodes; ++i) {
        cudaGraphNodeType t;
        if (cudaGraphNodeGetType(nodes[i], &t) == cudaSuccess && t == cudaGraphNodeTypeKernel) ++kernels;
      }
  }
  cudaGraphExec_t exec = nullptr;
  cudaError_t e = cudaGraphInstantiate(&exec, graph, 0);
  cudaGraphDestroy(graph);
  if (e != cudaSuccess) return vn_fail(ctx, VN_ERR_CUDA, "cudaGraphInstantiate: %s", cudaGetErrorString(e));
  *out_exec = (void*)new vn_graph_exec{exec, kernels};
  return VN_OK;
}

int32_t vn_graph_launch(vn_ctx* ctx, void* exec) {
  VN_CHECK_CTX(ctx);
  VN_REQUIRE(ctx, exec, "graph is null");
  vn_graph_exec* g = (vn_graph_exec*)exec;
  VN_CUDA(ctx, cudaGraphLaunch(g->exec, ctx->stream));
  ctx->launches += g->kernels;
  return VN_OK;
}

int32_t vn_graph_destroy(vn_ctx* ctx, void* exec) {
  VN_CHECK_CTX(ctx);
  if (exec) {
    vn_graph_exec* g = (vn_graph_exec*)exec;
    cudaGraphExecDestroy(g->exec);
    delete g;
  }
  return VN_OK;
}

}  // extern "C"
