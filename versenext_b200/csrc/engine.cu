// Device-side bookkeeping of a speculative-decoding round, so that a round needs no host synchronisation:
// assembling the verify input from the draft's proposals, and folding the acceptance result into the running
// state (last two committed tokens, per-request output history, number of cache entries to keep).
#include "common.cuh"
#include <math_constants.h>

namespace {

// step_tokens [k, B] (token proposed at draft step i for request b) and pair [B, 2] (the last two committed
// tokens) -> draft [B, k] and the target's verify input [B, n_verify] = (last committed, d_0, d_1, ...)
__global__ void spec_gather_kernel(const long long* __restrict__ step_tokens, const long long* __restrict__ pair, int B,
                                   int k, int n_verify, long long* __restrict__ draft, long long* __restrict__ verify) {
  pdl_trigger();
  pdl_wait();
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  // all of the request's proposals are requested before the first is stored (k <= 16)
  long long t[16];
  const long long last = pair[b * 2 + 1];
#pragma unroll
  for (int i = 0; i < 16; ++i) t[i] = i < k ? step_tokens[(long long)i * B + b] : 0;
  verify[(long long)b * n_verify] = last;
#pragma unroll
  for (int i = 0; i < 16; ++i)
    if (i < k) {
      draft[(long long)b * k + i] = t[i];
      if (i + 1 < n_verify) verify[(long long)b * n_verify + i + 1] = t[i];
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
  long long tk[17];                          // the round's tokens in one round trip (k <= 16)
#pragma unroll
  for (int i = 0; i < 17; ++i) tk[i] = i <= k ? out_tokens[(long long)b * (k + 1) + i] : -1;
#pragma unroll
  for (int i = 0; i < 17; ++i) {
    const long long t = tk[i];
    if (i > k || t < 0 || n != i) continue;  // stop at the first -1: later slots do not count
    if (c < cap) history[(long long)b * cap + c] = t;
    ++c; ++n;
    prev = last; last = t;
  }
  pair[b * 2] = prev; pair[b * 2 + 1] = last;
  count[b] = c;
  n_commit[b] = n;
}


// ---- tree proposals ---------------------------------------------------------------------------------------------
// The m largest logits of a row, in order (ties: the lower token id first): m passes of an arg-max over the
// elements that come after the previous pick in (value descending, id ascending) order.  One CTA per row; m <= 8.
constexpr int TOPM_MAX = 8;
__global__ void __launch_bounds__(1024) top_m_kernel(const float* __restrict__ logits, long long row_stride, int V, int m,
                                                     long long* __restrict__ out, long long out_stride) {
  const float* x = logits + (long long)blockIdx.x * row_stride;
  __shared__ float s_v[32];
  __shared__ int s_i[32];
  __shared__ float s_pv;
  __shared__ int s_pi;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  float pv = CUDART_INF_F; int pi = -1;              // previous pick: everything qualifies at first
  for (int j = 0; j < m; ++j) {
    float bv = -CUDART_INF_F; int bi = 0x7fffffff;
    for (int i = tid; i < V; i += blockDim.x) {
      const float v = x[i];
      const bool after = v < pv || (v == pv && i > pi);          // strictly behind the previous pick
      if (after && (v > bv || (v == bv && i < bi))) { bv = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) { s_v[warp] = bv; s_i[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
      bv = lane < (int)(blockDim.x >> 5) ? s_v[lane] : -CUDART_INF_F;
      bi = lane < (int)(blockDim.x >> 5) ? s_i[lane] : 0x7fffffff;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
      }
      if (lane == 0) {
        if (bi == 0x7fffffff) bi = 0;                              // fewer than m distinct elements (V < m)
        s_pv = bv; s_pi = bi;
        out[(long long)blockIdx.x * out_stride + j] = bi;
      }
    }
    __syncthreads();
    pv = s_pv; pi = s_pi;
  }
}

// Greedy acceptance on a verified tree.  Row 0 of a sequence is its last committed token, rows 1 .. T-1 the tree's
// nodes (parent[r] = row of the parent, 0 for the first level, -1 for row 0); target_arg[b, r] = the target's
// arg-max after row r.  Walk from row 0: take the child that carries the target's token, stop where none does; the
// target's token at the stop is committed as well.  out_tokens [B, depth + 1] (-1 padded), keep_t / keep_d
// [B, depth + 1]: the appended slots the target's / the draft's cache keeps (the draft appended the last two
// committed tokens at slots 0 and 1 and node row r at slot r + 1); both keep path length + 1 entries.
__global__ void tree_accept_greedy_kernel(const long long* __restrict__ tokens, const long long* __restrict__ target_arg,
                                          const int* __restrict__ parent, int B, int T, int depth,
                                          int* __restrict__ out_len, long long* __restrict__ out_tokens,
                                          int* __restrict__ keep_t, int* __restrict__ keep_d) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  const long long* tok = tokens + (long long)b * T;
  const long long* arg = target_arg + (long long)b * T;
  long long* ot = out_tokens + (long long)b * (depth + 1);
  int* kt = keep_t + (long long)b * (depth + 1);
  int* kd = keep_d + (long long)b * (depth + 1);
  for (int i = 0; i <= depth; ++i) { ot[i] = -1; kt[i] = 0; kd[i] = 0; }
  int cur = 0, a = 0;
  kt[0] = 0; kd[0] = 0;
  if (depth >= 1) kd[1] = 1;
  while (a < depth) {
    const long long want = arg[cur];
    int found = -1;
    for (int c = cur + 1; c < T; ++c)
      if (parent[c] == cur && tok[c] == want) { found = c; break; }
    if (found < 0) break;
    ot[a] = want;
    kt[a + 1] = found;
    if (a + 2 <= depth) kd[a + 2] = found + 1;
    cur = found;
    ++a;
  }
  ot[a] = arg[cur];
  if (out_len) out_len[b] = a;
}

}  // namespace

extern "C" {

int32_t vn_spec_gather(vn_ctx* ctx, const int64_t* step_tokens_dev, const int64_t* pair_dev, int32_t B, int32_t k,
                       int32_t n_verify, int64_t* draft_dev, int64_t* verify_dev) {
  VN_CHECK_CTX(ctx);
  VN_REQUIRE(ctx, step_tokens_dev && pair_dev && draft_dev && verify_dev && B >= 1 && k >= 1 && k <= 16 && n_verify >= 1 &&
             n_verify <= k + 1, "bad arguments (k in [1, 16], n_verify in [1, k + 1])");
  VN_LAUNCH_PDL(ctx, spec_gather_kernel, ceil_div(B, 128), 128, 0, (const long long*)step_tokens_dev,
            (const long long*)pair_dev, B, k, n_verify, (long long*)draft_dev, (long long*)verify_dev);
  return VN_OK;
}

int32_t vn_spec_advance(vn_ctx* ctx, const int64_t* out_tokens_dev, int32_t B, int32_t k, int64_t* pair_dev,
                        int64_t* history_dev, int32_t cap, int32_t* count_dev, int32_t* n_commit_dev) {
  VN_CHECK_CTX(ctx);
  VN_REQUIRE(ctx, out_tokens_dev && pair_dev && history_dev && count_dev && n_commit_dev && B >= 1 && k >= 0 && k <= 16 &&
             cap >= 0, "bad arguments (k in [0, 16])");
  VN_LAUNCH_PDL(ctx, spec_advance_kernel, ceil_div(B, 128), 128, 0, (const long long*)out_tokens_dev, B, k,
            (long long*)pair_dev, (long long*)history_dev, cap, count_dev, n_commit_dev,
            const_cast<unsigned*>(ctx->offset_src));
  return VN_OK;
}

int32_t vn_top_m(vn_ctx* ctx, const float* logits_dev, int64_t row_stride, int32_t R, int32_t V, int32_t m,
                 int64_t* out_dev, int64_t out_stride) {
  VN_CHECK_CTX(ctx);
  VN_REQUIRE(ctx, logits_dev && out_dev && R >= 0 && V >= 1 && m >= 1 && m <= TOPM_MAX && out_stride >= m,
             "vn_top_m: null buffer, or m outside [1, %d]", TOPM_MAX);
  if (R == 0) return VN_OK;
  VN_LAUNCH(ctx, top_m_kernel, R, 1024, 0, logits_dev, (long long)row_stride, V, m, (long long*)out_dev, (long long)out_stride);
  return VN_OK;
}

int32_t vn_tree_accept_greedy(vn_ctx* ctx, const int64_t* tokens_dev, const int64_t* target_arg_dev, const int32_t* parent_dev,
                              int32_t B, int32_t T, int32_t depth, int32_t* out_len_dev, int64_t* out_tokens_dev,
                              int32_t* keep_target_dev, int32_t* keep_draft_dev) {
  VN_CHECK_CTX(ctx);
  VN_REQUIRE(ctx, tokens_dev && target_arg_dev && parent_dev && out_tokens_dev && keep_target_dev && keep_draft_dev &&
             B >= 1 && T >= 1 && T <= 64 && depth >= 1 && depth < T, "vn_tree_accept_greedy: bad arguments");
  VN_LAUNCH(ctx, tree_accept_greedy_kernel, ceil_div(B, 64), 64, 0, (const long long*)tokens_dev,
            (const long long*)target_arg_dev, parent_dev, B, T, depth, out_len_dev, (long long*)out_tokens_dev,
            keep_target_dev, keep_draft_dev);
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
