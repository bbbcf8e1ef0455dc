// The whole layer stack of a small all-TriSparse model (the draft of a speculative round) in ONE cooperative kernel.
//
// A draft step is a chain of tiny dependent operations (norm, q|k|v, attention, projection, norm, gate|up, down, per
// layer): as separate launches each costs more in launch latency than in work.  Here the CTAs of one grid walk the
// chain together and meet at grid barriers; between two barriers every CTA owns a slice of the output features of the
// current projection (for all token rows), or some (sequence, head) pairs of the attention.  Activations cross the
// barriers through global memory and are read past L1 (cp.async.cg / __ldcg), since another SM wrote them.
//
// Arithmetic is that of the separate kernels: RMSNorm in float32 rounded to bf16, bf16 x bf16 products accumulated in
// float32, SwiGLU on float32, attention by the tensor-core tile routine (attn_tile), residual stream in float32.
// The summation order inside a dot product differs from the GEMM kernels', so logits agree to rounding, not bit for bit.
//
// Every barrier wait is bounded (the limit of the GEMM kernels, tc_detail::g_wait_limit_cycles): when it runs out the
// CTA raises the error word and walks on, so the grid always terminates and the host sees VN_ERR_TIMEOUT.
#pragma once
#include "attn_mma.cuh"
#include "gemm_tc.cuh"

namespace draft_detail {

constexpr int DT = attn_detail::AW * 32;          // threads per CTA
constexpr int MAX_LAYERS = 4;
constexpr int STAGE_BYTES = attn_detail::AW * attn_detail::RING * 4096;   // dynamic shared memory: attention ring / staged rows

struct LayerW {
  const __nv_bfloat16* wqkv;    // [(H + 2 n_kv) hd, D]
  const __nv_bfloat16* wproj;   // [D, H hd]
  const __nv_bfloat16* wgu;     // [2 hidden, D], rows interleaved gate_j, up_j
  const __nv_bfloat16* wdown;   // [D, hidden]
  const float* norm1;
  const float* norm2;
  const void* sink_k;
  const void* sink_v;
  void* kc;
  void* vc;
  float g_a, g_b, g_c;
};

struct Args {
  LayerW L[MAX_LAYERS];
  int n_layer, B, Tn, D, H, n_kv, hd, hidden, V;
  const long long* tokens;          // [B, Tn]
  const __nv_bfloat16* emb;         // [V, D]
  float emb_scale;
  const float* norm_f;
  float* x;                         // [M, D] residual stream
  float* q;                         // [M, H hd] query rows of the current layer
  __nv_bfloat16* attn;              // [M, H hd]
  __nv_bfloat16* act;               // [M, hidden]
  __nv_bfloat16* h_out;             // [rows_out, D] final-norm rows (what the LM head reads)
  float* hidden_out;                // the same in float32, or null
  const int* lens;
  int max_seq, window, n_sink, use_alibi, alibi_window, slot_offset, last_only;
  unsigned* bar;                    // [0] arrivals of the current barrier, [1] generation
  int* status;                      // token id out of range
  int* error_flag;                  // a barrier wait ran out
};

__device__ __forceinline__ void grid_barrier(const Args& a, int n_cta) {
  __syncthreads();
  if (threadIdx.x == 0) {
    volatile unsigned* gen = a.bar + 1;
    const unsigned my_gen = *gen;
    __threadfence();                                  // this CTA's writes before its arrival
    if (atomicAdd(a.bar, 1u) == (unsigned)n_cta - 1u) {
      a.bar[0] = 0u;
      __threadfence();
      atomicAdd(a.bar + 1, 1u);                       // releases everybody
    } else {
      const long long t0 = clock64();
      while (*gen == my_gen) {
        if ((unsigned long long)(clock64() - t0) > tc_detail::g_wait_limit_cycles) {
          if (a.error_flag) atomicExch(a.error_flag, 1);
          break;
        }
        __nanosleep(64);
      }
    }
    __threadfence();
  }
  __syncthreads();
}

__device__ __forceinline__ float bf16_round_f(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// dot of a staged bf16 row with a bf16 weight row, both in shared memory (the weight row is the same for the lanes of
// a warp that share an output feature: a broadcast)
__device__ __forceinline__ float dot_bf16(const __nv_bfloat16* __restrict__ s_row, const __nv_bfloat16* __restrict__ w, int K) {
  float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
  for (int k = 0; k < K; k += 8) {
    const uint4 sv = *reinterpret_cast<const uint4*>(s_row + k);
    const uint4 wv = *reinterpret_cast<const uint4*>(w + k);
    const __nv_bfloat162* s2 = reinterpret_cast<const __nv_bfloat162*>(&sv);
    const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wv);
    const float2 x0 = __bfloat1622float2(s2[0]), y0 = __bfloat1622float2(w2[0]);
    const float2 x1 = __bfloat1622float2(s2[1]), y1 = __bfloat1622float2(w2[1]);
    const float2 x2 = __bfloat1622float2(s2[2]), y2 = __bfloat1622float2(w2[2]);
    const float2 x3 = __bfloat1622float2(s2[3]), y3 = __bfloat1622float2(w2[3]);
    a0 = fmaf(x0.x, y0.x, a0); a1 = fmaf(x0.y, y0.y, a1);
    a2 = fmaf(x1.x, y1.x, a2); a3 = fmaf(x1.y, y1.y, a3);
    a0 = fmaf(x2.x, y2.x, a0); a1 = fmaf(x2.y, y2.y, a1);
    a2 = fmaf(x3.x, y3.x, a2); a3 = fmaf(x3.y, y3.y, a3);
  }
  return (a0 + a1) + (a2 + a3);
}

// Shared memory of a CTA: [0, STAGE_BYTES) the attention ring, or the staged bf16 rows a projection reads;
// then M * D floats for a copy of the residual rows; then the CTA's slice of the next projection's weights.
// The weights of the NEXT phase are fetched (cp.async) before the barrier that ends the current one, so their
// latency hides behind the barrier; every staging routine ends with a wait on all of the thread's copies.

// this CTA's rows [r0, r1) of a row-major bf16 matrix with K columns -> wbuf (asynchronous; no wait here)
__device__ __forceinline__ void prefetch_w(__nv_bfloat16* wbuf, const __nv_bfloat16* __restrict__ W, int r0, int r1, int K) {
  if (r1 <= r0) return;
  const int chunks = ((r1 - r0) * K) >> 3;
  const __nv_bfloat16* src = W + (long long)r0 * K;
  for (int i = threadIdx.x; i < chunks; i += DT) mma_detail::cp_async16(wbuf + i * 8, src + i * 8, true);
  mma_detail::cp_async_commit();
}

// RMSNorm of all M rows of the residual stream into shared memory as bf16 ([M][D + 8]).  first: the rows are the
// embeddings of the step's tokens (layer 0), and the rows this CTA owns (m % n_cta == cta) are also written to x.
__device__ __forceinline__ void stage_norm(const Args& a, const float* __restrict__ w, __nv_bfloat16* s, float* xs, int M,
                                           bool first, int cta, int n_cta) {
  const int D = a.D, ld = D + 8;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __nv_bfloat16* es = reinterpret_cast<__nv_bfloat16*>(xs);
  if (first) {
    const int chunks = D >> 3;
    for (int i = threadIdx.x; i < M * chunks; i += DT) {
      const int m = i / chunks, c = i - m * chunks;
      long long tok = a.tokens[m];
      if (tok < 0 || tok >= a.V) { atomicExch(a.status, 1); tok = tok < 0 ? 0 : a.V - 1; }
      mma_detail::cp_async16(es + m * D + c * 8, a.emb + tok * D + c * 8, true);
    }
  } else {
    const int chunks = D >> 2;
    for (int i = threadIdx.x; i < M * chunks; i += DT)
      mma_detail::cp_async16(xs + i * 4, a.x + (long long)i * 4, true);
  }
  mma_detail::cp_async_commit();
  mma_detail::cp_async_wait<0>();
  __syncthreads();
  for (int m = warp; m < M; m += DT / 32) {          // one warp per row
    float ss = 0.f;
    for (int d = lane; d < D; d += 32) {
      const float v = first ? __bfloat162float(es[m * D + d]) * a.emb_scale : xs[m * D + d];
      if (first && m % n_cta == cta) a.x[(long long)m * D + d] = v;
      ss += v * v;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float r = sqrtf(ss / (float)D + 1e-6f);
    for (int d = lane; d < D; d += 32) {
      const float v = first ? __bfloat162float(es[m * D + d]) * a.emb_scale : xs[m * D + d];
      s[m * ld + d] = __float2bfloat16_rn(v / r * w[d]);
    }
  }
  __syncthreads();
}

// rows of a bf16 matrix another CTA wrote -> shared memory [M][K + 8]
__device__ __forceinline__ void stage_rows(const __nv_bfloat16* __restrict__ src, __nv_bfloat16* s, int M, int K) {
  const int ld = K + 8, chunks = K >> 3;
  for (int i = threadIdx.x; i < M * chunks; i += DT) {
    const int m = i / chunks, c = i - m * chunks;
    mma_detail::cp_async16(s + m * ld + c * 8, src + (long long)m * K + c * 8, true);
  }
  mma_detail::cp_async_commit();
  mma_detail::cp_async_wait<0>();
  __syncthreads();
}

// bytes of dynamic shared memory the kernel needs for a model / step shape (host and device agree on the layout)
__host__ __device__ inline int slice_rows(int n, int n_cta) { return (n + n_cta - 1) / n_cta; }
__host__ __device__ inline size_t wbuf_bytes(int D, int qd, int n_qkv, int hidden, int n_cta) {
  size_t w = (size_t)slice_rows(n_qkv, n_cta) * D;
  const size_t c = (size_t)slice_rows(D, n_cta) * qd, d = (size_t)2 * slice_rows(hidden, n_cta) * D,
               e = (size_t)slice_rows(D, n_cta) * hidden;
  if (c > w) w = c;
  if (d > w) w = d;
  if (e > w) w = e;
  return (w * 2 + 127) & ~(size_t)127;
}

__global__ void __launch_bounds__(DT, 1) draft_layers_kernel(Args a) {
  extern __shared__ __align__(128) unsigned char dsm[];
  const int cta = blockIdx.x, n_cta = gridDim.x;
  const int M = a.B * a.Tn, D = a.D, hd = a.hd;
  const int qd = a.H * hd, kvd = a.n_kv * hd, n_qkv = qd + 2 * kvd;
  __nv_bfloat16* s = reinterpret_cast<__nv_bfloat16*>(dsm);
  float* xs = reinterpret_cast<float*>(dsm + STAGE_BYTES);
  __nv_bfloat16* wbuf = reinterpret_cast<__nv_bfloat16*>(dsm + STAGE_BYTES + (((size_t)M * D * 4 + 127) & ~(size_t)127));
  const int n_rep = a.H / a.n_kv;
  const int tiles = (a.Tn * n_rep + 15) >> 4;
  const int n_items = a.B * a.n_kv * tiles;
  // this CTA's slices of the four projections' output features
  const int perA = slice_rows(n_qkv, n_cta), a0 = min(n_qkv, cta * perA), a1 = min(n_qkv, a0 + perA);
  const int perC = slice_rows(D, n_cta), c0 = min(D, cta * perC), c1 = min(D, c0 + perC);
  const int perD = slice_rows(a.hidden, n_cta), d0 = min(a.hidden, cta * perD), d1 = min(a.hidden, d0 + perD);
  prefetch_w(wbuf, a.L[0].wqkv, a0, a1, D);
  for (int li = 0; li < a.n_layer; ++li) {
    const LayerW& L = a.L[li];
    // ---- A: norm1 + q|k|v for this CTA's output features; K / V rows go straight into the cache
    stage_norm(a, L.norm1, s, xs, M, li == 0, cta, n_cta);
    for (int i = threadIdx.x; i < (a1 - a0) * M; i += DT) {
      const int oi = i / M, o = a0 + oi, m = i - oi * M;
      const float v = dot_bf16(s + m * (D + 8), wbuf + oi * D, D);
      if (o < qd) {
        a.q[(long long)m * qd + o] = v;
      } else {
        const int b = m / a.Tn, t = m - b * a.Tn;
        const int slot = a.lens[b] + a.slot_offset + t;
        if (slot < a.max_seq) {
          const bool is_k = o < qd + kvd;
          const int c = is_k ? o - qd : o - qd - kvd;
          __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(is_k ? L.kc : L.vc) +
                               ((long long)b * a.max_seq + slot) * kvd + c;
          *dst = __float2bfloat16_rn(v);
        }
      }
    }
    __syncthreads();
    prefetch_w(wbuf, L.wproj, c0, c1, qd);
    grid_barrier(a, n_cta);
    // ---- B: attention, one (sequence, kv head, row tile) at a time
    {
      AttnArgs t;
      t.q = a.q; t.ld_q = qd; t.kc = L.kc; t.vc = L.vc; t.sink_k = L.sink_k; t.sink_v = L.sink_v; t.out = a.attn;
      t.lens = a.lens; t.depth = nullptr; t.anc = nullptr; t.Tn = a.Tn; t.H = a.H; t.n_kv = a.n_kv; t.hd = hd;
      t.max_seq = a.max_seq; t.window = a.window; t.n_sink = a.n_sink; t.slot_offset = a.slot_offset;
      t.use_alibi = a.use_alibi; t.alibi_max = 1024; t.alibi_window = a.alibi_window;
      t.g_a = L.g_a; t.g_b = L.g_b; t.g_c = L.g_c; t.scale = rsqrtf((float)hd);
      for (int it = cta; it < n_items; it += n_cta) {
        attn_detail::attn_tile(t, it / tiles, it % tiles, dsm, nullptr);
        __syncthreads();
      }
    }
    grid_barrier(a, n_cta);
    // ---- C: output projection + residual add for this CTA's features
    stage_rows(a.attn, s, M, qd);
    for (int i = threadIdx.x; i < (c1 - c0) * M; i += DT) {
      const int oi = i / M, o = c0 + oi, m = i - oi * M;
      const float v = dot_bf16(s + m * (qd + 8), wbuf + oi * qd, qd);
      float* xp = a.x + (long long)m * D + o;
      *xp = __ldcg(xp) + v;
    }
    __syncthreads();
    prefetch_w(wbuf, L.wgu, 2 * d0, 2 * d1, D);
    grid_barrier(a, n_cta);
    // ---- D: norm2 + gate|up + SwiGLU for this CTA's hidden units
    stage_norm(a, L.norm2, s, xs, M, false, cta, n_cta);
    for (int i = threadIdx.x; i < (d1 - d0) * M; i += DT) {
      const int ji = i / M, j = d0 + ji, m = i - ji * M;
      const float gt = dot_bf16(s + m * (D + 8), wbuf + (2 * ji) * D, D);
      const float up = dot_bf16(s + m * (D + 8), wbuf + (2 * ji + 1) * D, D);
      a.act[(long long)m * a.hidden + j] = __float2bfloat16_rn(silu_ref(gt) * up);
    }
    __syncthreads();
    prefetch_w(wbuf, L.wdown, c0, c1, a.hidden);
    grid_barrier(a, n_cta);
    // ---- E: down projection + residual add
    stage_rows(a.act, s, M, a.hidden);
    for (int i = threadIdx.x; i < (c1 - c0) * M; i += DT) {
      const int oi = i / M, o = c0 + oi, m = i - oi * M;
      const float v = dot_bf16(s + m * (a.hidden + 8), wbuf + oi * a.hidden, a.hidden);
      float* xp = a.x + (long long)m * D + o;
      *xp = __ldcg(xp) + v;
    }
    __syncthreads();
    if (li + 1 < a.n_layer) prefetch_w(wbuf, a.L[li + 1].wqkv, a0, a1, D);
    grid_barrier(a, n_cta);
  }
  // ---- final norm of the rows the head needs (every row, or the last position of every sequence)
  {
    const int rows_out = a.last_only ? a.B : M;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int r = cta * (DT / 32) + warp; r < rows_out; r += n_cta * (DT / 32)) {
      const long long src = a.last_only ? (long long)r * a.Tn + a.Tn - 1 : r;
      float ss = 0.f;
      for (int d = lane; d < D; d += 32) { const float v = __ldcg(a.x + src * D + d); ss += v * v; }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      const float rr = sqrtf(ss / (float)D + 1e-6f);
      for (int d = lane; d < D; d += 32) {
        const float v = __ldcg(a.x + src * D + d) / rr * a.norm_f[d];
        a.h_out[(long long)r * D + d] = __float2bfloat16_rn(v);
        if (a.hidden_out) a.hidden_out[(long long)r * D + d] = v;
      }
    }
  }
}

}  // namespace draft_detail
