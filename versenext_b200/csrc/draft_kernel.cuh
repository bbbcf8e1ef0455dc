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
  long long* trace;                 // optional [64] nanosecond stamps of CTA 0 at the phase boundaries, or null
};

// Sense-reversing grid barrier on two words (arrivals, generation).  Thread 0 of every CTA arrives with an
// acquire-release atomic at GPU scope -- the CTA's earlier writes are ordered before it through the block barrier in
// front -- the last one resets the count and bumps the generation with a release, the others poll the generation with
// acquire loads.  No full memory fences.  The wait is bounded.
__device__ __forceinline__ void grid_barrier(const Args& a, int n_cta) {
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned my_gen, prev;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(my_gen) : "l"(a.bar + 1) : "memory");
    asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(prev) : "l"(a.bar) : "memory");
    if (prev == (unsigned)n_cta - 1u) {
      asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" :: "l"(a.bar), "r"(0u) : "memory");
      asm volatile("red.release.gpu.global.add.u32 [%0], 1;" :: "l"(a.bar + 1) : "memory");
    } else {
      const long long t0 = clock64();
      const unsigned long long limit = tc_detail::g_wait_limit_cycles;
      unsigned g = my_gen;
      while (g == my_gen) {
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(g) : "l"(a.bar + 1) : "memory");
        if (g == my_gen && (unsigned long long)(clock64() - t0) > limit) {
          if (a.error_flag) atomicExch(a.error_flag, 1);
          break;
        }
      }
    }
  }
  __syncthreads();
}

__device__ __forceinline__ void stamp(const Args& a, int& n) {
  if (a.trace && blockIdx.x == 0 && threadIdx.x == 0 && n < 64) {
    long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    a.trace[n] = t;
  }
  ++n;
}

__device__ __forceinline__ float bf16_round_f(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// out[m][j] = sum_k s[m][k] * w[j][k] for the M staged rows and up to 16 weight rows, on the tensor cores
// (mma.sync m16n8k16, bf16 in, float32 accumulate).  The 8 warps split the row tiles and the K range; their partial
// tiles meet in `red` ([8 warps][16][16] floats), where sum_at() adds them in a fixed order.  Rows >= M of s and rows
// >= n of w hold whatever the memory held: they only feed outputs that nobody reads.
struct CtaGemm {
  int n_mt, mt_pad, ks;      // row tiles of 16, the same rounded up to a power of two, K slices (mt_pad * ks = 8)
};
__device__ __forceinline__ CtaGemm cta_gemm_shape(int M) {
  CtaGemm g;
  g.n_mt = (M + 15) >> 4;
  g.mt_pad = g.n_mt <= 1 ? 1 : (g.n_mt == 2 ? 2 : 4);
  g.ks = (DT / 32) / g.mt_pad;
  return g;
}
__device__ __forceinline__ void cta_gemm(const CtaGemm& g, const __nv_bfloat16* s, int lda, const __nv_bfloat16* w, int ldw,
                                         int K, float* red) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int mt = warp % g.mt_pad, sl = warp / g.mt_pad;
  float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
  if (mt < g.n_mt) {
    const __nv_bfloat16* a_p = s + (size_t)(mt * 16 + (lane & 15)) * lda + ((lane >> 4) << 3);
    const __nv_bfloat16* b_p = w + (size_t)((lane & 7) + ((lane >> 4) << 3)) * ldw + (((lane >> 3) & 1) << 3);
    for (int kk = sl * 16; kk < K; kk += g.ks * 16) {
      unsigned af[4], bf[2][2];
      mma_detail::ldmatrix_x4(af[0], af[1], af[2], af[3], a_p + kk);
      mma_detail::ldmatrix_x4(bf[0][0], bf[0][1], bf[1][0], bf[1][1], b_p + kk);
      mma_detail::mma_bf16(acc[0], af, bf[0]);
      mma_detail::mma_bf16(acc[1], af, bf[1]);
    }
  }
  float* r = red + warp * 256;
#pragma unroll
  for (int j = 0; j < 2; ++j)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int row = (lane >> 2) + h * 8, col = j * 8 + (lane & 3) * 2;
      r[row * 16 + col] = acc[j][h * 2];
      r[row * 16 + col + 1] = acc[j][h * 2 + 1];
    }
  __syncthreads();
}
__device__ __forceinline__ float sum_at(const CtaGemm& g, const float* red, int m, int j) {
  const int mt = m >> 4, row = m & 15;
  float v = 0.f;
  for (int sl = 0; sl < g.ks; ++sl) v += red[(sl * g.mt_pad + mt) * 256 + row * 16 + j];
  return v;
}

// Shared memory of a CTA: [0, STAGE_BYTES) the attention ring, or the staged bf16 rows a projection reads; then
// the warps' partial product tiles; then the CTA's slice of the next projection's weights.
// The weights of the NEXT phase are fetched (cp.async) before the barrier that ends the current one, so their
// latency hides behind the barrier; every staging routine ends with a wait on all of the thread's copies.

// this CTA's rows [r0, r1) of a row-major bf16 matrix with K columns -> wbuf rows of K + 8 (asynchronous; no wait here)
__device__ __forceinline__ void prefetch_w(__nv_bfloat16* wbuf, const __nv_bfloat16* __restrict__ W, int r0, int r1, int K) {
  if (r1 > r0) {
    const int cpr = K >> 3, chunks = (r1 - r0) * cpr, ld = K + 8;
    const __nv_bfloat16* src = W + (long long)r0 * K;
    for (int i = threadIdx.x; i < chunks; i += DT) {
      const int r = i / cpr, c = i - r * cpr;
      mma_detail::cp_async16(wbuf + r * ld + c * 8, src + (long long)i * 8, true);
    }
  }
  mma_detail::cp_async_commit();
}

// RMSNorm of all M rows of the residual stream into shared memory as bf16 ([M][D + 8]).  first: the rows are the
// embeddings of the step's tokens (layer 0), and the rows this CTA owns (m % n_cta == cta) are also written to x.
// A warp takes four rows at a time, a lane 8 consecutive elements of each (D <= 256): the rows'
// loads (past L1: other SMs wrote x) are all in flight together and the values stay in registers for the second pass.
constexpr int NORM_TRIPS = 1;
__device__ __forceinline__ void stage_norm(const Args& a, const float* __restrict__ w, __nv_bfloat16* s, int M, bool first,
                                           int cta, int n_cta) {
  const int D = a.D, ld = D + 8;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float wv[NORM_TRIPS][8];
#pragma unroll
  for (int t = 0; t < NORM_TRIPS; ++t) {
    const int d = t * 256 + lane * 8;
    if (d < D) {
      const float4 w0 = __ldg(reinterpret_cast<const float4*>(w + d)), w1 = __ldg(reinterpret_cast<const float4*>(w + d + 4));
      wv[t][0] = w0.x; wv[t][1] = w0.y; wv[t][2] = w0.z; wv[t][3] = w0.w;
      wv[t][4] = w1.x; wv[t][5] = w1.y; wv[t][6] = w1.z; wv[t][7] = w1.w;
    }
  }
  for (int m0 = warp; m0 < M; m0 += 4 * (DT / 32)) {
    float v[4][NORM_TRIPS][8];
    float ss[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int m = m0 + i * (DT / 32);
      if (m >= M) continue;
      const __nv_bfloat16* e = nullptr;
      if (first) {
        long long tok = a.tokens[m];
        if (tok < 0 || tok >= a.V) { if (lane == 0) atomicExch(a.status, 1); tok = tok < 0 ? 0 : a.V - 1; }
        e = a.emb + tok * D;
      }
#pragma unroll
      for (int t = 0; t < NORM_TRIPS; ++t) {
        const int d = t * 256 + lane * 8;
        if (d >= D) continue;
        if (first) {
          const uint4 raw = __ldg(reinterpret_cast<const uint4*>(e + d));
          const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(h2[j]);
            v[i][t][2 * j] = f.x * a.emb_scale; v[i][t][2 * j + 1] = f.y * a.emb_scale;
          }
        } else {
          const float4 lo = __ldcg(reinterpret_cast<const float4*>(a.x + (long long)m * D + d));
          const float4 hi = __ldcg(reinterpret_cast<const float4*>(a.x + (long long)m * D + d + 4));
          v[i][t][0] = lo.x; v[i][t][1] = lo.y; v[i][t][2] = lo.z; v[i][t][3] = lo.w;
          v[i][t][4] = hi.x; v[i][t][5] = hi.y; v[i][t][6] = hi.z; v[i][t][7] = hi.w;
        }
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int m = m0 + i * (DT / 32);
      if (m >= M) continue;
#pragma unroll
      for (int t = 0; t < NORM_TRIPS; ++t) {
        const int d = t * 256 + lane * 8;
        if (d >= D) continue;
        if (first && m % n_cta == cta) {
          float4* xp = reinterpret_cast<float4*>(a.x + (long long)m * D + d);
          xp[0] = make_float4(v[i][t][0], v[i][t][1], v[i][t][2], v[i][t][3]);
          xp[1] = make_float4(v[i][t][4], v[i][t][5], v[i][t][6], v[i][t][7]);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) ss[i] += v[i][t][j] * v[i][t][j];
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
      for (int i = 0; i < 4; ++i) ss[i] += __shfl_xor_sync(0xffffffffu, ss[i], o);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int m = m0 + i * (DT / 32);
      if (m >= M) continue;
      const float r = sqrtf(ss[i] / (float)D + 1e-6f);
#pragma unroll
      for (int t = 0; t < NORM_TRIPS; ++t) {
        const int d = t * 256 + lane * 8;
        if (d >= D) continue;
        __align__(16) __nv_bfloat16 o8[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o8[j] = __float2bfloat16_rn(v[i][t][j] / r * wv[t][j]);
        *reinterpret_cast<uint4*>(s + m * ld + d) = *reinterpret_cast<const uint4*>(o8);
      }
    }
  }
  mma_detail::cp_async_wait<0>();        // the weight slice fetched before the last barrier
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
__host__ __device__ inline size_t pad16(int n) { return (size_t)((n + 15) & ~15); }
__host__ __device__ inline size_t wbuf_bytes(int D, int qd, int n_qkv, int hidden, int n_cta) {
  size_t w = pad16(slice_rows(n_qkv, n_cta)) * (D + 8);
  const size_t c = pad16(slice_rows(D, n_cta)) * (qd + 8), d = pad16(2 * slice_rows(hidden, n_cta)) * (D + 8),
               e = pad16(slice_rows(D, n_cta)) * (hidden + 8);
  if (c > w) w = c;
  if (d > w) w = d;
  if (e > w) w = e;
  return (w * 2 + 127) & ~(size_t)127;
}
constexpr int RED_BYTES = (DT / 32) * 256 * 4;   // the warps' partial tiles

__global__ void __launch_bounds__(DT, 1) draft_layers_kernel(Args a) {
  extern __shared__ __align__(128) unsigned char dsm[];
  const int cta = blockIdx.x, n_cta = gridDim.x;
  const int M = a.B * a.Tn, D = a.D, hd = a.hd;
  const int qd = a.H * hd, kvd = a.n_kv * hd, n_qkv = qd + 2 * kvd;
  __nv_bfloat16* s = reinterpret_cast<__nv_bfloat16*>(dsm);
  float* red = reinterpret_cast<float*>(dsm + STAGE_BYTES);
  __nv_bfloat16* wbuf = reinterpret_cast<__nv_bfloat16*>(dsm + STAGE_BYTES + RED_BYTES);
  const CtaGemm cg = cta_gemm_shape(M);
  const int n_rep = a.H / a.n_kv;
  const int tiles = (a.Tn * n_rep + 15) >> 4;
  const int n_items = a.B * a.n_kv * tiles;
  // this CTA's slices of the four projections' output features
  const int perA = slice_rows(n_qkv, n_cta), a0 = min(n_qkv, cta * perA), a1 = min(n_qkv, a0 + perA);
  const int perC = slice_rows(D, n_cta), c0 = min(D, cta * perC), c1 = min(D, c0 + perC);
  const int perD = slice_rows(a.hidden, n_cta), d0 = min(a.hidden, cta * perD), d1 = min(a.hidden, d0 + perD);
  int ns = 0;
  stamp(a, ns);
  prefetch_w(wbuf, a.L[0].wqkv, a0, a1, D);
  for (int li = 0; li < a.n_layer; ++li) {
    const LayerW& L = a.L[li];
    // ---- A: norm1 + q|k|v for this CTA's output features; K / V rows go straight into the cache
    stage_norm(a, L.norm1, s, M, li == 0, cta, n_cta);
    stamp(a, ns);
    for (int nc = 0; nc < a1 - a0; nc += 16) {
      cta_gemm(cg, s, D + 8, wbuf + nc * (D + 8), D + 8, D, red);
      const int nn = min(16, a1 - a0 - nc);
      for (int i = threadIdx.x; i < nn * M; i += DT) {
        const int m = i / nn, oi = i - m * nn, o = a0 + nc + oi;
        const float v = sum_at(cg, red, m, oi);
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
    }
    prefetch_w(wbuf, L.wproj, c0, c1, qd);
    stamp(a, ns);
    grid_barrier(a, n_cta);
    stamp(a, ns);
    // ---- B: attention, one (sequence, kv head, row tile) at a time
    {
      AttnArgs t;
      t.q = a.q; t.ld_q = qd; t.kc = L.kc; t.vc = L.vc; t.sink_k = L.sink_k; t.sink_v = L.sink_v; t.out = a.attn;
      t.lens = a.lens; t.depth = nullptr; t.anc = nullptr; t.Tn = a.Tn; t.H = a.H; t.n_kv = a.n_kv; t.hd = hd;
      t.max_seq = a.max_seq; t.window = a.window; t.n_sink = a.n_sink; t.slot_offset = a.slot_offset;
      t.use_alibi = a.use_alibi; t.alibi_max = 1024; t.alibi_window = a.alibi_window;
      t.g_a = L.g_a; t.g_b = L.g_b; t.g_c = L.g_c; t.scale = rsqrtf((float)hd);
      for (int it = cta; it < n_items; it += n_cta) {
        attn_detail::attn_tile<0>(t, it / tiles, it % tiles, dsm, nullptr);
        __syncthreads();
      }
    }
    stamp(a, ns);
    grid_barrier(a, n_cta);
    stamp(a, ns);
    // ---- C: output projection + residual add for this CTA's features
    stage_rows(a.attn, s, M, qd);
    stamp(a, ns);
    for (int nc = 0; nc < c1 - c0; nc += 16) {
      cta_gemm(cg, s, qd + 8, wbuf + nc * (qd + 8), qd + 8, qd, red);
      const int nn = min(16, c1 - c0 - nc);
      for (int i = threadIdx.x; i < nn * M; i += DT) {
        const int m = i / nn, oi = i - m * nn;
        float* xp = a.x + (long long)m * D + c0 + nc + oi;
        *xp = __ldcg(xp) + sum_at(cg, red, m, oi);
      }
      __syncthreads();
    }
    prefetch_w(wbuf, L.wgu, 2 * d0, 2 * d1, D);
    stamp(a, ns);
    grid_barrier(a, n_cta);
    stamp(a, ns);
    // ---- D: norm2 + gate|up + SwiGLU for this CTA's hidden units (rows 2j, 2j + 1 of the interleaved matrix)
    stage_norm(a, L.norm2, s, M, false, cta, n_cta);
    stamp(a, ns);
    for (int nc = 0; nc < 2 * (d1 - d0); nc += 16) {
      cta_gemm(cg, s, D + 8, wbuf + nc * (D + 8), D + 8, D, red);
      const int np = min(8, d1 - d0 - nc / 2);
      for (int i = threadIdx.x; i < np * M; i += DT) {
        const int m = i / np, ji = i - m * np;
        const float gt = sum_at(cg, red, m, 2 * ji), up = sum_at(cg, red, m, 2 * ji + 1);
        a.act[(long long)m * a.hidden + d0 + nc / 2 + ji] = __float2bfloat16_rn(silu_ref(gt) * up);
      }
      __syncthreads();
    }
    prefetch_w(wbuf, L.wdown, c0, c1, a.hidden);
    stamp(a, ns);
    grid_barrier(a, n_cta);
    stamp(a, ns);
    // ---- E: down projection + residual add
    stage_rows(a.act, s, M, a.hidden);
    stamp(a, ns);
    for (int nc = 0; nc < c1 - c0; nc += 16) {
      cta_gemm(cg, s, a.hidden + 8, wbuf + nc * (a.hidden + 8), a.hidden + 8, a.hidden, red);
      const int nn = min(16, c1 - c0 - nc);
      for (int i = threadIdx.x; i < nn * M; i += DT) {
        const int m = i / nn, oi = i - m * nn;
        float* xp = a.x + (long long)m * D + c0 + nc + oi;
        *xp = __ldcg(xp) + sum_at(cg, red, m, oi);
      }
      __syncthreads();
    }
    if (li + 1 < a.n_layer) prefetch_w(wbuf, a.L[li + 1].wqkv, a0, a1, D);
    stamp(a, ns);
    grid_barrier(a, n_cta);
    stamp(a, ns);
  }
  // ---- final norm of the rows the head needs (every row, or the last position of every sequence)
  {
    const int rows_out = a.last_only ? a.B : M;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int r = cta + warp * n_cta; r < rows_out; r += n_cta * (DT / 32)) {     // spread over the CTAs first
      const long long src = a.last_only ? (long long)r * a.Tn + a.Tn - 1 : r;
      float ss = 0.f;
      for (int d = lane * 8; d < D; d += 256) {
        const float4 lo = __ldcg(reinterpret_cast<const float4*>(a.x + src * D + d));
        const float4 hi = __ldcg(reinterpret_cast<const float4*>(a.x + src * D + d + 4));
        ss += lo.x * lo.x + lo.y * lo.y + lo.z * lo.z + lo.w * lo.w + hi.x * hi.x + hi.y * hi.y + hi.z * hi.z + hi.w * hi.w;
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      const float rr = sqrtf(ss / (float)D + 1e-6f);
      for (int d = lane * 8; d < D; d += 256) {
        const float4 lo = __ldcg(reinterpret_cast<const float4*>(a.x + src * D + d));
        const float4 hi = __ldcg(reinterpret_cast<const float4*>(a.x + src * D + d + 4));
        const float xv[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
        const float4 w0 = __ldg(reinterpret_cast<const float4*>(a.norm_f + d));
        const float4 w1 = __ldg(reinterpret_cast<const float4*>(a.norm_f + d + 4));
        const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
        float v[8];
        __align__(16) __nv_bfloat16 o8[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) { v[i] = xv[i] / rr * wv[i]; o8[i] = __float2bfloat16_rn(v[i]); }
        *reinterpret_cast<uint4*>(a.h_out + (long long)r * D + d) = *reinterpret_cast<const uint4*>(o8);
        if (a.hidden_out) {
          float4* hp = reinterpret_cast<float4*>(a.hidden_out + (long long)r * D + d);
          hp[0] = make_float4(v[0], v[1], v[2], v[3]);
          hp[1] = make_float4(v[4], v[5], v[6], v[7]);
        }
      }
    }
  }
  stamp(a, ns);
}

}  // namespace draft_detail
