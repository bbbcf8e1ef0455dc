// Device kernels of the VerseNexLM forward other than the GEMMs: embedding, RMSNorm, RoPE + KV append,
// TriSparse attention over the KV cache (window / sinks / ALiBi paths, tree ancestor mask), MoD routing,
// expert combine, KV commit.
#pragma once
#include "common.cuh"
#include "gemm.cuh"
#include <math_constants.h>

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// ---- weight staging: fp32 host rows -> storage dtype, with a row map (dst_row = src_row * mul + off)
template <typename T>
__global__ void convert_rows_kernel(const float* __restrict__ src, T* __restrict__ dst, long long rows,
                                    long long cols, long long dst_ld, long long row_mul, long long row_off) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * cols) return;
  const long long r = i / cols, c = i % cols;
  dst[(r * row_mul + row_off) * dst_ld + c] = from_f<T>(src[i]);
}

// fp32 rows -> storage dtype (the GEMM's activation format)
template <typename T>
__global__ void cast_rows_kernel(const float* __restrict__ src, T* __restrict__ dst, long long n) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = from_f<T>(src[i]);
}

// ---- embedding gather (verse_torch/vnnn.py:453-460) + optional sqrt(dim) scale (base_model.py:201-203)
template <typename T>
__global__ void embed_kernel(const long long* __restrict__ tokens, const T* __restrict__ emb, float* __restrict__ x,
                             int D, int V, float scale, int* __restrict__ status) {
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x;
  long long tok = tokens[row];
  if (tok < 0 || tok >= V) {  // record and clamp: never read outside the table
    if (threadIdx.x == 0) atomicExch(status, 1);
    tok = tok < 0 ? 0 : V - 1;
  }
  const T* e = emb + tok * D;
  for (int d = threadIdx.x; d < D; d += blockDim.x) x[(long long)row * D + d] = to_f<T>(e[d]) * scale;
}

// ---- embedding gather + scale fused with the first block's RMSNorm (decode / verify path: one launch less)
template <typename T>
__global__ void __launch_bounds__(256) embed_norm_kernel(const long long* __restrict__ tokens, const T* __restrict__ emb,
                                                         float* __restrict__ x, const float* __restrict__ w,
                                                         T* __restrict__ y, int D, int V, float scale, float eps,
                                                         int* __restrict__ status) {
  pdl_trigger();
  pdl_wait();
  __shared__ float sm[8];
  const int row = blockIdx.x;
  long long tok = tokens[row];
  if (tok < 0 || tok >= V) {  // record and clamp: never read outside the table
    if (threadIdx.x == 0) atomicExch(status, 1);
    tok = tok < 0 ? 0 : V - 1;
  }
  const T* e = emb + tok * D;
  float* xr = x + (long long)row * D;
  float ss = 0.f;
  for (int d = threadIdx.x; d < D; d += 256) {
    const float v = to_f<T>(e[d]) * scale;
    xr[d] = v;
    ss += v * v;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) tot += sm[i];
  const float r = sqrtf(tot / (float)D + eps);
  for (int d = threadIdx.x; d < D; d += 256) y[(long long)row * D + d] = from_f<T>(xr[d] / r * w[d]);
}

// ---- RMSNorm: y = x / sqrt(mean(x^2) + eps) * w (vnnn.py:501-505).  Source row = i * row_mul + row_add; optional fp32 copy.
template <typename T>
__global__ void __launch_bounds__(256) rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                      T* __restrict__ y, float* __restrict__ y32,
                                                      int row_mul, int row_add, int D, float eps) {
  pdl_trigger();
  pdl_wait();
  __shared__ float sm[8];
  const long long src = (long long)blockIdx.x * row_mul + row_add;   // e.g. the last position of every sequence
  const float* xr = x + src * D;
  float ss = 0.f;
  for (int d = threadIdx.x; d < D; d += 256) ss += xr[d] * xr[d];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) tot += sm[i];
  const float r = sqrtf(tot / (float)D + eps);
  for (int d = threadIdx.x; d < D; d += 256) {
    const float v = xr[d] / r * w[d];
    if (y) y[(long long)blockIdx.x * D + d] = from_f<T>(v);
    if (y32) y32[(long long)blockIdx.x * D + d] = v;
  }
}

// ---- RoPE on q and k (tri_sparse_attn.py:182-206: x*cos + rotate_half(x)*sin, table built on the host in
// float32 exactly as :169-180) and append of k, v to the cache at slot len[b] + t.
// qkv: [M, (H + 2*n_kv) * hd] fp32 (q | k | v); q is rotated in place.
template <typename T>
__global__ void rope_append_kernel(float* __restrict__ qkv, const float* __restrict__ cos_t,
                                   const float* __restrict__ sin_t, const int* __restrict__ lens,
                                   const int* __restrict__ depth, T* __restrict__ kc, T* __restrict__ vc, int Tn,
                                   int H, int n_kv, int hd, int max_seq, int use_rope, int rope_rows, int slot_offset) {
  const int row = blockIdx.x, b = row / Tn, t = row % Tn;
  const int len = lens[b] + slot_offset;
  const int pos = len + (depth ? depth[t] : t);
  const int slot = len + t;
  const int half = hd / 2;
  const int ld = (H + 2 * n_kv) * hd;
  float* r = qkv + (long long)row * ld;
  const int p = pos < rope_rows ? pos : rope_rows - 1;
  // q and k heads: pairs (j, j + half)
  const int n_rot = (H + n_kv) * half;
  for (int i = threadIdx.x; i < n_rot; i += blockDim.x) {
    const int head = i / half, j = i % half;
    float x1 = r[head * hd + j], x2 = r[head * hd + half + j];
    float o1 = x1, o2 = x2;
    if (use_rope) {
      const float c = cos_t[(long long)p * half + j], s = sin_t[(long long)p * half + j];
      o1 = x1 * c + (-x2) * s;
      o2 = x2 * c + x1 * s;
    }
    if (head < H) {
      r[head * hd + j] = o1;
      r[head * hd + half + j] = o2;
    } else if (slot < max_seq) {
      const int kh = head - H;
      T* dst = kc + (((long long)b * max_seq + slot) * n_kv + kh) * hd;
      dst[j] = from_f<T>(o1);
      dst[half + j] = from_f<T>(o2);
    }
  }
  if (slot < max_seq) {
    const float* v = r + (H + n_kv) * hd;
    T* dst = vc + ((long long)b * max_seq + slot) * n_kv * hd;
    for (int i = threadIdx.x; i < n_kv * hd; i += blockDim.x) dst[i] = from_f<T>(v[i]);
  }
}

// ---- TriSparse attention (tri_sparse_attn.py:536-613) on top of the cache -------------------------------
struct AttnArgs {
  const float* q;        // [M, ld_q] fp32, head h at offset h*hd
  int ld_q;
  const void* kc;        // [B, max_seq, n_kv, hd]
  const void* vc;
  const void* sink_k;    // [n_sink, n_kv, hd]
  const void* sink_v;
  void* out;             // [M, H*hd] storage dtype
  const int* lens;       // [B] committed length per sequence
  const int* depth;      // [T] or null (chain: depth = t)
  const unsigned long long* anc;  // [T] ancestor-or-self bit mask over new slots, or null (chain: causal)
  int Tn, H, n_kv, hd, max_seq, window, n_sink, slot_offset;
  int use_alibi, alibi_max;
  // > 0: the ALiBi path of the reference's one-token recurrent step (tri_sparse_attn.py:676-731): its state keeps
  // the last `alibi_window` keys only, so the path sees those keys and is switched on while that count, not the
  // whole length, is at most alibi_max.  0: the whole-sequence rule (every earlier key, off beyond alibi_max).
  int alibi_window = 0;
  float g_a, g_b, g_c;   // sigmoid(gate_logits)
  float scale;
  long long* trace = nullptr;   // optional [CTAs][8] cycle stamps of the tensor-core kernel's phases
  // Tensor-core kernel only, fused q|k|v finalize: when `partial` is set, q / k / v of the new positions are still
  // split-K slices [splits][rows][partial_ld] of the projection; the attention CTA sums the columns it needs,
  // applies RoPE and appends K / V to the cache itself (q is then not read from `q`).
  const float* partial = nullptr;
  int splits = 0;
  long long pstride = 0, partial_ld = 0;
  const float* cos_t = nullptr;
  const float* sin_t = nullptr;
  int use_rope = 0, rope_rows = 0;
  // Tensor-core kernel only: a module of the delta attention family (verse_nex/delta_attention.py) on the same three
  // passes.  delta 1 = DSA (window + sinks + dense), 2 = KDA (one pass over all keys with the window | anchor mask),
  // 3 = GMLA (dense, or the window beyond alibi_max keys); the dense pass is the ALiBi pass without its bias and the
  // switch at alibi_max keys is the ALiBi path's.  head_w[5][H]: per-head weights of the window, sink and dense
  // results while the key count is at most alibi_max, then of the window and sink results beyond it; all times out_w.
  // acc_in / acc_out: fp32 [M, H * 64] running sum over the modules of a vda layer (out is written when non-null).
  int delta = 0;
  int row_tk = 0;        // delta: 1 = every row counts its own keys (position + 1) for the alibi_max switch even in a
                         // chain: the one-token route of the reference, where every token is a call of its own
  const float* head_w = nullptr;
  float out_w = 1.f;
  int anchor = 1;
  const float* acc_in = nullptr;
  float* acc_out = nullptr;
};

// online-softmax state of one 8-lane group: running max, running sum, 8 output dims per lane
struct GroupAcc {
  float m, l, o[8];
  __device__ __forceinline__ void init() {
    m = -CUDART_INF_F; l = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = 0.f;
  }
  __device__ __forceinline__ void push(float s, const float* v) {
    const float nm = fmaxf(m, s);
    const float c = expf(m - nm), e = expf(s - nm);
    l = l * c + e;
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = o[i] * c + e * v[i];
    m = nm;
  }
};

template <typename T>
__device__ __forceinline__ void load8(const T* p, float* out);
template <>
__device__ __forceinline__ void load8<float>(const float* p, float* out) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w; out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
}
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float* out) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); out[2 * i] = f.x; out[2 * i + 1] = f.y; }
}

// merge the 4 groups of a warp (lanes g*8 + i own dims i*? .. see below) and return the normalised output of the
// calling lane's dims; all lanes participate
__device__ __forceinline__ void merge_groups(GroupAcc& a) {
  __syncwarp();
#pragma unroll
  for (int o = 8; o <= 16; o <<= 1) {
    const float om = __shfl_xor_sync(0xffffffffu, a.m, o);
    const float ol = __shfl_xor_sync(0xffffffffu, a.l, o);
    const float nm = fmaxf(a.m, om);
    const float c1 = (a.m == -CUDART_INF_F) ? 0.f : expf(a.m - nm);
    const float c2 = (om == -CUDART_INF_F) ? 0.f : expf(om - nm);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float oo = __shfl_xor_sync(0xffffffffu, a.o[i], o);
      a.o[i] = a.o[i] * c1 + oo * c2;
    }
    a.l = a.l * c1 + ol * c2;
    a.m = nm;
  }
}

// One warp per (query row, head).  The warp is 4 groups of 8 lanes; a group scores one key at a time, each
// lane owning head dims [8*li, 8*li+8) with li = lane % 8 (head_dim 64) -- keys are strided over the groups.
// head_dim must be 64 (8 lanes x 8) or 32 (only 4 lanes of a group active) ... generalised by HD8 = hd / 8 <= 8.
template <typename T>
__global__ void __launch_bounds__(256) trisparse_attn_kernel(AttnArgs a) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int grp = lane >> 3, li = lane & 7;
  const int wid = blockIdx.x * 8 + warp;           // (row, head) index
  const int M = gridDim.y;                          // unused; rows come from blockIdx.y
  (void)M;
  const int row = blockIdx.y;
  const int h = wid;
  if (h >= a.H) return;
  const int b = row / a.Tn, t = row % a.Tn;
  const int hd = a.hd;
  const int hd8 = hd >> 3;                          // lanes of a group that carry dims
  const bool active = li < hd8;
  const int len = a.lens[b] + a.slot_offset;
  const int my_depth = a.depth ? a.depth[t] : t;
  const int pos = len + my_depth;
  const int kvh = h / (a.H / a.n_kv);
  const T* kc = reinterpret_cast<const T*>(a.kc) + ((long long)b * a.max_seq * a.n_kv + kvh) * hd;
  const T* vc = reinterpret_cast<const T*>(a.vc) + ((long long)b * a.max_seq * a.n_kv + kvh) * hd;
  const long long kstride = (long long)a.n_kv * hd;
  float q[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) q[i] = active ? a.q[(long long)row * a.ld_q + h * hd + li * 8 + i] : 0.f;
  const unsigned long long anc = a.anc ? a.anc[t] : 0ull;
  const unsigned gmask = 0xFFu << (grp * 8);

  auto score = [&](const T* kr) {
    float kv[8];
    float s = 0.f;
    if (active) {
      load8<T>(kr + li * 8, kv);
#pragma unroll
      for (int i = 0; i < 8; ++i) s = fmaf(q[i], kv[i], s);
    }
    // the 8 lanes of a group always take the same branches; other groups may be elsewhere in their loops
    s += __shfl_xor_sync(gmask, s, 1);
    s += __shfl_xor_sync(gmask, s, 2);
    s += __shfl_xor_sync(gmask, s, 4);
    return s * a.scale;
  };
  auto value = [&](const T* vr, float* v) {
    if (active) load8<T>(vr + li * 8, v);
    else {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = 0.f;
    }
  };

  float out[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) out[i] = 0.f;

  // total keys this query may see through paths A / C: cached [0, len) and new slots
  const int n_new = a.Tn;
  // ---- path A: sliding window, causal (tri_sparse_attn.py:341-346) ---------------------------------
  {
    GroupAcc acc; acc.init();
    const int lo = max(0, pos - a.window + 1);
    for (int j = lo + grp; j < len; j += 4) {        // cached keys: position == slot
      const float s = score(kc + (long long)j * kstride);
      float v[8]; value(vc + (long long)j * kstride, v);
      acc.push(s, v);
    }
    for (int n = grp; n < n_new; n += 4) {           // keys appended by this call
      const bool vis = a.anc ? ((anc >> n) & 1ull) : (n <= t);
      const int pn = len + (a.depth ? a.depth[n] : n);
      if (!vis || pos - pn >= a.window || pn > pos) continue;
      const float s = score(kc + (long long)(len + n) * kstride);
      float v[8]; value(vc + (long long)(len + n) * kstride, v);
      acc.push(s, v);
    }
    merge_groups(acc);
    const float inv = acc.l > 0.f ? a.g_a / acc.l : 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) out[i] += acc.o[i] * inv;
  }
  // ---- path B: global sink tokens, no mask, keys never rotated (:461-483, :223-242) -----------------
  {
    GroupAcc acc; acc.init();
    const T* sk = reinterpret_cast<const T*>(a.sink_k) + (long long)kvh * hd;
    const T* sv = reinterpret_cast<const T*>(a.sink_v) + (long long)kvh * hd;
    for (int j = grp; j < a.n_sink; j += 4) {
      const float s = score(sk + (long long)j * kstride);
      float v[8]; value(sv + (long long)j * kstride, v);
      acc.push(s, v);
    }
    merge_groups(acc);
    const float inv = acc.l > 0.f ? a.g_b / acc.l : 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) out[i] += acc.o[i] * inv;
  }
  // ---- path C: full causal + ALiBi bias -slope_h * (i - j), only while T_k <= 1024 (:489-530, :600) --
  int tk_eff = a.anc ? (pos + 1) : (len + n_new);
  if (a.alibi_window > 0) tk_eff = min(pos + 1, a.alibi_window);
  if (a.use_alibi && tk_eff <= a.alibi_max) {
    GroupAcc acc; acc.init();
    const float slope = 1.0f / exp2f((float)(h + 1) / (float)a.H);
    const int lo_c = a.alibi_window > 0 ? max(0, pos - a.alibi_window + 1) : 0;
    for (int j = lo_c + grp; j < len; j += 4) {
      const float s = score(kc + (long long)j * kstride) - slope * (float)(pos - j);
      float v[8]; value(vc + (long long)j * kstride, v);
      acc.push(s, v);
    }
    for (int n = grp; n < n_new; n += 4) {
      const bool vis = a.anc ? ((anc >> n) & 1ull) : (n <= t);
      const int pn = len + (a.depth ? a.depth[n] : n);
      if (!vis || pn > pos || (a.alibi_window > 0 && pos - pn >= a.alibi_window)) continue;
      const float s = score(kc + (long long)(len + n) * kstride) - slope * (float)(pos - pn);
      float v[8]; value(vc + (long long)(len + n) * kstride, v);
      acc.push(s, v);
    }
    merge_groups(acc);
    const float inv = acc.l > 0.f ? a.g_c / acc.l : 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) out[i] += acc.o[i] * inv;
  }
  if (grp == 0 && active) {
    T* o = reinterpret_cast<T*>(a.out) + (long long)row * a.H * hd + h * hd + li * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = from_f<T>(out[i]);
  }
}

// ---- MoD routing (mod.py:340-387, :748-770) ----------------------------------------------------------
// One warp per token.  Part router: softmax over all P part logits.  Expert router of every part: top-k on the
// logits (ties -> lower index first), softmax over the kept logits.  Slot s = p*top_k + j of a token holds
// (global expert id, weight of that expert, weight of the part), with the experts of a part in ascending id.
struct RouteArgs {
  const float* h;        // [M, D] fp32 normalised activations
  const float* gates;    // [(P + P*E), D] fp32: part router rows, then E rows per part
  int* slot_expert;      // [M, P*top_k]
  float* slot_w;         // [M, P*top_k] expert weight
  float* part_w;         // [M, P]
  int* expert_count;     // [P*E], zeroed before the launch
  int M, D, P, E, top_k;
};

__global__ void __launch_bounds__(512) mod_route_kernel(RouteArgs r) {
  pdl_trigger();
  pdl_wait();
  // one CTA per token: the warps split the gate rows (one or two each), warp 0 then selects
  __shared__ float lg[64];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x;
  const int n_logit = r.P + r.P * r.E;       // <= 64
  const float* x = r.h + (long long)row * r.D;
  const int n4 = r.D >> 7;                   // float4 chunks per lane (D multiple of 128), <= 16
  float4 xr[16];
#pragma unroll
  for (int i = 0; i < 16; ++i)
    xr[i] = i < n4 ? *reinterpret_cast<const float4*>(x + i * 128 + lane * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
  for (int g = warp; g < n_logit; g += (int)(blockDim.x >> 5)) {
    const float* w = r.gates + (long long)g * r.D;
    float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i)
      if (i < n4) {
        const float4 wv = *reinterpret_cast<const float4*>(w + i * 128 + lane * 4);
        s0 = fmaf(xr[i].x, wv.x, s0); s1 = fmaf(xr[i].y, wv.y, s1);
        s2 = fmaf(xr[i].z, wv.z, s2); s3 = fmaf(xr[i].w, wv.w, s3);
      }
    float sum = (s0 + s1) + (s2 + s3);
    for (int d = (n4 << 7) + lane; d < r.D; d += 32) sum = fmaf(x[d], w[d], sum);   // tail when D % 128 != 0
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (lane == 0) lg[g] = sum;
  }
  __syncthreads();
  if (warp != 0) return;
  if (lane == 31) {
    // part weights: softmax over all parts
    float m = -CUDART_INF_F;
    for (int p = 0; p < r.P; ++p) m = fmaxf(m, lg[p]);
    float den = 0.f;
    for (int p = 0; p < r.P; ++p) den += expf(lg[p] - m);
    for (int p = 0; p < r.P; ++p) r.part_w[(long long)row * r.P + p] = expf(lg[p] - m) / den;
  }
  // one lane per part: top-k of its expert logits (lowest index wins ties), softmax over the kept logits
  for (int p = lane; p < r.P; p += 31) {
    if (lane == 31) break;
    const float* el = lg + r.P + p * r.E;
    int sel[8]; float sl[8];
    unsigned long long used = 0ull;
    for (int j = 0; j < r.top_k; ++j) {
      int best = -1; float bv = -CUDART_INF_F;
      for (int e = 0; e < r.E; ++e)
        if (!((used >> e) & 1ull) && (best < 0 || el[e] > bv)) { best = e; bv = el[e]; }
      used |= 1ull << best;
      sel[j] = best; sl[j] = bv;
    }
    const float em = sl[0];
    float ed = 0.f;
    for (int j = 0; j < r.top_k; ++j) ed += expf(sl[j] - em);
    for (int i = 1; i < r.top_k; ++i)      // ascending expert id inside the part
      for (int j = i; j > 0 && sel[j - 1] > sel[j]; --j) {
        const int ti = sel[j]; sel[j] = sel[j - 1]; sel[j - 1] = ti;
        const float tf = sl[j]; sl[j] = sl[j - 1]; sl[j - 1] = tf;
      }
    for (int j = 0; j < r.top_k; ++j) {
      const long long s = (long long)row * r.P * r.top_k + p * r.top_k + j;
      const int ge = p * r.E + sel[j];
      r.slot_expert[s] = ge;
      r.slot_w[s] = expf(sl[j] - em) / ed;
      atomicAdd(&r.expert_count[ge], 1);
    }
  }
}

// exclusive prefix over the expert counts; resets the fill cursors
__global__ void mod_offsets_kernel(const int* __restrict__ count, int* __restrict__ offset, int* __restrict__ cursor,
                                   int n_expert) {
  pdl_trigger();
  pdl_wait();
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < n_expert; ++e) { offset[e] = acc; acc += count[e]; cursor[e] = 0; }
  }
}

// rows 0 .. M-1 in blocks of 256: off[i] = 256 i, cnt[i] = rows in block i
__global__ void row_segments_kernel(int* __restrict__ off, int* __restrict__ cnt, int nseg, int M) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < nseg) { off[i] = 256 * i; cnt[i] = min(256, M - 256 * i); }
}

// The experts' row segments cut into pieces of at most 256 rows (what one CTA of the tensor-core GEMM takes as its
// token dimension): sub_off / sub_cnt / sub_w [n_sub_max] = first row, rows and expert of piece i; unused pieces get 0 rows.
__global__ void mod_subseg_kernel(const int* __restrict__ count, const int* __restrict__ offset, int n_expert,
                                  int* __restrict__ sub_off, int* __restrict__ sub_cnt, int* __restrict__ sub_w, int n_sub_max) {
  pdl_trigger();
  pdl_wait();
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    int n = 0;
    for (int e = 0; e < n_expert; ++e)
      for (int r = 0; r < count[e] && n < n_sub_max; r += 256) {
        sub_off[n] = offset[e] + r; sub_cnt[n] = min(256, count[e] - r); sub_w[n] = e; ++n;
      }
    for (; n < n_sub_max; ++n) { sub_off[n] = 0; sub_cnt[n] = 0; sub_w[n] = 0; }
  }
}

// place every (token, slot) in its expert's segment; sorted_row[pos] = token row, slot_pos[token, slot] = pos
__global__ void mod_scatter_kernel(const int* __restrict__ slot_expert, const int* __restrict__ offset,
                                   int* __restrict__ cursor, int* __restrict__ sorted_row, int* __restrict__ slot_pos,
                                   int n_slots_total, int S) {
  pdl_trigger();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_slots_total) return;
  const int e = slot_expert[i];
  const int pos = offset[e] + atomicAdd(&cursor[e], 1);
  sorted_row[pos] = i / S;
  slot_pos[i] = pos;
}

// x[row] += sum_p part_w[p] * (sum_j slot_w[p, j] * y[slot_pos[p, j]])   (mod.py:196-211, :604-605, :779-781)
__global__ void mod_combine_kernel(float* __restrict__ x, const float* __restrict__ y, const int* __restrict__ slot_pos,
                                   const float* __restrict__ slot_w, const float* __restrict__ part_w, int D, int P,
                                   int top_k) {
  const int row = blockIdx.x;
  const int S = P * top_k;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float out = 0.f;
    for (int p = 0; p < P; ++p) {
      float comb = 0.f;
      for (int j = 0; j < top_k; ++j) {
        const long long s = (long long)row * S + p * top_k + j;
        comb += y[(long long)slot_pos[s] * D + d] * slot_w[s];
      }
      out += comb * part_w[(long long)row * P + p];
    }
    x[(long long)row * D + d] += out;
  }
}

// ---- KV commit / rollback: compact the kept slots of the last forward behind the committed prefix ---------
// grid (B, layers*2): one CTA moves the kept rows of one sequence in one K or V plane through shared memory.
template <typename T>
__global__ void kv_commit_kernel(T* const* __restrict__ planes, const int* __restrict__ lens,
                                 const int* __restrict__ keep_idx, int stride, const int* __restrict__ n_keep, int keep_add,
                                 int n_new, int max_seq, int row_elems) {
  extern __shared__ unsigned char smem_raw[];
  T* sm = reinterpret_cast<T*>(smem_raw);
  const int b = blockIdx.x;
  T* plane = planes[blockIdx.y] + (long long)b * max_seq * row_elems;
  const int len = lens[b];
  int nk = n_keep[b] + keep_add;
  nk = nk < 0 ? 0 : (nk > n_new ? n_new : nk);
  for (int i = 0; i < nk; ++i) {
    int src = keep_idx[b * stride + i];
    src = src < 0 ? 0 : (src >= n_new ? n_new - 1 : src);
    const T* s = plane + (long long)(len + src) * row_elems;
    for (int e = threadIdx.x; e < row_elems; e += blockDim.x) sm[i * row_elems + e] = s[e];
  }
  __syncthreads();
  for (int i = 0; i < nk; ++i) {
    T* d = plane + (long long)(len + i) * row_elems;
    for (int e = threadIdx.x; e < row_elems; e += blockDim.x) d[e] = sm[i * row_elems + e];
  }
}

__global__ void kv_advance_kernel(int* __restrict__ lens, const int* __restrict__ n_keep, int keep_add, int n_new, int max_seq, int B) {
  pdl_trigger();
  pdl_wait();
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  int nk = n_keep[b] + keep_add;
  nk = nk < 0 ? 0 : (nk > n_new ? n_new : nk);
  const int nl = lens[b] + nk;
  lens[b] = nl > max_seq ? max_seq : nl;
}

// gather rows of a [rows, D] fp32 matrix
__global__ void gather_rows_kernel(const float* __restrict__ src, const int* __restrict__ rows, float* __restrict__ dst,
                                   int D) {
  const long long s = rows[blockIdx.x];
  for (int d = threadIdx.x; d < D; d += blockDim.x) dst[(long long)blockIdx.x * D + d] = src[s * D + d];
}

// ---- split-K finalize kernels (partials [splits][rows][N] fp32, summed in split order: deterministic) -----
// x[row] += sum_s partial[s][row]; then, if norm_w, y = RMSNorm(x) * norm_w in the storage dtype (+ fp32 copy).
// One CTA per row; D <= 256 * 8.
template <typename T>
__global__ void __launch_bounds__(256) splitk_add_norm_kernel(const float* __restrict__ partial, int splits,
                                                              long long pstride, float* __restrict__ x,
                                                              const float* __restrict__ norm_w, T* __restrict__ y,
                                                              float* __restrict__ y32, int D, float eps) {
  pdl_trigger();
  // the norm weights never change: fetched before the wait on the preceding kernel, used after the row sum
  float4 wn[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int d = (threadIdx.x + i * 256) * 4;
    wn[i] = (norm_w && d < D) ? __ldg(reinterpret_cast<const float4*>(norm_w + d)) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  pdl_wait();
  __shared__ float sm[8];
  const long long row = blockIdx.x;
  float4 v[2];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int d = (threadIdx.x + i * 256) * 4;
    v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (d < D) {
      const float* p = partial + row * D + d;
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
      for (int s = 0; s < splits; ++s) {   // independent loads, summed in split order
        const float4 t = *reinterpret_cast<const float4*>(p + (long long)s * pstride);
        acc.x += t.x; acc.y += t.y; acc.z += t.z; acc.w += t.w;
      }
      const float4 xv = *reinterpret_cast<const float4*>(x + row * D + d);
      v[i] = make_float4(xv.x + acc.x, xv.y + acc.y, xv.z + acc.z, xv.w + acc.w);
      *reinterpret_cast<float4*>(x + row * D + d) = v[i];
      ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
    }
  }
  if (!norm_w) return;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) tot += sm[i];
  const float r = sqrtf(tot / (float)D + eps);
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int d = (threadIdx.x + i * 256) * 4;
    if (d < D) {
      const float4 w = wn[i];
      const float o0 = v[i].x / r * w.x, o1 = v[i].y / r * w.y, o2 = v[i].z / r * w.z, o3 = v[i].w / r * w.w;
      if (y) {
        __align__(16) T o4[4] = {from_f<T>(o0), from_f<T>(o1), from_f<T>(o2), from_f<T>(o3)};
        if (sizeof(T) == 2) *reinterpret_cast<uint2*>(y + row * D + d) = *reinterpret_cast<const uint2*>(o4);
        else *reinterpret_cast<float4*>(y + row * D + d) = *reinterpret_cast<const float4*>(o4);
      }
      if (y32) *reinterpret_cast<float4*>(y32 + row * D + d) = make_float4(o0, o1, o2, o3);
    }
  }
}

// out[row, n] = sum_s partial[s][row][n]
__global__ void splitk_store_kernel(const float* __restrict__ partial, int splits, long long pstride,
                                    float* __restrict__ out, long long ld, int N, long long total) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const long long row = i / N;
  const int n = (int)(i % N);
  float acc = 0.f;
  for (int s = 0; s < splits; ++s) acc += partial[(long long)s * pstride + i];
  out[row * ld + n] = acc;
}

// act[row, j] = silu(sum_s partial[.., 2j]) * sum_s partial[.., 2j+1]
template <typename T>
__global__ void splitk_swiglu_kernel(const float* __restrict__ partial, int splits, long long pstride,
                                     T* __restrict__ act, int N, long long total_pairs) {
  pdl_trigger();
  pdl_wait();
  const int half = N / 2;
  if ((N & 3) == 0) {
    // two neighbouring pairs per thread: one 16-byte load per split (independent loads, summed in split order)
    const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 2;
    if (i >= total_pairs) return;
    const long long row = i / half;
    const int j = (int)(i % half);
    const float* p = partial + row * N + 2 * j;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
    for (int s = 0; s < splits; ++s) {
      const float4 t = *reinterpret_cast<const float4*>(p + (long long)s * pstride);
      acc.x += t.x; acc.y += t.y; acc.z += t.z; acc.w += t.w;
    }
    act[row * half + j] = from_f<T>(silu_ref(acc.x) * acc.y);
    act[row * half + j + 1] = from_f<T>(silu_ref(acc.z) * acc.w);
    return;
  }
  for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 2, e = 0; e < 2 && i < total_pairs; ++e, ++i) {
    const long long row = i / half;
    const int j = (int)(i % half);
    float g = 0.f, u = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float2 p = *reinterpret_cast<const float2*>(partial + (long long)s * pstride + row * N + 2 * j);
      g += p.x; u += p.y;
    }
    act[row * half + j] = from_f<T>(silu_ref(g) * u);
  }
}

// copy the routed tokens' normalised activations into expert order: dst[pos] = src[sorted_row[pos]]
// ---- MoD dispatch in one launch: segment offsets, a place for every routed (token, slot) pair inside its
// expert's segment, and the copy of the token's normalised row to that place (the expert GEMMs load their rows
// contiguously with TMA).  One CTA per pair.  `cursor` must be zero on entry (the combine kernel leaves it so).
template <typename T>
__global__ void mod_dispatch_kernel(const T* __restrict__ src, const int* __restrict__ slot_expert,
                                    const int* __restrict__ count, int* __restrict__ offset, int* __restrict__ cursor,
                                    int* __restrict__ slot_pos, T* __restrict__ dst, int n_expert, int S, int D) {
  pdl_trigger();
  pdl_wait();
  __shared__ int s_pos;
  const int i = blockIdx.x;
  // the token's row is on its way while warp 0 finds the destination (up to two 16-byte pieces per thread)
  const uint4* a = reinterpret_cast<const uint4*>(src + (long long)(i / S) * D);
  const int n16 = D * (int)sizeof(T) / 16;
  uint4 piece[2];
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int j = threadIdx.x + u * blockDim.x;
    piece[u] = j < n16 ? a[j] : make_uint4(0u, 0u, 0u, 0u);
  }
  if (threadIdx.x < 32) {
    // exclusive prefix of the expert counts by the lanes of one warp: all counts are requested at once (a loop of
    // one thread waited for every count before it could ask for the next)
    const int lane = threadIdx.x;
    const int e = slot_expert[i];
    int base = 0, mine = 0;
    for (int x0 = 0; x0 < n_expert; x0 += 32) {
      const int x = x0 + lane;
      const int c = x < n_expert ? count[x] : 0;
      int incl = c;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
      }
      const int excl = base + incl - c;
      if (i == 0 && x < n_expert) offset[x] = excl;       // the GEMMs read the segment starts from here
      if (e >= x0 && e < x0 + 32) mine = __shfl_sync(0xffffffffu, excl, e - x0);
      base += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) {
      const int pos = mine + atomicAdd(&cursor[e], 1);
      slot_pos[i] = pos;
      s_pos = pos;
    }
  }
  __syncthreads();
  uint4* b = reinterpret_cast<uint4*>(dst + (long long)s_pos * D);
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int j = threadIdx.x + u * blockDim.x;
    if (j < n16) b[j] = piece[u];
  }
  for (int j = threadIdx.x + 2 * blockDim.x; j < n16; j += blockDim.x) b[j] = a[j];
}

template <typename T>
__global__ void gather_sorted_kernel(const T* __restrict__ src, const int* __restrict__ sorted_row, T* __restrict__ dst,
                                     int D) {
  pdl_trigger();
  pdl_wait();
  const long long s = sorted_row[blockIdx.x];
  const uint4* a = reinterpret_cast<const uint4*>(src + s * D);
  uint4* b = reinterpret_cast<uint4*>(dst + (long long)blockIdx.x * D);
  const int n16 = D * (int)sizeof(T) / 16;
  for (int i = threadIdx.x; i < n16; i += blockDim.x) b[i] = a[i];
}

// combine with split-K partials of the expert outputs: y = sum_s ypart[s]; x[row] += the weighted sum; then, if
// norm_w, h = RMSNorm(x) * norm_w in the storage dtype (the next block's first norm, saving its launch).
// One CTA per row; D <= 256 * 8.
template <typename T>
__global__ void __launch_bounds__(256) mod_combine_split_kernel(float* __restrict__ x, const float* __restrict__ ypart,
                                                                int splits, long long pstride,
                                                                const int* __restrict__ slot_pos,
                                                                const float* __restrict__ slot_w,
                                                                const float* __restrict__ part_w, int D, int P,
                                                                int top_k, int* __restrict__ zero_counts,
                                                                int* __restrict__ zero_cursor, int n_zero,
                                                                const float* __restrict__ norm_w, T* __restrict__ h,
                                                                float eps) {
  pdl_trigger();
  // the norm weights never change: fetched before the wait on the preceding kernel, used after the row sum
  float4 wn[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int d = (threadIdx.x + i * 256) * 4;
    wn[i] = (norm_w && d < D) ? __ldg(reinterpret_cast<const float4*>(norm_w + d)) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  pdl_wait();
  // the expert GEMMs were the last readers of the per-expert counts: leave them at zero for the next router
  if (blockIdx.x == 0)
    for (int i = threadIdx.x; i < n_zero; i += blockDim.x) { zero_counts[i] = 0; if (zero_cursor) zero_cursor[i] = 0; }
  __shared__ long long s_at[64];
  __shared__ float s_w[64];
  __shared__ float s_pw[16];
  __shared__ float sm[8];
  const int row = blockIdx.x;
  const int S = P * top_k;   // <= 64
  if (threadIdx.x < S) {
    const long long s = (long long)row * S + threadIdx.x;
    s_at[threadIdx.x] = (long long)slot_pos[s] * D;
    s_w[threadIdx.x] = slot_w[s];
  }
  if (threadIdx.x >= 64 && threadIdx.x < 64 + P && P <= 16) s_pw[threadIdx.x - 64] = part_w[(long long)row * P + threadIdx.x - 64];
  __syncthreads();
  float4 v[2];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int d = (threadIdx.x + i * 256) * 4;
    v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (d >= D) continue;
    float4* xp = reinterpret_cast<float4*>(x + (long long)row * D + d);
    float4 xv = *xp;                                   // independent of the expert outputs: on its way early
    float4 out = make_float4(0.f, 0.f, 0.f, 0.f);
    if (S <= 8 && splits <= 2) {
      // the usual shape (4 parts x top-2, one or two K slices): every slot's slices are requested before the first
      // is used -- one round trip to L2 instead of one per slot; the sums keep the order of the general loop below
      float4 t[8][2];
#pragma unroll
      for (int sl = 0; sl < 8; ++sl)
#pragma unroll
        for (int q = 0; q < 2; ++q)
          t[sl][q] = (sl < S && q < splits) ? *reinterpret_cast<const float4*>(ypart + (long long)q * pstride + s_at[sl] + d)
                                            : make_float4(0.f, 0.f, 0.f, 0.f);
      for (int p = 0; p < P; ++p) {
        float4 comb = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int j = 0; j < top_k; ++j) {
          const int sl = p * top_k + j;
          float4 yv = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int q = 0; q < 2; ++q) {
            float4 tq = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int z = 0; z < 8; ++z) tq = z == sl ? t[z][q] : tq;
            if (q < splits) { yv.x += tq.x; yv.y += tq.y; yv.z += tq.z; yv.w += tq.w; }
          }
          const float w = s_w[sl];
          comb.x += yv.x * w; comb.y += yv.y * w; comb.z += yv.z * w; comb.w += yv.w * w;
        }
        const float pw = P <= 16 ? s_pw[p] : part_w[(long long)row * P + p];
        out.x += comb.x * pw; out.y += comb.y * pw; out.z += comb.z * pw; out.w += comb.w * pw;
      }
    } else
    for (int p = 0; p < P; ++p) {
      float4 comb = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int j = 0; j < top_k; ++j) {
        const int sl = p * top_k + j;
        float4 yv = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
        for (int q = 0; q < splits; ++q) {
          const float4 t = *reinterpret_cast<const float4*>(ypart + (long long)q * pstride + s_at[sl] + d);
          yv.x += t.x; yv.y += t.y; yv.z += t.z; yv.w += t.w;
        }
        const float w = s_w[sl];
        comb.x += yv.x * w; comb.y += yv.y * w; comb.z += yv.z * w; comb.w += yv.w * w;
      }
      const float pw = P <= 16 ? s_pw[p] : part_w[(long long)row * P + p];
      out.x += comb.x * pw; out.y += comb.y * pw; out.z += comb.z * pw; out.w += comb.w * pw;
    }
    xv.x += out.x; xv.y += out.y; xv.z += out.z; xv.w += out.w;
    *xp = xv;
    v[i] = xv;
    ss += xv.x * xv.x + xv.y * xv.y + xv.z * xv.z + xv.w * xv.w;
  }
  if (!norm_w) return;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) tot += sm[i];
  const float r = sqrtf(tot / (float)D + eps);
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int d = (threadIdx.x + i * 256) * 4;
    if (d < D) {
      const float4 w = wn[i];
      __align__(16) T o4[4] = {from_f<T>(v[i].x / r * w.x), from_f<T>(v[i].y / r * w.y), from_f<T>(v[i].z / r * w.z),
                                 from_f<T>(v[i].w / r * w.w)};
      T* hp = h + (long long)row * D + d;
      if (sizeof(T) == 2) *reinterpret_cast<uint2*>(hp) = *reinterpret_cast<const uint2*>(o4);
      else *reinterpret_cast<float4*>(hp) = *reinterpret_cast<const float4*>(o4);
    }
  }
}

// ---- split-K finalize of the q|k|v projection fused with RoPE and the cache append ------------------------
// One CTA per new position: sums the partial slices of its row into shared memory, then does what
// rope_append_kernel does (q rotated and written to the fp32 q buffer, k rotated and v copied into the cache).
template <typename T>
__global__ void __launch_bounds__(256) qkv_finalize_kernel(const float* __restrict__ partial, int splits,
                                                           long long pstride, float* __restrict__ qkv,
                                                           const float* __restrict__ cos_t,
                                                           const float* __restrict__ sin_t,
                                                           const int* __restrict__ lens, const int* __restrict__ depth,
                                                           T* __restrict__ kc, T* __restrict__ vc, int Tn, int H,
                                                           int n_kv, int hd, int max_seq, int use_rope, int rope_rows,
                                                           int slot_offset) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ float s_row[];   // (H + 2 n_kv) * hd floats
  const int row = blockIdx.x, b = row / Tn, t = row % Tn;
  const int ld = (H + 2 * n_kv) * hd;
  for (int i = threadIdx.x * 4; i < ld; i += blockDim.x * 4) {
    const float* p = partial + (long long)row * ld + i;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
    for (int s = 0; s < splits; ++s) {
      const float4 v = *reinterpret_cast<const float4*>(p + (long long)s * pstride);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    *reinterpret_cast<float4*>(s_row + i) = acc;
  }
  __syncthreads();
  const int len = lens[b] + slot_offset;
  const int pos = len + (depth ? depth[t] : t);
  const int slot = len + t;
  const int half = hd / 2;
  float* r = qkv + (long long)row * ld;
  const int p = pos < rope_rows ? pos : rope_rows - 1;
  const int n_rot = (H + n_kv) * half;
  for (int i = threadIdx.x; i < n_rot; i += blockDim.x) {
    const int head = i / half, j = i % half;
    const float x1 = s_row[head * hd + j], x2 = s_row[head * hd + half + j];
    float o1 = x1, o2 = x2;
    if (use_rope) {
      const float c = cos_t[(long long)p * half + j], s = sin_t[(long long)p * half + j];
      o1 = x1 * c + (-x2) * s;
      o2 = x2 * c + x1 * s;
    }
    if (head < H) {
      r[head * hd + j] = o1;
      r[head * hd + half + j] = o2;
    } else if (slot < max_seq) {
      const int kh = head - H;
      T* dst = kc + (((long long)b * max_seq + slot) * n_kv + kh) * hd;
      dst[j] = from_f<T>(o1);
      dst[half + j] = from_f<T>(o2);
    }
  }
  if (slot < max_seq) {
    const float* v = s_row + (H + n_kv) * hd;
    T* dst = vc + ((long long)b * max_seq + slot) * n_kv * hd;
    for (int i = threadIdx.x; i < n_kv * hd; i += blockDim.x) dst[i] = from_f<T>(v[i]);
  }
}
