// VerseNext Delta Attention family on top of the cache: the DSA, KDA and GMLA modules of
// verse_nex/delta_attention.py, whole-sequence semantics (what the reference's forward without kv_cache computes,
// masks built from absolute positions), on cached keys plus the keys appended by this call (chain or tree).
//
//   DSA  (:555-574)  out = g_h * dense + (1 - g_h) * (window + sinks); dense = all earlier keys (:470-486), window =
//                    the last `window` keys (:492-538), sinks = the module's global tokens, never masked, never
//                    rotated (:451-459, :540-549); three separate soft-maxes.  Beyond max_t keys the dense term is
//                    itself window + sinks (:561-566).
//   KDA  (:678-698)  one soft-max over the window and every anchor key (position % anchor == 0).  Beyond max_t keys
//                    the reference goes chunk-wise and concatenates all anchors behind the window slice of the query's
//                    chunk (:704-768), so an anchor that also lies in the slice [k_lo, ..] is counted twice; the
//                    weights below reproduce that count.
//   GMLA (:876-930)  K / V rebuilt from a latent (done by the caller's GEMMs); dense soft-max, beyond max_t keys the
//                    window (:948-992); output times the head gate.
// "Beyond max_t keys" is decided as for the ALiBi path of the TriSparse kernel: a chain counts cached + new positions,
// a tree node its own position + 1.
#pragma once
#include "model_kernels.cuh"

struct DeltaArgs {
  const float* q;        // [M, ld_q] fp32, head h at offset h*hd (already rotated)
  int ld_q;
  const void* kc;        // this module's planes [B, max_seq, n_kv, hd]
  const void* vc;
  const void* sink_k;    // dsa: [n_sink, n_kv, hd]
  const void* sink_v;
  const float* head_gate;  // [H] sigmoid(head_gate_logits) (dsa, gmla), or null
  const float* acc_in;   // [M, H*hd] fp32 sum of the modules before this one (a vda layer), or null
  float* acc_out;        // where the running sum goes, or null
  void* out;             // [M, H*hd] storage dtype: the finished sum, or null
  float out_w;           // weight of this module in the sum (vda: sigmoid(gate_logits[i]); 1 for a single module)
  const int* lens;
  const int* depth;
  const unsigned long long* anc;
  int Tn, H, n_kv, hd, max_seq, window, n_sink, slot_offset;
  int anchor, max_t;
  int row_tk;            // 1: a chain's rows count their own keys (position + 1) for the max_t switch (one-token route)
  int mode;              // 0 dsa, 1 kda, 2 gmla
  float scale;
};

// weighted push: a key that enters the soft-max `w` times
__device__ __forceinline__ void group_push_w(GroupAcc& a, float s, const float* v, float w) {
  const float nm = fmaxf(a.m, s);
  const float c = expf(a.m - nm), e = expf(s - nm) * w;
  a.l = a.l * c + e;
#pragma unroll
  for (int i = 0; i < 8; ++i) a.o[i] = a.o[i] * c + e * v[i];
  a.m = nm;
}

// One warp per (query row, head), 4 groups of 8 lanes as in trisparse_attn_kernel.
template <typename T>
__global__ void __launch_bounds__(256) delta_attn_kernel(DeltaArgs a) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int grp = lane >> 3, li = lane & 7;
  const int h = blockIdx.x * 8 + warp;
  const int row = blockIdx.y;
  if (h >= a.H) return;
  const int b = row / a.Tn, t = row % a.Tn;
  const int hd = a.hd;
  const bool active = li < (hd >> 3);
  const int len = a.lens[b] + a.slot_offset;
  const int pos = len + (a.depth ? a.depth[t] : t);
  const int kvh = h / (a.H / a.n_kv);
  const T* kc = reinterpret_cast<const T*>(a.kc) + ((long long)b * a.max_seq * a.n_kv + kvh) * hd;
  const T* vc = reinterpret_cast<const T*>(a.vc) + ((long long)b * a.max_seq * a.n_kv + kvh) * hd;
  const long long kstride = (long long)a.n_kv * hd;
  float q[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) q[i] = active ? a.q[(long long)row * a.ld_q + h * hd + li * 8 + i] : 0.f;
  const unsigned long long anc = a.anc ? a.anc[t] : 0ull;
  const unsigned gmask = 0xFFu << (grp * 8);
  const int n_new = a.Tn;
  const int W = a.window;

  auto score = [&](const T* kr) {
    float kv[8];
    float s = 0.f;
    if (active) {
      load8<T>(kr + li * 8, kv);
#pragma unroll
      for (int i = 0; i < 8; ++i) s = fmaf(q[i], kv[i], s);
    }
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
  // position of the n-th key appended by this call, or -1 when this query does not see it
  auto new_pos = [&](int n) {
    const bool vis = a.anc ? ((anc >> n) & 1ull) : (n <= t);
    const int pn = len + (a.depth ? a.depth[n] : n);
    return (vis && pn <= pos) ? pn : -1;
  };
  // soft-max over every visible key at most `reach - 1` positions back, normalised into res[8]
  auto span = [&](int reach, float* res) {
    GroupAcc acc; acc.init();
    const int lo = reach > pos ? 0 : pos - reach + 1;
    for (int j = lo + grp; j < len; j += 4) {
      const float s = score(kc + (long long)j * kstride);
      float v[8]; value(vc + (long long)j * kstride, v);
      acc.push(s, v);
    }
    for (int n = grp; n < n_new; n += 4) {
      const int pn = new_pos(n);
      if (pn < 0 || pos - pn >= reach) continue;
      const float s = score(kc + (long long)(len + n) * kstride);
      float v[8]; value(vc + (long long)(len + n) * kstride, v);
      acc.push(s, v);
    }
    merge_groups(acc);
    const float inv = acc.l > 0.f ? 1.f / acc.l : 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) res[i] = acc.o[i] * inv;
  };
  constexpr int ALL = 0x7fffffff;

  const int tk_eff = (a.anc || a.row_tk) ? (pos + 1) : (len + n_new);
  const bool long_seq = tk_eff > a.max_t;
  float out[8];

  if (a.mode == 1) {
    // ---- KDA: window and anchors in one soft-max ----
    const int I = a.anchor;
    const int lo = max(0, pos - W + 1);                       // first window position
    const int k_lo = max(0, (pos / W) * W - W + 1);           // first key of the query's chunk slice (long route)
    GroupAcc acc; acc.init();
    for (int j = lo + grp; j < len; j += 4) {                 // cached window keys
      const float w = (long_seq && j % I == 0) ? 2.f : 1.f;
      const float s = score(kc + (long long)j * kstride);
      float v[8]; value(vc + (long long)j * kstride, v);
      group_push_w(acc, s, v, w);
    }
    const int a_end = min(lo, len);                           // cached anchors in front of the window
    for (int j = grp * I; j < a_end; j += 4 * I) {
      const float w = (long_seq && j >= k_lo) ? 2.f : 1.f;
      const float s = score(kc + (long long)j * kstride);
      float v[8]; value(vc + (long long)j * kstride, v);
      group_push_w(acc, s, v, w);
    }
    for (int n = grp; n < n_new; n += 4) {                    // keys appended by this call
      const int pn = new_pos(n);
      if (pn < 0) continue;
      const bool in_win = pos - pn < W, anch = pn % I == 0;
      float w;
      if (long_seq) w = ((in_win || (anch && pn >= k_lo)) ? 1.f : 0.f) + (anch ? 1.f : 0.f);
      else w = (in_win || anch) ? 1.f : 0.f;
      if (w == 0.f) continue;
      const float s = score(kc + (long long)(len + n) * kstride);
      float v[8]; value(vc + (long long)(len + n) * kstride, v);
      group_push_w(acc, s, v, w);
    }
    merge_groups(acc);
    const float inv = acc.l > 0.f ? 1.f / acc.l : 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) out[i] = acc.o[i] * inv;
  } else if (a.mode == 2) {
    // ---- GMLA: dense, or the window beyond max_t keys; head gate ----
    span(long_seq ? W : ALL, out);
    const float g = a.head_gate[h];
#pragma unroll
    for (int i = 0; i < 8; ++i) out[i] *= g;
  } else {
    // ---- DSA: g * dense + (1 - g) * (window + sinks) ----
    float sparse[8];
    span(W, sparse);
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
      const float inv = acc.l > 0.f ? 1.f / acc.l : 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) sparse[i] += acc.o[i] * inv;
    }
    const float g = a.head_gate[h];
    if (long_seq) {
#pragma unroll
      for (int i = 0; i < 8; ++i) out[i] = sparse[i] * g + sparse[i] * (1.f - g);
    } else {
      float dense[8];
      span(ALL, dense);
#pragma unroll
      for (int i = 0; i < 8; ++i) out[i] = dense[i] * g + sparse[i] * (1.f - g);
    }
  }
  if (grp == 0 && active) {
    const long long base = (long long)row * a.H * hd + h * hd + li * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float v = a.out_w * out[i];
      if (a.acc_in) v += a.acc_in[base + i];
      if (a.acc_out) a.acc_out[base + i] = v;
      if (a.out) reinterpret_cast<T*>(a.out)[base + i] = from_f<T>(v);
    }
  }
}

// ---- GMLA projections on the split-K GEMM: the reductions between the GEMMs ------------------------------------
// One CTA per new position sums the partial slices of its row (as qkv_finalize_kernel does).
// stage 1: the row is [q (H hd) | latent (lat)] of the stacked wq | w_kv_down product: q is rotated and written to the
//          fp32 q buffer (row stride ld_q), the latent goes to lat_out in the storage dtype (the next GEMM's operand).
// stage 2: the row is [k (n_kv hd) | v (n_kv hd)] rebuilt from the latent: k is rotated, both go to the cache.
template <typename T>
__global__ void __launch_bounds__(256) gmla_finalize_kernel(const float* __restrict__ partial, int splits, long long pstride,
                                                            int ld, int stage, float* __restrict__ q_out, int ld_q,
                                                            T* __restrict__ lat_out, int lat,
                                                            const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                                            const int* __restrict__ lens, const int* __restrict__ depth,
                                                            T* __restrict__ kc, T* __restrict__ vc, int Tn, int H, int n_kv,
                                                            int hd, int max_seq, int use_rope, int rope_rows, int slot_offset) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ float s_row[];   // ld floats
  const int row = blockIdx.x, b = row / Tn, t = row % Tn;
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
  const int p = pos < rope_rows ? pos : rope_rows - 1;
  const int heads = stage == 1 ? H : n_kv;
  for (int i = threadIdx.x; i < heads * half; i += blockDim.x) {
    const int head = i / half, j = i % half;
    const float x1 = s_row[head * hd + j], x2 = s_row[head * hd + half + j];
    float o1 = x1, o2 = x2;
    if (use_rope) {
      const float c = cos_t[(long long)p * half + j], s = sin_t[(long long)p * half + j];
      o1 = x1 * c + (-x2) * s;
      o2 = x2 * c + x1 * s;
    }
    if (stage == 1) {
      float* r = q_out + (long long)row * ld_q + head * hd;
      r[j] = o1;
      r[half + j] = o2;
    } else if (slot < max_seq) {
      T* dst = kc + (((long long)b * max_seq + slot) * n_kv + head) * hd;
      dst[j] = from_f<T>(o1);
      dst[half + j] = from_f<T>(o2);
    }
  }
  if (stage == 1) {
    const float* l = s_row + H * hd;
    for (int i = threadIdx.x; i < lat; i += blockDim.x) lat_out[(long long)row * lat + i] = from_f<T>(l[i]);
  } else if (slot < max_seq) {
    const float* v = s_row + n_kv * hd;
    T* dst = vc + ((long long)b * max_seq + slot) * n_kv * hd;
    for (int i = threadIdx.x; i < n_kv * hd; i += blockDim.x) dst[i] = from_f<T>(v[i]);
  }
}
