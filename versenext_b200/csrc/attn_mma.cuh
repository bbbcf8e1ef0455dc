// TriSparse attention on tensor cores for bf16 caches with head_dim 64 (tri_sparse_attn.py:536-613).
//
// One CTA per (sequence, kv head, tile of 16 query rows); the rows of a tile are (query head of the GQA
// group) x (new position), so every K / V row fetched from the cache serves all of them.  The 8 warps of the
// CTA take 16-key blocks round-robin, each with its own online-softmax state, and are merged through shared
// memory.  The three paths of the reference (window, sinks, ALiBi) keep their own softmax and are mixed by the
// sigmoid gates afterwards.
//
// mma.sync.m16n8k16 fragments are filled straight from global memory without a transposing stage by using the
// freedom to permute the contraction index (same permutation on both operands) and the output columns:
//   S = Q K^T : thread (g, t) of the warp loads dims [16t, 16t+16) of key row g     (32 contiguous bytes)
//   O = P V   : thread (g, t) loads dims [8g, 8g+8) of key rows 2t, 2t+1, 2t+8, 2t+9 (16 contiguous bytes each)
//               and pairs the rows with byte permutes; accumulator column n of tile j is output dim 8n + j.
#pragma once
#include <type_traits>
#include "model_kernels.cuh"
#include "gemm_mma.cuh"

namespace attn_detail {

constexpr int AW = 8;    // warps per CTA
#ifndef VN_ATTN_RING
#define VN_ATTN_RING 3
#endif
constexpr int RING = VN_ATTN_RING;  // key blocks per warp in shared memory (4 KB each)

__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}

__device__ __forceinline__ long long clock_stamp() {
  long long c;
  asm volatile("mov.u64 %0, %%clock64;" : "=l"(c) :: "memory");
  return c;
}

struct RowInfo {
  bool valid;
  bool long_row;   // delta modules: this row's key count is beyond alibi_max
  int tq, pos;
  float slope;
  unsigned long long anc;
};

// One block of 16 keys against the warp's 16 query rows: S = Q K^T, scale / bias / mask, online soft-max update,
// O += P V.  st: the block in shared memory (16 rows of 128 bytes for K, then the same for V at +2048, 16-byte chunks
// XOR-swizzled with the row).  CHAIN_NEW (chains only): appended keys that every row of the tile sees (the key's
// new-slot number <= tq_min) need no mask either.
template <int MODE, bool CHAIN_NEW = false>
__device__ __forceinline__ void attend_block(const AttnArgs& a, const unsigned char* st, int j0, int hi, int len,
                                             const RowInfo (&row)[2], const unsigned (&qf)[4][4], const int* s_depth,
                                             int pos_max, int tq_min, int g, int t, float (&o)[8][4], float (&m)[2],
                                             float (&l)[2]) {
  // ---- K: rows 8i + g, dims 16t .. 16t+15 (chunks 2t, 2t+1)
  unsigned kr[2][8];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const unsigned char* rp = st + (8 * i + g) * 128;
    const uint4 u0 = *reinterpret_cast<const uint4*>(rp + (((2 * t) ^ g) << 4));
    const uint4 u1 = *reinterpret_cast<const uint4*>(rp + (((2 * t + 1) ^ g) << 4));
    kr[i][0] = u0.x; kr[i][1] = u0.y; kr[i][2] = u0.z; kr[i][3] = u0.w;
    kr[i][4] = u1.x; kr[i][5] = u1.y; kr[i][6] = u1.z; kr[i][7] = u1.w;
  }
  // ---- V: rows {2t, 2t+1, 2t+8, 2t+9}, dims 8g .. 8g+7 (chunk g)
  unsigned vr[4][4];
#pragma unroll
  for (int x = 0; x < 4; ++x) {
    const int r = 2 * t + (x & 1) + ((x >> 1) << 3);
    const uint4 u = *reinterpret_cast<const uint4*>(st + 2048 + r * 128 + ((g ^ (r & 7)) << 4));
    vr[x][0] = u.x; vr[x][1] = u.y; vr[x][2] = u.z; vr[x][3] = u.w;
  }
  // ---- S = Q K^T for two tiles of 8 keys
  float c[2][4];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    c[i][0] = c[i][1] = c[i][2] = c[i][3] = 0.f;
#pragma unroll
    for (int s = 0; s < 4; ++s) {
      const unsigned bfrag[2] = {kr[i][2 * s], kr[i][2 * s + 1]};
      mma_detail::mma_bf16(c[i], qf[s], bfrag);
    }
  }
  // ---- scale, bias, mask.  A block of committed keys that every row of the tile sees needs no mask
  // (rows beyond R compute on real keys too; their result is never stored)
  const bool plain = j0 + 16 <= hi && (MODE == 1 || (MODE == 0 && pos_max - j0 < a.window &&
                                                       (j0 + 16 <= len || (CHAIN_NEW && j0 >= len && j0 + 15 - len <= tq_min))));
  if (plain) {
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) c[i][e] *= a.scale;
  } else {
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = j0 + 8 * i + 2 * t + (e & 1);
        const RowInfo& r = row[e >> 1];
        bool vis = r.valid && key < hi;
        float sc = c[i][e] * a.scale;
        if (MODE == 0 || MODE == 2 || MODE == 3) {
          int kpos = key;
          if (key >= len) {
            const int n = key - len;
            kpos = len + (s_depth ? s_depth[n < 64 ? n : 63] : n);
            vis = vis && (a.anc ? ((r.anc >> n) & 1ull) != 0 : n <= r.tq) && kpos <= r.pos;
          }
          if (MODE == 0) vis = vis && (r.pos - kpos) < a.window;
          else if (MODE == 2) {
            sc -= r.slope * (float)(r.pos - kpos);
            if (a.alibi_window > 0) vis = vis && (r.pos - kpos) < a.alibi_window;
          } else {
            // KDA: the window and every anchor key in one soft-max (delta_attention.py:678-698).  Beyond alibi_max
            // keys the reference scores the window slice of the query's chunk and all anchors, concatenated
            // (:704-768): an anchor inside the slice [k_lo, ..] counts twice, i.e. its score gains ln 2.
            const bool in_win = (r.pos - kpos) < a.window, anch = (kpos % a.anchor) == 0;
            if (!r.long_row) vis = vis && (in_win || anch);
            else {
              const int k_lo = max(0, (r.pos / a.window) * a.window - a.window + 1);
              const int mult = ((in_win || (anch && kpos >= k_lo)) ? 1 : 0) + (anch ? 1 : 0);
              vis = vis && mult > 0;
              if (mult == 2) sc += 0.6931471806f;
            }
          }
        }
        c[i][e] = vis ? sc : -CUDART_INF_F;
      }
  }
  // ---- online softmax (rows g and g+8; a row lives in the 4 lanes of a quad)
  float pr[2][4];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    float mx = fmaxf(fmaxf(c[0][2 * h], c[0][2 * h + 1]), fmaxf(c[1][2 * h], c[1][2 * h + 1]));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float mn = fmaxf(m[h], mx);
    float corr = 1.f;
    if (mn == -CUDART_INF_F) {
      pr[0][2 * h] = pr[0][2 * h + 1] = pr[1][2 * h] = pr[1][2 * h + 1] = 0.f;
    } else {
      corr = __expf(m[h] - mn);
      pr[0][2 * h] = __expf(c[0][2 * h] - mn);
      pr[0][2 * h + 1] = __expf(c[0][2 * h + 1] - mn);
      pr[1][2 * h] = __expf(c[1][2 * h] - mn);
      pr[1][2 * h + 1] = __expf(c[1][2 * h + 1] - mn);
    }
    l[h] = l[h] * corr + pr[0][2 * h] + pr[0][2 * h + 1] + pr[1][2 * h] + pr[1][2 * h + 1];
    m[h] = mn;
    if (corr != 1.f) {   // the running maximum moved: rare after the first blocks
#pragma unroll
      for (int j = 0; j < 8; ++j) { o[j][2 * h] *= corr; o[j][2 * h + 1] *= corr; }
    }
  }
  // ---- O += P V
  const unsigned pa[4] = {pack_bf16(pr[0][0], pr[0][1]), pack_bf16(pr[0][2], pr[0][3]),
                          pack_bf16(pr[1][0], pr[1][1]), pack_bf16(pr[1][2], pr[1][3])};
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const unsigned sel = (j & 1) ? 0x7632u : 0x5410u;
    const unsigned bfrag[2] = {__byte_perm(vr[0][j >> 1], vr[1][j >> 1], sel),
                               __byte_perm(vr[2][j >> 1], vr[3][j >> 1], sel)};
    mma_detail::mma_bf16(o[j], pa, bfrag);
  }
}

// mode 0: window path (cached keys within the window, appended keys by ancestry), 1: sinks, 2: ALiBi path (with a
// zero slope: plain causal attention), 3: all keys under the KDA window | anchor mask
template <int MODE>
__device__ __forceinline__ void attend(const AttnArgs& a, const __nv_bfloat16* __restrict__ Kb,
                                       const __nv_bfloat16* __restrict__ Vb, long long ks, int lo, int hi, int len,
                                       const RowInfo (&row)[2], const unsigned (&qf)[4][4], const int* s_depth,
                                       int warp, int nw, int lane, unsigned char* ring, float (&o)[8][4],
                                       float (&m)[2], float (&l)[2], int phase = 0) {
  // phase 0: everything.  phase 1: only put this warp's first key blocks on their way (they do not depend on the
  // query rows, so the caller can do that before its own set-up work).  phase 2: the rest, after a phase-1 call
  // with the same arguments.
  const int g = lane >> 2, t = lane & 3;
  if (phase != 1) {
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) o[j][e] = 0.f;
    m[0] = m[1] = -CUDART_INF_F;
    l[0] = l[1] = 0.f;
  }
  const int nblk = hi > lo ? (hi - lo + 15) >> 4 : 0;
  int pos_max = max(row[0].pos, row[1].pos);     // latest query position of the tile
#pragma unroll
  for (int o_ = 16; o_ > 0; o_ >>= 1) pos_max = max(pos_max, __shfl_xor_sync(0xffffffffu, pos_max, o_));
  // `warp` is this warp's index inside the group of `nw` warps that share this key range.
  // This warp's blocks (warp, warp + nw, ...) stream through its own ring of RING stages in shared memory:
  // 16 key rows of 128 bytes for K, then the same for V, 16-byte chunks XOR-swizzled with the row so that the
  // fragment loads below are free of bank conflicts.  cp.async keeps RING - 1 blocks in flight per warp.
  const int n_my = nblk > warp ? (nblk - warp + nw - 1) / nw : 0;
  auto issue = [&](int it) {
    const int j0 = lo + (warp + it * nw) * 16;
    unsigned char* st = ring + (it % RING) * 4096;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int ci = i * 32 + lane;
      const int r = ci >> 3, c = ci & 7;
      int key = j0 + r;
      key = key < hi ? key : hi - 1;
      const int soff = r * 128 + ((c ^ (r & 7)) << 4);
      mma_detail::cp_async16(st + soff, Kb + (long long)key * ks + c * 8, true);
      mma_detail::cp_async16(st + 2048 + soff, Vb + (long long)key * ks + c * 8, true);
    }
  };
  if (phase != 2) {
#pragma unroll
    for (int s = 0; s < RING - 1; ++s) {
      if (s < n_my) issue(s);
      mma_detail::cp_async_commit();
    }
  }
  if (phase == 1) return;
  for (int it = 0; it < n_my; ++it) {
    const int j0 = lo + (warp + it * nw) * 16;
    mma_detail::cp_async_wait<RING - 2>();
    __syncwarp();                                  // block `it` has landed; everyone is done with block it - 1
    if (it + RING - 1 < n_my) issue(it + RING - 1);
    mma_detail::cp_async_commit();
    const unsigned char* st = ring + (it % RING) * 4096;
    attend_block<MODE, false>(a, st, j0, hi, len, row, qf, s_depth, pos_max, 0, g, t, o, m, l);
  }
  __syncwarp();   // the ring is reused by the caller
  // row sums live spread over the quad
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
  }
}

// One (sequence, kv head, row tile) of the attention: bx = sequence * n_kv + kv head, by = tile of 16 query rows.
// Called by all AW * 32 threads of a CTA; attn_smem: AW * RING * 4096 bytes of shared memory, 128-byte aligned.
// Everything another kernel -- or, inside a persistent kernel, another CTA -- wrote shortly before is read past L1
// (cp.async.cg, __ldcg).
// DM: 0 = TriSparse; 1 / 2 / 3 = compiled for that delta-attention module (AttnArgs::delta: DSA / KDA / GMLA), each
// instance carrying only its own passes.
template <int DM>
__device__ __forceinline__ void attn_tile(const AttnArgs& a, int bx, int by, unsigned char* attn_smem, long long* tr) {
  constexpr bool DELTA = DM != 0;
  constexpr int dmode = DM;
  // per warp: a ring of RING key blocks; after a path's keys the first 4 KB of the warp's ring hold its
  // partial output (16 rows x 64 dims fp32, 16-byte chunks swizzled) for the merge across warps
  __shared__ float sM[AW][16], sL[AW][16];
  __shared__ int s_depth[64];
  __shared__ __align__(16) float s_q[16 * 64];     // fused mode: the tile's query rows after the split-K sum and RoPE
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int b = bx / a.n_kv, kvh = bx % a.n_kv;
  const int n_rep = a.H / a.n_kv;
  const int R = a.Tn * n_rep;
  const int tile0 = by * 16;
  const int len = a.lens[b] + a.slot_offset;
  if (a.depth) {
    if (tid < 64) s_depth[tid] = tid < a.Tn ? a.depth[tid] : 0;
    __syncthreads();
  }
  const int* depth = a.depth ? s_depth : nullptr;

  RowInfo row[2];
  int tq_min = 1 << 30, tq_max = -1, pos_min = 1 << 30, pos_top = -1;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = tile0 + g + 8 * h;
    row[h].valid = r < R;
    const int rr = row[h].valid ? r : 0;
    row[h].tq = rr % a.Tn;
    const int hrep = rr / a.Tn;
    row[h].pos = len + (depth ? depth[row[h].tq] : row[h].tq);
    row[h].slope = dmode ? 0.f : 1.0f / exp2f((float)(kvh * n_rep + hrep + 1) / (float)a.H);
    row[h].anc = a.anc ? a.anc[row[h].tq] : 0ull;
    row[h].long_row = DELTA && ((a.anc || a.row_tk) ? row[h].pos + 1 : len + a.Tn) > a.alibi_max;
  }
  // tile-wide key range (all threads compute the same numbers from the tile's rows)
  for (int r = tile0; r < tile0 + 16 && r < R; ++r) {
    const int tq = r % a.Tn;
    const int p = len + (depth ? depth[tq] : tq);
    tq_min = min(tq_min, tq); tq_max = max(tq_max, tq); pos_min = min(pos_min, p); pos_top = max(pos_top, p);
  }
  const int hi_new = a.anc ? len + a.Tn : len + tq_max + 1;  // appended slots this tile can see

  const long long ks = (long long)a.n_kv * 64;
  __nv_bfloat16* Kc = reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(a.kc)) + ((long long)b * a.max_seq * a.n_kv + kvh) * 64;
  __nv_bfloat16* Vc = reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(a.vc)) + ((long long)b * a.max_seq * a.n_kv + kvh) * 64;
  const __nv_bfloat16* Ks = reinterpret_cast<const __nv_bfloat16*>(a.sink_k) + (long long)kvh * 64;
  const __nv_bfloat16* Vs = reinterpret_cast<const __nv_bfloat16*>(a.sink_v) + (long long)kvh * 64;

  // ---- the warps are split between the window keys and the sink keys in proportion to their block counts (each
  // path keeps its own softmax; both are merged in one pass afterwards)
  const int lo_w = max(0, pos_min - a.window + 1);
  const int nblk_w = hi_new > lo_w ? (hi_new - lo_w + 15) >> 4 : 0;
  const int nblk_s = (a.n_sink + 15) >> 4;
  // which passes this tile runs: TriSparse and DSA take the window and the sinks; GMLA takes the window only for rows
  // beyond alibi_max keys (a chain is all on one side of the switch, a tree may straddle it); KDA has one pass
  const bool some_long = len + a.Tn > a.alibi_max;
  const bool need_ab = dmode == 0 || dmode == 1 || (dmode == 3 && some_long);
  const bool need_b = dmode == 0 || dmode == 1;
  int nw = 1;
  if (!need_b) nw = AW;
  else {
    int best = 1 << 30;
    for (int c = 1; c < AW; ++c) {           // the split whose busier group has the fewest blocks per warp
      const int cost = max((nblk_w + c - 1) / c, (nblk_s + AW - c - 1) / (AW - c));
      if (cost < best) { best = cost; nw = c; }
    }
  }
  unsigned char* ring = attn_smem + warp * (RING * 4096);
  // This warp's first key blocks go on their way now, under the set-up work below: cached window keys and sink keys
  // do not depend on this call's q | k | v.  A window warp whose first blocks reach into the rows that this very
  // CTA appends below has to wait for them.
  // DSA while every row's window still reaches back to the first key: its dense soft-max IS its window soft-max, so
  // the window result takes both weights and the dense pass is left out
  const bool c_is_a = DELTA && dmode == 1 && pos_top < a.window;
  const bool use_c = !c_is_a &&
                     (dmode == 2 ||
                      (a.use_alibi &&
                       ((a.anc || (DELTA && a.row_tk)) ? true
                            : (a.alibi_window > 0 ? min(len + a.Tn, a.alibi_window) : (len + a.Tn)) <= a.alibi_max)));
  const int lo_c = a.alibi_window > 0 ? max(0, pos_min - a.alibi_window + 1) : 0;
  // a module whose only pass is the one over all keys (GMLA up to alibi_max keys, KDA) starts that pass's first
  // cached blocks here as well
  bool early_c = false;
  if (DELTA && !need_ab && use_c) {
    const int nblk_c = hi_new > lo_c ? (hi_new - lo_c + 15) >> 4 : 0;
    const int last = warp + (RING - 2) * AW;
    early_c = lo_c + (min(last, max(nblk_c - 1, 0)) + 1) * 16 <= len;
  }
  bool early = need_ab;
  if (need_ab && warp < nw) {
    const int last = warp + (RING - 2) * nw;                 // its last block of the first batch
    early = lo_w + (min(last, max(nblk_w - 1, 0)) + 1) * 16 <= len;
  }
  {
    unsigned qf0[4][4] = {};
    float o0[8][4], m0[2], l0[2];
    if (early) {
      if (warp < nw) attend<0>(a, Kc, Vc, ks, lo_w, hi_new, len, row, qf0, depth, warp, nw, lane, ring, o0, m0, l0, 1);
      else attend<1>(a, Ks, Vs, ks, 0, a.n_sink, len, row, qf0, depth, warp - nw, AW - nw, lane, ring, o0, m0, l0, 1);
    }
    if constexpr (DELTA) {
      if (early_c) {
        if (dmode == 2) attend<3>(a, Kc, Vc, ks, lo_c, hi_new, len, row, qf0, depth, warp, AW, lane, ring, o0, m0, l0, 1);
        else attend<2>(a, Kc, Vc, ks, lo_c, hi_new, len, row, qf0, depth, warp, AW, lane, ring, o0, m0, l0, 1);
      }
    }
  }

  // The kernel is launched as a programmatic dependent of the kernel that produces q | k | v: everything above
  // touched only sequence lengths, static tables and cache entries below `len` (committed, or appended by earlier
  // forwards, which ended in plainly launched kernels), so it ran while that kernel was still finishing; its output
  // (the partial sums, or q and the appended K / V rows) is read from here on.
  pdl_wait();
  if (a.partial) {
    // ---- fused q|k|v finalize: this CTA sums the split-K slices of exactly the columns it needs -- the query rows
    // of its tile and the new K / V rows of its kv head -- applies RoPE, appends K / V to the cache (every tile of a
    // (sequence, kv head) writes the same values) and keeps the query rows in shared memory.  Work items are groups
    // of four feature pairs (j, j + 32): float4 loads from every slice.
    const long long ld = a.partial_ld;
    const int half = 32;
    auto sum4 = [&](long long at) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int sp = 0; sp < a.splits; ++sp) {
        const float4 v = *reinterpret_cast<const float4*>(a.partial + (long long)sp * a.pstride + at);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
      return acc;
    };
    auto rot4 = [&](float4& x1, float4& x2, int pos, int j) {
      if (!a.use_rope) return;
      const int pp = pos < a.rope_rows ? pos : a.rope_rows - 1;
      const float4 c = *reinterpret_cast<const float4*>(a.cos_t + (long long)pp * half + j);
      const float4 sn = *reinterpret_cast<const float4*>(a.sin_t + (long long)pp * half + j);
      const float4 o1 = make_float4(x1.x * c.x + (-x2.x) * sn.x, x1.y * c.y + (-x2.y) * sn.y,
                                    x1.z * c.z + (-x2.z) * sn.z, x1.w * c.w + (-x2.w) * sn.w);
      const float4 o2 = make_float4(x2.x * c.x + x1.x * sn.x, x2.y * c.y + x1.y * sn.y,
                                    x2.z * c.z + x1.z * sn.z, x2.w * c.w + x1.w * sn.w);
      x1 = o1; x2 = o2;
    };
    const int n_q = 16 * 8, n_k = a.Tn * 8, n_v = a.Tn * 16;
    for (int it = tid; it < n_q + n_k + n_v; it += AW * 32) {
      if (it < n_q) {
        const int rl = it >> 3, j = (it & 7) * 4, r = tile0 + rl;
        float4 x1 = make_float4(0.f, 0.f, 0.f, 0.f), x2 = x1;
        if (r < R) {
          const int tq = r % a.Tn, hrep = r / a.Tn;
          const long long at = (long long)(b * a.Tn + tq) * ld + (kvh * n_rep + hrep) * 64 + j;
          x1 = sum4(at); x2 = sum4(at + half);
          rot4(x1, x2, len + (depth ? depth[tq] : tq), j);
        }
        *reinterpret_cast<float4*>(s_q + rl * 64 + j) = x1;
        *reinterpret_cast<float4*>(s_q + rl * 64 + half + j) = x2;
      } else if (it < n_q + n_k) {
        const int i2 = it - n_q, tn = i2 >> 3, j = (i2 & 7) * 4;
        const int slot = len + tn;
        if (slot < a.max_seq) {
          const long long at = (long long)(b * a.Tn + tn) * ld + (a.H + kvh) * 64 + j;
          float4 x1 = sum4(at), x2 = sum4(at + half);
          rot4(x1, x2, len + (depth ? depth[tn] : tn), j);
          __nv_bfloat16* dst = Kc + (long long)slot * ks + j;
          reinterpret_cast<__nv_bfloat162*>(dst)[0] = __floats2bfloat162_rn(x1.x, x1.y);
          reinterpret_cast<__nv_bfloat162*>(dst)[1] = __floats2bfloat162_rn(x1.z, x1.w);
          reinterpret_cast<__nv_bfloat162*>(dst + half)[0] = __floats2bfloat162_rn(x2.x, x2.y);
          reinterpret_cast<__nv_bfloat162*>(dst + half)[1] = __floats2bfloat162_rn(x2.z, x2.w);
        }
      } else {
        const int i2 = it - n_q - n_k, tn = i2 >> 4, j = (i2 & 15) * 4;
        const int slot = len + tn;
        if (slot < a.max_seq) {
          const float4 x = sum4((long long)(b * a.Tn + tn) * ld + (a.H + a.n_kv + kvh) * 64 + j);
          __nv_bfloat16* dst = Vc + (long long)slot * ks + j;
          reinterpret_cast<__nv_bfloat162*>(dst)[0] = __floats2bfloat162_rn(x.x, x.y);
          reinterpret_cast<__nv_bfloat162*>(dst)[1] = __floats2bfloat162_rn(x.z, x.w);
        }
      }
    }
    __syncthreads();   // query rows are in shared memory; this CTA's K / V rows are visible to its own later loads
  }

  // Q fragments, dims permuted as described at the top of the file
  unsigned qf[4][4];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = tile0 + g + 8 * h;
    const int rr = r < R ? r : 0;
    const int tq = rr % a.Tn, hrep = rr / a.Tn;
    const float* q = a.partial ? s_q + (g + 8 * h) * 64 + 16 * t
                               : a.q + (long long)(b * a.Tn + tq) * a.ld_q + (kvh * n_rep + hrep) * 64 + 16 * t;
#pragma unroll
    for (int s = 0; s < 4; ++s) {
      const float4 v = a.partial ? *reinterpret_cast<const float4*>(q + 4 * s)
                                 : __ldcg(reinterpret_cast<const float4*>(q + 4 * s));
      qf[s][h] = r < R ? pack_bf16(v.x, v.y) : 0u;
      qf[s][2 + h] = r < R ? pack_bf16(v.z, v.w) : 0u;
    }
  }

  // final output of this thread after the cross-warp merge: row = tid / 16, dims 4 * (tid % 16) .. +3
  float fin[4] = {0.f, 0.f, 0.f, 0.f};
  const int mrow = tid >> 4, mcol = (tid & 15) * 4;
  // weight of a pass's result in this thread's output row: the sigmoid gates of TriSparse, or the delta module's
  // per-head weights on the row's side of the alibi_max switch (path 0 window, 1 sinks, 2 dense / KDA)
  auto gate_of = [&](int path) -> float {
    const int r = tile0 + mrow;
    const int rr = r < R ? r : 0;
    const int tq = rr % a.Tn, head = kvh * n_rep + rr / a.Tn;
    const int tk = (a.anc || (DELTA && a.row_tk)) ? len + (depth ? depth[tq] : tq) + 1 : len + a.Tn;
    if (!dmode) {
      if (path == 0) return a.g_a;
      if (path == 1) return a.g_b;
      // ALiBi path of a tree node is gated by its own T_k (position + 1 <= 1024)
      if (a.anc && (a.alibi_window > 0 ? min(tk, a.alibi_window) : tk) > a.alibi_max) return 0.f;
      return a.g_c;
    }
    const bool long_row = tk > a.alibi_max;
    if (path == 2) return (long_row && dmode != 2) ? 0.f : a.out_w * a.head_w[2 * a.H + head];
    return a.out_w * a.head_w[((long_row ? 3 : 0) + path) * a.H + head];
  };

  // each warp parks its partial result.  Column n of tile j is output dim 8n + j, so thread (g, t) holds dims
  // 16t .. 16t+15 of rows g and g + 8: four 16-byte chunks per row, chunk c stored at c ^ bit3(c) ^ 2*(row & 1),
  // which spreads the eight lanes of a quarter warp over all banks for the stores here and the loads of the merge
  auto park = [&](const float (&o)[8][4], const float (&m)[2], const float (&l)[2]) {
    float4* mine = reinterpret_cast<float4*>(ring);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = g + 8 * h;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int c = 4 * t + k, e = 2 * h + (k >> 1), j = (k & 1) * 4;
        mine[r * 16 + (c ^ ((c >> 3) & 1) ^ ((r & 1) << 1))] = make_float4(o[j][e], o[j + 1][e], o[j + 2][e], o[j + 3][e]);
      }
    }
    if (t == 0) {
      sM[warp][g] = m[0]; sL[warp][g] = l[0];
      sM[warp][g + 8] = m[1]; sL[warp][g + 8] = l[1];
    }
  };
  // merge of the warps [w0, w1) that shared one path: this thread's four output dims of row mrow, times gate / sum
  auto merge = [&](int w0, int w1, float gate) {
    float M = -CUDART_INF_F;
    for (int w = w0; w < w1; ++w) M = fmaxf(M, sM[w][mrow]);
    float L = 0.f, acc[4] = {0.f, 0.f, 0.f, 0.f};
    if (M != -CUDART_INF_F) {
      for (int w = w0; w < w1; ++w) {
        const float mw = sM[w][mrow];
        if (mw == -CUDART_INF_F) continue;
        const float cw = __expf(mw - M);
        L += sL[w][mrow] * cw;
        const int c = tid & 15;
        const float4 v = reinterpret_cast<const float4*>(attn_smem + w * (RING * 4096))[
            mrow * 16 + (c ^ ((c >> 3) & 1) ^ ((mrow & 1) << 1))];
        acc[0] += v.x * cw; acc[1] += v.y * cw; acc[2] += v.z * cw; acc[3] += v.w * cw;
      }
    }
    if (L > 0.f) {
      const float inv = gate / L;
#pragma unroll
      for (int e = 0; e < 4; ++e) fin[e] += acc[e] * inv;
    }
  };

  if (tr && tid == 0) tr[1] = clock_stamp();     // row setup and Q fragments done
  // ---- window path and sink path side by side
  if (need_ab) {
    float o[8][4], m[2], l[2];
    if (warp < nw) attend<0>(a, Kc, Vc, ks, lo_w, hi_new, len, row, qf, depth, warp, nw, lane, ring, o, m, l, early ? 2 : 0);
    else attend<1>(a, Ks, Vs, ks, 0, a.n_sink, len, row, qf, depth, warp - nw, AW - nw, lane, ring, o, m, l, early ? 2 : 0);
    if (tr && tid == 0) tr[2] = clock_stamp();   // this warp's keys done
    park(o, m, l);
    __syncthreads();
    merge(0, nw, gate_of(0) + (c_is_a ? gate_of(2) : 0.f));
    merge(nw, AW, gate_of(1));
    if (tr && tid == 0) tr[3] = clock_stamp();   // merge done
  }
  if (use_c) {
    __syncthreads();                             // everybody has read the parked tiles
    float o[8][4], m[2], l[2];
    if constexpr (DELTA) {
      if (dmode == 2) attend<3>(a, Kc, Vc, ks, lo_c, hi_new, len, row, qf, depth, warp, AW, lane, ring, o, m, l, early_c ? 2 : 0);
      else attend<2>(a, Kc, Vc, ks, lo_c, hi_new, len, row, qf, depth, warp, AW, lane, ring, o, m, l, early_c ? 2 : 0);
    } else {
      attend<2>(a, Kc, Vc, ks, lo_c, hi_new, len, row, qf, depth, warp, AW, lane, ring, o, m, l);
    }
    park(o, m, l);
    __syncthreads();
    merge(0, AW, gate_of(2));
  }
  const int r = tile0 + mrow;
  if (r < R) {
    const int tq = r % a.Tn, hrep = r / a.Tn;
    const long long at = (long long)(b * a.Tn + tq) * a.H * 64 + (kvh * n_rep + hrep) * 64 + mcol;
    if (DELTA && a.acc_in) {
      const float4 p = *reinterpret_cast<const float4*>(a.acc_in + at);
      fin[0] += p.x; fin[1] += p.y; fin[2] += p.z; fin[3] += p.w;
    }
    if (DELTA && a.acc_out) *reinterpret_cast<float4*>(a.acc_out + at) = make_float4(fin[0], fin[1], fin[2], fin[3]);
    if (!DELTA || a.out) {
      __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(a.out) + at;
      __nv_bfloat162 v0 = __floats2bfloat162_rn(fin[0], fin[1]), v1 = __floats2bfloat162_rn(fin[2], fin[3]);
      reinterpret_cast<__nv_bfloat162*>(out)[0] = v0;
      reinterpret_cast<__nv_bfloat162*>(out)[1] = v1;
    }
  }
}

__global__ void __launch_bounds__(AW * 32, 2) trisparse_attn_mma_kernel(AttnArgs a) {
  extern __shared__ __align__(128) unsigned char attn_smem_dyn[];
  long long* tr = a.trace ? a.trace + 8ll * (blockIdx.x + (long long)gridDim.x * blockIdx.y) : nullptr;
  if (tr && threadIdx.x == 0) tr[0] = clock_stamp();
  pdl_trigger();
  attn_tile<0>(a, blockIdx.x, blockIdx.y, attn_smem_dyn, tr);
}

// the same tile compiled for one delta-attention module (DM = AttnArgs::delta: 1 DSA, 2 KDA, 3 GMLA)
template <int DM>
__global__ void __launch_bounds__(AW * 32, 2) delta_attn_mma_kernel(AttnArgs a) {
  extern __shared__ __align__(128) unsigned char attn_smem_dyn[];
  pdl_trigger();
  attn_tile<DM>(a, blockIdx.x, blockIdx.y, attn_smem_dyn, nullptr);
}

// ---- prompt attention: the eight warps of a CTA take eight different 16-row tiles of one (sequence, kv head) --
// neighbouring positions, all of the kv head's query heads -- and share the key blocks, which the CTA streams once
// through a ring of three 32-key stages.  Every warp keeps its tile's two soft-max states (window, then sinks) to
// itself, so nothing is merged across warps and the tile is stored straight from the accumulators.  For chains
// without ALiBi (prompts of the mate target); everything else takes attn_tile.
constexpr int PF_STAGES = 3;
constexpr int PF_STAGE_BYTES = 8192;          // two 16-key blocks: K 2 KB + V 2 KB each

__global__ void __launch_bounds__(AW * 32, 2) trisparse_attn_prefill_kernel(AttnArgs a) {
  extern __shared__ __align__(128) unsigned char pf_smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int b = blockIdx.x / a.n_kv, kvh = blockIdx.x % a.n_kv;
  const int n_rep = a.H / a.n_kv;
  const int pb_per_cta = AW / n_rep;                       // blocks of 16 positions per CTA
  const int hrep = warp % n_rep, pb = blockIdx.y * pb_per_cta + warp / n_rep;
  const int len = a.lens[b] + a.slot_offset;
  const bool tile_on = 16 * pb < a.Tn;
  const int tq_min = 16 * pb, tq_max = min(a.Tn, 16 * pb + 16) - 1;
  RowInfo row[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int tq = 16 * pb + g + 8 * h;
    row[h].valid = tile_on && tq < a.Tn;
    row[h].tq = row[h].valid ? tq : 0;
    row[h].pos = len + row[h].tq;
    row[h].slope = 0.f;
    row[h].anc = 0ull;
    row[h].long_row = false;
  }
  const int pos_min = len + tq_min, pos_max = len + tq_max;
  const int P0 = blockIdx.y * pb_per_cta * 16, P1 = min(a.Tn, P0 + pb_per_cta * 16);
  const long long ks = (long long)a.n_kv * 64;
  const __nv_bfloat16* Kc = reinterpret_cast<const __nv_bfloat16*>(a.kc) + ((long long)b * a.max_seq * a.n_kv + kvh) * 64;
  const __nv_bfloat16* Vc = reinterpret_cast<const __nv_bfloat16*>(a.vc) + ((long long)b * a.max_seq * a.n_kv + kvh) * 64;
  const __nv_bfloat16* Ks = reinterpret_cast<const __nv_bfloat16*>(a.sink_k) + (long long)kvh * 64;
  const __nv_bfloat16* Vs = reinterpret_cast<const __nv_bfloat16*>(a.sink_v) + (long long)kvh * 64;

  // Q fragments of this warp's tile (dims permuted as in attn_tile)
  unsigned qf[4][4];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const float* q = a.q + (long long)(b * a.Tn + row[h].tq) * a.ld_q + (kvh * n_rep + hrep) * 64 + 16 * t;
#pragma unroll
    for (int s = 0; s < 4; ++s) {
      const float4 v = __ldcg(reinterpret_cast<const float4*>(q + 4 * s));
      qf[s][h] = row[h].valid ? pack_bf16(v.x, v.y) : 0u;
      qf[s][2 + h] = row[h].valid ? pack_bf16(v.z, v.w) : 0u;
    }
  }

  float fin[8][4];
#pragma unroll
  for (int j = 0; j < 8; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) fin[j][e] = 0.f;

  // one pass over the keys [lo, hi) of Kb / Vb: every thread copies one (key, 16-byte chunk) of K and of V per stage
  auto pass = [&](auto mode_tag, const __nv_bfloat16* Kb, const __nv_bfloat16* Vb, int lo, int hi, int hi_tile, float gate) {
    constexpr int MODE = decltype(mode_tag)::value;
    float o[8][4], m[2], l[2];
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) o[j][e] = 0.f;
    m[0] = m[1] = -CUDART_INF_F;
    l[0] = l[1] = 0.f;
    const int nst = hi > lo ? (hi - lo + 31) >> 5 : 0;
    auto issue = [&](int s) {
      unsigned char* st = pf_smem + (s % PF_STAGES) * PF_STAGE_BYTES;
      const int sb = tid >> 7, r = (tid & 127) >> 3, c = tid & 7;
      int key = lo + s * 32 + sb * 16 + r;
      key = key < hi ? key : hi - 1;
      const int soff = sb * 4096 + r * 128 + ((c ^ (r & 7)) << 4);
      mma_detail::cp_async16(st + soff, Kb + (long long)key * ks + c * 8, true);
      mma_detail::cp_async16(st + 2048 + soff, Vb + (long long)key * ks + c * 8, true);
    };
#pragma unroll
    for (int s = 0; s < PF_STAGES - 1; ++s) {
      if (s < nst) issue(s);
      mma_detail::cp_async_commit();
    }
    for (int s = 0; s < nst; ++s) {
      mma_detail::cp_async_wait<PF_STAGES - 2>();
      __syncthreads();                          // stage s has landed for everybody; stage s - 1 is free again
      if (s + PF_STAGES - 1 < nst) issue(s + PF_STAGES - 1);
      mma_detail::cp_async_commit();
      if (!tile_on) continue;
      const unsigned char* st = pf_smem + (s % PF_STAGES) * PF_STAGE_BYTES;
#pragma unroll
      for (int sb = 0; sb < 2; ++sb) {
        const int j0 = lo + s * 32 + sb * 16;
        if (j0 >= hi_tile) continue;                                        // behind the tile's last position
        if (MODE == 0 && pos_min - (j0 + 15) >= a.window) continue;         // before every row's window
        attend_block<MODE, MODE == 0>(a, st + sb * 4096, j0, hi_tile, len, row, qf, nullptr, pos_max, tq_min, g, t, o, m, l);
      }
    }
    mma_detail::cp_async_wait<0>();
    __syncthreads();                            // the ring is free for the next pass
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float L = l[h];
      L += __shfl_xor_sync(0xffffffffu, L, 1);
      L += __shfl_xor_sync(0xffffffffu, L, 2);
      if (L > 0.f) {
        const float inv = gate / L;
#pragma unroll
        for (int j = 0; j < 8; ++j) { fin[j][2 * h] += o[j][2 * h] * inv; fin[j][2 * h + 1] += o[j][2 * h + 1] * inv; }
      }
    }
  };
  const int lo_w = max(0, len + P0 - a.window + 1);
  pass(std::integral_constant<int, 0>(), Kc, Vc, lo_w, len + P1, len + tq_max + 1, a.g_a);
  pass(std::integral_constant<int, 1>(), Ks, Vs, 0, a.n_sink, a.n_sink, a.g_b);

  // thread (g, t) holds dims 16t .. 16t+15 of rows g and g + 8: dim 16t + 4k + i is fin[(k & 1) * 4 + i][2h + (k >> 1)]
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    if (!row[h].valid) continue;
    __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(a.out) + (long long)(b * a.Tn + row[h].tq) * a.H * 64 +
                         (kvh * n_rep + hrep) * 64 + 16 * t;
    unsigned w[8];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int e = 2 * h + (k >> 1), j = (k & 1) * 4;
      w[2 * k] = pack_bf16(fin[j][e], fin[j + 1][e]);
      w[2 * k + 1] = pack_bf16(fin[j + 2][e], fin[j + 3][e]);
    }
    reinterpret_cast<uint4*>(out)[0] = make_uint4(w[0], w[1], w[2], w[3]);
    reinterpret_cast<uint4*>(out)[1] = make_uint4(w[4], w[5], w[6], w[7]);
  }
}

}  // namespace attn_detail

inline bool attn_mma_supported(const AttnArgs& a, bool bf16) {
  return bf16 && a.hd == 64 && a.Tn <= (a.anc ? 64 : (1 << 20)) && (a.ld_q % 4) == 0;
}

inline int32_t launch_attn_mma(vn_ctx* ctx, const AttnArgs& a, int B) {
  const int n_rep = a.H / a.n_kv;
  dim3 grid(B * a.n_kv, ceil_div(a.Tn * n_rep, 16));
  const size_t smem = (size_t)attn_detail::AW * attn_detail::RING * 4096;
  static unsigned long long attr_set = 0;
  if (!((attr_set >> (ctx->device & 63)) & 1ull)) {
    VN_CUDA(ctx, cudaFuncSetAttribute(attn_detail::trisparse_attn_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)smem));
    VN_CUDA(ctx, cudaFuncSetAttribute(attn_detail::delta_attn_mma_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)smem));
    VN_CUDA(ctx, cudaFuncSetAttribute(attn_detail::delta_attn_mma_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)smem));
    VN_CUDA(ctx, cudaFuncSetAttribute(attn_detail::delta_attn_mma_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)smem));
    attr_set |= 1ull << (ctx->device & 63);
  }
  // VN_ATTN_PDL=0 (read once): plain launch
  static const bool attn_pdl = [] { const char* e = getenv("VN_ATTN_PDL"); return !(e && e[0] == '0'); }();
  const int level = ((vn_pdl_mask() & 1) || attn_pdl) ? 1 : 2;
  if (a.delta == 1) {
    VN_LAUNCH_PDL_LEVEL(ctx, level, "attn_detail::delta_attn_mma_kernel<dsa>", attn_detail::delta_attn_mma_kernel<1>, grid,
                        attn_detail::AW * 32, smem, a);
    return VN_OK;
  }
  if (a.delta == 2) {
    VN_LAUNCH_PDL_LEVEL(ctx, level, "attn_detail::delta_attn_mma_kernel<kda>", attn_detail::delta_attn_mma_kernel<2>, grid,
                        attn_detail::AW * 32, smem, a);
    return VN_OK;
  }
  if (a.delta == 3) {
    VN_LAUNCH_PDL_LEVEL(ctx, level, "attn_detail::delta_attn_mma_kernel<gmla>", attn_detail::delta_attn_mma_kernel<3>, grid,
                        attn_detail::AW * 32, smem, a);
    return VN_OK;
  }
  VN_LAUNCH_PDL_LEVEL(ctx, level, "attn_detail::trisparse_attn_mma_kernel", attn_detail::trisparse_attn_mma_kernel, grid,
                      attn_detail::AW * 32, smem, a);
  return VN_OK;
}

// prompts: many new rows per sequence, a chain, no ALiBi path, q already reduced (VN_ATTN_PREFILL=0, read per call,
// keeps the one-tile-per-CTA kernel)
inline bool attn_prefill_supported(const AttnArgs& a, bool bf16) {
  const char* e = getenv("VN_ATTN_PREFILL");
  if (e && e[0] == '0') return false;
  const int n_rep = a.n_kv > 0 ? a.H / a.n_kv : 0;
  return bf16 && a.hd == 64 && !a.anc && !a.depth && !a.use_alibi && !a.partial && a.Tn >= 32 && (a.ld_q % 4) == 0 &&
         (n_rep == 1 || n_rep == 2 || n_rep == 4 || n_rep == 8) && a.H == n_rep * a.n_kv && a.n_sink >= 1;
}

inline int32_t launch_attn_prefill(vn_ctx* ctx, const AttnArgs& a, int B) {
  const int n_rep = a.H / a.n_kv;
  const int pb_per_cta = attn_detail::AW / n_rep;
  dim3 grid(B * a.n_kv, ceil_div(ceil_div(a.Tn, 16), pb_per_cta));
  const size_t smem = (size_t)attn_detail::PF_STAGES * attn_detail::PF_STAGE_BYTES;
  VN_LAUNCH_NAMED(ctx, "trisparse_attn_prefill_kernel", attn_detail::trisparse_attn_prefill_kernel, grid, attn_detail::AW * 32,
                  smem, a);
  return VN_OK;
}
