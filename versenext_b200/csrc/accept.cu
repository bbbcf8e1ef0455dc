// Acceptance / rejection sampling over the vocabulary (HBM-streaming kernels).
//
// Full-vocabulary path (top_k <= 0), four launches on the context's stream:
//   accept_stats_kernel     every logit read once: per (row, 4096-float chunk) max / argmax /
//                           sum exp(x - chunk max)                     [the HBM-bound kernel]
//   accept_decide_kernel    per sequence: combine chunks, test u*q(x) < p(x), find the first
//                           rejected position
//   accept_residual_kernel  per (sequence, chunk): mass of max(0, p - q) of the ONE row pair
//                           that has to be resampled (or of p_k for the bonus token)
//   accept_pick_kernel      per sequence: inverse CDF over chunk masses, then inside one chunk
// Element-wise exponentials are float32; every sum, normalisation and CDF is float64, so a
// different summation order cannot move a decision relative to the CPU restatement.
//
// Top-k path: accept_topk_kernel reduces every row to its (token, scaled logit) list of the
// entries >= the k-th largest value (bound pass + rank counting, radix select as the fallback), the
// slices of a row are merged, and the same rule is applied on those short lists: three launches.
//
// Fused LM head (vn_k1_*, driven by vn_verify_accept): the target's logits never reach HBM.  A small GEMM over the
// first columns of the head gives every row a lower bound of its k-th largest logit (k1_bound_kernel), the full
// head GEMM's epilogue appends the logits at or above it to per-row candidate lists, k1_finish_kernel turns a
// candidate list into the same kept list the select above produces, and the decision kernel runs unchanged.  If a
// candidate list overflows (heavy ties), a device flag switches on the classic path inside the same launch
// sequence: its kernels return at once while the flag is clear.
#include <stdlib.h>
#include "common.cuh"
#include "k1.h"
#include <math_constants.h>

namespace {

constexpr int CHUNK = 4096;
constexpr int STATS_THREADS = 256;
constexpr int MAX_K = 16;            // draft positions per call
constexpr int KEEP_MAX = 1024;       // kept entries per row on the top-k path
constexpr int CAND_MAX = 1024;       // candidates gathered before the in-shared-memory select

struct RowSet {
  const float* p;
  const float* q;
  long long p_sb, p_si, q_sb, q_si;  // strides in elements
  int np, nq;                        // rows per sequence taken from p / q
  int V;
};

__device__ __forceinline__ const float* row_ptr(const RowSet& rs, int b, int j) {
  return j < rs.np ? rs.p + (long long)b * rs.p_sb + (long long)j * rs.p_si
                   : rs.q + (long long)b * rs.q_sb + (long long)(j - rs.np) * rs.q_si;
}

struct Partial {
  float m;
  int arg;
  double s;
};

struct Decision {
  int n_acc;     // accepted draft tokens
  int mode;      // 0 nothing to sample, 1 residual of (p_n, q_n), 2 plain p_n (bonus / fallback), 3 p_n with draft token removed
  int pos;       // row index n of the distribution to sample
  int x;         // draft token at pos (mode 3)
  float m_p, m_q;
  double inv_sp, inv_sq;
  float u;       // uniform for the inverse CDF
};

// ---- Philox4x32-10 -------------------------------------------------------
__device__ __forceinline__ uint32_t philox_word0(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3,
                                                 uint32_t k0, uint32_t k1) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    uint32_t n0 = hi1 ^ c1 ^ k0, n2 = hi0 ^ c3 ^ k1;
    c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
    k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
  }
  return c0;
}

__device__ __forceinline__ float philox_uniform(uint64_t seed, uint32_t offset, uint32_t row,
                                                uint32_t position, uint32_t purpose) {
  uint32_t w = philox_word0(position, row, purpose, offset, (uint32_t)seed, (uint32_t)(seed >> 32));
  return (float)(w >> 8) * 5.9604644775390625e-08f;  // 2^-24
}

__global__ void philox_uniform_kernel(uint64_t seed, uint32_t offset, int B, int n, int purpose, float* out) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < B * n) out[i] = philox_uniform(seed, offset, i / n, i % n, purpose);
}

// ---- block reductions -----------------------------------------------------
__device__ __forceinline__ void warp_argmax(float& m, int& a) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float om = __shfl_xor_sync(0xffffffffu, m, o);
    int oa = __shfl_xor_sync(0xffffffffu, a, o);
    if (om > m || (om == m && oa < a)) { m = om; a = oa; }
  }
}

__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ---- kernel A: streaming statistics ---------------------------------------
// One chunk = 4096 consecutive logits of one row (256 threads x 4 x float4); a work item is a PAIR of
// neighbouring chunks, so that the two block-wide reductions (max, then sum of exp) and their barriers are paid
// once per 8192 logits and every thread has eight 16-byte loads in flight.  Each chunk still gets its own
// (max, argmax, sum) record, computed exactly as if it were alone.  The arg-max index is only tracked for the
// greedy rule and exp only for the stochastic one.
template <bool VEC4, bool GREEDY>
__global__ void __launch_bounds__(STATS_THREADS)
accept_stats_kernel(RowSet rs, int B, int nchunks, float temp, Partial* __restrict__ out) {
  __shared__ float sm_m[2][STATS_THREADS / 32];
  __shared__ int sm_a[2][STATS_THREADS / 32];
  __shared__ double sm_s[2][STATS_THREADS / 32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int rows_per_seq = rs.np + rs.nq;
  const int npairs = (nchunks + 1) >> 1;
  const long long nitems = (long long)B * rows_per_seq * npairs;
  const bool scale = (temp != 1.0f) && !GREEDY;
  for (long long item = blockIdx.x; item < nitems; item += gridDim.x) {
    const int pi = (int)(item % npairs);
    const int r = (int)(item / npairs);
    const float* row = row_ptr(rs, r / rows_per_seq, r % rows_per_seq);
    const bool two = 2 * pi + 1 < nchunks;            // uniform over the CTA
    float x[2][16];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int start = (2 * pi + h) * CHUNK;
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int idx = start + u * (STATS_THREADS * 4) + tid * 4;
        if (VEC4 && idx + 3 < rs.V && (h == 0 || two)) {
          float4 v = __ldcs(reinterpret_cast<const float4*>(row + idx));
          x[h][u * 4 + 0] = v.x; x[h][u * 4 + 1] = v.y; x[h][u * 4 + 2] = v.z; x[h][u * 4 + 3] = v.w;
        } else {
#pragma unroll
          for (int e = 0; e < 4; ++e)
            x[h][u * 4 + e] = (idx + e < rs.V && (h == 0 || two)) ? __ldcs(row + idx + e) : -CUDART_INF_F;
        }
      }
    }
    if (scale) {
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int e = 0; e < 16; ++e) x[h][e] = __fdiv_rn(x[h][e], temp);
    }
    float m[2];
    int a[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      m[h] = -CUDART_INF_F;
      a[h] = 0x7fffffff;
      const int start = (2 * pi + h) * CHUNK;
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          if (GREEDY) {
            const int idx = start + u * (STATS_THREADS * 4) + tid * 4 + e;
            if (x[h][u * 4 + e] > m[h]) { m[h] = x[h][u * 4 + e]; a[h] = idx; }
          } else {
            m[h] = fmaxf(m[h], x[h][u * 4 + e]);
          }
        }
    }
    if (GREEDY) {
      warp_argmax(m[0], a[0]);
      warp_argmax(m[1], a[1]);
    } else {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        m[0] = fmaxf(m[0], __shfl_xor_sync(0xffffffffu, m[0], o));
        m[1] = fmaxf(m[1], __shfl_xor_sync(0xffffffffu, m[1], o));
      }
    }
    if (lane == 0) { sm_m[0][warp] = m[0]; sm_m[1][warp] = m[1]; if (GREEDY) { sm_a[0][warp] = a[0]; sm_a[1][warp] = a[1]; } }
    __syncthreads();
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      m[h] = sm_m[h][0];
      if (GREEDY) a[h] = sm_a[h][0];
#pragma unroll
      for (int w = 1; w < STATS_THREADS / 32; ++w) {
        const float om = sm_m[h][w];
        if (GREEDY) {
          const int oa = sm_a[h][w];
          if (om > m[h] || (om == m[h] && oa < a[h])) { m[h] = om; a[h] = oa; }
        } else {
          m[h] = fmaxf(m[h], om);
        }
      }
    }
    if (!GREEDY) {
      float sf0 = 0.f, sf1 = 0.f;
#pragma unroll
      for (int e = 0; e < 16; ++e) sf0 += expf(x[0][e] - m[0]);
      if (two) {
#pragma unroll
        for (int e = 0; e < 16; ++e) sf1 += expf(x[1][e] - m[1]);
      }
      const double s0 = warp_sum((double)sf0), s1 = warp_sum((double)sf1);
      if (lane == 0) { sm_s[0][warp] = s0; sm_s[1][warp] = s1; }
    }
    __syncthreads();
    if (tid < 2 && (tid == 0 || two)) {
      double tot = 0.0;
      if (!GREEDY)
#pragma unroll
        for (int w = 0; w < STATS_THREADS / 32; ++w) tot += sm_s[tid][w];
      Partial p; p.m = tid == 0 ? m[0] : m[1]; p.arg = GREEDY ? (tid == 0 ? a[0] : a[1]) : 0; p.s = tot;
      out[(long long)r * nchunks + 2 * pi + tid] = p;
    }
  }
}

// the four instantiations behind one call
static int32_t launch_accept_stats(vn_ctx* ctx, bool vec, bool greedy, int grid, const RowSet& rs, int B, int nchunks,
                                   float temp, Partial* part) {
  if (vec && greedy) VN_LAUNCH(ctx, (accept_stats_kernel<true, true>), grid, STATS_THREADS, 0, rs, B, nchunks, temp, part);
  else if (vec) VN_LAUNCH(ctx, (accept_stats_kernel<true, false>), grid, STATS_THREADS, 0, rs, B, nchunks, temp, part);
  else if (greedy) VN_LAUNCH(ctx, (accept_stats_kernel<false, true>), grid, STATS_THREADS, 0, rs, B, nchunks, temp, part);
  else VN_LAUNCH(ctx, (accept_stats_kernel<false, false>), grid, STATS_THREADS, 0, rs, B, nchunks, temp, part);
  return VN_OK;
}

// ---- kernel B: per-sequence decision --------------------------------------
__device__ __forceinline__ float scaled(float x, float temp) { return temp != 1.0f ? __fdiv_rn(x, temp) : x; }

// one warp per row of the sequence (at least 4 warps): the rows' chunk records are merged side by side
static inline int decide_threads(int rows_per_seq) { return 32 * std::min(32, std::max(4, rows_per_seq)); }

__global__ void accept_decide_kernel(RowSet rs, int B, int k, int nchunks, const Partial* __restrict__ part,
                                     const long long* __restrict__ draft, const float* __restrict__ u_acc,
                                     const float* __restrict__ u_smp, uint64_t seed, uint32_t offset_host,
                                     const unsigned* __restrict__ offset_dev,
                                     float temp, int greedy, int bonus, int smp_purpose, int pos_base,
                                     Decision* __restrict__ dec, int* __restrict__ out_len,
                                     long long* __restrict__ out_tok) {
  const int b = blockIdx.x;
  const uint32_t offset = offset_host + (offset_dev ? *offset_dev : 0u);  // device-side round counter, if any
  const int rows_per_seq = rs.np + rs.nq;
  __shared__ float r_m[2 * MAX_K + 1];
  __shared__ int r_a[2 * MAX_K + 1];
  __shared__ double r_s[2 * MAX_K + 1];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  for (int j = warp; j < rows_per_seq; j += nwarps) {
    const Partial* pp = part + ((long long)b * rows_per_seq + j) * nchunks;
    float m = -CUDART_INF_F; int a = 0x7fffffff;
    for (int c = lane; c < nchunks; c += 32) {
      Partial p = pp[c];
      if (p.m > m || (p.m == m && p.arg < a)) { m = p.m; a = p.arg; }
    }
    warp_argmax(m, a);
    double s = 0.0;
    if (!greedy)
      for (int c = lane; c < nchunks; c += 32) {
        Partial p = pp[c];
        s += p.s * exp((double)(p.m - m));
      }
    s = warp_sum(s);
    if (lane == 0) { r_m[j] = m; r_a[j] = a; r_s[j] = s; }
  }
  // the draft tokens' logits and the acceptance uniforms of all k positions in one round trip: the serial
  // accept loop below then runs on shared memory
  __shared__ long long s_x[MAX_K];
  __shared__ float s_lp[MAX_K], s_lq[MAX_K], s_u[MAX_K];
  if (!greedy && (int)threadIdx.x < k) {
    const int n = threadIdx.x;
    const long long x = draft[(long long)b * k + n];
    const bool x_ok = x >= 0 && x < rs.V;
    s_x[n] = x;
    s_lp[n] = x_ok ? scaled(row_ptr(rs, b, n)[x], temp) : -CUDART_INF_F;
    s_lq[n] = (rs.nq && x_ok) ? scaled(row_ptr(rs, b, rs.np + n)[x], temp) : -CUDART_INF_F;
    s_u[n] = u_acc ? u_acc[(long long)b * k + n] : philox_uniform(seed, offset, b, pos_base + n, 0);
  }
  __syncthreads();
  if (threadIdx.x != 0) return;
  Decision d;
  d.mode = 0; d.pos = 0; d.x = -1; d.m_p = d.m_q = 0.f; d.inv_sp = d.inv_sq = 0.0; d.u = 0.f;
  long long* tok = out_tok + (long long)b * (k + 1);
  for (int i = 0; i <= k; ++i) tok[i] = -1;
  int n = 0;
  if (greedy) {
    while (n < k && draft[(long long)b * k + n] == (long long)r_a[n]) { tok[n] = r_a[n]; ++n; }
    if (n < k) tok[n] = r_a[n];
    else if (bonus) tok[k] = r_a[k];
    d.n_acc = n;
    if (out_len) out_len[b] = n;
    dec[b] = d;
    return;
  }
  bool rejected = false;
  for (; n < k; ++n) {
    const long long x = s_x[n];
    const double p = (double)expf(s_lp[n] - r_m[n]) / r_s[n];
    double q = 1.0;
    if (rs.nq) q = (double)expf(s_lq[n] - r_m[rs.np + n]) / r_s[rs.np + n];
    const float u = s_u[n];
    if ((double)u * q < p) { tok[n] = x; continue; }
    rejected = true;
    d.mode = rs.nq ? 1 : 3;
    d.pos = n;
    d.x = (int)x;
    d.m_p = r_m[n]; d.inv_sp = 1.0 / r_s[n];
    if (rs.nq) { d.m_q = r_m[rs.np + n]; d.inv_sq = 1.0 / r_s[rs.np + n]; }
    break;
  }
  if (!rejected && bonus) {
    d.mode = 2; d.pos = k; d.m_p = r_m[k]; d.inv_sp = 1.0 / r_s[k];
  }
  if (d.mode) d.u = u_smp ? u_smp[(long long)b * (k + 1) + d.pos] : philox_uniform(seed, offset, b, pos_base + d.pos, smp_purpose);
  d.n_acc = n;
  if (out_len) out_len[b] = n;
  dec[b] = d;
}

// residual weight of one token under decision d (double)
__device__ __forceinline__ double residual_weight(const Decision& d, float xp, float xq, int token, bool plain) {
  double p = (double)expf(xp - d.m_p) * d.inv_sp;
  if (plain || d.mode == 2) return p;
  if (d.mode == 3) return token == d.x ? 0.0 : p;
  double q = (double)expf(xq - d.m_q) * d.inv_sq;
  double r = p - q;
  return r > 0.0 ? r : 0.0;
}

// ---- kernel C: residual mass per (sequence, chunk) ------------------------
// mass[b][c][0] = sum of max(0, p - q), mass[b][c][1] = sum of p (fallback when the residual vanishes)
template <bool VEC4>
__global__ void __launch_bounds__(STATS_THREADS)
accept_residual_kernel(RowSet rs, int nchunks, float temp, const Decision* __restrict__ dec,
                       double* __restrict__ mass) {
  const int b = blockIdx.y, c = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const Decision d = dec[b];
  if (d.mode == 0) return;
  __shared__ double sm[2][STATS_THREADS / 32];
  const float* rp = row_ptr(rs, b, d.pos);
  const float* rq = d.mode == 1 ? row_ptr(rs, b, rs.np + d.pos) : nullptr;
  const bool scale = temp != 1.0f;
  double acc_r = 0.0, acc_p = 0.0;
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int idx = c * CHUNK + u * (STATS_THREADS * 4) + tid * 4;
    float xp[4], xq[4] = {0.f, 0.f, 0.f, 0.f};
    if (VEC4 && idx + 3 < rs.V) {
      float4 v = *reinterpret_cast<const float4*>(rp + idx);
      xp[0] = v.x; xp[1] = v.y; xp[2] = v.z; xp[3] = v.w;
      if (rq) { float4 w = *reinterpret_cast<const float4*>(rq + idx); xq[0] = w.x; xq[1] = w.y; xq[2] = w.z; xq[3] = w.w; }
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        xp[e] = idx + e < rs.V ? rp[idx + e] : -CUDART_INF_F;
        if (rq) xq[e] = idx + e < rs.V ? rq[idx + e] : -CUDART_INF_F;
      }
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      if (idx + e >= rs.V) continue;
      const float a = scale ? __fdiv_rn(xp[e], temp) : xp[e];
      const double p = (double)expf(a - d.m_p) * d.inv_sp;
      double r = p;
      if (d.mode == 1) {
        const float qs = scale ? __fdiv_rn(xq[e], temp) : xq[e];
        r = p - (double)expf(qs - d.m_q) * d.inv_sq;
        r = r > 0.0 ? r : 0.0;
      } else if (d.mode == 3 && idx + e == d.x) {
        r = 0.0;
      }
      acc_r += r;
      acc_p += p;
    }
  }
  acc_r = warp_sum(acc_r);
  acc_p = warp_sum(acc_p);
  if (lane == 0) { sm[0][warp] = acc_r; sm[1][warp] = acc_p; }
  __syncthreads();
  if (tid == 0) {
    double r = 0.0, p = 0.0;
#pragma unroll
    for (int w = 0; w < STATS_THREADS / 32; ++w) { r += sm[0][w]; p += sm[1][w]; }
    mass[((long long)b * nchunks + c) * 2 + 0] = r;
    mass[((long long)b * nchunks + c) * 2 + 1] = p;
  }
}

// ---- kernel D: inverse CDF ------------------------------------------------
__global__ void __launch_bounds__(STATS_THREADS)
accept_pick_kernel(RowSet rs, int k, int nchunks, float temp, const Decision* __restrict__ dec,
                   const double* __restrict__ mass, long long* __restrict__ out_tok) {
  const int b = blockIdx.x, tid = threadIdx.x;
  const Decision d = dec[b];
  if (d.mode == 0) return;
  __shared__ int s_chunk, s_plain, s_thread;
  __shared__ double s_before, s_target;
  __shared__ double s_part[STATS_THREADS];
  // chunk masses of this sequence in shared memory (one round trip instead of dependent loads in thread 0)
  constexpr int PICK_MAX = 512;
  __shared__ double s_mass[2 * PICK_MAX];
  const double* mg = mass + (long long)b * nchunks * 2;
  const bool staged = nchunks <= PICK_MAX;
  if (staged)
    for (int i = tid; i < 2 * nchunks; i += STATS_THREADS) s_mass[i] = mg[i];
  __syncthreads();
  const double* mb = staged ? s_mass : mg;
  if (tid == 0) {
    double Z = 0.0;
    for (int c = 0; c < nchunks; ++c) Z += mb[c * 2];
    int plain = 0;
    if (!(Z > 0.0)) {  // residual vanished: fall back to p itself
      plain = 1; Z = 0.0;
      for (int c = 0; c < nchunks; ++c) Z += mb[c * 2 + 1];
    }
    const double target = (double)d.u * Z;
    double cum = 0.0; int chosen = -1; double before = 0.0; int last_nz = 0;
    for (int c = 0; c < nchunks; ++c) {
      const double w = mb[c * 2 + plain];
      if (w > 0.0) last_nz = c;
      if (chosen < 0 && cum + w > target) { chosen = c; before = cum; }
      cum += w;
    }
    if (chosen < 0) {  // rounding pushed the target past the total: last token that has weight
      chosen = last_nz; before = 0.0;
      for (int c = 0; c < last_nz; ++c) before += mb[c * 2 + plain];
    }
    s_chunk = chosen; s_plain = plain; s_before = before; s_target = target;
  }
  __syncthreads();
  const int c = s_chunk; const bool plain = s_plain != 0;
  const float* rp = row_ptr(rs, b, d.pos);
  const float* rq = d.mode == 1 ? row_ptr(rs, b, rs.np + d.pos) : nullptr;
  const bool scale = temp != 1.0f;
  // thread t owns 16 consecutive tokens so that the scan order is ascending token id
  double w[16];
  double local = 0.0;
  const int base = c * CHUNK + tid * 16;
#pragma unroll
  for (int e = 0; e < 16; ++e) {
    const int t = base + e;
    double v = 0.0;
    if (t < rs.V) {
      float a = scale ? __fdiv_rn(rp[t], temp) : rp[t];
      float q = rq ? (scale ? __fdiv_rn(rq[t], temp) : rq[t]) : 0.f;
      v = residual_weight(d, a, q, t, plain);
    }
    w[e] = v;
    local += v;
  }
  // which thread's 16 tokens hold the target: an exclusive scan of the threads' sums (warp shuffles, then the
  // warps' totals), the first thread whose running sum passes the target; the last thread with weight when
  // rounding pushed the target past the total
  {
    const int lane = tid & 31, warp = tid >> 5;
    double incl = local;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const double up = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += up;
    }
    if (lane == 31) s_part[warp] = incl;
    if (tid == 0) s_thread = 0x7fffffff;
    __shared__ int s_last;
    if (tid == 0) s_last = -1;
    __syncthreads();
    double before = s_before;
    for (int w2 = 0; w2 < warp; ++w2) before += s_part[w2];
    const double excl = before + (incl - local);
    if (excl + local > s_target) atomicMin(&s_thread, tid);
    if (local > 0.0) atomicMax(&s_last, tid);
    __syncthreads();
    const int chosen = s_thread;
    __syncthreads();
    if (chosen == 0x7fffffff) {
      if (tid == 0) { s_thread = s_last < 0 ? 0 : s_last; s_before = -1.0; }
    } else if (tid == chosen) {
      s_before = excl;
    }
    __syncthreads();
  }
  if (tid == s_thread) {
    int pick = -1, last_nz = -1;
    if (s_before >= 0.0) {
      double cum = s_before;
#pragma unroll
      for (int e = 0; e < 16; ++e) {
        if (w[e] > 0.0) last_nz = e;
        if (pick < 0 && cum + w[e] > s_target) pick = e;
        cum += w[e];
      }
    } else {
#pragma unroll
      for (int e = 0; e < 16; ++e) if (w[e] > 0.0) last_nz = e;
    }
    if (pick < 0) pick = last_nz < 0 ? 0 : last_nz;
    out_tok[(long long)b * (k + 1) + d.n_acc] = base + pick;
  }
}

// ---- top-k path -----------------------------------------------------------
__device__ __forceinline__ uint32_t order_key(float f) {
  uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_value(uint32_t k) {
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

// neighbours of a float in the ordering of the reals (NaN and the infinity in the direction of travel stay put)
__device__ __forceinline__ float next_up(float x) {
  if (x != x || x == CUDART_INF_F) return x;
  if (x == 0.f) return __int_as_float(1);
  int b = __float_as_int(x);
  b += b >= 0 ? 1 : -1;
  return __int_as_float(b);
}
__device__ __forceinline__ float next_down(float x) { return -next_up(-x); }

struct TopkRow {
  int n;                 // kept entries
  int overflow;          // 1 when ties at the threshold did not fit
  int tok[KEEP_MAX];     // ascending token id
  float val[KEEP_MAX];   // scaled logit
  int pad[30];           // whole 128-byte lines: no two lists share a cache line (a CTA reads lists that CTAs on
                         // other SMs wrote earlier in the same kernel; a shared line could be stale in its L1)
};
static_assert(sizeof(TopkRow) % 128 == 0, "TopkRow must cover whole cache lines");

// what the decision step needs besides the lists
struct DecideArgs {
  int B, k, np, nq;
  // kept lists: row j < np of sequence b at p_rows[b * p_sb + j], draft row i at q_rows[b * q_sb + i * q_si]
  const TopkRow* p_rows;
  const TopkRow* q_rows;
  long long p_sb, q_sb, q_si;
  const long long* draft;
  const float* u_acc;
  const float* u_smp;
  uint64_t seed;
  uint32_t offset_host;
  const unsigned* offset_dev;
  int bonus, smp_purpose, pos_base;
  int* out_len;
  long long* out_tok;
};

constexpr int DEC_ROWS = 16, DEC_ENT = 64;

// One CTA per row.  Radix select (11 + 11 + 10 bits) of the k-th largest key.  After each level
// the number of keys that can still be kept is known from the histogram; as soon as they fit in
// shared memory they are gathered (one more read of the row) and the select finishes there.
// `out_sb`: list of slice c of row j of sequence b goes to out[(b * out_sb + j) * chunks + c] (lets the rows of a
// call land inside a larger per-sequence array).  `run_if`: see the GEMM's TcArgs::run_if.
__global__ void __launch_bounds__(1024, 2)
accept_topk_kernel(RowSet rs, int top_k, float temp, int chunks, TopkRow* out, long long out_sb, const int* run_if) {
  pdl_trigger();
  pdl_wait();
  if (run_if && *reinterpret_cast<const volatile int*>(run_if) == 0) return;
  // blockIdx.x = row * chunks + chunk: every CTA selects inside its own slice of the row; the slices'
  // lists are merged by accept_topk_merge_kernel (the row's k largest are among the slices' k largest)
  const int rows_per_seq = rs.np + rs.nq;
  const int r = blockIdx.x / chunks, chunk = blockIdx.x % chunks;
  const int slice = (((rs.V + chunks - 1) / chunks) + 3) & ~3;
  const int base0 = chunk * slice;
  const float* row = row_ptr(rs, r / rows_per_seq, r % rows_per_seq) + base0;
  const int V = max(0, min(slice, rs.V - base0)), tid = threadIdx.x, nt = blockDim.x;
  const bool scale = temp != 1.0f;
  const int want = top_k < V ? top_k : V;
  // histogram + candidates (16 KB)
  __shared__ __align__(16) unsigned char s_pool[16384];
  uint32_t* hist = reinterpret_cast<uint32_t*>(s_pool);                   // [2048]
  uint32_t* c_key = reinterpret_cast<uint32_t*>(s_pool + 8192);           // [CAND_MAX]
  int* c_tok = reinterpret_cast<int*>(s_pool + 12288);                    // [CAND_MAX]
  __shared__ int wcount[32];
  __shared__ uint32_t s_prefix, s_mask, s_kth;
  __shared__ int s_need, s_ncand, s_done, s_nout, s_base;
  if (tid == 0) { s_prefix = 0; s_mask = 0; s_need = want; s_ncand = 0; s_done = 0; s_nout = 0; s_base = 0; s_kth = 0; }
  __syncthreads();
  // ---- bound pass.  Groups of four threads take the maximum of the entries they read; the want-th largest
  // of the 256 group maxima is a lower bound of the want-th largest entry (those maxima are want distinct
  // entries), so everything kept lies at or above it.  On logits this leaves a few more than want candidates
  // after one read of the slice and no histogram; adversarial orders or heavy ties overflow the candidate
  // buffer and take the radix select below.
  __shared__ uint32_t s_bmax[256];
  __shared__ uint32_t s_lo;
  __shared__ float s_xlo;
  __shared__ int s_fast;
  const bool vec = (reinterpret_cast<uintptr_t>(row) & 15) == 0;
  const int V4 = vec ? (V >> 2) : 0;
  const float4* row4 = reinterpret_cast<const float4*>(row);
  {
    float tmax = -CUDART_INF_F;
    int i = tid;
    for (; i + 3 * nt < V4; i += 4 * nt) {
      const float4 a0 = __ldg(row4 + i), a1 = __ldg(row4 + i + nt), a2 = __ldg(row4 + i + 2 * nt),
                   a3 = __ldg(row4 + i + 3 * nt);
      tmax = fmaxf(tmax, fmaxf(fmaxf(fmaxf(a0.x, a0.y), fmaxf(a0.z, a0.w)), fmaxf(fmaxf(a1.x, a1.y), fmaxf(a1.z, a1.w))));
      tmax = fmaxf(tmax, fmaxf(fmaxf(fmaxf(a2.x, a2.y), fmaxf(a2.z, a2.w)), fmaxf(fmaxf(a3.x, a3.y), fmaxf(a3.z, a3.w))));
    }
    for (; i < V4; i += nt) {
      const float4 a0 = __ldg(row4 + i);
      tmax = fmaxf(tmax, fmaxf(fmaxf(a0.x, a0.y), fmaxf(a0.z, a0.w)));
    }
    for (int j = (V4 << 2) + tid; j < V; j += nt) tmax = fmaxf(tmax, row[j]);
    tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
    tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
    if (tid == 0) s_lo = 0u;
    if ((tid & 3) == 0 && (tid >> 2) < 256) s_bmax[tid >> 2] = order_key(scale ? __fdiv_rn(tmax, temp) : tmax);
    __syncthreads();
    const int nb = min(nt >> 2, 256);
    if (tid < nb) {
      const uint32_t mine = s_bmax[tid];
      int greater = 0, geq = 0;
      for (int j = 0; j < nb; ++j) { const uint32_t o = s_bmax[j]; greater += o > mine; geq += o >= mine; }
      if (greater < want && geq >= want) s_lo = mine;   // every writer holds the same key
    }
    __syncthreads();
    // The gather pass compares raw logits: x / temp is monotone in x, so "scaled key >= lo" is "x >= x_lo" for the
    // smallest float x_lo whose quotient reaches lo's value; one thread finds it by stepping single floats around
    // lo * temp (a handful of steps).  The division then runs for the few candidates only, not for every logit.
    if (tid == 0) {
      int fast = 0;
      float xlo = -CUDART_INF_F;
      const uint32_t lo_key = s_lo;
      if (lo_key != 0u) {
        const float lo_val = key_value(lo_key);
        if (!scale) { xlo = lo_val; fast = lo_val == lo_val; }
        else if (lo_val == lo_val && fabsf(lo_val) != CUDART_INF_F) {
          float c = lo_val * temp;
          int it = 0;
          while (it < 64 && !(__fdiv_rn(c, temp) >= lo_val)) { c = next_up(c); ++it; }
          while (it < 64 && __fdiv_rn(next_down(c), temp) >= lo_val && next_down(c) != c) { c = next_down(c); ++it; }
          fast = it < 64 && c == c && __fdiv_rn(c, temp) >= lo_val && !(__fdiv_rn(next_down(c), temp) >= lo_val);
          xlo = c;
        }
      }
      s_xlo = xlo; s_fast = fast;
    }
    __syncthreads();
  }
  // candidates: every entry with key >= lo (slot order is arbitrary, the select below ranks them)
  auto gather = [&](uint32_t lo, bool fast, float xlo) {
    int i = tid;
    if (fast) {
      auto take = [&](const float4& a, int at) {
        if (fmaxf(fmaxf(a.x, a.y), fmaxf(a.z, a.w)) >= xlo) {
          const float xs[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
          for (int e = 0; e < 4; ++e)
            if (xs[e] >= xlo) {
              const uint32_t key = order_key(scale ? __fdiv_rn(xs[e], temp) : xs[e]);
              const int slot = atomicAdd(&s_ncand, 1);
              if (slot < CAND_MAX) { c_key[slot] = key; c_tok[slot] = base0 + 4 * at + e; }
            }
        }
      };
      // four loads in flight per thread, as in the bound pass: behind the atomic of a candidate the next load of a
      // one-at-a-time loop could not be issued early
      for (; i + 3 * nt < V4; i += 4 * nt) {
        const float4 a0 = __ldg(row4 + i), a1 = __ldg(row4 + i + nt), a2 = __ldg(row4 + i + 2 * nt),
                     a3 = __ldg(row4 + i + 3 * nt);
        take(a0, i); take(a1, i + nt); take(a2, i + 2 * nt); take(a3, i + 3 * nt);
      }
      for (; i < V4; i += nt) take(__ldg(row4 + i), i);
    }
    for (; i < V4; i += nt) {
      const float4 a = __ldg(row4 + i);
      const float xs[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const uint32_t key = order_key(scale ? __fdiv_rn(xs[e], temp) : xs[e]);
        if (key >= lo) {
          const int slot = atomicAdd(&s_ncand, 1);
          if (slot < CAND_MAX) { c_key[slot] = key; c_tok[slot] = base0 + 4 * i + e; }
        }
      }
    }
    for (int j = (V4 << 2) + tid; j < V; j += nt) {
      const float x = row[j];
      const uint32_t key = order_key(scale ? __fdiv_rn(x, temp) : x);
      if (key >= lo) {
        const int slot = atomicAdd(&s_ncand, 1);
        if (slot < CAND_MAX) { c_key[slot] = key; c_tok[slot] = base0 + j; }
      }
    }
  };
  bool have = false;
  if (want > 0) {
    gather(s_lo, s_fast != 0, s_xlo);
    __syncthreads();
    have = s_ncand <= CAND_MAX;
    __syncthreads();
  }
  if (!have) {
    if (tid == 0) s_ncand = 0;
    __syncthreads();
    for (int level = 0; level < 3; ++level) {
      const int sh = level == 0 ? 21 : (level == 1 ? 10 : 0);
      const uint32_t nb = level == 2 ? 1024u : 2048u;
      for (int i = tid; i < 2048; i += nt) hist[i] = 0;
      __syncthreads();
      const uint32_t prefix = s_prefix, mask = s_mask;
      for (int i = tid; i < V; i += nt) {
        float x = row[i];
        if (scale) x = __fdiv_rn(x, temp);
        const uint32_t key = order_key(x);
        if ((key & mask) == prefix) atomicAdd(&hist[(key >> sh) & (nb - 1)], 1u);
      }
      __syncthreads();
      {
        // digit of the threshold: the largest d with (keys in digits > d) < need <= (keys in digits >= d).
        // Block-wide suffix sums over the histogram; thread t owns digits 2t and 2t+1 (launched with 1024 threads).
        const int need = s_need;  // how many of the largest keys of this prefix class are kept
        const int lane = tid & 31, warp = tid >> 5;
        const int h0 = (2 * tid < (int)nb) ? (int)hist[2 * tid] : 0;
        const int h1 = (2 * tid + 1 < (int)nb) ? (int)hist[2 * tid + 1] : 0;
        const int local = h0 + h1;
        int incl = local;       // inclusive suffix sum inside the warp (lanes above me)
  #pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int v = __shfl_down_sync(0xffffffffu, incl, o);
          if (lane + o < 32) incl += v;
        }
        if (lane == 0) wcount[warp] = incl;   // warp total
        __syncthreads();
        int above_warps = 0;
        for (int w = warp + 1; w < (nt >> 5); ++w) above_warps += wcount[w];
        const int above_me = above_warps + incl - local;   // keys in digits owned by threads after me
        if (need > 0 && above_me < need && need <= above_me + local) {
          uint32_t digit; int above;
          if (above_me + h1 >= need) { digit = 2 * tid + 1; above = above_me; }
          else { digit = 2 * tid; above = above_me + h1; }
          s_need = need - above;                 // still needed from inside the digit class
          s_prefix = prefix | (digit << sh);
          s_mask = mask | ((nb - 1) << sh);
          const int ncand = want - (need - above) + (int)hist[digit];  // keys >= the smallest key of the class
          s_ncand = ncand;
          s_done = ncand <= CAND_MAX ? 2 : (level == 2 ? 1 : 0);
        }
        if (need <= 0 && tid == 0) { s_ncand = 0; s_done = 2; s_prefix = 0xFFFFFFFFu; }   // empty slice
      }
      __syncthreads();
      if (s_done) break;
    }
    if (s_done == 2) {
      const uint32_t lo = s_prefix;
      __syncthreads();
      if (tid == 0) s_ncand = 0;
      __syncthreads();
      gather(lo, false, 0.f);
      __syncthreads();
      have = true;
    }
  }
  TopkRow* o = out + ((long long)(r / rows_per_seq) * out_sb + (r % rows_per_seq)) * chunks + chunk;
  if (have) {
    const int nc = min(s_ncand, CAND_MAX);
    // exact k-th largest among the candidates by rank counting (nc is small)
    for (int i = tid; i < nc; i += nt) {
      const uint32_t ki = c_key[i];
      int greater = 0, geq = 0;
      for (int j = 0; j < nc; ++j) { greater += c_key[j] > ki; geq += c_key[j] >= ki; }
      if (greater < want && geq >= want) s_kth = ki;  // every writer holds the same key
    }
    __syncthreads();
    const uint32_t kth = s_kth;
    for (int i = tid; i < nc; i += nt)
      if (c_key[i] >= kth) {
        int pos = 0;  // kept candidates with a smaller token id: output is ascending in id
        for (int j = 0; j < nc; ++j) pos += (c_key[j] >= kth) && (c_tok[j] < c_tok[i]);
        if (pos < KEEP_MAX) { o->tok[pos] = c_tok[i]; o->val[pos] = key_value(c_key[i]); }
        atomicAdd(&s_nout, 1);
      }
    __syncthreads();
    if (tid == 0) { o->n = min(s_nout, KEEP_MAX); o->overflow = s_nout > KEEP_MAX; }
  } else {
    // every bit resolved and still too many ties at the threshold: stream the kept entries
    // out in id order, truncated to KEEP_MAX (overflow flag set)
    const uint32_t kth = s_prefix;
    const int lane = tid & 31, warp = tid >> 5;
    for (int start = 0; start < V; start += nt) {
      const int i = start + tid;
      bool keep = false; uint32_t key = 0;
      if (i < V) {
        float x = row[i];
        if (scale) x = __fdiv_rn(x, temp);
        key = order_key(x);
        keep = key >= kth;
      }
      const unsigned bal = __ballot_sync(0xffffffffu, keep);
      if (lane == 0) wcount[warp] = __popc(bal);
      __syncthreads();
      int off = s_base;
      for (int w = 0; w < warp; ++w) off += wcount[w];
      off += __popc(bal & ((1u << lane) - 1));
      if (keep && off < KEEP_MAX) { o->tok[off] = base0 + i; o->val[off] = key_value(key); }
      __syncthreads();
      if (tid == 0) { int tot = 0; for (int w = 0; w < (nt >> 5); ++w) tot += wcount[w]; s_base += tot; }
      __syncthreads();
    }
    if (tid == 0) { o->n = min(s_base, KEEP_MAX); o->overflow = s_base > KEEP_MAX; }
  }
}

// Merge the slices' lists of one row: the global k-th largest value is found among the candidates by rank
// counting, everything >= it is kept; slices are in ascending token order, so the output is too.
__device__ void topk_merge_rows(const TopkRow* pr, int chunks, int top_k, TopkRow* o, float* s_val, int* s_tok,
                                int* s_off, int* s_n, float* s_kth, int* s_cnt) {
  constexpr int MERGE_MAX = 4096;
  const int tid = threadIdx.x, nt = blockDim.x;
  __syncthreads();             // the caller's earlier use of the shared arrays is over
  // list lengths in one round trip (chunks <= 64), exclusive offsets by one thread
  if (tid < 64) s_n[tid] = tid < chunks ? pr[tid].n : 0;
  if (tid == 0) { *s_kth = -CUDART_INF_F; *s_cnt = 0; }
  __syncthreads();
  if (tid == 0) {
    int acc = 0;
    for (int c = 0; c < chunks; ++c) { s_off[c] = acc; acc += s_n[c]; }
    s_off[chunks] = acc < MERGE_MAX ? acc : MERGE_MAX;
  }
  __syncthreads();
  const int n = s_off[chunks];
  for (int at = tid; at < n; at += nt) {
    int c = 0;
    while (c + 1 < chunks && s_off[c + 1] <= at) ++c;
    const int i = at - s_off[c];
    s_val[at] = pr[c].val[i];
    s_tok[at] = pr[c].tok[i];
  }
  __syncthreads();
  const int want = top_k < n ? top_k : n;
  for (int i = tid; i < n; i += nt) {
    const float vi = s_val[i];
    int greater = 0, geq = 0;
    for (int j = 0; j < n; ++j) { greater += s_val[j] > vi; geq += s_val[j] >= vi; }
    if (greater < want && geq >= want) *s_kth = vi;   // every writer holds the same value
  }
  __syncthreads();
  const float kth = *s_kth;
  for (int i = tid; i < n; i += nt)
    if (s_val[i] >= kth) {
      int pos = 0;
      for (int j = 0; j < i; ++j) pos += s_val[j] >= kth;
      if (pos < KEEP_MAX) { o->tok[pos] = s_tok[i]; o->val[pos] = s_val[i]; }
      atomicAdd(s_cnt, 1);
    }
  __syncthreads();
  if (tid == 0) { o->n = min(*s_cnt, KEEP_MAX); o->overflow = *s_cnt > KEEP_MAX; }
}

// parts: [rows][chunks] in row order; row r = (sequence r / rps, row r % rps) goes to out[(r / rps) * out_sb + r % rps]
__global__ void __launch_bounds__(1024)
accept_topk_merge_kernel(const TopkRow* __restrict__ parts, int chunks, int top_k, TopkRow* __restrict__ out, int rps,
                         long long out_sb, const int* run_if) {
  pdl_trigger();
  pdl_wait();
  if (run_if && *reinterpret_cast<const volatile int*>(run_if) == 0) return;
  __shared__ float s_val[4096];
  __shared__ int s_tok[4096];
  __shared__ int s_off[65], s_n[64], s_cnt;
  __shared__ float s_kth;
  const int r = blockIdx.x;
  topk_merge_rows(parts + (long long)r * chunks, chunks, top_k, out + (long long)(r / rps) * out_sb + r % rps, s_val, s_tok,
                  s_off, s_n, &s_kth, &s_cnt);
}

// ---- warp-cooperative helpers on a kept list ------------------------------------------------------------
// a kept list where it currently lives: the row in global memory, or the warp's copy in shared memory
struct ListView {
  const int* tok;
  const float* val;
  int n;
};

__device__ __forceinline__ void list_stats(const ListView& r, int lane, float& m, double& s) {
  m = -CUDART_INF_F;
  for (int i = lane; i < r.n; i += 32) m = fmaxf(m, r.val[i]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  double acc = 0.0;
  for (int i = lane; i < r.n; i += 32) acc += (double)expf(r.val[i] - m);
  s = warp_sum(acc);
}

// value of `token` in the list, or -inf when it is not kept (all lanes get the result)
__device__ __forceinline__ float list_value(const ListView& r, int lane, int token) {
  float v = -CUDART_INF_F;
  for (int i = lane; i < r.n; i += 32)
    if (r.tok[i] == token) v = r.val[i];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// per-lane lookup: binary search of `token` in the list (ascending token ids); -inf when it is not kept
__device__ __forceinline__ float list_find(const ListView& r, int token) {
  int lo = 0, hi = r.n;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (r.tok[mid] < token) lo = mid + 1; else hi = mid;
  }
  return (lo < r.n && r.tok[lo] == token) ? r.val[lo] : -CUDART_INF_F;
}

// One warp per sequence: acceptance tests, then the inverse CDF over the kept list of the row to sample.
// s_tok / s_val / s_n: this warp's staging arrays in shared memory.
__device__ __noinline__ void topk_decide_seq(int b, int lane, const DecideArgs& da,
                                             int (*s_tok)[DEC_ENT], float (*s_val)[DEC_ENT], int* s_n) {
  const int k = da.k, np = da.np, nq = da.nq, bonus = da.bonus, smp_purpose = da.smp_purpose, pos_base = da.pos_base;
  const long long* draft = da.draft;
  const float* u_acc = da.u_acc;
  const float* u_smp = da.u_smp;
  const uint64_t seed = da.seed;
  int* out_len = da.out_len;
  long long* out_tok = da.out_tok;
  const uint32_t offset = da.offset_host + (da.offset_dev ? *da.offset_dev : 0u);
  const int rows_per_seq = np + nq;
  auto rowp = [&](int r) -> const TopkRow* {
    return r < np ? da.p_rows + (long long)b * da.p_sb + r : da.q_rows + (long long)b * da.q_sb + (long long)(r - np) * da.q_si;
  };
  // The lists of this sequence are read many times below, each read a dependent round trip to L2: copy them
  // into shared memory first when they fit (at most DEC_ROWS rows of DEC_ENT entries, the usual case).
  bool staged = rows_per_seq <= DEC_ROWS;
  if (staged) {
    int nmax = 0;
    for (int r = lane; r < rows_per_seq; r += 32) { const int nr = rowp(r)->n; s_n[r] = nr; nmax = max(nmax, nr); }
    __syncwarp();
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) nmax = max(nmax, __shfl_xor_sync(0xffffffffu, nmax, o));
    staged = nmax <= DEC_ENT;
  }
  if (staged) {
    // eight entries per lane are requested before the first is stored: a plain copy loop waits for every load
    // before it can issue the next (some forty round trips to L2 for nine rows)
    const int total = rows_per_seq * DEC_ENT;
    for (int idx0 = 0; idx0 < total; idx0 += 32 * 8) {
      int tk[8]; float vl[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int idx = idx0 + u * 32 + lane;
        const int r = idx / DEC_ENT, i = idx % DEC_ENT;
        tk[u] = 0; vl[u] = 0.f;
        if (idx < total && i < s_n[r]) { const TopkRow* rp = rowp(r); tk[u] = rp->tok[i]; vl[u] = rp->val[i]; }
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int idx = idx0 + u * 32 + lane;
        const int r = idx / DEC_ENT, i = idx % DEC_ENT;
        if (idx < total && i < s_n[r]) { s_tok[r][i] = tk[u]; s_val[r][i] = vl[u]; }
      }
    }
    __syncwarp();
  }
  auto view = [&](int r) {
    ListView v;
    const TopkRow* rp = rowp(r);
    v.n = staged ? s_n[r] : rp->n;
    v.tok = staged ? s_tok[r] : rp->tok;
    v.val = staged ? s_val[r] : rp->val;
    return v;
  };
  long long* tok = out_tok + (long long)b * (k + 1);
  for (int i = lane; i <= k; i += 32) tok[i] = -1;
  __syncwarp();
  int n = 0;
  int sample_row = -1, q_row = -1, removed = -1;
  // the k proposals and their uniforms in one round trip (lane n holds position n), not one per loop trip
  int x_lane = 0; float u_lane = 0.f;
  if (lane < k) {
    x_lane = (int)draft[(long long)b * k + lane];
    u_lane = u_acc ? u_acc[(long long)b * k + lane] : philox_uniform(seed, offset, b, pos_base + lane, 0);
  }
  for (; n < k; ++n) {
    const int x = __shfl_sync(0xffffffffu, x_lane, n);
    float mp; double sp;
    list_stats(view(n), lane, mp, sp);
    const float vp = list_value(view(n), lane, x);
    const double p = vp == -CUDART_INF_F ? 0.0 : (double)expf(vp - mp) / sp;
    double q = 1.0;
    if (nq) {
      float mq; double sq;
      list_stats(view(np + n), lane, mq, sq);
      const float vq = list_value(view(np + n), lane, x);
      q = vq == -CUDART_INF_F ? 0.0 : (double)expf(vq - mq) / sq;
    }
    const float u = __shfl_sync(0xffffffffu, u_lane, n);
    if ((double)u * q < p) { if (lane == 0) tok[n] = x; continue; }
    sample_row = n;
    if (nq) q_row = np + n; else removed = x;
    break;
  }
  if (lane == 0 && out_len) out_len[b] = n;
  if (sample_row < 0) {
    if (!bonus) return;
    sample_row = k;
  }
  const ListView P = view(sample_row);
  float mp; double sp;
  list_stats(P, lane, mp, sp);
  float mq = 0.f; double sq = 1.0;
  const ListView Q = view(q_row >= 0 ? q_row : 0);
  if (q_row >= 0) list_stats(Q, lane, mq, sq);
  const float u = u_smp ? u_smp[(long long)b * (k + 1) + sample_row]
                        : philox_uniform(seed, offset, b, pos_base + sample_row, smp_purpose);
  for (int pass = 0; pass < 2; ++pass) {
    // pass 0: residual max(0, p - q) (or p without the rejected token); pass 1, only when that vanished: p itself
    auto weight = [&](int i) -> double {
      const double p = (double)expf(P.val[i] - mp) / sp;
      if (pass == 1) return p;
      if (q_row >= 0) {
        // q's value for this token: all lanes of the warp look it up together
        return p;  // placeholder, replaced below (needs a warp-wide lookup)
      }
      return P.tok[i] == removed ? 0.0 : p;
    };
    // weights of the entries this lane owns, in chunks of 32 consecutive entries (ascending token id)
    double Z = 0.0;
    const int nchunk = (P.n + 31) >> 5;
    // first sweep: total mass
    for (int c = 0; c < nchunk; ++c) {
      const int i = c * 32 + lane;
      double w = 0.0;
      const int tk = i < P.n ? P.tok[i] : -1;
      if (pass == 0 && q_row >= 0) {
        // every lane needs q(tk) for its own token: loop over the 32 tokens of the chunk
        if (i < P.n) {   // every lane looks up q for its own token
          const float my_vq = list_find(Q, tk);
          const double pp = (double)expf(P.val[i] - mp) / sp;
          const double qq = my_vq == -CUDART_INF_F ? 0.0 : (double)expf(my_vq - mq) / sq;
          w = pp - qq > 0.0 ? pp - qq : 0.0;
        }
      } else if (i < P.n) {
        w = weight(i);
      }
      Z += w;
    }
    Z = warp_sum(Z);
    if (!(Z > 0.0)) continue;
    const double target = (double)u * Z;
    double run = 0.0;
    int pick = -1, last_nz = -1;
    for (int c = 0; c < nchunk && pick < 0; ++c) {
      const int i = c * 32 + lane;
      double w = 0.0;
      const int tk = i < P.n ? P.tok[i] : -1;
      if (pass == 0 && q_row >= 0) {
        if (i < P.n) {   // every lane looks up q for its own token
          const float my_vq = list_find(Q, tk);
          const double pp = (double)expf(P.val[i] - mp) / sp;
          const double qq = my_vq == -CUDART_INF_F ? 0.0 : (double)expf(my_vq - mq) / sq;
          w = pp - qq > 0.0 ? pp - qq : 0.0;
        }
      } else if (i < P.n) {
        w = weight(i);
      }
      // inclusive scan of the chunk in entry order
      double cum = w;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const double up = __shfl_up_sync(0xffffffffu, cum, o);
        if (lane >= o) cum += up;
      }
      cum += run;
      const unsigned hit = __ballot_sync(0xffffffffu, i < P.n && cum > target);
      const unsigned nz = __ballot_sync(0xffffffffu, i < P.n && w > 0.0);
      if (nz) last_nz = c * 32 + (31 - __clz(nz));
      if (hit) pick = c * 32 + (__ffs(hit) - 1);
      run = __shfl_sync(0xffffffffu, cum, 31);
    }
    if (pick < 0) pick = last_nz;
    if (lane == 0 && pick >= 0) tok[n] = P.tok[pick];
    return;
  }
}


__global__ void __launch_bounds__(128)
accept_topk_decide_kernel(DecideArgs da) {
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31, wslot = threadIdx.x >> 5;
  const int b = blockIdx.x * (blockDim.x >> 5) + wslot;
  if (b >= da.B) return;
  __shared__ int s_tok[4][DEC_ROWS][DEC_ENT];
  __shared__ float s_val[4][DEC_ROWS][DEC_ENT];
  __shared__ int s_n[4][DEC_ROWS];
  topk_decide_seq(b, lane, da, s_tok[wslot], s_val[wslot], s_n[wslot]);
}


// ---- stochastic acceptance on a verified tree with FIXED proposals -------------------------------------------
// The children of a node are given tokens (the draft's best ones, distinct, in order), so the test is rejection
// sampling with point-mass proposals, child after child: at a row with target distribution p (its kept list) and
// remaining mass R = 1, child c with token x is accepted iff u * R < p(x); otherwise x leaves the support
// (R -= p(x)) and the next child is tried -- the first child is taken with probability p(x1), the second with
// (1 - p(x1)) * p(x2) / (1 - p(x1)) = p(x2), and so on: every committed token has exactly its target probability.
// Where no child is accepted (or the row has none, or the path is `depth` long) the row's token is drawn from p
// without the rejected children: inverse CDF over ascending token ids, float64 sums, as in topk_decide_seq.
// One warp per sequence.  Row 0 = after the last committed token, row r = after node row r; outputs as
// tree_accept_greedy_kernel's (engine.cu).  A row may have at most TREE_CHILD_MAX children.
constexpr int TREE_CHILD_MAX = 8;

struct TreeSampleArgs {
  const TopkRow* rows;       // [B * T] kept lists of the target rows
  const long long* tokens;   // [B, T]
  const int* parent;         // [T] parent row (-1 for row 0)
  const float* u_child;      // [B, T] injected uniforms of the child tests, or null: Philox (row b, position c, purpose 0)
  const float* u_sample;     // [B, T] injected uniforms of the final draw, or null: Philox (row b, position row, purpose 1)
  uint64_t seed;
  uint32_t offset_host;
  const unsigned* offset_dev;
  int B, T, depth;
  int* out_len;
  long long* out_tok;        // [B, depth + 1]
  int* keep_t;               // [B, depth + 1]
  int* keep_d;
};

__global__ void __launch_bounds__(128) tree_accept_sample_kernel(TreeSampleArgs ta) {
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int b = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (b >= ta.B) return;
  const int T = ta.T, depth = ta.depth;
  const uint32_t offset = ta.offset_host + (ta.offset_dev ? *ta.offset_dev : 0u);
  const long long* tok = ta.tokens + (long long)b * T;
  long long* ot = ta.out_tok + (long long)b * (depth + 1);
  int* kt = ta.keep_t + (long long)b * (depth + 1);
  int* kd = ta.keep_d + (long long)b * (depth + 1);
  for (int i = lane; i <= depth; i += 32) { ot[i] = -1; kt[i] = 0; kd[i] = (i == 1) ? 1 : 0; }
  __syncwarp();
  int cur = 0, a = 0;
  for (;;) {
    const TopkRow* rp = ta.rows + (long long)b * T + cur;
    ListView P;
    P.tok = rp->tok; P.val = rp->val; P.n = rp->n;
    float mp; double sp;
    list_stats(P, lane, mp, sp);
    double R = 1.0;
    int removed[TREE_CHILD_MAX];
    int n_removed = 0, took = -1;
    long long took_tok = -1;
    if (a < depth) {
      for (int c = cur + 1; c < T; ++c) {
        if (ta.parent[c] != cur) continue;
        const long long x = tok[c];
        const float v = list_value(P, lane, (int)x);
        const double px = v == -CUDART_INF_F ? 0.0 : (double)expf(v - mp) / sp;
        const float u = ta.u_child ? ta.u_child[(long long)b * T + c] : philox_uniform(ta.seed, offset, b, c, 0);
        if ((double)u * R < px) { took = c; took_tok = x; break; }
        if (n_removed < TREE_CHILD_MAX) removed[n_removed++] = (int)x;
        R -= px;
      }
    }
    if (took >= 0) {
      if (lane == 0) {
        ot[a] = took_tok;
        kt[a + 1] = took;
        if (a + 2 <= depth) kd[a + 2] = took + 1;
      }
      cur = took;
      ++a;
      continue;
    }
    const float u = ta.u_sample ? ta.u_sample[(long long)b * T + cur] : philox_uniform(ta.seed, offset, b, cur, 1);
    const int nchunk = (P.n + 31) >> 5;
    for (int pass = 0; pass < 2; ++pass) {
      // pass 0: p without the rejected children; pass 1, only when nothing is left of it: p itself
      auto weight = [&](int i) -> double {
        if (i >= P.n) return 0.0;
        const int t = P.tok[i];
        if (pass == 0)
          for (int r = 0; r < n_removed; ++r)
            if (removed[r] == t) return 0.0;
        return (double)expf(P.val[i] - mp) / sp;
      };
      double Z = 0.0;
      for (int c = 0; c < nchunk; ++c) Z += weight(c * 32 + lane);
      Z = warp_sum(Z);
      if (!(Z > 0.0)) continue;
      const double target = (double)u * Z;
      double run = 0.0;
      int pick = -1, last_nz = -1;
      for (int c = 0; c < nchunk && pick < 0; ++c) {
        const int i = c * 32 + lane;
        const double w = weight(i);
        double cum = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const double up = __shfl_up_sync(0xffffffffu, cum, o);
          if (lane >= o) cum += up;
        }
        cum += run;
        const unsigned hit = __ballot_sync(0xffffffffu, i < P.n && cum > target);
        const unsigned nz = __ballot_sync(0xffffffffu, i < P.n && w > 0.0);
        if (nz) last_nz = c * 32 + (31 - __clz(nz));
        if (hit) pick = c * 32 + (__ffs(hit) - 1);
        run = __shfl_sync(0xffffffffu, cum, 31);
      }
      if (pick < 0) pick = last_nz;
      if (lane == 0 && pick >= 0) ot[a] = P.tok[pick];
      break;
    }
    break;
  }
  if (lane == 0 && ta.out_len) ta.out_len[b] = a;
}


// ---- fused LM head: bound, finish ---------------------------------------------------------------------------
// One CTA per target row.  Every thread takes the maximum of its share of the row's first nb logits; the k-th
// largest of those per-thread maxima is a lower bound of the k-th largest of the subset (they are k distinct
// entries), hence of the whole row (a subset's k-th largest never exceeds the full set's) -- and with k far below
// the number of threads it is almost as tight as the subset's own k-th largest.  The bound handed to the GEMM
// epilogue is the SMALLEST raw logit whose temperature-scaled value reaches the scaled bound, so that a logit whose
// quotient ties with the k-th value after rounding is still collected.  Also clears the row's candidate counter
// and the call's fallback flag.
__global__ void __launch_bounds__(1024)
k1_bound_kernel(const float* __restrict__ boot, int nb, int top_k, float temp, float* __restrict__ tau,
                int* __restrict__ count, int count_stride, int* __restrict__ fallback) {
  pdl_trigger();
  pdl_wait();
  __shared__ uint32_t s_max[1024];
  __shared__ uint32_t s_kth;
  const int row = blockIdx.x, tid = threadIdx.x, nt = blockDim.x;
  const float* src = boot + (long long)row * nb;
  float mx = -CUDART_INF_F;
  int mine = 0;
  for (int i0 = tid; i0 < nb; i0 += 8 * nt) {      // eight loads in flight per thread
    float x[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) x[u] = i0 + u * nt < nb ? src[i0 + u * nt] : -CUDART_INF_F;
#pragma unroll
    for (int u = 0; u < 8; ++u)
      if (i0 + u * nt < nb) { mx = fmaxf(mx, x[u]); ++mine; }
  }
  s_max[tid] = mine ? order_key(mx) : 0u;           // 0 sorts below every real key
  if (tid == 0) s_kth = 0u;
  __syncthreads();
  const int groups = nb < nt ? nb : nt;             // threads that hold a value
  if (top_k <= groups && tid < groups) {
    const uint32_t me = s_max[tid];
    int greater = 0, geq = 0;
    for (int j = 0; j < groups; ++j) { const uint32_t o = s_max[j]; greater += o > me; geq += o >= me; }
    if (greater < top_k && geq >= top_k) s_kth = me;    // every writer holds the same key
  }
  __syncthreads();
  if (tid == 0) {
    float t = -CUDART_INF_F;
    if (top_k <= groups && s_kth != 0u) {
      const float xk = key_value(s_kth);
      t = xk;
      if (xk != xk) {
        t = -CUDART_INF_F;
      } else if (temp != 1.0f && fabsf(xk) != CUDART_INF_F) {
        const float sk = __fdiv_rn(xk, temp);
        int it = 0;
        while (it < 64 && next_down(t) != t && __fdiv_rn(next_down(t), temp) >= sk) { t = next_down(t); ++it; }
        if (it >= 64) t = -CUDART_INF_F;      // could not pin the edge down: collect everything, the overflow path decides
      }
    }
    tau[row] = t;
    count[(long long)row * count_stride] = 0;
    if (row == 0) *fallback = 0;
  }
}

// One CTA (256 threads) per target row: candidates (raw logit, token) -> the kept list the select kernel would have
// produced: every entry whose scaled value is >= the k-th largest scaled value, ascending token id.  Rank counting
// over all candidates would cost n^2 comparisons, so the list is first cut down the same way the bound was made:
// the k-th largest of the per-thread maxima bounds the k-th largest candidate from below, and only the candidates
// at or above it (a few more than k as a rule) are ranked.  A list that ran past its capacity, or more than
// KEEP_MAX kept entries, raises the fallback flag instead.
constexpr int K1_FIN_THREADS = 256;
__global__ void __launch_bounds__(K1_FIN_THREADS)
k1_finish_kernel(const float* __restrict__ cand_val, const int* __restrict__ cand_tok, const int* __restrict__ count,
                 int count_stride, int cap, int top_k, float temp, int V, TopkRow* __restrict__ out,
                 int* __restrict__ fallback) {
  pdl_trigger();
  pdl_wait();
  __shared__ uint32_t s_key[VN_K1_CAP];
  __shared__ uint32_t s_gmax[K1_FIN_THREADS];
  __shared__ int s_ci[KEEP_MAX];            // indices (into the candidate list) of the short list
  __shared__ uint32_t s_ck[KEEP_MAX];
  __shared__ int s_ktok[KEEP_MAX];
  __shared__ uint32_t s_kkey[KEEP_MAX];
  __shared__ uint32_t s_lo, s_kth;
  __shared__ int s_nc, s_keep;
  const int row = blockIdx.x, tid = threadIdx.x, nt = blockDim.x;
  const int n = count[(long long)row * count_stride];
  const int want = top_k < V ? top_k : V;
  TopkRow* o = out + row;
  if (n > cap || n < want) {                 // uniform over the CTA
    if (tid == 0) { atomicExch(fallback, 1); o->n = 0; o->overflow = 1; }
    return;
  }
  const bool scale = temp != 1.0f;
  const float* cv = cand_val + (long long)row * cap;
  const int* ct = cand_tok + (long long)row * cap;
  uint32_t gmax = 0u;
  for (int i0 = tid; i0 < n; i0 += 8 * nt) {      // eight candidates per thread requested before the first is used
    float x[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) x[u] = i0 + u * nt < n ? cv[i0 + u * nt] : 0.f;
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int i = i0 + u * nt;
      if (i < n) {
        const uint32_t key = order_key(scale ? __fdiv_rn(x[u], temp) : x[u]);
        s_key[i] = key;
        gmax = key > gmax ? key : gmax;
      }
    }
  }
  s_gmax[tid] = gmax;                        // 0 (below every real key) for a thread without candidates
  if (tid == 0) { s_lo = 0u; s_kth = 0u; s_nc = 0; s_keep = 0; }
  __syncthreads();
  // lower bound of the k-th largest candidate: the k-th largest thread maximum (when at least k threads hold one)
  {
    const uint32_t me = s_gmax[tid];
    int greater = 0, geq = 0;
    for (int j = 0; j < nt; ++j) { const uint32_t k2 = s_gmax[j]; greater += k2 > me; geq += k2 >= me; }
    if (me != 0u && greater < want && geq >= want) s_lo = me;     // every writer holds the same key
  }
  __syncthreads();
  const uint32_t lo = s_lo;                  // 0: fewer than k threads have candidates, every candidate stays
  for (int i = tid; i < n; i += nt)
    if (s_key[i] >= lo) {
      const int slot = atomicAdd(&s_nc, 1);
      if (slot < KEEP_MAX) { s_ci[slot] = i; s_ck[slot] = s_key[i]; }
    }
  __syncthreads();
  const int nc = s_nc;
  if (nc > KEEP_MAX) {                       // heavy ties around the bound: the stored-logits path sorts it out
    if (tid == 0) { atomicExch(fallback, 1); o->n = 0; o->overflow = 1; }
    return;
  }
  // exact k-th largest among the short list (it holds every candidate >= lo, so at least k of them)
  for (int i = tid; i < nc; i += nt) {
    const uint32_t me = s_ck[i];
    int greater = 0, geq = 0;
    for (int j = 0; j < nc; ++j) { const uint32_t k2 = s_ck[j]; greater += k2 > me; geq += k2 >= me; }
    if (greater < want && geq >= want) s_kth = me;
  }
  __syncthreads();
  const uint32_t kth = s_kth;
  for (int i = tid; i < nc; i += nt)
    if (s_ck[i] >= kth) {
      const int slot = atomicAdd(&s_keep, 1);
      s_kkey[slot] = s_ck[i];                // slot < nc <= KEEP_MAX
      s_ktok[slot] = ct[s_ci[i]];
    }
  __syncthreads();
  const int keep = s_keep;
  // ascending token id: rank of each kept entry among the kept ones
  for (int i = tid; i < keep; i += nt) {
    const int ti = s_ktok[i];
    int pos = 0;
    for (int j = 0; j < keep; ++j) pos += s_ktok[j] < ti;
    o->tok[pos] = ti;
    o->val[pos] = key_value(s_kkey[i]);
  }
  if (tid == 0) { o->n = keep; o->overflow = 0; }
}


// ---- acceptance over a vocabulary split across ranks, on the device -------------------------------------------------
// Every rank holds columns [v_lo, v_lo + Vs) of the target and draft logits of ALL sequences (Bt = world x B of them).
// Three all-gathers of a few numbers per row make every rank take identical decisions (each rank merges the ranks'
// contributions in rank order, in float64):
//   1. per row (max, sum exp) of the shard and the shard's scaled logit of the draft token (-inf when another shard
//      owns it)  -> global softmax statistics, p(x), q(x), the accept tests, the row to sample;
//   2. the shard's residual mass sum max(0, p - q) (and sum p) of that row  -> the shard that holds the sampled token
//      (shards in ascending token order) and the fraction of its mass at which the token lies;
//   3. the token picked inside that shard.
// Same arithmetic as the single-GPU kernels above: float32 exp(x - max), float64 sums, accept iff u q(x) < p(x).

// exchange 1, send side: [6][Bt][k+1] doubles = p max, p sum, p logit of x, q max, q sum, q logit of x (q padded at k)
__global__ void shard_pack1_kernel(RowSet rs, int Bt, int k, int nchunks, const Partial* __restrict__ part, float temp,
                                   const long long* __restrict__ draft, int v_lo, double* __restrict__ send) {
  const int lane = threadIdx.x & 31;
  const int rows_per_seq = rs.np + rs.nq;
  const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= Bt * rows_per_seq) return;
  const int b = r / rows_per_seq, j = r % rows_per_seq;
  const Partial* pp = part + (long long)r * nchunks;
  float m = -CUDART_INF_F;
  for (int c = lane; c < nchunks; c += 32) m = fmaxf(m, pp[c].m);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  double s = 0.0;
  for (int c = lane; c < nchunks; c += 32) {
    const Partial p = pp[c];
    if (p.m != -CUDART_INF_F) s += p.s * exp((double)(p.m - m));
  }
  s = warp_sum(s);
  if (lane != 0) return;
  const bool is_q = j >= rs.np;
  const int pos = is_q ? j - rs.np : j;
  double x = -CUDART_INF;
  if (pos < k) {
    const long long t = draft[(long long)b * k + pos] - v_lo;
    if (t >= 0 && t < rs.V) x = (double)scaled(row_ptr(rs, b, j)[t], temp);
  }
  const long long plane = (long long)Bt * (k + 1), at = (long long)b * (k + 1) + pos;
  const int f = is_q ? 3 : 0;
  send[(f + 0) * plane + at] = (double)m;
  send[(f + 1) * plane + at] = s;
  send[(f + 2) * plane + at] = x;
  if (!is_q && rs.nq == 0) {       // no draft rows: neutral padding so that the merge below needs no special case
    send[3 * plane + at] = -CUDART_INF; send[4 * plane + at] = 0.0; send[5 * plane + at] = -CUDART_INF;
  }
  if (is_q && pos == k - 1) {      // pad the draft planes at position k
    const long long ak = (long long)b * (k + 1) + k;
    send[3 * plane + ak] = -CUDART_INF; send[4 * plane + ak] = 0.0; send[5 * plane + ak] = -CUDART_INF;
  }
}

// after exchange 1: one thread per sequence merges the ranks' statistics, runs the accept tests and fixes the row to
// sample.  Philox rows: sequence g of the gathered batch is request g % B_local of rank g / B_local, which draws
// with seed + (g / B_local) * seed_stride -- the numbers that rank's own single-GPU engine draws.
__global__ void shard_decide_kernel(const double* __restrict__ g1, int world, int Bt, int k, int has_q, int bonus,
                                    const long long* __restrict__ draft, int v_lo, uint64_t seed, uint64_t seed_stride,
                                    int B_local, uint32_t offset_host, const unsigned* __restrict__ offset_dev,
                                    Decision* __restrict__ dec, int* __restrict__ out_len,
                                    long long* __restrict__ out_tok) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= Bt) return;
  const uint32_t offset = offset_host + (offset_dev ? *offset_dev : 0u);
  const uint64_t sd = seed + (uint64_t)(b / B_local) * seed_stride;
  const uint32_t prow = (uint32_t)(b % B_local);
  const long long plane = (long long)Bt * (k + 1), rstride = 6 * plane;
  auto merged = [&](int f, int pos, double& M, double& S, double& X) {
    const long long at = (long long)b * (k + 1) + pos;
    M = -CUDART_INF; X = -CUDART_INF;
    for (int r = 0; r < world; ++r) {
      M = fmax(M, g1[r * rstride + (f + 0) * plane + at]);
      X = fmax(X, g1[r * rstride + (f + 2) * plane + at]);
    }
    S = 0.0;
    for (int r = 0; r < world; ++r) {
      const double mr = g1[r * rstride + (f + 0) * plane + at];
      if (mr != -CUDART_INF) S += g1[r * rstride + (f + 1) * plane + at] * exp(mr - M);
    }
  };
  Decision d;
  d.mode = 0; d.pos = 0; d.x = -1; d.m_p = d.m_q = 0.f; d.inv_sp = d.inv_sq = 0.0; d.u = 0.f;
  long long* tok = out_tok + (long long)b * (k + 1);
  for (int i = 0; i <= k; ++i) tok[i] = -1;
  int n = 0;
  for (; n < k; ++n) {
    double PM, PS, PX, QM = 0.0, QS = 1.0, QX = 0.0;
    merged(0, n, PM, PS, PX);
    const double p = PX == -CUDART_INF ? 0.0 : (double)expf((float)(PX - PM)) / PS;
    double q = 1.0;
    if (has_q) {
      merged(3, n, QM, QS, QX);
      q = QX == -CUDART_INF ? 0.0 : (double)expf((float)(QX - QM)) / QS;
    }
    const float u = philox_uniform(sd, offset, prow, n, 0);
    if ((double)u * q < p) { tok[n] = draft[(long long)b * k + n]; continue; }
    d.mode = has_q ? 1 : 3;
    d.pos = n;
    d.x = (int)(draft[(long long)b * k + n] - v_lo);      // column of this shard, or outside it
    d.m_p = (float)PM; d.inv_sp = 1.0 / PS;
    if (has_q) { d.m_q = (float)QM; d.inv_sq = 1.0 / QS; }
    break;
  }
  if (d.mode == 0 && bonus) {
    double PM, PS, PX;
    merged(0, k, PM, PS, PX);
    d.mode = 2; d.pos = k; d.m_p = (float)PM; d.inv_sp = 1.0 / PS;
  }
  if (d.mode) d.u = philox_uniform(sd, offset, prow, d.pos, 1);
  d.n_acc = n;
  out_len[b] = n;
  dec[b] = d;
}

// exchange 2, send side: the shard's residual mass and p mass of every sequence's sampled row
__global__ void shard_pack2_kernel(int Bt, int nchunks, const Decision* __restrict__ dec, const double* __restrict__ mass,
                                   double* __restrict__ send) {
  const int lane = threadIdx.x & 31;
  const int b = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (b >= Bt) return;
  double r = 0.0, p = 0.0;
  if (dec[b].mode) {
    // chunk order: lane-strided partial sums added in a fixed tree, the same on every rank for its own data
    for (int c = lane; c < nchunks; c += 32) { r += mass[((long long)b * nchunks + c) * 2]; p += mass[((long long)b * nchunks + c) * 2 + 1]; }
  }
  r = warp_sum(r); p = warp_sum(p);
  if (lane == 0) { send[b * 2] = r; send[b * 2 + 1] = p; }
}

// after exchange 2: which shard owns the sampled token; the owner gets the fraction of its own mass as its uniform
__global__ void shard_owner_kernel(const double* __restrict__ g2, int world, int rank, int Bt,
                                   const Decision* __restrict__ dec, Decision* __restrict__ dec_pick) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= Bt) return;
  Decision d = dec[b];
  const int mode_in = d.mode;
  d.mode = 0;
  if (mode_in) {
    double tot_r = 0.0;
    for (int r = 0; r < world; ++r) tot_r += g2[((long long)r * Bt + b) * 2];
    const int plain = !(tot_r > 0.0);                     // residual vanished everywhere: sample p itself
    double total = 0.0;
    for (int r = 0; r < world; ++r) total += g2[((long long)r * Bt + b) * 2 + plain];
    const double target0 = (double)d.u * total;
    double cum = 0.0, target = target0;
    int owner = -1, last_nz = -1;
    double before = 0.0;
    for (int r = 0; r < world; ++r) {
      const double w = g2[((long long)r * Bt + b) * 2 + plain];
      if (w > 0.0) last_nz = r;
      if (owner < 0 && cum + w > target0) { owner = r; before = cum; }
      cum += w;
    }
    if (owner < 0) {                                      // rounding pushed the target past the total
      owner = last_nz < 0 ? world - 1 : last_nz;
      before = 0.0;
      for (int r = 0; r < owner; ++r) before += g2[((long long)r * Bt + b) * 2 + plain];
      target = before + g2[((long long)owner * Bt + b) * 2 + plain];
    }
    if (owner == rank) {
      const double mine = g2[((long long)owner * Bt + b) * 2 + plain];
      double frac = mine > 0.0 ? (target - before) / mine : 0.0;
      frac = frac < 0.0 ? 0.0 : (frac > 1.0 ? 1.0 : frac);
      d.mode = plain ? 2 : mode_in;
      d.u = (float)frac;
    }
  }
  dec_pick[b] = d;
}

// exchange 3, send side: the global id of the token this shard picked, or -1
__global__ void shard_pack3_kernel(int Bt, int k, int v_lo, const Decision* __restrict__ dec_pick,
                                   const long long* __restrict__ picked, long long* __restrict__ send) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= Bt) return;
  const Decision d = dec_pick[b];
  send[b] = d.mode ? picked[(long long)b * (k + 1) + d.n_acc] + v_lo : -1;
}

__global__ void shard_finish_kernel(const long long* __restrict__ g3, int world, int Bt, int k,
                                    const Decision* __restrict__ dec, long long* __restrict__ out_tok) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= Bt || dec[b].mode == 0) return;
  long long t = -1;
  for (int r = 0; r < world; ++r) t = max(t, g3[(long long)r * Bt + b]);
  out_tok[(long long)b * (k + 1) + dec[b].pos] = t;
}

}  // namespace

// lists_out (top-k path only): the kept lists of the p rows are left there ([B][np] records) for a later call
int32_t vn_accept_impl(vn_ctx* ctx, const float* p, long long p_sb, long long p_si,
                           const float* q, long long q_sb, long long q_si, const int64_t* draft,
                           const float* u_acc, const float* u_smp, uint64_t seed, uint32_t offset,
                           float temperature, int32_t top_k, int32_t bonus, int32_t B, int32_t k, int32_t V,
                           int32_t* out_len, int64_t* out_tok, int32_t smp_purpose, int32_t pos_base,
                           void* lists_out) {
  VN_CHECK_CTX(ctx);
  VN_REQUIRE(ctx, B >= 0 && k >= 0 && k <= MAX_K && V >= 1, "bad sizes B=%d k=%d V=%d (k <= %d)", B, k, V, MAX_K);
  VN_REQUIRE(ctx, p && out_tok, "null pointer");
  VN_REQUIRE(ctx, k == 0 || draft, "draft tokens missing");
  VN_REQUIRE(ctx, (u_acc == nullptr) == (u_smp == nullptr) || k == 0, "inject both uniform arrays or neither");
  VN_REQUIRE(ctx, bonus || k > 0, "nothing to do: k == 0 without a bonus token");
  if (B == 0) return VN_OK;
  const bool greedy = temperature <= 0.f;
  const float temp = greedy ? 1.0f : fmaxf(temperature, 1e-8f);
  RowSet rs;
  rs.p = p; rs.q = greedy ? nullptr : q;
  rs.p_sb = p_sb; rs.p_si = p_si; rs.q_sb = q_sb; rs.q_si = q_si;
  rs.np = bonus ? k + 1 : k;
  rs.nq = (rs.q && k > 0) ? k : 0;
  rs.V = V;
  const int rows_per_seq = rs.np + rs.nq;
  const long long* d64 = reinterpret_cast<const long long*>(draft);
  long long* o64 = reinterpret_cast<long long*>(out_tok);

  if (!greedy && top_k > 0 && top_k < V) {
    VN_REQUIRE(ctx, top_k <= KEEP_MAX, "top_k %d above the supported maximum %d", top_k, KEEP_MAX);
    // slices per row: a little under one CTA per SM (measured on B200 for the draft's 32 rows: 4 slices per row
    // 2.325 ms per round, 3 slices 2.326, 5 slices 2.335, 2 slices 2.335, 10 slices 2.42: fewer, longer slices and
    // a smaller merge win), at least 8192 logits each
    const int n_rows = B * rows_per_seq;
    static const double topk_ctas_per_sm = [] { const char* e = getenv("VN_TOPK_CTAS_PER_SM"); return e ? std::max(0.05, atof(e)) : 0.75; }();
    const int cta_target = std::max(1, (int)(topk_ctas_per_sm * ctx->sm_count + 0.5));
    int chunks = std::min(std::min(16, std::max(1, V / 8192)), std::max(1, ceil_div(cta_target, n_rows)));
    chunks = std::max(1, std::min(chunks, 2048 / std::max(top_k, 1)));
    void* ws;
    int32_t st = vn_workspace(ctx, sizeof(TopkRow) * (size_t)n_rows * (chunks + 1), &ws);
    if (st) return st;
    TopkRow* rows = (TopkRow*)ws;                 // merged lists [B][rows_per_seq]
    TopkRow* parts = rows + n_rows;               // per-slice lists [n_rows * chunks]
    long long out_sb = rows_per_seq;
    if (lists_out) {
      VN_REQUIRE(ctx, rs.nq == 0, "kept lists can only be handed out for calls without draft rows");
      rows = (TopkRow*)lists_out;
      out_sb = rs.np;
    }
    DecideArgs da;
    da.B = B; da.k = k; da.np = rs.np; da.nq = rs.nq; da.draft = d64; da.u_acc = u_acc; da.u_smp = u_smp;
    da.seed = seed; da.offset_host = offset; da.offset_dev = ctx->offset_src; da.bonus = bonus;
    da.smp_purpose = smp_purpose; da.pos_base = pos_base; da.out_len = out_len; da.out_tok = o64;
    da.p_rows = rows; da.p_sb = out_sb; da.q_rows = rows + rs.np; da.q_sb = out_sb; da.q_si = 1;
    if (chunks > 1) {
      VN_LAUNCH_PDL_BIT(ctx, 64, accept_topk_kernel, n_rows * chunks, 1024, 0, rs, top_k, temp, chunks, parts,
                        (long long)rows_per_seq, (const int*)nullptr);
      VN_LAUNCH_PDL_BIT(ctx, 128, accept_topk_merge_kernel, n_rows, 1024, 0, parts, chunks, top_k, rows, rows_per_seq, out_sb,
                        (const int*)nullptr);
    } else {
      VN_LAUNCH_PDL_BIT(ctx, 64, accept_topk_kernel, n_rows, 1024, 0, rs, top_k, temp, 1, rows, out_sb, (const int*)nullptr);
    }
    VN_LAUNCH_PDL_BIT(ctx, 256, accept_topk_decide_kernel, ceil_div(B, 4), 128, 0, da);
    return VN_OK;
  }

  const int nchunks = ceil_div(V, CHUNK);
  const size_t n_part = (size_t)B * rows_per_seq * nchunks;
  const size_t off_dec = (n_part * sizeof(Partial) + 255) & ~(size_t)255;
  const size_t off_mass = (off_dec + (size_t)B * sizeof(Decision) + 255) & ~(size_t)255;
  const size_t total = off_mass + (size_t)B * nchunks * 2 * sizeof(double);
  void* ws;
  int32_t st = vn_workspace(ctx, total, &ws);
  if (st) return st;
  Partial* part = (Partial*)ws;
  Decision* dec = (Decision*)((char*)ws + off_dec);
  double* mass = (double*)((char*)ws + off_mass);

  auto aligned16 = [](const void* ptr) { return ((uintptr_t)ptr & 15) == 0; };
  const bool vec = (V % 4 == 0) && aligned16(p) && (p_sb % 4 == 0) && (p_si % 4 == 0) &&
                   (!rs.nq || (aligned16(q) && (q_sb % 4 == 0) && (q_si % 4 == 0)));
  const long long nitems = (long long)n_part;
  const int grid = (int)std::min<long long>(nitems, (long long)ctx->sm_count * 8);
  { const int32_t st_ = launch_accept_stats(ctx, vec, greedy, grid, rs, B, nchunks, temp, part); if (st_) return st_; }
  VN_LAUNCH(ctx, accept_decide_kernel, B, decide_threads(rows_per_seq), 0, rs, B, k, nchunks, part, d64, u_acc, u_smp, seed, offset,
            ctx->offset_src, temp, (int)greedy, bonus, smp_purpose, pos_base, dec, out_len, o64);
  if (!greedy) {
    dim3 g(nchunks, B);
    if (vec) VN_LAUNCH(ctx, accept_residual_kernel<true>, g, STATS_THREADS, 0, rs, nchunks, temp, dec, mass);
    else     VN_LAUNCH(ctx, accept_residual_kernel<false>, g, STATS_THREADS, 0, rs, nchunks, temp, dec, mass);
    VN_LAUNCH(ctx, accept_pick_kernel, B, STATS_THREADS, 0, rs, k, nchunks, temp, dec, mass, o64);
  }
  return VN_OK;
}

// ---- row-level pieces for a vocabulary split across GPUs ----------------------------------------------------
// The same kernels as above, driven row by row with the softmax statistics supplied from outside: a rank that
// holds a slice of the vocabulary computes the slice's statistics and residual mass, the ranks merge those few
// numbers, and the rank that owns the sampled token picks it.

// one warp per row: merge the chunk records of a row, read the logit of `tokens[row]` (a column of this block)
__global__ void row_stats_reduce_kernel(RowSet rs, int R, int nchunks, const Partial* __restrict__ part, float temp,
                                        const long long* __restrict__ tokens, float* __restrict__ out_m,
                                        double* __restrict__ out_s, float* __restrict__ out_x) {
  const int lane = threadIdx.x & 31;
  const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= R) return;
  const Partial* pp = part + (long long)r * nchunks;
  float m = -CUDART_INF_F;
  for (int c = lane; c < nchunks; c += 32) m = fmaxf(m, pp[c].m);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  double s = 0.0;
  for (int c = lane; c < nchunks; c += 32) {
    const Partial p = pp[c];
    if (p.m != -CUDART_INF_F) s += p.s * exp((double)(p.m - m));
  }
  s = warp_sum(s);
  if (lane == 0) {
    out_m[r] = m;
    out_s[r] = s;
    if (out_x) {
      const long long t = tokens ? tokens[r] : -1;
      out_x[r] = (t >= 0 && t < rs.V) ? scaled(row_ptr(rs, r, 0)[t], temp) : -CUDART_INF_F;
    }
  }
}

// decisions from outside: mode 1 residual of (p, q), 2 plain p, 3 p without `removed`, 0 nothing
__global__ void row_decision_kernel(int R, const int* __restrict__ mode, const float* __restrict__ m_p,
                                    const double* __restrict__ s_p, const float* __restrict__ m_q,
                                    const double* __restrict__ s_q, const long long* __restrict__ removed,
                                    const float* __restrict__ u, Decision* __restrict__ dec) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= R) return;
  Decision d;
  d.n_acc = 0; d.mode = mode[r]; d.pos = 0;
  d.x = removed ? (int)removed[r] : -1;
  d.m_p = m_p[r]; d.inv_sp = 1.0 / s_p[r];
  d.m_q = m_q ? m_q[r] : 0.f; d.inv_sq = s_q ? 1.0 / s_q[r] : 0.0;
  d.u = u ? u[r] : 0.f;
  dec[r] = d;
}

__global__ void row_mass_reduce_kernel(int R, int nchunks, const int* __restrict__ mode, const double* __restrict__ mass,
                                       double* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= R) return;
  double a = 0.0, b = 0.0;
  if (mode[r] != 0)
    for (int c = lane; c < nchunks; c += 32) { a += mass[((long long)r * nchunks + c) * 2]; b += mass[((long long)r * nchunks + c) * 2 + 1]; }
  a = warp_sum(a); b = warp_sum(b);
  if (lane == 0) { out[r * 2] = a; out[r * 2 + 1] = b; }
}

static int32_t row_set(vn_ctx* ctx, const float* p, long long p_stride, const float* q, long long q_stride, int R, int V,
                       RowSet* rs, bool* vec) {
  VN_REQUIRE(ctx, R >= 0 && V >= 1 && p, "bad sizes R=%d V=%d", R, V);
  rs->p = p; rs->q = q; rs->p_sb = p_stride; rs->p_si = 0; rs->q_sb = q_stride; rs->q_si = 0;
  rs->np = 1; rs->nq = q ? 1 : 0; rs->V = V;
  auto aligned16 = [](const void* ptr) { return ((uintptr_t)ptr & 15) == 0; };
  *vec = (V % 4 == 0) && aligned16(p) && (p_stride % 4 == 0) && (!q || (aligned16(q) && q_stride % 4 == 0));
  return VN_OK;
}

// residual chunk masses of R rows into the workspace; returns the pointers
static int32_t row_residual_chunks(vn_ctx* ctx, const RowSet& rs, bool vec, int R, float temp, const int* mode,
                                   const float* m_p, const double* s_p, const float* m_q, const double* s_q,
                                   const long long* removed, const float* u, Decision** dec_out, double** mass_out) {
  const int nchunks = ceil_div(rs.V, CHUNK);
  const size_t off_mass = ((size_t)R * sizeof(Decision) + 255) & ~(size_t)255;
  void* ws;
  int32_t st = vn_workspace(ctx, off_mass + (size_t)R * nchunks * 2 * sizeof(double), &ws);
  if (st) return st;
  Decision* dec = (Decision*)ws;
  double* mass = (double*)((char*)ws + off_mass);
  VN_LAUNCH(ctx, row_decision_kernel, ceil_div(R, 128), 128, 0, R, mode, m_p, s_p, m_q, s_q, removed, u, dec);
  dim3 g(nchunks, R);
  if (vec) VN_LAUNCH(ctx, accept_residual_kernel<true>, g, STATS_THREADS, 0, rs, nchunks, temp, dec, mass);
  else     VN_LAUNCH(ctx, accept_residual_kernel<false>, g, STATS_THREADS, 0, rs, nchunks, temp, dec, mass);
  *dec_out = dec; *mass_out = mass;
  return VN_OK;
}

struct vn_comm;
int32_t vn_comm_gather(vn_ctx* ctx, vn_comm* c, const void* send_dev, void* recv_dev, size_t bytes_per_rank, int* world,
                       int* rank);

extern "C" int32_t vn_shard_accept(vn_ctx* ctx, vn_comm* comm, const float* p_dev, const float* q_dev,
                                   const int64_t* draft_dev, int32_t v_lo, int32_t Vs, float temperature, uint64_t seed,
                                   uint64_t seed_stride, uint32_t offset, int32_t B_local, int32_t Bt, int32_t k,
                                   int32_t bonus, int32_t* out_len_dev, int64_t* out_tokens_dev) {
  VN_CHECK_CTX(ctx);
  VN_REQUIRE(ctx, p_dev && draft_dev && out_len_dev && out_tokens_dev, "null argument");
  VN_REQUIRE(ctx, temperature > 0.f, "the sharded rule is the stochastic one (temperature > 0)");
  VN_REQUIRE(ctx, Bt >= 1 && k >= 1 && k <= MAX_K && Vs >= 0 && B_local >= 1 && Bt % B_local == 0, "bad sizes");
  int world = 1, rank = 0;
  vn_comm_gather(ctx, comm, nullptr, nullptr, 0, &world, &rank);
  VN_REQUIRE(ctx, Bt == world * B_local, "Bt (%d) must be world (%d) x B_local (%d)", Bt, world, B_local);
  const float temp = fmaxf(temperature, 1e-8f);
  const int np = bonus ? k + 1 : k;
  VN_REQUIRE(ctx, bonus, "the sharded round always scores k + 1 positions");
  RowSet rs;
  rs.p = p_dev; rs.q = q_dev; rs.np = np; rs.nq = q_dev ? k : 0;
  rs.p_sb = (long long)np * Vs; rs.p_si = Vs; rs.q_sb = (long long)k * Vs; rs.q_si = Vs; rs.V = Vs;
  const int rows_per_seq = rs.np + rs.nq;
  const int nchunks = std::max(1, ceil_div(Vs, CHUNK));
  auto up = [](size_t v) { return (v + 255) & ~(size_t)255; };
  const size_t n_part = (size_t)Bt * rows_per_seq * nchunks;
  const size_t plane1 = (size_t)6 * Bt * (k + 1) * sizeof(double);
  const size_t o_part = 0;
  const size_t o_s1 = up(o_part + n_part * sizeof(Partial));
  const size_t o_g1 = up(o_s1 + plane1);
  const size_t o_dec = up(o_g1 + plane1 * world);
  const size_t o_dec2 = up(o_dec + (size_t)Bt * sizeof(Decision));
  const size_t o_mass = up(o_dec2 + (size_t)Bt * sizeof(Decision));
  const size_t o_s2 = up(o_mass + (size_t)Bt * nchunks * 2 * sizeof(double));
  const size_t o_g2 = up(o_s2 + (size_t)Bt * 2 * sizeof(double));
  const size_t o_pick = up(o_g2 + (size_t)Bt * 2 * sizeof(double) * world);
  const size_t o_s3 = up(o_pick + (size_t)Bt * (k + 1) * sizeof(long long));
  const size_t o_g3 = up(o_s3 + (size_t)Bt * sizeof(long long));
  const size_t total = o_g3 + (size_t)Bt * sizeof(long long) * world;
  void* ws;
  int32_t st = vn_workspace(ctx, total, &ws);
  if (st) return st;
  char* base = (char*)ws;
  Partial* part = (Partial*)(base + o_part);
  double* s1 = (double*)(base + o_s1); double* g1 = (double*)(base + o_g1);
  Decision* dec = (Decision*)(base + o_dec); Decision* dec2 = (Decision*)(base + o_dec2);
  double* mass = (double*)(base + o_mass);
  double* s2 = (double*)(base + o_s2); double* g2 = (double*)(base + o_g2);
  long long* picked = (long long*)(base + o_pick);
  long long* s3 = (long long*)(base + o_s3); long long* g3 = (long long*)(base + o_g3);
  const long long* d64 = reinterpret_cast<const long long*>(draft_dev);
  long long* o64 = reinterpret_cast<long long*>(out_tokens_dev);
  auto aligned16 = [](const void* ptr) { return ((uintptr_t)ptr & 15) == 0; };
  const bool vec = (Vs % 4 == 0) && aligned16(rs.p) && (!rs.nq || aligned16(rs.q));
  // ---- exchange 1
  if (Vs > 0) {
    const int grid = (int)std::min<long long>((long long)Bt * rows_per_seq * ((nchunks + 1) / 2), (long long)ctx->sm_count * 8);
    st = launch_accept_stats(ctx, vec, false, grid, rs, Bt, nchunks, temp, part);
    if (st) return st;
  } else {
    VN_CUDA(ctx, cudaMemsetAsync(part, 0xff, n_part * sizeof(Partial), ctx->stream));   // unreachable in practice
  }
  VN_LAUNCH(ctx, shard_pack1_kernel, ceil_div(Bt * rows_per_seq, 4), 128, 0, rs, Bt, k, nchunks, (const Partial*)part, temp, d64,
            v_lo, s1);
  st = vn_comm_gather(ctx, comm, s1, g1, plane1, nullptr, nullptr);
  if (st) return st;
  VN_LAUNCH(ctx, shard_decide_kernel, ceil_div(Bt, 128), 128, 0, (const double*)g1, world, Bt, k, rs.nq ? 1 : 0, bonus, d64,
            v_lo, seed, seed_stride, B_local, offset, ctx->offset_src, dec, out_len_dev, o64);
  // ---- exchange 2
  {
    dim3 g(nchunks, Bt);
    if (vec) VN_LAUNCH(ctx, accept_residual_kernel<true>, g, STATS_THREADS, 0, rs, nchunks, temp, (const Decision*)dec, mass);
    else     VN_LAUNCH(ctx, accept_residual_kernel<false>, g, STATS_THREADS, 0, rs, nchunks, temp, (const Decision*)dec, mass);
  }
  VN_LAUNCH(ctx, shard_pack2_kernel, ceil_div(Bt, 4), 128, 0, Bt, nchunks, (const Decision*)dec, (const double*)mass, s2);
  st = vn_comm_gather(ctx, comm, s2, g2, (size_t)Bt * 2 * sizeof(double), nullptr, nullptr);
  if (st) return st;
  VN_LAUNCH(ctx, shard_owner_kernel, ceil_div(Bt, 128), 128, 0, (const double*)g2, world, rank, Bt, (const Decision*)dec, dec2);
  // ---- exchange 3
  VN_LAUNCH(ctx, accept_pick_kernel, Bt, STATS_THREADS, 0, rs, k, nchunks, temp, (const Decision*)dec2, (const double*)mass, picked);
  VN_LAUNCH(ctx, shard_pack3_kernel, ceil_div(Bt, 128), 128, 0, Bt, k, v_lo, (const Decision*)dec2, (const long long*)picked, s3);
  st = vn_comm_gather(ctx, comm, s3, g3, (size_t)Bt * sizeof(long long), nullptr, nullptr);
  if (st) return st;
  VN_LAUNCH(ctx, shard_finish_kernel, ceil_div(Bt, 128), 128, 0, (const long long*)g3, world, Bt, k, (const Decision*)dec, o64);
  return VN_OK;
}

size_t vn_topk_row_bytes_impl() { return sizeof(TopkRow); }

int32_t vn_k1_layout(vn_ctx* ctx, int B, int np, int top_k, int V, vn_k1* out) {
  static const int boot_cols = [] { const char* e = getenv("VN_K1_BOOT"); return e ? std::max(256, std::min(8192, atoi(e))) : 8192; }();
  vn_k1 k;
  k.rows = B * np;
  k.cap = VN_K1_CAP;
  k.nb = std::min(V, boot_cols) & ~127;          // whole 128-column tiles of the head
  if (k.nb < 128) k.nb = std::min(V, 128);
  static const double topk_ctas_per_sm = [] { const char* e = getenv("VN_TOPK_CTAS_PER_SM"); return e ? std::max(0.05, atof(e)) : 0.75; }();
  const int cta_target = std::max(1, (int)(topk_ctas_per_sm * ctx->sm_count + 0.5));
  int chunks = std::min(std::min(16, std::max(1, V / 8192)), std::max(1, ceil_div(cta_target, std::max(k.rows, 1))));
  k.chunks = std::max(1, std::min(chunks, 2048 / std::max(top_k, 1)));
  auto up = [](size_t v) { return (v + 255) & ~(size_t)255; };
  const size_t o_boot = 0;
  const size_t o_tau = up(o_boot + (size_t)k.rows * k.nb * 4);
  const size_t o_cnt = up(o_tau + (size_t)k.rows * 4);
  k.count_stride = 32;                           // one 128-byte line per row's counter: the epilogue's atomics spread over L2
  const size_t o_flag = up(o_cnt + (size_t)k.rows * k.count_stride * 4);
  const size_t o_val = up(o_flag + 256);
  const size_t o_tok = up(o_val + (size_t)k.rows * k.cap * 4);
  const size_t o_lists = up(o_tok + (size_t)k.rows * k.cap * 4);
  const size_t o_parts = up(o_lists + (size_t)k.rows * sizeof(TopkRow));
  const size_t total = o_parts + (size_t)k.rows * k.chunks * sizeof(TopkRow);
  void* ws;
  int32_t st = vn_workspace(ctx, total, &ws);
  if (st) return st;
  char* base = (char*)ws;
  k.boot = (float*)(base + o_boot); k.tau = (float*)(base + o_tau); k.count = (int*)(base + o_cnt);
  k.fallback = (int*)(base + o_flag); k.cand_val = (float*)(base + o_val); k.cand_tok = (int*)(base + o_tok);
  k.p_lists = base + o_lists; k.parts = base + o_parts;
  *out = k;
  return VN_OK;
}

int32_t vn_k1_bound(vn_ctx* ctx, const vn_k1& k1, int top_k, float temp) {
  VN_REQUIRE(ctx, top_k >= 1, "top_k must be positive");
  // 256 threads: the k-th largest of 256 group maxima costs 256 x 256 comparisons, four times that many threads
  // would cost sixteen times as many for a bound that is hardly tighter
  VN_LAUNCH_PDL(ctx, k1_bound_kernel, k1.rows, 256, 0, (const float*)k1.boot, k1.nb, top_k, temp, k1.tau, k1.count,
                k1.count_stride, k1.fallback);
  return VN_OK;
}

int32_t vn_k1_accept(vn_ctx* ctx, const vn_k1& k1, const float* p_fallback, long long p_sb, long long p_si,
                     const void* q_lists, long long ql_sb, long long ql_si, const float* q_logits, long long q_sb,
                     long long q_si, const int64_t* draft, const float* u_acc, const float* u_smp, uint64_t seed,
                     uint32_t offset, float temperature, int32_t top_k, int32_t bonus, int32_t B, int32_t k, int32_t V,
                     int32_t* out_len, int64_t* out_tok) {
  VN_REQUIRE(ctx, temperature > 0.f && top_k >= 1 && top_k <= KEEP_MAX && top_k < V, "the fused head needs temperature > 0 and 0 < top_k < V");
  VN_REQUIRE(ctx, k >= 0 && k <= MAX_K && B >= 1 && out_tok, "bad arguments");
  const float temp = fmaxf(temperature, 1e-8f);
  const int np = bonus ? k + 1 : k;
  VN_REQUIRE(ctx, k1.rows == B * np, "candidate buffers were laid out for another shape");
  TopkRow* p_rows = (TopkRow*)k1.p_lists;
  VN_LAUNCH_PDL(ctx, k1_finish_kernel, k1.rows, K1_FIN_THREADS, 0, (const float*)k1.cand_val, (const int*)k1.cand_tok,
                (const int*)k1.count, k1.count_stride, k1.cap, top_k, temp, V, p_rows, k1.fallback);
  if (p_fallback) {
    // classic select on the stored logits, only when the flag is up (its kernels return at once otherwise)
    RowSet rs;
    rs.p = p_fallback; rs.q = nullptr; rs.p_sb = p_sb; rs.p_si = p_si; rs.q_sb = 0; rs.q_si = 0; rs.np = np; rs.nq = 0; rs.V = V;
    if (k1.chunks > 1) {
      VN_LAUNCH_PDL(ctx, accept_topk_kernel, k1.rows * k1.chunks, 1024, 0, rs, top_k, temp, k1.chunks, (TopkRow*)k1.parts,
                    (long long)np, (const int*)k1.fallback);
      VN_LAUNCH_PDL(ctx, accept_topk_merge_kernel, k1.rows, 1024, 0, (const TopkRow*)k1.parts, k1.chunks, top_k, p_rows, np,
                    (long long)np, (const int*)k1.fallback);
    } else {
      VN_LAUNCH_PDL(ctx, accept_topk_kernel, k1.rows, 1024, 0, rs, top_k, temp, 1, p_rows, (long long)np, (const int*)k1.fallback);
    }
  }
  DecideArgs da;
  da.B = B; da.k = k; da.np = np; da.nq = 0; da.draft = reinterpret_cast<const long long*>(draft);
  da.u_acc = u_acc; da.u_smp = u_smp; da.seed = seed; da.offset_host = offset; da.offset_dev = ctx->offset_src;
  da.bonus = bonus; da.smp_purpose = 1; da.pos_base = 0; da.out_len = out_len;
  da.out_tok = reinterpret_cast<long long*>(out_tok);
  da.p_rows = p_rows; da.p_sb = np; da.q_rows = nullptr; da.q_sb = 0; da.q_si = 0;
  if (k > 0 && q_lists) {
    da.nq = k; da.q_rows = (const TopkRow*)q_lists; da.q_sb = ql_sb; da.q_si = ql_si;
  } else if (k > 0 && q_logits) {
    // the draft rows' lists are selected here from their logits, into the slice-list region: the classic select of
    // the target rows (when it runs at all) has finished with that region by then (stream order)
    VN_REQUIRE(ctx, (size_t)B * k <= (size_t)k1.rows * k1.chunks, "no room for the draft rows' lists");
    TopkRow* q_rows = (TopkRow*)k1.parts;
    RowSet rs;
    rs.p = q_logits; rs.q = nullptr; rs.p_sb = q_sb; rs.p_si = q_si; rs.q_sb = 0; rs.q_si = 0; rs.np = k; rs.nq = 0; rs.V = V;
    VN_LAUNCH_PDL(ctx, accept_topk_kernel, B * k, 1024, 0, rs, top_k, temp, 1, q_rows, (long long)k, (const int*)nullptr);
    da.nq = k; da.q_rows = q_rows; da.q_sb = k; da.q_si = 1;
  }
  VN_LAUNCH_PDL_BIT(ctx, 256, accept_topk_decide_kernel, ceil_div(B, 4), 128, 0, da);
  return VN_OK;
}

extern "C" {

int32_t vn_row_stats(vn_ctx* ctx, const float* logits_dev, int64_t row_stride, int32_t R, int32_t V, float temperature,
                     const int64_t* tokens_dev, float* out_max_dev, double* out_sum_dev, float* out_logit_dev) {
  VN_CHECK_CTX(ctx);
  VN_REQUIRE(ctx, temperature > 0.f && out_max_dev && out_sum_dev, "temperature must be positive, outputs non-null");
  if (R == 0) return VN_OK;
  RowSet rs; bool vec;
  int32_t st = row_set(ctx, logits_dev, row_stride, nullptr, 0, R, V, &rs, &vec);
  if (st) return st;
  const float temp = fmaxf(temperature, 1e-8f);
  const int nchunks = ceil_div(V, CHUNK);
  void* ws;
  st = vn_workspace(ctx, (size_t)R * nchunks * sizeof(Partial), &ws);
  if (st) return st;
  Partial* part = (Partial*)ws;
  const int grid = (int)std::min<long long>((long long)R * ((nchunks + 1) / 2), (long long)ctx->sm_count * 8);
  st = launch_accept_stats(ctx, vec, false, grid, rs, R, nchunks, temp, part);
  if (st) return st;
  VN_LAUNCH(ctx, row_stats_reduce_kernel, ceil_div(R, 4), 128, 0, rs, R, nchunks, part, temp,
            reinterpret_cast<const long long*>(tokens_dev), out_max_dev, out_sum_dev, out_logit_dev);
  return VN_OK;
}

int32_t vn_row_residual(vn_ctx* ctx, const float* p_dev, int64_t p_stride, const float* q_dev, int64_t q_stride, int32_t R,
                        int32_t V, float temperature, const int32_t* mode_dev, const float* m_p_dev, const double* s_p_dev,
                        const float* m_q_dev, const double* s_q_dev, const int64_t* removed_dev, double* out_mass_dev) {
  VN_CHECK_CTX(ctx);
  VN_REQUIRE(ctx, temperature > 0.f && mode_dev && m_p_dev && s_p_dev && out_mass_dev, "null argument");
  VN_REQUIRE(ctx, !q_dev || (m_q_dev && s_q_dev), "draft statistics missing");
  if (R == 0) return VN_OK;
  RowSet rs; bool vec;
  int32_t st = row_set(ctx, p_dev, p_stride, q_dev, q_stride, R, V, &rs, &vec);
  if (st) return st;
  Decision* dec; double* mass;
  st = row_residual_chunks(ctx, rs, vec, R, fmaxf(temperature, 1e-8f), mode_dev, m_p_dev, s_p_dev, m_q_dev, s_q_dev,
                           reinterpret_cast<const long long*>(removed_dev), nullptr, &dec, &mass);
  if (st) return st;
  VN_LAUNCH(ctx, row_mass_reduce_kernel, ceil_div(R, 4), 128, 0, R, ceil_div(V, CHUNK), mode_dev, mass, out_mass_dev);
  return VN_OK;
}

int32_t vn_row_pick(vn_ctx* ctx, const float* p_dev, int64_t p_stride, const float* q_dev, int64_t q_stride, int32_t R,
                    int32_t V, float temperature, const int32_t* mode_dev, const float* m_p_dev, const double* s_p_dev,
                    const float* m_q_dev, const double* s_q_dev, const int64_t* removed_dev, const float* u_dev,
                    int64_t* out_token_dev) {
  VN_CHECK_CTX(ctx);
  VN_REQUIRE(ctx, temperature > 0.f && mode_dev && m_p_dev && s_p_dev && u_dev && out_token_dev, "null argument");
  VN_REQUIRE(ctx, !q_dev || (m_q_dev && s_q_dev), "draft statistics missing");
  if (R == 0) return VN_OK;
  RowSet rs; bool vec;
  int32_t st = row_set(ctx, p_dev, p_stride, q_dev, q_stride, R, V, &rs, &vec);
  if (st) return st;
  const float temp = fmaxf(temperature, 1e-8f);
  Decision* dec; double* mass;
  st = row_residual_chunks(ctx, rs, vec, R, temp, mode_dev, m_p_dev, s_p_dev, m_q_dev, s_q_dev,
                           reinterpret_cast<const long long*>(removed_dev), u_dev, &dec, &mass);
  if (st) return st;
  VN_LAUNCH(ctx, accept_pick_kernel, R, STATS_THREADS, 0, rs, 0, ceil_div(V, CHUNK), temp, dec, mass,
            reinterpret_cast<long long*>(out_token_dev));
  return VN_OK;
}

int32_t vn_accept(vn_ctx* ctx, const float* p_logits_dev, const float* q_logits_dev, const int64_t* draft_dev,
                  const float* u_accept_dev, const float* u_sample_dev, uint64_t seed, uint32_t offset,
                  float temperature, int32_t top_k, int32_t bonus, int32_t B, int32_t k, int32_t V,
                  int32_t* out_len_dev, int64_t* out_tokens_dev) {
  const long long np = bonus ? k + 1 : k;
  return vn_accept_impl(ctx, p_logits_dev, np * V, V, q_logits_dev, (long long)k * V, V, draft_dev, u_accept_dev,
                        u_sample_dev, seed, offset, temperature, top_k, bonus, B, k, V, out_len_dev, out_tokens_dev, 1, 0, nullptr);
}

int32_t vn_accept_strided(vn_ctx* ctx, const float* p_logits_dev, int64_t p_stride_b, int64_t p_stride_i,
                          const float* q_logits_dev, int64_t q_stride_b, int64_t q_stride_i,
                          const int64_t* draft_dev, const float* u_accept_dev, const float* u_sample_dev,
                          uint64_t seed, uint32_t offset, float temperature, int32_t top_k, int32_t bonus,
                          int32_t B, int32_t k, int32_t V, int32_t* out_len_dev, int64_t* out_tokens_dev) {
  return vn_accept_impl(ctx, p_logits_dev, p_stride_b, p_stride_i, q_logits_dev, q_stride_b, q_stride_i, draft_dev,
                        u_accept_dev, u_sample_dev, seed, offset, temperature, top_k, bonus, B, k, V, out_len_dev,
                        out_tokens_dev, 1, 0, nullptr);
}

int32_t vn_sample(vn_ctx* ctx, const float* logits_dev, int64_t row_stride, int32_t R, int32_t V, float temperature,
                  int32_t top_k, const float* uniforms_dev, uint64_t seed, uint32_t offset, uint32_t position,
                  uint32_t purpose, int64_t* out_tokens_dev) {
  VN_CHECK_CTX(ctx);
  VN_REQUIRE(ctx, R >= 0 && out_tokens_dev, "bad arguments");
  if (R == 0) return VN_OK;
  int32_t st = vn_accept_impl(ctx, logits_dev, row_stride, 0, nullptr, 0, 0, nullptr, uniforms_dev, uniforms_dev, seed,
                              offset, temperature, top_k, 1, R, 0, V, nullptr, out_tokens_dev, (int32_t)purpose,
                              (int32_t)position, nullptr);
  return st;
}

int32_t vn_sample_lists(vn_ctx* ctx, const float* logits_dev, int64_t row_stride, int32_t R, int32_t V, float temperature,
                        int32_t top_k, const float* uniforms_dev, uint64_t seed, uint32_t offset, uint32_t position,
                        uint32_t purpose, int64_t* out_tokens_dev, void* lists_out_dev) {
  VN_CHECK_CTX(ctx);
  VN_REQUIRE(ctx, R >= 0 && out_tokens_dev, "bad arguments");
  VN_REQUIRE(ctx, !lists_out_dev || (temperature > 0.f && top_k > 0 && top_k < V),
             "kept lists exist on the top-k path only (temperature > 0, 0 < top_k < V)");
  if (R == 0) return VN_OK;
  return vn_accept_impl(ctx, logits_dev, row_stride, 0, nullptr, 0, 0, nullptr, uniforms_dev, uniforms_dev, seed, offset,
                        temperature, top_k, 1, R, 0, V, nullptr, out_tokens_dev, (int32_t)purpose, (int32_t)position,
                        lists_out_dev);
}

size_t vn_topk_row_bytes(void) { return vn_topk_row_bytes_impl(); }

int32_t vn_tree_accept_sample(vn_ctx* ctx, const void* lists_dev, const int64_t* tokens_dev, const int32_t* parent_dev,
                              int32_t B, int32_t T, int32_t depth, const float* u_child_dev, const float* u_sample_dev,
                              uint64_t seed, uint32_t offset, int32_t* out_len_dev, int64_t* out_tokens_dev,
                              int32_t* keep_target_dev, int32_t* keep_draft_dev) {
  VN_CHECK_CTX(ctx);
  VN_REQUIRE(ctx, lists_dev && tokens_dev && parent_dev && out_tokens_dev && keep_target_dev && keep_draft_dev && B >= 1 &&
             T >= 1 && T <= 64 && depth >= 1 && depth < T, "vn_tree_accept_sample: bad arguments");
  VN_REQUIRE(ctx, (u_child_dev == nullptr) == (u_sample_dev == nullptr), "inject both uniform arrays or neither");
  TreeSampleArgs ta;
  ta.rows = (const TopkRow*)lists_dev; ta.tokens = (const long long*)tokens_dev; ta.parent = parent_dev;
  ta.u_child = u_child_dev; ta.u_sample = u_sample_dev; ta.seed = seed; ta.offset_host = offset; ta.offset_dev = ctx->offset_src;
  ta.B = B; ta.T = T; ta.depth = depth; ta.out_len = out_len_dev; ta.out_tok = (long long*)out_tokens_dev;
  ta.keep_t = keep_target_dev; ta.keep_d = keep_draft_dev;
  VN_LAUNCH_PDL(ctx, tree_accept_sample_kernel, ceil_div(B, 4), 128, 0, ta);
  return VN_OK;
}

}  // extern "C"

// ---- acceptance without any allocation ---------------------------------------------------------------
// Scratch of the full-vocabulary path (chunk statistics, per-sequence decisions, residual masses) held in a
// fixed array inside the library image instead of the context's growable workspace.  Every GPU that loads the
// library carries these 2 MiB until the process exits.
namespace {
constexpr size_t NOALLOC_SCRATCH_BYTES = 2u << 20;
static __device__ __align__(256) unsigned char g_accept_scratch[NOALLOC_SCRATCH_BYTES];
constexpr int NOALLOC_MAX_DEVICES = 64;
void* g_accept_scratch_ptr[NOALLOC_MAX_DEVICES] = {nullptr};  // device address of the array, per device
std::mutex g_accept_scratch_mutex;
}  // namespace

extern "C" {

int32_t vn_accept_noalloc(vn_ctx* ctx, const float* p_logits_dev, const float* q_logits_dev, const int64_t* draft_dev,
                          const float* u_accept_dev, const float* u_sample_dev, uint64_t seed, uint32_t offset,
                          float temperature, int32_t bonus, int32_t B, int32_t k, int32_t V, int32_t* out_len_dev,
                          int64_t* out_tokens_dev) {
  VN_CHECK_CTX(ctx);
  VN_REQUIRE(ctx, B >= 0 && k >= 0 && k <= MAX_K && V >= 1, "bad sizes B=%d k=%d V=%d (k <= %d)", B, k, V, MAX_K);
  VN_REQUIRE(ctx, p_logits_dev && out_len_dev && out_tokens_dev, "null pointer");
  VN_REQUIRE(ctx, k == 0 || draft_dev, "draft tokens missing");
  VN_REQUIRE(ctx, (u_accept_dev == nullptr) == (u_sample_dev == nullptr) || k == 0,
             "inject both uniform arrays or neither");
  VN_REQUIRE(ctx, bonus || k > 0, "nothing to do: k == 0 without a bonus token");
  VN_REQUIRE(ctx, ctx->device >= 0 && ctx->device < NOALLOC_MAX_DEVICES, "device index %d not supported here", ctx->device);
  if (B == 0) return VN_OK;
  const bool greedy = temperature <= 0.f;
  const float temp = greedy ? 1.0f : fmaxf(temperature, 1e-8f);
  RowSet rs;
  rs.p = p_logits_dev; rs.q = greedy ? nullptr : q_logits_dev;
  rs.np = bonus ? k + 1 : k;
  rs.nq = (rs.q && k > 0) ? k : 0;
  rs.p_sb = (long long)rs.np * V; rs.p_si = V; rs.q_sb = (long long)k * V; rs.q_si = V;
  rs.V = V;
  const int rows_per_seq = rs.np + rs.nq;
  const int nchunks = ceil_div(V, CHUNK);
  const size_t n_part = (size_t)B * rows_per_seq * nchunks;
  const size_t off_dec = (n_part * sizeof(Partial) + 255) & ~(size_t)255;
  const size_t off_mass = (off_dec + (size_t)B * sizeof(Decision) + 255) & ~(size_t)255;
  const size_t total = off_mass + (size_t)B * nchunks * 2 * sizeof(double);
  if (total > NOALLOC_SCRATCH_BYTES)
    return vn_fail(ctx, VN_ERR_INVALID,
                   "vn_accept_noalloc: B=%d k=%d V=%d needs %zu bytes of scratch, the built-in array holds %zu "
                   "(use vn_accept for larger problems)", B, k, V, total, NOALLOC_SCRATCH_BYTES);
  // One-time set-up per device, with that device current (VN_CHECK_CTX selected it): in host code the array's
  // name is only a stand-in for the symbol, so its device address has to be asked for.
  void* ws = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_accept_scratch_mutex);
    if (!g_accept_scratch_ptr[ctx->device]) {
      void* addr = nullptr;
      cudaError_t e = cudaGetSymbolAddress(&addr, g_accept_scratch);
      if (e != cudaSuccess || !addr)
        return vn_fail(ctx, VN_ERR_CUDA, "cudaGetSymbolAddress(g_accept_scratch) failed: %s", cudaGetErrorString(e));
      g_accept_scratch_ptr[ctx->device] = addr;
    }
    ws = g_accept_scratch_ptr[ctx->device];
  }
  Partial* part = (Partial*)ws;
  Decision* dec = (Decision*)((char*)ws + off_dec);
  double* mass = (double*)((char*)ws + off_mass);
  const long long* d64 = reinterpret_cast<const long long*>(draft_dev);
  long long* o64 = reinterpret_cast<long long*>(out_tokens_dev);
  auto aligned16 = [](const void* ptr) { return ((uintptr_t)ptr & 15) == 0; };
  const bool vec = (V % 4 == 0) && aligned16(rs.p) && (!rs.nq || aligned16(rs.q));
  // every kernel below overwrites the part of the scratch it owns before anything reads it (each chunk
  // statistic, decision and mass entry that is read was written earlier in this same call), so nothing left
  // over from the previous call has to be cleared
  const int grid = (int)std::min<long long>((long long)n_part, (long long)ctx->sm_count * 8);
  { const int32_t st_ = launch_accept_stats(ctx, vec, greedy, grid, rs, B, nchunks, temp, part); if (st_) return st_; }
  // the device-side round counter (vn_set_offset_source) shifts the Philox offset here exactly as in vn_accept
  VN_LAUNCH(ctx, accept_decide_kernel, B, 128, 0, rs, B, k, nchunks, part, d64, u_accept_dev, u_sample_dev, seed, offset,
            ctx->offset_src, temp, (int)greedy, bonus, 1, 0, dec, out_len_dev, o64);
  if (!greedy) {
    dim3 g(nchunks, B);
    if (vec) VN_LAUNCH(ctx, accept_residual_kernel<true>, g, STATS_THREADS, 0, rs, nchunks, temp, dec, mass);
    else     VN_LAUNCH(ctx, accept_residual_kernel<false>, g, STATS_THREADS, 0, rs, nchunks, temp, dec, mass);
    VN_LAUNCH(ctx, accept_pick_kernel, B, STATS_THREADS, 0, rs, k, nchunks, temp, dec, mass, o64);
  }
  return VN_OK;
}

int32_t vn_philox_uniform(vn_ctx* ctx, uint64_t seed, uint32_t offset, int32_t B, int32_t n, int32_t purpose,
                          float* out_dev) {
  VN_CHECK_CTX(ctx);
  VN_REQUIRE(ctx, B >= 0 && n >= 0 && out_dev, "bad arguments");
  if (B * n == 0) return VN_OK;
  VN_LAUNCH(ctx, philox_uniform_kernel, ceil_div(B * n, 256), 256, 0, seed, offset, B, n, purpose, out_dev);
  return VN_OK;
}

}  // extern "C"
