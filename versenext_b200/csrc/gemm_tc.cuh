// Weight-streaming skinny GEMM on the 5th-generation tensor cores (tcgen05 + TMEM), fed by TMA.
//
//   C[m, n] = sum_k X[m, k] * W[n, k]        X: tokens x K (bf16), W: features x K (bf16), few tokens (<= 256)
//
// The roles are swapped with respect to the usual layout: the WEIGHT tile is the UMMA "A" operand (M = 128
// output features -> 128 TMEM lanes) and the token block is the "B" operand (N = tokens, 16 .. 256), so one
// CTA streams a 128 x K slab of the weight matrix exactly once while the small activation block is re-read
// from L2.  D[feature, token] accumulates in TMEM (fp32), is read back with tcgen05.ld by four epilogue
// warps (lane = feature), and is written so that consecutive lanes hit consecutive features of one token.
//
// CTA = 6 warps: warp 0 issues TMA loads (one elected thread), warp 1 allocates TMEM and issues tcgen05.mma
// (one thread), warps 2..5 run the epilogue.  A ring of STAGES shared-memory stages (weight tile 128 x 64 +
// token tile NTOK x 64, both 128-byte swizzled, K-major) is handed over with mbarriers.  Every wait is
// bounded: when it runs out the kernel raises a flag in global memory, stops issuing work, and still frees
// its TMEM before returning.
//
// Split-K: blockIdx.y selects a K range; partial tiles go to a workspace [split][rows][N] and are reduced by
// the caller's finalize kernel (deterministic order).
#pragma once
#include <math_constants.h>
#include <cuda.h>
#include <stdlib.h>
#include "gemm.cuh"

namespace tc_detail {

constexpr int BF = 128;        // features per CTA (UMMA M)
constexpr int BK = 64;         // K elements per stage = one 128-byte swizzle row
constexpr int TC_THREADS = 320;      // TMA warp, MMA warp, two groups of four epilogue warps
constexpr int PERSIST_THREADS = 192; // persistent variant: one epilogue group
constexpr unsigned long long WAIT_LIMIT_CYCLES = 2000000000ull;  // ~1 s
// the limit every bounded wait of these kernels uses, in SM cycles; vn_model_set_wait_limit changes it (a test makes
// a wait run out in a millisecond instead of a second)
__device__ unsigned long long g_wait_limit_cycles = WAIT_LIMIT_CYCLES;

// RoPE + KV-cache append applied to the q | k | v projection (same meaning as in rope_append_kernel)
struct TcRope {
  const float* cos_t; const float* sin_t;
  const int* lens; const int* depth;
  void* kc; void* vc;      // bf16 caches [B, max_seq, n_kv, hd]
  float* q_out;            // fp32 [rows, ldq]: q heads rotated (k and v columns are not written)
  long long ldq;
  int Tn, H, n_kv, hd, max_seq, use_rope, rope_rows, slot_offset;
};

// Candidate lists filled by the LM-head epilogue in TC_FILTER mode: instead of storing a row's logits, every logit
// at or above the row's lower bound `tau` is appended to the row's list (order arbitrary; `count` may run past
// `cap`, entries beyond it are dropped and the consumer sees the overflow from the count).
struct CandBuf {
  const float* tau = nullptr;   // [rows] raw-logit bound per token row
  int* count = nullptr;         // row r's counter at count[r * count_stride]
  int count_stride = 1;
  float* val = nullptr;         // [rows][cap] raw logits
  int* tok = nullptr;           // [rows][cap] feature (vocabulary) index
  int cap = 0;
};

struct TcArgs {
  void* C;                 // see epi
  const float* bias;
  long long ldc;
  int M, N, K;             // tokens (per segment: upper bound), features, reduction
  int ntok;                // UMMA N: tokens rounded up to 16
  int x_box;               // token rows per TMA box: ntok (one box) for a dense block, 16 in segmented mode
  unsigned smem_budget;    // bytes of stage memory behind the 1024-byte aligned base
  int tma_out;             // fp32 output rows leave through TMA stores (dense PARTIAL / STORE only)
  int out_bufs;            // 16 KB staging tiles per epilogue group for that
  int kb_per_split;        // k blocks (of 64) per blockIdx.y
  int epi, c_bf16;
  const int* seg_off;      // segmented mode (blockIdx.z = segment)
  const int* seg_cnt;
  long long w_rows_per_seg;  // rows of W between consecutive weight matrices
  const int* seg_w;          // weight matrix of segment z, or null (matrix z)
  float* partial;          // split-K workspace [gridDim.y][rows_total][N] or null
  long long partial_stride;  // rows_total * N
  int* error_flag;
  long long* trace;        // optional [CTAs][8] clock64 stamps of the kernel's phases (null: no tracing)
  // cluster modes: the CTAs of one feature tile (blockIdx.y = K range) form a thread-block cluster and reduce
  // their partial tiles through distributed shared memory; the epilogue below runs on the reduced rows
  float* resid;            // TC_CL_ADD: resid[row, n] += value (fp32, pitch ldc)
  TcRope rope;             // TC_CL_QKV
  CandBuf cand;            // TC_FILTER
  const int* run_if;       // when set: the whole grid returns at once unless *run_if != 0 (read after the wait for
                           // the preceding kernels); lets a fallback sit in a captured graph at almost no cost
};

// SM cycle counter, ordered with the surrounding memory operations (for the optional phase stamps)
__device__ __forceinline__ long long clock_now() {
  long long c;
  asm volatile("mov.u64 %0, %%clock64;" : "=l"(c) :: "memory");
  return c;
}
__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned long long* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// adds to the transaction count of the current phase without arriving
__device__ __forceinline__ void mbar_expect_tx_only(unsigned long long* bar, unsigned bytes) {
  asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(unsigned long long* bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// bounded wait; false when the limit ran out
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity) {
  if (mbar_try(bar, parity)) return true;
  const long long t0 = clock64();
  const unsigned long long limit = g_wait_limit_cycles;
  while (!mbar_try(bar, parity)) {
    if ((unsigned long long)(clock64() - t0) > limit) return false;
  }
  return true;
}

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* tmap, unsigned long long* bar, int c0,
                                            int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(tmap), "r"(smem_u32(bar)), "r"(c0), "r"(c1) : "memory");
}

// one 32-token x 128-feature fp32 tile from shared memory to the output tensor (x = feature, y = row, z = slice);
// rows and columns beyond the tensor are clipped by the hardware
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* tmap, const void* smem_src, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
               ::"l"(tmap), "r"(smem_u32(smem_src)), "r"(x), "r"(y), "r"(z) : "memory");
}

// K-major, 128-byte swizzle: 8-row groups of 1024 bytes (SBO = 1024 B -> 64), LBO unused (= 1), version 1
__device__ __forceinline__ unsigned long long umma_desc(const void* smem_tile) {
  const unsigned addr = smem_u32(smem_tile);
  unsigned long long d = 0;
  d |= (unsigned long long)((addr & 0x3FFFFu) >> 4);
  d |= (unsigned long long)1 << 16;
  d |= (unsigned long long)64 << 32;
  d |= (unsigned long long)1 << 46;
  d |= (unsigned long long)2 << 61;
  return d;
}

__device__ __forceinline__ void umma_bf16(unsigned tmem_d, unsigned long long da, unsigned long long db, unsigned idesc,
                                          unsigned accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(unsigned long long* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(unsigned taddr, unsigned (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}

enum { TC_PARTIAL = 0, TC_STORE = 1, TC_SWIGLU = 2, TC_ADD = 3,
       TC_CL_STORE = 4, TC_CL_SWIGLU = 5, TC_CL_ADD = 6, TC_CL_QKV = 7,     // 4 .. 7: cluster split-K
       TC_FILTER = 8 };

__device__ __forceinline__ unsigned cluster_rank() { unsigned r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ unsigned cluster_size() { unsigned r; asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r)); return r; }
// every thread of every CTA of the cluster; release / acquire so that shared-memory writes before it are
// visible to distributed-shared-memory reads after it
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float4 ld_dsmem_f4(unsigned local_addr, unsigned rank) {
  unsigned ra; float4 v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(local_addr), "r"(rank));
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(ra));
  return v;
}

// TC_FILTER staging: hits parked in shared memory (behind a 16-byte header whose first int counts them)
struct FilterHit { int row; float val; int tok; };
constexpr int FILTER_STAGE = 1024;             // 12 KB of the epilogue's staging memory

// called by all `nthreads` epilogue threads after a barrier behind the last tc_epilogue_chunk<TC_FILTER> of a tile
__device__ __forceinline__ void filter_flush(const TcArgs& g, unsigned char* base, int tid_epi, int nthreads) {
  const int* s_n = reinterpret_cast<const int*>(base);
  const FilterHit* s_hit = reinterpret_cast<const FilterHit*>(base + 16);
  const int n = *s_n < FILTER_STAGE ? *s_n : FILTER_STAGE;
  for (int e = tid_epi; e < n; e += nthreads) {
    const FilterHit h = s_hit[e];
    const int slot = atomicAdd(g.cand.count + (long long)h.row * g.cand.count_stride, 1);
    if (slot < g.cand.cap) {
      g.cand.val[(long long)h.row * g.cand.cap + slot] = h.val;
      g.cand.tok[(long long)h.row * g.cand.cap + slot] = h.tok;
    }
  }
}

// Epilogue of one 32-token chunk of the accumulator (r[i] = feature f of token m0 + i for this thread).
// `base` points at 32 KB of shared memory for two staging tiles (`buf` selects one; callers alternate so that a
// tile is not rewritten while another warp still reads it) shared by the four warps that meet at named barrier
// `bar_id`.  split_y selects the slice of the split-K workspace.
template <int MODE>
__device__ __forceinline__ void tc_epilogue_chunk(const TcArgs& g, const unsigned (&r)[32], unsigned char* base,
                                                  int ch, int buf, int bar_id, int q, int lane, int n0, int row0,
                                                  int cnt, int split_y, bool vec_ok, bool swi_ok) {
  const int f = q * 32 + lane, n = n0 + f;
  const int m0 = ch * 32;
  const int mrem = cnt - m0;               // tokens left from this chunk on (>= 1)
    if (MODE == TC_FILTER) {
      // Logits never leave the SM: the few that reach the row's bound (well under one in a hundred) are parked in
      // shared memory as (row, value, column); filter_flush below hands them to the rows' lists in global memory
      // with all of the CTA's atomics in flight together -- an atomic per hit inside this loop would stall the warp
      // for an L2 round trip every time.
      // The rows' bounds first, all 32 loads in flight together: inside the compare loop below a load could not be
      // moved across the shared-memory atomic of a hit, and the loop ran at one exposed load latency per row
      // (5.6 us per 160-row tile with no hit at all; the plain store epilogue takes 2.4 us).
      const float* tau = g.cand.tau + row0 + m0;
      float tv[32];
      if (mrem >= 32 && (reinterpret_cast<uintptr_t>(tau) & 15) == 0) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float4 t4 = __ldg(reinterpret_cast<const float4*>(tau) + i);
          tv[4 * i] = t4.x; tv[4 * i + 1] = t4.y; tv[4 * i + 2] = t4.z; tv[4 * i + 3] = t4.w;
        }
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) tv[i] = i < mrem ? __ldg(tau + i) : CUDART_INF_F;
      }
      // which of the 32 rows hit: a bit mask without branches; three threads in four have no hit in a chunk and
      // leave here
      unsigned hit = 0u;
#pragma unroll
      for (int i = 0; i < 32; ++i) hit |= (__uint_as_float(r[i]) >= tv[i] ? 1u : 0u) << i;
      // Parking: one shared-memory atomic per warp and chunk reserves room for all of the warp's hits (a prefix
      // sum over the lanes' hit counts gives each lane its place); a lane then stores its hits one after the other.
      // An atomic per hit inside the diverged 32-way loop cost 4.5 us per tile.
      int* s_n = reinterpret_cast<int*>(base);
      FilterHit* s_hit = reinterpret_cast<FilterHit*>(base + 16);
      const unsigned mine = n < g.N ? hit : 0u;
      const int cntl = __popc(mine);
      int incl = cntl;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
      }
      const int total = __shfl_sync(0xffffffffu, incl, 31);
      if (total) {                               // uniform over the warp
        int first = 0;
        if (lane == 31) first = atomicAdd(s_n, total);
        first = __shfl_sync(0xffffffffu, first, 31);
        int pos = first + incl - cntl;
        // Straight-line, predicated stores: the 32 copies of this body must stay tiny.  With the overflow path
        // (64-bit addresses, a global atomic) inside, the rarely taken copies were fetched cold every time they ran:
        // 3 us per tile.
        const int pos0 = pos;
        bool over = false;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const bool bit = (mine >> i) & 1u;
          const bool ok = bit && pos < FILTER_STAGE;
          if (ok) {
            FilterHit* dst = s_hit + pos;
            dst->row = row0 + m0 + i; dst->val = __uint_as_float(r[i]); dst->tok = n;
          }
          over |= bit && !ok;
          pos += bit ? 1 : 0;
        }
        if (over) {                              // staging full (heavy ties): the rest goes straight to the lists
          pos = pos0;
#pragma unroll 1
          for (int i = 0; i < 32; ++i) {
            if (!((mine >> i) & 1u)) continue;
            if (pos >= FILTER_STAGE) {
              float v = 0.f;
#pragma unroll
              for (int j = 0; j < 32; ++j) v = j == i ? __uint_as_float(r[j]) : v;
              const long long rowg = row0 + m0 + i;
              const int slot = atomicAdd(g.cand.count + rowg * g.cand.count_stride, 1);
              if (slot < g.cand.cap) { g.cand.val[rowg * g.cand.cap + slot] = v; g.cand.tok[rowg * g.cand.cap + slot] = n; }
            }
            ++pos;
          }
        }
      }
    } else if (MODE >= TC_CL_STORE) {
      // whole partial tile [token][feature] in this CTA's shared memory; reduced after the cluster barrier
      float* tile = reinterpret_cast<float*>(base);
#pragma unroll
      for (int i = 0; i < 32; ++i) tile[(m0 + i) * BF + f] = __uint_as_float(r[i]);
    } else if (MODE == TC_PARTIAL || (MODE == TC_STORE && !g.c_bf16)) {
      // fp32 rows of the output: staged through shared memory (the pipeline stages are free once the
      // accumulator is complete) so that one instruction stores 512 contiguous bytes of a token row
      float* out; long long ld;
      if (MODE == TC_PARTIAL) { out = g.partial + (long long)split_y * g.partial_stride; ld = g.N; }
      else { out = reinterpret_cast<float*>(g.C); ld = g.ldc; }
      out += (long long)(row0 + m0) * ld + n0;
      const float bias = (MODE == TC_STORE && g.bias && n < g.N) ? g.bias[n] : 0.f;
      if (vec_ok) {
        float* tile = reinterpret_cast<float*>(base) + buf * (32 * BF);
#pragma unroll
        for (int i = 0; i < 32; ++i) tile[i * BF + f] = __uint_as_float(r[i]) + bias;
        asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
        const int c4 = lane * 4;
        if (n0 + c4 < g.N) {                 // N % 4 == 0: a float4 is inside or outside as a whole
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int row = q * 8 + j;
            if (row < mrem)
              *reinterpret_cast<float4*>(out + (long long)row * ld + c4) =
                  *reinterpret_cast<const float4*>(tile + row * BF + c4);
          }
        }
      } else if (n < g.N) {
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (i < mrem) out[(long long)i * ld + f] = __uint_as_float(r[i]) + bias;
      }
    } else if (MODE == TC_SWIGLU) {
      // (gate, up) sit in adjacent columns: stage the fp32 tile, then every lane turns two pairs of a token
      // row into two outputs, so that a warp stores 64 contiguous outputs of a row at once
      if (swi_ok) {
        float* tile = reinterpret_cast<float*>(base) + buf * (32 * BF);
#pragma unroll
        for (int i = 0; i < 32; ++i) tile[i * BF + f] = __uint_as_float(r[i]);
        asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
        const int c4 = lane * 4;
        if (n0 + c4 + 3 < g.N) {
#pragma unroll 2
          for (int j = 0; j < 8; ++j) {
            const int row = q * 8 + j;
            if (row < mrem) {
              const float4 v = *reinterpret_cast<const float4*>(tile + row * BF + c4);
              const float o0 = silu_ref(v.x) * v.y, o1 = silu_ref(v.z) * v.w;
              const long long at = (long long)(row0 + m0 + row) * g.ldc + ((n0 + c4) >> 1);
              if (g.c_bf16)
                *reinterpret_cast<__nv_bfloat162*>(reinterpret_cast<__nv_bfloat16*>(g.C) + at) =
                    __floats2bfloat162_rn(o0, o1);
              else
                *reinterpret_cast<float2*>(reinterpret_cast<float*>(g.C) + at) = make_float2(o0, o1);
            }
          }
        }
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float v = __uint_as_float(r[i]);
          const float other = __shfl_xor_sync(0xffffffffu, v, 1);
          if (i < mrem && !(lane & 1) && n + 1 < g.N)
            store_out<float>(g.C, (long long)(row0 + m0 + i) * g.ldc + (n >> 1), silu_ref(v) * other, g.c_bf16);
        }
      }
    } else if (MODE == TC_ADD) {
      if (n < g.N) {
        float* dst = reinterpret_cast<float*>(g.C) + (long long)(row0 + m0) * g.ldc + n;
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (i < mrem) dst[(long long)i * g.ldc] += __uint_as_float(r[i]);
      }
    } else {
      if (n < g.N) {
        const float bias = g.bias ? g.bias[n] : 0.f;
        const long long at = (long long)(row0 + m0) * g.ldc + n;
        if (g.c_bf16) {
          __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(g.C) + at;
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (i < mrem) dst[(long long)i * g.ldc] = __float2bfloat16_rn(__uint_as_float(r[i]) + bias);
        } else {
          float* dst = reinterpret_cast<float*>(g.C) + at;
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (i < mrem) dst[(long long)i * g.ldc] = __uint_as_float(r[i]) + bias;
        }
      }
    }
}

template <int MODE>
__global__ void __launch_bounds__(TC_THREADS)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
               const __grid_constant__ CUtensorMap tm_out, TcArgs g) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ unsigned long long bar_full[8], bar_empty[8], bar_acc;
  __shared__ unsigned tmem_base_slot;
  __shared__ int s_error;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int z = blockIdx.z;
  int row0 = 0, cnt = g.M;
  long long* tr = g.trace ? g.trace + 8ll * (blockIdx.x + gridDim.x * (blockIdx.y + (long long)gridDim.y * blockIdx.z)) : nullptr;
  if (tr && threadIdx.x == 0) {
    tr[0] = clock_now();
    unsigned long long ns;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(ns));
    tr[6] = (long long)ns;
  }
  pdl_trigger();
  if (g.run_if) {          // uniform over the grid: nothing has been allocated or initialised yet
    pdl_wait();
    if (*reinterpret_cast<const volatile int*>(g.run_if) == 0) return;
  }
  // segment sizes are written by the routing kernels that precede this one; a dense block only waits
  // once its first weight tiles are on their way (weights never change)
  if (g.seg_cnt) { pdl_wait(); row0 = g.seg_off[z]; cnt = g.seg_cnt[z]; }
  if (cnt > g.ntok) cnt = g.ntok;
  const int cnt16 = (cnt + 15) & ~15;      // UMMA N and token rows loaded by this CTA
  const int n0 = blockIdx.x * BF;
  const int nkb_total = (g.K + BK - 1) / BK;
  const int kb0 = blockIdx.y * g.kb_per_split;
  int nkb = nkb_total - kb0;
  if (nkb > g.kb_per_split) nkb = g.kb_per_split;
  // nothing to do for this CTA: uniform exit before any barrier or TMEM allocation
  if (cnt <= 0 || nkb <= 0) return;

  // stage buffers: 1024-byte aligned (swizzle atom), weight tile then token tile
  unsigned char* base = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  // a stage holds the weight tile and the token rows this CTA really has, so a short segment gets more
  // stages out of the same shared memory
  const unsigned w_bytes = BF * BK * 2, x_bytes = (unsigned)cnt16 * BK * 2;
  const unsigned stage_bytes = w_bytes + x_bytes;
  int S = (int)(g.smem_budget / stage_bytes);
  S = S > 8 ? 8 : S;
  S = S > nkb ? (nkb < 2 ? 2 : nkb) : S;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) { mbar_init(&bar_full[s], 1); mbar_init(&bar_empty[s], 1); }
    mbar_init(&bar_acc, 1);
    s_error = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  // TMEM: power of two >= ntok rounded to 32 columns
  unsigned ncols = 32;
  while (ncols < (unsigned)((g.ntok + 31) & ~31)) ncols <<= 1;
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned tmem_base = tmem_base_slot;
  if (tr && threadIdx.x == 0) tr[1] = clock_now();          // barriers initialised, TMEM allocated

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      const int w_row = (int)((long long)(g.seg_w ? g.seg_w[z] : z) * g.w_rows_per_seg) + n0;
      int kb_first = 0;
      if (!g.seg_cnt) {
        const int npre = nkb < S ? nkb : S;
        for (int kb = 0; kb < npre; ++kb) {
          mbar_expect_tx_only(&bar_full[kb], w_bytes);
          tma_load_2d(base + (size_t)kb * stage_bytes, &tm_w, &bar_full[kb], (kb0 + kb) * BK, w_row);
        }
        pdl_wait();
        for (int kb = 0; kb < npre; ++kb) {
          mbar_expect_tx(&bar_full[kb], (unsigned)cnt16 * BK * 2);
          for (int r16 = 0; r16 < cnt16; r16 += g.x_box)
            tma_load_2d(base + (size_t)kb * stage_bytes + w_bytes + (size_t)r16 * BK * 2, &tm_x, &bar_full[kb],
                        (kb0 + kb) * BK, row0 + r16);
        }
        kb_first = npre;
      }
      for (int kb = kb_first; kb < nkb; ++kb) {
        const int s = kb % S;
        if (!mbar_wait(&bar_empty[s], ((kb / S) & 1) ^ 1)) { s_error = 1; break; }
        unsigned char* st = base + (size_t)s * stage_bytes;
        mbar_expect_tx(&bar_full[s], w_bytes + (unsigned)cnt16 * BK * 2);
        const int kx = (kb0 + kb) * BK;
        tma_load_2d(st, &tm_w, &bar_full[s], kx, w_row);
        // tokens in boxes of 16 rows (two swizzle atoms each): only the rows this segment has
        for (int r16 = 0; r16 < cnt16; r16 += g.x_box)
          tma_load_2d(st + w_bytes + (size_t)r16 * BK * 2, &tm_x, &bar_full[s], kx, row0 + r16);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      // instruction descriptor: D fp32, A and B bf16, both K-major, N = ntok, M = 128
      const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(cnt16 >> 3) << 17) | ((unsigned)(BF >> 4) << 24);
      bool ok = true;
      for (int kb = 0; kb < nkb && ok; ++kb) {
        const int s = kb % S;
        if (!mbar_wait(&bar_full[s], (kb / S) & 1)) { s_error = 1; ok = false; break; }
        if (tr && kb == 0) tr[2] = clock_now();             // first stage landed
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        unsigned char* st = base + (size_t)s * stage_bytes;
        const unsigned long long da = umma_desc(st), db = umma_desc(st + w_bytes);
#pragma unroll
        for (int k4 = 0; k4 < BK / 16; ++k4)   // +32 bytes along K inside the swizzle row: +2 in the address field
          umma_bf16(tmem_base, da + 2ull * k4, db + 2ull * k4, idesc, (kb | k4) != 0);
        umma_commit(&bar_empty[s]);            // frees the stage when these MMAs have read it
      }
      umma_commit(&bar_acc);                   // accumulator complete (or abandoned)
      if (tr) tr[3] = clock_now();                          // last MMA issued
    }
  } else {
    // ---------------- epilogue: warps 2..9 in two groups of four (TMEM lane quarter = warp % 4); the groups take
    // the 32-token chunks of the accumulator alternately, each with its own staging tiles and named barrier
    const int q = warp & 3;
    const int grp = (warp - 2) >> 2;
    const int f = q * 32 + lane;               // feature within the tile
    const int n = n0 + f;
    pdl_wait();
    const bool acc_ok = mbar_wait(&bar_acc, 0);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (!acc_ok) s_error = 1;
    if (tr && threadIdx.x == 64) tr[4] = clock_now();       // accumulator complete
    // one decision for the four epilogue warps (named barrier 1 with an AND reduction): the TMEM loads are
    // warp-collective and the staged stores below synchronise the four warps with each other
    int go;
    {
      const int mine = (acc_ok && *(volatile int*)&s_error == 0) ? 1 : 0;
      asm volatile(
          "{\n\t.reg .pred p, q;\n\t"
          "setp.ne.b32 q, %1, 0;\n\t"
          "bar.red.and.pred p, 1, 256, q;\n\t"
          "selp.u32 %0, 1, 0, p;\n\t}"
          : "=r"(go) : "r"(mine) : "memory");
    }
    if (go) {
      // One instantiation per epilogue kind keeps this unrolled loop small: with all kinds in one body the
      // loop outgrew the instruction cache and the epilogue took 9 us for 160 tokens instead of about 1.
      const int nchunk = (cnt + 31) >> 5;
      if (MODE == TC_FILTER) {                 // the stage memory is free now: its head holds the parked hits
        if (threadIdx.x == 64) *reinterpret_cast<int*>(base) = 0;
        asm volatile("bar.sync 1, 256;" ::: "memory");
      }
      // float4 rows need 16-byte alignment of every row start (uniform over the CTA)
      const bool vec_ok = MODE == TC_PARTIAL
                              ? (g.N % 4 == 0 && ((uintptr_t)g.partial & 15) == 0)
                              : (g.ldc % 4 == 0 && g.N % 4 == 0 && ((uintptr_t)g.C & 15) == 0);
      // paired outputs: rows of C start on an 8-byte boundary and N covers whole groups of four columns
      const bool swi_ok = MODE == TC_SWIGLU && g.ldc % 4 == 0 && g.N % 4 == 0 && ((uintptr_t)g.C & 7) == 0;
      const bool tma_out = (MODE == TC_PARTIAL || MODE == TC_STORE) && g.tma_out;   // uniform over the CTA
      const bool issuer = ((warp - 2) & 3) == 0 && lane == 0;                        // one thread per group
      for (int ch = grp; ch < nchunk; ch += 2) {
        unsigned r[32];
        tmem_ld32(tmem_base + ((unsigned)(q * 32) << 16) + (unsigned)(ch * 32), r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (tma_out) {
          // registers -> shared memory once, then the tile leaves asynchronously: the load/store units move every
          // byte one time instead of three (staging store, staging load, global store)
          const int jb = ch >> 1;
          float* tile = reinterpret_cast<float*>(base + ((size_t)grp * g.out_bufs + (jb % g.out_bufs)) * (32 * BF * 4));
          if (jb >= g.out_bufs) {           // the tile is being reused: its earlier store must have read it
            if (issuer) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
            asm volatile("bar.sync %0, 128;" ::"r"(2 + grp) : "memory");
          }
          const int f = q * 32 + lane;
          const float bias = (MODE == TC_STORE && g.bias && n0 + f < g.N) ? g.bias[n0 + f] : 0.f;
#pragma unroll
          for (int i = 0; i < 32; ++i) tile[i * BF + f] = __uint_as_float(r[i]) + bias;
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          asm volatile("bar.sync %0, 128;" ::"r"(2 + grp) : "memory");
          if (issuer) {
            tma_store_3d(&tm_out, tile, n0, row0 + ch * 32, MODE == TC_PARTIAL ? (int)blockIdx.y : 0);
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
        } else {
          tc_epilogue_chunk<MODE>(g, r, (MODE >= TC_CL_STORE || MODE == TC_FILTER) ? base : base + grp * (32 * 1024), ch, (ch >> 1) & 1, 2 + grp,
                                  q, lane, n0, row0, cnt, (int)blockIdx.y, vec_ok, swi_ok);
        }
      }
      if (MODE == TC_FILTER) {
        asm volatile("bar.sync 1, 256;" ::: "memory");
        filter_flush(g, base, (int)threadIdx.x - 64, 256);
      }
      // the staging tiles must have been read before the CTA gives its shared memory back; the writes themselves
      // are complete and visible when the grid completes, which is what every consumer waits for
      if (tma_out && issuer) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    }
    if (tr && threadIdx.x == 64) tr[5] = clock_now();     // this warp's stores issued
  }
  if (MODE >= TC_CL_STORE && MODE != TC_FILTER) {
    __syncwarp();            // the single-lane roles above rejoin their warps before the aligned barriers
    cluster_sync_all();
    if (warp >= 2 && *(volatile int*)&s_error == 0) {
      const int q = warp - 2;                       // eight warps share the rows
      const unsigned rank = cluster_rank(), S = cluster_size();
      const unsigned tile_addr = smem_u32(base);
      const int c4 = lane * 4, n = n0 + c4;
      // rows rank, rank + S, ... of the tile belong to this CTA; its four epilogue warps take them in turn
      // (all peers' loads of a row are issued before the first add)
      auto reduce_row = [&](int m, float4 (&pv)[8]) {
        const unsigned at = tile_addr + (unsigned)((m * BF + c4) * 4);
#pragma unroll
        for (unsigned pr = 0; pr < 8; ++pr)
          if (pr < S) pv[pr] = ld_dsmem_f4(at, pr);
      };
      auto sum_row = [&](const float4 (&pv)[8]) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (unsigned pr = 0; pr < 8; ++pr)        // fixed order: the sum does not depend on scheduling
          if (pr < S) { acc.x += pv[pr].x; acc.y += pv[pr].y; acc.z += pv[pr].z; acc.w += pv[pr].w; }
        return acc;
      };
      auto finish = [&](int m, float4 acc) {
        const long long row = row0 + m;
        if (MODE == TC_CL_ADD) {
          if (n < g.N) {
            float4* dst = reinterpret_cast<float4*>(g.resid + row * g.ldc + n);
            float4 x = *dst;
            x.x += acc.x; x.y += acc.y; x.z += acc.z; x.w += acc.w;
            *dst = x;
          }
        } else if (MODE == TC_CL_SWIGLU) {
          if (n < g.N) {
            const float o0 = silu_ref(acc.x) * acc.y, o1 = silu_ref(acc.z) * acc.w;
            const long long o_at = row * g.ldc + (n >> 1);
            if (g.c_bf16)
              *reinterpret_cast<__nv_bfloat162*>(reinterpret_cast<__nv_bfloat16*>(g.C) + o_at) = __floats2bfloat162_rn(o0, o1);
            else
              *reinterpret_cast<float2*>(reinterpret_cast<float*>(g.C) + o_at) = make_float2(o0, o1);
          }
        } else if (MODE == TC_CL_QKV) {
          const TcRope& rp = g.rope;
          const int b = (int)(row / rp.Tn), t = (int)(row % rp.Tn);
          const int len = rp.lens[b] + rp.slot_offset;
          const int pos = len + (rp.depth ? rp.depth[t] : t);
          const int slot = len + t;
          const int half = rp.hd >> 1;
          const int head = n / rp.hd, j = n % rp.hd;       // the four features of a lane share head and half
          float v[4] = {acc.x, acc.y, acc.z, acc.w};
          const bool rot = rp.use_rope && head < rp.H + rp.n_kv;
          {
            const int pp = pos < rp.rope_rows ? pos : rp.rope_rows - 1;
            const int jj = j < half ? j : j - half;
            const int part = half >> 2;                    // lanes between a feature and its rotation partner
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float other = __shfl_xor_sync(0xffffffffu, v[e], part);
              if (rot && n < g.N) {
                const float c = rp.cos_t[(long long)pp * half + jj + e], sn = rp.sin_t[(long long)pp * half + jj + e];
                v[e] = j < half ? v[e] * c + (-other) * sn : v[e] * c + other * sn;
              }
            }
          }
          if (n < g.N) {
            if (head < rp.H) {
              *reinterpret_cast<float4*>(rp.q_out + row * rp.ldq + n) = make_float4(v[0], v[1], v[2], v[3]);
            } else if (slot < rp.max_seq) {
              const bool is_k = head < rp.H + rp.n_kv;
              const int kh = is_k ? head - rp.H : head - rp.H - rp.n_kv;
              __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(is_k ? rp.kc : rp.vc) +
                                   (((long long)b * rp.max_seq + slot) * rp.n_kv + kh) * rp.hd + j;
              reinterpret_cast<__nv_bfloat162*>(dst)[0] = __floats2bfloat162_rn(v[0], v[1]);
              reinterpret_cast<__nv_bfloat162*>(dst)[1] = __floats2bfloat162_rn(v[2], v[3]);
            }
          }
        } else {
          if (n < g.N) {
            if (g.bias) { acc.x += g.bias[n]; acc.y += g.bias[n + 1]; acc.z += g.bias[n + 2]; acc.w += g.bias[n + 3]; }
            if (g.c_bf16) {
              __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(g.C) + row * g.ldc + n;
              reinterpret_cast<__nv_bfloat162*>(dst)[0] = __floats2bfloat162_rn(acc.x, acc.y);
              reinterpret_cast<__nv_bfloat162*>(dst)[1] = __floats2bfloat162_rn(acc.z, acc.w);
            } else {
              *reinterpret_cast<float4*>(reinterpret_cast<float*>(g.C) + row * g.ldc + n) = acc;
            }
          }
        }
      };
      for (int m = (int)rank + (int)S * q; m < cnt; m += (int)S * 8) {
        float4 pa[8];
        reduce_row(m, pa);
        finish(m, sum_row(pa));
      }
    }
    __syncwarp();
    cluster_sync_all();      // nobody leaves while a peer may still read its tile
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (tr && threadIdx.x == 0) {
    unsigned long long ns;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(ns));
    tr[7] = (long long)ns;
  }
  if (s_error) {
    // give copies and MMAs that may still be in flight time to land before shared memory and TMEM are released
    if (threadIdx.x == 0 && g.error_flag) atomicExch(g.error_flag, 1);
    const long long t0 = clock64();
    while ((unsigned long long)(clock64() - t0) < 200000000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(ncols) : "memory");
  }
}

// ---- persistent variant: one CTA per SM walks a list of tiles -------------------------------------------
// For GEMMs with many more tiles than SM slots (LM head: 1940 tiles, expert gate|up: 672).  The roles are the
// same, but the stage ring keeps running across tiles and the accumulator is double buffered in TMEM, so the
// weight stream of tile t + 1 flows while the epilogue warps drain tile t, and there is no partial last wave.
// Tile id -> (segment z, K range y, feature tile x), x fastest, so that CTAs that run at the same time share a
// segment's token rows in L2.  Tiles of empty segments are skipped by every role alike.
constexpr int PERSIST_STAGING = 32 * 1024;   // two staging tiles for the epilogue, in front of the stages

template <int MODE>
__global__ void __launch_bounds__(PERSIST_THREADS, 1)
gemm_tc_persist_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x, TcArgs g,
                       int tiles_x, int tiles_y, int tiles_total) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ unsigned long long bar_full[8], bar_empty[8], acc_full[2], acc_empty[2];
  __shared__ unsigned tmem_base_slot;
  __shared__ int s_error;
  __shared__ int s_maxcnt;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_trigger();
  pdl_wait();
  if (g.run_if && *reinterpret_cast<const volatile int*>(g.run_if) == 0) return;
  // the longest segment fixes the stage size for the whole launch (uniform over the CTA)
  int maxcnt = g.M;
  if (g.seg_cnt) {
    if (threadIdx.x == 0) {
      int mx = 0;
      const int nseg = tiles_total / (tiles_x * tiles_y);
      for (int z = 0; z < nseg; ++z) mx = max(mx, g.seg_cnt[z]);
      s_maxcnt = mx;
    }
    __syncthreads();
    maxcnt = s_maxcnt;
  }
  if (maxcnt > g.ntok) maxcnt = g.ntok;
  if (maxcnt <= 0 || (int)blockIdx.x >= tiles_total) return;     // uniform: nothing allocated yet
  const int max16 = (maxcnt + 15) & ~15;

  unsigned char* base = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  unsigned char* stages = base + PERSIST_STAGING;
  const unsigned w_bytes = BF * BK * 2;
  const unsigned stage_bytes = w_bytes + (unsigned)max16 * BK * 2;
  int S = (int)((g.smem_budget - PERSIST_STAGING) / stage_bytes);
  S = S > 8 ? 8 : S;
  const int nkb_total = (g.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) { mbar_init(&bar_full[s], 1); mbar_init(&bar_empty[s], 1); }
    mbar_init(&acc_full[0], 1); mbar_init(&acc_full[1], 1);
    mbar_init(&acc_empty[0], 4); mbar_init(&acc_empty[1], 4);     // one arrival per epilogue warp
    s_error = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  unsigned ncols_buf = 32;
  while (ncols_buf < (unsigned)((g.ntok + 31) & ~31)) ncols_buf <<= 1;
  const unsigned ncols = ncols_buf * 2;
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned tmem_base = tmem_base_slot;

  // every role walks the same tile list and derives the same per-tile numbers
  auto tile_info = [&](int id, int& z, int& y, int& n0, int& row0, int& cnt, int& kb0, int& nkb) {
    const int per_seg = tiles_x * tiles_y;
    z = id / per_seg;
    const int rem = id - z * per_seg;
    y = rem / tiles_x;
    n0 = (rem - y * tiles_x) * BF;
    row0 = 0; cnt = g.M;
    if (g.seg_cnt) { row0 = g.seg_off[z]; cnt = g.seg_cnt[z]; }
    if (cnt > g.ntok) cnt = g.ntok;
    kb0 = y * g.kb_per_split;
    nkb = nkb_total - kb0;
    if (nkb > g.kb_per_split) nkb = g.kb_per_split;
  };

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      for (int id = blockIdx.x; id < tiles_total && ok; id += gridDim.x) {
        int z, y, n0, row0, cnt, kb0, nkb;
        tile_info(id, z, y, n0, row0, cnt, kb0, nkb);
        if (cnt <= 0 || nkb <= 0) continue;
        const int cnt16 = (cnt + 15) & ~15;
        const int w_row = (int)((long long)(g.seg_w ? g.seg_w[z] : z) * g.w_rows_per_seg) + n0;
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const int s = it % S;
          if (!mbar_wait(&bar_empty[s], ((it / S) & 1) ^ 1)) { s_error = 1; ok = false; break; }
          unsigned char* st = stages + (size_t)s * stage_bytes;
          mbar_expect_tx(&bar_full[s], w_bytes + (unsigned)cnt16 * BK * 2);
          const int kx = (kb0 + kb) * BK;
          tma_load_2d(st, &tm_w, &bar_full[s], kx, w_row);
          for (int r16 = 0; r16 < cnt16; r16 += g.x_box)
            tma_load_2d(st + w_bytes + (size_t)r16 * BK * 2, &tm_x, &bar_full[s], kx, row0 + r16);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      int it = 0, t = 0;
      bool ok = true;
      for (int id = blockIdx.x; id < tiles_total && ok; id += gridDim.x) {
        int z, y, n0, row0, cnt, kb0, nkb;
        tile_info(id, z, y, n0, row0, cnt, kb0, nkb);
        if (cnt <= 0 || nkb <= 0) continue;
        const int cnt16 = (cnt + 15) & ~15;
        const int buf = t & 1;
        // the epilogue warps must have drained this accumulator (two tiles ago)
        if (!mbar_wait(&acc_empty[buf], ((t >> 1) & 1) ^ 1)) { s_error = 1; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(cnt16 >> 3) << 17) | ((unsigned)(BF >> 4) << 24);
        const unsigned acc = tmem_base + (unsigned)buf * ncols_buf;
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const int s = it % S;
          if (!mbar_wait(&bar_full[s], (it / S) & 1)) { s_error = 1; ok = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          unsigned char* st = stages + (size_t)s * stage_bytes;
          const unsigned long long da = umma_desc(st), db = umma_desc(st + w_bytes);
#pragma unroll
          for (int k4 = 0; k4 < BK / 16; ++k4)
            umma_bf16(acc, da + 2ull * k4, db + 2ull * k4, idesc, (kb | k4) != 0);
          umma_commit(&bar_empty[s]);
        }
        umma_commit(&acc_full[buf]);
        ++t;
      }
    }
  } else {
    // ---------------- epilogue: warps 2..5 ----------------
    const int q = warp & 3;
    const bool vec_ok = MODE == TC_PARTIAL
                            ? (g.N % 4 == 0 && ((uintptr_t)g.partial & 15) == 0)
                            : (g.ldc % 4 == 0 && g.N % 4 == 0 && ((uintptr_t)g.C & 15) == 0);
    const bool swi_ok = MODE == TC_SWIGLU && g.ldc % 4 == 0 && g.N % 4 == 0 && ((uintptr_t)g.C & 7) == 0;
    int t = 0, chunk_no = 0;
    for (int id = blockIdx.x; id < tiles_total; id += gridDim.x) {
      int z, y, n0, row0, cnt, kb0, nkb;
      tile_info(id, z, y, n0, row0, cnt, kb0, nkb);
      if (cnt <= 0 || nkb <= 0) continue;
      const int buf = t & 1;
      const bool acc_ok = mbar_wait(&acc_full[buf], (t >> 1) & 1);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (!acc_ok) s_error = 1;
      int go;
      {
        const int mine = (acc_ok && *(volatile int*)&s_error == 0) ? 1 : 0;
        asm volatile(
            "{\n\t.reg .pred p, q;\n\t"
            "setp.ne.b32 q, %1, 0;\n\t"
            "bar.red.and.pred p, 1, 128, q;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(go) : "r"(mine) : "memory");
      }
      if (!go) break;                    // uniform over the four warps
      const int nchunk = (cnt + 31) >> 5;
      if (MODE == TC_FILTER) {                 // the staging area in front of the stages holds the parked hits
        if (threadIdx.x == 64) *reinterpret_cast<int*>(base) = 0;
        asm volatile("bar.sync 2, 128;" ::: "memory");
      }
      for (int ch = 0; ch < nchunk; ++ch, ++chunk_no) {
        unsigned r[32];
        tmem_ld32(tmem_base + (unsigned)buf * ncols_buf + ((unsigned)(q * 32) << 16) + (unsigned)(ch * 32), r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (ch == nchunk - 1) {          // accumulator read out: hand the buffer back before the stores
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          __syncwarp();
          if (lane == 0) mbar_arrive(&acc_empty[buf]);
        }
        tc_epilogue_chunk<MODE>(g, r, base, ch, chunk_no & 1, 2, q, lane, n0, row0, cnt, y, vec_ok, swi_ok);
      }
      if (MODE == TC_FILTER) {
        asm volatile("bar.sync 2, 128;" ::: "memory");
        filter_flush(g, base, (int)threadIdx.x - 64, 128);
        asm volatile("bar.sync 2, 128;" ::: "memory");   // nobody parks the next tile's hits while these are read
      }
      ++t;
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (s_error) {
    if (threadIdx.x == 0 && g.error_flag) atomicExch(g.error_flag, 1);
    const long long t0 = clock64();
    while ((unsigned long long)(clock64() - t0) < 200000000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(ncols) : "memory");
  }
}

// A wait that nothing ends: one thread waits on an mbarrier no one arrives at, exactly as the GEMM's roles wait for a
// stage, and raises the error word when the limit runs out.  Exercises the time-out path without a fault anywhere.
__global__ void wait_probe_kernel(int* error_flag, long long* waited_cycles) {
  __shared__ unsigned long long bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    const long long t0 = clock64();
    const bool ok = mbar_wait(&bar, 0);
    if (waited_cycles) *waited_cycles = clock64() - t0;
    if (!ok && error_flag) atomicExch(error_flag, 1);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

// fp32 output [slices][rows][N] (row pitch ld, slice pitch slice_stride, in elements): box = 128 x 32 x 1, no swizzle
inline bool make_out_map(CUtensorMap* out, const void* ptr, long long N, long long rows, long long slices, long long ld,
                         long long slice_stride) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[3] = {(cuuint64_t)N, (cuuint64_t)rows, (cuuint64_t)slices};
  cuuint64_t strides[2] = {(cuuint64_t)ld * 4, (cuuint64_t)slice_stride * 4};
  cuuint32_t box[3] = {(cuuint32_t)BF, 32, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  return fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void*>(ptr), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// 2-D bf16 tensor [rows, K] with row pitch ld (elements); box = 64 x box_rows, 128-byte swizzle, zero fill
inline bool make_map(CUtensorMap* out, const void* ptr, long long rows, long long K, long long ld, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  return fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace tc_detail

struct TcPlan {
  int splits = 1;
  bool force_partial = false;    // write to the workspace even when one K range is enough
  int splits_used = 1;           // out: number of partial slices written
  float* partial = nullptr;      // caller-provided workspace for split-K partials
  long long rows_total = 0;      // rows addressed in C (all segments)
  int* error_flag = nullptr;
  long long* trace = nullptr;    // device buffer [CTAs][8] for phase stamps, or null
  // cluster split-K: the K ranges of a feature tile run as one thread-block cluster (at most 8 CTAs) that
  // reduces its partial tiles through distributed shared memory and applies the epilogue itself
  int cluster_mode = 0;          // 0: off, else tc_detail::TC_CL_STORE / TC_CL_SWIGLU / TC_CL_ADD / TC_CL_QKV
  float* resid = nullptr;        // TC_CL_ADD target (pitch g.ldc)
  tc_detail::TcRope rope = {};   // TC_CL_QKV
  const tc_detail::CandBuf* filter = nullptr;   // set: candidate-filter epilogue instead of a store (TC_FILTER)
  const int* run_if = nullptr;   // see TcArgs::run_if
  bool force_persist = false;    // walk the tiles with one CTA per SM whatever the shape (a flag-gated launch that
                                 // mostly returns at once should not schedule thousands of CTAs to do so)
};

// cluster split-K needs whole float4 groups per lane and, for the RoPE epilogue, heads that tile the 128 features
inline bool gemm_tc_cluster_supported(const GemmArgs& g, int mode, const tc_detail::TcRope* rope) {
  if (g.seg_cnt || g.nseg != 1 || g.N % 4 != 0) return false;
  if (mode == tc_detail::TC_CL_QKV) {
    if (!rope) return false;
    const int hd = rope->hd;
    return (hd == 32 || hd == 64 || hd == 128) && rope->ldq % 4 == 0;
  }
  return g.ldc % 4 == 0;
}

// read on every launch so that a test can switch it
inline int persist_level_env() { const char* e = getenv("VN_TC_PERSIST"); return e ? atoi(e) : -1; }

// Supported: bf16 operands, K-major, 16-byte aligned rows, tokens <= 256, A rows contiguous (no gather).
inline bool gemm_tc_supported(const GemmArgs& g) {
  return g.M >= 1 && g.M <= 256 && g.a_rows == nullptr && g.ldw_k == 1 && g.K % 8 == 0 && g.lda % 8 == 0 &&
         g.ldw % 8 == 0 && ((uintptr_t)g.A & 15) == 0 && ((uintptr_t)g.W & 15) == 0 &&
         (g.seg_cnt != nullptr || g.nseg == 1) && tc_detail::encode_fn() != nullptr;
}

// a_rows_total: number of valid rows behind g.A (rows beyond are zero-filled by TMA)
inline int32_t launch_gemm_tc(vn_ctx* ctx, const GemmArgs& g, long long a_rows_total, TcPlan& plan) {
  using namespace tc_detail;
  if (g.M <= 0 || g.N <= 0) return VN_OK;
  const int ntok = (g.M + 15) & ~15;
  CUtensorMap tm_w, tm_x;
  const long long w_rows = g.seg_cnt ? (long long)((g.seg_w ? g.n_w : g.nseg) - 1) * (g.w_stride / g.ldw) + g.N : g.N;
  if (!make_map(&tm_w, g.W, w_rows, g.K, g.ldw, BF) || !make_map(&tm_x, g.A, a_rows_total, g.K, g.lda, g.seg_cnt ? 16 : ntok))
    return vn_fail(ctx, VN_ERR_CUDA, "cuTensorMapEncodeTiled failed");
  TcArgs a = {};
  a.C = g.C; a.bias = g.bias; a.ldc = g.ldc; a.M = g.M; a.N = g.N; a.K = g.K; a.ntok = ntok;
  a.x_box = g.seg_cnt ? 16 : ntok;
  const size_t stage_bytes = (size_t)BF * BK * 2 + (size_t)ntok * BK * 2;
  const int nkb = (g.K + BK - 1) / BK;
  const int splits = std::max(1, std::min(plan.splits, nkb));
  a.kb_per_split = (nkb + splits - 1) / splits;
  // about 108 KB of stages per CTA so that two CTAs share an SM (one drains its accumulator while the other
  // streams); at least two stages of the largest token block, and no more than the k range needs
  // (a grid that leaves SMs idle anyway gives each CTA the whole SM: a k range of four or five blocks is then in
  // flight at once instead of waiting for a stage to come back)
  const long long ctas = (long long)ceil_div(g.N, BF) * ceil_div(nkb, a.kb_per_split) * g.nseg;
  static const bool wide_on = [] { const char* e = getenv("VN_TC_WIDE"); return !(e && e[0] == '0'); }();
  const size_t cap = (wide_on && ctas <= ctx->sm_count) ? 200 * 1024 : 108 * 1024;
  size_t budget = std::min<size_t>(cap, stage_bytes * 8);
  budget = std::min(budget, std::max<size_t>(2, a.kb_per_split) * stage_bytes);
  budget = std::max(budget, 2 * stage_bytes);
  budget = std::max<size_t>(budget, 64 * 1024);       // the epilogue stages four 16 KB tiles in the freed stage memory
  a.smem_budget = (unsigned)budget;
  a.epi = g.epi; a.c_bf16 = g.c_bf16;
  a.seg_off = g.seg_off; a.seg_cnt = g.seg_cnt;
  a.w_rows_per_seg = g.seg_cnt ? g.w_stride / g.ldw : 0;
  a.seg_w = g.seg_w;
  const int gy = ceil_div(nkb, a.kb_per_split);
  plan.splits_used = gy;
  a.partial = (gy > 1 || plan.force_partial) ? plan.partial : nullptr;
  a.partial_stride = plan.rows_total * (long long)g.N;
  a.error_flag = plan.error_flag;
  a.trace = plan.trace;
  a.resid = plan.resid;
  a.rope = plan.rope;
  a.run_if = plan.run_if;
  if (plan.filter) a.cand = *plan.filter;
  if (plan.cluster_mode) {
    if (gy > 8 || g.seg_cnt) return vn_fail(ctx, VN_ERR_INVALID, "cluster split-K: at most 8 K ranges, dense rows only");
    a.partial = nullptr;
    budget = std::max(budget, (size_t)((g.M + 31) / 32) * 32 * BF * 4);   // the whole partial tile is staged
    a.smem_budget = (unsigned)budget;
  }
  if (!plan.cluster_mode && (gy > 1 || plan.force_partial) && !plan.partial)
    return vn_fail(ctx, VN_ERR_INVALID, "split-K needs a workspace");
  const int mode = plan.cluster_mode ? plan.cluster_mode
                   : plan.filter ? TC_FILTER
                   : a.partial ? TC_PARTIAL : g.epi == EPI_SWIGLU ? TC_SWIGLU : g.epi == EPI_ADD ? TC_ADD : TC_STORE;
  // dense fp32 outputs leave through TMA stores (VN_TC_TMA_STORE=0: staged float4 stores instead)
  static const bool tma_store_on = [] { const char* e = getenv("VN_TC_TMA_STORE"); return !(e && e[0] == '0'); }();
  CUtensorMap tm_out = tm_x;      // placeholder when unused
  a.tma_out = 0; a.out_bufs = 1;
  if (tma_store_on && !g.seg_cnt && g.N >= BF && g.N % 4 == 0 && (mode == TC_PARTIAL || (mode == TC_STORE && !g.c_bf16))) {
    const bool part = mode == TC_PARTIAL;
    const float* optr = part ? a.partial : reinterpret_cast<const float*>(g.C);
    const long long old_ = part ? g.N : g.ldc;
    const long long slice = part ? a.partial_stride : (long long)g.M * old_;
    const long long rows = part ? plan.rows_total : g.M;
    if (((uintptr_t)optr & 15) == 0 && old_ % 4 == 0 && slice % 4 == 0 &&
        make_out_map(&tm_out, optr, g.N, rows, part ? gy : 1, old_, slice)) {
      const int per_group = (((g.M + 31) / 32) + 1) / 2;               // chunks the busier epilogue group drains
      budget = std::max<size_t>(budget, (size_t)std::min(per_group, 3) * 2 * 32 * BF * 4);
      a.smem_budget = (unsigned)budget;
      a.out_bufs = (int)std::min<size_t>(per_group, budget / (2 * 32 * BF * 4));
      a.tma_out = a.out_bufs >= 1 ? 1 : 0;
    }
  }
  const size_t smem = budget + 1024;
  static unsigned long long attr_set = 0;
  if (!((attr_set >> (ctx->device & 63)) & 1ull)) {
    VN_CUDA(ctx, cudaFuncSetAttribute(gemm_tc_kernel<TC_PARTIAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, 210 * 1024));
    VN_CUDA(ctx, cudaFuncSetAttribute(gemm_tc_kernel<TC_STORE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 210 * 1024));
    VN_CUDA(ctx, cudaFuncSetAttribute(gemm_tc_kernel<TC_SWIGLU>, cudaFuncAttributeMaxDynamicSharedMemorySize, 210 * 1024));
    VN_CUDA(ctx, cudaFuncSetAttribute(gemm_tc_kernel<TC_ADD>, cudaFuncAttributeMaxDynamicSharedMemorySize, 210 * 1024));
    VN_CUDA(ctx, cudaFuncSetAttribute(gemm_tc_kernel<TC_CL_STORE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 210 * 1024));
    VN_CUDA(ctx, cudaFuncSetAttribute(gemm_tc_kernel<TC_CL_SWIGLU>, cudaFuncAttributeMaxDynamicSharedMemorySize, 210 * 1024));
    VN_CUDA(ctx, cudaFuncSetAttribute(gemm_tc_kernel<TC_CL_ADD>, cudaFuncAttributeMaxDynamicSharedMemorySize, 210 * 1024));
    VN_CUDA(ctx, cudaFuncSetAttribute(gemm_tc_kernel<TC_CL_QKV>, cudaFuncAttributeMaxDynamicSharedMemorySize, 210 * 1024));
    VN_CUDA(ctx, cudaFuncSetAttribute(gemm_tc_kernel<TC_FILTER>, cudaFuncAttributeMaxDynamicSharedMemorySize, 210 * 1024));
    attr_set |= 1ull << (ctx->device & 63);
  }
  dim3 grid(ceil_div(g.N, BF), gy, g.nseg);
  const char* name = g.tag ? g.tag : "gemm_tc_kernel";
  // Persistent variant (one CTA per SM walks the tiles, accumulator double buffered).  VN_TC_PERSIST=0 never,
  // =1 for GEMMs with more tiles than two per SM, =2 for every GEMM it supports.  Measured on B200 it matches the
  // one-tile-per-CTA kernel within 3 % on the target's LM head and expert GEMMs (their limit is the rate at which
  // TMA delivers weight plus re-fetched token tiles, about 7.3 TB/s over all SMs), so by default it is used only
  // for short K ranges (below).
  const int persist_level = persist_level_env();
  const long long tiles_total = (long long)grid.x * grid.y * grid.z;
  // Unset (-1): only where a tile's K range is at most four blocks and there are more than two tiles per SM (the
  // draft model's LM head: 1,940 tiles of four k blocks), where the per-tile set-up is what the tile loop saves;
  // measured -15 us per round there, +24 us on the target's GEMMs when forced everywhere.
  const bool persist_auto = persist_level < 0 && a.kb_per_split <= 4 && tiles_total > 2ll * ctx->sm_count;
  if ((persist_level > 0 || persist_auto || plan.force_persist) && (mode == TC_STORE || mode == TC_SWIGLU || mode == TC_PARTIAL || mode == TC_FILTER) &&
      (persist_level >= 2 || plan.force_persist || tiles_total > 2ll * ctx->sm_count) && tiles_total < (1ll << 30)) {
    const size_t stages_max = (216 * 1024 - PERSIST_STAGING) / stage_bytes;
    if (stages_max >= 2) {
      const size_t pbudget = PERSIST_STAGING + std::min<size_t>(8, stages_max) * stage_bytes;
      a.smem_budget = (unsigned)pbudget;
      const size_t psmem = pbudget + 1024;
      static unsigned long long pattr_set = 0;
      if (!((pattr_set >> (ctx->device & 63)) & 1ull)) {
        VN_CUDA(ctx, cudaFuncSetAttribute(gemm_tc_persist_kernel<TC_PARTIAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024));
        VN_CUDA(ctx, cudaFuncSetAttribute(gemm_tc_persist_kernel<TC_STORE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024));
        VN_CUDA(ctx, cudaFuncSetAttribute(gemm_tc_persist_kernel<TC_SWIGLU>, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024));
        VN_CUDA(ctx, cudaFuncSetAttribute(gemm_tc_persist_kernel<TC_FILTER>, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024));
        pattr_set |= 1ull << (ctx->device & 63);
      }
      const int pgrid = (int)std::min<long long>(tiles_total, ctx->sm_count);
      const int tx = (int)grid.x, ty = (int)grid.y, tt = (int)tiles_total;
      if (mode == TC_STORE)
        VN_LAUNCH_PDL_LEVEL(ctx, 1, name, gemm_tc_persist_kernel<TC_STORE>, pgrid, PERSIST_THREADS, psmem, tm_w, tm_x, a, tx, ty, tt);
      else if (mode == TC_SWIGLU)
        VN_LAUNCH_PDL_LEVEL(ctx, 1, name, gemm_tc_persist_kernel<TC_SWIGLU>, pgrid, PERSIST_THREADS, psmem, tm_w, tm_x, a, tx, ty, tt);
      else if (mode == TC_FILTER)
        VN_LAUNCH_PDL_LEVEL(ctx, 1, name, gemm_tc_persist_kernel<TC_FILTER>, pgrid, PERSIST_THREADS, psmem, tm_w, tm_x, a, tx, ty, tt);
      else
        VN_LAUNCH_PDL_LEVEL(ctx, 1, name, gemm_tc_persist_kernel<TC_PARTIAL>, pgrid, PERSIST_THREADS, psmem, tm_w, tm_x, a, tx, ty, tt);
      return VN_OK;
    }
  }
  switch (mode) {
    case TC_PARTIAL: VN_LAUNCH_PDL_LEVEL(ctx, 1, name, gemm_tc_kernel<TC_PARTIAL>, grid, TC_THREADS, smem, tm_w, tm_x, tm_out, a); break;
    case TC_SWIGLU:  VN_LAUNCH_PDL_LEVEL(ctx, 1, name, gemm_tc_kernel<TC_SWIGLU>, grid, TC_THREADS, smem, tm_w, tm_x, tm_out, a); break;
    case TC_ADD:     VN_LAUNCH_PDL_LEVEL(ctx, 1, name, gemm_tc_kernel<TC_ADD>, grid, TC_THREADS, smem, tm_w, tm_x, tm_out, a); break;
    case TC_FILTER:  VN_LAUNCH_PDL_LEVEL(ctx, 1, name, gemm_tc_kernel<TC_FILTER>, grid, TC_THREADS, smem, tm_w, tm_x, tm_out, a); break;
    case TC_CL_STORE:  VN_LAUNCH_CLUSTER(ctx, 1, gy, name, gemm_tc_kernel<TC_CL_STORE>, grid, TC_THREADS, smem, tm_w, tm_x, tm_out, a); break;
    case TC_CL_SWIGLU: VN_LAUNCH_CLUSTER(ctx, 1, gy, name, gemm_tc_kernel<TC_CL_SWIGLU>, grid, TC_THREADS, smem, tm_w, tm_x, tm_out, a); break;
    case TC_CL_ADD:    VN_LAUNCH_CLUSTER(ctx, 1, gy, name, gemm_tc_kernel<TC_CL_ADD>, grid, TC_THREADS, smem, tm_w, tm_x, tm_out, a); break;
    case TC_CL_QKV:    VN_LAUNCH_CLUSTER(ctx, 1, gy, name, gemm_tc_kernel<TC_CL_QKV>, grid, TC_THREADS, smem, tm_w, tm_x, tm_out, a); break;
    default:         VN_LAUNCH_PDL_LEVEL(ctx, 1, name, gemm_tc_kernel<TC_STORE>, grid, TC_THREADS, smem, tm_w, tm_x, tm_out, a); break;
  }
  return VN_OK;
}
