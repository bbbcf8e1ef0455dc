// Weight-only quantised weight-streaming GEMM on tcgen05: the INT8 / INT4 weight tile travels as raw bytes
// (verse_torch/quantize.py:187-258 layouts: one byte per weight, or two's-complement nibbles with the even index
// in the low nibble), is turned into the bf16, 128-byte-swizzled UMMA operand inside shared memory by four
// "transform" warps, and then takes the same path as the dense kernel in gemm_tc.cuh (TMEM accumulator, split-K
// partial or fused epilogues).  HBM and L2 see one half to one quarter of the bf16 weight bytes.
//
//   QMODE 1  INT8, one fp32 scale per output row: applied to the fp32 accumulator in the epilogue (exact:
//            small integers are exact in bf16, so the MMA computes x @ q^T in bf16 x bf16 -> fp32)
//   QMODE 2  INT4, one fp32 scale per output row: the same
//   QMODE 3  INT4, one scale per 128 input features: one TMEM accumulator cannot hold differently scaled k groups,
//            so the group's scale is folded into the operand, q * s rounded to bf16 (the scales are
//            bf16-representable, the product has up to 11 significant bits: relative error <= 2^-9 per weight,
//            an order of magnitude below the 4-bit quantisation step it rides on)
//
// Roles of the 10 warps: 0 TMA producer (raw weight tile + token tile), 1 MMA issuer, 2..5 transform warps during
// the main loop and epilogue group 0 afterwards, 6..9 epilogue group 1.  Per ring stage: bar_full (TMA bytes
// landed), bar_conv (operand converted, one arrival per transform warp), bar_empty (the MMAs have read the stage).
// The raw bytes land in the tail of the stage's own operand slot; the transform warps read all of them into
// registers, meet at a named barrier, and only then write the operand over them, so a stage costs no extra memory.
#pragma once
#include "gemm_tc.cuh"

namespace tc_detail {

// four biased bytes (value + 128 each) -> two bf16x2 words holding the exact integers
__device__ __forceinline__ void i8x4_to_bf16(unsigned x, unsigned& o0, unsigned& o1) {
  // 0x4B000000 | u is the float 8388608 + u; subtracting 8388736 leaves u - 128 exactly, an integer that bf16
  // holds exactly, so keeping the upper 16 bits of the float is a lossless conversion
  const float f0 = __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7540)) - 8388736.0f;
  const float f1 = __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7541)) - 8388736.0f;
  const float f2 = __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7542)) - 8388736.0f;
  const float f3 = __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7543)) - 8388736.0f;
  o0 = __byte_perm(__float_as_uint(f0), __float_as_uint(f1), 0x7632);
  o1 = __byte_perm(__float_as_uint(f2), __float_as_uint(f3), 0x7632);
}

// eight biased nibbles (value + 8 each, element e in bits 4e..4e+3) -> four bf16x2 words; SCALED: times sc, rounded
template <bool SCALED>
__device__ __forceinline__ void i4x8_to_bf16(unsigned x, float sc, unsigned (&o)[4]) {
#pragma unroll
  for (int h = 0; h < 4; ++h) {
    const float a = __uint_as_float(0x4B000000u | ((x >> (8 * h)) & 0xfu)) - 8388616.0f;
    const float b = __uint_as_float(0x4B000000u | ((x >> (8 * h + 4)) & 0xfu)) - 8388616.0f;
    if (SCALED) {
      __nv_bfloat162 r = __floats2bfloat162_rn(a * sc, b * sc);
      o[h] = *reinterpret_cast<unsigned*>(&r);
    } else {
      o[h] = __byte_perm(__float_as_uint(a), __float_as_uint(b), 0x7632);
    }
  }
}

template <int QMODE, int MODE>
__global__ void __launch_bounds__(TC_THREADS, 2)
gemm_tcq_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                const __grid_constant__ CUtensorMap tm_out, TcArgs g, const float* __restrict__ w_scale,
                long long ws_stride) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ unsigned long long bar_full[8], bar_empty[8], bar_conv[8], bar_acc;
  __shared__ unsigned tmem_base_slot;
  __shared__ int s_error;
  constexpr int RAW_ROW = QMODE == 1 ? BK : BK / 2;           // raw bytes per weight row and k block
  constexpr unsigned RAW_BYTES = BF * RAW_ROW;                // 8 KB or 4 KB
  constexpr int RAW_WORDS = QMODE == 1 ? 2 : 1;               // 32-bit words behind one 16-byte output chunk

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int z = blockIdx.z;
  int row0 = 0, cnt = g.M;
  pdl_trigger();
  // segment sizes are written by the routing kernels before this one; a dense block waits later, once its first
  // weight tiles are on their way (weights and scales never change)
  if (g.seg_cnt) { pdl_wait(); row0 = g.seg_off[z]; cnt = g.seg_cnt[z]; }
  if (cnt > g.ntok) cnt = g.ntok;
  const int cnt16 = (cnt + 15) & ~15;
  const int n0 = blockIdx.x * BF;
  const int nkb_total = (g.K + BK - 1) / BK;
  const int kb0 = blockIdx.y * g.kb_per_split;
  int nkb = nkb_total - kb0;
  if (nkb > g.kb_per_split) nkb = g.kb_per_split;
  if (cnt <= 0 || nkb <= 0) return;                            // uniform, before any barrier or TMEM allocation

  unsigned char* base = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const unsigned w_bytes = BF * BK * 2, x_bytes = (unsigned)cnt16 * BK * 2;
  const unsigned stage_bytes = w_bytes + x_bytes;
  int S = (int)(g.smem_budget / stage_bytes);
  S = S > 8 ? 8 : S;
  S = S > nkb ? (nkb < 2 ? 2 : nkb) : S;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) { mbar_init(&bar_full[s], 1); mbar_init(&bar_empty[s], 1); mbar_init(&bar_conv[s], 4); }
    mbar_init(&bar_acc, 1);
    s_error = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
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

  if (warp == 0) {
    // ---------------- TMA producer: raw weight bytes into the tail of the operand slot, token rows behind it
    if (lane == 0) {
      const int w_row = (int)((long long)z * g.w_rows_per_seg) + n0;
      int kb_first = 0;
      if (!g.seg_cnt) {
        const int npre = nkb < S ? nkb : S;
        for (int kb = 0; kb < npre; ++kb) {
          mbar_expect_tx_only(&bar_full[kb], RAW_BYTES);
          tma_load_2d(base + (size_t)kb * stage_bytes + (w_bytes - RAW_BYTES), &tm_w, &bar_full[kb], (kb0 + kb) * RAW_ROW, w_row);
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
        mbar_expect_tx(&bar_full[s], RAW_BYTES + (unsigned)cnt16 * BK * 2);
        tma_load_2d(st + (w_bytes - RAW_BYTES), &tm_w, &bar_full[s], (kb0 + kb) * RAW_ROW, w_row);
        const int kx = (kb0 + kb) * BK;
        for (int r16 = 0; r16 < cnt16; r16 += g.x_box)
          tma_load_2d(st + w_bytes + (size_t)r16 * BK * 2, &tm_x, &bar_full[s], kx, row0 + r16);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(cnt16 >> 3) << 17) | ((unsigned)(BF >> 4) << 24);
      for (int kb = 0; kb < nkb; ++kb) {
        const int s = kb % S;
        const unsigned ph = (kb / S) & 1;
        // converted implies landed; the wait on bar_full makes the TMA-written token rows visible to this thread
        if (!mbar_wait(&bar_conv[s], ph) || !mbar_wait(&bar_full[s], ph)) { s_error = 1; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        unsigned char* st = base + (size_t)s * stage_bytes;
        const unsigned long long da = umma_desc(st), db = umma_desc(st + w_bytes);
#pragma unroll
        for (int k4 = 0; k4 < BK / 16; ++k4)
          umma_bf16(tmem_base, da + 2ull * k4, db + 2ull * k4, idesc, (kb | k4) != 0);
        umma_commit(&bar_empty[s]);
      }
      umma_commit(&bar_acc);
    }
  } else {
    const int q = warp & 3;
    const int grp = (warp - 2) >> 2;
    if (grp == 0) {
      // ---------------- transform: item = i * 128 + t covers weight row item / 8, 16-byte output chunk item % 8.
      // A warp reads 128 or 256 contiguous raw bytes per step and its eight-lane groups write one whole swizzled
      // row each: no bank conflicts on either side.
      const int t = threadIdx.x - 64;                          // 0..127
      const int c = t & 7;
      const int groups = (g.K + 127) / 128;
      const float* sbase = w_scale + (long long)z * ws_stride;
      float sc[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) sc[i] = 1.0f;
      for (int kb = 0; kb < nkb; ++kb) {
        const int s = kb % S;
        if (QMODE == 3 && (kb == 0 || ((kb0 + kb) & 1) == 0)) {  // a 128-wide group spans two k blocks
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int n = n0 + i * 16 + (t >> 3);
            sc[i] = n < g.N ? sbase[(long long)n * groups + ((kb0 + kb) >> 1)] : 0.f;
          }
        }
        const int ok = mbar_wait(&bar_full[s], (kb / S) & 1) ? 1 : 0;
        unsigned char* st = base + (size_t)s * stage_bytes;
        const unsigned* raw = reinterpret_cast<const unsigned*>(st + (w_bytes - RAW_BYTES));
        unsigned v[8][RAW_WORDS];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          if (QMODE == 1) {
            const uint2 w2 = ok ? reinterpret_cast<const uint2*>(raw)[i * 128 + t] : make_uint2(0u, 0u);
            v[i][0] = w2.x; v[i][RAW_WORDS - 1] = w2.y;
          } else {
            v[i][0] = ok ? raw[i * 128 + t] : 0u;
          }
        }
        // every raw byte is in registers before any operand byte is written over it; the same barrier carries
        // the vote, so that the four warps leave the loop together
        int all_ok;
        asm volatile(
            "{\n\t.reg .pred p, q;\n\t"
            "setp.ne.b32 q, %1, 0;\n\t"
            "bar.red.and.pred p, 4, 128, q;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(all_ok) : "r"(ok) : "memory");
        if (!all_ok) { s_error = 1; break; }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int r = i * 16 + (t >> 3);
          unsigned o[4];
          if (QMODE == 1) {
            i8x4_to_bf16(v[i][0] ^ 0x80808080u, o[0], o[1]);
            i8x4_to_bf16(v[i][RAW_WORDS - 1] ^ 0x80808080u, o[2], o[3]);
          } else {
            i4x8_to_bf16<QMODE == 3>(v[i][0] ^ 0x88888888u, sc[i], o);
          }
          *reinterpret_cast<uint4*>(st + r * 128 + ((c ^ (r & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic writes -> tensor-core reads
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar_conv[s]);
      }
      __syncwarp();
    }
    // ---------------- epilogue (both groups) ----------------
    const int f = q * 32 + lane;
    if (!g.seg_cnt) pdl_wait();
    const bool acc_ok = mbar_wait(&bar_acc, 0);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (!acc_ok) s_error = 1;
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
      float rs = 1.0f;                                          // per output row (QMODE 1, 2)
      if (QMODE != 3) rs = (n0 + f < g.N) ? w_scale[(long long)z * ws_stride + n0 + f] : 0.f;
      const int nchunk = (cnt + 31) >> 5;
      const bool vec_ok = MODE == TC_PARTIAL
                              ? (g.N % 4 == 0 && ((uintptr_t)g.partial & 15) == 0)
                              : (g.ldc % 4 == 0 && g.N % 4 == 0 && ((uintptr_t)g.C & 15) == 0);
      const bool swi_ok = MODE == TC_SWIGLU && g.ldc % 4 == 0 && g.N % 4 == 0 && ((uintptr_t)g.C & 7) == 0;
      const bool tma_out = (MODE == TC_PARTIAL || MODE == TC_STORE) && g.tma_out;   // uniform over the CTA
      const bool issuer = ((warp - 2) & 3) == 0 && lane == 0;                        // one thread per group
      for (int ch = grp; ch < nchunk; ch += 2) {
        unsigned r[32];
        tmem_ld32(tmem_base + ((unsigned)(q * 32) << 16) + (unsigned)(ch * 32), r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (tma_out) {
          // scaled registers -> a 32 x 128 fp32 tile in the freed stage memory -> one asynchronous tensor store
          const int jb = ch >> 1;
          float* tile = reinterpret_cast<float*>(base + ((size_t)grp * g.out_bufs + (jb % g.out_bufs)) * (32 * BF * 4));
          if (jb >= g.out_bufs) {           // the tile is being reused: its earlier store must have read it
            if (issuer) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
            asm volatile("bar.sync %0, 128;" ::"r"(2 + grp) : "memory");
          }
#pragma unroll
          for (int i = 0; i < 32; ++i) tile[i * BF + f] = __uint_as_float(r[i]) * rs;
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          asm volatile("bar.sync %0, 128;" ::"r"(2 + grp) : "memory");
          if (issuer) {
            tma_store_3d(&tm_out, tile, n0, row0 + ch * 32, MODE == TC_PARTIAL ? (int)blockIdx.y : 0);
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
        } else {
          if (QMODE != 3) {
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * rs);
          }
          tc_epilogue_chunk<MODE>(g, r, base + grp * (32 * 1024), ch, (ch >> 1) & 1, 2 + grp, q, lane, n0, row0, cnt,
                                  (int)blockIdx.y, vec_ok, swi_ok);
        }
      }
      // the staging tiles must have been read before the CTA gives its shared memory back
      if (tma_out && issuer) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
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

// raw weight bytes [rows, row_bytes]: box = (64 or 32 bytes) x 128 rows, no swizzle, zero fill
inline bool make_raw_map(CUtensorMap* out, const void* ptr, long long rows, long long row_bytes, int box_bytes) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {(cuuint64_t)row_bytes, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
  cuuint32_t box[2] = {(cuuint32_t)box_bytes, (cuuint32_t)BF};
  cuuint32_t estr[2] = {1, 1};
  return fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace tc_detail

// bf16 activations, quantised weights (g.wq 1..3) stored densely ([N, K] bytes or nibbles), K a multiple of 64
inline bool gemm_tcq_supported(const GemmArgs& g) {
  const long long row_bytes = g.wq == 1 ? g.ldw : g.ldw / 2;
  return g.wq >= 1 && g.wq <= 3 && g.M >= 1 && g.M <= 256 && g.a_rows == nullptr && g.ldw_k == 1 && g.K % 64 == 0 &&
         g.ldw == g.K && g.lda % 8 == 0 && row_bytes % 16 == 0 && ((uintptr_t)g.A & 15) == 0 &&
         ((uintptr_t)g.W & 15) == 0 && g.w_scale != nullptr && g.bias == nullptr && g.epi != EPI_ADD &&
         (g.seg_cnt != nullptr || g.nseg == 1) && tc_detail::encode_fn() != nullptr;
}

template <int QMODE>
inline int32_t launch_gemm_tcq_mode(vn_ctx* ctx, const GemmArgs& g, long long a_rows_total, TcPlan& plan) {
  using namespace tc_detail;
  const int ntok = (g.M + 15) & ~15;
  constexpr int RAW_ROW = QMODE == 1 ? BK : BK / 2;
  const long long row_bytes = QMODE == 1 ? g.K : g.K / 2;
  const long long seg_rows = g.seg_cnt ? (g.w_stride / g.ldw) : 0;
  const long long w_rows = g.seg_cnt ? (long long)(g.nseg - 1) * seg_rows + g.N : g.N;
  CUtensorMap tm_w, tm_x;
  if (!make_raw_map(&tm_w, g.W, w_rows, row_bytes, RAW_ROW) ||
      !make_map(&tm_x, g.A, a_rows_total, g.K, g.lda, g.seg_cnt ? 16 : ntok))
    return vn_fail(ctx, VN_ERR_CUDA, "cuTensorMapEncodeTiled failed");
  TcArgs a = {};
  a.C = g.C; a.bias = nullptr; a.ldc = g.ldc; a.M = g.M; a.N = g.N; a.K = g.K; a.ntok = ntok;
  a.x_box = g.seg_cnt ? 16 : ntok;
  const size_t stage_bytes = (size_t)BF * BK * 2 + (size_t)ntok * BK * 2;
  const int nkb = (g.K + BK - 1) / BK;
  const int splits = std::max(1, std::min(plan.splits, nkb));
  a.kb_per_split = (nkb + splits - 1) / splits;
  // as in the dense kernel: about 108 KB of stages so that two CTAs share an SM, never less than the 64 KB the
  // epilogue's staging tiles take in the freed stage memory
  // (a grid that leaves SMs idle anyway gives each CTA the whole SM: a k range of four or five blocks is then in
  // flight at once instead of waiting for a stage to come back)
  const long long ctas = (long long)ceil_div(g.N, BF) * ceil_div(nkb, a.kb_per_split) * g.nseg;
  static const bool wide_on = [] { const char* e = getenv("VN_TC_WIDE"); return !(e && e[0] == '0'); }();
  const size_t cap = (wide_on && ctas <= ctx->sm_count) ? 200 * 1024 : 108 * 1024;
  size_t budget = std::min<size_t>(cap, stage_bytes * 8);
  budget = std::min(budget, std::max<size_t>(2, a.kb_per_split) * stage_bytes);
  budget = std::max(budget, 2 * stage_bytes);
  budget = std::max<size_t>(budget, 64 * 1024);
  a.smem_budget = (unsigned)budget;
  a.epi = g.epi; a.c_bf16 = g.c_bf16;
  a.seg_off = g.seg_off; a.seg_cnt = g.seg_cnt;
  a.w_rows_per_seg = seg_rows;
  const int gy = ceil_div(nkb, a.kb_per_split);
  plan.splits_used = gy;
  a.partial = (gy > 1 || plan.force_partial) ? plan.partial : nullptr;
  a.partial_stride = plan.rows_total * (long long)g.N;
  a.error_flag = plan.error_flag;
  if ((gy > 1 || plan.force_partial) && !plan.partial) return vn_fail(ctx, VN_ERR_INVALID, "split-K needs a workspace");
  const int mode = a.partial ? TC_PARTIAL : g.epi == EPI_SWIGLU ? TC_SWIGLU : TC_STORE;
  // dense fp32 outputs leave through TMA stores, as in the dense kernel (VN_TC_TMA_STORE=0: staged float4 stores)
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
    VN_CUDA(ctx, cudaFuncSetAttribute(gemm_tcq_kernel<QMODE, TC_PARTIAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, 210 * 1024));
    VN_CUDA(ctx, cudaFuncSetAttribute(gemm_tcq_kernel<QMODE, TC_STORE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 210 * 1024));
    VN_CUDA(ctx, cudaFuncSetAttribute(gemm_tcq_kernel<QMODE, TC_SWIGLU>, cudaFuncAttributeMaxDynamicSharedMemorySize, 210 * 1024));
    attr_set |= 1ull << (ctx->device & 63);
  }
  dim3 grid(ceil_div(g.N, BF), gy, g.nseg);
  const char* name = g.tag ? g.tag : "gemm_tcq_kernel";
  if (mode == TC_PARTIAL)
    VN_LAUNCH_PDL_LEVEL(ctx, 1, name, (gemm_tcq_kernel<QMODE, TC_PARTIAL>), grid, TC_THREADS, smem, tm_w, tm_x, tm_out, a, g.w_scale, g.ws_stride);
  else if (mode == TC_SWIGLU)
    VN_LAUNCH_PDL_LEVEL(ctx, 1, name, (gemm_tcq_kernel<QMODE, TC_SWIGLU>), grid, TC_THREADS, smem, tm_w, tm_x, tm_out, a, g.w_scale, g.ws_stride);
  else
    VN_LAUNCH_PDL_LEVEL(ctx, 1, name, (gemm_tcq_kernel<QMODE, TC_STORE>), grid, TC_THREADS, smem, tm_w, tm_x, tm_out, a, g.w_scale, g.ws_stride);
  return VN_OK;
}

// a_rows_total: number of valid rows behind g.A (rows beyond are zero-filled by TMA)
inline int32_t launch_gemm_tcq(vn_ctx* ctx, const GemmArgs& g, long long a_rows_total, TcPlan& plan) {
  if (g.M <= 0 || g.N <= 0) return VN_OK;
  if (!gemm_tcq_supported(g)) return vn_fail(ctx, VN_ERR_UNSUPPORTED, "quantised tcgen05 GEMM: shape K=%d unsupported", g.K);
  if (g.wq == 1) return launch_gemm_tcq_mode<1>(ctx, g, a_rows_total, plan);
  if (g.wq == 2) return launch_gemm_tcq_mode<2>(ctx, g, a_rows_total, plan);
  return launch_gemm_tcq_mode<3>(ctx, g, a_rows_total, plan);
}
