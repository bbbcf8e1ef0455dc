// bf16 tensor-core GEMM (mma.sync m16n8k16, fp32 accumulate) with a cp.async pipeline.
// C[M,N] = A[M,K] * W[N,K]^T; both operands K-major, which is the row.col fragment layout.
// CTA tile BM x 64 x 64 (BM = 64 or 128), 4-stage pipeline, warps of 32 x 32.
// The m-tile index varies fastest over the grid so that CTAs sharing a weight tile run together and the
// weight tile crosses HBM once.
#pragma once
#include "gemm.cuh"

namespace mma_detail {

constexpr int BN = 64, BK = 64, STAGES = 4, PAD = 8;
constexpr int LDS = BK + PAD;  // shared-memory row stride in elements (144 B: conflict-free ldmatrix)

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float* c, const unsigned* a, const unsigned* b) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

template <int BM>
__global__ void __launch_bounds__(BM * 2) gemm_mma_kernel(GemmArgs g) {
  constexpr int THREADS = BM * 2;            // BM/32 x 2 warps
  constexpr int WARPS_N = 2;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* sA = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __nv_bfloat16* sW = sA + (size_t)STAGES * BM * LDS;
  const int z = blockIdx.z;
  int row0 = 0, Mz = g.M;
  if (g.seg_cnt) { row0 = g.seg_off[z]; Mz = g.seg_cnt[z]; }
  const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;
  if (m0 >= Mz) return;
  const __nv_bfloat16* A = reinterpret_cast<const __nv_bfloat16*>(g.A);
  const __nv_bfloat16* W = reinterpret_cast<const __nv_bfloat16*>(g.W) + (long long)z * g.w_stride;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int wm = warp / WARPS_N, wn = warp % WARPS_N;
  const int KT = (g.K + BK - 1) / BK;

  // per-thread load assignments: 8 chunks of 16 B per row of 64 elements
  constexpr int A_ITERS = BM * 8 / THREADS;  // = 4
  constexpr int W_ITERS = BN * 8 / THREADS;  // 4 (BM 64) or 2 (BM 128)
  const __nv_bfloat16* a_src[A_ITERS];
  bool a_ok[A_ITERS];
#pragma unroll
  for (int i = 0; i < A_ITERS; ++i) {
    const int c = tid + i * THREADS, r = c >> 3;
    a_ok[i] = (m0 + r) < Mz;
    long long ar = 0;
    if (a_ok[i]) ar = g.a_rows ? g.a_rows[row0 + m0 + r] : (long long)(row0 + m0 + r);
    a_src[i] = A + ar * g.lda + (c & 7) * 8;
  }
  auto load_stage = [&](int stage, int kt) {
    const int k0 = kt * BK;
#pragma unroll
    for (int i = 0; i < A_ITERS; ++i) {
      const int c = tid + i * THREADS, r = c >> 3, kc = (c & 7) * 8;
      const bool ok = a_ok[i] && (k0 + kc) < g.K;
      cp_async16(sA + ((size_t)stage * BM + r) * LDS + kc, ok ? (const void*)(a_src[i] + k0) : (const void*)A, ok);
    }
#pragma unroll
    for (int i = 0; i < W_ITERS; ++i) {
      const int c = tid + i * THREADS, r = c >> 3, kc = (c & 7) * 8;
      const bool ok = (n0 + r) < g.N && (k0 + kc) < g.K;
      const __nv_bfloat16* src = W + (long long)(n0 + r) * g.ldw + k0 + kc;
      cp_async16(sW + ((size_t)stage * BN + r) * LDS + kc, ok ? (const void*)src : (const void*)W, ok);
    }
  };

  float acc[2][4][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.f;

#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < KT) load_stage(s, s);
    cp_async_commit();
  }
  for (int kt = 0; kt < KT; ++kt) {
    cp_async_wait<STAGES - 2>();
    __syncthreads();
    const int nxt = kt + STAGES - 1;
    if (nxt < KT) load_stage(nxt % STAGES, nxt);
    cp_async_commit();
    const __nv_bfloat16* a_st = sA + (size_t)(kt % STAGES) * BM * LDS;
    const __nv_bfloat16* w_st = sW + (size_t)(kt % STAGES) * BN * LDS;
#pragma unroll
    for (int kk = 0; kk < BK; kk += 16) {
      unsigned af[2][4], bf[4][2];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int r = wm * 32 + i * 16 + (lane & 15);
        const int c = kk + ((lane >> 4) << 3);
        ldmatrix_x4(af[i][0], af[i][1], af[i][2], af[i][3], a_st + (size_t)r * LDS + c);
      }
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        // two n8 tiles per ldmatrix.x4: rows n (8 + 8), k halves
        const int r = wn * 32 + j * 16 + (lane & 7) + ((lane >> 4) << 3);
        const int c = kk + (((lane >> 3) & 1) << 3);
        unsigned r0, r1, r2, r3;
        ldmatrix_x4(r0, r1, r2, r3, w_st + (size_t)r * LDS + c);
        bf[j * 2][0] = r0; bf[j * 2][1] = r1; bf[j * 2 + 1][0] = r2; bf[j * 2 + 1][1] = r3;
      }
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) mma_bf16(acc[i][j], af[i], bf[j]);
    }
  }
  cp_async_wait<0>();

  // epilogue: thread holds rows (lane/4) and (lane/4 + 8), columns 2*(lane%4) and +1 of every 16x8 tile
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int m = m0 + wm * 32 + i * 16 + (lane >> 2) + half * 8;
      if (m >= Mz) continue;
      const long long crow = (long long)(row0 + m);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int n = n0 + wn * 32 + j * 8 + (lane & 3) * 2;
        const float v0 = acc[i][j][half * 2], v1 = acc[i][j][half * 2 + 1];
        if (g.epi == EPI_SWIGLU) {
          if (n + 1 < g.N) store_out<float>(g.C, crow * g.ldc + (n >> 1), silu_ref(v0) * v1, g.c_bf16);
        } else if (g.epi == EPI_ADD) {
          float* c = reinterpret_cast<float*>(g.C) + crow * g.ldc + n;
          if (n < g.N) c[0] += v0;
          if (n + 1 < g.N) c[1] += v1;
        } else {
          if (n < g.N) store_out<float>(g.C, crow * g.ldc + n, v0 + (g.bias ? g.bias[n] : 0.f), g.c_bf16);
          if (n + 1 < g.N) store_out<float>(g.C, crow * g.ldc + n + 1, v1 + (g.bias ? g.bias[n + 1] : 0.f), g.c_bf16);
        }
      }
    }
}

}  // namespace mma_detail

inline bool gemm_mma_supported(const GemmArgs& g) {
  return g.K % 8 == 0 && g.lda % 8 == 0 && g.ldw % 8 == 0 && g.ldw_k == 1 && g.w_stride % 8 == 0 &&
         ((uintptr_t)g.A & 15) == 0 && ((uintptr_t)g.W & 15) == 0 && (g.seg_cnt != nullptr || g.nseg == 1);
}

inline int32_t launch_gemm_mma(vn_ctx* ctx, const GemmArgs& g) {
  using namespace mma_detail;
  if (g.M <= 0 || g.N <= 0) return VN_OK;
  const bool big = g.M > 64;
  const int BM = big ? 128 : 64;
  const size_t smem = (size_t)STAGES * (BM + BN) * LDS * sizeof(__nv_bfloat16);
  static unsigned long long attr_set = 0;  // one bit per device
  if (!((attr_set >> (ctx->device & 63)) & 1ull)) {
    VN_CUDA(ctx, cudaFuncSetAttribute(gemm_mma_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)((size_t)STAGES * (64 + BN) * LDS * 2)));
    VN_CUDA(ctx, cudaFuncSetAttribute(gemm_mma_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)((size_t)STAGES * (128 + BN) * LDS * 2)));
    attr_set |= 1ull << (ctx->device & 63);
  }
  dim3 grid(ceil_div(g.M, BM), ceil_div(g.N, BN), g.nseg);
  if (big) VN_LAUNCH_NAMED(ctx, g.tag ? g.tag : "gemm_mma_kernel<128>", gemm_mma_kernel<128>, grid, 256, smem, g);
  else VN_LAUNCH_NAMED(ctx, g.tag ? g.tag : "gemm_mma_kernel<64>", gemm_mma_kernel<64>, grid, 128, smem, g);
  return VN_OK;
}
