// GEMM kernels: C[M,N] = A[M,K] * W[N,K]^T (weights row-major (out, in) as in the reference's Linear).
#pragma once
#include "common.cuh"

enum GemmEpilogue {
  EPI_STORE = 0,    // C = acc (+ bias)
  EPI_ADD = 1,      // C += acc              (residual stream, fp32)
  EPI_SWIGLU = 2    // out[m, n/2] = silu(acc[m, n]) * acc[m, n+1], n even (gate / up rows interleaved in W)
};

struct GemmArgs {
  const void* A = nullptr;    // [rows, K]
  const void* W = nullptr;    // [N, K] (per segment: + z * w_stride)
  void* C = nullptr;          // fp32 or bf16 [rows, N] (EPI_SWIGLU: [rows, N/2])
  const float* bias = nullptr;
  long long lda = 0, ldw = 0, ldc = 0;
  int M = 0, N = 0, K = 0;
  // segmented (grouped) mode: blockIdx.z selects a segment of rows and its own weight matrix
  const int* seg_off = nullptr;   // [nseg] first row of the segment (device)
  const int* seg_cnt = nullptr;   // [nseg] rows in the segment (device)
  const int* seg_w = nullptr;     // [nseg] which of the n_w weight matrices a segment uses (device), or null: segment z uses matrix z
  int n_w = 0;                    // number of weight matrices when seg_w is given
  const int* a_rows = nullptr;    // optional gather: A row = a_rows[row]
  long long w_stride = 0;         // elements between consecutive segments' / batches' weights
  long long a_stride = 0, c_stride = 0;  // plain batched mode (no seg_cnt): per-z offsets of A and C
  long long ldw_k = 1;            // stride of W along k (1: W is [N,K]; N-major B of a plain matmul: ldw = 1, ldw_k = N)
  int nseg = 1;
  int epi = EPI_STORE;
  int c_bf16 = 0;
  const char* tag = nullptr;      // name of the call site in the per-kernel timing report (string literal)
  // weight-only quantisation: W points at INT8 / packed INT4 bytes, ldw and w_stride stay in ELEMENTS
  int wq = 0;                     // 0 dense, 1 int8, 2 int4 per output row, 3 int4 with one scale per 128 inputs
  const float* w_scale = nullptr; // [N] (wq 1, 2) or [N, K/128] (wq 3)
  long long ws_stride = 0;        // scales between consecutive segments
};

__device__ __forceinline__ float ld_f(const float* p) { return *p; }
__device__ __forceinline__ float ld_f(const __nv_bfloat16* p) { return __bfloat162float(*p); }

// silu as the reference computes it: x * 0.5 * (1 + tanh(x / 2))   (verse_torch/tensor.py:853-856)
__device__ __forceinline__ float silu_ref(float x) { return x * (0.5f * (1.0f + tanhf(0.5f * x))); }

template <typename T>
__device__ __forceinline__ void store_out(void* C, long long idx, float v, int c_bf16) {
  if (c_bf16) reinterpret_cast<__nv_bfloat16*>(C)[idx] = __float2bfloat16_rn(v);
  else reinterpret_cast<float*>(C)[idx] = v;
}

// SIMT tile kernel, fp32 accumulate, any shape.  64x64 tile, 16-deep k step, 256 threads, 4x4 per thread.
template <typename TA, typename TW>
__global__ void __launch_bounds__(256) gemm_nt_simt_kernel(GemmArgs g) {
  constexpr int BM = 64, BN = 64, BK = 16;
  __shared__ float sA[BK][BM + 1];
  __shared__ float sW[BK][BN + 1];
  const int z = blockIdx.z;
  int row0 = 0, Mz = g.M;
  if (g.seg_cnt) { row0 = g.seg_off[z]; Mz = g.seg_cnt[z]; }
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  if (m0 >= Mz) return;
  const TA* A = reinterpret_cast<const TA*>(g.A) + (g.seg_cnt ? 0 : (long long)z * g.a_stride);
  const TW* W = reinterpret_cast<const TW*>(g.W) + (long long)z * g.w_stride;
  const long long c_base = g.seg_cnt ? 0 : (long long)z * g.c_stride;
  const int tid = threadIdx.x;
  const int tx = tid % 16, ty = tid / 16;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < g.K; k0 += BK) {
    for (int e = tid; e < BM * BK; e += 256) {
      const int r = e / BK, c = e % BK;
      float va = 0.f, vw = 0.f;
      if (m0 + r < Mz && k0 + c < g.K) {
        const long long ar = g.a_rows ? g.a_rows[row0 + m0 + r] : (row0 + m0 + r);
        va = ld_f(A + ar * g.lda + k0 + c);
      }
      if (n0 + r < g.N && k0 + c < g.K) vw = ld_f(W + (long long)(n0 + r) * g.ldw + (long long)(k0 + c) * g.ldw_k);
      sA[c][r] = va;
      sW[c][r] = vw;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = sA[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) w[j] = sW[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= Mz) continue;
    const long long crow = (long long)(row0 + m);
    (void)c_base;
    if (g.epi == EPI_SWIGLU) {
#pragma unroll
      for (int j = 0; j < 4; j += 2) {
        const int n = n0 + tx * 4 + j;
        if (n + 1 < g.N) {
          const float v = silu_ref(acc[i][j]) * acc[i][j + 1];
          store_out<float>(g.C, c_base + crow * g.ldc + (n >> 1), v, g.c_bf16);
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int n = n0 + tx * 4 + j;
        if (n >= g.N) continue;
        float v = acc[i][j];
        if (g.bias) v += g.bias[n];
        const long long idx = c_base + crow * g.ldc + n;
        if (g.epi == EPI_ADD) reinterpret_cast<float*>(g.C)[idx] += v;
        else store_out<float>(g.C, idx, v, g.c_bf16);
      }
    }
  }
}

template <typename TA, typename TW>
inline int32_t launch_gemm_simt(vn_ctx* ctx, const GemmArgs& g) {
  if (g.M <= 0 || g.N <= 0) return VN_OK;
  dim3 grid(ceil_div(g.N, 64), ceil_div(g.M, 64), g.nseg);
  VN_LAUNCH(ctx, (gemm_nt_simt_kernel<TA, TW>), grid, 256, 0, g);
  return VN_OK;
}
