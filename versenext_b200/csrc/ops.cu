// DeviceBackend operator set in fp32 (verse_torch/device.py:219-270; NumPy semantics of :285-335).
#include "common.cuh"
#include "gemm.cuh"
#include <math_constants.h>
#include <stdint.h>
#include <stdlib.h>

namespace {

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sumf(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <int THREADS>
__device__ __forceinline__ float block_reduce(float v, bool is_max, float* sm) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = is_max ? warp_max(v) : warp_sumf(v);
  __syncthreads();
  if (lane == 0) sm[warp] = v;
  __syncthreads();
  float r = sm[0];
  for (int w = 1; w < THREADS / 32; ++w) r = is_max ? fmaxf(r, sm[w]) : r + sm[w];
  return r;
}

// softmax over the middle axis of (outer, n, inner); one block per (outer, inner) line
__global__ void __launch_bounds__(256) softmax_kernel(const float* __restrict__ x, float* __restrict__ y,
                                                      long long n, long long inner) {
  __shared__ float sm[8];
  const long long line = blockIdx.x;
  const long long base = (line / inner) * n * inner + (line % inner);
  float m = -CUDART_INF_F;
  for (long long i = threadIdx.x; i < n; i += 256) m = fmaxf(m, x[base + i * inner]);
  m = block_reduce<256>(m, true, sm);
  float s = 0.f;
  for (long long i = threadIdx.x; i < n; i += 256) s += expf(x[base + i * inner] - m);
  s = block_reduce<256>(s, false, sm);
  for (long long i = threadIdx.x; i < n; i += 256) y[base + i * inner] = expf(x[base + i * inner] - m) / s;
}

// mode 0: rmsnorm  y = x / sqrt(mean(x^2) + eps) * w
// mode 1: layernorm y = (x - mean) / sqrt(var + eps) * w + b
__global__ void __launch_bounds__(256) norm_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                   const float* __restrict__ b, float* __restrict__ y,
                                                   long long cols, float eps, int mode) {
  __shared__ float sm[8];
  const float* xr = x + (long long)blockIdx.x * cols;
  float* yr = y + (long long)blockIdx.x * cols;
  float mean = 0.f;
  if (mode == 1) {
    float s = 0.f;
    for (long long i = threadIdx.x; i < cols; i += 256) s += xr[i];
    mean = block_reduce<256>(s, false, sm) / (float)cols;
  }
  float ss = 0.f;
  for (long long i = threadIdx.x; i < cols; i += 256) { float d = xr[i] - mean; ss += d * d; }
  const float var = block_reduce<256>(ss, false, sm) / (float)cols;
  const float r = sqrtf(var + eps);
  for (long long i = threadIdx.x; i < cols; i += 256) {
    float v = (xr[i] - mean) / r * w[i];
    if (mode == 1 && b) v += b[i];
    yr[i] = v;
  }
}

__global__ void rope_kernel(const float* __restrict__ x, const float* __restrict__ cs, const float* __restrict__ sn,
                            float* __restrict__ y, long long total_rows, long long T, long long D) {
  const long long half = D / 2;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total_rows * half) return;
  const long long row = i / half, j = i % half, t = row % T;
  const float x1 = x[row * D + j], x2 = x[row * D + half + j];
  const float c = cs[t * half + j], s = sn[t * half + j];
  y[row * D + j] = x1 * c - x2 * s;
  y[row * D + half + j] = x1 * s + x2 * c;
}

// one warp per query row: scores over Tk keys, softmax, weighted sum of V
__global__ void __launch_bounds__(128) attention_kernel(const float* __restrict__ q, const float* __restrict__ k,
                                                        const float* __restrict__ v, const float* __restrict__ mask,
                                                        float* __restrict__ out, long long Tq, long long Tk, int D,
                                                        float scale) {
  extern __shared__ float smem[];  // 4 warps x Tk scores
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long qi = (long long)blockIdx.x * 4 + warp;
  const long long bh = blockIdx.y;
  if (qi >= Tq) return;
  float* sc = smem + (long long)warp * Tk;
  const float* qr = q + (bh * Tq + qi) * D;
  const float* kb = k + bh * Tk * D;
  const float* vb = v + bh * Tk * D;
  float m = -CUDART_INF_F;
  for (long long j = lane; j < Tk; j += 32) {
    float s = 0.f;
    for (int d = 0; d < D; ++d) s = fmaf(qr[d], kb[j * D + d], s);
    s *= scale;
    if (mask) s += mask[qi * Tk + j];
    sc[j] = s;
    m = fmaxf(m, s);
  }
  m = warp_max(m);
  float l = 0.f;
  for (long long j = lane; j < Tk; j += 32) { float e = expf(sc[j] - m); sc[j] = e; l += e; }
  l = warp_sumf(l);
  __syncwarp();
  for (int d = lane; d < D; d += 32) {
    float acc = 0.f;
    for (long long j = 0; j < Tk; ++j) acc = fmaf(sc[j] / l, vb[j * D + d], acc);
    out[(bh * Tq + qi) * D + d] = acc;
  }
}


// ---- fp32 linear for a few rows against a large weight matrix (the k draft heads of SpeculativeDecoder.draft:
// 4 x 248,320 x 1,024 fp32 = 4 GB of weights for 1 to 32 hidden rows, speculative.py:150-158) -------------------
// Weight streaming: a warp owns SK_NR consecutive output features and walks K in float4 steps, one 512-byte coalesced
// segment of every weight row per trip, against up to 8 rows of x at a time (x is a few KB: it stays in L1).  With
// more than 8 rows the warp makes one pass per group of 8 over the same weight rows, which it finds in L1 / L2, so
// DRAM still sees every weight once.  Per output: each lane sums its k = 4 * lane + 128 * i terms in order, then the
// lanes are added by a shuffle tree: deterministic.
constexpr int SK_NR = 4;
template <int MR>
__global__ void __launch_bounds__(256, 2) linear_skinny_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                            const float* __restrict__ bias, float* __restrict__ y,
                                                            int M, long long N, int K) {
  const int lane = threadIdx.x & 31;
  const long long n0 = ((long long)blockIdx.x * 8 + (threadIdx.x >> 5)) * SK_NR;
  if (n0 >= N) return;
  const float* wr[SK_NR];
#pragma unroll
  for (int j = 0; j < SK_NR; ++j) wr[j] = w + (n0 + j < N ? n0 + j : N - 1) * (long long)K;
  for (int m0 = 0; m0 < M; m0 += MR) {
    float acc[SK_NR][MR];
#pragma unroll
    for (int j = 0; j < SK_NR; ++j)
#pragma unroll
      for (int i = 0; i < MR; ++i) acc[j][i] = 0.f;
#pragma unroll 1
    for (int k = lane * 4; k < K; k += 128) {
      float4 wv[SK_NR];
#pragma unroll
      for (int j = 0; j < SK_NR; ++j) wv[j] = *reinterpret_cast<const float4*>(wr[j] + k);
#pragma unroll
      for (int i = 0; i < MR; ++i) {
        const int m = m0 + i < M ? m0 + i : M - 1;
        const float4 xv = __ldg(reinterpret_cast<const float4*>(x + (long long)m * K + k));
#pragma unroll
        for (int j = 0; j < SK_NR; ++j) {
          acc[j][i] = fmaf(xv.x, wv[j].x, acc[j][i]);
          acc[j][i] = fmaf(xv.y, wv[j].y, acc[j][i]);
          acc[j][i] = fmaf(xv.z, wv[j].z, acc[j][i]);
          acc[j][i] = fmaf(xv.w, wv[j].w, acc[j][i]);
        }
      }
    }
#pragma unroll
    for (int j = 0; j < SK_NR; ++j)
#pragma unroll
      for (int i = 0; i < MR; ++i) {
        float v = acc[j][i];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane == 0 && m0 + i < M && n0 + j < N) y[(long long)(m0 + i) * N + n0 + j] = v + (bias ? bias[n0 + j] : 0.f);
      }
  }
}

}  // namespace

extern "C" {

int32_t vn_matmul(vn_ctx* ctx, const float* a, const float* b, float* c, int64_t batch, int64_t M, int64_t N,
                  int64_t K, int32_t b_broadcast) {
  VN_CHECK_CTX(ctx);
  VN_REQUIRE(ctx, a && b && c, "null pointer");
  VN_REQUIRE(ctx, batch >= 0 && M >= 0 && N >= 0 && K >= 0 && batch < 65536, "bad shape");
  if (batch * M * N == 0) return VN_OK;
  GemmArgs g;
  g.A = a; g.lda = K; g.a_stride = M * K;
  g.W = b; g.ldw = 1; g.ldw_k = N; g.w_stride = b_broadcast ? 0 : K * N;
  g.C = c; g.ldc = N; g.c_stride = M * N;
  g.M = (int)M; g.N = (int)N; g.K = (int)K; g.nseg = (int)batch;
  return launch_gemm_simt<float, float>(ctx, g);
}

int32_t vn_linear(vn_ctx* ctx, const float* x, const float* w, const float* bias, float* y, int64_t M, int64_t N,
                  int64_t K) {
  VN_CHECK_CTX(ctx);
  VN_REQUIRE(ctx, x && w && y, "null pointer");
  VN_REQUIRE(ctx, M >= 0 && N >= 0 && K >= 0, "bad shape");
  if (M * N == 0) return VN_OK;
  // few rows against many output features: the weight-streaming kernel
  // VN_LINEAR_SKINNY_MAX: most rows the streaming kernel takes (default 32; 0 keeps the tiled kernel: A/B timing)
  static const int skinny_max = [] { const char* e = getenv("VN_LINEAR_SKINNY_MAX"); return e ? atoi(e) : 32; }();
  if (M <= skinny_max && N >= 1024 && K % 4 == 0 && K >= 128 && (((uintptr_t)x | (uintptr_t)w) & 15) == 0) {
    const unsigned grid = (unsigned)ceil_div(N, (int64_t)(8 * SK_NR));
    if (M == 1) VN_LAUNCH(ctx, linear_skinny_kernel<1>, grid, 256, 0, x, w, bias, y, (int)M, (long long)N, (int)K);
    else if (M == 2) VN_LAUNCH(ctx, linear_skinny_kernel<2>, grid, 256, 0, x, w, bias, y, (int)M, (long long)N, (int)K);
    else if (M <= 4) VN_LAUNCH(ctx, linear_skinny_kernel<4>, grid, 256, 0, x, w, bias, y, (int)M, (long long)N, (int)K);
    else VN_LAUNCH(ctx, linear_skinny_kernel<8>, grid, 256, 0, x, w, bias, y, (int)M, (long long)N, (int)K);
    return VN_OK;
  }
  GemmArgs g;
  g.A = x; g.lda = K; g.W = w; g.ldw = K; g.C = y; g.ldc = N; g.bias = bias;
  g.M = (int)M; g.N = (int)N; g.K = (int)K;
  return launch_gemm_simt<float, float>(ctx, g);
}

int32_t vn_softmax(vn_ctx* ctx, const float* x, float* y, int64_t outer, int64_t n, int64_t inner) {
  VN_CHECK_CTX(ctx);
  VN_REQUIRE(ctx, x && y && outer >= 0 && n >= 1 && inner >= 1, "bad arguments");
  if (outer * inner == 0) return VN_OK;
  VN_REQUIRE(ctx, outer * inner < (1ll << 31), "too many lines");
  VN_LAUNCH(ctx, softmax_kernel, (unsigned)(outer * inner), 256, 0, x, y, (long long)n, (long long)inner);
  return VN_OK;
}

int32_t vn_layernorm(vn_ctx* ctx, const float* x, const float* w, const float* b, float* y, int64_t rows,
                     int64_t cols, float eps) {
  VN_CHECK_CTX(ctx);
  VN_REQUIRE(ctx, x && w && y && rows >= 0 && cols >= 1, "bad arguments");
  if (rows == 0) return VN_OK;
  VN_LAUNCH(ctx, norm_kernel, (unsigned)rows, 256, 0, x, w, b, y, (long long)cols, eps, 1);
  return VN_OK;
}

int32_t vn_rmsnorm(vn_ctx* ctx, const float* x, const float* w, float* y, int64_t rows, int64_t cols, float eps) {
  VN_CHECK_CTX(ctx);
  VN_REQUIRE(ctx, x && w && y && rows >= 0 && cols >= 1, "bad arguments");
  if (rows == 0) return VN_OK;
  VN_LAUNCH(ctx, norm_kernel, (unsigned)rows, 256, 0, x, w, (const float*)nullptr, y, (long long)cols, eps, 0);
  return VN_OK;
}

int32_t vn_rope(vn_ctx* ctx, const float* x, const float* cs, const float* sn, float* y, int64_t outer, int64_t T,
                int64_t D) {
  VN_CHECK_CTX(ctx);
  VN_REQUIRE(ctx, x && cs && sn && y && D % 2 == 0 && outer >= 0 && T >= 1, "bad arguments");
  const long long n = outer * T * (D / 2);
  if (n == 0) return VN_OK;
  VN_LAUNCH(ctx, rope_kernel, (unsigned)ceil_div(n, 256ll), 256, 0, x, cs, sn, y, (long long)(outer * T),
            (long long)T, (long long)D);
  return VN_OK;
}

int32_t vn_attention(vn_ctx* ctx, const float* q, const float* k, const float* v, const float* mask, float* out,
                     int64_t BH, int64_t Tq, int64_t Tk, int64_t D) {
  VN_CHECK_CTX(ctx);
  VN_REQUIRE(ctx, q && k && v && out && BH >= 0 && Tq >= 0 && Tk >= 1 && D >= 1, "bad arguments");
  VN_REQUIRE(ctx, BH < 65536, "too many batch*heads");
  if (BH * Tq == 0) return VN_OK;
  const size_t smem = (size_t)4 * Tk * sizeof(float);
  VN_REQUIRE(ctx, smem <= 200 * 1024, "Tk %lld too long for the backend attention op", (long long)Tk);
  if (smem > 48 * 1024)
    VN_CUDA(ctx, cudaFuncSetAttribute(attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid((unsigned)ceil_div(Tq, (int64_t)4), (unsigned)BH);
  VN_LAUNCH(ctx, attention_kernel, grid, 128, smem, q, k, v, mask, out, (long long)Tq, (long long)Tk, (int)D,
            1.0f / sqrtf((float)D));
  return VN_OK;
}

}  // extern "C"
