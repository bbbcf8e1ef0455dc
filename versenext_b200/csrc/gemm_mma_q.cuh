// Weight-only quantised linears: y = (x @ q^T) * scale with q kept as INT8 or packed INT4 in HBM and
// dequantised on the way into the tensor cores (verse_torch/quantize.py:187-258, :277-309, :467-533).
//
//   QMODE 1  INT8, one fp32 scale per output row            (quantize_int8, :187-214)
//   QMODE 2  INT4 two's-complement nibbles, even index low, one fp32 scale per output row (quantize_int4, :231-258)
//   QMODE 3  INT4 with one scale per 128 input features (scales hold bf16-representable values)
//
// Same CTA tiling as the bf16 kernel (BM x 64 x 64, cp.async ring, mma.sync.m16n8k16 with fp32 accumulate);
// the weight tile travels as raw bytes (64 or 32 per row and k-tile) and the B fragments are built from 16-bit
// or 8-bit shared-memory reads: small integers are exact in bf16, so the product equals x @ q^T computed in
// bf16 x bf16 -> fp32, and the scale is applied to the fp32 accumulator (per row, or per 128-wide k group).
#pragma once
#include "gemm_mma.cuh"

namespace mmaq_detail {

using namespace mma_detail;

constexpr int WROW = 80;   // bytes per weight row in shared memory (64 data + 16 pad: conflict-free 16-bit reads)

__device__ __forceinline__ unsigned i8x2_to_bf16x2(unsigned short v) {
  const float a = (float)(signed char)(v & 0xff), b = (float)(signed char)(v >> 8);
  __nv_bfloat162 r = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<unsigned*>(&r);
}
__device__ __forceinline__ unsigned i4x2_to_bf16x2(unsigned char v) {
  int lo = v & 0xf, hi = v >> 4;
  lo = lo >= 8 ? lo - 16 : lo;
  hi = hi >= 8 ? hi - 16 : hi;
  __nv_bfloat162 r = __floats2bfloat162_rn((float)lo, (float)hi);
  return *reinterpret_cast<unsigned*>(&r);
}

template <int BM, int QMODE>
__global__ void __launch_bounds__(BM * 2) gemm_mma_q_kernel(GemmArgs g) {
  constexpr int THREADS = BM * 2;
  constexpr int WARPS_N = 2;
  constexpr int WBYTES = QMODE == 1 ? 64 : 32;          // weight bytes per row and k-tile
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* sA = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  unsigned char* sW = smem_raw + (size_t)STAGES * BM * LDS * 2;
  const int z = blockIdx.z;
  int row0 = 0, Mz = g.M;
  if (g.seg_cnt) { row0 = g.seg_off[z]; Mz = g.seg_cnt[z]; }
  const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;
  if (m0 >= Mz) return;
  const long long wrow_bytes = QMODE == 1 ? g.ldw : g.ldw / 2;
  const __nv_bfloat16* A = reinterpret_cast<const __nv_bfloat16*>(g.A);
  const unsigned char* W = reinterpret_cast<const unsigned char*>(g.W) +
                           (long long)z * (QMODE == 1 ? g.w_stride : g.w_stride / 2);
  const int groups = QMODE == 3 ? (g.K + 127) / 128 : 1;   // the last group may be half a group (K % 128 == 64)
  const float* scale = g.w_scale + (long long)z * g.ws_stride;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int wm = warp / WARPS_N, wn = warp % WARPS_N;
  const int KT = (g.K + BK - 1) / BK;

  constexpr int A_ITERS = BM * 8 / THREADS;
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
  constexpr int W_CHUNKS = BN * WBYTES / 16;            // 16-byte chunks of the weight tile
  auto load_stage = [&](int stage, int kt) {
    const int k0 = kt * BK;
#pragma unroll
    for (int i = 0; i < A_ITERS; ++i) {
      const int c = tid + i * THREADS, r = c >> 3, kc = (c & 7) * 8;
      const bool ok = a_ok[i] && (k0 + kc) < g.K;
      cp_async16(sA + ((size_t)stage * BM + r) * LDS + kc, ok ? (const void*)(a_src[i] + k0) : (const void*)A, ok);
    }
    for (int c = tid; c < W_CHUNKS; c += THREADS) {
      const int r = c / (WBYTES / 16), b = (c % (WBYTES / 16)) * 16;
      const int kbyte = (QMODE == 1 ? k0 : k0 / 2) + b;
      const bool ok = (n0 + r) < g.N && kbyte < wrow_bytes;
      const unsigned char* src = W + (long long)(n0 + r) * wrow_bytes + kbyte;
      cp_async16(sW + ((size_t)stage * BN + r) * WROW + b, ok ? (const void*)src : (const void*)W, ok);
    }
  };

  float acc[2][4][4], part[2][4][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) { acc[i][j][e] = 0.f; part[i][j][e] = 0.f; }

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
    const unsigned char* w_st = sW + (size_t)(kt % STAGES) * BN * WROW;
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
      for (int j = 0; j < 4; ++j) {
        const unsigned char* wr = w_st + (size_t)(wn * 32 + j * 8 + (lane >> 2)) * WROW;
        const int k = kk + (lane & 3) * 2;
        if (QMODE == 1) {
          bf[j][0] = i8x2_to_bf16x2(*reinterpret_cast<const unsigned short*>(wr + k));
          bf[j][1] = i8x2_to_bf16x2(*reinterpret_cast<const unsigned short*>(wr + k + 8));
        } else {
          bf[j][0] = i4x2_to_bf16x2(wr[k >> 1]);
          bf[j][1] = i4x2_to_bf16x2(wr[(k + 8) >> 1]);
        }
      }
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) mma_bf16(QMODE == 3 ? part[i][j] : acc[i][j], af[i], bf[j]);
    }
    if (QMODE == 3 && ((kt & 1) || kt + 1 == KT)) {
      // end of a 128-wide k group: fold the group's partial sums in with the group's scales
      const int grp = (kt * BK) / 128;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int n = n0 + wn * 32 + j * 8 + (lane & 3) * 2;
        const float s0 = n < g.N ? scale[(long long)n * groups + grp] : 0.f;
        const float s1 = n + 1 < g.N ? scale[(long long)(n + 1) * groups + grp] : 0.f;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          acc[i][j][0] += part[i][j][0] * s0; acc[i][j][1] += part[i][j][1] * s1;
          acc[i][j][2] += part[i][j][2] * s0; acc[i][j][3] += part[i][j][3] * s1;
          part[i][j][0] = part[i][j][1] = part[i][j][2] = part[i][j][3] = 0.f;
        }
      }
    }
  }
  cp_async_wait<0>();

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
        float v0 = acc[i][j][half * 2], v1 = acc[i][j][half * 2 + 1];
        if (QMODE != 3) {
          v0 *= n < g.N ? scale[n] : 0.f;
          v1 *= n + 1 < g.N ? scale[n + 1] : 0.f;
        }
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

// ---- quantisers: one CTA per output row ---------------------------------------------------------------
__device__ __forceinline__ float block_max_256(float v, float* sm) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  __syncthreads();
  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = sm[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) r = fmaxf(r, sm[i]);
  return r;
}

// QMODE 1 / 2: scale = max|w| / qmax (1 / qmax for an all-zero row), q = rint(w / scale) clipped
__device__ __forceinline__ float q_in(const __nv_bfloat16& v) { return __bfloat162float(v); }
__device__ __forceinline__ float q_in(const float& v) { return v; }

template <int QMODE, typename TW = __nv_bfloat16>
__global__ void __launch_bounds__(256) quantize_rows_kernel(const TW* __restrict__ w, int K,
                                                            unsigned char* __restrict__ q, float* __restrict__ scale) {
  __shared__ float sm[8];
  const long long row = blockIdx.x;
  const TW* wr = w + row * K;
  float mx = 0.f;
  for (int k = threadIdx.x; k < K; k += 256) mx = fmaxf(mx, fabsf(q_in(wr[k])));
  mx = block_max_256(mx, sm);
  const float qmax = QMODE == 1 ? 127.f : 7.f;
  const float sc = __fdiv_rn(mx > 0.f ? mx : 1.0f, qmax);
  if (threadIdx.x == 0) scale[row] = sc;
  if (QMODE == 1) {
    signed char* qr = reinterpret_cast<signed char*>(q) + row * K;
    for (int k = threadIdx.x; k < K; k += 256) {
      float v = rintf(__fdiv_rn(q_in(wr[k]), sc));
      qr[k] = (signed char)fminf(fmaxf(v, -127.f), 127.f);
    }
  } else {
    unsigned char* qr = q + row * ((K + 1) / 2);      // an odd K pads the last high nibble with zero (quantize.py:36-66)
    for (int k2 = threadIdx.x; k2 < (K + 1) / 2; k2 += 256) {
      const float a = fminf(fmaxf(rintf(__fdiv_rn(q_in(wr[2 * k2]), sc)), -8.f), 7.f);
      const float b = (2 * k2 + 1 < K) ? fminf(fmaxf(rintf(__fdiv_rn(q_in(wr[2 * k2 + 1]), sc)), -8.f), 7.f) : 0.f;
      qr[k2] = (unsigned char)(((int)a & 0xf) | (((int)b & 0xf) << 4));
    }
  }
}

// QMODE 3: one scale per 128 input features, rounded to bfloat16 before the division
template <typename TW = __nv_bfloat16>
__global__ void __launch_bounds__(128) quantize_g128_kernel(const TW* __restrict__ w, int K,
                                                            unsigned char* __restrict__ q, float* __restrict__ scale) {
  const long long row = blockIdx.x;
  const int grp = blockIdx.y, groups = (K + 127) / 128;
  const int col = grp * 128 + (int)threadIdx.x;            // a last group shorter than 128 is padded with zeros
  const float v = col < K ? q_in(w[row * K + col]) : 0.f;
  float mx = fabsf(v);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  __shared__ float sm[4];
  __shared__ float s_q[128];
  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = mx;
  __syncthreads();
  mx = fmaxf(fmaxf(sm[0], sm[1]), fmaxf(sm[2], sm[3]));
  const float sc = __bfloat162float(__float2bfloat16_rn(__fdiv_rn(mx > 0.f ? mx : 1.0f, 7.f)));
  if (threadIdx.x == 0) scale[row * groups + grp] = sc;
  s_q[threadIdx.x] = fminf(fmaxf(rintf(__fdiv_rn(v, sc)), -8.f), 7.f);
  __syncthreads();
  if (threadIdx.x < 64 && grp * 128 + 2 * (int)threadIdx.x < K) {
    const int a = (int)s_q[2 * threadIdx.x], b = (int)s_q[2 * threadIdx.x + 1];
    q[row * (K / 2) + grp * 64 + threadIdx.x] = (unsigned char)((a & 0xf) | ((b & 0xf) << 4));
  }
}

}  // namespace mmaq_detail

inline bool gemm_mma_q_supported(const GemmArgs& g) {
  return g.wq >= 1 && g.wq <= 3 && g.K % 64 == 0 && g.lda % 8 == 0 && g.ldw % 32 == 0 && g.ldw_k == 1 &&
         ((uintptr_t)g.A & 15) == 0 && ((uintptr_t)g.W & 15) == 0 &&
         (g.seg_cnt != nullptr || g.nseg == 1);
}

template <int QMODE>
inline int32_t launch_gemm_mma_q_mode(vn_ctx* ctx, const GemmArgs& g) {
  using namespace mmaq_detail;
  const bool big = g.M > 64;
  const int BM = big ? 128 : 64;
  const size_t smem = (size_t)STAGES * ((size_t)BM * LDS * 2 + (size_t)BN * WROW);
  VN_CUDA(ctx, cudaFuncSetAttribute(gemm_mma_q_kernel<64, QMODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    (int)((size_t)STAGES * (64 * LDS * 2 + BN * WROW))));
  VN_CUDA(ctx, cudaFuncSetAttribute(gemm_mma_q_kernel<128, QMODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    (int)((size_t)STAGES * (128 * LDS * 2 + BN * WROW))));
  dim3 grid(ceil_div(g.M, BM), ceil_div(g.N, BN), g.nseg);
  const char* name = g.tag ? g.tag : "gemm_mma_q_kernel";
  if (big) VN_LAUNCH_NAMED(ctx, name, (gemm_mma_q_kernel<128, QMODE>), grid, 256, smem, g);
  else VN_LAUNCH_NAMED(ctx, name, (gemm_mma_q_kernel<64, QMODE>), grid, 128, smem, g);
  return VN_OK;
}

inline int32_t launch_gemm_mma_q(vn_ctx* ctx, const GemmArgs& g) {
  if (g.M <= 0 || g.N <= 0) return VN_OK;
  if (g.wq == 1) return launch_gemm_mma_q_mode<1>(ctx, g);
  if (g.wq == 2) return launch_gemm_mma_q_mode<2>(ctx, g);
  return launch_gemm_mma_q_mode<3>(ctx, g);
}
