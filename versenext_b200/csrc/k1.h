// Internal interface between the model's LM-head GEMMs (model.cu) and the acceptance kernels (accept.cu) for the
// fused LM head -> top-k -> acceptance step: the target's logits never reach HBM, only per-row candidate lists do.
#pragma once
#include "common.cuh"

struct vn_k1 {
  int rows = 0;            // target rows of the call: B * np
  int cap = 0;             // candidate slots per row
  int nb = 0;              // head columns of the bound GEMM
  float* boot = nullptr;   // [rows][nb] logits of the first nb vocabulary columns
  float* tau = nullptr;    // [rows] raw-logit lower bound of the row's k-th largest logit
  int* count = nullptr;    // [rows * count_stride] candidates appended by the head GEMM's epilogue (row r at r * count_stride)
  int count_stride = 1;
  float* cand_val = nullptr;
  int* cand_tok = nullptr;  // [rows][cap]
  int* fallback = nullptr;  // device flag: a candidate list overflowed, the classic path below has to run
  void* p_lists = nullptr;  // [rows] kept lists of the target rows
  void* parts = nullptr;    // per-slice lists of the classic path
  int chunks = 1;
};

constexpr int VN_K1_CAP = 4096;

// carve everything above out of the context's workspace (grows it when needed: not inside a stream capture)
int32_t vn_k1_layout(vn_ctx* ctx, int B, int np, int top_k, int V, vn_k1* out);
// tau[row] from boot[row][0 .. nb), count[row] = 0, fallback = 0
int32_t vn_k1_bound(vn_ctx* ctx, const vn_k1& k1, int top_k, float temp);
// candidate lists -> kept lists (k1_finish_kernel), the classic select on p_fallback rows when the flag is up, the
// draft rows' lists (q_lists given, or selected from q_logits), then the decisions
int32_t vn_k1_accept(vn_ctx* ctx, const vn_k1& k1, const float* p_fallback, long long p_sb, long long p_si,
                     const void* q_lists, long long ql_sb, long long ql_si, const float* q_logits, long long q_sb,
                     long long q_si, const int64_t* draft, const float* u_acc, const float* u_smp, uint64_t seed,
                     uint32_t offset, float temperature, int32_t top_k, int32_t bonus, int32_t B, int32_t k, int32_t V,
                     int32_t* out_len, int64_t* out_tok);

// the classic acceptance entry (accept.cu): logits in HBM, see vn_accept_strided; lists_out keeps the p rows' lists
int32_t vn_accept_impl(vn_ctx* ctx, const float* p, long long p_sb, long long p_si, const float* q, long long q_sb,
                       long long q_si, const int64_t* draft, const float* u_acc, const float* u_smp, uint64_t seed,
                       uint32_t offset, float temperature, int32_t top_k, int32_t bonus, int32_t B, int32_t k, int32_t V,
                       int32_t* out_len, int64_t* out_tok, int32_t smp_purpose, int32_t pos_base, void* lists_out);
