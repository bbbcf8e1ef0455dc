// VerseNexLM on the device: weights, KV cache, one forward over new positions (chain or tree).
// Mirrors CometSparkNexLM.forward (verse_nex/cometspark.py:670-698) block by block, with the KV cache that
// TriSparseAttention.forward accepts (tri_sparse_attn.py:559-575) kept resident and updated in place.
#include "common.cuh"
#include "gemm.cuh"
#include "gemm_mma.cuh"
#include "model_kernels.cuh"
#include "attn_mma.cuh"
#include "delta_attn.cuh"
#include "draft_kernel.cuh"
#include "gemm_tc.cuh"
#include "gemm_mma_q.cuh"
#include "gemm_tcq.cuh"
#include "k1.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#include <algorithm>
#include <set>
#include <type_traits>

namespace {

struct Config {
  int vocab = 0, dim = 0, n_layer = 0, n_head = 0, n_kv = 0, hd = 0;
  int window = 512, n_sink = 64, use_alibi = 1, use_rope = 0, max_seq_len = 2048;
  int anchor = 128, latent = 0;   // delta attention: anchor_interval, latent_dim (0: n_kv * hd)
  double rope_theta = 10000.0;
  int P = 5, E = 8, top_k = 3, expert_hidden = 0, mlp_hidden = 0, mlp_mult = 4;
  int tie = 1, emb_scale = 0;
  int bf16 = 0;
  std::vector<int> kind;  // 0 trisparse, 1 mod (TriSparse attention + MoD feed-forward), 2 vda, 3 dsa, 4 kda, 5 gmla
};

inline bool is_delta(int kind) { return kind >= 2; }

// ---- minimal JSON field access (flat object, as json.dumps of the constructor kwargs yields) -------------
bool json_find(const std::string& s, const char* key, size_t* pos) {
  std::string k = std::string("\"") + key + "\"";
  size_t p = s.find(k);
  if (p == std::string::npos) return false;
  p = s.find(':', p + k.size());
  if (p == std::string::npos) return false;
  ++p;
  while (p < s.size() && isspace((unsigned char)s[p])) ++p;
  *pos = p;
  return true;
}
bool json_num(const std::string& s, const char* key, double* out) {
  size_t p;
  if (!json_find(s, key, &p)) return false;
  if (s.compare(p, 4, "null") == 0) return false;
  if (s.compare(p, 4, "true") == 0) { *out = 1; return true; }
  if (s.compare(p, 5, "false") == 0) { *out = 0; return true; }
  char* end = nullptr;
  double v = strtod(s.c_str() + p, &end);
  if (end == s.c_str() + p) return false;
  *out = v;
  return true;
}
bool json_str(const std::string& s, const char* key, std::string* out) {
  size_t p;
  if (!json_find(s, key, &p) || s[p] != '"') return false;
  size_t e = s.find('"', p + 1);
  if (e == std::string::npos) return false;
  *out = s.substr(p + 1, e - p - 1);
  return true;
}
bool json_str_list(const std::string& s, const char* key, std::vector<std::string>* out) {
  size_t p;
  if (!json_find(s, key, &p) || s[p] != '[') return false;
  size_t e = s.find(']', p);
  if (e == std::string::npos) return false;
  size_t i = p + 1;
  while (i < e) {
    size_t a = s.find('"', i);
    if (a == std::string::npos || a > e) break;
    size_t b = s.find('"', a + 1);
    out->push_back(s.substr(a + 1, b - a - 1));
    i = b + 1;
  }
  return true;
}

// one DSA / KDA / GMLA module of a delta-attention layer (verse_nex/delta_attention.py): a dsa / kda / gmla layer
// has one, a vda layer one of each
struct SubAttn {
  int mode = 0;              // 0 dsa, 1 kda, 2 gmla
  void* wqkv = nullptr;      // dsa, kda: [(H + 2 n_kv) hd, D] (q | k | v); gmla: [H hd + latent, D] (wq | w_kv_down)
  void* w_down = nullptr;    // gmla: the w_kv_down rows of wqkv (not a buffer of its own)
  void* w_up = nullptr;      // gmla: [2 n_kv hd, latent]      w_k_up | w_v_up
  // gmla, bf16 models whose latent is not much narrower than K | V: [(H + 2 n_kv) hd, D] = wq | w_k_up w_kv_down |
  // w_v_up w_kv_down, built by finalize.  K and V are linear in the latent, so the two projections collapse into one
  // matrix of about the same size (exactly the same at the default latent_dim = n_kv hd) and the module then runs
  // like a DSA / KDA module: one q | k | v GEMM, no latent buffer, no reduction kernels in between.
  void* w_abs = nullptr;
  // weight-only quantised copies (the dense buffers are freed once these exist): 0 = wqkv as stacked above, 1 = w_up
  void* q[2] = {nullptr, nullptr};
  float* qs[2] = {nullptr, nullptr};
  void* sink = nullptr;      // dsa: [n_sink, D] global_tokens.weight, and its K / V (finalize)
  void* sink_k = nullptr;
  void* sink_v = nullptr;
  float* head_gate = nullptr;  // dsa, gmla: device [H] sigmoid(head_gate_logits)
  std::vector<float> gate_host;  // the same on the host
  float* head_w = nullptr;     // device [5][H]: per-head weights of the tensor-core kernel's passes (finalize)
  int pair = 0;              // which K / V plane pair of the cache is this module's
};

struct Layer {
  int kind = 0;
  std::vector<SubAttn> sub;  // delta kinds only
  void* w_vda = nullptr;     // vda, dense bf16: the three modules' q|k|v matrices (GMLA's folded one) stacked into
                             // [3 (H + 2 n_kv) hd, D], so that the decode route projects all three with one GEMM
  float* norm1 = nullptr;
  float* norm2 = nullptr;
  float gate_logits[3] = {0.f, 0.f, 0.f};
  void* wqkv = nullptr;     // [(H + 2 n_kv) hd, D]
  void* wproj = nullptr;    // [D, H hd]
  void* sink = nullptr;     // [n_sink, D]   global_tokens.weight
  void* sink_kv = nullptr;  // [n_sink, 2 n_kv hd] computed by finalize: sink @ [wk; wv]^T
  void* sink_k = nullptr;   // [n_sink, n_kv hd] (compacted from sink_kv)
  void* sink_v = nullptr;
  void* w_gateup = nullptr; // trisparse: [2 hidden, D], rows interleaved gate_j, up_j
  void* w_down = nullptr;   // [D, hidden]
  float* router = nullptr;  // mod: [(P + P E), D] fp32
  void* e_gateup = nullptr; // mod: [P E][2 eh, D]
  void* e_down = nullptr;   // mod: [P E][D, eh]
  // weight-only quantised copies (dense buffers are freed once these exist): 0 qkv, 1 proj, 2 gate|up, 3 down,
  // 4 expert gate|up, 5 expert down
  void* q[6] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  float* qs[6] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
};

}  // namespace

struct vn_model {
  vn_ctx* ctx = nullptr;
  Config cfg;
  size_t esz = 4;           // bytes per stored weight / activation element
  void* emb = nullptr;      // [V, D]
  void* head = nullptr;     // [V, D] (== emb when tied)
  float* norm_f = nullptr;
  std::vector<Layer> layers;
  float* rope_cos = nullptr;  // [rope_rows, hd/2]
  float* rope_sin = nullptr;
  int rope_rows = 0;
  std::set<std::string> loaded;
  bool finalized = false;
  uint64_t param_bytes = 0;
  int* status = nullptr;    // device word: 1 = a token id was out of range
  // activations, grown on demand
  int cap_rows = 0;
  float* x = nullptr;       // [M, D] residual stream
  void* h = nullptr;        // [M, D] normalised, storage dtype
  float* h32 = nullptr;     // [M, D] fp32 copy for the routers
  float* qkv = nullptr;     // [M, (H + 2 n_kv) hd]
  void* attn = nullptr;     // [M, D]
  void* act = nullptr;      // [M * slots, max(hidden, eh)]
  float* y = nullptr;       // [M * slots, D]
  int* slot_expert = nullptr; float* slot_w = nullptr; float* part_w = nullptr;
  int* expert_count = nullptr; int* expert_off = nullptr; int* expert_cur = nullptr;
  int* sorted_row = nullptr; int* slot_pos = nullptr;
  int* depth_dev = nullptr; unsigned long long* anc_dev = nullptr; int* rows_dev = nullptr;
  std::vector<int> tree_parents;   // the tree whose depths and ancestor masks depth_dev / anc_dev hold
  float* stage = nullptr; size_t stage_elems = 0;
  int qmode = 0;                 // 0 dense, 1 int8, 2 int4 per channel, 3 int4 group-128 (vn_model_quantize)
  int preq_mode = 0;             // scheme of linears that arrive already quantised (vn_model_load_quant_tensor)
  void* head_q = nullptr;        // quantised LM head (its own copy: the embedding table stays dense)
  float* head_qs = nullptr;
  void* hs = nullptr;            // [M * slots, D] routed activations in expert order (tcgen05 path)
  float* partial = nullptr;      // split-K workspace of the tcgen05 path
  size_t partial_bytes = 0;
  int* tc_error = nullptr;       // device word raised by a bounded wait that ran out
  int* sub_seg = nullptr;        // [3][sub_cap] offsets, counts and experts of the experts' 256-row pieces (prompt forwards)
  int sub_cap = 0;
  int* row_seg = nullptr;        // [2][row_seg_n] offsets and counts of the 256-row segments a prompt's GEMMs use
  int row_seg_cap = 0;
  unsigned* stack_bar = nullptr; // two device words: arrivals and generation of the fused layer stack's grid barrier
  std::vector<int> pair0;        // per layer: its first K / V plane pair in a cache (a vda layer owns three pairs)
  int n_pairs = 0;
  bool has_delta = false;        // some layer is vda / dsa / kda / gmla
  void* lat = nullptr;           // [M, latent] gmla latents, storage dtype
  float* mix = nullptr;          // [M, H hd] running sum of a vda layer's modules
  bool recurrent = false;        // vn_model_set_recurrent: ALiBi path as in the reference's one-token recurrent step
  bool fused_stack = false;      // vn_model_set_fused_stack / VN_DRAFT_STACK=1: the layer stack as one cooperative kernel
  bool use_tc = true;            // VN_GEMM_TC=0 in the environment: keep the mma.sync GEMMs
  bool force_simt_attn = false;  // VN_ATTN_SIMT=1 in the environment: keep the SIMT attention kernel (A/B checks)
};

struct vn_kv {
  vn_model* m = nullptr;
  vn_ctx* ctx = nullptr;     // the model's context, kept here so that destroying the cache never reads the model (which a
                             // garbage collector may have destroyed first)
  int max_batch = 0, max_seq = 0;
  std::vector<void*> k, v;   // per layer [max_batch, max_seq, n_kv, hd]
  void** planes_dev = nullptr;  // [2 * n_layer] device array of plane pointers (k0, v0, k1, v1, ...)
  int* lens = nullptr;       // device [max_batch]
  std::vector<int> len_ub;   // host upper bound of every length
  vn_kv* parent = nullptr;   // set for a view (vn_kv_view): planes and lengths belong to the parent
  int parent_first = 0;      // first sequence of the parent this view covers
};

// host upper bound of sequence b's length; a view shares its parent's record
static inline int& kv_ub(vn_kv* kv, int b) {
  return kv->parent ? kv->parent->len_ub[kv->parent_first + b] : kv->len_ub[b];
}

namespace {

template <typename T>
int32_t upload_rows(vn_model* m, const float* host, void* dst, long long rows, long long cols, long long dst_ld,
                    long long row_mul, long long row_off) {
  vn_ctx* ctx = m->ctx;
  const size_t n = (size_t)rows * cols;
  if (n == 0) return VN_OK;
  if (n > m->stage_elems) {
    VN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (m->stage) VN_CUDA(ctx, cudaFree(m->stage));
    m->stage = nullptr; m->stage_elems = 0;
    VN_CUDA(ctx, cudaMalloc(&m->stage, n * sizeof(float)));
    m->stage_elems = n;
  }
  VN_CUDA(ctx, cudaMemcpyAsync(m->stage, host, n * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
  VN_LAUNCH(ctx, convert_rows_kernel<T>, (unsigned)ceil_div((long long)n, 256ll), 256, 0, m->stage, (T*)dst, rows, cols,
            dst_ld, row_mul, row_off);
  VN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));  // the host buffer may be reused by the caller
  return VN_OK;
}

int32_t upload(vn_model* m, const float* host, void* dst, long long rows, long long cols, long long dst_ld,
               long long row_mul = 1, long long row_off = 0, bool force_f32 = false) {
  if (m->cfg.bf16 && !force_f32)
    return upload_rows<__nv_bfloat16>(m, host, dst, rows, cols, dst_ld, row_mul, row_off);
  return upload_rows<float>(m, host, dst, rows, cols, dst_ld, row_mul, row_off);
}

int32_t dev_alloc(vn_ctx* ctx, void** p, size_t bytes) {
  VN_CUDA(ctx, cudaMalloc(p, bytes ? bytes : 16));
  return VN_OK;
}

#define TRY(expr) do { int32_t _s = (expr); if (_s != VN_OK) return _s; } while (0)

// bytes and scales of one row of a quantised matrix (mode 1 int8, 2 int4 per channel, 3 int4 group-128)
inline size_t q_row_bytes(int mode, long long K) { return (size_t)(mode == 1 ? K : K / 2); }
inline size_t q_row_scales(int mode, long long K) { return (size_t)(mode == 3 ? (K + 127) / 128 : 1); }

// a delta module's GEMM on the quantised copy: rows row0.. of slot `slot`
inline void pick_sub(const vn_model* m, GemmArgs& g, const SubAttn& S, int slot, long long row0) {
  if (!m->qmode) return;
  g.W = (const unsigned char*)S.q[slot] + (size_t)row0 * q_row_bytes(m->qmode, g.K);
  g.w_scale = S.qs[slot] + (size_t)row0 * q_row_scales(m->qmode, g.K);
  g.wq = m->qmode;
}

int32_t alloc_weights(vn_model* m) {
  vn_ctx* ctx = m->ctx;
  const Config& c = m->cfg;
  const size_t e = m->esz;
  const size_t D = c.dim, qkv_rows = (size_t)(c.n_head + 2 * c.n_kv) * c.hd;
  uint64_t bytes = 0;
  auto A = [&](void** p, size_t n) -> int32_t { bytes += n; return dev_alloc(ctx, p, n); };
  TRY(A(&m->emb, (size_t)c.vocab * D * e));
  if (c.tie) m->head = m->emb; else TRY(A(&m->head, (size_t)c.vocab * D * e));
  TRY(A((void**)&m->norm_f, D * 4));
  TRY(dev_alloc(ctx, (void**)&m->status, 4));
  VN_CUDA(ctx, cudaMemsetAsync(m->status, 0, 4, ctx->stream));
  m->layers.resize(c.n_layer);
  for (int i = 0; i < c.n_layer; ++i) {
    Layer& L = m->layers[i];
    L.kind = c.kind[i];
    TRY(A((void**)&L.norm1, D * 4));
    TRY(A((void**)&L.norm2, D * 4));
    TRY(A(&L.wproj, D * (size_t)c.n_head * c.hd * e));
    m->pair0.push_back(m->n_pairs);
    if (is_delta(L.kind)) {
      m->has_delta = true;
      const size_t qd = (size_t)c.n_head * c.hd, kvd = (size_t)c.n_kv * c.hd, lat = c.latent;
      const int modes[3] = {0, 1, 2};
      const int first = L.kind == 2 ? 0 : L.kind - 3, count = L.kind == 2 ? 3 : 1;
      for (int si = 0; si < count; ++si) {
        SubAttn S;
        S.mode = modes[first + si];
        S.pair = m->n_pairs++;
        if (S.mode == 2) {
          TRY(A(&S.wqkv, (qd + lat) * D * e));
          S.w_down = (char*)S.wqkv + qd * D * e;
          TRY(A(&S.w_up, 2 * kvd * lat * e));
        } else {
          TRY(A(&S.wqkv, qkv_rows * D * e));
        }
        if (S.mode == 0) {
          TRY(A(&S.sink, (size_t)c.n_sink * D * e));
          TRY(dev_alloc(ctx, &S.sink_k, (size_t)c.n_sink * kvd * e));
          TRY(dev_alloc(ctx, &S.sink_v, (size_t)c.n_sink * kvd * e));
        }
        if (S.mode != 1) TRY(A((void**)&S.head_gate, (size_t)c.n_head * 4));
        TRY(dev_alloc(ctx, (void**)&S.head_w, (size_t)5 * c.n_head * 4));
        L.sub.push_back(S);
      }
    } else {
      m->n_pairs++;
      TRY(A(&L.wqkv, qkv_rows * D * e));
      TRY(A(&L.sink, (size_t)c.n_sink * D * e));
      TRY(dev_alloc(ctx, &L.sink_k, (size_t)c.n_sink * c.n_kv * c.hd * e));
      TRY(dev_alloc(ctx, &L.sink_v, (size_t)c.n_sink * c.n_kv * c.hd * e));
    }
    if (L.kind != 1) {
      TRY(A(&L.w_gateup, (size_t)2 * c.mlp_hidden * D * e));
      TRY(A(&L.w_down, D * (size_t)c.mlp_hidden * e));
    } else {
      const size_t ne = (size_t)c.P * c.E;
      TRY(A((void**)&L.router, (size_t)(c.P + ne) * D * 4));
      TRY(A(&L.e_gateup, ne * 2 * c.expert_hidden * D * e));
      TRY(A(&L.e_down, ne * D * c.expert_hidden * e));
    }
  }
  m->param_bytes = bytes;
  return VN_OK;
}

int32_t ensure_rows(vn_model* m, int M) {
  if (M <= m->cap_rows) return VN_OK;
  vn_ctx* ctx = m->ctx;
  const Config& c = m->cfg;
  VN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  void** bufs[] = {(void**)&m->x, &m->h, (void**)&m->h32, (void**)&m->qkv, &m->attn, &m->act, (void**)&m->y,
                   (void**)&m->slot_expert, (void**)&m->slot_w, (void**)&m->part_w, (void**)&m->sorted_row,
                   (void**)&m->slot_pos, (void**)&m->rows_dev, &m->hs, &m->lat, (void**)&m->mix};
  for (void** b : bufs) { if (*b) cudaFree(*b); *b = nullptr; }
  const size_t e = m->esz, D = c.dim, R = (size_t)M + (M >> 2) + 32;
  bool has_mod = false;
  for (int k : c.kind) has_mod |= (k == 1);
  const size_t S = has_mod ? (size_t)c.P * c.top_k : 1;
  const size_t hid = std::max((size_t)c.mlp_hidden, has_mod ? (size_t)c.expert_hidden : 0);
  TRY(dev_alloc(ctx, (void**)&m->x, R * D * 4));
  TRY(dev_alloc(ctx, &m->h, R * D * e));
  TRY(dev_alloc(ctx, (void**)&m->h32, R * D * 4));
  TRY(dev_alloc(ctx, (void**)&m->qkv, R * (size_t)(c.n_head + 2 * c.n_kv) * c.hd * 4));
  TRY(dev_alloc(ctx, &m->attn, R * D * e));
  TRY(dev_alloc(ctx, &m->act, R * S * hid * e));
  TRY(dev_alloc(ctx, (void**)&m->rows_dev, R * 4));
  if (m->has_delta) {
    TRY(dev_alloc(ctx, &m->lat, R * (size_t)c.latent * e));
    TRY(dev_alloc(ctx, (void**)&m->mix, R * (size_t)c.n_head * c.hd * 4));
  }
  // segment tables of a prompt's GEMMs (rows in blocks of 256; the experts' pieces), sized for the row capacity so
  // that a forward never allocates them: filled by kernels on the stream
  if (m->row_seg) cudaFree(m->row_seg);
  if (m->sub_seg) cudaFree(m->sub_seg);
  m->row_seg = m->sub_seg = nullptr;
  m->row_seg_cap = (int)(R / 256 + 2);
  TRY(dev_alloc(ctx, (void**)&m->row_seg, (size_t)2 * m->row_seg_cap * sizeof(int)));
  m->sub_cap = (int)(c.P * c.E + R * S / 256 + 2);
  TRY(dev_alloc(ctx, (void**)&m->sub_seg, (size_t)3 * m->sub_cap * sizeof(int)));
  if (has_mod) {
    TRY(dev_alloc(ctx, (void**)&m->y, R * S * D * 4));
    if (c.bf16) TRY(dev_alloc(ctx, &m->hs, R * S * D * e));
    TRY(dev_alloc(ctx, (void**)&m->slot_expert, R * S * 4));
    TRY(dev_alloc(ctx, (void**)&m->slot_w, R * S * 4));
    TRY(dev_alloc(ctx, (void**)&m->part_w, R * c.P * 4));
    TRY(dev_alloc(ctx, (void**)&m->sorted_row, R * S * 4));
    TRY(dev_alloc(ctx, (void**)&m->slot_pos, R * S * 4));
    if (!m->expert_count) {
      const size_t ne = (size_t)c.P * c.E;
      TRY(dev_alloc(ctx, (void**)&m->expert_count, ne * 4));
      VN_CUDA(ctx, cudaMemsetAsync(m->expert_count, 0, ne * 4, ctx->stream));
      TRY(dev_alloc(ctx, (void**)&m->expert_off, ne * 4));
      TRY(dev_alloc(ctx, (void**)&m->expert_cur, ne * 4));
      VN_CUDA(ctx, cudaMemsetAsync(m->expert_cur, 0, ne * 4, ctx->stream));
    }
  }
  m->cap_rows = (int)R;
  return VN_OK;
}

// one Linear: C = A @ W^T with the epilogue, dispatching on the storage dtype
int32_t ensure_partial(vn_model* m, size_t bytes);

int32_t linear(vn_model* m, GemmArgs g) {
  vn_ctx* ctx = m->ctx;
  if (g.wq) {
    if (!gemm_mma_q_supported(g)) return vn_fail(ctx, VN_ERR_UNSUPPORTED, "quantised GEMM shape K=%d unsupported", g.K);
    return launch_gemm_mma_q(ctx, g);
  }
  if (m->cfg.bf16) {
    // Many rows (a prompt): the tcgen05 kernel takes the rows as segments of 256 -- the same code path as the experts'
    // row segments, every segment with the same weight matrix (stride 0).  A weight tile is then fetched once per
    // segment, from L2 after the first.  VN_PREFILL_TC=0 (read per call) keeps the mma.sync kernel.
    const char* pe = getenv("VN_PREFILL_TC");
    if (m->use_tc && !(pe && pe[0] == '0') && g.M > 256 && !g.seg_cnt && !g.a_rows && g.nseg == 1 && !g.bias &&
        g.K % tc_detail::BK == 0 && g.N >= tc_detail::BF && g.ldw_k == 1 && tc_detail::encode_fn() != nullptr &&
        (g.epi == EPI_STORE || g.epi == EPI_ADD || g.epi == EPI_SWIGLU)) {
      const int nseg = ceil_div(g.M, 256);
      if (nseg <= m->row_seg_cap) {
      VN_LAUNCH(ctx, row_segments_kernel, ceil_div(nseg, 128), 128, 0, m->row_seg, m->row_seg + m->row_seg_cap, nseg, g.M);
      TRY(ensure_partial(m, 1024));                               // the error word
      GemmArgs g2 = g;
      g2.M = 256; g2.seg_off = m->row_seg; g2.seg_cnt = m->row_seg + m->row_seg_cap; g2.nseg = nseg; g2.w_stride = 0;
      if (gemm_tc_supported(g2)) {
        TcPlan plan;
        plan.error_flag = m->tc_error;
        return launch_gemm_tc(ctx, g2, g.M, plan);
      }
      }
    }
    if (gemm_mma_supported(g)) return launch_gemm_mma(ctx, g);
    return launch_gemm_simt<__nv_bfloat16, __nv_bfloat16>(ctx, g);
  }
  return launch_gemm_simt<float, float>(ctx, g);
}

// The attention part of a vda / dsa / kda / gmla layer (verse_nex/delta_attention.py): m->h (normalised rows) ->
// m->attn (head-space output before the layer's projection).  Every module projects on its own, rotates and appends
// its K / V to its own plane pair and runs its attention; a vda layer sums its three modules with
// sigmoid(gate_logits) (:1167-1168) through the fp32 buffer m->mix.
float delta_mix_weight(const Layer& L, int si) {
  return L.sub.size() > 1 ? 0.5f * (1.0f + tanhf(0.5f * L.gate_logits[si])) : 1.0f;
}

// arguments of the tensor-core attention kernel for module `si` of a delta layer (bf16, head_dim 64)
AttnArgs delta_mma_args(vn_model* m, vn_kv* kv, Layer& L, int si, int Tn, bool tree, int slot_offset) {
  const Config& c = m->cfg;
  SubAttn& S = L.sub[si];
  const int n_sub = (int)L.sub.size();
  AttnArgs a;
  a.q = m->qkv; a.ld_q = (c.n_head + 2 * c.n_kv) * c.hd; a.kc = kv->k[S.pair]; a.vc = kv->v[S.pair];
  a.sink_k = S.sink_k; a.sink_v = S.sink_v;
  a.out = si + 1 == n_sub ? m->attn : nullptr;
  a.acc_in = si > 0 ? m->mix : nullptr;
  a.acc_out = si + 1 < n_sub ? m->mix : nullptr;
  a.lens = kv->lens; a.depth = tree ? m->depth_dev : nullptr; a.anc = tree ? m->anc_dev : nullptr;
  a.Tn = Tn; a.H = c.n_head; a.n_kv = c.n_kv; a.hd = c.hd; a.max_seq = kv->max_seq; a.window = c.window;
  a.n_sink = S.mode == 0 ? c.n_sink : 0; a.slot_offset = slot_offset;
  a.use_alibi = 1; a.alibi_max = 1024; a.alibi_window = 0;       // the dense pass and its switch at 1024 keys
  // the one-token route (vn_model_set_recurrent): every row is a call of its own; DSA and KDA have no switch there
  // (delta_attention.py:594-597, :788-799), GMLA's looks at the row's own key count (:1059)
  a.row_tk = m->recurrent ? 1 : 0;
  if (m->recurrent && S.mode != 2) a.alibi_max = 0x7fffffff;
  a.g_a = a.g_b = a.g_c = 0.f;
  a.scale = 1.0f / sqrtf((float)c.hd);
  a.delta = S.mode + 1; a.head_w = S.head_w; a.out_w = delta_mix_weight(L, si); a.anchor = c.anchor;
  return a;
}

template <typename T>
int32_t delta_attention(vn_model* m, vn_kv* kv, Layer& L, int B, int Tn, bool tree, int slot_offset) {
  vn_ctx* ctx = m->ctx;
  const Config& c = m->cfg;
  const int M = B * Tn, D = c.dim, H = c.n_head, hd = c.hd, n_kv = c.n_kv;
  const int qd = H * hd, kvd = n_kv * hd, qkv_ld = qd + 2 * kvd;
  const int n_sub = (int)L.sub.size();
  for (int si = 0; si < n_sub; ++si) {
    SubAttn& S = L.sub[si];
    GemmArgs g;
    g.A = m->h; g.lda = D; g.W = S.wqkv; g.ldw = D; g.C = m->qkv; g.ldc = qkv_ld; g.M = M; g.K = D;
    if (S.mode == 2 && S.w_abs) {
      g.W = S.w_abs; g.N = qkv_ld; g.tag = "gemm_qkv";
      TRY(linear(m, g));
    } else if (S.mode == 2) {
      // q; latent = w_kv_down(h) in the storage dtype; k | v = (w_k_up | w_v_up)(latent)   (:893-896)
      g.N = qd; g.tag = "gemm_gmla_q";
      pick_sub(m, g, S, 0, 0);
      TRY(linear(m, g));
      g = GemmArgs();
      g.A = m->h; g.lda = D; g.W = S.w_down; g.ldw = D; g.C = m->lat; g.ldc = c.latent; g.M = M; g.N = c.latent; g.K = D;
      g.c_bf16 = c.bf16; g.tag = "gemm_gmla_down";
      pick_sub(m, g, S, 0, qd);
      TRY(linear(m, g));
      g = GemmArgs();
      g.A = m->lat; g.lda = c.latent; g.W = S.w_up; g.ldw = c.latent; g.C = m->qkv + qd; g.ldc = qkv_ld; g.M = M;
      g.N = 2 * kvd; g.K = c.latent; g.tag = "gemm_gmla_up";
      pick_sub(m, g, S, 1, 0);
      TRY(linear(m, g));
    } else {
      g.N = qkv_ld; g.tag = "gemm_qkv";
      pick_sub(m, g, S, 0, 0);
      TRY(linear(m, g));
    }
    VN_LAUNCH(ctx, rope_append_kernel<T>, M, 128, 0, m->qkv, m->rope_cos, m->rope_sin, kv->lens,
              tree ? m->depth_dev : (const int*)nullptr, (T*)kv->k[S.pair], (T*)kv->v[S.pair], Tn, H, n_kv, hd, kv->max_seq,
              c.use_rope, m->rope_rows, slot_offset);
    AttnArgs am = delta_mma_args(m, kv, L, si, Tn, tree, slot_offset);
    if (attn_mma_supported(am, c.bf16 != 0) && !m->force_simt_attn) {
      TRY(launch_attn_mma(ctx, am, B));
      continue;
    }
    DeltaArgs a;
    a.q = m->qkv; a.ld_q = qkv_ld; a.kc = kv->k[S.pair]; a.vc = kv->v[S.pair]; a.sink_k = S.sink_k; a.sink_v = S.sink_v;
    a.head_gate = S.head_gate;
    a.acc_in = si > 0 ? m->mix : nullptr;
    a.acc_out = si + 1 < n_sub ? m->mix : nullptr;
    a.out = si + 1 == n_sub ? m->attn : nullptr;
    a.out_w = delta_mix_weight(L, si);
    a.lens = kv->lens; a.depth = tree ? m->depth_dev : nullptr; a.anc = tree ? m->anc_dev : nullptr;
    a.Tn = Tn; a.H = H; a.n_kv = n_kv; a.hd = hd; a.max_seq = kv->max_seq; a.window = c.window; a.n_sink = c.n_sink;
    a.slot_offset = slot_offset; a.anchor = c.anchor; a.max_t = (m->recurrent && S.mode != 2) ? 0x7fffffff : 1024;
    a.row_tk = m->recurrent ? 1 : 0; a.mode = S.mode;
    a.scale = 1.0f / sqrtf((float)hd);
    dim3 grid(ceil_div(H, 8), M);
    VN_LAUNCH(ctx, delta_attn_kernel<T>, grid, 256, 0, a);
  }
  return VN_OK;
}

template <typename T>
int32_t forward_t(vn_model* m, vn_kv* kv, const int64_t* tokens, int B, int Tn, bool tree, float* out_hidden,
                  float* out_logits, int last_only, int slot_offset) {
  vn_ctx* ctx = m->ctx;
  const Config& c = m->cfg;
  const int M = B * Tn, D = c.dim, H = c.n_head, hd = c.hd, n_kv = c.n_kv;
  const int qkv_ld = (H + 2 * n_kv) * hd;
  const float emb_scale = c.emb_scale ? sqrtf((float)D) : 1.0f;
  // dense weight, or its quantised copy with the scales (rows_per_seg: output rows of one expert)
  auto pick = [&](GemmArgs& g, void* dense, void* q, float* qs, long long rows_per_seg) {
    if (m->qmode) {
      g.W = q; g.w_scale = qs; g.wq = m->qmode;
      g.ws_stride = rows_per_seg * (m->qmode == 3 ? (g.K + 127) / 128 : 1);
    } else {
      g.W = dense;
    }
  };
  VN_LAUNCH(ctx, embed_kernel<T>, M, 128, 0, (const long long*)tokens, (const T*)m->emb, m->x, D, c.vocab, emb_scale,
            m->status);
  for (int li = 0; li < c.n_layer; ++li) {
    Layer& L = m->layers[li];
    VN_LAUNCH(ctx, rmsnorm_kernel<T>, M, 256, 0, m->x, L.norm1, (T*)m->h, (float*)nullptr, 1, 0, D, 1e-6f);
    GemmArgs g;
    if (is_delta(L.kind)) {
      TRY(delta_attention<T>(m, kv, L, B, Tn, tree, slot_offset));
    } else {
    const int pr = m->pair0[li];
    g.A = m->h; g.lda = D; g.W = L.wqkv; g.ldw = D; g.C = m->qkv; g.ldc = qkv_ld; g.M = M; g.N = qkv_ld; g.K = D;
    g.tag = "gemm_qkv";
    pick(g, L.wqkv, L.q[0], L.qs[0], 0);
    TRY(linear(m, g));
    VN_LAUNCH(ctx, rope_append_kernel<T>, M, 128, 0, m->qkv, m->rope_cos, m->rope_sin, kv->lens,
              tree ? m->depth_dev : (const int*)nullptr, (T*)kv->k[pr], (T*)kv->v[pr], Tn, H, n_kv, hd, kv->max_seq,
              c.use_rope, m->rope_rows, slot_offset);
    AttnArgs a;
    a.q = m->qkv; a.ld_q = qkv_ld; a.kc = kv->k[pr]; a.vc = kv->v[pr]; a.sink_k = L.sink_k; a.sink_v = L.sink_v;
    a.out = m->attn; a.lens = kv->lens; a.depth = tree ? m->depth_dev : nullptr; a.anc = tree ? m->anc_dev : nullptr;
    a.Tn = Tn; a.H = H; a.n_kv = n_kv; a.hd = hd; a.max_seq = kv->max_seq; a.window = c.window; a.n_sink = c.n_sink;
    a.use_alibi = c.use_alibi; a.alibi_max = 1024; a.slot_offset = slot_offset;
    a.alibi_window = m->recurrent ? c.window : 0;
    a.g_a = 1.f / (1.f + expf(-L.gate_logits[0]));
    a.g_b = 1.f / (1.f + expf(-L.gate_logits[1]));
    a.g_c = 1.f / (1.f + expf(-L.gate_logits[2]));
    a.scale = 1.0f / sqrtf((float)hd);
    if (attn_prefill_supported(a, c.bf16 != 0) && !m->force_simt_attn) {
      TRY(launch_attn_prefill(ctx, a, B));
    } else if (attn_mma_supported(a, c.bf16 != 0) && !m->force_simt_attn) {
      TRY(launch_attn_mma(ctx, a, B));
    } else {
      dim3 grid(ceil_div(H, 8), M);
      VN_LAUNCH(ctx, trisparse_attn_kernel<T>, grid, 256, 0, a);
    }
    }
    g = GemmArgs();
    g.A = m->attn; g.lda = H * hd; g.W = L.wproj; g.ldw = H * hd; g.C = m->x; g.ldc = D; g.M = M; g.N = D; g.K = H * hd;
    g.epi = EPI_ADD; g.tag = "gemm_proj";
    pick(g, L.wproj, L.q[1], L.qs[1], 0);
    TRY(linear(m, g));
    const bool mod = L.kind == 1;
    VN_LAUNCH(ctx, rmsnorm_kernel<T>, M, 256, 0, m->x, L.norm2, (T*)m->h, mod ? m->h32 : (float*)nullptr,
              1, 0, D, 1e-6f);
    if (!mod) {
      g = GemmArgs();
      g.A = m->h; g.lda = D; g.W = L.w_gateup; g.ldw = D; g.C = m->act; g.ldc = c.mlp_hidden; g.M = M;
      g.N = 2 * c.mlp_hidden; g.K = D; g.epi = EPI_SWIGLU; g.c_bf16 = c.bf16; g.tag = "gemm_gateup";
      pick(g, L.w_gateup, L.q[2], L.qs[2], 0);
      TRY(linear(m, g));
      g = GemmArgs();
      g.A = m->act; g.lda = c.mlp_hidden; g.W = L.w_down; g.ldw = c.mlp_hidden; g.C = m->x; g.ldc = D; g.M = M; g.N = D;
      g.K = c.mlp_hidden; g.epi = EPI_ADD; g.tag = "gemm_down";
      pick(g, L.w_down, L.q[3], L.qs[3], 0);
      TRY(linear(m, g));
    } else {
      const int ne = c.P * c.E, S = c.P * c.top_k, eh = c.expert_hidden;
      VN_CUDA(ctx, cudaMemsetAsync(m->expert_count, 0, ne * 4, ctx->stream));
      RouteArgs r;
      r.h = m->h32; r.gates = L.router; r.slot_expert = m->slot_expert; r.slot_w = m->slot_w; r.part_w = m->part_w;
      r.expert_count = m->expert_count; r.M = M; r.D = D; r.P = c.P; r.E = c.E; r.top_k = c.top_k;
      VN_LAUNCH(ctx, mod_route_kernel, M, 128, 0, r);
      VN_LAUNCH(ctx, mod_offsets_kernel, 1, 32, 0, m->expert_count, m->expert_off, m->expert_cur, ne);
      VN_LAUNCH(ctx, mod_scatter_kernel, ceil_div(M * S, 256), 256, 0, m->slot_expert, m->expert_off, m->expert_cur,
                m->sorted_row, m->slot_pos, M * S, S);
      // Many routed rows on a bf16 model: the experts' segments are cut into pieces of at most 256 rows and run on
      // the tcgen05 kernel (rows copied into expert order first, so that TMA loads them; a piece names its expert's
      // weights through seg_w).  Otherwise the mma.sync kernels gather the rows themselves.
      const char* pe = getenv("VN_PREFILL_TC");
      const int n_sub = ne + ceil_div(M * S, 256);
      const bool tc_experts = std::is_same<T, __nv_bfloat16>::value && m->use_tc && !m->qmode && !(pe && pe[0] == '0') &&
                              (long long)M * S > 256 && m->hs && D % 8 == 0 && eh % 8 == 0 && n_sub <= 65535 && n_sub <= m->sub_cap &&
                              tc_detail::encode_fn() != nullptr;
      if (tc_experts) {
        int* sub_off = m->sub_seg; int* sub_cnt = m->sub_seg + m->sub_cap; int* sub_w = m->sub_seg + 2 * m->sub_cap;
        VN_LAUNCH(ctx, mod_subseg_kernel, 1, 32, 0, (const int*)m->expert_count, (const int*)m->expert_off, ne, sub_off,
                  sub_cnt, sub_w, n_sub);
        VN_LAUNCH(ctx, gather_sorted_kernel<T>, M * S, 128, 0, (const T*)m->h, (const int*)m->sorted_row, (T*)m->hs, D);
        TRY(ensure_partial(m, 1024));
        TcPlan plan;
        plan.error_flag = m->tc_error;
        g = GemmArgs();
        g.A = m->hs; g.lda = D; g.W = L.e_gateup; g.ldw = D; g.w_stride = (long long)2 * eh * D;
        g.C = m->act; g.ldc = eh; g.M = 256; g.N = 2 * eh; g.K = D; g.epi = EPI_SWIGLU; g.c_bf16 = 1;
        g.seg_off = sub_off; g.seg_cnt = sub_cnt; g.seg_w = sub_w; g.n_w = ne; g.nseg = n_sub; g.tag = "gemm_expert_gateup";
        TRY(launch_gemm_tc(ctx, g, (long long)M * S, plan));
        g = GemmArgs();
        g.A = m->act; g.lda = eh; g.W = L.e_down; g.ldw = eh; g.w_stride = (long long)D * eh; g.C = m->y; g.ldc = D;
        g.M = 256; g.N = D; g.K = eh; g.seg_off = sub_off; g.seg_cnt = sub_cnt; g.seg_w = sub_w; g.n_w = ne; g.nseg = n_sub;
        g.tag = "gemm_expert_down";
        TcPlan plan2;
        plan2.error_flag = m->tc_error;
        TRY(launch_gemm_tc(ctx, g, (long long)M * S, plan2));
      } else {
      g = GemmArgs();
      g.A = m->h; g.lda = D; g.a_rows = m->sorted_row; g.W = L.e_gateup; g.ldw = D; g.w_stride = (long long)2 * eh * D;
      g.C = m->act; g.ldc = eh; g.M = M; g.N = 2 * eh; g.K = D; g.epi = EPI_SWIGLU; g.c_bf16 = c.bf16;
      g.seg_off = m->expert_off; g.seg_cnt = m->expert_count; g.nseg = ne; g.tag = "gemm_expert_gateup";
      pick(g, L.e_gateup, L.q[4], L.qs[4], 2 * eh);
      TRY(linear(m, g));
      g = GemmArgs();
      g.A = m->act; g.lda = eh; g.W = L.e_down; g.ldw = eh; g.w_stride = (long long)D * eh; g.C = m->y; g.ldc = D;
      g.M = M; g.N = D; g.K = eh; g.seg_off = m->expert_off; g.seg_cnt = m->expert_count; g.nseg = ne;
      g.tag = "gemm_expert_down";
      pick(g, L.e_down, L.q[5], L.qs[5], D);
      TRY(linear(m, g));
      }
      VN_LAUNCH(ctx, mod_combine_kernel, M, 256, 0, m->x, m->y, m->slot_pos, m->slot_w, m->part_w, D, c.P, c.top_k);
      VN_CUDA(ctx, cudaMemsetAsync(m->expert_count, 0, ne * 4, ctx->stream));   // zero between forwards
      VN_CUDA(ctx, cudaMemsetAsync(m->expert_cur, 0, ne * 4, ctx->stream));
    }
  }
  // final norm + head on every row, or on the last position of every sequence
  const int rows_out = last_only ? B : M;
  const int row_mul = last_only ? Tn : 1, row_add = last_only ? Tn - 1 : 0;
  VN_LAUNCH(ctx, rmsnorm_kernel<T>, rows_out, 256, 0, m->x, m->norm_f, (T*)m->h, out_hidden, row_mul, row_add, D, 1e-6f);
  if (out_logits) {
    GemmArgs g;
    g.A = m->h; g.lda = D; g.W = m->head; g.ldw = D; g.C = out_logits; g.ldc = c.vocab; g.M = rows_out; g.N = c.vocab;
    g.K = D; g.tag = "gemm_head";
    pick(g, m->head, m->head_q, m->head_qs, 0);
    TRY(linear(m, g));
  }
  return VN_OK;
}

// ---- decode / verify forward on the tcgen05 weight-streaming GEMM (bf16, at most 256 rows) ----------------
// Same arithmetic as forward_t<bf16>; the differences are scheduling: small-N GEMMs are split along K so that
// about two CTAs per SM stream weights, their partials are reduced by a finalize kernel that also applies the
// residual add and the next RMSNorm, and routed tokens are gathered into expert order so that TMA can load them.
int32_t ensure_partial(vn_model* m, size_t bytes) {
  vn_ctx* ctx = m->ctx;
  if (!m->tc_error) {
    TRY(dev_alloc(ctx, (void**)&m->tc_error, 4));
    VN_CUDA(ctx, cudaMemsetAsync(m->tc_error, 0, 4, ctx->stream));
    TRY(dev_alloc(ctx, (void**)&m->stack_bar, 8));
    VN_CUDA(ctx, cudaMemsetAsync(m->stack_bar, 0, 8, ctx->stream));
  }
  if (bytes <= m->partial_bytes) return VN_OK;
  VN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  if (m->partial) VN_CUDA(ctx, cudaFree(m->partial));
  m->partial = nullptr; m->partial_bytes = 0;
  const size_t want = bytes + (bytes >> 2);
  TRY(dev_alloc(ctx, (void**)&m->partial, want));
  m->partial_bytes = want;
  return VN_OK;
}

// choose a split count so that tiles * splits covers the GPU about twice, never more than the k blocks
int tc_splits(const vn_ctx* ctx, int N, int K, int nseg) {
  const int tiles = ceil_div(N, tc_detail::BF) * nseg;
  const int nkb = ceil_div(K, tc_detail::BK);
  // every slice costs a partial tile written and read back (rows x 128 x 4 bytes), so split only until the
  // GPU is covered about once, and never below VN_TC_MIN_KB k blocks per CTA
  static const int min_kb = [] { const char* e = getenv("VN_TC_MIN_KB"); return e ? std::max(1, atoi(e)) : 4; }();
  int s = ceil_div(ctx->sm_count, tiles);
  s = std::max(1, std::min(s, std::max(1, nkb / min_kb)));
  const int per = ceil_div(nkb, s);
  return ceil_div(nkb, per);   // effective number of K ranges
}

// dense bf16 weights or their quantised copy: the same pipeline, with the dequantising operand stage in front
int32_t tc_launch(vn_ctx* ctx, const GemmArgs& g, long long a_rows, TcPlan& plan) {
  return g.wq ? launch_gemm_tcq(ctx, g, a_rows, plan) : launch_gemm_tc(ctx, g, a_rows, plan);
}

// launches the GEMM into the split-K workspace; returns the number of partial slices through *splits_out
int32_t tc_partial(vn_model* m, GemmArgs g, long long a_rows, long long c_rows, int* splits_out) {
  vn_ctx* ctx = m->ctx;
  const int splits = tc_splits(ctx, g.N, g.K, g.nseg);
  TRY(ensure_partial(m, (size_t)splits * c_rows * g.N * 4));
  TcPlan plan;
  plan.splits = splits; plan.force_partial = true;
  plan.partial = m->partial; plan.rows_total = c_rows; plan.error_flag = m->tc_error;
  TRY(tc_launch(ctx, g, a_rows, plan));
  *splits_out = plan.splits_used;
  return VN_OK;
}

// a GEMM whose whole K range fits one CTA: the epilogue (SwiGLU, RoPE + cache append) runs in the GEMM itself
int32_t tc_cluster(vn_model* m, const GemmArgs& g, long long a_rows, int mode, float* resid,
                   const tc_detail::TcRope* rope) {
  vn_ctx* ctx = m->ctx;
  TcPlan plan;
  plan.splits = 1;
  plan.error_flag = m->tc_error;
  plan.cluster_mode = mode;
  plan.resid = resid;
  if (rope) plan.rope = *rope;
  return launch_gemm_tc(ctx, g, a_rows, plan);
}

// ---- the fused layer stack (draft_kernel.cuh): which models and shapes it takes, and its launch -----------
// Off unless vn_model_set_fused_stack(model, 1) or VN_DRAFT_STACK=1 in the environment asks for it: on B200 the
// chain of separate kernels with programmatic dependent launch is as fast (the ten grid barriers of a 2-layer model
// cost what the launches cost), so the chain stays the default.
bool draft_stack_ok(const vn_model* m, const vn_kv* kv, int B, int Tn, bool tree) {
  static const bool env_on = [] { const char* e = getenv("VN_DRAFT_STACK"); return e && e[0] == '1'; }();
  const Config& c = m->cfg;
  if (!(env_on || m->fused_stack) || tree || m->esz != 2 || m->qmode || !m->use_tc || m->force_simt_attn || c.use_rope) return false;
  if (c.n_layer > draft_detail::MAX_LAYERS || c.hd != 64 || c.n_head % c.n_kv) return false;
  for (int li = 0; li < c.n_layer; ++li)
    if (m->layers[li].kind != 0) return false;
  const int M = B * Tn, qd = c.n_head * c.hd;
  if (M < 1 || M > 64 || c.dim > 256 * draft_detail::NORM_TRIPS || (c.dim % 16) || (qd % 16) || (c.mlp_hidden % 16)) return false;
  const int widest = std::max(std::max(c.dim, qd), c.mlp_hidden);
  if ((size_t)((M + 15) & ~15) * (widest + 8) * 2 > (size_t)draft_detail::STAGE_BYTES) return false;
  if (draft_detail::wbuf_bytes(c.dim, qd, qd + 2 * c.n_kv * c.hd, c.mlp_hidden, 128) > 32768) return false;
  (void)kv;
  return true;
}

int32_t launch_draft_stack(vn_model* m, vn_kv* kv, const int64_t* tokens, int B, int Tn, float* out_hidden, int last_only,
                           int slot_offset) {
  vn_ctx* ctx = m->ctx;
  const Config& c = m->cfg;
  draft_detail::Args a;
  for (int li = 0; li < c.n_layer; ++li) {
    const Layer& L = m->layers[li];
    draft_detail::LayerW& w = a.L[li];
    w.wqkv = (const __nv_bfloat16*)L.wqkv; w.wproj = (const __nv_bfloat16*)L.wproj;
    w.wgu = (const __nv_bfloat16*)L.w_gateup; w.wdown = (const __nv_bfloat16*)L.w_down;
    w.norm1 = L.norm1; w.norm2 = L.norm2; w.sink_k = L.sink_k; w.sink_v = L.sink_v;
    w.kc = kv->k[li]; w.vc = kv->v[li];
    w.g_a = 1.f / (1.f + expf(-L.gate_logits[0]));
    w.g_b = 1.f / (1.f + expf(-L.gate_logits[1]));
    w.g_c = 1.f / (1.f + expf(-L.gate_logits[2]));
  }
  a.n_layer = c.n_layer; a.B = B; a.Tn = Tn; a.D = c.dim; a.H = c.n_head; a.n_kv = c.n_kv; a.hd = c.hd;
  a.hidden = c.mlp_hidden; a.V = c.vocab;
  a.tokens = (const long long*)tokens; a.emb = (const __nv_bfloat16*)m->emb;
  a.emb_scale = c.emb_scale ? sqrtf((float)c.dim) : 1.0f; a.norm_f = m->norm_f;
  a.x = m->x; a.q = m->qkv; a.attn = (__nv_bfloat16*)m->attn; a.act = (__nv_bfloat16*)m->act;
  a.h_out = (__nv_bfloat16*)m->h; a.hidden_out = out_hidden;
  a.lens = kv->lens; a.max_seq = kv->max_seq; a.window = c.window; a.n_sink = c.n_sink; a.use_alibi = c.use_alibi;
  a.alibi_window = m->recurrent ? c.window : 0; a.slot_offset = slot_offset; a.last_only = last_only;
  a.bar = m->stack_bar; a.status = m->status; a.error_flag = m->tc_error;
  // VN_STACK_TRACE=1 (debugging aid, eager launches only): CTA 0's time stamps at the phase boundaries go to stderr
  static const bool trace_on = [] { const char* e = getenv("VN_STACK_TRACE"); return e && e[0] == '1'; }();
  static long long* trace_dev = nullptr;
  cudaStreamCaptureStatus cap_st = cudaStreamCaptureStatusNone;
  a.trace = nullptr;
  if (trace_on) {
    cudaStreamIsCapturing(ctx->stream, &cap_st);
    if (cap_st == cudaStreamCaptureStatusNone) {
      if (!trace_dev) cudaMalloc(&trace_dev, 64 * sizeof(long long));
      cudaMemsetAsync(trace_dev, 0, 64 * sizeof(long long), ctx->stream);
      a.trace = trace_dev;
    }
  }
  const int n_rep = c.n_head / c.n_kv;
  const int n_items = B * c.n_kv * ceil_div(Tn * n_rep, 16);
  const int grid = std::min(ctx->sm_count, n_items > 128 ? ctx->sm_count : 128);
  const int qd = c.n_head * c.hd;
  const size_t smem = draft_detail::STAGE_BYTES + draft_detail::RED_BYTES + draft_detail::wbuf_bytes(c.dim, qd, qd + 2 * c.n_kv * c.hd, c.mlp_hidden, grid);
  static unsigned long long attr_set = 0;
  if (!((attr_set >> (ctx->device & 63)) & 1ull)) {
    VN_CUDA(ctx, cudaFuncSetAttribute(draft_detail::draft_layers_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      draft_detail::STAGE_BYTES + draft_detail::RED_BYTES + 32768));
    attr_set |= 1ull << (ctx->device & 63);
  }
  // cooperative: all CTAs are resident together, which the grid barriers need
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid); cfg.blockDim = dim3(draft_detail::DT); cfg.dynamicSmemBytes = smem; cfg.stream = ctx->stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeCooperative; at[0].val.cooperative = 1;
  cfg.attrs = at; cfg.numAttrs = 1;
  if (ctx->profiling) vn_prof_begin(ctx, "draft_layers_kernel");
  cudaError_t e = cudaLaunchKernelEx(&cfg, draft_detail::draft_layers_kernel, a);
  if (ctx->profiling) vn_prof_end(ctx);
  ctx->launches++;
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return vn_fail(ctx, VN_ERR_CUDA, "launch of draft_layers_kernel failed: %s", cudaGetErrorString(e));
  if (a.trace) {
    long long t[64];
    cudaStreamSynchronize(ctx->stream);
    cudaMemcpy(t, trace_dev, sizeof t, cudaMemcpyDeviceToHost);
    fprintf(stderr, "stack trace (us since start):");
    for (int i = 1; i < 64 && t[i]; ++i) fprintf(stderr, " %.2f", (t[i] - t[0]) * 1e-3);
    fprintf(stderr, "\n");
  }
  return VN_OK;
}

// The same on the decode / verify route (bf16, head_dim 64, at most 256 rows): every projection is a split-K
// tcgen05 GEMM; a DSA / KDA module's q | k | v slices are summed, rotated and appended by its attention CTAs (as for a
// TriSparse layer), a GMLA module goes through its latent (two GEMMs with a reduction kernel behind each).
bool delta_tc_ok(const vn_model* m, int Tn, bool tree) {
  const Config& c = m->cfg;
  return c.hd == 64 && c.latent % 8 == 0 && !m->force_simt_attn && (!tree || Tn <= 64);
}

int32_t delta_attention_tc(vn_model* m, vn_kv* kv, Layer& L, int B, int Tn, bool tree, int slot_offset) {
  typedef __nv_bfloat16 T;
  vn_ctx* ctx = m->ctx;
  const Config& c = m->cfg;
  const int M = B * Tn, D = c.dim, H = c.n_head, hd = c.hd, n_kv = c.n_kv, lat = c.latent;
  const int qd = H * hd, kvd = n_kv * hd, qkv_ld = qd + 2 * kvd;
  const long long cap = m->cap_rows;
  static const bool fuse_on = [] { const char* e = getenv("VN_ATTN_FUSE"); return !(e && e[0] == '0'); }();
  const int* depth = tree ? m->depth_dev : (const int*)nullptr;
  if (L.w_vda && !m->qmode && fuse_on && Tn <= 64 && qkv_ld % 4 == 0) {
    // one GEMM for the three modules' q | k | v; every module's attention CTAs reduce their own column block
    int sp = 1;
    GemmArgs g;
    g.A = m->h; g.lda = D; g.W = L.w_vda; g.ldw = D; g.M = M; g.N = 3 * qkv_ld; g.K = D; g.tag = "gemm_qkv";
    TRY(tc_partial(m, g, cap, M, &sp));
    for (int si = 0; si < 3; ++si) {
      AttnArgs a = delta_mma_args(m, kv, L, si, Tn, tree, slot_offset);
      a.partial = m->partial + (size_t)si * qkv_ld; a.splits = sp; a.pstride = (long long)M * 3 * qkv_ld;
      a.partial_ld = 3 * qkv_ld;
      a.cos_t = m->rope_cos; a.sin_t = m->rope_sin; a.use_rope = c.use_rope; a.rope_rows = m->rope_rows;
      TRY(launch_attn_mma(ctx, a, B));
    }
    return VN_OK;
  }
  for (int si = 0; si < (int)L.sub.size(); ++si) {
    SubAttn& S = L.sub[si];
    AttnArgs a = delta_mma_args(m, kv, L, si, Tn, tree, slot_offset);
    T* kc = (T*)kv->k[S.pair];
    T* vc = (T*)kv->v[S.pair];
    int sp = 1;
    GemmArgs g;
    g.A = m->h; g.lda = D; g.W = S.wqkv; g.ldw = D; g.M = M; g.K = D;
    if (S.mode != 2 || S.w_abs) {
      if (S.w_abs) g.W = S.w_abs;
      g.N = qkv_ld; g.tag = "gemm_qkv";
      pick_sub(m, g, S, 0, 0);
      TRY(tc_partial(m, g, cap, M, &sp));
      if (fuse_on && Tn <= 64 && qkv_ld % 4 == 0) {
        a.partial = m->partial; a.splits = sp; a.pstride = (long long)M * qkv_ld; a.partial_ld = qkv_ld;
        a.cos_t = m->rope_cos; a.sin_t = m->rope_sin; a.use_rope = c.use_rope; a.rope_rows = m->rope_rows;
      } else {
        VN_LAUNCH_PDL_BIT(ctx, 2, qkv_finalize_kernel<T>, M, 256, (size_t)qkv_ld * 4, m->partial, sp, (long long)M * qkv_ld,
                          m->qkv, m->rope_cos, m->rope_sin, kv->lens, depth, kc, vc, Tn, H, n_kv, hd, kv->max_seq,
                          c.use_rope, m->rope_rows, slot_offset);
      }
    } else {
      const int n1 = qd + lat, n2 = 2 * kvd;
      g.N = n1; g.tag = "gemm_gmla_q_down";
      pick_sub(m, g, S, 0, 0);
      TRY(tc_partial(m, g, cap, M, &sp));
      VN_LAUNCH_PDL_BIT(ctx, 2, gmla_finalize_kernel<T>, M, 256, (size_t)n1 * 4, m->partial, sp, (long long)M * n1, n1, 1,
                        m->qkv, qkv_ld, (T*)m->lat, lat, m->rope_cos, m->rope_sin, kv->lens, depth, kc, vc, Tn, H, n_kv,
                        hd, kv->max_seq, c.use_rope, m->rope_rows, slot_offset);
      g = GemmArgs();
      g.A = m->lat; g.lda = lat; g.W = S.w_up; g.ldw = lat; g.M = M; g.N = n2; g.K = lat; g.tag = "gemm_gmla_up";
      pick_sub(m, g, S, 1, 0);
      TRY(tc_partial(m, g, cap, M, &sp));
      VN_LAUNCH_PDL_BIT(ctx, 2, gmla_finalize_kernel<T>, M, 256, (size_t)n2 * 4, m->partial, sp, (long long)M * n2, n2, 2,
                        m->qkv, qkv_ld, (T*)m->lat, lat, m->rope_cos, m->rope_sin, kv->lens, depth, kc, vc, Tn, H, n_kv,
                        hd, kv->max_seq, c.use_rope, m->rope_rows, slot_offset);
    }
    TRY(launch_attn_mma(ctx, a, B));
  }
  return VN_OK;
}

int32_t forward_tc(vn_model* m, vn_kv* kv, const int64_t* tokens, int B, int Tn, bool tree, float* out_hidden,
                   float* out_logits, int last_only, int slot_offset) {
  typedef __nv_bfloat16 T;
  vn_ctx* ctx = m->ctx;
  const Config& c = m->cfg;
  const int M = B * Tn, D = c.dim, H = c.n_head, hd = c.hd, n_kv = c.n_kv;
  const int qkv_ld = (H + 2 * n_kv) * hd;
  const long long cap = m->cap_rows;
  const float emb_scale = c.emb_scale ? sqrtf((float)D) : 1.0f;
  TcPlan direct;
  TRY(ensure_partial(m, 1024));
  direct.error_flag = m->tc_error;
  // dense weight, or its quantised copy with the scales (rows_per_seg: output rows of one expert)
  auto pick = [&](GemmArgs& g, void* q, float* qs, long long rows_per_seg) {
    if (!m->qmode) return;
    g.W = q; g.w_scale = qs; g.wq = m->qmode;
    g.ws_stride = rows_per_seg * (m->qmode == 3 ? (g.K + 127) / 128 : 1);
  };
  // A GEMM whose whole K range fits one CTA (the draft model's projections) has nothing to reduce: as a cluster
  // of one it applies RoPE + cache append or SwiGLU itself and the finalize kernel behind it disappears.
  static const bool single_on = [] { const char* e = getenv("VN_TC_SINGLE"); return !(e && e[0] == '0'); }();
  auto fused = [&](const GemmArgs& g) {
    return single_on && !m->qmode && tc_splits(ctx, g.N, g.K, 1) == 1;
  };
  const int rows_out = last_only ? B : M;
  // a small all-TriSparse model (the draft): the whole layer stack and the final norm in one cooperative kernel
  const bool stack = draft_stack_ok(m, kv, B, Tn, tree);
  if (stack) {
    TRY(launch_draft_stack(m, kv, tokens, B, Tn, out_hidden, last_only, slot_offset));
  } else {
  // expert_count is zero between forwards: the combine kernel of every MoD layer leaves it so
  VN_LAUNCH_PDL_BIT(ctx, 32, embed_norm_kernel<T>, M, 256, 0, (const long long*)tokens, (const T*)m->emb, m->x,
                m->layers[0].norm1, (T*)m->h, D, c.vocab, emb_scale, 1e-6f, m->status);
  for (int li = 0; li < c.n_layer; ++li) {
    Layer& L = m->layers[li];
    const bool mod = L.kind == 1;
    const bool last = li + 1 == c.n_layer;
    int sp = 1;
    GemmArgs g;
    // ---- attention block
    if (is_delta(L.kind)) {
      TRY(delta_attention_tc(m, kv, L, B, Tn, tree, slot_offset));
    } else {
    g.A = m->h; g.lda = D; g.W = L.wqkv; g.ldw = D; g.M = M; g.N = qkv_ld; g.K = D; g.tag = "gemm_qkv";
    pick(g, L.q[0], L.qs[0], 0);
    tc_detail::TcRope rope;
    rope.cos_t = m->rope_cos; rope.sin_t = m->rope_sin; rope.lens = kv->lens;
    rope.depth = tree ? m->depth_dev : (const int*)nullptr;
    rope.kc = kv->k[m->pair0[li]]; rope.vc = kv->v[m->pair0[li]]; rope.q_out = m->qkv; rope.ldq = qkv_ld;
    rope.Tn = Tn; rope.H = H; rope.n_kv = n_kv; rope.hd = hd; rope.max_seq = kv->max_seq;
    rope.use_rope = c.use_rope; rope.rope_rows = m->rope_rows; rope.slot_offset = slot_offset;
    AttnArgs a;
    a.q = m->qkv; a.ld_q = qkv_ld; a.kc = kv->k[m->pair0[li]]; a.vc = kv->v[m->pair0[li]]; a.sink_k = L.sink_k; a.sink_v = L.sink_v;
    a.out = m->attn; a.lens = kv->lens; a.depth = tree ? m->depth_dev : nullptr; a.anc = tree ? m->anc_dev : nullptr;
    a.Tn = Tn; a.H = H; a.n_kv = n_kv; a.hd = hd; a.max_seq = kv->max_seq; a.window = c.window; a.n_sink = c.n_sink;
    a.use_alibi = c.use_alibi; a.alibi_max = 1024; a.slot_offset = slot_offset;
    a.alibi_window = m->recurrent ? c.window : 0;
    a.g_a = 1.f / (1.f + expf(-L.gate_logits[0]));
    a.g_b = 1.f / (1.f + expf(-L.gate_logits[1]));
    a.g_c = 1.f / (1.f + expf(-L.gate_logits[2]));
    a.scale = 1.0f / sqrtf((float)hd);
    const bool attn_tc = attn_mma_supported(a, true) && !m->force_simt_attn;
    // the tensor-core attention kernel sums the projection's split-K slices itself (with RoPE and the cache append)
    // when a tile's CTA has few new rows to reduce; VN_ATTN_FUSE=0 keeps the separate finalize kernel
    static const bool fuse_on = [] { const char* e = getenv("VN_ATTN_FUSE"); return !(e && e[0] == '0'); }();
    if (fused(g) && gemm_tc_cluster_supported(g, tc_detail::TC_CL_QKV, &rope)) {
      TRY(tc_cluster(m, g, cap, tc_detail::TC_CL_QKV, nullptr, &rope));
    } else {
      TRY(tc_partial(m, g, cap, M, &sp));
      if (attn_tc && fuse_on && Tn <= 64 && qkv_ld % 4 == 0) {
        a.partial = m->partial; a.splits = sp; a.pstride = (long long)M * qkv_ld; a.partial_ld = qkv_ld;
        a.cos_t = m->rope_cos; a.sin_t = m->rope_sin; a.use_rope = c.use_rope; a.rope_rows = m->rope_rows;
      } else {
        VN_LAUNCH_PDL_BIT(ctx, 2, qkv_finalize_kernel<T>, M, 256, (size_t)qkv_ld * 4, m->partial, sp, (long long)M * qkv_ld,
                      m->qkv, m->rope_cos, m->rope_sin, kv->lens, tree ? m->depth_dev : (const int*)nullptr,
                      (T*)kv->k[m->pair0[li]], (T*)kv->v[m->pair0[li]], Tn, H, n_kv, hd, kv->max_seq, c.use_rope, m->rope_rows, slot_offset);
      }
    }
    if (attn_tc) {
      TRY(launch_attn_mma(ctx, a, B));
    } else {
      dim3 grid(ceil_div(H, 8), M);
      VN_LAUNCH(ctx, trisparse_attn_kernel<T>, grid, 256, 0, a);
    }
    }
    g = GemmArgs();
    g.A = m->attn; g.lda = H * hd; g.W = L.wproj; g.ldw = H * hd; g.M = M; g.N = D; g.K = H * hd; g.tag = "gemm_proj";
    g.ldc = D;
    pick(g, L.q[1], L.qs[1], 0);
    TRY(tc_partial(m, g, cap, M, &sp));
    VN_LAUNCH_PDL_BIT(ctx, 4, splitk_add_norm_kernel<T>, M, 256, 0, m->partial, sp, (long long)M * D, m->x, L.norm2,
                  (T*)m->h, mod ? m->h32 : (float*)nullptr, D, 1e-6f);
    // ---- feed-forward block
    const float* next_norm = last ? nullptr : m->layers[li + 1].norm1;
    if (!mod) {
      g = GemmArgs();
      g.A = m->h; g.lda = D; g.W = L.w_gateup; g.ldw = D; g.M = M; g.N = 2 * c.mlp_hidden; g.K = D;
      g.tag = "gemm_gateup";
      g.C = m->act; g.ldc = c.mlp_hidden; g.c_bf16 = 1;
      pick(g, L.q[2], L.qs[2], 0);
      // VN_GATEUP_SPLIT=0: one CTA per feature tile over the whole K range with the SwiGLU epilogue (no finalize
      // kernel, fewer but longer CTAs); 1: split-K partial tiles + the finalize kernel
      static const bool gateup_split = [] { const char* e = getenv("VN_GATEUP_SPLIT"); return !(e && e[0] == '0'); }();
      if (fused(g) && gemm_tc_cluster_supported(g, tc_detail::TC_CL_SWIGLU, nullptr)) {
        TRY(tc_cluster(m, g, cap, tc_detail::TC_CL_SWIGLU, nullptr, nullptr));
      } else if (!gateup_split) {
        g.epi = EPI_SWIGLU;
        TRY(tc_launch(ctx, g, cap, direct));
      } else {
        TRY(tc_partial(m, g, cap, M, &sp));
        const long long pairs = (long long)M * c.mlp_hidden;
        VN_LAUNCH_PDL_BIT(ctx, 8, splitk_swiglu_kernel<T>, (unsigned)ceil_div(pairs, 512ll), 256, 0, m->partial, sp,
                  (long long)M * 2 * c.mlp_hidden, (T*)m->act, 2 * c.mlp_hidden, pairs);
      }
      g = GemmArgs();
      g.A = m->act; g.lda = c.mlp_hidden; g.W = L.w_down; g.ldw = c.mlp_hidden; g.M = M; g.N = D; g.K = c.mlp_hidden;
      g.tag = "gemm_down";
      g.ldc = D;
      pick(g, L.q[3], L.qs[3], 0);
      TRY(tc_partial(m, g, cap, M, &sp));
      VN_LAUNCH_PDL_BIT(ctx, 4, splitk_add_norm_kernel<T>, M, 256, 0, m->partial, sp, (long long)M * D, m->x, next_norm,
                    (T*)m->h, (float*)nullptr, D, 1e-6f);
    } else {
      const int ne = c.P * c.E, S = c.P * c.top_k, eh = c.expert_hidden;
      RouteArgs r;
      r.h = m->h32; r.gates = L.router; r.slot_expert = m->slot_expert; r.slot_w = m->slot_w; r.part_w = m->part_w;
      r.expert_count = m->expert_count; r.M = M; r.D = D; r.P = c.P; r.E = c.E; r.top_k = c.top_k;
      VN_LAUNCH_PDL_BIT(ctx, 16, mod_route_kernel, M, 512, 0, r);
      VN_LAUNCH_PDL_BIT(ctx, 16, mod_dispatch_kernel<T>, M * S, 128, 0, (const T*)m->h, m->slot_expert, m->expert_count,
                    m->expert_off, m->expert_cur, m->slot_pos, (T*)m->hs, ne, S, D);
      g = GemmArgs();
      g.A = m->hs; g.lda = D; g.W = L.e_gateup; g.ldw = D; g.w_stride = (long long)2 * eh * D;
      g.C = m->act; g.ldc = eh; g.M = M; g.N = 2 * eh; g.K = D; g.epi = EPI_SWIGLU; g.c_bf16 = 1;
      g.seg_off = m->expert_off; g.seg_cnt = m->expert_count; g.nseg = ne; g.tag = "gemm_expert_gateup";
      pick(g, L.q[4], L.qs[4], 2 * eh);
      TRY(tc_launch(ctx, g, (long long)M * S, direct));
      g = GemmArgs();
      g.A = m->act; g.lda = eh; g.W = L.e_down; g.ldw = eh; g.w_stride = (long long)D * eh;
      g.M = M; g.N = D; g.K = eh; g.seg_off = m->expert_off; g.seg_cnt = m->expert_count; g.nseg = ne;
      g.tag = "gemm_expert_down";
      pick(g, L.q[5], L.qs[5], D);
      TRY(tc_partial(m, g, (long long)M * S, (long long)M * S, &sp));
      // the next block's first RMSNorm rides on the combine (its rows are in registers there)
      VN_LAUNCH_PDL_BIT(ctx, 16, mod_combine_split_kernel<T>, M, 256, 0, m->x, m->partial, sp, (long long)M * S * D, m->slot_pos,
                m->slot_w, m->part_w, D, c.P, c.top_k, m->expert_count, m->expert_cur, ne, next_norm, (T*)m->h, 1e-6f);
    }
  }
  const int row_mul = last_only ? Tn : 1, row_add = last_only ? Tn - 1 : 0;
  VN_LAUNCH_PDL_BIT(ctx, 32, rmsnorm_kernel<T>, rows_out, 256, 0, m->x, m->norm_f, (T*)m->h, out_hidden, row_mul, row_add, D, 1e-6f);
  }
  if (out_logits) {
    GemmArgs g;
    g.A = m->h; g.lda = D; g.W = m->head; g.ldw = D; g.C = out_logits; g.ldc = c.vocab; g.M = rows_out; g.N = c.vocab;
    g.K = D; g.tag = "gemm_head";
    pick(g, m->head_q, m->head_qs, 0);
    TRY(tc_launch(ctx, g, cap, direct));
  }
  return VN_OK;
}


// ---- linears addressed by their state_dict name: where their rows live in the stacked / interleaved matrices ----
struct LinearSlot {
  int layer = -1;        // -1: the LM head
  int sub = -1;          // >= 0: a module of a delta layer (slot then indexes SubAttn::q / qs: 0 q|k|v or q|down, 1 k|v up)
  int slot = 0;          // index into Layer::q / qs (0 qkv, 1 proj, 2 gate|up, 3 down, 4 expert gate|up, 5 expert down)
  long long base = 0, row_mul = 1, row_off = 0;   // destination row of source row r: base + r * row_mul + row_off
  long long rows = 0, K = 0;                      // shape of the named tensor
};

bool locate_linear(const vn_model* m, const std::string& n, LinearSlot* o) {
  const Config& c = m->cfg;
  const long long D = c.dim, qd = (long long)c.n_head * c.hd, kvd = (long long)c.n_kv * c.hd;
  if (n == "head.weight") { o->layer = -1; o->rows = c.vocab; o->K = D; return true; }
  if (n.rfind("blocks.", 0) != 0) return false;
  const size_t dot = n.find('.', 7);
  if (dot == std::string::npos) return false;
  const int li = atoi(n.substr(7, dot - 7).c_str());
  if (li < 0 || li >= c.n_layer) return false;
  o->layer = li;
  const int kind = c.kind[li];
  const std::string rest = n.substr(dot + 1);
  if (is_delta(kind) && rest.rfind("attn.", 0) == 0 && rest != "attn.proj.weight") {
    std::string leaf = rest.substr(5);
    int which = 0;
    if (kind == 2) {
      const size_t d2 = leaf.find('.');
      if (d2 == std::string::npos) return false;
      const std::string sub = leaf.substr(0, d2);
      which = sub == "dsa" ? 0 : (sub == "kda" ? 1 : (sub == "gmla" ? 2 : -1));
      if (which < 0) return false;
      leaf = leaf.substr(d2 + 1);
    }
    const int mode = kind == 2 ? which : kind - 3;
    const long long lat = c.latent;
    o->sub = which;
    if (leaf == "wq.weight") { o->slot = 0; o->rows = qd; o->K = D; return true; }
    if (mode != 2 && leaf == "wk.weight") { o->slot = 0; o->base = qd; o->rows = kvd; o->K = D; return true; }
    if (mode != 2 && leaf == "wv.weight") { o->slot = 0; o->base = qd + kvd; o->rows = kvd; o->K = D; return true; }
    if (mode == 2 && leaf == "w_kv_down.weight") { o->slot = 0; o->base = qd; o->rows = lat; o->K = D; return true; }
    if (mode == 2 && leaf == "w_k_up.weight") { o->slot = 1; o->rows = kvd; o->K = lat; return true; }
    if (mode == 2 && leaf == "w_v_up.weight") { o->slot = 1; o->base = kvd; o->rows = kvd; o->K = lat; return true; }
    return false;
  }
  if (rest == "attn.wq.weight") { o->slot = 0; o->rows = qd; o->K = D; return true; }
  if (rest == "attn.wk.weight") { o->slot = 0; o->base = qd; o->rows = kvd; o->K = D; return true; }
  if (rest == "attn.wv.weight") { o->slot = 0; o->base = qd + kvd; o->rows = kvd; o->K = D; return true; }
  if (rest == "attn.proj.weight") { o->slot = 1; o->rows = D; o->K = qd; return true; }
  if (kind != 1) {
    if (rest == "ffn.w_gate.weight") { o->slot = 2; o->row_mul = 2; o->rows = c.mlp_hidden; o->K = D; return true; }
    if (rest == "ffn.w_up.weight") { o->slot = 2; o->row_mul = 2; o->row_off = 1; o->rows = c.mlp_hidden; o->K = D; return true; }
    if (rest == "ffn.w_down.weight") { o->slot = 3; o->rows = D; o->K = c.mlp_hidden; return true; }
    return false;
  }
  if (rest.rfind("ffn.parts.", 0) != 0) return false;
  const size_t d2 = rest.find('.', 10);
  if (d2 == std::string::npos) return false;
  const int p = atoi(rest.substr(10, d2 - 10).c_str());
  const std::string r2 = rest.substr(d2 + 1);
  if (p < 0 || p >= c.P || r2.rfind("experts.", 0) != 0) return false;
  const size_t d3 = r2.find('.', 8);
  if (d3 == std::string::npos) return false;
  const int ex = atoi(r2.substr(8, d3 - 8).c_str());
  if (ex < 0 || ex >= c.E) return false;
  const std::string r3 = r2.substr(d3 + 1);
  const long long ge = (long long)p * c.E + ex, eh = c.expert_hidden;
  if (r3 == "w_gate.weight") { o->slot = 4; o->base = ge * 2 * eh; o->row_mul = 2; o->rows = eh; o->K = D; return true; }
  if (r3 == "w_up.weight") { o->slot = 4; o->base = ge * 2 * eh; o->row_mul = 2; o->row_off = 1; o->rows = eh; o->K = D; return true; }
  if (r3 == "w_down.weight") { o->slot = 5; o->base = ge * D; o->rows = D; o->K = eh; return true; }
  return false;
}

// bytes of what stays dense in a quantised model: embedding, norms, router gates, sink tokens, head gates
uint64_t dense_keep_bytes(const vn_model* m) {
  const Config& c = m->cfg;
  const uint64_t D = c.dim;
  uint64_t keep = (uint64_t)c.vocab * D * m->esz + D * 4;
  for (auto& L : m->layers) {
    keep += 2ull * D * 4;
    if (!is_delta(L.kind)) keep += (uint64_t)c.n_sink * D * m->esz;
    for (auto& S : L.sub) {
      if (S.mode == 0) keep += (uint64_t)c.n_sink * D * m->esz;
      if (S.mode != 1) keep += (uint64_t)c.n_head * 4;
    }
    if (L.kind == 1) keep += (uint64_t)(c.P + c.P * c.E) * D * 4;
  }
  return keep;
}

// where the quantised bytes / scales of a located linear live
void* slot_q(vn_model* m, const LinearSlot& ls) {
  if (ls.layer < 0) return m->head_q;
  Layer& L = m->layers[ls.layer];
  return ls.sub >= 0 ? L.sub[ls.sub].q[ls.slot] : L.q[ls.slot];
}
float* slot_qs(vn_model* m, const LinearSlot& ls) {
  if (ls.layer < 0) return m->head_qs;
  Layer& L = m->layers[ls.layer];
  return ls.sub >= 0 ? L.sub[ls.sub].qs[ls.slot] : L.qs[ls.slot];
}

// buffers for linears that arrive quantised; the dense buffers of those linears are given back
int32_t alloc_quant(vn_model* m, int mode) {
  vn_ctx* ctx = m->ctx;
  const Config& c = m->cfg;
  const long long D = c.dim, qd = (long long)c.n_head * c.hd, kvd = (long long)c.n_kv * c.hd;
  auto A = [&](void** q, float** qs, long long rows, long long K) -> int32_t {
    TRY(dev_alloc(ctx, q, (size_t)rows * q_row_bytes(mode, K)));
    TRY(dev_alloc(ctx, (void**)qs, (size_t)rows * q_row_scales(mode, K) * 4));
    return VN_OK;
  };
  VN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  auto F = [](void** p) { if (*p) cudaFree(*p); *p = nullptr; };
  for (auto& L : m->layers) {
    if (!is_delta(L.kind)) TRY(A(&L.q[0], &L.qs[0], qd + 2 * kvd, D));
    for (auto& S : L.sub) {
      TRY(A(&S.q[0], &S.qs[0], S.mode == 2 ? qd + c.latent : qd + 2 * kvd, D));
      if (S.mode == 2) TRY(A(&S.q[1], &S.qs[1], 2 * kvd, c.latent));
      F(&S.wqkv); F(&S.w_up);
      S.w_down = nullptr;
    }
    TRY(A(&L.q[1], &L.qs[1], D, qd));
    F(&L.wqkv); F(&L.wproj);
    if (L.kind != 1) {
      TRY(A(&L.q[2], &L.qs[2], 2ll * c.mlp_hidden, D));
      TRY(A(&L.q[3], &L.qs[3], D, c.mlp_hidden));
      F(&L.w_gateup); F(&L.w_down);
    } else {
      const long long ne = (long long)c.P * c.E;
      TRY(A(&L.q[4], &L.qs[4], ne * 2 * c.expert_hidden, D));
      TRY(A(&L.q[5], &L.qs[5], ne * D, c.expert_hidden));
      F(&L.e_gateup); F(&L.e_down);
    }
  }
  TRY(A(&m->head_q, &m->head_qs, c.vocab, D));
  if (m->head != m->emb) F(&m->head);
  m->preq_mode = mode;
  return VN_OK;
}

// sink K / V = wk(global_tokens), wv(global_tokens): fixed per layer (tri_sparse_attn.py:223-242).  With quantised
// linears (mode != 0) the k / v rows of the quantised q|k|v matrix are dequantised inside the GEMM, which is what
// the reference's compressed model computes (its wk / wv are quantised linears by then).
int32_t compute_sinks(vn_model* m, int mode) {
  vn_ctx* ctx = m->ctx;
  const Config& c = m->cfg;
  const long long D = c.dim, qd = (long long)c.n_head * c.hd, kvd = (long long)c.n_kv * c.hd;
  for (auto& L : m->layers) {
    // a DSA module's sinks (delta_attention.py:451-459): the same product with the module's own wk / wv, dense only
    for (auto& S : L.sub) {
      if (S.mode != 0) continue;
      for (int which = 0; which < 2; ++which) {
        GemmArgs g;
        g.A = S.sink; g.lda = D; g.ldw = D;
        g.C = which ? S.sink_v : S.sink_k; g.ldc = kvd; g.M = c.n_sink; g.N = (int)kvd; g.K = (int)D; g.c_bf16 = c.bf16;
        if (mode) {
          const long long r0 = qd + which * kvd;
          g.W = (const unsigned char*)S.q[0] + (size_t)r0 * q_row_bytes(mode, D);
          g.w_scale = S.qs[0] + (size_t)r0 * q_row_scales(mode, D);
          g.wq = mode;
          if (!gemm_mma_q_supported(g)) return vn_fail(ctx, VN_ERR_UNSUPPORTED, "quantised GEMM shape K=%d unsupported", g.K);
          TRY(launch_gemm_mma_q(ctx, g));
          continue;
        }
        g.W = (char*)S.wqkv + (size_t)(qd + which * kvd) * D * m->esz;
        if (c.bf16) TRY((launch_gemm_simt<__nv_bfloat16, __nv_bfloat16>(ctx, g)));
        else TRY((launch_gemm_simt<float, float>(ctx, g)));
      }
    }
    if (is_delta(L.kind)) continue;
    for (int which = 0; which < 2; ++which) {
      GemmArgs g;
      g.A = L.sink; g.lda = D; g.ldw = D;
      g.C = which ? L.sink_v : L.sink_k; g.ldc = kvd; g.M = c.n_sink; g.N = (int)kvd; g.K = (int)D; g.c_bf16 = c.bf16;
      if (mode) {
        const long long r0 = qd + which * kvd;
        g.W = (const unsigned char*)L.q[0] + (size_t)r0 * q_row_bytes(mode, D);
        g.w_scale = L.qs[0] + (size_t)r0 * q_row_scales(mode, D);
        g.wq = mode;
        if (!gemm_mma_q_supported(g)) return vn_fail(ctx, VN_ERR_UNSUPPORTED, "quantised GEMM shape K=%d unsupported", g.K);
        TRY(launch_gemm_mma_q(ctx, g));
      } else {
        g.W = (char*)L.wqkv + (size_t)(qd + which * kvd) * D * m->esz;
        if (c.bf16) TRY((launch_gemm_simt<__nv_bfloat16, __nv_bfloat16>(ctx, g)));
        else TRY((launch_gemm_simt<float, float>(ctx, g)));
      }
    }
  }
  return VN_OK;
}

int scheme_mode(const char* scheme) {
  if (!scheme) return 0;
  const std::string s(scheme);
  return s == "int8" ? 1 : (s == "int4" ? 2 : (s == "int4g128" ? 3 : 0));
}

struct NameRoute { int layer; std::string rest; };

}  // namespace

extern "C" {

int32_t vn_model_create(vn_ctx* ctx, const char* config_json, vn_model** out) {
  VN_CHECK_CTX(ctx);
  VN_REQUIRE(ctx, config_json && out, "null argument");
  *out = nullptr;
  const std::string s(config_json);
  Config c;
  double v;
  auto need = [&](const char* key, int* dst) -> bool { if (!json_num(s, key, &v)) return false; *dst = (int)v; return true; };
  VN_REQUIRE(ctx, need("vocab_size", &c.vocab) && need("dim", &c.dim) && need("n_layer", &c.n_layer) &&
             need("n_head", &c.n_head), "config needs vocab_size, dim, n_layer, n_head");
  c.n_kv = c.n_head;
  need("n_kv_head", &c.n_kv);
  need("window_size", &c.window); need("num_global_tokens", &c.n_sink); need("use_alibi", &c.use_alibi);
  need("anchor_interval", &c.anchor); need("latent_dim", &c.latent);
  need("use_rope", &c.use_rope); need("max_seq_len", &c.max_seq_len);
  if (json_num(s, "rope_theta", &v)) c.rope_theta = v;
  need("num_dense_parts", &c.P); need("num_experts_per_part", &c.E); need("top_k", &c.top_k);
  need("expert_hidden", &c.expert_hidden); need("mlp_hidden_multiple", &c.mlp_mult);
  need("tie_weights", &c.tie); need("embedding_scale", &c.emb_scale);
  std::string dt;
  if (json_str(s, "dtype", &dt)) {
    VN_REQUIRE(ctx, dt == "f32" || dt == "bf16", "dtype must be \"f32\" or \"bf16\", got %s", dt.c_str());
    c.bf16 = dt == "bf16";
  }
  VN_REQUIRE(ctx, c.vocab > 0 && c.dim > 0 && c.n_layer > 0 && c.n_head > 0 && c.n_kv > 0, "non-positive size");
  VN_REQUIRE(ctx, c.dim % c.n_head == 0, "dim(%d) must be divisible by n_head(%d)", c.dim, c.n_head);
  VN_REQUIRE(ctx, c.n_head % c.n_kv == 0, "n_head(%d) must be divisible by n_kv_head(%d)", c.n_head, c.n_kv);
  c.hd = c.dim / c.n_head;
  VN_REQUIRE(ctx, c.hd % 8 == 0 && c.hd <= 64, "head_dim %d unsupported (multiple of 8, at most 64)", c.hd);
  VN_REQUIRE(ctx, c.window >= 1 && c.n_sink >= 1, "window_size and num_global_tokens must be positive");
  VN_REQUIRE(ctx, c.anchor >= 1, "anchor_interval must be >= 1, got %d", c.anchor);
  if (c.latent <= 0) c.latent = c.n_kv * c.hd;      // delta_attention.py:858
  std::vector<std::string> pat;
  if (json_str_list(s, "layer_pattern", &pat)) {
    VN_REQUIRE(ctx, (int)pat.size() == c.n_layer, "layer_pattern length (%zu) must equal n_layer (%d)", pat.size(), c.n_layer);
    for (auto& k : pat) {
      static const char* names[6] = {"trisparse", "mod", "vda", "dsa", "kda", "gmla"};
      int code = -1;
      for (int i = 0; i < 6; ++i) if (k == names[i]) code = i;
      VN_REQUIRE(ctx, code >= 0, "layer kind %s unknown (trisparse | mod | vda | dsa | kda | gmla)", k.c_str());
      c.kind.push_back(code);
    }
  } else {
    c.kind.assign(c.n_layer, 0);
  }
  if (c.expert_hidden <= 0) c.expert_hidden = std::max((int)(c.dim * 8.0 / 3.0 / 64.0) * 64, 64);  // mod.py:687-688
  c.mlp_hidden = (int)((long long)((c.mlp_mult * c.dim * 2.0 / 3.0 + 63) / 64)) * 64;              // vnnn.py:794
  VN_REQUIRE(ctx, c.top_k >= 1 && c.top_k <= c.E && c.top_k <= 8 && c.E <= 60 && c.P >= 1 &&
             c.P + c.P * c.E <= 64, "MoD shape unsupported (P=%d E=%d top_k=%d)", c.P, c.E, c.top_k);
  vn_model* m = new vn_model();
  m->ctx = ctx; m->cfg = c; m->esz = c.bf16 ? 2 : 4;
  { const char* e = getenv("VN_ATTN_SIMT"); m->force_simt_attn = e && e[0] == '1'; }
  { const char* e = getenv("VN_GEMM_TC"); m->use_tc = !(e && e[0] == '0'); }
  int32_t st = alloc_weights(m);
  if (st != VN_OK) { vn_model_destroy(m); return st; }
  *out = m;
  return VN_OK;
}

int32_t vn_model_destroy(vn_model* m) {
  if (!m) return VN_OK;
  cudaSetDevice(m->ctx->device);
  cudaStreamSynchronize(m->ctx->stream);
  auto F = [](void* p) { if (p) cudaFree(p); };
  F(m->emb); if (m->head != m->emb) F(m->head); F(m->norm_f); F(m->rope_cos); F(m->rope_sin); F(m->status);
  for (auto& L : m->layers) {
    F(L.norm1); F(L.norm2); F(L.wqkv); F(L.wproj); F(L.sink); F(L.sink_kv); F(L.sink_k); F(L.sink_v); F(L.w_gateup);
    F(L.w_down); F(L.router); F(L.e_gateup); F(L.e_down);
  }
  F(m->x); F(m->h); F(m->h32); F(m->qkv); F(m->attn); F(m->act); F(m->y); F(m->slot_expert); F(m->slot_w); F(m->part_w);
  F(m->expert_count); F(m->expert_off); F(m->expert_cur); F(m->sorted_row); F(m->slot_pos); F(m->depth_dev);
  F(m->anc_dev); F(m->rows_dev); F(m->stage); F(m->hs); F(m->partial); F(m->tc_error); F(m->stack_bar); F(m->row_seg); F(m->sub_seg); F(m->head_q); F(m->head_qs);
  for (auto& L : m->layers) for (int i = 0; i < 6; ++i) { F(L.q[i]); F(L.qs[i]); }
  for (auto& L : m->layers)
    for (auto& S : L.sub) { F(S.wqkv); F(S.w_up); F(S.sink); F(S.sink_k); F(S.sink_v); F(S.head_gate); F(S.head_w); F(S.w_abs); F(S.q[0]); F(S.q[1]); F(S.qs[0]); F(S.qs[1]); }
  for (auto& L : m->layers) F(L.w_vda);
  F(m->lat); F(m->mix);
  delete m;
  return VN_OK;
}

int32_t vn_model_load_tensor(vn_model* m, const char* name, const float* data, int32_t ndim, const int64_t* shape) {
  if (!m) return vn_fail(nullptr, VN_ERR_INVALID, "null model");
  vn_ctx* ctx = m->ctx;
  VN_CHECK_CTX(ctx);
  VN_REQUIRE(ctx, name && data && shape && ndim >= 1 && ndim <= 2, "bad tensor argument");
  VN_REQUIRE(ctx, m->qmode == 0, "the model is quantised: its dense weights are gone, create a new model to reload");
  const Config& c = m->cfg;
  const std::string n(name);
  if (m->preq_mode) {
    LinearSlot ls;
    VN_REQUIRE(ctx, !locate_linear(m, n, &ls), "%s: this model takes its linears quantised (vn_model_load_quant_tensor)", name);
  }
  const long long r = shape[0], cl = ndim == 2 ? shape[1] : 1;
  const long long D = c.dim;
  auto expect = [&](long long er, long long ec) -> bool { return r == er && cl == ec; };
#define SHAPE(er, ec) VN_REQUIRE(ctx, expect((er), (ec)), "%s: shape (%lld, %lld) expected (%lld, %lld)", name, r, cl, (long long)(er), (long long)(ec))
  if (n == "rope.cos" || n == "rope.sin") {
    // optional override of the RoPE table with one computed by the caller (rows x head_dim/2, float32)
    VN_REQUIRE(ctx, cl == c.hd / 2 && r >= 1, "%s: shape (%lld, %lld) expected (rows, %d)", name, r, cl, c.hd / 2);
    float** dst = n == "rope.cos" ? &m->rope_cos : &m->rope_sin;
    VN_REQUIRE(ctx, m->rope_rows == 0 || m->rope_rows == r || *dst == nullptr, "rope tables must have equal row counts");
    if (*dst) { VN_CUDA(ctx, cudaStreamSynchronize(ctx->stream)); VN_CUDA(ctx, cudaFree(*dst)); *dst = nullptr; }
    TRY(dev_alloc(ctx, (void**)dst, (size_t)r * cl * 4));
    VN_CUDA(ctx, cudaMemcpyAsync(*dst, data, (size_t)r * cl * 4, cudaMemcpyHostToDevice, ctx->stream));
    VN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    m->rope_rows = (int)r;
    return VN_OK;
  }
  else if (n == "tok_emb.weight") { SHAPE(c.vocab, D); TRY(upload(m, data, m->emb, r, cl, D)); }
  else if (n == "head.weight") { SHAPE(c.vocab, D); if (!c.tie) TRY(upload(m, data, m->head, r, cl, D)); }
  else if (n == "norm.weight") { SHAPE(D, 1); TRY(upload(m, data, m->norm_f, 1, D, D, 1, 0, true)); }
  else if (n.rfind("blocks.", 0) == 0) {
    const size_t dot = n.find('.', 7);
    VN_REQUIRE(ctx, dot != std::string::npos, "bad tensor name %s", name);
    const int li = atoi(n.substr(7, dot - 7).c_str());
    if (li < 0 || li >= c.n_layer) return vn_fail(ctx, VN_ERR_INDEX, "%s: layer %d out of range", name, li);
    Layer& L = m->layers[li];
    const std::string rest = n.substr(dot + 1);
    const long long qd = (long long)c.n_head * c.hd, kvd = (long long)c.n_kv * c.hd;
    if (rest == "norm1.weight") { SHAPE(D, 1); TRY(upload(m, data, L.norm1, 1, D, D, 1, 0, true)); }
    else if (rest == "norm2.weight") { SHAPE(D, 1); TRY(upload(m, data, L.norm2, 1, D, D, 1, 0, true)); }
    else if (rest == "attn.gate_logits" && (!is_delta(L.kind) || L.kind == 2)) { SHAPE(3, 1); memcpy(L.gate_logits, data, 12); }
    else if (is_delta(L.kind) && rest.rfind("attn.", 0) == 0 && rest != "attn.proj.weight") {
      // a module's tensor: blocks.i.attn.<leaf> (dsa / kda / gmla layer) or blocks.i.attn.<dsa|kda|gmla>.<leaf> (vda)
      std::string leaf = rest.substr(5);
      SubAttn* S = nullptr;
      if (L.kind == 2) {
        const size_t d2 = leaf.find('.');
        VN_REQUIRE(ctx, d2 != std::string::npos, "unexpected tensor %s", name);
        const std::string sub = leaf.substr(0, d2);
        const int which = sub == "dsa" ? 0 : (sub == "kda" ? 1 : (sub == "gmla" ? 2 : -1));
        VN_REQUIRE(ctx, which >= 0, "unexpected tensor %s", name);
        S = &L.sub[which];
        leaf = leaf.substr(d2 + 1);
      } else {
        S = &L.sub[0];
      }
      const long long lat = c.latent;
      if (leaf == "wq.weight") { SHAPE(qd, D); TRY(upload(m, data, S->wqkv, r, cl, D, 1, 0)); }
      else if (S->mode != 2 && leaf == "wk.weight") { SHAPE(kvd, D); TRY(upload(m, data, S->wqkv, r, cl, D, 1, qd)); }
      else if (S->mode != 2 && leaf == "wv.weight") { SHAPE(kvd, D); TRY(upload(m, data, S->wqkv, r, cl, D, 1, qd + kvd)); }
      else if (S->mode == 0 && leaf == "global_tokens.weight") { SHAPE(c.n_sink, D); TRY(upload(m, data, S->sink, r, cl, D)); }
      else if (S->mode == 2 && leaf == "w_kv_down.weight") { SHAPE(lat, D); TRY(upload(m, data, S->wqkv, r, cl, D, 1, qd)); }
      else if (S->mode == 2 && leaf == "w_k_up.weight") { SHAPE(kvd, lat); TRY(upload(m, data, S->w_up, r, cl, lat, 1, 0)); }
      else if (S->mode == 2 && leaf == "w_v_up.weight") { SHAPE(kvd, lat); TRY(upload(m, data, S->w_up, r, cl, lat, 1, kvd)); }
      else if (S->mode != 1 && leaf == "head_gate_logits") {
        SHAPE(c.n_head, 1);
        S->gate_host.resize(c.n_head);
        for (int i = 0; i < c.n_head; ++i) S->gate_host[i] = 0.5f * (1.0f + tanhf(0.5f * data[i]));   // Tensor.sigmoid, tensor.py:824
        VN_CUDA(ctx, cudaMemcpyAsync(S->head_gate, S->gate_host.data(), S->gate_host.size() * 4, cudaMemcpyHostToDevice, ctx->stream));
        VN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
      }
      else return vn_fail(ctx, VN_ERR_INVALID, "unexpected tensor %s", name);
    }
    else if (rest == "attn.wq.weight") { SHAPE(qd, D); TRY(upload(m, data, L.wqkv, r, cl, D, 1, 0)); }
    else if (rest == "attn.wk.weight") { SHAPE(kvd, D); TRY(upload(m, data, L.wqkv, r, cl, D, 1, qd)); }
    else if (rest == "attn.wv.weight") { SHAPE(kvd, D); TRY(upload(m, data, L.wqkv, r, cl, D, 1, qd + kvd)); }
    else if (rest == "attn.proj.weight") { SHAPE(D, qd); TRY(upload(m, data, L.wproj, r, cl, qd)); }
    else if (rest == "attn.global_tokens.weight") { SHAPE(c.n_sink, D); TRY(upload(m, data, L.sink, r, cl, D)); }
    else if (L.kind != 1 && rest == "ffn.w_gate.weight") { SHAPE(c.mlp_hidden, D); TRY(upload(m, data, L.w_gateup, r, cl, D, 2, 0)); }
    else if (L.kind != 1 && rest == "ffn.w_up.weight") { SHAPE(c.mlp_hidden, D); TRY(upload(m, data, L.w_gateup, r, cl, D, 2, 1)); }
    else if (L.kind != 1 && rest == "ffn.w_down.weight") { SHAPE(D, c.mlp_hidden); TRY(upload(m, data, L.w_down, r, cl, c.mlp_hidden)); }
    else if (L.kind == 1 && rest == "ffn.part_router.gate.weight") { SHAPE(c.P, D); TRY(upload(m, data, L.router, r, cl, D, 1, 0, true)); }
    else if (L.kind == 1 && rest.rfind("ffn.parts.", 0) == 0) {
      const size_t d2 = rest.find('.', 10);
      VN_REQUIRE(ctx, d2 != std::string::npos, "bad tensor name %s", name);
      const int p = atoi(rest.substr(10, d2 - 10).c_str());
      if (p < 0 || p >= c.P) return vn_fail(ctx, VN_ERR_INDEX, "%s: part %d out of range", name, p);
      const std::string r2 = rest.substr(d2 + 1);
      const long long eh = c.expert_hidden;
      if (r2 == "router.gate.weight") { SHAPE(c.E, D); TRY(upload(m, data, L.router, r, cl, D, 1, c.P + (long long)p * c.E, true)); }
      else if (r2.rfind("experts.", 0) == 0) {
        const size_t d3 = r2.find('.', 8);
        VN_REQUIRE(ctx, d3 != std::string::npos, "bad tensor name %s", name);
        const int ex = atoi(r2.substr(8, d3 - 8).c_str());
        if (ex < 0 || ex >= c.E) return vn_fail(ctx, VN_ERR_INDEX, "%s: expert %d out of range", name, ex);
        const std::string r3 = r2.substr(d3 + 1);
        const long long ge = (long long)p * c.E + ex;
        char* gu = (char*)L.e_gateup + (size_t)ge * 2 * eh * D * m->esz;
        char* dn = (char*)L.e_down + (size_t)ge * D * eh * m->esz;
        if (r3 == "w_gate.weight") { SHAPE(eh, D); TRY(upload(m, data, gu, r, cl, D, 2, 0)); }
        else if (r3 == "w_up.weight") { SHAPE(eh, D); TRY(upload(m, data, gu, r, cl, D, 2, 1)); }
        else if (r3 == "w_down.weight") { SHAPE(D, eh); TRY(upload(m, data, dn, r, cl, eh)); }
        else return vn_fail(ctx, VN_ERR_INVALID, "unexpected tensor %s", name);
      } else return vn_fail(ctx, VN_ERR_INVALID, "unexpected tensor %s", name);
    } else return vn_fail(ctx, VN_ERR_INVALID, "unexpected tensor %s", name);
  } else return vn_fail(ctx, VN_ERR_INVALID, "unexpected tensor %s", name);
#undef SHAPE
  m->loaded.insert(n);
  m->finalized = false;
  return VN_OK;
}

int32_t vn_model_finalize(vn_model* m) {
  if (!m) return vn_fail(nullptr, VN_ERR_INVALID, "null model");
  vn_ctx* ctx = m->ctx;
  VN_CHECK_CTX(ctx);
  if (m->qmode) return VN_OK;   // nothing left to derive once the weights are quantised
  const Config& c = m->cfg;
  // every tensor of the reference's state_dict must have arrived (head.weight may be omitted when tied)
  std::vector<std::string> want = {"tok_emb.weight", "norm.weight"};
  if (!c.tie || m->preq_mode) want.push_back("head.weight");   // a quantised head is its own copy (compress.py:817-822)
  for (int i = 0; i < c.n_layer; ++i) {
    const std::string p = "blocks." + std::to_string(i) + ".";
    for (const char* s : {"norm1.weight", "norm2.weight", "attn.proj.weight"}) want.push_back(p + s);
    if (!is_delta(c.kind[i])) {
      for (const char* s : {"attn.gate_logits", "attn.wq.weight", "attn.wk.weight", "attn.wv.weight",
                            "attn.global_tokens.weight"})
        want.push_back(p + s);
    } else {
      if (c.kind[i] == 2) want.push_back(p + "attn.gate_logits");
      static const char* sub_name[3] = {"dsa", "kda", "gmla"};
      for (const SubAttn& S : m->layers[i].sub) {
        const std::string q = p + "attn." + (c.kind[i] == 2 ? std::string(sub_name[S.mode]) + "." : std::string());
        want.push_back(q + "wq.weight");
        if (S.mode == 2) for (const char* s : {"w_kv_down.weight", "w_k_up.weight", "w_v_up.weight"}) want.push_back(q + s);
        else for (const char* s : {"wk.weight", "wv.weight"}) want.push_back(q + s);
        if (S.mode == 0) want.push_back(q + "global_tokens.weight");
        if (S.mode != 1) want.push_back(q + "head_gate_logits");
      }
    }
    if (c.kind[i] != 1) {
      for (const char* s : {"ffn.w_gate.weight", "ffn.w_up.weight", "ffn.w_down.weight"}) want.push_back(p + s);
    } else {
      want.push_back(p + "ffn.part_router.gate.weight");
      for (int q = 0; q < c.P; ++q) {
        const std::string pp = p + "ffn.parts." + std::to_string(q) + ".";
        want.push_back(pp + "router.gate.weight");
        for (int e = 0; e < c.E; ++e)
          for (const char* s : {"w_gate.weight", "w_up.weight", "w_down.weight"})
            want.push_back(pp + "experts." + std::to_string(e) + "." + s);
      }
    }
  }
  for (auto& w : want)
    if (!m->loaded.count(w)) return vn_fail(ctx, VN_ERR_INVALID, "missing tensor %s", w.c_str());
  // RoPE table, built on the host in float32 exactly as the reference does (tri_sparse_attn.py:169-180)
  if (c.use_rope && (!m->rope_cos || !m->rope_sin)) {
    if (m->rope_cos) { cudaFree(m->rope_cos); m->rope_cos = nullptr; }
    if (m->rope_sin) { cudaFree(m->rope_sin); m->rope_sin = nullptr; }
    const int half = c.hd / 2, rows = std::max(c.max_seq_len, 16) * 2;
    std::vector<float> cs((size_t)rows * half), sn((size_t)rows * half);
    for (int j = 0; j < half; ++j) {
      // float32 throughout, as NumPy evaluates 1.0 / (theta ** (2.0 * i / head_dim)) on a float32 arange
      const float ex = (2.0f * (float)j) / (float)c.hd;
      const float inv = 1.0f / powf((float)c.rope_theta, ex);
      for (int p = 0; p < rows; ++p) {
        const float ang = (float)p * inv;  // np.outer of two float32 arrays
        cs[(size_t)p * half + j] = cosf(ang);
        sn[(size_t)p * half + j] = sinf(ang);
      }
    }
    TRY(dev_alloc(ctx, (void**)&m->rope_cos, cs.size() * 4));
    TRY(dev_alloc(ctx, (void**)&m->rope_sin, sn.size() * 4));
    VN_CUDA(ctx, cudaMemcpyAsync(m->rope_cos, cs.data(), cs.size() * 4, cudaMemcpyHostToDevice, ctx->stream));
    VN_CUDA(ctx, cudaMemcpyAsync(m->rope_sin, sn.data(), sn.size() * 4, cudaMemcpyHostToDevice, ctx->stream));
    VN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    m->rope_rows = rows;
  }
  const long long D = c.dim, qd = (long long)c.n_head * c.hd, kvd = (long long)c.n_kv * c.hd;
  const int pm = m->preq_mode;
  TRY(compute_sinks(m, pm));
  // per-head weights of the tensor-core attention passes for the delta modules (window, sinks, dense up to 1024
  // keys; window, sinks beyond): DSA g*dense + (1-g)*(window + sinks), beyond 1024 keys window + sinks
  // (delta_attention.py:559-573); KDA one pass; GMLA gate * dense, beyond 1024 keys gate * window (:918-927)
  // GMLA: K | V projections folded through the latent (VN_GMLA_ABSORB=0, read here, keeps the two-step route)
  {
    const char* e = getenv("VN_GMLA_ABSORB");
    const bool absorb_on = !(e && e[0] == '0');
    const long long lat = c.latent;
    for (auto& L : m->layers)
      for (auto& S : L.sub) {
        if (S.mode != 2 || !c.bf16 || !absorb_on || pm) continue;
        if ((double)2 * kvd * D > 1.25 * (double)lat * (D + 2 * kvd)) continue;   // a narrow latent: two small GEMMs read less
        // (built again on every finalize: tensors may have been loaded anew since the last one)
        if (!S.w_abs) TRY(dev_alloc(ctx, &S.w_abs, (size_t)(qd + 2 * kvd) * D * m->esz));
        VN_CUDA(ctx, cudaMemcpyAsync(S.w_abs, S.wqkv, (size_t)qd * D * m->esz, cudaMemcpyDeviceToDevice, ctx->stream));
        GemmArgs g;       // C[2 kvd, D] = w_up[2 kvd, lat] x w_kv_down[lat, D]: the weight operand is read along its rows
        g.A = S.w_up; g.lda = lat; g.W = S.w_down; g.ldw = 1; g.ldw_k = D;
        g.C = (char*)S.w_abs + (size_t)qd * D * m->esz; g.ldc = D; g.M = (int)(2 * kvd); g.N = (int)D; g.K = (int)lat; g.c_bf16 = 1;
        TRY((launch_gemm_simt<__nv_bfloat16, __nv_bfloat16>(ctx, g)));
      }
  }
  // a vda layer's three projections as one matrix (VN_VDA_STACK=0 keeps three GEMMs)
  {
    const char* e = getenv("VN_VDA_STACK");
    const bool stack_on = !(e && e[0] == '0');
    const size_t one = (size_t)(qd + 2 * kvd) * D * m->esz;
    for (auto& L : m->layers) {
      if (L.kind != 2 || !c.bf16 || pm || !stack_on || !L.sub[2].w_abs) continue;
      if (!L.w_vda) TRY(dev_alloc(ctx, &L.w_vda, 3 * one));
      for (int si = 0; si < 3; ++si)
        VN_CUDA(ctx, cudaMemcpyAsync((char*)L.w_vda + si * one, si == 2 ? L.sub[2].w_abs : L.sub[si].wqkv, one,
                                     cudaMemcpyDeviceToDevice, ctx->stream));
    }
  }
  for (auto& L : m->layers)
    for (auto& S : L.sub) {
      const int H = c.n_head;
      std::vector<float> w((size_t)5 * H, 0.f);
      for (int h = 0; h < H; ++h) {
        const float g = S.mode == 1 ? 1.f : S.gate_host[h];
        if (S.mode == 0) { w[h] = 1.f - g; w[H + h] = 1.f - g; w[2 * H + h] = g; w[3 * H + h] = 1.f; w[4 * H + h] = 1.f; }
        else if (S.mode == 1) w[2 * H + h] = 1.f;
        else { w[2 * H + h] = g; w[3 * H + h] = g; }
      }
      VN_CUDA(ctx, cudaMemcpyAsync(S.head_w, w.data(), w.size() * 4, cudaMemcpyHostToDevice, ctx->stream));
      VN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    }
  VN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  if (pm) {
    // linears arrived quantised: the model is now what vn_model_quantize would have left behind
    uint64_t bytes = 0;
    auto add = [&](long long rows, long long K) { bytes += (uint64_t)rows * (q_row_bytes(pm, K) + q_row_scales(pm, K) * 4); };
    for (auto& L : m->layers) {
      if (!is_delta(L.kind)) add(qd + 2 * kvd, D);
      for (auto& S : L.sub) {
        add(S.mode == 2 ? qd + c.latent : qd + 2 * kvd, D);
        if (S.mode == 2) add(2 * kvd, c.latent);
      }
      add(D, qd);
      if (L.kind != 1) { add(2ll * c.mlp_hidden, D); add(D, c.mlp_hidden); }
      else { const long long ne = (long long)c.P * c.E; add(ne * 2 * c.expert_hidden, D); add(ne * D, c.expert_hidden); }
    }
    add(c.vocab, D);
    m->param_bytes = dense_keep_bytes(m) + bytes;
    m->qmode = pm;
    { const char* e = getenv("VN_GEMM_TCQ"); if (e && e[0] == '0') m->use_tc = false; }
  }
  m->finalized = true;
  return VN_OK;
}

// quantise one dense bf16 matrix [rows, K]; the dense buffer is released afterwards when `release` is set
static int32_t quantize_matrix(vn_model* m, void** dense, long long rows, int K, int mode, void** q, float** qs,
                               bool release, uint64_t* bytes) {
  vn_ctx* ctx = m->ctx;
  VN_REQUIRE(ctx, K % 64 == 0, "in_features %d not supported by the quantised kernels (multiple of 64 needed)", K);
  const size_t qbytes = (size_t)rows * (mode == 1 ? K : K / 2);
  const size_t nscale = (size_t)rows * (mode == 3 ? (K + 127) / 128 : 1);
  TRY(dev_alloc(ctx, q, qbytes));
  TRY(dev_alloc(ctx, (void**)qs, nscale * 4));
  const __nv_bfloat16* w = (const __nv_bfloat16*)*dense;
  if (mode == 1) VN_LAUNCH(ctx, mmaq_detail::quantize_rows_kernel<1>, (unsigned)rows, 256, 0, w, K, (unsigned char*)*q, *qs);
  else if (mode == 2) VN_LAUNCH(ctx, mmaq_detail::quantize_rows_kernel<2>, (unsigned)rows, 256, 0, w, K, (unsigned char*)*q, *qs);
  else {
    VN_REQUIRE(ctx, rows < (1ll << 31) && (K + 127) / 128 < 65536, "matrix too large");
    dim3 grid((unsigned)rows, (K + 127) / 128);
    VN_LAUNCH(ctx, mmaq_detail::quantize_g128_kernel<__nv_bfloat16>, grid, 128, 0, w, K, (unsigned char*)*q, *qs);
  }
  *bytes += qbytes + nscale * 4;
  if (release) {
    VN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    VN_CUDA(ctx, cudaFree(*dense));
    *dense = nullptr;
  }
  return VN_OK;
}

int32_t vn_model_quantize(vn_model* m, const char* scheme) {
  if (!m) return vn_fail(nullptr, VN_ERR_INVALID, "null model");
  vn_ctx* ctx = m->ctx;
  VN_CHECK_CTX(ctx);
  VN_REQUIRE(ctx, scheme, "scheme is null");
  const std::string s(scheme);
  const int mode = s == "int8" ? 1 : (s == "int4" ? 2 : (s == "int4g128" ? 3 : 0));
  VN_REQUIRE(ctx, mode != 0, "unknown quantisation scheme %s (int8 | int4 | int4g128)", scheme);
  VN_REQUIRE(ctx, m->finalized, "quantise after vn_model_finalize");
  VN_REQUIRE(ctx, m->qmode == 0, "model is already quantised");
  if (!m->cfg.bf16) return vn_fail(ctx, VN_ERR_UNSUPPORTED, "weight-only quantisation needs a bf16 model");
  const Config& c = m->cfg;
  const long long D = c.dim, qd = (long long)c.n_head * c.hd, kvd = (long long)c.n_kv * c.hd;
  uint64_t bytes = 0;
  // every Linear of the blocks and the LM head (verse_torch/compress.py:807-822 swaps every Linear and gives
  // the tied head its own quantised copy); the router gates and the embedding table stay dense
  for (auto& L : m->layers) {
    if (!is_delta(L.kind)) TRY(quantize_matrix(m, &L.wqkv, qd + 2 * kvd, (int)D, mode, &L.q[0], &L.qs[0], true, &bytes));
    for (auto& S : L.sub) {
      // a module's stacked projections as they are; a GMLA module goes back to its two projections (the folded
      // matrix is a product of the dense factors and is dropped)
      TRY(quantize_matrix(m, &S.wqkv, S.mode == 2 ? qd + c.latent : qd + 2 * kvd, (int)D, mode, &S.q[0], &S.qs[0], true, &bytes));
      if (S.mode == 2) TRY(quantize_matrix(m, &S.w_up, 2 * kvd, c.latent, mode, &S.q[1], &S.qs[1], true, &bytes));
      S.w_down = nullptr;
      if (S.w_abs) { VN_CUDA(ctx, cudaStreamSynchronize(ctx->stream)); VN_CUDA(ctx, cudaFree(S.w_abs)); S.w_abs = nullptr; }
    }
    if (L.w_vda) { VN_CUDA(ctx, cudaStreamSynchronize(ctx->stream)); VN_CUDA(ctx, cudaFree(L.w_vda)); L.w_vda = nullptr; }
    TRY(quantize_matrix(m, &L.wproj, D, (int)qd, mode, &L.q[1], &L.qs[1], true, &bytes));
    if (L.kind != 1) {
      TRY(quantize_matrix(m, &L.w_gateup, 2ll * c.mlp_hidden, (int)D, mode, &L.q[2], &L.qs[2], true, &bytes));
      TRY(quantize_matrix(m, &L.w_down, D, c.mlp_hidden, mode, &L.q[3], &L.qs[3], true, &bytes));
    } else {
      const long long ne = (long long)c.P * c.E;
      TRY(quantize_matrix(m, &L.e_gateup, ne * 2 * c.expert_hidden, (int)D, mode, &L.q[4], &L.qs[4], true, &bytes));
      TRY(quantize_matrix(m, &L.e_down, ne * D, c.expert_hidden, mode, &L.q[5], &L.qs[5], true, &bytes));
    }
  }
  void* head = m->head;
  TRY(quantize_matrix(m, &head, c.vocab, (int)D, mode, &m->head_q, &m->head_qs, false, &bytes));
  if (!c.tie && m->head) { VN_CUDA(ctx, cudaStreamSynchronize(ctx->stream)); VN_CUDA(ctx, cudaFree(m->head)); m->head = nullptr; }
  // the sink K / V are what the quantised wk / wv give from here on, as in the reference's compressed model
  TRY(compute_sinks(m, mode));
  VN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  m->qmode = mode;
  // VN_GEMM_TCQ=0 in the environment: keep the quantised mma.sync GEMMs instead of the tcgen05 ones
  { const char* e = getenv("VN_GEMM_TCQ"); if (e && e[0] == '0') m->use_tc = false; }
  // embedding + norms + routers + sinks stay as they were
  m->param_bytes = dense_keep_bytes(m) + bytes;
  return VN_OK;
}

int32_t vn_model_param_bytes(vn_model* m, uint64_t* out) {
  if (!m || !out) return vn_fail(nullptr, VN_ERR_INVALID, "null argument");
  *out = m->param_bytes;
  return VN_OK;
}

int32_t vn_quantize(vn_ctx* ctx, const float* w_dev, int64_t rows, int32_t K, const char* scheme, void* q_dev,
                    float* scale_dev) {
  VN_CHECK_CTX(ctx);
  const int mode = scheme_mode(scheme);
  VN_REQUIRE(ctx, mode != 0, "unknown quantisation scheme %s (int8 | int4 | int4g128)", scheme ? scheme : "(null)");
  VN_REQUIRE(ctx, w_dev && q_dev && scale_dev && rows >= 0 && K >= 1 && rows < (1ll << 31), "bad arguments");
  if (rows == 0) return VN_OK;
  if (mode == 1) {
    auto kfn = mmaq_detail::quantize_rows_kernel<1, float>;
    VN_LAUNCH_NAMED(ctx, "quantize_rows_kernel", kfn, (unsigned)rows, 256, 0, w_dev, K, (unsigned char*)q_dev, scale_dev);
  } else if (mode == 2) {
    auto kfn = mmaq_detail::quantize_rows_kernel<2, float>;
    VN_LAUNCH_NAMED(ctx, "quantize_rows_kernel", kfn, (unsigned)rows, 256, 0, w_dev, K, (unsigned char*)q_dev, scale_dev);
  } else {
    VN_REQUIRE(ctx, K % 2 == 0 && (K + 127) / 128 < 65536, "int4g128 needs an even in_features below 2^23");
    dim3 grid((unsigned)rows, (K + 127) / 128);
    auto kfn = mmaq_detail::quantize_g128_kernel<float>;
    VN_LAUNCH_NAMED(ctx, "quantize_g128_kernel", kfn, grid, 128, 0, w_dev, K, (unsigned char*)q_dev, scale_dev);
  }
  return VN_OK;
}

int32_t vn_model_load_quant_tensor(vn_model* m, const char* name, const char* scheme, const void* packed,
                                   const float* scale, int64_t rows, int64_t K) {
  if (!m) return vn_fail(nullptr, VN_ERR_INVALID, "null model");
  vn_ctx* ctx = m->ctx;
  VN_CHECK_CTX(ctx);
  VN_REQUIRE(ctx, name && packed && scale, "null argument");
  const int mode = scheme_mode(scheme);
  VN_REQUIRE(ctx, mode != 0, "unknown quantisation scheme %s (int8 | int4 | int4g128)", scheme ? scheme : "(null)");
  if (!m->cfg.bf16) return vn_fail(ctx, VN_ERR_UNSUPPORTED, "quantised linears need a bf16 model");
  VN_REQUIRE(ctx, m->qmode == 0, "the model is already quantised");
  VN_REQUIRE(ctx, m->preq_mode == 0 || m->preq_mode == mode, "%s: one scheme per model (linears so far arrived as scheme %d)", name, m->preq_mode);
  const std::string n(name);
  LinearSlot ls;
  VN_REQUIRE(ctx, locate_linear(m, n, &ls), "%s is not a linear of this model", name);
  VN_REQUIRE(ctx, rows == ls.rows && K == ls.K, "%s: shape (%lld, %lld) expected (%lld, %lld)", name, (long long)rows,
             (long long)K, ls.rows, ls.K);
  VN_REQUIRE(ctx, K % 64 == 0, "in_features %lld not supported by the quantised kernels (multiple of 64 needed)", (long long)K);
  if (!m->preq_mode) {
    for (const auto& w : m->loaded) {
      LinearSlot other;
      VN_REQUIRE(ctx, !locate_linear(m, w, &other), "%s was loaded dense: a model takes all its linears dense or all quantised", w.c_str());
    }
    TRY(alloc_quant(m, mode));
  }
  unsigned char* q = (unsigned char*)slot_q(m, ls);
  float* qs = slot_qs(m, ls);
  const size_t rb = q_row_bytes(mode, K), sb = q_row_scales(mode, K) * 4;
  VN_CUDA(ctx, cudaMemcpy2DAsync(q + (size_t)(ls.base + ls.row_off) * rb, (size_t)ls.row_mul * rb, packed, rb, rb, (size_t)rows,
                                 cudaMemcpyHostToDevice, ctx->stream));
  VN_CUDA(ctx, cudaMemcpy2DAsync((char*)qs + (size_t)(ls.base + ls.row_off) * sb, (size_t)ls.row_mul * sb, scale, sb, sb,
                                 (size_t)rows, cudaMemcpyHostToDevice, ctx->stream));
  VN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));     // the host buffers may be reused by the caller
  m->loaded.insert(n);
  m->finalized = false;
  return VN_OK;
}

int32_t vn_model_read_quant(vn_model* m, const char* name, void* q_host, size_t q_bytes, float* scale_host,
                            size_t n_scales) {
  if (!m) return vn_fail(nullptr, VN_ERR_INVALID, "null model");
  vn_ctx* ctx = m->ctx;
  VN_CHECK_CTX(ctx);
  VN_REQUIRE(ctx, name && q_host && scale_host, "null argument");
  const int mode = m->qmode ? m->qmode : m->preq_mode;
  VN_REQUIRE(ctx, mode != 0, "the model holds no quantised weights");
  LinearSlot ls;
  VN_REQUIRE(ctx, locate_linear(m, std::string(name), &ls), "%s is not a linear of this model", name);
  const size_t rb = q_row_bytes(mode, ls.K), sb = q_row_scales(mode, ls.K) * 4;
  VN_REQUIRE(ctx, q_bytes == (size_t)ls.rows * rb && n_scales * 4 == (size_t)ls.rows * sb,
             "%s: buffers of %zu bytes / %zu scales, expected %zu / %zu", name, q_bytes, n_scales,
             (size_t)ls.rows * rb, (size_t)ls.rows * sb / 4);
  const unsigned char* q = (const unsigned char*)slot_q(m, ls);
  const float* qs = slot_qs(m, ls);
  VN_REQUIRE(ctx, q && qs, "%s has no quantised copy", name);
  VN_CUDA(ctx, cudaMemcpy2DAsync(q_host, rb, q + (size_t)(ls.base + ls.row_off) * rb, (size_t)ls.row_mul * rb, rb,
                                 (size_t)ls.rows, cudaMemcpyDeviceToHost, ctx->stream));
  VN_CUDA(ctx, cudaMemcpy2DAsync(scale_host, sb, (const char*)qs + (size_t)(ls.base + ls.row_off) * sb, (size_t)ls.row_mul * sb,
                                 sb, (size_t)ls.rows, cudaMemcpyDeviceToHost, ctx->stream));
  VN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return VN_OK;
}

int32_t vn_model_head(vn_model* m, const float* hidden_dev, int32_t rows, int32_t v_lo, int32_t n_cols,
                      float* out_logits_dev, int64_t out_ld) {
  if (!m || !hidden_dev || !out_logits_dev) return vn_fail(nullptr, VN_ERR_INVALID, "null argument");
  vn_ctx* ctx = m->ctx;
  VN_CHECK_CTX(ctx);
  const Config& c = m->cfg;
  VN_REQUIRE(ctx, m->finalized, "model is not finalised");
  VN_REQUIRE(ctx, rows >= 0 && v_lo >= 0 && n_cols >= 0 && (long long)v_lo + n_cols <= c.vocab && out_ld >= n_cols,
             "column range [%d, %d) outside the vocabulary of %d", v_lo, v_lo + n_cols, c.vocab);
  if (rows == 0 || n_cols == 0) return VN_OK;
  const int D = c.dim;
  for (int r0 = 0; r0 < rows; r0 += 256) {          // blocks of at most 256 rows: the decode GEMM's limit
    const int nr = std::min(256, rows - r0);
    TRY(ensure_rows(m, nr));
    GemmArgs g;
    g.lda = D; g.ldw = D; g.C = out_logits_dev + (long long)r0 * out_ld; g.ldc = out_ld; g.M = nr; g.N = n_cols; g.K = D;
    g.tag = "gemm_head_shard";
    const long long n = (long long)nr * D;
    if (c.bf16) {
      VN_LAUNCH(ctx, cast_rows_kernel<__nv_bfloat16>, (unsigned)ceil_div(n, 256ll), 256, 0, hidden_dev + (long long)r0 * D,
                (__nv_bfloat16*)m->h, n);
      g.A = m->h;
      if (m->qmode) {     // the quantised head copy: rows v_lo .. of the bytes (or nibbles) and of the scales
        g.W = (const unsigned char*)m->head_q + (long long)v_lo * (m->qmode == 1 ? D : D / 2);
        g.w_scale = m->head_qs + (long long)v_lo * (m->qmode == 3 ? (D + 127) / 128 : 1);
        g.wq = m->qmode;
      } else {
        g.W = (const __nv_bfloat16*)m->head + (long long)v_lo * D;
      }
      GemmArgs probe = g;
      if (m->use_tc && (m->qmode ? gemm_tcq_supported(probe) : gemm_tc_supported(probe)) && out_ld % 4 == 0 && n_cols >= 1) {
        TRY(ensure_partial(m, 1024));
        TcPlan direct;
        direct.error_flag = m->tc_error;
        TRY(tc_launch(ctx, g, m->cap_rows, direct));
      } else {
        TRY(linear(m, g));
      }
    } else {
      g.A = hidden_dev + (long long)r0 * D;
      g.W = (const float*)m->head + (long long)v_lo * D;
      TRY(linear(m, g));
    }
  }
  return VN_OK;
}

int32_t vn_model_set_recurrent(vn_model* m, int32_t on) {
  if (!m) return vn_fail(nullptr, VN_ERR_INVALID, "null model");
  m->recurrent = on != 0;
  return VN_OK;
}

int32_t vn_model_set_fused_stack(vn_model* m, int32_t on) {
  if (!m) return vn_fail(nullptr, VN_ERR_INVALID, "null model");
  m->fused_stack = on != 0;
  return VN_OK;
}

int32_t vn_model_set_wait_limit(vn_model* m, uint64_t cycles) {
  if (!m) return vn_fail(nullptr, VN_ERR_INVALID, "null model");
  vn_ctx* ctx = m->ctx;
  VN_CHECK_CTX(ctx);
  const unsigned long long v = cycles ? (unsigned long long)cycles : tc_detail::WAIT_LIMIT_CYCLES;
  VN_CUDA(ctx, cudaMemcpyToSymbolAsync(tc_detail::g_wait_limit_cycles, &v, sizeof v, 0, cudaMemcpyHostToDevice, ctx->stream));
  VN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return VN_OK;
}

int32_t vn_model_probe_wait(vn_model* m, int64_t* waited_cycles) {
  if (!m) return vn_fail(nullptr, VN_ERR_INVALID, "null model");
  vn_ctx* ctx = m->ctx;
  VN_CHECK_CTX(ctx);
  TRY(ensure_partial(m, 1024));          // makes sure the error word exists
  long long* d_cycles = nullptr;
  TRY(dev_alloc(ctx, (void**)&d_cycles, 8));
  VN_LAUNCH(ctx, tc_detail::wait_probe_kernel, 1, 32, 0, m->tc_error, d_cycles);
  long long h = 0;
  VN_CUDA(ctx, cudaMemcpyAsync(&h, d_cycles, 8, cudaMemcpyDeviceToHost, ctx->stream));
  VN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  cudaFree(d_cycles);
  if (waited_cycles) *waited_cycles = h;
  return VN_OK;
}

int32_t vn_model_status(vn_model* m, int32_t* bad_token, int32_t* wait_timeout) {
  if (!m) return vn_fail(nullptr, VN_ERR_INVALID, "null argument");
  vn_ctx* ctx = m->ctx;
  VN_CHECK_CTX(ctx);
  int tok = 0, to = 0;
  VN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  if (m->status) {
    VN_CUDA(ctx, cudaMemcpyAsync(&tok, m->status, 4, cudaMemcpyDeviceToHost, ctx->stream));
    VN_CUDA(ctx, cudaMemsetAsync(m->status, 0, 4, ctx->stream));
  }
  if (m->tc_error) {
    VN_CUDA(ctx, cudaMemcpyAsync(&to, m->tc_error, 4, cudaMemcpyDeviceToHost, ctx->stream));
    VN_CUDA(ctx, cudaMemsetAsync(m->tc_error, 0, 4, ctx->stream));
    if (to && m->stack_bar) VN_CUDA(ctx, cudaMemsetAsync(m->stack_bar, 0, 8, ctx->stream));
  }
  VN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  if (bad_token) *bad_token = tok;
  if (wait_timeout) *wait_timeout = to;
  if (to) return vn_fail(ctx, VN_ERR_TIMEOUT, "a bounded wait inside a GEMM kernel ran out: results of the last forwards are undefined");
  if (tok) return vn_fail(ctx, VN_ERR_INDEX, "token id outside [0, %d) met by a forward (clamped on the device)", m->cfg.vocab);
  return VN_OK;
}

int32_t vn_kv_create(vn_model* m, int32_t max_batch, int32_t max_seq, vn_kv** out) {
  if (!m || !out) return vn_fail(nullptr, VN_ERR_INVALID, "null argument");
  vn_ctx* ctx = m->ctx;
  VN_CHECK_CTX(ctx);
  VN_REQUIRE(ctx, max_batch >= 1 && max_seq >= 1, "max_batch and max_seq must be positive");
  vn_kv* kv = new vn_kv();
  kv->m = m; kv->ctx = ctx; kv->max_batch = max_batch; kv->max_seq = max_seq;
  const size_t plane = (size_t)max_batch * max_seq * m->cfg.n_kv * m->cfg.hd * m->esz;
  std::vector<void*> planes;
  for (int i = 0; i < m->n_pairs; ++i) {
    void *k = nullptr, *v = nullptr;
    if (cudaMalloc(&k, plane) != cudaSuccess || cudaMalloc(&v, plane) != cudaSuccess) {
      if (k) cudaFree(k);
      vn_kv_destroy(kv);
      return vn_fail(ctx, VN_ERR_OOM, "KV cache allocation of %zu bytes per plane failed", plane);
    }
    kv->k.push_back(k); kv->v.push_back(v);
    planes.push_back(k); planes.push_back(v);
  }
  TRY(dev_alloc(ctx, (void**)&kv->planes_dev, planes.size() * sizeof(void*)));
  VN_CUDA(ctx, cudaMemcpyAsync(kv->planes_dev, planes.data(), planes.size() * sizeof(void*), cudaMemcpyHostToDevice,
                               ctx->stream));
  TRY(dev_alloc(ctx, (void**)&kv->lens, (size_t)max_batch * 4));
  VN_CUDA(ctx, cudaMemsetAsync(kv->lens, 0, (size_t)max_batch * 4, ctx->stream));
  VN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  kv->len_ub.assign(max_batch, 0);
  *out = kv;
  return VN_OK;
}

int32_t vn_kv_destroy(vn_kv* kv) {
  if (!kv) return VN_OK;
  if (kv->ctx) {
    cudaSetDevice(kv->ctx->device);
    cudaStreamSynchronize(kv->ctx->stream);
  }
  if (!kv->parent) {
    for (void* p : kv->k) cudaFree(p);
    for (void* p : kv->v) cudaFree(p);
    if (kv->lens) cudaFree(kv->lens);
  }
  if (kv->planes_dev) cudaFree(kv->planes_dev);
  delete kv;
  return VN_OK;
}

int32_t vn_kv_view(vn_kv* kv, int32_t first, int32_t count, vn_kv** out) {
  if (!kv || !out) return vn_fail(nullptr, VN_ERR_INVALID, "null argument");
  vn_model* m = kv->m;
  vn_ctx* ctx = m->ctx;
  VN_CHECK_CTX(ctx);
  if (first < 0 || count < 1 || first + count > kv->max_batch)
    return vn_fail(ctx, VN_ERR_INDEX, "sequences [%d, %d) outside the cache's %d", first, first + count, kv->max_batch);
  vn_kv* v = new vn_kv();
  v->m = m; v->ctx = ctx; v->max_batch = count; v->max_seq = kv->max_seq;
  v->parent = kv->parent ? kv->parent : kv;
  v->parent_first = kv->parent_first + first;
  const size_t seq_bytes = (size_t)kv->max_seq * m->cfg.n_kv * m->cfg.hd * m->esz;
  std::vector<void*> planes;
  for (int i = 0; i < m->n_pairs; ++i) {
    v->k.push_back((char*)kv->k[i] + (size_t)first * seq_bytes);
    v->v.push_back((char*)kv->v[i] + (size_t)first * seq_bytes);
    planes.push_back(v->k.back()); planes.push_back(v->v.back());
  }
  if (dev_alloc(ctx, (void**)&v->planes_dev, planes.size() * sizeof(void*)) != VN_OK) { delete v; return VN_ERR_OOM; }
  VN_CUDA(ctx, cudaMemcpyAsync(v->planes_dev, planes.data(), planes.size() * sizeof(void*), cudaMemcpyHostToDevice, ctx->stream));
  VN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  v->lens = kv->lens + first;
  *out = v;
  return VN_OK;
}

int32_t vn_kv_lengths(vn_kv* kv, int32_t* out_host) {
  if (!kv || !out_host) return vn_fail(nullptr, VN_ERR_INVALID, "null argument");
  vn_ctx* ctx = kv->m->ctx;
  VN_CHECK_CTX(ctx);
  VN_CUDA(ctx, cudaMemcpyAsync(out_host, kv->lens, (size_t)kv->max_batch * 4, cudaMemcpyDeviceToHost, ctx->stream));
  VN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  for (int b = 0; b < kv->max_batch; ++b) kv_ub(kv, b) = out_host[b];
  return VN_OK;
}

int32_t vn_kv_set_lengths(vn_kv* kv, const int32_t* lens_host) {
  if (!kv || !lens_host) return vn_fail(nullptr, VN_ERR_INVALID, "null argument");
  vn_ctx* ctx = kv->m->ctx;
  VN_CHECK_CTX(ctx);
  for (int b = 0; b < kv->max_batch; ++b)
    if (lens_host[b] < 0 || lens_host[b] > kv->max_seq)
      return vn_fail(ctx, VN_ERR_OVERFLOW, "length %d of sequence %d outside [0, %d]", lens_host[b], b, kv->max_seq);
  VN_CUDA(ctx, cudaMemcpyAsync(kv->lens, lens_host, (size_t)kv->max_batch * 4, cudaMemcpyHostToDevice, ctx->stream));
  VN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  for (int b = 0; b < kv->max_batch; ++b) kv_ub(kv, b) = lens_host[b];
  return VN_OK;
}

int32_t vn_kv_reset_seq(vn_kv* kv, int32_t seq) {
  if (!kv) return vn_fail(nullptr, VN_ERR_INVALID, "null argument");
  vn_ctx* ctx = kv->m->ctx;
  VN_CHECK_CTX(ctx);
  if (seq >= kv->max_batch) return vn_fail(ctx, VN_ERR_INDEX, "sequence %d out of range (%d)", seq, kv->max_batch);
  if (seq < 0) {
    VN_CUDA(ctx, cudaMemsetAsync(kv->lens, 0, (size_t)kv->max_batch * 4, ctx->stream));
    for (int b = 0; b < kv->max_batch; ++b) kv_ub(kv, b) = 0;
  } else {
    VN_CUDA(ctx, cudaMemsetAsync(kv->lens + seq, 0, 4, ctx->stream));
    kv_ub(kv, seq) = 0;
  }
  return VN_OK;
}

int32_t vn_kv_commit(vn_kv* kv, int32_t n_new, const int32_t* keep_idx_dev, int32_t stride, const int32_t* n_keep_dev,
                     int32_t keep_add) {
  if (!kv || !n_keep_dev) return vn_fail(nullptr, VN_ERR_INVALID, "null argument");
  vn_model* m = kv->m;
  vn_ctx* ctx = m->ctx;
  VN_CHECK_CTX(ctx);
  VN_REQUIRE(ctx, n_new >= 0 && n_new <= 4096, "n_new out of range");
  const int B = kv->max_batch;
  if (n_new == 0) return VN_OK;
  if (keep_idx_dev) {
    VN_REQUIRE(ctx, stride >= 1, "stride must be positive");
    const int row_elems = m->cfg.n_kv * m->cfg.hd;
    const size_t smem = (size_t)n_new * row_elems * m->esz;
    VN_REQUIRE(ctx, smem <= 200 * 1024, "tree of %d nodes too large to compact in shared memory", n_new);
    dim3 grid(B, 2 * m->n_pairs);
    if (m->cfg.bf16) {
      if (smem > 48 * 1024)
        VN_CUDA(ctx, cudaFuncSetAttribute(kv_commit_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      VN_LAUNCH(ctx, kv_commit_kernel<__nv_bfloat16>, grid, 256, smem, (__nv_bfloat16* const*)kv->planes_dev, kv->lens,
                keep_idx_dev, stride, n_keep_dev, keep_add, n_new, kv->max_seq, row_elems);
    } else {
      if (smem > 48 * 1024)
        VN_CUDA(ctx, cudaFuncSetAttribute(kv_commit_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      VN_LAUNCH(ctx, kv_commit_kernel<float>, grid, 256, smem, (float* const*)kv->planes_dev, kv->lens, keep_idx_dev, stride,
                n_keep_dev, keep_add, n_new, kv->max_seq, row_elems);
    }
  }
  VN_LAUNCH_PDL(ctx, kv_advance_kernel, ceil_div(B, 128), 128, 0, kv->lens, n_keep_dev, keep_add, n_new, kv->max_seq, B);
  for (int b = 0; b < B; ++b) kv_ub(kv, b) = std::min(kv_ub(kv, b) + n_new, kv->max_seq);
  return VN_OK;
}

int32_t vn_kv_read(vn_kv* kv, int32_t layer, int32_t seq, int32_t which, float* out_host, int32_t n_positions) {
  if (!kv || !out_host) return vn_fail(nullptr, VN_ERR_INVALID, "null argument");
  vn_model* m = kv->m;
  vn_ctx* ctx = m->ctx;
  VN_CHECK_CTX(ctx);
  if (layer < 0 || layer >= m->n_pairs) return vn_fail(ctx, VN_ERR_INDEX, "layer %d out of range (%d)", layer, m->n_pairs);
  if (seq < 0 || seq >= kv->max_batch) return vn_fail(ctx, VN_ERR_INDEX, "sequence %d out of range (%d)", seq, kv->max_batch);
  VN_REQUIRE(ctx, n_positions >= 0 && n_positions <= kv->max_seq, "n_positions out of range");
  const size_t row = (size_t)m->cfg.n_kv * m->cfg.hd, n = row * n_positions;
  const char* src = (const char*)(which ? kv->v[layer] : kv->k[layer]) + (size_t)seq * kv->max_seq * row * m->esz;
  if (!m->cfg.bf16) {
    VN_CUDA(ctx, cudaMemcpyAsync(out_host, src, n * 4, cudaMemcpyDeviceToHost, ctx->stream));
    VN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  } else {
    std::vector<uint16_t> tmp(n);
    VN_CUDA(ctx, cudaMemcpyAsync(tmp.data(), src, n * 2, cudaMemcpyDeviceToHost, ctx->stream));
    VN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    for (size_t i = 0; i < n; ++i) { uint32_t u = (uint32_t)tmp[i] << 16; memcpy(out_host + i, &u, 4); }
  }
  return VN_OK;
}

int32_t vn_model_forward(vn_model* m, vn_kv* kv, const int64_t* tokens_dev, int32_t B, int32_t T,
                         const int32_t* parents_host, float* out_hidden_dev, float* out_logits_dev, int32_t last_only,
                         int32_t slot_offset) {
  if (!m || !kv) return vn_fail(nullptr, VN_ERR_INVALID, "null argument");
  vn_ctx* ctx = m->ctx;
  VN_CHECK_CTX(ctx);
  VN_REQUIRE(ctx, m->finalized, "vn_model_finalize has not been called");
  VN_REQUIRE(ctx, kv->m == m, "KV cache belongs to another model");
  VN_REQUIRE(ctx, tokens_dev && B >= 1 && T >= 1, "bad arguments");
  VN_REQUIRE(ctx, B <= kv->max_batch, "batch %d exceeds the cache's max_batch %d", B, kv->max_batch);
  VN_REQUIRE(ctx, (long long)B * T < (1ll << 24), "too many rows");
  VN_REQUIRE(ctx, slot_offset >= 0, "slot_offset must be non-negative");
  // capacity: conservative host bound first, exact lengths only when that trips
  const int limit = m->cfg.use_rope ? std::min(kv->max_seq, m->rope_rows) : kv->max_seq;
  bool over = false;
  for (int b = 0; b < B; ++b) over |= kv_ub(kv, b) + slot_offset + T > limit;
  if (over) {
    std::vector<int32_t> lens(kv->max_batch);
    TRY(vn_kv_lengths(kv, lens.data()));
    for (int b = 0; b < B; ++b)
      if (lens[b] + slot_offset + T > limit)
        return vn_fail(ctx, VN_ERR_OVERFLOW, "KV cache overflow: sequence %d holds %d, +%d exceeds the capacity %d", b,
                       lens[b] + slot_offset, T, limit);
  }
  const bool tree = parents_host != nullptr;
  if (tree) {
    VN_REQUIRE(ctx, T <= 64, "a tree may have at most 64 nodes, got %d", T);
    std::vector<int> depth(T);
    std::vector<unsigned long long> anc(T);
    for (int i = 0; i < T; ++i) {
      const int p = parents_host[i];
      VN_REQUIRE(ctx, p >= -1 && p < i, "parents[%d] = %d is not an earlier node", i, p);
      depth[i] = p < 0 ? 0 : depth[p] + 1;
      anc[i] = (1ull << i) | (p < 0 ? 0ull : anc[p]);
    }
    if (!m->depth_dev) {
      TRY(dev_alloc(ctx, (void**)&m->depth_dev, 64 * 4));
      TRY(dev_alloc(ctx, (void**)&m->anc_dev, 64 * 8));
    }
    // the same tree as last time is already on the device: nothing to copy and nothing to wait for, so a forward
    // over a fixed tree shape can be captured into a CUDA graph once it has run eagerly
    // (a tree that is the first T nodes of the stored one has the same depths and masks: also nothing to copy, so a
    // caller that grows one tree level by level uploads it once)
    const std::vector<int> now(parents_host, parents_host + T);
    const bool is_prefix = now.size() <= m->tree_parents.size() &&
                           std::equal(now.begin(), now.end(), m->tree_parents.begin());
    if (!is_prefix) {
      VN_CUDA(ctx, cudaMemcpyAsync(m->depth_dev, depth.data(), T * 4, cudaMemcpyHostToDevice, ctx->stream));
      VN_CUDA(ctx, cudaMemcpyAsync(m->anc_dev, anc.data(), T * 8, cudaMemcpyHostToDevice, ctx->stream));
      VN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
      m->tree_parents = now;
    }
  }
  TRY(ensure_rows(m, B * T));
  if (m->cfg.bf16 && m->use_tc && (!m->has_delta || delta_tc_ok(m, T, tree)) && B * T <= 256 && m->cfg.dim % 8 == 0 && m->cfg.dim <= 2048 &&
      tc_detail::encode_fn() != nullptr)
    return forward_tc(m, kv, tokens_dev, B, T, tree, out_hidden_dev, out_logits_dev, last_only, slot_offset);
  if (m->cfg.bf16) return forward_t<__nv_bfloat16>(m, kv, tokens_dev, B, T, tree, out_hidden_dev, out_logits_dev, last_only, slot_offset);
  return forward_t<float>(m, kv, tokens_dev, B, T, tree, out_hidden_dev, out_logits_dev, last_only, slot_offset);
}

int32_t vn_draft_propose(vn_model* draft, vn_kv* kv, const int64_t* pair_dev, int32_t B, int32_t k, float temperature,
                         int32_t top_k, uint64_t seed, uint32_t offset, float* q_logits_dev, int64_t* step_tokens_dev,
                         void* q_lists_dev) {
  if (!draft || !kv) return vn_fail(nullptr, VN_ERR_INVALID, "null draft model or cache");
  vn_ctx* ctx = draft->ctx;
  VN_CHECK_CTX(ctx);
  if (!pair_dev || !q_logits_dev || !step_tokens_dev || B < 1 || k < 1)
    return vn_fail(ctx, VN_ERR_INVALID, "vn_draft_propose: null buffer, B < 1 or k < 1");
  const long long V = draft->cfg.vocab;
  const size_t row_bytes = vn_topk_row_bytes();
  for (int i = 0; i < k; ++i) {
    float* q_i = q_logits_dev + (long long)i * B * V;
    // step 0 consumes the last two committed tokens (the cache holds everything before them); step i the proposal i - 1
    if (i == 0) TRY(vn_model_forward(draft, kv, pair_dev, B, 2, nullptr, nullptr, q_i, 1, 0));
    else TRY(vn_model_forward(draft, kv, step_tokens_dev + (long long)(i - 1) * B, B, 1, nullptr, nullptr, q_i, 1, i + 1));
    void* lists_i = q_lists_dev ? (void*)((unsigned char*)q_lists_dev + (size_t)i * B * row_bytes) : nullptr;
    TRY(vn_sample_lists(ctx, q_i, V, B, (int32_t)V, temperature, top_k, nullptr, seed, offset, (uint32_t)i, 2u,
                        step_tokens_dev + (long long)i * B, lists_i));
  }
  return VN_OK;
}

int32_t vn_verify_accept(vn_model* m, vn_kv* kv, const int64_t* tokens_dev, int32_t B, int32_t T, int32_t k,
                         const void* q_lists_dev, int64_t ql_stride_b, int64_t ql_stride_i, const float* q_logits_dev,
                         int64_t q_stride_b, int64_t q_stride_i, const int64_t* draft_dev, const float* u_accept_dev,
                         const float* u_sample_dev, uint64_t seed, uint32_t offset, float temperature, int32_t top_k,
                         int32_t bonus, float* p_logits_scratch_dev, int32_t* out_len_dev, int64_t* out_tokens_dev) {
  if (!m || !kv) return vn_fail(nullptr, VN_ERR_INVALID, "null argument");
  vn_ctx* ctx = m->ctx;
  VN_CHECK_CTX(ctx);
  const Config& c = m->cfg;
  const int np = bonus ? k + 1 : k;
  VN_REQUIRE(ctx, k >= 0 && T == np && T >= 1, "T (%d) must be k + 1 with a bonus token, k without (k = %d)", T, k);
  VN_REQUIRE(ctx, out_tokens_dev && (k == 0 || draft_dev), "null argument");
  const int V = c.vocab;
  // VN_K1=0 in the environment (read on every call, so that a test can compare the two routes): logits through HBM
  const char* k1_env = getenv("VN_K1");
  const bool k1_on = !(k1_env && k1_env[0] == '0');
  const bool fused_head = k1_on && c.bf16 && m->use_tc && !m->qmode && (long long)B * T <= 256 && c.dim % 8 == 0 &&
                          c.dim <= 2048 && tc_detail::encode_fn() != nullptr && temperature > 0.f && top_k > 0 &&
                          top_k < V && top_k <= 128 && V >= 1024;
  if (!fused_head) {
    // logits through HBM: the forward with the head, then the acceptance kernels on the stored rows
    if (!p_logits_scratch_dev)
      return vn_fail(ctx, VN_ERR_UNSUPPORTED, "this model / rule needs the logits in memory: pass p_logits_scratch_dev [B, T, V]");
    VN_REQUIRE(ctx, q_lists_dev == nullptr || q_logits_dev != nullptr || temperature <= 0.f || k == 0,
               "this model / rule selects from the draft rows' logits: pass q_logits_dev as well");
    TRY(vn_model_forward(m, kv, tokens_dev, B, T, nullptr, nullptr, p_logits_scratch_dev, 0, 0));
    return vn_accept_impl(ctx, p_logits_scratch_dev, (long long)T * V, V, q_logits_dev, q_stride_b, q_stride_i, draft_dev,
                          u_accept_dev, u_sample_dev, seed, offset, temperature, top_k, bonus, B, k, V, out_len_dev,
                          out_tokens_dev, 1, 0, nullptr);
  }
  // the logits buffer is only written when a row's candidate list overflows (heavy ties), but it has to exist
  VN_REQUIRE(ctx, p_logits_scratch_dev, "p_logits_scratch_dev [B, T, V] is needed (used only when a candidate list overflows)");
  // final-norm hidden rows of the B * T new positions (bf16, in the model's activation buffer)
  TRY(vn_model_forward(m, kv, tokens_dev, B, T, nullptr, nullptr, nullptr, 0, 0));
  const int rows = B * T, D = c.dim;
  vn_k1 k1;
  TRY(vn_k1_layout(ctx, B, np, top_k, V, &k1));
  const float temp = fmaxf(temperature, 1e-8f);
  TcPlan plain;
  plain.error_flag = m->tc_error;
  GemmArgs g;
  g.A = m->h; g.lda = D; g.W = m->head; g.ldw = D; g.M = rows; g.K = D;
  // (1) logits of the first head columns -> a lower bound of every row's k-th largest logit
  g.C = k1.boot; g.ldc = k1.nb; g.N = k1.nb; g.tag = "gemm_head_bound";
  TRY(launch_gemm_tc(ctx, g, m->cap_rows, plain));
  TRY(vn_k1_bound(ctx, k1, top_k, temp));
  // (2) the whole head: logits at or above the bound go to the rows' candidate lists, nothing else leaves the SMs
  tc_detail::CandBuf cb;
  cb.tau = k1.tau; cb.count = k1.count; cb.count_stride = k1.count_stride; cb.val = k1.cand_val; cb.tok = k1.cand_tok; cb.cap = k1.cap;
  TcPlan filt;
  filt.error_flag = m->tc_error; filt.filter = &cb;
  g.C = nullptr; g.ldc = V; g.N = V; g.tag = "gemm_head_filter";
  TRY(launch_gemm_tc(ctx, g, m->cap_rows, filt));
  // (3) only when a candidate list overflowed: the head once more with its logits stored
  if (p_logits_scratch_dev) {
    TcPlan fb;
    fb.error_flag = m->tc_error; fb.run_if = k1.fallback; fb.force_persist = true;
    g.C = p_logits_scratch_dev; g.ldc = V; g.N = V; g.tag = "gemm_head_fallback";
    TRY(launch_gemm_tc(ctx, g, m->cap_rows, fb));
  }
  return vn_k1_accept(ctx, k1, p_logits_scratch_dev, (long long)T * V, V, q_lists_dev, ql_stride_b, ql_stride_i, q_logits_dev,
                      q_stride_b, q_stride_i, draft_dev, u_accept_dev, u_sample_dev, seed, offset, temperature, top_k, bonus,
                      B, k, V, out_len_dev, out_tokens_dev);
}

}  // extern "C"
