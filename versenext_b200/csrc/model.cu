// placeholder until the model forward lands
#include "common.cuh"
extern "C" {
#define STUB(ctxexpr) return vn_fail(ctxexpr, VN_ERR_UNSUPPORTED, "model path not built yet")
int32_t vn_model_create(vn_ctx* ctx, const char*, vn_model**) { STUB(ctx); }
int32_t vn_model_destroy(vn_model*) { return VN_OK; }
int32_t vn_model_load_tensor(vn_model*, const char*, const float*, int32_t, const int64_t*) { STUB(nullptr); }
int32_t vn_model_finalize(vn_model*) { STUB(nullptr); }
int32_t vn_model_quantize(vn_model*, const char*) { STUB(nullptr); }
int32_t vn_model_param_bytes(vn_model*, uint64_t*) { STUB(nullptr); }
int32_t vn_kv_create(vn_model*, int32_t, int32_t, vn_kv**) { STUB(nullptr); }
int32_t vn_kv_destroy(vn_kv*) { return VN_OK; }
int32_t vn_kv_reset_seq(vn_kv*, int32_t) { STUB(nullptr); }
int32_t vn_kv_lengths(vn_kv*, int32_t*) { STUB(nullptr); }
int32_t vn_kv_set_lengths(vn_kv*, const int32_t*) { STUB(nullptr); }
int32_t vn_kv_commit(vn_kv*, int32_t, const int32_t*, int32_t, const int32_t*) { STUB(nullptr); }
int32_t vn_kv_read(vn_kv*, int32_t, int32_t, int32_t, float*, int32_t) { STUB(nullptr); }
int32_t vn_model_forward(vn_model*, vn_kv*, const int64_t*, int32_t, int32_t, const int32_t*, float*, float*, int32_t) { STUB(nullptr); }
}
