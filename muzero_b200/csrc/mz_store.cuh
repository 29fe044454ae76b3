// Validation and addressing helpers for mz_kv_store (host + device).
#pragma once
#include "mz_common.cuh"

struct MzStoreGeom {
  int B, KVH, D, G, bits, NG, QB, top;
  int meta_dt, kv_dt;
};

static inline MzStoreGeom mz_geom(const mz_kv_store& s) {
  MzStoreGeom g;
  g.B = s.batch; g.KVH = s.kv_heads; g.D = s.head_dim; g.G = s.group; g.bits = s.bits;
  g.NG = (s.head_dim + s.group - 1) / s.group;
  g.QB = mz_row_bytes(s.group, s.bits);
  g.top = (1 << s.bits) - 1;
  g.meta_dt = s.meta_dtype; g.kv_dt = s.kv_dtype;
  return g;
}

// Checks everything that does not depend on which tensors a call touches.
static inline int mz_check_store_basic(const mz_kv_store* s) {
  MZ_REQUIRE(s != nullptr, "store is NULL");
  MZ_REQUIRE(s->batch > 0 && s->kv_heads > 0 && s->head_dim > 0, "bad store shape B=%d KVH=%d D=%d", s->batch, s->kv_heads,
             s->head_dim);
  MZ_REQUIRE(s->group > 0 && s->group <= 1024, "group must be 1..1024, got %d", s->group);
  MZ_REQUIRE(s->bits >= 1 && s->bits <= 8, "bits must be 1..8, got %d", s->bits);
  MZ_REQUIRE(mz_dtype_ok(s->meta_dtype), "bad meta_dtype %d", s->meta_dtype);
  MZ_REQUIRE(s->kv_dtype == MZ_BF16 || s->kv_dtype == MZ_F16, "kv_dtype must be bf16 or fp16");
  MZ_REQUIRE(s->alpha_key > 0.f && s->alpha_value > 0.f, "alpha must be > 0");
  MZ_REQUIRE(s->k_groups >= 0 && s->v_tokens >= 0 && s->res_start >= 0 && s->res_len >= 0, "negative length in store");
  return MZ_OK;
}

static inline int mz_check_store_quantized(const mz_kv_store* s) {
  MZ_REQUIRE(s->packed_k && s->k_mn && s->k_scale && s->packed_v && s->v_mn && s->v_scale, "store tensor pointer is NULL");
  return MZ_OK;
}

static inline int mz_check_store_residual(const mz_kv_store* s) {
  MZ_REQUIRE(s->res_k && s->res_v, "residual pointer is NULL");
  MZ_REQUIRE(s->res_stride_t >= s->head_dim, "res_stride_t %lld < head_dim", s->res_stride_t);
  return MZ_OK;
}
