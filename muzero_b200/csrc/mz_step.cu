// mz_decode_step: the steady-state decode step of one layer as a single C call:
// append the new token to the residual window, move the oldest residual tokens into the
// quantized store when the window has outgrown `residual_length` by a whole flush unit, then
// run the fused decode attention over the updated cache.  It is the sequence the host otherwise
// drives from Python (append, flush check, flush, attention); the counters of args->store are
// advanced in place so that the host can mirror them.
#include "mz_decode.cuh"

namespace {
// counters of the store after the append and the flush the step would do; returns the tokens flushed
int advance(mz_kv_store* s, int residual_length, int flush_unit) {
  const int after = s->res_len + 1;
  const int excess = after - residual_length;
  const int n = excess > 0 ? (excess / flush_unit) * flush_unit : 0;
  s->res_len = after - n;
  s->res_start += n;
  s->k_groups += n / s->group;
  s->v_tokens += n;
  return n;
}
}  // namespace

extern "C" size_t mz_decode_step_workspace_bytes(const mz_decode_args* a, int residual_length, int flush_unit) {
  if (a == nullptr || a->store.group <= 0 || flush_unit <= 0 || flush_unit % a->store.group != 0) return 0;
  mz_decode_args post = *a;
  advance(&post.store, residual_length, flush_unit);
  return mz_decode_workspace_bytes(&post);
}

extern "C" int mz_decode_step(mz_decode_args* a, const void* k_new, const void* v_new, long long new_stride_b,
                              long long new_stride_h, int residual_length, int flush_unit, int group_capacity,
                              int window_capacity, float eps, void* stream) {
  MZ_RANGE("mz_decode_step");
  MZ_REQUIRE(a != nullptr, "args is NULL");
  mz_kv_store* s = &a->store;
  MZ_REQUIRE(s->group > 0 && residual_length >= 0, "bad group %d / residual_length %d", s->group, residual_length);
  MZ_REQUIRE(flush_unit > 0 && flush_unit % s->group == 0, "flush_unit %d is not a multiple of group %d", flush_unit, s->group);
  if (s->res_start + s->res_len + 1 > window_capacity)
    return mz_fail(MZ_ERR_WORKSPACE, "residual window ends at row %d of %d: move it to the front of its buffer first",
                   s->res_start + s->res_len, window_capacity);
  // everything is validated and planned on the store as it will be after the step, before anything is
  // launched; the caller's counters move only when all launches were accepted
  mz_decode_args post = *a;
  const int n = advance(&post.store, residual_length, flush_unit);
  MzDecodePlan plan;
  int rc = mz_decode_plan(&post, &plan);
  if (rc) return rc;
  if (a->workspace == nullptr || a->workspace_bytes < plan.ws_bytes)
    return mz_fail(MZ_ERR_WORKSPACE, "workspace of %zu bytes needed after the step, %zu given", plan.ws_bytes, a->workspace_bytes);
  MZ_REQUIRE((uintptr_t)a->workspace % 16 == 0, "workspace must be 16-byte aligned");
  MZ_REQUIRE(k_new != nullptr && v_new != nullptr, "new key/value is NULL");
  if (n > 0 && s->k_groups + n / s->group > group_capacity)
    return mz_fail(MZ_ERR_WORKSPACE, "store holds %d of %d key groups, the flush needs %d more", s->k_groups, group_capacity,
                   n / s->group);
  rc = mz_append_kv(s, k_new, v_new, new_stride_b, new_stride_h, stream);
  if (rc) return rc;
  if (n > 0) {
    mz_kv_store appended = *s;
    appended.res_len += 1;
    rc = mz_flush_kv(&appended, n, eps, stream);
    if (rc) return rc;
  }
  rc = mz_decode_run_plan(&post, &plan, (cudaStream_t)stream);
  if (rc) return rc;
  *s = post.store;
  return MZ_OK;
}
