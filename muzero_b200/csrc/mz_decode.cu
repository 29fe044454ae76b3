// Decode attention entry points: argument checks, split selection, workspace carving,
// kernel dispatch, and the deterministic log-sum-exp combine.
#include <cstdlib>
#include <cstring>
#include <atomic>
#include <mutex>

#include "mz_decode.cuh"

namespace {

// Strided views of partial triples: record (row, part) has its m / l at m[row*m_row + part*m_part] and its
// acc[D] at acc + row*a_row + part*a_part.
struct PartialView {
  const float* m; const float* l; const float* acc;
  long long m_row, m_part, a_row, a_part;
};

// out[row, :] = sum_p acc[p,row,:] * exp(m[p,row] - m*) (/ sum_p l[p,row] * exp(m[p,row] - m*) when normalising)
__global__ void lse_combine_kernel(const PartialView v, int n_parts, int D, const MzDecodeOut o) {
  const long long row = blockIdx.x;
  float mx = -INFINITY;
  for (int p = 0; p < n_parts; ++p) mx = fmaxf(mx, v.m[row * v.m_row + p * v.m_part]);
  float lsum = 0.f;
  for (int p = 0; p < n_parts; ++p) {
    const long long i = row * v.m_row + p * v.m_part;
    const float w = (v.m[i] > -INFINITY) ? __expf(v.m[i] - mx) : 0.f;
    lsum += v.l[i] * w;
  }
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float a = 0.f;
    for (int p = 0; p < n_parts; ++p) {
      const float mi = v.m[row * v.m_row + p * v.m_part];
      const float w = (mi > -INFINITY) ? __expf(mi - mx) : 0.f;
      a = fmaf(v.acc[row * v.a_row + p * v.a_part + d], w, a);
    }
    if (o.out) mz_store_from_float(o.out, row * D + d, a / fmaxf(lsum, 1e-20f), o.out_dt);
    else o.acc[row * o.acc_stride + d] = a;
  }
  if (!o.out && threadIdx.x == 0) { o.m[row * o.ml_stride] = mx; o.l[row * o.ml_stride] = lsum; }
}

// SM count of the current device (cached per device index: a process may drive unlike GPUs)
constexpr int kMaxDevices = 64;
std::mutex g_sm_mu;
int g_sm_count[kMaxDevices] = {};
int sm_count() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
  std::lock_guard<std::mutex> lk(g_sm_mu);
  if (g_sm_count[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    g_sm_count[dev] = n;
  }
  return g_sm_count[dev];
}

// Which decode kernel serves a call.  0 = automatic (tensor-core mma.sync kernel where it applies, else the SIMT
// tiled kernel, else the shape-generic kernel), 1 = generic, 2 = no tensor-core kernel, 3 = the same as 0,
// 4 = the tcgen05 kernel where it applies (an opt-in: correct, but slower than the mma.sync kernel so far).
// MZ_DECODE_KERNEL = generic | tiles | mma | umma sets the initial value (read once, at the first call);
// mz_debug_force_kernel changes it for later calls, so that tests can cross-check the kernels in one process.
std::atomic<int> g_kernel_override{-1};
int kernel_override() {
  int v = g_kernel_override.load(std::memory_order_relaxed);
  if (v < 0) {
    const char* e = std::getenv("MZ_DECODE_KERNEL");
    v = 0;
    if (e && std::strcmp(e, "generic") == 0) v = 1;
    if (e && std::strcmp(e, "tiles") == 0) v = 2;
    if (e && std::strcmp(e, "mma") == 0) v = 3;
    if (e && std::strcmp(e, "umma") == 0) v = 4;
    int expected = -1;
    g_kernel_override.compare_exchange_strong(expected, v);
    v = g_kernel_override.load(std::memory_order_relaxed);
  }
  return v;
}

using Plan = MzDecodePlan;

int make_plan(const mz_decode_args* a, Plan* plan, bool need_tables) {
  MZ_REQUIRE(a != nullptr, "args is NULL");
  const mz_kv_store* s = &a->store;
  int rc = mz_check_store_basic(s);
  if (rc) return rc;
  MZ_REQUIRE(a->q_heads > 0 && a->q_heads % s->kv_heads == 0, "q_heads %d is not a multiple of kv_heads %d", a->q_heads, s->kv_heads);
  const int v_lead = s->v_tokens - s->k_groups * s->group;
  MZ_REQUIRE(v_lead >= 0 && v_lead <= s->res_len, "value prefix (%d tokens) must cover the key prefix (%d tokens) and end inside the residual window (%d tokens)",
             s->v_tokens, s->k_groups * s->group, s->res_len);
  MZ_REQUIRE(s->k_groups > 0 || s->res_len > 0, "no tokens to attend to");
  if ((s->k_groups > 0 || v_lead > 0) && (rc = mz_check_store_quantized(s))) return rc;
  if (s->res_len > 0 && (rc = mz_check_store_residual(s))) return rc;
  MZ_REQUIRE(a->query != nullptr, "query is NULL");
  MZ_REQUIRE(a->mask == nullptr || mz_dtype_ok(a->mask_dtype), "bad mask dtype");
  MZ_REQUIRE(a->splits >= 0, "splits must be >= 0");
  MzDecodeParams& p = plan->p;
  p.s = *s;
  p.H = a->q_heads;
  p.gqa = a->q_heads / s->kv_heads;
  p.query = a->query; p.q_stride_b = a->q_stride_b; p.q_stride_h = a->q_stride_h;
  p.scaling = a->scaling;
  p.mask = a->mask; p.mask_dtype = a->mask_dtype; p.mask_stride_b = a->mask_stride_b;
  p.QB = mz_row_bytes(s->group, s->bits);
  p.NG = (s->head_dim + s->group - 1) / s->group;
  p.eps = 1e-8f;
  p.v_lead = v_lead;
  p.table_k = p.table_v = nullptr;
  p.lut = nullptr;
  p.hetero = 0;
  const int force = kernel_override();
  plan->tiles = force != 1 && mz_decode_tiles_supported(p);
  if (v_lead > 0 && !plan->tiles)
    return mz_fail(MZ_ERR_UNSUPPORTED, "a value prefix ahead of the key prefix is served by the tiled kernel only (head_dim 128, group 32/64/128)");
  if (plan->tiles) {
    p.tp2 = MzTilesPlan{};
    p.slots_a = 0;
    if (force == 4 && mz_decode_umma_supported(p)) rc = mz_plan_umma(p, a->splits, sm_count(), &plan->slots);
    else if (force != 2 && mz_decode_mma_supported(p)) rc = mz_plan_mma(p, a->splits, sm_count(), &plan->slots);
    else rc = mz_plan_tiles(p, a->splits, sm_count(), &plan->slots);
    if (rc) return rc;
    p.splits = 0;
  } else {
    const int units = mz_decode_units_generic(*s);
    int splits = a->splits;
    if (splits == 0) {
      // aim for about two waves of CTAs over the SMs, but at least 4 units per CTA
      const long long pairs = (long long)s->batch * s->kv_heads;
      splits = (int)((2LL * sm_count() * 4 + pairs - 1) / pairs);
      if (splits > units / 4) splits = units / 4;
      if (splits < 1) splits = 1;
    }
    if (splits > units) splits = units;
    p.splits = splits;
    plan->slots = (size_t)s->batch * a->q_heads * splits;
  }
  // the three arrays (m, l, acc) follow each other in the workspace; a record count that is a multiple of 4 keeps
  // the acc rows 16-byte aligned (the kernels store them as vectors)
  plan->slots = (plan->slots + 3) & ~(size_t)3;
  plan->ws_bytes = plan->slots * sizeof(float) * (2 + (size_t)s->head_dim);
  if (need_tables && !plan->tiles) {
    if ((rc = mz_get_expand_table(s->bits, s->alpha_key, &p.table_k))) return rc;
    if ((rc = mz_get_expand_table(s->bits, s->alpha_value, &p.table_v))) return rc;
  }
  return MZ_OK;
}

// launches the main kernel of an existing plan (the workspace is checked here)
int launch_partials(const mz_decode_args* a, Plan* plan, cudaStream_t st) {
  if (a->workspace == nullptr || a->workspace_bytes < plan->ws_bytes)
    return mz_fail(MZ_ERR_WORKSPACE, "workspace of %zu bytes needed, %zu given", plan->ws_bytes, a->workspace_bytes);
  MZ_REQUIRE((uintptr_t)a->workspace % 16 == 0, "workspace must be 16-byte aligned");
  MzDecodeParams& p = plan->p;
  p.part.m = (float*)a->workspace;
  p.part.l = p.part.m + plan->slots;
  p.part.acc = p.part.l + plan->slots;
  p.part.slots = (long long)plan->slots;
  if (!plan->tiles) return mz_launch_decode_generic(p, st);
  if (p.tp.kind == 2) return mz_launch_decode_umma(p, st);
  return p.tp.kind == 1 ? mz_launch_decode_mma(p, st) : mz_launch_decode_tiles(p, st);
}

int run_partials(const mz_decode_args* a, Plan* plan, cudaStream_t st) {
  int rc = make_plan(a, plan, true);
  if (rc) return rc;
  return launch_partials(a, plan, st);
}

int finish(const Plan& plan, const MzDecodeOut& o, cudaStream_t st) {
  const MzDecodeParams& p = plan.p;
  if (plan.tiles) return mz_combine_tiles(p, o, st);
  const int D = p.s.head_dim;
  const int threads = D >= 128 ? 128 : ((D + 31) / 32) * 32;
  const PartialView v = {p.part.m, p.part.l, p.part.acc, p.splits, 1, (long long)p.splits * D, D};
  lse_combine_kernel<<<(unsigned)(p.s.batch * p.H), threads, 0, st>>>(v, p.splits, D, o);
  MZ_LAUNCH_CHECK("lse_combine");
  return MZ_OK;
}
}  // namespace

// Internal (used by the static-scratch entry point): scratch bytes a call needs and whether it
// would use the lazily allocated lookup tables.  Returns the validation status.
int mz_decode_plan_info(const mz_decode_args* args, size_t* ws_bytes, int* needs_tables) {
  Plan plan;
  int rc = make_plan(args, &plan, false);
  if (rc) return rc;
  *ws_bytes = plan.ws_bytes;
  *needs_tables = plan.tiles ? 0 : 1;
  return MZ_OK;
}

// Internal (used by mz_decode_step): validation and planning of a normalising call, then its launches.
int mz_decode_plan(const mz_decode_args* a, MzDecodePlan* plan) {
  MZ_REQUIRE(a != nullptr && a->out != nullptr && mz_dtype_ok(a->out_dtype), "bad output");
  return make_plan(a, plan, true);
}
int mz_decode_run_plan(const mz_decode_args* a, MzDecodePlan* plan, cudaStream_t st) {
  int rc = launch_partials(a, plan, st);
  if (rc) return rc;
  const MzDecodeOut o = {a->out, a->out_dtype, nullptr, nullptr, nullptr, 0, 0};
  return finish(*plan, o, st);
}

extern "C" int mz_debug_force_kernel(int which) {
  const int before = kernel_override();
  if (which >= 0 && which <= 4) g_kernel_override.store(which, std::memory_order_relaxed);
  return before;
}

extern "C" size_t mz_decode_workspace_bound(const mz_decode_args* a) {
  if (a == nullptr || mz_check_store_basic(&a->store) != MZ_OK) return 0;
  const mz_kv_store& s = a->store;
  if (a->q_heads <= 0 || a->q_heads % s.kv_heads != 0 || a->splits < 0) {
    mz_fail(MZ_ERR_ARG, "q_heads %d / splits %d", a->q_heads, a->splits);
    return 0;
  }
  const long long pairs = (long long)s.batch * s.kv_heads, gqa = a->q_heads / s.kv_heads;
  const long long sms = sm_count();
  // tiled kernels: slots = W * max_segs * gqa <= gqa * (pairs + 3 W) per plan; at most two plans (packed and
  // residual tiles) with W <= 3 + 12 workers per SM (or pairs * splits + pairs)
  const long long w_max = a->splits > 0 ? pairs * (a->splits + 1) : sms * 15;
  const long long tiled = gqa * (2 * pairs + 3 * w_max);
  // generic kernel: one slot per (batch, head, split)
  const long long splits = a->splits > 0 ? a->splits : (2 * sms * 4 + pairs - 1) / pairs;
  const long long generic = (long long)s.batch * a->q_heads * (splits < 1 ? 1 : splits);
  return (size_t)((tiled > generic ? tiled : generic) + 3) * sizeof(float) * (2 + (size_t)s.head_dim);
}

extern "C" size_t mz_decode_workspace_bytes(const mz_decode_args* args) {
  Plan plan;
  if (make_plan(args, &plan, false) != MZ_OK) return 0;
  return plan.ws_bytes;
}

extern "C" int mz_decode_attention(const mz_decode_args* a, void* stream) {
  MZ_RANGE("mz_decode_attention");
  Plan plan;
  cudaStream_t st = (cudaStream_t)stream;
  MZ_REQUIRE(a != nullptr && a->out != nullptr && mz_dtype_ok(a->out_dtype), "bad output");
  int rc = run_partials(a, &plan, st);
  if (rc) return rc;
  const MzDecodeOut o = {a->out, a->out_dtype, nullptr, nullptr, nullptr, 0, 0};
  return finish(plan, o, st);
}

extern "C" int mz_decode_attention_partial(const mz_decode_args* a, float* m, float* l, float* acc, void* stream) {
  MZ_RANGE("mz_decode_attention_partial");
  Plan plan;
  cudaStream_t st = (cudaStream_t)stream;
  MZ_REQUIRE(m && l && acc, "NULL partial output");
  int rc = run_partials(a, &plan, st);
  if (rc) return rc;
  const MzDecodeOut o = {nullptr, MZ_F32, m, l, acc, a->store.head_dim, 1};
  return finish(plan, o, st);
}

extern "C" int mz_decode_attention_partial_packed(const mz_decode_args* a, float* records, void* stream) {
  MZ_RANGE("mz_decode_attention_partial_packed");
  Plan plan;
  cudaStream_t st = (cudaStream_t)stream;
  MZ_REQUIRE(records != nullptr, "NULL partial output");
  int rc = run_partials(a, &plan, st);
  if (rc) return rc;
  const int D = a->store.head_dim;
  const MzDecodeOut o = {nullptr, MZ_F32, records + D, records + D + 1, records, D + 2, D + 2};
  return finish(plan, o, st);
}

namespace {
int merge_launch(const PartialView& v, int n_parts, long long rows, int head_dim, void* out, int out_dtype, void* stream) {
  MZ_REQUIRE(v.m && v.l && v.acc && out, "NULL pointer");
  MZ_REQUIRE(n_parts > 0 && rows > 0 && head_dim > 0, "bad shape");
  MZ_REQUIRE(mz_dtype_ok(out_dtype), "bad out_dtype");
  MZ_REQUIRE(rows < (1LL << 31), "too many rows");
  const int threads = head_dim >= 128 ? 128 : ((head_dim + 31) / 32) * 32;
  const MzDecodeOut o = {out, out_dtype, nullptr, nullptr, nullptr, 0, 0};
  lse_combine_kernel<<<(unsigned)rows, threads, 0, (cudaStream_t)stream>>>(v, n_parts, head_dim, o);
  MZ_LAUNCH_CHECK("lse_merge");
  return MZ_OK;
}
}  // namespace

extern "C" int mz_lse_merge(const float* m, const float* l, const float* acc, int n_parts, long long rows, int head_dim, void* out,
                            int out_dtype, void* stream) {
  MZ_RANGE("mz_lse_merge");
  const PartialView v = {m, l, acc, 1, rows, head_dim, rows * head_dim};
  return merge_launch(v, n_parts, rows, head_dim, out, out_dtype, stream);
}

extern "C" int mz_lse_merge_packed(const float* records, int n_parts, long long rows, int head_dim, void* out, int out_dtype,
                                   void* stream) {
  MZ_RANGE("mz_lse_merge_packed");
  MZ_REQUIRE(records != nullptr, "NULL pointer");
  const long long rec = head_dim + 2;
  const PartialView v = {records + head_dim, records + head_dim + 1, records, rec, rows * rec, rec, rows * rec};
  return merge_launch(v, n_parts, rows, head_dim, out, out_dtype, stream);
}
