// Stand-alone QK logits and AV output over the quantized prefix (the two-kernel path
// of the reference's API).  Exact fp32 dequantization, fp32 accumulation, deterministic.
#include "mz_store.cuh"

namespace {
constexpr int MAX_GQA = 16;

// one CTA per (key group, kv head, batch): row parameters of the D rows go to shared
// memory once, then each thread owns (query head, token) pairs.
__global__ void __launch_bounds__(256) qk_logits_kernel(const mz_kv_store s, const void* __restrict__ query, long long qsb,
                                                        long long qsh, int gqa, float scaling, int QB, float eps,
                                                        const float* __restrict__ table, void* __restrict__ out, int out_dt) {
  extern __shared__ float sm[];
  const int D = s.head_dim, G = s.group, top = (1 << s.bits) - 1, tw = top + 1;
  const int g = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z, H = s.kv_heads * gqa;
  MzRowParams* rp = (MzRowParams*)sm;           // [D]
  float* q_s = (float*)(rp + D);                 // [gqa][D]
  const long long m0 = b * s.km_stride_b + kvh * s.km_stride_h + (long long)g * D;
  for (int d = threadIdx.x; d < D; d += blockDim.x)
    rp[d] = mz_row_params(mz_load_as_float(s.k_mn, m0 + d, s.meta_dtype), mz_load_as_float(s.k_scale, m0 + d, s.meta_dtype), top, eps);
  for (int i = threadIdx.x; i < gqa * D; i += blockDim.x)
    q_s[i] = mz_load_as_float(query, b * qsb + (long long)(kvh * gqa + i / D) * qsh + (i % D), s.kv_dtype);
  __syncthreads();
  const uint8_t* rows = s.packed_k + b * s.pk_stride_b + kvh * s.pk_stride_h + (long long)g * D * QB;
  const long long S = (long long)s.k_groups * G;
  for (int i = threadIdx.x; i < gqa * G; i += blockDim.x) {
    const int hh = i / G, t = i % G;
    float dot = 0.f;
    for (int d = 0; d < D; ++d) {
      const int code = mz_extract_code(rows + (long long)d * QB, t, s.bits, QB);
      dot = fmaf(q_s[hh * D + d], mz_dequant_exact(rp[d], code, table, tw), dot);
    }
    mz_store_from_float(out, ((long long)b * H + kvh * gqa + hh) * S + (long long)g * G + t, dot * scaling, out_dt);
  }
}

// one CTA per (kv head, batch): warps stride over tokens, lanes over channels.
__global__ void __launch_bounds__(256) av_output_kernel(const mz_kv_store s, const void* __restrict__ w, int w_dt, int n_tokens,
                                                        int gqa, int QB, int NG, float eps, const float* __restrict__ table,
                                                        void* __restrict__ out, int out_dt) {
  extern __shared__ float sm[];                 // [warps][gqa][D]
  const int D = s.head_dim, G = s.group, top = (1 << s.bits) - 1, tw = top + 1;
  const int kvh = blockIdx.x, b = blockIdx.y, H = s.kv_heads * gqa;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  float* mine = sm + (long long)warp * gqa * D;
  for (int i = lane; i < gqa * D; i += 32) mine[i] = 0.f;
  __syncwarp();
  const uint8_t* pv = s.packed_v + b * s.pv_stride_b + kvh * s.pv_stride_h;
  const long long vm0 = b * s.vm_stride_b + kvh * s.vm_stride_h;
  for (int t = warp; t < n_tokens; t += warps) {
    float wt[MAX_GQA];
#pragma unroll
    for (int hh = 0; hh < MAX_GQA; ++hh)
      wt[hh] = hh < gqa ? mz_load_as_float(w, ((long long)b * H + kvh * gqa + hh) * n_tokens + t, w_dt) : 0.f;
    for (int d = lane; d < D; d += 32) {
      const int grp = d / G, idx = d % G;
      const long long m = vm0 + (long long)t * NG + grp;
      const MzRowParams r = mz_row_params(mz_load_as_float(s.v_mn, m, s.meta_dtype), mz_load_as_float(s.v_scale, m, s.meta_dtype), top, eps);
      const float v = mz_dequant_exact(r, mz_extract_code(pv + ((long long)t * NG + grp) * QB, idx, s.bits, QB), table, tw);
#pragma unroll
      for (int hh = 0; hh < MAX_GQA; ++hh)
        if (hh < gqa) mine[hh * D + d] = fmaf(wt[hh], v, mine[hh * D + d]);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < gqa * D; i += blockDim.x) {
    float a = 0.f;
    for (int k = 0; k < warps; ++k) a += sm[(long long)k * gqa * D + i];
    mz_store_from_float(out, ((long long)b * H + kvh * gqa + i / D) * D + (i % D), a, out_dt);
  }
}
}  // namespace

extern "C" int mz_qk_logits(const mz_kv_store* s, const void* query, long long qsb, long long qsh, int q_heads, float scaling,
                            void* out, int out_dtype, void* stream) {
  MZ_RANGE("mz_qk_logits");
  int rc = mz_check_store_basic(s);
  if (rc) return rc;
  if ((rc = mz_check_store_quantized(s))) return rc;
  MZ_REQUIRE(query && out && mz_dtype_ok(out_dtype), "bad query/out");
  MZ_REQUIRE(q_heads > 0 && q_heads % s->kv_heads == 0, "q_heads %d not a multiple of kv_heads %d", q_heads, s->kv_heads);
  const int gqa = q_heads / s->kv_heads;
  if (s->k_groups == 0) return MZ_OK;
  const float* table;
  if ((rc = mz_get_expand_table(s->bits, s->alpha_key, &table))) return rc;
  const size_t smem = (size_t)s->head_dim * sizeof(MzRowParams) + (size_t)gqa * s->head_dim * sizeof(float);
  if (smem > 48 * 1024) MZ_CUDA(cudaFuncSetAttribute(qk_logits_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid((unsigned)s->k_groups, (unsigned)s->kv_heads, (unsigned)s->batch);
  qk_logits_kernel<<<grid, 256, smem, (cudaStream_t)stream>>>(*s, query, qsb, qsh, gqa, scaling, mz_row_bytes(s->group, s->bits), 1e-8f,
                                                             table, out, out_dtype);
  MZ_LAUNCH_CHECK("qk_logits");
  return MZ_OK;
}

extern "C" int mz_av_output(const mz_kv_store* s, const void* weights, int w_dtype, int n_tokens, int q_heads, void* out,
                            int out_dtype, void* stream) {
  MZ_RANGE("mz_av_output");
  int rc = mz_check_store_basic(s);
  if (rc) return rc;
  if ((rc = mz_check_store_quantized(s))) return rc;
  MZ_REQUIRE(weights && out && mz_dtype_ok(out_dtype) && mz_dtype_ok(w_dtype), "bad weights/out");
  MZ_REQUIRE(q_heads > 0 && q_heads % s->kv_heads == 0, "q_heads %d not a multiple of kv_heads %d", q_heads, s->kv_heads);
  MZ_REQUIRE(n_tokens >= 0 && n_tokens <= s->v_tokens, "n_tokens %d outside [0,%d]", n_tokens, s->v_tokens);
  const int gqa = q_heads / s->kv_heads;
  if (gqa > MAX_GQA) return mz_fail(MZ_ERR_UNSUPPORTED, "%d query heads per kv head > %d", gqa, MAX_GQA);
  const float* table;
  if ((rc = mz_get_expand_table(s->bits, s->alpha_value, &table))) return rc;
  const size_t smem = (size_t)8 * gqa * s->head_dim * sizeof(float);
  if (smem > 200 * 1024) return mz_fail(MZ_ERR_UNSUPPORTED, "head_dim*gqa too large");
  if (smem > 48 * 1024) MZ_CUDA(cudaFuncSetAttribute(av_output_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid((unsigned)s->kv_heads, (unsigned)s->batch);
  av_output_kernel<<<grid, 256, smem, (cudaStream_t)stream>>>(*s, weights, w_dtype, n_tokens, gqa, mz_row_bytes(s->group, s->bits),
                                                             (s->head_dim + s->group - 1) / s->group, 1e-8f, table, out, out_dtype);
  MZ_LAUNCH_CHECK("av_output");
  return MZ_OK;
}
