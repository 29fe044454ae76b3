// Residual-window flush, single-token append, and store -> dense dequantization.
//
// Flush is one launch: the first n_k CTAs each take one key tile
// [G tokens x D channels] of one (b, kvh): the tile is staged in shared memory
// with 16-byte row loads, then one thread per channel reduces min/max down its
// column, quantizes it and writes the packed row straight into the store (the
// transpose never touches global memory).  The remaining CTAs quantize value
// rows (G contiguous channels of one token) with G/8 lanes per row.
#include "mz_quant_math.cuh"
#include "mz_store.cuh"

namespace {

struct FlushParams {
  mz_kv_store s;
  int n_tiles;               // key tiles (groups of G tokens) to flush, from the window's first token
  int v_first, n_vtokens;    // value tokens to flush: window rows [v_first, v_first + n_vtokens)
  int QB, NG;
  float eps;
  const uint16_t* ctab_k; int ctab_k_n;
  const uint16_t* ctab_v; int ctab_v_n;
  unsigned n_k_blocks;
  long long v_rows;          // B*KVH*n_vtokens*NG
  int v_fast;                // G/8 lanes per value row, D % 8 == 0
  int k_vec;                 // key tile rows can be loaded as 16-byte vectors
};

template <int DT>
__device__ void flush_key_tile(const FlushParams& p, uint16_t* tile) {
  const mz_kv_store& s = p.s;
  const int G = s.group, D = s.head_dim;
  unsigned blk = blockIdx.x;
  const int j = blk % p.n_tiles; blk /= p.n_tiles;
  const int h = blk % s.kv_heads;
  const int b = blk / s.kv_heads;
  const uint16_t* src = (const uint16_t*)s.res_k + b * s.res_stride_b + h * s.res_stride_h +
                        (long long)(s.res_start + j * G) * s.res_stride_t;
  if (p.k_vec) {
    const int vec_per_row = D >> 3;
    for (int i = threadIdx.x; i < G * vec_per_row; i += blockDim.x) {
      const int t = i / vec_per_row, c = i % vec_per_row;
      ((uint4*)tile)[i] = *(const uint4*)(src + (long long)t * s.res_stride_t + c * 8);
    }
  } else {
    for (int i = threadIdx.x; i < G * D; i += blockDim.x) tile[i] = src[(long long)(i / D) * s.res_stride_t + (i % D)];
  }
  __syncthreads();
  const int grp = s.k_groups + j;
  uint8_t* dst_rows = s.packed_k + b * s.pk_stride_b + h * s.pk_stride_h + (long long)grp * D * p.QB;
  const long long meta0 = b * s.km_stride_b + h * s.km_stride_h + (long long)grp * D;
  // checked build: the last byte of this group's rows and its last metadata element lie inside the pair's slab
  if (!MZ_IN_BOUNDS((long long)(grp + 1) * D * p.QB - 1, s.pk_stride_h, 1) ||
      !MZ_IN_BOUNDS((long long)(grp + 1) * D - 1, s.km_stride_h, 2)) return;
  // A channel's G tokens are split over `parts` threads when the CTA has more threads than channels (2 for
  // head_dim 128 and 256 threads): partial min/max meet in shared memory, then each thread quantizes and packs
  // its own share of the row (whole octets, so the byte ranges of the parts do not overlap).
  const int parts = (blockDim.x >= 2 * D && G % 16 == 0) ? 2 : 1;
  float* red = (float*)(tile + ((G * D + 1) & ~1));          // [parts][2][D]
  const int share = G / parts;
  for (int idx = threadIdx.x; idx < D * parts; idx += blockDim.x) {
    const int d = idx % D, part = idx / D;
    float mn = INFINITY, mx = -INFINITY;
    for (int t = part * share; t < (part + 1) * share; ++t) {
      const float v = mz_u16_to_float(tile[t * D + d], DT);
      mn = fminf(mn, v); mx = fmaxf(mx, v);
    }
    red[(part * 2) * D + d] = mn;
    red[(part * 2 + 1) * D + d] = mx;
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < D * parts; idx += blockDim.x) {
    const int d = idx % D, part = idx / D;
    float mn = red[d], mx = red[D + d];
    if (parts == 2) { mn = fminf(mn, red[2 * D + d]); mx = fmaxf(mx, red[3 * D + d]); }
    MzQuantRow<DT> r;
    r.setup(mn, mx, s.bits, s.alpha_key, p.eps, p.ctab_k, p.ctab_k_n);
    uint8_t* dst = dst_rows + (long long)d * p.QB;
    for (int t0 = part * share; t0 < (part + 1) * share; t0 += 8) {
      const int n = min(8, (part + 1) * share - t0);
      unsigned long long word = 0;
      for (int k = 0; k < n; ++k)
        word |= ((unsigned long long)r.code(mz_u16_to_float(tile[(t0 + k) * D + d], DT))) << (k * s.bits);
      uint8_t* o = dst + (t0 >> 3) * s.bits;
      if (n == 8) mz_store_octet(o, word, s.bits);
      else {
        const int nb = (n * s.bits + 7) >> 3;
        for (int i = 0; i < nb; ++i) o[i] = (uint8_t)(word >> (8 * i));
      }
    }
    if (part == 0) {
      mz_store_from_float(s.k_mn, meta0 + d, r.lo, s.meta_dtype);
      mz_store_from_float(s.k_scale, meta0 + d, r.span, s.meta_dtype);
    }
  }
}

// value rows, G/8 lanes per row (G power of two in 8..256, D % 8 == 0)
template <int DT>
__device__ void flush_value_rows_fast(const FlushParams& p) {
  const mz_kv_store& s = p.s;
  const int G = s.group, D = s.head_dim, lpr = G >> 3;
  const int rows_per_cta = blockDim.x / lpr;
  const int sub = threadIdx.x % lpr;
  const long long row = (long long)(blockIdx.x - p.n_k_blocks) * rows_per_cta + threadIdx.x / lpr;
  const bool live = row < p.v_rows;
  long long r = live ? row : 0;
  const int grp = (int)(r % p.NG); r /= p.NG;
  const int t = (int)(r % p.n_vtokens); r /= p.n_vtokens;
  const int h = (int)(r % s.kv_heads);
  const int b = (int)(r / s.kv_heads);
  const int c0 = grp * G + sub * 8;
  float v[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = 0.f;
  if (live && c0 < D) {
    const uint16_t* src = (const uint16_t*)s.res_v + b * s.res_stride_b + h * s.res_stride_h +
                          (long long)(s.res_start + p.v_first + t) * s.res_stride_t + c0;
    if (p.k_vec) {
      const uint4 raw = *(const uint4*)src;
      const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        v[2 * i] = mz_u16_to_float((uint16_t)(w[i] & 0xffffu), DT);
        v[2 * i + 1] = mz_u16_to_float((uint16_t)(w[i] >> 16), DT);
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = mz_u16_to_float(src[i], DT);
    }
  }
  float mn = v[0], mx = v[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) { mn = fminf(mn, v[i]); mx = fmaxf(mx, v[i]); }
  for (int off = lpr >> 1; off > 0; off >>= 1) {
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, off));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
  }
  if (!live) return;
  MzQuantRow<DT> q;
  q.setup(mn, mx, s.bits, s.alpha_value, p.eps, p.ctab_v, p.ctab_v_n);
  unsigned long long word = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) word |= ((unsigned long long)q.code(v[i])) << (i * s.bits);
  const long long tok = s.v_tokens + t;
  uint8_t* dst = s.packed_v + b * s.pv_stride_b + h * s.pv_stride_h + (tok * p.NG + grp) * p.QB + sub * s.bits;
  if (!MZ_IN_BOUNDS((tok * p.NG + grp + 1) * p.QB - 1, s.pv_stride_h, 3) || !MZ_IN_BOUNDS(tok * p.NG + grp, s.vm_stride_h, 4)) return;
  mz_store_octet(dst, word, s.bits);
  if (sub == 0) {
    const long long m = b * s.vm_stride_b + h * s.vm_stride_h + tok * p.NG + grp;
    mz_store_from_float(s.v_mn, m, q.lo, s.meta_dtype);
    mz_store_from_float(s.v_scale, m, q.span, s.meta_dtype);
  }
}

// value rows, any G / D: one warp per row, bits written one byte at a time
template <int DT>
__device__ void flush_value_rows_generic(const FlushParams& p) {
  const mz_kv_store& s = p.s;
  const int G = s.group, D = s.head_dim;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long row = (long long)(blockIdx.x - p.n_k_blocks) * (blockDim.x >> 5) + warp;
  if (row >= p.v_rows) return;
  long long r = row;
  const int grp = (int)(r % p.NG); r /= p.NG;
  const int t = (int)(r % p.n_vtokens); r /= p.n_vtokens;
  const int h = (int)(r % s.kv_heads);
  const int b = (int)(r / s.kv_heads);
  const uint16_t* src = (const uint16_t*)s.res_v + b * s.res_stride_b + h * s.res_stride_h +
                        (long long)(s.res_start + p.v_first + t) * s.res_stride_t;
  float mn = INFINITY, mx = -INFINITY;
  for (int i = lane; i < G; i += 32) {
    const int c = grp * G + i;
    const float v = c < D ? mz_u16_to_float(src[c], DT) : 0.f;
    mn = fminf(mn, v); mx = fmaxf(mx, v);
  }
  for (int off = 16; off > 0; off >>= 1) {
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, off));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
  }
  MzQuantRow<DT> q;
  q.setup(mn, mx, s.bits, s.alpha_value, p.eps, p.ctab_v, p.ctab_v_n);
  const long long tok = s.v_tokens + t;
  uint8_t* dst = s.packed_v + b * s.pv_stride_b + h * s.pv_stride_h + (tok * p.NG + grp) * p.QB;
  if (!MZ_IN_BOUNDS((tok * p.NG + grp + 1) * p.QB - 1, s.pv_stride_h, 5) || !MZ_IN_BOUNDS(tok * p.NG + grp, s.vm_stride_h, 6)) return;
  for (int byte = lane; byte < p.QB; byte += 32) {
    uint32_t out = 0;
    const int first = (byte * 8) / s.bits, last = min(G - 1, (byte * 8 + 7) / s.bits);
    for (int i = first; i <= last; ++i) {
      const int c = grp * G + i;
      const uint32_t code = (uint32_t)q.code(c < D ? mz_u16_to_float(src[c], DT) : 0.f);
      const int sh = i * s.bits - byte * 8;
      out |= sh >= 0 ? (code << sh) : (code >> (-sh));
    }
    dst[byte] = (uint8_t)out;
  }
  if (lane == 0) {
    const long long m = b * s.vm_stride_b + h * s.vm_stride_h + tok * p.NG + grp;
    mz_store_from_float(s.v_mn, m, q.lo, s.meta_dtype);
    mz_store_from_float(s.v_scale, m, q.span, s.meta_dtype);
  }
}

template <int DT>
__global__ void __launch_bounds__(256) flush_kv_kernel(const FlushParams p) {
  extern __shared__ __align__(16) uint16_t s_tile[];
  if (blockIdx.x < p.n_k_blocks) flush_key_tile<DT>(p, s_tile);
  else if (p.v_fast) flush_value_rows_fast<DT>(p);
  else flush_value_rows_generic<DT>(p);
}

__global__ void append_kv_kernel(const mz_kv_store s, const uint16_t* __restrict__ k_new, const uint16_t* __restrict__ v_new,
                                 long long nsb, long long nsh) {
  // launched as a programmatic dependent: nothing is read or written before the previous kernel has completed,
  // and the next kernel (the decode attention) may start its own prologue right away
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int D = s.head_dim;
  const long long n = (long long)s.batch * s.kv_heads * D;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int d = (int)(i % D);
  const int h = (int)((i / D) % s.kv_heads);
  const int b = (int)(i / ((long long)D * s.kv_heads));
  const long long dst = b * s.res_stride_b + h * s.res_stride_h + (long long)(s.res_start + s.res_len) * s.res_stride_t + d;
  const long long src = b * nsb + h * nsh + d;
  ((uint16_t*)s.res_k)[dst] = k_new[src];
  ((uint16_t*)s.res_v)[dst] = v_new[src];
}

// store -> dense.  Keys: thread = (octet of tokens, channel) with channel fastest so that
// the 8 writes of a warp are contiguous; values: thread = (token, group, octet of channels).
__global__ void __launch_bounds__(256) dequant_keys_kernel(const mz_kv_store s, int g0, int g1, int QB, float eps,
                                                           const float* __restrict__ table, void* __restrict__ out, int out_dt) {
  const int G = s.group, D = s.head_dim, octs = (G + 7) >> 3, top = (1 << s.bits) - 1;
  const long long per_bh = (long long)(g1 - g0) * octs * D;
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= per_bh * s.batch * s.kv_heads) return;
  const int d = (int)(i % D); i /= D;
  const int oct = (int)(i % octs); i /= octs;
  const int g = g0 + (int)(i % (g1 - g0)); i /= (g1 - g0);
  const int h = (int)(i % s.kv_heads);
  const int b = (int)(i / s.kv_heads);
  const long long m = b * s.km_stride_b + h * s.km_stride_h + (long long)g * D + d;
  const MzRowParams r = mz_row_params(mz_load_as_float(s.k_mn, m, s.meta_dtype), mz_load_as_float(s.k_scale, m, s.meta_dtype), top, eps);
  const uint8_t* row = s.packed_k + b * s.pk_stride_b + h * s.pk_stride_h + ((long long)g * D + d) * QB;
  const long long S = (long long)(g1 - g0) * G;
  const long long o0 = (((long long)b * s.kv_heads + h) * S + (long long)(g - g0) * G + oct * 8) * D + d;
  const int n = min(8, G - oct * 8);
  for (int k = 0; k < n; ++k) {
    const int q = mz_extract_code(row, oct * 8 + k, s.bits, QB);
    mz_store_from_float(out, o0 + (long long)k * D, mz_dequant_exact(r, q, table, top + 1), out_dt);
  }
}

__global__ void __launch_bounds__(256) dequant_values_kernel(const mz_kv_store s, int t0, int t1, int QB, int NG, float eps,
                                                             const float* __restrict__ table, void* __restrict__ out, int out_dt) {
  const int G = s.group, D = s.head_dim, octs = (G + 7) >> 3, top = (1 << s.bits) - 1;
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long total = (long long)s.batch * s.kv_heads * (t1 - t0) * NG * octs;
  if (i >= total) return;
  const int oct = (int)(i % octs); i /= octs;
  const int grp = (int)(i % NG); i /= NG;
  const int t = t0 + (int)(i % (t1 - t0)); i /= (t1 - t0);
  const int h = (int)(i % s.kv_heads);
  const int b = (int)(i / s.kv_heads);
  const long long m = b * s.vm_stride_b + h * s.vm_stride_h + (long long)t * NG + grp;
  const MzRowParams r = mz_row_params(mz_load_as_float(s.v_mn, m, s.meta_dtype), mz_load_as_float(s.v_scale, m, s.meta_dtype), top, eps);
  const uint8_t* row = s.packed_v + b * s.pv_stride_b + h * s.pv_stride_h + ((long long)t * NG + grp) * QB;
  const long long o0 = (((long long)b * s.kv_heads + h) * (t1 - t0) + (t - t0)) * D;
  for (int k = 0; k < 8; ++k) {
    const int idx = oct * 8 + k, c = grp * G + idx;
    if (idx >= G || c >= D) break;
    const int q = mz_extract_code(row, idx, s.bits, QB);
    mz_store_from_float(out, o0 + c, mz_dequant_exact(r, q, table, top + 1), out_dt);
  }
}

bool pow2(int v) { return v > 0 && (v & (v - 1)) == 0; }
}  // namespace

extern "C" int mz_flush_kv_parts(const mz_kv_store* s, int n_key_tokens, int value_first, int n_value_tokens, float eps,
                                 void* stream) {
  MZ_RANGE("mz_flush_kv_parts");
  int rc = mz_check_store_basic(s);
  if (rc) return rc;
  if ((rc = mz_check_store_quantized(s))) return rc;
  if ((rc = mz_check_store_residual(s))) return rc;
  MZ_REQUIRE(n_key_tokens >= 0 && n_key_tokens % s->group == 0, "n_key_tokens %d is not a multiple of group %d", n_key_tokens,
             s->group);
  MZ_REQUIRE(n_key_tokens <= s->res_len, "flush of %d key tokens but residual holds %d", n_key_tokens, s->res_len);
  MZ_REQUIRE(value_first >= 0 && n_value_tokens >= 0 && value_first + n_value_tokens <= s->res_len,
             "value tokens [%d, %d) outside the residual window of %d", value_first, value_first + n_value_tokens, s->res_len);
  if (n_key_tokens == 0 && n_value_tokens == 0) return MZ_OK;
  const MzStoreGeom g = mz_geom(*s);
  FlushParams p;
  p.s = *s; p.n_tiles = n_key_tokens / g.G; p.v_first = value_first; p.n_vtokens = n_value_tokens;
  p.QB = g.QB; p.NG = g.NG; p.eps = eps;
  if ((rc = mz_get_compand_table(g.kv_dt, s->alpha_key, &p.ctab_k, &p.ctab_k_n))) return rc;
  if ((rc = mz_get_compand_table(g.kv_dt, s->alpha_value, &p.ctab_v, &p.ctab_v_n))) return rc;
  const long long kb = (long long)g.B * g.KVH * p.n_tiles;
  p.v_rows = (long long)g.B * g.KVH * n_value_tokens * g.NG;
  p.v_fast = pow2(g.G) && g.G >= 8 && g.G <= 256 && g.D % 8 == 0;
  p.k_vec = g.D % 8 == 0 && s->res_stride_t % 8 == 0 && s->res_stride_h % 8 == 0 && s->res_stride_b % 8 == 0 &&
            (uintptr_t)s->res_k % 16 == 0 && (uintptr_t)s->res_v % 16 == 0;
  const int rows_per_cta = p.v_fast ? 256 / (g.G / 8) : 8;
  const long long vb = (p.v_rows + rows_per_cta - 1) / rows_per_cta;
  MZ_REQUIRE(kb + vb < (1LL << 31), "flush too large");
  p.n_k_blocks = (unsigned)kb;
  const size_t smem = (size_t)((g.G * g.D + 1) & ~1) * 2 + (size_t)g.D * 4 * sizeof(float);   // key tile + partial min/max of two parts
  if (smem > 200 * 1024) return mz_fail(MZ_ERR_UNSUPPORTED, "key tile of %zu bytes exceeds shared memory", smem);
  cudaStream_t st = (cudaStream_t)stream;
  if (g.kv_dt == MZ_BF16) {
    if (smem > 48 * 1024) MZ_CUDA(cudaFuncSetAttribute(flush_kv_kernel<MZ_BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    flush_kv_kernel<MZ_BF16><<<(unsigned)(kb + vb), 256, smem, st>>>(p);
  } else {
    if (smem > 48 * 1024) MZ_CUDA(cudaFuncSetAttribute(flush_kv_kernel<MZ_F16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    flush_kv_kernel<MZ_F16><<<(unsigned)(kb + vb), 256, smem, st>>>(p);
  }
  MZ_LAUNCH_CHECK("flush_kv");
  return MZ_OK;
}

extern "C" int mz_flush_kv(const mz_kv_store* s, int n_tokens, float eps, void* stream) {
  return mz_flush_kv_parts(s, n_tokens, 0, n_tokens, eps, stream);
}

extern "C" int mz_append_kv(const mz_kv_store* s, const void* k_new, const void* v_new, long long nsb, long long nsh, void* stream) {
  MZ_RANGE("mz_append_kv");
  int rc = mz_check_store_basic(s);
  if (rc) return rc;
  if ((rc = mz_check_store_residual(s))) return rc;
  MZ_REQUIRE(k_new && v_new, "NULL new token pointer");
  const long long n = (long long)s->batch * s->kv_heads * s->head_dim;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)((n + 255) / 256));
  cfg.blockDim = dim3(256);
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  MZ_CUDA(cudaLaunchKernelEx(&cfg, append_kv_kernel, *s, (const uint16_t*)k_new, (const uint16_t*)v_new, nsb, nsh));
  MZ_LAUNCH_CHECK("append_kv");
  return MZ_OK;
}

extern "C" int mz_dequantize_kv(const mz_kv_store* s, int g0, int g1, void* out_k, int t0, int t1, void* out_v, int out_dtype,
                                float eps, void* stream) {
  MZ_RANGE("mz_dequantize_kv");
  int rc = mz_check_store_basic(s);
  if (rc) return rc;
  if ((rc = mz_check_store_quantized(s))) return rc;
  MZ_REQUIRE(mz_dtype_ok(out_dtype), "bad out_dtype");
  const MzStoreGeom g = mz_geom(*s);
  cudaStream_t st = (cudaStream_t)stream;
  if (out_k && g1 > g0) {
    MZ_REQUIRE(g0 >= 0 && g1 <= s->k_groups, "key group range [%d,%d) outside [0,%d)", g0, g1, s->k_groups);
    const float* table;
    if ((rc = mz_get_expand_table(g.bits, s->alpha_key, &table))) return rc;
    const long long n = (long long)g.B * g.KVH * (g1 - g0) * ((g.G + 7) / 8) * g.D;
    dequant_keys_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(*s, g0, g1, g.QB, eps, table, out_k, out_dtype);
    MZ_LAUNCH_CHECK("dequant_keys");
  }
  if (out_v && t1 > t0) {
    MZ_REQUIRE(t0 >= 0 && t1 <= s->v_tokens, "value token range [%d,%d) outside [0,%d)", t0, t1, s->v_tokens);
    const float* table;
    if ((rc = mz_get_expand_table(g.bits, s->alpha_value, &table))) return rc;
    const long long n = (long long)g.B * g.KVH * (t1 - t0) * g.NG * ((g.G + 7) / 8);
    dequant_values_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(*s, t0, t1, g.QB, g.NG, eps, table, out_v, out_dtype);
    MZ_LAUNCH_CHECK("dequant_values");
  }
  return MZ_OK;
}
