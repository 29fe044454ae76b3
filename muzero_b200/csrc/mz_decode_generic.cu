// Decode attention, shape-generic kernel: any bits 1..8, any group size, head_dim <= 512,
// up to 16 query heads per kv head.  One CTA per (split, kv head, batch) walks its share of
// the sequence in units of 32 tokens: dequantize K unit -> shared, logits, online softmax,
// dequantize V unit -> shared, accumulate.  Used for shapes the tiled kernel does not cover
// and as an on-device cross-check of it.
#include "mz_decode.cuh"

namespace {
constexpr int TT = 32;        // tokens per unit
constexpr int MAX_GQA = 16;
constexpr int THREADS = 256;

__device__ __forceinline__ float load_kv_elem(const void* p, long long i, int dt) {
  return mz_u16_to_float(((const uint16_t*)p)[i], dt);
}

__global__ void __launch_bounds__(THREADS) decode_generic_kernel(const MzDecodeParams p) {
  extern __shared__ float smem[];
  const mz_kv_store& s = p.s;
  const int D = s.head_dim, G = s.group, gqa = p.gqa, top = (1 << s.bits) - 1;
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x;
  const int ldk = D + 1;
  float* q_s = smem;                       // [gqa][D]
  float* kv_s = q_s + gqa * D;             // [TT][D+1]
  float* p_s = kv_s + TT * ldk;            // [gqa][TT]
  float* m_s = p_s + gqa * TT;             // [gqa]
  float* l_s = m_s + gqa;                  // [gqa]
  float* c_s = l_s + gqa;                  // [gqa] correction of this unit

  for (int i = tid; i < gqa * D; i += THREADS) {
    const int hh = i / D, d = i % D;
    q_s[i] = load_kv_elem(p.query, b * p.q_stride_b + (long long)(kvh * gqa + hh) * p.q_stride_h + d, s.kv_dtype);
  }
  if (tid < gqa) { m_s[tid] = -INFINITY; l_s[tid] = 0.f; }
  float acc[MAX_GQA][2];
#pragma unroll
  for (int hh = 0; hh < MAX_GQA; ++hh) acc[hh][0] = acc[hh][1] = 0.f;

  const int nq = s.k_groups * G;                 // quantized tokens
  const int units_q = (nq + TT - 1) / TT;
  const int units_d = (s.res_len + TT - 1) / TT;
  const int units = units_q + units_d;
  const int u0 = (int)((long long)units * split / p.splits);
  const int u1 = (int)((long long)units * (split + 1) / p.splits);

  const uint8_t* pk = s.packed_k + b * s.pk_stride_b + kvh * s.pk_stride_h;
  const uint8_t* pv = s.packed_v + b * s.pv_stride_b + kvh * s.pv_stride_h;
  const long long km0 = b * s.km_stride_b + kvh * s.km_stride_h;
  const long long vm0 = b * s.vm_stride_b + kvh * s.vm_stride_h;
  const long long res0 = b * s.res_stride_b + kvh * s.res_stride_h;
  __syncthreads();

  for (int u = u0; u < u1; ++u) {
    const bool dense = u >= units_q;
    const int t0 = dense ? (u - units_q) * TT : u * TT;            // first token inside its region
    const int ntok = min(TT, (dense ? s.res_len : nq) - t0);
    // ---- K unit -> shared
    for (int i = tid; i < ntok * D; i += THREADS) {
      const int tt = i / D, d = i % D, t = t0 + tt;
      float v;
      if (dense) {
        v = load_kv_elem(s.res_k, res0 + (long long)(s.res_start + t) * s.res_stride_t + d, s.kv_dtype);
      } else {
        const int g = t / G, idx = t % G;
        const long long mrow = km0 + (long long)g * D + d;
        const MzRowParams r = mz_row_params(mz_load_as_float(s.k_mn, mrow, s.meta_dtype),
                                            mz_load_as_float(s.k_scale, mrow, s.meta_dtype), top, p.eps);
        const int code = mz_extract_code(pk + ((long long)g * D + d) * p.QB, idx, s.bits, p.QB);
        v = mz_dequant_exact(r, code, p.table_k, top + 1);
      }
      kv_s[tt * ldk + d] = v;
    }
    __syncthreads();
    // ---- logits
    for (int i = tid; i < gqa * TT; i += THREADS) {
      const int hh = i / TT, tt = i % TT;
      float sc = -INFINITY;
      if (tt < ntok) {
        float dot = 0.f;
        for (int d = 0; d < D; ++d) dot = fmaf(q_s[hh * D + d], kv_s[tt * ldk + d], dot);
        sc = dot * p.scaling;
        if (p.mask) sc += mz_load_as_float(p.mask, b * p.mask_stride_b + (dense ? nq : 0) + t0 + tt, p.mask_dtype);
      }
      p_s[i] = sc;
    }
    __syncthreads();
    // ---- online softmax, one thread per head
    if (tid < gqa) {
      float mx = m_s[tid];
      for (int tt = 0; tt < ntok; ++tt) mx = fmaxf(mx, p_s[tid * TT + tt]);
      float sum = 0.f;
      for (int tt = 0; tt < TT; ++tt) {
        const float e = (tt < ntok && mx > -INFINITY) ? __expf(p_s[tid * TT + tt] - mx) : 0.f;
        p_s[tid * TT + tt] = e;
        sum += e;
      }
      const float corr = (m_s[tid] > -INFINITY) ? __expf(m_s[tid] - mx) : 0.f;
      c_s[tid] = corr;
      l_s[tid] = l_s[tid] * corr + sum;
      m_s[tid] = mx;
    }
    // ---- V unit -> shared (K values are no longer needed once logits are written)
    for (int i = tid; i < ntok * D; i += THREADS) {
      const int tt = i / D, d = i % D, t = t0 + tt;
      float v;
      if (dense) {
        v = load_kv_elem(s.res_v, res0 + (long long)(s.res_start + t) * s.res_stride_t + d, s.kv_dtype);
      } else {
        const int grp = d / G, idx = d % G;
        const long long mrow = vm0 + (long long)t * p.NG + grp;
        const MzRowParams r = mz_row_params(mz_load_as_float(s.v_mn, mrow, s.meta_dtype),
                                            mz_load_as_float(s.v_scale, mrow, s.meta_dtype), top, p.eps);
        const int code = mz_extract_code(pv + ((long long)t * p.NG + grp) * p.QB, idx, s.bits, p.QB);
        v = mz_dequant_exact(r, code, p.table_v, top + 1);
      }
      kv_s[tt * ldk + d] = v;
    }
    __syncthreads();
    // ---- accumulate
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int d = tid + j * THREADS;
      if (d < D) {
#pragma unroll
        for (int hh = 0; hh < MAX_GQA; ++hh) {
          if (hh < gqa) {
            float a = acc[hh][j] * c_s[hh];
            for (int tt = 0; tt < ntok; ++tt) a = fmaf(p_s[hh * TT + tt], kv_s[tt * ldk + d], a);
            acc[hh][j] = a;
          }
        }
      }
    }
    __syncthreads();
  }
  // ---- partial out
  for (int hh = 0; hh < gqa; ++hh) {
    const long long slot = ((long long)b * p.H + kvh * gqa + hh) * p.splits + split;
    if (tid == 0 && MZ_IN_BOUNDS(slot, p.part.slots, 13)) { p.part.m[slot] = m_s[hh]; p.part.l[slot] = l_s[hh]; }
  }
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int d = tid + j * THREADS;
    if (d < D) {
#pragma unroll
      for (int hh = 0; hh < MAX_GQA; ++hh) {
        if (hh < gqa) {
          const long long slot = ((long long)b * p.H + kvh * gqa + hh) * p.splits + split;
          if (MZ_IN_BOUNDS(slot, p.part.slots, 14)) p.part.acc[slot * D + d] = acc[hh][j];
        }
      }
    }
  }
}
}  // namespace

int mz_decode_units_generic(const mz_kv_store& s) {
  return (s.k_groups * s.group + TT - 1) / TT + (s.res_len + TT - 1) / TT;
}

int mz_launch_decode_generic(const MzDecodeParams& p, cudaStream_t st) {
  const mz_kv_store& s = p.s;
  if (s.head_dim > 2 * THREADS) return mz_fail(MZ_ERR_UNSUPPORTED, "head_dim %d > %d unsupported", s.head_dim, 2 * THREADS);
  if (p.gqa > MAX_GQA) return mz_fail(MZ_ERR_UNSUPPORTED, "%d query heads per kv head > %d unsupported", p.gqa, MAX_GQA);
  const size_t smem = sizeof(float) * ((size_t)p.gqa * s.head_dim + (size_t)TT * (s.head_dim + 1) + (size_t)p.gqa * TT + 3 * p.gqa);
  if (smem > 48 * 1024) MZ_CUDA(cudaFuncSetAttribute(decode_generic_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid((unsigned)p.splits, (unsigned)s.kv_heads, (unsigned)s.batch);
  decode_generic_kernel<<<grid, THREADS, smem, st>>>(p);
  MZ_LAUNCH_CHECK("decode_generic");
  return MZ_OK;
}
