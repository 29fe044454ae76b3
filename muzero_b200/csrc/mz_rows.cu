// Row quantizer / dequantizer: x[n_rows, G] <-> packed codes + (mn, scale).
//
// Fast path (G a power of two, 8..256): G/8 lanes own one row, each lane owns
// 8 consecutive values = one 16-byte load of 16-bit input and exactly `bits`
// packed bytes; the row min/max is a shuffle reduction over those lanes.
// Any other G takes the warp-per-row kernel.
#include "mz_quant_math.cuh"

namespace {

template <int DT>
__device__ __forceinline__ void load8(const void* x, long long elem0, float (&v)[8]) {
  if (DT == MZ_F32) {
    const float4* p = (const float4*)((const float*)x + elem0);
    float4 a = p[0], b = p[1];
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  } else {
    uint4 raw = *(const uint4*)((const uint16_t*)x + elem0);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = mz_u16_to_float((uint16_t)(w[i] & 0xffffu), DT);
      v[2 * i + 1] = mz_u16_to_float((uint16_t)(w[i] >> 16), DT);
    }
  }
}

template <int DT>
__global__ void __launch_bounds__(256) quantize_rows_octet_kernel(
    const void* __restrict__ x, long long n_rows, int group, int bits, float alpha, float eps,
    uint8_t* __restrict__ packed, void* __restrict__ mn_out, void* __restrict__ scale_out, int meta_dtype,
    const uint16_t* __restrict__ ctab, int ctab_n) {
  const int lpr = group >> 3;                      // lanes per row
  const int rows_per_cta = blockDim.x / lpr;
  const int sub = threadIdx.x % lpr;
  const long long row = (long long)blockIdx.x * rows_per_cta + threadIdx.x / lpr;
  const bool live = row < n_rows;
  float v[8];
  if (live) load8<DT>(x, row * group + sub * 8, v);
  else {
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = 0.f;
  }
  float mn = v[0], mx = v[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) { mn = fminf(mn, v[i]); mx = fmaxf(mx, v[i]); }
  for (int off = lpr >> 1; off > 0; off >>= 1) {
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, off));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
  }
  if (!live) return;
  MzQuantRow<DT> r;
  r.setup(mn, mx, bits, alpha, eps, ctab, ctab_n);
  unsigned long long word = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) word |= ((unsigned long long)r.code(v[i])) << (i * bits);
  mz_store_octet(packed + row * (long long)(lpr * bits) + sub * bits, word, bits);
  if (sub == 0) {
    mz_store_from_float(mn_out, row, r.lo, meta_dtype);
    mz_store_from_float(scale_out, row, r.span, meta_dtype);
  }
}

// any G <= 1024: one warp per row, codes staged in shared memory
template <int DT>
__global__ void __launch_bounds__(128) quantize_rows_generic_kernel(
    const void* __restrict__ x, long long n_rows, int group, int bits, float alpha, float eps,
    uint8_t* __restrict__ packed, void* __restrict__ mn_out, void* __restrict__ scale_out, int meta_dtype,
    const uint16_t* __restrict__ ctab, int ctab_n) {
  extern __shared__ uint8_t s_codes[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
  if (row >= n_rows) return;
  uint8_t* codes = s_codes + warp * group;
  float mn = INFINITY, mx = -INFINITY;
  for (int i = lane; i < group; i += 32) {
    float f = MzType<DT>::load(x, row * group + i);
    mn = fminf(mn, f); mx = fmaxf(mx, f);
  }
  for (int off = 16; off > 0; off >>= 1) {
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, off));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
  }
  MzQuantRow<DT> r;
  r.setup(mn, mx, bits, alpha, eps, ctab, ctab_n);
  for (int i = lane; i < group; i += 32) codes[i] = (uint8_t)r.code(MzType<DT>::load(x, row * group + i));
  __syncwarp();
  const int qb = (group * bits + 7) >> 3;
  for (int b = lane; b < qb; b += 32) {
    uint32_t byte = 0;
    for (int k = 0; k < 8; ++k) {
      int bit = b * 8 + k, idx = bit / bits;
      if (idx < group) byte |= ((codes[idx] >> (bit % bits)) & 1u) << k;
    }
    packed[row * qb + b] = (uint8_t)byte;
  }
  if (lane == 0) {
    mz_store_from_float(mn_out, row, r.lo, meta_dtype);
    mz_store_from_float(scale_out, row, r.span, meta_dtype);
  }
}

__global__ void __launch_bounds__(256) dequantize_rows_kernel(
    const uint8_t* __restrict__ packed, const void* __restrict__ mn, const void* __restrict__ scale, int meta_dtype,
    long long n_rows, int group, int bits, float eps, const float* __restrict__ table,
    void* __restrict__ out, int out_dtype) {
  const int octets = (group + 7) >> 3;
  const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long row = gid / octets;
  const int oct = (int)(gid % octets);
  if (row >= n_rows) return;
  const int qb = (group * bits + 7) >> 3;
  const int top = (1 << bits) - 1;
  const MzRowParams r = mz_row_params(mz_load_as_float(mn, row, meta_dtype), mz_load_as_float(scale, row, meta_dtype), top, eps);
  const uint8_t* src = packed + row * qb;
  const int n = min(8, group - oct * 8);
  for (int i = 0; i < n; ++i) {
    const int idx = oct * 8 + i;
    const int q = mz_extract_code(src, idx, bits, qb);
    mz_store_from_float(out, row * group + idx, mz_dequant_exact(r, q, table, top + 1), out_dtype);
  }
}

bool pow2(int v) { return v > 0 && (v & (v - 1)) == 0; }

template <int DT>
int launch_quantize(const void* x, long long n_rows, int group, int bits, float alpha, float eps, uint8_t* packed,
                    void* mn, void* scale, int meta_dtype, cudaStream_t st) {
  const uint16_t* ctab = nullptr;
  int ctab_n = 0;
  if (DT != MZ_F32) {
    int rc = mz_get_compand_table(DT, alpha, &ctab, &ctab_n);
    if (rc != MZ_OK) return rc;
  }
  const bool aligned = ((uintptr_t)x % 16 == 0) && ((uintptr_t)packed % 8 == 0);
  if (pow2(group) && group >= 8 && group <= 256 && aligned) {
    const int rows_per_cta = 256 / (group / 8);
    const long long blocks = (n_rows + rows_per_cta - 1) / rows_per_cta;
    quantize_rows_octet_kernel<DT><<<(unsigned)blocks, 256, 0, st>>>(x, n_rows, group, bits, alpha, eps, packed, mn, scale,
                                                                      meta_dtype, ctab, ctab_n);
  } else {
    if (group > 1024) return mz_fail(MZ_ERR_UNSUPPORTED, "group %d > 1024 unsupported", group);
    const long long blocks = (n_rows + 3) / 4;
    quantize_rows_generic_kernel<DT><<<(unsigned)blocks, 128, 4 * group, st>>>(x, n_rows, group, bits, alpha, eps, packed, mn,
                                                                              scale, meta_dtype, ctab, ctab_n);
  }
  MZ_LAUNCH_CHECK("quantize_rows");
  return MZ_OK;
}
}  // namespace

extern "C" int mz_quantize_rows(const void* x, int x_dtype, long long n_rows, int group, int bits, float alpha, float eps,
                                uint8_t* packed, void* mn, void* scale, int meta_dtype, void* stream) {
  MZ_RANGE("mz_quantize_rows");
  MZ_REQUIRE(mz_dtype_ok(x_dtype) && mz_dtype_ok(meta_dtype), "bad dtype code");
  MZ_REQUIRE(bits >= 1 && bits <= 8, "bits must be 1..8, got %d", bits);
  MZ_REQUIRE(group > 0 && n_rows >= 0, "bad shape: n_rows=%lld group=%d", n_rows, group);
  MZ_REQUIRE(alpha > 0.f, "alpha must be > 0");
  if (n_rows == 0) return MZ_OK;
  MZ_REQUIRE(x && packed && mn && scale, "NULL pointer");
  MZ_REQUIRE(n_rows < (1LL << 31) * 8, "n_rows too large");
  cudaStream_t st = (cudaStream_t)stream;
  switch (x_dtype) {
    case MZ_F32: return launch_quantize<MZ_F32>(x, n_rows, group, bits, alpha, eps, packed, mn, scale, meta_dtype, st);
    case MZ_F16: return launch_quantize<MZ_F16>(x, n_rows, group, bits, alpha, eps, packed, mn, scale, meta_dtype, st);
    default: return launch_quantize<MZ_BF16>(x, n_rows, group, bits, alpha, eps, packed, mn, scale, meta_dtype, st);
  }
}

extern "C" int mz_dequantize_rows(const uint8_t* packed, const void* mn, const void* scale, int meta_dtype, long long n_rows,
                                  int group, int bits, float alpha, float eps, void* out, int out_dtype, void* stream) {
  MZ_RANGE("mz_dequantize_rows");
  MZ_REQUIRE(mz_dtype_ok(out_dtype) && mz_dtype_ok(meta_dtype), "bad dtype code");
  MZ_REQUIRE(bits >= 1 && bits <= 8, "bits must be 1..8, got %d", bits);
  MZ_REQUIRE(group > 0 && n_rows >= 0, "bad shape: n_rows=%lld group=%d", n_rows, group);
  MZ_REQUIRE(alpha > 0.f, "alpha must be > 0");
  if (n_rows == 0) return MZ_OK;
  MZ_REQUIRE(packed && mn && scale && out, "NULL pointer");
  const float* table = nullptr;
  int rc = mz_get_expand_table(bits, alpha, &table);
  if (rc != MZ_OK) return rc;
  const long long threads = n_rows * ((group + 7) / 8);
  const long long blocks = (threads + 255) / 256;
  MZ_REQUIRE(blocks < (1LL << 31), "problem too large");
  dequantize_rows_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(packed, mn, scale, meta_dtype, n_rows, group, bits,
                                                                           eps, table, out, out_dtype);
  MZ_LAUNCH_CHECK("dequantize_rows");
  return MZ_OK;
}
