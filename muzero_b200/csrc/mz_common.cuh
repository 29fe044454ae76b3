// Shared host/device helpers of the muzero_b200 CUDA library (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/muzero_b200.h"

// ---------------------------------------------------------------------------
// error reporting (thread-local text, status codes from the public header)
// ---------------------------------------------------------------------------
int mz_fail(int code, const char* fmt, ...);

#define MZ_REQUIRE(cond, ...)                         \
  do {                                                \
    if (!(cond)) return mz_fail(MZ_ERR_ARG, __VA_ARGS__); \
  } while (0)

#define MZ_CUDA(call)                                                                  \
  do {                                                                                 \
    cudaError_t e__ = (call);                                                          \
    if (e__ != cudaSuccess)                                                            \
      return mz_fail(MZ_ERR_CUDA, "%s failed: %s", #call, cudaGetErrorString(e__));    \
  } while (0)

#define MZ_LAUNCH_CHECK(name)                                                          \
  do {                                                                                 \
    cudaError_t e__ = cudaGetLastError();                                              \
    if (e__ != cudaSuccess)                                                            \
      return mz_fail(MZ_ERR_CUDA, "launch of %s failed: %s", name, cudaGetErrorString(e__)); \
  } while (0)

// ---------------------------------------------------------------------------
// NVTX range around an entry point: named in Nsight timelines, a few ns when no tool is attached.
// ---------------------------------------------------------------------------
#include <nvtx3/nvToolsExt.h>
struct MzRange {
  explicit MzRange(const char* name) { nvtxRangePushA(name); }
  ~MzRange() { nvtxRangePop(); }
  MzRange(const MzRange&) = delete;
  MzRange& operator=(const MzRange&) = delete;
};
#define MZ_RANGE(name) MzRange mz_range__(name)

// ---------------------------------------------------------------------------
// checked build (-DMZ_BOUNDS): every guarded global access compares its element index with the extent the
// host passed; an access outside is SKIPPED and counted (first offender kept), never trapped, so the context
// stays usable and mz_bounds_violations() reports it.  Without the flag the guard compiles to `true`.
// ---------------------------------------------------------------------------
#ifdef MZ_BOUNDS
struct MzBoundsRecord { unsigned long long count; long long index; long long extent; int site; int pad; };
extern __device__ MzBoundsRecord g_mz_bounds;
__device__ __forceinline__ bool mz_in_bounds(long long i, long long n, int site) {
  if (i >= 0 && i < n) return true;
  if (atomicAdd(&g_mz_bounds.count, 1ull) == 0) { g_mz_bounds.index = i; g_mz_bounds.extent = n; g_mz_bounds.site = site; }
  return false;
}
#define MZ_IN_BOUNDS(i, n, site) mz_in_bounds((long long)(i), (long long)(n), (site))
#else
#define MZ_IN_BOUNDS(i, n, site) true
#endif

static inline int mz_dtype_size(int dt) { return dt == MZ_F32 ? 4 : 2; }
static inline bool mz_dtype_ok(int dt) { return dt == MZ_F32 || dt == MZ_F16 || dt == MZ_BF16; }
static inline int mz_row_bytes(int group, int bits) { return (group * bits + 7) / 8; }

// ---------------------------------------------------------------------------
// per-device lookup tables (built lazily, cached for the life of the process)
// ---------------------------------------------------------------------------
// fp32 table [(2^bits) x (2^bits)]: expm1(clamp(numer/denom)*log1p(alpha))/alpha, row = denom.
int mz_get_expand_table(int bits, float alpha, const float** dev_table);
// u16 table over every value p of `dtype` in [0,1] (index = bit pattern of p):
// round_T(round_T(log1p(round_T(alpha*p))) / log1p_f32(alpha)), stored as bits of `dtype`.
int mz_get_compand_table(int dtype, float alpha, const uint16_t** dev_table, int* n_entries);

// ---------------------------------------------------------------------------
// device: element type traits
// ---------------------------------------------------------------------------
template <int DT> struct MzType;
template <> struct MzType<MZ_F32> {
  using T = float;
  static __device__ __forceinline__ float load(const void* p, long long i) { return ((const float*)p)[i]; }
  static __device__ __forceinline__ void store(void* p, long long i, float v) { ((float*)p)[i] = v; }
  static __device__ __forceinline__ float round(float v) { return v; }
};
template <> struct MzType<MZ_F16> {
  using T = __half;
  static __device__ __forceinline__ float load(const void* p, long long i) { return __half2float(((const __half*)p)[i]); }
  static __device__ __forceinline__ void store(void* p, long long i, float v) { ((__half*)p)[i] = __float2half_rn(v); }
  static __device__ __forceinline__ float round(float v) { return __half2float(__float2half_rn(v)); }
};
template <> struct MzType<MZ_BF16> {
  using T = __nv_bfloat16;
  static __device__ __forceinline__ float load(const void* p, long long i) { return __bfloat162float(((const __nv_bfloat16*)p)[i]); }
  static __device__ __forceinline__ void store(void* p, long long i, float v) { ((__nv_bfloat16*)p)[i] = __float2bfloat16_rn(v); }
  static __device__ __forceinline__ float round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
};

// runtime-typed scalar access (metadata, outputs on cold paths)
__device__ __forceinline__ float mz_load_as_float(const void* p, long long i, int dt) {
  if (dt == MZ_F32) return ((const float*)p)[i];
  if (dt == MZ_F16) return __half2float(((const __half*)p)[i]);
  return __bfloat162float(((const __nv_bfloat16*)p)[i]);
}
__device__ __forceinline__ void mz_store_from_float(void* p, long long i, float v, int dt) {
  if (dt == MZ_F32) ((float*)p)[i] = v;
  else if (dt == MZ_F16) ((__half*)p)[i] = __float2half_rn(v);
  else ((__nv_bfloat16*)p)[i] = __float2bfloat16_rn(v);
}
__device__ __forceinline__ float mz_u16_to_float(uint16_t u, int dt) {
  if (dt == MZ_F16) return __half2float(__ushort_as_half(u));
  return __uint_as_float(((uint32_t)u) << 16);
}

// ---------------------------------------------------------------------------
// device: per-row compander parameters of the fp32 dequantizer
// (za, zero level, side extents; one rounding per op, no fused multiply-add)
// ---------------------------------------------------------------------------
struct MzRowParams {
  float lo, span;   // stored metadata as fp32
  float anchor;     // za
  float room_up, room_dn;
  int zero_code, steps_up, steps_dn;
};

__device__ __forceinline__ MzRowParams mz_row_params(float lo, float span, int top, float eps) {
  MzRowParams r;
  r.lo = lo;
  r.span = span;
  float a = __fdiv_rn(__fsub_rn(0.0f, lo), span);
  a = fminf(fmaxf(a, 0.0f), 1.0f);
  r.anchor = a;
  float z = rintf(__fmul_rn(a, (float)top));
  r.zero_code = (int)z;
  r.steps_up = max(top - r.zero_code, 1);
  r.steps_dn = max(r.zero_code, 1);
  r.room_up = fmaxf(__fsub_rn(1.0f, a), eps);
  r.room_dn = fmaxf(a, eps);
  return r;
}

// exact fp32 value of code q; `table` is the expand table with row stride `tw`=2^bits
__device__ __forceinline__ float mz_dequant_exact(const MzRowParams& r, int q, const float* __restrict__ table, int tw) {
  float unit;
  if (q >= r.zero_code) {
    float grow = table[r.steps_up * tw + min(q - r.zero_code, r.steps_up)];
    unit = __fadd_rn(r.anchor, __fmul_rn(r.room_up, grow));
  } else {
    float grow = table[r.steps_dn * tw + min(r.zero_code - q, r.steps_dn)];
    unit = __fsub_rn(r.anchor, __fmul_rn(r.room_dn, grow));
  }
  unit = fminf(fmaxf(unit, 0.0f), 1.0f);
  return __fadd_rn(__fmul_rn(unit, r.span), r.lo);
}

// code `idx` of a packed row (LSB-first bitstream), any bits 1..8
__device__ __forceinline__ int mz_extract_code(const uint8_t* __restrict__ row, int idx, int bits, int row_bytes) {
  int bit = idx * bits;
  int byte = bit >> 3;
  uint32_t w = row[byte];
  if (byte + 1 < row_bytes) w |= ((uint32_t)row[byte + 1]) << 8;
  return (w >> (bit & 7)) & ((1u << bits) - 1u);
}
