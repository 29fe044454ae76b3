// Helpers shared by the two tensor-core decode kernels (mma.sync and tcgen05): shared memory by
// shared-window address, the replicated lookup table, the per-row constants of the folded dequantizer.
#pragma once
#include "mz_tiles_common.cuh"

namespace mzm {
using mzt::cp_async_commit;
using mzt::cp_async_wait;
using mzt::D;
using mzt::ex2f;
using mzt::LOG2E;
using mzt::prmt;

constexpr int G = 64;                       // tokens per packed tile
constexpr uint32_t TBL = 65536;             // shared-window address of the lookup table

// ---- shared memory by shared-window address (no generic-address arithmetic in the loops) ----
__device__ __forceinline__ uint32_t lds32(uint32_t a) {
  uint32_t v;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ uint32_t lds16(uint32_t a) {
  uint16_t v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ uint32_t lds8(uint32_t a) {
  uint16_t v;
  asm volatile("ld.shared.u8 %0, [%1];" : "=h"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ float ldsf(uint32_t a) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
  return v;
}
__device__ __forceinline__ void sts32(uint32_t a, uint32_t v) { asm volatile("st.shared.b32 [%0], %1;" ::"r"(a), "r"(v) : "memory"); }
__device__ __forceinline__ void sts16(uint32_t a, uint32_t v) {
  asm volatile("st.shared.u16 [%0], %1;" ::"r"(a), "h"((uint16_t)v) : "memory");
}
__device__ __forceinline__ void sts8(uint32_t a, uint32_t v) {
  asm volatile("st.shared.u8 [%0], %1;" ::"r"(a), "h"((uint16_t)v) : "memory");
}
__device__ __forceinline__ uint2 lds64(uint32_t a) {
  uint2 v;
  asm volatile("ld.shared.v2.b32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
  return v;
}
__device__ __forceinline__ void stsf(uint32_t a, float v) { asm volatile("st.shared.f32 [%0], %1;" ::"r"(a), "f"(v) : "memory"); }
__device__ __forceinline__ void sts128(uint32_t a, uint4 v) {
  asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(a), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void cp16(uint32_t sa, const void* g) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(sa), "l"(g) : "memory");
}
__device__ __forceinline__ void warp_sync() { __syncwarp(); }

// D(16x8, fp32) += A(16x16) * B(16x8), 16-bit operands of the named type
__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t h2_bits(__half2 v) { return *reinterpret_cast<uint32_t*>(&v); }
__device__ __forceinline__ __half2 bits_h2(uint32_t v) { return *reinterpret_cast<__half2*>(&v); }
__device__ __forceinline__ __half2 dup_lo(uint32_t v) { return __half2half2(__low2half(bits_h2(v))); }
__device__ __forceinline__ __half2 dup_hi(uint32_t v) { return __half2half2(__high2half(bits_h2(v))); }

// ---- the lookup table at shared-window address TBL: entry (zc, e) -> half2(u+, u-), one copy per lane for the
// keys' alpha (first 128 bytes of an entry's 256) and for the values' alpha (second 128 bytes).  The idle half
// of an entry carries the fp16 remainder of the active half, pre-scaled by the nominal ratio Bdn / Bup of a row
// in that zero-code bin (anchor at the bin centre); the end bins have codes on one side only and row_constants
// makes their two constants equal.  Called by every thread of the CTA; the caller synchronises afterwards.
// entry idx = (zc << BITS | e) of the table for `alpha`, as the bits of half2(u+, u-)
template <int BITS>
__device__ __forceinline__ uint32_t lookup_entry(float alpha, int idx) {
  constexpr int NE = 1 << BITS, TOP = NE - 1;
  const int zc = idx >> BITS, e = idx & TOP;
  const float lb = log1pf(alpha);
  const float zac = (float)zc / (float)TOP;
  const float ratio = (zc == 0 || zc == TOP) ? 1.0f : zac / (1.0f - zac);
  __half2 ent;
  if (e >= zc) {
    const int up = max(TOP - zc, 1);
    const float u = expm1f((float)min(e - zc, up) / (float)up * lb) / alpha;
    const float uh = __half2float(__float2half_rn(u));
    ent = __floats2half2_rn(uh, (u - uh) / ratio);
  } else {
    const int dn = max(zc, 1);
    const float u = -expm1f((float)(zc - e) / (float)dn * lb) / alpha;
    const float uh = __half2float(__float2half_rn(u));
    ent = __floats2half2_rn((u - uh) * ratio, uh);
  }
  return h2_bits(ent);
}
// stores one entry to the 32 lane copies of its slot half (rotated so that the lanes of a warp, which hold
// consecutive entries, hit different banks)
__device__ __forceinline__ void store_entry_copies(uint32_t row, uint32_t bits) {
#pragma unroll 4
  for (int c = 0; c < 32; ++c) sts32(row + (((c + threadIdx.x) & 31) << 2), bits);
}
template <int BITS>
__device__ __forceinline__ void fill_lookup_table(float alpha_key, float alpha_value) {
  constexpr int NE = 1 << BITS;
  // one table when keys and values use the same alpha (the usual case): each entry is computed once and stored
  // to both halves of its 256-byte slot
  const bool same = alpha_key == alpha_value;
  const int n = same ? NE * NE : 2 * NE * NE;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int which = i / (NE * NE), idx = i % (NE * NE);
    const uint32_t bits = lookup_entry<BITS>(which ? alpha_value : alpha_key, idx);
    store_entry_copies(TBL + idx * 256 + which * 128, bits);
    if (same) store_entry_copies(TBL + idx * 256 + 128, bits);
  }
}
// the same table from a copy in global memory: [2][NE * NE] entries (keys' alpha, values' alpha), built once
// per device and (bits, alphas) by the host side
template <int BITS>
__device__ __forceinline__ void fill_lookup_table_from(const uint32_t* __restrict__ entries) {
  constexpr int NE = 1 << BITS;
  for (int i = threadIdx.x; i < 2 * NE * NE; i += blockDim.x) {
    const int which = i / (NE * NE), idx = i % (NE * NE);
    store_entry_copies(TBL + idx * 256 + which * 128, entries[i]);
  }
}

// ---- per-row constants of the folded dequantizer: value(code e) = A + Bup * u+[zc][e] + Bdn * u-[zc][e].
// A is the value of the zero code: exactly 0 when the row's range straddles zero, up to the rounding of the
// anchor (a few 2^-24 of |lo|), which is dropped.  IEEE division and multiply: the zero code must round exactly
// as the dequantizer's does.
template <int BITS>
__device__ __forceinline__ void row_constants(float lo, float span, int& zc, float& A, float& Bup, float& Bdn) {
  constexpr int TOP = (1 << BITS) - 1;
  float anchor = __fdiv_rn(__fsub_rn(0.0f, lo), fmaxf(span, 1e-8f));
  anchor = fminf(fmaxf(anchor, 0.0f), 1.0f);
  zc = __float2int_rn(__fmul_rn(anchor, (float)TOP));
  A = fmaf(span, anchor, lo);
  if (fabsf(A) <= 9.5367431640625e-7f * fmaxf(fabsf(lo), span)) A = 0.0f;
  Bup = fminf(span * fmaxf(1.0f - anchor, 1e-8f), 65504.f);
  Bdn = fminf(span * fmaxf(anchor, 1e-8f), 65504.f);
  // a row whose zero code is the first / last code has no codes on the other side: that side's constant only
  // ever multiplies the remainder half of the table entries
  if (zc == 0) Bdn = Bup;
  if (zc == TOP) Bup = Bdn;
}
}  // namespace mzm
