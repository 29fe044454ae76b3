// Device arithmetic of the zero-anchored log compander (quantizer side).
//
// The rounding model: every operation of the reference's torch backend is one
// IEEE fp32 operation followed by a round-to-nearest-even to the input dtype
// T (identity for fp32); log1p(alpha) stays fp32.  For 16-bit T the chain
// p -> round_T(round_T(log1p(round_T(alpha*p))) / log1p(alpha)) has one value
// per p in [0,1], so it is a table lookup (built once per device on the host).
#pragma once
#include "mz_common.cuh"

template <int DT>
struct MzQuantRow {
  float lo, span, anchor, zero_code, steps_up, steps_dn, room_up, room_dn;
  float inv_span, inv_up, inv_dn;   // correctly rounded reciprocals of the three per-row divisors
  bool row_nan;                     // the zero anchor is NaN (0/0 range): every code of the row is 0
  float alpha, log_base, top;
  const uint16_t* __restrict__ ctab;
  int ctab_n;

  using TT = MzType<DT>;

  __device__ __forceinline__ void setup(float mn, float mx, int bits, float alpha_, float eps, const uint16_t* tab, int tab_n) {
    alpha = alpha_;
    ctab = tab;
    ctab_n = tab_n;
    top = (float)((1 << bits) - 1);
    log_base = (float)log1p((double)alpha_);
    const float eps_t = TT::round(eps);
    lo = mn;
    span = fmaxf(TT::round(__fsub_rn(mx, mn)), eps_t);
    float a = TT::round(__fdiv_rn(TT::round(__fsub_rn(0.0f, mn)), span));
    anchor = fminf(fmaxf(a, 0.0f), 1.0f);
    if (a != a) anchor = a;  // torch.clamp keeps NaN
    zero_code = rintf(TT::round(__fmul_rn(anchor, top)));
    steps_up = fmaxf(TT::round(__fsub_rn(top, zero_code)), 1.0f);
    steps_dn = fmaxf(zero_code, 1.0f);
    room_up = fmaxf(TT::round(__fsub_rn(1.0f, anchor)), eps_t);
    room_dn = fmaxf(anchor, eps_t);
    inv_span = __frcp_rn(span);
    inv_up = __frcp_rn(room_up);
    inv_dn = __frcp_rn(room_dn);
    row_nan = anchor != anchor;
  }

  // round_T(num / den) for a per-row divisor `den` with inv = RN(1/den).  bf16: num*inv is within 1.5
  // fp32 ulps of the correctly rounded fp32 quotient, and the two round to the same bf16 value unless a
  // bf16 rounding boundary (low half-word 0x8000) lies that close; only then the IEEE division is
  // done.  Other types take the division.
  __device__ __forceinline__ float quotient(float num, float den, float inv) const {
    if (DT == MZ_BF16) {
      const float y = __fmul_rn(num, inv);
      const uint32_t low = __float_as_uint(y) & 0xffffu;
      if (low - 0x7ffcu > 8u) return TT::round(y);
    }
    return TT::round(__fdiv_rn(num, den));
  }

  // round_T(round_T(log1p(round_T(alpha*p))) / log_base) for p in [0,1]
  __device__ __forceinline__ float compand(float p) const {
    if (DT == MZ_F32) {
      const float ap = __fmul_rn(alpha, p);
      return __fdiv_rn((float)log1p((double)ap), log_base);
    } else {
      uint32_t idx;
      if (DT == MZ_BF16) idx = __float_as_uint(p) >> 16;
      else idx = (uint32_t)__half_as_ushort(__float2half_rn(p));
      idx = min(idx, (uint32_t)(ctab_n - 1));
      return mz_u16_to_float(ctab[idx], DT);
    }
  }

  __device__ __forceinline__ int code(float x) const {
    // NaN (0/0 when the row range or a side extent rounds to zero in T) propagates through the
    // reference's chain and its final cast to uint8 yields 0; mirror that outcome.
    float unit = quotient(TT::round(__fsub_rn(x, lo)), span, inv_span);
    if (unit != unit || row_nan) return 0;
    unit = fminf(fmaxf(unit, 0.0f), 1.0f);
    // one path for both sides of the zero anchor (lanes of a warp straddle it): round(a-b) == -round(b-a)
    const bool up = unit >= anchor;
    const float num = fabsf(TT::round(__fsub_rn(unit, anchor)));
    float p = quotient(num, up ? room_up : room_dn, up ? inv_up : inv_dn);
    if (p != p) return 0;
    p = fminf(fmaxf(p, 0.0f), 1.0f);
    // round-half-even of a value in [0, 255] by adding and removing 1.5 * 2^23 (keeps the conversion pipe free)
    constexpr float kMagic = 12582912.0f;
    const float rr = __fsub_rn(__fadd_rn(TT::round(__fmul_rn(compand(p), up ? steps_up : steps_dn)), kMagic), kMagic);
    // zero_code +- rr: integers; where rounding to T would change them (beyond 256) the clamp below decides anyway
    float q = up ? __fadd_rn(zero_code, rr) : __fsub_rn(zero_code, rr);
    q = fminf(fmaxf(q, 0.0f), top);
    return __float_as_int(__fadd_rn(q, kMagic)) & 0x1ff;
  }
};

// writes the `bits` bytes holding 8 consecutive codes (codes64 = sum code_k << k*bits)
__device__ __forceinline__ void mz_store_octet(uint8_t* dst, unsigned long long codes64, int bits) {
  const unsigned mis = (unsigned)(uintptr_t)dst & (unsigned)(bits - 1);  // bits 2/4/8: natural alignment
  if (mis != 0 && (bits == 2 || bits == 4 || bits == 8)) {
    for (int i = 0; i < bits; ++i) dst[i] = (uint8_t)(codes64 >> (8 * i));
  } else if (bits == 4) {
    *(uint32_t*)dst = (uint32_t)codes64;
  } else if (bits == 8) {
    *(unsigned long long*)dst = codes64;
  } else if (bits == 2) {
    *(uint16_t*)dst = (uint16_t)codes64;
  } else {
    for (int i = 0; i < bits; ++i) dst[i] = (uint8_t)(codes64 >> (8 * i));
  }
}

// reads the `bits` bytes holding 8 consecutive codes
__device__ __forceinline__ unsigned long long mz_load_octet(const uint8_t* src, int bits) {
  if (bits == 4) return *(const uint32_t*)src;
  if (bits == 8) return *(const unsigned long long*)src;
  if (bits == 2) return *(const uint16_t*)src;
  unsigned long long v = 0;
  for (int i = 0; i < bits; ++i) v |= ((unsigned long long)src[i]) << (8 * i);
  return v;
}
