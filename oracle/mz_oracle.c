/*
 * Plain-C restatement of the reference's row quantizer / dequantizer with an
 * explicit rounding model.  TEST INFRASTRUCTURE ONLY: nothing in the product
 * links or loads this file; tests use it as a second, torch-free checker and
 * bench.py never times it.
 *
 * Parity status: PINNED — tests/test_oracle_c.py checks it bit for bit against
 * the reference's own outputs in tests/golden/rows_quant.npz / rows_dequant.npz.
 *
 * Follows (paths inside the reference project):
 *   mzo_quantize_rows    muzero/quantizer.py:161-202  (_quantize_rows_torch, _pack_q)
 *   mzo_dequantize_rows  muzero/quantizer.py:229-266  (_dequantize_rows_torch, _unpack_q)
 *
 * Rounding model of the quantizer: the reference evaluates every torch op in
 * the input dtype T, i.e. one IEEE fp32 operation followed by round-to-nearest
 * -even to T (identity when T is fp32); log1p(alpha) alone stays fp32.
 * The dequantizer is all fp32; its expm1 values come from a caller-supplied
 * table (the host's libm/torch), so that its last bit follows the host.
 *
 * Build: see oracle/Makefile (gcc -O2 -ffp-contract=off -shared -fPIC).
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

enum { MZO_F32 = 0, MZO_F16 = 1, MZO_BF16 = 2 };

static uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

static uint16_t f32_to_bf16(float f) {
  uint32_t u = f2u(f);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}
static float bf16_to_f32(uint16_t h) { return u2f(((uint32_t)h) << 16); }

static uint16_t f32_to_f16(float f) {
  uint32_t u = f2u(f), sign = (u >> 16) & 0x8000u, a = u & 0x7fffffffu;
  if (a > 0x7f800000u) return (uint16_t)(sign | 0x7e00u);
  if (a >= 0x47800000u) return (uint16_t)(sign | 0x7c00u);          /* >= 65536 -> inf (65520 handled below) */
  if (a < 0x33000000u) return (uint16_t)sign;                       /* < 2^-25 -> 0 */
  int e = (int)(a >> 23) - 127;
  uint32_t m = (a & 0x7fffffu) | 0x800000u;
  int shift = (e < -14) ? (13 + (-14 - e)) : 13;
  uint32_t half = m >> shift, rem = m & ((1u << shift) - 1u), mid = 1u << (shift - 1);
  if (rem > mid || (rem == mid && (half & 1u))) half++;
  uint32_t out = (e < -14) ? half : (((uint32_t)(e + 15) << 10) + (half - 0x400u));
  return (uint16_t)(sign | out);                                    /* carry into exponent / inf is natural */
}
static float f16_to_f32(uint16_t h) {
  uint32_t sign = ((uint32_t)h & 0x8000u) << 16, e = (h >> 10) & 0x1fu, m = h & 0x3ffu;
  if (e == 0) {
    if (m == 0) return u2f(sign);
    float v = (float)m * 5.9604644775390625e-8f;                    /* 2^-24 */
    return sign ? -v : v;
  }
  if (e == 31) return u2f(sign | 0x7f800000u | (m << 13));
  return u2f(sign | ((e + 112u) << 23) | (m << 13));
}

static float rnd(int dt, float v) {
  if (dt == MZO_BF16) return bf16_to_f32(f32_to_bf16(v));
  if (dt == MZO_F16) return f16_to_f32(f32_to_f16(v));
  return v;
}
static float load_elem(const void* p, long long i, int dt) {
  if (dt == MZO_BF16) return bf16_to_f32(((const uint16_t*)p)[i]);
  if (dt == MZO_F16) return f16_to_f32(((const uint16_t*)p)[i]);
  return ((const float*)p)[i];
}
static void store_elem(void* p, long long i, int dt, float v) {
  if (dt == MZO_BF16) ((uint16_t*)p)[i] = f32_to_bf16(v);
  else if (dt == MZO_F16) ((uint16_t*)p)[i] = f32_to_f16(v);
  else ((float*)p)[i] = v;
}
static float clamp01(float v) { return v != v ? v : (v < 0.f ? 0.f : (v > 1.f ? 1.f : v)); }
static float maxf_(float a, float b) { return a != a ? a : (a > b ? a : b); }

int mzo_row_bytes(int group, int bits) { return (group * bits + 7) / 8; }

/* x[n_rows*group] of dtype dt -> packed[n_rows*qb], mn/scale[n_rows] of dtype meta_dt */
int mzo_quantize_rows(const void* x, int dt, long long n_rows, int group, int bits, float alpha, float eps,
                      uint8_t* packed, void* mn_out, void* scale_out, int meta_dt) {
  if (bits < 1 || bits > 8 || group <= 0) return 1;
  const float top = (float)((1 << bits) - 1);
  const float lb = (float)log1p((double)alpha);      /* fp32 scalar, never rounded to T */
  const float eps_t = rnd(dt, eps);
  const int qb = mzo_row_bytes(group, bits);
  for (long long r = 0; r < n_rows; ++r) {
    float lo = INFINITY, hi = -INFINITY;
    for (int i = 0; i < group; ++i) {
      float v = load_elem(x, r * group + i, dt);
      if (v < lo) lo = v;
      if (v > hi) hi = v;
    }
    const float span = maxf_(rnd(dt, hi - lo), eps_t);
    const float anchor = clamp01(rnd(dt, rnd(dt, 0.0f - lo) / span));
    const float zc = rintf(rnd(dt, anchor * top));
    const float up = maxf_(rnd(dt, top - zc), 1.0f), dn = maxf_(zc, 1.0f);
    const float room_up = maxf_(rnd(dt, 1.0f - anchor), eps_t), room_dn = maxf_(anchor, eps_t);
    uint8_t* row = packed + r * qb;
    memset(row, 0, (size_t)qb);
    for (int i = 0; i < group; ++i) {
      const float v = load_elem(x, r * group + i, dt);
      const float unit = clamp01(rnd(dt, rnd(dt, v - lo) / span));
      float q;
      if (unit >= anchor) {
        const float p = clamp01(rnd(dt, rnd(dt, unit - anchor) / room_up));
        const float c = rnd(dt, rnd(dt, (float)log1p((double)rnd(dt, alpha * p))) / lb);
        q = rnd(dt, zc + rintf(rnd(dt, c * up)));
      } else {
        const float p = clamp01(rnd(dt, rnd(dt, anchor - unit) / room_dn));
        const float c = rnd(dt, rnd(dt, (float)log1p((double)rnd(dt, alpha * p))) / lb);
        q = rnd(dt, zc - rintf(rnd(dt, c * dn)));
      }
      if (!(q > 0.f)) q = 0.f;
      if (q > top) q = top;
      const unsigned code = (unsigned)q;
      const int bit = i * bits;
      row[bit >> 3] |= (uint8_t)(code << (bit & 7));
      if ((bit & 7) + bits > 8) row[(bit >> 3) + 1] |= (uint8_t)(code >> (8 - (bit & 7)));
    }
    store_elem(mn_out, r, meta_dt, lo);
    store_elem(scale_out, r, meta_dt, span);
  }
  return 0;
}

/* table[(2^bits)*(2^bits)]: expm1(clamp(numer/denom)*log1p(alpha))/alpha, row = denom */
int mzo_dequantize_rows(const uint8_t* packed, const void* mn, const void* scale, int meta_dt, long long n_rows,
                        int group, int bits, float eps, const float* table, void* out, int out_dt) {
  if (bits < 1 || bits > 8 || group <= 0) return 1;
  const int tw = 1 << bits, topi = tw - 1, qb = mzo_row_bytes(group, bits);
  for (long long r = 0; r < n_rows; ++r) {
    const float lo = load_elem(mn, r, meta_dt), span = load_elem(scale, r, meta_dt);
    const float anchor = clamp01((0.0f - lo) / span);
    const int zc = (int)rintf(anchor * (float)topi);
    const int up = topi - zc > 1 ? topi - zc : 1, dn = zc > 1 ? zc : 1;
    const float room_up = maxf_(1.0f - anchor, eps), room_dn = maxf_(anchor, eps);
    const uint8_t* row = packed + r * qb;
    for (int i = 0; i < group; ++i) {
      const int bit = i * bits;
      unsigned w = row[bit >> 3];
      if ((bit >> 3) + 1 < qb) w |= ((unsigned)row[(bit >> 3) + 1]) << 8;
      const int q = (int)((w >> (bit & 7)) & (unsigned)topi);
      float unit;
      if (q >= zc) {
        const float t = room_up * table[up * tw + (q - zc > up ? up : q - zc)];
        unit = anchor + t;
      } else {
        const float t = room_dn * table[dn * tw + (zc - q > dn ? dn : zc - q)];
        unit = anchor - t;
      }
      unit = clamp01(unit);
      const float scaled = unit * span;
      store_elem(out, r * group + i, out_dt, scaled + lo);
    }
  }
  return 0;
}
