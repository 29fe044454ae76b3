// Building blocks of the tiled decode-attention kernel (head_dim 128).
#pragma once
#include "mz_decode.cuh"

namespace mzt {

constexpr int D = 128;
constexpr float LOG2E = 1.4426950408889634f;

template <int BITS, int G, int GQA>
struct Cfg {
  static constexpr int NE = 1 << BITS;             // codebook entries
  static constexpr int QB = G * BITS / 8;          // packed bytes of one row of G codes
  static constexpr int LPR = G / 8;                // lanes that share one key row (8 tokens each)
  static constexpr int RPS = 32 / LPR;             // key rows a warp covers per step
  static constexpr int NG = D / G;                 // value groups per token
  static constexpr int TILE_BYTES = D * QB;        // packed bytes of a key tile == of a value tile
  static constexpr bool BOOKS = BITS <= 4;         // per-row codebooks; wider codes are expanded arithmetically
  static constexpr int BOOK_STRIDE = !BOOKS ? 8 : NE;   // floats per row
  static constexpr int STEPS = D / RPS;            // steps per tile side (keys: 128 rows / RPS; values: G/2 token pairs)
  // expansion rows are stored [row % RPS][row / RPS][BOOK_STRIDE]: the rows one lane visits are
  // contiguous, so a lookup address is lane_base + step*ROW_BYTES + code*4
  static constexpr int ROW_BYTES = BOOK_STRIDE * 4;
  static constexpr int LANE_BLOCK_BYTES = STEPS * ROW_BYTES;
  static constexpr int UNROLL = 4;
  // with 4-bit codes and 256-byte aligned bases the address of a lookup is one byte permute
  static constexpr bool PRMT_ADDR = BITS == 4 && (LANE_BLOCK_BYTES % 256 == 0) && ((UNROLL * ROW_BYTES) % 256 == 0);
  static constexpr int ROUNDS = (GQA + RPS - 1) / RPS;  // softmax rounds: a lane owns head r*RPS+dl in round r
  static constexpr int META_BYTES = 1024;          // 2 x 128 entries x up to 4 bytes
  // per-warp shared memory, in bytes (every region 16-byte aligned)
  static constexpr int KBUF = TILE_BYTES + META_BYTES;
  static constexpr int VBUF = TILE_BYTES + META_BYTES;
  static constexpr int BOOK_BYTES = D * BOOK_STRIDE * 4;
  static constexpr int PDUP = G * GQA * 8;
  static constexpr int QDUP = D * GQA * 8;
  static constexpr int MISC = 64;
  static constexpr int PER_WARP = ((KBUF + VBUF + BOOK_BYTES + PDUP + QDUP + MISC + 255) / 256) * 256;
  // per-CTA shared: two universal tables [NE][NE+1] float2 (keys, values)
  static constexpr int UNIV_FLOAT2 = BOOKS ? NE * (NE + 1) : 0;
  static constexpr int SHARED = ((2 * UNIV_FLOAT2 * 8 + 255) / 256) * 256 + 256;   // + slack to align the base to 256
};

// ---- asynchronous copies (global -> shared, 16 bytes per lane per call) ----
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  const unsigned sa = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(sa), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

// warp-cooperative copy of `bytes` (multiple of 16) contiguous bytes
__device__ __forceinline__ void warp_copy_async(uint8_t* dst, const uint8_t* src, int bytes, int lane) {
  for (int off = lane * 16; off < bytes; off += 512) cp_async16(dst + off, src + off);
}

// ---- packed fp32 pairs: d += a * b on both halves (one issue slot on sm_100) ----
__device__ __forceinline__ void ffma2(float2& d, const float2 a, const float2 b) {
#if defined(MZ_NO_F32X2)
  d.x = fmaf(a.x, b.x, d.x);
  d.y = fmaf(a.y, b.y, d.y);
#else
  unsigned long long dd = *reinterpret_cast<unsigned long long*>(&d);
  const unsigned long long aa = *reinterpret_cast<const unsigned long long*>(&a);
  const unsigned long long bb = *reinterpret_cast<const unsigned long long*>(&b);
  asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(dd) : "l"(aa), "l"(bb));
  d = *reinterpret_cast<float2*>(&dd);
#endif
}

__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// metadata element `i` of a staged array (runtime storage type)
__device__ __forceinline__ float meta_at(const uint8_t* base, int i, int dt) {
  if (dt == MZ_F32) return ((const float*)base)[i];
  return mz_u16_to_float(((const uint16_t*)base)[i], dt);
}

// the BITS bytes that hold 8 consecutive codes, from shared memory
template <int BITS>
__device__ __forceinline__ unsigned long long load_octet(const uint8_t* p) {
  if (BITS == 4) return *(const uint32_t*)p;
  if (BITS == 8) return *(const unsigned long long*)p;
  if (BITS == 2) return *(const uint16_t*)p;
  if (BITS == 1) return *p;
  if (BITS == 6) {
    const uint16_t* q = (const uint16_t*)p;
    return (unsigned long long)q[0] | ((unsigned long long)q[1] << 16) | ((unsigned long long)q[2] << 32);
  }
  unsigned long long v = 0;
#pragma unroll
  for (int i = 0; i < BITS; ++i) v |= ((unsigned long long)p[i]) << (8 * i);
  return v;
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
  return d;
}
template <int IMM>
__device__ __forceinline__ float lds_f32(uint32_t addr) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1+%2];" : "=f"(v) : "r"(addr), "n"(IMM));
  return v;
}
template <int IMM>
__device__ __forceinline__ float4 lds_f32x4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4+%5];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr), "n"(IMM));
  return v;
}

// 8 codes -> 8 values.  `rb` is the shared-window address of the lane's expansion rows for the
// current unrolled block (aligned to 64 bytes, to 256 when PRMT is set); IMM selects the row.
// BOOKS: the row is a codebook.  Otherwise it holds {A, Bup, Bdn, kup, kdn, zero_code, -, -}:
// value = A + Bup*(2^(n*kup)-1) above the zero code, A - Bdn*(2^(n*kdn)-1) below it.
template <int BITS, bool BOOKS, bool PRMT, int IMM>
__device__ __forceinline__ void expand8(unsigned long long codes, uint32_t rb, float (&v)[8]) {
  constexpr unsigned MASK = (1u << BITS) - 1u;
  if (BOOKS) {
    const uint32_t c32 = (uint32_t)codes;   // BITS <= 4: all 8 codes fit 32 bits
    if (PRMT) {
      const uint32_t even = (c32 << 2) & 0x3C3C3C3Cu;   // byte j = 4 * code(2j)
      const uint32_t odd = (c32 >> 2) & 0x3C3C3C3Cu;    // byte j = 4 * code(2j+1)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        v[2 * j] = lds_f32<IMM>(prmt(even, rb, 0x7650u + j));
        v[2 * j + 1] = lds_f32<IMM>(prmt(odd, rb, 0x7650u + j));
      }
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const int sh = BITS * k - 2;
        const uint32_t off = sh >= 0 ? ((c32 >> (sh >= 0 ? sh : 0)) & (MASK << 2)) : ((c32 << (sh < 0 ? -sh : 0)) & (MASK << 2));
        v[k] = lds_f32<IMM>(rb | off);
      }
    }
  } else {
    const float4 a = lds_f32x4<IMM>(rb);
    const float4 b = lds_f32x4<IMM + 16>(rb);
    const int zc = __float_as_int(b.y);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int c = (int)((codes >> (BITS * k)) & MASK);
      const int n = c - zc;
      const float e = n >= 0 ? ex2f((float)n * a.w) : ex2f((float)(-n) * b.x);
      v[k] = n >= 0 ? fmaf(a.y, e - 1.0f, a.x) : fmaf(-a.z, e - 1.0f, a.x);
    }
  }
}

// raw 16-bit pair -> two floats
__device__ __forceinline__ float2 unpack2(uint32_t w, int dt) {
  if (dt == MZ_BF16) return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
  return __half22float2(*reinterpret_cast<const __half2*>(&w));
}

}  // namespace mzt
