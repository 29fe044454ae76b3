// Building blocks of the tiled decode-attention kernel (head_dim 128).
#pragma once
#include "mz_decode.cuh"

namespace mzt {

constexpr int D = 128;
constexpr float LOG2E = 1.4426950408889634f;

// Lane mappings (one warp per tile of G tokens):
//   keys   : 16 lanes share a row (one channel, G tokens), each lane owns TPL = G/16 consecutive
//            tokens; the two half-warps take rows 2*step and 2*step+1            -> 64 steps
//   values : 16 lanes share a token, each lane owns TPL consecutive channels of every group; the
//            two half-warps take tokens 2*step and 2*step+1                      -> G/2 steps
// so one shared-memory lookup instruction touches two codebooks: with 16-entry books they cover
// the 32 banks exactly once, no conflicts.
template <int BITS, int G, int GQA>
struct Cfg {
  static constexpr int NE = 1 << BITS;             // codebook entries
  static constexpr int QB = G * BITS / 8;          // packed bytes of one row of G codes
  static constexpr int TPL = G / 16;               // tokens per lane per key row
  static constexpr int NG = D / G;                 // value groups per token
  static constexpr int VROW_BYTES = 16 * BITS;     // packed bytes of one token's 128 value codes
  static constexpr int TILE_BYTES = D * QB;        // packed bytes of a key tile == of a value tile
  // staging buffer of one side; a residual tile is DT un-quantized tokens (256 bytes each) in the same buffer
  static constexpr int STAGE_BYTES = TILE_BYTES > 4096 ? TILE_BYTES : 4096;
  static constexpr int DT = STAGE_BYTES / (2 * D);
  static constexpr bool BOOKS = BITS <= 4;         // per-row codebooks; wider codes are expanded arithmetically
  static constexpr int BOOK_STRIDE = !BOOKS ? 8 : (NE < 4 ? 4 : NE);   // floats per row
  static constexpr int ROW_BYTES = BOOK_STRIDE * 4;
  static constexpr int KSTEPS = D / 2;             // key steps per tile
  static constexpr int UNROLL = 4;
  // warps per CTA the kernel is compiled for: 8 heads per kv head hold twice the accumulators, and get
  // the registers of a 256-thread block
  static constexpr int MAX_WARPS = GQA > 4 ? 8 : 12;
  static constexpr int ROUNDS = (GQA + 1) / 2;     // softmax rounds: half-warp dl owns head 2*r + dl in round r
  static constexpr int META_BYTES = 1024;          // 2 x 128 entries x up to 4 bytes
  // 4-bit codes, 256-byte aligned lane blocks: the address of a lookup is one byte permute
  static constexpr bool PRMT_ADDR = BITS == 4;
  // the expansion rows of a tile side are built and used in PASSES parts, so they never take more than 4 KB
  static constexpr int PASSES = D * ROW_BYTES > 4096 ? 2 : 1;
  static constexpr int RP = D / PASSES;            // rows per pass
  static constexpr int TP = G / PASSES;            // value tokens per pass
  // per-warp shared memory, in bytes
  static constexpr int BOOK_BYTES = RP * ROW_BYTES;
  static constexpr int KBUF = STAGE_BYTES + META_BYTES;
  static constexpr int VBUF = STAGE_BYTES + META_BYTES;
  static constexpr int PBUF = G * GQA * 4;         // probabilities [token][head]; also dense-key logits
  static constexpr int QBUF = D * GQA * 4;         // scaled query [channel][head]
  static constexpr int MISC = 64;
  static constexpr int PER_WARP = ((BOOK_BYTES + KBUF + VBUF + PBUF + QBUF + MISC + 255) / 256) * 256;
  // per-CTA shared: two shape tables (keys, values) [zero code][entry] of floats, rows padded by 4 floats
  // so that the 16-byte reads of rows with different zero codes fall into different bank groups;
  // + slack to align to 256
  static constexpr int UROW = NE >= 4 ? NE + 4 : NE;
  static constexpr int UNIV_FLOATS = BOOKS ? NE * UROW : 0;
  static constexpr int SHARED = ((2 * UNIV_FLOATS * 4 + 255) / 256) * 256 + 256;
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

// packed fp32 pair: d += a * b on both halves (one issue slot on sm_100)
__device__ __forceinline__ void ffma2(float2& d, const float2 a, const float2 b) {
  unsigned long long dd = *reinterpret_cast<unsigned long long*>(&d);
  const unsigned long long aa = *reinterpret_cast<const unsigned long long*>(&a);
  const unsigned long long bb = *reinterpret_cast<const unsigned long long*>(&b);
  asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(dd) : "l"(aa), "l"(bb));
  d = *reinterpret_cast<float2*>(&dd);
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

// N consecutive codes of BITS bits starting at code index `first` of the packed row at `row`
// (shared memory, 4-byte aligned); returned LSB-first in up to 64 bits.
template <int BITS, int N>
__device__ __forceinline__ unsigned long long load_codes(const uint8_t* row, int first) {
  constexpr int NB = BITS * N;                      // bits wanted
  if (NB == 8) return row[first * BITS >> 3];
  if (NB == 16) return *(const uint16_t*)(row + (first * BITS >> 3));
  if (NB == 32) return *(const uint32_t*)(row + (first * BITS >> 3));
  if (NB == 64) return *(const unsigned long long*)(row + (first * BITS >> 3));
  const int bit = first * BITS;
  const uint32_t* w = (const uint32_t*)row + (bit >> 5);
  const int sh = bit & 31;
  if (NB <= 32) {
    const uint32_t lo = w[0], hi = (sh + NB > 32) ? w[1] : 0u;
    return __funnelshift_r(lo, hi, sh) & (NB == 32 ? 0xffffffffu : ((1u << (NB & 31)) - 1u));
  }
  const unsigned long long a = (unsigned long long)w[0] | ((unsigned long long)w[1] << 32);
  const unsigned long long b = (sh + NB > 64) ? (unsigned long long)w[2] : 0ull;
  unsigned long long v = a >> sh;
  if (sh) v |= b << (64 - sh);
  return NB == 64 ? v : (v & ((1ull << (NB & 63)) - 1ull));
}

// N codes -> N values.  `rb` is the shared-window address of the expansion rows of the current
// unrolled block (256-byte aligned), `lane_off` (< 256, multiple of ROW_BYTES) the byte offset of
// this lane's row inside a step, IMM the byte offset of the step.
// BOOKS: the row is a codebook.  Otherwise it holds {A, Bup, Bdn, kup, kdn, zero_code, -, -}:
// value = A + Bup*(2^(n*kup)-1) above the zero code, A - Bdn*(2^(n*kdn)-1) below it.
template <int BITS, bool BOOKS, bool PRMT, int N, int IMM>
__device__ __forceinline__ void expand(unsigned long long codes, uint32_t rb, uint32_t lane_off, float (&v)[N]) {
  constexpr unsigned MASK = (1u << BITS) - 1u;
  if (BOOKS) {
    const uint32_t c32 = (uint32_t)codes;   // BITS <= 4, N <= 8: all codes fit 32 bits
    if (PRMT && (N % 2 == 0)) {
      const uint32_t lo4 = lane_off * 0x01010101u;      // lane_off in every byte
      const uint32_t even = ((c32 << 2) & 0x3C3C3C3Cu) | lo4;   // byte j = 4 * code(2j) + lane_off
      const uint32_t odd = ((c32 >> 2) & 0x3C3C3C3Cu) | lo4;    // byte j = 4 * code(2j+1) + lane_off
#pragma unroll
      for (int j = 0; j < N / 2; ++j) {
        v[2 * j] = lds_f32<IMM>(prmt(even, rb, 0x7650u + j));
        v[2 * j + 1] = lds_f32<IMM>(prmt(odd, rb, 0x7650u + j));
      }
    } else {
#pragma unroll
      for (int k = 0; k < N; ++k) {
        const int sh = BITS * k - 2;
        const uint32_t off = sh >= 0 ? ((c32 >> (sh >= 0 ? sh : 0)) & (MASK << 2)) : ((c32 << (sh < 0 ? -sh : 0)) & (MASK << 2));
        v[k] = lds_f32<IMM>((rb + lane_off) | off);
      }
    }
  } else {
    const float4 a = lds_f32x4<IMM>(rb + lane_off);
    const float4 b = lds_f32x4<IMM + 16>(rb + lane_off);
    const int zc = __float_as_int(b.y);
#pragma unroll
    for (int k = 0; k < N; ++k) {
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
