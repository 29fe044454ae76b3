// Tensor-core decode attention for head_dim 128, group 64, 2- and 4-bit codes, 1/2/4 query heads
// per kv head (sm_100a).
//
// The dequantized value of code e in a row with metadata (lo, span) is
//     A + Bup * u+[zc][e] + Bdn * u-[zc][e]
// where zc is the row's zero code, A / Bup / Bdn are per-row constants and u+ / u- are the positive
// and negative part of ONE normalised table that depends on (zc, e) only.  Key rows run along the
// tokens and value rows along the channels, i.e. always along the dimension a contraction does NOT
// reduce over, so the per-row constants can be folded into the other operand:
//     logit[h,t]  = sum_d  (q[h,d]*Bup_d) u+  +  (q[h,d]*Bdn_d) u-   + sum_d q[h,d] A_d
//     out[h,c]    = sum_t  (p[h,t]*Bup_tg) u+ +  (p[h,t]*Bdn_tg) u-  + sum_t p[h,t] A_tg
// Both contractions run on the tensor cores (mma.sync m16n8k16, fp16 operands, fp32 accumulate):
//   * the A operand holds table values; one code = one 32-bit shared-memory lookup that returns the
//     fp16 pair (u+, u-), which is one A-fragment register (the reduction index is doubled: one slot for
//     the part above the zero code, one for the part below it)
//   * the table is replicated once per lane (entry stride 256 bytes: 32 lanes x 4 bytes for the key
//     table, the same for the value table), so no lookup pattern can cause a bank conflict, and it sits
//     at shared-window address 65536, so that the address of a lookup is one byte permute:
//     byte 1 of the address <- (zc << BITS | e)
//   * the B operand holds the folded query (keys) or folded probabilities (values); its 8 columns are
//     4 heads x {product rounded to fp16, its exact fp16 remainder (+ the remainder of the probability)}
//   * the idle half of a table entry (u- of a code above the zero code, u+ of one below) carries the fp16
//     remainder of the active half, pre-scaled by the nominal ratio of the two side constants of the
//     zero-code bin, which recovers most of the table's own fp16 rounding
//   * M rows are tokens (keys) or channels (values), permuted so that one 32-bit load of packed codes
//     feeds a thread's rows of four M tiles.
// Residual (un-quantized) tiles of 16 tokens run through the same tensor-core path with the cache's own
// 16-bit type.  Work decomposition, staging (cp.async into per-warp buffers), online softmax per warp
// and the partial records are those of the SIMT tiled kernel; the records are merged by
// combine_tiles_kernel.
#include <mutex>

#include "mz_mma_common.cuh"

namespace mzm {
constexpr int DT = 16;                      // tokens per residual tile
constexpr int DENSE_STRIDE = 2 * D + 16;    // padded row of a staged residual tile (bank spread)
constexpr int DENSE_BYTES = DT * DENSE_STRIDE;
constexpr int Z_BYTES = 128;                // zero codes of one tile side: [t][32 rows of lane class t], one byte each
constexpr int RI_BYTES = Z_BYTES + 512;     // + fold constants: 64 x {half2(Bup, Bdn) of slot 0, of slot 1}
constexpr int A_BYTES = 512;                // per-row constant A (fp32) of one tile side
constexpr int PBUF_BYTES = 1024;            // folded-probability source: [8 k-blocks][32 lanes] half2
constexpr int DBUF_BYTES = 256;             // residual-tile probabilities [16 tokens][4 heads] fp32; shares the value side's A array
constexpr int MAX_WARPS = 12;


// ---- lookup machinery.  A thread (g = lane / 4, t = lane % 4) holds the codes of two rows (the two
// halves of the reduction block: slot 0 and slot 1) for eight consecutive positions 8g .. 8g+7 along
// the row; position 8g + 2m + r belongs to M tile m, fragment row g + 8r.
template <int BITS>
struct Codes {
  uint32_t r[4];   // bytes hold (zc << BITS | code)
};
// 4-bit: w0 / w1 are the 32-bit code words of slot 0 / 1, z0 / z1 hold (zc << 4) in every byte
template <int BITS>
__device__ __forceinline__ Codes<BITS> spread_codes(uint32_t w0, uint32_t w1, uint32_t z0, uint32_t z1);
template <>
__device__ __forceinline__ Codes<4> spread_codes<4>(uint32_t w0, uint32_t w1, uint32_t z0, uint32_t z1) {
  Codes<4> c;
  c.r[0] = (w0 & 0x0F0F0F0Fu) | z0;          // slot 0, even positions (fragment row g), byte = M tile
  c.r[1] = ((w0 >> 4) & 0x0F0F0F0Fu) | z0;   // slot 0, odd positions (fragment row g + 8)
  c.r[2] = (w1 & 0x0F0F0F0Fu) | z1;
  c.r[3] = ((w1 >> 4) & 0x0F0F0F0Fu) | z1;
  return c;
}
// 2-bit: w0 / w1 are 16-bit code half-words; z0 holds (zc0 << 2) in bytes 0-1 and (zc1 << 2) in bytes 2-3
template <>
__device__ __forceinline__ Codes<2> spread_codes<2>(uint32_t w0, uint32_t w1, uint32_t z0, uint32_t) {
  const uint32_t w = prmt(w0, w1, 0x5410u);
  Codes<2> c;
#pragma unroll
  for (int k = 0; k < 4; ++k) c.r[k] = ((w >> (2 * k)) & 0x03030303u) | z0;   // byte 2*slot + (i >> 2) of r[i & 3] = position i
  return c;
}
// the table address of (slot, M tile m, fragment-row half r)
template <int BITS>
__device__ __forceinline__ uint32_t lookup(const Codes<BITS>& c, uint32_t lane_base, int slot, int m, int r) {
  if (BITS == 4) return lds32(prmt(c.r[2 * slot + r], lane_base, 0x7604u | (uint32_t)(m << 4)));
  const int i = 2 * m + r;
  return lds32(prmt(c.r[i & 3], lane_base, 0x7604u | (uint32_t)((2 * slot + (i >> 2)) << 4)));
}
// the 16 table values of one reduction block (four M tiles x four fragment registers)
template <int BITS>
__device__ __forceinline__ void lookups16(const Codes<BITS>& c, uint32_t lane_base, uint32_t (&a)[16]) {
#pragma unroll
  for (int m = 0; m < 4; ++m) {
    a[4 * m + 0] = lookup<BITS>(c, lane_base, 0, m, 0);
    a[4 * m + 1] = lookup<BITS>(c, lane_base, 0, m, 1);
    a[4 * m + 2] = lookup<BITS>(c, lane_base, 1, m, 0);
    a[4 * m + 3] = lookup<BITS>(c, lane_base, 1, m, 1);
  }
}
// four M tiles of one reduction block: acc[m] += a[m] x b
__device__ __forceinline__ void mma4(float (*acc)[4], const uint32_t (&a)[16], uint32_t b0, uint32_t b1) {
#pragma unroll
  for (int m = 0; m < 4; ++m) mma_f16(acc[m], a[4 * m], a[4 * m + 1], a[4 * m + 2], a[4 * m + 3], b0, b1);
}
// The zero codes of a lane's rows sit in registers, one byte (zc << BITS) per row; bytes b0 and b0 + 1 of
// `zreg` belong to slot 0 and slot 1 of a block.  Returns them in the form spread_codes wants.
template <int BITS>
__device__ __forceinline__ void zero_words(uint32_t zreg, int b0, uint32_t& z0, uint32_t& z1) {
  if (BITS == 4) {
    z0 = prmt(zreg, 0u, (uint32_t)b0 * 0x1111u);
    z1 = prmt(zreg, 0u, (uint32_t)(b0 + 1) * 0x1111u);
  } else {
    z0 = prmt(zreg, 0u, (uint32_t)(b0 * 0x0011 + (b0 + 1) * 0x1100));
    z1 = 0u;
  }
}

// One B-operand register of a lane: x * B for the pair B = (Bup, Bdn).  mask = 0 (even column): the fp16
// product; mask = all ones (odd column): what that rounding dropped, exactly.
__device__ __forceinline__ uint32_t fold_pair(__half2 x, uint32_t B, uint32_t mask) {
  const uint32_t h = h2_bits(__hmul2(x, bits_h2(B))) & mask;
  return h2_bits(__hfma2(x, bits_h2(B), __hneg2(bits_h2(h))));
}

// swizzle of the folded-probability buffer: word (j, t', g') lives at j*32 + ((8t' + g') ^ pswz(j)), which
// spreads both the softmax lanes' stores (j = their g) and the fold's loads over all banks
__host__ __device__ constexpr int pswz(int j) { return (j & 1) | (((j >> 1) & 3) << 3); }

struct Layout {
  uint32_t kbuf, vbuf, riK, riV, aK, aV, pbuf, dbuf;
};

template <int BITS, int GQA>
__global__ void __launch_bounds__(MAX_WARPS * 32, 1) decode_mma_kernel(const MzDecodeParams p) {
  constexpr int NE = 1 << BITS, TOP = NE - 1;
  constexpr int QB = G * BITS / 8;            // bytes of one packed row of 64 codes
  constexpr int CODE_BYTES = D * QB;          // one tile side
  constexpr int VROW = 16 * BITS;             // bytes of one token's 128 value codes
  extern __shared__ __align__(128) uint8_t smem[];
  const mz_kv_store& s = p.s;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  // tiles 0 .. kt-1 of a pair are packed groups, the rest residual tiles; a plan without packed tiles (the
  // residual-only companion launch of the tcgen05 kernel) needs no table
  // one launch may carry two plans: the first p.hetero CTAs take the packed tiles, the others the residual tiles
  // (a residual tile is a short latency-bound chain; kept apart it no longer sits in the packed tiles' warps)
  const bool second = p.hetero > 0 && (int)blockIdx.x >= p.hetero;
  const MzTilesPlan& tp = second ? p.tp2 : p.tp;
  const long long first_record = second ? p.slots_a : 0;      // in records of one head
  const int kt = tp.packed_tiles;

  const int W = tp.total_warps, T = tp.tiles_per_pair;
  const int gw = ((int)blockIdx.x - (second ? p.hetero : 0)) * (blockDim.x >> 5) + warp;
  long long f0 = 0, f1 = 0;
  if (gw < W) mz_warp_tiles(tp, gw, &f0, &f1);

  // ---- this warp's buffers (absolute shared-window addresses; the planner sized the pools)
  const int msz = s.meta_dtype == MZ_F32 ? 4 : 2;
  const uint32_t SB = tp.stage_bytes;
  const uint32_t nw = blockDim.x >> 5;
  Layout L;
  L.kbuf = tp.low_base + warp * SB;
  L.aK = tp.low_base + nw * SB + warp * A_BYTES;
  const uint32_t hb = tp.high_base + warp * (SB + 2 * RI_BYTES + A_BYTES + PBUF_BYTES);
  L.vbuf = hb;
  L.riK = hb + SB;
  L.riV = L.riK + RI_BYTES;
  L.aV = L.riV + RI_BYTES;
  L.pbuf = L.aV + A_BYTES;
  L.dbuf = L.aV;                // residual tiles have no per-row constants
  const bool active = gw < W && f0 < f1;

  const uint32_t lbK = TBL + lane * 4, lbV = TBL + 128 + lane * 4;
  const int hq = g >> 1;                       // head this lane folds for (B operand column g)
  const uint32_t rem_mask = (g & 1) ? 0xFFFFFFFFu : 0u;   // odd columns carry the fp16 remainder of the folded query
  const bool bf = s.kv_dtype == MZ_BF16;
  const int nq = s.k_groups * G;

  struct Cursor { int pair, tile, b, kvh; };
  auto advance = [&](Cursor& c) {
    if (++c.tile == T) {
      c.tile = 0; ++c.pair;
      if (++c.kvh == s.kv_heads) { c.kvh = 0; ++c.b; }
    }
  };
  // residual tile: up to DT rows of 128 elements in padded rows; rows past the end are zeroed (they are
  // multiplied by probability 0, which must not meet a NaN bit pattern)
  auto stage_dense = [&](uint32_t dst, const uint16_t* res, int b, int kvh, int tile) {
    const int tok0 = (tile - kt) * DT;
    const int ntok = min(DT, s.res_len - tok0);
    const uint16_t* src = res + b * s.res_stride_b + kvh * s.res_stride_h + (long long)(s.res_start + tok0) * s.res_stride_t;
    for (int i = lane; i < DT * 16; i += 32) {
      const int row = i >> 4, c = i & 15;
      if (row < ntok) cp16(dst + row * DENSE_STRIDE + c * 16, src + (long long)row * s.res_stride_t + c * 8);
      else sts128(dst + row * DENSE_STRIDE + c * 16, make_uint4(0, 0, 0, 0));
    }
  };
  auto stage_k = [&](const Cursor& c, bool valid) {
    if (valid) {
      if (c.tile < kt) {
        const uint8_t* src = s.packed_k + c.b * s.pk_stride_b + c.kvh * s.pk_stride_h + (long long)c.tile * CODE_BYTES;
        for (int off = lane * 16; off < CODE_BYTES; off += 512) cp16(L.kbuf + off, src + off);
        const long long m0 = (c.b * s.km_stride_b + c.kvh * s.km_stride_h + (long long)c.tile * D) * msz;
        for (int off = lane * 16; off < D * msz; off += 512) {
          cp16(L.kbuf + CODE_BYTES + off, (const uint8_t*)s.k_mn + m0 + off);
          cp16(L.kbuf + CODE_BYTES + D * msz + off, (const uint8_t*)s.k_scale + m0 + off);
        }
      } else {
        stage_dense(L.kbuf, (const uint16_t*)s.res_k, c.b, c.kvh, c.tile);
      }
    }
    cp_async_commit();
  };
  auto stage_v = [&](const Cursor& c, bool valid) {
    if (valid) {
      if (c.tile < kt) {
        const uint8_t* src = s.packed_v + c.b * s.pv_stride_b + c.kvh * s.pv_stride_h + (long long)c.tile * CODE_BYTES;
        for (int i = lane; i < CODE_BYTES / 16; i += 32) {
          // 4-bit: a token's row is 64 bytes; its two 32-byte halves are swapped for tokens with bit 1 set so
          // that the four tokens one load instruction touches fall into different banks
          const int di = BITS == 4 ? (i ^ ((i >> 2) & 2)) : i;
          cp16(L.vbuf + di * 16, src + i * 16);
        }
        const long long m0 = (c.b * s.vm_stride_b + c.kvh * s.vm_stride_h + (long long)c.tile * D) * msz;
        for (int off = lane * 16; off < D * msz; off += 512) {
          cp16(L.vbuf + CODE_BYTES + off, (const uint8_t*)s.v_mn + m0 + off);
          cp16(L.vbuf + CODE_BYTES + D * msz + off, (const uint8_t*)s.v_scale + m0 + off);
        }
      } else {
        stage_dense(L.vbuf, (const uint16_t*)s.res_v, c.b, c.kvh, c.tile);
      }
    }
    cp_async_commit();
  };

  // ---- per-row constants of one staged tile side.  Row r of the side: keys r = channel; values r = token*2 + group.
  // A row's position along the reduction dimension is pos = 8j + 4*slot + tt (block j, slot, lane class tt).
  // Written: the zero code (zc << BITS) as byte [tt][index] of the side's zero-code array, index = 2j + slot for
  // keys and 4j + 2*group + slot for values; half2(Bup, Bdn) as word `slot` of pair (block, tt); A per row.
  // A is the value of the zero code: exactly 0 when the row's range straddles zero, up to the rounding of
  // the anchor (a few 2^-24 of |lo|), which is dropped.  Returns whether any row has a real A.
  auto prep_rows = [&](uint32_t buf, uint32_t ri, uint32_t aout, bool values) -> bool {
    bool any = false;
#pragma unroll
    for (int i = 0; i < D / 32; ++i) {
      const int r = lane + 32 * i;
      float lo, span;
      if (msz == 4) {
        lo = ldsf(buf + CODE_BYTES + r * 4);
        span = ldsf(buf + CODE_BYTES + D * 4 + r * 4);
      } else {
        lo = mz_u16_to_float((uint16_t)lds16(buf + CODE_BYTES + r * 2), s.meta_dtype);
        span = mz_u16_to_float((uint16_t)lds16(buf + CODE_BYTES + D * 2 + r * 2), s.meta_dtype);
      }
      int zc;
      float A, Bup, Bdn;
      row_constants<BITS>(lo, span, zc, A, Bup, Bdn);
      any |= A != 0.0f;
      const int pos = values ? (r >> 1) : r, grp = values ? (r & 1) : 0;
      const int j = pos >> 3, slot = (pos >> 2) & 1, tt = pos & 3;
      sts8(ri + tt * 32 + (values ? 4 * j + 2 * grp + slot : 2 * j + slot), (uint32_t)(zc << BITS));
      sts32(ri + Z_BYTES + (((values ? 2 * j + grp : j) * 4 + tt) * 8) + slot * 4, h2_bits(__floats2half2_rn(Bup, Bdn)));
      stsf(aout + (values ? grp * 64 + pos : pos) * 4, A);
    }
    return __any_sync(0xffffffffu, any);
  };

  float out[8][4];          // M tile m of the output: channels (m < 4 ? 0 : 64) + 8g + 2(m%4) + {0,1}, head t, columns {value, 0-column}
  float m_st, l_st;         // softmax state of head t (l: this lane's tokens only, reduced at the end)
  float base_v[2];          // sum p * A of the two channel groups (this lane's tokens only)
  uint32_t qh2[16];         // folded-query source: half2(q[8j+t], q[8j+4+t]) of head hq, scaled into [0.5, 1)
  float qs = 0.f;           // logit scale of head t for packed tiles: 2^k * scaling * log2(e)
  int cur_pair = -1, seg = 0;

  auto reset_state = [&]() {
#pragma unroll
    for (int m = 0; m < 8; ++m)
#pragma unroll
      for (int k = 0; k < 4; ++k) out[m][k] = 0.f;
    m_st = -INFINITY; l_st = 0.f; base_v[0] = base_v[1] = 0.f;
  };
  auto write_partial = [&]() {
    float lsum = l_st, b0 = base_v[0], b1 = base_v[1];
#pragma unroll
    for (int off = 4; off < 32; off <<= 1) {
      lsum += __shfl_xor_sync(0xffffffffu, lsum, off);
      b0 += __shfl_xor_sync(0xffffffffu, b0, off);
      b1 += __shfl_xor_sync(0xffffffffu, b1, off);
    }
    if (t < GQA) {
      const long long slot = first_record + ((long long)gw * tp.max_segs + seg) * GQA + t;
      if (!MZ_IN_BOUNDS(slot, p.part.slots, 10)) return;
      float* dst = p.part.acc + slot * D + 8 * g;
      float4 v;
      v = make_float4(out[0][0] + out[0][1] + b0, out[0][2] + out[0][3] + b0, out[1][0] + out[1][1] + b0, out[1][2] + out[1][3] + b0);
      *(float4*)(dst) = v;
      v = make_float4(out[2][0] + out[2][1] + b0, out[2][2] + out[2][3] + b0, out[3][0] + out[3][1] + b0, out[3][2] + out[3][3] + b0);
      *(float4*)(dst + 4) = v;
      v = make_float4(out[4][0] + out[4][1] + b1, out[4][2] + out[4][3] + b1, out[5][0] + out[5][1] + b1, out[5][2] + out[5][3] + b1);
      *(float4*)(dst + 64) = v;
      v = make_float4(out[6][0] + out[6][1] + b1, out[6][2] + out[6][3] + b1, out[7][0] + out[7][1] + b1, out[7][2] + out[7][3] + b1);
      *(float4*)(dst + 68) = v;
      if (g == 0) {
        p.part.m[slot] = m_st * (1.0f / LOG2E);   // back to natural-log units
        p.part.l[slot] = lsum;
      }
    }
  };
  // online-softmax update of head t with this lane's logits (base 2): the logits become probabilities in
  // place and the running state is rescaled
  auto softmax_update = [&](auto& sv) {
    constexpr int n = (int)(sizeof(sv) / sizeof(float));
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < n; ++i) mx = fmaxf(mx, sv[i]);
#pragma unroll
    for (int off = 4; off < 32; off <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    const float m_new = fmaxf(m_st, mx);
    const bool dead = !(m_new > -INFINITY);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < n; ++i) {
      sv[i] = dead ? 0.f : ex2f(sv[i] - m_new);
      sum += sv[i];
    }
    const float c = dead ? 1.0f : ex2f(m_st - m_new);   // m_st = -inf -> 0
    l_st = l_st * c + sum;
    m_st = m_new;
    if (__any_sync(0xffffffffu, c != 1.0f)) {
#pragma unroll
      for (int m = 0; m < 8; ++m)
#pragma unroll
        for (int k = 0; k < 4; ++k) out[m][k] *= c;
      base_v[0] *= c; base_v[1] *= c;
    }
  };

  Cursor cur;
  cur.pair = (int)((unsigned)f0 / (unsigned)T); cur.tile = (int)((unsigned)f0 % (unsigned)T);
  cur.b = cur.pair / s.kv_heads; cur.kvh = cur.pair % s.kv_heads;
  Cursor nxt = cur;
  // Everything up to here reads kernel parameters only, and the table build touches shared memory only: when the
  // kernel was launched as a programmatic dependent of the previous kernel in the stream (the merge kernel of the
  // previous call, the append of this step) this prologue runs while that kernel drains.  Global memory is first
  // touched after the wait.
  if (kt > 0) {
    if (p.lut != nullptr) fill_lookup_table_from<BITS>(p.lut);      // written long before the previous kernel started
    else fill_lookup_table<BITS>(s.alpha_key, s.alpha_value);
  }
  for (int i = lane; i < PBUF_BYTES / 4; i += 32) sts32(L.pbuf + i * 4, 0u);   // the odd columns stay zero for good
  asm volatile("griddepcontrol.wait;" ::: "memory");
  stage_k(cur, active);
  stage_v(cur, active);
  __syncthreads();
  if (!active) return;
  reset_state();
  const uint16_t* qrow = nullptr;       // query row of head hq (elements of the cache's 16-bit type)
  for (int left = (int)(f1 - f0); left > 0; --left, cur = nxt) {
    const int pair = cur.pair, tile = cur.tile, b = cur.b, kvh = cur.kvh;
    advance(nxt);
    if (pair != cur_pair) {
      if (cur_pair >= 0) { write_partial(); ++seg; }
      cur_pair = pair;
      reset_state();
      // the query of head hq at this lane's reduction positions, scaled by a power of two into [0.5, 1)
      qrow = (const uint16_t*)p.query + b * p.q_stride_b + (long long)(kvh * GQA + min(hq, GQA - 1)) * p.q_stride_h;
      float qv[32];
      float amax = 0.f;
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        qv[2 * j] = hq < GQA ? mz_u16_to_float(qrow[8 * j + t], s.kv_dtype) : 0.f;
        qv[2 * j + 1] = hq < GQA ? mz_u16_to_float(qrow[8 * j + 4 + t], s.kv_dtype) : 0.f;
        amax = fmaxf(amax, fmaxf(fabsf(qv[2 * j]), fabsf(qv[2 * j + 1])));
      }
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
      int ex = (__float_as_int(amax) >> 23) & 0xff;            // amax in [2^(ex-127), 2^(ex-126))
      ex = min(max(ex, 1), 253);
      const float down = __int_as_float((253 - ex) << 23);     // 2^(126-ex): amax*down in [0.5, 1)
      const float up = __int_as_float((ex + 1) << 23);         // 2^(ex-126)
#pragma unroll
      for (int j = 0; j < 16; ++j) qh2[j] = h2_bits(__floats2half2_rn(qv[2 * j] * down, qv[2 * j + 1] * down));
      // head t's scale sits in the lanes that fold for head t (g = 2t)
      qs = __shfl_sync(0xffffffffu, up, 8 * t) * p.scaling * LOG2E;
    }
    const bool dense = tile >= kt;
    const int tok0 = dense ? (tile - kt) * DT : tile * G;
    const int ntok = dense ? min(DT, s.res_len - tok0) : G;
    const long long mask0 = p.mask ? b * p.mask_stride_b + (dense ? nq : 0) + tok0 : 0;

    cp_async_wait<1>();
    warp_sync();
    if (!dense) {
      // ================= keys =================
      const bool hasA = prep_rows(L.kbuf, L.riK, L.aK, false);
      warp_sync();
      float acc[4][4];
#pragma unroll
      for (int m = 0; m < 4; ++m)
#pragma unroll
        for (int k = 0; k < 4; ++k) acc[m][k] = 0.f;
      {
        // zero codes of this lane's 32 rows; then a two-stage pipeline over the 16 reduction blocks: the code
        // words and fold constants of block j+2 and the table values of block j+1 are in flight while the
        // tensor cores work on block j
        uint32_t zr[8];
        {
          const uint4 za = lds128(L.riK + t * 32), zb = lds128(L.riK + t * 32 + 16);
          zr[0] = za.x; zr[1] = za.y; zr[2] = za.z; zr[3] = za.w; zr[4] = zb.x; zr[5] = zb.y; zr[6] = zb.z; zr[7] = zb.w;
        }
        uint32_t cw[3][2], av[2][16], bf[2][2];
        uint2 Bw[3];
        auto load_block = [&](int j, uint32_t (&w)[2], uint2& B) {
          if (BITS == 4) {
            w[0] = lds32(L.kbuf + (8 * j + t) * QB + 4 * g);
            w[1] = lds32(L.kbuf + (8 * j + 4 + t) * QB + 4 * g);
          } else {
            w[0] = lds16(L.kbuf + (8 * j + t) * QB + 2 * g);
            w[1] = lds16(L.kbuf + (8 * j + 4 + t) * QB + 2 * g);
          }
          B = lds64(L.riK + Z_BYTES + (j * 4 + t) * 8);
        };
        auto open_block = [&](int j, const uint32_t (&w)[2], const uint2& B, uint32_t (&a)[16], uint32_t (&b)[2]) {
          uint32_t z0, z1;
          zero_words<BITS>(zr[j >> 1], 2 * (j & 1), z0, z1);
          lookups16<BITS>(spread_codes<BITS>(w[0], w[1], z0, z1), lbK, a);
          // fold q * B: even columns the product rounded to fp16, odd columns what that rounding dropped
          b[0] = fold_pair(dup_lo(qh2[j]), B.x, rem_mask);
          b[1] = fold_pair(dup_hi(qh2[j]), B.y, rem_mask);
        };
        load_block(0, cw[0], Bw[0]);
        load_block(1, cw[1], Bw[1]);
        open_block(0, cw[0], Bw[0], av[0], bf[0]);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          if (j + 2 < 16) load_block(j + 2, cw[(j + 2) % 3], Bw[(j + 2) % 3]);
          if (j + 1 < 16) open_block(j + 1, cw[(j + 1) % 3], Bw[(j + 1) % 3], av[(j + 1) & 1], bf[(j + 1) & 1]);
          mma4(acc, av[j & 1], bf[j & 1][0], bf[j & 1][1]);
        }
      }
      // constant term sum_d q[t][d] * A_d (rows whose range does not straddle zero)
      float cA = 0.f;
      if (hasA) {
        float part[GQA];
#pragma unroll
        for (int h = 0; h < GQA; ++h) part[h] = 0.f;
        const uint16_t* q0 = (const uint16_t*)p.query + b * p.q_stride_b + (long long)(kvh * GQA) * p.q_stride_h;
        for (int i = 0; i < D / 32; ++i) {
          const int d = lane + 32 * i;
          const float a = ldsf(L.aK + d * 4);
#pragma unroll
          for (int h = 0; h < GQA; ++h) part[h] = fmaf(mz_u16_to_float(q0[h * p.q_stride_h + d], s.kv_dtype), a, part[h]);
        }
#pragma unroll
        for (int h = 0; h < GQA; ++h) {
#pragma unroll
          for (int off = 1; off < 32; off <<= 1) part[h] += __shfl_xor_sync(0xffffffffu, part[h], off);
          if (h == t) cA = part[h] * p.scaling * LOG2E;
        }
      }
      warp_sync();                  // every lane is done with kbuf and the key row info
      stage_k(nxt, left > 1);
      // ================= softmax: this lane has head t, tokens 8g .. 8g+7 =================
      float sv[8];
#pragma unroll
      for (int m = 0; m < 4; ++m) {
        sv[2 * m] = fmaf(acc[m][0] + acc[m][1], qs, cA);
        sv[2 * m + 1] = fmaf(acc[m][2] + acc[m][3], qs, cA);
      }
      if (p.mask) {
#pragma unroll
        for (int i = 0; i < 8; ++i) sv[i] += mz_load_as_float(p.mask, mask0 + 8 * g + i, p.mask_dtype) * LOG2E;
      }
      softmax_update(sv);
      if (t < GQA) {
        // probabilities as fp16 pairs: column 2t the rounded value, column 2t+1 its remainder
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const __half2 ph = __floats2half2_rn(sv[i], sv[i + 4]);
          const float2 phf = __half22float2(ph);
          const uint32_t wa = L.pbuf + g * 128;
          sts32(wa + (((8 * i + 2 * t) ^ pswz(g)) << 2), h2_bits(ph));
          sts32(wa + (((8 * i + 2 * t + 1) ^ pswz(g)) << 2), h2_bits(__floats2half2_rn(sv[i] - phf.x, sv[i + 4] - phf.y)));
        }
      }
      cp_async_wait<1>();
      warp_sync();                  // value tile landed; probabilities visible
      // ================= values =================
      const bool hasAV = prep_rows(L.vbuf, L.riV, L.aV, true);
      warp_sync();
      if (hasAV && t < GQA) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float pi = sv[i];
          base_v[0] = fmaf(pi, ldsf(L.aV + (8 * g + i) * 4), base_v[0]);
          base_v[1] = fmaf(pi, ldsf(L.aV + (64 + 8 * g + i) * 4), base_v[1]);
        }
      }
      {
        // this lane folds for head hq: the rounded probabilities sit in column 2*hq, their remainders in 2*hq+1
        const int lwh = 8 * t + (g & ~1), lwl = lwh + 1;
        uint32_t zr[8], pwh[8], pwl[8];   // zero codes of this lane's 32 rows; half2(p[8j+t], p[8j+4+t]) high parts / remainders
        {
          const uint4 za = lds128(L.riV + t * 32), zb = lds128(L.riV + t * 32 + 16);
          zr[0] = za.x; zr[1] = za.y; zr[2] = za.z; zr[3] = za.w; zr[4] = zb.x; zr[5] = zb.y; zr[6] = zb.z; zr[7] = zb.w;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          pwh[j] = lds32(L.pbuf + j * 128 + ((lwh ^ pswz(j)) << 2));
          pwl[j] = lds32(L.pbuf + j * 128 + ((lwl ^ pswz(j)) << 2)) & rem_mask;
        }
        // 16 reduction blocks: block = 2*j + group; same two-stage pipeline as the keys
        uint32_t cw[3][2], av[2][16], bf[2][2];
        uint2 Bw[3];
        auto load_block = [&](int blk, uint32_t (&w)[2], uint2& B) {
          const int j = blk >> 1, grp = blk & 1;
          if (BITS == 4) {
            const uint32_t vo = ((grp ^ (t >> 1)) * 32) + 4 * g;
            w[0] = lds32(L.vbuf + (8 * j + t) * VROW + vo);
            w[1] = lds32(L.vbuf + (8 * j + 4 + t) * VROW + vo);
          } else {
            w[0] = lds16(L.vbuf + (8 * j + t) * VROW + grp * QB + 2 * g);
            w[1] = lds16(L.vbuf + (8 * j + 4 + t) * VROW + grp * QB + 2 * g);
          }
          B = lds64(L.riV + Z_BYTES + (blk * 4 + t) * 8);
        };
        auto open_block = [&](int blk, const uint32_t (&w)[2], const uint2& B, uint32_t (&a)[16], uint32_t (&b)[2]) {
          const int j = blk >> 1, grp = blk & 1;
          uint32_t z0, z1;
          zero_words<BITS>(zr[j], 2 * grp, z0, z1);
          lookups16<BITS>(spread_codes<BITS>(w[0], w[1], z0, z1), lbV, a);
          // fold (ph + pl) * B: even columns fp16(ph * B), odd columns its remainder + pl * B
          b[0] = h2_bits(__hfma2(dup_lo(pwl[j]), bits_h2(B.x), bits_h2(fold_pair(dup_lo(pwh[j]), B.x, rem_mask))));
          b[1] = h2_bits(__hfma2(dup_hi(pwl[j]), bits_h2(B.y), bits_h2(fold_pair(dup_hi(pwh[j]), B.y, rem_mask))));
        };
        load_block(0, cw[0], Bw[0]);
        load_block(1, cw[1], Bw[1]);
        open_block(0, cw[0], Bw[0], av[0], bf[0]);
#pragma unroll
        for (int blk = 0; blk < 16; ++blk) {
          if (blk + 2 < 16) load_block(blk + 2, cw[(blk + 2) % 3], Bw[(blk + 2) % 3]);
          if (blk + 1 < 16) open_block(blk + 1, cw[(blk + 1) % 3], Bw[(blk + 1) % 3], av[(blk + 1) & 1], bf[(blk + 1) & 1]);
          mma4(out + (blk & 1) * 4, av[blk & 1], bf[blk & 1][0], bf[blk & 1][1]);
        }
      }
    } else {
      // ================= residual keys: 16 tokens x 128 channels of the cache's 16-bit type =================
      float dacc[4] = {0.f, 0.f, 0.f, 0.f};
      const bool fold_lane = (g & 1) == 0 && hq < GQA;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t ka = L.kbuf + g * DENSE_STRIDE + (16 * j + 2 * t) * 2;
        const uint32_t a0 = lds32(ka), a1 = lds32(ka + 8 * DENSE_STRIDE), a2 = lds32(ka + 16), a3 = lds32(ka + 8 * DENSE_STRIDE + 16);
        const uint32_t b0 = fold_lane ? *(const uint32_t*)(qrow + 16 * j + 2 * t) : 0u;
        const uint32_t b1 = fold_lane ? *(const uint32_t*)(qrow + 16 * j + 8 + 2 * t) : 0u;
        if (bf) mma_bf16(dacc, a0, a1, a2, a3, b0, b1);
        else mma_f16(dacc, a0, a1, a2, a3, b0, b1);
      }
      warp_sync();
      stage_k(nxt, left > 1);
      // this lane: head t, tokens g and g + 8
      float sv[2] = {dacc[0] * p.scaling * LOG2E, dacc[2] * p.scaling * LOG2E};
      if (p.mask) {
        if (g < ntok) sv[0] += mz_load_as_float(p.mask, mask0 + g, p.mask_dtype) * LOG2E;
        if (g + 8 < ntok) sv[1] += mz_load_as_float(p.mask, mask0 + g + 8, p.mask_dtype) * LOG2E;
      }
      if (g >= ntok) sv[0] = -INFINITY;
      if (g + 8 >= ntok) sv[1] = -INFINITY;
      softmax_update(sv);
      if (t < GQA) {
        stsf(L.dbuf + (g * 4 + t) * 4, sv[0]);
        stsf(L.dbuf + ((g + 8) * 4 + t) * 4, sv[1]);
      }
      cp_async_wait<1>();
      warp_sync();
      // ================= residual values =================
      // B operand: probabilities of head hq, split into the 16-bit value (even columns) and its remainder
      uint32_t bb[2];
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        float pv[2];
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          const float pf = hq < GQA ? ldsf(L.dbuf + ((2 * t + 8 * half + k) * 4 + hq) * 4) : 0.f;
          const float hi = bf ? __bfloat162float(__float2bfloat16_rn(pf)) : __half2float(__float2half_rn(pf));
          pv[k] = (g & 1) ? pf - hi : hi;
        }
        if (bf) {
          const __nv_bfloat162 v = __floats2bfloat162_rn(pv[0], pv[1]);
          bb[half] = *reinterpret_cast<const uint32_t*>(&v);
        } else {
          bb[half] = h2_bits(__floats2half2_rn(pv[0], pv[1]));
        }
      }
#pragma unroll
      for (int grp = 0; grp < 2; ++grp) {
        const uint32_t va = L.vbuf + (2 * t) * DENSE_STRIDE + (grp * 64 + 8 * g) * 2;
        const uint4 x0 = lds128(va), x1 = lds128(va + DENSE_STRIDE), x2 = lds128(va + 8 * DENSE_STRIDE), x3 = lds128(va + 9 * DENSE_STRIDE);
        const uint32_t c0[4] = {x0.x, x0.y, x0.z, x0.w}, c1[4] = {x1.x, x1.y, x1.z, x1.w};
        const uint32_t c2[4] = {x2.x, x2.y, x2.z, x2.w}, c3[4] = {x3.x, x3.y, x3.z, x3.w};
#pragma unroll
        for (int m = 0; m < 4; ++m) {
          // rows g / g+8 = channels 8g+2m / 8g+2m+1; columns = tokens (2t, 2t+1) and (2t+8, 2t+9)
          const uint32_t a0 = prmt(c0[m], c1[m], 0x5410u), a1 = prmt(c0[m], c1[m], 0x7632u);
          const uint32_t a2 = prmt(c2[m], c3[m], 0x5410u), a3 = prmt(c2[m], c3[m], 0x7632u);
          if (bf) mma_bf16(out[grp * 4 + m], a0, a1, a2, a3, bb[0], bb[1]);
          else mma_f16(out[grp * 4 + m], a0, a1, a2, a3, bb[0], bb[1]);
        }
      }
    }
    warp_sync();                    // every lane is done with vbuf, the value row info and the probabilities
    stage_v(nxt, left > 1);
  }
  cp_async_wait<0>();
  write_partial();
}

// first byte of a kernel's dynamic shared memory inside the shared window
__global__ void smem_base_probe_kernel(unsigned* out) {
  extern __shared__ __align__(128) uint8_t smem[];
  *out = (unsigned)__cvta_generic_to_shared(smem);
}
__device__ unsigned g_probe_result;

template <int BITS, int GQA>
int launch_one(const MzDecodeParams& p, cudaStream_t st) {
  auto kern = decode_mma_kernel<BITS, GQA>;
  MZ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)p.tp.smem_bytes));
  // programmatic dependent launch: harmless after a kernel that never signals (the launch then happens at its
  // completion, as usual); after one that does, the prologue overlaps it
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(p.hetero > 0 ? p.tp.ctas + p.tp2.ctas : p.tp.ctas));
  cfg.blockDim = dim3((unsigned)p.tp.warps_per_cta * 32);
  cfg.dynamicSmemBytes = p.tp.smem_bytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  MZ_CUDA(cudaLaunchKernelEx(&cfg, kern, p));
  MZ_LAUNCH_CHECK("decode_mma");
  return MZ_OK;
}
template <int BITS>
int launch_gqa(const MzDecodeParams& p, cudaStream_t st) {
  switch (p.gqa) {
    case 1: return launch_one<BITS, 1>(p, st);
    case 2: return launch_one<BITS, 2>(p, st);
    case 4: return launch_one<BITS, 4>(p, st);
  }
  return mz_fail(MZ_ERR_UNSUPPORTED, "gqa %d", p.gqa);
}

constexpr int kMaxDevices = 64;
std::mutex g_mu;
int g_window_base[kMaxDevices];      // 0 = not probed yet, -1 = probe failed, else the address

// Lookup-table entries kept in a static device array (no allocation): one slot per (bits, alpha of keys, alpha
// of values) seen on a device.
constexpr int kLutSlots = 16;
__device__ uint32_t g_lut[kLutSlots][512];
template <int BITS>
__global__ void build_lut_kernel(int slot, float alpha_key, float alpha_value) {
  constexpr int NE = 1 << BITS;
  for (int i = threadIdx.x; i < 2 * NE * NE; i += blockDim.x)
    g_lut[slot][i] = lookup_entry<BITS>(i / (NE * NE) ? alpha_value : alpha_key, i % (NE * NE));
}
struct LutKey { int bits; float ak, av; };
struct LutDevice { uint32_t* base; int used; LutKey keys[kLutSlots]; };
LutDevice g_lut_dev[kMaxDevices];
}  // namespace mzm

// Device pointer to the table entries for (bits, alphas) on the current device, or nullptr when they cannot be
// provided (all slots taken, or the one-time build is not possible right now, e.g. during stream capture): the
// kernel then computes the entries in every CTA.  The first request for a combination launches a one-block
// kernel on the default stream and waits for it, so that any stream may use the entries afterwards.
const unsigned* mz_mma_lookup_entries(int bits, float alpha_key, float alpha_value) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= mzm::kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lk(mzm::g_mu);
  mzm::LutDevice& d = mzm::g_lut_dev[dev];
  for (int i = 0; i < d.used; ++i)
    if (d.keys[i].bits == bits && d.keys[i].ak == alpha_key && d.keys[i].av == alpha_value) return d.base + i * 512;
  if (d.used >= mzm::kLutSlots) return nullptr;
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(cudaStreamLegacy, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) {
    (void)cudaGetLastError();
    return nullptr;
  }
  if (d.base == nullptr && cudaGetSymbolAddress((void**)&d.base, mzm::g_lut) != cudaSuccess) {
    (void)cudaGetLastError();
    d.base = nullptr;
    return nullptr;
  }
  const int slot = d.used;
  if (bits == 4) mzm::build_lut_kernel<4><<<1, 256>>>(slot, alpha_key, alpha_value);
  else mzm::build_lut_kernel<2><<<1, 32>>>(slot, alpha_key, alpha_value);
  if (cudaGetLastError() != cudaSuccess || cudaStreamSynchronize(cudaStreamLegacy) != cudaSuccess) {
    (void)cudaGetLastError();
    return nullptr;
  }
  d.keys[slot] = {bits, alpha_key, alpha_value};
  d.used = slot + 1;
  return d.base + slot * 512;
}

// Shared-window address at which this device places dynamic shared memory (a kernel without static shared
// memory).  The tensor-core kernel addresses its buffers absolutely (the lookup table must sit at 65536),
// so the planner needs the number; it is measured once per device with a one-thread kernel and a
// synchronous 4-byte read of a device variable, no allocation.
int mz_smem_window_base() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= mzm::kMaxDevices) return -1;
  std::lock_guard<std::mutex> lk(mzm::g_mu);
  if (mzm::g_window_base[dev] == 0) {
    unsigned* dptr = nullptr;
    unsigned v = 0;
    cudaError_t e = cudaGetSymbolAddress((void**)&dptr, mzm::g_probe_result);
    if (e == cudaSuccess) {
      mzm::smem_base_probe_kernel<<<1, 1, 1024>>>(dptr);
      e = cudaGetLastError();
    }
    if (e == cudaSuccess) e = cudaMemcpyFromSymbol(&v, mzm::g_probe_result, sizeof(v));
    mzm::g_window_base[dev] = (e == cudaSuccess && v > 0 && v < 8192) ? (int)v : -1;
    if (e != cudaSuccess) (void)cudaGetLastError();
  }
  return mzm::g_window_base[dev];
}

bool mz_decode_mma_supported(const MzDecodeParams& p) {
  const mz_kv_store& s = p.s;
  if (!mz_decode_tiles_supported(p)) return false;
  if (s.group != 64 || (s.bits != 2 && s.bits != 4) || p.v_lead != 0) return false;
  if (p.gqa != 1 && p.gqa != 2 && p.gqa != 4) return false;
  // the residual-tile path reads the query in 4-byte pieces
  if (((uintptr_t)p.query & 3) || ((p.q_stride_b | p.q_stride_h) & 1)) return false;
  return mz_smem_window_base() > 0;
}

namespace {
int plan_single(MzDecodeParams& p, int splits_request, int sm_count, size_t* slots);
}
// Cost of a residual tile in CTAs that hold residual tiles only, in the units of cost_q = 64 for a packed tile
// among 12 busy warps (6.4 us).  Such a warp is bound by memory latency (its copies run one tile ahead and a
// tile's arithmetic is short): 2.4 us per tile, measured by sweeping this constant (8 .. 48) at residual lengths
// 128 and 192.
constexpr int kDenseCtaCost = 24;

int mz_plan_mma(MzDecodeParams& p, int splits_request, int sm_count, size_t* slots) {
  const mz_kv_store& s = p.s;
  p.hetero = 0;
  const long long pairs = (long long)s.batch * s.kv_heads;
  const int dense_tiles = (s.res_len + mzm::DT - 1) / mzm::DT;
  // enough packed work to fill every warp of the machine, and a residual window: split the CTAs
  if (splits_request == 0 && s.k_groups > 0 && dense_tiles > 0 && sm_count >= 8 &&
      pairs * s.k_groups >= (long long)sm_count * mzm::MAX_WARPS * 2) {
    const long long cost_d = (long long)dense_tiles * kDenseCtaCost, cost_p = (long long)s.k_groups * 64;
    int n_d = (int)((sm_count * cost_d + cost_d + cost_p - 1) / (cost_d + cost_p));
    if (n_d < 1) n_d = 1;
    if (n_d > sm_count / 2) n_d = sm_count / 2;
    MzDecodeParams a = p, b = p;
    a.s.res_len = 0;
    b.s.k_groups = 0; b.s.v_tokens = 0;
    size_t slots_a = 0, slots_b = 0;
    int rc = plan_single(a, 0, sm_count - n_d, &slots_a);
    if (rc == MZ_OK) rc = plan_single(b, 0, n_d, &slots_b);
    const bool same_shape = rc == MZ_OK && a.tp.warps_per_cta == b.tp.warps_per_cta && a.tp.smem_bytes == b.tp.smem_bytes &&
                            a.tp.stage_bytes == b.tp.stage_bytes && a.tp.low_base == b.tp.low_base && a.tp.high_base == b.tp.high_base;
    if (same_shape) {
      p.tp = a.tp;
      p.tp2 = b.tp;
      p.lut = a.lut;
      p.slots_a = (long long)slots_a;
      p.hetero = a.tp.ctas;
      *slots = slots_a + slots_b;
      return MZ_OK;
    }
  }
  return plan_single(p, splits_request, sm_count, slots);
}

namespace {
int plan_single(MzDecodeParams& p, int splits_request, int sm_count, size_t* slots) {
  const mz_kv_store& s = p.s;
  MzTilesPlan& t = p.tp;
  const int msz = s.meta_dtype == MZ_F32 ? 4 : 2;
  const unsigned code_bytes = mzm::D * (mzm::G * s.bits / 8);
  unsigned sb = code_bytes + 2 * mzm::D * msz;
  if (sb < (unsigned)mzm::DENSE_BYTES) sb = mzm::DENSE_BYTES;
  sb = (sb + 127u) & ~127u;
  const unsigned table_bytes = (1u << (2 * s.bits)) * 256u;
  const unsigned wb = (unsigned)mz_smem_window_base();
  const unsigned low_base = (wb + 127u) & ~127u;
  const unsigned high_base = mzm::TBL + table_bytes;
  const unsigned per_low = sb + mzm::A_BYTES;
  const unsigned per_high = sb + 2 * mzm::RI_BYTES + mzm::A_BYTES + mzm::PBUF_BYTES;
  const unsigned window_end = wb + 227u * 1024u;      // the most dynamic shared memory a block may ask for
  int warps = mzm::MAX_WARPS;
  if ((unsigned)warps > (mzm::TBL - low_base) / per_low) warps = (int)((mzm::TBL - low_base) / per_low);
  if ((unsigned)warps > (window_end - high_base) / per_high) warps = (int)((window_end - high_base) / per_high);
  if (warps < 1) return mz_fail(MZ_ERR_UNSUPPORTED, "tile does not fit shared memory");
  t.kind = 1;
  p.lut = s.k_groups > 0 ? mz_mma_lookup_entries(s.bits, s.alpha_key, s.alpha_value) : nullptr;
  t.stage_bytes = sb;
  t.low_base = low_base;
  t.high_base = high_base;
  t.packed_tiles = s.k_groups;
  t.dense_tokens = mzm::DT;
  const int dense_tiles = (s.res_len + t.dense_tokens - 1) / t.dense_tokens;
  t.tiles_per_pair = t.packed_tiles + dense_tiles;
  // relative cost of a packed tile of 64 tokens and of a residual tile of 16: the ratio of the time a warp
  // spends on one of each while the other warps of its SM keep the pipes busy (measured 6.4 us and 2.0 us)
  t.cost_q = 64;
  t.cost_d = 20;
  const long long pairs = (long long)s.batch * s.kv_heads;
  t.total_tiles = pairs * t.tiles_per_pair;
  t.pair_cost = (long long)t.packed_tiles * t.cost_q + (long long)dense_tiles * t.cost_d;
  if (t.pair_cost < 1) t.pair_cost = 1;
  t.total_cost = pairs * t.pair_cost;
  if (t.total_cost >= (1LL << 31)) return mz_fail(MZ_ERR_UNSUPPORTED, "cache too large for the tiled kernel");
  long long W;
  if (splits_request > 0) {
    W = pairs * splits_request;
  } else {
    W = (long long)sm_count * warps;              // one resident CTA per SM
    const long long one_tile = t.total_cost / t.cost_q;          // at least one packed tile's worth per warp
    if (W > one_tile) W = one_tile;
    if (W < 1) W = 1;
  }
  if (W > (1LL << 30)) return mz_fail(MZ_ERR_ARG, "too many splits");
  t.total_warps = (int)W;
  t.cost_quot = (unsigned)(t.total_cost / W);
  t.cost_rem = (unsigned)(t.total_cost % W);
  if (W < (long long)sm_count * warps) warps = (int)((W + sm_count - 1) / sm_count);
  t.warps_per_cta = warps;
  t.smem_per_warp = per_low + per_high;
  t.smem_bytes = high_base + per_high * warps - wb;
  t.ctas = (int)((W + warps - 1) / warps);
  const long long len = t.total_cost / W + 2;
  t.max_segs = (int)((len - 1) / t.pair_cost + 2);
  *slots = (size_t)W * t.max_segs * p.gqa;
  return MZ_OK;
}

}  // namespace

int mz_launch_decode_mma(const MzDecodeParams& p, cudaStream_t st) {
  if (p.s.bits == 4) return mzm::launch_gqa<4>(p, st);
  if (p.s.bits == 2) return mzm::launch_gqa<2>(p, st);
  return mz_fail(MZ_ERR_UNSUPPORTED, "bits %d", p.s.bits);
}
