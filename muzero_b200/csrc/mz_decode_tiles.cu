// Tiled decode attention for head_dim 128 (sm_100a).
//
// Work item = one tile of G tokens of one (batch, kv head) pair: a packed key group
// [128 rows x QB bytes] with its value rows [G tokens x 128 codes], or G dense residual tokens.
// The flat list of items is cut into equal contiguous ranges, one per WARP; a warp streams its
// range on its own: cp.async stages the next packed tile into its private shared-memory
// buffers while it works on the current one, codes are expanded in registers through
// per-row codebooks (<= 4 bits) or arithmetically (wider codes), all query heads of the kv
// head are served from one read of the tile, softmax is kept online per warp in base 2, and
// each (warp, pair) segment ends in one partial (m, l, acc) record.  A second small kernel
// merges the records of a pair deterministically.  No atomics, no inter-CTA waits.
#include <type_traits>

#include "mz_tiles_common.cuh"

namespace mzt {

template <int BITS, int G, int GQA>
struct Warp {
  using C = Cfg<BITS, G, GQA>;
  float* books; uint8_t* kbuf; uint8_t* vbuf;
  float* pbuf; float* qbuf; float* corr;
  const float* univ_k; const float* univ_v;
  int lane, dl, q16;      // key phase: half-warp (row parity) and token slot within the row
};

// ---- per-row expansion data for one staged tile side (128 rows), one row per ROW_BYTES; the two
// rows that one lookup instruction touches are neighbours, i.e. sit in different bank halves.
// A pass covers D / PASSES rows: channels [pass*RP, +RP) of a key tile, tokens [pass*G/PASSES, ..) of
// a value tile (all groups).
template <int BITS, int G, int GQA, bool VALUES>
__device__ __forceinline__ void build_rows(const Warp<BITS, G, GQA>& w, const uint8_t* meta, int meta_dt, const float* univ,
                                           float alpha, float lg2a, int pass) {
  using C = Cfg<BITS, G, GQA>;
  constexpr int TOP = C::NE - 1;
  const uint8_t* lo_p = meta;
  const uint8_t* sp_p = meta + C::META_BYTES / 2;
  // rotation of the 4-entry store groups that makes the 16-byte stores of 8 neighbouring lanes hit 8 bank groups
  const int rot = (w.lane >> 1) & 3;
#pragma unroll
  for (int i = 0; i < C::RP / 32; ++i) {
    // keys: slot = channel, natural order.  values: slot g*TP + t for token t of the pass and group g
    // (metadata row t*NG + g), so that the rows of two consecutive tokens (the two half-warps of a
    // lookup) are neighbours
    const int slot = w.lane + 32 * i;
    const int r = VALUES ? (pass * C::TP + slot % C::TP) * C::NG + slot / C::TP : pass * C::RP + slot;
    const float lo = meta_at(lo_p, r, meta_dt);
    const float span = meta_at(sp_p, r, meta_dt);
    // IEEE division and multiply: the zero code must round exactly as the dequantizer's does
    // (a symmetric row has anchor == 0.5 and anchor*TOP on a rounding tie)
    float anchor = __fdiv_rn(__fsub_rn(0.0f, lo), fmaxf(span, 1e-8f));
    anchor = fminf(fmaxf(anchor, 0.0f), 1.0f);
    const int zc = __float2int_rn(__fmul_rn(anchor, (float)TOP));
    const float A = fmaf(span, anchor, lo);
    const float Bup = span * fmaxf(1.0f - anchor, 1e-8f);
    const float Bdn = span * fmaxf(anchor, 1e-8f);
    float* dst = w.books + slot * C::BOOK_STRIDE;
    if (C::BOOKS) {
      // entry e = A + B * shape[zc][e], B = Bup at and above the zero code (shape >= 0), Bdn below it
      const float* u = univ + zc * C::UROW;
      if (C::NE >= 4) {
#pragma unroll
        for (int g = 0; g < C::NE / 4; ++g) {
          const int e = (C::NE >= 16 ? ((g + rot) & (C::NE / 4 - 1)) : g) * 4;
          const float4 u4 = *(const float4*)(u + e);
          float4 o4;
          o4.x = fmaf(u4.x < 0.f ? Bdn : Bup, u4.x, A);
          o4.y = fmaf(u4.y < 0.f ? Bdn : Bup, u4.y, A);
          o4.z = fmaf(u4.z < 0.f ? Bdn : Bup, u4.z, A);
          o4.w = fmaf(u4.w < 0.f ? Bdn : Bup, u4.w, A);
          *(float4*)(dst + e) = o4;
        }
      } else {
        dst[0] = fmaf(u[0] < 0.f ? Bdn : Bup, u[0], A);
        dst[1] = fmaf(u[1] < 0.f ? Bdn : Bup, u[1], A);
      }
    } else {
      const float inv_a = 1.0f / alpha;
      const int up = max(TOP - zc, 1), dn = max(zc, 1);
      *(float4*)dst = make_float4(A, Bup * inv_a, Bdn * inv_a, lg2a / (float)up);
      *(float4*)(dst + 4) = make_float4(lg2a / (float)dn, __int_as_float(zc), 0.f, 0.f);
    }
  }
}

// ---- online softmax over one tile.  s[r][k]: base-2 logits of this lane's TPL tokens for the
// head it owns in round r (head = 2*r + dl).  Writes probabilities to pbuf and corrections to corr.
template <int BITS, int G, int GQA>
__device__ __forceinline__ void softmax_tile(const Warp<BITS, G, GQA>& w, float (&s)[Cfg<BITS, G, GQA>::ROUNDS][Cfg<BITS, G, GQA>::TPL],
                                             float (&m_st)[Cfg<BITS, G, GQA>::ROUNDS], float (&l_st)[Cfg<BITS, G, GQA>::ROUNDS]) {
  using C = Cfg<BITS, G, GQA>;
#pragma unroll
  for (int r = 0; r < C::ROUNDS; ++r) {
    const int h = 2 * r + w.dl;
    float mx = s[r][0];
#pragma unroll
    for (int k = 1; k < C::TPL; ++k) mx = fmaxf(mx, s[r][k]);
#pragma unroll
    for (int off = 1; off < 16; off <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    const float m_new = fmaxf(m_st[r], mx);
    const bool dead = !(m_new > -INFINITY);
    float sum = 0.f;
    float pr[C::TPL];
#pragma unroll
    for (int k = 0; k < C::TPL; ++k) {
      pr[k] = dead ? 0.f : ex2f(s[r][k] - m_new);
      sum += pr[k];
    }
#pragma unroll
    for (int off = 1; off < 16; off <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
    const float c = dead ? 1.0f : ex2f(m_st[r] - m_new);   // m_st = -inf -> 0
    l_st[r] = l_st[r] * c + sum;
    m_st[r] = m_new;
    if (h < GQA) {
#pragma unroll
      for (int k = 0; k < C::TPL; ++k) w.pbuf[(w.q16 * C::TPL + k) * GQA + h] = pr[k];
      if (w.q16 == 0) w.corr[h] = c;
    }
  }
}

// Two neighbouring codes (idx, idx + 1) of a packed row in global memory, dequantized with the reference's fp32
// formula (muzero/quantizer.py:229-255; expm1 evaluated directly).  Cold path: residual tokens whose values
// were flushed ahead of their keys.
template <int BITS>
__device__ __noinline__ float2 dequant_pair(const uint8_t* row, int idx, int row_bytes, float lo, float span, float alpha) {
  const MzRowParams r = mz_row_params(lo, span, (1 << BITS) - 1, 1e-8f);
  const float lb = log1pf(alpha);
  float out[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int q = mz_extract_code(row, idx + i, BITS, row_bytes);
    float unit;
    if (q >= r.zero_code) {
      const float grow = expm1f((float)min(q - r.zero_code, r.steps_up) / (float)r.steps_up * lb) / alpha;
      unit = r.anchor + r.room_up * grow;
    } else {
      const float grow = expm1f((float)min(r.zero_code - q, r.steps_dn) / (float)r.steps_dn * lb) / alpha;
      unit = r.anchor - r.room_dn * grow;
    }
    out[i] = fminf(fmaxf(unit, 0.0f), 1.0f) * span + lo;
  }
  return make_float2(out[0], out[1]);
}

template <int BITS, int G, int GQA>
__global__ void __launch_bounds__(Cfg<BITS, G, GQA>::MAX_WARPS * 32, 1) decode_tiles_kernel(const MzDecodeParams p) {
  using C = Cfg<BITS, G, GQA>;
  extern __shared__ __align__(16) uint8_t smem[];
  const mz_kv_store& s = p.s;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // the merge kernel waits for this grid's completion itself

  // signed shape tables: row zc, entry e -> normalised value of code e (>= 0 at and above the zero code, < 0 below)
  uint8_t* smem_al = smem + ((256u - ((unsigned)__cvta_generic_to_shared(smem) & 255u)) & 255u);
  float* univ_k = (float*)smem_al;
  float* univ_v = univ_k + C::UNIV_FLOATS;
  if (C::BOOKS) {
    constexpr int TOP = C::NE - 1;
    for (int i = threadIdx.x; i < 2 * C::NE * C::NE; i += blockDim.x) {
      const int which = i / (C::NE * C::NE), j = i % (C::NE * C::NE);
      const int zc = j / C::NE, e = j % C::NE;
      const float alpha = which ? s.alpha_value : s.alpha_key;
      const float lb = log1pf(alpha);
      float u;
      if (e >= zc) {
        const int up = max(TOP - zc, 1);
        u = expm1f((float)min(e - zc, up) / (float)up * lb) / alpha;
      } else {
        const int dn = max(zc, 1);
        u = -expm1f((float)(zc - e) / (float)dn * lb) / alpha;
      }
      (which ? univ_v : univ_k)[zc * C::UROW + e] = u;
    }
  }
  __syncthreads();

  const int W = p.tp.total_warps, T = p.tp.tiles_per_pair;
  const int gw = blockIdx.x * (blockDim.x >> 5) + warp;
  if (gw >= W) return;
  long long f0, f1;
  mz_warp_tiles(p.tp, gw, &f0, &f1);
  if (f0 >= f1) return;

  Warp<BITS, G, GQA> w;
  uint8_t* base = smem_al + (C::SHARED - 256) + (size_t)warp * C::PER_WARP;   // 256-byte aligned
  w.books = (float*)base;
  w.kbuf = base + C::BOOK_BYTES;
  w.vbuf = w.kbuf + C::KBUF;
  w.pbuf = (float*)(w.vbuf + C::VBUF);
  w.qbuf = (float*)((uint8_t*)w.pbuf + C::PBUF);
  w.corr = (float*)((uint8_t*)w.qbuf + C::QBUF);
  w.univ_k = univ_k; w.univ_v = univ_v;
  w.lane = lane; w.dl = lane >> 4; w.q16 = lane & 15;

  const int msz = s.meta_dtype == MZ_F32 ? 4 : 2;
  const float lg2a_k = log2f(1.0f + s.alpha_key), lg2a_v = log2f(1.0f + s.alpha_value);
  const int nq = s.k_groups * G;
  const uint32_t books_sa = (uint32_t)__cvta_generic_to_shared(w.books);

  // position of a tile; walked incrementally (no divisions in the tile loop)
  struct Cursor { int pair, tile, b, kvh; };
  auto advance = [&](Cursor& c) {
    if (++c.tile == T) {
      c.tile = 0; ++c.pair;
      if (++c.kvh == s.kv_heads) { c.kvh = 0; ++c.b; }
    }
  };
  // residual tile: up to DT rows of 128 un-quantized elements, 16 lanes per row
  auto stage_dense = [&](uint8_t* dst, const uint16_t* res, int b, int kvh, int tile) {
    const int tok0 = (tile - s.k_groups) * C::DT;
    const int ntok = min(C::DT, s.res_len - tok0);
    const uint16_t* src = res + b * s.res_stride_b + kvh * s.res_stride_h + (long long)(s.res_start + tok0) * s.res_stride_t;
    for (int i = lane; i < ntok * 16; i += 32) cp_async16(dst + i * 16, src + (long long)(i >> 4) * s.res_stride_t + (i & 15) * 8);
  };
  auto stage_k = [&](const Cursor& c, bool valid) {
    if (valid) {
      const int b = c.b, kvh = c.kvh, tile = c.tile;
      if (tile < s.k_groups) {
        const uint8_t* src = s.packed_k + b * s.pk_stride_b + kvh * s.pk_stride_h + (long long)tile * C::TILE_BYTES;
        warp_copy_async(w.kbuf, src, C::TILE_BYTES, lane);
        const long long m0 = (b * s.km_stride_b + kvh * s.km_stride_h + (long long)tile * D) * msz;
        warp_copy_async(w.kbuf + C::STAGE_BYTES, (const uint8_t*)s.k_mn + m0, D * msz, lane);
        warp_copy_async(w.kbuf + C::STAGE_BYTES + C::META_BYTES / 2, (const uint8_t*)s.k_scale + m0, D * msz, lane);
      } else {
        stage_dense(w.kbuf, (const uint16_t*)s.res_k, b, kvh, tile);
      }
    }
    cp_async_commit();
  };
  auto stage_v = [&](const Cursor& c, bool valid) {
    if (valid) {
      const int b = c.b, kvh = c.kvh, tile = c.tile;
      if (tile < s.k_groups) {
        const uint8_t* src = s.packed_v + b * s.pv_stride_b + kvh * s.pv_stride_h + (long long)tile * C::TILE_BYTES;
        warp_copy_async(w.vbuf, src, C::TILE_BYTES, lane);
        const long long m0 = (b * s.vm_stride_b + kvh * s.vm_stride_h + (long long)tile * D) * msz;
        warp_copy_async(w.vbuf + C::STAGE_BYTES, (const uint8_t*)s.v_mn + m0, D * msz, lane);
        warp_copy_async(w.vbuf + C::STAGE_BYTES + C::META_BYTES / 2, (const uint8_t*)s.v_scale + m0, D * msz, lane);
      } else {
        stage_dense(w.vbuf, (const uint16_t*)s.res_v, b, kvh, tile);
      }
    }
    cp_async_commit();
  };

  // value phase: lane (tp = lane>>4, j = lane&15) owns, in every group g, channels g*G + j*TPL .. +TPL-1
  // (8 channels in all) of the tokens of parity tp; pairs of neighbouring channels per head
  float2 out2[4][GQA];
  float m_st[C::ROUNDS], l_st[C::ROUNDS];
  int cur_pair = -1, seg = 0;

  auto reset_state = [&]() {
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int h = 0; h < GQA; ++h) out2[j][h] = make_float2(0.f, 0.f);
#pragma unroll
    for (int r = 0; r < C::ROUNDS; ++r) { m_st[r] = -INFINITY; l_st[r] = 0.f; }
  };
  auto write_partial = [&]() {
    const long long slot0 = ((long long)gw * p.tp.max_segs + seg) * GQA;
    if (!MZ_IN_BOUNDS(slot0 + GQA - 1, p.part.slots, 11)) return;
#pragma unroll
    for (int h = 0; h < GQA; ++h) {
      float2 t[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {      // add the tokens of the other parity
        t[j].x = out2[j][h].x + __shfl_xor_sync(0xffffffffu, out2[j][h].x, 16);
        t[j].y = out2[j][h].y + __shfl_xor_sync(0xffffffffu, out2[j][h].y, 16);
      }
      if (lane < 16) {
        float* dst = p.part.acc + (slot0 + h) * D;
#pragma unroll
        for (int g = 0; g < C::NG; ++g)
#pragma unroll
          for (int k = 0; k < C::TPL; k += 2) *(float2*)(dst + g * G + lane * C::TPL + k) = t[g * (C::TPL / 2) + k / 2];
      }
    }
#pragma unroll
    for (int r = 0; r < C::ROUNDS; ++r) {
      const int h = 2 * r + w.dl;
      if (h < GQA && w.q16 == 0) {
        p.part.m[slot0 + h] = m_st[r] * (1.0f / LOG2E);   // back to natural-log units
        p.part.l[slot0 + h] = l_st[r];
      }
    }
  };

  Cursor cur;
  cur.pair = (int)((unsigned)f0 / (unsigned)T); cur.tile = (int)((unsigned)f0 % (unsigned)T);
  cur.b = cur.pair / s.kv_heads; cur.kvh = cur.pair % s.kv_heads;
  Cursor nxt = cur;
  stage_k(cur, true);
  stage_v(cur, true);
  for (int left = (int)(f1 - f0); left > 0; --left, cur = nxt) {
    const int pair = cur.pair, tile = cur.tile, b = cur.b, kvh = cur.kvh;
    advance(nxt);
    if (pair != cur_pair) {
      if (cur_pair >= 0) { write_partial(); ++seg; }
      cur_pair = pair;
      reset_state();
      __syncwarp();
      const float qs = p.scaling * LOG2E;
      for (int i = lane; i < D * GQA; i += 32) {
        const int d = i / GQA, h = i % GQA;
        w.qbuf[i] = mz_load_as_float(p.query, b * p.q_stride_b + (long long)(kvh * GQA + h) * p.q_stride_h + d, s.kv_dtype) * qs;
      }
      __syncwarp();
    }
    const bool dense = tile >= s.k_groups;
    const int tok0 = dense ? (tile - s.k_groups) * C::DT : tile * G;      // first token inside its region
    const int ntok = dense ? min(C::DT, s.res_len - tok0) : G;
    const long long mask0 = p.mask ? b * p.mask_stride_b + (dense ? nq : 0) + tok0 : 0;
    float sl[C::ROUNDS][C::TPL];

    cp_async_wait<1>();
    __syncwarp();
    if (!dense) {
      // ---------------- keys: expansion rows, then QK with all heads per code
      float2 acc2[C::TPL / 2][GQA];      // token pairs (2j, 2j+1)
#pragma unroll
      for (int k = 0; k < C::TPL / 2; ++k)
#pragma unroll
        for (int h = 0; h < GQA; ++h) acc2[k][h] = make_float2(0.f, 0.f);
#pragma unroll 1
      for (int pass = 0; pass < C::PASSES; ++pass) {
        if (pass) __syncwarp();                               // every lane is done with the previous pass' rows
        build_rows<BITS, G, GQA, false>(w, w.kbuf + C::STAGE_BYTES, s.meta_dtype, w.univ_k, s.alpha_key, lg2a_k, pass);
        __syncwarp();
        const uint32_t lane_off = w.dl * C::ROW_BYTES;        // row 2*step + dl
        const uint8_t* krow = w.kbuf + w.dl * C::QB;
        const float* qd = w.qbuf + w.dl * GQA;
        const int sb0 = pass * (C::KSTEPS / C::PASSES);
#pragma unroll 1
        for (int sb = sb0; sb < sb0 + C::KSTEPS / C::PASSES; sb += C::UNROLL) {
          const uint32_t rb = books_sa + (sb - sb0) * (2 * C::ROW_BYTES);
          auto one_step = [&](auto uc) {
            constexpr int u = decltype(uc)::value;
            const int step = sb + u;
            const unsigned long long codes = load_codes<BITS, C::TPL>(krow + step * (2 * C::QB), w.q16 * C::TPL);
            float v[C::TPL];
            expand<BITS, C::BOOKS, C::PRMT_ADDR, C::TPL, u * (2 * C::ROW_BYTES)>(codes, rb, lane_off, v);
            float qh[GQA];
            if (GQA % 4 == 0) {
#pragma unroll
              for (int h = 0; h < GQA; h += 4) {
                const float4 t4 = *(const float4*)(qd + step * (2 * GQA) + h);
                qh[h] = t4.x; qh[h + 1] = t4.y; qh[h + 2] = t4.z; qh[h + 3] = t4.w;
              }
            } else {
#pragma unroll
              for (int h = 0; h < GQA; ++h) qh[h] = qd[step * (2 * GQA) + h];
            }
#pragma unroll
            for (int h = 0; h < GQA; ++h) {
              const float2 qq = make_float2(qh[h], qh[h]);
#pragma unroll
              for (int k = 0; k < C::TPL; k += 2) ffma2(acc2[k / 2][h], make_float2(v[k], v[k + 1]), qq);
            }
          };
          one_step(std::integral_constant<int, 0>{});
          one_step(std::integral_constant<int, 1>{});
          one_step(std::integral_constant<int, 2>{});
          one_step(std::integral_constant<int, 3>{});
        }
      }
      // add the rows handled by the other half-warp
#pragma unroll
      for (int k = 0; k < C::TPL / 2; ++k)
#pragma unroll
        for (int h = 0; h < GQA; ++h) {
          acc2[k][h].x += __shfl_xor_sync(0xffffffffu, acc2[k][h].x, 16);
          acc2[k][h].y += __shfl_xor_sync(0xffffffffu, acc2[k][h].y, 16);
        }
#pragma unroll
      for (int r = 0; r < C::ROUNDS; ++r)
#pragma unroll
        for (int k = 0; k < C::TPL; ++k) {
          float val = 0.f;
#pragma unroll
          for (int h = 0; h < GQA; ++h)
            if (h / 2 == r && (h & 1) == w.dl) val = (k & 1) ? acc2[k / 2][h].y : acc2[k / 2][h].x;
          sl[r][k] = val;
        }
    } else {
      // ---------------- residual keys (staged rows of 128 elements): half-warp dl takes tokens
      // NB*(2*batch + dl) .. +NB-1, lane j of it channels 8j .. 8j+7; the 16 partial dots of every
      // (token, head) are then summed by a reduce-scatter; logits go through shared memory
      float* sbuf = w.pbuf;
      for (int i = lane; i < G * GQA; i += 32) sbuf[i] = -INFINITY;
      constexpr int HB = GQA > 4 ? 4 : GQA;             // heads per sweep (bounds the registers held)
      constexpr int NB = 32 / HB;                       // tokens per half-warp and batch: 32 partial sums per lane
      __syncwarp();
#pragma unroll 1
      for (int h0 = 0; h0 < GQA; h0 += HB) {
        float qr[8][HB];
#pragma unroll
        for (int c = 0; c < 8; ++c)
#pragma unroll
          for (int h = 0; h < HB; ++h) qr[c][h] = w.qbuf[(w.q16 * 8 + c) * GQA + h0 + h];
#pragma unroll 1
        for (int t0 = 0; t0 < ntok; t0 += 2 * NB) {
          float part[32];
#pragma unroll
          for (int tt = 0; tt < NB; ++tt) {
            const int t = min(t0 + w.dl * NB + tt, C::DT - 1);   // rows past ntok hold stale bytes; their logits are dropped below
            const uint4 raw = *(const uint4*)(w.kbuf + t * (2 * D) + w.q16 * 16);
            const uint32_t ww[4] = {raw.x, raw.y, raw.z, raw.w};
            float dot[HB];
#pragma unroll
            for (int h = 0; h < HB; ++h) dot[h] = 0.f;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 x = unpack2(ww[e], s.kv_dtype);
#pragma unroll
              for (int h = 0; h < HB; ++h) dot[h] = fmaf(x.y, qr[2 * e + 1][h], fmaf(x.x, qr[2 * e][h], dot[h]));
            }
#pragma unroll
            for (int h = 0; h < HB; ++h) part[tt * HB + h] = dot[h];
          }
          // reduce-scatter over the 16 lanes of the half-warp: lane j ends with sums 2j and 2j+1
#pragma unroll
          for (int n = 16, bit = 8; bit >= 1; n >>= 1, bit >>= 1) {
            const bool upper = (w.q16 & bit) != 0;
#pragma unroll
            for (int i = 0; i < n; ++i) {
              const float keep = upper ? part[i + n] : part[i];
              const float send = upper ? part[i] : part[i + n];
              part[i] = keep + __shfl_xor_sync(0xffffffffu, send, bit);
            }
          }
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            const int idx = 2 * w.q16 + i;
            const int t = t0 + w.dl * NB + idx / HB;
            if (t < ntok) sbuf[t * GQA + h0 + idx % HB] = part[i];
          }
        }
      }
      __syncwarp();
#pragma unroll
      for (int r = 0; r < C::ROUNDS; ++r) {
        const int h = min(2 * r + w.dl, GQA - 1);
#pragma unroll
        for (int k = 0; k < C::TPL; ++k) sl[r][k] = sbuf[(w.q16 * C::TPL + k) * GQA + h];
      }
    }
    __syncwarp();                 // every lane is done with kbuf, the rows and sbuf
    stage_k(nxt, left > 1);
    if (p.mask) {
#pragma unroll
      for (int k = 0; k < C::TPL; ++k) {
        const int t = w.q16 * C::TPL + k;
        const float mv = t < ntok ? mz_load_as_float(p.mask, mask0 + t, p.mask_dtype) * LOG2E : 0.f;
#pragma unroll
        for (int r = 0; r < C::ROUNDS; ++r) sl[r][k] += mv;
      }
    }
    softmax_tile<BITS, G, GQA>(w, sl, m_st, l_st);
    cp_async_wait<1>();
    __syncwarp();                 // value tile landed; probabilities and corrections visible
    {
      bool rescale = false;
      float cr[GQA];
#pragma unroll
      for (int h = 0; h < GQA; ++h) { cr[h] = w.corr[h]; rescale |= cr[h] != 1.0f; }
      if (rescale) {
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
          for (int h = 0; h < GQA; ++h) { out2[j][h].x *= cr[h]; out2[j][h].y *= cr[h]; }
      }
    }
    if (!dense) {
#pragma unroll 1
      for (int pass = 0; pass < C::PASSES; ++pass) {
        if (pass) __syncwarp();
        build_rows<BITS, G, GQA, true>(w, w.vbuf + C::STAGE_BYTES, s.meta_dtype, w.univ_v, s.alpha_value, lg2a_v, pass);
        __syncwarp();
        const uint32_t lane_off = w.dl * C::ROW_BYTES;        // token 2*step + tp inside a step's pair of rows
        const uint8_t* vrow = w.vbuf + w.dl * C::VROW_BYTES;
        const float* pd = w.pbuf + w.dl * GQA;
        const int sb0 = pass * (C::TP / 2);
#pragma unroll 1
        for (int sb = sb0; sb < sb0 + C::TP / 2; sb += C::UNROLL) {
          const uint32_t rb = books_sa + (sb - sb0) * (2 * C::ROW_BYTES);
          auto one_step = [&](auto uc) {
            constexpr int u = decltype(uc)::value;
            const int step = sb + u;
            float ph[GQA];
            if (GQA % 4 == 0) {
#pragma unroll
              for (int h = 0; h < GQA; h += 4) {
                const float4 t4 = *(const float4*)(pd + step * (2 * GQA) + h);
                ph[h] = t4.x; ph[h + 1] = t4.y; ph[h + 2] = t4.z; ph[h + 3] = t4.w;
              }
            } else {
#pragma unroll
              for (int h = 0; h < GQA; ++h) ph[h] = pd[step * (2 * GQA) + h];
            }
#pragma unroll
            for (int g = 0; g < C::NG; ++g) {
              const unsigned long long codes = load_codes<BITS, C::TPL>(vrow + step * (2 * C::VROW_BYTES) + g * C::QB, w.q16 * C::TPL);
              float v[C::TPL];
              expand<BITS, C::BOOKS, C::PRMT_ADDR, C::TPL, u * (2 * C::ROW_BYTES)>(codes, rb + g * (C::TP * C::ROW_BYTES), lane_off, v);
#pragma unroll
              for (int h = 0; h < GQA; ++h) {
                const float2 pp = make_float2(ph[h], ph[h]);
#pragma unroll
                for (int k = 0; k < C::TPL; k += 2) ffma2(out2[g * (C::TPL / 2) + k / 2][h], make_float2(v[k], v[k + 1]), pp);
              }
            }
          };
          one_step(std::integral_constant<int, 0>{});
          one_step(std::integral_constant<int, 1>{});
          one_step(std::integral_constant<int, 2>{});
          one_step(std::integral_constant<int, 3>{});
        }
      }
    } else {
      const uint16_t* rv = (const uint16_t*)w.vbuf + w.q16 * C::TPL;
#pragma unroll 2
      for (int t = w.dl; t < ntok; t += 2) {
        const uint16_t* row = rv + t * D;
        float ph[GQA];
#pragma unroll
        for (int h = 0; h < GQA; ++h) ph[h] = w.pbuf[t * GQA + h];
        // a residual token whose value already sits in the packed store (the value prefix runs ahead of the
        // key prefix): its channels are dequantized from there in fp32, the stale window row is not used
        const bool from_store = tok0 + t < p.v_lead;
        const long long vrow = (long long)nq + tok0 + t;
#pragma unroll
        for (int g = 0; g < C::NG; ++g)
#pragma unroll
          for (int k = 0; k < C::TPL; k += 2) {
            float2 x;
            if (from_store) {
              const uint8_t* pr = s.packed_v + b * s.pv_stride_b + kvh * s.pv_stride_h + (vrow * C::NG + g) * C::QB;
              const long long mi = b * s.vm_stride_b + kvh * s.vm_stride_h + vrow * C::NG + g;
              x = dequant_pair<BITS>(pr, w.q16 * C::TPL + k, C::QB, mz_load_as_float(s.v_mn, mi, s.meta_dtype),
                                     mz_load_as_float(s.v_scale, mi, s.meta_dtype), s.alpha_value);
            } else {
              x = unpack2(*(const uint32_t*)(row + g * G + k), s.kv_dtype);
            }
#pragma unroll
            for (int h = 0; h < GQA; ++h) ffma2(out2[g * (C::TPL / 2) + k / 2][h], x, make_float2(ph[h], ph[h]));
          }
      }
    }
    __syncwarp();                 // every lane is done with vbuf, the rows and pbuf
    stage_v(nxt, left > 1);
  }
  cp_async_wait<0>();
  write_partial();
}

// ---- merge of the records of one (batch, kv head) pair: one CTA per pair, one warp-quad (128
// threads) per query head.  The warps of the main kernel that hold records of the pair are found from
// the partition functions the main kernel uses: warp g owns the tiles whose start cost lies in
// [cost(g), cost(g+1)), and cost(g) is within [g*quot, g*(quot+1)), so every contributor lies in the
// candidate range [c_lo/(quot+1) - 1, (c_hi-1)/quot + 1], c_lo..c_hi being the pair's cost interval.
// All threads test candidates at once; the list keeps the candidates' order (a fixed merge order).
// WIDE (many records per pair, few pairs): one CTA per (pair, head); its four warp-quads each merge every
// fourth chunk of records and the four partial states are merged in a fixed order at the end.
constexpr int kMaxCombineSlots = 4096;
// The workers of plan `tp` that can hold records of `pair` lie in [first, last] (a superset; see above).
struct WorkerRange { long long first, last; };
__device__ __forceinline__ WorkerRange candidate_workers(const MzTilesPlan& tp, int pair) {
  WorkerRange r = {0, -1};
  if (tp.total_warps <= 0) return r;
  const unsigned quot = tp.cost_quot ? tp.cost_quot : 1u;
  const unsigned c_lo = (unsigned)pair * (unsigned)tp.pair_cost, c_hi = c_lo + (unsigned)tp.pair_cost;
  r.first = (long long)(c_lo / (quot + 1u)) - 1;
  r.last = (long long)((c_hi - 1u) / quot) + 1;
  if (r.first < 0 || tp.cost_quot == 0) r.first = 0;
  if (r.last > tp.total_warps - 1 || tp.cost_quot == 0) r.last = tp.total_warps - 1;   // more workers than cost units: test them all
  return r;
}
// record index of worker gw's segment for `pair` (first_record = index of the plan's first record), or -1
__device__ __forceinline__ long long record_of(const MzTilesPlan& tp, long long gw, int pair, long long first_record) {
  const int T = tp.tiles_per_pair;
  const long long lo = (long long)pair * T, hi = lo + T;
  long long f0, f1;
  mz_warp_tiles(tp, gw, &f0, &f1);
  if (!(f0 < hi && f1 > lo && f0 < f1)) return -1;
  return first_record + gw * tp.max_segs + (pair - (int)((unsigned)f0 / (unsigned)T));
}
template <bool WIDE>
__global__ void __launch_bounds__(512, 4) combine_tiles_kernel(const MzDecodeParams p, const MzDecodeOut o) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // a dependent waits for this grid's completion itself
  __shared__ int s_slot[kMaxCombineSlots];     // record of candidate i, or -1
  __shared__ float s_part[WIDE ? 4 : 1][WIDE ? 130 : 1];
  const int pair = WIDE ? blockIdx.x / p.gqa : blockIdx.x;
  const int gqa = p.gqa;
  // candidates of the main plan, then of the residual-tile plan of the tcgen05 route (its records follow)
  const WorkerRange ra = candidate_workers(p.tp, pair), rb = candidate_workers(p.tp2, pair);
  const long long cand_a = ra.last - ra.first + 1, cand_b = rb.last - rb.first + 1;
  const long long cand = cand_a + cand_b;
  const long long first_b = p.slots_a / gqa;
  const bool listed = cand <= kMaxCombineSlots &&
                      first_b + (long long)p.tp.total_warps * p.tp.max_segs + (long long)p.tp2.total_warps * p.tp2.max_segs < (1LL << 31);
  if (listed) {
    for (int i = threadIdx.x; i < cand; i += blockDim.x)
      s_slot[i] = (int)(i < cand_a ? record_of(p.tp, ra.first + i, pair, 0) : record_of(p.tp2, rb.first + (i - cand_a), pair, first_b));
  }
  // everything above is arithmetic on the plans; the records themselves are the main kernels' output
  asm volatile("griddepcontrol.wait;" ::: "memory");
  __syncthreads();
  const int n = (int)cand;
  // more candidates than the list holds (a huge explicit split count): every thread walks them itself
  auto for_each_slot = [&](auto&& fn) {
    for (long long gw = ra.first; gw <= ra.last; ++gw) {
      const long long rec = record_of(p.tp, gw, pair, 0);
      if (rec >= 0) fn(rec);
    }
    for (long long gw = rb.first; gw <= rb.last; ++gw) {
      const long long rec = record_of(p.tp2, gw, pair, first_b);
      if (rec >= 0) fn(rec);
    }
  };
  const int quad = threadIdx.x >> 7, quads = blockDim.x >> 7;
  for (int h = WIDE ? blockIdx.x % gqa : quad; h < gqa; h += WIDE ? gqa : quads) {
    const int d = threadIdx.x & 127;
    float mx = -INFINITY, lsum = 0.f, a = 0.f;
    if (listed) {
      // four records at a time: their loads are independent and in flight together; the running
      // maximum is carried along (one pass)
      for (int i0 = WIDE ? 4 * quad : 0; i0 < n; i0 += WIDE ? 4 * quads : 4) {
        float mi[4], li[4], ai[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int sl = i0 + j < n ? s_slot[i0 + j] : -1;
          const bool on = sl >= 0;
          const long long slot = on ? (long long)sl * gqa + h : 0;
          mi[j] = on ? p.part.m[slot] : -INFINITY;
          li[j] = on ? p.part.l[slot] : 0.f;
          ai[j] = on ? p.part.acc[slot * D + d] : 0.f;
        }
        const float m_new = fmaxf(fmaxf(mx, fmaxf(mi[0], mi[1])), fmaxf(mi[2], mi[3]));
        const float keep = mx > -INFINITY ? __expf(mx - m_new) : 0.f;
        lsum *= keep; a *= keep;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float wgt = mi[j] > -INFINITY ? __expf(mi[j] - m_new) : 0.f;
          lsum = fmaf(li[j], wgt, lsum);
          a = fmaf(ai[j], wgt, a);
        }
        mx = m_new;
      }
      if (WIDE) {
        // the quads' states, merged in quad order by quad 0
        s_part[quad][d] = a;
        if (d == 0) { s_part[quad][128] = mx; s_part[quad][129] = lsum; }
        __syncthreads();
        if (quad != 0) continue;      // WIDE visits one head per CTA: nothing follows for these threads
        float m_all = -INFINITY;
        for (int k = 0; k < quads; ++k) m_all = fmaxf(m_all, s_part[k][128]);
        lsum = 0.f; a = 0.f;
        for (int k = 0; k < quads; ++k) {
          const float mk = s_part[k][128];
          const float wgt = mk > -INFINITY ? __expf(mk - m_all) : 0.f;
          lsum = fmaf(s_part[k][129], wgt, lsum);
          a = fmaf(s_part[k][d], wgt, a);
        }
        mx = m_all;
      }
    } else if (!WIDE || quad == 0) {
      for_each_slot([&](long long sl) { mx = fmaxf(mx, p.part.m[sl * gqa + h]); });
      for_each_slot([&](long long sl) {
        const long long slot = sl * gqa + h;
        const float mi = p.part.m[slot];
        const float wgt = mi > -INFINITY ? __expf(mi - mx) : 0.f;
        lsum = fmaf(p.part.l[slot], wgt, lsum);
        a = fmaf(p.part.acc[slot * D + d], wgt, a);
      });
    } else {
      continue;
    }
    const long long row = (long long)pair * gqa + h;
    if (o.out) mz_store_from_float(o.out, row * D + d, a / fmaxf(lsum, 1e-20f), o.out_dt);
    else {
      o.acc[row * o.acc_stride + d] = a;
      if (d == 0) { o.m[row * o.ml_stride] = mx; o.l[row * o.ml_stride] = lsum; }
    }
  }
}

// The common case (a handful of records per pair): one WARP per (pair, head), no shared memory and no block
// barrier.  Each lane finds one candidate's record before the wait (pure arithmetic), then up to eight records
// are loaded at once (their m / l words and one float4 of acc per lane) and merged in candidate order; the
// records of a second plan (residual tiles of a split launch) follow those of the first.
__global__ void __launch_bounds__(256) combine_tiles_warp_kernel(const MzDecodeParams p, const MzDecodeOut o) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // a dependent waits for this grid's completion itself
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long rows = (long long)p.s.batch * p.H;
  const int gqa = p.gqa;
  const int pair = (int)(row / gqa), h = (int)(row % gqa);
  const bool live = row < rows;
  const WorkerRange ca = live ? candidate_workers(p.tp, pair) : WorkerRange{0, -1};
  const WorkerRange cb = live ? candidate_workers(p.tp2, pair) : WorkerRange{0, -1};
  const long long first_b = p.slots_a / gqa;
  // first chunk of candidates of each plan (one per lane); nearly always the only chunk
  long long rec_a = -1, rec_b = -1;
  if (ca.first + lane <= ca.last) rec_a = record_of(p.tp, ca.first + lane, pair, 0);
  if (cb.first + lane <= cb.last) rec_b = record_of(p.tp2, cb.first + lane, pair, first_b);
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (!live) return;
  float mx = -INFINITY, lsum = 0.f;
  float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
  auto merge_chunk = [&](long long my_rec) {
    unsigned todo = __ballot_sync(0xffffffffu, my_rec >= 0);
    while (todo) {
      float mi[8], li[8];
      float4 ai[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const bool on = todo != 0;
        const int src = on ? __ffs(todo) - 1 : 0;
        if (on) todo &= todo - 1;
        const long long rec = __shfl_sync(0xffffffffu, my_rec, src);
        const long long slot = on ? rec * gqa + h : 0;
        mi[j] = on ? p.part.m[slot] : -INFINITY;
        li[j] = on ? p.part.l[slot] : 0.f;
        ai[j] = on ? *((const float4*)(p.part.acc + slot * D) + lane) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
      float m_new = mx;
#pragma unroll
      for (int j = 0; j < 8; ++j) m_new = fmaxf(m_new, mi[j]);
      const float keep = mx > -INFINITY ? __expf(mx - m_new) : 0.f;
      lsum *= keep; a.x *= keep; a.y *= keep; a.z *= keep; a.w *= keep;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float wgt = mi[j] > -INFINITY ? __expf(mi[j] - m_new) : 0.f;
        lsum = fmaf(li[j], wgt, lsum);
        a.x = fmaf(ai[j].x, wgt, a.x); a.y = fmaf(ai[j].y, wgt, a.y);
        a.z = fmaf(ai[j].z, wgt, a.z); a.w = fmaf(ai[j].w, wgt, a.w);
      }
      mx = m_new;
    }
  };
  for (long long base = ca.first; base <= ca.last; base += 32) {
    if (base != ca.first) rec_a = base + lane <= ca.last ? record_of(p.tp, base + lane, pair, 0) : -1;
    merge_chunk(rec_a);
  }
  for (long long base = cb.first; base <= cb.last; base += 32) {
    if (base != cb.first) rec_b = base + lane <= cb.last ? record_of(p.tp2, base + lane, pair, first_b) : -1;
    merge_chunk(rec_b);
  }
  const int d = 4 * lane;
  if (o.out) {
    const float den = fmaxf(lsum, 1e-20f);
    mz_store_from_float(o.out, row * D + d, a.x / den, o.out_dt);
    mz_store_from_float(o.out, row * D + d + 1, a.y / den, o.out_dt);
    mz_store_from_float(o.out, row * D + d + 2, a.z / den, o.out_dt);
    mz_store_from_float(o.out, row * D + d + 3, a.w / den, o.out_dt);
  } else {
    float* dst = o.acc + row * o.acc_stride + d;
    dst[0] = a.x; dst[1] = a.y; dst[2] = a.z; dst[3] = a.w;
    if (lane == 0) { o.m[row * o.ml_stride] = mx; o.l[row * o.ml_stride] = lsum; }
  }
}

template <int BITS, int G, int GQA>
int launch_one(const MzDecodeParams& p, cudaStream_t st) {
  auto kern = decode_tiles_kernel<BITS, G, GQA>;
  if (p.tp.smem_bytes > 48 * 1024) MZ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)p.tp.smem_bytes));
  kern<<<(unsigned)p.tp.ctas, p.tp.warps_per_cta * 32, p.tp.smem_bytes, st>>>(p);
  MZ_LAUNCH_CHECK("decode_tiles");
  return MZ_OK;
}

template <int BITS, int G>
int launch_gqa(const MzDecodeParams& p, cudaStream_t st) {
  switch (p.gqa) {
    case 1: return launch_one<BITS, G, 1>(p, st);
    case 2: return launch_one<BITS, G, 2>(p, st);
    case 4: return launch_one<BITS, G, 4>(p, st);
    case 8: return launch_one<BITS, G, 8>(p, st);
  }
  return mz_fail(MZ_ERR_UNSUPPORTED, "gqa %d", p.gqa);
}

template <int BITS>
int launch_group(const MzDecodeParams& p, cudaStream_t st) {
  switch (p.s.group) {
    case 32: return launch_gqa<BITS, 32>(p, st);
    case 64: return launch_gqa<BITS, 64>(p, st);
    case 128: return launch_gqa<BITS, 128>(p, st);
  }
  return mz_fail(MZ_ERR_UNSUPPORTED, "group %d", p.s.group);
}

template <int BITS, int G, int GQA>
void sizes_one(unsigned* per_warp, unsigned* shared, unsigned* stage) {
  *per_warp = Cfg<BITS, G, GQA>::PER_WARP;
  *shared = Cfg<BITS, G, GQA>::SHARED;
  *stage = Cfg<BITS, G, GQA>::STAGE_BYTES;
}
template <int BITS, int G>
void sizes_gqa(int gqa, unsigned* a, unsigned* b, unsigned* c) {
  if (gqa == 1) sizes_one<BITS, G, 1>(a, b, c);
  else if (gqa == 2) sizes_one<BITS, G, 2>(a, b, c);
  else if (gqa == 4) sizes_one<BITS, G, 4>(a, b, c);
  else sizes_one<BITS, G, 8>(a, b, c);
}
template <int BITS>
void sizes_group(int group, int gqa, unsigned* a, unsigned* b, unsigned* c) {
  if (group == 32) sizes_gqa<BITS, 32>(gqa, a, b, c);
  else if (group == 64) sizes_gqa<BITS, 64>(gqa, a, b, c);
  else sizes_gqa<BITS, 128>(gqa, a, b, c);
}
void sizes_any(int bits, int group, int gqa, unsigned* a, unsigned* b, unsigned* c) {
  switch (bits) {
    case 1: sizes_group<1>(group, gqa, a, b, c); break;
    case 2: sizes_group<2>(group, gqa, a, b, c); break;
    case 3: sizes_group<3>(group, gqa, a, b, c); break;
    case 4: sizes_group<4>(group, gqa, a, b, c); break;
    case 5: sizes_group<5>(group, gqa, a, b, c); break;
    case 6: sizes_group<6>(group, gqa, a, b, c); break;
    case 7: sizes_group<7>(group, gqa, a, b, c); break;
    default: sizes_group<8>(group, gqa, a, b, c); break;
  }
}
}  // namespace mzt

bool mz_decode_tiles_supported(const MzDecodeParams& p) {
  const mz_kv_store& s = p.s;
  if (s.head_dim != 128) return false;
  if (s.group != 32 && s.group != 64 && s.group != 128) return false;
  if (p.gqa != 1 && p.gqa != 2 && p.gqa != 4 && p.gqa != 8) return false;
  auto al16 = [](const void* q) { return ((uintptr_t)q & 15) == 0; };
  const int msz = s.meta_dtype == MZ_F32 ? 4 : 2;
  if (s.k_groups > 0) {
    if (!al16(s.packed_k) || !al16(s.packed_v) || !al16(s.k_mn) || !al16(s.k_scale) || !al16(s.v_mn) || !al16(s.v_scale)) return false;
    if ((s.pk_stride_b | s.pk_stride_h | s.pv_stride_b | s.pv_stride_h) & 15) return false;
    if (((s.km_stride_b | s.km_stride_h | s.vm_stride_b | s.vm_stride_h) * msz) & 15) return false;
  }
  if (s.res_len > 0) {
    if (!al16(s.res_k) || !al16(s.res_v)) return false;
    if ((s.res_stride_b | s.res_stride_h | s.res_stride_t) & 7) return false;
  }
  return true;
}

int mz_plan_tiles(MzDecodeParams& p, int splits_request, int sm_count, size_t* slots) {
  const mz_kv_store& s = p.s;
  MzTilesPlan& t = p.tp;
  unsigned per_warp = 0, shared = 0, stage = 0;
  mzt::sizes_any(s.bits, s.group, p.gqa, &per_warp, &shared, &stage);
  const unsigned budget = 220 * 1024;
  int warps = (int)((budget - shared) / per_warp);
  if (warps < 1) return mz_fail(MZ_ERR_UNSUPPORTED, "tile does not fit shared memory");
  const int max_warps = p.gqa > 4 ? 8 : 12;      // Cfg::MAX_WARPS
  if (warps > max_warps) warps = max_warps;
  t.kind = 0;
  t.stage_bytes = t.low_base = t.high_base = 0;
  t.warps_per_cta = warps;
  t.smem_per_warp = per_warp;
  t.smem_bytes = shared + per_warp * warps;
  t.packed_tiles = s.k_groups;
  t.dense_tokens = (int)(stage / (2 * mzt::D));
  const int dense_tiles = (s.res_len + t.dense_tokens - 1) / t.dense_tokens;
  t.tiles_per_pair = t.packed_tiles + dense_tiles;
  // relative cost of a packed tile of `group` tokens and of a residual tile, fitted to per-warp times
  // measured on B200 (4-bit and 2-bit caches, group 64)
  t.cost_q = s.group + 10;
  t.cost_d = t.dense_tokens + 16;
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
  // a grid that does not fill the machine is spread over all SMs (a warp alone on its scheduler is faster)
  if (W < (long long)sm_count * warps) warps = (int)((W + sm_count - 1) / sm_count);
  t.warps_per_cta = warps;
  t.smem_bytes = shared + per_warp * warps;
  t.ctas = (int)((W + warps - 1) / warps);
  // a warp's tiles start inside a cost interval of at most total_cost/W + 1
  const long long len = t.total_cost / W + 2;
  t.max_segs = (int)((len - 1) / t.pair_cost + 2);
  *slots = (size_t)W * t.max_segs * p.gqa;
  return MZ_OK;
}

int mz_launch_decode_tiles(const MzDecodeParams& p, cudaStream_t st) {
  switch (p.s.bits) {
    case 1: return mzt::launch_group<1>(p, st);
    case 2: return mzt::launch_group<2>(p, st);
    case 3: return mzt::launch_group<3>(p, st);
    case 4: return mzt::launch_group<4>(p, st);
    case 5: return mzt::launch_group<5>(p, st);
    case 6: return mzt::launch_group<6>(p, st);
    case 7: return mzt::launch_group<7>(p, st);
    case 8: return mzt::launch_group<8>(p, st);
  }
  return mz_fail(MZ_ERR_UNSUPPORTED, "bits %d", p.s.bits);
}

int mz_combine_tiles(const MzDecodeParams& p, const MzDecodeOut& o, cudaStream_t st) {
  if (p.tp.max_segs < 1) return mz_fail(MZ_ERR_ARG, "bad plan");
  // programmatic dependent launch: the merge grid may start while the main kernel drains; it finds its
  // records (pure arithmetic) and then waits for the main grid's results (griddepcontrol.wait)
  cudaLaunchConfig_t cfg = {};
  // many records per pair and few pairs: one CTA per (pair, head) with the records split over its quads
  const long long pairs = (long long)p.s.batch * p.s.kv_heads;
  const bool wide = p.tp.total_warps / pairs >= 24 && pairs * p.gqa <= 4096;
  cfg.gridDim = dim3((unsigned)(wide ? pairs * p.gqa : pairs));
  cfg.blockDim = dim3(wide ? 512 : 128 * (p.gqa < 4 ? p.gqa : 4));
  cfg.dynamicSmemBytes = 0;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  // one plan and a few records per pair (workers per pair below 8): the warp-per-row kernel
  const bool per_warp = !wide && (p.tp2.total_warps == 0 || p.hetero > 0) && p.tp.total_warps / pairs < 8;
  if (per_warp) {
    cfg.blockDim = dim3(256);
    cfg.gridDim = dim3((unsigned)((pairs * p.gqa + 7) / 8));
  }
  if (per_warp) MZ_CUDA(cudaLaunchKernelEx(&cfg, mzt::combine_tiles_warp_kernel, p, o));
  else if (wide) MZ_CUDA(cudaLaunchKernelEx(&cfg, mzt::combine_tiles_kernel<true>, p, o));
  else MZ_CUDA(cudaLaunchKernelEx(&cfg, mzt::combine_tiles_kernel<false>, p, o));
  MZ_LAUNCH_CHECK("combine_tiles");
  return MZ_OK;
}
