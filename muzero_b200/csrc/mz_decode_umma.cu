// tcgen05 / TMEM decode attention over the packed tiles of a cache: head_dim 128, group 64, 2- or 4-bit codes,
// 1/2/4 query heads per kv head (sm_100a).
//
// Same mathematics as the mma.sync kernel (mz_decode_mma.cu): the value of a code is
// A + Bup * u+[zc][e] + Bdn * u-[zc][e], the per-row constants are folded into the other operand of each
// contraction, and one 32-bit shared-memory lookup per code returns the fp16 pair (u+, u-).  What changes is
// where the contractions run: the legacy mma.sync pipe of this GPU needs 32 cycles per m16n8k16, which bounds
// that kernel; here they are tcgen05.mma instructions with the table values as the A operand in tensor memory:
//   * a warpgroup (4 warps, 128 threads) is one worker; it takes two packed tiles (128 tokens) of a
//     (batch, kv head) pair per step
//   * keys: the 128 tokens are the 128 rows (TMEM lanes) of A, a reduction block is 8 channels x {above, below
//     the zero code} = 16 fp16 = 8 TMEM columns; a thread looks up the codes of 4 tokens x 2 channels per block
//     and writes them with tcgen05.st.16x128b.x2, whose register layout is the A fragment of mma.sync.  The B
//     operand (folded query, N = 16: two tiles x 4 heads x {product, remainder}) is built in shared memory in
//     the no-swizzle K-major layout; 16 MMAs of 128x16x16 produce the logits in TMEM
//   * values: the 128 channels are the rows, a reduction block is 8 tokens; B holds the folded probabilities
//     (N = 16: two channel groups x 4 heads x {product, remainder}); the output accumulates in TMEM across
//     steps and is rescaled in place (tcgen05.ld / st) when the running maximum of a head grows
//   * online softmax state, the exchange of maxima and probabilities between the four warps, and the fold go
//     through shared memory and named barriers; MMA completion is tracked with mbarriers (tcgen05.commit), and
//     every wait on one is bounded: when it runs out the worker poisons its records (the merged output
//     becomes NaN) and carries on
// Residual (un-quantized) tiles are not handled here: the mma.sync kernel runs them in a companion launch and the
// merge kernel combines the records of both.
#include <mutex>

#include "mz_mma_common.cuh"

namespace mzu {
using namespace mzm;

constexpr int WGS = 3;                     // warpgroups (workers) per CTA
constexpr int THREADS = WGS * 128;
constexpr int TM_PER_WG = 160;             // TMEM columns of a worker: A operand 128, logits 16, output 16
constexpr int TM_A = 0, TM_L = 128, TM_O = 144;
// B operands in shared memory: per reduction block the four 8x8 core matrices (k chunk kc, n block nb) of 128
// bytes sit at kc*LBO + nb*SBO; the strides carry a skew of 16 / 32 / 64 bytes so that the folding threads' stores
// of one instruction fall into 32 different banks
constexpr int KOP_BLOCK = 544, KOP_LBO = 272, KOP_SBO = 128;
constexpr int VOP_BLOCK = 576, VOP_LBO = 288, VOP_SBO = 144;
constexpr int KOP_BYTES = 16 * KOP_BLOCK, VOP_BYTES = 16 * VOP_BLOCK;
constexpr int ZK_BYTES = 2 * 128, ZV_BYTES = 2 * 2 * 64;
constexpr int PB_HEAD = 65;                // probabilities [tile][head][65]: the odd stride spreads the softmax lanes' stores
constexpr int PB_BYTES = 2 * 4 * PB_HEAD * 4;
constexpr int RED_BYTES = 768;             // reductions between the four warps, and the two mbarriers
constexpr int SPIN_LIMIT = 4000000;

__host__ __device__ constexpr unsigned wg_bytes(unsigned stage) {
  return 4 * stage + KOP_BYTES + VOP_BYTES + ZK_BYTES + ZV_BYTES + ((PB_BYTES + 127) / 128) * 128 + RED_BYTES;
}

// ---- tcgen05 / mbarrier wrappers --------------------------------------------------------------------------------
__device__ __forceinline__ void tm_st4(uint32_t taddr, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3) {
  asm volatile("tcgen05.st.sync.aligned.16x128b.x2.b32 [%0], {%1, %2, %3, %4};" ::"r"(taddr), "r"(a0), "r"(a1), "r"(a2), "r"(a3) : "memory");
}
__device__ __forceinline__ void tm_ld_frag(uint32_t taddr, float (&c)[4]) {      // 16 lanes x 8 columns, mma.sync C-fragment layout
  uint32_t r0, r1, r2, r3;
  asm volatile("tcgen05.ld.sync.aligned.16x256b.x1.b32 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(taddr));
  c[0] = __uint_as_float(r0); c[1] = __uint_as_float(r1); c[2] = __uint_as_float(r2); c[3] = __uint_as_float(r3);
}
__device__ __forceinline__ void tm_ld_row8(uint32_t taddr, uint32_t (&v)[8]) {    // this lane's row, 8 columns
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]) : "r"(taddr));
}
__device__ __forceinline__ void tm_st_row8(uint32_t taddr, const uint32_t (&v)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
               ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]) : "memory");
}
__device__ __forceinline__ void tm_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tm_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tm_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tm_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void proxy_fence() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void wg_barrier(int wg) { asm volatile("bar.sync %0, 128;" ::"r"(wg + 1) : "memory"); }

// D[128 x 16] (+)= A[128 x 16] (TMEM) * B[16 x 16]^T (shared memory descriptor), fp16 operands, fp32 accumulate
__device__ __forceinline__ void umma(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t accumulate) {
  const uint32_t idesc = (1u << 4) | (2u << 17) | (8u << 24);     // D fp32; A, B fp16, K-major; N = 16; M = 128
  const uint32_t zero = 0;
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %6, %7, %8}, p;\n\t}\n"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(zero), "r"(zero), "r"(zero), "r"(zero) : "memory");
}
__device__ __forceinline__ uint64_t b_descriptor(uint32_t sa, int lbo, int sbo) {
  return (uint64_t)((sa >> 4) & 0x3FFF) | ((uint64_t)((lbo >> 4) & 0x3FFF) << 16) | ((uint64_t)((sbo >> 4) & 0x3FFF) << 32) | (1ull << 46);
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// waits for phase `parity` of an mbarrier with a limit; false = gave up
__device__ __forceinline__ bool bar_wait(uint32_t bar, uint32_t parity) {
  for (int it = 0; it < SPIN_LIMIT; ++it) {
    uint32_t done;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}\n"
                 : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    if (done) return true;
  }
  return false;
}

// ---- codes of one reduction block for this thread: two rows (slot 0 / 1) x four positions (4g .. 4g+3 inside the
// warp's 32), as bytes (zc << BITS | code).  4-bit: r[0] / r[1] = even / odd positions, byte = 2*slot + (pos >> 1).
// 2-bit: r[pos], byte = slot.
template <int BITS>
struct Codes4 { uint32_t r[4]; };
template <int BITS>
__device__ __forceinline__ Codes4<BITS> spread4(uint32_t x0, uint32_t x1, uint32_t z) {
  Codes4<BITS> c;
  if (BITS == 4) {
    const uint32_t w = prmt(x0, x1, 0x5410u);              // 16 bits of row 0, 16 bits of row 1
    c.r[0] = (w & 0x0F0F0F0Fu) | z;
    c.r[1] = ((w >> 4) & 0x0F0F0F0Fu) | z;
    c.r[2] = c.r[3] = 0;
  } else {
    const uint32_t w = prmt(x0, x1, 0x4440u);              // byte 0 = row 0, byte 1 = row 1
#pragma unroll
    for (int k = 0; k < 4; ++k) c.r[k] = ((w >> (2 * k)) & 0x0303u) | z;
  }
  return c;
}
// table value of (slot, position 2h + r): the A-fragment register (M tile h, row half r, column half = slot)
template <int BITS>
__device__ __forceinline__ uint32_t look(const Codes4<BITS>& c, uint32_t lane_base, int slot, int h, int r) {
  if (BITS == 4) return lds32(prmt(c.r[r], lane_base, 0x7604u | (uint32_t)((2 * slot + h) << 4)));
  return lds32(prmt(c.r[2 * h + r], lane_base, 0x7604u | (uint32_t)(slot << 4)));
}
// zero-code bytes of slot 0 / 1 (bytes b0, b0 + 1 of zreg) in the form spread4 wants
template <int BITS>
__device__ __forceinline__ uint32_t zero_bytes(uint32_t zreg, int b0) {
  if (BITS == 4) return prmt(zreg, 0u, (uint32_t)(b0 * 0x0011 + (b0 + 1) * 0x1100));   // (z0, z0, z1, z1)
  return prmt(zreg, 0u, (uint32_t)(b0 + ((b0 + 1) << 4)) | 0x4400u);                   // (z0, z1, 0, 0)
}

template <int BITS, int GQA>
__global__ void __launch_bounds__(THREADS, 1) decode_umma_kernel(const MzDecodeParams p) {
  constexpr int QB = G * BITS / 8;            // bytes of a packed key row (64 tokens)
  constexpr int CODE_BYTES = D * QB;          // packed bytes of one tile side
  constexpr int VROW = 16 * BITS;             // bytes of one token's 128 value codes
  constexpr int QUAD = BITS / 2;              // bytes holding a thread's 4 codes of one row
  extern __shared__ __align__(128) uint8_t smem[];
  const mz_kv_store& s = p.s;
  const int wg = threadIdx.x >> 7, tid = threadIdx.x & 127, w = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t0 = lane & 3;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  // ---- shared-memory layout of this worker (absolute shared-window addresses, sized by the planner)
  const int msz = s.meta_dtype == MZ_F32 ? 4 : 2;
  const uint32_t SB = p.tp.stage_bytes;
  const uint32_t base = wg == 0 ? p.tp.low_base : p.tp.high_base + (wg - 1) * wg_bytes(SB);
  const uint32_t kbuf0 = base, vbuf0 = base + 2 * SB;
  const uint32_t kop = base + 4 * SB, vop = kop + KOP_BYTES;
  const uint32_t zK = vop + VOP_BYTES, zV = zK + ZK_BYTES, pbuf = zV + ZV_BYTES;
  const uint32_t red = pbuf + ((PB_BYTES + 127) / 128) * 128;
  // the TMEM base address is kept right behind worker 0's block (the kernel has no static shared memory: its
  // buffers are addressed absolutely from the start of the dynamic region)
  const uint32_t s_tmem = p.tp.low_base + wg_bytes(SB);
  const uint32_t r_max = red, r_ca = red + 64, r_l = red + 192, r_base = red + 256, r_q = red + 384, bar_k = red + 512, bar_v = red + 520;

  if (threadIdx.x < 32) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s_tmem), "r"(512));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar_k), "r"(1));
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar_v), "r"(1));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  fill_lookup_table<BITS>(s.alpha_key, s.alpha_value);
  tm_fence_before();
  __syncthreads();
  tm_fence_after();
  const uint32_t tm_base = lds32(s_tmem);
  const uint32_t tm = tm_base + wg * TM_PER_WG;      // column base of this worker (lane field 0)
  const uint32_t tm_warp = tm + ((uint32_t)(32 * w) << 16);

  const int T = p.tp.tiles_per_pair;                  // packed tiles per (batch, kv head) pair
  const int gwg = blockIdx.x * WGS + wg;
  long long f0 = 0, f1 = 0;
  if (gwg < p.tp.total_warps) mz_warp_tiles(p.tp, gwg, &f0, &f1);

  const uint32_t lbK = TBL + lane * 4, lbV = TBL + 128 + lane * 4;
  const bool bf = s.kv_dtype == MZ_BF16;
  (void)bf;

  // ---- state of the current (batch, kv head) segment
  float m_run[GQA];          // running maximum per head (base-2 logits), identical in all threads of the worker
  float l_part = 0.f;        // sum of probabilities of this thread's tokens for head t0
  float base_part[GQA];      // sum p * A of this thread's value rows (its channel group is tid & 1)
  float qn[GQA];             // query of row d = tid, scaled by a power of two per head into [0.5, 1)
  float qs[GQA];             // logit scale per head: 2^k * scaling * log2(e)
  float qraw[GQA];           // the unscaled query values (for the constant term)
  int cur_pair = -1, seg = 0;
  uint32_t ph_k = 0, ph_v = 0;
  bool v_pending = false, first_step = true, failed = false;
#pragma unroll
  for (int h = 0; h < GQA; ++h) { m_run[h] = -INFINITY; base_part[h] = 0.f; qn[h] = qs[h] = qraw[h] = 0.f; }

  // position of a flat tile index
  auto stage_tiles = [&](long long f, int n, bool keys) {
    // n tiles starting at flat index f (same pair): codes + metadata of the keys (or values) into buffers 0 .. n-1
    const int pair = (int)(f / T), tile = (int)(f % T);
    const int b = pair / s.kv_heads, kvh = pair % s.kv_heads;
    const uint8_t* codes = keys ? s.packed_k + b * s.pk_stride_b + kvh * s.pk_stride_h : s.packed_v + b * s.pv_stride_b + kvh * s.pv_stride_h;
    const long long mbase = keys ? b * s.km_stride_b + kvh * s.km_stride_h : b * s.vm_stride_b + kvh * s.vm_stride_h;
    const uint8_t* mn = (const uint8_t*)(keys ? s.k_mn : s.v_mn);
    const uint8_t* sc = (const uint8_t*)(keys ? s.k_scale : s.v_scale);
    for (int x = 0; x < n; ++x) {
      const uint32_t dst = (keys ? kbuf0 : vbuf0) + x * SB;
      const uint8_t* src = codes + (long long)(tile + x) * CODE_BYTES;
      for (int i = tid; i < CODE_BYTES / 16; i += 128) {
        // 4-bit values: a token's row is 64 bytes; its two 32-byte halves are swapped for tokens with bit 1 set so
        // that the four tokens one load instruction touches fall into different banks
        const int di = (!keys && BITS == 4) ? (i ^ ((i >> 2) & 2)) : i;
        cp16(dst + di * 16, src + i * 16);
      }
      const long long m0 = (mbase + (long long)(tile + x) * D) * msz;
      for (int off = tid * 16; off < D * msz; off += 128 * 16) {
        cp16(dst + CODE_BYTES + off, mn + m0 + off);
        cp16(dst + CODE_BYTES + D * msz + off, sc + m0 + off);
      }
    }
  };
  auto tiles_of_step = [&](long long f) -> int {       // two tiles when the next one is in the same pair and in range
    return (f + 1 < f1 && (int)((f + 1) % T) != 0) ? 2 : 1;
  };
  auto meta_at = [&](uint32_t buf, int r, float& lo, float& span) {
    if (msz == 4) {
      lo = ldsf(buf + CODE_BYTES + r * 4);
      span = ldsf(buf + CODE_BYTES + D * 4 + r * 4);
    } else {
      lo = mz_u16_to_float((uint16_t)lds16(buf + CODE_BYTES + r * 2), s.meta_dtype);
      span = mz_u16_to_float((uint16_t)lds16(buf + CODE_BYTES + D * 2 + r * 2), s.meta_dtype);
    }
  };

  // ---- end of a segment: the partial record (m, l, acc) of this worker for the pair it just left
  auto write_partial = [&]() {
    if (v_pending) { failed |= !bar_wait(bar_v, ph_v); ph_v ^= 1; v_pending = false; }
    tm_fence_after();
    // l: over the g lanes of a warp, then over the warps
    float lsum = l_part;
#pragma unroll
    for (int off = 4; off < 32; off <<= 1) lsum += __shfl_xor_sync(0xffffffffu, lsum, off);
    if (g == 0 && t0 < GQA) stsf(r_l + (w * 4 + t0) * 4, lsum);
    // constant term of the values: over the lanes of the same channel group (lane parity), then over the warps
#pragma unroll
    for (int h = 0; h < GQA; ++h) {
      float bsum = base_part[h];
#pragma unroll
      for (int off = 2; off < 32; off <<= 1) bsum += __shfl_xor_sync(0xffffffffu, bsum, off);
      if (lane < 2) stsf(r_base + ((w * 2 + lane) * 4 + h) * 4, bsum);
    }
    wg_barrier(wg);
    const int grp = w >> 1;
    uint32_t v[8];
    tm_ld_row8(tm_warp + TM_O + 8 * grp, v);
    tm_wait_ld();
    // TMEM lane 16h' + 8r + g' of this warp holds channel 32w + 4g' + 2h' + r
    const int chan = 32 * w + 4 * (lane & 7) + 2 * (lane >> 4) + ((lane >> 3) & 1);
    const long long slot0 = ((long long)gwg * p.tp.max_segs + seg) * GQA;
    const bool in_range = MZ_IN_BOUNDS(slot0 + GQA - 1, p.part.slots, 12);   // always true outside the checked build
#pragma unroll
    for (int h = 0; h < GQA && in_range; ++h) {
      const float bs = ldsf(r_base + ((0 * 2 + grp) * 4 + h) * 4) + ldsf(r_base + ((1 * 2 + grp) * 4 + h) * 4) +
                       ldsf(r_base + ((2 * 2 + grp) * 4 + h) * 4) + ldsf(r_base + ((3 * 2 + grp) * 4 + h) * 4);
      p.part.acc[(slot0 + h) * D + chan] = __uint_as_float(v[2 * h]) + __uint_as_float(v[2 * h + 1]) + bs;
    }
    if (tid < GQA && in_range) {
      const float lt = ldsf(r_l + (0 * 4 + tid) * 4) + ldsf(r_l + (1 * 4 + tid) * 4) + ldsf(r_l + (2 * 4 + tid) * 4) + ldsf(r_l + (3 * 4 + tid) * 4);
      float mv = -INFINITY;
#pragma unroll
      for (int h = 0; h < GQA; ++h) if (h == tid) mv = m_run[h];
      p.part.m[slot0 + tid] = failed ? INFINITY : mv * (1.0f / LOG2E);   // a wait ran out: +inf turns the merged output into NaN
      p.part.l[slot0 + tid] = lt;
    }
    tm_fence_before();
    wg_barrier(wg);
  };

  if (f0 < f1) {
    long long f = f0;
    int n_cur = tiles_of_step(f);
    stage_tiles(f, n_cur, true);
    cp_async_commit();
    stage_tiles(f, n_cur, false);
    cp_async_commit();
    while (f < f1) {
      const int ntile = n_cur;
      const int pair = (int)(f / T), tile = (int)(f % T);
      const int b = pair / s.kv_heads, kvh = pair % s.kv_heads;
      const long long fn = f + ntile;
      const int n_next = fn < f1 ? tiles_of_step(fn) : 0;
      if (pair != cur_pair) {
        if (cur_pair >= 0) { write_partial(); ++seg; }
        cur_pair = pair;
        first_step = true;
        l_part = 0.f;
#pragma unroll
        for (int h = 0; h < GQA; ++h) { m_run[h] = -INFINITY; base_part[h] = 0.f; }
        // query of row d = tid for every head; per head a power of two brings max |q| into [0.5, 1) so that the
        // folded query fits fp16 whatever the row constants (<= 65504) are
        float amax[GQA];
#pragma unroll
        for (int h = 0; h < GQA; ++h) {
          qraw[h] = mz_load_as_float(p.query, b * p.q_stride_b + (long long)(kvh * GQA + h) * p.q_stride_h + tid, s.kv_dtype);
          amax[h] = fabsf(qraw[h]);
#pragma unroll
          for (int off = 1; off < 32; off <<= 1) amax[h] = fmaxf(amax[h], __shfl_xor_sync(0xffffffffu, amax[h], off));
          if (lane == 0) stsf(r_q + (w * 4 + h) * 4, amax[h]);
        }
        wg_barrier(wg);
#pragma unroll
        for (int h = 0; h < GQA; ++h) {
          const float am = fmaxf(fmaxf(ldsf(r_q + h * 4), ldsf(r_q + (4 + h) * 4)), fmaxf(ldsf(r_q + (8 + h) * 4), ldsf(r_q + (12 + h) * 4)));
          int ex = (__float_as_int(am) >> 23) & 0xff;
          ex = min(max(ex, 1), 253);
          qn[h] = qraw[h] * __int_as_float((253 - ex) << 23);
          qs[h] = __int_as_float((ex + 1) << 23) * p.scaling * LOG2E;
        }
      }
      // ================= keys: row constants and folded query of row d = tid of each tile =================
      cp_async_wait<1>();                     // this step's key tiles have landed (the value tiles may still be in flight)
      wg_barrier(wg);
      {
        float ca[2][GQA];
        bool any = false;
#pragma unroll
        for (int x = 0; x < 2; ++x) {
#pragma unroll
          for (int h = 0; h < GQA; ++h) ca[x][h] = 0.f;
          if (x < ntile) {
            float lo, span, A, Bup, Bdn;
            int zc;
            meta_at(kbuf0 + x * SB, tid, lo, span);
            row_constants<BITS>(lo, span, zc, A, Bup, Bdn);
            sts8(zK + x * 128 + (tid & 3) * 32 + (tid >> 2), (uint32_t)(zc << BITS));
            any |= A != 0.0f;
            const uint32_t dst = kop + (tid >> 3) * KOP_BLOCK + ((tid >> 2) & 1) * KOP_LBO + x * KOP_SBO + (tid & 3) * 4;
#pragma unroll
            for (int h = 0; h < GQA; ++h) {
              const float wu = qn[h] * Bup, wd = qn[h] * Bdn;
              const __half2 hi = __floats2half2_rn(wu, wd);
              const float2 hf = __half22float2(hi);
              sts32(dst + (2 * h) * 16, h2_bits(hi));
              sts32(dst + (2 * h + 1) * 16, h2_bits(__floats2half2_rn(wu - hf.x, wd - hf.y)));
              ca[x][h] = qraw[h] * A;
            }
          }
        }
        // constant term sum_d q[h][d] A_d per tile and head (rows whose range does not straddle zero)
        if (__any_sync(0xffffffffu, any)) {
#pragma unroll
          for (int x = 0; x < 2; ++x)
#pragma unroll
            for (int h = 0; h < GQA; ++h) {
              float v = ca[x][h];
#pragma unroll
              for (int off = 1; off < 32; off <<= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
              if (lane == 0) stsf(r_ca + ((w * 2 + x) * 4 + h) * 4, v);
            }
        } else if (lane < 2 * GQA) {
          stsf(r_ca + ((w * 2 + lane / GQA) * 4 + lane % GQA) * 4, 0.f);
        }
      }
      proxy_fence();
      if (v_pending) { failed |= !bar_wait(bar_v, ph_v); ph_v ^= 1; v_pending = false; }   // the A operand region is free again
      tm_fence_after();
      wg_barrier(wg);
      // ================= keys: table values of this warp's 32 tokens -> A operand =================
      {
        const int x = w >> 1, wh = w & 1;            // tile and half of the tile this warp covers
        if (x < ntile) {
          uint32_t zr[8];
          {
            const uint4 za = lds128(zK + x * 128 + t0 * 32), zb = lds128(zK + x * 128 + t0 * 32 + 16);
            zr[0] = za.x; zr[1] = za.y; zr[2] = za.z; zr[3] = za.w; zr[4] = zb.x; zr[5] = zb.y; zr[6] = zb.z; zr[7] = zb.w;
          }
          const uint32_t kb = kbuf0 + x * SB + 4 * BITS * wh + QUAD * g;
          auto load_codes = [&](int j, uint32_t& x0, uint32_t& x1) {
            if (BITS == 4) { x0 = lds16(kb + (8 * j + t0) * QB); x1 = lds16(kb + (8 * j + 4 + t0) * QB); }
            else { x0 = lds8(kb + (8 * j + t0) * QB); x1 = lds8(kb + (8 * j + 4 + t0) * QB); }
          };
          uint32_t c0, c1, n0 = 0, n1 = 0;
          load_codes(0, c0, c1);
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if (j + 1 < 16) load_codes(j + 1, n0, n1);
            const Codes4<BITS> c = spread4<BITS>(c0, c1, zero_bytes<BITS>(zr[j >> 1], 2 * (j & 1)));
#pragma unroll
            for (int h = 0; h < 2; ++h)
              tm_st4(tm_warp + ((uint32_t)(16 * h) << 16) + TM_A + 8 * j, look<BITS>(c, lbK, 0, h, 0), look<BITS>(c, lbK, 0, h, 1),
                     look<BITS>(c, lbK, 1, h, 0), look<BITS>(c, lbK, 1, h, 1));
            c0 = n0; c1 = n1;
          }
        }
      }
      tm_wait_st();
      cp_async_wait<0>();                     // this step's value tiles have landed
      tm_fence_before();
      wg_barrier(wg);
      if (tid == 0) {
        tm_fence_after();
#pragma unroll 1
        for (int j = 0; j < 16; ++j) umma(tm + TM_L, tm + TM_A + 8 * j, b_descriptor(kop + j * KOP_BLOCK, KOP_LBO, KOP_SBO), j > 0);
        umma_commit(bar_k);
      }
      if (n_next > 0) stage_tiles(fn, n_next, true);
      cp_async_commit();
      // ================= values: row constants of row (token, group) = (tid / 2, tid % 2) of each tile =================
      float vA[2], vBu[2], vBd[2];
#pragma unroll
      for (int x = 0; x < 2; ++x) {
        vA[x] = vBu[x] = vBd[x] = 0.f;
        if (x < ntile) {
          float lo, span;
          int zc;
          meta_at(vbuf0 + x * SB, tid, lo, span);
          row_constants<BITS>(lo, span, zc, vA[x], vBu[x], vBd[x]);
          const int tok = tid >> 1;
          sts8(zV + x * 128 + (tid & 1) * 64 + (tok & 3) * 16 + (tok >> 2), (uint32_t)(zc << BITS));
        }
      }
      // ================= logits of this warp's 32 tokens, softmax across the worker =================
      failed |= !bar_wait(bar_k, ph_k);
      ph_k ^= 1;
      tm_fence_after();
      float sv[4];                            // head t0; positions 2h + r of the thread's four tokens
      {
        const int x = w >> 1;
        if (x < ntile) {
          float c[2][4];
          tm_ld_frag(tm_warp + TM_L + 8 * x, c[0]);
          tm_ld_frag(tm_warp + ((uint32_t)16 << 16) + TM_L + 8 * x, c[1]);
          tm_wait_ld();
          float q_scale = 0.f;
#pragma unroll
          for (int h = 0; h < GQA; ++h) if (h == t0) q_scale = qs[h];
          const float cterm = t0 < GQA ? (ldsf(r_ca + ((0 * 2 + x) * 4 + t0) * 4) + ldsf(r_ca + ((1 * 2 + x) * 4 + t0) * 4) +
                                          ldsf(r_ca + ((2 * 2 + x) * 4 + t0) * 4) + ldsf(r_ca + ((3 * 2 + x) * 4 + t0) * 4)) * p.scaling * LOG2E
                                       : 0.f;
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            sv[2 * h] = fmaf(c[h][0] + c[h][1], q_scale, cterm);
            sv[2 * h + 1] = fmaf(c[h][2] + c[h][3], q_scale, cterm);
          }
          if (p.mask) {
            const long long m0 = b * p.mask_stride_b + (long long)(tile + x) * G + 32 * (w & 1) + 4 * g;
#pragma unroll
            for (int i = 0; i < 4; ++i) sv[i] += mz_load_as_float(p.mask, m0 + i, p.mask_dtype) * LOG2E;
          }
        } else {
          sv[0] = sv[1] = sv[2] = sv[3] = -INFINITY;
        }
        float mx = fmaxf(fmaxf(sv[0], sv[1]), fmaxf(sv[2], sv[3]));
#pragma unroll
        for (int off = 4; off < 32; off <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
        if (g == 0) stsf(r_max + (w * 4 + t0) * 4, mx);
      }
      tm_fence_before();
      wg_barrier(wg);
      float corr[GQA];
      bool grow = false;
#pragma unroll
      for (int h = 0; h < GQA; ++h) {
        const float mx = fmaxf(fmaxf(ldsf(r_max + h * 4), ldsf(r_max + (4 + h) * 4)), fmaxf(ldsf(r_max + (8 + h) * 4), ldsf(r_max + (12 + h) * 4)));
        const float m_new = fmaxf(m_run[h], mx);
        corr[h] = (m_new > -INFINITY) ? ex2f(m_run[h] - m_new) : 1.0f;     // m_run = -inf -> 0
        grow |= m_new > m_run[h];
        m_run[h] = m_new;
      }
      {
        float m_mine = -INFINITY, c_mine = 1.0f;
#pragma unroll
        for (int h = 0; h < GQA; ++h) if (h == t0) { m_mine = m_run[h]; c_mine = corr[h]; }
        const bool dead = !(m_mine > -INFINITY);
        float sum = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          sv[i] = dead ? 0.f : ex2f(sv[i] - m_mine);
          sum += sv[i];
        }
        l_part = l_part * c_mine + sum;
        const int x = w >> 1;
        if (t0 < GQA && x < ntile) {
#pragma unroll
          for (int i = 0; i < 4; ++i) stsf(pbuf + ((x * 4 + t0) * PB_HEAD + 32 * (w & 1) + 4 * g + i) * 4, sv[i]);
        }
      }
      // the output so far belongs to the old maxima: rescale it in place (all earlier value MMAs have completed: the
      // wait before the key lookups).  Nothing to do in the first step of a segment, where the accumulator is unset.
      if (grow && !first_step) {
        tm_fence_after();
        uint32_t v[8];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          tm_ld_row8(tm_warp + TM_O + 8 * half, v);
          tm_wait_ld();
#pragma unroll
          for (int c = 0; c < 8; ++c) v[c] = c / 2 < GQA ? __float_as_uint(__uint_as_float(v[c]) * corr[c / 2 < GQA ? c / 2 : 0]) : v[c];
          tm_st_row8(tm_warp + TM_O + 8 * half, v);
        }
        tm_wait_st();
      }
#pragma unroll
      for (int h = 0; h < GQA; ++h) base_part[h] *= corr[h];
      tm_fence_before();
      wg_barrier(wg);
      // ================= values: folded probabilities of row (token, group) -> B operand =================
#pragma unroll
      for (int x = 0; x < 2; ++x) {
        if (x < ntile) {
          const int tok = tid >> 1, grp = tid & 1;
          const uint32_t dst = vop + (x * 8 + (tok >> 3)) * VOP_BLOCK + ((tok >> 2) & 1) * VOP_LBO + grp * VOP_SBO + (tok & 3) * 4;
#pragma unroll
          for (int h = 0; h < GQA; ++h) {
            const float pr = ldsf(pbuf + ((x * 4 + h) * PB_HEAD + tok) * 4);
            const float wu = pr * vBu[x], wd = pr * vBd[x];
            const __half2 hi = __floats2half2_rn(wu, wd);
            const float2 hf = __half22float2(hi);
            sts32(dst + (2 * h) * 16, h2_bits(hi));
            sts32(dst + (2 * h + 1) * 16, h2_bits(__floats2half2_rn(wu - hf.x, wd - hf.y)));
            base_part[h] = fmaf(pr, vA[x], base_part[h]);
          }
        }
      }
      proxy_fence();
      // ================= values: table values of this warp's 32 channels -> A operand =================
      {
        const int grp = w >> 1;
#pragma unroll 1
        for (int x = 0; x < ntile; ++x) {
          const uint4 zr4 = lds128(zV + x * 128 + grp * 64 + t0 * 16);
          const uint32_t zr[4] = {zr4.x, zr4.y, zr4.z, zr4.w};
          // 4-bit: the warp's 16 bytes of a token row sit in 16-byte chunk w, swapped with chunk w ^ 2 for tokens with bit 1 set
          const uint32_t vb = vbuf0 + x * SB + (BITS == 4 ? ((w ^ (2 * (t0 >> 1))) * 16) : 4 * BITS * w) + QUAD * g;
          auto load_codes = [&](int j, uint32_t& x0, uint32_t& x1) {
            if (BITS == 4) { x0 = lds16(vb + (8 * j + t0) * VROW); x1 = lds16(vb + (8 * j + 4 + t0) * VROW); }
            else { x0 = lds8(vb + (8 * j + t0) * VROW); x1 = lds8(vb + (8 * j + 4 + t0) * VROW); }
          };
          uint32_t c0, c1, n0 = 0, n1 = 0;
          load_codes(0, c0, c1);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            if (j + 1 < 8) load_codes(j + 1, n0, n1);
            const Codes4<BITS> c = spread4<BITS>(c0, c1, zero_bytes<BITS>(zr[j >> 1], 2 * (j & 1)));
#pragma unroll
            for (int h = 0; h < 2; ++h)
              tm_st4(tm_warp + ((uint32_t)(16 * h) << 16) + TM_A + 64 * x + 8 * j, look<BITS>(c, lbV, 0, h, 0), look<BITS>(c, lbV, 0, h, 1),
                     look<BITS>(c, lbV, 1, h, 0), look<BITS>(c, lbV, 1, h, 1));
            c0 = n0; c1 = n1;
          }
        }
      }
      tm_wait_st();
      tm_fence_before();
      wg_barrier(wg);
      if (tid == 0) {
        tm_fence_after();
#pragma unroll 1
        for (int blk = 0; blk < 8 * ntile; ++blk)
          umma(tm + TM_O, tm + TM_A + 8 * blk, b_descriptor(vop + blk * VOP_BLOCK, VOP_LBO, VOP_SBO), !(first_step && blk == 0));
        umma_commit(bar_v);
      }
      v_pending = true;
      first_step = false;
      if (n_next > 0) stage_tiles(fn, n_next, false);
      cp_async_commit();
      f = fn;
      n_cur = n_next;
    }
    cp_async_wait<0>();
    write_partial();
  }
  tm_fence_before();
  __syncthreads();
  if (threadIdx.x < 32) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tm_base), "r"(512));
}

template <int BITS, int GQA>
int launch_one(const MzDecodeParams& p, cudaStream_t st) {
  auto kern = decode_umma_kernel<BITS, GQA>;
  MZ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)p.tp.smem_bytes));
  kern<<<(unsigned)p.tp.ctas, THREADS, p.tp.smem_bytes, st>>>(p);
  MZ_LAUNCH_CHECK("decode_umma");
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
}  // namespace mzu


bool mz_decode_umma_supported(const MzDecodeParams& p) {
  return mz_decode_mma_supported(p) && p.s.k_groups > 0;
}

// Plan of the packed tiles for the tcgen05 kernel (p.tp, workers = warpgroups) and, when there is a residual
// window, of the residual tiles for the companion launch of the mma.sync kernel (p.tp2); the records of the
// second plan follow those of the first in the workspace.
int mz_plan_umma(MzDecodeParams& p, int splits_request, int sm_count, size_t* slots) {
  const mz_kv_store& s = p.s;
  MzTilesPlan& t = p.tp;
  const int msz = s.meta_dtype == MZ_F32 ? 4 : 2;
  unsigned sb = mzm::D * (mzm::G * s.bits / 8) + 2 * mzm::D * msz;
  sb = (sb + 127u) & ~127u;
  const unsigned table_bytes = (1u << (2 * s.bits)) * 256u;
  const unsigned wb = (unsigned)mz_smem_window_base();
  const unsigned wgb = mzu::wg_bytes(sb);
  t = MzTilesPlan{};
  t.kind = 2;
  t.stage_bytes = sb;
  t.low_base = (wb + 127u) & ~127u;
  t.high_base = mzm::TBL + table_bytes;
  if (t.low_base + wgb + 16 > mzm::TBL || t.high_base + 2 * wgb > wb + 227u * 1024u)
    return mz_fail(MZ_ERR_UNSUPPORTED, "tile does not fit shared memory");
  t.packed_tiles = s.k_groups;
  t.dense_tokens = 0;
  t.tiles_per_pair = s.k_groups;
  t.cost_q = 1;
  t.cost_d = 1;
  const long long pairs = (long long)s.batch * s.kv_heads;
  t.total_tiles = pairs * t.tiles_per_pair;
  t.pair_cost = t.tiles_per_pair;
  t.total_cost = t.total_tiles;
  if (t.total_cost >= (1LL << 31)) return mz_fail(MZ_ERR_UNSUPPORTED, "cache too large for the tiled kernel");
  long long W;
  if (splits_request > 0) {
    W = pairs * splits_request;
  } else {
    W = (long long)sm_count * mzu::WGS;             // one resident CTA per SM
    const long long steps = (t.total_tiles + 1) / 2;  // at least one step of two tiles per worker
    if (W > steps) W = steps;
    if (W < 1) W = 1;
  }
  if (W > (1LL << 30)) return mz_fail(MZ_ERR_ARG, "too many splits");
  t.total_warps = (int)W;
  t.cost_quot = (unsigned)(t.total_cost / W);
  t.cost_rem = (unsigned)(t.total_cost % W);
  t.warps_per_cta = mzu::WGS * 4;
  t.smem_per_warp = wgb / 4;
  t.smem_bytes = t.high_base + 2 * wgb - wb;
  t.ctas = (int)((W + mzu::WGS - 1) / mzu::WGS);
  const long long len = t.total_cost / W + 2;
  t.max_segs = (int)((len - 1) / t.pair_cost + 2);
  size_t slots_a = (size_t)W * t.max_segs * p.gqa;
  p.slots_a = (long long)slots_a;
  p.tp2 = MzTilesPlan{};
  size_t slots_b = 0;
  if (s.res_len > 0) {
    // the residual tiles alone, as a plan of the mma.sync kernel: the same arithmetic with zero packed tiles
    MzDecodeParams q = p;
    q.s.k_groups = 0;
    int rc = mz_plan_mma(q, splits_request > 0 ? 1 : 0, sm_count, &slots_b);
    if (rc) return rc;
    p.tp2 = q.tp;
  }
  *slots = slots_a + slots_b;
  return MZ_OK;
}

int mz_launch_decode_umma(const MzDecodeParams& p, cudaStream_t st) {
  if (p.tp2.total_warps > 0) {
    // residual tiles: the mma.sync kernel on its own plan, records behind those of the packed tiles
    MzDecodeParams q = p;
    q.tp = p.tp2;
    q.part.m = p.part.m + p.slots_a;
    q.part.l = p.part.l + p.slots_a;
    q.part.acc = p.part.acc + p.slots_a * p.s.head_dim;
    q.part.slots = p.part.slots - (long long)p.slots_a;
    int rc = mz_launch_decode_mma(q, st);
    if (rc) return rc;
  }
  if (p.s.bits == 4) return mzu::launch_gqa<4>(p, st);
  if (p.s.bits == 2) return mzu::launch_gqa<2>(p, st);
  return mz_fail(MZ_ERR_UNSUPPORTED, "bits %d", p.s.bits);
}
