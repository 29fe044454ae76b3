// Shared declarations of the decode-attention kernels.
#pragma once
#include "mz_store.cuh"

// Partial results (un-normalised softmax state) written by the main kernels:
//   m   running maximum of the scaled logits      l   sum of exp(logit - m)
//   acc sum of exp(logit - m) * V
// generic kernel : slot = (b*H + h) * splits + split
// tiled kernel   : slot = (warp * max_segs + seg) * gqa + head_in_group
struct MzPartials {
  float* m;
  float* l;
  float* acc;  // [slots][D]
  long long slots;   // records the three arrays hold (read by the checked build only)
};

// Work decomposition of the tiled kernel: the flat list of (pair, tile) items, pair = b*KVH+kvh,
// is cut into `total_warps` contiguous ranges, one per warp.
struct MzTilesPlan {
  int total_warps, warps_per_cta, ctas, max_segs;
  int tiles_per_pair;      // k_groups packed tiles + ceil(res_len / dense_tokens) residual tiles
  long long total_tiles;   // pairs * tiles_per_pair
  unsigned smem_bytes, smem_per_warp;
  // Work is cut into per-warp ranges by cost, not by tile count: a packed tile of G tokens costs
  // cost_q, a residual tile of dense_tokens un-quantized tokens costs cost_d.
  int packed_tiles, dense_tokens, cost_q, cost_d;
  long long pair_cost, total_cost;   // packed_tiles*cost_q + dense_tiles*cost_d ; pairs * pair_cost (< 2^31)
  unsigned cost_quot, cost_rem;      // total_cost / total_warps and the remainder
  // which main kernel the plan is for (0: SIMT tiled kernel, 1: tensor-core kernel) and, for the latter,
  // its per-warp staging size and the shared-window addresses of its two buffer pools
  int kind;
  unsigned stage_bytes, low_base, high_base;
};

// Number of tiles (in flat order: pair-major, packed tiles before residual tiles) whose start cost
// is below `c`.  Warp g owns the tiles [mz_tiles_before(g*total_cost/W), mz_tiles_before((g+1)*total_cost/W)).
// total_cost < 2^31 (checked by the planner), so everything but g*total_cost fits 32 bits; with fewer
// than 65536 warps that product is split as g*quot + g*rem/W and the whole computation uses 32-bit
// divisions (a 64-bit division costs hundreds of cycles on the device).
__host__ __device__ inline long long mz_tiles_before(const MzTilesPlan& t, unsigned c) {
  const unsigned pc = (unsigned)t.pair_cost, cq = (unsigned)t.cost_q, cd = (unsigned)t.cost_d;
  const unsigned pair = c / pc, r = c - pair * pc;
  const unsigned qcost = (unsigned)t.packed_tiles * cq;
  const unsigned in = r <= qcost ? (r + cq - 1) / cq : (unsigned)t.packed_tiles + (r - qcost + cd - 1) / cd;
  return (long long)pair * t.tiles_per_pair + in;
}
__host__ __device__ inline unsigned mz_cost_at(const MzTilesPlan& t, long long g) {
  if (t.total_warps < 65536) return (unsigned)g * t.cost_quot + (unsigned)g * t.cost_rem / (unsigned)t.total_warps;
  return (unsigned)((unsigned long long)g * (unsigned long long)t.total_cost / (unsigned long long)t.total_warps);
}
__host__ __device__ inline void mz_warp_tiles(const MzTilesPlan& t, long long g, long long* f0, long long* f1) {
  const unsigned c0 = mz_cost_at(t, g);
  *f0 = mz_tiles_before(t, c0);
  if (g + 1 >= t.total_warps) { *f1 = t.total_tiles; return; }
  *f1 = mz_tiles_before(t, mz_cost_at(t, g + 1));
}

struct MzDecodeParams {
  mz_kv_store s;
  int H, gqa, splits;
  const void* query; long long q_stride_b, q_stride_h;
  float scaling;
  const void* mask; int mask_dtype; long long mask_stride_b;
  MzPartials part;
  int QB, NG;
  const float* table_k;  // exact expand tables (generic kernel)
  const float* table_v;
  float eps;
  // value prefix tokens beyond the key prefix (logq_compatible_layout): the first v_lead tokens of the residual
  // window have their values in the packed store (rows k_groups*G ..), the rest in the dense window
  int v_lead;
  MzTilesPlan tp;
  // tcgen05 route: the packed tiles run on plan `tp`, the residual tiles on plan `tp2` (mma.sync kernel,
  // total_warps == 0 when there is no residual window); the records of tp2 start at record slots_a
  MzTilesPlan tp2;
  long long slots_a;
  // tensor-core kernel: the lookup-table entries in global memory (built once per device and (bits, alphas));
  // nullptr = every CTA computes them itself
  const unsigned* lut;
  // tensor-core kernel, one launch over two plans: CTAs [0, hetero) work on plan `tp` (packed tiles only), the
  // rest on plan `tp2` (residual tiles only, records from slots_a on).  0 = one plan per launch.
  int hetero;
};

// where a call's result goes: normalised output, or the merged (m, l, acc) triple.  The triple is addressed
// with strides so that it can be written as separate arrays (acc_stride = D, ml_stride = 1) or as one packed
// record per row, [acc[D], m, l] (acc_stride = ml_stride = D + 2, m = acc + D, l = acc + D + 1).
struct MzDecodeOut {
  void* out; int out_dt;
  float* m; float* l; float* acc;
  long long acc_stride, ml_stride;
};

// A validated call: which kernel runs, its parameters, the partial records and scratch bytes it needs.
struct MzDecodePlan {
  MzDecodeParams p;
  bool tiles;
  size_t slots;     // partial records
  size_t ws_bytes;
};
// validation + planning of mz_decode_attention(a), and the launches of an existing plan
int mz_decode_plan(const mz_decode_args* a, MzDecodePlan* plan);
int mz_decode_run_plan(const mz_decode_args* a, MzDecodePlan* plan, cudaStream_t st);

// generic kernel: any bits / group / head_dim<=512 / gqa<=16
int mz_launch_decode_generic(const MzDecodeParams& p, cudaStream_t st);
int mz_decode_units_generic(const mz_kv_store& s);

// tiled kernel: head_dim 128, group in {32,64,128}, gqa in {1,2,4,8}, 16-byte aligned store
bool mz_decode_tiles_supported(const MzDecodeParams& p);
int mz_plan_tiles(MzDecodeParams& p, int splits_request, int sm_count, size_t* slots);
int mz_launch_decode_tiles(const MzDecodeParams& p, cudaStream_t st);
int mz_combine_tiles(const MzDecodeParams& p, const MzDecodeOut& o, cudaStream_t st);

// tensor-core kernel: head_dim 128, group 64, 2- or 4-bit codes, gqa in {1,2,4}; shares the partition,
// the partial records and the merge kernel with the tiled kernel
bool mz_decode_mma_supported(const MzDecodeParams& p);
int mz_plan_mma(MzDecodeParams& p, int splits_request, int sm_count, size_t* slots);
int mz_launch_decode_mma(const MzDecodeParams& p, cudaStream_t st);
int mz_smem_window_base();

// tcgen05 kernel (A operand in tensor memory): the packed tiles of head_dim 128 / group 64 / 2- or 4-bit caches;
// the residual tiles go to the mma.sync kernel in a companion launch
bool mz_decode_umma_supported(const MzDecodeParams& p);
int mz_plan_umma(MzDecodeParams& p, int splits_request, int sm_count, size_t* slots);
int mz_launch_decode_umma(const MzDecodeParams& p, cudaStream_t st);
