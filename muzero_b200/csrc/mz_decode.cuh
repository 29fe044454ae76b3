// Shared declarations of the decode-attention kernels.
#pragma once
#include "mz_store.cuh"

// Partial results of one sequence split: slot = (b*H + h) * splits + split.
struct MzPartials {
  float* m;    // [B*H*splits]       running maximum of the scaled logits
  float* l;    // [B*H*splits]       sum of exp(logit - m)
  float* acc;  // [B*H*splits*D]     sum of exp(logit - m) * V
};

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
};

// generic kernel: any bits / group / head_dim<=512 / gqa<=16
int mz_launch_decode_generic(const MzDecodeParams& p, cudaStream_t st);
// tuned kernel: head_dim 128, group in {32,64,128}, gqa in {1,2,4,8}; returns MZ_ERR_UNSUPPORTED otherwise
int mz_launch_decode_tiles(const MzDecodeParams& p, cudaStream_t st);
bool mz_decode_tiles_supported(const MzDecodeParams& p);

// units of work a call is split over (sequence positions / unit size), per kernel family
int mz_decode_units_generic(const mz_kv_store& s);
int mz_decode_units_tiles(const mz_kv_store& s);
