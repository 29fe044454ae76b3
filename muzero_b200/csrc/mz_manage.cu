// Store management: batch re-indexing of a whole layer cache in one launch (beam-search reorder, batch
// selection, batch repetition).  The reference does this with eight tensor-indexing calls per layer.
#include "mz_store.cuh"

namespace {
// One of the eight tensors of a cache: per (batch, kv head) `bytes` valid bytes starting `offset` bytes into
// the (b, h) block; blocks are `stride_b` / `stride_h` bytes apart in source and destination.
struct Segment {
  const uint8_t* src; uint8_t* dst;
  long long src_sb, src_sh, dst_sb, dst_sh;
  long long bytes;
};
struct GatherParams {
  Segment seg[8];
  int n_seg, kv_heads, dst_batch, src_batch;
  const long long* index;   // dst batch entry i takes source entry index[i]
  int* status;              // set to 1 when an index is out of range (that entry is skipped)
};

// grid: (chunks of 4 KB of one (b, h) block, dst_batch * kv_heads, segment)
__global__ void __launch_bounds__(256) gather_batch_kernel(const GatherParams p) {
  const Segment& sg = p.seg[blockIdx.z];
  const long long first = (long long)blockIdx.x * 4096;
  if (first >= sg.bytes) return;
  const int h = blockIdx.y % p.kv_heads, b = blockIdx.y / p.kv_heads;
  const long long sb = p.index[b];
  if (sb < 0 || sb >= p.src_batch) {
    if (threadIdx.x == 0) atomicExch(p.status, 1);
    return;
  }
  const uint8_t* src = sg.src + sb * sg.src_sb + h * sg.src_sh;
  uint8_t* dst = sg.dst + b * sg.dst_sb + h * sg.dst_sh;
  const long long end = min(sg.bytes, first + 4096);
  if ((((uintptr_t)src | (uintptr_t)dst | (uintptr_t)sg.bytes) & 15) == 0) {
    for (long long i = first + threadIdx.x * 16; i < end; i += 256 * 16) *(uint4*)(dst + i) = *(const uint4*)(src + i);
  } else {
    for (long long i = first + threadIdx.x; i < end; i += 256) dst[i] = src[i];
  }
}
}  // namespace

// dst := src re-indexed along the batch: entry i of dst is entry index[i] of src (index on the device, int64).
// Copies the valid part of all eight tensors: packed codes and metadata of keys and values, and the
// residual window (which lands at the front of dst's window buffers).  dst must have the capacities it
// needs; its counters are set by the caller (they equal src's, with res_start = 0).  *status (device int,
// zeroed by the caller) is set to 1 if an index was out of range.
extern "C" int mz_store_gather_batch(const mz_kv_store* src, const mz_kv_store* dst, const long long* index, int* status,
                                     void* stream) {
  MZ_RANGE("mz_store_gather_batch");
  int rc = mz_check_store_basic(src);
  if (rc) return rc;
  if ((rc = mz_check_store_basic(dst))) return rc;
  MZ_REQUIRE(index != nullptr && status != nullptr, "NULL index / status");
  MZ_REQUIRE(src->kv_heads == dst->kv_heads && src->head_dim == dst->head_dim && src->group == dst->group && src->bits == dst->bits &&
                 src->meta_dtype == dst->meta_dtype && src->kv_dtype == dst->kv_dtype,
             "source and destination caches differ in shape or types");
  const MzStoreGeom g = mz_geom(*src);
  const long long msz = mz_dtype_size(g.meta_dt), esz = 2;
  GatherParams p = {};
  p.kv_heads = g.KVH; p.dst_batch = dst->batch; p.src_batch = src->batch; p.index = index; p.status = status;
  long long max_bytes = 0;
  auto add = [&](const void* s, void* d, long long ssb, long long ssh, long long dsb, long long dsh, long long bytes) {
    if (bytes <= 0) return;
    Segment& sg = p.seg[p.n_seg++];
    sg.src = (const uint8_t*)s; sg.dst = (uint8_t*)d;
    sg.src_sb = ssb; sg.src_sh = ssh; sg.dst_sb = dsb; sg.dst_sh = dsh; sg.bytes = bytes;
    if (bytes > max_bytes) max_bytes = bytes;
  };
  if (src->k_groups > 0 || src->v_tokens > 0) {
    if ((rc = mz_check_store_quantized(src))) return rc;
    if ((rc = mz_check_store_quantized(dst))) return rc;
    const long long kb = (long long)src->k_groups * g.D * g.QB, km = (long long)src->k_groups * g.D * msz;
    const long long vb = (long long)src->v_tokens * g.NG * g.QB, vm = (long long)src->v_tokens * g.NG * msz;
    add(src->packed_k, dst->packed_k, src->pk_stride_b, src->pk_stride_h, dst->pk_stride_b, dst->pk_stride_h, kb);
    add(src->k_mn, dst->k_mn, src->km_stride_b * msz, src->km_stride_h * msz, dst->km_stride_b * msz, dst->km_stride_h * msz, km);
    add(src->k_scale, dst->k_scale, src->km_stride_b * msz, src->km_stride_h * msz, dst->km_stride_b * msz, dst->km_stride_h * msz, km);
    add(src->packed_v, dst->packed_v, src->pv_stride_b, src->pv_stride_h, dst->pv_stride_b, dst->pv_stride_h, vb);
    add(src->v_mn, dst->v_mn, src->vm_stride_b * msz, src->vm_stride_h * msz, dst->vm_stride_b * msz, dst->vm_stride_h * msz, vm);
    add(src->v_scale, dst->v_scale, src->vm_stride_b * msz, src->vm_stride_h * msz, dst->vm_stride_b * msz, dst->vm_stride_h * msz, vm);
  }
  if (src->res_len > 0) {
    if ((rc = mz_check_store_residual(src))) return rc;
    if ((rc = mz_check_store_residual(dst))) return rc;
    MZ_REQUIRE(src->res_stride_t == g.D && dst->res_stride_t == g.D, "residual windows must be dense in (token, channel)");
    const long long rb = (long long)src->res_len * g.D * esz;
    const long long so = (long long)src->res_start * g.D * esz, d0 = (long long)dst->res_start * g.D * esz;
    add((const uint8_t*)src->res_k + so, (uint8_t*)dst->res_k + d0, src->res_stride_b * esz, src->res_stride_h * esz,
        dst->res_stride_b * esz, dst->res_stride_h * esz, rb);
    add((const uint8_t*)src->res_v + so, (uint8_t*)dst->res_v + d0, src->res_stride_b * esz, src->res_stride_h * esz,
        dst->res_stride_b * esz, dst->res_stride_h * esz, rb);
  }
  if (p.n_seg == 0) return MZ_OK;
  const long long chunks = (max_bytes + 4095) / 4096, pairs = (long long)dst->batch * g.KVH;
  MZ_REQUIRE(chunks < (1LL << 31) && pairs < 65536, "cache too large for one gather launch");
  gather_batch_kernel<<<dim3((unsigned)chunks, (unsigned)pairs, (unsigned)p.n_seg), 256, 0, (cudaStream_t)stream>>>(p);
  MZ_LAUNCH_CHECK("gather_batch");
  return MZ_OK;
}
