/*
 * muzero_b200 — C ABI of the B200 (sm_100a) KV-cache hot path.
 *
 * Every entry point takes raw device pointers, explicit sizes/strides and a
 * CUDA stream (passed as void*; NULL = legacy default stream), launches
 * asynchronously on that stream and returns an int status (0 = MZ_OK).
 * The callee never retains caller pointers and never allocates per call;
 * small per-device lookup tables are created on the first call that needs
 * them (a synchronous cudaMalloc + copy, so make that first call outside any
 * stream capture).  On a non-zero status mz_last_error() returns the text.
 *
 * Each declaration cites the interface of the reference (muZeroQuant/muZero,
 * paths inside that project) that it replaces.
 */
#ifndef MUZERO_B200_H
#define MUZERO_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* status codes */
#define MZ_OK 0
#define MZ_ERR_ARG 1          /* bad pointer / size / stride / alignment */
#define MZ_ERR_UNSUPPORTED 2  /* valid request this build has no kernel for */
#define MZ_ERR_CUDA 3         /* a CUDA runtime call failed */
#define MZ_ERR_WORKSPACE 4    /* workspace missing or too small */

/* element types */
#define MZ_F32 0
#define MZ_F16 1
#define MZ_BF16 2

/* Library version (major*10000 + minor*100 + patch). */
int mz_version(void);

/* Copies the calling thread's last error text into buf (NUL terminated); returns its length. */
int mz_last_error(char* buf, int len);

/*
 * Installs the compander-inverse table used by mz_dequantize_rows /
 * mz_dequantize_kv for (bits, alpha) on the current device:
 *   table[denom * (2^bits) + numer] = expm1(clamp(numer/denom,0,1) * log1p(alpha)) / alpha   (fp32)
 * Optional: without it the library builds the table itself in double
 * precision, which differs from a given libm's fp32 expm1 in the last bit of
 * a few entries.  A host that must match torch bit for bit passes torch's.
 * Replaces: the constant table MU_ZERO_ALPHA2_COMPAND and expm1f calls of
 * muzero/kernels/loader.py:133-150,197-225; values per muzero/quantizer.py:249-253.
 */
int mz_set_expand_table(int bits, float alpha, const float* host_table);

/*
 * Row quantizer: x[n_rows, group] (x_dtype) -> packed[n_rows, ceil(group*bits/8)],
 * mn[n_rows], scale[n_rows] (meta_dtype).  bits 1..8.  Arithmetic follows the
 * reference's torch backend (one rounding to x_dtype per op, log1p(alpha) kept
 * in fp32): codes and metadata are bit-exact for bf16/fp16 input.
 * Replaces: mu_zero_quantize_cuda, muzero/kernels/loader.py:268-351,1290-1322 and
 * the Triton pack kernel muzero/kernels/muzero_triton.py:29-104;
 * arithmetic per muzero/quantizer.py:161-202.
 */
int mz_quantize_rows(const void* x, int x_dtype, long long n_rows, int group, int bits,
                     float alpha, float eps, uint8_t* packed, void* mn, void* scale,
                     int meta_dtype, void* stream);

/*
 * Row dequantizer: inverse of mz_quantize_rows, fp32 arithmetic, out[n_rows, group] (out_dtype).
 * Replaces: mu_zero_dequantize_cuda, muzero/kernels/loader.py:356-383,1324-1358;
 * arithmetic per muzero/quantizer.py:229-266.
 */
int mz_dequantize_rows(const uint8_t* packed, const void* mn, const void* scale, int meta_dtype,
                       long long n_rows, int group, int bits, float alpha, float eps,
                       void* out, int out_dtype, void* stream);

/*
 * The quantized store of one layer plus its dense residual window.
 * Layouts (reference: muzero/cache/layer.py:271-301):
 *   packed_k [B,KVH,k_group_cap,D,QB] u8     row = G consecutive tokens of one channel
 *   k_mn,k_scale [B,KVH,k_group_cap,D]       meta_dtype
 *   packed_v [B,KVH,v_token_cap,NG,QB] u8    row = G consecutive channels of one token, NG=ceil(D/G)
 *   v_mn,v_scale [B,KVH,v_token_cap,NG]      meta_dtype
 *   res_k,res_v  [B,KVH,res_cap,D]           kv_dtype (bf16/fp16), innermost contiguous
 * Inside one (b,kvh) every store tensor is contiguous; *_stride_b / *_stride_h
 * give the distance between batches / heads (bytes for packed_*, elements otherwise).
 */
typedef struct mz_kv_store {
  int batch, kv_heads, head_dim;
  int group, bits;
  int meta_dtype, kv_dtype;
  float alpha_key, alpha_value;
  uint8_t* packed_k; void* k_mn; void* k_scale;
  long long pk_stride_b, pk_stride_h, km_stride_b, km_stride_h;
  uint8_t* packed_v; void* v_mn; void* v_scale;
  long long pv_stride_b, pv_stride_h, vm_stride_b, vm_stride_h;
  int k_groups;   /* quantized key groups currently valid   */
  int v_tokens;   /* quantized value tokens currently valid */
  void* res_k; void* res_v;
  long long res_stride_b, res_stride_h, res_stride_t;  /* elements */
  int res_start;  /* index of the oldest residual token in res_k/res_v */
  int res_len;    /* residual tokens currently valid */
} mz_kv_store;

/*
 * Residual-window flush: quantizes the n_tokens oldest residual tokens
 * (n_tokens a multiple of group) and writes them into the store at key group
 * k_groups and value token v_tokens, in one launch for K (transposed,
 * grouped over tokens) and V (grouped over channels).  The caller then
 * advances k_groups / v_tokens / res_start / res_len itself.
 * Replaces: compress_residual_prefix + _quantize_key_block + _quantize_value_block +
 * _append_{key,value}_quantized, muzero/cache/layer.py:271-301,351-401 (the
 * permute/contiguous copy, the quantize launches and the torch.cat of the store).
 */
int mz_flush_kv(const mz_kv_store* store, int n_tokens, float eps, void* stream);

/*
 * The same flush with separate extents for keys and values: the n_key_tokens oldest residual tokens
 * (a multiple of group) go to key group k_groups.., the residual rows [value_first, value_first +
 * n_value_tokens) go to value tokens v_tokens...  For the reference's `logq_compatible_layout`, where
 * every value token beyond the residual length is flushed while keys flush by whole groups, so the
 * value prefix runs ahead of the key prefix (muzero/cache/layer.py:389-396).
 */
int mz_flush_kv_parts(const mz_kv_store* store, int n_key_tokens, int value_first, int n_value_tokens, float eps,
                      void* stream);

/*
 * Appends one token per (b,kvh) to the residual window at index res_start+res_len:
 * k_new,v_new [B,KVH,1,D] with element strides (new_stride_b,new_stride_h).
 * Replaces: the two single-token buffer copies of _append_dense, muzero/cache/layer.py:183-193.
 */
int mz_append_kv(const mz_kv_store* store, const void* k_new, const void* v_new,
                 long long new_stride_b, long long new_stride_h, void* stream);

/*
 * Dequantizes store key groups [g0,g1) into out_k[B,KVH,(g1-g0)*G,D] and value
 * tokens [t0,t1) into out_v[B,KVH,t1-t0,D] (contiguous, out_dtype); either
 * output may be NULL.  Bit-exact with the reference's fp32 dequantizer.
 * Replaces: _dequantize_{key,value}_{prefix,range}, muzero/cache/layer.py:303-345
 * (dequantize launch + un-permute copy).
 */
int mz_dequantize_kv(const mz_kv_store* store, int g0, int g1, void* out_k,
                     int t0, int t1, void* out_v, int out_dtype, float eps, void* stream);

/*
 * Re-indexes a whole layer cache along the batch in one launch: entry i of dst takes entry index[i] of
 * src (index: int64 on the device), for the valid part of all eight tensors (packed codes and metadata
 * of keys and values, residual window).  dst has the same shape parameters, its own buffers with the
 * capacities it needs, and res_start where the window shall land; the caller sets dst's counters
 * (k_groups, v_tokens, res_len as in src).  *status (a device int the caller zeroed) becomes 1 if an
 * index lies outside [0, src->batch); that entry is skipped.
 * Replaces: the per-tensor indexing of reorder_cache / batch_select_indices / batch_repeat_interleave,
 * muzero/cache/layer.py:508-523.
 */
int mz_store_gather_batch(const mz_kv_store* src, const mz_kv_store* dst, const long long* index, int* status,
                          void* stream);

/* One decode-attention call. */
typedef struct mz_decode_args {
  mz_kv_store store;
  int q_heads;                       /* multiple of store.kv_heads */
  const void* query;                 /* [B,H,1,D] kv_dtype */
  long long q_stride_b, q_stride_h;  /* elements */
  float scaling;
  const void* mask;                  /* NULL or additive [B,1,1,>=k_groups*G+res_len] */
  int mask_dtype;
  long long mask_stride_b;           /* elements */
  void* out;                         /* [B,1,H,D] contiguous */
  int out_dtype;                     /* MZ_BF16 / MZ_F16 / MZ_F32 */
  int splits;                        /* 0 = choose; else sequence splits per (b,kvh) */
  void* workspace; size_t workspace_bytes;
} mz_decode_args;

/*
 * Testing aid: selects the decode-attention kernel for later calls of this process and returns the previous
 * selection.  0 = automatic, 1 = shape-generic kernel, 2 = SIMT tiled kernel (no tensor cores), 3 = automatic,
 * 4 = tcgen05 / tensor-memory kernel where it applies (head_dim 128, group 64, 2- or 4-bit codes).  The
 * environment variable MZ_DECODE_KERNEL = generic | tiles | mma | umma gives the initial selection.  Workspace
 * sizes depend on the selection: query them again after changing it.  No counterpart in the reference, which
 * picks its kernels by shape only (muzero/kernels/loader.py:1382-1440).
 */
int mz_debug_force_kernel(int which);

/*
 * Testing aid of the checked build (library compiled with -DMZ_BOUNDS): the number of guarded global
 * accesses on the current device that fell outside the extent the host passed and were skipped; the
 * index, extent and site number of the first one go to the optional pointers; `reset` != 0 clears the
 * record.  Synchronizes the device.  Returns -1 from a library built without the flag, -2 when the
 * record cannot be read.  Every entry point also opens an NVTX range named after itself.  No counterpart
 * in the reference, whose kernels carry no bounds assertions (muzero/kernels/loader.py).
 */
long long mz_bounds_violations(long long* first_index, long long* first_extent, int* first_site, int reset);

/* Bytes of workspace mz_decode_attention needs for these arguments (splits resolved as the call would). */
size_t mz_decode_workspace_bytes(const mz_decode_args* args);

/*
 * Bytes of workspace that suffice for mz_decode_attention / mz_decode_step with this batch, head
 * counts, head_dim and `splits`, whatever the number of cached tokens: a host that keeps one argument
 * block per layer sizes its scratch once with this instead of asking before every step.  0 = invalid
 * arguments.  Replaces: the per-call allocations of partial buffers in muzero/cache/attention.py:107-109,130-132.
 */
size_t mz_decode_workspace_bound(const mz_decode_args* args);

/*
 * Fused decode attention over packed K/V + residual window with GQA:
 * QK, online softmax, AV per sequence split, then a deterministic
 * log-sum-exp combine.  fp32 accumulation throughout.
 * Replaces: mu_zero_decode_attention_forward's device work,
 * muzero/cache/attention.py:104-151,186-201,229-239,248-263,286-290 — i.e. the
 * qk / av / prefix_decode / prefix_decode_chunked entry points of
 * muzero/kernels/loader.py:86-93 and the torch matmul/cat/softmax between them.
 */
int mz_decode_attention(const mz_decode_args* args, void* stream);

/*
 * One decode step of one layer in a single call: mz_append_kv of the new token, then -- when the
 * residual window exceeds `residual_length` by at least `flush_unit` tokens (a multiple of the group
 * size: one group, or four in the reference's default decode mode) -- mz_flush_kv of
 * floor(excess / flush_unit) * flush_unit oldest tokens, then mz_decode_attention.  The counters of
 * args->store (k_groups, v_tokens, res_start, res_len) are advanced in place; the caller mirrors them.
 * Capacities are the caller's: `window_capacity` rows behind store.res_k/res_v, `group_capacity` key
 * groups (and group_capacity * group value tokens) in the packed store; MZ_ERR_WORKSPACE, with nothing
 * launched, when the step would not fit.  alpha_key / alpha_value must already be chosen.
 * Replaces the per-token host sequence MuZeroCacheLayer.update -> compress_residual_prefix ->
 * mu_zero_decode_attention_forward, muzero/cache/layer.py:407-459,369-401 and
 * muzero/cache/attention.py:48-295 (callers: muzero/integrations/transformers_patch.py:529-592).
 */
int mz_decode_step(mz_decode_args* args, const void* k_new, const void* v_new, long long new_stride_b,
                   long long new_stride_h, int residual_length, int flush_unit, int group_capacity,
                   int window_capacity, float eps, void* stream);

/* Bytes of workspace mz_decode_step needs: those of mz_decode_attention on the store as it will be
 * after the append and the flush of the step (0 on invalid arguments). */
size_t mz_decode_step_workspace_bytes(const mz_decode_args* args, int residual_length, int flush_unit);

/*
 * Decode attention for callers that cannot allocate device memory.
 * (No counterpart in the reference: its kernels always receive torch-allocated buffers.)
 *
 * Some hosts of this library may not call cudaMalloc at all once they are running: a serving
 * process whose memory pool was carved up at start-up and hands out nothing afterwards, a
 * latency-critical decode loop that forbids cudaMalloc because it synchronises the device, or a
 * plug-in loaded into a runtime that owns the allocator.  mz_decode_attention needs a caller-provided workspace for the per-split
 * partial results; this variant keeps that scratch inside the library instead, in one
 * file-scope device array of MZ_STATIC_SCRATCH_BYTES (8 MiB) that every GPU holds from the
 * moment it loads the library until the process exits.
 *
 * Same arguments and result as mz_decode_attention; args->workspace and
 * args->workspace_bytes are ignored.  The call itself makes no cudaMalloc / cudaFree and calls
 * no allocating routine.  Limits and rules:
 *   - the call is refused (MZ_ERR_WORKSPACE, with the sizes in the message) when the partial
 *     results of the request do not fit MZ_STATIC_SCRATCH_BYTES;
 *   - it is refused (MZ_ERR_UNSUPPORTED) for shapes that run on the shape-generic kernel,
 *     because that kernel reads lookup tables which are allocated on first use;
 *   - the first call on each device looks up the device address of the array
 *     (cudaGetSymbolAddress, with that device current); make that first call outside any
 *     stream capture;
 *   - all calls on a device share the one array and it keeps the previous call's contents.
 *     Nothing in it has to start at zero (every record a call reads it has written itself),
 *     but two calls that overlap on the GPU - different streams, or different host threads -
 *     race on it: serialise them on one stream.
 */
#define MZ_STATIC_SCRATCH_BYTES (8u << 20)
int mz_decode_attention_static(const mz_decode_args* args, void* stream);

/*
 * Same, but stops before normalisation: writes the merged partial triple of
 * this call's tokens, m[B,H], l[B,H], acc[B,H,D] (fp32).  Used when the KV
 * sequence is split across GPUs.  args->out is ignored.
 * Replaces: mu_zero_prefix_decode_chunked_cuda's (acc,m,l) outputs,
 * muzero/kernels/loader.py:1146-1285,1689-1858.
 */
int mz_decode_attention_partial(const mz_decode_args* args, float* m, float* l, float* acc, void* stream);

/*
 * Log-sum-exp merge of n_parts partial triples laid out [n_parts][B*H] (m,l)
 * and [n_parts][B*H][D] (acc) -> out[B*H, D] (out_dtype), normalised.
 * Replaces: mu_zero_prefix_decode_reduce_kernel, muzero/kernels/loader.py:1249-1285,
 * and the torch merge of muzero/cache/attention.py:153-169.
 */
int mz_lse_merge(const float* m, const float* l, const float* acc, int n_parts,
                 long long rows, int head_dim, void* out, int out_dtype, void* stream);

/*
 * The same two steps with one packed record per (batch, head) row, records[B*H][D+2] =
 * {acc[D], m, l} (fp32): the partial call writes it, the merge reads n_parts of them laid out
 * [n_parts][B*H][D+2].  This is the unit that crosses GPUs when the KV sequence is split: one
 * contiguous buffer per rank for the all-gather, no re-packing on either side.
 * Replaces: the same reference code as mz_decode_attention_partial / mz_lse_merge.
 */
int mz_decode_attention_partial_packed(const mz_decode_args* args, float* records, void* stream);
int mz_lse_merge_packed(const float* records, int n_parts, long long rows, int head_dim, void* out,
                        int out_dtype, void* stream);

/*
 * Stand-alone halves of the attention, kept for callers of the reference's
 * two-kernel path (the fused call above is the fast one):
 *   mz_qk_logits: out[B,H,k_groups*G] (out_dtype) = scaling * <q[b,h,:], K^[b,h/gqa,t,:]>
 *   mz_av_output: out[B,H,D] (out_dtype) = sum_t w[b,h,t] * V^[b,h/gqa,t,:],
 *                 w[B,H,n_tokens] contiguous (w_dtype), n_tokens <= v_tokens.
 * Replace: mu_zero_qk_cuda / mu_zero_av_cuda, muzero/kernels/loader.py:388-671,1360-1503
 * and :676-1040,1505-1687.
 */
int mz_qk_logits(const mz_kv_store* store, const void* query, long long q_stride_b, long long q_stride_h,
                 int q_heads, float scaling, void* out, int out_dtype, void* stream);
int mz_av_output(const mz_kv_store* store, const void* weights, int w_dtype, int n_tokens, int q_heads,
                 void* out, int out_dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MUZERO_B200_H */
