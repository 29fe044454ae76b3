"""Per-layer quantized KV cache: dense residual window + preallocated quantized store.

Public surface and attribute names follow the reference's ``MuZeroCacheLayer``
(muzero/cache/layer.py:26-563) so that its callers, tests and benchmark keep
working: ``update``, ``compress_residual_prefix``, ``get_attention_state``,
``keys/values``, ``_packed_key_q``, ``_key_mn``, ``_key_scale``,
``_packed_value_q``, ``_value_mn``, ``_value_scale``, ``_key_buffer`` ...

What differs is how the state is kept:

* the quantized store lives in capacity-doubling buffers; a flush writes new
  groups in place through one CUDA launch (no concatenation of the store, no
  transposed copy of the key block); the reference-named attributes are views;
* the residual window slides inside a ring-like buffer: a decode step appends
  at the end, a flush advances the start, and the window is moved back to the
  front only when it reaches the end of the buffer;
* a prefill block is quantized straight from the caller's (possibly strided)
  tensors.
"""
from __future__ import annotations

import ctypes
from typing import Any, Optional

import torch

from ..config import MuZeroConfig
from ..kernels import _cabi
from ..kernels._cabi import KVStore, MuZeroKernelError, check, dtype_code, stream_ptr
from ..kernels.loader import ensure_expand_table, load_mu_zero_cuda_extension
from ..quantizer import _magnitude_ratios, _anchor_offset, alpha_from_stats, select_alpha_key_block
from .policy import grown_capacity, plan_flush, residual_capacity

_STORE_ATTRS = ("_packed_key_q", "_key_mn", "_key_scale", "_packed_value_q", "_value_mn", "_value_scale")


class MuZeroCacheLayer:
    is_sliding = False
    is_compileable = False

    def __init__(self, cfg: MuZeroConfig):
        self.cfg = cfg
        self.nbits = cfg.bits
        self.q_group_size = cfg.q_group_size
        self.residual_length = cfg.residual_length
        self.amax_dtype = getattr(torch, cfg.amax_dtype)
        self.amax_eps = 1e-8
        self.quant_qmax = float((1 << self.nbits) - 1)
        self.backend = cfg.backend
        self.max_cache_length: Optional[int] = None   # optional hint: presize the store
        self._clear_state()

    def _clear_state(self) -> None:
        self._selected_alpha_key = self.cfg.alpha_key
        self._selected_alpha_value = self.cfg.alpha_value
        self.is_initialized = False
        self.cumulative_length = 0
        self.dtype = None
        self.device = None
        self.k_head_dim = self.v_head_dim = None
        self.v_head_dim_padded = self.v_num_groups = None
        self._keys = None
        self._values = None
        self._window_stale = False     # decode_step moved the window; the views are rebuilt on first use
        self._window_len = 0           # residual tokens after the last one-call decode step
        self._step_args = None         # C argument block kept across steady-state decode steps
        self._step_base = 0            # _res_start at the time the block was built
        self._step_ws_bound = 0
        self._key_buffer = None
        self._value_buffer = None
        self._buffer_capacity = 0
        self._res_start = 0
        # logq_compatible_layout: tokens by which the value prefix is ahead of the key prefix.  The window
        # rows [0, _value_lead) then still hold keys only; `values` is the window without them.
        self._value_lead = 0
        for name in _STORE_ATTRS:
            setattr(self, name, None)
        self._bufs: dict[str, torch.Tensor] = {}
        self._key_group_count = 0
        self._value_storage_len = 0

    # `keys` / `values` (the residual window, attribute names of the reference) are views into the window
    # buffers; the one-call decode step only moves counters and leaves rebuilding the views to the first reader
    @property
    def keys(self):
        if self._window_stale:
            self._rebuild_window_views()
        return self._keys

    @keys.setter
    def keys(self, value):
        if self._window_stale:
            self._rebuild_window_views()
        self._keys = value
        self._step_args = None

    @property
    def values(self):
        if self._window_stale:
            self._rebuild_window_views()
        return self._values

    @values.setter
    def values(self, value):
        if self._window_stale:
            self._rebuild_window_views()
        self._values = value
        self._step_args = None

    def _rebuild_window_views(self) -> None:
        self._window_stale = False
        a, n = self._res_start, self._window_len
        self._keys = self._key_buffer[:, :, a:a + n]
        self._values = self._value_buffer[:, :, a + self._value_lead:a + n]

    # ------------------------------------------------------------------ init
    def lazy_initialization(self, key_states: torch.Tensor, value_states: torch.Tensor) -> None:
        self.dtype, self.device = key_states.dtype, key_states.device
        self.keys = torch.empty(0, dtype=self.dtype, device=self.device)
        self.values = torch.empty(0, dtype=self.dtype, device=self.device)
        self.k_head_dim = key_states.shape[-1]
        self.v_head_dim = value_states.shape[-1]
        g = self.q_group_size
        self.v_head_dim_padded = -(-self.v_head_dim // g) * g
        self.v_num_groups = self.v_head_dim_padded // g
        self.is_initialized = True

    def _q_bytes(self) -> int:
        return (self.q_group_size * self.nbits + 7) // 8

    def _require_device_path(self) -> None:
        if self.device is None or self.device.type != "cuda":
            raise MuZeroKernelError("MuZeroCacheLayer needs CUDA tensors; this package has no CPU path")
        if self.dtype not in (torch.bfloat16, torch.float16):
            raise MuZeroKernelError(f"KV dtype must be bfloat16 or float16, got {self.dtype}")
        if self.k_head_dim != self.v_head_dim:
            raise MuZeroKernelError("key and value head_dim must match")

    # ------------------------------------------------------------ descriptors
    def _store_struct(self) -> KVStore:
        """C descriptor of the current state (pointers, strides, counters)."""
        s = KVStore()
        k = self.keys
        b = self._bufs
        # the batch comes from the store when there is one: an empty residual window may be a bare tensor
        s.batch, s.kv_heads = (b["pk"].shape[0], b["pk"].shape[1]) if b else (k.shape[0], k.shape[1])
        s.head_dim = self.k_head_dim
        s.group, s.bits = self.q_group_size, self.nbits
        s.meta_dtype, s.kv_dtype = dtype_code(self.amax_dtype), dtype_code(self.dtype)
        s.alpha_key = float(self._selected_alpha_key if self._selected_alpha_key is not None else 2.0)
        s.alpha_value = float(self._selected_alpha_value if self._selected_alpha_value is not None else 2.0)
        if b:
            s.packed_k, s.k_mn, s.k_scale = b["pk"].data_ptr(), b["kmn"].data_ptr(), b["ksc"].data_ptr()
            s.pk_stride_b, s.pk_stride_h = b["pk"].stride(0), b["pk"].stride(1)
            s.km_stride_b, s.km_stride_h = b["kmn"].stride(0), b["kmn"].stride(1)
            s.packed_v, s.v_mn, s.v_scale = b["pv"].data_ptr(), b["vmn"].data_ptr(), b["vsc"].data_ptr()
            s.pv_stride_b, s.pv_stride_h = b["pv"].stride(0), b["pv"].stride(1)
            s.vm_stride_b, s.vm_stride_h = b["vmn"].stride(0), b["vmn"].stride(1)
        s.k_groups, s.v_tokens = self._key_group_count, self._value_storage_len
        v = self.values
        if self._key_buffer is not None:
            kb, vb = self._key_buffer, self._value_buffer
            off = self._res_start * kb.stride(2) * kb.element_size()
            s.res_k, s.res_v = kb.data_ptr() + off, vb.data_ptr() + off
            s.res_stride_b, s.res_stride_h, s.res_stride_t = kb.stride(0), kb.stride(1), kb.stride(2)
            s.res_start, s.res_len = 0, k.shape[2]     # pointers already address the window's first token
        elif k.numel() > 0:
            if k.stride(-1) != 1 or v.stride(-1) != 1 or k.stride() != v.stride():
                raise MuZeroKernelError("residual keys/values must share strides and be contiguous in head_dim")
            s.res_k, s.res_v = k.data_ptr(), v.data_ptr()
            s.res_stride_b, s.res_stride_h, s.res_stride_t = k.stride(0), k.stride(1), k.stride(2)
            s.res_start, s.res_len = 0, k.shape[2]
        return s

    # ----------------------------------------------------------- dense window
    def _rehome_residual(self, min_tokens: int) -> None:
        """Puts the residual window at the front of a buffer with room for ``min_tokens``."""
        cur = int(self.keys.shape[2]) if self.keys.numel() else 0
        lead = self._value_lead
        if self._key_buffer is None or self._buffer_capacity < min_tokens:
            cap = residual_capacity(min_tokens, self.residual_length, self.q_group_size)
            shape_k = (*self.keys.shape[:2], cap, self.k_head_dim)
            shape_v = (*self.values.shape[:2], cap, self.v_head_dim)
            kb = torch.empty(shape_k, dtype=self.dtype, device=self.device)
            vb = torch.empty(shape_v, dtype=self.dtype, device=self.device)
            if cur:
                kb[:, :, :cur].copy_(self.keys)
                vb[:, :, lead:cur].copy_(self.values)
            self._key_buffer, self._value_buffer, self._buffer_capacity = kb, vb, cap
        elif self._res_start > 0 and cur:
            src_k, src_v = self.keys, self.values
            if self._res_start < cur:          # overlapping move
                src_k, src_v = src_k.clone(), src_v.clone()
            self._key_buffer[:, :, :cur].copy_(src_k)
            self._value_buffer[:, :, lead:cur].copy_(src_v)
        self._res_start = 0
        self.keys = self._key_buffer[:, :, :cur]
        self.values = self._value_buffer[:, :, lead:cur]

    def _append_dense(self, key_states: torch.Tensor, value_states: torch.Tensor) -> None:
        n_new = int(key_states.shape[2])
        if self.keys.numel() == 0 and self._key_buffer is None:
            self.keys, self.values = key_states, value_states      # alias the caller's block
            self._res_start = 0
            if key_states.stride(-1) != 1 or value_states.stride(-1) != 1 or key_states.stride() != value_states.stride():
                # the kernels address keys and values of the window with one set of strides: a block whose two
                # tensors are laid out differently is copied into the layer's own buffers instead
                self._rehome_residual(n_new + 1)
            return
        if n_new == 1:
            cur = int(self.keys.shape[2])
            if self._key_buffer is None or self._res_start + cur + 1 > self._buffer_capacity:
                self._rehome_residual(cur + 1)
            if self.device.type == "cuda" and key_states.stride(-1) == 1 and value_states.stride(-1) == 1 \
                    and key_states.stride()[:2] == value_states.stride()[:2]:
                s = self._store_struct()
                with torch.cuda.device(self.device):
                    check(load_mu_zero_cuda_extension().mz_append_kv(
                        ctypes.byref(s), key_states.data_ptr(), value_states.data_ptr(), key_states.stride(0),
                        key_states.stride(1), stream_ptr(self.device)), "mz_append_kv")
            else:
                pos = self._res_start + cur
                self._key_buffer[:, :, pos:pos + 1].copy_(key_states)
                self._value_buffer[:, :, pos:pos + 1].copy_(value_states)
            a = self._res_start
            self.keys = self._key_buffer[:, :, a:a + cur + 1]
            self.values = self._value_buffer[:, :, a + self._value_lead:a + cur + 1]
            return
        self.keys = torch.cat([self.keys, key_states], dim=-2)
        self.values = torch.cat([self.values, value_states], dim=-2)
        self._key_buffer = self._value_buffer = None
        self._buffer_capacity = 0
        self._res_start = 0
        if self._value_lead:                   # keep keys and values addressable as one window
            self._rehome_residual(int(self.keys.shape[2]) + 1)

    def _drop_residual_prefix(self, n: int, n_values: Optional[int] = None) -> None:
        """Forgets the ``n`` oldest residual keys and ``n_values`` (default ``n``) oldest residual values
        (they are in the store now)."""
        n_values = n if n_values is None else n_values
        if n <= 0 and n_values <= 0:
            return
        lead = self._value_lead + n_values - n
        if self._key_buffer is not None:
            self._res_start += n
            self._value_lead = lead
            a, cur = self._res_start, int(self.keys.shape[2]) - n
            self.keys = self._key_buffer[:, :, a:a + cur]
            self.values = self._value_buffer[:, :, a + lead:a + cur]
        else:
            # aliased prefill block: keep only the tail, in a buffer of its own
            self.keys = self.keys[:, :, n:]
            self.values = self.values[:, :, n_values:]
            self._value_lead = lead
            self._rehome_residual(int(self.keys.shape[2]) + 1)

    # ----------------------------------------------------------------- store
    def _ensure_store(self, groups: int, tokens: int) -> None:
        b, kvh = self.keys.shape[0], self.keys.shape[1]
        d, ng, qb = self.k_head_dim, self.v_num_groups, self._q_bytes()
        have_g = self._bufs["pk"].shape[2] if self._bufs else 0
        have_t = self._bufs["pv"].shape[2] if self._bufs else 0
        if groups <= have_g and tokens <= have_t:
            return
        hint_t = 0
        if self.max_cache_length:
            hint_t = max(int(self.max_cache_length) - self.residual_length, 0)
        g = self.q_group_size
        cap_g = max(grown_capacity(have_g, groups), -(-hint_t // g))
        cap_t = max(grown_capacity(have_t, tokens, slack=8 * g), hint_t, cap_g * g)
        cap_g = max(cap_g, cap_t // g)
        dev, md = self.device, self.amax_dtype
        new = {
            "pk": torch.empty((b, kvh, cap_g, d, qb), dtype=torch.uint8, device=dev),
            "kmn": torch.empty((b, kvh, cap_g, d, 1), dtype=md, device=dev),
            "ksc": torch.empty((b, kvh, cap_g, d, 1), dtype=md, device=dev),
            "pv": torch.empty((b, kvh, cap_t, ng, qb), dtype=torch.uint8, device=dev),
            "vmn": torch.empty((b, kvh, cap_t, ng, 1), dtype=md, device=dev),
            "vsc": torch.empty((b, kvh, cap_t, ng, 1), dtype=md, device=dev),
        }
        if self._bufs:
            kg, vt = self._key_group_count, self._value_storage_len
            for name in ("pk", "kmn", "ksc"):
                new[name][:, :, :kg].copy_(self._bufs[name][:, :, :kg])
            for name in ("pv", "vmn", "vsc"):
                new[name][:, :, :vt].copy_(self._bufs[name][:, :, :vt])
        self._bufs = new
        self._step_args = None
        self._refresh_views()

    def _refresh_views(self) -> None:
        kg, vt = self._key_group_count, self._value_storage_len
        if not self._bufs or (kg == 0 and vt == 0):
            for name in _STORE_ATTRS:
                setattr(self, name, None)
            return
        b = self._bufs
        self._packed_key_q, self._key_mn, self._key_scale = b["pk"][:, :, :kg], b["kmn"][:, :, :kg], b["ksc"][:, :, :kg]
        self._packed_value_q, self._value_mn, self._value_scale = b["pv"][:, :, :vt], b["vmn"][:, :, :vt], b["vsc"][:, :, :vt]

    def _adopt_store(self, tensors: dict[str, torch.Tensor]) -> None:
        """Replaces the store by exact-size tensors (after batch reindexing / device moves)."""
        self._bufs = {k: v.contiguous() for k, v in tensors.items()}
        self._step_args = None
        self._refresh_views()

    # ------------------------------------------------------------------ alpha
    def _ensure_alpha(self, n_flush: int, n_values: Optional[int] = None) -> None:
        n_values = n_flush if n_values is None else n_values
        g, bits, mp = self.q_group_size, self.nbits, self.cfg.stats_max_points
        if self._selected_alpha_key is None and n_flush > 0:
            self._selected_alpha_key = select_alpha_key_block(self.keys[:, :, :n_flush], bits=bits, q_group_size=g,
                                                              max_points=mp)
        if self._selected_alpha_value is None and n_values > 0:
            self._selected_alpha_value = _select_alpha_value_block(self.values[:, :, :n_values], bits=bits, group=g,
                                                                   d_pad=self.v_head_dim_padded, max_points=mp)

    # ------------------------------------------------------------------ flush
    def compress_residual_prefix(self, *, decode_flush: bool = False) -> None:
        """Moves the oldest residual tokens beyond ``residual_length`` into the quantized store."""
        if not self.is_initialized or self.keys is None or self.values is None or self.keys.numel() == 0:
            return
        plan = plan_flush(key_len=int(self.keys.shape[2]), value_len=int(self.values.shape[2]),
                          residual_length=self.residual_length, group=self.q_group_size, decode_flush=decode_flush,
                          flush_by_group=self.cfg.decode_flush_by_group, logq_layout=self.cfg.logq_compatible_layout)
        n, nv = plan.key_tokens, plan.value_tokens
        if n == 0 and nv == 0:
            return
        self._require_device_path()
        self._ensure_alpha(n, nv)
        g = self.q_group_size
        self._ensure_store(self._key_group_count + n // g, self._value_storage_len + nv)
        if self._value_lead and self._key_buffer is None:
            self._rehome_residual(int(self.keys.shape[2]) + 1)      # one window for keys and values
        s = self._store_struct()
        with torch.cuda.device(self.device):
            # value rows are addressed inside the key window: they start `_value_lead` rows in
            check(load_mu_zero_cuda_extension().mz_flush_kv_parts(ctypes.byref(s), n, self._value_lead, nv, self.amax_eps,
                                                                  stream_ptr(self.device)), "mz_flush_kv_parts")
        self._key_group_count += n // g
        self._value_storage_len += nv
        self._refresh_views()
        self._drop_residual_prefix(n, nv)

    # ---------------------------------------------------------------- dequant
    def _dequantize(self, g0: int, g1: int, t0: int, t1: int, want_k: bool, want_v: bool):
        self._require_device_path()
        b, kvh = self.keys.shape[0], self.keys.shape[1]
        g = self.q_group_size
        out_k = torch.empty((b, kvh, max(g1 - g0, 0) * g, self.k_head_dim), dtype=self.dtype, device=self.device) if want_k else None
        out_v = torch.empty((b, kvh, max(t1 - t0, 0), self.v_head_dim), dtype=self.dtype, device=self.device) if want_v else None
        if (want_k and g1 > g0) or (want_v and t1 > t0):
            ensure_expand_table(self.nbits, self._selected_alpha_key, self.device)
            ensure_expand_table(self.nbits, self._selected_alpha_value, self.device)
            s = self._store_struct()
            with torch.cuda.device(self.device):
                check(load_mu_zero_cuda_extension().mz_dequantize_kv(
                    ctypes.byref(s), g0, g1, out_k.data_ptr() if (want_k and g1 > g0) else None, t0, t1,
                    out_v.data_ptr() if (want_v and t1 > t0) else None, dtype_code(self.dtype), self.amax_eps,
                    stream_ptr(self.device)), "mz_dequantize_kv")
        return out_k, out_v

    def _dequantize_key_prefix(self) -> torch.Tensor:
        return self._dequantize(0, self._key_group_count, 0, 0, True, False)[0]

    def _dequantize_value_prefix(self) -> torch.Tensor:
        return self._dequantize(0, 0, 0, self._value_storage_len, False, True)[1]

    def _dequantize_key_range(self, start_group: int, end_group: int) -> torch.Tensor:
        return self._dequantize(start_group, min(end_group, self._key_group_count), 0, 0, True, False)[0]

    def _dequantize_value_range(self, start_token: int, end_token: int) -> torch.Tensor:
        return self._dequantize(0, 0, start_token, min(end_token, self._value_storage_len), False, True)[1]

    # ----------------------------------------------------------------- update
    def update(self, key_states: torch.Tensor, value_states: torch.Tensor,
               cache_kwargs: dict[str, Any] | None = None) -> tuple[torch.Tensor, torch.Tensor]:
        """Appends K/V, flushes what exceeds the residual window, returns K/V for attention.

        First call: the raw block.  ``materialize_full_kv=False`` (decode through the fused
        attention): the residual window only.  Otherwise: dequantized prefix + residual.
        """
        kw = cache_kwargs or {}
        materialize = kw.get("materialize_full_kv", True)
        defer = kw.get("defer_quantize", False)
        first = not self.is_initialized
        if first:
            self.lazy_initialization(key_states, value_states)
        self._append_dense(key_states, value_states)
        self.cumulative_length += key_states.shape[-2]
        raw_k, raw_v = self.keys, self.values
        if not defer:
            self.compress_residual_prefix(decode_flush=key_states.shape[-2] == 1)
        if first:
            return raw_k, raw_v
        if not materialize:
            return self.keys, self.values
        return self._full_kv()

    def decode_step(self, key_states: torch.Tensor, value_states: torch.Tensor, query: torch.Tensor, scaling: float,
                    attention_mask: torch.Tensor | None = None) -> torch.Tensor:
        """One decode step: append ``[B,KVH,1,D]`` K/V, flush when due, attend with ``query [B,H,1,D]``.

        Equivalent to ``update(..., {"materialize_full_kv": False})`` followed by the fused decode
        attention (reference: muzero/cache/layer.py:407-459 and muzero/cache/attention.py:48-295), but in the
        steady state (window inside its buffer, store with room, alphas chosen) it is a single C call,
        ``mz_decode_step``.  Anything else takes the two-call route.  Returns ``[B,1,H,D]``."""
        from .attention import build_decode_args, decode_attention, _workspace
        g = self.q_group_size
        fast = (self.is_initialized and self._key_buffer is not None and key_states.shape[2] == 1 and key_states.is_cuda
                and key_states.dtype == self.dtype and not self.cfg.logq_compatible_layout
                and key_states.stride(-1) == 1 and value_states.stride(-1) == 1
                and key_states.stride()[:2] == value_states.stride()[:2])
        unit = g if self.cfg.decode_flush_by_group else 4 * g
        if fast:
            args = self._step_args
            cur = args.store.res_len if args is not None else int(self.keys.shape[2])
            if self._res_start + cur + 1 > self._buffer_capacity:
                fast = False                      # the window has to move back to the front of its buffer
            excess = cur + 1 - self.residual_length
            n = (excess // unit) * unit if excess > 0 else 0
            if fast and n > 0:
                if self._selected_alpha_key is None or self._selected_alpha_value is None:
                    fast = False                  # the first flush chooses the alphas from the data
                else:
                    self._ensure_store(self._key_group_count + n // g, self._value_storage_len + n)
        if not fast:
            self.update(key_states, value_states, {"materialize_full_kv": False})
            return decode_attention(self, query, scaling, attention_mask)
        b, h, _, d = query.shape
        out = torch.empty((b, 1, h, d), dtype=query.dtype, device=query.device)
        lib = load_mu_zero_cuda_extension()
        args = self._step_args
        if attention_mask is not None or args is None or query.stride(-1) != 1 or query.dtype != self.dtype:
            # (re)build the argument block: pointers, strides and counters of the current state.  With a mask
            # the block is built per call (the mask tensor may be converted and has to stay alive).
            args = build_decode_args(self, query, scaling, attention_mask, out, step=(self.residual_length, unit), bound=True)
            self._step_base = self._res_start
            self._step_ws_bound = args.workspace_bytes
            self._step_args = args if attention_mask is None else None
        else:
            # steady state: the block kept from the last step already holds the advanced counters
            args.query, args.q_stride_b, args.q_stride_h = query.data_ptr(), query.stride(0), query.stride(1)
            args.q_heads, args.scaling = h, float(scaling)
            args.out, args.out_dtype = out.data_ptr(), dtype_code(out.dtype)
            ws = _workspace(query.device, self._step_ws_bound)
            args.workspace, args.workspace_bytes = ws.data_ptr(), ws.numel()
        with torch.cuda.device(self.device):
            rc = lib.mz_decode_step(
                ctypes.byref(args), key_states.data_ptr(), value_states.data_ptr(), key_states.stride(0), key_states.stride(1),
                self.residual_length, unit, int(self._bufs["pk"].shape[2]) if self._bufs else 0,
                self._buffer_capacity - self._step_base, self.amax_eps, stream_ptr(self.device))
        if rc != 0:
            self._step_args = None                # nothing moved (the library commits counters last); rebuild next time
            check(rc, "mz_decode_step")
        st = args.store
        flushed = st.k_groups != self._key_group_count
        self._res_start = self._step_base + st.res_start     # the block's window starts at its own pointer
        self._key_group_count, self._value_storage_len = st.k_groups, st.v_tokens
        self._window_len = st.res_len
        self.cumulative_length += 1
        if self._step_args is None:
            a = self._res_start
            self._keys = self._key_buffer[:, :, a:a + st.res_len]
            self._values = self._value_buffer[:, :, a:a + st.res_len]
        else:
            self._window_stale = True
        if flushed:
            self._refresh_views()
        return out

    def get_attention_state(self) -> dict[str, Any] | None:
        if not self.is_initialized:
            return None
        return {"backend": "mu_zero", "layer": self,
                "key_prefix_length": self._key_group_count * self.q_group_size,
                "value_prefix_length": self._value_storage_len}

    # ---------------------------------------------------------------- lengths
    def get_seq_length(self) -> int:
        return self.cumulative_length

    def get_mask_sizes(self, query_length) -> tuple[int, int]:
        if isinstance(query_length, torch.Tensor):
            query_length = int(query_length.numel())
        return self.get_seq_length() + query_length, 0

    def get_max_cache_shape(self) -> int:
        return -1

    # ------------------------------------------------------ cache management
    def _full_kv(self) -> tuple[torch.Tensor, torch.Tensor]:
        k = torch.cat([self._dequantize_key_prefix(), self.keys], dim=2) if self._key_group_count else self.keys
        v = torch.cat([self._dequantize_value_prefix(), self.values], dim=2) if self._value_storage_len else self.values
        return k, v

    def crop(self, max_length: int) -> None:
        """Keeps the first ``max_length`` tokens.  As in the reference (muzero/cache/layer.py:494-506) the kept
        tokens become a dense window again and are re-quantized by the next update; only the groups / tokens
        that survive are dequantized (the reference materialises the whole cache and slices it)."""
        if max_length < 0:
            max_length = max(0, self.get_seq_length() + max_length)
        if max_length >= self.get_seq_length():
            return
        g = self.q_group_size
        nk, nv = self._key_group_count * g, self._value_storage_len
        k_pre = self._dequantize(0, min(self._key_group_count, -(-max_length // g)), 0, 0, True, False)[0] if nk else None
        v_pre = self._dequantize(0, 0, 0, min(nv, max_length), False, True)[1] if nv else None
        k = torch.cat([k_pre, self.keys], dim=2)[..., :max_length, :] if k_pre is not None else self.keys[..., :max_length, :]
        v = torch.cat([v_pre, self.values], dim=2)[..., :max_length, :] if v_pre is not None else self.values[..., :max_length, :]
        k, v = k.contiguous(), v.contiguous()
        self.reset()
        if max_length > 0:
            self.lazy_initialization(k[:, :, :1], v[:, :, :1])
            self.keys, self.values = k, v
            self.cumulative_length = max_length

    def _reindex_batch(self, fn) -> None:
        """Generic batch re-indexing with tensor ops (state that is not on a GPU)."""
        if self.keys is not None and self.keys.dim() == 4:
            # also with zero residual tokens (residual_length=0 right after a flush): the window's shape
            # carries the batch size, and its old buffers belong to the old batch
            self.keys, self.values = fn(self.keys).contiguous(), fn(self.values).contiguous()
            self._key_buffer = self._value_buffer = None
            self._buffer_capacity, self._res_start = 0, 0
        if self._bufs and (self._key_group_count or self._value_storage_len):
            kg, vt = self._key_group_count, self._value_storage_len
            b = self._bufs
            self._adopt_store({"pk": fn(b["pk"][:, :, :kg]), "kmn": fn(b["kmn"][:, :, :kg]), "ksc": fn(b["ksc"][:, :, :kg]),
                               "pv": fn(b["pv"][:, :, :vt]), "vmn": fn(b["vmn"][:, :, :vt]), "vsc": fn(b["vsc"][:, :, :vt])})

    def _gather_batch(self, index: torch.Tensor) -> None:
        """Entry i of the new cache := entry ``index[i]`` of the current one, all eight tensors in one launch
        (``mz_store_gather_batch``); the reference indexes tensor by tensor (muzero/cache/layer.py:508-523)."""
        if not self.is_initialized or self.keys is None or self.keys.dim() != 4:
            return
        if not self.keys.is_cuda or self._value_lead:
            self._reindex_batch(lambda t: t[index.to(t.device), ...])
            return
        index = index.to(device=self.device, dtype=torch.int64).contiguous()
        n, kvh = int(index.numel()), self.keys.shape[1]
        cur = int(self.keys.shape[2])
        if self._key_buffer is None:
            self._rehome_residual(cur + 1)
        src = self._store_struct()
        # the source stays alive during the launch, and comes back if an index turns out to be out of range
        old = (self._bufs, self._key_buffer, self._value_buffer, self._res_start, self._keys, self._values)
        cap = self._buffer_capacity
        kb = torch.empty((n, kvh, cap, self.k_head_dim), dtype=self.dtype, device=self.device)
        vb = torch.empty((n, kvh, cap, self.v_head_dim), dtype=self.dtype, device=self.device)
        new = {name: torch.empty((n, *t.shape[1:]), dtype=t.dtype, device=self.device) for name, t in self._bufs.items()}
        self._bufs, self._key_buffer, self._value_buffer, self._res_start = new, kb, vb, 0
        self._step_args = None
        self._keys, self._values = kb[:, :, :cur], vb[:, :, :cur]
        self._window_stale = False
        dst = self._store_struct()
        status = torch.zeros(1, dtype=torch.int32, device=self.device)
        with torch.cuda.device(self.device):
            check(load_mu_zero_cuda_extension().mz_store_gather_batch(
                ctypes.byref(src), ctypes.byref(dst), index.data_ptr(), status.data_ptr(), stream_ptr(self.device)),
                "mz_store_gather_batch")
        if int(status.item()):
            self._bufs, self._key_buffer, self._value_buffer, self._res_start, self._keys, self._values = old
            self._step_args = None
            self._refresh_views()
            raise MuZeroKernelError("batch index out of range")
        del old
        self._refresh_views()

    def batch_repeat_interleave(self, repeats: int) -> None:
        if self.is_initialized and self.keys is not None and self.keys.dim() == 4:
            self._gather_batch(torch.arange(self.keys.shape[0]).repeat_interleave(repeats))

    def batch_select_indices(self, indices: torch.Tensor) -> None:
        self._gather_batch(indices)

    def reorder_cache(self, beam_idx: torch.LongTensor) -> None:
        self._gather_batch(beam_idx)

    # offload / prefetch: the valid part of every tensor moves to pinned host memory and back on a side
    # stream, so that the copies neither block the host nor serialise with the compute stream's kernels
    def offload(self) -> None:
        if not self.is_initialized or self.keys is None or not self.keys.is_cuda:
            return
        side = _side_stream(self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))

        def to_host(t: torch.Tensor) -> torch.Tensor:
            host = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
            host.copy_(t, non_blocking=True)
            t.record_stream(side)
            return host
        with torch.cuda.stream(side):
            self._reindex_batch(to_host)
        self._offload_done = torch.cuda.Event()
        self._offload_done.record(side)

    def prefetch(self) -> None:
        if not self.is_initialized or self.keys is None or self.keys.device == self.device:
            return
        side = _side_stream(self.device)
        done = getattr(self, "_offload_done", None)
        if done is not None:
            side.wait_event(done)
        with torch.cuda.stream(side):
            self._reindex_batch(lambda t: t.to(self.device, non_blocking=True))
        torch.cuda.current_stream(self.device).wait_stream(side)

    def reset(self) -> None:
        self._clear_state()


_side_streams: dict = {}


def _side_stream(device: torch.device) -> "torch.cuda.Stream":
    """One copy stream per device for cache offload / prefetch."""
    st = _side_streams.get(device)
    if st is None:
        st = torch.cuda.Stream(device)
        _side_streams[device] = st
    return st


def _select_alpha_value_block(block: torch.Tensor, *, bits: int, group: int, d_pad: int, max_points: int) -> float:
    """``select_alpha(rows, kind="value")`` for the rows [B*KVH*S*NG, G] of a value block
    [B,KVH,S,D] (channels zero-padded to ``d_pad``), sampling through index arithmetic."""
    if bits == 4:
        return 2.0
    b, h, s, d = block.shape
    total = b * h * s * d_pad
    if total > max_points:
        step = max(1, total // max_points)
        idx = torch.arange(0, total, step, device=block.device)[:max_points]
    else:
        idx = torch.arange(0, total, device=block.device)
    c = idx % d_pad
    rest = idx // d_pad
    t = rest % s
    rest = rest // s
    hh = rest % h
    bb = rest // h
    sample = torch.where(c < d, block[bb, hh, t, c.clamp_max(d - 1)].float(), torch.zeros((), device=block.device))
    tail, conc = _magnitude_ratios(sample)
    work = block.float()
    if d_pad != d:
        work = torch.nn.functional.pad(work, (0, d_pad - d))
    grouped = work.reshape(b, h, s, d_pad // group, group)
    return alpha_from_stats(bits=bits, kind="value", tail_ratio=tail, concentration_ratio=conc,
                            anchor_offset=_anchor_offset(grouped))
