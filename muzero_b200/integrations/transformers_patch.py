"""Hugging Face ``transformers`` plug-in: ``patch_transformers()`` and ``MuZeroCache``.

After ``patch_transformers()``, ``model.generate(cache_implementation="mu_zero_4bit",
cache_config={...})`` (bits 1,2,3,4,7,8) builds a ``MuZeroCache`` and Llama / Qwen3
attention layers route single-token decode steps to the fused CUDA attention.
The hook points are the ones the reference uses
(muzero/integrations/transformers_patch.py:207-596): the cache registry and
allow-lists, ``GenerationMixin._prepare_cache_for_generation``, the module-level
``eager_attention_forward`` and the attention classes' ``forward``.
"""
from __future__ import annotations

import importlib
import os
from typing import Any, Optional

import torch

from ..cache.attention import mu_zero_decode_attention_forward, mu_zero_decode_step_forward
from ..cache.layer import MuZeroCacheLayer
from ..config import SUPPORTED_BITS, MuZeroConfig

try:
    from transformers.cache_utils import Cache as _HFCache
except Exception:  # pragma: no cover - transformers is an install requirement
    _HFCache = object

_CACHE_NAMES = {f"mu_zero_{b}bit": b for b in SUPPORTED_BITS}
_HOOKED_MODULES = (
    ("transformers.models.llama.modeling_llama", "LlamaAttention", False),
    ("transformers.models.qwen3.modeling_qwen3", "Qwen3Attention", True),
    ("transformers.models.qwen3.modular_qwen3", "Qwen3Attention", True),
)


class MuZeroCache(_HFCache):
    """All layers' ``MuZeroCacheLayer``s behind the ``transformers`` cache protocol."""

    def __init__(self, cfg: MuZeroConfig, max_cache_length: Optional[int] = None):
        self.cfg = cfg
        self._seen_tokens = 0
        self.defer_prefill_quantization = False
        self.single_shot_prefill = False      # the whole prompt arrives as one block per layer
        self.max_cache_length = max_cache_length
        # routing switches, read once per cache (i.e. once per generate() call), not per layer and token:
        # MUZERO_DISABLE_FUSED_DECODE=1 -> dequantized K/V + stock attention; MUZERO_DISABLE_DECODE_STEP=1 ->
        # fused attention, but append / flush / attention as separate calls
        self.fused_decode = os.environ.get("MUZERO_DISABLE_FUSED_DECODE", "0") != "1"
        # MUZERO_PARITY_MODE=1 -> decode attention with the reference's rounding points (slow, for token comparisons)
        self.parity_mode = os.environ.get("MUZERO_PARITY_MODE", "0") == "1"
        self.fused_step = (self.fused_decode and not self.parity_mode
                           and os.environ.get("MUZERO_DISABLE_DECODE_STEP", "0") != "1")
        # MUZERO_QUANTIZE_PREFILL_CHUNKS=1 -> a chunked prefill quantizes every chunk as it arrives, as the
        # reference's throughput bench does when it prefills in chunks (benchmarks/bench_throughput.py:244-279:
        # no deferral there), instead of keeping every layer's dense K/V until the first decode step, as its
        # generate() hook does.  Later chunks then attend to dequantized earlier tokens; memory stays bounded.
        self.quantize_prefill_chunks = os.environ.get("MUZERO_QUANTIZE_PREFILL_CHUNKS", "0") == "1"
        if _HFCache is object:
            self.layers = []
            self.layer_class_to_replicate = None
            self.offloading = False
        else:
            super().__init__(layer_class_to_replicate=self._new_layer)

    def _new_layer(self) -> MuZeroCacheLayer:
        layer = MuZeroCacheLayer(self.cfg)
        layer.max_cache_length = self.max_cache_length
        return layer

    @property
    def _layers(self) -> dict[int, MuZeroCacheLayer]:
        return dict(enumerate(self.layers))

    def _ensure_layer(self, layer_idx: int) -> MuZeroCacheLayer:
        while len(self.layers) <= layer_idx:
            self.layers.append(self._new_layer())
        return self.layers[layer_idx]

    def update(self, key_states, value_states, layer_idx: int, cache_kwargs: dict[str, Any] | None = None):
        if layer_idx == 0:
            self._seen_tokens += key_states.shape[-2]
        kwargs = dict(cache_kwargs or {})
        kwargs.setdefault("materialize_full_kv", True)   # unknown callers get ordinary dense K/V back
        return self._ensure_layer(layer_idx).update(key_states, value_states, kwargs)

    def prefill_block_defers(self, layer_idx: int) -> bool:
        """Whether a multi-token (prefill) block for this layer has to stay dense until the first decode step.

        The reference defers every prefill block and quantizes all layers at the first decode forward
        (muzero/integrations/transformers_patch.py:546-555), which keeps the dense K/V of every layer alive
        through the prefill.  When ``generate()`` prefills in one forward (``single_shot_prefill``, set by the
        generation hook), the layer's first block is the whole prompt: it is quantized inside its own ``update``
        call, straight from the projection output.  The codes are the ones the deferred flush would produce (the
        same tokens, the same whole-block alpha selection) and the prompt's own attention still sees the raw
        block, so tokens do not change; what changes is that only the residual window stays dense.  A chunked
        prefill keeps the reference's deferral: later chunks attend to the exact dense K/V of earlier ones."""
        if not self.defer_prefill_quantization:
            return False
        if self.quantize_prefill_chunks and not self.single_shot_prefill:
            return False
        first_block = layer_idx >= len(self.layers) or not self.layers[layer_idx].is_initialized
        return not (self.single_shot_prefill and first_block)

    def finalize_prefill_quantization(self) -> None:
        for layer in self.layers:
            layer.compress_residual_prefix(decode_flush=False)

    def get_seq_length(self, layer_idx: int = 0) -> int:
        return self.layers[layer_idx].get_seq_length() if layer_idx < len(self.layers) else 0

    def get_max_length(self) -> Optional[int]:
        return None

    def get_usable_length(self, new_seq_length: int, layer_idx: int = 0) -> int:
        return self.get_seq_length(layer_idx)

    def get_mask_sizes(self, query_length, layer_idx: int = 0) -> tuple[int, int]:
        if isinstance(query_length, torch.Tensor):
            query_length = int(query_length.numel())
        if layer_idx >= len(self.layers):
            return query_length, 0
        return self.layers[layer_idx].get_mask_sizes(query_length)

    def get_max_cache_shape(self, layer_idx: int = 0) -> int:
        return self.layers[layer_idx].get_max_cache_shape() if layer_idx < len(self.layers) else -1

    def get_attention_state(self, layer_idx: int):
        return self.layers[layer_idx].get_attention_state() if layer_idx < len(self.layers) else None

    def reorder_cache(self, beam_idx) -> None:
        for layer in self.layers:
            layer.reorder_cache(beam_idx)

    def crop(self, max_length: int) -> None:
        for layer in self.layers:
            layer.crop(max_length)

    def batch_repeat_interleave(self, repeats: int) -> None:
        for layer in self.layers:
            layer.batch_repeat_interleave(repeats)

    def batch_select_indices(self, indices) -> None:
        for layer in self.layers:
            layer.batch_select_indices(indices)

    def reset(self) -> None:
        for layer in self.layers:
            layer.reset()
        self._seen_tokens = 0

    @property
    def seen_tokens(self) -> int:
        return self._seen_tokens

    def __len__(self) -> int:
        return len(self.layers)

    def __iter__(self):
        return iter(self.layers)

    def __getitem__(self, layer_idx: int):
        if layer_idx >= len(self.layers) or not self.layers[layer_idx].is_initialized:
            return [], []
        k, v = self.layers[layer_idx]._full_kv()
        return [k], [v]


def _cache_class_for(bits: int):
    class _FixedBitsCache(MuZeroCache):
        _bits = bits

        def __init__(self, **kwargs):
            if "quant_backend" in kwargs and "backend" not in kwargs:
                kwargs["backend"] = kwargs["quant_backend"]
            kwargs["bits"] = bits
            super().__init__(MuZeroConfig.from_dict(kwargs))

    _FixedBitsCache.__name__ = _FixedBitsCache.__qualname__ = f"MuZero{bits}bitCache"
    return _FixedBitsCache


# ---------------------------------------------------------------------------
_PATCHED = False


def patch_transformers() -> None:
    """Registers ``mu_zero_{1,2,3,4,7,8}bit`` and installs the decode-attention hooks (idempotent)."""
    global _PATCHED
    if _PATCHED:
        return
    try:
        import transformers.cache_utils as cache_utils
    except ImportError as exc:
        raise ImportError("transformers is not installed") from exc
    registry = getattr(cache_utils, "CACHE_CLASS_REGISTRY", None)
    if registry is None:
        registry = {}
        cache_utils.CACHE_CLASS_REGISTRY = registry
    for name, bits in _CACHE_NAMES.items():
        registry[name] = _cache_class_for(bits)
    _extend_allow_lists()
    _wrap_get_cache(cache_utils, registry)
    _wrap_cache_preparation()
    for module_name, cls_name, qk_norm in _HOOKED_MODULES:
        try:
            module = importlib.import_module(module_name)
        except Exception:
            continue
        _wrap_eager_attention(module)
        _wrap_attention_forward(module, cls_name, qk_norm)
    _PATCHED = True
    print("[mu-Zero/B200] registered mu_zero_{1,2,3,4,7,8}bit cache implementations.")


def _extend_allow_lists() -> None:
    try:
        import transformers.generation.configuration_utils as gcu
    except Exception:
        return
    names = tuple(_CACHE_NAMES)
    for attr in ("ALL_CACHE_IMPLEMENTATIONS", "DYNAMIC_CACHE_IMPLEMENTATIONS"):
        current = getattr(gcu, attr, None)
        if current is not None and names[0] not in current:
            setattr(gcu, attr, tuple(current) + names)


def _wrap_get_cache(cache_utils, registry) -> None:
    original = getattr(cache_utils, "_get_cache", None)
    if original is None or getattr(original, "_muzero_patched", False):
        return

    def _get_cache(cache_implementation, model, *args, **kwargs):
        if cache_implementation in _CACHE_NAMES:
            return registry[cache_implementation](**(kwargs.pop("cache_config", None) or {}))
        return original(cache_implementation, model, *args, **kwargs)

    _get_cache._muzero_patched = True
    cache_utils._get_cache = _get_cache


def _legacy_backend_bits(cache_implementation, cache_config: dict) -> Optional[int]:
    """``cache_implementation="quantized"`` with a ``logq{N}_zeroanchor_stat_cuda[_opt]`` backend."""
    backend = cache_config.get("backend")
    if cache_implementation != "quantized" or not isinstance(backend, str):
        return None
    for bits in SUPPORTED_BITS:
        if backend in (f"logq{bits}_zeroanchor_stat_cuda", f"logq{bits}_zeroanchor_stat_cuda_opt"):
            return bits
    return None


def _wrap_cache_preparation() -> None:
    try:
        import transformers.generation.utils as gen_utils
    except Exception:
        return
    mixin = getattr(gen_utils, "GenerationMixin", None)
    if mixin is None or hasattr(mixin, "_muzero_original_prepare_cache_for_generation"):
        return
    original = getattr(mixin, "_prepare_cache_for_generation", None)
    if original is None:
        return

    def _prepare_cache_for_generation(self, generation_config, model_kwargs, generation_mode, batch_size,
                                      max_cache_length, *args, **kwargs):
        impl = getattr(generation_config, "cache_implementation", None)
        cache_config = dict(getattr(generation_config, "cache_config", None) or {})
        bits = _CACHE_NAMES.get(impl) if isinstance(impl, str) else None
        legacy = _legacy_backend_bits(impl, cache_config)
        if bits is None and legacy is None:
            return original(self, generation_config, model_kwargs, generation_mode, batch_size, max_cache_length,
                            *args, **kwargs)
        if getattr(self.config, "is_encoder_decoder", False):
            raise ValueError("mu_zero cache currently supports decoder-only models")
        cache_config.pop("config", None)
        if legacy is not None:
            cache_config.pop("backend", None)
        if "quant_backend" in cache_config and "backend" not in cache_config:
            cache_config["backend"] = cache_config.pop("quant_backend")
        cache_config["bits"] = bits if bits is not None else legacy
        hint = max_cache_length if isinstance(max_cache_length, int) and max_cache_length > 0 else None
        cache = MuZeroCache(MuZeroConfig.from_dict(cache_config), max_cache_length=hint)
        cache.defer_prefill_quantization = True
        cache.single_shot_prefill = getattr(generation_config, "prefill_chunk_size", None) is None
        model_kwargs["past_key_values"] = cache
        return None

    mixin._muzero_original_prepare_cache_for_generation = original
    mixin._prepare_cache_for_generation = _prepare_cache_for_generation


def _wrap_eager_attention(module) -> None:
    original = getattr(module, "eager_attention_forward", None)
    if original is None or getattr(original, "_muzero_patched", False):
        return

    def eager_attention_forward(attn_module, query, key, value, attention_mask, scaling, dropout: float = 0.0, **kwargs):
        state = kwargs.get("kv_cache_state")
        if state is not None and state.get("backend") == "mu_zero" and not attn_module.training and dropout == 0.0:
            result = mu_zero_decode_attention_forward(attn_module, query, attention_mask, scaling, state)
            if result is not None:
                return result
        kwargs.pop("kv_cache_state", None)
        return original(attn_module, query, key, value, attention_mask, scaling, dropout=dropout, **kwargs)

    eager_attention_forward._muzero_patched = True
    eager_attention_forward._muzero_original = original
    module.eager_attention_forward = eager_attention_forward


def _wrap_attention_forward(module, cls_name: str, qk_norm: bool) -> None:
    cls = getattr(module, cls_name, None)
    if cls is None or getattr(cls.forward, "_muzero_patched", False):
        return
    original = cls.forward

    def forward(self, hidden_states, position_embeddings=None, attention_mask=None, past_key_values=None, **kwargs):
        if position_embeddings is None or not isinstance(past_key_values, MuZeroCache):
            return original(self, hidden_states, position_embeddings, attention_mask, past_key_values, **kwargs)
        batch_shape = hidden_states.shape[:-1]
        per_head = (*batch_shape, -1, self.head_dim)
        q = self.q_proj(hidden_states).view(per_head)
        k = self.k_proj(hidden_states).view(per_head)
        if qk_norm:
            q, k = self.q_norm(q), self.k_norm(k)
        q, k = q.transpose(1, 2), k.transpose(1, 2)
        v = self.v_proj(hidden_states).view(per_head).transpose(1, 2)
        cos, sin = position_embeddings
        q, k = module.apply_rotary_pos_emb(q, k, cos, sin)

        cache = past_key_values
        single = q.shape[-2] == 1 and not self.training
        if cache.defer_prefill_quantization and single:
            cache.finalize_prefill_quantization()
            cache.defer_prefill_quantization = False
        fused = single and cache.fused_decode
        if fused and cache.fused_step and self.layer_idx < len(cache.layers):
            # steady-state decode: append, flush when due and attention in one call into the library
            if self.layer_idx == 0:
                cache._seen_tokens += 1
            out, weights = mu_zero_decode_step_forward(self, cache.layers[self.layer_idx], k, v, q, attention_mask, self.scaling)
            out = out.reshape(*batch_shape, -1).contiguous()
            return self.o_proj(out), weights
        k, v = cache.update(k, v, self.layer_idx, {
            "sin": sin, "cos": cos, "cache_position": kwargs.get("cache_position"),
            "materialize_full_kv": not fused,
            "defer_quantize": bool(q.shape[-2] > 1 and cache.prefill_block_defers(self.layer_idx)),
        })
        if fused and cache.parity_mode:
            from ..cache.attention import decode_attention_reference_rounding
            out = decode_attention_reference_rounding(cache.layers[self.layer_idx], q, self.scaling, attention_mask)
            return self.o_proj(out.reshape(*batch_shape, -1).contiguous()), None
        if fused:
            kwargs["kv_cache_state"] = cache.get_attention_state(self.layer_idx)
            attend = module.eager_attention_forward
        else:
            attend = module.ALL_ATTENTION_FUNCTIONS.get_interface(self.config._attn_implementation,
                                                                  module.eager_attention_forward)
        extra = {"sliding_window": getattr(self, "sliding_window", None)} if qk_norm else {}
        out, weights = attend(self, q, k, v, attention_mask, dropout=0.0 if not self.training else self.attention_dropout,
                              scaling=self.scaling, **extra, **kwargs)
        out = out.reshape(*batch_shape, -1).contiguous()
        return self.o_proj(out), weights

    forward._muzero_patched = True
    forward._muzero_original = original
    cls.forward = forward
