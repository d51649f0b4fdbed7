"""The stage-A compressor hooks over this package's CUDA prompt and decode tiers.

Same hooks as the reference's ``src/phasekv/compressor.py:41-175`` ``PhaseKVCompressor`` — ``reset``,
``on_prefill`` (``prompt_tier.select_and_pack``), ``on_decode_step`` (``decode_tier.maintain``),
``cache_memory_bytes``, ``describe`` — reading the same hyper-parameters from a configuration object with the
fields of the evaluation pipeline's ``CompressionConfig`` (``prefill_keep_ratio``, ``decode_keep_ratio``,
``recent_window``, ``sink_tokens``, ``bits`` and the ``extra`` dictionary).  The class does not import the
evaluation pipeline: an evaluation harness registers it by subclassing its own ``KVCompressor`` together with this
one, or simply calls the hooks.  The reference's roofline planner (``use_planner`` / ``target_memory_ratio``) is a
separate component and is refused here rather than silently ignored.

The cache is a standard dense transformers cache of either generation, on CUDA.
"""
from __future__ import annotations

from . import decode_tier
from . import hetero_cache as hc
from . import prompt_tier

_VALID_BITS = (2, 3, 4, 8, 16)


class PhaseKVCompressor:
    requires_attention = True   # the prompt selection needs the prefill attention matrices
    physically_evicts = True    # prompt selection and cold-tier eviction shrink the tensors

    def __init__(self, config):
        base = super()
        if hasattr(base, "__init__") and type(self).__mro__[1] is not object:
            base.__init__(config)  # cooperative: a harness may mix this class with its own KVCompressor
        self.config = config
        extra = dict(getattr(config, "extra", None) or {})
        if extra.get("use_planner") or extra.get("target_memory_ratio") is not None:
            raise ValueError("the roofline planner is not part of this package; pass the hyper-parameters explicitly")

        def given(name, default):
            value = getattr(config, name, None)
            return default if value is None else value
        self.prefill_keep_ratio = float(given("prefill_keep_ratio", 0.5))
        self.decode_keep_ratio = float(given("decode_keep_ratio", 1.0))
        self.recent_window = int(given("recent_window", 32))
        self.sink_tokens = int(given("sink_tokens", 0))
        self.prompt_bits = int(extra.get("prompt_bits", given("bits", 2)))
        self.cold_bits = int(extra.get("cold_bits", 4))
        self.group_size = int(extra.get("group_size", 32))
        self.lazy_g = int(extra.get("lazy_g", 16))
        self.obs_window = int(extra.get("obs_window", 32))
        self.pool_kernel = int(extra.get("pool_kernel", 7))
        self.pooling = str(extra.get("pooling", "maxpool"))
        for name, bits in (("prompt_bits", self.prompt_bits), ("cold_bits", self.cold_bits)):
            if bits not in _VALID_BITS:
                raise ValueError(f"{name} 仅支持 {_VALID_BITS} (supported widths), got {bits}")
        for name in ("prefill_keep_ratio", "decode_keep_ratio"):
            if not 0.0 < getattr(self, name) <= 1.0:
                raise ValueError(f"{name} 必须落在 (0,1] (must lie in (0, 1]), got {getattr(self, name)}")
        for name in ("recent_window", "group_size", "lazy_g", "obs_window"):
            if getattr(self, name) <= 0:
                raise ValueError(f"{name} 必须为正整数 (must be a positive integer)")
        self.state = self._fresh_state()

    def _fresh_state(self) -> hc.HeteroTierState:
        return hc.HeteroTierState(prompt_bits=self.prompt_bits, cold_bits=self.cold_bits, group_size=self.group_size,
                                  recent_window=self.recent_window)

    def reset(self, model_config=None) -> None:
        self.state = self._fresh_state()

    def on_prefill(self, cache, *, attentions=None, prompt_len, model_config):
        prompt_tier.select_and_pack(cache, attentions=attentions, prompt_len=prompt_len, model_config=model_config,
                                    state=self.state, prefill_keep_ratio=self.prefill_keep_ratio,
                                    sink_tokens=self.sink_tokens, obs_window=self.obs_window,
                                    pool_kernel=self.pool_kernel, pooling=self.pooling)
        return cache

    def on_decode_step(self, cache, *, attentions=None, step, model_config):
        decode_tier.maintain(cache, step=step, model_config=model_config, state=self.state,
                             decode_keep_ratio=self.decode_keep_ratio, lazy_g=self.lazy_g)
        return cache

    def cache_memory_bytes(self, cache) -> int:
        return self.state.logical_bytes(cache)

    def describe(self) -> dict:
        return {"phasekv": {name: getattr(self, name) for name in (
            "prefill_keep_ratio", "decode_keep_ratio", "recent_window", "sink_tokens", "prompt_bits", "cold_bits",
            "group_size", "lazy_g", "obs_window", "pool_kernel", "pooling")}}
