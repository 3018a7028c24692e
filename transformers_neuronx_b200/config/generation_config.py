"""How tokens are chosen on the device, under the reference's names.

`GenerationConfig` has the fields of the reference's class of that name
(src/transformers_neuronx/config.py:106-131) with the same defaults and meanings;
`NeuronConfig(on_device_generation=GenerationConfig(...))` is how a caller of the reference hands it to
a model (config.py:220, opt/model.py:47-48, :187-189).  Every other option of the reference's
NeuronConfig describes its compiler, its tensor layouts, quantization or several devices; they are
accepted and reported as ignored.
"""
from __future__ import annotations

import warnings
from typing import List, Optional, Sequence, Union

Number = Union[int, float]


class GenerationConfig:
    """max_length        longest sequence (None: the model's)
    do_sample         False: the most likely token (unless `dynamic`, see below)
    top_k             keep the k most likely tokens (None: all)
    top_p             of those, the most likely ones until their probability reaches top_p
    top_p_min_tokens  ... but never fewer than this many
    global_top_k      an upper bound of every top_k (needs `dynamic`)
    eos_token_id      None: generation runs to the asked length; an id or a list of ids: a row that
                      produced one is finished and is filled with the (first) id from there on, and
                      generation ends when every row is finished
    temperature       scores are divided by it first
    dynamic           parameters may differ from call to call; as in the reference, a dynamic
                      configuration always samples (top_k=1 is its greedy)
    deterministic     the uniform number of every draw is 0.5 (for tests)
    per_batch_line    top_k, top_p, temperature and top_p_min_tokens are lists, one entry a row
    """

    def __init__(self, *, max_length: Optional[int] = None, do_sample: bool = False,
                 top_k: Union[None, int, Sequence[int]] = 50, top_p: Union[float, Sequence[float]] = 1.0,
                 top_p_min_tokens: Union[int, Sequence[int]] = 1, global_top_k: Optional[int] = None,
                 eos_token_id: Union[None, int, Sequence[int]] = None,
                 temperature: Union[float, Sequence[float]] = 1.0, dynamic: bool = False,
                 deterministic: bool = False, per_batch_line: bool = False):
        self.max_length = max_length
        self.do_sample = bool(do_sample)
        self.per_batch_line = bool(per_batch_line)
        self.top_k = top_k
        self.top_p = [float(p) for p in top_p] if isinstance(top_p, (list, tuple)) else float(top_p)
        self.temperature = ([float(t) for t in temperature] if isinstance(temperature, (list, tuple))
                            else float(temperature))
        self.top_p_min_tokens = top_p_min_tokens
        self.global_top_k = global_top_k
        self.eos_token_id = eos_token_id
        self.dynamic = bool(dynamic)
        self.deterministic = bool(deterministic)
        self._check()

    def _check(self) -> None:
        def each(v):
            return list(v) if isinstance(v, (list, tuple)) else [v]
        for p in each(self.top_p):
            if not (0.0 <= p <= 1.0):
                raise ValueError(f"`top_p` has to be a float >= 0 and <= 1, but is {p}")
        for n in each(self.top_p_min_tokens):
            if not isinstance(n, int) or n < 1:
                raise ValueError(f"`top_p_min_tokens` has to be a positive integer, but is {n}")
        for k in each(self.top_k):
            if k is not None and (not isinstance(k, int) or k < 1):
                raise ValueError(f"`top_k` has to be a positive integer or None, but is {k}")
        for t in each(self.temperature):
            if not t > 0.0:
                raise ValueError(f"`temperature` has to be positive, but is {t}")
        if self.global_top_k is not None and not self.dynamic:
            raise ValueError("dynamic on-device generation must be enabled when global_top_k is set")
        lists = [v for v in (self.top_k, self.top_p, self.temperature, self.top_p_min_tokens)
                 if isinstance(v, (list, tuple))]
        if lists and not self.per_batch_line:
            raise ValueError("lists of sampling parameters need per_batch_line=True")

    def is_greedy(self) -> bool:
        return not self.dynamic and not self.do_sample

    def eos_ids(self) -> Optional[List[int]]:
        e = self.eos_token_id
        if e is None:
            return None
        return [int(e)] if isinstance(e, int) else [int(x) for x in e]

    def for_row(self, b: int):
        """(top_k or 0, top_p, temperature, top_p_min_tokens) of batch line b."""
        def pick(v, name):
            if isinstance(v, (list, tuple)):
                if b >= len(v):
                    raise ValueError(f"`{name}` has {len(v)} entries; the batch has a row {b}")
                return v[b]
            return v
        k = pick(self.top_k, "top_k")
        k = 0 if k is None else int(k)
        if self.global_top_k is not None:
            k = int(self.global_top_k) if k == 0 else min(k, int(self.global_top_k))
        return (k, float(pick(self.top_p, "top_p")), float(pick(self.temperature, "temperature")),
                int(pick(self.top_p_min_tokens, "top_p_min_tokens")))

    def __eq__(self, other) -> bool:
        return isinstance(other, GenerationConfig) and self.__dict__ == other.__dict__

    def __repr__(self) -> str:
        return "GenerationConfig(" + ", ".join(f"{k}={v!r}" for k, v in self.__dict__.items()) + ")"


class SlidingWindowAttnConfig:
    """(sparse_attn_utils.py:80-83)"""

    def __init__(self, window_size: int = 128):
        if int(window_size) < 1:
            raise ValueError("window_size must be at least 1")
        self.window_size = int(window_size)


class BlkSparseAttnConfig:
    """(sparse_attn_utils.py:72-78) kept so that a configuration written for the reference is understood; the
    engine's attention kernels have no block-sparse mask and SparseAttnConfig refuses it."""

    def __init__(self, blk_size: int = 128, num_global_blks: int = 0, num_local_blks: int = 1, num_random_blks: int = 0):
        self.blk_size, self.num_global_blks = blk_size, num_global_blks
        self.num_local_blks, self.num_random_blks = num_local_blks, num_random_blks


class SparseAttnConfig:
    """Attention over part of the earlier tokens (sparse_attn_utils.py:86-160).  The engine builds the causal
    sliding window: a token attends to itself and to the `window_size` tokens before it, in prompts
    (create_sliding_window_mask, :140-150) and when decoding (the reference then slices the last window_size
    cached positions, opt/model.py:470-482).  Pages that have fallen out of every later token's window go
    back to the pool.  Block-sparse and caller-supplied masks, and the window that looks both ways, are refused."""

    def __init__(self, attn_type: str = "blk_sparse", causal: bool = False, sparse_attn_config=None,
                 same_mask_per_layer: bool = True, sparse_mask_dict=None):
        if attn_type not in ("blk_sparse", "window", "custom"):
            raise ValueError("Supported attention types are: ['blk_sparse', 'window', 'custom']")
        if attn_type != "window":
            raise NotImplementedError(f"sparse attention of type {attn_type!r} is not built: the attention kernels mask by "
                                      "position (causal, sliding window), not by an arbitrary mask")
        if not isinstance(sparse_attn_config, SlidingWindowAttnConfig):
            raise ValueError("Must provide a valid sliding window attention config!")
        if not causal:
            raise NotImplementedError("a window that looks both ways has no meaning for a decoder that generates; "
                                      "pass causal=True")
        self.attn_type, self.causal, self.sparse_attn_config = attn_type, True, sparse_attn_config
        self.same_mask_per_layer = bool(same_mask_per_layer)
        self.skip_masking_decode = True

    @property
    def keys_attended(self) -> int:
        """The token itself and window_size before it."""
        return self.sparse_attn_config.window_size + 1


class ContinuousBatchingConfig:
    """The reference's settings for a batch whose rows are sequences that come and go
    (config.py:73-103): `max_num_seqs` (or its older name `batch_size_for_shared_caches`) cache lines that
    forward() addresses by sequence id.  Block size and number of blocks are the engine's own business here."""

    def __init__(self, **kwargs):
        n = kwargs.pop("max_num_seqs", None)
        if n is None:
            n = kwargs.pop("batch_size_for_shared_caches", None)
        else:
            kwargs.pop("batch_size_for_shared_caches", None)
        if n is None or int(n) < 1:
            raise ValueError("ContinuousBatchingConfig needs max_num_seqs (or batch_size_for_shared_caches) >= 1")
        self.max_num_seqs = int(n)
        self.max_model_len = kwargs.pop("max_model_len", None)
        self.optimized_paged_attention = bool(kwargs.pop("optimized_paged_attention", False))
        self.enable_chunked_prefill = bool(kwargs.pop("enable_chunked_prefill", False))
        if kwargs:
            raise TypeError(f"unexpected key word arguments: {sorted(kwargs)}")

    @property
    def batch_size_for_shared_caches(self) -> int:
        return self.max_num_seqs


class NeuronConfig:
    """The reference's bag of options (config.py:160-330).  `on_device_generation`,
    `output_all_logits`, `continuous_batching`, `cast_logits_dtype` and `sparse_attn` (sliding window) have a
    meaning here; `on_device_embedding`, `fuse_qkv` and
    `padding_side='left'` name what this engine does anyway.  Anything else set to a value of its own is kept in
    `ignored` and reported once."""

    _AS_BUILT = {"on_device_embedding", "fuse_qkv", "fuse_mlp", "padding_side",
                 "attention_layout", "collectives_layout", "cache_layout", "compilation_worker_count"}

    def __init__(self, *, on_device_generation: Optional[GenerationConfig] = None, output_all_logits: bool = False,
                 continuous_batching: Optional[ContinuousBatchingConfig] = None, cast_logits_dtype: str = "float32",
                 sparse_attn: Optional[SparseAttnConfig] = None, **options):
        if on_device_generation is not None and not isinstance(on_device_generation, GenerationConfig):
            raise TypeError("on_device_generation must be a GenerationConfig")
        if continuous_batching is not None and not isinstance(continuous_batching, ContinuousBatchingConfig):
            raise TypeError("continuous_batching must be a ContinuousBatchingConfig")
        if cast_logits_dtype not in ("float32", "float16", "bfloat16"):      # config.py:247-250
            raise ValueError(f"The `cast_logits_dtype={cast_logits_dtype}` argument must be one of "
                             "['float32', 'float16', 'bfloat16']")
        self.on_device_generation = on_device_generation
        self.continuous_batching = continuous_batching        # forward() then takes sequence ids as start_ids
        self.cast_logits_dtype = cast_logits_dtype            # the type forward() hands its logits out in (base.py:641-647)
        if sparse_attn is not None and not isinstance(sparse_attn, SparseAttnConfig):
            raise TypeError("sparse_attn must be a SparseAttnConfig")
        self.sparse_attn = sparse_attn                        # a causal sliding window for every attention layer
        self.output_all_logits = bool(output_all_logits)      # forward() of a prompt returns every position's logits
        self.ignored = {k: v for k, v in options.items()
                        if k not in self._AS_BUILT and v not in (None, False)}
        if self.ignored:
            warnings.warn("NeuronConfig options without a meaning for the one-GPU engine are ignored: "
                          + ", ".join(sorted(self.ignored)))
