"""The OPT architecture as data: its configuration's keys -> a ModelSpec naming parts, sizes,
constants and the tensors of the checkpoint.

Names and shapes of tensors: src/transformers_neuronx/opt/gen_random_pretrained.py:49-76 and
opt/model.py:94-130.  Constants that the reference fixes in code rather than in config.json:
position offset 2 (opt/model.py:78), attention scale 1/sqrt(head_dim) (opt/model.py:458-459),
key/value heads = heads (decoder.py:59), no window.  project_in / project_out
(word_embed_proj_dim != hidden_size), post-LN and the bias / affine switches are not in the
reference; their conventions are stated in parts/embedding.py and parts/block.py.
"""
from __future__ import annotations

import math

from ..config.model_config import OPTConfig
from ..config.registry import Architecture, register_architecture
from ..parts.spec import (AttentionSpec, DenseFeedForwardSpec, EmbeddingSpec, HeadSpec, LayerSpec,
                          LinearSpec, ModelSpec, NormSpec, PositionSpec, ScheduleEntry)

POSITION_OFFSET = 2


def _norm(cfg: OPTConfig, prefix: str) -> NormSpec:
    affine = cfg.layer_norm_elementwise_affine
    return NormSpec("layer_norm", cfg.hidden_size, cfg.layer_norm_eps,
                    weight=prefix + ".weight" if affine else None,
                    bias=prefix + ".bias" if affine else None)


def _linear(cfg: OPTConfig, prefix: str, n_in: int, n_out: int, bias=None) -> LinearSpec:
    bias = cfg.enable_bias if bias is None else bias
    return LinearSpec(n_in, n_out, prefix + ".weight", prefix + ".bias" if bias else None)


def build_spec(cfg: OPTConfig) -> ModelSpec:
    H, E, F, d = cfg.hidden_size, cfg.word_embed_proj_dim, cfg.ffn_dim, cfg.head_dim
    dec = "model.decoder."
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"{dec}layers.{i}."
        attn = AttentionSpec(
            kind="attention", hidden=H, n_heads=cfg.num_attention_heads, n_kv_heads=cfg.num_attention_heads,
            head_dim=d, scale=1.0 / math.sqrt(d),
            q=_linear(cfg, p + "self_attn.q_proj", H, H), k=_linear(cfg, p + "self_attn.k_proj", H, H),
            v=_linear(cfg, p + "self_attn.v_proj", H, H), out=_linear(cfg, p + "self_attn.out_proj", H, H),
            window=None, position=None)
        ff = DenseFeedForwardSpec(kind="dense", fc1=_linear(cfg, p + "fc1", H, F), fc2=_linear(cfg, p + "fc2", F, H),
                                  activation=cfg.activation_function)
        layers.append(LayerSpec(block="pre_norm" if cfg.do_layer_norm_before else "post_norm",
                                norm1=_norm(cfg, p + "self_attn_layer_norm"), mixer=attn,
                                norm2=_norm(cfg, p + "final_layer_norm"), feed_forward=ff))
    embedding = EmbeddingSpec(
        table=dec + "embed_tokens.weight", vocab=cfg.vocab_size, dim=E,
        project_in=_linear(cfg, dec + "project_in", E, H, bias=False) if cfg.has_projection else None,
        position=PositionSpec("learned", table=dec + "embed_positions.weight",
                              rows=cfg.max_position_embeddings + POSITION_OFFSET, dim=H, offset=POSITION_OFFSET))
    head = HeadSpec(
        weight="lm_head.weight", vocab=cfg.vocab_size, dim=E, tied_to=dec + "embed_tokens.weight",
        final_norm=_norm(cfg, dec + "final_layer_norm") if cfg.has_final_layer_norm else None,
        project_out=_linear(cfg, dec + "project_out", H, E, bias=False) if cfg.has_projection else None)
    return ModelSpec(hidden_size=H, vocab_size=cfg.vocab_size, max_positions=cfg.max_position_embeddings,
                     embedding=embedding, layers=tuple(layers),
                     schedule=tuple(ScheduleEntry(i, i) for i in range(cfg.num_hidden_layers)), head=head,
                     eos_token_id=cfg.eos_token_id, pad_token_id=cfg.pad_token_id, bos_token_id=cfg.bos_token_id)


register_architecture(Architecture(name="OPTForCausalLM", model_type="opt", config_class=OPTConfig,
                                   build_spec=build_spec))
