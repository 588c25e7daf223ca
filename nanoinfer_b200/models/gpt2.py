"""GPT-2 as a ModelSpec: learned absolute positions, pre-LayerNorm blocks of causal attention
and a dense GELU MLP, a final LayerNorm and a head tied to the token embedding unless the
configuration says otherwise.

Tensor names are the bare names of the Hugging Face checkpoint that the reference reads
(crates/core/src/weights.rs:77-108): ``wte.weight``, ``wpe.weight``, ``h.{i}.ln_1.*``,
``h.{i}.attn.c_attn.*``, ``h.{i}.attn.c_proj.*``, ``h.{i}.ln_2.*``, ``h.{i}.mlp.c_fc.*``,
``h.{i}.mlp.c_proj.*``, ``ln_f.*``; the four matrices are stored [in, out] (Conv1D) and are
transposed at load (weights.rs:48-57).  ``lm_head.weight`` [vocab, width] is read when the
head is not tied.  A ``transformer.`` prefix is accepted, and the causal-mask buffers some
checkpoints carry (``h.{i}.attn.bias``, ``h.{i}.attn.masked_bias``) are ignored, as the
reference ignores every tensor it does not ask for.
"""
from __future__ import annotations

import math

from ..config.gpt2 import GPT2Config
from ..parts.base import TensorRef
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def build_gpt2_spec(cfg: GPT2Config) -> ModelSpec:
    c, hd = cfg.n_embd, cfg.head_dim
    layers = []
    for i in range(cfg.n_layer):
        p = f"h.{i}."
        scale = 1.0 / math.sqrt(hd) if cfg.scale_attn_weights else 1.0
        if cfg.scale_attn_by_inverse_layer_idx:
            scale = scale / float(i + 1)
        layers.append(LayerSpec(
            arrangement="pre_norm",
            norm_1=PartSpec("layernorm", dict(width=c, eps=cfg.layer_norm_epsilon),
                            {"weight": TensorRef(p + "ln_1.weight"), "bias": TensorRef(p + "ln_1.bias")}),
            mixer=PartSpec("causal_attention",
                           dict(width=c, n_head=cfg.n_head, n_kv_head=cfg.n_head, head_dim=hd, scale=scale,
                                window=0, bias=True),
                           {"qkv_weight": TensorRef(p + "attn.c_attn.weight", transposed=True),
                            "qkv_bias": TensorRef(p + "attn.c_attn.bias"),
                            "out_weight": TensorRef(p + "attn.c_proj.weight", transposed=True),
                            "out_bias": TensorRef(p + "attn.c_proj.bias")}),
            norm_2=PartSpec("layernorm", dict(width=c, eps=cfg.layer_norm_epsilon),
                            {"weight": TensorRef(p + "ln_2.weight"), "bias": TensorRef(p + "ln_2.bias")}),
            feed_forward=PartSpec("dense_mlp",
                                  dict(width=c, inner=cfg.inner_dim, activation=cfg.gelu_kind, bias=True),
                                  {"fc_weight": TensorRef(p + "mlp.c_fc.weight", transposed=True),
                                   "fc_bias": TensorRef(p + "mlp.c_fc.bias"),
                                   "proj_weight": TensorRef(p + "mlp.c_proj.weight", transposed=True),
                                   "proj_bias": TensorRef(p + "mlp.c_proj.bias")}),
        ))
    head_tensor = "wte.weight" if cfg.tie_word_embeddings else "lm_head.weight"
    ignorable = [r"h\.\d+\.attn\.bias", r"h\.\d+\.attn\.masked_bias"]
    if cfg.tie_word_embeddings:
        ignorable.append(r"lm_head\.weight")
    return ModelSpec(
        width=c,
        embedding=PartSpec("token_embedding", dict(vocab_size=cfg.vocab_size, width=c),
                           {"table": TensorRef("wte.weight")}),
        position=PartSpec("learned_absolute", dict(n_positions=cfg.n_positions, width=c),
                          {"table": TensorRef("wpe.weight")}),
        layers=layers,
        schedule=[ScheduleEntry(i) for i in range(cfg.n_layer)],
        final_norm=PartSpec("layernorm", dict(width=c, eps=cfg.layer_norm_epsilon),
                            {"weight": TensorRef("ln_f.weight"), "bias": TensorRef("ln_f.bias")}),
        head=PartSpec("linear_head", dict(vocab_size=cfg.vocab_size, width=c),
                      {"weight": TensorRef(head_tensor)}),
        max_positions=cfg.n_positions,
        name_prefixes=["", "transformer."],
        ignorable=ignorable,
        eos_token_id=cfg.eos_token_id,
    )
