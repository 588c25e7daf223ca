"""GPT-2's configuration, read from the keys of its own config.json.

The reference's ``Config`` holds ``n_vocab, n_ctx, n_embd, n_head, n_layer``
(crates/core/src/config.rs:6-17) and fixes everything else in code: eps 1e-5
(config.rs:20-21), head size 64 (weights.rs:70-73), inner width 4C
(weights.rs:95-98), tanh GELU (kernels/reference.rs:53-61), a tied head
(stages/blocks.rs:152-157).  Here each of those is a key of config.json.
"""
from __future__ import annotations

import dataclasses
from typing import ClassVar, Optional, Tuple

from .base import ConfigError, ModelConfig, field

#: activation_function values this engine computes
GELU_TANH_NAMES = ("gelu_new", "gelu_pytorch_tanh", "gelu_fast")
GELU_ERF_NAMES = ("gelu",)


@dataclasses.dataclass
class GPT2Config(ModelConfig):
    architecture_names: ClassVar[Tuple[str, ...]] = ("GPT2LMHeadModel",)

    vocab_size: int = field()
    n_positions: int = field()
    n_embd: int = field()
    n_layer: int = field()
    n_head: int = field()
    layer_norm_epsilon: float = field()
    activation_function: str = field()
    #: width of the MLP; config.json may give null, which the architecture defines as 4 * n_embd
    n_inner: Optional[int] = field(default=None)
    #: divide attention scores by sqrt(head size)
    scale_attn_weights: bool = field(default=True)
    #: additionally divide the scores of layer l by (l + 1)
    scale_attn_by_inverse_layer_idx: bool = field(default=False)
    #: the LM head shares wte; if false the folder holds lm_head.weight [vocab, n_embd]
    tie_word_embeddings: bool = field(default=True)
    bos_token_id: Optional[int] = field(default=None)
    eos_token_id: Optional[int] = field(default=None)

    def validate(self) -> None:
        bad = []
        for name in ("vocab_size", "n_positions", "n_embd", "n_layer", "n_head"):
            if getattr(self, name) <= 0:
                bad.append(f"{name} must be positive, got {getattr(self, name)}")
        if self.n_head > 0 and self.n_embd > 0 and self.n_embd % self.n_head != 0:
            bad.append(f"n_embd {self.n_embd} is not divisible by n_head {self.n_head}")
        if self.n_inner is not None and self.n_inner <= 0:
            bad.append(f"n_inner must be positive, got {self.n_inner}")
        if not self.layer_norm_epsilon > 0.0:
            bad.append(f"layer_norm_epsilon must be positive, got {self.layer_norm_epsilon}")
        if self.activation_function not in GELU_TANH_NAMES + GELU_ERF_NAMES:
            bad.append(
                f"activation_function {self.activation_function!r} is not one of "
                f"{GELU_TANH_NAMES + GELU_ERF_NAMES}"
            )
        if bad:
            raise ConfigError("config.json: " + "; ".join(bad))

    # derived sizes -----------------------------------------------------
    @property
    def head_dim(self) -> int:
        return self.n_embd // self.n_head

    @property
    def inner_dim(self) -> int:
        return self.n_inner if self.n_inner is not None else 4 * self.n_embd

    @property
    def gelu_kind(self) -> str:
        return "tanh" if self.activation_function in GELU_TANH_NAMES else "erf"

    def n_params(self) -> int:
        """Weights and biases, the count of crates/core/src/config.rs:29-39 with
        the inner width and an untied head as parameters."""
        c, i = self.n_embd, self.inner_dim
        per_layer = 2 * c + c * 3 * c + 3 * c + c * c + c + 2 * c + c * i + i + i * c + c
        total = self.vocab_size * c + self.n_positions * c + self.n_layer * per_layer + 2 * c
        if not self.tie_word_embeddings:
            total += self.vocab_size * c
        return total

    def to_dict(self):
        out = {"architectures": list(self.architecture_names), "model_type": "gpt2"}
        out.update(super().to_dict())
        return out
