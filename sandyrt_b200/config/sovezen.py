"""SovezenConfig: the typed form of a Sovezen config.json.

The design stacks layers that run attention over a low-rank latent of keys and values beside their feed-forward,
both on one normed input, each result scaled per channel before it joins the stream.  Two forms of the attention
("latent_attention": rotary positions on a part of every head and a sink in the softmax; "latent_attention_2": no
positions, queries through a latent of their own), a dense or routed feed-forward or none, layers that use another
layer's tensors (`weights_of`), a tied head times `logit_scale`.  Keys: `vocab`, `width`, `logit_scale`, `norm.eps`,
`layers[i].{type, mixer, mlp, weights_of}`; core/sovezen.cpp lists them all.

Reading, type checks and validation are the host library's (core/sovezen.cpp, SovezenConfig); this dataclass
carries the result.  Its layer records stay plain dictionaries, as config.json writes them.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Dict, List

from .. import core
from .base import ModelConfig


@dataclasses.dataclass(frozen=True)
class SovezenConfig(ModelConfig):
    architecture = "Sovezen"

    vocab: int = 0
    width: int = 0
    logit_scale: float = 1.0
    norm: Dict[str, Any] = dataclasses.field(default_factory=lambda: {"eps": 1e-6})
    layers: List[Dict[str, Any]] = dataclasses.field(default_factory=list)

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "SovezenConfig":
        """Type checks only; `validate` checks the sizes against one another."""
        n = core.call("global", None, "parse_config", config=raw, architecture=cls.architecture, validate=False)
        names = {f.name for f in dataclasses.fields(cls)}
        return cls(**{k: v for k, v in n.items() if k in names})

    def to_dict(self) -> Dict[str, Any]:
        d = dataclasses.asdict(self)
        d["architecture"] = self.architecture
        return d

    def validate(self) -> None:
        core.call("global", None, "parse_config", config=self.to_dict(), architecture=self.architecture, validate=True)
