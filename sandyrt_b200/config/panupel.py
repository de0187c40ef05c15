"""PanupelConfig: the typed form of a Panupel config.json.

The design stacks layers of two kinds, each with sizes of its own: a "parallel" layer runs grouped-query
attention (whole-row q/k norm, partial rotary positions, a sink in the softmax, a gate per head) beside a matrix
memory, a "delta" layer runs the gated delta rule behind short convolutions; a span of layers may run several
times on the same weights.  Keys: `vocab`, `width`, `norm.eps`, `residual_mult`, `layers[i].{type, mixer, mlp}`,
`loop.{start, stop, times}`; core/panupel.cpp lists them all.

Reading, type checks and validation are the host library's (core/panupel.cpp, PanupelConfig); this dataclass
carries the result.  Its layer records stay plain dictionaries, as config.json writes them.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Dict, List, Optional

from .. import core
from .base import ModelConfig


@dataclasses.dataclass(frozen=True)
class PanupelConfig(ModelConfig):
    architecture = "Panupel"

    vocab: int = 0
    width: int = 0
    norm: Dict[str, Any] = dataclasses.field(default_factory=lambda: {"eps": 1e-6})
    residual_mult: float = 1.0
    layers: List[Dict[str, Any]] = dataclasses.field(default_factory=list)
    loop: Optional[Dict[str, int]] = None

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "PanupelConfig":
        """Type checks only; `validate` checks the sizes against one another."""
        n = core.call("global", None, "parse_config", config=raw, architecture=cls.architecture, validate=False)
        names = {f.name for f in dataclasses.fields(cls)}
        return cls(**{k: v for k, v in n.items() if k in names})

    def to_dict(self) -> Dict[str, Any]:
        d = dataclasses.asdict(self)
        if d["loop"] is None:
            del d["loop"]
        d["architecture"] = self.architecture
        return d

    def validate(self) -> None:
        core.call("global", None, "parse_config", config=self.to_dict(), architecture=self.architecture, validate=True)
