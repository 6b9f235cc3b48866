"""Configuration schema of the Pubopel decoder-only language model (``config.json`` of a model folder).

Every size and every per-model constant comes from the file.  Optional entries that are absent switch their
mechanism off: no ``mask`` is full causal attention, no ``softcap`` leaves scores uncapped, ``mlp: null`` is a layer
without feed-forward, no ``shared`` a mixture without shared expert.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Literal, Optional

from pydantic import BaseModel, Field


class MaskConfig(BaseModel, frozen=True):
    size: int = Field(gt=0)                      # key j is seen from i when i - j < size ...
    keep_first: int = Field(default=0, ge=0)     # ... or j < keep_first


class AttentionMixerConfig(BaseModel, frozen=True):
    heads: int = Field(gt=0)
    kv_heads: int = Field(gt=0)
    dim: int = Field(gt=0)
    vdim: int = Field(gt=0)
    scale: float
    softcap: Optional[float] = None
    mask: Optional[MaskConfig] = None


class ExpertConfig(BaseModel, frozen=True):
    ff: int = Field(gt=0)


class RouterConfig(BaseModel, frozen=True):
    experts: int = Field(gt=0)
    top: int = Field(gt=0)


class MlpConfig(BaseModel, frozen=True):
    kind: Literal["moe"] = "moe"
    expert: ExpertConfig
    router: RouterConfig
    shared: Optional[ExpertConfig] = None


class LayerConfig(BaseModel, frozen=True):
    type: Literal["attention"]
    mixer: AttentionMixerConfig
    mlp: Optional[MlpConfig] = None


class TapConfig(BaseModel, frozen=True):
    taps: int = Field(ge=1)


class NormConfig(BaseModel, frozen=True):
    eps: float = Field(ge=0.0)


class PubopelConfig(BaseModel, frozen=True):
    architecture: Literal["Pubopel"] = "Pubopel"
    vocab: int = Field(gt=0)
    width: int = Field(gt=0)
    layers: list[LayerConfig] = Field(min_length=1)
    canon: TapConfig
    norm: NormConfig

    @classmethod
    def load(cls, path: str | Path) -> "PubopelConfig":
        return cls.model_validate(json.loads(Path(path).read_text(encoding="utf-8")))

    def check(self) -> None:
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            if m.heads % m.kv_heads:
                raise ValueError(f"layer {i}: heads ({m.heads}) must be a multiple of kv_heads ({m.kv_heads})")
            if m.vdim != m.dim:
                raise ValueError(f"layer {i}: the values are the projected keys, so vdim ({m.vdim}) must equal dim ({m.dim})")
            if layer.mlp is not None and layer.mlp.router.top > layer.mlp.router.experts:
                raise ValueError(f"layer {i}: top ({layer.mlp.router.top}) exceeds experts ({layer.mlp.router.experts})")
