"""Configuration of the Lekapel decoder family: a per-layer list of (mixer, feed-forward) descriptions plus a few model-wide
constants, read from the `config.json` that ships with the weights.  Every size and constant comes from that file (or from a
tensor's shape at load time); nothing is assumed equal between layers."""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import List, Optional


@dataclass
class RotarySpec:
    base: float
    dims: int                      # leading dimensions of the rotated part that are actually turned
    layout: str = "interleaved"    # "interleaved": columns 2i and 2i + 1 turn together; "halves": column i with column i + dims / 2
    factor: float = 1.0            # linear scaling: every frequency is divided by this

    def inv_freq(self, device):
        """base^(-2 i / dims) / factor for the dims / 2 pairs, float64 (the kernels take the angle in fp64)"""
        import torch
        i = torch.arange(self.dims // 2, dtype=torch.float64)
        return (float(self.base) ** (-2.0 * i / max(self.dims, 1)) / float(self.factor)).to(device)

    @property
    def layout_code(self) -> int:
        return {"interleaved": 0, "halves": 1}[self.layout]


@dataclass
class LatentAttentionSpec:
    heads: int
    dim: int                       # un-rotated query/key size per head
    rot_dim: int                   # rotated query/key size per head (one key part shared by all heads)
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    rot: RotarySpec
    window: Optional[int] = None   # query i sees keys j with 0 <= i - j < window; None: all earlier keys
    sink: bool = True              # a value-less term exp(sink_h) in the soft-max denominator
    gate: bool = True              # a sigmoid output gate read from the mixer's input
    # q_rank = 0: the query is one full-rank projection of the mixer's input (no query latent, no norm)

    def cache_row_width(self) -> int:
        return self.kv_rank + self.rot_dim

    def state_width(self) -> int:
        return 0

    @classmethod
    def from_dict(cls, d: dict) -> "LatentAttentionSpec":
        rot = d.get("rot") or {}
        rot_dim = int(d.get("rot_dim", 0))
        mask = d.get("mask") or {}
        return cls(heads=int(d["heads"]), dim=int(d["dim"]), rot_dim=rot_dim, vdim=int(d["vdim"]), kv_rank=int(d["kv_rank"]),
                   q_rank=int(d["q_rank"]), scale=float(d.get("scale", (int(d["dim"]) + rot_dim) ** -0.5)),
                   rot=RotarySpec(float(rot.get("base", 10000.0)), int(rot.get("dims", rot_dim))),
                   window=int(mask["size"]) if mask.get("size") is not None else None)


@dataclass
class MlpSpec:
    kind: str                      # "dense" (PolyNorm activation) or "moe" (soft-max top-k router over gated-SiLU experts)
    ff: int
    experts: int = 0
    top: int = 0

    @classmethod
    def from_dict(cls, d: Optional[dict]) -> Optional["MlpSpec"]:
        if d is None:
            return None
        if d["kind"] == "dense":
            return cls("dense", int(d["ff"]))
        if d["kind"] == "moe":
            return cls("moe", int(d["expert"]["ff"]), int(d["router"]["experts"]), int(d["router"]["top"]))
        raise ValueError(f"unknown feed-forward kind {d['kind']!r}")


@dataclass
class LayerSpec:
    type: str
    mixer: LatentAttentionSpec
    mlp: Optional[MlpSpec]


MIXER_SPECS = {"latent_attention": LatentAttentionSpec}


@dataclass
class LekapelConfig:
    architecture: str = "Lekapel"
    vocab: int = 0
    width: int = 0
    norm_eps: float = 1e-5
    norm_groups: int = 1
    residual_mult: float = 1.0
    logit_scale: float = 1.0
    layers: List[LayerSpec] = field(default_factory=list)

    @classmethod
    def from_dict(cls, d: dict) -> "LekapelConfig":
        layers = []
        for i, l in enumerate(d["layers"]):
            if l["type"] not in MIXER_SPECS:
                raise ValueError(f"layer {i}: unknown mixer type {l['type']!r}")
            layers.append(LayerSpec(l["type"], MIXER_SPECS[l["type"]].from_dict(l["mixer"]), MlpSpec.from_dict(l.get("mlp"))))
        norm = d.get("norm") or {}
        return cls(architecture=d.get("architecture", "Lekapel"), vocab=int(d["vocab"]), width=int(d["width"]),
                   norm_eps=float(norm.get("eps", 1e-5)), norm_groups=int(norm.get("groups", 1)),
                   residual_mult=float(d.get("residual_mult", 1.0)), logit_scale=float(d.get("logit_scale", 1.0)), layers=layers)

    @classmethod
    def from_pretrained(cls, path: str) -> "LekapelConfig":
        with open(os.path.join(path, "config.json") if os.path.isdir(path) else path) as f:
            return cls.from_dict(json.load(f))

    # what the cache manager asks of a model
    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    def cache_row_widths(self) -> List[int]:
        return [l.mixer.kv_rank + l.mixer.rot_dim for l in self.layers]

    def max_window(self) -> Optional[int]:
        """Keys further back than this are never read again by any layer (None: some layer reads everything)."""
        w = [l.mixer.window for l in self.layers]
        return None if any(x is None for x in w) else max(w)
