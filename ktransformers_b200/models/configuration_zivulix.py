"""Configuration of the Zivulix decoder family: a list of layers, each a mixer and an optional gated-GELU feed-forward, with an
RMS norm (zero-centred weights) on every sublayer's OUTPUT.  Mixers: "attention" (grouped heads, biased projections,
partial rotation with stretched wavelengths, unit-rms queries and keys, capped scores, sliding window, values blended with the
first such layer's), "latent_attention" (keys and values up-projected from one cached latent per token plus one shared rotated
key part, no window) and "delta" (the gated delta rule behind short convolutions, a recurrent matrix state per head).  Every
size and constant is read from the checkpoint's `config.json`; nothing is assumed equal between layers."""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import List, Optional

from .configuration_lekapel import LatentAttentionSpec, RotarySpec


def _rotary(d: Optional[dict], default_dims: int) -> Optional[RotarySpec]:
    """the design turns column i together with column i + dims / 2"""
    if not d:
        return None
    scaling = d.get("scaling") or {}
    return RotarySpec(float(d.get("base", 10000.0)), int(d.get("dims", default_dims)), layout="halves", factor=float(scaling.get("factor", 1.0)))


@dataclass
class CappedWindowAttentionSpec:
    heads: int
    kv_heads: int
    dim: int                       # query / key size per head
    vdim: int
    scale: float
    softcap: Optional[float]       # scores s become c tanh(s / c) with c = softcap; None: scores are not capped
    window: Optional[int]          # query i sees keys j with 0 <= i - j < window; None: all earlier keys
    rot: Optional[RotarySpec]
    unit_rms: bool                 # once rotated, queries and keys are scaled to unit rms head by head
    v_mix: bool                    # values blended with those of the first layer that says so (that layer itself does not blend)

    @classmethod
    def from_dict(cls, d: dict) -> "CappedWindowAttentionSpec":
        heads, dim = int(d["heads"]), int(d["dim"])
        mask = d.get("mask") or {}
        return cls(heads=heads, kv_heads=int(d.get("kv_heads", heads)), dim=dim, vdim=int(d.get("vdim", dim)), scale=float(d.get("scale", dim ** -0.5)),
                   softcap=float(d["softcap"]) if d.get("softcap") else None, window=int(mask["size"]) if mask.get("size") is not None else None,
                   rot=_rotary(d.get("rot"), dim), unit_rms=True, v_mix=bool(d.get("v_mix", False)))

    def cache_row_width(self) -> int:
        return self.kv_heads * (self.dim + self.vdim)

    def state_width(self) -> int:
        return 0


def latent_spec_from_dict(d: dict) -> LatentAttentionSpec:
    """latent attention as this family has it: a full-rank query, no window, no sink, no output gate"""
    rot_dim = int(d.get("rot_dim", 0))
    rot = _rotary(d.get("rot") or {"base": 10000.0}, rot_dim)
    mask = d.get("mask") or {}
    return LatentAttentionSpec(heads=int(d["heads"]), dim=int(d["dim"]), rot_dim=rot_dim, vdim=int(d["vdim"]), kv_rank=int(d["kv_rank"]), q_rank=0,
                               scale=float(d.get("scale", (int(d["dim"]) + rot_dim) ** -0.5)), rot=rot,
                               window=int(mask["size"]) if mask.get("size") is not None else None, sink=False, gate=False)


@dataclass
class GatedDeltaSpec:
    heads: int                     # value heads (one state matrix each)
    kv_heads: int                  # query / key heads, shared by heads / kv_heads value heads each
    dim: int
    vdim: int
    conv: int                      # taps of the causal convolution in front of q, k and v
    unit_eps: float = 1e-6         # q and k become x * rsqrt(|x|^2 + unit_eps)

    @classmethod
    def from_dict(cls, d: dict) -> "GatedDeltaSpec":
        heads, dim = int(d["heads"]), int(d["dim"])
        return cls(heads=heads, kv_heads=int(d.get("kv_heads", heads)), dim=dim, vdim=int(d.get("vdim", dim)), conv=int(d.get("conv", 1)))

    @property
    def channels(self) -> int:
        return 2 * self.kv_heads * self.dim + self.heads * self.vdim

    def cache_row_width(self) -> int:
        return 0

    def state_width(self) -> int:
        """the state matrices, then the last conv - 1 inputs of every convolved channel"""
        return self.heads * self.dim * self.vdim + (self.conv - 1) * self.channels


@dataclass
class MlpSpec:
    kind: str                      # "dense": W_down (gelu_tanh(W_gate h) * (W_up h))
    ff: int

    @classmethod
    def from_dict(cls, d: Optional[dict]) -> Optional["MlpSpec"]:
        if d is None:
            return None
        if d["kind"] == "dense":
            return cls("dense", int(d["ff"]))
        raise ValueError(f"unknown feed-forward kind {d['kind']!r}")


@dataclass
class LayerSpec:
    type: str
    mixer: object
    mlp: Optional[MlpSpec]


MIXER_SPECS = {"attention": CappedWindowAttentionSpec.from_dict, "latent_attention": latent_spec_from_dict, "delta": GatedDeltaSpec.from_dict}


@dataclass
class ZivulixConfig:
    architecture: str = "Zivulix"
    vocab: int = 0
    width: int = 0
    norm_eps: float = 1e-6
    layers: List[LayerSpec] = field(default_factory=list)

    @classmethod
    def from_dict(cls, d: dict) -> "ZivulixConfig":
        layers = []
        for i, l in enumerate(d["layers"]):
            if l["type"] not in MIXER_SPECS:
                raise ValueError(f"layer {i}: unknown mixer type {l['type']!r}")
            layers.append(LayerSpec(l["type"], MIXER_SPECS[l["type"]](l["mixer"]), MlpSpec.from_dict(l.get("mlp"))))
        norm = d.get("norm") or {}
        return cls(architecture=d.get("architecture", "Zivulix"), vocab=int(d["vocab"]), width=int(d["width"]), norm_eps=float(norm.get("eps", 1e-6)), layers=layers)

    @classmethod
    def from_pretrained(cls, path: str) -> "ZivulixConfig":
        with open(os.path.join(path, "config.json") if os.path.isdir(path) else path) as f:
            return cls.from_dict(json.load(f))

    def first_value_mixer(self) -> Optional[int]:
        """the layer whose values the other value-blending layers blend in (it does not blend itself)"""
        for i, l in enumerate(self.layers):
            if l.type == "attention" and l.mixer.v_mix:
                return i
        return None

    # what the cache manager asks of a model
    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    def cache_row_widths(self) -> List[int]:
        return [l.mixer.cache_row_width() for l in self.layers]

    def state_widths(self) -> List[int]:
        return [l.mixer.state_width() for l in self.layers]

    def max_window(self) -> Optional[int]:
        """Keys further back than this are never read again by any layer that caches rows (None: some layer reads everything)."""
        w = [l.mixer.window for l in self.layers if l.mixer.cache_row_width() > 0]
        return None if (not w or any(x is None for x in w)) else max(w)
