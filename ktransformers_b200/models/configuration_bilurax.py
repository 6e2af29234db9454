"""Configuration of the Bilurax decoder family: a list of pre-norm layers, each a token-shifted mixer ("attention": soft-max
attention inside chunks of the sequence, queries and keys normed over their whole projection, unit-rms values, a temperature per
head, capped scores, no positions in the scores) and a feed-forward (relu-squared dense, a mixture of clamped gated experts behind a
grouped sigmoid router, or none); a span of layers that runs several times in a row with the same weights and separate caches; a
scaled embedding whose table is also the output projection; capped logits.  Every size and constant is read from the checkpoint's
`config.json`; nothing is assumed equal between layers."""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import List, Optional

from .configuration_mabidra import LoopSpec


@dataclass
class ChunkedAttentionSpec:
    heads: int
    kv_heads: int
    dim: int                       # query / key size per head
    vdim: int
    scale: float                   # multiplies q . k, together with the head's learned temperature
    softcap: Optional[float]       # scores s become c tanh(s / c) with c = softcap; None: scores are not capped
    chunk: Optional[int]           # position i sees j <= i with floor(j / chunk) == floor(i / chunk); None: every earlier position

    @classmethod
    def from_dict(cls, d: dict) -> "ChunkedAttentionSpec":
        heads, dim = int(d["heads"]), int(d["dim"])
        mask = d.get("mask") or {}
        return cls(heads=heads, kv_heads=int(d.get("kv_heads", heads)), dim=dim, vdim=int(d.get("vdim", dim)), scale=float(d.get("scale", dim ** -0.5)),
                   softcap=float(d["softcap"]) if d.get("softcap") else None, chunk=int(mask["size"]) if mask.get("size") else None)

    def cache_row_width(self) -> int:
        return self.kv_heads * (self.dim + self.vdim)


@dataclass
class MlpSpec:
    kind: str                      # "dense": W_down relu(W_up h)^2;  "moe": grouped sigmoid router over clamped gated experts
    ff: int
    experts: int = 0
    top: int = 0
    groups: int = 1                # experts form `groups` equal groups of neighbours, of which the best `keep_groups` can be chosen from
    keep_groups: int = 1
    out_scale: float = 1.0         # multiplies the normalised weights of the chosen experts
    limit: float = 0.0             # the experts' clamp: gate <= limit, |up| <= limit

    @classmethod
    def from_dict(cls, d: Optional[dict]) -> Optional["MlpSpec"]:
        if d is None:
            return None
        if d["kind"] == "dense":
            return cls("dense", int(d["ff"]))
        if d["kind"] == "moe":
            r, e = d["router"], d["expert"]
            g = r.get("groups") or {}
            return cls("moe", int(e["ff"]), experts=int(r["experts"]), top=int(r["top"]), groups=int(g.get("count", 1)), keep_groups=int(g.get("keep", g.get("count", 1))),
                       out_scale=float(r.get("scale", 1.0)), limit=float(e["limit"]))
        raise ValueError(f"unknown feed-forward kind {d['kind']!r}")


@dataclass
class LayerSpec:
    type: str
    mixer: ChunkedAttentionSpec
    mlp: Optional[MlpSpec]


MIXER_SPECS = {"attention": ChunkedAttentionSpec}


@dataclass
class BiluraxConfig:
    architecture: str = "Bilurax"
    vocab: int = 0
    width: int = 0
    norm_eps: float = 1e-6
    embedding_scale: float = 1.0
    logit_softcap: Optional[float] = None
    layers: List[LayerSpec] = field(default_factory=list)
    loop: Optional[LoopSpec] = None

    @classmethod
    def from_dict(cls, d: dict) -> "BiluraxConfig":
        layers = []
        for i, l in enumerate(d["layers"]):
            if l["type"] not in MIXER_SPECS:
                raise ValueError(f"layer {i}: unknown mixer type {l['type']!r}")
            layers.append(LayerSpec(l["type"], MIXER_SPECS[l["type"]].from_dict(l["mixer"]), MlpSpec.from_dict(l.get("mlp"))))
        norm = d.get("norm") or {}
        loop = d.get("loop")
        if loop is not None:
            loop = LoopSpec(int(loop["start"]), int(loop["stop"]), int(loop["times"]))
            if not (0 <= loop.start < loop.stop <= len(layers)) or loop.times < 1:
                raise ValueError(f"loop {loop} does not fit {len(layers)} layers")
        cap = d.get("logit_softcap")
        return cls(architecture=d.get("architecture", "Bilurax"), vocab=int(d["vocab"]), width=int(d["width"]), norm_eps=float(norm.get("eps", 1e-6)),
                   embedding_scale=float((d.get("embedding") or {}).get("scale", 1.0)), logit_softcap=float(cap) if cap else None, layers=layers, loop=loop)

    @classmethod
    def from_pretrained(cls, path: str) -> "BiluraxConfig":
        with open(os.path.join(path, "config.json") if os.path.isdir(path) else path) as f:
            return cls.from_dict(json.load(f))

    def layer_runs(self):
        """The order in which layers run: (layer index, number of the pass that this run OPENS or None).  A looped span
        contributes `times` runs of each of its layers; every run has a cache layer and a state row of its own."""
        n, lp = len(self.layers), self.loop
        if lp is None:
            return [(i, None) for i in range(n)]
        runs = [(i, None) for i in range(lp.start)]
        for t in range(lp.times):
            runs += [(i, t if i == lp.start else None) for i in range(lp.start, lp.stop)]
        return runs + [(i, None) for i in range(lp.stop, n)]

    # what the cache manager asks of a model
    @property
    def num_hidden_layers(self) -> int:
        return len(self.layer_runs())

    def cache_row_widths(self) -> List[int]:
        return [self.layers[i].mixer.cache_row_width() for i, _ in self.layer_runs()]

    def state_widths(self) -> List[int]:
        """every layer run keeps the previous token's mixer input (before the shift) per sequence"""
        return [self.width for _ in self.layer_runs()]

    def chunks(self) -> Optional[List[int]]:
        """The chunk lengths of the layers, when every layer's mask is chunked (then keys before the start of the current chunk of
        the longest chunk length are never read again); None when some layer reads every earlier position."""
        c = [l.mixer.chunk for l in self.layers]
        return None if any(x is None for x in c) else c
