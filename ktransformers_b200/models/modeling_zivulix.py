"""Zivulix — a decoder whose sublayers read the residual stream itself and norm only what they add to it,

    r <- r + N1(mix(r)) ;  r <- r + N2(ffn(r))          (N: RMS norms with zero-centred weights; r: the fp32 residual stream)

with one of three mixers per layer — soft-max attention over grouped heads with a partial rotation, unit-rms queries and keys,
capped scores, a sliding window and values blended with the first such layer's; latent attention (one cached latent per token
plus a shared rotated key part); the gated delta rule behind short convolutions, a recurrent matrix state per head — and a
gated GELU feed-forward or none.  The embedding is normed before the first layer.  The layer list, every size and every
constant come from `ZivulixConfig`.

The model is assembled from the framework's operators (operators/norm.py, attention.py, linear_attention.py, mlp.py); its
`forward(batch, cache)` is the step function the engine drives: a flattened ragged batch of prompt portions and decode tokens
(models/custom_cache.ForwardBatch) against the paged cache rows and per-sequence state rows of
models/custom_cache.PagedStateCache.  Every residual sum is folded into a norm launch: a sublayer's output is normed, added,
and the sum rounded once to the compute dtype for the next sublayer's GEMMs."""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.nn.functional as F
from torch import nn

from ..operators.attention import KCappedWindowAttention, KLatentWindowAttention
from ..operators.linear_attention import KGatedDeltaRule
from ..operators.mlp import KGatedMLP
from ..operators.norm import KGroupRMSNorm
from .configuration_zivulix import ZivulixConfig
from .custom_cache import ForwardBatch, PagedStateCache


class ZivulixDecoderLayer(nn.Module):
    def __init__(self, config: ZivulixConfig, layer_idx: int, dtype, device):
        super().__init__()
        spec = config.layers[layer_idx]
        norm = lambda: KGroupRMSNorm(config.width, 1, config.norm_eps, dtype=dtype, device=device, weight_offset=1.0)
        self.layer_idx, self.type = layer_idx, spec.type
        if spec.type == "attention":
            self.mix = KCappedWindowAttention(config.width, spec.mixer, config.norm_eps, dtype=dtype, device=device)
        elif spec.type == "latent_attention":
            self.mix = KLatentWindowAttention(config.width, spec.mixer, config.norm_eps, layer_idx, dtype=dtype, device=device)
        else:
            self.mix = KGatedDeltaRule(config.width, spec.mixer, config.norm_eps, dtype=dtype, device=device)
        self.norm1 = norm()
        if spec.mlp is None:
            self.mlp = self.norm2 = None
        else:
            self.mlp, self.norm2 = KGatedMLP(config.width, spec.mlp.ff, act="gelu_tanh", dtype=dtype, device=device), norm()

    def load(self, loader, prefix: str):
        self.norm1.load(loader, prefix + "norm1")
        self.mix.load(loader, prefix + "mix.")
        if self.mlp is not None:
            self.norm2.load(loader, prefix + "norm2")
            self.mlp.load(loader, prefix + "mlp.")


class ZivulixForCausalLM(nn.Module):
    config_class = ZivulixConfig

    def __init__(self, config: ZivulixConfig, dtype=torch.bfloat16, device="cuda"):
        super().__init__()
        self.config, self.dtype, self.device = config, dtype, torch.device(device)
        P = lambda *shape: nn.Parameter(torch.empty(shape, dtype=dtype, device=device), requires_grad=False)
        norm = lambda: KGroupRMSNorm(config.width, 1, config.norm_eps, dtype=dtype, device=device, weight_offset=1.0)
        self.embed, self.embed_norm = P(config.vocab, config.width), norm()
        self.layers = nn.ModuleList([ZivulixDecoderLayer(config, i, dtype, device) for i in range(len(config.layers))])
        self.first_value_mixer = config.first_value_mixer()
        self.final_norm = norm()
        self.head = P(config.vocab, config.width)

    def load(self, loader):
        self.embed.data.copy_(loader.load_tensor("embed", "cpu"))
        self.embed_norm.load(loader, "embed.norm")
        for i, layer in enumerate(self.layers):
            layer.load(loader, f"l{i}.")
        self.final_norm.load(loader, "final.norm")
        self.head.data.copy_(loader.load_tensor("head", "cpu"))

    def make_cache(self, max_tokens: int, max_slots: int = 8, page_size: int = 64) -> PagedStateCache:
        c = self.config
        return PagedStateCache(c.cache_row_widths(), c.state_widths(), max_tokens, max_slots, self.device, dtype=self.dtype, page_size=page_size, window=c.max_window())

    def decode_is_capturable(self, max_batch: int = 47) -> bool:
        """No launch of a step reads anything back on the host (the value blend's weight is read on the device)."""
        return True

    @torch.no_grad()
    def forward(self, batch: ForwardBatch, cache: PagedStateCache, residual_trace: Optional[List[torch.Tensor]] = None) -> torch.Tensor:
        """Runs the batch's tokens from the cache and state earlier steps left; returns fp32 logits [len(batch.want), vocab]."""
        fused = KGroupRMSNorm.fused
        x, h = fused(None, self.embed.index_select(0, batch.tokens), self.embed_norm, None, cast_h=True)
        v_first = None
        # (x, y, post): the residual before the pending sublayer output y, whose norm `post` joins the next fused launch
        y = post = None
        for i, layer in enumerate(self.layers):
            if y is not None:
                x, h = fused(x, y, post, None, cast_h=True)
            if layer.type == "attention":
                blends = layer.mix.spec.v_mix and i != self.first_value_mixer
                y, v_own = layer.mix(h, batch, cache, i, v_first if blends else None)
                if i == self.first_value_mixer:
                    v_first = v_own
            else:
                y = layer.mix(h, batch, cache, i)
            post = layer.norm1
            if layer.mlp is not None:
                x, h = fused(x, y, post, None, cast_h=True)
                y, post = layer.mlp(h), layer.norm2
            if residual_trace is not None:
                residual_trace.append(fused(x, y, post, None)[0])
        # the last sum and the final norm in one launch, for the rows asked for only
        _, h = fused(x.index_select(0, batch.want), y.index_select(0, batch.want), post, self.final_norm, keep_x=False)
        return F.linear(h, self.head).float()
