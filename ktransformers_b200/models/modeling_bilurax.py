"""Bilurax — a pre-norm decoder whose mixers read a token-shifted input,

    h = norm1(x) ;  x <- x + mixer(h + (h_prev - h) * mu) ;  x <- x + ff(norm2(x))          (fp32 residual stream)

with soft-max attention inside chunks of the sequence as the mixer (queries and keys normed over their whole projection, unit-rms
values, a learned temperature per head, capped scores, no positions in the scores), a relu-squared feed-forward or a mixture of
clamped gated experts behind a grouped sigmoid router (or none), and a span of layers that runs several times in a row with the
same weights: every pass but the first opens with x <- x + x0 (x0: the scaled embedding), every pass with x <- x + step[pass], and
keeps caches and shift states of its own.  The embedding table is also the output projection; the logits are capped.  The layer
list, the span, every size and every constant come from `BiluraxConfig`.

The model is assembled from the framework's operators (operators/norm.py, attention.py, mlp.py, experts.py, gate.py); its
`forward(batch, cache)` is the step function the engine drives: a flattened ragged batch of prompt portions and decode tokens
(models/custom_cache.ForwardBatch) against the paged cache rows and per-sequence state rows of
models/custom_cache.PagedStateCache, one cache layer and one state row per layer RUN.  Every residual sum is folded into the next
norm launch, together with the pass openings."""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.nn.functional as F
from torch import nn

from .. import native
from ..operators.attention import KChunkedSoftmaxAttention
from ..operators.experts import KGroupedSigmoidMoE
from ..operators.mlp import KReluSquaredMLP
from ..operators.norm import GGML_OF, KGroupRMSNormShift
from .configuration_bilurax import BiluraxConfig
from .custom_cache import ForwardBatch, PagedStateCache

MIXERS = {"attention": KChunkedSoftmaxAttention}


class BiluraxDecoderLayer(nn.Module):
    def __init__(self, config: BiluraxConfig, layer_idx: int, dtype, device):
        super().__init__()
        spec = config.layers[layer_idx]
        self.layer_idx = layer_idx
        self.norm1 = KGroupRMSNormShift(config.width, 1, config.norm_eps, shift=True, dtype=dtype, device=device)
        self.mix = MIXERS[spec.type](config.width, spec.mixer, config.norm_eps, dtype=dtype, device=device)
        f = spec.mlp
        if f is None:
            self.mlp = self.norm2 = None
        else:
            self.norm2 = KGroupRMSNormShift(config.width, 1, config.norm_eps, shift=False, dtype=dtype, device=device)
            if f.kind == "dense":
                self.mlp = KReluSquaredMLP(config.width, f.ff, dtype=dtype, device=device)
            else:
                self.mlp = KGroupedSigmoidMoE(config.width, f.ff, f.experts, f.top, f.groups, f.keep_groups, f.out_scale, f.limit, dtype=dtype, device=device)

    def load(self, loader, prefix: str):
        self.norm1.load(loader, prefix + "norm1", prefix + "shift")
        self.mix.load(loader, prefix + "mix.")
        if self.mlp is not None:
            self.norm2.load(loader, prefix + "norm2")
            self.mlp.load(loader, prefix + "mlp.")


class BiluraxForCausalLM(nn.Module):
    config_class = BiluraxConfig

    def __init__(self, config: BiluraxConfig, dtype=torch.bfloat16, device="cuda"):
        super().__init__()
        self.config, self.dtype, self.device = config, dtype, torch.device(device)
        self.embed = nn.Parameter(torch.empty((config.vocab, config.width), dtype=dtype, device=device), requires_grad=False)
        self.layers = nn.ModuleList([BiluraxDecoderLayer(config, i, dtype, device) for i in range(len(config.layers))])
        self.runs = config.layer_runs()
        if config.loop is not None:
            self.loop_step = nn.Parameter(torch.empty((config.loop.times, config.width), dtype=torch.float32, device=device), requires_grad=False)
        self.final_norm = KGroupRMSNormShift(config.width, 1, config.norm_eps, shift=False, dtype=dtype, device=device)

    def load(self, loader):
        self.embed.data.copy_(loader.load_tensor("embed", "cpu"))
        for i, layer in enumerate(self.layers):
            layer.load(loader, f"l{i}.")
        if self.config.loop is not None:
            self.loop_step.data.copy_(loader.load_tensor("loop.step", "cpu").float())
        self.final_norm.load(loader, "final.norm")

    def make_cache(self, max_tokens: int, max_slots: int = 8, page_size: int = 64) -> PagedStateCache:
        c = self.config
        return PagedStateCache(c.cache_row_widths(), c.state_widths(), max_tokens, max_slots, self.device, dtype=self.dtype, page_size=page_size, window=None,
                               chunks=c.chunks())

    def decode_is_capturable(self, max_batch: int = 47) -> bool:
        """Whether a decode step of up to `max_batch` sequences makes no host read (then the engine may replay it as a CUDA
        graph)."""
        for layer in self.layers:
            e = getattr(layer.mlp, "experts", None)
            if e is not None and not e.small_batches_stay_on_device(layer.mlp.router.top, self.dtype, max_batch):
                return False
        return True

    @torch.no_grad()
    def forward(self, batch: ForwardBatch, cache: PagedStateCache, residual_trace: Optional[List[torch.Tensor]] = None) -> torch.Tensor:
        """Runs the batch's tokens from the cache and state earlier steps left; returns fp32 logits [len(batch.want), vocab]."""
        c = self.config
        x0 = self.embed.index_select(0, batch.tokens).float() * c.embedding_scale
        # x: the residual before the pending sublayer output y (None: nothing pending), which the next norm launch adds
        x, y = x0, None
        for run, (i, opens_pass) in enumerate(self.runs):
            layer = self.layers[i]
            again = x0 if opens_pass is not None and opens_pass > 0 else None                                      # every pass but the first re-reads the embedding
            row = self.loop_step[opens_pass] if opens_pass is not None else None
            x, _, hs = layer.norm1(x, y, again, 1.0, batch, cache.state[run], want_h=False, row_add=row)
            y = layer.mix(hs, batch, cache, run)
            if layer.mlp is not None:
                x, h, _ = layer.norm2(x, y)
                y = layer.mlp(h)
            if residual_trace is not None:
                residual_trace.append(x + y.float())
        rows = batch.want
        if rows.shape[0] == 0:      # a prompt portion whose logits nobody asked for: its cache rows and states are written, that is all
            return torch.empty((0, c.vocab), dtype=torch.float32, device=x.device)
        _, h, _ = self.final_norm(x.index_select(0, rows), y.index_select(0, rows) if y is not None else None)
        z = F.linear(h, self.embed)
        if c.logit_softcap is None:
            return z.float()
        out = torch.empty(z.shape, dtype=torch.float32, device=z.device)
        native.check_seq(native.seq_lib().ktb200_softcap(z.data_ptr(), out.data_ptr(), z.numel(), float(c.logit_softcap), GGML_OF[z.dtype],
                                                         torch.cuda.current_stream(z.device).cuda_stream))
        return out
