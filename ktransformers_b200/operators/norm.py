"""KGroupRMSNormShift — grouped RMS norm fused with the residual sum before it and the token shift after it.

One launch of `ktb200_group_rmsnorm_shift` (csrc/seq_ops.cu) per call:

    x_out = x_in + mult * (a + b) + row                   (a, b: the previous layer's branch outputs, when passed in; row: one
                                                           vector added to every token, e.g. the step vector of a looped pass)
    h     = x_out / sqrt(mean_g(x_out^2) + eps) * weight   per group g of `groups` equal consecutive parts, fp32
    hs_t  = h_t + (h_{t-1} - h_t) * shift                  (layers that mix in the previous token's normed row)

The residual stream stays fp32; h and hs are rounded once to the compute dtype.  h_{t-1} of the first token of a portion
comes from the cache manager's state rows (models/custom_cache.PagedStateCache), which hold it in fp32 — the same value the
kernel recomputes when the previous token is part of the same launch, so results do not depend on where a prompt was cut.
(The reference's norms are plain torch modules, archive/ktransformers/models/modeling_deepseek_v3.py:65-80.)"""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from .. import native

GGML_OF = {torch.bfloat16: native.GGML_BF16, torch.float32: native.GGML_F32}


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


class KGroupRMSNormShift(nn.Module):
    def __init__(self, width: int, groups: int, eps: float, shift: bool, dtype=torch.bfloat16, device="cuda"):
        super().__init__()
        if width % groups:
            raise ValueError("the width must divide into the norm groups")
        self.width, self.groups, self.eps = width, groups, eps
        self.weight = nn.Parameter(torch.ones(width, dtype=dtype, device=device), requires_grad=False)
        self.shift = nn.Parameter(torch.zeros(width, dtype=dtype, device=device), requires_grad=False) if shift else None

    def load(self, loader, norm_key: str, shift_key: Optional[str] = None):
        self.weight.data.copy_(loader.load_tensor(norm_key, "cpu"))
        if self.shift is not None:
            self.shift.data.copy_(loader.load_tensor(shift_key, "cpu"))

    def forward(self, x: torch.Tensor, delta_a=None, delta_b=None, mult: float = 1.0, batch=None, state: Optional[torch.Tensor] = None, want_h: bool = True,
                row_add: Optional[torch.Tensor] = None):
        """x [T, width] fp32; delta_a / delta_b [T, width] fp32 or the compute dtype; row_add [width] fp32.  Returns (residual after
        the sum, h or None, hs or None)."""
        T = x.shape[0]
        dt = self.weight.dtype
        add = delta_a is not None or delta_b is not None or row_add is not None
        assert row_add is None or (row_add.dtype == torch.float32 and row_add.is_contiguous() and row_add.shape == (self.width,))
        x_out = torch.empty_like(x) if add else x
        h = torch.empty((T, self.width), dtype=dt, device=x.device) if want_h else None
        hs = torch.empty((T, self.width), dtype=dt, device=x.device) if self.shift is not None else None
        for d in (delta_a, delta_b):
            assert d is None or (d.is_contiguous() and d.shape == x.shape)
        native.check_seq(native.seq_lib().ktb200_group_rmsnorm_shift(
            x.data_ptr(), _ptr(delta_a), GGML_OF[delta_a.dtype] if delta_a is not None else 0, _ptr(delta_b),
            GGML_OF[delta_b.dtype] if delta_b is not None else 0, float(mult), _ptr(row_add), x_out.data_ptr() if add else None, self.weight.data_ptr(), self.groups,
            float(self.eps), _ptr(self.shift), _ptr(batch.prev_idx) if hs is not None else None, _ptr(batch.rd_row) if hs is not None else None,
            _ptr(batch.wr_row) if hs is not None else None, _ptr(state) if hs is not None else None, _ptr(h), _ptr(hs), T, self.width, GGML_OF[dt],
            torch.cuda.current_stream(x.device).cuda_stream))
        return x_out, h, hs


class KGroupRMSNorm(nn.Module):
    """One grouped RMS norm weight of a layer that norms BOTH sides of every sublayer, `x <- x + post(sublayer(pre(x)))`.
    The norms never run alone: `KGroupRMSNorm.fused` is one `ktb200_group_rmsnorm_sandwich` launch (csrc/seq_mixers.cu) for

        x_out = x_in + gnorm(y) * post.weight + row       the sublayer's output y normed and added to the fp32 residual
        h     = gnorm(x_out) * pre.weight                  the NEXT sublayer's input, rounded once to the compute dtype

    with every term optional (no x_in / post: the stream restarts from y; no pre: nothing follows, or with `cast_h` the next
    sublayer reads the residual itself and h is x_out rounded to the compute dtype).  `weight_offset = 1`: the weight is
    zero-centred and the row is scaled by 1 + weight (added in fp32 in the kernel)."""

    def __init__(self, width: int, groups: int, eps: float, dtype=torch.bfloat16, device="cuda", weight_offset: float = 0.0):
        super().__init__()
        if width % groups:
            raise ValueError("the width must divide into the norm groups")
        self.width, self.groups, self.eps, self.weight_offset = width, groups, eps, float(weight_offset)
        self.weight = nn.Parameter(torch.full((width,), 1.0 - float(weight_offset), dtype=dtype, device=device), requires_grad=False)

    def load(self, loader, key: str):
        self.weight.data.copy_(loader.load_tensor(key, "cpu"))

    @staticmethod
    def fused(x_in: Optional[torch.Tensor], y: torch.Tensor, post: Optional["KGroupRMSNorm"], pre: Optional["KGroupRMSNorm"], row_add: Optional[torch.Tensor] = None,
              keep_x: bool = True, cast_h: bool = False):
        """x_in [T, width] fp32 or None, y [T, width] fp32 or the compute dtype.  Returns (x_out fp32 or None, h or None); with
        `cast_h` and no `pre`, h is x_out in the compute dtype (x_out itself when that is fp32)."""
        ref = pre if pre is not None else post
        T, D = y.shape
        assert y.is_contiguous() and (x_in is None or x_in.is_contiguous()) and D == ref.width
        dt = ref.weight.dtype
        x_out = torch.empty((T, D), dtype=torch.float32, device=y.device) if keep_x or pre is None else None
        plain_h = cast_h and pre is None and dt != torch.float32
        h = torch.empty((T, D), dtype=dt, device=y.device) if pre is not None or plain_h else None
        native.check_seq(native.seq_lib().ktb200_group_rmsnorm_sandwich(
            _ptr(x_in), y.data_ptr(), GGML_OF[y.dtype], post.weight.data_ptr() if post is not None else None, _ptr(row_add), _ptr(x_out),
            pre.weight.data_ptr() if pre is not None else None, _ptr(h), ref.groups, float(ref.eps), float(ref.weight_offset), T, D, GGML_OF[dt],
            torch.cuda.current_stream(y.device).cuda_stream))
        if cast_h and pre is None and not plain_h:
            h = x_out
        return x_out, h
