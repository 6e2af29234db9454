"""KPolyNormMLP — a two-matrix feed-forward whose activation is a cubic polynomial of per-token normalised powers:

    z = W_up h ;  act = c0 N(z) + c1 N(z^2) + c2 N(z^3) + c3 ,  N(y) = y / sqrt(mean(y^2) + eps) over the ff values ;  W_down act

The two products are library GEMMs; the activation is one `ktb200_poly_norm` launch (csrc/seq_ops.cu: the three mean squares
and the polynomial in fp32, one rounding to the compute dtype).  (The reference's gated MLP: modeling_deepseek_v3.py:385-397.)"""
from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import nn

from .. import native
from .norm import GGML_OF


class KPolyNormMLP(nn.Module):
    def __init__(self, width: int, ff: int, eps: float, dtype=torch.bfloat16, device="cuda"):
        super().__init__()
        self.width, self.ff, self.eps = width, ff, eps
        self.up = nn.Parameter(torch.empty((ff, width), dtype=dtype, device=device), requires_grad=False)
        self.down = nn.Parameter(torch.empty((width, ff), dtype=dtype, device=device), requires_grad=False)
        self.coef = nn.Parameter(torch.zeros(4, dtype=torch.float32, device=device), requires_grad=False)

    def load(self, loader, prefix: str):
        self.up.data.copy_(loader.load_tensor(prefix + "up", "cpu"))
        self.down.data.copy_(loader.load_tensor(prefix + "down", "cpu"))
        self.coef.data.copy_(loader.load_tensor(prefix + "act", "cpu").float())

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        z = F.linear(h, self.up)
        a = torch.empty_like(z)
        native.check_seq(native.seq_lib().ktb200_poly_norm(z.data_ptr(), a.data_ptr(), self.coef.data_ptr(), float(self.eps), z.shape[0], self.ff,
                                                           GGML_OF[z.dtype], torch.cuda.current_stream(z.device).cuda_stream))
        return F.linear(a, self.down)


class KXIELUMLP(nn.Module):
    """A two-matrix feed-forward with the xIELU activation, a quadratic above zero and a saturating exponential below:

        z = W_up h ;  act(z) = sp(p) z^2 + z/2            (z > 0)
                      act(z) = (1/2 + sp(q)) (e^z - 1 - z) + z/2   (z <= 0) ,  sp = softplus ;  W_down act

    The two products are library GEMMs; the activation is one `ktb200_xielu` launch (csrc/seq_mixers.cu, fp32 inside, softplus
    of the two learned numbers on the device)."""

    def __init__(self, width: int, ff: int, dtype=torch.bfloat16, device="cuda"):
        super().__init__()
        self.width, self.ff = width, ff
        self.up = nn.Parameter(torch.empty((ff, width), dtype=dtype, device=device), requires_grad=False)
        self.down = nn.Parameter(torch.empty((width, ff), dtype=dtype, device=device), requires_grad=False)
        self.pq = nn.Parameter(torch.zeros(2, dtype=torch.float32, device=device), requires_grad=False)

    def load(self, loader, prefix: str):
        self.up.data.copy_(loader.load_tensor(prefix + "up", "cpu"))
        self.down.data.copy_(loader.load_tensor(prefix + "down", "cpu"))
        self.pq.data.copy_(loader.load_tensor(prefix + "act", "cpu").float())

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        z = F.linear(h, self.up)
        a = torch.empty_like(z)
        native.check_seq(native.seq_lib().ktb200_xielu(z.data_ptr(), a.data_ptr(), self.pq.data_ptr(), z.numel(), GGML_OF[z.dtype],
                                                       torch.cuda.current_stream(z.device).cuda_stream))
        return F.linear(a, self.down)


class KGatedMLP(nn.Module):
    """A three-matrix gated feed-forward, W_down (act(W_gate h) * (W_up h)), act = "silu" or "gelu_tanh"
    (u / 2 * (1 + tanh(0.7978845608 (u + 0.044715 u^3)))).  Gate and up are one stacked GEMM, the activation and the product one
    `ktb200_gated_act_mul` launch (csrc/seq_mixers.cu, fp32 inside), down a GEMM.  (The reference's gated MLP:
    modeling_deepseek_v3.py:385-397.)"""

    ACTS = {"silu": 0, "gelu_tanh": 1}

    def __init__(self, width: int, ff: int, act: str = "silu", dtype=torch.bfloat16, device="cuda"):
        super().__init__()
        self.width, self.ff, self.act = width, ff, self.ACTS[act]
        self.gate_up = nn.Parameter(torch.empty((2 * ff, width), dtype=dtype, device=device), requires_grad=False)
        self.down = nn.Parameter(torch.empty((width, ff), dtype=dtype, device=device), requires_grad=False)

    def load(self, loader, prefix: str):
        self.gate_up.data.copy_(torch.cat([loader.load_tensor(prefix + "gate", "cpu"), loader.load_tensor(prefix + "up", "cpu")], 0))
        self.down.data.copy_(loader.load_tensor(prefix + "down", "cpu"))

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        gu = F.linear(h, self.gate_up)
        a = torch.empty((h.shape[0], self.ff), dtype=gu.dtype, device=gu.device)
        native.check_seq(native.seq_lib().ktb200_gated_act_mul(gu.data_ptr(), gu.data_ptr() + self.ff * gu.element_size(), 2 * self.ff, a.data_ptr(), gu.shape[0], self.ff,
                                                               self.act, 0.0, GGML_OF[gu.dtype], torch.cuda.current_stream(gu.device).cuda_stream))
        return F.linear(a, self.down)


class KReluSquaredMLP(nn.Module):
    """A two-matrix feed-forward without biases, W_down relu(W_up h)^2.  The two products are library GEMMs; the activation is one
    `ktb200_relu_squared` launch (csrc/seq_mixers.cu, fp32 inside, one rounding to the compute dtype)."""

    def __init__(self, width: int, ff: int, dtype=torch.bfloat16, device="cuda"):
        super().__init__()
        self.width, self.ff = width, ff
        self.up = nn.Parameter(torch.empty((ff, width), dtype=dtype, device=device), requires_grad=False)
        self.down = nn.Parameter(torch.empty((width, ff), dtype=dtype, device=device), requires_grad=False)

    def load(self, loader, prefix: str):
        self.up.data.copy_(loader.load_tensor(prefix + "up", "cpu"))
        self.down.data.copy_(loader.load_tensor(prefix + "down", "cpu"))

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        z = F.linear(h, self.up)
        a = torch.empty_like(z)
        native.check_seq(native.seq_lib().ktb200_relu_squared(z.data_ptr(), a.data_ptr(), z.numel(), GGML_OF[z.dtype], torch.cuda.current_stream(z.device).cuda_stream))
        return F.linear(a, self.down)
