"""Recurrent mixers with a matrix state per head.  KGatedDeltaRule (below) — the gated delta rule behind short convolutions.
KGatedLinearAttention — linear attention with a decay per key channel and a recurrent matrix state per head:

    q = W_q h / sqrt(dim) ,  k = W_k h ,  v = W_v h ,  a = sigmoid(W_a2 (W_a1 h) + b) ** (1 / tau)        (a per head and key channel)
    S_t = diag(a_t) S_{t-1} + k_t v_t^T ,  o_t = S_t^T q_t                                                  (S: dim x vdim per head, fp32)
    out = W_o (rmsnorm_vdim(o) * w * silu(W_g h))

    P     = [W_q ; W_k ; W_v ; W_g ; W_a1] h        one GEMM over the matrices that read the mixer input
    z     = W_a2 P[a1]                              GEMM (the low-rank decay logits; the bias joins in fp32 in the kernel)
    o     = scan over each sequence portion         ktb200_gla_scan: state rows of the cache manager in, state rows out
    out   = W_o (norm, gate)                        ktb200_gla_out + GEMM

The state starts at zero, is carried per sequence in the cache manager's double-buffered fp32 state rows
(models/custom_cache.PagedStateCache) and is the only thing a step keeps: there are no per-token cache rows.  Decay logits,
their log-sigmoid and exponential, the state and the per-head norm are fp32.  Tokens of a portion run in order, so a position's
result does not depend on where the prompt was cut.  `cache_idx` picks the cache layer (state rows), so one set of weights
can run several times per step with separate states.  (The reference has no recurrent mixer; its caches are per-token:
archive/ktransformers/models/custom_cache.py:26-200.)"""
from __future__ import annotations

import torch
from torch import nn

from .. import native


class KGatedLinearAttention(nn.Module):
    def __init__(self, width: int, spec, eps: float, dtype=torch.bfloat16, device="cuda"):
        super().__init__()
        P = lambda *shape: nn.Parameter(torch.zeros(shape, dtype=dtype, device=device), requires_grad=False)
        s = self.spec = spec
        self.width, self.eps = width, eps
        self.n_qk, self.n_v = s.heads * s.dim, s.heads * s.vdim
        self.rank = None           # rows of W_a1: known when the weights arrive
        self.w_in = None
        self.a2, self.a2_b = None, P(self.n_qk)
        self.norm = P(s.vdim)
        self.o = P(width, self.n_v)
        self._dtype, self._device = dtype, device

    def set_rank(self, rank: int):
        self.rank = rank
        n = 2 * self.n_qk + 2 * self.n_v + rank
        self.n_in = (n + 7) // 8 * 8
        self.a1_off = 2 * self.n_qk + 2 * self.n_v
        self.w_in = nn.Parameter(torch.zeros((self.n_in, self.width), dtype=self._dtype, device=self._device), requires_grad=False)
        self.a2 = nn.Parameter(torch.zeros((self.n_qk, rank), dtype=self._dtype, device=self._device), requires_grad=False)

    def load(self, loader, prefix: str):
        t = lambda n: loader.load_tensor(prefix + n, "cpu")
        a1 = t("a1")
        self.set_rank(a1.shape[0])
        self.w_in.data[:self.a1_off + self.rank].copy_(torch.cat([t("q"), t("k"), t("v"), t("g"), a1], 0))
        self.a2.data.copy_(t("a2"))
        self.a2_b.data.copy_(t("a2.b"))
        self.norm.data.copy_(t("norm"))
        self.o.data.copy_(t("o"))

    def forward(self, h: torch.Tensor, batch, cache, cache_idx: int) -> torch.Tensor:
        s, T, dev, dt = self.spec, h.shape[0], h.device, h.dtype
        lib, code, st = native.seq_lib(), native.GGML_BF16 if dt == torch.bfloat16 else native.GGML_F32, torch.cuda.current_stream(h.device).cuda_stream
        proj = torch.nn.functional.linear(h, self.w_in)
        z = torch.nn.functional.linear(proj[:, self.a1_off:self.a1_off + self.rank], self.a2)
        o = torch.empty((T, self.n_v), dtype=torch.float32, device=dev)
        native.check_seq(lib.ktb200_gla_scan(proj.data_ptr(), self.n_in, 0, self.n_qk, 2 * self.n_qk, z.data_ptr(), self.n_qk, self.a2_b.data_ptr(), float(s.tau), s.heads,
                                             s.dim, s.vdim, batch.seqs.data_ptr(), batch.seqs.stride(0), batch.n_seqs, T, cache.state[cache_idx].data_ptr(), o.data_ptr(),
                                             code, st))
        og = torch.empty((T, self.n_v), dtype=dt, device=dev)
        native.check_seq(lib.ktb200_gla_out(o.data_ptr(), self.norm.data_ptr(), float(self.eps), proj[:, 2 * self.n_qk + self.n_v:].data_ptr(), self.n_in, og.data_ptr(), T,
                                            s.heads, s.vdim, code, st))
        return torch.nn.functional.linear(og, self.o)


class KGatedDeltaRule(nn.Module):
    """The gated delta rule behind short causal convolutions — a recurrent mixer with a matrix state per value head:

        q, k, v = silu(conv(W_q h)), silu(conv(W_k h)), silu(conv(W_v h))     conv: a causal filter of `conv` taps along time on every channel, without bias
        q, k    = x * rsqrt(|x|^2 + unit_eps) per head ;  q also / sqrt(dim)              (kv_heads query/key heads, shared by
                                                                                            heads / kv_heads value heads each)
        eta     = sigmoid(W_b h) ;  a = exp(-rate * softplus(W_a h + dt_bias)), rate = exp(A_log)      one of each per value head
        M <- a M ;  r = eta (v - M^T k) ;  M <- M + k r^T ;  y = M^T q                     (M: dim x vdim per head, fp32)
        out     = W_o (rmsnorm_vdim(o) * w * silu(W_g h))

        P     = [W_q ; W_k ; W_v ; W_g ; W_b ; W_a] h      one GEMM over the matrices that read the mixer input
        prep                                               ktb200_delta_prep: convolution, activations, unit vectors, eta, a
        o     = scan over each sequence portion            ktb200_delta_scan: state rows of the cache manager in, state rows out
        out   = W_o (norm, gate)                           ktb200_gla_out + GEMM

    A sequence's state — the matrices and the last conv - 1 inputs of every convolved channel — lives in the cache manager's
    double-buffered fp32 state rows (models/custom_cache.PagedStateCache); there are no per-token cache rows.  Tokens of a
    portion run in order with the same arithmetic wherever the portion starts, so a position's result does not depend on
    where the prompt was cut.  `cache_idx` picks the cache layer.  (The reference has no recurrent mixer.)"""

    def __init__(self, width: int, spec, eps: float, dtype=torch.bfloat16, device="cuda"):
        super().__init__()
        P = lambda *shape, dt=dtype: nn.Parameter(torch.zeros(shape, dtype=dt, device=device), requires_grad=False)
        s = self.spec = spec
        if s.heads % s.kv_heads:
            raise ValueError("value heads must divide into the query/key heads")
        self.width, self.eps = width, eps
        self.n_qk, self.n_v = s.kv_heads * s.dim, s.heads * s.vdim
        self.g_off = 2 * self.n_qk + self.n_v
        self.b_off = self.g_off + self.n_v
        self.a_off = self.b_off + s.heads
        self.n_in = (self.a_off + s.heads + 7) // 8 * 8
        self.w_in = P(self.n_in, width)
        self.conv_w = P(s.channels, s.conv)
        self.a_log, self.dt_bias = P(s.heads, dt=torch.float32), P(s.heads, dt=torch.float32)
        self.norm = P(s.vdim)
        self.o = P(width, self.n_v)

    def load(self, loader, prefix: str):
        t = lambda n: loader.load_tensor(prefix + n, "cpu")
        self.w_in.data[:self.a_off + self.spec.heads].copy_(torch.cat([t("q"), t("k"), t("v"), t("g"), t("b"), t("a")], 0))
        self.conv_w.data.copy_(torch.cat([t("q.conv"), t("k.conv"), t("v.conv")], 0))
        self.a_log.data.copy_(t("A_log").float())
        self.dt_bias.data.copy_(t("dt_bias").float())
        self.norm.data.copy_(t("norm"))
        self.o.data.copy_(t("o"))

    def forward(self, h: torch.Tensor, batch, cache, cache_idx: int) -> torch.Tensor:
        s, T, dev, dt = self.spec, h.shape[0], h.device, h.dtype
        lib, code, st = native.seq_lib(), native.GGML_BF16 if dt == torch.bfloat16 else native.GGML_F32, torch.cuda.current_stream(h.device).cuda_stream
        state = cache.state[cache_idx]
        proj = torch.nn.functional.linear(h, self.w_in)
        f32 = lambda *shape: torch.empty(shape, dtype=torch.float32, device=dev)
        qn, kn, vv, beta, decay = f32(T, self.n_qk), f32(T, self.n_qk), f32(T, self.n_v), f32(T, s.heads), f32(T, s.heads)
        native.check_seq(lib.ktb200_delta_prep(proj.data_ptr(), self.n_in, 0, self.b_off, self.a_off, self.conv_w.data_ptr(), s.conv, self.a_log.data_ptr(),
                                               self.dt_bias.data_ptr(), s.heads, s.kv_heads, s.dim, s.vdim, float(s.unit_eps), batch.seq_of.data_ptr(), batch.seqs.data_ptr(),
                                               batch.seqs.stride(0), state.data_ptr(), state.stride(0), qn.data_ptr(), kn.data_ptr(), vv.data_ptr(), beta.data_ptr(),
                                               decay.data_ptr(), T, code, st))
        o = f32(T, self.n_v)
        native.check_seq(lib.ktb200_delta_scan(qn.data_ptr(), kn.data_ptr(), vv.data_ptr(), beta.data_ptr(), decay.data_ptr(), s.heads, s.kv_heads, s.dim, s.vdim,
                                               batch.seqs.data_ptr(), batch.seqs.stride(0), batch.n_seqs, state.data_ptr(), state.stride(0), o.data_ptr(), st))
        og = torch.empty((T, self.n_v), dtype=dt, device=dev)
        native.check_seq(lib.ktb200_gla_out(o.data_ptr(), self.norm.data_ptr(), float(self.eps), proj[:, self.g_off:].data_ptr(), self.n_in, og.data_ptr(), T,
                                            s.heads, s.vdim, code, st))
        return torch.nn.functional.linear(og, self.o)
