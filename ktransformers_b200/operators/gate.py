"""MoE router operators.  API mirror of archive/ktransformers/operators/gate.py:

    KMoEGateBase  :23-89   load_weights(weight, e_score_correction_bias) contract
    KMoEGate      :91-127  the reference delegates to the torch MoEGate.forward (≈10 ATen kernels)
    KMoEGateB200  the same routing as two sm_100a kernels (ktb200_moe_gate_forward): fp32 GEMV +
                  warp-shuffle grouped top-k; ids are bit-exact vs torch up to fp32 summation-order ties.
"""
from __future__ import annotations

import ctypes as C

import torch
from torch import nn

from .. import native
from ..util.custom_gguf import TORCH_TO_GGML_HIDDEN
from .base_operator import BaseInjectedModule

_SCORING = {"sigmoid": 0, "softmax": 1, "topk_softmax": 2}
_TOPK = {"noaux_tc": 0, "greedy": 1, "group_limited_greedy": 2}


class KMoEGateBase:
    def __init__(self, key, gguf_loader, config, orig_module, device: str = "cuda", **kwargs):
        self.key = key
        self.gguf_loader = gguf_loader
        self.config = config
        self.device = device
        self.orig_module = orig_module

    def load_weights(self, override_key=None, device: str = "cpu"):
        keys = override_key if override_key is not None else [self.key]
        for key in keys:
            if self.gguf_loader.has_tensor(key + ".weight"):
                res = {"weight": self.gguf_loader.load_gguf_tensor(key + ".weight", device=device, target_dtype=torch.float32)}
                if self.gguf_loader.has_tensor(key + ".e_score_correction_bias"):
                    res["e_score_correction_bias"] = self.gguf_loader.load_gguf_tensor(key + ".e_score_correction_bias", device=device, target_dtype=torch.float32)
                return res
        raise ValueError(f"Experts {keys} not found in gguf_loader")


class KMoEGate(BaseInjectedModule, KMoEGateBase):
    """Reference behaviour: torch MoEGate.forward on the loaded weights."""

    def __init__(self, key, gguf_loader, config, orig_module=None, generate_device: str = "cuda", prefill_device: str = "cuda", **kwargs):
        BaseInjectedModule.__init__(self, key, gguf_loader, config, orig_module, prefill_device, generate_device, **kwargs)
        KMoEGateBase.__init__(self, key, gguf_loader, config, orig_module, generate_device, **kwargs)

    def forward(self, hidden_states):
        return self.orig_module.forward(hidden_states)

    def load(self, w=None, device: str | None = None):
        device = device or self.device
        if w is None:
            w = self.load_weights(device=device)
        if not isinstance(w, dict):
            raise ValueError("Invalid weight type")
        self.orig_module.weight = nn.Parameter(w["weight"].to(device), requires_grad=False)
        if "e_score_correction_bias" in w:
            self.orig_module.e_score_correction_bias = nn.Parameter(w["e_score_correction_bias"].to(device), requires_grad=False)

    def unload(self):
        self.orig_module.weight = None
        if hasattr(self.orig_module, "e_score_correction_bias"):
            self.orig_module.e_score_correction_bias = None


class KMoEGateB200(KMoEGate):
    """Same interface, routing done by libktb200 on the GPU (no torch ops on the decode path)."""

    def load(self, w=None, device: str | None = None):
        native.lib()  # fail loudly without the CUDA library
        super().load(w, device)
        m = self.orig_module
        self._w = m.weight.data.to(torch.float32).contiguous()
        b = getattr(m, "e_score_correction_bias", None)
        self._b = b.data.to(torch.float32).contiguous() if b is not None else None

    def forward(self, hidden_states, bsz_tensor=None):
        m = self.orig_module
        x = hidden_states.reshape(-1, hidden_states.shape[-1]).contiguous()
        n = x.shape[0]
        idx = torch.empty((n, m.top_k), dtype=torch.int64, device=x.device)
        wt = torch.empty((n, m.top_k), dtype=torch.float32, device=x.device)
        cfg = native.GateConfig(m.n_routed_experts, x.shape[1], m.top_k, m.n_group or 1, m.topk_group or 1,
                                _SCORING[m.scoring_func], _TOPK[m.topk_method], int(bool(m.norm_topk_prob)),
                                float(m.routed_scaling_factor), self._w.data_ptr(),
                                self._b.data_ptr() if self._b is not None else None, TORCH_TO_GGML_HIDDEN[x.dtype])
        native.check(native.lib().ktb200_moe_gate_forward(
            C.byref(cfg), n, x.data_ptr(), idx.data_ptr(), wt.data_ptr(), None,
            bsz_tensor.data_ptr() if bsz_tensor is not None else None, torch.cuda.current_stream(x.device).cuda_stream))
        return idx, wt


class KSoftmaxTopKGate(nn.Module):
    """Soft-max over all experts, the `top` largest kept with their scores as weights (no re-scaling): the router kernel's
    `scoring = softmax, topk_method = greedy, norm_topk_prob = 0, routed_scaling_factor = 1` case (DeepSeek-V2's gate,
    archive/ktransformers/models/modeling_deepseek.py:386-459), as a plain module for models that are built on the operators
    directly.  Logits are an fp32 GEMV over fp32 router weights.  The kernel is built for decode-sized batches (one CTA row per
    token); from `gemm_min_tokens` tokens the logits are one fp32 library GEMM (TF32 off) followed by torch's soft-max and
    top-k, the way the reference's KMoEGate runs its torch gate (operators/gate.py:91-127)."""

    gemm_min_tokens = 48

    def __init__(self, width: int, experts: int, top: int, device="cuda"):
        super().__init__()
        self.width, self.experts, self.top = width, experts, top
        self.weight = nn.Parameter(torch.empty((experts, width), dtype=torch.float32, device=device), requires_grad=False)

    def load(self, loader, key: str):
        self.weight.data.copy_(loader.load_tensor(key, "cpu").float())

    def forward(self, x: torch.Tensor):
        n = x.shape[0]
        kernel_fits = self.width % 4 == 0 and self.experts <= 512 and self.top <= 32        # the router kernel's shape limits
        if n >= self.gemm_min_tokens or not kernel_fits:
            scores = torch.softmax(nn.functional.linear(x.float(), self.weight), dim=-1)
            wt, idx = torch.topk(scores, self.top, dim=-1)
            return idx, wt.contiguous()
        idx = torch.empty((n, self.top), dtype=torch.int64, device=x.device)
        wt = torch.empty((n, self.top), dtype=torch.float32, device=x.device)
        cfg = native.GateConfig(self.experts, self.width, self.top, 1, 1, _SCORING["softmax"], _TOPK["greedy"], 0, 1.0, self.weight.data_ptr(), None,
                                TORCH_TO_GGML_HIDDEN[x.dtype])
        native.check_seq(native.seq_lib().ktb200_moe_gate_forward(C.byref(cfg), n, x.data_ptr(), idx.data_ptr(), wt.data_ptr(), None, None,
                                                                  torch.cuda.current_stream(x.device).cuda_stream))
        return idx, wt


class KTopKSoftmaxGate(nn.Module):
    """Logits `W x + b` in fp32, the `top` largest chosen, weights = soft-max over the chosen logits only (so one chosen expert
    weighs 1): the router kernel's `scoring = topk_softmax` case, where the bias belongs to the logits.  As for
    KSoftmaxTopKGate, batches from `gemm_min_tokens` tokens run an fp32 library GEMM (TF32 off) and torch's top-k."""

    gemm_min_tokens = 48

    def __init__(self, width: int, experts: int, top: int, device="cuda"):
        super().__init__()
        self.width, self.experts, self.top = width, experts, top
        self.weight = nn.Parameter(torch.empty((experts, width), dtype=torch.float32, device=device), requires_grad=False)
        self.bias = nn.Parameter(torch.zeros(experts, dtype=torch.float32, device=device), requires_grad=False)

    def load(self, loader, key: str):
        self.weight.data.copy_(loader.load_tensor(key, "cpu").float())
        self.bias.data.copy_(loader.load_tensor(key + ".b", "cpu").float())

    def forward(self, x: torch.Tensor):
        n = x.shape[0]
        kernel_fits = self.width % 4 == 0 and self.experts <= 512 and self.top <= 32
        if n >= self.gemm_min_tokens or not kernel_fits:
            val, idx = torch.topk(torch.addmm(self.bias, x.float(), self.weight.t()), self.top, dim=-1)
            return idx, torch.softmax(val, dim=-1).contiguous()
        idx = torch.empty((n, self.top), dtype=torch.int64, device=x.device)
        wt = torch.empty((n, self.top), dtype=torch.float32, device=x.device)
        cfg = native.GateConfig(self.experts, self.width, self.top, 1, 1, _SCORING["topk_softmax"], _TOPK["greedy"], 1, 1.0, self.weight.data_ptr(),
                                self.bias.data_ptr(), TORCH_TO_GGML_HIDDEN[x.dtype])
        native.check_seq(native.seq_lib().ktb200_moe_gate_forward(C.byref(cfg), n, x.data_ptr(), idx.data_ptr(), wt.data_ptr(), None, None,
                                                                  torch.cuda.current_stream(x.device).cuda_stream))
        return idx, wt


class KGroupedSigmoidGate(nn.Module):
    """Sigmoid scores s = sigmoid(W x) in fp32; experts are CHOSEN by s + correction among the experts of the `keep_groups` groups
    (of experts / groups neighbours) whose two largest choice scores sum highest, every other expert counting as minus infinity;
    the WEIGHTS are the chosen experts' s, divided by their sum (+ 1e-20) and multiplied by `out_scale`: the router kernel's
    `scoring = sigmoid, topk_method = noaux_tc` case (DeepSeek-V3's gate, archive/ktransformers/models/modeling_deepseek_v3.py:430-481)
    with `norm_topk_prob = 2`: the weights are normalised also when a token uses ONE expert (whose weight is then `out_scale`; the
    reference's gate leaves a single choice un-normalised), as a plain module for models that are built on the operators
    directly.  Decode-sized batches run the one-launch router kernel (fp32 GEMV + selection); from `gemm_min_tokens` tokens the
    logits are one fp32 library GEMM (TF32 off) and the selection is `ktb200_moe_gate_select`, a CTA per token."""

    gemm_min_tokens = 48

    def __init__(self, width: int, experts: int, top: int, groups: int, keep_groups: int, out_scale: float, device="cuda"):
        super().__init__()
        if experts % groups or not (1 <= keep_groups <= groups) or top > keep_groups * (experts // groups):
            raise ValueError(f"router: {experts} experts do not divide into {groups} groups of which {keep_groups} hold {top} choices")
        if experts > 512 or top > 32 or groups > 32:
            raise ValueError("router: at most 512 experts, 32 groups and 32 choices per token")
        self.width, self.experts, self.top, self.groups, self.keep_groups, self.out_scale = width, experts, top, groups, keep_groups, float(out_scale)
        self.weight = nn.Parameter(torch.empty((experts, width), dtype=torch.float32, device=device), requires_grad=False)
        self.correction = nn.Parameter(torch.zeros(experts, dtype=torch.float32, device=device), requires_grad=False)

    def load(self, loader, key: str, correction_key: str):
        self.weight.data.copy_(loader.load_tensor(key, "cpu").float())
        self.correction.data.copy_(loader.load_tensor(correction_key, "cpu").float())

    def forward(self, x: torch.Tensor):
        n = x.shape[0]
        idx = torch.empty((n, self.top), dtype=torch.int64, device=x.device)
        wt = torch.empty((n, self.top), dtype=torch.float32, device=x.device)
        cfg = native.GateConfig(self.experts, self.width, self.top, self.groups, self.keep_groups, _SCORING["sigmoid"], _TOPK["noaux_tc"], 2, self.out_scale,
                                self.weight.data_ptr(), self.correction.data_ptr(), TORCH_TO_GGML_HIDDEN[x.dtype])
        st = torch.cuda.current_stream(x.device).cuda_stream
        if n >= self.gemm_min_tokens or self.width % 4:
            logits = nn.functional.linear(x.float(), self.weight)
            native.check_seq(native.seq_lib().ktb200_moe_gate_select(C.byref(cfg), n, logits.data_ptr(), idx.data_ptr(), wt.data_ptr(), st))
        else:
            native.check_seq(native.seq_lib().ktb200_moe_gate_forward(C.byref(cfg), n, x.data_ptr(), idx.data_ptr(), wt.data_ptr(), None, None, st))
        return idx, wt
