"""KDeepseekV2Attention — absorbed multi-head latent attention for decode (V3 MLA is the same as V2).

Mirrors archive/ktransformers/operators/attention.py:49-75 (`get_absorbed`) and :349-478 (`forward_linux_flashinfer`,
decode branch): q projections -> RoPE -> paged latent-cache update -> q_nope . W_UK (batched matmul) -> MLA paged decode
over the 576-wide latents -> . W_UV^T -> o_proj.  The attention itself is `MLAWrapper.run` = ktb200_mla_decode (tcgen05 +
TMEM + TMA, csrc/mla.cu); the cache write is ktb200_mla_kv_write; the projections are whatever modules the rules injected
(KLinearB200 on raw GGUF blocks, or nn.Linear); the two absorb products are ktb200_mla_absorb_q / _o (HBM-bound batched
GEMVs over the bf16 halves of kv_b_proj; torch.matmul for other dtypes).  Prefill (q_len > 1 without absorb) is outside this path and raises."""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from .. import native
from ..models.modeling_deepseek_v3 import DeepseekV3Attention, apply_rotary_pos_emb
from .base_operator import BaseInjectedModule
from .flashinfer_wrapper import MLAWrapperSingleton


class KDeepseekV2Attention(BaseInjectedModule, DeepseekV3Attention):
    def __init__(self, key, gguf_loader, config, orig_module, prefill_device: str = "cuda", generate_device: str = "cuda",
                 chunck_size: int = 1000, absorb_for_prefill: bool = False, **kwargs):
        BaseInjectedModule.__init__(self, key, gguf_loader, config, orig_module, prefill_device, generate_device, **kwargs)
        self.chunck_size = chunck_size
        self.mla_wrapper = None
        self.absorb_for_prefill = absorb_for_prefill

    def get_absorbed(self) -> Tuple[torch.Tensor, torch.Tensor]:
        """kv_b_proj [heads * (128 + 128), 512] viewed per head: q_absorb = W_UK [h, 128, 512], out_absorb = W_UV [h, 128, 512]
        (attention.py:69-75); kv_b_proj is the one projection the rules keep dense."""
        if not (hasattr(self, "q_absorb") and hasattr(self, "out_absorb")):
            kv_b = self.kv_b_proj.weight.view(self.num_heads, -1, self.kv_lora_rank)
            object.__setattr__(self, "q_absorb", kv_b[:, : self.qk_nope_head_dim, :].contiguous())
            object.__setattr__(self, "out_absorb", kv_b[:, self.qk_nope_head_dim:, :].contiguous())
        return self.q_absorb, self.out_absorb

    def forward(self, hidden_states: torch.Tensor, attention_mask: Optional[torch.Tensor] = None,
                position_ids: Optional[torch.Tensor] = None, past_key_value=None, output_attentions: bool = False,
                use_cache: bool = False, cache_position: Optional[torch.Tensor] = None, **kwargs):
        bsz, q_len, _ = hidden_states.size()
        if q_len != 1 and not self.absorb_for_prefill:
            raise NotImplementedError("KDeepseekV2Attention: the B200 path covers absorbed decode (q_len == 1)")
        assert past_key_value is not None, "decode needs the paged latent cache (models/custom_cache.StaticCache)"
        q = self.q_proj(hidden_states) if self.q_lora_rank is None else self.q_b_proj(self.q_a_layernorm(self.q_a_proj(hidden_states)))
        q = q.view(bsz, q_len, self.num_heads, self.q_head_dim)
        q_nope, q_pe = torch.split(q, [self.qk_nope_head_dim, self.qk_rope_head_dim], dim=-1)
        compressed_kv = self.kv_a_proj_with_mqa(hidden_states)
        compressed_kv, k_pe = torch.split(compressed_kv, [self.kv_lora_rank, self.qk_rope_head_dim], dim=-1)
        compressed_kv = self.kv_a_layernorm(compressed_kv).view(bsz, q_len, 1, self.kv_lora_rank)
        k_pe = k_pe.view(bsz, q_len, 1, self.qk_rope_head_dim)
        cos, sin = self.rotary_emb(q_pe, position_ids)
        q_pe, k_pe = apply_rotary_pos_emb(q_pe, k_pe, cos, sin, unsqueeze_dim=2)

        cache_kwargs = {"sin": sin, "cos": cos, "cache_position": cache_position}
        kv_with_k_pe, page_table = past_key_value.update(compressed_kv, k_pe, self.layer_idx, cache_kwargs)
        ckv_pages = kv_with_k_pe[:, :, :, : self.kv_lora_rank].view(-1, past_key_value.page_size, self.kv_lora_rank)
        kpe_pages = kv_with_k_pe[:, :, :, self.kv_lora_rank:].view(-1, past_key_value.page_size, self.qk_rope_head_dim)

        q_absorb, out_absorb = self.get_absorbed()
        fused = (q.dtype == torch.bfloat16 and q_absorb.dtype == torch.bfloat16 and q.is_contiguous())
        stream = torch.cuda.current_stream(hidden_states.device).cuda_stream
        if fused:   # q_nope . W_UK straight from the q_b output (no slice copy): ktb200_mla_absorb_q
            q_abs = torch.empty((bsz * q_len, self.num_heads, self.kv_lora_rank), dtype=q.dtype, device=q.device)
            native.check(native.lib().ktb200_mla_absorb_q(q.data_ptr(), self.q_head_dim, self.num_heads * self.q_head_dim, q_absorb.data_ptr(), self.num_heads,
                                                          self.qk_nope_head_dim, self.kv_lora_rank, q_abs.data_ptr(), bsz * q_len, stream))
            q_nope = q_abs
        else:
            q_nope = torch.matmul(q_nope.transpose(1, 2), q_absorb).transpose(1, 2).contiguous().reshape(bsz * q_len, self.num_heads, self.kv_lora_rank)
        q_pe = q_pe.reshape(bsz * q_len, self.num_heads, self.qk_rope_head_dim)

        if self.mla_wrapper is None:
            self.mla_wrapper = MLAWrapperSingleton.get_instance(str(hidden_states.device), bsz, past_key_value.max_pages * bsz, use_cuda_graph=True)
        w = self.mla_wrapper
        if w.need_plan:
            # decode: one query per sequence, kv length = position + 1, identity page table of the static cache
            kv_len = (position_ids.reshape(bsz, -1)[:, -1] + 1).to(torch.int32)
            pages = past_key_value.max_pages
            indptr = torch.arange(0, bsz + 1, dtype=torch.int32, device=hidden_states.device) * pages
            w.plan(None, indptr, page_table.reshape(-1), kv_len, None, self.num_heads, self.kv_lora_rank, self.qk_rope_head_dim,
                   past_key_value.page_size, self.softmax_scale, q_nope.dtype, ckv_pages.dtype)
            w.max_pages_per_seq = pages
        else:   # the plan is static (identity page table); only the lengths move from step to step (a captured device copy)
            w.kv_len_arr_buf[:bsz].copy_((position_ids.reshape(bsz, -1)[:, -1] + 1).to(torch.int32))
        attn = w.run(q_nope, q_pe.contiguous(), ckv_pages, kpe_pages).view(bsz, q_len, self.num_heads, self.kv_lora_rank)
        if fused:
            o = torch.empty((bsz, q_len, self.num_heads, self.v_head_dim), dtype=attn.dtype, device=attn.device)
            native.check(native.lib().ktb200_mla_absorb_o(attn.data_ptr(), out_absorb.data_ptr(), self.num_heads, self.v_head_dim, self.kv_lora_rank, o.data_ptr(),
                                                          bsz * q_len, stream))
            attn = o
        else:
            attn = torch.matmul(attn.transpose(1, 2), out_absorb.mT).transpose(1, 2).contiguous()     # [b, 1, h, 128]
        attn = self.o_proj(attn.reshape(bsz, q_len, self.num_heads * self.v_head_dim))
        return attn, None, past_key_value


class KLatentWindowAttention(torch.nn.Module):
    """Latent attention with a low-rank query, a sliding window, a soft-max sink and a sigmoid output gate, run absorbed over
    the paged latent cache — the same formulation KDeepseekV2Attention uses for decode, here for prompt portions as well.
    Each of the four is optional (`q_rank = 0`: the query is one full-rank projection `W_q`; `window = None`; `sink` /
    `gate = False`), and the rotation pairs columns in either layout (`rot.layout`).

        P        = [W_dq ; W_dkv ; W_g] hs                      one GEMM over the three matrices that read the mixer input
        cq, c, k_r -> cache                                      ktb200_latent_prep (two RMS norms, rotation, paged write)
        q        = W_uq cq                                       GEMM
        qa_h     = W_uk,h^T q_h[:dim]                            batched GEMM (absorb)
        lat_h    = sum_j softmax_sink(qa_h . c_j + rot(q_h[dim:]) . k_r,j) c_j     ktb200_latent_window_attn, or on tcgen05:
                                                                 ktb200_rope_rows + ktb200_latent_window_attn_tc
        o_h      = W_uv,h lat_h                                  batched GEMM (absorb)
        out      = W_o (o * sigmoid(g))                          ktb200_sigmoid_gate_mul + GEMM

    Only c and k_r are cached (`kv_rank + rot_dim` values per token and layer).  Sizes, window, sink, scale and the rotation
    constants are constructor parameters (models/configuration_lekapel.LatentAttentionSpec).

    Two attention kernels: with bf16, kv_rank 512, rot_dim 64 and pages that are a multiple of 32 tokens (DeepSeek's latent
    sizes) the tcgen05 / TMEM / TMA kernel of MLA decode runs, one CTA per (token, 64 heads, key split), with the
    probabilities split into two bf16 terms so that they keep fp32-like precision; any other size, and fp32, runs the
    CUDA-core kernel of csrc/window_attn.cu."""

    use_tensor_path = True

    def __init__(self, width: int, spec, eps: float, layer_idx: int, dtype=torch.bfloat16, device="cuda"):
        super().__init__()
        P = lambda *shape, dt=dtype: torch.nn.Parameter(torch.empty(shape, dtype=dt, device=device), requires_grad=False)
        s = self.spec = spec
        self.width, self.eps, self.layer_idx = width, eps, layer_idx
        # rows of the one matrix that reads the mixer input: [query latent, or the whole query when there is none | kv latent | rotated key part | gate]
        self.n_q = s.q_rank if s.q_rank else s.heads * (s.dim + s.rot_dim)
        self.n_in = self.n_q + s.kv_rank + s.rot_dim + (s.heads * s.vdim if s.gate else 0)
        self.w_in = P(self.n_in, width)
        self.q_norm, self.kv_norm = (P(s.q_rank) if s.q_rank else None), P(s.kv_rank)
        self.uq = P(s.heads * (s.dim + s.rot_dim), s.q_rank) if s.q_rank else None
        self.w_uk = P(s.heads, s.dim, s.kv_rank)
        self.w_uv_t = P(s.heads, s.kv_rank, s.vdim)
        self.sink = P(s.heads, dt=torch.float32) if s.sink else None
        self.o = P(width, s.heads * s.vdim)
        self.register_buffer("inv_freq", s.rot.inv_freq(device), persistent=False)

    def load(self, loader, prefix: str):
        s, t = self.spec, lambda n: loader.load_tensor(prefix + n, "cpu")
        self.w_in.data.copy_(torch.cat([t("dq") if s.q_rank else t("q"), t("dkv")] + ([t("g")] if s.gate else []), 0))
        if s.q_rank:
            self.q_norm.data.copy_(t("dq.norm"))
            self.uq.data.copy_(t("uq"))
        self.kv_norm.data.copy_(t("dkv.norm"))
        self.w_uk.data.copy_(t("uk").view(s.heads, s.dim, s.kv_rank))
        self.w_uv_t.data.copy_(t("uv").view(s.heads, s.vdim, s.kv_rank).transpose(1, 2))
        if s.sink:
            self.sink.data.copy_(t("sink").float())
        self.o.data.copy_(t("o"))

    def pick_splits(self, n_tokens: int, max_kv: int) -> int:
        """Cut the key range when a small batch would leave most SMs idle on a long window."""
        s = self.spec
        keys = min(s.window, max_kv) if s.window else max_kv
        ctas = n_tokens * ((s.heads + 7) // 8)
        if ctas >= 148 or keys <= 256:
            return 1
        return max(1, min(32, keys // 128, 296 // ctas))

    def forward(self, hs: torch.Tensor, batch, cache, cache_idx: Optional[int] = None) -> torch.Tensor:
        s, T, dev, dt = self.spec, hs.shape[0], hs.device, hs.dtype
        lib, code, st = native.seq_lib(), native.GGML_BF16 if dt == torch.bfloat16 else native.GGML_F32, torch.cuda.current_stream(hs.device).cuda_stream
        kv = cache.key_cache[self.layer_idx if cache_idx is None else cache_idx]
        lay, sink = s.rot.layout_code, (self.sink.data_ptr() if self.sink is not None else None)
        proj = torch.nn.functional.linear(hs, self.w_in)
        cq = torch.empty((T, s.q_rank), dtype=dt, device=dev) if s.q_rank else None
        # the prep kernel reads [query latent (q_rank) | kv latent | rotated key part] from its row pointer
        lat_in = proj if s.q_rank else proj[:, self.n_q:]
        native.check_seq(lib.ktb200_latent_prep(lat_in.data_ptr(), self.n_in, s.q_rank, s.kv_rank, s.rot_dim, s.rot.dims, lay, self.inv_freq.data_ptr(),
                                                self.q_norm.data_ptr() if s.q_rank else None, self.kv_norm.data_ptr(), float(self.eps), batch.pos.data_ptr(),
                                                batch.slot.data_ptr(), cache.page_table.data_ptr(), cache.max_pages_per_seq, cache.page_size, kv.data_ptr(),
                                                cq.data_ptr() if s.q_rank else None, T, code, st))
        q = torch.nn.functional.linear(cq, self.uq) if s.q_rank else proj[:, :self.n_q].contiguous()
        if s.dim:       # [H, T, R] out of the batched product, token-major for the attention kernels
            q_abs = torch.bmm(q.view(T, s.heads, s.dim + s.rot_dim)[:, :, : s.dim].transpose(0, 1), self.w_uk).transpose(0, 1).contiguous()
        else:
            q_abs = torch.zeros((T, s.heads, s.kv_rank), dtype=dt, device=dev)
        lat = torch.empty((T, s.heads, s.kv_rank), dtype=dt, device=dev)
        if self.use_tensor_path and dt == torch.bfloat16 and s.kv_rank == 512 and s.rot_dim == 64 and cache.page_size % 32 == 0:
            q_rot = torch.empty((T, s.heads, s.rot_dim), dtype=dt, device=dev)
            native.check_seq(lib.ktb200_rope_rows(q.data_ptr(), s.heads, s.dim, s.rot_dim, s.rot.dims, lay, self.inv_freq.data_ptr(), batch.pos.data_ptr(), q_rot.data_ptr(), T, code, st))
            wsb = lib.ktb200_latent_window_attn_tc_workspace(T, s.heads, s.window or 0, batch.max_kv)
            ws = torch.empty(wsb // 4, dtype=torch.float32, device=dev)
            native.check_seq(lib.ktb200_latent_window_attn_tc(q_abs.data_ptr(), q_rot.data_ptr(), s.heads, float(s.scale), sink, s.window or 0, batch.pos.data_ptr(),
                                                              batch.slot.data_ptr(), cache.page_table.data_ptr(), cache.max_pages_per_seq, cache.page_size, kv.data_ptr(),
                                                              kv.shape[0] * kv.shape[1], lat.data_ptr(), T, batch.max_kv, ws.data_ptr(), wsb, st))
        else:
            splits = self.pick_splits(T, batch.max_kv)
            ws = torch.empty(lib.ktb200_latent_window_attn_workspace(T, s.heads, s.kv_rank, splits) // 4, dtype=torch.float32, device=dev) if splits > 1 else None
            native.check_seq(lib.ktb200_latent_window_attn(q.data_ptr(), q_abs.data_ptr(), s.heads, s.dim, s.rot_dim, s.kv_rank, s.rot.dims, lay, self.inv_freq.data_ptr(),
                                                           float(s.scale), sink, s.window or 0, batch.pos.data_ptr(), batch.slot.data_ptr(),
                                                           cache.page_table.data_ptr(), cache.max_pages_per_seq, cache.page_size, kv.data_ptr(), lat.data_ptr(), T, splits,
                                                           ws.data_ptr() if ws is not None else None, code, st))
        o = torch.bmm(lat.transpose(0, 1), self.w_uv_t)
        if s.gate:
            og = torch.empty((T, s.heads * s.vdim), dtype=dt, device=dev)
            native.check_seq(lib.ktb200_sigmoid_gate_mul(o.data_ptr(), proj[:, self.n_q + s.kv_rank + s.rot_dim:].data_ptr(), self.n_in, og.data_ptr(), T, s.heads, s.vdim, code, st))
        else:
            og = o.transpose(0, 1).reshape(T, s.heads * s.vdim)
        return torch.nn.functional.linear(og, self.o)


def distance_bias_table(rel: torch.Tensor, bias_max: float) -> torch.Tensor:
    """A learned bias per (distance bucket, head), expanded to one entry per DISTANCE and laid out per head, [heads, n]: entries
    0 .. n - 1 with n - 1 the first distance whose bucket is the last one, so a kernel indexes `[h][min(i - j, n - 1)]`.  With B rows in `rel` and half = B // 2:
    bucket(n) = n below half, else min(B - 1, half + floor(ln(n / half) / ln(bias_max / half) * (B - half))) — exact below half,
    logarithmic up to `bias_max`, constant beyond."""
    B = rel.shape[0]
    half = B // 2
    if half < 1 or not bias_max > half:
        raise ValueError(f"a distance bias table of {B} rows needs at least 2 rows and a reach beyond {half} (got {bias_max})")
    buckets, n = [], 0
    while True:
        b = n if n < half else min(B - 1, half + int(math.floor(math.log(n / half) / math.log(bias_max / half) * (B - half))))
        buckets.append(b)
        if b == B - 1 and n >= half:
            break
        n += 1
    return rel.float().index_select(0, torch.tensor(buckets, dtype=torch.int64, device=rel.device)).t().contiguous()


class KSigmoidBiasAttention(torch.nn.Module):
    """Causal attention without a soft-max over grouped key/value heads: the weight of key j for query i of head h is

        sigmoid(scale * q_i . k_j + rel[bucket(i - j)][h] + pb[h])          (not normalised over the keys)

    with per-head RMS norms of queries and keys (one weight per norm, shared by the heads), no rotation, a query temperature
    `1 + coef * ln(floor((pos + 1) / every) + 1)`, and one sigmoid output gate per head read from the mixer's input.

        P     = [W_q ; W_k ; W_v ; W_g] h + b                  one GEMM over the matrices that read the mixer input
        q, k  -> norms, temperature; [k | v] -> paged cache    ktb200_qk_norm_cache_write
        o_h   = sum_j weight_ij v_j * sigmoid(g_h)             ktb200_sigmoid_bias_attn (fp32 scores and weights)
        out   = W_o o + b_o                                    GEMM

    Two attention kernels (csrc/seq_mixers.cu): in bf16 with head sizes that are multiples of 16 up to 128, tiles of 64 (token,
    head) rows against 64 keys on the tensor cores (the weights leave the fp32 sigmoid as bf16 operands of the second
    product); any other size, and fp32, on CUDA cores with fp32 products throughout.

    Sizes, scale, the bias table's reach and the temperature constants are constructor parameters
    (models/configuration_mabidra.SigmoidAttentionSpec).  `cache_idx` picks the cache layer, so one set of weights can run
    several times per step with separate caches."""

    def __init__(self, width: int, spec, eps: float, dtype=torch.bfloat16, device="cuda"):
        super().__init__()
        P = lambda *shape, dt=dtype: torch.nn.Parameter(torch.zeros(shape, dtype=dt, device=device), requires_grad=False)
        s = self.spec = spec
        if s.heads % s.kv_heads:
            raise ValueError("query heads must divide into the key/value heads")
        self.width, self.eps = width, eps
        self.n_q, self.n_kv = s.heads * s.dim, s.kv_heads * (s.dim + s.vdim)
        self.n_in = (self.n_q + self.n_kv + s.heads + 7) // 8 * 8       # rows padded so that every row of P starts 16-byte aligned
        self.w_in, self.b_in = P(self.n_in, width), P(self.n_in)
        self.q_norm, self.k_norm = P(s.dim), P(s.dim)
        self.head_bias = P(s.heads, dt=torch.float32)
        self.o, self.o_b = P(width, s.heads * s.vdim), P(width)
        self.register_buffer("bias_table", torch.zeros((s.heads, 1), dtype=torch.float32, device=device), persistent=False)

    def load(self, loader, prefix: str):
        s, t = self.spec, lambda n: loader.load_tensor(prefix + n, "cpu")
        rows = self.n_q + self.n_kv + s.heads
        self.w_in.data[:rows].copy_(torch.cat([t("q"), t("k"), t("v"), t("g")], 0))
        self.b_in.data[:self.n_q + self.n_kv].copy_(torch.cat([t("q.b"), t("k.b"), t("v.b")], 0))
        self.q_norm.data.copy_(t("q.norm"))
        self.k_norm.data.copy_(t("k.norm"))
        self.head_bias.data.copy_(t("pb").float())
        self.o.data.copy_(t("o"))
        self.o_b.data.copy_(t("o.b"))
        self.bias_table = distance_bias_table(t("rel"), s.bias_max).to(self.w_in.device)

    use_tensor_cores = True

    def pick_splits(self, n_tokens: int, max_kv: int, n_seqs: int = 0, tensor_cores: bool = False) -> int:
        """Cut the key range when a small batch would leave most SMs idle on a long context."""
        s = self.spec
        if tensor_cores:
            ctas = native.seq_lib().ktb200_sigmoid_bias_attn_tiles(s.heads, s.kv_heads, n_tokens, n_seqs) * s.kv_heads
        else:
            ctas = n_tokens * s.kv_heads * ((s.heads // s.kv_heads + 7) // 8)
        if ctas >= 148 or max_kv <= 256:
            return 1
        if tensor_cores:      # four CTAs per SM; parts of 64 keys or more
            return max(1, min(128, max_kv // 64, 1184 // ctas))
        return max(1, min(64, max_kv // 128, 592 // ctas))

    def forward(self, h: torch.Tensor, batch, cache, cache_idx: int) -> torch.Tensor:
        s, T, dev, dt = self.spec, h.shape[0], h.device, h.dtype
        lib, code, st = native.seq_lib(), native.GGML_BF16 if dt == torch.bfloat16 else native.GGML_F32, torch.cuda.current_stream(h.device).cuda_stream
        kv = cache.key_cache[cache_idx]
        proj = torch.nn.functional.linear(h, self.w_in, self.b_in)
        q = torch.empty((T, s.heads, s.dim), dtype=dt, device=dev)
        native.check_seq(lib.ktb200_qk_norm_cache_write(proj.data_ptr(), self.n_in, s.heads, s.kv_heads, s.dim, s.vdim, self.q_norm.data_ptr(), self.k_norm.data_ptr(),
                                                        float(self.eps), float(s.temp_coef), int(s.temp_every), batch.pos.data_ptr(), batch.slot.data_ptr(),
                                                        cache.page_table.data_ptr(), cache.max_pages_per_seq, cache.page_size, kv.data_ptr(), q.data_ptr(), T, code, st))
        gate = proj[:, self.n_q + self.n_kv:]
        o = torch.empty((T, s.heads * s.vdim), dtype=dt, device=dev)
        tc = bool(self.use_tensor_cores and batch.seqs is not None and lib.ktb200_sigmoid_bias_attn_uses_tensor_cores(s.heads, s.kv_heads, s.dim, s.vdim, code))
        splits = self.pick_splits(T, batch.max_kv, batch.n_seqs, tc)
        ws = torch.empty(lib.ktb200_sigmoid_bias_attn_workspace(T, s.heads, s.vdim, splits) // 4, dtype=torch.float32, device=dev) if splits > 1 else None
        native.check_seq(lib.ktb200_sigmoid_bias_attn(q.data_ptr(), s.heads, s.kv_heads, s.dim, s.vdim, float(s.scale), self.bias_table.data_ptr(), self.bias_table.shape[1],
                                                      self.head_bias.data_ptr(), batch.pos.data_ptr(), batch.slot.data_ptr(),
                                                      batch.seqs.data_ptr() if tc else None, batch.seqs.stride(0) if tc else 0, batch.n_seqs if tc else 0,
                                                      cache.page_table.data_ptr(), cache.max_pages_per_seq, cache.page_size, kv.data_ptr(), gate.data_ptr(), self.n_in,
                                                      o.data_ptr(), T, splits, ws.data_ptr() if ws is not None else None, code, int(tc), st))
        return torch.nn.functional.linear(o, self.o, self.o_b)


def softmax_attention_splits(heads: int, kv_heads: int, keys: int, n_tokens: int, n_seqs: int = 0, tensor_cores: bool = False) -> int:
    """Into how many parts `ktb200_window_softmax_attn` cuts a key range of up to `keys` keys: more than one when a small batch
    would leave most SMs idle on a long range."""
    if tensor_cores:
        ctas = native.seq_lib().ktb200_window_softmax_attn_tiles(heads, kv_heads, n_tokens, n_seqs) * kv_heads
    else:
        ctas = n_tokens * kv_heads * ((heads // kv_heads + 7) // 8)
    if ctas >= 148 or keys <= 256:
        return 1
    if tensor_cores:      # four CTAs per SM; parts of 64 keys or more
        return max(1, min(128, keys // 64, 1184 // ctas))
    return max(1, min(64, keys // 128, 592 // ctas))


def paged_softmax_attention(q: torch.Tensor, kv: torch.Tensor, batch, cache, heads: int, kv_heads: int, dim: int, vdim: int, scale: float,
                            head_scale: Optional[torch.Tensor] = None, softcap: Optional[float] = None, window: Optional[int] = None, chunk: Optional[int] = None,
                            tensor_cores: bool = True) -> torch.Tensor:
    """o [T, heads * vdim] = soft-max attention of the prepared queries q [T, heads, dim] over the [k | v] rows of cache layer `kv`
    (`ktb200_window_softmax_attn`, csrc/softmax_attn.cu): the key at position j is seen from position i when j <= i,
    i - j < window (if a window is given) and floor(j / chunk) == floor(i / chunk) (if a chunk length is given, chunks counted from the
    sequence's position 0); scores scale * head_scale[h] * q.k, squashed to c tanh(s / c) with c = softcap; fp32 scores and weights."""
    T, dev, dt = q.shape[0], q.device, q.dtype
    lib, code, st = native.seq_lib(), native.GGML_BF16 if dt == torch.bfloat16 else native.GGML_F32, torch.cuda.current_stream(dev).cuda_stream
    o = torch.empty((T, heads * vdim), dtype=dt, device=dev)
    tc = bool(tensor_cores and batch.seqs is not None and lib.ktb200_window_softmax_attn_uses_tensor_cores(heads, kv_heads, dim, vdim, code))
    keys = min(x for x in (window, chunk, batch.max_kv) if x)
    splits = softmax_attention_splits(heads, kv_heads, keys, T, batch.n_seqs, tc)
    ws = torch.empty(lib.ktb200_window_softmax_attn_workspace(T, heads, vdim, splits) // 4, dtype=torch.float32, device=dev) if splits > 1 else None
    native.check_seq(lib.ktb200_window_softmax_attn(q.data_ptr(), heads, kv_heads, dim, vdim, float(scale), head_scale.data_ptr() if head_scale is not None else None,
                                                    float(softcap or 0.0), int(window or 0), int(chunk or 0), batch.pos.data_ptr(), batch.slot.data_ptr(),
                                                    batch.seqs.data_ptr() if tc else None, batch.seqs.stride(0) if tc else 0, batch.n_seqs if tc else 0,
                                                    cache.page_table.data_ptr(), cache.max_pages_per_seq, cache.page_size, kv.data_ptr(), o.data_ptr(), T, splits,
                                                    ws.data_ptr() if ws is not None else None, code, int(tc), st))
    return o


class KCappedWindowAttention(torch.nn.Module):
    """Causal soft-max attention over grouped key/value heads with biased projections, a partial rotation, unit-rms queries and
    keys, capped scores, a sliding window, and values blended with another layer's values of the same token:

        P       = [W_q ; W_k ; W_v] h + b                       one GEMM over the matrices that read the mixer input
        q, k    = x / sqrt(mean(x^2) + eps) per head of rot(P[q]), rot(P[k])      (rotation over the first rot.dims columns,
                                                                                   frequencies divided by rot.factor)
        v       = (1 - t) P[v] + t v_other                      when `v_other` is handed in (t: one learned number)
        [k | v] -> paged cache                                  ktb200_rope_norm_cache_write, all of the above in one launch
        s_ij    = c tanh(scale q_i . k_j / c), c = softcap      for 0 <= i - j < window
        o_i     = sum_j softmax_j(s_ij) v_j                     ktb200_window_softmax_attn (fp32 scores and weights)
        out     = W_o o                                         GEMM

    Two attention kernels (csrc/softmax_attn.cu): in bf16 with head sizes that are multiples of 16 up to 128, tiles of 64 (token,
    head) rows against 32 keys on the tensor cores (the weights leave the fp32 soft-max as bf16 operands of the second product);
    any other size, and fp32, on CUDA cores with fp32 products throughout.

    The blended v is what is cached.  `forward` also returns the layer's own values before the blend (a view of P), which the
    model hands to later layers as their `v_other`.  Sizes, scale, cap, window, the rotation's constants and layout and the
    unit-rms switch are constructor parameters (models/configuration_zivulix.CappedWindowAttentionSpec); `cache_idx` picks
    the cache layer.  (The reference's attention operators: archive/ktransformers/operators/attention.py.)"""

    def __init__(self, width: int, spec, eps: float, dtype=torch.bfloat16, device="cuda"):
        super().__init__()
        P = lambda *shape, dt=dtype: torch.nn.Parameter(torch.zeros(shape, dtype=dt, device=device), requires_grad=False)
        s = self.spec = spec
        if s.heads % s.kv_heads:
            raise ValueError("query heads must divide into the key/value heads")
        self.width, self.eps = width, eps
        self.n_q, self.n_k, self.n_v = s.heads * s.dim, s.kv_heads * s.dim, s.kv_heads * s.vdim
        self.n_in = (self.n_q + self.n_k + self.n_v + 7) // 8 * 8       # rows padded so that every row of P starts 16-byte aligned
        self.w_in, self.b_in = P(self.n_in, width), P(self.n_in)
        self.vmix = P(1, dt=torch.float32)
        self.o = P(width, s.heads * s.vdim)
        self.register_buffer("inv_freq", s.rot.inv_freq(device) if s.rot is not None and s.rot.dims else torch.zeros(1, dtype=torch.float64, device=device), persistent=False)

    def load(self, loader, prefix: str):
        t = lambda n: loader.load_tensor(prefix + n, "cpu")
        rows = self.n_q + self.n_k + self.n_v
        self.w_in.data[:rows].copy_(torch.cat([t("q"), t("k"), t("v")], 0))
        self.b_in.data[:rows].copy_(torch.cat([t("q.b"), t("k.b"), t("v.b")], 0))
        if self.spec.v_mix:
            self.vmix.data.copy_(t("vmix").float().reshape(1))
        self.o.data.copy_(t("o"))

    use_tensor_cores = True

    def pick_splits(self, n_tokens: int, max_kv: int, n_seqs: int = 0, tensor_cores: bool = False) -> int:
        s = self.spec
        return softmax_attention_splits(s.heads, s.kv_heads, min(s.window, max_kv) if s.window else max_kv, n_tokens, n_seqs, tensor_cores)

    def forward(self, h: torch.Tensor, batch, cache, cache_idx: int, v_other: Optional[torch.Tensor] = None):
        s, T, dev, dt = self.spec, h.shape[0], h.device, h.dtype
        lib, code, st = native.seq_lib(), native.GGML_BF16 if dt == torch.bfloat16 else native.GGML_F32, torch.cuda.current_stream(h.device).cuda_stream
        kv = cache.key_cache[cache_idx]
        proj = torch.nn.functional.linear(h, self.w_in, self.b_in)
        v_own = proj[:, self.n_q + self.n_k: self.n_q + self.n_k + self.n_v]
        if v_other is not None and v_other.shape != v_own.shape:
            raise ValueError("blended values must have this layer's key/value heads and value size")
        q = torch.empty((T, s.heads, s.dim), dtype=dt, device=dev)
        rot_dims = s.rot.dims if s.rot is not None else 0
        native.check_seq(lib.ktb200_rope_norm_cache_write(proj.data_ptr(), self.n_in, 0, self.n_q, self.n_q + self.n_k, s.heads, s.kv_heads, s.dim, s.vdim, rot_dims,
                                                          s.rot.layout_code if rot_dims else 0, self.inv_freq.data_ptr(), int(s.unit_rms), None, None, 0, float(self.eps),
                                                          v_other.data_ptr() if v_other is not None else None, v_other.stride(0) if v_other is not None else 0,
                                                          self.vmix.data_ptr(), batch.pos.data_ptr(), batch.slot.data_ptr(), cache.page_table.data_ptr(),
                                                          cache.max_pages_per_seq, cache.page_size, kv.data_ptr(), q.data_ptr(), T, code, st))
        o = paged_softmax_attention(q, kv, batch, cache, s.heads, s.kv_heads, s.dim, s.vdim, s.scale, softcap=s.softcap, window=s.window,
                                    tensor_cores=self.use_tensor_cores)
        return torch.nn.functional.linear(o, self.o), v_own


class KChunkedSoftmaxAttention(torch.nn.Module):
    """Causal soft-max attention over grouped key/value heads inside chunks of the sequence, with biased projections, queries and
    keys normed over their whole projection, unit-rms values, a learned temperature per query head and capped scores; no position
    enters the scores:

        P       = [W_q ; W_k ; W_v] h + b                       one GEMM over the matrices that read the mixer input
        q, k    = P[q] / sqrt(mean(P[q]^2) + eps) * w_q  (all heads of a token at once; k likewise with w_k)
        v_g     = P[v]_g / sqrt(mean(P[v]_g^2) + eps)            head by head, no weight
        [k | v] -> paged cache                                  ktb200_rope_norm_cache_write, all of the above in one launch
        s_ij    = c tanh(scale t_h q_i . k_j / c), c = softcap   for j <= i with floor(j / C) == floor(i / C), C = chunk
        o_i     = sum_j softmax_j(s_ij) v_j                     ktb200_window_softmax_attn (fp32 scores and weights)
        out     = W_o o + b_o                                   GEMM

    The chunk mask shares the attention kernels of KCappedWindowAttention (tensor-core tiles in bf16 with head sizes that are
    multiples of 16 up to 128, CUDA cores otherwise and in fp32): a chunk is a window whose first key depends on the query's
    position, p - p mod C.  Sizes, scale, cap and the chunk length are constructor parameters
    (models/configuration_bilurax.ChunkedAttentionSpec); `cache_idx` picks the cache layer, so one set of weights can run several
    times per step with separate caches.  (The reference's attention operators: archive/ktransformers/operators/attention.py.)"""

    use_tensor_cores = True

    def __init__(self, width: int, spec, eps: float, dtype=torch.bfloat16, device="cuda"):
        super().__init__()
        P = lambda *shape, dt=dtype: torch.nn.Parameter(torch.zeros(shape, dtype=dt, device=device), requires_grad=False)
        s = self.spec = spec
        if s.heads % s.kv_heads:
            raise ValueError("query heads must divide into the key/value heads")
        self.width, self.eps = width, eps
        self.n_q, self.n_k, self.n_v = s.heads * s.dim, s.kv_heads * s.dim, s.kv_heads * s.vdim
        self.n_in = (self.n_q + self.n_k + self.n_v + 7) // 8 * 8       # rows padded so that every row of P starts 16-byte aligned
        self.w_in, self.b_in = P(self.n_in, width), P(self.n_in)
        self.q_norm, self.k_norm = P(self.n_q), P(self.n_k)
        self.temp = P(s.heads, dt=torch.float32)
        self.o, self.o_b = P(width, s.heads * s.vdim), P(width)

    def load(self, loader, prefix: str):
        t = lambda n: loader.load_tensor(prefix + n, "cpu")
        rows = self.n_q + self.n_k + self.n_v
        self.w_in.data[:rows].copy_(torch.cat([t("q"), t("k"), t("v")], 0))
        self.b_in.data[:rows].copy_(torch.cat([t("q.b"), t("k.b"), t("v.b")], 0))
        self.q_norm.data.copy_(t("q.norm"))
        self.k_norm.data.copy_(t("k.norm"))
        self.temp.data.copy_(t("temp").float())
        self.o.data.copy_(t("o"))
        self.o_b.data.copy_(t("o.b"))

    def forward(self, h: torch.Tensor, batch, cache, cache_idx: int) -> torch.Tensor:
        s, T, dev, dt = self.spec, h.shape[0], h.device, h.dtype
        lib, code, st = native.seq_lib(), native.GGML_BF16 if dt == torch.bfloat16 else native.GGML_F32, torch.cuda.current_stream(h.device).cuda_stream
        kv = cache.key_cache[cache_idx]
        proj = torch.nn.functional.linear(h, self.w_in, self.b_in)
        q = torch.empty((T, s.heads, s.dim), dtype=dt, device=dev)
        native.check_seq(lib.ktb200_rope_norm_cache_write(proj.data_ptr(), self.n_in, 0, self.n_q, self.n_q + self.n_k, s.heads, s.kv_heads, s.dim, s.vdim, 0, 0, None,
                                                          2, self.q_norm.data_ptr(), self.k_norm.data_ptr(), 1, float(self.eps), None, 0, None, batch.pos.data_ptr(),
                                                          batch.slot.data_ptr(), cache.page_table.data_ptr(), cache.max_pages_per_seq, cache.page_size, kv.data_ptr(),
                                                          q.data_ptr(), T, code, st))
        o = paged_softmax_attention(q, kv, batch, cache, s.heads, s.kv_heads, s.dim, s.vdim, s.scale, head_scale=self.temp, softcap=s.softcap, chunk=s.chunk,
                                    tensor_cores=self.use_tensor_cores)
        return torch.nn.functional.linear(o, self.o, self.o_b)
