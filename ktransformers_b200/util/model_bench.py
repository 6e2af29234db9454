"""Throughput and per-kernel rooflines of a step-function model at layer sizes of real models, with random weights, beside
the closest existing model's kernels at equal size (`bench.py --model lekapel`, `bench.py --model mabidra`,
`bench.py --model zivulix`, `bench.py --model bilurax`).

Two parts:
  * end to end through the Engine (scheduler, paged cache, step function): prompt tokens/s for a long prompt cut into portions,
    decode tokens/s for 1 and 8 concurrent sequences, CUDA events around the steps;
  * kernel by kernel at DeepSeek-V3 attention / MoE sizes: each token-major kernel against its counterpart of the DeepSeek path
    (fused norm, latent prep, paged latent attention for decode, expert GEMVs), algorithmic bytes / event time / measured HBM
    peak.  L2 is flushed between timed launches (a 256 MB write)."""
from __future__ import annotations

import ctypes as C
import json
import os
import statistics
import sys

import torch

from .. import native

SIZES = {
    # name: (width, layers, mixer, dense ff, experts, top, expert ff, vocab)
    "2k-wide": dict(width=2048, n_layers=6, heads=16, dim=128, rot_dim=64, vdim=128, kv_rank=512, q_rank=768, window=1024, dense_ff=8192, experts=32, top=4, ff=1024, vocab=32768),
    "v3-layer": dict(width=7168, n_layers=2, heads=128, dim=128, rot_dim=64, vdim=128, kv_rank=512, q_rank=1536, window=4096, dense_ff=18432, experts=32, top=8, ff=2048, vocab=32768),
}


def make_config(s):
    mixer = {"heads": s["heads"], "dim": s["dim"], "rot_dim": s["rot_dim"], "vdim": s["vdim"], "kv_rank": s["kv_rank"], "q_rank": s["q_rank"],
             "rot": {"base": 10000.0, "dims": s["rot_dim"]}, "scale": (s["dim"] + s["rot_dim"]) ** -0.5, "mask": {"size": s["window"]}}
    layers = [{"type": "latent_attention", "mixer": mixer, "mlp": {"kind": "dense", "ff": s["dense_ff"]}}]
    layers += [{"type": "latent_attention", "mixer": mixer, "mlp": {"kind": "moe", "expert": {"ff": s["ff"]}, "router": {"experts": s["experts"], "top": s["top"]}}}
               for _ in range(s["n_layers"] - 1)]
    return {"architecture": "Lekapel", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-5, "groups": 4}, "residual_mult": 0.6, "logit_scale": 1.0, "layers": layers}


MABIDRA_SIZES = {
    # the same widths, feed-forward sizes and layer-run counts as SIZES; attention and linear-attention layers alternate, and the
    # span `loop` runs twice (6 layer runs for 5 layers / 3 for 2)
    "2k-wide": dict(width=2048, heads=16, kv_heads=4, dim=128, vdim=128, gla_heads=16, gla_dim=128, gla_vdim=128, rank=64, dense_ff=8192, experts=32, top=4, ff=1024, vocab=32768,
                    order="AGAGA", loop=(1, 2, 2), ctx=2048),
    "v3-layer": dict(width=7168, heads=64, kv_heads=8, dim=128, vdim=128, gla_heads=56, gla_dim=128, gla_vdim=128, rank=128, dense_ff=18432, experts=32, top=8, ff=2048, vocab=32768,
                     order="AG", loop=(1, 2, 2), ctx=4096),
}


def make_mabidra_config(s):
    attn = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["vdim"], "scale": s["dim"] ** -0.5, "bias_max": 1024, "q_temp": {"coef": 0.1, "every": 512}}
    gla = {"heads": s["gla_heads"], "dim": s["gla_dim"], "vdim": s["gla_vdim"], "tau": 16.0}
    moe = {"kind": "moe", "expert": {"ff": s["ff"]}, "router": {"experts": s["experts"], "top": s["top"]}}
    layers = [{"type": "attention" if c == "A" else "gla", "mixer": attn if c == "A" else gla, "mlp": {"kind": "dense", "ff": s["dense_ff"]} if i == 0 else moe}
              for i, c in enumerate(s["order"])]
    return {"architecture": "Mabidra", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-5, "groups": 4}, "embedding": {"scale": 1.0}, "layers": layers,
            "loop": {"start": s["loop"][0], "stop": s["loop"][1], "times": s["loop"][2]}}


ZIVULIX_SIZES = {
    # the same widths and feed-forward sizes as SIZES, every feed-forward dense; A: soft-max window attention over grouped heads, D: gated
    # delta rule, L: latent attention at DeepSeek's latent sizes.  The closest existing model at equal size is Mabidra with sigmoid
    # attention where this has A or L and gated linear attention where this has D, the same dense feed-forward in every layer, no loop.
    "2k-wide": dict(width=2048, heads=16, kv_heads=4, dim=128, vdim=128, window=1024, d_heads=16, d_kv_heads=8, d_dim=128, d_vdim=128, conv=4, l_heads=16, dense_ff=8192,
                    vocab=32768, order="ADLAD", ctx=2048, rank=64),
    "v3-layer": dict(width=7168, heads=64, kv_heads=8, dim=128, vdim=128, window=4096, d_heads=56, d_kv_heads=28, d_dim=128, d_vdim=128, conv=4, l_heads=128, dense_ff=18432,
                     vocab=32768, order="ADL", ctx=4096, rank=128),
}


def make_zivulix_config(s):
    attn = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["vdim"], "scale": s["dim"] ** -0.5, "softcap": 30.0, "mask": {"size": s["window"]},
            "rot": {"base": 10000.0, "dims": s["dim"] // 2, "scaling": {"factor": 4.0}}, "v_mix": True}
    delta = {"heads": s["d_heads"], "kv_heads": s["d_kv_heads"], "dim": s["d_dim"], "vdim": s["d_vdim"], "conv": s["conv"]}
    latent = {"heads": s["l_heads"], "dim": 128, "rot_dim": 64, "vdim": 128, "kv_rank": 512, "scale": 192 ** -0.5, "rot": {"base": 10000.0, "dims": 64}}
    kinds = {"A": ("attention", attn), "D": ("delta", delta), "L": ("latent_attention", latent)}
    return {"architecture": "Zivulix", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-6},
            "layers": [{"type": kinds[c][0], "mixer": kinds[c][1], "mlp": {"kind": "dense", "ff": s["dense_ff"]}} for c in s["order"]]}


BILURAX_SIZES = {
    # the same widths, feed-forward sizes, expert counts and layer-run counts as MABIDRA_SIZES (6 layer runs for 5 layers / 3 for 2, the first
    # layer dense, the others mixtures of experts, the span `loop` running twice); every mixer is chunked soft-max attention over the grouped
    # heads of Mabidra's attention layers.  The chunk is as long as the benchmark's context, and `ctx` puts the decoded token at a chunk's last
    # position, so that a decode step reads as many keys as Mabidra's attention does.  The closest existing model at equal size is Mabidra with
    # sigmoid attention in every layer (its experts have two matrices where these have three).
    "2k-wide": dict(width=2048, heads=16, kv_heads=4, dim=128, vdim=128, chunk=2048, dense_ff=8192, experts=32, top=4, groups=4, keep=2, ff=1024, vocab=32768, n_layers=5,
                    loop=(1, 2, 2), ctx=2047, rank=64),
    "v3-layer": dict(width=7168, heads=64, kv_heads=8, dim=128, vdim=128, chunk=4096, dense_ff=18432, experts=32, top=8, groups=4, keep=2, ff=2048, vocab=32768, n_layers=2,
                     loop=(1, 2, 2), ctx=4095, rank=128),
}


def make_bilurax_config(s):
    attn = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["vdim"], "scale": s["dim"] ** -0.5, "softcap": 30.0, "mask": {"size": s["chunk"]}}
    moe = {"kind": "moe", "expert": {"ff": s["ff"], "limit": 7.0}, "router": {"experts": s["experts"], "top": s["top"], "groups": {"count": s["groups"], "keep": s["keep"]}, "scale": 2.0}}
    layers = [{"type": "attention", "mixer": attn, "mlp": {"kind": "dense", "ff": s["dense_ff"]} if i == 0 else moe} for i in range(s["n_layers"])]
    return {"architecture": "Bilurax", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0}, "logit_softcap": 50.0, "layers": layers,
            "loop": {"start": s["loop"][0], "stop": s["loop"][1], "times": s["loop"][2]}}


def make_mabidra_attn_config(s):
    """Mabidra at the sizes of a Bilurax size entry: sigmoid attention in every layer, the same dense and expert feed-forward sizes, the same loop"""
    attn = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["vdim"], "scale": s["dim"] ** -0.5, "bias_max": 1024, "q_temp": {"coef": 0.1, "every": 512}}
    moe = {"kind": "moe", "expert": {"ff": s["ff"]}, "router": {"experts": s["experts"], "top": s["top"]}}
    layers = [{"type": "attention", "mixer": attn, "mlp": {"kind": "dense", "ff": s["dense_ff"]} if i == 0 else moe} for i in range(s["n_layers"])]
    return {"architecture": "Mabidra", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-5, "groups": 4}, "embedding": {"scale": 1.0}, "layers": layers,
            "loop": {"start": s["loop"][0], "stop": s["loop"][1], "times": s["loop"][2]}}


def make_mabidra_dense_config(s):
    """Mabidra at the sizes of a Zivulix size entry: sigmoid attention for A and L, gated linear attention for D, dense feed-forwards"""
    attn = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["vdim"], "scale": s["dim"] ** -0.5, "bias_max": 1024, "q_temp": {"coef": 0.1, "every": 512}}
    gla = {"heads": s["d_heads"], "dim": s["d_dim"], "vdim": s["d_vdim"], "tau": 16.0}
    return {"architecture": "Mabidra", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-5, "groups": 4}, "embedding": {"scale": 1.0},
            "layers": [{"type": "gla" if c == "D" else "attention", "mixer": gla if c == "D" else attn, "mlp": {"kind": "dense", "ff": s["dense_ff"]}} for c in s["order"]]}


def random_model(cfg_dict, dtype=torch.bfloat16, device="cuda", size=None):
    if cfg_dict["architecture"] == "Bilurax":
        from ..models.configuration_bilurax import BiluraxConfig
        from ..models.modeling_bilurax import BiluraxForCausalLM
        model = BiluraxForCausalLM(BiluraxConfig.from_dict(cfg_dict), dtype=dtype, device=device)
    elif cfg_dict["architecture"] == "Zivulix":
        from ..models.configuration_zivulix import ZivulixConfig
        from ..models.modeling_zivulix import ZivulixForCausalLM
        model = ZivulixForCausalLM(ZivulixConfig.from_dict(cfg_dict), dtype=dtype, device=device)
    elif cfg_dict["architecture"] == "Mabidra":
        from ..models.configuration_mabidra import MabidraConfig
        from ..models.modeling_mabidra import MabidraForCausalLM
        from ..operators.attention import distance_bias_table
        model = MabidraForCausalLM(MabidraConfig.from_dict(cfg_dict), dtype=dtype, device=device)
        for layer in model.layers:
            if hasattr(layer.mix, "set_rank"):
                layer.mix.set_rank(size["rank"])
            else:
                layer.mix.bias_table = distance_bias_table(torch.randn(64, layer.mix.spec.heads, device=device), layer.mix.spec.bias_max)
    else:
        from ..models.configuration_lekapel import LekapelConfig
        from ..models.modeling_lekapel import LekapelForCausalLM
        model = LekapelForCausalLM(LekapelConfig.from_dict(cfg_dict), dtype=dtype, device=device)
    g = torch.Generator(device=device).manual_seed(1)
    for name, p in model.named_parameters():
        if p.dim() == 1:
            p.data.copy_(1 + 0.1 * torch.randn(p.shape, generator=g, device=device))
        else:
            p.data.copy_(torch.randn(p.shape, generator=g, device=device, dtype=torch.float32) * p.shape[-1] ** -0.5)
    return model.eval()


def model_bytes(model):
    return sum(p.numel() * p.element_size() for p in model.parameters())


def progress(msg):
    print("[model_bench] " + msg, file=sys.stderr, flush=True)


class Flusher:
    def __init__(self, dev):
        self.buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def __call__(self):
        self.buf.fill_(1)


def timed(fn, flush, iters=10, warmup=3):
    for _ in range(warmup):
        fn()
    ts = []
    for _ in range(iters):
        flush()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    return statistics.median(ts)


def engine_leg(name, size, flush, steps, warmup, family="lekapel"):
    from .engine import Engine
    cfg = {"lekapel": make_config, "mabidra": make_mabidra_config, "zivulix": make_zivulix_config, "mabidra-dense": make_mabidra_dense_config,
           "bilurax": make_bilurax_config, "mabidra-attn": make_mabidra_attn_config}[family](size)
    model = random_model(cfg, size=size)
    if family == "zivulix":      # norm weights are zero-centred, decays and the value blend inside their usual ranges
        for pname, p in model.named_parameters():
            if pname.endswith("weight") or pname.endswith("vmix") or pname.endswith("dt_bias"):
                p.data.sub_(1.0)
            if pname.endswith("a_log"):
                p.data.sub_(3.0)
    prompt_len, chunk, ctx = 4096, 2048, min(4096, size["window"] * 2) if family == "lekapel" else size["ctx"]
    eng = Engine(model, max_tokens=8 * (ctx + 64) + prompt_len, max_slots=9, max_step_tokens=chunk)
    g = torch.Generator().manual_seed(0)
    tok = lambda n: torch.randint(0, size["vocab"], (n,), generator=g).tolist()
    out = {"size": name, "config": {k: v for k, v in size.items()}, "weights_GB": model_bytes(model) / 1e9}
    progress(f"{family} {name}: model built")

    def prefill():
        p = tok(prompt_len)
        for lo in range(0, prompt_len, chunk):
            eng.step([("p", p[lo:lo + chunk], [len(p[lo:lo + chunk]) - 1] if lo + chunk >= prompt_len else [])], ["p"] if lo + chunk >= prompt_len else [])
    ms = timed(prefill, flush, iters=max(3, steps // 4), warmup=max(1, warmup // 2))
    out["prefill"] = {"prompt_tokens": prompt_len, "portion": chunk, "ms": ms, "tok_s": prompt_len / ms * 1e3}
    progress(f"{family} {name}: prefill {ms:.1f} ms")
    for bs in (1, 8):
        ids = [("d", i) for i in range(bs)]
        for i in ids:                                     # fill each sequence's cache to ctx tokens
            p = tok(ctx)
            for lo in range(0, ctx, chunk):
                eng.step([(i, p[lo:lo + chunk], [])])
        nxt = tok(bs)
        ms = timed(lambda: eng.step([(i, [t], [0]) for i, t in zip(ids, nxt)]), flush, iters=steps, warmup=warmup)
        for i in ids:
            eng.cache.close(i)
        out[f"decode_bs{bs}"] = {"ctx": ctx, "ms_per_step": ms, "tok_s": bs / ms * 1e3}
        progress(f"{family} {name}: decode x{bs} {ms:.3f} ms")
    return out


def kernel_leg(flush, peak_gbs, have_main_lib):
    """Token-major kernels against the DeepSeek path's kernels at DeepSeek-V3 sizes (bf16)."""
    dev, bf = torch.device("cuda"), torch.bfloat16
    seq = native.seq_lib()
    S = lambda: torch.cuda.current_stream().cuda_stream  # noqa: E731
    D, NH, R, ROPE, NOPE, QL, PAGE = 7168, 128, 512, 64, 128, 1536, 64
    rows = []

    def row(kernel, what, ms, nbytes, peer=None):
        r = {"kernel": kernel, "case": what, "us": ms * 1e3, "GBps": nbytes / ms / 1e6, "frac_of_measured_hbm": nbytes / ms / 1e6 / peak_gbs}
        if peer:
            r["closest"] = peer
        rows.append(r)
        return r

    g = torch.Generator(device=dev).manual_seed(7)
    rn = lambda *s, dt=bf: torch.randn(*s, generator=g, device=dev, dtype=torch.float32).to(dt)
    main = native.lib() if have_main_lib else None
    for T in (1, 8, 2048):
        # ---- fused residual sum + grouped norm + shift  vs  add_rmsnorm
        x, a, b = rn(T, D, dt=torch.float32), rn(T, D), rn(T, D)
        w, mu = rn(D), rn(D)
        xo, h, hs = torch.empty_like(x), torch.empty(T, D, dtype=bf, device=dev), torch.empty(T, D, dtype=bf, device=dev)
        meta = torch.tensor([[-1] + list(range(T - 1)), [-1] * T, [-1] * (T - 1) + [0]], dtype=torch.int32, device=dev)
        st = torch.zeros(2, D, device=dev)
        fn = lambda: native.check_seq(seq.ktb200_group_rmsnorm_shift(x.data_ptr(), a.data_ptr(), 30, b.data_ptr(), 30, 0.6, None, xo.data_ptr(), w.data_ptr(), 4, 1e-5, mu.data_ptr(),
                                                                     meta[0].data_ptr(), meta[1].data_ptr(), meta[2].data_ptr(), st.data_ptr(), h.data_ptr(), hs.data_ptr(), T, D, 30, S()))
        ours = timed(fn, flush)
        peer = None
        if main is not None:
            r16, d16, o16 = rn(T, D), rn(T, D), torch.empty(T, D, dtype=bf, device=dev)
            ms = timed(lambda: native.check(main.ktb200_add_rmsnorm(r16.data_ptr(), d16.data_ptr(), w.data_ptr(), 1e-6, o16.data_ptr(), T, D, S())), flush)
            peer = {"kernel": "add_rmsnorm_kernel", "us": ms * 1e3, "GBps": T * D * 8 / ms / 1e6, "frac_of_measured_hbm": T * D * 8 / ms / 1e6 / peak_gbs}
        row("group_norm_shift_kernel", f"T={T} width={D}", ours, T * D * (4 + 2 + 2 + 4 + 2 + 2), peer)
    # ---- paged latent attention, decode, ctx 4096: ours (window 4096, sink) vs the tcgen05 MLA decode kernel
    for B, ctx in ((1, 4096), (8, 4096), (1, 32768)):
        pages = (ctx + PAGE - 1) // PAGE
        cache = rn(B * pages + 1, PAGE, R + ROPE)
        ptab = torch.arange(B * pages, dtype=torch.int32, device=dev).reshape(B, pages)
        q, q_abs, lat = rn(B, NH, NOPE + ROPE), rn(B, NH, R), torch.empty(B, NH, R, dtype=bf, device=dev)
        pos = torch.full((B,), ctx - 1, dtype=torch.int32, device=dev)
        slot = torch.arange(B, dtype=torch.int32, device=dev)
        inv = torch.arange(ROPE // 2, dtype=torch.float64, device=dev).mul(-2.0 / ROPE).exp2()
        sink = torch.zeros(NH, device=dev)
        splits = max(1, min(32, ctx // 128, 296 // (B * NH // 8)))
        ws = torch.empty(max(1, seq.ktb200_latent_window_attn_workspace(B, NH, R, splits) // 4), device=dev)
        fn = lambda: native.check_seq(seq.ktb200_latent_window_attn(q.data_ptr(), q_abs.data_ptr(), NH, NOPE, ROPE, R, ROPE, 0, inv.data_ptr(), 0.07, sink.data_ptr(), ctx, pos.data_ptr(),
                                                                    slot.data_ptr(), ptab.data_ptr(), pages, PAGE, cache.data_ptr(), lat.data_ptr(), B, splits, ws.data_ptr(), 30, S()))
        ours = timed(fn, flush)
        nbytes = B * ctx * (R + ROPE) * 2
        peer = None
        if main is not None:
            qn, qp, o = rn(B, NH, R), rn(B, NH, ROPE), torch.empty(B, NH, R, dtype=bf, device=dev)
            kl = torch.full((B,), ctx, dtype=torch.int32, device=dev)
            wsb = main.ktb200_mla_workspace_bytes(B, NH, 0)
            mws = torch.zeros(max(wsb, 16), dtype=torch.uint8, device=dev)
            mp = native.MlaParams(B, NH, PAGE, pages, 0, 0.07, qn.data_ptr(), qp.data_ptr(), cache.data_ptr(), ptab.data_ptr(), kl.data_ptr(), o.data_ptr(), None, mws.data_ptr(), wsb,
                                  (B * pages + 1) * PAGE)
            ms = timed(lambda: native.check(main.ktb200_mla_decode(C.byref(mp), S())), flush)
            peer = {"kernel": "mla_decode_tc_kernel", "us": ms * 1e3, "GBps": nbytes / ms / 1e6, "frac_of_measured_hbm": nbytes / ms / 1e6 / peak_gbs}
        row("latent_window_attn_kernel (+merge)", f"decode B={B} ctx={ctx} heads={NH} splits={splits}", ours, nbytes, peer)
        q_rot = rn(B, NH, ROPE)
        wsb = seq.ktb200_latent_window_attn_tc_workspace(B, NH, ctx, ctx)
        tws = torch.empty(wsb // 4, device=dev)
        fn = lambda: native.check_seq(seq.ktb200_latent_window_attn_tc(q_abs.data_ptr(), q_rot.data_ptr(), NH, 0.07, sink.data_ptr(), ctx, pos.data_ptr(), slot.data_ptr(),
                                                                       ptab.data_ptr(), pages, PAGE, cache.data_ptr(), (B * pages + 1) * PAGE, lat.data_ptr(), B, ctx, tws.data_ptr(), wsb, S()))
        row("mla_decode_tc_kernel<split P> (+merge with sink)", f"decode B={B} ctx={ctx} heads={NH}", timed(fn, flush), nbytes, peer)
    # ---- a prompt portion: 2048 tokens of one sequence at positions 2048..4095, window 4096 (work is FLOP-shaped: per token
    #      and head a (576 + 512)-long multiply-add per visible key)
    T, ctx = 2048, 4096
    pages = ctx // PAGE
    cache = rn(pages + 1, PAGE, R + ROPE)
    ptab = torch.arange(pages, dtype=torch.int32, device=dev).reshape(1, pages)
    q, q_abs, q_rot, lat = rn(T, NH, NOPE + ROPE), rn(T, NH, R), rn(T, NH, ROPE), torch.empty(T, NH, R, dtype=bf, device=dev)
    pos = torch.arange(ctx - T, ctx, dtype=torch.int32, device=dev)
    slot = torch.zeros(T, dtype=torch.int32, device=dev)
    inv = torch.arange(ROPE // 2, dtype=torch.float64, device=dev).mul(-2.0 / ROPE).exp2()
    sink = torch.zeros(NH, device=dev)
    flops = float(sum(range(ctx - T + 1, ctx + 1))) * NH * (R + ROPE + R) * 2
    wsb = seq.ktb200_latent_window_attn_tc_workspace(T, NH, ctx, ctx)
    tws = torch.empty(wsb // 4, device=dev)
    f_tc = lambda: native.check_seq(seq.ktb200_latent_window_attn_tc(q_abs.data_ptr(), q_rot.data_ptr(), NH, 0.07, sink.data_ptr(), ctx, pos.data_ptr(), slot.data_ptr(), ptab.data_ptr(),
                                                                     pages, PAGE, cache.data_ptr(), (pages + 1) * PAGE, lat.data_ptr(), T, ctx, tws.data_ptr(), wsb, S()))
    f_cc = lambda: native.check_seq(seq.ktb200_latent_window_attn(q.data_ptr(), q_abs.data_ptr(), NH, NOPE, ROPE, R, ROPE, 0, inv.data_ptr(), 0.07, sink.data_ptr(), ctx, pos.data_ptr(),
                                                                  slot.data_ptr(), ptab.data_ptr(), pages, PAGE, cache.data_ptr(), lat.data_ptr(), T, 1, None, 30, S()))
    for name, f, it in (("mla_decode_tc_kernel<split P> (+merge with sink)", f_tc, 5), ("latent_window_attn_kernel", f_cc, 2)):
        ms = timed(f, flush, iters=it, warmup=1)
        rows.append({"kernel": name, "case": f"prompt portion T={T} positions {ctx - T}..{ctx - 1} heads={NH}", "us": ms * 1e3, "TFLOPs": flops / ms / 1e9})
    # ---- dense experts per pair (the fallback for rows too long for the by-expert kernels) : bytes = pairs * 3 * ff * width * 2
    E, top, ff = 32, 8, 2048
    Wg, Wu, Wd = rn(E, ff, D), rn(E, ff, D), rn(E, D, ff)
    for T in (1, 8):
        x = rn(T, D)
        ids = torch.stack([torch.randperm(E, generator=g, device=dev)[:top] for _ in range(T)]).to(torch.int64)
        wts = torch.rand(T, top, generator=g, device=dev)
        act, out = torch.empty(T * top, ff, dtype=bf, device=dev), torch.empty(T, D, device=dev)
        f1 = lambda: native.check_seq(seq.ktb200_experts_gate_up(x.data_ptr(), ids.data_ptr(), top, Wg.data_ptr(), Wu.data_ptr(), act.data_ptr(), T, D, ff, 0, 0.0, 30, S()))
        f2 = lambda: native.check_seq(seq.ktb200_experts_down(act.data_ptr(), ids.data_ptr(), wts.data_ptr(), top, Wd.data_ptr(), out.data_ptr(), T, D, ff, 30, S()))
        uniq = len(set(ids.flatten().tolist()))                            # every chosen expert is read from HBM at least once
        row("experts_gate_up_kernel", f"T={T} top={top} width={D} ff={ff} bf16", timed(f1, flush), uniq * 2 * ff * D * 2,
            {"kernel": "moe_block_kernel (Q4_K/Q6_K, whole block)", "frac_of_measured_hbm": 0.55, "note": "committed measurement of the DeepSeek path, one token"})
        row("experts_down_kernel", f"T={T} top={top} width={D} ff={ff} bf16", timed(f2, flush), uniq * ff * D * 2)
    # ---- the same by expert (what decode steps run): an expert's rows cross HBM once per two or four pairs routed to it
    for T in (1, 8, 16):
        x = rn(T, D)
        ids = torch.stack([torch.randperm(E, generator=g, device=dev)[:top] for _ in range(T)]).to(torch.int64)
        wts = torch.rand(T, top, generator=g, device=dev)
        act, out, pair_rows = torch.empty(T * top, ff, dtype=bf, device=dev), torch.empty(T, D, device=dev), torch.empty(T * top, D, device=dev)
        f1 = lambda: native.check_seq(seq.ktb200_experts_gate_up_by_expert(x.data_ptr(), ids.data_ptr(), top, E, Wg.data_ptr(), Wu.data_ptr(), act.data_ptr(), T, D, ff, 0, 0, 0.0, 30, S()))
        f2 = lambda: native.check_seq(seq.ktb200_experts_down_by_expert(act.data_ptr(), ids.data_ptr(), wts.data_ptr(), top, E, Wd.data_ptr(), pair_rows.data_ptr(), out.data_ptr(),
                                                                        T, D, ff, 0, 30, S()))
        uniq = len(set(ids.flatten().tolist()))
        row("experts_gate_up_by_expert_kernel", f"T={T} top={top} width={D} ff={ff} bf16", timed(f1, flush), uniq * 2 * ff * D * 2,
            {"kernel": "moe_block_kernel (Q4_K/Q6_K, whole block)", "frac_of_measured_hbm": 0.55, "note": "committed measurement of the DeepSeek path, one token"})
        row("experts_down_by_expert_kernel (+combine)", f"T={T} top={top} width={D} ff={ff} bf16", timed(f2, flush), uniq * ff * D * 2)
    return rows


def mabidra_kernel_leg(flush, peak_gbs, peak_tflops):
    """The kernels of the Mabidra operators at real layer sizes (bf16), each beside the like kernel of the Lekapel path."""
    dev, bf = torch.device("cuda"), torch.bfloat16
    seq = native.seq_lib()
    S = lambda: torch.cuda.current_stream().cuda_stream  # noqa: E731
    rows = []
    g = torch.Generator(device=dev).manual_seed(7)
    rn = lambda *s, dt=bf: torch.randn(*s, generator=g, device=dev, dtype=torch.float32).to(dt)

    def row(kernel, what, ms, nbytes=None, flops=None, peer=None):
        r = {"kernel": kernel, "case": what, "us": ms * 1e3}
        progress(f"{kernel} {what}: {ms * 1e3:.1f} us")
        if nbytes is not None:
            r.update(GBps=nbytes / ms / 1e6, frac_of_measured_hbm=nbytes / ms / 1e6 / peak_gbs)
        if flops is not None:
            r.update(TFLOPs=flops / ms / 1e9, frac_of_measured_bf16=flops / ms / 1e9 / peak_tflops)
        if peer:
            r["closest"] = peer
        rows.append(r)

    D = 7168
    for T in (1, 8, 2048):      # residual sum + two grouped norms  vs  residual sum + grouped norm + token shift
        x, y, w1, w2 = rn(T, D, dt=torch.float32), rn(T, D), rn(D), rn(D)
        xo, h = torch.empty_like(x), torch.empty(T, D, dtype=bf, device=dev)
        ours = timed(lambda: native.check_seq(seq.ktb200_group_rmsnorm_sandwich(x.data_ptr(), y.data_ptr(), 30, w1.data_ptr(), None, xo.data_ptr(), w2.data_ptr(), h.data_ptr(), 4,
                                                                                1e-5, 0.0, T, D, 30, S())), flush)
        a, b, mu, hs = rn(T, D), rn(T, D), rn(D), torch.empty(T, D, dtype=bf, device=dev)
        meta = torch.tensor([[-1] + list(range(T - 1)), [-1] * T, [-1] * (T - 1) + [0]], dtype=torch.int32, device=dev)
        st = torch.zeros(2, D, device=dev)
        ms = timed(lambda: native.check_seq(seq.ktb200_group_rmsnorm_shift(x.data_ptr(), a.data_ptr(), 30, b.data_ptr(), 30, 0.6, None, xo.data_ptr(), w1.data_ptr(), 4, 1e-5, mu.data_ptr(),
                                                                           meta[0].data_ptr(), meta[1].data_ptr(), meta[2].data_ptr(), st.data_ptr(), h.data_ptr(), hs.data_ptr(), T, D, 30,
                                                                           S())), flush)
        pb = T * D * (4 + 2 + 2 + 4 + 2 + 2)
        row("sandwich_norm_kernel", f"T={T} width={D}", ours, nbytes=T * D * (4 + 2 + 4 + 2),
            peer={"kernel": "group_norm_shift_kernel", "us": ms * 1e3, "frac_of_measured_hbm": pb / ms / 1e6 / peak_gbs})

    # ---- attention over the paged cache: 64 query heads on 8 key/value heads of 128 + 128 values; the Lekapel kernel beside it reads
    #      one latent row of 512 + 64 values per key for 128 heads (its tcgen05 path), the same bytes per key within 2x
    H, G, d, dv, PAGE = 64, 8, 128, 128, 64
    cw = G * (d + dv)
    bias, hb = rn(H, 1026, dt=torch.float32), rn(H, dt=torch.float32)

    def lekapel_attn(B, ctx, pos, slot, ptab, pages, T):
        R, ROPE, NH = 512, 64, 128
        cache = rn(B * pages + 1, PAGE, R + ROPE)
        q_abs, q_rot, lat = rn(T, NH, R), rn(T, NH, ROPE), torch.empty(T, NH, R, dtype=bf, device=dev)
        sink = torch.zeros(NH, device=dev)
        wsb = seq.ktb200_latent_window_attn_tc_workspace(T, NH, ctx, ctx)
        tws = torch.empty(wsb // 4, device=dev)
        return lambda: native.check_seq(seq.ktb200_latent_window_attn_tc(q_abs.data_ptr(), q_rot.data_ptr(), NH, 0.07, sink.data_ptr(), ctx, pos.data_ptr(), slot.data_ptr(),
                                                                         ptab.data_ptr(), pages, PAGE, cache.data_ptr(), (B * pages + 1) * PAGE, lat.data_ptr(), T, ctx, tws.data_ptr(),
                                                                         wsb, S()))

    from ..operators.attention import KSigmoidBiasAttention
    from ..models.configuration_mabidra import SigmoidAttentionSpec
    spec = SigmoidAttentionSpec(H, G, d, dv, d ** -0.5, 1024.0, 0.1, 512)
    picker = KSigmoidBiasAttention.pick_splits
    for B, ctx in ((1, 4096), (8, 4096), (1, 32768)):
        pages = (ctx + PAGE - 1) // PAGE
        cache = rn(B * pages + 1, PAGE, cw)
        ptab = torch.arange(B * pages, dtype=torch.int32, device=dev).reshape(B, pages)
        q, gate, out = rn(B, H, d), rn(B, H), torch.empty(B, H * dv, dtype=bf, device=dev)
        pos = torch.full((B,), ctx - 1, dtype=torch.int32, device=dev)
        slot = torch.arange(B, dtype=torch.int32, device=dev)
        holder = type("X", (), {"spec": spec})()
        seqs = torch.tensor([list(range(B)), [1] * B, [-1] * B, [-1] * B], dtype=torch.int32, device=dev)
        ours = {}
        for tc in (1, 0):
            splits = picker(holder, B, ctx, B, bool(tc))
            ws = torch.empty(max(1, seq.ktb200_sigmoid_bias_attn_workspace(B, H, dv, splits) // 4), device=dev)
            fn = lambda: native.check_seq(seq.ktb200_sigmoid_bias_attn(q.data_ptr(), H, G, d, dv, d ** -0.5, bias.data_ptr(), bias.shape[1], hb.data_ptr(), pos.data_ptr(), slot.data_ptr(),
                                                                       seqs.data_ptr(), B, B, ptab.data_ptr(), pages, PAGE, cache.data_ptr(), gate.data_ptr(), H, out.data_ptr(), B, splits,
                                                                       ws.data_ptr(), 30, tc, S()))
            ours[tc] = (timed(fn, flush), splits)
        ms = timed(lekapel_attn(B, ctx, pos, slot, ptab, pages, B), flush)
        lb = B * ctx * 576 * 2
        peer = {"kernel": "mla_decode_tc_kernel<split P> (+merge)", "case": "128 heads, latent 512 + 64", "us": ms * 1e3, "frac_of_measured_hbm": lb / ms / 1e6 / peak_gbs}
        row("sigmoid_attn_mma_kernel (+merge)", f"decode B={B} ctx={ctx} heads={H}/{G} splits={ours[1][1]}", ours[1][0], nbytes=B * ctx * cw * 2, peer=peer)
        row("sigmoid_attn_kernel (+merge), CUDA cores", f"decode B={B} ctx={ctx} heads={H}/{G} splits={ours[0][1]}", ours[0][0], nbytes=B * ctx * cw * 2, peer=peer)
    T, ctx = 2048, 4096
    pages = ctx // PAGE
    cache = rn(pages + 1, PAGE, cw)
    ptab = torch.arange(pages, dtype=torch.int32, device=dev).reshape(1, pages)
    q, gate, out = rn(T, H, d), rn(T, H), torch.empty(T, H * dv, dtype=bf, device=dev)
    pos = torch.arange(ctx - T, ctx, dtype=torch.int32, device=dev)
    slot = torch.zeros(T, dtype=torch.int32, device=dev)
    keys = float(sum(range(ctx - T + 1, ctx + 1)))
    seqs = torch.tensor([[0], [T], [-1], [-1]], dtype=torch.int32, device=dev)
    fn = lambda tc: native.check_seq(seq.ktb200_sigmoid_bias_attn(q.data_ptr(), H, G, d, dv, d ** -0.5, bias.data_ptr(), bias.shape[1], hb.data_ptr(), pos.data_ptr(), slot.data_ptr(),
                                                                  seqs.data_ptr(), 1, 1, ptab.data_ptr(), pages, PAGE, cache.data_ptr(), gate.data_ptr(), H, out.data_ptr(), T, 1, None, 30,
                                                                  tc, S()))
    ours = timed(lambda: fn(1), flush, iters=5, warmup=2)
    slow = timed(lambda: fn(0), flush, iters=2, warmup=1)
    ms = timed(lekapel_attn(1, ctx, pos, slot, ptab, pages, T), flush, iters=3, warmup=1)
    lf = keys * 128 * (576 + 512) * 2
    row("sigmoid_attn_kernel, CUDA cores", f"prompt portion T={T} positions {ctx - T}..{ctx - 1} heads={H}/{G}", slow, flops=keys * H * (d + dv) * 2)
    row("sigmoid_attn_mma_kernel", f"prompt portion T={T} positions {ctx - T}..{ctx - 1} heads={H}/{G}", ours, flops=keys * H * (d + dv) * 2,
        peer={"kernel": "mla_decode_tc_kernel<split P>", "case": "128 heads, latent 512 + 64", "us": ms * 1e3, "TFLOPs": lf / ms / 1e9, "frac_of_measured_bf16": lf / ms / 1e9 / peak_tflops})

    # ---- gated linear attention: decode reads and writes the fp32 state once (bytes); a prompt portion is a chain of T dependent steps
    GH, gd, gdv = 56, 128, 128
    n_in = 2 * GH * gd + 2 * GH * gdv
    for B, T in ((1, 1), (8, 1), (1, 2048)):
        proj, z, zb = rn(B * T, n_in), rn(B * T, GH * gd), rn(GH * gd)
        state, o = torch.zeros(2 * B, GH * gd * gdv, device=dev), torch.empty(B * T, GH * gdv, device=dev)
        seqs = torch.tensor([[i * T for i in range(B)], [T] * B, [2 * i for i in range(B)], [2 * i + 1 for i in range(B)]], dtype=torch.int32, device=dev)
        fn = lambda: native.check_seq(seq.ktb200_gla_scan(proj.data_ptr(), n_in, 0, GH * gd, 2 * GH * gd, z.data_ptr(), GH * gd, zb.data_ptr(), 16.0, GH, gd, gdv, seqs.data_ptr(), B, B,
                                                          B * T, state.data_ptr(), o.data_ptr(), 30, S()))
        ms = timed(fn, flush, iters=5 if T > 1 else 10)
        if T == 1:
            row("gla_scan_kernel", f"decode B={B} heads={GH} dim={gd} vdim={gdv}", ms, nbytes=B * GH * gd * gdv * 8,
                peer={"note": "no recurrent mixer in the Lekapel path; its decode attention reads the cache rows once, as this reads the state once"})
        else:
            row("gla_scan_kernel", f"prompt portion T={T} heads={GH} dim={gd} vdim={gdv}", ms, flops=float(T) * GH * gd * gdv * 4,
                peer={"note": "fp32 CUDA-core recurrence (state and decays are fp32 by design): %.2f us per token step" % (ms * 1e3 / T)})
        og, gt, nw = torch.empty(B * T, GH * gdv, dtype=bf, device=dev), rn(B * T, GH * gdv), rn(gdv)
        ms = timed(lambda: native.check_seq(seq.ktb200_gla_out(o.data_ptr(), nw.data_ptr(), 1e-5, gt.data_ptr(), GH * gdv, og.data_ptr(), B * T, GH, gdv, 30, S())), flush)
        row("gla_out_kernel", f"T={B * T} heads={GH} vdim={gdv}", ms, nbytes=B * T * GH * gdv * (4 + 2 + 2))
    # ---- activation
    for T, ff in ((8, 18432), (2048, 18432)):
        zz, oo, pq, cf = rn(T, ff), torch.empty(T, ff, dtype=bf, device=dev), torch.tensor([0.3, -0.2], device=dev), torch.tensor([0.3, -0.2, 0.1, 0.0], device=dev)
        ours = timed(lambda: native.check_seq(seq.ktb200_xielu(zz.data_ptr(), oo.data_ptr(), pq.data_ptr(), zz.numel(), 30, S())), flush)
        ms = timed(lambda: native.check_seq(seq.ktb200_poly_norm(zz.data_ptr(), oo.data_ptr(), cf.data_ptr(), 1e-5, T, ff, 30, S())), flush)
        row("xielu_kernel", f"T={T} ff={ff}", ours, nbytes=T * ff * 4, peer={"kernel": "poly_norm_kernel", "us": ms * 1e3, "frac_of_measured_hbm": T * ff * 4 / ms / 1e6 / peak_gbs})
    # ---- experts without a gate matrix, by expert, beside the gated ones (same kernels, two thirds of the bytes)
    E, top, ff = 32, 8, 2048
    Wg, Wu, Wd = rn(E, ff, D), rn(E, ff, D), rn(E, D, ff)
    for T in (1, 8, 16):
        x = rn(T, D)
        ids = torch.stack([torch.randperm(E, generator=g, device=dev)[:top] for _ in range(T)]).to(torch.int64)
        act = torch.empty(T * top, ff, dtype=bf, device=dev)
        uniq = len(set(ids.flatten().tolist()))
        ours = timed(lambda: native.check_seq(seq.ktb200_experts_gate_up_by_expert(x.data_ptr(), ids.data_ptr(), top, E, None, Wu.data_ptr(), act.data_ptr(), T, D, ff, 0, 0, 0.0, 30, S())), flush)
        ms = timed(lambda: native.check_seq(seq.ktb200_experts_gate_up_by_expert(x.data_ptr(), ids.data_ptr(), top, E, Wg.data_ptr(), Wu.data_ptr(), act.data_ptr(), T, D, ff, 0, 0, 0.0, 30, S())), flush)
        row("experts_gate_up_by_expert_kernel (no gate, relu^2)", f"T={T} top={top} width={D} ff={ff} bf16", ours, nbytes=uniq * ff * D * 2,
            peer={"kernel": "experts_gate_up_by_expert_kernel (gated)", "us": ms * 1e3, "frac_of_measured_hbm": uniq * 2 * ff * D * 2 / ms / 1e6 / peak_gbs})
    return rows


def zivulix_kernel_leg(flush, peak_gbs, peak_tflops):
    """The kernels of the Zivulix operators at real layer sizes (bf16), each beside the like kernel of the Mabidra path."""
    dev, bf = torch.device("cuda"), torch.bfloat16
    seq = native.seq_lib()
    S = lambda: torch.cuda.current_stream().cuda_stream  # noqa: E731
    rows = []
    g = torch.Generator(device=dev).manual_seed(7)
    rn = lambda *s, dt=bf: torch.randn(*s, generator=g, device=dev, dtype=torch.float32).to(dt)

    def row(kernel, what, ms, nbytes=None, flops=None, peer=None):
        r = {"kernel": kernel, "case": what, "us": ms * 1e3}
        progress(f"{kernel} {what}: {ms * 1e3:.1f} us")
        if nbytes is not None:
            r.update(GBps=nbytes / ms / 1e6, frac_of_measured_hbm=nbytes / ms / 1e6 / peak_gbs)
        if flops is not None:
            r.update(TFLOPs=flops / ms / 1e9, frac_of_measured_bf16=flops / ms / 1e9 / peak_tflops)
        if peer:
            r["closest"] = peer
        rows.append(r)

    def peer_of(kernel, ms, nbytes=None, flops=None):
        r = {"kernel": kernel, "us": ms * 1e3}
        if nbytes is not None:
            r["frac_of_measured_hbm"] = nbytes / ms / 1e6 / peak_gbs
        if flops is not None:
            r.update(TFLOPs=flops / ms / 1e9, frac_of_measured_bf16=flops / ms / 1e9 / peak_tflops)
        return r

    D = 7168
    for T in (1, 8, 2048):      # residual sum + norm of the added term, the sum rounded for the next GEMM  vs  residual sum + two grouped norms
        x, y, w1, w2 = rn(T, D, dt=torch.float32), rn(T, D), rn(D), rn(D)
        xo, h = torch.empty_like(x), torch.empty(T, D, dtype=bf, device=dev)
        ours = timed(lambda: native.check_seq(seq.ktb200_group_rmsnorm_sandwich(x.data_ptr(), y.data_ptr(), 30, w1.data_ptr(), None, xo.data_ptr(), None, h.data_ptr(), 1, 1e-6, 1.0,
                                                                                T, D, 30, S())), flush)
        ms = timed(lambda: native.check_seq(seq.ktb200_group_rmsnorm_sandwich(x.data_ptr(), y.data_ptr(), 30, w1.data_ptr(), None, xo.data_ptr(), w2.data_ptr(), h.data_ptr(), 4, 1e-5,
                                                                              0.0, T, D, 30, S())), flush)
        nb = T * D * (4 + 2 + 4 + 2)
        row("sandwich_norm_kernel (zero-centred weights, plain h)", f"T={T} width={D}", ours, nbytes=nb, peer=peer_of("sandwich_norm_kernel (two grouped norms)", ms, nb))

    # ---- attention: 64 query heads on 8 key/value heads of 128 + 128 values, as the Mabidra attention beside it
    H, G, d, dv, PAGE = 64, 8, 128, 128, 64
    cw, n_in = G * (d + dv), (64 + 8) * 128 + 8 * 128
    inv = torch.arange(d // 4, dtype=torch.float64, device=dev).mul(-4.0 / d).exp2() / 4.0
    lam = torch.tensor([0.3], device=dev)
    for T in (8, 2048):         # rotation + unit rms + value blend + cache write  vs  per-head norms + temperature + cache write
        pages = (T + PAGE - 1) // PAGE
        proj, vo, cache, qo = rn(T, n_in), rn(T, G * dv), rn(pages + 1, PAGE, cw), torch.empty(T, H, d, dtype=bf, device=dev)
        ptab = torch.arange(pages, dtype=torch.int32, device=dev).reshape(1, pages)
        pos, slot = torch.arange(T, dtype=torch.int32, device=dev), torch.zeros(T, dtype=torch.int32, device=dev)
        ours = timed(lambda: native.check_seq(seq.ktb200_rope_norm_cache_write(proj.data_ptr(), n_in, 0, H * d, (H + G) * d, H, G, d, dv, d // 2, 1, inv.data_ptr(), 1, None, None, 0, 1e-6,
                                                                               vo.data_ptr(), G * dv, lam.data_ptr(), pos.data_ptr(), slot.data_ptr(), ptab.data_ptr(), pages, PAGE,
                                                                               cache.data_ptr(), qo.data_ptr(), T, 30, S())), flush)
        qw, kw = rn(d), rn(d)
        ms = timed(lambda: native.check_seq(seq.ktb200_qk_norm_cache_write(proj.data_ptr(), n_in, H, G, d, dv, qw.data_ptr(), kw.data_ptr(), 1e-5, 0.1, 512, pos.data_ptr(),
                                                                           slot.data_ptr(), ptab.data_ptr(), pages, PAGE, cache.data_ptr(), qo.data_ptr(), T, 30, S())), flush)
        nb = T * (n_in + H * d + cw) * 2
        row("rope_norm_cache_write_kernel", f"T={T} heads={H}/{G} dim={d}", ours, nbytes=nb + T * G * dv * 2, peer=peer_of("qk_norm_cache_write_kernel", ms, nb))

    bias, hb = rn(H, 1026, dt=torch.float32), rn(H, dt=torch.float32)
    from ..models.configuration_mabidra import SigmoidAttentionSpec
    from ..models.configuration_zivulix import CappedWindowAttentionSpec
    from ..operators.attention import KCappedWindowAttention, KSigmoidBiasAttention
    for B, ctx in ((1, 4096), (8, 4096), (1, 32768)):
        pages = (ctx + PAGE - 1) // PAGE
        cache = rn(B * pages + 1, PAGE, cw)
        ptab = torch.arange(B * pages, dtype=torch.int32, device=dev).reshape(B, pages)
        q, gate, out = rn(B, H, d), rn(B, H), torch.empty(B, H * dv, dtype=bf, device=dev)
        pos = torch.full((B,), ctx - 1, dtype=torch.int32, device=dev)
        slot = torch.arange(B, dtype=torch.int32, device=dev)
        seqs = torch.tensor([list(range(B)), [1] * B, [-1] * B, [-1] * B], dtype=torch.int32, device=dev)
        mine = type("X", (), {"spec": CappedWindowAttentionSpec(H, G, d, dv, d ** -0.5, 30.0, ctx, None, True, True)})()
        theirs = type("X", (), {"spec": SigmoidAttentionSpec(H, G, d, dv, d ** -0.5, 1024.0, 0.1, 512)})()
        sp = KSigmoidBiasAttention.pick_splits(theirs, B, ctx, B, True)
        ws = torch.empty(max(1, seq.ktb200_sigmoid_bias_attn_workspace(B, H, dv, sp) // 4), device=dev)
        ms = timed(lambda: native.check_seq(seq.ktb200_sigmoid_bias_attn(q.data_ptr(), H, G, d, dv, d ** -0.5, bias.data_ptr(), bias.shape[1], hb.data_ptr(), pos.data_ptr(), slot.data_ptr(),
                                                                         seqs.data_ptr(), B, B, ptab.data_ptr(), pages, PAGE, cache.data_ptr(), gate.data_ptr(), H, out.data_ptr(), B, sp,
                                                                         ws.data_ptr(), 30, 1, S())), flush)
        nb = B * ctx * cw * 2
        peer = peer_of("sigmoid_attn_mma_kernel (+merge)", ms, nb)
        for tc in (1, 0):
            splits = KCappedWindowAttention.pick_splits(mine, B, ctx, B, bool(tc))
            ws2 = torch.empty(max(1, seq.ktb200_window_softmax_attn_workspace(B, H, dv, splits) // 4), device=dev)
            fn = lambda: native.check_seq(seq.ktb200_window_softmax_attn(q.data_ptr(), H, G, d, dv, d ** -0.5, None, 30.0, ctx, 0, pos.data_ptr(), slot.data_ptr(), seqs.data_ptr(), B, B,
                                                                         ptab.data_ptr(), pages, PAGE, cache.data_ptr(), out.data_ptr(), B, splits, ws2.data_ptr(), 30, tc, S()))
            row("window_softmax_attn_mma_kernel (+merge)" if tc else "window_softmax_attn_kernel (+merge), CUDA cores", f"decode B={B} ctx={ctx} heads={H}/{G} splits={splits}",
                timed(fn, flush), nbytes=nb, peer=peer)
    T, ctx = 2048, 4096
    pages = ctx // PAGE
    cache = rn(pages + 1, PAGE, cw)
    ptab = torch.arange(pages, dtype=torch.int32, device=dev).reshape(1, pages)
    q, gate, out = rn(T, H, d), rn(T, H), torch.empty(T, H * dv, dtype=bf, device=dev)
    pos = torch.arange(ctx - T, ctx, dtype=torch.int32, device=dev)
    slot = torch.zeros(T, dtype=torch.int32, device=dev)
    keys = float(sum(range(ctx - T + 1, ctx + 1)))
    seqs = torch.tensor([[0], [T], [-1], [-1]], dtype=torch.int32, device=dev)
    fl = keys * H * (d + dv) * 2
    ms = timed(lambda: native.check_seq(seq.ktb200_sigmoid_bias_attn(q.data_ptr(), H, G, d, dv, d ** -0.5, bias.data_ptr(), bias.shape[1], hb.data_ptr(), pos.data_ptr(), slot.data_ptr(),
                                                                     seqs.data_ptr(), 1, 1, ptab.data_ptr(), pages, PAGE, cache.data_ptr(), gate.data_ptr(), H, out.data_ptr(), T, 1, None, 30,
                                                                     1, S())), flush, iters=5, warmup=2)
    peer = peer_of("sigmoid_attn_mma_kernel", ms, flops=fl)
    fn = lambda tc, win: native.check_seq(seq.ktb200_window_softmax_attn(q.data_ptr(), H, G, d, dv, d ** -0.5, None, 30.0, win, 0, pos.data_ptr(), slot.data_ptr(), seqs.data_ptr(), 1, 1,
                                                                         ptab.data_ptr(), pages, PAGE, cache.data_ptr(), out.data_ptr(), T, 1, None, 30, tc, S()))
    row("window_softmax_attn_mma_kernel", f"prompt portion T={T} positions {ctx - T}..{ctx - 1} heads={H}/{G}, every earlier key in sight", timed(lambda: fn(1, ctx), flush, iters=5, warmup=2),
        flops=fl, peer=peer)
    row("window_softmax_attn_mma_kernel", f"the same, window 1024", timed(lambda: fn(1, 1024), flush, iters=5, warmup=2), flops=float(T) * 1024 * H * (d + dv) * 2)
    row("window_softmax_attn_kernel, CUDA cores", f"prompt portion T={T} positions {ctx - T}..{ctx - 1} heads={H}/{G}", timed(lambda: fn(0, ctx), flush, iters=2, warmup=1), flops=fl)

    # ---- the gated delta rule: decode reads and writes the fp32 state once (bytes); a prompt portion is a chain of T dependent steps
    DH, DG, dd, ddv, taps = 56, 28, 128, 128, 4
    C_ = 2 * DG * dd + DH * ddv
    n_in = C_ + DH * ddv + 2 * DH
    n_in = (n_in + 7) // 8 * 8
    sw = DH * dd * ddv + (taps - 1) * C_
    GH, gd, gdv = 56, 128, 128
    g_in = 2 * GH * gd + 2 * GH * gdv
    for B, T in ((1, 1), (8, 1), (1, 2048)):
        proj, cwt = rn(B * T, n_in), rn(C_, taps)
        al, dtb = rn(DH, dt=torch.float32) - 3.0, rn(DH, dt=torch.float32)
        state = torch.zeros(2 * B, sw, device=dev)
        f32 = lambda *s: torch.empty(*s, device=dev)
        qn, kn, vv, be, de, o = f32(B * T, DG * dd), f32(B * T, DG * dd), f32(B * T, DH * ddv), f32(B * T, DH), f32(B * T, DH), f32(B * T, DH * ddv)
        seqs = torch.tensor([[i * T for i in range(B)], [T] * B, [2 * i for i in range(B)], [2 * i + 1 for i in range(B)]], dtype=torch.int32, device=dev)
        seq_of = torch.arange(B, dtype=torch.int32, device=dev).repeat_interleave(T)
        prep = lambda: native.check_seq(seq.ktb200_delta_prep(proj.data_ptr(), n_in, 0, C_ + DH * ddv, C_ + DH * ddv + DH, cwt.data_ptr(), taps, al.data_ptr(), dtb.data_ptr(), DH, DG, dd,
                                                              ddv, 1e-6, seq_of.data_ptr(), seqs.data_ptr(), B, state.data_ptr(), sw, qn.data_ptr(), kn.data_ptr(), vv.data_ptr(),
                                                              be.data_ptr(), de.data_ptr(), B * T, 30, S()))
        scan = lambda: native.check_seq(seq.ktb200_delta_scan(qn.data_ptr(), kn.data_ptr(), vv.data_ptr(), be.data_ptr(), de.data_ptr(), DH, DG, dd, ddv, seqs.data_ptr(), B, B,
                                                              state.data_ptr(), sw, o.data_ptr(), S()))
        prep()
        gproj, z, zb = rn(B * T, g_in), rn(B * T, GH * gd), rn(GH * gd)
        gstate, go = torch.zeros(2 * B, GH * gd * gdv, device=dev), torch.empty(B * T, GH * gdv, device=dev)
        gla = lambda: native.check_seq(seq.ktb200_gla_scan(gproj.data_ptr(), g_in, 0, GH * gd, 2 * GH * gd, z.data_ptr(), GH * gd, zb.data_ptr(), 16.0, GH, gd, gdv, seqs.data_ptr(), B, B,
                                                           B * T, gstate.data_ptr(), go.data_ptr(), 30, S()))
        it = 5 if T > 1 else 10
        ms_prep, ms_scan, ms_gla = timed(prep, flush, iters=it), timed(scan, flush, iters=it), timed(gla, flush, iters=it)
        row("delta_prep_kernel", f"B={B} T={T} heads={DH}/{DG} taps={taps}", ms_prep, nbytes=B * T * (C_ * 2 + C_ * 4 + 2 * DH * 4) + B * (taps - 1) * C_ * 8)
        if T == 1:
            nb = B * DH * dd * ddv * 8
            row("delta_scan_kernel", f"decode B={B} heads={DH}/{DG} dim={dd} vdim={ddv}", ms_scan, nbytes=nb, peer=peer_of("gla_scan_kernel", ms_gla, B * GH * gd * gdv * 8))
        else:
            fl = float(T) * DH * dd * ddv * 6
            row("delta_scan_kernel", f"prompt portion T={T} heads={DH}/{DG} dim={dd} vdim={ddv} ({ms_scan * 1e3 / T:.2f} us per token step)", ms_scan, flops=fl,
                peer=dict(peer_of("gla_scan_kernel", ms_gla, flops=float(T) * GH * gd * gdv * 4), us_per_token_step=ms_gla * 1e3 / T))
    # ---- activation
    for T, ff in ((8, 18432), (2048, 18432)):
        gu, oo, zz, pq = rn(T, 2 * ff), torch.empty(T, ff, dtype=bf, device=dev), rn(T, ff), torch.tensor([0.3, -0.2], device=dev)
        ours = timed(lambda: native.check_seq(seq.ktb200_gated_act_mul(gu.data_ptr(), gu.data_ptr() + 2 * ff, 2 * ff, oo.data_ptr(), T, ff, 1, 0.0, 30, S())), flush)
        ms = timed(lambda: native.check_seq(seq.ktb200_xielu(zz.data_ptr(), oo.data_ptr(), pq.data_ptr(), zz.numel(), 30, S())), flush)
        row("gated_act_mul_kernel (gelu_tanh)", f"T={T} ff={ff}", ours, nbytes=T * ff * 6, peer=peer_of("xielu_kernel", ms, T * ff * 4))
    return rows


def bilurax_kernel_leg(flush, peak_gbs, peak_tflops):
    """The kernels of the Bilurax operators at real layer sizes (bf16), each beside the like kernel of the closest existing path."""
    dev, bf = torch.device("cuda"), torch.bfloat16
    seq = native.seq_lib()
    S = lambda: torch.cuda.current_stream().cuda_stream  # noqa: E731
    rows = []
    g = torch.Generator(device=dev).manual_seed(7)
    rn = lambda *s, dt=bf: torch.randn(*s, generator=g, device=dev, dtype=torch.float32).to(dt)

    def peer_of(kernel, ms, nbytes=None, flops=None):
        r = {"kernel": kernel, "us": ms * 1e3}
        if nbytes is not None:
            r["frac_of_measured_hbm"] = nbytes / ms / 1e6 / peak_gbs
        if flops is not None:
            r.update(TFLOPs=flops / ms / 1e9, frac_of_measured_bf16=flops / ms / 1e9 / peak_tflops)
        return r

    def row(kernel, what, ms, nbytes=None, flops=None, peer=None):
        r = dict(peer_of(kernel, ms, nbytes, flops), case=what)
        if nbytes is not None:
            r["GBps"] = nbytes / ms / 1e6
        progress(f"{kernel} {what}: {ms * 1e3:.1f} us")
        if peer:
            r["closest"] = peer
        rows.append(r)

    D = 7168
    from ..operators.norm import KGroupRMSNormShift
    for T in (1, 8, 2048):      # a pass opening: x + y + x0 + step, norm, shift  vs  Lekapel's x + m (a + b), norm in 4 groups, shift
        x, y, x0, step = rn(T, D, dt=torch.float32), rn(T, D), rn(T, D, dt=torch.float32), rn(D, dt=torch.float32)
        state = torch.zeros(2, D, device=dev)
        meta = torch.zeros(5, T, dtype=torch.int32, device=dev)
        meta[2] = torch.arange(-1, T - 1, dtype=torch.int32, device=dev)
        meta[3], meta[4] = -1, -1
        batch = type("B", (), {"prev_idx": meta[2], "rd_row": meta[3], "wr_row": meta[4]})()
        mine, theirs = KGroupRMSNormShift(D, 1, 1e-6, True), KGroupRMSNormShift(D, 4, 1e-5, True)
        ours = timed(lambda: mine(x, y, x0, 1.0, batch, state, want_h=False, row_add=step), flush)
        ms = timed(lambda: theirs(x, y, y, 0.6, batch, state, want_h=True), flush)
        row("group_norm_shift_kernel (two addends of which one fp32, a row vector, shifted output only)", f"T={T} width={D}", ours, nbytes=T * D * (4 + 2 + 4 + 4 + 2),
            peer=peer_of("group_norm_shift_kernel (two bf16 addends, 4 groups, both outputs)", ms, T * D * (4 + 2 + 2 + 4 + 2 + 2)))

    # ---- attention: 64 query heads on 8 key/value heads of 128 + 128 values
    H, G, d, dv, PAGE = 64, 8, 128, 128, 64
    cw, n_in = G * (d + dv), (64 + 8) * 128 + 8 * 128
    inv = torch.arange(d // 4, dtype=torch.float64, device=dev).mul(-4.0 / d).exp2() / 4.0
    lam = torch.tensor([0.3], device=dev)
    for T in (8, 2048):         # row-wide weighted q / k norms + value unit rms + cache write  vs  rotation + per-head unit rms + value blend + cache write
        pages = (T + PAGE - 1) // PAGE
        proj, vo, cache, qo = rn(T, n_in), rn(T, G * dv), rn(pages + 1, PAGE, cw), torch.empty(T, H, d, dtype=bf, device=dev)
        qw, kw = rn(H * d), rn(G * d)
        ptab = torch.arange(pages, dtype=torch.int32, device=dev).reshape(1, pages)
        pos, slot = torch.arange(T, dtype=torch.int32, device=dev), torch.zeros(T, dtype=torch.int32, device=dev)
        ours = timed(lambda: native.check_seq(seq.ktb200_rope_norm_cache_write(proj.data_ptr(), n_in, 0, H * d, (H + G) * d, H, G, d, dv, 0, 0, None, 2, qw.data_ptr(), kw.data_ptr(), 1,
                                                                               1e-6, None, 0, None, pos.data_ptr(), slot.data_ptr(), ptab.data_ptr(), pages, PAGE, cache.data_ptr(),
                                                                               qo.data_ptr(), T, 30, S())), flush)
        ms = timed(lambda: native.check_seq(seq.ktb200_rope_norm_cache_write(proj.data_ptr(), n_in, 0, H * d, (H + G) * d, H, G, d, dv, d // 2, 1, inv.data_ptr(), 1, None, None, 0, 1e-6,
                                                                             vo.data_ptr(), G * dv, lam.data_ptr(), pos.data_ptr(), slot.data_ptr(), ptab.data_ptr(), pages, PAGE,
                                                                             cache.data_ptr(), qo.data_ptr(), T, 30, S())), flush)
        nb = T * (n_in + H * d + cw) * 2
        row("rope_norm_cache_write_kernel (row-wide q/k norms, unit-rms values)", f"T={T} heads={H}/{G} dim={d}", ours, nbytes=nb,
            peer=peer_of("rope_norm_cache_write_kernel (rotation, per-head unit rms, value blend)", ms, nb + T * G * dv * 2))

    from ..operators.attention import softmax_attention_splits
    temp = 0.5 + torch.rand(H, device=dev)
    for B, ctx in ((1, 4096), (8, 4096), (1, 32768)):      # the chunk mask with a head temperature  vs  the window mask of the same kernel
        pages = (ctx + PAGE - 1) // PAGE
        cache = rn(B * pages + 1, PAGE, cw)
        ptab = torch.arange(B * pages, dtype=torch.int32, device=dev).reshape(B, pages)
        q, out = rn(B, H, d), torch.empty(B, H * dv, dtype=bf, device=dev)
        pos = torch.full((B,), ctx - 1, dtype=torch.int32, device=dev)
        slot = torch.arange(B, dtype=torch.int32, device=dev)
        seqs = torch.tensor([list(range(B)), [1] * B, [-1] * B, [-1] * B], dtype=torch.int32, device=dev)
        nb = B * ctx * cw * 2
        for tc in (1, 0):
            splits = softmax_attention_splits(H, G, ctx, B, B, bool(tc))
            ws2 = torch.empty(max(1, seq.ktb200_window_softmax_attn_workspace(B, H, dv, splits) // 4), device=dev)
            fn = lambda hs, win, ch: native.check_seq(seq.ktb200_window_softmax_attn(q.data_ptr(), H, G, d, dv, d ** -0.5, hs, 30.0, win, ch, pos.data_ptr(), slot.data_ptr(),
                                                                                     seqs.data_ptr(), B, B, ptab.data_ptr(), pages, PAGE, cache.data_ptr(), out.data_ptr(), B, splits,
                                                                                     ws2.data_ptr(), 30, tc, S()))
            ms = timed(lambda: fn(None, ctx, 0), flush)
            name = "window_softmax_attn_mma_kernel (+merge)" if tc else "window_softmax_attn_kernel (+merge), CUDA cores"
            row(name + ", chunk mask, head temperature", f"decode B={B} last position of a chunk of {ctx} heads={H}/{G} splits={splits}",
                timed(lambda: fn(temp.data_ptr(), 0, ctx), flush), nbytes=nb, peer=peer_of(name + ", window mask", ms, nb))
    T, ctx = 2048, 4096
    pages = ctx // PAGE
    cache = rn(pages + 1, PAGE, cw)
    ptab = torch.arange(pages, dtype=torch.int32, device=dev).reshape(1, pages)
    q, out = rn(T, H, d), torch.empty(T, H * dv, dtype=bf, device=dev)
    pos = torch.arange(ctx - T, ctx, dtype=torch.int32, device=dev)
    slot = torch.zeros(T, dtype=torch.int32, device=dev)
    seqs = torch.tensor([[0], [T], [-1], [-1]], dtype=torch.int32, device=dev)
    fn = lambda hs, win, ch: native.check_seq(seq.ktb200_window_softmax_attn(q.data_ptr(), H, G, d, dv, d ** -0.5, hs, 30.0, win, ch, pos.data_ptr(), slot.data_ptr(), seqs.data_ptr(), 1, 1,
                                                                             ptab.data_ptr(), pages, PAGE, cache.data_ptr(), out.data_ptr(), T, 1, None, 30, 1, S()))
    fl = float(sum(range(ctx - T + 1, ctx + 1))) * H * (d + dv) * 2
    ms = timed(lambda: fn(None, ctx, 0), flush, iters=5, warmup=2)
    row("window_softmax_attn_mma_kernel, chunk mask, head temperature", f"prompt portion T={T} positions {ctx - T}..{ctx - 1} heads={H}/{G}, one chunk of {ctx}",
        timed(lambda: fn(temp.data_ptr(), 0, ctx), flush, iters=5, warmup=2), flops=fl, peer=peer_of("window_softmax_attn_mma_kernel, window mask", ms, flops=fl))
    fl = 2 * float(sum(range(1, 1025))) * H * (d + dv) * 2
    ms = timed(lambda: fn(None, 1024, 0), flush, iters=5, warmup=2)
    row("window_softmax_attn_mma_kernel, chunk mask, head temperature", f"the same, chunks of 1024 (half the keys of a window of 1024)",
        timed(lambda: fn(temp.data_ptr(), 0, 1024), flush, iters=5, warmup=2), flops=fl, peer=peer_of("window_softmax_attn_mma_kernel, window of 1024", ms, flops=float(T) * 1024 * H * (d + dv) * 2))

    # ---- router: 256 experts in 8 groups of which 4 are kept, 8 choices (DeepSeek-V3's shape)  vs  soft-max over all, 8 largest
    from ..operators.gate import KGroupedSigmoidGate, KSoftmaxTopKGate
    E, top = 256, 8
    mine, theirs = KGroupedSigmoidGate(D, E, top, 8, 4, 2.0), KSoftmaxTopKGate(D, E, top)
    mine.weight.data.copy_(rn(E, D, dt=torch.float32) * D ** -0.5)
    theirs.weight.data.copy_(mine.weight.data)
    mine.correction.data.copy_(rn(E, dt=torch.float32) * 0.1)
    for T in (1, 8, 2048):
        x = rn(T, D)
        ours, ms = timed(lambda: mine(x), flush), timed(lambda: theirs(x), flush)
        nb = E * D * 4 + T * D * 2
        small = T < mine.gemm_min_tokens
        row("gate_kernel (sigmoid, correction, groups)" if small else "fp32 GEMM + gate_select_kernel", f"T={T} experts={E} width={D} top={top}", ours, nbytes=nb,
            peer=peer_of("gate_kernel (soft-max, greedy)" if small else "fp32 GEMM + torch soft-max and top-k", ms, nb))

    # ---- experts: the clamped sigmoid form beside silu(gate) * up in the same kernels
    E, top, ff = 32, 8, 2048
    Wg, Wu = rn(E, ff, D) * D ** -0.5, rn(E, ff, D) * D ** -0.5
    for T in (1, 8):
        x, act = rn(T, D), torch.empty(T * top, ff, dtype=bf, device=dev)
        ids = torch.stack([torch.randperm(E, generator=g, device=dev)[:top] for _ in range(T)])
        uniq = int(ids.unique().numel())
        fn = lambda kind, lim: native.check_seq(seq.ktb200_experts_gate_up_by_expert(x.data_ptr(), ids.data_ptr(), top, E, Wg.data_ptr(), Wu.data_ptr(), act.data_ptr(), T, D, ff, 0, kind,
                                                                                     lim, 30, S()))
        ours, ms = timed(lambda: fn(2, 7.0), flush), timed(lambda: fn(0, 0.0), flush)
        nb = uniq * 2 * ff * D * 2
        row("experts_gate_up_by_expert_kernel (clamped sigmoid form)", f"T={T} top={top} width={D} ff={ff} bf16", ours, nbytes=nb,
            peer=peer_of("experts_gate_up_by_expert_kernel (silu)", ms, nb))
    # ---- elementwise: expert activation over grouped-GEMM outputs, relu squared, capped logits
    for P in (64, 2048 * 8):
        gg, uu, oo = rn(P, ff), rn(P, ff), torch.empty(P, ff, dtype=bf, device=dev)
        gu = rn(P, 2 * ff)
        ours = timed(lambda: native.check_seq(seq.ktb200_gated_act_mul(gg.data_ptr(), uu.data_ptr(), ff, oo.data_ptr(), P, ff, 2, 7.0, 30, S())), flush)
        ms = timed(lambda: native.check_seq(seq.ktb200_gated_act_mul(gu.data_ptr(), gu.data_ptr() + 2 * ff, 2 * ff, oo.data_ptr(), P, ff, 1, 0.0, 30, S())), flush)
        row("gated_act_mul_kernel (clamped sigmoid form, separate gate and up rows)", f"pairs={P} ff={ff}", ours, nbytes=P * ff * 6,
            peer=peer_of("gated_act_mul_kernel (gelu_tanh, stacked rows)", ms, P * ff * 6))
    for T, F_ in ((8, 18432), (2048, 18432)):
        zz, oo, pq = rn(T, F_), torch.empty(T, F_, dtype=bf, device=dev), torch.tensor([0.3, -0.2], device=dev)
        ours = timed(lambda: native.check_seq(seq.ktb200_relu_squared(zz.data_ptr(), oo.data_ptr(), zz.numel(), 30, S())), flush)
        ms = timed(lambda: native.check_seq(seq.ktb200_xielu(zz.data_ptr(), oo.data_ptr(), pq.data_ptr(), zz.numel(), 30, S())), flush)
        row("relu_squared_kernel", f"T={T} ff={F_}", ours, nbytes=T * F_ * 4, peer=peer_of("xielu_kernel", ms, T * F_ * 4))
    for T, V in ((8, 32768), (2048, 32768)):
        zz, of, oo, pq = rn(T, V), torch.empty(T, V, device=dev), torch.empty(T, V, dtype=bf, device=dev), torch.tensor([0.3, -0.2], device=dev)
        ours = timed(lambda: native.check_seq(seq.ktb200_softcap(zz.data_ptr(), of.data_ptr(), zz.numel(), 30.0, 30, S())), flush)
        ms = timed(lambda: native.check_seq(seq.ktb200_xielu(zz.data_ptr(), oo.data_ptr(), pq.data_ptr(), zz.numel(), 30, S())), flush)
        row("softcap_kernel (bf16 in, fp32 out)", f"T={T} vocab={V}", ours, nbytes=T * V * 6, peer=peer_of("xielu_kernel", ms, T * V * 4))
    return rows


def run_bilurax(args):
    torch.cuda.set_device(0)
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    try:
        m = json.load(open(os.path.join(root, "MEASURED_PEAKS.json")))
        peak, tf, src = float(m["hbm_gbs"]), float(m["bf16_tflops"]), "measured (MEASURED_PEAKS.json hbm_gbs, bf16_tflops)"
    except Exception:
        peak, tf, src = 6650.0, 1590.0, "fallback"
    flush = Flusher("cuda")
    n0 = native.seq_lib().ktb200_launch_count()
    out = {"bench": "bilurax", "dtype": "bf16", "data": "synthetic (random weights and tokens)", "hbm_peak_GBps": peak, "bf16_peak_TFLOPs": tf, "peak_source": src,
           "timing": "CUDA events, median, 256 MB L2 flush between timed calls", "kernels": [] if getattr(args, "no_kernels", False) else bilurax_kernel_leg(flush, peak, tf),
           "models": [], "closest_models": []}
    for name in (args.sizes.split(",") if getattr(args, "sizes", None) else BILURAX_SIZES):
        out["models"].append(engine_leg(name, BILURAX_SIZES[name], flush, args.steps, args.warmup, family="bilurax"))
        torch.cuda.empty_cache()
        out["closest_models"].append(engine_leg(name, BILURAX_SIZES[name], flush, args.steps, args.warmup, family="mabidra-attn"))      # Mabidra at the same sizes, in the same process
        torch.cuda.empty_cache()
    out["gpu_launches"] = int(native.seq_lib().ktb200_launch_count() - n0)
    print(json.dumps(out))


def run_zivulix(args):
    torch.cuda.set_device(0)
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    try:
        m = json.load(open(os.path.join(root, "MEASURED_PEAKS.json")))
        peak, tf, src = float(m["hbm_gbs"]), float(m["bf16_tflops"]), "measured (MEASURED_PEAKS.json hbm_gbs, bf16_tflops)"
    except Exception:
        peak, tf, src = 6650.0, 1590.0, "fallback"
    flush = Flusher("cuda")
    n0 = native.seq_lib().ktb200_launch_count()
    out = {"bench": "zivulix", "dtype": "bf16", "data": "synthetic (random weights and tokens)", "hbm_peak_GBps": peak, "bf16_peak_TFLOPs": tf, "peak_source": src,
           "timing": "CUDA events, median, 256 MB L2 flush between timed calls", "kernels": [] if getattr(args, "no_kernels", False) else zivulix_kernel_leg(flush, peak, tf),
           "models": [], "closest_models": []}
    for name in (args.sizes.split(",") if getattr(args, "sizes", None) else ZIVULIX_SIZES):
        out["models"].append(engine_leg(name, ZIVULIX_SIZES[name], flush, args.steps, args.warmup, family="zivulix"))
        torch.cuda.empty_cache()
        out["closest_models"].append(engine_leg(name, ZIVULIX_SIZES[name], flush, args.steps, args.warmup, family="mabidra-dense"))      # Mabidra at the same sizes, in the same process
        torch.cuda.empty_cache()
    out["gpu_launches"] = int(native.seq_lib().ktb200_launch_count() - n0)
    print(json.dumps(out))


def run(args):
    """`bench.py --model lekapel | mabidra | zivulix | bilurax`: prints one JSON line."""
    if args.model == "mabidra":
        return run_mabidra(args)
    if args.model == "zivulix":
        return run_zivulix(args)
    if args.model == "bilurax":
        return run_bilurax(args)
    torch.cuda.set_device(0)
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    try:
        peak, src = float(json.load(open(os.path.join(root, "MEASURED_PEAKS.json")))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    except Exception:
        peak, src = 6650.0, "fallback"
    flush = Flusher("cuda")
    have_main = os.path.exists(native.LIB_PATH)
    n0 = native.seq_lib().ktb200_launch_count()
    out = {"bench": "lekapel", "dtype": "bf16", "data": "synthetic (random weights and tokens)", "hbm_peak_GBps": peak, "peak_source": src,
           "timing": "CUDA events, median, 256 MB L2 flush between timed calls", "kernels": kernel_leg(flush, peak, have_main), "models": []}
    for name in (args.sizes.split(",") if getattr(args, "sizes", None) else SIZES):
        out["models"].append(engine_leg(name, SIZES[name], flush, args.steps, args.warmup))
        torch.cuda.empty_cache()
    out["gpu_launches"] = int(native.seq_lib().ktb200_launch_count() - n0)
    print(json.dumps(out))


def run_mabidra(args):
    torch.cuda.set_device(0)
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    try:
        m = json.load(open(os.path.join(root, "MEASURED_PEAKS.json")))
        peak, tf, src = float(m["hbm_gbs"]), float(m["bf16_tflops"]), "measured (MEASURED_PEAKS.json hbm_gbs, bf16_tflops)"
    except Exception:
        peak, tf, src = 6650.0, 1590.0, "fallback"
    flush = Flusher("cuda")
    n0 = native.seq_lib().ktb200_launch_count()
    out = {"bench": "mabidra", "dtype": "bf16", "data": "synthetic (random weights and tokens)", "hbm_peak_GBps": peak, "bf16_peak_TFLOPs": tf, "peak_source": src,
           "timing": "CUDA events, median, 256 MB L2 flush between timed calls", "kernels": [] if getattr(args, "no_kernels", False) else mabidra_kernel_leg(flush, peak, tf),
           "models": [], "closest_models": []}
    for name in (args.sizes.split(",") if getattr(args, "sizes", None) else MABIDRA_SIZES):
        out["models"].append(engine_leg(name, MABIDRA_SIZES[name], flush, args.steps, args.warmup, family="mabidra"))
        torch.cuda.empty_cache()
        out["closest_models"].append(engine_leg(name, SIZES[name], flush, args.steps, args.warmup))      # Lekapel at the same widths, in the same process
        torch.cuda.empty_cache()
    out["gpu_launches"] = int(native.seq_lib().ktb200_launch_count() - n0)
    print(json.dumps(out))
