"""Small random Zivulix checkpoints for the tests: a config dict, a tensor dict in the checkpoint's naming, and a writer."""
import json
import os

import torch


def attn(heads=4, kv_heads=2, dim=12, vdim=10, scale=None, softcap=5.0, window=9, rot_dims=8, base=100.0, factor=2.0, v_mix=False):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5, "v_mix": v_mix}
    if softcap is not None:
        m["softcap"] = softcap
    if window is not None:
        m["mask"] = {"size": window}
    if rot_dims:
        m["rot"] = {"base": base, "dims": rot_dims}
        if factor is not None:
            m["rot"]["scaling"] = {"factor": factor}
    return {"type": "attention", "mixer": m}


def latent(heads=3, dim=6, rot_dim=4, vdim=5, kv_rank=10, scale=None, base=50.0):
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
                                                  "scale": scale if scale is not None else (dim + rot_dim) ** -0.5, "rot": {"base": base, "dims": rot_dim}}}


def delta(heads=4, kv_heads=2, dim=6, vdim=5, conv=3):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}}


def dense(ff=40):
    return {"kind": "dense", "ff": ff}


def config(layers, vocab=50, width=24, eps=1e-5):
    """layers: [(mixer description from attn() / latent() / delta(), feed-forward or None)]"""
    return {"architecture": "Zivulix", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "layers": [{"type": m["type"], "mixer": m["mixer"], "mlp": f} for m, f in layers]}


def weights(cfg, seed=0, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    D = cfg["width"]
    rn = lambda *s, k=1.0: torch.randn(*s, generator=g) * k
    lin = lambda o, i, s=1.0: rn(o, i, k=s / i ** 0.5)
    nw = lambda n: 0.3 * rn(n)                                   # norm weights are zero-centred
    w = {"embed": rn(cfg["vocab"], D), "embed.norm": nw(D), "final.norm": nw(D), "head": lin(cfg["vocab"], D)}
    for i, l in enumerate(cfg["layers"]):
        m, p = l["mixer"], f"l{i}."
        w[p + "norm1"] = nw(D)
        if l["type"] == "attention":
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            w[p + "mix.q"], w[p + "mix.k"], w[p + "mix.v"], w[p + "mix.o"] = lin(H * d, D, 2.0), lin(G * d, D, 2.0), lin(G * dv, D), lin(D, H * dv)
            w[p + "mix.q.b"], w[p + "mix.k.b"], w[p + "mix.v.b"] = rn(H * d, k=0.3), rn(G * d, k=0.3), rn(G * dv, k=0.3)
            w[p + "mix.vmix"] = torch.tensor(0.35) + 0.1 * rn(1)[0]
        elif l["type"] == "latent_attention":
            H, d, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            w[p + "mix.q"], w[p + "mix.dkv"], w[p + "mix.dkv.norm"] = lin(H * (d + dr), D, 2.0), lin(R + dr, D, 2.0), 1 + 0.2 * rn(R)
            w[p + "mix.uk"], w[p + "mix.uv"], w[p + "mix.o"] = lin(H * d, R, 1.5), lin(H * dv, R), lin(D, H * dv)
        else:
            H, G, d, dv, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            w[p + "mix.q"], w[p + "mix.k"], w[p + "mix.v"], w[p + "mix.g"], w[p + "mix.o"] = lin(G * d, D, 2.0), lin(G * d, D, 2.0), lin(H * dv, D, 2.0), lin(H * dv, D, 2.0), lin(D, H * dv)
            w[p + "mix.q.conv"], w[p + "mix.k.conv"], w[p + "mix.v.conv"] = rn(G * d, taps, k=0.6), rn(G * d, taps, k=0.6), rn(H * dv, taps, k=0.6)
            w[p + "mix.b"], w[p + "mix.a"] = lin(H, D, 2.0), lin(H, D, 2.0)
            w[p + "mix.A_log"], w[p + "mix.dt_bias"], w[p + "mix.norm"] = rn(H, k=0.5) - 1.0, rn(H, k=0.5), 1 + 0.2 * rn(dv)
        f = l["mlp"]
        if f is not None:
            w[p + "norm2"] = nw(D)
            w[p + "mlp.gate"], w[p + "mlp.up"], w[p + "mlp.down"] = lin(f["ff"], D, 1.5), lin(f["ff"], D, 1.5), lin(D, f["ff"])
    return {k: v.to(dtype).contiguous() for k, v in w.items()}


def save(path, cfg, w):
    from safetensors.torch import save_file
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file(w, os.path.join(path, "model.safetensors"))
    return str(path)
