"""Small random Bilurax checkpoints for the tests: a config dict, a tensor dict in the checkpoint's naming, and a writer."""
import json
import os

import torch


def attn(heads=4, kv_heads=2, dim=6, vdim=5, scale=None, softcap=8.0, chunk=7):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5}
    if softcap is not None:
        m["softcap"] = softcap
    m["mask"] = {"size": chunk}
    return {"type": "attention", "mixer": m}


def dense(ff=40):
    return {"kind": "dense", "ff": ff}


def moe(ff=10, experts=6, top=2, groups=3, keep=2, scale=1.7, limit=0.8):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top, "groups": {"count": groups, "keep": keep}, "scale": scale}}


def config(layers, vocab=50, width=24, eps=1e-5, loop=None, embed_scale=3.0, logit_softcap=9.0):
    """layers: [(mixer description from attn(), feed-forward from dense() / moe() or None)]; loop: (start, stop, times) or None"""
    c = {"architecture": "Bilurax", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": embed_scale}, "logit_softcap": logit_softcap,
         "layers": [{"type": m["type"], "mixer": m["mixer"], "mlp": f} for m, f in layers]}
    if loop is not None:
        c["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return c


def weights(cfg, seed=0, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    D = cfg["width"]
    rn = lambda *s, k=1.0: torch.randn(*s, generator=g) * k
    lin = lambda o, i, s=1.0: rn(o, i, k=s / i ** 0.5)
    nw = lambda n: 1.0 + 0.3 * rn(n)
    w = {"embed": rn(cfg["vocab"], D, k=0.5), "final.norm": nw(D)}
    if cfg.get("loop"):
        w["loop.step"] = rn(cfg["loop"]["times"], D, k=0.5)
    for i, l in enumerate(cfg["layers"]):
        m, p = l["mixer"], f"l{i}."
        H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        w[p + "norm1"], w[p + "shift"] = nw(D), torch.rand(D, generator=g)
        w[p + "mix.q"], w[p + "mix.k"], w[p + "mix.v"], w[p + "mix.o"] = lin(H * d, D, 2.0), lin(G * d, D, 2.0), lin(G * dv, D), lin(D, H * dv)
        w[p + "mix.q.b"], w[p + "mix.k.b"], w[p + "mix.v.b"], w[p + "mix.o.b"] = rn(H * d, k=0.3), rn(G * d, k=0.3), rn(G * dv, k=0.3), rn(D, k=0.1)
        w[p + "mix.q.norm"], w[p + "mix.k.norm"] = nw(H * d) * 1.5, nw(G * d) * 1.5
        w[p + "mix.temp"] = 0.5 + 1.5 * torch.rand(H, generator=g)
        f = l["mlp"]
        if f is None:
            continue
        w[p + "norm2"] = nw(D)
        if f["kind"] == "dense":
            w[p + "mlp.up"], w[p + "mlp.down"] = lin(f["ff"], D, 1.5), lin(D, f["ff"])
        else:
            E, ff = f["router"]["experts"], f["expert"]["ff"]
            w[p + "mlp.router"] = lin(E, D, 3.0)
            w[p + "mlp.correction"] = rn(E, k=0.6) - 0.7            # choice scores fall on both sides of zero
            for e in range(E):
                w[p + f"mlp.e{e}.gate"], w[p + f"mlp.e{e}.up"], w[p + f"mlp.e{e}.down"] = lin(ff, D, 2.0), lin(ff, D, 2.0), lin(D, ff)
    return {k: v.to(dtype).contiguous() for k, v in w.items()}


def save(path, cfg, w):
    from safetensors.torch import save_file
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file(w, os.path.join(path, "model.safetensors"))
    return str(path)
