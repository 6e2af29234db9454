"""TEST-ONLY plain restatement of the Bilurax decoder, one function per mechanism, float64 (or float32) torch on the CPU.

Nothing here is imported by the product path and nothing of the product path is imported here.  Every function works on one
sequence `[tokens, features]`; `Model.forward` runs a token range over explicit Python state (per layer run: the previous
token's mixer input and the tensors of cached key and value rows), with no paging and no batching.

Notation: `T` tokens, `D` model width, `H` query heads, `G` key/value heads, `d` query/key size and `dv` value size per head,
`C` the chunk length of the attention mask, `E` experts, `n` the experts a token uses.
"""
from __future__ import annotations

import math

import torch

from .lekapel_oracle import read_safetensors  # noqa: F401  (the same file format)


def rms(x, eps):
    """x over its last axis divided by sqrt(mean(x^2) + eps)"""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, w, eps):
    return rms(x, eps) * w


def token_shift(h, prev, mu):
    """Row t becomes h_t + (h_{t-1} - h_t) * mu with the un-shifted rows on the right-hand side; `prev` stands before row 0
    (zeros at the start of a sequence).  Returns (shifted rows, the last un-shifted row)."""
    before = torch.cat([prev.reshape(1, -1), h[:-1]], 0)
    return h + (before - h) * mu, h[-1].clone()


def chunk_softmax_attention(q, k, v, qpos, kpos, scale, temp, softcap, chunk):
    """q [T, H, d], k [N, G, d], v [N, G, dv].  Query at position i sees the key at position j when j <= i and both lie in the
    same chunk, floor(i / C) == floor(j / C).  score = scale * temp_h * q.k, squashed to c tanh(score / c) when a cap c is given;
    soft-max over the seen keys.  One query, head and key at a time."""
    T, H, _ = q.shape
    G, dv = k.shape[1], v.shape[2]
    out = torch.zeros(T, H, dv, dtype=q.dtype)
    for t in range(T):
        i = int(qpos[t])
        seen = [n for n in range(k.shape[0]) if int(kpos[n]) <= i and int(kpos[n]) // chunk == i // chunk]
        for h in range(H):
            g = h // (H // G)
            s = torch.stack([(q[t, h] * k[n, g]).sum() for n in seen]) * scale * temp[h]
            if softcap is not None:
                s = softcap * torch.tanh(s / softcap)
            p = torch.exp(s - s.max())
            p = p / p.sum()
            out[t, h] = sum(p[a] * v[n, g] for a, n in enumerate(seen))
    return out


def attention_mixer(h, pos, cache, W, m, eps):
    """h [T, D] (already token-shifted); cache = (K [N, G, d], V [N, G, dv], positions [N]) of the earlier tokens.
    Queries and keys are normed over the WHOLE projection (all heads at once, a weight per column); each head's value is scaled
    to unit rms (no weight) before it is cached; no position enters the scores."""
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = rms_norm(h @ W["q"].T + W["q.b"], W["q.norm"], eps).reshape(T, H, d)
    k = rms_norm(h @ W["k"].T + W["k.b"], W["k.norm"], eps).reshape(T, G, d)
    v = rms((h @ W["v"].T + W["v.b"]).reshape(T, G, dv), eps)
    K, V, P = torch.cat([cache[0], k]), torch.cat([cache[1], v]), torch.cat([cache[2], pos])
    o = chunk_softmax_attention(q, K, V, pos, P, m["scale"], W["temp"], m.get("softcap"), m["mask"]["size"])
    return o.reshape(T, H * dv) @ W["o"].T + W["o.b"], (K, V, P)


def relu2_mlp(h, up, down):
    return torch.relu(h @ up.T).square() @ down.T


def grouped_sigmoid_router(h, router, correction, top, n_groups, keep, out_scale):
    """(ids [T, n], weights [T, n]).  s = sigmoid(W h); experts are CHOSEN by s + correction, restricted to the `keep` groups
    (of E / n_groups neighbouring experts) whose two largest choice scores sum highest; their WEIGHTS are s without the
    correction, divided by their sum and multiplied by out_scale."""
    T, E = h.shape[0], router.shape[0]
    s = torch.sigmoid(h @ router.T)
    ids = torch.zeros(T, top, dtype=torch.long)
    wts = torch.zeros(T, top, dtype=h.dtype)
    size = E // n_groups
    for t in range(T):
        choice = [float(s[t, e] + correction[e]) for e in range(E)]
        gscore = [sum(sorted(choice[g * size:(g + 1) * size], reverse=True)[:2]) for g in range(n_groups)]
        kept = sorted(range(n_groups), key=lambda g: (-gscore[g], g))[:keep]
        allowed = [e for e in range(E) if e // size in kept]
        best = sorted(allowed, key=lambda e: (-choice[e], e))[:top]
        ids[t] = torch.tensor(best)
        wts[t] = s[t, best] / (s[t, best].sum() + 1e-20) * out_scale
    return ids, wts


def clamped_glu_expert(x, gate, up, down, limit):
    """g = min(W_gate x, limit), u = clamp(W_up x, -limit, limit);  W_down (g sigmoid(1.702 g) (u + 1))"""
    g = (gate @ x).clamp(max=limit)
    u = (up @ x).clamp(-limit, limit)
    return down @ (g * torch.sigmoid(1.702 * g) * (u + 1.0))


def moe_mlp(h, W, f):
    r = f["router"]
    ids, wts = grouped_sigmoid_router(h, W["router"], W["correction"], r["top"], r["groups"]["count"], r["groups"]["keep"], r["scale"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(r["top"]):
            e = int(ids[t, j])
            out[t] += wts[t, j] * clamped_glu_expert(h[t], W[f"e{e}.gate"], W[f"e{e}.up"], W[f"e{e}.down"], f["expert"]["limit"])
    return out


def layer_runs(config):
    """[(layer, pass that this run opens or None)]: layers start .. stop - 1 run `times` times in a row"""
    n, lp = len(config["layers"]), config.get("loop")
    if lp is None:
        return [(i, None) for i in range(n)]
    runs = [(i, None) for i in range(lp["start"])]
    for t in range(lp["times"]):
        runs += [(i, t if i == lp["start"] else None) for i in range(lp["start"], lp["stop"])]
    return runs + [(i, None) for i in range(lp["stop"], n)]


class Model:
    def __init__(self, config, tensors, dtype=torch.float64):
        self.c, self.dtype = config, dtype
        self.W = {k: v.to(dtype) for k, v in tensors.items()}
        self.runs = layer_runs(config)

    def sub(self, prefix):
        return {k[len(prefix):]: v for k, v in self.W.items() if k.startswith(prefix)}

    def new_state(self):
        st = {"pos": 0, "runs": []}
        for i, _ in self.runs:
            m = self.c["layers"][i]["mixer"]
            st["runs"].append({"prev": torch.zeros(self.c["width"], dtype=self.dtype),
                               "kv": (torch.zeros(0, m["kv_heads"], m["dim"], dtype=self.dtype), torch.zeros(0, m["kv_heads"], m["vdim"], dtype=self.dtype),
                                      torch.zeros(0, dtype=torch.long))})
        return st

    def forward(self, tokens, state, trace=None):
        """logits [len(tokens), vocab] of the next tokens of ONE sequence; `state` is advanced"""
        c, W = self.c, self.W
        eps = c["norm"]["eps"]
        pos = torch.arange(state["pos"], state["pos"] + len(tokens))
        x0 = W["embed"][torch.tensor(tokens)] * c["embedding"]["scale"]
        x = x0
        for r, (i, opens) in enumerate(self.runs):
            if opens is not None:
                if opens > 0:
                    x = x + x0
                x = x + W["loop.step"][opens]
            l, p, st = c["layers"][i], f"l{i}.", state["runs"][r]
            h, st["prev"] = token_shift(rms_norm(x, W[p + "norm1"], eps), st["prev"], W[p + "shift"])
            y, st["kv"] = attention_mixer(h, pos, st["kv"], self.sub(p + "mix."), l["mixer"], eps)
            x = x + y
            f = l["mlp"]
            if f is not None:
                h = rms_norm(x, W[p + "norm2"], eps)
                x = x + (relu2_mlp(h, W[p + "mlp.up"], W[p + "mlp.down"]) if f["kind"] == "dense" else moe_mlp(h, self.sub(p + "mlp."), f))
            if trace is not None:
                trace.append(x.clone())
        state["pos"] += len(tokens)
        z = rms_norm(x, W["final.norm"], eps) @ W["embed"].T
        cap = c.get("logit_softcap")
        return z if cap is None else cap * torch.tanh(z / cap)
