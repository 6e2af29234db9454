"""TEST-ONLY plain restatement of the Zivulix decoder, one function per mechanism, float64 (or float32) torch on the CPU.

Nothing here is imported by the product path and nothing of the product path is imported here.  Every function works on one
sequence `[tokens, features]`; `Model.forward` runs a token range over explicit Python state (tensors of cached rows, one
state matrix per head, a short list of earlier convolution inputs), with no paging and no batching, token by token where a
recurrence is involved.

Notation: `T` tokens, `D` model width, `H` query heads, `G` key/value (or query/key) heads, `d` query/key size and `dv` value
size per head, `R` latent size, `dr` rotated size.
"""
from __future__ import annotations

import math

import torch

from .lekapel_oracle import read_safetensors  # noqa: F401  (the same file format)


def rms(x, eps):
    """x over its last axis divided by sqrt(mean(x^2) + eps)"""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def offset_rms_norm(x, w, eps):
    """zero-centred weight: the row is scaled by 1 + w"""
    return rms(x, eps) * (1.0 + w)


def unit_vector(x, eps=1e-6):
    """x over its last axis scaled to length one: x * rsqrt(|x|^2 + eps)"""
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def rotate_halves(x, pos, base, dims, factor=1.0):
    """x [T, heads, n]: of each head's first `dims` columns, column i < dims / 2 pairs with column i + dims / 2; the pair turns
    by the angle pos * base^(-2 i / dims) / factor.  Columns from `dims` on pass unchanged."""
    half = dims // 2
    out = x.clone()
    for t in range(x.shape[0]):
        for i in range(half):
            a = float(pos[t]) * (float(base) ** (-2.0 * i / dims)) / factor
            c, s = math.cos(a), math.sin(a)
            u, v = x[t, :, i], x[t, :, i + half]
            out[t, :, i] = u * c - v * s
            out[t, :, i + half] = v * c + u * s
    return out


def softmax_attention(q, k, v, qpos, kpos, scale, window=None, softcap=None):
    """q [T, H, d], k [N, G, d], v [N, G, dv].  Query i sees key j when 0 <= qpos_i - kpos_j (< window, if one is given);
    score = scale q.k, squashed to c tanh(score / c) if a cap c is given; soft-max over the seen keys."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[-1], dtype=q.dtype)
    n = qpos[:, None] - kpos[None, :]
    seen = n >= 0
    if window is not None:
        seen = seen & (n < window)
    for h in range(H):
        g = h // (H // G)
        s = q[:, h] @ k[:, g].T * scale
        if softcap is not None:
            s = softcap * torch.tanh(s / softcap)
        s = s.masked_fill(~seen, float("-inf"))
        out[:, h] = torch.softmax(s, -1) @ v[:, g]
    return out


def softmax_attention_slow(q, k, v, qpos, kpos, scale, window=None, softcap=None):
    """the same sums key by key (checks the matrix form above)"""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[-1], dtype=q.dtype)
    for i in range(T):
        for h in range(H):
            g = h // (H // G)
            scores, rows = [], []
            for j in range(k.shape[0]):
                n = int(qpos[i]) - int(kpos[j])
                if n < 0 or (window is not None and n >= window):
                    continue
                s = float((q[i, h] * k[j, g]).sum()) * scale
                if softcap is not None:
                    s = softcap * math.tanh(s / softcap)
                scores.append(s)
                rows.append(j)
            m = max(scores)
            e = [math.exp(s - m) for s in scores]
            for w, j in zip(e, rows):
                out[i, h] += w / sum(e) * v[j, g]
    return out


def capped_window_mixer(h, pos, past, W, m, eps, v_first=None):
    """Grouped-head attention with biased projections, a partial rotation with stretched wavelengths, unit-rms queries and
    keys, capped scores, a sliding window and values blended with an earlier layer's.
    h [T, D] -> ([T, D], new past, this layer's values before the blend).  past = (keys, values, positions)."""
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    rot = m.get("rot") or {}
    q = (h @ W["q"].T + W["q.b"]).reshape(T, H, d)
    k = (h @ W["k"].T + W["k.b"]).reshape(T, G, d)
    v = (h @ W["v"].T + W["v.b"]).reshape(T, G, dv)
    if rot.get("dims"):
        factor = float((rot.get("scaling") or {}).get("factor", 1.0))
        q = rotate_halves(q, pos, rot["base"], rot["dims"], factor)
        k = rotate_halves(k, pos, rot["base"], rot["dims"], factor)
    q, k = rms(q, eps), rms(k, eps)
    v_own = v
    if v_first is not None:
        lam = W["vmix"]
        v = (1.0 - lam) * v + lam * v_first
    keys, values, kpos = torch.cat([past[0], k]), torch.cat([past[1], v]), torch.cat([past[2], pos])
    window = (m.get("mask") or {}).get("size")
    o = softmax_attention(q, keys, values, pos, kpos, m["scale"], window, m.get("softcap"))
    return o.reshape(T, H * dv) @ W["o"].T, (keys, values, kpos), v_own


def latent_mixer(h, pos, past, W, m, eps):
    """Attention whose keys and values are up-projections of one normed latent per token, plus one rotated key part that all
    heads share.  h [T, D] -> ([T, D], new past).  past = (latents [N, R], rotated key parts [N, dr], positions)."""
    H, d, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    T = h.shape[0]
    q = (h @ W["q"].T).reshape(T, H, d + dr)
    low = h @ W["dkv"].T
    c = rms(low[:, :R], eps) * W["dkv.norm"]
    kr = low[:, R:].reshape(T, 1, dr)
    rot = m["rot"]
    q_rot = rotate_halves(q[:, :, d:], pos, rot["base"], rot["dims"])
    kr = rotate_halves(kr, pos, rot["base"], rot["dims"]).reshape(T, dr)
    lat, krs, kpos = torch.cat([past[0], c]), torch.cat([past[1], kr]), torch.cat([past[2], pos])
    N = lat.shape[0]
    k_plain = (lat @ W["uk"].T).reshape(N, H, d)
    val = (lat @ W["uv"].T).reshape(N, H, dv)
    keys = torch.cat([k_plain, krs[:, None, :].expand(N, H, dr)], -1)
    o = softmax_attention(torch.cat([q[:, :, :d], q_rot], -1), keys, val, pos, kpos, m["scale"])
    return o.reshape(T, H * dv) @ W["o"].T, (lat, krs, kpos)


def short_conv(x, w, before):
    """x [T, C], w [C, taps] (last column weighs the current token), before [taps - 1, C] the inputs ahead of row 0 (zeros at a
    sequence's start).  Returns (y [T, C], the last taps - 1 inputs)."""
    taps = w.shape[1]
    full = torch.cat([before, x])
    y = torch.zeros_like(x)
    for t in range(x.shape[0]):
        for j in range(taps):
            y[t] += w[:, j] * full[t + j]
    return y, full[full.shape[0] - (taps - 1):]


def delta_recurrence(q, k, v, beta, g, S):
    """q, k [T, H, d], v [T, H, dv], beta, g [T, H], S [H, d, dv].  Per token: S decays by g, the value that S holds under k
    is moved toward v by the step beta, and the read-out under q sees that write."""
    out = []
    for t in range(q.shape[0]):
        S = g[t][:, None, None] * S
        held = (S * k[t][:, :, None]).sum(1)
        u = beta[t][:, None] * (v[t] - held)
        S = S + k[t][:, :, None] * u[:, None, :]
        out.append((S * q[t][:, :, None]).sum(1))
    return torch.stack(out), S


def delta_mixer(h, state, W, m, eps):
    """h [T, D] -> ([T, D], new state).  state = (S [H, d, dv], earlier conv inputs of q, of k, of v)."""
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    S, bq, bk, bv = state
    q, bq = short_conv(h @ W["q"].T, W["q.conv"], bq)
    k, bk = short_conv(h @ W["k"].T, W["k.conv"], bk)
    v, bv = short_conv(h @ W["v"].T, W["v.conv"], bv)
    q = unit_vector(silu(q).reshape(T, G, d)) * d ** -0.5
    k = unit_vector(silu(k).reshape(T, G, d))
    v = silu(v).reshape(T, H, dv)
    rep = H // G
    q, k = q.repeat_interleave(rep, 1), k.repeat_interleave(rep, 1)
    beta = torch.sigmoid(h @ W["b"].T)
    g = torch.exp(-torch.exp(W["A_log"]) * torch.nn.functional.softplus(h @ W["a"].T + W["dt_bias"]))
    o, S = delta_recurrence(q, k, v, beta, g, S)
    o = rms(o, eps) * W["norm"] * silu(h @ W["g"].T).reshape(T, H, dv)
    return o.reshape(T, H * dv) @ W["o"].T, (S, bq, bk, bv)


def gated_gelu_mlp(h, gate, up, down):
    return (gelu_tanh(h @ gate.T) * (h @ up.T)) @ down.T


class Model:
    def __init__(self, config, tensors, dtype=torch.float64):
        self.c, self.dtype = config, dtype
        self.W = {k: v.to(dtype) for k, v in tensors.items()}
        mixing = [i for i, l in enumerate(config["layers"]) if l["type"] == "attention" and l["mixer"].get("v_mix")]
        self.first_mixing = mixing[0] if mixing else None

    def sub(self, prefix):
        return {k[len(prefix):]: v for k, v in self.W.items() if k.startswith(prefix)}

    def new_state(self):
        st = {"pos": 0, "layers": []}
        z = lambda *s: torch.zeros(*s, dtype=self.dtype)
        for l in self.c["layers"]:
            m = l["mixer"]
            if l["type"] == "attention":
                st["layers"].append((z(0, m["kv_heads"], m["dim"]), z(0, m["kv_heads"], m["vdim"]), torch.zeros(0, dtype=torch.long)))
            elif l["type"] == "latent_attention":
                st["layers"].append((z(0, m["kv_rank"]), z(0, m["rot_dim"]), torch.zeros(0, dtype=torch.long)))
            else:
                n = m["conv"] - 1
                st["layers"].append((z(m["heads"], m["dim"], m["vdim"]), z(n, m["kv_heads"] * m["dim"]), z(n, m["kv_heads"] * m["dim"]), z(n, m["heads"] * m["vdim"])))
        return st

    def forward(self, tokens, state, trace=None):
        """logits [len(tokens), vocab] of the next tokens of ONE sequence; `state` is advanced"""
        c, W = self.c, self.W
        eps = c["norm"]["eps"]
        pos = torch.arange(state["pos"], state["pos"] + len(tokens))
        x = offset_rms_norm(W["embed"][torch.tensor(tokens)], W["embed.norm"], eps)
        v_first = None
        for i, l in enumerate(c["layers"]):
            p, m = f"l{i}.", l["mixer"]
            if l["type"] == "attention":
                blend = v_first if (m.get("v_mix") and i != self.first_mixing) else None
                y, state["layers"][i], v_own = capped_window_mixer(x, pos, state["layers"][i], self.sub(p + "mix."), m, eps, blend)
                if i == self.first_mixing:
                    v_first = v_own
            elif l["type"] == "latent_attention":
                y, state["layers"][i] = latent_mixer(x, pos, state["layers"][i], self.sub(p + "mix."), m, eps)
            else:
                y, state["layers"][i] = delta_mixer(x, state["layers"][i], self.sub(p + "mix."), m, eps)
            x = x + offset_rms_norm(y, W[p + "norm1"], eps)
            if l["mlp"] is not None:
                y = gated_gelu_mlp(x, W[p + "mlp.gate"], W[p + "mlp.up"], W[p + "mlp.down"])
                x = x + offset_rms_norm(y, W[p + "norm2"], eps)
            if trace is not None:
                trace.append(x.clone())
        state["pos"] += len(tokens)
        return offset_rms_norm(x, W["final.norm"], eps) @ W["head"].T
