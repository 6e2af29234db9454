"""Zivulix through the framework (registry, loader, paged state cache, scheduler, engine, CUDA operators) against the plain
restatement in oracle/zivulix_oracle.py, on small random checkpoints made here.  CPU tests cover the host logic."""
import json
import math
import random

import pytest
import torch

import zivulix_util as U
from oracle import zivulix_oracle as O

gpu = pytest.mark.gpu
F32_TOL, BF16_TOL = 3e-4, 6e-2


def rel(a, b):
    a, b = a.detach().double().cpu(), b.detach().double().cpu()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))


def rel_rows(a, b, q=0.8):
    """the q-quantile of the per-row errors, for bf16 runs of whole models"""
    a, b = a.detach().double().cpu(), b.detach().double().cpu()
    return float(((a - b).abs().amax(-1) / b.abs().max()).quantile(q))


class DictLoader:
    def __init__(self, w):
        self.w = w

    def load_tensor(self, key, device="cpu"):
        return self.w[key].to(device)


MIXED = [(U.attn(v_mix=True), U.dense()), (U.delta(), None), (U.latent(), U.dense(16)), (U.attn(heads=6, kv_heads=2, dim=12, vdim=10, window=5, rot_dims=12, factor=None, v_mix=True), None),
         (U.delta(heads=2, kv_heads=2, dim=17, vdim=33, conv=4), U.dense(8)), (U.attn(heads=2, kv_heads=1, dim=6, vdim=3, softcap=None, window=None, rot_dims=0), None)]


def serve(tmp_path, cfg, dtype, seed=0, **engine_kw):
    from ktransformers_b200.models import load_model
    from ktransformers_b200.util.engine import Engine
    w = U.weights(cfg, seed, torch.bfloat16 if dtype == "bfloat16" else torch.float32)
    path = U.save(tmp_path / f"ckpt{seed}", cfg, w)
    torch.backends.cuda.matmul.allow_tf32 = False
    model = load_model(path, dtype)
    return Engine(model, **engine_kw), O.Model(cfg, w, torch.float64)


def oracle_logits(om, tokens):
    return om.forward(tokens, om.new_state()).float()


def run_steps(eng, steps):
    """steps: list of lists of (id, tokens, last); every position's logits are asked for; returns {id: [n, V]}"""
    out = {}
    for step in steps:
        lg = eng.step([(i, t, list(range(len(t)))) for i, t, _ in step], [i for i, _, last in step if last]).cpu()
        k = 0
        for i, t, _ in step:
            out.setdefault(i, []).append(lg[k:k + len(t)])
            k += len(t)
    return {i: torch.cat(v) for i, v in out.items()}


def cut(seq_id, tokens, sizes):
    """portions of the given sizes (repeating the last) as single-entry steps"""
    steps, at, k = [], 0, 0
    while at < len(tokens):
        n = min(sizes[min(k, len(sizes) - 1)], len(tokens) - at)
        steps.append([(seq_id, tokens[at:at + n], at + n == len(tokens))])
        at, k = at + n, k + 1
    return steps


def toks(n, vocab=50, seed=0):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


# ------------------------------------------------------------------------------------------------ host logic (CPU)
def test_config_reads_sizes_and_constants_per_layer():
    from ktransformers_b200.models.configuration_zivulix import ZivulixConfig
    c = ZivulixConfig.from_dict(U.config(MIXED, vocab=77, width=36, eps=1e-3))
    assert (c.vocab, c.width, c.norm_eps, len(c.layers)) == (77, 36, 1e-3, 6)
    a0, a3, a5 = c.layers[0].mixer, c.layers[3].mixer, c.layers[5].mixer
    assert (a0.heads, a0.kv_heads, a0.dim, a0.vdim, a0.window, a0.softcap, a0.v_mix) == (4, 2, 12, 10, 9, 5.0, True)
    assert (a0.rot.dims, a0.rot.base, a0.rot.factor, a0.rot.layout) == (8, 100.0, 2.0, "halves") and a3.rot.factor == 1.0 and a3.rot.dims == 12 and a3.window == 5
    assert a5.rot is None and a5.window is None and a5.softcap is None and not a5.v_mix
    l2 = c.layers[2].mixer
    assert (l2.q_rank, l2.kv_rank, l2.rot_dim, l2.sink, l2.gate, l2.window, l2.rot.layout) == (0, 10, 4, False, False, None, "halves")
    d1, d4 = c.layers[1].mixer, c.layers[4].mixer
    assert (d1.heads, d1.kv_heads, d1.conv, d4.conv, d4.vdim) == (4, 2, 3, 4, 33) and c.layers[1].mlp is None and c.layers[4].mlp.ff == 8
    assert c.cache_row_widths() == [2 * 22, 0, 14, 2 * 22, 0, 9]
    assert c.state_widths() == [0, 4 * 6 * 5 + 2 * (2 * 2 * 6 + 4 * 5), 0, 0, 2 * 17 * 33 + 3 * (2 * 2 * 17 + 2 * 33), 0]
    assert c.max_window() is None and c.first_value_mixer() == 0              # the latent layer and the last layer see everything
    windowed = ZivulixConfig.from_dict(U.config([(U.delta(), None), (U.attn(window=7), None), (U.attn(window=30, v_mix=True), U.dense())]))
    assert windowed.max_window() == 30 and windowed.first_value_mixer() == 2
    f = windowed.layers[1].mixer.rot.inv_freq("cpu")
    assert f.dtype == torch.float64 and f.tolist() == pytest.approx([100.0 ** (-2 * i / 8) / 2.0 for i in range(4)], rel=1e-15)
    with pytest.raises(ValueError):
        ZivulixConfig.from_dict(U.config([({"type": "conv", "mixer": {}}, None)]))


def test_registry_picks_the_class_by_config():
    from ktransformers_b200.models import architecture_of, model_class
    assert model_class(architecture_of({"architecture": "Zivulix"})).__name__ == "ZivulixForCausalLM"


def test_oracle_portions_equal_whole_prompt_and_both_attention_forms_agree():
    cfg = U.config(MIXED)
    om = O.Model(cfg, U.weights(cfg, 3, torch.float32), torch.float64)
    t = toks(19)
    whole = oracle_logits(om, t)
    st, parts = om.new_state(), []
    for lo, hi in ((0, 1), (1, 3), (3, 10), (10, 11), (11, 19)):
        parts.append(om.forward(t[lo:hi], st).float())
    assert rel(torch.cat(parts), whole) < 1e-6
    g = torch.Generator().manual_seed(0)
    q, k, v = torch.randn(5, 4, 3, generator=g).double() * 4, torch.randn(9, 2, 3, generator=g).double(), torch.randn(9, 2, 2, generator=g).double()
    for window, cap in ((None, None), (3, None), (4, 1.5), (1, 2.0)):
        args = (q, k, v, torch.arange(4, 9), torch.arange(9), 0.7, window, cap)
        assert rel(O.softmax_attention(*args), O.softmax_attention_slow(*args)) < 1e-12
    one = O.softmax_attention(q, k, v, torch.arange(4, 9), torch.arange(9), 0.7, 1, None)      # a window of one: every query reads its own value
    assert rel(one[:, 0], v[4:9, 0]) < 1e-12 and rel(one[:, 3], v[4:9, 1]) < 1e-12


def test_oracle_rotation_turns_pairs_of_halves():
    x = torch.randn(6, 2, 10, generator=torch.Generator().manual_seed(1)).double()
    pos = torch.tensor([0, 1, 2, 50, 51, 1000])
    r = O.rotate_halves(x, pos, 300.0, 6, 4.0)
    assert torch.equal(r[0], x[0]) and torch.equal(r[:, :, 6:], x[:, :, 6:])                       # position 0 and the columns beyond `dims` pass
    assert rel((r[:, :, :6] ** 2).sum(-1), (x[:, :, :6] ** 2).sum(-1)) < 1e-12
    a = 50 * 300.0 ** (-2 / 6) / 4.0                                                               # pair (1, 4) at position 50
    assert abs(float(r[3, 0, 1]) - float(x[3, 0, 1] * math.cos(a) - x[3, 0, 4] * math.sin(a))) < 1e-12
    assert abs(float(r[3, 0, 4]) - float(x[3, 0, 4] * math.cos(a) + x[3, 0, 1] * math.sin(a))) < 1e-12
    # scores depend on the distance only
    q, k = torch.randn(1, 1, 6, generator=torch.Generator().manual_seed(2)).double(), torch.randn(1, 1, 6, generator=torch.Generator().manual_seed(3)).double()
    s = lambda i, j: float((O.rotate_halves(q, [i], 300.0, 6) * O.rotate_halves(k, [j], 300.0, 6)).sum())
    assert abs(s(9, 4) - s(105, 100)) < 1e-9


def test_oracle_delta_recurrence_overwrites_the_value_under_a_key():
    """with g = 1 and beta = 1 the state holds exactly the newest value under a unit key, and a key orthogonal to it keeps its own"""
    k = torch.tensor([[[1.0, 0.0]], [[0.0, 1.0]], [[1.0, 0.0]]]).double()
    v = torch.tensor([[[3.0]], [[5.0]], [[7.0]]]).double()
    one = torch.ones(3, 1).double()
    o, S = O.delta_recurrence(k, k, v, one, one, torch.zeros(1, 2, 1).double())
    assert o.flatten().tolist() == [3.0, 5.0, 7.0] and S.flatten().tolist() == [7.0, 5.0]
    y, last = O.short_conv(torch.arange(1.0, 5.0).double()[:, None], torch.tensor([[100.0, 10.0, 1.0]]).double(), torch.zeros(2, 1).double())
    assert y.flatten().tolist() == [1.0, 12.0, 123.0, 234.0] and last.flatten().tolist() == [3.0, 4.0]


def test_batch_lists_the_portion_of_every_token():
    from ktransformers_b200.models.custom_cache import ForwardBatch, PagedStateCache
    c = PagedStateCache([6, 0], [0, 12], max_tokens=32, max_slots=2, device="cpu", dtype=torch.float32, page_size=4)
    b = c.build_batch([("a", [1, 2, 3], [2]), ("b", [7], [0])])
    assert ForwardBatch.N_META == 10 and b.seq_of.tolist() == [0, 0, 0, 1] and b.seqs[:, :2].tolist() == [[0, 3], [3, 1], [-1, -1], [1, 3]]
    c.commit()
    b = c.build_batch([("b", [9, 9], []), ("a", [4], [0])])
    assert b.seq_of.tolist() == [0, 0, 1] and b.seqs[:, :2].tolist() == [[0, 2], [2, 1], [3, 1], [2, 0]]


# ------------------------------------------------------------------------------------------------ mechanisms alone (GPU)
@gpu
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("width", [20, 36, 256, 35, 6, 1024])
def test_output_side_norm_with_weights_around_zero(dtype, tol, width):
    from ktransformers_b200.operators.norm import KGroupRMSNorm
    g = torch.Generator().manual_seed(1)
    x, y = torch.randn(7, width, generator=g), torch.randn(7, width, generator=g) * 3
    post, pre = (KGroupRMSNorm(width, 1, 1e-4, dtype=dtype, weight_offset=1.0) for _ in range(2))
    assert float(post.weight.abs().max()) == 0.0                 # an unloaded weight scales by one
    for n in (post, pre):
        n.load(DictLoader({"w": (0.3 * torch.randn(width, generator=g)).to(dtype)}), "w")
    wp, wq = post.weight.double().cpu(), pre.weight.double().cpu()
    for y_dt in (dtype, torch.float32):
        yd = y.to(y_dt)
        want_x = x.double() + O.offset_rms_norm(yd.double(), wp, 1e-4)
        xo, h = KGroupRMSNorm.fused(x.cuda(), yd.cuda(), post, None, cast_h=True)       # the next sublayer reads the residual itself
        assert rel(xo, want_x) < 1e-6 and h.dtype == dtype and rel(h, want_x) < (tol if dtype == torch.bfloat16 else 1e-6)
        xo, h = KGroupRMSNorm.fused(None, yd.cuda(), post, None, cast_h=True)           # the normed embedding opens the stream
        assert rel(xo, O.offset_rms_norm(yd.double(), wp, 1e-4)) < 1e-6 and rel(h, xo) < tol
        xo, h = KGroupRMSNorm.fused(x.cuda(), yd.cuda(), post, pre, keep_x=False)       # the last sum and the final norm
        assert xo is None and rel(h, O.offset_rms_norm(want_x, wq, 1e-4)) < tol
        xo, h = KGroupRMSNorm.fused(x.cuda(), yd.cuda(), post, None)
        assert h is None and rel(xo, want_x) < 1e-6


@gpu
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 3e-2)])
def test_gated_mlp_with_both_activations(dtype, tol):
    from ktransformers_b200.operators.mlp import KGatedMLP
    g = torch.Generator().manual_seed(2)
    W = {"gate": (torch.randn(52, 24, generator=g) * 0.8).to(dtype), "up": (torch.randn(52, 24, generator=g) * 0.6).to(dtype), "down": torch.randn(24, 52, generator=g).to(dtype)}
    h = (torch.randn(9, 24, generator=g) * 2).to(dtype)
    Wd = {k: v.double() for k, v in W.items()}
    op = KGatedMLP(24, 52, act="gelu_tanh", dtype=dtype)
    op.load(DictLoader(W), "")
    assert rel(op(h.cuda()), O.gated_gelu_mlp(h.double(), Wd["gate"], Wd["up"], Wd["down"])) < tol
    op = KGatedMLP(24, 52, act="silu", dtype=dtype)
    op.load(DictLoader(W), "")
    assert rel(op(h.cuda()), (O.silu(h.double() @ Wd["gate"].T) * (h.double() @ Wd["up"].T)) @ Wd["down"].T) < tol
    z = torch.tensor([-30.0, -3.0, -1.0, -1e-4, 0.0, 1e-4, 0.5, 2.0, 30.0])
    assert rel(O.gelu_tanh(z.double()), torch.nn.functional.gelu(z.double(), approximate="tanh")) < 1e-12


def mixer_alone(desc, dtype, n, page_size, portions, big_at=None, big=30.0, seed=4, width=24, tweak=None, v_other=False, tensor_path=True, h_tweak=None):
    """one mixer operator over one sequence cut into `portions`, against the restatement over the whole sequence; `big_at`:
    the input row of that token is scaled, so its value (and what it writes into a recurrence) stands out"""
    from ktransformers_b200.models.configuration_zivulix import MIXER_SPECS
    from ktransformers_b200.models.custom_cache import PagedStateCache
    from ktransformers_b200.operators.attention import KCappedWindowAttention, KLatentWindowAttention
    from ktransformers_b200.operators.linear_attention import KGatedDeltaRule
    cfg = U.config([(desc, None)], width=width)
    W = {k[len("l0.mix."):]: v for k, v in U.weights(cfg, seed, dtype).items() if k.startswith("l0.mix.")}
    if tweak:
        tweak(W)
    m = desc["mixer"]
    spec = MIXER_SPECS[desc["type"]](m)
    if desc["type"] == "attention":
        op = KCappedWindowAttention(width, spec, 1e-5, dtype=dtype)
        op.use_tensor_cores = tensor_path
    elif desc["type"] == "latent_attention":
        op = KLatentWindowAttention(width, spec, 1e-5, 0, dtype=dtype)
        op.use_tensor_path = tensor_path
    else:
        op = KGatedDeltaRule(width, spec, 1e-5, dtype=dtype)
    op.load(DictLoader(W), "")
    g = torch.Generator().manual_seed(seed)
    h = torch.randn(n, width, generator=g)
    if big_at is not None:
        h[big_at] *= big
    if h_tweak:
        h_tweak(h)
    h = h.to(dtype)
    other = torch.randn(n, m["kv_heads"] * m["vdim"], generator=g).to(dtype) if v_other else None
    Wd = {k: v.double() for k, v in W.items()}
    z = lambda *s: torch.zeros(*s, dtype=torch.float64)
    if desc["type"] == "attention":
        past = (z(0, m["kv_heads"], m["dim"]), z(0, m["kv_heads"], m["vdim"]), torch.zeros(0, dtype=torch.long))
        want, _, v_own = O.capped_window_mixer(h.double(), torch.arange(n), past, Wd, m, 1e-5, other.double().reshape(n, m["kv_heads"], m["vdim"]) if v_other else None)
    elif desc["type"] == "latent_attention":
        want, _ = O.latent_mixer(h.double(), torch.arange(n), (z(0, m["kv_rank"]), z(0, m["rot_dim"]), torch.zeros(0, dtype=torch.long)), Wd, m, 1e-5)
    else:
        C = m["kv_heads"] * m["dim"]
        want, _ = O.delta_mixer(h.double(), (z(m["heads"], m["dim"], m["vdim"]), z(m["conv"] - 1, C), z(m["conv"] - 1, C), z(m["conv"] - 1, m["heads"] * m["vdim"])), Wd, m, 1e-5)
    cache = PagedStateCache([spec.cache_row_width()], [spec.state_width()], n + page_size, 2, "cuda", dtype=dtype, page_size=page_size)
    got, at, k = [], 0, 0
    while at < n:                                                # the last size repeats
        p = min(portions[min(k, len(portions) - 1)], n - at)
        batch = cache.build_batch([("s", [0] * p, [])])
        hp = h[at:at + p].cuda().contiguous()
        if desc["type"] == "attention":
            o, v_mine = op(hp, batch, cache, 0, other[at:at + p].cuda() if v_other else None)
            assert rel(v_mine.reshape(p, m["kv_heads"], m["vdim"]), v_own[at:at + p]) < (1e-5 if dtype == torch.float32 else 3e-2)
        else:
            o = op(hp, batch, cache, 0)
        got.append(o)
        cache.commit()
        at, k = at + p, k + 1
    return torch.cat(got), want


ATTN_SHAPES = [U.attn(), U.attn(heads=6, kv_heads=6, dim=6, vdim=3, window=4, rot_dims=2, factor=None), U.attn(heads=9, kv_heads=1, dim=16, vdim=40, window=33, rot_dims=16, softcap=1.5),
               U.attn(heads=20, kv_heads=2, dim=7, vdim=70, window=None, rot_dims=6, base=7.0, factor=16.0), U.attn(heads=1, kv_heads=1, dim=33, vdim=1, scale=0.9, softcap=None, window=64, rot_dims=0),
               U.attn(heads=4, kv_heads=4, dim=130, vdim=130, window=1, rot_dims=128, softcap=30.0)]


@gpu
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 3e-5), (torch.bfloat16, 4e-2)])
@pytest.mark.parametrize("desc", ATTN_SHAPES)
def test_capped_window_attention_alone(dtype, tol, desc):
    got, want = mixer_alone(desc, dtype, 70, 8, [70])
    assert rel(got, want) < tol
    assert rel(got[:3], want[:3]) < tol                          # the first tokens: one, two, three visible keys
    got2, _ = mixer_alone(desc, dtype, 70, 8, [33, 1, 1, 2, 30, 3])
    assert rel(got2, want) < tol and rel(got2, got) < (1e-5 if dtype == torch.float32 else tol)
    got3, want3 = mixer_alone(dict(desc, mixer=dict(desc["mixer"], v_mix=True)), dtype, 40, 4, [17, 2, 1], v_other=True)          # values blended with handed-in ones
    assert rel(got3, want3) < tol


@gpu
@pytest.mark.parametrize("window", [1, 2, 7, 32, 33, 40])
@pytest.mark.parametrize("decode", [False, True])
def test_window_edge_with_a_value_that_stands_out(window, decode):
    """token 20's value dominates every row that sees it: rows 20 .. 20 + window - 1 do, row 20 + window does not.  Page size 4
    puts the edges on and off page borders; a window one longer or shorter must differ."""
    desc = U.attn(heads=4, kv_heads=2, window=window, softcap=None)
    n = 20 + window + 12
    got, want = mixer_alone(desc, torch.float32, n, 4, [21] + [1] * n if decode else [n], big_at=20)
    assert rel(got, want) < 3e-5
    for r in (20, 20 + window - 1, 20 + window, 20 + window + 1):
        assert rel(got[r], want[r]) < 3e-5
    for other in (window + 1, max(1, window - 1)):
        if other != window:
            _, shifted = mixer_alone(U.attn(heads=4, kv_heads=2, window=other, softcap=None), torch.float32, n, 4, [n], big_at=20)
            assert max(rel(shifted[r], want[r]) for r in (20 + window - 1, 20 + window)) > 1e-2      # the test bites


@gpu
def test_score_cap_bites_and_stretched_rotation_matters():
    """unit-rms queries and keys of 12 columns under scale 1 give raw scores up to 12, far beyond the cap of 2; the same inputs
    without the cap, with another stretch of the wavelengths or with fewer rotated columns must differ"""
    loud = None
    desc = U.attn(heads=4, kv_heads=2, softcap=2.0, window=16, rot_dims=12, factor=8.0, scale=1.0)
    got, want = mixer_alone(desc, torch.float32, 60, 8, [31, 2, 1], tweak=loud)
    assert rel(got, want) < 3e-5
    for other in (U.attn(heads=4, kv_heads=2, softcap=None, window=16, rot_dims=12, factor=8.0, scale=1.0), U.attn(heads=4, kv_heads=2, softcap=2.0, window=16, rot_dims=12, factor=1.0, scale=1.0),
                  U.attn(heads=4, kv_heads=2, softcap=2.0, window=16, rot_dims=8, factor=8.0, scale=1.0)):
        _, differs = mixer_alone(other, torch.float32, 60, 8, [60], tweak=loud)
        assert rel(differs, want) > 1e-2


@gpu
def test_far_value_among_hundreds_and_the_split_path():
    """decode over a long range cuts the keys into parts; a value far back stands out, and so does one at a part's edge"""
    for at in (3, 127, 128, 383, 384):
        got, want = mixer_alone(U.attn(heads=3, kv_heads=1, dim=12, vdim=9, window=None, softcap=None), torch.float32, 700, 16, [690] + [1] * 10, big_at=at)
        assert rel(got, want) < 3e-5
    got, want = mixer_alone(U.attn(heads=3, kv_heads=1, dim=12, vdim=9, window=600, softcap=20.0), torch.float32, 700, 16, [690] + [1] * 10, big_at=95)       # leaves the window while decoding
    assert rel(got, want) < 3e-5 and rel(got[690:], want[690:]) < 3e-5
    got, want = mixer_alone(U.attn(heads=16, kv_heads=2, window=500), torch.bfloat16, 600, 64, [590, 2] + [1] * 8, big_at=164)
    assert rel(got, want) < 4e-2


MMA_SHAPES = [U.attn(heads=8, kv_heads=2, dim=16, vdim=32, window=40, rot_dims=16), U.attn(heads=9, kv_heads=1, dim=48, vdim=16, window=None, softcap=None, rot_dims=32),
              U.attn(heads=34, kv_heads=2, dim=32, vdim=32, window=33), U.attn(heads=4, kv_heads=4, dim=128, vdim=128, window=100, rot_dims=64, softcap=30.0),
              U.attn(heads=12, kv_heads=1, dim=64, vdim=80, window=64, factor=None), U.attn(heads=40, kv_heads=2, dim=16, vdim=112, window=7, softcap=0.8)]


@gpu
@pytest.mark.parametrize("desc", MMA_SHAPES)
def test_tensor_core_attention_path(desc):
    """bf16 with head sizes that are multiples of 16 takes the tensor-core tiles: against the restatement, and against the
    CUDA-core kernel on the same bf16 inputs (between the two: bf16 weights in the second product, and the order of the sums).
    200 tokens cross several key tiles; portions start and end inside tiles; the value that stands out sits at a tile's edge"""
    for portions, at in (([200], 7), ([129, 1, 1, 30, 2, 37], 63), ([64, 64, 8, 1], 64), ([190] + [1] * 10, 127)):
        got, want = mixer_alone(desc, torch.bfloat16, 200, 16, portions, big_at=at, big=4.0)
        simple, _ = mixer_alone(desc, torch.bfloat16, 200, 16, portions, big_at=at, big=4.0, tensor_path=False)
        assert rel(got, want) < 4e-2 and rel(simple, want) < 4e-2
        assert rel(got, simple) < 1.5e-2
        assert rel(got[:3], want[:3]) < 4e-2 and rel(got[at:at + 3], want[at:at + 3]) < 4e-2


@gpu
@pytest.mark.parametrize("window", [1, 2, 31, 32, 33, 64, 65, 100])
@pytest.mark.parametrize("decode", [False, True])
def test_tensor_core_window_edges_inside_and_between_key_tiles(window, decode):
    """the value of token 40 stands out: the last row that sees it and the first that does not, for windows that end inside,
    on and just behind a 32-key tile; a window one longer must differ at that row"""
    mk = lambda w: U.attn(heads=8, kv_heads=2, dim=32, vdim=32, window=w, softcap=None, rot_dims=16)
    n = 40 + window + 12
    portions = [41] + [1] * n if decode else [37, 2, n]
    got, want = mixer_alone(mk(window), torch.bfloat16, n, 16, portions, big_at=40, big=6.0)
    assert rel(got, want) < 4e-2
    for r in (40, 40 + window - 1, 40 + window, 40 + window + 1):
        assert rel(got[r], want[r]) < 4e-2
    _, shifted = mixer_alone(mk(window + 1), torch.bfloat16, n, 16, [n], big_at=40, big=6.0)
    assert rel(shifted[40 + window], want[40 + window]) > 0.08      # the test bites: twice the tolerance even with a hundred keys in sight


@gpu
def test_tensor_core_attention_far_value_and_split_edges():
    """decode over a long range on the tensor-core path cuts the keys into parts of whole tiles"""
    for window in (None, 600):
        desc = U.attn(heads=16, kv_heads=2, dim=32, vdim=48, window=window)
        for at in (3, 127, 128, 383, 384, 640):
            got, want = mixer_alone(desc, torch.bfloat16, 700, 64, [690] + [1] * 10, big_at=at, big=4.0)
            simple, _ = mixer_alone(desc, torch.bfloat16, 700, 64, [690] + [1] * 10, big_at=at, big=4.0, tensor_path=False)
            assert rel(got, want) < 4e-2 and rel(got[690:], want[690:]) < 4e-2 and rel(got, simple) < 1.5e-2


LATENT_SHAPES = [U.latent(), U.latent(heads=1, dim=3, rot_dim=2, vdim=7, kv_rank=33), U.latent(heads=9, dim=16, rot_dim=16, vdim=8, kv_rank=40, base=5e5), U.latent(heads=16, dim=8, rot_dim=6, vdim=20, kv_rank=130)]


@gpu
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 3e-5), (torch.bfloat16, 5e-2)])
@pytest.mark.parametrize("desc", LATENT_SHAPES)
def test_latent_attention_with_a_full_rank_query_alone(dtype, tol, desc):
    got, want = mixer_alone(desc, dtype, 70, 8, [70])
    assert rel(got, want) < tol and rel(got[:3], want[:3]) < tol
    got2, _ = mixer_alone(desc, dtype, 70, 8, [33, 1, 1, 2, 30, 3])
    assert rel(got2, want) < tol and rel(got2, got) < (1e-5 if dtype == torch.float32 else tol)


@gpu
def test_latent_attention_far_key_and_the_tensor_core_latent_sizes():
    for at in (3, 128, 383):
        got, want = mixer_alone(U.latent(heads=3, dim=6, rot_dim=4, vdim=5, kv_rank=12), torch.float32, 700, 16, [690] + [1] * 10, big_at=at)
        assert rel(got, want) < 3e-5
    desc = U.latent(heads=8, dim=32, rot_dim=64, vdim=32, kv_rank=512)
    for portions in ([150], [70, 3, 2, 40, 1, 34], [140] + [1] * 10):
        got, want = mixer_alone(desc, torch.bfloat16, 150, 32, portions, width=64, big_at=40, big=3.0)      # a louder row's scores would lose their fraction to bf16
        simple, _ = mixer_alone(desc, torch.bfloat16, 150, 32, portions, width=64, big_at=40, big=3.0, tensor_path=False)
        assert rel(got, want) < 5e-2 and rel(simple, want) < 5e-2 and rel(got, simple) < 2e-2


DELTA_SHAPES = [U.delta(), U.delta(heads=2, kv_heads=2, dim=17, vdim=33, conv=4), U.delta(heads=6, kv_heads=1, dim=64, vdim=64, conv=2), U.delta(heads=5, kv_heads=5, dim=3, vdim=1, conv=1),
                U.delta(heads=2, kv_heads=1, dim=130, vdim=70, conv=5)]


@gpu
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 3e-5), (torch.bfloat16, 4e-2)])
@pytest.mark.parametrize("desc", DELTA_SHAPES)
def test_gated_delta_rule_alone(dtype, tol, desc):
    got, want = mixer_alone(desc, dtype, 70, 8, [70])
    assert rel(got, want) < tol and rel(got[:5], want[:5]) < tol                     # the first tokens: nothing precedes them, the filter reads zeros there
    for portions in ([33, 1, 1, 2, 30, 3], [2], [15, 1, 16, 17, 1], [1], [3, 1]):     # the scan stages 16 tokens at a time; portions shorter than the convolution
        got2, _ = mixer_alone(desc, dtype, 70, 8, portions)
        assert rel(got2, want) < tol and rel(got2, got) < (1e-5 if dtype == torch.float32 else tol)


@gpu
@pytest.mark.parametrize("decode", [False, True])
def test_recurrent_state_carries_a_far_token(decode):
    """almost no decay (exp(A_log) tiny) and small steps: what token 5 wrote, scaled up, still shows 300 tokens later; a state
    that were lost, reset or decayed wrongly on the way would show at once"""
    def slow(W):                                                 # input column 0 drives the step size: 5 there makes beta ~ 5e-4
        W["A_log"] = W["A_log"] - 7.0
        W["b"] = W["b"] * 0.05
        W["b"][:, 0] = -1.5

    def quiet_but_one(h):                                        # every token writes with a tiny step, token 5 with a large one
        h[:, 0] = 5.0
        h[5, 0] = 0.0
    desc = U.delta(heads=2, kv_heads=1, dim=12, vdim=9, conv=3)
    got, want = mixer_alone(desc, torch.float32, 320, 8, [200] + [1] * 120 if decode else [7, 100, 2, 211], big_at=5, tweak=slow, h_tweak=quiet_but_one)
    assert rel(got, want) < 3e-5 and rel(got[300:], want[300:]) < 3e-5
    plain, _ = mixer_alone(desc, torch.float32, 320, 8, [320], tweak=slow, h_tweak=lambda h: h.__setitem__((slice(None), 0), 5.0))
    assert rel(plain[300:], want[300:]) > 3e-2                   # the test bites: without the far token the late rows differ
    fast = lambda W: (slow(W), W.__setitem__("A_log", W["A_log"] + 7.0))
    decayed, _ = mixer_alone(desc, torch.float32, 320, 8, [320], big_at=5, tweak=fast, h_tweak=quiet_but_one)
    assert rel(decayed[300:], want[300:]) > 3e-2                 # and so does the decay


@gpu
def test_convolution_inputs_cross_portion_cuts():
    """a loud token's input reaches the next conv - 1 outputs only; cut right behind it, one token at a time, the later outputs
    must read it from the state row"""
    desc = U.delta(heads=2, kv_heads=2, dim=8, vdim=8, conv=4)
    for portions in ([11, 1, 1, 1, 1, 20], [10, 2, 1, 3], [1]):
        got, want = mixer_alone(desc, torch.float32, 40, 8, portions, big_at=10, big=8.0)
        assert rel(got, want) < 3e-5 and rel(got[10:15], want[10:15]) < 3e-5


# ------------------------------------------------------------------------------------------------ whole model (GPU)
@gpu
@pytest.mark.parametrize("dtype,tol", [("float32", F32_TOL), ("bfloat16", BF16_TOL)])
def test_prompt_decode_and_portions_agree_with_the_restatement(tmp_path, dtype, tol):
    cfg = U.config(MIXED)
    eng, om = serve(tmp_path, cfg, dtype, max_tokens=128, max_slots=2, page_size=4)
    t = toks(75)
    want = oracle_logits(om, t)
    err = rel if dtype == "float32" else rel_rows
    whole = run_steps(eng, cut("w", t, [75]))["w"]
    assert err(whole, want) < tol
    assert err(whole[:4], want[:4]) < tol                       # the first tokens of a sequence
    for sizes in ([1], [2], [3, 2, 7, 1, 5], [20, 2, 2, 1]):
        got = run_steps(eng, cut("p", t, sizes))["p"]
        assert err(got, want) < tol
        assert err(got, whole) < (2e-5 if dtype == "float32" else tol)   # the cut does not matter beyond rounding


@gpu
def test_whole_model_in_bf16_on_tensor_core_head_sizes(tmp_path):
    """head sizes that are multiples of 16: bf16 attention runs on the tensor-core tiles inside a whole model (grouped heads,
    blended values, 150 tokens over several key tiles), whole, in portions and with a decoded tail"""
    layers = [(U.attn(heads=6, kv_heads=2, dim=32, vdim=48, window=40, rot_dims=16, v_mix=True), U.dense(96)), (U.delta(heads=4, kv_heads=2, dim=32, vdim=16), None),
              (U.attn(heads=4, kv_heads=2, dim=16, vdim=48, window=None, v_mix=True), U.dense(64)), (U.latent(heads=4, dim=16, rot_dim=16, vdim=16, kv_rank=32), None)]
    cfg = U.config(layers, width=64, vocab=90)
    eng, om = serve(tmp_path, cfg, "bfloat16", seed=3, max_tokens=512, max_slots=2, page_size=16)
    t = toks(150, 90, seed=9)
    want = oracle_logits(om, t)
    for k, sizes in enumerate(([150], [70, 3, 2, 40, 1, 34], [130] + [1] * 20)):
        assert rel_rows(run_steps(eng, cut(("m", k), t, sizes))[("m", k)], want) < BF16_TOL


@gpu
def test_residual_stream_after_every_layer(tmp_path):
    cfg = U.config(MIXED)
    eng, om = serve(tmp_path, cfg, "float32", max_tokens=64, max_slots=2, page_size=8)
    t = toks(11, seed=2)
    want, got = [], []
    om.forward(t, om.new_state(), want)
    eng.model(eng.cache.build_batch([("r", t, [])]), eng.cache, got)
    assert len(got) == len(want) == 6
    for a, b in zip(got, want):
        assert rel(a, b) < 1e-4


@gpu
def test_value_blend_takes_the_first_blending_layer_whatever_its_place(tmp_path):
    """the first layer that blends sits behind a layer that does not and a recurrent one; with the blend weights zeroed the
    logits must differ (the test bites), and a model whose later layers do not blend must equal that"""
    layers = [(U.attn(v_mix=False), None), (U.delta(), None), (U.attn(v_mix=True), U.dense()), (U.attn(v_mix=False, window=4), None), (U.attn(v_mix=True, window=30), None)]
    cfg = U.config(layers)
    eng, om = serve(tmp_path, cfg, "float32", seed=1, max_tokens=64, max_slots=2, page_size=8)
    t = toks(30, seed=4)
    want = oracle_logits(om, t)
    assert rel(run_steps(eng, cut("a", t, [13, 2, 1]))["a"], want) < F32_TOL
    w = U.weights(cfg, 1, torch.float32)
    w["l4.mix.vmix"] = torch.tensor(0.0)
    assert rel(oracle_logits(O.Model(cfg, w, torch.float64), t), want) > 1e-3


@gpu
def test_other_sizes_and_layer_orders(tmp_path):
    cases = [
        ([(U.delta(heads=1, kv_heads=1, dim=2, vdim=2, conv=2), U.dense(3))], dict(width=8)),                                                                     # one recurrent layer
        ([(U.latent(heads=16, dim=12, rot_dim=10, vdim=10, kv_rank=48), U.dense(100)), (U.attn(heads=16, kv_heads=4, dim=12, vdim=10, window=12, v_mix=True), None)] * 2, dict(width=72, vocab=31)),
        ([(U.delta(heads=5, kv_heads=5, dim=24, vdim=24), U.dense(20)), (U.attn(heads=2, kv_heads=1, dim=8, vdim=8, rot_dims=8), U.dense(8)), (U.latent(), None)], dict(width=40)),
        ([(U.attn(), None), (U.attn(window=3, softcap=0.7), U.dense(16)), (U.delta(conv=1), U.dense(24))], dict(width=16, eps=1e-3)),
        ([(U.latent(heads=2, dim=4, rot_dim=8, vdim=4, kv_rank=6), None)], dict(width=12, vocab=7))]
    for k, (layers, kw) in enumerate(cases):
        cfg = U.config(layers, **kw)
        eng, om = serve(tmp_path, cfg, "float32", seed=10 + k, max_tokens=64, max_slots=2, page_size=8)
        t = toks(30, cfg["vocab"], seed=k)
        assert rel(run_steps(eng, cut("a", t, [13, 2, 1]))["a"], oracle_logits(om, t)) < F32_TOL


@gpu
@pytest.mark.parametrize("seed", range(8))
def test_drawn_configurations(tmp_path, seed):
    """sizes, layer order and constants drawn per seed: one prompt whole, in uneven portions, and with a decoded tail"""
    r = random.Random(seed)
    width = r.choice([16, 40, 136, 320])
    layers, kv_shape = [], (r.choice([1, 2, 3]), r.choice([5, 8, 48]))          # blending layers share their value shape
    for _ in range(r.randint(1, 6)):
        kind = r.random()
        if kind < 0.4:
            mix = r.random() < 0.6
            G, dv = kv_shape if mix else (r.choice([1, 2, 4]), r.choice([5, 8, 96]))
            d = r.choice([4, 6, 24, 64])
            m = U.attn(heads=G * r.choice([1, 2, 5, 9]), kv_heads=G, dim=d, vdim=dv, scale=r.choice([None, 0.11, 1.0]), softcap=r.choice([None, 0.5, 30.0]),
                       window=r.choice([None, 1, 5, 31, 32, 33, 64, 100]), rot_dims=r.choice([0, 2, d // 2 * 2]), base=r.choice([10.0, 1e4, 1e6]), factor=r.choice([None, 1.0, 4.0, 32.0]), v_mix=mix)
        elif kind < 0.65:
            m = U.latent(heads=r.choice([1, 2, 5, 9]), dim=r.choice([4, 7, 24]), rot_dim=r.choice([2, 8, 32]), vdim=r.choice([5, 8, 48]), kv_rank=r.choice([8, 33, 96]), scale=r.choice([None, 0.2]),
                         base=r.choice([10.0, 1e4, 1e6]))
        else:
            G = r.choice([1, 2, 4])
            m = U.delta(heads=G * r.choice([1, 2, 3]), kv_heads=G, dim=r.choice([4, 7, 24, 64, 100]), vdim=r.choice([5, 8, 32, 48, 65]), conv=r.choice([1, 2, 3, 4, 6]))
        layers.append((m, r.choice([None, U.dense(ff=r.choice([8, 100, 1030]))])))
    cfg = U.config(layers, vocab=r.choice([31, 77, 1000]), width=width, eps=r.choice([1e-6, 1e-5, 1e-3]))
    eng, om = serve(tmp_path, cfg, "float32", seed=seed, max_tokens=256, max_slots=2, page_size=r.choice([4, 16, 64]))
    t = toks(r.choice([40, 90, 150]), cfg["vocab"], seed=seed)
    want = oracle_logits(om, t)
    for k, sizes in enumerate(([len(t)], [3, 17, 2, 1, 33, 2, 64], [len(t) - 20] + [1] * 20)):
        assert rel(run_steps(eng, cut(("d", k), t, sizes))[("d", k)], want) < F32_TOL


@gpu
def test_captured_decode_steps_with_a_key_range_cut_for_a_large_cache(tmp_path):
    """a roomy cache makes the replayed decode step cut its key range into many parts, most of them empty for a short sequence;
    the recurrent state rows flip between the replays"""
    cfg = U.config(MIXED)
    eng, om = serve(tmp_path, cfg, "float32", max_tokens=8192, max_slots=2, page_size=16)
    for r, n in enumerate((40, 330)):
        t = toks(n, seed=40 + r)
        got = run_steps(eng, cut(("g", r), t, [n - 12] + [1] * 12))[("g", r)]
        assert rel(got, oracle_logits(om, t)) < F32_TOL
    assert 1 in eng._captured and eng._captured[1].graph is not None


@gpu
def test_unequal_requests_in_one_batch_equal_each_alone(tmp_path):
    cfg = U.config(MIXED)
    eng, om = serve(tmp_path, cfg, "float32", max_tokens=256, max_slots=4, page_size=4)
    ta, tb, tc = toks(23, seed=1), toks(9, seed=2), toks(14, seed=3)
    steps = [[("a", ta[:10], False), ("b", tb[:1], False)],
             [("a", ta[10:11], False), ("b", tb[1:9], True), ("c", tc[:2], False)],
             [("c", tc[2:14], True), ("a", ta[11:23], True)]]
    got = run_steps(eng, steps)
    for i, t in (("a", ta), ("b", tb), ("c", tc)):
        assert rel(got[i], oracle_logits(om, t)) < F32_TOL
        alone = run_steps(eng, cut(i + "'", t, [len(t)]))[i + "'"]
        assert rel(got[i], alone) < 2e-5


@gpu
def test_long_decode_over_reused_pages_and_slots(tmp_path):
    """pages of 4 and 2 slots: sequences come and go, pages and state rows are handed out again un-cleared, and a new sequence in
    a used slot must start from an empty state and zero convolution inputs.  Every caching layer has a window, so pages behind
    the largest one are given back while a sequence runs and its page table row wraps around."""
    layers = [(U.attn(window=9, v_mix=True), U.dense()), (U.delta(), None), (U.attn(heads=6, kv_heads=2, window=21, v_mix=True), None), (U.delta(heads=2, kv_heads=2, dim=8, vdim=8, conv=4), U.dense(8))]
    cfg = U.config(layers)
    eng, om = serve(tmp_path, cfg, "float32", max_tokens=48, max_slots=2, page_size=4)
    assert eng.cache.window == 21
    for r in range(3):
        t = toks(150, seed=20 + r)                              # longer than the cache: only the window's pages are held
        got = run_steps(eng, cut(("s", r), t, [6] + [1] * 144))[("s", r)]
        assert rel(got, oracle_logits(om, t)) < F32_TOL
        short = toks(3, seed=30 + r)
        assert rel(run_steps(eng, cut(("t", r), short, [3]))[("t", r)], oracle_logits(om, short)) < F32_TOL
    assert len(eng.cache._free_pages) == eng.cache.num_pages and len(eng.cache._free_slots) == 2


@gpu
def test_greedy_generation_through_the_scheduler_and_the_command_line(tmp_path, capsys):
    from ktransformers_b200 import local_chat
    cfg = U.config(MIXED)
    eng, om = serve(tmp_path, cfg, "float32", max_tokens=256, max_slots=3, page_size=4, max_step_tokens=7)
    prompts = [toks(12, seed=5), toks(3, seed=6), toks(20, seed=7), toks(1, seed=8)]
    want = []
    for p in prompts:
        st, out = om.new_state(), []
        nxt = int(om.forward(p, st)[-1].argmax())
        for _ in range(6):
            out.append(nxt)
            nxt = int(om.forward([nxt], st)[-1].argmax())
        want.append(out)
    assert eng.generate(prompts, 6) == want                      # 4 requests, 3 slots, 7 tokens per step: portions and decode mix
    assert len(eng.cache._free_slots) == 3
    args = ["--model_path", str(tmp_path / "ckpt0"), "--dtype", "float32", "--max_new_tokens", "6", "--chunk_size", "5"]
    for p in prompts[:2]:
        args += ["--prompt_ids", ",".join(map(str, p))]
    assert local_chat.main(args) == 0
    lines = [json.loads(l) for l in capsys.readouterr().out.strip().splitlines() if l.startswith("{")]
    assert [l["output"] for l in lines] == want[:2]


@gpu
@pytest.mark.parametrize("dtype,tol", [("float32", F32_TOL), ("bfloat16", BF16_TOL)])
def test_trace_replay_runner(tmp_path, dtype, tol):
    """bin/trace_run as a process: steps on standard input, one logits file per step that asks for some, `done <n>` lines"""
    import os
    import subprocess
    import sys

    import numpy as np
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = U.config(MIXED[:4], vocab=41)
    w = U.weights(cfg, 5, torch.bfloat16 if dtype == "bfloat16" else torch.float32)
    path = U.save(tmp_path / "m", cfg, w)
    om = O.Model(cfg, w, torch.float64)
    a, b = toks(21, 41, seed=1), toks(9, 41, seed=2)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:15], "want": [0, 14]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[15:17], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": a[17:18], "want": [0]}], "end": []},
             {"step": 3, "entries": [{"id": "a", "tokens": a[18:21], "want": [2, 1]}], "end": ["a"]},
             {"step": 4, "entries": [{"id": "b", "tokens": b, "want": [8]}], "end": ["b"]}]
    out = tmp_path / "out"
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", path, "--dtype", dtype, "--out", str(out), "--max-tokens", "64"],
                       input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done ")] == [f"done {i}" for i in range(5)]
    la, lb = oracle_logits(om, a), oracle_logits(om, b)
    want = {0: la[[0, 14]], 2: la[[17]], 3: la[[20, 19]], 4: lb[[8]]}
    assert not (out / "1.f32").exists()
    err = rel if dtype == "float32" else rel_rows
    for n, ref in want.items():
        got = torch.from_numpy(np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(-1, 41))
        assert got.shape == ref.shape and err(got, ref) < tol
