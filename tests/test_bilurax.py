"""Bilurax through the framework (registry, loader, paged state cache, scheduler, engine, CUDA operators) against the plain
restatement in oracle/bilurax_oracle.py, on small random checkpoints made here.  CPU tests cover the host logic."""
import json
import random

import pytest
import torch

import bilurax_util as U
from oracle import bilurax_oracle as O

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


MIXED = [(U.attn(), U.dense()), (U.attn(heads=6, kv_heads=3, dim=4, vdim=7, chunk=5, softcap=2.0), U.moe()), (U.attn(heads=2, kv_heads=1, dim=8, vdim=3, chunk=16), None),
         (U.attn(heads=3, kv_heads=3, dim=5, vdim=5, chunk=9, softcap=None), U.moe(ff=7, experts=9, top=2, groups=3, keep=1, scale=2.0, limit=1.5))]


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
    from ktransformers_b200.models.configuration_bilurax import BiluraxConfig
    cfg = U.config(MIXED, vocab=77, width=40, eps=2e-4, loop=(1, 3, 3), embed_scale=5.5, logit_softcap=11.0)
    c = BiluraxConfig.from_dict(cfg)
    assert (c.vocab, c.width, c.norm_eps, c.embedding_scale, c.logit_softcap) == (77, 40, 2e-4, 5.5, 11.0)
    a = c.layers[1].mixer
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.chunk, a.softcap) == (6, 3, 4, 7, 5, 2.0) and abs(a.scale - 0.5) < 1e-12
    assert c.layers[3].mixer.softcap is None and c.layers[2].mlp is None and c.layers[0].mlp.kind == "dense" and c.layers[0].mlp.ff == 40
    f = c.layers[3].mlp
    assert (f.kind, f.ff, f.experts, f.top, f.groups, f.keep_groups, f.out_scale, f.limit) == ("moe", 7, 9, 2, 3, 1, 2.0, 1.5)
    assert c.layer_runs() == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (1, 2), (2, None), (3, None)]
    assert c.cache_row_widths() == [2 * 11, 3 * 11, 1 * 11, 3 * 11, 1 * 11, 3 * 11, 1 * 11, 3 * 10] and c.state_widths() == [40] * 8
    assert c.chunks() == [7, 5, 16, 9]
    assert BiluraxConfig.from_dict(U.config(MIXED[:1])).layer_runs() == [(0, None)]
    with pytest.raises(ValueError):
        BiluraxConfig.from_dict(U.config(MIXED, loop=(2, 5, 2)))
    with pytest.raises(ValueError):
        BiluraxConfig.from_dict(dict(cfg, layers=[dict(cfg["layers"][0], type="conv")]))


def test_registry_picks_the_class_by_config():
    from ktransformers_b200.models import architecture_of, model_class
    assert model_class(architecture_of(U.config(MIXED))).__name__ == "BiluraxForCausalLM"


def test_oracle_portions_equal_whole_prompt_and_the_mask_is_what_it_says():
    cfg = U.config(MIXED, loop=(0, 2, 2))
    om = O.Model(cfg, U.weights(cfg, 3, torch.float32))
    t = toks(23, seed=1)
    whole = om.forward(t, om.new_state())
    st = om.new_state()
    parts = torch.cat([om.forward(t[a:b], st) for a, b in ((0, 6), (6, 7), (7, 9), (9, 23))])
    assert rel(parts, whole) < 1e-9
    # the chunked mask against a matrix form: a block-diagonal lower triangle
    g = torch.Generator().manual_seed(0)
    q, k, v = torch.randn(11, 4, 3, generator=g).double(), torch.randn(11, 2, 3, generator=g).double(), torch.randn(11, 2, 2, generator=g).double()
    temp, pos = torch.tensor([0.5, 1.0, 1.5, 2.0]).double(), torch.arange(11)
    got = O.chunk_softmax_attention(q, k, v, pos, pos, 0.7, temp, 3.0, 4)
    s = torch.einsum("thd,nhd->htn", q, k.repeat_interleave(2, 1)) * 0.7 * temp.reshape(4, 1, 1)
    s = 3.0 * torch.tanh(s / 3.0)
    ok = (pos[None, :] <= pos[:, None]) & (pos[None, :] // 4 == pos[:, None] // 4)
    want = torch.einsum("htn,nhv->thv", torch.softmax(s.masked_fill(~ok, float("-inf")), -1), v.repeat_interleave(2, 1))
    assert rel(got, want) < 1e-12
    assert rel(got[4], v.repeat_interleave(2, 1)[4]) < 1e-12          # the first token of a chunk sees itself alone


def test_oracle_router_keeps_negative_choice_scores_inside_the_best_groups():
    """all choice scores negative: an expert outside the kept groups must not be chosen although 0 would beat every score"""
    router = torch.zeros(6, 4, dtype=torch.float64)
    corr = torch.tensor([-2.0, -2.1, -3.0, -3.0, -2.5, -2.6], dtype=torch.float64)
    ids, w = O.grouped_sigmoid_router(torch.ones(1, 4, dtype=torch.float64), router, corr, 3, 3, 2, 2.0)
    assert ids.tolist() == [[0, 1, 4]]                               # groups {0, 1} and {4, 5} are kept; 5 loses to 4
    assert rel(w, torch.full((1, 3), 2.0 / 3.0, dtype=torch.float64)) < 1e-12             # equal scores 0.5: a third each, times the scale


def test_cache_gives_back_pages_before_the_current_chunk():
    from ktransformers_b200.models.custom_cache import PagedStateCache
    c = PagedStateCache([4, 4], [0, 0], 64, 2, "cpu", dtype=torch.float32, page_size=4, chunks=[6, 10])
    s = c.open("a")
    free0 = len(c._free_pages)
    c.extend(s, 9)
    c.commit()                       # next position 9: chunks start at 6 and 0 -> position 0 may still be read
    assert c._first_page[s] == 0 and len(c._free_pages) == free0 - 3
    c.extend(s, 4)
    c.commit()                       # next position 13: chunk starts 12 and 10 -> keys before 10 are dead: pages 0 and 1
    assert c._first_page[s] == 2 and len(c._free_pages) == free0 - 4 + 2
    c.extend(s, 60)                  # far beyond the pool's share: only live pages count
    c.commit()
    assert c._first_page[s] == (73 - 73 % 10) // 4
    c.close("a")
    assert len(c._free_pages) == free0
    roomy = PagedStateCache([4], [0], 64, 2, "cpu", dtype=torch.float32, page_size=4)
    s = roomy.open("b")
    roomy.extend(s, 40)
    roomy.commit()
    assert roomy._first_page[s] == 0


# ------------------------------------------------------------------------------------------------ mechanisms alone (GPU)
@gpu
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("width", [20, 36, 256, 35, 6, 1024])
def test_norm_with_sum_row_vector_and_token_shift(dtype, tol, width):
    """x + a + b + row, its norm, and the shift whose previous row comes from the same launch or from the state rows"""
    from ktransformers_b200.models.custom_cache import PagedStateCache
    from ktransformers_b200.operators.norm import KGroupRMSNormShift
    g = torch.Generator().manual_seed(width)
    n = 9
    x, a, b, row = torch.randn(n, width, generator=g), torch.randn(n, width, generator=g).to(dtype), torch.randn(n, width, generator=g), torch.randn(width, generator=g)
    w, mu = (1 + 0.3 * torch.randn(width, generator=g)).to(dtype), torch.rand(width, generator=g).to(dtype)
    op = KGroupRMSNormShift(width, 1, 1e-5, shift=True, dtype=dtype)
    op.load(DictLoader({"n": w, "s": mu}), "n", "s")
    xs = x.double() + a.double() + b.double() + row.double()
    h = O.rms_norm(xs, w.double(), 1e-5)
    hs, last = O.token_shift(h, torch.zeros(width, dtype=torch.float64), mu.double())
    cache = PagedStateCache([0], [width], 32, 2, "cuda", dtype=dtype, page_size=4)
    outs, at = [], 0
    for p in (4, 1, 2, 2):
        batch = cache.build_batch([("s", [0] * p, [])])
        sl = slice(at, at + p)
        x_out, h_out, hs_out = op(x[sl].cuda().contiguous(), a[sl].cuda().contiguous(), b[sl].cuda().contiguous(), 1.0, batch, cache.state[0], row_add=row.cuda())
        assert rel(x_out, xs[sl]) < 1e-6 and rel(h_out, h[sl]) < tol
        outs.append(hs_out)
        cache.commit()
        at += p
    assert rel(torch.cat(outs), hs) < tol
    assert rel(torch.cat(outs)[0], h[0] * (1 - mu.double())) < tol                  # nothing stands before the first token
    # a row vector alone (no other addend), no shift
    plain = KGroupRMSNormShift(width, 1, 1e-5, shift=False, dtype=dtype)
    plain.load(DictLoader({"n": w}), "n")
    x_out, h_out, _ = plain(x.cuda(), row_add=row.cuda())
    assert rel(x_out, x.double() + row.double()) < 1e-6 and rel(h_out, O.rms_norm(x.double() + row.double(), w.double(), 1e-5)) < tol


@gpu
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 3e-2)])
def test_relu_squared_mlp(dtype, tol):
    from ktransformers_b200.operators.mlp import KReluSquaredMLP
    g = torch.Generator().manual_seed(2)
    for width, ff, n in ((24, 40, 5), (33, 7, 70)):
        up, down = (torch.randn(ff, width, generator=g) / width ** 0.5).to(dtype), (torch.randn(width, ff, generator=g) / ff ** 0.5).to(dtype)
        h = torch.randn(n, width, generator=g).to(dtype)
        op = KReluSquaredMLP(width, ff, dtype=dtype)
        op.load(DictLoader({"up": up, "down": down}), "")
        assert rel(op(h.cuda()), O.relu2_mlp(h.double(), up.double(), down.double())) < tol


ROUTERS = [dict(experts=6, top=2, groups=3, keep=2, scale=1.7), dict(experts=10, top=3, groups=2, keep=1, scale=2.0), dict(experts=16, top=4, groups=1, keep=1, scale=1.0),
           dict(experts=12, top=5, groups=4, keep=3, scale=0.5), dict(experts=4, top=2, groups=4, keep=2, scale=1.0), dict(experts=64, top=8, groups=8, keep=4, scale=2.0),
           dict(experts=5, top=1, groups=1, keep=1, scale=3.0)]


@gpu
@pytest.mark.parametrize("r", ROUTERS)
@pytest.mark.parametrize("width,n", [(24, 7), (24, 130), (30, 5)])
def test_grouped_sigmoid_router(r, width, n):
    """decode-sized batches (one launch), prompt-sized ones (GEMM + selection) and a width the GEMV kernel does not take"""
    from ktransformers_b200.operators.gate import KGroupedSigmoidGate
    g = torch.Generator().manual_seed(n + r["experts"])
    W, corr = torch.randn(r["experts"], width, generator=g) * 0.6, torch.randn(r["experts"], generator=g) * 0.6 - 0.7
    x = torch.randn(n, width, generator=g)
    op = KGroupedSigmoidGate(width, r["experts"], r["top"], r["groups"], r["keep"], r["scale"])
    op.load(DictLoader({"r": W, "c": corr}), "r", "c")
    ids, wts = op(x.cuda())
    want_ids, want_w = O.grouped_sigmoid_router(x.double(), W.double(), corr.double(), r["top"], r["groups"], r["keep"], r["scale"])
    assert ids.cpu().tolist() == want_ids.tolist()
    assert rel(wts, want_w) < 1e-5
    if r["groups"] > r["keep"] and r["experts"] > r["groups"]:       # the test bites: choosing among ALL experts picks others somewhere
        free_ids, _ = O.grouped_sigmoid_router(x.double(), W.double(), corr.double(), r["top"], 1, 1, r["scale"])
        assert n < 10 or free_ids.tolist() != want_ids.tolist()


@gpu
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 3e-2)])
@pytest.mark.parametrize("n,path", [(1, "pair"), (5, "pair"), (3, "expert"), (9, "expert"), (70, "grouped")])
def test_clamped_gated_experts_on_every_path(dtype, tol, n, path):
    from ktransformers_b200.operators.experts import KExpertsDense
    g = torch.Generator().manual_seed(n)
    for width, ff, E, top, limit in ((24, 16, 6, 2, 0.8), (40, 9, 5, 3, 2.0)):
        W = {}
        for e in range(E):
            W[f"e{e}.gate"], W[f"e{e}.up"], W[f"e{e}.down"] = [(torch.randn(*s, generator=g) * k).to(dtype) for s, k in (((ff, width), 0.5), ((ff, width), 0.5), ((width, ff), 0.3))]
        op = KExpertsDense(width, ff, E, dtype=dtype, act="clamped_glu", limit=limit)
        op.load(DictLoader(W), "")
        if path == "pair":
            op.by_expert_min_tokens = 10 ** 9
        elif path == "grouped":
            assert n >= op.grouped_min_tokens
        x = torch.randn(n, width, generator=g).to(dtype)
        ids = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(n)])
        wts = torch.rand(n, top, generator=g)
        got = op(x.cuda(), ids.cuda(), wts.cuda())
        Wd = {k: v.double() for k, v in W.items()}
        want = torch.stack([sum(wts[t, j].double() * O.clamped_glu_expert(x[t].double(), Wd[f"e{int(ids[t, j])}.gate"], Wd[f"e{int(ids[t, j])}.up"], Wd[f"e{int(ids[t, j])}.down"], limit)
                                for j in range(top)) for t in range(n)])
        assert rel(got, want) < tol
        pre = x.double() @ Wd["e0.gate"].T                         # both clamps bite on these inputs
        assert (pre > limit).any() and (pre < -limit).any()


def standout(j):
    """Makes token j's key the one every query looks for: all queries become one vector per key/value head (no query weights, the
    bias repeated over the group's heads), the key biases vanish, and row j of the mixer input is solved so that its key is that
    vector while every other token's key is orthogonal to it.  Queries and keys are normed over their whole projection, so only
    directions count; values are unit-rms, so nothing else can make a token stand out."""
    def tweak(W, h, m):
        H, G, d = m["heads"], m["kv_heads"], m["dim"]
        g = torch.Generator().manual_seed(99)
        c = torch.randn(G, d, generator=g)
        W["q"] = torch.zeros_like(W["q"])
        W["q.b"] = c.repeat_interleave(H // G, 0).reshape(-1).to(W["q.b"].dtype)
        W["k.b"] = torch.zeros_like(W["k.b"])
        W["q.norm"], W["k.norm"] = torch.ones_like(W["q.norm"]), torch.ones_like(W["k.norm"])
        W["temp"] = torch.ones_like(W["temp"])
        h[j] = torch.linalg.lstsq(W["k"].double(), c.reshape(-1, 1).double()).solution.reshape(-1).to(h.dtype) * 3.0
        # every other token's key is made orthogonal to the looked-for vector, head by head: its score is zero
        a = torch.stack([W["k"][g * d:(g + 1) * d].double().T @ c[g].double() for g in range(G)], 1)
        basis = torch.linalg.qr(a).Q
        for i in range(h.shape[0]):
            if i != j:
                h[i] = (h[i].double() - basis @ (basis.T @ h[i].double())).to(h.dtype)
    return tweak


def attention_alone(desc, dtype, n, page_size, portions, seed=4, width=24, tweak=None, tensor_path=True):
    """the attention operator over one sequence cut into `portions`, against the restatement over the whole sequence"""
    from ktransformers_b200.models.configuration_bilurax import ChunkedAttentionSpec
    from ktransformers_b200.models.custom_cache import PagedStateCache
    from ktransformers_b200.operators.attention import KChunkedSoftmaxAttention
    cfg = U.config([(desc, None)], width=width)
    W = {k[len("l0.mix."):]: v for k, v in U.weights(cfg, seed, dtype).items() if k.startswith("l0.mix.")}
    m = desc["mixer"]
    g = torch.Generator().manual_seed(seed)
    h = torch.randn(n, width, generator=g)
    if tweak:
        tweak(W, h, m)
    h = h.to(dtype)
    spec = ChunkedAttentionSpec.from_dict(m)
    op = KChunkedSoftmaxAttention(width, spec, 1e-5, dtype=dtype)
    op.use_tensor_cores = tensor_path
    op.load(DictLoader(W), "")
    Wd = {k: v.double() for k, v in W.items()}
    past = (torch.zeros(0, m["kv_heads"], m["dim"], dtype=torch.float64), torch.zeros(0, m["kv_heads"], m["vdim"], dtype=torch.float64), torch.zeros(0, dtype=torch.long))
    want, _ = O.attention_mixer(h.double(), torch.arange(n), past, Wd, m, 1e-5)
    cache = PagedStateCache([spec.cache_row_width()], [0], n + page_size, 2, "cuda", dtype=dtype, page_size=page_size)
    got, at, k = [], 0, 0
    while at < n:                                                # the last size repeats
        p = min(portions[min(k, len(portions) - 1)], n - at)
        batch = cache.build_batch([("s", [0] * p, [])])
        got.append(op(h[at:at + p].cuda().contiguous(), batch, cache, 0))
        cache.commit()
        at, k = at + p, k + 1
    return torch.cat(got), want


ATTN_SHAPES = [U.attn(), U.attn(heads=6, kv_heads=6, dim=6, vdim=3, chunk=4, softcap=None), U.attn(heads=9, kv_heads=1, dim=16, vdim=40, chunk=33, softcap=1.5),
               U.attn(heads=20, kv_heads=2, dim=7, vdim=70, chunk=1000, scale=0.4), U.attn(heads=1, kv_heads=1, dim=33, vdim=1, scale=0.9, chunk=64), U.attn(heads=4, kv_heads=4, dim=130, vdim=130, chunk=1)]


@gpu
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 3e-5), (torch.bfloat16, 4e-2)])
@pytest.mark.parametrize("desc", ATTN_SHAPES)
def test_chunked_attention_alone(dtype, tol, desc):
    width = 24 if desc["mixer"]["dim"] < 100 else 48
    got, want = attention_alone(desc, dtype, 70, 8, [70], width=width)
    assert rel(got, want) < tol
    assert rel(got[:3], want[:3]) < tol                          # the first tokens: one, two, three visible keys
    got2, _ = attention_alone(desc, dtype, 70, 8, [33, 1, 1, 2, 30, 3], width=width)
    assert rel(got2, want) < tol and rel(got2, got) < (1e-5 if dtype == torch.float32 else tol)


@gpu
def test_each_norm_and_the_temperature_matter():
    """the restatement with one ingredient changed differs from the kernels' result: the tests above would catch a kernel that
    normed queries head by head, left the values alone or forgot a head's temperature"""
    desc = U.attn(heads=4, kv_heads=2, dim=6, vdim=5, chunk=20, softcap=None)
    got, want = attention_alone(desc, torch.float32, 40, 8, [40])
    assert rel(got, want) < 3e-5
    real = O.rms_norm, O.rms
    try:
        O.rms_norm = lambda x, w, eps: (real[1](x.reshape(x.shape[0], -1, 6), eps).reshape(x.shape) * w if x.shape[-1] in (24, 12) else real[0](x, w, eps))
        _, per_head = attention_alone(desc, torch.float32, 40, 8, [40])
        O.rms_norm = real[0]
        O.rms = lambda x, eps: x if x.dim() == 3 else real[1](x, eps)
        _, raw_values = attention_alone(desc, torch.float32, 40, 8, [40])
    finally:
        O.rms_norm, O.rms = real
    assert rel(per_head, want) > 1e-2 and rel(raw_values, want) > 1e-2

    def flat_temp(W, h, m):
        W["temp"] = torch.ones_like(W["temp"])
    _, no_temp = attention_alone(desc, torch.float32, 40, 8, [40], tweak=flat_temp)
    assert rel(no_temp, want) > 1e-2


@gpu
@pytest.mark.parametrize("chunk", [1, 2, 7, 32, 33, 40])
@pytest.mark.parametrize("decode", [False, True])
def test_chunk_edge_with_a_key_that_stands_out(chunk, decode):
    """every query looks for token j's key, the second token of a chunk: the rows from j to the end of that chunk return its value, the
    last row of the chunk before and the first of the chunk after do not.  Page size 4 puts the edges on and off page borders; a
    chunk one longer or shorter must differ."""
    desc = U.attn(heads=4, kv_heads=2, chunk=chunk, softcap=None, scale=6.0)
    j = 2 * chunk + min(1, chunk - 1)
    n = 4 * chunk + 3
    got, want = attention_alone(desc, torch.float32, n, 4, [j + 1] + [1] * n if decode else [n], tweak=standout(j))
    assert rel(got, want) < 3e-5
    edges = (2 * chunk - 1, 2 * chunk, j, 3 * chunk - 1, 3 * chunk, 3 * chunk + 1)
    for r in edges:
        assert rel(got[r], want[r]) < 3e-5
    if chunk > 2:
        assert rel(got[3 * chunk - 1], got[j]) < 1e-3 and rel(got[3 * chunk], got[j]) > 1e-2       # seen to the chunk's end, not beyond
    for other in (chunk + 1, max(1, chunk - 1)):
        if other != chunk:
            _, shifted = attention_alone(U.attn(heads=4, kv_heads=2, chunk=other, softcap=None, scale=6.0), torch.float32, n, 4, [n], tweak=standout(j))
            assert max(rel(shifted[r], want[r]) for r in edges) > 1e-2      # the test bites


@gpu
def test_score_cap_bites():
    hot = lambda c: U.attn(heads=4, kv_heads=2, chunk=50, scale=3.0, softcap=c)
    got, want = attention_alone(hot(1.5), torch.float32, 50, 8, [50])
    assert rel(got, want) < 3e-5
    _, uncapped = attention_alone(hot(None), torch.float32, 50, 8, [50])
    assert rel(uncapped, want) > 1e-2


@gpu
def test_far_key_among_hundreds_and_the_split_path():
    """token 3's key is the one every query looks for; 600 tokens later (one chunk, pages of 16) each decoded token still returns its
    value.  A single decoded token on a long range cuts the range into several parts."""
    from ktransformers_b200.operators.attention import softmax_attention_splits
    desc = U.attn(heads=4, kv_heads=2, chunk=4096, softcap=None, scale=6.0)
    assert softmax_attention_splits(4, 2, 600, 1) > 1
    got, want = attention_alone(desc, torch.float32, 600, 16, [590] + [1] * 10, tweak=standout(3))
    assert rel(got, want) < 3e-5 and rel(got[-10:], want[-10:]) < 3e-5
    assert rel(got[599], got[3]) < 1e-3
    got_b, _ = attention_alone(desc, torch.bfloat16, 600, 16, [590] + [1] * 10, tweak=standout(3))
    assert rel(got_b, want) < 4e-2


MMA_SHAPES = [U.attn(heads=4, kv_heads=2, dim=16, vdim=16, chunk=40), U.attn(heads=8, kv_heads=1, dim=32, vdim=48, chunk=33, softcap=1.5),
              U.attn(heads=6, kv_heads=2, dim=64, vdim=32, chunk=1000, softcap=None), U.attn(heads=20, kv_heads=1, dim=128, vdim=128, chunk=64), U.attn(heads=3, kv_heads=3, dim=48, vdim=16, chunk=1),
              U.attn(heads=40, kv_heads=2, dim=16, vdim=64, chunk=17)]


@gpu
@pytest.mark.parametrize("desc", MMA_SHAPES)
def test_tensor_core_attention_path(desc):
    """bf16 with head sizes that are multiples of 16: the tensor-core tiles against the restatement and against the CUDA-core kernel"""
    width = 32 if desc["mixer"]["dim"] * desc["mixer"]["kv_heads"] <= 32 else 160
    for portions in ([150], [70, 3, 2, 40, 1, 34], [130] + [1] * 20):
        got, want = attention_alone(desc, torch.bfloat16, 150, 16, portions, width=width)
        plain, _ = attention_alone(desc, torch.bfloat16, 150, 16, portions, width=width, tensor_path=False)
        assert rel(got, want) < 4e-2 and rel(got, plain) < 4e-2


@gpu
@pytest.mark.parametrize("chunk", [1, 2, 31, 32, 33, 64, 65, 100])
@pytest.mark.parametrize("decode", [False, True])
def test_tensor_core_chunk_edges_inside_and_between_key_tiles(chunk, decode):
    """(the keys that are not looked for score zero up to bf16 rounding of their rows, times the scale: rows that average over
    such keys carry a few percent of noise)"""
    desc = U.attn(heads=4, kv_heads=2, dim=16, vdim=16, chunk=chunk, softcap=None, scale=3.0)
    j = 2 * chunk + min(1, chunk - 1)
    n = 4 * chunk + 3
    got, want = attention_alone(desc, torch.bfloat16, n, 16, [j + 1] + [1] * n if decode else [n], tweak=standout(j), width=48)
    assert rel(got, want) < 6e-2
    edges = (2 * chunk - 1, 2 * chunk, j, 3 * chunk - 1, 3 * chunk, 3 * chunk + 1)
    for r in edges:
        assert rel(got[r], want[r]) < 6e-2
    for other in (chunk + 1, max(1, chunk - 1)):
        if other != chunk:
            _, shifted = attention_alone(U.attn(heads=4, kv_heads=2, dim=16, vdim=16, chunk=other, softcap=None, scale=3.0), torch.bfloat16, n, 16, [n], tweak=standout(j), width=48)
            assert max(rel(shifted[r], want[r]) for r in edges) > 0.2


@gpu
def test_tensor_core_attention_far_key_and_split_edges():
    desc = U.attn(heads=8, kv_heads=2, dim=32, vdim=32, chunk=2048, softcap=None, scale=4.0)
    got, want = attention_alone(desc, torch.bfloat16, 700, 64, [690] + [1] * 10, tweak=standout(5), width=96)
    assert rel(got, want) < 4e-2 and rel(got[-10:], want[-10:]) < 4e-2
    assert rel(got[699], got[5]) < 2e-2


# ------------------------------------------------------------------------------------------------ whole model (GPU)
@gpu
@pytest.mark.parametrize("dtype,tol", [("float32", F32_TOL), ("bfloat16", BF16_TOL)])
def test_prompt_decode_and_portions_agree_with_the_restatement(tmp_path, dtype, tol):
    cfg = U.config(MIXED, loop=(1, 3, 2))
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
    """head sizes that are multiples of 16: bf16 attention runs on the tensor-core tiles inside a whole model (grouped heads, a looped
    span, 150 tokens over several key tiles and chunks), whole, in portions and with a decoded tail"""
    layers = [(U.attn(heads=6, kv_heads=2, dim=32, vdim=48, chunk=40), U.dense(96)), (U.attn(heads=4, kv_heads=1, dim=16, vdim=16, chunk=64), U.moe(ff=32, experts=4, top=2, groups=2, keep=2)),
              (U.attn(heads=4, kv_heads=2, dim=16, vdim=48, chunk=33), None)]
    cfg = U.config(layers, width=64, vocab=90, loop=(0, 2, 2))
    eng, om = serve(tmp_path, cfg, "bfloat16", seed=3, max_tokens=512, max_slots=2, page_size=16)
    t = toks(150, 90, seed=9)
    want = oracle_logits(om, t)
    for k, sizes in enumerate(([150], [70, 3, 2, 40, 1, 34], [130] + [1] * 20)):
        assert rel_rows(run_steps(eng, cut(("m", k), t, sizes))[("m", k)], want) < BF16_TOL


@gpu
def test_residual_stream_after_every_layer_run(tmp_path):
    cfg = U.config(MIXED, loop=(0, 3, 3))
    eng, om = serve(tmp_path, cfg, "float32", max_tokens=64, max_slots=2, page_size=8)
    t = toks(11, seed=2)
    want, got = [], []
    om.forward(t, om.new_state(), want)
    eng.model(eng.cache.build_batch([("r", t, [])]), eng.cache, got)
    assert len(got) == len(want) == 10
    for a, b in zip(got, want):
        assert rel(a, b) < 1e-4


@gpu
def test_pass_openings_matter(tmp_path):
    """the restatement without the re-read embedding, or with the step vectors swapped, differs: the whole-model tests would catch
    a model that forgot either; a span that runs once adds its one step vector and no embedding"""
    cfg = U.config(MIXED, loop=(1, 3, 3))
    eng, om = serve(tmp_path, cfg, "float32", seed=1, max_tokens=64, max_slots=2, page_size=8)
    t = toks(20, seed=4)
    want = oracle_logits(om, t)
    assert rel(run_steps(eng, cut("a", t, [13, 2, 1]))["a"], want) < F32_TOL
    w = U.weights(cfg, 1, torch.float32)
    w["loop.step"] = w["loop.step"].flip(0).contiguous()
    assert rel(oracle_logits(O.Model(cfg, w, torch.float64), t), want) > 1e-3
    once = U.config(MIXED, loop=(1, 3, 1))
    eng1, om1 = serve(tmp_path, once, "float32", seed=2, max_tokens=64, max_slots=2, page_size=8)
    assert rel(run_steps(eng1, cut("b", t, [20]))["b"], oracle_logits(om1, t)) < F32_TOL
    no_loop = dict(once)
    del no_loop["loop"]
    assert rel(oracle_logits(O.Model(no_loop, U.weights(once, 2, torch.float32), torch.float64), t), oracle_logits(om1, t)) > 1e-3


@gpu
def test_other_sizes_and_layer_orders(tmp_path):
    cases = [
        ([(U.attn(heads=1, kv_heads=1, dim=2, vdim=2, chunk=3), U.dense(3))], dict(width=8)),                                                                     # one small layer
        ([(U.attn(heads=16, kv_heads=4, dim=12, vdim=10, chunk=12), U.moe(ff=20, experts=16, top=4, groups=4, keep=2)), (U.attn(heads=16, kv_heads=16, dim=3, vdim=9, chunk=30), None)] * 2,
         dict(width=72, vocab=31, loop=(1, 4, 2))),
        ([(U.attn(heads=5, kv_heads=5, dim=24, vdim=24, chunk=2), U.moe(ff=5, experts=3, top=3, groups=1, keep=1, scale=1.0)), (U.attn(heads=2, kv_heads=1, dim=8, vdim=8), U.dense(8))], dict(width=40, loop=(1, 2, 4))),
        ([(U.attn(), None), (U.attn(chunk=3, softcap=0.7), U.dense(16)), (U.attn(chunk=1), U.moe(experts=4, top=1, groups=4, keep=1))], dict(width=16, eps=1e-3, embed_scale=1.0, logit_softcap=None)),
        ([(U.attn(heads=2, kv_heads=2, dim=4, vdim=4, chunk=500), U.moe(ff=33, experts=10, top=2, groups=2, keep=2, limit=0.1))], dict(width=14, vocab=7, loop=(0, 1, 3)))]
    for k, (layers, kw) in enumerate(cases):
        cfg = U.config(layers, **kw)
        eng, om = serve(tmp_path, cfg, "float32", seed=10 + k, max_tokens=64, max_slots=2, page_size=8)
        t = toks(30, cfg["vocab"], seed=k)
        assert rel(run_steps(eng, cut("a", t, [13, 2, 1]))["a"], oracle_logits(om, t)) < F32_TOL


@gpu
@pytest.mark.parametrize("seed", range(8))
def test_drawn_configurations(tmp_path, seed):
    """sizes, layer order, loop and constants drawn per seed: one prompt whole, in uneven portions, and with a decoded tail"""
    r = random.Random(seed)
    width = r.choice([16, 40, 136, 320])
    layers = []
    for _ in range(r.randint(1, 5)):
        G = r.choice([1, 2, 4])
        m = U.attn(heads=G * r.choice([1, 2, 5, 9]), kv_heads=G, dim=r.choice([4, 6, 24, 64]), vdim=r.choice([5, 8, 80]), scale=r.choice([None, 0.11, 1.0]), softcap=r.choice([None, 0.5, 20.0]),
                   chunk=r.choice([1, 5, 31, 32, 33, 64, 100, 1000]))
        kind = r.random()
        if kind < 0.3:
            f = None
        elif kind < 0.6:
            f = U.dense(ff=r.choice([8, 100, 1030]))
        else:
            groups = r.choice([1, 2, 4])
            per = r.choice([2, 3, 8])
            keep = r.randint(1, groups)
            f = U.moe(ff=r.choice([8, 24, 100]), experts=groups * per, top=r.randint(1, min(keep * per, 6)), groups=groups, keep=keep, scale=r.choice([1.0, 2.0]), limit=r.choice([0.5, 1.5, 7.0]))
        layers.append((m, f))
    loop = None
    if r.random() < 0.7:
        start = r.randrange(len(layers))
        loop = (start, r.randint(start + 1, len(layers)), r.randint(1, 3))
    cfg = U.config(layers, vocab=r.choice([31, 77, 1000]), width=width, eps=r.choice([1e-6, 1e-5, 1e-3]), loop=loop, embed_scale=r.choice([1.0, 4.0, 12.5]), logit_softcap=r.choice([None, 5.0, 40.0]))
    eng, om = serve(tmp_path, cfg, "float32", seed=seed, max_tokens=256, max_slots=2, page_size=r.choice([4, 16, 64]))
    t = toks(r.choice([40, 90, 150]), cfg["vocab"], seed=seed)
    want = oracle_logits(om, t)
    for k, sizes in enumerate(([len(t)], [3, 17, 2, 1, 33, 2, 64], [len(t) - 20] + [1] * 20)):
        assert rel(run_steps(eng, cut(("d", k), t, sizes))[("d", k)], want) < F32_TOL


@gpu
def test_captured_decode_steps_in_a_large_cache(tmp_path):
    """decode steps replay a captured graph; the shift state rows flip between the replays, and a roomy cache changes nothing"""
    cfg = U.config(MIXED, loop=(0, 2, 2))
    eng, om = serve(tmp_path, cfg, "float32", max_tokens=8192, max_slots=2, page_size=16)
    for r, n in enumerate((40, 330)):
        t = toks(n, seed=40 + r)
        got = run_steps(eng, cut(("g", r), t, [n - 12] + [1] * 12))[("g", r)]
        assert rel(got, oracle_logits(om, t)) < F32_TOL
    assert 1 in eng._captured and eng._captured[1].graph is not None


@gpu
def test_unequal_requests_in_one_batch_equal_each_alone(tmp_path):
    cfg = U.config(MIXED, loop=(1, 3, 2))
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
    """pages of 4 and 2 slots: sequences come and go, pages and state rows are handed out again un-cleared, and a new sequence in a
    used slot must start from an empty shift state.  Every layer's mask is chunked, so the pages before the current chunk are given back
    while a sequence runs and its page table row wraps around."""
    layers = [(U.attn(chunk=9), U.dense()), (U.attn(heads=6, kv_heads=2, chunk=21), U.moe()), (U.attn(heads=2, kv_heads=2, dim=8, vdim=8, chunk=4), None)]
    cfg = U.config(layers, loop=(0, 2, 2))
    eng, om = serve(tmp_path, cfg, "float32", max_tokens=48, max_slots=2, page_size=4)
    assert eng.cache.chunks == [4, 9, 21]
    for r in range(3):
        t = toks(150, seed=20 + r)                              # longer than the cache: only the current chunks' pages are held
        got = run_steps(eng, cut(("s", r), t, [6] + [1] * 144))[("s", r)]
        assert rel(got, oracle_logits(om, t)) < F32_TOL
        short = toks(3, seed=30 + r)
        assert rel(run_steps(eng, cut(("t", r), short, [3]))[("t", r)], oracle_logits(om, short)) < F32_TOL
    assert len(eng.cache._free_pages) == eng.cache.num_pages and len(eng.cache._free_slots) == 2


@gpu
def test_greedy_generation_through_the_scheduler_and_the_command_line(tmp_path, capsys):
    from ktransformers_b200 import local_chat
    cfg = U.config(MIXED, loop=(1, 3, 2))
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
    cfg = U.config(MIXED, vocab=41, loop=(0, 2, 2))
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
