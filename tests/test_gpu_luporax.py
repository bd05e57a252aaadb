"""Luporax: every mechanism alone against the plain functions of ``plain_luporax``, then whole
models of several shapes replayed whole, decoded, in portions and mixed, and greedy generation
through the engine's own entry point."""

import json
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_luporax as plain
import trace_tools

pytestmark = pytest.mark.gpu

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def dev(a, dtype=torch.float32):
    return torch.as_tensor(np.ascontiguousarray(a)).to(dtype).cuda()


def host(t):
    return t.double().cpu().numpy()


def tol(dtype, scale=1.0):
    return (2e-5 if dtype == "float32" else 2e-2) * scale


# ------------------------------------------------------------------ configs --

def moe(experts, top, ff, limit, sff, slimit):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit},
            "shared": {"ff": sff, "limit": slimit}}


def attention(heads, kv, dim, vdim, dims, base, scale, cap, mlp):
    return {"type": "attention", "mlp": mlp, "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim,
                                                       "rot": {"dims": dims, "base": base}, "scale": scale, "softcap": cap}}


def mingru(width, mlp):
    return {"type": "mingru", "mlp": mlp, "mixer": {"width": width}}


def rglru(width, blocks, conv, mlp):
    return {"type": "rglru", "mlp": mlp, "mixer": {"width": width, "blocks": blocks, "conv": conv}}


def again(layer, j):
    return {**layer, "weights_of": j}


# A: multipliers of 1, fewer rotated dimensions than the head holds, values narrower than keys, a
# layer without feed-forward, odd sizes, layers that run twice (one of each cache kind).
_A0 = attention(4, 2, 20, 12, 8, 10000.0, 0.2, 20.0, moe(5, 2, 40, 2.0, 24, 1.0))
_A1 = mingru(100, None)
_A2 = rglru(96, 3, 3, moe(4, 1, 36, 1.5, 50, 3.0))
CONFIG_A = {"architecture": "Luporax", "vocab": 211, "width": 72, "norm": {"eps": 1e-5}, "residual_mult": 1.0,
            "logit_scale": 1.0, "layers": [_A0, _A1, _A2, again(_A0, 0), again(_A2, 2), again(_A1, 1)]}
# B: a recurrent layer first, one block and one tap (no convolution state), a minGRU as wide as the
# model, every head with keys of its own, values wider than keys, all dimensions rotated, every expert chosen.
CONFIG_B = {"architecture": "Luporax", "vocab": 130, "width": 64, "norm": {"eps": 1e-6}, "residual_mult": 0.6,
            "logit_scale": 0.3,
            "layers": [rglru(64, 1, 1, moe(3, 3, 30, 2.5, 16, 2.0)), mingru(64, moe(9, 2, 24, 2.0, 8, 1.5)),
                       attention(3, 3, 16, 40, 16, 500.0, 0.3, 5.0, None), rglru(40, 5, 6, None)]}
# C: sizes of the tensor-core kernels (heads of 64, one key/value head for eight query heads, widths in
# multiples of 8), sixteen experts of which four are chosen.
_C0 = attention(8, 1, 64, 64, 32, 20000.0, 0.11, 25.0, moe(16, 4, 64, 2.5, 120, 1.25))
CONFIG_C = {"architecture": "Luporax", "vocab": 300, "width": 128, "norm": {"eps": 1e-6}, "residual_mult": 0.5,
            "logit_scale": 0.2, "layers": [_C0, rglru(192, 3, 4, moe(16, 4, 64, 2.5, 120, 1.25)), mingru(160, None), again(_C0, 0)]}
CONFIGS = {"A": CONFIG_A, "B": CONFIG_B, "C": CONFIG_C}
LENGTHS = {"A": [1, 2, 19, 77, 150], "B": [3, 33, 64, 129], "C": [5, 48, 100, 300]}
PAGE = {"A": 16, "B": 8, "C": 16}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    base = tmp_path_factory.mktemp("luporax")
    out = {}
    for tag, cfg in CONFIGS.items():
        tensors = plain.random_tensors(cfg, seed=40 + ord(tag))
        folder = plain.write_folder(base / tag, cfg, tensors)
        rs = np.random.RandomState(ord(tag))
        reqs = {f"{tag.lower()}{i}": rs.randint(0, cfg["vocab"], n).tolist() for i, n in enumerate(LENGTHS[tag])}
        t64 = {k: v.astype(np.float64) for k, v in tensors.items()}
        want = {rid: oracle(cfg, t64, toks) for rid, toks in reqs.items()}
        out[tag] = (folder, cfg, t64, reqs, want)
    return out


class Logits(np.ndarray):
    """Logits [T, V] with ``close``: the places where a router's choice was a close call."""


def oracle(cfg, t64, toks):
    margins = []
    out = plain.forward(cfg, t64, toks, margins=margins).view(Logits)
    out.close = np.min(np.stack(margins), axis=0) < 0.02 if margins else np.zeros(len(toks), dtype=bool)
    return out


def limit(dtype, want):
    if dtype == "float32":
        return 1e-4
    return 0.03 * max(float(np.abs(w).max()) for w in want.values())


def replay(folder, dtype, trace, page_size, max_tokens=None):
    from ayaka_py_b200.replay import ReplaySession
    session = ReplaySession(folder, dtype, max_tokens or trace_tools.tokens_needed(trace), page_size)
    outputs = []
    for record in trace:
        logits = session.step(record)
        outputs.append(None if logits is None or logits.shape[0] == 0 else logits.cpu().numpy())
    session.cache.assert_clean()
    return outputs, session


def check(models, tag, dtype, trace, want=None, folder=None, **kw):
    """In 32-bit every position must agree.  In bfloat16 rounding can turn a router's close call, which
    moves that position's logits visibly and the ones after it a little: the places that the plain model
    marks as close calls are not compared, and of the others at most 2 in 100 may differ, which a lost
    state, a wrong page or a wrong edge would exceed at once."""
    folder = folder or models[tag][0]
    want = want or models[tag][4]
    outputs, session = replay(folder, dtype, trace, PAGE[tag], **kw)
    got = trace_tools.collect(trace, outputs)
    if dtype == "float32":
        bad = trace_tools.first_difference(got, want, limit(dtype, want))
        assert bad is None, f"first wrong place: request {bad[0]} position {bad[1]} |diff| {bad[2]:.3e}"
        return session
    over, total, first = 0, 0, None
    for rid, rows in want.items():
        for p in range(rows.shape[0]):
            assert p in got.get(rid, {}), f"request {rid} position {p} was not answered"
            if rows.close[p]:
                continue
            d = float(np.abs(got[rid][p] - np.asarray(rows[p])).max())
            total += 1
            if not d <= limit(dtype, want):
                over += 1
                first = first or (rid, p, d)
    assert over <= 0.02 * total, f"{over} of {total} places differ; the first: request {first[0]} position {first[1]} |diff| {first[2]:.3e}"
    return session


# ---------------------------------------------------------- a step context --

def context_for(groups, dtype, max_requests=4, page_size=8, pages=64, positions=1024):
    from ayaka_py_b200.cache import CacheManager
    from ayaka_py_b200.engine.step import StepRunner
    cache = CacheManager(groups, kv_pages=pages, page_size=page_size, max_requests=max_requests, max_len=positions,
                         dtype=DT[dtype], device="cuda")
    model = SimpleNamespace(device="cuda", dtype=DT[dtype], max_positions=positions, vocab_size=10)
    return cache, StepRunner(model, cache, max_tokens=positions)


def step_of(cache, runner, counts):
    """A reserved step in which request i brings counts[i] tokens."""
    from ayaka_py_b200.engine.step import StepEntry
    entries = []
    for i, n in counts.items():
        slot = cache.slot_of.get(i)
        if slot is None:
            slot = cache.open(i)
        entries.append(StepEntry(slot, int(cache.length[slot]), [0] * n, []))
    res = cache.reserve([(e.slot, e.start, len(e.tokens)) for e in entries])
    return runner.prepare(entries), res


def run_cut(cache, runner, rows, cuts, fn):
    """Feeds rows[i] (one array per request) in portions: cuts is a list of {request: count} steps;
    fn(ctx, packed rows of the step) returns the step's output rows.  Gives back per-request outputs."""
    at = {i: 0 for i in rows}
    got = {i: [] for i in rows}
    for counts in cuts:
        ctx, res = step_of(cache, runner, counts)
        order = [int(i) for i in ctx.host["order"]]
        ids = list(counts)
        packed = [ids[k] for k in order]
        x = torch.cat([rows[i][at[i]:at[i] + counts[i]] for i in packed])
        y = fn(ctx, x)
        a = 0
        for i in packed:
            got[i].append(y[a:a + counts[i]].float().cpu().numpy())
            a += counts[i]
            at[i] += counts[i]
        cache.commit(res)
    return {i: np.concatenate(v) for i, v in got.items()}


def cuts_for(lengths, sizes):
    out, k = [], 0
    for i, n in lengths.items():
        p = 0
        while p < n:
            c = min(sizes[k % len(sizes)], n - p)
            out.append({i: c})
            p += c
            k += 1
    return out


PLANS = [lambda L: cuts_for(L, [1000]), lambda L: cuts_for(L, [1]), lambda L: cuts_for(L, [2, 1, 3, 5, 2, 2, 1, 8, 70]),
         lambda L: [{0: 5, 1: 1}, {0: 1, 1: 2, 2: L[2]}, {0: 2, 1: 1}, {0: L[0] - 8, 1: L[1] - 4}]]


def layer_tensors(layer, d, seed, prefix="l0.mix."):
    cfg = {"vocab": 4, "width": d, "layers": [layer]}
    t = plain.random_tensors(cfg, seed)
    return {k: v.astype(np.float64) for k, v in t.items()}, {k[len(prefix):]: v for k, v in t.items() if k.startswith(prefix)}


def bind(part, tensors, names, dtype):
    decl = part.tensors()
    part.bind({names[k]: dev(v, DT[dtype] if decl[names[k]].kind == "matrix" else torch.float32) for k, v in tensors.items()})


def mixer_alone(part, binding_need, dtype, d, want_fn, lengths, scale=1.0, seed=5, rows=None):
    """A mixer part over several requests, cut four ways (whole, token by token, ragged, batched with
    unequal requests), and once more in slots that were used before."""
    from ayaka_py_b200.cache import CacheBinding, CacheGroupSpec
    rs = np.random.RandomState(seed)
    xs = rows or {i: plain.round_bf16(rs.randn(n, d).astype(np.float32)) for i, n in lengths.items()}
    want = {i: want_fn(x.astype(np.float64)) for i, x in xs.items()}
    big = max(float(np.abs(w).max()) for w in want.values())
    rows_d = {i: dev(x, DT[dtype]) for i, x in xs.items()}
    binding = CacheBinding(0, "g", 0, True)
    fn = lambda ctx, x: part.forward(x.contiguous(), None, ctx, binding)
    for plan in PLANS:
        cache, runner = context_for([CacheGroupSpec("g", binding_need, 1)], dtype, max_requests=3, page_size=8, pages=96)
        got = run_cut(cache, runner, rows_d, plan(lengths), fn)
        for i in lengths:
            assert np.abs(got[i] - want[i]).max() < tol(dtype, 3 * big * scale), (i, float(np.abs(got[i] - want[i]).max()))
        for i in list(cache.slot_of):
            cache.close(cache.slot_of[i])
        got = run_cut(cache, runner, rows_d, cuts_for(lengths, [4, 1, 33]), fn)      # slots and pages used again
        for i in lengths:
            assert np.abs(got[i] - want[i]).max() < tol(dtype, 3 * big * scale)
    return want


# ------------------------------------------------------- mechanisms alone --

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("d", [7, 64, 300])
def test_token_shift_whole_in_portions_batched_and_in_used_slots(dtype, d):
    from ayaka_py_b200.cache import CacheBinding, CacheGroupSpec
    from ayaka_py_b200.parts import PartSpec, make_part
    rs = np.random.RandomState(1)
    part = make_part(PartSpec("token_shift", {"width": d}), DT[dtype], "cuda")
    mu = (0.5 + 0.3 * rs.randn(d)).astype(np.float32)
    part.bind({"weight": dev(mu)})
    lengths = {0: 23, 1: 9, 2: 14}
    xs = {i: rs.randn(n, d).astype(np.float32) for i, n in lengths.items()}
    want = {i: plain.token_shift(x.astype(np.float64), mu.astype(np.float64)) for i, x in xs.items()}
    binding = CacheBinding(0, "g", 0, True)
    fn = lambda ctx, x: part.forward(x.contiguous(), ctx, binding)
    for plan in PLANS:
        cache, runner = context_for([CacheGroupSpec("g", part.cache_need(), 1)], dtype, max_requests=3)
        got = run_cut(cache, runner, {i: dev(x) for i, x in xs.items()}, plan(lengths), fn)
        for i in lengths:
            assert np.abs(got[i] - want[i]).max() < tol(dtype, 4)
        for i in list(cache.slot_of):
            cache.close(cache.slot_of[i])
        got = run_cut(cache, runner, {i: dev(x) for i, x in xs.items()}, cuts_for(lengths, [3, 1]), fn)
        for i in lengths:
            assert np.abs(got[i] - want[i]).max() < tol(dtype, 4)       # the first token sees zeros again
    assert torch.equal(part.convert(dev(xs[0])), dev(xs[0]).to(DT[dtype]))


def test_norm_weight_stored_around_zero_and_scaled_head():
    from ayaka_py_b200.parts import PartSpec, make_part
    rs = np.random.RandomState(2)
    d, V = 40, 24
    x, w = rs.randn(5, d).astype(np.float32) * 3, (0.2 * rs.randn(d)).astype(np.float32)
    norm = make_part(PartSpec("rmsnorm", {"width": d, "eps": 1e-5, "offset": 1.0, "out_scale": 0.7}), torch.float32, "cuda")
    stored = dev(w)
    norm.bind({"weight": stored})
    assert torch.equal(stored, dev(w))                                   # the checkpoint's tensor is left alone
    want = plain.norm_one_plus(x.astype(np.float64), w.astype(np.float64), 1e-5)
    base = rs.randn(5, d).astype(np.float32)
    assert np.abs(host(norm.add_normed(dev(base), dev(x))) - (base + 0.7 * want)).max() < 2e-5
    table = plain.round_bf16(rs.randn(V, d).astype(np.float32))
    for dtype in ("float32", "bfloat16"):
        head = make_part(PartSpec("lm_head", {"vocab": V, "width": d, "scale": 0.3}), DT[dtype], "cuda")
        head.bind({"weight": dev(table, DT[dtype])})
        h = plain.round_bf16(rs.randn(3, d).astype(np.float32))
        got = head.forward(dev(h, DT[dtype]), None)
        assert np.abs(host(got) - 0.3 * (h.astype(np.float64) @ table.astype(np.float64).T)).max() < 1e-4


def test_rotary_in_halves():
    from ayaka_py_b200.parts import PartSpec, make_part
    rs = np.random.RandomState(3)
    dims, head, heads, base = 12, 20, 3, 5000.0
    rot = make_part(PartSpec("rotary", {"dims": dims, "base": base, "layout": "halves"}), torch.float32, "cuda")
    x = rs.randn(4, heads * head).astype(np.float32)
    positions = np.array([0, 1, 63, 700])
    t = dev(x)
    rot.rotate(t, torch.tensor(positions, dtype=torch.int32, device="cuda"), heads, head)
    want = plain.rotate_half(x.astype(np.float64).reshape(4, heads, head), positions, dims, base).reshape(4, -1)
    assert np.abs(host(t) - want).max() < 1e-4 and np.abs(host(t)[:3] - want[:3]).max() < 2e-5


MINGRU_NAMES = {"z": "z_weight", "z.b": "z_bias", "x": "x_weight", "x.b": "x_bias", "g": "g_weight", "o": "out_weight"}
RGLRU_NAMES = {"y": "y_weight", "y.b": "y_bias", "x": "x_weight", "x.b": "x_bias", "conv": "conv_weight", "conv.b": "conv_bias",
               "ra": "ra_weight", "ra.b": "ra_bias", "ri": "ri_weight", "ri.b": "ri_bias", "lam": "lam", "o": "out_weight"}
ATTN_NAMES = {"q": "q_weight", "q.b": "q_bias", "k": "k_weight", "k.b": "k_bias", "v": "v_weight", "v.b": "v_bias",
              "q.norm": "q_norm", "k.norm": "k_norm", "pb": "head_bias", "o": "out_weight"}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("d,W", [(48, 100), (40, 40), (64, 33)])
def test_mingru_alone(dtype, d, W):
    from ayaka_py_b200.parts import PartSpec, make_part
    layer = mingru(W, None)
    t64, w = layer_tensors(layer, d, 7)
    part = make_part(PartSpec("mingru", {"width": d, "inner": W}), DT[dtype], "cuda")
    bind(part, w, MINGRU_NAMES, dtype)
    mixer_alone(part, part.cache_need(), dtype, d, lambda h: plain.mingru(h, t64, "l0.mix.", layer["mixer"]),
                {0: 150, 1: 9, 2: 70})


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("d,W,blocks,taps", [(48, 96, 3, 4), (40, 40, 1, 1), (64, 70, 5, 2), (32, 64, 4, 9)])
def test_rglru_alone_with_its_convolution_state(dtype, d, W, blocks, taps):
    from ayaka_py_b200.parts import PartSpec, make_part
    layer = rglru(W, blocks, taps, None)
    t64, w = layer_tensors(layer, d, 8)
    part = make_part(PartSpec("rglru", {"width": d, "inner": W, "blocks": blocks, "taps": taps}), DT[dtype], "cuda")
    bind(part, w, RGLRU_NAMES, dtype)
    mixer_alone(part, part.cache_need(), dtype, d, lambda h: plain.rglru(h, t64, "l0.mix.", layer["mixer"]),
                {0: 150, 1: 9, 2: 70})


def test_recurrences_remember_for_hundreds_of_tokens_and_forget_at_once():
    """Decays next to one (a large negative lam; an update gate that stays shut) keep the first token's
    input alive over 600 tokens, in one portion and decoded; decays next to zero drop it at once."""
    from ayaka_py_b200 import ops
    from ayaka_py_b200.cache import CacheGroupSpec
    from ayaka_py_b200.parts import StateNeed
    W, n = 40, 600
    for lam, keeps in ((-12.0, True), (6.0, False)):
        outs = []
        for cuts in ([n], [1] * n, [70, 2, 500, 28]):
            cache, runner = context_for([CacheGroupSpec("g", StateNeed((2, W)), 1)], "float32", max_requests=2)
            state = cache.state_layer(0, 0)
            got, at = [], 0
            for c in cuts:
                ctx, res = step_of(cache, runner, {0: c})
                T = ctx.num_rows
                proj = torch.zeros(T, W, device="cuda") + 3.0           # gelu(3) ~ 3
                u = torch.zeros(T, W, device="cuda")
                if at == 0:
                    u[0] = 5.0
                gates = torch.zeros(T, 1, 2 * W, device="cuda")
                got.append(ops.rglru_scan(proj, u, gates, torch.zeros(2 * W, device="cuda"), torch.full((W,), lam, device="cuda"),
                                          state, ctx, W, 1, 8.0, torch.float32))
                cache.commit(res)
                at += c
            outs.append(torch.cat(got))
        a = np.exp(-8.0 * 0.5 * np.log1p(np.exp(lam)))
        want = np.sqrt(1 - a * a) * 0.5 * 5.0 * a ** np.arange(n) * plain.gelu_tanh(3.0)
        for o in outs:
            assert np.abs(host(o)[:, 0] - want).max() < 2e-5 * max(1.0, want.max())
        assert (want[-1] > 0.5 * want[0]) == keeps and (keeps or want[1] < 1e-6)


def standing_out_rows(rs, n, d, places):
    """Random rows, and at ``places`` one common row: with equal query and key matrices those places
    score high against one another and everything else scores around zero."""
    x = plain.round_bf16(rs.randn(n, d).astype(np.float32))
    x[places] = plain.round_bf16(rs.randn(d).astype(np.float32))
    return x


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,D,Dv,dims,cap", [(4, 2, 20, 12, 8, 20.0), (3, 3, 16, 40, 16, 6.0), (8, 1, 64, 64, 32, 30.0),
                                              (2, 1, 64, 64, 64, 12.0)])
def test_sigmoid_attention_alone_with_keys_that_stand_out(dtype, H, G, D, Dv, dims, cap):
    """Keys that dominate (weight near one among hundreds near sigmoid of the head's negative bias) sit at
    the first token, around page borders and hundreds of tokens back; the queries that match them sit just
    before them (must not see them), on them and after them.  Whole, in portions, decoded, batched."""
    from ayaka_py_b200.parts import PartSpec, make_part
    rs = np.random.RandomState(9)
    d, P = 48, 8
    layer = attention(H, G, D, Dv, dims, 10000.0, 4.0 / np.sqrt(H * D) * np.sqrt(H), cap, None)
    t64, w = layer_tensors(layer, d, 11)
    # keys equal to the queries of their group's first head; no biases, so that equal inputs give equal rows
    per = H // G
    w["k"] = np.concatenate([w["q"][g * per * D:(g * per + 1) * D] for g in range(G)])
    w["q.b"][:], w["k.b"][:] = 0, 0
    w["q.norm"][:], w["k.norm"][:] = 1, 1
    w["pb"][:] = -6.0
    for k, v in w.items():
        t64["l0.mix." + k] = v.astype(np.float64)
    layer["mixer"]["scale"] = float(8.0 * np.sqrt(H * D) / D)        # equal rows score about 8 G / H .. 8
    part = make_part(PartSpec("sigmoid_attention", {"width": d, "heads": H, "kv_heads": G, "dim": D, "vdim": Dv,
                                                    "scale": layer["mixer"]["scale"], "softcap": cap, "eps": 1e-5,
                                                    "rot": layer["mixer"]["rot"]}), DT[dtype], "cuda")
    bind(part, w, ATTN_NAMES, dtype)
    lengths = {0: 330, 1: 9, 2: 70}
    places = {0: [0, 2, P - 1, P, P + 1, 5 * P - 1, 5 * P, 300, 301, 329], 1: [0, 8], 2: [3, 2 * P, 69]}
    rows = {i: standing_out_rows(rs, n, d, places[i]) for i, n in lengths.items()}
    want = mixer_alone(part, part.cache_need(), dtype, d,
                       lambda h: plain.sigmoid_attention(h, t64, "l0.mix.", layer["mixer"], 1e-5), lengths, rows=rows)
    # the test has teeth: a matching query's output differs visibly from its neighbour's
    assert np.abs(want[0][300] - want[0][299]).max() > 0.05 * np.abs(want[0]).max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("d,E,top,ff,sff", [(48, 5, 2, 40, 24), (64, 3, 3, 30, 16), (40, 9, 1, 36, 50), (128, 16, 4, 64, 128),
                                            (64, 40, 8, 16, 8)])
def test_mixture_of_experts_alone(dtype, d, E, top, ff, sff):
    """Few rows (most experts idle), and more rows than a tile holds per expert; every row is checked, so a
    wrong expert, a wrong weight or a dropped pair shows."""
    from ayaka_py_b200.parts import PartSpec, make_part
    rs = np.random.RandomState(13)
    layer = mingru(8, moe(E, top, ff, 1.5, sff, 2.5))
    t64, w = layer_tensors(layer, d, 17, prefix="l0.mlp.")
    w["router"] = plain.round_bf16(w["router"] * 4.0)                  # clear choices
    t64["l0.mlp.router"] = w["router"].astype(np.float64)
    part = make_part(PartSpec("moe", {"width": d, "experts": E, "top": top, "inner": ff, "limit": 1.5, "shared_inner": sff,
                                      "shared_limit": 2.5}), DT[dtype], "cuda")
    names = {"router": "router_weight", "shared.gate": "shared_gate", "shared.up": "shared_up", "shared.down": "shared_down",
             "shared.sg": "shared_mix"}
    for e in range(E):
        names.update({f"e{e}.gate": f"gate_{e}", f"e{e}.up": f"up_{e}", f"e{e}.down": f"down_{e}"})
    bind(part, w, names, dtype)
    for n in (1, 3, 260):
        h = plain.round_bf16(rs.randn(n, d).astype(np.float32) * 1.5)
        want = plain.moe(h.astype(np.float64), t64, "l0.mlp.", layer["mlp"])
        got = part.forward(dev(h, DT[dtype]), None, None)
        assert got.dtype == torch.float32
        assert np.abs(host(got) - want).max() < tol(dtype, 3 * float(np.abs(want).max()))
    base = rs.randn(n, d).astype(np.float32)
    got = part.forward(dev(h, DT[dtype]), dev(base), None)
    assert np.abs(host(got) - (base + want)).max() < tol(dtype, 3 * float(np.abs(want).max()))


# ------------------------------------------------- the faster kernels against the plain ones --

@pytest.mark.parametrize("H,G,D,Dv,P", [(8, 1, 64, 64, 16), (6, 2, 64, 64, 16), (4, 4, 128, 128, 16), (3, 1, 64, 128, 8),
                                        (2, 2, 128, 64, 32), (5, 5, 32, 32, 16), (4, 2, 16, 16, 16)])
def test_tensor_core_sigmoid_attention_against_the_32_bit_pipes(H, G, D, Dv, P):
    """Prompts, portions on top of a cached context, single rows (whose context is cut into partitions
    and added up), all in one cache: both kernels read the same pages."""
    from ayaka_py_b200 import ops
    from ayaka_py_b200.cache import CacheGroupSpec
    from ayaka_py_b200.parts import KVNeed
    cache, runner = context_for([CacheGroupSpec("g", KVNeed(G, D, None, G, Dv), 1)], "bfloat16", max_requests=4,
                                page_size=P, pages=2048 // P, positions=1024)
    kp, vp = cache.kv_layer(0, 0)
    gen = torch.Generator(device="cuda").manual_seed(1)
    kp.copy_(torch.randn(kp.shape, generator=gen, device="cuda"))
    vp.copy_(torch.randn(vp.shape, generator=gen, device="cuda"))
    bias = torch.linspace(-3.0, -1.0, H, device="cuda")
    for plan in ({0: 500, 1: 33, 2: 1}, {0: 7, 2: 130}, {0: 1, 1: 1, 2: 1}, {1: 1}, {0: 64, 1: 1, 2: 1, 3: 17}, {3: 300}):
        ctx, res = step_of(cache, runner, plan)
        q = (torch.randn(ctx.num_rows, H * D, generator=gen, device="cuda") * 0.5).to(torch.bfloat16)
        for cap in (0.0, 3.0):
            a = ops.sigmoid_attention(q, kp, vp, ctx.tables[0], ctx, H, 0.2, cap, bias, tensor_cores=False)
            b = ops.sigmoid_attention(q, kp, vp, ctx.tables[0], ctx, H, 0.2, cap, bias, tensor_cores=True)
            assert not torch.isnan(b.float()).any()
            assert float((a.float() - b.float()).abs().max()) < 0.01 * float(a.float().abs().max()) + 1e-3, (plan, cap)
        cache.commit(res)


@pytest.mark.parametrize("d,E,top,ff,T", [(128, 16, 2, 64, 6), (64, 4, 3, 128, 40), (256, 8, 1, 96, 300)])
def test_the_experts_products_agree_on_every_path(d, E, top, ff, T):
    """bfloat16: the grouped tcgen05 form (pairs padded to 128-row tiles per expert), the pair-by-pair
    matrix-vector kernel, the mma.sync tiles and the FP32 pipes (on float32 copies) from one routing."""
    from ayaka_py_b200 import ops
    gen = torch.Generator(device="cuda").manual_seed(21)
    h = torch.randn(T, d, generator=gen, device="cuda").to(torch.bfloat16)
    w1 = (torch.randn(E, 2 * ff, d, generator=gen, device="cuda") / d ** 0.5).to(torch.bfloat16)
    w2 = (torch.randn(E, d, ff, generator=gen, device="cuda") / ff ** 0.5).to(torch.bfloat16)
    route = ops.moe_route(torch.randn(T, E, generator=gen, device="cuda") * 3, E, top)
    act = (1.5, 1.702)
    hidden32 = ops.moe_gemm(h.float(), w1.float(), route, glu=act, out_dtype=torch.float32)
    want = ops.moe_gemm(hidden32, w2.float(), route, glu=None, out_dtype=torch.float32)          # [T * top, d], pair by pair
    tiles = ops.moe_gemm(ops.moe_gemm(h, w1, route, glu=act, out_dtype=torch.bfloat16), w2, route, glu=None, out_dtype=torch.float32)
    by_pair = ops.moe_gemv(ops.moe_gemv(h, w1, route, glu=act), w2, route, glu=None)
    padded, rows = ops.moe_experts_tc(h, w1, w2, route, *act)
    scale = float(want.abs().max())
    for name, got in (("mma.sync tiles", tiles), ("pair by pair", by_pair), ("tcgen05 grouped", padded[rows.long()])):
        assert not torch.isnan(got).any(), name
        assert float((got - want).abs().max()) < 0.02 * scale, (name, float((got - want).abs().max()), scale)
    assert ops.tc_error() == 0


# --------------------------------------------------------------- whole models --

def test_layers_one_by_one_in_32_bit(models):
    """The residual stream after every layer run against the plain implementation."""
    from ayaka_py_b200.engine.step import StepEntry
    from ayaka_py_b200.replay import ReplaySession
    for tag in CONFIGS:
        folder, cfg, t64, reqs, _ = models[tag]
        toks = list(reqs.values())[2]
        after = []
        plain.forward(cfg, t64, toks, after)
        s = ReplaySession(folder, "float32", 256, PAGE[tag])
        slot = s.cache.open("x")
        res = s.cache.reserve([(slot, 0, len(toks))])
        ctx = s.runner.prepare([StepEntry(slot, 0, toks, [0])])
        x = s.model.embedding.forward(ctx, s.model.position)
        assert len(s.model.spec.order) == len(cfg["layers"])
        for i, (step, caches) in enumerate(zip(s.model.spec.order, s.model.bindings)):
            x = s.model.blocks[step.layer].forward(x, ctx, caches)
            assert np.abs(host(x) - after[i]).max() < 1e-4 * max(1.0, float(np.abs(after[i]).max())), (tag, i)
        s.cache.commit(res)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag", ["A", "B", "C"])
def test_each_request_alone_and_whole(models, tag, dtype):
    check(models, tag, dtype, trace_tools.whole(models[tag][3]))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag", ["A", "B", "C"])
def test_prefill_against_token_by_token_decoding(models, tag, dtype):
    check(models, tag, dtype, trace_tools.tail_decoded(models[tag][3], 40))
    few = dict(list(models[tag][3].items())[:3])
    check(models, tag, dtype, trace_tools.tail_decoded(few, 10_000), want={k: models[tag][4][k] for k in few})


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag", ["A", "B", "C"])
def test_portions_down_to_two_tokens(models, tag, dtype):
    check(models, tag, dtype, trace_tools.portions(models[tag][3]))
    check(models, tag, dtype, trace_tools.portions(models[tag][3], sizes=(2, 2, 1, 2, 3, 2)))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag", ["A", "B", "C"])
def test_mixed_batches_with_pages_and_slots_used_again(models, tag, dtype):
    reqs = dict(models[tag][3])
    extra = {f"{rid}+": toks[::-1] for rid, toks in reqs.items()}      # more requests than slots
    _, cfg, t64, _, want = models[tag]
    want = dict(want)
    want.update({rid: oracle(cfg, t64, toks) for rid, toks in extra.items()})
    reqs.update(extra)
    for seed in (0, 1):
        trace = trace_tools.mixed(reqs, seed=seed)
        assert max(len(s["entries"]) for s in trace) >= 3
        session = check(models, tag, dtype, trace, want=want)
        assert any(g["reused"] > 0 for g in session.cache.stats()["groups"].values())
    longer = {rid: toks for rid, toks in reqs.items() if len(toks) >= 19}
    check(models, tag, dtype, trace_tools.reopened(longer, seed=3), want={rid: want[rid] for rid in longer})


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(models, dtype):
    folder, cfg, t64, _, _ = models["B"]
    toks = np.random.RandomState(11).randint(0, cfg["vocab"], 420).tolist()
    want = {"long": oracle(cfg, t64, toks)}
    check(models, "B", dtype, trace_tools.tail_decoded({"long": toks}, 400), want=want)


def test_the_batch_does_not_change_a_request(models):
    """A request alone, cut one way, and the same request beside others, cut another way (32-bit)."""
    folder, cfg, _, reqs, _ = models["A"]
    alone = trace_tools.portions({"a4": reqs["a4"]}, sizes=(16, 1, 5))
    out_alone, _ = replay(folder, "float32", alone, 16)
    got_alone = trace_tools.collect(alone, out_alone)["a4"]
    both = trace_tools.mixed(reqs, seed=4)
    out_both, _ = replay(folder, "float32", both, 16)
    got_both = trace_tools.collect(both, out_both)["a4"]
    worst = max(float(np.abs(got_alone[p] - got_both[p]).max()) for p in got_alone)
    assert worst < 2e-5


# --------------------------------------------- the engine's own entry point --

@pytest.mark.parametrize("graphs", [True, False])
def test_greedy_generation_through_the_scheduler(models, graphs):
    from ayaka_py_b200.engine.llm import LLM
    from ayaka_py_b200.engine.request import StopCriteria
    from ayaka_py_b200.sampling.params import SamplingParams
    folder, cfg, t64, reqs, _ = models["A"]
    prompts = [reqs["a2"], reqs["a3"][:40], reqs["a0"], reqs["a3"][5:30], reqs["a1"], reqs["a4"][:70]]
    llm = LLM(folder, dtype="float32", kv_pages=24, page_size=16, max_requests=3, batch_tokens=48, prefill_chunk=20,
              max_model_len=128, decode_graph=graphs)
    results = llm.generate(prompts, SamplingParams(temperature=0.0), StopCriteria(max_tokens=12, ignore_eos=True))
    for prompt, result in zip(prompts, results):
        want = plain.greedy_generate(cfg, t64, prompt, 12)
        k = next((i for i, (a, b) in enumerate(zip(result.token_ids, want)) if a != b), None)
        if k is not None:                     # a near tie may turn a token
            logits = plain.forward(cfg, t64, prompt + want[:k])[-1]
            assert abs(logits[result.token_ids[k]] - logits[want[k]]) < 1e-3
        else:
            assert result.token_ids == want
    llm.engine.cache.assert_clean()


def test_bfloat16_generation_with_decode_graphs_equals_eager(models):
    from ayaka_py_b200.engine.llm import LLM
    from ayaka_py_b200.engine.request import StopCriteria
    from ayaka_py_b200.sampling.params import SamplingParams
    folder, cfg, _, reqs, _ = models["C"]
    prompts = [reqs["c1"], reqs["c0"], reqs["c2"][:33]]
    out = []
    for graphs in (True, False):
        llm = LLM(folder, dtype="bfloat16", kv_pages=40, page_size=16, max_requests=4, max_model_len=160, decode_graph=graphs)
        out.append([r.token_ids for r in llm.generate(prompts, SamplingParams(temperature=0.0),
                                                      StopCriteria(max_tokens=16, ignore_eos=True))])
    assert out[0] == out[1]


def test_random_weights_mode_and_command_line(tmp_path):
    """A folder written by the engine's own random-weights mode loads and generates from the command line."""
    import subprocess
    import sys
    from pathlib import Path
    from ayaka_py_b200.config.model import LuporaxConfig
    from ayaka_py_b200.weights import write_random_model
    folder = write_random_model(tmp_path / "m", LuporaxConfig.from_dict(CONFIG_B), seed=3)
    assert json.loads((folder / "config.json").read_text())["architecture"] == "Luporax"
    root = Path(__file__).resolve().parent.parent
    proc = subprocess.run([sys.executable, "-m", "ayaka_py_b200", "generate", str(folder), "--prompt-ids", "1,2,3,4,5",
                           "--max-tokens", "5", "--temperature", "0", "--ignore-eos", "--max-model-len", "64", "--kv-pages", "16"],
                          cwd=root, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    line = json.loads(proc.stdout.strip().splitlines()[-1])
    assert len(line["token_ids"]) == 5
