"""Rakalix: every mechanism alone against the plain functions of ``plain_rakalix``, then whole
models of several shapes replayed whole, decoded, in portions and mixed, and greedy generation
through the engine's own entry point."""

import json
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_rakalix as plain
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

ROT_PLAIN = {"dims": 8, "base": 10000.0}
ROT_SCALED = {"dims": 16, "base": 50000.0, "scaling": {"factor": 8.0, "original": 64, "fast": 16.0, "slow": 2.0}}


def latent(heads, dim, rot_dim, vdim, rank, rot, scale, ff):
    return {"type": "latent_attention", "mlp": None if ff is None else {"kind": "dense", "ff": ff},
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "rot": rot, "scale": scale}}


def recurrent(heads, dim, vdim, ff):
    return {"type": "hgrn2", "mlp": None if ff is None else {"kind": "dense", "ff": ff},
            "mixer": {"heads": heads, "dim": dim, "vdim": vdim}}


# A: no embedding scale, no residual multiplier, three taps, a layer without feed-forward, fewer
# rotated dimensions than the rotated part holds, an inner width that is no multiple of 8.
CONFIG_A = {"architecture": "Rakalix", "vocab": 211, "width": 72, "norm": {"eps": 1e-5}, "canon": {"taps": 3},
            "embedding": {"scale": 1.0}, "residual_mult": 1.0,
            "layers": [latent(3, 20, 12, 24, 40, ROT_PLAIN, 0.2, 100), recurrent(2, 10, 36, None),
                       latent(2, 8, 16, 40, 24, ROT_SCALED, 0.31, 56), recurrent(3, 24, 8, 100)]}
# B: one head, odd sizes, five taps, recurrent layer first, a latent wider than 64.
CONFIG_B = {"architecture": "Rakalix", "vocab": 130, "width": 64, "norm": {"eps": 1e-6}, "canon": {"taps": 5},
            "embedding": {"scale": 3.0}, "residual_mult": 0.7,
            "layers": [recurrent(1, 33, 70, 96), latent(5, 16, 16, 8, 96, ROT_SCALED, 0.25, 40), recurrent(4, 6, 6, 48)]}
# C: two taps, more heads than one block of the attention kernel serves, a recurrent head of 64 x 64.
CONFIG_C = {"architecture": "Rakalix", "vocab": 300, "width": 128, "norm": {"eps": 1e-6}, "canon": {"taps": 2},
            "embedding": {"scale": 8.0}, "residual_mult": 0.5,
            "layers": [latent(40, 8, 4, 8, 32, {"dims": 4, "base": 100.0}, 0.3, 64), recurrent(2, 64, 64, 256)]}
CONFIGS = {"A": CONFIG_A, "B": CONFIG_B, "C": CONFIG_C}
LENGTHS = {"A": [1, 2, 19, 77, 150], "B": [3, 33, 64, 129], "C": [5, 48, 100]}
PAGE = {"A": 16, "B": 8, "C": 16}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    base = tmp_path_factory.mktemp("rakalix")
    out = {}
    for tag, cfg in CONFIGS.items():
        tensors = plain.random_tensors(cfg, seed=20 + ord(tag))
        folder = plain.write_folder(base / tag, cfg, tensors)
        rs = np.random.RandomState(ord(tag))
        reqs = {f"{tag.lower()}{i}": rs.randint(0, cfg["vocab"], n).tolist() for i, n in enumerate(LENGTHS[tag])}
        t64 = {k: v.astype(np.float64) for k, v in tensors.items()}
        want = {rid: plain.forward(cfg, t64, toks) for rid, toks in reqs.items()}
        out[tag] = (folder, cfg, t64, reqs, want)
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
    folder = folder or models[tag][0]
    want = want or models[tag][4]
    outputs, session = replay(folder, dtype, trace, PAGE[tag], **kw)
    got = trace_tools.collect(trace, outputs)
    bad = trace_tools.first_difference(got, want, limit(dtype, want))
    assert bad is None, f"first wrong place: request {bad[0]} position {bad[1]} |diff| {bad[2]:.3e}"
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
    """A reserved step in which request i brings counts[i] tokens (0: left out)."""
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
    """Each request alone, in portions of the given sizes in turn."""
    out, k = [], 0
    for i, n in lengths.items():
        p = 0
        while p < n:
            c = min(sizes[k % len(sizes)], n - p)
            out.append({i: c})
            p += c
            k += 1
    return out


# ------------------------------------------------------- mechanisms alone --

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_rms_norm_gathered_strided_and_added(dtype):
    from ayaka_py_b200 import ops
    rs = np.random.RandomState(0)
    for d in (7, 64, 300):
        x, w = rs.randn(9, d).astype(np.float32) * 3, (1 + 0.2 * rs.randn(d)).astype(np.float32)
        want = plain.rms_norm(x.astype(np.float64), w, 1e-5)
        got = ops.rmsnorm(dev(x), dev(w), 1e-5, DT[dtype])
        assert np.abs(host(got) - want).max() < tol(dtype, 4)
        rows = torch.tensor([8, 0, 3], dtype=torch.int32, device="cuda")
        got = ops.rmsnorm(dev(x), dev(w), 1e-5, DT[dtype], rows=rows)
        assert np.abs(host(got) - want[[8, 0, 3]]).max() < tol(dtype, 4)
        wide = dev(np.concatenate([rs.randn(9, 5).astype(np.float32), x], axis=1))
        got = ops.rmsnorm(wide[:, 5:], dev(w), 1e-5, DT[dtype])
        assert np.abs(host(got) - want).max() < tol(dtype, 4)
        base = rs.randn(9, d).astype(np.float32)
        out = ops.rmsnorm_residual(dev(base), dev(x), dev(w), 1e-5, 0.3)
        assert np.abs(host(out) - (base + 0.3 * want)).max() < 2e-5


def test_rms_norm_of_tiny_rows_keeps_eps_inside_the_root():
    from ayaka_py_b200 import ops
    x = np.full((1, 16), 1e-4, dtype=np.float32)
    got = host(ops.rmsnorm(dev(x), None, 1e-6, torch.float32))
    assert np.allclose(got, 1e-4 / np.sqrt(1e-8 + 1e-6), rtol=1e-5)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_poly_norm(dtype):
    from ayaka_py_b200 import ops
    rs = np.random.RandomState(1)
    for n in (5, 100, 320):
        z = rs.randn(6, n).astype(np.float32) * 2
        coeff = np.array([0.7, -0.4, 0.25, 0.1], dtype=np.float32)
        want = plain.poly_norm(z.astype(np.float64), coeff, 1e-6)
        got = ops.polynorm(dev(z), dev(coeff), 1e-6, DT[dtype])
        assert np.abs(host(got) - want).max() < tol(dtype, 6)


@pytest.mark.parametrize("scaling", [None, ROT_SCALED["scaling"], {"factor": 4.0, "original": 1000, "fast": 32.0, "slow": 1.0}])
def test_rotary_frequencies_and_turning(scaling):
    from ayaka_py_b200.parts import PartSpec, make_part
    rs = np.random.RandomState(2)
    dims, head, heads, offset, base = 12, 20, 3, 6, 5000.0
    rot = make_part(PartSpec("rotary", {"dims": dims, "base": base, "scaling": scaling}), torch.float32, "cuda")
    f, gain = plain.rotary_frequencies(dims, base, scaling)
    assert np.allclose(host(rot.freq), f, rtol=1e-7) and abs(rot.gain - gain) < 1e-12
    x = rs.randn(5, heads * head + 2).astype(np.float32)
    positions = np.array([0, 1, 63, 700, 1500])
    t = dev(x)
    rot.rotate(t, torch.tensor(positions, dtype=torch.int32, device="cuda"), heads, head, offset)
    want = x.astype(np.float64).copy()
    for h in range(heads):
        a = h * head + offset
        want[:, a:a + dims] = plain.rotate(want[:, a:a + dims], positions, dims, base, scaling)
    assert np.abs(host(t) - want).max() < 5e-4 * gain       # 32-bit angles at position 1500
    assert np.abs(host(t)[:3] - want[:3]).max() < 2e-5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_rotary_as_the_position_encoding_of_the_paged_attention_part(dtype):
    """The rotation is a part of its own: the engine's multi-head attention takes it through the
    declared hook (grouped queries, fewer rotated dimensions than the head holds), whole and continued."""
    from ayaka_py_b200.cache import CacheBinding, CacheGroupSpec
    from ayaka_py_b200.parts import PartSpec, make_part
    rs = np.random.RandomState(12)
    d, H, Hkv, Dh, dims, base, scale = 48, 4, 2, 16, 12, 3000.0, 0.25
    part = make_part(PartSpec("attention", {"width": d, "num_heads": H, "kv_heads": Hkv, "head_dim": Dh, "scale": scale,
                                            "window": None, "bias": False}), DT[dtype], "cuda")
    rot = make_part(PartSpec("rotary", {"dims": dims, "base": base, "scaling": ROT_SCALED["scaling"]}), DT[dtype], "cuda")
    part.set_position(rot)
    wq = plain.bf16_round(rs.randn((H + 2 * Hkv) * Dh, d).astype(np.float32) / np.sqrt(d))
    wo = plain.bf16_round(rs.randn(d, H * Dh).astype(np.float32) / np.sqrt(H * Dh))
    part.bind({"qkv_weight": dev(wq, DT[dtype]), "out_weight": dev(wo, DT[dtype])})
    n = 45
    h = plain.bf16_round(rs.randn(n, d).astype(np.float32))
    qkv = h.astype(np.float64) @ wq.astype(np.float64).T
    pos = np.arange(n)
    q = plain.rotate(qkv[:, :H * Dh].reshape(n, H, Dh), pos, dims, base, ROT_SCALED["scaling"])
    k = plain.rotate(qkv[:, H * Dh:(H + Hkv) * Dh].reshape(n, Hkv, Dh), pos, dims, base, ROT_SCALED["scaling"])
    v = qkv[:, (H + Hkv) * Dh:].reshape(n, Hkv, Dh)
    o = np.zeros((n, H, Dh))
    for head in range(H):
        sc = q[:, head] @ k[:, head // (H // Hkv)].T * scale
        sc = np.where(np.tril(np.ones((n, n), dtype=bool)), sc, -np.inf)
        w = np.exp(sc - sc.max(axis=1, keepdims=True))
        o[:, head] = (w / w.sum(axis=1, keepdims=True)) @ v[:, head // (H // Hkv)]
    want = o.reshape(n, H * Dh) @ wo.astype(np.float64).T
    cache, runner = context_for([CacheGroupSpec("g", part.cache_need(), 1)], dtype, page_size=8)
    binding = CacheBinding(0, "g", 0, True)
    fn = lambda ctx, x: part.forward(x.contiguous(), torch.zeros(x.shape[0], d, device="cuda"), ctx, binding)
    got = run_cut(cache, runner, {0: dev(h, DT[dtype])}, cuts_for({0: n}, [17, 2, 1, 9, 16]), fn)[0]
    assert np.abs(got - want).max() < tol(dtype, 3 * float(np.abs(want).max()))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("taps,d", [(1, 40), (2, 30), (4, 40), (4, 35), (7, 264), (11, 48)])
def test_time_conv_whole_in_portions_and_batched(dtype, taps, d):
    """The convolution's state: portions shorter than the taps, single tokens, two requests in
    one step, a slot that is used again."""
    from ayaka_py_b200.cache import CacheBinding, CacheGroupSpec
    from ayaka_py_b200.parts import PartSpec, make_part
    rs = np.random.RandomState(3)
    eps = 1e-5
    conv = make_part(PartSpec("time_conv", {"width": d, "taps": taps}), DT[dtype], "cuda")
    norm = make_part(PartSpec("rmsnorm", {"width": d, "eps": eps}), DT[dtype], "cuda")
    w, g = rs.randn(d, taps).astype(np.float32) * 0.5, (1 + 0.1 * rs.randn(d)).astype(np.float32)
    conv.bind({"weight": dev(w)}); norm.bind({"weight": dev(g)})
    binding = CacheBinding(0, "g", 0, True)
    lengths = {0: 23, 1: 9, 2: 14}
    xs = {i: rs.randn(n, d).astype(np.float32) for i, n in lengths.items()}
    want = {i: plain.time_conv(plain.rms_norm(x.astype(np.float64), g, eps), w) for i, x in xs.items()}
    rows = {i: dev(x) for i, x in xs.items()}
    fn = lambda ctx, x: conv.forward(x.contiguous(), norm, ctx, binding)
    plans = [cuts_for(lengths, [100]), cuts_for(lengths, [1]), cuts_for(lengths, [2, 1, 3, 5, 2, 2, 1, 8]),
             [{0: 5, 1: 1}, {0: 1, 1: 2, 2: 14}, {0: 2, 1: 1}, {0: 15, 1: 5}]]
    for cuts in plans:
        cache, runner = context_for([CacheGroupSpec("g", conv.cache_need(), 1)], dtype, max_requests=3)
        got = run_cut(cache, runner, rows, cuts, fn)
        for i in lengths:
            assert np.abs(got[i] - want[i]).max() < tol(dtype, 8), (taps, i, len(cuts))
        # the same slots once more, after closing: the state starts at zero again
        for i in list(cache.slot_of):
            cache.close(cache.slot_of[i])
        got = run_cut(cache, runner, rows, cuts_for(lengths, [4, 1]), fn)
        for i in lengths:
            assert np.abs(got[i] - want[i]).max() < tol(dtype, 8)


def mixer_tensors(cfg_layer, d, seed):
    cfg = {"vocab": 4, "width": d, "canon": {"taps": 2}, "layers": [cfg_layer]}
    t = plain.random_tensors(cfg, seed)
    return {k[len("l0.mix."):]: v for k, v in t.items() if k.startswith("l0.mix.")}


LATENT_NAMES = {"q": "q_weight", "dkv": "down_weight", "dkv.norm": "down_norm", "uk": "uk_weight", "uv": "uv_weight",
                "g": "gate_weight", "o": "out_weight"}
HGRN2_NAMES = {"q": "q_weight", "f": "f_weight", "f.b": "f_bias", "lower": "lower", "v": "v_weight", "norm": "norm",
               "o": "out_weight"}


def bind(part, tensors, names, dtype):
    decl = part.tensors()
    part.bind({names[k]: dev(v, DT[dtype] if decl[names[k]].kind == "matrix" else torch.float32) for k, v in tensors.items()})


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("spec", [latent(3, 20, 12, 24, 40, ROT_PLAIN, 0.2, None), latent(1, 56, 24, 48, 72, ROT_SCALED, 0.1, None),
                                  latent(6, 8, 16, 4, 130, ROT_SCALED, 0.3, None)])
def test_latent_attention_alone_with_keys_that_stand_out(dtype, spec):
    """Rows of the input at chosen places are made large, so that their rotated key part
    dominates the scores of later queries: the first token, the places around page borders and
    a place hundreds of tokens back.  Whole, in portions (down to two tokens) and decoded."""
    from ayaka_py_b200.cache import CacheBinding, CacheGroupSpec
    from ayaka_py_b200.parts import PartSpec, make_part
    rs = np.random.RandomState(4)
    d, eps, P = 48, 1e-5, 8
    p = spec["mixer"]
    part = make_part(PartSpec("latent_attention", {"width": d, "heads": p["heads"], "dim": p["dim"], "rot_dim": p["rot_dim"],
                                                   "vdim": p["vdim"], "kv_rank": p["kv_rank"], "scale": p["scale"], "eps": eps,
                                                   "rot": p["rot"]}), DT[dtype], "cuda")
    w = mixer_tensors(spec, d, 7)
    bind(part, w, LATENT_NAMES, dtype)
    n = 300
    h = rs.randn(n, d).astype(np.float32)
    for place in (0, P - 1, P, P + 1, 37, 5 * P - 1, 5 * P):
        h[place] *= 12.0
    h = plain.bf16_round(h)
    want = plain.latent_attention(h.astype(np.float64), {k: v.astype(np.float64) for k, v in w.items()}, p, eps)
    rows = {0: dev(h, DT[dtype])}
    binding = CacheBinding(0, "g", 0, True)
    fn = lambda ctx, x: part.forward(x.contiguous(), None, ctx, binding)
    scale = float(np.abs(want).max())
    for cuts in (cuts_for({0: n}, [n]), cuts_for({0: n}, [7, 2, 64, 3, 2, 33, 100, 1]),
                 cuts_for({0: n}, [270] + [1] * 30), cuts_for({0: n}, [P] * 3 + [1] * (2 * P + 2) + [2, 9])):
        cache, runner = context_for([CacheGroupSpec("g", part.cache_need(), 1)], dtype, page_size=P)
        got = run_cut(cache, runner, rows, cuts, fn)[0]
        diff = np.abs(got - want).max(axis=1)
        assert diff.max() < tol(dtype, 3 * scale), f"first wrong row {int(np.argmax(diff > tol(dtype, 3 * scale)))}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("spec", [recurrent(2, 10, 36, None), recurrent(1, 33, 70, None), recurrent(3, 64, 64, None),
                                  recurrent(2, 130, 20, None)])
def test_hgrn2_alone_state_carried_and_slots_used_again(dtype, spec):
    from ayaka_py_b200.cache import CacheBinding, CacheGroupSpec
    from ayaka_py_b200.parts import PartSpec, make_part
    rs = np.random.RandomState(5)
    d, eps = 40, 1e-5
    p = spec["mixer"]
    part = make_part(PartSpec("hgrn2", {"width": d, "heads": p["heads"], "dim": p["dim"], "vdim": p["vdim"], "eps": eps}),
                     DT[dtype], "cuda")
    w = mixer_tensors(spec, d, 8)
    bind(part, w, HGRN2_NAMES, dtype)
    lengths = {0: 70, 1: 5, 2: 31}
    hs = {i: plain.bf16_round(rs.randn(n, d).astype(np.float32)) for i, n in lengths.items()}
    w64 = {k: v.astype(np.float64) for k, v in w.items()}
    want = {i: plain.hgrn2(h.astype(np.float64), w64, p, eps)[0] for i, h in hs.items()}
    rows = {i: dev(h, DT[dtype]) for i, h in hs.items()}
    binding = CacheBinding(0, "g", 0, True)
    fn = lambda ctx, x: part.forward(x.contiguous(), None, ctx, binding)
    scale = max(float(np.abs(v).max()) for v in want.values())
    cache, runner = context_for([CacheGroupSpec("g", part.cache_need(), 1)], dtype, max_requests=3)
    for cuts in (cuts_for(lengths, [100]), cuts_for(lengths, [1]), cuts_for(lengths, [17, 2, 16, 1, 3]),
                 [{0: 40, 1: 1, 2: 2}, {1: 1, 2: 29}, {0: 1, 1: 3}, {0: 29}]):
        got = run_cut(cache, runner, rows, cuts, fn)
        for i in lengths:
            assert np.abs(got[i] - want[i]).max() < tol(dtype, 3 * scale), (i, len(cuts))
        for i in list(cache.slot_of):          # the slots are used again by the next plan: their state must start at zero
            cache.close(cache.slot_of[i])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_hgrn2_long_memory(dtype):
    """Lower bounds near one: what was written 400 tokens ago still weighs; decoded one by one."""
    from ayaka_py_b200.cache import CacheBinding, CacheGroupSpec
    from ayaka_py_b200.parts import PartSpec, make_part
    rs = np.random.RandomState(6)
    d, eps, spec = 32, 1e-6, recurrent(2, 16, 24, None)
    p = spec["mixer"]
    part = make_part(PartSpec("hgrn2", {"width": d, "heads": 2, "dim": 16, "vdim": 24, "eps": eps}), DT[dtype], "cuda")
    w = mixer_tensors(spec, d, 9)
    w["lower"] = plain.bf16_round(np.full_like(w["lower"], 0.996))
    bind(part, w, HGRN2_NAMES, dtype)
    n = 450
    h = plain.bf16_round(rs.randn(n, d).astype(np.float32))
    h[3] *= 20
    want = plain.hgrn2(h.astype(np.float64), {k: v.astype(np.float64) for k, v in w.items()}, p, eps)[0]
    cache, runner = context_for([CacheGroupSpec("g", part.cache_need(), 1)], dtype)
    binding = CacheBinding(0, "g", 0, True)
    got = run_cut(cache, runner, {0: dev(h, DT[dtype])}, cuts_for({0: n}, [50] + [1] * 400),
                  lambda ctx, x: part.forward(x.contiguous(), None, ctx, binding))[0]
    assert np.abs(got - want).max() < tol(dtype, 3 * float(np.abs(want).max()))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_poly_norm_feed_forward_part(dtype):
    from ayaka_py_b200.parts import PartSpec, make_part
    rs = np.random.RandomState(10)
    d, ff, eps = 40, 100, 1e-6
    part = make_part(PartSpec("polynorm_mlp", {"width": d, "inner": ff, "eps": eps}), DT[dtype], "cuda")
    up, down = plain.bf16_round(rs.randn(ff, d) / 6), plain.bf16_round(rs.randn(d, ff) / 10)
    coeff = np.array([0.5, 0.25, -0.125, 0.0625], dtype=np.float32)
    part.bind({"up_weight": dev(up, DT[dtype]), "down_weight": dev(down, DT[dtype]), "coeff": dev(coeff)})
    h = plain.bf16_round(rs.randn(11, d).astype(np.float32))
    want = plain.feed_forward(h.astype(np.float64), {"up": up.astype(np.float64), "down": down.astype(np.float64), "act": coeff}, eps)
    got = part.forward(dev(h, DT[dtype]), None, None)
    assert got.dtype == torch.float32 and np.abs(host(got) - want).max() < tol(dtype, 3 * float(np.abs(want).max()))
    res = rs.randn(11, d).astype(np.float32)
    got = part.forward(dev(h, DT[dtype]), dev(res), None)
    assert np.abs(host(got) - (res + want)).max() < tol(dtype, 3 * float(np.abs(want).max()))


# ------------------------------------------------- the faster kernels against the plain ones --

def kv_context(H, rank, rot, P, plan_lengths):
    """A cache with one latent group filled with random pages, and a runner."""
    from ayaka_py_b200.cache import CacheGroupSpec
    from ayaka_py_b200.parts import KVNeed
    cache, runner = context_for([CacheGroupSpec("g", KVNeed(1, rot, None, 1, rank), 1)], "bfloat16", max_requests=4,
                                page_size=P, pages=2048 // P, positions=1024)
    rope, lat = cache.kv_layer(0, 0)
    gen = torch.Generator(device="cuda").manual_seed(1)
    lat.copy_(torch.randn(lat.shape, generator=gen, device="cuda"))
    rope.copy_(torch.randn(rope.shape, generator=gen, device="cuda"))
    return cache, runner, lat[:, :, 0], rope[:, :, 0]


@pytest.mark.parametrize("H,rank,rot,P", [(4, 72, 24, 16), (16, 512, 64, 16), (6, 40, 8, 8), (40, 32, 8, 16), (1, 264, 24, 16)])
def test_tensor_core_latent_attention_against_the_32_bit_pipes(H, rank, rot, P):
    """Prompts, portions on top of a cached context, single rows (whose context is cut into
    partitions and merged), all in one cache: both kernels read the same pages."""
    from ayaka_py_b200 import ops
    cache, runner, lat, rope = kv_context(H, rank, rot, P, None)
    gen = torch.Generator(device="cuda").manual_seed(2)
    for plan in ({0: 500, 1: 33, 2: 1}, {0: 7, 2: 130}, {0: 1, 1: 1, 2: 1}, {1: 1}, {0: 64, 1: 1, 2: 1, 3: 17}):
        ctx, res = step_of(cache, runner, plan)
        q = torch.randn(ctx.num_rows, H, rank + rot, generator=gen, device="cuda") * 0.5
        a = ops.latent_attention(q, lat, rope, ctx.tables[0], ctx, 0.2, tensor_cores=False)
        b = ops.latent_attention(q, lat, rope, ctx.tables[0], ctx, 0.2, tensor_cores=True)
        assert not torch.isnan(b).any()
        assert float((a - b).abs().max()) < 0.01 * float(a.abs().max()) + 1e-3, plan
        cache.commit(res)


@pytest.mark.parametrize("H,N,K", [(3, 24, 40), (16, 512, 128), (2, 70, 264), (5, 8, 96)])
def test_per_head_products_on_both_pipes(H, N, K):
    from ayaka_py_b200 import ops
    gen = torch.Generator(device="cuda").manual_seed(3)
    for T in (1, 17, 130):
        wide = torch.randn(T, H * (K + 4) + 8, generator=gen, device="cuda")
        a = wide[:, :H * (K + 4)].view(T, H, K + 4)[:, :, :K]              # strided rows and heads
        w = (torch.randn(H, N, K, generator=gen, device="cuda") / K ** 0.5).to(torch.bfloat16)
        gate = torch.randn(T, H + 3, generator=gen, device="cuda")[:, :H]
        want = torch.einsum("thk,hnk->thn", a.double(), w.double()) * torch.sigmoid(gate.double())[:, :, None]
        for out_dtype in (torch.float32, torch.bfloat16):
            out = torch.zeros(T, H, N + 2, dtype=out_dtype, device="cuda")[:, :, :N]
            ops.head_matmul(a, w, out, gate=gate)
            assert float((out.double() - want).abs().max()) < (2e-4 if out_dtype == torch.float32 else 2e-2)
        plain_out = torch.empty(T, H, N, device="cuda")
        ops.head_matmul(a, w.float(), plain_out)                            # 32-bit weights: the FP32 pipes
        assert float((plain_out.double() - torch.einsum("thk,hnk->thn", a.double(), w.double())).abs().max()) < 1e-4


@pytest.mark.parametrize("heads,dim,vdim", [(2, 10, 36), (1, 128, 128), (3, 33, 70)])
def test_hgrn2_in_chunks_against_the_walk_with_strong_and_weak_decay(heads, dim, vdim):
    """Both forms from the same projections: gates near zero (everything forgotten at once, logs
    of tiny numbers) and near one (hundreds of tokens remembered)."""
    from ayaka_py_b200 import ops
    from ayaka_py_b200.cache import CacheGroupSpec
    from ayaka_py_b200.parts import StateNeed
    gen = torch.Generator(device="cuda").manual_seed(4)
    width = heads * (2 * dim + vdim)
    for bias, lower in ((-30.0, 0.0), (0.0, 0.3), (8.0, 0.99)):
        f_bias = torch.full((heads * dim,), bias, device="cuda")
        low = torch.full((heads * dim,), lower, device="cuda")
        outs = []
        for chunked in (False, True):
            cache, runner = context_for([CacheGroupSpec("g", StateNeed((heads, dim, vdim)), 1)], "float32", max_requests=3)
            state = cache.state_layer(0, 0)
            got = []
            g2 = torch.Generator(device="cuda").manual_seed(5)
            for plan in ({0: 37, 1: 3}, {0: 16, 1: 1, 2: 50}, {0: 1, 2: 15}):
                ctx, res = step_of(cache, runner, plan)
                proj = torch.randn(ctx.num_rows, width + 4, generator=g2, device="cuda")
                got.append(ops.hgrn2(proj, state, f_bias, low, ctx, heads, dim, vdim, chunked=chunked))
                cache.commit(res)
            outs.append((torch.cat(got), state.clone()))
        (a, sa), (b, sb) = outs
        assert not torch.isnan(b).any() and not torch.isnan(sb).any()
        scale = float(a.abs().max()) + 1e-6
        assert float((a - b).abs().max()) < 2e-5 * max(1.0, scale), (bias, lower)
        assert float((sa - sb).abs().max()) < 2e-5 * max(1.0, float(sa.abs().max()))


# --------------------------------------------------------------- whole models --

def test_layers_one_by_one_in_32_bit(models):
    """The residual stream after every layer against the plain implementation."""
    from ayaka_py_b200.engine.step import StepEntry
    from ayaka_py_b200.replay import ReplaySession
    for tag in CONFIGS:
        folder, cfg, t64, reqs, _ = models[tag]
        toks = list(reqs.values())[2]
        _, after = plain.forward(cfg, t64, toks, return_layers=True)
        s = ReplaySession(folder, "float32", 256, PAGE[tag])
        slot = s.cache.open("x")
        res = s.cache.reserve([(slot, 0, len(toks))])
        ctx = s.runner.prepare([StepEntry(slot, 0, toks, [0])])
        x = s.model.embedding.forward(ctx, s.model.position)
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
    # more requests than slots: every slot is used more than once
    extra = {f"{rid}+": toks[::-1] for rid, toks in reqs.items()}
    _, cfg, t64, _, want = models[tag]
    want = dict(want)
    want.update({rid: plain.forward(cfg, t64, toks) for rid, toks in extra.items()})
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
    want = {"long": plain.forward(cfg, t64, toks)}
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


@pytest.mark.parametrize("kind", ["recurrent_only", "latent_only"])
def test_models_of_one_kind_of_layer(tmp_path, kind):
    """Only state slots and no pages at all, or only pages: replayed mixed and generated from through the engine."""
    from ayaka_py_b200.engine.llm import LLM
    from ayaka_py_b200.engine.request import StopCriteria
    from ayaka_py_b200.sampling.params import SamplingParams
    layers = ([recurrent(2, 12, 20, 40), recurrent(1, 8, 48, None)] if kind == "recurrent_only"
              else [latent(2, 12, 8, 20, 16, ROT_PLAIN, 0.3, None), latent(3, 8, 8, 8, 24, ROT_SCALED | {"dims": 8}, 0.35, 40)])
    cfg = {"architecture": "Rakalix", "vocab": 90, "width": 40, "norm": {"eps": 1e-5}, "canon": {"taps": 4},
           "embedding": {"scale": 2.0}, "residual_mult": 0.6, "layers": layers}
    tensors = plain.random_tensors(cfg, seed=77)
    folder = plain.write_folder(tmp_path / kind, cfg, tensors)
    t64 = {k: v.astype(np.float64) for k, v in tensors.items()}
    rs = np.random.RandomState(13)
    reqs = {f"q{i}": rs.randint(0, 90, n).tolist() for i, n in enumerate([40, 9, 70, 23, 55])}
    want = {rid: plain.forward(cfg, t64, toks) for rid, toks in reqs.items()}
    trace = trace_tools.mixed(reqs, seed=5)
    outputs, session = replay(folder, "float32", trace, 16)
    assert trace_tools.first_difference(trace_tools.collect(trace, outputs), want, 1e-4) is None
    kinds = {type(g.need).__name__ for g in session.model.groups}
    assert kinds == ({"StateNeed"} if kind == "recurrent_only" else {"StateNeed", "KVNeed"})
    llm = LLM(folder, dtype="float32", kv_pages=12, page_size=16, max_requests=2, max_model_len=96)
    prompts = [reqs["q1"], reqs["q3"], reqs["q0"][:30]]
    for prompt, result in zip(prompts, llm.generate(prompts, SamplingParams(temperature=0.0), StopCriteria(max_tokens=6, ignore_eos=True))):
        want_tokens = plain.greedy_generate(cfg, t64, prompt, 6)
        k = next((i for i, (a, b) in enumerate(zip(result.token_ids, want_tokens)) if a != b), None)
        if k is not None:                     # a near tie may turn a token
            logits = plain.forward(cfg, t64, prompt + want_tokens[:k])[-1]
            assert abs(logits[result.token_ids[k]] - logits[want_tokens[k]]) < 1e-3


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
        # a near tie may turn a token; what came before it must be equal and the logits close
        k = next((i for i, (a, b) in enumerate(zip(result.token_ids, want)) if a != b), None)
        if k is not None:
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
    from ayaka_py_b200.config.model import RakalixConfig
    from ayaka_py_b200.weights import write_random_model
    folder = write_random_model(tmp_path / "m", RakalixConfig.from_dict(CONFIG_B), seed=3)
    assert json.loads((folder / "config.json").read_text())["architecture"] == "Rakalix"
    root = Path(__file__).resolve().parent.parent
    proc = subprocess.run([sys.executable, "-m", "ayaka_py_b200", "generate", str(folder), "--prompt-ids", "1,2,3,4,5",
                           "--max-tokens", "5", "--temperature", "0", "--ignore-eos", "--max-model-len", "64", "--kv-pages", "16"],
                          cwd=root, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    line = json.loads(proc.stdout.strip().splitlines()[-1])
    assert len(line["token_ids"]) == 5
