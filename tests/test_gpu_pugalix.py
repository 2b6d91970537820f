"""The Pugalix design on the GPU against the plain implementation (tests/plain/pugalix_plain.py):
each mixer alone, whole prompts against token-by-token decoding, prompts in portions, batches of
unequal requests, slots and pages that are used again, the edges of the window, far tokens, long
decoding, odd sizes, the kernels by themselves, and greedy generation through the entry point.
Every model here is made by the test (its own sizes, random weights that bfloat16 holds exactly)."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from tests.plain import pugalix_plain as P

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def attention(heads=4, kv_heads=2, dim=32, vdim=16, rot=16, base=1000.0, size=24, keep=3, scale=0.2, kv_from=None, ff=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "rot": {"dims": rot, "base": base},
         "mask": {"size": size, "keep_first": keep}, "scale": scale}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def gla(heads=2, dim=16, vdim=24, tau=8.0, ff=None):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def mlstm(heads=3, dim=8, vdim=40, cap=10.0, ff=None):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def config(layers, width=64, vocab=96, scale=3.0, eps=1e-5):
    return {"architecture": "Pugalix", "embedding": {"scale": scale}, "layers": layers, "norm": {"eps": eps},
            "vocab": vocab, "width": width}


CONFIGS = {
    "attention": config([attention(ff=96)]),
    "gla": config([gla(ff=None)]),
    "mlstm": config([mlstm(ff=80)]),
    # the four kinds of layer together; the last attention layer reads the first one's keys with a
    # window and kept tokens of its own
    "mix": config([gla(ff=96), attention(), mlstm(), attention(size=9, keep=0, kv_from=1, ff=80), gla(heads=4, dim=8, vdim=8, tau=2.0)]),
    # key and value heads of one size that the tensor-core attention kernels take in bfloat16 (32, 64),
    # grouped heads, a window shorter and longer than a page
    "tensor": config([attention(heads=4, kv_heads=2, dim=32, vdim=32, rot=8, size=40, keep=2, ff=64), mlstm(heads=2, dim=16, vdim=16),
                      attention(heads=6, kv_heads=2, dim=64, vdim=64, rot=64, size=100, keep=70, scale=0.1),
                      attention(heads=6, kv_heads=2, dim=64, vdim=64, rot=64, size=7, keep=1, scale=0.1, kv_from=2),
                      # heads of 128: prompts of 65 rows and more run on the tcgen05 attention kernel
                      attention(heads=2, kv_heads=1, dim=128, vdim=128, rot=32, size=70, keep=3, scale=0.09)], width=96, vocab=80),
    # heads of 128 and 256 key channels: the scan kernel in which a warp's lanes are 32 slices of the channels
    "wide": config([gla(heads=1, dim=128, vdim=24, tau=4.0), mlstm(heads=2, dim=128, vdim=16), gla(heads=1, dim=256, vdim=8, tau=2.0),
                    mlstm(heads=1, dim=256, vdim=20, cap=8.0, ff=48)], width=64, vocab=70),
    # attention first, one kv head for four heads, two later layers reading the first one's keys with
    # masks of their own, and an attention layer of another head size with a cache group of its own
    "shared": config([attention(heads=4, kv_heads=1, dim=16, vdim=32, rot=4, size=30, keep=2, ff=64), gla(ff=72),
                      attention(heads=4, kv_heads=1, dim=16, vdim=32, rot=4, size=8, keep=0, kv_from=0), mlstm(ff=40),
                      attention(heads=4, kv_heads=1, dim=16, vdim=32, rot=4, size=200, keep=5, kv_from=0, ff=64),
                      attention(heads=2, kv_heads=2, dim=48, vdim=48, rot=48, size=16, keep=1, scale=0.14)], width=72, vocab=90),
    # sizes that are odd, equal, or 1: one head everywhere, key and value sizes equal in attention and not
    # multiples of 8 elsewhere, the whole head rotated, more kept tokens than the window is long
    "odd": config([attention(heads=1, kv_heads=1, dim=24, vdim=24, rot=24, size=5, keep=8, scale=0.31, ff=56),
                   gla(heads=1, dim=40, vdim=8, tau=1.0), mlstm(heads=1, dim=20, vdim=17, cap=4.0),
                   attention(heads=6, kv_heads=1, dim=8, vdim=40, rot=0, size=1, keep=0, scale=1.0)], width=48, vocab=61, scale=1.0, eps=1e-6),
}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for i, (name, cfg) in enumerate(CONFIGS.items()):
        w = P.random_weights(cfg, seed=50 + i, rank=5 + i)
        d = P.write_model(str(tmp_path_factory.mktemp(f"pugalix_{name}")), cfg, w)
        out[name] = (cfg, w, d)
    return out


_engines = {}


def engine_for(models, name, dtype, graphs=True, max_tokens=4096):
    from gophonic_b200.engine.model import Model
    from gophonic_b200.engine.step import Engine
    key = (name, dtype, graphs, max_tokens)
    if key not in _engines:
        _engines[key] = Engine(Model.from_dir(models[name][2], dtype=dtype), max_tokens=max_tokens, use_graphs=graphs)
    return _engines[key]


def tokens_for(cfg, seed, n):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], size=n).tolist()


def feed(engine, tokens, cuts=None):
    """All logits of one sequence fed in portions of the sizes ``cuts`` (the rest in one piece)."""
    slot = engine.new_sequence()
    out, at = [], 0
    sizes = list(cuts or []) + [len(tokens)]
    for n in sizes:
        n = min(n, len(tokens) - at)
        if n <= 0:
            break
        out.append(engine.step([(slot, tokens[at:at + n])], [list(range(n))]).cpu().numpy())
        at += n
    engine.end_sequence(slot)
    engine.check_kernels()
    return np.concatenate(out)


def close(got, want, tol):
    err = np.abs(got - want).max() / max(1.0, np.abs(want).max())
    assert err < tol, f"relative error {err:.3e} (tolerance {tol})"


TOL = {"float32": 3e-5, "bfloat16": 6e-2}


# ---- each mechanism alone, and all together ---------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["attention", "gla", "mlstm", "mix", "odd", "tensor", "wide", "shared"])
def test_whole_prompts_match_the_plain_model(models, name, dtype):
    cfg, w, _ = models[name]
    toks = tokens_for(cfg, 1, 230)      # from 192 rows on the output projections add into the residual themselves
    close(feed(engine_for(models, name, dtype), toks), P.forward(cfg, w, toks), TOL[dtype])


def test_the_residual_after_every_layer(models):
    import torch
    from gophonic_b200.parts.block import PreNormBlock
    cfg, w, _ = models["mix"]
    eng = engine_for(models, "mix", "float32", graphs=False)
    toks = tokens_for(cfg, 2, 70)
    seen, orig = [], PreNormBlock.forward

    def spy(self, batch, h, pending, cache, next_norm=None):
        out = orig(self, batch, h, pending, cache, next_norm=next_norm)
        seen.append((h + out if isinstance(out, torch.Tensor) else h.clone()).cpu().numpy())
        return out
    PreNormBlock.forward = spy
    try:
        feed(eng, toks)
    finally:
        PreNormBlock.forward = orig
    _, layers = P.forward(cfg, w, toks, return_layers=True)
    assert len(seen) == len(layers)
    for got, want in zip(seen, layers):
        close(got, want, 2e-5)


# ---- prompts against decoding, portions, batches ----------------------------------------------
@pytest.mark.parametrize("graphs", [True, False])
@pytest.mark.parametrize("name", ["mix", "odd", "wide", "shared"])
def test_token_by_token_equals_the_whole_prompt(models, name, graphs):
    cfg, w, _ = models[name]
    eng = engine_for(models, name, "float32", graphs=graphs)
    toks = tokens_for(cfg, 3, 90)
    whole = feed(eng, toks)
    single = feed(eng, toks, cuts=[1] * len(toks))
    close(single, whole, 2e-5)
    close(single, P.forward(cfg, w, toks), TOL["float32"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mix", "tensor", "wide"])
@pytest.mark.parametrize("cuts", [[2] * 40, [3, 64, 1, 2, 61], [63, 1, 1, 64], [130, 2]])
def test_portions_of_a_prompt(models, cuts, dtype, name):
    cfg, w, _ = models[name]
    eng = engine_for(models, name, dtype)
    toks = tokens_for(cfg, 4, 140)
    got = feed(eng, toks, cuts=cuts)
    close(got, P.forward(cfg, w, toks), TOL[dtype])
    if dtype == "float32":
        close(got, feed(eng, toks), 2e-5)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_batch_of_unequal_requests_equals_each_alone(models, dtype):
    cfg, w, _ = models["mix"]
    eng = engine_for(models, "mix", dtype)
    prompts = [tokens_for(cfg, 10 + i, n) for i, n in enumerate([1, 70, 9, 33])]
    more = [tokens_for(cfg, 20 + i, 12) for i in range(4)]
    slots = [eng.new_sequence() for _ in prompts]
    got = [[] for _ in prompts]
    first = eng.step(list(zip(slots, prompts)), [list(range(len(p))) for p in prompts]).cpu().numpy()
    at = 0
    for i, p in enumerate(prompts):
        got[i].append(first[at:at + len(p)])
        at += len(p)
    live = list(range(len(prompts)))
    for t in range(12):
        if t == 5:                      # one request ends early; the others go on
            eng.end_sequence(slots[live.pop(1)])
        logits = eng.step([(slots[i], [more[i][t]]) for i in live]).cpu().numpy()
        for j, i in enumerate(live):
            got[i].append(logits[j:j + 1])
    for i in live:
        eng.end_sequence(slots[i])
    eng.cache.check()
    for i, p in enumerate(prompts):
        n = 12 if i != 1 else 5
        want = P.forward(cfg, w, p + more[i][:n])
        close(np.concatenate(got[i]), want, TOL[dtype])


def test_slots_and_pages_that_are_used_again(models):
    """A sequence that takes over the slot, the pages and the state of one that ended sees nothing of it."""
    cfg, w, _ = models["mix"]
    eng = engine_for(models, "mix", "float32", max_tokens=256)     # four pages: the second sequence must reuse them
    a, b = tokens_for(cfg, 30, 200), tokens_for(cfg, 31, 130)
    close(feed(eng, a, cuts=[100]), P.forward(cfg, w, a), TOL["float32"])
    assert eng.cache.pages.held() == 0
    close(feed(eng, b, cuts=[64, 1, 1]), P.forward(cfg, w, b), TOL["float32"])
    s1 = eng.new_sequence()
    eng.step([(s1, a[:50])])
    eng.end_sequence(s1)
    s2 = eng.new_sequence()
    assert s2 == s1
    got = eng.step([(s2, b[:20])], [list(range(20))]).cpu().numpy()
    eng.end_sequence(s2)
    close(got, P.forward(cfg, w, b[:20]), TOL["float32"])


@pytest.mark.parametrize("name", ["mix", "tensor"])
def test_long_decoding_past_windows_and_pages(models, name):
    cfg, w, _ = models[name]
    toks = tokens_for(cfg, 5, 40 + 230)
    want = P.forward(cfg, w, toks)
    for dtype in ("float32", "bfloat16"):
        got = feed(engine_for(models, name, dtype), toks, cuts=[40] + [1] * 230)
        close(got, want, TOL[dtype])


# ---- far tokens: a state that forgets nothing -------------------------------------------------
@pytest.mark.parametrize("kind", ["gla", "mlstm"])
def test_a_token_far_back_stays_in_the_state(tmp_path, kind):
    """With decays (forget gates) pushed to one, what the first tokens wrote is still most of the state
    hundreds of tokens later: a state that were reset, cut or clipped on the way would show."""
    from gophonic_b200.engine.model import Model
    from gophonic_b200.engine.step import Engine
    cfg = config([gla(heads=2, dim=16, vdim=16, tau=4.0) if kind == "gla" else mlstm(heads=2, dim=16, vdim=16, cap=30.0)], width=32, vocab=40)
    w = P.random_weights(cfg, seed=9)
    if kind == "gla":
        w["l0.mix.a2.b"][:] = 14.0
    else:
        w["l0.mix.f.b"][:] = 20.0
        w["l0.mix.i.b"][:] = -1.0
    d = P.write_model(str(tmp_path / kind), cfg, w)
    toks = tokens_for(cfg, 6, 400)
    want = P.forward(cfg, w, toks)
    other = P.forward(cfg, w, [(toks[0] + 1) % cfg["vocab"]] + toks[1:])
    assert np.abs(want[-1] - other[-1]).max() > 1e-3          # the first token does matter at the end
    eng = Engine(Model.from_dir(d, dtype="float32"), max_tokens=1024)
    close(feed(eng, toks, cuts=[333] + [1] * 67), want, TOL["float32"])


# ---- the attention kernel by itself: edges of the window, kept tokens, pages, the sink ------------
def _attention_case(rng, T, heads, kv_heads, d, dv, window, keep):
    q = 0.3 * rng.standard_normal((T, heads, d))
    k = 0.3 * rng.standard_normal((T, kv_heads, d))
    v = rng.standard_normal((T, kv_heads, dv))
    # for chosen query positions one key each stands out (a score near 12), placed just inside and just
    # outside the window, at the last kept position and the first one that is not kept, at page borders, far back
    pairs = []
    for i in range(window + keep + 2, T, 7):
        j = [i - window + 1, i - window, keep - 1, keep, 63, 64, 1, i][(i // 7) % 8]
        if 0 <= j <= i:
            pairs.append((i, j))
    for i, j in pairs:
        u = rng.standard_normal(d)
        u /= np.linalg.norm(u)
        k[j, :, :] = 6.0 * u
        q[i, :, :] = 4.0 * u
    return q, k, v


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", [(2, 1, 16, 8, 37, 5), (4, 4, 24, 24, 70, 0), (3, 1, 8, 40, 64, 64),
                                   (4, 2, 32, 32, 70, 5), (2, 1, 64, 64, 37, 66), (3, 3, 128, 128, 130, 1)])
def test_attention_kernel_at_the_edges(shape, dtype):
    import torch
    from gophonic_b200 import ops
    heads, kv_heads, d, dv, window, keep = shape
    T, scale = 330, 0.5
    rng = np.random.default_rng(sum(shape))
    q, k, v = _attention_case(rng, T, heads, kv_heads, d, dv, window, keep)
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    dev = torch.device("cuda:0")
    ops.use_device(0)
    as_t = lambda a: torch.tensor(a, dtype=torch.float32).to(td).to(dev)
    qt, kt, vt = as_t(q), as_t(k), as_t(v)
    q, k, v = (t.float().cpu().numpy().astype(np.float64) for t in (qt, kt, vt))      # what the kernel sees
    want = P.windowed_sink_attention(q, k, v, scale, window, keep)
    pages = (T + 63) // 64
    perm = [3, 0, 5, 1, 4, 2][:pages]                                                  # physical pages in another order
    k_plane = torch.zeros((pages, kv_heads, 64, d), dtype=td, device=dev)
    v_plane = torch.zeros((pages, kv_heads, 64, dv), dtype=td, device=dev)
    for lp, pp in enumerate(perm):
        n = min(64, T - lp * 64)
        k_plane[pp, :, :n] = kt[lp * 64:lp * 64 + n].transpose(0, 1)
        v_plane[pp, :, :n] = vt[lp * 64:lp * 64 + n].transpose(0, 1)
    table = torch.tensor([[0] * pages, perm], dtype=torch.int32, device=dev)
    i32 = lambda *a: torch.tensor(a, dtype=torch.int32, device=dev)
    tol = 2e-5 if dtype == "float32" else 2e-2

    def run(rows, first, kv_len, splits=1):
        qq = qt[first:first + rows].reshape(rows, heads * d).contiguous()
        out = torch.zeros((rows, heads * dv), dtype=td, device=dev)
        scratch = torch.empty(ops.attention_scratch_floats(1, heads, dv, splits), dtype=torch.float32, device=dev) if splits > 1 else None
        ops.attention(qq, out, k_plane, v_plane, table, i32(1), i32(0), i32(rows), i32(kv_len), 1, rows, heads, kv_heads, d, scale,
                      window, splits, scratch, value_dim=dv, keep_first=keep, sink=True)
        return out.float().cpu().numpy().reshape(rows, heads, dv)
    close(run(T, 0, T), want, tol)                                   # the whole prompt
    close(run(T - 200, 200, T), want[200:], tol)                     # a portion that continues a cached prefix
    for i in list(range(window + keep + 2, T, 7)) + [0, 1, 63, 64, T - 1]:
        for splits in (1, 3):                                        # single tokens, keys uncut and cut
            close(run(1, i, i + 1, splits), want[i:i + 1], tol)


def test_the_sink_matters_and_is_applied():
    """A query whose scores are all very negative gives nearly nothing: the unit in the denominator wins."""
    import torch
    from gophonic_b200 import ops
    ops.use_device(0)
    dev = torch.device("cuda:0")
    d = 16
    q = torch.full((1, d), 2.0, device=dev)
    k_plane = torch.zeros((1, 1, 64, d), device=dev)
    k_plane[0, 0, :3] = -2.0
    v_plane = torch.ones((1, 1, 64, d), device=dev)
    out = torch.empty((1, d), device=dev)
    i32 = lambda *a: torch.tensor(a, dtype=torch.int32, device=dev)
    args = (q, out, k_plane, v_plane, i32(0).view(1, 1), i32(0), i32(0), i32(1), i32(3), 1, 1, 1, 1, d, 0.25)
    ops.attention(*args, sink=True)
    want = 3 * np.exp(-16.0) / (1 + 3 * np.exp(-16.0))
    assert abs(out[0, 0].item() - want) < 1e-9
    ops.attention(*args, sink=False)
    assert abs(out[0, 0].item() - 1.0) < 1e-6


# ---- the small kernels by themselves ------------------------------------------------------------
@pytest.mark.parametrize("size", [20, 128, 384])      # heads of whole 128s take 16 bytes a lane
def test_head_norm_gate_and_decay_kernels(size):
    import torch
    from gophonic_b200 import ops
    ops.use_device(0)
    dev = torch.device("cuda:0")
    rng = np.random.default_rng(0)
    rows, heads = 7, (5 if size == 128 else 3)     # five heads of 128: a warp with four heads and one with one
    x = rng.standard_normal((rows, heads * size))
    g = rng.standard_normal((rows, heads * size))
    div = 0.5 + rng.random((rows, heads, 4))
    for weight in (1 + 0.1 * rng.standard_normal(size), 1 + 0.1 * rng.standard_normal(heads * size), None):
        for kind, eps, use_div in ((ops.GATE_SILU, 1e-5, False), (ops.GATE_SIGMOID, 1e-6, True), (ops.GATE_SIGMOID, None, False)):
            xt, gt = torch.tensor(x, dtype=torch.float32, device=dev), torch.tensor(g, dtype=torch.float32, device=dev)
            dt = torch.tensor(div, dtype=torch.float32, device=dev)
            wt = None if weight is None else torch.tensor(weight, dtype=torch.float32, device=dev)
            y = torch.empty_like(xt)
            ops.head_norm_gate(xt, gt, y, heads, size, kind, weight=wt, eps=eps, divisor=dt[:, :, 3:] if use_div else None)
            v = x.reshape(rows, heads, size).copy()
            if use_div:
                v = v / div[:, :, 3:]
            if eps is not None:
                v = P.rms_unit(v, eps)
            if weight is not None:
                v = v * (weight.reshape(heads, size) if weight.size == heads * size else weight)
            gate = P.silu(g) if kind == ops.GATE_SILU else P.sigmoid(g)
            close(y.cpu().numpy(), v.reshape(rows, -1) * gate, 1e-5)
    z = 4 * rng.standard_normal((rows, 24))
    b = rng.standard_normal(24)
    zt = torch.tensor(z, dtype=torch.float32, device=dev)
    ops.gla_decay(zt, torch.tensor(b, dtype=torch.float32, device=dev), 6.0)
    close(zt.cpu().numpy(), P.sigmoid(z + b) ** (1 / 6.0), 1e-6)


# ---- generation through the entry point -----------------------------------------------------------
@pytest.mark.parametrize("fmt", ["f32", "bf16"])
def test_greedy_generation_through_the_entry_point(models, fmt):
    import gophonic_b200 as g
    cfg, w, d = models["mix"]
    m = g.Open(d, g.Options(Format=fmt, CacheTokens=2048, Batch=3))
    gen = g.Lane(m, g.TokensGenerator)
    prompts = [tokens_for(cfg, 40 + i, n) for i, n in enumerate([5, 31, 2, 66])]      # four requests, batches of three
    got = gen.Generate(prompts, g.ChatOptions(MaxTokens=10))
    for p, reply in zip(prompts, got):
        assert len(reply) == 10
        ids = list(p)
        for t in reply:       # every token is the plain model's choice given what came before, or a near-tie of it
            logits = P.forward(cfg, w, ids)[-1]
            assert logits.max() - logits[t] <= (1e-4 if fmt == "f32" else 0.15), "a token the plain model would not have chosen"
            ids.append(t)
    gen.engine.cache.check()
    assert gen.engine.cache.pages.held() == 0
    m.Close()


def test_the_trace_runner_on_a_pugalix_folder(models, tmp_path):
    cfg, w, d = models["odd"]
    a, b = tokens_for(cfg, 60, 30), tokens_for(cfg, 61, 11)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:20], "want": [0, 19]}, {"id": "b", "tokens": b[:10], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[20:21], "want": [0]}, {"id": "b", "tokens": b[10:11], "want": [0]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": a[21:], "want": [8]}], "end": ["a"]}]
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", "float32", "--out", str(out),
                        "--max-tokens", "64"], input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    la, lb = P.forward(cfg, w, a), P.forward(cfg, w, b)
    V = cfg["vocab"]
    read = lambda n: np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(-1, V)
    close(read(0), la[[0, 19]], TOL["float32"])
    close(read(1), np.stack([la[20], lb[10]]), TOL["float32"])
    close(read(2), la[29:30], TOL["float32"])


def test_the_command_line_writes_and_runs_a_named_configuration(tmp_path):
    """-random-config NAME -write-model DIR, then -model DIR: the plain model reads the written folder
    and would have chosen the same tokens."""
    out = tmp_path / "written"
    run = lambda *a: subprocess.run([sys.executable, "-m", "gophonic_b200", *a], cwd=ROOT, capture_output=True, text=True, timeout=600)
    r = run("-random-config", "pugalix-tiny", "-weights-seed", "4", "-write-model", str(out))
    assert r.returncode == 0, r.stderr[-2000:]
    cfg, w = P.read_model(str(out))
    assert cfg["architecture"] == "Pugalix" and {n: tuple(a.shape) for n, a in w.items()} == P.tensor_shapes(cfg)
    r = run("-model", str(out), "-format", "f32", "-max-tokens", "6", "3,9,27", "100")
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{")]
    assert [l["prompt"] for l in lines] == [[3, 9, 27], [100]]
    for l in lines:
        ids = list(l["prompt"])
        assert len(l["tokens"]) == 6
        for t in l["tokens"]:
            logits = P.forward(cfg, w, ids)[-1]
            assert logits.max() - logits[t] <= 1e-5
            ids.append(t)
