"""The Vepitar design on the GPU against the plain implementation (tests/plain/vepitar_plain.py): each
mechanism alone, whole prompts against token-by-token decoding, prompts in portions down to two tokens,
batches of unequal requests, slots and pages that are used again, the edges of the window in prompts and
in decoding, the first tokens, a token far back in the state, long decoding, odd sizes, the kernels by
themselves, and greedy generation through the entry point.  Every model here is made by the test (its own
sizes, random weights that bfloat16 holds exactly)."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from tests.plain import vepitar_plain as P

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def attention(heads=4, kv_heads=2, dim=32, vdim=16, size=24, conv=3, scale=0.2, mlp=None, **more):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": size}, "conv": conv, "scale": scale}
    m.update(more)
    return {"type": "attention", "mixer": {k: v for k, v in m.items() if v is not None}, "mlp": mlp}


def delta(heads=2, dim=16, mlp=None, **more):
    return {"type": "general_delta", "mixer": dict({"heads": heads, "dim": dim}, **more), "mlp": mlp}


def config(layers, width=64, vocab=96, streams=3, mult=0.5, eps=1e-5):
    cfg = {"architecture": "Vepitar", "layers": layers, "norm": {"eps": eps}, "residual_mult": mult, "vocab": vocab, "width": width}
    if streams is not None:
        cfg["streams"] = streams
    return cfg


CONFIGS = {
    "attention": config([attention(mlp=dense(96))]),
    "delta": config([delta(mlp=None)]),
    "moe": config([delta(heads=1, dim=8, mlp=moe(6, 2, 24))], streams=2),
    # both mixers and both feed-forwards together, a window shorter than a page and one longer
    "mix": config([delta(mlp=dense(96)), attention(mlp=moe(5, 2, 40)), delta(heads=4, dim=8, mlp=moe(3, 1, 16)),
                   attention(heads=6, kv_heads=3, dim=16, vdim=24, size=100, conv=4, scale=0.3, mlp=None), delta(mlp=moe(4, 4, 24))]),
    # heads of 128 and 256 key channels, one kv head for all heads, a convolution of two taps
    "wide": config([delta(heads=1, dim=128), attention(heads=4, kv_heads=1, dim=128, vdim=128, size=70, conv=2, scale=0.09, mlp=dense(64)),
                    delta(heads=1, dim=256, mlp=moe(7, 3, 16))], width=128, vocab=70, streams=4),
    # key and value heads the tensor-core attention kernel takes in bfloat16, of unequal sizes, windows around a page
    "tensor": config([attention(heads=4, kv_heads=2, dim=32, vdim=48, size=36, conv=5, mlp=moe(4, 2, 32)), delta(heads=2, dim=32),
                      attention(heads=6, kv_heads=2, dim=64, vdim=64, size=100, conv=2, scale=0.1, mlp=dense(64)),
                      attention(heads=2, kv_heads=1, dim=96, vdim=32, size=64, conv=3, scale=0.1),
                      attention(heads=2, kv_heads=1, dim=128, vdim=128, size=7, conv=4, scale=0.09)], width=96, vocab=80),
    # no streams at all (the plain residual with its factor), one stream with coefficients, a factor of 1
    "plain": config([delta(mlp=dense(40)), attention(mlp=moe(4, 2, 24))], streams=None, mult=0.7),
    "one": config([attention(mlp=dense(40)), delta(mlp=moe(4, 2, 24))], streams=1, mult=1.0),
    # what a file may leave out of an attention mixer: no convolution, no window, no grouping, values as wide
    # as keys; sizes that are odd, equal or 1: one head, one expert of which one is used, a window of 1,
    # a convolution of one tap, key sizes that are not multiples of 8
    "odd": config([attention(heads=3, kv_heads=None, dim=24, vdim=None, size=None, conv=None, scale=0.31, mask=None, mlp=moe(1, 1, 56)),
                   delta(heads=1, dim=40), attention(heads=1, kv_heads=1, dim=20, vdim=17, size=1, conv=1, scale=1.0),
                   delta(heads=3, dim=12, vdim=20, mlp=dense(24)),
                   attention(heads=6, kv_heads=1, dim=8, vdim=40, size=5, conv=7, scale=0.5, mlp=None)], width=48, vocab=61, streams=5, eps=1e-6),
}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for i, (name, cfg) in enumerate(CONFIGS.items()):
        w = P.random_weights(cfg, seed=70 + i, rank=5 + i)
        d = P.write_model(str(tmp_path_factory.mktemp(f"vepitar_{name}")), cfg, w)
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


def close(got, want, tol, most=1.0):
    """Every row within ``tol`` (relative to the largest wanted value); with ``most`` < 1 that share of the rows
    must be, and the rest within five times as much: in bfloat16 a router may take another expert than the
    plain model where two scores nearly tie, and the rows that follow carry the difference."""
    scale = max(1.0, np.abs(want).max())
    err = np.abs(got - want).reshape(got.shape[0], -1).max(-1) / scale
    if most >= 1.0:
        assert err.max() < tol, f"relative error {err.max():.3e} (tolerance {tol})"
    else:
        assert (err < tol).mean() >= most and err.max() < 5 * tol, f"{(err >= tol).sum()} of {len(err)} rows over {tol}, worst {err.max():.3e}"


TOL = {"float32": 3e-5, "bfloat16": 6e-2}
MOST = {"float32": 1.0, "bfloat16": 0.95}


# ---- each mechanism alone, and all together ---------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_whole_prompts_match_the_plain_model(models, name, dtype):
    cfg, w, _ = models[name]
    toks = tokens_for(cfg, 1, 230)      # from 192 rows on the output projections run on the paired tensor-core kernel
    close(feed(engine_for(models, name, dtype), toks), P.forward(cfg, w, toks), TOL[dtype], MOST[dtype])


def test_the_residual_after_every_layer(models):
    import torch
    from gophonic_b200.parts.hyper import HyperBlock
    cfg, w, _ = models["mix"]
    eng = engine_for(models, "mix", "float32", graphs=False)
    toks = tokens_for(cfg, 2, 70)
    seen, orig = [], HyperBlock.forward

    def spy(self, batch, streams, pending, cache):
        out = orig(self, batch, streams, pending, cache)
        mix = out.mix if out.mix is not None else torch.eye(streams.shape[0], device=streams.device)
        coef = out.out if out.out is not None else torch.ones(streams.shape[0], device=streams.device)
        after = torch.einsum("st,srw->rw", mix, streams) + out.mult * coef.sum() * out.y       # the sum of the streams once y is spread
        seen.append(after.cpu().numpy())
        return out
    HyperBlock.forward = spy
    try:
        feed(eng, toks)
    finally:
        HyperBlock.forward = orig
    _, layers = P.forward(cfg, w, toks, return_layers=True)
    assert len(seen) == len(layers)
    for got, want in zip(seen, layers):
        close(got, want, 2e-5)


# ---- prompts against decoding, portions, batches ----------------------------------------------
@pytest.mark.parametrize("graphs", [True, False])
@pytest.mark.parametrize("name", ["mix", "odd", "wide", "plain"])
def test_token_by_token_equals_the_whole_prompt(models, name, graphs):
    cfg, w, _ = models[name]
    eng = engine_for(models, name, "float32", graphs=graphs)
    toks = tokens_for(cfg, 3, 90)
    whole = feed(eng, toks)
    single = feed(eng, toks, cuts=[1] * len(toks))
    close(single, whole, 2e-5)
    close(single, P.forward(cfg, w, toks), TOL["float32"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mix", "wide", "odd", "tensor"])
@pytest.mark.parametrize("cuts", [[2] * 40, [3, 64, 1, 2, 61], [63, 1, 1, 64], [130, 2]])
def test_portions_of_a_prompt(models, cuts, dtype, name):
    cfg, w, _ = models[name]
    eng = engine_for(models, name, dtype)
    toks = tokens_for(cfg, 4, 140)
    got = feed(eng, toks, cuts=cuts)
    close(got, P.forward(cfg, w, toks), TOL[dtype], MOST[dtype])
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
        close(np.concatenate(got[i]), want, TOL[dtype], MOST[dtype])


def test_slots_and_pages_that_are_used_again(models):
    """A sequence that takes over the slot, the pages and the state (the matrix state and the convolution's last
    rows) of one that ended sees nothing of it."""
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
    got = eng.step([(s2, b[:2])], [[0, 1]]).cpu().numpy()          # the first tokens of a sequence: the convolution reads zeros
    got = np.concatenate([got, eng.step([(s2, b[2:20])], [list(range(18))]).cpu().numpy()])
    eng.end_sequence(s2)
    close(got, P.forward(cfg, w, b[:20]), TOL["float32"])


@pytest.mark.parametrize("name", ["mix", "wide", "tensor"])
def test_long_decoding_past_windows_and_pages(models, name):
    cfg, w, _ = models[name]
    toks = tokens_for(cfg, 5, 40 + 230)
    want = P.forward(cfg, w, toks)
    for dtype in ("float32", "bfloat16"):
        got = feed(engine_for(models, name, dtype), toks, cuts=[40] + [1] * 230)
        close(got, want, TOL[dtype], MOST[dtype])


# ---- far tokens: a state that forgets nothing -------------------------------------------------
def test_a_token_far_back_stays_in_the_state(tmp_path):
    """With decays pushed to one and removal rates to nothing, what the first tokens wrote is still in the state
    hundreds of tokens later: a state that were reset, cut or clipped on the way would show."""
    from gophonic_b200.engine.model import Model
    from gophonic_b200.engine.step import Engine
    cfg = config([delta(heads=2, dim=16)], width=32, vocab=40, streams=2)
    w = P.random_weights(cfg, seed=9)
    w["l0.mix.w0"][:] = -16.0
    w["l0.mix.a.b"][:] = -9.0
    d = P.write_model(str(tmp_path / "far"), cfg, w)
    toks = tokens_for(cfg, 6, 400)
    want = P.forward(cfg, w, toks)
    other = P.forward(cfg, w, [(toks[0] + 1) % cfg["vocab"]] + toks[1:])
    assert np.abs(want[-1] - other[-1]).max() > 1e-3          # the first token does matter at the end
    eng = Engine(Model.from_dir(d, dtype="float32"), max_tokens=1024)
    close(feed(eng, toks, cuts=[333] + [1] * 67), want, TOL["float32"])


# ---- the attention kernel by itself: edges of the window, pages, the bias, the gate -------------
def _attention_case(rng, T, heads, kv_heads, d, dv, window):
    q = 0.3 * rng.standard_normal((T, heads, d))
    k = 0.3 * rng.standard_normal((T, kv_heads, d))
    v = rng.standard_normal((T, kv_heads, dv))
    # for chosen query positions one key each stands out (a weight near 1 among weights near 0), placed just
    # inside and just outside the window, at page borders, at the start, on the row itself
    pairs = []
    for i in range(window + 2, T, 7):
        j = [i - window + 1, i - window, 0, 63, 64, 1, i, i - 1][(i // 7) % 8]
        if 0 <= j <= i:
            pairs.append((i, j))
    for i, j in pairs:
        u = rng.standard_normal(d)
        u /= np.linalg.norm(u)
        k[j, :, :] = 6.0 * u
        q[i, :, :] = 4.0 * u
    return q, k, v


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("algo", ["auto", "mma", "simt"])
@pytest.mark.parametrize("shape", [(2, 1, 16, 8, 37), (4, 4, 24, 24, 70), (3, 1, 8, 40, 64), (4, 2, 32, 32, 65), (2, 1, 64, 64, 1),
                                   (3, 3, 128, 128, 130), (2, 2, 16, 16, 0), (4, 1, 96, 32, 44), (2, 2, 64, 48, 200), (2, 1, 32, 128, 0)])
def test_attention_kernel_at_the_edges(shape, dtype, algo):
    import torch
    from types import SimpleNamespace
    from gophonic_b200 import ops
    heads, kv_heads, d, dv, window = shape
    T, scale = 330, 0.5
    rng = np.random.default_rng(sum(shape))
    q, k, v = _attention_case(rng, T, heads, kv_heads, d, dv, window)
    bias = rng.standard_normal(heads) - 6.0              # an ordinary key weighs little, the one that stands out nearly 1
    gate = rng.standard_normal((T, heads))
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    dev = torch.device("cuda:0")
    ops.use_device(0)
    as_t = lambda a: torch.tensor(a, dtype=torch.float32).to(td).to(dev)
    qt, kt, vt, gt = as_t(q), as_t(k), as_t(v), as_t(gate)
    q, k, v, gate = (t.float().cpu().numpy().astype(np.float64) for t in (qt, kt, vt, gt))      # what the kernel sees
    want = P.sigmoid_window_attention(q, k, v, scale, window, bias) * P.sigmoid(gate)[:, :, None]
    assert np.abs(want).max() > 0.5
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
    bt = torch.tensor(bias, dtype=torch.float32, device=dev)
    tol = 2e-5 if dtype == "float32" else 2e-2

    def run(rows, first, kv_len):
        qq = qt[first:first + rows].reshape(rows, heads * d).contiguous()
        out = torch.zeros((rows, heads * dv), dtype=td, device=dev)
        batch = SimpleNamespace(seq_slot=i32(1), seq_q_start=i32(0), seq_q_len=i32(rows), seq_kv_len=i32(kv_len), nseq=1, max_q_len=rows)
        ops.attention_sigmoid(qq, out, k_plane, v_plane, table, batch, heads, kv_heads, d, scale, window, value_dim=dv, score_bias=bt,
                              gate=gt[first:first + rows], algo=algo)
        return out.float().cpu().numpy().reshape(rows, heads, dv)
    close(run(T, 0, T), want, tol)                                   # the whole prompt
    close(run(T - 200, 200, T), want[200:], tol)                     # a portion that continues a cached prefix
    close(run(2, 129, 131), want[129:131], tol)                      # a portion of two tokens
    for i in list(range(window + 2, T, 7)) + [0, 1, 63, 64, T - 1]:  # single tokens
        close(run(1, i, i + 1), want[i:i + 1], tol)


# ---- the convolution, the norms and the cache write by themselves ----------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", [(3, 1, 16, 24, 4), (2, 2, 40, 8, 2), (1, 1, 8, 8, 1), (4, 2, 128, 64, 7), (2, 1, 16, 16, 0)])
def test_convolution_norm_and_cache_write(shape, dtype):
    import torch
    from types import SimpleNamespace
    from gophonic_b200 import ops
    heads, kv_heads, d, dv, taps = shape
    ops.use_device(0)
    dev = torch.device("cuda:0")
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    rng = np.random.default_rng(sum(shape))
    qd, kd, vd = heads * d, kv_heads * d, kv_heads * dv
    C, eps = qd + kd + vd, 1e-5
    lengths = [150, 3, 70]
    extra = 5                                            # columns after q | k | v that the kernel leaves alone
    conv = rng.standard_normal((C, max(taps, 1)))
    conv_t = torch.tensor(conv, dtype=torch.float32, device=dev) if taps else None
    seqs = []
    for n in lengths:
        u = torch.tensor(rng.standard_normal((n, C + extra)), dtype=torch.float32).to(td)
        x = u.float().numpy().astype(np.float64)[:, :C]
        y = P.causal_conv(x, conv) if taps else x
        seqs.append((u.to(dev), P.rms_unit(y[:, :qd].reshape(n, heads, d), eps), P.rms_unit(y[:, qd:qd + kd].reshape(n, kv_heads, d), eps),
                     P.rms_unit(y[:, qd + kd:].reshape(n, kv_heads, dv), eps)))
    pages_per = 3
    table = torch.tensor([[0] * pages_per, [7, 2, 5], [1, 8, 0], [3, 6, 4]], dtype=torch.int32, device=dev)
    k_plane = torch.zeros((9, kv_heads, 64, d), dtype=td, device=dev)
    v_plane = torch.zeros((9, kv_heads, 64, dv), dtype=td, device=dev)
    state = torch.zeros((4, max(taps - 1, 1) * C), dtype=torch.float32, device=dev)
    i32 = lambda a: torch.tensor(a, dtype=torch.int32, device=dev)
    tol = 2e-5 if dtype == "float32" else 2e-2
    at = [0, 0, 0]
    # the three sequences advance together in portions of unequal sizes, then by single tokens (whose kernel moves the
    # state on itself), then in portions again
    for sizes in ([62, 1, 30], [2, 1, 0], [1, 1, 1], [1, 0, 1], [84, 0, 38]):
        live = [i for i in range(3) if sizes[i] > 0]
        rows = sum(sizes)
        qkv = torch.cat([seqs[i][0][at[i]:at[i] + sizes[i]] for i in live])
        row_pos = np.concatenate([np.arange(at[i], at[i] + sizes[i]) for i in live])
        row_seq = np.concatenate([np.full(sizes[i], j) for j, i in enumerate(live)])
        starts = np.cumsum([0] + [sizes[i] for i in live])[:-1]
        batch = SimpleNamespace(row_pos=i32(row_pos), row_seq=i32(row_seq), seq_slot=i32([i + 1 for i in live]), seq_q_start=i32(starts),
                                seq_q_len=i32([sizes[i] for i in live]), nseq=len(live), max_q_len=max(sizes))
        q_out = torch.empty((rows, qd), dtype=td, device=dev)
        ops.conv_qkv(qkv, q_out, heads, kv_heads, d, dv, conv_t, state if taps > 1 else None, True, True, eps, batch, table, k_plane, v_plane)
        got = q_out.float().cpu().numpy().reshape(rows, heads, d)
        for j, i in enumerate(live):
            close(got[starts[j]:starts[j] + sizes[i]], seqs[i][1][at[i]:at[i] + sizes[i]], tol)
            at[i] += sizes[i]
    for i, n in enumerate(lengths):
        for lp in range((n + 63) // 64):
            m = min(64, n - lp * 64)
            page = int(table[i + 1, lp])
            close(k_plane[page, :, :m].float().cpu().numpy().transpose(1, 0, 2), seqs[i][2][lp * 64:lp * 64 + m], tol)
            close(v_plane[page, :, :m].float().cpu().numpy().transpose(1, 0, 2), seqs[i][3][lp * 64:lp * 64 + m], tol)


# ---- the recurrence by itself ------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", [(2, 16, 16), (1, 40, 8), (3, 12, 20), (1, 128, 24), (1, 256, 16), (2, 64, 64), (1, 100, 33)])
def test_delta_recurrence_kernel(shape, dtype):
    import torch
    from gophonic_b200 import ops
    heads, d, dv = shape
    ops.use_device(0)
    dev = torch.device("cuda:0")
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    rng = np.random.default_rng(sum(shape))
    lengths = [45, 1, 19]
    scale_w, key_eps = 0.6, 1e-6
    width = 2 * heads * d + heads * dv
    # the decay's pre-activation is itself a product, w2 tanh(low): steps of single tokens are given its factors
    rank = 6
    w2 = torch.tensor(rng.standard_normal((heads * d, rank)), dtype=torch.float32).to(td)
    seqs = []
    for n in lengths:
        rkv = torch.tensor(rng.standard_normal((n, width)), dtype=torch.float32).to(td)
        low = rng.standard_normal((n, rank)).astype(np.float32)
        zw, za = np.tanh(low.astype(np.float64)) @ w2.float().numpy().astype(np.float64).T, 2.0 * rng.standard_normal((n, heads * d))
        seqs.append((rkv, zw.astype(np.float32), za.astype(np.float32), low))
    bw, ba = rng.standard_normal(heads * d).astype(np.float32), rng.standard_normal(heads * d).astype(np.float32)
    want = []
    for rkv, zw, za, _ in seqs:
        x = rkv.float().numpy().astype(np.float64)
        n = x.shape[0]
        r, k = x[:, :heads * d].reshape(n, heads, d), x[:, heads * d:2 * heads * d].reshape(n, heads, d)
        v = x[:, 2 * heads * d:].reshape(n, heads, dv)
        decay = np.exp(-scale_w * P.sigmoid(zw.astype(np.float64) + bw)).reshape(n, heads, d)
        rate = P.sigmoid(za.astype(np.float64) + ba).reshape(n, heads, d)
        want.append(P.delta_recurrence(r, k, v, decay, rate))
    state = torch.zeros((5, heads, d * dv), dtype=torch.float32, device=dev)
    state[0] = 7.0                                       # a slot nobody uses
    i32 = lambda a: torch.tensor(a, dtype=torch.int32, device=dev)
    f32 = lambda a: torch.tensor(a, dtype=torch.float32, device=dev)
    tol = 3e-5 if dtype == "float32" else 2e-2
    at = [0, 0, 0]
    for sizes in ([20, 1, 2], [1, 0, 1], [2, 0, 9], [1, 0, 1], [21, 0, 6]):      # portions, and steps of one token each
        live = [i for i in range(3) if sizes[i] > 0]
        rows = sum(sizes)
        cat = lambda k: np.concatenate([seqs[i][k][at[i]:at[i] + sizes[i]] for i in live])
        rkv = torch.cat([seqs[i][0][at[i]:at[i] + sizes[i]] for i in live]).to(dev)
        starts = np.cumsum([0] + [sizes[i] for i in live])[:-1]
        out = torch.empty((rows, heads * dv), dtype=torch.float32, device=dev)
        if max(sizes) == 1:
            ops.delta_scan(rkv, 0, heads * d, 2 * heads * d, heads, d, dv, None, f32(bw), scale_w, f32(cat(2)), f32(ba), key_eps, state, out,
                           i32([i + 1 for i in live]), i32(starts), i32([sizes[i] for i in live]), len(live), max_q_len=1,
                           low=f32(cat(3)), w2=w2.to(dev))
        else:
            ops.delta_scan(rkv, 0, heads * d, 2 * heads * d, heads, d, dv, f32(cat(1)), f32(bw), scale_w, f32(cat(2)), f32(ba), key_eps, state, out,
                           i32([i + 1 for i in live]), i32(starts), i32([sizes[i] for i in live]), len(live), max_q_len=max(sizes))
        got = out.cpu().numpy().reshape(rows, heads, dv)
        for j, i in enumerate(live):
            ref = want[i][0][at[i]:at[i] + sizes[i]]
            close(got[starts[j]:starts[j] + sizes[i]], ref, tol)
            at[i] += sizes[i]
    for i in range(3):
        close(state[i + 1].cpu().numpy().reshape(heads, d, dv), want[i][1], tol)
    assert float(state[0].min()) == 7.0 and float(state[4].abs().max()) == 0.0


# ---- the streams' kernel by itself ---------------------------------------------------------------------
@pytest.mark.parametrize("S", [1, 2, 4, 7])
def test_stream_mix_and_norm_kernel(S):
    import torch
    from gophonic_b200 import ops
    ops.use_device(0)
    dev = torch.device("cuda:0")
    rng = np.random.default_rng(S)
    rows, width, eps, mult = 9, 200, 1e-5, 0.4
    x = rng.standard_normal((S, rows, width))
    y = rng.standard_normal((rows, width))
    c_in, c_out, c_mix, nw = rng.standard_normal(S), rng.standard_normal(S), rng.standard_normal((S, S)), 1 + 0.1 * rng.standard_normal(width)
    f32 = lambda a: torch.tensor(a, dtype=torch.float32, device=dev)
    new = P.stream_write(list(x), y, c_mix, c_out, mult)
    # write and read in one pass
    st, out = f32(x), torch.empty((rows, width), dtype=torch.float32, device=dev)
    ops.hyper_mix_norm(st, y=f32(y), mix=f32(c_mix), out_coef=f32(c_out), mult=mult, in_coef=f32(c_in), norm_weight=f32(nw), eps=eps, x_out=out)
    close(st.cpu().numpy(), np.stack(new), 1e-5)
    close(out.cpu().numpy(), P.rms_unit(P.stream_read(new, c_in), eps) * nw, 1e-5)
    # read alone; the plain sum; picked rows, with the streams left as they were; bfloat16 out
    st = f32(x)
    ops.hyper_mix_norm(st, in_coef=f32(c_in), norm_weight=f32(nw), eps=eps, x_out=out)
    close(out.cpu().numpy(), P.rms_unit(P.stream_read(list(x), c_in), eps) * nw, 1e-5)
    picked = torch.tensor([5, 0, 8], dtype=torch.int32, device=dev)
    few = torch.empty((3, width), dtype=torch.bfloat16, device=dev)
    ops.hyper_mix_norm(st, y=f32(y), mix=f32(c_mix), out_coef=f32(c_out), mult=mult, norm_weight=f32(nw), eps=eps, x_out=few, rows=picked)
    close(few.float().cpu().numpy(), (P.rms_unit(sum(new), eps) * nw)[[5, 0, 8]], 1e-2)
    assert np.array_equal(st.cpu().numpy(), x.astype(np.float32))
    # no coefficients at all: the plain residual x + mult * y
    one = f32(x[:1])
    ops.hyper_mix_norm(one, y=f32(y), mult=mult)
    close(one.cpu().numpy()[0], x[0] + mult * y, 1e-6)


# ---- the router and the experts by themselves ------------------------------------------------------------
@pytest.mark.parametrize("shape", [(8, 3, 24, 40), (1, 1, 16, 16), (40, 6, 8, 72), (5, 5, 32, 24)])
def test_router_and_experts(shape):
    import torch
    from gophonic_b200 import ops
    from gophonic_b200.config.spec import MoESpec
    from gophonic_b200.parts.base import Runtime
    from gophonic_b200.parts.moe import MoE
    experts, top, ff, width = shape
    ops.use_device(0)
    dev = torch.device("cuda:0")
    rng = np.random.default_rng(sum(shape))
    cfg = {"architecture": "Vepitar", "layers": [], "norm": {"eps": 1e-5}, "vocab": 4, "width": width}
    w = {"router": 3.0 * rng.standard_normal((experts, width)) / np.sqrt(width)}
    for e in range(experts):
        w[f"e{e}.up"], w[f"e{e}.down"] = rng.standard_normal((ff, width)) / np.sqrt(width), rng.standard_normal((width, ff)) / np.sqrt(ff)
    spec = MoESpec(hidden=width, experts=experts, top=top, intermediate=ff)
    tensors = {n: torch.tensor(a, dtype=torch.float32, device=dev) for n, a in w.items()}
    w = {n: t.cpu().numpy().astype(np.float64) for n, t in tensors.items()}
    part = MoE(spec, "", tensors, Runtime(dev, torch.float32, ops))
    for rows in (1, 3, 12, 50, 300):              # few rows read the chosen experts only (pair by pair, or sorted by expert), more run the stacked products, many every expert on its own rows
        h = rng.standard_normal((rows, width)).astype(np.float32)
        out = torch.empty((rows, width), dtype=torch.float32, device=dev)
        part.forward(None, torch.tensor(h, device=dev), out)
        close(out.cpu().numpy(), P.mixture_feed_forward(h.astype(np.float64), w, "", {"router": {"top": top}}), 2e-5)
    # the choice itself: indices, weights, zeros elsewhere
    z = rng.standard_normal((7, experts)).astype(np.float32)
    dense = torch.empty((7, experts), dtype=torch.float32, device=dev)
    index, weight = torch.empty((7, top), dtype=torch.int32, device=dev), torch.empty((7, top), dtype=torch.float32, device=dev)
    ops.moe_route(torch.tensor(z, device=dev), top, 1e-20, dense, index, weight)
    s = np.exp(z.astype(np.float64))
    s /= s.sum(-1, keepdims=True)
    order = np.argsort(-s, -1, kind="stable")[:, :top]
    assert np.array_equal(index.cpu().numpy(), order)
    picked = np.take_along_axis(s, order, -1)
    close(weight.cpu().numpy(), picked / picked.sum(-1, keepdims=True), 1e-6)
    full = np.zeros_like(s)
    np.put_along_axis(full, order, picked / picked.sum(-1, keepdims=True), -1)
    close(dense.cpu().numpy(), full, 1e-6)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_products_with_a_block_of_columns_as_weights(dtype):
    """An expert's down matrix is a block of columns of the stacked one: the product takes the wider matrix's row stride,
    for one row as for hundreds (an expert few rows chose)."""
    import torch
    from gophonic_b200 import ops
    ops.use_device(0)
    dev = torch.device("cuda:0")
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    rng = np.random.default_rng(3)
    N, K, wide = 72, 40, 5 * 40
    w_all = torch.tensor(rng.standard_normal((N, wide)) / np.sqrt(K), dtype=torch.float32).to(td).to(dev)
    for M in (1, 5, 130, 200, 300):
        a = torch.tensor(rng.standard_normal((M, K)), dtype=torch.float32).to(td).to(dev)
        for block in (0, 3):
            w = w_all[:, block * K:(block + 1) * K]
            out = torch.empty((M, N), dtype=torch.float32, device=dev)
            ops.gemm_w_cols(a, w, out)
            want = a.float().cpu().numpy().astype(np.float64) @ w.float().cpu().numpy().astype(np.float64).T
            close(out.cpu().numpy(), want, 2e-5 if dtype == "float32" else 2e-3)


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
            assert logits.max() - logits[t] <= (1e-4 if fmt == "f32" else 0.25), "a token the plain model would not have chosen"
            ids.append(t)
    gen.engine.cache.check()
    assert gen.engine.cache.pages.held() == 0
    m.Close()


def test_the_trace_runner_on_a_vepitar_folder(models, tmp_path):
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
    r = run("-random-config", "vepitar-tiny", "-weights-seed", "4", "-write-model", str(out))
    assert r.returncode == 0, r.stderr[-2000:]
    cfg, w = P.read_model(str(out))
    assert cfg["architecture"] == "Vepitar" and {n: tuple(a.shape) for n, a in w.items()} == P.tensor_shapes(cfg)
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
