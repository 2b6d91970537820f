"""A plain, slow Vepitar decoder in numpy float64: whole sequences, no cache, one function for each
mechanism.  It is the oracle of the Vepitar tests and shares no code with ``gophonic_b200``.

Vepitar is a pre-norm decoder whose residual may be kept in several streams.  Its norms multiply by
1 + w, its head is the embedding table, every sublayer's output is multiplied by one factor, and a layer
carries one of two mixers and, optionally, a dense gated feed-forward or a mixture of experts:

* ``general_delta``: a matrix state per head; every token decays it per key channel, takes away a part of
  what lies along the token's unit key, and adds k v^T;
* ``attention``: grouped-query attention without positions, a short causal convolution on q, k and v,
  unit-RMS q, k and v, a sliding window, sigmoid weights with a bias per head, a gate per head.

Everything takes the weights as a dict name -> float64 array and the configuration as the parsed
config.json.
"""
from __future__ import annotations

import math
from typing import Dict, List, Tuple

import numpy as np

from .pugalix_plain import from_bf16_bits, read_model, to_bf16_bits, write_model  # noqa: F401  (file helpers of the tests)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def rms_unit(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def offset_norm(x, w, eps):
    """Unit RMS, then times 1 + w."""
    return rms_unit(x, eps) * (1.0 + w)


# ---- the residual in streams -------------------------------------------------------------------
def stream_read(streams: List[np.ndarray], c_in) -> np.ndarray:
    return sum(c_in[s] * streams[s] for s in range(len(streams)))


def stream_write(streams: List[np.ndarray], y, c_mix, c_out, mult) -> List[np.ndarray]:
    S = len(streams)
    return [sum(c_mix[s, t] * streams[s] for s in range(S)) + mult * c_out[t] * y for t in range(S)]


# ---- the delta-rule mixer ----------------------------------------------------------------------
def delta_decay(h, w, p):
    return np.exp(-math.exp(-0.5) * sigmoid(np.tanh(h @ w[p + "w1"].T) @ w[p + "w2"].T + w[p + "w0"]))


def delta_recurrence(r, k, v, decay, rate, state=None):
    """r, k, decay, rate: [T, H, d]; v: [T, H, dv].  Returns the outputs [T, H, dv] and the last state."""
    T, H, d = k.shape
    dv = v.shape[-1]
    S = np.zeros((H, d, dv)) if state is None else state.copy()
    out = np.zeros((T, H, dv))
    for t in range(T):
        for hh in range(H):
            u = k[t, hh] / math.sqrt(float(k[t, hh] @ k[t, hh]) + 1e-6)
            along = u @ S[hh]                                      # what the old state holds along the unit key
            S[hh] = decay[t, hh][:, None] * S[hh] - np.outer(rate[t, hh] * u, along) + np.outer(k[t, hh], v[t, hh])
            out[t, hh] = S[hh].T @ r[t, hh]
    return out, S


def delta_mixer(h, w, p, m, eps):
    T = h.shape[0]
    H, d = m["heads"], m["dim"]
    dv = m.get("vdim", d)
    r, k = (h @ w[p + "r"].T).reshape(T, H, d), (h @ w[p + "k"].T).reshape(T, H, d)
    v = (h @ w[p + "v"].T).reshape(T, H, dv)
    decay = delta_decay(h, w, p).reshape(T, H, d)
    rate = sigmoid(h @ w[p + "a"].T + w[p + "a.b"]).reshape(T, H, d)
    o, _ = delta_recurrence(r, k, v, decay, rate)
    o = rms_unit(o, eps).reshape(T, H * dv) * w[p + "norm"] * sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


# ---- the attention mixer -----------------------------------------------------------------------
def causal_conv(u, c):
    """u: [T, channels]; c: [channels, taps]; y_t = sum_j c[:, j] u_(t - taps + 1 + j), zeros before the start."""
    T, taps = u.shape[0], c.shape[1]
    padded = np.concatenate([np.zeros((taps - 1, u.shape[1])), u])
    return sum(c[:, j] * padded[j:j + T] for j in range(taps))


def sigmoid_window_attention(q, k, v, scale, window, bias):
    """q: [T, H, d]; k: [T, G, d]; v: [T, G, dv]; bias: [H].  Row i weighs key j <= i (i - j < window if window
    > 0) by sigmoid(q_i . k_j * scale + bias_h); nothing is normalised."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[-1]))
    for hh in range(H):
        g = hh // (H // G)
        s = (q[:, hh] @ k[:, g].T) * scale + bias[hh]
        i, j = np.arange(T)[:, None], np.arange(T)[None, :]
        seen = (j <= i) & ((i - j < window) if window > 0 else True)
        out[:, hh] = (sigmoid(s) * seen) @ v[:, g]
    return out


def attention_mixer(h, w, p, m, eps):
    T = h.shape[0]
    H, d = m["heads"], m["dim"]
    G, dv = m.get("kv_heads", H), m.get("vdim", d)
    q, k, v = h @ w[p + "q"].T, h @ w[p + "k"].T, h @ w[p + "v"].T
    if "conv" in m:
        q, k, v = causal_conv(q, w[p + "q.conv"]), causal_conv(k, w[p + "k.conv"]), causal_conv(v, w[p + "v.conv"])
    q, k, v = rms_unit(q.reshape(T, H, d), eps), rms_unit(k.reshape(T, G, d), eps), rms_unit(v.reshape(T, G, dv), eps)
    window = m["mask"]["size"] if "mask" in m else 0
    o = sigmoid_window_attention(q, k, v, m["scale"], window, w[p + "pb"])
    o = o * sigmoid(h @ w[p + "g"].T)[:, :, None]
    return o.reshape(T, H * dv) @ w[p + "o"].T


# ---- feed-forwards -----------------------------------------------------------------------------
def dense_feed_forward(h, w, p):
    g = h @ w[p + "gate"].T
    return (g * sigmoid(g) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def route(h, w, p, top):
    """The chosen experts [T, top] and their weights."""
    z = h @ w[p + "router"].T
    s = np.exp(z - z.max(-1, keepdims=True))
    s /= s.sum(-1, keepdims=True)
    chosen = np.argsort(-s, axis=-1, kind="stable")[:, :top]
    picked = np.take_along_axis(s, chosen, -1)
    return chosen, picked / (picked.sum(-1, keepdims=True) + 1e-20)


def expert_feed_forward(h, w, p):
    return (np.maximum(h @ w[p + "up"].T, 0.0) ** 2) @ w[p + "down"].T


def mixture_feed_forward(h, w, p, mlp):
    chosen, weight = route(h, w, p, mlp["router"]["top"])
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, g in zip(chosen[t], weight[t]):
            out[t] += g * expert_feed_forward(h[t:t + 1], w, p + f"e{e}.")[0]
    return out


# ---- the model -----------------------------------------------------------------------------------
def forward(cfg: dict, w: Dict[str, np.ndarray], tokens, return_layers: bool = False):
    eps, mult, S = cfg["norm"]["eps"], cfg.get("residual_mult", 1.0), cfg.get("streams")
    x = w["embed"][np.asarray(tokens)]
    streams = [x.copy() for _ in range(S)] if S else [x]
    after = []

    def sublayer(q, i, fn):
        nonlocal streams
        p = f"l{i}."
        if S:
            u = stream_read(streams, w[p + f"hc{q}.in"])
            y = fn(offset_norm(u, w[p + f"norm{q}"], eps))
            streams = stream_write(streams, y, w[p + f"hc{q}.mix"], w[p + f"hc{q}.out"], mult)
        else:
            streams = [streams[0] + mult * fn(offset_norm(streams[0], w[p + f"norm{q}"], eps))]

    for i, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], f"l{i}.mix."
        mixer = delta_mixer if layer["type"] == "general_delta" else attention_mixer
        sublayer(1, i, lambda h: mixer(h, w, p, m, eps))
        mlp = layer.get("mlp")
        if mlp is not None:
            if mlp["kind"] == "dense":
                sublayer(2, i, lambda h: dense_feed_forward(h, w, f"l{i}.mlp."))
            else:
                sublayer(2, i, lambda h: mixture_feed_forward(h, w, f"l{i}.mlp.", mlp))
        after.append(sum(streams))
    logits = offset_norm(sum(streams), w["final.norm"], eps) @ w["embed"].T
    return (logits, np.stack(after)) if return_layers else logits


# ---- making test models ----------------------------------------------------------------------------
def tensor_shapes(cfg: dict, rank: int = 8) -> Dict[str, tuple]:
    W, V, S = cfg["width"], cfg["vocab"], cfg.get("streams")
    out = {"embed": (V, W), "final.norm": (W,)}
    for i, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], f"l{i}.mix."
        H, d = m["heads"], m["dim"]
        dv = m.get("vdim", d)
        out[f"l{i}.norm1"] = (W,)
        if layer["type"] == "attention":
            G = m.get("kv_heads", H)
            out.update({p + "q": (H * d, W), p + "k": (G * d, W), p + "v": (G * dv, W), p + "pb": (H,), p + "g": (H, W), p + "o": (W, H * dv)})
            if "conv" in m:
                out.update({p + "q.conv": (H * d, m["conv"]), p + "k.conv": (G * d, m["conv"]), p + "v.conv": (G * dv, m["conv"])})
        else:
            r = m.get("rank", rank)
            out.update({p + "r": (H * d, W), p + "k": (H * d, W), p + "v": (H * dv, W), p + "g": (H * dv, W), p + "a": (H * d, W),
                        p + "a.b": (H * d,), p + "w1": (r, W), p + "w2": (H * d, r), p + "w0": (H * d,), p + "norm": (H * dv,),
                        p + "o": (W, H * dv)})
        mlp = layer.get("mlp")
        if mlp is not None:
            out[f"l{i}.norm2"] = (W,)
            q = f"l{i}.mlp."
            if mlp["kind"] == "dense":
                out.update({q + "gate": (mlp["ff"], W), q + "up": (mlp["ff"], W), q + "down": (W, mlp["ff"])})
            else:
                out[q + "router"] = (mlp["router"]["experts"], W)
                for e in range(mlp["router"]["experts"]):
                    out.update({q + f"e{e}.up": (mlp["expert"]["ff"], W), q + f"e{e}.down": (W, mlp["expert"]["ff"])})
        if S:
            for c in ("hc1.", "hc2.") if mlp is not None else ("hc1.",):
                out.update({f"l{i}.{c}in": (S,), f"l{i}.{c}out": (S,), f"l{i}.{c}mix": (S, S)})
    return out


def random_weights(cfg: dict, seed: int, rank: int = 8) -> Dict[str, np.ndarray]:
    """Random weights whose values bfloat16 holds exactly: matrices of deviation 1/sqrt(inputs), norm
    differences near 0, stream coefficients that really mix, a router whose choices are not close calls."""
    rng = np.random.default_rng(seed)
    w = {}
    S = cfg.get("streams") or 1
    for name, shape in tensor_shapes(cfg, rank).items():
        last = name.rsplit(".", 1)[-1]
        if last in ("norm1", "norm2") or name == "final.norm":
            v = 0.2 * rng.standard_normal(shape)
        elif last == "norm":
            v = 1.0 + 0.2 * rng.standard_normal(shape)
        elif last == "in":
            v = (1.0 + 0.3 * rng.standard_normal(shape)) / S
        elif last == "out":
            v = 1.0 + 0.3 * rng.standard_normal(shape)
        elif last == "mix":
            v = 0.7 * np.eye(shape[0]) + 0.3 / S + 0.1 * rng.standard_normal(shape)
        elif last == "conv":
            v = rng.standard_normal(shape) / math.sqrt(shape[-1])
        elif last in ("b", "w0", "pb"):
            v = rng.standard_normal(shape)
        elif last == "router":
            v = 3.0 * rng.standard_normal(shape) / math.sqrt(shape[-1])
        elif name == "embed":
            v = rng.standard_normal(shape)
        else:
            v = rng.standard_normal(shape) / math.sqrt(shape[-1])
        w[name] = from_bf16_bits(to_bf16_bits(v)).reshape(shape)
    return w


def greedy_generate(cfg, w, prompt, n: int) -> Tuple[List[int], List[float]]:
    ids, out, margins = list(prompt), [], []
    for _ in range(n):
        logits = forward(cfg, w, ids)[-1]
        order = np.argsort(logits)
        out.append(int(order[-1]))
        margins.append(float(logits[order[-1]] - logits[order[-2]]))
        ids.append(out[-1])
    return out, margins
