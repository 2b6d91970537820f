"""A plain, slow Pugalix decoder in numpy float64: whole sequences, no cache, one function for each
mechanism.  It is the oracle of the Pugalix tests and shares no code with ``gophonic_b200``.

Pugalix is a pre-norm decoder whose layers each carry one of three mixers and, optionally, a gated
feed-forward:

* ``attention``: grouped-query attention with biased q/k/v projections, a rotation of neighbouring
  pairs over the first ``rot.dims`` channels of a head, a sliding window that also keeps the first
  tokens of the sequence, a softmax whose denominator carries one extra unit (a sink of score zero
  without a value), a sigmoid output gate, and optionally the keys and values of an earlier layer;
* ``gla``: a matrix state per head that decays per key channel;
* ``mlstm``: a matrix state per head with scalar exponential gates and a running maximum.

Everything below takes the weights as a dict name -> float64 array and the configuration as the
parsed config.json.
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional, Tuple

import numpy as np


# ---- checkpoint reading (independent of the library's reader) ------------------------------
def read_safetensors(path: str) -> Dict[str, np.ndarray]:
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n).decode("utf-8"))
        data = f.read()
    out = {}
    for name, e in header.items():
        if name == "__metadata__":
            continue
        lo, hi = e["data_offsets"]
        raw = data[lo:hi]
        if e["dtype"] == "BF16":
            bits = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16
            vals = bits.view(np.float32).astype(np.float64)
        elif e["dtype"] == "F32":
            vals = np.frombuffer(raw, dtype="<f4").astype(np.float64)
        elif e["dtype"] == "I32":
            vals = np.frombuffer(raw, dtype="<i4").astype(np.int64)
        else:
            raise ValueError(f"{name}: dtype {e['dtype']}")
        out[name] = vals.reshape(e["shape"])
    return out


def read_model(model_dir: str):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(model_dir, "model.safetensors"))


# ---- elementary functions --------------------------------------------------------------------
def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def log_sigmoid(z):
    return -np.logaddexp(0.0, -z)


def silu(z):
    return z * sigmoid(z)


def rms_unit(x, eps):
    """x over its root mean square along the last axis, eps under the root."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def rms_norm(x, w, eps):
    return rms_unit(x, eps) * w


# ---- rotation ---------------------------------------------------------------------------------
def rotate_pairs(x, positions, dims: int, base: float):
    """x [T, heads, d]: channels 2i and 2i+1 (i < dims/2) turn by the angle pos * base^(-2i/dims);
    channels from ``dims`` on are left alone."""
    out = x.copy()
    i = np.arange(dims // 2, dtype=np.float64)
    freq = np.power(float(base), -2.0 * i / dims)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * freq[None, :]      # [T, dims/2]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


# ---- attention --------------------------------------------------------------------------------
def visible(i: int, j: int, size: int, keep_first: int) -> bool:
    return j <= i and (i - j < size or j < keep_first)


def windowed_sink_attention(q, k, v, scale, size, keep_first, first_pos: int = 0):
    """q [Tq, H, d] at positions first_pos.., k [Tk, G, d], v [Tk, G, dv] at positions 0..: per head
    softmax((q . k) scale) over the visible keys with one more unit in the denominator; [Tq, H, dv]."""
    Tq, H, _ = q.shape
    Tk, G, dv = v.shape
    mask = np.array([[visible(first_pos + i, j, size, keep_first) for j in range(Tk)] for i in range(Tq)])
    out = np.zeros((Tq, H, dv))
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head, :] @ k[:, g, :].T) * scale
        s = np.where(mask, s, -np.inf)
        top = np.maximum(s.max(axis=1, keepdims=True), 0.0)
        e = np.exp(s - top)
        denom = np.exp(-top) + e.sum(axis=1, keepdims=True)      # the sink: one more unit, no value
        out[:, head, :] = (e / denom) @ v[:, g, :]
    return out


def attention_keys_values(h, w, p, m):
    """Rotated keys [T, G, d] and values [T, G, dv] of an attention layer with projections of its own."""
    T = h.shape[0]
    G, d, dv = m["kv_heads"], m["dim"], m["vdim"]
    k = (h @ w[p + "k"].T + w[p + "k.b"]).reshape(T, G, d)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).reshape(T, G, dv)
    k = rotate_pairs(k, np.arange(T), m["rot"]["dims"], m["rot"]["base"])
    return k, v


def attention_mixer(h, w, p, m, kv):
    """h [T, width] -> [T, width].  ``kv`` = (keys, values) as ``attention_keys_values`` gives them,
    this layer's own or an earlier layer's."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).reshape(T, H, d)
    q = rotate_pairs(q, np.arange(T), m["rot"]["dims"], m["rot"]["base"])
    k, v = kv
    out = windowed_sink_attention(q, k, v, m["scale"], m["mask"]["size"], m["mask"]["keep_first"])
    gate = sigmoid(h @ w[p + "g"].T)
    return (out.reshape(T, H * dv) * gate) @ w[p + "o"].T


# ---- gla ----------------------------------------------------------------------------------------
def gla_mixer(h, w, p, m, eps, state=None):
    """Matrix state per head with a decay per key channel; returns (output [T, width], last state)."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).reshape(T, H, d) / math.sqrt(d)
    k = (h @ w[p + "k"].T).reshape(T, H, d)
    v = (h @ w[p + "v"].T).reshape(T, H, dv)
    z = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "a2.b"]
    alpha = np.exp(log_sigmoid(z) / m["tau"]).reshape(T, H, d)
    S = np.zeros((H, d, dv)) if state is None else state.copy()
    o = np.zeros((T, H, dv))
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = np.einsum("hcv,hc->hv", S, q[t])
    o = rms_norm(o, w[p + "norm"], eps)                            # per head, one weight of size dv
    y = o.reshape(T, H * dv) * silu(h @ w[p + "g"].T)
    return y @ w[p + "o"].T, S


# ---- mlstm --------------------------------------------------------------------------------------
def mlstm_mixer(h, w, p, m, eps, state=None):
    """Matrix memory with scalar gates per head, stabilised by a running maximum that starts at 0."""
    T = h.shape[0]
    H, d, dv, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    q = (h @ w[p + "q"].T).reshape(T, H, d) / math.sqrt(d)
    k = (h @ w[p + "k"].T).reshape(T, H, d)
    v = (h @ w[p + "v"].T).reshape(T, H, dv)
    gi = cap * np.tanh((h @ w[p + "i"].T + w[p + "i.b"]) / cap)                  # [T, H]
    gf = log_sigmoid(cap * np.tanh((h @ w[p + "f"].T + w[p + "f.b"]) / cap))
    if state is None:
        S, n, mx = np.zeros((H, d, dv)), np.zeros((H, d)), np.zeros(H)
    else:
        S, n, mx = (a.copy() for a in state)
    o = np.zeros((T, H, dv))
    for t in range(T):
        new = np.maximum(gf[t] + mx, gi[t])
        keep, take = np.exp(gf[t] + mx - new), np.exp(gi[t] - new)
        S = keep[:, None, None] * S + take[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = keep[:, None] * n + take[:, None] * k[t]
        mx = new
        num = np.einsum("hcv,hc->hv", S, q[t])
        den = np.maximum(np.abs(np.einsum("hc,hc->h", n, q[t])), np.exp(-mx)) + 1e-6
        o[t] = num / den[:, None]
    o = rms_unit(o, eps).reshape(T, H * dv) * w[p + "norm"]
    y = o * sigmoid(h @ w[p + "g"].T)
    return y @ w[p + "o"].T, (S, n, mx)


# ---- feed-forward -------------------------------------------------------------------------------
def dense_feed_forward(h, w, p):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


# ---- the model ----------------------------------------------------------------------------------
def forward(cfg: dict, w: Dict[str, np.ndarray], tokens, return_layers: bool = False):
    """Logits [T, vocab] of one whole sequence (and the residual after every layer, if asked)."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][np.asarray(tokens)] * cfg["embedding"]["scale"]
    kv_of: Dict[int, Tuple[np.ndarray, np.ndarray]] = {}
    after = []
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.mix.", layer["mixer"]
        h = rms_norm(x, w[f"l{i}.norm1"], eps)
        if layer["type"] == "attention":
            src = m.get("kv_from")
            if src is None:
                kv_of[i] = attention_keys_values(h, w, p, m)
                src = i
            y = attention_mixer(h, w, p, m, kv_of[src])
        elif layer["type"] == "gla":
            y, _ = gla_mixer(h, w, p, m, eps)
        elif layer["type"] == "mlstm":
            y, _ = mlstm_mixer(h, w, p, m, eps)
        else:
            raise ValueError(f"layer {i}: mixer '{layer['type']}'")
        x = x + y
        if layer.get("mlp") is not None:
            if layer["mlp"]["kind"] != "dense":
                raise ValueError(f"layer {i}: feed-forward '{layer['mlp']['kind']}'")
            x = x + dense_feed_forward(rms_norm(x, w[f"l{i}.norm2"], eps), w, f"l{i}.mlp.")
        after.append(x.copy())
    logits = rms_norm(x, w["final.norm"], eps) @ w["head"].T
    return (logits, np.stack(after)) if return_layers else logits


# ---- making test models (own writer, so the tests share nothing with the library's) ----------
def tensor_shapes(cfg: dict, rank: int = 8) -> Dict[str, tuple]:
    """Every tensor of a Pugalix checkpoint by name; ``rank``: rows of a gla mixer's first decay matrix
    where the configuration does not say."""
    W, V = cfg["width"], cfg["vocab"]
    out = {"embed": (V, W), "final.norm": (W,), "head": (V, W)}
    for i, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], f"l{i}.mix."
        H, d, dv = m["heads"], m["dim"], m["vdim"]
        out[f"l{i}.norm1"] = (W,)
        out.update({p + "q": (H * d, W), p + "g": (H * dv, W), p + "o": (W, H * dv)})
        if layer["type"] == "attention":
            G = m["kv_heads"]
            out[p + "q.b"] = (H * d,)
            if m.get("kv_from") is None:
                out.update({p + "k": (G * d, W), p + "k.b": (G * d,), p + "v": (G * dv, W), p + "v.b": (G * dv,)})
        else:
            out.update({p + "k": (H * d, W), p + "v": (H * dv, W)})
            if layer["type"] == "gla":
                r = m.get("rank", rank)
                out.update({p + "norm": (dv,), p + "a1": (r, W), p + "a2": (H * d, r), p + "a2.b": (H * d,)})
            else:
                out.update({p + "norm": (H * dv,), p + "i": (H, W), p + "i.b": (H,), p + "f": (H, W), p + "f.b": (H,)})
        if layer.get("mlp") is not None:
            F = layer["mlp"]["ff"]
            out[f"l{i}.norm2"] = (W,)
            out.update({f"l{i}.mlp.gate": (F, W), f"l{i}.mlp.up": (F, W), f"l{i}.mlp.down": (W, F)})
    return out


def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """float -> bfloat16 bit patterns, round to nearest even."""
    b = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((b + 0x7FFF + ((b >> 16) & 1)) >> 16).astype(np.uint16)


def from_bf16_bits(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32).astype(np.float64)


def random_weights(cfg: dict, seed: int, rank: int = 8) -> Dict[str, np.ndarray]:
    """Random weights whose values bfloat16 holds exactly: matrices of deviation 1/sqrt(inputs), norm
    weights near 1, biases that matter, decays and forget gates that keep a state alive for a while."""
    rng = np.random.default_rng(seed)
    w = {}
    for name, shape in tensor_shapes(cfg, rank).items():
        last = name.rsplit(".", 1)[-1]
        if last in ("norm", "norm1", "norm2"):
            v = 1.0 + 0.2 * rng.standard_normal(shape)
        elif name.endswith("a2.b"):
            v = 2.0 + rng.standard_normal(shape)
        elif name.endswith("f.b"):
            v = 2.0 + rng.standard_normal(shape)
        elif name.endswith(".b"):
            v = 0.5 * rng.standard_normal(shape)
        elif name == "embed":
            v = rng.standard_normal(shape)
        else:
            v = rng.standard_normal(shape) / math.sqrt(shape[-1])
        w[name] = from_bf16_bits(to_bf16_bits(v)).reshape(shape)
    return w


def write_model(model_dir: str, cfg: dict, w: Dict[str, np.ndarray]) -> str:
    """config.json and model.safetensors (bfloat16) of a model whose weights bfloat16 holds exactly."""
    os.makedirs(model_dir, exist_ok=True)
    header, blobs, at = {}, [], 0
    for name in sorted(w):
        raw = to_bf16_bits(w[name]).astype("<u2").tobytes()
        header[name] = {"dtype": "BF16", "shape": list(w[name].shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    text = json.dumps(header, separators=(",", ":")).encode()
    text += b" " * (-len(text) % 8)
    with open(os.path.join(model_dir, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(text)) + text + b"".join(blobs))
    with open(os.path.join(model_dir, "config.json"), "w") as f:
        json.dump(cfg, f, indent=1)
    return model_dir


def greedy_generate(cfg, w, prompt, n: int) -> Tuple[List[int], List[float]]:
    """``n`` greedy tokens after ``prompt`` and, for each, the margin of its logit over the runner-up."""
    ids, out, margins = list(prompt), [], []
    for _ in range(n):
        logits = forward(cfg, w, ids)[-1]
        order = np.argsort(logits)
        out.append(int(order[-1]))
        margins.append(float(logits[order[-1]] - logits[order[-2]]))
        ids.append(out[-1])
    return out, margins
