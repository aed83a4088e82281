"""Plain, slow restatement of the Lasizen decoder in numpy float64: whole sequences, no cache, no batching, one
function per mechanism.  It shares nothing with the engine and is what the engine's results are held against.

A model is (config, weights): ``config`` the parsed config.json, ``weights`` a dict name -> float64 array.

Notation: n tokens, d the model width; a linear map stored [out, in] is applied as ``x @ W.T``; positions count from 0.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np


# ---- elementwise pieces -------------------------------------------------------------------------------------------
def silu(z):
    return z / (1.0 + np.exp(-z))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def softplus(z):
    return np.logaddexp(0.0, z)


def rms_unit(x, eps):
    """x over its root mean square along the last axis, eps under the root."""
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)


def xielu(z, p, q):
    """Quadratic above zero, a scaled exponential below, both with slope 1/2 added."""
    below = np.minimum(z, 0.0)
    pos = softplus(p) * z * z + 0.5 * z
    neg = (0.5 + softplus(q)) * (np.expm1(below) - below) + 0.5 * below
    return np.where(z > 0, pos, neg)


# ---- the layer's own pieces -----------------------------------------------------------------------------------------
def token_shift(h, mu):
    """Row t becomes h[t] + (h[t-1] - h[t]) * mu; the row before the first is zero."""
    prev = np.vstack([np.zeros((1, h.shape[1])), h[:-1]])
    return h + (prev - h) * mu


def causal_conv(x, taps_w):
    """x [n, channels], taps_w [channels, taps]; the last column weighs the current token, zeros before the start."""
    n, c = x.shape
    k = taps_w.shape[1]
    padded = np.vstack([np.zeros((k - 1, c)), x])
    out = np.zeros((n, c))
    for j in range(k):
        out += padded[j:j + n] * taps_w[:, j]
    return out


# ---- rotation -------------------------------------------------------------------------------------------------------------
def rotation_frequencies(rot):
    """Angular frequency of each of the dims/2 pairs, and the factor on cos and sin."""
    dims, base = rot["dims"], rot["base"]
    i = np.arange(dims // 2, dtype=np.float64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    def turn(t):
        return dims * math.log(sc["original"] / (2.0 * math.pi * t)) / (2.0 * math.log(base))
    lo = max(math.floor(turn(sc["fast"])), 0)
    hi = min(math.ceil(turn(sc["slow"])), dims - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / sc["factor"] * ramp + f * (1.0 - ramp), 0.1 * math.log(sc["factor"]) + 1.0


def rotate_half(v, positions, rot):
    """v [n, heads, dim]: value i of the first dims is paired with value i + dims/2; the rest pass."""
    if not rot or not rot.get("dims"):
        return v
    dims = rot["dims"]
    f, m = rotation_frequencies(rot)
    a = positions[:, None].astype(np.float64) * f[None, :]
    cos, sin = (np.cos(a) * m)[:, None, :], (np.sin(a) * m)[:, None, :]
    out = v.copy()
    u, w = v[..., :dims // 2], v[..., dims // 2:dims]
    out[..., :dims // 2] = u * cos - w * sin
    out[..., dims // 2:dims] = w * cos + u * sin
    return out


# ---- mixers ---------------------------------------------------------------------------------------------------------------
def windowed_sink_attention(h, w, p, m, eps, positions=None):
    """Grouped-query attention over a sliding window; the softmax's denominator holds one more term, exp(0)."""
    n = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = np.arange(n) if positions is None else positions
    q = (h @ w[p + "q"].T).reshape(n, H, dk)
    k = (h @ w[p + "k"].T).reshape(n, G, dk)
    v = (h @ w[p + "v"].T).reshape(n, G, dv)
    q = rms_unit(rotate_half(q, pos, m.get("rot")), eps)
    k = rms_unit(rotate_half(k, pos, m.get("rot")), eps)
    size = (m.get("mask") or {}).get("size")
    out = np.zeros((n, H, dv))
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ k[:, g].T) * m["scale"]
        i, j = np.arange(n)[:, None], np.arange(n)[None, :]
        seen = (j <= i) if size is None else ((j <= i) & (i - j < size))
        s = np.where(seen, s, -np.inf)
        top = np.maximum(s.max(axis=1, keepdims=True), 0.0)
        e = np.exp(s - top)
        out[:, head] = (e / (np.exp(-top) + e.sum(axis=1, keepdims=True))) @ v[:, g]
    return out.reshape(n, H * dv) @ w[p + "o"].T


def gated_delta(h, w, p, m, eps):
    """The gated delta rule, token by token: per head a matrix S [dim, vdim] decays, is corrected towards the token's
    value along the token's key, and is read with the token's query."""
    n = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ w[p + "q"].T, w[p + "q.conv"])).reshape(n, G, dk)
    k = silu(causal_conv(h @ w[p + "k"].T, w[p + "k.conv"])).reshape(n, G, dk)
    v = silu(causal_conv(h @ w[p + "v"].T, w[p + "v.conv"])).reshape(n, H, dv)
    q = q / np.sqrt((q * q).sum(axis=-1, keepdims=True) + 1e-6) * dk ** -0.5
    k = k / np.sqrt((k * k).sum(axis=-1, keepdims=True) + 1e-6)
    beta = sigmoid(h @ w[p + "b"].T)
    decay = np.exp(-np.exp(w[p + "A_log"]) * softplus(h @ w[p + "a"].T + w[p + "dt_bias"]))
    gate = silu(h @ w[p + "g"].T).reshape(n, H, dv)
    out = np.zeros((n, H, dv))
    for head in range(H):
        g = head // (H // G)
        S = np.zeros((dk, dv))
        for t in range(n):
            S = decay[t, head] * S
            u = beta[t, head] * (v[t, head] - S.T @ k[t, g])
            S = S + np.outer(k[t, g], u)
            out[t, head] = S.T @ q[t, g]
    out = rms_unit(out, eps) * w[p + "norm"] * gate
    return out.reshape(n, H * dv) @ w[p + "o"].T


def dense_ff(h, w, p):
    a = w[p + "act"]
    return xielu(h @ w[p + "up"].T, a[0], a[1]) @ w[p + "down"].T


# ---- the model --------------------------------------------------------------------------------------------------------------
def run_order(config):
    """Layer indices in the order they run: the loop's layers `times` times in a row."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = loop["start"], loop["stop"], loop["times"]
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def forward(config, w, tokens, return_layers=False):
    """Logits [n, vocab] of a whole sequence (and the stream after every layer run)."""
    eps = config["norm"]["eps"]
    x = w["embed"][np.asarray(tokens)] * (config.get("embedding") or {}).get("scale", 1.0)
    streams = []
    for i in run_order(config):
        layer, p = config["layers"][i], f"l{i}."
        h = token_shift(rms_unit(x, eps) * w[p + "norm1"], w[p + "shift"])
        if layer["type"] == "attention":
            y = windowed_sink_attention(h, w, p + "mix.", layer["mixer"], eps)
        elif layer["type"] == "delta":
            y = gated_delta(h, w, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        x = x + rms_unit(y, eps) * w[p + "norm1b"]
        if layer.get("mlp"):
            y = dense_ff(rms_unit(x, eps) * w[p + "norm2"], w, p + "mlp.")
            x = x + rms_unit(y, eps) * w[p + "norm2b"]
        streams.append(x.copy())
    logits = (rms_unit(x, eps) * w["final.norm"]) @ w["head"].T * config.get("logit_scale", 1.0)
    return (logits, np.stack(streams)) if return_layers else logits


# ---- model folders ------------------------------------------------------------------------------------------------------
def tensor_shapes(config):
    """name -> shape of every tensor a model of this configuration has."""
    d, V = config["width"], config["vocab"]
    shapes = {"embed": (V, d), "final.norm": (d,), "head": (V, d)}
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        shapes[p + "norm1"] = shapes[p + "norm1b"] = shapes[p + "shift"] = (d,)
        H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        if layer["type"] == "attention":
            shapes.update({p + "mix.q": (H * dk, d), p + "mix.k": (G * dk, d), p + "mix.v": (G * dv, d), p + "mix.o": (d, H * dv)})
        else:
            K = m["conv"]
            shapes.update({p + "mix.q": (G * dk, d), p + "mix.q.conv": (G * dk, K), p + "mix.k": (G * dk, d), p + "mix.k.conv": (G * dk, K),
                           p + "mix.v": (H * dv, d), p + "mix.v.conv": (H * dv, K), p + "mix.b": (H, d), p + "mix.a": (H, d), p + "mix.A_log": (H,),
                           p + "mix.dt_bias": (H,), p + "mix.norm": (dv,), p + "mix.g": (H * dv, d), p + "mix.o": (d, H * dv)})
        mlp = layer.get("mlp")
        if mlp:
            shapes[p + "norm2"] = shapes[p + "norm2b"] = (d,)
            shapes.update({p + "mlp.up": (mlp["ff"], d), p + "mlp.down": (d, mlp["ff"]), p + "mlp.act": (2,)})
    return shapes


def to_bf16_bits(a):
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def from_bf16_bits(b):
    return (b.astype(np.uint32) << 16).view(np.float32)


def random_weights(config, seed, overrides=None):
    """Random weights (rounded to bfloat16, as a model file stores them) of sizes that keep activations of order one."""
    rng = np.random.default_rng(seed)
    w = {}
    for name, shape in tensor_shapes(config).items():
        leaf = name.split(".")[-1]
        if leaf in ("norm1", "norm2", "norm") or name == "final.norm":
            v = 1.0 + 0.2 * rng.standard_normal(shape)
        elif leaf in ("norm1b", "norm2b"):
            v = 0.5 + 0.1 * rng.standard_normal(shape)
        elif leaf == "shift":
            v = rng.uniform(0.0, 1.0, shape)
        elif leaf == "A_log":
            v = np.log(rng.uniform(0.3, 4.0, shape))
        elif leaf == "dt_bias":
            v = np.log(np.expm1(rng.uniform(0.01, 0.5, shape)))
        elif leaf == "act":
            v = rng.standard_normal(shape)
        elif leaf == "conv":
            v = rng.standard_normal(shape) * 0.5
        elif name == "embed":
            v = rng.standard_normal(shape) * 0.1
        else:
            v = rng.standard_normal(shape) * (1.5 / math.sqrt(shape[-1]))
        w[name] = from_bf16_bits(to_bf16_bits(v)).astype(np.float64)
    for name, v in (overrides or {}).items():
        w[name] = from_bf16_bits(to_bf16_bits(v)).astype(np.float64)
    return w


def write_model_dir(folder, config, w):
    """config.json and model.safetensors (bfloat16) as the engine reads them."""
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(config))
    header, blobs, at = {}, [], 0
    for name in sorted(w):
        raw = to_bf16_bits(w[name]).tobytes()
        header[name] = {"dtype": "BF16", "shape": list(w[name].shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    head = json.dumps(header).encode()
    head += b" " * (-len(head) % 8)
    with open(folder / "model.safetensors", "wb") as f:
        f.write(struct.pack("<Q", len(head)) + head + b"".join(blobs))
    return folder


def read_model_dir(folder):
    folder = Path(folder)
    config = json.loads((folder / "config.json").read_text())
    raw = (folder / "model.safetensors").read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    w = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        buf = raw[8 + n + lo:8 + n + hi]
        if meta["dtype"] == "BF16":
            a = from_bf16_bits(np.frombuffer(buf, dtype=np.uint16))
        elif meta["dtype"] == "F32":
            a = np.frombuffer(buf, dtype=np.float32)
        else:
            a = np.frombuffer(buf, dtype=np.int32)
        w[name] = a.reshape(meta["shape"]).astype(np.float64)
    return config, w
