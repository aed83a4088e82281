"""Plain, slow restatement of the Gufanex decoder in numpy float64: whole sequences, no cache, no batching, one
function per mechanism.  It shares nothing with the engine and is what the engine's results are held against.

A model is (config, weights): ``config`` the parsed config.json, ``weights`` a dict name -> float64 array.

Notation: n tokens, d the model width; a linear map stored [out, in] is applied as ``x @ W.T``.
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


def layer_norm(x, gain, bias, eps):
    mu = x.mean(axis=-1, keepdims=True)
    var = ((x - mu) ** 2).mean(axis=-1, keepdims=True)
    return (x - mu) / np.sqrt(var + eps) * gain + bias


def rms_unit(x, gain, eps):
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps) * gain


def softmax(z, axis=-1):
    z = z - z.max(axis=axis, keepdims=True)
    e = np.exp(z)
    return e / e.sum(axis=axis, keepdims=True)


# ---- rotation of neighbouring pairs --------------------------------------------------------------------------------
def rotate_pairs(v, positions, base, dims):
    """v [n, ..., r]: over the first ``dims`` of the last axis, the pair (2i, 2i+1) of the token at position p turns by
    the angle p * base^(-2i/dims); what lies behind ``dims`` stays."""
    out = v.copy()
    half = dims // 2
    freq = base ** (-2.0 * np.arange(half) / dims)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * freq[None, :]            # [n, half]
    shape = (len(positions),) + (1,) * (v.ndim - 2) + (half,)
    c, s = np.cos(ang).reshape(shape), np.sin(ang).reshape(shape)
    a, b = v[..., 0:dims:2], v[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


# ---- the selective-scan mixer ----------------------------------------------------------------------------------------
def causal_conv(x, taps_w, bias):
    """x [n, C]; taps_w [C, K] whose last column weighs the current token; zeros before the sequence."""
    n, C = x.shape
    K = taps_w.shape[1]
    padded = np.concatenate([np.zeros((K - 1, C)), x], axis=0)
    out = np.tile(bias[None, :], (n, 1)).astype(np.float64)
    for j in range(K):
        out += padded[j:j + n] * taps_w[:, j][None, :]
    return out


def selective_scan(u, dt, A, B, C, D):
    """u, dt [n, I]; A [I, N]; B, C [n, N]; D [I].  S_t = exp(dt_t A) * S_{t-1} + dt_t u_t B_t; y_t = S_t C_t + D u_t."""
    n, inner = u.shape
    S = np.zeros_like(A)
    y = np.zeros((n, inner))
    for t in range(n):
        S = np.exp(dt[t][:, None] * A) * S + (dt[t] * u[t])[:, None] * B[t][None, :]
        y[t] = S @ C[t] + D * u[t]
    return y


def mamba1(h, w, p, m):
    inner, rank, N = m["inner"], m["dt_rank"], m["state"]
    xz = h @ w[p + "in"].T
    x, z = xz[:, :inner], xz[:, inner:]
    x = silu(causal_conv(x, w[p + "conv"], w[p + "conv.b"]))
    low = x @ w[p + "x"].T
    dt = softplus(low[:, :rank] @ w[p + "dt"].T + w[p + "dt.b"])
    B, C = low[:, rank:rank + N], low[:, rank + N:rank + 2 * N]
    y = selective_scan(x, dt, -np.exp(w[p + "A_log"]), B, C, w[p + "D"])
    return (y * silu(z)) @ w[p + "o"].T


# ---- attention through a latent ------------------------------------------------------------------------------------------
def latent_attention(h, w, p, m, eps, positions=None):
    n = h.shape[0]
    positions = np.arange(n) if positions is None else positions
    H, dn, dr, dv, rk = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    base, rdims = m["rot"]["base"], m["rot"]["dims"]
    cq = rms_unit(h @ w[p + "dq"].T, w[p + "dq.norm"], eps)
    q = (cq @ w[p + "uq"].T).reshape(n, H, dn + dr)
    q_plain, q_rot = q[..., :dn], rotate_pairs(q[..., dn:], positions, base, rdims)
    down = h @ w[p + "dkv"].T
    c = rms_unit(down[:, :rk], w[p + "dkv.norm"], eps)
    k_rot = rotate_pairs(down[:, rk:], positions, base, rdims)                        # [n, dr], one for all heads
    k_plain = (c @ w[p + "uk"].T).reshape(n, H, dn)
    v = (c @ w[p + "uv"].T).reshape(n, H, dv)
    out = np.zeros((n, H, dv))
    visible = np.tril(np.ones((n, n), dtype=bool))
    for a in range(H):
        s = (q_plain[:, a] @ k_plain[:, a].T + q_rot[:, a] @ k_rot.T) * m["scale"]
        s = np.where(visible, s, -np.inf)
        sink = w[p + "sink"][a]
        top = np.maximum(s.max(axis=1), sink)
        e = np.exp(s - top[:, None])
        out[:, a] = (e / (e.sum(axis=1) + np.exp(sink - top))[:, None]) @ v[:, a]
    return out.reshape(n, H * dv) @ w[p + "o"].T


# ---- routed feed-forward ---------------------------------------------------------------------------------------------
def gated_unit(h, w, p):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def route(h, w, p, r):
    """(chosen [n, top], weight [n, top]): softmax over all router outputs; the choice adds the correction, the weight does not."""
    s = softmax(h @ w[p + "router"].T)
    chosen = np.argsort(-(s + w[p + "correction"]), axis=1, kind="stable")[:, :r["top"]]
    return chosen, np.take_along_axis(s, chosen, axis=1)


def moe(h, w, p, mlp):
    r = mlp["router"]
    chosen, weight = route(h, w, p, r)
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, g in zip(chosen[t], weight[t]):
            out[t] += g * (h[t] if e >= r["experts"] else gated_unit(h[t:t + 1], w, f"{p}e{e}.")[0])
    if mlp.get("shared"):
        out += sigmoid(h @ w[p + "shared.sg"].T) * gated_unit(h, w, p + "shared.")
    return out


# ---- the model --------------------------------------------------------------------------------------------------------
def run_order(config):
    """Layer indices in the order they run, with the number of the pass that starts at each (or None)."""
    n = len(config["layers"])
    loop = config.get("loop") or {"start": 0, "stop": 0, "times": 1}
    order = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"] if loop["stop"] > loop["start"] else 0):
        order += [(i, t if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
    order += [(i, None) for i in range(loop["stop"], n)]
    return order


def forward(config, w, tokens, return_layers=False):
    """Logits [n, vocab] for one whole sequence (and, if asked, the residual stream after every layer run)."""
    eps = config["norm"]["eps"]
    e0 = w["embed"][np.asarray(tokens)]
    x = e0.copy()
    streams = []
    for i, starts_pass in run_order(config):
        layer = config["layers"][i]
        p = f"l{i}."
        if starts_pass is not None:
            if starts_pass > 0:
                x = x + e0
            x = x + w["loop.step"][starts_pass]
        a = layer_norm(x, w[p + "norm1"], w[p + "norm1.b"], eps)
        if layer["type"] == "mamba1":
            mixed = mamba1(a, w, p + "mix.", layer["mixer"])
        elif layer["type"] == "latent_attention":
            mixed = latent_attention(a, w, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        fed = 0.0
        if layer.get("mlp"):
            fed = moe(layer_norm(x, w[p + "norm2"], w[p + "norm2.b"], eps), w, p + "mlp.", layer["mlp"])
        x = x + (mixed + fed)
        streams.append(x.copy())
    y = layer_norm(x, w["final.norm"], w["final.norm.b"], eps) @ w["head"].T
    cap = config.get("logit_softcap")
    if cap:
        y = cap * np.tanh(y / cap)
    return (y, np.stack(streams)) if return_layers else y


# ---- model folders ------------------------------------------------------------------------------------------------------
def tensor_shapes(config):
    """name -> shape of every tensor a model of this configuration has."""
    d, V = config["width"], config["vocab"]
    shapes = {"embed": (V, d), "final.norm": (d,), "final.norm.b": (d,), "head": (V, d)}
    loop = config.get("loop")
    if loop:
        shapes["loop.step"] = (loop["times"], d)
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        shapes[p + "norm1"] = shapes[p + "norm1.b"] = (d,)
        if layer["type"] == "mamba1":
            I, N, R, K = m["inner"], m["state"], m["dt_rank"], m["conv"]
            shapes.update({p + "mix.in": (2 * I, d), p + "mix.conv": (I, K), p + "mix.conv.b": (I,), p + "mix.x": (R + 2 * N, I),
                           p + "mix.dt": (I, R), p + "mix.dt.b": (I,), p + "mix.A_log": (I, N), p + "mix.D": (I,), p + "mix.o": (d, I)})
        else:
            H, dn, dr, dv = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
            shapes.update({p + "mix.dq": (m["q_rank"], d), p + "mix.dq.norm": (m["q_rank"],), p + "mix.uq": (H * (dn + dr), m["q_rank"]),
                           p + "mix.dkv": (m["kv_rank"] + dr, d), p + "mix.dkv.norm": (m["kv_rank"],), p + "mix.uk": (H * dn, m["kv_rank"]),
                           p + "mix.uv": (H * dv, m["kv_rank"]), p + "mix.sink": (H,), p + "mix.o": (d, H * dv)})
        mlp = layer.get("mlp")
        if mlp:
            shapes[p + "norm2"] = shapes[p + "norm2.b"] = (d,)
            r, f = mlp["router"], mlp["expert"]["ff"]
            for e in range(r["experts"]):
                shapes.update({f"{p}mlp.e{e}.gate": (f, d), f"{p}mlp.e{e}.up": (f, d), f"{p}mlp.e{e}.down": (d, f)})
            shapes[p + "mlp.router"] = (r["experts"] + r["identity"], d)
            shapes[p + "mlp.correction"] = (r["experts"] + r["identity"],)
            if mlp.get("shared"):
                fs = mlp["shared"]["ff"]
                shapes.update({p + "mlp.shared.gate": (fs, d), p + "mlp.shared.up": (fs, d), p + "mlp.shared.down": (d, fs), p + "mlp.shared.sg": (1, d)})
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
        if name.endswith("norm") or name.endswith("dq.norm") or name.endswith("dkv.norm"):
            v = 1.0 + 0.2 * rng.standard_normal(shape)
        elif leaf == "b" and "norm" in name:
            v = 0.1 * rng.standard_normal(shape)
        elif leaf == "A_log":
            v = np.log(rng.uniform(0.5, 8.0, shape))
        elif name.endswith("dt.b"):
            v = np.log(np.expm1(rng.uniform(0.01, 0.3, shape)))
        elif leaf == "D":
            v = 1.0 + 0.2 * rng.standard_normal(shape)
        elif leaf in ("sink", "correction"):
            v = 0.5 * rng.standard_normal(shape) * (0.2 if leaf == "correction" else 1.0)
        elif name.endswith("conv.b"):
            v = 0.1 * rng.standard_normal(shape)
        elif name in ("embed", "loop.step"):
            v = rng.standard_normal(shape) * (1.0 if name == "embed" else 0.3)
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
