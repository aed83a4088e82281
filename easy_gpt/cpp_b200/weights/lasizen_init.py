"""Random-weights mode for the Lasizen decoder: the names and shapes of the tensors a configuration asks for, and a
writer of a model folder (config.json, model.safetensors in bfloat16) from a configuration and a seed.

Made for models of several gigabytes: matrices are cut out of one pool of random bfloat16 values at offsets drawn
per tensor, so a folder is written at the speed of the disk.  Constants that must be sane for the model to run
(norm gains, shift weights, the decays' logarithms, the step sizes' biases) get values of their own.  numpy only.
"""
from __future__ import annotations

import json
import struct
from pathlib import Path

import numpy as np


def tensor_shapes(config: dict) -> dict:
    d, vocab = config["width"], config["vocab"]
    shapes = {"embed": (vocab, d), "final.norm": (d,), "head": (vocab, d)}
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        shapes[p + "norm1"] = shapes[p + "norm1b"] = shapes[p + "shift"] = (d,)
        heads, groups, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        if layer["type"] == "attention":
            shapes.update({p + "mix.q": (heads * dk, d), p + "mix.k": (groups * dk, d), p + "mix.v": (groups * dv, d), p + "mix.o": (d, heads * dv)})
        elif layer["type"] == "delta":
            taps = m["conv"]
            shapes.update({p + "mix.q": (groups * dk, d), p + "mix.q.conv": (groups * dk, taps), p + "mix.k": (groups * dk, d),
                           p + "mix.k.conv": (groups * dk, taps), p + "mix.v": (heads * dv, d), p + "mix.v.conv": (heads * dv, taps),
                           p + "mix.b": (heads, d), p + "mix.a": (heads, d), p + "mix.A_log": (heads,), p + "mix.dt_bias": (heads,),
                           p + "mix.norm": (dv,), p + "mix.g": (heads * dv, d), p + "mix.o": (d, heads * dv)})
        else:
            raise ValueError(f"layers[{i}].type '{layer['type']}' is no mixer of this design")
        mlp = layer.get("mlp")
        if mlp:
            shapes[p + "norm2"] = shapes[p + "norm2b"] = (d,)
            shapes.update({p + "mlp.up": (mlp["ff"], d), p + "mlp.down": (d, mlp["ff"]), p + "mlp.act": (2,)})
    return shapes


def _bf16_bits(a: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def write_random_model(folder, config: dict, seed: int, std: float = 0.02) -> Path:
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    shapes = tensor_shapes(config)
    rng = np.random.default_rng(seed)
    pool = _bf16_bits(rng.standard_normal(1 << 24) * std)
    (folder / "config.json").write_text(json.dumps(config, indent=1))

    def values(name, shape):
        n = int(np.prod(shape))
        leaf = name.split(".")[-1]
        if leaf in ("norm", "norm1", "norm2", "norm1b", "norm2b"):
            return _bf16_bits(np.ones(n))
        if leaf == "shift":
            return _bf16_bits(np.full(n, 0.5))
        if leaf == "A_log":
            return _bf16_bits(np.log(rng.uniform(1.0, 16.0, n)))
        if leaf == "dt_bias":
            return _bf16_bits(np.log(np.expm1(rng.uniform(1e-3, 1e-1, n))))      # step sizes between 1e-3 and 1e-1 at zero input
        if leaf == "act":
            return _bf16_bits(rng.standard_normal(n))
        if leaf == "conv":
            return _bf16_bits(rng.standard_normal(n) * 0.3)
        out = np.empty(n, dtype=np.uint16)
        at = 0
        while at < n:
            take = min(n - at, len(pool) // 2)
            start = int(rng.integers(0, len(pool) - take))
            out[at:at + take] = pool[start:start + take]
            at += take
        return out

    header, at = {}, 0
    for name, shape in shapes.items():
        size = int(np.prod(shape)) * 2
        header[name] = {"dtype": "BF16", "shape": list(shape), "data_offsets": [at, at + size]}
        at += size
    head = json.dumps(header).encode()
    head += b" " * (-len(head) % 8)
    with open(folder / "model.safetensors", "wb") as f:
        f.write(struct.pack("<Q", len(head)) + head)
        for name, shape in shapes.items():
            f.write(values(name, shape).tobytes())
    return folder
