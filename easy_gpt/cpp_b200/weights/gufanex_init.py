"""Random-weights mode for the Gufanex decoder: the names and shapes of the tensors a configuration asks for, and a
writer of a model folder (config.json, model.safetensors in bfloat16) from a configuration and a seed.

Made for models of several gigabytes: matrices are cut out of one pool of random bfloat16 values at offsets drawn
per tensor, so a folder is written at the speed of the disk.  Constants that must be sane for the model to run
(norm gains, the decays' logarithms, the step sizes' biases) get values of their own.  numpy only.
"""
from __future__ import annotations

import json
import struct
from pathlib import Path

import numpy as np


def tensor_shapes(config: dict) -> dict:
    d, vocab = config["width"], config["vocab"]
    shapes = {"embed": (vocab, d), "final.norm": (d,), "final.norm.b": (d,), "head": (vocab, d)}
    loop = config.get("loop")
    if loop and loop["stop"] > loop["start"]:
        shapes["loop.step"] = (loop["times"], d)
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        shapes[p + "norm1"] = shapes[p + "norm1.b"] = (d,)
        if layer["type"] == "mamba1":
            inner, n, r, k = m["inner"], m["state"], m["dt_rank"], m["conv"]
            shapes.update({p + "mix.in": (2 * inner, d), p + "mix.conv": (inner, k), p + "mix.conv.b": (inner,), p + "mix.x": (r + 2 * n, inner),
                           p + "mix.dt": (inner, r), p + "mix.dt.b": (inner,), p + "mix.A_log": (inner, n), p + "mix.D": (inner,), p + "mix.o": (d, inner)})
        elif layer["type"] == "latent_attention":
            h, dn, dr, dv = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
            shapes.update({p + "mix.dq": (m["q_rank"], d), p + "mix.dq.norm": (m["q_rank"],), p + "mix.uq": (h * (dn + dr), m["q_rank"]),
                           p + "mix.dkv": (m["kv_rank"] + dr, d), p + "mix.dkv.norm": (m["kv_rank"],), p + "mix.uk": (h * dn, m["kv_rank"]),
                           p + "mix.uv": (h * dv, m["kv_rank"]), p + "mix.sink": (h,), p + "mix.o": (d, h * dv)})
        else:
            raise ValueError(f"layers[{i}].type '{layer['type']}' is no mixer of this design")
        mlp = layer.get("mlp")
        if mlp:
            shapes[p + "norm2"] = shapes[p + "norm2.b"] = (d,)
            r = mlp["router"]
            outputs = r["experts"] + r.get("identity", 0)
            for e in range(r["experts"]):
                f = mlp["expert"]["ff"]
                shapes.update({f"{p}mlp.e{e}.gate": (f, d), f"{p}mlp.e{e}.up": (f, d), f"{p}mlp.e{e}.down": (d, f)})
            shapes[p + "mlp.router"] = (outputs, d)
            shapes[p + "mlp.correction"] = (outputs,)
            if mlp.get("shared"):
                f = mlp["shared"]["ff"]
                shapes.update({p + "mlp.shared.gate": (f, d), p + "mlp.shared.up": (f, d), p + "mlp.shared.down": (d, f), p + "mlp.shared.sg": (1, d)})
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
        if leaf in ("norm", "norm1", "norm2", "D"):
            return _bf16_bits(np.ones(n))
        if leaf in ("sink", "correction") or (leaf == "b" and "norm" in name):
            return _bf16_bits(np.zeros(n))
        if leaf == "b":
            return _bf16_bits(rng.standard_normal(n) * std)
        if leaf == "A_log":
            return _bf16_bits(np.log(rng.uniform(1.0, 16.0, n)))
        if name.endswith("conv"):
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
            if name.endswith("dt.b"):
                # step sizes between 1e-3 and 1e-1 at zero input: softplus^-1
                f.write(_bf16_bits(np.log(np.expm1(rng.uniform(1e-3, 1e-1, int(np.prod(shape)))))).tobytes())
            else:
                f.write(values(name, shape).tobytes())
    return folder
