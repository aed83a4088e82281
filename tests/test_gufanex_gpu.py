"""The Gufanex decoder in the native engine against the plain numpy restatement (tests/plain_gufanex.py): each
mechanism alone, prompts cut in every way, batches, reused pages and slots, long decoding, odd sizes, generation.

Every test makes its own small configuration and random weights.  Errors are the largest difference of a logit over
the largest logit: float32 must stay within 1e-4, bfloat16 within 3e-2.
"""
import copy
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

import plain_gufanex as pg

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
TOL = {"float32": 1e-4, "bfloat16": 3e-2}


def scan(inner=96, state=8, dt_rank=5, conv=4):
    return {"type": "mamba1", "mixer": {"inner": inner, "state": state, "dt_rank": dt_rank, "conv": conv}}


def latent(heads=2, dim=16, rot_dim=8, vdim=24, kv_rank=40, q_rank=48, scale=0.2, base=10000.0):
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
                                                  "scale": scale, "rot": {"base": base, "dims": rot_dim}}}


def routed(experts=4, identity=2, top=2, ff=48, shared=40):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "identity": identity, "top": top}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def model(layers, width=64, vocab=131, loop=None, softcap=8.0, eps=1e-5):
    cfg = {"architecture": "Gufanex", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": []}
    for mixer, mlp in layers:
        cfg["layers"].append({**copy.deepcopy(mixer), "mlp": copy.deepcopy(mlp)})
    if loop:
        cfg["loop"] = dict(zip(("start", "stop", "times"), loop))
    if softcap:
        cfg["logit_softcap"] = softcap
    return cfg


GENERAL = model([(scan(), routed()), (latent(), routed(top=3)), (scan(inner=80, state=6, dt_rank=3, conv=3), None),
                 (latent(heads=3, dim=8, rot_dim=4, vdim=8, kv_rank=24, q_rank=16, scale=0.35, base=300.0), routed(top=1, identity=0, shared=0))],
                loop=(1, 3, 2))
# widths that leave the decode product's alignment rule, a state count that is no power of two, single heads and taps
ODD = model([(latent(heads=3, dim=12, rot_dim=6, vdim=10, kv_rank=20, q_rank=28, scale=0.3), routed(experts=1, identity=1, top=1, ff=20, shared=12)),
             (scan(inner=40, state=3, dt_rank=1, conv=2), routed(experts=3, identity=0, top=3, ff=24, shared=0))], width=72, vocab=77, softcap=None)
# sizes of one: one head, one state, one tap (no convolution state), one pass of a loop over everything, every output chosen
ONES = model([(scan(inner=32, state=1, dt_rank=2, conv=1), routed(experts=2, identity=1, top=3, ff=16, shared=16)),
              (latent(heads=1, dim=16, rot_dim=16, vdim=16, kv_rank=16, q_rank=16, scale=0.25), None)], width=48, vocab=64, loop=(0, 2, 1), softcap=20.0)


def tokens(vocab, n, seed):
    return np.random.default_rng(seed).integers(0, vocab, n).tolist()


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    made = {}

    def get(name, cfg, seed=0, overrides=None):
        if name not in made:
            w = pg.random_weights(cfg, seed, overrides)
            made[name] = (pg.write_model_dir(tmp_path_factory.mktemp(name), cfg, w), cfg, w)
        return made[name]

    return get


def runner(folder, dtype, pool_tokens=512, page_size=16, slots=4, graphs=True):
    from easy_gpt.cpp_b200.native import NativeStepRunner

    return NativeStepRunner(folder, dtype, page_size=page_size, num_pages=pool_tokens // page_size, max_slots=slots, max_tokens_per_request=pool_tokens,
                            use_graphs=graphs)


def close(got, want, dtype, what=""):
    err = float(np.abs(got - want).max() / np.abs(want).max())
    assert err <= TOL[dtype], f"{what}: error {err:.3g} over {TOL[dtype]:.3g}"


ALONE = {
    "scan": model([(scan(), None)], loop=None),
    "scan_many_states": model([(scan(inner=24, state=70, dt_rank=4, conv=5), None)]),
    "latent": model([(latent(), None)]),
    "latent_wide": model([(latent(heads=4, dim=24, rot_dim=16, vdim=32, kv_rank=200, q_rank=72, scale=0.1), None)]),
    "routed": model([(scan(inner=16, state=2, dt_rank=1, conv=2), routed())]),
    "routed_many": model([(scan(inner=16, state=2, dt_rank=1, conv=2), routed(experts=40, identity=5, top=6, ff=16, shared=0))]),
    "loop": model([(scan(inner=32, state=4), None), (latent(), None)], loop=(0, 2, 3)),
    # more heads than one tile of the tensor-core attention has rows
    "latent_many_heads": model([(latent(heads=20, dim=8, rot_dim=8, vdim=8, kv_rank=16, q_rank=16, scale=0.25), None)]),
    # sizes that the grouped product on the tensor cores takes (steps of 33 tokens and more, bfloat16)
    "routed_grouped": model([(scan(inner=16, state=2, dt_rank=8, conv=2), routed(experts=5, identity=2, top=3, ff=64, shared=64))], width=128),
    "scan_wide_rank": model([(scan(inner=64, state=16, dt_rank=16, conv=4), None)], width=64),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ALONE))
def test_each_mechanism_alone(folders, name, dtype):
    folder, cfg, w = folders(name, ALONE[name], seed=3)
    toks = tokens(cfg["vocab"], 45, 1)
    got = runner(folder, dtype).run([("a", toks, list(range(45)))])
    close(got, pg.forward(cfg, w, toks), dtype, name)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,cfg", [("general", GENERAL), ("odd", ODD), ("ones", ONES), ("alone_scan_wide_rank", None), ("alone_routed_grouped", None),
                                      ("alone_latent_many_heads", None), ("alone_latent_wide", None)])
def test_prompt_whole_and_token_by_token(folders, name, cfg, dtype):
    if cfg is None:                                  # the single-mechanism models whose decode steps take other kernels than their prompts
        name = name[len("alone_"):]
        cfg = ALONE[name]
    folder, cfg, w = folders(name, cfg, seed=3 if name in ALONE else 5)
    toks = tokens(cfg["vocab"], 70, 2)
    want = pg.forward(cfg, w, toks)
    r = runner(folder, dtype)
    close(r.run([("whole", toks, list(range(70)))]), want, dtype, "whole")
    r.end("whole")
    rows = [r.run([("single", [t], [0])])[0] for t in toks]
    close(np.stack(rows), want, dtype, "token by token")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("sizes", [[2] * 20, [3, 1, 2, 17, 1, 1, 30, 5, 2, 2, 16, 15, 1, 33], [16, 16, 16, 16, 1, 15, 48], [1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12]])
def test_portions(folders, sizes, dtype):
    """Portions down to two tokens, shorter than the convolution's reach, ending on and beside page borders."""
    folder, cfg, w = folders("general", GENERAL, seed=5)
    toks = tokens(cfg["vocab"], sum(sizes), 7)
    want = pg.forward(cfg, w, toks)
    r = runner(folder, dtype, page_size=16)
    at, rows = 0, []
    for n in sizes:
        rows.append(r.run([("p", toks[at:at + n], list(range(n)))]))
        at += n
    close(np.concatenate(rows), want, dtype, f"portions {sizes}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_batches_of_unequal_requests(folders, dtype):
    """Four requests of different lengths advance together, portions beside single tokens; each must come out as alone."""
    folder, cfg, w = folders("general", GENERAL, seed=5)
    lengths = {"a": 61, "b": 9, "c": 130, "d": 33}
    toks = {k: tokens(cfg["vocab"], n, 10 + i) for i, (k, n) in enumerate(lengths.items())}
    want = {k: pg.forward(cfg, w, v) for k, v in toks.items()}
    plans = {"a": [40] + [1] * 21, "b": [1] * 9, "c": [2, 64, 31, 1, 1, 30, 1], "d": [16, 17]}
    r = runner(folder, dtype, pool_tokens=512)
    at = {k: 0 for k in toks}
    got = {k: [] for k in toks}
    step = 0
    while any(plans.values()):
        entries, names = [], []
        for k in sorted(plans):
            if plans[k] and (step % 3 != 2 or k != "b"):            # b sits out every third step
                n = plans[k].pop(0)
                entries.append((k, toks[k][at[k]:at[k] + n], list(range(n))))
                names.append((k, n))
                at[k] += n
        if entries:
            out = r.run(entries)
            row = 0
            for k, n in names:
                got[k].append(out[row:row + n])
                row += n
        step += 1
    for k in toks:
        close(np.concatenate(got[k]), want[k], dtype, f"request {k}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_pages_and_slots_are_used_again(folders, dtype):
    """Two slots and a pool of four pages: every request takes a slot and pages that another one has left full."""
    folder, cfg, w = folders("general", GENERAL, seed=5)
    r = runner(folder, dtype, pool_tokens=64, page_size=16, slots=2)
    for i in range(6):
        a, b = tokens(cfg["vocab"], 20 + i, 40 + i), tokens(cfg["vocab"], 31 - i, 60 + i)
        out = r.run([(f"a{i}", a[:7], []), (f"b{i}", b, [len(b) - 1])])
        close(out, pg.forward(cfg, w, b)[-1:], dtype, f"b{i}")
        r.end(f"b{i}")
        out = r.run([(f"a{i}", a[7:], list(range(len(a) - 7)))])
        close(out, pg.forward(cfg, w, a)[7:], dtype, f"a{i}")
        r.end(f"a{i}")
    assert r.info("live_requests") == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_far_keys_and_slow_states(folders, dtype):
    """Weights made so that faults far back show: sharp attention (large query maps, so single keys carry the softmax),
    states that hardly decay, sinks that take most of the weight of some heads.  A prompt over many pages, then decoding."""
    cfg = GENERAL
    base = pg.random_weights(cfg, 9)
    over = {}
    for i, layer in enumerate(cfg["layers"]):
        if layer["type"] == "latent_attention":
            over[f"l{i}.mix.uq"] = base[f"l{i}.mix.uq"] * 3.0
            over[f"l{i}.mix.sink"] = np.linspace(-2.0, 5.0, layer["mixer"]["heads"])
        else:
            over[f"l{i}.mix.A_log"] = np.log(np.full_like(base[f"l{i}.mix.A_log"], 2e-3))
    folder, cfg, w = folders("pointed", cfg, seed=9, overrides=over)
    toks = tokens(cfg["vocab"], 400, 21)
    want = pg.forward(cfg, w, toks)
    r = runner(folder, dtype, pool_tokens=448, page_size=16)
    ask = [0, 1, 15, 16, 17, 255, 256, 330, 339]
    rows = [r.run([("f", toks[:340], ask)])] + [r.run([("f", [t], [0])]) for t in toks[340:]]
    close(np.concatenate(rows), np.concatenate([want[ask], want[340:]]), dtype, "pointed weights")
    # the sinks matter: without them the logits are elsewhere
    no_sink = dict(w)
    for i, layer in enumerate(cfg["layers"]):
        if layer["type"] == "latent_attention":
            no_sink[f"l{i}.mix.sink"] = np.full(layer["mixer"]["heads"], -1e9)
    assert np.abs(pg.forward(cfg, no_sink, toks[:64]) - want[:64]).max() > 20 * TOL[dtype] * np.abs(want).max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_through_captured_steps(folders, dtype):
    folder, cfg, w = folders("odd", ODD, seed=5)
    toks = tokens(cfg["vocab"], 240, 31)
    want = pg.forward(cfg, w, toks)
    r = runner(folder, dtype, pool_tokens=512)
    rows = [r.run([("x", toks[:5], [4]), ("y", toks[:3], [])])]
    rows += [r.run([("x", [t], [0]), ("y", [u], [0])])[:1] for t, u in zip(toks[5:], toks[3:])]
    close(np.concatenate(rows), want[4:], dtype, "decoding")
    assert r.info("graph_replays") > 200


def test_first_tokens_of_a_sequence(folders):
    """Position 0 alone, then position 1: nothing before the sequence leaks in (zeros before the convolution, an empty
    state, a softmax over one key and the sink)."""
    folder, cfg, w = folders("general", GENERAL, seed=5)
    r = runner(folder, "float32")
    for seed in range(3):
        toks = tokens(cfg["vocab"], 2, 80 + seed)
        want = pg.forward(cfg, w, toks)
        close(r.run([(seed, toks[:1], [0])]), want[:1], "float32", "first token")
        close(r.run([(seed, toks[1:], [0])]), want[1:], "float32", "second token")
        r.end(seed)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(folders, dtype):
    """The scheduler's own entry point: prompts in portions beside decoding requests, greedy; each generated token must be
    (within the tolerance) the plain implementation's best token after the same prefix."""
    from easy_gpt.cpp_b200.native import NativeEngine

    folder, cfg, w = folders("general", GENERAL, seed=5)
    prompts = [tokens(cfg["vocab"], n, 90 + n) for n in (3, 41, 18, 70, 9, 26)]
    engine = NativeEngine(folder, dtype=dtype, page_size=16, cache_tokens=512, max_active=4, chunk_size=16, max_batch_tokens=48)
    outputs = engine.generate(prompts, max_new_tokens=12, greedy=True)
    for prompt, out in zip(prompts, outputs):
        assert len(out) == 12
        logits = pg.forward(cfg, w, prompt + out)
        for i, tok in enumerate(out):
            row = logits[len(prompt) + i - 1]
            assert float(row.max() - row[tok]) <= 4 * TOL[dtype] * np.abs(row).max(), (dtype, i, tok, int(row.argmax()))


def test_trace_replay_program(folders, tmp_path):
    """bin/trace_run on a model folder of this design: steps in, logits files out."""
    import json

    folder, cfg, w = folders("odd", ODD, seed=5)
    toks = tokens(cfg["vocab"], 40, 55)
    steps = [{"step": 0, "entries": [{"id": "q", "tokens": toks[:30], "want": [0, 29]}], "end": []},
             {"step": 1, "entries": [{"id": "q", "tokens": toks[30:], "want": [9]}, {"id": "z", "tokens": toks[:2], "want": []}], "end": ["q", "z"]}]
    out = tmp_path / "out"
    run = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", "float32", "--out", str(out), "--max-tokens", "128"],
                         input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, run.stderr
    assert [l for l in run.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1"]
    want = pg.forward(cfg, w, toks)
    close(np.fromfile(out / "0.f32", dtype="<f4").reshape(2, -1), want[[0, 29]], "float32", "step 0")
    close(np.fromfile(out / "1.f32", dtype="<f4").reshape(1, -1), want[[39]], "float32", "step 1")


def test_command_line_with_random_weights(tmp_path):
    """The engine's own program on this design: random-weights mode writes a folder from a config.json (with the
    per-tensor hints that keep norms, decays and step sizes sane), then prompts of token ids are decoded greedily; the
    tokens must be the plain implementation's for the weights that were written."""
    import json

    cfg = model([(scan(inner=48, state=4, dt_rank=8, conv=3), routed(experts=3, identity=1, top=2, ff=32, shared=32)), (latent(), None)], width=64,
                vocab=97, loop=(0, 2, 2))
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    prompts = tmp_path / "prompts.txt"
    prompts.write_text("5 17 3\n9,8,7,6\n")
    folder = tmp_path / "model"
    folder.mkdir()
    cmd = [sys.executable, str(ROOT / "bin" / "easy_llm"), "--model", str(folder), "--random-weights", "7", "--config", str(tmp_path / "config.json"),
           "--token-ids", "--greedy", "--max-steps", "10", "--dtype", "float32", "-f", str(prompts)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    outs = [[int(t) for t in line.split()] for line in (tmp_path / "prompts_output.txt").read_text().splitlines()]
    assert len(outs) == 2 and len(outs[0]) == 8 and len(outs[1]) == 7
    cfg_read, w = pg.read_model_dir(folder)
    assert np.all(w["l0.norm1"] == 1.0) and np.all(w["l0.mix.D"] == 1.0) and np.all(w["l1.mix.sink"] == 0.0) and w["l0.mix.A_log"].min() >= 0.0
    for prompt, out in zip([[5, 17, 3], [9, 8, 7, 6]], outs):
        logits = pg.forward(cfg_read, w, prompt + out)
        for i, tok in enumerate(out):
            row = logits[len(prompt) + i - 1]
            assert float(row.max() - row[tok]) <= 4e-4 * np.abs(row).max(), (i, tok, int(row.argmax()))
