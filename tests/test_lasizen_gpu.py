"""The Lasizen decoder in the native engine against the plain numpy restatement (tests/plain_lasizen.py): each mechanism
alone, prompts cut in every way, batches, reused pages and slots, window edges, far keys, long decoding, odd sizes,
generation.

Every test makes its own small configuration and random weights.  Errors are the largest difference of a logit over
the largest logit: float32 must stay within 1e-4.  In bfloat16 every branch's input and output is rounded to eight bits
of mantissa before it joins the stream, and these untrained models pass nothing else on (the restatement with those
roundings put in is 4e-2 away at its worst logit): there the bound is 3e-2 on the root mean square of all differences
(over the root mean square of the logits) and 8e-2 on the largest one; the faults that the pointed tests plant move
logits by 0.25 and more.
"""
import copy
import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

import plain_lasizen as pl

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
TOL = {"float32": 1e-4, "bfloat16": 3e-2}
LARGEST = {"float32": 1e-4, "bfloat16": 8e-2}


def attention(heads=4, kv_heads=2, dim=16, vdim=24, scale=0.3, window=20, rot_dims=8, base=10000.0, scaling=(4.0, 64, 16.0, 2.0)):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window:
        m["mask"] = {"size": window}
    if rot_dims:
        m["rot"] = {"base": base, "dims": rot_dims}
        if scaling:
            m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return {"type": "attention", "mixer": m}


def delta(heads=4, kv_heads=2, dim=16, vdim=24, conv=4):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}}


def model(layers, width=64, vocab=131, loop=None, eps=1e-5, embedding_scale=4.0, logit_scale=0.5):
    cfg = {"architecture": "Lasizen", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": []}
    for mixer, ff in layers:
        cfg["layers"].append({**copy.deepcopy(mixer), "mlp": {"kind": "dense", "ff": ff} if ff else None})
    if loop:
        cfg["loop"] = dict(zip(("start", "stop", "times"), loop))
    if embedding_scale:
        cfg["embedding"] = {"scale": embedding_scale}
    if logit_scale:
        cfg["logit_scale"] = logit_scale
    return cfg


GENERAL = model([(attention(), 96), (delta(), 80), (attention(heads=3, kv_heads=1, dim=8, vdim=8, scale=0.5, window=33, rot_dims=8, scaling=None), None),
                 (delta(heads=2, kv_heads=2, dim=24, vdim=8, conv=3), 48)], loop=(1, 3, 2))
# widths that leave the decode product's alignment rule, head sizes that are no powers of two, two taps, a rotation over part of an odd-sized head
ODD = model([(delta(heads=3, kv_heads=1, dim=20, vdim=10, conv=2), 52), (attention(heads=3, kv_heads=3, dim=12, vdim=10, scale=0.4, window=7, rot_dims=6, base=300.0), 36)],
            width=72, vocab=77, embedding_scale=None)
# values that are one or equal: one head, one key head, one tap (no convolution state), a window of one (a token sees itself and
# the sink), one pass of a loop over everything, key and value sizes equal, the whole head rotated, no scales
ONES = model([(delta(heads=1, kv_heads=1, dim=16, vdim=16, conv=1), None), (attention(heads=1, kv_heads=1, dim=16, vdim=16, scale=1.0, window=1, rot_dims=16), 32),
              (attention(heads=2, kv_heads=2, dim=8, vdim=8, scale=0.7, window=None, rot_dims=None), None)], width=48, vocab=64, loop=(0, 3, 1),
             embedding_scale=None, logit_scale=None)

ALONE = {
    "attention": model([(attention(), None)]),
    "attention_all_keys": model([(attention(window=None), None)]),
    "attention_no_rotation": model([(attention(rot_dims=None), None)]),
    "attention_wide": model([(attention(heads=8, kv_heads=2, dim=64, vdim=48, scale=0.11, window=40, rot_dims=24, base=5e5, scaling=(6.0, 1024, 24.0, 2.0)), None)], width=128),
    # key and value sizes equal: keys and values in planes of their own, which the tensor-core kernels read in bfloat16
    "attention_planes_64": model([(attention(heads=4, kv_heads=2, dim=64, vdim=64, scale=0.125, window=40, rot_dims=32), None)], width=128),
    "attention_planes_128": model([(attention(heads=2, kv_heads=1, dim=128, vdim=128, scale=0.09, window=None, rot_dims=64, scaling=None), None)], width=128),
    "attention_planes_32": model([(attention(heads=6, kv_heads=3, dim=32, vdim=32, scale=0.2, window=33, rot_dims=8), 64)]),
    "attention_planes_256": model([(attention(heads=2, kv_heads=2, dim=256, vdim=256, scale=0.06, window=45, rot_dims=128, scaling=None), None)], width=96),
    # a width that is no multiple of four, sizes that are no multiples of four either
    "odd_width": model([(attention(heads=3, kv_heads=1, dim=10, vdim=6, scale=0.4, window=9, rot_dims=4), 27), (delta(heads=2, kv_heads=1, dim=6, vdim=10, conv=3), None)],
                       width=90, vocab=53),
    "attention_large_values": model([(attention(heads=2, kv_heads=1, dim=24, vdim=136, scale=0.25, window=50), None)]),
    "delta": model([(delta(), None)]),
    "delta_wide": model([(delta(heads=4, kv_heads=2, dim=128, vdim=64, conv=4), None)], width=128),
    "delta_long_keys": model([(delta(heads=2, kv_heads=1, dim=200, vdim=40, conv=5), None)]),
    "delta_many_values": model([(delta(heads=2, kv_heads=2, dim=40, vdim=200, conv=2), None)]),
    "feed_forward": model([(delta(conv=2), 100)]),
    "loop": model([(delta(), None), (attention(), 64)], loop=(0, 2, 3)),
}


def tokens(vocab, n, seed):
    return np.random.default_rng(seed).integers(0, vocab, n).tolist()


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    made = {}

    def get(name, cfg, seed=0, overrides=None):
        if name not in made:
            w = pl.random_weights(cfg, seed, overrides)
            made[name] = (pl.write_model_dir(tmp_path_factory.mktemp(name), cfg, w), cfg, w)
        return made[name]

    return get


def runner(folder, dtype, pool_tokens=512, page_size=16, slots=4, graphs=True, most_tokens=None):
    from easy_gpt.cpp_b200.native import NativeStepRunner

    return NativeStepRunner(folder, dtype, page_size=page_size, num_pages=pool_tokens // page_size, max_slots=slots,
                            max_tokens_per_request=most_tokens or pool_tokens, use_graphs=graphs)


def close(got, want, dtype, what=""):
    diff = np.asarray(got, dtype=np.float64) - want
    largest = float(np.abs(diff).max() / np.abs(want).max())
    assert largest <= LARGEST[dtype], f"{what}: largest error {largest:.3g} over {LARGEST[dtype]:.3g}"
    spread = float(np.sqrt((diff * diff).mean()) / np.sqrt((want * want).mean()))
    assert spread <= TOL[dtype] or dtype == "float32", f"{what}: error {spread:.3g} over {TOL[dtype]:.3g}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ALONE))
def test_each_mechanism_alone(folders, name, dtype):
    folder, cfg, w = folders(name, ALONE[name], seed=3)
    toks = tokens(cfg["vocab"], 75, 1)
    got = runner(folder, dtype).run([("a", toks, list(range(75)))])
    close(got, pl.forward(cfg, w, toks), dtype, name)


def test_residual_stream_after_every_layer_run():
    """The restatement's own pieces against each other: the loop's passes are separate runs, and a run order without a loop
    is the layers in order."""
    cfg = GENERAL
    assert pl.run_order(cfg) == [0, 1, 2, 1, 2, 3]
    w = pl.random_weights(cfg, 1)
    logits, streams = pl.forward(cfg, w, tokens(cfg["vocab"], 9, 0), return_layers=True)
    assert streams.shape == (6, 9, cfg["width"]) and logits.shape == (9, cfg["vocab"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,cfg", [("general", GENERAL), ("odd", ODD), ("ones", ONES), ("alone_attention_wide", None), ("alone_delta_wide", None),
                                      ("alone_delta_long_keys", None), ("alone_attention_large_values", None), ("alone_attention_planes_64", None),
                                      ("alone_attention_planes_128", None), ("alone_attention_planes_32", None), ("alone_attention_planes_256", None),
                                      ("alone_odd_width", None)])
def test_prompt_whole_and_token_by_token(folders, name, cfg, dtype):
    if cfg is None:
        name = name[len("alone_"):]
        cfg = ALONE[name]
    folder, cfg, w = folders(name, cfg, seed=3 if name in ALONE else 5)
    toks = tokens(cfg["vocab"], 70, 2)
    want = pl.forward(cfg, w, toks)
    r = runner(folder, dtype)
    close(r.run([("whole", toks, list(range(70)))]), want, dtype, "whole")
    r.end("whole")
    rows = [r.run([("single", [t], [0])])[0] for t in toks]
    close(np.stack(rows), want, dtype, "token by token")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("sizes", [[2] * 20, [3, 1, 2, 17, 1, 1, 30, 5, 2, 2, 16, 15, 1, 33], [16, 16, 16, 16, 1, 15, 48], [1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12]])
def test_portions(folders, sizes, dtype):
    """Portions down to two tokens, shorter than the convolution's reach and than the windows, ending on and beside page borders."""
    folder, cfg, w = folders("general", GENERAL, seed=5)
    toks = tokens(cfg["vocab"], sum(sizes), 7)
    want = pl.forward(cfg, w, toks)
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
    want = {k: pl.forward(cfg, w, v) for k, v in toks.items()}
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
    """Two slots and a pool of four pages: every request takes a slot (shift rows, convolution inputs, delta states) and
    pages that another one has left full."""
    folder, cfg, w = folders("general", GENERAL, seed=5)
    r = runner(folder, dtype, pool_tokens=64, page_size=16, slots=2)
    for i in range(6):
        a, b = tokens(cfg["vocab"], 20 + i, 40 + i), tokens(cfg["vocab"], 31 - i, 60 + i)
        out = r.run([(f"a{i}", a[:7], []), (f"b{i}", b, [len(b) - 1])])
        close(out, pl.forward(cfg, w, b)[-1:], dtype, f"b{i}")
        r.end(f"b{i}")
        out = r.run([(f"a{i}", a[7:], list(range(len(a) - 7)))])
        close(out, pl.forward(cfg, w, a)[7:], dtype, f"a{i}")
        r.end(f"a{i}")
    assert r.info("live_requests") == 0


def test_windowed_pool_holds_long_requests(folders):
    """A request far longer than the pool: the windows give pages back while it runs."""
    cfg = model([(attention(window=20), 32), (attention(heads=2, kv_heads=1, dim=8, vdim=8, window=33, rot_dims=4), None)])
    folder, cfg, w = folders("windows_only", cfg, seed=8)
    toks = tokens(cfg["vocab"], 300, 3)
    want = pl.forward(cfg, w, toks)
    r = runner(folder, "float32", pool_tokens=96, page_size=16, slots=2, most_tokens=512)
    rows, at = [], 0
    for n in [30, 17, 2, 31] + [20] * 11:
        rows.append(r.run([("long", toks[at:at + n], list(range(n)))]))
        at += n
    close(np.concatenate(rows), want, "float32", "300 tokens through six pages")


def aimed(cfg, seed, a, b, sharp=6.0):
    """Weights under which one score stands out in the first layer (an attention layer): the key maps are the query maps of
    their groups' first heads behind a reflection of the model's width that carries token b's normed embedding onto token
    a's.  A token b that follows another b (the shift then leaves its row as it is) is the key that a token a behind
    another a looks for, whatever lies between them; b's value is its own.  Delta states hardly decay."""
    cfg = copy.deepcopy(cfg)
    base = pl.random_weights(cfg, seed)
    m = cfg["layers"][0]["mixer"]
    m["scale"] = sharp / float(np.sqrt(m["dim"]))
    eps = cfg["norm"]["eps"]
    na, nb = (pl.rms_unit(base["embed"][t] * cfg.get("embedding", {}).get("scale", 1.0), eps) * base["l0.norm1"] for t in (a, b))
    u = na / np.linalg.norm(na) - nb / np.linalg.norm(nb)
    u /= np.linalg.norm(u)
    q = base["l0.mix.q"].reshape(m["heads"], m["dim"], -1)[::m["heads"] // m["kv_heads"]].reshape(m["kv_heads"] * m["dim"], -1)
    over = {"l0.mix.k": q - 2.0 * np.outer(q @ u, u)}
    for i, layer in enumerate(cfg["layers"]):
        if layer["type"] == "delta":
            over[f"l{i}.mix.A_log"] = np.log(np.full_like(base[f"l{i}.mix.A_log"], 2e-3))
    return cfg, over


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("offset", ["inside", "outside"])
@pytest.mark.parametrize("how", ["prompt", "decoded"])
@pytest.mark.parametrize("dim", [16, 64])
def test_window_edges(folders, dtype, offset, how, dim):
    """The one key that the last token looks for lies on the last position the window still holds, or on the first it does
    not.  The restatement with a window one longer or shorter gives other logits at that place (checked), so a window that
    is one off shows."""
    W = 20
    cfg, over = aimed(model([(attention(heads=2, kv_heads=1, dim=dim, vdim=dim, window=W, rot_dims=4, scaling=None), None)], vocab=90), 4, 88, 89)
    folder, cfg, w = folders(f"edge{dim}", cfg, seed=4, overrides=over)
    n = 70                                                        # the key lies on and beside a page border in turn
    for end in (n - 1, n - 2, n - 6):
        toks = tokens(80, n, 100 + end)                           # ids 80.. are kept for the two tokens
        back = W - 1 if offset == "inside" else W
        toks[end - 1:end + 1] = [88, 88]
        toks[end - back - 1:end - back + 1] = [89, 89]
        want = pl.forward(cfg, w, toks)
        other = copy.deepcopy(cfg)
        other["layers"][0]["mixer"]["mask"]["size"] = W - 1 if offset == "inside" else W + 1
        moved = np.abs(pl.forward(other, w, toks)[end] - want[end]).max() / np.abs(want).max()
        assert moved > 4 * TOL[dtype], f"the test's weights do not show the edge ({moved:.3g})"
        r = runner(folder, dtype, pool_tokens=128)
        if how == "prompt":
            got = r.run([("e", toks, [end])])
        else:
            r.run([("e", toks[:end - 3], [])])
            got = np.concatenate([r.run([("e", [t], [0])]) for t in toks[end - 3:end + 1]])[-1:]
        close(got, want[end:end + 1], dtype, f"{offset} {how} end {end}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_far_keys_sinks_and_slow_states(folders, dtype):
    """Sharp attention without a window over many pages (one key far back that the last tokens look for), delta states that
    hardly decay, then decoding; and checks that the far key and the sink matter."""
    cfg, over = aimed(model([(attention(window=None, rot_dims=4), 64), (delta(), None), (attention(heads=2, kv_heads=2, dim=8, vdim=8, window=None, rot_dims=None), 32)],
                            vocab=140, loop=(0, 2, 2)), 9, 138, 139)
    folder, cfg, w = folders("pointed", cfg, seed=9, overrides=over)
    toks = tokens(130, 400, 21)
    toks[15:17] = [139, 139]                                      # the key, at a page's border
    toks[349:351] = toks[394:396] = [138, 138]                    # looked for in the prompt's tail and again while decoding
    want = pl.forward(cfg, w, toks)
    r = runner(folder, dtype, pool_tokens=448, page_size=16)
    ask = [0, 1, 15, 16, 17, 255, 256, 330, 339]
    rows = [r.run([("f", toks[:340], ask)])] + [r.run([("f", [t], [0])]) for t in toks[340:]]
    close(np.concatenate(rows), np.concatenate([want[ask], want[340:]]), dtype, "pointed weights")
    # the far key carries weight: with it replaced the logits at the places that look for it are elsewhere
    changed = list(toks)
    changed[15:17] = [1, 2]
    for place in (350, 395):
        assert np.abs(pl.forward(cfg, w, changed)[place] - want[place]).max() > 4 * TOL[dtype] * np.abs(want).max()
    # the sink matters: a softmax without the extra term gives other logits
    plain_softmax = windowless_softmax_logits(cfg, w, toks[:64])
    assert np.abs(plain_softmax - want[:64]).max() > 4 * TOL[dtype] * np.abs(want).max()


def windowless_softmax_logits(cfg, w, toks):
    """The restatement with the sink's term taken out of the denominator (its score at minus infinity)."""
    saved = pl.windowed_sink_attention

    def no_sink(h, w_, p, m, eps, positions=None):
        n = h.shape[0]
        H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        pos = np.arange(n)
        q = pl.rms_unit(pl.rotate_half((h @ w_[p + "q"].T).reshape(n, H, dk), pos, m.get("rot")), eps)
        k = pl.rms_unit(pl.rotate_half((h @ w_[p + "k"].T).reshape(n, G, dk), pos, m.get("rot")), eps)
        v = (h @ w_[p + "v"].T).reshape(n, G, dv)
        out = np.zeros((n, H, dv))
        for head in range(H):
            g = head // (H // G)
            s = np.where(np.tril(np.ones((n, n), bool)), (q[:, head] @ k[:, g].T) * m["scale"], -np.inf)
            e = np.exp(s - s.max(axis=1, keepdims=True))
            out[:, head] = (e / e.sum(axis=1, keepdims=True)) @ v[:, g]
        return out.reshape(n, H * dv) @ w_[p + "o"].T

    pl.windowed_sink_attention = no_sink
    try:
        return pl.forward(cfg, w, toks)
    finally:
        pl.windowed_sink_attention = saved


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_through_captured_steps(folders, dtype):
    folder, cfg, w = folders("odd", ODD, seed=5)
    toks = tokens(cfg["vocab"], 240, 31)
    want = pl.forward(cfg, w, toks)
    r = runner(folder, dtype, pool_tokens=512)
    rows = [r.run([("x", toks[:5], [4]), ("y", toks[:3], [])])]
    rows += [r.run([("x", [t], [0]), ("y", [u], [0])])[:1] for t, u in zip(toks[5:], toks[3:])]
    close(np.concatenate(rows), want[4:], dtype, "decoding")
    assert r.info("graph_replays") > 200


def test_first_tokens_of_a_sequence(folders):
    """Position 0 alone, then position 1: nothing before the sequence leaks in (a zero row in front of the shift, zeros before
    the convolution, an empty state, a softmax over one key and the sink), also in a slot that another request has used."""
    folder, cfg, w = folders("general", GENERAL, seed=5)
    r = runner(folder, "float32", slots=1)
    for seed in range(3):
        toks = tokens(cfg["vocab"], 2, 80 + seed)
        want = pl.forward(cfg, w, toks)
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
        logits = pl.forward(cfg, w, prompt + out)
        for i, tok in enumerate(out):
            row = logits[len(prompt) + i - 1]
            assert float(row.max() - row[tok]) <= 4 * TOL[dtype] * np.abs(row).max(), (dtype, i, tok, int(row.argmax()))


def test_trace_replay_program(folders, tmp_path):
    """bin/trace_run on a model folder of this design: steps in, logits files out."""
    folder, cfg, w = folders("odd", ODD, seed=5)
    toks = tokens(cfg["vocab"], 40, 55)
    steps = [{"step": 0, "entries": [{"id": "q", "tokens": toks[:30], "want": [0, 29]}], "end": []},
             {"step": 1, "entries": [{"id": "q", "tokens": toks[30:], "want": [9]}, {"id": "z", "tokens": toks[:2], "want": []}], "end": ["q", "z"]}]
    out = tmp_path / "out"
    run = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", "float32", "--out", str(out), "--max-tokens", "128"],
                         input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, run.stderr
    assert [l for l in run.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1"]
    want = pl.forward(cfg, w, toks)
    close(np.fromfile(out / "0.f32", dtype="<f4").reshape(2, -1), want[[0, 29]], "float32", "step 0")
    close(np.fromfile(out / "1.f32", dtype="<f4").reshape(1, -1), want[[39]], "float32", "step 1")


def test_command_line_with_random_weights(tmp_path):
    """The engine's own program on this design: random-weights mode writes a folder from a config.json (with the per-tensor
    hints that keep norms, shifts, decays and step sizes sane), then prompts of token ids are decoded greedily; the tokens must
    be the plain implementation's for the weights that were written."""
    cfg = model([(delta(heads=2, kv_heads=1, dim=16, vdim=16, conv=3), 40), (attention(heads=2, kv_heads=1, dim=16, vdim=8, window=12), None)], width=64,
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
    cfg_read, w = pl.read_model_dir(folder)
    assert np.all(w["l0.norm1"] == 1.0) and np.all(w["l1.shift"] == 0.5) and np.all(w["l0.mix.norm"] == 1.0) and w["l0.mix.A_log"].min() >= 0.0
    for prompt, out in zip([[5, 17, 3], [9, 8, 7, 6]], outs):
        logits = pl.forward(cfg_read, w, prompt + out)
        for i, tok in enumerate(out):
            row = logits[len(prompt) + i - 1]
            assert float(row.max() - row[tok]) <= 4e-4 * np.abs(row).max(), (i, tok, int(row.argmax()))
