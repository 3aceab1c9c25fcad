"""The Dezolorn parts on the GPU against the plain statement in plain_dezolorn.py: every mixer alone, whole prompts against
token-by-token decoding, portions down to two tokens, unequal batches, pages and state slots that are used again, keys
just inside and just outside the window and the kept first keys, long decoding, odd sizes, and greedy generation through
the engine.  Each test makes its own small configuration and its own random weights."""

from __future__ import annotations

import json
import math

import pytest
import torch

import plain_dezolorn as plain

pytestmark = pytest.mark.gpu

# ---- configurations ---------------------------------------------------------------------------------------------------


def attention_layer(heads=4, kv_heads=2, dim=16, vdim=16, size=6, keep=2, dims=None, scaling=True, scale=None, ff=None):
    rot = {"dims": dim if dims is None else dims, "base": 10000.0}
    if scaling:
        rot["scaling"] = {"factor": 4.0, "original": 16, "fast": 8.0, "slow": 1.0}
    return {"type": "attention", "mlp": None if ff is None else {"kind": "dense", "ff": ff},
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale or dim ** -0.5,
                      "mask": {"size": size, "keep_first": keep}, "rot": rot}}


def retention_layer(heads=3, dim=16, vdim=8, dims=None, decay=None, ff=None):
    return {"type": "retention", "mlp": None if ff is None else {"kind": "dense", "ff": ff},
            "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay or [1 - 2.0 ** -(3 + h) for h in range(heads)],
                      "rot": {"dims": dim if dims is None else dims, "base": 5000.0}}}


def delta_layer(heads=4, kv_heads=2, dim=8, vdim=12, conv=3, ff=None):
    return {"type": "delta", "mlp": None if ff is None else {"kind": "dense", "ff": ff},
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}}


def config(layers, width=48, vocab=97, loop=None, logit_scale=0.5, softcap=8.0, eps=1e-5):
    return {"architecture": "Dezolorn", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers,
            "loop": loop or {"start": 0, "stop": 0, "times": 1}, "logit_scale": logit_scale, "logit_softcap": softcap}


def mixed_config(**kw):
    """All three mixers, a span of two layers that runs three times, sizes that differ from one another everywhere."""
    layers = [delta_layer(ff=40), attention_layer(heads=6, kv_heads=3, dim=8, vdim=12, size=7, keep=3, dims=4, ff=56),
              retention_layer(dims=8), attention_layer(heads=2, kv_heads=2, dim=24, vdim=8, size=9, keep=0, scaling=False)]
    return config(layers, loop={"start": 1, "stop": 3, "times": 3}, **kw)


def random_weights(cfg: dict, seed: int, qk_gain: float = 1.0) -> dict[str, torch.Tensor]:
    """Names and shapes from the framework's own list, values from here: bfloat16-representable, so that the float32
    and the bfloat16 engine and the float64 oracle read the same numbers."""
    from nanospec_b200.weights import build_model

    model, _ = build_model(cfg, None, torch.float32, "cpu")
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, spec in sorted(model.weight_specs().items()):
        t = torch.randn(spec.shape, generator=g)
        leaf = name.split(".")[-1]
        if len(spec.shape) == 2 and leaf != "conv":
            t = t * (1.5 / math.sqrt(spec.shape[1]))
            if leaf in ("q", "k") and ".mix." in name:
                t = t * qk_gain
        elif leaf in ("norm", "norm1", "norm2"):
            t = 1.0 + 0.2 * t
        else:
            t = 0.5 * t
        out[name] = t.to(torch.bfloat16).float()
    return out


def write_folder(folder, cfg, weights):
    from nanospec_b200.weights import write_safetensors

    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    write_safetensors(folder / "model.safetensors", {k: v.to(torch.bfloat16) for k, v in weights.items()})
    return folder


def make(tmp_path, cfg, seed=0, dtype=torch.float32, blocks=64, page=4, slots=4, qk_gain=1.0):
    from nanospec_b200 import load_model
    from nanospec_b200.engine.step import ModelRunner

    w = random_weights(cfg, seed, qk_gain)
    model = load_model(write_folder(tmp_path / f"m{seed}", cfg, w), device="cuda", dtype=dtype)
    return ModelRunner(model, num_blocks=blocks, block_size=page, max_requests=slots), w


def tokens(n, vocab, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def run_cut(runner, req_id, ids, cuts):
    """One request alone, its tokens in portions of the given sizes (the rest one by one); logits of every position."""
    from nanospec_b200.engine.step import StepEntry

    runner.begin(req_id)
    rows, at = [], 0
    sizes = list(cuts)
    while at < len(ids):
        n = min(sizes.pop(0) if sizes else 1, len(ids) - at)
        rows.append(runner.step([StepEntry(req_id, ids[at: at + n], list(range(n)))]).float().cpu())
        at += n
    runner.end(req_id)
    runner.manager.check()
    return torch.cat(rows)


def close(got, want, dtype, what=""):
    """float32: a few float32 roundings, relative to the size of the logits, at every position.  bfloat16: the roundings of a
    bfloat16 pipeline, which grow with the depth of the model and stand out where a read-out nearly cancels before its norm:
    the error of a position (root mean square over the vocabulary, the mean taken off) is set against the spread of the
    logits - small at the median position, moderate at nine in ten, never of the logits' own size, which is what a lost
    state, a wrong window or a wrong slot gives."""
    want = want.float()
    if dtype == torch.float32:
        err = (got - want).abs().amax(-1)
        lim = 1e-4 * max(5.0, float(want.abs().max()))
        assert err.max() <= lim, f"{what}: largest difference {float(err.max())} at position {int(err.argmax())} (limit {lim})"
        return
    d = got - want
    ratio = (d - d.mean(-1, keepdim=True)).pow(2).mean(-1).sqrt() / want.std()
    q = ratio.sort().values
    median, most, worst = float(q[len(q) // 2]), float(q[int(0.9 * (len(q) - 1))]), float(q[-1])
    assert (median <= 0.05 or len(q) < 8) and most <= 0.2 and worst <= 0.5, \
        f"{what}: error over spread {median:.3f} at the median position, {most:.3f} at nine in ten, {worst:.3f} at the worst (limits 0.05, 0.2, 0.5)"


# ---- every mixer alone, and their parts -------------------------------------------------------------------------------

SINGLE = {
    "attention": lambda: config([attention_layer()]),
    "attention, other widths for values, part of the head rotated": lambda: config([attention_layer(dim=24, vdim=8, dims=12, size=5, keep=1)]),
    "attention, no kept keys, no scaling": lambda: config([attention_layer(keep=0, scaling=False)]),
    "attention, one head": lambda: config([attention_layer(heads=1, kv_heads=1, dim=6, vdim=10, dims=2, size=1, keep=1)]),
    "retention": lambda: config([retention_layer()]),
    "retention, part rotated, one head": lambda: config([retention_layer(heads=1, dim=20, vdim=40, dims=6, decay=[0.5])]),
    "retention, wide head": lambda: config([retention_layer(heads=2, dim=136, vdim=33, dims=136)]),
    "delta": lambda: config([delta_layer()]),
    "delta, one tap, equal heads": lambda: config([delta_layer(heads=2, kv_heads=2, dim=5, vdim=7, conv=1)]),
    "delta, five taps, wide head": lambda: config([delta_layer(heads=3, kv_heads=1, dim=72, vdim=36, conv=5)]),
    "feed-forward and no soft cap": lambda: config([delta_layer(ff=30)], logit_scale=1.0, softcap=0.0),
    "a width and a feed-forward that are no multiples of 8": lambda: config(
        [attention_layer(ff=30), retention_layer(ff=77), delta_layer()], width=50, vocab=101),
}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", list(SINGLE))
def test_each_mixer_alone(name, dtype, tmp_path):
    cfg = SINGLE[name]()
    runner, w = make(tmp_path, cfg, seed=3, dtype=dtype)
    ids = tokens(29, cfg["vocab"], 5)
    want = plain.forward(cfg, w, ids)
    close(run_cut(runner, 0, ids, [len(ids)]), want, dtype, name + " whole")
    close(run_cut(runner, 1, ids, []), want, dtype, name + " token by token")
    close(run_cut(runner, 2, ids, [2, 3, 2, 7, 2, 5]), want, dtype, name + " portions")


def test_layernorm_and_rotation_kernels():
    from nanospec_b200 import ops
    from nanospec_b200.parts.position import rotary_frequencies

    g = torch.Generator().manual_seed(1)
    x = torch.randn(5, 100, generator=g) * 3 + 2
    gain = torch.randn(100, generator=g)
    resid = x.cuda().clone()
    out = torch.empty(5, 100, device="cuda")
    ops.add_layernorm(resid, None, gain.cuda(), 1e-3, out)
    assert (out.cpu() - plain.layer_norm(x.double(), gain.double(), 1e-3).float()).abs().max() < 1e-5
    for width in (1024, 2048 + 8, 4096):  # the widths that take the kernel with the row in registers, with a branch to add
        x, br, gain = torch.randn(7, width, generator=g) * 2 - 1, torch.randn(7, width, generator=g).bfloat16(), torch.randn(width, generator=g)
        resid, out = x.cuda().clone(), torch.empty(7, width, device="cuda", dtype=torch.bfloat16)
        ops.add_layernorm(resid, br.cuda(), gain.cuda(), 1e-6, out)
        want = plain.layer_norm(x.double() + br.double(), gain.double(), 1e-6)
        assert (resid.cpu().double() - (x.double() + br.double())).abs().max() < 1e-6
        assert (out.cpu().double() - want).abs().max() < 0.02 * want.abs().max()
        rows = torch.tensor([5, 0, 3], dtype=torch.int32, device="cuda")
        picked = torch.empty(3, width, device="cuda")
        ops.add_layernorm(resid, None, gain.cuda(), 1e-6, picked, rows=rows)
        assert (picked.cpu().double() - want[[5, 0, 3]]).abs().max() < 1e-4
    for rot in ({"dims": 12, "base": 100.0}, {"dims": 16, "base": 50000.0, "scaling": {"factor": 8.0, "original": 64, "fast": 16.0, "slow": 2.0}}):
        f, mag = rotary_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
        f_want, mag_want = plain.rotary_frequencies(rot)
        assert (f.double() - f_want).abs().max() < 1e-7 and abs(mag - mag_want) < 1e-12


# ---- the window's edge and the kept first keys, in prompts and in decoding ----------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_window_edges_and_kept_keys(dtype, tmp_path):
    """Sharp scores (q and k weights scaled up) make single keys carry the result: a window one key too wide or too
    narrow, or a lost kept key, moves the logits far beyond rounding.  Pages of 4, a window of 6 and 3 kept keys put
    the edges inside pages and on their borders; the oracle is checked to be sensitive first."""
    cfg = config([attention_layer(size=6, keep=3, ff=32), attention_layer(size=9, keep=5, dim=8, vdim=24)], softcap=0.0, logit_scale=1.0)
    runner, w = make(tmp_path, cfg, seed=11, dtype=dtype, qk_gain=4.0)
    ids = tokens(41, cfg["vocab"], 12)
    want = plain.forward(cfg, w, ids)
    for size, keep in ((7, 3), (5, 3), (6, 2), (6, 4)):
        other = json.loads(json.dumps(cfg))
        other["layers"][0]["mixer"]["mask"] = {"size": size, "keep_first": keep}
        moved = (plain.forward(other, w, ids) - want).abs().amax(-1)
        assert (moved[12:] > 0.05).float().mean() > 0.5, "the oracle does not feel the window"
    lim = 2e-4 if dtype == torch.float32 else 0.3
    for cuts in ([41], [], [3, 4, 5, 6, 7], [13, 2, 2, 2]):
        got = run_cut(runner, 0, ids, cuts)
        assert (got - want.float()).abs().max() <= lim, f"cuts {cuts}"


@pytest.mark.parametrize("dim,size,keep,heads,kv_heads,page", [(64, 80, 5, 8, 2, 16), (128, 200, 70, 4, 4, 8), (32, 64, 64, 6, 1, 16),
                                                               (64, 130, 1, 2, 1, 32)])
def test_tensor_core_attention_with_a_window_and_kept_keys(dim, size, keep, heads, kv_heads, page, tmp_path):
    """Head sizes that the bfloat16 tensor-core kernels take, prompts that cross their tiles of 64 keys and 128 queries,
    kept keys that fill more than a tile.  Portions run the prefill kernel, single tokens the decode kernel.  Each mask that
    is off by one (the window or the kept keys, either way) moves the oracle at some positions by twice the tolerance."""
    cfg = config([attention_layer(heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim, size=size, keep=keep, dims=dim // 2)], width=64,
                 softcap=0.0, logit_scale=1.0)
    runner, w = make(tmp_path, cfg, seed=13, dtype=torch.bfloat16, blocks=64, page=page)
    ids = tokens(470, cfg["vocab"], 14)
    want = plain.forward(cfg, w, ids)
    for d_size, d_keep in ((-1, 0), (1, 0), (0, -1), (0, 1)):
        other = json.loads(json.dumps(cfg))
        other["layers"][0]["mixer"]["mask"] = {"size": size + d_size, "keep_first": keep + d_keep}
        assert (plain.forward(other, w, ids) - want).abs().max() > 0.3, "the oracle does not feel the mask"
    for cuts in ([470], [300, 2, 129, 30], [260] + [1] * 150 + [50]):
        got = run_cut(runner, 0, ids, cuts)
        err = (got - want.float()).abs().amax(-1)
        assert err.max() <= 0.15, f"cuts {cuts[:4]}: position {int(err.argmax())} differs by {float(err.max())}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_far_tokens_reach_through_the_state(dtype, tmp_path):
    """A slow decay keeps the first tokens in the state for hundreds of steps: changing token 0 must move the last
    logits, in the oracle and in the engine alike, through portions and through decoding."""
    cfg = config([retention_layer(heads=2, dim=8, vdim=8, decay=[1.0 - 2.0 ** -12, 0.999]), delta_layer(heads=2, kv_heads=1)])
    runner, w = make(tmp_path, cfg, seed=21, dtype=dtype, blocks=256)
    ids = tokens(300, cfg["vocab"], 22)
    other = [(ids[0] + 1) % cfg["vocab"]] + ids[1:]
    want, want_other = plain.forward(cfg, w, ids), plain.forward(cfg, w, other)
    assert (want[-1] - want_other[-1]).abs().max() > 0.01
    for seq, ref in ((ids, want), (other, want_other)):
        close(run_cut(runner, 0, seq, [100, 64, 2, 70]), ref, dtype, "far tokens")


# ---- batches, reuse of pages and slots, long decoding -----------------------------------------------------------------

def drawn_config(seed: int) -> dict:
    """A configuration drawn from a seed: layer kinds in any order, every size from a short list, a span that runs one to
    three times anywhere in the stack."""
    import random

    r = random.Random(seed)
    pick = r.choice
    layers = []
    for _ in range(r.randint(3, 6)):
        kind = pick(["attention", "retention", "delta"])
        ff = pick([None, 24, 64, 100])
        if kind == "attention":
            kv = pick([1, 2, 3])
            dim = pick([8, 16, 32, 40, 64])
            layers.append(attention_layer(heads=kv * pick([1, 2, 4]), kv_heads=kv, dim=dim, vdim=pick([dim, dim, 8, 24]), size=pick([1, 3, 16, 33, 500]),
                                          keep=pick([0, 1, 4, 9, 40]), dims=pick([dim, dim // 2 // 2 * 2, 2]), scaling=pick([True, False]), ff=ff))
        elif kind == "retention":
            h = pick([1, 2, 5])
            dim = pick([4, 12, 32, 64, 68])
            layers.append(retention_layer(heads=h, dim=dim, vdim=pick([4, 10, 32, 48]), dims=pick([dim, 4, 0]),
                                          decay=[1 - 2.0 ** -r.randint(1, 9) for _ in range(h)], ff=ff))
        else:
            kv = pick([1, 2])
            layers.append(delta_layer(heads=kv * pick([1, 2, 3]), kv_heads=kv, dim=pick([4, 16, 20, 64]), vdim=pick([4, 16, 40]),
                                      conv=pick([1, 2, 4, 6]), ff=ff))
    start = r.randint(0, len(layers) - 1)
    stop = r.randint(start, len(layers))
    return config(layers, width=pick([40, 64, 72, 136]), vocab=pick([64, 97, 300]), loop={"start": start, "stop": stop, "times": r.randint(1, 3)},
                  logit_scale=pick([1.0, 0.5, 2.0]), softcap=pick([0.0, 5.0, 20.0]), eps=pick([1e-5, 1e-6]))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("which", ["mixed", 1, 2, 3, 4, 5, 6])
def test_unequal_batches_and_reuse(which, dtype, tmp_path):
    """Four requests of unequal length share steps - portions beside single tokens - on a pool that only their peak
    fits; requests end and others take their pages and state slots.  Every position against the oracle, which is each
    request alone.  Once on the configuration with all three mixers, then on configurations drawn from seeds."""
    from nanospec_b200.engine.step import StepEntry

    cfg = mixed_config() if which == "mixed" else drawn_config(which)
    runner, w = make(tmp_path, cfg, seed=31, dtype=dtype, blocks=30, page=4, slots=3)
    seqs = {i: tokens(n, cfg["vocab"], 40 + i) for i, n in enumerate([37, 2, 19, 50, 1, 23])}
    want = {i: plain.forward(cfg, w, s) for i, s in seqs.items()}
    got = {i: [] for i in seqs}
    at = {i: 0 for i in seqs}
    waiting, live = list(seqs), []
    portion = {0: [5, 2, 9], 1: [2], 2: [19], 3: [2, 2, 30], 4: [1], 5: [7, 7]}
    step = 0
    while waiting or live:
        while waiting and len(live) < 3:
            i = waiting.pop(0)
            runner.begin(i)
            live.append(i)
        entries = []
        for i in live:
            n = min(portion[i].pop(0) if portion[i] else 1, len(seqs[i]) - at[i])
            entries.append((i, StepEntry(i, seqs[i][at[i]: at[i] + n], list(range(n)))))
            at[i] += n
        if step % 3 == 2 and len(entries) > 1:  # a request may sit a step out
            i, e = entries.pop()
            at[i] -= len(e.tokens)
            portion[i].insert(0, len(e.tokens))
        logits = runner.step([e for _, e in entries]).float().cpu()
        row = 0
        for i, e in entries:
            got[i].append(logits[row: row + len(e.tokens)])
            row += len(e.tokens)
        for i in [i for i in live if at[i] == len(seqs[i])]:
            runner.end(i)
            live.remove(i)
        runner.manager.check()
        step += 1
    for i in seqs:
        close(torch.cat(got[i]), want[i], dtype, f"request {i}")


def test_long_decoding_and_a_span_that_runs_once(tmp_path):
    cfg = mixed_config()
    cfg["loop"] = {"start": 0, "stop": 4, "times": 1}
    runner, w = make(tmp_path, cfg, seed=51, blocks=80)
    ids = tokens(260, cfg["vocab"], 52)
    close(run_cut(runner, 0, ids, [9]), plain.forward(cfg, w, ids), torch.float32, "long decoding")


def test_pages_behind_the_window_go_back_and_kept_ones_stay(tmp_path):
    """A prompt far longer than the pool could hold whole: the window's pages are given back as it moves, the kept
    first keys' pages are not."""
    cfg = config([attention_layer(size=6, keep=3)])
    runner, w = make(tmp_path, cfg, seed=61, blocks=8, page=4)
    ids = tokens(90, cfg["vocab"], 62)
    close(run_cut(runner, 0, ids, [8, 8, 8, 8, 2, 3]), plain.forward(cfg, w, ids), torch.float32, "small pool")


# ---- through the engine: scheduler, graphs, sampling ----------------------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("graphs", [False, True])
def test_greedy_generation_through_the_engine(dtype, graphs, tmp_path):
    from nanospec_b200 import Engine, EngineConfig, SamplingParams, load_model

    cfg = mixed_config(softcap=0.0, logit_scale=1.0)
    w = random_weights(cfg, 71)
    model = load_model(write_folder(tmp_path / "gen", cfg, w), device="cuda", dtype=dtype)
    eng = Engine(model, EngineConfig(num_blocks=64, block_size=4, max_running=3, prefill_chunk=11, cuda_graphs=graphs,
                                     graph_buckets=(1, 2, 4)))
    prompts = [tokens(n, cfg["vocab"], 80 + n) for n in (3, 30, 1, 17, 12)]
    outs = eng.generate(prompts, SamplingParams(max_tokens=12, ignore_eos=True))
    for p, out in zip(prompts, outs):
        assert len(out) == 12
        z = plain.forward(cfg, w, p + out)
        for j, tok in enumerate(out):
            row = z[len(p) + j - 1]
            gap = float(row.max() - row[tok])
            assert gap <= (1e-3 if dtype == torch.float32 else 0.3), f"token {j}: the oracle prefers another by {gap}"


def test_command_line_and_sampling(tmp_path):
    """The package's command line on a Dezolorn folder: random weights from a config.json, then generation with
    temperature, top-k and top-p under fixed seeds (twice the same), and greedy generation."""
    import subprocess
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parent.parent
    cfg_path = tmp_path / "cfg.json"
    cfg_path.write_text(json.dumps(mixed_config()))
    run = lambda *a: subprocess.run([sys.executable, "-m", "nanospec_b200", *a], cwd=root, capture_output=True, text=True, timeout=600)
    r = run("random-weights", "--config", str(cfg_path), "--out", str(tmp_path / "model"), "--seed", "4")
    assert r.returncode == 0, r.stderr
    outs = []
    for _ in range(2):
        r = run("generate", "--model", str(tmp_path / "model"), "--prompt-lens", "5", "21", "--max-tokens", "9", "--temperature", "0.8",
                "--top-k", "20", "--top-p", "0.9", "--seed", "3", "--ignore-eos")
        assert r.returncode == 0, r.stderr
        outs.append([json.loads(line)["output_ids"] for line in r.stdout.splitlines() if '"output_ids"' in line])
    assert outs[0] == outs[1] and [len(o) for o in outs[0]] == [9, 9]
    r = run("generate", "--model", str(tmp_path / "model"), "--dtype", "float32", "--prompt-ids", "1 2 3 4", "--max-tokens", "6", "--ignore-eos")
    assert r.returncode == 0, r.stderr
    assert len(json.loads(r.stdout.splitlines()[0])["output_ids"]) == 6
