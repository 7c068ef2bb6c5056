"""Balalorn through the engine against the plain implementation (``plain_balalorn.py``).

Small configurations of their own (sizes that differ in every field; groups, key heads,
norm parts and picked experts that are neither 1 nor equal to one another; a rotation over
fewer entries than the rotated part has; a layer without feed-forward; a layer that reads
the latent cache of a layer two before it).  Each mixer and feed-forward alone as a
one-layer model; whole prompts against token-by-token decoding and against portions down to
two tokens; unequal requests in one batch against each alone; slots and pages used again;
far keys and page borders with attention made sharp; first tokens; long decoding; greedy
generation through the entry point and its scheduler.
"""
import copy
import json
import os
import random

import numpy as np
import pytest
import torch

import helpers
import plain_balalorn as P

pytestmark = pytest.mark.gpu

LATENT = {"type": "latent_attention",
          "mixer": {"heads": 3, "dim": 16, "rot_dim": 8, "vdim": 12, "kv_rank": 20, "scale": 0.21,
                    "rot": {"base": 10000.0, "dims": 4}},
          "mlp": None}
LATENT_SHARED = {"type": "latent_attention",
                 "mixer": {"heads": 2, "dim": 8, "rot_dim": 8, "vdim": 16, "kv_rank": 20, "scale": 0.3, "kv_from": 0,
                           "rot": {"base": 10000.0, "dims": 4}},
                 "mlp": {"kind": "dense", "ff": 40}}
SSD = {"type": "mamba2", "mixer": {"heads": 6, "vdim": 8, "state": 12, "groups": 3, "norm_groups": 1, "conv": 2}, "mlp": None}
SSD_B = {"type": "mamba2", "mixer": {"heads": 4, "vdim": 20, "state": 9, "groups": 1, "norm_groups": 5, "conv": 5},
         "mlp": {"kind": "moe", "expert": {"ff": 24}, "router": {"experts": 5, "top": 2}}}
DELTA = {"type": "delta", "mixer": {"heads": 6, "kv_heads": 2, "dim": 12, "vdim": 10, "conv": 5},
         "mlp": {"kind": "moe", "expert": {"ff": 16}, "router": {"experts": 4, "top": 3}}}
DELTA_B = {"type": "delta", "mixer": {"heads": 2, "kv_heads": 2, "dim": 40, "vdim": 7, "conv": 2}, "mlp": {"kind": "dense", "ff": 48}}


def config_of(layers, width=64, vocab=200, eps=1e-5):
    return {"architecture": "Balalorn", "width": width, "vocab": vocab, "norm": {"eps": eps}, "layers": copy.deepcopy(layers)}


CONFIGS = {
    "mixed": config_of([LATENT, SSD, LATENT_SHARED, DELTA, DELTA_B]),
    "other": config_of([DELTA_B, SSD_B, LATENT, dict(LATENT_SHARED, mixer=dict(LATENT_SHARED["mixer"], kv_from=2))], width=72, vocab=150, eps=1e-6),
    # wide enough for the tensor-core products of the bfloat16 path
    "wide": config_of([
        {"type": "latent_attention", "mixer": {"heads": 4, "dim": 128, "rot_dim": 16, "vdim": 128, "kv_rank": 128, "scale": 0.08,
                                                "rot": {"base": 50000.0, "dims": 16}},
         "mlp": {"kind": "moe", "expert": {"ff": 128}, "router": {"experts": 6, "top": 2}}},
        {"type": "mamba2", "mixer": {"heads": 8, "vdim": 32, "state": 16, "groups": 2, "norm_groups": 2, "conv": 4},
         "mlp": {"kind": "dense", "ff": 256}},
        {"type": "delta", "mixer": {"heads": 4, "kv_heads": 2, "dim": 64, "vdim": 64, "conv": 3}, "mlp": {"kind": "dense", "ff": 256}},
    ], width=256, vocab=500),
}
ALONE = {"latent": [LATENT], "latent+shared": [LATENT, LATENT_SHARED], "ssd": [SSD], "ssd_b": [SSD_B], "delta": [DELTA],
         "delta_b": [DELTA_B]}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    made = {}

    def get(name, raw, seed=5, touch=None):
        if name not in made:
            d = str(tmp_path_factory.mktemp(f"balalorn_{name.replace('+', '_')}"))
            helpers.write_model(d, raw, seed=seed)
            if touch is not None:
                touch(d)
            made[name] = (d, P.read_model(d))
        return made[name]
    return get


def runner_for(model_dir, dtype, max_seqs=4, max_tokens=512, num_pages=None, cuda_graphs=True, page=16):
    import cajeta_llm_b200  # noqa: F401
    from cajeta_llm_b200.engine.model import load_model
    from cajeta_llm_b200.engine.step import ModelRunner
    from cajeta_llm_b200.parts.base import Runtime
    model, _ = load_model(model_dir, Runtime(dtype, "cuda:0"))
    return ModelRunner(model, page_tokens=page, max_seqs=max_seqs, max_tokens_per_seq=max_tokens,
                       num_pages=num_pages if num_pages is not None else -(-max_tokens // page) * max_seqs, cuda_graphs=cuda_graphs)


def oracle(W, cfg, tokens):
    """The plain implementation's logits and, by tensor-name prefix of a routed feed-forward, its picks."""
    picks = {}
    want, _ = P.forward(tokens, W, cfg, picks=picks)
    return want, {f"l{i}.mlp": v for i, v in picks.items()}


def pin_rows(picks, spans):
    """The step's routing pin: for every routed feed-forward the plain implementation's experts of the
    step's rows; spans = [(request's picks, first position, count)] in the step's order."""
    if not spans or not spans[0][0]:
        return None
    return {prefix: torch.cat([p[prefix][lo:lo + n] for p, lo, n in spans]).to(torch.int32).cuda().contiguous() for prefix in spans[0][0]}


def feed(runner, slot, tokens, cuts, picks=None):
    """The request's tokens in steps of the given sizes; logits of every position.  ``picks``: the
    experts of every position are given (the plain implementation's) instead of chosen, which
    takes the discontinuity of a near-tie out of a reduced-precision comparison."""
    from cajeta_llm_b200.engine.step import StepEntry
    out, at = [], 0
    for n in cuts:
        pin = pin_rows(picks, [(picks, at, n)]) if picks else None
        out.append(runner.step([StepEntry(slot, tokens[at:at + n], list(range(n)))], routing_pin=pin).cpu())
        at += n
    assert at == len(tokens)
    return torch.cat(out)


def rel_err(got, want):
    """Per row: RMS of the difference (mean taken off) over the RMS of the wanted logits."""
    d = got.double() - want.double()
    d = d - d.mean(dim=-1, keepdim=True)
    w = want.double() - want.double().mean(dim=-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / w.pow(2).mean(-1).sqrt().clamp_min(1e-9)


def check(got, want, dtype, what, free_routing=False):
    """float32: every row to rounding.  bfloat16 (activations and cache rounded to 8 bits of mantissa):
    every row within 6 % of the logits' spread when the routing is pinned; with the routing free a
    row near a tie may swap an expert, and the recurrent layers carry that on to later rows, so
    only the bulk of the rows is held to the bound."""
    e = rel_err(got, want)
    if dtype == "float32":
        assert float(e.max()) < 3e-5, f"{what}: worst row {int(e.argmax())} differs by {float(e.max()):.2e}"
    elif not free_routing:
        assert float(e.max()) < 6e-2, f"{what}: worst row {int(e.argmax())} differs by {float(e.max()):.3f} (median {float(e.median()):.3f})"
    else:
        assert float(e.median()) < 2e-2 and float((e > 6e-2).float().mean()) <= 0.15, \
            f"{what}: median {float(e.median()):.3f}, worst {float(e.max()):.3f}, over 0.06: {int((e > 6e-2).sum())} of {e.numel()}"


@pytest.mark.parametrize("name", sorted(ALONE))
def test_each_mechanism_alone_as_a_one_layer_model(folders, name):
    d, (cfg, W) = folders(name, config_of(ALONE[name], width=48, vocab=90), seed=3)
    toks = helpers.random_tokens(90, 41, seed=1)
    want, picks = oracle(W, cfg, toks)
    for dtype in ("float32", "bfloat16"):
        pins = picks if dtype == "bfloat16" else None
        r = runner_for(d, dtype, max_tokens=64)
        s = r.admit()
        check(feed(r, s, toks, [41], pins), want, dtype, f"{name} whole {dtype}")
        r.release(s)
        s = r.admit()                                  # the same slot again: its state starts at zero
        check(feed(r, s, toks, [5, 2, 17, 2, 3] + [1] * 12, pins), want, dtype, f"{name} portions {dtype}")


@pytest.mark.parametrize("name", sorted(CONFIGS))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_decoded_and_in_portions(folders, name, dtype):
    d, (cfg, W) = folders(name, CONFIGS[name], seed=7)
    toks = helpers.random_tokens(cfg["vocab"], 75, seed=2)
    want, picks = oracle(W, cfg, toks)
    r = runner_for(d, dtype, max_tokens=128)
    results = []
    for cuts in ([75], [43] + [1] * 32, [1] * 75 if name != "wide" else [2] * 37 + [1], [7, 2, 16, 3, 2, 9, 5, 2, 15, 14]):
        s = r.admit()
        results.append(feed(r, s, toks, cuts))                       # routing free: decode steps replay from graphs in bfloat16
        check(results[-1], want, dtype, f"{name} {dtype} cuts {cuts[:4]}", free_routing=True)
        r.release(s)
        if dtype == "bfloat16":
            s = r.admit()
            check(feed(r, s, toks, cuts, picks), want, dtype, f"{name} {dtype} cuts {cuts[:4]}, routing pinned")
            r.release(s)
    if dtype == "float32":
        # the cut changes nothing but the rounding of the products' sums
        for other in results[1:]:
            assert float(rel_err(other, results[0]).max()) < 1e-5


def test_unequal_requests_in_one_batch_slots_and_pages_used_again(folders):
    """Up to four live requests, portions of some beside single tokens of others, requests
    that sit a step out, in a pool so small that pages and slots come back into use: every
    position equals the plain implementation's, and in float32 the request run alone."""
    from cajeta_llm_b200.engine.step import StepEntry
    d, (cfg, W) = folders("mixed", CONFIGS["mixed"], seed=7)
    rng = random.Random(4)
    lens = [23, 48, 17, 64, 35, 29, 52, 2, 41, 1]
    toks = {i: helpers.random_tokens(cfg["vocab"], n, seed=50 + i) for i, n in enumerate(lens)}
    both = {i: oracle(W, cfg, t) for i, t in toks.items()}
    want = {i: b[0] for i, b in both.items()}
    for dtype in ("float32", "bfloat16"):
        r = runner_for(d, dtype, max_seqs=4, max_tokens=64, num_pages=14)
        waiting, live, got = list(toks), {}, {i: [] for i in toks}
        while waiting or live:
            while waiting and len(live) < 4:
                i = waiting[0]
                if sum(-(-(len(toks[j]) + 15) // 16) for j in live) + -(-(len(toks[i]) + 15) // 16) > 14:
                    break
                waiting.pop(0)
                live[i] = [r.admit(), 0, max(1, len(toks[i]) - rng.randint(3, 12))]
            entries, who, spans = [], [], []
            for i, st in list(live.items()):
                if len(live) > 1 and rng.random() < 0.2:
                    continue
                n = 1 if st[1] >= st[2] else min(rng.randint(2, 11), st[2] - st[1])
                entries.append(StepEntry(st[0], toks[i][st[1]:st[1] + n], list(range(n))))
                who.append((i, n))
                spans.append((both[i][1], st[1], n))
                st[1] += n
            if not entries:
                continue
            out = r.step(entries, routing_pin=pin_rows(spans[0][0], spans) if dtype == "bfloat16" else None).cpu()
            at = 0
            for i, n in who:
                got[i].append(out[at:at + n])
                at += n
                if live[i][1] == len(toks[i]):
                    r.release(live.pop(i)[0])
        for i in toks:
            check(torch.cat(got[i]), want[i], dtype, f"request {i} in the mixed batch ({dtype})")
        r.cache.books.check()


def sharpen(scale):
    def touch(model_dir):
        path = os.path.join(model_dir, "config.json")
        with open(path) as f:
            c = json.load(f)
        for layer in c["layers"]:
            if layer["type"] == "latent_attention":
                layer["mixer"]["scale"] = scale
        with open(path, "w") as f:
            json.dump(c, f)
    return touch


def test_far_keys_and_page_borders_with_sharp_attention(folders):
    """With random weights a softmax over hundreds of keys is nearly flat and a lost key hides
    in it.  Here the scores are multiplied up until a row's weight sits on a few keys anywhere
    in its past - a missing or shifted key, a page's first or last entry, then shows in that
    row's logits.  Prompt portions that end inside, on and just past page borders, then decoding."""
    raw = config_of([LATENT, LATENT_SHARED], width=48, vocab=90)
    d, (cfg, W) = folders("sharp", raw, seed=9, touch=sharpen(40.0))
    assert cfg["layers"][0]["mixer"]["scale"] == 40.0
    toks = helpers.random_tokens(90, 330, seed=8)
    want, _ = P.forward(toks, W, cfg)
    # the weights really are concentrated: the largest softmax weight of late rows is far from 1/t
    c, kr = P.latent_keys(W["embed"][torch.tensor(toks)], P.sub(W, "l0.mix"), cfg["layers"][0]["mixer"], cfg["norm"]["eps"], range(330))
    assert c.shape == (330, 20)
    r = runner_for(d, "float32", max_tokens=336)
    for cuts in ([330], [15, 1, 1, 15, 16, 17, 31, 33, 64, 63, 2, 40] + [1] * 32, [255, 2, 41] + [1] * 32):
        s = r.admit()
        e = rel_err(feed(r, s, toks, cuts), want)
        assert float(e.max()) < 1e-4, f"cuts {cuts[:5]}: row {int(e.argmax())} differs by {float(e.max()):.2e}"
        r.release(s)
    # and a deliberately wrong oracle (the far half of the keys dropped) is told apart by this test's bound
    m = cfg["layers"][0]["mixer"]
    near, _ = P.latent_attention(W["embed"][torch.tensor(toks[200:])], P.sub(W, "l0.mix"), m, cfg["norm"]["eps"], range(200, 330))
    full, _ = P.latent_attention(W["embed"][torch.tensor(toks)], P.sub(W, "l0.mix"), m, cfg["norm"]["eps"], range(330))
    assert float(rel_err(near[-30:], full[-30:]).max()) > 1e-2


def test_first_tokens_and_long_decoding(folders):
    """Single-token requests, requests shorter than a convolution's taps, and 150 tokens decoded
    one by one after a 3-token prompt (state carried 150 times, two graph buckets of decode)."""
    d, (cfg, W) = folders("other", CONFIGS["other"], seed=7)
    for dtype in ("float32", "bfloat16"):
        r = runner_for(d, dtype, max_tokens=192)
        for n in (1, 2, 3, 4, 6):
            toks = helpers.random_tokens(cfg["vocab"], n, seed=20 + n)
            s = r.admit()
            check(feed(r, s, toks, [1] * n), P.forward(toks, W, cfg)[0], dtype, f"{n} first tokens one by one ({dtype})", free_routing=True)
            r.release(s)
        toks = helpers.random_tokens(cfg["vocab"], 153, seed=33)
        s = r.admit()
        check(feed(r, s, toks, [3] + [1] * 150), P.forward(toks, W, cfg)[0], dtype, f"long decoding ({dtype})", free_routing=True)
        r.release(s)


def test_captured_steps_equal_uncaptured_ones(folders):
    """bfloat16 steps replayed from CUDA graphs (decode steps and step shapes that come again)
    give the bits of steps launched kernel by kernel, state included."""
    from cajeta_llm_b200.engine.step import StepEntry
    d, (cfg, W) = folders("wide", CONFIGS["wide"], seed=7)
    toks = [helpers.random_tokens(cfg["vocab"], 60, seed=70 + i) for i in range(3)]
    outs = []
    for graphs in (True, False):
        r = runner_for(d, "bfloat16", max_tokens=128, cuda_graphs=graphs)
        slots = [r.admit() for _ in toks]
        got = []
        for lo, hi in ((0, 12), (12, 24), (24, 36)):                # the same shape three times: captured, then replayed
            got.append(r.step([StepEntry(s, t[lo:hi], [hi - lo - 1]) for s, t in zip(slots, toks)]).cpu())
        for i in range(36, 60):
            got.append(r.step([StepEntry(s, [t[i]], [0]) for s, t in zip(slots, toks)]).cpu())
        outs.append(torch.cat(got))
        if graphs:
            assert r.graph_replays > 0
    assert torch.equal(outs[0], outs[1])


def test_greedy_generation_through_the_entry_point_and_its_scheduler(folders):
    from cajeta_llm_b200.engine.llm_engine import LlmEngine
    from cajeta_llm_b200.engine.options import EngineOptions
    from cajeta_llm_b200.sampling.params import SamplingParams
    d, (cfg, W) = folders("mixed", CONFIGS["mixed"], seed=7)
    prompts = [helpers.random_tokens(cfg["vocab"], n, seed=90 + n) for n in (5, 9, 17, 30, 3, 12)]
    want = [P.greedy(cfg, W, p, 6) for p in prompts]
    # more requests than slots, portions of at most 8 tokens under a budget of 24 a step
    eng = LlmEngine.load(EngineOptions(model=d, dtype="float32", ctx=64, max_seqs=3, chunk=8, max_batch_tokens=24))
    got = eng.generate(prompts, SamplingParams(max_new_tokens=6, stop_token_ids=()))
    assert got == want
    eng.close()
    eng = LlmEngine.load(EngineOptions(model=d, dtype="bfloat16", ctx=64, max_seqs=4))
    got = eng.generate(prompts, SamplingParams(max_new_tokens=6, stop_token_ids=()))
    same = sum(g == w for g, w in zip(got, want))
    assert same >= len(prompts) - 1, f"bfloat16 greedy tokens differ for {len(prompts) - same} prompts"
    eng.close()


def test_replay_tool_on_a_model_folder(folders, tmp_path):
    d, (cfg, W) = folders("other", CONFIGS["other"], seed=7)
    a, b = helpers.random_tokens(cfg["vocab"], 20, seed=1), helpers.random_tokens(cfg["vocab"], 9, seed=2)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:11], "want": [10]}, {"id": "b", "tokens": b[:8], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "b", "tokens": b[8:], "want": [0]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": a[11:], "want": [0, 8]}], "end": ["a"]}]
    import subprocess
    import sys
    cmd = [sys.executable, os.path.join(helpers.ROOT, "bin", "trace_run"), "--model", d, "--dtype", "float32", "--out", str(tmp_path),
           "--max-tokens", "128"]
    proc = subprocess.run(cmd, input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    wa, wb = P.forward(a, W, cfg)[0], P.forward(b, W, cfg)[0]
    got = {n: torch.from_numpy(np.fromfile(os.path.join(str(tmp_path), f"{n}.f32"), dtype="<f4").reshape(-1, cfg["vocab"])) for n in range(3)}
    check(got[0], wa[10:11], "float32", "step 0")
    check(got[1], wb[8:9], "float32", "step 1")
    check(got[2], wa[[11, 19]], "float32", "step 2")


def random_config(seed):
    """A configuration drawn at random: layer order, every size, which layers share a latent cache."""
    rng = random.Random(seed)
    width = rng.choice([40, 72, 136, 256])
    big = width >= 128

    def pick(lo, hi):
        return rng.randint(lo, hi)

    layers, owners = [], []
    for i in range(rng.randint(2, 5)):
        kind = rng.choice(["latent_attention", "mamba2", "delta"])
        if kind == "latent_attention":
            rot_dim = 2 * pick(1, 8)
            m = {"heads": pick(1, 10), "dim": rng.choice([128, 136]) if big and rng.random() < 0.4 else pick(3, 40), "rot_dim": rot_dim,
                 "vdim": rng.choice([128, 144]) if big and rng.random() < 0.4 else pick(3, 40),
                 "kv_rank": rng.choice([128, 160]) if big and rng.random() < 0.5 else pick(5, 70),
                 "scale": rng.choice([0.1, 0.3, 1.0]), "rot": {"base": rng.choice([100.0, 10000.0, 500000.0]), "dims": 2 * pick(1, rot_dim // 2)}}
            if owners and rng.random() < 0.5:
                j = rng.choice(owners)
                src = layers[j]["mixer"]
                m.update(kv_from=j, kv_rank=src["kv_rank"], rot_dim=src["rot_dim"], rot=dict(src["rot"]))
            else:
                owners.append(i)
        elif kind == "mamba2":
            g = pick(1, 3)
            heads, vdim = g * pick(1, 3), pick(3, 24)
            divisors = [d for d in range(1, heads * vdim + 1) if (heads * vdim) % d == 0 and d <= 8]
            m = {"heads": heads, "vdim": vdim, "state": pick(2, 70), "groups": g, "norm_groups": rng.choice(divisors), "conv": pick(1, 5)}
        else:
            kv = pick(1, 3)
            m = {"heads": kv * pick(1, 3), "kv_heads": kv, "dim": pick(3, 70), "vdim": pick(3, 40), "conv": pick(1, 5)}
        ff = rng.choice([None, "dense", "moe", "moe"])
        if ff == "dense":
            mlp = {"kind": "dense", "ff": rng.choice([pick(8, 60), 128, 200]) if big else pick(8, 60)}
        elif ff == "moe":
            e = pick(1, 9)
            mlp = {"kind": "moe", "expert": {"ff": rng.choice([pick(8, 60), 128, 136]) if big else pick(8, 60)},
                   "router": {"experts": e, "top": pick(1, e)}}
        else:
            mlp = None
        layers.append({"type": kind, "mixer": m, "mlp": mlp})
    return config_of(layers, width=width, vocab=rng.choice([70, 131, 300]), eps=rng.choice([1e-5, 1e-6]))


@pytest.mark.parametrize("seed", range(8))
def test_configurations_drawn_at_random(folders, seed):
    raw = random_config(1000 + seed)
    d, (cfg, W) = folders(f"random{seed}", raw, seed=100 + seed)
    toks = helpers.random_tokens(cfg["vocab"], 45, seed=seed)
    want, picks = oracle(W, cfg, toks)
    for dtype in ("float32", "bfloat16"):
        r = runner_for(d, dtype, max_tokens=64)
        for cuts in ([45], [17, 2, 9] + [1] * 17):
            s = r.admit()
            check(feed(r, s, toks, cuts, picks if dtype == "bfloat16" else None), want, dtype,
                  f"{json.dumps(raw['layers'])} {dtype} cuts {cuts[:3]}")
            r.release(s)


def test_portions_of_one_shape_replayed_from_graphs_at_growing_contexts(folders):
    """bfloat16: a 400-token prompt in portions of 16 rows (the shape is captured at its second
    appearance and replayed while the context grows far beyond what it was at capture), then
    single tokens: every position against the plain implementation."""
    d, (cfg, W) = folders("mixed", CONFIGS["mixed"], seed=7)
    toks = helpers.random_tokens(cfg["vocab"], 420, seed=12)
    want, _ = P.forward(toks, W, cfg)
    r = runner_for(d, "bfloat16", max_tokens=448)
    s = r.admit()
    got = feed(r, s, toks, [16] * 25 + [1] * 20)
    assert r.graph_replays > 20
    check(got, want, "bfloat16", "portions of 16 from graphs", free_routing=True)
    e = rel_err(got, want)
    assert float(e[300:].median()) < 2e-2, "late positions, whose keys lie beyond the capture-time context, drift"


@pytest.mark.parametrize("name", ["mixed", "other", "wide"])
def test_plain_form_of_latent_attention_for_long_portions(folders, name, monkeypatch):
    """Steps with many rows build per-head keys and values and run the flash kernel; here the
    threshold is lowered so that portions of 40 rows do, beside cached tokens of earlier
    portions, and with three unequal requests in one step."""
    from cajeta_llm_b200.engine.step import StepEntry
    from cajeta_llm_b200.parts.latent_attention import LatentAttention
    monkeypatch.setattr(LatentAttention, "EXPAND_MIN_ROWS", 8)
    d, (cfg, W) = folders(name, CONFIGS[name], seed=7)
    toks = [helpers.random_tokens(cfg["vocab"], n, seed=40 + n) for n in (150, 75, 33)]
    both = [oracle(W, cfg, t) for t in toks]
    want = [b[0] for b in both]
    r = runner_for(d, "bfloat16", max_tokens=192)
    assert r.capture_max_rows == 7
    s = r.admit()
    check(feed(r, s, toks[0], [150], both[0][1]), want[0], "bfloat16", f"{name} whole prompt, plain form")
    r.release(s)
    s = r.admit()
    check(feed(r, s, toks[0], [40, 70, 9, 31], both[0][1]), want[0], "bfloat16", f"{name} portions, plain form")
    r.release(s)
    slots = [r.admit() for _ in toks]
    cuts = [(0, 70, 0, 40, 0, 20), (70, 150, 40, 75, 20, 33)]
    got = [[], [], []]
    for c in cuts:
        entries = [StepEntry(slots[i], toks[i][c[2 * i]:c[2 * i + 1]], list(range(c[2 * i + 1] - c[2 * i]))) for i in range(3)]
        spans = [(both[i][1], c[2 * i], c[2 * i + 1] - c[2 * i]) for i in range(3)]
        out = r.step(entries, routing_pin=pin_rows(spans[0][0], spans)).cpu()
        at = 0
        for i in range(3):
            n = c[2 * i + 1] - c[2 * i]
            got[i].append(out[at:at + n])
            at += n
    for i in range(3):
        check(torch.cat(got[i]), want[i], "bfloat16", f"{name} request {i} of three in one step, plain form")


def test_state_sizes_agree_between_the_host_and_the_kernel_library():
    import ctypes
    from cajeta_llm_b200.csrc import kernels as K
    fn = K.library("recurrent").cj_state_scan_floats
    fn.restype = ctypes.c_longlong
    for heads, rows, cols in [(1, 1, 1), (4, 5, 6), (6, 48, 48), (3, 12, 70), (16, 128, 128), (64, 128, 64), (2, 300, 33), (1, 2048, 8),
                              (128, 128, 64), (8, 128, 128), (32, 64, 64), (512, 16, 64), (40, 2048, 256)]:
        assert fn(heads, rows, cols) == K.state_scan_floats(heads, rows, cols) >= heads * rows * cols
