"""Saropel through the engine against the plain implementation (``plain_saropel.py``).

Small configurations of their own: sizes that differ in every field, head groups and picked
experts that are neither 1 nor equal to one another, value sizes other than key sizes, windows
that are no multiple of a page, a rotation over fewer entries than a head has with and without
stretched frequencies, layers without a feed-forward, without a window, without a cap; loops of
one and of three passes, over the first, the last and all layers; no loop, no pair table, no
side input.  Each mechanism alone as a one-layer model; whole prompts against token-by-token
decoding and against portions down to two tokens; unequal requests in one batch against each
alone; slots and pages used again; keys just inside and just outside a window, at page borders,
in prompts and in decoding, with attention made sharp; first tokens; long decoding; greedy
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
import plain_saropel as P

pytestmark = pytest.mark.gpu

CAPPED = {"type": "attention",
          "mixer": {"heads": 6, "kv_heads": 2, "dim": 12, "vdim": 20, "scale": 0.4, "softcap": 3.0, "mask": {"size": 21}},
          "mlp": None}
CAPPED_B = {"type": "attention",
            "mixer": {"heads": 2, "kv_heads": 1, "dim": 40, "vdim": 8, "scale": 0.2, "softcap": 30.0, "mask": {"size": 5}},
            "mlp": {"kind": "dense", "ff": 44}}
ROTATED = {"type": "attention_2",
           "mixer": {"heads": 4, "kv_heads": 2, "dim": 24, "vdim": 24, "scale": 0.3, "mask": {"size": 37},
                     "rot": {"base": 900.0, "dims": 10, "scaling": {"factor": 4.0, "original": 16, "fast": 8.0, "slow": 0.5}}},
           "mlp": None}
ROTATED_B = {"type": "attention_2",
             "mixer": {"heads": 3, "kv_heads": 3, "dim": 16, "vdim": 16, "scale": 0.25, "mask": {"size": 16},
                       "rot": {"base": 10000.0, "dims": 16}},
             "mlp": {"kind": "moe", "expert": {"ff": 20, "limit": 0.05}, "router": {"experts": 6, "top": 3, "groups": {"count": 3, "keep": 2}},
                     "shared": {"ff": 28, "limit": 0.02}}}
ROUTED = {"type": "attention",
          "mixer": {"heads": 2, "kv_heads": 2, "dim": 8, "vdim": 8, "scale": 0.35, "softcap": 8.0, "mask": {"size": 64}},
          "mlp": {"kind": "moe", "expert": {"ff": 24, "limit": 0.03}, "router": {"experts": 9, "top": 3}}}
GROUPED = {"type": "attention_2",
           "mixer": {"heads": 2, "kv_heads": 1, "dim": 8, "vdim": 8, "scale": 0.35, "mask": {"size": 9}},
           "mlp": {"kind": "moe", "expert": {"ff": 16, "limit": 1.5}, "router": {"experts": 12, "top": 3, "groups": {"count": 4, "keep": 1}},
                   "shared": {"ff": 16, "limit": 1.5}}}


def config_of(layers, width=64, vocab=200, eps=1e-5, loop=None, bigram=(53, 3, 11), side=6):
    c = {"architecture": "Saropel", "width": width, "vocab": vocab, "norm": {"eps": eps}, "layers": copy.deepcopy(layers)}
    if loop:
        c["loop"] = dict(zip(("start", "stop", "times"), loop))
    if bigram:
        c["embedding"] = {"bigram": dict(zip(("buckets", "mul_prev", "mul_cur"), bigram))}
    if side:
        c["token_side"] = {"dim": side}
    return c


WIDE = [
    {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 64, "vdim": 64, "scale": 0.125, "softcap": 20.0, "mask": {"size": 48}},
     "mlp": {"kind": "moe", "expert": {"ff": 128, "limit": 0.08}, "router": {"experts": 8, "top": 2, "groups": {"count": 2, "keep": 1}},
             "shared": {"ff": 256, "limit": 0.08}}},
    {"type": "attention_2", "mixer": {"heads": 4, "kv_heads": 1, "dim": 128, "vdim": 128, "scale": 0.09, "mask": {"size": 70},
                                      "rot": {"base": 50000.0, "dims": 64, "scaling": {"factor": 2.0, "original": 64, "fast": 16.0, "slow": 1.0}}},
     "mlp": {"kind": "dense", "ff": 256}},
    {"type": "attention", "mixer": {"heads": 2, "kv_heads": 2, "dim": 96, "vdim": 96, "scale": 0.1, "softcap": 50.0, "mask": {"size": 33}},
     "mlp": {"kind": "moe", "expert": {"ff": 128, "limit": 0.05}, "router": {"experts": 4, "top": 2}, "shared": {"ff": 128, "limit": 0.1}}},
    {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 128, "vdim": 128, "scale": 0.09, "softcap": 6.0, "mask": {"size": 40}},
     "mlp": None},
    {"type": "attention_2", "mixer": {"heads": 2, "kv_heads": 1, "dim": 32, "vdim": 32, "scale": 0.2, "rot": {"base": 100.0, "dims": 32}},
     "mlp": None},
]
CONFIGS = {
    "mixed": config_of([CAPPED, ROTATED_B, CAPPED_B, ROTATED, ROUTED], loop=(1, 4, 2)),
    "other": config_of([ROTATED, GROUPED, CAPPED_B], width=72, vocab=150, eps=1e-6, loop=(0, 2, 3), bigram=(17, 5, 1), side=3),
    "bare": config_of([GROUPED, CAPPED], width=40, vocab=90, loop=None, bigram=None, side=0),
    # wide enough for the tensor-core products and the tensor-core attention of the bfloat16 path
    "wide": config_of(WIDE, width=256, vocab=500, loop=(1, 3, 2), bigram=(257, 29, 5), side=16),
}
ALONE = {"capped": [CAPPED], "capped_b": [CAPPED_B], "rotated": [ROTATED], "rotated_b": [ROTATED_B], "routed": [ROUTED],
         "grouped": [GROUPED]}


def louder(model_dir):
    """The random-weights mode draws small values (standard deviation 0.02): with them every softmax is
    flat, no cap and no limit is ever reached and the router is near a tie everywhere.  The projections
    that feed scores, routers and gates are multiplied up so that the mechanisms bite."""
    from cajeta_llm_b200.weights.safetensors_io import Checkpoint, write_safetensors
    ck = Checkpoint(model_dir)
    tensors = {n: ck.load(n).float() for n in ck.names()}
    ck.close()
    for n, t in tensors.items():
        leaf = n.split(".")[-1]
        if n.endswith(".mix.q") or n.endswith(".mix.k"):
            t *= 6.0
        elif leaf in ("router", "sg", "g"):
            t *= 15.0
        elif leaf in ("gate", "up", "down", "proj", "v", "o") or n in ("bigram", "side.embed", "loop.step"):
            t *= 4.0
        elif leaf == "norm" and ".mix." in n:
            t += 0.3 * torch.randn(t.shape, generator=torch.Generator().manual_seed(len(n)))
    write_safetensors(os.path.join(model_dir, "model.safetensors"), {n: t.to(torch.bfloat16) for n, t in tensors.items()})


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    made = {}

    def get(name, raw, seed=5, touch=louder):
        if name not in made:
            d = str(tmp_path_factory.mktemp(f"saropel_{name}"))
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


def oracle(cfg, W, tokens):
    """The plain implementation's logits and its picks by the engine's routing keys: '<prefix>' for a routed
    layer's first run in a step, '<prefix>#1', ... for the runs of later passes."""
    runs = []
    want = torch.from_numpy(P.forward(cfg, W, tokens, picks=runs))
    picks, seen = {}, {}
    for i, picked in runs:
        if picked is None:
            continue
        n = seen.get(i, 0)
        seen[i] = n + 1
        picks[f"l{i}.mlp" + (f"#{n}" if n else "")] = torch.tensor(picked, dtype=torch.int32)
    return want, picks


def pin_rows(spans):
    """A step's routing pin from [(request's picks, first position, count)] in the step's order."""
    if not spans or not spans[0][0]:
        return None
    return {key: torch.cat([p[key][lo:lo + n] for p, lo, n in spans]).cuda().contiguous() for key in spans[0][0]}


def feed(runner, slot, tokens, cuts, picks=None):
    from cajeta_llm_b200.engine.step import StepEntry
    out, at = [], 0
    for n in cuts:
        pin = pin_rows([(picks, at, n)]) if picks else None
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
    """float32: every row to rounding.  bfloat16 with the routing pinned: the median row within 2 % of the logits'
    spread, at most 3 % of the rows beyond 6 %, none beyond 20 % - these weights are loud (sharp softmaxes, gates
    and limits at work), and a row now and then carries a rounding of the stored activations several times the
    usual size; such rows come out the same on the float32-arithmetic kernels with bfloat16 storage, so they are
    the storage's, and a fault of a kernel (an edge, a lost key: see the edge tests, which hold every row to 6 %)
    is far larger.  With the routing free a row near a tie may also swap an expert: only the bulk is held."""
    e = rel_err(got, want)
    if dtype == "float32":
        assert float(e.max()) < 5e-5, f"{what}: worst row {int(e.argmax())} differs by {float(e.max()):.2e}"
        return
    over = int((e > 6e-2).sum())
    allowed = max(1, int((0.15 if free_routing else 0.03) * e.numel()))
    assert float(e.median()) < 2e-2 and over <= allowed and (free_routing or float(e.max()) < 0.2), \
        f"{what}: median {float(e.median()):.3f}, worst {float(e.max()):.3f} (row {int(e.argmax())}), over 0.06: {over} of {e.numel()}"


@pytest.mark.parametrize("name", sorted(ALONE))
def test_each_mechanism_alone_as_a_one_layer_model(folders, name):
    # without the pair table, the side input and the loop, then with all three around the same layer
    for extra, raw in (("", config_of(ALONE[name], width=48, vocab=90, bigram=None, side=0)),
                       ("+ends", config_of(ALONE[name], width=48, vocab=90, loop=(0, 1, 2)))):
        d, (cfg, W) = folders(name + extra, raw, seed=3)
        toks = helpers.random_tokens(90, 83, seed=1)
        want, picks = oracle(cfg, W, toks)
        for dtype in ("float32", "bfloat16"):
            pins = picks if dtype == "bfloat16" else None
            r = runner_for(d, dtype, max_tokens=96)
            s = r.admit()
            check(feed(r, s, toks, [83], pins), want, dtype, f"{name}{extra} whole {dtype}")
            r.release(s)
            s = r.admit()                                  # the same slot and pages again
            check(feed(r, s, toks, [5, 2, 17, 2, 3, 30] + [1] * 24, pins), want, dtype, f"{name}{extra} portions {dtype}")


def test_the_mechanisms_bite(folders):
    """The tests' weights reach the cap, the limits and the windows: an oracle without one of them differs."""
    d, (cfg, W) = folders("mixed", CONFIGS["mixed"], seed=7)
    toks = helpers.random_tokens(cfg["vocab"], 90, seed=2)
    want = torch.from_numpy(P.forward(cfg, W, toks))

    def without(change):
        c = copy.deepcopy(cfg)
        change(c)
        return float(rel_err(torch.from_numpy(P.forward(c, W, toks)), want)[40:].max())

    assert without(lambda c: c["layers"][0]["mixer"].pop("softcap")) > 1e-3
    assert without(lambda c: c["layers"][0]["mixer"]["mask"].update(size=22)) > 1e-3
    assert without(lambda c: c["layers"][3]["mixer"]["mask"].update(size=36)) > 1e-3
    assert without(lambda c: c["layers"][1]["mlp"]["expert"].update(limit=50.0)) > 1e-3
    assert without(lambda c: c["layers"][1]["mlp"]["shared"].update(limit=50.0)) > 1e-3
    assert without(lambda c: c["layers"][1]["mlp"]["router"].pop("groups")) > 1e-3
    assert without(lambda c: c["layers"][3]["mixer"]["rot"].pop("scaling")) > 1e-3
    assert without(lambda c: c["loop"].update(times=1)) > 1e-3
    assert without(lambda c: c["embedding"]["bigram"].update(mul_prev=4)) > 1e-3
    assert without(lambda c: c.pop("token_side")) > 1e-3


@pytest.mark.parametrize("name", sorted(CONFIGS))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_decoded_and_in_portions(folders, name, dtype):
    d, (cfg, W) = folders(name, CONFIGS[name], seed=7)
    toks = helpers.random_tokens(cfg["vocab"], 150, seed=2)
    want, picks = oracle(cfg, W, toks)
    r = runner_for(d, dtype, max_tokens=160)
    results = []
    for cuts in ([150], [86] + [1] * 64, [2] * 75, [7, 2, 16, 3, 2, 9, 5, 2, 15, 14, 33, 2, 40]):
        s = r.admit()
        results.append(feed(r, s, toks, cuts))                       # routing free: steps replay from graphs in bfloat16
        check(results[-1], want, dtype, f"{name} {dtype} cuts {cuts[:4]}", free_routing=True)
        r.release(s)
        if dtype == "bfloat16":
            s = r.admit()
            check(feed(r, s, toks, cuts, picks), want, dtype, f"{name} {dtype} cuts {cuts[:4]}, routing pinned")
            r.release(s)
    if dtype == "float32":
        for other in results[1:]:                                    # the cut changes nothing but the rounding of sums
            assert float(rel_err(other, results[0]).max()) < 1e-5


def test_unequal_requests_in_one_batch_slots_and_pages_used_again(folders):
    """Up to four live requests, portions of some beside single tokens of others, requests that sit a
    step out, in a pool so small that pages and slots come back into use: every position equals the
    plain implementation's."""
    from cajeta_llm_b200.engine.step import StepEntry
    d, (cfg, W) = folders("mixed", CONFIGS["mixed"], seed=7)
    rng = random.Random(4)
    lens = [23, 48, 17, 64, 35, 29, 52, 2, 41, 1]
    toks = {i: helpers.random_tokens(cfg["vocab"], n, seed=50 + i) for i, n in enumerate(lens)}
    both = {i: oracle(cfg, W, t) for i, t in toks.items()}
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
            out = r.step(entries, routing_pin=pin_rows(spans) if dtype == "bfloat16" else None).cpu()
            at = 0
            for i, n in who:
                got[i].append(out[at:at + n])
                at += n
                if live[i][1] == len(toks[i]):
                    r.release(live.pop(i)[0])
        for i in toks:
            check(torch.cat(got[i]), both[i][0], dtype, f"request {i} in the mixed batch ({dtype})")
        r.cache.books.check()


MARKER, ASKER = 7, 9


def marked(model_dir):
    """Weights made so that one far key decides a row.  Token MARKER's embedding is large along the stream's
    entry 0, token ASKER's along entry 1, no other token has either; W_k sends entry 0, and W_q entry 1, to the
    last entry of every head.  So a row of ASKER scores large exactly at keys of MARKER, its values are
    MARKER's (unlike its own), and whether it sees that key decides its logits."""
    from cajeta_llm_b200.weights.safetensors_io import Checkpoint, write_safetensors
    ck = Checkpoint(model_dir)
    tensors = {n: ck.load(n).float() for n in ck.names()}
    ck.close()
    with open(os.path.join(model_dir, "config.json")) as f:
        dim = json.load(f)["layers"][0]["mixer"]["dim"]
    g = torch.Generator().manual_seed(1)
    emb = tensors["embed"]
    emb.copy_(torch.randn(emb.shape, generator=g) * 0.3)
    emb[:, :2] = 0.0
    emb[MARKER, 0] = 6.0
    emb[ASKER, 1] = 6.0
    for n, t in tensors.items():
        if n.endswith(".mix.q") or n.endswith(".mix.k"):
            t.copy_(torch.randn(t.shape, generator=g) * 0.1)
            t[:, :2] = 0.0
            t[dim - 1::dim, 1 if n.endswith(".q") else 0] = 3.0
        elif n.endswith(".mix.v") or n.endswith(".mix.o"):
            t *= 30.0
        elif n.endswith(".mix.g"):
            t *= 20.0
        elif n in ("bigram", "side.embed", "loop.step") or n.endswith("side.proj"):
            t *= 0.0
    write_safetensors(os.path.join(model_dir, "model.safetensors"), {n: t.to(torch.bfloat16) for n, t in tensors.items()})


EDGE_LAYERS = {
    # head sizes of the general kernel (float32 and bfloat16) and of the bfloat16 tensor-core kernels
    "capped16": {"type": "attention", "mixer": {"heads": 2, "kv_heads": 1, "dim": 16, "vdim": 12, "scale": 0.1, "softcap": 40.0, "mask": {"size": 37}}, "mlp": None},
    "capped64": {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 64, "vdim": 64, "scale": 0.1, "softcap": 40.0, "mask": {"size": 37}}, "mlp": None},
    "capped128": {"type": "attention", "mixer": {"heads": 2, "kv_heads": 1, "dim": 128, "vdim": 128, "scale": 0.1, "softcap": 40.0, "mask": {"size": 130}}, "mlp": None},
    "rotated96": {"type": "attention_2", "mixer": {"heads": 2, "kv_heads": 2, "dim": 96, "vdim": 96, "scale": 0.3, "mask": {"size": 48},
                                                   "rot": {"base": 100.0, "dims": 8}}, "mlp": None},
    "rotated128": {"type": "attention_2", "mixer": {"heads": 2, "kv_heads": 1, "dim": 128, "vdim": 128, "scale": 0.25, "mask": {"size": 33},
                                                    "rot": {"base": 1000.0, "dims": 64, "scaling": {"factor": 2.0, "original": 16, "fast": 8.0, "slow": 1.0}}},
                   "mlp": None},
}


@pytest.mark.parametrize("name", sorted(EDGE_LAYERS))
def test_keys_at_the_window_edge_and_at_page_borders(folders, name):
    """MARKER appears once, then filler, then ASKER: placed so that the marker lies just inside and just
    outside the window, for starts that put both on either side of page borders, for rows inside a
    prompt portion and rows decoded one by one.  An oracle whose window is one token off is told apart
    by a wide margin in the same rows."""
    layer = EDGE_LAYERS[name]
    w = layer["mixer"]["mask"]["size"]
    raw = config_of([layer], width=32, vocab=60, bigram=(13, 1, 1), side=4)
    d, (cfg, W) = folders("edge_" + name, raw, seed=9, touch=marked)
    rng = random.Random(3)
    fill = [t for t in range(60) if t not in (MARKER, ASKER)]
    runners = {dtype: runner_for(d, dtype, max_tokens=256) for dtype in ("float32", "bfloat16")}
    for dist in (w - 2, w - 1, w, w + 1):
        for start in (0, 5, 15, 16, 31):
            toks = [rng.choice(fill) for _ in range(start)] + [MARKER] + [rng.choice(fill) for _ in range(dist - 1)] + [ASKER]
            toks += [rng.choice(fill) for _ in range(3)]
            row, n = start + dist, start + dist + 4
            want = torch.from_numpy(P.forward(cfg, W, toks))
            off = copy.deepcopy(cfg)
            off["layers"][0]["mixer"]["mask"]["size"] = w + (1 if dist >= w else -1)
            wrong = torch.from_numpy(P.forward(off, W, toks))
            shows = dist in (w - 1, w)
            if shows:
                assert float(rel_err(wrong[row:row + 1], want[row:row + 1])) > 0.3, "the test's weights do not show the edge"
            for dtype, r in runners.items():
                for cuts in ([n], [row] + [1] * 4, [start + 1, 2, row - start - 4, 2] + [1] * 3):
                    s = r.admit()
                    got = feed(r, s, toks, cuts)
                    r.release(s)
                    e = rel_err(got, want)
                    bound = 1e-4 if dtype == "float32" else 6e-2
                    assert float(e.max()) < bound, f"{dtype} distance {dist}, start {start}, cuts {cuts[:4]}: row {int(e.argmax())} differs by {float(e.max()):.2e}"
                    if shows:
                        assert float(rel_err(got[row:row + 1], wrong[row:row + 1])) > 0.2


def test_far_keys_without_a_window(folders):
    """No ``mask``: every earlier key is seen.  The marker sits hundreds of tokens back, across many pages."""
    layer = {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 64, "vdim": 64, "scale": 0.1}, "mlp": None}
    raw = config_of([layer], width=32, vocab=60, bigram=None, side=0)
    d, (cfg, W) = folders("far", raw, seed=9, touch=marked)
    rng = random.Random(5)
    fill = [t for t in range(60) if t not in (MARKER, ASKER)]
    toks = [rng.choice(fill) for _ in range(3)] + [MARKER] + [rng.choice(fill) for _ in range(300)] + [ASKER, fill[0], ASKER]
    want = torch.from_numpy(P.forward(cfg, W, toks))
    near = torch.from_numpy(P.forward(cfg, W, toks[4:]))
    assert float(rel_err(near[-3:-2], want[-3:-2])) > 0.3
    for dtype in ("float32", "bfloat16"):
        r = runner_for(d, dtype, max_tokens=320)
        for cuts in ([307], [300, 4] + [1] * 3, [17] * 18 + [1]):
            s = r.admit()
            check(feed(r, s, toks, cuts), want, dtype, f"far keys {dtype} cuts {cuts[:3]}")
            r.release(s)


def test_first_tokens_and_long_decoding(folders):
    d, (cfg, W) = folders("other", CONFIGS["other"], seed=7)
    for dtype in ("float32", "bfloat16"):
        r = runner_for(d, dtype, max_tokens=192)
        for n in (1, 2, 3, 4, 6):
            toks = helpers.random_tokens(cfg["vocab"], n, seed=20 + n)
            s = r.admit()
            check(feed(r, s, toks, [1] * n), oracle(cfg, W, toks)[0], dtype, f"{n} first tokens one by one ({dtype})", free_routing=True)
            r.release(s)
        toks = helpers.random_tokens(cfg["vocab"], 183, seed=33)
        s = r.admit()
        check(feed(r, s, toks, [3] + [1] * 180), oracle(cfg, W, toks)[0], dtype, f"long decoding ({dtype})", free_routing=True)
        r.release(s)


def test_captured_steps_equal_uncaptured_ones(folders):
    from cajeta_llm_b200.engine.step import StepEntry
    d, (cfg, W) = folders("wide", CONFIGS["wide"], seed=7)
    toks = [helpers.random_tokens(cfg["vocab"], 100, seed=70 + i) for i in range(3)]
    outs = []
    for graphs in (True, False):
        r = runner_for(d, "bfloat16", max_tokens=128, cuda_graphs=graphs)
        slots = [r.admit() for _ in toks]
        got = []
        for lo, hi in ((0, 12), (12, 24), (24, 36), (36, 48)):       # the same shape again and again: captured, then replayed
            got.append(r.step([StepEntry(s, t[lo:hi], [hi - lo - 1]) for s, t in zip(slots, toks)]).cpu())
        for i in range(48, 100):
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
    wa, wb = oracle(cfg, W, a)[0], oracle(cfg, W, b)[0]
    got = {n: torch.from_numpy(np.fromfile(os.path.join(str(tmp_path), f"{n}.f32"), dtype="<f4").reshape(-1, cfg["vocab"])) for n in range(3)}
    check(got[0], wa[10:11], "float32", "step 0")
    check(got[1], wb[8:9], "float32", "step 1")
    check(got[2], wa[[11, 19]], "float32", "step 2")


def random_config(seed):
    """A configuration drawn at random: layer order, every size, the loop, which extras exist."""
    rng = random.Random(seed)
    width = rng.choice([40, 72, 136, 256])
    big = width >= 128

    def pick(lo, hi):
        return rng.randint(lo, hi)

    layers = []
    for _ in range(rng.randint(1, 5)):
        kind = rng.choice(MIXERS)
        kv = pick(1, 3)
        dim = rng.choice([64, 96, 128]) if big and rng.random() < 0.5 else 2 * pick(2, 24)
        m = {"heads": kv * pick(1, 3), "kv_heads": kv, "dim": dim, "scale": rng.choice([0.1, 0.3, 1.0])}
        if rng.random() < 0.8:
            m["mask"] = {"size": rng.choice([1, 2, 7, 16, 17, 33, 64, 100])}
        if kind == "attention":
            m["vdim"] = dim if rng.random() < 0.5 else pick(3, 40)
            if rng.random() < 0.7:
                m["softcap"] = rng.choice([2.0, 10.0, 50.0])
        else:
            m["vdim"] = dim
            if rng.random() < 0.8:
                m["rot"] = {"base": rng.choice([100.0, 10000.0, 500000.0]), "dims": 2 * pick(1, dim // 2)}
                if rng.random() < 0.6:
                    m["rot"]["scaling"] = {"factor": rng.choice([2.0, 8.0]), "original": rng.choice([8, 32, 4096]),
                                           "fast": rng.choice([4.0, 32.0]), "slow": rng.choice([0.25, 1.0])}
        ff = rng.choice([None, "dense", "moe", "moe"])
        if ff == "dense":
            mlp = {"kind": "dense", "ff": rng.choice([pick(8, 60), 128, 200]) if big else pick(8, 60)}
        elif ff == "moe":
            count = pick(1, 4)
            per = pick(1, 3)
            keep = pick(1, count)
            mlp = {"kind": "moe", "expert": {"ff": rng.choice([pick(8, 60), 128, 136]) if big else pick(8, 60), "limit": rng.choice([0.02, 0.1, 7.0])},
                   "router": {"experts": count * per, "top": pick(1, keep * per)}}
            if rng.random() < 0.7:
                mlp["router"]["groups"] = {"count": count, "keep": keep}
            if rng.random() < 0.6:
                mlp["shared"] = {"ff": rng.choice([mlp["expert"]["ff"], 2 * mlp["expert"]["ff"], pick(8, 40)]), "limit": rng.choice([0.02, 7.0])}
        else:
            mlp = None
        layers.append({"type": kind, "mixer": m, "mlp": mlp})
    loop = None
    if rng.random() < 0.7:
        a = pick(0, len(layers) - 1)
        loop = (a, pick(a + 1, len(layers)), pick(1, 3))
    return config_of(layers, width=width, vocab=rng.choice([70, 131, 300]), eps=rng.choice([1e-5, 1e-6]), loop=loop,
                     bigram=rng.choice([None, (1, 0, 1), (31, 7, 2), (1013, 29, 5)]), side=rng.choice([0, 1, 5, 24]))


MIXERS = ("attention", "attention_2")


@pytest.mark.parametrize("seed", range(10))
def test_configurations_drawn_at_random(folders, seed):
    raw = random_config(2000 + seed)
    d, (cfg, W) = folders(f"random{seed}", raw, seed=100 + seed)
    toks = helpers.random_tokens(cfg["vocab"], 120, seed=seed)
    want, picks = oracle(cfg, W, toks)
    for dtype in ("float32", "bfloat16"):
        r = runner_for(d, dtype, max_tokens=128)
        for cuts in ([120], [17, 2, 9, 60] + [1] * 32):
            s = r.admit()
            check(feed(r, s, toks, cuts, picks if dtype == "bfloat16" else None), want, dtype,
                  f"{json.dumps(raw)} {dtype} cuts {cuts[:3]}")
            r.release(s)
