"""Saropel restated plainly: one function per mechanism, float64, loops over tokens.

Nothing here is shared with the engine: weights arrive as a dict of numpy arrays by tensor
name, the configuration as the parsed ``config.json``.  Slow on purpose; the tests use small
sizes.  Notation: ``x`` a row of the residual stream, ``h`` its normed form, ``p`` a position.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import numpy as np


def rms(x: np.ndarray, eps: float) -> np.ndarray:
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def norm_one_plus(x, w, eps):
    return rms(x, eps) * (1.0 + w)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def embed_rows(cfg, W, tokens: List[int]) -> np.ndarray:
    """Token rows plus the row of the pair table that (previous token, token) hashes to."""
    out = np.zeros((len(tokens), W["embed"].shape[1]))
    bg = (cfg.get("embedding") or {}).get("bigram")
    for t, tok in enumerate(tokens):
        out[t] = W["embed"][tok]
        if bg:
            row = bg["buckets"] if t == 0 else (tokens[t - 1] * bg["mul_prev"] + tok * bg["mul_cur"]) % bg["buckets"]
            out[t] += W["bigram"][row]
    return out


def rotary_tables(rot: dict, positions: np.ndarray):
    """cos and sin [T, dims/2] of the rotation, with the stretched frequencies when ``scaling`` is given."""
    dims, base = rot["dims"], float(rot["base"])
    half = dims // 2
    i = np.arange(half, dtype=np.float64)
    f = base ** (-2.0 * i / dims)
    mag = 1.0
    sc = rot.get("scaling")
    if sc:
        factor, orig = float(sc["factor"]), float(sc["original"])

        def corr(turns):
            return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

        lo = max(math.floor(corr(float(sc["fast"]))), 0)
        hi = min(math.ceil(corr(float(sc["slow"]))), dims - 1)
        ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        f = f / factor * ramp + f * (1.0 - ramp)
        mag = 0.1 * math.log(factor) + 1.0
    ang = positions[:, None].astype(np.float64) * f[None, :]
    return np.cos(ang) * mag, np.sin(ang) * mag


def rotate(v: np.ndarray, cos: np.ndarray, sin: np.ndarray, dims: int) -> np.ndarray:
    """v [heads, dim] at one position; entry i is paired with entry i + dims/2."""
    half = dims // 2
    out = v.copy()
    a, b = v[:, :half], v[:, half:dims]
    out[:, :half] = a * cos - b * sin
    out[:, half:dims] = b * cos + a * sin
    return out


def attention_mixer(m: dict, kind: str, W, pre: str, h: np.ndarray, eps: float) -> np.ndarray:
    """Both attention mixers over a whole sequence h [T, width] (positions 0..T-1)."""
    T = h.shape[0]
    H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ W[pre + "q"].T).reshape(T, H, dim)
    k = (h @ W[pre + "k"].T).reshape(T, G, dim)
    if kind == "attention_2":
        v = k.copy()
        q = rms(q, eps) * W[pre + "q.norm"]
        k = rms(k, eps) * W[pre + "k.norm"]
        rot = m.get("rot")
        if rot:
            cos, sin = rotary_tables(rot, np.arange(T))
            q = np.stack([rotate(q[t], cos[t], sin[t], rot["dims"]) for t in range(T)])
            k = np.stack([rotate(k[t], cos[t], sin[t], rot["dims"]) for t in range(T)])
    else:
        v = (h @ W[pre + "v"].T).reshape(T, G, vdim)
    window = (m.get("mask") or {}).get("size", 0)
    cap = m.get("softcap") if kind == "attention" else None
    out = np.zeros((T, H, v.shape[-1]))
    for t in range(T):
        lo = max(0, t - window + 1) if window else 0
        for hh in range(H):
            g = hh // (H // G)
            s = (k[lo:t + 1, g] @ q[t, hh]) * m["scale"]
            if cap:
                s = cap * np.tanh(s / cap)
            e = np.exp(s - s.max())
            out[t, hh] = (e / e.sum()) @ v[lo:t + 1, g]
    if kind == "attention_2":
        gate = sigmoid(h @ W[pre + "g"].T)            # [T, H]
        out = out * gate[:, :, None]
    return out.reshape(T, -1) @ W[pre + "o"].T


def dense_ff(W, pre: str, h):
    a = h @ W[pre + "gate"].T
    return ((a * sigmoid(a)) * (h @ W[pre + "up"].T)) @ W[pre + "down"].T


def capped_expert(W, pre: str, h, limit: float):
    g = np.minimum(h @ W[pre + "gate"].T, limit)
    u = np.clip(h @ W[pre + "up"].T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ W[pre + "down"].T


def route(z: np.ndarray, top: int, groups: Optional[dict]):
    """Scores and the chosen experts of one token's router logits z."""
    s = np.exp(z - z.max())
    s = s / s.sum()
    E = len(s)
    allowed = np.ones(E, dtype=bool)
    if groups and groups.get("count", 1) > 1:
        n = groups["count"]
        per = E // n
        gs = s.reshape(n, per).max(axis=1)
        best = np.argsort(-gs, kind="stable")[: groups["keep"]]
        allowed = np.zeros(E, dtype=bool)
        for b in best:
            allowed[b * per:(b + 1) * per] = True
    order = [e for e in np.argsort(-s, kind="stable") if allowed[e]][:top]
    return s, order


def moe_ff(ff: dict, W, pre: str, h, picked=None):
    T = h.shape[0]
    out = np.zeros((T, W[pre + "e0.down"].shape[0]))
    r = ff["router"]
    for t in range(T):
        s, picks = route(W[pre + "router"] @ h[t], r["top"], r.get("groups"))
        if picked is not None:
            picked.append([int(e) for e in picks])
        for e in picks:
            out[t] += s[e] * capped_expert(W, f"{pre}e{e}.", h[t:t + 1], ff["expert"]["limit"])[0]
    if ff.get("shared"):
        sh = capped_expert(W, pre + "shared.", h, ff["shared"]["limit"])
        out += sh * sigmoid(h @ W[pre + "shared.sg"].T)
    return out


def token_side(cfg, W, i: int, x, tokens, eps):
    dim = cfg["token_side"]["dim"]
    e = W["side.embed"][np.asarray(tokens)][:, i * dim:(i + 1) * dim]
    g = gelu_tanh(x @ W[f"l{i}.side.gate"].T) * e
    y = g @ W[f"l{i}.side.proj"].T
    return x + rms(y, eps) * W[f"l{i}.side.norm"]


def layer(cfg, W, i: int, x, tokens, picked=None):
    L, eps = cfg["layers"][i], cfg["norm"]["eps"]
    h = norm_one_plus(x, W[f"l{i}.norm1"], eps)
    y = attention_mixer(L["mixer"], L["type"], W, f"l{i}.mix.", h, eps)
    ff = L.get("mlp")
    if ff is not None:
        y = y + (dense_ff(W, f"l{i}.mlp.", h) if ff["kind"] == "dense" else moe_ff(ff, W, f"l{i}.mlp.", h, picked))
    x = x + y
    if cfg.get("token_side"):
        x = token_side(cfg, W, i, x, tokens, eps)
    return x


def layer_runs(cfg):
    """[(layer, pass number or None, first of its pass)] in run order."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None, False) for i in range(n)]
    runs = [(i, None, False) for i in range(loop["start"])]
    for t in range(loop["times"]):
        for i in range(loop["start"], loop["stop"]):
            runs.append((i, t, i == loop["start"]))
    return runs + [(i, None, False) for i in range(loop["stop"], n)]


def forward(cfg, W, tokens: List[int], keep_layers: bool = False, picks: Optional[list] = None):
    """Logits [T, vocab] of a whole sequence (and the stream after every layer run).  ``picks``: a list
    that receives, per layer run, None or the experts every token picked ([T][top])."""
    W = {k: np.asarray(v, dtype=np.float64) for k, v in W.items()}
    x0 = embed_rows(cfg, W, tokens)
    x = x0.copy()
    kept = []
    for i, t, first in layer_runs(cfg):
        if first:
            if t > 0:
                x = x + x0
            x = x + W["loop.step"][t]
        picked = [] if (cfg["layers"][i].get("mlp") or {}).get("kind") == "moe" else None
        x = layer(cfg, W, i, x, tokens, picked)
        if picks is not None:
            picks.append((i, picked))
        if keep_layers:
            kept.append(x.copy())
    logits = norm_one_plus(x, W["final.norm"], cfg["norm"]["eps"]) @ W["head"].T
    return (logits, np.stack(kept)) if keep_layers else logits


def greedy(cfg, W, prompt: List[int], new_tokens: int) -> List[int]:
    toks, out = list(prompt), []
    for _ in range(new_tokens):
        nxt = int(np.argmax(forward(cfg, W, toks)[-1]))
        out.append(nxt)
        toks.append(nxt)
    return out


def read_model(model_dir: str):
    """config.json and the tensors of model.safetensors as float64 arrays (a reader of its own)."""
    import json
    import os
    import struct

    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    with open(os.path.join(model_dir, "model.safetensors"), "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    W = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        raw = data[lo:hi]
        if info["dtype"] == "BF16":
            bits = np.frombuffer(raw, dtype=np.uint16).astype(np.uint32) << 16
            arr = bits.view(np.float32)
        elif info["dtype"] == "F32":
            arr = np.frombuffer(raw, dtype=np.float32)
        else:
            raise ValueError(f"{name}: dtype {info['dtype']}")
        W[name] = arr.astype(np.float64).reshape(info["shape"])
    return cfg, W
