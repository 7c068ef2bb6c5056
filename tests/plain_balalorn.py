"""A plain, slow restatement of the Balalorn design in float64, one function per mechanism.

Nothing here is shared with the engine: whole sequences, Python loops over tokens, no
cache and no batch.  ``weights`` maps tensor names to float64 torch tensors, ``config``
is the parsed config.json.  Notation: ``h`` is a sublayer's input [T, width].

Layer:            x <- x + rms(mixer(x)) * w1 ;  x <- x + rms(ff(x)) * w2   (norm on the
                  sublayer's OUTPUT; a layer may have no feed-forward)
rms(v):           v / sqrt(mean(v^2) + eps)
"""
import math

import torch

F64 = torch.float64


def rms_unit(v, eps):
    return v / torch.sqrt((v * v).mean(dim=-1, keepdim=True) + eps)


def silu(v):
    return v * torch.sigmoid(v)


def softplus(v):
    return torch.where(v > 30.0, v, torch.log1p(torch.exp(torch.clamp(v, max=30.0))))


def short_conv(x, w, bias=None):
    """Causal convolution per channel: y[t, c] = sum_j w[c, taps-1-j] x[t-j, c] (+ bias),
    x before the sequence's start being zero."""
    T, C = x.shape
    taps = w.shape[1]
    y = torch.zeros((T, C), dtype=F64)
    for t in range(T):
        for j in range(taps):
            if t - j >= 0:
                y[t] += w[:, taps - 1 - j] * x[t - j]
    if bias is not None:
        y = y + bias
    return y


def rotate_pairs(v, positions, base, dims):
    """Rotate the first ``dims`` entries of the last axis, (2i, 2i+1) being pair i, by the
    angle p * base^(-2i/dims).  v: [T, ..., D]."""
    out = v.clone()
    for t, p in enumerate(positions):
        for i in range(dims // 2):
            a = float(p) * base ** (-2.0 * i / dims)
            c, s = math.cos(a), math.sin(a)
            u, w = v[t, ..., 2 * i].clone(), v[t, ..., 2 * i + 1].clone()
            out[t, ..., 2 * i] = u * c - w * s
            out[t, ..., 2 * i + 1] = w * c + u * s
    return out


# -- mixers ---------------------------------------------------------------------------
def mamba2(h, W, m, eps):
    """State-space mixer.  m: heads, vdim, state, groups, norm_groups, conv."""
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    T = h.shape[0]
    proj = h @ W["in"].T
    z = proj[:, :inner]
    xbc = proj[:, inner:2 * inner + 2 * G * N]
    dt = proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(short_conv(xbc, W["conv"], W["conv.b"]))
    x = xbc[:, :inner].reshape(T, H, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + W["dt_bias"])
    A = torch.exp(W["A_log"])
    y = torch.zeros((T, H, P), dtype=F64)
    for hd in range(H):
        g = hd // (H // G)
        S = torch.zeros((N, P), dtype=F64)
        for t in range(T):
            S = torch.exp(-A[hd] * dt[t, hd]) * S + dt[t, hd] * torch.outer(B[t, g], x[t, hd])
            y[t, hd] = S.T @ C[t, g] + W["D"][hd] * x[t, hd]
    y = y.reshape(T, inner) * silu(z)
    parts = m["norm_groups"]
    y = rms_unit(y.reshape(T, parts, inner // parts), eps).reshape(T, inner) * W["norm"]
    return y @ W["o"].T


def delta(h, W, m, eps):
    """Gated delta rule.  m: heads, kv_heads, dim, vdim, conv."""
    H, KH, D, P = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = silu(short_conv(h @ W["q"].T, W["q.conv"])).reshape(T, KH, D)
    k = silu(short_conv(h @ W["k"].T, W["k.conv"])).reshape(T, KH, D)
    v = silu(short_conv(h @ W["v"].T, W["v.conv"])).reshape(T, H, P)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ W["b"].T)
    decay = torch.exp(-torch.exp(W["A_log"]) * softplus(h @ W["a"].T + W["dt_bias"]))
    o = torch.zeros((T, H, P), dtype=F64)
    for hd in range(H):
        kh = hd // (H // KH)
        S = torch.zeros((D, P), dtype=F64)
        for t in range(T):
            S = decay[t, hd] * S
            u = beta[t, hd] * (v[t, hd] - S.T @ k[t, kh])
            S = S + torch.outer(k[t, kh], u)
            o[t, hd] = S.T @ q[t, kh]
    o = rms_unit(o, eps) * W["norm"]
    o = o.reshape(T, H * P) * silu(h @ W["g"].T)
    return o @ W["o"].T


def latent_keys(h, W, m, eps, positions):
    """What a latent-attention layer caches: the normed latent c [T, kv_rank] and the one
    rotated key part [T, rot_dim] all heads share."""
    R = m["kv_rank"]
    d = h @ W["dkv"].T
    c = rms_unit(d[:, :R], eps) * W["dkv.norm"]
    kr = rotate_pairs(d[:, R:], positions, m["rot"]["base"], m["rot"]["dims"])
    return c, kr


def latent_attention(h, W, m, eps, positions, shared=None):
    """Attention over a compressed latent.  ``shared``: (c, kr) of the layer named by
    ``kv_from``; None when the layer projects its own.  Returns (output, (c, kr))."""
    H, D, RD, P = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    T = h.shape[0]
    c, kr = shared if shared is not None else latent_keys(h, W, m, eps, positions)
    q = (h @ W["q"].T).reshape(T, H, D + RD)
    q_plain = q[:, :, :D]
    q_rot = rotate_pairs(q[:, :, D:], positions, m["rot"]["base"], m["rot"]["dims"])
    k_plain = (c @ W["uk"].T).reshape(T, H, D)
    val = (c @ W["uv"].T).reshape(T, H, P)
    gate = torch.sigmoid(h @ W["g"].T)
    out = torch.zeros((T, H, P), dtype=F64)
    for hd in range(H):
        for t in range(T):
            s = (k_plain[:t + 1, hd] @ q_plain[t, hd] + kr[:t + 1] @ q_rot[t, hd]) * m["scale"]
            w = torch.softmax(s, dim=0)
            out[t, hd] = (w[:, None] * val[:t + 1, hd]).sum(0) * gate[t, hd]
    return out.reshape(T, H * P) @ W["o"].T, (c, kr)


# -- feed-forwards --------------------------------------------------------------------
def gated_ff(h, gate, up, down):
    return (silu(h @ gate.T) * (h @ up.T)) @ down.T


def routed_ff(h, W, experts, top):
    """Sigmoid router; the ``top`` largest scores pick the experts; a score multiplies its
    expert's INPUT and is not renormalised.  Returns (output, picks [T, top])."""
    s = torch.sigmoid(h @ W["router"].T)
    T = h.shape[0]
    out = torch.zeros_like(h)
    picks = torch.zeros((T, top), dtype=torch.long)
    for t in range(T):
        order = sorted(range(experts), key=lambda e: (-float(s[t, e]), e))[:top]
        for j, e in enumerate(order):
            picks[t, j] = e
            out[t] += gated_ff(s[t, e] * h[t:t + 1], W[f"e{e}.gate"], W[f"e{e}.up"], W[f"e{e}.down"])[0]
    return out, picks


# -- the model ------------------------------------------------------------------------
def sub(weights, prefix):
    n = len(prefix) + 1
    return {k[n:]: v for k, v in weights.items() if k.startswith(prefix + ".")}


def forward(tokens, weights, config, positions=None, picks=None):
    """Logits [T, vocab] and the residual stream after every layer [layers, T, width].
    ``picks`` (a dict): receives, by layer index, the experts each position picked [T, top]."""
    eps = config["norm"]["eps"]
    T = len(tokens)
    positions = list(range(T)) if positions is None else positions
    x = weights["embed"][torch.tensor(tokens, dtype=torch.long)].clone()
    kept, after = {}, []
    for i, layer in enumerate(config["layers"]):
        W, m = sub(weights, f"l{i}.mix"), layer["mixer"]
        if layer["type"] == "mamba2":
            y = mamba2(x, W, m, eps)
        elif layer["type"] == "delta":
            y = delta(x, W, m, eps)
        elif layer["type"] == "latent_attention":
            src = m.get("kv_from")
            y, kept[i] = latent_attention(x, W, m, eps, positions, kept[src] if src is not None else None)
        else:
            raise ValueError(layer["type"])
        x = x + rms_unit(y, eps) * weights[f"l{i}.norm1"]
        ff = layer.get("mlp")
        if ff is not None:
            Wf = sub(weights, f"l{i}.mlp")
            if ff["kind"] == "dense":
                y = gated_ff(x, Wf["gate"], Wf["up"], Wf["down"])
            else:
                y, chosen = routed_ff(x, Wf, ff["router"]["experts"], ff["router"]["top"])
                if picks is not None:
                    picks[i] = chosen
            x = x + rms_unit(y, eps) * weights[f"l{i}.norm2"]
        after.append(x.clone())
    logits = (rms_unit(x, eps) * weights["final.norm"]) @ weights["head"].T
    return logits, torch.stack(after)


# -- reading a model folder (a reader of its own: 8-byte length, JSON header, raw data) -------
def read_model(model_dir):
    import json
    import os
    import struct

    import numpy as np

    with open(os.path.join(model_dir, "config.json")) as f:
        config = json.load(f)
    with open(os.path.join(model_dir, "model.safetensors"), "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    weights = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        raw = data[lo:hi]
        if info["dtype"] == "BF16":
            bits = np.frombuffer(raw, dtype=np.uint16).astype(np.uint32) << 16
            t = torch.from_numpy(bits.view(np.float32).copy()).to(F64)
        elif info["dtype"] == "F32":
            t = torch.from_numpy(np.frombuffer(raw, dtype=np.float32).copy()).to(F64)
        else:
            raise ValueError(f"{name}: dtype {info['dtype']}")
        weights[name] = t.reshape(info["shape"])
    return config, weights


def greedy(config, weights, prompt, n):
    toks, out = list(prompt), []
    for _ in range(n):
        logits, _ = forward(toks, weights, config)
        out.append(int(torch.argmax(logits[-1])))
        toks.append(out[-1])
    return out
