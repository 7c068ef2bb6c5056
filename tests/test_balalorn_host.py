"""Balalorn on the host: configuration and plan, the random-weights folder, and the plain
implementation's own mechanisms against independent closed forms."""
import copy
import json
import os

import pytest
import torch

import helpers
import plain_balalorn as P

RAW = {"architecture": "Balalorn", "width": 32, "vocab": 50, "norm": {"eps": 1e-6}, "layers": [
    {"type": "latent_attention", "mixer": {"heads": 2, "dim": 8, "rot_dim": 4, "vdim": 6, "kv_rank": 10, "scale": 0.3,
                                           "rot": {"base": 100.0, "dims": 2}}, "mlp": None},
    {"type": "mamba2", "mixer": {"heads": 4, "vdim": 6, "state": 5, "groups": 2, "norm_groups": 3, "conv": 3},
     "mlp": {"kind": "moe", "expert": {"ff": 12}, "router": {"experts": 3, "top": 2}}},
    {"type": "latent_attention", "mixer": {"heads": 3, "dim": 4, "rot_dim": 4, "vdim": 8, "kv_rank": 10, "scale": 0.5, "kv_from": 0,
                                           "rot": {"base": 100.0, "dims": 2}}, "mlp": {"kind": "dense", "ff": 20}},
    {"type": "delta", "mixer": {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 5, "conv": 2}, "mlp": None},
]}


def plan_of(raw):
    import cajeta_llm_b200  # noqa: F401
    from cajeta_llm_b200.config import parse_config_dict
    from cajeta_llm_b200.config.base import get_architecture
    cfg = parse_config_dict(raw)
    return cfg, get_architecture(cfg.architecture).build_plan(cfg)


def test_the_plan_follows_the_list_of_layers():
    cfg, plan = plan_of(RAW)
    assert [l.mixer.kind for l in plan.layers] == ["latent_attention", "ssd", "latent_attention", "gated_delta"]
    assert [None if l.feed_forward is None else l.feed_forward.kind for l in plan.layers] == [None, "sparse_moe", "dense_swiglu", None]
    assert [e.cache_from for e in plan.schedule] == [None, None, 0, None]
    assert plan.layers[1].feed_forward["score"] == "sigmoid" and plan.layers[1].feed_forward["weight_on"] == "input"
    assert plan.layers[0].mixer["position"]["rotary_dim"] == 2 and plan.layers[2].mixer["owns_cache"] is False
    assert cfg.to_json_dict()["layers"] == RAW["layers"]


def test_tensor_names_and_shapes():
    from cajeta_llm_b200.engine.model import build_model
    from cajeta_llm_b200.parts.base import Runtime
    cfg, _ = plan_of(RAW)
    model = build_model(cfg, Runtime("float32", "cpu"))
    p = {n: tuple(s.shape) for n, s in model.params().items()}
    assert p["embed"] == (50, 32) and p["head"] == (50, 32) and p["final.norm"] == (32,) and p["l0.norm1"] == (32,)
    assert "l0.norm2" not in p and "l3.norm2" not in p and p["l1.norm2"] == (32,)
    assert p["l0.mix.q"] == (2 * 12, 32) and p["l0.mix.dkv"] == (14, 32) and p["l0.mix.dkv.norm"] == (10,) and p["l0.mix.g"] == (2, 32)
    assert p["l0.mix.uk"] == (16, 10) and p["l0.mix.uv"] == (12, 10) and p["l0.mix.o"] == (32, 12)
    assert "l2.mix.dkv" not in p and p["l2.mix.q"] == (3 * 8, 32)
    assert p["l1.mix.in"] == (2 * 24 + 2 * 10 + 4, 32) and p["l1.mix.conv"] == (44, 3) and p["l1.mix.conv.b"] == (44,)
    assert p["l1.mix.D"] == (4,) and p["l1.mix.norm"] == (24,) and p["l1.mix.o"] == (32, 24)
    assert p["l1.mlp.router"] == (3, 32) and p["l1.mlp.e2.gate"] == (12, 32) and p["l1.mlp.e0.down"] == (32, 12)
    assert p["l2.mlp.up"] == (20, 32)
    assert p["l3.mix.q"] == (12, 32) and p["l3.mix.v.conv"] == (20, 2) and p["l3.mix.a"] == (4, 32) and p["l3.mix.norm"] == (5,)
    needs, states = model.kv_needs(), model.state_needs()
    assert needs[0].head_dim == 14 and needs[0].kv_heads == 1 and not needs[0].values and needs[1] is None
    from cajeta_llm_b200.csrc.kernels import state_scan_floats
    assert states[1].shape == (2 * 44 + state_scan_floats(4, 5, 6),) and states[3].shape == (1 * 44 + state_scan_floats(4, 6, 5),)
    assert states[0] is None and state_scan_floats(4, 5, 6) >= 4 * 5 * 6 and state_scan_floats(16, 128, 128) == 16 * 128 * 128 == state_scan_floats(64, 128, 32)


@pytest.mark.parametrize("change, message", [
    (lambda c: c["layers"][0].update(type="attention"), "type"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=3), "kv_from"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=1), "owns no latent cache"),
    (lambda c: c["layers"][2]["mixer"].update(kv_rank=12), "must equal"),
    (lambda c: c["layers"][1]["mixer"].update(groups=3), "multiple"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=4), "top"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=6), "dims"),
    (lambda c: c.pop("norm"), "norm.eps"),
    (lambda c: c["layers"][3]["mixer"].pop("conv"), "conv"),
])
def test_configuration_errors_name_the_key(change, message):
    from cajeta_llm_b200.config.base import ConfigError
    raw = copy.deepcopy(RAW)
    change(raw)
    with pytest.raises(ConfigError) as e:
        plan_of(raw)
    assert message in str(e.value)


def test_random_weights_folder_round_trip(tmp_path):
    helpers.write_model(str(tmp_path), RAW, seed=3)
    cfg, W = P.read_model(str(tmp_path))
    assert cfg["layers"] == RAW["layers"] and W["l1.mix.conv"].shape == (44, 3)
    logits, after = P.forward([1, 2, 3, 4, 5], W, cfg)
    assert logits.shape == (5, 50) and after.shape == (4, 5, 32) and bool(torch.isfinite(logits).all())


# -- the plain implementation's mechanisms against closed forms of their own --------------
def test_short_conv_is_a_causal_correlation():
    g = torch.Generator().manual_seed(0)
    x, w, b = torch.randn(9, 5, generator=g).double(), torch.randn(5, 4, generator=g).double(), torch.randn(5, generator=g).double()
    want = torch.nn.functional.conv1d(torch.nn.functional.pad(x.T[None], (3, 0)), w[:, None, :], b, groups=5)[0].T
    assert torch.allclose(P.short_conv(x, w, b), want, atol=1e-12)


def test_rotation_keeps_lengths_and_relative_angles():
    g = torch.Generator().manual_seed(1)
    q, k = torch.randn(1, 6, generator=g).double(), torch.randn(1, 6, generator=g).double()
    a = (P.rotate_pairs(q, [7], 100.0, 4) * P.rotate_pairs(k, [3], 100.0, 4)).sum()
    b = (P.rotate_pairs(q, [14], 100.0, 4) * P.rotate_pairs(k, [10], 100.0, 4)).sum()
    assert abs(float(a - b)) < 1e-12
    r = P.rotate_pairs(q, [5], 100.0, 4)
    assert torch.allclose(r[0, 4:], q[0, 4:]) and abs(float(r[0, :4].norm() - q[0, :4].norm())) < 1e-12
    # pair (0, 1) turns by p * base^0 = p radians
    e = P.rotate_pairs(torch.tensor([[1.0, 0.0, 0.0, 0.0]], dtype=torch.float64), [2], 100.0, 4)
    assert torch.allclose(e[0, :2], torch.tensor([torch.cos(torch.tensor(2.0)), torch.sin(torch.tensor(2.0))], dtype=torch.float64))


def test_state_space_scan_equals_its_unrolled_sum():
    """y_t = sum_{s<=t} (prod_{s<r<=t} a_r) dt_s (C_t . B_s) x_s + D x_t for one head."""
    g = torch.Generator().manual_seed(2)
    m = {"heads": 1, "vdim": 3, "state": 4, "groups": 1, "norm_groups": 1, "conv": 1}
    W = {"in": torch.randn(2 * 3 + 2 * 4 + 1, 6, generator=g).double(), "conv": torch.ones(3 + 8, 1).double(), "conv.b": torch.zeros(11).double(),
         "dt_bias": torch.tensor([0.3]).double(), "A_log": torch.tensor([-0.4]).double(), "D": torch.tensor([0.7]).double(),
         "norm": torch.ones(3).double(), "o": torch.eye(3).double()}
    h = torch.randn(5, 6, generator=g).double()
    got = P.mamba2(h, W, m, 1e-6)
    proj = h @ W["in"].T
    z, xbc, dt = proj[:, :3], P.silu(proj[:, 3:14]), P.softplus(proj[:, 14] + 0.3)
    x, B, C = xbc[:, :3], xbc[:, 3:7], xbc[:, 7:]
    a = torch.exp(-torch.exp(torch.tensor(-0.4, dtype=torch.float64)) * dt)
    y = torch.zeros(5, 3, dtype=torch.float64)
    for t in range(5):
        for s in range(t + 1):
            y[t] += a[s + 1:t + 1].prod() * dt[s] * (C[t] @ B[s]) * x[s]
        y[t] += 0.7 * x[t]
    want = P.rms_unit(y * P.silu(z), 1e-6)
    assert torch.allclose(got, want, atol=1e-10)


def test_delta_rule_writes_what_it_then_reads():
    """With beta = 1 and no decay, after a token's update S^T k_t = v_t exactly (k is a unit vector)."""
    g = torch.Generator().manual_seed(3)
    k = torch.randn(4, 6, generator=g).double()
    k = k / k.norm(dim=-1, keepdim=True)
    v = torch.randn(4, 5, generator=g).double()
    S = torch.zeros(6, 5, dtype=torch.float64)
    for t in range(4):
        u = v[t] - S.T @ k[t]
        S = S + torch.outer(k[t], u)
        assert torch.allclose(S.T @ k[t], v[t], atol=1e-12)


def test_routed_feed_forward_weights_the_input():
    g = torch.Generator().manual_seed(4)
    W = {"router": torch.randn(3, 4, generator=g).double()}
    for e in range(3):
        W[f"e{e}.gate"], W[f"e{e}.up"], W[f"e{e}.down"] = (torch.randn(5, 4, generator=g).double(), torch.randn(5, 4, generator=g).double(),
                                                           torch.randn(4, 5, generator=g).double())
    h = torch.randn(2, 4, generator=g).double()
    out, picks = P.routed_ff(h, W, 3, 2)
    s = torch.sigmoid(h @ W["router"].T)
    for t in range(2):
        top = torch.topk(s[t], 2).indices.tolist()
        assert picks[t].tolist() == top
        want = sum(P.gated_ff(s[t, e] * h[t:t + 1], W[f"e{e}.gate"], W[f"e{e}.up"], W[f"e{e}.down"])[0] for e in top)
        assert torch.allclose(out[t], want, atol=1e-12)


def test_command_line_writes_a_random_model_folder(tmp_path):
    import subprocess
    import sys
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(RAW))
    out = tmp_path / "model"
    r = subprocess.run([sys.executable, "-m", "cajeta_llm_b200", "random-weights", "--config", str(cfg), "--seed", "4", "--out", str(out)],
                       cwd=helpers.ROOT, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-1000:]
    config, W = P.read_model(str(out))
    assert config["architecture"] == "Balalorn" and config["layers"] == RAW["layers"] and W["head"].shape == (50, 32)
