"""Saropel on the host: configuration and plan, tensor names, the random-weights folder, and the
plain implementation's own mechanisms against independent closed forms."""
import copy
import json
import math

import numpy as np
import pytest

import helpers
import plain_saropel as P

RAW = {"architecture": "Saropel", "width": 32, "vocab": 50, "norm": {"eps": 1e-6},
       "embedding": {"bigram": {"buckets": 11, "mul_prev": 3, "mul_cur": 5}}, "token_side": {"dim": 4},
       "loop": {"start": 1, "stop": 3, "times": 3},
       "layers": [
           {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 6, "scale": 0.3, "softcap": 9.0, "mask": {"size": 7}},
            "mlp": {"kind": "dense", "ff": 20}},
           {"type": "attention_2", "mixer": {"heads": 3, "kv_heads": 1, "dim": 10, "vdim": 10, "scale": 0.5, "mask": {"size": 12},
                                             "rot": {"base": 100.0, "dims": 6, "scaling": {"factor": 2.0, "original": 8, "fast": 4.0, "slow": 1.0}}},
            "mlp": {"kind": "moe", "expert": {"ff": 12, "limit": 2.5}, "router": {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 2}},
                    "shared": {"ff": 14, "limit": 1.5}}},
           {"type": "attention", "mixer": {"heads": 2, "kv_heads": 2, "dim": 4, "vdim": 4, "scale": 0.4}, "mlp": None},
           {"type": "attention_2", "mixer": {"heads": 2, "kv_heads": 2, "dim": 6, "vdim": 6, "scale": 0.4, "mask": {"size": 3}},
            "mlp": {"kind": "moe", "expert": {"ff": 8, "limit": 1.0}, "router": {"experts": 3, "top": 3}}},
       ]}


def plan_of(raw):
    import cajeta_llm_b200  # noqa: F401
    from cajeta_llm_b200.config import parse_config_dict
    from cajeta_llm_b200.config.base import get_architecture
    cfg = parse_config_dict(raw)
    return cfg, get_architecture(cfg.architecture).build_plan(cfg)


def test_the_plan_follows_the_list_of_layers_and_the_loop():
    cfg, plan = plan_of(RAW)
    assert [l.mixer.kind for l in plan.layers] == ["attention"] * 4 and [l.block.kind for l in plan.layers] == ["parallel"] * 4
    assert [None if l.feed_forward is None else l.feed_forward.kind for l in plan.layers] == ["dense_swiglu", "sparse_moe", None, "sparse_moe"]
    # layers 1 and 2 three times in a row, each run an entry (and so a cache plane) of its own, then layer 3
    assert [e.layer for e in plan.schedule] == [0, 1, 2, 1, 2, 1, 2, 3]
    starts = [(i, e.before["row"], e.before["add_embedding"]) for i, e in enumerate(plan.schedule) if e.before is not None]
    assert starts == [(1, 0, False), (3, 1, True), (5, 2, True)]
    a, b = plan.layers[0].mixer, plan.layers[1].mixer
    assert a["softcap"] == 9.0 and a["window"] == 7 and a["value_dim"] == 6 and a["position"].kind == "none" and not a.get("values_from_keys")
    assert b["values_from_keys"] and b["head_gate"] == "g" and b["qk_norm"]["eps"] == 1e-6 and b["position"]["rotary_dim"] == 6
    assert plan.layers[2].mixer["window"] == 0 and plan.layers[2].mixer["softcap"] == 0.0
    ff = plan.layers[1].feed_forward
    assert ff["route_groups"] == (3, 2) and ff["act_limit"] == 2.5 and ff["shared_act_limit"] == 1.5 and ff["act_alpha"] == 1.702
    assert plan.layers[3].feed_forward["route_groups"] is None and plan.layers[3].feed_forward["shared_intermediate_size"] == 0
    assert plan.layers[2].stream_after["offset"] == 8 and plan.embedding.kind == "pair_hash_embedding"
    assert cfg.to_json_dict() == RAW


def test_a_model_without_the_optional_pieces():
    raw = {k: v for k, v in RAW.items() if k not in ("embedding", "token_side", "loop")}
    cfg, plan = plan_of(raw)
    assert plan.embedding.kind == "token_embedding" and [e.layer for e in plan.schedule] == [0, 1, 2, 3]
    assert all(e.before is None for e in plan.schedule) and all(l.stream_after is None for l in plan.layers)


def test_tensor_names_shapes_and_needs():
    from cajeta_llm_b200.engine.model import build_model
    from cajeta_llm_b200.parts.base import Runtime
    cfg, _ = plan_of(RAW)
    model = build_model(cfg, Runtime("float32", "cpu"))
    p = {n: tuple(s.shape) for n, s in model.params().items()}
    assert p["embed"] == (50, 32) and p["bigram"] == (12, 32) and p["loop.step"] == (3, 32) and p["side.embed"] == (50, 16)
    assert p["head"] == (50, 32) and p["final.norm"] == (32,) and p["l0.norm1"] == (32,) and "l0.norm2" not in p
    assert p["l0.mix.q"] == (32, 32) and p["l0.mix.k"] == (16, 32) and p["l0.mix.v"] == (12, 32) and p["l0.mix.o"] == (32, 24)
    assert p["l1.mix.q"] == (30, 32) and p["l1.mix.k"] == (10, 32) and "l1.mix.v" not in p and p["l1.mix.g"] == (3, 32)
    assert p["l1.mix.q.norm"] == (10,) and p["l1.mix.k.norm"] == (10,) and p["l1.mix.o"] == (32, 30) and "l0.mix.g" not in p
    assert p["l1.mlp.router"] == (6, 32) and p["l1.mlp.e5.gate"] == (12, 32) and p["l1.mlp.e0.down"] == (32, 12)
    assert p["l1.mlp.shared.up"] == (14, 32) and p["l1.mlp.shared.sg"] == (1, 32) and "l3.mlp.shared.sg" not in p
    assert p["l0.mlp.up"] == (20, 32) and not any(n.startswith("l2.mlp") for n in p)
    assert p["l2.side.gate"] == (4, 32) and p["l2.side.proj"] == (32, 4) and p["l2.side.norm"] == (32,)
    needs = model.kv_needs()
    assert len(needs) == 8 and (needs[0].head_dim, needs[0].value_dim, needs[0].window) == (8, 6, 7)
    assert (needs[1].head_dim, needs[1].value_dim, needs[1].window, needs[1].kv_heads) == (10, 0, 12, 1) and needs[2].window == 0
    assert model.state_needs() == [None] * 8 and model.named_state_needs()["embedding"].shape == (1,)
    assert model.keeps_embedding_output


def test_cache_planes_of_a_looped_layer_are_its_own():
    from cajeta_llm_b200.cache.manager import CacheManager
    from cajeta_llm_b200.engine.model import build_model
    from cajeta_llm_b200.parts.base import Runtime
    import torch
    cfg, _ = plan_of(RAW)
    model = build_model(cfg, Runtime("float32", "cpu"))
    m = CacheManager(model.kv_needs(), model.state_needs(), model.cache_from(), 4, 2, 32, 8, torch.float32, None,
                     named_state_needs=model.named_state_needs())
    # the three runs of layer 1 share a group (one page table) and own planes 0, 1, 2 of it
    assert len({m.entry_group[i] for i in (1, 3, 5)}) == 1 and [m.entry_plane[i] for i in (1, 3, 5)] == [0, 1, 2]
    assert m.entry_group[0] != m.entry_group[1] and m.num_groups == 4


@pytest.mark.parametrize("change, message", [
    (lambda c: c["layers"][0].update(type="mamba2"), "type"),
    (lambda c: c["layers"][0]["mixer"].update(heads=3), "multiple"),
    (lambda c: c["layers"][1]["mixer"].update(vdim=8), "vdim must equal dim"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=5), "dims"),
    (lambda c: c["layers"][1]["mixer"]["rot"]["scaling"].pop("fast"), "scaling.fast"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=7), "top"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=4), "equal groups"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(keep=1, count=6), "fewer than 'top'"),
    (lambda c: c["layers"][1]["mlp"]["expert"].pop("limit"), "limit"),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda c: c["loop"].update(stop=5), "loop"),
    (lambda c: c["embedding"]["bigram"].update(buckets=0), "buckets"),
    (lambda c: c.pop("norm"), "norm.eps"),
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
    assert cfg == RAW and W["l1.mix.q.norm"].shape == (10,) and W["bigram"].shape == (12, 32)
    logits, after = P.forward(cfg, W, [1, 2, 3, 4, 5], keep_layers=True)
    assert logits.shape == (5, 50) and after.shape == (8, 5, 32) and bool(np.isfinite(logits).all())


def test_the_engine_s_frequency_table_equals_the_plain_one():
    from cajeta_llm_b200.parts.base import Runtime, make_part
    from cajeta_llm_b200.parts.plan import PartSpec
    for rot in ({"base": 100.0, "dims": 6, "scaling": {"factor": 2.0, "original": 8, "fast": 4.0, "slow": 1.0}},
                {"base": 50000.0, "dims": 48, "scaling": {"factor": 8.0, "original": 300, "fast": 32.0, "slow": 0.5}},
                {"base": 10000.0, "dims": 16}):
        part = make_part("position", PartSpec("rope", {"head_dim": 64, "rotary_dim": rot["dims"], "theta": rot["base"],
                                                       "scaling": rot.get("scaling")}), "", Runtime("float32", "cpu"))
        cos, sin = P.rotary_tables(rot, np.array([1]))
        mag = 0.1 * math.log(rot["scaling"]["factor"]) + 1.0 if "scaling" in rot else 1.0
        assert abs(part.magnitude - mag) < 1e-12
        ang = part.inv_freq.double().numpy()
        assert np.allclose(np.cos(ang) * mag, cos[0], atol=1e-6) and np.allclose(np.sin(ang) * mag, sin[0], atol=1e-6)


# -- the plain implementation's mechanisms against closed forms of their own --------------
def test_rotation_keeps_relative_angles_and_scales_lengths():
    g = np.random.default_rng(1)
    rot = {"base": 100.0, "dims": 4, "scaling": {"factor": 2.0, "original": 8, "fast": 4.0, "slow": 1.0}}
    q, k = g.standard_normal((1, 6)), g.standard_normal((1, 6))

    def at(v, p):
        cos, sin = P.rotary_tables(rot, np.array([p]))
        return P.rotate(v, cos[0], sin[0], 4)

    a = (at(q, 7)[0, :4] * at(k, 3)[0, :4]).sum()
    b = (at(q, 14)[0, :4] * at(k, 10)[0, :4]).sum()
    assert abs(a - b) < 1e-12
    mag = 0.1 * math.log(2.0) + 1.0
    r = at(q, 5)
    assert np.allclose(r[0, 4:], q[0, 4:]) and abs(np.linalg.norm(r[0, :4]) - mag * np.linalg.norm(q[0, :4])) < 1e-12
    # entry 0 is paired with entry 2 (not 1) and turns by p * f_0
    plain = {"base": 100.0, "dims": 4}
    cos, sin = P.rotary_tables(plain, np.array([2]))
    e = P.rotate(np.array([[1.0, 0.0, 0.0, 0.0]]), cos[0], sin[0], 4)
    assert np.allclose(e[0], [math.cos(2.0), 0.0, math.sin(2.0), 0.0])


def test_router_groups_limit_the_choice():
    z = np.log(np.array([0.30, 0.02, 0.05, 0.25, 0.20, 0.18]))      # groups (0,1) (2,3) (4,5): best scores .30 .25 .20
    s, picks = P.route(z, 3, {"count": 3, "keep": 2})
    assert picks == [0, 3, 2] and abs(s.sum() - 1.0) < 1e-12          # 4 and 5 beat 2 but their group is out
    assert P.route(z, 3, None)[1] == [0, 3, 4] and P.route(z, 2, {"count": 3, "keep": 1})[1] == [0, 1]
    assert P.route(z, 3, {"count": 1, "keep": 1})[1] == [0, 3, 4]


def test_capped_expert_and_pair_rows():
    W = {"e.gate": np.array([[1.0], [1.0]]), "e.up": np.array([[1.0], [-1.0]]), "e.down": np.eye(2)}
    y = P.capped_expert(W, "e.", np.array([[10.0]]), 2.0)[0]         # gate 10 -> 2; up 10 -> 2 and -10 -> -2
    g = 2.0 / (1.0 + math.exp(-1.702 * 2.0))
    assert np.allclose(y, [g * 3.0, g * -1.0])
    y = P.capped_expert(W, "e.", np.array([[-10.0]]), 2.0)[0]        # the gate is capped from above only
    g = -10.0 / (1.0 + math.exp(17.02))
    assert np.allclose(y, [g * -1.0, g * 3.0])
    cfg = {"embedding": {"bigram": {"buckets": 5, "mul_prev": 3, "mul_cur": 2}}}
    Wt = {"embed": np.zeros((9, 6)), "bigram": np.arange(6)[:, None] * np.ones((1, 6))}
    rows = P.embed_rows(cfg, Wt, [4, 1, 8])[:, 0]
    assert rows.tolist() == [5.0, (4 * 3 + 1 * 2) % 5, (1 * 3 + 8 * 2) % 5]


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
    assert config == RAW and W["head"].shape == (50, 32)
