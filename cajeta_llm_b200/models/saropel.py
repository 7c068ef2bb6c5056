"""Saropel: configuration, layer plan and tensor names.

A decoder whose ``config.json`` lists its layers one by one (``layers``: ``type``, ``mixer`` sizes,
``mlp`` or null).  What it is put together from:

* the embedding adds a row of a second table chosen by a hash of (previous token, token)
  (``embedding.bigram``: ``buckets``, ``mul_prev``, ``mul_cur``; part ``pair_hash_embedding``);
* a layer is a ``parallel`` block: one norm (``1 + w`` weight), mixer and feed-forward both read
  it, their sum is added; then, with ``token_side``, a per-layer input chosen by the token
  (part ``token_side``);
* ``type`` ``attention``: grouped-query attention without rotation, scores capped by
  ``softcap * tanh(s / softcap)``, a sliding window of ``mask.size``; ``attention_2``: the values
  are the keys as projected, q and k are RMS-normed per head, rotated over their first
  ``rot.dims`` entries (entry i with i + dims/2; ``rot.scaling`` stretches the slow frequencies),
  windowed, and every head's output passes a sigmoid gate of its own.  Both are the engine's
  ``attention`` mixer with other parameters;
* ``mlp.kind`` ``dense``: the gated SiLU feed-forward; ``moe``: experts of the capped form
  (``limit``), softmax scores, the ``top`` largest picked among the experts of the ``groups.keep``
  best of ``groups.count`` groups, weights not renormalised, plus a shared expert behind a sigmoid
  gate;
* ``loop``: layers ``start .. stop-1`` run ``times`` times with the same weights, each pass with a
  cache of its own (the plan's schedule names those layers once per pass); before every pass the
  vector ``loop.step[t]`` is added to the stream, and before every pass but the first the
  embedding's output too (part ``pass_start``).

Tensor names: ``embed``, ``bigram``, ``loop.step``, ``side.embed``, ``l<i>.norm1``, ``l<i>.mix.q|k|v|o|g``,
``l<i>.mix.q.norm|k.norm``, ``l<i>.mlp.gate|up|down``, ``l<i>.mlp.e<k>.gate|up|down``, ``l<i>.mlp.router``,
``l<i>.mlp.shared.gate|up|down|sg``, ``l<i>.side.gate|proj|norm``, ``final.norm``, ``head``.  Every size and
every constant that can differ between models comes from ``config.json``.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from typing import Any, Dict, Tuple

from ..config.base import ConfigError, ConfigReader, ModelConfig, register_architecture
from ..parts.plan import LayerSpec, ModelPlan, PartSpec, ScheduleEntry

ARCHITECTURE = "Saropel"
MIXER_TYPES = ("attention", "attention_2")
EXPERT_GATE_SLOPE = 1.702          # the capped expert's gate is g * sigmoid(1.702 g)


@dataclass(frozen=True)
class SaropelConfig(ModelConfig):
    width: int
    vocab: int
    norm_eps: float
    layers_json: str              # ``layers`` as canonical JSON (a frozen dataclass holds no dicts)
    extras_json: str              # ``embedding``, ``loop`` and ``token_side`` as canonical JSON
    eos_token_ids: Tuple[int, ...] = ()

    @property
    def layers(self):
        return json.loads(self.layers_json)

    @property
    def extras(self) -> Dict[str, Any]:
        return json.loads(self.extras_json)

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @classmethod
    def from_reader(cls, r: ConfigReader) -> "SaropelConfig":
        raw = r.raw
        arch = raw["architectures"][0] if "architectures" in raw else raw["architecture"]
        norm = raw.get("norm")
        if not isinstance(norm, dict) or "eps" not in norm:
            raise ConfigError(f"{r.source}: required key 'norm.eps' is missing")
        eps = float(norm["eps"])
        if eps <= 0.0:
            raise ConfigError(f"{r.source}: norm.eps must be positive, found {eps}")
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError(f"{r.source}: required key 'layers' is missing or is not a list of layers")
        for i, layer in enumerate(layers):
            _check_layer(r.source, i, layer)
        extras = {}
        bigram = (raw.get("embedding") or {}).get("bigram")
        if bigram is not None:
            _need_ints(r.source, "embedding.bigram", bigram, ("buckets",))
            _need_ints(r.source, "embedding.bigram", bigram, ("mul_prev", "mul_cur"), minimum=0)
            extras["embedding"] = {"bigram": bigram}
        loop = raw.get("loop")
        if loop is not None:
            _need_ints(r.source, "loop", loop, ("times",))
            _need_ints(r.source, "loop", loop, ("start", "stop"), minimum=0)
            if not loop["start"] < loop["stop"] <= len(layers):
                raise ConfigError(f"{r.source}: loop must name layers start < stop <= {len(layers)}, found {loop['start']} .. {loop['stop']}")
            extras["loop"] = loop
        side = raw.get("token_side")
        if side is not None:
            _need_ints(r.source, "token_side", side, ("dim",))
            extras["token_side"] = side
        return cls(architecture=arch, width=r.integer("width", minimum=1), vocab=r.integer("vocab", minimum=1), norm_eps=eps,
                   layers_json=json.dumps(layers, sort_keys=True), extras_json=json.dumps(extras, sort_keys=True),
                   eos_token_ids=tuple(r.integer_list("eos_token_id", ())))

    def to_json_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"architecture": self.architecture, "width": self.width, "vocab": self.vocab,
                             "norm": {"eps": self.norm_eps}, "layers": self.layers}
        d.update(self.extras)
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d


def _need_ints(source: str, where: str, d: Any, keys, minimum: int = 1) -> None:
    if not isinstance(d, dict):
        raise ConfigError(f"{source}: {where} must be an object")
    for k in keys:
        v = d.get(k)
        if isinstance(v, bool) or not isinstance(v, int) or v < minimum:
            raise ConfigError(f"{source}: {where}.{k} must be an integer >= {minimum}, found {v!r}")


def _number(source: str, where: str, v: Any, positive: bool = True) -> float:
    if isinstance(v, bool) or not isinstance(v, (int, float)) or (positive and v <= 0):
        raise ConfigError(f"{source}: {where} must be a{' positive' if positive else ''} number, found {v!r}")
    return float(v)


def _check_expert(source: str, where: str, e: Any) -> None:
    _need_ints(source, where, e, ("ff",))
    _number(source, f"{where}.limit", e.get("limit"))


def _check_layer(source: str, i: int, layer: Any) -> None:
    where = f"layers[{i}]"
    if not isinstance(layer, dict) or layer.get("type") not in MIXER_TYPES:
        raise ConfigError(f"{source}: {where}.type must be one of {', '.join(MIXER_TYPES)}, "
                          f"found {layer.get('type') if isinstance(layer, dict) else layer!r}")
    m, kind = layer.get("mixer"), layer["type"]
    _need_ints(source, f"{where}.mixer", m, ("heads", "kv_heads", "dim", "vdim"))
    if m["heads"] % m["kv_heads"] != 0:
        raise ConfigError(f"{source}: {where}.mixer: heads {m['heads']} is not a multiple of kv_heads {m['kv_heads']}")
    _number(source, f"{where}.mixer.scale", m.get("scale"))
    if m.get("mask") is not None:
        _need_ints(source, f"{where}.mixer.mask", m["mask"], ("size",))
    if kind == "attention":
        if m.get("softcap") is not None:
            _number(source, f"{where}.mixer.softcap", m["softcap"])
    else:
        if m["vdim"] != m["dim"]:
            raise ConfigError(f"{source}: {where}.mixer: the values are the keys, so vdim must equal dim")
        rot = m.get("rot")
        if rot is not None:
            _need_ints(source, f"{where}.mixer.rot", rot, ("dims",))
            if rot["dims"] % 2 != 0 or rot["dims"] > m["dim"] or _number(source, f"{where}.mixer.rot.base", rot.get("base")) <= 1.0:
                raise ConfigError(f"{source}: {where}.mixer.rot: dims must be even and at most dim, base larger than 1")
            sc = rot.get("scaling")
            if sc is not None:
                if not isinstance(sc, dict):
                    raise ConfigError(f"{source}: {where}.mixer.rot.scaling must be an object")
                for k in ("factor", "original", "fast", "slow"):
                    _number(source, f"{where}.mixer.rot.scaling.{k}", sc.get(k))
    ff = layer.get("mlp")
    if ff is None:
        return
    if not isinstance(ff, dict) or ff.get("kind") not in ("dense", "moe"):
        raise ConfigError(f"{source}: {where}.mlp.kind must be 'dense' or 'moe'")
    if ff["kind"] == "dense":
        _need_ints(source, f"{where}.mlp", ff, ("ff",))
        return
    _check_expert(source, f"{where}.mlp.expert", ff.get("expert"))
    router = ff.get("router")
    _need_ints(source, f"{where}.mlp.router", router, ("experts", "top"))
    if router["top"] > router["experts"]:
        raise ConfigError(f"{source}: {where}.mlp.router.top is larger than .experts")
    groups = router.get("groups")
    if groups is not None:
        _need_ints(source, f"{where}.mlp.router.groups", groups, ("count", "keep"))
        if router["experts"] % groups["count"] != 0 or groups["keep"] > groups["count"]:
            raise ConfigError(f"{source}: {where}.mlp.router.groups: experts must form 'count' equal groups and keep <= count")
        if groups["keep"] * (router["experts"] // groups["count"]) < router["top"]:
            raise ConfigError(f"{source}: {where}.mlp.router.groups: the kept groups hold fewer than 'top' experts")
    if ff.get("shared") is not None:
        _check_expert(source, f"{where}.mlp.shared", ff["shared"])


def _mixer_spec(h: int, eps: float, kind: str, m: Dict[str, Any]) -> PartSpec:
    params: Dict[str, Any] = {"hidden_size": h, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
                              "value_dim": m["vdim"], "window": (m.get("mask") or {}).get("size", 0), "scale": float(m["scale"]),
                              "names": {"q": "q", "k": "k", "v": "v", "o": "o"}, "position": PartSpec("none")}
    if kind == "attention":
        params["softcap"] = float(m.get("softcap") or 0.0)
        return PartSpec("attention", params)
    params.update(values_from_keys=True, head_gate="g", qk_norm={"q": "q.norm", "k": "k.norm", "eps": eps})
    rot = m.get("rot")
    if rot is not None:
        params["position"] = PartSpec("rope", {"head_dim": m["dim"], "rotary_dim": rot["dims"], "theta": float(rot["base"]),
                                               "scaling": rot.get("scaling")})
    return PartSpec("attention", params)


def _feed_forward_spec(h: int, ff: Any):
    if ff is None:
        return None
    if ff["kind"] == "dense":
        return PartSpec("dense_swiglu", {"hidden_size": h, "intermediate_size": ff["ff"],
                                         "names": {"gate": "gate", "up": "up", "down": "down"}})
    router, shared = ff["router"], ff.get("shared")
    groups = router.get("groups")
    return PartSpec("sparse_moe", {
        "hidden_size": h, "num_experts": router["experts"], "top_k": router["top"], "expert_intermediate_size": ff["expert"]["ff"],
        "norm_topk_prob": False, "score": "softmax", "weight_on": "output",
        "act_limit": float(ff["expert"]["limit"]), "act_alpha": EXPERT_GATE_SLOPE,
        "shared_intermediate_size": shared["ff"] if shared else 0, "shared_gate": bool(shared),
        "shared_act_limit": float(shared["limit"]) if shared else 0.0, "shared_act_alpha": EXPERT_GATE_SLOPE,
        "route_groups": (groups["count"], groups["keep"]) if groups else None,
        "names": {"router": "router", "gate": "e{e}.gate", "up": "e{e}.up", "down": "e{e}.down",
                  "shared_gate": "shared.gate", "shared_up": "shared.up", "shared_down": "shared.down", "shared_sg": "shared.sg"}})


def build_plan(cfg: SaropelConfig) -> ModelPlan:
    h, eps, extras = cfg.width, cfg.norm_eps, cfg.extras
    raw_layers = cfg.layers
    norm = PartSpec("rmsnorm", {"dim": h, "eps": eps, "weight_name": "", "offset": 1.0})
    block = PartSpec("parallel", {"mixer_norm_name": "norm1", "mixer_name": "mix", "feed_forward_name": "mlp",
                                  "stream_after_name": "side"})
    side = extras.get("token_side")
    layers = []
    for i, layer in enumerate(raw_layers):
        after = None
        if side:
            after = PartSpec("token_side", {"hidden_size": h, "dim": side["dim"], "offset": i * side["dim"], "eps": eps,
                                            "table_name": "side.embed", "table_shape": (cfg.vocab, len(raw_layers) * side["dim"])})
        layers.append(LayerSpec(prefix=f"l{i}", block=block, mixer=_mixer_spec(h, eps, layer["type"], layer["mixer"]),
                                feed_forward=_feed_forward_spec(h, layer.get("mlp")), mixer_norm=norm, feed_forward_norm=None,
                                stream_after=after))
    # the run order: a looped stretch of layers appears once per pass, each appearance with a cache
    # plane of its own; a pass begins with the stream step that adds the pass's vector (and, from the
    # second pass on, the embedding's output)
    loop = extras.get("loop")
    schedule = []
    if loop:
        schedule += [ScheduleEntry(layer=i) for i in range(loop["start"])]
        for t in range(loop["times"]):
            for i in range(loop["start"], loop["stop"]):
                before = None
                if i == loop["start"]:
                    before = PartSpec("pass_start", {"hidden_size": h, "table_name": "loop.step", "rows": loop["times"], "row": t,
                                                     "add_embedding": t > 0})
                schedule.append(ScheduleEntry(layer=i, before=before))
        schedule += [ScheduleEntry(layer=i) for i in range(loop["stop"], len(raw_layers))]
    else:
        schedule = [ScheduleEntry(layer=i) for i in range(len(raw_layers))]
    bigram = (extras.get("embedding") or {}).get("bigram")
    embedding = PartSpec("token_embedding")
    if bigram:
        embedding = PartSpec("pair_hash_embedding", {"buckets": bigram["buckets"], "mul_prev": bigram["mul_prev"],
                                                     "mul_cur": bigram["mul_cur"], "pair_name": "bigram"})
    plan = ModelPlan(architecture=cfg.architecture, hidden_size=h, vocab_size=cfg.vocab, embedding_name="embed",
                     layers=tuple(layers), schedule=tuple(schedule), final_norm=norm, final_norm_prefix="final.norm",
                     lm_head_name="head", eog_token_ids=cfg.eos_token_ids, max_position=None, embedding=embedding)
    plan.validate()
    return plan


register_architecture(ARCHITECTURE, SaropelConfig, build_plan, replace=True)
