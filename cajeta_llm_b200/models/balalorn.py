"""Balalorn: configuration, layer plan and tensor names.

A decoder whose ``config.json`` lists its layers one by one (``layers``: ``type``, ``mixer``
sizes, ``mlp`` or null), so that every layer may have another mixer and another
feed-forward:

* ``type`` ``mamba2`` -> the state-space mixer (part ``ssd``), ``delta`` -> the gated delta
  rule (``gated_delta``), ``latent_attention`` -> attention over a compressed latent
  (``latent_attention``); a latent-attention layer with ``kv_from: j`` owns no cache and
  reads layer j's;
* ``mlp.kind`` ``dense`` -> the gated SiLU feed-forward of ``mlp.ff``; ``moe`` ->
  ``mlp.router.experts`` experts of ``mlp.expert.ff`` of which ``mlp.router.top`` are picked
  by the largest sigmoid scores, the score multiplying the expert's input, not renormalised;
* the block norms each sublayer's OUTPUT (``outnorm``); norms are RMS norms with
  ``norm.eps``.

Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``
(experts ``l<i>.mlp.e<k>.gate|up|down``, router ``l<i>.mlp.router``), ``final.norm``,
``head``.  Every size and constant comes from ``config.json``.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from typing import Any, Dict, Tuple

from ..config.base import ConfigError, ConfigReader, ModelConfig, register_architecture
from ..parts.plan import LayerSpec, ModelPlan, PartSpec, ScheduleEntry

ARCHITECTURE = "Balalorn"
MIXER_TYPES = ("mamba2", "delta", "latent_attention")


@dataclass(frozen=True)
class BalalornConfig(ModelConfig):
    width: int
    vocab: int
    norm_eps: float
    layers_json: str              # the ``layers`` list as canonical JSON (a frozen dataclass holds no dicts)
    eos_token_ids: Tuple[int, ...] = ()

    @property
    def layers(self):
        return json.loads(self.layers_json)

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @classmethod
    def from_reader(cls, r: ConfigReader) -> "BalalornConfig":
        raw = r.raw
        arch = raw["architectures"][0] if "architectures" in raw else raw["architecture"]
        norm = raw.get("norm")
        if not isinstance(norm, dict) or "eps" not in norm:
            raise ConfigError(f"{r.source}: required key 'norm.eps' is missing")
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError(f"{r.source}: required key 'layers' is missing or is not a list of layers")
        for i, layer in enumerate(layers):
            _check_layer(r.source, i, layer, layers)
        eps = float(norm["eps"])
        if eps <= 0.0:
            raise ConfigError(f"{r.source}: norm.eps must be positive, found {eps}")
        return cls(architecture=arch, width=r.integer("width", minimum=1), vocab=r.integer("vocab", minimum=1), norm_eps=eps,
                   layers_json=json.dumps(layers, sort_keys=True), eos_token_ids=tuple(r.integer_list("eos_token_id", ())))

    def to_json_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"architecture": self.architecture, "width": self.width, "vocab": self.vocab,
                             "norm": {"eps": self.norm_eps}, "layers": self.layers}
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d


def _need_ints(source: str, where: str, d: Any, keys) -> None:
    if not isinstance(d, dict):
        raise ConfigError(f"{source}: {where} must be an object")
    for k in keys:
        v = d.get(k)
        if isinstance(v, bool) or not isinstance(v, int) or v < 1:
            raise ConfigError(f"{source}: {where}.{k} must be a positive integer, found {v!r}")


def _check_layer(source: str, i: int, layer: Any, layers) -> None:
    where = f"layers[{i}]"
    if not isinstance(layer, dict) or layer.get("type") not in MIXER_TYPES:
        raise ConfigError(f"{source}: {where}.type must be one of {', '.join(MIXER_TYPES)}, found {layer.get('type') if isinstance(layer, dict) else layer!r}")
    m, kind = layer.get("mixer"), layer["type"]
    if kind == "mamba2":
        _need_ints(source, f"{where}.mixer", m, ("heads", "vdim", "state", "groups", "norm_groups", "conv"))
        if m["heads"] % m["groups"] != 0 or (m["heads"] * m["vdim"]) % m["norm_groups"] != 0:
            raise ConfigError(f"{source}: {where}.mixer: heads must be a multiple of groups and heads * vdim of norm_groups")
    elif kind == "delta":
        _need_ints(source, f"{where}.mixer", m, ("heads", "kv_heads", "dim", "vdim", "conv"))
        if m["heads"] % m["kv_heads"] != 0:
            raise ConfigError(f"{source}: {where}.mixer: heads {m['heads']} is not a multiple of kv_heads {m['kv_heads']}")
    else:
        _need_ints(source, f"{where}.mixer", m, ("heads", "dim", "rot_dim", "vdim", "kv_rank"))
        rot = m.get("rot")
        if not isinstance(rot, dict) or not isinstance(rot.get("dims"), int) or not isinstance(rot.get("base"), (int, float)):
            raise ConfigError(f"{source}: {where}.mixer.rot must give 'base' and 'dims'")
        if rot["dims"] % 2 != 0 or not 0 < rot["dims"] <= m["rot_dim"] or rot["base"] <= 0:
            raise ConfigError(f"{source}: {where}.mixer.rot: dims must be even and within (0, rot_dim], base positive")
        if not isinstance(m.get("scale"), (int, float)) or isinstance(m.get("scale"), bool):
            raise ConfigError(f"{source}: {where}.mixer.scale must be a number")
        src = m.get("kv_from")
        if src is not None:
            if isinstance(src, bool) or not isinstance(src, int) or not 0 <= src < i:
                raise ConfigError(f"{source}: {where}.mixer.kv_from must name an earlier layer, found {src!r}")
            other = layers[src]
            om = other.get("mixer") if isinstance(other, dict) else None
            if other.get("type") != "latent_attention" or om.get("kv_from") is not None:
                raise ConfigError(f"{source}: {where}.mixer.kv_from names layer {src}, which owns no latent cache")
            if (om.get("kv_rank"), om.get("rot_dim"), om.get("rot")) != (m["kv_rank"], m["rot_dim"], rot):
                raise ConfigError(f"{source}: {where}.mixer: kv_rank, rot_dim and rot must equal those of layer {src}")
    ff = layer.get("mlp")
    if ff is None:
        return
    if not isinstance(ff, dict) or ff.get("kind") not in ("dense", "moe"):
        raise ConfigError(f"{source}: {where}.mlp.kind must be 'dense' or 'moe'")
    if ff["kind"] == "dense":
        _need_ints(source, f"{where}.mlp", ff, ("ff",))
    else:
        _need_ints(source, f"{where}.mlp.expert", ff.get("expert"), ("ff",))
        _need_ints(source, f"{where}.mlp.router", ff.get("router"), ("experts", "top"))
        if ff["router"]["top"] > ff["router"]["experts"]:
            raise ConfigError(f"{source}: {where}.mlp.router.top is larger than .experts")


def build_plan(cfg: BalalornConfig) -> ModelPlan:
    h, eps = cfg.width, cfg.norm_eps
    norm = PartSpec("rmsnorm", {"dim": h, "eps": eps, "weight_name": ""})
    block = PartSpec("outnorm", {"mixer_norm_name": "norm1", "feed_forward_norm_name": "norm2", "mixer_name": "mix",
                                 "feed_forward_name": "mlp"})
    layers, schedule = [], []
    for i, layer in enumerate(cfg.layers):
        m, kind = layer["mixer"], layer["type"]
        cache_from = None
        if kind == "mamba2":
            mixer = PartSpec("ssd", {"hidden_size": h, "heads": m["heads"], "vdim": m["vdim"], "state": m["state"],
                                     "groups": m["groups"], "norm_groups": m["norm_groups"], "conv": m["conv"], "eps": eps})
        elif kind == "delta":
            mixer = PartSpec("gated_delta", {"hidden_size": h, "heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"],
                                             "vdim": m["vdim"], "conv": m["conv"], "eps": eps})
        else:
            cache_from = m.get("kv_from")
            position = PartSpec("rope", {"head_dim": m["rot_dim"], "rotary_dim": m["rot"]["dims"], "theta": float(m["rot"]["base"])})
            mixer = PartSpec("latent_attention", {"hidden_size": h, "heads": m["heads"], "dim": m["dim"], "rot_dim": m["rot_dim"],
                                                  "vdim": m["vdim"], "kv_rank": m["kv_rank"], "scale": float(m["scale"]), "eps": eps,
                                                  "position": position, "owns_cache": cache_from is None})
        ff = layer.get("mlp")
        if ff is None:
            ffn = None
        elif ff["kind"] == "dense":
            ffn = PartSpec("dense_swiglu", {"hidden_size": h, "intermediate_size": ff["ff"],
                                            "names": {"gate": "gate", "up": "up", "down": "down"}})
        else:
            ffn = PartSpec("sparse_moe", {"hidden_size": h, "num_experts": ff["router"]["experts"], "top_k": ff["router"]["top"],
                                          "expert_intermediate_size": ff["expert"]["ff"], "norm_topk_prob": False,
                                          "score": "sigmoid", "weight_on": "input",
                                          "names": {"router": "router", "gate": "e{e}.gate", "up": "e{e}.up", "down": "e{e}.down"}})
        layers.append(LayerSpec(prefix=f"l{i}", block=block, mixer=mixer, feed_forward=ffn, mixer_norm=norm,
                                feed_forward_norm=norm if ffn is not None else None))
        # the schedule runs the layers in order, so a layer's index is its schedule entry's
        schedule.append(ScheduleEntry(layer=i, cache_from=cache_from))
    plan = ModelPlan(architecture=cfg.architecture, hidden_size=h, vocab_size=cfg.vocab, embedding_name="embed",
                     layers=tuple(layers), schedule=tuple(schedule), final_norm=norm, final_norm_prefix="final.norm",
                     lm_head_name="head", eog_token_ids=cfg.eos_token_ids, max_position=None)
    plan.validate()
    return plan


register_architecture(ARCHITECTURE, BalalornConfig, build_plan, replace=True)
