"""Typed configuration of the Mefepel decoder: learned positions, layers listed one by one, norms before and after
every sublayer, latent attention with a sink per head, and per layer a dense clamped-gate feed-forward, a mixture of
small experts, or none.

config.json (every size and every constant that differs between models of the design is read from it):
  architecture      "Mefepel"
  vocab, width, max_positions
  norm.eps          eps of every RMS norm, the latents' included
  layers[i].type    the mixer's kind; "latent_attention" is the one there is
  layers[i].mixer   heads, dim, vdim, kv_rank, q_rank, scale
  layers[i].mlp     null | {kind: "dense", ff, limit} | {kind: "moe", expert: {ff}, router: {experts, top}}
What the design fixes stands here as constants: the dense gate's sigmoid slope, the router's sigmoid scores that are
not renormalised and multiply the expert's input.

Tensor names: embed, pos, l<i>.norm1 / norm1b (before / after the mixer), l<i>.norm2 / norm2b (feed-forward),
l<i>.mix.{dq, dq.norm, uq, dkv, dkv.norm, uk, uv, sink, o}, l<i>.mlp.{gate, up, down} or
l<i>.mlp.router and l<i>.mlp.e<j>.{gate, up, down}, final.norm, head.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Mapping

from .registry import ModelConfig, register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

DENSE_GATE_SLOPE = 1.702   # g * sigmoid(1.702 g): the sigmoid approximation of GELU as the gate


def _need(data: Mapping[str, Any], key: str, where: str = "config.json"):
    if not isinstance(data, Mapping) or key not in data or data[key] is None:
        raise ValueError(f"{where}: required key {key!r} is missing")
    return data[key]


@dataclass(frozen=True)
class MefepelConfig(ModelConfig):
    vocab: int
    width: int
    max_positions: int
    eps: float
    layers: tuple          # the config's own layer entries (plain dicts), validated
    torch_dtype: str = "bfloat16"

    architecture = "Mefepel"
    model_type = "mefepel"

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "MefepelConfig":
        layers = _need(data, "layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ValueError("config.json: 'layers' must be a non-empty list")
        config = cls(vocab=int(_need(data, "vocab")), width=int(_need(data, "width")),
                     max_positions=int(_need(data, "max_positions")), eps=float(_need(_need(data, "norm"), "eps", "config.json norm")),
                     layers=tuple(copy.deepcopy(dict(layer)) for layer in layers),
                     torch_dtype=str(data.get("torch_dtype", data.get("dtype", "bfloat16"))))
        config.validate()
        return config

    def validate(self) -> None:
        for key in ("vocab", "width", "max_positions"):
            if getattr(self, key) <= 0:
                raise ValueError(f"config.json: {key} must be positive, got {getattr(self, key)}")
        if self.eps <= 0:
            raise ValueError("config.json: norm.eps must be positive")
        for i, layer in enumerate(self.layers):
            where = f"config.json layers[{i}]"
            kind = _need(layer, "type", where)
            if kind != "latent_attention":
                raise ValueError(f"{where}: mixer type {kind!r} is not supported (only 'latent_attention')")
            mixer = _need(layer, "mixer", where)
            for key in ("heads", "dim", "vdim", "kv_rank", "q_rank"):
                if int(_need(mixer, key, where + ".mixer")) <= 0:
                    raise ValueError(f"{where}.mixer: {key} must be positive")
            if float(_need(mixer, "scale", where + ".mixer")) <= 0:
                raise ValueError(f"{where}.mixer: scale must be positive")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            kind = _need(mlp, "kind", where + ".mlp")
            if kind == "dense":
                if int(_need(mlp, "ff", where + ".mlp")) <= 0 or float(_need(mlp, "limit", where + ".mlp")) <= 0:
                    raise ValueError(f"{where}.mlp: ff and limit must be positive")
            elif kind == "moe":
                router = _need(mlp, "router", where + ".mlp")
                experts, top = int(_need(router, "experts", where + ".mlp.router")), int(_need(router, "top", where + ".mlp.router"))
                if int(_need(_need(mlp, "expert", where + ".mlp"), "ff", where + ".mlp.expert")) <= 0 or not 1 <= top <= experts:
                    raise ValueError(f"{where}.mlp: expert.ff must be positive and 1 <= router.top <= router.experts")
            else:
                raise ValueError(f"{where}.mlp: kind {kind!r} is not supported ('dense', 'moe' or null)")

    def to_dict(self) -> dict:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "max_positions": self.max_positions, "norm": {"eps": self.eps},
                "layers": [copy.deepcopy(layer) for layer in self.layers], "torch_dtype": self.torch_dtype}

    def model_spec(self) -> ModelSpec:
        def norm(name: str) -> PartSpec:
            return PartSpec("rms_norm", {"width": self.width, "eps": self.eps}, {"weight": name})

        layers, ignored = [], []
        for i, layer in enumerate(self.layers):
            p, m = f"l{i}.", layer["mixer"]
            mixer = PartSpec(
                "latent_attention",
                {"hidden_size": self.width, "num_heads": int(m["heads"]), "head_dim": int(m["dim"]), "value_dim": int(m["vdim"]),
                 "kv_rank": int(m["kv_rank"]), "q_rank": int(m["q_rank"]), "scale": float(m["scale"]), "eps": self.eps,
                 "sinks": True, "window": 0},
                {"q_down": p + "mix.dq", "q_norm": p + "mix.dq.norm", "q_up": p + "mix.uq", "kv_down": p + "mix.dkv",
                 "kv_norm": p + "mix.dkv.norm", "k_up": p + "mix.uk", "v_up": p + "mix.uv", "sink": p + "mix.sink",
                 "o_weight": p + "mix.o"})
            parts = {"mixer_norm": norm(p + "norm1"), "mixer": mixer, "mixer_post_norm": norm(p + "norm1b")}
            mlp = layer.get("mlp")
            if mlp is None:
                ignored += [p + "norm2", p + "norm2b"]   # a file may still carry them
            else:
                parts["feed_forward_norm"] = norm(p + "norm2")
                parts["feed_forward_post_norm"] = norm(p + "norm2b")
                if mlp["kind"] == "dense":
                    parts["feed_forward"] = PartSpec(
                        "clamped_glu",
                        {"hidden_size": self.width, "intermediate_size": int(mlp["ff"]), "limit": float(mlp["limit"]),
                         "alpha": DENSE_GATE_SLOPE},
                        {"gate_weight": p + "mlp.gate", "up_weight": p + "mlp.up", "down_weight": p + "mlp.down"})
                else:
                    experts = int(mlp["router"]["experts"])
                    tensors = {"router": p + "mlp.router"}
                    for e in range(experts):
                        for which in ("gate", "up", "down"):
                            tensors[f"{which}.{e}"] = f"{p}mlp.e{e}.{which}"
                    parts["feed_forward"] = PartSpec(
                        "routed_experts",
                        {"hidden_size": self.width, "expert_size": int(mlp["expert"]["ff"]), "experts": experts,
                         "top": int(mlp["router"]["top"]), "score": "sigmoid", "renormalize": False, "weight_on": "input"},
                        tensors)
            layers.append(LayerSpec("sandwich_norm", parts))
        spec = ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=self.width, max_positions=self.max_positions,
            embedding=PartSpec("token_position_embedding",
                               {"vocab_size": self.vocab, "width": self.width, "max_positions": self.max_positions},
                               {"weight": "embed", "positions": "pos"}),
            layers=tuple(layers), schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
            final_norm=norm("final.norm"),
            head=PartSpec("linear_head", {"vocab_size": self.vocab, "width": self.width, "tied": False}, {"weight": "head"}),
            ignored_tensors=tuple(ignored))
        spec.validate()
        return spec


register_architecture(MefepelConfig.architecture, MefepelConfig, MefepelConfig.model_type)
