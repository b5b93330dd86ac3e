"""Typed configuration of the Zebovik decoder: layers listed one by one, each a mixer (attention in blocks with capped
scores and a unit sink, an mLSTM matrix memory, or a Mamba-2 state space) and an optional dense feed-forward, with RMS
norms before and after every sublayer, and capped logits.

config.json (every size and every constant that differs between models of the design is read from it):
  architecture      "Zebovik"
  vocab, width
  norm.eps          eps of every RMS norm and unit norm
  logit_softcap     logits <- c * tanh(logits / c)
  layers[i].type    "attention" | "mlstm" | "mamba2"
  layers[i].mixer   attention: heads, kv_heads, dim, vdim, scale, softcap, mask.size, rot.{dims, base}, and optionally
                               kv_from: j (no key and value projections: layer j's cache is read)
                    mlstm:     heads, dim, vdim, gate_cap
                    mamba2:    heads, vdim, state, groups, conv, norm_groups
  layers[i].mlp     null | {kind: "dense", ff}
What the design fixes stands here as constants: the feed-forward's activation (the square of relu) and biases, the
biases of q, k and v, the unit norm of q and k, the sink of score 0, the floor of the mLSTM's denominator.
A sequence has no longest length: nothing in the design depends on one.

Tensor names: embed, l<i>.norm1 / norm1b (before / after the mixer), l<i>.norm2 / norm2b (feed-forward),
attention l<i>.mix.{q, k, v}(.b), l<i>.mix.o; mlstm l<i>.mix.{q, k, v, g, o, norm, i, i.b, f, f.b};
mamba2 l<i>.mix.{in, conv, conv.b, dt_bias, A_log, D, norm, o}; l<i>.mlp.{up, up.b, down, down.b}; final.norm, head.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Mapping

from .registry import ModelConfig, register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

FEED_FORWARD_ACTIVATION = "relu2"   # the square of relu
MLSTM_DENOMINATOR_FLOOR = 1e-6      # added to max(|n . q|, exp(-m))
NO_LENGTH_LIMIT = 1 << 30           # what the runtime is told where it asks for a longest sequence


def _need(data: Mapping[str, Any], key: str, where: str = "config.json"):
    if not isinstance(data, Mapping) or key not in data or data[key] is None:
        raise ValueError(f"{where}: required key {key!r} is missing")
    return data[key]


def _positive(data, keys, where):
    for key in keys:
        if not float(_need(data, key, where)) > 0:
            raise ValueError(f"{where}: {key} must be positive")


@dataclass(frozen=True)
class ZebovikConfig(ModelConfig):
    vocab: int
    width: int
    eps: float
    logit_softcap: float
    layers: tuple          # the config's own layer entries (plain dicts), validated
    torch_dtype: str = "bfloat16"

    architecture = "Zebovik"
    model_type = "zebovik"

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "ZebovikConfig":
        layers = _need(data, "layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ValueError("config.json: 'layers' must be a non-empty list")
        config = cls(vocab=int(_need(data, "vocab")), width=int(_need(data, "width")),
                     eps=float(_need(_need(data, "norm"), "eps", "config.json norm")),
                     logit_softcap=float(data.get("logit_softcap") or 0.0),
                     layers=tuple(copy.deepcopy(dict(layer)) for layer in layers),
                     torch_dtype=str(data.get("torch_dtype", data.get("dtype", "bfloat16"))))
        config.validate()
        return config

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0 or self.eps <= 0 or self.logit_softcap < 0:
            raise ValueError("config.json: vocab, width and norm.eps must be positive, logit_softcap not negative")
        for i, layer in enumerate(self.layers):
            where = f"config.json layers[{i}]"
            kind, mixer = _need(layer, "type", where), _need(layer, "mixer", where)
            where += ".mixer"
            if kind == "attention":
                _positive(mixer, ("heads", "kv_heads", "dim", "vdim", "scale"), where)
                if int(mixer["heads"]) % int(mixer["kv_heads"]):
                    raise ValueError(f"{where}: kv_heads must divide heads")
                rot = _need(mixer, "rot", where)
                if int(_need(rot, "dims", where + ".rot")) % 2 or not 0 <= int(rot["dims"]) <= int(mixer["dim"]):
                    raise ValueError(f"{where}.rot: dims must be even and at most dim")
                if int(rot["dims"]):
                    _positive(rot, ("base",), where + ".rot")
                if mixer.get("mask") is not None:
                    _positive(mixer["mask"], ("size",), where + ".mask")
                source = mixer.get("kv_from")
                if source is not None:
                    source = int(source)
                    other = self.layers[source] if 0 <= source < i else None
                    if other is None or other.get("type") != "attention" or other["mixer"].get("kv_from") is not None:
                        raise ValueError(f"{where}: kv_from must name an earlier attention layer with keys and values of its own")
                    for key in ("heads", "kv_heads", "dim", "vdim"):
                        if int(other["mixer"][key]) != int(mixer[key]):
                            raise ValueError(f"{where}: {key} differs from layer {source}'s, whose keys and values it reads")
                    if other["mixer"]["rot"] != mixer["rot"]:
                        raise ValueError(f"{where}: rot differs from layer {source}'s, whose keys it reads")
            elif kind == "mlstm":
                _positive(mixer, ("heads", "dim", "vdim", "gate_cap"), where)
            elif kind == "mamba2":
                _positive(mixer, ("heads", "vdim", "state", "groups", "conv", "norm_groups"), where)
                if int(mixer["heads"]) % int(mixer["groups"]) or int(mixer["heads"]) * int(mixer["vdim"]) % int(mixer["norm_groups"]):
                    raise ValueError(f"{where}: groups must divide heads, norm_groups must divide heads * vdim")
            else:
                raise ValueError(f"config.json layers[{i}]: mixer type {kind!r} is not supported ('attention', 'mlstm', 'mamba2')")
            mlp = layer.get("mlp")
            if mlp is not None:
                if _need(mlp, "kind", f"config.json layers[{i}].mlp") != "dense":
                    raise ValueError(f"config.json layers[{i}].mlp: kind {mlp['kind']!r} is not supported ('dense' or null)")
                _positive(mlp, ("ff",), f"config.json layers[{i}].mlp")

    def to_dict(self) -> dict:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
                "logit_softcap": self.logit_softcap, "layers": [copy.deepcopy(layer) for layer in self.layers],
                "torch_dtype": self.torch_dtype}

    def _mixer_spec(self, kind: str, m: Mapping[str, Any], p: str) -> PartSpec:
        if kind == "attention":
            own = m.get("kv_from") is None
            dims = int(m["rot"]["dims"])
            position = PartSpec("rotary_half", {"head_dim": int(m["dim"]), "rotary_dim": dims, "theta": float(m["rot"]["base"]),
                                                "precise": True}) \
                if dims else None
            tensors = {"q_weight": p + "q", "q_bias": p + "q.b", "o_weight": p + "o"}
            if own:
                tensors.update({"k_weight": p + "k", "k_bias": p + "k.b", "v_weight": p + "v", "v_bias": p + "v.b"})
            return PartSpec(
                "gqa_attention",
                {"hidden_size": self.width, "num_heads": int(m["heads"]), "num_kv_heads": int(m["kv_heads"]), "head_dim": int(m["dim"]),
                 "value_dim": int(m["vdim"]), "qkv_bias": True, "out_bias": False, "scale": float(m["scale"]), "window": 0,
                 "position": position, "unit_norm_eps": self.eps, "softcap": float(m.get("softcap") or 0.0),
                 "chunk": int((m.get("mask") or {}).get("size") or 0), "sink": "unit", "own_kv": own},
                tensors)
        if kind == "mlstm":
            return PartSpec(
                "matrix_memory",
                {"hidden_size": self.width, "num_heads": int(m["heads"]), "head_dim": int(m["dim"]), "value_dim": int(m["vdim"]),
                 "gate_cap": float(m["gate_cap"]), "eps": self.eps, "floor": MLSTM_DENOMINATOR_FLOOR},
                {"q_weight": p + "q", "k_weight": p + "k", "v_weight": p + "v", "g_weight": p + "g", "o_weight": p + "o",
                 "norm": p + "norm", "i_weight": p + "i", "i_bias": p + "i.b", "f_weight": p + "f", "f_bias": p + "f.b"})
        return PartSpec(
            "state_space",
            {"hidden_size": self.width, "num_heads": int(m["heads"]), "value_dim": int(m["vdim"]), "state_size": int(m["state"]),
             "groups": int(m["groups"]), "conv_taps": int(m["conv"]), "norm_parts": int(m["norm_groups"]), "eps": self.eps},
            {"in_weight": p + "in", "conv_weight": p + "conv", "conv_bias": p + "conv.b", "dt_bias": p + "dt_bias",
             "rate_log": p + "A_log", "skip": p + "D", "norm": p + "norm", "o_weight": p + "o"})

    def model_spec(self) -> ModelSpec:
        def norm(name: str) -> PartSpec:
            return PartSpec("rms_norm", {"width": self.width, "eps": self.eps}, {"weight": name})

        layers, schedule, ignored = [], [], []
        for i, layer in enumerate(self.layers):
            p = f"l{i}."
            parts = {"mixer_norm": norm(p + "norm1"), "mixer": self._mixer_spec(layer["type"], layer["mixer"], p + "mix."),
                     "mixer_post_norm": norm(p + "norm1b")}
            mlp = layer.get("mlp")
            if mlp is None:
                ignored += [p + "norm2", p + "norm2b"]   # a file may still carry them
            else:
                parts["feed_forward_norm"] = norm(p + "norm2")
                parts["feed_forward_post_norm"] = norm(p + "norm2b")
                parts["feed_forward"] = PartSpec(
                    "activated_mlp",
                    {"hidden_size": self.width, "intermediate_size": int(mlp["ff"]), "activation": FEED_FORWARD_ACTIVATION, "bias": True},
                    {"up_weight": p + "mlp.up", "up_bias": p + "mlp.up.b", "down_weight": p + "mlp.down", "down_bias": p + "mlp.down.b"})
            layers.append(LayerSpec("sandwich_norm", parts))
            source = layer["mixer"].get("kv_from") if layer["type"] == "attention" else None
            schedule.append(ScheduleEntry(i, None if source is None else int(source)))
        spec = ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=self.width, max_positions=NO_LENGTH_LIMIT,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab, "width": self.width}, {"weight": "embed"}),
            layers=tuple(layers), schedule=tuple(schedule), final_norm=norm("final.norm"),
            head=PartSpec("linear_head", {"vocab_size": self.vocab, "width": self.width, "tied": False,
                                          "softcap": self.logit_softcap}, {"weight": "head"}),
            ignored_tensors=tuple(ignored))
        spec.validate()
        return spec


register_architecture(ZebovikConfig.architecture, ZebovikConfig, ZebovikConfig.model_type)
