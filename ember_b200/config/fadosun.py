"""Fadosun: a decoder whose layers are listed one by one in config.json, each with one of three mixers and a
gated feed-forward, every sublayer between two layer norms and under an element-wise gate.

config.json keys: ``architecture`` "Fadosun"; ``vocab``; ``width``; ``norm.eps``; ``layers``: a list of
``{"type", "mixer", "mlp"}`` where ``type`` is "mlstm" (mixer: heads, dim, vdim, gate_cap), "channel_delta"
(heads, kv_heads, dim, vdim, conv) or "parallel" (left: heads, kv_heads, dim, vdim, scale, rot.dims, rot.base;
right: heads, vdim, state, groups, norm_groups, conv; left_scale, right_scale), and ``mlp`` is
``{"kind": "dense", "ff"}`` or null.  Tensor names: ``embed``, ``head``, ``final.norm`` (+ ``.b``), and per layer
``l<i>.`` + norm1, norm1b, norm2, norm2b (+ ``.b``), rg1, rg2 (+ ``.b``), ``mix.*``, ``mlp.gate|up|down``.

Two optional keys are this engine's own: ``max_positions`` (longest sequence; default 1,048,576) and, in a
"channel_delta" mixer, ``decay_rank`` / ``gate_rank`` (the low-rank projections' inner sizes, which a stored model
gives by its tensors' shapes; the random-weights mode needs them written down).
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Mapping, Optional, Tuple

from .registry import register_architecture
from .spec import (ConfigError, GatedDeltaSpec, GatedMLPSpec, LayerNormSpec, LayerSpec, MatrixMemorySpec, ModelSpec,
                   ParallelMixerSpec, RotarySpec, SigmoidAttentionSpec, SigmoidGateSpec, StateSpaceSpec, default_schedule)


def _need(d: Mapping, key: str, where: str):
    if not isinstance(d, Mapping) or d.get(key) is None:
        raise ConfigError(f"config.json: {where} lacks the key {key!r}")
    return d[key]


def _int(d: Mapping, key: str, where: str) -> int:
    v = _need(d, key, where)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v or int(v) <= 0:
        raise ConfigError(f"config.json: {where}.{key} must be a positive integer, got {v!r}")
    return int(v)


def _float(d: Mapping, key: str, where: str) -> float:
    v = _need(d, key, where)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: {where}.{key} must be a number, got {v!r}")
    return float(v)


@dataclass(frozen=True)
class FadosunConfig:
    vocab: int
    width: int
    eps: float
    layers: Tuple[dict, ...]            # as config.json lists them (checked)
    max_positions: int = 1 << 20

    architecture = "Fadosun"
    model_type = "fadosun"

    @classmethod
    def from_json(cls, config: Mapping, generation_config: Optional[Mapping] = None) -> "FadosunConfig":
        layers = _need(config, "layers", "the model")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: layers must be a non-empty list")
        out = cls(vocab=_int(config, "vocab", "the model"), width=_int(config, "width", "the model"),
                  eps=_float(_need(config, "norm", "the model"), "eps", "norm"),
                  layers=tuple(copy.deepcopy(dict(l)) for l in layers),
                  max_positions=int(config.get("max_positions") or (1 << 20)))
        # every layer's keys are read and every part is built (without a device) now, so that a bad value is
        # refused here and not at the first step
        from ..model.causal_lm import CausalLM
        CausalLM(out.to_model_spec())
        return out

    # ------------------------------------------------------------------ mixers
    def _mixer(self, i: int, kind: str, m: Mapping):
        where = f"layers[{i}].mixer"
        if kind == "mlstm":
            return MatrixMemorySpec(hidden_size=self.width, num_heads=_int(m, "heads", where), head_dim=_int(m, "dim", where),
                                    value_dim=_int(m, "vdim", where), gate_cap=_float(m, "gate_cap", where), norm_eps=self.eps)
        if kind == "channel_delta":
            return GatedDeltaSpec(hidden_size=self.width, num_heads=_int(m, "heads", where),
                                  num_kv_heads=_int(m, "kv_heads", where), head_dim=_int(m, "dim", where),
                                  value_dim=_int(m, "vdim", where), conv_taps=_int(m, "conv", where),
                                  decay_rank=int(m.get("decay_rank") or 0), gate_rank=int(m.get("gate_rank") or 0),
                                  norm_eps=self.eps)
        if kind == "parallel":
            l, r = _need(m, "left", where), _need(m, "right", where)
            rot = _need(l, "rot", where + ".left")
            dim = _int(l, "dim", where + ".left")
            left = SigmoidAttentionSpec(
                hidden_size=self.width, num_heads=_int(l, "heads", where + ".left"),
                num_kv_heads=_int(l, "kv_heads", where + ".left"), head_dim=dim, value_dim=_int(l, "vdim", where + ".left"),
                scale=_float(l, "scale", where + ".left"),
                position=RotarySpec(head_dim=dim, rotary_dim=_int(rot, "dims", where + ".left.rot"),
                                    theta=_float(rot, "base", where + ".left.rot"), frequency_precision="float64"))
            right = StateSpaceSpec(
                hidden_size=self.width, num_heads=_int(r, "heads", where + ".right"), value_dim=_int(r, "vdim", where + ".right"),
                state_size=_int(r, "state", where + ".right"), num_groups=_int(r, "groups", where + ".right"),
                norm_groups=_int(r, "norm_groups", where + ".right"), conv_taps=_int(r, "conv", where + ".right"),
                norm_eps=self.eps)
            return ParallelMixerSpec(hidden_size=self.width, left=left, right=right,
                                     left_scale=_float(m, "left_scale", where), right_scale=_float(m, "right_scale", where))
        raise ConfigError(f"config.json: layers[{i}].type {kind!r} is not a mixer of this design "
                          f"(mlstm, channel_delta, parallel)")

    # --------------------------------------------------------------- as a model
    def to_model_spec(self) -> ModelSpec:
        def norm(i=None):
            return LayerNormSpec(size=self.width, eps=self.eps, weight_suffix="", bias_suffix=".b")

        gate = SigmoidGateSpec(size=self.width, weight_suffix="", bias_suffix=".b")
        layers = []
        for i, l in enumerate(self.layers):
            p = f"l{i}."
            parts = [("mixer_norm", norm(), p + "norm1"),
                     ("mixer", self._mixer(i, _need(l, "type", f"layers[{i}]"), _need(l, "mixer", f"layers[{i}]")), p + "mix."),
                     ("mixer_gate", gate, p + "rg1"), ("mixer_out_norm", norm(), p + "norm1b")]
            mlp = l.get("mlp")
            if mlp is not None:
                if mlp.get("kind") != "dense":
                    raise ConfigError(f"config.json: layers[{i}].mlp.kind {mlp.get('kind')!r} is not a feed-forward of this design (dense)")
                ff = GatedMLPSpec(hidden_size=self.width, intermediate_size=_int(mlp, "ff", f"layers[{i}].mlp"),
                                  activation="relu", names=("gate", "up", "down"))
                parts += [("feed_forward_norm", norm(), p + "norm2"), ("feed_forward", ff, p + "mlp."),
                          ("feed_forward_gate", gate, p + "rg2"), ("feed_forward_out_norm", norm(), p + "norm2b")]
            layers.append(LayerSpec("gated_sandwich", tuple(parts)))
        return ModelSpec(architecture=self.architecture, vocab_size=self.vocab, hidden_size=self.width, layers=tuple(layers),
                         schedule=default_schedule(len(layers)), final_norm=norm(), final_norm_prefix="final.norm",
                         embedding_name="embed", head_name="head", tie_embeddings=False, head_optional=False,
                         max_positions=self.max_positions, eos_ids=(), init_std=0.05, init_norm_std=0.1)

    def to_json(self) -> dict:
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
             "layers": [copy.deepcopy(l) for l in self.layers]}
        if self.max_positions != 1 << 20:
            d["max_positions"] = self.max_positions
        return d

    def kv_bytes_per_token(self, elem_bytes: int) -> int:
        """Bytes of paged cache one token takes: keys and values of the attention halves of the parallel layers."""
        total = 0
        for l in self.layers:
            if l["type"] == "parallel":
                a = l["mixer"]["left"]
                total += a["kv_heads"] * (a["dim"] + a["vdim"]) * elem_bytes
        return total

    def state_bytes_per_request(self) -> int:
        """Bytes of fixed-size fp32 state one request holds (matrices, normalisers, convolution inputs)."""
        from ..cache.storage import state_bytes_per_request
        from ..model.causal_lm import CausalLM
        return state_bytes_per_request(CausalLM(self.to_model_spec()).cache_needs())

    def describe(self) -> str:
        kinds = ", ".join(l["type"] for l in self.layers[:8]) + (", ..." if len(self.layers) > 8 else "")
        return f"fadosun: {len(self.layers)} layers ({kinds}), width {self.width}, vocab {self.vocab}"


register_architecture(FadosunConfig.architecture, FadosunConfig, model_type=FadosunConfig.model_type)
