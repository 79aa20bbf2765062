"""Zufusun: a decoder whose layers are listed one by one in config.json.  A layer adds the RMS norm of its mixer's
result to the residual stream, then the RMS norm of its feed-forward's; both sublayers read the stream itself (there
is no norm in front of them).  Three mixers: softmax attention with a sink under a window that keeps the first
tokens, latent attention (low-rank queries, a cached key/value latent with a rotated shared key part, a sink, an
output gate; a layer may read another layer's latent), and gated linear attention with a fixed-size state.  The
feed-forward is a mixture of experts.  The logits are the embedding table applied to the normed stream.

config.json keys: ``architecture`` "Zufusun"; ``vocab``; ``width``; ``norm.eps``; ``layers``: a list of
``{"type", "mixer", "mlp"}`` where ``type`` is "attention" (mixer: heads, kv_heads, dim, vdim, scale,
mask.size, mask.keep_first), "latent_attention" (heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, rot.dims, rot.base,
and kv_from for a layer that reads another's latent) or "gla" (heads, dim, vdim, tau), and ``mlp`` is
``{"kind": "moe", "expert": {"ff", "limit"}, "router": {"experts", "top"}}`` or null.  Tensor names: ``embed``,
``final.norm``, and per layer ``l<i>.`` + norm1, norm2, ``mix.*``, ``mlp.router``, ``mlp.e<j>.gate|up|down``.

Two optional keys are this engine's own: ``max_positions`` (longest sequence; default 1,048,576) and, in a "gla" mixer,
``decay_rank`` (the inner size of the decay's low-rank projection, which a stored model gives by its tensors' shapes;
the random-weights mode needs it written down).
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Mapping, Optional, Tuple

from .registry import register_architecture
from .spec import (ConfigError, GatedLinearAttentionSpec, LatentAttentionSpec, LayerSpec, ModelSpec, NoPositionSpec,
                   RMSNormSpec, RotarySpec, RoutedMLPSpec, ScheduleEntry, SinkAttentionSpec)


def _need(d: Mapping, key: str, where: str):
    if not isinstance(d, Mapping) or d.get(key) is None:
        raise ConfigError(f"config.json: {where} lacks the key {key!r}")
    return d[key]


def _int(d: Mapping, key: str, where: str, least: int = 1) -> int:
    v = _need(d, key, where)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v or int(v) < least:
        raise ConfigError(f"config.json: {where}.{key} must be an integer >= {least}, got {v!r}")
    return int(v)


def _float(d: Mapping, key: str, where: str) -> float:
    v = _need(d, key, where)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: {where}.{key} must be a number, got {v!r}")
    return float(v)


MIXERS = ("attention", "latent_attention", "gla")


@dataclass(frozen=True)
class ZufusunConfig:
    vocab: int
    width: int
    eps: float
    layers: Tuple[dict, ...]            # as config.json lists them (checked)
    max_positions: int = 1 << 20

    architecture = "Zufusun"
    model_type = "zufusun"

    @classmethod
    def from_json(cls, config: Mapping, generation_config: Optional[Mapping] = None) -> "ZufusunConfig":
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
    def _latent_source(self, i: int, m: Mapping) -> int:
        """The layer whose cached latent layer i reads: itself, or ``kv_from``."""
        src = m.get("kv_from")
        if src is None:
            return i
        where = f"layers[{i}].mixer"
        j = _int(m, "kv_from", where, least=0)
        if j >= i or self.layers[j].get("type") != "latent_attention" or self.layers[j]["mixer"].get("kv_from") is not None:
            raise ConfigError(f"config.json: {where}.kv_from = {j} must name an earlier latent_attention layer with a "
                              f"key/value projection of its own")
        a, b = self.layers[j]["mixer"], m
        same = all(a.get(k) == b.get(k) for k in ("kv_rank", "rot_dim")) and a.get("rot") == b.get("rot")
        if not same:
            raise ConfigError(f"config.json: {where} reads the latent of layer {j}: kv_rank, rot_dim and rot must be equal")
        return j

    def _mixer(self, i: int, kind: str, m: Mapping):
        where = f"layers[{i}].mixer"
        if kind == "attention":
            mask = m.get("mask")
            window = _int(mask, "size", where + ".mask") if mask is not None else 0
            keep = _int(mask, "keep_first", where + ".mask", least=0) if mask is not None and mask.get("keep_first") is not None else 0
            return SinkAttentionSpec(hidden_size=self.width, num_heads=_int(m, "heads", where), num_kv_heads=_int(m, "kv_heads", where),
                                     head_dim=_int(m, "dim", where), value_dim=_int(m, "vdim", where), scale=_float(m, "scale", where),
                                     bias=True, qk_norm="whole", qk_norm_eps=self.eps, window=window, keep_first=keep, sink=True)
        if kind == "latent_attention":
            rot_dim = _int(m, "rot_dim", where, least=0)
            position = NoPositionSpec()
            if rot_dim:
                rot = _need(m, "rot", where)
                position = RotarySpec(head_dim=rot_dim, rotary_dim=_int(rot, "dims", where + ".rot"),
                                      theta=_float(rot, "base", where + ".rot"), frequency_precision="float64", layout="interleaved")
            return LatentAttentionSpec(hidden_size=self.width, num_heads=_int(m, "heads", where), head_dim=_int(m, "dim", where),
                                       rot_dim=rot_dim, value_dim=_int(m, "vdim", where), q_rank=_int(m, "q_rank", where),
                                       kv_rank=_int(m, "kv_rank", where), scale=_float(m, "scale", where), norm_eps=self.eps,
                                       sink=True, gate=True, own_kv=self._latent_source(i, m) == i, position=position)
        if kind == "gla":
            return GatedLinearAttentionSpec(hidden_size=self.width, num_heads=_int(m, "heads", where), head_dim=_int(m, "dim", where),
                                            value_dim=_int(m, "vdim", where), tau=_float(m, "tau", where),
                                            decay_rank=int(m.get("decay_rank") or 0), norm_eps=self.eps)
        raise ConfigError(f"config.json: layers[{i}].type {kind!r} is not a mixer of this design ({', '.join(MIXERS)})")

    def _feed_forward(self, i: int, mlp: Mapping):
        where = f"layers[{i}].mlp"
        if mlp.get("kind") != "moe":
            raise ConfigError(f"config.json: {where}.kind {mlp.get('kind')!r} is not a feed-forward of this design (moe)")
        expert, router = _need(mlp, "expert", where), _need(mlp, "router", where)
        return RoutedMLPSpec(hidden_size=self.width, intermediate_size=_int(expert, "ff", where + ".expert"),
                             experts=_int(router, "experts", where + ".router"), top=_int(router, "top", where + ".router"),
                             limit=_float(expert, "limit", where + ".expert"), alpha=1.702)

    # --------------------------------------------------------------- as a model
    def to_model_spec(self) -> ModelSpec:
        def norm():
            return RMSNormSpec(size=self.width, eps=self.eps, weight_suffix="")

        layers, schedule = [], []
        for i, l in enumerate(self.layers):
            p = f"l{i}."
            kind, m = _need(l, "type", f"layers[{i}]"), _need(l, "mixer", f"layers[{i}]")
            parts = [("mixer", self._mixer(i, kind, m), p + "mix."), ("mixer_out_norm", norm(), p + "norm1")]
            if l.get("mlp") is not None:
                parts += [("feed_forward", self._feed_forward(i, l["mlp"]), p + "mlp."), ("feed_forward_out_norm", norm(), p + "norm2")]
            layers.append(LayerSpec("gated_sandwich", tuple(parts)))
            src = self._latent_source(i, m) if kind == "latent_attention" else i
            schedule.append(ScheduleEntry(i, cache_of=-1 if src == i else src))
        return ModelSpec(architecture=self.architecture, vocab_size=self.vocab, hidden_size=self.width, layers=tuple(layers),
                         schedule=tuple(schedule), final_norm=norm(), final_norm_prefix="final.norm",
                         embedding_name="embed", head_name="head", tie_embeddings=True, head_optional=True,
                         max_positions=self.max_positions, eos_ids=(), init_std=0.05, init_norm_std=0.1)

    def to_json(self) -> dict:
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
             "layers": [copy.deepcopy(l) for l in self.layers]}
        if self.max_positions != 1 << 20:
            d["max_positions"] = self.max_positions
        return d

    def _needs(self):
        from ..model.causal_lm import CausalLM
        return CausalLM(self.to_model_spec()).cache_needs()

    def kv_bytes_per_token(self, elem_bytes: int) -> int:
        """Bytes of paged cache one token takes: keys and values of the windowed layers (while inside the window), one
        latent row of every latent layer that owns one."""
        return sum(n.num_kv_heads * (n.head_dim + (0 if n.keys_only else (n.value_dim or n.head_dim))) * elem_bytes
                   for n in self._needs().values() if n is not None and n.kind in ("full", "window"))

    def state_bytes_per_request(self) -> int:
        """Bytes of fixed-size fp32 state one request holds (the matrices of the gated-linear-attention layers)."""
        from ..cache.storage import state_bytes_per_request
        return state_bytes_per_request(self._needs())

    def describe(self) -> str:
        kinds = ", ".join(l["type"] for l in self.layers[:8]) + (", ..." if len(self.layers) > 8 else "")
        return f"zufusun: {len(self.layers)} layers ({kinds}), width {self.width}, vocab {self.vocab}"


register_architecture(ZufusunConfig.architecture, ZufusunConfig, model_type=ZufusunConfig.model_type)
