"""The tests' own small Zufusun configurations.  They differ from one another in every size, in the order and number
of layers, in the constants, and in which values happen to be equal (heads and key heads, key and value sizes, the
rotated part and the rotation, experts and choices) or 1."""
from __future__ import annotations

import json
import os

import torch


def _moe(ff, limit, experts, top):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}


ZUFUSUN = {
    # widths the tensor-core product takes; values wider than keys; a layer without feed-forward; one choice of four
    # experts, and as many choices as experts; a latent layer read by a later one with other heads and head sizes
    "u": dict(seed=11, json={
        "architecture": "Zufusun", "vocab": 300, "width": 96, "norm": {"eps": 1e-5}, "layers": [
            {"type": "attention", "mixer": {"heads": 6, "kv_heads": 2, "dim": 16, "vdim": 24, "scale": 0.25,
                                            "mask": {"size": 20, "keep_first": 3}}, "mlp": _moe(40, 1.5, 5, 2)},
            {"type": "gla", "mixer": {"heads": 3, "dim": 24, "vdim": 40, "tau": 8.0, "decay_rank": 8}, "mlp": None},
            {"type": "latent_attention", "mixer": {"heads": 3, "dim": 24, "rot_dim": 8, "vdim": 20, "q_rank": 48, "kv_rank": 40,
                                                   "scale": 0.17, "rot": {"dims": 8, "base": 10000.0}}, "mlp": _moe(64, 3.0, 4, 1)},
            {"type": "latent_attention", "mixer": {"heads": 5, "dim": 16, "rot_dim": 8, "vdim": 32, "q_rank": 32, "kv_rank": 40,
                                                   "scale": 0.2, "rot": {"dims": 8, "base": 10000.0}, "kv_from": 2},
             "mlp": _moe(24, 0.8, 3, 3)},
            {"type": "attention", "mixer": {"heads": 2, "kv_heads": 2, "dim": 32, "vdim": 32, "scale": 0.18,
                                            "mask": {"size": 33, "keep_first": 0}}, "mlp": _moe(48, 2.5, 6, 4)},
        ]}),
    # a width no tensor-core product takes; more first tokens kept than the window is long; one key head; one
    # recurrent head; a rotation over a part of the rotated part; forty query heads on one latent; two latent sources
    "v": dict(seed=23, json={
        "architecture": "Zufusun", "vocab": 257, "width": 100, "norm": {"eps": 1e-6}, "layers": [
            {"type": "latent_attention", "mixer": {"heads": 2, "dim": 32, "rot_dim": 16, "vdim": 48, "q_rank": 24, "kv_rank": 72,
                                                   "scale": 0.12, "rot": {"dims": 8, "base": 500.0}}, "mlp": _moe(30, 2.0, 6, 2)},
            {"type": "attention", "mixer": {"heads": 4, "kv_heads": 1, "dim": 20, "vdim": 12, "scale": 0.3,
                                            "mask": {"size": 7, "keep_first": 9}}, "mlp": None},
            {"type": "gla", "mixer": {"heads": 1, "dim": 40, "vdim": 72, "tau": 4.0, "decay_rank": 5}, "mlp": _moe(50, 1.0, 2, 2)},
            {"type": "attention", "mixer": {"heads": 3, "kv_heads": 3, "dim": 18, "vdim": 18, "scale": 0.2,
                                            "mask": {"size": 1, "keep_first": 1}}, "mlp": _moe(20, 4.0, 7, 3)},
            {"type": "latent_attention", "mixer": {"heads": 40, "dim": 8, "rot_dim": 4, "vdim": 6, "q_rank": 16, "kv_rank": 20,
                                                   "scale": 0.3, "rot": {"dims": 4, "base": 77.0}}, "mlp": None},
            {"type": "latent_attention", "mixer": {"heads": 2, "dim": 12, "rot_dim": 4, "vdim": 30, "q_rank": 40, "kv_rank": 20,
                                                   "scale": 0.25, "rot": {"dims": 4, "base": 77.0}, "kv_from": 4},
             "mlp": _moe(36, 2.0, 3, 1)},
        ]}),
    # head sizes of a real model's layers (128; a latent of 256 with 64 rotated; a recurrence of 288 key channels, which
    # the register-resident scan does not take), few layers
    "w": dict(seed=31, json={
        "architecture": "Zufusun", "vocab": 512, "width": 256, "norm": {"eps": 1e-6}, "layers": [
            {"type": "gla", "mixer": {"heads": 2, "dim": 128, "vdim": 128, "tau": 16.0, "decay_rank": 16}, "mlp": _moe(256, 7.0, 8, 2)},
            {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 128, "vdim": 128, "scale": 0.0884,
                                            "mask": {"size": 128, "keep_first": 4}}, "mlp": _moe(256, 7.0, 8, 2)},
            {"type": "latent_attention", "mixer": {"heads": 4, "dim": 128, "rot_dim": 64, "vdim": 128, "q_rank": 192, "kv_rank": 256,
                                                   "scale": 0.0722, "rot": {"dims": 64, "base": 1e6}}, "mlp": _moe(128, 7.0, 4, 2)},
            {"type": "gla", "mixer": {"heads": 1, "dim": 288, "vdim": 64, "tau": 16.0, "decay_rank": 32}, "mlp": None},
        ]}),
}


def zufusun_config(name: str):
    from ember_b200.config import ZufusunConfig
    return ZufusunConfig.from_json(ZUFUSUN[name]["json"])


def write_zufusun_dir(name: str, out_dir: str, drop_ranks: bool = True) -> str:
    """A model folder with random weights.  ``drop_ranks``: config.json is written without the low-rank size, as a
    stored model's is (it is read from the tensors' shapes)."""
    from ember_b200.weights import write_model_dir
    write_model_dir(zufusun_config(name), out_dir, seed=ZUFUSUN[name]["seed"], dtype=torch.bfloat16)
    if drop_ranks:
        path = os.path.join(out_dir, "config.json")
        with open(path) as f:
            c = json.load(f)
        for l in c["layers"]:
            l["mixer"].pop("decay_rank", None)
        with open(path, "w") as f:
            json.dump(c, f)
    return out_dir


def plain_inputs(model_dir: str):
    """(config dictionary, name -> float64 tensor) as the plain implementation takes them."""
    from tests.plain.qwen3_plain import read_safetensors
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    W = read_safetensors(os.path.join(model_dir, "model.safetensors"))
    return cfg, {k: (v.double() if v.is_floating_point() else v) for k, v in W.items()}
