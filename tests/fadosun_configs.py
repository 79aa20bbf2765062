"""The tests' own small Fadosun configurations.  They differ from one another in every size, in the order and
number of layers, in the constants, and in which values happen to be equal (heads and key heads, groups and heads,
rotated and whole head size) or 1."""
from __future__ import annotations

import json
import os

import torch

FADOSUN = {
    # sizes the tensor-core product takes (widths a multiple of 8); a layer without feed-forward; key heads shared
    "p": dict(seed=7, json={
        "architecture": "Fadosun", "vocab": 300, "width": 96, "norm": {"eps": 1e-5}, "layers": [
            {"type": "channel_delta", "mixer": {"heads": 4, "kv_heads": 2, "dim": 24, "vdim": 40, "conv": 3,
                                                "decay_rank": 16, "gate_rank": 8}, "mlp": {"kind": "dense", "ff": 160}},
            {"type": "parallel", "mixer": {
                "left": {"heads": 6, "kv_heads": 2, "dim": 32, "vdim": 24, "scale": 0.2, "rot": {"dims": 16, "base": 10000.0}},
                "right": {"heads": 4, "vdim": 20, "state": 16, "groups": 1, "norm_groups": 1, "conv": 2},
                "left_scale": 0.7, "right_scale": 1.3}, "mlp": None},
            {"type": "mlstm", "mixer": {"heads": 3, "dim": 16, "vdim": 32, "gate_cap": 8.0}, "mlp": {"kind": "dense", "ff": 72}},
        ]}),
    # a width no tensor-core product takes, one head, whole-head rotation, value heads wider than a block of columns,
    # two attention layers (one page group), five taps, ranks that are no multiple of 8
    "q": dict(seed=19, json={
        "architecture": "Fadosun", "vocab": 257, "width": 100, "norm": {"eps": 1e-6}, "layers": [
            {"type": "mlstm", "mixer": {"heads": 1, "dim": 40, "vdim": 72, "gate_cap": 15.0}, "mlp": {"kind": "dense", "ff": 50}},
            {"type": "parallel", "mixer": {
                "left": {"heads": 2, "kv_heads": 2, "dim": 64, "vdim": 160, "scale": 0.11, "rot": {"dims": 64, "base": 500.0}},
                "right": {"heads": 6, "vdim": 12, "state": 8, "groups": 3, "norm_groups": 3, "conv": 5},
                "left_scale": 1.0, "right_scale": 0.5}, "mlp": {"kind": "dense", "ff": 120}},
            {"type": "channel_delta", "mixer": {"heads": 2, "kv_heads": 2, "dim": 70, "vdim": 130, "conv": 4,
                                                "decay_rank": 6, "gate_rank": 10}, "mlp": None},
            {"type": "parallel", "mixer": {
                "left": {"heads": 2, "kv_heads": 2, "dim": 64, "vdim": 160, "scale": 0.2, "rot": {"dims": 2, "base": 77.0}},
                "right": {"heads": 2, "vdim": 36, "state": 40, "groups": 2, "norm_groups": 1, "conv": 1},
                "left_scale": 0.3, "right_scale": 1.9}, "mlp": {"kind": "dense", "ff": 64}},
        ]}),
    # head sizes of a real model's layers (128 / 256), few layers
    "r": dict(seed=29, json={
        "architecture": "Fadosun", "vocab": 512, "width": 256, "norm": {"eps": 1e-6}, "layers": [
            {"type": "parallel", "mixer": {
                "left": {"heads": 4, "kv_heads": 2, "dim": 128, "vdim": 128, "scale": 0.0884, "rot": {"dims": 32, "base": 1e6}},
                "right": {"heads": 8, "vdim": 64, "state": 64, "groups": 2, "norm_groups": 4, "conv": 4},
                "left_scale": 1.0, "right_scale": 1.0}, "mlp": {"kind": "dense", "ff": 512}},
            {"type": "channel_delta", "mixer": {"heads": 4, "kv_heads": 1, "dim": 128, "vdim": 128, "conv": 4,
                                                "decay_rank": 32, "gate_rank": 32}, "mlp": {"kind": "dense", "ff": 512}},
            {"type": "mlstm", "mixer": {"heads": 2, "dim": 128, "vdim": 256, "gate_cap": 15.0}, "mlp": {"kind": "dense", "ff": 512}},
        ]}),
}


def fadosun_config(name: str):
    from ember_b200.config import FadosunConfig
    return FadosunConfig.from_json(FADOSUN[name]["json"])


def write_fadosun_dir(name: str, out_dir: str, drop_ranks: bool = True) -> str:
    """A model folder with random weights.  ``drop_ranks``: config.json is written without the low-rank sizes, as a
    stored model's is (they are read from the tensors' shapes)."""
    from ember_b200.weights import write_model_dir
    write_model_dir(fadosun_config(name), out_dir, seed=FADOSUN[name]["seed"], dtype=torch.bfloat16)
    if drop_ranks:
        path = os.path.join(out_dir, "config.json")
        with open(path) as f:
            c = json.load(f)
        for l in c["layers"]:
            l["mixer"].pop("decay_rank", None)
            l["mixer"].pop("gate_rank", None)
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
