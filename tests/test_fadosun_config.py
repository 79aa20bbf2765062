"""Fadosun without a device: reading config.json, the tensors a model declares, cache needs, the random-weights
folder, and the plain implementation's own consistency (a recurrence fed in two halves with a carried state is
not needed there: it only ever runs whole sequences)."""
import json
import os

import pytest
import torch

from tests.fadosun_configs import FADOSUN, fadosun_config, plain_inputs, write_fadosun_dir


def test_registered_and_resolved_by_the_architecture_key():
    from ember_b200.config import FadosunConfig, config_from_dict, registered_architectures
    assert "Fadosun" in registered_architectures()
    cfg = config_from_dict(FADOSUN["p"]["json"])
    assert isinstance(cfg, FadosunConfig) and cfg.width == 96 and len(cfg.layers) == 3
    assert config_from_dict(cfg.to_json()) == cfg


@pytest.mark.parametrize("name", sorted(FADOSUN))
def test_spec_layers_and_cache_needs(name):
    from ember_b200.model.causal_lm import CausalLM
    cfg = fadosun_config(name)
    spec = cfg.to_model_spec()
    model = CausalLM(spec)
    needs = model.cache_needs()
    for i, l in enumerate(FADOSUN[name]["json"]["layers"]):
        m = l["mixer"]
        roles = spec.layers[i].roles()
        assert ("feed_forward" in roles) == (l["mlp"] is not None)
        if l["type"] == "parallel":
            left, right = needs[(i, "left")], needs[(i, "right")]
            assert (left.kind, left.num_kv_heads, left.head_dim, left.value_dim) == \
                ("full", m["left"]["kv_heads"], m["left"]["dim"], m["left"]["vdim"])
            r = m["right"]
            channels = r["heads"] * r["vdim"] + 2 * r["groups"] * r["state"]
            assert right.state_shape == (r["heads"] * r["state"] * r["vdim"] + (r["conv"] - 1) * channels,)
        elif l["type"] == "mlstm":
            assert needs[i].state_shape == (m["heads"] * (m["dim"] * m["vdim"] + m["dim"] + 1),)
        else:
            channels = 2 * m["kv_heads"] * m["dim"] + m["heads"] * m["vdim"]
            assert needs[i].state_shape == (m["heads"] * m["dim"] * m["vdim"] + (m["conv"] - 1) * channels,)


def test_bad_configurations_are_refused_when_read():
    from ember_b200.config import ConfigError, config_from_dict
    good = FADOSUN["p"]["json"]
    for edit in (lambda c: c.pop("width"), lambda c: c["norm"].pop("eps"), lambda c: c["layers"][0].update(type="attention"),
                 lambda c: c["layers"][0]["mixer"].pop("conv"), lambda c: c["layers"][2]["mlp"].update(kind="experts"),
                 lambda c: c["layers"][1]["mixer"]["left"].update(heads=5), lambda c: c.update(layers=[])):
        c = json.loads(json.dumps(good))
        edit(c)
        with pytest.raises(ConfigError):
            config_from_dict(c)


def test_random_folder_declares_what_the_plain_implementation_reads(tmp_path):
    from tests.plain import fadosun_plain as plain
    d = write_fadosun_dir("p", str(tmp_path), drop_ranks=True)
    cfg, W = plain_inputs(d)
    assert "decay_rank" not in json.dumps(cfg)
    logits = plain.forward(cfg, W, [1, 5, 9, 200, 4])
    assert logits.shape == (5, 300) and bool(torch.isfinite(logits).all())
    # every stored tensor is one the model declares, and the other way round
    from ember_b200.model.causal_lm import CausalLM
    declared = {x.name: tuple(x.shape) for x in CausalLM(fadosun_config("p").to_model_spec()).weight_decls()}
    assert declared == {k: tuple(v.shape) for k, v in W.items()}


def test_plain_recurrences_do_not_look_ahead(tmp_path):
    """Causality of the plain implementation itself: logits of a prefix equal the prefix of the logits."""
    from tests.plain import fadosun_plain as plain
    cfg, W = plain_inputs(write_fadosun_dir("q", str(tmp_path)))
    toks = torch.randint(0, 257, (23,), generator=torch.Generator().manual_seed(3)).tolist()
    whole = plain.forward(cfg, W, toks)
    assert torch.allclose(plain.forward(cfg, W, toks[:9]), whole[:9], atol=1e-10)


def test_command_line_random_then_info(tmp_path, capsys):
    from ember_b200.cli import main
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(FADOSUN["p"]["json"]))
    out = tmp_path / "model"
    assert main(["random", "--config", str(cfg), "--out", str(out), "--seed", "3"]) == 0
    assert sorted(os.listdir(out)) == ["config.json", "model.safetensors"]
    capsys.readouterr()
    assert main(["info", "-m", str(out)]) == 0
    text = capsys.readouterr().out
    assert "fadosun" in text and "3 layers" in text and "state per request" in text
    # keys and values of the one attention layer: 2 key heads of 32 + 24, bfloat16
    assert "KV cache per token, bfloat16: 0.2 KiB" in text
