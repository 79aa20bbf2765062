"""Zufusun without a device: reading config.json, the tensors a model declares, cache needs and the run order, the
random-weights folder, pages of kept first tokens in the cache manager, and the plain implementation's own mechanisms
on cases whose answer is known."""
import json
import math

import pytest
import torch

from tests.zufusun_configs import ZUFUSUN, plain_inputs, write_zufusun_dir, zufusun_config


def test_registered_and_resolved_by_the_architecture_key():
    from ember_b200.config import ZufusunConfig, config_from_dict, registered_architectures
    assert "Zufusun" in registered_architectures()
    cfg = config_from_dict(ZUFUSUN["u"]["json"])
    assert isinstance(cfg, ZufusunConfig) and cfg.width == 96 and len(cfg.layers) == 5
    assert config_from_dict(cfg.to_json()) == cfg


@pytest.mark.parametrize("name", sorted(ZUFUSUN))
def test_spec_layers_cache_needs_and_run_order(name):
    from ember_b200.model.causal_lm import CausalLM
    cfg = zufusun_config(name)
    spec = cfg.to_model_spec()
    needs = CausalLM(spec).cache_needs()
    assert spec.tie_embeddings
    for i, l in enumerate(ZUFUSUN[name]["json"]["layers"]):
        m, roles = l["mixer"], spec.layers[i].roles()
        assert ("feed_forward" in roles) == (l["mlp"] is not None)
        assert "mixer_norm" not in roles and "feed_forward_norm" not in roles          # the sublayers read the stream itself
        if l["type"] == "attention":
            n = needs[i]
            assert (n.kind, n.num_kv_heads, n.head_dim, n.window, n.keep_first) == \
                ("window", m["kv_heads"], m["dim"], m["mask"]["size"], m["mask"]["keep_first"])
            assert (n.value_dim or n.head_dim) == m["vdim"]
        elif l["type"] == "gla":
            assert needs[i].state_shape == (m["heads"] * m["dim"] * m["vdim"],)
        elif "kv_from" in m:
            assert i not in needs and spec.schedule[i].cache_of == m["kv_from"]       # it owns no cache: it reads another's
        else:
            n = needs[i]
            assert (n.kind, n.num_kv_heads, n.head_dim, n.keys_only) == ("full", 1, m["kv_rank"] + m["rot_dim"], True)
            assert spec.schedule[i].cache_of == -1


def test_bad_configurations_are_refused_when_read():
    from ember_b200.config import ConfigError, config_from_dict
    good = ZUFUSUN["u"]["json"]
    for edit in (lambda c: c.pop("width"), lambda c: c["norm"].pop("eps"), lambda c: c["layers"][0].update(type="mlstm"),
                 lambda c: c["layers"][1]["mixer"].pop("tau"), lambda c: c["layers"][0]["mlp"].update(kind="dense"),
                 lambda c: c["layers"][0]["mixer"].update(heads=5), lambda c: c.update(layers=[]),
                 lambda c: c["layers"][3]["mixer"].update(kv_from=3), lambda c: c["layers"][3]["mixer"].update(kv_from=1),
                 lambda c: c["layers"][3]["mixer"].update(kv_rank=48), lambda c: c["layers"][0]["mlp"]["router"].update(top=6),
                 lambda c: c["layers"][2]["mixer"]["rot"].update(dims=10), lambda c: c["layers"][0]["mixer"]["mask"].update(size=0)):
        c = json.loads(json.dumps(good))
        edit(c)
        with pytest.raises(ConfigError):
            config_from_dict(c)


def test_random_folder_declares_what_the_plain_implementation_reads(tmp_path):
    from tests.plain import zufusun_plain as plain
    d = write_zufusun_dir("u", str(tmp_path), drop_ranks=True)
    cfg, W = plain_inputs(d)
    assert "decay_rank" not in json.dumps(cfg)
    logits = plain.forward(cfg, W, [5, 17, 3, 200, 41, 7, 7, 250])
    assert logits.shape == (8, 300) and bool(torch.isfinite(logits).all())
    from ember_b200.config import load_config
    from ember_b200.model.causal_lm import CausalLM
    from ember_b200.weights import WeightStore
    store = WeightStore.from_dir(d)
    model = CausalLM(load_config(d).to_model_spec())
    gla = model.blocks[1].parts["mixer"]
    assert gla.decay_rank == 0 and store.shape("l1.mix.a1") == (8, 96)      # the rank is the stored tensor's


def test_pages_of_the_kept_first_tokens_are_never_given_back():
    """A window group gives back the pages its window has passed, except those that hold a kept first token."""
    from ember_b200.cache.manager import CacheManager
    from ember_b200.parts.base import CacheNeed
    needs = {0: CacheNeed(kind="window", num_kv_heads=1, head_dim=8, window=10, keep_first=5),
             1: CacheNeed(kind="window", num_kv_heads=1, head_dim=8, window=10),
             2: CacheNeed(kind="window", num_kv_heads=1, head_dim=8, window=10, keep_first=4)}
    cm = CacheManager(needs, page_tokens=4, capacity_tokens=64, max_requests=2)
    assert len(cm.groups) == 3
    cm.admit("a")
    assert cm.ensure("a", 30)
    cm.advance("a", 30)                     # the next query sees keys >= 21: pages 0..4 are behind the window
    t = cm.get("a").tables
    assert [p >= 0 for p in t[0]] == [True, True, False, False, False, True, True, True]       # 5 kept tokens: two pages
    assert [p >= 0 for p in t[1]] == [False] * 5 + [True] * 3
    assert [p >= 0 for p in t[2]] == [True, False, False, False, False, True, True, True]      # 4 kept tokens: one page
    assert cm.check() == ""
    assert cm.ensure("a", 47)
    cm.advance("a", 47)
    assert [p >= 0 for p in cm.get("a").tables[0]][:3] == [True, True, False]
    cm.release("a")
    assert cm.used_pages() == [0, 0, 0] and cm.check() == ""


# ------------------------------------------------------------- the plain implementation on known answers
def test_plain_window_and_kept_tokens():
    from tests.plain.zufusun_plain import visible
    m = visible(12, window=4, keep_first=2)
    assert m[9].nonzero().flatten().tolist() == [0, 1, 6, 7, 8, 9]
    assert m[3].nonzero().flatten().tolist() == [0, 1, 2, 3]
    assert visible(5).tolist() == torch.tril(torch.ones(5, 5)).bool().tolist()


def test_plain_sink_takes_its_share_of_the_weights():
    from tests.plain.zufusun_plain import sink_softmax
    s = torch.zeros(1, 3, 3, dtype=torch.float64)
    w = sink_softmax(s, torch.tril(torch.ones(3, 3)).bool(), torch.tensor([math.log(2.0)]))
    assert torch.allclose(w[0, 2], torch.full((3,), 1 / 5, dtype=torch.float64))            # 3 keys of weight 1, a sink of 2
    assert torch.allclose(w[0, 0], torch.tensor([1 / 3, 0, 0], dtype=torch.float64))


def test_plain_pairs_rotate_by_position_times_frequency():
    from tests.plain.zufusun_plain import interleaved_rotation
    x = torch.zeros(3, 1, 6, dtype=torch.float64)
    x[:, 0, 0] = 1.0
    x[:, 0, 2] = 1.0
    x[:, 0, 5] = 7.0
    y = interleaved_rotation(x, 100.0, 4)
    for p in range(3):
        assert torch.allclose(y[p, 0, :2], torch.tensor([math.cos(p), math.sin(p)], dtype=torch.float64))
        assert torch.allclose(y[p, 0, 2:4], torch.tensor([math.cos(p * 0.1), math.sin(p * 0.1)], dtype=torch.float64))
        assert y[p, 0, 5] == 7.0


def test_plain_router_and_expert():
    from tests.plain.zufusun_plain import clamped_expert, routed_experts, router_choice
    W = {"r.router": torch.tensor([[1.0, 0.0], [0.0, 1.0], [0.5, 0.5]], dtype=torch.float64)}
    for e in range(3):
        W[f"r.e{e}.gate"] = torch.eye(2, dtype=torch.float64) * (e + 1)
        W[f"r.e{e}.up"] = torch.zeros(2, 2, dtype=torch.float64)
        W[f"r.e{e}.down"] = torch.eye(2, dtype=torch.float64)
    mlp = {"router": {"experts": 3, "top": 2}, "expert": {"limit": 2.0}}
    h = torch.tensor([[3.0, 1.0]], dtype=torch.float64)
    idx, wgt = router_choice(h, W, "r.", mlp)
    assert idx.tolist() == [[0, 2]] and torch.allclose(wgt, torch.softmax(torch.tensor([[3.0, 2.0]], dtype=torch.float64), -1))
    g = torch.tensor([2.0, 1.0], dtype=torch.float64)                      # expert 0: gate (3, 1) -> min(., 2); up 0 -> u + 1 = 1
    assert torch.allclose(clamped_expert(h, W, "r.e0.", 2.0)[0], g * torch.sigmoid(1.702 * g))
    out = routed_experts(h, W, "r.", mlp)
    want = wgt[0, 0] * clamped_expert(h, W, "r.e0.", 2.0) + wgt[0, 1] * clamped_expert(h, W, "r.e2.", 2.0)
    assert torch.allclose(out, want)


def test_cli_info_and_random(tmp_path, capsys):
    """`python -m ember_b200 info` on a folder written by the random-weights mode."""
    from ember_b200 import cli
    d = write_zufusun_dir("u", str(tmp_path / "m"), drop_ranks=False)
    assert cli.main(["info", "-m", d]) in (0, None)
    out = capsys.readouterr().out
    assert "zufusun: 5 layers" in out and "state per request" in out
