"""Fadosun on the device against the plain implementation: each mechanism alone (fed in portions beside another
request), whole models under every way of cutting the work, slots and pages used again, a far key that dominates,
long decoding through captured graphs, and greedy generation through the entry point and its scheduler."""
import json
import os

import numpy as np
import pytest
import torch

from tests.fadosun_configs import FADOSUN, plain_inputs, write_fadosun_dir
from tests.plain import fadosun_plain as plain
from tests.replay_helpers import (collect, first_mismatch, max_live_tokens, trace_mixed, trace_portions,
                                  trace_tail_decode, trace_whole)

pytestmark = pytest.mark.gpu

TOL = {"float32": 3e-5, "bfloat16": 6e-2}


def assert_close(got, want, dtype, what=""):
    """float32 is the sharp test: no position over the tolerance.  In bfloat16 a head's read-out that is close to zero
    before its norm (the first tokens of a request, where S^T q is one k . q times a vector) multiplies rounding, so
    a few positions of a random model may be several times over: none far over, and at most one in fifty over."""
    first, worst = first_mismatch(got, want, TOL[dtype])
    if dtype == "float32":
        assert first is None, f"{what} {dtype}: first mismatch at {first}, worst {worst:.3g}"
        return
    errs = [float(np.linalg.norm(rows[p] - want[r][p]) / max(np.linalg.norm(want[r][p]), 1e-30)) for r, rows in got.items() for p in rows]
    over = sum(e > TOL[dtype] for e in errs)
    assert worst < 0.3 and over <= max(1, len(errs) // 50), f"{what} {dtype}: {over} of {len(errs)} over, first {first}, worst {worst:.3g}"


@pytest.fixture(scope="module")
def dirs(tmp_path_factory):
    return {name: write_fadosun_dir(name, str(tmp_path_factory.mktemp("fadosun_" + name))) for name in FADOSUN}


@pytest.fixture(scope="module")
def plain_logits(dirs):
    cache, inputs = {}, {}

    def get(name, requests):
        if name not in inputs:
            inputs[name] = plain_inputs(dirs[name])
        out = {}
        for rid, toks in requests.items():
            key = (name, tuple(toks))
            if key not in cache:
                cache[key] = plain.forward(*inputs[name], toks).numpy()
            out[rid] = cache[key]
        return out

    return get


def make_requests(name, lengths, seed):
    rng = np.random.default_rng(seed)
    return {f"r{i}": rng.integers(0, FADOSUN[name]["json"]["vocab"], size=n).tolist() for i, n in enumerate(lengths)}


def replay(model_dir, dtype, steps, capacity, page_tokens=16, max_requests=4, max_batch_tokens=512, **kw):
    import tempfile
    from ember_b200.engine.replay import TraceReplayer
    from ember_b200.engine.runner import ModelRunner
    runner = ModelRunner.from_dir(model_dir, dtype=dtype, capacity_tokens=capacity, max_batch_tokens=max_batch_tokens,
                                  max_requests=max_requests, page_tokens=page_tokens, **kw)
    with tempfile.TemporaryDirectory() as out:
        rp = TraceReplayer(runner, out)
        outputs = {}
        for s in steps:
            got = rp.run_step(s)
            if got is not None:
                outputs[s["step"]] = got.copy()
            assert runner.cache.check() == ""
    assert runner.cache.used_pages() == [0] * len(runner.cache.groups)
    return outputs, runner


LENGTHS = {"p": (1, 2, 37, 130), "q": (3, 18, 65, 150), "r": (2, 70, 129)}


@pytest.mark.parametrize("page", [16, 64])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(FADOSUN))
@pytest.mark.parametrize("mode", ["whole", "tail", "portions", "mixed"])
def test_replay_modes(name, dtype, mode, page, dirs, plain_logits):
    """Whole prompts, a decoded tail, portions down to two tokens (and single ones), and four live requests whose
    slots and pages are used again, against each request alone in the plain implementation."""
    requests = make_requests(name, LENGTHS[name], seed=5)
    if mode == "mixed":
        requests = make_requests(name, LENGTHS[name] + (40, 21, 66, 9), seed=6)
    steps = {"whole": trace_whole, "tail": lambda r: trace_tail_decode(r, tail=20),
             "portions": lambda r: trace_portions(r, sizes=(7, 2, 19, 1, 3, 33, 2, 16, 5, 64)),
             "mixed": lambda r: trace_mixed(r, live=4, seed=3)}[mode](requests)
    outputs, _ = replay(dirs[name], dtype, steps, max_live_tokens(steps, round_to=page), page_tokens=page)
    assert_close(collect(steps, outputs), plain_logits(name, requests), dtype, f"{name} {mode}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_through_graphs_equals_the_prompt(dtype, dirs, plain_logits):
    """300 tokens one by one (captured graphs after the second step) against the whole sequence."""
    requests = make_requests("p", (300,), seed=11)
    steps = trace_tail_decode(requests, tail=299)
    outputs, runner = replay(dirs["p"], dtype, steps, 320)
    assert runner.graph_replays > 250
    assert_close(collect(steps, outputs), plain_logits("p", requests), dtype, "long decoding")
    eager, _ = replay(dirs["p"], dtype, steps, 320, cuda_graphs=False)
    assert max(float(np.abs(outputs[k] - eager[k]).max()) for k in outputs) < (1e-5 if dtype == "float32" else 1e-1)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_long_prompt_then_decoding(dtype, dirs, plain_logits):
    """1,300 tokens at a real model's head sizes: keys more than a thousand positions back and a state that has seen
    as many tokens, as one prompt with a decoded tail and as portions of 500."""
    requests = make_requests("r", (1300,), seed=17)
    for steps in (trace_tail_decode(requests, tail=24), trace_portions(requests, sizes=(500, 37, 500, 2))):
        outputs, _ = replay(dirs["r"], dtype, steps, 1344, page_tokens=64, max_batch_tokens=2048)
        assert_close(collect(steps, outputs), plain_logits("r", requests), dtype, "long prompt")


def test_a_slot_used_again_starts_from_zero(dirs, plain_logits):
    """One slot only: the second request gets the state, the convolution inputs and the pages the first left."""
    requests = make_requests("q", (90, 75, 33), seed=21)
    steps = trace_portions(requests, sizes=(40, 3, 1, 31))
    outputs, _ = replay(dirs["q"], "float32", steps, 96, max_requests=1)
    assert_close(collect(steps, outputs), plain_logits("q", requests), "float32", "one slot")


# ------------------------------------------------------------------------------ each mechanism alone
def _run_mixer(spec, weights, x_all, dtype, portions=((40, 7), (3, 1), (1, 1), (2, 2), (44, 19)), prefix="m."):
    """The mixer fed in portions next to another request's portions; returns its stored output [T, hidden]."""
    from ember_b200.parts import build_part
    from tests.test_parts_gpu import Bench, store_of
    part = build_part("mixer", spec, prefix)
    needs = {("x", k) if k else 0: v for k, v in part.cache_needs().items()}
    b = Bench(needs, dtype, capacity=512)
    part.load(store_of(weights), b.rt)
    hidden = x_all.shape[1]
    other = torch.randn(64, hidden, generator=torch.Generator().manual_seed(1)).bfloat16()
    got, at, oat = torch.zeros(x_all.shape[0], hidden), 0, 0
    for n, m in portions:
        ctx = b.ctx([("x", n), ("o", m)], tile_sizes=getattr(part, "tile_requests", lambda: ())())
        x = torch.zeros(256, hidden, device=b.dev, dtype=dtype)
        x[:n] = x_all[at:at + n].to(dtype)
        x[n:n + m] = other[oat:oat + m].to(dtype)
        out = torch.full((256, hidden), 7.0, device=b.dev)
        keys = list(part.cache_needs())
        cache = b.storage.layer(0) if keys == [""] else {k: b.storage.layer(("x", k)) for k in keys}
        part.forward(ctx, x, out, cache, accumulate=False)
        got[at:at + n] = out[:n].cpu()
        at, oat = at + n, oat + m
    assert int(b.err.item()) == 0
    return got


def _rel(a, b):
    return float((a.double() - b.double()).norm() / b.double().norm())


def _weights(part_spec, prefix="m.", seed=0, std=0.08):
    from ember_b200.parts import build_part
    g = torch.Generator().manual_seed(seed)
    out = {}
    for d in build_part("mixer", part_spec, prefix).weight_decls():
        if d.init == "norm":
            t = 1 + 0.1 * torch.randn(d.shape, generator=g)
        elif d.init == "uniform":
            t = d.lo + (d.hi - d.lo) * torch.rand(d.shape, generator=g)
        else:
            t = std * torch.randn(d.shape, generator=g)
        out[d.name] = t.bfloat16()
    return out


MIX_TOL = {torch.float32: 2e-5, torch.bfloat16: 2e-2}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv,dim,vdim,taps,hidden", [(4, 2, 24, 40, 3, 64), (2, 2, 70, 130, 4, 100), (3, 1, 128, 64, 2, 128)])
def test_channel_delta_alone(dtype, heads, kv, dim, vdim, taps, hidden):
    from ember_b200.config import GatedDeltaSpec
    spec = GatedDeltaSpec(hidden_size=hidden, num_heads=heads, num_kv_heads=kv, head_dim=dim, value_dim=vdim, conv_taps=taps,
                          decay_rank=8, gate_rank=16, norm_eps=1e-5)
    w = _weights(spec, seed=heads)
    x = torch.randn(90, hidden, generator=torch.Generator().manual_seed(2)).bfloat16()
    want = plain.channel_delta(x.double(), {k: v.double() for k, v in w.items()}, "m.",
                               {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim}, 1e-5)
    assert _rel(_run_mixer(spec, w, x, dtype), want) < MIX_TOL[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,dim,vdim,cap,hidden", [(3, 16, 32, 8.0, 64), (1, 40, 72, 15.0, 100), (2, 128, 256, 3.0, 128)])
def test_matrix_memory_alone(dtype, heads, dim, vdim, cap, hidden):
    from ember_b200.config import MatrixMemorySpec
    spec = MatrixMemorySpec(hidden_size=hidden, num_heads=heads, head_dim=dim, value_dim=vdim, gate_cap=cap, norm_eps=1e-6)
    w = _weights(spec, seed=heads, std=0.15)
    w["m.i"] = (w["m.i"].float() * 20).bfloat16()           # input gates that reach the cap and move the maximum
    x = torch.randn(90, hidden, generator=torch.Generator().manual_seed(3)).bfloat16()
    want = plain.mlstm(x.double(), {k: v.double() for k, v in w.items()}, "m.",
                       {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}, 1e-6)
    assert _rel(_run_mixer(spec, w, x, dtype), want) < MIX_TOL[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,vdim,state,groups,parts,taps,hidden", [(4, 20, 16, 1, 1, 2, 64), (6, 12, 8, 3, 3, 5, 100),
                                                                       (8, 64, 128, 2, 4, 4, 128), (2, 36, 40, 2, 1, 1, 72)])
def test_state_space_alone(dtype, heads, vdim, state, groups, parts, taps, hidden):
    from ember_b200.config import StateSpaceSpec
    spec = StateSpaceSpec(hidden_size=hidden, num_heads=heads, value_dim=vdim, state_size=state, num_groups=groups,
                          norm_groups=parts, conv_taps=taps, norm_eps=1e-6)
    w = _weights(spec, seed=heads)
    w["m.conv.b"] = (0.2 * torch.randn(w["m.conv.b"].shape, generator=torch.Generator().manual_seed(9))).bfloat16()
    x = torch.randn(90, hidden, generator=torch.Generator().manual_seed(4)).bfloat16()
    want = plain.mamba2(x.double(), {k: v.double() for k, v in w.items()}, "m.",
                        {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "norm_groups": parts}, 1e-6)
    assert _rel(_run_mixer(spec, w, x, dtype), want) < MIX_TOL[dtype]


def _attention_spec(heads, kv, dim, vdim, rot, base, scale, hidden):
    from ember_b200.config import RotarySpec, SigmoidAttentionSpec
    return SigmoidAttentionSpec(hidden_size=hidden, num_heads=heads, num_kv_heads=kv, head_dim=dim, value_dim=vdim, scale=scale,
                                position=RotarySpec(head_dim=dim, rotary_dim=rot, theta=base, frequency_precision="float64"))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv,dim,vdim,rot,base,hidden", [(6, 2, 32, 24, 16, 1e4, 64), (2, 2, 64, 160, 64, 500.0, 100),
                                                                (4, 1, 128, 256, 64, 2.5e5, 128), (3, 3, 20, 300, 2, 77.0, 72)])
def test_sigmoid_attention_alone(dtype, heads, kv, dim, vdim, rot, base, hidden):
    spec = _attention_spec(heads, kv, dim, vdim, rot, base, 0.3, hidden)
    w = _weights(spec, seed=heads)
    x = torch.randn(90, hidden, generator=torch.Generator().manual_seed(5)).bfloat16()
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": 0.3, "rot": {"dims": rot, "base": base}}
    want = plain.sigmoid_attention(x.double(), {k: v.double() for k, v in w.items()}, "m.", m)
    assert _rel(_run_mixer(spec, w, x, dtype), want) < MIX_TOL[dtype]


def test_a_far_key_that_dominates_is_seen_across_pages_and_portions():
    """Head biases so low that ordinary keys weigh nothing, one early key and two late queries scaled so that their
    scores stand out: the read-out at those queries is that one key's value, in a prompt portion and decoded alone."""
    heads, kv, dim, vdim, hidden, T, far = 2, 1, 32, 48, 64, 200, 3
    spec = _attention_spec(heads, kv, dim, vdim, 8, 1e4, 1.0, hidden)
    w = _weights(spec, seed=3, std=0.05)
    w["m.pb"] = torch.full((heads,), -30.0).bfloat16()
    eye = torch.zeros(dim, hidden)
    eye[8:, :dim - 8] = torch.eye(dim - 8)                   # the elements that are not rotated copy the input
    w["m.q"], w["m.k"] = torch.cat([eye] * heads).bfloat16(), eye.bfloat16()
    x = 0.1 * torch.randn(T, hidden, generator=torch.Generator().manual_seed(6))
    x[far, :dim - 8] = 3.0
    for t in (150, 199):
        x[t, :dim - 8] = 3.0
    x = x.bfloat16()
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": 1.0, "rot": {"dims": 8, "base": 1e4}}
    W = {k: v.double() for k, v in w.items()}
    want = plain.sigmoid_attention(x.double(), W, "m.", m)
    without = plain.sigmoid_attention(torch.cat([x[:far], torch.zeros(1, hidden).bfloat16(), x[far + 1:]]).double(), W, "m.", m)
    # (the query's own key scores as high as the far one: the far key is half of what is read)
    assert float((want[150] - without[150]).norm() / want[150].norm()) > 0.4
    got = _run_mixer(spec, w, x, torch.float32, portions=((120, 3), (40, 30), (38, 1), (1, 1), (1, 1)))
    for t in (150, 199):
        assert _rel(got[t], want[t]) < 1e-4
    assert _rel(got, want) < 1e-4


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_layer_norm_gate_and_sandwich_kernels(dtype):
    """layer_norm, the fused gate + norm + add, and the per-group norm with both kinds of gate."""
    from ember_b200 import ops
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(8)
    for H in (96, 100, 1000):
        x = (3 * torch.randn(11, H, generator=g) + 1.5).to(dev)
        w, b = (1 + 0.1 * torch.randn(H, generator=g)).to(dev), (0.1 * torch.randn(H, generator=g)).to(dev)
        out = torch.empty(11, H, device=dev, dtype=dtype)
        ops.layer_norm(x, w, b, 1e-5, out, 11)
        want = plain.layer_norm(x.cpu().double(), w.cpu(), b.cpu(), 1e-5)
        assert _rel(out.float().cpu(), want) < (5e-3 if dtype == torch.bfloat16 else 1e-6)
        y, logits, gb = torch.randn(11, H, generator=g).to(dev), torch.randn(11, H, generator=g).to(dev), torch.randn(H, generator=g).to(dev)
        res = x.clone()
        ops.gated_norm_add(y, logits, w, b, 1e-5, True, res, 11, gate_bias=gb)
        want = x.cpu().double() + plain.layer_norm(y.cpu().double() * torch.sigmoid((logits + gb).cpu().double()), w.cpu(), b.cpu(), 1e-5)
        assert _rel(res.cpu(), want) < 1e-6
    for T, groups, V in ((9, 3, 44), (5, 2, 600)):            # a warp per short group, a block per wide one
        o, gate = torch.randn(T, groups * V + 5, generator=g).to(dev), torch.randn(T, 7 + groups * V, generator=g).to(dev)
        for per_group, mode in ((True, ops.GATE_SIGMOID_AFTER), (False, ops.GATE_SILU_BEFORE), (False, ops.GATE_NONE)):
            w = (1 + 0.1 * torch.randn(groups * V if per_group else V, generator=g)).to(dev)
            out = torch.empty(T, groups * V, device=dev, dtype=dtype)
            ops.group_norm_gate(o, 5, gate, 7, w, per_group, 1e-6, mode, out, T, groups, V)
            v, z = o[:, 5:].cpu().double().view(T, groups, V), gate[:, 7:].cpu().double().view(T, groups, V)
            if mode == ops.GATE_SILU_BEFORE:
                v = v * plain.silu(z)
            want = plain.rms_div(v, 1e-6) * (w.cpu().double().view(groups, V) if per_group else w.cpu().double())
            if mode == ops.GATE_SIGMOID_AFTER:
                want = want * torch.sigmoid(z)
            assert _rel(out.float().cpu().view(T, groups, V), want) < (5e-3 if dtype == torch.bfloat16 else 1e-6)


# ------------------------------------------------------------------------ through the programs
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(dtype, dirs, plain_logits, tmp_path):
    """bin/trace_run as a user runs it (config.json without the low-rank sizes, four state slots, steps on standard
    input): portions beside single tokens of up to four live requests, and a step larger than any one batch."""
    import subprocess
    import sys
    root = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..")
    requests = make_requests("q", (300, 41, 75, 2, 33, 64), seed=9)
    steps = trace_mixed(requests, live=4, seed=1, max_portion=70)
    out = tmp_path / "out"
    proc = subprocess.run(
        [sys.executable, os.path.join(root, "bin", "trace_run"), "--model", dirs["q"], "--dtype", dtype, "--out", str(out),
         "--max-tokens", str(max_live_tokens(steps))],
        input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done ")] == [f"done {s['step']}" for s in steps]
    vocab = FADOSUN["q"]["json"]["vocab"]
    outputs = {s["step"]: np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(-1, vocab) for s in steps}
    assert_close(collect(steps, outputs), plain_logits("q", requests), dtype, "trace_run")


# ------------------------------------------------------------------------ through the entry point
def test_greedy_generation_through_the_engine(dirs):
    """Greedy tokens from ``ember_b200.load(...).generate`` (scheduler, portions of 16, few pages, four prompts of
    unequal length) against greedy decoding with the plain implementation."""
    import ember_b200
    cfg, W = plain_inputs(dirs["p"])
    prompts = list(make_requests("p", (5, 40, 1, 23), seed=31).values())
    llm = ember_b200.load(dirs["p"], dtype="float32", kv_cache_tokens=256, max_batch_tokens=64, max_seqs=3, prefill_chunk=16,
                          page_tokens=16)
    got = llm.generate(prompts, max_tokens=12, ignore_eos=True)
    for p, ids in zip(prompts, got):
        seq = list(p)
        for _ in range(12):
            seq.append(int(plain.forward(cfg, W, seq)[-1].argmax()))
        assert list(ids) == seq[len(p):]
    assert llm.runner.cache.check() == ""
