"""Petanex without a GPU: configuration and weights, and the engine's host logic (pages, state slots, portions,
mixed batches) with the kernels replaced by the CPU stand-in, against the plain implementation."""
import json

import pytest
import torch

import helpers
import petanex_cases as px
import plain_petanex
from kungfu_b200 import api, registry
from kungfu_b200.config.base import ConfigError
from kungfu_b200.weights.store import WeightError, WeightStore


def _runner(folder, page, max_tokens, max_requests=4):
    cfg, model = api.load_model(folder, dtype="float32", device="cpu")
    return api.make_runner(cfg, model, dtype="float32", device="cpu", page_size=page, max_tokens=max_tokens,
                           max_requests=max_requests, max_context=512)


def _rel(got, ref):
    assert got
    scale = max(float(r.abs().max()) for r in ref.values())
    return max(float((row - ref[rid][pos].float()).abs().max()) for (rid, pos), row in got.items()) / scale


def test_config_reads_every_size_and_round_trips():
    cfg = api.load_config(dict(px.PX_A))
    assert cfg.architecture == "Petanex" and cfg.width == 64 and cfg.vocab == 300 and len(cfg.layers) == 4 and cfg.side_dim == 8
    d = cfg.layers[0].mixer
    assert (d.heads, d.kv_heads, d.dim, d.vdim, d.conv, d.decay_rank) == (4, 2, 16, 24, 3, None)
    f = cfg.layers[0].mlp
    assert (f.kind, f.experts, f.top, f.scale, f.groups, f.keep, f.expert.ff, f.expert.limit, f.shared.ff, f.shared.limit) == \
        ("moe", 8, 2, 2.0, 4, 2, 32, 1.0, 48, 2.0)
    a = cfg.layers[1].mixer
    assert (a.heads, a.dim, a.vdim, a.kv_rank, a.scale) == (4, 16, 24, 20, 0.3)
    assert cfg.layers[2].mlp is None and cfg.layers[3].mlp.shared is None and cfg.layers[3].mlp.groups == 1
    assert api.load_config(cfg.to_dict()) == cfg
    assert api.load_config(json.loads(json.dumps(cfg.to_dict()))) == cfg
    assert api.load_config(dict(px.PX_B)).side_dim == 0
    kinds = [s["kind"] for s in cfg.state_summary()]
    assert kinds == ["recurrent+conv_tail", "latent_cache", "recurrent+conv_tail", "latent_cache"]


@pytest.mark.parametrize("change,word", [
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][0].update(type="attention"), "type"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=9), "top"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=3), "groups"),
    (lambda c: c["layers"][0]["mlp"]["expert"].pop("limit"), "limit"),
    (lambda c: c["norm"].pop("eps"), "eps"),
])
def test_config_errors_name_the_key(change, word):
    raw = json.loads(json.dumps(px.PX_A))
    change(raw)
    with pytest.raises(ConfigError) as e:
        api.load_config(raw)
    assert word in str(e.value)


def test_weights_bind_by_name_ranks_come_from_shapes_and_faults_are_listed_together():
    cfg = api.load_config(dict(px.PX_A))
    arch = registry.find("Petanex")
    t = px.draw_tensors(px.PX_A, 1, ranks=(5, 7))
    assert t["l2.mix.a1"].shape == (5, 64) and t["l2.mix.g2"].shape == (3 * 12, 7) and t["side.embed"].shape == (300, 4 * 8)
    assert "l2.norm2" not in t and "l3.mlp.shared.gate" not in t and "l0.mlp.e7.down" in t
    model = arch.build(cfg, WeightStore.from_tensors(t, device="cpu", compute_dtype=torch.float32))
    m = model.layers[2].mixer
    assert (m.a_width, m.g_width, m.per_channel, m.gate) == (5, 7, True, "sigmoid")
    assert model.layers[0].mixer.gate == "silu" and model.layers[1].mixer.head_dim == 32 and model.layers[3].mixer.head_dim == 16
    assert model.head.weight.data_ptr() == model.embedding.table.data_ptr()
    bad = dict(t)
    del bad["l1.mix.uk"]
    bad["l0.mix.b"] = torch.zeros(5, 64, dtype=torch.bfloat16)
    bad["extra"] = torch.zeros(1)
    with pytest.raises(WeightError) as e:
        arch.build(cfg, WeightStore.from_tensors(bad, device="cpu", compute_dtype=torch.float32))
    assert "l1.mix.uk" in e.value.missing or any(n == "l0.mix.b" for n, _, _ in e.value.wrong_shape)


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
@pytest.mark.parametrize("mode", ["whole", "chunks", "mixed"])
def test_host_logic_on_the_cpu_stand_in(name, mode, tmp_path, cpu_ops):
    cfg, lengths, page = px.CASES[name]
    folder = px.write_model(str(tmp_path / "m"), cfg, seed=3, sharp=True, ranks=px.RANKS[name])
    reqs = {f"r{i}": helpers.random_tokens(n, cfg["vocab"], 100 + i) for i, n in enumerate(lengths)}
    tensors = helpers.read_tensors(folder)
    ref = {rid: plain_petanex.forward(cfg, tensors, toks).float() for rid, toks in reqs.items()}
    steps = {"whole": helpers.trace_whole, "chunks": helpers.trace_chunks, "mixed": lambda r: helpers.trace_mixed(r, seed=4)}[mode](reqs)
    runner = _runner(folder, page, helpers.trace_max_tokens(steps, page))
    got = helpers.run_trace_with_runner(runner, steps)
    assert len(got) == sum(lengths)
    assert _rel(got, ref) < 3e-4
    assert runner.cache.n_live == 0
    runner.cache.check()


def test_the_router_alone_against_a_hand_count():
    """Groups decide before experts do: an expert with the largest choice score loses when its group's best two sum lower;
    the weights use the scores without the correction."""
    f = {"router": {"experts": 6, "top": 2, "scale": 3.0, "groups": {"count": 3, "keep": 1}}}
    logits = torch.tensor([[4.0, -9.0, 1.0, 1.2, -3.0, -3.0]], dtype=torch.float64)
    t = {"p.router": torch.eye(6), "p.correction": torch.tensor([0.0, 0.0, 0.3, 0.0, 0.0, 0.0])}
    ids, w = plain_petanex.route(logits, f, t, "p.")
    s = torch.sigmoid(logits[0])
    assert sorted(ids[0].tolist()) == [2, 3]                       # group 1 (0.73 + 0.3 + 0.77) beats group 0 (0.98 + 0.0001)
    pair = {int(i): float(x) for i, x in zip(ids[0], w[0])}
    assert abs(pair[2] - float(s[2] / (s[2] + s[3]) * 3.0)) < 1e-12 and abs(pair[3] - float(s[3] / (s[2] + s[3]) * 3.0)) < 1e-12
