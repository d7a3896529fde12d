"""Bolonex without a GPU: configuration and weights, and the engine's host logic (pages, state slots, portions,
mixed batches, the scheduler) with the kernels replaced by the CPU stand-in, against the plain implementation."""
import json

import pytest
import torch

import bolonex_cases as bx
import helpers
import plain_bolonex
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


# ---- configuration ----------------------------------------------------------------------------------------------

def test_config_reads_every_size_and_round_trips():
    cfg = api.load_config(dict(bx.BX_B))
    assert cfg.architecture == "Bolonex" and cfg.width == 96 and cfg.vocab == 257 and len(cfg.layers) == 5
    a = cfg.layers[2].mixer
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.conv, a.scale, a.softcap) == (3, 3, 32, 16, 4, 0.2, 10.0)
    assert a.rot.scaling == (8.0, 1.0, 4.0, 64.0) and a.rot.dims == 32
    m = cfg.layers[4].mixer
    assert (m.heads, m.vdim, m.state, m.groups, m.norm_groups, m.conv) == (4, 24, 24, 4, 1, 2)
    assert cfg.layers[1].mlp is None and cfg.layers[0].mlp.ff == 160
    assert cfg.source_of(0) == 2 and cfg.source_of(3) == 1 and cfg.source_of(4) == 4
    assert api.load_config(cfg.to_dict()) == cfg
    assert api.load_config(json.loads(json.dumps(cfg.to_dict()))) == cfg


@pytest.mark.parametrize("change,word", [
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["layers"][1]["mixer"].pop("state"), "state"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=2), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=33), "rot.dims"),
    (lambda c: c["layers"][0].update(type="hyena"), "type"),
    (lambda c: c["layers"][1].update(weights_of=0), "weights"),
    (lambda c: c["layers"][1]["mixer"].update(norm_groups=5), "norm_groups"),
    (lambda c: c["norm"].pop("eps"), "eps"),
])
def test_config_errors_name_the_key(change, word):
    raw = json.loads(json.dumps(bx.BX_B))
    change(raw)
    with pytest.raises(ConfigError) as e:
        api.load_config(raw)
    assert word in str(e.value)


def test_weights_bind_by_name_and_faults_are_listed_together():
    cfg = api.load_config(dict(bx.BX_A))
    arch = registry.find("Bolonex")
    names = [s.name for s in arch.tensor_specs(cfg)]
    assert "l0.mix.in" in names and "l1.mix.q.conv" in names and not any(n.startswith(("l2.", "l3.")) for n in names)
    assert "l1.mlp.up" not in names and "l0.mlp.up" in names
    t = bx.draw_tensors(bx.BX_A, 1)
    model = arch.build(cfg, WeightStore.from_tensors(t, device="cpu", compute_dtype=torch.float32))
    assert len(model.schedule) == 4 and [c.layer for c in model.schedule] == [0, 1, 0, 1]
    assert [c.cache for c in model.schedule] == [0, 1, 2, 3] and len(model.state_needs()) == 4
    bad = dict(t)
    del bad["l1.mix.g"]
    bad["l0.mix.A_log"] = torch.zeros(3)
    bad["extra"] = torch.zeros(2)
    with pytest.raises(WeightError) as e:
        arch.build(cfg, WeightStore.from_tensors(bad, device="cpu", compute_dtype=torch.float32))
    assert e.value.missing == ["l1.mix.g"] and e.value.unexpected == ["extra"] and e.value.wrong_shape[0][0] == "l0.mix.A_log"


def test_rotary_frequencies_keep_scale_and_blend():
    from kungfu_b200.parts import Rope
    rot = bx.BX_B["layers"][2]["mixer"]["rot"]
    ours = Rope(32, rot["base"], "cpu", rot["dims"], interleaved=True, scaling=rot["scaling"]).inv_freq.double()
    ref = plain_bolonex.rotary_frequencies(rot)
    plain = plain_bolonex.rotary_frequencies({"base": rot["base"], "dims": rot["dims"]})
    kinds = {"kept": 0, "divided": 0, "blended": 0}
    for f, p in zip(ref.tolist(), plain.tolist()):
        kinds["kept" if f == p else "divided" if abs(f - p / 8.0) < 1e-12 * p else "blended"] += 1
    assert all(v > 0 for v in kinds.values()), kinds          # the test's constants reach all three regimes
    assert float(((ours - ref) / ref).abs().max()) < 1e-7


# ---- the engine's host logic against the plain implementation ---------------------------------------------------------

@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name, (cfg, lengths, page) in bx.CASES.items():
        folder = bx.write_model(str(tmp_path_factory.mktemp(name) / "m"), cfg, seed=7, sharp=True)
        reqs = {f"r{i}": helpers.random_tokens(n, cfg["vocab"], 100 + i) for i, n in enumerate(lengths)}
        tensors = helpers.read_tensors(folder)
        ref = {rid: plain_bolonex.forward(cfg, tensors, toks) for rid, toks in reqs.items()}
        out[name] = (folder, cfg, reqs, ref, page)
    return out


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
@pytest.mark.parametrize("mode", ["whole", "tail", "chunks", "mixed"])
def test_cpu_modes_match_plain(models, cpu_ops, name, mode):
    folder, cfg, reqs, ref, page = models[name]
    steps = {"whole": helpers.trace_whole, "tail": lambda r: helpers.trace_decode_tail(r, 12),
             "chunks": helpers.trace_chunks, "mixed": lambda r: helpers.trace_mixed(r, seed=3)}[mode](reqs)
    runner = _runner(folder, page, helpers.trace_max_tokens(steps, page))
    got = helpers.run_trace_with_runner(runner, steps)
    assert len(got) == sum(len(t) for t in reqs.values())
    assert _rel(got, ref) < 2e-4
    assert runner.cache.n_live == 0
    assert all(f == g.pool.n_pages for f, g in zip(runner.cache.free_pages(), runner.cache.groups))
    if mode == "mixed":                                    # six requests went through four state slots
        assert all(n > g.pool.n_pages for n, g in zip(runner.cache.pages_handed_out(), runner.cache.groups))


def test_a_slot_that_is_used_again_starts_from_zero(models, cpu_ops):
    """The fixed-size states (recurrent memory, convolution tails) of a request that ended must not leak into the
    request that gets its slot: one slot, three requests one after the other."""
    folder, cfg, reqs, ref, page = models["A"]
    runner = _runner(folder, page, 64, max_requests=1)
    from kungfu_b200.engine import StepEntry
    for rid in ("r1", "r2", "r1"):
        toks = reqs[rid]
        runner.cache.add_request(rid)
        assert runner.cache.state_slot(rid) == 0
        a = runner.step([StepEntry(rid, toks[:5], [4])]).clone()
        b = runner.step([StepEntry(rid, toks[5:], [len(toks) - 6])]).clone()
        runner.cache.release(rid)
        scale = float(ref[rid].abs().max())
        assert float((a[0] - ref[rid][4].float()).abs().max()) / scale < 2e-4
        assert float((b[0] - ref[rid][len(toks) - 1].float()).abs().max()) / scale < 2e-4


def test_generate_through_the_engine_matches_plain_greedy(models, cpu_ops):
    from kungfu_b200.engine.engine import Engine
    from kungfu_b200.sampling import Sampling
    folder, cfg, reqs, _, page = models["B"]
    tensors = helpers.read_tensors(folder)
    cfg_, model = api.load_model(folder, dtype="float32", device="cpu")
    runner = api.make_runner(cfg_, model, dtype="float32", device="cpu", page_size=page, max_tokens=256, max_requests=3,
                             max_context=128)
    eng = Engine(runner=runner, batch=16, parallel=3)
    prompts = [reqs["r1"], reqs["r4"], reqs["r2"][:20], reqs["r0"]]
    outs = eng.generate(prompts, Sampling(temperature=0.0), max_tokens=6, ignore_eos=True)
    for p, o in zip(prompts, outs):
        seq = list(p)
        for tok in o:
            logits = plain_bolonex.forward(cfg, tensors, seq)[-1]
            top = torch.topk(logits, 2).values
            if float(top[0] - top[1]) > 1e-3 * float(logits.abs().max()):     # a near tie may fall either way
                assert int(torch.argmax(logits)) == tok
            seq.append(tok)
        assert len(o) == 6
