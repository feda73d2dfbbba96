"""Darotar on the host backend: configuration, plan and weights; the engine's cache, pages and batching with the design's
mixers and routed experts against the plain whole-sequence implementation (no GPU: the kernels' plain statements of
tests/torch_ops.py stand in for them)."""
import json
import os

import pytest
import torch

from darotar_util import CFG_A, CFG_B, attention, latent, moe, plain_logits, read_model, tokens, write_model
from torch_ops import TorchOps


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {"A": write_model(str(tmp_path_factory.mktemp("dar_a")), CFG_A, 11),
            "B": write_model(str(tmp_path_factory.mktemp("dar_b")), CFG_B, 12)}


def host_engine(folder, page=4, pages=64, slots=4):
    from nanoinfer_b200.config import EngineConfig
    from nanoinfer_b200.engine import Engine
    return Engine(folder, EngineConfig(dtype="float32", page_size=page, num_pages=pages, max_batch=slots, device="cpu",
                                       cuda_graphs=False), ops=TorchOps())


def run_cut(eng, name, ids, cuts):
    """The request fed in portions of the given sizes; logits of every position."""
    from nanoinfer_b200.engine import StepEntry
    rc = eng.open(name)
    out, pos = [], 0
    for n in cuts:
        out.append(eng.step([StepEntry(rc, ids[pos:pos + n], list(range(n)))]))
        pos += n
    assert pos == len(ids)
    eng.close(rc)
    return torch.cat(out).double()


def close(a, b, tol=2e-4):
    assert a.shape == b.shape
    assert (a - b).abs().max().item() <= tol * max(1.0, b.abs().max().item()), (a - b).abs().max().item()


def test_config_reads_every_key_and_round_trips(folders):
    from nanoinfer_b200.config.model_config import read_config_json
    from nanoinfer_b200.registry import config_from_json_dict, plan_for
    cfg = config_from_json_dict(read_config_json(folders["A"]))
    assert cfg.architecture == "Darotar" and cfg.vocab_size == 131 and cfg.hidden_size == 64
    assert cfg.norm_eps == 1e-6 and cfg.residual_mult == 0.7
    plan = plan_for(cfg)
    assert all(layer.arrangement == "output_norm" and layer.params == {"mult": 0.7} for layer in plan.layers)
    first = plan.layers[0].parts["mixer"]
    assert first.kind == "flex_attention" and first.params["rot"] == (8, 500.0) and first.params["rot_factor"] == 2.0
    assert first.params["rot_layout"] == "interleaved" and first.params["unit_norm_after_rot"] and first.params["values_from_keys"]
    assert first.params["window"] == 5 and first.params["scale"] == 0.25 and "v" not in first.tensors
    assert plan.layers[0].parts["ffn"].params == {"hidden": 64, "ff": 24, "experts": 5, "top": 2}
    second, third = plan.layers[1].parts["mixer"], plan.layers[2].parts["mixer"]
    assert second.kind == "latent_attention" and second.params["sink"] and second.params["out_gate"] and second.params["owns_kv"]
    assert "ffn" not in plan.layers[1].parts and "ffn_norm" not in plan.layers[1].parts
    assert not third.params["owns_kv"] and "dkv" not in third.tensors and plan.schedule[2].reads_cache_of == 1
    assert third.params["heads"] == 2 and third.params["vdim"] == 10 and third.params["q_rank"] == 7
    assert plan.positions[second.params["position"]].params["layout"] == "half"
    assert plan.lm_head.tensors["weight"].name == "head" and [t.name for t in plan.final_norm.tensors.values()] == ["final.norm"]
    again = config_from_json_dict(json.loads(json.dumps(cfg.to_json_dict())))
    assert again == cfg


def test_config_refuses_what_it_cannot_run():
    from nanoinfer_b200.config.model_config import ConfigError
    from nanoinfer_b200.registry import config_from_json_dict

    def changed(fn):
        bad = json.loads(json.dumps(CFG_A))
        fn(bad)
        return bad

    for fn in (lambda c: c["layers"][0]["mixer"].update(heads=3),                 # no multiple of its two kv heads
               lambda c: c["layers"][1].update(type="attention_2"),
               lambda c: c["layers"][0]["mixer"]["rot"].update(dims=14),          # wider than the head
               lambda c: c["layers"][0]["mixer"].update(vdim=8),                  # values are the keys: one width
               lambda c: c["layers"][1]["mixer"]["rot"].update(dims=2),           # the rotated part is turned as a whole
               lambda c: c["layers"][2]["mixer"].update(kv_from=3),               # a later layer
               lambda c: c["layers"][2]["mixer"].update(kv_from=0),               # a layer that caches no latent
               lambda c: c["layers"][2]["mixer"].update(kv_rank=16),              # not the cached rows' width
               lambda c: c["layers"][0]["mlp"]["router"].update(top=6),           # more than there are experts
               lambda c: c["layers"][0]["mlp"].update(kind="dense"),
               lambda c: c.pop("norm")):
        with pytest.raises(ConfigError):
            config_from_json_dict(changed(fn))


def test_loader_names_missing_and_misshapen_tensors(folders, tmp_path):
    from nanoinfer_b200.weights.loader import WeightError
    from nanoinfer_b200.weights.safetensors_io import save_safetensors
    cfg, w = read_model(folders["B"])
    del w["l0.mix.sink"]
    w["l1.mlp.e3.down"] = torch.zeros(5, 5, dtype=torch.bfloat16)
    with open(os.path.join(tmp_path, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_safetensors(os.path.join(tmp_path, "model.safetensors"), w)
    with pytest.raises(WeightError) as e:
        host_engine(str(tmp_path))
    assert "l0.mix.sink" in str(e.value) and "l1.mlp.e3.down" in str(e.value)


def test_pages_the_model_asks_for(folders):
    eng = host_engine(folders["A"])
    needs = eng.model.cache_needs()
    assert [t.width for t in needs[0][0].tensors] == [12, 12] and needs[0][0].window == 5 and needs[0][1] is None
    assert [(t.heads, t.width) for t in needs[1][0].tensors] == [(1, 16)] and needs[1][0].window == 0
    assert needs[3][0].window == 300 and [(t.heads, t.width) for t in needs[4][0].tensors] == [(1, 8)]


@pytest.mark.parametrize("name,n", [("A", 37), ("B", 29)])
def test_whole_prompt_equals_plain(folders, name, n):
    ids = tokens(n, 77, 5)
    close(run_cut(host_engine(folders[name]), "r", ids, [n]), plain_logits(folders[name], ids))


@pytest.mark.parametrize("name", ["A", "B"])
def test_token_by_token_and_portions_down_to_two(folders, name):
    ids = tokens(31, 77, 6)
    ref = plain_logits(folders[name], ids)
    eng = host_engine(folders[name])
    close(run_cut(eng, "one", ids, [1] * 31), ref)
    close(run_cut(eng, "cut", ids, [2, 5, 2, 9, 1, 1, 7, 2, 2]), ref)
    close(run_cut(eng, "tail", ids, [20] + [1] * 11), ref)
    eng.cache.check()


def test_unequal_requests_in_one_batch_and_reused_slots_and_pages(folders):
    """Requests of different lengths advance together in portions and single tokens; when one ends, another takes its
    slot and pages (two slots only, a pool that forces reuse)."""
    from nanoinfer_b200.engine import StepEntry
    eng = host_engine(folders["A"], page=4, pages=24, slots=2)
    seqs = {k: tokens(n, 131, s) for k, n, s in (("p", 23, 1), ("q", 9, 2), ("r", 17, 3), ("s", 12, 4))}
    ref = {k: plain_logits(folders["A"], v) for k, v in seqs.items()}
    got, at, live, slots_used = {k: [] for k in seqs}, {k: 0 for k in seqs}, {}, {}
    plan = [[("p", 6), ("q", 2)], [("p", 1), ("q", 5)], [("p", 7), ("q", 2)], [("p", 1), ("r", 9)], [("r", 1), ("p", 1)],
            [("p", 7), ("r", 7)], [("s", 3)], [("s", 1)], [("s", 8)]]
    for step in plan:
        entries = []
        for k, n in step:
            if k not in live:
                live[k] = eng.open(k)
                slots_used[k] = live[k].slot
            entries.append(StepEntry(live[k], seqs[k][at[k]:at[k] + n], list(range(n))))
        logits = eng.step(entries).double()
        row = 0
        for k, n in step:
            got[k].append(logits[row:row + n])
            row += n
            at[k] += n
            if at[k] == len(seqs[k]):
                eng.close(live.pop(k))
        eng.cache.check()
    assert slots_used["r"] == slots_used["q"] and slots_used["s"] in (slots_used["p"], slots_used["r"])
    for k in seqs:
        close(torch.cat(got[k]), ref[k])


def test_pages_behind_a_window_go_back_to_the_pool(tmp_path):
    """A model of windowed layers only: a long request holds no more pages than its window needs."""
    cfg = {"architecture": "Darotar", "vocab": 50, "width": 32, "norm": {"eps": 1e-6}, "residual_mult": 0.8, "layers": [
        attention(2, 1, 8, 8, 100.0, factor=2.0, window=6, mlp=moe(3, 1, 16))]}
    d = write_model(str(tmp_path), cfg, 3)
    eng = host_engine(d, page=2, pages=8, slots=1)
    ids = tokens(40, 50, 9)
    close(run_cut(eng, "long", ids, [3, 2] + [1] * 35), plain_logits(d, ids))
    eng.cache.check()


def test_a_latent_read_by_later_layers_is_cached_once(tmp_path):
    """Two layers read the first layer's rows: the pool is sized for one set of pages, and a request longer than a
    second set would allow still runs."""
    layers = [latent(2, 8, 4, 8, 8, 12, 1000.0, mlp=moe(2, 1, 16)), latent(3, 4, 4, 4, 6, 12, 1000.0, kv_from=0),
              latent(1, 8, 4, 16, 8, 12, 1000.0, kv_from=0, mlp=moe(2, 2, 8))]
    cfg = {"architecture": "Darotar", "vocab": 40, "width": 24, "norm": {"eps": 1e-6}, "residual_mult": 1.0, "layers": layers}
    d = write_model(str(tmp_path), cfg, 4)
    eng = host_engine(d, page=4, pages=6, slots=1)
    assert sum(1 for need in eng.model.cache_needs() if need[0] is not None) >= 1
    ids = tokens(23, 40, 2)
    close(run_cut(eng, "x", ids, [9, 2, 1, 1, 10]), plain_logits(d, ids))
    eng.cache.check()


def test_the_sink_takes_weight_and_the_gate_scales(tmp_path):
    """One latent layer: a large sink must shrink the mixer's output as the plain softmax says, and a closed gate must
    remove it (the logits then come from the embedding alone)."""
    cfg = {"architecture": "Darotar", "vocab": 40, "width": 24, "norm": {"eps": 1e-6}, "residual_mult": 1.0, "layers": [
        latent(2, 8, 4, 8, 8, 12, 1000.0)]}
    ids = tokens(9, 40, 1)
    refs = []
    for name, change in (("plain", lambda t: None), ("sink", lambda t: t["l0.mix.sink"].fill_(6.0)),
                         ("small", lambda t: t["l0.mix.sink"].fill_(-20.0))):
        d = write_model(str(tmp_path / name), cfg, 4, weights=change)
        ref = plain_logits(d, ids)
        close(run_cut(host_engine(d), "x", ids, [4, 1, 4]), ref)
        refs.append(ref)
    assert (refs[0] - refs[1]).abs().max().item() > 1e-2 and (refs[0] - refs[2]).abs().max().item() > 1e-3


def test_a_score_multiplies_the_experts_input_and_is_not_renormalized(tmp_path):
    """Router logits far below zero: the chosen experts' scores are tiny, and so is what the experts add (a weight on the
    output would scale it linearly, a renormalized one not at all; on the input it enters the gate twice)."""
    cfg = {"architecture": "Darotar", "vocab": 40, "width": 24, "norm": {"eps": 1e-2}, "residual_mult": 1.0, "layers": [
        attention(2, 1, 8, 4, 100.0, factor=2.0, window=4, mlp=moe(4, 2, 16))]}

    def low(t):
        t["l0.mlp.router"].mul_(0.05)

    ids = tokens(11, 40, 1)
    for name, change in (("as_is", lambda t: None), ("low", low)):
        d = write_model(str(tmp_path / name), cfg, 6, weights=change)
        close(run_cut(host_engine(d), "x", ids, [5, 1, 1, 4]), plain_logits(d, ids))


def test_greedy_generation_through_the_scheduler(folders):
    """The framework's own entry point: a Model, its Scheduler with a small token budget (prompts go in portions,
    requests join and leave), three slots."""
    from nanoinfer_b200.api import Model
    from nanoinfer_b200.config import EngineConfig
    from nanoinfer_b200.engine.scheduler import Request, Scheduler
    model = Model(folders["B"], EngineConfig(dtype="float32", page_size=4, num_pages=64, max_batch=3, max_tokens_per_step=8,
                                             device="cpu", cuda_graphs=False), ops=TorchOps())
    sched = Scheduler(model)
    prompts = [tokens(13, 77, 21), tokens(5, 77, 22), tokens(19, 77, 23), tokens(3, 77, 24)]
    for i, p in enumerate(prompts):
        sched.add(Request(f"g{i}", p, max_tokens=6))
    done = sched.run()
    for i, p in enumerate(prompts):
        ids = list(p)
        for _ in range(6):
            ids.append(int(plain_logits(folders["B"], ids)[-1].argmax()))
        assert done[f"g{i}"] == ids[len(p):], i
    model.engine.cache.check()
