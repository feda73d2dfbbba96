"""Dusilorn on the host backend: configuration, plan and weights; the engine's cache, pages and batching with the design's
mixers and feed-forwards against the plain whole-sequence implementation (no GPU: the kernels' plain statements of
tests/torch_ops.py stand in for them)."""
import json
import os
import random

import pytest
import torch

from dusilorn_util import CFG_A, CFG_B, chunked, dense, model, moe, plain_logits, random_config, read_model, tokens, windowed, write_model
from torch_ops import TorchOps


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {"A": write_model(str(tmp_path_factory.mktemp("dus_a")), CFG_A, 11),
            "B": write_model(str(tmp_path_factory.mktemp("dus_b")), CFG_B, 12)}


def host_engine(folder, page=4, pages=96, slots=4):
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
    assert cfg.architecture == "Dusilorn" and cfg.vocab_size == 131 and cfg.hidden_size == 64
    assert cfg.norm_eps == 1e-6 and cfg.embedding_scale == 2.0 and cfg.logit_scale == 1.5
    plan = plan_for(cfg)
    assert all(layer.arrangement == "sandwich_norm" for layer in plan.layers)
    assert plan.embedding.params["scale"] == 2.0 and plan.final_norm.params["gain_scale"] == 1.5 and plan.final_norm.params["gain_offset"] == 1.0
    first, second = plan.layers[0].parts["mixer"], plan.layers[1].parts["mixer"]
    assert first.kind == "flex_attention" and first.params["rot"] == (8, 500.0) and first.params["window"] == 5 and first.params["chunk"] == 0
    assert not first.params["qk_norm"] and not first.params["sink"] and first.params["v_mix"] is None and first.params["softcap"] == 25.0
    assert first.params["dim"] == 12 and first.params["vdim"] == 6 and "vmix" not in first.tensors
    assert second.params["qk_norm"] == "whole" and second.params["sink"] and second.params["chunk"] == 3 and second.params["window"] == 0
    assert second.params["rot"] is None and second.params["v_mix"] == "first" and second.params["softcap"] == 5.0
    assert second.tensors["q_norm"].shape == (24,) and second.tensors["k_norm"].shape == (8,) and second.tensors["sink"].shape == (3,)
    assert plan.layers[3].parts["mixer"].params["v_mix"] == "blend" and plan.layers[3].parts["mixer"].tensors["vmix"].shape == ()
    assert plan.layers[2].parts["mixer"].params["v_mix"] is None and plan.layers[2].parts["mixer"].params["softcap"] == 0.0
    assert plan.layers[0].parts["ffn"].kind == "swiglu" and "ffn" not in plan.layers[2].parts and "ffn_out_norm" not in plan.layers[2].parts
    assert plan.layers[1].parts["ffn"].params == {"hidden": 64, "ff": 24, "experts": 5, "top": 2, "score": "softmax", "correction": True,
                                                  "renormalize": True, "weight_on": "output", "gated": False, "identity": 2, "shared": 40}
    assert plan.layers[1].parts["ffn"].tensors["router"].shape == (7, 64) and "identity" not in plan.layers[3].parts["ffn"].params
    assert {"l0.mix.vmix", "l1.mix.vmix", "l2.norm2", "l2.norm2b"} <= set(plan.ignored_tensors)
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
               lambda c: c["layers"][1].update(type="attention_3"),
               lambda c: c["layers"][0]["mixer"]["rot"].update(dims=14),          # wider than the head
               lambda c: c["layers"][0]["mixer"].pop("rot"),                      # the rotated mixer needs its constants
               lambda c: c["layers"][3]["mixer"].update(vdim=3),                  # blended values of another size
               lambda c: c["layers"][1]["mlp"]["router"].update(top=8),           # more than the router has outputs
               lambda c: c["layers"][1]["mlp"].update(kind="gated"),
               lambda c: c["layers"][1]["mlp"]["shared"].pop("ff"),
               lambda c: c.pop("norm")):
        with pytest.raises(ConfigError):
            config_from_json_dict(changed(fn))


def test_loader_names_missing_tensors_and_takes_the_unused_ones(folders, tmp_path):
    from nanoinfer_b200.weights.loader import WeightError
    from nanoinfer_b200.weights.safetensors_io import save_safetensors
    cfg, w = read_model(folders["B"])
    with open(os.path.join(tmp_path, "config.json"), "w") as f:
        json.dump(cfg, f)
    # a checkpoint may hold the blend's number of the layer that never blends
    w["l0.mix.vmix"] = torch.tensor(0.5, dtype=torch.bfloat16)
    save_safetensors(os.path.join(tmp_path, "model.safetensors"), w)
    ids = tokens(9, 77, 1)
    close(run_cut(host_engine(str(tmp_path)), "x", ids, [9]), plain_logits(folders["B"], ids))
    del w["l0.mix.sink"]
    w["l0.mlp.e3.down"] = torch.zeros(5, 5, dtype=torch.bfloat16)
    save_safetensors(os.path.join(tmp_path, "model.safetensors"), w)
    with pytest.raises(WeightError) as e:
        host_engine(str(tmp_path))
    assert "l0.mix.sink" in str(e.value) and "l0.mlp.e3.down" in str(e.value)


def test_pages_the_model_asks_for(folders):
    eng = host_engine(folders["A"])
    needs = eng.model.cache_needs()
    assert [(t.heads, t.width) for t in needs[0][0].tensors] == [(2, 12), (2, 6)] and needs[0][0].window == 5 and needs[0][1] is None
    assert [(t.heads, t.width) for t in needs[1][0].tensors] == [(1, 8), (1, 10)] and needs[1][0].window == 3
    assert needs[2][0].window == 300 and needs[3][0].window == 7


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
    eng = host_engine(folders["A"], page=4, pages=30, slots=2)
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


def test_pages_behind_a_window_and_behind_a_chunk_go_back_to_the_pool(tmp_path):
    """A model of a windowed and a chunked layer: a long request holds no more pages than both need."""
    cfg = model(50, 32, [windowed(2, 1, 8, 4, 6, 8, 100.0, mlp=moe(3, 1, 16, identity=1)), chunked(2, 1, 8, 4, 5, mlp=None)])
    d = write_model(str(tmp_path), cfg, 3)
    eng = host_engine(d, page=2, pages=12, slots=1)
    ids = tokens(60, 50, 9)
    close(run_cut(eng, "long", ids, [3, 2] + [1] * 30 + [7, 11, 2, 5]), plain_logits(d, ids))
    eng.cache.check()


def one_layer(tmp_path, name, layer, change, seed=4, **kw):
    cfg = model(40, 24, [layer], **kw)
    return write_model(str(tmp_path / name), cfg, seed, weights=change)


def test_the_sink_takes_weight_once(tmp_path):
    """One chunked layer: a large sink must shrink the mixer's output as the plain softmax says, a very small one must
    change nothing; the engine agrees with the plain implementation in each case, in portions too."""
    layer = chunked(2, 1, 8, 6, 4, mlp=None)
    ids = tokens(11, 40, 1)
    refs = []
    for name, change in (("plain", lambda t: None), ("sink", lambda t: t["l0.mix.sink"].fill_(6.0)),
                         ("small", lambda t: t["l0.mix.sink"].fill_(-30.0))):
        d = one_layer(tmp_path, name, layer, change)
        ref = plain_logits(d, ids)
        close(run_cut(host_engine(d), "x", ids, [4, 1, 1, 5]), ref)
        refs.append(ref)
    assert (refs[0] - refs[1]).abs().max().item() > 1e-2 and (refs[0] - refs[2]).abs().max().item() > 1e-3


def test_blended_values_follow_the_factor(tmp_path):
    """Two layers that share values: with a factor of 0 the second layer's values are its own, with 1 they are the first
    layer's; a layer that does not say v_mix between them changes nothing of that."""
    layers = [windowed(2, 2, 8, 4, 6, 4, 100.0, mlp=None), chunked(1, 1, 6, 5, 4, v_mix=False, mlp=None), chunked(4, 1, 4, 8, 5, mlp=dense(16))]
    ids = tokens(13, 40, 2)
    refs = []
    for name, lam in (("zero", 0.0), ("half", 0.5), ("one", 1.0)):
        d = write_model(str(tmp_path / name), model(40, 24, layers), 5, weights=lambda t: t["l2.mix.vmix"].fill_(lam))
        ref = plain_logits(d, ids)
        close(run_cut(host_engine(d), "x", ids, [5, 1, 2, 5]), ref)
        refs.append(ref)
    assert (refs[0] - refs[1]).abs().max().item() > 1e-3 and (refs[1] - refs[2]).abs().max().item() > 1e-3


def test_router_options_each_move_the_result(tmp_path):
    """The correction decides the choice but is no part of the weight; identity outputs pass the input through; the shared
    expert is scaled by its gate."""
    layer = windowed(2, 1, 8, 4, 4, 4, 100.0, mlp=moe(4, 2, 16, identity=2, shared=8))
    ids = tokens(12, 40, 1)

    def favour_identity(t):
        t["l0.mlp.correction"][:4] = -1.0       # every token now chooses the two identity outputs: the mixture adds h itself

    def other_choice(t):
        t["l0.mlp.correction"].copy_(torch.tensor([0.9, -0.9, 0.5, -0.5, -0.7, -0.8]).to(torch.bfloat16))

    def closed_gate(t):
        t["l0.mlp.shared.sg"].zero_()           # sigmoid(0) = 1/2 on the shared expert

    refs = []
    for name, change in (("as_is", lambda t: None), ("identity", favour_identity), ("choice", other_choice), ("gate", closed_gate)):
        d = one_layer(tmp_path, name, layer, change, seed=6)
        ref = plain_logits(d, ids)
        close(run_cut(host_engine(d), "x", ids, [5, 1, 1, 5]), ref)
        refs.append(ref)
    for other in refs[1:]:
        assert (refs[0] - other).abs().max().item() > 1e-3


def test_scales_on_embedding_and_logits(tmp_path):
    layer = chunked(2, 2, 4, 4, 3, mlp=dense(8))
    ids = tokens(7, 40, 3)
    a = one_layer(tmp_path, "a", layer, None, emb=1.0, logit=1.0)
    b = one_layer(tmp_path, "b", layer, None, emb=1.0, logit=4.0)
    c = one_layer(tmp_path, "c", layer, None, emb=5.0, logit=1.0)
    got = [run_cut(host_engine(d), "x", ids, [3, 4]) for d in (a, b, c)]
    for d, g in zip((a, b, c), got):
        close(g, plain_logits(d, ids))
    close(got[1], 4.0 * got[0])
    assert (got[2] - got[0]).abs().max().item() > 1e-3


@pytest.mark.parametrize("seed", [400, 401, 402, 403, 404, 405])
def test_random_configurations(seed, tmp_path):
    rng = random.Random(seed)
    cfg = random_config(rng)
    d = write_model(str(tmp_path), cfg, seed)
    ids = tokens(rng.choice([19, 41, 70]), cfg["vocab"], seed)
    ref = plain_logits(d, ids)
    eng = host_engine(d, page=rng.choice([2, 4, 8]), pages=200)
    close(run_cut(eng, "w", ids, [len(ids)]), ref)
    cuts, left = [], len(ids)
    while left:
        cuts.append(min(left, rng.choice([1, 1, 2, 3, 7, 16])))
        left -= cuts[-1]
    close(run_cut(eng, "c", ids, cuts), ref)
    eng.cache.check()


def test_greedy_generation_through_the_scheduler(folders):
    """The framework's own entry point: a Model, its Scheduler with a small token budget (prompts go in portions,
    requests join and leave), three slots."""
    from nanoinfer_b200.api import Model
    from nanoinfer_b200.config import EngineConfig
    from nanoinfer_b200.engine.scheduler import Request, Scheduler
    m = Model(folders["B"], EngineConfig(dtype="float32", page_size=4, num_pages=96, max_batch=3, max_tokens_per_step=8,
                                         device="cpu", cuda_graphs=False), ops=TorchOps())
    sched = Scheduler(m)
    prompts = [tokens(13, 77, 21), tokens(5, 77, 22), tokens(19, 77, 23), tokens(3, 77, 24)]
    for i, p in enumerate(prompts):
        sched.add(Request(f"g{i}", p, max_tokens=6))
    done = sched.run()
    for i, p in enumerate(prompts):
        ids = list(p)
        for _ in range(6):
            ids.append(int(plain_logits(folders["B"], ids)[-1].argmax()))
        assert done[f"g{i}"] == ids[len(p):], i
    m.engine.cache.check()
