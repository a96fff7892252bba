"""Nezalorn on the host backend: configuration, plan and weights; the engine's cache, state slots and batching with
the design's mixers against the plain whole-sequence implementation (no GPU: the kernels' plain statements of
tests/torch_ops.py stand in for them)."""
import json
import os

import pytest
import torch

from nezalorn_util import CFG_A, CFG_B, DECAY_RANK, config_with_rank, plain_logits, tokens, write_model
from torch_ops import TorchOps


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {"A": write_model(str(tmp_path_factory.mktemp("nez_a")), config_with_rank(CFG_A, DECAY_RANK["A"]), 11, strip_rank=True),
            "B": write_model(str(tmp_path_factory.mktemp("nez_b")), config_with_rank(CFG_B, DECAY_RANK["B"]), 12)}


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
    from nanoinfer_b200.config.model_config import ConfigError, read_config_json
    from nanoinfer_b200.registry import config_from_json_dict, plan_for
    from nanoinfer_b200.weights.loader import tensor_shapes
    cfg = config_from_json_dict(read_config_json(folders["A"]))
    assert cfg.architecture == "Nezalorn" and cfg.vocab_size == 131 and cfg.hidden_size == 64 and cfg.norm_eps == 1e-6
    with pytest.raises(ConfigError):        # the decay map's width is in neither place yet
        plan_for(cfg)
    cfg = cfg.with_tensor_shapes(tensor_shapes(folders["A"]))
    plan = plan_for(cfg)
    assert [e.reads_cache_of for e in plan.schedule] == [None, None, None, 1, None, None]
    assert plan.layers[2].parts["mixer"].params["decay_rank"] == DECAY_RANK["A"]
    # the owner keeps what its widest reader sees; each layer masks with its own window
    assert plan.layers[1].parts["mixer"].params["keep"] == 11 and plan.layers[1].parts["mixer"].params["window"] == 7
    assert plan.layers[3].parts["mixer"].params["window"] == 11 and "dkv" not in plan.layers[3].parts["mixer"].tensors
    assert "ffn" not in plan.layers[2].parts
    again = config_from_json_dict(json.loads(json.dumps(cfg.to_json_dict())))
    assert again.layers == cfg.layers and again.norm_eps == cfg.norm_eps


@pytest.mark.parametrize("bad", [
    lambda c: c["layers"][0].update(type="mamba"),
    lambda c: c["layers"][3]["mixer"].update(kv_from=5),
    lambda c: c["layers"][3]["mixer"].update(kv_from=0),
    lambda c: c["layers"][3]["mixer"].update(kv_rank=24),
    lambda c: c["layers"][0]["mixer"].update(blocks=5),
    lambda c: c["layers"][1]["mixer"]["rot"].update(dims=6),
    lambda c: c.pop("norm"),
    lambda c: c["layers"][0].update(mlp={"kind": "experts", "ff": 8}),
])
def test_config_refuses_what_the_design_does_not_have(bad):
    from nanoinfer_b200.config.model_config import ConfigError
    from nanoinfer_b200.registry import config_from_json_dict
    c = json.loads(json.dumps(CFG_A))
    bad(c)
    with pytest.raises(ConfigError):
        config_from_json_dict(c)


def test_weights_missing_and_unexpected_are_reported(folders, tmp_path):
    from nanoinfer_b200.weights.loader import WeightError
    from nanoinfer_b200.weights.safetensors_io import open_model_files, save_safetensors
    f = open_model_files(folders["B"])[0]
    t = {n: f.tensor(n) for n in f.names()}
    t["l9.mix.r"] = t.pop("l1.mix.r")
    d = str(tmp_path)
    save_safetensors(os.path.join(d, "model.safetensors"), t)
    with open(os.path.join(folders["B"], "config.json")) as src, open(os.path.join(d, "config.json"), "w") as dst:
        dst.write(src.read())
    with pytest.raises(WeightError) as e:
        host_engine(d)
    assert "l1.mix.r" in e.value.missing and "l9.mix.r" in e.value.unexpected


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
    """Three requests of different lengths advance together in portions and single tokens; when one ends, another takes
    its slot and pages (two slots only, a pool that forces reuse) and must start from zero state."""
    from nanoinfer_b200.engine import StepEntry
    eng = host_engine(folders["A"], page=4, pages=24, slots=2)
    seqs = {k: tokens(n, 131, s) for k, n, s in (("p", 23, 1), ("q", 9, 2), ("r", 17, 3), ("s", 12, 4))}
    ref = {k: plain_logits(folders["A"], v) for k, v in seqs.items()}
    got = {k: [] for k in seqs}
    at = {k: 0 for k in seqs}
    live = {}
    plan = [[("p", 6), ("q", 2)], [("p", 1), ("q", 5)], [("p", 7), ("q", 2)], [("p", 1), ("r", 9)], [("r", 1), ("p", 1)],
            [("p", 7), ("r", 7)], [("s", 3)], [("s", 1)], [("s", 8)]]
    slots_used = {}
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


def test_greedy_generation_through_the_scheduler(folders):
    """The framework's own entry point: a Model, its Scheduler with a small token budget (prompts go in portions,
    requests join and leave), three state slots."""
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
