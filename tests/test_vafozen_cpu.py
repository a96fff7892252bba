"""Vafozen on the host backend: configuration, plan and weights; the engine's cache, state slots and batching with the
design's mixers against the plain whole-sequence implementation (no GPU: the kernels' plain statements of
tests/torch_ops.py stand in for them)."""
import json
import os

import pytest
import torch

from torch_ops import TorchOps
from vafozen_util import CFG_A, CFG_B, pair, plain_logits, softmax_half, tokens, with_mlp, write_model


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {"A": write_model(str(tmp_path_factory.mktemp("vaf_a")), CFG_A, 11, strip_rank=True),
            "B": write_model(str(tmp_path_factory.mktemp("vaf_b")), CFG_B, 12)}


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
    assert cfg.architecture == "Vafozen" and cfg.vocab_size == 131 and cfg.hidden_size == 64
    assert cfg.norm_eps == 1e-6 and cfg.embedding_scale == 3.0
    with pytest.raises(ConfigError):        # the decay maps' widths are in neither place yet
        plan_for(cfg)
    plan = plan_for(cfg.with_tensor_shapes(tensor_shapes(folders["A"])))
    first = plan.layers[0].parts["mixer"].params
    assert first["left"].kind == "flex_attention" and first["right"].kind == "time_mix"
    assert first["left"].params["conv"] == 2 and first["left"].params["rot"] == (4, 500.0) and first["left"].params["softcap"] == 5.0
    assert first["left"].params["out_gate"] and not first["left"].params["qk_norm"] and first["left"].params["out_scale"] == 1.1
    assert first["right"].params["vdim"] == 4 and first["right"].params["decay_rank"] == 6
    third = plan.layers[2].parts["mixer"].params
    assert third["left"].params["chunk"] == 7 and third["left"].params["slope_span"] == 8.0 and third["left"].params["qk_norm"]
    assert third["right"].kind == "gated_linear_attention" and third["right"].params["tau"] == 4.0
    assert plan.layers[1].parts["mixer"].kind == "mamba2" and "ffn" not in plan.layers[2].parts
    assert "ffn_norm" not in plan.layers[0].parts and plan.layers[0].parts["mixer_norm"].params["gain_offset"] == 1.0
    assert plan.embedding.params["scale"] == 3.0 and plan.lm_head.tensors["weight"].name == "head"
    again = config_from_json_dict(json.loads(json.dumps(cfg.to_json_dict())))
    assert again == cfg


def test_config_refuses_what_it_cannot_run():
    from nanoinfer_b200.config.model_config import ConfigError
    from nanoinfer_b200.registry import config_from_json_dict
    bad = json.loads(json.dumps(CFG_A))
    bad["layers"][0]["mixer"]["left"]["heads"] = 3       # no multiple of its two kv heads
    with pytest.raises(ConfigError):
        config_from_json_dict(bad)
    bad = json.loads(json.dumps(CFG_A))
    bad["layers"][1]["type"] = "mamba3"
    with pytest.raises(ConfigError):
        config_from_json_dict(bad)
    bad = json.loads(json.dumps(CFG_A))
    bad["layers"][0]["mixer"]["left"]["rot"]["dims"] = 10       # wider than the head
    with pytest.raises(ConfigError):
        config_from_json_dict(bad)
    bad = json.loads(json.dumps(CFG_A))
    del bad["layers"][2]["mixer"]["right"]["tau"]
    with pytest.raises(ConfigError):
        config_from_json_dict(bad)


def test_loader_names_missing_and_misshapen_tensors(folders, tmp_path):
    from nanoinfer_b200.weights.loader import WeightError
    from nanoinfer_b200.weights.safetensors_io import save_safetensors
    from vafozen_util import read_model
    cfg, w = read_model(folders["B"])
    del w["l1.mix.A_log"]
    w["l0.mix.left.q.norm"] = torch.zeros(5, dtype=torch.bfloat16)
    with open(os.path.join(tmp_path, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_safetensors(os.path.join(tmp_path, "model.safetensors"), w)
    with pytest.raises(WeightError) as e:
        host_engine(str(tmp_path))
    assert "l1.mix.A_log" in str(e.value) and "l0.mix.left.q.norm" in str(e.value)


def test_state_and_pages_the_model_asks_for(folders):
    eng = host_engine(folders["A"])
    needs = eng.model.cache_needs()
    # pair 2: conv tails of q, k, v (one row of 32 + 16 + 24) + the last h (64) + S (3 heads x 4 x 8)
    assert needs[0][1].shape == ((2 - 1) * (4 * 8 + 2 * 8 + 2 * 12) + 64 + 3 * 4 * 8,)
    assert [t.width for t in needs[0][0].tensors] == [8, 12] and needs[0][0].window == 0
    assert needs[1][0] is None and needs[1][1].shape == (2 * (3 * 8 + 2 * 6) + 3 * 8 * 6,)
    assert needs[2][0].window == 7 and needs[2][1].shape == (1 * 6 * 10,)
    assert needs[3][1].shape == (2 * 12 * 5,)        # one tap: no history


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
    slot and pages (two slots only, a pool that forces reuse) and must start from zero state and an empty history."""
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


def test_pages_behind_a_chunk_go_back_to_the_pool(folders, tmp_path):
    """A model of chunked layers only: a long request holds no more pages than a chunk needs."""
    cfg = {"architecture": "Vafozen", "vocab": 50, "width": 32, "norm": {"eps": 1e-6}, "embedding": {"scale": 2.0}, "layers": [
        with_mlp(pair(softmax_half(2, 1, 8, 8, mask=6), 1, 8, rank=4), 48)]}
    d = write_model(str(tmp_path), cfg, 3)
    eng = host_engine(d, page=2, pages=8, slots=1)
    ids = tokens(40, 50, 9)
    close(run_cut(eng, "long", ids, [3, 2] + [1] * 35), plain_logits(d, ids))
    eng.cache.check()


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
