"""Small Nezalorn configurations and weights for the tests: sizes that differ from layer to layer, include 1 and
values that are no powers of two, and weights large enough that every mechanism moves the logits."""
import json
import os

import torch

LATENT_ROT = {"dims": 4, "base": 500.0, "scaling": {"factor": 3.0, "original": 16, "fast": 4.0, "slow": 0.5}}


def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, window, rot=None, kv_from=None, scale=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
         "mask": {"size": window}, "rot": rot or dict(LATENT_ROT, dims=rot_dim),
         "scale": scale if scale is not None else (dim + rot_dim) ** -0.5}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m}


def delta(heads, dim):
    return {"type": "general_delta", "mixer": {"heads": heads, "dim": dim}}


def lru(width, conv, blocks):
    return {"type": "rglru", "mixer": {"width": width, "conv": conv, "blocks": blocks}}


def with_mlp(layer, ff):
    return dict(layer, mlp=None if ff is None else {"kind": "dense", "ff": ff})


# Every mixer, a layer without a feed-forward, a reader of another layer's latent with a WIDER window than its
# owner's, a convolution of one tap, one block, one head.
CFG_A = {"architecture": "Nezalorn", "vocab": 131, "width": 64, "norm": {"eps": 1e-6}, "layers": [
    with_mlp(lru(48, 3, 3), 96),
    with_mlp(latent(3, 8, 4, 12, 24, 20, 7), 80),
    with_mlp(delta(2, 24), None),
    with_mlp(latent(2, 16, 4, 8, 16, 20, 11, kv_from=1), 72),
    with_mlp(lru(32, 1, 1), 64),
    with_mlp(delta(1, 40), 96),
]}
# No frequency scaling, a window longer than any test sequence, a convolution of five taps, heads of 16.
CFG_B = {"architecture": "Nezalorn", "vocab": 77, "width": 96, "norm": {"eps": 1e-5}, "layers": [
    with_mlp(latent(1, 16, 8, 16, 16, 32, 300, rot={"dims": 8, "base": 10000.0}), 128),
    with_mlp(delta(3, 16), 112),
    with_mlp(lru(64, 5, 2), 128),
]}
DECAY_RANK = {"A": 6, "B": 8}


def config_with_rank(cfg, rank):
    out = json.loads(json.dumps(cfg))
    for layer in out["layers"]:
        if layer["type"] == "general_delta":
            layer["mixer"]["decay_rank"] = rank
    return out


def make_weights(plan, seed):
    """bfloat16 tensors for every tensor of ``plan``: matrices N(0, 1/fan_in), so activations stay of order one."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for ts in plan.tensor_specs():
        x = torch.randn(ts.shape, generator=g, dtype=torch.float32)
        if ts.init == "matrix":
            x = x * (1.2 / ts.shape[-1] ** 0.5)
        elif ts.init == "gain":
            x = 1.0 + 0.1 * x
        elif ts.init == "bias":
            x = 0.1 * x
        elif ts.init == "unit":
            x = 0.7 * x
        elif ts.init == "mix":
            x = (1.0 + 0.3 * x) / x.numel()
        out[ts.name] = x.to(torch.bfloat16)
    return out


def write_model(folder, cfg, seed, strip_rank=False):
    """A model folder of ``cfg`` (which names decay_rank). With ``strip_rank`` the written config.json leaves the decay
    map's width to the shape of the tensor."""
    from nanoinfer_b200.registry import config_from_json_dict, plan_for
    from nanoinfer_b200.weights.safetensors_io import save_safetensors
    plan = plan_for(config_from_json_dict(cfg))
    os.makedirs(folder, exist_ok=True)
    written = json.loads(json.dumps(cfg))
    if strip_rank:
        for layer in written["layers"]:
            layer["mixer"].pop("decay_rank", None)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(written, f)
    save_safetensors(os.path.join(folder, "model.safetensors"), make_weights(plan, seed))
    return folder


def plain_logits(folder, ids):
    """Float64 logits [len(ids), vocab] of the plain implementation."""
    import plain_nezalorn as plain
    from plain_qwen2 import read_weights
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    return plain.forward(cfg, read_weights(folder), list(ids))


def tokens(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def random_config(rng):
    """A configuration with random layer order, sizes (odd ones, ones, sizes no kernel's fast path takes) and constants."""
    width = rng.choice([40, 64, 72, 100, 128, 192, 258, 320])
    vocab = rng.choice([50, 131, 257, 448, 1000])
    n_layers = rng.randint(2, 9)
    layers, owners = [], []
    for i in range(n_layers):
        kind = rng.choice(["latent", "delta", "lru"])
        ff = rng.choice([None, 48, 96, 130, 256, 300])
        if kind == "delta":
            layer = delta(rng.choice([1, 2, 3, 4, 6]), rng.choice([8, 12, 16, 20, 24, 32, 40, 48, 64, 72, 96, 128]))
        elif kind == "lru":
            blocks = rng.choice([1, 2, 3, 4, 8])
            layer = lru(blocks * rng.choice([4, 8, 12, 16, 20, 32, 64]), rng.choice([1, 2, 3, 4, 5, 7]), blocks)
        else:
            rot_dim = rng.choice([2, 4, 8, 12, 16, 32, 64])
            scaling = rng.choice([None, {"factor": rng.choice([2.0, 4.0, 8.0, 32.0]), "original": rng.choice([16, 64, 1024, 4096]),
                                         "fast": rng.choice([8.0, 32.0]), "slow": rng.choice([0.5, 1.0, 2.0])}])
            rot = {"dims": rot_dim, "base": rng.choice([100.0, 10000.0, 20000.0, 1e6])}
            if scaling: rot["scaling"] = scaling
            kv_rank = rng.choice([8, 12, 16, 20, 24, 32, 48, 64, 80, 96, 128, 160, 200, 256])
            window = rng.choice([1, 2, 3, 5, 16, 17, 31, 32, 33, 63, 64, 65, 100, 136, 500])
            heads = rng.choice([1, 2, 3, 4, 6, 8, 16, 17, 20])
            dim, vdim, q_rank = rng.choice([4, 8, 16, 24, 32, 48, 64, 136]), rng.choice([3, 4, 8, 16, 32, 48, 64]), rng.choice([8, 16, 24, 48, 128])
            src = None
            if owners and rng.random() < 0.4:
                src = rng.choice(owners)
                o = layers[src]["mixer"]
                layer = latent(heads, dim, o["rot_dim"], vdim, q_rank, o["kv_rank"], window, rot=o["rot"], kv_from=src, scale=rng.choice([None, 0.1, 0.3]))
            else:
                layer = latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, window, rot=rot, scale=rng.choice([None, 0.1, 0.3]))
                owners.append(i)
        layers.append(with_mlp(layer, ff))
    for layer in layers:
        if layer["type"] == "general_delta":
            layer["mixer"]["decay_rank"] = rng.choice([1, 4, 8, 16, 24, 64])
    return {"architecture": "Nezalorn", "vocab": vocab, "width": width, "norm": {"eps": rng.choice([1e-6, 1e-5, 1e-4])}, "layers": layers}
