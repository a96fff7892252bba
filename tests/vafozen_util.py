"""Small Vafozen configurations and weights for the tests: sizes that differ from layer to layer, include 1 and values
that are no powers of two, and weights large enough that every mechanism moves the logits."""
import json
import os

import torch


def softmax_half(heads, kv_heads, dim, vdim, scale=None, conv=None, rot=None, softcap=None, mask=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5}
    if conv is not None:
        m["conv"] = conv
    if rot is not None:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    if softcap is not None:
        m["softcap"] = softcap
    if mask is not None:
        m["mask"] = {"size": mask}
    return m


def pair(left, heads, dim, vdim=None, tau=4.0, rank=6, left_scale=0.7, right_scale=1.3):
    """A ``parallel`` layer: chunked softmax attention beside gated linear attention."""
    right = {"heads": heads, "dim": dim, "tau": tau, "decay_rank": rank}
    if vdim is not None:
        right["vdim"] = vdim
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale}}


def pair2(left, heads, dim, vdim=None, rank=6, left_scale=1.1, right_scale=0.6):
    """A ``parallel_2`` layer: rotated, capped, gated softmax attention beside a time mix."""
    right = {"heads": heads, "dim": dim, "decay_rank": rank}
    if vdim is not None:
        right["vdim"] = vdim
    return {"type": "parallel_2", "mixer": {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale}}


def ssm(heads, vdim, state, groups, norm_groups, conv):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "norm_groups": norm_groups, "conv": conv}}


def with_mlp(layer, ff):
    return dict(layer, mlp=None if ff is None else {"kind": "dense", "ff": ff})


# Every mixer; keys and values of different widths; a rotation of part of a head; a chunk of 7 (no multiple of a page);
# one kv head; a time mix whose values are narrower than its keys; a layer without a feed-forward.
CFG_A = {"architecture": "Vafozen", "vocab": 131, "width": 64, "norm": {"eps": 1e-6}, "embedding": {"scale": 3.0}, "layers": [
    with_mlp(pair2(softmax_half(4, 2, 8, 12, scale=0.3, conv=2, rot=(4, 500.0), softcap=5.0), 3, 8, vdim=4), 96),
    with_mlp(ssm(3, 8, 6, 1, 3, 3), 80),
    with_mlp(pair(softmax_half(3, 1, 12, 8, mask=7), 1, 10, vdim=6, rank=5), None),
    with_mlp(ssm(2, 12, 5, 2, 1, 1), 72),
    with_mlp(pair2(softmax_half(2, 2, 16, 16, conv=4, rot=(16, 10000.0), softcap=30.0), 2, 12), 64),
]}
# No embedding factor to speak of, a chunk longer than any test sequence, heads of 16 and 32, a convolution of five taps.
CFG_B = {"architecture": "Vafozen", "vocab": 77, "width": 96, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0}, "layers": [
    with_mlp(pair(softmax_half(2, 1, 16, 32, mask=300), 3, 16, tau=16.0), 128),
    with_mlp(ssm(4, 16, 16, 2, 2, 5), 112),
    with_mlp(pair2(softmax_half(6, 3, 32, 16, conv=3, rot=(8, 100.0), softcap=10.0), 2, 32, vdim=16), 128),
]}


def make_weights(plan, seed):
    """bfloat16 tensors for every tensor of ``plan``: matrices N(0, 1.2^2 / fan_in), so activations stay of order one."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for ts in plan.tensor_specs():
        x = torch.randn(ts.shape, generator=g, dtype=torch.float32)
        if ts.init == "matrix":
            x = x * (1.2 / ts.shape[-1] ** 0.5)
        elif ts.init == "embedding":
            x = x * (1.0 if ts.name == "embed" else 1.2 / ts.shape[-1] ** 0.5)
        elif ts.init == "gain":
            x = 1.0 + 0.1 * x
        elif ts.init == "bias":
            x = 0.1 * x
        elif ts.init == "unit":
            x = 0.7 * x
        elif ts.init == "mix01":
            x = torch.rand(ts.shape, generator=g, dtype=torch.float32)
        else:
            raise ValueError(ts.init)
        out[ts.name] = x.to(torch.bfloat16)
    return out


def write_model(folder, cfg, seed, strip_rank=False, weights=None):
    """A model folder of ``cfg``. With ``strip_rank`` the written config.json leaves the decay maps' widths to the shapes
    of their tensors. ``weights``: a function that changes the random tensors in place before they are written."""
    from nanoinfer_b200.registry import config_from_json_dict, plan_for
    from nanoinfer_b200.weights.safetensors_io import save_safetensors
    plan = plan_for(config_from_json_dict(cfg))
    os.makedirs(folder, exist_ok=True)
    written = json.loads(json.dumps(cfg))
    if strip_rank:
        for layer in written["layers"]:
            if "right" in layer["mixer"]:
                layer["mixer"]["right"].pop("decay_rank", None)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(written, f)
    tensors = make_weights(plan, seed)
    if weights is not None:
        weights(tensors)
    save_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    return folder


def read_model(folder):
    from nanoinfer_b200.weights.safetensors_io import SafetensorsFile
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    sf = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    return cfg, {n: sf.tensor(n) for n in sf.names()}


def plain_logits(folder, ids):
    """Float64 logits [len(ids), vocab] of the plain implementation."""
    import plain_vafozen as plain
    cfg, w = read_model(folder)
    return plain.logits(cfg, w, list(ids))


def tokens(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def random_config(rng):
    """A configuration with random layer order, sizes (odd ones, ones, sizes no kernel's fast path takes) and constants."""
    width = rng.choice([40, 64, 72, 100, 128, 192, 258])
    layers = []
    for _ in range(rng.randint(2, 7)):
        kind = rng.choice(["parallel", "parallel_2", "mamba2"])
        ff = rng.choice([None, 48, 96, 130, 256])
        if kind == "mamba2":
            groups = rng.choice([1, 2, 3])
            heads = groups * rng.choice([1, 2, 4])
            vdim = rng.choice([4, 8, 12, 16, 33, 64])
            ng = rng.choice([g for g in (1, 2, 3, 4, heads) if (heads * vdim) % g == 0])
            layer = ssm(heads, vdim, rng.choice([1, 5, 16, 32, 48, 70, 128]), groups, ng, rng.choice([1, 2, 3, 4, 6]))
        else:
            kv = rng.choice([1, 2, 3])
            heads = kv * rng.choice([1, 2, 4])
            dim = rng.choice([4, 8, 12, 16, 24, 40, 64, 96, 136])
            vdim = rng.choice([3, 8, 16, 24, 64, 100])
            rh, rd = rng.choice([1, 2, 3, 5]), rng.choice([4, 8, 20, 32, 48, 64, 130])
            rv = rng.choice([None, 4, 16, 40])
            if kind == "parallel":
                left = softmax_half(heads, kv, dim, vdim, scale=rng.choice([None, 0.2]), mask=rng.choice([1, 2, 5, 16, 17, 31, 32, 33, 64, 100]))
                layer = pair(left, rh, rd, vdim=rv, tau=rng.choice([1.0, 4.0, 16.0]), rank=rng.choice([1, 4, 8, 16]),
                             left_scale=rng.choice([0.5, 1.0, 1.2]), right_scale=rng.choice([0.9, 1.0]))
            else:
                rot = rng.choice([d for d in (2, 4, 8, 16, 32, dim) if d <= dim and d % 2 == 0])
                left = softmax_half(heads, kv, dim, vdim, scale=rng.choice([None, 0.2]), conv=rng.choice([1, 2, 3, 4, 6]),
                                    rot=(rot, rng.choice([100.0, 10000.0, 1e6])), softcap=rng.choice([2.0, 15.0, 50.0]))
                layer = pair2(left, rh, rd, vdim=rv, rank=rng.choice([1, 4, 8, 16]), left_scale=rng.choice([0.5, 1.0]),
                              right_scale=rng.choice([0.9, 1.3]))
        layers.append(with_mlp(layer, ff))
    return {"architecture": "Vafozen", "vocab": rng.choice([50, 131, 257, 1000]), "width": width,
            "norm": {"eps": rng.choice([1e-6, 1e-5, 1e-4])}, "embedding": {"scale": rng.choice([1.0, 4.0, 11.0])}, "layers": layers}
