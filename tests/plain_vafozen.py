"""Vafozen, slowly and plainly: whole sequences in float64, one function per mechanism, loops over tokens where the
design is a recurrence. Shares no code with the package; the tests compare the engine with it.

A model is ``(config dict, {tensor name: tensor})``. ``logits(cfg, w, ids)`` returns ``[len(ids), vocab]``;
``forward(cfg, w, ids)`` also returns the residual stream after every layer.
"""
import math

import torch

F = torch.float64


def rms_unit(x, eps):
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def norm_one_plus(x, w, eps):
    return rms_unit(x, eps) * (1.0 + w)


def norm_plain(x, w, eps):
    return rms_unit(x, eps) * w


def silu(z):
    return z * torch.sigmoid(z)


def short_conv(u, w, bias=None):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the start."""
    t_len, taps = u.shape[0], w.shape[1]
    y = torch.zeros_like(u)
    for t in range(t_len):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                y[t] += w[:, j] * u[s]
    if bias is not None:
        y = y + bias
    return y


def rotate_half(x, dims, base):
    """x [T, heads, d]: the first ``dims`` of every head turned by position; pair (i, i + dims/2)."""
    t_len = x.shape[0]
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F)
    a = torch.arange(t_len, dtype=F)[:, None] * f[None, :]
    c, s = a.cos()[:, None, :], a.sin()[:, None, :]
    out = x.clone()
    u, v = x[..., :half], x[..., half:dims]
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


def visible(t_len, chunk=None):
    """[T, T] bool: j <= i, and with ``chunk`` also the same block of ``chunk`` positions."""
    i = torch.arange(t_len)[:, None]
    j = torch.arange(t_len)[None, :]
    m = j <= i
    if chunk:
        m = m & ((i // chunk) == (j // chunk))
    return m


def softmax_attention(q, k, v, scale, mask, slopes=None, softcap=None):
    """q [T, H, d], k [T, G, d], v [T, G, dv] -> [T, H, dv]."""
    t_len, heads = q.shape[0], q.shape[1]
    rep = heads // k.shape[1]
    out = torch.zeros(t_len, heads, v.shape[2], dtype=F)
    dist = (torch.arange(t_len)[:, None] - torch.arange(t_len)[None, :]).to(F)
    for h in range(heads):
        s = (q[:, h] @ k[:, h // rep].t()) * scale
        if softcap:
            s = softcap * torch.tanh(s / softcap)
        if slopes is not None:
            s = s - slopes[h] * dist
        s = s.masked_fill(~mask, -math.inf)
        out[:, h] = torch.softmax(s, dim=-1) @ v[:, h // rep]
    return out


def linear_state_walk(q, k, v, decay, bonus=None):
    """S_t = diag(decay_t) S_(t-1) + k_t v_t^T per head; o_t = S_t^T q_t, or with ``bonus`` u:
    o_t = (S_(t-1) + diag(u) k_t v_t^T)^T q_t. q, k, decay [T, H, dk]; v [T, H, dv]; u [H, dk]."""
    t_len, heads, dk = k.shape
    dv = v.shape[2]
    s = torch.zeros(heads, dk, dv, dtype=F)
    out = torch.zeros(t_len, heads, dv, dtype=F)
    for t in range(t_len):
        kv = k[t][:, :, None] * v[t][:, None, :]
        if bonus is not None:
            out[t] = torch.einsum("hkv,hk->hv", s + bonus[:, :, None] * kv, q[t])
            s = decay[t][:, :, None] * s + kv
        else:
            s = decay[t][:, :, None] * s + kv
            out[t] = torch.einsum("hkv,hk->hv", s, q[t])
    return out


def softmax_side(h, w, p, m, eps, kind):
    t_len = h.shape[0]
    heads, groups, d = m["heads"], m["kv_heads"], m["dim"]
    dv = m.get("vdim", d)
    q = h @ w[p + ".q"].t() + w[p + ".q.b"]
    k = h @ w[p + ".k"].t() + w[p + ".k.b"]
    v = h @ w[p + ".v"].t() + w[p + ".v.b"]
    if "conv" in m:
        q, k, v = short_conv(q, w[p + ".q.conv"]), short_conv(k, w[p + ".k.conv"]), short_conv(v, w[p + ".v.conv"])
    q, k, v = q.view(t_len, heads, d), k.view(t_len, groups, d), v.view(t_len, groups, dv)
    if p + ".q.norm" in w:
        q, k = norm_plain(q, w[p + ".q.norm"], eps), norm_plain(k, w[p + ".k.norm"], eps)
    if "rot" in m:
        q, k = rotate_half(q, m["rot"]["dims"], m["rot"]["base"]), rotate_half(k, m["rot"]["dims"], m["rot"]["base"])
    slopes = None
    if kind == "parallel":
        slopes = [2.0 ** (-8.0 * (i + 1) / heads) for i in range(heads)]
    chunk = m["mask"]["size"] if "mask" in m else None
    o = softmax_attention(q, k, v, m["scale"], visible(t_len, chunk), slopes, m.get("softcap")).reshape(t_len, heads * dv)
    if p + ".g" in w:
        o = o * torch.sigmoid(h @ w[p + ".g"].t())
    return o @ w[p + ".o"].t() + w[p + ".o.b"]


def gated_linear_side(h, w, p, m, eps):
    t_len, heads, d = h.shape[0], m["heads"], m["dim"]
    dv = m.get("vdim", d)
    q = (h @ w[p + ".q"].t()).view(t_len, heads, d) * d ** -0.5
    k = (h @ w[p + ".k"].t()).view(t_len, heads, d)
    v = (h @ w[p + ".v"].t()).view(t_len, heads, dv)
    z = (h @ w[p + ".a1"].t()) @ w[p + ".a2"].t() + w[p + ".a2.b"]
    alpha = torch.sigmoid(z).pow(1.0 / m["tau"]).view(t_len, heads, d)
    o = linear_state_walk(q, k, v, alpha)
    o = norm_plain(o, w[p + ".norm"], eps).reshape(t_len, heads * dv)
    return (o * silu(h @ w[p + ".g"].t())) @ w[p + ".o"].t()


def time_mix_side(h, w, p, m, eps):
    t_len, heads, d = h.shape[0], m["heads"], m["dim"]
    dv = m.get("vdim", d)
    prev = torch.cat([torch.zeros(1, h.shape[1], dtype=F), h[:-1]])
    mix = {s: h + (prev - h) * w[f"{p}.mu.{s}"] for s in "rkvgw"}
    r = (mix["r"] @ w[p + ".r"].t()).view(t_len, heads, d)
    k = (mix["k"] @ w[p + ".k"].t()).view(t_len, heads, d)
    v = (mix["v"] @ w[p + ".v"].t()).view(t_len, heads, dv)
    gate = silu(mix["g"] @ w[p + ".g"].t())
    decay = torch.exp(-torch.exp(torch.tanh(mix["w"] @ w[p + ".w1"].t()) @ w[p + ".w2"].t() + w[p + ".w0"])).view(t_len, heads, d)
    o = linear_state_walk(r, k, v, decay, bonus=w[p + ".u"])
    o = rms_unit(o, eps).reshape(t_len, heads * dv) * w[p + ".norm"]
    return (o * gate) @ w[p + ".o"].t()


def mamba2_mixer(h, w, p, m, eps):
    t_len = h.shape[0]
    heads, dv, n, groups = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = heads * dv
    zxbcdt = h @ w[p + ".in"].t()
    z, xbc, dt = zxbcdt[:, :inner], zxbcdt[:, inner:2 * inner + 2 * groups * n], zxbcdt[:, 2 * inner + 2 * groups * n:]
    xbc = silu(short_conv(xbc, w[p + ".conv"], w[p + ".conv.b"]))
    x = xbc[:, :inner].view(t_len, heads, dv)
    b = xbc[:, inner:inner + groups * n].view(t_len, groups, n)
    c = xbc[:, inner + groups * n:].view(t_len, groups, n)
    dt = torch.nn.functional.softplus(dt + w[p + ".dt_bias"], threshold=1e9)
    rep = heads // groups
    decay = torch.exp(-torch.exp(w[p + ".A_log"]) * dt)                      # [T, heads]
    bh, ch = b.repeat_interleave(rep, dim=1), c.repeat_interleave(rep, dim=1)
    y = linear_state_walk(ch, bh, x * dt[:, :, None], decay[:, :, None].expand(t_len, heads, n))
    y = (y + w[p + ".D"][None, :, None] * x).reshape(t_len, inner) * silu(z)
    parts = m["norm_groups"]
    y = rms_unit(y.view(t_len, parts, inner // parts), eps).reshape(t_len, inner) * w[p + ".norm"]
    return y @ w[p + ".o"].t()


def feed_forward(h, w, p):
    return (silu(h @ w[p + ".gate"].t()) * (h @ w[p + ".up"].t())) @ w[p + ".down"].t()


def mixer(h, w, layer, p, eps):
    m, kind = layer["mixer"], layer["type"]
    if kind == "mamba2":
        return mamba2_mixer(h, w, p, m, eps)
    left = softmax_side(h, w, p + ".left", m["left"], eps, kind)
    if kind == "parallel":
        right = gated_linear_side(h, w, p + ".right", m["right"], eps)
    elif kind == "parallel_2":
        right = time_mix_side(h, w, p + ".right", m["right"], eps)
    else:
        raise ValueError(kind)
    return m["left_scale"] * left + m["right_scale"] * right


def forward(cfg, weights, ids):
    w = {k: v.to(F) for k, v in weights.items() if v.is_floating_point()}
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.as_tensor(ids, dtype=torch.long)] * cfg["embedding"]["scale"]
    streams = []
    for i, layer in enumerate(cfg["layers"]):
        h = norm_one_plus(x, w[f"l{i}.norm1"], eps)
        y = mixer(h, w, layer, f"l{i}.mix", eps)
        if layer.get("mlp") is not None:
            y = y + feed_forward(h, w, f"l{i}.mlp")
        x = x + y
        streams.append(x)
    return norm_one_plus(x, w["final.norm"], eps) @ w["head"].t(), streams


def logits(cfg, weights, ids):
    return forward(cfg, weights, ids)[0]
