"""A plain, slow implementation of the Nezalorn decoder for whole sequences: no cache, no batching, one
function per mechanism, float64 by default. It shares no code with ``nanoinfer_b200``.

The design in this file's notation (T tokens, row t is position t, ``W`` stored [out, in]):

* a layer takes x and gives ``X = x + mixer(rms(x, g1)) + ff(rms(x, g2))`` (both branches read the same x);
  what the next layer reads is the depth mix ``sum_j d[j] X_j`` over the embedding output X_0 and all layer
  results so far;
* mixers: ``latent_attention`` (queries and keys/values through low-rank latents, one rotated key part shared by
  the heads, interleaved rotary pairs with YaRN-scaled frequencies, a sliding window, optionally the latents of an
  earlier layer), ``general_delta`` (a matrix state per head with per-channel decay, removal along the unit key
  and a rank-one write), ``rglru`` (a short causal convolution and a gated diagonal linear recurrence);
* feed-forward: up, PolyNorm (a mix of the rms-normed first three powers), down, with biases;
* logits through the embedding table after the final norm.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def rms_norm(x, gain, eps):
    return rms(x, eps) * gain


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z.pow(3))))


def poly_norm_ff(h, up_w, up_b, down_w, down_b, coef, eps):
    """down(c0 N(z) + c1 N(z^2) + c2 N(z^3) + c3) with z = up(h), N = division by the row's root mean square."""
    z = h @ up_w.t() + up_b
    act = coef[0] * rms(z, eps) + coef[1] * rms(z.pow(2), eps) + coef[2] * rms(z.pow(3), eps) + coef[3]
    return act @ down_w.t() + down_b


# ------------------------------------------------------------------------------------- rotary with YaRN
def yarn_frequencies(dims: int, base: float, scaling: Optional[dict]):
    """(frequency of each of the dims/2 pairs, factor on cos and sin)."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = base ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, orig = float(scaling["factor"]), float(scaling["original"])

    def turn_dim(t):
        return dims * math.log(orig / (2.0 * math.pi * t)) / (2.0 * math.log(base))
    lo = max(math.floor(turn_dim(float(scaling["fast"]))), 0)
    hi = min(math.ceil(turn_dim(float(scaling["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_interleaved(x, positions, freq, mag):
    """x [..., T, n, dims]: pair (2i, 2i+1) turned by positions * freq[i]; cos and sin scaled by mag."""
    ang = positions.to(torch.float64)[:, None] * freq[None, :]          # [T, dims/2]
    c, s = (ang.cos() * mag)[:, None, :], (ang.sin() * mag)[:, None, :]
    u, v = x[..., 0::2], x[..., 1::2]
    out = torch.empty_like(x)
    out[..., 0::2] = u * c - v * s
    out[..., 1::2] = v * c + u * s
    return out


# ------------------------------------------------------------------------------------- latent attention
def latent_kv(h, w, p, m):
    """(latent [T, kv_rank] after its norm, rotated shared key part [T, rot_dim]) of a layer that owns them."""
    T = h.shape[0]
    z = h @ w[p + "dkv"].t()
    c = rms_norm(z[:, :m["kv_rank"]], w[p + "dkv.norm"], m["eps"])
    freq, mag = yarn_frequencies(m["rot"]["dims"], m["rot"]["base"], m["rot"].get("scaling"))
    kr = rotate_interleaved(z[:, m["kv_rank"]:].reshape(T, 1, m["rot_dim"]), torch.arange(T), freq, mag)[:, 0]
    return c, kr


def latent_attention(h, w, p, m, kv):
    """kv = (c, kr) of this layer or of the layer it borrows from. Explicit per-head keys and values."""
    T = h.shape[0]
    H, dn, dr, dv = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    c, kr = kv
    cq = rms_norm(h @ w[p + "dq"].t(), w[p + "dq.norm"], m["eps"])
    q = (cq @ w[p + "uq"].t()).view(T, H, dn + dr)
    freq, mag = yarn_frequencies(m["rot"]["dims"], m["rot"]["base"], m["rot"].get("scaling"))
    q_rot = rotate_interleaved(q[..., dn:], torch.arange(T), freq, mag)
    k_plain = (c @ w[p + "uk"].t()).view(T, H, dn)
    val = (c @ w[p + "uv"].t()).view(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    window = m["mask"]["size"]
    for t in range(T):
        lo = max(0, t - window + 1)
        for hd in range(H):
            s = (k_plain[lo:t + 1, hd] @ q[t, hd, :dn] + kr[lo:t + 1] @ q_rot[t, hd]) * m["scale"]
            e = torch.exp(s - s.max())
            out[t, hd] = (e / e.sum()) @ val[lo:t + 1, hd]
    return out.reshape(T, H * dv) @ w[p + "o"].t()


# ------------------------------------------------------------------------------------- generalized delta rule
def general_delta(h, w, p, m, state=None):
    """state: [H, dim, dim] (key channel x value channel) or None for zeros. Returns (output, last state)."""
    T = h.shape[0]
    H, d = m["heads"], m["dim"]
    r = (h @ w[p + "r"].t()).view(T, H, d)
    k = (h @ w[p + "k"].t()).view(T, H, d)
    v = (h @ w[p + "v"].t()).view(T, H, d)
    decay = torch.exp(-math.exp(-0.5) * torch.sigmoid(torch.tanh(h @ w[p + "w1"].t()) @ w[p + "w2"].t() + w[p + "w0"])).view(T, H, d)
    rate = torch.sigmoid(h @ w[p + "a"].t() + w[p + "a.b"]).view(T, H, d)
    unit = k / torch.sqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)
    S = torch.zeros(H, d, d, dtype=h.dtype) if state is None else state.clone()
    o = torch.zeros(T, H, d, dtype=h.dtype)
    for t in range(T):
        proj = torch.einsum("hk,hkv->hv", unit[t], S)                       # u^T S, from the old state
        S = decay[t][:, :, None] * S - (rate[t] * unit[t])[:, :, None] * proj[:, None, :] + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, r[t])
    o = rms(o, m["eps"]).reshape(T, H * d) * w[p + "norm"] * torch.sigmoid(h @ w[p + "g"].t())
    return o @ w[p + "o"].t(), S


# ------------------------------------------------------------------------------------- gated linear recurrence
def rglru(h, w, p, m, state=None):
    """state: (S [width], the last taps-1 convolution inputs [taps-1, width]) or None. Returns (output, state)."""
    T = h.shape[0]
    W, taps, nb = m["width"], m["conv"], m["blocks"]
    y = gelu_tanh(h @ w[p + "y"].t() + w[p + "y.b"])
    xin = h @ w[p + "x"].t() + w[p + "x.b"]
    hist = torch.zeros(taps - 1, W, dtype=h.dtype) if state is None else state[1]
    padded = torch.cat([hist, xin], 0)
    u = torch.zeros(T, W, dtype=h.dtype) + w[p + "conv.b"]
    for j in range(taps):                                                   # column taps-1 is the current token's
        u = u + padded[j:j + T] * w[p + "conv"][:, j]
    ub = u.view(T, nb, W // nb)
    gr = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, w[p + "ra"]) + w[p + "ra.b"]).reshape(T, W)
    gi = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, w[p + "ri"]) + w[p + "ri.b"]).reshape(T, W)
    log_a = -8.0 * gr * torch.nn.functional.softplus(w[p + "lam"])
    a = torch.exp(log_a)
    S = torch.zeros(W, dtype=h.dtype) if state is None else state[0].clone()
    out = torch.zeros(T, W, dtype=h.dtype)
    for t in range(T):
        S = a[t] * S + torch.sqrt(1.0 - a[t] ** 2) * gi[t] * u[t]
        out[t] = S
    return (out * y) @ w[p + "o"].t(), (S, padded[T:T + taps - 1] if taps > 1 else hist)


# ------------------------------------------------------------------------------------- the model
def forward(cfg: dict, w: Dict[str, torch.Tensor], ids: List[int], return_streams: bool = False):
    """Logits [T, vocab] of a whole sequence; with ``return_streams`` also what every layer hands on."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(ids, dtype=torch.long)]
    results = [x]
    kv_of = {}
    streams = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = dict(layer["mixer"], eps=eps)
        h = rms_norm(x, w[p + "norm1"], eps)
        if layer["type"] == "latent_attention":
            src = m.get("kv_from")
            if src is None:
                kv_of[i] = latent_kv(h, w, p + "mix.", m)
                src = i
            mixed = latent_attention(h, w, p + "mix.", m, kv_of[src])
        elif layer["type"] == "general_delta":
            mixed, _ = general_delta(h, w, p + "mix.", m)
        elif layer["type"] == "rglru":
            mixed, _ = rglru(h, w, p + "mix.", m)
        else:
            raise ValueError(layer["type"])
        out = x + mixed
        if layer.get("mlp") is not None:
            q = p + "mlp."
            out = out + poly_norm_ff(rms_norm(x, w[p + "norm2"], eps), w[q + "up"], w[q + "up.b"], w[q + "down"],
                                     w[q + "down.b"], w[q + "act"], eps)
        results.append(out)
        x = sum(w[p + "dwa"][j] * results[j] for j in range(i + 2))
        streams.append(x)
    logits = rms_norm(x, w["final.norm"], eps) @ w["embed"].t()
    return (logits, streams) if return_streams else logits
