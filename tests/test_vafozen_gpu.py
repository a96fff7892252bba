"""Vafozen on the GPU: every new kernel alone against its plain statement (tests/torch_ops.py, float64), with inputs made
so that a chunk or a window that is one token off, a lost state, a wrong page or a missing bias shows; then the engine in
both precisions against the plain whole-sequence implementation: prompts, token-by-token decoding, portions down to two
tokens, unequal requests in one batch, slots and pages that are used again, long decoding through captured graphs, greedy
generation through the scheduler."""
from types import SimpleNamespace

import pytest
import torch

from gpu_util import assert_close
from torch_ops import TorchOps
from vafozen_util import CFG_A, CFG_B, pair, pair2, plain_logits, softmax_half, ssm, tokens, with_mlp, write_model

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def ops():
    from nanoinfer_b200.csrc.lib import load_kernels
    return load_kernels()


def batch(q_lens, before, page_size=4, slots=None, seed=0, num_pages=0, device=DEV):
    """A step's context as the engine builds it: requests with ``before`` tokens cached bring ``q_lens`` new ones.
    Pages are handed out in a shuffled order."""
    r = len(q_lens)
    ctx_lens = [b + q for b, q in zip(before, q_lens)]
    need = sum(-(-c // page_size) for c in ctx_lens)
    num_pages = max(num_pages, need + 3)
    order = torch.randperm(num_pages, generator=torch.Generator().manual_seed(seed)).tolist()
    width = max(-(-c // page_size) for c in ctx_lens)
    bt = torch.full((r, width), -1, dtype=torch.int32)
    for i, c in enumerate(ctx_lens):
        for p in range(-(-c // page_size)):
            bt[i, p] = order.pop()
    q_start = torch.zeros(r + 1, dtype=torch.int32)
    q_start[1:] = torch.tensor(q_lens).cumsum(0)
    slots = list(slots) if slots is not None else list(range(r))
    ctx = SimpleNamespace(
        num_tokens=sum(q_lens),
        positions=torch.cat([torch.arange(b, b + q, dtype=torch.int32) for b, q in zip(before, q_lens)]).to(device),
        req_index=torch.cat([torch.full((q,), i, dtype=torch.int32) for i, q in enumerate(q_lens)]).to(device),
        q_start=q_start.to(device), ctx_lens=torch.tensor(ctx_lens, dtype=torch.int32, device=device),
        state_slots=torch.tensor(slots, dtype=torch.int32, device=device),
        host=SimpleNamespace(q_lens=list(q_lens), ctx_lens=ctx_lens, slots=slots, num_requests=r))
    return ctx, bt.to(device), num_pages


def to_cpu(ctx):
    return SimpleNamespace(num_tokens=ctx.num_tokens, positions=ctx.positions.cpu(), req_index=ctx.req_index.cpu(),
                           q_start=ctx.q_start.cpu(), ctx_lens=ctx.ctx_lens.cpu(), state_slots=ctx.state_slots.cpu(), host=ctx.host)


def rnd(*shape, seed=0, scale=1.0):
    return (torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale).to(DEV)


# ------------------------------------------------------------------------------------------ pointwise kernels
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("m,heads,d", [(5, 3, 20), (3, 4, 300)])        # narrow parts: a warp each; wide parts: a block each
@pytest.mark.parametrize("case", ["head_norm_shared_gain_silu", "gate_first_skip_groups", "gate_only", "norm_only_full_gain"])
def test_gate_norm_and_skip(ops, dtype, case, m, heads, d):
    n = heads * d
    wide = rnd(m, 3 * n + 7, seed=1, scale=1.5)
    o, gate, skip = wide[:, 1:1 + n], wide[:, n + 3:2 * n + 3], wide[:, 2 * n + 5:3 * n + 5]        # rows lie apart
    kw = {"head_norm_shared_gain_silu": dict(groups=heads, eps=1e-5, gain32=rnd(d, seed=2), gate32=gate, gate_kind="silu", out_scale=0.9),
          "gate_first_skip_groups": dict(groups=2, eps=1e-6, gain32=rnd(n, seed=3), gate32=gate, gate_kind="silu", gate_first=True,
                                         skip32=skip, skip_coef32=rnd(heads, seed=4), out_scale=1.0),
          "gate_only": dict(gate32=gate, gate_kind="sigmoid", out_scale=0.8),
          "norm_only_full_gain": dict(groups=heads, eps=1e-5, gain32=rnd(n, seed=5))}[case]
    out = torch.empty(m, n, dtype=dtype, device=DEV)
    ops.gated_norm(o, out, **kw)
    ref = torch.empty(m, n, dtype=torch.float64)
    TorchOps().gated_norm(o.cpu(), ref, **{k: (v.cpu() if torch.is_tensor(v) else v) for k, v in kw.items()})
    assert_close(out, ref, dtype, case)


def test_embedding_factor(ops):
    table = rnd(50, 24, seed=1).to(torch.bfloat16)
    ids = torch.tensor([3, 49, 0, 7], dtype=torch.int32, device=DEV)
    out = torch.empty(4, 24, dtype=torch.float32, device=DEV)
    ops.embed(ids, table, out, 11.0)
    assert torch.equal(out, table[ids.long()].float() * 11.0)


def test_decays_and_step_sizes(ops):
    z = torch.cat([rnd(6, 40, seed=1, scale=3.0), torch.tensor([[-40.0, 40.0, 0.0, -100.0, 90.0] * 8], device=DEV)])
    for kind, param in (("sigmoid_root", 16.0), ("sigmoid_root", 1.0), ("exp_neg_exp", 1.0)):
        out, ref = torch.empty_like(z), torch.empty(z.shape, dtype=torch.float32)
        ops.decay_map(z, out, kind, param)
        TorchOps().decay_map(z.cpu(), ref, kind, param)
        assert torch.isfinite(out).all()
        assert (out.cpu().double() - ref.double()).abs().max().item() <= 1e-7, kind      # rounded once from 64 bits
    raw, bias, a_log = rnd(9, 5, seed=2, scale=4.0), rnd(5, seed=3), rnd(5, seed=4)
    raw[0, 0], raw[1, 1] = 60.0, -60.0          # no clamp: the step follows its input up, and goes to zero below
    dt, decay = torch.empty(9, 5, device=DEV), torch.empty(9, 5, device=DEV)
    ops.step_sizes(raw, bias, a_log, dt, decay)
    rdt, rdecay = torch.empty(9, 5), torch.empty(9, 5)
    TorchOps().step_sizes(raw.cpu(), bias.cpu(), a_log.cpu(), rdt, rdecay)
    assert torch.allclose(dt.cpu(), rdt, rtol=1e-6, atol=1e-30)
    assert (decay.cpu() - rdecay).abs().max().item() <= 2e-7          # a decay is at most one
    assert dt[0, 0].item() > 55.0 and 0.0 < dt[1, 1].item() < 1e-20


# ------------------------------------------------------------------------------------------ convolution, token shift
@pytest.mark.parametrize("width,taps,act", [(12, 1, "none"), (48, 2, "silu"), (64, 4, "none"), (40, 5, "silu"), (130, 7, "none")])
def test_short_convolution_in_steps_keeps_its_history(ops, width, taps, act):
    """Three steps of unequal requests (portions shorter than the history among them), then a request that takes over a
    slot; the state lies in the middle of a wider state row."""
    off, total = 5, 5 + (taps - 1) * width + 9
    state = torch.zeros(4, total, device=DEV)
    state[:, :off], state[:, off + (taps - 1) * width:] = 7.0, -7.0       # neighbours that must stay as they are
    ref_state = state.cpu().clone()
    w, bias = rnd(width, taps, seed=1), rnd(width, seed=2)
    for step, (q_lens, slots) in enumerate([([5, 1, 2], [2, 0, 1]), ([1, 3, 1], [2, 0, 1]), ([2, 6], [0, 2])]):
        ctx, _, _ = batch(q_lens, [0] * len(q_lens), slots=slots)
        wide = rnd(sum(q_lens), width + 3, seed=10 + step)
        x = wide[:, 2:2 + width]
        out, ref = torch.empty(sum(q_lens), width, device=DEV), torch.empty(sum(q_lens), width)
        ops.conv_tokens(x, w, bias if act == "silu" else None, act, state, off, ctx, out, taps)
        if taps > 1:
            ops.conv_tail(x, state, off, ctx, taps)
        TorchOps().conv_tokens(x.cpu(), w.cpu(), bias.cpu() if act == "silu" else None, act, ref_state, off, to_cpu(ctx), ref, taps)
        if taps > 1:
            TorchOps().conv_tail(x.cpu(), ref_state, off, to_cpu(ctx), taps)
        assert_close(out, ref, torch.float32, f"step {step}")
        assert_close(state, ref_state, torch.float32, f"state after step {step}")
    assert (state[:, :off] == 7.0).all() and (state[:, off + (taps - 1) * width:] == -7.0).all()
    # both in one call: few tokens take one launch, many take two; the same bits either way
    for q_lens in ([3, 1, 16], [40, 2]):
        ctx, _, _ = batch(q_lens, [0] * len(q_lens), slots=[1, 3, 0][:len(q_lens)])
        x = rnd(sum(q_lens), width, seed=30 + len(q_lens))
        s_a, s_b = state.clone(), state.clone()
        out_a, out_b = torch.empty(sum(q_lens), width, device=DEV), torch.empty(sum(q_lens), width, device=DEV)
        ops.conv_step(x, w, bias, act, s_a, off, ctx, out_a, taps)
        ops.conv_tokens(x, w, bias, act, s_b, off, ctx, out_b, taps)
        if taps > 1:
            ops.conv_tail(x, s_b, off, ctx, taps)
        assert torch.equal(out_a, out_b) and torch.equal(s_a, s_b)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_token_shift_reads_the_token_before_and_keeps_the_last(ops, dtype):
    width, off = 70, 3
    state = torch.zeros(3, off + width + 2, device=DEV)
    ref_state = state.cpu().clone()
    mu = torch.rand(5, width, generator=torch.Generator().manual_seed(1)).to(DEV)
    for step, (q_lens, slots) in enumerate([([4, 1], [1, 0]), ([1, 1], [1, 0]), ([3, 2], [0, 2])]):
        ctx, _, _ = batch(q_lens, [0] * len(q_lens), slots=slots)
        h = rnd(sum(q_lens), width, seed=20 + step).to(dtype)
        out, ref = torch.empty(5, sum(q_lens), width, dtype=dtype, device=DEV), torch.empty(5, sum(q_lens), width, dtype=torch.float64)
        ops.token_shift(h, mu, state, off, ctx, out)
        TorchOps().token_shift(h.cpu(), mu.cpu(), ref_state, off, to_cpu(ctx), ref)
        assert_close(out, ref, dtype, f"step {step}")
        assert torch.equal(state.cpu(), ref_state)
    assert (state[:, :off] == 0).all() and (state[:, off + width:] == 0).all()


# ------------------------------------------------------------------------------------------ the walk over matrix states
def _walk_inputs(m, heads, kq_heads, dk, dv, seed, per_head_decay):
    q, k = rnd(m, kq_heads * dk, seed=seed), rnd(m, kq_heads * dk, seed=seed + 1, scale=0.5)
    v = rnd(m, heads * dv, seed=seed + 2)
    w = torch.sigmoid(rnd(m, heads if per_head_decay else heads * dk, seed=seed + 3) + 2.0)
    return q, k, v, w


@pytest.mark.parametrize("heads,kq_heads,dk,dv,mode", [(1, 1, 8, 5, "post"), (3, 3, 20, 12, "bonus"), (4, 2, 48, 40, "scalar"),
                                                      (2, 2, 64, 64, "post"), (2, 1, 100, 33, "scalar"), (1, 1, 130, 70, "bonus"),
                                                      (6, 3, 1, 8, "scalar")])
def test_walk_against_plain_and_cut_anywhere(ops, heads, kq_heads, dk, dv, mode):
    """Whole, then in portions (two tokens, one token, across the kernel's staging size) beside another request: the
    same bits whatever the cut; the state sits behind other columns of a wider state row."""
    n, off = 37, 11
    size = heads * dv * dk
    q, k, v, w = _walk_inputs(n, heads, kq_heads, dk, dv, 1, mode == "scalar")
    bonus = rnd(heads, dk, seed=7) if mode == "bonus" else None
    v_scale = torch.rand(n, heads, generator=torch.Generator().manual_seed(8)).to(DEV) if mode == "scalar" else None
    kw = dict(q_scale=0.5 if mode == "post" else 1.0)
    state = torch.zeros(3, off + size + 4, device=DEV)
    ctx, _, _ = batch([n], [0], slots=[1])
    whole = torch.empty(n, heads * dv, device=DEV)
    ops.linear_state_scan(q, k, v, w, state, off, ctx, whole, heads, kq_heads, dk, dv, bonus32=bonus, v_scale32=v_scale, **kw)
    ref_state = torch.zeros(3, off + size + 4)
    ref = torch.empty(n, heads * dv)
    TorchOps().linear_state_scan(q.cpu(), k.cpu(), v.cpu(), w.cpu(), ref_state, off, to_cpu(ctx), ref, heads, kq_heads, dk, dv,
                                 bonus32=None if bonus is None else bonus.cpu(), v_scale32=None if v_scale is None else v_scale.cpu(), **kw)
    assert_close(whole, ref, torch.float32, "whole")
    assert_close(state, ref_state, torch.float32, "state")
    assert (state[[0, 2]] == 0).all() and (state[1, :off] == 0).all() and (state[1, off + size:] == 0).all()
    # in portions, beside another request whose rows come first
    state2 = torch.zeros(3, off + size + 4, device=DEV)
    got, pos = [], 0
    oq, ok_, ov, ow = _walk_inputs(60, heads, kq_heads, dk, dv, 50, mode == "scalar")
    opos = 0
    for c in [2, 1, 9, 17, 1, 2, 5]:
        oc = min(3, 60 - opos)
        ctx, _, _ = batch([oc, c], [0, 0], slots=[2, 0])
        cat = lambda a, b: torch.cat([a[opos:opos + oc], b[pos:pos + c]])
        out = torch.empty(oc + c, heads * dv, device=DEV)
        vs = None if v_scale is None else torch.cat([torch.ones(oc, heads, device=DEV), v_scale[pos:pos + c]])
        ops.linear_state_scan(cat(oq, q), cat(ok_, k), cat(ov, v), cat(ow, w), state2, off, ctx, out, heads, kq_heads, dk, dv,
                              bonus32=bonus, v_scale32=vs, **kw)
        got.append(out[oc:])
        pos, opos = pos + c, opos + oc
    assert torch.equal(torch.cat(got), whole), "the cut changed bits"
    assert torch.equal(state2[0], state[1])


@pytest.mark.parametrize("heads,kq_heads,dk,dv,mode", [(2, 2, 20, 12, "bonus"), (4, 2, 48, 40, "scalar"), (2, 2, 64, 64, "post"), (1, 1, 130, 70, "bonus")])
def test_long_prompts_walked_in_segments(ops, heads, kq_heads, dk, dv, mode):
    """A prompt of 700 tokens beside a short request and a decoded token: segments side by side give what the walk in
    order gives, up to rounding; the states go on from there (a second step in order)."""
    q_lens, slots, off = [700, 3, 1], [2, 0, 1], 7
    m, size = sum(q_lens), heads * dv * dk
    q, k, v, w = _walk_inputs(m, heads, kq_heads, dk, dv, 3, mode == "scalar")
    bonus = rnd(heads, dk, seed=7) if mode == "bonus" else None
    v_scale = torch.rand(m, heads, generator=torch.Generator().manual_seed(8)).to(DEV) if mode == "scalar" else None
    ctx, _, _ = batch(q_lens, [0, 0, 0], slots=slots)
    start = rnd(3, off + size + 2, seed=9, scale=0.3)          # the requests do not start from zero
    outs, states = [], []
    for seg_len in (0, None, 64):
        state, out = start.clone(), torch.empty(m, heads * dv, device=DEV)
        ops.linear_state_scan(q, k, v, w, state, off, ctx, out, heads, kq_heads, dk, dv, bonus32=bonus, v_scale32=v_scale, seg_len=seg_len)
        outs.append(out); states.append(state)
    ref_state, ref = start.cpu().clone(), torch.empty(m, heads * dv)
    TorchOps().linear_state_scan(q.cpu(), k.cpu(), v.cpu(), w.cpu(), ref_state, off, to_cpu(ctx), ref, heads, kq_heads, dk, dv,
                                 bonus32=None if bonus is None else bonus.cpu(), v_scale32=None if v_scale is None else v_scale.cpu())
    for out, state, what in zip(outs, states, ("in order", "segments of 128", "segments of 64")):
        assert_close(out, ref, torch.float32, what)
        assert_close(state, ref_state, torch.float32, what + ": state")
        assert torch.equal(state[:, :off], start[:, :off]) and torch.equal(state[:, off + size:], start[:, off + size:])
    assert torch.equal(outs[0][700:], outs[1][700:])            # the short requests are walked in order either way
    assert not torch.equal(outs[0][:700], outs[1][:700]) or dk == 1


def test_walk_remembers_a_far_key(ops):
    """One token writes a value under a key no other token uses; 600 tokens later a query for that key still finds it,
    scaled by the product of the decays in between."""
    n, dk, dv = 640, 16, 8
    q, k, v = torch.zeros(n, dk, device=DEV), rnd(n, dk, seed=1, scale=0.3), rnd(n, dv, seed=2)
    k[:, 3] = 0.0
    k[20] = 0.0
    k[20, 3] = 1.0
    q[630, 3] = 1.0
    w = torch.full((n, dk), 0.999, device=DEV)
    state = torch.zeros(1, dk * dv, device=DEV)
    out = torch.empty(n, dv, device=DEV)
    ctx, _, _ = batch([n], [0])
    ops.linear_state_scan(q, k, v, w, state, 0, ctx, out, 1, 1, dk, dv)
    want = v[20].double() * 0.999 ** 610
    assert (out[630].double() - want).abs().max().item() <= 1e-5 * want.abs().max().item() + 1e-7
    assert out[631].abs().max().item() == 0.0


# ------------------------------------------------------------------------------------------ attention with options
def _fill_pages(ops, dtype, ctx, bt, page, num_pages, heads, kv, dk, dv, qkv, gains=None, freq=None, rot=0, eps=1e-6):
    kp = torch.zeros(num_pages, kv, page, dk, dtype=dtype, device=DEV)
    vp = torch.zeros(num_pages, kv, page, dv, dtype=dtype, device=DEV)
    q = torch.empty(qkv.shape[0], heads * dk, dtype=dtype, device=DEV)
    g = gains or (None, None)
    ops.attention_prepare(qkv, q, heads, kv, dk, dv, g[0], g[1], eps, freq, rot, ctx, bt, page, kp, vp, True)
    return q, kp, vp


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv,dk,dv,rot,normed,page", [(3, 1, 12, 8, 0, True, 4), (4, 2, 8, 12, 4, False, 4), (2, 2, 64, 64, 64, False, 16),
                                                            (6, 3, 96, 40, 32, True, 8), (1, 1, 130, 3, 2, False, 16)])
def test_prepare_norms_rotates_and_writes_pages(ops, dtype, heads, kv, dk, dv, rot, normed, page):
    q_lens, before = [5, 1, 9], [3, 40, 0]
    ctx, bt, num_pages = batch(q_lens, before, page_size=page)
    m = sum(q_lens)
    wide = rnd(m, (heads + kv) * dk + kv * dv + 3, seed=1)
    qkv = wide[:, 1:1 + (heads + kv) * dk + kv * dv]
    gains = (rnd(dk, seed=2), rnd(dk, seed=3)) if normed else None
    freq = torch.pow(torch.tensor(50000.0, dtype=torch.float64), -2.0 * torch.arange(rot // 2, dtype=torch.float64) / max(rot, 1)).float().to(DEV) if rot else None
    q, kp, vp = _fill_pages(ops, dtype, ctx, bt, page, num_pages, heads, kv, dk, dv, qkv, gains, freq, rot)
    rq = torch.empty(m, heads * dk, dtype=torch.float64)
    rk, rv = torch.zeros(kp.shape, dtype=torch.float64), torch.zeros(vp.shape, dtype=torch.float64)
    TorchOps().attention_prepare(qkv.cpu(), rq, heads, kv, dk, dv, None if gains is None else gains[0].cpu(), None if gains is None else gains[1].cpu(),
                                 1e-6, None if freq is None else freq.cpu(), rot, to_cpu(ctx), bt.cpu(), page, rk, rv, True)
    assert_close(q, rq, dtype, "queries")
    assert_close(kp, rk, dtype, "key pages")
    assert_close(vp, rv, dtype, "value pages")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("opts", [dict(), dict(chunk=7), dict(chunk=32), dict(chunk=33, slopes=True), dict(window=9), dict(softcap=2.0),
                                  dict(softcap=12.0, slopes=True, chunk=100), dict(window=40, chunk=64)])
@pytest.mark.parametrize("heads,kv,dk,dv,page", [(3, 1, 12, 8, 4), (4, 2, 96, 64, 16), (2, 2, 40, 104, 8), (8, 1, 128, 128, 16), (2, 2, 36, 100, 8)])
def test_attention_over_pages_with_options(ops, dtype, opts, heads, kv, dk, dv, page):
    """Prompt portions beside decoded tokens over contexts that span pages, chunks and windows; float and storage-type
    outputs; an output factor."""
    q_lens, before = [1, 1, 30, 7], [150, 6, 100, 0]
    ctx, bt, num_pages = batch(q_lens, before, page_size=page)
    # the cached positions before this step: written by an earlier "step" that covers 0 .. before
    full_ctx, full_bt, _ = batch([b + q for b, q in zip(before, q_lens)], [0] * 4, page_size=page)
    m_full = sum(b + q for b, q in zip(before, q_lens))
    qkv = rnd(m_full, (heads + kv) * dk + kv * dv, seed=3, scale=0.7)
    q_all, kp, vp = _fill_pages(ops, dtype, full_ctx, full_bt, page, num_pages, heads, kv, dk, dv, qkv)
    rows = torch.cat([torch.arange(s + b, s + b + q) for s, b, q in zip(full_ctx.q_start.cpu().tolist(), before, q_lens)]).to(DEV)
    q = q_all[rows].contiguous()
    slopes = torch.pow(2.0, -8.0 * torch.arange(1, heads + 1, dtype=torch.float64) / heads).float().to(DEV) if opts.get("slopes") else None
    args = (heads, kv, dk, dv, 0.3, opts.get("softcap", 0.0), slopes, opts.get("window", 0), opts.get("chunk", 0))
    ref = torch.empty(sum(q_lens), heads * dv, dtype=torch.float64)
    TorchOps().attention_flex(q.cpu(), ref, *args[:6], None if slopes is None else slopes.cpu(), *args[7:], 0.8, to_cpu(ctx), full_bt.cpu(),
                              page, kp.cpu(), vp.cpu())
    paths = [ops] if dtype == torch.float32 else [ops, ops.with_options(force_general_attention=True)]      # tensor cores; the general kernel
    if dtype == torch.bfloat16:       # decoded tokens alone: their keys are shared out to several CTAs and merged
        dq, dbefore = [1, 1, 1], [150, 6, 129]
        dctx, _, _ = batch(dq, dbefore, page_size=page)
        drows = torch.tensor([full_ctx.q_start[i].item() + b for i, b in enumerate(dbefore)], device=DEV)
        dref = torch.empty(3, heads * dv, dtype=torch.float64)
        TorchOps().attention_flex(q_all[drows].cpu(), dref, *args[:6], None if slopes is None else slopes.cpu(), *args[7:], 0.8, to_cpu(dctx),
                                  full_bt.cpu(), page, kp.cpu(), vp.cpu())
        for k in (ops, ops.with_options(fixed_decode_splits=5)):
            out = torch.empty(3, heads * dv, dtype=dtype, device=DEV)
            k.attention_flex(q_all[drows].contiguous(), out, *args, 0.8, dctx, full_bt, page, kp, vp)
            assert_close(out, dref, dtype, f"{opts} decoded tokens, splits fixed {k is not ops}")
    for k in paths:
        for out_dtype in {torch.float32, dtype}:
            out = torch.empty(sum(q_lens), heads * dv, dtype=out_dtype, device=DEV)
            k.attention_flex(q, out, *args, 0.8, ctx, full_bt, page, kp, vp)
            assert_close(out, ref, dtype, f"{opts} out {out_dtype} general {k is not ops}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("decode", [False, True])
@pytest.mark.parametrize("chunk,page", [(6, 4), (32, 8), (40, 16), (64, 16), (100, 16)])
def test_a_key_at_the_chunks_start_is_seen_and_the_one_before_is_not(ops, chunk, page, decode, dtype):
    """All keys are alike but two: the first key of the query's chunk and the last key of the chunk before carry values of
    their own and a score that stands out. The query at the chunk's last position must return the first one's value; the
    query one position on (a new chunk) neither."""
    dk, dv, n = 16, 8, 3 * chunk + 1
    qkv = torch.zeros(n, 2 * dk + dv, device=DEV)
    qkv[:, dk] = 1.0                                     # every key: e0
    first, before_it = 2 * chunk, 2 * chunk - 1
    for pos, mark in ((first, 1.0), (before_it, 2.0)):
        qkv[pos, dk + 1] = 9.0                           # the two marked keys also carry e1
        qkv[pos, 2 * dk:] = mark
    qkv[:, 1] = 9.0                                      # every query asks for e1
    q_pos = [first, first + 1, first + chunk - 1]        # the chunk's own first position, the next one, its last one
    full_ctx, bt, num_pages = batch([n], [0], page_size=page)
    q_all, kp, vp = _fill_pages(ops, dtype, full_ctx, bt, page, num_pages, 1, 1, dk, dv, qkv)
    for p in q_pos:
        if p >= n:
            continue
        ctx, _, _ = (batch([1], [p], page_size=page) if decode else batch([2], [p - 1], page_size=page))
        rows = [p] if decode else [p - 1, p]
        out = torch.empty(len(rows), dv, device=DEV)
        ops.attention_flex(q_all[rows].contiguous(), out, 1, 1, dk, dv, 1.0, 0.0, None, 0, chunk, 1.0, ctx, bt, page, kp, vp)
        got = out[-1, 0].item()
        assert abs(got - 1.0) < 1e-3, (p, got)           # the chunk's first key, never the one before it
    # the very next position opens a new chunk: only itself is visible
    p = first + chunk
    if p < n:
        ctx, _, _ = batch([1], [p], page_size=page)
        out = torch.empty(1, dv, device=DEV)
        ops.attention_flex(q_all[[p]].contiguous(), out, 1, 1, dk, dv, 1.0, 0.0, None, 0, chunk, 1.0, ctx, bt, page, kp, vp)
        assert out.abs().max().item() < 1e-6


def test_distance_bias_and_cap_show_in_the_weights(ops):
    """Equal keys everywhere: with a slope the weights fall off by exp(-slope * distance); a cap far below the raw score
    flattens a key that would otherwise take everything."""
    dk, dv, n, page = 8, 4, 20, 4
    qkv = torch.zeros(n, 2 * dk + dv, device=DEV)
    qkv[:, 2 * dk] = torch.arange(n, dtype=torch.float32)             # value = own position
    full_ctx, bt, num_pages = batch([n], [0], page_size=page)
    q_all, kp, vp = _fill_pages(ops, torch.float32, full_ctx, bt, page, num_pages, 1, 1, dk, dv, qkv)
    ctx, _, _ = batch([1], [n - 1], page_size=page)
    out = torch.empty(1, dv, device=DEV)
    slope = torch.tensor([0.5], device=DEV)
    ops.attention_flex(q_all[[n - 1]].contiguous(), out, 1, 1, dk, dv, 1.0, 0.0, slope, 0, 0, 1.0, ctx, bt, page, kp, vp)
    wts = torch.exp(-0.5 * torch.arange(n - 1, -1, -1, dtype=torch.float64))
    want = (wts * torch.arange(n, dtype=torch.float64)).sum() / wts.sum()
    assert abs(out[0, 0].item() - want.item()) < 1e-4
    qkv[:, 0], qkv[:, dk] = 10.0, 0.0
    qkv[5, dk] = 10.0                                                 # raw score 100 at position 5, 0 elsewhere
    q_all, kp, vp = _fill_pages(ops, torch.float32, full_ctx, bt, page, num_pages, 1, 1, dk, dv, qkv)
    ops.attention_flex(q_all[[n - 1]].contiguous(), out, 1, 1, dk, dv, 1.0, 2.0, None, 0, 0, 1.0, ctx, bt, page, kp, vp)
    wts = torch.ones(n, dtype=torch.float64)
    wts[5] = torch.exp(torch.tensor(2.0, dtype=torch.float64) * torch.tanh(torch.tensor(50.0, dtype=torch.float64)))
    want = (wts * torch.arange(n, dtype=torch.float64)).sum() / wts.sum()
    assert abs(out[0, 0].item() - want.item()) < 1e-4


# ------------------------------------------------------------------------------------------ the engine
# Sizes near a real layer's ratios: the matrix products take the tensor-core kernels, the prompt spans pages and chunks.
CFG_C = {"architecture": "Vafozen", "vocab": 509, "width": 256, "norm": {"eps": 1e-5}, "embedding": {"scale": 8.0}, "layers": [
    with_mlp(pair2(softmax_half(4, 2, 64, 32, conv=3, rot=(32, 40000.0), softcap=15.0), 2, 64), 512),
    with_mlp(ssm(8, 32, 64, 2, 4, 4), 384),
    with_mlp(pair(softmax_half(4, 1, 32, 64, mask=40), 2, 32, vdim=64, tau=8.0, rank=16), 512),
    with_mlp(ssm(4, 64, 32, 1, 1, 2), None),
]}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {"A": write_model(str(tmp_path_factory.mktemp("vaf_a")), CFG_A, 11, strip_rank=True),
            "B": write_model(str(tmp_path_factory.mktemp("vaf_b")), CFG_B, 12),
            "C": write_model(str(tmp_path_factory.mktemp("vaf_c")), CFG_C, 13)}


def gpu_engine(folder, dtype, page=4, pages=96, slots=4, graphs=True):
    from nanoinfer_b200.config import EngineConfig
    from nanoinfer_b200.engine import Engine
    return Engine(folder, EngineConfig(dtype=dtype, page_size=page, num_pages=pages, max_batch=slots, cuda_graphs=graphs))


def run_cut(eng, name, ids, cuts):
    from nanoinfer_b200.engine import StepEntry
    rc = eng.open(name)
    out, pos = [], 0
    for n in cuts:
        out.append(eng.step([StepEntry(rc, ids[pos:pos + n], list(range(n)))]).clone())
        pos += n
    assert pos == len(ids)
    eng.close(rc)
    eng.check_device()
    return torch.cat(out)


def vocab_of(folder):
    import json, os
    with open(os.path.join(folder, "config.json")) as f:
        return json.load(f)["vocab"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,n,page", [("A", 45, 4), ("B", 41, 8), ("C", 300, 16)])
def test_engine_prompts_decoding_and_portions_equal_plain(folders, dtype, name, n, page):
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    ids = tokens(n, vocab_of(folders[name]), 5)
    ref = plain_logits(folders[name], ids)
    eng = gpu_engine(folders[name], dtype, page=page, pages=64)
    whole = run_cut(eng, "whole", ids, [n])
    assert_close(whole, ref, td, "whole prompt")
    tail = 12 if n > 100 else n - 1
    assert_close(run_cut(eng, "decode", ids, [n - tail] + [1] * tail), ref, td, "prompt, then token by token")
    cuts = [2, 7, 2, 13, 1, 1, 5, 2]
    cuts = cuts + [n - sum(cuts) - 2, 2]
    got = run_cut(eng, "cut", ids, cuts)
    assert_close(got, ref, td, "portions")
    if dtype == "float32":      # the same arithmetic per position whatever the cut
        assert (got - whole).abs().max().item() <= 1e-5 * max(1.0, ref.abs().max().item())
    eng.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_engine_unequal_requests_and_reused_slots_and_pages(folders, dtype):
    from nanoinfer_b200.engine import StepEntry
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    eng = gpu_engine(folders["A"], dtype, page=4, pages=24, slots=2)
    seqs = {k: tokens(n, 131, s) for k, n, s in (("p", 23, 1), ("q", 9, 2), ("r", 17, 3), ("s", 12, 4))}
    got, at, live = {k: [] for k in seqs}, {k: 0 for k in seqs}, {}
    plan = [[("p", 6), ("q", 2)], [("p", 1), ("q", 5)], [("p", 7), ("q", 2)], [("p", 1), ("r", 9)], [("r", 1), ("p", 1)],
            [("p", 7), ("r", 7)], [("s", 3)], [("s", 1)], [("s", 8)]]
    for step in plan:
        entries = []
        for k, n in step:
            if k not in live:
                live[k] = eng.open(k)
            entries.append(StepEntry(live[k], seqs[k][at[k]:at[k] + n], list(range(n))))
        logits = eng.step(entries).clone()
        row = 0
        for k, n in step:
            got[k].append(logits[row:row + n])
            row += n
            at[k] += n
            if at[k] == len(seqs[k]):
                eng.close(live.pop(k))
        eng.cache.check()
    for k in seqs:
        assert_close(torch.cat(got[k]), plain_logits(folders["A"], seqs[k]), td, f"request {k}")


def test_long_decoding_through_captured_graphs_passes_chunks_and_pages(folders):
    """150 tokens one by one (two requests side by side, so the steps are replayed from a captured graph): the chunk of 7
    is passed many times, pages behind it go back to the pool, the states and histories carry on."""
    from nanoinfer_b200.engine import StepEntry
    eng = gpu_engine(folders["A"], "float32", page=4, pages=96, slots=2)
    seqs = [tokens(150, 131, 31), tokens(140, 131, 32)]
    rcs = [eng.open("a"), eng.open("b")]
    got = [[], []]
    for t in range(150):
        entries = [StepEntry(rcs[i], [seqs[i][t]], [0]) for i in range(2) if t < len(seqs[i])]
        logits = eng.step(entries).clone()
        for j, i in enumerate(i for i in range(2) if t < len(seqs[i])):
            got[i].append(logits[j])
    assert eng.graph_launches > 0
    for i in range(2):
        assert_close(torch.stack(got[i]), plain_logits(folders["A"], seqs[i]), torch.float32, f"request {i}")


@pytest.mark.parametrize("portion", [8, 256])
def test_prompt_portions_replayed_from_a_captured_graph(folders, portion):
    """Portions of one recurring shape are captured the third time the shape is seen and replayed from then on: states,
    histories, pages and (for portions of 256 tokens) the segments' scratch must go on through captured steps as through
    eager ones."""
    from nanoinfer_b200.engine import StepEntry
    eng = gpu_engine(folders["A"], "float32", page=4 if portion == 8 else 16, pages=400, slots=2)
    assert eng._portion_graphs is not None
    eng._portion_graphs.min_tokens = 8
    n = 12 * portion if portion == 8 else 9 * portion      # a shape includes the block tables' widths, rounded up to powers of two
    ids = tokens(n, 131, 77)
    rc = eng.open("p")
    got = [eng.step([StepEntry(rc, ids[i:i + portion], list(range(portion)))]).clone() for i in range(0, n, portion)]
    assert eng._portion_graphs.captured and eng.graph_launches > 0
    assert_close(torch.cat(got), plain_logits(folders["A"], ids), torch.float32, "portions through a graph")
    eng.close(rc)
    eng.cache.check()


def test_greedy_generation_through_the_scheduler(folders):
    from nanoinfer_b200.api import Model
    from nanoinfer_b200.config import EngineConfig
    from nanoinfer_b200.engine.scheduler import Request, Scheduler
    model = Model(folders["B"], EngineConfig(dtype="float32", page_size=8, num_pages=32, max_batch=3, max_tokens_per_step=8))
    sched = Scheduler(model)
    prompts = [tokens(13, 77, 21), tokens(5, 77, 22), tokens(19, 77, 23), tokens(3, 77, 24)]
    for i, p in enumerate(prompts):
        sched.add(Request(f"g{i}", p, max_tokens=8))
    done = sched.run()
    for i, p in enumerate(prompts):
        ids = list(p)
        for _ in range(8):
            row = plain_logits(folders["B"], ids)[-1]
            top = row.topk(2).values
            assert top[0] - top[1] > 1e-3, "the test's model has a tie here; pick another seed"
            ids.append(int(row.argmax()))
        assert done[f"g{i}"] == ids[len(p):], i
    model.engine.cache.check()


def test_a_far_token_reaches_the_logits_through_every_kind_of_memory(tmp_path):
    """One layer at a time (softmax attention over all keys, a slowly decaying matrix state, a state-space state): changing
    the FIRST token of a 400-token prompt must move the last position's logits as the plain implementation says."""
    from nanoinfer_b200.engine import StepEntry
    slow = lambda t: [t[k].fill_(-6.0) for k in t if k.endswith((".w0", ".A_log"))] and None      # decays close to one
    cases = {"softmax": [with_mlp(pair2(softmax_half(2, 1, 16, 16, conv=2, rot=(8, 1e4), softcap=30.0), 1, 8), 64)],
             "time_mix": [with_mlp(pair2(softmax_half(1, 1, 8, 8, conv=1, rot=(2, 1e4), softcap=30.0), 2, 16, right_scale=3.0), None)],
             "ssm": [with_mlp(ssm(2, 16, 16, 1, 1, 2), None)]}
    for name, layers in cases.items():
        cfg = {"architecture": "Vafozen", "vocab": 64, "width": 48, "norm": {"eps": 1e-6}, "embedding": {"scale": 2.0}, "layers": layers}
        d = write_model(str(tmp_path / name), cfg, 5, weights=slow)
        ids = tokens(400, 64, 3)
        other = [(ids[0] + 1) % 64] + ids[1:]
        ref_a, ref_b = plain_logits(d, ids)[-1], plain_logits(d, other)[-1]
        assert (ref_a - ref_b).abs().max().item() > 1e-3, f"{name}: the test's model forgets its first token"
        eng = gpu_engine(d, "float32", page=16, pages=64, slots=2)
        for seq, ref in ((ids, ref_a), (other, ref_b)):
            rc = eng.open("x")
            eng.step([StepEntry(rc, seq[:390], [])])
            last = None
            for t in seq[390:]:
                last = eng.step([StepEntry(rc, [t], [0])]).clone()
            eng.close(rc)
            assert_close(last[0], ref, torch.float32, name)


@pytest.mark.parametrize("seed,dtype", [(200, "float32"), (201, "float32"), (203, "float32"), (207, "float32"), (212, "float32"), (213, "float32"),
                                        (207, "bfloat16"), (209, "bfloat16"), (214, "bfloat16")])
def test_random_configurations(seed, dtype, tmp_path):
    """Layer orders, sizes and constants drawn at random (one head, chunks of 1, one tap, values wider than keys, widths
    that no vector path takes ...): a prompt in portions with a decoded tail beside a second request, against the plain
    implementation. In bfloat16 only configurations whose embedding factor keeps the residual stream large against one
    layer's rounding: with a factor of 1 such a random model amplifies a rounding of 2^-9 to 1.6 % of the logits whichever
    kernels compute it (the CUDA-core products and the general attention give the same figure), above the stated tolerance."""
    import random
    from vafozen_util import random_config
    from nanoinfer_b200.engine import StepEntry
    rng = random.Random(seed)
    cfg = random_config(rng)
    d = write_model(str(tmp_path), cfg, seed, strip_rank=seed % 2 == 0)
    n = 70
    ids, other = tokens(n, cfg["vocab"], seed), tokens(33, cfg["vocab"], seed + 1)
    ref, ref2 = plain_logits(d, ids), plain_logits(d, other)
    eng = gpu_engine(d, dtype, page=rng.choice([4, 16]), pages=64, slots=2)
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    a, b = eng.open("a"), eng.open("b")
    got, got2, pos, pos2 = [], [], 0, 0
    for c in [17, 2, 1, 30, 3, 11] + [1] * 6:
        entries = [StepEntry(a, ids[pos:pos + c], list(range(c)))]
        m = min(len(other) - pos2, max(1, c // 2))
        if m > 0:
            entries.insert(0, StepEntry(b, other[pos2:pos2 + m], list(range(m))))
        lg = eng.step(entries).clone()
        if m > 0:
            got2.append(lg[:m]); lg = lg[m:]; pos2 += m
        got.append(lg); pos += c
    assert pos == n
    assert_close(torch.cat(got), ref, td, "first request")
    assert_close(torch.cat(got2), ref2[:pos2], td, "second request")
    eng.check_device()
    eng.cache.check()


def test_trace_replay_as_a_child_process(folders, tmp_path):
    """``bin/trace_run`` as a child process on a model of this design."""
    import json, os, subprocess, sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    ids = tokens(20, 77, 9)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": ids[:11], "want": [10]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": ids[11:], "want": [0, 8]}], "end": ["a"]}]
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folders["B"], "--dtype", "float32",
                        "--out", str(tmp_path), "--max-tokens", "64"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [line for line in r.stdout.splitlines() if line.startswith("done")] == ["done 0", "done 1"]
    ref = plain_logits(folders["B"], ids)
    import numpy as np
    got0 = torch.from_numpy(np.fromfile(os.path.join(tmp_path, "0.f32"), dtype="<f4").reshape(1, -1))
    got1 = torch.from_numpy(np.fromfile(os.path.join(tmp_path, "1.f32"), dtype="<f4").reshape(2, -1))
    assert_close(got0, ref[[10]], torch.float32, "step 0")
    assert_close(got1, ref[[11, 19]], torch.float32, "step 1")


def test_command_line_tools_generate_and_serve(folders):
    """bin/generate (with the cache and recomputing every token) and bin/serve as child processes, in 32-bit: the plain
    implementation's greedy tokens."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

    def tool(name, argv):
        done = subprocess.run([sys.executable, os.path.join(root, "bin", name)] + argv, capture_output=True, text=True, timeout=600)
        assert done.returncode == 0, done.stderr[-2000:]
        return [[int(t) for t in line.split("Completion: ", 1)[1].split()] for line in done.stdout.splitlines()
                if line.startswith("Completion: ")]

    def greedy(prompt, n):
        ids = list(prompt)
        for _ in range(n):
            ids.append(int(plain_logits(folders["B"], ids)[-1].argmax()))
        return ids[len(prompt):]

    prompts = [tokens(9, 77, 41), tokens(26, 77, 42)]
    common = ["--model-dir", folders["B"], "--dtype", "float32", "--block-size", "8", "--num-blocks", "32", "--max-tokens", "6"]
    for extra in ([], ["--no-cache"]):
        (got,) = tool("generate", common + ["--prompt", " ".join(map(str, prompts[0]))] + extra)
        assert got == greedy(prompts[0], 6), extra
    argv = common + ["--max-batch", "2", "--max-tokens-per-step", "16"]
    for p in prompts:
        argv += ["--prompt", " ".join(map(str, p))]
    got = tool("serve", argv)
    assert got == [greedy(p, 6) for p in prompts]
