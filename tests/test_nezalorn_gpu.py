"""Nezalorn on the GPU: every new kernel alone against its plain statement (tests/torch_ops.py, float64), with inputs
made so that a window that is one token off, a lost state or a wrong page shows; then the engine in both precisions
against the plain whole-sequence implementation: prompts, token-by-token decoding, portions down to two tokens,
unequal requests in one batch, slots and pages that are used again, long decoding through captured graphs, greedy
generation through the scheduler."""
from types import SimpleNamespace

import pytest
import torch

from gpu_util import assert_close
from nezalorn_util import CFG_A, CFG_B, DECAY_RANK, config_with_rank, delta, latent, lru, plain_logits, tokens, with_mlp, write_model
from torch_ops import TorchOps

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
@pytest.mark.parametrize("rows,width", [(1, 8), (5, 333), (3, 4096)])
def test_poly_norm(ops, dtype, rows, width):
    wide = rnd(rows, width + 5, seed=1, scale=1.7)
    z = wide[:, 2:2 + width]                                       # rows lie apart
    coef = torch.tensor([0.7, -0.4, 0.25, 0.1], device=DEV)
    out = torch.empty(rows, width, dtype=dtype, device=DEV)
    ops.poly_norm(z, coef, 1e-5, out)
    ref = torch.empty(rows, width, dtype=torch.float64)
    TorchOps().poly_norm(z.cpu(), coef.cpu(), 1e-5, ref)
    assert_close(out, ref, dtype, "poly_norm")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,width", [(1, 64), (9, 1000), (5, 4096), (3, 90)])
def test_two_norms_of_one_row(ops, dtype, rows, width):
    x, ga, gb = rnd(rows, width, seed=1, scale=3.0), rnd(width, seed=2), rnd(width, seed=3)
    a, b = torch.empty(rows, width, dtype=dtype, device=DEV), torch.empty(rows, width, dtype=dtype, device=DEV)
    ops.rmsnorm_pair(x, ga, gb, 1e-5, a, b)
    base = x.double() / torch.sqrt(x.double().pow(2).mean(-1, keepdim=True) + 1e-5)
    assert_close(a, base * ga.double(), dtype, "first norm")
    assert_close(b, base * gb.double(), dtype, "second norm")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,width", [(1, 64), (9, 1000), (3, 4096), (5, 90), (40, 64), (33, 2048), (70, 3000)])
def test_depth_mix_and_two_norms_in_one_pass(ops, dtype, rows, width):
    hist, x = rnd(4, rows, width, seed=2), rnd(rows, width, seed=3)
    coef, ga, gb = torch.tensor([0.5, -0.25, 1.5], device=DEV), rnd(width, seed=4), rnd(width, seed=5)
    h_ref, x_ref = hist.cpu().clone(), x.cpu().clone()
    a_ref, b_ref = torch.empty(rows, width, dtype=torch.float64), torch.empty(rows, width, dtype=torch.float64)
    TorchOps().depth_mix_norm_pair(h_ref, x_ref, coef.cpu(), 3, ga.cpu(), gb.cpu(), 1e-5, a_ref, b_ref)
    a, b = torch.empty(rows, width, dtype=dtype, device=DEV), torch.empty(rows, width, dtype=dtype, device=DEV)
    ops.depth_mix_norm_pair(hist, x, coef, 3, ga, gb, 1e-5, a, b)
    assert_close(x, x_ref, torch.float32, "weighted sum")
    assert_close(hist, h_ref, torch.float32, "streams")
    assert_close(a, a_ref, dtype, "first norm")
    assert_close(b, b_ref, dtype, "second norm")


@pytest.mark.parametrize("shape", [(7, 33), (16, 64)])
def test_depth_mix_other_shapes(ops, shape):
    hist, x = rnd(3, *shape, seed=2), rnd(*shape, seed=3)
    coef = torch.tensor([0.5, -0.25, 1.5], device=DEV)
    h_ref, x_ref = hist.cpu().clone(), x.cpu().clone()
    TorchOps().depth_mix(h_ref, x_ref, coef.cpu(), 3)
    ops.depth_mix(hist, x, coef, 3)
    assert_close(x, x_ref, torch.float32, "depth_mix")
    assert_close(hist, h_ref, torch.float32, "depth_mix history")


def test_depth_mix_keeps_streams_and_sums_them(ops):
    hist = rnd(5, 7, 33, seed=2)
    x = rnd(7, 33, seed=3)
    coef = torch.tensor([0.5, -0.25, 1.5, 0.125], device=DEV)
    h_ref, x_ref = hist.cpu().clone(), x.cpu().clone()
    TorchOps().depth_mix(h_ref, x_ref, coef.cpu(), 4)
    before = x.clone()
    ops.depth_mix(hist, x, coef, 4)
    assert torch.equal(hist[3], before) and torch.equal(hist[4].cpu(), h_ref[4])
    assert_close(x, x_ref, torch.float32, "depth_mix")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_unary_and_head_norm_gate(ops, dtype):
    wide = rnd(9, 50, seed=4, scale=2.0)
    out = torch.empty(9, 12, dtype=dtype, device=DEV)
    ops.unary(wide[:, 30:42], out, "tanh")
    assert_close(out, torch.tanh(wide[:, 30:42].double()), dtype, "tanh")
    heads, d = 3, 10
    o, gate, gain = rnd(6, heads * d, seed=5, scale=3.0), rnd(6, 2 * heads * d, seed=6)[:, heads * d:], rnd(heads * d, seed=7)
    got = torch.empty(6, heads * d, dtype=dtype, device=DEV)
    ops.head_norm_gate(o, gate, gain, 1e-4, heads, d, got)
    ref = torch.empty(6, heads * d, dtype=torch.float64)
    TorchOps().head_norm_gate(o.cpu(), gate.cpu(), gain.cpu(), 1e-4, heads, d, ref)
    assert_close(got, ref, dtype, "head_norm_gate")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("blocks,m,n,k", [(1, 1, 8, 8), (3, 5, 32, 16), (4, 16, 256, 128), (2, 40, 64, 32), (4, 300, 128, 64)])
def test_block_diagonal_product(ops, dtype, blocks, m, n, k):
    a, w, bias = rnd(blocks, m, k, seed=1).to(dtype), rnd(blocks, n, k, seed=2, scale=k ** -0.5).to(dtype), rnd(blocks, n, seed=3)
    out = torch.empty(blocks, m, n, device=DEV)
    ops.block_diag_linear(a, w, bias, out)
    ref = torch.empty(blocks, m, n)
    TorchOps().block_diag_linear(a.cpu(), w.cpu(), bias.cpu(), ref)
    assert_close(out, ref, torch.float32, "block-diagonal product")
    # with the activations also given as floats, token-major (many tokens then take one launch on the tensor cores)
    a32 = a.float().transpose(0, 1).reshape(m, blocks * k).contiguous()
    out2 = torch.empty(blocks, m, n, device=DEV)
    ops.block_diag_linear(a, w, bias, out2, a32=a32)
    assert_close(out2, ref, torch.float32, "block-diagonal product from floats")


# ------------------------------------------------------------------------------------------ generalized delta rule
def _delta_inputs(m, heads, d, seed):
    wide = rnd(m, 4 * heads * d + 3, seed=seed)
    n = heads * d
    r, k, v, a = (wide[:, i * n:(i + 1) * n] for i in range(4))
    return r, k, v, a, rnd(m, n, seed=seed + 1, scale=2.0)


@pytest.mark.parametrize("heads,d", [(1, 8), (2, 24), (3, 40), (1, 64), (2, 80), (1, 128)])
def test_delta_rule_scan_against_plain_and_cut_anywhere(ops, heads, d):
    q_lens = [1, 19, 2, 37]
    slots = [4, 0, 2, 1]
    ctx, _, _ = batch(q_lens, [0] * 4, slots=slots)
    m = sum(q_lens)
    r, k, v, a, w = _delta_inputs(m, heads, d, 10 + d)
    state = rnd(6, heads, d, d, seed=3, scale=0.3)
    untouched = state[3].clone()
    ref_state, ref_o = state.cpu().clone(), torch.zeros(m, heads * d)
    TorchOps().delta_rule_scan(r.cpu(), k.cpu(), v.cpu(), a.cpu(), w.cpu(), ref_state, to_cpu(ctx), ref_o, heads, d)
    whole_state, o = state.clone(), torch.empty(m, heads * d, device=DEV)
    ops.delta_rule_scan(r, k, v, a, w, whole_state, ctx, o, heads, d)
    assert_close(o, ref_o, torch.float32, "delta o")
    assert_close(whole_state, ref_state, torch.float32, "delta state")
    assert torch.equal(whole_state[3], untouched) and torch.equal(whole_state[5], state[5])
    # the same tokens in two steps, cut inside every request that has two tokens or more: bit-equal results
    first = [1, 7, 1, 16]
    rows_a = torch.cat([torch.arange(s, s + f) for s, f in zip(ctx.q_start.tolist(), first)]).to(DEV)
    rows_b = torch.cat([torch.arange(s + f, s + q) for s, f, q in zip(ctx.q_start.tolist(), first, q_lens)]).to(DEV)
    cut_state, o_cut = state.clone(), torch.empty(m, heads * d, device=DEV)
    for rows, lens, sl in ((rows_a, first, slots), (rows_b, [q - f for q, f in zip(q_lens, first) if q > f], [s for s, q, f in zip(slots, q_lens, first) if q > f])):
        c2, _, _ = batch(lens, [0] * len(lens), slots=sl)
        part = [x[rows].contiguous() for x in (r, k, v, a)]
        packed = torch.cat(part, dim=1)
        n = heads * d
        o2 = torch.empty(len(rows), n, device=DEV)
        ops.delta_rule_scan(packed[:, :n], packed[:, n:2 * n], packed[:, 2 * n:3 * n], packed[:, 3 * n:], w[rows].contiguous(), cut_state, c2, o2, heads, d)
        o_cut[rows] = o2
    assert torch.equal(o_cut, o) and torch.equal(cut_state, whole_state)


def test_delta_rule_remembers_a_far_key(ops):
    """One early token writes a value under a key that nothing else touches; decays near one keep it for hundreds of
    tokens, and the query of the last token reads it back."""
    heads, d, m = 1, 16, 400
    k = torch.zeros(m, d, device=DEV); v = torch.zeros(m, d, device=DEV); r = torch.zeros(m, d, device=DEV)
    k[:, 1] = 1.0                                # everyone writes under channel 1 ...
    v[:, 2] = 0.5
    k[5] = 0; k[5, 0] = 2.0                      # ... but token 5 under channel 0
    v[5] = 0; v[5, 3] = 7.0
    r[m - 1, 0] = 1.0
    packed = torch.cat([r, k, v, torch.full((m, d), -30.0, device=DEV)], 1)     # removal rate ~ 0
    w_logit = torch.full((m, d), -30.0, device=DEV)                             # decay ~ 1
    ctx, _, _ = batch([m], [0])
    state, o = torch.zeros(1, heads, d, d, device=DEV), torch.empty(m, d, device=DEV)
    ops.delta_rule_scan(packed[:, :d], packed[:, d:2 * d], packed[:, 2 * d:3 * d], packed[:, 3 * d:], w_logit, state, ctx, o, heads, d)
    assert abs(o[m - 1, 3].item() - 14.0) < 1e-3 and abs(o[m - 1, 2].item()) < 1e-3


# ------------------------------------------------------------------------------------------ convolution and recurrence
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width,taps,blocks", [(12, 1, 1), (48, 2, 3), (64, 4, 2), (40, 5, 1), (160, 4, 5)])
def test_conv_and_recurrence_in_steps(ops, dtype, width, taps, blocks):
    """Three steps: requests start, go on with one or two tokens (fewer than the convolution looks back), and one slot
    is taken over by a new request. Against the plain statement, state included."""
    bw = width // blocks
    cw, cb, sp = rnd(width, taps, seed=1, scale=0.6), rnd(width, seed=2, scale=0.1), torch.nn.functional.softplus(rnd(width, seed=3))
    state = torch.zeros(5, taps, width, device=DEV)
    ref_state = state.cpu().clone()
    steps = [([9, 1, 3], [2, 0, 4]), ([1, 2, 6], [2, 0, 4]), ([2, 5], [4, 1])]
    for i, (q_lens, slots) in enumerate(steps):
        if i == 2:
            state[1].zero_(); ref_state[1].zero_()
        ctx, _, _ = batch(q_lens, [0] * len(q_lens), slots=slots)
        m = sum(q_lens)
        xy = rnd(m, 2 * width + 1, seed=20 + i)
        x, y = xy[:, :width], xy[:, width:2 * width]
        gates = rnd(blocks, m, 2 * bw, seed=30 + i, scale=1.5)
        u32, ub = torch.empty(m, width, device=DEV), torch.empty(blocks, m, bw, dtype=dtype, device=DEV)
        ops.causal_conv(x, cw, cb, state, 1, ctx, u32, ub, taps, blocks)
        out = torch.empty(m, width, dtype=dtype, device=DEV)
        ops.rglru_scan(u32, gates, y, x, sp, state, ctx, out, taps, blocks)
        ru32, rub, rout = torch.empty(m, width), torch.empty(blocks, m, bw, dtype=torch.float64), torch.empty(m, width, dtype=torch.float64)
        t = TorchOps()
        t.causal_conv(x.cpu(), cw.cpu(), cb.cpu(), ref_state, 1, to_cpu(ctx), ru32, rub, taps, blocks)
        t.rglru_scan(ru32, gates.cpu(), y.cpu(), x.cpu(), sp.cpu(), ref_state, to_cpu(ctx), rout, taps, blocks)
        assert_close(u32, ru32, torch.float32, f"conv step {i}")
        assert_close(ub, rub, dtype, f"conv blocks step {i}")
        assert_close(out, rout, dtype, f"recurrence step {i}")
        assert_close(state, ref_state, torch.float32, f"state step {i}")


def test_a_slow_decay_keeps_its_accuracy_over_thousands_of_tokens(ops):
    """Decays within a thousandth of one, 3,000 tokens: the state must stay within 2e-6 of a 64-bit recurrence. (With the
    decay from a 32-bit exponential, which may be two units in the last place off, it drifts to about 9e-6.)"""
    width, m = 64, 3000
    g = torch.Generator().manual_seed(0)
    gates = torch.empty(1, m, 2 * width)
    gates[..., :width] = -5.0 + 0.5 * torch.randn(m, width, generator=g)       # the recurrence gate near 0.007
    gates[..., width:] = 3.0
    sp = torch.full((width,), 0.02)                                             # log a near -1e-3
    u, y = torch.randn(m, width, generator=g), torch.randn(m, width, generator=g)
    ctx, _, _ = batch([m], [0])
    state, out = torch.zeros(1, 1, width, device=DEV), torch.empty(m, width, device=DEV)
    ops.rglru_scan(u.to(DEV), gates.to(DEV), y.to(DEV), u.to(DEV), sp.to(DEV), state, ctx, out, 1, 1)
    la = -8.0 * torch.sigmoid(gates[0, :, :width].double()) * sp.double()
    a, b = torch.exp(la), torch.sqrt(-torch.expm1(2 * la)) * torch.sigmoid(gates[0, :, width:].double()) * u.double()
    ref = torch.zeros(width, dtype=torch.float64)
    for t in range(m):
        ref = a[t] * ref + b[t]
    err = ((state[0, 0].double().cpu() - ref).abs().max() / ref.abs().max()).item()
    assert err < 2e-6, err


# ------------------------------------------------------------------------------------------ attention through a latent
def _freq(rot):
    from nanoinfer_b200.parts.position import scaled_frequencies
    f, mag = scaled_frequencies(rot, 3000.0, {"factor": 2.5, "original": 32, "fast": 8.0, "slow": 1.0})
    return f.to(torch.float32).to(DEV), mag


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rank,rot,page", [(20, 4, 4), (64, 16, 16), (40, 0, 8), (96, 32, 16)])
def test_latent_store_and_query(ops, dtype, rank, rot, page):
    q_lens, before = [5, 1, 11], [3, 40, 0]
    ctx, bt, num_pages = batch(q_lens, before, page_size=page)
    m = sum(q_lens)
    freq, mag = _freq(rot) if rot else (torch.zeros(0, device=DEV), 1.0)
    z, gain = rnd(m, rank + rot + 2, seed=1)[:, :rank + rot], rnd(rank, seed=2)
    pages = torch.zeros(num_pages, 1, page, rank + rot, dtype=dtype, device=DEV)
    ops.latent_store(z, gain, 1e-5, freq, mag, ctx, bt, page, pages, rank, rot)
    ref = torch.zeros(num_pages, 1, page, rank + rot, dtype=torch.float64)
    TorchOps().latent_store(z.cpu(), gain.cpu(), 1e-5, freq.cpu(), mag, to_cpu(ctx), bt.cpu(), page, ref, rank, rot)
    assert_close(pages, ref, dtype, "latent rows")
    heads, dn = 3, 12
    q = rnd(m, heads * (dn + rot), seed=3)
    w_uk = rnd(heads * dn, rank, seed=4).to(dtype)
    qa = torch.empty(m, heads * (rank + rot), device=DEV)
    ops.latent_query(q, w_uk, freq, mag, ctx.positions, qa, heads, dn, rank, rot)
    qref = torch.empty(m, heads * (rank + rot))
    TorchOps().latent_query(q.cpu(), w_uk.cpu(), freq.cpu(), mag, ctx.positions.cpu(), qref, heads, dn, rank, rot)
    assert_close(qa, qref, torch.float32, "queries in the latent space")
    lat, w_uv = rnd(m, heads * rank, seed=5), rnd(heads * 7, rank, seed=6).to(dtype)
    out = torch.empty(m, heads * 7, dtype=dtype, device=DEV)
    ops.latent_value(lat, w_uv, out, heads, 7, rank)
    oref = torch.empty(m, heads * 7, dtype=torch.float64)
    TorchOps().latent_value(lat.cpu(), w_uv.cpu(), oref, heads, 7, rank)
    assert_close(out, oref, dtype, "values out of the latent space")


def _query_rows(ops, values, dtype, heads, rank, rot):
    """``values`` [m, heads, rank + rot] floats in the layout the attention kernel reads for a cache of ``dtype``;
    returns (the rows for the kernel, the values it will see as floats)."""
    m = values.shape[0]
    qw, qdt = ops.latent_query_layout(dtype, rank, rot)
    qa = torch.zeros(m, heads, qw, dtype=qdt, device=DEV)
    qa[:, :, :rank + rot] = values.to(qdt)
    return qa.view(m, heads * qw), qa[:, :, :rank + rot].float().reshape(m, -1)


@pytest.mark.parametrize("m", [1, 8, 70, 300])
@pytest.mark.parametrize("heads,dn,rank,rot,dv", [(3, 8, 24, 8, 12), (16, 64, 128, 32, 64), (5, 48, 64, 16, 40), (2, 128, 192, 0, 128), (4, 20, 40, 8, 6)])
def test_per_head_products_on_the_tensor_cores(ops, m, heads, dn, rank, rot, dv):
    """The tensor-core forms of the two maps between a head's space and the latent space (bfloat16 weights, rows for the
    tensor-core attention), from one token to hundreds; against the plain statements."""
    freq, mag = _freq(rot) if rot else (torch.zeros(0, device=DEV), 1.0)
    positions = torch.arange(5, 5 + m, dtype=torch.int32, device=DEV)
    q = rnd(m, heads * (dn + rot) + 3, seed=3)[:, :heads * (dn + rot)]
    w_uk = rnd(heads * dn, rank, seed=4, scale=dn ** -0.5).to(torch.bfloat16)
    qw, qdt = ops.latent_query_layout(torch.bfloat16, rank, rot)
    qa = torch.full((m, heads * qw), 7.0, dtype=qdt, device=DEV)
    ops.latent_query(q, w_uk, freq, mag, positions, qa, heads, dn, rank, rot)
    qref = torch.empty(m, heads * (rank + rot))
    TorchOps().latent_query(q.cpu(), w_uk.cpu(), freq.cpu(), mag, positions.cpu(), qref, heads, dn, rank, rot)
    got = qa.view(m, heads, qw)
    assert_close(got[:, :, :rank + rot].reshape(m, -1), qref, torch.bfloat16, "queries in the latent space")
    assert (got[:, :, rank + rot:] == 0).all()
    lat, w_uv = rnd(m, heads * rank, seed=5), rnd(heads * dv, rank, seed=6, scale=rank ** -0.5).to(torch.bfloat16)
    wide = torch.empty(m, heads * dv + 8, dtype=torch.bfloat16, device=DEV)
    out = wide[:, :heads * dv]
    ops.latent_value(lat, w_uv, out, heads, dv, rank)
    oref = torch.empty(m, heads * dv, dtype=torch.float64)
    TorchOps().latent_value(lat.cpu(), w_uv.cpu(), oref, heads, dv, rank)
    assert_close(out, oref, torch.bfloat16, "values out of the latent space")


@pytest.mark.parametrize("dtype,general", [(torch.float32, False), (torch.bfloat16, False), (torch.bfloat16, True)])
@pytest.mark.parametrize("window,page", [(0, 4), (5, 4), (32, 16), (33, 8), (64, 16), (200, 16)])
@pytest.mark.parametrize("heads,rank,rot", [(3, 24, 8), (16, 64, 16), (20, 128, 32)])
def test_latent_attention_over_pages_and_windows(ops, dtype, general, window, page, heads, rank, rot):
    """First tokens, a prompt, decoding far into a sequence, a portion that starts inside a page, a token on a page's
    edge: one-token requests lead the batch (they take the decode kernel), with contexts long enough for split keys."""
    k = ops.with_options(force_general_attention=True) if general else ops
    q_lens, before = [1, 1, 1, 70, 9], [0, 331, 63, 0, 60]
    ctx, bt, num_pages = batch(q_lens, before, page_size=page)
    m = sum(q_lens)
    pages = rnd(num_pages, 1, page, rank + rot, seed=1).to(dtype)
    qa, seen = _query_rows(k, rnd(m, heads, rank + rot, seed=2), dtype, heads, rank, rot)
    lat = torch.empty(m, heads * rank, device=DEV)
    k.latent_attention(qa, lat, ctx, bt, page, pages, heads, rank, rot, 0.3, window)
    ref = torch.empty(m, heads * rank)
    TorchOps().latent_attention(seen.cpu(), ref, to_cpu(ctx), bt.cpu(), page, pages.cpu(), heads, rank, rot, 0.3, window)
    # the tensor-core kernels round the softmax weights to bfloat16 before they meet the values
    assert_close(lat, ref, torch.float32 if (dtype == torch.float32 or general) else torch.bfloat16, "latent attention")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("decode", [False, True])
@pytest.mark.parametrize("window,page", [(6, 4), (32, 8), (40, 16), (64, 16), (129, 16)])
def test_a_key_at_the_windows_edge_is_seen_and_the_one_before_is_not(ops, window, page, decode, dtype):
    """All cached rows are small but one, which matches the query and carries a mark in its latent. A query whose
    window just reaches the row returns the mark; one position later it is gone. In a prompt's portion and decoded,
    on the general kernel (32-bit rows) and on the tensor-core kernels (bfloat16 rows)."""
    heads, rank, rot = 2, 16, 8
    edge = 37                                     # the marked row's position
    last = edge + window                          # sees edge+1 .. edge+window
    if decode:
        q_lens, before = [1, 1], [edge + window - 1, last]
    else:
        q_lens, before = [window + 3], [edge - 1]
    ctx, bt, num_pages = batch(q_lens, before, page_size=page, seed=3)
    pages = rnd(num_pages, 1, page, rank + rot, seed=1, scale=0.01).to(dtype)
    for r in range(len(q_lens)):
        pg = bt[r, edge // page].item()
        pages[pg, 0, edge % page, :] = 0
        pages[pg, 0, edge % page, 0] = 5.0        # matches the query below
        pages[pg, 0, edge % page, 1] = 9.0        # the mark
    values = torch.zeros(sum(q_lens), heads, rank + rot, device=DEV)
    values[:, :, 0] = 4.0
    qa, _ = _query_rows(ops, values, dtype, heads, rank, rot)
    lat = torch.empty(sum(q_lens), heads * rank, device=DEV)
    ops.latent_attention(qa, lat, ctx, bt, page, pages, heads, rank, rot, 1.0, window)
    pos = ctx.positions.tolist()
    mark = lat.view(-1, heads, rank)[:, :, 1]
    for row, p in enumerate(pos):
        if edge <= p < edge + window:
            assert (mark[row] > 8.9).all(), (p, mark[row])
        else:
            assert (mark[row].abs() < 0.1).all(), (p, mark[row])
    assert any(p == edge + window - 1 for p in pos) and any(p == edge + window for p in pos)


# ------------------------------------------------------------------------------------------ the engine
# Sizes near a real layer's ratios: the matrix products take the tensor-core kernels, the prompt spans pages and windows.
CFG_C = {"architecture": "Nezalorn", "vocab": 509, "width": 256, "norm": {"eps": 1e-5}, "layers": [
    with_mlp(delta(2, 64), 512),
    with_mlp(latent(4, 32, 16, 32, 96, 64, 40), 384),
    with_mlp(lru(256, 4, 4), 512),
    with_mlp(latent(4, 32, 16, 32, 96, 64, 24, kv_from=1), 512),
]}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {"A": write_model(str(tmp_path_factory.mktemp("nez_a")), config_with_rank(CFG_A, DECAY_RANK["A"]), 11, strip_rank=True),
            "B": write_model(str(tmp_path_factory.mktemp("nez_b")), config_with_rank(CFG_B, DECAY_RANK["B"]), 12),
            "C": write_model(str(tmp_path_factory.mktemp("nez_c")), config_with_rank(CFG_C, 32), 13)}


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


def test_long_decoding_through_captured_graphs_passes_windows_and_pages(folders):
    """150 tokens one by one (two requests side by side, so the steps are replayed from a captured graph): the windows
    of 7 and 11 pass over decoded tokens many times, pages behind them go back to the pool, the states carry on."""
    from nanoinfer_b200.engine import StepEntry
    eng = gpu_engine(folders["A"], "float32", page=4, pages=16, slots=2)
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


def test_prompt_portions_replayed_from_a_captured_graph(folders):
    """Portions of one recurring shape are captured the third time the shape is seen and replayed from then on: states,
    latents and the depth average's streams must go on through captured steps as through eager ones."""
    from nanoinfer_b200.engine import StepEntry
    eng = gpu_engine(folders["A"], "float32", page=4, pages=64, slots=2)
    assert eng._portion_graphs is not None
    eng._portion_graphs.min_tokens = 8
    ids = tokens(96, 131, 77)
    rc = eng.open("p")
    got = [eng.step([StepEntry(rc, ids[i:i + 8], list(range(8)))]).clone() for i in range(0, 96, 8)]
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


@pytest.mark.parametrize("seed", [100, 101, 103, 107, 112])
def test_random_configurations_in_32_bit(seed, tmp_path):
    """Layer orders, sizes and constants drawn at random (heads of 17, latents of 200, windows of 1, one tap, widths that
    no vector path takes ...): a prompt in portions with a decoded tail beside a second request, against the plain
    implementation."""
    import random
    from nezalorn_util import random_config
    from nanoinfer_b200.engine import StepEntry
    rng = random.Random(seed)
    cfg = random_config(rng)
    d = write_model(str(tmp_path), cfg, seed, strip_rank=seed % 2 == 0)
    n = 70
    ids, other = tokens(n, cfg["vocab"], seed), tokens(33, cfg["vocab"], seed + 1)
    ref, ref2 = plain_logits(d, ids), plain_logits(d, other)
    eng = gpu_engine(d, "float32", page=rng.choice([4, 16]), pages=64, slots=2)
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
    assert_close(torch.cat(got), ref, torch.float32, "first request")
    assert_close(torch.cat(got2), ref2[:pos2], torch.float32, "second request")
    eng.check_device()
    eng.cache.check()


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
