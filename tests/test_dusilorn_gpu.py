"""Dusilorn on a GPU: what the design added to the kernels (a norm after and before sublayers in one pass, a router with
softmax scores, a correction and renormalized weights, experts without a gate whose weight stands on the output, identity
outputs, a shared expert's activation, a norm of q and k over the whole projection, blended values, a sink beside chunked
and windowed masks) each against a plain statement, then whole models through the engine in both precisions, the
scheduler and the command-line tools."""
import json
import math
import os
import random
from types import SimpleNamespace

import pytest
import torch

import plain_dusilorn as plain
from dusilorn_util import (CFG_A, CFG_B, CFG_C, CFG_D, assert_within_rounding, chunked, dense, mixed_schedule, model, moe, pin_routing, plain_logits,
                           random_config, tokens, windowed, write_model)
from gpu_util import assert_close
from torch_ops import TorchOps

pytestmark = pytest.mark.gpu
DEV = "cuda"
DTYPES = [torch.float32, torch.bfloat16]


@pytest.fixture(scope="module")
def ops():
    from nanoinfer_b200.csrc.lib import load_kernels
    return load_kernels()


def batch(q_lens, before, page_size=4, seed=0, num_pages=0, device=DEV):
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
    ctx = SimpleNamespace(
        num_tokens=sum(q_lens),
        positions=torch.cat([torch.arange(b, b + q, dtype=torch.int32) for b, q in zip(before, q_lens)]).to(device),
        req_index=torch.cat([torch.full((q,), i, dtype=torch.int32) for i, q in enumerate(q_lens)]).to(device),
        q_start=q_start.to(device), ctx_lens=torch.tensor(ctx_lens, dtype=torch.int32, device=device),
        host=SimpleNamespace(q_lens=list(q_lens), ctx_lens=ctx_lens, num_requests=r, max_q_len=max(q_lens), max_ctx_len=max(ctx_lens)))
    return ctx, bt.to(device), num_pages


def to_cpu(ctx):
    return SimpleNamespace(num_tokens=ctx.num_tokens, positions=ctx.positions.cpu(), req_index=ctx.req_index.cpu(),
                           q_start=ctx.q_start.cpu(), ctx_lens=ctx.ctx_lens.cpu(), host=ctx.host)


def rnd(*shape, seed=0, scale=1.0):
    return (torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale).to(DEV)


# ------------------------------------------------------------------------------------------ norms around a sublayer
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m,n", [(1, 8), (7, 100), (5, 256), (3, 1030), (70, 192)])
def test_the_norm_on_an_output_and_the_next_norm_in_one_pass(ops, dtype, m, n):
    y, x, gain, nxt = rnd(m, n, seed=1, scale=3.0), rnd(m, n, seed=2), rnd(n, seed=3), rnd(n, seed=4)
    new = x.double().cpu() + plain.unit_rms(y.double().cpu(), 1e-3) * gain.double().cpu()
    ref_h = plain.unit_rms(new, 1e-5) * nxt.double().cpu()
    h = torch.empty(m, n, dtype=dtype, device=DEV)
    ops.rmsnorm_add(y, gain, 1e-3, 1.0, x, h, True, next_gain32=nxt, next_eps=1e-5)
    assert_close(x, new, torch.float32, "stream")
    assert_close(h, ref_h, dtype, "the next sublayer's input")
    assert y.abs().max().item() == 0.0


# ------------------------------------------------------------------------------------------ the router
@pytest.mark.parametrize("m,outputs,top", [(1, 1, 1), (9, 7, 2), (40, 35, 4), (6, 3, 3), (130, 70, 1), (5, 18, 2)])
def test_router_softmax_scores_correction_for_the_choice_renormalized_weights(ops, m, outputs, top):
    z = rnd(m, outputs + 2, seed=5, scale=2.0)           # two more columns that are no router outputs
    corr = rnd(outputs, seed=6, scale=0.2)
    s = torch.softmax(z[:, :outputs].double().cpu(), -1)
    choice = s + corr.double().cpu()
    sel_e = torch.empty(m, top, dtype=torch.int32, device=DEV)
    sel_w = torch.empty(m, top, dtype=torch.float32, device=DEV)
    keep = z.clone()
    ops.moe_route(z[:, :outputs], top, sel_e, sel_w, score="softmax", renormalize=True, correction32=corr)
    want = torch.topk(choice, top, dim=-1).indices
    assert torch.equal(sel_e.cpu().long(), want)
    w = torch.gather(s, 1, want)
    assert_close(sel_w, w / (w.sum(-1, keepdim=True) + 1e-20), torch.float32, "weights")
    assert torch.equal(z[:, outputs:], keep[:, outputs:])
    # without renormalization the weights are the scores; with sigmoid scores and a correction the choice changes alone
    z2 = keep.clone()
    ops.moe_route(z2[:, :outputs], top, sel_e, sel_w, score="sigmoid", correction32=corr)
    sg = torch.sigmoid(keep[:, :outputs].double().cpu())
    want = torch.topk(sg + corr.double().cpu(), top, dim=-1).indices
    assert torch.equal(sel_e.cpu().long(), want)
    assert_close(sel_w, torch.gather(sg, 1, want), torch.float32, "sigmoid scores")


def test_router_takes_the_first_of_equal_choice_scores(ops):
    z = torch.zeros(3, 6, device=DEV)
    corr = torch.tensor([0.0, 0.5, 0.5, 0.0, 0.5, 0.0], device=DEV)
    sel_e = torch.empty(3, 2, dtype=torch.int32, device=DEV)
    sel_w = torch.empty(3, 2, dtype=torch.float32, device=DEV)
    ops.moe_route(z, 2, sel_e, sel_w, score="softmax", renormalize=True, correction32=corr)
    assert sel_e.cpu().tolist() == [[1, 2]] * 3 and torch.allclose(sel_w.cpu(), torch.full((3, 2), 0.5))


def expert_weights(experts, hidden, ff, dtype, outputs=None):
    w = {"r.router": rnd(outputs or experts, hidden, seed=2, scale=2.0 * hidden ** -0.5).to(dtype),
         "r.correction": rnd(outputs or experts, seed=4, scale=0.05).to(dtype)}
    for e in range(experts):
        w[f"r.e{e}.up"] = rnd(ff, hidden, seed=11 + 3 * e, scale=hidden ** -0.5).to(dtype)
        w[f"r.e{e}.down"] = rnd(hidden, ff, seed=12 + 3 * e, scale=ff ** -0.5).to(dtype)
    up = torch.stack([w[f"r.e{e}.up"] for e in range(experts)]).contiguous()
    down = torch.stack([w[f"r.e{e}.down"] for e in range(experts)]).contiguous()
    return w, up, down


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m,hidden,ff,experts,identity,top", [(1, 32, 8, 1, 0, 1), (9, 64, 24, 5, 2, 2), (300, 72, 40, 3, 1, 1), (150, 100, 130, 6, 0, 3),
                                                              (33, 128, 64, 4, 3, 4), (200, 256, 64, 16, 2, 2), (700, 256, 136, 5, 1, 2),
                                                              (513, 64, 16, 2, 2, 1), (8, 512, 320, 8, 0, 2), (1100, 192, 72, 3, 1, 3)])
def test_experts_without_a_gate_weighted_on_the_output_with_identity_outputs(ops, dtype, m, hidden, ff, experts, identity, top):
    """Against the plain loop over tokens and choices: relu squared, the renormalized weight on the expert's result, the
    router's last outputs passing the token's input through; the sum goes onto what the row already holds. Both product
    paths in bfloat16 (row tiles of 32 and of 128 on the tensor cores), one choice per token and several."""
    outputs = experts + identity
    h = rnd(m, hidden, seed=1).to(dtype)
    w, up, down = expert_weights(experts, hidden, ff, dtype, outputs)
    z = (h.double() @ w["r.router"].double().t()).float()
    corr = w["r.correction"].float()
    sel_e = torch.empty(m, top, dtype=torch.int32, device=DEV)
    sel_w = torch.empty(m, top, dtype=torch.float32, device=DEV)
    ops.moe_route(z, top, sel_e, sel_w, score="softmax", renormalize=True, correction32=corr)
    mlp = {"router": {"experts": experts, "identity": identity, "top": top}}
    wd = {k: v.double().cpu() for k, v in w.items()}
    chosen, _ = plain.route(mlp, wd, "r", h.double().cpu())
    assert sel_e.cpu().tolist() == chosen
    ref = plain.mixture(mlp, wd, "r", h.double().cpu())
    before = rnd(m, hidden, seed=3)
    for name, o in (("", ops),) + ((("CUDA cores", ops.with_options(force_simt_gemm=True)),) if dtype == torch.bfloat16 else ()):
        out = before.clone()
        o.moe_experts(h, sel_e, sel_w, up, down, out, gated=False, weight_on="output", outputs=outputs)
        if identity:
            o.moe_identity(h, out, sel_e, sel_w, experts)
        assert_close(out - before, ref, dtype, "mixture " + name)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m,hidden,ff,experts,identity,top", [(1, 32, 8, 1, 1, 1), (8, 256, 64, 8, 2, 2), (5, 72, 40, 30, 3, 4), (16, 128, 24, 12, 0, 1),
                                                              (3, 100, 130, 6, 1, 3), (64, 64, 16, 5, 2, 2)])
def test_a_short_step_with_the_router_options_in_one_launch(ops, dtype, m, hidden, ff, experts, identity, top):
    """Router logits (with one more row whose logit is a gate), scores, choice, grouping and gathered rows in one launch:
    the same choices and weights as the separate steps, no row tile for an identity output, and the mixture through its
    plan equals the plain loop."""
    outputs = experts + identity
    h = rnd(m, hidden, seed=1).to(dtype)
    w, up, down = expert_weights(experts, hidden, ff, dtype, outputs)
    sg = rnd(1, hidden, seed=7, scale=hidden ** -0.5).to(dtype)
    corr = w["r.correction"].float()
    sel_e = torch.full((m, top), -1, dtype=torch.int32, device=DEV)
    sel_w = torch.zeros(m, top, dtype=torch.float32, device=DEV)
    gate = torch.zeros(m, 1, device=DEV)
    plan = ops.moe_step(h, torch.cat([w["r.router"], sg]).contiguous(), top, up, down, sel_e, sel_w, score="softmax", renormalize=True,
                        correction32=corr, n_real=experts, extra=1, z_extra=gate)
    assert plan is not None, "a step of these sizes fits one block"
    mlp = {"router": {"experts": experts, "identity": identity, "top": top}}
    wd = {k: v.double().cpu() for k, v in w.items()}
    chosen, weights = plain.route(mlp, wd, "r", h.double().cpu())
    assert sel_e.cpu().tolist() == chosen
    assert_close(sel_w, torch.stack(weights), torch.float32, "weights")
    assert_close(gate, h.double().cpu() @ sg.double().cpu().t(), torch.float32, "the gate's logit")
    tiles = plan.tiles.cpu().view(-1, 3)[:int(plan.n_tiles.cpu())]
    assert (tiles[:, 0] < experts).all() and int(tiles[:, 2].sum()) == sum(e < experts for row in chosen for e in row)
    before = rnd(m, hidden, seed=3)
    out = before.clone()
    ops.moe_experts(h, sel_e, sel_w, up, down, out, plan=plan, gated=False, weight_on="output", outputs=outputs)
    ops.moe_identity(h, out, sel_e, sel_w, experts)
    assert_close(out - before, plain.mixture(mlp, wd, "r", h.double().cpu()), dtype, "mixture of a short step")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m,hidden,ff,shared,experts,identity,top", [(1, 32, 8, 8, 1, 0, 1), (9, 64, 24, 40, 5, 2, 2), (300, 72, 40, 8, 3, 1, 1),
                                                                     (33, 128, 64, 128, 4, 3, 4), (700, 256, 136, 200, 5, 0, 2), (8, 512, 320, 320, 8, 1, 2)])
def test_a_shared_expert_runs_as_pieces_that_every_token_uses(ops, dtype, m, hidden, ff, shared, experts, identity, top):
    """The shared expert cut into pieces of the experts' width (the last filled up with zero rows) in front of the stacked
    experts: the router's kernel gives every token those pieces with the weight sigmoid(gate logit) and moves the chosen
    outputs behind them; the whole mixture (chosen experts, identity outputs, shared expert times its gate) equals the
    plain loop, through the separate launches and through the one launch of a short step."""
    outputs = experts + identity
    h = rnd(m, hidden, seed=1).to(dtype)
    w, up, down = expert_weights(experts, hidden, ff, dtype, outputs)
    w["r.shared.up"] = rnd(shared, hidden, seed=8, scale=hidden ** -0.5).to(dtype)
    w["r.shared.down"] = rnd(hidden, shared, seed=9, scale=shared ** -0.5).to(dtype)
    w["r.shared.sg"] = rnd(1, hidden, seed=7, scale=2.0 * hidden ** -0.5).to(dtype)
    pieces = -(-shared // ff)
    s_up = torch.zeros(pieces * ff, hidden, dtype=dtype, device=DEV)
    s_up[:shared] = w["r.shared.up"]
    s_down = torch.zeros(hidden, pieces * ff, dtype=dtype, device=DEV)
    s_down[:, :shared] = w["r.shared.down"]
    up = torch.cat([s_up.view(pieces, ff, hidden), up]).contiguous()
    down = torch.cat([s_down.view(hidden, pieces, ff).permute(1, 0, 2), down]).contiguous()
    router = torch.cat([w["r.router"], w["r.shared.sg"]]).contiguous()
    corr = w["r.correction"].float()
    mlp = {"router": {"experts": experts, "identity": identity, "top": top}, "shared": {"ff": shared}}
    wd = {k: v.double().cpu() for k, v in w.items()}
    chosen, weights = plain.route(mlp, wd, "r", h.double().cpu())
    ref = plain.mixture(mlp, wd, "r", h.double().cpu())
    gate = torch.sigmoid(h.double().cpu() @ wd["r.shared.sg"].t())
    before = rnd(m, hidden, seed=3)
    for short in (False, True):
        sel_e = torch.full((m, top + pieces), -1, dtype=torch.int32, device=DEV)
        sel_w = torch.zeros(m, top + pieces, dtype=torch.float32, device=DEV)
        options = dict(score="softmax", renormalize=True, correction32=corr, always=pieces)
        plan = None
        if short:
            plan = ops.moe_step(h, router, top, up, down, sel_e, sel_w, n_real=experts + pieces, extra=1, **options)
            if plan is None:
                continue        # too large for one block
        else:
            z = (h.double() @ router.double().t()).float()
            ops.moe_route(z[:, :outputs], top, sel_e, sel_w, **options)
        assert (sel_e[:, :top].cpu() - pieces).tolist() == chosen and sel_e[:, top:].cpu().tolist() == [list(range(pieces))] * m
        assert_close(sel_w[:, :top], torch.stack(weights), torch.float32, "weights")
        assert_close(sel_w[:, top:], gate.expand(m, pieces), torch.float32, "the shared expert's gate")
        out = before.clone()
        ops.moe_experts(h, sel_e, sel_w, up, down, out, plan=plan, gated=False, weight_on="output", outputs=outputs + pieces)
        if identity:
            ops.moe_identity(h, out, sel_e, sel_w, experts + pieces)
        assert_close(out - before, ref, dtype, "mixture with a shared expert" + (" (short step)" if short else ""))


# ------------------------------------------------------------------------------------------ operands of the attention
def rows_of(pages, bt, req, positions, page):
    return torch.stack([pages[int(bt[req, p // page]), :, p % page, :] for p in positions])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("q_lens,before", [([4, 1], [0, 9]), ([280, 1, 3], [5, 700, 0])])
@pytest.mark.parametrize("heads,kv,dim,vdim,rot,page", [(4, 2, 12, 6, 8, 4), (6, 3, 80, 40, 48, 16), (16, 2, 64, 64, 32, 16), (2, 1, 128, 128, 128, 8),
                                                        (3, 3, 40, 8, 16, 4), (2, 2, 32, 16, 0, 16)])
def test_operands_rotated_in_half_split_pairs_and_values_blended(ops, dtype, heads, kv, dim, vdim, rot, page, q_lens, before):
    """The first ``rot`` elements of every q and k head turned by position (element i with i + rot/2), the rest unchanged,
    values blended; both kernels (a warp per head; eight elements a thread), read back from the pages."""
    ctx, bt, num_pages = batch(q_lens, before, page_size=page)
    m, nq, nk, nv = sum(q_lens), heads * dim, kv * dim, kv * vdim
    qkv = rnd(m, nq + nk + nv, seed=1, scale=1.5)
    first = rnd(m, nv, seed=2)
    lam = torch.tensor([0.8], device=DEV)
    freq = torch.tensor([10000.0 ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float64).float().to(DEV) if rot else None
    kp = torch.zeros(num_pages, kv, page, dim, dtype=dtype, device=DEV)
    vp = torch.zeros(num_pages, kv, page, vdim, dtype=dtype, device=DEV)
    q = torch.empty(m, nq, dtype=dtype, device=DEV)
    ops.attention_prepare(qkv, q, heads, kv, dim, vdim, None, None, 1e-6, freq, rot, ctx, bt, page, kp, vp, True, v_first32=first, vmix32=lam)
    x = qkv.double().cpu()
    row = 0
    for r, (n, b) in enumerate(zip(q_lens, before)):
        xq, xk = x[row:row + n, :nq].view(n, heads, dim), x[row:row + n, nq:nq + nk].view(n, kv, dim)
        if rot:     # the design forms the angle in 32-bit: position times frequency, rounded once
            ang = (torch.arange(b, b + n, dtype=torch.float32)[:, None] * freq.cpu()[None, :]).double()
            cs, sn = ang.cos()[:, None, :], ang.sin()[:, None, :]

            def turn(y):
                u, v = y[..., :rot // 2].clone(), y[..., rot // 2:rot].clone()
                y = y.clone()
                y[..., :rot // 2], y[..., rot // 2:rot] = u * cs - v * sn, v * cs + u * sn
                return y
            xq, xk = turn(xq), turn(xk)
        assert_close(q[row:row + n], xq.reshape(n, nq), dtype, "queries")
        assert_close(rows_of(kp, bt.cpu(), r, range(b, b + n), page).reshape(n, nk), xk.reshape(n, nk), dtype, "cached keys")
        ref_v = 0.2 * x[row:row + n, nq + nk:] + 0.8 * first.double().cpu()[row:row + n]
        assert_close(rows_of(vp, bt.cpu(), r, range(b, b + n), page).reshape(n, nv), ref_v, dtype, "cached values")
        row += n


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("q_lens,before", [([5, 1, 9], [3, 17, 0]), ([300, 2, 270], [0, 40, 33])])
@pytest.mark.parametrize("heads,kv,dim,vdim,page", [(4, 2, 12, 6, 4), (3, 1, 16, 10, 4), (8, 4, 64, 40, 16), (5, 5, 4, 2, 8), (2, 1, 136, 24, 16),
                                                    (16, 2, 128, 128, 16), (3, 3, 96, 8, 8)])
def test_operands_normed_over_the_whole_projection_and_values_blended(ops, dtype, heads, kv, dim, vdim, page, q_lens, before):
    """Steps of few tokens (a warp per head) and of hundreds (a block per token; in bfloat16 with widths in multiples of 8,
    eight elements a thread)."""
    ctx, bt, num_pages = batch(q_lens, before, page_size=page)
    m, nq, nk, nv = sum(q_lens), heads * dim, kv * dim, kv * vdim
    wide = rnd(m, nq + nk + nv + 3, seed=1, scale=1.5)   # rows that lie apart
    qkv = wide[:, :nq + nk + nv]
    first = rnd(m, nv + 5, seed=2)[:, :nv]
    qg, kg, lam = rnd(nq, seed=3), rnd(nk, seed=4), torch.tensor([0.3], device=DEV)
    kp = torch.zeros(num_pages, kv, page, dim, dtype=dtype, device=DEV)
    vp = torch.zeros(num_pages, kv, page, vdim, dtype=dtype, device=DEV)
    q = torch.empty(m, nq, dtype=dtype, device=DEV)
    ops.attention_prepare(qkv, q, heads, kv, dim, vdim, qg, kg, 1e-4, None, 0, ctx, bt, page, kp, vp, True, norm_whole=True, v_first32=first, vmix32=lam)
    x = qkv.double().cpu()
    ref_q = plain.unit_rms(x[:, :nq], 1e-4) * qg.double().cpu()
    ref_k = plain.unit_rms(x[:, nq:nq + nk], 1e-4) * kg.double().cpu()
    ref_v = 0.7 * x[:, nq + nk:] + 0.3 * first.double().cpu()
    assert_close(q, ref_q, dtype, "queries")
    row = 0
    for r, (n, b) in enumerate(zip(q_lens, before)):
        assert_close(rows_of(kp, bt.cpu(), r, range(b, b + n), page).reshape(n, nk), ref_k[row:row + n], dtype, "cached keys")
        assert_close(rows_of(vp, bt.cpu(), r, range(b, b + n), page).reshape(n, nv), ref_v[row:row + n], dtype, "cached values")
        row += n


def filled_pages(dtype, ctx_lens, bt, num_pages, kv, dim, vdim, page, seed):
    """Random keys and values at every position the requests hold."""
    kp = torch.zeros(num_pages, kv, page, dim, dtype=dtype, device=DEV)
    vp = torch.zeros(num_pages, kv, page, vdim, dtype=dtype, device=DEV)
    g = torch.Generator().manual_seed(seed)
    for r, n in enumerate(ctx_lens):
        for p in range(n):
            kp[int(bt[r, p // page]), :, p % page] = torch.randn(kv, dim, generator=g).to(dtype)
            vp[int(bt[r, p // page]), :, p % page] = torch.randn(kv, vdim, generator=g).to(dtype)
    return kp, vp


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv,dim,vdim,window,chunk,page,q_lens,before", [
    (4, 2, 12, 6, 0, 3, 4, [5, 1, 9], [3, 17, 0]), (8, 4, 64, 40, 0, 48, 16, [70, 1, 1], [130, 200, 47]), (6, 2, 80, 40, 130, 0, 16, [1, 1, 40], [300, 129, 120]),
    (3, 1, 16, 24, 0, 17, 8, [33, 2], [0, 40]), (2, 2, 128, 128, 0, 100, 16, [1, 1, 1, 1], [99, 100, 450, 0]), (6, 3, 40, 8, 9, 0, 4, [12, 1], [4, 30]),
    (8, 2, 64, 64, 0, 64, 16, [70, 1, 130], [130, 200, 63]), (4, 2, 128, 128, 130, 0, 16, [200, 3], [100, 0]), (16, 2, 64, 64, 100, 0, 64, [300], [17]),
    (4, 4, 128, 128, 0, 1000, 32, [129, 65], [0, 700])])
def test_attention_with_a_sink_beside_chunks_and_windows(ops, dtype, heads, kv, dim, vdim, window, chunk, page, q_lens, before):
    """The kernels (tensor cores for bfloat16, one token per request with keys split over CTAs included) against the plain
    statement: capped scores, chunked or windowed mask by absolute position, exp(sink) once in the denominator."""
    ctx, bt, num_pages = batch(q_lens, before, page_size=page)
    kp, vp = filled_pages(dtype, ctx.host.ctx_lens, bt.cpu(), num_pages, kv, dim, vdim, page, 3)
    m = sum(q_lens)
    q = rnd(m, heads * dim, seed=4).to(dtype)
    sinks = rnd(heads, seed=5, scale=2.0)
    out = torch.empty(m, heads * vdim, dtype=torch.float32, device=DEV)
    ops.attention_flex(q, out, heads, kv, dim, vdim, dim ** -0.5, 25.0, None, window, chunk, 1.0, ctx, bt, page, kp, vp, sinks32=sinks)
    ref = torch.empty(m, heads * vdim, dtype=torch.float64)
    TorchOps().attention_flex(q.cpu(), ref, heads, kv, dim, vdim, dim ** -0.5, 25.0, None, window, chunk, 1.0, to_cpu(ctx), bt.cpu(), page,
                              kp.cpu(), vp.cpu(), sinks32=sinks.cpu())
    assert_close(out, ref, dtype, "attention with a sink")
    if dtype == torch.bfloat16:
        # output in the storage type: prompt portions with heads of 64 or 128 take the kernel with scores in tensor memory
        out_b = torch.empty(m, heads * vdim, dtype=dtype, device=DEV)
        ops.attention_flex(q, out_b, heads, kv, dim, vdim, dim ** -0.5, 25.0, None, window, chunk, 1.0, ctx, bt, page, kp, vp, sinks32=sinks)
        assert_close(out_b, ref, dtype, "attention with a sink, output in the storage type")
        assert ops.gemm_tc_error() == 0 and ops.attention_tc_error() == 0
    no_sink = torch.empty_like(out)
    ops.attention_flex(q, no_sink, heads, kv, dim, vdim, dim ** -0.5, 25.0, None, window, chunk, 1.0, ctx, bt, page, kp, vp)
    assert (no_sink - out).abs().max().item() > 1e-3


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("decode", [False, True])
@pytest.mark.parametrize("kind,size,page", [("chunk", 1, 4), ("chunk", 2, 4), ("chunk", 6, 4), ("chunk", 33, 16), ("chunk", 64, 16), ("chunk", 100, 16),
                                            ("window", 1, 4), ("window", 5, 4), ("window", 64, 16), ("window", 130, 16), ("window", 257, 64)])
def test_keys_just_inside_and_just_outside_an_edge_with_a_sink(ops, kind, size, page, decode, dtype):
    """All keys are alike but one, whose score stands out and whose value carries a mark. A query sees it while it lies in
    the query's chunk (or window) and not one position later; the sink takes its share either way: with the marked key
    visible the mark's weight is e^9 / (e^9 + others + e^sink), without it zero."""
    dim, n = 16, 2 * size + 70
    a = (n // 2 // size) * size + size - 1 if kind == "chunk" else 37    # chunk: the last position of a block
    if kind == "chunk" and size > 1:
        a -= 1                                          # ... or the one before, so that one later position still sees it
    qkv = torch.zeros(n, 3 * dim, device=DEV)
    qkv[:, dim] = 1.0                                   # every key: e0
    qkv[a, dim + 1] = 9.0
    qkv[a, 2 * dim + 2] = 4.0                           # the marked key's value
    qkv[:, 1] = 1.0                                     # every query asks for e1
    ctx_all, bt, num_pages = batch([n], [0], page_size=page)
    kp = torch.zeros(num_pages, 1, page, dim, dtype=dtype, device=DEV)
    vp = torch.zeros(num_pages, 1, page, dim, dtype=dtype, device=DEV)
    q_all = torch.empty(n, dim, dtype=dtype, device=DEV)
    ops.attention_prepare(qkv, q_all, 1, 1, dim, dim, None, None, 1e-6, None, 0, ctx_all, bt, page, kp, vp, True)
    sink = torch.tensor([math.log(3.0)], device=DEV)
    last = (a // size) * size + size - 1 if kind == "chunk" else a + size - 1     # the last position that sees key a
    window, chunk = (0, size) if kind == "chunk" else (size, 0)
    for p in (last, last + 1):
        sees = p == last
        lo = max((p // size) * size, 0) if kind == "chunk" else max(0, p - size + 1)
        others = (p - lo + 1) - (1 if sees else 0)
        want = 4.0 * math.exp(9.0) / (math.exp(9.0) + others + 3.0) if sees else 0.0
        ctx, _, _ = (batch([1], [p], page_size=page) if decode or p == 0 else batch([2], [p - 1], page_size=page))
        rows = [p] if decode or p == 0 else [p - 1, p]
        out = torch.empty(len(rows), dim, device=DEV)
        ops.attention_flex(q_all[rows].contiguous(), out, 1, 1, dim, dim, 1.0, 0.0, None, window, chunk, 1.0, ctx, bt, page, kp, vp, sinks32=sink)
        assert abs(out[-1, 2].item() - want) < 3e-2, (p, sees, out[-1, :4].tolist(), want)


@pytest.mark.parametrize("kind,size,page", [("chunk", 64, 16), ("chunk", 100, 16), ("chunk", 128, 64), ("window", 64, 16), ("window", 130, 16), ("window", 257, 64)])
def test_prompt_portions_with_scores_in_tensor_memory_see_the_same_edges(ops, kind, size, page):
    """Heads of 64 in bfloat16, portions of 80 tokens that end just inside and just outside the edge: the marked key's
    weight beside the sink, as above, on the tcgen05 path (and the same from the mma.sync path when it is pinned)."""
    dim, n = 64, 2 * size + 150
    a = (n // 2 // size) * size + size - 2 if kind == "chunk" else 37
    qkv = torch.zeros(n, 3 * dim, device=DEV)
    qkv[:, dim] = 1.0
    qkv[a, dim + 1] = 9.0
    qkv[a, 2 * dim + 2] = 4.0
    qkv[:, 1] = 1.0
    ctx_all, bt, num_pages = batch([n], [0], page_size=page)
    kp = torch.zeros(num_pages, 1, page, dim, dtype=torch.bfloat16, device=DEV)
    vp = torch.zeros(num_pages, 1, page, dim, dtype=torch.bfloat16, device=DEV)
    q_all = torch.empty(n, dim, dtype=torch.bfloat16, device=DEV)
    ops.attention_prepare(qkv, q_all, 1, 1, dim, dim, None, None, 1e-6, None, 0, ctx_all, bt, page, kp, vp, True)
    sink = torch.tensor([math.log(3.0)], device=DEV)
    last = (a // size) * size + size - 1 if kind == "chunk" else a + size - 1
    window, chunk = (0, size) if kind == "chunk" else (size, 0)
    for o in (ops, ops.with_options(force_mma_prefill=True)):
        for p in (last, last + 1):
            sees = p == last
            lo = (p // size) * size if kind == "chunk" else max(0, p - size + 1)
            others = (p - lo + 1) - (1 if sees else 0)
            want = 4.0 * math.exp(9.0) / (math.exp(9.0) + others + 3.0) if sees else 0.0
            ctx, _, _ = batch([80], [p - 79], page_size=page)
            out = torch.empty(80, dim, dtype=torch.bfloat16, device=DEV)
            o.attention_flex(q_all[p - 79:p + 1].contiguous(), out, 1, 1, dim, dim, 1.0, 0.0, None, window, chunk, 1.0, ctx, bt, page, kp, vp, sinks32=sink)
            assert abs(out[-1, 2].item() - want) < 3e-2, (p, sees, out[-1, :4].float().tolist(), want)
    assert ops.attention_tc_error() == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("decode", [False, True])
@pytest.mark.parametrize("page,n,far", [(16, 700, 3), (16, 1500, 0), (4, 300, 1), (64, 2100, 64)])
def test_a_far_key_among_hundreds_is_found_and_the_sink_counts_once(ops, page, n, far, decode, dtype):
    """One key far back stands out among n alike (no mask reaches: a chunk as long as the sequence): its value's mark must
    come out with the weight the plain softmax gives it beside exp(sink), whatever the number of tiles and splits."""
    dim = 16
    qkv = torch.zeros(n, 3 * dim, device=DEV)
    qkv[:, dim] = 1.0
    qkv[far, dim + 1] = 12.0
    qkv[far, 2 * dim + 2] = 4.0
    qkv[:, 1] = 1.0
    ctx_all, bt, num_pages = batch([n], [0], page_size=page)
    kp = torch.zeros(num_pages, 1, page, dim, dtype=dtype, device=DEV)
    vp = torch.zeros(num_pages, 1, page, dim, dtype=dtype, device=DEV)
    q_all = torch.empty(n, dim, dtype=dtype, device=DEV)
    ops.attention_prepare(qkv, q_all, 1, 1, dim, dim, None, None, 1e-6, None, 0, ctx_all, bt, page, kp, vp, True)
    sink = torch.tensor([math.log(500.0)], device=DEV)
    ctx, _, _ = batch([1], [n - 1], page_size=page) if decode else batch([7], [n - 7], page_size=page)
    rows = [n - 1] if decode else list(range(n - 7, n))
    out = torch.empty(len(rows), dim, device=DEV)
    ops.attention_flex(q_all[rows].contiguous(), out, 1, 1, dim, dim, 1.0, 0.0, None, 0, 4096, 1.0, ctx, bt, page, kp, vp, sinks32=sink)
    want = 4.0 * math.exp(12.0) / (math.exp(12.0) + (n - 1) + 500.0)
    assert abs(out[-1, 2].item() - want) < 3e-2, (out[-1, :4].tolist(), want)


# ------------------------------------------------------------------------------------------ whole models through the engine
@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    """Three models, each twice: with random routers (the 32-bit tests) and, under ``<name>/pinned``, with a routing that
    rounding cannot change (the bfloat16 tests: two choice scores that differ in the third digit would otherwise decide
    whether a position passes)."""
    out = {}
    for name, cfg, seed in (("A", CFG_A, 11), ("B", CFG_B, 12), ("C", CFG_C, 13), ("D", CFG_D, 14)):
        out[name] = write_model(str(tmp_path_factory.mktemp("dus_" + name.lower())), cfg, seed)
        out[name + "/pinned"] = write_model(str(tmp_path_factory.mktemp("dus_pin_" + name.lower())), cfg, seed, weights=pin_routing(cfg))
    return out


def folder_for(folders, name, dtype):
    return folders[name if dtype == "float32" else name + "/pinned"]


def judge(folder, dtype):
    """32-bit: element by element. bfloat16: by a multiple of what rounding alone does to this model."""
    if dtype == "float32":
        return lambda got, ref, ids, what: assert_close(got, ref, torch.float32, what)
    return lambda got, ref, ids, what: assert_within_rounding(got, ref, plain_logits(folder, ids, stored_as=torch.bfloat16)[:ref.shape[0]], what)


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
    with open(os.path.join(folder, "config.json")) as f:
        return json.load(f)["vocab"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,n,page", [("A", 45, 4), ("B", 141, 8), ("C", 300, 16), ("D", 330, 16)])
def test_engine_prompts_decoding_and_portions_equal_plain(folders, dtype, name, n, page):
    folder = folder_for(folders, name, dtype)
    ids = tokens(n, vocab_of(folder), 5)
    ref = plain_logits(folder, ids)
    eng = gpu_engine(folder, dtype, page=page, pages=128)
    close = judge(folder, dtype)
    whole = run_cut(eng, "whole", ids, [n])
    close(whole, ref, ids, "whole prompt")
    tail = 40 if n > 100 else n - 1
    close(run_cut(eng, "decode", ids, [n - tail] + [1] * tail), ref, ids, "prompt, then token by token")
    cuts = [2, 7, 2, 13, 1, 1, 5, 2]
    cuts = cuts + [n - sum(cuts) - 2, 2]
    got = run_cut(eng, "cut", ids, cuts)
    close(got, ref, ids, "portions")
    if dtype == "float32":      # the same arithmetic per position whatever the cut
        assert (got - whole).abs().max().item() <= 1e-5 * max(1.0, ref.abs().max().item())
    eng.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_engine_unequal_requests_and_reused_slots_and_pages(folders, dtype):
    from nanoinfer_b200.engine import StepEntry
    folder = folder_for(folders, "A", dtype)
    eng = gpu_engine(folder, dtype, page=4, pages=30, slots=2)
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
        judge(folder, dtype)(torch.cat(got[k]), plain_logits(folder, seqs[k]), seqs[k], f"request {k}")


def test_long_decoding_through_captured_graphs_passes_windows_chunks_and_pages(folders):
    """150 tokens one by one (two requests side by side, so the steps are replayed from a captured graph): the window of 5
    and the chunks of 3 and 7 are passed many times, pages behind them go back to the pool."""
    from nanoinfer_b200.engine import StepEntry
    eng = gpu_engine(folders["A"], "float32", page=4, pages=200, slots=2)
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


def test_greedy_generation_through_the_scheduler(folders):
    from nanoinfer_b200.api import Model
    from nanoinfer_b200.config import EngineConfig
    from nanoinfer_b200.engine.scheduler import Request, Scheduler
    m = Model(folders["B"], EngineConfig(dtype="float32", page_size=8, num_pages=48, max_batch=3, max_tokens_per_step=8))
    sched = Scheduler(m)
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
    m.engine.cache.check()


def test_the_first_tokens_of_a_sequence_behind_windows_and_chunks(tmp_path):
    """Changing the FIRST token of a 300-token prompt must not move the last position's logits when every layer has a
    window or a chunk that ended long ago, and the engine must agree with the plain implementation at the first positions,
    where a window or chunk is not yet full, decoded one by one from position 0."""
    from nanoinfer_b200.engine import StepEntry
    cfg = model(64, 48, [windowed(2, 1, 16, 8, 50, 8, 1e4, mlp=moe(3, 1, 32, identity=1)), chunked(2, 1, 16, 8, 64, mlp=dense(32))])
    d = write_model(str(tmp_path), cfg, 5)
    ids = tokens(300, 64, 3)
    other = [(ids[0] + 1) % 64] + ids[1:]
    ref_a, ref_b = plain_logits(d, ids), plain_logits(d, other)
    assert (ref_a[-1] - ref_b[-1]).abs().max().item() < 1e-9 and (ref_a[5] - ref_b[5]).abs().max().item() > 1e-3
    eng = gpu_engine(d, "float32", page=16, pages=64, slots=2)
    for seq, ref in ((ids, ref_a), (other, ref_b)):
        rc = eng.open("x")
        head = torch.cat([eng.step([StepEntry(rc, [t], [0])]).clone() for t in seq[:70]])
        eng.step([StepEntry(rc, seq[70:290], [])])
        last = None
        for t in seq[290:]:
            last = eng.step([StepEntry(rc, [t], [0])]).clone()
        eng.close(rc)
        assert_close(head, ref[:70], torch.float32, "the first positions")
        assert_close(last[0], ref[-1], torch.float32, "the last position")


@pytest.mark.parametrize("seed,dtype", [(500, "float32"), (501, "float32"), (502, "float32"), (503, "float32"), (504, "float32"), (505, "float32"),
                                        (506, "float32"), (507, "float32"), (501, "bfloat16"), (503, "bfloat16"), (506, "bfloat16"),
                                        (549, "float32"), (549, "bfloat16"), (553, "bfloat16")])
def test_random_configurations(seed, dtype, tmp_path):
    """Layer orders, sizes and constants drawn at random (one head, a window of 1, one expert, all outputs chosen, widths
    that no vector path takes ...): a prompt in portions with a decoded tail beside a second request, against the plain
    implementation."""
    from nanoinfer_b200.engine import StepEntry
    rng = random.Random(seed)
    cfg = random_config(rng)
    d = write_model(str(tmp_path), cfg, seed, weights=None if dtype == "float32" else pin_routing(cfg))
    n = 70
    ids, other = tokens(n, cfg["vocab"], seed), tokens(33, cfg["vocab"], seed + 1)
    ref, ref2 = plain_logits(d, ids), plain_logits(d, other)
    eng = gpu_engine(d, dtype, page=rng.choice([4, 16]), pages=200, slots=2)
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
    judge(d, dtype)(torch.cat(got), ref, ids, "first request")
    judge(d, dtype)(torch.cat(got2), ref2[:pos2], other, "second request")
    eng.check_device()
    eng.cache.check()


@pytest.mark.parametrize("seed,dtype", [(21, "float32"), (21, "bfloat16"), (34, "float32"), (34, "bfloat16"), (47, "bfloat16")])
def test_larger_configurations_under_a_mixed_schedule(seed, dtype, tmp_path):
    """Six requests of 60 to 230 tokens, at most four live: portions of 2 to 100 tokens beside single tokens, requests left
    out of a step, slots and pages given back and used again in a pool made for four; sizes of a small real model
    (tensor-core paths of every kernel in bfloat16). Every position of every request against the plain implementation."""
    from nanoinfer_b200.engine import StepEntry
    rng = random.Random(seed)
    cfg = random_config(rng, small=False)
    lens = [rng.randint(60, 230) for _ in range(6)]
    seqs = [tokens(n, cfg["vocab"], seed * 10 + i) for i, n in enumerate(lens)]
    plan = mixed_schedule(rng, lens)
    assert max(len(step) for step in plan) == 4 and any(c > 1 for step in plan for _, c in step if len(step) > 1)
    page = rng.choice([16, 64])
    d = write_model(str(tmp_path), cfg, seed, weights=None if dtype == "float32" else pin_routing(cfg))
    eng = gpu_engine(d, dtype, page=page, pages=4 * (-(-max(lens) // page) + 1) + 2, slots=4)
    got, at, live = {i: [] for i in range(6)}, {i: 0 for i in range(6)}, {}
    for step in plan:
        entries = []
        for r, c in step:
            if r not in live:
                live[r] = eng.open(f"r{r}")
            entries.append(StepEntry(live[r], seqs[r][at[r]:at[r] + c], list(range(c))))
        logits = eng.step(entries).clone()
        row = 0
        for r, c in step:
            got[r].append(logits[row:row + c])
            row += c
            at[r] += c
            if at[r] == lens[r]:
                eng.close(live.pop(r))
        eng.cache.check()
    eng.check_device()
    for r in range(6):
        judge(d, dtype)(torch.cat(got[r]), plain_logits(d, seqs[r]), seqs[r], f"request {r}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_mixed_schedule_with_heads_of_64_and_128(folders, dtype):
    """Five requests, four live, portions of 2 to 100 tokens beside single tokens on the model whose prompt portions take the
    attention kernel with scores in tensor memory; pages of 16 in a pool made for four."""
    from nanoinfer_b200.engine import StepEntry
    rng = random.Random(5)
    folder = folder_for(folders, "D", dtype)
    lens = [211, 97, 160, 75, 130]
    seqs = [tokens(n, 200, 70 + i) for i, n in enumerate(lens)]
    plan = mixed_schedule(rng, lens)
    eng = gpu_engine(folder, dtype, page=16, pages=4 * (-(-max(lens) // 16) + 1) + 2, slots=4)
    got, at, live = {i: [] for i in range(5)}, {i: 0 for i in range(5)}, {}
    for step in plan:
        entries = []
        for r, c in step:
            if r not in live:
                live[r] = eng.open(f"r{r}")
            entries.append(StepEntry(live[r], seqs[r][at[r]:at[r] + c], list(range(c))))
        logits = eng.step(entries).clone()
        row = 0
        for r, c in step:
            got[r].append(logits[row:row + c])
            row += c
            at[r] += c
            if at[r] == lens[r]:
                eng.close(live.pop(r))
        eng.cache.check()
    eng.check_device()
    for r in range(5):
        judge(folder, dtype)(torch.cat(got[r]), plain_logits(folder, seqs[r]), seqs[r], f"request {r}")


def test_trace_replay_as_a_child_process(folders, tmp_path):
    """``bin/trace_run`` as a child process on a model of this design."""
    import subprocess
    import sys
    import numpy as np
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    ids = tokens(20, 77, 9)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": ids[:11], "want": [10]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": ids[11:], "want": [0, 8]}], "end": ["a"]}]
    for dtype, td in (("float32", torch.float32), ("bfloat16", torch.bfloat16)):
        out = tmp_path / dtype
        out.mkdir()
        r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folders["B"], "--dtype", dtype,
                            "--out", str(out), "--max-tokens", "64"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                           capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]
        assert [line for line in r.stdout.splitlines() if line.startswith("done")] == ["done 0", "done 1"]
        ref = plain_logits(folders["B"], ids)
        got0 = torch.from_numpy(np.fromfile(os.path.join(out, "0.f32"), dtype="<f4").reshape(1, -1))
        got1 = torch.from_numpy(np.fromfile(os.path.join(out, "1.f32"), dtype="<f4").reshape(2, -1))
        assert_close(got0, ref[[10]], td, "step 0")
        assert_close(got1, ref[[11, 19]], td, "step 1")


def test_command_line_tools_generate_and_serve(folders):
    """bin/generate (with the cache and recomputing every token) and bin/serve as child processes, in 32-bit: the plain
    implementation's greedy tokens."""
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
    common = ["--model-dir", folders["B"], "--dtype", "float32", "--block-size", "8", "--num-blocks", "48", "--max-tokens", "6"]
    for extra in ([], ["--no-cache"]):
        (got,) = tool("generate", common + ["--prompt", " ".join(map(str, prompts[0]))] + extra)
        assert got == greedy(prompts[0], 6), extra
    argv = common + ["--max-batch", "2", "--max-tokens-per-step", "16"]
    for p in prompts:
        argv += ["--prompt", " ".join(map(str, p))]
    got = tool("serve", argv)
    assert got == [greedy(p, 6) for p in prompts]
