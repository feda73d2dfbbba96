"""Darotar on a GPU: the kernels it added (the norm on a branch's output, router and experts, interleaved pairs with scaled
positions and a unit norm, values that are the keys, a sink and a gate in the latent attention) each against the plain
implementation, then whole models through the engine in both precisions, the scheduler and the command-line tools."""
import math
import random
from types import SimpleNamespace

import pytest
import torch

import plain_darotar as plain
from darotar_util import CFG_A, CFG_B, CFG_C, assert_within_rounding, attention, larger_config, latent, mixed_schedule, moe, pin_routing, plain_logits, random_config, tokens, write_model
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
        host=SimpleNamespace(q_lens=list(q_lens), ctx_lens=ctx_lens, num_requests=r))
    return ctx, bt.to(device), num_pages


def to_cpu(ctx):
    return SimpleNamespace(num_tokens=ctx.num_tokens, positions=ctx.positions.cpu(), req_index=ctx.req_index.cpu(),
                           q_start=ctx.q_start.cpu(), ctx_lens=ctx.ctx_lens.cpu(), host=ctx.host)


def rnd(*shape, seed=0, scale=1.0):
    return (torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale).to(DEV)


# ------------------------------------------------------------------------------------------ the norm on a branch's output
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m,n", [(1, 8), (7, 100), (5, 256), (3, 1030)])
def test_norm_of_a_branch_output_goes_into_the_stream(ops, dtype, m, n):
    y, x, gain = rnd(m, n, seed=1, scale=3.0), rnd(m, n, seed=2), rnd(n, seed=3)
    ref = x.double().cpu() + 0.6 * plain.norm(y.double().cpu(), gain.double().cpu(), 1e-3)
    h = torch.empty(m, n, dtype=dtype, device=DEV)
    ops.rmsnorm_add(y, gain, 1e-3, 0.6, x, h, True)
    assert_close(x, ref, torch.float32, "stream")
    assert_close(h, ref, dtype, "the stream in the storage type")
    assert y.abs().max().item() == 0.0
    y2 = rnd(m, n, seed=4)
    keep = y2.clone()
    ref = ref + 1.5 * plain.norm(y2.double().cpu(), gain.double().cpu(), 1e-3)
    ops.rmsnorm_add(y2, gain, 1e-3, 1.5, x)
    assert_close(x, ref, torch.float32, "stream, second branch")
    assert torch.equal(y2, keep)


# ------------------------------------------------------------------------------------------ router and experts
@pytest.mark.parametrize("m,experts,top", [(1, 1, 1), (9, 5, 2), (40, 33, 4), (6, 3, 3), (130, 70, 1)])
def test_router_picks_the_largest_scores(ops, m, experts, top):
    z = rnd(m, experts + 2, seed=5, scale=2.0)[:, 1:1 + experts]       # rows that lie apart
    sel_e = torch.empty(m, top, dtype=torch.int32, device=DEV)
    sel_w = torch.empty(m, top, dtype=torch.float32, device=DEV)
    ops.moe_route(z, top, sel_e, sel_w)
    s = torch.sigmoid(z.double().cpu())
    want = torch.topk(s, top, dim=-1)
    assert torch.equal(sel_e.cpu().long(), want.indices)
    assert_close(sel_w, want.values, torch.float32, "scores")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m,hidden,ff,experts,top", [(1, 32, 8, 1, 1), (9, 64, 24, 5, 2), (300, 72, 40, 3, 1), (150, 100, 130, 6, 3),
                                                     (33, 128, 64, 4, 4), (200, 256, 64, 16, 2), (700, 256, 136, 5, 2), (40, 128, 264, 8, 2),
                                                     (513, 64, 16, 2, 1), (8, 512, 320, 8, 2), (1100, 192, 72, 3, 3)])
def test_experts_read_the_weighted_token(ops, dtype, m, hidden, ff, experts, top):
    """Against the plain loop over tokens and choices: the score multiplies the expert's input, is not renormalized, and a
    token's choices are summed into what the stream's row already holds. 300 tokens for 3 experts make several row tiles
    per expert; 150 tokens with 3 choices take the path that sums the choices afterwards. In bfloat16, widths in multiples
    of 8 take the tensor-core products: row tiles of 32 while an expert gets few rows and of 128 beyond, feature tiles that
    end inside the 128 (the next rows of the weight matrix are the up rows or the next expert's), a K that ends inside a
    stage of 64."""
    h = rnd(m, hidden, seed=1).to(dtype)
    w = {"r.router": rnd(experts, hidden, seed=2, scale=hidden ** -0.5).to(dtype)}
    for e in range(experts):
        w[f"r.e{e}.gate"] = rnd(ff, hidden, seed=10 + 3 * e, scale=hidden ** -0.5).to(dtype)
        w[f"r.e{e}.up"] = rnd(ff, hidden, seed=11 + 3 * e, scale=hidden ** -0.5).to(dtype)
        w[f"r.e{e}.down"] = rnd(hidden, ff, seed=12 + 3 * e, scale=ff ** -0.5).to(dtype)
    z = (h.double() @ w["r.router"].double().t()).float()
    sel_e = torch.empty(m, top, dtype=torch.int32, device=DEV)
    sel_w = torch.empty(m, top, dtype=torch.float32, device=DEV)
    ops.moe_route(z, top, sel_e, sel_w)
    before = rnd(m, hidden, seed=3)
    out = before.clone()
    gate_up = torch.stack([torch.cat([w[f"r.e{e}.gate"], w[f"r.e{e}.up"]]) for e in range(experts)]).contiguous()
    down = torch.stack([w[f"r.e{e}.down"] for e in range(experts)]).contiguous()
    ops.moe_experts(h, sel_e, sel_w, gate_up, down, out)
    mlp = {"router": {"experts": experts, "top": top}}
    ref = plain.routed_experts(mlp, {k: v.double().cpu() for k, v in w.items()}, "r", h.double().cpu())
    assert_close(out - before, ref, dtype, "experts")
    if dtype == torch.bfloat16:       # the path on the CUDA cores gives the same
        slow = before.clone()
        ops.with_options(force_simt_gemm=True).moe_experts(h, sel_e, sel_w, gate_up, down, slow)
        assert_close(slow - before, ref, dtype, "experts, CUDA cores")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m,hidden,ff,experts,top", [(1, 32, 8, 1, 1), (8, 256, 64, 8, 2), (5, 72, 40, 33, 4), (16, 128, 24, 12, 1), (3, 100, 130, 6, 3),
                                                     (64, 64, 16, 5, 2)])
def test_a_short_step_routes_groups_and_gathers_in_one_launch(ops, dtype, m, hidden, ff, experts, top):
    """Router, choice, grouping and gathered rows of a short step in one launch: the same choices and scores as the
    separate steps, and the experts' result through its plan equals the plain loop."""
    h = rnd(m, hidden, seed=1).to(dtype)
    w = {"r.router": rnd(experts, hidden, seed=2, scale=hidden ** -0.5).to(dtype)}
    for e in range(experts):
        w[f"r.e{e}.gate"] = rnd(ff, hidden, seed=10 + 3 * e, scale=hidden ** -0.5).to(dtype)
        w[f"r.e{e}.up"] = rnd(ff, hidden, seed=11 + 3 * e, scale=hidden ** -0.5).to(dtype)
        w[f"r.e{e}.down"] = rnd(hidden, ff, seed=12 + 3 * e, scale=ff ** -0.5).to(dtype)
    gate_up = torch.stack([torch.cat([w[f"r.e{e}.gate"], w[f"r.e{e}.up"]]) for e in range(experts)]).contiguous()
    down = torch.stack([w[f"r.e{e}.down"] for e in range(experts)]).contiguous()
    sel_e = torch.full((m, top), -1, dtype=torch.int32, device=DEV)
    sel_w = torch.zeros(m, top, dtype=torch.float32, device=DEV)
    plan = ops.moe_step(h, w["r.router"], top, gate_up, down, sel_e, sel_w)
    assert plan is not None, "a step of these sizes fits one block"
    s = torch.sigmoid(h.double().cpu() @ w["r.router"].double().cpu().t())
    want = torch.topk(s, top, dim=-1)
    assert torch.equal(sel_e.cpu().long(), want.indices)
    assert_close(sel_w, want.values, torch.float32, "scores")
    # the grouping: every entry has a row, rows of one expert are together, the tiles cover them
    row_of, src_of = plan.row_of.cpu().long(), plan.src_of.cpu().long()
    assert torch.equal(src_of[row_of], torch.arange(m * top))
    by_row = sel_e.cpu().flatten()[src_of]
    assert torch.equal(by_row, by_row.sort().values)
    before = rnd(m, hidden, seed=3)
    out = before.clone()
    ops.moe_experts(h, sel_e, sel_w, gate_up, down, out, plan=plan)
    mlp = {"router": {"experts": experts, "top": top}}
    ref = plain.routed_experts(mlp, {k: v.double().cpu() for k, v in w.items()}, "r", h.double().cpu())
    assert_close(out - before, ref, dtype, "experts of a short step")
    assert ops.with_options(no_moe_step=True).moe_step(h, w["r.router"], top, gate_up, down, sel_e, sel_w) is None


# ------------------------------------------------------------------------------------------ attention whose values are the keys
def _prepared(ops, dtype, ctx, bt, page, num_pages, heads, kv, dim, qk, freq, rot, eps=1e-6):
    kp = torch.zeros(num_pages, kv, page, dim, dtype=dtype, device=DEV)
    vp = torch.zeros(num_pages, kv, page, dim, dtype=dtype, device=DEV)
    q = torch.empty(qk.shape[0], heads * dim, dtype=dtype, device=DEV)
    ops.attention_prepare(qk, q, heads, kv, dim, dim, None, None, eps, freq, rot, ctx, bt, page, kp, vp, True, layout="interleaved",
                          unit_norm_after=True, values_are_keys=True)
    return q, kp, vp


def _rows_of(pages, bt, req, positions, page):
    """The cached rows [positions, kv heads, width] of one request."""
    pg = bt[req, torch.as_tensor(positions) // page].long().cpu()
    return pages.cpu()[pg, :, torch.as_tensor(positions) % page, :].double()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv,dim,rot,factor,page", [(4, 2, 12, 8, 2.0, 4), (3, 1, 16, 16, 1.0, 4), (2, 2, 64, 64, 4.0, 16), (6, 3, 40, 2, 32.0, 8),
                                                          (1, 1, 130, 130, 8.0, 16)])
def test_operands_interleaved_pairs_scaled_positions_unit_norm(ops, dtype, heads, kv, dim, rot, factor, page):
    """Queries and cached keys: pairs (2i, 2i + 1) of the first ``rot`` elements turned by position * base^(-2i/rot) / factor,
    then every head divided by its root mean square; cached values: the keys as projected."""
    q_lens, before = [5, 1, 9], [3, 40, 0]
    ctx, bt, num_pages = batch(q_lens, before, page_size=page)
    m = sum(q_lens)
    qk = rnd(m, (heads + kv) * dim + 3, seed=1)[:, 1:1 + (heads + kv) * dim]
    cfg_rot = {"dims": rot, "base": 700.0, "scaling": {"factor": factor}}
    freq = plain.frequencies(cfg_rot).float().to(DEV)
    q, kp, vp = _prepared(ops, dtype, ctx, bt, page, num_pages, heads, kv, dim, qk, freq, rot, eps=1e-5)
    at = 0
    for r, (n, b) in enumerate(zip(q_lens, before)):
        rows = qk[at:at + n].double().cpu()
        rq = plain.rms_unit(plain.rotate_interleaved(rows[:, :heads * dim].view(n, heads, dim), cfg_rot, first=b), 1e-5)
        rk = plain.rms_unit(plain.rotate_interleaved(rows[:, heads * dim:].view(n, kv, dim), cfg_rot, first=b), 1e-5)
        assert_close(q[at:at + n].view(n, heads, dim), rq, dtype, "queries")
        assert_close(_rows_of(kp, bt, r, list(range(b, b + n)), page), rk, dtype, "cached keys")
        assert_close(_rows_of(vp, bt, r, list(range(b, b + n)), page), rows[:, heads * dim:].view(n, kv, dim), dtype, "cached values")
        at += n


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv,dim,rot,window,page", [(4, 2, 12, 8, 5, 4), (3, 1, 16, 16, 300, 4), (8, 2, 64, 64, 70, 16), (4, 4, 32, 16, 129, 16),
                                                          (2, 1, 96, 48, 33, 8), (2, 2, 136, 136, 64, 16)])
def test_windowed_mixer_in_portions_and_decoding_equals_plain(ops, dtype, heads, kv, dim, rot, window, page):
    """The mixer up to its output product against the plain one: a prompt of 150 tokens in portions (2 tokens, a portion
    that crosses pages and the window, single tokens) beside a second request, through the kernel's both paths."""
    n, n2, width = 150, 21, 48
    mixer = {"heads": heads, "kv_heads": kv, "dim": dim, "rot": {"dims": rot, "base": 5000.0, "scaling": {"factor": 2.0}},
             "scale": 2.5 / dim, "mask": {"size": window}}
    w = {"a.q": rnd(heads * dim, width, seed=1, scale=width ** -0.5).to(dtype), "a.k": rnd(kv * dim, width, seed=2, scale=width ** -0.5).to(dtype),
         "a.o": torch.eye(heads * dim, device=DEV)}
    hs = [rnd(n, width, seed=3).to(dtype), rnd(n2, width, seed=4).to(dtype)]
    refs = [plain.attention_mixer(mixer, {k: v.double().cpu() for k, v in w.items()}, "a", h.double().cpu(), 1e-6) for h in hs]
    freq = plain.frequencies(mixer["rot"]).float().to(DEV)
    w_in = torch.cat([w["a.q"], w["a.k"]]).double()
    paths = [ops] if dtype == torch.float32 else [ops, ops.with_options(force_general_attention=True), ops.with_options(fixed_decode_splits=3)]
    for k in paths:
        num_pages = -(-n // page) + -(-n2 // page) + 4
        order = torch.randperm(num_pages, generator=torch.Generator().manual_seed(7)).tolist()
        bt = torch.full((2, -(-n // page)), -1, dtype=torch.int32)
        kp = torch.zeros(num_pages, kv, page, dim, dtype=dtype, device=DEV)
        vp = torch.zeros_like(kp)
        done, got = [0, 0], [[], []]
        for step in ([2, 5], [61, 1], [1, 1], [70, 2], [1, 12], [2, 0], [1, 0], [12, 0]):
            reqs = [i for i in (0, 1) if step[i] > 0]
            q_lens, before = [step[i] for i in reqs], [done[i] for i in reqs]
            for i in reqs:
                for p in range(-(-(done[i] + step[i]) // page)):
                    if bt[i, p] < 0:
                        bt[i, p] = order.pop()
            ctx, _, _ = batch(q_lens, before, page_size=page)
            bt_step = bt[reqs].to(DEV).contiguous()
            h = torch.cat([hs[i][done[i]:done[i] + step[i]] for i in reqs])
            qk = (h.double() @ w_in.t()).float()
            q = torch.empty(h.shape[0], heads * dim, dtype=dtype, device=DEV)
            k.attention_prepare(qk, q, heads, kv, dim, dim, None, None, 1e-6, freq, rot, ctx, bt_step, page, kp, vp, True, layout="interleaved",
                                unit_norm_after=True, values_are_keys=True)
            out = torch.empty(h.shape[0], heads * dim, dtype=torch.float32, device=DEV)
            k.attention_flex(q, out, heads, kv, dim, dim, mixer["scale"], 0.0, None, window, 0, 1.0, ctx, bt_step, page, kp, vp)
            at = 0
            for i in reqs:
                got[i].append(out[at:at + step[i]])
                at += step[i]
                done[i] += step[i]
        assert done == [n, n2]
        for i in (0, 1):
            assert_close(torch.cat(got[i]), refs[i], dtype, f"request {i}, path {paths.index(k)}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("decode", [False, True])
@pytest.mark.parametrize("window,page", [(1, 4), (2, 4), (6, 4), (32, 8), (33, 16), (64, 16), (100, 16), (257, 64)])
def test_a_key_at_the_windows_edge_is_seen_and_the_one_before_is_not(ops, window, page, decode, dtype):
    """All keys are alike but two neighbours, whose scores stand out and which carry marks of their own in elements 2 and 3
    (the values are the keys as projected). A query sees the later one while it lies within the window, and never the
    earlier one after that; one position before, both."""
    dim, n = 16, 2 * window + 70
    qk = torch.zeros(n, 2 * dim, device=DEV)
    qk[:, dim] = 1.0                                     # every key: e0
    a = 37                                               # the later of the two marked keys; a - 1 is the earlier one
    qk[a, dim + 1], qk[a, dim + 2] = 9.0, 4.0
    qk[a - 1, dim + 1], qk[a - 1, dim + 3] = 9.0, 4.0
    qk[:, 1] = 9.0                                       # every query asks for e1
    full_ctx, bt, num_pages = batch([n], [0], page_size=page)
    q_all, kp, vp = _prepared(ops, dtype, full_ctx, bt, page, num_pages, 1, 1, dim, qk, None, 0)
    last = a + window - 1                                # the last position that sees key a
    for p, want2, want3 in ((last, 4.0, 0.0), (last + 1, 0.0, 0.0), (last - 1, 2.0, 2.0)):
        if p - 1 < a:                                    # a window of one or two: the query's own key is a marked one
            continue
        ctx, _, _ = (batch([1], [p], page_size=page) if decode else batch([2], [p - 1], page_size=page))
        rows = [p] if decode else [p - 1, p]
        out = torch.empty(len(rows), dim, device=DEV)
        ops.attention_flex(q_all[rows].contiguous(), out, 1, 1, dim, dim, 1.0, 0.0, None, window, 0, 1.0, ctx, bt, page, kp, vp)
        assert abs(out[-1, 2].item() - want2) < 2e-2 and abs(out[-1, 3].item() - want3) < 2e-2, (p, out[-1, :4].tolist())
    ctx, _, _ = batch([1], [a], page_size=page)          # the marked key's own position: with a window of one, itself alone
    out = torch.empty(1, dim, device=DEV)
    ops.attention_flex(q_all[[a]].contiguous(), out, 1, 1, dim, dim, 1.0, 0.0, None, window, 0, 1.0, ctx, bt, page, kp, vp)
    want3 = 0.0 if window == 1 else 2.0
    assert abs(out[0, 3].item() - want3) < 2e-2, out[0, :4].tolist()


# ------------------------------------------------------------------------------------------ attention through a latent
def _latent_pages(ops, dtype, n, rank, rot, page, z, freq, layout="half"):
    ctx, bt, num_pages = batch([n], [0], page_size=page)
    pages = torch.zeros(num_pages, 1, page, rank + rot, dtype=dtype, device=DEV)
    ops.latent_store(z, torch.ones(rank, device=DEV), 1e-6, freq, 1.0, ctx, bt, page, pages, rank, rot, layout=layout)
    return bt, pages


def _query_rows(ops, dtype, rank, rot, q_lat, q_rot):
    """Query rows [tokens, heads, width] in the layout the attention kernel reads (latent part, rotated part, zeros)."""
    width, qdt = ops.latent_query_layout(dtype, rank, rot)
    m, heads = q_lat.shape[:2]
    qa = torch.zeros(m, heads, width, dtype=qdt, device=DEV)
    qa[..., :rank] = q_lat.to(qdt)
    qa[..., rank:rank + rot] = q_rot.to(qdt)
    return qa.view(m, heads * width)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,dim,rdim,vdim,q_rank,rank,page", [(3, 8, 4, 6, 10, 12, 4), (4, 16, 8, 16, 24, 32, 8), (8, 32, 16, 24, 40, 48, 16),
                                                                  (1, 4, 2, 4, 5, 6, 4), (5, 40, 30, 3, 16, 50, 16)])
def test_latent_mixer_with_sink_and_gate_in_portions_equals_plain(ops, dtype, heads, dim, rdim, vdim, q_rank, rank, page):
    """The mixer up to its output product against the plain one (half-split pairs, a sink per head, a gate on the heads):
    a prompt in portions and single tokens beside a second request, through the general and the tensor-core path."""
    n, n2, width = 140, 19, 40
    mixer = {"heads": heads, "dim": dim, "rot_dim": rdim, "vdim": vdim, "kv_rank": rank, "rot": {"dims": rdim, "base": 3000.0},
             "scale": (dim + rdim) ** -0.5}
    shapes = {"dq": (q_rank, width), "uq": (heads * (dim + rdim), q_rank), "dkv": (rank + rdim, width), "uk": (heads * dim, rank),
              "uv": (heads * vdim, rank), "g": (heads * vdim, width)}
    w = {f"a.{k}": rnd(*s, seed=20 + i, scale=1.2 * s[1] ** -0.5).to(dtype) for i, (k, s) in enumerate(shapes.items())}
    w["a.dq.norm"], w["a.dkv.norm"] = (1 + 0.1 * rnd(q_rank, seed=30)).to(dtype), (1 + 0.1 * rnd(rank, seed=31)).to(dtype)
    w["a.sink"] = rnd(heads, seed=32, scale=1.5).to(dtype)
    w["a.o"] = torch.eye(heads * vdim, device=DEV)
    hs = [rnd(n, width, seed=3).to(dtype), rnd(n2, width, seed=4).to(dtype)]
    w64 = {k: v.double().cpu() for k, v in w.items()}
    refs = [plain.latent_mixer(mixer, w64, "a", h.double().cpu(), 1e-6, plain.latent_rows(mixer, w64, "a", h.double().cpu(), 1e-6)) for h in hs]
    freq = plain.frequencies(mixer["rot"]).float().to(DEV)
    f32 = lambda name: w[name].float().contiguous()
    paths = [ops] if dtype == torch.float32 else [ops, ops.with_options(force_general_attention=True), ops.with_options(fixed_decode_splits=3)]
    for k in paths:
        num_pages = -(-n // page) + -(-n2 // page) + 4
        order = torch.randperm(num_pages, generator=torch.Generator().manual_seed(7)).tolist()
        bt = torch.full((2, -(-n // page)), -1, dtype=torch.int32)
        pages = torch.zeros(num_pages, 1, page, rank + rdim, dtype=dtype, device=DEV)
        done, got = [0, 0], [[], []]
        for step in ([1, 1], [1, 1], [2, 5], [61, 1], [1, 1], [60, 2], [1, 8], [2, 0], [1, 0], [10, 0]):
            reqs = [i for i in (0, 1) if step[i] > 0]
            q_lens, before = [step[i] for i in reqs], [done[i] for i in reqs]
            for i in reqs:
                for p in range(-(-(done[i] + step[i]) // page)):
                    if bt[i, p] < 0:
                        bt[i, p] = order.pop()
            ctx, _, _ = batch(q_lens, before, page_size=page)
            bt_step = bt[reqs].to(DEV).contiguous()
            h = torch.cat([hs[i][done[i]:done[i] + step[i]] for i in reqs])
            m = h.shape[0]
            z = (h.double() @ w["a.dkv"].double().t()).float()
            k.latent_store(z, f32("a.dkv.norm"), 1e-6, freq, 1.0, ctx, bt_step, page, pages, rank, rdim, layout="half")
            cq = plain.norm(h.double() @ w["a.dq"].double().t(), w["a.dq.norm"].double(), 1e-6).to(dtype)
            q32 = (cq.double() @ w["a.uq"].double().t()).float()
            qw, qdt = k.latent_query_layout(dtype, rank, rdim)
            qa = torch.empty(m, heads * qw, dtype=qdt, device=DEV)
            k.latent_query(q32, w["a.uk"], freq, 1.0, ctx.positions, qa, heads, dim, rank, rdim, layout="half")
            lat = torch.empty(m, heads * rank, dtype=torch.float32, device=DEV)
            k.latent_attention(qa, lat, ctx, bt_step, page, pages, heads, rank, rdim, mixer["scale"], 0, sink32=f32("a.sink"))
            gate = (h.double() @ w["a.g"].double().t()).float()
            out = torch.empty(m, heads * vdim, dtype=dtype, device=DEV)
            k.latent_value(lat, w["a.uv"], out, heads, vdim, rank, gate32=gate)
            at = 0
            for i in reqs:
                got[i].append(out[at:at + step[i]])
                at += step[i]
                done[i] += step[i]
        assert done == [n, n2]
        for i in (0, 1):
            assert_close(torch.cat(got[i]), refs[i], dtype, f"request {i}, path {paths.index(k)}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("decode", [False, True])
@pytest.mark.parametrize("rank,rot,page,n,far", [(16, 8, 16, 700, 3), (32, 8, 16, 1500, 0), (12, 4, 4, 300, 1), (64, 16, 64, 2100, 64)])
def test_a_far_key_among_hundreds_is_found_and_the_sink_counts_once(ops, rank, rot, page, n, far, decode, dtype):
    """Rows that are all alike but one far back whose score stands out: the query at the end returns that row. With a
    query that scores every key alike, a sink of log(keys) halves the mean of the rows, and one of -30 leaves it."""
    z = torch.zeros(n, rank + rot, device=DEV)
    z[:, 0] = 1.0
    z[far, 1] = 2.0
    bt, pages = _latent_pages(ops, dtype, n, rank, rot, page, z, torch.zeros(rot // 2, device=DEV))
    rows = _rows_of(pages, bt, 0, [far, far + 1], page)[:, 0, :rank]
    ctx, _, _ = batch([1], [n - 1], page_size=page) if decode else batch([2], [n - 2], page_size=page)
    m, heads = ctx.num_tokens, 2
    q_lat = torch.zeros(m, heads, rank, device=DEV)
    q_lat[:, 0, 1] = 8.0                                   # head 0 asks for the mark; head 1 scores every row alike
    qa = _query_rows(ops, dtype, rank, rot, q_lat, torch.zeros(m, heads, rot, device=DEV))
    for sink, share in ((-30.0, 1.0), (math.log(n), 0.5)):
        lat = torch.empty(m, heads * rank, dtype=torch.float32, device=DEV)
        sinks = torch.tensor([-30.0, sink], device=DEV)
        ops.latent_attention(qa, lat, ctx, bt, page, pages, heads, rank, rot, 1.0, 0, sink32=sinks)
        got = lat[-1].view(heads, rank).double().cpu()
        assert (got[0] - rows[0]).abs().max().item() < 2e-2 * rows[0].abs().max().item(), got[0, :3].tolist()
        mean = (rows[1] * (n - 1) + rows[0]) / n           # every row but the marked one equals its neighbour
        assert (got[1] - share * mean).abs().max().item() < 2e-2 * mean.abs().max().item(), (got[1, :3].tolist(), share)


# ------------------------------------------------------------------------------------------ whole models through the engine
@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    """Three models, each twice: with random routers (the 32-bit tests) and, under ``<name>/pinned``, with a routing
    that no rounding can change (the bfloat16 tests: two experts whose scores differ in the third digit would otherwise
    decide whether a position passes)."""
    out = {}
    for name, cfg, seed in (("A", CFG_A, 11), ("B", CFG_B, 12), ("C", CFG_C, 13)):
        out[name] = write_model(str(tmp_path_factory.mktemp("dar_" + name.lower())), cfg, seed)
        out[name + "/pinned"] = write_model(str(tmp_path_factory.mktemp("dar_pin_" + name.lower())), cfg, seed, weights=pin_routing(cfg))
    return out


def folder_for(folders, name, dtype):
    return folders[name if dtype == "float32" else name + "/pinned"]


def judge(folder, dtype):
    """How a whole model's logits are compared with the plain implementation's: in 32-bit element by element; in bfloat16
    by a multiple of what rounding alone does to this model (its norms stand on the branches' outputs, so a branch's
    relative error enters the stream undamped, layer after layer)."""
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
    import json, os
    with open(os.path.join(folder, "config.json")) as f:
        return json.load(f)["vocab"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,n,page", [("A", 45, 4), ("B", 41, 8), ("C", 300, 16)])
def test_engine_prompts_decoding_and_portions_equal_plain(folders, dtype, name, n, page):
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    folder = folder_for(folders, name, dtype)
    ids = tokens(n, vocab_of(folder), 5)
    ref = plain_logits(folder, ids)
    eng = gpu_engine(folder, dtype, page=page, pages=64)
    close = judge(folder, dtype)
    whole = run_cut(eng, "whole", ids, [n])
    close(whole, ref, ids, "whole prompt")
    tail = 12 if n > 100 else n - 1
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
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    folder = folder_for(folders, "A", dtype)
    eng = gpu_engine(folder, dtype, page=4, pages=24, slots=2)
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


def test_long_decoding_through_captured_graphs_passes_windows_and_pages(folders):
    """150 tokens one by one (two requests side by side, so the steps are replayed from a captured graph): the window of 5
    is passed many times, pages behind it go back to the pool, the latent rows grow page by page."""
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


def test_the_first_token_reaches_the_logits_through_the_latent_rows(tmp_path):
    """Latent layers alone (one reads the other's rows): changing the FIRST token of a 400-token prompt must move the last
    position's logits as the plain implementation says; behind a window it must not move them at all."""
    from nanoinfer_b200.engine import StepEntry
    cases = {"latent": ([latent(2, 16, 8, 16, 16, 24, 1e4, mlp=moe(3, 1, 32)), latent(3, 8, 8, 8, 8, 24, 1e4, kv_from=0)], True),
             "window": ([attention(2, 1, 16, 8, 1e4, factor=2.0, window=50, mlp=moe(3, 1, 32))], False)}
    for name, (layers, reaches) in cases.items():
        cfg = {"architecture": "Darotar", "vocab": 64, "width": 48, "norm": {"eps": 1e-6}, "residual_mult": 0.9, "layers": layers}
        d = write_model(str(tmp_path / name), cfg, 5)
        ids = tokens(400, 64, 3)
        other = [(ids[0] + 1) % 64] + ids[1:]
        ref_a, ref_b = plain_logits(d, ids)[-1], plain_logits(d, other)[-1]
        assert ((ref_a - ref_b).abs().max().item() > 1e-3) == reaches, f"{name}: the test's model does not show what it should"
        eng = gpu_engine(d, "float32", page=16, pages=64, slots=2)
        for seq, ref in ((ids, ref_a), (other, ref_b)):
            rc = eng.open("x")
            eng.step([StepEntry(rc, seq[:390], [])])
            last = None
            for t in seq[390:]:
                last = eng.step([StepEntry(rc, [t], [0])]).clone()
            eng.close(rc)
            assert_close(last[0], ref, torch.float32, name)


@pytest.mark.parametrize("seed,dtype", [(300, "float32"), (301, "float32"), (302, "float32"), (303, "float32"), (304, "float32"), (305, "float32"),
                                        (306, "float32"), (307, "float32"), (301, "bfloat16"), (303, "bfloat16"), (306, "bfloat16"),
                                        (449, "float32"), (449, "bfloat16"), (453, "bfloat16")])
def test_random_configurations(seed, dtype, tmp_path):
    """Layer orders, sizes and constants drawn at random (one head, a window of 1, one expert, all experts chosen, widths
    that no vector path takes ...): a prompt in portions with a decoded tail beside a second request, against the plain
    implementation."""
    from nanoinfer_b200.engine import StepEntry
    rng = random.Random(seed)
    cfg = random_config(rng)
    d = write_model(str(tmp_path), cfg, seed, weights=None if dtype == "float32" else pin_routing(cfg))
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
    judge(d, dtype)(torch.cat(got), ref, ids, "first request")
    judge(d, dtype)(torch.cat(got2), ref2[:pos2], other, "second request")
    eng.check_device()
    eng.cache.check()


@pytest.mark.parametrize("seed,dtype", [(21, "float32"), (21, "bfloat16"), (34, "float32"), (34, "bfloat16"), (47, "bfloat16")])
def test_larger_configurations_under_a_mixed_schedule(seed, dtype, tmp_path):
    """Six requests of 60 to 230 tokens, at most four live: portions of 2 to 100 tokens beside single tokens, requests left out of a
    step, slots and pages given back and used again in a pool made for four; sizes of a small real model (tensor-core paths of
    every kernel in bfloat16). Every position of every request against the plain implementation."""
    from nanoinfer_b200.engine import StepEntry
    rng = random.Random(seed)
    cfg = larger_config(rng)
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


def test_trace_replay_as_a_child_process(folders, tmp_path):
    """``bin/trace_run`` as a child process on a model of this design."""
    import json, os, subprocess, sys
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
