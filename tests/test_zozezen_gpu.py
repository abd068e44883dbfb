"""Zozezen on the GPU against the plain implementation (``plain_zozezen``): every new kernel alone, every new part alone
(fed in portions and token by token through the cache and the state slots, with keys that stand out far back, a sink that
decides, slots that are used again), and the whole model through the engine's own session, scheduler and command line, in
float32 and bfloat16, at sizes of its own."""

from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import helpers
import plain_ops
import plain_zozezen as plain
import zozezen_helpers as zh
from test_parts_gpu import Harness, rand, tol

pytestmark = pytest.mark.gpu
REPO = Path(__file__).resolve().parent.parent
DTYPES = [torch.float32, torch.bfloat16]


def bound_of(dtype, expected):
    return (1e-5 if dtype in ("float32", torch.float32) else 1.5e-2) * max(1.0, float(expected.abs().max()))


def cpu(tensor):
    return None if tensor is None else tensor.detach().cpu().clone()


# --------------------------------------------------------------------------- kernels alone


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("size", [40, 200, 1000, 4100])
def test_output_norm_add_and_norm(dtype, size):
    from miniserve_b200 import kernels

    rows = 7
    residual, delta = rand((rows, size), torch.float32, 1, 2.0), rand((rows, size), dtype, 2, 3.0)
    post, weight = 0.2 + rand((size,), torch.float32, 3, 0.05), 1 + rand((size,), torch.float32, 4, 0.1)
    out = torch.empty((rows, size), dtype=dtype).cuda()
    expected_res, expected_out = cpu(residual), cpu(out)
    plain_ops.postnorm_add_rmsnorm(expected_res, cpu(delta), cpu(post), 1e-5, cpu(weight), 1e-6, expected_out)
    picked = torch.tensor([5, 0, 5], dtype=torch.int32).cuda()
    gathered = torch.empty((3, size), dtype=dtype).cuda()
    before = residual.clone()
    kernels.postnorm_add_rmsnorm(residual, delta, post, 1e-5, weight, 1e-6, gathered, picked)
    assert torch.equal(residual, before)                       # gathered rows leave the stream alone
    kernels.postnorm_add_rmsnorm(residual, delta, post, 1e-5, weight, 1e-6, out)
    assert torch.allclose(residual.cpu().double(), expected_res.double(), atol=1e-5)
    assert torch.allclose(out.cpu().double(), expected_out.double(), **tol(dtype, 3.0))
    assert torch.equal(gathered.cpu(), out.cpu()[picked.cpu().long()])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n_q,n_kv,d,dv,rotary,own", [(6, 3, 24, 40, 16, True), (5, 5, 6, 14, 2, True), (4, 1, 32, 8, 32, True),
                                                      (3, 3, 24, 40, 16, False), (8, 2, 128, 128, 64, True), (2, 1, 10, 3, 0, True)])
def test_prepare_of_free_layouts(dtype, n_q, n_kv, d, dv, rotary, own):
    from miniserve_b200 import kernels

    n, page = 9, 4
    q_col, k_col, v_col = 8, 8 + n_q * d, 8 + n_q * d + n_kv * d
    ld = (v_col + n_kv * dv + 11) // 8 * 8
    proj = rand((n, ld), dtype, 5)
    slots = torch.tensor([3, 0, -1, 7, 8, 9, 20, 21, 2], dtype=torch.int32).cuda()
    qw, kw = 1 + rand((d,), torch.float32, 6, 0.2), 1 + rand((d,), torch.float32, 7, 0.2)
    table = None
    if rotary:
        angles = rand((n, rotary // 2), torch.float32, 8, 3.0)
        table = torch.stack([angles.cos(), angles.sin()], dim=-1).contiguous()
    pools = [torch.zeros((6, n_kv, page, size), dtype=dtype).cuda() for size in (d, dv)]
    q_out = torch.empty((n, n_q, d), dtype=dtype).cuda()
    expected = [cpu(pools[0]), cpu(pools[1]), cpu(q_out)]
    plain_ops.qkv_prepare(cpu(proj), q_col, k_col if own else -1, v_col, n_q, n_kv, d, dv, cpu(slots), cpu(qw), cpu(kw), 1e-5, cpu(table), rotary,
                          expected[0], expected[1], expected[2])
    kernels.qkv_prepare(proj, q_col, k_col if own else -1, v_col, n_q, n_kv, d, dv, slots, qw, kw if own else None, 1e-5, table, rotary,
                        pools[0], pools[1], q_out)
    for got, want in zip((pools[0], pools[1], q_out), expected):
        assert torch.allclose(got.cpu().double(), want.double(), **tol(dtype, 4.0))
    if not own:
        assert float(pools[0].abs().max()) == 0 and float(pools[1].abs().max()) == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,P,N,G,taps,parts", [(6, 20, 24, 3, 4, 2), (1, 20, 6, 1, 1, 1), (3, 6, 36, 3, 5, 3), (4, 32, 128, 1, 4, 1),
                                                    (8, 16, 64, 2, 2, 8), (2, 5, 200, 2, 8, 2)])
def test_state_space_kernels(dtype, heads, P, N, G, taps, parts):
    """Convolution, recurrence and gated norm over a batch of unequal requests (a single token, a portion shorter than the
    convolution's reach, portions longer than the kernels' chunks) from states that are not zero, in slots out of order."""
    from miniserve_b200 import kernels

    inner = heads * P
    channels = inner + 2 * G * N
    ld = (2 * inner + 2 * G * N + heads + 7) // 8 * 8
    starts = [0, 1, 3, 3 + 150, 153 + 70]
    n = starts[-1]
    proj = rand((n, ld), dtype, 10)
    conv_w, conv_b = rand((channels, taps), torch.float32, 11, 0.5), rand((channels,), torch.float32, 12, 0.1)
    total = (taps - 1) * channels + inner * N
    states = rand((6, total), torch.float32, 13, 0.3)
    slots = torch.tensor([4, 0, 2, 5], dtype=torch.int32).cuda()
    query_start = torch.tensor(starts, dtype=torch.int32).cuda()
    conv = torch.empty((n, channels), dtype=torch.float32).cuda()
    states_c, conv_c = cpu(states), cpu(conv)
    plain_ops.causal_conv_silu(cpu(proj), inner, cpu(conv_w), cpu(conv_b), states_c, 0, cpu(slots), cpu(query_start), 150, conv_c)
    kernels.causal_conv_silu(proj, inner, conv_w, conv_b, states, 0, slots, query_start, 150, conv)
    assert torch.allclose(conv.cpu(), conv_c, atol=2e-5, rtol=2e-5)
    assert torch.allclose(states.cpu(), states_c, atol=1e-6)
    dt_bias, a_log, skip = rand((heads,), torch.float32, 14), rand((heads,), torch.float32, 15, 0.5) - 1.0, rand((heads,), torch.float32, 16)
    y = torch.empty((n, inner), dtype=torch.float32).cuda()
    y_c = cpu(y)
    offset = (taps - 1) * channels
    plain_ops.selective_scan(conv_c, cpu(proj), inner + channels, cpu(dt_bias), cpu(a_log), cpu(skip), states_c, offset, cpu(slots),
                             cpu(query_start), heads, P, N, G, y_c)
    kernels.selective_scan(conv, proj, inner + channels, dt_bias, a_log, skip, states, offset, slots, query_start, heads, P, N, G, y)
    scale = float(y_c.abs().max())
    assert torch.allclose(y.cpu(), y_c, atol=2e-5 * scale, rtol=2e-5)
    assert torch.allclose(states.cpu(), states_c, atol=2e-5 * float(states_c.abs().max()))
    assert torch.equal(states.cpu()[[1, 3]], rand((6, total), torch.float32, 13, 0.3).cpu()[[1, 3]])       # other slots untouched
    weight = 1 + rand((inner,), torch.float32, 17, 0.1)
    gated = torch.empty((n, inner), dtype=dtype).cuda()
    gated_c = cpu(gated)
    plain_ops.gated_group_norm(y_c, cpu(proj), 0, cpu(weight), parts, 1e-5, gated_c)
    kernels.gated_group_norm(y, proj, 0, weight, parts, 1e-5, gated)
    assert torch.allclose(gated.cpu().double(), gated_c.double(), **tol(dtype, 4.0))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("experts,identity,top,count,keep,width,inner,rows", [(10, 2, 3, 3, 2, 72, 24, 37), (3, 0, 1, 3, 1, 40, 9, 5),
                                                                              (2, 1, 3, 1, 1, 33, 20, 1), (12, 4, 2, 4, 1, 128, 32, 300),
                                                                              (60, 4, 6, 8, 3, 64, 16, 70)])
def test_grouped_router_and_clamped_experts(dtype, experts, identity, top, count, keep, width, inner, rows):
    """Router (scores over all outputs, correction for the choice, groups), routing with identity experts sorted behind the
    others, both products with the clamped gated activation in the first, and the weighted sum with a gated shared expert."""
    from miniserve_b200 import kernels

    total = experts + identity
    x = rand((rows, width), dtype, 20)
    router = rand((total + 1, width), torch.float32, 21, 0.4)
    correction = rand((total,), torch.float32, 22, 0.05) - 0.3
    ids, weights = torch.empty((rows, top), dtype=torch.int32).cuda(), torch.empty((rows, top), dtype=torch.float32).cuda()
    logits = torch.empty((rows, total + 1), dtype=torch.float32).cuda()
    ids_c, weights_c, logits_c = cpu(ids), cpu(weights), cpu(logits)
    plain_ops.router_topk(cpu(x), cpu(router), None, top, ids_c, weights_c, logits_c, choose_from=total, scoring="all_softmax",
                          correction=cpu(correction), groups=(count, keep))
    kernels.router_topk(x, router, None, top, ids, weights, logits, choose_from=total, scoring="all_softmax", correction=correction,
                        groups=(count, keep))
    assert torch.allclose(logits.cpu(), logits_c, atol=1e-4)
    same = (ids.cpu() == ids_c).all(dim=1)
    assert float(same.float().mean()) > 0.97                   # (a row may rest on a close call between two outputs)
    assert torch.allclose(weights.cpu()[same], weights_c[same], atol=1e-5)
    offsets, order = torch.empty(total + 1, dtype=torch.int32).cuda(), torch.empty(rows * top, dtype=torch.int32).cuda()
    place = torch.empty_like(order)
    kernels.expert_route(ids, total, offsets, order, place)
    up, down = rand((experts, 2 * inner, width), dtype, 23, 0.2), rand((experts, width, inner), dtype, 24, 0.2)
    hidden = torch.zeros((rows * top, inner), dtype=dtype).cuda()
    hidden_c = cpu(hidden)
    plain_ops.expert_linear(cpu(x), cpu(order), top, cpu(up), hidden_c, cpu(offsets), activation="clamped_glu", limit=0.7)
    kernels.expert_linear(x, order, top, up, hidden, offsets, activation="clamped_glu", limit=0.7)
    assert torch.allclose(hidden.cpu().double(), hidden_c.double(), **tol(dtype, 2.0))
    assert float(hidden_c.abs().max()) > 0.5                   # the limit is met
    results = torch.zeros((rows * top, width), dtype=dtype).cuda()
    results_c = cpu(results)
    plain_ops.expert_linear(hidden_c, None, top, cpu(down), results_c, cpu(offsets))
    kernels.expert_linear(hidden, None, top, down, results, offsets)
    assert torch.allclose(results.cpu().double(), results_c.double(), **tol(dtype, 2.0))
    shared = rand((rows, width), dtype, 25)
    out = torch.empty((rows, width), dtype=dtype).cuda()
    out_c = cpu(out)
    plain_ops.expert_combine(results_c, cpu(place), cpu(weights), cpu(shared), out_c, ids=cpu(ids), first_identity=experts, x=cpu(x),
                             shared_gate=logits_c, shared_gate_col=total)
    kernels.expert_combine(results, place, weights, shared, out, ids=ids, first_identity=experts, x=x, shared_gate=logits, shared_gate_col=total)
    assert torch.allclose(out.cpu().double(), out_c.double(), **tol(dtype, 3.0))
    both = rand((rows, 2 * inner), dtype, 26, 2.0)
    act = torch.empty((rows, inner), dtype=dtype).cuda()
    act_c = cpu(act)
    plain_ops.clamped_glu(cpu(both), 1.3, act_c)
    kernels.clamped_glu(both, 1.3, act)
    assert torch.allclose(act.cpu().double(), act_c.double(), **tol(dtype, 2.0))


def test_router_with_negative_choice_scores_and_ties():
    """All choice scores negative: a group that is not kept must not come back as a zero; equal outputs go to the lower index."""
    from miniserve_b200 import kernels

    x = torch.zeros((2, 8), dtype=torch.float32).cuda()
    x[0, 4], x[1, 0] = 1.0, 1.0
    router = torch.zeros((6, 8), dtype=torch.float32).cuda()
    router[:, :6] = 4 * torch.eye(6)
    correction = torch.tensor([-1.0, -1.0, -1.0, -1.2, -1.2, -1.2], dtype=torch.float32).cuda()
    ids, weights = torch.empty((2, 2), dtype=torch.int32).cuda(), torch.empty((2, 2), dtype=torch.float32).cuda()
    kernels.router_topk(x, router, None, 2, ids, weights, None, scoring="all_softmax", correction=correction, groups=(2, 1))
    assert ids.cpu().tolist() == [[4, 3], [0, 1]]
    scores = torch.softmax(x.cpu() @ router.cpu().T, dim=-1)
    assert torch.allclose(weights.cpu(), torch.gather(scores, 1, ids.cpu().long()), atol=1e-6)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n_q,n_kv,d,dv,page", [(8, 1, 64, 64, 16), (4, 2, 128, 128, 8), (6, 3, 32, 32, 16), (6, 3, 24, 40, 4), (16, 4, 128, 128, 64),
                                                 (6, 2, 48, 80, 16), (4, 2, 64, 32, 8), (8, 1, 96, 96, 16), (2, 2, 16, 128, 4), (4, 4, 112, 80, 16),
                                                 (34, 2, 48, 48, 16)])
@pytest.mark.parametrize("single", [False, True])
def test_attention_kernels_with_sink_and_gate(dtype, n_q, n_kv, d, dv, page, single):
    """``paged_attention`` with the sink and the gate over unequal requests: prompt portions that continue long contexts, or
    (``single``) one token per request over contexts of up to a few thousand keys, whose keys the tensor-core kernel cuts
    into ranges (the sink must be counted once, also where a range is empty).  Scores lie well below zero, so that the
    sink holds much of the weight; one key far back in every request stands out."""
    from miniserve_b200 import kernels

    contexts = [1, 70, 1500, 3000] if single else [40, 300, 129, 1000]
    new = [1, 1, 1, 1] if single else [40, 130, 2, 257]
    n_pages = sum((c + page - 1) // page for c in contexts)
    k_pool, v_pool = rand((n_pages + 1, n_kv, page, d), dtype, 40, 1.0), rand((n_pages + 1, n_kv, page, dv), dtype, 41, 1.0)
    width = max((c + page - 1) // page for c in contexts)
    tables = torch.full((len(contexts), width), n_pages, dtype=torch.int32)
    order = torch.randperm(n_pages, generator=torch.Generator().manual_seed(3)).int()
    at = 0
    for r, c in enumerate(contexts):
        count = (c + page - 1) // page
        tables[r, :count] = order[at:at + count]
        at += count
    starts = [0]
    for count in new:
        starts.append(starts[-1] + count)
    n = starts[-1]
    q = rand((n, n_q, d), dtype, 42, 1.0)
    q[..., 0] = 10.0
    k_pool[..., 0] = -10.0                      # every score gets -100 * scale: far below the sink's 0
    for r, c in enumerate(contexts):            # but one key far back in each request points the queries' way
        far = max(0, c - new[r] - 900) if c > 10 else 0
        k_pool[tables[r, far // page].long(), :, far % page, 0] = 0.5      # (its weight is of the sink's order)
    request_of = torch.cat([torch.full((count,), r, dtype=torch.int32) for r, count in enumerate(new)]).cuda()
    positions = torch.cat([torch.arange(c - count, c, dtype=torch.int32) for c, count in zip(contexts, new)]).cuda()
    gate = rand((n, n_q + 5), dtype, 43, 2.0)
    scale = 0.11
    out = torch.empty((n, n_q, dv), dtype=dtype).cuda()
    args = [torch.tensor(starts, dtype=torch.int32).cuda(), torch.tensor(contexts, dtype=torch.int32).cuda(), max(new), max(contexts), scale, None]
    kernels.paged_attention(q, k_pool, v_pool, tables.cuda(), request_of, positions, *args, out, starts, sink=True, gate=gate, gate_col=3)
    expected = cpu(out)
    plain_ops.paged_attention(cpu(q), cpu(k_pool), cpu(v_pool), tables, cpu(request_of), cpu(positions), *[cpu(a) if torch.is_tensor(a) else a for a in args],
                              expected, sink=True, gate=cpu(gate), gate_col=3)
    kernels.check_device_errors(q.device)
    assert torch.allclose(out.cpu().double(), expected.double(), **tol(dtype, float(expected.abs().max())))
    no_sink = cpu(out)
    plain_ops.paged_attention(cpu(q), cpu(k_pool), cpu(v_pool), tables, cpu(request_of), cpu(positions), *[cpu(a) if torch.is_tensor(a) else a for a in args],
                              no_sink, sink=False, gate=cpu(gate), gate_col=3)
    assert float((no_sink.double() - expected.double()).abs().max()) > 0.1 * float(expected.abs().max())     # the sink decides


# --------------------------------------------------------------------------- parts alone


def attention_weights(width, m, dtype, seed, own=True):
    shapes = {"q": (m["heads"] * m["dim"], width), "g": (m["heads"], width), "o": (width, m["heads"] * m["vdim"])}
    if own:
        shapes.update({"k": (m["kv_heads"] * m["dim"], width), "v": (m["kv_heads"] * m["vdim"], width)})
    w = {"x.mix." + name: rand(shape, dtype, seed + i, 0.12) for i, (name, shape) in enumerate(sorted(shapes.items()))}
    w["x.mix.q.norm"] = (1 + rand((m["dim"],), torch.float32, seed + 9, 0.1)).to(dtype)
    if own:
        w["x.mix.k.norm"] = (1 + rand((m["dim"],), torch.float32, seed + 10, 0.1)).to(dtype)
    return w


def build_attention(width, m, eps, own=True, window=None):
    from miniserve_b200.parts import MIXERS, PartSpec

    position = PartSpec("rope", dict(head_dim=m["dim"], theta=m["rot"]["base"], rotary_dim=m["rot"]["dims"], frequencies="float64"))
    return MIXERS.build(PartSpec("attention", dict(
        hidden_size=width, num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"], value_dim=m["vdim"], qk_norm=True, eps=eps,
        position=position, scale=m["scale"], sink=True, output_gate=True, own_kv=own, window=window, q_name="mix.q", k_name="mix.k",
        v_name="mix.v", o_name="mix.o", q_norm_name="mix.q.norm", k_norm_name="mix.k.norm", gate_name="mix.g")), prefix="x.")


ATTENTION_ALONE = [
    (88, zh.attn(6, 3, 24, 40, 0.23, 16, 5000.0)["mixer"]),
    (72, zh.attn(1, 1, 12, 10, 0.4, 6, 100.0)["mixer"]),
    (64, zh.attn(8, 1, 64, 64, 0.125, 64, 1000000.0)["mixer"]),
    (96, zh.attn(4, 2, 128, 32, 0.09, 64, 10000.0)["mixer"]),
    (80, zh.attn(8, 2, 48, 80, 0.14, 32, 250000.0)["mixer"]),
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", range(len(ATTENTION_ALONE)))
@pytest.mark.parametrize("window", [None, 23])
def test_attention_part_far_keys_sink_and_borrowed_keys(dtype, case, window):
    """The mixer alone, fed in portions and then token by token through a paged cache, and a second mixer without keys of
    its own that reads the first one's pages.  Inputs are made so that faults show: one token far back (and the tokens just
    inside and just outside a window's edge) carries a loud key; a constant input column that queries and keys read with
    opposite signs pushes all other scores far below zero, so that the sink holds most of the softmax's weight and leaving
    it out changes every row."""
    width, m = ATTENTION_ALONE[case]
    lender, borrower = build_attention(width, m, 1e-5, True, window), build_attention(width, m, 1e-5, False, window)
    assert lender.cache_need() == borrower.cache_need()
    w, w2 = attention_weights(width, m, dtype, 30), attention_weights(width, m, dtype, 60, own=False)
    dim = m["dim"]
    for weights, names in ((w, ("x.mix.q", "x.mix.k")), (w2, ("x.mix.q",))):
        for name in names:
            rows = weights[name].view(-1, dim, width)
            rows[:, dim - 2:, 0] = 8.0 if name.endswith("q") else -8.0        # (a head's last two entries are not rotated, or hardly)
    assert sorted(s.name for s in lender.param_specs()) == sorted(w) and sorted(s.name for s in borrower.param_specs()) == sorted(w2)
    lender.load(w)
    borrower.load(w2)
    total = 333
    x = rand((total, width), dtype, 50)
    x[:, 0] = 1.0
    loud = {5: 6.0, 250: 3.0} if window is None else {total - 40 - window: 6.0, total - 40 - window + 1: 3.0,
                                                      total - 3 - window: 6.0, total - 3 - window + 1: 3.0}
    for token, factor in loud.items():
        x[token, 0] = -factor            # this token's keys point the queries' way
    harness = Harness([lender.cache_need()], dtype, page_size=8, num_pages=64, max_len=512)
    cuts = [(0, 3), (3, 5), (5, 130), (130, 131), (131, 290)] + [(i, i + 1) for i in range(290, total)]
    got, got2 = [], []
    for start, end in cuts:
        ctx = harness.context({"r": end - start})
        ctx.dtype = dtype
        view = harness.view(ctx)
        got.append(lender.forward(x[start:end].contiguous(), ctx, view).clone())
        view.writable = False
        got2.append(borrower.forward(x[start:end].contiguous(), ctx, view).clone())
    xd = x.double().cpu()
    positions = torch.arange(total)
    wd, wd2 = {k: v.double().cpu() for k, v in w.items()}, {k: v.double().cpu() for k, v in w2.items()}
    keys, values = plain.attention_keys_values(xd, wd, "x.", m, 1e-5, positions)
    expected = plain.attention(xd, wd, "x.", m, 1e-5, positions, keys, values, window)
    expected2 = plain.attention(xd, wd2, "x.", m, 1e-5, positions, keys, values, window)
    # with no loud key in sight the sink holds a good part of the weight and the rows are small; a loud key takes it all
    quiet = xd.clone()
    quiet[:, 0] = 1.0
    keys_q, values_q = plain.attention_keys_values(quiet, wd, "x.", m, 1e-5, positions)
    expected_quiet = plain.attention(quiet, wd, "x.", m, 1e-5, positions, keys_q, values_q, window)
    assert float(expected_quiet[-40:].abs().max()) < 0.2 * float(expected[-40:].abs().max())       # quiet rows: the sink holds the weight
    assert torch.allclose(torch.cat(got).double().cpu(), expected, **tol(dtype, float(expected.abs().max())))
    assert torch.allclose(torch.cat(got2).double().cpu(), expected2, **tol(dtype, float(expected2.abs().max())))


def state_space_weights(width, m, dtype, seed):
    inner = m["heads"] * m["vdim"]
    channels = inner + 2 * m["groups"] * m["state"]
    w = {"x.mix.in": rand((2 * inner + 2 * m["groups"] * m["state"] + m["heads"], width), dtype, seed, 0.2),
         "x.mix.conv": rand((channels, m["conv"]), dtype, seed + 1, 0.4), "x.mix.conv.b": rand((channels,), dtype, seed + 2, 0.1),
         "x.mix.dt_bias": rand((m["heads"],), dtype, seed + 3, 0.5), "x.mix.A_log": (rand((m["heads"],), torch.float32, seed + 4, 0.3) - 2.0).to(dtype),
         "x.mix.D": rand((m["heads"],), dtype, seed + 5), "x.mix.norm": (1 + rand((inner,), torch.float32, seed + 6, 0.1)).to(dtype),
         "x.mix.o": rand((width, inner), dtype, seed + 7, 0.15)}
    return w


STATE_SPACE_ALONE = [
    (88, zh.ssm(6, 12, 20, 3, 4, 2)["mixer"]),
    (72, zh.ssm(1, 20, 6, 1, 1, 1)["mixer"]),
    (40, zh.ssm(3, 6, 36, 3, 5, 3)["mixer"]),
    (64, zh.ssm(4, 32, 128, 1, 4, 1)["mixer"]),
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", range(len(STATE_SPACE_ALONE)))
def test_state_space_part_in_portions_and_slots_used_again(dtype, case):
    """The mixer alone: a sequence in portions (down to one and two tokens, shorter than the convolution reaches) and then
    token by token, beside a second request in the same steps; then a third request in the slot the first one gave back,
    which must start from nothing.  Decays near one make the state remember hundreds of tokens, so a state that is lost,
    mixed up between slots or not cleared shows at once."""
    from miniserve_b200.parts import MIXERS, PartSpec

    width, m = STATE_SPACE_ALONE[case]
    part = MIXERS.build(PartSpec("state_space", dict(
        hidden_size=width, heads=m["heads"], head_dim=m["vdim"], state=m["state"], groups=m["groups"], taps=m["conv"],
        norm_groups=m["norm_groups"], eps=1e-5, in_name="mix.in", conv_name="mix.conv", conv_bias_name="mix.conv.b",
        dt_bias_name="mix.dt_bias", a_log_name="mix.A_log", d_name="mix.D", norm_name="mix.norm", o_name="mix.o")), prefix="x.")
    w = state_space_weights(width, m, dtype, 70)
    assert sorted(s.name for s in part.param_specs()) == sorted(w)
    part.load(w)
    wd = {k: v.double().cpu() for k, v in w.items()}
    harness = Harness([part.cache_need()], dtype, page_size=8, num_pages=8, max_seqs=2, max_len=512)
    first, second, third = rand((200, width), dtype, 80), rand((131, width), dtype, 81), rand((40, width), dtype, 82)
    cuts = [0, 1, 3, 5, 70, 72, 150] + list(range(151, 201))
    got_first, got_second, at = [], [], 0
    for start, end in zip(cuts[:-1], cuts[1:]):
        portions = {"a": end - start}
        take = min(len(second) - at, 1 if end - start > 20 else 17) if at < len(second) else 0
        if take:
            portions["b"] = take
        ctx = harness.context(portions)
        ctx.dtype = dtype
        batch = torch.cat([first[start:end]] + ([second[at:at + take]] if take else []))
        out = part.forward(batch.contiguous(), ctx, harness.view(ctx))
        got_first.append(out[:end - start].clone())
        if take:
            got_second.append(out[end - start:].clone())
            at += take
    expected = plain.state_space(first.double().cpu(), wd, "x.", m, 1e-5)
    scale = float(expected.abs().max())
    assert torch.allclose(torch.cat(got_first).double().cpu(), expected, **tol(dtype, scale))
    expected_second = plain.state_space(second.double().cpu()[:at], wd, "x.", m, 1e-5)
    assert torch.allclose(torch.cat(got_second).double().cpu(), expected_second, **tol(dtype, scale))
    # the state matters: without what the first 150 tokens left, the last rows would be others
    fresh = plain.state_space(first.double().cpu()[150:], wd, "x.", m, 1e-5)
    assert float((fresh[:3] - expected[150:153]).abs().max()) > 0.02 * scale
    slot = harness.manager.requests["a"].slot
    harness.manager.release("a")
    ctx = harness.context({"c": len(third)})
    ctx.dtype = dtype
    assert harness.manager.requests["c"].slot == slot
    out = part.forward(third, ctx, harness.view(ctx))
    assert torch.allclose(out.double().cpu(), plain.state_space(third.double().cpu(), wd, "x.", m, 1e-5), **tol(dtype, scale))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,index", [("a", 0), ("a", 2), ("a", 3), ("b", 0), ("b", 1), ("b", 3), ("c", 1)])
def test_mixture_part(dtype, name, index):
    from miniserve_b200.parts import FEED_FORWARDS, PagedKVNeed, PartSpec

    mlp, width = zh.CONFIGS[name]["layers"][index]["mlp"], zh.CONFIGS[name]["width"]
    router = mlp["router"]
    shared = mlp["shared"]
    part = FEED_FORWARDS.build(PartSpec("routed_experts", dict(
        hidden_size=width, experts=router["experts"], top=router["top"], expert_size=mlp["expert"]["ff"],
        shared_size=shared["ff"] if shared else None, router_bias=False, activation="clamped_glu", limit=mlp["expert"]["limit"],
        shared_limit=shared["limit"] if shared else None, identity=router["identity"], scoring="all_softmax",
        correction_name="mlp.correction", groups=(router["groups"]["count"], router["groups"]["keep"]),
        shared_gate_name="mlp.shared.sg", router_name="mlp.router", expert_name="mlp.e{index}.", shared_name="mlp.shared.")), prefix="f.")
    total = router["experts"] + router["identity"]
    w = {"f.mlp.router": rand((total, width), dtype, 60, 0.6), "f.mlp.correction": (rand((total,), torch.float32, 61, 0.05) - 0.2).to(dtype)}
    for e in range(router["experts"]):
        for i, (piece, shape) in enumerate((("gate", (mlp["expert"]["ff"], width)), ("up", (mlp["expert"]["ff"], width)), ("down", (width, mlp["expert"]["ff"])))):
            w[f"f.mlp.e{e}.{piece}"] = rand(shape, dtype, 100 + 3 * e + i, 0.3)
    if shared:
        w.update({"f.mlp.shared.gate": rand((shared["ff"], width), dtype, 90, 0.3), "f.mlp.shared.up": rand((shared["ff"], width), dtype, 91, 0.3),
                  "f.mlp.shared.down": rand((width, shared["ff"]), dtype, 92, 0.3), "f.mlp.shared.sg": rand((1, width), dtype, 93, 0.3)})
    assert sorted(s.name for s in part.param_specs()) == sorted(w)
    part.load(w)
    rows = 150
    x = rand((rows, width), dtype, 99)
    wd = {k: v.double().cpu() for k, v in w.items()}
    expected = plain.mixture(x.double().cpu(), wd, "f.", mlp)
    # rows whose routing is a close call in this number format are left out (the plain scores decide which)
    threshold = 1e-5 if dtype == torch.float32 else 4e-3
    clear = torch.tensor([plain.route(x.double().cpu()[i:i + 1], wd, "f.", mlp)[2] > threshold for i in range(rows)])
    out = part.forward(x, Harness([PagedKVNeed(1, 16, None)], dtype, num_pages=128, max_len=512).context({"a": rows}))
    assert int(clear.sum()) >= rows // 2
    assert torch.allclose(out.double().cpu()[clear], expected[clear], **tol(dtype, float(expected.abs().max())))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("with_feed_forward", [True, False])
def test_sandwich_block(dtype, with_feed_forward):
    """Two blocks in a row and the last norm on gathered rows: every sublayer's output passes its own norm on the way into
    the float32 stream.  The sublayers are a state-space mixer and a plain gated feed-forward."""
    from miniserve_b200.parts import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, PartSpec

    width, m = 88, zh.ssm(6, 12, 20, 3, 4, 2)["mixer"]
    blocks, weights = [], []
    for b in range(2):
        prefix = f"b{b}."
        mixer = MIXERS.build(PartSpec("state_space", dict(
            hidden_size=width, heads=m["heads"], head_dim=m["vdim"], state=m["state"], groups=m["groups"], taps=m["conv"],
            norm_groups=m["norm_groups"], eps=1e-5, in_name="mix.in", conv_name="mix.conv", conv_bias_name="mix.conv.b",
            dt_bias_name="mix.dt_bias", a_log_name="mix.A_log", d_name="mix.D", norm_name="mix.norm", o_name="mix.o")), prefix=prefix)
        w = {prefix + k[2:]: v for k, v in state_space_weights(width, m, dtype, 200 + 20 * b).items()}
        norms = {}
        for name in ("norm1", "norm1b", "norm2", "norm2b"):
            if with_feed_forward or name.startswith("norm1"):
                norms[name] = NORMS.build(PartSpec("rms", dict(name=name, size=width, eps=1e-5, one_plus=True)), prefix=prefix)
                w[prefix + name] = rand((width,), dtype, 210 + 20 * b + len(norms), 0.2)
        feed_forward = None
        if with_feed_forward:
            feed_forward = FEED_FORWARDS.build(PartSpec("gated_mlp", dict(hidden_size=width, intermediate_size=48, gate_name="gate", up_name="up",
                                                                          down_name="down")), prefix=prefix)
            w.update({prefix + "gate": rand((48, width), dtype, 230 + b, 0.2), prefix + "up": rand((48, width), dtype, 232 + b, 0.2),
                      prefix + "down": rand((width, 48), dtype, 234 + b, 0.2)})
        block = BLOCKS.build(PartSpec("sandwich"), mixer=mixer, feed_forward=feed_forward, mixer_norm=norms["norm1"],
                             feed_forward_norm=norms.get("norm2"), mixer_post_norm=norms["norm1b"], feed_forward_post_norm=norms.get("norm2b"))
        for part in block.parts():
            part.load({s.name: w[s.name] for s in part.param_specs()})
        blocks.append(block)
        weights.append({k: v.double().cpu() for k, v in w.items()})
    final = NORMS.build(PartSpec("rms", dict(name="final", size=width, eps=1e-5, one_plus=True)))
    final_weight = rand((width,), dtype, 300, 0.2)
    final.load({"final": final_weight})
    rows = 21
    stream = rand((rows, width), torch.float32, 301)
    x = stream.double().cpu()
    harness = Harness([blocks[0].mixer.cache_need()] * 1, dtype, max_len=64)
    # (two mixers with states of the same form: each block gets a harness of its own, so that each has its state)
    harness2 = Harness([blocks[1].mixer.cache_need()] * 1, dtype, max_len=64)
    pending = None
    for block, wd, h in zip(blocks, weights, (harness, harness2)):
        ctx = h.context({"r": rows})
        ctx.dtype = dtype
        pending = block.forward(stream, pending, ctx, h.view(ctx))
        prefix = [k for k in wd if k.endswith("norm1")][0][:-5]
        hidden = plain.norm_one_plus(x, wd[prefix + "norm1"], 1e-5)
        mixed = plain.state_space(hidden, {"x." + k[len(prefix):]: v for k, v in wd.items()}, "x.", m, 1e-5)
        x = x + plain.norm_one_plus(mixed, wd[prefix + "norm1b"], 1e-5)
        if with_feed_forward:
            hidden = plain.norm_one_plus(x, wd[prefix + "norm2"], 1e-5)
            inner = (hidden @ wd[prefix + "gate"].T)
            out = (inner * torch.sigmoid(inner) * (hidden @ wd[prefix + "up"].T)) @ wd[prefix + "down"].T
            x = x + plain.norm_one_plus(out, wd[prefix + "norm2b"], 1e-5)
    picked = torch.tensor([20, 3], dtype=torch.int32).cuda()
    out = torch.empty((2, width), dtype=dtype).cuda()
    final.add_and_norm(stream, pending, out, rows=picked)
    expected = plain.norm_one_plus(x, final_weight.double().cpu(), 1e-5)[[20, 3]]
    assert torch.allclose(out.double().cpu(), expected, **tol(dtype, float(expected.abs().max())))


# --------------------------------------------------------------------------- the whole model through the engine


def build(folder, dtype, num_pages, page_size, max_seqs=4, execution="eager"):
    import miniserve_b200  # noqa: F401
    from miniserve_b200.config import EngineConfig
    from miniserve_b200.engine.runtime import build_runtime

    return build_runtime(folder, EngineConfig(dtype=dtype, kv_block_size=page_size, num_kv_blocks=num_pages, max_num_seqs=max_seqs,
                                              enable_prefix_cache=False, decode_execution=execution))


def replay(runtime, steps):
    from miniserve_b200 import kernels
    from miniserve_b200.trace import TraceSession

    session, outputs = TraceSession(runtime), {}
    for record in steps:
        logits = session.run(record)
        if logits is not None:
            outputs[record["step"]] = logits.double().cpu()
    kernels.check_device_errors(runtime.step_function.device)
    runtime.manager.check_invariants()
    return outputs


_ORACLE: dict = {}


def oracle(folder, tokens):
    key = (str(folder), tuple(tokens))
    if key not in _ORACLE:
        config, weights = plain.load_folder(folder)
        _ORACLE[key] = plain.forward(tokens, weights, config)
    return _ORACLE[key]


def check(folder, dtype, requests, got, positions_of=None):
    worst = 0.0
    for rid, tokens in requests.items():
        expected = oracle(folder, tokens)
        bound = bound_of(dtype, expected)
        wanted = sorted(got[rid]) if positions_of is None else positions_of[rid]
        assert sorted(got[rid]) == list(wanted), rid
        for position, row in got[rid].items():
            error = float((row - expected[position]).abs().max())
            worst = max(worst, error / bound)
            assert error <= bound, (rid, position, error, bound)
    return worst


CUTTINGS = {
    "whole": helpers.cut_whole,
    "tail": lambda r: helpers.cut_decode_tail(r, 32),
    "portions": lambda r: helpers.cut_portions(r, seed=3),
    "mixed": lambda r: helpers.cut_mixed(r, seed=4),
}
# lengths at the borders of pages of 8 and 16 tokens and of the kernels' chunks of 16 and 64, a single token, a few hundred
LENGTHS = (1, 7, 8, 9, 16, 17, 33, 64, 65, 150, 301)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,page_size", [("a", 8), ("b", 16), ("c", 16), ("b", 4), ("d", 8)])
@pytest.mark.parametrize("cutting", list(CUTTINGS))
def test_cuttings_against_plain(tmp_path, request, dtype, name, page_size, cutting):
    """Whole prompts; last tokens decoded one by one; portions down to two tokens; unequal requests batched together in a
    pool so small that pages and slots are used again: always the logits of the plain whole-sequence computation."""
    folder = zh.make_folder(tmp_path, name, seed=11)
    vocab = zh.CONFIGS[name]["vocab"]
    requests = {f"r{i}": helpers.random_tokens(vocab, n, seed=400 + i) for i, n in enumerate(LENGTHS)}
    steps = CUTTINGS[cutting](requests)
    granule = max(64, page_size)
    runtime = build(folder, dtype, helpers.max_live_tokens(steps, granule=granule) // page_size, page_size)
    got = helpers.collect(steps, replay(runtime, steps))
    worst = check(folder, dtype, requests, got)
    helpers.note_ratio(request.node.name, worst)
    assert not runtime.manager.requests and all(a.free_count == a.num_pages for a in runtime.manager.allocators)


@pytest.mark.parametrize("name,page_size", [("a", 8), ("c", 16)])
def test_float32_logits_do_not_depend_on_cutting_or_batch(tmp_path, name, page_size):
    """In float32 every sum has an order that depends on the position alone (products with one thread per element, keys in
    blocks from absolute key 0, the recurrence token by token, routed rows computed independently), so a request alone and
    whole, in portions, and batched with others on other pages and in other slots must give the same logits to the last
    bit or two."""
    folder = zh.make_folder(tmp_path, name, seed=16)
    vocab = zh.CONFIGS[name]["vocab"]
    requests = {f"r{i}": helpers.random_tokens(vocab, n, seed=900 + i) for i, n in enumerate((1, 9, 33, 64, 65, 150))}
    results = {}
    for cutting in ("whole", "portions", "mixed"):
        steps = CUTTINGS[cutting](requests)
        runtime = build(folder, "float32", helpers.max_live_tokens(steps, granule=64) // page_size, page_size)
        results[cutting] = helpers.collect(steps, replay(runtime, steps))
    for rid, tokens in requests.items():
        for position in range(len(tokens)):
            alone = results["whole"][rid][position]
            scale = max(1.0, float(alone.abs().max()))
            for cutting in ("portions", "mixed"):
                assert float((results[cutting][rid][position] - alone).abs().max()) <= 2e-6 * scale, (rid, position, cutting)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "c", "d"])
def test_prefill_against_decoding_every_token(tmp_path, dtype, name):
    """The same sequence as one prompt and token by token from its first token on (a long decode over several pages, the
    state carried through every step): the two agree with the plain logits and so, within rounding, with each other."""
    folder = zh.make_folder(tmp_path, name, seed=12)
    tokens = helpers.random_tokens(zh.CONFIGS[name]["vocab"], 140, seed=500)
    runtime = build(folder, dtype, 40, 8)
    whole = replay(runtime, helpers.cut_whole({"w": tokens}))[0]
    steps = helpers.cut_decode_tail({"d": tokens}, tail=len(tokens))
    single = helpers.collect(steps, replay(runtime, steps))["d"]
    expected = oracle(folder, tokens)
    bound = bound_of(dtype, expected)
    for position in range(len(tokens)):
        assert float((whole[position] - expected[position]).abs().max()) <= bound
        assert float((single[position] - expected[position]).abs().max()) <= bound
        assert float((single[position] - whole[position]).abs().max()) <= bound


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("execution", ["eager", "cuda_graph"])
def test_many_live_requests_decoding(tmp_path, dtype, execution):
    """Seven requests live at once, decoded in steps of single tokens whose live set changes (captured graphs with padding
    rows when graphs are on: the recurrence, the borrowed keys and the routed experts inside a replayed step)."""
    folder = zh.make_folder(tmp_path, "c", seed=13)
    vocab = zh.CONFIGS["c"]["vocab"]
    prompt_lens = {f"m{i}": n for i, n in enumerate((3, 1, 17, 40, 9, 64, 25))}
    requests = {rid: helpers.random_tokens(vocab, n + 11, seed=600 + i) for i, (rid, n) in enumerate(prompt_lens.items())}
    steps = helpers.cut_many_live(requests, prompt_lens, seed=2)
    runtime = build(folder, dtype, 7 * 6, 16, max_seqs=7, execution=execution)
    got = helpers.collect(steps, replay(runtime, steps))
    if execution == "cuda_graph":
        assert runtime.step_function.graph_replays > 0
    check(folder, dtype, requests, got, {rid: range(prompt_lens[rid] - 1, len(requests[rid])) for rid in requests})


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("execution", ["eager", "cuda_graph"])
def test_greedy_generation_through_the_scheduler(tmp_path, dtype, execution):
    """``LLM.generate``: the engine's own entry point, scheduler (chunked prompts, a token budget that forces portions, more
    prompts than state slots) and sampler; every generated token is the plain implementation's choice, or as good as it
    within rounding."""
    from miniserve_b200.engine.llm import LLM
    from miniserve_b200.sampling import SamplingParams

    folder = zh.make_folder(tmp_path, "a", seed=14)
    config, weights = plain.load_folder(folder)
    prompts = [helpers.random_tokens(config["vocab"], n, seed=700 + n) for n in (1, 5, 30, 77)]
    llm = LLM(str(folder), dtype=dtype, kv_block_size=8, num_kv_blocks=48, max_num_seqs=3, max_num_batched_tokens=24,
              decode_execution=execution)
    results = llm.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=12))
    for prompt, result in zip(prompts, results):
        assert len(result.token_ids) == 12
        tokens = list(prompt)
        for produced in result.token_ids:
            logits = plain.forward(tokens, weights, config)[-1]
            best = int(torch.argmax(logits))
            if produced != best:
                assert float(logits[best] - logits[produced]) <= 2 * bound_of(dtype, logits), (produced, best)
            tokens.append(produced)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program_and_command_line(tmp_path, dtype):
    """``bin/trace_run`` and ``python -m miniserve_b200.generate`` on a Zozezen folder, as a user runs them."""
    folder = zh.make_folder(tmp_path, "b", seed=15)
    vocab = zh.CONFIGS["b"]["vocab"]
    requests = {f"q{i}": helpers.random_tokens(vocab, n, seed=800 + i) for i, n in enumerate((2, 19, 70, 45, 33))}
    steps = helpers.cut_mixed(requests, seed=6)
    out_dir = tmp_path / "out"
    process = subprocess.run([sys.executable, str(REPO / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype, "--out", str(out_dir),
                              "--max-tokens", str(helpers.max_live_tokens(steps, granule=64))],
                             input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert process.returncode == 0, process.stderr[-2000:]
    assert [line for line in process.stdout.splitlines() if line.startswith("done")] == [f"done {s['step']}" for s in steps]
    outputs = {s["step"]: torch.from_numpy(np.fromfile(out_dir / f"{s['step']}.f32", dtype="<f4").reshape(-1, vocab)).double()
               for s in steps}
    check(folder, dtype, requests, helpers.collect(steps, outputs))
    generated = subprocess.run([sys.executable, "-m", "miniserve_b200.generate", "--model", str(folder), "--dtype", dtype,
                                "--prompt-ids", ",".join(map(str, requests["q1"])), "--max-new-tokens", "5", "--num-kv-blocks", "32",
                                "--kv-block-size", "8", "--json"], capture_output=True, text=True, timeout=600, cwd=str(REPO))
    assert generated.returncode == 0, generated.stderr[-2000:]
    produced = json.loads(generated.stdout.strip().splitlines()[-1])["token_ids"]
    assert len(produced) == 5
    tokens = list(requests["q1"])
    for token in produced:
        logits = oracle(folder, tokens)[-1]
        best = int(torch.argmax(logits))
        assert token == best or float(logits[best] - logits[token]) <= 2 * bound_of(dtype, logits)
        tokens.append(token)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width", [40, 44])
def test_odd_heads_no_rotation_and_norms_that_nothing_reads(tmp_path, dtype, width):
    """An odd head size without any rotation, a width that is no multiple of eight, and a checkpoint that carries feed-forward
    norms for a layer that has no feed-forward (the loader lets them be), in portions and in a mixed batch."""
    from safetensors.torch import save_file

    from miniserve_b200.weights import random_tensors

    config = dict(architecture="Zozezen", vocab=61, width=width, norm=dict(eps=1e-5), layers=[
        zh.layer(zh.attn(3, 1, 7, 5, 0.3, 0), None),
        zh.layer(zh.ssm(2, 9, 5, 2, 3, 3), zh.moe(2, 2, 2, 6, 0.9, 2, 2, 10, 1.1)),
        zh.layer(zh.attn(2, 1, 7, 5, 0.6, 0, kv_from=0), zh.moe(3, 0, 2, 6, 0.9, 1, 1, None)),
    ])
    tensors = random_tensors(config, 5, "bfloat16", 0.1)
    zh.steer_routers(tensors, config)
    tensors["l0.norm2"], tensors["l0.norm2b"] = torch.zeros(width, dtype=torch.bfloat16), torch.zeros(width, dtype=torch.bfloat16)
    folder = tmp_path / "odd"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(config))
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(folder / "model.safetensors"))
    requests = {f"r{i}": helpers.random_tokens(61, n, seed=30 + i) for i, n in enumerate((1, 19, 40, 9))}
    for cutting in ("portions", "mixed"):
        steps = CUTTINGS[cutting](requests)
        runtime = build(folder, dtype, helpers.max_live_tokens(steps, granule=64) // 4, 4)
        check(folder, dtype, requests, helpers.collect(steps, replay(runtime, steps)))


def test_which_attention_kernels_a_build_reports(tmp_path):
    """bfloat16: heads of 64 and 128 with values of the same size on the unrolled tensor-core kernels; heads of 48 with values
    of 80 (and 112 with 16) on the tensor-core kernel for any multiple of 16; sizes that are no multiples of 16 on the general
    kernel, as everything in float32."""
    expected = {"c": [("tcgen05", "mma.sync"), ("tcgen05", "mma.sync")],
                "d": [("mma.sync (any size)", "mma.sync (any size)"), ("mma.sync (any size)", "mma.sync (any size)")],
                "b": [("general", "general"), ("general", "general")]}
    for name, kinds in expected.items():
        folder = zh.make_folder(tmp_path, name, seed=17)
        runtime = build(folder, "bfloat16", 16, 16)
        assert [(k["prompt"], k["decode"]) for k in runtime.attention_kernels] == kinds, name
        runtime = build(folder, "float32", 16, 16)
        assert all(k["prompt"] == k["decode"] == "general" for k in runtime.attention_kernels)
