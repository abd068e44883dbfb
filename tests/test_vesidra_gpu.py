"""Vesidra on the GPU against the plain implementation (``plain_vesidra``): every new kernel alone, every new part
alone (also fed in portions through the cache, with keys that stand out far back and at a window's edges), and the
whole model through the engine's own session, scheduler and command line, in float32 and bfloat16, at sizes of its own."""

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
import plain_vesidra as plain
import vesidra_helpers as vh
from test_parts_gpu import Harness, rand, tol

pytestmark = pytest.mark.gpu
REPO = Path(__file__).resolve().parent.parent
DTYPES = [torch.float32, torch.bfloat16]


def bound_of(dtype, expected):
    # (seen on B200: at most 0.13 of the float32 bound and 0.23 of the bfloat16 bound)
    return (8e-6 if dtype in ("float32", torch.float32) else 1e-2) * max(1.0, float(expected.abs().max()))


# --------------------------------------------------------------------------- kernels alone


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("size", [40, 136, 1000])
def test_add_norm_with_two_outputs(dtype, size):
    from miniserve_b200 import kernels

    weight = (1 + rand((size,), torch.float32, 1, 0.2)).to(dtype)
    residual, first, second = rand((6, size), torch.float32, 2, 2.0), rand((6, size), dtype, 3), rand((6, size), dtype, 4)
    expected_sum = residual.double() + (first.double() + second.double())
    out = torch.empty((6, size), dtype=dtype).cuda()
    kernels.add_rmsnorm(residual, first, weight, 1e-5, out, None, second)
    assert torch.allclose(residual.double(), expected_sum, atol=2e-6)
    expected = plain.rms_norm(expected_sum, weight.double(), 1e-5)
    assert torch.allclose(out.double(), expected, **tol(dtype, 3.0))
    rows = torch.tensor([4, 0], dtype=torch.int32).cuda()
    before = residual.clone()
    gathered = torch.empty((2, size), dtype=dtype).cuda()
    kernels.add_rmsnorm(residual, first, weight, 1e-5, gathered, rows, second)
    assert torch.equal(residual, before)                                   # gathered rows leave the stream alone
    again = plain.rms_norm((before.double() + (first.double() + second.double()))[rows.long()], weight.double(), 1e-5)
    assert torch.allclose(gathered.double(), again, **tol(dtype, 3.0))


def test_rotation_table_with_magnitude():
    from miniserve_b200 import kernels

    positions = torch.tensor([0, 1, 63, 64, 1000, 70000], dtype=torch.int32).cuda()
    freqs, magnitude = plain.rotary_frequencies(dict(base=5000.0, dims=16, scaling=vh.YARN_B))
    table = torch.empty((6, 8, 2), dtype=torch.float32).cuda()
    kernels.rope_table(positions, freqs.float().cuda(), table, magnitude)
    angles = positions.cpu().float()[:, None].double() * freqs.float().double()[None, :]
    assert torch.allclose(table[..., 0].double().cpu(), magnitude * angles.cos(), atol=1e-5 + 70000 * 1e-7)
    assert torch.allclose(table[..., 1].double().cpu(), magnitude * angles.sin(), atol=1e-5 + 70000 * 1e-7)
    assert magnitude > 1.1


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,dim,rot,rank,rot_dims", [(3, 24, 16, 40, 8), (1, 12, 6, 22, 6), (8, 32, 32, 64, 32), (2, 5, 0, 9, 0)])
def test_latent_prepare(dtype, heads, dim, rot, rank, rot_dims):
    from miniserve_b200 import kernels

    n, page = 11, 4
    ld = (heads * (dim + rot) + rank + rot + heads + 7) // 8 * 8
    proj = rand((n, ld), dtype, 5)
    weight = (1 + rand((rank,), torch.float32, 6, 0.2)).to(dtype)
    positions = torch.tensor([0, 1, 2, 3, 40, 41, 42, 43, 44, 500, 501], dtype=torch.int32).cuda()
    table = None
    if rot_dims:
        freqs, magnitude = plain.rotary_frequencies(dict(base=300.0, dims=rot_dims, scaling=vh.YARN_A))
        table = torch.empty((n, rot_dims // 2, 2), dtype=torch.float32).cuda()
        kernels.rope_table(positions, freqs.float().cuda(), table, magnitude)
    slots = torch.tensor([3, 2, 1, 0, 8, 9, 10, 11, -1, 20, 21], dtype=torch.int32).cuda()
    cache, q_full = torch.zeros((6, page, rank + rot), dtype=dtype).cuda(), torch.zeros((n, heads, rank + rot), dtype=dtype).cuda()
    kernels.latent_prepare(proj, 0, heads * (dim + rot), heads, dim, rot, rank, slots, weight, 1e-5, table, rot_dims, cache, q_full)
    want_cache, want_q = torch.zeros_like(cache, dtype=torch.float64), torch.zeros_like(q_full, dtype=torch.float64)
    plain_ops.latent_prepare(proj, 0, heads * (dim + rot), heads, dim, rot, rank, slots, weight, 1e-5, table, rot_dims, want_cache, want_q)
    assert torch.allclose(cache.double(), want_cache, **tol(dtype, 3.0))
    assert torch.allclose(q_full.double(), want_q, **tol(dtype, 3.0))
    assert float(q_full[:, :, :rank].abs().max()) == 0 and float(cache.view(-1, rank + rot)[4:8].abs().max()) == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,rank,rot,page,window", [(3, 40, 16, 4, None), (1, 22, 6, 8, None), (8, 64, 16, 16, None),
                                                        (16, 96, 32, 8, 21), (5, 128, 64, 16, None), (2, 9, 0, 4, 7),
                                                        (20, 256, 32, 16, None), (16, 512, 64, 8, 40), (6, 128, 0, 4, None)])
@pytest.mark.parametrize("single", [False, True])
def test_latent_attention_kernel(dtype, heads, rank, rot, page, window, single):
    """Prompt portions beside single tokens (or single tokens only, as a decode step has them: the keys are then cut
    into ranges that a second kernel merges) over a paged cache of latent rows, against the plain statement.  The sizes
    cover the tensor-core kernel's (bfloat16; latent 64, 96, 128, 256, 512 with a rotated part that is a multiple of 16)
    and others, which run the general kernel."""
    from miniserve_b200 import kernels

    dk = rank + rot
    lens = [70, 33, 1, 130]                                   # context lengths, and how many of their tokens are new
    news = [1, 1, 1, 1] if single else [70, 1, 1, 9]
    pages_of, tables, next_page = [], [], 0
    order = torch.randperm(64, generator=torch.Generator().manual_seed(7)).tolist()
    width = max((l + page - 1) // page for l in lens)
    for l in lens:
        count = (l + page - 1) // page
        tables.append(order[next_page:next_page + count] + [0] * (width - count))
        next_page += count
    cache = rand((64, page, dk), dtype, 8)
    request_of, positions, starts = [], [], [0]
    for r, (l, new) in enumerate(zip(lens, news)):
        request_of += [r] * new
        positions += list(range(l - new, l))
        starts.append(starts[-1] + new)
    n = len(positions)
    q = rand((n, heads, dk), dtype, 9, 0.5)
    args = [torch.tensor(tables, dtype=torch.int32).cuda(), torch.tensor(request_of, dtype=torch.int32).cuda(),
            torch.tensor(positions, dtype=torch.int32).cuda(), torch.tensor(starts, dtype=torch.int32).cuda(),
            torch.tensor(lens, dtype=torch.int32).cuda()]
    out = torch.empty((n, heads, rank), dtype=dtype).cuda()
    kernels.latent_attention(q, cache, *args, max(news), max(lens), rank, 0.3, window, out)
    expected = torch.zeros((n, heads, rank), dtype=torch.float64)
    plain_ops.latent_attention(q.cpu(), cache.cpu(), *(a.cpu() for a in args), max(news), max(lens), rank, 0.3, window, expected)
    assert torch.allclose(out.double().cpu(), expected, **tol(dtype, float(expected.abs().max())))


@pytest.mark.parametrize("heads,rank,rot,page", [(16, 256, 32, 16), (6, 128, 32, 64), (20, 64, 16, 8), (16, 512, 64, 16), (3, 96, 0, 4)])
def test_latent_attention_decode_over_long_contexts(heads, rank, rot, page):
    """A decode step over contexts of thousands of tokens: the keys are cut into many ranges (up to 32, more than the
    merge kernel's usual form takes), blocks walk many tiles through all their key buffers, and the part of the page
    table that a block keeps in shared memory is long.  One key far back stands out in every request."""
    from miniserve_b200 import kernels

    dtype, dk = torch.bfloat16, rank + rot
    lens = [3000, 2111, 5]
    total_pages = sum((l + page - 1) // page for l in lens)
    order = torch.randperm(total_pages, generator=torch.Generator().manual_seed(3)).tolist()
    width = max((l + page - 1) // page for l in lens)
    tables, next_page = [], 0
    for l in lens:
        count = (l + page - 1) // page
        tables.append(order[next_page:next_page + count] + [0] * (width - count))
        next_page += count
    cache = rand((total_pages, page, dk), dtype, 21, 0.5)
    q = rand((len(lens), heads, dk), dtype, 22, 0.5)
    for r, l in enumerate(lens):                      # key 7 of every request points where the request's first head looks
        cache[tables[r][7 // page], 7 % page] = (q[r, 0].float() * 3.0).to(dtype)
    args = [torch.tensor(tables, dtype=torch.int32).cuda(), torch.arange(len(lens), dtype=torch.int32).cuda(),
            torch.tensor([l - 1 for l in lens], dtype=torch.int32).cuda(), torch.arange(len(lens) + 1, dtype=torch.int32).cuda(),
            torch.tensor(lens, dtype=torch.int32).cuda()]
    out = torch.empty((len(lens), heads, rank), dtype=dtype).cuda()
    kernels.latent_attention(q, cache, *args, 1, max(lens), rank, 0.3, None, out)
    expected = torch.zeros((len(lens), heads, rank), dtype=torch.float64)
    plain_ops.latent_attention(q.cpu(), cache.cpu(), *(a.cpu() for a in args), 1, max(lens), rank, 0.3, None, expected)
    assert torch.allclose(out.double().cpu(), expected, **tol(dtype, float(expected.abs().max())))
    far = cache[tables[0][7 // page], 7 % page, :rank].double().cpu()
    assert float((expected[0, 0] - far).abs().max()) < 0.05 * float(far.abs().max())      # the far key decides head 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_head_gate_and_batched_product(dtype):
    from miniserve_b200 import kernels

    n, heads, vdim, rank = 13, 5, 14, 18
    x, gate = rand((n, heads, vdim), dtype, 10), rand((n, 24), dtype, 11, 2.0)
    expected = x.double() * torch.sigmoid(gate[:, 9:9 + heads].double())[:, :, None]
    kernels.head_gate(x, gate, 9)
    assert torch.allclose(x.double(), expected, **tol(dtype, 2.0))
    # one product per head on strided views: a head's columns of wider rows in, a head's columns of wider rows out
    wide, weight = rand((n, heads * (rank + 3)), dtype, 12), rand((heads, vdim, rank), dtype, 13, 0.3)
    source = wide.view(n, heads, rank + 3)[:, :, :rank].transpose(0, 1)
    target = torch.zeros((n, heads, vdim + 2), dtype=dtype).cuda()
    kernels.linear_batched(source, weight, target[:, :, :vdim].transpose(0, 1))
    want = torch.einsum("hnk,hvk->nhv", source.double(), weight.double())
    assert torch.allclose(target[:, :, :vdim].double(), want, **tol(dtype, float(want.abs().max())))
    assert float(target[:, :, vdim:].abs().max()) == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("experts,top,width", [(5, 2, 96), (3, 3, 72), (64, 6, 40), (12, 1, 33)])
def test_router_and_routing(dtype, experts, top, width):
    from miniserve_b200 import kernels

    n = 37
    x = rand((n, width), dtype, 14)
    weight, bias = rand((experts, width), torch.float32, 15, 0.3), rand((experts,), torch.float32, 16, 0.5)
    if experts >= 5:
        weight[3] = weight[1]                # a tie between experts 1 and 3 for every token: the lower index goes first
        bias[3] = bias[1]
    ids, weights = torch.empty((n, top), dtype=torch.int32).cuda(), torch.empty((n, top), dtype=torch.float32).cuda()
    kernels.router_topk(x, weight, bias, top, ids, weights)
    want_ids, want_weights = torch.empty((n, top), dtype=torch.int64), torch.empty((n, top), dtype=torch.float64)
    plain_ops.router_topk(x.cpu(), weight.cpu(), bias.cpu(), top, want_ids, want_weights)
    logits = x.double().cpu() @ weight.double().cpu().T + bias.double().cpu()
    ranked = logits.sort(dim=1, descending=True).values
    clear = (ranked[:, :-1] - ranked[:, 1:]).clamp(min=0)
    clear = torch.where(clear == 0, torch.full_like(clear, 1.0), clear).min(dim=1).values > 1e-4      # exact ties are decided by index
    assert torch.equal(ids.cpu().long()[clear], want_ids[clear]) and int(clear.sum()) > n // 2
    assert torch.allclose(weights.double().cpu()[clear], want_weights[clear], atol=1e-5)
    assert torch.allclose(weights.sum(dim=1), torch.ones(n).cuda(), atol=1e-5)
    # the sort of the pairs by expert
    offsets = torch.empty(experts + 1, dtype=torch.int32).cuda()
    order, place = torch.empty(n * top, dtype=torch.int32).cuda(), torch.empty(n * top, dtype=torch.int32).cuda()
    kernels.expert_route(ids, experts, offsets, order, place)
    flat = ids.reshape(-1).cpu().long()
    assert offsets.cpu().tolist() == [0] + torch.bincount(flat, minlength=experts).cumsum(0).tolist()
    assert sorted(order.cpu().tolist()) == list(range(n * top))
    assert torch.equal(place.cpu().long()[order.cpu().long()], torch.arange(n * top))
    for e in range(experts):
        segment = order.cpu().long()[int(offsets[e]):int(offsets[e + 1])]
        assert bool((flat[segment] == e).all())
    # the experts' products over their segments, and the weighted sum
    inner = 20
    up, down = rand((experts, inner, width), dtype, 17, 0.2), rand((experts, width, inner), dtype, 18, 0.2)
    hidden, results = torch.empty((n * top, inner), dtype=dtype).cuda(), torch.empty((n * top, width), dtype=dtype).cuda()
    kernels.expert_linear(x, order, top, up, hidden, offsets, relu_square=True)
    kernels.expert_linear(hidden, None, top, down, results, offsets)
    shared, out = rand((n, width), dtype, 19), torch.empty((n, width), dtype=dtype).cuda()
    kernels.expert_combine(results, place, weights, shared, out)
    want = shared.double().cpu().clone()
    for t in range(n):
        for k in range(top):
            e = int(ids[t, k])
            h = (up[e].double().cpu() @ x[t].double().cpu()).clamp(min=0).pow(2)
            if dtype == torch.bfloat16:
                h = h.to(dtype).double()
            want[t] += float(weights[t, k]) * (down[e].double().cpu() @ h)
    assert torch.allclose(out.double().cpu(), want, **tol(dtype, float(want.abs().max())))
    y = rand((7, 9), dtype, 20)
    expected = y.double().clamp(min=0).pow(2)
    kernels.relu_square(y)
    assert torch.allclose(y.double(), expected, **tol(dtype, 2.0))


# --------------------------------------------------------------------------- parts alone


def mixer_weights(width, m, dtype, seed):
    heads = m["heads"]
    shapes = {"q": (heads * (m["dim"] + m["rot_dim"]), width), "dkv": (m["kv_rank"] + m["rot_dim"], width),
              "uk": (heads * m["dim"], m["kv_rank"]), "uv": (heads * m["vdim"], m["kv_rank"]), "g": (heads, width),
              "o": (width, heads * m["vdim"])}
    w = {"x." + name: rand(shape, dtype, seed + i, 0.12) for i, (name, shape) in enumerate(shapes.items())}
    w["x.dkv.norm"] = (1 + rand((m["kv_rank"],), torch.float32, seed + 9, 0.1)).to(dtype)
    return w


def build_mixer(width, m, eps, window=None):
    from miniserve_b200.parts import MIXERS, PartSpec

    position = PartSpec("rope", dict(head_dim=m["rot_dim"], theta=m["rot"]["base"], rotary_dim=m["rot"]["dims"], scaling=m["rot"]["scaling"]))
    return MIXERS.build(PartSpec("latent_attention", dict(
        hidden_size=width, num_heads=m["heads"], dim=m["dim"], rot_dim=m["rot_dim"], vdim=m["vdim"], kv_rank=m["kv_rank"],
        scale=m["scale"], eps=eps, position=position, window=window)), prefix="x.")


MIXERS_ALONE = [
    (88, vh.mixer(3, 24, 16, 20, 40, 0.21, vh.rot(8, 5000.0, vh.YARN_A))),
    (72, vh.mixer(1, 12, 6, 10, 22, 0.4, vh.rot(6, 100.0, None))),
    (128, vh.mixer(8, 32, 16, 32, 64, 0.15, vh.rot(16, 10000.0, vh.YARN_B))),
    (64, vh.mixer(16, 16, 32, 24, 96, 0.2, vh.rot(32, 10000.0, vh.YARN_A))),
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", range(len(MIXERS_ALONE)))
@pytest.mark.parametrize("window", [None, 23])
def test_latent_attention_part_far_keys_and_edges(dtype, case, window):
    """The mixer alone, fed in portions and then token by token through a paged cache.  One token far back, and
    the tokens just inside and just outside the window of the last queries, are scaled up so that their rotated key
    part (which no norm tames) decides the scores wherever it is seen: a key that is lost, read from a wrong page
    or let in from beyond the edge changes the result by far more than rounding."""
    from miniserve_b200.parts import PagedLatentNeed

    width, m = MIXERS_ALONE[case]
    part = build_mixer(width, m, 1e-5, window)
    assert part.cache_need() == PagedLatentNeed(m["kv_rank"], m["rot_dim"], window)
    w = mixer_weights(width, m, dtype, 30)
    assert sorted(s.name for s in part.param_specs()) == sorted(w)
    part.load(w)
    total = 333
    x = rand((total, width), dtype, 50)
    quiet_x = x.clone()
    # (two keys of the same loudness in one query's sight would compete, and bfloat16 rounds scores of 50 by 0.2: the
    # keys just outside are the loudest, so that letting one in would show most)
    loud = {5: 25.0, 250: 5.0} if window is None else {total - 40 - window: 25.0, total - 40 - window + 1: 5.0,
                                                       total - 3 - window: 25.0, total - 3 - window + 1: 5.0}
    for token, factor in loud.items():
        x[token] *= factor
    harness = Harness([part.cache_need()], dtype, page_size=8, num_pages=64, max_len=512)
    cuts = [(0, 3), (3, 5), (5, 130), (130, 131), (131, 290)] + [(i, i + 1) for i in range(290, total)]
    got = []
    for start, end in cuts:
        ctx = harness.context({"r": end - start})
        ctx.dtype = dtype
        got.append(part.forward(x[start:end].contiguous(), ctx, harness.view(ctx)).clone())
    wd = {k: v.double().cpu() for k, v in w.items()}
    expected = plain.latent_attention(x.double().cpu(), wd, "x.", m, 1e-5, torch.arange(total), window)
    quiet = plain.latent_attention(quiet_x.double().cpu(), wd, "x.", m, 1e-5, torch.arange(total), window)
    assert float((expected[-40:] - quiet[-40:]).abs().max()) > 0.1 * float(expected[-40:].abs().max())      # the loud keys decide
    assert torch.allclose(torch.cat(got).double().cpu(), expected, **tol(dtype, float(expected.abs().max())))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width,experts,top,inner,shared,rows", [(96, 5, 2, 24, 40, 23), (72, 3, 3, 20, None, 1), (128, 16, 4, 32, 64, 300),
                                                                 (40, 7, 1, 9, 5, 8)])
def test_routed_experts_part(dtype, width, experts, top, inner, shared, rows):
    from miniserve_b200.parts import FEED_FORWARDS, PagedKVNeed, PartSpec

    part = FEED_FORWARDS.build(PartSpec("routed_experts", dict(hidden_size=width, experts=experts, top=top, expert_size=inner,
                                                               shared_size=shared)), prefix="f.")
    w = {"f.router": rand((experts, width), dtype, 60, 0.5), "f.router.b": rand((experts,), dtype, 61, 0.3)}
    for e in range(experts):
        w[f"f.e{e}.up"], w[f"f.e{e}.down"] = rand((inner, width), dtype, 62 + 2 * e, 0.15), rand((width, inner), dtype, 63 + 2 * e, 0.15)
    if shared:
        w["f.shared.up"], w["f.shared.down"] = rand((shared, width), dtype, 97, 0.15), rand((width, shared), dtype, 98, 0.15)
    assert sorted(s.name for s in part.param_specs()) == sorted(w)
    part.load(w)
    x = rand((rows, width), dtype, 99)
    wd = {k: v.double().cpu() for k, v in w.items()}
    mlp = dict(router=dict(experts=experts, top=top), shared=dict(ff=shared) if shared else None)
    expected, _ = plain.routed_feed_forward(x.double().cpu(), wd, "f.", mlp)
    # rows whose routing is a close call in this number format are left out (the plain logits decide which)
    logits = (x.double().cpu() @ wd["f.router"].T + wd["f.router.b"]).sort(dim=1, descending=True).values
    clear = torch.ones(rows, dtype=torch.bool) if top == experts else (logits[:, top - 1] - logits[:, top]) > (1e-4 if dtype == torch.float32 else 0.05)
    out = part.forward(x, Harness([PagedKVNeed(1, 16, None)], dtype, num_pages=128, max_len=512).context({"a": rows}))
    assert int(clear.sum()) >= (rows + 1) // 2
    assert torch.allclose(out.double().cpu()[clear], expected[clear], **tol(dtype, float(expected.abs().max())))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("with_feed_forward", [True, False])
def test_parallel_block(dtype, with_feed_forward):
    """One norm, two readers, both outputs handed on unadded; the norm of the next block adds their sum."""
    from miniserve_b200.parts import BLOCKS, FEED_FORWARDS, NORMS, PartSpec

    width, m = MIXERS_ALONE[0]
    mixer = build_mixer(width, m, 1e-6)
    ffn = FEED_FORWARDS.build(PartSpec("gated_mlp", dict(hidden_size=width, intermediate_size=120, gate_name="gate", up_name="up",
                                                         down_name="down")), prefix="f.") if with_feed_forward else None
    norm = NORMS.build(PartSpec("rms", dict(name="n1", size=width, eps=1e-6)), prefix="")
    block = BLOCKS.build(PartSpec("parallel"), mixer=mixer, feed_forward=ffn, mixer_norm=norm, feed_forward_norm=None)
    w = mixer_weights(width, m, dtype, 130)
    w.update({"f.gate": rand((120, width), dtype, 140, 0.1), "f.up": rand((120, width), dtype, 141, 0.1),
              "f.down": rand((width, 120), dtype, 142, 0.1), "n1": (1 + rand((width,), torch.float32, 143, 0.1)).to(dtype)})
    for part in block.parts():
        part.load({s.name: w[s.name] for s in part.param_specs()})
    harness = Harness([mixer.cache_need()], dtype)
    n = 19
    residual, pending = rand((n, width), torch.float32, 151), (rand((n, width), dtype, 152), rand((n, width), dtype, 153))
    ctx = harness.context({"r": n})
    ctx.dtype = dtype
    x0 = residual.double().cpu() + (pending[0].double().cpu() + pending[1].double().cpu())
    handed = block.forward(residual, pending, ctx, harness.view(ctx))
    wd = {k: v.double().cpu() for k, v in w.items()}
    h = plain.rms_norm(x0, wd["n1"], 1e-6)
    mixed = plain.latent_attention(h, wd, "x.", m, 1e-6, torch.arange(n))
    assert torch.allclose(residual.double().cpu(), x0, atol=2e-6)
    if with_feed_forward:
        assert isinstance(handed, tuple) and len(handed) == 2
        assert torch.allclose(handed[0].double().cpu(), mixed, **tol(dtype, float(mixed.abs().max())))
        fed = plain.dense_feed_forward(h, wd, "f.")
        assert torch.allclose(handed[1].double().cpu(), fed, **tol(dtype, float(fed.abs().max())))
    else:
        assert torch.allclose(handed.double().cpu(), mixed, **tol(dtype, float(mixed.abs().max())))


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
        logits, _, gap = plain.forward(tokens, weights, config, return_layers=True)
        assert gap > 0.2, "the routing is too close to a tie for this test to mean anything"
        _ORACLE[key] = logits
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
# lengths at the borders of pages of 8 and 16 tokens, a single token, and a few hundred
LENGTHS = (1, 7, 8, 9, 16, 17, 33, 64, 65, 150, 301)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,page_size", [("a", 8), ("b", 16), ("c", 16), ("d", 4)])
@pytest.mark.parametrize("cutting", list(CUTTINGS))
def test_cuttings_against_plain(tmp_path, request, dtype, name, page_size, cutting):
    """Whole prompts; last tokens decoded one by one; portions down to two tokens; unequal requests batched together in a
    pool so small that pages and slots are used again: always the logits of the plain whole-sequence computation."""
    folder = vh.make_folder(tmp_path, name, seed=11)
    vocab = vh.CONFIGS[name]["vocab"]
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
    blocks from absolute key 0, routed rows computed independently), so a request alone and whole, in portions, and
    batched with others on other pages must give the same logits to the last bit or two: far tighter than the bound
    against the plain implementation, and independent of it."""
    folder = vh.make_folder(tmp_path, name, seed=16)
    vocab = vh.CONFIGS[name]["vocab"]
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
                assert float((results[cutting][rid][position] - alone).abs().max()) <= 1e-6 * scale, (rid, position, cutting)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "c"])
def test_prefill_against_decoding_every_token(tmp_path, dtype, name):
    """The same sequence as one prompt and token by token from its first token on (a long decode over several pages):
    the two agree with the plain logits and so, within rounding, with each other."""
    folder = vh.make_folder(tmp_path, name, seed=12)
    tokens = helpers.random_tokens(vh.CONFIGS[name]["vocab"], 140, seed=500)
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
    rows when graphs are on: the routed experts and the latent cache inside a replayed step)."""
    folder = vh.make_folder(tmp_path, "c", seed=13)
    vocab = vh.CONFIGS["c"]["vocab"]
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
    """``LLM.generate``: the engine's own entry point, scheduler (chunked prompts, a token budget that forces portions) and
    sampler; every generated token is the plain implementation's choice, or as good as it within rounding."""
    from miniserve_b200.engine.llm import LLM
    from miniserve_b200.sampling import SamplingParams

    folder = vh.make_folder(tmp_path, "a", seed=14)
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
    """``bin/trace_run`` and ``python -m miniserve_b200.generate`` on a Vesidra folder, as a user runs them."""
    folder = vh.make_folder(tmp_path, "b", seed=15)
    vocab = vh.CONFIGS["b"]["vocab"]
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
    config, weights = plain.load_folder(folder)
    tokens = list(requests["q1"])
    for token in produced:
        logits = plain.forward(tokens, weights, config)[-1]
        assert float(logits.max() - logits[token]) <= 2 * bound_of(dtype, logits)
        tokens.append(token)
    assert len(produced) == 5
