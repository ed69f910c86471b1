"""Baselix in the engine against the plain implementation (tests/plain/baselix_plain.py): every mechanism alone,
then whole models under every way of cutting the work, long decoding, generation through the Python entry point and
the trace program."""
import json
import os
import random
import subprocess
import sys

import numpy as np
import pytest
import torch

import baselix_tiny as BT
import traces
from plain import baselix_plain as BP
from replay_util import run_trace

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
F64 = torch.float64


def tol_for(dtype):
    return 2e-4 if dtype in ("float32", torch.float32) else 6e-2


def rel_err(got, ref):
    """Largest difference relative to the size of the reference (at least 1)."""
    return float((got.double().cpu() - ref.double()).abs().max()) / max(1.0, float(ref.abs().max()))


def plain_ctx(n, dtype):
    from zedinfer_b200.parts import StepContext
    return StepContext(n, 1, dtype, torch.device(DEV), None, None, None, [], None, [0], [n], [0], [-1])


def step_context(cache, dtype, portions, table_width=64):
    from zedinfer_b200.engine.core import PinnedStaging, StepEntry, build_step_context
    entries, rcs = [], []
    for rid, n in portions:
        rc = cache.get(rid) or cache.open(rid)
        cache.ensure(rc, rc.length + n)
        entries.append(StepEntry(rid, [0] * n, []))
        rcs.append(rc)
    ctx, _ = build_step_context(entries, rcs, cache, table_width, dtype, torch.device(DEV), 10, PinnedStaging())
    return ctx, entries, rcs


# ---------------------------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows", [3, 70, 300])
def test_norm_with_a_weight_around_zero_and_a_scaled_residual(dtype, rows):
    from zedinfer_b200.parts import ResidualStream, RMSNorm
    norm = RMSNorm(size=136, eps=1e-3, name="norm1", unit_offset=True)
    assert list(norm.tensor_specs()) == ["norm1"]
    w = (0.05 * torch.randn(136)).to(dtype)
    norm.bind({"norm1": w.to(DEV)})
    assert norm.weight.dtype == torch.float32           # 1 + w keeps w's low bits
    h = torch.randn(rows, 136)
    delta = torch.randn(rows, 136).to(dtype)
    stream = ResidualStream(h.clone().to(DEV), delta.to(DEV), delta_scale=0.3)
    out = torch.empty(rows, 136, dtype=dtype, device=DEV)
    norm.forward_residual(stream, out)
    x = h.double() + 0.3 * delta.double()
    assert rel_err(stream.h, x) < 1e-6
    assert rel_err(out, BP.norm_around_zero(x, w.double(), 1e-3)) < (1e-5 if dtype == torch.float32 else 1e-2)
    # rows picked by index (the final norm of the wanted rows) use the same factor and leave the stream alone
    stream = ResidualStream(h.clone().to(DEV), delta.to(DEV), delta_scale=0.3)
    idx = torch.tensor([rows - 1, 0], dtype=torch.int32, device=DEV)
    out2 = torch.empty(2, 136, dtype=dtype, device=DEV)
    norm.forward_residual(stream, out2, row_idx=idx)
    assert torch.equal(out2.cpu(), out[[rows - 1, 0]].cpu()) and torch.equal(stream.h.cpu(), h)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_partial_sums_enter_the_stream_with_the_residual_factor(dtype):
    from zedinfer_b200 import ops
    h = torch.randn(20, 64, device=DEV)
    parts = torch.randn(4, 20, 64, device=DEV)
    w = torch.ones(64, device=DEV)
    out = torch.empty(20, 64, dtype=dtype, device=DEV)
    res = h.clone()
    ops.add_rmsnorm(res, parts, w, 1e-6, out, delta_scale=0.25)
    want = h.double().cpu() + 0.25 * parts.sum(0).to(dtype).double().cpu()
    assert rel_err(res, want) < 1e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_with_learned_positions_and_the_logit_cap(dtype):
    from zedinfer_b200.parts import LearnedPositionEmbedding, OutputHead
    emb = LearnedPositionEmbedding(50, 24, 40, name="embed", position_name="pos")
    t = {"embed": torch.randn(50, 24).to(dtype), "pos": torch.randn(40, 24).to(dtype)}
    emb.bind({k: v.to(DEV) for k, v in t.items()})
    ids = [3, 49, 0, 7]
    pos = [0, 39, 5, 6]
    ctx = plain_ctx(4, dtype)
    ctx.token_ids = torch.tensor(ids, dtype=torch.int32, device=DEV)
    ctx.positions = torch.tensor(pos, dtype=torch.int32, device=DEV)
    out = torch.empty(4, 24, dtype=torch.float32, device=DEV)
    emb.forward_step(ctx, out)
    want = t["embed"].double()[ids] + t["pos"].double()[pos]
    assert rel_err(out, want) < 1e-6
    assert not torch.allclose(out.cpu().double(), BP.embed(ids, t["embed"].double(), t["pos"].double()))   # positions count
    head = OutputHead(50, 24, tied=True, name="head", softcap=2.5)
    head.bind({}, embedding=emb.tied_weight())
    x = (3 * torch.randn(4, 24)).to(dtype)
    logits = torch.empty(4, 50, dtype=torch.float32, device=DEV)
    head.forward(x.to(DEV), logits)
    want = BP.capped_logits(x.double(), t["embed"].double(), 2.5)
    assert float(want.abs().max()) > 2.0                                # the cap is at work
    assert rel_err(logits, want) < (1e-5 if dtype == torch.float32 else 2e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows", [5, 12, 150, 300])
@pytest.mark.parametrize("hidden", [72, 96])
def test_squared_relu_and_clamped_gated_feed_forwards(dtype, rows, hidden):
    """bfloat16 with a width that is a multiple of 32 and up to 16 rows: the activation runs in the epilogue of the
    weight-streaming product; from 128 rows in that of the tcgen05 product; otherwise in a kernel of its own."""
    from zedinfer_b200.parts import ClampedGatedMLP, SquaredReluMLP
    g = torch.Generator().manual_seed(5)
    x = torch.randn(rows, hidden, generator=g).to(dtype)
    ctx = plain_ctx(rows, dtype)
    r = (lambda z: z.to(dtype).double()) if dtype == torch.bfloat16 else (lambda z: z)
    tol = 1e-5 if dtype == torch.float32 else 3e-2

    ff = SquaredReluMLP(hidden, 200)
    t = {k: (0.3 * torch.randn(v.shape, generator=g)).to(dtype) for k, v in ff.tensor_specs().items()}
    assert sorted(t) == ["down", "up"]
    ff.bind({k: v.to(DEV) for k, v in t.items()})
    got = ff.forward(x.to(DEV), ctx)
    a = torch.relu(r(x.double() @ t["up"].double().T))
    assert rel_err(got, r(a * a) @ t["down"].double().T) < tol

    for limit in (0.7, None):
        ff = ClampedGatedMLP(hidden, 104, limit=limit, slope=1.702, up_offset=1.0)
        t = {k: (0.3 * torch.randn(v.shape, generator=g)).to(dtype) for k, v in ff.tensor_specs().items()}
        ff.bind({k: v.to(DEV) for k, v in t.items()})
        got = ff.forward(x.to(DEV), ctx)
        gate, up = r(x.double() @ t["gate"].double().T), r(x.double() @ t["up"].double().T)
        if limit is not None:
            assert float(gate.max()) > limit and float(up.min()) < -limit         # the clamps are at work
            gate, up = gate.clamp(max=limit), up.clamp(-limit, limit)
        want = r(gate * torch.sigmoid(1.702 * gate) * (up + 1.0)) @ t["down"].double().T
        assert rel_err(got, want) < tol
    if dtype == torch.float32:
        w = {k: v.double() for k, v in t.items()}
        # the same numbers from the plain expert, for a limit that never binds
        assert rel_err(got, BP.clamped_expert(x.double(), w["gate"], w["up"], w["down"], 1e9)) < tol


def test_router_top_choices_and_their_weights():
    from zedinfer_b200 import ops
    g = torch.Generator().manual_seed(2)
    for experts, top in ((6, 2), (5, 1), (3, 3), (40, 7), (130, 4)):
        z = torch.randn(37, experts, generator=g)
        idx = torch.empty(37, top, dtype=torch.int32, device=DEV)
        wts = torch.empty(37, top, dtype=torch.float32, device=DEV)
        ops.route_topk(z.to(DEV), top, idx, wts)
        vals, want_idx = torch.topk(z.double(), top, dim=-1)
        assert torch.equal(idx.cpu().long(), want_idx)
        assert rel_err(wts, torch.softmax(vals, -1)) < 1e-6
        assert torch.allclose(wts.sum(1).cpu(), torch.ones(37), atol=1e-6)
    # equal logits: the lower index is chosen first
    z = torch.tensor([[1.0, 3.0, 3.0, 0.0, 3.0]], device=DEV)
    idx = torch.empty(1, 2, dtype=torch.int32, device=DEV)
    wts = torch.empty(1, 2, dtype=torch.float32, device=DEV)
    ops.route_topk(z, 2, idx, wts)
    assert idx.tolist() == [[1, 2]] and wts.tolist() == [[0.5, 0.5]]


@pytest.mark.parametrize("streaming", [False, True])
@pytest.mark.parametrize("tensor_cores", [False, True])
@pytest.mark.parametrize("rows,experts,top", [(1, 4, 2), (9, 6, 2), (200, 5, 1), (70, 3, 3), (30, 4, 2)])
def test_grouped_product_over_experts(rows, experts, top, tensor_cores, streaming, monkeypatch):
    """The grouped product alone against one product per row, experts without rows among them: the weight-streaming
    form (up to 64 sorted rows), the ``wmma`` form (bfloat16) and the SIMT form (float32, and what the others leave)."""
    from zedinfer_b200 import ops
    monkeypatch.setattr(ops, "MOE_TENSOR_CORES", tensor_cores)
    monkeypatch.setattr(ops, "MOE_FEW_ROWS_STREAMING", streaming)
    dtype = torch.bfloat16 if tensor_cores else torch.float32
    g = torch.Generator().manual_seed(rows)
    k, n = 72, 40
    x = torch.randn(rows, k, generator=g).to(dtype)
    w = (0.3 * torch.randn(experts, 2 * n, k, generator=g)).to(dtype)
    idx = torch.stack([torch.randperm(experts, generator=g)[:top] for _ in range(rows)]).int()
    if experts > 3:
        idx[idx == 1] = 0 if top == 1 else 3        # expert 1 gets no row
        if top > 1:                                  # keep a token's choices distinct
            for t in range(rows):
                if len(set(idx[t].tolist())) < top:
                    idx[t] = torch.tensor([0, 2][:top] if top <= 2 else list(range(top)))
    offsets = torch.empty(experts + 1, dtype=torch.int32, device=DEV)
    row_pair = torch.empty(rows * top, dtype=torch.int32, device=DEV)
    pair_row = torch.empty(rows * top, dtype=torch.int32, device=DEV)
    ops.moe_group(idx.to(DEV), experts, offsets, row_pair, pair_row)
    counts = torch.bincount(idx.flatten().long(), minlength=experts)
    assert offsets.tolist() == [0] + torch.cumsum(counts, 0).tolist()
    rp, pr = row_pair.cpu().long(), pair_row.cpu().long()
    assert torch.equal(rp[pr], torch.arange(rows * top)) and sorted(rp.tolist()) == list(range(rows * top))
    expert_of_row = idx.flatten().long()[rp]
    assert torch.equal(expert_of_row, torch.sort(expert_of_row).values)         # rows are sorted by expert
    out = torch.empty(rows * top, n, dtype=dtype, device=DEV)
    ops.moe_gemm(x.to(DEV), row_pair, top, w.to(DEV), offsets, out, gated=(0.8, 1.702, 1.0))
    plain = torch.empty(rows * top, 2 * n, dtype=dtype, device=DEV)
    ops.moe_gemm(x.to(DEV), row_pair, top, w.to(DEV), offsets, plain)
    r = (lambda z: z.to(dtype).double()) if dtype == torch.bfloat16 else (lambda z: z)
    xs = x.double()[rp // top]
    both = r(torch.einsum("rk,rnk->rn", xs, w.double()[expert_of_row]))
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert rel_err(plain, both) < tol
    gate, up = both[:, :n].clamp(max=0.8), both[:, n:].clamp(-0.8, 0.8)
    assert rel_err(out, gate * torch.sigmoid(1.702 * gate) * (up + 1.0)) < tol


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows", [1, 6, 90, 700])
@pytest.mark.parametrize("experts,top,shared", [(6, 2, True), (5, 1, False), (3, 3, True)])
def test_routed_feed_forward_part(dtype, rows, experts, top, shared):
    """700 rows in bfloat16: the grouped products run on the tcgen05 kernel over rows copied into sorted order, every
    expert's share padded to whole tiles; fewer rows, and float32: the kernels of ``csrc/moe.cu``."""
    from zedinfer_b200.config import PartSpec
    from zedinfer_b200.parts import RoutedExperts
    sh = PartSpec("clamped_gated_mlp", {"hidden_size": 64, "intermediate_size": 24, "limit": 0.6, "slope": 1.702,
                                        "up_offset": 1.0}) if shared else None
    ff = RoutedExperts(64, 40, experts, top, limit=0.9, slope=1.702, up_offset=1.0, shared=sh)
    assert ff.capture_safe
    g = torch.Generator().manual_seed(experts * 100 + rows)
    t = {k: (0.3 * torch.randn(v.shape, generator=g)).to(dtype) for k, v in ff.tensor_specs().items()}
    t["router"] = (2.0 * torch.randn(experts, 64, generator=g)).to(dtype)         # clear choices
    ff.bind({k: v.to(DEV) for k, v in t.items()})
    x = torch.randn(rows, 64, generator=g).to(dtype)
    got = ff.forward(x.to(DEV), plain_ctx(rows, dtype))
    w = {k: v.double() for k, v in t.items()}
    mlp = {"router": {"top": top}, "expert": {"limit": 0.9}, "shared": {"limit": 0.6} if shared else None}
    want = BP.routed_ff(x.double(), w, mlp)
    idx, wts = ff.route(x.to(DEV))
    pidx, pw = BP.route(x.double(), w["router"], w["router.b"], top)
    assert torch.equal(idx.cpu().long(), pidx) and rel_err(wts, pw) < 1e-5
    assert rel_err(got, want) < (2e-5 if dtype == torch.float32 else 4e-2)
    from zedinfer_b200 import ops
    assert ff._tcgen05_ok(x.to(DEV), rows * top) == (dtype == torch.bfloat16 and rows * top >= ops.MOE_TCGEN05_MIN_PAIRS)
    assert ops.MOE_TCGEN05_MIN_PAIRS <= 90 * 2
    ops.raise_if_tcgen05_failed(torch.device(DEV))


def test_padded_grouping_leaves_whole_tiles_to_every_expert():
    from zedinfer_b200 import ops
    g = torch.Generator().manual_seed(0)
    experts, top, rows, pad = 7, 2, 333, 128
    idx = torch.stack([torch.randperm(experts, generator=g)[:top] for _ in range(rows)]).int()
    idx[idx == 4] = 5                                   # expert 4 gets nothing
    pairs = rows * top
    tiles = (pairs + experts * (pad - 1) + pad - 1) // pad
    starts = torch.empty(experts + 1, dtype=torch.int32, device=DEV)
    row_pair = torch.empty(tiles * pad, dtype=torch.int32, device=DEV)
    pair_row = torch.empty(pairs, dtype=torch.int32, device=DEV)
    tile_expert = torch.empty(tiles, dtype=torch.int32, device=DEV)
    ops.moe_group_padded(idx.to(DEV), experts, pad, starts, row_pair, pair_row, tile_expert)
    counts = torch.bincount(idx.flatten().long(), minlength=experts)
    want_starts = [0]
    for c in counts.tolist():
        want_starts.append(want_starts[-1] + -(-c // pad) * pad)
    assert starts.tolist() == want_starts
    rp, pr, te = row_pair.cpu().long(), pair_row.cpu().long(), tile_expert.tolist()
    assert torch.equal(rp[pr], torch.arange(pairs)) and int((rp >= 0).sum()) == pairs
    flat = idx.flatten().long()
    for e in range(experts):
        mine = rp[want_starts[e]:want_starts[e + 1]]
        assert int((mine >= 0).sum()) == int(counts[e]) and all(int(flat[p]) == e for p in mine[mine >= 0].tolist())
        assert te[want_starts[e] // pad:want_starts[e + 1] // pad] == [e] * ((want_starts[e + 1] - want_starts[e]) // pad)
    assert all(t == -1 for t in te[want_starts[-1] // pad:])
    x = torch.randn(rows, 40, generator=g).bfloat16().to(DEV)
    out = torch.empty(tiles * pad, 40, dtype=torch.bfloat16, device=DEV)
    ops.moe_gather_rows(x, row_pair, top, out)
    ref = torch.where((rp >= 0)[:, None], x.cpu()[(rp.clamp(min=0) // top)], torch.zeros(1, 40, dtype=torch.bfloat16))
    assert torch.equal(out.cpu(), ref)


def write_latents(view, tables, c):
    """Put the rows of ``c`` (one request, positions from 0) into the pages of ``tables`` (a list of page numbers)."""
    ps = view.page_size
    for p in range(c.shape[0]):
        view.tensor[tables[p // ps], 0, 0, p % ps] = c[p].to(view.tensor.dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rank,heads,window,page", [(64, 4, 21, 8), (128, 6, 37, 16), (32, 3, 7, 4), (320, 2, 33, 16),
                                                   (64, 20, 16, 16), (64, 5, 70, 24), (128, 2, 50, 12), (128, 17, 9, 128)])
def test_attention_over_latents_sees_exactly_its_window_and_the_sink(dtype, rank, heads, window, page):
    """One score made to stand out: a query is aligned with the latent of one chosen key whose other coordinates carry a
    mark.  The key just inside the window shows in the output, the key just outside does not, whether the query comes
    in a prompt portion or alone; a far key and keys on both sides of a page border likewise.  A sink of weight
    comparable to the keys' shows as well.  bfloat16 with ranks 64 and 128 runs on the tensor-core kernels (pages of a
    power of two: TMA and tcgen05; other pages: cp.async and mma.sync), the rest on the general kernel."""
    from zedinfer_b200 import ops
    from zedinfer_b200.cache import CacheManager
    from zedinfer_b200.cache.manager import PagedKVNeed
    T = 3 * window + 5 + (page if page > 3 * window else 0)      # at least one page border before the query
    g = torch.Generator().manual_seed(rank + window)
    cache = CacheManager([(0, PagedKVNeed(1, rank, None, planes=1))], page, max_requests=2)
    cache.allocate_device(2 * (T // page + 2), dtype, DEV)
    view = cache.view_for_call(0)
    scale = 0.5
    sinks = torch.linspace(0.5, 12.0, heads)                  # the last head's sink weighs as much as the chosen key
    P = T - 1                                                  # the query's position
    marks = [P - window, P - window + 1, 0, P, (P // page) * page, (P // page) * page - 1]
    for mark in marks:
        c = 0.1 * torch.randn(T, rank, generator=g)
        c[:, 0] = 0.0
        c[mark, 0] = 6.0                                       # the chosen key
        c[mark, 1:] += 3.0                                     # ... and its mark in the values
        c = c.to(dtype)
        q = 0.1 * torch.randn(T, heads, rank, generator=g)
        q[:, :, 0] = 4.0                                       # every query is aligned with coordinate 0
        q = q.to(dtype)
        k = c.double()[:, None, :].expand(T, heads, rank)
        want = BP.windowed_sink_attention(q.double(), k, k, sinks.double(), scale, window)
        seen = P - window < mark <= P
        assert (float(want[P].mean()) > 1.5) == seen           # the case shows what it is meant to show
        for cut in ((T,), (T - 1, 1), (P - window, 3, window - 4, 2)):
            rid = f"r{mark}_{len(cut)}"
            done = 0
            for n in cut:
                ctx, entries, rcs = step_context(cache, dtype, [(rid, n)])
                write_latents(view, rcs[0].tables[0], c[:done + n])
                out = torch.empty(n, heads, rank, dtype=dtype, device=DEV)
                ops.attention(q[done:done + n].contiguous().to(DEV), view, out, ctx, heads, 1, rank, window, scale,
                              sinks=sinks.to(DEV))
                cache.commit(rcs[0], rcs[0].length + n)
                err = rel_err(out, want[done:done + n])
                assert err < (1e-5 if dtype == torch.float32 else 2e-2), (mark, cut, done, err)
                done += n
            cache.close(cache.get(rid))
        if mark == marks[1]:                                   # leaving the sink out would show
            no_sink = BP.windowed_sink_attention(q.double(), k, k, torch.full((heads,), -1e30, dtype=F64), scale, window)
            assert rel_err(no_sink[P], want[P]) > 0.02


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,dim,vdim,rank,window,wide", [(3, 16, 24, 32, 9, 14), (4, 32, 16, 64, 20, 20), (2, 64, 32, 128, 33, 40)])
def test_latent_attention_mixer_over_portions_and_a_borrower(dtype, heads, dim, vdim, rank, window, wide):
    """The mixer alone: a prompt fed in portions gives what the plain whole-sequence function gives, for the layer that
    writes the latents and for a second layer that reads them with projections, sinks and a wider window of its own."""
    from zedinfer_b200.cache import CacheManager
    from zedinfer_b200.parts import LatentAttentionMixer
    hidden, eps = 72, 1e-5
    owner = LatentAttentionMixer(hidden, heads, dim, vdim, rank, eps, scale=0.21, window=window, cache_window=wide)
    reader = LatentAttentionMixer(hidden, heads, dim, vdim, rank, eps, scale=0.4, window=wide, cache_window=wide, own_latent=False)
    assert "dkv" in owner.tensor_specs() and "dkv" not in reader.tensor_specs() and "dkv.norm" not in reader.tensor_specs()
    g = torch.Generator().manual_seed(rank)
    tens = []
    for mixer in (owner, reader):
        t = {k: (torch.randn(v.shape, generator=g) * 0.3).to(dtype) for k, v in mixer.tensor_specs().items()}
        t["sink"] = torch.linspace(-0.5, 1.5, heads).to(dtype)
        mixer.bind({k: v.to(DEV) for k, v in t.items()})
        tens.append({k: v.double() for k, v in t.items()})
    cache = CacheManager([(0, owner.cache_need())], 8, max_requests=2)
    cache.allocate_device(24, dtype, DEV)
    view = cache.view_for_call(0)
    total = 75
    x = torch.randn(total, hidden, generator=g).to(dtype)
    got_a, got_b, done = [], [], 0
    for n in (7, 2, 1, 30, 1, 1, 33):
        ctx, entries, rcs = step_context(cache, dtype, [("r", n)])
        xs = x[done:done + n].to(DEV)
        got_a.append(owner.forward(xs, ctx, view, owns_cache=True).cpu())
        got_b.append(reader.forward(xs, ctx, view, owns_cache=False).cpu())
        cache.commit(rcs[0], rcs[0].length + n)
        done += n
    assert cache.get("r").tables[0][0] == -1                    # pages behind the wider window went back
    c = BP.latent(x.double(), tens[0]["dkv"], tens[0]["dkv.norm"], eps)
    if dtype == torch.bfloat16:
        c = c.to(dtype).double()
    tol = 2e-5 if dtype == torch.float32 else 4e-2
    mk = lambda w, s: {"heads": heads, "dim": dim, "vdim": vdim, "mask": {"size": w}, "scale": s}
    assert rel_err(torch.cat(got_a), BP.latent_attention(x.double(), c, tens[0], mk(window, 0.21))) < tol
    assert rel_err(torch.cat(got_b), BP.latent_attention(x.double(), c, tens[1], mk(wide, 0.4))) < tol


# ---------------------------------------------------------------------------------------------
# whole models
# ---------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("baselix_models")
    return {name: BT.make_model_dir(root, name) for name in BT.CONFIGS}


def make_requests(cfg, lengths, seed):
    rng = random.Random(seed)
    return {f"r{i}": [rng.randrange(cfg["vocab"]) for _ in range(n)] for i, n in enumerate(lengths)}


_plain_cache = {}


def expected_logits(model_dir, requests):
    if model_dir not in _plain_cache:
        _plain_cache[model_dir] = BP.read_model(model_dir, F64)
    cfg, w = _plain_cache[model_dir]
    return {rid: BP.forward(cfg, w, toks).float() for rid, toks in requests.items()}


def judge(got, exp, dtype):
    """float32: every position within the tolerance.  bfloat16: a close call of a router may go the other way, which
    moves one token's output by more than rounding does: at most 2 % of the positions may be beyond the tolerance."""
    tol = tol_for(dtype)
    errs = {key: float((row - exp[key[0]][key[1]]).abs().max()) / max(1.0, float(exp[key[0]].abs().max()))
            for key, row in got.items()}
    over = sorted((k for k, e in errs.items() if not e <= tol), key=lambda k: (str(k[0]), k[1]))
    allowed = 0 if dtype == "float32" else max(1, len(errs) // 50)
    assert len(over) <= allowed, f"{len(over)} of {len(errs)} positions beyond {tol}; first {over[0]} with {errs[over[0]]}"
    assert all(e == e and e < 1e30 for e in errs.values())


LENGTHS = {"A": [7, 13, 95, 45], "B": [1, 17, 120, 64], "C": [150, 5, 80], "D": [50, 2, 61], "E": [66, 3, 140]}
PAGES = {"A": 4, "B": 16, "C": 16, "D": 8, "E": 16}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
@pytest.mark.parametrize("family", ["whole", "tail", "chunks", "mixed"])
def test_cuts_match_plain(models, name, dtype, family):
    """Whole prompts; a tail decoded token by token (longer than every window); portions down to two tokens; mixed
    batches of unequal requests in a pool so small that pages are handed out again."""
    from zedinfer_b200.engine.core import EngineCore
    cfg, _ = BT.CONFIGS[name]
    requests = make_requests(cfg, LENGTHS[name] + ([64, 31, 77] if family == "mixed" else []), seed=5)
    if family == "tail":
        steps = traces.tail_decode(requests, tail=48)
    else:
        steps = {"whole": traces.whole, "chunks": traces.chunks, "mixed": traces.mixed}[family](requests)
    page = PAGES[name]
    need = traces.max_live_tokens(steps, round_to=page)
    core = EngineCore(models[name], dtype, page_size=page, num_pages=need // page, max_requests=4)
    got = run_trace(core, steps)
    judge(got, expected_logits(models[name], requests), dtype)
    assert core.cache.num_live == 0 and all(g.pool.num_used == 0 for g in core.cache.groups)


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "float32"), ("B", "bfloat16"), ("C", "bfloat16")])
def test_many_decoding_requests_with_and_without_graphs(models, name, dtype, graphs):
    """Steps as a scheduler makes them: up to 12 decoding requests beside one prompt portion, then decode-only steps whose
    number of rows falls to one; with graphs the decode-only steps replay captured buckets (bfloat16 with ranks 64 and 128:
    the TMA decode kernel and the tcgen05 prefill kernel with sinks inside captured steps)."""
    from zedinfer_b200.engine.core import EngineCore
    cfg, _ = BT.CONFIGS[name]
    rng = random.Random(8)
    requests = make_requests(cfg, [rng.randint(40, 90) for _ in range(15)], seed=3)
    steps = traces.decode_heavy(requests, seed=4, max_live=12, tail=(8, 30), portion=32)
    need = traces.max_live_tokens(steps, round_to=16)
    core = EngineCore(models[name], dtype, page_size=16, num_pages=need // 16, max_requests=16, cuda_graphs=graphs)
    core.GPU_BOUND_RATIO = float("inf")
    assert core.capture_safe, core.capture_blockers
    got = run_trace(core, steps)
    core.check_kernels()
    judge(got, expected_logits(models[name], requests), dtype)
    if graphs:
        assert core._decode_graphs
    assert core.cache.num_live == 0 and all(g.pool.num_used == 0 for g in core.cache.groups)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_the_first_tokens(models, dtype):
    """One token, two tokens, and a request decoded for 260 steps from a prompt of three: every window slides over decoded
    tokens many times, pages go back behind it, positions run far beyond any window."""
    from zedinfer_b200.engine.core import EngineCore
    cfg, _ = BT.CONFIGS["A"]
    requests = make_requests(cfg, [1, 2, 263], seed=9)
    steps = traces.tail_decode(requests, tail=260)
    core = EngineCore(models["A"], dtype, page_size=4, num_pages=80, max_requests=2)
    got = run_trace(core, steps)
    judge(got, expected_logits(models["A"], requests), dtype)
    # the windowed groups never held more than a window and a page
    assert all(g.pool.num_used == 0 for g in core.cache.groups)


@pytest.mark.parametrize("name", ["A", "C"])
def test_float32_is_the_same_however_it_is_cut(models, name):
    """The same positions through four different schedules: the same bits (every float32 sum of the design has one
    order, which depends on constants alone)."""
    from zedinfer_b200.engine.core import EngineCore
    cfg, _ = BT.CONFIGS[name]
    requests = make_requests(cfg, [90, 41], seed=2)
    runs = []
    for steps in (traces.whole(requests), traces.tail_decode(requests, tail=20), traces.chunks(requests), traces.mixed(requests)):
        core = EngineCore(models[name], "float32", page_size=16, num_pages=40, max_requests=4)
        runs.append(run_trace(core, steps))
    for other in runs[1:]:
        assert all(torch.equal(other[k], runs[0][k]) for k in runs[0])


@pytest.mark.parametrize("name,graphs", [("A", False), ("A", True), ("B", True), ("D", False)])
def test_greedy_generation_equals_plain(models, name, graphs):
    """Through the Python entry point and its scheduler: prompts in portions of five, a pool of pages that the requests
    fill again, greedy tokens equal to the plain implementation's."""
    from zedinfer_b200 import GenerationConfig, SchedulerConfig
    from zedinfer_b200.engine import InferenceEngine
    cfg, _ = BT.CONFIGS[name]
    rng = random.Random(4)
    prompts = [[rng.randrange(cfg["vocab"]) for _ in range(n)] for n in (9, 23, 1, 14)]
    engine = InferenceEngine.create(models[name], SchedulerConfig(num_kv_pages=30, kv_block_size=4, max_batch_requests=3,
                                                                  max_prefill_tokens=5, cuda_graphs=graphs),
                                    dtype="float32")
    results = engine.generate_batch(prompts, GenerationConfig(max_new_tokens=24, ignore_eos=True))
    pcfg, w = BP.read_model(models[name], F64)
    for p, r in zip(prompts, results):
        assert r.finish_reason == "length"
        assert r.output_ids == BP.greedy(pcfg, w, p, 24)
    st = engine.cache_stats()
    assert st["live_requests"] == 0 and st["free_pages"] == st["pages_per_group"]


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_trace_program_on_a_baselix_folder(models, tmp_path, dtype):
    cfg, _ = BT.CONFIGS["B"]
    requests = make_requests(cfg, [70, 9, 33, 50, 21], seed=6)
    steps = traces.mixed(requests, seed=1)
    need = traces.max_live_tokens(steps, round_to=64)
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", models["B"], "--dtype", dtype,
                           "--out", str(out), "--max-tokens", str(need)],
                          input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done ")] == [f"done {i}" for i in range(len(steps))]
    got, progress = {}, {}
    for st in steps:
        rows = np.fromfile(out / f"{st['step']}.f32", dtype="<f4").reshape(-1, cfg["vocab"])
        row = 0
        for e in st["entries"]:
            base = progress.get(e["id"], 0)
            for j in e["want"]:
                got[(e["id"], base + j)] = torch.from_numpy(rows[row].copy())
                row += 1
            progress[e["id"]] = base + len(e["tokens"])
        assert row == rows.shape[0]
    judge(got, expected_logits(models["B"], requests), dtype)


def test_command_line_programs_take_the_design(tmp_path, capsys):
    """From a bare config.json with weights drawn on the device: the bench program, continuous batching, and the
    consistency program, which returns 0 only if every float32 logit is the same bit pattern however the work is cut
    (also with fewer layers than the configuration lists)."""
    from zedinfer_b200.cli import batch_bench, bench, consistency
    path = tmp_path / "config.json"
    path.write_text(json.dumps(BT.BX_A))
    common = [str(path), "--random-weights", "7", "--kv-pages", "40", "--max-seq-len", "128"]
    assert bench.main(common + ["-p", "24", "-d", "5", "-r", "1"]) == 0
    out = capsys.readouterr().out
    assert "Prefill:" in out and "Decode :" in out
    assert batch_bench.main(common + ["-b", "5", "-p", "6", "--prefill-len-max", "40", "-d", "7", "-r", "1",
                                      "--warmup-rounds", "1", "--max-prefill-tokens", "16"]) == 0
    assert "5 requests, 35 tokens generated" in capsys.readouterr().out
    assert consistency.main([str(path), "--random-weights", "5", "--tokens", "120", "--requests", "5", "--layers", "3"]) == 0
    lines = [json.loads(l) for l in capsys.readouterr().out.strip().splitlines()]
    assert {(l["dtype"], l["mode"]) for l in lines} >= {("float32", "tail"), ("float32", "portions"), ("float32", "mixed"),
                                                        ("bfloat16", "mixed"), ("bfloat16", "whole")}
    assert all(l["values_not_bit_equal"] == 0 for l in lines if l["dtype"] == "float32")
