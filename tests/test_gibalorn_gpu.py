"""Gibalorn in the engine against the plain implementation (tests/plain/gibalorn_plain.py): every mechanism alone,
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

import gibalorn_tiny as GT
import traces
from plain import gibalorn_plain as GP
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


def step_context(cache, dtype, portions, table_width=64):
    """A step's context for ``portions = [(request id, tokens), ...]`` on ``cache`` (requests are opened as they appear)."""
    from zedinfer_b200.engine.core import PinnedStaging, StepEntry, build_step_context
    entries, rcs = [], []
    for rid, n in portions:
        rc = cache.get(rid) or cache.open(rid)
        cache.ensure(rc, rc.length + n)
        entries.append(StepEntry(rid, [0] * n, []))
        rcs.append(rc)
    ctx, _ = build_step_context(entries, rcs, cache, table_width, dtype, torch.device(DEV), 10, PinnedStaging())
    return ctx, entries, rcs


def feed(mixer, cache, view, dtype, xs, schedule, table_width=64):
    """Run ``mixer`` over the requests ``xs = {id: [T, hidden]}`` cut as ``schedule = [[(id, tokens), ...], ...]`` says (a
    step may hold portions of several requests; ``"end:<id>"`` closes one); returns ``{id: [T, hidden]}``."""
    done = {rid: 0 for rid in xs}
    out = {rid: [] for rid in xs}
    for step in schedule:
        portions = [p for p in step if not isinstance(p, str)]
        if portions:
            ctx, entries, rcs = step_context(cache, dtype, portions, table_width)
            x = torch.cat([xs[rid][done[rid]:done[rid] + n] for rid, n in portions]).to(DEV)
            y = mixer.forward(x, ctx, view, owns_cache=True).cpu()
            at = 0
            for (rid, n), rc in zip(portions, rcs):
                out[rid].append(y[at:at + n])
                at += n
                done[rid] += n
                cache.commit(rc, rc.length + n)
        for p in step:
            if isinstance(p, str):
                cache.close(cache.get(p[4:]))
    return {rid: torch.cat(v) for rid, v in out.items() if v}


def bind_random(part, dtype, seed, scale=0.3, overrides=None):
    """Random tensors for a part (its own names), bound on the device; returns them as float64 on the host."""
    g = torch.Generator().manual_seed(seed)
    t = {k: (torch.randn(v.shape, generator=g) * scale).to(dtype) for k, v in part.tensor_specs().items()}
    for k, v in (overrides or {}).items():
        t[k] = v.to(dtype)
    part.bind({k: v.to(DEV) for k, v in t.items()})
    return {k: v.double() for k, v in t.items()}


# ---------------------------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,dim,offset,dims,interleaved", [(3, 16, 0, 16, False), (2, 32, 0, 8, False), (4, 24, 16, 8, True),
                                                              (1, 40, 0, 40, True), (5, 48, 32, 6, True), (2, 64, 0, 2, False)])
def test_a_span_of_a_head_turns_in_either_pairing(dtype, heads, dim, offset, dims, interleaved):
    """Entries offset .. offset + dims of every head turn by the position, the rest pass unchanged, in place and into a
    second tensor, at positions near 0 and far out."""
    from zedinfer_b200 import ops
    from zedinfer_b200.parts import SpanRotaryPosition
    rule = SpanRotaryPosition(dim, dims, 3000.0, interleaved=interleaved, offset=offset)
    pos = torch.tensor([0, 1, 2, 77, 4095, 30000], dtype=torch.int32)
    x = torch.randn(len(pos), heads, dim).to(dtype)
    span = x[..., offset:offset + dims].double()
    ref = x.double().clone()
    ref[..., offset:offset + dims] = GP.rotate(span.contiguous(), pos, 3000.0, dims, "interleaved" if interleaved else "half")
    xd = x.view(len(pos), heads * dim).to(DEV)
    out = torch.empty_like(xd)
    ops.rotary(xd, out, pos.to(DEV), rule.table(torch.device(DEV)), heads, 0, dim, offset, dims, interleaved)
    tol = 2e-3 if dtype == torch.float32 else 2e-2          # float32 angles far out: 30000 * 2^-24 radians
    assert rel_err(out.view(len(pos), heads, dim), ref) < tol
    assert rel_err(out.view(len(pos), heads, dim)[:4], ref[:4]) < (1e-5 if dtype == torch.float32 else 2e-2)
    ops.rotary(xd, xd, pos.to(DEV), rule.table(torch.device(DEV)), heads, 0, dim, offset, dims, interleaved)
    assert torch.equal(xd.cpu(), out.cpu())
    # outside the span nothing changes, not even by a rounding
    keep = [d for d in range(dim) if not offset <= d < offset + dims]
    assert torch.equal(out.view(len(pos), heads, dim)[..., keep].cpu(), x[..., keep])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("taps,channels", [(4, 20), (3, 300), (2, 7), (1, 12)])
def test_causal_convolution_carries_its_last_inputs_from_step_to_step(dtype, taps, channels):
    """Two requests cut into unequal portions (down to one token, shorter than the kernel's reach) in shared steps equal
    the plain convolution of each whole sequence; a slot that is freed and used again starts from zeros."""
    from zedinfer_b200 import ops
    g = torch.Generator().manual_seed(taps * 100 + channels)
    w = torch.randn(channels, taps, generator=g).to(dtype)
    b = torch.randn(channels, generator=g).to(dtype)
    seqs = {"a": torch.randn(23, channels, generator=g).to(dtype), "b": torch.randn(9, channels, generator=g).to(dtype),
            "c": torch.randn(6, channels, generator=g).to(dtype)}
    ref = {k: GP.silu(GP.causal_conv(v.double(), w.double(), b.double())) for k, v in seqs.items()}
    state = torch.full((2, 5 + (taps - 1) * channels), 7.0, device=DEV)           # 5 entries of something else in front
    slot = {"a": 1, "b": 0, "c": 0}
    schedule = [[("a", 5), ("b", 2)], [("b", 1), ("a", 1)], [("a", 1)], [("a", 2), ("b", 6)], [("a", 14), ("c", 1)], [("c", 5)]]
    done = {k: 0 for k in seqs}
    got = {k: [] for k in seqs}
    for step in schedule:
        for rid, _ in step:
            if done[rid] == 0:
                state[slot[rid], 5:] = 0.0                                        # what opening a request does
        u = torch.cat([seqs[rid][done[rid]:done[rid] + n] for rid, n in step]).to(DEV)
        tok_seg = torch.tensor([i for i, (_, n) in enumerate(step) for _ in range(n)], dtype=torch.int32, device=DEV)
        pos = torch.tensor([done[rid] + j for rid, n in step for j in range(n)], dtype=torch.int32, device=DEV)
        slots = torch.tensor([slot[rid] for rid, _ in step], dtype=torch.int32, device=DEV)
        bounds = torch.empty(len(step), 2, dtype=torch.int32, device=DEV)
        ops.segment_bounds(tok_seg, len(step), bounds)
        out = torch.empty_like(u)
        ops.causal_conv_silu(u, w.to(DEV), b.to(DEV), state, 5, slots, tok_seg, pos, out)
        ops.conv_state_update(u, taps, state, 5, slots, bounds, pos, len(step))
        at = 0
        for rid, n in step:
            got[rid].append(out[at:at + n].cpu())
            at += n
            done[rid] += n
    assert bool((state[:, :5] == 7.0).all())
    for k in seqs:
        assert rel_err(torch.cat(got[k]), ref[k]) < (1e-5 if dtype == torch.float32 else 2e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,vdim,n_state,groups", [(4, 8, 16, 2), (2, 24, 40, 1), (3, 12, 8, 3), (2, 70, 136, 2), (1, 33, 5, 1)])
def test_the_scan_carries_its_state_from_step_to_step(dtype, heads, vdim, n_state, groups):
    """The recurrence over two requests in shared steps, cut into unequal portions, against the plain token-by-token
    recurrence in float64; one head's step size is made large (its state forgets at once) and another's tiny (its state
    remembers the first token for the whole sequence), so that a state that is lost or not carried shows."""
    from zedinfer_b200 import ops
    g = torch.Generator().manual_seed(heads * 1000 + n_state)
    inner, width = heads * vdim, heads * vdim + 2 * groups * n_state
    seqs = {"a": 40, "b": 11}
    xbc = {k: torch.randn(n, width, generator=g).to(dtype) for k, n in seqs.items()}
    dt = {k: torch.randn(n, heads, generator=g).to(dtype) for k, n in seqs.items()}
    dt_bias = torch.randn(heads, generator=g)
    dt_bias[0] = -9.0                                            # step sizes near 1e-4: the first head hardly forgets
    if heads > 1:
        dt_bias[1] = 6.0                                         # and the second forgets within a token
    a_log, d_skip = torch.randn(heads, generator=g) * 0.5, torch.randn(heads, generator=g)

    def plain(x, d):
        t = x.shape[0]
        xs, b, c = x[:, :inner].view(t, heads, vdim), x[:, inner:inner + groups * n_state].view(t, groups, n_state), \
            x[:, inner + groups * n_state:].view(t, groups, n_state)
        step = torch.nn.functional.softplus(d + dt_bias.double(), threshold=1e9)
        y = torch.empty(t, heads, vdim, dtype=F64)
        for a in range(heads):
            s = torch.zeros(n_state, vdim, dtype=F64)
            for i in range(t):
                s = torch.exp(-torch.exp(a_log[a].double()) * step[i, a]) * s + step[i, a] * torch.outer(b[i, a // (heads // groups)], xs[i, a])
                y[i, a] = s.T @ c[i, a // (heads // groups)] + d_skip[a].double() * xs[i, a]
        return y.view(t, inner)

    ref = {k: plain(xbc[k].double(), dt[k].double()) for k in seqs}
    state = torch.zeros(3, inner * n_state + 11, device=DEV)
    slot = {"a": 2, "b": 0}
    schedule = [[("b", 3), ("a", 7)], [("a", 1)], [("a", 1), ("b", 1)], [("a", 2)], [("b", 7), ("a", 29)]]
    done = {k: 0 for k in seqs}
    got = {k: [] for k in seqs}
    par = [t.to(DEV) for t in (dt_bias, a_log, d_skip)]
    for step in schedule:
        x = torch.cat([xbc[rid][done[rid]:done[rid] + n] for rid, n in step]).to(DEV)
        d = torch.cat([dt[rid][done[rid]:done[rid] + n] for rid, n in step]).to(DEV)
        tok_seg = torch.tensor([i for i, (_, n) in enumerate(step) for _ in range(n)], dtype=torch.int32, device=DEV)
        slots = torch.tensor([slot[rid] for rid, _ in step], dtype=torch.int32, device=DEV)
        single = all(n == 1 for _, n in step)
        bounds = None
        if not single:
            bounds = torch.empty(len(step), 2, dtype=torch.int32, device=DEV)
            ops.segment_bounds(tok_seg, len(step), bounds)
        y = torch.empty(x.shape[0], inner, dtype=torch.float32, device=DEV)
        ops.ssm_scan(x, d, *par, state, slots, bounds, y, len(step), heads, vdim, n_state, groups)
        at = 0
        for rid, n in step:
            got[rid].append(y[at:at + n].cpu())
            at += n
            done[rid] += n
    assert bool((state[1] == 0).all()) and bool((state[:, inner * n_state:] == 0).all())     # nobody else's entries touched
    for k in seqs:
        assert rel_err(torch.cat(got[k]), ref[k]) < 1e-5          # float32 inside whatever the inputs' type
    # a row of padding (slot -1) reads zeros and writes nothing
    before = state.clone()
    y = torch.empty(1, inner, dtype=torch.float32, device=DEV)
    ops.ssm_scan(xbc["a"][:1].to(DEV), dt["a"][:1].to(DEV), *par, state, torch.tensor([-1], dtype=torch.int32, device=DEV), None, y,
                 1, heads, vdim, n_state, groups)
    assert torch.equal(state, before) and rel_err(y.cpu(), ref["a"][:1]) < 1e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,vdim,n_state,groups", [(2, 64, 128, 1), (3, 12, 8, 3), (2, 20, 40, 2)])
def test_long_portions_in_stretches_side_by_side_equal_the_plain_walk(dtype, heads, vdim, n_state, groups):
    """Segments of 1, 127, 128, 129 and 700 tokens in one step, one of them continuing from a state that an earlier step
    left and one a row of padding: cut into stretches that run side by side, the outputs and the states left behind agree
    with the plain walk of every segment to float32 rounding."""
    from zedinfer_b200 import ops
    g = torch.Generator().manual_seed(n_state)
    inner, width = heads * vdim, heads * vdim + 2 * groups * n_state
    lens = [1, 127, 128, 129, 700, 1]
    slots = torch.tensor([3, 0, 5, 1, 2, -1], dtype=torch.int32, device=DEV)
    n = sum(lens)
    xbc = (torch.randn(n, width, generator=g) * 0.5).to(dtype).to(DEV)
    dt = torch.randn(n, heads, generator=g).to(dtype).to(DEV)
    par = [t.to(DEV) for t in (torch.randn(heads, generator=g) - 1.0, torch.randn(heads, generator=g) * 0.5, torch.randn(heads, generator=g))]
    tok_seg = torch.tensor([i for i, k in enumerate(lens) for _ in range(k)], dtype=torch.int32, device=DEV)
    bounds = torch.empty(len(lens), 2, dtype=torch.int32, device=DEV)
    ops.segment_bounds(tok_seg, len(lens), bounds)
    start = torch.randn(6, inner * n_state + 3, generator=g).to(DEV)
    out, left = [], []
    for stretchwise in (False, True):
        state = start.clone()
        y = torch.empty(n, inner, dtype=torch.float32, device=DEV)
        ops.ssm_scan(xbc, dt, *par, state, slots, bounds, y, len(lens), heads, vdim, n_state, groups, stretchwise=stretchwise)
        out.append(y.cpu())
        left.append(state.cpu())
    assert rel_err(out[1], out[0].double()) < 2e-5 and rel_err(left[1], left[0].double()) < 2e-5
    assert torch.equal(left[1][4], start[4].cpu()) and torch.equal(left[1][:, inner * n_state:], start[:, inner * n_state:].cpu())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("inner,parts", [(48, 1), (96, 3), (1200, 2), (20, 20)])
def test_gate_then_norm_in_equal_parts(dtype, inner, parts):
    from zedinfer_b200 import ops
    y, z = torch.randn(9, inner) * 3, torch.randn(9, inner + 5).to(dtype)
    w = (1 + 0.1 * torch.randn(inner)).to(dtype)
    out = torch.empty(9, inner, dtype=dtype, device=DEV)
    ops.gated_group_rmsnorm(y.to(DEV), z.to(DEV)[:, 5:], w.to(DEV), parts, 1e-4, out)
    v = y.double() * GP.silu(z[:, 5:].double())
    ref = GP.rms_unit(v.view(9, parts, inner // parts), 1e-4).reshape(9, inner) * w.double()
    assert rel_err(out, ref) < (1e-5 if dtype == torch.float32 else 2e-2)


def test_router_with_sigmoid_scores():
    """The largest scores are chosen (the lowest index among equals) and used as they are, not renormalised."""
    from zedinfer_b200 import ops
    g = torch.Generator().manual_seed(3)
    x, wr = torch.randn(37, 48, generator=g), torch.randn(9, 48, generator=g)
    x[5] = 0.0                                                    # all scores 0.5: the first `top` experts
    for top in (1, 3, 9):
        idx = torch.empty(37, top, dtype=torch.int32, device=DEV)
        wts = torch.empty(37, top, dtype=torch.float32, device=DEV)
        ops.route(x.to(DEV), wr.to(DEV), None, top, idx, wts, score="sigmoid")
        ridx, rw = GP.route(x.double(), wr.double(), top)
        assert torch.equal(idx.cpu().long(), ridx) and rel_err(wts, rw) < 1e-6
        assert idx[5].tolist() == list(range(top)) and bool((wts[5] == 0.5).all())
        logits = (x.double() @ wr.double().T).float().to(DEV)
        idx2, wts2 = torch.empty_like(idx), torch.empty_like(wts)
        ops.route_topk(logits, top, idx2, wts2, score="sigmoid")
        assert torch.equal(idx2, idx) and rel_err(wts2, rw) < 1e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows", [1, 6, 90, 700])
@pytest.mark.parametrize("experts,top,hidden,ff", [(6, 2, 96, 40), (5, 1, 72, 56), (3, 3, 128, 24)])
def test_routed_experts_weighted_on_their_inputs(dtype, rows, experts, top, hidden, ff):
    """Sigmoid scores multiply the experts' inputs; an expert is down(max(up x, 0)^2).  1 and 6 rows take the
    weight-streaming grouped product, 90 the ``wmma`` or tcgen05 one, 700 the tcgen05 one (bfloat16); float32 the SIMT form.
    With the weight on the output instead the result would differ by the weight itself (checked)."""
    from zedinfer_b200.parts import RoutedExperts, StepContext
    part = RoutedExperts(hidden, ff, experts, top, router_bias=False, activation="relu2", score="sigmoid", weight_on="input")
    assert not any(k.endswith("gate") for k in part.tensor_specs()) and "router.b" not in part.tensor_specs()
    # a small router: scores near one half, so that a weight on the output (w) and one on the input (w^2 behind the squared
    # ReLU) are far apart
    small = 0.03 * torch.randn(experts, hidden, generator=torch.Generator().manual_seed(experts))
    t = bind_random(part, dtype, seed=rows + experts, scale=0.25, overrides={"router": small})
    x = torch.randn(rows, hidden, generator=torch.Generator().manual_seed(rows)).to(dtype)
    ctx = StepContext(rows, 1, dtype, torch.device(DEV), None, None, None, [], None, [0], [rows], [0], [-1])
    got = part.forward(x.to(DEV), ctx).cpu()
    f = {"router": {"experts": experts, "top": top}}
    ref = GP.routed_feed_forward(x.double(), f, t, "")
    tol = 2e-5 if dtype == torch.float32 else 4e-2
    errs = (got.double() - ref).abs().amax(dim=1) / max(1.0, float(ref.abs().max()))
    # a close call of the router in bfloat16 moves a whole row
    assert int((errs > tol).sum()) <= (0 if dtype == torch.float32 else max(1, rows // 50)), float(errs.max())
    other = RoutedExperts(hidden, ff, experts, top, router_bias=False, activation="relu2", score="sigmoid", weight_on="output")
    other.bind({k: v.to(dtype).to(DEV) for k, v in t.items()})
    assert rel_err(other.forward(x.to(DEV), ctx), ref) > 0.1


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv,dim,rot,page", [(4, 2, 32, 16, 4), (2, 2, 64, 64, 16), (6, 3, 16, 8, 8), (8, 2, 128, 32, 16), (3, 1, 64, 2, 24)])
def test_attention_whose_values_are_its_keys_with_a_term_of_one_below(dtype, heads, kv, dim, rot, page):
    """The mixer alone over portions and single tokens of two requests against the plain whole-sequence function.  Keys
    are made short, so that the sum of exp(s) stays near the added 1 and leaving the 1 out would double the output."""
    from zedinfer_b200.cache import CacheManager
    from zedinfer_b200.config import PartSpec
    from zedinfer_b200.parts import AttentionMixer
    hidden = 80
    mixer = AttentionMixer(hidden, heads, kv, dim, PartSpec("rope_span", {"head_dim": dim, "dims": rot, "theta": 2000.0}),
                           qkv_bias=False, scale=0.3, value_from_key=True, unit_sink=True, names={"q": "q", "k": "k", "o": "o"})
    assert sorted(mixer.tensor_specs()) == ["k", "o", "q"]
    t = bind_random(mixer, dtype, seed=dim + heads, scale=0.08)
    cache = CacheManager([(0, mixer.cache_need())], page, max_requests=2)
    cache.allocate_device(40, dtype, DEV)
    view = cache.view_for_call(0)
    g = torch.Generator().manual_seed(7)
    xs = {"a": torch.randn(61, hidden, generator=g).to(dtype), "b": torch.randn(19, hidden, generator=g).to(dtype)}
    schedule = [[("a", 9), ("b", 2)], [("b", 1), ("a", 1)], [("a", 1)], [("a", 33), ("b", 15)], [("b", 1)], [("a", 2)], [("a", 15)]]
    got = feed(mixer, cache, view, dtype, xs, schedule)
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "scale": 0.3, "rot": {"base": 2000.0, "dims": rot}}
    for rid, x in xs.items():
        ref = GP.attention_mixer(x.double(), torch.arange(x.shape[0]), m, t, "")
        assert rel_err(got[rid], ref) < (2e-5 if dtype == torch.float32 else 3e-2), rid
    # the weights do not sum to one: with the 1 left out the first token would return its own key whole
    x0 = xs["a"][:1].double()
    k0 = (x0 @ t["k"].T).view(kv, dim).repeat_interleave(heads // kv, 0).reshape(1, -1) @ t["o"].T
    assert float((got["a"][:1].double() - k0).abs().max()) > 0.2 * float(k0.abs().max())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,dim,rd,vdim,rank,q_rank,rot", [(3, 16, 8, 24, 24, 40, 8), (4, 32, 16, 16, 48, 24, 16), (2, 48, 16, 40, 112, 64, 16),
                                                               (1, 24, 6, 12, 20, 16, 4), (5, 8, 32, 8, 96 + 8, 12, 32)])
def test_latent_attention_with_a_turned_key_part_a_query_latent_and_a_gate(dtype, heads, dim, rd, vdim, rank, q_rank, rot):
    """The mixer alone over portions and single tokens of two requests against the plain whole-sequence function: cache
    rows of 32 (general kernel), 64 and 128 (tensor-core kernels), 26 (padded to 32) and 136 entries."""
    from zedinfer_b200.cache import CacheManager
    from zedinfer_b200.parts import LatentAttentionMixer
    hidden, eps = 88, 1e-5
    mixer = LatentAttentionMixer(hidden, heads, dim, vdim, rank, eps, scale=0.2, window=None, sinks=False, rot_dim=rd, rot_dims=rot,
                                 rot_base=500.0, rot_interleaved=True, q_rank=q_rank, out_gate=True)
    assert sorted(mixer.tensor_specs()) == ["dkv", "dkv.norm", "dq", "dq.norm", "g", "o", "uk", "uq", "uv"]
    t = bind_random(mixer, dtype, seed=rank + heads, scale=0.3)
    cache = CacheManager([(0, mixer.cache_need())], 16, max_requests=2)
    cache.allocate_device(12, dtype, DEV)
    view = cache.view_for_call(0)
    g = torch.Generator().manual_seed(11)
    xs = {"a": torch.randn(70, hidden, generator=g).to(dtype), "b": torch.randn(21, hidden, generator=g).to(dtype)}
    schedule = [[("a", 7), ("b", 2)], [("b", 1), ("a", 1)], [("a", 1)], [("a", 30), ("b", 17)], [("b", 1)], [("a", 2)], [("a", 29)]]
    got = feed(mixer, cache, view, dtype, xs, schedule)
    m = {"heads": heads, "dim": dim, "rot_dim": rd, "vdim": vdim, "kv_rank": rank, "q_rank": q_rank, "scale": 0.2,
         "rot": {"base": 500.0, "dims": rot}}
    for rid, x in xs.items():
        ref = GP.latent_attention_mixer(x.double(), torch.arange(x.shape[0]), m, t, "", eps)
        assert rel_err(got[rid], ref) < (3e-5 if dtype == torch.float32 else 4e-2), rid


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,vdim,n_state,groups,taps,parts", [(6, 8, 16, 2, 4, 3), (2, 24, 40, 1, 2, 1), (3, 12, 8, 3, 1, 1), (4, 20, 136, 2, 3, 4)])
def test_state_space_mixer_over_portions_and_slots_used_again(dtype, heads, vdim, n_state, groups, taps, parts):
    """The mixer alone: two requests in shared steps, cut down to single tokens, then a third request in the slot the
    second gave back (it must start from zeros, not from what the slot last held)."""
    from zedinfer_b200.cache import CacheManager
    from zedinfer_b200.parts import Mamba2Mixer
    hidden, eps = 64, 1e-5
    mixer = Mamba2Mixer(hidden, heads, vdim, n_state, groups, taps, parts, eps)
    over = {"A_log": torch.linspace(-1.0, 1.0, heads), "dt_bias": torch.linspace(-4.0, 2.0, heads), "D": torch.ones(heads),
            "norm": 1 + 0.1 * torch.randn(heads * vdim)}
    t = bind_random(mixer, dtype, seed=n_state, scale=0.3, overrides=over)
    cache = CacheManager([(0, mixer.cache_need())], 16, max_requests=2)
    cache.allocate_device(1, dtype, DEV)
    view = cache.view_for_call(0)
    assert view.kind == "state" and view.tensor.shape == (2, heads * vdim * n_state + (taps - 1) * (heads * vdim + 2 * groups * n_state))
    g = torch.Generator().manual_seed(5)
    xs = {"a": torch.randn(45, hidden, generator=g).to(dtype), "b": torch.randn(10, hidden, generator=g).to(dtype),
          "c": torch.randn(12, hidden, generator=g).to(dtype)}
    schedule = [[("a", 6), ("b", 2)], [("b", 1), ("a", 1)], [("a", 1)], [("a", 2), ("b", 7), "end:b"], [("c", 3), ("a", 20)],
                [("c", 1), ("a", 1)], [("c", 8), ("a", 14)]]
    got = feed(mixer, cache, view, dtype, xs, schedule)
    m = {"heads": heads, "vdim": vdim, "state": n_state, "groups": groups, "conv": taps, "norm_groups": parts}
    for rid, x in xs.items():
        ref = GP.mamba2_mixer(x.double(), m, t, "", eps)
        assert rel_err(got[rid], ref) < (3e-5 if dtype == torch.float32 else 5e-2), rid


def _one_key_answers(total, asks, dims, base, layout, gain=25.0):
    """Key parts and query parts (``[total, dims]`` each, zero almost everywhere) such that the query at position P of
    ``asks = {P: j}`` scores ``8 * gain`` against the key at j and clearly less against its neighbours j - 1 and j + 1, which
    carry the same part: the query is that part turned by j - P positions, so that after both are turned by their own
    positions they are aligned.  Every other key's part is zero."""
    raw = torch.zeros(dims, dtype=F64)
    if layout == "interleaved":
        raw[0::2] = 1.0
    else:
        raw[:dims // 2] = 1.0
    keys, queries = torch.zeros(total, dims, dtype=F64), torch.zeros(total, dims, dtype=F64)
    for p_query, j in asks.items():
        for d in (-1, 0, 1):
            keys[j + d] = raw * (dims // 2 / 8.0) ** -0.5
        queries[p_query] = gain * GP.rotate(keys[j][None], torch.tensor([j - p_query]), base, dims, layout)[0]
    return keys, queries


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rank,rd,page", [(16, 16, 16), (48, 16, 8), (112, 16, 16), (40, 8, 4)])
def test_a_far_key_among_hundreds_answers_through_the_turned_part(dtype, rank, rd, page):
    """Latent attention, one head, plain parts of queries and keys zero: a score rests on the turned parts alone.  Only
    the chosen key answers, among 600 and next to two neighbours with the same part, if queries and keys are turned by
    their own positions with the right pairing and frequencies; asked from inside a prompt portion and by a token
    decoded alone, for a key far back and for keys on both sides of a page border."""
    from zedinfer_b200.cache import CacheManager
    from zedinfer_b200.parts import LatentAttentionMixer
    dim, vdim, base, total = 8, 8, 50.0, 600
    hidden = rank + 2 * rd                               # x = [what the latent is made of | query part | key part]
    mixer = LatentAttentionMixer(hidden, 1, dim, vdim, rank, 1e-6, scale=1.0, window=None, sinks=False, rot_dim=rd,
                                 rot_base=base, rot_interleaved=True, q_rank=None, out_gate=False)
    wq, wdkv = torch.zeros(dim + rd, hidden), torch.zeros(rank + rd, hidden)
    wq[dim:, rank:rank + rd] = torch.eye(rd)
    wdkv[:rank, :rank] = torch.eye(rank)
    wdkv[rank:, rank + rd:] = torch.eye(rd)
    tens = {"q": wq, "dkv": wdkv, "dkv.norm": torch.ones(rank), "uk": torch.zeros(dim, rank), "uv": torch.eye(vdim, rank),
            "o": torch.eye(hidden, vdim)}
    mixer.bind({k: v.to(dtype).to(DEV) for k, v in tens.items()})
    cache = CacheManager([(0, mixer.cache_need())], page, max_requests=1)
    cache.allocate_device(total // page + 2, dtype, DEV)
    view = cache.view_for_call(0)
    asks = {599: 37, 450: 5, 300: 2 * page * 8 - 1, 520: 2 * page * 8 + 3}      # decoded alone; inside portions
    keys, queries = _one_key_answers(total, asks, rd, base, "interleaved")
    marks = torch.randn(total, rank, generator=torch.Generator().manual_seed(rank)).double()
    x = torch.cat([marks, queries, keys], dim=1).to(dtype)
    out = feed(mixer, cache, view, dtype, {"r": x}, [[("r", 200)], [("r", 399)], [("r", 1)]], table_width=160)["r"]
    xd = x.double()
    c = GP.rms_unit(xd[:, :rank], 1e-6)
    pos = torch.arange(total)
    s = GP.rotate(xd[:, rank:rank + rd].contiguous(), pos, base, rd, "interleaved") @ GP.rotate(xd[:, rank + rd:].contiguous(), pos, base, rd, "interleaved").T
    w = GP.causal_weights(s[None], sink_one=False)[0]
    for p_query, j in asks.items():
        assert float(w[p_query, j]) > 0.99                       # the test's own premise
        assert rel_err(out[p_query, :vdim], c[j, :vdim]) < (1e-3 if dtype == torch.float32 else 3e-2), (p_query, j)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dim,rot,page", [(32, 16, 16), (64, 32, 8), (128, 64, 16), (48, 16, 4)])
def test_a_far_key_returns_itself_unturned(dtype, dim, rot, page):
    """Attention whose values are its keys, one head: queries live in the turned span only, keys carry marks outside it.
    The chosen key answers (rotate-half pairing, its own position) and what comes back is that key as projected, its
    span not turned, times exp(s) / (1 + exp(s) + ...)."""
    from zedinfer_b200.cache import CacheManager
    from zedinfer_b200.config import PartSpec
    from zedinfer_b200.parts import AttentionMixer
    base, total = 300.0, 600
    hidden = 2 * rot + (dim - rot)                       # x = [query span | key span | key marks]
    mixer = AttentionMixer(hidden, 1, 1, dim, PartSpec("rope_span", {"head_dim": dim, "dims": rot, "theta": base}),
                           qkv_bias=False, scale=1.0, value_from_key=True, unit_sink=True, names={"q": "q", "k": "k", "o": "o"})
    wq, wk = torch.zeros(dim, hidden), torch.zeros(dim, hidden)
    wq[:rot, :rot] = torch.eye(rot)
    wk[:rot, rot:2 * rot] = torch.eye(rot)
    wk[rot:, 2 * rot:] = torch.eye(dim - rot)
    mixer.bind({k: v.to(dtype).to(DEV) for k, v in {"q": wq, "k": wk, "o": torch.eye(hidden, dim)}.items()})
    cache = CacheManager([(0, mixer.cache_need())], page, max_requests=1)
    cache.allocate_device(total // page + 2, dtype, DEV)
    view = cache.view_for_call(0)
    asks = {599: 37, 450: 5, 300: 2 * page * 8 - 1, 520: 2 * page * 8 + 3}
    keys, queries = _one_key_answers(total, asks, rot, base, "half")
    marks = torch.randn(total, dim - rot, generator=torch.Generator().manual_seed(dim)).double()
    x = torch.cat([queries, keys, marks], dim=1).to(dtype)
    out = feed(mixer, cache, view, dtype, {"r": x}, [[("r", 200)], [("r", 399)], [("r", 1)]], table_width=160)["r"]
    xd = x.double()
    pos = torch.arange(total)
    s = GP.rotate(xd[:, :rot].contiguous(), pos, base, rot, "half") @ GP.rotate(xd[:, rot:2 * rot].contiguous(), pos, base, rot, "half").T
    w = GP.causal_weights(s[None], sink_one=True)[0]
    k_plain = xd[:, rot:]                                  # a key as projected: [span, not turned | marks]
    for p_query, j in asks.items():
        assert float(w[p_query, j]) > 0.99
        assert rel_err(out[p_query, :dim], k_plain[j]) < (1e-3 if dtype == torch.float32 else 3e-2), (p_query, j)
    # a token none of whose keys scores: the weights are 1 / (1 + n) each, not 1 / n
    quiet = 100
    assert rel_err(out[quiet, :dim], k_plain[:quiet + 1].sum(0) * (w[quiet, 0])) < (1e-3 if dtype == torch.float32 else 3e-2)
    assert abs(float(w[quiet, 0]) - 1.0 / (quiet + 2)) < 1e-12


# ---------------------------------------------------------------------------------------------
# whole models
# ---------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("gibalorn_models")
    return {name: GT.make_model_dir(root, name) for name in GT.CONFIGS}


def make_requests(cfg, lengths, seed):
    rng = random.Random(seed)
    return {f"r{i}": [rng.randrange(cfg["vocab"]) for _ in range(n)] for i, n in enumerate(lengths)}


_plain_cache = {}


def variant(name, dtype):
    """bfloat16 runs the models whose routers choose every expert (``gibalorn_tiny.all_chosen``); the choice among experts
    is compared in float32, where no close call can turn."""
    return name if dtype == "float32" else name + "x"


def expected_logits(model_dir, requests):
    if model_dir not in _plain_cache:
        _plain_cache[model_dir] = GP.read_model(model_dir, F64)
    cfg, w = _plain_cache[model_dir]
    return {rid: GP.forward(cfg, w, toks).float() for rid, toks in requests.items()}


def judge(got, exp, dtype):
    """float32: every position within the tolerance.  bfloat16: rounding errors have a tail (the mean error of these models
    is a quarter of the tolerance, single positions reach three times it, the same in whatever way the work is cut): at
    most 2 % of the positions may be beyond the tolerance, none beyond four times it."""
    tol = tol_for(dtype)
    errs = {key: float((row - exp[key[0]][key[1]]).abs().max()) / max(1.0, float(exp[key[0]].abs().max()))
            for key, row in got.items()}
    over = sorted((k for k, e in errs.items() if not e <= tol), key=lambda k: (str(k[0]), k[1]))
    allowed = 0 if dtype == "float32" else max(1, len(errs) // 50)
    assert len(over) <= allowed, f"{len(over)} of {len(errs)} positions beyond {tol}; first {over[0]} with {errs[over[0]]}"
    assert all(e <= 4 * tol for e in errs.values()), max(errs.values())


LENGTHS = {"A": [7, 13, 95, 45], "B": [1, 17, 120, 64], "C": [110, 5, 60], "D": [50, 2, 61], "E": [40, 3, 70], "F": [33, 1, 52]}
PAGES = {"A": 4, "B": 16, "C": 16, "D": 8, "E": 8, "F": 8}


def test_the_run_order_and_the_caches_of_every_pass(models):
    """Layers inside the loop appear once per pass, each appearance with a cache or a state of its own; the embedding is
    added again at the first layer of every pass but the first."""
    from zedinfer_b200.config.registry import load_model_config
    from zedinfer_b200.engine.model import Model
    _, cfg, spec = load_model_config(models["A"])
    assert [(c.layer, c.add_embedding) for c in spec.schedule] == [(0, False), (1, False), (2, False), (1, True), (2, False), (3, False)]
    assert [c.layer for c in spec.schedule] == GP.run_order(GT.GB_A)
    needs = Model(spec).cache_needs()
    assert [k for k, _ in needs] == [0, 1, 2, 3, 4, 5] and all(c.cache_of is None for c in spec.schedule)
    _, _, spec_c = load_model_config(models["C"])
    assert [c.add_embedding for c in spec_c.schedule] == [False, False, False, True, False, False, True, False, False]
    _, _, spec_d = load_model_config(models["D"])
    assert not any(c.add_embedding for c in spec_d.schedule) and len(spec_d.schedule) == 2


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E", "F"])
@pytest.mark.parametrize("family", ["whole", "tail", "chunks", "mixed"])
def test_cuts_match_plain(models, name, dtype, family):
    """Whole prompts; a tail decoded token by token; portions down to two tokens; mixed batches of unequal requests in a
    pool so small that pages and state slots are handed out again."""
    from zedinfer_b200.engine.core import EngineCore
    cfg, _ = GT.CONFIGS[name]
    model = models[variant(name, dtype)]
    requests = make_requests(cfg, LENGTHS[name] + ([64, 31, 77] if family == "mixed" else []), seed=5)
    if family == "tail":
        steps = traces.tail_decode(requests, tail=40)
    else:
        steps = {"whole": traces.whole, "chunks": traces.chunks, "mixed": traces.mixed}[family](requests)
    page = PAGES[name]
    need = traces.max_live_tokens(steps, round_to=page)
    core = EngineCore(model, dtype, page_size=page, num_pages=max(1, need // page), max_requests=4)
    got = run_trace(core, steps)
    core.check_kernels()
    judge(got, expected_logits(model, requests), dtype)
    assert core.cache.num_live == 0 and all(g.pool.num_used == 0 for g in core.cache.groups)
    assert core.cache.slots.num_free_slots == core.cache.slots.num_slots           # 4 where the model keeps state, else none


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "float32"), ("B", "bfloat16"), ("C", "bfloat16")])
def test_many_decoding_requests_with_and_without_graphs(models, name, dtype, graphs):
    """Steps as a scheduler makes them: up to 12 decoding requests beside one prompt portion, then decode-only steps whose
    number of rows falls to one; with graphs the decode-only steps replay captured buckets whose rows of padding hold no
    state slot, and mixed steps are captured too."""
    from zedinfer_b200.engine.core import EngineCore
    cfg, _ = GT.CONFIGS[name]
    rng = random.Random(8)
    requests = make_requests(cfg, [rng.randint(40, 90) for _ in range(15)], seed=3)
    steps = traces.decode_heavy(requests, seed=4, max_live=12, tail=(8, 30), portion=32)
    need = traces.max_live_tokens(steps, round_to=16)
    model = models[variant(name, dtype)]
    core = EngineCore(model, dtype, page_size=16, num_pages=need // 16, max_requests=16, cuda_graphs=graphs)
    core.GPU_BOUND_RATIO = float("inf")
    assert core.capture_safe, core.capture_blockers
    got = run_trace(core, steps)
    core.check_kernels()
    judge(got, expected_logits(model, requests), dtype)
    if graphs:
        assert core._decode_graphs
    assert core.cache.num_live == 0 and all(g.pool.num_used == 0 for g in core.cache.groups)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_the_first_tokens(models, dtype):
    """One token, two tokens, and a request decoded for 260 steps from a prompt of three: the recurrent state and the
    convolution's ring go through hundreds of single-token steps."""
    from zedinfer_b200.engine.core import EngineCore
    cfg, _ = GT.CONFIGS["A"]
    requests = make_requests(cfg, [1, 2, 263], seed=9)
    steps = traces.tail_decode(requests, tail=260)
    model = models[variant("A", dtype)]
    core = EngineCore(model, dtype, page_size=4, num_pages=80, max_requests=2)
    got = run_trace(core, steps)
    judge(got, expected_logits(model, requests), dtype)


@pytest.mark.parametrize("name", ["A", "C", "D"])
def test_float32_is_the_same_however_it_is_cut(models, name):
    """The same positions through four different schedules: the same bits (every float32 sum of the design has one
    order, which depends on constants alone; the recurrence runs token by token whatever the portions)."""
    from zedinfer_b200.engine.core import EngineCore
    cfg, _ = GT.CONFIGS[name]
    requests = make_requests(cfg, [90, 41], seed=2)
    runs = []
    for steps in (traces.whole(requests), traces.tail_decode(requests, tail=20), traces.chunks(requests), traces.mixed(requests)):
        core = EngineCore(models[name], "float32", page_size=16, num_pages=40, max_requests=4)
        runs.append(run_trace(core, steps))
    for other in runs[1:]:
        assert all(torch.equal(other[k], runs[0][k]) for k in runs[0])


@pytest.mark.parametrize("name,graphs", [("A", False), ("A", True), ("B", True), ("C", False)])
def test_greedy_generation_equals_plain(models, name, graphs):
    """Through the Python entry point and its scheduler: prompts in portions of five, a pool of pages and three state
    slots that the requests fill again, greedy tokens equal to the plain implementation's."""
    from zedinfer_b200 import GenerationConfig, SchedulerConfig
    from zedinfer_b200.engine import InferenceEngine
    cfg, _ = GT.CONFIGS[name]
    rng = random.Random(4)
    prompts = [[rng.randrange(cfg["vocab"]) for _ in range(n)] for n in (9, 23, 1, 14, 6)]
    engine = InferenceEngine.create(models[name], SchedulerConfig(num_kv_pages=30, kv_block_size=4, max_batch_requests=3,
                                                                  max_prefill_tokens=5, cuda_graphs=graphs),
                                    dtype="float32")
    results = engine.generate_batch(prompts, GenerationConfig(max_new_tokens=20, ignore_eos=True))
    pcfg, w = GP.read_model(models[name], F64)
    for p, r in zip(prompts, results):
        assert r.finish_reason == "length"
        assert r.output_ids == GP.greedy(pcfg, w, p, 20)
    st = engine.cache_stats()
    assert st["live_requests"] == 0 and st["free_pages"] == st["pages_per_group"]


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_trace_program_on_a_gibalorn_folder(models, tmp_path, dtype):
    cfg, _ = GT.CONFIGS["B"]
    requests = make_requests(cfg, [70, 9, 33, 50, 21], seed=6)
    steps = traces.mixed(requests, seed=1)
    need = traces.max_live_tokens(steps, round_to=64)
    out = tmp_path / "out"
    model = models[variant("B", dtype)]
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model, "--dtype", dtype,
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
    judge(got, expected_logits(model, requests), dtype)


def test_command_line_programs_take_the_design(tmp_path, capsys):
    """From a bare config.json with weights drawn on the device: the bench program, continuous batching, and the
    consistency program, which returns 0 only if every float32 logit is the same bit pattern however the work is cut."""
    from zedinfer_b200.cli import batch_bench, bench, consistency
    path = tmp_path / "config.json"
    path.write_text(json.dumps(GT.GB_A))
    common = [str(path), "--random-weights", "7", "--kv-pages", "40", "--max-seq-len", "128"]
    assert bench.main(common + ["-p", "24", "-d", "5", "-r", "1"]) == 0
    out = capsys.readouterr().out
    assert "Prefill:" in out and "Decode :" in out
    assert batch_bench.main(common + ["-b", "5", "-p", "6", "--prefill-len-max", "40", "-d", "7", "-r", "1",
                                      "--warmup-rounds", "1", "--max-prefill-tokens", "16"]) == 0
    assert "5 requests, 35 tokens generated" in capsys.readouterr().out
    assert consistency.main([str(path), "--random-weights", "5", "--tokens", "120", "--requests", "5"]) == 0
    lines = [json.loads(l) for l in capsys.readouterr().out.strip().splitlines()]
    assert {(l["dtype"], l["mode"]) for l in lines} >= {("float32", "tail"), ("float32", "portions"), ("float32", "mixed"),
                                                        ("bfloat16", "mixed"), ("bfloat16", "whole")}
    assert all(l["values_not_bit_equal"] == 0 for l in lines if l["dtype"] == "float32")
