"""A plain, slow implementation of the Gibalorn forward pass: whole sequences, no cache, one function per mechanism,
on the CPU in float64 (or float32).  It shares no code with ``zedinfer_b200``: it reads ``config.json`` with ``json``
and ``model.safetensors`` with its own few lines.

The design in this file's notation (``x`` the residual stream, ``N(v) = v / sqrt(mean(v^2) + eps)``):

    e_t = E[token_t];  x = e
    run order:  layers a .. b-1 are run r times in a row with the same weights (``loop``), then the rest once;
                before every pass but the first, x += e
    per layer:  x += mixer(N(x) * w1);   x += ff(N(x) * w2)      (ff may be absent)
    rotation R(v, t; base, d): the pair (v_lo, v_hi) -> (v_lo cos a - v_hi sin a, v_hi cos a + v_lo sin a),
                a = t * base^(-2i/d); "half": lo = i, hi = i + d/2; "interleaved": lo = 2i, hi = 2i + 1; only the
                first d entries of a vector turn

    attention:          q = Wq h, k = Wk h, v = k (unrotated);  q, k turned (half) on their first rot.dims entries
                        s_tj = scale * q_t . k_j (j <= t),  p_tj = exp(s_tj) / (1 + sum_j' exp(s_tj'))
                        out = Wo concat(sum_j p_tj v_j)         query head a reads key head a // (H / G)
    latent attention:   cq = N(Wdq h) * gq,  q = Wuq cq, per head [dim plain | rot_dim turned (interleaved)]
                        [c' | kr] = Wdkv h,  c = N(c') * gkv,  kr turned (interleaved), shared by all heads
                        k_a = Wuk_a c, v_a = Wuv_a c,  s = scale * (q_plain . k_a + q_rot . kr),  softmax over j <= t
                        out = Wo (concat_a(sum_j p v_a) * sigmoid(Wg h))
    mamba2:             [z | xs | B | C | dt] = Win h;  [xs | B | C] through a causal per-channel convolution with bias
                        and silu;  dt = softplus(dt + dt_bias);  per head a (group a // (H / G)):
                        S_t = exp(-exp(A_log_a) dt_t) S_(t-1) + dt_t B_t xs_t^T,   y_t = S_t^T C_t + D_a xs_t
                        out = Wo (Ngroups(y * silu(z)) * g)
    routed ff:          s = sigmoid(Wr h); the ``top`` largest s (lowest index wins a tie);
                        out = sum_e Wdown_e relu(Wup_e (s_e h))^2
    logits = head (N(x) * wf)
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional

import torch


# ---------------------------------------------------------------------------------------------
# files
# ---------------------------------------------------------------------------------------------
def read_safetensors(path: str, dtype=torch.float64) -> Dict[str, torch.Tensor]:
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    kinds = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16, "I32": torch.int32, "F64": torch.float64}
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        b, e = info["data_offsets"]
        t = torch.frombuffer(bytearray(data[b:e]), dtype=kinds[info["dtype"]]).reshape(info["shape"])
        out[name] = t.to(dtype) if t.is_floating_point() else t.clone()
    return out


def read_model(model_dir: str, dtype=torch.float64):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(model_dir, "model.safetensors"), dtype)


# ---------------------------------------------------------------------------------------------
# mechanisms, one function each
# ---------------------------------------------------------------------------------------------
def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return rms_unit(x, eps) * w


def rotate(v: torch.Tensor, positions: torch.Tensor, base: float, dims: int, layout: str) -> torch.Tensor:
    """``v [T, ..., D]``: the first ``dims`` entries of the last axis turn by the token's position, the rest pass."""
    half = dims // 2
    i = torch.arange(half, dtype=v.dtype)
    freq = torch.pow(torch.tensor(base, dtype=v.dtype), -2.0 * i / dims)
    ang = positions.to(v.dtype)[:, None] * freq[None, :]                  # [T, half]
    shape = [v.shape[0]] + [1] * (v.dim() - 2) + [half]
    cos, sin = torch.cos(ang).view(shape), torch.sin(ang).view(shape)
    out = v.clone()
    if layout == "half":
        lo, hi = v[..., :half], v[..., half:dims]
        out[..., :half] = lo * cos - hi * sin
        out[..., half:dims] = hi * cos + lo * sin
    elif layout == "interleaved":
        lo, hi = v[..., 0:dims:2], v[..., 1:dims:2]
        out[..., 0:dims:2] = lo * cos - hi * sin
        out[..., 1:dims:2] = hi * cos + lo * sin
    else:
        raise ValueError(layout)
    return out


def causal_weights(scores: torch.Tensor, sink_one: bool) -> torch.Tensor:
    """``scores [H, T, T]`` (query, key) -> weights; key j is visible to query t when j <= t.  ``sink_one``: a term
    exp(0) joins the denominator."""
    t = scores.shape[-1]
    mask = torch.ones(t, t, dtype=torch.bool).tril()
    s = scores.masked_fill(~mask, float("-inf"))
    m = s.max(dim=-1, keepdim=True).values
    if sink_one:
        m = torch.clamp(m, min=0.0)
    e = torch.exp(s - m)
    den = e.sum(dim=-1, keepdim=True)
    if sink_one:
        den = den + torch.exp(-m)
    return e / den


def attention_mixer(h: torch.Tensor, positions: torch.Tensor, m: dict, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    t = h.shape[0]
    heads, groups, dim = m["heads"], m["kv_heads"], m["dim"]
    q = (h @ w[p + "q"].T).view(t, heads, dim)
    k = (h @ w[p + "k"].T).view(t, groups, dim)
    v = k                                                                  # the values are the unrotated keys
    q = rotate(q, positions, m["rot"]["base"], m["rot"]["dims"], "half")
    kr = rotate(k, positions, m["rot"]["base"], m["rot"]["dims"], "half")
    per = heads // groups
    out = torch.empty(t, heads, dim, dtype=h.dtype)
    for a in range(heads):
        g = a // per
        s = (q[:, a] @ kr[:, g].T)[None] * m["scale"]
        pr = causal_weights(s, sink_one=True)[0]
        out[:, a] = pr @ v[:, g]
    return out.reshape(t, heads * dim) @ w[p + "o"].T


def latent_attention_mixer(h: torch.Tensor, positions: torch.Tensor, m: dict, w: Dict[str, torch.Tensor], p: str,
                           eps: float) -> torch.Tensor:
    t = h.shape[0]
    heads, dim, rd, vd, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    cq = rms_norm(h @ w[p + "dq"].T, w[p + "dq.norm"], eps)
    q = (cq @ w[p + "uq"].T).view(t, heads, dim + rd)
    q_plain, q_rot = q[..., :dim], rotate(q[..., dim:].contiguous(), positions, m["rot"]["base"], m["rot"]["dims"], "interleaved")
    ckr = h @ w[p + "dkv"].T
    c = rms_norm(ckr[:, :rank], w[p + "dkv.norm"], eps)
    kr = rotate(ckr[:, rank:].contiguous(), positions, m["rot"]["base"], m["rot"]["dims"], "interleaved")
    k = (c @ w[p + "uk"].T).view(t, heads, dim)
    v = (c @ w[p + "uv"].T).view(t, heads, vd)
    out = torch.empty(t, heads, vd, dtype=h.dtype)
    for a in range(heads):
        s = (q_plain[:, a] @ k[:, a].T + q_rot[:, a] @ kr.T)[None] * m["scale"]
        pr = causal_weights(s, sink_one=False)[0]
        out[:, a] = pr @ v[:, a]
    gate = torch.sigmoid(h @ w[p + "g"].T)
    return (out.reshape(t, heads * vd) * gate) @ w[p + "o"].T


def silu(x: torch.Tensor) -> torch.Tensor:
    return x * torch.sigmoid(x)


def causal_conv(u: torch.Tensor, kernel: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """``u [T, C]``, ``kernel [C, taps]`` whose last column meets the current token; zeros before the start."""
    t, c = u.shape
    taps = kernel.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, c, dtype=u.dtype), u], dim=0)
    out = bias[None, :].expand(t, c).clone()
    for j in range(taps):
        out = out + padded[j:j + t] * kernel[:, j][None, :]
    return out


def mamba2_mixer(h: torch.Tensor, m: dict, w: Dict[str, torch.Tensor], p: str, eps: float) -> torch.Tensor:
    t = h.shape[0]
    heads, vd, n, groups = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = heads * vd
    proj = h @ w[p + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * groups * n], proj[:, 2 * inner + 2 * groups * n:]
    xbc = silu(causal_conv(xbc, w[p + "conv"], w[p + "conv.b"]))
    xs = xbc[:, :inner].view(t, heads, vd)
    b = xbc[:, inner:inner + groups * n].view(t, groups, n)
    c = xbc[:, inner + groups * n:].view(t, groups, n)
    dt = torch.nn.functional.softplus(dt + w[p + "dt_bias"][None, :], threshold=1e9)
    decay = torch.exp(-torch.exp(w[p + "A_log"])[None, :] * dt)            # [T, heads]
    per = heads // groups
    y = torch.empty(t, heads, vd, dtype=h.dtype)
    for a in range(heads):
        g = a // per
        s = torch.zeros(n, vd, dtype=h.dtype)
        for i in range(t):
            s = decay[i, a] * s + dt[i, a] * torch.outer(b[i, g], xs[i, a])
            y[i, a] = s.T @ c[i, g] + w[p + "D"][a] * xs[i, a]
    y = y.reshape(t, inner) * silu(z)
    ng = m["norm_groups"]
    y = rms_unit(y.view(t, ng, inner // ng), eps).reshape(t, inner) * w[p + "norm"]
    return y @ w[p + "o"].T


def route(h: torch.Tensor, w_router: torch.Tensor, top: int):
    """(indices ``[T, top]`` by falling score, the lowest index first among equals; scores ``[T, top]``)."""
    s = torch.sigmoid(h @ w_router.T)
    order = torch.sort(s, dim=-1, descending=True, stable=True).indices[:, :top]
    return order, torch.gather(s, 1, order)


def route_margin(h: torch.Tensor, w_router: torch.Tensor, top: int) -> torch.Tensor:
    """Per token, how far the last chosen expert's logit lies above the first one left out (infinite when all are chosen):
    a choice with a small margin is a close call that rounding may turn the other way."""
    z = torch.sort(h @ w_router.T, dim=-1, descending=True).values
    if top >= z.shape[1]:
        return torch.full((h.shape[0],), float("inf"), dtype=h.dtype)
    return z[:, top - 1] - z[:, top]


def routed_feed_forward(h: torch.Tensor, f: dict, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    idx, wts = route(h, w[p + "router"], f["router"]["top"])
    out = torch.zeros_like(h)
    for i in range(h.shape[0]):
        for j in range(idx.shape[1]):
            e = int(idx[i, j])
            u = torch.relu(w[f"{p}e{e}.up"] @ (wts[i, j] * h[i]))
            out[i] = out[i] + w[f"{p}e{e}.down"] @ (u * u)
    return out


# ---------------------------------------------------------------------------------------------
# the model
# ---------------------------------------------------------------------------------------------
def run_order(cfg: dict) -> List[int]:
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b, r = loop["start"], loop["stop"], loop["times"]
    return list(range(a)) + list(range(a, b)) * r + list(range(b, n))


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], layer_outputs: Optional[list] = None,
            margins: Optional[list] = None) -> torch.Tensor:
    """Logits ``[T, vocab]`` of every position of one sequence.  ``layer_outputs`` receives the residual stream after every
    layer run, ``margins`` the router's margin per token (:func:`route_margin`) of every routed layer run."""
    eps = cfg["norm"]["eps"]
    dtype = w["embed"].dtype
    positions = torch.arange(len(tokens))
    e = w["embed"][torch.tensor(tokens, dtype=torch.long)]
    x = e.clone()
    loop = cfg.get("loop")
    order = run_order(cfg)
    first_pass_seen = False
    for pos, i in enumerate(order):
        if loop and i == loop["start"] and loop["stop"] > loop["start"]:
            if first_pass_seen:
                x = x + e
            first_pass_seen = True
        layer = cfg["layers"][i]
        h = rms_norm(x, w[f"l{i}.norm1"], eps)
        p = f"l{i}.mix."
        if layer["type"] == "attention":
            y = attention_mixer(h, positions, layer["mixer"], w, p)
        elif layer["type"] == "latent_attention":
            y = latent_attention_mixer(h, positions, layer["mixer"], w, p, eps)
        elif layer["type"] == "mamba2":
            y = mamba2_mixer(h, layer["mixer"], w, p, eps)
        else:
            raise ValueError(layer["type"])
        x = x + y
        if layer.get("mlp") is not None:
            h = rms_norm(x, w[f"l{i}.norm2"], eps)
            x = x + routed_feed_forward(h, layer["mlp"], w, f"l{i}.mlp.")
            if margins is not None:
                margins.append(route_margin(h, w[f"l{i}.mlp.router"], layer["mlp"]["router"]["top"]))
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    return rms_norm(x, w["final.norm"], eps).to(dtype) @ w["head"].T


def greedy(cfg: dict, w: Dict[str, torch.Tensor], prompt: List[int], n_new: int) -> List[int]:
    """``n_new`` tokens, each the most likely one (the lowest index among equals), the whole sequence run again each time."""
    seq, out = list(prompt), []
    for _ in range(n_new):
        tok = int(torch.argmax(forward(cfg, w, seq)[-1]))
        out.append(tok)
        seq.append(tok)
    return out
