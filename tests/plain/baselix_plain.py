"""A plain, slow implementation of the Baselix forward pass: whole sequences, no cache, one function per
mechanism, on the CPU in float64 (or float32).  It shares no code with ``zedinfer_b200``: it reads
``config.json`` with ``json`` and ``model.safetensors`` with its own few lines.

The design in this file's notation (``x`` the residual stream, ``m = residual_mult``, ``N(x, w) =
x / sqrt(mean(x^2) + eps)`` times a weight):

    x_t      = E[token_t] + P[t]                                   learned absolute positions, t from 0
    per layer:  x += m * mixer(N(x) * (1 + w1));   x += m * ff(N(x) * (1 + w2))   (ff may be absent)
    mixer:      q = Wq h;  c = N(Wdkv h) * g   (g a plain weight; a layer with ``kv_from: j`` takes layer j's c)
                per head a:  k = Wuk_a c,  v = Wuv_a c,  s_tj = scale * q_ta . k_ja  for  0 <= t - j < window
                p_tj = exp(s_tj) / (exp(sink_a) + sum_j' exp(s_tj'))            the sink has no value
                out = Wo concat_a(sum_j p_tj v_ja)
    dense ff:   Wdown relu(Wup h)^2
    routed ff:  z = Wr h + b;  the ``top`` largest z;  weights = softmax over those;  sum of weight_e * expert_e(h)
                + shared expert(h);   expert: g = min(Wg h, L), u = clamp(Wu h, -L, L),
                Wd (g * sigmoid(1.702 g) * (u + 1))
    logits   = cap * tanh((E N(x) * (1 + wf)) / cap)
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional

import torch

GATE_SLOPE = 1.702


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
        key = name[6:] if name.startswith("model.") else name          # folders written with that prefix
        out[key] = t.to(dtype) if t.is_floating_point() else t.clone()
    return out


def read_model(model_dir: str, dtype=torch.float64):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(model_dir, "model.safetensors"), dtype)


# ---------------------------------------------------------------------------------------------
# mechanisms, one function each
# ---------------------------------------------------------------------------------------------
def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm_around_zero(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """The layer norms and the final norm: the stored weight is an offset from one."""
    return unit_rms(x, eps) * (1.0 + w)


def norm_plain_weight(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """The latent's norm: the stored weight is the factor itself."""
    return unit_rms(x, eps) * w


def embed(tokens: List[int], table: torch.Tensor, pos_table: torch.Tensor, first_position: int = 0) -> torch.Tensor:
    ids = torch.tensor(tokens, dtype=torch.long)
    return table[ids] + pos_table[first_position:first_position + len(tokens)]


def latent(h: torch.Tensor, w_dkv: torch.Tensor, g: torch.Tensor, eps: float) -> torch.Tensor:
    return norm_plain_weight(h @ w_dkv.T, g, eps)


def windowed_sink_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, sink: torch.Tensor, scale: float,
                            window: Optional[int]) -> torch.Tensor:
    """q, k ``[T, H, d]``, v ``[T, H, dv]``, sink ``[H]``; query t sees keys j with ``0 <= t - j < window``."""
    T, H, _ = q.shape
    out = torch.zeros((T, H, v.shape[2]), dtype=q.dtype)
    for t in range(T):
        lo = 0 if window is None else max(0, t - window + 1)
        for a in range(H):
            s = (k[lo:t + 1, a] @ q[t, a]) * scale
            top = max(float(s.max()), float(sink[a]))
            e = torch.exp(s - top)
            denom = e.sum() + math.exp(float(sink[a]) - top)
            out[t, a] = (e / denom) @ v[lo:t + 1, a]
    return out


def latent_attention(h: torch.Tensor, c: torch.Tensor, w: Dict[str, torch.Tensor], mixer: dict) -> torch.Tensor:
    H, d, dv = mixer["heads"], mixer["dim"], mixer["vdim"]
    T = h.shape[0]
    q = (h @ w["q"].T).reshape(T, H, d)
    k = (c @ w["uk"].T).reshape(T, H, d)
    v = (c @ w["uv"].T).reshape(T, H, dv)
    window = (mixer.get("mask") or {}).get("size")
    o = windowed_sink_attention(q, k, v, w["sink"], float(mixer["scale"]), window)
    return o.reshape(T, H * dv) @ w["o"].T


def squared_relu_ff(h: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor) -> torch.Tensor:
    a = torch.relu(h @ w_up.T)
    return (a * a) @ w_down.T


def clamped_expert(h: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor,
                   limit: float) -> torch.Tensor:
    g = torch.clamp(h @ w_gate.T, max=limit)
    u = torch.clamp(h @ w_up.T, min=-limit, max=limit)
    return (g * torch.sigmoid(GATE_SLOPE * g) * (u + 1.0)) @ w_down.T


def route(h: torch.Tensor, w_router: torch.Tensor, bias: torch.Tensor, top: int):
    """(indices ``[T, top]``, weights ``[T, top]``): the largest logits, softmax over those alone."""
    z = h @ w_router.T + bias
    vals, idx = torch.topk(z, top, dim=-1)
    return idx, torch.softmax(vals, dim=-1)


def routed_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], mlp: dict) -> torch.Tensor:
    idx, wts = route(h, w["router"], w["router.b"], mlp["router"]["top"])
    limit = float(mlp["expert"]["limit"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(idx.shape[1]):
            e = int(idx[t, j])
            out[t] += wts[t, j] * clamped_expert(h[t:t + 1], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"], limit)[0]
    if mlp.get("shared"):
        out = out + clamped_expert(h, w["shared.gate"], w["shared.up"], w["shared.down"], float(mlp["shared"]["limit"]))
    return out


def capped_logits(x: torch.Tensor, table: torch.Tensor, cap: Optional[float]) -> torch.Tensor:
    z = x @ table.T
    return z if not cap else cap * torch.tanh(z / cap)


# ---------------------------------------------------------------------------------------------
# the model
# ---------------------------------------------------------------------------------------------
def _sub(w: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in w.items() if k.startswith(prefix)}


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], return_layers: bool = False):
    """Logits ``[T, vocab]`` of a whole sequence (and the residual stream after every layer)."""
    eps = float(cfg["norm"]["eps"])
    m = float(cfg.get("residual_mult", 1.0))
    x = embed(tokens, w["embed"], w["pos"])
    latents: Dict[int, torch.Tensor] = {}
    after = []
    for i, layer in enumerate(cfg["layers"]):
        lw = _sub(w, f"l{i}.")
        mixer = layer["mixer"]
        h = norm_around_zero(x, lw["norm1"], eps)
        mw = _sub(lw, "mix.")
        if mixer.get("kv_from") is None:
            latents[i] = latent(h, mw["dkv"], mw["dkv.norm"], eps)
            c = latents[i]
        else:
            c = latents[int(mixer["kv_from"])]
        x = x + m * latent_attention(h, c, mw, mixer)
        mlp = layer.get("mlp")
        if mlp:
            h = norm_around_zero(x, lw["norm2"], eps)
            fw = _sub(lw, "mlp.")
            if mlp["kind"] == "dense":
                x = x + m * squared_relu_ff(h, fw["up"], fw["down"])
            else:
                x = x + m * routed_ff(h, fw, mlp)
        after.append(x.clone())
    logits = capped_logits(norm_around_zero(x, w["final.norm"], eps), w["embed"], cfg.get("logit_softcap"))
    return (logits, torch.stack(after)) if return_layers else logits


def greedy(cfg: dict, w: Dict[str, torch.Tensor], prompt: List[int], n_new: int) -> List[int]:
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(torch.argmax(forward(cfg, w, toks)[-1])))
    return toks[len(prompt):]
