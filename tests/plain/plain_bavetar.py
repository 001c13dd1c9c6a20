"""Plain, slow implementation of the Bavetar decoder: the tests' oracle for that design.

Whole sequences, no cache, no paging, one function for each mechanism, elementary torch
arithmetic on the CPU in the dtype of the tensors it is given (float32 or float64).  It
shares no code with the engine: ``config.json`` is a plain dict and the weights a plain
``{name: tensor}`` dict with the checkpoint's own names.

The design in this file's notation (t: position in the sequence, counted from 0):

* a layer reads one residual x and adds two branches computed from the same x:
  x <- x + mixer(n1(x)) + ff(n2(x)), n1 and n2 RMS norms with gains of their own;
* two mixers: ``mamba2`` (a selective state-space recurrence with a short causal
  convolution in front, a gate and a grouped RMS norm behind) and ``latent_attention``
  (softmax attention whose keys and values are expanded from one small latent per token
  plus one rotated key part shared by all heads; a learned sink in the softmax's
  denominator; a sigmoid gate per head);
* two feed-forwards: dense with relu(z)^2, and routed experts (softmax router, groups of
  experts of which only the best may be chosen from, gated silu experts);
* logits from the embedding table, scaled and soft-capped with tanh.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

Tensor = torch.Tensor


def rms_unit(x: Tensor, eps: float) -> Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def silu(x: Tensor) -> Tensor:
    return x * torch.sigmoid(x)


def softplus(x: Tensor) -> Tensor:
    """log(1 + exp(x)), written so that large x does not overflow."""
    return torch.where(x > 20, x, torch.log1p(torch.exp(torch.clamp(x, max=20))))


def rotate_pairs(x: Tensor, positions: Tensor, base: float, dims: int) -> Tensor:
    """Rotary encoding on neighbouring pairs (2i, 2i+1) of the first ``dims`` dimensions of the
    last axis; x is [T, ..., d].  Pair i at position t turns by t * base^(-2i/dims)."""
    out = x.clone()
    i = torch.arange(dims // 2, dtype=x.dtype)
    freq = base ** (-2.0 * i / dims)
    ang = positions.to(x.dtype)[:, None] * freq[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [dims // 2]
    c, s = torch.cos(ang).reshape(shape), torch.sin(ang).reshape(shape)
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


# ---------------------------------------------------------------------------- mamba2
def causal_conv(u: Tensor, w: Tensor, b: Tensor) -> Tensor:
    """y[t, c] = b[c] + sum_j w[c, j] u[t - (taps - 1) + j, c], inputs before the start are zero;
    u [T, C], w [C, taps]: the last column multiplies the current token."""
    T, C = u.shape
    taps = w.shape[1]
    pad = torch.cat([torch.zeros(taps - 1, C, dtype=u.dtype), u], dim=0)
    y = b.expand(T, C).clone()
    for j in range(taps):
        y = y + pad[j:j + T] * w[:, j]
    return y


def selective_scan(x: Tensor, dt: Tensor, a_log: Tensor, B: Tensor, C: Tensor, D: Tensor) -> Tensor:
    """Per head h (group g of h): S_t = exp(-exp(a_log_h) dt_t) S_{t-1} + dt_t B_t x_t^T (S: [N, P]),
    y_t = S_t^T C_t + D_h x_t.  x [T, H, P], dt [T, H], B and C [T, G, N]; returns [T, H, P]."""
    T, H, P = x.shape
    G, N = B.shape[1], B.shape[2]
    per = H // G
    y = torch.zeros_like(x)
    for h in range(H):
        g = h // per
        S = torch.zeros(N, P, dtype=x.dtype)
        rate = torch.exp(a_log[h])
        for t in range(T):
            S = torch.exp(-rate * dt[t, h]) * S + dt[t, h] * torch.outer(B[t, g], x[t, h])
            y[t, h] = S.t() @ C[t, g] + D[h] * x[t, h]
    return y


def grouped_rms(y: Tensor, parts: int, gain: Tensor, eps: float) -> Tensor:
    """The last axis in ``parts`` equal parts, each divided by its own root mean square; times gain."""
    T, n = y.shape
    return (rms_unit(y.reshape(T, parts, n // parts), eps).reshape(T, n)) * gain


def mamba2_mixer(h: Tensor, w: Dict[str, Tensor], p: str, m: dict, eps: float) -> Tensor:
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    T = h.shape[0]
    proj = h @ w[p + "in"].t()
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w[p + "conv"], w[p + "conv.b"]))
    x = xbc[:, :inner].reshape(T, H, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + w[p + "dt_bias"])
    y = selective_scan(x, dt, w[p + "A_log"], B, C, w[p + "D"]).reshape(T, inner)
    y = grouped_rms(y * silu(z), m["norm_groups"], w[p + "norm"], eps)
    return y @ w[p + "o"].t()


# ---------------------------------------------------------------------------- latent attention
def sink_softmax_weights(scores: Tensor, sink: Tensor) -> Tensor:
    """Softmax over the last axis whose denominator also holds exp(sink); scores [H, T, T] with
    -inf where masked, sink [H].  The weights of a row sum to less than one."""
    m = torch.maximum(scores.max(dim=-1, keepdim=True).values, sink[:, None, None])
    e = torch.exp(scores - m)
    return e / (e.sum(dim=-1, keepdim=True) + torch.exp(sink[:, None, None] - m))


def latent_attention_mixer(h: Tensor, w: Dict[str, Tensor], p: str, m: dict, eps: float,
                           positions: Optional[Tensor] = None) -> Tensor:
    H, D, R, V, kv = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    T = h.shape[0]
    positions = torch.arange(T) if positions is None else positions
    base, dims = float(m["rot"]["base"]), int(m["rot"]["dims"])
    cq = rms_unit(h @ w[p + "dq"].t(), eps) * w[p + "dq.norm"]
    q = (cq @ w[p + "uq"].t()).reshape(T, H, D + R)
    q_plain, q_rot = q[..., :D], rotate_pairs(q[..., D:], positions, base, dims)
    ckr = h @ w[p + "dkv"].t()
    c = rms_unit(ckr[:, :kv], eps) * w[p + "dkv.norm"]
    k_rot = rotate_pairs(ckr[:, kv:], positions, base, dims)                 # [T, R], one for all heads
    k_plain = (c @ w[p + "uk"].t()).reshape(T, H, D)
    v = (c @ w[p + "uv"].t()).reshape(T, H, V)
    scores = (torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihr,jr->hij", q_rot, k_rot)) * m["scale"]
    mask = positions[None, :] <= positions[:, None]
    scores = scores.masked_fill(~mask[None], float("-inf"))
    wts = sink_softmax_weights(scores, w[p + "sink"].to(h.dtype))
    out = torch.einsum("hij,jhv->ihv", wts, v)
    gate = torch.sigmoid(h @ w[p + "g"].t())                                 # [T, H]
    return (out * gate[:, :, None]).reshape(T, H * V) @ w[p + "o"].t()


# ---------------------------------------------------------------------------- feed-forwards
def dense_ff(h: Tensor, w: Dict[str, Tensor], p: str) -> Tensor:
    a = torch.relu(h @ w[p + "up"].t())
    return (a * a) @ w[p + "down"].t()


def route(h: Tensor, w_router: Tensor, r: dict):
    """(chosen experts [T, top], their weights [T, top]).  Scores are the softmax of the router's
    logits over all experts; experts outside the best ``keep`` groups (a group's score: its
    largest score) cannot be chosen; weights are the chosen scores over their sum, times scale."""
    E, top = r["experts"], r["top"]
    s = torch.softmax(h @ w_router.t(), dim=-1)
    groups = r.get("groups")
    allowed = torch.ones_like(s, dtype=torch.bool)
    if groups:
        n, keep = groups["count"], groups["keep"]
        best = s.reshape(-1, n, E // n).max(dim=-1).values
        kept = best.topk(keep, dim=-1).indices
        gmask = torch.zeros_like(best, dtype=torch.bool).scatter_(1, kept, True)
        allowed = gmask[:, :, None].expand(-1, n, E // n).reshape(-1, E)
    picked = s.masked_fill(~allowed, -1.0).topk(top, dim=-1).indices
    chosen = s.gather(1, picked)
    return picked, chosen / (chosen.sum(dim=-1, keepdim=True) + 1e-20) * r["scale"]


def expert_ff(h: Tensor, w: Dict[str, Tensor], p: str) -> Tensor:
    return (silu(h @ w[p + "gate"].t()) * (h @ w[p + "up"].t())) @ w[p + "down"].t()


def routed_ff(h: Tensor, w: Dict[str, Tensor], p: str, mlp: dict) -> Tensor:
    picked, weights = route(h, w[p + "router"], mlp["router"])
    out = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for e, g in zip(picked[t].tolist(), weights[t]):
            out[t] = out[t] + g * expert_ff(h[t:t + 1], w, f"{p}e{e}.")[0]
    return out


# ---------------------------------------------------------------------------- the model
def forward(config: dict, weights: Dict[str, Tensor], tokens, dtype=torch.float64, residuals: Optional[List[Tensor]] = None
            ) -> Tensor:
    """Logits [T, vocab] of one whole sequence; ``residuals`` (a list) receives the residual after
    every layer."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = float(config["norm"]["eps"])
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        u = rms_unit(x, eps)
        h1 = u * w[p + "norm1"]
        if layer["type"] == "mamba2":
            y = mamba2_mixer(h1, w, p + "mix.", layer["mixer"], eps)
        elif layer["type"] == "latent_attention":
            y = latent_attention_mixer(h1, w, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        mlp = layer.get("mlp")
        if mlp is not None:
            h2 = u * w[p + "norm2"]
            y = y + (dense_ff(h2, w, p + "mlp.") if mlp["kind"] == "dense" else routed_ff(h2, w, p + "mlp.", mlp))
        x = x + y
        if residuals is not None:
            residuals.append(x.clone())
    x = rms_unit(x, eps) * w["final.norm"]
    logits = (x @ w["embed"].t()) * float(config.get("logit_scale", 1.0))
    cap = config.get("logit_softcap")
    if cap:
        logits = float(cap) * torch.tanh(logits / float(cap))
    return logits
