"""Plain, slow implementation of the Gebadra decoder: the tests' oracle for that design.

Whole sequences, no cache, no paging, one function for each mechanism, elementary torch
arithmetic on the CPU in the dtype of the tensors it is given (float32 or float64).  It
shares no code with the engine: ``config.json`` is a plain dict and the weights a plain
``{name: tensor}`` dict with the checkpoint's own names.

The design in this file's notation (t: position in the sequence, counted from 0):

* several residual streams r_1..r_S (all equal to the embedding at the start); a sublayer
  reads a = sum_s alpha_s r_s, computes y = f(LayerNorm(a)) and every stream becomes
  r'_j = sum_s M[s, j] r_s + beta_j y; the model's output is the sum of the streams;
* two kinds of layers: ``lightning`` (linear attention with a per-head decay on silu'd
  q, k, v; joint RMS norm, sigmoid gate) and ``parallel`` (the mean of two branches, each
  RMS-normed: softmax attention over a sliding window plus mean-pooled blocks of older
  tokens with probabilities mixed across heads; and retention, a decayed linear attention
  with a per-head unit RMS norm and a silu gate);
* a gated feed-forward with silu.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import torch

Tensor = torch.Tensor


def layer_norm(x: Tensor, w: Tensor, b: Tensor, eps: float) -> Tensor:
    """(x - mean) / sqrt(mean((x - mean)^2) + eps) * w + b over the last axis."""
    mu = x.mean(dim=-1, keepdim=True)
    d = x - mu
    var = (d * d).mean(dim=-1, keepdim=True)
    return d / torch.sqrt(var + eps) * w + b


def rms_unit(x: Tensor, eps: float) -> Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def silu(x: Tensor) -> Tensor:
    return x * torch.sigmoid(x)


def rotate_pairs(x: Tensor, positions: Tensor, base: float, dims: int, factor: float) -> Tensor:
    """Rotary encoding on neighbouring pairs (2i, 2i+1) of the first ``dims`` dimensions of
    every head; x is [T, heads, d].  Pair i turns by the angle t * base^(-2i/dims) / factor."""
    out = x.clone()
    i = torch.arange(dims // 2, dtype=x.dtype)
    freq = base ** (-2.0 * i / dims) / factor
    ang = positions.to(x.dtype)[:, None] * freq[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def decayed_linear_attention(q: Tensor, k: Tensor, v: Tensor, decay: Sequence[float]) -> Tensor:
    """Per head h: S_t = decay_h S_{t-1} + k_t v_t^T (S_{-1} = 0), o_t = S_t^T q_t.
    q, k: [T, H, d]; v: [T, H, e]; returns [T, H, e].  Token by token."""
    T, H, d = q.shape
    e = v.shape[-1]
    S = torch.zeros(H, d, e, dtype=q.dtype)
    lam = torch.tensor(list(decay), dtype=q.dtype)[:, None, None]
    out = torch.zeros(T, H, e, dtype=q.dtype)
    for t in range(T):
        S = lam * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hde,hd->he", S, q[t])
    return out


def visible_keys(t: int, window: int, pool: int):
    """What position t sees: (number of pooled blocks, first token).  Tokens j with
    0 <= t - j < window; block b (positions b*pool .. b*pool+pool-1) when its last position
    is at most t - window."""
    first = max(0, t - window + 1)
    blocks = 0
    while blocks * pool + pool - 1 <= t - window:
        blocks += 1
    return blocks, first


def pooled_window_attention(q: Tensor, k: Tensor, v: Tensor, talk: Tensor, scale: float,
                            window: int, pool: int) -> Tensor:
    """q: [T, H, d]; k: [T, G, d]; v: [T, G, e] (k after norm and rotation).  For every
    position one softmax over the pooled blocks it sees and the tokens of its window; the
    probabilities of the heads are then mixed, w'_h = sum_g talk[h, g] w_g, and head h
    applies w'_h to the values of its own key/value head."""
    T, H, d = q.shape
    G, e = k.shape[1], v.shape[-1]
    rep = H // G
    n_blocks = T // pool
    kp = k[:n_blocks * pool].reshape(n_blocks, pool, G, d).mean(dim=1) if n_blocks else k[:0]
    vp = v[:n_blocks * pool].reshape(n_blocks, pool, G, e).mean(dim=1) if n_blocks else v[:0]
    out = torch.zeros(T, H, e, dtype=q.dtype)
    for t in range(T):
        nb, first = visible_keys(t, window, pool)
        keys = torch.cat([kp[:nb], k[first:t + 1]], dim=0)      # [n, G, d]
        vals = torch.cat([vp[:nb], v[first:t + 1]], dim=0)      # [n, G, e]
        w = torch.zeros(H, keys.shape[0], dtype=q.dtype)
        for h in range(H):
            s = (keys[:, h // rep, :] @ q[t, h]) * scale
            w[h] = torch.softmax(s, dim=0)
        w = talk.to(q.dtype) @ w                               # [H, n]
        for h in range(H):
            out[t, h] = w[h] @ vals[:, h // rep, :]
    return out


def softmax_branch(h: Tensor, W: Dict[str, Tensor], p: str, m: dict, eps: float) -> Tensor:
    T = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v = h @ W[p + "q"].T, h @ W[p + "k"].T, h @ W[p + "v"].T
    q = rms_unit(q, eps) * W[p + "q.norm"]          # over the whole projection, before the split
    k = rms_unit(k, eps) * W[p + "k.norm"]
    pos = torch.arange(T)
    rot = m["rot"]
    factor = float(rot.get("scaling", {}).get("factor", 1.0)) if rot.get("scaling") else 1.0
    q = rotate_pairs(q.reshape(T, H, d), pos, float(rot["base"]), int(rot["dims"]), factor)
    k = rotate_pairs(k.reshape(T, G, d), pos, float(rot["base"]), int(rot["dims"]), factor)
    o = pooled_window_attention(q, k, v.reshape(T, G, e), W[p + "talk"], float(m["scale"]),
                                int(m["mask"]["size"]), int(m["mask"]["pool"]))
    return o.reshape(T, H * e) @ W[p + "o"].T


def retention_branch(h: Tensor, W: Dict[str, Tensor], p: str, m: dict, eps: float) -> Tensor:
    T = h.shape[0]
    H, d, e = m["heads"], m["dim"], m["vdim"]
    q = (h @ W[p + "q"].T).reshape(T, H, d)
    k = (h @ W[p + "k"].T).reshape(T, H, d) * d ** -0.5
    v = (h @ W[p + "v"].T).reshape(T, H, e)
    o = rms_unit(decayed_linear_attention(q, k, v, m["decay"]), eps)     # per head, no gain
    return (o.reshape(T, H * e) * silu(h @ W[p + "g"].T)) @ W[p + "o"].T


def parallel_mixer(h: Tensor, W: Dict[str, Tensor], p: str, m: dict, eps: float) -> Tensor:
    left = softmax_branch(h, W, p + "left.", m["left"], eps)
    right = retention_branch(h, W, p + "right.", m["right"], eps)
    return 0.5 * (rms_unit(left, eps) * W[p + "left.out"] + rms_unit(right, eps) * W[p + "right.out"])


def lightning_mixer(h: Tensor, W: Dict[str, Tensor], p: str, m: dict, eps: float) -> Tensor:
    T = h.shape[0]
    H, d, e = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ W[p + "q"].T).reshape(T, H, d)
    k = silu(h @ W[p + "k"].T).reshape(T, H, d)
    v = silu(h @ W[p + "v"].T).reshape(T, H, e)
    o = decayed_linear_attention(q, k, v, m["decay"]).reshape(T, H * e)
    o = rms_unit(o, eps) * W[p + "norm"]             # all heads together
    return (o * torch.sigmoid(h @ W[p + "g"].T)) @ W[p + "o"].T


def gated_mlp(h: Tensor, W: Dict[str, Tensor], p: str) -> Tensor:
    return (silu(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def forward(cfg: dict, W: Dict[str, Tensor], tokens: Sequence[int], return_layers: bool = False):
    """Logits [T, vocab] of one whole sequence (and the summed streams after every layer)."""
    eps = float(cfg["norm"]["eps"])
    S = cfg.get("streams")
    x = W["embed"][torch.as_tensor(list(tokens), dtype=torch.long)]
    streams = [x.clone() for _ in range(S or 1)]
    after = []
    for i, layer in enumerate(cfg["layers"]):
        src = layer.get("weights_of", i)
        p = f"l{src}."

        def sublayer(q, f):
            nonlocal streams
            norm = lambda z: layer_norm(z, W[f"{p}norm{q}"], W[f"{p}norm{q}.b"], eps)
            if S is None:
                streams = [streams[0] + f(norm(streams[0]))]
                return
            a_in, b_out, M = W[f"{p}hc{q}.in"], W[f"{p}hc{q}.out"], W[f"{p}hc{q}.mix"]
            y = f(norm(sum(a_in[s] * streams[s] for s in range(S))))
            streams = [sum(M[s, j] * streams[s] for s in range(S)) + b_out[j] * y for j in range(S)]

        if layer["type"] == "lightning":
            sublayer(1, lambda z: lightning_mixer(z, W, p + "mix.", layer["mixer"], eps))
        elif layer["type"] == "parallel":
            sublayer(1, lambda z: parallel_mixer(z, W, p + "mix.", layer["mixer"], eps))
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp") is not None:
            sublayer(2, lambda z: gated_mlp(z, W, p + "mlp."))
        after.append(sum(streams))
    x = sum(streams)
    logits = layer_norm(x, W["final.norm"], W["final.norm.b"], eps) @ W["head"].T
    return (logits, torch.stack(after)) if return_layers else logits
