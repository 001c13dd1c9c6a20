"""Linear attention with a fixed decay per head, kept as a recurrent state per request."""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from ..csrc import ops
from ..weights.loader import ParamSpec
from .base import Mixer, StateNeed, register_part


class DecayLinearAttention(Mixer):
    """q, k (``key_dim`` per head), v, g (``value_dim`` per head) = x W^T as one fused product;
    per head S_t = decay_h S_{t-1} + k_t v_t^T, o_t = S_t^T q_t with S in float32, carried in a
    state row per request; then o / rms(o) (over all heads together, ``out_norm="joint"``, or
    head by head, ``"head"``), an optional gain, times sigmoid or silu of g; output projection.

    Constants that select a variant: ``activation`` ("silu": q, k and v pass through silu;
    "none"), ``key_scale`` (k is multiplied by it), ``out_norm``, ``norm_gain`` (a gain tensor
    of heads * value_dim under the name ``norm``), ``gate`` ("sigmoid" or "silu").
    Checkpoint tensors under the prefix: q, k [H*D, hidden]; v, g [H*E, hidden]; o [hidden, H*E];
    ``tensor_names`` renames them and ``weight_suffix`` is what follows a name (".weight" or "")."""
    TENSOR_NAMES = dict(q="q_proj", k="k_proj", v="v_proj", g="g_proj", o="o_proj", norm="norm")
    decode_capturable = True      # stepped from the step's device arrays alone

    def __init__(self, hidden_size: int, num_heads: int, key_dim: int, value_dim: int, decay: Sequence[float],
                 eps: float, dtype, device, activation: str = "none", key_scale: float = 1.0,
                 out_norm: str = "head", norm_gain: bool = False, gate: str = "sigmoid",
                 tensor_names: Optional[dict] = None, weight_suffix: str = ".weight"):
        unknown = set(tensor_names or {}) - set(self.TENSOR_NAMES)
        if unknown:
            raise ValueError(f"tensor_names knows q, k, v, g, o and norm; got {sorted(unknown)}")
        if len(decay) != num_heads:
            raise ValueError(f"one decay per head: {len(decay)} given for {num_heads} heads")
        if activation not in ("none", "silu") or out_norm not in ("joint", "head") or gate not in ("sigmoid", "silu"):
            raise ValueError("activation is none|silu, out_norm joint|head, gate sigmoid|silu")
        self.names = dict(self.TENSOR_NAMES, **(tensor_names or {}))
        self.suffix = weight_suffix
        self.hidden_size, self.num_heads, self.key_dim, self.value_dim = hidden_size, num_heads, key_dim, value_dim
        self.eps, self.activation, self.key_scale = float(eps), activation, float(key_scale)
        self.out_norm, self.norm_gain, self.gate = out_norm, bool(norm_gain), gate
        self.dtype, self.device = dtype, device
        self.decay = torch.tensor([float(d) for d in decay], dtype=torch.float32).to(device)
        self.w_in = self.w_o = self.gain = None

    def cache_need(self):
        return StateNeed((self.num_heads, self.key_dim, self.value_dim), torch.float32)

    def kernel_libraries(self, dtype):
        return [("linear_attention", None), ("streams", None)] + ops.gemm_libraries(dtype)

    def param_specs(self, prefix):
        n, s = self.names, self.suffix
        hd, he, w = self.num_heads * self.key_dim, self.num_heads * self.value_dim, self.hidden_size
        specs = [ParamSpec(prefix + n["q"] + s, (hd, w)), ParamSpec(prefix + n["k"] + s, (hd, w)),
                 ParamSpec(prefix + n["v"] + s, (he, w)), ParamSpec(prefix + n["g"] + s, (he, w)),
                 ParamSpec(prefix + n["o"] + s, (w, he))]
        if self.norm_gain:
            specs.append(ParamSpec(prefix + n["norm"], (he,)))
        return specs

    def load(self, tensors, prefix):
        n, s = self.names, self.suffix
        ws = [tensors.pop(prefix + n[x] + s) for x in "qkvg"]
        if len({w.dtype for w in ws}) != 1:
            ws = [w.to(torch.float32) for w in ws]
        self.w_in = torch.cat(ws, dim=0).contiguous()
        del ws
        self.w_o = tensors.pop(prefix + n["o"] + s).contiguous()
        if self.norm_gain:
            self.gain = tensors.pop(prefix + n["norm"]).to(torch.float32).contiguous()

    def chunk_rows(self, rows: int) -> int:
        """Rows of a chunk for a step of that many rows: as long as the chunks of all heads and
        column slices still fill the GPU about once (a chunk costs its start-up and runs twice), a
        power of two from 64 to 512.  One 2,048-token prompt, 16 heads of 128 x 128: 406 us with
        chunks of 64, 378 with 128, 429 with 256, 481 with 512, against 698 in sequence."""
        blocks_per_chunk = self.num_heads * ((self.value_dim + 31) // 32)
        want = rows * blocks_per_chunk // 1024
        chunk = 64
        while chunk < want and chunk < 512:
            chunk *= 2
        return chunk

    def forward(self, x, ctx, cache):
        H, D, E = self.num_heads, self.key_dim, self.value_dim
        proj = ops.linear(x, self.w_in, None, out_dtype=self.dtype, kind=1)
        q, k = proj[:, :H * D], proj[:, H * D:2 * H * D]
        v, g = proj[:, 2 * H * D:2 * H * D + H * E], proj[:, 2 * H * D + H * E:]
        # long portions run as chunks side by side; a captured step (single tokens) has no plan
        plan = None if getattr(ctx, "captured", False) else ctx.recurrence_plan(self.chunk_rows(ctx.num_tokens))
        o = ops.linear_attention(q, k, v, cache.state, self.decay, ctx.q_start, ctx.q_len, ctx.state_slots,
                                 ctx.num_requests, H, self.key_scale, self.activation == "silu", plan)
        y = ops.gated_rms(o, g, self.gain, H, self.eps, self.out_norm == "head", self.gate, self.dtype)
        return ops.linear(y, self.w_o, None, out_dtype=self.dtype, kind=2)


register_part("mixer", "linear_attention", DecayLinearAttention, replace=True)
