"""A selective state-space mixer (state-space duality form) with a recurrent state per request."""
from __future__ import annotations

from typing import Optional

import torch

from ..csrc import ops
from ..weights.loader import ParamSpec
from .base import CompositeNeed, Mixer, StateNeed, register_part


class SelectiveStateSpace(Mixer):
    """One input projection gives, side by side, z (``heads * head_dim``, the gate), x (the same
    width), B and C (``groups * state_dim`` each) and dt (``heads``).  x, B and C together pass a
    causal convolution per channel (``conv_taps`` taps, bias, the last tap on the current token)
    and silu.  dt <- softplus(dt + dt_bias).  Per head h, whose B and C are those of group
    h // (heads / groups):

        S_t = exp(-exp(A_log_h) dt_t) S_{t-1} + dt_t B_t x_t^T,    y_t = S_t^T C_t + D_h x_t

    with S ([state_dim, head_dim]) in float32, kept per request, as are the convolution's last
    taps - 1 inputs.  Then u = y * silu(z), u divided by its root mean square in ``norm_groups``
    equal parts, times a gain, and the output projection.  Step sizes, decays and the recurrence
    are float32.

    Checkpoint tensors under the prefix (names in ``tensor_names``): in [2*inner + 2*G*N + H,
    hidden], conv [inner + 2*G*N, taps], conv.b, dt_bias [H], A_log [H], D [H], norm [inner],
    o [hidden, inner]."""
    TENSOR_NAMES = dict(inp="in", conv="conv", conv_bias="conv.b", dt_bias="dt_bias", a_log="A_log", skip="D",
                        norm="norm", o="o")
    decode_capturable = True      # stepped from the step's device arrays alone

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, state_dim: int, groups: int,
                 conv_taps: int, norm_groups: int, eps: float, dtype, device, tensor_names: Optional[dict] = None):
        unknown = set(tensor_names or {}) - set(self.TENSOR_NAMES)
        if unknown:
            raise ValueError(f"tensor_names knows {sorted(self.TENSOR_NAMES)}; got {sorted(unknown)}")
        if num_heads % groups:
            raise ValueError("heads must be a multiple of groups")
        if (num_heads * head_dim) % norm_groups:
            raise ValueError("the inner width must divide into norm_groups equal parts")
        if not 1 <= conv_taps <= 16:
            raise ValueError("the convolution has 1 to 16 taps")
        if state_dim > 512:
            raise ValueError("state_dim is at most 512")
        self.names = dict(self.TENSOR_NAMES, **(tensor_names or {}))
        self.hidden_size, self.num_heads, self.head_dim, self.state_dim = hidden_size, num_heads, head_dim, state_dim
        self.groups, self.conv_taps, self.norm_groups, self.eps = groups, conv_taps, norm_groups, float(eps)
        self.inner = num_heads * head_dim
        self.conv_channels = self.inner + 2 * groups * state_dim
        self.dtype, self.device = dtype, device
        self.w_in = self.w_o = self.conv_w = self.conv_b = self.dt_bias = self.a_log = self.skip = self.gain = None

    def cache_need(self):
        H, N, P = self.num_heads, self.state_dim, self.head_dim
        need = dict(ssm=StateNeed((H, N, P), torch.float32))
        if self.conv_taps > 1:
            need["conv"] = StateNeed((self.conv_taps - 1, self.conv_channels), torch.float32)
        return CompositeNeed.of(**need)

    def kernel_libraries(self, dtype):
        return [("short_conv", None), ("linear_attention", None), ("streams", None)] + ops.gemm_libraries(dtype)

    def param_specs(self, prefix):
        n, w = self.names, self.hidden_size
        H, C = self.num_heads, self.conv_channels
        return [ParamSpec(prefix + n["inp"], (2 * self.inner + 2 * self.groups * self.state_dim + H, w)),
                ParamSpec(prefix + n["conv"], (C, self.conv_taps)), ParamSpec(prefix + n["conv_bias"], (C,)),
                ParamSpec(prefix + n["dt_bias"], (H,)), ParamSpec(prefix + n["a_log"], (H,)),
                ParamSpec(prefix + n["skip"], (H,)), ParamSpec(prefix + n["norm"], (self.inner,)),
                ParamSpec(prefix + n["o"], (w, self.inner))]

    def load(self, tensors, prefix):
        n = self.names
        f32 = lambda name: tensors.pop(prefix + n[name]).to(torch.float32).contiguous()
        self.w_in = tensors.pop(prefix + n["inp"]).contiguous()
        self.w_o = tensors.pop(prefix + n["o"]).contiguous()
        self.conv_w, self.conv_b = f32("conv"), f32("conv_bias")
        self.conv_wt = self.conv_w.t().contiguous()        # [taps, C]: the layout the eight-channel kernel reads
        self.dt_bias, self.a_log, self.skip, self.gain = f32("dt_bias"), f32("a_log"), f32("skip"), f32("norm")

    def chunk_rows(self, rows: int) -> int:
        """Rows of a chunk when a long portion's recurrence runs as chunks side by side: so long that
        the chunks of all heads and column slices fill the GPU about once, a power of two, 64 to 512."""
        blocks_per_chunk = self.num_heads * ((self.head_dim + 31) // 32)
        want = rows * blocks_per_chunk // 1024
        chunk = 64
        while chunk < want and chunk < 512:
            chunk *= 2
        return chunk

    def forward(self, x, ctx, cache):
        H, P, N, G = self.num_heads, self.head_dim, self.state_dim, self.groups
        inner, C = self.inner, self.conv_channels
        proj = ops.linear(x, self.w_in, None, out_dtype=self.dtype, kind=1)
        z, xbc_in, dt_in = proj[:, :inner], proj[:, inner:inner + C], proj[:, inner + C:]
        if self.conv_taps > 1:
            conv_state = cache.sub["conv"].state
        else:
            conv_state = torch.empty((1, 0, C), dtype=torch.float32, device=x.device)
        xbc = ops.short_conv(xbc_in, self.conv_w, self.conv_b, conv_state, ctx.request_of_row, ctx.q_start, ctx.q_len,
                             ctx.state_slots, ctx.num_requests, silu=True, update_state=cache.writes,
                             weight_t=self.conv_wt)
        dt, decay = ops.step_sizes(dt_in, self.dt_bias, self.a_log)
        xs, B, Cm = xbc[:, :inner], xbc[:, inner:inner + G * N], xbc[:, inner + G * N:]
        plan = None if getattr(ctx, "captured", False) else ctx.recurrence_plan(self.chunk_rows(ctx.num_tokens))
        y = ops.linear_attention(Cm, B, xs, cache.sub["ssm"].state, None, ctx.q_start, ctx.q_len, ctx.state_slots,
                                 ctx.num_requests, H, 1.0, False, plan, tok_decay=decay, tok_scale=dt,
                                 skip=self.skip, kq_share=H // G)
        u = ops.gated_rms(y, z, self.gain, self.norm_groups, self.eps, True, "silu", self.dtype, gate_first=True)
        return ops.linear(u, self.w_o, None, out_dtype=self.dtype, kind=2)


register_part("mixer", "selective_state_space", SelectiveStateSpace, replace=True)
