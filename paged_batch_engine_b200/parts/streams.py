"""Several residual streams per row, and the layer arrangement that reads and writes them."""
from __future__ import annotations

from typing import Optional

import torch

from ..config.specs import BlockSpec
from ..weights.loader import ParamSpec
from .base import Block, Part, build_part, register_part
from .norm import PendingUpdate


class StreamConnection(Part):
    """How one sublayer is wired to S residual streams r_1..r_S: it reads a = sum_s alpha_s r_s
    and its output y updates every stream at once, r'_j = sum_s M[s, j] r_s + beta_j y.
    Checkpoint tensors under its prefix: ``in`` [S] (alpha), ``out`` [S] (beta), ``mix`` [S, S]
    (M, indexed [from, to]).  ``streams`` None: one stream with alpha = beta = M = 1 and no
    tensors, which is the plain residual add."""

    def __init__(self, streams: Optional[int], dtype, device):
        self.streams, self.device = streams, device
        self.alpha = self.beta = self.mix = None
        if streams is None:
            self.alpha = torch.ones(1, dtype=torch.float32, device=device)
            self.beta = torch.ones(1, dtype=torch.float32, device=device)
            self.mix = torch.ones((1, 1), dtype=torch.float32, device=device)

    @property
    def width(self) -> int:
        return self.streams or 1

    def param_specs(self, prefix):
        if self.streams is None:
            return []
        s = self.streams
        return [ParamSpec(prefix + "in", (s,)), ParamSpec(prefix + "out", (s,)), ParamSpec(prefix + "mix", (s, s))]

    def load(self, tensors, prefix):
        if self.streams is None:
            return
        self.alpha = tensors.pop(prefix + "in").to(torch.float32).contiguous()
        self.beta = tensors.pop(prefix + "out").to(torch.float32).contiguous()
        self.mix = tensors.pop(prefix + "mix").to(torch.float32).contiguous()


class StreamBlock(Block):
    """Pre-norm layer over S residual streams: the mixer, then (if the layer has one) the
    feed-forward, each reading the norm of its connection's mixture of the streams and
    updating all streams.  A sublayer's output is carried as a ``PendingUpdate`` into the next
    norm's launch, which folds it in, collapses the streams and normalises in one pass.
    ``spec.args["streams"]``: S, or None for the plain single residual stream."""

    def __init__(self, spec: BlockSpec, dtype, device):
        self.spec = spec
        self.prefix = spec.prefix
        n = spec.names
        streams = spec.args.get("streams")
        self.streams = streams
        self.p_mixer = self.prefix + n.get("mixer", "mixer.")
        self.p_ffn = self.prefix + n.get("feed_forward", "feed_forward.")
        self.p_norm1 = self.prefix + n.get("norm_mixer", "norm_mixer.")
        self.p_norm2 = self.prefix + n.get("norm_feed_forward", "norm_feed_forward.")
        self.p_c1 = self.prefix + n.get("streams_mixer", "streams_mixer.")
        self.p_c2 = self.prefix + n.get("streams_feed_forward", "streams_feed_forward.")
        self.norm1 = build_part("norm", spec.norm_mixer, dtype, device)
        self.mixer = build_part("mixer", spec.mixer, dtype, device)
        self.c1 = StreamConnection(streams, dtype, device)
        self.ffn = self.norm2 = self.c2 = None
        if spec.feed_forward is not None:
            self.norm2 = build_part("norm", spec.norm_feed_forward, dtype, device)
            self.ffn = build_part("feed_forward", spec.feed_forward, dtype, device)
            self.c2 = StreamConnection(streams, dtype, device)
        for norm in (self.norm1, self.norm2):
            if norm is not None and not hasattr(norm, "norm_streams"):
                raise TypeError("a block over residual streams needs norms that read streams (norm_streams)")

    def parts(self):
        out = [(self.norm1, self.p_norm1), (self.mixer, self.p_mixer), (self.c1, self.p_c1)]
        if self.ffn is not None:
            out += [(self.norm2, self.p_norm2), (self.ffn, self.p_ffn), (self.c2, self.p_c2)]
        return out

    def param_specs(self, prefix=""):
        out = []
        for part, p in self.parts():
            out += part.param_specs(p)
        return out

    def load(self, tensors, prefix=""):
        for part, p in self.parts():
            part.load(tensors, p)

    def kernel_libraries(self, dtype):
        out = [("streams", None)]
        for part, _ in self.parts():
            out += part.kernel_libraries(dtype)
        return out

    def forward(self, residual, delta, ctx, cache):
        streams = residual if residual.dim() == 3 else residual.view(residual.shape[0], 1, residual.shape[1])
        if streams.shape[1] != self.c1.width:
            raise ValueError(f"the block is wired to {self.c1.width} residual streams, the model runs {streams.shape[1]}")
        if delta is not None and not isinstance(delta, PendingUpdate):
            delta = self.norm1.as_pending(delta, streams)
        h = self.norm1.norm_streams(streams, delta, self.c1.alpha)
        pending = PendingUpdate(self.mixer.forward(h, ctx, cache), self.c1.mix, self.c1.beta)
        if self.ffn is not None:
            f = self.norm2.norm_streams(streams, pending, self.c2.alpha)
            pending = PendingUpdate(self.ffn.forward(f, ctx), self.c2.mix, self.c2.beta)
        return residual, pending


register_part("block", "streams", lambda spec, dtype, device: StreamBlock(spec, dtype, device), replace=True)
