"""Several mixers side by side on the same input."""
from __future__ import annotations

from typing import Sequence, Tuple

import torch

from ..config.specs import PartSpec
from ..csrc import ops
from ..weights.loader import ParamSpec
from .base import CompositeNeed, Mixer, build_part, register_part


class ParallelMixer(Mixer):
    """y = mean over the branches b of  out_b / rms(out_b) * gain_b : every branch is a mixer of
    its own kind reading the same rows, its output divided by its root mean square over the model
    width and multiplied by a gain before the branches are averaged.

    ``branches``: (name, PartSpec) pairs; branch ``name`` has its tensors under ``prefix + name +
    "."`` and its gain at ``prefix + name + "." + gain_name``; each branch keeps a cache of its
    own kind (the parts of a ``CompositeNeed`` by branch name)."""

    def __init__(self, hidden_size: int, branches: Sequence[Tuple[str, PartSpec]], eps: float, dtype, device,
                 gain_name: str = "out"):
        if not 1 <= len(branches) <= 4:
            raise ValueError("one to four branches")
        self.hidden_size, self.eps, self.gain_name = hidden_size, float(eps), gain_name
        self.dtype, self.device = dtype, device
        self.branches = [(name, build_part("mixer", spec, dtype, device)) for name, spec in branches]
        self.gains = []

    @property
    def decode_capturable(self):
        return all(getattr(m, "decode_capturable", False) for _, m in self.branches)

    def cache_need(self):
        return CompositeNeed(tuple((name, m.cache_need()) for name, m in self.branches))

    def work_keys(self):
        out = []
        for _, m in self.branches:
            out += m.work_keys()
        return out

    def kernel_libraries(self, dtype):
        out = [("streams", None)]
        for _, m in self.branches:
            out += m.kernel_libraries(dtype)
        return out

    def param_specs(self, prefix):
        out = []
        for name, m in self.branches:
            out += m.param_specs(prefix + name + ".")
            out.append(ParamSpec(prefix + name + "." + self.gain_name, (self.hidden_size,)))
        return out

    def load(self, tensors, prefix):
        self.gains = []
        for name, m in self.branches:
            m.load(tensors, prefix + name + ".")
            self.gains.append(tensors.pop(prefix + name + "." + self.gain_name).to(torch.float32).contiguous())

    def forward(self, x, ctx, cache):
        outs = [m.forward(x, ctx, cache.sub[name]) for name, m in self.branches]
        return ops.branch_rms_mean(outs, self.gains, self.eps)


register_part("mixer", "parallel", ParallelMixer, replace=True)
