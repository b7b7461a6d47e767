"""Position encodings.  'learned': a table row per position, added where tokens are embedded, with
the row offset as a parameter (OPT's table starts at row 2:
src/transformers_neuronx/opt/model.py:232-244).  'sinusoidal': a computed vector, column 2i = sin(p base^(-2i/dim)),
column 2i + 1 the cosine, added in the same kernel (the frequencies are computed in 64-bit on the host and rounded once
to 32-bit; the angle and its sine and cosine are 32-bit in the kernel).  'none': nothing."""
from __future__ import annotations

import torch

from ..weights.loader import TensorSpec
from .base import PositionEncoding, weight_to_device
from .registry import register_position
from .spec import PositionSpec


class LearnedPositions(PositionEncoding):
    graph_safe = True
    libraries = ("embedding",)

    def __init__(self, spec: PositionSpec):
        self.spec = spec
        self.table = None

    def tensor_specs(self):
        return [TensorSpec(self.spec.table, (self.spec.rows, self.spec.dim), "table")]

    def load(self, tensors, device, act_dtype):
        self.table = weight_to_device(tensors[self.spec.table], device, act_dtype, self.spec.table)

    def parameter_bytes(self):
        return self.table.numel() * self.table.element_size()

    def max_position(self) -> int:
        return self.spec.rows - self.spec.offset

    def table_for_embedding(self):
        return self.table, self.spec.offset


class SinusoidalPositions(PositionEncoding):
    graph_safe = True
    libraries = ("embedding",)

    def __init__(self, spec: PositionSpec):
        if spec.dim <= 0 or not (spec.base > 1):
            raise ValueError(f"a sinusoidal encoding needs its width and a base above 1, got {spec.dim} and {spec.base}")
        self.spec = spec
        self.freq = None

    def load(self, tensors, device, act_dtype):
        i = torch.arange((self.spec.dim + 1) // 2, dtype=torch.float64)
        f = torch.pow(torch.tensor(float(self.spec.base), dtype=torch.float64), -2.0 * i / self.spec.dim)
        self.freq = f.to(torch.float32).to(device)

    def frequencies_for_embedding(self):
        return self.freq


class NoPositions(PositionEncoding):
    graph_safe = True
    def __init__(self, spec=None):
        self.spec = spec


register_position("learned", LearnedPositions)
register_position("sinusoidal", SinusoidalPositions)
register_position("none", NoPositions)
