"""RMSNorm part (tinyinfer/layers/layernorm.py:7-25 of the reference; kernel formula
tinyinfer/csrc/rmsnorm.cu:22-50). The weight is kept in float32 because the norm is computed in
float32 whatever the compute dtype."""
from __future__ import annotations

from .. import ops
from .base import Norm, TensorSpec, register_norm


class RMSNorm(Norm):
    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        self.weight = None

    def tensors(self):
        # a weight stored around zero (the norm multiplies by offset + w) is drawn around zero too
        init = "ones_noise" if not getattr(self.spec, "offset", 0.0) else "normal"
        return {self.spec.tensor: TensorSpec((self.spec.size,), role="vector32", init=init)}

    def load(self, tensors):
        self.weight = tensors[self.spec.tensor]
        offset = float(getattr(self.spec, "offset", 0.0))
        if offset:
            self.weight = (self.weight + offset).contiguous()      # float32: the sum is made once, here

    def forward(self, x):
        return ops.rmsnorm(x, self.weight, self.spec.eps)

    def forward_rows(self, x, rows):
        return ops.rmsnorm(x, self.weight, self.spec.eps, rows=rows)

    def as_rms(self):
        return self.weight, self.spec.eps


register_norm("rmsnorm", RMSNorm)
