"""RMSNorm: y = x * rsqrt(mean(x^2) + eps) * weight, the weight used as it is
(src/src-cuda/norm.cu:3-49), fused with the residual add that precedes it
(norm.cu:51-101).  `size` and `eps` are parameters; sums are float32."""
from __future__ import annotations

from ..ops import kernels
from ..weights.loader import TensorWant
from .base import Norm, register_part


class RMSNorm(Norm):
    kind = "rms_norm"
    graph_safe = True

    @classmethod
    def wanted(cls, params):
        return {"weight": TensorWant((params["size"],), "norm")}

    def __init__(self, params, load, rt):
        super().__init__(params, load, rt)
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.weight = load("weight")

    def add_norm(self, delta, residual, rows=None, write_residual=True):
        """normed(residual + delta) in the activation type.  The float32 sum is written back to
        `residual` unless `rows` picks rows or `write_residual` is False; `delta` may be None."""
        return kernels.add_rmsnorm(delta, residual, self.weight, self.eps, self.rt.dtype, rows=rows,
                                   write_residual=write_residual)


register_part(RMSNorm.kind, RMSNorm)
