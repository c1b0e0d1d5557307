"""RMSNorm:  y = x * rsqrt(mean(x^2) + eps) * w   (reference: src/operators/cuda/cuda_rms_norm.cu:10-36); with ``offset`` the
stored weight is w - offset (a design that keeps its weights around zero has offset 1), with ``scale`` the output is multiplied
by it (a design that scales its logits: the head is linear, so the factor may ride on the final norm's weight).
LayerNorm:  y = (x - mean) / sqrt(mean((x - mean)^2) + eps) * w + b."""
from .. import kernels
from ..weights.loader import TensorSpec
from .base import Part, register_part


class RMSNorm(Part):
    graph_safe = True
    def __init__(self, rt, size, eps, names=None, offset=0.0, scale=1.0, required=True):
        self.rt, self.size, self.eps = rt, int(size), float(eps)
        self.offset, self.scale, self.required = float(offset), float(scale), bool(required)
        self.names = {"weight": "weight", **(names or {})}
        self.weight = None

    def tensor_specs(self):
        return {self.names["weight"]: TensorSpec((self.size,), role="norm_offset" if self.offset else "norm", required=self.required)}

    def bind(self, tensors):
        w = self._vector_f32(tensors[self.names["weight"]])
        if self.offset or self.scale != 1.0:
            w = ((w + self.offset) * self.scale).contiguous()          # fp32: the stored weights are exact in it
        self.weight = w

    def replay_tensors(self):
        return [self.weight] if type(self) is RMSNorm else None

    def replay_key(self):
        return ("rmsnorm", self.size, self.eps, self.rt.dtype)

    def forward(self, x, out_dtype=None, rows=None):
        """x: fp32 [T,size] (the residual stream); returns [T or len(rows), size] in ``out_dtype``."""
        return kernels.rmsnorm(x, self.weight, self.eps, out_dtype or self.rt.dtype, rows=rows)


class LayerNorm(Part):
    """Layer norm with a weight and a bias per channel; ``names``: the two tensors' names."""
    graph_safe = True

    def __init__(self, rt, size, eps, names=None):
        self.rt, self.size, self.eps = rt, int(size), float(eps)
        self.names = {"weight": "weight", "bias": "bias", **(names or {})}
        self.weight = self.bias = None

    def tensor_specs(self):
        return {self.names["weight"]: TensorSpec((self.size,), role="norm"), self.names["bias"]: TensorSpec((self.size,), role="bias")}

    def bind(self, tensors):
        self.weight = self._vector_f32(tensors[self.names["weight"]])
        self.bias = self._vector_f32(tensors[self.names["bias"]])

    def forward(self, x, out_dtype=None, rows=None):
        """x: fp32 [T,size] (the residual stream); returns [T or len(rows), size] in ``out_dtype``."""
        return kernels.layernorm(x, self.weight, self.bias, self.eps, out_dtype or self.rt.dtype, rows=rows)


register_part("norm", "rmsnorm", RMSNorm, replace=True)
register_part("norm", "layernorm", LayerNorm, replace=True)
