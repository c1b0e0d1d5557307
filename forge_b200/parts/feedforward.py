"""Gated feed-forward:  residual += ( act(x.Wg^T) * (x.Wu^T) ) . Wd^T, act = silu ("swiglu",
reference: src/inference/engines/generic_engine.cpp:776-780, 809, 1080) or the tanh form of gelu ("geglu").  Gate and up are one matrix
product: their rows are interleaved at load time (row 2j = gate j, row 2j+1 = up j) so the product's
epilogue sees each (gate, up) pair side by side.
"""
import torch

from ..weights.loader import TensorSpec
from .base import Part, register_part
from .linear import Linear

DEFAULT_NAMES = {"gate": "mlp.gate_proj", "up": "mlp.up_proj", "down": "mlp.down_proj"}


class SwiGLU(Part):
    graph_safe = True
    activation = "swiglu"          # the name of the product's gated epilogue

    def __init__(self, rt, hidden_size, intermediate_size, names=None, suffix=".weight"):
        """``names``: the three matrices' tensor names without ``suffix`` (a design whose files say "mlp.gate" gives
        suffix "")."""
        self.rt, self.hidden_size, self.intermediate_size = rt, hidden_size, intermediate_size
        self.names = {k: v + suffix for k, v in {**DEFAULT_NAMES, **(names or {})}.items()}
        self.gate_up = self.down = None

    def tensor_specs(self):
        n, H, I = self.names, self.hidden_size, self.intermediate_size
        return {n["gate"]: TensorSpec((I, H)), n["up"]: TensorSpec((I, H)), n["down"]: TensorSpec((H, I))}

    def bind(self, tensors):
        n = self.names
        g, u = tensors[n["gate"]], tensors[n["up"]]
        gu = torch.stack([g, u], dim=1).reshape(2 * self.intermediate_size, self.hidden_size)
        self.gate_up = Linear(self._matrix(gu), None, self.rt)
        self.down = Linear(self._matrix(tensors[n["down"]]), None, self.rt)

    def replay_tensors(self):
        return self.gate_up.replay_tensors() + self.down.replay_tensors() if type(self) is SwiGLU else None

    def replay_key(self):
        return (self.activation, self.gate_up.replay_key(), self.down.replay_key())

    def forward(self, x, residual):
        """Adds the output into ``residual``, or (``residual`` None) returns it as a new fp32 [T, H]."""
        act = self.gate_up.forward(x, epilogue=self.activation)    # [T,I] in the activation type
        return self.down.forward(act, accumulate_into=residual)


class GeGLU(SwiGLU):
    """The same with gelu_tanh(g) = g/2 (1 + tanh(sqrt(2/pi) (g + 0.044715 g^3))) on the gate."""
    activation = "geglu"


class DenseFeedForward(Part):
    """Ungated feed-forward:  residual += act(x.Wu^T) . Wd^T; ``activation``: "gelu" (the exact one, with erf),
    "gelu_tanh" or "silu"; ``names``: the two matrices' tensor names."""
    graph_safe = True

    def __init__(self, rt, hidden_size, intermediate_size, activation="gelu", names=None):
        from .. import kernels
        if activation not in kernels.ACTIVATIONS:
            from ..config.base import ConfigError
            raise ConfigError(f"feed-forward activation must be one of {sorted(kernels.ACTIVATIONS)}, got {activation!r}")
        self.rt, self.hidden_size, self.intermediate_size, self.activation = rt, hidden_size, intermediate_size, activation
        self.names = {"up": "mlp.up", "down": "mlp.down", **(names or {})}
        self.up = self.down = None

    def tensor_specs(self):
        n, H, I = self.names, self.hidden_size, self.intermediate_size
        return {n["up"]: TensorSpec((I, H)), n["down"]: TensorSpec((H, I))}

    def bind(self, tensors):
        self.up = Linear(self._matrix(tensors[self.names["up"]]), None, self.rt)
        self.down = Linear(self._matrix(tensors[self.names["down"]]), None, self.rt)

    def forward(self, x, residual):
        act = self.up.forward(x, epilogue=self.activation)          # [T,I] in the activation type
        self.down.forward(act, accumulate_into=residual)


class NoFeedForward(Part):
    """A layer without a feed-forward: adds nothing."""
    graph_safe = True

    def __init__(self, rt):
        self.rt = rt

    def forward(self, x, residual):
        return None


register_part("feed_forward", "swiglu", SwiGLU, replace=True)
register_part("feed_forward", "geglu", GeGLU, replace=True)
register_part("feed_forward", "dense", DenseFeedForward, replace=True)
register_part("feed_forward", "none", NoFeedForward, replace=True)
