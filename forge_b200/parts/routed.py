"""A feed-forward made of many small gated feed-forwards ("experts"), of which a router picks ``top`` per token:

    s = sigmoid(Wr x)  (or softmax(Wr x));   the ``top`` largest s choose the experts (the lower index wins a tie)
    y = sum over the chosen e of s_e * Wdown_e (silu(Wgate_e x) * (Wup_e x))          (s_e divided by their sum with ``renormalize``)

Options: experts may be ranked by s + ``correction`` (a number per expert; the weights stay s); the experts may be cut into ``groups``
consecutive blocks of equal size, each ranked by the largest ranking number in it, of which only the ``keep`` best take part; the weights
may be multiplied by ``route_scale``; a ``shared`` feed-forward (any feed-forward part) may run for every token and be added.

The router's arithmetic is fp32.  Three paths, all with everything but the last one's row counts read from device memory:

  by pairs      fewer (token, expert) pairs than experts: each pair on its own streams its expert's rows once (32-bit runs: every
                step below the last path's size, from two tokens on expert by expert with the same numbers to the last bit)
  with room     16-bit steps of up to 127 tokens, and every larger step that a CUDA graph replays: the pairs are ranked by expert into
                a buffer with room for a step's tokens per expert (an expert is chosen at most once per token), every expert's rows go
                through the tensor-core products, and a product whose expert nobody chose is skipped on the device by its row count
  ranked        steps of many tokens: the pairs lie packed by expert, the row counts come to the host (one wait per layer) and
                every expert's rows go through the ordinary matrix products
A token's experts are added up in the router's order in all three.
"""
import torch

from .. import kernels
from ..config.base import ConfigError
from ..weights.loader import TensorSpec
from .base import Part, build_part, register_part
from .linear import Linear


class RoutedExperts(Part):
    graph_safe = True
    SORTED_FROM = 128          # tokens in a step from which the pairs are ranked by expert
    BY_EXPERT_FROM = 2         # ... and from which the path by pairs goes expert by expert (the same numbers, fewer reads)

    def __init__(self, rt, hidden_size, intermediate_size, experts, top, score="sigmoid", renormalize=False, prefix="mlp.",
                 correction=False, groups=0, keep=0, route_scale=1.0, shared=None):
        """``shared``: the PartSpec of a feed-forward part that every token passes through beside its experts, or None."""
        if not 1 <= top <= experts:
            raise ConfigError(f"routed feed-forward: {top} of {experts} experts")
        groups, keep = int(groups or 0), int(keep or 0)
        if groups > 1 and (experts % groups or not 1 <= keep <= groups or top > keep * (experts // groups)):
            raise ConfigError(f"routed feed-forward: {experts} experts in {groups} groups of which {keep} are kept cannot give {top} a token")
        self.correction, self.groups, self.keep, self.route_scale = bool(correction), groups if groups > 1 else 0, keep, float(route_scale)
        self.shared = None if shared is None else build_part("feed_forward", shared, rt)
        self.bias = None
        if score not in ("sigmoid", "softmax"):
            raise ConfigError(f"routed feed-forward: scores are 'sigmoid' or 'softmax', not {score!r}")
        self.rt, self.hidden_size, self.intermediate_size = rt, hidden_size, intermediate_size
        self.experts, self.top, self.score, self.renormalize, self.prefix = experts, top, score, bool(renormalize), prefix

    def _n(self, short):
        return self.prefix + short

    def tensor_specs(self):
        W, F = self.hidden_size, self.intermediate_size
        specs = {}
        for e in range(self.experts):
            specs.update({self._n(f"e{e}.gate"): TensorSpec((F, W)), self._n(f"e{e}.up"): TensorSpec((F, W)),
                          self._n(f"e{e}.down"): TensorSpec((W, F))})
        specs[self._n("router")] = TensorSpec((self.experts, W))
        if self.correction:
            specs[self._n("correction")] = TensorSpec((self.experts,), role="route_bias")
        if self.shared is not None:
            specs.update(self.shared.tensor_specs())
        return specs

    def sub_parts(self):
        return [] if self.shared is None else [self.shared]

    def bind(self, tensors):
        W, F, E = self.hidden_size, self.intermediate_size, self.experts
        self.router = self._vector_f32(tensors[self._n("router")])                     # fp32 whatever the runtime
        self.bias = self._vector_f32(tensors[self._n("correction")]) if self.correction else None
        if self.shared is not None:
            self.shared.bind({n: tensors[n] for n in self.shared.tensor_specs()})
        # one tensor per kind for all experts; gate and up rows alternate so that the product's epilogue sees (gate, up) pairs
        gu = torch.stack([torch.stack([tensors[self._n(f"e{e}.gate")], tensors[self._n(f"e{e}.up")]], dim=1).reshape(2 * F, W)
                          for e in range(E)])
        self.gate_up = self._matrix(gu)                                                # [E, 2F, W]
        self.down = self._matrix(torch.stack([tensors[self._n(f"e{e}.down")] for e in range(E)]))      # [E, W, F]
        self.gate_up_of = [Linear(self.gate_up[e], None, self.rt) for e in range(E)]   # views, no copies
        self.down_of = [Linear(self.down[e], None, self.rt) for e in range(E)]

    def _ranked(self, x, idx, wts):
        """The path of many tokens.  The number of rows of every expert has to be known on the host: one wait per layer."""
        T, W, F = x.shape[0], self.hidden_size, self.intermediate_size
        xg, counts, dest = kernels.moe_sort(x, idx, self.experts)
        counts = counts.tolist()
        act = kernels.new_tensor((T * self.top, F), self.rt.dtype, x.device)
        ys = kernels.new_tensor((T * self.top, W), torch.float32, x.device)
        off = 0
        for e, n in enumerate(counts):
            if n:
                self.gate_up_of[e].forward(xg[off:off + n], epilogue="swiglu", out=act[off:off + n])
                self.down_of[e].forward(act[off:off + n], out=ys[off:off + n])
                off += n
        return kernels.moe_combine(ys, dest, wts)

    def _with_room(self, x, idx, wts):
        """Nothing waits for the device: expert e's rows lie from row e * T on, and its two products are skipped where counts[e] is 0.
        The rows beyond an expert's count hold whatever the buffer held; a product's rows do not mix, and nobody reads theirs."""
        T, W, F, E = x.shape[0], self.hidden_size, self.intermediate_size, self.experts
        xg, counts, dest = kernels.moe_sort(x, idx, E, cap=T)
        act = kernels.new_tensor((E * T, F), self.rt.dtype, x.device)
        ys = kernels.new_tensor((E * T, W), torch.float32, x.device)
        for e in range(E):
            rows, live = slice(e * T, (e + 1) * T), counts[e:e + 1]
            self.gate_up_of[e].forward(xg[rows], epilogue="swiglu", out=act[rows], live=live)
            self.down_of[e].forward(act[rows], out=ys[rows], live=live)
        return kernels.moe_combine(ys, dest, wts)

    def _pairs_fit(self):
        """Whether the path by pairs holds a token's input and its experts' activations in a CTA's shared memory."""
        return self.hidden_size <= 12000 and self.top * self.intermediate_size * 4 <= 200 * 1024

    def forward(self, x, residual):
        """Adds the output into ``residual`` fp32 [T, W], or (``residual`` None) returns it as a new fp32 [T, W]."""
        idx, wts = kernels.moe_route(x, self.router, self.top, softmax=self.score == "softmax", renorm=self.renormalize,
                                     correction=self.bias, groups=self.groups, keep=self.keep, factor=self.route_scale)
        T = x.shape[0]
        tensor_core = self.gate_up_of[0].tensor_core and self.down_of[0].tensor_core
        if T >= self.SORTED_FROM and not torch.cuda.is_current_stream_capturing():
            y = self._ranked(x, idx, wts)
        elif tensor_core and (T * self.top >= self.experts or T >= self.SORTED_FROM or not self._pairs_fit()):
            y = self._with_room(x, idx, wts)
        elif tensor_core:
            y = kernels.moe_pairs(x, idx, wts, self.gate_up, self.down)
        elif x.shape[0] >= self.BY_EXPERT_FROM and kernels.moe_experts_supported(x.shape[0] * self.top, self.hidden_size, self.intermediate_size):
            y = kernels.moe_experts(x, idx, wts, self.gate_up, self.down)
        else:
            y = kernels.moe_pairs(x, idx, wts, self.gate_up, self.down)
        if self.shared is not None:
            self.shared.forward(x, y)              # its last product adds into the experts' sum
        if residual is None:
            return y
        residual.add_(y)
        return residual


register_part("feed_forward", "routed_experts", RoutedExperts, replace=True)
