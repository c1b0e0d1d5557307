"""Mixers that carry a matrix of state per head from token to token instead of a cache of keys and values.

Both have N heads of K channels, keep S [K, K] per head and request in 32-bit (a row of the layer's state tensor per
request slot, zero at admission), make their decay from a low-rank projection, x = W2 tanh(W1 .) + w0, divide every head's
output by its root mean square, multiply by a weight per channel and by a gate, and project back to the model's width.

"wkv" (decay and bonus, with a look at the previous token):
    each of r, k, v, g, w reads h + (h_prev - h) * mu_s;  w_t = exp(-exp(x_t));  gate = silu(g)
    o_t = (S + diag(u) k_t v_t^T)^T r_t;   S <- diag(w_t) S + k_t v_t^T          (the previous token's h is state too)
"general_delta" (generalized delta rule):
    w_t = exp(-exp(-1/2) sigmoid(x_t));  a_t = sigmoid(Wa h + b);  n_t = k_t / sqrt(|k_t|^2 + 1e-6);  gate = sigmoid(g)
    S <- diag(w_t) S - (a_t * n_t)(n_t^T S) + k_t v_t^T;   o_t = S^T r_t

The rank of the decay's projection is read from the file's tensors (``rank`` is only what random weights take).

"gated_write" (HGRN2; N heads of K key and V value channels, state [K, V], no key and no low-rank decay):
    q_t = silu(Wq h);  f_t = l + (1 - l) sigmoid(Wf h + b)  (l: a lower bound per channel);  v_t = Wv h
    S <- diag(f_t) S + (1 - f_t) v_t^T;   o_t = S^T q_t;   every head's o divided by its root mean square, times a weight per
    value channel that the heads share; projected back.  ``out_scale`` multiplies the mixer's output.

"retention" (N heads of K key and V value channels, state [K, V], one fixed decay g_n per head, no softmax, no denominator):
    q_t, k_t rotated by the position (a position part with ``inv_freq``; channel i paired with i + half), k_t times K^-1/2
    S <- g_n S + k_t v_t^T;   o_t = S^T q_t;   every head's o divided by its root mean square (no weight), times silu(Wg h);
    projected back.
"""
import torch

from .. import kernels
from ..config.base import ConfigError
from ..weights.loader import TensorSpec
from .base import Part, StateSpec, register_part
from .linear import Linear


class _StateMixer(Part):
    graph_safe = True       # request boundaries and state rows come from the batch's device tensors (q_start, slots)
    MATRICES = ()

    def __init__(self, rt, hidden_size, num_heads, head_dim, eps, rank=16, names=None, prefix="mix."):
        if head_dim > 128:
            raise ConfigError(f"state mixers take heads of up to 128 channels, not {head_dim}")
        self.rt, self.hidden_size, self.num_heads, self.head_dim = rt, hidden_size, num_heads, head_dim
        self.eps, self.rank, self.prefix = float(eps), int(rank), prefix
        self.names = dict(names or {})

    def _n(self, short):
        return self.names.get(short, self.prefix + short)

    def _common_specs(self):
        W, NK = self.hidden_size, self.num_heads * self.head_dim
        specs = {self._n(m): TensorSpec((NK, W)) for m in self.MATRICES}
        specs.update({self._n("w1"): TensorSpec((-1, W), default_shape=(self.rank, W)),
                      self._n("w2"): TensorSpec((NK, -1), default_shape=(NK, self.rank)),
                      self._n("w0"): TensorSpec((NK,), role="bias"), self._n("norm"): TensorSpec((NK,), role="norm"),
                      self._n("o"): TensorSpec((W, NK))})
        return specs

    def _bind_common(self, tensors):
        w1, w2 = tensors[self._n("w1")], tensors[self._n("w2")]
        if w1.shape[0] != w2.shape[1]:
            from ..weights.loader import WeightError
            raise WeightError(self._n("w1"), wrong=[f"{self._n('w1')} has {w1.shape[0]} rows, {self._n('w2')} {w2.shape[1]} columns"])
        self.w2 = Linear(self._matrix(w2), None, self.rt)
        self.w0 = self._vector_f32(tensors[self._n("w0")])
        self.norm = self._vector_f32(tensors[self._n("norm")])
        self.o = Linear(self._matrix(tensors[self._n("o")]), None, self.rt)
        return w1

    def _decay_input(self, hidden):
        """hidden: (fp32 matrix, first column) of W1's product; returns fp32 [T, N*K], W2 tanh(.) (w0 is added where
        the decay is made)."""
        return self.w2.forward(kernels.tanh_rows(hidden, self.rt.dtype, n=self.w2.in_features))


class WKVMixer(_StateMixer):
    MATRICES = ("r", "k", "v", "g")
    SHIFTED = ("r", "k", "v", "g", "w")

    def tensor_specs(self):
        specs = self._common_specs()
        specs.update({self._n("mu." + s): TensorSpec((self.hidden_size,), role="fraction") for s in self.SHIFTED})
        specs[self._n("u")] = TensorSpec((self.num_heads, self.head_dim), role="bias")
        return specs

    def bind(self, tensors):
        self.w1 = Linear(self._matrix(self._bind_common(tensors)), None, self.rt)
        self.lin = {m: Linear(self._matrix(tensors[self._n(m)]), None, self.rt) for m in self.MATRICES}
        self.mu = torch.stack([self._vector_f32(tensors[self._n("mu." + s)]) for s in self.SHIFTED]).contiguous()
        self.bonus = self._vector_f32(tensors[self._n("u")]).reshape(-1).contiguous()

    def cache_spec(self):
        n = self.num_heads * self.head_dim * self.head_dim
        return StateSpec((n + self.hidden_size,), torch.float32)      # the heads' matrices, then the previous token's input

    def forward(self, x, batch, cache, residual):
        N, K = self.num_heads, self.head_dim
        prev_off = N * K * K
        shifted = kernels.token_shift(x, cache.state, prev_off, batch, self.mu)            # [5, T, W]
        r, k, v, g = (self.lin[m].forward(shifted[i]) for i, m in enumerate(self.MATRICES))
        decay_in = self._decay_input((self.w1.forward(shifted[4]), 0))
        o = kernels.state_scan("decay_bonus", (r, 0), (k, 0), (v, 0), (decay_in, 0), self.w0, cache.state, batch, N, K,
                               bonus=self.bonus, last_in=x, prev_off=prev_off)
        y = kernels.head_finish(o, self.norm, (g, 0), N, K, self.eps, "silu", self.rt.dtype)
        self.o.forward(y, accumulate_into=residual)


class GeneralDeltaMixer(_StateMixer):
    MATRICES = ("r", "k", "v", "g", "a")

    def tensor_specs(self):
        specs = self._common_specs()
        specs[self._n("a.b")] = TensorSpec((self.num_heads * self.head_dim,), role="bias")
        return specs

    def bind(self, tensors):
        w1 = self._bind_common(tensors)
        # r, k, v, g, a and the decay's first matrix read the same input: one product
        self.proj = Linear(self._matrix(torch.cat([tensors[self._n(m)] for m in self.MATRICES] + [w1], dim=0)), None, self.rt)
        self.a0 = self._vector_f32(tensors[self._n("a.b")])

    def cache_spec(self):
        return StateSpec((self.num_heads * self.head_dim * self.head_dim,), torch.float32)

    def forward(self, x, batch, cache, residual):
        N, K = self.num_heads, self.head_dim
        NK = N * K
        p = self.proj.forward(x)                                     # fp32 [T, 5*N*K + rank]: r | k | v | g | a | hidden
        decay_in = self._decay_input((p, 5 * NK))
        o = kernels.state_scan("delta", (p, 0), (p, NK), (p, 2 * NK), (decay_in, 0), self.w0, cache.state, batch, N, K,
                               y=(p, 4 * NK), a0=self.a0)
        y = kernels.head_finish(o, self.norm, (p, 3 * NK), N, K, self.eps, "sigmoid", self.rt.dtype)
        self.o.forward(y, accumulate_into=residual)


class GatedWriteMixer(Part):
    graph_safe = True       # request boundaries and state rows come from the batch's device tensors (q_start, slots)

    def __init__(self, rt, hidden_size, num_heads, head_dim, eps, v_head_dim=None, out_scale=1.0, prefix="mix."):
        if head_dim > 256:
            raise ConfigError(f"the gated-write mixer takes heads of up to 256 key channels, not {head_dim}")
        self.rt, self.hidden_size, self.num_heads, self.head_dim = rt, hidden_size, num_heads, head_dim
        self.v_head_dim = head_dim if v_head_dim is None else v_head_dim
        self.eps, self.out_scale, self.prefix = float(eps), float(out_scale), prefix

    def _n(self, short):
        return self.prefix + short

    def tensor_specs(self):
        W, NK, NV = self.hidden_size, self.num_heads * self.head_dim, self.num_heads * self.v_head_dim
        return {self._n("q"): TensorSpec((NK, W)), self._n("f"): TensorSpec((NK, W)), self._n("f.b"): TensorSpec((NK,), role="bias"),
                self._n("lower"): TensorSpec((NK,), role="fraction"), self._n("v"): TensorSpec((NV, W)),
                self._n("norm"): TensorSpec((self.v_head_dim,), role="norm"), self._n("o"): TensorSpec((W, NV))}

    def bind(self, tensors):
        # q, f and v read the same input: one product
        self.proj = Linear(self._matrix(torch.cat([tensors[self._n(m)] for m in ("q", "f", "v")], dim=0)), None, self.rt)
        self.f_bias = self._vector_f32(tensors[self._n("f.b")])
        self.lower = self._vector_f32(tensors[self._n("lower")])
        self.norm = self._vector_f32(tensors[self._n("norm")])
        self.o = Linear(self._matrix(tensors[self._n("o")]), None, self.rt)

    def cache_spec(self):
        return StateSpec((self.num_heads * self.head_dim * self.v_head_dim,), torch.float32)

    def in_width(self):
        return self.num_heads * (2 * self.head_dim + self.v_head_dim)

    def out_width(self):
        return self.num_heads * self.v_head_dim

    def mix(self, p, col, batch, cache, out=None):
        """p fp32 [T, >= col + in_width]: [q | f | v] from column ``col`` (q and f are overwritten); returns the normed heads
        [T, N*V] (or writes them into ``out`` = (matrix, first column))."""
        N, K, V = self.num_heads, self.head_dim, self.v_head_dim
        NK = N * K
        o = kernels.state_scan("gated_write", (p, col), None, (p, col + 2 * NK), (p, col + NK), self.f_bias, cache.state, batch, N, K,
                               a0=self.lower, KV=V)
        return kernels.head_finish(o, self.norm, None, N, V, self.eps, "none", self.rt.dtype, scale=self.out_scale, out=out)

    def forward(self, x, batch, cache, residual):
        y = self.mix(self.proj.forward(x), 0, batch, cache)          # the projection: fp32 [T, 2*N*K + N*V]
        self.o.forward(y, accumulate_into=residual)


class RetentionMixer(Part):
    graph_safe = True       # positions, request boundaries and state rows come from the batch's device tensors

    def __init__(self, rt, hidden_size, num_heads, head_dim, decay, eps, position, v_head_dim=None, prefix="mix."):
        from .base import build_part
        if head_dim > 256:
            raise ConfigError(f"the retention mixer takes heads of up to 256 key channels, not {head_dim}")
        if len(decay) != num_heads:
            raise ConfigError(f"retention: {len(decay)} decays for {num_heads} heads")
        self.rt, self.hidden_size, self.num_heads, self.head_dim = rt, hidden_size, num_heads, head_dim
        self.v_head_dim = head_dim if v_head_dim is None else v_head_dim
        self.eps, self.prefix = float(eps), prefix
        self.decay = torch.tensor([float(g) for g in decay], dtype=torch.float64).to(torch.float32).to(rt.device)
        self.position = build_part("position", position, rt)
        if not hasattr(self.position, "inv_freq"):
            raise ConfigError("retention rotates inside its own scan and needs a position part with 'inv_freq'")
        self.ones = torch.ones(self.v_head_dim, dtype=torch.float32, device=rt.device)       # the head norm has no weight

    def sub_parts(self):
        return [self.position]

    def _n(self, short):
        return self.prefix + short

    def tensor_specs(self):
        W, NK, NV = self.hidden_size, self.num_heads * self.head_dim, self.num_heads * self.v_head_dim
        return {self._n("q"): TensorSpec((NK, W)), self._n("k"): TensorSpec((NK, W)), self._n("v"): TensorSpec((NV, W)),
                self._n("g"): TensorSpec((NV, W)), self._n("o"): TensorSpec((W, NV))}

    def bind(self, tensors):
        # q, k, v and the gate read the same input: one product
        self.proj = Linear(self._matrix(torch.cat([tensors[self._n(m)] for m in ("q", "k", "v", "g")], dim=0)), None, self.rt)
        self.o = Linear(self._matrix(tensors[self._n("o")]), None, self.rt)

    def cache_spec(self):
        return StateSpec((self.num_heads * self.head_dim * self.v_head_dim,), torch.float32)

    def forward(self, x, batch, cache, residual):
        """Adds the mixer's output into ``residual``, or (``residual`` None) returns it as a new fp32 [T, W]."""
        N, K, V = self.num_heads, self.head_dim, self.v_head_dim
        NK, NV = N * K, N * V
        p = self.proj.forward(x)                                     # fp32 [T, 2*N*K + 2*N*V]: q | k | v | g
        freq = self.position.inv_freq
        o = kernels.retention_scan((p, 0), (p, NK), (p, 2 * NK), batch, freq if freq.numel() else None, K ** -0.5, self.decay,
                                   cache.state, N, K, V)
        y = kernels.head_finish(o, self.ones, (p, 2 * NK + NV), N, V, self.eps, "silu", self.rt.dtype)
        return self.o.forward(y, accumulate_into=residual)


register_part("mixer", "retention", RetentionMixer, replace=True)
register_part("mixer", "gated_write", GatedWriteMixer, replace=True)
register_part("mixer", "wkv", WKVMixer, replace=True)
register_part("mixer", "general_delta", GeneralDeltaMixer, replace=True)
