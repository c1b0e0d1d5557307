"""Three causal softmax attentions whose scores are shaped before the softmax, all on the paged cache and on the same
kernels (``kernels.scored_prepare`` / ``kernels.scored_attention``); query/key heads and value heads may differ in size.

"differential_attention": every head has two maps (q and k carry two vectors of D channels per head, [map 1 | map 2]),
each a softmax of its own over the same values; with a_1, a_2 the maps' outputs
    lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff              (one number for the layer)
    o = a_1 - lambda a_2;   o <- o / sqrt(mean(o^2) + eps) * (1 - diff)
Rotary positions on the first ``rotary_dims`` channels of every map, channel i paired with i + rotary_dims/2.

"distance_attention": no rotation; biases in every projection; an RMS norm over ALL query channels of a token (and all
key channels) with a weight per channel; a query temperature 1 + coef ln(floor((p + 1) / every) + 1) at position p; and
    score(i, j) = scale q(i) . k(j) - r1_h ln(1 + r2_h (i - j))

"masked_attention": no rotation (positions do not enter the scores); optional biases in q, k and v; the scale is a parameter;
optionally  score <- softcap tanh(score / softcap);  and a position i sees j <= i only
    within a sliding ``window``  (i - window < j),  or  within its own ``chunk``  (i // chunk == j // chunk),
chunks counted from the sequence's first position.  Pages whose keys no future query sees go back to the pool.

``out_scale`` multiplies the mixer's output (a mixer that runs beside another with weights of their own).
"""
import math

import torch

from .. import kernels
from ..config.base import ConfigError
from ..weights.loader import TensorSpec
from .base import KVCacheSpec, Part, build_part, register_part
from .linear import Linear


class _ScoredAttention(Part):
    graph_safe = True       # positions, tables, slots and request boundaries are read from the batch's device tensors
    MAPS = 1

    def _sizes(self, rt, hidden_size, num_heads, num_kv_heads, head_dim, v_head_dim, scale, out_scale, prefix):
        if num_heads % num_kv_heads:
            raise ConfigError(f"{num_heads} query heads cannot share {num_kv_heads} key/value heads")
        self.rt, self.hidden_size = rt, hidden_size
        self.num_heads, self.num_kv_heads, self.head_dim = num_heads, num_kv_heads, head_dim
        self.v_head_dim = head_dim if v_head_dim is None else v_head_dim
        self.scale = head_dim ** -0.5 if scale is None else float(scale)
        self.out_scale, self.prefix = float(out_scale), prefix
        self.proj = self.o = None

    def _n(self, short):
        return self.prefix + short

    def cache_spec(self):
        return KVCacheSpec(self.num_kv_heads, self.MAPS * self.head_dim, None, v_head_dim=self.v_head_dim)

    def sub_parts(self):
        return []

    # A mixer that runs beside others may share their input and output products: it says how many columns of the fused
    # projection are its own and how many of the output product's input, and offers ``mix`` (everything between the two).
    def in_width(self):
        return (self.num_heads + self.num_kv_heads) * self.MAPS * self.head_dim + self.num_kv_heads * self.v_head_dim

    def out_width(self):
        return self.num_heads * self.v_head_dim

    def forward(self, x, batch, cache, residual):
        """x [T,W] normed input; cache: the layer's key/value pages; adds the output projection into residual."""
        o = self.mix(self.proj.forward(x), 0, batch, cache)            # the projection: fp32 [T, in_width], biases added
        self.o.forward(o, accumulate_into=residual)

    def _matrix_specs(self, bias):
        W, H, G, D, E, M = self.hidden_size, self.num_heads, self.num_kv_heads, self.head_dim, self.v_head_dim, self.MAPS
        specs = {self._n("q"): TensorSpec((H * M * D, W)), self._n("k"): TensorSpec((G * M * D, W)), self._n("v"): TensorSpec((G * E, W)),
                 self._n("o"): TensorSpec((W, H * E))}
        if bias:
            specs.update({self._n("q.b"): TensorSpec((H * M * D,), role="bias"), self._n("k.b"): TensorSpec((G * M * D,), role="bias"),
                          self._n("v.b"): TensorSpec((G * E,), role="bias"), self._n("o.b"): TensorSpec((W,), role="bias")})
        return specs

    def _bind_matrices(self, tensors, bias):
        rows = torch.cat([tensors[self._n(m)] for m in "qkv"], dim=0)
        b = self._vector_f32(torch.cat([tensors[self._n(m + ".b")].float() for m in "qkv"])) if bias else None
        self.proj = Linear(self._matrix(rows), b, self.rt)              # q, k, v in one product
        ob = self._vector_f32(tensors[self._n("o.b")].float() * self.out_scale) if bias else None
        self.o = Linear(self._matrix(tensors[self._n("o")]), ob, self.rt)


class DifferentialAttention(_ScoredAttention):
    MAPS = 2

    def __init__(self, rt, hidden_size, num_heads, num_kv_heads, head_dim, position, diff, eps, v_head_dim=None, scale=None,
                 out_scale=1.0, prefix="mix."):
        self._sizes(rt, hidden_size, num_heads, num_kv_heads, head_dim, v_head_dim, scale, out_scale, prefix)
        self.diff, self.eps = float(diff), float(eps)
        self.position = build_part("position", position, rt)
        if not hasattr(self.position, "inv_freq"):
            raise ConfigError("this attention rotates inside its own prepare step and needs a position part with 'inv_freq'")
        self.lam = None

    def sub_parts(self):
        return [self.position]

    def tensor_specs(self):
        specs = self._matrix_specs(bias=False)
        specs.update({self._n(v): TensorSpec((self.head_dim,), role="lambda_part") for v in ("lq1", "lk1", "lq2", "lk2")})
        return specs

    def bind(self, tensors):
        self._bind_matrices(tensors, bias=False)
        v = {n: tensors[self._n(n)].to(torch.float64) for n in ("lq1", "lk1", "lq2", "lk2")}
        self.lam = math.exp(float((v["lq1"] * v["lk1"]).sum())) - math.exp(float((v["lq2"] * v["lk2"]).sum())) + self.diff

    def mix(self, proj, col, batch, cache, out=None):
        """proj fp32 [T, >= col + in_width]: [q | k | v] from column ``col``; returns the heads' outputs [T, H*E] (or writes them
        into ``out`` = (matrix, first column))."""
        H, G, D, E = self.num_heads, self.num_kv_heads, self.head_dim, self.v_head_dim
        g = batch.groups[cache.group]
        freq = self.position.inv_freq
        q = kernels.scored_prepare(proj, batch.positions, g.slot_mapping if cache.writable else None,
                                   cache.kv if cache.writable else None, H, G, 2, D, E, cache.page_size, self.rt.dtype,
                                   inv_freq=freq if freq.numel() else None, col=col)
        return kernels.scored_attention(q, cache.kv, g, batch, H, G, 2, D, E, cache.page_size, self.scale, lam=self.lam,
                                        post=1.0 - self.diff, eps=self.eps, out_scale=self.out_scale, out=out)


class DistanceBiasAttention(_ScoredAttention):
    def __init__(self, rt, hidden_size, num_heads, num_kv_heads, head_dim, eps, v_head_dim=None, scale=None, temp_coef=0.0,
                 temp_every=0.0, out_scale=1.0, prefix="mix."):
        """``temp_every`` 0: no query temperature."""
        self._sizes(rt, hidden_size, num_heads, num_kv_heads, head_dim, v_head_dim, scale, out_scale, prefix)
        self.eps, self.temp_coef, self.temp_every = float(eps), float(temp_coef), float(temp_every)
        self.q_norm = self.k_norm = self.r1 = self.r2 = None

    def tensor_specs(self):
        H, G, D = self.num_heads, self.num_kv_heads, self.head_dim
        specs = self._matrix_specs(bias=True)
        specs.update({self._n("q.norm"): TensorSpec((H * D,), role="norm"), self._n("k.norm"): TensorSpec((G * D,), role="norm"),
                      self._n("r1"): TensorSpec((H,), role="fraction"), self._n("r2"): TensorSpec((H,), role="fraction")})
        return specs

    def bind(self, tensors):
        self._bind_matrices(tensors, bias=True)
        self.q_norm, self.k_norm = self._vector_f32(tensors[self._n("q.norm")]), self._vector_f32(tensors[self._n("k.norm")])
        self.r1, self.r2 = self._vector_f32(tensors[self._n("r1")]), self._vector_f32(tensors[self._n("r2")])

    def mix(self, proj, col, batch, cache, out=None):
        """proj fp32 [T, >= col + in_width]: [q | k | v] from column ``col``, biases added; returns the heads' outputs
        [T, H*E] (or writes them into ``out`` = (matrix, first column))."""
        H, G, D, E = self.num_heads, self.num_kv_heads, self.head_dim, self.v_head_dim
        g = batch.groups[cache.group]
        q = kernels.scored_prepare(proj, batch.positions, g.slot_mapping if cache.writable else None,
                                   cache.kv if cache.writable else None, H, G, 1, D, E, cache.page_size, self.rt.dtype,
                                   q_norm=self.q_norm, k_norm=self.k_norm, eps=self.eps, temp_coef=self.temp_coef,
                                   temp_every=self.temp_every, col=col)
        return kernels.scored_attention(q, cache.kv, g, batch, H, G, 1, D, E, cache.page_size, self.scale, r1=self.r1, r2=self.r2,
                                        out_scale=self.out_scale, out=out)


class MaskedAttention(_ScoredAttention):
    def __init__(self, rt, hidden_size, num_heads, num_kv_heads, head_dim, v_head_dim=None, scale=None, window=None, chunk=None,
                 softcap=None, qkv_bias=False, out_scale=1.0, prefix="mix."):
        """``window`` / ``chunk``: None or a number of positions (both may be given: a key must pass both); ``softcap``: None or the
        cap; ``qkv_bias``: tensors ``q.b``, ``k.b``, ``v.b`` are added in the projection."""
        self._sizes(rt, hidden_size, num_heads, num_kv_heads, head_dim, v_head_dim, scale, out_scale, prefix)
        self.window, self.chunk = (int(window) if window else None), (int(chunk) if chunk else None)
        self.softcap, self.qkv_bias = (float(softcap) if softcap else None), bool(qkv_bias)
        if (self.window is not None and self.window < 1) or (self.chunk is not None and self.chunk < 1) or \
                (self.softcap is not None and not self.softcap > 0.0):
            raise ConfigError(f"masked attention: window {window}, chunk {chunk}, softcap {softcap}")

    def tensor_specs(self):
        W, H, G, D, E = self.hidden_size, self.num_heads, self.num_kv_heads, self.head_dim, self.v_head_dim
        specs = {self._n("q"): TensorSpec((H * D, W)), self._n("k"): TensorSpec((G * D, W)), self._n("v"): TensorSpec((G * E, W)),
                 self._n("o"): TensorSpec((W, H * E))}
        if self.qkv_bias:
            specs.update({self._n("q.b"): TensorSpec((H * D,), role="bias"), self._n("k.b"): TensorSpec((G * D,), role="bias"),
                          self._n("v.b"): TensorSpec((G * E,), role="bias")})
        return specs

    def bind(self, tensors):
        rows = torch.cat([tensors[self._n(m)] for m in "qkv"], dim=0)
        b = self._vector_f32(torch.cat([tensors[self._n(m + ".b")].float() for m in "qkv"])) if self.qkv_bias else None
        self.proj = Linear(self._matrix(rows), b, self.rt)              # q, k, v in one product, the biases in its epilogue
        self.o = Linear(self._matrix(tensors[self._n("o")]), None, self.rt)

    def cache_spec(self):
        return KVCacheSpec(self.num_kv_heads, self.head_dim, self.window, v_head_dim=self.v_head_dim, chunk=self.chunk)

    def forward(self, x, batch, cache, residual):
        """Adds the mixer's output into ``residual``, or (``residual`` None) returns it as a new fp32 [T, W]."""
        o = self.mix(self.proj.forward(x), 0, batch, cache)
        return self.o.forward(o, accumulate_into=residual)

    def mix(self, proj, col, batch, cache, out=None):
        """proj fp32 [T, >= col + in_width]: [q | k | v] from column ``col``, biases added; returns the heads' outputs
        [T, H*E] (or writes them into ``out`` = (matrix, first column))."""
        H, G, D, E = self.num_heads, self.num_kv_heads, self.head_dim, self.v_head_dim
        g = batch.groups[cache.group]
        q = kernels.scored_prepare(proj, batch.positions, g.slot_mapping if cache.writable else None,
                                   cache.kv if cache.writable else None, H, G, 1, D, E, cache.page_size, self.rt.dtype, col=col)
        return kernels.scored_attention(q, cache.kv, g, batch, H, G, 1, D, E, cache.page_size, self.scale, out_scale=self.out_scale,
                                        out=out, window=self.window or 0, chunk=self.chunk or 0, softcap=self.softcap or 0.0)


register_part("mixer", "differential_attention", DifferentialAttention, replace=True)
register_part("mixer", "masked_attention", MaskedAttention, replace=True)
register_part("mixer", "distance_attention", DistanceBiasAttention, replace=True)
