"""Attention whose keys and values are made from one small latent per token.

With h the mixer's input, H heads, D unrotated and R rotated query/key channels a head, E value channels, C the key/value
latent's width and Cq the query latent's:

    cq = rmsnorm(Wdq h) * wq;            q_h = Wuq_h cq = [qf_h (D) | qr_h (R)],  qr_h rotated by the position
    [c' | kr'] = Wdkv h;                 c = rmsnorm(c') * wc;   kr = kr' rotated by the position (one for all heads)
    score_h(i, j) = scale (qf_h(i) . Wuk_h c(j) + qr_h(i) . kr(j)),  causal softmax over j <= i
    o_h(i) = Wuv_h sum_j p_h(i, j) c(j);   output = Wo [o_1 .. o_H]

A token leaves the row [c | kr] in the cache and nothing else.  The per-head matrices move to the query and the output
(qa_h = [Wuk_h^T qf_h | qr_h] attends over the rows themselves, Wuv_h is applied to the weighted sum of latents), so keys
and values per head are never formed: one path for prompt portions and single tokens.  A layer with ``cache_from`` has no
Wdkv: it reads the rows that the named layer wrote, with matrices of its own.

The rotation pairs channel 2i with 2i+1; its frequencies (and the factor on cos and sin) come from the position part.

Options, each a constructor parameter: ``window`` (position i sees j only if i - j < window; the rows behind every future query's
window go back to the pool), ``sink`` (one learned number per head, b_h: the softmax denominator becomes sum_j exp(score_j) + exp(b_h), as if
one more key with the unscaled score b_h and a zero value were always visible), ``out_gate`` (the concatenated heads are multiplied by sigmoid(Wg h) before Wo; Wg rides
in the down-projections' product).
"""
import torch

from .. import kernels
from ..config.base import ConfigError
from ..weights.loader import TensorSpec
from .base import KVCacheSpec, Part, build_part, register_part
from .linear import Linear


class LatentAttention(Part):
    graph_safe = True       # positions, tables, slots and request boundaries are read from the batch's device tensors

    def __init__(self, rt, hidden_size, num_heads, head_dim, rot_dim, v_head_dim, kv_rank, q_rank, scale, eps, position,
                 own_latent=True, prefix="mix.", window=None, sink=False, out_gate=False):
        if rot_dim % 2:
            raise ConfigError(f"latent attention: the rotated part has {rot_dim} channels, an odd number")
        self.rt, self.hidden_size, self.num_heads = rt, hidden_size, num_heads
        self.head_dim, self.rot_dim, self.v_head_dim = head_dim, rot_dim, v_head_dim
        self.kv_rank, self.q_rank, self.scale, self.eps = kv_rank, q_rank, float(scale), float(eps)
        self.own_latent, self.prefix = bool(own_latent), prefix
        self.window, self.sink, self.out_gate = (int(window) if window else None), bool(sink), bool(out_gate)
        if self.window is not None and self.window < 1:
            raise ConfigError(f"latent attention: a window of {window} positions")
        self.sinks = None
        self.position = build_part("position", position, rt)
        if not hasattr(self.position, "inv_freq") or 2 * self.position.inv_freq.numel() != rot_dim:
            raise ConfigError("latent attention rotates inside its own kernels and needs a position part with 'inv_freq' over the "
                              "whole of the rotated part")

    def sub_parts(self):
        return [self.position]

    def _n(self, short):
        return self.prefix + short

    def tensor_specs(self):
        W, H, D, R, E, C, Cq = self.hidden_size, self.num_heads, self.head_dim, self.rot_dim, self.v_head_dim, self.kv_rank, self.q_rank
        specs = {self._n("dq"): TensorSpec((Cq, W)), self._n("dq.norm"): TensorSpec((Cq,), role="norm"),
                 self._n("uq"): TensorSpec((H * (D + R), Cq)), self._n("uk"): TensorSpec((H * D, C)), self._n("uv"): TensorSpec((H * E, C)),
                 self._n("o"): TensorSpec((W, H * E))}
        if self.own_latent:
            specs.update({self._n("dkv"): TensorSpec((C + R, W)), self._n("dkv.norm"): TensorSpec((C,), role="norm")})
        if self.sink:
            specs[self._n("sink")] = TensorSpec((H,), role="bias")
        if self.out_gate:
            specs[self._n("g")] = TensorSpec((H * E, W))
        return specs

    def bind(self, tensors):
        H, D, E, C = self.num_heads, self.head_dim, self.v_head_dim, self.kv_rank
        down = [tensors[self._n("dq")]] + ([tensors[self._n("dkv")]] if self.own_latent else []) + \
            ([tensors[self._n("g")]] if self.out_gate else [])
        self.down = Linear(self._matrix(torch.cat(down, dim=0)), None, self.rt)          # the down-projections (and the gate): one product
        self.sinks = self._vector_f32(tensors[self._n("sink")]) if self.sink else None
        self.wq = self._vector_f32(tensors[self._n("dq.norm")])
        self.wc = self._vector_f32(tensors[self._n("dkv.norm")]) if self.own_latent else None
        self.uq = Linear(self._matrix(tensors[self._n("uq")]), None, self.rt)
        # per head [inputs, outputs]: Wuk_h as stored ([D, C]: it is applied transposed, to the query), Wuv_h transposed ([C, E])
        self.uk = self._matrix(tensors[self._n("uk")].reshape(H, D, C))
        self.uv = self._matrix(tensors[self._n("uv")].reshape(H, E, C).transpose(1, 2))
        self.o = Linear(self._matrix(tensors[self._n("o")]), None, self.rt)

    def cache_spec(self):
        # one key/value head whose rows are [c | kr]; no separate values (they are a row's first C channels)
        return KVCacheSpec(1, self.kv_rank + self.rot_dim, self.window, v_head_dim=0)

    def forward(self, x, batch, cache, residual):
        """Adds the mixer's output into ``residual``, or (``residual`` None) returns it as a new fp32 [T, W]."""
        H, D, R, E, C, Cq = self.num_heads, self.head_dim, self.rot_dim, self.v_head_dim, self.kv_rank, self.q_rank
        g = batch.groups[cache.group]
        freq, amp = self.position.inv_freq, self.position.amplitude
        store = self.own_latent and cache.writable
        proj = self.down.forward(x)                                                    # fp32 [T, Cq (+ C + R) (+ H*E)]
        cq = kernels.latent_prepare(proj, batch, g.slot_mapping if store else None, cache.kv if store else None, freq, amp,
                                    self.wq, self.wc, Cq, C if self.own_latent else 0, R, self.eps, self.rt.dtype)
        q = self.uq.forward(cq)                                                        # fp32 [T, H*(D+R)]
        qa = kernels.head_linear(q, self.uk, H, D, C, self.rt.dtype, R=R, positions=batch.positions, freq=freq, amp=amp)
        lat = kernels.latent_attention(qa, cache.kv, g, batch, H, C, R, cache.page_size, self.scale, window=self.window or 0, sink=self.sinks)
        gate = (proj, Cq + (C + R if self.own_latent else 0)) if self.out_gate else None
        o = kernels.head_linear(lat, self.uv, H, C, E, self.rt.dtype, gate=gate)
        return self.o.forward(o, accumulate_into=residual)


register_part("mixer", "latent_attention", LatentAttention, replace=True)
