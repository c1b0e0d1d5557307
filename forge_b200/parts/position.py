"""Position encodings applied to q and k on their way into attention and the cache.

"rope": half-split rotary embedding of the whole head (reference: src/operators/cuda/cuda_rope.cu:8-34,
generic_engine.cpp:428-433).  "none": no encoding (keys are stored as projected).  Both are one fused
kernel that also writes k and v into the paged cache.

A position part may also offer its encoding to the decode step's one-launch attention kernel, which rotates
q and k itself: ``fused_decode()`` returns the kernel's parameters, or None.  Only a part whose
``encode_and_store`` computes exactly what that kernel computes may return them; a subclass with other
arithmetic inherits None and keeps one path for prompt and decode steps.
"""
from .. import kernels
from .base import Part, register_part


class RotaryEmbedding(Part):
    rotary = True
    graph_safe = True       # angles come from ``positions`` on the device

    def __init__(self, rt, head_dim, theta=10000.0):
        self.rt, self.head_dim, self.theta = rt, int(head_dim), float(theta)

    def fused_decode(self):
        """{"theta", "rotary"} for the decode attention kernel that encodes by itself, or None.  The kernel
        hard-wires the half-split rotation of the whole head, so only the two stock classes offer it."""
        if type(self) not in (RotaryEmbedding, NoPosition):
            return None
        return {"theta": self.theta, "rotary": self.rotary}

    def replay_tensors(self):
        return [] if type(self) in (RotaryEmbedding, NoPosition) else None      # no tensors: the angles come from positions

    def replay_key(self):
        return (type(self).__name__, self.head_dim, self.theta, self.rotary)

    def _table(self, positions, batch, by_pair=False):
        """The step's cos/sin table, computed once per step (kept in the batch's ``attention_plan``), not once per
        layer.  A batch that a CUDA graph replays keeps no table: the table of the captured step would be replayed
        with every later step's positions.  ``by_pair``: the layout [head_dim/2, tokens, 2] that the fused projection
        reads."""
        if not self.rotary or batch is None or getattr(batch, "decode_only", False):
            return None
        key = ("rope", self.head_dim, self.theta, positions.data_ptr(), by_pair)
        table = batch.attention_plan.get(key)
        if table is None:
            table = batch.attention_plan[key] = kernels.rope_table(positions, self.head_dim, self.theta, by_pair=by_pair)
        return table

    def fused_projection(self, positions, batch):
        """For the q/k/v product whose epilogue encodes and stores by itself (prompt portions): {"table": the step's
        (cos, sin) table by pair, or None for no rotation}, or None if this part does not offer it.  As with
        ``fused_decode`` only the stock classes do: that epilogue computes the half-split rotation of the whole head."""
        if type(self) not in (RotaryEmbedding, NoPosition) or batch is None or getattr(batch, "decode_only", False):
            return None
        return {"table": self._table(positions, batch, by_pair=True)}

    def encode_and_store(self, qkv, positions, slot_mapping, kv_cache, num_heads, num_kv_heads, page_size, batch=None):
        """``batch`` (optional): the step's batch, which keeps the step's table of angles."""
        table = self._table(positions, batch) if qkv.shape[0] >= 64 else None
        return kernels.rope_kv_write(qkv, positions, slot_mapping, kv_cache, num_heads, num_kv_heads, self.head_dim,
                                     page_size, self.theta, self.rt.dtype, rotary=self.rotary, table=table)


class NoPosition(RotaryEmbedding):
    rotary = False

    def __init__(self, rt, head_dim):
        super().__init__(rt, head_dim, 1.0)


class PairedRotary(Part):
    """Rotary encoding of neighbouring channels (2i, 2i+1) on the first ``rotary_dims`` channels of a head; the rest pass
    unchanged.  Pair i turns by position * theta^(-2i/rotary_dims); the frequencies are worked out in 64-bit on the host
    and kept as a small fp32 table, the angles and their sines are 32-bit on the device.  It offers no ``encode_and_store``:
    the mixers that use it rotate inside their own prepare step (``kernels.headmix_prepare``) and ask for ``inv_freq``."""
    graph_safe = True

    def __init__(self, rt, head_dim, rotary_dims=None, theta=10000.0, scaling=None):
        """``scaling`` {"factor", "original", "fast", "slow"} (optional): the pairs that turn fewer than ``slow`` times within
        ``original`` positions are slowed down by ``factor``, those that turn more than ``fast`` times are left alone, a ramp
        over the pair index between the two; cos and sin are then multiplied by ``amplitude`` = 0.1 ln(factor) + 1."""
        import math
        import torch
        self.rt, self.head_dim, self.theta = rt, int(head_dim), float(theta)
        self.rotary_dims = self.head_dim if rotary_dims is None else int(rotary_dims)
        if self.rotary_dims % 2 or not 0 <= self.rotary_dims <= self.head_dim:
            from ..config.base import ConfigError
            raise ConfigError(f"rotary encoding of {self.rotary_dims} channels does not fit heads of {self.head_dim}")
        i = torch.arange(self.rotary_dims // 2, dtype=torch.float64)
        freq = torch.pow(torch.tensor(self.theta, dtype=torch.float64), -2.0 * i / max(1, self.rotary_dims))
        self.amplitude = 1.0
        if scaling and self.rotary_dims:
            from ..config.base import ConfigError
            try:
                factor, orig = float(scaling["factor"]), float(scaling["original"])
                fast, slow = float(scaling["fast"]), float(scaling["slow"])
            except (KeyError, TypeError, ValueError):
                raise ConfigError("a rotation's scaling needs the numbers factor, original, fast and slow") from None
            if not (factor > 0.0 and orig > 0.0 and fast > 0.0 and slow > 0.0 and self.theta > 1.0):
                raise ConfigError("a rotation's scaling needs positive numbers and a base above one")

            def pair_that_turns(times):      # the (fractional) pair index whose wave fits ``times`` times into ``orig`` positions
                return self.rotary_dims * math.log(orig / (2.0 * math.pi * times)) / (2.0 * math.log(self.theta))
            lo = max(math.floor(pair_that_turns(fast)), 0)
            hi = min(math.ceil(pair_that_turns(slow)), self.rotary_dims - 1)
            ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
            freq = freq / factor * ramp + freq * (1.0 - ramp)
            self.amplitude = 0.1 * math.log(factor) + 1.0
        self.inv_freq = freq.to(torch.float32).to(rt.device)


class SplitHalfRotary(PairedRotary):
    """The same frequencies, but channel i of the first ``rotary_dims`` channels is paired with channel i + rotary_dims/2
    (the rest pass unchanged).  Like its base it only keeps ``inv_freq``; the mixer's prepare step rotates."""


register_part("position", "rope", RotaryEmbedding, replace=True)
register_part("position", "rope_halves", SplitHalfRotary, replace=True)
register_part("position", "rope_pairs", PairedRotary, replace=True)
register_part("position", "none", NoPosition, replace=True)
