"""Arrangements of a layer's parts around the fp32 residual stream.

"pre_norm":  r += mixer(norm_in(r));  r += feed_forward(norm_post(r))     (a layer without feed-forward has one norm)
(reference: src/inference/engines/generic_engine.cpp:931-938, 1045-1052, 1080).
"parallel":  r += mixer(norm_a(r)) + feed_forward(norm_b(r)), both branches of the same r.  The additions happen in
the epilogue of each part's last matrix product, in fp32.
"sandwich":  r += m * norm_b(mixer(norm_a(r)));  r += m * norm_d(feed_forward(norm_c(r))): every sublayer's OUTPUT goes
through an RMS norm of its own before it joins the stream, times a number m.  The output norm, the addition and the next
sublayer's input norm are one kernel.
"hyper_connections":  the stream is S copies x_1 .. x_S (all equal to the embedding output at the start; their sum is what the
model's last norm reads).  Around sublayer q (1: mixer, 2: feed-forward), with weights in_q [S], out_q [S], mix_q [S, S]:
    u = sum_s in_q[s] x_s;   y = sublayer(norm_q(u));   x_t <- sum_s mix_q[s, t] x_s + out_q[t] y   (all t at once, from the old copies)
in place of the residual sum.  A sublayer's write and the next sublayer's read and norm are one kernel, also across layers: where the
model says which block runs next (``batch.shared["following_block"]``), a layer's last write leaves that block's first input.
"""
from ..weights.loader import TensorSpec  # noqa: F401  (re-exported for part authors)
from .base import Part, build_part, register_part


class PreNormBlock(Part):
    graph_safe = True       # the arrangement itself looks at nothing of the step; its parts answer for themselves

    def sub_parts(self):
        return [p for p in (self.mixer, self.feed_forward, self.norm_in, self.norm_post) if p is not None]
    NORM_NAMES = {"input": "input_layernorm.", "post_mixer": "post_attention_layernorm."}

    def __init__(self, rt, layer_spec):
        self.rt = rt
        self.mixer = build_part("mixer", layer_spec.mixer, rt)
        self.feed_forward = build_part("feed_forward", layer_spec.feed_forward, rt)
        self.norm_in = build_part("norm", layer_spec.norms["input"], rt)
        post = layer_spec.norms.get("post_mixer")
        self.norm_post = None if post is None else build_part("norm", post, rt)
        self.norm_prefixes = {**self.NORM_NAMES, **(layer_spec.norm_prefixes or {})}

    def _children(self):
        out = [("", self.mixer), ("", self.feed_forward), (self.norm_prefixes["input"], self.norm_in)]
        return out if self.norm_post is None else out + [(self.norm_prefixes["post_mixer"], self.norm_post)]

    def tensor_specs(self):
        specs = {}
        for prefix, part in self._children():
            for name, s in part.tensor_specs().items():
                specs[prefix + name] = s
        return specs

    def bind(self, tensors):
        for prefix, part in self._children():
            part.bind({name: tensors[prefix + name] for name in part.tensor_specs() if prefix + name in tensors})

    def fused_decode(self):
        """What the kernel that runs all layers of a decode step at once needs of this layer, or None: the layer
        must be exactly the stock arrangement of the stock parts (that kernel computes RMSNorm, rotary attention
        over the paged cache and SwiGLU, and nothing else), in bfloat16 on the tensor-core products."""
        from .attention import GQAAttention
        from .feedforward import SwiGLU
        from .norm import RMSNorm
        m, f, n1, n2 = self.mixer, self.feed_forward, self.norm_in, self.norm_post
        if n2 is None or type(self) is not PreNormBlock or type(m) is not GQAAttention or type(f) is not SwiGLU \
                or type(n1) is not RMSNorm or type(n2) is not RMSNorm or self.rt.full_precision:
            return None
        pos = m.position.fused_decode() if hasattr(m.position, "fused_decode") else None
        if pos is None or m.out_bias or n1.eps != n2.eps or m.qkv is None:
            return None
        if not all(lin.tensor_core for lin in (m.qkv, m.o, f.gate_up, f.down)):
            return None
        return {"hidden": m.hidden_size, "intermediate": f.intermediate_size, "num_heads": m.num_heads,
                "num_kv_heads": m.num_kv_heads, "head_dim": m.head_dim, "theta": pos["theta"], "rotary": pos["rotary"],
                "eps": n1.eps, "window": m.window or 0, "scale": m.scale,
                "tensors": {"wqkv": m.qkv.weight, "wo": m.o.weight, "wgu": f.gate_up.weight, "wdown": f.down.weight,
                            "norm1": n1.weight, "norm2": n2.weight, "bias": m.qkv.bias}}

    def _replay_parts(self):
        from .base import replay_of
        if self.norm_post is None:
            return None
        parts = [replay_of(p) for p in (self.norm_in, self.mixer, self.norm_post, self.feed_forward)]
        return None if type(self) is not PreNormBlock or any(p is None for p in parts) else parts

    def replay_tensors(self):
        parts = self._replay_parts()
        return None if parts is None else [t for _, tensors in parts for t in tensors]

    def replay_key(self):
        parts = self._replay_parts()
        return None if parts is None else ("pre_norm",) + tuple(k for k, _ in parts)

    def forward(self, residual, batch, cache):
        x = self.norm_in.forward(residual)
        self.mixer.forward(x, batch, cache, residual)
        if self.norm_post is not None:
            x = self.norm_post.forward(residual)
            self.feed_forward.forward(x, residual)


class ParallelBlock(Part):
    """Both branches read the residual stream as the layer found it: the two norms run before either branch adds its
    output.  ``norms``: {"mixer": spec, "feed_forward": spec or None}; a norm's spec carries its tensor's name."""
    graph_safe = True

    def sub_parts(self):
        return [p for p in (self.mixer, self.feed_forward, self.norm_mixer, self.norm_ff) if p is not None]

    def __init__(self, rt, layer_spec):
        self.rt = rt
        self.mixer = build_part("mixer", layer_spec.mixer, rt)
        self.feed_forward = build_part("feed_forward", layer_spec.feed_forward, rt)
        self.norm_mixer = build_part("norm", layer_spec.norms["mixer"], rt)
        ff_norm = layer_spec.norms.get("feed_forward")
        self.norm_ff = None if ff_norm is None else build_part("norm", ff_norm, rt)

    def _children(self):
        return [p for p in (self.mixer, self.feed_forward, self.norm_mixer, self.norm_ff) if p is not None]

    def tensor_specs(self):
        specs = {}
        for part in self._children():
            specs.update(part.tensor_specs())
        return specs

    def bind(self, tensors):
        for part in self._children():
            part.bind({name: tensors[name] for name in part.tensor_specs() if name in tensors})

    def _norms(self, residual):
        from .. import kernels
        from .norm import RMSNorm
        a, b = self.norm_mixer, self.norm_ff
        if b is None:
            return a.forward(residual), None
        if type(a) is RMSNorm and type(b) is RMSNorm and a.eps == b.eps and a.size == b.size:
            return kernels.rmsnorm_pair(residual, a.weight, b.weight, a.eps, self.rt.dtype)      # one read of the residual
        return a.forward(residual), b.forward(residual)

    def forward(self, residual, batch, cache):
        x, x_ff = self._norms(residual)
        self.mixer.forward(x, batch, cache, residual)
        if x_ff is not None:
            self.feed_forward.forward(x_ff, residual)


class SandwichBlock(Part):
    """``norms``: {"mixer_in", "mixer_out", "ff_in", "ff_out"} (the last two None in a layer without feed-forward), all RMS norms
    with one eps; ``layer_spec.block_params``: {"residual_mult": m}.  Mixer and feed-forward are called without a stream to add
    into and return their output."""
    graph_safe = True

    def sub_parts(self):
        return [p for p in (self.mixer, self.feed_forward, *self.norms.values()) if p is not None]

    def __init__(self, rt, layer_spec):
        from ..config.base import ConfigError
        from .norm import RMSNorm
        self.rt = rt
        self.mult = float((layer_spec.block_params or {}).get("residual_mult", 1.0))
        self.mixer = build_part("mixer", layer_spec.mixer, rt)
        self.feed_forward = build_part("feed_forward", layer_spec.feed_forward, rt)
        self.norms = {k: None if layer_spec.norms.get(k) is None else build_part("norm", layer_spec.norms[k], rt)
                      for k in ("mixer_in", "mixer_out", "ff_in", "ff_out")}
        present = [n for n in self.norms.values() if n is not None]
        if self.norms["mixer_in"] is None or self.norms["mixer_out"] is None or (self.norms["ff_in"] is None) != (self.norms["ff_out"] is None):
            raise ConfigError("a sandwich layer needs a norm before and after its mixer, and both or none around its feed-forward")
        if any(not isinstance(n, RMSNorm) or n.eps != present[0].eps for n in present):
            raise ConfigError("a sandwich layer's norms are RMS norms with one eps")

    def _children(self):
        return [p for p in (self.mixer, self.feed_forward, *self.norms.values()) if p is not None]

    def tensor_specs(self):
        specs = {}
        for part in self._children():
            specs.update(part.tensor_specs())
        return specs

    def bind(self, tensors):
        for part in self._children():
            part.bind({name: tensors[name] for name in part.tensor_specs() if name in tensors})

    def forward(self, residual, batch, cache):
        from .. import kernels
        n = self.norms
        y = self.mixer.forward(n["mixer_in"].forward(residual), batch, cache, None)
        if n["ff_in"] is None:
            kernels.rmsnorm_add(y, n["mixer_out"].weight, residual, n["mixer_out"].eps, self.mult)
            return
        x = kernels.rmsnorm_add(y, n["mixer_out"].weight, residual, n["mixer_out"].eps, self.mult, w_next=n["ff_in"].weight,
                                out_dtype=self.rt.dtype)
        y = self.feed_forward.forward(x, None)
        kernels.rmsnorm_add(y, n["ff_out"].weight, residual, n["ff_out"].eps, self.mult)


class HyperConnectionBlock(Part):
    """``norms``: {"mixer_in", "ff_in"} (the second None in a layer without feed-forward), RMS norms; ``layer_spec.block_params``:
    {"streams": S}.  ``residual`` is fp32 [T, S*W], a token's copies side by side.  Mixer and feed-forward are called without a
    stream to add into and return their output.  Tensors: ``hc1.in``, ``hc1.out``, ``hc1.mix``, and ``hc2.*`` with a feed-forward."""
    graph_safe = True

    def sub_parts(self):
        return [p for p in (self.mixer, self.feed_forward, *self.norms.values()) if p is not None]

    def __init__(self, rt, layer_spec):
        from ..config.base import ConfigError
        from .norm import RMSNorm
        self.rt = rt
        self.streams = int((layer_spec.block_params or {}).get("streams", 1))
        if self.streams < 1:
            raise ConfigError(f"a stream of {self.streams} copies")
        self.mixer = build_part("mixer", layer_spec.mixer, rt)
        self.feed_forward = build_part("feed_forward", layer_spec.feed_forward, rt)
        self.norms = {k: None if layer_spec.norms.get(k) is None else build_part("norm", layer_spec.norms[k], rt) for k in ("mixer_in", "ff_in")}
        # the norm of a feed-forward that the layer does not have: only so that its weight, if a file holds one, has a name
        spare = layer_spec.norms.get("ff_in_unused")
        self.spare_norm = None if spare is None else build_part("norm", spare, rt)
        if self.norms["mixer_in"] is None or any(n is not None and type(n) is not RMSNorm for n in self.norms.values()):
            raise ConfigError("a layer on a stream of several copies needs an RMS norm before its mixer (and one before its feed-forward)")
        self.weights = {}

    def _children(self):
        return [p for p in (self.mixer, self.feed_forward, *self.norms.values()) if p is not None]

    def _sublayers(self):
        return (1, 2) if self.norms["ff_in"] is not None else (1,)

    def tensor_specs(self):
        S = self.streams
        specs = {}
        for part in self._children():
            specs.update(part.tensor_specs())
        for q in (1, 2):
            # a layer without a feed-forward has no second sublayer; a file that carries its weights all the same is not refused
            need = q in self._sublayers()
            specs.update({f"hc{q}.in": TensorSpec((S,), required=need, role="stream_in"), f"hc{q}.out": TensorSpec((S,), required=need, role="stream_in"),
                          f"hc{q}.mix": TensorSpec((S, S), required=need, role="head_mix")})
        if self.norms["ff_in"] is None and self.spare_norm is not None:
            specs.update(self.spare_norm.tensor_specs())
        return specs

    def bind(self, tensors):
        for part in self._children():
            part.bind({name: tensors[name] for name in part.tensor_specs() if name in tensors})
        for q in self._sublayers():
            for k in ("in", "out", "mix"):
                self.weights[f"{q}.{k}"] = self._vector_f32(tensors[f"hc{q}.{k}"])

    def _last_write(self, residual, batch, y, q):
        """The layer's last write; where the block that runs next is one of this kind, the same pass leaves its first input (in one
        of two buffers that live as long as the step, taken in turn) under ``batch.shared["stream_input"]``."""
        from .. import kernels
        S, w = self.streams, self.weights
        nxt = batch.shared.get("following_block")
        if not isinstance(nxt, HyperConnectionBlock) or nxt.streams != S or nxt.rt.dtype != self.rt.dtype:
            kernels.streams_mix(residual, S, y=y, mix=w[f"{q}.mix"], out_w=w[f"{q}.out"])
            return
        bufs = batch.shared.setdefault("stream_input_buffers", [None, None])
        turn = batch.shared["stream_input_turn"] = 1 - batch.shared.get("stream_input_turn", 1)
        if bufs[turn] is None:
            bufs[turn] = kernels.new_tensor((y.shape[0], y.shape[1]), self.rt.dtype, y.device, whole_step=True)
        n1 = nxt.norms["mixer_in"]
        x = kernels.streams_mix(residual, S, y=y, mix=w[f"{q}.mix"], out_w=w[f"{q}.out"], in_next=nxt.weights["1.in"], w_next=n1.weight,
                                eps=n1.eps, out_dtype=self.rt.dtype, out=bufs[turn])
        batch.shared["stream_input"] = (nxt, x)

    def forward(self, residual, batch, cache):
        from .. import kernels
        S, w, n1, n2 = self.streams, self.weights, self.norms["mixer_in"], self.norms["ff_in"]
        left = batch.shared.pop("stream_input", None)          # (the block it is meant for, its first input) from the layer before
        if left is not None and left[0] is self:
            x = left[1]
        else:
            x = kernels.streams_mix(residual, S, in_next=w["1.in"], w_next=n1.weight, eps=n1.eps, out_dtype=self.rt.dtype)
        y = self.mixer.forward(x, batch, cache, None)
        if n2 is None:
            self._last_write(residual, batch, y, 1)
            return
        x = kernels.streams_mix(residual, S, y=y, mix=w["1.mix"], out_w=w["1.out"], in_next=w["2.in"], w_next=n2.weight, eps=n2.eps,
                                out_dtype=self.rt.dtype)
        y = self.feed_forward.forward(x, None)
        self._last_write(residual, batch, y, 2)


def build_block(layer_spec, rt):
    from .base import _REGISTRY
    from ..config.base import ConfigError
    try:
        cls = _REGISTRY["block"][layer_spec.block]
    except KeyError:
        raise ConfigError(f"no block arrangement named {layer_spec.block!r}") from None
    return cls(rt, layer_spec)


register_part("block", "pre_norm", PreNormBlock, replace=True)
register_part("block", "parallel", ParallelBlock, replace=True)
register_part("block", "sandwich", SandwichBlock, replace=True)
register_part("block", "hyper_connections", HyperConnectionBlock, replace=True)
