"""Typed configuration of the Natalorn decoder: pre-norm layers (RMS norms) listed in config.json on a residual stream that is
kept as ``streams`` copies (hyper-connections: every sublayer reads a weighted sum of the copies and its output rewrites all of
them through a small mixing matrix), each layer with one of three mixers and a routed feed-forward or none; a span of the layers
may run several times in a row with the same weights, every pass with a cache of its own; untied output head.  A config.json without
``streams`` describes the same decoder on one ordinary residual stream (x <- x + sublayer(norm(x)), no ``hc`` tensors).

  "attention"         grouped-query softmax attention without rotation over a sliding window (``mask.size`` positions)
  "attention_2"       the same with q/k/v biases, scores capped by ``softcap`` tanh(score / ``softcap``), and chunks instead of a
                      window: a position sees the earlier positions of its own chunk of ``mask.size`` positions
  "latent_attention"  softmax attention whose keys and values are made per head from one cached latent per token beside one
                      rotated key part that all heads share (channel 2i paired with 2i+1), over a sliding window, with a sink
                      per head in the softmax denominator and a sigmoid gate on the concatenated heads
  mlp "moe"           routed experts: softmax scores; ranking by score + correction inside the best-ranked blocks of experts;
                      weights = the picked scores times ``router.scale`` (their sum is left as it is); a shared expert beside them

config.json keys: ``architecture`` "Natalorn", ``vocab``, ``width``, ``norm.eps``, ``streams``, ``layers`` (per layer ``type``,
``mixer`` {sizes and constants}, ``mlp`` {``kind`` "moe", ``expert.ff``, ``router`` {``experts``, ``top``, ``scale``, ``groups``
{``count``, ``keep``}}, ``shared.ff``} or null), optionally ``loop`` {``start``, ``stop``, ``times``} and ``max_positions``.
Tensor names: ``embed``, ``final.norm``, ``head``, per layer ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.hc1.{in,out,mix}``,
``l<i>.hc2.{in,out,mix}``, ``l<i>.mix.*``, ``l<i>.mlp.{e<n>.{gate,up,down}, router, correction, shared.{gate,up,down}}``.
"""
import copy
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .base import ConfigError, LayerSpec, ModelPlan, PartSpec, optional, require

MIXERS = ("attention", "attention_2", "latent_attention")
DEFAULT_MAX_POSITIONS = 1 << 17


def _section(d, key, where):
    v = d.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"config.json: {where}'{key}' must be an object")
    return v


def _positive(m, keys, where):
    for k in keys:
        if require(m, k, int) <= 0:
            raise ConfigError(f"config.json: {where}'{k}' must be positive")


@dataclass(frozen=True)
class NatalornConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    streams: Optional[int] = None          # None: one ordinary residual stream, no hyper-connection weights
    layers: List[Dict[str, Any]] = field(default_factory=list)
    loop: Optional[Dict[str, int]] = None
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_id: Optional[int] = None

    # what the command line and the benchmark ask any configuration
    @property
    def vocab_size(self):
        return self.vocab

    @property
    def hidden_size(self):
        return self.width

    @property
    def num_hidden_layers(self):
        return len(self.schedule())

    @classmethod
    def from_dict(cls, d, architecture="Natalorn"):
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        loop = d.get("loop")
        if loop is not None:
            loop = {k: require(_section(d, "loop", ""), k, int) for k in ("start", "stop", "times")}
        cfg = cls(architecture=architecture, vocab=require(d, "vocab", int), width=require(d, "width", int),
                  norm_eps=require(_section(d, "norm", ""), "eps", float), streams=optional(d, "streams", int, None),
                  layers=copy.deepcopy(layers), loop=loop, max_positions=optional(d, "max_positions", int, DEFAULT_MAX_POSITIONS),
                  eos_token_id=optional(d, "eos_token_id", int, None))
        cfg.validate()
        return cfg

    def validate(self):
        if self.vocab <= 0 or self.width <= 0 or self.max_positions <= 0 or not self.norm_eps > 0.0:
            raise ConfigError("config.json: vocab, width, max_positions and norm.eps must be positive")
        if self.streams is not None and not 1 <= self.streams <= 16:
            raise ConfigError("config.json: 'streams' must lie between 1 and 16")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]: "
            if not isinstance(layer, dict) or layer.get("type") not in MIXERS:
                raise ConfigError(f"config.json: {where}'type' must be one of {MIXERS}")
            m = _section(layer, "mixer", where)
            _positive(m, ("heads", "dim"), where)
            if optional(m, "vdim", int, m["dim"]) <= 0:
                raise ConfigError(f"config.json: {where}'vdim' must be positive")
            require(m, "scale", float)
            _positive(_section(m, "mask", where), ("size",), where + "mask: ")
            if layer["type"] == "latent_attention":
                _positive(m, ("kv_rank", "q_rank", "rot_dim", "vdim"), where)
                rot = _section(m, "rot", where)
                if m["rot_dim"] % 2 or optional(rot, "dims", int, m["rot_dim"]) != m["rot_dim"] or not require(rot, "base", float) > 0.0:
                    raise ConfigError(f"config.json: {where}rot_dim must be even, rot.dims equal to it, rot.base positive")
            else:
                g = optional(m, "kv_heads", int, m["heads"])
                if g <= 0 or m["heads"] % g:
                    raise ConfigError(f"config.json: {where}{m['heads']} heads cannot share {g} kv_heads")
                if layer["type"] == "attention_2" and m.get("softcap") is not None and not require(m, "softcap", float) > 0.0:
                    raise ConfigError(f"config.json: {where}softcap must be positive")
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") != "moe":
                    raise ConfigError(f"config.json: {where}mlp.kind must be 'moe' (or mlp null)")
                _positive(_section(mlp, "expert", where + "mlp: "), ("ff",), where + "mlp.expert: ")
                r = _section(mlp, "router", where + "mlp: ")
                _positive(r, ("experts", "top"), where + "mlp.router: ")
                optional(r, "scale", float, 1.0)
                if r["top"] > r["experts"]:
                    raise ConfigError(f"config.json: {where}mlp.router.top exceeds the number of experts")
                if r.get("groups") is not None:
                    g = _section(r, "groups", where + "mlp.router: ")
                    _positive(g, ("count", "keep"), where + "mlp.router.groups: ")
                    if r["experts"] % g["count"] or g["keep"] > g["count"] or r["top"] > g["keep"] * (r["experts"] // g["count"]):
                        raise ConfigError(f"config.json: {where}mlp.router.groups: {r['experts']} experts do not form {g['count']} equal groups "
                                          f"of which {g['keep']} hold {r['top']} experts")
                if mlp.get("shared") is not None:
                    _positive(_section(mlp, "shared", where + "mlp: "), ("ff",), where + "mlp.shared: ")
        if self.loop is not None:
            a, b, times = self.loop["start"], self.loop["stop"], self.loop["times"]
            if not 0 <= a < b <= len(self.layers) or times < 1:
                raise ConfigError("config.json: loop needs 0 <= start < stop <= number of layers and times >= 1")

    def to_dict(self):
        d = {"architecture": self.architecture, "layers": copy.deepcopy(self.layers), "norm": {"eps": self.norm_eps},
             "vocab": self.vocab, "width": self.width}
        if self.streams is not None:
            d["streams"] = self.streams
        if self.loop is not None:
            d["loop"] = dict(self.loop)
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_positions
        if self.eos_token_id is not None:
            d["eos_token_id"] = self.eos_token_id
        return d

    def schedule(self):
        """The order in which the layers run: the looped span ``times`` times in a row, then the rest."""
        n = len(self.layers)
        if self.loop is None:
            return list(range(n))
        a, b, times = self.loop["start"], self.loop["stop"], self.loop["times"]
        return list(range(a)) + list(range(a, b)) * times + list(range(b, n))

    def _mixer(self, layer):
        m, W, eps = layer["mixer"], self.width, self.norm_eps
        size = m["mask"]["size"]
        if layer["type"] == "latent_attention":
            return PartSpec("latent_attention", {
                "hidden_size": W, "num_heads": m["heads"], "head_dim": m["dim"], "rot_dim": m["rot_dim"], "v_head_dim": m["vdim"],
                "kv_rank": m["kv_rank"], "q_rank": m["q_rank"], "scale": float(m["scale"]), "eps": eps, "window": size, "sink": True,
                "out_gate": True,
                "position": PartSpec("rope_pairs", {"head_dim": m["rot_dim"], "rotary_dims": m["rot_dim"], "theta": float(m["rot"]["base"])})})
        params = {"hidden_size": W, "num_heads": m["heads"], "num_kv_heads": m.get("kv_heads", m["heads"]), "head_dim": m["dim"],
                  "v_head_dim": m.get("vdim", m["dim"]), "scale": float(m["scale"])}
        if layer["type"] == "attention":
            params.update(window=size)
        else:
            params.update(chunk=size, softcap=m.get("softcap"), qkv_bias=True)
        return PartSpec("masked_attention", params)

    def _feed_forward(self, mlp):
        if mlp is None:
            return PartSpec("none", {})
        W, r = self.width, mlp["router"]
        groups = r.get("groups") or {}
        shared = None
        if mlp.get("shared") is not None:
            shared = PartSpec("swiglu", {"hidden_size": W, "intermediate_size": mlp["shared"]["ff"], "suffix": "",
                                         "names": {"gate": "mlp.shared.gate", "up": "mlp.shared.up", "down": "mlp.shared.down"}})
        return PartSpec("routed_experts", {
            "hidden_size": W, "intermediate_size": mlp["expert"]["ff"], "experts": r["experts"], "top": r["top"], "score": "softmax",
            "renormalize": False, "prefix": "mlp.", "correction": True, "groups": groups.get("count", 0), "keep": groups.get("keep", 0),
            "route_scale": float(r.get("scale", 1.0)), "shared": shared})

    def plan(self) -> ModelPlan:
        W = self.width

        def norm(name, required=True):
            return PartSpec("rmsnorm", {"size": W, "eps": self.norm_eps, "names": {"weight": name}, "required": required})
        layers = []
        for i, layer in enumerate(self.layers):
            mlp = layer.get("mlp")
            if self.streams is None:
                layers.append(LayerSpec(block="pre_norm", mixer=self._mixer(layer), feed_forward=self._feed_forward(mlp),
                                        norms={"input": norm("norm1"), "post_mixer": None if mlp is None else norm("norm2")},
                                        weight_prefix=f"l{i}.", norm_prefixes={"input": "", "post_mixer": ""}))
                continue
            layers.append(LayerSpec(block="hyper_connections", mixer=self._mixer(layer), feed_forward=self._feed_forward(mlp),
                                    norms={"mixer_in": norm("norm1"), "ff_in": None if mlp is None else norm("norm2"),
                                           "ff_in_unused": norm("norm2", required=False) if mlp is None else None},
                                    weight_prefix=f"l{i}.", block_params={"streams": self.streams}))
        return ModelPlan(
            hidden_size=W, vocab_size=self.vocab, max_positions=self.max_positions,
            embedding=PartSpec("embedding", {"vocab_size": self.vocab, "hidden_size": W, "names": {"weight": "embed"}}),
            final_norm=norm("final.norm"),
            lm_head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": W, "tied": False, "names": {"weight": "head"}}),
            layers=layers, schedule=self.schedule(), embedding_prefix="", final_norm_prefix="", lm_head_prefix="", streams=self.streams or 1)
