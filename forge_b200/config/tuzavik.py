"""Typed configuration of the Tuzavik decoder: layers listed in config.json, each a mixer and an optional feed-forward whose
OUTPUTS pass through RMS norms of their own before they join the stream, times ``residual_mult``; all norm weights are stored
as their distance from one; an embedding that adds a row chosen by the token and the one before it; logits times ``logit_scale``.

  "retention"         linear attention with one fixed decay per head (no softmax, no denominator), rotary positions on q and k
                      (channel i paired with i + dims/2), a gate
  "latent_attention"  softmax attention whose keys and values are made per head from one cached latent per token, beside one
                      rotated key part that all heads share (channel 2i paired with 2i+1, optionally with stretched
                      frequencies); a layer may read the rows that another layer cached (``kv_from``)
  mlp "dense"         gated feed-forward, silu
  mlp "moe"           routed experts: sigmoid scores, the ``top`` largest, not renormalised

config.json keys: ``architecture`` "Tuzavik", ``vocab``, ``width``, ``norm.eps``, ``residual_mult``, ``logit_scale``,
``embedding.bigram`` {``buckets``, ``mul_prev``, ``mul_cur``} (optional), ``layers`` (per layer ``type``, ``mixer`` {sizes and
constants}, ``mlp`` {``kind``, ...} or null), optionally ``max_positions``.  Tensor names: ``embed``, ``bigram``, ``final.norm``,
``head``, per layer ``l<i>.norm1``, ``norm1b``, ``norm2``, ``norm2b``, ``l<i>.mix.*``, ``l<i>.mlp.*``.
"""
import copy
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .base import ConfigError, LayerSpec, ModelPlan, PartSpec, optional, require

MIXERS = ("retention", "latent_attention")
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
class TuzavikConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float = 1.0
    logit_scale: float = 1.0
    embedding: Optional[Dict[str, Any]] = None
    layers: List[Dict[str, Any]] = field(default_factory=list)
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
        return len(self.layers)

    @classmethod
    def from_dict(cls, d, architecture="Tuzavik"):
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        emb = d.get("embedding")
        if emb is not None and not isinstance(emb, dict):
            raise ConfigError("config.json: 'embedding' must be an object")
        cfg = cls(architecture=architecture, vocab=require(d, "vocab", int), width=require(d, "width", int),
                  norm_eps=require(_section(d, "norm", ""), "eps", float), residual_mult=optional(d, "residual_mult", float, 1.0),
                  logit_scale=optional(d, "logit_scale", float, 1.0), embedding=copy.deepcopy(emb), layers=copy.deepcopy(layers),
                  max_positions=optional(d, "max_positions", int, DEFAULT_MAX_POSITIONS), eos_token_id=optional(d, "eos_token_id", int, None))
        cfg.validate()
        return cfg

    def _bigram(self):
        return (self.embedding or {}).get("bigram")

    def validate(self):
        if self.vocab <= 0 or self.width <= 0 or self.max_positions <= 0 or not self.norm_eps > 0.0:
            raise ConfigError("config.json: vocab, width, max_positions and norm.eps must be positive")
        bg = self._bigram()
        if bg is not None:
            if not isinstance(bg, dict):
                raise ConfigError("config.json: 'embedding.bigram' must be an object")
            _positive(bg, ("buckets",), "embedding.bigram: ")
            require(bg, "mul_prev", int)
            require(bg, "mul_cur", int)
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]: "
            if not isinstance(layer, dict) or layer.get("type") not in MIXERS:
                raise ConfigError(f"config.json: {where}'type' must be one of {MIXERS}")
            m = _section(layer, "mixer", where)
            _positive(m, ("heads", "dim"), where)
            if optional(m, "vdim", int, m["dim"]) <= 0:
                raise ConfigError(f"config.json: {where}'vdim' must be positive")
            rot = m.get("rot")
            if layer["type"] == "retention":
                decay = m.get("decay")
                if not isinstance(decay, list) or len(decay) != m["heads"] or any(isinstance(g, bool) or not isinstance(g, (int, float)) for g in decay):
                    raise ConfigError(f"config.json: {where}'decay' must list one number per head")
                if rot is not None:
                    rot = _section(m, "rot", where)
                    dims = optional(rot, "dims", int, m["dim"])
                    if dims % 2 or not 0 <= dims <= m["dim"] or not require(rot, "base", float) > 0.0:
                        raise ConfigError(f"config.json: {where}rot.dims must be even and at most dim, rot.base positive")
            else:
                _positive(m, ("kv_rank", "q_rank", "rot_dim", "vdim"), where)
                require(m, "scale", float)
                rot = _section(m, "rot", where)
                if m["rot_dim"] % 2 or optional(rot, "dims", int, m["rot_dim"]) != m["rot_dim"] or not require(rot, "base", float) > 0.0:
                    raise ConfigError(f"config.json: {where}rot_dim must be even, rot.dims equal to it, rot.base positive")
                if rot.get("scaling") is not None:
                    sc = _section(rot, "scaling", where + "rot: ")
                    for k in ("factor", "original", "fast", "slow"):
                        if not require(sc, k, float) > 0.0:
                            raise ConfigError(f"config.json: {where}rot.scaling.{k} must be positive")
                src = m.get("kv_from")
                if src is not None:
                    if isinstance(src, bool) or not isinstance(src, int) or not 0 <= src < i or self.layers[src].get("type") != "latent_attention" \
                            or self.layers[src]["mixer"].get("kv_from") is not None:
                        raise ConfigError(f"config.json: {where}kv_from must name an earlier latent_attention layer that caches rows of its own")
                    other = self.layers[src]["mixer"]
                    if (other.get("kv_rank"), other.get("rot_dim"), other.get("rot")) != (m["kv_rank"], m["rot_dim"], m["rot"]):
                        raise ConfigError(f"config.json: {where}kv_rank, rot_dim and rot must equal those of layer {src}, whose rows it reads")
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
                    raise ConfigError(f"config.json: {where}mlp.kind must be 'dense' or 'moe' (or mlp null)")
                if mlp["kind"] == "dense":
                    _positive(mlp, ("ff",), where + "mlp: ")
                else:
                    _positive(_section(mlp, "expert", where + "mlp: "), ("ff",), where + "mlp.expert: ")
                    r = _section(mlp, "router", where + "mlp: ")
                    _positive(r, ("experts", "top"), where + "mlp.router: ")
                    if r["top"] > r["experts"]:
                        raise ConfigError(f"config.json: {where}mlp.router.top exceeds the number of experts")

    def to_dict(self):
        d = {"architecture": self.architecture, "layers": copy.deepcopy(self.layers), "logit_scale": self.logit_scale,
             "norm": {"eps": self.norm_eps}, "residual_mult": self.residual_mult, "vocab": self.vocab, "width": self.width}
        if self.embedding is not None:
            d["embedding"] = copy.deepcopy(self.embedding)
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_positions
        if self.eos_token_id is not None:
            d["eos_token_id"] = self.eos_token_id
        return d

    def _mixer(self, layer):
        m, W, eps = layer["mixer"], self.width, self.norm_eps
        if layer["type"] == "retention":
            rot = m.get("rot") or {"dims": 0, "base": 10000.0}
            return PartSpec("retention", {
                "hidden_size": W, "num_heads": m["heads"], "head_dim": m["dim"], "v_head_dim": m.get("vdim", m["dim"]),
                "decay": [float(g) for g in m["decay"]], "eps": eps,
                "position": PartSpec("rope_halves", {"head_dim": m["dim"], "rotary_dims": rot.get("dims", m["dim"]), "theta": float(rot["base"])})})
        rot = m["rot"]
        return PartSpec("latent_attention", {
            "hidden_size": W, "num_heads": m["heads"], "head_dim": m["dim"], "rot_dim": m["rot_dim"], "v_head_dim": m["vdim"],
            "kv_rank": m["kv_rank"], "q_rank": m["q_rank"], "scale": float(m["scale"]), "eps": eps, "own_latent": m.get("kv_from") is None,
            "position": PartSpec("rope_pairs", {"head_dim": m["rot_dim"], "rotary_dims": m["rot_dim"], "theta": float(rot["base"]),
                                                "scaling": copy.deepcopy(rot.get("scaling"))})})

    def plan(self) -> ModelPlan:
        W = self.width

        def norm(name, **more):
            return PartSpec("rmsnorm", {"size": W, "eps": self.norm_eps, "offset": 1.0, "names": {"weight": name}, **more})
        layers = []
        for i, layer in enumerate(self.layers):
            mlp = layer.get("mlp")
            if mlp is None:
                ff = PartSpec("none", {})
            elif mlp["kind"] == "dense":
                ff = PartSpec("swiglu", {"hidden_size": W, "intermediate_size": mlp["ff"], "suffix": "",
                                         "names": {"gate": "mlp.gate", "up": "mlp.up", "down": "mlp.down"}})
            else:
                ff = PartSpec("routed_experts", {"hidden_size": W, "intermediate_size": mlp["expert"]["ff"], "experts": mlp["router"]["experts"],
                                                 "top": mlp["router"]["top"], "score": "sigmoid", "renormalize": False, "prefix": "mlp."})
            norms = {"mixer_in": norm("norm1"), "mixer_out": norm("norm1b"),
                     "ff_in": None if mlp is None else norm("norm2"), "ff_out": None if mlp is None else norm("norm2b")}
            layers.append(LayerSpec(block="sandwich", mixer=self._mixer(layer), feed_forward=ff, norms=norms, weight_prefix=f"l{i}.",
                                    cache_from=layer["mixer"].get("kv_from"), block_params={"residual_mult": self.residual_mult}))
        bg = self._bigram()
        if bg is None:
            emb = PartSpec("embedding", {"vocab_size": self.vocab, "hidden_size": W, "names": {"weight": "embed"}})
        else:
            emb = PartSpec("pair_embedding", {"vocab_size": self.vocab, "hidden_size": W, "buckets": bg["buckets"],
                                              "mul_prev": bg["mul_prev"], "mul_cur": bg["mul_cur"]})
        return ModelPlan(
            hidden_size=W, vocab_size=self.vocab, max_positions=self.max_positions, embedding=emb,
            # the head is linear: the factor on the logits rides on the final norm's weight
            final_norm=norm("final.norm", scale=self.logit_scale),
            lm_head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": W, "tied": False, "names": {"weight": "head"}}),
            layers=layers, schedule=list(range(len(layers))), embedding_prefix="", final_norm_prefix="", lm_head_prefix="")
