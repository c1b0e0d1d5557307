from .base import ConfigError, LayerSpec, ModelPlan, PartSpec
from .llama import LlamaConfig
from .zatupel import ZatupelConfig
from .tidenex import TidenexConfig
from .tuzavik import TuzavikConfig
from .natalorn import NatalornConfig
from .registry import (config_from_dict, load_config, register_architecture, registered_architectures,
                       unregister_architecture)

# LLaMA-architecture checkpoints; Qwen2 files are the same decoder with q/k/v biases on by default
# (the reference routes both names to one engine, src/model/arch_registrations.cpp:46-71).
register_architecture("LlamaForCausalLM", LlamaConfig, replace=True)
register_architecture("Qwen2ForCausalLM", LlamaConfig, replace=True)

# a hybrid of windowed attention and two state-keeping mixers; its files name it with one string, "architecture"
register_architecture("Zatupel", ZatupelConfig, replace=True)

# pre-norm layers of differential attention, or of an attention beside a gated linear recurrence; a span of layers may repeat
register_architecture("Tidenex", TidenexConfig, replace=True)

# layers of retention or of attention over one cached latent per token, every sublayer's output normed before it joins the stream,
# dense or routed feed-forwards, an embedding that also looks at the token before
register_architecture("Tuzavik", TuzavikConfig, replace=True)

# pre-norm layers on a residual stream kept as several copies (hyper-connections): windowed and chunked attention without rotation,
# attention over one cached latent per token with a sink and a gate, routed experts chosen within groups beside a shared expert
register_architecture("Natalorn", NatalornConfig, replace=True)

__all__ = ["ZatupelConfig", "TidenexConfig", "TuzavikConfig", "NatalornConfig", "ConfigError", "LayerSpec", "ModelPlan", "PartSpec", "LlamaConfig", "config_from_dict", "load_config",
           "register_architecture", "registered_architectures", "unregister_architecture"]
