"""Random-weights mode: from a configuration and a seed to a model folder (config.json + model.safetensors)
that loads like any other.  Matrices and biases are N(0, std) (0.02 as in the reference's
tools/create_test_model.py:14-63, which however also draws the norm weights from it; here norm weights are
1, or 1 + N(0, norm_std) when asked).  Matrices are stored in bfloat16, norm weights in float32.
"""
import json
import os

import torch

from .safetensors_io import write_safetensors


def random_tensors(config, seed=0, std=0.02, embed_std=None, norm_std=0.0, bias_std=None, dtype=torch.bfloat16,
                   device="cpu"):
    """{file tensor name: tensor} for every tensor the configuration's model expects, in file order."""
    from ..engine.model import Model
    from ..parts import Runtime
    model = Model(config.plan(), Runtime(torch.device("cpu"), dtype))
    gen = torch.Generator(device=device)
    gen.manual_seed(int(seed))
    out = {}
    for name, spec in model.tensor_specs().items():
        if not spec.required:
            continue
        shape = tuple(spec.shape)
        if -1 in shape:
            if spec.default_shape is None:
                raise ValueError(f"{name}: a size is left to the file and no default is given for random weights")
            shape = tuple(spec.default_shape)
        spec = type(spec)(shape, spec.required, spec.integer, spec.role)
        if spec.integer:
            out[name] = torch.zeros(spec.shape, dtype=torch.int32, device=device)
        elif spec.role == "fraction":
            out[name] = torch.rand(spec.shape, generator=gen, dtype=torch.float32, device=device).to(dtype)
        elif spec.role == "head_mix":
            t = torch.eye(spec.shape[0], dtype=torch.float32, device=device)
            out[name] = (t + torch.randn(spec.shape, generator=gen, dtype=torch.float32, device=device) * 0.3).to(dtype)
        elif spec.role == "stream_in":        # what a copy of the stream adds to a sublayer's input, or takes of its output
            out[name] = (0.7 + 0.3 * torch.randn(spec.shape, generator=gen, dtype=torch.float32, device=device)).to(dtype)
        elif spec.role == "route_bias":       # what is added to a router's scores (of order 1 / experts) before the choice
            out[name] = (0.05 * torch.randn(spec.shape, generator=gen, dtype=torch.float32, device=device)).to(dtype)
        elif spec.role == "lambda_part":      # vectors whose pairwise dot products are exponentiated: keep those of order 1/2
            n = max(1, int(torch.tensor(spec.shape).prod()))
            out[name] = (torch.randn(spec.shape, generator=gen, dtype=torch.float32, device=device) * (0.7 / n ** 0.25)).to(dtype)
        elif spec.role == "norm_offset":      # a norm weight stored as its distance from one
            t = torch.zeros(spec.shape, dtype=torch.float32, device=device)
            if norm_std:
                t += torch.randn(spec.shape, generator=gen, dtype=torch.float32, device=device) * norm_std
            out[name] = t
        elif spec.role == "norm":
            t = torch.ones(spec.shape, dtype=torch.float32, device=device)
            if norm_std:
                t += torch.randn(spec.shape, generator=gen, dtype=torch.float32, device=device) * norm_std
            out[name] = t
        else:
            s = std
            if spec.role == "bias" and bias_std is not None:
                s = bias_std
            if spec.role == "embedding" and embed_std is not None:
                s = embed_std
            out[name] = (torch.randn(spec.shape, generator=gen, dtype=torch.float32, device=device) * s).to(dtype)
    return out


def write_random_model(config, out_dir, seed=0, **kwargs):
    """Writes ``out_dir/config.json`` and ``out_dir/model.safetensors``; returns out_dir."""
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(config.to_dict(), f, indent=1)
    write_safetensors(os.path.join(out_dir, "model.safetensors"), random_tensors(config, seed=seed, **kwargs),
                      metadata={"format": "pt", "seed": seed})
    return out_dir
