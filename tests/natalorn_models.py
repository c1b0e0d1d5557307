"""Small Natalorn configurations for the tests, and model folders with random weights made from them.

The first three differ in every size, in the order and number of the layers, in the repeated span and in every constant; among them
they have what a single model can hide: one copy of the stream, two and four; no repeated span, one in the middle and one over
all layers; attention with as many key/value heads as query heads, with one, and with a number between; value heads narrower
and wider than key heads; windows shorter than a page, of one position, and longer than any sequence; chunks shorter than a
page, of a page and a half, and longer than any sequence; a cap on the scores that bites and one that does not; a latent
narrower and wider than a head, rotated parts of other widths than the unrotated ones; a layer without a feed-forward; experts
in one group, in groups that are all kept, and in groups of which some are dropped; one expert a token and all experts of the
kept groups; a router factor above and below one; a layer without a shared expert; and (N) the same decoder on one ordinary
residual stream, without the weights of the copies.
"""
import copy

from forge_b200.config import config_from_dict
from forge_b200.weights import write_random_model


def _att(heads, kv, dim, vdim, size, scale):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "mask": {"size": size}, "scale": scale}}


def _att2(heads, kv, dim, vdim, size, scale, softcap):
    return {"type": "attention_2", "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "mask": {"size": size}, "scale": scale,
                                             "softcap": softcap}}


def _lat(heads, dim, rot_dim, vdim, kv_rank, q_rank, size, scale, base):
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
                                                  "q_rank": q_rank, "mask": {"size": size}, "scale": scale, "rot": {"dims": rot_dim, "base": base}}}


def _moe(layer, ff, experts, top, scale, groups=None, shared=None):
    router = {"experts": experts, "top": top, "scale": scale}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    mlp = {"kind": "moe", "expert": {"ff": ff}, "router": router}
    if shared is not None:
        mlp["shared"] = {"ff": shared}
    return dict(layer, mlp=mlp)


def _bare(layer):
    return dict(layer, mlp=None)


NAT = {
    "K": {"architecture": "Natalorn", "vocab": 211, "width": 80, "norm": {"eps": 1e-4}, "streams": 2,
          "loop": {"start": 1, "stop": 3, "times": 3},
          "layers": [_moe(_att(6, 2, 8, 12, 5, 0.4), 24, 6, 2, 1.7, groups=(3, 2), shared=40),
                     _moe(_lat(3, 8, 4, 12, 20, 28, 9, 0.4, 50.0), 16, 4, 1, 0.6, groups=(1, 1), shared=8),
                     _bare(_att2(4, 4, 6, 6, 7, 0.6, 1.5)),
                     _moe(_att2(3, 1, 10, 4, 1000, 0.3, 30.0), 20, 8, 4, 1.0, groups=(4, 2))]},
    "L": {"architecture": "Natalorn", "vocab": 130, "width": 48, "norm": {"eps": 1e-2}, "streams": 1,
          "layers": [_moe(_lat(2, 16, 8, 8, 40, 10, 1000, 0.25, 10000.0), 40, 3, 3, 0.8, shared=16),
                     _bare(_att(4, 1, 12, 20, 1, 0.3)),
                     _moe(_att2(2, 2, 14, 10, 96, 0.35, 3.0), 12, 9, 3, 2.0, groups=(3, 1), shared=24),
                     _moe(_att(5, 5, 4, 6, 1000, 0.7), 8, 5, 1, 1.0, groups=(5, 5), shared=8)]},
    # widths at which the bfloat16 path takes the tensor-core products and the tensor-core attention kernels
    "M": {"architecture": "Natalorn", "vocab": 520, "width": 256, "norm": {"eps": 1e-6}, "streams": 4,
          "loop": {"start": 0, "stop": 3, "times": 2},
          "layers": [_moe(_lat(4, 32, 16, 48, 96, 64, 70, 0.15, 250000.0), 128, 8, 2, 1.5, groups=(4, 2), shared=64),
                     _moe(_att(8, 2, 32, 24, 100, 0.2), 64, 4, 2, 0.9, groups=(2, 2), shared=128),
                     _moe(_att2(4, 4, 64, 64, 72, 0.12, 4.0), 128, 6, 3, 1.2, groups=(2, 1), shared=64)]},
    # no 'streams': x <- x + sublayer(norm(x))
    "N": {"architecture": "Natalorn", "vocab": 97, "width": 64, "norm": {"eps": 1e-5}, "loop": {"start": 0, "stop": 1, "times": 2},
          "layers": [_moe(_att2(4, 2, 16, 8, 24, 0.3, 5.0), 32, 4, 2, 1.3, groups=(2, 1), shared=32),
                     _bare(_lat(2, 16, 16, 16, 32, 24, 20, 0.2, 1000.0)),
                     _moe(_att(2, 2, 8, 8, 17, 0.5), 16, 2, 1, 0.7)]},
}
SEEDS = {"K": 41, "L": 42, "M": 43, "N": 44}
STDS = {"K": dict(std=0.14, embed_std=0.6, norm_std=0.2, bias_std=0.4), "L": dict(std=0.16, embed_std=0.8, norm_std=0.2, bias_std=0.4),
        "M": dict(std=0.07, embed_std=0.6, norm_std=0.2, bias_std=0.4), "N": dict(std=0.15, embed_std=0.7, norm_std=0.2, bias_std=0.4)}
LENGTHS = {"K": [70, 129, 33, 150, 64, 97], "L": [90, 47, 16, 140, 81], "M": [160, 20, 131, 45], "N": [60, 33, 90, 41]}


def nat_config(name):
    return config_from_dict(copy.deepcopy(NAT[name]))


def make_nat_dir(tmp_path_factory, name):
    d = str(tmp_path_factory.mktemp(f"nat{name}"))
    write_random_model(nat_config(name), d, seed=SEEDS[name], **STDS[name])
    return d
