"""Small Tuzavik configurations for the tests, and model folders with random weights made from them.

The three differ in every size, in the order and number of the layers and in every constant; among them they have what a
single model can hide: retention heads with more key than value channels and the reverse, a rotation over a part of a head,
over all of it and none, channel counts that are no multiple of four, a decay of one and a fast one; latent attention whose
unrotated, rotated and value channel counts all differ, with and without stretched frequencies, a latent narrower and wider
than a head, a layer that reads another layer's rows across layers of other kinds and two layers that read the same rows; one
expert of many, all experts, experts wider than the model; a layer without a feed-forward; a model without the two-token
table; multipliers on the stream and on the logits above and below one.
"""
import copy

from forge_b200.config import config_from_dict
from forge_b200.weights import write_random_model


def _ret(heads, dim, vdim, decay, rot, base):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}
    if rot is not None:
        m["rot"] = {"dims": rot, "base": base}
    return {"type": "retention", "mixer": m}


def _lat(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, base, scaling=None, kv_from=None):
    rot = {"dims": rot_dim, "base": base}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale, "rot": rot}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m}


def _dense(layer, ff):
    return dict(layer, mlp=None if ff is None else {"kind": "dense", "ff": ff})


def _moe(layer, ff, experts, top):
    return dict(layer, mlp={"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}})


TUZ = {
    "X": {"architecture": "Tuzavik", "vocab": 211, "width": 80, "norm": {"eps": 1e-4}, "residual_mult": 0.6, "logit_scale": 1.7,
          "embedding": {"bigram": {"buckets": 37, "mul_prev": 5, "mul_cur": 11}},
          "layers": [_moe(_ret(3, 10, 6, [0.9, 1.0, 0.5], 4, 300.0), 24, 5, 1),
                     _dense(_lat(3, 8, 4, 12, 20, 28, 0.4, 50.0, scaling=(4.0, 64, 8.0, 2.0)), 96),
                     _dense(_ret(2, 6, 14, [0.97, 0.8], 6, 5000.0), None),
                     _moe(_lat(2, 12, 4, 8, 20, 16, 0.3, 50.0, scaling=(4.0, 64, 8.0, 2.0), kv_from=1), 100, 3, 3),
                     _dense(_lat(5, 4, 4, 6, 20, 12, 0.7, 50.0, scaling=(4.0, 64, 8.0, 2.0), kv_from=1), 72)]},
    "Y": {"architecture": "Tuzavik", "vocab": 130, "width": 48, "norm": {"eps": 1e-2}, "residual_mult": 1.2, "logit_scale": 0.8,
          "layers": [_dense(_lat(2, 16, 8, 8, 40, 10, 0.25, 10000.0), 40),
                     _moe(_ret(1, 40, 24, [0.99], None, None), 16, 4, 2),
                     _dense(_lat(4, 6, 10, 20, 12, 36, 0.35, 77.0, scaling=(16.0, 40, 4.0, 1.0)), None)]},
    # widths at which the bfloat16 path takes the tensor-core products and the tensor-core attention
    "Z": {"architecture": "Tuzavik", "vocab": 520, "width": 192, "norm": {"eps": 1e-6}, "residual_mult": 0.45, "logit_scale": 0.25,
          "embedding": {"bigram": {"buckets": 1021, "mul_prev": 1000003, "mul_cur": 3}},
          "layers": [_dense(_lat(4, 32, 16, 48, 96, 64, 0.15, 250000.0, scaling=(8.0, 128, 16.0, 2.0)), 256),
                     _moe(_ret(3, 32, 64, [0.95, 0.999, 0.9925], 16, 1e5), 128, 6, 2),
                     _moe(_lat(8, 16, 16, 24, 96, 32, 0.2, 250000.0, scaling=(8.0, 128, 16.0, 2.0), kv_from=0), 64, 4, 2),
                     _dense(_ret(2, 128, 32, [0.98, 0.875], 128, 10000.0), 384)]},
}
SEEDS = {"X": 31, "Y": 32, "Z": 33}
STDS = {"X": dict(std=0.14, embed_std=0.6, norm_std=0.2), "Y": dict(std=0.16, embed_std=0.8, norm_std=0.2),
        "Z": dict(std=0.08, embed_std=0.6, norm_std=0.2)}
LENGTHS = {"X": [70, 129, 33, 150, 64, 97], "Y": [90, 47, 16, 140, 81], "Z": [160, 20, 131, 45]}


def tuz_config(name):
    return config_from_dict(copy.deepcopy(TUZ[name]))


def make_tuz_dir(tmp_path_factory, name):
    d = str(tmp_path_factory.mktemp(f"tuz{name}"))
    write_random_model(tuz_config(name), d, seed=SEEDS[name], **STDS[name])
    return d
