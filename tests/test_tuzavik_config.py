"""Tuzavik on the CPU: configuration, plan, tensor names, refusals, cache needs, and the plain implementation against itself."""
import copy
import math

import pytest
import torch

from forge_b200.cache.storage import plan_groups
from forge_b200.config import ConfigError, config_from_dict
from forge_b200.engine.model import Model
from forge_b200.parts import KVCacheSpec, Runtime, StateSpec
from plain import tuzavik as PZ
from tuzavik_models import TUZ, tuz_config
from zatupel_models import rand


def _model(name):
    return Model(tuz_config(name).plan(), Runtime(torch.device("cpu"), torch.bfloat16))


def test_registered_by_its_architecture_name():
    from forge_b200.config.tuzavik import TuzavikConfig
    assert isinstance(tuz_config("X"), TuzavikConfig)
    p = tuz_config("X").plan()
    assert p.schedule == [0, 1, 2, 3, 4] and [l.block for l in p.layers] == ["sandwich"] * 5
    assert [l.mixer.kind for l in p.layers] == ["retention", "latent_attention", "retention", "latent_attention", "latent_attention"]
    assert [l.cache_from for l in p.layers] == [None, None, None, 1, 1]
    assert p.embedding.kind == "pair_embedding" and tuz_config("Y").plan().embedding.kind == "embedding"


def test_tensor_names_and_shapes():
    specs = _model("X").tensor_specs()
    for name, shape in {"embed": (211, 80), "bigram": (38, 80), "final.norm": (80,), "head": (211, 80), "l0.norm1": (80,), "l0.norm1b": (80,),
                        "l0.norm2": (80,), "l0.norm2b": (80,), "l0.mix.q": (30, 80), "l0.mix.k": (30, 80), "l0.mix.v": (18, 80),
                        "l0.mix.g": (18, 80), "l0.mix.o": (80, 18), "l0.mlp.router": (5, 80), "l0.mlp.e4.gate": (24, 80),
                        "l0.mlp.e0.down": (80, 24), "l1.mix.dq": (28, 80), "l1.mix.dq.norm": (28,), "l1.mix.uq": (36, 28),
                        "l1.mix.dkv": (24, 80), "l1.mix.dkv.norm": (20,), "l1.mix.uk": (24, 20), "l1.mix.uv": (36, 20), "l1.mix.o": (80, 36),
                        "l1.mlp.gate": (96, 80), "l1.mlp.down": (80, 96), "l3.mix.uk": (24, 20), "l3.mix.uv": (16, 20), "l3.mix.uq": (32, 16),
                        "l4.mix.o": (80, 30)}.items():
        assert tuple(specs[name].shape) == shape, name
    assert "l2.norm2" not in specs and "l2.mlp.up" not in specs and "l2.norm2b" not in specs      # a layer without a feed-forward
    assert "l3.mix.dkv" not in specs and "l3.mix.dkv.norm" not in specs and "l4.mix.dkv" not in specs   # they read layer 1's rows
    assert "l0.mlp.e5.gate" not in specs and "bigram" not in _model("Y").tensor_specs()


def test_cache_needs():
    m = _model("X")
    specs = m.cache_specs()
    assert specs[0] == StateSpec((3 * 10 * 6,), torch.float32) and specs[2] == StateSpec((2 * 6 * 14,), torch.float32)
    assert specs[1] == KVCacheSpec(1, 24, None, v_head_dim=0)            # one row of latent + rotated part a token, no values beside it
    groups, _ = plan_groups(specs, m.cache_from())
    assert len(groups) == 1                                               # the readers of layer 1's rows own no pages


@pytest.mark.parametrize("change, message", [
    (lambda d: d["layers"][1].update(type="conv"), "type"),
    (lambda d: d["layers"][0]["mixer"].update(decay=[0.5, 0.5]), "decay"),
    (lambda d: d["layers"][0]["mixer"]["rot"].update(dims=5), "rot.dims"),
    (lambda d: d["layers"][0]["mixer"]["rot"].update(dims=12), "rot.dims"),
    (lambda d: d["layers"][1]["mixer"].pop("scale"), "scale"),
    (lambda d: d["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda d: d["layers"][1]["mixer"]["rot"].update(dims=2), "rot"),
    (lambda d: d["layers"][1]["mixer"]["rot"]["scaling"].pop("fast"), "fast"),
    (lambda d: d["layers"][3]["mixer"].update(kv_from=3), "kv_from"),
    (lambda d: d["layers"][3]["mixer"].update(kv_from=0), "kv_from"),
    (lambda d: d["layers"][4]["mixer"].update(kv_from=3), "kv_from"),
    (lambda d: d["layers"][3]["mixer"].update(kv_rank=24), "kv_rank"),
    (lambda d: d["layers"][0]["mlp"]["router"].update(top=6), "top"),
    (lambda d: d["layers"][1]["mlp"].update(kind="conv"), "mlp.kind"),
    (lambda d: d["embedding"]["bigram"].update(buckets=0), "buckets"),
    (lambda d: d.pop("norm"), "norm"),
    (lambda d: d.update(layers=[]), "layers"),
])
def test_refusals(change, message):
    d = copy.deepcopy(TUZ["X"])
    change(d)
    with pytest.raises(ConfigError, match=message):
        config_from_dict(d)


def test_what_config_does_not_mention_does_not_exist():
    d = copy.deepcopy(TUZ["X"])
    d["layers"][0]["mixer"].pop("rot")
    d["layers"][0]["mixer"].pop("vdim")
    d.pop("residual_mult")
    d.pop("logit_scale")
    d.pop("embedding")
    p = config_from_dict(d).plan()
    assert p.layers[0].mixer.params["position"].params["rotary_dims"] == 0 and p.layers[0].mixer.params["v_head_dim"] == 10
    assert p.layers[0].block_params["residual_mult"] == 1.0 and p.final_norm.params["scale"] == 1.0 and p.embedding.kind == "embedding"
    assert tuz_config("Y").plan().layers[0].mixer.params["position"].params["scaling"] is None


def test_to_dict_round_trip():
    for name in TUZ:
        c = tuz_config(name)
        assert config_from_dict(c.to_dict()) == c


def test_the_engine_frequencies_are_the_plain_ones():
    """The position parts work their frequencies out on the host: both layouts, with and without the stretch."""
    from forge_b200.config import PartSpec
    from forge_b200.parts import build_part
    rt = Runtime(torch.device("cpu"), torch.float32)
    for sc in (None, {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 2.0}, {"factor": 16.0, "original": 40, "fast": 4.0, "slow": 1.0},
               {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0}):
        for dims, base in ((4, 50.0), (10, 77.0), (64, 1e6)):
            part = build_part("position", PartSpec("rope_pairs", {"head_dim": dims, "rotary_dims": dims, "theta": base, "scaling": sc}), rt)
            f, amp = PZ.stretched_frequencies(base, dims, sc) if sc else (PZ.plain_frequencies(base, dims), 1.0)
            assert torch.allclose(part.inv_freq.double(), f, rtol=1e-6, atol=0) and math.isclose(part.amplitude, amp, rel_tol=1e-6)
    part = build_part("position", PartSpec("rope_halves", {"head_dim": 10, "rotary_dims": 4, "theta": 300.0}), rt)
    assert torch.allclose(part.inv_freq.double(), PZ.plain_frequencies(300.0, 4), rtol=1e-6, atol=0)


# ------------------------------------------------------------------------------------- the plain implementation against itself

def test_plain_rotations():
    x = rand(5, 2, 12, seed=1).double()
    pos = torch.tensor([0, 1, 2, 50, 1000])
    f = PZ.plain_frequencies(100.0, 8)
    assert torch.allclose(f, torch.tensor([100.0 ** (-2.0 * i / 8) for i in range(4)]).double())
    y = PZ.rotate(x, pos, f, 8, "halves")
    z = PZ.rotate(x, pos, f, 8, "pairs", amplitude=1.5)
    assert torch.equal(y[..., 8:], x[..., 8:]) and torch.equal(y[0], x[0]) and torch.equal(z[..., 8:], x[..., 8:])
    for i in range(4):
        a = pos.double() * 100.0 ** (-2.0 * i / 8)
        c, s = torch.cos(a)[:, None], torch.sin(a)[:, None]
        u, v = x[:, :, i], x[:, :, i + 4]
        assert torch.allclose(y[:, :, i], u * c - v * s, atol=1e-12) and torch.allclose(y[:, :, i + 4], v * c + u * s, atol=1e-12)
        u, v = x[:, :, 2 * i], x[:, :, 2 * i + 1]
        assert torch.allclose(z[:, :, 2 * i], 1.5 * (u * c - v * s), atol=1e-12) and torch.allclose(z[:, :, 2 * i + 1], 1.5 * (v * c + u * s), atol=1e-12)


def test_plain_stretched_frequencies_in_closed_form():
    """base 16, 8 channels, 64 original positions: pair i turns 64 f_i / 2 pi times; fast 4 and slow 1 put the ramp between
    pair 1 (floor of 1.35) and pair 4 (ceil of 3.35, which the last pair, 3, does not reach): ramp 0, 0, 1/3, 2/3."""
    f, amp = PZ.stretched_frequencies(16.0, 8, {"factor": 4.0, "original": 64, "fast": 4.0, "slow": 1.0})
    plain = [16.0 ** (-2.0 * i / 8) for i in range(4)]
    want = [plain[0], plain[1], plain[2] / 4.0 / 3.0 + plain[2] * 2.0 / 3.0, plain[3] / 4.0 * 2.0 / 3.0 + plain[3] / 3.0]
    assert torch.allclose(f, torch.tensor(want).double(), rtol=1e-12) and math.isclose(amp, 0.1 * math.log(4.0) + 1.0)


def test_plain_two_token_rows():
    assert PZ.two_token_rows([3, 9, 9, 0], 7, 5, 11) == [7, (15 + 99) % 7, (45 + 99) % 7, 45 % 7]


def test_plain_mixers_do_not_look_ahead_and_retention_has_a_closed_form():
    W, T = 32, 40
    h = rand(T, W, seed=2).double()
    h2 = h.clone()
    h2[25:] = rand(T - 25, W, seed=3).double()
    m = {"heads": 2, "dim": 6, "vdim": 10, "decay": [0.9, 0.5], "rot": {"dims": 4, "base": 50.0}}
    w = {"q": rand(12, W, seed=4), "k": rand(12, W, seed=5), "v": rand(20, W, seed=6), "g": rand(20, W, seed=7), "o": rand(W, 20, seed=8)}
    w = {k: v.double() * 0.3 for k, v in w.items()}
    a = PZ.retention(h, w, m, 1e-5)
    assert torch.allclose(a[:25], PZ.retention(h2, w, m, 1e-5)[:25], atol=1e-10)
    # o_t = sum_j decay^(t-j) (q_t . k_j) v_j
    pos = torch.arange(T)
    f = PZ.plain_frequencies(50.0, 4)
    q = PZ.rotate((h @ w["q"].t()).view(T, 2, 6), pos, f, 4, "halves")
    k = PZ.rotate((h @ w["k"].t()).view(T, 2, 6), pos, f, 4, "halves") / math.sqrt(6.0)
    v = (h @ w["v"].t()).view(T, 2, 10)
    t = 31
    o = torch.stack([sum(m["decay"][n] ** (t - j) * (q[t, n] @ k[j, n]) * v[j, n] for j in range(t + 1)) for n in range(2)])
    want = (PZ.rms_unit(o, 1e-5).reshape(20) * PZ.silu(h[t] @ w["g"].t())) @ w["o"].t()
    assert torch.allclose(a[t], want, atol=1e-10)
    ml = {"heads": 3, "dim": 8, "rot_dim": 4, "vdim": 12, "kv_rank": 20, "q_rank": 28, "scale": 0.4,
          "rot": {"dims": 4, "base": 50.0, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 2.0}}}
    wl = {"dq": rand(28, W, seed=9), "dq.norm": 1 + rand(28, seed=10, scale=0.2), "uq": rand(36, 28, seed=11), "dkv": rand(24, W, seed=12),
          "dkv.norm": 1 + rand(20, seed=13, scale=0.2), "uk": rand(24, 20, seed=14), "uv": rand(36, 20, seed=15), "o": rand(W, 36, seed=16)}
    wl = {k: v.double() for k, v in wl.items()}
    b, kept = PZ.latent_attention(h, wl, ml, 1e-5)
    b2, kept2 = PZ.latent_attention(h2, wl, ml, 1e-5)
    assert torch.allclose(b[:25], b2[:25], atol=1e-10) and torch.allclose(kept[0][:25], kept2[0][:25]) and kept[1].shape == (T, 4)
    # rows handed over from another layer are used instead of the layer's own
    wl.pop("dkv"), wl.pop("dkv.norm")
    assert torch.allclose(PZ.latent_attention(h, wl, ml, 1e-5, shared=kept)[0], b, atol=1e-12)


def test_plain_routing_takes_the_largest_scores_as_they_are():
    W = 8
    x = rand(3, W, seed=20).double()
    w = {"router": torch.zeros(4, W).double()}
    w["router"][:, 0] = torch.tensor([0.1, 3.0, -2.0, 1.0]).double()
    for e in range(4):
        w.update({f"e{e}.gate": rand(5, W, seed=21 + e).double(), f"e{e}.up": rand(5, W, seed=31 + e).double(), f"e{e}.down": rand(W, 5, seed=41 + e).double()})
    x[:, 0] = torch.tensor([1.0, -1.0, 1.0]).double()
    out = PZ.routed_ff(x, w, {"router": {"experts": 4, "top": 2}})
    for t, (first, second) in enumerate([(1, 3), (2, 0), (1, 3)]):
        s = torch.sigmoid(w["router"] @ x[t])
        want = sum(s[e] * PZ.gated_ff(x[t:t + 1], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"])[0] for e in (first, second))
        assert torch.allclose(out[t], want, atol=1e-12)
