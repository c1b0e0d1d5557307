"""Natalorn on the CPU: configuration, plan, tensor names, refusals, cache needs (pages given back behind windows and chunks), and
the plain implementation against itself."""
import copy
import math

import pytest
import torch

from forge_b200.cache import CacheManager
from forge_b200.cache.manager import GroupSpec
from forge_b200.cache.storage import plan_groups
from forge_b200.config import ConfigError, config_from_dict
from forge_b200.engine.model import Model
from forge_b200.parts import KVCacheSpec, Runtime
from natalorn_models import NAT, nat_config
from plain import natalorn as PN
from zatupel_models import rand


def _model(name):
    return Model(nat_config(name).plan(), Runtime(torch.device("cpu"), torch.bfloat16))


def test_registered_by_its_architecture_name():
    from forge_b200.config.natalorn import NatalornConfig
    assert isinstance(nat_config("K"), NatalornConfig)
    p = nat_config("K").plan()
    assert p.schedule == [0, 1, 2, 1, 2, 1, 2, 3] and p.streams == 2 and [l.block for l in p.layers] == ["hyper_connections"] * 4
    assert [l.mixer.kind for l in p.layers] == ["masked_attention", "latent_attention", "masked_attention", "masked_attention"]
    assert nat_config("L").plan().schedule == [0, 1, 2, 3] and nat_config("M").plan().schedule == [0, 1, 2, 0, 1, 2]
    assert nat_config("K").num_hidden_layers == 8 and nat_config("K").schedule() == PN.layer_order(NAT["K"])


def test_tensor_names_and_shapes():
    specs = _model("K").tensor_specs()
    for name, shape in {"embed": (211, 80), "final.norm": (80,), "head": (211, 80), "l0.norm1": (80,), "l0.norm2": (80,), "l0.hc1.in": (2,),
                        "l0.hc1.out": (2,), "l0.hc1.mix": (2, 2), "l0.hc2.mix": (2, 2), "l0.mix.q": (48, 80), "l0.mix.k": (16, 80),
                        "l0.mix.v": (24, 80), "l0.mix.o": (80, 72), "l0.mlp.router": (6, 80), "l0.mlp.correction": (6,),
                        "l0.mlp.e5.gate": (24, 80), "l0.mlp.e0.down": (80, 24), "l0.mlp.shared.gate": (40, 80), "l0.mlp.shared.down": (80, 40),
                        "l1.mix.dq": (28, 80), "l1.mix.dq.norm": (28,), "l1.mix.uq": (36, 28), "l1.mix.dkv": (24, 80), "l1.mix.dkv.norm": (20,),
                        "l1.mix.uk": (24, 20), "l1.mix.uv": (36, 20), "l1.mix.sink": (3,), "l1.mix.g": (36, 80), "l1.mix.o": (80, 36),
                        "l2.mix.q.b": (24,), "l2.mix.k.b": (24,), "l2.mix.v.b": (24,), "l3.mix.k": (10, 80), "l3.mix.v.b": (4,)}.items():
        assert tuple(specs[name].shape) == shape, name
    # a layer without a feed-forward: a file need not hold (but may hold) the second sublayer's norm and stream weights
    assert not specs["l2.norm2"].required and not specs["l2.hc2.in"].required and not specs["l2.hc2.mix"].required and "l2.mlp.router" not in specs
    assert specs["l0.norm2"].required and specs["l0.hc2.in"].required
    assert "l0.mix.q.b" not in specs and "l2.mix.o.b" not in specs and "l0.mlp.e6.gate" not in specs
    assert "l3.mlp.shared.gate" not in specs and "l3.mlp.correction" in specs                            # a layer without a shared expert


def test_cache_needs():
    m = _model("K")
    specs = m.cache_specs()
    assert len(specs) == 8                                               # every run of a repeated layer keeps a cache of its own
    assert specs[0] == KVCacheSpec(2, 8, 5, v_head_dim=12)
    assert specs[1] == specs[3] == specs[5] == KVCacheSpec(1, 24, 9, v_head_dim=0)     # rows of latent + rotated part, a window of 9
    assert specs[2] == KVCacheSpec(4, 6, None, v_head_dim=6, chunk=7) and specs[7] == KVCacheSpec(1, 10, None, v_head_dim=4, chunk=1000)
    groups, per_run = plan_groups(specs, m.cache_from())
    assert len(groups) == 4 and per_run[1] == per_run[3] == per_run[5] and per_run[2] == per_run[4] and per_run[2] != per_run[7]


def test_pages_behind_a_chunk_go_back():
    """Pages of 8, chunks of 20: once the next position lies in chunk c, the pages wholly before position 20 c are free; a page that
    the chunk's start cuts stays."""
    cm = CacheManager([GroupSpec("g", 16, None, 0, 20)], 8, 2)
    cm.admit("a")
    held = []
    for n in (19, 1, 1, 19, 1, 7, 40):
        cm.append("a", n)
        cm.release_out_of_window("a")
        cm.check()
        held.append([i for i, p in enumerate(cm.block_table("a", "g")) if p >= 0])
    # tokens so far: 19, 20, 21, 40, 41, 48, 88 -> the chunk of the next position starts at 0, 20, 20, 40, 40, 40, 80
    assert held == [[0, 1, 2], [2], [2], [], [5], [5], [10]]       # at 40 tokens every page lies behind the next chunk
    cm.free("a")
    assert cm.num_free_pages("g") == 16


def test_pages_behind_a_window_and_a_chunk():
    cm = CacheManager([GroupSpec("g", 16, 12, 0, 32)], 8, 1)
    cm.admit("a")
    cm.append("a", 30)
    cm.release_out_of_window("a")          # next position 30 reads from max(30 - 11, 0) = 19: pages 0 and 1 are dead
    assert [p >= 0 for p in cm.block_table("a", "g")] == [False, False, True, True]
    cm.append("a", 3)
    cm.release_out_of_window("a")          # next position 33 lies in the chunk from 32
    assert [p >= 0 for p in cm.block_table("a", "g")] == [False, False, False, False, True]


@pytest.mark.parametrize("change, message", [
    (lambda d: d["layers"][1].update(type="conv"), "type"),
    (lambda d: d["layers"][0]["mixer"].update(kv_heads=4), "kv_heads"),
    (lambda d: d["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda d: d["layers"][0]["mixer"].pop("mask"), "mask"),
    (lambda d: d["layers"][2]["mixer"]["mask"].update(size=0), "size"),
    (lambda d: d["layers"][2]["mixer"].update(softcap=-1.0), "softcap"),
    (lambda d: d["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda d: d["layers"][1]["mixer"]["rot"].update(dims=2), "rot"),
    (lambda d: d["layers"][1]["mixer"].update(rot_dim=3), "rot"),
    (lambda d: d["layers"][0]["mlp"]["router"].update(top=7), "top"),
    (lambda d: d["layers"][0]["mlp"]["router"].update(top=5), "groups"),
    (lambda d: d["layers"][0]["mlp"]["router"]["groups"].update(count=4), "groups"),
    (lambda d: d["layers"][0]["mlp"]["router"]["groups"].update(keep=4), "groups"),
    (lambda d: d["layers"][1]["mlp"].update(kind="dense"), "mlp.kind"),
    (lambda d: d["layers"][0]["mlp"]["shared"].update(ff=0), "ff"),
    (lambda d: d.update(streams=0), "streams"),
    (lambda d: d["loop"].update(stop=5), "loop"),
    (lambda d: d["loop"].update(times=0), "loop"),
    (lambda d: d.pop("norm"), "norm"),
    (lambda d: d.update(layers=[]), "layers"),
])
def test_refusals(change, message):
    d = copy.deepcopy(NAT["K"])
    change(d)
    with pytest.raises(ConfigError, match=message):
        config_from_dict(d)


def test_to_dict_round_trip_and_keys_that_are_absent():
    for name in NAT:
        cfg = nat_config(name)
        assert config_from_dict(cfg.to_dict()) == cfg
    d = copy.deepcopy(NAT["L"])
    assert "loop" not in nat_config("L").to_dict() and nat_config("L").streams == 1
    d.pop("streams")                                                      # one ordinary residual stream: no hyper-connection weights
    bare = config_from_dict(d)
    assert bare.plan().streams == 1 and [l.block for l in bare.plan().layers] == ["pre_norm"] * 4 and "streams" not in bare.to_dict()
    names = Model(bare.plan(), Runtime(torch.device("cpu"), torch.bfloat16)).tensor_specs()
    assert "l0.norm1" in names and "l0.norm2" in names and "l1.norm2" not in names and not any(".hc" in n for n in names)
    assert any(".hc" in n for n in _model("L").tensor_specs())
    d["layers"][2]["mixer"].pop("softcap")                                # a chunked layer without a cap
    assert config_from_dict(d).plan().layers[2].mixer.params["softcap"] is None


# ------------------------------------------------------------------------------------ the plain implementation against itself

def test_what_a_position_sees():
    ok = PN.visible(12, window=4)
    assert ok[7].tolist() == [False] * 4 + [True] * 4 + [False] * 4 and ok[2].tolist() == [True] * 3 + [False] * 9
    ok = PN.visible(12, chunk=5)
    assert ok[7].tolist() == [False] * 5 + [True] * 3 + [False] * 4 and ok[5].tolist() == [False] * 5 + [True] + [False] * 6
    assert ok[4].tolist() == [True] * 5 + [False] * 7
    assert bool(PN.visible(6, window=1).diag().all()) and int(PN.visible(6, window=1).sum()) == 6


def test_a_sink_takes_its_share_and_nothing_else():
    s = rand(5, 5, seed=1).double()
    ok = PN.visible(5)
    free = PN.softmax_rows(s, ok)
    assert torch.allclose(free.sum(-1), torch.ones(5, dtype=torch.float64))
    sunk = PN.softmax_rows(s, ok, sink=torch.tensor([[0.3]], dtype=torch.float64))
    share = math.exp(0.3) / (torch.exp(s.masked_fill(~ok, -math.inf)).sum(-1) + math.exp(0.3))
    assert torch.allclose(sunk.sum(-1), 1.0 - share) and torch.allclose(sunk / sunk.sum(-1, keepdim=True), free)
    assert torch.allclose(PN.softmax_rows(s, ok, sink=torch.tensor([[-1e9]], dtype=torch.float64)), free)


def test_the_rotation_turns_pairs_of_neighbours_and_no_more():
    x = rand(4, 3, 10, seed=2).double()
    y = PN.rotate_pairs(x, torch.tensor([0, 1, 5, 9]), 100.0, 6)
    assert torch.equal(y[..., 6:], x[..., 6:]) and torch.equal(y[0], x[0])
    a = 5 * 100.0 ** (-2 / 6)
    assert torch.allclose(y[2, 1, 2], x[2, 1, 2] * math.cos(a) - x[2, 1, 3] * math.sin(a))
    assert torch.allclose(y[2, 1, 3], x[2, 1, 3] * math.cos(a) + x[2, 1, 2] * math.sin(a))
    # scores of rotated queries and keys depend on the distance alone
    q, k = rand(1, 6, seed=3).double(), rand(1, 6, seed=4).double()
    at = lambda i, j: float(PN.rotate_pairs(q, torch.tensor([i]), 50.0, 6) @ PN.rotate_pairs(k, torch.tensor([j]), 50.0, 6).T)
    assert abs(at(9, 4) - at(105, 100)) < 1e-9


def test_no_look_ahead_and_the_masks_cut():
    W = 24
    x = rand(40, W, seed=5).double()
    m = {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 10, "scale": 0.5, "mask": {"size": 8}, "softcap": 2.0}
    w = {"q": rand(24, W, seed=6).double(), "k": rand(12, W, seed=7).double(), "v": rand(20, W, seed=8).double(), "o": rand(W, 40, seed=9).double(),
         "q.b": rand(24, seed=10).double(), "k.b": rand(12, seed=11).double(), "v.b": rand(20, seed=12).double()}
    for fn in (PN.sliding_attention, PN.chunked_attention):
        whole = fn(x, w, m)
        assert torch.allclose(fn(x[:23], w, m), whole[:23])
    # a window: what lies 8 or more positions back does not matter; chunks: nothing before the chunk's start does
    x2 = x.clone()
    x2[:16] += 1.0
    assert torch.allclose(PN.sliding_attention(x2, w, m)[23:], PN.sliding_attention(x, w, m)[23:])
    assert not torch.allclose(PN.sliding_attention(x2, w, m)[22], PN.sliding_attention(x, w, m)[22])
    assert torch.allclose(PN.chunked_attention(x2, w, m)[16:], PN.chunked_attention(x, w, m)[16:])
    # a cap far above the scores changes nothing, one that bites does
    loose = PN.chunked_attention(x, w, dict(m, softcap=1e6))
    assert torch.allclose(loose, PN.grouped_attention(x, w, m, bias=True, chunk=8)) and not torch.allclose(loose, PN.chunked_attention(x, w, m))


def test_choice_by_corrected_scores_within_the_best_groups():
    W, E = 16, 8
    w = {"router": rand(E, W, seed=1).double(), "correction": torch.zeros(E, dtype=torch.float64)}
    x = rand(50, W, seed=2).double()
    s = torch.softmax(x @ w["router"].T, -1)
    r = {"experts": E, "top": 2, "scale": 1.5}
    idx, wts, _ = PN.route(x, w, r)
    assert torch.equal(idx, s.topk(2).indices) and torch.allclose(wts, 1.5 * s.topk(2).values)
    # a correction moves the choice, not the weights
    w2 = dict(w, correction=torch.tensor([0, 0, 0, 0, 0, 0, 0, 5.0], dtype=torch.float64))
    idx2, wts2, _ = PN.route(x, w2, r)
    assert bool((idx2[:, 0] == 7).all()) and torch.allclose(wts2[:, 0], 1.5 * s[:, 7])
    # groups of two of which one is kept: both experts come from the block that holds the best ranking number
    idx3, _, _ = PN.route(x, w, dict(r, groups={"count": 4, "keep": 1}))
    assert bool((idx3[:, 0] // 2 == idx3[:, 1] // 2).all()) and torch.equal(idx3[:, 0], s.argmax(-1))
    # negative ranking numbers: an expert outside the kept blocks is never taken, although its score is above theirs
    w4 = dict(w, correction=torch.tensor([-3.0, -3.5, 0, 0, 0, 0, 0, 0], dtype=torch.float64))
    idx4, _, _ = PN.route(x, w4, dict(r, top=4, groups={"count": 4, "keep": 2}))
    assert bool(((idx4 // 2).sort(-1).values[:, 0] == (idx4 // 2).sort(-1).values[:, 1]).all()) and not bool((idx4 < 2).any())


def test_copies_of_the_stream():
    xs = rand(3, 5, 7, seed=1).double()
    y = rand(5, 7, seed=2).double()
    eye, ones = torch.eye(3, dtype=torch.float64), torch.ones(3, dtype=torch.float64)
    assert torch.allclose(PN.hyper_write(xs, y, eye, ones), xs + y)                      # the ordinary residual sum, three times
    mix = rand(3, 3, seed=3).double()
    out = PN.hyper_write(xs, y, mix, torch.zeros(3, dtype=torch.float64))
    assert torch.allclose(out[2], mix[0, 2] * xs[0] + mix[1, 2] * xs[1] + mix[2, 2] * xs[2])      # indexed [from, to]
    assert torch.allclose(PN.hyper_read(xs, torch.tensor([1.0, 0.0, 2.0], dtype=torch.float64)), xs[0] + 2 * xs[2])
