"""The Natalorn design in the engine against the plain implementation: each mechanism alone, then whole models under every
way of cutting and batching, long decoding, generation through the scheduler, and the trace replay."""
import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import schedules
from helpers import TOL, assert_greedy_follows_plain, max_rel_err, random_tokens
from natalorn_models import LENGTHS, NAT, make_nat_dir
from plain import natalorn as PN
from test_engine_gpu import first_bad, run_schedule
from test_zatupel_gpu import CUTS, DEV, DT, DTYPES, PART_TOL, _bf16_weights, _feed, _rt, make_runner
from zatupel_models import rand

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LONG_CUTS = [(0, 64), (64, 130), (130, 131), (131, 133), (133, 150), (150, 152), (152, 230)]


class _Adds:
    """The mixers of this design return their output; the feeding helper wants it added to a stream."""
    def __init__(self, mixer):
        self.mixer = mixer

    def forward(self, x, batch, cache, residual):
        residual.add_(self.mixer.forward(x, batch, cache, None))


# ----------------------------------------------------------------------------------------------- the stream's copies

@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("S, W", [(1, 48), (2, 7), (3, 1030), (4, 256), (7, 33), (16, 40)])
def test_copies_of_the_stream(dtype, S, W):
    from forge_b200 import kernels
    T = 9
    e = rand(T, W, seed=S)
    xs = kernels.streams_expand(e.to(DEV), S)
    assert torch.equal(xs.cpu().view(T, S, W), e[:, None, :].expand(T, S, W))
    x0 = rand(T, S, W, seed=S + 1, scale=2.0)
    y, mix = rand(T, W, seed=S + 2), torch.eye(S) + rand(S, S, seed=S + 3, scale=0.4)
    w_out, w_in, wn = rand(S, seed=S + 4), rand(S, seed=S + 5), 1.0 + rand(W, seed=S + 6, scale=0.3)
    plain_x = x0.double().permute(1, 0, 2)                                  # the plain functions keep the copies in front
    # reading alone
    xs = x0.reshape(T, S * W).to(DEV).contiguous()
    got = kernels.streams_mix(xs, S, in_next=w_in.to(DEV), w_next=wn.to(DEV), eps=1e-3, out_dtype=dtype)
    assert torch.equal(xs.cpu(), x0.reshape(T, S * W))
    assert max_rel_err(got, PN.rms_norm(PN.hyper_read(plain_x, w_in.double()), wn.double(), 1e-3)) <= PART_TOL[dtype]
    # chosen rows
    rows = torch.tensor([7, 0, 3], dtype=torch.int32)
    got = kernels.streams_mix(xs, S, in_next=w_in.to(DEV), w_next=wn.to(DEV), eps=1e-3, out_dtype=dtype, rows=rows.to(DEV))
    assert max_rel_err(got, PN.rms_norm(PN.hyper_read(plain_x, w_in.double()), wn.double(), 1e-3)[rows.long()]) <= PART_TOL[dtype]
    # writing, and writing followed by the next sublayer's read
    new = PN.hyper_write(plain_x, y.double(), mix.double(), w_out.double())
    for with_read in (False, True):
        xs = x0.reshape(T, S * W).to(DEV).contiguous()
        got = kernels.streams_mix(xs, S, y=y.to(DEV), mix=mix.to(DEV), out_w=w_out.to(DEV), in_next=w_in.to(DEV) if with_read else None,
                                  w_next=wn.to(DEV) if with_read else None, eps=1e-3, out_dtype=dtype if with_read else None)
        assert max_rel_err(xs.view(T, S, W).permute(1, 0, 2), new) <= 2e-6
        if with_read:
            assert max_rel_err(got, PN.rms_norm(PN.hyper_read(new, w_in.double()), wn.double(), 1e-3)) <= PART_TOL[dtype]
        else:
            assert got is None


# ----------------------------------------------------------------------------------------------- attention without rotation

MASKED = {
    # sizes that only the kernel of fp32 arithmetic takes
    "window_shorter_than_a_page": dict(num_heads=6, num_kv_heads=2, head_dim=8, v_head_dim=12, scale=0.4, window=5),
    "window_of_one": dict(num_heads=4, num_kv_heads=1, head_dim=12, v_head_dim=20, scale=0.3, window=1),
    "window_longer_than_all": dict(num_heads=5, num_kv_heads=5, head_dim=4, v_head_dim=6, scale=0.7, window=1000),
    "chunks_and_cap_and_bias": dict(num_heads=4, num_kv_heads=4, head_dim=6, v_head_dim=6, scale=0.6, chunk=7, softcap=1.5, qkv_bias=True),
    "one_chunk_for_all": dict(num_heads=3, num_kv_heads=1, head_dim=10, v_head_dim=4, scale=0.3, chunk=1000, softcap=30.0, qkv_bias=True),
    "window_and_chunk": dict(num_heads=2, num_kv_heads=2, head_dim=8, v_head_dim=8, scale=0.5, window=11, chunk=16),
    # sizes that the tensor-core kernel takes in bfloat16, with edges inside and across its tiles of 64 keys
    "tc_window_70": dict(num_heads=8, num_kv_heads=2, head_dim=32, v_head_dim=24, scale=0.2, window=70, tokens=230, cuts=LONG_CUTS),
    "tc_window_64": dict(num_heads=2, num_kv_heads=2, head_dim=16, v_head_dim=64, scale=0.25, window=64, tokens=230, cuts=LONG_CUTS),
    "tc_chunk_72_cap": dict(num_heads=4, num_kv_heads=4, head_dim=64, v_head_dim=64, scale=0.12, chunk=72, softcap=2.0, qkv_bias=True,
                            tokens=230, cuts=LONG_CUTS),
    "tc_chunk_130": dict(num_heads=6, num_kv_heads=3, head_dim=48, v_head_dim=48, scale=0.15, chunk=130, softcap=50.0, qkv_bias=True,
                         tokens=230, cuts=LONG_CUTS),
    "tc_values_of_two_chunks": dict(num_heads=2, num_kv_heads=1, head_dim=16, v_head_dim=136, scale=0.25, window=33, tokens=150,
                                    cuts=LONG_CUTS[:5]),
}


def _masked(dtype, W, o):
    from forge_b200.config import PartSpec
    from forge_b200.parts import build_part
    o = {k: v for k, v in o.items() if k not in ("tokens", "cuts")}
    return build_part("mixer", PartSpec("masked_attention", dict(o, hidden_size=W)), _rt(dtype))


def _plain_masked(o, x, w):
    m = {"heads": o["num_heads"], "kv_heads": o["num_kv_heads"], "dim": o["head_dim"], "vdim": o["v_head_dim"], "scale": o["scale"]}
    return PN.grouped_attention(x, w, m, bias=o.get("qkv_bias", False), softcap=o.get("softcap"), window=o.get("window"), chunk=o.get("chunk"))


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("kind", list(MASKED))
def test_masked_attention_alone(dtype, kind):
    """Two requests side by side, fed in portions down to one token; pages behind the window or the chunk go back on the way."""
    from forge_b200.cache import CacheStorage
    o = MASKED[kind]
    W, T, cuts = 40, o.get("tokens", 62), o.get("cuts", CUTS)
    mixer = _masked(dtype, W, o)
    t, w = _bf16_weights(mixer, 0.35, seed=len(kind))
    mixer.bind(t)
    storage = CacheStorage([mixer.cache_spec()], [None], 8, 2 * -(-T // 8), 2, dtype, torch.device(DEV))
    x = rand(T, W, seed=50).to(dtype)
    got = _feed(_Adds(mixer), storage, x, cuts, requests=("a", "b"))
    want = _plain_masked(o, x.double(), w)
    for r in ("a", "b"):
        assert max_rel_err(got[r], want) <= PART_TOL[dtype], (kind, r)
    table = storage.manager.block_table("a", next(iter(storage.manager.groups)))
    reach = min(o.get("window") or T, (T % o["chunk"]) if o.get("chunk") else T)
    assert sum(p >= 0 for p in table) <= reach // 8 + 2, (kind, table)


def _stands_out_mixer(dtype, kind, size, W=16, D=16, E=8, H=2, G=1):
    """A mixer whose head 0 asks with a large number in query channel 0 whenever input channel 1 is set, whose keys carry input
    channel 0 there, and whose value channel 0 is input channel 2; the output projection hands the heads' value channel 0 through."""
    o = dict(num_heads=H, num_kv_heads=G, head_dim=D, v_head_dim=E, scale=0.5)
    if kind == "window":
        o.update(window=size)
    else:
        o.update(chunk=size, softcap=30.0, qkv_bias=True)
    mixer = _masked(dtype, W, o)
    t = {n: torch.zeros(s.shape, dtype=torch.bfloat16) for n, s in mixer.tensor_specs().items()}
    t["mix.q"][0, 1] = 10.0            # head 0, channel 0
    t["mix.k"][0, 0] = 10.0
    t["mix.v"][0, 2] = 1.0
    for h in range(H):
        t["mix.o"][h, h * E] = 1.0     # output channel h = head h's value channel 0
    mixer.bind(t)
    return mixer


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("page_size", [8, 64])
@pytest.mark.parametrize("kind, size, D, E", [("window", 40, 8, 4), ("window", 40, 16, 8), ("window", 136, 16, 8), ("chunk", 100, 8, 4),
                                              ("chunk", 100, 16, 8), ("chunk", 64, 16, 8)])
def test_one_key_that_stands_out(dtype, page_size, kind, size, D, E):
    """All keys are zero except one whose score is huge for head 0; values carry their position.  Head 0 returns that position where
    the token sees the key and the mean of the visible positions where it does not; head 1 always the mean.  The key lies far back,
    just inside and just outside the window (or the chunk), at a page's border, ahead in the same portion, or is the token itself;
    for the tokens of a prompt's portion (whose edges lie inside a tile and across pages) and for tokens that come alone; on pages
    that the case before gave back.  (D, E) = (16, 8) is a shape the tensor-core kernel takes in bfloat16."""
    from forge_b200.cache import CacheStorage
    from forge_b200.engine import StepEntry, build_step_batch
    N, P, W = 290, 27, 16
    dev = torch.device(DEV)
    mixer = _stands_out_mixer(dtype, kind, size, W, D, E)
    storage = CacheStorage([mixer.cache_spec()], [None], page_size, 64 * 8 // page_size, 2, dtype, dev)
    total = N + P + 2

    def sees(i, j):
        return j <= i and (i - j < size if kind == "window" else i // size == j // size)
    stars = [0, 150, N - size, N - size + 1, N - size + 5, N + P - size, N + P + 1 - size, 255, 256, N - 1, N, N + 5, N + P - 1, N + P, N + P + 1]
    stars += [size * (N // size + 1) - 1, size * (N // size + 1), size * (N // size + 1) + 3] if kind == "chunk" else []
    for case, star in enumerate(s for s in stars if 0 <= s < total):
        rid = f"r{case}"
        storage.manager.admit(rid)
        x = torch.zeros(total, W)
        x[star, 0] = 1.0
        x[:, 1] = 1.0
        x[:, 2] = torch.arange(total, dtype=torch.float32) / 4.0            # quarters of the position: exact in bfloat16 up to 64
        done = 0
        for n in (N, P, 1, 1):                                               # the context, a portion, two single tokens
            batch = build_step_batch([StepEntry(rid, [0] * n, [])], storage.manager, dev, 64)
            out = mixer.forward(x[done:done + n].to(DEV).to(dtype).contiguous(), batch, storage.layers[0], None).cpu()
            storage.manager.release_out_of_window(rid)
            for t in range(n) if n <= P else ():
                i = done + t
                seen = [j for j in range(i + 1) if sees(i, j)]
                mean = sum(seen) / len(seen) / 4.0
                tol = (1e-4 if dtype == torch.float32 else 2e-2) * max(1.0, i / 4.0)
                want0 = star / 4.0 if sees(i, star) else mean
                assert abs(float(out[t, 0]) - want0) <= tol and abs(float(out[t, 1]) - mean) <= tol, (kind, size, star, i, out[t, :2].tolist(), want0, mean)
            done += n
        storage.manager.free(rid)                                            # the next case takes over these pages
        storage.manager.check()


# ----------------------------------------------------------------------------------------------- latent attention

LATENT = {
    "all_sizes_differ": dict(num_heads=3, head_dim=8, rot_dim=4, v_head_dim=12, kv_rank=20, q_rank=28, scale=0.4, theta=50.0, window=9),
    "one_head_window_of_one": dict(num_heads=1, head_dim=16, rot_dim=8, v_head_dim=8, kv_rank=40, q_rank=10, scale=0.25, theta=1e4, window=1),
    "window_longer_than_all": dict(num_heads=4, head_dim=6, rot_dim=10, v_head_dim=20, kv_rank=12, q_rank=36, scale=0.35, theta=77.0, window=1000),
    # sizes of the tensor-core kernel (latent and rotated part multiples of 16), in portions that cross its tiles of 64 rows
    "tc_window_70": dict(num_heads=4, head_dim=32, rot_dim=16, v_head_dim=48, kv_rank=96, q_rank=64, scale=0.15, theta=250000.0, window=70,
                         tokens=230, cuts=LONG_CUTS),
    "tc_window_40_many_heads": dict(num_heads=8, head_dim=16, rot_dim=16, v_head_dim=24, kv_rank=96, q_rank=32, scale=0.2, theta=250000.0,
                                    window=40, tokens=230, cuts=LONG_CUTS),
    "tc_window_128_two_value_chunks": dict(num_heads=6, head_dim=16, rot_dim=16, v_head_dim=24, kv_rank=416, q_rank=32, scale=0.2, theta=5e3,
                                           window=128, tokens=230, cuts=LONG_CUTS),
}


def _latent(dtype, W, o, eps=1e-4, sink=True, out_gate=True):
    from forge_b200.config import PartSpec
    from forge_b200.parts import build_part
    o = {k: v for k, v in o.items() if k not in ("tokens", "cuts")}
    theta = o.pop("theta")
    return build_part("mixer", PartSpec("latent_attention", dict(o, hidden_size=W, eps=eps, sink=sink, out_gate=out_gate, position=PartSpec(
        "rope_pairs", {"head_dim": o["rot_dim"], "rotary_dims": o["rot_dim"], "theta": theta}))), _rt(dtype))


def _plain_latent_sizes(o):
    return {"heads": o["num_heads"], "dim": o["head_dim"], "rot_dim": o["rot_dim"], "vdim": o["v_head_dim"], "kv_rank": o["kv_rank"],
            "q_rank": o["q_rank"], "scale": o["scale"], "rot": {"dims": o["rot_dim"], "base": o["theta"]}, "mask": {"size": o["window"]}}


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("kind", list(LATENT))
def test_latent_attention_with_window_sink_and_gate(dtype, kind):
    from forge_b200.cache import CacheStorage
    o = LATENT[kind]
    W, T, cuts = 40, o.get("tokens", 62), o.get("cuts", CUTS)
    mixer = _latent(dtype, W, o)
    t, w = _bf16_weights(mixer, 0.35, seed=len(kind))
    mixer.bind(t)
    storage = CacheStorage([mixer.cache_spec()], [None], 8, 2 * -(-T // 8), 2, dtype, torch.device(DEV))
    x = rand(T, W, seed=50).to(dtype)
    got = _feed(_Adds(mixer), storage, x, cuts, requests=("a", "b"))
    want = PN.latent_attention(x.double(), w, _plain_latent_sizes(o), 1e-4)
    for r in ("a", "b"):
        assert max_rel_err(got[r], want) <= PART_TOL[dtype], (kind, r)
    table = storage.manager.block_table("a", next(iter(storage.manager.groups)))
    assert sum(p >= 0 for p in table) <= min(o["window"], T) // 8 + 2, (kind, table)


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("kind", ["all_sizes_differ", "tc_window_70"])
def test_a_sink_that_is_left_out_shows(dtype, kind):
    """One head's sink is large: that head's share of the output all but vanishes while the others keep theirs; a sink far below
    every score changes nothing; a gate that is shut (a large negative bias through a constant input channel) shuts the output."""
    from forge_b200.cache import CacheStorage
    o = LATENT[kind]
    W, T = 40, 62
    H, E = o["num_heads"], o["v_head_dim"]
    x = rand(T, W, seed=50)
    x[:, 0] = 1.0
    x = x.to(dtype)
    outs = {}
    for what in ("as_drawn", "head_0_sunk", "no_sink_at_all", "gate_shut"):
        mixer = _latent(dtype, W, o)
        t, w = _bf16_weights(mixer, 0.35, seed=3)
        if what == "head_0_sunk":
            t["mix.sink"][0] = 120.0
        if what == "no_sink_at_all":
            t["mix.sink"][:] = -1e4
        if what == "gate_shut":
            t["mix.g"][:E, 0] = -200.0                                       # head 0's gate, through the constant channel
        w = {n.split("mix.", 1)[-1]: v.double() for n, v in t.items()}
        mixer.bind(t)
        storage = CacheStorage([mixer.cache_spec()], [None], 8, 2 * -(-T // 8), 1, dtype, torch.device(DEV))
        outs[what] = (_feed(_Adds(mixer), storage, x, CUTS)["r"], PN.latent_attention(x.double(), w, _plain_latent_sizes(o), 1e-4), w)
        assert max_rel_err(outs[what][0], outs[what][1]) <= PART_TOL[dtype], what
    # what head 0 adds to the output is the difference to the output with its columns of W_o removed
    base, w = outs["as_drawn"][1], outs["as_drawn"][2]
    assert max_rel_err(outs["head_0_sunk"][0], outs["gate_shut"][1]) <= PART_TOL[dtype]      # both silence head 0 and nothing else
    assert float((outs["head_0_sunk"][1] - base).abs().max()) > 0.05 * float(base.abs().max())
    assert float((outs["no_sink_at_all"][1] - base).abs().max()) > 0.02 * float(base.abs().max())


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("page_size", [8, 64])
@pytest.mark.parametrize("C, R, H, window", [(6, 2, 2, 40), (96, 16, 8, 40), (96, 16, 4, 136), (448, 32, 4, 64)])
def test_one_row_that_stands_out_in_a_window(dtype, page_size, C, R, H, window):
    """Latent rows are zero except one whose score is huge for head 0; a row's second channel carries its position, its third is
    one.  Head 0 returns the row's position where the token sees it and the mean of the visible positions where it does not (it
    lies behind the window, or ahead); the other heads the mean.  A sink of zero takes 1 / (visible + 1) of the other heads'
    weights and next to nothing of head 0's where it sees the row."""
    from forge_b200 import kernels
    from forge_b200.cache import CacheStorage
    from forge_b200.engine import StepEntry, build_step_batch
    from forge_b200.parts import KVCacheSpec
    N, P, KD = 290, 27, C + R
    dev = torch.device(DEV)
    storage = CacheStorage([KVCacheSpec(1, KD, window, v_head_dim=0)], [None], page_size, 64 * 8 // page_size, 2, dtype, dev)
    group = next(iter(storage.manager.groups))
    rows_of = storage.layers[0].kv.view(-1, KD)
    sink = torch.zeros(H, device=DEV)
    total = N + P + 2
    stars = [(0, 0), (150, 0), (N - window, C), (N - window + 1, 0), (N + 3 - window, C + R - 1), (N + P - window, 0), (N + P + 1 - window, C),
             (255, 0), (256, 0), (N - 1, 0), (N, C), (N + 5, 0), (N + P, 0), (N + P + 1, C)]
    for case, (star, where) in enumerate((s, c) for s, c in stars if 0 <= s < total):
        rid = f"r{case}"
        storage.manager.admit(rid)
        rows = torch.zeros(total, KD)
        rows[star, where] = 10.0                                           # in the latent's channels or in the shared rotated part
        rows[:, 1] += torch.arange(total, dtype=torch.float32) / 4.0
        rows[:, 2] = 1.0
        q = torch.zeros(total, H, KD)
        q[:, 0, where] = 10.0                                              # head 0 asks for the row; the others for nothing
        q[:, :, 1:3] = 0.0
        done = 0
        for n in (N, P, 1, 1):
            batch = build_step_batch([StepEntry(rid, [0] * n, [])], storage.manager, dev, 64)
            g = batch.groups[group]
            rows_of[g.slot_mapping.long()] = rows[done:done + n].to(DEV).to(dtype)
            for sk in (None, sink):
                out = kernels.latent_attention(q[done:done + n].reshape(n, H * KD).to(DEV).to(dtype).contiguous(), storage.layers[0].kv, g, batch,
                                               H, C, R, page_size, 1.0, window=window, sink=sk).float().cpu().view(n, H, C)
                for t in range(n) if n <= P else ():
                    i = done + t
                    lo = max(0, i - window + 1)
                    count, mean = i + 1 - lo, (lo + i) / 2.0 / 4.0
                    tol = (1e-4 if dtype == torch.float32 else 2e-2) * max(1.0, i / 4.0)
                    for h in range(H):
                        found = h == 0 and lo <= star <= i and where != 1
                        share = 1.0 if sk is None else (1.0 if found else count / (count + 1.0))
                        want = (star / 4.0 if found else mean) * share
                        assert abs(out[t, h, 1] - want) <= tol and abs(out[t, h, 2] - share) <= 1e-2, (star, where, i, h, out[t, h, :3].tolist(), want)
            storage.manager.release_out_of_window(rid)
            done += n
        storage.manager.free(rid)                                          # the next case takes over these pages
        storage.manager.check()


# ----------------------------------------------------------------------------------------------- routed experts

def test_the_router_chooses_by_corrected_scores_within_the_best_groups():
    from forge_b200 import kernels
    for seed, (E, top, groups, keep, factor) in enumerate([(8, 2, 4, 2, 1.5), (12, 3, 3, 2, 1.5), (9, 3, 3, 1, 0.5), (6, 6, 1, 1, 1.0), (10, 1, 5, 5, 2.0),
                                                           (16, 4, 8, 2, 1.0), (7, 2, 0, 0, 1.0), (64, 6, 8, 3, 2.5)]):
        W, T = 24, 200
        w = {"router": rand(E, W, seed=seed, scale=0.5), "correction": rand(E, seed=seed + 50, scale=0.08)}
        x = rand(T, W, seed=seed + 100)
        r = {"experts": E, "top": top, "scale": factor}
        if groups:
            r["groups"] = {"count": groups, "keep": keep}
        want_idx, want_w, margin = PN.route(x.double(), {k: v.double() for k, v in w.items()}, r)
        idx, wts = kernels.moe_route(x.to(DEV), w["router"].to(DEV), top, softmax=True, correction=w["correction"].to(DEV), groups=groups, keep=keep,
                                     factor=factor)
        clear = margin > 1e-5
        assert int(clear.sum()) > T * 0.9
        assert torch.equal(idx.cpu().long()[clear], want_idx[clear]), (E, top, groups, keep)
        assert max_rel_err(wts.cpu()[clear], want_w[clear]) <= 1e-5
    # negative ranking numbers: experts of the dropped blocks are out although zero would beat the kept ones
    router, corr = torch.zeros(6, 8), torch.tensor([-0.5, -0.9, -0.6, -0.7, -0.8, -0.95])
    idx, wts = kernels.moe_route(torch.ones(2, 8).to(DEV), router.to(DEV), 2, softmax=True, correction=corr.to(DEV), groups=3, keep=1, factor=3.0)
    assert idx.cpu().tolist() == [[0, 1], [0, 1]] and torch.allclose(wts.cpu(), torch.full((2, 2), 0.5))


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("W, F, E, top, groups, keep, shared, T", [(40, 24, 6, 2, 3, 2, 40, 19), (40, 16, 4, 1, 1, 1, 8, 3), (64, 20, 8, 4, 4, 2, None, 2),
                                                                  (64, 48, 9, 3, 3, 1, 24, 300), (192, 128, 8, 2, 4, 2, 64, 130), (256, 64, 4, 2, 2, 2, 128, 1),
                                                                  (64, 16, 12, 3, 3, 2, 16, 11)])
def test_routed_experts_with_groups_and_a_shared_expert(dtype, W, F, E, top, groups, keep, shared, T):
    """Few tokens, some more and many (the three paths), with the shared expert added into the experts' sum."""
    from forge_b200.config import PartSpec
    from forge_b200.parts import build_part
    sh = None if shared is None else PartSpec("swiglu", {"hidden_size": W, "intermediate_size": shared, "suffix": "",
                                                        "names": {"gate": "mlp.shared.gate", "up": "mlp.shared.up", "down": "mlp.shared.down"}})
    ff = build_part("feed_forward", PartSpec("routed_experts", {"hidden_size": W, "intermediate_size": F, "experts": E, "top": top, "score": "softmax",
                                                                "correction": True, "groups": groups, "keep": keep, "route_scale": 1.7, "shared": sh}),
                    _rt(dtype))
    t = {n: rand(*s.shape, seed=i, scale=0.05 if n.endswith("correction") else 0.3).to(torch.bfloat16) for i, (n, s) in enumerate(ff.tensor_specs().items())}
    ff.bind(t)
    x = rand(T, W, seed=9, scale=1.5).to(dtype)
    w = {k.split("mlp.", 1)[1]: v.double() for k, v in t.items()}
    mlp = {"router": {"experts": E, "top": top, "scale": 1.7, "groups": {"count": groups, "keep": keep}}, "shared": shared}
    want, _, margin = PN.routed_ff(x.double(), w, mlp)
    clear = margin > 1e-3                                                   # no test rests on a close call
    assert int(clear.sum()) >= max(1, T // 3)
    got = ff.forward(x.to(DEV), None).cpu()
    assert max_rel_err(got[clear], want[clear]) <= PART_TOL[dtype]
    r0 = rand(T, W, seed=10)
    res = r0.clone().to(DEV)
    ff.forward(x.to(DEV), res)
    assert max_rel_err(res.cpu()[clear], (r0.double() + want)[clear]) <= PART_TOL[dtype]


# ----------------------------------------------------------------------------------------------- whole models

class _Plain:
    def __init__(self, d):
        self.dir = d
        self.cfg, self.tensors = PN.load(d)
        self.close = {}

    def forward(self, toks, layers_out=None, margins=None, choices=None):
        return PN.forward(self.cfg, self.tensors, list(toks), layers_out=layers_out, margins=margins, choices=choices)

    def forward_as_routed_in_16_bits(self, toks):
        """Where two experts' (or two blocks') ranking numbers lie within the rounding of 16-bit activations, either choice is right
        and the outputs differ.  So the 16-bit runtime is compared with the plain implementation taking the experts that the engine
        took for the whole prompt, and every choice that is not the plain router's own must be such a close call."""
        theirs = _engine_choices(self.dir, list(toks))
        if not theirs:
            return self.forward(toks)
        margins = []
        out = self.forward(toks, margins=margins, choices=theirs)
        assert len(margins) == len(theirs)
        for k, (own, m) in enumerate(margins):
            for t in torch.nonzero(m > 0.02).flatten().tolist():
                assert sorted(theirs[k][t].tolist()) == sorted(own[t].tolist()), f"routed run {k}, token {t}: the engine chose other experts on a clear call"
        # tokens with a close call somewhere: cut otherwise (a token alone, a portion) the 16-bit runtime may decide them the other way
        self.close[tuple(toks)] = torch.stack([m for _, m in margins]).min(dim=0).values < 0.008
        return out

    def close_calls(self, toks):
        return self.close.get(tuple(toks), torch.zeros(len(toks), dtype=torch.bool))


def _first_bad(plain, reqs, got, want, dtype):
    """``first_bad`` of the schedule's logits; in 16 bits the rows of tokens with a close call are not compared (no test rests on one)."""
    if dtype == "bfloat16":
        skipped = 0
        for rid, toks in reqs.items():
            skip = plain.close_calls(toks)
            skipped += int(skip.sum())
            got[rid][skip] = want[rid][skip]
        assert skipped <= 0.4 * sum(len(t) for t in reqs.values()), "too many of the router's calls are close"
    return first_bad(got, want, TOL[dtype])


def _engine_choices(d, toks):
    """The experts that the engine's bfloat16 runtime chooses for one whole prompt, one [T, top] tensor per routed layer run."""
    from forge_b200 import kernels
    from forge_b200.engine import StepEntry
    rec, orig = [], kernels.moe_route

    def spy(*a, **k):
        idx, wts = orig(*a, **k)
        rec.append(idx.cpu().long())
        return idx, wts
    kernels.moe_route = spy
    try:
        runner = make_runner(d, "bfloat16", -(-len(toks) // 8) * 8, cuda_graphs=False)
        runner.admit("x")
        runner.step([StepEntry("x", toks, [])])
    finally:
        kernels.moe_route = orig
    return rec


@pytest.fixture(scope="module", params=["K", "L", "M", "N"])
def nat(request, tmp_path_factory):
    name = request.param
    d = make_nat_dir(tmp_path_factory, name)
    plain = _Plain(d)
    reqs = {f"r{i}": random_tokens(n, NAT[name]["vocab"], seed=10 * i + ord(name)) for i, n in enumerate(LENGTHS[name])}
    want = {"float32": {rid: plain.forward(toks).float() for rid, toks in reqs.items()},
            "bfloat16": {rid: plain.forward_as_routed_in_16_bits(toks).float() for rid, toks in reqs.items()}}
    return name, d, plain, reqs, want


def test_layer_by_layer(nat):
    """The sum of the stream's copies after every layer run, in 32-bit."""
    name, d, plain, reqs, want = nat
    from forge_b200.engine import StepEntry
    runner = make_runner(d, "float32", 256)
    S, W = NAT[name].get("streams", 1), NAT[name]["width"]
    sums = []
    for b in set(runner.model.blocks):
        def wrap(orig):
            def f(residual, batch, cache):
                orig(residual, batch, cache)
                sums.append(residual.view(residual.shape[0], S, W).sum(dim=1))
            return f
        b.forward = wrap(b.forward)
    toks = reqs["r2"]
    runner.admit("x")
    runner.step([StepEntry("x", toks, [])])
    ref = []
    plain.forward(toks, layers_out=ref)
    assert len(sums) == len(ref) == len(PN.layer_order(NAT[name]))
    for i, s in enumerate(sums):
        assert max_rel_err(s, ref[i]) <= 2e-5, f"layer run {i}"


def test_weights_of_a_sublayer_that_is_not_there_are_let_pass(tmp_path_factory):
    """A layer without a feed-forward needs no norm and no stream weights for it; a file that holds some loads and computes the same."""
    from forge_b200.engine import ModelRunner, StepEntry
    from forge_b200.weights import random_tensors
    from natalorn_models import nat_config
    cfg = nat_config("L")
    tensors = random_tensors(cfg, seed=3, std=0.15, embed_std=0.7)
    assert "l1.norm2" not in tensors and "l1.hc2.in" not in tensors
    more = dict(tensors, **{"l1.norm2": torch.ones(48, dtype=torch.bfloat16), "l1.hc2.in": torch.ones(1, dtype=torch.bfloat16),
                            "l1.hc2.out": torch.ones(1, dtype=torch.bfloat16), "l1.hc2.mix": torch.ones(1, 1, dtype=torch.bfloat16)})
    toks = random_tokens(40, 130, seed=5)
    outs = []
    for t in (tensors, more):
        runner = ModelRunner(config=cfg, tensors=t, dtype="float32", page_size=8, cache_tokens=64, max_requests=1)
        runner.admit("x")
        outs.append(runner.step([StepEntry("x", toks, list(range(40)))]).cpu())
    assert torch.equal(outs[0], outs[1])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("schedule", ["whole", "last_one_by_one", "changing_portions", "mixed"])
def test_schedules_equal_plain(nat, dtype, schedule):
    name, d, plain, reqs, want = nat
    steps = getattr(schedules, schedule)(reqs)
    # exactly as many pages as the schedule's peak needs: freed pages and slots are taken again at once
    runner = make_runner(d, dtype, schedules.peak_tokens(reqs, steps, round_to=8))
    got = run_schedule(runner, reqs, steps)
    msg = _first_bad(plain, reqs, got, want[dtype], dtype)
    assert msg is None, msg
    assert runner.manager.num_free_pages() == {g: runner.num_pages for g in runner.manager.groups}


@pytest.mark.parametrize("dtype", DTYPES)
def test_page_size_and_graphs_do_not_matter(nat, dtype):
    name, d, plain, reqs, want = nat
    small = {k: reqs[k] for k in list(reqs)[:3]}
    for ps, graphs in ((16, True), (64, True), (8, False)):
        steps = schedules.mixed(small, max_live=2)
        runner = make_runner(d, dtype, schedules.peak_tokens(small, steps, round_to=ps), page_size=ps, cuda_graphs=graphs)
        got = run_schedule(runner, small, steps)
        msg = _first_bad(plain, small, got, {k: want[dtype][k] for k in small}, dtype)
        assert msg is None, f"page size {ps}: {msg}"


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_and_first_tokens(nat, dtype):
    """Two tokens, one, then hundreds one by one: windows and chunks pass over decoded tokens, pages fill, follow and go back."""
    name, d, plain, reqs, want = nat
    n = {"K": 230, "L": 260, "M": 170, "N": 120}[name]
    toks = random_tokens(n, NAT[name]["vocab"], seed=77)
    ref = (plain.forward(toks) if dtype == "float32" else plain.forward_as_routed_in_16_bits(toks)).float()
    runner = make_runner(d, dtype, -(-n // 8) * 8)
    steps = [([("x", 0, 2)], [])] + [([("x", p, 1)], []) for p in range(2, n)]
    got = run_schedule(runner, {"x": toks}, steps)
    msg = _first_bad(plain, {"x": toks}, got, {"x": ref}, dtype)
    assert msg is None, msg


def test_fp32_logits_do_not_depend_on_the_cut(nat):
    """In 32-bit every sum is taken in an order that the position alone decides: the four schedules agree to rounding."""
    name, d, plain, reqs, want = nat
    small = {k: reqs[k] for k in list(reqs)[:3]}
    outs = []
    for schedule in ("whole", "last_one_by_one", "changing_portions", "mixed"):
        steps = getattr(schedules, schedule)(small)
        runner = make_runner(d, "float32", schedules.peak_tokens(small, steps, round_to=8), cuda_graphs=False)
        outs.append(run_schedule(runner, small, steps))
    for o in outs[1:]:
        for rid in small:
            assert float((o[rid] - outs[0][rid]).abs().max()) <= 2e-5 * float(outs[0][rid].abs().max()), rid


@pytest.mark.parametrize("dtype", DTYPES)
def test_generation_through_the_scheduler(nat, dtype):
    """Greedy generation through forge.Model and through RequestScheduler with more requests than slots and few pages."""
    import forge_b200 as forge
    name, d, plain, reqs, want = nat
    model = forge.Model(d, dtype=dtype, block_size=8, max_num_seqs=2, cache_tokens=512, max_tokens_per_step=48)
    prompt = reqs["r1"][:37]
    out = model.generate(prompt, max_new_tokens=12, do_sample=False)
    assert out["num_generated_tokens"] == 12 and out["finish_reason"] == "length"
    logits_fn = lambda ids: (plain.forward(ids) if dtype == "float32" else plain.forward_as_routed_in_16_bits(ids)).float()
    assert_greedy_follows_plain(logits_fn, prompt, out["token_ids"], TOL[dtype], what="generate")
    sched = forge.RequestScheduler(model, max_num_seqs=2, max_tokens_per_step=48)
    prompts = [reqs["r0"][:50], reqs["r2"][:9], reqs["r3"][:31], reqs["r1"][:3]]
    ids = [sched.submit(p, 8, -1, forge.SamplerConfig(do_sample=False)) for p in prompts]
    done = {r.request_id: r for r in sched.run()}
    for rid, p in zip(ids, prompts):
        assert done[rid].num_generated == 8
        assert_greedy_follows_plain(logits_fn, p, list(done[rid].output_tokens), TOL[dtype], what=f"request {rid}")
    model.runner.manager.check()
    model.runner.check_status()


def test_trace_replay_as_a_subprocess(nat, tmp_path):
    name, d, plain, reqs, want = nat
    small = {k: reqs[k] for k in list(reqs)[:3]}
    steps = schedules.mixed(small, max_live=2)
    lines, asked = [], {}
    for n, (entries, end) in enumerate(steps):
        es = []
        for rid, p, cnt in entries:
            w = [cnt - 1] if (p + cnt) % 3 == 0 or p + cnt == len(small[rid]) else []
            es.append({"id": rid, "tokens": small[rid][p:p + cnt], "want": w})
            if w:
                asked.setdefault(n, []).extend((rid, p + i) for i in w)
        lines.append(json.dumps({"step": n, "entries": es, "end": end}))
    out = tmp_path / "out"
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", "float32", "--out", str(out),
                        "--max-tokens", str(schedules.peak_tokens(small, steps, round_to=64))], input="\n".join(lines) + "\n",
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done ")] == [f"done {n}" for n in range(len(steps))]
    V = NAT[name]["vocab"]
    for n, rows in asked.items():
        got = torch.from_numpy(np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(len(rows), V))
        ref = torch.stack([want["float32"][rid][pos] for rid, pos in rows])
        assert max_rel_err(got, ref) <= TOL["float32"], n
    assert sorted(os.listdir(out)) == sorted(f"{n}.f32" for n in asked)


def test_command_line(nat):
    """bin/forge-cli on a Natalorn folder: greedy tokens in 32-bit follow the plain implementation; sampling runs."""
    name, d, plain, reqs, want = nat
    prompt = reqs["r1"][:6]
    cli = [sys.executable, os.path.join(ROOT, "bin", "forge-cli"), "-m", d, "-p", " ".join(map(str, prompt)), "-n", "5", "--no-stream",
           "--page-size", "8", "--kv-pages", "2"]
    proc = subprocess.run(cli + ["--temp", "0", "--repeat-penalty", "1.0", "--dtype", "float32"], capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stderr[-2000:]
    got = [int(t) for t in proc.stdout.strip().splitlines()[0].split()]
    assert len(got) == 5 and "6 prompt" in proc.stdout and "5 generated" in proc.stdout
    assert_greedy_follows_plain(lambda ids: plain.forward(ids).float(), prompt, got, TOL["float32"], what="forge-cli")
    proc = subprocess.run(cli + ["--temp", "0.8", "--top-k", "20", "--seed", "3", "--dtype", "bfloat16"], capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert len(proc.stdout.strip().splitlines()[0].split()) == 5
