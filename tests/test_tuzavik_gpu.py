"""The Tuzavik design in the engine against the plain implementation: each mechanism alone, then whole models under every
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
from plain import tuzavik as PZ
from test_engine_gpu import first_bad, run_schedule
from test_zatupel_gpu import CUTS, DEV, DT, DTYPES, PART_TOL, _bf16_weights, _feed, _rt, make_runner
from tuzavik_models import LENGTHS, TUZ, make_tuz_dir
from zatupel_models import rand

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LONG_CUTS = [(0, 64), (64, 130), (130, 131), (131, 133), (133, 150)]


# ----------------------------------------------------------------------------------------------- small kernels

@pytest.mark.parametrize("dtype", DT)
def test_two_token_embedding_keeps_the_previous_token_per_slot(dtype):
    """Portions of two requests side by side, down to one token; a slot that another request used starts from the first-token
    row again; multipliers whose products pass 2^31."""
    from forge_b200.cache import CacheStorage
    from forge_b200.config import PartSpec
    from forge_b200.engine import StepEntry, build_step_batch
    from forge_b200.parts import StateSpec, build_part
    V, W, buckets, mp, mc = 50000, 24, 37, 1000003, 77777
    emb = build_part("embedding", PartSpec("pair_embedding", {"vocab_size": V, "hidden_size": W, "buckets": buckets, "mul_prev": mp, "mul_cur": mc}),
                     _rt(dtype))
    t = {n: rand(*s.shape, seed=i + 1).to(torch.bfloat16) for i, (n, s) in enumerate(emb.tensor_specs().items())}
    emb.bind(t)
    dev = torch.device(DEV)
    storage = CacheStorage([StateSpec((1,), torch.float32)], [None], 8, 8, 2, dtype, dev, embedding_spec=emb.cache_spec())
    toks = {"a": random_tokens(40, V, 1), "b": random_tokens(40, V, 2), "c": random_tokens(9, V, 3)}
    table, pair = t["embed"].double(), t["bigram"].double()
    want = {r: PZ.embed(x, table, pair, {"bigram": {"buckets": buckets, "mul_prev": mp, "mul_cur": mc}}) for r, x in toks.items()}
    storage.manager.admit("c")
    batch = build_step_batch([StepEntry("c", toks["c"], [])], storage.manager, dev, 64)
    storage.zero_state_slots(storage.manager.take_fresh_slots())
    assert max_rel_err(emb.forward_step(batch, storage.embedding), want["c"]) <= 1e-6
    storage.manager.free("c")
    for r in ("a", "b"):
        storage.manager.admit(r)
    done = {"a": 0, "b": 0}
    for na, nb in ((5, 1), (1, 7), (2, 2), (1, 1), (20, 0), (11, 29)):
        entries = [StepEntry(r, toks[r][done[r]:done[r] + n], []) for r, n in (("a", na), ("b", nb)) if n]
        batch = build_step_batch(entries, storage.manager, dev, 64)
        storage.zero_state_slots(storage.manager.take_fresh_slots())
        out = emb.forward_step(batch, storage.embedding).cpu()
        o = 0
        for e in entries:
            n = len(e.tokens)
            ref = want[e.req_id][done[e.req_id]:done[e.req_id] + n]
            assert max_rel_err(out[o:o + n], ref) <= 1e-6, (e.req_id, done)
            done[e.req_id] += n
            o += n


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("H", [7, 48, 1030])
def test_output_norm_added_to_the_stream(dtype, H):
    from forge_b200 import kernels
    y, r0 = rand(9, H, seed=H, scale=3.0), rand(9, H, seed=H + 1)
    wy, wn = rand(H, seed=1, scale=0.3), rand(H, seed=2, scale=0.3)
    r = r0.clone().to(DEV)
    nxt = kernels.rmsnorm_add(y.to(DEV), (1 + wy).to(DEV), r, 1e-3, 0.6, w_next=(1 + wn).to(DEV), out_dtype=dtype)
    want = r0.double() + 0.6 * PZ.norm_around_zero(y.double(), wy.double(), 1e-3)
    assert max_rel_err(r, want) <= 2e-6
    assert max_rel_err(nxt, PZ.norm_around_zero(want, wn.double(), 1e-3)) <= PART_TOL[dtype]
    r = r0.clone().to(DEV)
    assert kernels.rmsnorm_add(y.to(DEV), (1 + wy).to(DEV), r, 1e-3, 0.6) is None and max_rel_err(r, want) <= 2e-6


# ----------------------------------------------------------------------------------------------- retention

RETENTION = [(3, 10, 6, 4), (2, 6, 14, 6), (1, 40, 24, 0), (4, 64, 32, 64), (2, 32, 64, 16), (2, 128, 16, 128), (1, 8, 130, 2), (1, 160, 8, 100),
             (2, 256, 24, 256)]


def _retention(dtype, W, heads, dim, vdim, rot, decay, eps=1e-4, base=300.0):
    from forge_b200.config import PartSpec
    from forge_b200.parts import build_part
    return build_part("mixer", PartSpec("retention", {
        "hidden_size": W, "num_heads": heads, "head_dim": dim, "v_head_dim": vdim, "decay": decay, "eps": eps,
        "position": PartSpec("rope_halves", {"head_dim": dim, "rotary_dims": rot, "theta": base})}), _rt(dtype))


class _Adds:
    """The mixers of this design return their output; the feeding helper wants it added to a stream."""
    def __init__(self, mixer):
        self.mixer = mixer

    def forward(self, x, batch, cache, residual):
        residual.add_(self.mixer.forward(x, batch, cache, None))


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("heads, dim, vdim, rot", RETENTION)
def test_retention_alone(dtype, heads, dim, vdim, rot):
    from forge_b200.cache import CacheStorage
    W, T, eps = 56, 62, 1e-4
    decay = [(0.5, 1.0, 0.97, 0.9)[n % 4] for n in range(heads)]
    mixer = _retention(dtype, W, heads, dim, vdim, rot, decay, eps)
    t, w = _bf16_weights(mixer, 0.25, seed=heads + dim)
    mixer.bind(t)
    storage = CacheStorage([mixer.cache_spec()], [None], 8, 8, 3, dtype, torch.device(DEV))
    x = rand(T, W, seed=60).to(dtype)
    # a slot that another request used before: its rows must come back as zeros
    _feed(_Adds(mixer), storage, x, [(0, 9)], requests=("old",))
    storage.manager.free("old")
    got = _feed(_Adds(mixer), storage, x, CUTS, requests=("a", "b"))
    m = {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay, "rot": {"dims": rot, "base": 300.0}}
    want = PZ.retention(x.double(), w, m, eps)
    for r in ("a", "b"):
        assert max_rel_err(got[r], want) <= PART_TOL[dtype], r


@pytest.mark.parametrize("dtype", DT)
def test_a_state_that_is_lost_shows(dtype):
    """No decay, and tokens after the first write little: what the first token wrote is most of the output 60 tokens later, so a
    state that was dropped or zeroed between steps could not pass."""
    from forge_b200.cache import CacheStorage
    W, T = 32, 61
    mixer = _retention(dtype, W, 2, 8, 8, 4, [1.0, 0.9995])
    t, w = _bf16_weights(mixer, 0.25, seed=5)
    mixer.bind(t)
    storage = CacheStorage([mixer.cache_spec()], [None], 8, 8, 2, dtype, torch.device(DEV))
    x = rand(T, W, seed=61).to(dtype)
    x[1:] *= 0.05
    got = _feed(_Adds(mixer), storage, x, [(0, 1)] + [(i, i + 1) for i in range(1, 40)] + [(40, 42), (42, 61)])["r"]
    m = {"heads": 2, "dim": 8, "vdim": 8, "decay": [1.0, 0.9995], "rot": {"dims": 4, "base": 300.0}}
    want = PZ.retention(x.double(), w, m, 1e-4)
    assert max_rel_err(got, want) <= PART_TOL[dtype]
    # without the first token every later output is another: the head norm hides sizes, not directions
    x2 = x.clone()
    x2[0] = 0
    assert max_rel_err(PZ.retention(x2.double(), w, m, 1e-4)[1:], want[1:]) > 0.3


@pytest.mark.parametrize("dtype", DT)
def test_retention_positions_count_from_the_request_start(dtype):
    """The rotation's angle is the position in the request, not the place in the step: the same tokens as a second request in the
    same step, and fed from position 0 in portions, give the same as alone."""
    from forge_b200.cache import CacheStorage
    W, T = 40, 150
    mixer = _retention(dtype, W, 2, 16, 8, 16, [0.99, 0.95], base=20.0)
    t, w = _bf16_weights(mixer, 0.3, seed=8)
    mixer.bind(t)
    storage = CacheStorage([mixer.cache_spec()], [None], 8, 8, 2, dtype, torch.device(DEV))
    x = rand(T, W, seed=62).to(dtype)
    got = _feed(_Adds(mixer), storage, x, LONG_CUTS, requests=("a", "b"))
    want = PZ.retention(x.double(), w, {"heads": 2, "dim": 16, "vdim": 8, "decay": [0.99, 0.95], "rot": {"dims": 16, "base": 20.0}}, 1e-4)
    assert max_rel_err(got["a"], want) <= PART_TOL[dtype] and max_rel_err(got["b"], want) <= PART_TOL[dtype]


# ----------------------------------------------------------------------------------------------- the products per head

@pytest.mark.parametrize("in_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T, H, K, N, R", [(1, 3, 8, 20, 4), (150, 2, 72, 70, 6), (67, 5, 128, 64, 0), (9, 1, 200, 129, 2), (130, 4, 64, 136, 8)])
def test_products_per_head_on_the_tensor_cores(in_dtype, T, H, K, N, R):
    """Token, channel and reduction counts that do not fill the kernel's tiles of 64; the rotated channels behind the outputs."""
    from forge_b200 import kernels
    x = rand(T, H * (K + R), seed=T + K).to(in_dtype)
    w = rand(H, K, N, seed=N, scale=0.2).to(torch.bfloat16)
    pos = torch.arange(5, 5 + T, dtype=torch.int32)
    freq = torch.tensor([0.5 ** i for i in range(R // 2)], dtype=torch.float32)
    args = dict(R=R, positions=pos.to(DEV), freq=freq.to(DEV), amp=1.25) if R else {}
    got = kernels.head_linear(x.to(DEV), w.to(DEV), H, K, N, torch.bfloat16, **args).float().cpu().view(T, H, N + R)
    simt = kernels.head_linear(x.to(DEV), w.to(DEV), H, K, N, torch.bfloat16, simt=True, **args).float().cpu().view(T, H, N + R)
    xd = x.double().view(T, H, K + R)
    want = torch.einsum("thk,hkn->thn", xd[..., :K].to(torch.bfloat16).double(), w.double())
    assert max_rel_err(got[..., :N], want) <= 6e-3 and max_rel_err(simt[..., :N], want) <= 8e-3
    if R:
        a = pos.double()[:, None] * freq.double()[None, :]
        u, v = xd[..., K::2], xd[..., K + 1::2]
        rot = torch.stack([u * a.cos()[:, None] - v * a.sin()[:, None], v * a.cos()[:, None] + u * a.sin()[:, None]], dim=-1).flatten(-2) * 1.25
        assert max_rel_err(got[..., N:], rot) <= 6e-3 and max_rel_err(simt[..., N:], rot) <= 6e-3


# ----------------------------------------------------------------------------------------------- latent attention

STRETCH = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 2.0}
LATENT = {
    "all_sizes_differ": dict(num_heads=3, head_dim=8, rot_dim=4, v_head_dim=12, kv_rank=20, q_rank=28, scale=0.4, theta=50.0, scaling=STRETCH),
    "one_head_no_stretch": dict(num_heads=1, head_dim=16, rot_dim=8, v_head_dim=8, kv_rank=40, q_rank=10, scale=0.25, theta=10000.0, scaling=None),
    "rotated_wider_than_the_rest": dict(num_heads=4, head_dim=6, rot_dim=10, v_head_dim=20, kv_rank=12, q_rank=36, scale=0.35, theta=77.0,
                                        scaling={"factor": 16.0, "original": 40, "fast": 4.0, "slow": 1.0}),
    # sizes that the tensor-core kernel takes in bfloat16, fed in portions that cross its tiles
    "wide": dict(num_heads=8, head_dim=32, rot_dim=16, v_head_dim=48, kv_rank=96, q_rank=64, scale=0.15, theta=250000.0,
                 scaling={"factor": 8.0, "original": 128, "fast": 16.0, "slow": 2.0}, tokens=150, cuts=LONG_CUTS),
    "latent_of_two_value_chunks": dict(num_heads=6, head_dim=16, rot_dim=16, v_head_dim=24, kv_rank=416, q_rank=32, scale=0.2, theta=5e3,
                                       scaling=None, tokens=150, cuts=LONG_CUTS),
    "wide_latent_of_128": dict(num_heads=5, head_dim=24, rot_dim=32, v_head_dim=16, kv_rank=128, q_rank=48, scale=0.2, theta=1e4, scaling=None,
                               tokens=150, cuts=LONG_CUTS),
}


def _latent(dtype, W, o, own=True, eps=1e-4):
    from forge_b200.config import PartSpec
    from forge_b200.parts import build_part
    o = {k: v for k, v in o.items() if k not in ("tokens", "cuts")}
    theta, scaling = o.pop("theta"), o.pop("scaling")
    return build_part("mixer", PartSpec("latent_attention", dict(o, hidden_size=W, eps=eps, own_latent=own, position=PartSpec(
        "rope_pairs", {"head_dim": o["rot_dim"], "rotary_dims": o["rot_dim"], "theta": theta, "scaling": scaling}))), _rt(dtype))


def _plain_latent_sizes(o):
    rot = {"dims": o["rot_dim"], "base": o["theta"]}
    if o["scaling"]:
        rot["scaling"] = o["scaling"]
    return {"heads": o["num_heads"], "dim": o["head_dim"], "rot_dim": o["rot_dim"], "vdim": o["v_head_dim"], "kv_rank": o["kv_rank"],
            "q_rank": o["q_rank"], "scale": o["scale"], "rot": rot}


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("kind", list(LATENT))
def test_latent_attention_alone(dtype, kind):
    from forge_b200.cache import CacheStorage
    o = LATENT[kind]
    W, T, cuts = 40, o.get("tokens", 62), o.get("cuts", CUTS)
    mixer = _latent(dtype, W, o)
    t, w = _bf16_weights(mixer, 0.35, seed=len(kind))
    mixer.bind(t)
    storage = CacheStorage([mixer.cache_spec()], [None], 8, 48, 2, dtype, torch.device(DEV))
    x = rand(T, W, seed=50).to(dtype)
    got = _feed(_Adds(mixer), storage, x, cuts, requests=("a", "b"))
    want, _ = PZ.latent_attention(x.double(), w, _plain_latent_sizes(o), 1e-4)
    for r in ("a", "b"):
        assert max_rel_err(got[r], want) <= PART_TOL[dtype], (kind, r)


@pytest.mark.parametrize("dtype", DT)
def test_a_layer_reads_the_rows_that_another_layer_cached(dtype):
    """Two mixers on one set of pages: the first writes rows from ITS input, the second has no down-projection for keys and
    values and attends over the first one's rows with matrices, heads and a scale of its own, whatever its own input is."""
    from forge_b200.cache import CacheStorage
    from forge_b200.engine import StepEntry, build_step_batch
    W, T = 40, 62
    first = dict(LATENT["all_sizes_differ"])
    second = dict(first, num_heads=5, head_dim=4, v_head_dim=6, q_rank=12, scale=0.7)
    a, b = _latent(dtype, W, first), _latent(dtype, W, second, own=False)
    ta, wa = _bf16_weights(a, 0.35, seed=1)
    tb, wb = _bf16_weights(b, 0.35, seed=2)
    assert "mix.dkv" not in tb and "mix.dkv.norm" not in tb
    a.bind(ta), b.bind(tb)
    dev = torch.device(DEV)
    storage = CacheStorage([a.cache_spec(), b.cache_spec()], [None, 0], 8, 16, 1, dtype, dev)
    assert storage.layers[1].kv.data_ptr() == storage.layers[0].kv.data_ptr() and not storage.layers[1].writable
    xa, xb = rand(T, W, seed=51).to(dtype), rand(T, W, seed=52).to(dtype)
    want_a, kept = PZ.latent_attention(xa.double(), wa, _plain_latent_sizes(first), 1e-4)
    want_b, _ = PZ.latent_attention(xb.double(), wb, _plain_latent_sizes(second), 1e-4, shared=kept)
    storage.manager.admit("r")
    got_a, got_b = torch.zeros(T, W), torch.zeros(T, W)
    for lo, hi in CUTS:
        batch = build_step_batch([StepEntry("r", [0] * (hi - lo), [])], storage.manager, dev, 64)
        got_a[lo:hi] = a.forward(xa[lo:hi].to(DEV).contiguous(), batch, storage.layers[0], None).cpu()
        got_b[lo:hi] = b.forward(xb[lo:hi].to(DEV).contiguous(), batch, storage.layers[1], None).cpu()
    assert max_rel_err(got_a, want_a) <= PART_TOL[dtype] and max_rel_err(got_b, want_b) <= PART_TOL[dtype]


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("page_size", [8, 64])
# the second is a shape that the tensor-core kernel takes in bfloat16, the third one whose value columns it takes in two chunks (eight warps)
@pytest.mark.parametrize("C, R, H", [(6, 2, 2), (96, 16, 8), (448, 32, 4)])
def test_one_row_that_stands_out(dtype, page_size, C, R, H):
    """Latent rows are zero except one whose score is huge for head 0; a row's second channel carries its position, its third
    is one.  Head 0 returns the row's position if the token sees it (far back among hundreds, at a page's border, the token
    itself) and the mean of the visible positions if it does not (the row lies ahead, in the same portion); the other heads
    return the mean.  For a prompt's portion and for single tokens, on pages that the case before gave back."""
    from forge_b200 import kernels
    from forge_b200.cache import CacheStorage
    from forge_b200.engine import StepEntry, build_step_batch
    from forge_b200.parts import KVCacheSpec
    N, P, KD = 300, 27, C + R
    dev = torch.device(DEV)
    storage = CacheStorage([KVCacheSpec(1, KD, None, v_head_dim=0)], [None], page_size, 64 * 8 // page_size, 2, dtype, dev)
    group = next(iter(storage.manager.groups))
    rows_of = storage.layers[0].kv.view(-1, KD)
    for case, (star, where) in enumerate([(0, 0), (150, 0), (63, C), (64, 0), (N - 1, C + R - 1), (N, 0), (N + 5, C), (N + P - 1, 0), (N + P, 0),
                                          (N + P + 1, C)]):
        rid = f"r{case}"
        storage.manager.admit(rid)
        total = N + P + 2
        rows = torch.zeros(total, KD)
        rows[star, where] = 10.0                                           # in the latent's channels or in the shared rotated part
        rows[:, 1] += torch.arange(total, dtype=torch.float32)
        rows[:, 2] = 1.0
        q = torch.zeros(total, H, KD)
        q[:, 0, where] = 10.0                                              # head 0 asks for the row; the others for nothing
        q[:, :, 1:3] = 0.0
        done = 0
        for n in (N, P, 1, 1):                                             # the context, a portion, two single tokens
            batch = build_step_batch([StepEntry(rid, [0] * n, [])], storage.manager, dev, 64)
            g = batch.groups[group]
            rows_of[g.slot_mapping.long()] = rows[done:done + n].to(DEV).to(dtype)
            out = kernels.latent_attention(q[done:done + n].reshape(n, H * KD).to(DEV).to(dtype).contiguous(), storage.layers[0].kv, g, batch,
                                           H, C, R, page_size, 1.0).float().cpu().view(n, H, C)
            for t in range(n) if n <= P else ():
                i = done + t
                mean = i / 2.0
                tol = (1e-4 if dtype == torch.float32 else 2e-2) * max(1.0, i)
                for h in range(H):
                    want = float(star) if (h == 0 and star <= i and where != 1) else mean
                    assert abs(out[t, h, 1] - want) <= tol and abs(out[t, h, 2] - 1.0) <= 1e-2, (star, where, i, h, out[t, h, :3].tolist(), want)
            done += n
        storage.manager.free(rid)                                          # the next case takes over these pages
        storage.manager.check()


# ----------------------------------------------------------------------------------------------- routed experts

@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("W, F, E, top, T", [(40, 24, 5, 1, 19), (40, 100, 3, 3, 19), (64, 16, 8, 2, 3), (64, 48, 6, 2, 300), (192, 128, 4, 3, 130),
                                             (64, 16, 8, 1, 3), (64, 16, 8, 3, 2), (40, 24, 5, 1, 2), (64, 24, 10, 3, 3), (72, 40, 7, 2, 1),
                                             (520, 264, 12, 5, 2)])
def test_routed_experts_alone(dtype, W, F, E, top, T):
    """Few tokens (every pair on its own, an odd and an even number of experts a token, rows longer than a warp's pass), some more (room
    for the step's tokens per expert) and many (pairs ranked by expert), one expert, all experts."""
    from forge_b200.config import PartSpec
    from forge_b200.parts import build_part
    ff = build_part("feed_forward", PartSpec("routed_experts", {"hidden_size": W, "intermediate_size": F, "experts": E, "top": top}), _rt(dtype))
    t = {n: rand(*s.shape, seed=i, scale=0.3).to(torch.bfloat16) for i, (n, s) in enumerate(ff.tensor_specs().items())}
    ff.bind(t)
    x = rand(T, W, seed=9, scale=1.5).to(dtype)
    w = {k.split("mlp.", 1)[1]: v.double() for k, v in t.items()}
    # no test rests on a close call: tokens whose last chosen score is nearly the next one's are left out
    s = torch.sigmoid(x.double() @ w["router"].t()).sort(dim=-1, descending=True).values
    clear = torch.ones(T, dtype=torch.bool) if top == E else (s[:, top - 1] - s[:, top]) > 1e-2
    assert int(clear.sum()) >= max(1, T // 2)
    got = ff.forward(x.to(DEV), None).cpu()
    want = PZ.routed_ff(x.double(), w, {"router": {"experts": E, "top": top}})
    assert max_rel_err(got[clear], want[clear]) <= PART_TOL[dtype]
    r0 = rand(T, W, seed=10)
    res = r0.clone().to(DEV)
    ff.forward(x.to(DEV), res)
    assert max_rel_err(res.cpu()[clear], (r0.double() + want)[clear]) <= PART_TOL[dtype]


@pytest.mark.parametrize("T", [4, 11, 127])
def test_experts_that_nobody_chose_run_no_product(T):
    """bfloat16 steps below the ranked path's size give every expert room for the step's tokens and skip, on the device, the products
    of an expert without tokens: five of eight experts can never be chosen here (one input channel is constant and their router rows
    weigh it down), and whatever their rows of the buffers hold must not show."""
    from forge_b200.config import PartSpec
    from forge_b200.parts import build_part
    W, F, E, top = 64, 32, 8, 2
    ff = build_part("feed_forward", PartSpec("routed_experts", {"hidden_size": W, "intermediate_size": F, "experts": E, "top": top}),
                    _rt(torch.bfloat16))
    t = {n: rand(*s.shape, seed=40 + i, scale=0.3).to(torch.bfloat16) for i, (n, s) in enumerate(ff.tensor_specs().items())}
    t["mlp.router"][3:, 0] = -6.0
    ff.bind(t)
    assert ff.gate_up_of[0].tensor_core and T * top >= E
    x = rand(T, W, seed=T, scale=1.0)
    x[:, 0] = 4.0
    x = x.to(torch.bfloat16)
    w = {k.split("mlp.", 1)[1]: v.double() for k, v in t.items()}
    s_ = torch.sigmoid(x.double() @ w["router"].t())
    assert bool((s_[:, 3:].max(dim=1).values < s_[:, :3].sort(dim=1, descending=True).values[:, top - 1]).all())
    srt = s_.sort(dim=-1, descending=True).values
    clear = (srt[:, top - 1] - srt[:, top]) > 1e-2
    assert int(clear.sum()) >= max(1, T // 2)
    want = PZ.routed_ff(x.double(), w, {"router": {"experts": E, "top": top}})
    for _ in range(2):                                                      # the second time over buffers that the first left filled
        got = ff.forward(x.to(DEV), None).cpu()
        assert torch.isfinite(got).all() and max_rel_err(got[clear], want[clear]) <= PART_TOL[torch.bfloat16]


def test_router_scores_are_not_renormalised_and_the_lower_index_wins_a_tie():
    from forge_b200 import kernels
    router = torch.zeros(6, 8)
    router[:, 0] = torch.tensor([0.5, 2.0, -1.0, 2.0, 0.0, 2.0])
    x = torch.zeros(3, 8)
    x[:, 0] = torch.tensor([1.0, -1.0, 0.0])
    idx, wts = kernels.moe_route(x.to(DEV), router.to(DEV), 2)
    assert idx.cpu().tolist() == [[1, 3], [2, 4], [0, 1]]
    sg = lambda z: 1.0 / (1.0 + math.exp(-z))
    assert torch.allclose(wts.cpu(), torch.tensor([[sg(2.0), sg(2.0)], [sg(1.0), sg(0.0)], [0.5, 0.5]]), atol=1e-6)
    idx, wts = kernels.moe_route(x.to(DEV), router.to(DEV), 2, softmax=True, renorm=True)
    assert idx.cpu().tolist()[0] == [1, 3] and torch.allclose(wts.cpu().sum(-1), torch.ones(3), atol=1e-6)


# ----------------------------------------------------------------------------------------------- whole models

class _Plain:
    def __init__(self, d):
        self.dir = d
        self.cfg, self.tensors = PZ.load(d)

    def forward(self, toks, streams=None, margins=None, choices=None):
        return PZ.forward(self.cfg, self.tensors, list(toks), streams=streams, margins=margins, choices=choices)

    def forward_as_routed_in_16_bits(self, toks):
        """Where two experts' router logits lie within the rounding of 16-bit activations, either choice is right and the
        outputs differ.  So the 16-bit runtime is compared with the plain implementation taking the experts that the engine
        took for the whole prompt, and every choice that is not the plain router's own must be such a close call."""
        theirs = _engine_choices(self.dir, list(toks))
        if not theirs:
            return self.forward(toks)
        margins = []
        out = self.forward(toks, margins=margins, choices=theirs)
        own = _plain_choices(self.cfg, self.tensors, list(toks), theirs)
        for k, m in enumerate(margins):
            for t in torch.nonzero(m > 0.02).flatten().tolist():
                assert sorted(theirs[k][t].tolist()) == own[k][t], f"routed layer {k}, token {t}: the engine chose other experts on a clear call"
        return out


def _plain_choices(cfg, tensors, toks, choices):
    """Per routed layer and token the sorted experts that the plain router chooses, given the stream that ``choices`` lead to."""
    seen = []
    orig = PZ.routed_ff

    def spy(x, w, mlp, margins=None, chosen=None):
        z = x @ w["router"].t()
        seen.append([sorted(r) for r in torch.topk(z, mlp["router"]["top"], dim=-1).indices.tolist()])
        return orig(x, w, mlp, margins, chosen)
    PZ.routed_ff = spy
    try:
        PZ.forward(cfg, tensors, toks, choices=choices)
    finally:
        PZ.routed_ff = orig
    return seen


def _engine_choices(d, toks):
    """The experts that the engine's bfloat16 runtime chooses for one whole prompt, one [T, top] tensor per routed layer."""
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


@pytest.fixture(scope="module", params=["X", "Y", "Z"])
def tuz(request, tmp_path_factory):
    name = request.param
    d = make_tuz_dir(tmp_path_factory, name)
    plain = _Plain(d)
    reqs = {f"r{i}": random_tokens(n, TUZ[name]["vocab"], seed=10 * i + ord(name)) for i, n in enumerate(LENGTHS[name])}
    want = {"float32": {rid: plain.forward(toks).float() for rid, toks in reqs.items()},
            "bfloat16": {rid: plain.forward_as_routed_in_16_bits(toks).float() for rid, toks in reqs.items()}}
    return name, d, plain, reqs, want


def test_layer_by_layer(tuz):
    """The residual stream after every layer, in 32-bit."""
    name, d, plain, reqs, want = tuz
    from forge_b200.engine import StepEntry
    runner = make_runner(d, "float32", 256)
    streams = []
    for b in set(runner.model.blocks):
        def wrap(orig):
            def f(residual, batch, cache):
                orig(residual, batch, cache)
                streams.append(residual.clone())
            return f
        b.forward = wrap(b.forward)
    toks = reqs["r2"]
    runner.admit("x")
    runner.step([StepEntry("x", toks, [])])
    ref = []
    plain.forward(toks, streams=ref)
    assert len(streams) == len(ref) == len(TUZ[name]["layers"])
    for i, s in enumerate(streams):
        assert max_rel_err(s, ref[i]) <= 2e-5, f"layer {i}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("schedule", ["whole", "last_one_by_one", "changing_portions", "mixed"])
def test_schedules_equal_plain(tuz, dtype, schedule):
    name, d, plain, reqs, want = tuz
    steps = getattr(schedules, schedule)(reqs)
    # exactly as many pages as the schedule's peak needs: freed pages and slots are taken again at once
    runner = make_runner(d, dtype, schedules.peak_tokens(reqs, steps, round_to=8))
    got = run_schedule(runner, reqs, steps)
    assert first_bad(got, want[dtype], TOL[dtype]) is None, first_bad(got, want[dtype], TOL[dtype])
    assert runner.manager.num_free_pages() == {g: runner.num_pages for g in runner.manager.groups}


@pytest.mark.parametrize("dtype", DTYPES)
def test_page_size_and_graphs_do_not_matter(tuz, dtype):
    name, d, plain, reqs, want = tuz
    small = {k: reqs[k] for k in list(reqs)[:3]}
    for ps, graphs in ((16, True), (64, True), (8, False)):
        steps = schedules.mixed(small, max_live=2)
        runner = make_runner(d, dtype, schedules.peak_tokens(small, steps, round_to=ps), page_size=ps, cuda_graphs=graphs)
        got = run_schedule(runner, small, steps)
        msg = first_bad(got, {k: want[dtype][k] for k in small}, TOL[dtype])
        assert msg is None, f"page size {ps}: {msg}"


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_and_first_tokens(tuz, dtype):
    """Two tokens, one, then hundreds one by one: the state runs long, pages fill and follow, the stretched rotation turns."""
    name, d, plain, reqs, want = tuz
    n = {"X": 230, "Y": 260, "Z": 170}[name]
    toks = random_tokens(n, TUZ[name]["vocab"], seed=77)
    ref = (plain.forward(toks) if dtype == "float32" else plain.forward_as_routed_in_16_bits(toks)).float()
    runner = make_runner(d, dtype, -(-n // 8) * 8)
    steps = [([("x", 0, 2)], [])] + [([("x", p, 1)], []) for p in range(2, n)]
    got = run_schedule(runner, {"x": toks}, steps)
    msg = first_bad(got, {"x": ref}, TOL[dtype])
    assert msg is None, msg


def test_fp32_logits_do_not_depend_on_the_cut(tuz):
    """In 32-bit every sum is taken in an order that the position alone decides: the four schedules agree to rounding."""
    name, d, plain, reqs, want = tuz
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
def test_generation_through_the_scheduler(tuz, dtype):
    """Greedy generation through forge.Model and through RequestScheduler with more requests than slots and few pages."""
    import forge_b200 as forge
    name, d, plain, reqs, want = tuz
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


def test_trace_replay_as_a_subprocess(tuz, tmp_path):
    name, d, plain, reqs, want = tuz
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
    V = TUZ[name]["vocab"]
    for n, rows in asked.items():
        got = torch.from_numpy(np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(len(rows), V))
        ref = torch.stack([want["float32"][rid][pos] for rid, pos in rows])
        assert max_rel_err(got, ref) <= TOL["float32"], n
    assert sorted(os.listdir(out)) == sorted(f"{n}.f32" for n in asked)


def test_command_line(tuz):
    """bin/forge-cli on a Tuzavik folder: greedy tokens in 32-bit follow the plain implementation; sampling runs."""
    name, d, plain, reqs, want = tuz
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
