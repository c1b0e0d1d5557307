"""Whole-sequence Tuzavik decoder, written from the design's equations: one request, all of its tokens, every time; no
cache, no state carried over calls, no batching, no fusing, no absorbed products.  float64 on the CPU.  One function per
mechanism.

Notation: T tokens, W model width, H heads, D unrotated and R rotated query/key channels of a head, E value channels of a
head, C the key/value latent's width, Cq the query latent's width; N retention heads with K key and V value channels.
"""
import json
import math
import os

import torch

from .safetensors_reader import read_safetensors


def rms_unit(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm_around_zero(x, w, eps):
    """RMS norm whose stored weight is the distance of the factor from one."""
    return rms_unit(x, eps) * (1.0 + w)


def silu(z):
    return z * torch.sigmoid(z)


def two_token_rows(tokens, buckets, mul_prev, mul_cur):
    """Row of the two-token table for every token: (previous * mul_prev + current * mul_cur) mod buckets; the first token of a
    sequence takes the row after the hashed ones."""
    rows = [buckets]
    for a, b in zip(tokens[:-1], tokens[1:]):
        rows.append((a * mul_prev + b * mul_cur) % buckets)
    return rows


def embed(tokens, table, pair_table, emb):
    x = table[torch.tensor(tokens)]
    bg = emb.get("bigram") if emb else None
    if bg:
        x = x + pair_table[torch.tensor(two_token_rows(tokens, bg["buckets"], bg["mul_prev"], bg["mul_cur"]))]
    return x


def plain_frequencies(base, dims, dtype=torch.float64):
    i = torch.arange(dims // 2, dtype=dtype)
    return torch.pow(torch.tensor(float(base), dtype=dtype), -2.0 * i / dims)


def stretched_frequencies(base, dims, scaling, dtype=torch.float64):
    """(frequencies, amplitude) of a rotation whose slow pairs are slowed down by ``factor``: a ramp over the pair index
    between the pairs that turn ``fast`` and ``slow`` times within ``original`` positions; cos and sin are multiplied by
    0.1 ln(factor) + 1."""
    f = plain_frequencies(base, dims, dtype)
    factor, orig = float(scaling["factor"]), float(scaling["original"])

    def pair_that_turns(times):
        return dims * math.log(orig / (2.0 * math.pi * times)) / (2.0 * math.log(base))
    lo = max(math.floor(pair_that_turns(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair_that_turns(float(scaling["slow"]))), dims - 1)
    i = torch.arange(dims // 2, dtype=dtype)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x, positions, freq, dims, layout, amplitude=1.0):
    """x [T, heads, channels]: the first ``dims`` channels turn by position * freq; "halves": channel i with i + dims/2,
    "pairs": channel 2i with 2i + 1.  The pair (u, v) becomes (u cos - v sin, v cos + u sin), cos and sin times amplitude."""
    out = x.clone()
    if dims == 0:
        return out
    ang = positions.to(x.dtype)[:, None] * freq[None, :]
    c, s = (torch.cos(ang) * amplitude)[:, None, :], (torch.sin(ang) * amplitude)[:, None, :]
    if layout == "halves":
        u, v = x[..., :dims // 2], x[..., dims // 2:dims]
        out[..., :dims // 2] = u * c - v * s
        out[..., dims // 2:dims] = v * c + u * s
    else:
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * c - v * s
        out[..., 1:dims:2] = v * c + u * s
    return out


def retention(h, w, m, eps):
    """h [T, W]; w: {"q", "k", "v", "g", "o"}; linear attention with one decay per head, no softmax, no denominator:
    S_t = decay S_{t-1} + k_t v_t^T, o_t = S_t^T q_t, walked token by token."""
    T = h.shape[0]
    N, K, V = m["heads"], m["dim"], m.get("vdim", m["dim"])
    pos = torch.arange(T)
    rot = m.get("rot") or {"dims": 0, "base": 10000.0}
    dims = rot.get("dims", K)
    freq = plain_frequencies(rot["base"], dims, h.dtype) if dims else None
    q = rotate((h @ w["q"].t()).view(T, N, K), pos, freq, dims, "halves")
    k = rotate((h @ w["k"].t()).view(T, N, K), pos, freq, dims, "halves") * K ** -0.5
    v = (h @ w["v"].t()).view(T, N, V)
    o = torch.zeros(T, N, V, dtype=h.dtype)
    for n in range(N):
        S = torch.zeros(K, V, dtype=h.dtype)
        for t in range(T):
            S = float(m["decay"][n]) * S + torch.outer(k[t, n], v[t, n])
            o[t, n] = S.t() @ q[t, n]
    y = rms_unit(o, eps).reshape(T, N * V) * silu(h @ w["g"].t())
    return y @ w["o"].t()


def latent_of(h, w, m, eps, positions):
    """(normed latent [T, C], rotated shared key part [T, R]) of the layer that owns the key/value down-projection."""
    C, R = m["kv_rank"], m["rot_dim"]
    both = h @ w["dkv"].t()
    c = rms_unit(both[:, :C], eps) * w["dkv.norm"]
    freq, amp = _rot(m, h.dtype)
    return c, rotate(both[:, None, C:], positions, freq, R, "pairs", amp)[:, 0]


def _rot(m, dtype):
    rot, R = m["rot"], m["rot_dim"]
    if rot.get("scaling"):
        return stretched_frequencies(rot["base"], R, rot["scaling"], dtype)
    return plain_frequencies(rot["base"], R, dtype), 1.0


def latent_attention(h, w, m, eps, shared=None):
    """h [T, W]; queries through a normed latent; keys and values made per head from one normed latent a token, plus one
    rotated key part that all heads share.  ``shared``: (latent, rotated key part) of another layer to use instead of this
    layer's own.  Returns (output, (latent, rotated key part))."""
    T = h.shape[0]
    H, D, R, E = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    pos = torch.arange(T)
    cq = rms_unit(h @ w["dq"].t(), eps) * w["dq.norm"]
    q = (cq @ w["uq"].t()).view(T, H, D + R)
    freq, amp = _rot(m, h.dtype)
    q_flat, q_rot = q[..., :D], rotate(q[..., D:], pos, freq, R, "pairs", amp)
    c, k_rot = shared if shared is not None else latent_of(h, w, m, eps, pos)
    k_flat = (c @ w["uk"].t()).view(T, H, D)
    v = (c @ w["uv"].t()).view(T, H, E)
    scores = (torch.einsum("ihd,jhd->hij", q_flat, k_flat) + torch.einsum("ihr,jr->hij", q_rot, k_rot)) * float(m["scale"])
    mask = torch.ones(T, T, dtype=torch.bool).tril()
    p = torch.softmax(scores.masked_fill(~mask, float("-inf")), dim=-1)
    o = torch.einsum("hij,jhe->ihe", p, v).reshape(T, H * E)
    return o @ w["o"].t(), (c, k_rot)


def gated_ff(x, w_gate, w_up, w_down):
    return (silu(x @ w_gate.t()) * (x @ w_up.t())) @ w_down.t()


def routed_ff(x, w, mlp, margins=None, chosen=None):
    """Every token goes through the ``top`` experts with the largest sigmoid(router logits); their outputs are added with
    those sigmoids as weights, not renormalised.  ``margins``: a list that receives, per token, how far the last chosen expert's
    router logit lies above the first one left out, as a fraction of the largest logit's size (inf when all are chosen).
    ``chosen`` [T, top]: experts to take instead of the router's own choice (their weights are still the router's scores)."""
    n, top = mlp["router"]["experts"], mlp["router"]["top"]
    z = x @ w["router"].t()
    score = torch.sigmoid(z)
    if margins is not None:
        zs = z.sort(dim=-1, descending=True).values
        margins.append(torch.full((x.shape[0],), float("inf"), dtype=x.dtype) if top == n else
                       (zs[:, top - 1] - zs[:, top]) / z.abs().amax(dim=-1).clamp_min(1e-30))
    if chosen is None:
        chosen = torch.topk(score, top, dim=-1).indices
    out = torch.zeros(x.shape[0], w["e0.down"].shape[0], dtype=x.dtype)
    for t in range(x.shape[0]):
        for e in chosen[t].tolist():
            out[t] += score[t, e] * gated_ff(x[t:t + 1], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"])[0]
    return out


def _sub(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(cfg, tensors, tokens, dtype=torch.float64, streams=None, margins=None, choices=None):
    """Logits [T, vocab] of one sequence.  ``streams``: a list that receives the residual stream after every layer;
    ``margins``: one that receives every routed layer's margins (see routed_ff); ``choices``: per routed layer, in order, the
    experts to take instead of the router's own."""
    w = {k: torch.as_tensor(v).to(dtype) for k, v in tensors.items() if torch.as_tensor(v).dtype.is_floating_point}
    eps, mult = float(cfg["norm"]["eps"]), float(cfg.get("residual_mult", 1.0))
    x = embed(list(tokens), w["embed"], w.get("bigram"), cfg.get("embedding"))
    kept, routed = {}, 0
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        h = norm_around_zero(x, w[p + "norm1"], eps)
        if layer["type"] == "retention":
            y = retention(h, _sub(w, p + "mix."), m, eps)
        else:
            src = m.get("kv_from")
            y, kept[i] = latent_attention(h, _sub(w, p + "mix."), m, eps, shared=None if src is None else kept[src])
        x = x + mult * norm_around_zero(y, w[p + "norm1b"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = norm_around_zero(x, w[p + "norm2"], eps)
            mw = _sub(w, p + "mlp.")
            if mlp["kind"] == "dense":
                y = gated_ff(h, mw["gate"], mw["up"], mw["down"])
            else:
                y = routed_ff(h, mw, mlp, margins, None if choices is None else choices[routed])
                routed += 1
            x = x + mult * norm_around_zero(y, w[p + "norm2b"], eps)
        if streams is not None:
            streams.append(x.clone())
    return (norm_around_zero(x, w["final.norm"], eps) @ w["head"].t()) * float(cfg.get("logit_scale", 1.0))


def load(model_dir):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(model_dir, "model.safetensors"))
