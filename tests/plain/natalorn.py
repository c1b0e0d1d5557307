"""Whole-sequence Natalorn decoder, written from the design's equations: one request, all of its tokens, every time; no
cache, no batching, no fusing, keys and values formed per head.  float64 on the CPU.  One function per mechanism.

Notation: T tokens, W model width, S streams, H query heads, G key/value heads, D query/key channels of a head (unrotated
ones in the latent mixer), R rotated channels, E value channels, C the key/value latent's width, Cq the query latent's.
"""
import json
import math
import os

import torch

from .safetensors_reader import read_safetensors


def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * w


def silu(z):
    return z * torch.sigmoid(z)


def visible(T, window=None, chunk=None):
    """[T, T] booleans: may position i (row) see position j (column)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if window is not None:
        ok = ok & (i - j < window)
    if chunk is not None:
        ok = ok & (i // chunk == j // chunk)
    return ok


def softmax_rows(scores, ok, sink=None):
    """Softmax over the visible columns of every row; ``sink`` (one number per row group) joins the denominator only."""
    s = scores.masked_fill(~ok, -math.inf)
    m = s.max(dim=-1, keepdim=True).values
    if sink is not None:
        m = torch.maximum(m, sink)
    p = torch.exp(s - m)
    den = p.sum(dim=-1, keepdim=True)
    if sink is not None:
        den = den + torch.exp(sink - m)
    return p / den


def rotate_pairs(x, positions, base, dims):
    """x [T, ..., >= dims]: channel 2i turns with channel 2i + 1 by position * base^(-2i/dims); the rest pass."""
    i = torch.arange(dims // 2, dtype=x.dtype)
    f = torch.pow(torch.tensor(float(base), dtype=x.dtype), -2.0 * i / dims)
    a = positions.to(x.dtype)[:, None] * f[None, :]                    # [T, dims/2]
    while a.dim() < x.dim():
        a = a.unsqueeze(1)
    c, s = torch.cos(a), torch.sin(a)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def grouped_attention(h, w, m, bias=False, softcap=None, window=None, chunk=None):
    """Softmax attention without positions in its scores: query head n reads key/value head n // (H/G)."""
    T = h.shape[0]
    H, G, D, E = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m.get("vdim", m["dim"])
    q, k, v = h @ w["q"].T, h @ w["k"].T, h @ w["v"].T
    if bias:
        q, k, v = q + w["q.b"], k + w["k.b"], v + w["v.b"]
    q, k, v = q.view(T, H, D), k.view(T, G, D), v.view(T, G, E)
    ok = visible(T, window, chunk)
    heads = []
    for n in range(H):
        g = n // (H // G)
        s = (q[:, n] @ k[:, g].T) * m["scale"]
        if softcap is not None:
            s = softcap * torch.tanh(s / softcap)
        heads.append(softmax_rows(s, ok) @ v[:, g])
    return torch.cat(heads, dim=-1) @ w["o"].T


def sliding_attention(h, w, m):
    return grouped_attention(h, w, m, window=m["mask"]["size"])


def chunked_attention(h, w, m):
    return grouped_attention(h, w, m, bias=True, softcap=m.get("softcap"), chunk=m["mask"]["size"])


def latent_attention(h, w, m, eps):
    T = h.shape[0]
    H, D, R, E, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    cq = rms_norm(h @ w["dq"].T, w["dq.norm"], eps)
    q = (cq @ w["uq"].T).view(T, H, D + R)
    down = h @ w["dkv"].T
    c = rms_norm(down[:, :C], w["dkv.norm"], eps)
    kr = rotate_pairs(down[:, C:], pos, m["rot"]["base"], R)             # [T, R], one for all heads
    qr = rotate_pairs(q[..., D:], pos, m["rot"]["base"], R)              # [T, H, R]
    ku = (c @ w["uk"].T).view(T, H, D)
    val = (c @ w["uv"].T).view(T, H, E)
    ok = visible(T, window=m["mask"]["size"])
    heads = []
    for n in range(H):
        s = (q[:, n, :D] @ ku[:, n].T + qr[:, n] @ kr.T) * m["scale"]
        heads.append(softmax_rows(s, ok, sink=w["sink"][n].reshape(1, 1)) @ val[:, n])
    o = torch.cat(heads, dim=-1) * torch.sigmoid(h @ w["g"].T)
    return o @ w["o"].T


def gated_ff(x, w_gate, w_up, w_down):
    return (silu(x @ w_gate.T) * (x @ w_up.T)) @ w_down.T


def route(x, w, r):
    """(chosen experts [T, top], their weights [T, top], margin [T]: how far the choice is from another one, the smaller of the
    gap between the last picked and the first passed-over ranking number and the gap between the last kept and the first dropped block)."""
    s = torch.softmax(x @ w["router"].T, dim=-1)
    choice = s + w["correction"]
    n, groups = r["experts"], r.get("groups")
    margin = torch.full((x.shape[0],), math.inf, dtype=x.dtype)
    if groups:
        per = n // groups["count"]
        best = choice.view(-1, groups["count"], per).max(dim=-1).values
        ranked = best.sort(dim=-1, descending=True)
        if groups["keep"] < groups["count"]:
            margin = ranked.values[:, groups["keep"] - 1] - ranked.values[:, groups["keep"]]
        allowed = torch.zeros_like(best, dtype=torch.bool).scatter_(1, ranked.indices[:, :groups["keep"]], True)
        choice = choice.masked_fill(~allowed.repeat_interleave(per, dim=1), -math.inf)
    ranked = choice.sort(dim=-1, descending=True)
    idx = ranked.indices[:, :r["top"]]
    if r["top"] < n:
        margin = torch.minimum(margin, ranked.values[:, r["top"] - 1] - ranked.values[:, r["top"]])
    return idx, s.gather(1, idx) * r.get("scale", 1.0), margin


def routed_ff(x, w, mlp, chosen=None):
    """``chosen`` (optional, [T, top]): take these experts instead of the router's own choice (their weights stay the router's)."""
    r = mlp["router"]
    idx, wts, margin = route(x, w, r)
    if chosen is not None:
        idx = chosen
        wts = torch.softmax(x @ w["router"].T, dim=-1).gather(1, idx) * r.get("scale", 1.0)
    y = torch.zeros_like(x)
    for t in range(x.shape[0]):
        for k in range(idx.shape[1]):
            e = int(idx[t, k])
            y[t] += wts[t, k] * gated_ff(x[t:t + 1], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"])[0]
    if mlp.get("shared"):
        y = y + gated_ff(x, w["shared.gate"], w["shared.up"], w["shared.down"])
    return y, idx, margin


def hyper_read(xs, w_in):
    """xs [S, T, W] -> what the sublayer's norm sees."""
    return torch.einsum("s,stw->tw", w_in, xs)


def hyper_write(xs, y, w_mix, w_out):
    """All streams at once from the old ones: new_t = sum_s mix[s, t] old_s + out[t] y."""
    return torch.einsum("st,sjw->tjw", w_mix, xs) + w_out[:, None, None] * y[None]


def _sub(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def layer_order(cfg):
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b = loop["start"], loop["stop"]
    return list(range(a)) + list(range(a, b)) * loop["times"] + list(range(b, n))


def mixer(kind, h, w, m, eps):
    if kind == "attention":
        return sliding_attention(h, w, m)
    if kind == "attention_2":
        return chunked_attention(h, w, m)
    if kind == "latent_attention":
        return latent_attention(h, w, m, eps)
    raise ValueError(kind)


def forward(cfg, tensors, tokens, dtype=torch.float64, layers_out=None, choices=None, margins=None):
    """Logits [T, vocab] of one sequence.  ``layers_out``: a list that receives the sum of the streams after every layer run.
    ``choices``: per routed feed-forward that runs, in order, the experts [T, top] to take instead of the router's own;
    ``margins``: a list that receives (the router's own experts, its margins) of every routed feed-forward that runs."""
    t = {k: torch.as_tensor(v).to(dtype) for k, v in tensors.items()}
    eps, S = cfg["norm"]["eps"], cfg.get("streams")
    x = t["embed"][torch.tensor(tokens)]
    xs = x[None].repeat(S or 1, 1, 1)               # without 'streams': one ordinary residual stream
    routed = 0
    for i in layer_order(cfg):
        layer, p = cfg["layers"][i], f"l{i}."
        for q in (1, 2):
            if q == 2 and layer.get("mlp") is None:
                continue
            h = rms_norm(xs[0] if S is None else hyper_read(xs, t[f"{p}hc{q}.in"]), t[f"{p}norm{q}"], eps)
            if q == 1:
                y = mixer(layer["type"], h, _sub(t, p + "mix."), layer["mixer"], eps)
            else:
                y, idx, margin = routed_ff(h, _sub(t, p + "mlp."), layer["mlp"], None if choices is None else choices[routed])
                routed += 1
                if margins is not None:
                    margins.append((idx, margin))
            xs = xs + y[None] if S is None else hyper_write(xs, y, t[f"{p}hc{q}.mix"], t[f"{p}hc{q}.out"])
        if layers_out is not None:
            layers_out.append(xs.sum(dim=0))
    return rms_norm(xs.sum(dim=0), t["final.norm"], eps) @ t["head"].T


def load(model_dir):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(model_dir, "model.safetensors"))
