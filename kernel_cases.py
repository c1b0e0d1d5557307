"""Runs ONE kernel at a named workload a few times: the small, self-contained cases that profiles/ are
captured from (`ncu ... python kernel_cases.py <case>`), each also timed with CUDA events.

Cases use the layer sizes of the TinyLlama-1.1B shape: hidden 2048, 32 heads / 4 kv heads of 64, feed-forward 5632.
"""
import sys
from types import SimpleNamespace

import torch

from forge_b200.kernels import (decode_attention_fused, gemm_sm100, gemm_sm100_qkv_rope, paged_attention, paged_attention_mma,
                                rope_table)

DEV = "cuda:0"
H, I, NH, NKV, HD, PS = 2048, 5632, 32, 4, 64, 16


def _bf16(*shape, scale=1.0):
    return (torch.randn(*shape, device=DEV) * scale).to(torch.bfloat16)


def _attention_inputs(reqs, NH=NH, NKV=NKV, HD=HD):
    """reqs: [(context_before, q_len)]; pages laid out in order."""
    pages = sum(-(-(c + q) // PS) for c, q in reqs)
    max_pages = max(-(-(c + q) // PS) for c, q in reqs)
    table = torch.zeros(len(reqs), max_pages, dtype=torch.int32)
    q_start, nxt = [0], 0
    for s, (c, q) in enumerate(reqs):
        n = -(-(c + q) // PS)
        table[s, :n] = torch.arange(nxt, nxt + n, dtype=torch.int32)
        nxt += n
        q_start.append(q_start[-1] + q)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    batch = SimpleNamespace(num_requests=len(reqs), host_q_start=q_start, host_context_before=[c for c, _ in reqs],
                            q_start=i32(q_start), context_before=i32([c for c, _ in reqs]), attention_plan={})
    return (_bf16(q_start[-1], NH * HD), _bf16(pages, 2, NKV, PS, HD), SimpleNamespace(block_table=table.to(DEV)), batch)


def case(name):
    if name == "gemm_decode_gateup":         # 8 tokens x [11264, 2048] weights, SwiGLU epilogue: 46 MB streamed
        x, w = _bf16(8, H), _bf16(2 * I, H, scale=0.02)
        return (lambda: gemm_sm100(x, w, epilogue="swiglu")), w.numel() * 2, 2 * 8 * w.numel()
    if name == "gemm_decode_down":           # 8 tokens x [2048, 5632], residual accumulate, K cut over a cluster
        x, w, r = _bf16(8, I), _bf16(H, I, scale=0.02), torch.zeros(8, H, device=DEV)
        return (lambda: gemm_sm100(x, w, accumulate_into=r)), w.numel() * 2, 2 * 8 * w.numel()
    if name == "gemm_decode_lmhead":         # 8 tokens x [32000, 2048]: 250 row tiles, dealt out evenly (stream-K)
        x, w = _bf16(8, H), _bf16(32000, H, scale=0.02)
        return (lambda: gemm_sm100(x, w)), w.numel() * 2, 2 * 8 * w.numel()
    if name == "gemm_prefill_qkv":           # 2048 tokens x [2560, 2048]: tiles of 128 x 160 fill two waves
        x, w = _bf16(2048, H), _bf16((NH + 2 * NKV) * HD, H, scale=0.02)
        return (lambda: gemm_sm100(x, w)), (x.numel() + w.numel()) * 2 + 2048 * w.shape[0] * 4, 2 * 2048 * w.numel()
    if name == "gemm_prefill_gateup":        # 2048 tokens x [11264, 2048], SwiGLU epilogue: 94.5 GFLOP
        x, w = _bf16(2048, H), _bf16(2 * I, H, scale=0.02)
        return (lambda: gemm_sm100(x, w, epilogue="swiglu")), (x.numel() + w.numel() + 2048 * I) * 2, 2 * 2048 * w.numel()
    if name == "gemm_prefill_down":          # 2048 tokens x [2048, 5632], residual accumulate: 47.2 GFLOP
        x, w, r = _bf16(2048, I), _bf16(H, I, scale=0.02), torch.zeros(2048, H, device=DEV)
        return (lambda: gemm_sm100(x, w, accumulate_into=r)), (x.numel() + w.numel()) * 2 + r.numel() * 8, 2 * 2048 * w.numel()
    if name == "attention_decode":           # 64 requests, 1024 cached tokens each, one new token: 67 MB of K/V
        q, kv, g, b = _attention_inputs([(1023, 1)] * 64)
        return (lambda: paged_attention_mma(q, kv, g, b, NH, NKV, HD, PS)), 64 * 1024 * 2 * NKV * HD * 2, 4 * 64 * 1024 * NH * HD
    if name == "attention_decode_fused":     # the same decode step as one kernel: rotary + cache write + attention
        q, kv, g, b = _attention_inputs([(1023, 1)] * 64)
        qkv = torch.randn(64, (NH + 2 * NKV) * HD, device=DEV)
        pos = torch.full((64,), 1023, dtype=torch.int32, device=DEV)
        slots = (g.block_table[:, 1023 // PS] * PS + 1023 % PS).to(torch.int32).contiguous()
        return (lambda: decode_attention_fused(qkv, kv, g.block_table, pos, slots, NH, NKV, HD, PS, 1e4)), \
            64 * 1024 * 2 * NKV * HD * 2, 4 * 64 * 1024 * NH * HD
    if name == "attention_decode_stream":    # 32 requests x 8192 cached tokens through the TMA ring: 268 MB of keys and values
        from forge_b200.kernels import decode_attention_stream
        ctx, S, ps = 8192, 32, 64
        pages_per = ctx // ps + 1
        table = torch.arange(S * pages_per, dtype=torch.int32, device=DEV).reshape(S, pages_per)
        kv = _bf16(S * pages_per, 2, NKV, ps, HD)
        qkv = torch.randn(S, (NH + 2 * NKV) * HD, device=DEV)
        pos = torch.full((S,), ctx, dtype=torch.int32, device=DEV)
        slots = (table[:, ctx // ps] * ps + ctx % ps).to(torch.int32)
        return (lambda: decode_attention_stream(qkv, kv, table, pos, slots, NH, NKV, HD, ps, 1e4, max_context=ctx + 1)), \
            S * ctx * 2 * NKV * HD * 2, 4 * S * ctx * NH * HD
    if name == "attention_prefill":          # one request, 2048 tokens, causal: 17.2 GFLOP
        q, kv, g, b = _attention_inputs([(0, 2048)])
        return (lambda: paged_attention(q, kv, g, b, NH, NKV, HD, PS)), 0, 2 * 2048 * 2048 * NH * HD
    if name == "attention_prefill_hd128":    # the Llama-3-8B heads: 32 / 8 kv heads of 128, one request of 2048 tokens: 34.4 GFLOP
        q, kv, g, b = _attention_inputs([(0, 2048)], 32, 8, 128)
        return (lambda: paged_attention(q, kv, g, b, 32, 8, 128, PS)), 0, 2 * 2048 * 2048 * 32 * 128
    if name == "attention_prefill_shared_keys":     # 256 new tokens on 20,000 cached: 16 tiles x 4 kv heads, each tile's keys shared out among 4 CTAs
        q, kv, g, b = _attention_inputs([(20000, 256)])
        return (lambda: paged_attention(q, kv, g, b, NH, NKV, HD, PS)), 20256 * 2 * NKV * HD * 2, 4 * 256 * 20128 * NH * HD
    if name == "gemm_prefill_qkv_rope":      # 2048 tokens x [2560, 2048]; the epilogue rotates q, k and writes q (bf16) and the cache
        x, w = _bf16(2048, H), _bf16((NH + 2 * NKV) * HD, H, scale=0.02)
        pos = torch.arange(2048, dtype=torch.int32, device=DEV)
        table, kv = rope_table(pos, HD, 1e4, by_pair=True), _bf16(2048 // PS, 2, NKV, PS, HD)
        return (lambda: gemm_sm100_qkv_rope(x, w, None, table, pos, kv, NH, NKV, HD, PS)), \
            (x.numel() + w.numel()) * 2 + 2048 * w.shape[0] * 2, 2 * 2048 * w.numel()
    if name == "attention_prefill_mma":      # the same through the mma.sync kernel, for comparison
        q, kv, g, b = _attention_inputs([(0, 2048)])
        return (lambda: paged_attention_mma(q, kv, g, b, NH, NKV, HD, PS)), 0, 2 * 2048 * 2048 * NH * HD
    if name in ("headmix_attention_prefill", "headmix_attention_decode"):
        # attention whose heads exchange weights: 32 / 4 kv heads of 64, window 1,024 + 4 kept first tokens, pages of 64;
        # one request of 2,048 tokens (12.9 GFLOP of Q K^T and P V for the visible pairs; the kernel executes 32.3: the value
        # product runs over all 4 kv heads' values), or 8 requests of one token on 1,023 cached
        from forge_b200.kernels import headmix_attention
        ps, window, keep = 64, 1024, 4
        reqs = [(0, 2048)] if name.endswith("prefill") else [(1023, 1)] * 8
        pages_per = [-(-(c + n) // ps) for c, n in reqs]
        table = torch.full((len(reqs), max(pages_per)), -1, dtype=torch.int32)
        q_start, nxt = [0], 0
        for s_, n in enumerate(pages_per):
            table[s_, :n] = torch.arange(nxt, nxt + n, dtype=torch.int32)
            nxt += n
            q_start.append(q_start[-1] + reqs[s_][1])
        T = q_start[-1]
        i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
        batch = SimpleNamespace(num_requests=len(reqs), num_tokens=T, host_q_start=q_start, attention_plan={},
                                tok_req=i32([s_ for s_, (c, n) in enumerate(reqs) for _ in range(n)]),
                                positions=i32([c + j for c, n in reqs for j in range(n)]))
        if name.endswith("decode"):
            batch.decode_only, batch.max_context = True, 1024
        g = SimpleNamespace(block_table=table.to(DEV))
        q, cache = _bf16(T, NH * HD), _bf16(nxt, 2, NKV, ps, HD)
        mix, gate = torch.eye(NH, device=DEV) + 0.1 * torch.randn(NH, NH, device=DEV), torch.rand(T, NH, device=DEV)
        pairs = sum(min(c + j + 1, window + keep) for c, n in reqs for j in range(n))
        return (lambda: headmix_attention(q, cache, g, batch, NH, NKV, HD, HD, ps, HD ** -0.5, window=window, keep_first=keep, mix=mix,
                                          gate=gate)), pairs * NKV * 2 * HD * 2 // max(1, T // len(reqs)), 2 * pairs * NH * 2 * HD
    if name in ("state_scan_wkv", "state_scan_delta"):
        # the recurrence of a state mixer alone: one request of 1,024 tokens, 32 heads of 64 channels (6 or 8 FLOPs per state
        # element and token), with the kernel that makes the decays in front of it
        from forge_b200.kernels import state_scan
        T, N, K = 1024, 32, 64
        mk = lambda: torch.randn(T, N * K, device=DEV) * 0.5
        r, k, v, x, y = mk(), mk(), mk(), mk(), mk()
        x0, y0 = x.clone(), y.clone()
        w0, u = torch.randn(N * K, device=DEV), torch.randn(N * K, device=DEV)
        state = torch.zeros(2, N * K * K, device=DEV)
        i32 = lambda z: torch.tensor(z, dtype=torch.int32, device=DEV)
        batch = SimpleNamespace(q_start=i32([0, T]), slots=i32([1]), num_requests=1)

        def run():
            x.copy_(x0)             # the scan overwrites x (and y) with the decays (and removal rates)
            y.copy_(y0)
            if name.endswith("delta"):
                state_scan("delta", (r, 0), (k, 0), (v, 0), (x, 0), w0, state, batch, N, K, y=(y, 0), a0=w0)
            else:
                state_scan("decay_bonus", (r, 0), (k, 0), (v, 0), (x, 0), w0, state, batch, N, K, bonus=u)
        return run, 4 * T * N * K * 4, (8 if name.endswith("delta") else 6) * T * N * K * K
    if name in ("scored_attention_prefill", "scored_attention_decode", "distance_attention_prefill"):
        # attention with shaped scores: differential (16 / 4 kv heads, two maps of 64 channels, values of 128) or with the
        # distance term (32 / 4 kv heads of 64); pages of 64; one request of 2,048 tokens, or 8 requests of one token on 1,023
        from forge_b200.kernels import scored_attention
        ps = 64
        Hh, G, M, D, E = (32, 4, 1, 64, 64) if name.startswith("distance") else (16, 4, 2, 64, 128)
        reqs = [(1023, 1)] * 8 if name.endswith("decode") else [(0, 2048)]
        pages_per = [-(-(c + n) // ps) for c, n in reqs]
        table = torch.full((len(reqs), max(pages_per)), -1, dtype=torch.int32)
        q_start, nxt = [0], 0
        for s_, n in enumerate(pages_per):
            table[s_, :n] = torch.arange(nxt, nxt + n, dtype=torch.int32)
            nxt += n
            q_start.append(q_start[-1] + reqs[s_][1])
        T = q_start[-1]
        i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
        batch = SimpleNamespace(num_requests=len(reqs), num_tokens=T, host_q_start=q_start, attention_plan={},
                                tok_req=i32([s_ for s_, (c, n) in enumerate(reqs) for _ in range(n)]),
                                positions=i32([c + j for c, n in reqs for j in range(n)]))
        if name.endswith("decode"):
            batch.decode_only, batch.max_context = True, 1024
        g = SimpleNamespace(block_table=table.to(DEV))
        q, cache = _bf16(T, Hh * M * D), _bf16(nxt, G * ps * (M * D + E))
        r1 = torch.rand(Hh, device=DEV) if M == 1 else None
        r2 = torch.rand(Hh, device=DEV) if M == 1 else None
        pairs = sum(c + j + 1 for c, n in reqs for j in range(n))
        return (lambda: scored_attention(q, cache, g, batch, Hh, G, M, D, E, ps, D ** -0.5, r1=r1, r2=r2, lam=0.7, post=0.4, eps=1e-5)), \
            pairs * G * (M * D + E) * 2 // max(1, T // len(reqs)), 2 * pairs * Hh * M * (D + E)
    if name == "state_scan_gated":
        # the gated-write recurrence alone: one request of 1,024 tokens, 32 heads of 64 key and 64 value channels (4 FLOPs per
        # state element and token), with the kernel that makes the gates in front of it
        from forge_b200.kernels import state_scan
        T, N, K = 1024, 32, 64
        mk = lambda: torch.randn(T, N * K, device=DEV) * 0.5
        r, v, x = mk(), mk(), mk()
        r0, x0 = r.clone(), x.clone()
        fb, low = torch.randn(N * K, device=DEV), torch.rand(N * K, device=DEV)
        state = torch.zeros(2, N * K * K, device=DEV)
        i32 = lambda z: torch.tensor(z, dtype=torch.int32, device=DEV)
        batch = SimpleNamespace(q_start=i32([0, T]), slots=i32([1]), num_requests=1)

        def run():
            r.copy_(r0)             # the scan overwrites r with silu(r) and x with the gates
            x.copy_(x0)
            state_scan("gated_write", (r, 0), None, (v, 0), (x, 0), fb, state, batch, N, K, a0=low, KV=K)
        return run, 3 * T * N * K * 4, 4 * T * N * K * K
    if name in ("latent_attention_prefill", "latent_attention_decode", "latent_attention_prefill_512"):
        # attention over latent rows: 32 heads whose absorbed queries (256 + 32 channels; 512 + 64 in the last case) read the same
        # rows; one prompt of 2,048 tokens, or 8 requests of 1,023 cached tokens and one new one.  FLOPs as executed: per visible
        # (token, row) pair and head 2 (C + R) for the score and 2 C for the weighted sum
        from forge_b200.kernels import latent_attention
        ps = 64
        Hh, C, R = (32, 512, 64) if name.endswith("512") else (32, 256, 32)
        reqs = [(1023, 1)] * 8 if name.endswith("decode") else [(0, 2048)]
        pages_per = [-(-(c + n) // ps) for c, n in reqs]
        table = torch.full((len(reqs), max(pages_per)), -1, dtype=torch.int32)
        q_start, nxt = [0], 0
        for s_, n in enumerate(pages_per):
            table[s_, :n] = torch.arange(nxt, nxt + n, dtype=torch.int32)
            nxt += n
            q_start.append(q_start[-1] + reqs[s_][1])
        T = q_start[-1]
        i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
        batch = SimpleNamespace(num_requests=len(reqs), num_tokens=T, host_q_start=q_start, attention_plan={},
                                tok_req=i32([s_ for s_, (c, n) in enumerate(reqs) for _ in range(n)]),
                                positions=i32([c + j for c, n in reqs for j in range(n)]))
        if name.endswith("decode"):
            batch.decode_only, batch.max_context = True, 1024
        g = SimpleNamespace(block_table=table.to(DEV))
        q, cache = _bf16(T, Hh * (C + R), scale=0.3), _bf16(nxt, ps * (C + R))
        pairs = sum(c + j + 1 for c, n in reqs for j in range(n))
        return (lambda: latent_attention(q, cache, g, batch, Hh, C, R, ps, (C + R) ** -0.5)), \
            pairs * (C + R) * 2 // max(1, T // len(reqs)), 2 * pairs * Hh * (2 * C + R)
    if name in ("windowed_attention_prefill", "chunked_attention_prefill", "windowed_attention_decode", "windowed_latent_prefill", "windowed_latent_decode"):
        # attention without rotation over a window of 1,024 positions (32 / 4 kv heads of 64), the same in chunks of 1,024 with scores
        # capped at 50, and attention over latent rows (32 heads, 256 + 32 channels) in a window of 1,024 with a sink per head: one
        # prompt of 4,096 tokens, or 8 requests of 2,047 cached tokens and one new one.  FLOPs as executed, visible pairs only
        from forge_b200.kernels import latent_attention, scored_attention
        ps, size = 64, 1024
        latent, chunked = "latent" in name, name.startswith("chunked")
        Hh, G, D, E, C, R = 32, 4, 64, 64, 256, 32
        reqs = [(2047, 1)] * 8 if name.endswith("decode") else [(0, 4096)]
        pages_per = [-(-(c + n) // ps) for c, n in reqs]
        table = torch.full((len(reqs), max(pages_per)), -1, dtype=torch.int32)
        q_start, nxt = [0], 0
        for s_, n in enumerate(pages_per):
            table[s_, :n] = torch.arange(nxt, nxt + n, dtype=torch.int32)
            nxt += n
            q_start.append(q_start[-1] + reqs[s_][1])
        T = q_start[-1]
        i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
        batch = SimpleNamespace(num_requests=len(reqs), num_tokens=T, host_q_start=q_start, attention_plan={},
                                tok_req=i32([s_ for s_, (c, n) in enumerate(reqs) for _ in range(n)]),
                                positions=i32([c + j for c, n in reqs for j in range(n)]))
        if name.endswith("decode"):
            batch.decode_only, batch.max_context = True, 2048
        g = SimpleNamespace(block_table=table.to(DEV))
        seen = lambda p: (p % size) + 1 if chunked else min(p + 1, size)
        pairs = sum(seen(c + j) for c, n in reqs for j in range(n))
        if latent:
            q, cache, sink = _bf16(T, Hh * (C + R), scale=0.3), _bf16(nxt, ps * (C + R)), torch.randn(Hh, device=DEV)
            return (lambda: latent_attention(q, cache, g, batch, Hh, C, R, ps, (C + R) ** -0.5, window=size, sink=sink)), \
                pairs * (C + R) * 2 // max(1, T // len(reqs)), 2 * pairs * Hh * (2 * C + R)
        q, cache = _bf16(T, Hh * D), _bf16(nxt, G * ps * (D + E))
        return (lambda: scored_attention(q, cache, g, batch, Hh, G, 1, D, E, ps, D ** -0.5, window=0 if chunked else size,
                                         chunk=size if chunked else 0, softcap=50.0 if chunked else 0.0)), \
            pairs * G * (D + E) * 2 // max(1, T // len(reqs)), 2 * pairs * Hh * (D + E)
    if name in ("streams_mix_prefill", "streams_mix_decode"):
        # a stream of four copies of 2,048 channels: a sublayer's write and the next sublayer's read and norm in one pass, for 4,096
        # tokens (the copies read and written once: 268 MB) or 8
        from forge_b200.kernels import streams_mix
        T, S, W_ = (4096 if name.endswith("prefill") else 8), 4, 2048
        xs, y = torch.randn(T, S * W_, device=DEV), torch.randn(T, W_, device=DEV)
        mix, ow, iw, wn = torch.eye(S, device=DEV), torch.ones(S, device=DEV) * 0.1, torch.ones(S, device=DEV) * 0.25, torch.ones(W_, device=DEV)
        return (lambda: streams_mix(xs, S, y=y, mix=mix, out_w=ow, in_next=iw, w_next=wn, eps=1e-5, out_dtype=torch.bfloat16)), \
            T * W_ * (2 * S * 4 + 4 + 2), 2 * T * W_ * S * (S + 2)
    if name == "routed_pairs_decode":
        # routed experts, one token: 2 of 8 experts of [7168 x 4096] gate, up and down matrices, each (token, expert) pair streaming
        # its expert's rows once (352 MB read, far more than L2 holds); router included
        from forge_b200.kernels import moe_pairs, moe_route
        W_, F_, E_, top = 4096, 7168, 8, 2
        x = _bf16(1, W_)
        router = torch.randn(E_, W_, device=DEV) * 0.02
        gate_up, down = _bf16(E_, 2 * F_, W_, scale=0.02), _bf16(E_, W_, F_, scale=0.02)

        def run():
            idx, wts = moe_route(x, router, top)
            moe_pairs(x, idx, wts, gate_up, down)
        return run, top * 3 * W_ * F_ * 2, top * 3 * W_ * F_ * 2
    if name == "retention_scan":
        # the retention recurrence alone: one request of 1,024 tokens, 32 heads of 64 key and 64 value channels (4 FLOPs per
        # state element and token), with the kernel that rotates q and k in front of it
        from forge_b200.kernels import retention_scan
        T, N, K = 1024, 32, 64
        mk = lambda: torch.randn(T, N * K, device=DEV) * 0.5
        qq, kk, v = mk(), mk(), mk()
        q0, k0 = qq.clone(), kk.clone()
        freq = torch.pow(torch.tensor(10000.0), -torch.arange(K // 2, dtype=torch.float32) * 2 / K).to(DEV)
        decay = torch.linspace(0.97, 0.999, N, device=DEV)
        state = torch.zeros(2, N * K * K, device=DEV)
        i32 = lambda z: torch.tensor(z, dtype=torch.int32, device=DEV)
        batch = SimpleNamespace(q_start=i32([0, T]), slots=i32([1]), num_requests=1, positions=torch.arange(T, dtype=torch.int32, device=DEV))

        def run():
            qq.copy_(q0)            # the scan rotates q and k in place
            kk.copy_(k0)
            retention_scan((qq, 0), (kk, 0), (v, 0), batch, freq, K ** -0.5, decay, state, N, K, K)
        return run, 3 * T * N * K * 4, 4 * T * N * K * K
    raise SystemExit(f"unknown case {name!r}; known: windowed_attention_prefill chunked_attention_prefill windowed_attention_decode windowed_latent_prefill windowed_latent_decode streams_mix_prefill streams_mix_decode routed_pairs_decode latent_attention_prefill latent_attention_prefill_512 latent_attention_decode retention_scan scored_attention_prefill scored_attention_decode distance_attention_prefill state_scan_gated headmix_attention_prefill headmix_attention_decode state_scan_wkv state_scan_delta "
                     "gemm_decode_gateup gemm_decode_down gemm_decode_lmhead gemm_prefill_qkv "
                     "gemm_prefill_gateup "
                     "gemm_prefill_qkv_rope gemm_prefill_down attention_decode attention_decode_fused attention_decode_stream attention_prefill "
                     "attention_prefill_hd128 attention_prefill_mma attention_prefill_shared_keys")


def main(argv):
    name = argv[1] if len(argv) > 1 else ""
    fn, nbytes, flops = case(name)
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(3):
        fn()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) / 3 * 1e3
    print(f"{name}: {us:.1f} us per launch (3 launches back to back, warm L2), "
          f"{nbytes / us / 1e3:.0f} GB/s of algorithmic bytes, {flops / us / 1e6:.1f} TFLOP/s")


if __name__ == "__main__":
    main(sys.argv)
