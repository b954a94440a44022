"""Timing of single kernels at the sizes of a model, for profiling.

    python -m rllm_b200.kernels.microbench attention_decode --batch 8 --context 4096
    python -m rllm_b200.kernels.microbench attention_prefill --tokens 2048 [--impl tcgen05]
    python -m rllm_b200.kernels.microbench gemm_small_m --rows 8 [--variant residual|rstd]
    python -m rllm_b200.kernels.microbench gemm_tcgen05 --rows 2048
    python -m rllm_b200.kernels.microbench latent_attention --tokens 2048 --heads 16 --kv-rank 512 --rot-dim 64
    python -m rllm_b200.kernels.microbench latent_attention --batch 8 --context 4096 --tokens 1 ...
    python -m rllm_b200.kernels.microbench routed_experts --rows 2048 --experts 32 --top 4 --intermediate 1024
    python -m rllm_b200.kernels.microbench lightning_scan --tokens 2048 --heads 16 --head-dim 128 --v-dim 128
    python -m rllm_b200.kernels.microbench selective_scan --tokens 2048 --channels 4096 --state 16
    python -m rllm_b200.kernels.microbench mlstm_scan --tokens 2048 --heads 8 --head-dim 128 --v-dim 256
    python -m rllm_b200.kernels.microbench streams --tokens 2048 --hidden 2048 --streams 4

Sizes default to the Llama-3.2-1B shape (32 heads, 8 kv heads, head 64, hidden
2048, intermediate 8192).  Times are CUDA-event times over ``--iters`` launches
after warm-up; inputs rotate over several buffers larger than L2 together, so
that weights and caches come from HBM as in a model step.  One line per case:
microseconds, and GB/s (memory-bound kernels) or TFLOP/s (products, attention
over prompts).
"""
from __future__ import annotations

import argparse
import math
import sys

import torch

from . import ops

DEV = "cuda:0"


def time_us(fn, iters: int, warmup: int = 3) -> float:
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / iters


def time_graph_us(fn, iters: int) -> float:
    """Back-to-back launches inside one CUDA graph: no host gaps between kernels."""
    for i in range(3):
        fn(i)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        with torch.cuda.graph(g):
            for i in range(iters):
                fn(i)
    torch.cuda.synchronize()
    g.replay()                      # the first replay also uploads the graph
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / iters


def _mask_options(args, rows: int, nq: int, d: int):
    """The attention kernels' options from the command line: (keyword arguments, a word for the report)."""
    kw = {}
    if args.keep_first:
        kw["keep_first"] = args.keep_first
    if args.chunk:
        kw["chunk"] = args.chunk
    if args.softcap:
        kw["softcap"] = args.softcap
    if args.sinks:
        kw["sinks"] = torch.randn(nq, device=DEV)
    if args.slopes:
        kw["slopes"] = torch.tensor([2.0 ** (-args.slopes * (h + 1) / nq) for h in range(nq)], device=DEV)
    if args.gate:
        kw["gate"] = torch.randn(rows, nq if args.gate == "head" else nq * d, device=DEV).bfloat16()
        kw["gate_per_head"] = args.gate == "head"
    return kw, (" with " + ", ".join(sorted(k for k in kw if k != "gate_per_head")) if kw else "")


def _seen(p: int, window: int, keep: int, chunk: int) -> int:
    """Keys that the query at position p sees."""
    lo = max(0, p - window + 1) if window else 0
    if chunk:
        lo = max(lo, p // chunk * chunk)
    return p + 1 - lo + (min(keep, lo) if window else 0)


def attention_decode(args) -> None:
    nq, nkv, d, page = args.heads, args.kv_heads, args.head_dim, args.page
    B, ctx = args.batch, args.context
    pages = B * (ctx // page) + 8
    nc = max(2, min(8, int(300e6 // (pages * nkv * page * d * 4)) + 1))
    caches = [(torch.randn(pages, nkv, page, d, device=DEV).bfloat16(),
               torch.randn(pages, nkv, page, d, device=DEV).bfloat16()) for _ in range(nc)]
    table = torch.randperm(pages - 8, device=DEV).int().view(B, ctx // page).contiguous()
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    q = torch.randn(B, nq * d, device=DEV).bfloat16()
    out = torch.empty_like(q)
    seq_lens = torch.full((B,), ctx, dtype=torch.int32, device=DEV)
    ws = torch.empty(ops.attention_decode_workspace(B, nq, d, ctx), device=DEV)
    scale = 1 / math.sqrt(d)

    kw, word = _mask_options(args, B, nq, d)

    def run(i):
        k, v = caches[i % nc]
        ops.attention_decode_bf16(q, nq * d, out, k, v, table, seq_lens, B, ctx, nq, nkv, d, args.window, scale, err, ws,
                                  **kw)
    us = time_graph_us(run, args.iters)
    nbytes = B * _seen(ctx - 1, args.window, args.keep_first, args.chunk) * nkv * d * 2 * 2
    print(f"attention_decode batch {B} context {ctx} window {args.window}{word}: {us:.1f} us, "
          f"{nbytes / us / 1e3:.0f} GB/s of visible K and V")


def attention_prefill(args) -> None:
    nq, nkv, d, page = args.heads, args.kv_heads, args.head_dim, args.page
    T = args.tokens
    pages = T // page + 8
    k = torch.randn(pages, nkv, page, d, device=DEV).bfloat16()
    v = torch.randn(pages, nkv, page, d, device=DEV).bfloat16()
    table = torch.randperm(pages - 8, device=DEV).int().view(1, T // page).contiguous()
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    q = torch.randn(T, nq * d, device=DEV).bfloat16()
    out = torch.empty_like(q)
    seq_lens = torch.tensor([T], dtype=torch.int32, device=DEV)
    q_start = torch.tensor([0, T], dtype=torch.int32, device=DEV)
    scale = 1 / math.sqrt(d)

    fn = ops.attention_prefill_tcgen05 if args.impl == "tcgen05" else ops.attention_prefill_bf16
    kw, word = _mask_options(args, T, nq, d)

    def run(i):
        fn(q, nq * d, out, k, v, table, q_start, seq_lens, 0, 1, T, nq, nkv, d, args.window, scale, err, **kw)
    us = time_us(run, args.iters)
    flops = 4 * d * nq * sum(_seen(p, args.window, args.keep_first, args.chunk) for p in range(T))
    print(f"attention_prefill ({args.impl}) tokens {T} window {args.window}{word}: {us:.1f} us, "
          f"{flops / us / 1e6:.0f} TFLOP/s (visible pairs)")
    if int(err.item()):
        print(f"error word {int(err.item())}", file=sys.stderr)


def latent_attention(args) -> None:
    """--tokens > 1: one prompt of that many tokens; --tokens 1: --batch sequences of --context cached rows."""
    heads, dv, dk, page = args.heads, args.kv_rank, args.kv_rank + args.rot_dim, args.page
    if args.tokens > 1:
        S, nq, ctx = 1, args.tokens, args.tokens
    else:
        S, nq, ctx = args.batch, 1, args.context
    per = -(-ctx // page)
    cache = torch.randn(S * per + 4, 1, page, dk, device=DEV).bfloat16()
    table = torch.randperm(S * per, device=DEV).int().view(S, per).contiguous()
    T = S * nq
    q = torch.randn(T, heads * dk, device=DEV).bfloat16()
    out = torch.empty(T, heads * dv, device=DEV, dtype=torch.bfloat16)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    q_start = torch.arange(0, T + 1, nq, dtype=torch.int32, device=DEV)
    seq_lens = torch.full((S,), ctx, dtype=torch.int32, device=DEV)
    scale = 1 / math.sqrt(dk)

    def run(i):
        ops.latent_attention_mma(q, out, cache, table, q_start, seq_lens, S, nq, heads, dk, dv, args.window, scale, None,
                                 err, max_seq_len=ctx)
    us = time_us(run, args.iters)
    vis = sum(min(p + 1, args.window or p + 1) for p in range(ctx - nq, ctx)) * S
    flops = 2 * (dk + dv) * heads * vis
    gb = 2 * S * min(ctx, (args.window or ctx) + nq) * dk / 1e9
    print(f"latent_attention tokens {T} context {ctx} heads {heads} rows of {dk} (values {dv}): {us:.1f} us, "
          f"{flops / us / 1e6:.1f} TFLOP/s, rows read once {gb / us * 1e6:.0f} GB/s")
    if int(err.item()):
        print(f"error word {int(err.item())}", file=sys.stderr)


def routed_experts(args) -> None:
    T, H, F, E, top = args.rows, args.hidden, args.intermediate, args.experts, args.top
    x = torch.randn(T, H, device=DEV).bfloat16()
    wgu = (torch.randn(E, 2 * F, H, device=DEV) * 0.02).bfloat16()
    wd = (torch.randn(E, H, F, device=DEV) * 0.02).bfloat16()
    ids = torch.stack([torch.randperm(E, device=DEV)[:top] for _ in range(T)]).int().contiguous()

    def run(i):
        ops.moe_experts(x, ids, wgu, wd, 7.0, 1.702)
    us = time_us(run, args.iters)
    used = min(E, T * top)
    print(f"routed_experts rows {T} x top {top} of {E} experts ({H} -> {F} -> {H}): {us:.1f} us, "
          f"{2 * 3 * H * F * T * top / us / 1e6:.1f} TFLOP/s, touched weights once {used * 3 * H * F * 2 / us / 1e3:.0f} GB/s")


def _shapes(args):
    H, I = args.hidden, args.intermediate
    qkv = (args.heads + 2 * args.kv_heads) * args.head_dim
    return [("qkv", qkv, H), ("o_proj", H, args.heads * args.head_dim), ("gate_up", 2 * I, H), ("down", H, I)]


def gemm_small_m(args) -> None:
    """--variant plain: the four projections.  residual: o and down adding into a float32 stream and
    preparing the next norm.  rstd: qkv and gate_up applying the norm's row factors."""
    M = args.rows
    for name, N, K in _shapes(args):
        silu = name == "gate_up"
        if args.only and name != args.only:
            continue
        if args.variant == "residual" and name not in ("o_proj", "down"):
            continue
        if args.variant == "rstd" and name not in ("qkv", "gate_up"):
            continue
        nw = max(2, int(300e6 // (N * K * 2)) + 1)
        ws = [(torch.randn(N, K, device=DEV) * 0.02).bfloat16() for _ in range(nw)]
        x = torch.randn(M, K, device=DEV).bfloat16()
        out = torch.empty(M, N // 2 if silu else N, device=DEV, dtype=torch.bfloat16)
        h = torch.randn(M, N, device=DEV)
        wn = torch.ones(N, device=DEV)
        parts = torch.ones(128, M, device=DEV)

        def run(i):
            if args.variant == "residual":
                ops.gemm_small_m_residual(x, ws[i % nw], h, wn)
            elif args.variant == "rstd":
                ops.gemm_small_m_rstd(x, parts, 1e-5, ws[i % nw], out, "silu_mul" if silu else "store")
            else:
                ops.gemm_small_m(x, ws[i % nw], out, "silu_mul" if silu else "store")
        us = time_graph_us(run, args.iters)
        print(f"gemm_small_m ({args.variant}) rows {M} {name}{' +silu' if silu else ''} [{N} x {K}]: {us:.1f} us, "
              f"{N * K * 2 / us / 1e3:.0f} GB/s of weight")


def gemm_tcgen05(args) -> None:
    M = args.rows
    for name, N, K in _shapes(args):
        if args.only and name != args.only:
            continue
        w = (torch.randn(N, K, device=DEV) * 0.02).bfloat16()
        x = torch.randn(M, K, device=DEV).bfloat16()
        silu = name == "gate_up"
        out = torch.empty(M, N // 2 if silu else N, device=DEV, dtype=torch.bfloat16)

        def run(i):
            ops.gemm_tcgen05(x, w, out, "silu_mul" if silu else "store")
        us = time_us(run, args.iters)
        print(f"gemm_tcgen05 rows {M} {name}{' +silu' if silu else ''} [{N} x {K}]: {us:.1f} us, "
              f"{2 * M * N * K / us / 1e6:.0f} TFLOP/s")
    ops.check_gemm_errors(torch.device(DEV))


def _one_sequence(T, batch):
    """(q_start, token_seq, slots, number of sequences, longest): one portion of T tokens, or ``batch``
    sequences of one token each when T == 1."""
    S = batch if T == 1 else 1
    per = 1 if T == 1 else T
    q_start = torch.arange(0, S * per + 1, per, dtype=torch.int32, device=DEV)
    token_seq = torch.arange(S, dtype=torch.int32, device=DEV).repeat_interleave(per)
    return q_start, token_seq, torch.arange(S, dtype=torch.int32, device=DEV), S, per


def lightning_scan(args) -> None:
    """The lightning-attention recurrence over one prompt portion, or one token of ``--batch`` sequences."""
    heads, d, dv = args.heads, args.head_dim, args.v_dim or args.head_dim
    q_start, _, slots, S, per = _one_sequence(args.tokens, args.batch)
    T, qk = S * per, heads * d
    bufs = [torch.randn(T, 2 * qk + 2 * heads * dv, device=DEV).bfloat16() for _ in range(4)]
    decay = torch.linspace(0.9, 0.999, heads, device=DEV)
    state = torch.zeros(S, heads, d, dv, device=DEV)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)

    def run(i):
        a = bufs[i % 4]
        ops.lightning_scan(a[:, :qk], a[:, qk:2 * qk], a[:, 2 * qk:2 * qk + heads * dv], decay, state, q_start, slots,
                           S, err, max_q_len=per)
    us = time_us(run, args.iters)
    moved = T * heads * (4 * d + 6 * dv) + 8 * S * heads * d * dv
    print(f"lightning_scan tokens {T} ({S} sequences) heads {heads} x {d} x {dv}: {us:.1f} us, {moved / us / 1e3:.0f} GB/s "
          f"of rows and state, {4.0 * T * heads * d * dv / us / 1e6:.2f} TFLOP/s float32")


def mlstm_scan(args) -> None:
    """The matrix memory's recurrence over one prompt portion, or one token of ``--batch`` sequences."""
    heads, d, dv = args.heads, args.head_dim, args.v_dim or args.head_dim
    q_start, _, slots, S, per = _one_sequence(args.tokens, args.batch)
    T, qk = S * per, heads * d
    bufs = [torch.randn(T, 2 * qk + 2 * heads * dv, device=DEV).bfloat16() for _ in range(4)]
    pre = torch.randn(T, 2 * heads, device=DEV) * 2
    gates = torch.empty_like(pre)
    bias = torch.zeros(heads, device=DEV)
    state = torch.zeros(S, heads, ops.mlstm_state_size(d, dv), device=DEV)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)

    def run(i):
        a = bufs[i % 4]
        gates.copy_(pre)                 # (the call turns the pre-activations into log gates in place)
        ops.mlstm_scan(a[:, :qk], a[:, qk:2 * qk], a[:, 2 * qk:2 * qk + heads * dv], gates, bias, bias, 10.0, d ** -0.5,
                       state, q_start, slots, S, heads, d, dv, err, q_lens=[per] * S)
    us = time_us(run, args.iters)
    moved = T * heads * (4 * d + 6 * dv) + 8 * S * heads * d * dv
    print(f"mlstm_scan tokens {T} ({S} sequences) heads {heads} x {d} x {dv}: {us:.1f} us (with a copy of the gates), "
          f"{moved / us / 1e3:.0f} GB/s of rows and state, {4.0 * T * heads * d * dv / us / 1e6:.2f} TFLOP/s float32")


def selective_scan(args) -> None:
    """The convolution and the selective recurrence over one prompt portion, or one token of ``--batch`` sequences."""
    E, N, R = args.channels, args.state, max(1, args.channels // 32)
    q_start, token_seq, slots, S, per = _one_sequence(args.tokens, args.batch)
    T = S * per
    xz = [torch.randn(T, 2 * E, device=DEV).bfloat16() for _ in range(4)]
    proj = torch.randn(T, R + 2 * N, device=DEV).bfloat16()
    dt_raw = torch.randn(T, E, device=DEV)
    small = lambda *shape: torch.randn(*shape, device=DEV).bfloat16()
    w_conv, b_conv, dt_b, a_log, dskip = small(E, 4), small(E), small(E), small(E, N), small(E)
    state, tail = torch.zeros(S, N, E, device=DEV), torch.zeros(S, 3, E, device=DEV)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    keep = {}

    def conv(i):
        keep["c"] = ops.causal_conv(xz[i % 4][:, :E], w_conv, b_conv, tail, q_start, token_seq, slots, S, per > 1, err)

    def scan(i):
        ops.selective_scan(keep["c"], dt_raw, dt_b, proj, R, R + N, a_log, dskip, xz[i % 4][:, E:], state, q_start, slots,
                           S, err, max_q_len=per)
    us = time_us(conv, args.iters)
    print(f"causal_conv tokens {T} channels {E} taps 4: {us:.1f} us, {4.0 * T * E / us / 1e3:.0f} GB/s")
    us = time_us(scan, args.iters)
    print(f"selective_scan tokens {T} ({S} sequences) channels {E} states {N}: {us:.1f} us, "
          f"{(10.0 * T * E + 8.0 * S * N * E) / us / 1e3:.0f} GB/s of rows and state")


def streams(args) -> None:
    """The write-back into all residual streams with the next read and its norm."""
    S, T, H = args.streams, args.tokens, args.hidden
    xs = [torch.randn(S, T, H, device=DEV) for _ in range(3)]
    y = torch.randn(T, H, device=DEV).bfloat16()
    vec = lambda n: torch.randn(n, device=DEV)
    mix, write, read, scale = torch.randn(S, S, device=DEV), vec(S), vec(S), vec(H).bfloat16()
    norm = (torch.tensor([0.5], device=DEV), vec(H).bfloat16(), vec(H).bfloat16())

    def run(i):
        ops.streams_write(xs[i % 3], y, scale, mix, write, next_read=read, norm=norm)
    us = time_us(run, args.iters)
    print(f"streams_write {S} streams x {T} x {H}: {us:.1f} us, {(8.0 * S + 4.0) * T * H / us / 1e3:.0f} GB/s")


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="python -m rllm_b200.kernels.microbench", description=__doc__.split("\n\n")[0])
    p.add_argument("kernel", choices=["attention_decode", "attention_prefill", "gemm_small_m", "gemm_tcgen05",
                                      "latent_attention", "routed_experts", "lightning_scan", "selective_scan",
                                      "streams", "mlstm_scan"])
    p.add_argument("--batch", type=int, default=8)
    p.add_argument("--context", type=int, default=4096)
    p.add_argument("--tokens", type=int, default=2048)
    p.add_argument("--rows", type=int, default=8)
    p.add_argument("--iters", type=int, default=20)
    p.add_argument("--heads", type=int, default=32)
    p.add_argument("--kv-heads", type=int, default=8)
    p.add_argument("--head-dim", type=int, default=64)
    p.add_argument("--hidden", type=int, default=2048)
    p.add_argument("--intermediate", type=int, default=8192)
    p.add_argument("--page", type=int, default=16)
    p.add_argument("--kv-rank", type=int, default=512, help="latent_attention: values of a cached row")
    p.add_argument("--rot-dim", type=int, default=64, help="latent_attention: the rows' rotated key part")
    p.add_argument("--window", type=int, default=0, help="the attention kernels: keys a query sees (0: all)")
    p.add_argument("--keep-first", type=int, default=0, help="attention_*: with a window, first keys that stay visible")
    p.add_argument("--chunk", type=int, default=0, help="attention_*: a query sees the keys of its own chunk")
    p.add_argument("--softcap", type=float, default=0.0, help="attention_*: the tanh cap of the scaled scores")
    p.add_argument("--sinks", action="store_true", help="attention_*: one more term a head in the denominator")
    p.add_argument("--slopes", type=float, default=0.0,
                   help="attention_*: a distance bias with the slopes 2^(-x (h + 1) / heads) (0: none)")
    p.add_argument("--gate", choices=["head", "element"], default=None, help="attention_*: a sigmoid gate on the result")
    p.add_argument("--v-dim", type=int, default=0, help="lightning_scan: a value head's size (0: --head-dim)")
    p.add_argument("--channels", type=int, default=4096, help="selective_scan: inner channels")
    p.add_argument("--state", type=int, default=16, help="selective_scan: states a channel")
    p.add_argument("--streams", type=int, default=4, help="streams: residual streams")
    p.add_argument("--experts", type=int, default=32)
    p.add_argument("--top", type=int, default=4)
    p.add_argument("--variant", choices=["plain", "residual", "rstd"], default="plain",
                   help="gemm_small_m: which epilogue / operand form")
    p.add_argument("--only", choices=["qkv", "o_proj", "gate_up", "down"], default=None,
                   help="gemm_small_m, gemm_tcgen05: this projection alone")
    p.add_argument("--impl", choices=["mma", "tcgen05"], default="mma",
                   help="attention_prefill: the mma.sync kernel or the tcgen05 kernel")
    args = p.parse_args(argv)
    if not torch.cuda.is_available():
        print("microbench needs a CUDA device", file=sys.stderr)
        return 1
    {"attention_decode": attention_decode, "attention_prefill": attention_prefill,
     "gemm_small_m": gemm_small_m, "gemm_tcgen05": gemm_tcgen05, "latent_attention": latent_attention,
     "routed_experts": routed_experts, "lightning_scan": lightning_scan, "selective_scan": selective_scan,
     "streams": streams, "mlstm_scan": mlstm_scan}[args.kernel](args)
    return 0


if __name__ == "__main__":
    sys.exit(main())
