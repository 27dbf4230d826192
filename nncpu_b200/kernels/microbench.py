"""Single kernels at chosen sizes, timed on the device: the library's
counterpart of the reference's ignored micro-benchmarks
(crates/nncpu/src/kernels/tests.rs:1295-1482), which print streaming GB/s and
GFLOP/s for its row kernels and one attention block.

    python -m nncpu_b200.kernels.microbench linear M N K [--epilogue swiglu] [--accumulate] [--norm producer|consumer]
    python -m nncpu_b200.kernels.microbench linear-qkv TOKENS [--hidden K]
    python -m nncpu_b200.kernels.microbench attention-decode BATCH CONTEXT [--splits S] [--cluster] [--from-projections]
    python -m nncpu_b200.kernels.microbench attention-prefill BATCH TOKENS
    python -m nncpu_b200.kernels.microbench rmsnorm ROWS DIM

Timing: the kernel is captured in a CUDA graph over enough different buffers
that no launch finds its operands in L2, replayed, and timed with CUDA events.
``--once`` runs three plain launches instead (for a profiler).  Shapes default
to heads 32 / kv heads 8 / head size 128 for attention.
"""
from __future__ import annotations

import argparse
import math
import sys

import torch

from . import ops

DEV = "cuda:0"
L2_BYTES = 126 << 20


def _time(fns, once: bool) -> float:
    """Milliseconds per call of the functions in ``fns`` (each a different buffer set)."""
    for f in fns:
        f()
    torch.cuda.synchronize()
    if once:
        for f in fns[:3]:
            f()
        torch.cuda.synchronize()
        return float("nan")
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for f in fns:
            f()
    g.replay()
    torch.cuda.synchronize()
    best = None
    for _ in range(5):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        g.replay()
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / len(fns)
        best = ms if best is None else min(best, ms)
    return best


def linear(args) -> None:
    m, n, k = args.m, args.n, args.k
    copies = max(2, 4 * L2_BYTES // (n * k * 2) + 1)
    # weights of the size that models have (N(0, 0.02)): with unit weights the products reach the hundreds, and the
    # gated epilogue's exponential and division leave their fast paths, which no model's activations do
    ws = [(torch.randn(n, k, device=DEV) * 0.02).bfloat16() for _ in range(copies)]
    x = torch.randn(m, k, device=DEV).bfloat16()
    n_out = n // 2 if args.epilogue == "swiglu" else n
    out = torch.zeros(m, n_out, device=DEV, dtype=torch.float32 if args.accumulate else torch.bfloat16)
    work = ops.GemmWorkspace(DEV)

    # the norms around the product riding on it: as the norm's producer it also leaves out * gamma and the rows' sums
    # of squares, as its consumer it applies the rows' scales (few tokens, or 512 and more)
    few = m <= ops.SKINNY_MAX_TOKENS and not args.tensor_cores
    ops.linear_skinny_force_warps(args.warps)
    rows = ops.SKINNY_MAX_TOKENS if few else m
    norm_out = norm_in = None
    if args.norm == "producer":
        gamma = torch.ones(n, device=DEV).bfloat16()
        bins = torch.zeros(2, rows, ops.NORM_ROW_WORDS, dtype=torch.int64, device=DEV)
        xg = torch.empty(m, n, device=DEV).bfloat16()
        norm_out = (xg, gamma, bins[0].view(-1) if few else bins[0], bins[1].view(-1) if few else bins[1])
    elif args.norm == "consumer":
        bins = torch.zeros(rows, ops.NORM_ROW_WORDS, dtype=torch.int64, device=DEV)
        bins[:, 5] = max(1, k // 1024)  # a sum of squares of k in every row (bin 5 counts units of 2^10): scales near 1,
        #                                 as a model's are (large ones push the gated epilogue off its fast paths)
        norm_in = (bins.view(-1) if few else bins, 1e-6)

    def call(w):
        if few:
            ops.linear_skinny(x, w, None, out, args.accumulate, args.epilogue, norm_out, norm_in)
        else:
            ops.linear_tc(x, w, None, out, work, args.accumulate, args.epilogue, plan=args.plan, norm_out=norm_out,
                          norm_in=norm_in)
    ms = _time([lambda w=w: call(w) for w in ws], args.once)
    print(f"linear M={m} N={n} K={k} epilogue={args.epilogue}{' norm ' + args.norm if args.norm else ''}: {ms * 1e3:.1f} us, "
          f"{n * k * 2 / ms / 1e6:.0f} GB/s of weights, {2 * m * n * k / ms / 1e9:.1f} TFLOP/s")


def linear_qkv(args) -> None:
    """The q/k/v projection of one prompt with norm, rotation and cache append in its epilogue."""
    m, k, nh, nkv, hd = args.tokens, args.hidden, args.heads, args.kv_heads, args.head_dim
    n = (nh + 2 * nkv) * hd
    copies = max(2, 4 * L2_BYTES // (n * k * 2) + 1)
    ws = [(torch.randn(n, k, device=DEV) / math.sqrt(k)).bfloat16() for _ in range(copies)]
    x = torch.randn(m, k, device=DEV).bfloat16()
    gamma = torch.ones(hd, device=DEV).bfloat16()
    seq = torch.zeros(m, dtype=torch.int32, device=DEV)
    pos = torch.arange(m, dtype=torch.int32, device=DEV)
    pages = (m + 63) // 64
    table = torch.randperm(pages, device=DEV).to(torch.int32).view(1, -1)
    kp = torch.zeros(pages, nkv, 64, hd, device=DEV).bfloat16()
    vp = torch.zeros_like(kp)
    inv = torch.pow(torch.tensor(1e6, dtype=torch.float64), -2.0 * torch.arange(hd // 2, dtype=torch.float64) / hd)
    cs = torch.empty(hd // 2, m, 2, device=DEV)
    ops.rope_table(pos, inv.float().to(DEV), cs, by_pair=True)
    q = torch.empty(m, nh * hd, device=DEV).bfloat16()
    work = ops.GemmWorkspace(DEV)
    ms = _time([lambda w=w: ops.linear_tc_qkv(x, w, gamma, gamma, 1e-6, cs, seq, pos, table, kp, vp, q, work, nh, nkv, hd)
                for w in ws], args.once)
    if int(work.status.item()):
        raise SystemExit(f"the kernel gave up waiting (status {int(work.status.item())})")
    print(f"linear-qkv M={m} N={n} K={k}: {ms * 1e3:.1f} us, {2 * m * n * k / ms / 1e9:.1f} TFLOP/s")


def _cache(batch, ctx, nkv, hd, copies):
    pages = batch * ((ctx + 63) // 64)
    sets = [(torch.randn(pages, nkv, 64, hd, device=DEV).bfloat16(), torch.randn(pages, nkv, 64, hd, device=DEV).bfloat16())
            for _ in range(copies)]
    table = torch.randperm(pages, device=DEV).to(torch.int32).view(batch, -1)
    return sets, table


def attention_decode(args) -> None:
    nh, nkv, hd, b, ctx = args.heads, args.kv_heads, args.head_dim, args.batch, args.context
    kv_bytes = b * ctx * nkv * hd * 2 * 2
    sets, table = _cache(b, ctx, nkv, hd, max(2, 4 * L2_BYTES // kv_bytes + 1))
    seq = torch.arange(b, dtype=torch.int32, device=DEV)
    pos = torch.full((b,), ctx - 1, dtype=torch.int32, device=DEV)
    q = torch.randn(b, nh * hd, device=DEV).bfloat16()
    out = torch.empty_like(q)
    splits = args.splits or max(1, min(296 // (b * nkv), ctx // 256))
    floats = 0 if args.cluster else ops.attention_decode_scratch_floats(b, nh, nkv, hd, splits)
    scratch = torch.empty(floats, device=DEV) if floats else None
    if args.from_projections:
        # as a decode step runs it: from the float32 q/k/v projections, with per-head norm, rotation and cache append
        qkv = torch.randn(b, (nh + 2 * nkv) * hd, device=DEV)
        gamma = torch.ones(hd, device=DEV).bfloat16()
        inv = torch.pow(torch.tensor(1e6, dtype=torch.float64), -2.0 * torch.arange(hd // 2, dtype=torch.float64) / hd)
        cs = torch.empty(b, hd // 2, 2, device=DEV)
        ops.rope_table(pos, inv.float().to(DEV), cs)
        run = lambda kp, vp: ops.attention_decode_mma_from_qkv(qkv, gamma, gamma, 1e-6, cs, kp, vp, True, table, seq, pos, out,
                                                               scratch, nh, nkv, hd, 1 / math.sqrt(hd), 0, splits)
    else:
        run = lambda kp, vp: ops.attention_decode_mma(q, kp, vp, table, seq, pos, out, scratch, nh, nkv, hd,
                                                      1 / math.sqrt(hd), 0, splits)
    ms = _time([lambda kp=kp, vp=vp: run(kp, vp) for kp, vp in sets], args.once)
    print(f"attention-decode batch={b} context={ctx} splits={splits}{' from projections' if args.from_projections else ''}: "
          f"{ms * 1e3:.1f} us, {kv_bytes / ms / 1e6:.0f} GB/s of cache")


def attention_prefill(args) -> None:
    nh, nkv, hd, b, t = args.heads, args.kv_heads, args.head_dim, args.batch, args.tokens
    sets, table = _cache(b, t, nkv, hd, 1)
    kp, vp = sets[0]
    pos = torch.arange(t, dtype=torch.int32, device=DEV).repeat(b)
    cu = torch.arange(b + 1, dtype=torch.int32, device=DEV) * t
    q = torch.randn(b * t, nh * hd, device=DEV).bfloat16()
    out = torch.empty_like(q)
    if args.legacy:
        run = lambda: ops.attention_prefill_mma(q, kp, vp, table, cu, pos, out, b, nh, nkv, hd, 1 / math.sqrt(hd), 0)
    else:
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        run = lambda: ops.attention_prefill_tc(q, kp, vp, table, cu, pos, out, status, b, nh, nkv, hd,
                                               1 / math.sqrt(hd), 0)
    ms = _time([run] * 3, args.once)
    if not args.legacy and int(status.item()):
        raise SystemExit(f"the kernel gave up waiting (status {int(status.item())})")
    flops = 4.0 * nh * hd * b * t * (t + 1) / 2
    print(f"attention-prefill batch={b} tokens={t}: {ms * 1e3:.1f} us, {flops / ms / 1e9:.0f} TFLOP/s (causal)")


def rmsnorm(args) -> None:
    rows, dim = args.rows, args.dim
    copies = max(2, 4 * L2_BYTES // (rows * dim * 4) + 1)
    xs = [torch.randn(rows, dim, device=DEV) for _ in range(min(copies, 64))]
    gamma = torch.ones(dim, device=DEV).bfloat16()
    out = torch.empty(rows, dim, device=DEV, dtype=torch.bfloat16)
    ms = _time([lambda x=x: ops.rmsnorm(x, gamma, 1e-6, out) for x in xs], args.once)
    print(f"rmsnorm rows={rows} dim={dim}: {ms * 1e3:.1f} us, {rows * dim * 6 / ms / 1e6:.0f} GB/s")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--once", action="store_true", help="three plain launches, no timing (for a profiler)")
    ap.add_argument("--no-overlap", action="store_true",
                    help="every kernel waits for the end of the one before it (no programmatic dependent launch)")
    sub = ap.add_subparsers(dest="kernel", required=True)
    p = sub.add_parser("linear")
    p.add_argument("m", type=int); p.add_argument("n", type=int); p.add_argument("k", type=int)
    p.add_argument("--epilogue", default="plain", choices=["plain", "swiglu"])
    p.add_argument("--accumulate", action="store_true")
    p.add_argument("--tensor-cores", action="store_true", help="up to 16 tokens too on the tcgen05 kernels")
    p.add_argument("--plan", default="auto", choices=sorted(ops.PLANS), help="another tcgen05 kernel than the sizes' own")
    p.add_argument("--warps", type=int, default=0, choices=[0, 4, 8],
                   help="few tokens: blocks of 8 or of 4 warps (0: chosen by the sizes)")
    p.add_argument("--norm", choices=["producer", "consumer"],
                   help="the product also carries the norm after it (with --accumulate) or the norm before it")
    p.set_defaults(fn=linear)
    for name, fn, a, b in (("attention-decode", attention_decode, "batch", "context"),
                           ("attention-prefill", attention_prefill, "batch", "tokens")):
        p = sub.add_parser(name)
        p.add_argument(a, type=int); p.add_argument(b, type=int)
        p.add_argument("--heads", type=int, default=32); p.add_argument("--kv-heads", type=int, default=8)
        p.add_argument("--head-dim", type=int, default=128); p.add_argument("--splits", type=int, default=0)
        p.add_argument("--cluster", action="store_true", help="merge the splits inside a cluster (at most 8)")
        p.add_argument("--legacy", action="store_true", help="prefill: the mma.sync kernel instead of tcgen05")
        p.add_argument("--from-projections", action="store_true",
                       help="decode: start from the float32 q/k/v projections (norm, rotation, append inside), as a step does")
        p.set_defaults(fn=fn)
    p = sub.add_parser("linear-qkv")
    p.add_argument("tokens", type=int); p.add_argument("--hidden", type=int, default=4096)
    p.add_argument("--heads", type=int, default=32); p.add_argument("--kv-heads", type=int, default=8)
    p.add_argument("--head-dim", type=int, default=128)
    p.set_defaults(fn=linear_qkv)
    p = sub.add_parser("rmsnorm")
    p.add_argument("rows", type=int); p.add_argument("dim", type=int)
    p.set_defaults(fn=rmsnorm)
    args = ap.parse_args(argv)
    if args.no_overlap:
        ops.launch_overlap(False)
    args.fn(args)
    return 0


if __name__ == "__main__":
    sys.exit(main())
