"""Micro-benchmarks of the hand-written kernels on the shapes of the headline configuration.

    python benchmark/kernel_bench.py gemm      [--m 65536 --n 512 --k 128] [--bias] [--ref]
    python benchmark/kernel_bench.py attention [--b 128 --h 8 --len 256] [--backward]
    python benchmark/kernel_bench.py layernorm [--rows 65536 --c 128] [--backward]
    python benchmark/kernel_bench.py global_attention [--b 256 --len 5120 --h 8]
    python benchmark/kernel_bench.py global_attention_bwd [--b 256 --len 5120 --h 8]
    python benchmark/kernel_bench.py ipa       [--len 1024]
    python benchmark/kernel_bench.py floor     (per-launch floor of small dependent kernels inside a CUDA graph)
    python benchmark/kernel_bench.py all

Every timing is taken on the device: the op is captured ``--iters`` times in a CUDA graph, each instance preceded
by a write of a buffer larger than the L2 cache, and the time of the flush-only graph is subtracted, so the figure
is a cold-cache kernel time without host launch overhead.  ``--plain`` skips graphs and flushes and just launches
the op a few times (the form to put under a profiler).  Roofline fractions are printed against the measured peaks in
``MEASURED_PEAKS.json`` at the repository root when that file exists.
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from fastfold_b200 import ops as K  # noqa: E402
from fastfold_b200.ops import flash  # noqa: E402

DEV = "cuda"


def _peaks():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return d.get("hbm_gbs", 6650.0) * 1e9, d.get("bf16_tflops", 1590.0) * 1e12, "of measured"
    return 6650e9, 1590e12, "of fallback"


def _graph_time(fn, iters, reps=3):
    fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        fn()
        with torch.cuda.graph(g, stream=s):
            for _ in range(iters):
                fn()
    torch.cuda.synchronize()
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (iters * reps)          # us


class Timer:
    def __init__(self, iters, plain):
        self.iters, self.plain = iters, plain
        self.flush = None if plain else torch.empty(192 << 20, device=DEV, dtype=torch.uint8)

    def __call__(self, fn):
        if self.plain:
            for _ in range(4):
                fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(self.iters):
                fn()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) * 1e3 / self.iters

        def both():
            self.flush.zero_()
            fn()
        return _graph_time(both, self.iters) - _graph_time(lambda: self.flush.zero_(), self.iters)


def _rand(*shape, scale=1.0):
    return (torch.randn(*shape, device=DEV) * scale).to(torch.bfloat16)


def bench_gemm(t, M, N, Kd, bias, ref):
    hbm, flops_peak, tag = _peaks()
    a, b = _rand(M, Kd), _rand(N, Kd)
    out = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    bv = _rand(N) if bias else None
    us = t(lambda: K.gemm(a, b, out=out, bias=bv))
    byt = (M * Kd + N * Kd + M * N) * 2
    fl = 2.0 * M * N * Kd
    floor = max(byt / hbm, fl / flops_peak) * 1e6
    line = "gemm M=%d N=%d K=%d%s: %.1f us  (%.0f GB/s, %.0f TFLOP/s; roofline floor %.1f us -> %.2f %s)" % (
        M, N, Kd, " +bias" if bias else "", us, byt / us / 1e3, fl / us / 1e6, floor, floor / us, tag)
    if ref:
        line += "  | torch.matmul %.1f us" % t(lambda: torch.matmul(a, b.t(), out=out))
    print(line)


def bench_attention(t, B, H, n, backward):
    hbm, _, tag = _peaks()
    qkv = _rand(1, B, n, 3, H, 32, scale=0.7)
    bias = _rand(1, 1, H, n, n)
    mask = (torch.rand(1, B, n, device=DEV) > 0.1).to(torch.bfloat16)
    byt = (4 * B * n * H * 32 + H * n * n) * 2
    if not backward:
        with torch.no_grad():
            us = t(lambda: flash.flash_attention_packed(qkv, mask, bias, 32 ** -0.5))
        mufu = B * H * n * n / (148 * 16 * 1.9e9) * 1e6
        print("attention fwd B=%d H=%d n=%d d=32: %.1f us  (HBM floor %.1f us, exp-unit floor %.1f us -> %.2f %s)" % (
            B, H, n, us, byt / hbm * 1e6, mufu, max(byt / hbm * 1e6, mufu) / us, tag))
        return
    qkv.requires_grad_(True)
    bias.requires_grad_(True)

    def both():      # forward and backward in one go (autograd runs the backward on the stream of its forward)
        out = flash.flash_attention_packed(qkv, mask, bias, 32 ** -0.5)
        out.backward(g)
        qkv.grad = None
        bias.grad = None
    g = torch.randn(1, B, n, H * 32, device=DEV).to(torch.bfloat16)
    with torch.no_grad():
        fwd = t(lambda: flash.flash_attention_packed(qkv, mask, bias, 32 ** -0.5))
    us = t(both)
    print("attention fwd+bwd (+ bias-gradient reduction) B=%d H=%d n=%d d=32: %.1f us  (backward alone ~ %.1f us)" % (B, H, n, us, us - fwd))


def bench_layernorm(t, rows, C, backward):
    hbm, _, tag = _peaks()
    x = _rand(rows, C)
    ln = K.LayerNorm(C).to(DEV, torch.bfloat16)
    if not backward:
        with torch.no_grad():
            us = t(lambda: ln(x))
        byt = 2 * rows * C * 2
        print("layernorm fwd rows=%d C=%d: %.1f us  (%.0f GB/s -> %.2f %s)" % (rows, C, us, byt / us / 1e3, byt / hbm * 1e6 / us, tag))
        return
    x.requires_grad_(True)
    g = torch.randn(rows, C, device=DEV).to(torch.bfloat16)

    def both():
        y = ln(x)
        y.backward(g)
        x.grad = None
        ln.weight.grad = None
        ln.bias.grad = None
    with torch.no_grad():
        fwd = t(lambda: ln(x))
    us = t(both) - fwd
    byt = 3 * rows * C * 2
    print("layernorm bwd rows=%d C=%d: %.1f us  (%.0f GB/s -> %.2f %s)" % (rows, C, us, byt / us / 1e3, byt / hbm * 1e6 / us, tag))


def bench_global_attention(t, R, S, H):
    """Global column attention core of the extra-MSA stack (c = 8 per head): R columns, S sequences."""
    hbm, _, tag = _peaks()
    c = 8
    q = _rand(R, H, c, scale=0.8)
    kv = _rand(R, S, 2 * c)
    mask = (torch.rand(R, S, device=DEV) > 0.1).to(torch.bfloat16)
    gate = _rand(R, S, H * c)
    gb = _rand(H * c)
    with torch.no_grad():
        us = t(lambda: K.global_attention_core(q, kv, mask, gate, gb))
    byt = (kv.numel() + mask.numel() + 2 * gate.numel()) * 2
    print("global attention R=%d S=%d H=%d c=8: %.1f us  (%.0f GB/s -> %.2f %s)" % (R, S, H, us, byt / us / 1e3, byt / hbm * 1e6 / us, tag))


def bench_global_attention_bwd(t, R, S, H):
    """Backward of the global column attention core (d q, d kv, d gate): two passes over kv, gate and dout, two writes."""
    hbm, _, tag = _peaks()
    c = 8
    q = _rand(R, H, c, scale=0.8).requires_grad_(True)
    kv = _rand(R, S, 2 * c).requires_grad_(True)
    mask = (torch.rand(R, S, device=DEV) > 0.1).to(torch.bfloat16)
    gate = _rand(R, S, H * c).requires_grad_(True)
    gb = _rand(H * c)
    dout = _rand(R, S, H * c)

    def both():      # autograd runs the backward on the stream of its forward, so both are timed and the forward subtracted
        out = K.global_attention_core(q, kv, mask, gate, gb)
        out.backward(dout)
        q.grad = kv.grad = gate.grad = None
    with torch.no_grad():
        fwd = t(lambda: K.global_attention_core(q, kv, mask, gate, gb))
    us = t(both) - fwd
    byt = (2 * kv.numel() + 2 * mask.numel() + 2 * gate.numel() + 2 * dout.numel() + kv.numel() + gate.numel()) * 2
    print("global attention backward R=%d S=%d H=%d c=8: %.1f us  (%.0f GB/s -> %.2f %s)" % (R, S, H, us, byt / us / 1e3, byt / hbm * 1e6 / us, tag))


def bench_epilogues(t):
    """Every fused GEMM epilogue the model uses against the fast-path GEMM followed by the separate kernel it replaces
    (a fused path must beat its unfused equivalent, not only sit at some fraction of a roofline)."""
    line = lambda name, us: print("  %-62s %8.1f us" % (name, us))
    for (M, N, Kd) in [(65536, 128, 128), (32768, 256, 256), (65536, 128, 512), (32768, 256, 1024)]:
        a, w, bias = _rand(M, Kd), _rand(N, Kd), _rand(N)
        res, mul = _rand(M, N), _rand(M, N)
        out = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
        dm = (torch.rand(256, N, device=DEV) > 0.15).to(torch.bfloat16)
        rs = torch.rand(M, device=DEV)
        print("gemm epilogues M=%d N=%d K=%d" % (M, N, Kd))
        with torch.no_grad():
            line("plain + bias (fast path)", t(lambda: K.gemm(a, w, bias=bias, out=out)))
            line("bias + resid", t(lambda: K.gemm(a, w, bias=bias, resid=res, out=out)))
            line("bias + resid, in place (out = resid)", t(lambda: K.gemm(a, w, bias=bias, resid=res, out=res)))
            line("bias + sigmoid * mul", t(lambda: K.gemm(a, w, bias=bias, act="sigmoid", mul=mul, out=out)))
            line("bias + dmask + resid", t(lambda: K.gemm(a, w, bias=bias, dmask=(dm, M // 256, 256), resid=res, out=out)))
            line("bias + rowscale + resid", t(lambda: K.gemm(a, w, bias=bias, rowscale=rs, resid=res, out=out)))
            line("unfused: gemm + bias, then torch add of the residual", t(lambda: torch.add(K.gemm(a, w, bias=bias, out=out), res)))
            line("unfused: gemm, then the bias-sigmoid-mul kernel", t(lambda: K.bias_sigmod_ele(K.gemm(a, w, out=out), bias, mul)))
            w2, b2 = _rand(2 * N, Kd), _rand(2 * N)
            line("GLU pairing + row scale, transposed store (2N -> N)", t(lambda: K.gemm(a, w2, bias=b2, glu=True, rowscale=rs, trans_out=True)))
            line("plain transposed store (2N)", t(lambda: K.gemm(a, w2, bias=b2, trans_out=True)))


def bench_grad_gemms(t):
    """Weight-gradient (split-K into an fp32 buffer) and input-gradient GEMMs at the model's shapes against torch.matmul."""
    from fastfold_b200.ops.gemm import _wgrad_splits
    hbm, _, tag = _peaks()
    shapes = [(128, 128, 65536), (512, 128, 65536), (384, 128, 65536), (128, 512, 65536), (768, 256, 32768), (256, 256, 32768),
              (1024, 256, 32768), (256, 1024, 32768)]
    print("weight gradient dW[n_out, n_in] += dY^T X (tokens contracted)")
    for (no, ni, T) in shapes:
        dy, x = _rand(T, no), _rand(T, ni)
        sink = torch.zeros(no, ni, device=DEV)
        sp = _wgrad_splits(T, ((no + 127) // 128) * ((ni + 127) // 128))
        us = t(lambda: K.gemm(dy, x, a_mn=True, b_mn=True, out=sink, accumulate=True, splits=sp))
        ref = t(lambda: torch.matmul(dy.t(), x))
        print("  n_out %4d n_in %4d tokens %d: %.1f us (splits %d) | torch.matmul %.1f us | HBM floor %.1f us %s" % (
            no, ni, T, us, sp, ref, (T * no + T * ni) * 2 / hbm * 1e6, tag))
    print("input gradient dX[tokens, n_in] = dY W (W stored [n_out, n_in])")
    for (no, ni, T) in shapes:
        dy, w = _rand(T, no), _rand(no, ni)
        out = torch.empty(T, ni, device=DEV, dtype=torch.bfloat16)
        us = t(lambda: K.gemm(dy, w, b_mn=True, out=out))
        ref = t(lambda: torch.matmul(dy, w, out=out))
        print("  n_out %4d n_in %4d tokens %d: %.1f us | torch.matmul %.1f us | HBM floor %.1f us %s" % (
            no, ni, T, us, ref, (T * no + T * ni) * 2 / hbm * 1e6, tag))


def bench_ipa(t, N):
    """Invariant point attention core (12 heads, 16 channels, 4 + 8 points, c_z 128): the pair tensor [N, N, 128] is read once."""
    import math
    from fastfold_b200.ops.ipa import ipa_core
    hbm, _, tag = _peaks()
    H, C, PQ, PV, CZ = 12, 16, 4, 8, 128
    f = lambda *s: torch.randn(*s, device=DEV)
    q, k, v = f(N, H, C), f(N, H, C), f(N, H, C)
    qp, kp, vp = f(N, H, PQ, 3) * 8, f(N, H, PQ, 3) * 8, f(N, H, PV, 3) * 8
    z = _rand(N, N, CZ)
    wb, bb, gamma, mask = f(H, CZ) * 0.1, f(H) * 0.1, torch.rand(H, device=DEV) * 0.1, torch.ones(N, device=DEV)
    with torch.no_grad():
        us = t(lambda: ipa_core(q, k, v, qp, kp, vp, z, wb, bb, gamma, mask, math.sqrt(1 / 48), math.sqrt(1 / 3), 1e5))
    byt = z.numel() * 2
    flops = 2.0 * N * N * H * (C + 3 * PQ + CZ + C + 3 * PV + CZ)
    print("ipa core N=%d: %.1f us  (pair tensor %.0f MB -> %.0f GB/s, %.2f %s; %.1f fp32 TFLOP/s)" % (
        N, us, byt / 1e6, byt / us / 1e3, byt / hbm * 1e6 / us, tag, flops / us / 1e6))


def bench_floor(iters):
    """Per-launch time of back-to-back DEPENDENT launches inside one CUDA graph (warm cache): the floor every small
    kernel of a DAP-sharded step pays, for the kernels of this package, a PyTorch elementwise kernel and cuBLAS.  Each op
    consumes the previous one's output so that the launches serialise as they do in the model."""
    n = max(iters, 50)
    rows = {}
    for (M, N, Kd) in [(128, 128, 128), (4096, 256, 256), (4096, 1024, 256), (16384, 128, 128)]:
        a = _rand(M, Kd)
        w = _rand(N, Kd, scale=0.05)
        w2 = _rand(Kd, N, scale=0.05)

        def ours():
            y = K.gemm(a, w)
            return K.gemm(y, w2)

        def cublas():
            y = torch.matmul(a, w.t())
            return torch.matmul(y, w2.t())
        rows["gemm %dx%dx%d" % (M, N, Kd)] = (_graph_time(ours, n) / 2, _graph_time(cublas, n) / 2)
    x = _rand(4096, 256)
    g, b = _rand(256), _rand(256)

    def ln2():
        y = K.layer_norm(x, g, b, 1e-5)
        return K.layer_norm(y, g, b, 1e-5)

    def tln2():
        y = torch.nn.functional.layer_norm(x, (256,), g, b, 1e-5)
        return torch.nn.functional.layer_norm(y, (256,), g, b, 1e-5)
    rows["layernorm 4096x256"] = (_graph_time(ln2, n) / 2, _graph_time(tln2, n) / 2)

    def add2():
        y = x + x
        return y + x
    t_add = _graph_time(add2, n) / 2
    rows["torch add 4096x256"] = (t_add, t_add)
    qkv = (_rand(1, 16, 256, 3, 8, 32) * 0.5)

    def att():
        return flash.flash_attention_packed(qkv, None, None, 32 ** -0.5)
    rows["attention B16 H8 n256"] = (_graph_time(att, n), float("nan"))
    print("per-launch time inside a CUDA graph, dependent launches, warm cache (us): ours | library")
    for k, (a_, b_) in rows.items():
        print("  %-26s %8.2f | %8.2f" % (k, a_, b_))


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("op", choices=["gemm", "attention", "layernorm", "global_attention", "global_attention_bwd", "ipa", "floor", "epilogues", "grad_gemms", "all"])
    ap.add_argument("--m", type=int, default=65536)
    ap.add_argument("--n", type=int, default=512)
    ap.add_argument("--k", type=int, default=128)
    ap.add_argument("--bias", action="store_true")
    ap.add_argument("--ref", action="store_true", help="also time torch.matmul (cuBLAS) on the same shape")
    ap.add_argument("--b", type=int, default=128)
    ap.add_argument("--h", type=int, default=8)
    ap.add_argument("--len", type=int, default=256)
    ap.add_argument("--rows", type=int, default=65536)
    ap.add_argument("--c", type=int, default=128)
    ap.add_argument("--backward", action="store_true")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--plain", action="store_true", help="no graphs, no cache flush: a few plain launches (for profilers)")
    args = ap.parse_args()
    t = Timer(args.iters, args.plain)
    if args.op == "gemm":
        bench_gemm(t, args.m, args.n, args.k, args.bias, args.ref)
    elif args.op == "attention":
        bench_attention(t, args.b, args.h, args.len, args.backward)
    elif args.op == "layernorm":
        bench_layernorm(t, args.rows, args.c, args.backward)
    elif args.op == "ipa":
        bench_ipa(t, args.len if args.len != 256 else 1024)
    elif args.op == "global_attention_bwd":
        bench_global_attention_bwd(t, args.b if args.b != 128 else 256, args.len if args.len != 256 else 5120, args.h)
    elif args.op == "epilogues":
        bench_epilogues(t)
    elif args.op == "grad_gemms":
        bench_grad_gemms(t)
    elif args.op == "floor":
        bench_floor(args.iters)
    elif args.op == "global_attention":
        bench_global_attention(t, args.b if args.b != 128 else 256, args.len if args.len != 256 else 5120, args.h)
    else:
        for (M, N, Kd) in [(65536, 128, 128), (65536, 512, 128), (65536, 384, 128), (65536, 128, 512), (32768, 768, 256), (32768, 1024, 256),
                           (32768, 256, 1024), (32768, 256, 256), (8192, 8192, 128), (8192, 8192, 8192)]:
            bench_gemm(t, M, N, Kd, True, True)
        for (B, H, n) in [(128, 8, 256), (256, 8, 128), (256, 4, 256)]:
            bench_attention(t, B, H, n, False)
            bench_attention(t, B, H, n, True)
        for (rows, C) in [(65536, 128), (32768, 256)]:
            bench_layernorm(t, rows, C, False)
            bench_layernorm(t, rows, C, True)
        bench_global_attention(t, 256, 5120, 8)
        bench_global_attention_bwd(t, 256, 5120, 8)
        bench_ipa(t, 1024)
        bench_ipa(t, 2048)
    from fastfold_b200.ops import _lib
    st = _lib.read_status()
    if st[0]:
        print("device status:", st)


if __name__ == "__main__":
    main()
