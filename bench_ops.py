"""Per-operator measurements on one B200 for every operator of the library, at the
shapes of the benchmark configurations (synthetic seeded data).  Prints one JSON
line per measurement: time, algorithmic bytes, achieved GB/s and the fraction of
the measured HBM copy peak.  bench.py stays the headline benchmark; this script
covers the remaining operators.

    python bench_ops.py [--suite small|edgeconv|micro|project|gather|all] [--iters 20]

Timing: CUDA events around each call on the launching stream, 3 warm-up calls,
an L2 flush (256 MB write) before every timed call of the small configurations.
Algorithmic bytes follow the no-reuse gather model (every gathered row counts in
full, every dense stream once per required pass)."""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from dgnn_b200 import kernels, synth  # noqa: E402


def peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return float(json.load(open(path))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


PEAK, PEAK_KIND = peak()
_flush = None


def timed(fn, iters, flush):
    global _flush
    if flush and _flush is None:
        _flush = torch.empty(64 * 1024 * 1024, dtype=torch.float32, device="cuda")
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        if flush:
            _flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record(); fn(); e.record()
        torch.cuda.synchronize()
        total += s.elapsed_time(e)
    return total / iters


def report(op, config, ms, alg_bytes, **extra):
    gbs = alg_bytes / (ms * 1e-3) / 1e9
    line = {"op": op, "config": config, "ms": round(ms, 5), "algorithmic_bytes": int(alg_bytes),
            "achieved_gbs": round(gbs, 1), "frac_of_hbm_peak": round(gbs / PEAK, 4), "peak_gbs": PEAK,
            "peak_kind": PEAK_KIND}
    line.update(extra)
    print(json.dumps(line), flush=True)


def gat_bytes(n, e, h, f, p):
    fwd = (n + 1) * p + 4 * e + 4 * e * h + 4 * n * h + 4 * e * h * f + 4 * n * h * f + 8 * n * h
    bwd = (n + 1) * p + 8 * e + 12 * e * h + 4 * n * h + 4 * e * h * f + 12 * n * h * f + 4 * n * h * f + 8 * e * h + 8 * n * h
    return fwd, bwd


def suite_small(iters):
    """Configs 1 and 2: the 2708-node graph (latency-bound: a few tens of MB of traffic)."""
    dev = torch.device("cuda")
    rp, ci = synth.powerlaw_graph()
    n, e = rp.numel() - 1, ci.numel()
    rp, ci = rp.to(dev), ci.to(dev)
    cp, ri, pm = kernels.csr2csc(rp, ci)
    g = torch.Generator(device=dev).manual_seed(1)
    h, f = 4, 64
    ar, ac = torch.randn(n, h, device=dev, generator=g), torch.randn(n, h, device=dev, generator=g)
    x, go = torch.randn(n, h, f, device=dev, generator=g), torch.randn(n, h, f, device=dev, generator=g)
    out, emax, esum = kernels.gat_forward(ar, ac, rp, ci, 0.2, x)
    fb, bb = gat_bytes(n, e, h, f, 4)
    cfg = f"config 1: {n} nodes / {e} edges, 4 heads x 64"
    report("gat_forward", cfg, timed(lambda: kernels.gat_forward(ar, ac, rp, ci, 0.2, x), iters, True), fb)
    report("gat_backward", cfg, timed(lambda: kernels.gat_backward(0.2, 0.0, rp, cp, ri, pm, emax, esum, None, x, out, ar, ac, go), iters, True), bb)
    report("csr2csc", cfg, timed(lambda: kernels.csr2csc(rp, ci), iters, True), 2 * (n + 1) * 4 + 20 * e)
    # the whole layer step of config 1 (in = 1433 -> 4 x 64), eager and replayed from a CUDA graph
    from dgnn_b200.layers import GATConv
    torch.manual_seed(1)
    layer = GATConv(1433, f, h).to(dev).train()
    xin = (torch.rand(n, 1433, device=dev, generator=g) < 0.013).float()
    cot = torch.randn(n, h, f, device=dev, generator=g)

    def layer_step():
        layer.zero_grad(set_to_none=False)
        (layer(rp, ci, cp, ri, pm, xin) * cot).sum().backward()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            layer_step()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        layer_step()
    layer_b = fb + bb + 4 * n * 1433 + 2 * 4 * 1433 * h * f
    report("GATConv layer fwd+bwd, eager", cfg, timed(layer_step, iters, True), layer_b)
    report("GATConv layer fwd+bwd, CUDA graph replay", cfg, timed(graph.replay, iters, True), layer_b)
    # config 2: MoNet, 3 kernels, 16 channels, pseudo dim 2
    k, fo, dim = 3, 16, 2
    feat = torch.randn(n, k, fo, device=dev, generator=g)
    pseudo = synth.monet_pseudo(rp, ci)
    mu, sig = torch.rand(k, dim, device=dev, generator=g), torch.ones(k, dim, device=dev)
    gout = torch.randn(n, k, fo, device=dev, generator=g)
    cfg = f"config 2: {n} nodes / {e} edges, 3 kernels x 16, pseudo dim 2"
    gmm_b = (n + 1) * 4 + 4 * e + 4 * e * dim + 4 * e * k * fo + 4 * n * k * fo
    report("gmm_forward", cfg, timed(lambda: kernels.gmm_forward(rp, ci, feat, pseudo, mu, sig), iters, True), gmm_b)
    sd_b = (n + 1) * 4 + 4 * e + 4 * e * k * fo + 4 * n * k * fo + 4 * e * k
    report("mhsddmm", cfg, timed(lambda: kernels.mhsddmm(rp, ci, gout, feat), iters, True), sd_b)
    report("mhtranspose", cfg, timed(lambda: kernels.mhtranspose(pm, pseudo), iters, True), 4 * e + 8 * e * dim)
    gg = kernels.mhsddmm(rp, ci, gout, feat)
    report("gaussian_bp", cfg, timed(lambda: kernels.gaussian_bp(pseudo, mu, sig, gg), iters, True), 4 * e * (2 * dim + k))

    def gmm_bwd():
        gg_ = kernels.mhsddmm(rp, ci, gout, feat)
        pt = kernels.mhtranspose(pm, pseudo)
        kernels.gmm_forward(cp, ri, gout, pt, mu, sig)
        kernels.gaussian_bp(pseudo, mu, sig, gg_)
    report("gmm_backward (4 calls)", cfg, timed(gmm_bwd, iters, True), sd_b + gmm_b + 4 * e + 8 * e * dim + 4 * e * (2 * dim + k))


def suite_edgeconv(iters):
    """Config 3: 32 clouds x 2048 points, k = 20, widths 64 / 64 / 128."""
    dev = torch.device("cuda")
    x = synth.unit_sphere_clouds(32, 2048, seed=3, device=dev)
    src = synth.knn_src_ind(x, 20)
    m, k = 32 * 2048, 20
    g = torch.Generator(device=dev).manual_seed(3)
    for f in (64, 128):
        hs, hd, go = (torch.randn(m, f, device=dev, generator=g) for _ in range(3))
        _, idx = kernels.edgeconv_forward(k, src, hs, hd)
        cfg = f"config 3: {m} points, k={k}, F={f}"
        report("edgeconv_forward", cfg, timed(lambda: kernels.edgeconv_forward(k, src, hs, hd), iters, True),
               4 * m * k + 4 * m * k * f + 12 * m * f, compulsory_bytes=4 * m * k + 16 * m * f)
        report("edgeconv_backward", cfg, timed(lambda: kernels.edgeconv_backward(go, idx), iters, True), 20 * m * f)
        report("edgeconv_backward_ordered (csr2csc of the kNN graph + gather, reproducible)", cfg,
               timed(lambda: kernels.edgeconv_backward_ordered(k, src, go, idx), iters, True), 20 * m * f)


def check_csc(rp, ci, cp, ri, pm, n):
    """Bit-exact invariants of csr2csc, on the device (no host copy at 256 M entries)."""
    e = ci.numel()
    counts = torch.bincount(ci.long(), minlength=n)
    ref = torch.zeros(n + 1, dtype=torch.int64, device=ci.device)
    torch.cumsum(counts, 0, out=ref[1:])
    ok = torch.equal(cp.long(), ref)
    del counts, ref
    cols = torch.repeat_interleave(torch.arange(n, device=ci.device, dtype=torch.int32), (cp[1:] - cp[:-1]).long())
    ok = ok and torch.equal(ci[pm.long()], cols)
    del cols
    ok = ok and torch.equal((torch.searchsorted(rp.long(), pm.long(), right=True) - 1).int(), ri)
    inc = pm[1:] > pm[:-1]
    b = cp[1:-1].long()
    b = b[(b > 0) & (b < e)] - 1
    inc[b] = True
    return bool(ok and inc.all())


def suite_micro(iters, edges, degrees, heads, cap_gb):
    """Config 5: SDDMM, edge-softmax + SpMM (the GAT forward) and csr2csc on R-MAT graphs of a fixed
    edge count, average degree swept by the node count, F = 64."""
    dev = torch.device("cuda")
    f = 64
    for deg in degrees:
        n = edges // deg
        rp, ci = synth.rmat_graph(n, edges, seed=5, device=dev, ptr_dtype=torch.int64)
        cfg0 = f"config 5: R-MAT {n} nodes / {edges} edges (avg degree {deg})"
        ms = timed(lambda: kernels.csr2csc(rp, ci), max(3, iters // 4), False)
        cp, ri, pm = kernels.csr2csc(rp, ci)
        report("csr2csc", cfg0, ms, 2 * (n + 1) * 8 + 20 * edges, bit_exact_invariants=check_csc(rp, ci, cp, ri, pm, n))
        del cp, ri
        tr_in = torch.randn(edges, 8, device=dev)
        report("mhtranspose", cfg0 + ", 8 values per edge",
               timed(lambda: kernels.mhtranspose(pm, tr_in), max(3, iters // 4), False), 4 * edges + 8 * edges * 8)
        del tr_in, pm
        for h in heads:
            tensor_gb = n * h * f * 4 / 1e9
            cfg = cfg0 + f", {h} heads x {f}"
            # peak use: two [N,H,F] tensors (SDDMM operands; then input and output of the forward), the [E,H] SDDMM
            # result and the long-row partials; what does not fit the free device memory is reported, not tried
            free_gb = torch.cuda.mem_get_info(dev)[0] / 1e9
            need_gb = 2 * tensor_gb + edges * h * 4 / 1e9 + 2 * (edges / 1024) * 2 * (2 * h * f + 3 * h) * 4 / 1e9 + 2.0
            limit_gb = min(free_gb, cap_gb) if cap_gb > 0 else free_gb
            if h * f > 1024:
                print(json.dumps({"op": "skipped", "config": cfg, "reason": "heads x width above 1024 floats per row: outside the float4 layout of the kernels"}), flush=True)
                continue
            if need_gb > limit_gb:
                print(json.dumps({"op": "skipped", "config": cfg,
                                  "reason": f"needs {need_gb:.0f} GB (two [N,H,F] tensors of {tensor_gb:.1f} GB, the [E,H] result, partials) "
                                            f"but {limit_gb:.0f} GB are available on one GPU"}), flush=True)
                continue
            a = torch.randn(n, h, f, device=dev)
            b = torch.randn(n, h, f, device=dev)
            it = max(3, iters // 4)
            sd_b = (n + 1) * 8 + 4 * edges + 4 * edges * h * f + 4 * n * h * f + 4 * edges * h
            report("mhsddmm", cfg, timed(lambda: kernels.mhsddmm(rp, ci, a, b), it, False), sd_b)
            del a
            torch.cuda.empty_cache()
            ar, ac = torch.randn(n, h, device=dev), torch.randn(n, h, device=dev)
            fb, _ = gat_bytes(n, edges, h, f, 8)
            report("edge_softmax+spmm (gat_forward)", cfg, timed(lambda: kernels.gat_forward(ar, ac, rp, ci, 0.2, b), it, False), fb)
            del b, ar, ac
            torch.cuda.empty_cache()
        del rp, ci
        torch.cuda.empty_cache()


def suite_gather(iters, nodes, edges):
    """What bounds the fused forward sweep at the headline shape (8 heads x 32, R-MAT): the same kernel on the same
    graph with the source ids folded into a window of W rows, so that every gathered row comes out of the L2
    (W x 1 KB <= 32 MB) -- the time that is left is the L2 -> SM delivery and the arithmetic, not HBM -- and with
    the most referenced rows held in the L2 (hot rows + set-aside), which cuts DRAM reads but not the row bytes
    that cross the L2 -> SM path."""
    dev = torch.device("cuda")
    h, f = 8, 32
    rp, ci = synth.rmat_graph(nodes, edges, seed=4, device=dev, ptr_dtype=torch.int64)
    x = torch.randn(nodes, h, f, device=dev)
    ar, ac = torch.randn(nodes, h, device=dev), torch.randn(nodes, h, device=dev)
    fb, _ = gat_bytes(nodes, edges, h, f, 8)
    cfg0 = f"R-MAT {nodes} nodes / {edges} edges, {h} heads x {f}, forward with negative-side outputs"
    it = max(3, iters // 2)
    report("gat_forward", cfg0 + ", sources as generated", timed(lambda: kernels.gat_forward(ar, ac, rp, ci, 0.2, x, neg=True), it, False),
           fb, gathered_row_bytes=4 * edges * h * f)
    cp, _, _ = kernels.csr2csc(rp, ci)
    hot = kernels.hot_rows(cp, 64 * 2**20 // (4 * h * (f + 1)))
    aside = kernels.l2_set_aside(80 * 2**20)
    report("gat_forward", cfg0 + f", 64 MB of the most referenced source rows loaded evict_last, {aside / 2**20:.0f} MB of L2 set aside",
           timed(lambda: kernels.gat_forward(ar, ac, rp, ci, 0.2, x, neg=True, hot=hot), it, False), fb,
           gathered_row_bytes=4 * edges * h * f)
    kernels.l2_set_aside(0)
    del cp, hot
    for w in (8192, 32768):
        folded = ci % w
        report("gat_forward", cfg0 + f", source ids folded into {w} rows ({w * h * f * 4 / 2**20:.0f} MB: every gather is an L2 hit)",
               timed(lambda: kernels.gat_forward(ar, ac, rp, folded, 0.2, x, neg=True), it, False), fb,
               gathered_row_bytes=4 * edges * h * f)
        del folded


def suite_project(iters, rows):
    """The dense node projection of the bench configuration (in=100 -> 8 x 32) on the tensor cores, forward and
    weight gradient, beside the fp32 library GEMM (TF32 off) that torch.matmul runs for the same product."""
    dev = torch.device("cuda")
    k, n = 100, 256
    g = torch.Generator(device=dev).manual_seed(7)
    x = torch.randn(rows, k, device=dev, generator=g)
    w = torch.randn(k, n, device=dev, generator=g)
    go = torch.randn(rows, n, device=dev, generator=g)
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    cfg = f"projection {rows} x {k} -> {n}"
    flops = 2.0 * rows * k * n
    for name, fn, nbytes in (("project_forward (tcgen05, 3 x tf32)", lambda: kernels.project_forward(x, w, w_kn=True), 4 * rows * (k + n)),
                             ("torch.matmul fp32 (library)", lambda: x @ w, 4 * rows * (k + n)),
                             ("project_wgrad (tcgen05, 3 x tf32)", lambda: kernels.project_wgrad(x, go, w_kn=True), 4 * rows * (k + n)),
                             ("x.t() @ grad fp32 (library)", lambda: x.t() @ go, 4 * rows * (k + n))):
        ms = timed(fn, iters, False)
        report(name, cfg, ms, nbytes, fp32_equivalent_tflops=round(flops / (ms * 1e-3) / 1e12, 1))
    torch.backends.cuda.matmul.allow_tf32 = prev


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--suite", default="all", choices=["small", "edgeconv", "micro", "project", "gather", "all"])
    ap.add_argument("--project-rows", type=int, default=2_400_000)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--gather-nodes", type=int, default=2_400_000)
    ap.add_argument("--gather-edges", type=int, default=120_000_000)
    ap.add_argument("--micro-edges", type=int, default=256_000_000)
    ap.add_argument("--micro-degrees", default="4,16,64,128")
    ap.add_argument("--micro-heads", default="1,4,8,16")
    ap.add_argument("--cap-gb", type=float, default=0.0, help="memory cap for one configuration (0: the free device memory)")
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("bench_ops.py needs a CUDA device: there is no CPU path")
    if args.suite in ("small", "all"):
        suite_small(args.iters)
    if args.suite in ("edgeconv", "all"):
        suite_edgeconv(args.iters)
    if args.suite in ("project", "all"):
        suite_project(args.iters, args.project_rows)
    if args.suite in ("gather", "all"):
        suite_gather(args.iters, args.gather_nodes, args.gather_edges)
    if args.suite in ("micro", "all"):
        suite_micro(args.iters, args.micro_edges, [int(d) for d in args.micro_degrees.split(",")],
                    [int(h) for h in args.micro_heads.split(",")], args.cap_gb)


if __name__ == "__main__":
    main()
