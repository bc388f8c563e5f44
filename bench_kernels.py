"""Kernel micro-benchmarks with roofline fractions (CUDA events, warm-up, L2-exceeding inputs).

  python bench_kernels.py                      # every case at its benchmark size
  python bench_kernels.py --case wgrad --small # one small launch set, sized for an ncu capture
  python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 bench_kernels.py --case wgrad-rs
  python bench_kernels.py --impl reference     # the reference's own Triton / library kernels on the same shapes
                                               # (unmodified code from baseline/_ref; nothing of this package is loaded)
  python bench_kernels.py --case compare       # this package's kernels on exactly those shapes
  python bench_kernels.py --case sustained     # seconds-long power-capped loops: pair GEMM / GLU against the library, with clocks
  python bench_kernels.py --case short-k       # GPT-2-sized products, graph-timed over rotating buffers
  python bench_kernels.py --case head          # output head: fused head + cross-entropy against plain GEMMs
  python bench_kernels.py --case pair-small    # one launch per GEMM kernel on a small case (for counter captures)

Each line is JSON: achieved TFLOP/s or GB/s and the fraction "of measured" peak, where the peaks come from
MEASURED_PEAKS.json next to this file (cuBLAS bf16 burst and a STREAM-style copy), else the documented fallback
(1590 TFLOP/s, 6650 GB/s, marked "of fallback").
"""
from __future__ import annotations

import argparse
import json
import os

import torch


def peaks():
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return p["bf16_tflops"], p["hbm_gbs"], "of measured"
    return 1590.0, 6650.0, "of fallback"


def timeit(fn, iters=20, warm=5, flush=None):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        if flush is not None:
            flush.add_(1.0)                      # > L2-sized write between timed launches
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        total += a.elapsed_time(b)
    return total / iters


def fused_reduce_scatter_case():
    """Clip-weighted weight gradient with its reduce-scatter fused in, on W ranks (launch with torch.distributed.run).

    Every rank multiplies its own microbatch and reduces the fp32 tiles straight into the owners' shards through peer
    pointers.  Roofline per rank = max(FLOPs / measured GEMM peak, bytes leaving over NVLink / 770 GB/s measured peer
    copy rate); device-timed, max over ranks.  Compared with the same product followed by an NCCL reduce-scatter.
    """
    import torch.distributed as dist
    from opaque_b200 import ops
    from opaque_b200.parallel.peer import PeerGroup
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank)))
    torch.cuda.set_device(dev)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=dev)
    tf_peak, _, tag = peaks()
    group = PeerGroup(dev)
    st = group.status
    flush = torch.zeros(64 * 1024 * 1024, device=dev)
    for T, M, N in [(16384, 3072, 768), (16384, 4096, 4096), (16384, 8192, 2048)]:
        a = torch.randn(T, M, device=dev).bfloat16()
        b = torch.randn(T, N, device=dev).bfloat16()
        c = torch.rand(T // 1024, device=dev)
        total = M * N
        shard = (total + world * 64 - 1) // (world * 64) * 64
        buf = group.buffer(shard, torch.float32)
        local = torch.zeros(shard * world, device=dev)

        def fused():
            ops.wgrad_clip_per_example(a, b, None, ex_scale=c, rows_per_example=1024, ldm=N, peer_table=buf.table,
                                       shard_elems=shard, status=st)

        def unfused():
            ops.wgrad_clip_per_example(a, b, local, ex_scale=c, rows_per_example=1024, ldm=N, status=st)   # same split-K, local destination
            dist.reduce_scatter_tensor(buf.local, local)
        rows = {}
        for name, fn in (("fused (peer red.add in the epilogue)", fused), ("same kernel + NCCL reduce-scatter", unfused)):
            dist.barrier()
            ms = timeit(fn, 10, 3, flush)
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            rows[name] = float(t)
        group.barrier()
        torch.cuda.synchronize()
        if rank == 0:
            flops = 2.0 * T * M * N
            t_compute = flops / (tf_peak * 1e9)                      # ms
            t_link = total * 4 * (world - 1) / world / 770e6         # ms at 770 GB/s per direction
            roof = max(t_compute, t_link)
            for name, ms in rows.items():
                print(json.dumps({"kernel": f"wgrad_clip -> reduce-scatter {T}x{M}x{N} on {world} GPUs, {name}", "ms": round(ms, 4),
                                  "tflops_per_gpu": round(flops / ms / 1e9, 1), "roofline_ms": round(roof, 4),
                                  "bound": "compute" if t_compute >= t_link else "nvlink",
                                  "frac_of_roofline_" + tag.replace(" ", "_"): round(roof / ms, 3)}), flush=True)
    if st.read():
        raise SystemExit(f"a device wait timed out (status {st.read()})")
    dist.barrier()
    group.close()
    dist.destroy_process_group()


COMPARE_SHAPES = {"rows": 16384, "hidden": 4096, "ffn": 14336, "vocab": 128256, "ce_rows": 4096, "lce_rows": 8192,
                  "heads": 32, "kv_heads": 8, "head_dim": 128, "seq": 1024, "lora_r": 16}


def _fwd_bwd(fn, *inputs, dy=None):
    """Forward, then the gradients of every input that requires one for the fixed output gradient ``dy``."""
    out = fn(*inputs)
    out = out[0] if isinstance(out, tuple) else out
    wrt = [t for t in inputs if isinstance(t, torch.Tensor) and t.requires_grad]
    torch.autograd.grad(out, wrt, dy if dy is not None else torch.ones_like(out))


def compare_cases(impl: str):
    """One row per operation on COMPARE_SHAPES, for ``impl`` = ``ours`` (this package) or ``reference`` (the reference's
    unmodified Triton / library kernels, packages/opaque-patches/src/opaque/api/patches/kernels/*.py).  Both arms time
    the same algorithmic work with CUDA events after warm-up and with an L2-sized write between launches."""
    S = COMPARE_SHAPES
    dev = torch.device("cuda", 0)
    tf_peak, bw_peak, tag = peaks()
    flush = torch.zeros(64 * 1024 * 1024, device=dev)
    if impl == "reference":
        import sys
        here = os.path.dirname(os.path.abspath(__file__))
        sys.path[:0] = [os.path.join(here, "baseline", "_ref"), os.path.join(here, "baseline", "shims")]
        from opaque.api.patches.kernels.cross_entropy import opaque_cross_entropy_loss
        from opaque.api.patches.kernels.fused_add_rms_norm import opaque_fused_add_rms_norm
        from opaque.api.patches.kernels.linear_cross_entropy import Opaque_LinearCrossEntropyLoss
        from opaque.api.patches.kernels.lora import opaque_lora_w
        from opaque.api.patches.kernels.rms_norm import opaque_rms_norm
        from opaque.api.patches.kernels.rope_embedding import opaque_rope_qk
        from opaque.api.patches.kernels.swiglu import opaque_swiglu
        rms = lambda x, w: opaque_rms_norm(x, w, 1e-5)
        add_rms = lambda x, r, w: opaque_fused_add_rms_norm(x, r, w, 1e-5)
        swiglu = opaque_swiglu
        ce = lambda z, lab: opaque_cross_entropy_loss(z, lab)
        lora = lambda x, w, a, b: opaque_lora_w(x, w, a.t(), b.t(), 2.0)       # the reference takes A [in, r] and B [r, out]

        def lce(h, w, lab):
            return Opaque_LinearCrossEntropyLoss.apply(h, w, lab, -100, 0, 0.0, False)

        def rope(q, k, cos, sin):       # the reference takes [B, heads, T, D]
            return opaque_rope_qk(q, k, cos, sin)
        rope_layout = "bhtd"
    else:
        from opaque_b200 import ops
        from opaque_b200.engine.fused import lora_linear
        from opaque_b200.models.layers import linear_cross_entropy
        rms = lambda x, w: ops.rms_norm(x, w, 1e-5)
        add_rms = lambda x, r, w: ops.fused_add_rms_norm(x, r, w, 1e-5)
        swiglu = ops.swiglu
        ce = lambda z, lab: ops.cross_entropy(z, lab)
        lora = lambda x, w, a, b: lora_linear(x, w, None, a, b, 2.0)

        def lce(h, w, lab):
            return linear_cross_entropy(h, w, lab, torch.ones(lab.shape, device=lab.device))

        def rope(q, k, cos, sin):
            return ops.rope_qk(q, k, cos, sin)
        rope_layout = "bthd"

    def emit(name, ms, flops=None, bytes_=None):
        row = {"impl": impl, "kernel": name, "ms": round(ms, 4)}
        if flops:
            row["tflops"] = round(flops / ms / 1e9, 1)
            row["frac_" + tag.replace(" ", "_")] = round(flops / ms / 1e9 / tf_peak, 3)
        if bytes_:
            row["GBs"] = round(bytes_ / ms / 1e6, 1)
            row["frac_" + tag.replace(" ", "_")] = round(bytes_ / ms / 1e6 / bw_peak, 3)
        print(json.dumps(row), flush=True)

    R, H, I, V = S["rows"], S["hidden"], S["ffn"], S["vocab"]
    bf = dict(device=dev, dtype=torch.bfloat16)
    x = torch.randn(R, H, **bf)
    w = torch.ones(H, **bf)
    emit(f"rms_norm fwd {R}x{H}", timeit(lambda: rms(x, w), 20, 5, flush), bytes_=2 * x.numel() * 2)
    xg = x.clone().requires_grad_(True)
    dyx = torch.randn(R, H, **bf)
    emit(f"rms_norm fwd+bwd (dx; frozen weight) {R}x{H}", timeit(lambda: _fwd_bwd(rms, xg, w, dy=dyx), 20, 5, flush), bytes_=5 * x.numel() * 2)
    res = torch.randn(R, H, **bf)
    emit(f"fused add + rms_norm fwd {R}x{H}", timeit(lambda: add_rms(x, res, w), 20, 5, flush), bytes_=4 * x.numel() * 2)
    g, u = torch.randn(R, I, **bf), torch.randn(R, I, **bf)
    emit(f"swiglu fwd {R}x{I}", timeit(lambda: swiglu(g, u), 20, 5, flush), bytes_=3 * g.numel() * 2)
    gg, ug = g.clone().requires_grad_(True), u.clone().requires_grad_(True)
    dyh = torch.randn(R, I, **bf)
    emit(f"swiglu fwd+bwd {R}x{I}", timeit(lambda: _fwd_bwd(swiglu, gg, ug, dy=dyh), 20, 5, flush), bytes_=8 * g.numel() * 2)
    del g, u, gg, ug, dyh
    B, T, nh, nkv, hd = R // S["seq"], S["seq"], S["heads"], S["kv_heads"], S["head_dim"]
    if rope_layout == "bhtd":
        q, k = torch.randn(B, nh, T, hd, **bf), torch.randn(B, nkv, T, hd, **bf)
        inv = 1.0 / (500000.0 ** (torch.arange(0, hd, 2, device=dev).float() / hd))
        ang = torch.outer(torch.arange(T, device=dev).float(), inv)
        cos, sin = ang.cos().bfloat16(), ang.sin().bfloat16()
    else:
        q, k = torch.randn(B, T, nh, hd, **bf), torch.randn(B, T, nkv, hd, **bf)
        cos, sin = ops.rope_tables(hd, T, 500000.0, device=dev)
    emit(f"rope q,k fwd {B}x{T}x({nh}+{nkv})x{hd}", timeit(lambda: rope(q, k, cos, sin), 20, 5, flush),
         bytes_=2 * (q.numel() + k.numel()) * 2)
    CR = S["ce_rows"]
    z = torch.randn(CR, V, **bf)
    lab = torch.randint(0, V, (CR,), device=dev)
    zg = z.clone().requires_grad_(True)
    emit(f"cross_entropy loss + dlogits (autograd op, logits kept) {CR}x{V}", timeit(lambda: _fwd_bwd(ce, zg, lab), 10, 3, flush),
         bytes_=2 * z.numel() * 2)
    if impl == "ours":
        from opaque_b200.ops.functional import cross_entropy_fused_
        emit(f"cross_entropy loss + dlogits in place (one pass, as the engine calls it) {CR}x{V}",
             timeit(lambda: cross_entropy_fused_(z, lab), 10, 3, flush), bytes_=2 * z.numel() * 2)
    del z, zg
    LR = S["lce_rows"]
    h = (torch.randn(LR, H, **bf) * 0.5).requires_grad_(True)
    wv = (torch.randn(V, H, **bf) * 0.02)
    labl = torch.randint(0, V, (LR,), device=dev)
    # fused linear + cross-entropy with a frozen head: logits (forward) and dlogits @ W (backward) = 4 R V H FLOPs as
    # the algorithmic minimum (a recomputing backward does 6)
    def lce_step():
        out = lce(h, wv, labl)
        torch.autograd.grad(out.sum() if out.ndim else out, [h])
    emit(f"linear + cross_entropy fwd+bwd (frozen head) {LR}x{H}x{V}", timeit(lce_step, 5, 2, flush), flops=4.0 * LR * V * H)
    del h, wv
    xl = torch.randn(R, H, **bf).requires_grad_(True)
    wl = torch.randn(H, H, **bf) * 0.02
    la = torch.randn(S["lora_r"], H, **bf).requires_grad_(True)
    lb = torch.randn(H, S["lora_r"], **bf).requires_grad_(True)
    emit(f"LoRA linear fwd (frozen W + r{S['lora_r']}) {R}x{H}x{H}", timeit(lambda: lora(xl, wl, la, lb), 20, 5, flush),
         flops=2.0 * R * H * H)
    dyl = torch.randn(R, H, **bf)
    emit(f"LoRA linear fwd+bwd (dx, dA, dB summed over rows) {R}x{H}x{H}", timeit(lambda: _fwd_bwd(lora, xl, wl, la, lb, dy=dyl), 20, 5, flush),
         flops=4.0 * R * H * H)
    if impl == "ours":
        # the dense products of the model path on CTA pairs, beside the library GEMM on the same shapes
        st = ops.StatusWord(dev)
        for M, N, K in [(16384, 4096, 4096), (16384, 14336, 4096), (16384, 4096, 14336), (16384, 6144, 4096)]:
            xx = torch.randn(M, K, **bf)
            ww = torch.randn(N, K, **bf) * 0.02
            fl = 2.0 * M * N * K
            emit(f"gemm x W^T, CTA pairs {M}x{N}x{K}", timeit(lambda: ops.gemm_pair(xx, ww, status=st), 20, 5, flush), flops=fl)
            emit(f"gemm x W^T, single CTA {M}x{N}x{K}", timeit(lambda: ops.gemm(xx, ww, status=st, kernel="single"), 20, 5, flush), flops=fl)
            emit(f"library x W^T {M}x{N}x{K}", timeit(lambda: torch.matmul(xx, ww.t()), 20, 5, flush), flops=fl)
            wk = ww.t().contiguous()
            emit(f"gemm dY W ([K,N] operand), CTA pairs {M}x{N}x{K}", timeit(lambda: ops.gemm_pair(xx, wk, b_layout="kn", status=st), 20, 5, flush), flops=fl)
            emit(f"library dY W {M}x{N}x{K}", timeit(lambda: torch.matmul(xx, wk), 20, 5, flush), flops=fl)
            del xx, ww, wk
        M, I, K = 16384, 14336, 4096
        xx, wg_, wu_ = torch.randn(M, K, **bf), torch.randn(I, K, **bf) * 0.02, torch.randn(I, K, **bf) * 0.02
        fl = 4.0 * M * I * K
        emit(f"gate+up GEMM with SwiGLU epilogue (h, gate, up stored) {M}x2x{I}x{K}", timeit(lambda: ops.gemm_glu(xx, wg_, wu_, status=st), 10, 3, flush), flops=fl)
        emit(f"gate+up GEMM with SwiGLU epilogue (h only) {M}x2x{I}x{K}", timeit(lambda: ops.gemm_glu(xx, wg_, wu_, save_preact=False, status=st), 10, 3, flush), flops=fl)
        emit(f"library gate, up GEMMs + SwiGLU kernel {M}x2x{I}x{K}", timeit(lambda: ops.swiglu(torch.matmul(xx, wg_.t()), torch.matmul(xx, wu_.t())), 10, 3, flush), flops=fl)
        if st.read():
            raise SystemExit(f"a device wait timed out (status {st.read()})")


def pair_small_case():
    """Two rounds of one launch each: CTA-pair GEMM (512 x 256 tiles), its 256 x 256 variant, the single-CTA kernel, the
    gated up-projection and the library GEMM on y[8192, 8192] = x[8192, 4096] W^T (inputs + output 192 MB > L2).  A small
    case for counter captures (one launch per kernel and round; nothing is timed here)."""
    from opaque_b200 import ops
    dev = torch.device("cuda", 0)
    M, N, K = 8192, 8192, 4096
    x = torch.randn(M, K, device=dev).bfloat16()
    w = (torch.randn(N, K, device=dev) * 0.02).bfloat16()
    st = ops.StatusWord(dev)
    for _ in range(2):
        y = ops.gemm_pair(x, w, status=st)
        y2 = ops.gemm_pair(x, w, status=st, tile="256x256")
        y3 = ops.gemm(x, w, status=st, kernel="single")
        h, g, u = ops.gemm_glu(x, w[: N // 2], w[N // 2:], status=st)
        ref = torch.matmul(x, w.t())
    torch.cuda.synchronize()
    if st.read():
        raise SystemExit(f"a device wait timed out (status {st.read()})")
    err = [float((t.float() - ref.float()).abs().max()) for t in (y, y2, y3)]
    print(json.dumps({"case": "pair-small", "max_abs_diff_vs_library": err}))


def _graph_time(fns, launches=16, reps=7):
    """ms per launch of ``launches`` back-to-back calls (cycling through ``fns``) captured in ONE CUDA graph: neither host
    launch latency nor a warm L2 enters when the functions work on rotating buffers larger than L2 in total."""
    for f in fns:
        f()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        with torch.cuda.graph(g, stream=side):
            for i in range(launches):
                fns[i % len(fns)]()
    ts = []
    for _ in range(reps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        g.replay()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b) / launches)
    ts.sort()
    return ts[len(ts) // 2]


def short_k_case():
    """GPT-2-sized products (K = 768 / N = 768) and two Llama-sized ones: single-CTA / pair 256x256 / pair 512x256 / library,
    forward form (x W^T + bias) and data-gradient form (dY W), graph-timed over four rotating buffer sets."""
    from opaque_b200 import ops
    dev = torch.device("cuda", 0)
    st = ops.StatusWord(dev)
    nset = 4
    for M, N, K in [(16384, 2304, 768), (16384, 768, 768), (16384, 3072, 768), (16384, 768, 3072), (16384, 4096, 4096),
                    (8192, 4096, 4096)]:
        xs = [torch.randn(M, K, device=dev).bfloat16() for _ in range(nset)]
        outs = [torch.empty(M, N, device=dev, dtype=torch.bfloat16) for _ in range(nset)]
        w = (torch.randn(N, K, device=dev) * 0.02).bfloat16()
        b = torch.randn(N, device=dev).bfloat16()
        wk = w.t().contiguous()
        row = {"case": "short-k", "shape": [M, N, K]}
        mk = lambda f: [(lambda i=i: f(i)) for i in range(nset)]
        row["single_nk_bias"] = _graph_time(mk(lambda i: ops.gemm(xs[i], w, bias=b, out=outs[i], status=st, kernel="single")))
        row["pair256_nk_bias"] = _graph_time(mk(lambda i: ops.gemm_pair(xs[i], w, bias=b, out=outs[i], status=st, tile="256x256")))
        row["pair512_nk_bias"] = _graph_time(mk(lambda i: ops.gemm_pair(xs[i], w, bias=b, out=outs[i], status=st)))
        row["library_nk_bias"] = _graph_time(mk(lambda i: torch.addmm(b, xs[i], w.t(), out=outs[i])))
        row["single_kn"] = _graph_time(mk(lambda i: ops.gemm(xs[i], wk, b_layout="kn", out=outs[i], status=st, kernel="single")))
        row["pair256_kn"] = _graph_time(mk(lambda i: ops.gemm_pair(xs[i], wk, b_layout="kn", out=outs[i], status=st, tile="256x256")))
        row["pair512_kn"] = _graph_time(mk(lambda i: ops.gemm_pair(xs[i], wk, b_layout="kn", out=outs[i], status=st)))
        row["library_kn"] = _graph_time(mk(lambda i: torch.matmul(xs[i], wk, out=outs[i])))
        row["auto_pick"] = ops.pick_gemm_kernel(M, N, K)
        print(json.dumps({k: (round(v, 4) if isinstance(v, float) else v) for k, v in row.items()}), flush=True)
    if st.read():
        raise SystemExit(f"a device wait timed out (status {st.read()})")


def head_case():
    """Output head alone on 8192 rows: fused head + cross-entropy forward (logits stored / not stored), with the in-place
    dlogits, against the plain pair GEMM that only stores the logits, and the library GEMM (back-to-back launches)."""
    from opaque_b200 import ops
    dev = torch.device("cuda", 0)
    st = ops.StatusWord(dev)

    def run(fn, n=8, w=2):
        for _ in range(w):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / n
    for M, K, V in [(8192, 768, 50257), (8192, 4096, 128256)]:
        h = torch.randn(M, K, device=dev).bfloat16()
        w = (torch.randn(V, K, device=dev) * 0.02).bfloat16()
        lab = torch.randint(0, V, (M,), device=dev)
        buf = torch.empty(M, (V + 7) // 8 * 8, device=dev, dtype=torch.bfloat16)
        rw = torch.ones(M, device=dev)

        def fused():
            nll, lse, lg = ops.linear_ce_forward(h, w, lab, store_logits=True, status=st)
            ops.linear_ce_dlogits_(lg, lab, lse, rw)
        row = {"case": "head", "shape": [M, K, V],
               "fused_fwd_logits_stored": run(lambda: ops.linear_ce_forward(h, w, lab, store_logits=True, status=st)),
               "fused_fwd_nothing_stored": run(lambda: ops.linear_ce_forward(h, w, lab, store_logits=False, status=st)),
               "fused_fwd_plus_dlogits": run(fused),
               "plain_pair_gemm": run(lambda: ops.gemm_pair(h, w, out=buf[:, :V], status=st))}
        if V % 8 == 0:
            row["library_gemm"] = run(lambda: torch.matmul(h, w.t(), out=buf[:, :V]))
        print(json.dumps({k: (round(v, 4) if isinstance(v, float) else v) for k, v in row.items()}), flush=True)
    if st.read():
        raise SystemExit(f"a device wait timed out (status {st.read()})")


def sustained_case(seconds: float = 2.5):
    """Seconds-long back-to-back loops (the power-capped regime of a training step) with SM clock and power sampled by
    nvidia-smi during each loop: pair GEMM, its variants, the gated up-projection, and the library on the same box."""
    import statistics
    import subprocess
    import threading
    import time
    from opaque_b200 import ops
    dev = torch.device("cuda", 0)
    st = ops.StatusWord(dev)

    def sample(fn):
        for _ in range(20):
            fn()
        torch.cuda.synchronize()
        rows = []
        proc = subprocess.Popen(["nvidia-smi", "--query-gpu=clocks.sm,power.draw", "--format=csv,noheader,nounits", "-i", "0",
                                 "-lms", "100"], stdout=subprocess.PIPE, text=True)
        t = threading.Thread(target=lambda: [rows.append(l) for l in proc.stdout], daemon=True)
        t.start()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n, t0 = 0, time.time()
        a.record()
        while time.time() - t0 < seconds:
            for _ in range(20):
                fn()
            n += 20
            torch.cuda.synchronize()
        b.record()
        torch.cuda.synchronize()
        proc.terminate()
        vals = [r.split(",") for r in rows[3:] if r.strip()]
        clk = statistics.median(float(v[0]) for v in vals) if vals else 0.0
        pw = statistics.median(float(v[1]) for v in vals) if vals else 0.0
        return a.elapsed_time(b) / n, clk, pw
    for M, N, K in [(16384, 4096, 4096), (16384, 14336, 4096)]:
        x = torch.randn(M, K, device=dev).bfloat16()
        w = (torch.randn(N, K, device=dev) * 0.02).bfloat16()
        wk = w.t().contiguous()
        fl = 2.0 * M * N * K
        for name, fn in (("pair 512x256", lambda: ops.gemm_pair(x, w, status=st)), ("library", lambda: torch.matmul(x, w.t())),
                         ("pair 256x256", lambda: ops.gemm_pair(x, w, status=st, tile="256x256")),
                         ("single CTA", lambda: ops.gemm(x, w, status=st, kernel="single")),
                         ("gate+up+SwiGLU fused", lambda: ops.gemm_glu(x, w[: N // 2], w[N // 2:], status=st)),
                         ("two library GEMMs + SwiGLU kernel", lambda: ops.swiglu(torch.matmul(x, w[: N // 2].t()), torch.matmul(x, w[N // 2:].t()))),
                         ("pair 512x256, [K,N] operand", lambda: ops.gemm_pair(x, wk, b_layout="kn", status=st)),
                         ("library, [K,N] operand", lambda: torch.matmul(x, wk))):
            ms, clk, pw = sample(fn)
            print(json.dumps({"case": "sustained", "shape": [M, N, K], "kernel": name, "tflops": round(fl / ms / 1e9), "sm_mhz": clk,
                              "watts": round(pw, 1), "tflops_per_ghz": round(fl / ms / 1e9 / (clk / 1000)) if clk else None}), flush=True)
    if st.read():
        raise SystemExit(f"a device wait timed out (status {st.read()})")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", default="all")
    ap.add_argument("--small", action="store_true", help="one or two launches of a small case (for ncu)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"],
                    help="reference: time the reference's unmodified kernels (baseline/_ref) on the comparison shapes")
    args = ap.parse_args()
    if args.impl == "reference":
        return compare_cases("reference")
    if args.case == "compare":
        return compare_cases("ours")
    if args.case == "pair-small":
        return pair_small_case()
    if args.case == "short-k":
        return short_k_case()
    if args.case == "head":
        return head_case()
    if args.case == "sustained":
        return sustained_case()
    if args.case == "wgrad-rs":
        return fused_reduce_scatter_case()
    from opaque_b200 import ops
    from opaque_b200.ops.functional import cross_entropy_fused_
    dev = torch.device("cuda", 0)
    tf_peak, bw_peak, tag = peaks()
    flush = torch.zeros(64 * 1024 * 1024, device=dev)     # 256 MB > 126 MB L2
    st = ops.StatusWord(dev)
    iters, warm = (1, 1) if args.small else (20, 5)

    def emit(name, ms, flops=None, bytes_=None, **extra):
        row = {"kernel": name, "ms": round(ms, 4), **extra}
        if flops:
            row["tflops"] = round(flops / ms / 1e9, 1)
            row["frac_" + tag.replace(" ", "_")] = round(flops / ms / 1e9 / tf_peak, 3)
        if bytes_:
            row["GBs"] = round(bytes_ / ms / 1e6, 1)
            row["frac_" + tag.replace(" ", "_")] = round(bytes_ / ms / 1e6 / bw_peak, 3)
        print(json.dumps(row), flush=True)

    want = lambda c: args.case in ("all", c)
    if want("wgrad"):
        shapes = [(16384, 4096, 2048)] if args.small else [(16384, 3072, 768), (16384, 768, 3072), (32768, 4096, 4096), (16384, 8192, 2048)]
        for T, M, N in shapes:
            a = torch.randn(T, M, device=dev).bfloat16()
            b = torch.randn(T, N, device=dev).bfloat16()
            out = torch.zeros(M * N, device=dev)
            sc = torch.rand(T, device=dev)
            fl = 2.0 * T * M * N
            emit(f"wgrad_clip scaled {T}x{M}x{N}", timeit(lambda: ops.wgrad_clip(a, b, out, ldm=N, row_scale=sc, status=st), iters, warm, flush), fl)
            emit(f"wgrad_clip unscaled {T}x{M}x{N}", timeit(lambda: ops.wgrad_clip(a, b, out, ldm=N, status=st), iters, warm, flush), fl)
            exs = torch.rand(T // 1024, device=dev)
            emit(f"wgrad_clip per-example factor in epilogue {T}x{M}x{N}", timeit(lambda: ops.wgrad_clip_per_example(a, b, out, ex_scale=exs, rows_per_example=1024, ldm=N, status=st), iters, warm, flush), fl)
            if not args.small:
                emit(f"cublas a^T b (bf16 out) {T}x{M}x{N}", timeit(lambda: torch.matmul(a.t(), b), iters, warm, flush), fl)
                emit(f"prescale pass + cublas {T}x{M}x{N}", timeit(lambda: torch.matmul((a * sc[:, None].bfloat16()).t(), b), iters, warm, flush), fl)
    if want("gemm"):
        # forward / data-gradient products of the model path: y = x W^T (+ LoRA segment), dX = dY W, grouped experts
        shapes = [(8192, 4096, 4096)] if args.small else [(16384, 4096, 4096), (16384, 14336, 4096), (16384, 4096, 14336), (16384, 768, 3072)]
        for M, N, K in shapes:
            x = torch.randn(M, K, device=dev).bfloat16()
            w = (torch.randn(N, K, device=dev) * 0.02).bfloat16()
            xa = torch.randn(M, 16, device=dev).bfloat16()
            lb = torch.randn(N, 16, device=dev).bfloat16()
            fl = 2.0 * M * N * K
            emit(f"gemm x W^T {M}x{N}x{K}", timeit(lambda: ops.gemm(x, w, status=st), iters, warm, flush), fl)
            emit(f"gemm x W^T + LoRA r16 (one pass) {M}x{N}x{K}", timeit(lambda: ops.gemm(x, w, a2=xa, b2=lb, status=st), iters, warm, flush), fl)
            if not args.small:
                emit(f"cublas x W^T {M}x{N}x{K}", timeit(lambda: torch.matmul(x, w.t()), iters, warm, flush), fl)
                y0 = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
                emit(f"cublas x W^T then addmm LoRA {M}x{N}x{K}", timeit(lambda: torch.addmm(torch.matmul(x, w.t(), out=y0), xa, lb.t(), out=y0), iters, warm, flush), fl)
                wk = w.t().contiguous()
                emit(f"gemm dY W ([K,N] operand) {M}x{N}x{K}", timeit(lambda: ops.gemm(x, wk, b_layout="kn", status=st), iters, warm, flush), fl)
        if not args.small:
            E, rows, K, N = 60, 32768, 2048, 2816
            offs = torch.linspace(0, rows, E + 1, device=dev).to(torch.int32)
            xg = torch.randn(rows, K, device=dev).bfloat16()
            wg = (torch.randn(E, N, K, device=dev) * 0.02).bfloat16()
            fl = 2.0 * rows * N * K
            emit(f"grouped gemm {E} experts {rows}x{N}x{K}", timeit(lambda: ops.gemm(xg, wg, group_offs=offs, status=st), iters, warm, flush), fl)
            if hasattr(torch, "_grouped_mm"):
                wgt = wg.transpose(1, 2)
                o64 = offs[1:].contiguous()
                emit(f"torch._grouped_mm {E} experts {rows}x{N}x{K}", timeit(lambda: torch._grouped_mm(xg, wgt, offs=o64), iters, warm, flush), fl)
    if want("ghost"):
        shapes = [(8, 512, 768, 768)] if args.small else [(32, 512, 768, 3072), (16, 1024, 2048, 8192), (16, 1024, 4096, 4096)]
        for B, T, Da, Dg in shapes:
            a = torch.randn(B * T, Da, device=dev).bfloat16()
            g = torch.randn(B * T, Dg, device=dev).bfloat16()
            n2 = torch.zeros(B, device=dev)
            nt = (T + 127) // 128
            fl = 2.0 * B * (nt * (nt + 1) / 2) * 128 * 128 * (Da + Dg)
            ops.ghost_set_wide(2)
            emit(f"ghost_norm 128x256 blocks {B}x{T}x{Da}x{Dg}", timeit(lambda: ops.ghost_norm(a, g, n2, T, status=st), iters, warm, flush), fl)
            if not args.small:
                ops.ghost_set_wide(0)
                emit(f"ghost_norm 128x128 blocks {B}x{T}x{Da}x{Dg}", timeit(lambda: ops.ghost_norm(a, g, n2, T, status=st), iters, warm, flush), fl)
            ops.ghost_set_wide(1)
    if want("lora"):
        E, T, M, r = (4, 1024, 4096, 16) if args.small else (16, 1024, 4096, 16)
        a = torch.randn(E * T, M, device=dev).bfloat16()
        b = torch.zeros(E * T, 64, device=dev, dtype=torch.bfloat16)
        b[:, :r] = torch.randn(E * T, r, device=dev).bfloat16()
        seg = torch.arange(0, (E + 1) * T, T, device=dev, dtype=torch.int32)
        out = torch.zeros(E, M * r, device=dev)
        ms = timeit(lambda: ops.wgrad_clip(a, b, out, seg_offsets=seg, num_groups=E, ldm=1, ldn=M, n_valid=r, accumulate=False,
                                           group_stride=M * r, block_n=64, status=st), iters, warm, flush)
        emit(f"per-example LoRA wgrad {E}x{T}x{M}xr{r}", ms, bytes_=a.numel() * 2 + b.numel() * 2 + out.numel() * 4)
    if want("rmsnorm"):
        rows = 8192 if args.small else 65536
        x = torch.randn(rows, 4096, device=dev).bfloat16()
        w = torch.ones(4096, device=dev).bfloat16()
        emit(f"rms_norm fwd {rows}x4096", timeit(lambda: ops.rms_norm(x, w), iters, warm, flush), bytes_=2 * x.numel() * 2)
    if want("rmsnorm") and not args.small:
        xg = x.clone().requires_grad_(True)
        y = ops.rms_norm(xg, w)
        dy = torch.randn_like(y)
        emit(f"rms_norm bwd dx {rows}x4096", timeit(lambda: torch.autograd.grad(y, xg, dy, retain_graph=True), iters, warm, flush), bytes_=3 * x.numel() * 2)
    if want("layernorm"):
        rows_l = 8192 if args.small else 131072
        xl = torch.randn(rows_l, 768, device=dev).bfloat16()
        wl, bl = torch.ones(768, device=dev).bfloat16(), torch.zeros(768, device=dev).bfloat16()
        emit(f"layer_norm fwd {rows_l}x768", timeit(lambda: ops.layer_norm(xl, wl, bl), iters, warm, flush), bytes_=2 * xl.numel() * 2)
    if want("swiglu"):
        rows = 4096 if args.small else 16384
        g = torch.randn(rows, 14336, device=dev).bfloat16()
        u = torch.randn_like(g)
        emit(f"swiglu fwd {rows}x14336", timeit(lambda: ops.swiglu(g, u), iters, warm, flush), bytes_=3 * g.numel() * 2)
    if want("ce"):
        rows = 1024 if args.small else 4096
        z = torch.randn(rows, 128256, device=dev).bfloat16()
        lab = torch.randint(0, 128256, (rows,), device=dev)
        emit(f"cross_entropy fwd+dlogits {rows}x128256", timeit(lambda: cross_entropy_fused_(z, lab), iters, warm, flush), bytes_=2 * z.numel() * 2)
    if want("shard_step"):
        n = (16_000_000 if args.small else 124_000_000) // 8 * 8
        grad, master = torch.zeros(n, device=dev), torch.randn(n, device=dev)
        m, v = torch.zeros(n, device=dev), torch.zeros(n, device=dev)
        pl = torch.zeros(n, device=dev, dtype=torch.bfloat16)
        emit(f"shard_step noise+AdamW-BC {n}", timeit(lambda: ops.shard_step(grad=grad, master=master, m=m, v=v, params_local=pl, seed=1, noise_std=1.0, step=2),
                                                      iters, warm, flush), bytes_=n * (4 * 4 * 2 + 2))
        # pull form: the shard's gradient summed in rank order out of W full-length buffers (here W buffers on this GPU, so
        # the reads cost HBM bandwidth instead of NVLink bandwidth); nothing is cleared by the kernel
        W = 4
        shard = n // W // 8 * 8
        bufs = [torch.randn(n, device=dev) for _ in range(W)]
        table = torch.tensor([b.data_ptr() for b in bufs], dtype=torch.int64, device=dev)
        ms, ss, vs = master[:shard], m[:shard], v[:shard]
        emit(f"shard_step pull x{W} + noise + AdamW-BC {shard}",
             timeit(lambda: ops.shard_step(peer_grad=table, world=W, global_offset=shard, master=ms, m=ss, v=vs, params_local=pl, seed=1,
                                           noise_std=1.0, step=2), iters, warm, flush), bytes_=shard * (4 * W + 4 * 3 * 2 + 2))
    if st.read():
        raise SystemExit(f"a device wait timed out (status {st.read()})")


if __name__ == "__main__":
    main()
