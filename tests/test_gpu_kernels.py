"""sm_100a kernels against plain PyTorch fp32 references (run on a B200: ``pytest -m gpu``)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    from opaque_b200.ops import lib
    assert lib.available(), "the sm_100a kernel library must load on a GPU machine"
    return torch.device("cuda", 0)


def rel(x, y):
    return float((x.float() - y.float()).norm() / (y.float().norm() + 1e-30))


def rz_bf16(x):
    """Round fp32 toward zero to bf16 precision (what the clip GEMM does to row factors)."""
    return (x.contiguous().view(torch.int32) & -65536).view(torch.float32)


@pytest.mark.parametrize("T,M,N,bn", [(256, 128, 64, 64), (512, 128, 128, 128), (1024, 256, 256, 256),
                                      (1000, 200, 328, 256), (4096, 768, 3072, 256), (8192, 2048, 1024, 256)])
def test_wgrad_clip_matches_reference(dev, T, M, N, bn):
    from opaque_b200 import ops
    torch.manual_seed(T + M)
    st = ops.StatusWord(dev)
    a = torch.randn(T, M, device=dev).bfloat16()
    b = torch.randn(T, N, device=dev).bfloat16()
    out = torch.zeros(M * N + 16, device=dev)
    ops.wgrad_clip(a, b, out, out_offset=16, ldm=N, block_n=bn, status=st)
    ref = ops.wgrad_clip_ref(a, b)[0]
    assert st.read() == 0 and rel(out[16:].view(M, N), ref) < 2e-5 and float(out[:16].abs().max()) == 0
    # accumulate on top, with per-row clip factors (bf16 round-toward-zero factor, bf16 product)
    sc = torch.rand(T, device=dev)
    ops.wgrad_clip(a, b, out, out_offset=16, ldm=N, row_scale=sc, block_n=bn, status=st)
    scaled = (a.float() * rz_bf16(sc)[:, None]).bfloat16()
    ref2 = ref + ops.wgrad_clip_ref(scaled, b)[0]
    assert st.read() == 0 and rel(out[16:].view(M, N), ref2) < 2e-5
    # every scaled product is bounded by the unrounded one up to one bf16 ulp
    assert bool((scaled.float().abs() <= (a.float() * sc[:, None]).abs() * (1 + 2 ** -8)).all())


@pytest.mark.parametrize("B,R,M,N", [(2, 64, 128, 256), (5, 128, 200, 328), (16, 512, 768, 3072), (8, 1024, 2048, 1024)])
def test_wgrad_clip_per_example_epilogue_scaling(dev, B, R, M, N):
    from opaque_b200 import ops
    torch.manual_seed(B + R)
    st = ops.StatusWord(dev)
    a = torch.randn(B * R, M, device=dev).bfloat16()
    b = torch.randn(B * R, N, device=dev).bfloat16()
    c = torch.rand(B, device=dev)
    ref = ops.wgrad_clip_ref(a, b, row_scale=c.repeat_interleave(R))[0]
    out = torch.zeros(8 + M * N, device=dev)
    ops.wgrad_clip_per_example(a, b, out, ex_scale=c, rows_per_example=R, out_offset=8, accumulate=False, status=st)
    assert st.read() == 0 and rel(out[8:].view(M, N), ref) < 2e-5 and float(out[:8].abs().max()) == 0
    ops.wgrad_clip_per_example(a, b, out, ex_scale=c, rows_per_example=R, out_offset=8, accumulate=True, status=st)   # split-K + reduce
    assert st.read() == 0 and rel(out[8:].view(M, N), 2 * ref) < 2e-5
    ops.wgrad_clip_per_example(a, b, out, ex_scale=None, rows_per_example=R, out_offset=8, accumulate=False, splits=1, status=st)
    assert rel(out[8:].view(M, N), ops.wgrad_clip_ref(a, b)[0]) < 2e-5


def test_wgrad_clip_is_deterministic_without_split_k(dev):
    from opaque_b200 import ops
    a = torch.randn(2048, 256, device=dev).bfloat16()
    b = torch.randn(2048, 256, device=dev).bfloat16()
    outs = []
    for _ in range(2):
        o = torch.zeros(256 * 256, device=dev)
        ops.wgrad_clip(a, b, o, ldm=256, splits=1)
        outs.append(o)
    assert torch.equal(outs[0], outs[1])


def test_wgrad_clip_grouped_store_modes(dev):
    from opaque_b200 import ops
    st = ops.StatusWord(dev)
    for E, Tper, M, r in [(5, 96, 256, 16), (3, 128, 64, 8), (20, 64, 1024, 16)]:
        a = torch.randn(E * Tper, M, device=dev).bfloat16()
        b = torch.zeros(E * Tper, 64, device=dev, dtype=torch.bfloat16)
        b[:, :r] = torch.randn(E * Tper, r, device=dev).bfloat16()
        seg = torch.arange(0, (E + 1) * Tper, Tper, device=dev, dtype=torch.int32)
        ref = ops.wgrad_clip_ref(a, b[:, :r], seg_offsets=seg, num_groups=E)
        P = M * r + 64
        out = torch.full((E, P), 7.0, device=dev)
        ops.wgrad_clip(a, b, out, seg_offsets=seg, num_groups=E, out_offset=64, ldm=r, ldn=1, n_valid=r,
                       accumulate=False, group_stride=P, block_n=64, status=st)
        assert st.read() == 0 and rel(out[:, 64:].reshape(E, M, r), ref) < 1e-5 and bool((out[:, :64] == 7.0).all())
        out = torch.full((E, P), 7.0, device=dev)
        ops.wgrad_clip(a, b, out, seg_offsets=seg, num_groups=E, out_offset=64, ldm=1, ldn=M, n_valid=r,
                       accumulate=False, group_stride=P, block_n=64, status=st)
        assert st.read() == 0 and rel(out[:, 64:].reshape(E, r, M), ref.transpose(1, 2)) < 1e-5
    with pytest.raises(ValueError):
        ops.wgrad_clip(a, b, torch.zeros(10, device=dev), ldm=64)


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (300, 520, 200), (1024, 768, 3072), (4096, 4096, 1024)])
def test_gemm_layouts_bias_and_low_rank_segment(dev, M, N, K):
    from opaque_b200 import ops
    torch.manual_seed(M + N)
    st = ops.StatusWord(dev)
    a = torch.randn(M, K, device=dev).bfloat16()
    w = (torch.randn(N, K, device=dev) / math.sqrt(K)).bfloat16()
    bias = torch.randn(N, device=dev).bfloat16()
    y = ops.gemm(a, w, status=st)
    assert st.read() == 0 and rel(y, ops.gemm_ref(a, w)) < 4e-3
    y = ops.gemm(a, w, bias=bias, status=st)
    assert rel(y, ops.gemm_ref(a, w, bias=bias)) < 4e-3
    wt = w.t().contiguous()                                   # [K, N]
    y = ops.gemm(a, wt, b_layout="kn", status=st)
    assert st.read() == 0 and rel(y, ops.gemm_ref(a, wt, b_layout="kn")) < 4e-3
    for r in (8, 16, 80):
        xa = torch.randn(M, r, device=dev).bfloat16()
        lb = torch.randn(N, r, device=dev).bfloat16()
        y = ops.gemm(a, w, a2=xa, b2=lb, bias=bias, status=st)
        assert st.read() == 0 and rel(y, ops.gemm_ref(a, w, a2=xa, b2=lb, bias=bias)) < 4e-3


def test_gemm_grouped_by_expert(dev):
    from opaque_b200 import ops
    torch.manual_seed(5)
    st = ops.StatusWord(dev)
    E, K, N = 6, 128, 320
    lens = [0, 37, 128, 300, 0, 129]
    offs = torch.tensor([0] + torch.tensor(lens).cumsum(0).tolist(), dtype=torch.int32, device=dev)
    M = sum(lens)
    a = torch.randn(M, K, device=dev).bfloat16()
    w = (torch.randn(E, N, K, device=dev) / math.sqrt(K)).bfloat16()
    y = torch.full((M, N), 7.0, device=dev).bfloat16()
    ops.gemm(a, w, group_offs=offs, out=y, status=st)
    assert st.read() == 0 and rel(y, ops.gemm_ref(a, w, group_offs=offs)) < 4e-3
    dy = torch.randn(M, N, device=dev).bfloat16()
    dx = ops.gemm(dy, w, b_layout="kn", group_offs=offs, status=st)          # w[e] read as [K'=N, N'=K]
    ref = ops.gemm_ref(dy, w, b_layout="kn", group_offs=offs)       # [M, N] @ [N, K] per group
    assert st.read() == 0 and dx.shape == (M, K) and rel(dx, ref) < 4e-3


def test_tensor_map_kernels_work_from_a_fresh_thread(dev):
    """Worker threads (autograd) have no driver context bound until the library binds one."""
    import threading
    from opaque_b200 import ops
    a = torch.randn(256, 64, device=dev).bfloat16()
    g = torch.randn(256, 128, device=dev).bfloat16()
    got, err = torch.zeros(2, device=dev), []

    def work():
        try:
            ops.ghost_norm(a, g, got, 128)
        except Exception as e:           # noqa: BLE001
            err.append(e)
    t = threading.Thread(target=work)
    t.start()
    t.join()
    torch.cuda.synchronize()
    assert not err, err
    assert rel(got, ops.ghost_norm_ref(a, g, 128)) < 1e-3


@pytest.mark.parametrize("wide", [2, 1, 0])
@pytest.mark.parametrize("B,T,Da,Dg", [(2, 128, 64, 64), (3, 256, 192, 320), (4, 512, 768, 3072), (2, 200, 800, 72), (3, 384, 128, 136),
                                       (2, 1024, 256, 512), (5, 129, 64, 200)])
def test_ghost_norm_matches_gram_and_direct(dev, B, T, Da, Dg, wide):
    from opaque_b200 import ops
    st = ops.StatusWord(dev)
    a = torch.randn(B * T, Da, device=dev).bfloat16()
    g = torch.randn(B * T, Dg, device=dev).bfloat16()
    n2 = torch.zeros(B, device=dev)
    old = ops.ghost_set_wide(wide)
    try:
        ops.ghost_norm(a, g, n2, T, status=st)
    finally:
        ops.ghost_set_wide(old)
    direct = torch.stack([(a[i * T:(i + 1) * T].float().t() @ g[i * T:(i + 1) * T].float()).pow(2).sum() for i in range(B)])
    assert st.read() == 0 and rel(n2, ops.ghost_norm_ref(a, g, T)) < 2e-5 and rel(n2, direct) < 5e-5


def test_ghost_norm_ragged_segments_both_tile_shapes(dev):
    from opaque_b200 import ops
    torch.manual_seed(9)
    lens = [5, 300, 0, 129, 256, 77]
    offs = torch.tensor([0] + torch.tensor(lens).cumsum(0).tolist(), dtype=torch.int32, device=dev)
    rows = sum(lens)
    a = torch.randn(rows, 96, device=dev).bfloat16()
    g = torch.randn(rows, 160, device=dev).bfloat16()
    seg_out = torch.tensor([0, 1, 2, 0, 1, 2], dtype=torch.int32, device=dev)
    want = torch.zeros(3, device=dev)
    for i, (lo, n) in enumerate(zip(offs.tolist(), lens)):
        if n:
            want[i % 3] += (a[lo:lo + n].float().t() @ g[lo:lo + n].float()).pow(2).sum()
    for wide in (2, 0):
        got = torch.zeros(3, device=dev)
        old = ops.ghost_set_wide(wide)
        try:
            ops.ghost_norm(a, g, got, 300, seg_offsets=offs, seg_out=seg_out)
        finally:
            ops.ghost_set_wide(old)
        assert rel(got, want) < 5e-5, wide


def test_ghost_norm_embedding_ids(dev):
    from opaque_b200 import ops
    B, T, D = 3, 256, 128
    g = torch.randn(B * T, D, device=dev).bfloat16()
    ids = torch.randint(0, 20, (B * T,), device=dev, dtype=torch.int32)
    n2 = torch.zeros(B, device=dev)
    ops.ghost_norm(None, g, n2, T, ids=ids)
    assert rel(n2, ops.ghost_norm_ref(None, g, T, ids=ids)) < 1e-5


def test_norm_activation_rope_kernels(dev):
    from opaque_b200 import ops
    torch.manual_seed(0)
    x = torch.randn(512, 1024, device=dev).bfloat16()
    w = (torch.randn(1024, device=dev) * 0.1 + 1).bfloat16()
    r = torch.randn_like(x)
    xg, wg = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    y = ops.rms_norm(xg, wg, 1e-5)
    assert rel(y, ops.rms_norm_ref(x, w, 1e-5)) < 1e-4
    dy = torch.randn_like(y)
    y.backward(dy)
    xr, wr = x.float().requires_grad_(True), w.float().requires_grad_(True)
    (xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-5) * wr).backward(dy.float())
    # bf16 error floor: the kernel may not be worse than 3x the rounding of the fp32 result
    floor = rel(xr.grad.bfloat16(), xr.grad)
    assert rel(xg.grad, xr.grad) < 3 * floor + 1e-6 and rel(wg.grad, wr.grad) < 3 * rel(wr.grad.bfloat16(), wr.grad) + 1e-6
    y2, s2 = ops.fused_add_rms_norm(x, r, w, 1e-5)
    yr2, sr2 = ops.rms_norm_ref(x, w, 1e-5, residual=r)
    assert rel(y2, yr2) < 1e-4 and torch.equal(s2, sr2)
    y3 = ops.rms_norm(x, w, 1e-6, offset=1.0, casting_mode="gemma")
    assert rel(y3, ops.rms_norm_ref(x, w, 1e-6, 1.0, "gemma")) < 1e-4
    g = torch.randn(256, 2048, device=dev).bfloat16().requires_grad_(True)
    u = torch.randn(256, 2048, device=dev).bfloat16().requires_grad_(True)
    for act in (0, 1, 2):
        g.grad = u.grad = None
        h = ops.swiglu(g, u) if act == 0 else ops.geglu(g, u, approximate=(act == 2))
        dh = torch.randn_like(h)
        h.backward(dh)
        gf, uf = g.detach().float().requires_grad_(True), u.detach().float().requires_grad_(True)
        a = torch.nn.functional.silu(gf) if act == 0 else torch.nn.functional.gelu(gf, approximate="tanh" if act == 2 else "none")
        (a * uf).backward(dh.float())
        assert rel(h, a * uf) < 4e-3 and rel(g.grad, gf.grad) < 4e-3 and rel(u.grad, uf.grad) < 4e-3
    q = torch.randn(2, 64, 8, 64, device=dev).bfloat16().requires_grad_(True)
    k = torch.randn(2, 64, 2, 64, device=dev).bfloat16().requires_grad_(True)
    cos, sin = ops.rope_tables(64, 128, 500000.0, device=dev)
    pos = torch.randint(0, 128, (2, 64), device=dev)
    for p in (None, pos):
        q1, k1 = ops.rope_qk(q, k, cos, sin, p)
        q2, k2 = ops.rope_qk_ref(q.detach(), k.detach(), cos, sin, p)
        assert torch.equal(q1, q2) and torch.equal(k1, k2)
    gq = torch.randn_like(q1)
    q.grad = None
    q1.backward(gq)
    back, _ = ops.rope_qk_ref(gq, k.detach(), cos, sin, pos, sign=-1.0)
    assert rel(q.grad, back) < 1e-3
    # strided views are read through their strides: slices of a fused q|k|v buffer, [B, H, T, D]-laid-out tensors
    buf = torch.randn(2, 64, (8 + 2 + 2) * 64, device=dev).bfloat16()
    qv, kv = buf[..., : 8 * 64].view(2, 64, 8, 64), buf[..., 8 * 64: 10 * 64].view(2, 64, 2, 64)
    qt = torch.randn(2, 8, 64, 64, device=dev).bfloat16().transpose(1, 2)
    kt = torch.randn(2, 2, 64, 64, device=dev).bfloat16().transpose(1, 2)
    for qq, kk in ((qv, kv), (qt, kt)):
        assert not qq.is_contiguous()
        q3, k3 = ops.rope_qk(qq, kk, cos, sin, pos)
        q4, k4 = ops.rope_qk_ref(qq.contiguous(), kk.contiguous(), cos, sin, pos)
        assert q3.is_contiguous() and torch.equal(q3, q4) and torch.equal(k3, k4)
    # head sizes the 16-byte kernel does not take fall back to the general one
    q5 = torch.randn(2, 64, 4, 24, device=dev).bfloat16()
    k5 = torch.randn(2, 64, 2, 24, device=dev).bfloat16()
    c5, s5 = ops.rope_tables(24, 128, 10000.0, device=dev)
    a5, b5 = ops.rope_qk(q5, k5, c5, s5, None)
    a6, b6 = ops.rope_qk_ref(q5, k5, c5, s5, None)
    assert rel(a5, a6) < 4e-3 and rel(b5, b6) < 4e-3          # fused multiply-adds round differently from the eager reference


@pytest.mark.parametrize("H", [1024, 2048, 4096, 8192, 1536])
def test_rms_norm_register_resident_widths(dev, H):
    """Widths with a register-resident kernel (and one without), odd row count, with and without the fused residual add."""
    from opaque_b200 import ops
    torch.manual_seed(H)
    rows = 37
    x = torch.randn(rows, H, device=dev).bfloat16()
    r = torch.randn(rows, H, device=dev).bfloat16()
    w = (torch.randn(H, device=dev) * 0.1 + 1).bfloat16()
    xg, wg = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    y = ops.rms_norm(xg, wg, 1e-5)
    assert rel(y, ops.rms_norm_ref(x, w, 1e-5)) < 1e-4
    dy = torch.randn_like(y)
    y.backward(dy)
    xr, wr = x.float().requires_grad_(True), w.float().requires_grad_(True)
    (xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-5) * wr).backward(dy.float())
    assert rel(xg.grad, xr.grad) < 3 * rel(xr.grad.bfloat16(), xr.grad) + 1e-6
    assert rel(wg.grad, wr.grad) < 3 * rel(wr.grad.bfloat16(), wr.grad) + 1e-6
    y2, s2 = ops.fused_add_rms_norm(x, r, w, 1e-5)
    yr2, sr2 = ops.rms_norm_ref(x, w, 1e-5, residual=r)
    assert rel(y2, yr2) < 1e-4 and torch.equal(s2, sr2)
    xa, ra = x.clone().requires_grad_(True), r.clone().requires_grad_(True)
    ya, sa = ops.fused_add_rms_norm(xa, ra, w, 1e-5)
    (ya.float().sum() + 2 * sa.float().sum()).backward()
    xb, rb = x.float().requires_grad_(True), r.float().requires_grad_(True)
    sb = xb + rb
    ((sb * torch.rsqrt(sb.pow(2).mean(-1, keepdim=True) + 1e-5) * w.float()).sum() + 2 * sb.sum()).backward()
    assert rel(xa.grad, xb.grad) < 2e-2 and torch.equal(xa.grad, ra.grad)


def test_layernorm_group_sum_and_activation_kernels(dev):
    from opaque_b200 import ops
    torch.manual_seed(3)
    B, T, H = 4, 96, 768
    x = (torch.randn(B * T, H, device=dev) * 2 + 0.5).bfloat16()
    w = (torch.randn(H, device=dev) * 0.2 + 1).bfloat16()
    b = (torch.randn(H, device=dev) * 0.1).bfloat16()
    xg, wg, bg = (t.clone().requires_grad_(True) for t in (x, w, b))
    y = ops.layer_norm(xg, wg, bg, 1e-5)
    xr, wr, br = (t.float().requires_grad_(True) for t in (x, w, b))
    yr = torch.nn.functional.layer_norm(xr, (H,), wr, br, 1e-5)
    assert rel(y, yr) < 4e-3
    dy = torch.randn_like(y)
    y.backward(dy)
    yr.backward(dy.float())
    assert rel(xg.grad, xr.grad) < 6e-3 and rel(wg.grad, wr.grad) < 6e-3 and rel(bg.grad, br.grad) < 6e-3
    # per-example reductions into a strided fp32 destination, accumulating
    g = torch.randn(B * T, 3072, device=dev).bfloat16()
    out = torch.ones(B, 4000, device=dev)
    ops.rows_group_sum_(out[:, 100:3172], g, B)
    assert rel(out[:, 100:3172], 1 + g.float().view(B, T, -1).sum(1)) < 1e-5 and float(out[:, :100].min()) == 1.0
    for kind in ("silu", "gelu", "gelu_tanh", "relu"):
        a = torch.randn(512, 3072, device=dev).bfloat16().requires_grad_(True)
        o = ops.activation(a, kind)
        da = torch.randn_like(o)
        o.backward(da)
        af = a.detach().float().requires_grad_(True)
        of = {"silu": torch.nn.functional.silu, "relu": torch.relu, "gelu": torch.nn.functional.gelu,
              "gelu_tanh": lambda t: torch.nn.functional.gelu(t, approximate="tanh")}[kind](af)
        of.backward(da.float())
        assert rel(o, of) < 4e-3 and rel(a.grad, af.grad) < 4e-3, kind


@pytest.mark.parametrize("V,dt", [(1000, torch.bfloat16), (50257, torch.float32), (128256, torch.bfloat16)])
def test_cross_entropy_kernel(dev, V, dt):
    from opaque_b200 import ops
    z = (torch.randn(64, V, device=dev) * 3).to(dt)
    lab = torch.randint(0, V, (64,), device=dev)
    lab[::7] = -100
    zf = z.detach().float().clone().requires_grad_(True)
    nr = ops.cross_entropy_ref(zf, lab)
    nr.sum().backward()
    zz = z.detach().clone().requires_grad_(True)
    n = ops.cross_entropy(zz, lab)
    n.sum().backward()
    assert rel(n, nr) < 1e-5 and rel(zz.grad, zf.grad) < (5e-3 if dt == torch.bfloat16 else 1e-5)
    assert float(n[::7].abs().max()) == 0 and float(zz.grad[::7].abs().max()) == 0


def test_cross_entropy_options(dev):
    from opaque_b200 import ops
    z = (torch.randn(32, 4096, device=dev) * 3).bfloat16()
    lab = torch.randint(0, 4096, (32,), device=dev)
    kw = dict(logit_softcapping=30.0, logit_scaling=0.5, label_smoothing=0.1)
    zf = z.float().requires_grad_(True)
    nr = ops.cross_entropy_ref(zf, lab, **kw)
    nr.sum().backward()
    zz = z.clone().requires_grad_(True)
    n = ops.cross_entropy(zz, lab, **kw)
    n.sum().backward()
    assert rel(n, nr) < 1e-4 and rel(zz.grad, zf.grad) < 5e-3


def test_philox_statistics_and_layout_independence(dev):
    from opaque_b200 import ops
    x = torch.zeros(4_000_003, device=dev)
    ops.philox_normal_add_(x, seed=123, offset=5, std=2.0)
    assert abs(float(x.mean())) < 5e-3 and abs(float(x.std()) - 2.0) < 5e-3
    assert abs(float(((x / 2.0) ** 4).mean()) - 3.0) < 0.03
    from scipy import stats
    assert stats.kstest((x[:200_000] / 2.0).cpu().numpy(), "norm").pvalue > 1e-3
    # a coordinate's noise depends on (seed, global index) only: any split reproduces it exactly once
    parts = []
    for lo, hi in [(5, 1001), (1001, 1002), (1002, 70_001)]:
        y = torch.zeros(hi - lo, device=dev)
        ops.philox_normal_add_(y, seed=123, offset=lo, std=2.0)
        parts.append(y)
    assert torch.equal(torch.cat(parts), x[:69_996])
    z = torch.zeros(1000, device=dev)
    ops.philox_normal_add_(z, seed=124, offset=5, std=2.0)
    assert abs(float((z * x[:1000]).mean())) < 0.5      # different keys are uncorrelated


def test_direct_path_kernels(dev):
    from opaque_b200 import ops
    g = torch.randn(6, 10_000, device=dev)
    n2 = torch.zeros(6, device=dev)
    ops.rows_sumsq(g, n2)
    assert rel(n2, (g ** 2).sum(1)) < 1e-6
    c = torch.rand(6, device=dev)
    out = torch.zeros(20_000, device=dev)
    ops.clip_weighted_sum(g, c, out, flat_offset=4000)
    assert rel(out[4000:14_000], c @ g) < 1e-6 and float(out[:4000].abs().max()) == 0
    gg = torch.randn(300, 64, device=dev).bfloat16()
    ids = torch.randint(0, 50, (300,), device=dev)
    sc = torch.rand(300, device=dev)
    out = torch.zeros(50 * 64 + 8, device=dev)
    ops.embedding_wgrad(gg, ids, out, row_scale=sc, flat_offset=8)
    ref = torch.zeros(50, 64, device=dev).index_add_(0, ids, gg.float() * sc[:, None])
    assert rel(out[8:].view(50, 64), ref) < 1e-6


def test_shard_step_adamw_noise_and_ftrl_modes(dev):
    from opaque_b200 import ops
    n = 10_007
    grad, master = torch.randn(n, device=dev), torch.randn(n, device=dev)
    m, v = torch.zeros(n, device=dev), torch.zeros(n, device=dev)
    pl = torch.zeros(n + 64, device=dev, dtype=torch.bfloat16)
    wt = torch.nn.Parameter(master.clone())
    opt = torch.optim.AdamW([wt], lr=1e-2, weight_decay=0.1)
    for step in range(1, 4):
        gs = torch.randn(n, device=dev)
        grad.copy_(gs * 4)
        wt.grad = gs.clone()
        opt.step()
        ops.shard_step(grad=grad, master=master, m=m, v=v, params_local=pl, global_offset=64, inv_normalize=0.25,
                       lr=1e-2, weight_decay=0.1, step=step)
    assert rel(master, wt.detach()) < 1e-6 and rel(pl[64:], wt.detach()) < 3e-3 and float(grad.abs().max()) == 0
    no = torch.zeros(n, device=dev)
    ops.shard_step(grad=grad, master=master, m=m, v=v, global_offset=64, seed=77, noise_std=3.0, inv_normalize=0.5,
                   noisy_out=no, skip_update=True)
    ref = torch.zeros(n, device=dev)
    ops.philox_normal_add_(ref, seed=77, offset=64, std=1.5)
    assert torch.equal(no, ref)
    # noise bias correction: phi_hat is removed from the second moment where that stays positive
    m.zero_(); v.zero_(); master.fill_(1.0); grad.fill_(0.2)
    ops.shard_step(grad=grad, master=master, m=m, v=v, lr=1.0, betas=(0.0, 0.0), eps=0.0, step=1, phi_hat=0.03)
    assert abs(float(master[0]) - (1.0 - 0.2 / math.sqrt(0.04 - 0.03))) < 1e-4

    def draws(seed):
        z = torch.zeros(n, device=dev)
        ops.philox_normal_add_(z, seed=seed, offset=0, std=1.0)
        return z
    s, d = [0.3, 0.2, 0.1], [0.9, 0.5, 0.1]
    state, sref = torch.zeros(3, n, device=dev), torch.zeros(3, n, device=dev)
    for t in range(4):
        grad.zero_()
        ops.shard_step(grad=grad, master=master, m=m, v=v, seed=100 + t, noise_std=1.0, noisy_out=no, skip_update=True,
                       ftrl_state=state, ftrl_mode=1, ftrl_coef=s + d, nbuf=3)
        x = draws(100 + t) - sum(s[j] * sref[j] for j in range(3))
        for j in range(3):
            sref[j] = d[j] * sref[j] + x
        assert float((no - x).abs().max()) < 1e-5
    coef, hist, zs = [1.0, 0.5, 0.25], [], []
    st_iir, st_fir = torch.zeros(2, n, device=dev), torch.zeros(2, n, device=dev)
    for t in range(5):
        z = draws(200 + t)
        grad.zero_()
        ops.shard_step(grad=grad, master=master, m=m, v=v, seed=200 + t, noise_std=1.0, noisy_out=no, skip_update=True,
                       ftrl_state=st_iir, ftrl_mode=2, ftrl_coef=coef, nbuf=2, ring_head=t % 2)
        x = (z - sum(coef[k] * hist[-k] for k in (1, 2) if len(hist) >= k)) / coef[0]
        hist.append(x)
        assert float((no - x).abs().max()) < 1e-5
        grad.zero_()
        ops.shard_step(grad=grad, master=master, m=m, v=v, seed=200 + t, noise_std=1.0, noisy_out=no, skip_update=True,
                       ftrl_state=st_fir, ftrl_mode=3, ftrl_coef=coef, nbuf=2, ring_head=t % 2)
        y = coef[0] * z + sum(coef[k] * zs[-k] for k in (1, 2) if len(zs) >= k)
        zs.append(z)
        assert float((no - y).abs().max()) < 1e-5


def test_bounded_wait_reports_timeout_without_hanging(dev):
    """A peer flag that nothing sets: the barrier kernel gives up after its budget and records a status."""
    import ctypes
    from opaque_b200.ops import lib
    st = lib.StatusWord(dev)
    flags = torch.zeros(64, dtype=torch.int32, device=dev)
    table = torch.tensor([flags.data_ptr(), flags.data_ptr()], dtype=torch.int64, device=dev)
    # two "ranks" aliasing one array: rank 0 publishes slot 0, slot 1 is never written
    rc = lib.load().ob_peer_barrier(table.data_ptr(), flags.data_ptr(), 0, 2, 1, st.ptr(), 0.05, lib.stream())
    assert rc == 0
    torch.cuda.synchronize()
    assert st.read() == 6
    with pytest.raises(lib.DeviceWaitTimeout):
        st.raise_if_set("test")
    assert st.read() == 0 and float(torch.ones(4, device=dev).sum()) == 4.0     # the context is still usable


@pytest.mark.gpu
@pytest.mark.parametrize("H", [64, 256, 264, 512, 768, 1000, 1024, 1536, 4096, 5120])
def test_layer_norm_all_row_widths(dev, H):
    """Warp-per-row (H <= 1024), CTA-per-row-pair (H <= 4096) and streaming LayerNorm kernels against fp32 torch,
    with a row count that leaves the last CTA partly empty."""
    from opaque_b200 import ops
    torch.manual_seed(H)
    rows = 203
    x = (torch.randn(rows, H, device=dev) * 1.5 - 0.3).bfloat16()
    w = (torch.randn(H, device=dev) * 0.2 + 1).bfloat16()
    b = (torch.randn(H, device=dev) * 0.1).bfloat16()
    xg = x.clone().requires_grad_(True)
    y = ops.layer_norm(xg, w, b, 1e-5)
    xr = x.float().requires_grad_(True)
    yr = torch.nn.functional.layer_norm(xr, (H,), w.float(), b.float(), 1e-5)
    assert rel(y, yr) < 4e-3
    dy = torch.randn_like(y)
    y.backward(dy)
    yr.backward(dy.float())
    assert rel(xg.grad, xr.grad) < 6e-3


@pytest.mark.gpu
def test_layernorm_weight_and_bias_sums_in_one_pass_and_head_merge(dev):
    from opaque_b200 import ops
    torch.manual_seed(11)
    B, T, H = 3, 160, 768
    g = torch.randn(B * T, H, device=dev).bfloat16()
    x = (torch.randn(B * T, H, device=dev) * 2 + 1).bfloat16()
    mean, rstd = x.float().mean(1), (x.float().var(1, unbiased=False) + 1e-5).rsqrt()
    dw, db = torch.zeros(B, H, device=dev), torch.full((B, H + 8), 2.0, device=dev)
    ops.rows_group_sum_(dw, g, B, x2d=x, mean=mean, rstd=rstd, out_plain=db[:, 4:4 + H])
    xh = (x.float() - mean[:, None]) * rstd[:, None]
    assert rel(dw, (g.float() * xh).view(B, T, H).sum(1)) < 1e-5
    assert rel(db[:, 4:4 + H], 2 + g.float().view(B, T, H).sum(1)) < 1e-5 and float(db[:, :4].min()) == 2.0
    # gradient gather of the fused q/k/v projection: sources in two different layouts
    heads, hd = 12, 64
    gq = torch.randn(B, heads, T, hd, device=dev).bfloat16()                                  # [B, H, T, hd] contiguous
    gk = torch.randn(B, T, heads, hd, device=dev).bfloat16().transpose(1, 2)                  # [B, T, H, hd] memory
    big = torch.randn(B, T, 3, heads, hd, device=dev).bfloat16()
    gv = big[:, :, 2].transpose(1, 2)                                                        # a slice of a fused buffer
    out = ops.merge_heads3(gq, gk, gv)
    ref = torch.stack([t.transpose(1, 2) for t in (gq, gk, gv)], dim=2).reshape(B, T, 3 * heads * hd)
    assert torch.equal(out, ref)


def test_philox_gaussian_tails_follow_the_normal_law(dev):
    """Tail mass of the device Gaussian over 1e9 draws: P(|z| > 4) and P(|z| > 5) against the normal law, and the cut.

    The radius of the Box-Muller pair uses 32 uniform bits, so no draw exceeds sqrt(-2 ln 2^-33) = 6.76 standard
    deviations.  (The reference's CPU sampler clamps its uniform to [eps, 1 - eps] of its compute dtype, fp32: a cut at
    5.2 standard deviations, packages/opaque-dpsgd/src/opaque/api/dpsgd/noise/_gaussian.py:257-264.)
    """
    from opaque_b200 import ops
    n_chunk, chunks = 250_000_000, 4
    over4 = over5 = 0
    top = 0.0
    s1 = s2 = 0.0
    buf = torch.empty(n_chunk, device=dev)
    for c in range(chunks):
        buf.zero_()
        ops.philox_normal_add_(buf, seed=20240611, offset=c * n_chunk, std=1.0)
        a = buf.abs()
        over4 += int((a > 4.0).sum())
        over5 += int((a > 5.0).sum())
        top = max(top, float(a.max()))
        s1 += float(buf.double().sum())
        s2 += float((buf.double() ** 2).sum())
    n = n_chunk * chunks
    p4, p5 = math.erfc(4 / math.sqrt(2)), math.erfc(5 / math.sqrt(2))          # two-sided tail mass
    for got, p in ((over4, p4), (over5, p5)):
        sd = math.sqrt(n * p)
        assert abs(got - n * p) < 5 * sd, (got, n * p, sd)
    assert 5.5 < top <= 6.77
    assert abs(s1 / n) < 5 / math.sqrt(n) and abs(s2 / n - 1.0) < 5 * math.sqrt(2.0 / n)


@pytest.mark.parametrize("name", ["identity", "mf_band16", "mf_blt10", "mf_bsr8", "mf_bisr4", "mf_lambda_cgd"])
def test_fused_correlated_noise_equals_the_streaming_path_for_every_strategy(dev, name):
    """The fused shard step's correlated noise (any history length) against the strategy's streaming ``C⁻¹`` applied to the
    SAME Philox draws, over 50 steps; the mechanism dictionary comes from the strategy's own ``fused_mechanism``."""
    from opaque_b200 import dpftrl, ops
    from opaque_b200.parallel.peer import PeerGroup
    from opaque_b200.parallel.sharded import DPStepConfig, FlatSpace, ShardedDPOptimizer
    from opaque_b200.random import fold_in, key
    steps = 50
    strat = {"identity": lambda: dpftrl.identity_strategy(), "mf_band16": lambda: dpftrl.band_mf_strategy(bands=16),
             "mf_blt10": lambda: dpftrl.blt_strategy(max_buffers=10), "mf_bsr8": lambda: dpftrl.bsr_strategy(bandwidth=8),
             "mf_bisr4": lambda: dpftrl.bisr_strategy(bandwidth=4),
             "mf_lambda_cgd": lambda: dpftrl.lambda_cgd_strategy(lambda_=0.7, normalized=True)}[name]()
    p = torch.nn.Parameter(torch.zeros(1024, 8, device=dev, dtype=torch.bfloat16))
    space = FlatSpace([("w", p)], PeerGroup(dev))
    space.bind()
    k = key(11)
    mech = strat.fused_mechanism(steps)
    opt = ShardedDPOptimizer(space, DPStepConfig(lr=0.0), key=k, mechanism=mech)
    if name in ("mf_band16", "mf_blt10"):
        assert opt.nbuf > 8                                    # beyond the unrolled fast path
    sm = strat.streaming_matrix(steps)
    n = space.shard
    state = sm.init_multiply(torch.zeros(n, device=dev))
    out = torch.zeros(n, device=dev)
    worst = 0.0
    for t in range(steps):
        z = torch.zeros(n, device=dev)
        ops.philox_normal_add_(z, seed=fold_in(k, t).seed, offset=0, std=1.0)
        want, state = sm.multiply_next(z, state)
        opt.step(noise_std=1.0, normalize_by=1.0, noisy_out=out, skip_update=True)
        worst = max(worst, float((out - want).abs().max()) / (float(want.abs().max()) + 1e-12))
    assert worst < 2e-4, worst


@pytest.mark.parametrize("B,T,Da,Dg", [(3, 64, 96, 200), (2, 4096, 128, 256), (5, 256, 768, 768), (4, 512, 136, 72)])
def test_direct_per_example_norms_match_the_products(dev, B, T, Da, Dg):
    """``‖A_eᵀ G_e‖²`` from the product kernel's norm epilogue against fp32 products, and against the Gram-matrix kernel."""
    from opaque_b200 import ops
    torch.manual_seed(B * T + Da)
    a = torch.randn(B * T, Da, device=dev).bfloat16()
    g = (torch.randn(B * T, Dg, device=dev) / math.sqrt(T)).bfloat16()
    st = ops.StatusWord(dev)
    n2 = torch.full((B,), 0.5, device=dev)                     # the kernel ADDS
    ops.direct_norm2(a, g, n2, T, status=st)
    want = torch.stack([(a[e * T:(e + 1) * T].float().t() @ g[e * T:(e + 1) * T].float()).square().sum() for e in range(B)])
    assert st.read() == 0 and rel(n2 - 0.5, want) < 2e-3
    ghost = torch.zeros(B, device=dev)
    ops.ghost_norm(a, g, ghost, T, status=st)
    assert rel(ghost, want) < 2e-3
    for splits in (1, B):
        n3 = torch.zeros(B, device=dev)
        ops.direct_norm2(a, g, n3, T, splits=splits, status=st)
        assert rel(n3, want) < 2e-3
    assert ops.pick_norm_path(4096, 128, 256) == "direct" and ops.pick_norm_path(512, 4096, 4096) == "ghost"
    assert ops.pick_norm_path(4100, 128, 256) == "ghost"       # not a multiple of 64 rows


@pytest.mark.parametrize("name,kw", [("sgd", dict(momentum=0.0)), ("sgd", dict(momentum=0.9)), ("sgd", dict(momentum=0.9, nesterov=True)),
                                     ("lion", dict(betas=(0.9, 0.99)))])
def test_shard_step_sgd_and_lion_match_the_functional_optimizers(dev, name, kw):
    """The fused update for SGD (momentum, Nesterov, L2 decay in the gradient) and Lion (decoupled decay) against the
    functional optimizer chain over several noiseless steps."""
    from opaque_b200 import ops, optimizers as O
    torch.manual_seed(5)
    n, lr, wd = 4096, 0.05, 0.01
    w0 = torch.randn(n, device=dev)
    grads = [torch.randn(n, device=dev) for _ in range(5)]
    if name == "sgd":
        opt = O.sgd(lr, momentum=kw["momentum"], weight_decay=wd, nesterov=kw.get("nesterov", False))
        betas, dec = (kw["momentum"], 0.0), False
    else:
        opt = O.lion(lr, kw["betas"], wd)
        betas, dec = kw["betas"], True
    params = {"w": w0.clone()}
    state = opt.init(params)
    master, m, v = w0.clone(), torch.zeros(n, device=dev), torch.zeros(n, device=dev)
    for t, g in enumerate(grads, start=1):
        upd, state = opt.update({"w": g}, state, params=params)
        params = O.apply_updates(params, upd)
        ops.shard_step(grad=g.clone(), master=master, m=m, v=v, lr=lr, betas=betas, weight_decay=wd, step=t, decoupled_wd=dec,
                       optimizer=name, nesterov=kw.get("nesterov", False))
        assert torch.allclose(master, params["w"], rtol=2e-5, atol=2e-6), (name, kw, t)


@pytest.mark.parametrize("world", [1, 3, 8, 11])
def test_shard_step_pull_form_sums_rank_buffers_in_rank_order(dev, world):
    """The pull form of the fused shard step: the shard's gradient is read out of ``world`` full-length accumulation
    buffers (here all on one GPU: plain loads, no kernel waits on another) and added in rank order.  The result equals
    the ordinary step fed with that rank-ordered sum BIT FOR BIT, twice in a row, and the buffers are left as they were."""
    from opaque_b200 import ops
    torch.manual_seed(3)
    total, lo, n = 8192 + 2048, 2048, 4096 + 8 * 3 + 3          # a shard in the middle of the flat space
    bufs = [torch.randn(total, device=dev) * (10.0 ** (r % 3 - 1)) for r in range(world)]
    table = torch.tensor([b.data_ptr() for b in bufs], dtype=torch.int64, device=dev)
    ordered = torch.zeros(n, device=dev)
    for b in bufs:
        ordered += b[lo:lo + n]
    keep = [b.clone() for b in bufs]
    w0 = torch.randn(n, device=dev)
    results = []
    for form in ("pull", "pull", "push"):
        master, m, v = w0.clone(), torch.zeros(n, device=dev), torch.zeros(n, device=dev)
        pl = torch.zeros(total, device=dev, dtype=torch.bfloat16)
        noisy = torch.empty(n, device=dev)
        kw = dict(master=master, m=m, v=v, params_local=pl, global_offset=lo, seed=9, noise_std=0.5, inv_normalize=0.125,
                  lr=1e-2, weight_decay=0.1, step=1, phi_hat=1e-3, noisy_out=noisy)
        if form == "pull":
            ops.shard_step(peer_grad=table, world=world, **kw)
        else:
            ops.shard_step(grad=ordered.clone(), **kw)
        results.append((master, m, v, pl, noisy))
    for a, b in zip(results[0], results[1]):
        assert torch.equal(a, b)
    for a, b in zip(results[0], results[2]):
        assert torch.equal(a, b)
    assert all(torch.equal(b, k) for b, k in zip(bufs, keep))
    with pytest.raises(ValueError):
        ops.shard_step(master=w0, m=w0, v=w0)
