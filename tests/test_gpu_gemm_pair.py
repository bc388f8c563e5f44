"""The CTA-pair GEMM (tcgen05 cta_group::2) against fp32 PyTorch references (run on a B200: ``pytest -m gpu``)."""
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


@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (128, 256, 128), (300, 520, 200), (1000, 136, 72), (1024, 768, 3072),
                                   (4096, 4096, 1024), (2048, 1536, 8192)])
@pytest.mark.parametrize("tile", ["512x256", "256x256"])
def test_pair_gemm_layouts_bias_segments(dev, M, N, K, tile):
    from opaque_b200 import ops as _ops
    import functools
    import types
    # both tile variants must satisfy the same contract
    ops = types.SimpleNamespace(**{k: getattr(_ops, k) for k in ("StatusWord", "gemm_ref", "gemm")},
                                gemm_pair=functools.partial(_ops.gemm_pair, tile=tile))
    torch.manual_seed(M + N + K)
    st = ops.StatusWord(dev)
    a = torch.randn(M, K, device=dev).bfloat16()
    w = (torch.randn(N, K, device=dev) / math.sqrt(K)).bfloat16()
    bias = torch.randn(N, device=dev).bfloat16()
    y = torch.full((M + 1, N), 7.0, device=dev).bfloat16()
    ops.gemm_pair(a, w, out=y[:M], status=st)
    assert st.read() == 0 and rel(y[:M], ops.gemm_ref(a, w)) < 4e-3 and bool((y[M] == 7.0).all())     # no write past row M
    assert rel(ops.gemm_pair(a, w, bias=bias, status=st), ops.gemm_ref(a, w, bias=bias)) < 4e-3
    wt = w.t().contiguous()                                   # [K, N]
    y = ops.gemm_pair(a, wt, b_layout="kn", status=st)
    assert st.read() == 0 and rel(y, ops.gemm_ref(a, wt, b_layout="kn")) < 4e-3
    for r in (8, 16, 80):
        xa = torch.randn(M, r, device=dev).bfloat16()
        lb = torch.randn(N, r, device=dev).bfloat16()
        y = ops.gemm_pair(a, w, a2=xa, b2=lb, bias=bias, status=st)
        assert st.read() == 0 and rel(y, ops.gemm_ref(a, w, a2=xa, b2=lb, bias=bias)) < 4e-3
        # data gradient of a LoRA linear: dY W + q A with both operands stored [K, N]
        la = torch.randn(r, N, device=dev).bfloat16()
        y = ops.gemm_pair(a, wt, b_layout="kn", a2=xa, b2=la, b2_layout="kn", status=st)
        ref = a.float() @ wt.float() + xa.float() @ la.float()
        assert st.read() == 0 and rel(y, ref) < 4e-3
    # two full-width [K, N] segments: dX = dG Wg + dU Wu
    a2 = torch.randn(M, K, device=dev).bfloat16()
    wt2 = (torch.randn(K, N, device=dev) / math.sqrt(K)).bfloat16()
    y = ops.gemm_pair(a, wt, b_layout="kn", a2=a2, b2=wt2, b2_layout="kn", status=st)
    assert st.read() == 0 and rel(y, a.float() @ wt.float() + a2.float() @ wt2.float()) < 4e-3
    # the single-CTA kernel stays available and agrees
    assert rel(ops.gemm(a, w, bias=bias, kernel="single", status=st), ops.gemm_ref(a, w, bias=bias)) < 4e-3


@pytest.mark.parametrize("M,I,K,act", [(256, 128, 64, "silu"), (300, 328, 200, "silu"), (2048, 1408, 2048, "silu"),
                                       (1024, 512, 256, "gelu_pytorch_tanh"), (512, 256, 128, "gelu")])
def test_pair_gemm_glu_epilogue(dev, M, I, K, act):
    from opaque_b200 import ops
    torch.manual_seed(M + I)
    st = ops.StatusWord(dev)
    a = torch.randn(M, K, device=dev).bfloat16()
    wg = (torch.randn(I, K, device=dev) / math.sqrt(K)).bfloat16()
    wu = (torch.randn(I, K, device=dev) / math.sqrt(K)).bfloat16()
    h, g, u = ops.gemm_glu(a, wg, wu, act=act, status=st)
    assert st.read() == 0
    assert rel(g, a.float() @ wg.float().t()) < 4e-3 and rel(u, a.float() @ wu.float().t()) < 4e-3
    assert rel(h, ops.gemm_glu_ref(a, wg, wu, act=act)) < 6e-3
    # the activation is formed from the stored (rounded) pre-activations: the backward pass sees the same values
    gf, uf = g.float(), u.float()
    act_g = torch.nn.functional.silu(gf) if act == "silu" else torch.nn.functional.gelu(gf, approximate="tanh" if "tanh" in act else "none")
    assert rel(h, act_g * uf) < 3e-3
    h2, g2, u2 = ops.gemm_glu(a, wg, wu, act=act, save_preact=False, status=st)
    assert g2 is None and u2 is None and rel(h2, ops.gemm_glu_ref(a, wg, wu, act=act)) < 6e-3


@pytest.mark.parametrize("M,I,K,act", [(256, 128, 64, "silu"), (300, 320, 200, "silu"), (2048, 1408, 2048, "silu"),
                                       (512, 256, 128, "gelu_pytorch_tanh"), (512, 256, 128, "gelu")])
def test_down_projection_data_gradient_with_glu_backward_epilogue(dev, M, I, K, act):
    """dH = dY W_down stays in tensor memory; the epilogue's (dGate, dUp) equal the element-wise backward applied to the
    bf16-rounded dH, and the whole frozen-MLP function matches autograd through the separate operations."""
    from opaque_b200 import ops
    from opaque_b200.engine import fused
    torch.manual_seed(M + I + K)
    st = ops.StatusWord(dev)
    dy = torch.randn(M, K, device=dev).bfloat16()
    wd = (torch.randn(K, I, device=dev) / math.sqrt(K)).bfloat16()           # down projection as stored: [d, I]
    g = torch.randn(M, I, device=dev).bfloat16()
    u = torch.randn(M, I, device=dev).bfloat16()
    dg, du = ops.gemm_glu_bwd(dy, wd, g, u, act=act, status=st)
    assert st.read() == 0
    dh = (dy.float() @ wd.float()).bfloat16().float()
    gf = g.float().requires_grad_(True)
    a = torch.nn.functional.silu(gf) if act == "silu" else torch.nn.functional.gelu(gf, approximate="tanh" if "tanh" in act else "none")
    (a * u.float()).backward(dh)
    assert rel(dg, gf.grad) < 6e-3 and rel(du, dh * a.detach()) < 6e-3
    if act != "silu" or I % 64:
        return
    # the frozen MLP as one function against the composed path
    x = torch.randn(M, K, device=dev).bfloat16().requires_grad_(True)
    wg = (torch.randn(I, K, device=dev) / math.sqrt(K)).bfloat16()
    wu = (torch.randn(I, K, device=dev) / math.sqrt(K)).bfloat16()
    old, fused.FUSE_GLU_MLP = fused.FUSE_GLU_MLP, True          # the fused form is an option (off by default)
    try:
        y = fused.glu_mlp(x, wg, wu, wd, "silu")
    finally:
        fused.FUSE_GLU_MLP = old
    assert y is not None
    gy = torch.randn_like(y)
    y.backward(gy)
    xr = x.detach().float().requires_grad_(True)
    yr = (torch.nn.functional.silu(xr @ wg.float().t()) * (xr @ wu.float().t())) @ wd.float().t()
    yr.backward(gy.float())
    assert rel(y, yr) < 1e-2 and rel(x.grad, xr.grad) < 2e-2


def test_instruction_descriptor_bitfields():
    """kind::f16 instruction descriptor: D format [4,6), A / B format [7,10) / [10,13), majors 15 / 16, N>>3 [17,23), M>>4 [24,29)."""
    from opaque_b200.ops import lib
    f = lib.load().ob_debug_idesc_bf16
    base = (1 << 4) | (1 << 7) | (1 << 10)
    assert f(128, 256, 0, 0) == base | (32 << 17) | (8 << 24)
    assert f(256, 256, 0, 1) == base | (1 << 16) | (32 << 17) | (16 << 24)
    assert f(128, 128, 1, 1) == base | (1 << 15) | (1 << 16) | (16 << 17) | (8 << 24)


@pytest.mark.parametrize("R,V,K,softcap,smoothing", [(300, 50257, 256, 0.0, 0.0), (260, 128256, 128, 0.0, 0.0),
                                                     (130, 151936, 64, 0.0, 0.1), (512, 1000, 512, 30.0, 0.0),
                                                     (256, 256, 64, 0.0, 0.0)])
def test_fused_head_cross_entropy_forward_and_dlogits(dev, R, V, K, softcap, smoothing):
    """Head GEMM with the cross-entropy statistics in its epilogue against the fp32 statement of the same loss."""
    from opaque_b200 import ops
    torch.manual_seed(R + V)
    st = ops.StatusWord(dev)
    h = torch.randn(R, K, device=dev).bfloat16()
    w = (torch.randn(V, K, device=dev) * (3.0 / math.sqrt(K))).bfloat16()
    lab = torch.randint(0, V, (R,), device=dev)
    lab[::7] = -100
    rw = torch.rand(R, device=dev)

    def oracle(z):
        return ops.cross_entropy_ref(z, lab, logit_softcapping=softcap, label_smoothing=smoothing)
    z_ref = (h.float() @ w.float().t()).requires_grad_(True)
    nll_ref = oracle(z_ref)
    # forward only: no logits reach memory
    nll, lse, z = ops.linear_ce_forward(h, w, lab, softcap=softcap, label_smoothing=smoothing, status=st)
    assert st.read() == 0 and z is None
    err = (nll - nll_ref.detach()).abs()
    assert float(err.max()) < 2e-2, (int(err.argmax()), nll[int(err.argmax())].item(), nll_ref[int(err.argmax())].item())
    assert bool((nll[::7] == 0).all())
    # bit-reproducible: per-tile partials are combined in a fixed order
    nll2, _, _ = ops.linear_ce_forward(h, w, lab, softcap=softcap, label_smoothing=smoothing, status=st)
    assert torch.equal(nll, nll2)
    # with stored logits: statistics are those of the stored (bf16) values; gradients in place
    nll_s, lse_s, z = ops.linear_ce_forward(h, w, lab, softcap=softcap, label_smoothing=smoothing, store_logits=True, status=st)
    zc = z_ref.detach() if not softcap else softcap * torch.tanh(z_ref.detach() / softcap)
    assert st.read() == 0 and z.shape == (R, V) and rel(z, zc) < 4e-3
    # the statistics are those of the STORED (bf16-rounded, already capped) logits, which is what the backward pass reads
    nll_of_stored = ops.cross_entropy_ref(z.float(), lab, label_smoothing=smoothing)
    assert float((nll_s - nll_of_stored).abs().max()) < 2e-3
    assert float((nll_s - nll_ref.detach()).abs().max()) < 0.1
    (nll_ref * rw).sum().backward()
    ops.linear_ce_dlogits_(z, lab, lse_s, rw, softcap=softcap, label_smoothing=smoothing)
    assert rel(z, z_ref.grad) < 2e-2 and bool((z[::7] == 0).all())


def test_die_map_splits_the_sms_and_pairs_agree(dev):
    from opaque_b200 import ops
    dm = ops.die_map()
    if dm is None:
        pytest.skip("no two-die split measured on this device")
    assert len(dm) == torch.cuda.get_device_properties(dev).multi_processor_count
    assert 0 < sum(dm) < len(dm)                                             # both dies present
    assert all(dm[i] == dm[i + 1] for i in range(0, len(dm) - 1, 2))         # the two SMs of a pair share a die
    assert ops.die_map() == dm                                               # cached, not re-measured


@pytest.mark.parametrize("tile", ["512x256", "256x256"])
def test_claimed_tile_schedule_covers_every_tile_across_ring_wraps(dev, tile):
    """The die-aware assignment claims one slot per cluster from a ring of self-resetting words: every tile must be
    computed exactly once, also after more launches than the ring has words and for grids smaller than the GPU."""
    from opaque_b200 import ops
    if ops.die_map() is None:
        pytest.skip("no two-die split measured on this device")
    torch.manual_seed(7)
    st = ops.StatusWord(dev)
    old = ops.set_die_aware_tiles(True)
    try:
        _claimed_schedule_cases(ops, st, dev, tile)
    finally:
        ops.set_die_aware_tiles(old)


def _claimed_schedule_cases(ops, st, dev, tile):
    for M, N, K in [(1024, 1024, 128), (4096, 2048, 64), (5000, 3000, 192)]:
        a = torch.randn(M, K, device=dev).bfloat16()
        w = (torch.randn(N, K, device=dev) / math.sqrt(K)).bfloat16()
        ref = ops.gemm_ref(a, w)
        y = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        for i in range(1500):
            if i % 500 == 0:
                y.fill_(float("nan"))                                        # a skipped tile would stay NaN
            ops.gemm_pair(a, w, out=y, status=st, tile=tile)
            if i % 500 == 0:
                assert st.read() == 0 and rel(y, ref) < 4e-3
        assert st.read() == 0 and rel(y, ref) < 4e-3
