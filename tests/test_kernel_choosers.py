"""Shape-based choices between kernel variants (pure functions: no GPU needed)."""
from opaque_b200 import ops


def test_gemm_kernel_choice_follows_tile_fill_and_k():
    # long K and enough 512 x 256 tiles for every SM pair: CTA pairs
    for shape in [(16384, 4096, 4096), (16384, 14336, 4096), (16384, 4096, 14336), (16384, 6144, 4096), (16384, 1024, 4096)]:
        assert ops.pick_gemm_kernel(*shape) == "pair", shape
    # short K (the big tile's drain is not amortised) or too few pair tiles: single CTA
    for shape in [(16384, 2304, 768), (16384, 768, 768), (16384, 3072, 768), (16384, 768, 3072), (2048, 512, 4096)]:
        assert ops.pick_gemm_kernel(*shape) == "single", shape
    # the answer depends on the SM count it is asked for (a full last wave of pair tiles), not on a device being present
    assert ops.pick_gemm_kernel(16384, 4096, 4096, sms=148) in ("pair", "single")
    assert ops.pick_gemm_kernel(512, 256, 64, sms=148) in ("pair", "single")


def test_norm_path_choice_crosses_over_with_sequence_length():
    # Gram matrices cost T^2 (d_in + d_out), the product 2 T d_in d_out: short sequences on big layers take the Gram form
    assert ops.pick_norm_path(512, 768, 768) == "ghost"
    assert ops.pick_norm_path(1024, 4096, 4096) == "ghost"
    assert ops.pick_norm_path(1024, 2048, 8192) == "ghost"
    # long sequences on small layers take the product
    assert ops.pick_norm_path(4096, 128, 256) == "direct"
    assert ops.pick_norm_path(2048, 768, 768) == "direct"
    # the product kernel needs examples of a multiple of 64 rows
    assert ops.pick_norm_path(4100, 128, 256) == "ghost"
    # monotone in T for a fixed layer
    seen_direct = False
    for t in range(64, 8192 + 1, 64):
        path = ops.pick_norm_path(t, 1024, 1024)
        assert not (seen_direct and path == "ghost")
        seen_direct = seen_direct or path == "direct"
    assert seen_direct
