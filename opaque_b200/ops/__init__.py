"""Python front-ends of the sm_100a kernels, each with a plain-PyTorch reference.

Every ``*_ref`` function is the fp32 PyTorch statement of the same operation; it is the
numerics oracle in the tests and the implementation used on CPU.  The CUDA entry points fail
loudly when the kernel library cannot be loaded on a GPU machine — there is no silent
fallback on device tensors.

Kernel inventory (reference counterparts: packages/opaque-patches/src/opaque/api/patches/kernels/*,
packages/opaque-engine/src/opaque/api/engine/clipping/_pytree.py:475-564,
packages/opaque-dpsgd/src/opaque/api/dpsgd/noise/_gaussian.py:235-278,
packages/opaque-optimizers/src/opaque/api/optimizers/_adam.py:120-270):
  wgrad_clip            clip-weighted weight-gradient GEMM with (peer) reduce epilogue   [tcgen05]
  ghost_norm            per-example gradient norms of linear / embedding layers          [tcgen05]
  rms_norm / fused add  forward, dX, per-example dW
  glu                   SwiGLU / GeGLU forward and backward
  rope_qk               joint rotary embedding of Q and K (GQA, position ids)
  cross_entropy         online-softmax NLL with in-place dlogits (softcap, scale, smoothing)
  philox_normal_add_    counter-based Gaussian noise
  rows_sumsq / clip_weighted_sum / embedding_wgrad   direct-norm path for small parameters
  shard_step            noise (iid | BLT | banded) + AdamW-BC + bf16 write-back to every rank
"""
from __future__ import annotations

import math
from typing import Sequence

import torch

from . import lib
from .lib import DeviceWaitTimeout, KernelLibraryError, StatusWord

DEFAULT_WAIT_BUDGET_S = 2.0


def _c(t: torch.Tensor) -> torch.Tensor:
    return t if t.is_contiguous() else t.contiguous()


def _need_bf16(*ts: torch.Tensor) -> None:
    for t in ts:
        if t.dtype != torch.bfloat16:
            raise TypeError(f"expected bf16 tensors, got {t.dtype}")


# =============================================================================== wgrad / ghost

def pick_block_n(n: int) -> int:
    """Output tile width of the clip-weighted GEMM for ``n`` columns."""
    if n > 128:
        return 256
    return 128 if n > 64 else 64


def pick_splits(work_tiles: int, rows: int, sms: int, *, max_splits: int | None = None) -> int:
    """K-splits that balance the persistent grid: maximise ``items / (waves · sms)`` for ``items = tiles · splits``.

    Every split keeps at least 8 k-blocks of 64 rows; ties go to the smaller split count (less reduction traffic).
    """
    cap = max(1, rows // (64 * 8))
    if max_splits is not None:
        cap = min(cap, max_splits)
    cap = min(cap, max(1, 2 * sms // max(work_tiles, 1)) if work_tiles < sms else 4)
    best, best_eff = 1, 0.0
    for s in range(1, cap + 1):
        items = work_tiles * s
        eff = items / (math.ceil(items / sms) * sms)
        if eff > best_eff + 0.02:
            best, best_eff = s, eff
    return best


def wgrad_clip(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None, *, row_scale: torch.Tensor | None = None,
               seg_offsets: torch.Tensor | None = None, num_groups: int = 1, splits: int | None = None,
               out_offset: int = 0, ldm: int | None = None, ldn: int = 1, n_valid: int = 0, accumulate: bool = True,
               group_stride: int = 0, group_out_offset: torch.Tensor | None = None,
               peer_table: torch.Tensor | None = None, shard_elems: int = 0, block_n: int | None = None,
               status: StatusWord | None = None, wait_budget_s: float = DEFAULT_WAIT_BUDGET_S) -> None:
    """``flat[out_offset + g_off + m*ldm + n*ldn] (+)= Σ_t s[t]·a[t, m]·b[t, n]`` over each segment.

    ``a`` is ``[T, M]`` (scaled operand, e.g. output gradients), ``b`` is ``[T, N]`` (layer inputs),
    both bf16 with 16-byte aligned rows.  ``out`` is the flat fp32 destination, or ``None`` with a
    ``peer_table`` (int64 device tensor of per-rank shard base pointers) and ``shard_elems``.
    """
    _need_bf16(a, b)
    T, M = a.shape
    N = b.shape[1]
    if b.shape[0] != T:
        raise ValueError("a and b must have the same number of rows")
    if a.stride(1) != 1 or b.stride(1) != 1:
        raise ValueError("operands must be row-major")
    if ldm is None:
        ldm = N
    bn = block_n or pick_block_n(min(N, n_valid) if n_valid else N)
    sms = lib.sm_count()
    if splits is None:
        tiles = num_groups * math.ceil(M / 128) * math.ceil(N / bn)
        splits = pick_splits(tiles, T // max(num_groups, 1), sms) if accumulate else 1
    if not accumulate and splits != 1:
        raise ValueError("store mode cannot split K")
    n_lim = min(N, n_valid) if n_valid else N
    if out is not None:
        if out.dtype != torch.float32:
            raise TypeError("the destination must be fp32")
        last_group = int(group_out_offset.max()) if group_out_offset is not None else (num_groups - 1) * group_stride
        hi = out_offset + last_group + (M - 1) * ldm + (n_lim - 1) * ldn
        room = out.untyped_storage().nbytes() // 4 - out.storage_offset()
        if min(out_offset, ldm, ldn) < 0 or hi >= room:
            raise ValueError(f"wgrad_clip would write element {hi} of a destination holding {room}")
    elif peer_table is None or shard_elems <= 0:
        raise ValueError("give either a destination tensor or a peer table with shard_elems")
    rc = lib.load().ob_wgrad_clip(
        a.data_ptr(), b.data_ptr(), T, M, N, a.stride(0), b.stride(0), lib.ptr(row_scale), lib.ptr(seg_offsets),
        num_groups, splits, lib.ptr(out), lib.ptr(peer_table), shard_elems, lib.ptr(group_out_offset), group_stride,
        out_offset, ldm, ldn, n_valid, int(accumulate), bn, status.ptr() if status else None, wait_budget_s, sms,
        lib.stream())
    lib.check(rc, "wgrad_clip")


def direct_norm2(a: torch.Tensor, g: torch.Tensor, norm2: torch.Tensor, rows_per_example: int, *, splits: int | None = None,
                 status: StatusWord | None = None, wait_budget_s: float = DEFAULT_WAIT_BUDGET_S) -> torch.Tensor:
    """``norm2[e] += ‖a_eᵀ g_e‖²_F`` for example e = rows ``[e·R, (e+1)·R)`` of ``a [T, d_in]`` and ``g [T, d_out]``.

    The direct form of a per-example gradient norm: the per-example products pass through tensor memory tile by tile
    (the clip-weighted weight-gradient kernel with a different epilogue) and only their squares are summed.
    ``2·R·d_in·d_out`` FLOPs per example against ``R²·(d_in + d_out)`` for :func:`ghost_norm`; see
    :func:`pick_norm_path`.  ``R % 64 == 0``.
    """
    _need_bf16(a, g)
    T, M = a.shape
    N = g.shape[1]
    if g.shape[0] != T or a.stride(1) != 1 or g.stride(1) != 1:
        raise ValueError("a [T, d_in] and g [T, d_out] must be row-major with the same number of rows")
    if rows_per_example <= 0 or rows_per_example % 64 or T % rows_per_example:
        raise ValueError("rows_per_example must be a multiple of 64 that divides the number of rows")
    B = T // rows_per_example
    if norm2.dtype != torch.float32 or norm2.numel() < B or not norm2.is_contiguous():
        raise ValueError("norm2 must hold one contiguous fp32 value per example")
    sms = lib.sm_count()
    if splits is None:
        tiles = math.ceil(M / 128) * math.ceil(N / 256)
        splits = pick_splits(tiles, T, sms, max_splits=B)
    rc = lib.load().ob_direct_norm2(a.data_ptr(), g.data_ptr(), B, rows_per_example, M, N, a.stride(0), g.stride(0), splits,
                                    norm2.data_ptr(), status.ptr() if status else None, wait_budget_s, sms, lib.stream())
    lib.check(rc, "direct_norm2")
    return norm2


def pick_norm_path(rows_per_example: int, d_in: int, d_out: int) -> str:
    """``"ghost"`` (Gram matrices, ``R²·(d_in + d_out)`` FLOPs on the upper triangle) or ``"direct"`` (the per-example
    product itself, ``2·R·d_in·d_out``) for one layer.  The Gram kernel runs at about 0.7 of the product kernel's rate, so
    the direct form wins once ``R > 1.4·d_in·d_out / (d_in + d_out)``; it needs ``R % 64 == 0``."""
    if rows_per_example % 64:
        return "ghost"
    return "direct" if rows_per_example * (d_in + d_out) > 1.4 * d_in * d_out else "ghost"


def wgrad_clip_per_example(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None, *, ex_scale: torch.Tensor | None,
                           rows_per_example: int, out_offset: int = 0, ldm: int | None = None, accumulate: bool = True,
                           splits: int | None = None, peer_table: torch.Tensor | None = None, shard_elems: int = 0,
                           status: StatusWord | None = None, wait_budget_s: float = DEFAULT_WAIT_BUDGET_S) -> None:
    """``flat[out_offset + m*ldm + n] (+)= Σ_e c[e] · a_eᵀ b_e`` with example e = rows ``[e·R, (e+1)·R)``, ``R % 64 == 0``.

    The clip factor multiplies each example's fp32 partial product in the epilogue (TMEM → registers), so the operand
    tiles go from TMA straight to the tensor core and ``c`` is applied unrounded.
    """
    _need_bf16(a, b)
    T, M = a.shape
    N = b.shape[1]
    if b.shape[0] != T or a.stride(1) != 1 or b.stride(1) != 1:
        raise ValueError("a [T, M] and b [T, N] must be row-major with the same number of rows")
    if rows_per_example <= 0 or rows_per_example % 64 or T % rows_per_example:
        raise ValueError("rows_per_example must be a multiple of 64 that divides the number of rows")
    B = T // rows_per_example
    if ex_scale is not None and (ex_scale.dtype != torch.float32 or ex_scale.numel() < B or not ex_scale.is_contiguous()):
        raise ValueError("ex_scale must hold one contiguous fp32 factor per example")
    if ldm is None:
        ldm = N
    sms = lib.sm_count()
    if splits is None:
        tiles = math.ceil(M / 128) * math.ceil(N / 256)
        splits = pick_splits(tiles, T, sms, max_splits=B) if accumulate else 1
        if peer_table is not None and tiles * 2 >= sms:
            splits = 1                      # every extra split sends the whole tile over NVLink once more
    if out is not None:
        if out.dtype != torch.float32:
            raise TypeError("the destination must be fp32")
        hi = out_offset + (M - 1) * ldm + N - 1
        room = out.untyped_storage().nbytes() // 4 - out.storage_offset()
        if min(out_offset, ldm) < 0 or hi >= room:
            raise ValueError(f"wgrad_clip_per_example would write element {hi} of a destination holding {room}")
    elif peer_table is None or shard_elems <= 0:
        raise ValueError("give either a destination tensor or a peer table with shard_elems")
    rc = lib.load().ob_wgrad_clip_pe(a.data_ptr(), b.data_ptr(), B, rows_per_example, M, N, a.stride(0), b.stride(0),
                                     lib.ptr(ex_scale), splits, lib.ptr(out), lib.ptr(peer_table), shard_elems, out_offset,
                                     ldm, int(accumulate), status.ptr() if status else None, wait_budget_s, sms,
                                     lib.stream())
    lib.check(rc, "wgrad_clip_per_example")


def wgrad_clip_ref(a, b, *, row_scale=None, seg_offsets=None, num_groups=1):
    """fp32 oracle: returns ``[num_groups, M, N]``."""
    af, bf = a.float(), b.float()
    if row_scale is not None:
        af = af * row_scale.float()[:, None]
    if seg_offsets is None:
        return (af.t() @ bf)[None]
    offs = seg_offsets.tolist()
    return torch.stack([af[offs[g]:offs[g + 1]].t() @ bf[offs[g]:offs[g + 1]] for g in range(num_groups)])


def ghost_norm(a: torch.Tensor | None, g: torch.Tensor, norm2: torch.Tensor, tokens_per_example: int, *,
               ids: torch.Tensor | None = None, seg_offsets: torch.Tensor | None = None,
               seg_out: torch.Tensor | None = None, status: StatusWord | None = None,
               wait_budget_s: float = DEFAULT_WAIT_BUDGET_S) -> None:
    """``norm2[i] += ‖A_iᵀ G_i‖_F²`` for every segment i of rows.

    Uniform layout: segment i is rows ``[i·T, (i+1)·T)``.  Ragged layout: ``seg_offsets`` (int32 ``[S+1]``) gives the
    row range of each segment (none longer than ``tokens_per_example``) and ``seg_out`` (int32 ``[S]``) the
    accumulator each segment adds to (e.g. the example an (expert, example) group belongs to).
    With ``ids`` (int32, one per row) the inputs are one-hot rows (embedding layer) and ``a`` is unused.
    """
    _need_bf16(g)
    rows, dg = g.shape
    if seg_offsets is None:
        B = rows // tokens_per_example
        if B * tokens_per_example != rows:
            raise ValueError("rows must be a multiple of tokens_per_example")
        if norm2.numel() < B:
            raise ValueError("one accumulator per example is required")
    else:
        if seg_offsets.dtype != torch.int32 or (seg_out is not None and seg_out.dtype != torch.int32):
            raise TypeError("segment tables must be int32")
        B = seg_offsets.numel() - 1
        if seg_out is not None and seg_out.numel() != B:
            raise ValueError("seg_out needs one entry per segment")
    if ids is None:
        _need_bf16(a)
        if a.shape[0] != rows:
            raise ValueError("a and g must have the same number of rows")
        da, lda, ap = a.shape[1], a.stride(0), a.data_ptr()
    else:
        if ids.dtype != torch.int32 or ids.numel() != rows:
            raise TypeError("ids must be int32 with one entry per row")
        da, lda, ap = 0, 0, None
    rc = lib.load().ob_ghost_norm(ap, g.data_ptr(), lib.ptr(ids), B, tokens_per_example, da, dg, lda, g.stride(0),
                                  norm2.data_ptr(), lib.ptr(seg_offsets), lib.ptr(seg_out), rows,
                                  status.ptr() if status else None, wait_budget_s, lib.sm_count(), lib.stream())
    lib.check(rc, "ghost_norm")


PAIR_GEMM = True          # dense (ungrouped) products run on CTA pairs (256 x 256 tiles, tcgen05 cta_group::2)


def _check_b(b: torch.Tensor, layout: str, K: int, what: str) -> int:
    if b.ndim != 2 or b.stride(1) != 1:
        raise ValueError(f"{what} must be a row-major 2-D matrix")
    kn = layout == "kn"
    if (b.shape[0] if kn else b.shape[1]) != K:
        raise ValueError(f"{what}: inner dimensions differ")
    return b.shape[1] if kn else b.shape[0]


def gemm_pair(a: torch.Tensor, b: torch.Tensor, *, b_layout: str = "nk", a2: torch.Tensor | None = None,
              b2: torch.Tensor | None = None, b2_layout: str = "nk", bias: torch.Tensor | None = None,
              out: torch.Tensor | None = None, status: StatusWord | None = None,
              wait_budget_s: float = DEFAULT_WAIT_BUDGET_S, tile: str = "512x256") -> torch.Tensor:
    """``a @ op(b) + a2 @ op(b2) + bias`` on CTA pairs (``tcgen05 … cta_group::2``; bf16 in/out, fp32 accumulation).

    Layouts as in :func:`gemm`; the second segment has its own layout, so ``dX = dG·Wg + dU·Wu`` (both weights
    stored ``[K, N]`` from the product's point of view) and the LoRA data gradient ``dY·W + q·A`` are one launch each.
    ``tile``: ``"512x256"`` (one tile fills tensor memory; fewest operand bytes per FLOP, for long K) or ``"256x256"``
    (two accumulators alternate, so a tile drains during the whole main loop of the next; for short K).
    """
    _need_bf16(a, b)
    if a.ndim != 2 or a.stride(1) != 1:
        raise ValueError("a must be a row-major 2-D matrix")
    M, K = a.shape
    N = _check_b(b, b_layout, K, "b")
    K2 = 0
    if a2 is not None:
        _need_bf16(a2, b2)
        if a2.ndim != 2 or a2.shape[0] != M or a2.stride(1) != 1:
            raise ValueError("second segment: a2 must be [M, K2] row-major")
        K2 = a2.shape[1]
        if _check_b(b2, b2_layout, K2, "b2") != N:
            raise ValueError("second segment: b2 must cover the same N")
    if bias is not None:
        _need_bf16(bias)
        if bias.numel() != N or not bias.is_contiguous():
            raise ValueError("bias must hold N contiguous values")
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=a.device)
    elif out.shape != (M, N) or out.dtype != torch.bfloat16 or out.stride(1) != 1:
        raise ValueError("out must be a row-major bf16 [M, N] matrix")
    if tile == "256x256":
        rc = lib.load().ob_gemm_pair_db(
            a.data_ptr(), b.data_ptr(), lib.ptr(a2), lib.ptr(b2), lib.ptr(bias), out.data_ptr(),
            M, N, K, K2, a.stride(0), b.stride(0), a2.stride(0) if a2 is not None else 0,
            b2.stride(0) if b2 is not None else 0, out.stride(0), int(b_layout == "kn"), int(b2_layout == "kn"),
            status.ptr() if status else None, wait_budget_s, lib.sm_count(), lib.stream())
        lib.check(rc, "gemm_pair (256x256)")
        return out
    if tile != "512x256":
        raise ValueError("tile must be '512x256' or '256x256'")
    rc = lib.load().ob_gemm_pair(
        a.data_ptr(), b.data_ptr(), None, lib.ptr(a2), lib.ptr(b2), None, lib.ptr(bias), out.data_ptr(), None, None,
        M, N, K, K2, a.stride(0), b.stride(0), a2.stride(0) if a2 is not None else 0,
        b2.stride(0) if b2 is not None else 0, out.stride(0), int(b_layout == "kn"), int(b2_layout == "kn"), 0, 0,
        status.ptr() if status else None, wait_budget_s, lib.sm_count(), lib.stream())
    lib.check(rc, "gemm_pair")
    return out


def die_map() -> list[int] | None:
    """Die (0 / 1) of every SM of the current device by ``%smid``, or ``None`` when no two-die split was measured.

    Probed once per device and process by timing atomics from every SM (a line's home L2 slice answers faster to SMs of
    its own die); the CTA-pair GEMMs use it to keep tiles that share operands on one die.  Synchronises the device on
    the first call, so call it outside CUDA-graph captures (the GEMM entry points skip the probe while capturing).
    """
    import ctypes
    buf = (ctypes.c_ubyte * 256)()
    n = lib.load().ob_die_map(buf, 256)
    return [int(buf[i]) for i in range(n)] if n > 0 else None


def set_die_aware_tiles(on: bool) -> bool:
    """Switch the die-aware tile assignment of the CTA-pair GEMMs on or off for later launches; returns the old setting.

    On: the clusters of each die (see :func:`die_map`) claim tiles from one contiguous range of the raster, so operands
    shared by neighbouring tiles cross the die-to-die link once.  Off (default): cluster ``c`` takes tiles ``c, c + n, …``.
    Measured: fewer sectors over the link, no change in kernel time.
    """
    return bool(lib.load().ob_pair_set_die_aware(1 if on else 0))


_GLU_ACT = {"silu": 0, "gelu": 1, "gelu_pytorch_tanh": 2, "gelu_tanh": 2}


def gemm_glu(a: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, *, act: str = "silu", save_preact: bool = True,
             status: StatusWord | None = None, wait_budget_s: float = DEFAULT_WAIT_BUDGET_S):
    """Gated-MLP up-projection in ONE launch: ``act(a W_gᵀ) * (a W_uᵀ)`` with both products in one accumulator tile.

    ``w_gate`` and ``w_up`` are ``[I, K]`` as stored.  Returns ``(h, gate, up)``; ``gate`` / ``up`` (the bf16
    pre-activations the backward pass needs) are ``None`` with ``save_preact=False``.
    """
    _need_bf16(a, w_gate, w_up)
    if a.ndim != 2 or a.stride(1) != 1 or w_gate.ndim != 2 or w_gate.shape != w_up.shape or w_gate.stride(1) != 1 \
            or w_up.stride(1) != 1 or w_gate.stride(0) != w_up.stride(0) or w_gate.shape[1] != a.shape[1]:
        raise ValueError("gemm_glu: a [M, K] and w_gate, w_up [I, K] row-major with equal pitch")
    M, K = a.shape
    inter = w_gate.shape[0]
    h = torch.empty(M, inter, dtype=torch.bfloat16, device=a.device)
    g = torch.empty_like(h) if save_preact else None
    u = torch.empty_like(h) if save_preact else None
    rc = lib.load().ob_gemm_pair(
        a.data_ptr(), w_gate.data_ptr(), w_up.data_ptr(), None, None, None, None, h.data_ptr(), lib.ptr(g), lib.ptr(u),
        M, 2 * inter, K, 0, a.stride(0), w_gate.stride(0), 0, 0, h.stride(0), 0, 0, 1, _GLU_ACT[act],
        status.ptr() if status else None, wait_budget_s, lib.sm_count(), lib.stream())
    lib.check(rc, "gemm_glu")
    return h, g, u


def gemm_glu_bwd(dy: torch.Tensor, w_down: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, *, act: str = "silu",
                 status: StatusWord | None = None, wait_budget_s: float = DEFAULT_WAIT_BUDGET_S):
    """Backward of ``y = (act(gate) * up) @ w_downᵀ`` up to the pre-activations, in ONE launch: ``(dgate, dup)``.

    ``dy [M, d]``, ``w_down [d, I]`` as stored, ``gate`` / ``up [M, I]`` (the bf16 pre-activations :func:`gemm_glu` kept).
    The product ``dH = dy @ w_down`` lives only in tensor memory: the epilogue rounds it to bf16 (what a stored ``dH``
    would hold), multiplies with ``up * act'(gate)`` and ``act(gate)`` and stores the two gradients.  ``I % 64 == 0``.
    """
    _need_bf16(dy, w_down, gate, up)
    if dy.ndim != 2 or dy.stride(1) != 1 or w_down.ndim != 2 or w_down.stride(1) != 1 or w_down.shape[0] != dy.shape[1]:
        raise ValueError("gemm_glu_bwd: dy [M, d] and w_down [d, I] must be row-major")
    M, K = dy.shape
    inter = w_down.shape[1]
    if gate.shape != (M, inter) or up.shape != (M, inter) or gate.stride(1) != 1 or up.stride(1) != 1 \
            or gate.stride(0) != up.stride(0) or inter % 64:
        raise ValueError("gemm_glu_bwd: gate / up must be [M, I] with equal pitch and I % 64 == 0")
    dg = torch.empty(M, inter, dtype=torch.bfloat16, device=dy.device)
    du = torch.empty_like(dg)
    rc = lib.load().ob_gemm_pair_glu_bwd(dy.data_ptr(), w_down.data_ptr(), gate.data_ptr(), up.data_ptr(), dg.data_ptr(),
                                         du.data_ptr(), M, inter, K, dy.stride(0), w_down.stride(0), gate.stride(0),
                                         dg.stride(0), 1, _GLU_ACT[act], status.ptr() if status else None, wait_budget_s,
                                         lib.sm_count(), lib.stream())
    lib.check(rc, "gemm_glu_bwd")
    return dg, du


def gemm_glu_ref(a, w_gate, w_up, *, act="silu"):
    """fp32 oracle of :func:`gemm_glu` (returns ``h`` only)."""
    g, u = a.float() @ w_gate.float().t(), a.float() @ w_up.float().t()
    if act == "silu":
        return torch.nn.functional.silu(g) * u
    return torch.nn.functional.gelu(g, approximate="tanh" if "tanh" in act else "none") * u


def linear_ce_forward(hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor, *, ignore_index: int = -100,
                      softcap: float = 0.0, label_smoothing: float = 0.0, store_logits: bool = False,
                      status: StatusWord | None = None, wait_budget_s: float = DEFAULT_WAIT_BUDGET_S):
    """Output head and token cross-entropy in one tcgen05 kernel: ``(nll, lse, logits | None)``.

    ``hidden [R, d]``, ``weight [V, d]`` (bf16), ``labels [R]`` (int64).  Every 256-column logits tile is reduced to
    per-row statistics in the GEMM epilogue, straight out of tensor memory; a small second kernel combines the tiles of
    a row in a fixed order (bit-reproducible).  The logits reach memory only with ``store_logits=True`` (bf16, after
    the soft cap), which is what :func:`linear_ce_dlogits_` turns into gradients in place.
    Reference counterpart: packages/opaque-patches/src/opaque/api/patches/kernels/linear_cross_entropy.py:98-208.
    """
    _need_bf16(hidden, weight)
    if hidden.ndim != 2 or weight.ndim != 2 or hidden.stride(1) != 1 or weight.stride(1) != 1 or hidden.shape[1] != weight.shape[1]:
        raise ValueError("linear_ce_forward: hidden [R, d] and weight [V, d] must be row-major")
    R, K = hidden.shape
    V = weight.shape[0]
    lab = labels.reshape(-1).to(torch.int64).contiguous()
    if lab.numel() != R:
        raise ValueError("one label per row is required")
    tiles = 2 * ((V + 255) // 256)                  # two column groups per 256-wide tile
    partials = torch.empty(max(R, 1) * tiles * 4, dtype=torch.float32, device=hidden.device)     # scratch of the epilogue
    nll = torch.empty(R, dtype=torch.float32, device=hidden.device)
    lse = torch.empty(R, dtype=torch.float32, device=hidden.device)
    logits = None
    ldo = 0
    if store_logits:
        ldo = (V + 7) // 8 * 8                       # 16-byte aligned rows for the vector stores
        logits = torch.empty(R, ldo, dtype=torch.bfloat16, device=hidden.device)[:, :V]
    rc = lib.load().ob_linear_ce_fwd(hidden.data_ptr(), weight.data_ptr(), lab.data_ptr(), lib.ptr(logits), partials.data_ptr(),
                                     nll.data_ptr(), lse.data_ptr(), R, V, K, hidden.stride(0), weight.stride(0), ldo,
                                     float(softcap), float(label_smoothing), ignore_index,
                                     status.ptr() if status else None, wait_budget_s, lib.sm_count(), lib.stream())
    lib.check(rc, "linear_ce_forward")
    return nll, lse, logits


def linear_ce_dlogits_(logits: torch.Tensor, labels: torch.Tensor, lse: torch.Tensor, row_weight: torch.Tensor | None = None, *,
                       ignore_index: int = -100, softcap: float = 0.0, label_smoothing: float = 0.0) -> torch.Tensor:
    """In place: the logits stored by :func:`linear_ce_forward` become ``row_weight · ∂nll/∂(raw logits)`` (one read, one write)."""
    _need_bf16(logits)
    if logits.ndim != 2 or logits.stride(1) != 1:
        raise ValueError("logits must be a row-major matrix")
    lab = labels.reshape(-1).to(torch.int64).contiguous()
    rc = lib.load().ob_linear_ce_dlogits(logits.data_ptr(), lab.data_ptr(), lse.data_ptr(), lib.ptr(row_weight), logits.shape[0],
                                         logits.shape[1], logits.stride(0), float(softcap), float(label_smoothing), ignore_index,
                                         lib.stream())
    lib.check(rc, "linear_ce_dlogits")
    return logits


def pick_gemm_kernel(M: int, N: int, K: int, sms: int = 148) -> str:
    """``"pair"`` or ``"single"`` for an ungrouped ``[M, K] x [K, N]`` product.

    The pair kernel (512 x 256 output tiles on SM pairs, half the operand bytes per FLOP) wins on large products; its
    tiles are coarse, so a product with few tiles or a short K leaves SM pairs idle in the last wave or pays the
    un-overlapped part of its epilogue too often.  The estimate is work / (waves x capacity), times the measured
    steady-state rate of each kernel, times K / (K + per-tile overhead in k).
    """
    clusters = max(sms // 2, 1)
    t_pair = -(-M // 512) * -(-N // 256)
    t_single = -(-M // 128) * -(-N // 256)
    # constants fitted to sustained runs: single-CTA steady rate 0.93 of the pair kernel's; un-overlapped part of a tile
    # worth about 128 (pair: one tile fills tensor memory) and 48 (single: double-buffered accumulators) elements of K
    eff_pair = t_pair / (-(-t_pair // clusters) * clusters) * (K / (K + 128.0))
    eff_single = 0.93 * t_single / (-(-t_single // sms) * sms) * (K / (K + 48.0))
    return "pair" if eff_pair >= eff_single else "single"


def gemm(a: torch.Tensor, b: torch.Tensor, *, b_layout: str = "nk", a2: torch.Tensor | None = None,
         b2: torch.Tensor | None = None, bias: torch.Tensor | None = None, group_offs: torch.Tensor | None = None,
         out: torch.Tensor | None = None, status: StatusWord | None = None,
         wait_budget_s: float = DEFAULT_WAIT_BUDGET_S, kernel: str = "auto") -> torch.Tensor:
    """``a @ op(b) + a2 @ b2ᵀ + bias`` on the tcgen05 path (bf16 in/out, fp32 accumulation).

    ``b_layout="nk"``: ``b`` is ``[N, K]`` (a weight matrix as stored; ``op(b) = bᵀ``);  ``"kn"``: ``b`` is ``[K, N]``
    (``op(b) = b`` — data gradients ``dY @ W`` without a transposed copy).  ``a2 [M, r]``, ``b2 [N, r]`` add a
    low-rank segment accumulated in the same tile (LoRA-fused linear).  With ``group_offs`` (int32 ``[E + 1]`` row
    offsets, rows sorted by group) ``b`` is ``[E, N, K]`` / ``[E, K, N]`` and rows of group e use slab e (MoE experts).
    ``kernel``: ``"pair"`` (two CTAs per 512 x 256 tile), ``"single"`` (one CTA per 128 x 256 tile) or ``"auto"``
    (:func:`pick_gemm_kernel` for ungrouped products while :data:`PAIR_GEMM` is on; grouped products always run on
    single CTAs).
    """
    if group_offs is None and kernel == "auto" and PAIR_GEMM:
        kernel = pick_gemm_kernel(a.shape[0], b.shape[1] if b_layout == "kn" else b.shape[0], a.shape[1], lib.sm_count())
    if group_offs is None and kernel == "pair":
        return gemm_pair(a, b, b_layout=b_layout, a2=a2, b2=b2, bias=bias, out=out, status=status,
                         wait_budget_s=wait_budget_s)
    _need_bf16(a, b)
    if a.ndim != 2 or a.stride(1) != 1:
        raise ValueError("a must be a row-major 2-D matrix")
    M, K = a.shape
    kn = {"nk": 0, "kn": 1}[b_layout]
    grouped = group_offs is not None
    if grouped:
        if group_offs.dtype != torch.int32 or b.ndim != 3 or not b.is_contiguous():
            raise TypeError("grouped mode needs int32 offsets and a contiguous [E, ., .] weight stack")
        E = group_offs.numel() - 1
        if b.shape[0] != E:
            raise ValueError("one weight slab per group is required")
        b2d = b.view(-1, b.shape[-1])
        N = b.shape[2] if kn else b.shape[1]
        if (b.shape[1] if kn else b.shape[2]) != K:
            raise ValueError("inner dimensions differ")
        if kn and K % 64:
            raise ValueError("grouped [K, N] slabs need K to be a multiple of 64")
    else:
        if b.ndim != 2 or b.stride(1) != 1:
            raise ValueError("b must be a row-major 2-D matrix")
        E, b2d = 0, b
        N = b.shape[1] if kn else b.shape[0]
        if (b.shape[0] if kn else b.shape[1]) != K:
            raise ValueError("inner dimensions differ")
    K2 = 0
    if a2 is not None:
        _need_bf16(a2, b2)
        if a2.shape[0] != M or b2.shape[0] != N or a2.shape[1] != b2.shape[1] or a2.stride(1) != 1 or b2.stride(1) != 1:
            raise ValueError("low-rank segment: a2 [M, r], b2 [N, r]")
        K2 = a2.shape[1]
    if bias is not None:
        _need_bf16(bias)
        if bias.numel() != N or not bias.is_contiguous():
            raise ValueError("bias must hold N contiguous values")
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=a.device)
    elif out.shape != (M, N) or out.dtype != torch.bfloat16 or out.stride(1) != 1:
        raise ValueError("out must be a row-major bf16 [M, N] matrix")
    rc = lib.load().ob_gemm_tn(a.data_ptr(), b2d.data_ptr(), lib.ptr(a2), lib.ptr(b2), lib.ptr(bias), out.data_ptr(), M, N,
                               K, K2, a.stride(0), b2d.stride(0), a2.stride(0) if a2 is not None else 0,
                               b2.stride(0) if b2 is not None else 0, out.stride(0), kn, lib.ptr(group_offs), E,
                               status.ptr() if status else None, wait_budget_s, lib.sm_count(), lib.stream())
    lib.check(rc, "gemm")
    return out


def gemm_ref(a, b, *, b_layout="nk", a2=None, b2=None, bias=None, group_offs=None):
    """fp32 oracle of :func:`gemm`."""
    af = a.float()
    if group_offs is None:
        y = af @ (b.float() if b_layout == "kn" else b.float().t())
    else:
        offs = group_offs.tolist()
        N = b.shape[2] if b_layout == "kn" else b.shape[1]
        y = af.new_zeros(a.shape[0], N)
        for e in range(len(offs) - 1):
            be = b[e].float() if b_layout == "kn" else b[e].float().t()
            y[offs[e]:offs[e + 1]] = af[offs[e]:offs[e + 1]] @ be
    if a2 is not None:
        y = y + a2.float() @ b2.float().t()
    if bias is not None:
        y = y + bias.float()
    return y


def ghost_set_wide(mode: int | bool) -> int:
    """Gram block shape of :func:`ghost_norm`: 1 = 128x256 blocks for examples of >= 1024 rows (default), 2 = 128x256
    whenever an example spans two row blocks, 0 = always 128x128.  Returns the previous setting."""
    return int(lib.load().ob_ghost_set_wide(int(mode)))


def ghost_norm_ref(a, g, tokens_per_example, *, ids=None):
    """PyTorch reference of ``ghost_norm``: per-example squared gradient norms from Gram matrices."""
    B = g.shape[0] // tokens_per_example
    gg = g.float().view(B, tokens_per_example, -1)
    sg = gg @ gg.transpose(1, 2)
    if ids is None:
        aa = a.float().view(B, tokens_per_example, -1)
        sa = aa @ aa.transpose(1, 2)
    else:
        i = ids.view(B, tokens_per_example)
        sa = (i[:, :, None] == i[:, None, :]).float()
    return (sa * sg).sum(dim=(1, 2))


# =============================================================================== small DP kernels

def philox_normal_add_(x: torch.Tensor, *, seed: int, offset: int = 0, std: float = 1.0, stream_id: int = 0) -> torch.Tensor:
    """In place ``x[i] += std·z(seed, offset + i)`` with ``z`` standard normal, counter-based."""
    if not x.is_contiguous():
        raise ValueError("philox_normal_add_ needs a contiguous tensor")
    code = {torch.float32: 0, torch.bfloat16: 1}[x.dtype]
    rc = lib.load().ob_philox_normal_add(x.data_ptr(), code, x.numel(), seed & (2**64 - 1), offset, float(std),
                                         stream_id, lib.sm_count(), lib.stream())
    lib.check(rc, "philox_normal_add")
    return x


def rows_sumsq(g: torch.Tensor, norm2: torch.Tensor) -> None:
    """``norm2[e] += Σ_p g[e, p]²`` for fp32 ``g [E, P]``."""
    if g.dtype != torch.float32 or g.stride(1) != 1 or norm2.numel() < g.shape[0]:
        raise ValueError("rows_sumsq needs a row-major fp32 matrix and one accumulator per row")
    rc = lib.load().ob_rows_sumsq(g.data_ptr(), g.shape[0], g.shape[1], g.stride(0), norm2.data_ptr(), lib.sm_count(),
                                  lib.stream())
    lib.check(rc, "rows_sumsq")


def clip_weighted_sum(g: torch.Tensor, c: torch.Tensor, out: torch.Tensor | None, *, flat_offset: int = 0,
                      peer_table: torch.Tensor | None = None, shard_elems: int = 0) -> None:
    """``flat[flat_offset + p] += Σ_e c[e]·g[e, p]`` (to the owning rank when a peer table is given)."""
    if out is not None and flat_offset + g.shape[1] > out.numel():
        raise ValueError("clip_weighted_sum would write past the end of the destination")
    if c.numel() < g.shape[0]:
        raise ValueError("one clip factor per example is required")
    rc = lib.load().ob_clip_weighted_sum(g.data_ptr(), c.data_ptr(), g.shape[0], g.shape[1], g.stride(0),
                                         lib.ptr(out), lib.ptr(peer_table), shard_elems, flat_offset, lib.sm_count(),
                                         lib.stream())
    lib.check(rc, "clip_weighted_sum")


def embedding_wgrad(g: torch.Tensor, ids: torch.Tensor, out: torch.Tensor | None, *, row_scale=None, flat_offset=0,
                    peer_table=None, shard_elems=0) -> None:
    """``flat[flat_offset + ids[t]·D + d] += s[t]·g[t, d]``."""
    _need_bf16(g)
    if ids.dtype != torch.int64:
        raise TypeError("ids must be int64")
    if ids.numel() != g.shape[0]:
        raise ValueError("one id per gradient row is required")
    rc = lib.load().ob_embedding_wgrad(g.data_ptr(), ids.data_ptr(), lib.ptr(row_scale), g.shape[0], g.shape[1],
                                       g.stride(0), lib.ptr(out), lib.ptr(peer_table), shard_elems, flat_offset,
                                       lib.sm_count(), lib.stream())
    lib.check(rc, "embedding_wgrad")


def push_grad_(local: torch.Tensor, peer_table: torch.Tensor, shard_elems: int, *, status: StatusWord | None = None) -> None:
    """Add a full-length local fp32 gradient into the owners' shards (peer reductions) and clear it.

    With a ``status`` word that is already set (a bounded wait expired earlier) the kernel does nothing."""
    if local.dtype != torch.float32 or not local.is_contiguous() or local.numel() % 4 or shard_elems % 4:
        raise ValueError("push_grad_: contiguous fp32 buffer with a length and shard size that are multiples of 4")
    rc = lib.load().ob_push_grad(local.data_ptr(), local.numel(), peer_table.data_ptr(), shard_elems,
                                 status.ptr() if status else None, lib.sm_count(), lib.stream())
    lib.check(rc, "push_grad")


def shard_step(*, grad=None, peer_grad=None, master, m, v, params_local=None, peer_params=None, world=1, global_offset=0, seed=0,
               noise_std=0.0, inv_normalize=1.0, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, step=1,
               phi_hat=0.0, decoupled_wd=True, ftrl_state=None, ftrl_mode=0, ftrl_coef: Sequence[float] = (),
               nbuf=0, ring_head=0, noisy_out=None, skip_update=False, status: StatusWord | None = None,
               optimizer: str = "adam", nesterov: bool = False) -> None:
    """One fused pass over a shard: noise, optimizer update on fp32 masters, bf16 write-back to all ranks.

    ``optimizer``: ``"adam"`` (Adam / AdamW / AdamW-BC by ``decoupled_wd`` and ``phi_hat``), ``"sgd"`` (momentum
    ``betas[0]``, PyTorch semantics, optional Nesterov; ``v`` unused) or ``"lion"`` (``betas``; ``v`` unused).

    ``peer_grad`` (int64 device table of ``world`` full-length fp32 accumulation buffers, one per rank) selects the
    pull form: the shard's gradient is the sum over ranks, in rank order, of ``buffer_r[global_offset + i]``, read through
    peer pointers inside this kernel — the reduce-scatter is fused in, uses no atomics and gives the same bits on every
    run.  ``grad`` is then unused and nothing is cleared (each rank clears its own buffer after the closing barrier).

    ``step`` is 1-based; ``phi_hat`` is the bias-corrected noise-variance EMA (0 disables the correction).  With a
    ``status`` word that is already set (the gradient barrier before this call gave up) the kernel touches nothing:
    a partially reduced shard is neither noised, applied nor cleared.
    """
    if (grad is None) == (peer_grad is None):
        raise ValueError("shard_step takes either grad (this shard's reduced gradient) or peer_grad (the pull form)")
    if grad is not None and grad.numel() != master.numel():
        raise ValueError("grad and master must have the shard's length")
    coef = torch.tensor(list(ftrl_coef) or [0.0], dtype=torch.float32)
    import ctypes
    arr = (ctypes.c_float * len(coef))(*coef.tolist())
    rc = lib.load().ob_shard_step(
        lib.ptr(grad), lib.ptr(peer_grad), lib.ptr(master), lib.ptr(m), lib.ptr(v), lib.ptr(ftrl_state), lib.ptr(peer_params),
        lib.ptr(params_local), lib.ptr(noisy_out), master.numel(), global_offset, world, seed & (2**64 - 1),
        float(noise_std), float(inv_normalize), ftrl_mode, nbuf, ring_head, ctypes.cast(arr, ctypes.c_void_p),
        len(coef), float(lr), float(betas[0]), float(betas[1]), float(eps), float(weight_decay),
        1.0 - betas[0] ** step, 1.0 - betas[1] ** step, float(phi_hat), int(decoupled_wd), int(skip_update),
        {"adam": 0, "sgd": 1, "lion": 2}[optimizer], int(nesterov),
        status.ptr() if status else None, lib.sm_count(), lib.stream())
    lib.check(rc, "shard_step")


from . import functional  # noqa: E402
from .functional import (activation, cross_entropy, cross_entropy_ref, fused_add_rms_norm, geglu, glu_ref,  # noqa: E402
                         layer_norm, merge_heads3, plain_torch_ops, rms_norm, rms_norm_ref, rope_qk, rope_qk_ref, rope_tables, rows_group_sum_, swiglu)

__all__ = [
    "gemm", "gemm_pair", "gemm_glu", "gemm_glu_bwd", "direct_norm2", "pick_norm_path", "pick_gemm_kernel", "die_map", "set_die_aware_tiles", "linear_ce_forward", "linear_ce_dlogits_", "gemm_glu_ref", "gemm_ref", "ghost_set_wide", "push_grad_", "wgrad_clip_per_example", "plain_torch_ops", "layer_norm", "activation", "rows_group_sum_", "merge_heads3",
    "DeviceWaitTimeout", "KernelLibraryError", "StatusWord", "clip_weighted_sum", "cross_entropy",
    "cross_entropy_ref", "embedding_wgrad", "fused_add_rms_norm", "geglu", "ghost_norm", "ghost_norm_ref", "glu_ref",
    "philox_normal_add_", "pick_block_n", "pick_splits", "rms_norm", "rms_norm_ref", "rope_qk", "rope_qk_ref",
    "rope_tables", "rows_sumsq", "shard_step", "swiglu", "wgrad_clip", "wgrad_clip_ref",
]
