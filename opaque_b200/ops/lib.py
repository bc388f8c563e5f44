"""ctypes loader of the in-tree sm_100a kernel library.

The library is plain ``extern "C"`` over raw device pointers and a stream handle, so loading
it needs neither the torch C++ headers nor a JIT cache.  ``load()`` builds it on demand when
the shared object is missing or older than its sources and nvcc is present.
"""
from __future__ import annotations

import ctypes
import functools
from ctypes import c_char_p, c_double, c_float, c_int, c_longlong, c_uint, c_ulonglong, c_void_p

import torch

from ..utils import build as _build

P, I, LL, F, D, U, ULL = c_void_p, c_int, c_longlong, c_float, c_double, c_uint, c_ulonglong

_SIGNATURES = {
    "ob_wgrad_clip": [P, P, I, I, I, LL, LL, P, P, I, I, P, P, LL, P, LL, LL, LL, LL, I, I, I, P, D, I, P],
    "ob_wgrad_clip_pe": [P, P, I, I, I, I, LL, LL, P, I, P, P, LL, LL, LL, I, P, D, I, P],
    "ob_direct_norm2": [P, P, I, I, I, I, LL, LL, I, P, P, D, I, P],
    "ob_ghost_norm": [P, P, P, I, I, I, I, LL, LL, P, P, P, LL, P, D, I, P],
    "ob_gemm_tn": [P, P, P, P, P, P, LL, I, I, I, LL, LL, LL, LL, LL, I, P, I, P, D, I, P],
    "ob_gemm_pair": [P, P, P, P, P, P, P, P, P, P, LL, I, I, I, LL, LL, LL, LL, LL, I, I, I, I, P, D, I, P],
    "ob_pair_init": [],
    "ob_pair_set_die_aware": [I],
    "ob_die_map": [P, I],
    "ob_gemm_pair_glu_bwd": [P, P, P, P, P, P, LL, I, I, LL, LL, LL, LL, I, I, P, D, I, P],
    "ob_gemm_pair_db": [P, P, P, P, P, P, LL, I, I, I, LL, LL, LL, LL, LL, I, I, P, D, I, P],
    "ob_linear_ce_fwd": [P, P, P, P, P, P, P, LL, I, I, LL, LL, LL, F, F, LL, P, D, I, P],
    "ob_linear_ce_dlogits": [P, P, P, P, LL, I, LL, F, F, LL, P],
    "ob_layernorm_fwd": [P, P, P, P, P, P, LL, I, F, P],
    "ob_layernorm_bwd_dx": [P, P, P, P, P, P, LL, I, P],
    "ob_rows_group_sum": [P, P, P, P, I, I, I, LL, P, LL, I, P, LL, P],
    "ob_merge_heads3": [P, P, P, P, P, LL, I, I, I, I, P],
    "ob_activation": [P, P, P, LL, I, I, P],
    "ob_ghost_set_wide": [I],
    "ob_push_grad": [P, LL, P, LL, P, I, P],
    "ob_rmsnorm_fwd": [P, P, P, P, P, P, LL, I, F, F, I, P],
    "ob_rmsnorm_bwd": [P, P, P, P, P, P, P, P, I, I, LL, I, F, P],
    "ob_glu_fwd": [P, P, P, LL, I, LL, I, I, P],
    "ob_glu_bwd": [P, P, P, P, P, LL, I, LL, LL, I, I, P],
    "ob_rope_qk": [P, P, P, P, P, LL, I, I, I, I, LL, LL, I, I, P],
    "ob_rope_qk_oop": [P, P, P, P, P, P, P, LL, I, I, I, I, LL, LL, LL, LL, LL, LL, I, I, P],
    "ob_cross_entropy": [P, I, P, P, P, P, LL, I, LL, F, F, F, LL, I, P],
    "ob_philox_normal_add": [P, I, LL, ULL, LL, F, U, I, P],
    "ob_rows_sumsq": [P, I, LL, LL, P, I, P],
    "ob_clip_weighted_sum": [P, P, I, LL, LL, P, P, LL, LL, I, P],
    "ob_embedding_wgrad": [P, P, P, LL, I, LL, P, P, LL, LL, I, P],
    "ob_shard_step": [P, P, P, P, P, P, P, P, P, LL, LL, I, ULL, F, F, I, I, I, P, I, F, F, F, F, F, F, F, F, I, I, I, I, P, I, P],
    "ob_peer_barrier": [P, P, I, I, I, P, D, P],
    "ob_ipc_alloc": [P, LL],
    "ob_ipc_free": [P],
    "ob_ipc_get_handle": [P, P],
    "ob_ipc_open_handle": [P, P],
    "ob_ipc_close_handle": [P],
    "ob_last_cuda_error": [c_char_p, I],
    "ob_last_detail": [c_char_p, I],
}


class KernelLibraryError(RuntimeError):
    pass


@functools.lru_cache(maxsize=None)
def load() -> ctypes.CDLL:
    try:
        path = _build.build_kernels()
    except Exception as exc:
        if not _build.KERNEL_LIB.exists():
            raise KernelLibraryError(f"sm_100a kernel library is missing and could not be built: {exc}") from exc
        path = _build.KERNEL_LIB
    import os
    override = os.environ.get("OPAQUE_B200_KERNEL_LIB")          # a differently built library (kernel experiments)
    lib = ctypes.CDLL(override or str(path))
    for name, argtypes in _SIGNATURES.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = c_int
    lib.ob_debug_idesc_bf16.argtypes = [I, I, I, I]
    lib.ob_debug_idesc_bf16.restype = c_uint
    return lib


def available() -> bool:
    """True when a CUDA device is present and the library loads."""
    if not torch.cuda.is_available():
        return False
    try:
        load()
        return True
    except Exception:
        return False


LAUNCHES = 0   # entry points called so far (each launches at least one kernel of this library)


def check(rc: int, what: str) -> None:
    global LAUNCHES
    LAUNCHES += 1
    if rc != 0:
        buf = ctypes.create_string_buffer(256)
        try:
            load().ob_last_cuda_error(buf, 256)
        except Exception:
            pass
        detail = ctypes.create_string_buffer(256)
        try:
            load().ob_last_detail(detail, 256)
        except Exception:
            pass
        raise KernelLibraryError(f"{what} failed with code {rc} ({buf.value.decode(errors='replace')}) "
                                 f"{detail.value.decode(errors='replace')}")


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


@functools.lru_cache(maxsize=None)
def sm_count(device_index: int | None = None) -> int:
    idx = torch.cuda.current_device() if device_index is None else device_index
    return torch.cuda.get_device_properties(idx).multi_processor_count


_WAIT_ERRORS = {1: "a consumer timed out waiting for a TMA stage", 2: "the producer timed out waiting for a free stage",
                3: "the epilogue timed out waiting for an accumulator", 4: "the MMA issuer timed out waiting for TMEM",
                5: "the MMA issuer timed out waiting for the scaler warps", 6: "a peer's flag did not arrive in time",
                7: "draining in-flight copies timed out"}


class DeviceWaitTimeout(KernelLibraryError):
    """A bounded device-side wait expired; the context is still usable."""


class StatusWord:
    """A device int32 that kernels set when a bounded wait expires."""

    def __init__(self, device: torch.device | str | None = None):
        self.tensor = torch.zeros(1, dtype=torch.int32, device=device or "cuda")

    def ptr(self) -> int:
        return self.tensor.data_ptr()

    def read(self) -> int:
        return int(self.tensor.item())

    def raise_if_set(self, what: str = "kernel") -> None:
        code = self.read()
        if code:
            self.tensor.zero_()
            raise DeviceWaitTimeout(f"{what}: {_WAIT_ERRORS.get(code, 'unknown device status')} (code {code})")
