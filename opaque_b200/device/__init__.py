"""Device capability probe.

The framework targets one accelerator: NVIDIA B200 (compute capability 10.0,
``sm_100a``).  ``fused_kernels_available()`` is true when a CUDA device of that
generation is visible *and* the in-tree kernel library loads; CPU runs use the
plain PyTorch reference implementations of every op.

Parity: packages/opaque-engine/src/opaque/api/engine/device/_capabilities.py.
"""
from __future__ import annotations

import dataclasses
import functools

import torch


@dataclasses.dataclass(frozen=True)
class DeviceCapabilities:
    device_type: str
    name: str
    compute_capability: tuple[int, int] | None
    is_blackwell: bool
    total_memory_bytes: int
    multiprocessor_count: int
    supports_bf16: bool
    fused_kernels: bool
    peer_access: bool

    # the reference's names for the same facts
    @property
    def is_accelerator(self) -> bool:
        return self.device_type != "cpu"

    @property
    def supports_fused_kernels(self) -> bool:
        return self.fused_kernels

    @property
    def supports_compile(self) -> bool:
        """No tracing compiler is used on the hot path; ``torch.compile`` itself works wherever PyTorch supports it."""
        return self.device_type in ("cuda", "cpu")

    @property
    def recommended_compile_backend(self) -> str | None:
        return None

    @property
    def peak_memory_trackable(self) -> bool:
        return self.device_type == "cuda"

    @property
    def supports_pin_memory(self) -> bool:
        return self.device_type == "cuda"


@functools.lru_cache(maxsize=None)
def _probe(index: int) -> DeviceCapabilities:
    if not torch.cuda.is_available():
        return DeviceCapabilities("cpu", "cpu", None, False, 0, 0, True, False, False)
    p = torch.cuda.get_device_properties(index)
    cc = (p.major, p.minor)
    blackwell = cc[0] == 10
    fused = False
    if blackwell:
        try:
            from ..ops import lib
            fused = lib.available()
        except Exception:
            fused = False
    peers = torch.cuda.device_count() > 1
    return DeviceCapabilities("cuda", p.name, cc, blackwell, p.total_memory,
                              p.multi_processor_count, True, fused, peers)


def device_capabilities(device: torch.device | str | int | None = None) -> DeviceCapabilities:
    """What the current device offers (bf16, fused kernels, peer access, memory) as a ``DeviceCapabilities``."""
    if device is None:
        idx = torch.cuda.current_device() if torch.cuda.is_available() else 0
    elif isinstance(device, int):
        idx = device
    else:
        d = torch.device(device)
        if d.type != "cuda":
            return DeviceCapabilities(d.type, d.type, None, False, 0, 0, True, False, False)
        idx = d.index if d.index is not None else torch.cuda.current_device()
    return _probe(idx)


def fused_kernels_available() -> bool:
    """True on a B200 with the sm_100a kernel library loaded."""
    return device_capabilities().fused_kernels


def sdpa_autocast_under_vmap_broken(device_type: str | None = None) -> bool:
    """An Apple-MPS quirk of the reference; never true on CUDA or CPU (``device_type`` is accepted for call compatibility)."""
    return False


__all__ = ["DeviceCapabilities", "device_capabilities", "fused_kernels_available",
           "sdpa_autocast_under_vmap_broken"]
