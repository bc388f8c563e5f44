"""Flat parameter space with ZeRO-style sharded DP state and the fused DP optimizer step.

Layout.  Trainable parameters are laid out back to back (each start aligned to 64 elements) in
one flat index space, *direct* parameters first (those whose per-example gradients are
materialised: LoRA factors, biases, norm weights) and *ghost* parameters after them (large
matrices handled by the ghost-norm / clip-GEMM pair).  The space is padded so that it splits
into W equal contiguous shards.

  * ``params``  bf16, full length, one copy per rank in peer memory — model parameters are views
                 of it, and owners store updated values into EVERY rank's copy;
  * ``grad``    fp32, one shard per rank in peer memory — producers on any rank reduce
                 (``red.global.add``) clipped gradient sums straight into the owner's shard;
  * ``master``, ``m``, ``v`` (and DP-FTRL buffers) fp32, one shard per rank, local.

Step.  ``barrier → shard_step → barrier`` on the compute stream: the first barrier orders all
ranks' gradient reductions before the owner reads its shard, the fused kernel adds Philox (or
correlated) noise exactly once per coordinate, applies AdamW with noise bias correction to the
fp32 masters and pushes bf16 parameters to all peers, and the second barrier orders those
stores before the next forward pass.

Replaces: per-leaf NCCL all-reduce (packages/opaque-engine/src/opaque/api/engine/distributed/
gradients.py:183-193), CPU-generated noise (packages/opaque-dpsgd/src/opaque/api/dpsgd/noise/
_gaussian.py:235-278), tree-mapped AdamW-BC (packages/opaque-optimizers/src/opaque/api/optimizers/
_adam.py:120-270) and the streaming C⁻¹ noise (packages/opaque-dpftrl/src/opaque/api/dpftrl/noise/
_engine.py:359-410).
"""
from __future__ import annotations

import dataclasses
import math
from collections.abc import Callable, Sequence
from typing import Any

import torch
import torch.distributed as dist

from .. import ops
from ..random import RngKey, fold_in
from .peer import PeerGroup

ALIGN = 64
LOCAL_ACCUMULATE_LIMIT_BYTES = 16 << 30      # "auto": accumulate locally when the full fp32 gradient fits in 16 GiB
LOCAL_ACCUMULATE_RESERVE_BYTES = 32 << 30    # ... or when this much device memory stays free after it and the optimizer shards


@dataclasses.dataclass(frozen=True)
class Slot:
    name: str
    offset: int
    numel: int
    shape: tuple[int, ...]
    direct: bool


def default_direct(name: str, p: torch.nn.Parameter) -> bool:
    """Vectors (biases, norm weights) and LoRA factors get materialised per-example gradients."""
    return p.ndim < 2 or "lora_" in name.rsplit(".", 1)[-1]


class FlatSpace:
    """Offsets of every trainable parameter in the flat space, and the peer buffers behind it."""

    def __init__(self, named_params: Sequence[tuple[str, torch.nn.Parameter]], group: PeerGroup, *,
                 direct: Callable[[str, torch.nn.Parameter], bool] | None = None,
                 group_of: Callable[[str], str] | None = None, accumulate: str = "peer"):
        """``accumulate="peer"`` (default): producer kernels reduce every microbatch's tiles straight into the owners'
        shards.  ``"local"``: they add into a full-length local fp32 buffer and ONE push per step reduces it into the
        owners' shards — (microbatches per step)× less reduction traffic over NVLink at the price of ``4·P`` bytes.
        ``"pull"``: like ``"local"``, but the buffer lives in peer-mapped memory and nothing is pushed: the fused shard
        step READS its shard from every rank's buffer through peer pointers and adds the W values in rank order — the
        reduce-scatter runs inside the optimizer kernel, without atomics and with the same bits whatever the arrival
        order; one kernel and one pass over the gradient fewer per step.
        ``"auto"``: the pull form while that buffer stays under ``LOCAL_ACCUMULATE_LIMIT_BYTES`` or leaves
        ``LOCAL_ACCUMULATE_RESERVE_BYTES`` of device memory free."""
        if accumulate not in ("peer", "local", "pull", "auto"):
            raise ValueError("accumulate must be 'peer', 'local', 'pull' or 'auto'")
        self.group = group
        is_direct = direct or default_direct
        label = group_of or (lambda name: "")
        # stable: direct parameters first, and inside them every clipping group contiguous.  The LoRA `A` factors of the
        # q, k and v projections of one attention block are placed back to back (at the position of the block's first
        # one), so their per-example gradients `[q_i | k_i | v_i]ᵀ x_i` are ONE GEMM launch writing one contiguous range.
        names = [n for n, _ in named_params]
        index = {n: i for i, n in enumerate(names)}

        def position(name: str) -> tuple:
            for j, proj in enumerate(("q_proj", "k_proj", "v_proj")):
                tail = f".{proj}.lora_A"
                if name.endswith(tail):
                    first = name[: -len(tail)] + ".q_proj.lora_A"
                    if first in index and all(name[: -len(tail)] + f".{p}.lora_A" in index for p in ("k_proj", "v_proj")):
                        return (index[first], j)
            return (index[name], 0)
        ordered = sorted(named_params, key=lambda np_: (not is_direct(*np_), label(np_[0]) if is_direct(*np_) else "",
                                                        position(np_[0])))
        self.slots: dict[str, Slot] = {}
        self.group_label: dict[str, str] = {}
        self.direct_ranges: dict[str, tuple[int, int]] = {}
        self.direct_elems = 0
        off = 0
        for name, p in ordered:
            d = bool(is_direct(name, p))
            self.slots[name] = Slot(name, off, p.numel(), tuple(p.shape), d)
            self.group_label[name] = label(name)
            end = off + (p.numel() + ALIGN - 1) // ALIGN * ALIGN
            if d:
                lo, _ = self.direct_ranges.get(label(name), (off, off))
                self.direct_ranges[label(name)] = (lo, end)
                self.direct_elems = end
            off = end
        chunk = group.world * ALIGN
        self.used = off                    # flat length without the padding that depends on the number of ranks
        self.total = max((off + chunk - 1) // chunk * chunk, chunk)
        self.shard = self.total // group.world
        self.shard_lo = group.rank * self.shard
        self.params = group.buffer(self.total, torch.bfloat16)
        self.grad = group.buffer(self.shard, torch.float32)
        dev = group.device
        can_pull = group.world == 1 or group.use_ipc       # the pull form needs every rank's buffer mapped here
        if accumulate == "pull" and not can_pull:
            raise ValueError("accumulate='pull' needs peer-mapped buffers (PeerGroup(use_ipc=True))")
        if accumulate == "auto":     # measured on 4 GPUs: per-microbatch peer reductions cost 15-35 % for 0.1-1 B parameter
            # models; between the two once-per-step forms the pull form saves the push kernel and its pass over the buffer
            accumulate = ("pull" if can_pull else "local") if self._local_accumulation_fits() else "peer"
        self.accumulate = accumulate if group.world > 1 else "peer"
        self.grad_full = torch.zeros(self.total, dtype=torch.float32, device=dev) if self.accumulate == "local" else None
        self.grad_full_table = None        # "pull": device table of every rank's accumulation buffer
        if self.accumulate == "pull":
            self._grad_full_buffer = group.buffer(self.total, torch.float32)
            self.grad_full, self.grad_full_table = self._grad_full_buffer.local, self._grad_full_buffer.table
        self.master = torch.zeros(self.shard, dtype=torch.float32, device=dev)
        self.m = torch.zeros_like(self.master)
        self.v = torch.zeros_like(self.master)
        self._named = list(ordered)
        import hashlib
        self.layout_hash = hashlib.sha256(";".join(f"{sl.name}@{sl.offset}+{sl.numel}" for sl in self.slots.values()).encode()).hexdigest()[:16]

    # ---- binding --------------------------------------------------------------------------
    @torch.no_grad()
    def bind(self) -> None:
        """Move parameter storage into the flat bf16 buffer and initialise the fp32 masters of this rank's shard.

        Rank 0's values win (one broadcast per parameter) so that replicas start identical.  Works slot by slot: no
        full-length temporary is created, so a model that fills most of the GPU can still be bound.
        """
        pg = self.group.pg
        lo_s, hi_s = self.shard_lo, self.shard_lo + self.shard
        for name, p in self._named:
            if self.group.world > 1:
                src = dist.get_global_rank(pg, 0) if pg is not dist.group.WORLD else 0
                dist.broadcast(p.data, src=src, group=pg)
            s = self.slots[name]
            flat = p.detach().reshape(-1)
            self.params.local[s.offset:s.offset + s.numel].copy_(flat)                  # rounds to bf16
            lo, hi = max(s.offset, lo_s), min(s.offset + s.numel, hi_s)
            if lo < hi:                                                                   # masters keep the source precision
                self.master[lo - lo_s:hi - lo_s].copy_(flat[lo - s.offset:hi - s.offset])
            p.data = self.params.local[s.offset:s.offset + s.numel].view(s.shape)         # frees the old storage
        if self.group.world > 1:
            torch.cuda.synchronize(self.group.device)
            dist.barrier(group=pg)

    def view_of(self, name: str, flat: torch.Tensor) -> torch.Tensor:
        s = self.slots[name]
        return flat[s.offset:s.offset + s.numel].view(s.shape)

    # ---- gradient destinations for producers ------------------------------------------------
    def grad_target(self) -> dict[str, Any]:
        """Keyword arguments that route a producer kernel's output into the sharded gradient."""
        if self.group.world == 1:
            return {"out": self.grad.local, "peer_table": None, "shard_elems": 0}
        if self.grad_full is not None:
            return {"out": self.grad_full, "peer_table": None, "shard_elems": 0}
        return {"out": None, "peer_table": self.grad.table, "shard_elems": self.shard}

    def _local_accumulation_fits(self) -> bool:
        """``accumulate="auto"``: take the local fp32 buffer when it is small (under ``LOCAL_ACCUMULATE_LIMIT_BYTES``) or
        when, after it and the optimizer shards, ``LOCAL_ACCUMULATE_RESERVE_BYTES`` of device memory stay free for
        activations.  Ranks agree on the answer (the minimum), so one tight GPU keeps every rank on peer reductions."""
        local_bytes = 4 * self.total
        fits = local_bytes <= LOCAL_ACCUMULATE_LIMIT_BYTES
        dev = self.group.device
        if not fits and dev.type == "cuda" and self.group.world > 1:
            free, _total = torch.cuda.mem_get_info(dev)
            shards = 3 * 4 * self.shard                      # master, m, v (allocated right after this decision)
            fits = free - local_bytes - shards >= LOCAL_ACCUMULATE_RESERVE_BYTES
        if self.group.world > 1 and torch.distributed.is_available() and torch.distributed.is_initialized():
            flag = torch.tensor([1 if fits else 0], dtype=torch.int32, device=dev)
            torch.distributed.all_reduce(flag, op=torch.distributed.ReduceOp.MIN)
            fits = bool(int(flag.item()))
        return fits

    def push_local_gradient(self) -> None:
        """``accumulate="local"``: reduce this rank's accumulated gradient into the owners' shards (before the barrier)."""
        if self.grad_full is not None and self.grad_full_table is None:
            ops.push_grad_(self.grad_full, self.grad.table, self.shard, status=self.group.status)

    @torch.no_grad()
    def gather_full(self, shard_tensor: torch.Tensor) -> torch.Tensor:
        """All ranks' shards of a local fp32 state concatenated (checkpointing / tests)."""
        if self.group.world == 1:
            return shard_tensor.clone()
        out = torch.empty(self.total, dtype=shard_tensor.dtype, device=shard_tensor.device)
        dist.all_gather_into_tensor(out, shard_tensor.contiguous(), group=self.group.pg)
        return out


@dataclasses.dataclass
class DPStepConfig:
    lr: float | Callable[[int], float] = 1e-3
    betas: tuple[float, float] = (0.9, 0.999)
    eps: float = 1e-8
    weight_decay: float = 0.0
    decoupled_weight_decay: bool = True
    noise_bias_correction: bool = True
    optimizer: str = "adam"            # "adam" (Adam / AdamW / AdamW-BC), "sgd" (momentum = betas[0]) or "lion" (betas)
    nesterov: bool = False             # SGD only


class ShardedDPOptimizer:
    """Noise + AdamW-BC over the owner's shard, fused with the parameter all-gather.

    ``mechanism`` is ``None`` (iid Gaussian, DP-SGD) or a dict describing a DP-FTRL inverse:
    ``{"kind": "blt", "scale": [...], "decay": [...]}``, ``{"kind": "banded", "coef": [...]}``
    (``coef[0]`` the diagonal of ``C``; the state holds ``len(coef) − 1`` previous outputs) or
    ``{"kind": "fir", "coef": [...]}`` (taps of a banded ``C⁻¹``; the state holds previous raw draws).  A ``"coef_fn"``
    entry (``step -> coefficients`` of the same length) replaces the coefficients before every step: mechanisms whose
    rows are scaled step by step (column-normalised λ-CGD).  Up to 63 history buffers (32 BLT pairs).
    """

    def __init__(self, space: FlatSpace, config: DPStepConfig, *, key: RngKey, mechanism: dict | None = None):
        self.space, self.cfg, self.key = space, config, key
        self.step_count = 0
        self.phi = 0.0
        self.mechanism = mechanism
        self.timing: list[tuple] | None = None     # set to [] to record CUDA events around barrier / step / barrier
        self.ftrl_state = None
        self.nbuf = 0
        self.mode = 0
        self.coef: list[float] = []
        if mechanism is not None:
            if mechanism["kind"] == "blt":
                s, d = list(mechanism["scale"]), list(mechanism["decay"])
                if len(s) != len(d) or not 1 <= len(s) <= 32:
                    raise ValueError("BLT needs 1..32 (scale, decay) pairs")
                self.mode, self.nbuf, self.coef = 1, len(s), [float(x) for x in s + d]
            elif mechanism["kind"] == "banded":
                c = [float(x) for x in mechanism["coef"]]
                if not 2 <= len(c) <= 64 or c[0] == 0:
                    raise ValueError("banded inverse needs 2..64 coefficients with a non-zero diagonal")
                self.mode, self.nbuf, self.coef = 2, len(c) - 1, c
            elif mechanism["kind"] == "fir":
                c = [float(x) for x in mechanism["coef"]]
                if not 2 <= len(c) <= 64:
                    raise ValueError("FIR noise needs 2..64 taps")
                self.mode, self.nbuf, self.coef = 3, len(c) - 1, c
            else:
                raise ValueError(f"unknown mechanism kind {mechanism['kind']!r}")
            self.ftrl_state = torch.zeros(self.nbuf, space.shard, dtype=torch.float32, device=space.group.device)

    def noise_row_norm(self) -> float:
        """``‖row_t(C⁻¹)‖`` for the current step (1 for iid noise): the factor between σ and the realised std."""
        return 1.0

    @torch.no_grad()
    def step(self, *, noise_std: float, normalize_by: float, noisy_out: torch.Tensor | None = None,
             skip_update: bool = False) -> None:
        sp, g = self.space, self.space.group
        t = self.step_count + 1
        lr = float(self.cfg.lr(self.step_count)) if callable(self.cfg.lr) else float(self.cfg.lr)
        b1, b2 = self.cfg.betas
        var = (noise_std / normalize_by) ** 2
        bc = self.cfg.noise_bias_correction and self.cfg.optimizer == "adam"
        if bc:
            self.phi = b2 * self.phi + (1 - b2) * var
        phi_hat = self.phi / (1 - b2 ** t) if bc else 0.0
        if self.mechanism is not None and callable(self.mechanism.get("coef_fn")):
            c = [float(x) for x in self.mechanism["coef_fn"](self.step_count)]
            if len(c) != len(self.coef):
                raise ValueError("coef_fn must keep the number of coefficients")
            self.coef = c
        seed = fold_in(self.key, self.step_count).seed
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)] if self.timing is not None else None
        if ev:
            ev[0].record()
        sp.push_local_gradient()
        g.barrier()
        if ev:
            ev[1].record()
        pull = sp.grad_full_table is not None
        ops.shard_step(
            grad=None if pull else sp.grad.local, peer_grad=sp.grad_full_table if pull else None, master=sp.master, m=sp.m, v=sp.v,
            params_local=sp.params.local if g.world == 1 else None,
            peer_params=sp.params.table if g.world > 1 else None, world=g.world, global_offset=sp.shard_lo,
            seed=seed, noise_std=noise_std, inv_normalize=1.0 / normalize_by, lr=lr, betas=(b1, b2),
            eps=self.cfg.eps, weight_decay=self.cfg.weight_decay, step=t, phi_hat=phi_hat,
            decoupled_wd=self.cfg.decoupled_weight_decay, ftrl_state=self.ftrl_state, ftrl_mode=self.mode,
            ftrl_coef=self.coef, nbuf=self.nbuf, ring_head=(self.step_count % self.nbuf) if self.mode in (2, 3) else 0,
            noisy_out=noisy_out, skip_update=skip_update, status=g.status if g.world > 1 else None,
            optimizer=self.cfg.optimizer, nesterov=self.cfg.nesterov)
        if ev:
            ev[2].record()
        g.barrier()
        if pull:            # every rank has read its shard out of this buffer: clear it for the next step's producers
            sp.grad_full.zero_()
        if ev:
            ev[3].record()
            self.timing.append(tuple(ev))
        self.step_count = t

    def timing_ms(self) -> dict[str, float]:
        """Mean milliseconds per step of: waiting for all ranks' gradient reductions, the fused noise + optimizer +
        parameter push kernel, and waiting for all ranks' parameter stores (needs ``timing = []`` before the steps)."""
        rows = self.timing or []
        if not rows:
            return {"grad_barrier_ms": 0.0, "shard_step_ms": 0.0, "param_barrier_ms": 0.0}
        torch.cuda.synchronize(self.space.group.device)
        n = len(rows)
        return {"grad_barrier_ms": sum(r[0].elapsed_time(r[1]) for r in rows) / n,
                "shard_step_ms": sum(r[1].elapsed_time(r[2]) for r in rows) / n,
                "param_barrier_ms": sum(r[2].elapsed_time(r[3]) for r in rows) / n}

    # ---- checkpoint -----------------------------------------------------------------------
    def state_dict(self) -> dict[str, Any]:
        """Full (unsharded) optimizer state on every rank; rank 0 writes it.

        The tensors are cut to ``used`` elements — the layout's own length, without the tail padding that makes the
        space divisible by the number of ranks — so a run saved on N GPUs resumes on any other number."""
        sp = self.space
        n = sp.used
        sd = {"step": self.step_count, "phi": self.phi, "key_seed": str(self.key.seed),
              "master": sp.gather_full(sp.master)[:n].cpu(), "m": sp.gather_full(sp.m)[:n].cpu(),
              "v": sp.gather_full(sp.v)[:n].cpu(), "used": n, "layout": sp.layout_hash}
        if self.ftrl_state is not None:
            sd["ftrl_state"] = torch.stack([sp.gather_full(self.ftrl_state[b])[:n] for b in range(self.nbuf)]).cpu()
        return sd

    @torch.no_grad()
    def load_state_dict(self, sd: dict[str, Any]) -> None:
        sp = self.space
        n = int(sd["used"]) if "used" in sd else min(int(sd["total"]), sp.used)   # older files stored the padded length
        if n != sp.used or ("used" not in sd and int(sd["total"]) < sp.used):
            raise ValueError(f"checkpoint was written for a different parameter layout ({n} flat elements, this model has {sp.used})")
        if sd.get("layout") is not None and sd["layout"] != sp.layout_hash:
            raise ValueError("checkpoint was written for a different order of the parameters in the flat space "
                             f"(layout {sd['layout']}, this build lays them out as {sp.layout_hash})")
        lo, hi = sp.shard_lo, sp.shard_lo + sp.shard
        self.step_count, self.phi = int(sd["step"]), float(sd["phi"])

        def shard_of(full: torch.Tensor) -> torch.Tensor:
            """This rank's slice of a saved flat tensor, zero beyond the saved length (re-padding for this world size)."""
            out = torch.zeros(*full.shape[:-1], sp.shard, dtype=full.dtype)
            a, b = min(lo, n), min(hi, n)
            if b > a:
                out[..., :b - a] = full[..., a:b]
            return out
        sp.master.copy_(shard_of(sd["master"]))
        sp.m.copy_(shard_of(sd["m"]))
        sp.v.copy_(shard_of(sd["v"]))
        sp.params.local[:n].copy_(sd["master"][:n].to(torch.bfloat16))
        if self.ftrl_state is not None and "ftrl_state" in sd:
            self.ftrl_state.copy_(shard_of(sd["ftrl_state"]))
