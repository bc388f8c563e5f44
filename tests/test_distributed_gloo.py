"""Two CPU ranks over gloo: collectives, state sync, gradient reduction, empty batches, host-side failure detection."""
import dataclasses
import datetime
import os
import socket
import traceback

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.distributed


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, fn_name, q, timeout_s):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
        dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=timeout_s))
        out = globals()[fn_name](rank, world)
        q.put((rank, "ok", out))
    except Exception as exc:      # noqa: BLE001
        q.put((rank, "error", f"{type(exc).__name__}: {exc}\n{traceback.format_exc()[-800:]}"))
    finally:
        if dist.is_initialized():
            try:
                dist.destroy_process_group()
            except Exception:      # noqa: BLE001
                pass


def run_ranks(fn_name, world=2, timeout_s=60):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, fn_name, q, timeout_s)) for r in range(world)]
    for p in procs:
        p.start()
    results = {}
    for _ in range(world):
        rank, status, payload = q.get(timeout=180)
        results[rank] = (status, payload)
    for p in procs:
        p.join(30)
    return results


# ----------------------------------------------------------------------------------- worker bodies

def w_collectives(rank, world):
    from opaque_b200 import distributed as D
    assert D.is_distributed() and D.get_rank() == rank and D.get_world_size() == 2
    t = D.all_reduce(torch.tensor([float(rank + 1)]))
    assert float(t) == 3.0 and float(D.all_reduce(torch.tensor([float(rank + 1)]), "mean")) == 1.5
    assert D.reduce_scalar(rank + 1, "sum") == 3 and isinstance(D.reduce_scalar(rank + 1, "sum"), int)
    assert D.reduce_scalar(0.5 * (rank + 1), "max") == 1.0
    g = D.gather_tensors(torch.arange(rank + 1).float())
    assert g.tolist() == [0.0, 0.0, 1.0]
    assert D.gather_tensors(torch.zeros(0)).numel() == 0
    shard = D.local_shard(list(range(7)))
    assert shard == ([0, 1, 2] if rank == 0 else [3, 4, 5, 6])
    D.assert_scalar_equal(4.0, name="same")
    try:
        D.assert_scalar_equal(float(rank), name="differs")
        raise AssertionError("expected a mismatch")
    except RuntimeError:
        pass
    try:
        D.assert_string_equal(f"seed-{rank}")
        raise AssertionError("expected a mismatch")
    except RuntimeError:
        pass
    D.assert_pytree_equal({"a": torch.ones(3)})
    return True


def w_gradients(rank, world):
    from opaque_b200 import distributed as D
    from opaque_b200.types import clipped, noised
    tree = clipped({"w": torch.full((3,), float(rank + 1)), "b": torch.full((2,), 1.0)}, 0.5)
    out = D.sum_gradients_(tree)
    assert out.pytree["w"].tolist() == [3.0] * 3 and out.max_norm == 0.5
    n = D.reduce_pytree(noised({"w": torch.ones(2)}, 1.0, 2.0), "sum")
    assert abs(n.noise_stddev - 2.0 * 2 ** 0.5) < 1e-12 and n.max_norm == 1.0
    m = D.reduce_pytree(noised({"w": torch.ones(2)}, 1.0, 2.0), "mean")
    assert abs(m.noise_stddev - 2.0 / 2 ** 0.5) < 1e-12 and m.max_norm == 0.5
    try:
        D.sum_gradients_(clipped({"w": torch.ones(1)}, 1.0 + rank))
        raise AssertionError("metadata mismatch must raise")
    except RuntimeError:
        pass
    return True


@dataclasses.dataclass(frozen=True)
class _State:
    count: int
    total: float
    local_only: str
    step: int


def w_sync_object(rank, world):
    from opaque_b200 import distributed as D
    st = _State(rank + 1, 0.5, f"r{rank}", 7)
    out = D.sync_object(st, {"count": "sum", "total": "max", "local_only": "local", "step": "assert_equal"})
    assert out == _State(3, 0.5, f"r{rank}", 7)
    # a bad schema raises on every rank BEFORE any collective is issued (nobody is left waiting)
    for bad in ({"count": "sum"}, {"count": "sum", "total": "nope", "local_only": "local", "step": "local"}):
        try:
            D.sync_object(st, bad)
            raise AssertionError("schema must be rejected")
        except ValueError:
            pass
    try:
        D.sync_object(_State(1, 0.5, "x", rank), {"count": "sum", "total": "max", "local_only": "local", "step": "assert_equal"})
        raise AssertionError("diverged field must raise")
    except RuntimeError:
        pass
    return True


def _train(rank, world, steps=3):
    """Shared-noise DP-SGD on a tiny model; rank 1 gets an EMPTY batch on step 1."""
    from opaque_b200 import optimizers
    from opaque_b200.distributed import sum_gradients_, sync
    from opaque_b200.dpsgd import clipped_grad, gaussian_noise
    from opaque_b200.random import key
    torch.manual_seed(0)
    X, Y = torch.randn(16, 4), torch.randn(16, 2)
    params = {"w": torch.zeros(2, 4)}

    def loss(p, x, y):
        return ((p["w"] @ x - y) ** 2).sum()
    gf, cs = clipped_grad(loss, clipping_norm=1.0, normalize_by=8.0, batch_argnums=(1, 2), return_aux=True)
    nf, ns = gaussian_noise(noise_multiplier=0.5, key=key(1))
    opt = optimizers.sgd(lr=0.1)
    os_ = opt.init(params)
    for t in range(steps):
        lo = t * 4
        idx = list(range(lo, lo + 4))
        if world == 2:
            idx = idx[:2] if rank == 0 else idx[2:]
            if t == 1:
                idx = idx + list(range(lo + 2, lo + 4)) if rank == 0 else []
        gi = torch.as_tensor(idx, dtype=torch.long)
        (g, aux), cs = gf(params, X[gi], Y[gi], state=cs)
        cs, aux = sync(cs, aux)
        g = sum_gradients_(g)
        noisy, ns = nf(g, ns)
        ns = sync(ns)
        u, os_ = opt.update(noisy, os_, params=params)
        params = optimizers.apply_updates(params, u)
        assert aux.batch_size == 4
    optimizers.sync_optimizer_state(os_)
    return params["w"].tolist()


def w_training_parity(rank, world):
    return _train(rank, world)


def w_rank_raises(rank, world):
    """Rank 1 fails on the host before the step; rank 0 learns of it through the packed consensus flag."""
    from opaque_b200.distributed import reduce_scalar
    failed = False
    try:
        if rank == 1:
            raise MemoryError("simulated out of memory on rank 1")
    except MemoryError:
        failed = True
    anyone = bool(reduce_scalar(int(failed), "max"))
    assert anyone
    return "stepped down together"


def w_peer_never_joins(rank, world):
    """Rank 1 leaves between steps without joining the collective; rank 0's collective ends with an error."""
    if rank == 1:
        return "left"
    try:
        dist.all_reduce(torch.ones(1))
    except Exception as exc:      # noqa: BLE001
        return f"detected: {type(exc).__name__}"
    return "no error"


# ----------------------------------------------------------------------------------- tests

@pytest.mark.parametrize("fn", ["w_collectives", "w_gradients", "w_sync_object", "w_rank_raises"])
def test_two_rank_contracts(fn):
    res = run_ranks(fn)
    assert all(s == "ok" for s, _ in res.values()), res


def test_two_rank_training_matches_single_process():
    res = run_ranks("w_training_parity")
    assert all(s == "ok" for s, _ in res.values()), res
    single = _train(0, 1)
    for r in (0, 1):
        assert torch.allclose(torch.tensor(res[r][1]), torch.tensor(single), atol=1e-6)


def test_missing_peer_is_detected_by_timeout():
    res = run_ranks("w_peer_never_joins", timeout_s=5)
    assert res[1] == ("ok", "left")
    assert res[0][0] == "ok" and res[0][1].startswith("detected"), res


def test_leave_notice_is_seen_on_the_host_before_the_next_step():
    """A rank that leaves between steps announces it through the store; the others raise before launching anything."""
    import torch.distributed as dist
    from opaque_b200.parallel.peer import Liveness, PeerLeftError
    store = dist.HashStore()
    a, b, c = (Liveness(r, 3, store=store) for r in range(3))
    a.check(), b.check(), c.check()
    b.announce_leave("preempted")
    with pytest.raises(PeerLeftError, match="preempted"):
        a.check()
    assert c.left() == [1] and b.left() == []


class _EvalLM(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.emb = torch.nn.Embedding(32, 8)
        self.head = torch.nn.Linear(8, 32)

    def forward(self, ids):
        return self.head(self.emb(ids))


def _eval_once(rank, world):
    from opaque_b200.transformers import DPTrainer, TrainingArguments
    torch.manual_seed(0)
    g = torch.Generator().manual_seed(4)
    # ragged: the second half of the set is longer, so the two ranks' shards are padded to different lengths
    data = [{"input_ids": torch.randint(0, 32, (6 if i < 7 else 10,), generator=g).tolist()} for i in range(14)]
    seen = {}

    def metrics(ep):
        seen["shape"] = tuple(ep.predictions.shape)
        keep = ep.label_ids != -100
        return {"labelled_tokens": int(keep.sum()), "loss_mean": float(ep.losses.mean())}

    args = TrainingArguments(output_dir=None, use_cpu=True, privacy_noise_multiplier=1.0, per_device_eval_batch_size=3,
                             eval_accumulation_steps=1, include_for_metrics=["loss"], seed=1)
    tr = DPTrainer(model=_EvalLM(), args=args, train_dataset=data, eval_dataset=data, compute_metrics=metrics)
    out = tr.evaluate()
    return {"shape": seen["shape"], "tokens": out["eval_labelled_tokens"], "loss": out["eval_loss"], "loss_mean": out["eval_loss_mean"],
            "samples": out["eval_samples"]}


def w_trainer_evaluate(rank, world):
    return _eval_once(rank, world)


def test_two_rank_evaluation_gathers_predictions_for_compute_metrics():
    """Each rank evaluates its shard; ``compute_metrics`` gets ALL predictions (shards padded to a common length and gathered)."""
    res = run_ranks("w_trainer_evaluate")
    assert all(s == "ok" for s, _ in res.values()), res
    single = _eval_once(0, 1)
    for r in (0, 1):
        got = res[r][1]
        assert got["shape"] == (14, 10, 32) == single["shape"] and got["samples"] == 14.0
        assert got["tokens"] == single["tokens"]
        assert abs(got["loss"] - single["loss"]) < 1e-5 and abs(got["loss_mean"] - single["loss_mean"]) < 1e-5
