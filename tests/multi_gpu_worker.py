"""Worker for the multi-GPU test: W ranks (one per GPU) against a single-process per-example oracle.

Launched by ``tests/test_gpu_multi.py`` through ``python -m torch.distributed.run``.  Every rank holds the same
model; rank r takes examples ``r::W`` of a common batch.  Checks, on the device and through the peer-memory path only:

  (mode ``pull``: nothing is pushed; the shard step reads every rank's accumulation buffer through peer pointers and
  adds them in rank order — checked bit for bit.)

  1. the clip-weighted gradient sums that all ranks reduce into the owners' shards equal the oracle's sum over the
     whole batch (peer ``red.add`` reduce-scatter fused into the producer kernels);
  2. the noise that each owner adds to its shard is the same Philox stream a single rank would draw (exactly once
     per coordinate, no overlap or gap at shard boundaries);
  3. after the step every rank's bf16 parameter copy is bit-identical (owners push their slices to all peers).
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def short_run(rank: int, world: int, dev, out_path: str) -> int:
    """Five full DP steps (noise on) over common global batches; rank 0 writes the final parameters.

    The batches are dealt out ``rank::world``, the noise is keyed by the global coordinate, so a 1-rank and a W-rank run
    must end at (nearly) the same parameters: only the order of fp32 reductions differs.
    """
    from opaque_b200.engine.fused import FusedDPEngine
    from opaque_b200.models import LlamaConfig, LlamaForCausalLM, shift_labels
    from opaque_b200.parallel.sharded import DPStepConfig
    from opaque_b200.random import key
    torch.manual_seed(0)
    cfg = LlamaConfig(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=256)
    model = LlamaForCausalLM(cfg, device=dev)
    eng = FusedDPEngine(model, clipping_norm=1.0, noise_multiplier=0.6, normalize_by=8.0, key=key(21),
                        step_config=DPStepConfig(lr=3e-3, noise_bias_correction=False), microbatch_size=2)
    # plain AdamW here: with the noise bias correction a coordinate whose corrected second moment lands within one ulp of
    # zero switches between sqrt(v - phi) and sqrt(v) on a last-bit difference of the reduction order, and its update
    # changes by orders of magnitude -- expected for that formula, but not what this comparison is about
    g = torch.Generator().manual_seed(5)
    losses = []
    for step in range(5):
        ids = torch.randint(0, 512, (8, 128), generator=g).to(dev)
        labels = shift_labels(ids, 1.0)
        res = eng.step(model.per_example_loss, {"input_ids": ids[rank::world], "labels": labels[rank::world]})
        t = torch.tensor([res.loss * res.batch_size, float(res.batch_size)], device=dev)
        if world > 1:
            dist.all_reduce(t)
        losses.append(float(t[0] / t[1]))
    torch.cuda.synchronize()
    ok = eng.status.read() == 0
    if rank == 0:
        torch.save({"params": {n: p.detach().float().cpu() for n, p in model.named_parameters()}, "losses": losses}, out_path)
    if world > 1:
        dist.barrier()
    eng.group.close()
    if world > 1:
        dist.destroy_process_group()
    return 0 if ok else 1


def main() -> int:
    from opaque_b200 import ops
    from opaque_b200.engine.fused import CLIP_GUARD, FusedDPEngine
    from opaque_b200.models import LlamaConfig, LlamaForCausalLM, shift_labels
    from opaque_b200.parallel.sharded import DPStepConfig
    from opaque_b200.random import fold_in, key
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank)))
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    mode = sys.argv[1] if len(sys.argv) > 1 else "full"
    if mode == "parity":
        return short_run(rank, world, dev, sys.argv[2])
    torch.manual_seed(0)
    cfg = LlamaConfig(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=256)
    model = LlamaForCausalLM(cfg, device=dev)
    if mode == "lora":
        model.add_lora(16, 32.0)
        with torch.no_grad():
            for n, p in model.named_parameters():
                if "lora_B" in n:
                    p.normal_(0, 0.05)
    B, C = 4 * world, 1.0
    ids = torch.randint(0, 512, (B, 128), device=dev)
    dist.broadcast(ids, 0)
    labels = shift_labels(ids, 1.0)
    eng = FusedDPEngine(model, clipping_norm=C, noise_multiplier=0.0, normalize_by=float(B), key=key(11),
                        step_config=DPStepConfig(lr=1e-2), microbatch_size=2, accumulate={"local": "local", "pull": "pull", "full": "peer"}.get(mode, "auto"))
    sp = eng.space
    # oracle AFTER binding (parameters are now the broadcast bf16 values), per example, on every rank
    total = {n: torch.zeros_like(p, dtype=torch.float32) for n, p in model.named_parameters() if p.requires_grad}
    for i in range(B):
        model.zero_grad(set_to_none=True)
        model.per_example_loss(ids[i:i + 1], labels[i:i + 1]).sum().backward()
        g = {n: p.grad.float() for n, p in model.named_parameters() if p.requires_grad}
        nrm = torch.sqrt(sum((v ** 2).sum() for v in g.values()))
        c = min(1.0, C / float(nrm)) * CLIP_GUARD
        for n in total:
            total[n] += c * g[n]
    model.zero_grad(set_to_none=True)
    flat_ref = torch.zeros(sp.total, device=dev)
    for n, g in total.items():
        s = sp.slots[n]
        flat_ref[s.offset:s.offset + s.numel] = g.reshape(-1)

    mine = {"input_ids": ids[rank::world], "labels": labels[rank::world]}
    eng.accumulate(model.per_example_loss, mine)
    sp.push_local_gradient()                 # no-op unless gradients were accumulated locally
    eng.group.barrier()
    torch.cuda.synchronize()
    eng.group.check("accumulate")
    if mode == "pull":
        assert sp.accumulate == "pull"
    if sp.accumulate == "pull":              # also what "auto" picks for a model this small
        # nothing was pushed: the shard's gradient is the rank-ordered sum of every rank's accumulation buffer, which the
        # shard step forms itself.  Read it here the same way (peer views), and check the kernel's sum against it bit by bit.
        assert sp.grad_full_table is not None
        got = torch.zeros(sp.shard, device=dev)
        for r in range(world):
            got += sp._grad_full_buffer.peer_view(r)[sp.shard_lo:sp.shard_lo + sp.shard]
        pulled = [torch.empty(sp.shard, device=dev) for _ in range(2)]
        for out in pulled:
            ops.shard_step(peer_grad=sp.grad_full_table, master=sp.master, m=sp.m, v=sp.v, world=world,
                           global_offset=sp.shard_lo, noisy_out=out, skip_update=True)
        torch.cuda.synchronize()
        bits = torch.equal(pulled[0], got) and torch.equal(pulled[0], pulled[1])
        print(f"[rank {rank}] pull form: rank-ordered sum reproduced bit for bit: {bits}", flush=True)
        sp.grad.local.copy_(got)             # the checks below read the reduced shard from here
        pull_ok = bits
    else:
        got = sp.grad.local
        pull_ok = True
    ref = flat_ref[sp.shard_lo:sp.shard_lo + sp.shard]
    err = float((got - ref).norm() / (ref.norm() + 1e-12))
    ok = err < 3e-2 and pull_ok
    print(f"[rank {rank}] reduce-scatter shard rel err {err:.3e}", flush=True)

    # noise: exactly once per coordinate across shard boundaries
    noisy = torch.zeros(sp.shard, device=dev)
    before = sp.grad.local.clone()
    eng.opt.step(noise_std=2.0, normalize_by=float(B), noisy_out=noisy, skip_update=True)
    torch.cuda.synchronize()
    full = torch.zeros(sp.total, device=dev)
    ops.philox_normal_add_(full, seed=fold_in(key(11), 0).seed, offset=0, std=2.0 / B)
    want = before / B + full[sp.shard_lo:sp.shard_lo + sp.shard]
    nerr = float((noisy - want).abs().max())
    print(f"[rank {rank}] noise max abs err {nerr:.3e}", flush=True)
    ok = ok and nerr < 1e-5

    # a real step: parameters identical on all ranks afterwards and changed
    p0 = sp.params.local.clone()
    eng.noise_multiplier = 0.5
    res = eng.step(model.per_example_loss, mine)
    torch.cuda.synchronize()
    gathered = [torch.empty_like(sp.params.local) for _ in range(world)]
    dist.all_gather(gathered, sp.params.local.clone())
    same = all(torch.equal(gathered[0], g) for g in gathered)
    moved = float((sp.params.local.float() - p0.float()).abs().max()) > 0
    print(f"[rank {rank}] params identical {same}, moved {moved}, loss {res.loss:.4f}", flush=True)
    ok = ok and same and moved and eng.status.read() == 0
    flag = torch.tensor([int(ok)], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    torch.cuda.synchronize()
    dist.barrier()
    eng.group.close()
    dist.destroy_process_group()
    return 0 if int(flag.item()) == 1 else 1


if __name__ == "__main__":
    sys.exit(main())
