"""Comparator arm: the UNMODIFIED reference library driving its own stock DP-SGD path on the benchmark configurations.

Everything on the timed path is the reference's code from ``baseline/_ref`` (installed by
``baseline/install_reference.sh``): ``apply_model_patches`` (its Triton kernels and fused linear-cross-entropy),
``make_functional``, ``clipped_grad`` (``vmap(grad)`` in microbatches), ``sync`` / ``sum_gradients_`` (NCCL),
``gaussian_noise``, ``adamw(noise_bias_correction=True)`` and ``PoissonSampler`` — the loop of the reference's
``examples/train_dpsgd.py:1884-1915``.  The models are Hugging Face ``LlamaForCausalLM`` / ``GPT2LMHeadModel`` built
from a config with random weights.  Nothing from ``opaque_b200`` is imported and none of its shared objects is loaded.

Two pieces are not the reference's and are declared in the JSON line:

* ``optree`` and ``torchopt`` are not installable offline; ``baseline/shims`` holds small pure-Python stand-ins with
  the handful of functions the reference calls (``deps_standins``).
* ``peft`` is absent, so the LoRA factors are attached by the plain-PyTorch module below (``"lora": "harness module"``);
  the reference's PEFT kernel patches then have nothing to rewrite and its per-example gradient path treats the factors
  as ordinary trainable parameters.
"""
from __future__ import annotations

import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF = HERE / "_ref"
SHIMS = HERE / "shims"


def available() -> str | None:
    """``None`` when the reference tree is importable, else the reason in one line."""
    if not (REF / "opaque" / "api" / "engine").is_dir():
        return "baseline/_ref holds no reference code (run baseline/install_reference.sh)"
    return None


class _Clocks:
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "200"], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        mhz = [float(r[0]) for r in self.rows if r and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) > 1 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({names[i] for r in self.rows if len(r) >= 6 for i in range(4) if r[2 + i].lower() == "active"})
        return {"sm_mhz": statistics.median(mhz) if mhz else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(mhz)}


def _lora_module(torch):
    nn = torch.nn

    class HarnessLoRALinear(nn.Module):
        """``base(x) + (alpha / r) * B(A(x))`` with the PEFT initialisation (A Kaiming-uniform, B zero)."""

        def __init__(self, base: nn.Linear, r: int, alpha: float):
            super().__init__()
            self.base_layer = base
            self.lora_A = nn.Linear(base.in_features, r, bias=False, dtype=base.weight.dtype, device=base.weight.device)
            self.lora_B = nn.Linear(r, base.out_features, bias=False, dtype=base.weight.dtype, device=base.weight.device)
            nn.init.zeros_(self.lora_B.weight)
            self.scaling = alpha / r

        def forward(self, x):
            return self.base_layer(x) + self.lora_B(self.lora_A(x)) * self.scaling

    return HarnessLoRALinear


def build_model(config: str, dev, layers: int = 0):
    """Random-init Hugging Face model of the named benchmark configuration (same shapes as ``bench.py``)."""
    import torch
    import transformers

    if config in ("llama8b-lora", "llama-tiny"):
        if config == "llama8b-lora":
            cfg = transformers.LlamaConfig(vocab_size=128256, hidden_size=4096, intermediate_size=14336, num_hidden_layers=layers or 32,
                                           num_attention_heads=32, num_key_value_heads=8, rms_norm_eps=1e-5, rope_theta=500000.0,
                                           max_position_embeddings=8192, tie_word_embeddings=False, attention_bias=False)
            seq, per_gpu, mb, frac, vocab = 1024, 64, 32, 0.5, 128256
            name = "Llama-3-8B (LoRA r16 a32 on q/k/v/o, base frozen)"
        else:
            cfg = transformers.LlamaConfig(vocab_size=256, hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                                           num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=256,
                                           tie_word_embeddings=False)
            seq, per_gpu, mb, frac, vocab = 128, 16, 8, 0.5, 256
            name = "Llama-tiny (LoRA)"
        cfg._attn_implementation = "sdpa"
        prev = torch.get_default_dtype()
        torch.set_default_dtype(torch.bfloat16)
        try:
            with torch.device(dev):
                model = transformers.LlamaForCausalLM(cfg)
        finally:
            torch.set_default_dtype(prev)
        for p in model.parameters():
            p.requires_grad_(False)
        lora_cls = _lora_module(torch)
        for layer in model.model.layers:
            attn = layer.self_attn
            for proj in ("q_proj", "k_proj", "v_proj", "o_proj"):
                setattr(attn, proj, lora_cls(getattr(attn, proj), 16, 32.0))
        dp = dict(clipping_norm=1.0, noise_multiplier=0.7, lr=2e-4)
        return model, dict(seq=seq, per_gpu=per_gpu, mb=mb, frac=frac, vocab=vocab, name=name, lora="harness module", dp=dp,
                           logical_size=None)
    if config == "gpt2":
        cfg = transformers.GPT2Config(vocab_size=50257, n_positions=1024, n_embd=768, n_layer=layers or 12, n_head=12,
                                      resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0)
        cfg._attn_implementation = "sdpa"
        prev = torch.get_default_dtype()
        torch.set_default_dtype(torch.bfloat16)
        try:
            with torch.device(dev):
                model = transformers.GPT2LMHeadModel(cfg)
        finally:
            torch.set_default_dtype(prev)
        dp = dict(clipping_norm=1.0, noise_multiplier=0.8, lr=1e-4)
        return model, dict(seq=512, per_gpu=128, mb=64, frac=1.0, vocab=50257, name="GPT-2-small full-parameter", lora=None,
                           dp=dp, logical_size=1_000_000)
    raise ValueError(f"the reference arm has no configuration {config!r}")


def run(args) -> None:
    """Runs the arm and prints one JSON line on rank 0 (same keys as ``bench.py``'s own arm, ``impl = reference``)."""
    why = available()
    if why or args.config not in ("llama8b-lora", "gpt2", "llama-tiny"):
        print(json.dumps({"impl": "reference", "unavailable": why or f"no reference arm for --config {args.config}"}))
        return
    sys.path[:0] = [str(REF), str(SHIMS)]
    import torch
    import torch.distributed as dist

    try:
        import torchopt
        from opaque.distributed import sync
        from opaque.distributed.gradients import sum_gradients_
        from opaque.dpsgd.clipping import clipped_grad
        from opaque.dpsgd.noise import gaussian_noise
        from opaque.dpsgd.sampling import PoissonSampler
        from opaque.functional import make_functional
        from opaque.optimizers import adamw
        from opaque.patches import apply_model_patches
        from opaque.random import fold_in, key
    except Exception as exc:       # the exact import that fails is the report
        print(json.dumps({"impl": "reference", "unavailable": f"{type(exc).__name__}: {exc}"[:300]}))
        return

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    use_cuda = torch.cuda.is_available() and not getattr(args, "cpu", False)
    if use_cuda:
        torch.cuda.set_device(local)
        dev = torch.device("cuda", local)
    else:
        dev = torch.device("cpu")
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        if use_cuda:
            dist.init_process_group("nccl", device_id=dev)
        else:
            dist.init_process_group("gloo")
    torch.manual_seed(1234)
    model, spec = build_model(args.config, dev, getattr(args, "layers", 0))
    seq, frac, vocab, dp = spec["seq"], spec["frac"], spec["vocab"], spec["dp"]
    per_gpu = args.per_gpu_batch or spec["per_gpu"]
    # vmap microbatch: the fastest of the sizes measured for the reference on a B200 (Llama-3-8B LoRA: 4 -> 10.9 k,
    # 8 -> 14.8 k, 16 -> 20.9 k, 32 -> 22.2 k tokens/s at 126 GB; GPT-2: 32 -> 55.0 k, 64 -> 61.9 k tokens/s)
    mb = args.microbatch or spec["mb"]
    model.train()
    # the reference's stock configuration for a run whose only consumer of the forward output is the loss
    # (examples/train_dpsgd.py:1134-1136): Triton kernels and the fused linear-cross-entropy on CUDA
    # (its fused linear-CE forward reads ``self.model`` and so exists for the Llama-shaped families only: GPT-2 keeps the
    # kernel patches without it)
    apply_model_patches(model, kernels=use_cuda, fused_linear_cross_entropy=use_cuda and args.config != "gpt2")
    fmodel, trainable, frozen = make_functional(model, disable_autograd_tracking=True, partition_trainable=True)
    cut = int(seq * (1.0 - frac))

    def per_example_loss(tr, input_ids):
        labels = input_ids
        if cut:
            labels = torch.where(torch.arange(input_ids.shape[-1], device=input_ids.device) < cut, -100, input_ids)
        return fmodel({**frozen, **tr}, input_ids, labels=labels).loss

    grad_fn, clip_state = clipped_grad(per_example_loss, argnums=0, batch_argnums=(1,), clipping_norm=dp["clipping_norm"],
                                       normalize_by=float(per_gpu * world), microbatch_size=mb, return_aux=True)
    noise_fn, noise_state = gaussian_noise(noise_multiplier=dp["noise_multiplier"], key=key(42))
    opt = adamw(lr=dp["lr"], weight_decay=0.0, noise_bias_correction=True)
    opt_state = opt.init(trainable)

    data_size = per_gpu * 100 * world
    gen = torch.Generator().manual_seed(99)
    data = torch.randint(0, vocab, (data_size, seq), generator=gen, dtype=torch.int32)
    if use_cuda:
        data = data.pin_memory()
    # per-rank Poisson draws over this rank's share (the reference's DDP recipe: key folded with the rank)
    # (GPT-2 is specified over 1e6 records: the draw runs over 1e6 logical records that map onto the stored rows modulo)
    logical = spec["logical_size"] or data_size
    shard = range(rank, logical, world)
    sampler = PoissonSampler(shard, sample_rate=per_gpu * world / logical, n_steps=args.warmup + 2 * args.steps + 2,
                             key=fold_in(key(7), rank))
    batches = iter(sampler)

    def host_batch():
        idx = [shard[i] for i in next(batches)]
        hb = data[torch.as_tensor(idx, dtype=torch.long) % data_size] if idx else data[:0]
        return hb.pin_memory() if use_cuda and len(idx) else hb

    def step(hb):
        nonlocal trainable, clip_state, noise_state, opt_state
        ids = hb.to(dev, non_blocking=True).long()
        (grads, aux), clip_state = grad_fn(trainable, ids, state=clip_state)
        if world > 1:
            clip_state, aux = sync(clip_state, aux)
            sum_gradients_(grads)
        noisy, noise_state = noise_fn(grads, noise_state)
        if world > 1:
            noise_state = sync(noise_state)
        updates, opt_state = opt.update(noisy, opt_state, params=trainable)
        trainable = torchopt.apply_updates(trainable, updates)
        return float(aux.loss_values.mean().item()) if ids.shape[0] else 0.0     # the step's result, read on the host

    def barrier():
        if world > 1:
            dist.barrier()
        if use_cuda:
            torch.cuda.synchronize()

    for _ in range(args.warmup):
        step(host_batch())
    barrier()
    hbs = [host_batch() for _ in range(args.steps)]
    tokens = sum(b.numel() for b in hbs)
    clocks = _Clocks(local)
    if use_cuda:
        clocks.start()
    barrier()
    if use_cuda:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
    t0 = time.perf_counter()
    last = 0.0
    for hb in hbs:
        last = step(hb)                                   # H2D of the batch and D2H of the loss every step
    if use_cuda:
        e1.record()
        torch.cuda.synchronize()
    wall_ms = (time.perf_counter() - t0) * 1e3
    dev_ms = e0.elapsed_time(e1) if use_cuda else wall_ms
    barrier()
    stats = torch.tensor([dev_ms, wall_ms, float(tokens)], device=dev, dtype=torch.float64)
    if world > 1:
        mx, sm = stats.clone(), stats.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        stats = torch.stack([mx[0], mx[1], sm[2]])
    dev_ms, wall_ms, tokens = stats.tolist()
    if rank == 0:
        h2d = sum(b.numel() * b.element_size() for b in hbs) / max(args.steps, 1)
        loaded = [ln.split()[-1] for ln in open("/proc/self/maps") if "opaque_b200" in ln and ".so" in ln] if os.path.exists("/proc/self/maps") else []
        print(json.dumps({
            "metric": "DP-SGD tokens/sec (box, max over ranks)", "value": tokens / (dev_ms / 1e3), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dev_ms / max(args.steps, 1),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16" if use_cuda else "bf16 (cpu)",
            "data": "synthetic uniform token ids, random-init weights", "impl": "reference",
            "config": {"model": spec["name"], "global_batch": per_gpu * world, "seq_len": seq, "parallelism": f"ddp{world}",
                       "microbatch": mb, "loss_fraction": frac, "clip": dp["clipping_norm"], "sigma": dp["noise_multiplier"],
                       "optimizer": "AdamW-BC (reference adamw, noise_bias_correction=True)", "lr": dp["lr"],
                       "sampling": "reference PoissonSampler per rank over the rank's shard (key folded with the rank)",
                       "path": "reference stock path: apply_model_patches(kernels, fused linear-CE) -> make_functional -> "
                               "clipped_grad (vmap(grad), microbatched) -> sync + sum_gradients_ -> gaussian_noise -> adamw -> apply_updates",
                       "l2": "inputs larger than L2 (per-step working set >> 126 MB; no explicit flush)"},
            "deps_standins": ["optree", "torchopt"], "lora": spec["lora"], "accountant": "not called (sigma passed directly)",
            "our_shared_objects_loaded": loaded,
            "clocks": clocks.stop() if use_cuda else None,
            "e2e": {"value": tokens / (wall_ms / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 8,
                    "last_loss": last},
            "gpu_launches": 0,
            "peak_mem_gb": torch.cuda.max_memory_allocated(dev) / 2 ** 30 if use_cuda else None}))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
