"""TRL-shaped task trainers on top of :class:`DPTrainer`: ``SFTTrainer`` and ``DPOTrainer``.

SFT: tokenises ``dataset_text_field`` (or prompt / completion pairs), optionally scores completion tokens only,
and uses NLL / DFT per-example losses.  DPO: the privacy unit is one preference PAIR — both completions of a pair
are evaluated inside one per-example loss; reference log-probabilities are computed once up front (the reference
model is public, so this costs no privacy) and cached on the dataset rows; TR-DPO style reference syncing mixes
the policy into the reference every ``ref_model_sync_steps``.

Parity: packages/opaque-transformers/src/opaque/api/transformers/trl/{_sft_trainer,_sft_config,_dpo_trainer,
_dpo_config}.py; packages/opaque-alignment/src/opaque/api/alignment/dpo/reference/*.py.
"""
from __future__ import annotations

import copy
import dataclasses
import os
from collections.abc import Mapping, Sequence
from typing import Any

import torch

from ..alignment import data as adata
from ..alignment import dpo as dpo_losses
from ..alignment import sft as sft_losses
from .trainer import DPTrainer
from .training_args import TrainingArguments


# ---- conversion from TRL configuration objects ---------------------------------------------------------------------------
# Parity: packages/opaque-transformers/src/opaque/api/transformers/trl/{_convert,_sft_convert,_dpo_convert}.py.

_TRL_REFUSED = {
    "packing": "sequence packing merges several records into one row: a row would no longer be one privacy unit",
    "eval_packing": "sequence packing is not supported (see packing)",
    "padding_free": "padding-free batches flatten the batch dimension that per-example clipping works on",
    "shuffle_dataset": "batches are drawn by the DP sampler; an extra shuffle has no meaning and would suggest otherwise",
    "use_liger_loss": "the fused head + cross-entropy kernel of this package is always used on the B200 engine",
    "precompute_ref_log_probs": None,          # always done here; accepted
}
_TRL_DROPPED = {"dataset_kwargs": "preprocessing is done by the tokenizer and the collator",
                "packing_strategy": "only meaningful with packing", "router_aux_loss_coef": "no auxiliary router loss is added",
                "generate_during_eval": "no generation during evaluation", "padding_value": "the tokenizer's pad token is used",
                "label_pad_token_id": "labels are padded with -100", "max_prompt_length": "prompts are kept whole; max_length truncates the pair",
                "max_completion_length": "max_length truncates the pair", "tools": "chat templates are rendered without tool schemas"}


def _from_trl(cls, trl_config: Any, overrides: dict) -> Any:
    import warnings
    from .hf_convert import _as_dict
    raw = _as_dict(trl_config)
    mode = raw.pop("truncation_mode", None)
    if mode not in (None, "keep_start"):
        raise ValueError(f"truncation_mode={mode!r} is not supported: sequences are truncated at the end (keep_start)")
    if raw.pop("pad_token", None):
        raise ValueError("pad_token is taken from the tokenizer (processing_class); set it there")
    for name, why in _TRL_REFUSED.items():
        value = raw.pop(name, None)
        if value and why is not None:
            raise ValueError(f"{name}={value!r} is not supported: {why}")
    for name, why in _TRL_DROPPED.items():
        value = raw.pop(name, None)
        if value not in (None, False, {}, [], ""):
            warnings.warn(f"{cls.__name__}.from_trl: {name}={value!r} is dropped ({why})", RuntimeWarning, stacklevel=3)
    return cls.from_hf(raw, **overrides)


@dataclasses.dataclass
class SFTConfig(TrainingArguments):
    learning_rate: float = 2e-5
    dataset_text_field: str = "text"
    max_length: int | None = 1024
    completion_only_loss: bool | None = None
    assistant_only_loss: bool = False
    loss_type: str = "nll"                      # nll | dft | chunked_nll
    pad_to_multiple_of: int | None = None
    logging_steps: int = 10
    use_performance_kernels: bool = True
    model_init_kwargs: dict | None = None       # used when ``model`` is a local checkpoint path
    trust_remote_code: bool = False
    eos_token: str | None = None                # set on the tokenizer before tokenisation
    chat_template_path: str | None = None       # a template file (or a directory holding chat_template.jinja) for the tokenizer
    dataset_num_proc: int | None = None         # accepted; tokenisation here is single-process
    log_completion_metrics: bool = False        # evaluate() adds mean token accuracy and entropy on the evaluation set

    def __post_init__(self):
        super().__post_init__()
        if self.loss_type not in ("nll", "dft", "chunked_nll"):
            raise ValueError("loss_type must be nll | dft | chunked_nll")

    @classmethod
    def from_trl(cls, trl_config: Any, **overrides: Any) -> "SFTConfig":
        """Build from a ``trl.SFTConfig`` (object or mapping); ``overrides`` carry the DP settings.  Options that would break
        the one-row-one-record contract (packing, padding-free batches, an extra shuffle) are refused by name, fields
        without meaning here are dropped with a warning, the rest goes through :meth:`TrainingArguments.from_hf`."""
        return _from_trl(cls, trl_config, overrides)


class SFTTrainer(DPTrainer):
    _INERT_FIELDS = DPTrainer._INERT_FIELDS + ("dataset_num_proc",)

    def __init__(self, model=None, args: SFTConfig | None = None, train_dataset=None, eval_dataset=None,
                 processing_class=None, data_collator=None, **kw: Any):
        args = args or SFTConfig()
        self._sft = args
        model = _load_if_path(model, args)
        _prepare_tokenizer(processing_class, args)
        train_dataset = self._prepare_dataset(train_dataset, processing_class, args)
        eval_dataset = self._prepare_dataset(eval_dataset, processing_class, args)
        completion_only = self._resolve_completion_only(args, train_dataset)
        if data_collator is None:
            pad = getattr(processing_class, "pad_token_id", None) or 0
            data_collator = lambda rows: adata.language_modeling_collator(
                rows, pad_token_id=pad, completion_only=completion_only, pad_to_multiple_of=args.pad_to_multiple_of,
                max_length=args.max_length)
        super().__init__(model=model, args=args, train_dataset=train_dataset, eval_dataset=eval_dataset,
                         processing_class=processing_class, data_collator=data_collator, **kw)

    @staticmethod
    def _resolve_completion_only(args: SFTConfig, dataset) -> bool:
        if args.assistant_only_loss:            # chat data: only assistant turns carry loss (they are the completion mask)
            return True
        if args.completion_only_loss is not None:
            return bool(args.completion_only_loss)
        return bool(dataset is not None and len(dataset) and "completion_mask" in dataset[0])

    @staticmethod
    def tokenize_row(row: Mapping[str, Any], tokenizer: Any, args: SFTConfig) -> dict[str, Any]:
        if "input_ids" in row:
            return dict(row)
        if tokenizer is None:
            raise ValueError("a processing_class (tokenizer) is required for text datasets")
        if "prompt" in row and "completion" in row:
            p = tokenizer(row["prompt"], add_special_tokens=True)["input_ids"]
            c = tokenizer(row["completion"], add_special_tokens=False)["input_ids"]
            ids = (p + c)[: args.max_length] if args.max_length else p + c
            return {"input_ids": ids, "completion_mask": adata.completion_mask(len(ids), len(p))}
        if "messages" in row and args.assistant_only_loss and getattr(tokenizer, "chat_template", None):
            # every assistant turn of a multi-turn conversation carries loss: the mask comes from the template's
            # {% generation %} markers (installed on a private copy of the template when they are missing)
            template = adata.get_training_chat_template(tokenizer)
            enc = adata.apply_chat_template_with_mask(tokenizer, list(row["messages"]), chat_template=template)
            ids, mask = enc["input_ids"], enc["completion_mask"]
            if args.max_length:
                ids, mask = ids[: args.max_length], mask[: args.max_length]
            return {"input_ids": ids, "completion_mask": mask}
        if "messages" in row:
            prompt, completion = adata.split_prompt_completion(row["messages"])
            p = tokenizer(adata.apply_chat_template(prompt, tokenizer, add_generation_prompt=True))["input_ids"]
            full = tokenizer(adata.apply_chat_template(row["messages"], tokenizer))["input_ids"]
            ids = full[: args.max_length] if args.max_length else full
            return {"input_ids": ids, "completion_mask": adata.completion_mask(len(ids), len(p))}
        ids = tokenizer(row[args.dataset_text_field])["input_ids"]
        return {"input_ids": ids[: args.max_length] if args.max_length else ids}

    @classmethod
    def _prepare_dataset(cls, dataset, tokenizer, args: SFTConfig):
        if dataset is None or len(dataset) == 0 or "input_ids" in dataset[0]:
            return dataset
        return [cls.tokenize_row(dataset[i], tokenizer, args) for i in range(len(dataset))]

    def compute_per_example_loss(self, model_call, example):
        logits = model_call(example["input_ids"].unsqueeze(0))
        logits = getattr(logits, "logits", logits)
        fn = sft_losses.dft_loss if self._sft.loss_type == "dft" else sft_losses.nll_loss
        return fn(logits, example["labels"].unsqueeze(0)).squeeze(0)

    @torch.no_grad()
    def evaluate(self, eval_dataset: Any = None, ignore_keys=None, metric_key_prefix: str = "eval") -> dict[str, float]:
        metrics = super().evaluate(eval_dataset, ignore_keys, metric_key_prefix)
        data = eval_dataset if eval_dataset is not None else self.eval_dataset
        if self._sft.log_completion_metrics and data is not None and len(data):
            # token statistics of the EVALUATION set (not training data): accuracy and entropy on the scored positions
            from ..distributed import local_shard, reduce_scalar
            a = self.args
            shard = local_shard(data, rank=a.process_index, world_size=a.world_size)
            was_training = self.model.training
            self.model.eval()
            acc_sum = ent_sum = count = 0.0
            for lo in range(0, len(shard), a.eval_batch_size):
                batch = self._to_device(self.data_collator([shard[i] for i in range(lo, min(len(shard), lo + a.eval_batch_size))]))
                logits = self.model(batch["input_ids"])
                logits = getattr(logits, "logits", logits).float()
                keep = batch["labels"] != -100                               # labels are already aligned with the logits
                n = float(keep.sum())
                acc_sum += float(((logits.argmax(-1) == batch["labels"]) & keep).sum())
                logp = logits.log_softmax(-1)
                ent_sum += float((-(logp.exp() * logp).sum(-1) * keep).sum())
                count += n
            self.model.train(was_training)
            acc_sum, ent_sum, count = (float(reduce_scalar(v, "sum")) for v in (acc_sum, ent_sum, count))
            extra = {f"{metric_key_prefix}_mean_token_accuracy": acc_sum / max(count, 1.0), f"{metric_key_prefix}_entropy": ent_sum / max(count, 1.0)}
            metrics.update(extra)
            self.log(extra)
        return metrics


def _load_if_path(model: Any, args: Any) -> Any:
    """A local checkpoint directory instead of a model object: load it with Hugging Face (offline) and convert it."""
    if not isinstance(model, (str, os.PathLike)):
        return model
    import transformers
    from .. import patches
    hf = transformers.AutoModelForCausalLM.from_pretrained(model, local_files_only=True, trust_remote_code=bool(args.trust_remote_code),
                                                           **(args.model_init_kwargs or {}))
    return patches.apply_model_patches(hf, dtype=torch.bfloat16 if args.bf16 else torch.float32)


def _prepare_tokenizer(tokenizer: Any, args: Any) -> None:
    if tokenizer is None:
        return
    if getattr(args, "eos_token", None):
        tokenizer.eos_token = args.eos_token
    path = getattr(args, "chat_template_path", None)
    if path:
        if os.path.isdir(path):
            path = os.path.join(path, "chat_template.jinja")
        with open(path, encoding="utf-8") as f:
            tokenizer.chat_template = f.read()


@dataclasses.dataclass
class DPOConfig(TrainingArguments):
    learning_rate: float = 1e-6
    beta: float = 0.1
    loss_type: Any = "sigmoid"
    loss_weights: Any = None
    label_smoothing: float = 0.0
    f_divergence_type: str = "reverse_kl"
    f_alpha_divergence_coef: float = 0.5
    ld_alpha: float | None = None
    use_weighting: bool = False
    discopop_tau: float = 0.05
    simpo_gamma: float = 0.5
    cpo_alpha: float = 1.0
    orpo_lambda: float = 1.0
    precompute_ref_batch_size: int | None = None
    disable_dropout: bool = True
    sync_ref_model: bool = False
    ref_model_mixup_alpha: float = 0.6
    ref_model_sync_steps: int = 512
    max_length: int | None = 1024
    pad_to_multiple_of: int | None = None
    model_init_kwargs: dict | None = None       # used when ``model`` is a local checkpoint path
    trust_remote_code: bool = False
    dataset_num_proc: int | None = None         # accepted; tokenisation here is single-process
    log_completion_metrics: bool = False        # accepted; reward accuracies and margins are always logged

    def __post_init__(self):
        super().__post_init__()
        types = [self.loss_type] if isinstance(self.loss_type, str) else list(self.loss_type)
        for t in types:
            if t not in dpo_losses.ALL_LOSS_TYPES:
                raise ValueError(f"unknown DPO loss_type {t!r}")
        if self.loss_weights is not None and len(self.loss_weights) != len(types):
            raise ValueError("loss_weights must match loss_type")

    @classmethod
    def from_trl(cls, trl_config: Any, **overrides: Any) -> "DPOConfig":
        """Build from a ``trl.DPOConfig`` (object or mapping); see :meth:`SFTConfig.from_trl`."""
        return _from_trl(cls, trl_config, overrides)


class DPOTrainer(DPTrainer):
    """DP-DPO; ``ref_model=None`` uses a frozen copy of the initial policy (or the base model under LoRA)."""
    _INERT_FIELDS = DPTrainer._INERT_FIELDS + ("dataset_num_proc", "log_completion_metrics")

    def __init__(self, model=None, ref_model=None, args: DPOConfig | None = None, train_dataset=None, eval_dataset=None,
                 processing_class=None, data_collator=None, **kw: Any):
        args = args or DPOConfig()
        self._dpo = args
        model = _load_if_path(model, args)
        if data_collator is None:
            pad = getattr(processing_class, "pad_token_id", None) or 0
            data_collator = lambda rows: adata.preference_collator(rows, pad_token_id=pad, max_length=args.max_length,
                                                                   pad_to_multiple_of=args.pad_to_multiple_of)
        train_dataset = self._prepare(train_dataset, processing_class)
        eval_dataset = self._prepare(eval_dataset, processing_class)
        if args.disable_dropout:
            for m in model.modules():
                if isinstance(m, torch.nn.Dropout):
                    m.p = 0.0
        self._reference_free = all(t in dpo_losses.REFERENCE_FREE for t in ([args.loss_type] if isinstance(args.loss_type, str) else args.loss_type))
        # The reference log-probabilities are computed ONCE, before the first update.  Without an explicit ref_model that
        # needs no second copy of the weights: the policy itself at its initial point (adapters switched off under LoRA,
        # so the reference is the frozen base model).  Only TR-DPO (sync_ref_model) owns a separate, moving reference.
        self.ref_model = ref_model
        if ref_model is None and args.sync_ref_model and not self._reference_free:
            self.ref_model = copy.deepcopy(model).requires_grad_(False)
        super().__init__(model=model, args=args, train_dataset=train_dataset, eval_dataset=eval_dataset,
                         processing_class=processing_class, data_collator=data_collator, **kw)
        if not self._reference_free:
            if self.ref_model is not None:
                self.ref_model.to(self.device).eval()
            self.train_dataset = self._precompute_ref_logps(self.train_dataset, "train")
            if self.eval_dataset is not None:
                self.eval_dataset = self._precompute_ref_logps(self.eval_dataset, "eval")
        self._bco_delta = 0.0

    # ---- engine selection ------------------------------------------------------------------------------------------
    def _fused_blockers(self) -> list[str]:
        why = [w for w in super()._fused_blockers() if "per_example_loss" not in w]
        if not hasattr(self.model, "token_nll"):
            why.append("the model has no token_nll (convert it with opaque_b200.patches)")
        if self._dpo.ld_alpha is not None:
            why.append("ld_alpha (length-desensitised log-probabilities) needs token-level terms")
        if self._dpo.use_weighting:
            why.append("use_weighting (WPO) needs token-level terms")
        return why

    def _fused_payload(self, batch) -> dict[str, torch.Tensor]:
        """One privacy unit = one preference pair: ``input_ids`` / ``labels`` ``[B, 2, T]`` (chosen, rejected; both padded
        to the same length) and the precomputed reference log-probabilities ``[B, 2]``."""
        ci, ri, cl, rl = batch["chosen_input_ids"], batch["rejected_input_ids"], batch["chosen_labels"], batch["rejected_labels"]
        T = max(ci.shape[1], ri.shape[1])
        T = (T + 63) // 64 * 64                          # whole 64-row blocks per pair for the per-example GEMM path

        def pad(t, value):
            return torch.nn.functional.pad(t, (0, T - t.shape[1]), value=value)
        ids = torch.stack([pad(ci, 0), pad(ri, 0)], dim=1)
        labels = torch.stack([pad(cl, -100), pad(rl, -100)], dim=1)
        B = ids.shape[0]
        ref = torch.zeros(B, 2, device=ids.device)
        if "ref_chosen_logps" in batch:
            ref = torch.stack([batch["ref_chosen_logps"], batch["ref_rejected_logps"]], dim=1).to(ids.device, torch.float32)
        return {"input_ids": ids, "labels": labels, "ref_logps": ref}

    def _fused_loss_fn(self):
        return self._fused_pair_loss

    def _sequence_logps(self, model, ids, labels):
        """``(sum, mean)`` log-probability of the scored tokens of every sequence (``[N]`` each), differentiable."""
        nll = model.token_nll(ids, labels)
        cnt = (labels != -100).sum(1).clamp_min(1)
        s = -nll.sum(1)
        return s, s / cnt

    def _fused_pair_loss(self, input_ids, labels, ref_logps):
        a = self._dpo
        B, _, T = input_ids.shape
        s, m = self._sequence_logps(self.model, input_ids.reshape(2 * B, T), labels.reshape(2 * B, T))
        s, m = s.view(B, 2), m.view(B, 2)
        c_sum, r_sum, c_avg, r_avg = s[:, 0], s[:, 1], m[:, 0], m[:, 1]
        use_avg = a.loss_type == "ipo" or (not isinstance(a.loss_type, str) and "ipo" in a.loss_type)
        c_ratio = (c_avg if use_avg else c_sum) - ref_logps[:, 0]
        r_ratio = (r_avg if use_avg else r_sum) - ref_logps[:, 1]
        return dpo_losses.dpo_loss(a.loss_type, chosen_logratio=c_ratio, rejected_logratio=r_ratio, beta=a.beta,
                                   label_smoothing=a.label_smoothing, loss_weights=a.loss_weights, chosen_nll=-c_avg,
                                   chosen_avg_logp=c_avg, rejected_avg_logp=r_avg, bco_delta=self._bco_delta,
                                   discopop_tau=a.discopop_tau, simpo_gamma=a.simpo_gamma, orpo_lambda=a.orpo_lambda,
                                   f_divergence_type=a.f_divergence_type, f_alpha=a.f_alpha_divergence_coef,
                                   chosen_logp=c_sum, rejected_logp=r_sum, cpo_alpha=a.cpo_alpha)

    @staticmethod
    def tokenize_row(row, tokenizer):
        if "prompt_input_ids" in row:
            return dict(row)
        if tokenizer is None:
            raise ValueError("a processing_class (tokenizer) is required for text preference data")
        return {"prompt_input_ids": tokenizer(row["prompt"])["input_ids"],
                "chosen_input_ids": tokenizer(row["chosen"], add_special_tokens=False)["input_ids"],
                "rejected_input_ids": tokenizer(row["rejected"], add_special_tokens=False)["input_ids"]}

    @classmethod
    def _prepare(cls, dataset, tokenizer):
        if dataset is None:
            return None
        return [cls.tokenize_row(dataset[i], tokenizer) for i in range(len(dataset))]

    def _seq_logps(self, call, ids, labels, average=False):
        logits = call(ids)
        logits = getattr(logits, "logits", logits)
        if self._dpo.ld_alpha is not None and not average:
            lp, mask = sft_losses.token_logps(logits, labels)
            return lp, mask
        return sft_losses.sequence_logp(logits, labels, average=average)

    def _reference_forward(self):
        """``(module, context)`` that evaluates the reference policy: the explicit / TR-DPO reference model, or the
        policy itself with its adapters switched off (equal to the initial policy: LoRA starts at zero)."""
        import contextlib

        from ..models.layers import adapters_disabled
        if self.ref_model is not None:
            return self.ref_model, contextlib.nullcontext()
        return self.model, adapters_disabled()

    def _ref_cache_path(self, dataset, split: str) -> str | None:
        """File under ``output_dir`` keyed by the data and the reference weights, or ``None`` when caching is off."""
        import hashlib
        import os
        if not self.args.output_dir or not len(dataset):
            return None
        h = hashlib.blake2b(digest_size=12)
        h.update(f"{len(dataset)}|{self._dpo.max_length}|{self._dpo.loss_type}".encode())
        for i in (0, len(dataset) // 2, len(dataset) - 1):
            row = dataset[i]
            h.update(repr((list(row["prompt_input_ids"])[:64], list(row["chosen_input_ids"])[:64], list(row["rejected_input_ids"])[:64])).encode())
        module, _ = self._reference_forward()
        for n, p in list(module.named_parameters())[:4]:
            if "lora_" not in n:
                h.update(n.encode())
                h.update(p.detach().float().flatten()[:256].cpu().numpy().tobytes())
        return os.path.join(self.args.output_dir, f"ref_logps_{split}_{h.hexdigest()}.pt")

    @torch.no_grad()
    def _precompute_ref_logps(self, dataset, split: str = "train"):
        """Reference log-probabilities of every pair, computed once: each rank scores every ``world``-th pair, the
        results are gathered with one tensor all-gather, and rank 0 keeps them in a cache file under ``output_dir``
        (parity: packages/opaque-alignment/src/opaque/api/alignment/dpo/reference/_precompute.py:270-321, 449)."""
        import os

        from ..distributed import get_rank, get_world_size, is_distributed
        if dataset is None or (len(dataset) and "ref_chosen_logps" in dataset[0]):
            return dataset
        n = len(dataset)
        cache = self._ref_cache_path(dataset, split)
        table = None
        if cache and os.path.exists(cache):
            got = torch.load(cache, map_location="cpu")
            if tuple(got.shape) == (n, 2):
                table = got
        if table is None:
            rank, world = (get_rank(), get_world_size()) if is_distributed() else (0, 1)
            mine = list(range(rank, n, world))
            bs = self._dpo.precompute_ref_batch_size or self.args.eval_batch_size
            module, ctx = self._reference_forward()
            was_training = module.training
            module.eval()
            local = torch.zeros(len(mine), 2, dtype=torch.float32, device=self.device)
            with ctx:
                for lo in range(0, len(mine), bs):
                    rows = [dataset[i] for i in mine[lo:lo + bs]]
                    batch = self._to_device(self.data_collator(rows))
                    for col, side in enumerate(("chosen", "rejected")):
                        if hasattr(module, "token_nll") and self.device.type == "cuda":
                            lp = -module.token_nll(batch[f"{side}_input_ids"], batch[f"{side}_labels"]).sum(1)
                        else:
                            lp = sft_losses.sequence_logp(_logits(module(batch[f"{side}_input_ids"])), batch[f"{side}_labels"])
                        local[lo:lo + len(rows), col] = lp.float()
            module.train(was_training)
            table = torch.zeros(n, 2, dtype=torch.float32)
            if world > 1:
                per = (n + world - 1) // world                      # equal-length pieces for the tensor all-gather
                padded = torch.zeros(per, 2, dtype=torch.float32, device=self.device)
                padded[:len(mine)] = local
                pieces = [torch.zeros_like(padded) for _ in range(world)]
                torch.distributed.all_gather(pieces, padded)
                for r, piece in enumerate(pieces):
                    idx = list(range(r, n, world))
                    table[idx] = piece[:len(idx)].cpu()
            else:
                table[mine] = local.cpu()
            if cache and rank == 0:
                os.makedirs(os.path.dirname(cache), exist_ok=True)
                torch.save(table, cache)
        vals = table.tolist()
        return [{**dataset[i], "ref_chosen_logps": vals[i][0], "ref_rejected_logps": vals[i][1]} for i in range(n)]

    def _pair_terms(self, call, ex):
        cl, rl = ex["chosen_labels"].unsqueeze(0), ex["rejected_labels"].unsqueeze(0)
        ci, ri = ex["chosen_input_ids"].unsqueeze(0), ex["rejected_input_ids"].unsqueeze(0)
        c_logits, r_logits = _logits(call(ci)), _logits(call(ri))
        c_lp, c_mask = sft_losses.token_logps(c_logits, cl)
        r_lp, r_mask = sft_losses.token_logps(r_logits, rl)
        if self._dpo.ld_alpha is not None:
            common = torch.minimum(c_mask.sum(-1), r_mask.sum(-1))
            c_sum = dpo_losses.ld_dpo_logp(c_lp, c_mask, common, self._dpo.ld_alpha)
            r_sum = dpo_losses.ld_dpo_logp(r_lp, r_mask, common, self._dpo.ld_alpha)
        else:
            c_sum, r_sum = c_lp.sum(-1), r_lp.sum(-1)
        c_avg = c_lp.sum(-1) / c_mask.sum(-1).clamp_min(1)
        r_avg = r_lp.sum(-1) / r_mask.sum(-1).clamp_min(1)
        weight = dpo_losses.wpo_weight(c_lp, c_mask, r_lp, r_mask) if self._dpo.use_weighting else None
        return c_sum.squeeze(0), r_sum.squeeze(0), c_avg.squeeze(0), r_avg.squeeze(0), weight

    def compute_per_example_loss(self, model_call, example):
        a = self._dpo
        c_sum, r_sum, c_avg, r_avg, weight = self._pair_terms(model_call, example)
        ref_c = example.get("ref_chosen_logps", torch.zeros((), device=c_sum.device))
        ref_r = example.get("ref_rejected_logps", torch.zeros((), device=c_sum.device))
        use_avg = a.loss_type == "ipo" or (not isinstance(a.loss_type, str) and "ipo" in a.loss_type)
        c_ratio = (c_avg if use_avg else c_sum) - ref_c
        r_ratio = (r_avg if use_avg else r_sum) - ref_r
        return dpo_losses.dpo_loss(a.loss_type, chosen_logratio=c_ratio, rejected_logratio=r_ratio, beta=a.beta,
                                   label_smoothing=a.label_smoothing, loss_weights=a.loss_weights, chosen_nll=-c_avg,
                                   chosen_avg_logp=c_avg, rejected_avg_logp=r_avg, bco_delta=self._bco_delta,
                                   discopop_tau=a.discopop_tau, simpo_gamma=a.simpo_gamma, orpo_lambda=a.orpo_lambda,
                                   f_divergence_type=a.f_divergence_type, f_alpha=a.f_alpha_divergence_coef,
                                   pair_weight=weight.squeeze(0) if weight is not None else None,
                                   chosen_logp=c_sum, rejected_logp=r_sum, cpo_alpha=a.cpo_alpha)

    def compute_ref_log_probs(self, dataset: Any = None, split: str = "train") -> Any:
        """The dataset with ``ref_chosen_logps`` / ``ref_rejected_logps`` on every pair (rank-sharded, gathered, cached);
        rows that already carry them come back unchanged.  Called by the constructor for the training and evaluation sets."""
        return self._precompute_ref_logps(dataset if dataset is not None else self.train_dataset, split)

    def dpo_loss(self, chosen_logratio: torch.Tensor, rejected_logratio: torch.Tensor, **terms: Any) -> torch.Tensor:
        """The configured preference loss for given log-ratios, one value per pair (``loss_type``, ``beta``, label smoothing,
        mixture weights and the head-specific tunables come from the ``DPOConfig``; ``terms`` supplies what reference-free
        heads need: ``chosen_nll``, ``chosen_avg_logp``, ``rejected_avg_logp``, ``chosen_logp``, ``rejected_logp``)."""
        a = self._dpo
        return dpo_losses.dpo_loss(a.loss_type, chosen_logratio=chosen_logratio, rejected_logratio=rejected_logratio, beta=a.beta,
                                   label_smoothing=a.label_smoothing, loss_weights=a.loss_weights, bco_delta=self._bco_delta,
                                   discopop_tau=a.discopop_tau, simpo_gamma=a.simpo_gamma, orpo_lambda=a.orpo_lambda,
                                   f_divergence_type=a.f_divergence_type, f_alpha=a.f_alpha_divergence_coef, cpo_alpha=a.cpo_alpha, **terms)

    def compute_batch_per_example_loss(self, batch):
        n = batch["chosen_input_ids"].shape[0]
        rows = [self.compute_per_example_loss(self.model, {k: v[i] for k, v in batch.items() if isinstance(v, torch.Tensor)}) for i in range(n)]
        return torch.stack(rows) if rows else torch.zeros(0, device=self.device)

    def _reference_step(self, batch, sp):
        payload = {k: v for k, v in batch.items() if isinstance(v, torch.Tensor)}
        payload.setdefault("input_ids", payload["chosen_input_ids"])
        payload.setdefault("labels", payload["chosen_labels"])
        out = super()._reference_step(payload, sp)
        if self._dpo.sync_ref_model and self.ref_model is not None and self.state.global_step % self._dpo.ref_model_sync_steps == 0 and self.state.global_step:
            self._ema_update_reference()
        return out

    @torch.no_grad()
    def _ema_update_reference(self) -> None:
        """TR-DPO: ``ref ← α·policy + (1−α)·ref`` (then reference log-probs are recomputed lazily)."""
        self._write_back()
        al = self._dpo.ref_model_mixup_alpha
        for (n, p), (_, r) in zip(self.model.named_parameters(), self.ref_model.named_parameters()):
            r.mul_(1 - al).add_(p.detach().to(r.dtype), alpha=al)
        strip = lambda rows: [{k: v for k, v in row.items() if not k.startswith("ref_")} for row in rows]
        self.train_dataset = self._precompute_ref_logps(strip(self.train_dataset), f"train_step{self.state.global_step}")
        self._local_data = None      # rebuilt on the next epoch boundary by _setup; current sampler keeps its indices


def _logits(out):
    return getattr(out, "logits", out)


__all__ = ["DPOConfig", "DPOTrainer", "SFTConfig", "SFTTrainer"]
