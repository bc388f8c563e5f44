"""Per-example DPO-family preference losses (17 heads) and their dispatcher.

Every head maps per-example log-ratios (policy minus reference log-probability of the chosen / rejected
response) to one loss per preference PAIR, which is the privacy unit of DP-DPO: clipping acts on the gradient
of one pair.  All functions are elementwise, so they work on ``(B,)`` tensors and on 0-dim scalars.

Parity: packages/opaque-alignment/src/opaque/api/alignment/dpo/loss/_{sigmoid,hinge,ipo,apo,bco,chosen_nll,
discopop,exo,f_divergence,ld_dpo,mpo,nca,orpo,robust,simpo,sppo,wpo}.py and
packages/opaque-transformers/src/opaque/api/transformers/trl/_dpo_trainer.py:878 (dispatch, mixtures).
"""
from __future__ import annotations

import math
from collections.abc import Mapping, Sequence
from typing import Any

import torch
import torch.nn.functional as F


def sigmoid_loss(chosen_logratio, rejected_logratio, *, beta: float, label_smoothing: float = 0.0):
    """DPO (Rafailov et al. 2023): ``−logσ(βΔ)(1−ε) − logσ(−βΔ)ε``."""
    c, r = chosen_logratio, rejected_logratio
    d = c - r
    return -F.logsigmoid(beta * d) * (1 - label_smoothing) - F.logsigmoid(-beta * d) * label_smoothing


def hinge_loss(chosen_logratio, rejected_logratio, *, beta: float):
    """SLiC-style hinge: ``relu(1 − βΔ)``."""
    c, r = chosen_logratio, rejected_logratio
    return torch.relu(1 - beta * (c - r))


def ipo_loss(chosen_logratio, rejected_logratio, *, beta: float):
    """IPO (Azar et al. 2023): ``(Δ − 1/(2β))²`` (log-ratios are expected length-averaged)."""
    c, r = chosen_logratio, rejected_logratio
    return (c - r - 1 / (2 * beta)) ** 2


def exo_loss(chosen_logratio, rejected_logratio, *, beta: float, label_smoothing: float = 1e-3):
    """EXO pairwise (Ji et al. 2024): reverse KL between the preference and the label distribution."""
    c, r = chosen_logratio, rejected_logratio
    eps = label_smoothing if label_smoothing > 0 else 1e-3
    d = beta * (c - r)
    return (torch.sigmoid(d) * (F.logsigmoid(d) - math.log(1 - eps))
            + torch.sigmoid(-d) * (F.logsigmoid(-d) - math.log(eps)))


def nca_loss(chosen_logratio, rejected_logratio, *, beta: float):
    """NCA pairwise (Chen et al. 2024)."""
    c, r = chosen_logratio, rejected_logratio
    return -F.logsigmoid(beta * c) - 0.5 * F.logsigmoid(-beta * c) - 0.5 * F.logsigmoid(-beta * r)


def robust_loss(chosen_logratio, rejected_logratio, *, beta: float, label_smoothing: float = 0.0):
    """Robust DPO (Chowdhury et al. 2024): unbiased under label-flip probability ε."""
    c, r = chosen_logratio, rejected_logratio
    if not 0 <= label_smoothing < 0.5:
        raise ValueError("robust DPO needs label_smoothing in [0, 0.5)")
    d = beta * (c - r)
    return (-F.logsigmoid(d) * (1 - label_smoothing) + F.logsigmoid(-d) * label_smoothing) / (1 - 2 * label_smoothing)


def bco_loss(chosen_logratio, rejected_logratio, *, beta: float, delta: float | torch.Tensor = 0.0):
    """BCO pairwise (Jung et al. 2024); ``delta`` is the running mean reward (public state)."""
    c, r = chosen_logratio, rejected_logratio
    return -F.logsigmoid(beta * c - delta) - F.logsigmoid(-(beta * r - delta))


def sppo_loss(chosen_logratio, rejected_logratio, *, beta: float):
    """SPPO hard-label (Wu et al. 2024)."""
    c, r = chosen_logratio, rejected_logratio
    return (c - 0.5 / beta) ** 2 + (r + 0.5 / beta) ** 2


def apo_zero_loss(chosen_logratio, rejected_logratio, *, beta: float):
    """APO-zero (D'Oosterlinck et al. 2024): push chosen up, rejected down."""
    c, r = chosen_logratio, rejected_logratio
    return 1 - torch.sigmoid(beta * c) + torch.sigmoid(beta * r)


def apo_down_loss(chosen_logratio, rejected_logratio, *, beta: float):
    """APO-down: push both down, the rejected one further."""
    c, r = chosen_logratio, rejected_logratio
    return torch.sigmoid(beta * c) + 1 - torch.sigmoid(beta * (c - r))


def discopop_loss(chosen_logratio, rejected_logratio, *, beta: float, discopop_tau: float = 0.05):
    """DiscoPOP (Lu et al. 2024): log-ratio-modulated blend of logistic and exponential losses."""
    c, r = chosen_logratio, rejected_logratio
    d = beta * (c - r)
    mod = torch.sigmoid(d / discopop_tau)
    cap = 80.0 if d.dtype in (torch.float32, torch.float64) else 10.0
    return -F.logsigmoid(d) * (1 - mod) + torch.exp((-d).clamp(max=cap)) * mod


def chosen_nll_loss(chosen_logp, /, *_args, **_kwargs):
    """SFT regulariser on the chosen response: ``−chosen_logp`` (the argument is the policy's log-probability of the chosen
    completion, not a log-ratio; further arguments are ignored so that it can sit in a mixture next to the pair heads).

    Parity: packages/opaque-alignment/src/opaque/api/alignment/dpo/loss/_chosen_nll.py:34."""
    return -chosen_logp


def simpo_loss(chosen_logratio, rejected_logratio, *, beta: float, gamma: float = 0.0, label_smoothing: float = 0.0):
    """SimPO (Meng et al. 2024): reference-free, with target margin ``γ/β``; the two arguments are the LENGTH-NORMALISED
    policy log-probabilities (the "log-ratios" of a reference-free head)."""
    d = beta * (chosen_logratio - rejected_logratio - gamma / beta)
    return -F.logsigmoid(d) * (1 - label_smoothing) - F.logsigmoid(-d) * label_smoothing


def orpo_loss(chosen_avg_logp, rejected_avg_logp, chosen_nll, *, lambda_: float = 1.0):
    """ORPO (Hong et al. 2024): ``nll − λ·logσ(log odds ratio)``."""
    log_odds = (chosen_avg_logp - rejected_avg_logp) - (torch.log1p(-torch.exp(chosen_avg_logp.clamp(max=-1e-7)))
                                                        - torch.log1p(-torch.exp(rejected_avg_logp.clamp(max=-1e-7))))
    return chosen_nll - lambda_ * F.logsigmoid(log_odds)


def ld_dpo_logp(token_logps: torch.Tensor, mask: torch.Tensor, common_len: torch.Tensor | int, alpha: float):
    """LD-DPO (Liu et al. 2024) sequence log-probability: tokens past the shorter response's length weigh ``α``."""
    pos = torch.cumsum(mask.long(), dim=-1)
    common = torch.as_tensor(common_len, device=mask.device).reshape(-1, 1) if token_logps.ndim > 1 else common_len
    head = (pos <= common) & mask.bool()
    tail = (pos > common) & mask.bool()
    return (token_logps * head).sum(-1) + alpha * (token_logps * tail).sum(-1)


def wpo_weight(chosen_token_logps, chosen_mask, rejected_token_logps, rejected_mask, chosen_probs_sq=None,
               rejected_probs_sq=None):
    """WPO (Zhou et al. 2024) pair weight ``exp(Σ adjusted avg logp)`` clamped to 1 (treated as a constant)."""
    def avg(lp, m, sq):
        lp_adj = lp if sq is None else lp - sq
        return (lp_adj * m).sum(-1) / m.sum(-1).clamp_min(1)
    w = torch.exp(avg(chosen_token_logps, chosen_mask, chosen_probs_sq) + avg(rejected_token_logps, rejected_mask, rejected_probs_sq))
    return w.clamp(max=1.0).detach()


def f_divergence_logits(chosen_logratio, rejected_logratio, *, f_divergence_type: str = "reverse_kl", alpha: float = 0.5):
    """Pair logit for f-DPO (Wang et al. 2023): ``g(chosen) − g(rejected)`` with the per-side remap ``g`` of
    :func:`f_divergence_remap` (reverse KL: the plain difference).  ``alpha`` follows the reference's convention,
    ``g(x) = (e^{(α−1)x} − 1)/(α − 1)`` — TRL's coefficient is ``1 − α`` of this one; both agree at 0.5."""
    c, r = chosen_logratio, rejected_logratio
    if f_divergence_type == "reverse_kl":
        return c - r
    return (f_divergence_remap(c, f_divergence_type=f_divergence_type, alpha=alpha)
            - f_divergence_remap(r, f_divergence_type=f_divergence_type, alpha=alpha))


PAIR_HEADS = {"sigmoid": sigmoid_loss, "hinge": hinge_loss, "ipo": ipo_loss, "exo_pair": exo_loss, "nca_pair": nca_loss,
              "robust": robust_loss, "bco_pair": bco_loss, "sppo_hard": sppo_loss, "apo_zero": apo_zero_loss,
              "apo_down": apo_down_loss, "discopop": discopop_loss}
ALL_LOSS_TYPES = tuple(PAIR_HEADS) + ("sft", "chosen_nll", "cpo", "simpo", "orpo", "ld_dpo", "mpo", "wpo", "f_divergence")
REFERENCE_FREE = frozenset({"sft", "chosen_nll", "cpo", "simpo", "orpo"})      # heads that never read the reference policy
MPO_MIX = (("sigmoid", 0.8), ("bco_pair", 0.2), ("sft", 1.0))


def dpo_loss(loss_type: str | Sequence[str], *, chosen_logratio, rejected_logratio, beta: float = 0.1,
             label_smoothing: float = 0.0, loss_weights: Sequence[float] | None = None, chosen_nll=None,
             chosen_avg_logp=None, rejected_avg_logp=None, bco_delta=0.0, discopop_tau: float = 0.05,
             simpo_gamma: float = 0.5, orpo_lambda: float = 1.0, f_divergence_type: str = "reverse_kl",
             f_alpha: float = 0.5, pair_weight=None, chosen_logp=None, rejected_logp=None, cpo_alpha: float = 1.0):
    """Dispatch one head or a weighted mixture of heads; returns one loss per pair.

    ``cpo`` is reference-free: the sigmoid head on the SUMMED policy log-probabilities (``chosen_logp``,
    ``rejected_logp``) plus ``cpo_alpha`` times the per-token-mean chosen NLL
    (parity: packages/opaque-transformers/src/opaque/api/transformers/trl/_dpo_trainer.py:934-941)."""
    types = [loss_type] if isinstance(loss_type, str) else list(loss_type)
    if types == ["mpo"]:
        types, loss_weights = [t for t, _ in MPO_MIX], [w for _, w in MPO_MIX]
    weights = list(loss_weights) if loss_weights is not None else [1.0] * len(types)
    if len(weights) != len(types):
        raise ValueError("loss_weights must match loss_type")
    c, r = chosen_logratio, rejected_logratio
    if f_divergence_type != "reverse_kl":
        d = f_divergence_logits(c, r, f_divergence_type=f_divergence_type, alpha=f_alpha)
        c, r = d, torch.zeros_like(d)
    total = 0.0
    for t, w in zip(types, weights):
        if t in ("sigmoid", "ld_dpo", "wpo", "f_divergence"):
            term = sigmoid_loss(c, r, beta=beta, label_smoothing=label_smoothing)
        elif t in ("robust", "exo_pair"):
            term = PAIR_HEADS[t](c, r, beta=beta, label_smoothing=label_smoothing or (0.1 if t == "robust" else 1e-3))
        elif t == "bco_pair":
            term = bco_loss(c, r, beta=beta, delta=bco_delta)
        elif t == "discopop":
            term = discopop_loss(c, r, beta=beta, discopop_tau=discopop_tau)
        elif t in PAIR_HEADS:
            term = PAIR_HEADS[t](c, r, beta=beta)
        elif t in ("sft", "chosen_nll"):
            term = chosen_nll                      # already the per-example mean NLL of the chosen response
        elif t == "cpo":
            if chosen_logp is None or rejected_logp is None:
                raise ValueError("cpo needs the policy log-probabilities chosen_logp / rejected_logp")
            term = sigmoid_loss(chosen_logp, rejected_logp, beta=beta, label_smoothing=label_smoothing) \
                + cpo_alpha * chosen_nll
        elif t == "simpo":
            term = simpo_loss(chosen_avg_logp, rejected_avg_logp, beta=beta, gamma=simpo_gamma, label_smoothing=label_smoothing)
        elif t == "orpo":
            term = orpo_loss(chosen_avg_logp, rejected_avg_logp, chosen_nll, lambda_=orpo_lambda)
        else:
            raise ValueError(f"unknown DPO loss type {t!r}; expected one of {ALL_LOSS_TYPES}")
        total = total + w * term
    if pair_weight is not None:
        total = total * pair_weight
    return total


def reward_margins(chosen_logratio, rejected_logratio, beta: float):
    """Implicit rewards ``β·logratio`` and their margin / accuracy (logging metrics)."""
    cr, rr = beta * chosen_logratio.detach(), beta * rejected_logratio.detach()
    return {"rewards/chosen": cr, "rewards/rejected": rr, "rewards/margins": cr - rr,
            "rewards/accuracies": (cr > rr).float()}


__all__ = ["ALL_LOSS_TYPES", "PAIR_HEADS", "REFERENCE_FREE", "apo_down_loss", "apo_zero_loss", "bco_loss", "chosen_nll_loss",
           "discopop_loss", "dpo_loss", "exo_loss", "f_divergence_logits", "hinge_loss", "ipo_loss", "ld_dpo_logp",
           "nca_loss", "orpo_loss", "reward_margins", "robust_loss", "sigmoid_loss", "simpo_loss", "sppo_loss",
           "wpo_weight"]


# ------------------------------------------------------------------------------------------------------------------
# Building blocks under the names of the reference's ``alignment.dpo.loss`` / ``.metric`` / ``.data`` namespaces.
# Parity: packages/opaque-alignment/src/opaque/api/alignment/dpo/loss/{_orpo,_f_divergence,_mpo,_wpo,_ld_dpo}.py,
# dpo/metric/_reward.py, dpo/data/_prompt.py.

def _log1mexp(x: torch.Tensor) -> torch.Tensor:
    """``log(1 − eˣ)`` for ``x < 0`` without cancellation (two branches around ``−ln 2``)."""
    x = x.clamp(max=-1e-7)
    return torch.where(x > -0.6931471805599453, torch.log(-torch.expm1(x)), torch.log1p(-torch.exp(x)))


def odds_ratio_loss(chosen_logp: torch.Tensor, rejected_logp: torch.Tensor) -> torch.Tensor:
    """ORPO's odds-ratio term ``−log σ(log odds(y_w) − log odds(y_l))`` with ``log odds(y) = log p − log(1 − p)``;
    both arguments are length-normalised log-probabilities (``< 0``).  The full ORPO loss adds the chosen NLL."""
    log_odds = (chosen_logp - _log1mexp(chosen_logp)) - (rejected_logp - _log1mexp(rejected_logp))
    return -F.logsigmoid(log_odds)


def f_divergence_remap(logratio: torch.Tensor, *, f_divergence_type: str = "reverse_kl", alpha: float = 1.0) -> torch.Tensor:
    """Per-side remap ``g`` of a log-ratio for f-DPO: ``reverse_kl`` ``g(x) = x``; ``forward_kl`` ``1 − e^{−x}``;
    ``js_divergence`` ``ln 2 + log σ(x)``; ``alpha_divergence`` ``(e^{(α−1)x} − 1)/(α − 1)`` (identity at ``α = 1``).
    Exponentials are capped at ``e⁸⁰``.  The pair logit is ``g(chosen) − g(rejected)``."""
    cap = 80.0
    if f_divergence_type == "reverse_kl":
        return logratio
    if f_divergence_type == "forward_kl":
        return 1.0 - torch.exp((-logratio).clamp(max=cap))
    if f_divergence_type == "js_divergence":
        return math.log(2.0) + F.logsigmoid(logratio)
    if f_divergence_type == "alpha_divergence":
        if abs(alpha - 1.0) < 1e-6:
            return logratio
        return (torch.exp(((alpha - 1.0) * logratio).clamp(max=cap)) - 1.0) / (alpha - 1.0)
    raise ValueError(f"unknown f-divergence {f_divergence_type!r}")


def mpo_combine(losses: Mapping[str, torch.Tensor], weights: Mapping[str, float]) -> torch.Tensor:
    """``Σ_k weights[k] · losses[k]`` over the keys of ``weights`` (a mixture of heads; ``losses`` may hold more)."""
    missing = sorted(set(weights) - set(losses))
    if missing:
        raise KeyError(f"weights name losses that were not computed: {missing} (available: {sorted(losses)})")
    if not weights:
        raise ValueError("weights is empty")
    total = None
    for name, w in weights.items():
        term = float(w) * losses[name]
        total = term if total is None else total + term
    return total


def wpo_weights(per_token_logps: torch.Tensor, completion_mask: torch.Tensor) -> torch.Tensor:
    """WPO's per-sequence weight: ``exp`` of the policy's mean per-token log-probability on the completion, DETACHED
    (a multiplicative reweighting, no gradient).  Shapes ``(..., T)`` → ``(...)``; an empty mask gives weight 1."""
    mask = completion_mask.to(per_token_logps.dtype)
    count = (completion_mask != 0).sum(-1).clamp(min=1)
    avg = (per_token_logps.float() * mask.float()).sum(-1) / count
    return avg.detach().exp()


def ld_dpo_split(per_token_logps: torch.Tensor, completion_mask: torch.Tensor, shared_prefix_len, alpha: float) -> torch.Tensor:
    """LD-DPO sequence log-probability: the first ``shared_prefix_len`` completion tokens weigh 1, later ones ``alpha``
    (``alpha = 1`` is the plain masked sum).  ``shared_prefix_len`` is an int or a per-example tensor."""
    mask = completion_mask.to(per_token_logps.dtype)
    pos = (completion_mask != 0).cumsum(-1)
    limit = shared_prefix_len
    if isinstance(limit, torch.Tensor):
        while limit.ndim < pos.ndim:
            limit = limit.unsqueeze(-1)
    head = (pos >= 1) & (pos <= limit)
    weight = torch.where(head, torch.ones_like(mask), torch.full_like(mask, float(alpha)))
    return (per_token_logps * mask * weight).sum(-1)


def reward_metrics(chosen_logratio: torch.Tensor, rejected_logratio: torch.Tensor, *, beta: float) -> dict[str, torch.Tensor]:
    """``rewards/chosen``, ``rewards/rejected``, ``rewards/accuracies``, ``rewards/margins`` (detached means) from the
    per-pair log-ratios; implicit reward = ``β · logratio``.  For logging on NON-private data (or add noise first)."""
    c, r = chosen_logratio.detach().float(), rejected_logratio.detach().float()
    return {"rewards/chosen": (beta * c).mean(), "rewards/rejected": (beta * r).mean(),
            "rewards/accuracies": (c > r).float().mean(), "rewards/margins": (beta * (c - r)).mean()}


def extract_prompt(example: Mapping[str, Any]) -> dict:
    """Split the longest common prefix of ``chosen`` and ``rejected`` (lists: tokens or chat messages) off as ``prompt``.
    Rows that already have a ``prompt``, or no chosen / rejected pair, come back unchanged; other keys are kept."""
    row = dict(example)
    if "prompt" in row or "chosen" not in row or "rejected" not in row:
        return row
    chosen, rejected = row["chosen"], row["rejected"]
    if not isinstance(chosen, (list, tuple)) or not isinstance(rejected, (list, tuple)):
        raise TypeError("extract_prompt needs list-valued 'chosen' and 'rejected' (token ids or messages)")
    k = 0
    while k < min(len(chosen), len(rejected)) and chosen[k] == rejected[k]:
        k += 1
    row["prompt"], row["chosen"], row["rejected"] = list(chosen[:k]), list(chosen[k:]), list(rejected[k:])
    return row


def completion_logp(logits: torch.Tensor, input_ids: torch.Tensor, completion_mask: torch.Tensor, *, ld_alpha: float | None = None,
                    shared_prefix_len=None, length_normalized: bool = False) -> torch.Tensor:
    """Per-sequence log-probability of the COMPLETION tokens from UNSHIFTED tensors: ``logits (..., T, V)``, ``input_ids`` and
    ``completion_mask`` ``(..., T)``; position ``t`` scores token ``t + 1`` (the shift happens here).  ``ld_alpha`` with
    ``shared_prefix_len`` applies the LD-DPO weighting (:func:`ld_dpo_split`); ``length_normalized`` divides by the number
    of completion tokens.  This is ``sequence_logp`` of the reference's ``alignment.dpo.loss`` namespace; the
    ``(logits, labels)`` form with pre-aligned labels is ``alignment.sft.sequence_logp``.

    Parity: packages/opaque-alignment/src/opaque/api/alignment/logprob/_sequence.py:31."""
    if ld_alpha is not None and shared_prefix_len is None:
        raise ValueError("ld_alpha needs shared_prefix_len")
    z = logits[..., :-1, :].float()
    target, mask = input_ids[..., 1:], completion_mask[..., 1:]
    lp = torch.gather(z.log_softmax(-1), -1, target.unsqueeze(-1).long()).squeeze(-1)
    if ld_alpha is not None:
        total = ld_dpo_split(lp, mask, shared_prefix_len, ld_alpha)
    else:
        total = (lp * mask.to(lp.dtype)).sum(-1)
    if length_normalized:
        total = total / (mask != 0).sum(-1).clamp(min=1)
    return total


def fused_completion_logp(hidden_states: torch.Tensor, lm_head_weight: torch.Tensor, input_ids: torch.Tensor,
                          completion_mask: torch.Tensor, *, length_normalized: bool = False) -> torch.Tensor:
    """:func:`completion_logp` from final hidden states ``[B, T, d]`` and the output head, without keeping logits (the fused
    head + cross-entropy node); no LD-DPO weighting here — that needs per-token values."""
    from .sft import IGNORE_INDEX, fused_sequence_logp
    labels = torch.full_like(input_ids, IGNORE_INDEX)
    keep = completion_mask[..., 1:] != 0
    labels[..., :-1] = torch.where(keep, input_ids[..., 1:], torch.full_like(input_ids[..., 1:], IGNORE_INDEX))
    return fused_sequence_logp(hidden_states, lm_head_weight, labels, average=length_normalized)


__all__ += ["completion_logp", "fused_completion_logp", "extract_prompt", "f_divergence_remap", "ld_dpo_split", "mpo_combine", "odds_ratio_loss", "reward_metrics", "wpo_weights"]
