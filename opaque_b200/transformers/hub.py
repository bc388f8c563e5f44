"""Uploading a trained model to the Hugging Face Hub.

``DPTrainer.push_to_hub()`` saves the model and its model card into ``output_dir`` and uploads that folder in ONE commit
through a client object with the two calls ``create_repo(repo_id, token=, private=, exist_ok=)`` and
``upload_folder(repo_id=, folder_path=, commit_message=, token=, revision=, ignore_patterns=, run_as_future=)`` —
``huggingface_hub.HfApi`` by default, any stand-in with those two methods in tests or behind a company mirror.

What is NEVER uploaded: ``checkpoint-*`` folders and the run-state files inside or beside them (``dp_state.pt``,
``optimizer.pt``, ``rng_state*.pth``, ``dp_noise_buffers.pt``).  They hold the keys of the noise generator and of the
batch sampler; publishing them lets a reader subtract the noise and voids the privacy guarantee, so the ignore list is
fixed here rather than left to the caller.

Parity: packages/opaque-transformers/src/opaque/api/transformers/trainer/_hub.py (repo creation, one-commit folder upload
with checkpoint folders ignored, model card with the privacy section).
"""
from __future__ import annotations

import os
from typing import Any

# folder upload: everything below output_dir except these
NEVER_UPLOADED = ("checkpoint-*", "checkpoint-*/**", "_*", "runs/**", "*.tmp", "*.tmp/**", "dp_state.pt", "optimizer.pt",
                  "rng_state*.pth", "dp_noise_buffers.pt")


def default_client() -> Any:
    """``huggingface_hub.HfApi()``: the client used when neither ``client=`` nor ``trainer.hub_client`` is given."""
    try:
        from huggingface_hub import HfApi
    except ImportError as exc:       # pragma: no cover - the library ships with transformers
        raise RuntimeError("push_to_hub needs the huggingface_hub package (or pass client=...)") from exc
    return HfApi()


def resolve_repo_id(args: Any) -> str:
    """``hub_model_id`` if given, else the last component of ``output_dir``."""
    if args.hub_model_id:
        return str(args.hub_model_id)
    if not args.output_dir:
        raise ValueError("push_to_hub needs hub_model_id or an output_dir to name the repository after")
    return os.path.basename(os.path.abspath(args.output_dir))


def init_hub_repo(trainer: Any, token: str | None = None, client: Any = None) -> str:
    """Create the repository if it does not exist; remembers and returns its full id (``user/name``)."""
    a = trainer.args
    client = client or getattr(trainer, "hub_client", None) or default_client()
    made = client.create_repo(resolve_repo_id(a), token=token or a.hub_token, private=a.hub_private_repo, exist_ok=True)
    trainer.hub_repo_id = str(getattr(made, "repo_id", None) or resolve_repo_id(a))
    return trainer.hub_repo_id


def push_to_hub(trainer: Any, commit_message: str | None = "End of training", blocking: bool = True, token: str | None = None,
                revision: str | None = None, client: Any = None, model_name: str | None = None, **card_fields: Any) -> Any:
    """Save model + model card into ``output_dir`` (rank 0 writes) and upload the folder; other ranks return ``None``.

    Returns what the client's ``upload_folder`` returns (a commit description, or a future with ``blocking=False``).
    """
    a = trainer.args
    if not a.output_dir:
        raise ValueError("push_to_hub uploads output_dir: set it")
    client = client or getattr(trainer, "hub_client", None) or default_client()
    trainer.save_model(a.output_dir)                      # collective on several ranks (write-back, barriers)
    if not trainer.is_world_process_zero():
        return None
    if getattr(trainer, "hub_repo_id", None) is None:
        init_hub_repo(trainer, token=token, client=client)
    name = model_name or trainer.hub_repo_id.split("/")[-1]
    trainer.create_model_card(model_name=name, **card_fields)
    return client.upload_folder(repo_id=trainer.hub_repo_id, folder_path=a.output_dir, commit_message=commit_message or "End of training",
                                token=token or a.hub_token, revision=revision or a.hub_revision,
                                ignore_patterns=list(NEVER_UPLOADED), run_as_future=not blocking)


__all__ = ["NEVER_UPLOADED", "default_client", "init_hub_repo", "push_to_hub", "resolve_repo_id"]
