"""Chat templates for alignment training: assistant-only loss masks and template cloning.

``assistant_only_loss`` needs to know which tokens of a rendered conversation were produced by assistant turns.
Hugging Face tokenizers report that (``return_assistant_tokens_mask=True``) only for templates whose assistant content
sits inside ``{% generation %} … {% endgeneration %}``; most published templates do not carry the markers.

:func:`get_training_chat_template` installs them with ONE rewrite rule that covers explicit assistant branches
(ChatML, Llama-3, Phi-3), role-agnostic shared clauses (Qwen-2.5) and templates that rename the role on output
(Gemma's ``model``): every ``{{ … <msg>['content'] … }}`` expression inside the message loop becomes ::

    {% if <msg>['role'] == 'assistant' %}{% generation %}{{ … }}{% endgeneration %}{% else %}{{ … }}{% endif %}

and the result is accepted only after a probe render (distinct user / assistant probe strings, spans recorded by a
small Jinja extension) shows that the marked spans contain the assistant text and none of the user text.  A template
that cannot be verified is refused — a wrong mask would silently train on prompts.

Parity: packages/opaque-alignment/src/opaque/api/alignment/data/_chat_template.py (clone_chat_template,
get_training_chat_template) and _completion_mask.py (apply_chat_template_with_mask); the reference reaches the same
markers through four template-specific strategies.
"""
from __future__ import annotations

import re
from typing import Any

GEN_START, GEN_END = "{% generation %}", "{% endgeneration %}"
_USER_PROBE, _ASSISTANT_PROBE, _SYSTEM_PROBE = "uuUSERPROBEuu", "aaASSISTANTPROBEaa", "ssSYSTEMPROBEss"


def _jinja_env():
    import jinja2
    from jinja2.ext import Extension
    from jinja2.sandbox import ImmutableSandboxedEnvironment

    class GenerationSpans(Extension):
        """``{% generation %}`` blocks render their body and record its character span in ``environment.spans``."""
        tags = {"generation"}

        def parse(self, parser):
            lineno = next(parser.stream).lineno
            body = parser.parse_statements(["name:endgeneration"], drop_needle=True)
            return jinja2.nodes.CallBlock(self.call_method("_mark"), [], [], body).set_lineno(lineno)

        def _mark(self, caller):
            text = caller()
            self.environment.marked.append(text)
            return text

    env = ImmutableSandboxedEnvironment(trim_blocks=True, lstrip_blocks=True, extensions=[GenerationSpans])
    env.marked = []
    env.globals["raise_exception"] = lambda msg: (_ for _ in ()).throw(ValueError(msg))
    env.globals["strftime_now"] = lambda fmt: ""
    return env


def _probe_marks_only_assistant(template: str, tokenizer: Any = None) -> bool:
    """Render a two-turn probe conversation and check what the generation blocks captured."""
    try:
        env = _jinja_env()
        tpl = env.from_string(template)
        special = {k: getattr(tokenizer, k, "") or "" for k in ("bos_token", "eos_token", "pad_token", "unk_token")} if tokenizer else {}
        for with_system in (False, True):
            msgs = ([{"role": "system", "content": _SYSTEM_PROBE}] if with_system else []) + [
                {"role": "user", "content": _USER_PROBE}, {"role": "assistant", "content": _ASSISTANT_PROBE},
                {"role": "user", "content": _USER_PROBE + "2"}, {"role": "assistant", "content": _ASSISTANT_PROBE + "2"}]
            env.marked.clear()
            try:
                tpl.render(messages=msgs, add_generation_prompt=False, **special)
            except Exception:      # noqa: BLE001 — some templates refuse system turns; the plain conversation decides
                if with_system:
                    continue
                return False
            marked = "".join(env.marked)
            if marked.count(_ASSISTANT_PROBE) < 2 or _USER_PROBE in marked or _SYSTEM_PROBE in marked:
                return False
        return True
    except Exception:      # noqa: BLE001
        return False


def _loop_variable(template: str) -> str | None:
    m = re.search(r"{%-?\s*for\s+(\w+)\s+in\s+(?:loop_)?messages", template)
    return m.group(1) if m else None


def get_training_chat_template(tokenizer: Any) -> str:
    """The tokenizer's chat template with ``{% generation %}`` markers around assistant content (idempotent).

    Raises ``ValueError`` when the template is missing or when no rewrite passes the probe check.
    """
    template = getattr(tokenizer, "chat_template", None)
    if not template:
        raise ValueError("tokenizer.chat_template is not set: assign a Jinja chat template first")
    if GEN_START in template:
        return template
    if "{{ generation_token }}" in template:            # explicit placeholder some templates carry for this purpose
        cand = template.replace("{{ generation_token }}", f"{GEN_START}{{{{ generation_token }}}}{GEN_END}", 1)
        if _probe_marks_only_assistant(cand, tokenizer):
            return cand
    var = _loop_variable(template)
    if var is not None:
        # every output expression that mentions the loop message's content (subscript or attribute access, any quotes)
        content = rf"{var}(?:\[\s*['\"]content['\"]\s*\]|\.content)"
        expr = re.compile(r"{{-?\s*(?:(?!}}).)*?" + content + r"(?:(?!}}).)*?-?}}", re.S)
        role = f"{var}['role']"

        def guard(m: re.Match) -> str:
            e = m.group(0)
            return f"{{% if {role} == 'assistant' %}}{GEN_START}{e}{GEN_END}{{% else %}}{e}{{% endif %}}"
        cand, n = expr.subn(guard, template)
        if n and _probe_marks_only_assistant(cand, tokenizer):
            return cand
        # content copied into a local first ({% set content = message['content'] %} … {{ content }}): guard those outputs
        local = re.search(r"{%-?\s*set\s+(\w+)\s*=\s*(?:(?!%}).)*?" + content, template, re.S)
        if local is not None:
            name = local.group(1)
            expr2 = re.compile(r"{{-?\s*(?:(?!}}).)*?\b" + re.escape(name) + r"\b(?:(?!}}).)*?-?}}", re.S)
            cand, n = expr2.subn(guard, template)
            if n and _probe_marks_only_assistant(cand, tokenizer):
                return cand
    raise ValueError("could not mark the assistant turns of this chat template in a way that passes the probe check; "
                     f"add '{GEN_START}' / '{GEN_END}' around the assistant content by hand")


def apply_chat_template_with_mask(tokenizer: Any, conversation: list[dict[str, Any]], **kwargs: Any) -> dict[str, Any]:
    """Tokenize one conversation; returns ``input_ids`` and ``completion_mask`` (1 on assistant-turn tokens).

    The active template (``kwargs['chat_template']`` or the tokenizer's) must carry the generation markers: without
    them Hugging Face returns an all-zero mask with only a log line, so the check happens here and raises.
    """
    active = kwargs.get("chat_template") or getattr(tokenizer, "chat_template", None)
    if not active or GEN_START not in active:
        raise ValueError("the active chat template has no '{% generation %}' markers, so no assistant-token mask can be "
                         "produced: tokenizer.chat_template = get_training_chat_template(tokenizer)")
    for fixed in ("tokenize", "return_assistant_tokens_mask", "return_dict"):
        if fixed in kwargs:
            raise TypeError(f"{fixed} is set by apply_chat_template_with_mask")
    enc = tokenizer.apply_chat_template(conversation, tokenize=True, return_assistant_tokens_mask=True, return_dict=True, **kwargs)
    mask = enc.get("assistant_masks")
    if mask is None or len(mask) == 0 or not any(mask):
        raise ValueError("the tokenizer returned no assistant-token mask for this conversation (no assistant turn, or a "
                         "template whose markers do not enclose it)")
    out = {"input_ids": list(enc["input_ids"]), "completion_mask": [int(x) for x in mask]}
    if enc.get("attention_mask") is not None:
        out["attention_mask"] = list(enc["attention_mask"])
    return out


def clone_chat_template(model: Any, tokenizer: Any, source_tokenizer_or_path: Any):
    """Copy the chat template and the special tokens it needs from a source tokenizer; grow the embeddings to match.

    Returns ``(model, tokenizer, added_token_ids)``.  Do this BEFORE building a functional / flat view of the model's
    parameters: resizing replaces the embedding tensor.
    """
    src = source_tokenizer_or_path
    if isinstance(src, str):
        from transformers import AutoTokenizer
        src = AutoTokenizer.from_pretrained(src, trust_remote_code=False)
    if not getattr(src, "chat_template", None):
        raise ValueError("the source tokenizer has no chat template")
    tokenizer.chat_template = src.chat_template
    have = set(tokenizer.get_vocab())
    special = [t for t in getattr(src, "all_special_tokens", []) if t not in have]
    extra = [str(t) for t in getattr(src, "additional_special_tokens", []) if str(t) not in have and str(t) not in special]
    added = tokenizer.add_special_tokens({"additional_special_tokens": special + extra}) if special or extra else 0
    for name in ("eos_token", "pad_token", "bos_token"):
        tok = getattr(src, name, None)
        if tok is not None and tok in tokenizer.get_vocab() and name == "eos_token":
            tokenizer.eos_token = tok
        if tok is not None and getattr(tokenizer, name, None) is None and tok in tokenizer.get_vocab():
            setattr(tokenizer, name, tok)
    ids = tokenizer.convert_tokens_to_ids(special + extra) if added else []
    if added and model is not None and hasattr(model, "resize_token_embeddings"):
        model.resize_token_embeddings(len(tokenizer))
    return model, tokenizer, list(ids)


__all__ = ["apply_chat_template_with_mask", "clone_chat_template", "get_training_chat_template"]
