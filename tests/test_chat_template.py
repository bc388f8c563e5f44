"""Assistant-only loss masks from chat templates: marker installation on several template styles, mask extraction."""
import pytest

from opaque_b200.alignment.chat_template import (GEN_START, apply_chat_template_with_mask, clone_chat_template,
                                                 get_training_chat_template)

CHATML = ("{% for message in messages %}{{'<|im_start|> ' + message['role'] + ' \n ' + message['content'] + ' <|im_end|> ' + '\n '}}"
          "{% endfor %}{% if add_generation_prompt %}{{ '<|im_start|> assistant \n ' }}{% endif %}")
LLAMA3 = ("{% set loop_messages = messages %}{% for message in loop_messages %}{% set content = '<|start_header_id|>' + message['role'] + "
          "'<|end_header_id|>\n\n'+ message['content'] | trim + '<|eot_id|>' %}{% if loop.index0 == 0 %}{% set content = bos_token + content %}"
          "{% endif %}{{ content }}{% endfor %}{% if add_generation_prompt %}{{ '<|start_header_id|>assistant<|end_header_id|>\n\n' }}{% endif %}")
GEMMA = ("{{ bos_token }}{% for message in messages %}{% if (message['role'] == 'assistant') %}{% set role = 'model' %}{% else %}"
         "{% set role = message['role'] %}{% endif %}{{ '<start_of_turn>' + role + '\n' + message['content'] | trim + '<end_of_turn>\n' }}"
         "{% endfor %}{% if add_generation_prompt %}{{'<start_of_turn>model\n'}}{% endif %}")
PHI3 = ("{% for message in messages %}{% if message['role'] == 'system' %}{{'<|system|>\n' + message['content'] + '<|end|>\n'}}"
        "{% elif message['role'] == 'user' %}{{'<|user|>\n' + message['content'] + '<|end|>\n'}}{% elif message['role'] == 'assistant' %}"
        "{{'<|assistant|>\n' + message['content'] + '<|end|>\n'}}{% endif %}{% endfor %}")
QWEN = ("{%- for message in messages %}{%- if (message.role == \"user\") or (message.role == \"system\" and not loop.first) or "
        "(message.role == \"assistant\" and not message.tool_calls) %}{{- '<|im_start|>' + message.role + '\n' + message.content + "
        "'<|im_end|>' + '\n' }}{%- elif message.role == \"assistant\" %}{{- '<|im_start|>' + message.role }}{%- endif %}{%- endfor %}")


class _Tok:
    bos_token, eos_token, pad_token, unk_token = "<s>", "</s>", None, None

    def __init__(self, template):
        self.chat_template = template


@pytest.mark.parametrize("template", [CHATML, LLAMA3, GEMMA, PHI3, QWEN], ids=["chatml", "llama3", "gemma", "phi3", "qwen"])
def test_generation_markers_are_installed_and_verified(template):
    out = get_training_chat_template(_Tok(template))
    assert GEN_START in out
    assert get_training_chat_template(_Tok(out)) == out            # idempotent


def test_unmarkable_templates_are_refused():
    with pytest.raises(ValueError):
        get_training_chat_template(_Tok("{{ messages | length }}"))
    with pytest.raises(ValueError):
        get_training_chat_template(_Tok(None))


def _tokenizer():
    from tokenizers import Tokenizer, models, pre_tokenizers
    from transformers import PreTrainedTokenizerFast
    vocab = {w: i for i, w in enumerate(["<unk>", "<|im_start|>", "<|im_end|>", "user", "assistant", "system", "hello", "world", "hi",
                                          "there", "be", "brief", "bye"])}
    tk = Tokenizer(models.WordLevel(vocab, unk_token="<unk>"))
    tk.pre_tokenizer = pre_tokenizers.WhitespaceSplit()
    tok = PreTrainedTokenizerFast(tokenizer_object=tk, unk_token="<unk>")
    # (turns separated by a literal outside the content expression: this toy tokenizer has no whitespace tokens, so a marked
    # span must begin and end on token characters for Hugging Face's character-to-token mapping)
    tok.chat_template = "{% for message in messages %}{{'<|im_start|> ' + message['role'] + ' ' + message['content'] + ' <|im_end|>'}}{{ ' ' }}{% endfor %}"
    return tok


def test_assistant_mask_covers_exactly_the_assistant_turns():
    tok = _tokenizer()
    conv = [{"role": "system", "content": "be brief"}, {"role": "user", "content": "hello world"},
            {"role": "assistant", "content": "hi there"}, {"role": "user", "content": "bye"}, {"role": "assistant", "content": "bye"}]
    with pytest.raises(ValueError, match="generation"):
        apply_chat_template_with_mask(tok, conv)                     # no markers yet
    tok.chat_template = get_training_chat_template(tok)
    out = apply_chat_template_with_mask(tok, conv)
    toks = tok.convert_ids_to_tokens(out["input_ids"])
    assert len(toks) == len(out["completion_mask"])
    role = None
    for i, t in enumerate(toks):                                     # content tokens inherit the role named after <|im_start|>
        if t == "<|im_start|>":
            role = toks[i + 1]
        elif t not in ("<|im_end|>", "user", "assistant", "system") and toks[i - 1] != "<|im_start|>":
            assert out["completion_mask"][i] == int(role == "assistant"), (i, t, role)   # (turn delimiters depend on the tokenizer's offsets)
    with pytest.raises(TypeError):
        apply_chat_template_with_mask(tok, conv, tokenize=False)
    # the SFT collator consumes the mask as the completion mask
    from opaque_b200.alignment.data import language_modeling_collator
    batch = language_modeling_collator([out], completion_only=True)
    scored = (batch["labels"][0] != -100).sum().item()
    assert 0 < scored <= sum(out["completion_mask"])


def test_clone_chat_template_adds_missing_special_tokens():
    src, dst = _tokenizer(), _tokenizer()
    src.add_special_tokens({"additional_special_tokens": ["<|tool|>"]})
    dst.chat_template = None
    grown = []

    class M:
        def resize_token_embeddings(self, n):
            grown.append(n)
    _, dst, added = clone_chat_template(M(), dst, src)
    assert dst.chat_template == src.chat_template and "<|tool|>" in dst.get_vocab() and len(added) == 1 and grown == [len(dst)]
