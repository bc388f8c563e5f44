"""Converted Hugging Face models run on the CUDA kernels (bf16) and stay close to the source model's fp32 logits (B200)."""
import pytest
import torch

pytestmark = pytest.mark.gpu
transformers = pytest.importorskip("transformers")

COMMON = dict(vocab_size=320, hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
              max_position_embeddings=128)


def _cases():
    T = transformers
    yield "llama", T.LlamaConfig(**COMMON), T.LlamaForCausalLM
    yield "qwen2", T.Qwen2Config(**COMMON), T.Qwen2ForCausalLM
    yield "qwen3", T.Qwen3Config(**COMMON, head_dim=32), T.Qwen3ForCausalLM
    yield "gemma", T.GemmaConfig(**COMMON, head_dim=32), T.GemmaForCausalLM
    yield "gpt2", T.GPT2Config(vocab_size=320, n_positions=128, n_embd=128, n_layer=2, n_head=4), T.GPT2LMHeadModel
    yield "mixtral", T.MixtralConfig(**COMMON, num_local_experts=6, num_experts_per_tok=2), T.MixtralForCausalLM


@pytest.mark.parametrize("name,cfg,cls", list(_cases()), ids=[c[0] for c in _cases()])
def test_kernels_path_matches_hf(name, cfg, cls):
    from opaque_b200 import patches
    torch.manual_seed(0)
    hf = cls(cfg).eval().float()
    dev = torch.device("cuda", 0)
    ours = patches.apply_model_patches(hf, dtype=torch.bfloat16, device=dev).eval()
    ids = torch.randint(0, 320, (2, 64))
    with torch.no_grad():
        want = hf(ids).logits                                   # fp32 on the host
        got = ours(ids.to(dev)).float().cpu()[..., :want.shape[-1]]
        ref_bf16 = hf.to(torch.bfloat16)(ids).logits.float()    # what plain bf16 PyTorch loses against fp32
    err = float((got - want).norm() / want.norm())
    floor = float((ref_bf16 - want).norm() / want.norm())
    assert err < 3 * floor + 2e-3, (name, err, floor)
