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
    # capped attention scores and a sliding window shorter than the sequence: the flash-attention library path
    yield "gemma2", T.Gemma2Config(**COMMON, head_dim=32, sliding_window=32, query_pre_attn_scalar=32), T.Gemma2ForCausalLM
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


def test_inplace_patched_qwen3_next_modules_match_the_hugging_face_code():
    """The in-place family path on the GPU, module by module: RMSNorm, gated MLP and routed experts of Qwen3-Next run on this
    package's kernels (grouped tcgen05 GEMM for the experts) and reproduce the Hugging Face forward and backward in bf16.
    Only the patched module classes are instantiated: the model's delta-net layers (third-party Triton kernels) are not
    part of what is patched and are not run here."""
    import transformers
    import transformers.models.qwen3_next.modeling_qwen3_next as mq
    from opaque_b200.ops import lib
    from opaque_b200.patches import inplace
    cfg = transformers.Qwen3NextConfig(vocab_size=256, hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                                       num_attention_heads=4, num_key_value_heads=2, head_dim=32, num_experts=4,
                                       num_experts_per_tok=2, moe_intermediate_size=128, shared_expert_intermediate_size=128)
    torch.manual_seed(0)
    rel = lambda a, b: float((a.float() - b.float()).norm() / (b.float().norm() + 1e-30))

    class Box(torch.nn.Module):                      # a holder whose config names the family
        def __init__(self):
            super().__init__()
            self.config = cfg
            self.norm = mq.Qwen3NextRMSNorm(128, eps=1e-6)
            self.mlp = mq.Qwen3NextMLP(cfg, intermediate_size=256)
            self.experts = mq.Qwen3NextExperts(cfg)
    box = Box()
    with torch.no_grad():
        box.norm.weight.normal_(0, 0.1)
        box.experts.gate_up_proj.normal_(0, 0.05)
        box.experts.down_proj.normal_(0, 0.05)
    box = box.to("cuda", torch.bfloat16)
    x = torch.randn(96, 128, device="cuda").bfloat16()
    idx = torch.stack([torch.randperm(4, device="cuda")[:2] for _ in range(96)])
    wts = torch.rand(96, 2, device="cuda").bfloat16()

    def run():
        out = []
        for fn in (lambda v: box.norm(v), lambda v: box.mlp(v), lambda v: box.experts(v, idx, wts)):
            v = x.clone().requires_grad_(True)
            y = fn(v)
            y.float().square().mean().backward()
            out.append((y.detach(), v.grad))
        return out

    want = run()
    counts = inplace.apply_inplace_patches(box)
    assert counts == {"rms_norm": 1, "mlp": 1, "experts": 1}
    before = lib.LAUNCHES
    got = run()
    assert lib.LAUNCHES > before, "the kernel path did not run"
    for (y, gx), (yw, gw), name in zip(got, want, ("rms_norm", "mlp", "experts")):
        assert rel(y, yw) < 2e-2 and rel(gx, gw) < 4e-2, name
    assert inplace.remove_inplace_patches(box) == 3
