"""Converted Hugging Face models (tiny random-init configs, no downloads) give the source model's logits on CPU."""
import pytest
import torch

transformers = pytest.importorskip("transformers")

from opaque_b200 import patches  # noqa: E402

COMMON = dict(vocab_size=320, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
              max_position_embeddings=128)


def _cases():
    T = transformers
    yield "llama", T.LlamaConfig(**COMMON, tie_word_embeddings=False), T.LlamaForCausalLM
    yield "llama-tied", T.LlamaConfig(**COMMON, tie_word_embeddings=True), T.LlamaForCausalLM
    yield "llama-rope-llama3", T.LlamaConfig(**COMMON, rope_parameters={
        "rope_type": "llama3", "rope_theta": 10000.0, "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
        "original_max_position_embeddings": 32}), T.LlamaForCausalLM
    yield "llama-rope-linear", T.LlamaConfig(**COMMON, rope_parameters={"rope_type": "linear", "rope_theta": 10000.0, "factor": 4.0}), T.LlamaForCausalLM
    yield "llama-rope-yarn", T.LlamaConfig(**COMMON, rope_parameters={
        "rope_type": "yarn", "rope_theta": 10000.0, "factor": 4.0, "original_max_position_embeddings": 32}), T.LlamaForCausalLM
    yield "llama-rope-dynamic", T.LlamaConfig(**{**COMMON, "max_position_embeddings": 128}, rope_parameters={
        "rope_type": "dynamic", "rope_theta": 10000.0, "factor": 2.0}), T.LlamaForCausalLM
    yield "mistral", T.MistralConfig(**COMMON, sliding_window=4096), T.MistralForCausalLM
    yield "mistral-window-shorter-than-sequence", T.MistralConfig(**COMMON, sliding_window=8), T.MistralForCausalLM
    yield "qwen2", T.Qwen2Config(**COMMON), T.Qwen2ForCausalLM
    yield "qwen3", T.Qwen3Config(**COMMON, head_dim=16), T.Qwen3ForCausalLM
    yield "gemma", T.GemmaConfig(**COMMON, head_dim=16), T.GemmaForCausalLM
    four = {**COMMON, "num_hidden_layers": 4}
    yield "gemma2", T.Gemma2Config(**four, head_dim=16, sliding_window=8, query_pre_attn_scalar=16), T.Gemma2ForCausalLM
    yield "gemma3_text", T.Gemma3TextConfig(**four, head_dim=16, sliding_window=8, query_pre_attn_scalar=16,
                                            layer_types=["sliding_attention", "sliding_attention", "full_attention", "sliding_attention"]), T.Gemma3ForCausalLM
    yield "olmo3", T.Olmo3Config(**four, sliding_window=8, pad_token_id=0), T.Olmo3ForCausalLM
    yield "exaone4", T.Exaone4Config(**four, sliding_window=8, pad_token_id=0), T.Exaone4ForCausalLM
    yield "cohere", T.CohereConfig(**COMMON, logit_scale=0.25, pad_token_id=0), T.CohereForCausalLM
    yield "cohere2", T.Cohere2Config(**four, sliding_window=8, logit_scale=0.25, pad_token_id=0), T.Cohere2ForCausalLM
    yield "glm4", T.Glm4Config(**four, head_dim=16, pad_token_id=0), T.Glm4ForCausalLM
    yield "phi3-partial-rotary", T.Phi3Config(**COMMON, pad_token_id=0, rope_parameters={"rope_type": "default", "rope_theta": 10000.0,
                                                                                        "partial_rotary_factor": 0.5}), T.Phi3ForCausalLM
    yield "phi3", T.Phi3Config(**COMMON, pad_token_id=0), T.Phi3ForCausalLM
    yield "granite", T.GraniteConfig(**COMMON, embedding_multiplier=6.0, attention_multiplier=0.11, residual_multiplier=0.4, logits_scaling=3.0), T.GraniteForCausalLM
    yield "olmo2", T.Olmo2Config(**COMMON, pad_token_id=0), T.Olmo2ForCausalLM
    yield "smollm3", T.SmolLM3Config(**COMMON, no_rope_layers=[1, 0], pad_token_id=0), T.SmolLM3ForCausalLM
    yield "qwen3_moe", T.Qwen3MoeConfig(**COMMON, moe_intermediate_size=32, num_experts=6, num_experts_per_tok=2, head_dim=16,
                                        norm_topk_prob=True), T.Qwen3MoeForCausalLM
    yield "qwen3_moe-dense-interleaved", T.Qwen3MoeConfig(**{**COMMON, "num_hidden_layers": 4}, moe_intermediate_size=32, num_experts=6,
                                                          num_experts_per_tok=2, head_dim=16, norm_topk_prob=True,
                                                          mlp_only_layers=[0], decoder_sparse_step=2), T.Qwen3MoeForCausalLM
    yield "hunyuan_v1_moe", T.HunYuanMoEV1Config(**{**COMMON, "intermediate_size": 48}, head_dim=16, num_experts=6, moe_topk=2,
                                                 pad_token_id=0), T.HunYuanMoEV1ForCausalLM
    yield "gpt_oss", T.GptOssConfig(**{**COMMON, "num_hidden_layers": 4, "intermediate_size": 48}, head_dim=16, num_local_experts=6,
                                    num_experts_per_tok=2, sliding_window=8, pad_token_id=0,
                                    rope_parameters={"rope_type": "yarn", "rope_theta": 150000.0, "factor": 4.0, "beta_fast": 32.0,
                                                     "beta_slow": 1.0, "truncate": False, "original_max_position_embeddings": 32}), T.GptOssForCausalLM
    yield "gpt2", T.GPT2Config(vocab_size=320, n_positions=128, n_embd=64, n_layer=2, n_head=4), T.GPT2LMHeadModel
    yield "mixtral", T.MixtralConfig(**COMMON, num_local_experts=6, num_experts_per_tok=2), T.MixtralForCausalLM
    yield "qwen2_moe", T.Qwen2MoeConfig(**COMMON, moe_intermediate_size=32, shared_expert_intermediate_size=48, num_experts=6,
                                        num_experts_per_tok=2), T.Qwen2MoeForCausalLM


@pytest.mark.parametrize("name,cfg,cls", list(_cases()), ids=[c[0] for c in _cases()])
def test_converted_model_matches_hf_logits(name, cfg, cls):
    torch.manual_seed(0)
    hf = cls(cfg).eval().float()
    with torch.no_grad():                                   # biases and attention sinks start at zero: make them count
        for n, p in hf.named_parameters():
            if n.endswith("bias") or "sinks" in n:
                p.normal_(0.0, 0.2)
    ours = patches.apply_model_patches(hf, dtype=torch.float32).eval()
    ids = torch.randint(0, 320, (2, 24))
    with torch.no_grad():
        want = hf(ids).logits
        got = ours(ids)
    got = got[..., :want.shape[-1]]                      # GPT-2 pads its vocabulary to a multiple of 64
    assert got.shape == want.shape
    assert float((got - want).abs().max()) < 2e-4 * max(1.0, float(want.abs().max())), name
    # and the per-example loss is the usual shifted mean NLL
    labels = torch.full_like(ids, -100)
    labels[:, :-1] = ids[:, 1:]
    ref = torch.stack([torch.nn.functional.cross_entropy(want[i, :-1], ids[i, 1:]) for i in range(2)])
    assert torch.allclose(ours.per_example_loss(ids, labels), ref, atol=2e-4)


def _tiny_qwen3_next(**kw):
    cfg = transformers.Qwen3NextConfig(
        vocab_size=128, hidden_size=64, intermediate_size=128, num_hidden_layers=4, num_attention_heads=4,
        num_key_value_heads=2, head_dim=16, max_position_embeddings=64, num_experts=4, num_experts_per_tok=2,
        moe_intermediate_size=64, shared_expert_intermediate_size=64, linear_num_value_heads=4, linear_num_key_heads=2,
        linear_key_head_dim=16, linear_value_head_dim=16, linear_conv_kernel_dim=4, full_attention_interval=2, **kw)
    torch.manual_seed(0)
    return transformers.Qwen3NextForCausalLM(cfg)


def test_inplace_families_keep_the_hugging_face_model_and_swap_forwards():
    """qwen3_next / qwen3_5_moe / deepseek_v4 are not converted: the Hugging Face model gets kernel forwards in place, which
    fall back to the original code off the GPU, so outputs are unchanged here; removing the patches restores the classes'
    forwards."""
    from opaque_b200.patches import inplace
    assert {"deepseek_v4", "qwen3_next", "qwen3_5_moe"} <= set(patches.supported_families())
    hf = _tiny_qwen3_next().float().eval()
    ids = torch.randint(0, 128, (2, 12))
    with torch.no_grad():
        want = hf(ids).logits
    out = patches.apply_model_patches(hf)
    assert out is hf
    counts = inplace.apply_inplace_patches(hf)                       # idempotent
    assert counts["rms_norm"] >= 9 and counts["mlp"] >= 4 and counts["experts"] == 4
    norm = next(m for m in hf.modules() if type(m).__name__ == "Qwen3NextRMSNorm")
    assert "forward" in norm.__dict__
    with torch.no_grad():
        got = hf(ids).logits
    assert torch.equal(got, want)
    assert inplace.remove_inplace_patches(hf) == sum(counts.values()) and "forward" not in norm.__dict__
    with pytest.raises(ValueError, match="instantiated"):
        patches.apply_model_patches({"model_type": "deepseek_v4"})
    with pytest.raises(ValueError, match="not an in-place family"):
        inplace.apply_inplace_patches(torch.nn.Linear(2, 2), "llama")


def test_unsupported_families_are_refused_with_a_reason():
    with pytest.raises(NotImplementedError, match="multimodal"):
        patches.apply_model_patches({"model_type": "gemma3"})
    with pytest.raises(NotImplementedError, match="per-head weights"):
        patches.apply_model_patches(transformers.CohereConfig(**COMMON, use_qk_norm=True))
    with pytest.raises(ValueError, match="no registered family"):
        patches.apply_model_patches({"model_type": "not_a_model"})


def test_lora_attach_through_the_patch_api():
    hf = transformers.LlamaForCausalLM(transformers.LlamaConfig(**COMMON)).float()
    m = patches.apply_model_patches(hf, dtype=torch.float32, r=8, lora_alpha=16, target_modules=("q_proj", "v_proj"))
    names = [n for n, p in m.named_parameters() if p.requires_grad]
    assert names and all("lora_" in n for n in names) and any("q_proj" in n for n in names) and not any("k_proj" in n for n in names)


@pytest.mark.parametrize("family", ["gemma2", "cohere", "glm4", "hunyuan_v1_moe", "gpt_oss"])
def test_converted_families_train_through_the_trainer_on_the_reference_engine(family, tmp_path):
    """Conversion output + ``DPTrainer`` + ``vmap`` per-example gradients: explicit capped attention, bias-free LayerNorm,
    permuted rotary layout and the dense expert form all have to pass through ``torch.func``."""
    from opaque_b200.transformers import DPTrainer, TrainingArguments
    T = transformers
    cfg, cls = {
        "gemma2": (T.Gemma2Config(**COMMON, head_dim=16, sliding_window=8, query_pre_attn_scalar=16), T.Gemma2ForCausalLM),
        "cohere": (T.CohereConfig(**COMMON, pad_token_id=0), T.CohereForCausalLM),
        "glm4": (T.Glm4Config(**COMMON, head_dim=16, pad_token_id=0), T.Glm4ForCausalLM),
        "hunyuan_v1_moe": (T.HunYuanMoEV1Config(**{**COMMON, "intermediate_size": 48}, head_dim=16, num_experts=6, moe_topk=2,
                                                pad_token_id=0), T.HunYuanMoEV1ForCausalLM),
        "gpt_oss": (T.GptOssConfig(**{**COMMON, "intermediate_size": 48}, head_dim=16, num_local_experts=6, num_experts_per_tok=2,
                                   sliding_window=8, pad_token_id=0), T.GptOssForCausalLM)}[family]
    torch.manual_seed(0)
    model = patches.apply_model_patches(cls(cfg).float(), dtype=torch.float32)
    g = torch.Generator().manual_seed(0)
    rows = [{"input_ids": torch.randint(0, 320, (24,), generator=g).tolist()} for _ in range(64)]
    args = TrainingArguments(output_dir=str(tmp_path), per_device_train_batch_size=8, max_steps=2, learning_rate=1e-3,
                             privacy_noise_multiplier=1.0, clipping_norm=1.0, use_cpu=True, save_steps=0, logging_steps=1)
    before = {n: p.detach().clone() for n, p in model.named_parameters()}
    out = DPTrainer(model=model, args=args, train_dataset=rows).train()
    assert out["global_step"] == 2 and out["epsilon"] > 0
    assert any(not torch.equal(p, before[n]) for n, p in model.named_parameters())


def _fake_peft_wrap(hf, r, alpha, targets, adapter="default", rslora=False):
    """The object layout that ``peft.get_peft_model(hf, LoraConfig(...))`` produces, rebuilt by hand (the library is not
    installed here): target linears replaced by a module with ``base_layer`` / ``lora_A[adapter]`` / ``lora_B[adapter]``,
    and a wrapper with ``peft_config`` and ``base_model.model``."""
    import types

    class LoraLinear(torch.nn.Module):
        def __init__(self, base):
            super().__init__()
            self.base_layer = base
            self.lora_A = torch.nn.ModuleDict({adapter: torch.nn.Linear(base.in_features, r, bias=False)})
            self.lora_B = torch.nn.ModuleDict({adapter: torch.nn.Linear(r, base.out_features, bias=False)})
            self.scaling = {adapter: alpha / (r ** 0.5 if rslora else r)}
            torch.nn.init.normal_(self.lora_B[adapter].weight, std=0.05)

        def forward(self, x):
            return self.base_layer(x) + self.lora_B[adapter](self.lora_A[adapter](x)) * self.scaling[adapter]

    for parent in list(hf.modules()):
        for name, child in list(parent.named_children()):
            if name in targets and isinstance(child, torch.nn.Linear):
                setattr(parent, name, LoraLinear(child))

    class Wrapper(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.base_model = torch.nn.Module()
            self.base_model.model = hf
            self.peft_config = {adapter: types.SimpleNamespace(peft_type="LORA", r=r, lora_alpha=alpha, target_modules=set(targets),
                                                               lora_dropout=0.0, bias="none", use_rslora=rslora,
                                                               use_dora=False, modules_to_save=None, fan_in_fan_out=False)}
            self.active_adapter = adapter

        def forward(self, ids):
            return self.base_model.model(ids)
    return Wrapper()


@pytest.mark.parametrize("family,rslora", [("llama", False), ("qwen2", True), ("llama-mlp", False), ("cohere", False)])
def test_peft_wrapped_model_converts_with_its_adapter(family, rslora):
    """A PEFT-wrapped Hugging Face model becomes a framework model with the same base weights and LoRA factors: same
    logits, only the factors trainable.  ``cohere`` rotates interleaved pairs: the conversion permutes the q / k output
    rows, and with them the rows of the q / k ``lora_B`` factors."""
    import transformers as T
    from opaque_b200 import patches
    torch.manual_seed(0)
    common = dict(vocab_size=320, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                  num_key_value_heads=2, max_position_embeddings=64)
    if family == "qwen2":
        hf = T.Qwen2ForCausalLM(T.Qwen2Config(**common)).eval()
        targets = ("q_proj", "k_proj", "v_proj")
    elif family == "cohere":
        hf = T.CohereForCausalLM(T.CohereConfig(**common, pad_token_id=0)).eval()
        targets = ("q_proj", "k_proj")
    elif family == "llama":
        hf = T.LlamaForCausalLM(T.LlamaConfig(**common)).eval()
        targets = ("q_proj", "k_proj", "v_proj", "o_proj")
    else:
        hf = T.LlamaForCausalLM(T.LlamaConfig(**common)).eval()
        targets = ("o_proj", "down_proj")
    wrapped = _fake_peft_wrap(hf, 4, 8.0, targets, rslora=rslora)
    ids = torch.randint(0, 320, (2, 16))
    with torch.no_grad():
        want = wrapped(ids).logits
    ours = patches.apply_model_patches(wrapped, dtype=torch.float32).eval()
    with torch.no_grad():
        got = ours(ids)[..., :320]
    assert float((got - want).norm() / want.norm()) < 1e-4
    trainable = sorted({n.split(".")[-1] for n, p in ours.named_parameters() if p.requires_grad})
    assert trainable == ["lora_A", "lora_B"]
    n_adapters = sum(1 for n, p in ours.named_parameters() if n.endswith("lora_A"))
    assert n_adapters == 2 * len(targets)
    # the adapter-disabled model is the base model
    for m in wrapped.modules():
        if hasattr(m, "scaling") and isinstance(m.scaling, dict):
            m.scaling = {k: 0.0 for k in m.scaling}
    from opaque_b200.models import layers
    with torch.no_grad(), layers.adapters_disabled():
        base = ours(ids)[..., :320]
        assert float((base - wrapped(ids).logits).norm() / want.norm()) < 1e-4


def test_peft_options_without_a_counterpart_are_refused():
    import transformers as T
    from opaque_b200 import patches
    hf = T.LlamaForCausalLM(T.LlamaConfig(vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=1,
                                          num_attention_heads=2, num_key_value_heads=2))
    wrapped = _fake_peft_wrap(hf, 2, 4.0, ("q_proj",))
    wrapped.peft_config["default"].use_dora = True
    with pytest.raises(NotImplementedError, match="DoRA"):
        patches.apply_model_patches(wrapped)
    wrapped.peft_config["default"].use_dora = False
    wrapped.peft_config["default"].lora_dropout = 0.1
    with pytest.raises(NotImplementedError, match="dropout"):
        patches.convert_peft_model(wrapped)
    with pytest.raises(ValueError, match="adapter"):
        wrapped.peft_config["default"].lora_dropout = 0.0
        patches.convert_peft_model(wrapped, adapter_name="other")


@pytest.mark.parametrize("family", ["llama", "cohere"])
def test_peft_adapter_files_round_trip(family, tmp_path):
    """Export writes the adapter under the PEFT library's names and row order (equal, tensor by tensor, to what the wrapped
    Hugging Face model holds); loading those files into a freshly converted base model reproduces the logits."""
    import json
    import transformers as T
    from opaque_b200 import patches
    torch.manual_seed(1)
    common = dict(vocab_size=320, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                  num_key_value_heads=2, max_position_embeddings=64)
    cls, cfg = ((T.CohereForCausalLM, T.CohereConfig(**common, pad_token_id=0)) if family == "cohere"
                else (T.LlamaForCausalLM, T.LlamaConfig(**common)))
    hf = cls(cfg).eval()
    base_sd = {k: v.clone() for k, v in hf.state_dict().items()}
    wrapped = _fake_peft_wrap(hf, 4, 8.0, ("q_proj", "k_proj", "v_proj"))
    ours = patches.apply_model_patches(wrapped, dtype=torch.float32).eval()
    out = patches.export_peft_adapter(ours, str(tmp_path / "adapter"), base_model_name_or_path="tiny")
    saved = patches.peft_adapter_state_dict(ours)
    theirs = {"base_model.model." + k.replace(".default.", "."): v for k, v in hf.state_dict().items() if ".lora_" in k}
    assert sorted(saved) == sorted(theirs)
    for k in saved:
        assert torch.allclose(saved[k], theirs[k]), k
    cfg_json = json.load(open(tmp_path / "adapter" / "adapter_config.json"))
    assert cfg_json["r"] == 4 and cfg_json["lora_alpha"] == 8.0 and cfg_json["target_modules"] == ["k_proj", "q_proj", "v_proj"]
    fresh_hf = cls(cfg).eval()
    fresh_hf.load_state_dict(base_sd)
    fresh = patches.apply_model_patches(fresh_hf, dtype=torch.float32).eval()
    patches.load_peft_adapter(fresh, out)
    ids = torch.randint(0, 320, (2, 16))
    with torch.no_grad():
        assert torch.allclose(fresh(ids), ours(ids), atol=1e-5)
        assert float((fresh(ids)[..., :320] - wrapped(ids).logits).abs().max()) < 1e-3
