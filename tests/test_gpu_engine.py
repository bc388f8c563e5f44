"""Fused DP engine vs a per-example autograd loop on tiny models; smoke of a full DP step (B200)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _oracle(model, ids, labels, C, guard):
    total = {n: torch.zeros_like(p, dtype=torch.float32) for n, p in model.named_parameters() if p.requires_grad}
    norms = []
    for i in range(ids.shape[0]):
        model.zero_grad(set_to_none=True)
        model.per_example_loss(ids[i:i + 1], labels[i:i + 1]).sum().backward()
        g = {n: p.grad.float() for n, p in model.named_parameters() if p.requires_grad}
        nrm = torch.sqrt(sum((v ** 2).sum() for v in g.values()))
        norms.append(nrm)
        c = min(1.0, C / float(nrm)) * guard
        for n in total:
            total[n] += c * g[n]
    model.zero_grad(set_to_none=True)
    return total, torch.stack(norms)


def _check(model, vocab, frac, C, tol_norm, tol_grad):
    from opaque_b200.engine.fused import CLIP_GUARD, FusedDPEngine
    from opaque_b200.models import shift_labels
    from opaque_b200.random import key
    dev = next(model.parameters()).device
    ids = torch.randint(0, vocab, (6, 128), device=dev)
    labels = shift_labels(ids, frac)
    total, norms = _oracle(model, ids, labels, C, CLIP_GUARD)
    eng = FusedDPEngine(model, clipping_norm=C, noise_multiplier=0.0, normalize_by=1.0, key=key(0), microbatch_size=4)
    res = eng.accumulate(model.per_example_loss, {"input_ids": ids, "labels": labels})
    torch.cuda.synchronize()
    assert eng.status.read() == 0
    assert float(((res.norms - norms).abs() / norms).max()) < tol_norm
    flat = eng.space.grad.local
    for n, g in total.items():
        s = eng.space.slots[n]
        got = flat[s.offset:s.offset + s.numel].view(s.shape)
        assert float((got - g).norm() / (g.norm() + 1e-12)) < tol_grad, n
    # clipped sum respects the sensitivity bound per example (here: total <= B*C trivially, and scales <= 1)
    eng.noise_multiplier, eng.normalize_by = 0.5, 6.0
    before = eng.space.params.local.float().clone()
    out = eng.step(model.per_example_loss, {"input_ids": ids, "labels": labels})
    assert math.isfinite(out.loss) and float((eng.space.params.local.float() - before).abs().max()) > 0
    assert float(eng.space.grad.local.abs().max()) == 0          # consumed and zeroed by the shard step
    return eng


def test_llama_lora_matches_per_example_loop():
    from opaque_b200.models import LlamaConfig, LlamaForCausalLM
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    m = LlamaForCausalLM(LlamaConfig.tiny(), device=dev)
    m.add_lora(16, 32.0)
    with torch.no_grad():
        for n, p in m.named_parameters():
            if "lora_B" in n:
                p.normal_(0, 0.05)
    _check(m, 256, 0.5, 0.05, 1e-3, 1e-2)


def test_llama_full_parameter_untied_and_tied():
    from opaque_b200.models import LlamaConfig, LlamaForCausalLM
    dev = torch.device("cuda", 0)
    torch.manual_seed(1)
    cfg = LlamaConfig(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=256)
    _check(LlamaForCausalLM(cfg, device=dev), 512, 1.0, 1.0, 5e-3, 2e-2)
    cfg.tie_word_embeddings = True
    _check(LlamaForCausalLM(cfg, device=dev), 512, 1.0, 1.0, 5e-3, 2e-2)


@pytest.mark.parametrize("variant", [dict(attention_bias=True), dict(qk_norm=True, head_dim=32),
                                     dict(hidden_act="gelu_pytorch_tanh", norm_offset=1.0, norm_casting="gemma", embedding_scale=128 ** 0.5),
                                     dict(post_norm=True, qk_norm_full=True), dict(residual_multiplier=0.5, attention_multiplier=0.2, logits_scaling=2.0),
                                     dict(sandwich_norm=True, attn_logit_softcap=50.0, final_logit_softcap=30.0, layer_windows=(64, None),
                                          hidden_act="gelu_pytorch_tanh", norm_offset=1.0, norm_casting="gemma"),
                                     dict(post_norm=True, qk_norm=True, head_dim=32, layer_windows=(64, None), no_rope_layers=(1, 0)),
                                     dict(sandwich_norm=True, qk_norm=True, head_dim=32, layer_windows=(64, None), local_rope_theta=10000.0,
                                          rope_scaling={"rope_type": "linear", "factor": 8.0}),
                                     dict(norm_type="layernorm", parallel_block=True, logits_scaling=4.0),
                                     dict(sandwich_norm=True, partial_rotary_factor=0.5, attention_bias=True)])
def test_llama_family_variants_full_parameter(variant):
    """Qwen2 biases, Qwen3 q/k norms, Gemma GeGLU / (1+w) norms / scaled embeddings, OLMo-2 post-norm, Granite multipliers,
    Gemma-2 capping and sandwich norms with a windowed layer, EXAONE-4 hybrid layers, Gemma-3 local rotary base,
    Cohere parallel block with bias-free LayerNorm, GLM-4 partial rotary embedding."""
    from opaque_b200.models import LlamaConfig, LlamaForCausalLM
    dev = torch.device("cuda", 0)
    torch.manual_seed(7)
    cfg = LlamaConfig(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, max_position_embeddings=256, **variant)
    m = LlamaForCausalLM(cfg, device=dev)
    with torch.no_grad():
        for n, p in m.named_parameters():
            if n.endswith(".bias"):
                p.normal_(0, 0.02)
    _check(m, 512, 1.0, 1.0, 1e-2, 3e-2)


def test_gpt2_full_parameter():
    from opaque_b200.models import GPT2Config, GPT2LMHeadModel
    dev = torch.device("cuda", 0)
    torch.manual_seed(2)
    _check(GPT2LMHeadModel(GPT2Config.tiny(), device=dev), 500, 1.0, 1.0, 5e-3, 2e-2)


def test_moe_full_parameter_ragged_ghost_and_grouped_wgrad():
    from opaque_b200.models import MoEConfig, MoEForCausalLM
    dev = torch.device("cuda", 0)
    torch.manual_seed(3)
    _check(MoEForCausalLM(MoEConfig.tiny(), device=dev), 512, 1.0, 1.0, 1e-2, 3e-2)


def test_per_group_and_adaptive_clipping_in_the_fused_engine():
    from opaque_b200.dpsgd.clipping import AdaptiveClipState, next_clipping_norm
    from opaque_b200.engine.fused import CLIP_GUARD, FusedDPEngine
    from opaque_b200.models import LlamaConfig, LlamaForCausalLM, shift_labels
    from opaque_b200.random import fold_in, generator_from_key, key
    dev = torch.device("cuda", 0)
    torch.manual_seed(4)
    cfg = LlamaConfig(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=256)
    m = LlamaForCausalLM(cfg, device=dev)
    ids = torch.randint(0, 512, (5, 128), device=dev)
    labels = shift_labels(ids, 1.0)
    bounds = {"mlp": 0.3, "norm": 0.05, "fallback": 0.7}
    group_of = lambda n: next((p for p in ("mlp", "norm") if p in n), "fallback")
    eng = FusedDPEngine(m, clipping_norm=bounds, group_of=group_of, noise_multiplier=0.0, normalize_by=1.0, key=key(0),
                        microbatch_size=3)
    assert abs(eng.sensitivity() - math.sqrt(0.3 ** 2 + 0.05 ** 2 + 0.7 ** 2)) < 1e-12
    total = {n: torch.zeros_like(p, dtype=torch.float32) for n, p in m.named_parameters()}
    gn = {g: [] for g in bounds}
    for i in range(5):
        m.zero_grad(set_to_none=True)
        m.per_example_loss(ids[i:i + 1], labels[i:i + 1]).sum().backward()
        grads = {n: p.grad.float() for n, p in m.named_parameters()}
        for g, C in bounds.items():
            nrm = torch.sqrt(sum((v ** 2).sum() for n, v in grads.items() if group_of(n) == g))
            gn[g].append(nrm)
            c = min(1.0, C / float(nrm)) * CLIP_GUARD
            for n, v in grads.items():
                if group_of(n) == g:
                    total[n] += c * v
    m.zero_grad(set_to_none=True)
    res = eng.accumulate(m.per_example_loss, {"input_ids": ids, "labels": labels})
    torch.cuda.synchronize()
    assert eng.status.read() == 0
    for g in bounds:
        want = torch.stack(gn[g])
        assert float(((res.group_norms[g] - want).abs() / want).max()) < 5e-3, g
    flat = eng.space.grad.local
    for n, gref in total.items():
        s_ = eng.space.slots[n]
        got = flat[s_.offset:s_.offset + s_.numel].view(s_.shape)
        assert float((got - gref).norm() / (gref.norm() + 1e-12)) < 2e-2, n

    # adaptive: the threshold follows the geometric quantile update with the state's own noise draw
    m2 = LlamaForCausalLM(cfg, device=dev)
    st = AdaptiveClipState(0.5, 0, 0.5, 0.2, 0.01, 100.0, 0.05, key(9))
    eng2 = FusedDPEngine(m2, clipping_norm=123.0, noise_multiplier=0.5, normalize_by=5.0, key=key(1), microbatch_size=5,
                         adaptive=st)
    assert eng2.clipping_norm == 0.5
    out = eng2.step(m2.per_example_loss, {"input_ids": ids, "labels": labels})
    rate = float((out.norms > 0.5).float().mean())
    z = float(torch.randn(1, generator=generator_from_key(fold_in(key(9), 0))))
    assert abs(eng2.clipping_norm - next_clipping_norm(0.5, rate, z, st)) < 1e-9 and eng2.adaptive.step == 1


def test_cuda_graph_microbatches_match_eager_execution():
    from opaque_b200.engine.fused import FusedDPEngine
    from opaque_b200.models import GPT2Config, GPT2LMHeadModel, shift_labels
    from opaque_b200.random import key
    dev = torch.device("cuda", 0)
    ids = torch.randint(0, 500, (11, 128), device=dev)          # 3 microbatches of 4: eager, captured, replayed (partial)
    labels = shift_labels(ids, 1.0)
    flats, norms = [], []
    for graph in (False, True):
        torch.manual_seed(6)
        m = GPT2LMHeadModel(GPT2Config.tiny(), device=dev)
        eng = FusedDPEngine(m, clipping_norm=1.0, noise_multiplier=0.0, normalize_by=1.0, key=key(0), microbatch_size=4,
                            cuda_graph=graph)
        for _ in range(2):                                       # second pass replays only
            eng.space.grad.local.zero_()
            res = eng.accumulate(m.per_example_loss, {"input_ids": ids, "labels": labels})
        torch.cuda.synchronize()
        assert eng.status.read() == 0
        flats.append(eng.space.grad.local.clone())
        norms.append(res.norms.clone())
    assert float((norms[0] - norms[1]).abs().max() / norms[0].max()) < 1e-4
    assert float((flats[0] - flats[1]).norm() / flats[0].norm()) < 1e-3     # atomics reorder sums, nothing else differs


def test_noise_is_added_exactly_once_and_matches_sigma():
    from opaque_b200.engine.fused import FusedDPEngine
    from opaque_b200.models import LlamaConfig, LlamaForCausalLM
    from opaque_b200.random import fold_in, key
    from opaque_b200 import ops
    dev = torch.device("cuda", 0)
    m = LlamaForCausalLM(LlamaConfig.tiny(), device=dev)
    m.add_lora(16, 32.0)
    eng = FusedDPEngine(m, clipping_norm=2.0, noise_multiplier=1.5, normalize_by=4.0, key=key(5), microbatch_size=4)
    noisy = torch.zeros(eng.space.shard, device=dev)
    eng.opt.step(noise_std=3.0, normalize_by=4.0, noisy_out=noisy, skip_update=True)      # empty batch: noise only
    ref = torch.zeros(eng.space.shard, device=dev)
    ops.philox_normal_add_(ref, seed=fold_in(key(5), 0).seed, offset=0, std=0.75)
    assert torch.equal(noisy, ref) and abs(float(noisy.std()) - 0.75) < 0.01


def test_smoke_entry_point():
    import __graft_entry__ as g
    g.smoke()


def test_cuda_graph_microbatches_match_eager_execution_moe():
    """The MoE microbatch (routing sort, grouped GEMMs, ragged ghost norms, grouped clip-weighted GEMM) has static
    shapes and no host synchronisation, so it replays as one graph too.  Kept last in the file: a failed capture would
    leave the process's RNG offset bookkeeping unusable for later captures."""
    from opaque_b200.engine.fused import FusedDPEngine
    from opaque_b200.models import MoEConfig, MoEForCausalLM, shift_labels
    from opaque_b200.random import key
    dev = torch.device("cuda", 0)
    ids = torch.randint(0, 500, (7, 128), device=dev)           # microbatches of 4 and 3 (padded to a graphed size)
    labels = shift_labels(ids, 1.0)
    flats, norms = [], []
    for graph in (False, True):
        torch.manual_seed(8)
        m = MoEForCausalLM(MoEConfig.tiny(), device=dev)
        eng = FusedDPEngine(m, clipping_norm=1.0, noise_multiplier=0.0, normalize_by=1.0, key=key(0), microbatch_size=4,
                            cuda_graph=graph)
        for _ in range(2):
            eng.space.grad.local.zero_()
            res = eng.accumulate(m.per_example_loss, {"input_ids": ids, "labels": labels})
        torch.cuda.synchronize()
        assert eng.status.read() == 0
        flats.append(eng.space.grad.local.clone())
        norms.append(res.norms.clone())
    assert float((norms[0] - norms[1]).abs().max() / norms[0].max()) < 1e-3
    assert float((flats[0] - flats[1]).norm() / flats[0].norm()) < 2e-3


def test_trainable_parameter_outside_the_dp_layers_is_refused():
    """A plain ``nn.Parameter`` used through an ordinary op gets a summed, unclipped gradient from autograd: refused."""
    from opaque_b200.engine.fused import FusedDPEngine
    from opaque_b200.models import LlamaConfig, LlamaForCausalLM, shift_labels
    from opaque_b200.random import key
    dev = torch.device("cuda", 0)

    class WithStray(LlamaForCausalLM):
        def __init__(self, cfg, **kw):
            super().__init__(cfg, **kw)
            self.stray_scale = torch.nn.Parameter(torch.ones(cfg.hidden_size, device=kw.get("device"), dtype=torch.bfloat16))

        def hidden_states(self, input_ids, position_ids=None):
            return super().hidden_states(input_ids, position_ids) * self.stray_scale

    m = WithStray(LlamaConfig.tiny(), device=dev)
    eng = FusedDPEngine(m, clipping_norm=1.0, noise_multiplier=0.0, normalize_by=1.0, key=key(0), microbatch_size=4)
    ids = torch.randint(0, 256, (4, 64), device=dev)
    with pytest.raises(RuntimeError, match="stray_scale"):
        eng.accumulate(m.per_example_loss, {"input_ids": ids, "labels": shift_labels(ids, 1.0)})


@pytest.mark.parametrize("act,bias", [("gpt_oss", True), ("swiglu", True)])
def test_frozen_biased_experts_run_on_the_grouped_gemm_and_match_the_dense_form(act, bias):
    """GPT-OSS style experts (bias rows, clamped activation) that are frozen take the sorted grouped-GEMM path; outputs
    and the gradients reaching tokens and routing weights equal the dense every-expert-for-every-token form."""
    from opaque_b200.models.moe import MoEConfig, MoEExperts
    from opaque_b200.ops import lib
    torch.manual_seed(3)
    cfg = MoEConfig(vocab_size=64, hidden_size=128, num_hidden_layers=1, num_attention_heads=4, num_key_value_heads=4,
                    num_experts=6, moe_intermediate_size=64, num_shared_experts=0, num_experts_per_tok=2,
                    max_position_embeddings=64, expert_act=act, expert_bias=bias)
    ex = MoEExperts(cfg, torch.bfloat16, "cuda")
    with torch.no_grad():
        if bias:
            ex.gate_up_bias.normal_(0, 0.5)
            ex.down_bias.normal_(0, 0.5)
        ex.gate_up_proj.normal_(0, 0.1)
        ex.down_proj.normal_(0, 0.1)
    for p_ in ex.parameters():
        p_.requires_grad_(False)
    T = 96
    x = torch.randn(T, 128, device="cuda").bfloat16()
    idx = torch.stack([torch.randperm(6, device="cuda")[:2] for _ in range(T)])
    w = torch.rand(T, 2, device="cuda").bfloat16()
    gy = torch.randn(T, 128, device="cuda").bfloat16()

    def run(fn):
        xx, ww = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
        y = fn(xx, ww)
        y.backward(gy)
        return y.detach().float(), xx.grad.float(), ww.grad.float()

    before = lib.LAUNCHES
    got = run(lambda xx, ww: ex(xx, idx, ww, 2, T // 2))
    assert lib.LAUNCHES > before, "the grouped path did not run"
    want = run(lambda xx, ww: ex._dense(xx, idx, ww))
    rel = lambda a, b: float((a - b).norm() / (b.norm() + 1e-30))
    assert rel(got[0], want[0]) < 2e-2 and rel(got[1], want[1]) < 3e-2 and rel(got[2], want[2]) < 3e-2


def test_direct_norm_path_gives_the_same_clipped_step_as_the_ghost_path():
    """Forcing every weight matrix through the direct norm kernel changes nothing but rounding: norms and the clipped
    gradient sum equal the Gram-matrix path's."""
    from opaque_b200.engine import fused
    from opaque_b200.models import GPT2Config, GPT2LMHeadModel
    from opaque_b200.random import key
    results = {}
    for path in ("ghost", "direct"):
        torch.manual_seed(11)
        cfg = GPT2Config(vocab_size=256, n_positions=128, n_embd=128, n_layer=2, n_head=4)
        model = GPT2LMHeadModel(cfg, dtype=torch.bfloat16, device="cuda")
        ids = torch.randint(0, 256, (4, 128), device="cuda")
        old, fused.NORM_PATH = fused.NORM_PATH, path
        try:
            eng = fused.FusedDPEngine(model, clipping_norm=0.5, noise_multiplier=0.0, normalize_by=1.0, key=key(0), microbatch_size=4)
            res = eng.accumulate(model.per_example_loss, {"input_ids": ids, "labels": ids})
            torch.cuda.synchronize()
            assert eng.status.read() == 0
        finally:
            fused.NORM_PATH = old
        results[path] = (res.norms.float().cpu().clone(), eng.space.grad.local.float().cpu().clone())
    (n_g, g_g), (n_d, g_d) = results["ghost"], results["direct"]
    assert torch.allclose(n_g, n_d, rtol=5e-3)
    assert float((g_g - g_d).norm() / (g_g.norm() + 1e-30)) < 1e-2
