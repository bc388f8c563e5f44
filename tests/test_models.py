"""Model families on CPU: per-example losses, LoRA math, MoE expert path vs a dense loop, vmap compatibility."""
import torch

from opaque_b200.dpsgd import clipped_grad
from opaque_b200.functional import make_functional
from opaque_b200.models import (GPT2Config, GPT2LMHeadModel, LlamaConfig, LlamaForCausalLM, MoEConfig, MoEForCausalLM,
                                shift_labels)


def _ref_losses(model, ids, labels):
    logits = model(ids)
    return torch.stack([torch.nn.functional.cross_entropy(logits[i].float(), labels[i], ignore_index=-100) for i in range(len(ids))])


def test_llama_per_example_loss_and_lora_gradients():
    torch.manual_seed(0)
    m = LlamaForCausalLM(LlamaConfig.tiny(), dtype=torch.float32)
    m.add_lora(4, 8.0)
    with torch.no_grad():
        for n, p in m.named_parameters():
            if "lora_B" in n:
                p.normal_(0, 0.1)
    ids = torch.randint(0, 256, (3, 16))
    lab = shift_labels(ids, 0.5)
    loss = m.per_example_loss(ids, lab)
    assert torch.allclose(loss, _ref_losses(m, ids, lab), atol=1e-5)
    assert (lab[:, :8] == -100).all() and (lab[:, -1] == -100).all()
    trainable = [n for n, p in m.named_parameters() if p.requires_grad]
    assert trainable and all("lora_" in n for n in trainable)
    loss.sum().backward()
    lin = m.model.layers[0].self_attn.q_proj
    g_a = lin.lora_A.grad.clone()
    # finite-difference check of one LoRA coordinate
    eps = 1e-3
    with torch.no_grad():
        lin.lora_A[0, 0] += eps
        up = m.per_example_loss(ids, lab).sum()
        lin.lora_A[0, 0] -= 2 * eps
        dn = m.per_example_loss(ids, lab).sum()
        lin.lora_A[0, 0] += eps
    assert abs(float((up - dn) / (2 * eps)) - float(g_a[0, 0])) < 1e-3


def test_gpt2_tied_head_and_padding():
    torch.manual_seed(1)
    g = GPT2LMHeadModel(GPT2Config.tiny(), dtype=torch.float32)
    assert g.wte.weight.shape[0] == 512 and g.config.vocab_size == 500
    ids = torch.randint(0, 500, (2, 16))
    lab = shift_labels(ids)
    loss = g.per_example_loss(ids, lab)
    assert torch.allclose(loss, _ref_losses(g, ids, lab), atol=1e-5)
    loss.sum().backward()
    ref = GPT2LMHeadModel(GPT2Config.tiny(), dtype=torch.float32)
    ref.load_state_dict(g.state_dict())
    _ref_losses(ref, ids, lab).sum().backward()
    assert torch.allclose(g.wte.weight.grad, ref.wte.weight.grad, atol=1e-5)      # embedding + head contributions


def test_moe_expert_path_matches_dense_loop_forward_and_backward():
    torch.manual_seed(2)
    cfg = MoEConfig.tiny()
    m = MoEForCausalLM(cfg, dtype=torch.float32)
    blk = m.layers[0].mlp
    x = torch.randn(2, 16, cfg.hidden_size, requires_grad=True)
    y = blk(x)

    def dense(xx):
        probs = torch.softmax(blk.gate(xx).float()[..., :cfg.num_experts], -1)
        w, idx = torch.topk(probs, cfg.num_experts_per_tok, -1)
        out = torch.zeros_like(xx)
        I = cfg.moe_intermediate_size
        for e in range(cfg.num_experts):
            h = xx @ blk.experts.gate_up_proj[e].t()
            ye = (torch.nn.functional.silu(h[..., :I]) * h[..., I:]) @ blk.experts.down_proj[e].t()
            out = out + ye * (w * (idx == e)).sum(-1, keepdim=True)
        return out + blk.shared_expert(xx)
    x2 = x.detach().clone().requires_grad_(True)
    y2 = dense(x2)
    assert torch.allclose(y, y2, atol=1e-5)
    go = torch.randn_like(y)
    params = [blk.experts.gate_up_proj, blk.experts.down_proj, blk.gate.weight]
    g1 = torch.autograd.grad(y, [x, *params], go)
    g2 = torch.autograd.grad(y2, [x2, *params], go)
    for a, b in zip(g1, g2):
        assert torch.allclose(a, b, atol=1e-4)
    ids = torch.randint(0, 512, (2, 16))
    assert torch.allclose(m.per_example_loss(ids, shift_labels(ids)), _ref_losses(m, ids, shift_labels(ids)), atol=1e-5)


def test_models_work_under_the_vmap_reference_engine():
    torch.manual_seed(3)
    m = LlamaForCausalLM(LlamaConfig.tiny(), dtype=torch.float32)
    m.add_lora(2, 4.0)
    fmodel, trainable, frozen = make_functional(m, disable_autograd_tracking=True, partition_trainable=True)

    def loss(tr, ids, lab):
        logits = fmodel({**frozen, **tr}, ids.unsqueeze(0))
        return torch.nn.functional.cross_entropy(logits[0], lab, ignore_index=-100)
    ids = torch.randint(0, 256, (4, 12))
    lab = shift_labels(ids)
    fn, st = clipped_grad(loss, clipping_norm=1.0, batch_argnums=(1, 2), return_aux=True)
    (g, aux), _ = fn(trainable, ids, lab)
    assert aux.batch_size == 4 and torch.allclose(aux.loss_values, _ref_losses(m, ids, lab), atol=1e-5)
    assert all(torch.isfinite(v).all() for v in g.pytree.values())


def test_moe_dense_reference_form_matches_the_sorted_form():
    """``plain_torch_ops()`` switches the experts to the vmap-safe dense evaluation: same loss, same gradients."""
    import torch
    from opaque_b200.models import MoEConfig, MoEForCausalLM, shift_labels
    from opaque_b200.ops.functional import plain_torch_ops
    torch.manual_seed(0)
    m = MoEForCausalLM(MoEConfig.tiny(), dtype=torch.float32)
    ids = torch.randint(0, 500, (3, 32))
    labels = shift_labels(ids, 1.0)
    m.per_example_loss(ids, labels).sum().backward()
    sorted_loss = m.per_example_loss(ids, labels).detach()
    sorted_grads = {n: p.grad.clone() for n, p in m.named_parameters() if p.grad is not None}
    m.zero_grad(set_to_none=True)
    with plain_torch_ops():
        dense = m.per_example_loss(ids, labels)
        dense.sum().backward()
    assert torch.allclose(dense.detach(), sorted_loss, atol=1e-5)
    for n, g in sorted_grads.items():
        assert torch.allclose(dict(m.named_parameters())[n].grad, g, atol=1e-5, rtol=1e-4), n
