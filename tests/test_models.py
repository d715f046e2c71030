"""Forward / backward of the benchmark model families on tiny configurations (CPU)."""
import torch

from nangila.models import BertConfig, BertMLM, GPT2, GPT2Config, Llama, LlamaConfig, mask_tokens, resnet50, resnet_tiny


def _grads_finite(model):
    return all(p.grad is None or torch.isfinite(p.grad).all() for p in model.parameters())


def test_gpt2_tiny_learns_a_batch():
    torch.manual_seed(0)
    m = GPT2(GPT2Config.tiny())
    opt = torch.optim.AdamW(m.parameters(), lr=3e-3)
    tok = torch.randint(0, 1000, (4, 33))
    first = None
    for _ in range(8):
        loss = m(tok[:, :-1], tok[:, 1:])
        first = first if first is not None else loss.item()
        loss.backward()
        opt.step()
        opt.zero_grad()
    assert loss.item() < first and _grads_finite(m)


def test_bert_mlm_masks_and_trains():
    torch.manual_seed(0)
    cfg = BertConfig.tiny()
    m = BertMLM(cfg)
    ids = torch.randint(5, cfg.vocab_size, (4, 64))
    x, labels = mask_tokens(ids, cfg)
    frac = (labels != -100).float().mean().item()
    assert 0.05 < frac < 0.3
    assert torch.equal(x[labels == -100], ids[labels == -100])  # unselected positions are untouched
    loss = m(x, labels)
    loss.backward()
    assert torch.isfinite(loss) and _grads_finite(m)
    assert m(x).shape == (4, 64, cfg.padded_vocab)
    large = BertConfig.large()
    assert (large.n_layer, large.d_model, large.n_head, large.d_mlp, large.vocab_size) == (24, 1024, 16, 4096, 30522)


def test_resnet_shapes_and_parameter_count():
    m = resnet_tiny()
    loss = m(torch.randn(2, 3, 64, 64), torch.tensor([1, 2]))
    loss.backward()
    assert torch.isfinite(loss) and _grads_finite(m)
    assert abs(resnet50().num_params() - 25_557_032) == 0  # the standard ResNet-50 count


def test_llama_tiny_and_config():
    torch.manual_seed(0)
    m = Llama(LlamaConfig.tiny())
    idx = torch.randint(0, 1024, (2, 16))
    loss = m(idx, idx)
    loss.backward()
    assert torch.isfinite(loss) and _grads_finite(m)
    c = LlamaConfig.llama_1_3b()
    est = c.vocab_size * c.d_model * 2 + c.n_layer * (4 * c.d_model ** 2 + 3 * c.d_model * c.d_mlp)
    assert 1.3e9 < est < 1.4e9
    # rotary embedding keeps norms
    from nangila.models.llama import apply_rope, rope_table

    x = torch.randn(1, 8, 2, 16)
    y = apply_rope(x, rope_table(8, 16, 10000.0, x.device))
    assert torch.allclose(x.norm(dim=-1), y.norm(dim=-1), atol=1e-5)
