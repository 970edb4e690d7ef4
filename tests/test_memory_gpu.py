"""Activation swap to pinned host memory: gradients must be identical with and without it."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _model():
    import torch.nn.functional as F
    from mindspeed_b200.config import TransformerConfig
    from mindspeed_b200.models import GPTModel
    cfg = TransformerConfig(num_layers=3, hidden_size=512, num_attention_heads=4, num_query_groups=2, ffn_hidden_size=1024,
                            gated_linear_unit=True, activation_func=F.silu, add_bias_linear=False, normalization="RMSNorm",
                            params_dtype=torch.bfloat16, bf16=True, optimization_level=1, use_flash_attn=True,
                            hidden_dropout=0.0, attention_dropout=0.0)
    torch.manual_seed(0)
    return GPTModel(cfg, vocab_size=1024, max_sequence_length=1024, position_embedding_type="rope").cuda()


def test_swap_attention_grads_match():
    from mindspeed_b200.memory.swap_attention import SwapManager, install_swap_attention
    m = _model()
    tok = torch.randint(0, 1024, (1, 1024), device="cuda")
    lab = torch.randint(0, 1024, (1, 1024), device="cuda")
    pos = torch.arange(1024, device="cuda").unsqueeze(0)
    m(tok, pos, None, labels=lab).mean().backward()
    ref = {n: p.grad.clone() for n, p in m.named_parameters()}
    m.zero_grad()
    mgr = install_swap_attention([m], None, "self_attention,mlp", SwapManager(min_bytes=1 << 16))
    m(tok, pos, None, labels=lab).mean().backward()
    torch.cuda.synchronize()
    assert mgr.bytes_swapped > 0
    for n, p in m.named_parameters():
        torch.testing.assert_close(p.grad, ref[n], atol=0, rtol=0, msg=n)
