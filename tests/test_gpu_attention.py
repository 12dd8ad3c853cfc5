"""The in-tree attention kernels against the plain fp32 formula."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _qkv(b, h, s, d, seed, layout):
    g = torch.Generator(device="cuda").manual_seed(seed)
    if layout == "interleaved":          # [B * S, H * 3 * D], per-head [q | k | v] (GPT-NeoX)
        qkv = torch.randn(b * s, h * 3 * d, device="cuda", generator=g).bfloat16()
        return tuple(t.transpose(1, 2) for t in qkv.view(b, s, h, 3 * d).split(d, dim=-1))
    if layout == "blocked":              # [B * S, 3 * H * D], [Q | K | V] (GPT-2, BERT)
        qkv = torch.randn(b * s, 3 * h * d, device="cuda", generator=g).bfloat16()
        return tuple(t.view(b, s, h, d).transpose(1, 2) for t in qkv.split(h * d, dim=-1))
    return tuple(torch.randn(b, h, s, d, device="cuda", generator=g).bfloat16() for _ in range(3))     # [B, H, S, D] dense


@pytest.mark.parametrize("b,h,s,d,causal,layout", [
    (2, 4, 256, 128, True, "interleaved"),
    (1, 3, 384, 64, True, "blocked"),
    (2, 2, 200, 64, False, "dense"),          # ragged last tile
    (1, 2, 72, 128, True, "dense"),           # less than one tile
    (2, 16, 1024, 128, True, "interleaved"),
    (1, 20, 1024, 64, True, "blocked"),
    (3, 2, 130, 64, True, "interleaved"),     # a batch boundary inside a key tile: rows of the next entry must be masked
])
def test_flash_forward_matches_the_formula(b, h, s, d, causal, layout):
    from stacr_b200.ops import _lib, attention

    q, k, v = _qkv(b, h, s, d, 7 * s + d, layout)
    out, lse = attention.forward(q, k, v, causal=causal)
    torch.cuda.synchronize()
    _lib.check_status()
    ref = attention.reference(q, k, v, causal=causal)
    assert out.shape == ref.shape
    assert float((out.float() - ref).abs().max()) < 2e-2, float((out.float() - ref).abs().max())
    scores = (q.float() @ k.float().transpose(-1, -2)) / d ** 0.5
    if causal:
        scores = scores.masked_fill(~torch.ones(s, s, dtype=torch.bool, device="cuda").tril(), float("-inf"))
    torch.testing.assert_close(lse, torch.logsumexp(scores, dim=-1), rtol=1e-3, atol=2e-3)


def test_flash_forward_with_padding_keys_and_large_scores():
    from stacr_b200.ops import _lib, attention

    b, h, s, d = 2, 4, 320, 64
    q, k, v = _qkv(b, h, s, d, 3, "dense")
    q = q * 6.0                                       # scores of a few tens: the lazy rescale of the accumulator is exercised
    keep = torch.ones(b, s, dtype=torch.bool, device="cuda")
    keep[0, 250:] = False
    keep[1, :5] = False
    for causal in (False, True):
        out, _ = attention.forward(q, k, v, causal=causal, key_mask=keep)
        torch.cuda.synchronize()
        _lib.check_status()
        ref = attention.reference(q, k, v, causal=causal, key_mask=keep)
        assert bool(torch.isfinite(out.float()).all())
        assert float((out.float() - ref).abs().max()) < 3e-2


def test_model_attention_uses_the_in_tree_kernel_without_grad(monkeypatch):
    """``STACR_ATTENTION=intree``: evaluation goes through the tcgen05 forward and agrees with the default path."""
    from stacr_b200.models import GPTNeoXForCausalLM, NeoXConfig
    from stacr_b200.ops import _lib

    torch.manual_seed(5)
    cfg = NeoXConfig(vocab_size=512, hidden_size=256, num_hidden_layers=2, num_attention_heads=4, intermediate_size=512, max_position_embeddings=256)
    model = GPTNeoXForCausalLM(cfg).cuda().eval()
    ids = torch.randint(0, 512, (2, 200), device="cuda")
    with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
        ref = model(input_ids=ids).logits.float()
        monkeypatch.setenv("STACR_ATTENTION", "intree")
        got = model(input_ids=ids).logits.float()
    torch.cuda.synchronize()
    _lib.check_status()
    assert float((got - ref).abs().max()) < 0.1 * float(ref.abs().max())
    assert float(torch.nn.functional.cosine_similarity(got.flatten(), ref.flatten(), dim=0)) > 0.999


@pytest.mark.parametrize("b,h,s,causal,layout", [
    (2, 4, 256, True, "interleaved"),
    (1, 3, 200, True, "blocked"),            # ragged: the last key tile and the last query tile are partial
    (2, 2, 130, False, "interleaved"),
    (1, 2, 72, True, "blocked"),
    (2, 16, 1024, True, "interleaved"),
])
def test_flash_backward_matches_autograd_of_the_formula(b, h, s, causal, layout):
    """dq, dk, dv of the in-tree backward (written into one fused gradient matrix) against autograd through the fp32 formula."""
    from stacr_b200.ops import _lib, attention

    d = 128
    g = torch.Generator(device="cuda").manual_seed(11 * s + h)
    qkv = (0.5 * torch.randn(b * s, 3 * h * d, device="cuda", generator=g)).bfloat16().requires_grad_(True)
    up = torch.randn(b, s, h * d, device="cuda", generator=g).bfloat16()
    assert attention.fused_supported(qkv, d)
    out = attention.fused_qkv_attention(qkv, b, s, h, d, layout=layout, causal=causal)
    out.backward(up)
    torch.cuda.synchronize()
    _lib.check_status()
    ref_in = qkv.detach().float().requires_grad_(True)
    q, k, v = attention.qkv_views(ref_in, b, s, h, d, layout)
    ref = attention.reference(q, k, v, causal=causal)
    ref.backward(up.float())
    assert float((out.float() - ref).abs().max()) < 2e-2
    got, want = qkv.grad.float(), ref_in.grad
    scale = float(want.abs().max())
    assert bool(torch.isfinite(got).all())
    assert float((got - want).abs().max()) < 3e-2 * scale + 1e-3, (float((got - want).abs().max()), scale)
    cos = torch.nn.functional.cosine_similarity(got.flatten(), want.flatten(), dim=0)
    assert float(cos) > 0.999, float(cos)
