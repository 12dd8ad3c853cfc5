"""LayerNorm / GELU / cross-entropy / optimizer kernels against fp32 PyTorch references."""

import pytest
import torch
from torch.nn import functional as F

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,n", [(64, 256), (1000, 768), (4096, 2048), (300, 4096), (77, 1280)])
def test_layernorm_forward_backward(rows, n):
    from stacr_b200.ops import nn_ops

    torch.manual_seed(rows + n)
    x = torch.randn(rows, n, device="cuda").bfloat16().requires_grad_(True)
    w = torch.randn(n, device="cuda").requires_grad_(True)
    b = torch.randn(n, device="cuda").requires_grad_(True)
    y = nn_ops.layer_norm(x, w, b, 1e-5)
    xr = x.detach().float().requires_grad_(True)
    wr, br = w.detach().clone().requires_grad_(True), b.detach().clone().requires_grad_(True)
    yr = F.layer_norm(xr, (n,), wr, br, 1e-5)
    torch.testing.assert_close(y.float(), yr, rtol=2e-2, atol=2e-2)
    g = torch.randn_like(yr)
    y.backward(g.bfloat16())
    yr.backward(g.bfloat16().float())
    torch.testing.assert_close(x.grad.float(), xr.grad, rtol=3e-2, atol=3e-2)
    torch.testing.assert_close(w.grad, wr.grad, rtol=2e-2, atol=rows ** 0.5 * 2e-2)
    torch.testing.assert_close(b.grad, br.grad, rtol=2e-2, atol=rows ** 0.5 * 2e-2)


@pytest.mark.parametrize("form", ["none", "tanh"])
def test_gelu_forward_backward(form):
    from stacr_b200.ops import nn_ops

    x = (3 * torch.randn(513, 1024, device="cuda")).bfloat16().requires_grad_(True)
    y = nn_ops.gelu(x, form)
    xr = x.detach().float().requires_grad_(True)
    yr = F.gelu(xr, approximate=form)
    torch.testing.assert_close(y.float(), yr, rtol=1e-2, atol=1e-2)
    g = torch.randn_like(yr).bfloat16()
    y.backward(g)
    yr.backward(g.float())
    torch.testing.assert_close(x.grad.float(), xr.grad, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("rows,n,form", [(513, 1024, "none"), (37, 4104, "tanh"), (3, 8, "none"), (4096, 2048, "none")])
def test_gelu_backward_leaves_the_column_sums_of_its_result(rows, n, form):
    """The fused derivative + column-sum kernel against fp32: the sums are those of the stored (bf16) result."""
    from stacr_b200.ops import nn_kernels

    x = (2 * torch.randn(rows, n, device="cuda")).bfloat16()
    dy = torch.randn(rows, n, device="cuda").bfloat16()
    dx, sums = nn_kernels.gelu_bwd_colsum(dy, x, form == "tanh")
    xr = x.float().requires_grad_(True)
    F.gelu(xr, approximate=form).backward(dy.float())
    torch.testing.assert_close(dx.float(), xr.grad, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(sums, dx.float().sum(0), rtol=1e-4, atol=1e-3 * max(1.0, rows ** 0.5))
    plain = nn_kernels.gelu_bwd(dy, x, form == "tanh")
    assert torch.equal(plain, dx)


def test_bias_gradient_of_a_linear_feeding_gelu_comes_from_the_activation_backward():
    """Linear -> GELU -> Linear: the first layer's bias gradient is the by-product of the activation's backward, and equals autograd's."""
    from stacr_b200.models.common import GELU, Linear
    from stacr_b200.ops import nn_ops, stacr_ops

    torch.manual_seed(0)
    a, act, b = Linear(256, 512).cuda(), GELU("none"), Linear(512, 256).cuda()
    x = torch.randn(4, 96, 256, device="cuda")
    calls = {"n": 0}
    real = stacr_ops.colsum

    def counting(t):
        calls["n"] += 1
        return real(t)

    stacr_ops.colsum = counting
    try:
        with torch.autocast("cuda", dtype=torch.bfloat16):
            y = b(act(a(x)))
        y.float().square().mean().backward()
    finally:
        stacr_ops.colsum = real
    assert calls["n"] == 1                      # only the last layer summed its gradient matrix itself
    ra, rb = torch.nn.Linear(256, 512).cuda(), torch.nn.Linear(512, 256).cuda()
    ra.load_state_dict(a.state_dict())
    rb.load_state_dict(b.state_dict())
    rb(F.gelu(ra(x))).square().mean().backward()
    for got, want in ((a.bias.grad, ra.bias.grad), (b.bias.grad, rb.bias.grad), (a.weight.grad, ra.weight.grad)):
        assert float((got - want).norm() / want.norm()) < 3e-2
    assert nn_ops.column_sums.offered is None


@pytest.mark.parametrize("rows,v", [(515, 50304), (252, 1024), (7, 8)])
def test_cross_entropy_loss_and_gradient(rows, v):
    """The small vocabularies leave most threads of a row's CTA without an element (their running max stays -inf)."""
    from stacr_b200.ops import nn_ops

    logits = (2 * torch.randn(rows, v, device="cuda")).bfloat16().requires_grad_(True)
    target = torch.randint(0, v, (rows,), device="cuda")
    target[::7] = -100
    loss = nn_ops.cross_entropy(logits, target)
    lr = logits.detach().float().requires_grad_(True)
    ref = F.cross_entropy(lr, target, ignore_index=-100)
    torch.testing.assert_close(loss, ref, rtol=1e-3, atol=1e-3)
    (loss * 3.0).backward()
    (ref * 3.0).backward()
    err = (logits.grad.float() - lr.grad).abs().max() / lr.grad.abs().max()
    assert err < 2e-2, float(err)
    assert logits.grad[0::7].abs().max() == 0


@pytest.mark.parametrize("eight_bit", [False, True])
def test_adamw_kernel_tracks_torch(eight_bit):
    from stacr_b200.optim import AdamW

    torch.manual_seed(3)
    shapes = [(1024, 512), (300,), (4097,), (64, 64)]
    mine = [torch.nn.Parameter(torch.randn(s, device="cuda")) for s in shapes]
    ref = [torch.nn.Parameter(p.detach().clone()) for p in mine]
    o1 = AdamW(mine, lr=1e-2, weight_decay=0.1, eight_bit=eight_bit)
    o2 = torch.optim.AdamW(ref, lr=1e-2, weight_decay=0.1)
    for _ in range(10):
        for a, b in zip(mine, ref):
            g = torch.randn_like(a)
            a.grad, b.grad = g.clone(), g.clone()
        o1.step()
        o2.step()
    tol = 5e-3 if eight_bit else 1e-5
    for a, b in zip(mine, ref):
        assert (a - b).abs().max() < tol * max(1.0, float(b.abs().max()))
    assert o1.kernel_launches == 10
    if eight_bit:
        big = o1.state[mine[0]]
        assert big["eight_bit"] and big["m8"].dtype == torch.uint8
        assert not o1.state[mine[1]]["eight_bit"]


def test_smoke_entry_point():
    import __graft_entry__ as entry

    entry.smoke()


def test_fused_rotary_matches_framework_ops():
    from stacr_b200.models.neox import apply_rotary, rotary_tables
    from stacr_b200.ops import nn_ops

    torch.manual_seed(5)
    b, s, h, hd, rot = 2, 96, 4, 64, 16
    qkv = torch.randn(b, s, h * 3 * hd, device="cuda").bfloat16()
    ref_in = qkv.detach().clone().float().requires_grad_(True)
    q, k, v = (t.transpose(1, 2) for t in ref_in.view(b, s, h, 3 * hd).split(hd, dim=-1))
    cos, sin = rotary_tables(s, rot, 10000.0, "cuda")
    ref = torch.cat([apply_rotary(q, cos, sin, rot).transpose(1, 2), apply_rotary(k, cos, sin, rot).transpose(1, 2), v.transpose(1, 2)], dim=-1)
    inv = 1.0 / (10000.0 ** (torch.arange(0, rot, 2, device="cuda", dtype=torch.float32) / rot))
    ang = torch.outer(torch.arange(s, device="cuda", dtype=torch.float32), inv)
    x = (qkv.clone() * 1.0).requires_grad_(True)
    y = x * 1.0  # non-leaf, so the in-place op is legal
    out = nn_ops.rotary_qk(y, ang.cos().contiguous(), ang.sin().contiguous(), s, h, hd, rot)
    torch.testing.assert_close(out.float().view(b, s, h, 3 * hd), ref, rtol=2e-2, atol=2e-2)
    g = torch.randn_like(ref)
    ref.backward(g)
    out.view(b, s, h, 3 * hd).backward(g.bfloat16())
    torch.testing.assert_close(x.grad.float().view(b, s, h, 3 * hd), ref_in.grad.view(b, s, h, 3 * hd), rtol=3e-2, atol=3e-2)


def test_padded_vocabulary_head_matches_fp32_reference():
    """Head + loss on a logits buffer padded from an odd vocabulary (GPT-2's 50257 in miniature), forward and backward."""
    from stacr_b200.ops import _lib, nn_ops

    torch.manual_seed(3)
    rows, d, v = 520, 256, 1003
    h = (torch.randn(rows, d, device="cuda") * 0.5).requires_grad_(True)
    w = (torch.randn(v, d, device="cuda") * 0.05).requires_grad_(True)
    t = torch.randint(0, v, (rows,), device="cuda")
    t[::7] = -100
    with torch.autocast("cuda", dtype=torch.bfloat16):
        loss = nn_ops.linear_cross_entropy(h, w, t)
    loss.backward()
    torch.cuda.synchronize()
    _lib.check_status()
    hr, wr = h.detach().clone().requires_grad_(True), w.detach().clone().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(hr @ wr.t(), t, ignore_index=-100)
    ref.backward()
    assert abs(float(loss) - float(ref)) < 2e-2
    assert float((h.grad - hr.grad).abs().max() / hr.grad.abs().max()) < 3e-2
    assert float((w.grad - wr.grad).abs().max() / wr.grad.abs().max()) < 3e-2
    # chunked evaluation gives the same mean
    with torch.autocast("cuda", dtype=torch.bfloat16):
        chunked = nn_ops.linear_cross_entropy(h.detach(), w.detach(), t, chunk=128)
    assert abs(float(chunked) - float(ref)) < 2e-2


def test_plain_linear_writes_fp32_weight_gradient_and_uses_a_lent_slot():
    from stacr_b200.models.common import Linear
    from stacr_b200.ops import _lib

    torch.manual_seed(5)
    lin = Linear(264, 520, device="cuda")
    ref = torch.nn.Linear(264, 520, device="cuda")
    ref.load_state_dict(lin.state_dict())
    x = torch.randn(3, 200, 264, device="cuda", requires_grad=True)
    xr = x.detach().clone().requires_grad_(True)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y = lin(x)
        yr = ref(xr)
    assert y.dtype == torch.bfloat16 and type(y.grad_fn).__name__ == "ViewBackward0"      # 3-D input: reshaped outside the function
    with torch.autocast("cuda", dtype=torch.bfloat16):
        assert type(lin(x.detach().reshape(-1, 264)).grad_fn).__name__.startswith("_LinearFn")
    torch.testing.assert_close(y.float(), yr.float(), rtol=2e-2, atol=2e-2)
    g = torch.randn_like(y)
    y.backward(g)
    yr.backward(g)
    torch.cuda.synchronize()
    _lib.check_status()
    assert lin.weight.grad.dtype == torch.float32
    exact = g.float().reshape(-1, 520).t() @ x.detach().reshape(-1, 264).bfloat16().float()
    assert float((lin.weight.grad - exact).abs().max() / exact.abs().max()) < 2e-3          # fp32 accumulation and output
    torch.testing.assert_close(lin.weight.grad, ref.weight.grad, rtol=3e-2, atol=3e-2 * float(exact.abs().max()))
    torch.testing.assert_close(lin.bias.grad, ref.bias.grad, rtol=2e-2, atol=0.5)
    torch.testing.assert_close(x.grad, xr.grad, rtol=3e-2, atol=3e-2)
    # a lent slot is written in place and becomes the gradient; a second backward accumulates into it
    lin.zero_grad(set_to_none=True)
    flat = torch.full((64 + lin.weight.numel() + 64,), -77.0, device="cuda")
    slot = flat[64:64 + lin.weight.numel()].view_as(lin.weight)
    lin.weight._sb_grad_out, lin.weight._sb_grad_fresh = slot, True
    lin.weight._sb_grad_ready = lambda: setattr(lin.weight, "grad", slot)       # what a gradient synchroniser installs
    with torch.autocast("cuda", dtype=torch.bfloat16):
        lin(x.detach()).backward(g)
    assert lin.weight.grad.data_ptr() == slot.data_ptr() and not lin.weight._sb_grad_fresh
    torch.testing.assert_close(slot, exact, rtol=2e-3, atol=2e-3 * float(exact.abs().max()))
    assert bool((flat[:64] == -77.0).all()) and bool((flat[-64:] == -77.0).all())
    with torch.autocast("cuda", dtype=torch.bfloat16):
        lin(x.detach()).backward(g)
    torch.testing.assert_close(lin.weight.grad, 2 * exact, rtol=2e-3, atol=4e-3 * float(exact.abs().max()))
    # fp32 inputs outside autocast and tiny heads keep the stock path
    assert "_LinearFn" not in type(lin(x.detach().reshape(-1, 264)).grad_fn).__name__


@pytest.mark.parametrize("rows,n", [(1000, 776), (4096, 2048), (37, 256)])
def test_parallel_block_norms_match_two_layer_norms_and_a_residual(rows, n):
    """(LN1(x), LN2(x), x) from one kernel, and one backward kernel for the three gradients that meet at x."""
    from stacr_b200.ops import _lib, nn_ops

    g = torch.Generator(device="cuda").manual_seed(rows + n)
    x = torch.randn(rows, n, device="cuda", generator=g).bfloat16().requires_grad_(True)
    params = [torch.randn(n, device="cuda", generator=g).requires_grad_(True) for _ in range(4)]
    up = [torch.randn(rows, n, device="cuda", generator=g).bfloat16() for _ in range(3)]
    assert nn_ops.parallel_norms_supported(x, *params)
    y1, y2, skip = nn_ops.parallel_layer_norms(x, *params, 1e-5)
    out = nn_ops.add3(skip * 1.0, y1, y2)
    (y1.float() * up[0].float()).sum().backward(retain_graph=True)
    (y2.float() * up[1].float()).sum().backward(retain_graph=True)
    (skip.float() * up[2].float()).sum().backward()
    torch.cuda.synchronize()
    _lib.check_status()
    got = [x.grad.float().clone()] + [p.grad.clone() for p in params]
    xr = x.detach().float().requires_grad_(True)
    pr = [p.detach().clone().requires_grad_(True) for p in params]
    r1 = torch.nn.functional.layer_norm(xr, (n,), pr[0], pr[1], 1e-5)
    r2 = torch.nn.functional.layer_norm(xr, (n,), pr[2], pr[3], 1e-5)
    ((r1 * up[0].float()).sum() + (r2 * up[1].float()).sum() + (xr * up[2].float()).sum()).backward()
    assert float((y1.float() - r1).abs().max()) < 5e-2 and float((y2.float() - r2).abs().max()) < 5e-2
    assert torch.equal(skip, x)
    torch.testing.assert_close(out.float(), (x.float() + y1.float() + y2.float()), rtol=2e-2, atol=5e-2)
    scale = float(xr.grad.abs().max())
    assert float((got[0] - xr.grad).abs().max()) < 2e-2 * scale + 2e-2
    for mine, ref in zip(got[1:], pr):
        torch.testing.assert_close(mine, ref.grad, rtol=2e-2, atol=2e-2 * float(ref.grad.abs().max()))


def test_neox_layer_with_fused_norms_matches_the_unfused_layer():
    from stacr_b200.models.neox import NeoXConfig, NeoXLayer

    torch.manual_seed(3)
    cfg = NeoXConfig(vocab_size=128, hidden_size=256, num_hidden_layers=1, num_attention_heads=4, intermediate_size=512, max_position_embeddings=64)
    layer = NeoXLayer(cfg).cuda().train()
    x = torch.randn(2, 64, 256, device="cuda").bfloat16()
    xa, xb = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        fused = layer(xa)
        handle = layer.input_layernorm.register_forward_hook(lambda m, i, o: None)     # a hooked norm keeps the module-by-module route
        plain = layer(xb)
        handle.remove()
    up = torch.randn_like(fused)
    fused.backward(up)
    grads_fused = {n: p.grad.clone() for n, p in layer.named_parameters()}
    layer.zero_grad(set_to_none=True)
    plain.backward(up)
    torch.testing.assert_close(fused.float(), plain.float(), rtol=3e-2, atol=3e-2)
    torch.testing.assert_close(xa.grad.float(), xb.grad.float(), rtol=5e-2, atol=5e-2)
    for n, p in layer.named_parameters():
        ref = p.grad.float()
        assert float((grads_fused[n].float() - ref).abs().max()) <= 5e-2 * float(ref.abs().max()) + 1e-3, n


@pytest.mark.parametrize("rows,cols,view_off", [(1000, 776, 0), (8192, 2048, 0), (300, 264, 8), (129, 1030, 0), (64, 6, 0)])
def test_column_sums_match_the_fp32_sum(rows, cols, view_off):
    """Bias-gradient column sums: ragged row counts, widths that are no multiple of 8, and a strided view."""
    from stacr_b200.ops import _lib, stacr_ops

    g = torch.Generator(device="cuda").manual_seed(rows + cols)
    frame = torch.randn(rows, cols + 2 * view_off, device="cuda", generator=g).bfloat16()
    dy = frame[:, view_off:view_off + cols] if view_off else frame
    got = stacr_ops.colsum(dy)
    torch.cuda.synchronize()
    _lib.check_status()
    want = dy.float().sum(0)
    torch.testing.assert_close(got, want, rtol=1e-3, atol=1e-2 * float(want.abs().max()) + 1e-3)
