"""Compressed-linear kernels (selection, basis update, weight gradient, full layer) against fp32 PyTorch references."""

import copy

import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup(rows, n, r, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    base = torch.randn(rows, r, device="cuda", generator=g) @ torch.randn(r, n, device="cuda", generator=g)
    x = (base + 0.3 * torch.randn(rows, n, device="cuda", generator=g)).bfloat16()
    q = torch.linalg.qr(torch.randn(n, r, device="cuda", generator=g)).Q.contiguous()
    qb = q.bfloat16().contiguous()
    c = (x.float() @ qb.float()).bfloat16().contiguous()
    e = (x.float() - c.float() @ qb.float().t()).bfloat16()
    return x, q, qb, c, e


@pytest.mark.parametrize("rows,n,r", [(256, 512, 8), (1000, 2048, 8), (512, 768, 16), (300, 1280, 32), (2048, 8192, 8)])
@pytest.mark.parametrize("bits", [0, 8, 4])
def test_global_topk_matches_reference_value_set(rows, n, r, bits):
    from stacr_b200.ops import _lib, stacr_ops

    x, q, qb, c, e = _setup(rows, n, r)
    k = int(round(0.01 * rows * n))
    idx, val, scale = stacr_ops.residual_topk(x, c, qb, [k], rows, bits, torch.int32)
    torch.cuda.synchronize()
    _lib.check_status()
    assert idx.numel() == k and idx.unique().numel() == k
    ref_top = e.reshape(-1).float().abs().topk(k).values.sort().values
    got_e = e.reshape(-1)[idx.long()].float()
    # the kernel recomputes the residual with its own fp32 summation order: allow one bf16 ulp
    torch.testing.assert_close(got_e.abs().sort().values, ref_top, rtol=2e-2, atol=1e-3)
    if bits == 0:
        torch.testing.assert_close(val.float(), got_e, rtol=2e-2, atol=1e-3)
    else:
        qmax = 127.0 if bits == 8 else 7.0
        assert abs(float(scale) - float(ref_top[-1]) / qmax) <= 2e-2 * float(scale)
        deq = val.float() * scale
        assert (deq - got_e).abs().max() <= 0.51 * float(scale) + 2e-2 * float(got_e.abs().max())


def _kernel_order_residual(x, c, qb):
    """bf16 residual with the kernel's own arithmetic: a chain of fp32 fused multiply-adds over the rank, then one subtraction.

    Each fused step is emulated in float64 (the product of two bf16 values and its sum with an fp32 accumulator are exact
    there) and rounded to fp32, so the result is bit-identical to the kernel's except for double-rounding ties.
    """
    acc = torch.zeros(x.shape, dtype=torch.float32, device=x.device)
    for j in range(c.shape[1]):
        acc = (c[:, j:j + 1].double() * qb[:, j].double()[None, :] + acc.double()).float()
    return (x.float() - acc).bfloat16()


def _assert_exact_topk(e, idx, k):
    """The selected magnitudes are exactly the k largest magnitudes of ``e`` (as a multiset)."""
    flat = e.reshape(-1).float().abs()
    assert idx.numel() == k and idx.unique().numel() == k
    got = flat[idx.long()].sort().values
    want = flat.topk(k).values.sort().values
    mism = int((got != want).sum())
    assert mism <= max(2, k // 50000), f"{mism} of {k} selected magnitudes differ from the exact top-k"


@pytest.mark.parametrize("rows,n,r,bits", [(2048, 8192, 8, 8), (4096, 2048, 8, 0), (1024, 4096, 16, 4), (1100, 1280, 32, 0)])
def test_sampled_threshold_selection_is_the_exact_topk(rows, n, r, bits):
    from stacr_b200.ops import _lib, stacr_ops

    x, q, qb, c, _ = _setup(rows, n, r, seed=11)
    e = _kernel_order_residual(x, c, qb)
    k = int(round(0.005 * rows * n))
    idx, val, scale = stacr_ops.residual_topk(x, c, qb, [k], rows, bits, torch.int32, sampled=True)
    torch.cuda.synchronize()
    _lib.check_status()
    stats = stacr_ops.last_sampled_selection_stats()
    assert stats["fell_back"] == [0], stats
    assert k <= stats["candidates"][0] <= 3 * k + 8192, stats
    _assert_exact_topk(e, idx, k)
    got_e = e.reshape(-1)[idx.long()].float()
    if bits == 0:
        assert torch.equal(val.float(), got_e)
    else:
        qmax = 127.0 if bits == 8 else 7.0
        want_scale = float(e.float().abs().max()) / qmax
        assert abs(float(scale) - want_scale) <= 1e-6 * want_scale
        assert (val.float() * scale - got_e).abs().max() <= 0.5001 * float(scale)
    # same selection as the two-pass form
    idx2, _, scale2 = stacr_ops.residual_topk(x, c, qb, [k], rows, bits, torch.int32, sampled=False)
    _assert_exact_topk(e, idx2, k)
    assert float(scale2) == float(scale)


def test_sampled_threshold_selection_per_chunk_quotas():
    from stacr_b200.ops import _lib, stacr_ops

    rows, n, r, chunk = 2560, 2048, 8, 512
    x, q, qb, c, _ = _setup(rows, n, r, seed=5)
    x[700:720] *= 6.0                       # a stretch of heavy rows inside one chunk
    c = (x.float() @ qb.float()).bfloat16().contiguous()
    e = _kernel_order_residual(x, c, qb)
    quotas = [int(round(0.005 * chunk * n))] * 5
    idx, val, _ = stacr_ops.residual_topk(x, c, qb, quotas, chunk, 0, torch.int32, sampled=True)
    torch.cuda.synchronize()
    _lib.check_status()
    rows_of = idx.long() // n
    for ci, k in enumerate(quotas):
        mine = idx[(rows_of >= ci * chunk) & (rows_of < (ci + 1) * chunk)]
        lo = ci * chunk * n
        _assert_exact_topk(e[ci * chunk:(ci + 1) * chunk], mine - lo, k)


@pytest.mark.parametrize("case", ["sample_overestimates", "all_ties"])
def test_sampled_threshold_selection_redoes_a_misjudged_chunk_exactly(case):
    """Inputs built to fool the sample: the chunk must be flagged, redone by the exact passes, and still be the exact top-k."""
    from stacr_b200.ops import _lib, stacr_ops

    rows, n, r = 1024, 2048, 8
    g = torch.Generator(device="cuda").manual_seed(7)
    qb = torch.linalg.qr(torch.randn(n, r, device="cuda", generator=g)).Q.bfloat16().contiguous()
    c = torch.zeros(rows, r, device="cuda", dtype=torch.bfloat16)          # zero coefficients: the residual is the input
    k = int(round(0.005 * rows * n))
    if case == "all_ties":
        x = (torch.randint(0, 2, (rows, n), device="cuda", generator=g).float() * 2 - 1).bfloat16()
    else:
        x = (0.01 * torch.randn(rows, n, device="cuda", generator=g)).bfloat16()
        # large entries only where the sampler looks (line + row divisible by 16): it believes they are 16 times as many
        rr = torch.arange(rows, device="cuda")[:, None]
        line = torch.arange(n, device="cuda")[None, :] // 64
        seen = ((line + rr) % 16 == 0)
        pick = seen & (torch.rand(rows, n, device="cuda", generator=g) < (k / 6) / seen.sum())
        x = torch.where(pick, torch.full_like(x, 5.0), x)
    idx, val, _ = stacr_ops.residual_topk(x, c, qb, [k], rows, 0, torch.int32, sampled=True)
    torch.cuda.synchronize()
    _lib.check_status()
    assert stacr_ops.last_sampled_selection_stats()["fell_back"] == [1]
    _assert_exact_topk(x, idx, k)
    assert torch.equal(val.float(), x.reshape(-1)[idx.long()].float())


def test_chunk_quota_selection_counts_and_values():
    from stacr_b200.ops import _lib, stacr_ops

    rows, n, r, chunk = 1536, 1024, 8, 512
    x, q, qb, c, e = _setup(rows, n, r, seed=3)
    quotas = [int(round(0.005 * chunk * n))] * 3
    idx, val, _ = stacr_ops.residual_topk(x, c, qb, quotas, chunk, 0, torch.int32)
    torch.cuda.synchronize()
    _lib.check_status()
    rows_of = idx.long() // n
    for ci, k in enumerate(quotas):
        mine = idx[(rows_of >= ci * chunk) & (rows_of < (ci + 1) * chunk)]
        assert mine.numel() == k
        ref = e[ci * chunk:(ci + 1) * chunk].reshape(-1).float().abs().topk(k).values.sort().values
        got = e.reshape(-1)[mine.long()].float().abs().sort().values
        torch.testing.assert_close(got, ref, rtol=2e-2, atol=1e-3)


def test_oja_update_matches_framework_step():
    from stacr_b200.oja import oja_step
    from stacr_b200.ops import _lib
    from stacr_b200.ops.basis import oja_step_kernels

    rows, n, r = 2048, 1024, 8
    x, q, qb, c, e = _setup(rows, n, r, seed=5)
    new = oja_step_kernels(q, x, 0.05)
    torch.cuda.synchronize()
    _lib.check_status()
    ref = oja_step(q, x, 0.05)
    gram = new.t() @ new
    torch.testing.assert_close(gram, torch.eye(r, device="cuda"), atol=1e-4, rtol=0)
    # same subspace: projector difference small
    diff = (new @ new.t() - ref @ ref.t()).norm() / (ref @ ref.t()).norm()
    assert diff < 2e-2, float(diff)


@pytest.mark.parametrize("transposed", [False, True])
@pytest.mark.parametrize("bits", [0, 8, 4])
def test_weight_grad_matches_fp32_formula(transposed, bits):
    from stacr_b200.ops import _lib, stacr_ops
    from stacr_b200.quant import quantize_values

    rows, n, o, r = 1024, 512, 768, 8
    x, q, qb, c, e = _setup(rows, n, r, seed=7)
    dy = torch.randn(rows, o, device="cuda").bfloat16()
    k = 4000
    idx = torch.randperm(rows * n, device="cuda")[:k].to(torch.int32)
    vals = e.reshape(-1)[idx.long()]
    packed = quantize_values(vals, bits)
    out = stacr_ops.weight_grad(dy, c, qb.float(), (idx, packed.data, packed.scale, packed.bits, packed.length), o, n, transposed, torch.float32)
    torch.cuda.synchronize()
    _lib.check_status()
    s = torch.zeros(rows * n, device="cuda")
    s[idx.long()] = packed.dequantize(torch.float32)
    ref = (dy.float().t() @ c.float()) @ qb.float().t() + dy.float().t() @ s.reshape(rows, n)
    if transposed:
        ref = ref.t()
    err = (out - ref).abs().max() / ref.abs().max()
    assert err < 1e-2, float(err)


@pytest.mark.parametrize("transposed", [False, True])
@pytest.mark.parametrize("bits", [0, 8, 4])
def test_weight_grad_dense_route_matches_fp32_formula(transposed, bits):
    """The tensor-core route: the input is rebuilt in bf16 for the call and multiplied with dY by the CTA-pair GEMM."""
    from stacr_b200.ops import _lib, stacr_ops
    from stacr_b200.quant import quantize_values

    rows, n, o, r = 1024, 512, 768, 8
    x, q, qb, c, e = _setup(rows, n, r, seed=9)
    dy = torch.randn(rows, o, device="cuda").bfloat16()
    k = 4001                                                  # odd: the last 4-bit code shares its byte with padding
    idx = torch.randperm(rows * n, device="cuda")[:k].to(torch.int32)
    packed = quantize_values(e.reshape(-1)[idx.long()], bits)
    residual = (idx, packed.data, packed.scale, packed.bits, packed.length)
    s = torch.zeros(rows * n, device="cuda")
    s[idx.long()] = packed.dequantize(torch.float32)
    xhat = stacr_ops.rebuild_input(c, qb.float(), residual, rows, n)
    want_x = c.float() @ qb.float().t() + s.reshape(rows, n)
    torch.testing.assert_close(xhat.float(), want_x, rtol=1e-2, atol=1e-2)
    out = stacr_ops.weight_grad(dy, c, qb.float(), residual, o, n, transposed, torch.float32, dense=True)
    sparse = stacr_ops.weight_grad(dy, c, qb.float(), residual, o, n, transposed, torch.float32, dense=False)
    torch.cuda.synchronize()
    _lib.check_status()
    ref = dy.float().t() @ want_x
    if transposed:
        ref = ref.t()
    assert out.shape == ref.shape
    assert float((out - ref).abs().max() / ref.abs().max()) < 1e-2
    assert float((out - sparse).abs().max() / ref.abs().max()) < 1e-2
    # low-rank only (no residual entries) through the same route
    lr = stacr_ops.weight_grad(dy, c, qb.float(), None, o, n, transposed, torch.float32, dense=True)
    ref_lr = (dy.float().t() @ c.float()) @ qb.float().t()
    assert float((lr - (ref_lr.t() if transposed else ref_lr)).abs().max() / ref_lr.abs().max()) < 1e-2


@pytest.mark.parametrize("mode", ["chunk_topk", "global_topk", "block_sparse", "uniform", "none"])
def test_layer_forward_backward_on_kernel_path(mode):
    import stacr_b200 as S
    from stacr_b200.ops import _lib

    torch.manual_seed(11)
    lin = torch.nn.Linear(1024, 512, device="cuda")
    ref = copy.deepcopy(lin)
    layer = S.STACRLinear.from_linear(lin, rank=8, residual_budget=0.01, residual_mode=mode)
    base = torch.randn(2048, 8, device="cuda") @ torch.randn(8, 1024, device="cuda")
    x = (base + 0.2 * torch.randn(2048, 1024, device="cuda")).requires_grad_(True)
    xr = x.detach().clone().requires_grad_(True)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y = layer(x)
        yr = ref(xr)
    assert y.dtype == torch.bfloat16
    torch.testing.assert_close(y.float(), yr.float(), rtol=3e-2, atol=3e-2)
    # nothing as large as the input is saved
    saved = [t for t in y.grad_fn.saved_tensors if t is not lin.weight]
    assert all(t.numel() < x.numel() // 4 for t in saved)
    assert len(saved) == (2 if mode == "none" else 5)
    g = torch.randn_like(y)
    y.backward(g)
    yr.backward(g)
    torch.cuda.synchronize()
    _lib.check_status()
    torch.testing.assert_close(x.grad, xr.grad, rtol=3e-2, atol=3e-2)
    cos = float(S.cosine_similarity(ref.weight.grad, lin.weight.grad))
    # the bar is the fp32 oracle path of the same layer on the same input (no autocast: framework ops, exact SVD-based
    # initialisation), not a fixed number: the kernels may lose at most a small margin to it
    oracle_lin = copy.deepcopy(ref)
    oracle_lin.weight.grad = None
    oracle_lin.bias.grad = None
    oracle = S.STACRLinear.from_linear(oracle_lin, rank=8, residual_budget=0.01, residual_mode=mode)
    xo = x.detach().clone().requires_grad_(True)
    oracle(xo).backward(g.float())
    cos_oracle = float(S.cosine_similarity(ref.weight.grad, oracle_lin.weight.grad))
    assert cos > cos_oracle - 0.02, (cos, cos_oracle)
    assert cos > 0.9, cos
    torch.testing.assert_close(lin.bias.grad, ref.bias.grad, rtol=2e-2, atol=2e-1)


@pytest.mark.parametrize("mode", ["topk", "block_sparse", "adaptive_threshold", "threshold", "sparse_only"])
def test_adaptive_engine_selects_on_kernels_without_a_dense_residual(mode, monkeypatch):
    """Every residual mode of the adaptive engine on a bf16 CUDA layer runs on the selection kernels (the framework
    selector is not reached) and still trains: the weight gradient stays close to the dense one."""
    from stacr_b200 import adaptive

    torch.manual_seed(0)
    lin = torch.nn.Linear(512, 256).cuda()
    cfg = adaptive.STACRConfig(rank=8, residual_mode=mode, residual_budget=0.02, residual_threshold=1.5, warmup_steps=0, quantize_coefficients=True,
                               quantize_residuals=True, residual_quantize_bits=8, update_trigger="fixed", update_interval=1000)
    layer = adaptive.STACRLinear(512, 256, config=cfg).cuda()
    layer.linear.load_state_dict(lin.state_dict())
    calls = {"n": 0}
    real = adaptive._select_adaptive

    def spy(*a, **k):
        calls["n"] += 1
        return real(*a, **k)

    monkeypatch.setattr(adaptive, "_select_adaptive", spy)
    base = torch.randn(2048, 8, device="cuda") @ torch.randn(8, 512, device="cuda")
    x = (base + 0.2 * torch.randn(2048, 512, device="cuda")).requires_grad_(True)
    layer.train()
    for _ in range(2):                                   # first call initialises the basis
        layer.zero_grad()
        with torch.autocast("cuda", dtype=torch.bfloat16):
            y = layer(x)
        y.float().square().mean().backward()
    assert calls["n"] == 0
    with torch.autocast("cuda", dtype=torch.bfloat16):
        yr = lin(x)
    yr.float().square().mean().backward()
    got, want = layer.linear.weight.grad.float().reshape(-1), lin.weight.grad.float().reshape(-1)
    cos = float(torch.dot(got, want) / (got.norm() * want.norm()))
    assert cos > (0.6 if mode == "sparse_only" else 0.9), cos


def test_sampled_selector_runs_on_the_kernels_and_agrees_with_the_framework_form(monkeypatch):
    """``sampled``: probe by the gather kernel, one pass over X for the entries above the probe's quantile, no dense residual."""
    from stacr_b200 import layers
    from stacr_b200.ops import _lib

    rows, n, r = 2048, 1024, 8
    x, q, qb, c, e = _setup(rows, n, r, seed=21)
    budget, ratio = 0.005, 0.05
    monkeypatch.setattr(layers, "_select_residual", lambda *a, **k: (_ for _ in ()).throw(AssertionError("framework selector reached")))
    idx, packed = layers._select_residual_kernels(x, c, qb, budget, 512, "sampled", 16, ratio, 8)
    torch.cuda.synchronize()
    _lib.check_status()
    monkeypatch.undo()
    k_total = int(round(budget * rows * n))
    assert 0 < idx.numel() <= k_total and packed.length == idx.numel()
    assert bool((idx[1:] > idx[:-1]).all())                          # index order, unique
    ref_idx, ref_val = layers._select_residual(x.float(), c.float(), qb.float(), budget, 512, "sampled", 16, ratio)
    common = torch.isin(idx.long(), ref_idx.long()).sum().item()
    assert common >= 0.9 * min(idx.numel(), ref_idx.numel()), (common, idx.numel(), ref_idx.numel())
    got = e.reshape(-1)[idx.long()].float().abs()
    assert float(got.min()) >= 0.9 * float(ref_val.float().abs().min())


def test_saved_tensor_compressor_runs_on_the_kernels_and_agrees_with_the_framework_codec():
    """``STACRCompressor`` on a bf16 CUDA activation: projection, exact global top-k and the rebuild all on the kernels, against
    the same basis version through the framework codec in fp32."""
    from stacr_b200 import compressor as C

    torch.manual_seed(0)
    x = (torch.randn(768, 12, device="cuda") @ torch.randn(12, 512, device="cuda") + 0.2 * torch.randn(768, 512, device="cuda")).bfloat16()
    x[5, 7] = 40.0                                                  # an outlier the residual channel must carry
    comp = C.STACRCompressor(C.STACRConfig(rank=8, residual_budget=0.01, min_features=1, min_numel=1, update_interval=10 ** 9))
    comp.pack(x)                                                    # step 0: the basis is initialised from this batch
    comp.set_step(1)
    packed = comp.pack(x.view(4, 192, 512))
    assert packed.codec == "kernels" and packed.residual[4] == round(0.01 * x.numel())
    got = comp.unpack(packed)
    assert got.shape == (4, 192, 512) and got.dtype == torch.bfloat16
    xf = x.float()
    oracle = C._FrameworkCodec.encode(xf, xf, comp._tracker(x), 0.01)
    want = C._FrameworkCodec.decode(oracle)
    got2d = got.reshape(768, 512).float()
    # bf16 basis, coefficients and output against fp32 cost ~0.3 %; the rest is entries near the selection threshold that the two
    # forms rank differently (each one moves the reconstruction by about the threshold value)
    assert (got2d - want).norm() / want.norm() < 0.05
    assert (got2d - xf).norm() <= 1.05 * (want - xf).norm() + 1e-3
    assert abs(float(got2d[5, 7]) - 40.0) < 0.5
    # through autograd: the saved activation of tanh is replaced and rebuilt, parameters are left alone
    w = torch.nn.Parameter(torch.randn(64, 512, device="cuda", dtype=torch.bfloat16) * 0.05)
    inp = (x * 0.05).detach().requires_grad_(True)
    comp.set_step(2)
    with C.stacr_saved_tensors(comp):
        y = inp.tanh() @ w.t()
    y.float().sum().backward()
    plain = (x * 0.05).detach().requires_grad_(True)
    (plain.tanh() @ w.detach().t()).float().sum().backward()
    cos = torch.nn.functional.cosine_similarity(inp.grad.float().flatten(), plain.grad.float().flatten(), dim=0)
    assert torch.isfinite(inp.grad).all() and float(cos) > 0.9
