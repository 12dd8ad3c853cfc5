"""Weight-gradient kernel that delivers into the flat gradient buffer, and the bounded flag wait."""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(rows=1024, n=512, o=768, r=8, budget=0.01, seed=0):
    from stacr_b200.ops import stacr_ops

    g = torch.Generator(device="cuda").manual_seed(seed)
    x = (torch.randn(rows, r, device="cuda", generator=g) @ torch.randn(r, n, device="cuda", generator=g)
         + 0.3 * torch.randn(rows, n, device="cuda", generator=g)).bfloat16()
    q = torch.linalg.qr(torch.randn(n, r, device="cuda", generator=g)).Q.contiguous()
    qb = q.bfloat16().contiguous()
    c = stacr_ops.project(x, stacr_ops.pad_basis_transpose(qb))[:, :r].bfloat16().contiguous()
    k = int(round(budget * rows * n))
    idx, val, scale = stacr_ops.residual_topk(x, c, qb, [k], rows, 8, torch.int32)
    dy = torch.randn(rows, o, device="cuda", generator=g).bfloat16()
    return dy, c, q, (idx, val, scale, 8, k), o, n


class _Sink:
    def __init__(self, flat, mode, off, world=1, peers=None, scale=1.0, region=None):
        self.flat, self.mode, self.param_off, self.world, self.scale = flat, mode, off, world, scale
        lo, hi = region if region else (off, flat.numel())
        self.region_lo = lo
        self.per_vecs = max(1, ((hi - lo) // 4 + world - 1) // world)
        self.peer_ptrs = peers


@pytest.mark.parametrize("transposed", [False, True])
def test_local_sink_accumulates_exactly_what_the_plain_kernel_returns(transposed):
    from stacr_b200.ops import _lib, stacr_ops

    dy, c, q, res, o, n = _case()
    want = stacr_ops.weight_grad(dy, c, q, res, o, n, transposed, torch.float32)
    off = 64
    flat = torch.full((off + o * n + 32,), 0.5, device="cuda")
    out = stacr_ops.weight_grad(dy, c, q, res, o, n, transposed, torch.float32, sink=_Sink(flat, 1, off, scale=2.0))
    assert out is None
    _lib.check_status()
    got = flat[off:off + o * n].view_as(want)
    torch.testing.assert_close(got, 0.5 + 2.0 * want, rtol=3e-4, atol=2e-3)  # the split-K partial sums of T add up in a different order per call
    assert bool((flat[:off] == 0.5).all()) and bool((flat[off + o * n:] == 0.5).all())     # nothing outside the slot is touched


def test_owner_sink_places_each_slice_in_its_owners_copy():
    """Two ranks emulated on one device as two flat buffers and two sequential launches (no launch waits on another)."""
    from stacr_b200.ops import _lib, stacr_ops

    off, world = 128, 2
    cases = [_case(seed=s) for s in (1, 2)]
    o, n = cases[0][4], cases[0][5]
    numel = o * n
    bufs = [torch.zeros(off + numel, device="cuda") for _ in range(world)]
    peers = torch.tensor([b.data_ptr() for b in bufs], dtype=torch.int64, device="cuda")
    grads = []
    for rank, (dy, c, q, res, _, _) in enumerate(cases):
        grads.append(stacr_ops.weight_grad(dy, c, q, res, o, n, False, torch.float32))
        stacr_ops.weight_grad(dy, c, q, res, o, n, False, torch.float32, sink=_Sink(bufs[rank], 2, off, world, peers, region=(off, off + numel)))
    _lib.check_status()
    total = (grads[0] + grads[1]).reshape(-1)
    per = ((numel // 4 + world - 1) // world) * 4
    torch.testing.assert_close(bufs[0][off:off + per], total[:per], rtol=3e-4, atol=2e-3)          # rank 0 owns the first slice
    torch.testing.assert_close(bufs[1][off + per:], total[per:], rtol=3e-4, atol=2e-3)             # rank 1 owns the second
    assert float(bufs[0][off + per:].abs().max()) == 0.0 and float(bufs[1][off:off + per].abs().max()) == 0.0


def test_sink_rejects_a_parameter_outside_its_region():
    from stacr_b200.ops import _lib, stacr_ops

    dy, c, q, res, o, n = _case(rows=256, n=256, o=256)
    flat = torch.zeros(o * n, device="cuda")
    peers = torch.tensor([flat.data_ptr()], dtype=torch.int64, device="cuda")
    with pytest.raises(_lib.KernelError):
        stacr_ops.weight_grad(dy, c, q, res, o, n, False, torch.float32, sink=_Sink(flat, 2, 0, 1, peers, region=(0, 1024)))
    with pytest.raises(_lib.KernelError):
        stacr_ops.weight_grad(dy, c, q, res, o, n, False, torch.float32, sink=_Sink(flat, 1, 2))  # slot not 16-byte aligned


def test_gradsync_single_rank_fused_parameters_match_autograd():
    import stacr_b200 as S
    from stacr_b200.models import build_model
    from stacr_b200.parallel import GradSync

    torch.manual_seed(0)
    ids = torch.randint(0, 1024, (4, 64), device="cuda")

    def grads(fused):
        torch.manual_seed(1)
        model = build_model("gpt-tiny", n_layer=2, resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0).cuda().train()
        layers = S.apply_stacr(model, rank=4, residual_budget=0.01, min_features=8, turbo_after_step=None)
        sync = GradSync(model.parameters(), fused=[l.weight for l in layers] if fused else ())
        S.set_step(layers, 0)
        sync.zero_grad()
        with torch.autocast("cuda", dtype=torch.bfloat16):
            model(input_ids=ids, labels=ids).loss.backward()
        sync.finish()
        out = {n: p.grad.detach().clone() for n, p in model.named_parameters()}
        assert sync.n_fused == (len(layers) if fused else 0)
        sync.close()
        return out

    a, b = grads(False), grads(True)
    for name in a:
        # bf16 atomics in the embedding backward and split-K sums make two runs differ in the last bits
        x, y = a[name].float().reshape(-1), b[name].float().reshape(-1)
        # (the compressed layers also pick slightly different residual entries when their inputs differ in the last bit;
        # the delivery path itself is checked exactly by the operator-level tests above)
        cos = float(torch.dot(x, y) / (x.norm() * y.norm() + 1e-30))
        assert cos > 0.99, (name, cos)


def test_a_wait_that_nothing_satisfies_runs_out_and_leaves_the_context_usable():
    from stacr_b200.ops import _lib
    from stacr_b200.parallel import flags

    dev = torch.device("cuda", torch.cuda.current_device())
    _lib.check_status(dev)
    flag = flags.new_flag(dev)
    seen = torch.full((1,), -1, dtype=torch.int32, device=dev)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    flags.wait(flag, expected=1, limit_s=0.05, observed=seen)     # no one ever sets the flag
    stop.record()
    torch.cuda.synchronize()
    assert 40.0 <= start.elapsed_time(stop) < 1000.0
    with pytest.raises(_lib.KernelError, match="21"):
        _lib.check_status(dev)
    assert int(seen.item()) == 0
    _lib.check_status(dev)                                         # status was cleared; the context still works
    assert float((torch.ones(8, device=dev) * 2).sum()) == 16.0
    flags.set_(flag, 3)
    flags.wait(flag, expected=3, limit_s=0.05, observed=seen)      # satisfied at once: no timeout recorded
    torch.cuda.synchronize()
    _lib.check_status(dev)
    assert int(seen.item()) == 3


@pytest.mark.parametrize("transposed,o", [(False, 2048), (True, 2048), (False, 768)])
def test_skewed_residual_is_split_over_several_ctas_and_still_exact(transposed, o):
    """A third of the residual entries sit in two features: their strips are cut into pieces that add with reductions."""
    from stacr_b200.ops import _lib, stacr_ops

    torch.manual_seed(3)
    rows, n, r, k = 2048, 512, 8, 20000
    cols = torch.randint(0, n, (k,), device="cuda")
    cols[: k // 3] = torch.where(torch.rand(k // 3, device="cuda") < 0.5, 17, 300)
    rows_i = torch.randint(0, rows, (k,), device="cuda")
    flat = torch.unique(rows_i.long() * n + cols.long())          # one entry per position
    k = flat.numel()
    vals = torch.randn(k, device="cuda").bfloat16()
    dy = torch.randn(rows, o, device="cuda").bfloat16()
    c = torch.randn(rows, r, device="cuda").bfloat16()
    q = torch.linalg.qr(torch.randn(n, r, device="cuda")).Q.contiguous()
    scale = torch.ones(1, device="cuda")
    got = stacr_ops.weight_grad(dy, c, q, (flat.int(), vals, scale, 0, k), o, n, transposed, torch.float32)
    _lib.check_status()
    sparse = torch.zeros(rows, n, device="cuda")
    sparse.view(-1)[flat] = vals.float()
    want = (dy.float().t() @ c.float()) @ q.t() + dy.float().t() @ sparse
    if transposed:
        want = want.t()
    torch.testing.assert_close(got, want, rtol=2e-3, atol=2e-2)
    heavy = int((flat % n == 17).sum())
    assert heavy > 4 * stacr_ops._plan_target()                     # the case really exercises the split
