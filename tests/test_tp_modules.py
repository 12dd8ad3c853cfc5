"""Row/column-parallel linears: on one rank (and on the CPU) they must be plain linears, forward and backward."""

import torch
from torch import nn

from stacr_b200.parallel.tp import ColumnParallelLinear, RowParallelLinear, column_parallel_linear, engine_for, row_parallel_linear


def _check(wrapper_cls, functional):
    torch.manual_seed(0)
    lin = nn.Linear(48, 32)
    x = torch.randn(3, 5, 48, requires_grad=True)
    ref = lin(x)
    ref.square().sum().backward()
    want = (x.grad.clone(), lin.weight.grad.clone(), lin.bias.grad.clone())
    for call in (wrapper_cls(lin), lambda t: functional(t, lin)):
        x.grad = None
        lin.zero_grad()
        out = call(x)
        torch.testing.assert_close(out, ref)
        out.square().sum().backward()
        for got, exp in zip((x.grad, lin.weight.grad, lin.bias.grad), want):
            torch.testing.assert_close(got, exp, rtol=1e-5, atol=1e-6)


def test_row_parallel_is_a_linear_on_one_rank():
    _check(RowParallelLinear, row_parallel_linear)


def test_column_parallel_is_a_linear_on_one_rank():
    _check(ColumnParallelLinear, column_parallel_linear)


def test_no_fused_engine_without_peers():
    assert engine_for(torch.device("cpu"), 1024) is None
    wrapped = RowParallelLinear(nn.Linear(16, 16), fused=True)
    assert wrapped._engine(torch.randn(2, 16), 32) is None
    assert "fused=True" in wrapped.extra_repr()


def test_fused_tensor_parallel_degree_limit_is_configurable(monkeypatch):
    from stacr_b200.parallel import tp

    monkeypatch.delenv("STACR_TP_FUSED_MAX_WORLD", raising=False)
    assert tp._max_fused_world() == 2
    monkeypatch.setenv("STACR_TP_FUSED_MAX_WORLD", "4")
    assert tp._max_fused_world() == 4
