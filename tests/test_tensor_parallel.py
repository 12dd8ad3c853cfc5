"""Tensor-parallel algebra: two gloo ranks against the unsharded model (output, loss and gradients)."""

import os
import subprocess
import sys

import pytest
import torch
from torch import nn

from stacr_b200.protocols.tensor_parallel import convert_conv1d_to_linear, shard_linear_column, shard_linear_row
from stacr_b200.protocols.tp_gpt2 import get_tp_stacr_targets, shard_gpt2_qkv_column

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shards_reassemble_the_full_projection():
    torch.manual_seed(0)
    lin = nn.Linear(12, 8)
    x = torch.randn(5, 12)
    cols = [shard_linear_column(lin, r, 2) for r in range(2)]
    torch.testing.assert_close(torch.cat([c(x) for c in cols], dim=-1), lin(x))
    rows = [shard_linear_row(lin, r, 2) for r in range(2)]
    assert rows[0].bias is not None and rows[1].bias is None
    torch.testing.assert_close(sum(rw(x[:, r * 6:(r + 1) * 6]) for r, rw in enumerate(rows)), lin(x))
    with pytest.raises(AssertionError):
        shard_linear_column(lin, 0, 3)


def test_qkv_sharding_takes_whole_heads_of_each_part():
    lin = nn.Linear(8, 3 * 8)
    with torch.no_grad():
        lin.weight.copy_(torch.arange(24.0)[:, None].expand(24, 8))
    shard = shard_gpt2_qkv_column(lin, 1, 2, num_heads=4, head_dim=2)
    assert shard.weight[:, 0].tolist() == [4, 5, 6, 7, 12, 13, 14, 15, 20, 21, 22, 23]


def test_conv1d_conversion_keeps_the_function():
    class Conv1D(nn.Module):
        def __init__(self):
            super().__init__()
            self.weight = nn.Parameter(torch.randn(6, 4))
            self.bias = nn.Parameter(torch.randn(4))

        def forward(self, x):
            return torch.addmm(self.bias, x, self.weight)

    net = nn.Sequential(Conv1D())
    x = torch.randn(3, 6)
    want = net(x)
    assert convert_conv1d_to_linear(net) == 1 and isinstance(net[0], nn.Linear)
    torch.testing.assert_close(net(x), want)


_WORKER = r'''
import os, sys, copy, torch, torch.distributed as dist
sys.path.insert(0, os.environ["REPO"])
import stacr_b200 as S
from stacr_b200.models import build_model
from stacr_b200.parallel import init_distributed
from stacr_b200.protocols.tensor_parallel import sync_replicated_grads, replicated_parameters
from stacr_b200.protocols.tp_gpt2 import apply_tensor_parallel_gpt2, get_tp_stacr_targets, disable_tp_dropout
rank, world, _ = init_distributed("gloo")
torch.manual_seed(0)
full = build_model("gpt-tiny", n_layer=2)
tp = copy.deepcopy(full)
apply_tensor_parallel_gpt2(tp, rank, world, None, scope=os.environ["SCOPE"])
disable_tp_dropout(tp)
ids = torch.randint(0, 1024, (2, 16), generator=torch.Generator().manual_seed(1))
ref = full(input_ids=ids, labels=ids)
out = tp(input_ids=ids, labels=ids)
assert torch.allclose(ref.logits, out.logits, atol=2e-4), float((ref.logits - out.logits).abs().max())
ref.loss.backward(); out.loss.backward()
n = sync_replicated_grads(tp)
assert n > 0
full_params = dict(full.named_parameters())
for name, p in replicated_parameters(tp):
    assert torch.allclose(p.grad, full_params[name].grad, atol=2e-4), name
# a sharded weight's gradient is the matching slice of the full gradient
g_full = full_params["transformer.h.0.mlp.c_fc.weight"].grad
g_tp = dict(tp.named_parameters())["transformer.h.0.mlp.c_fc.weight"].grad
size = g_full.shape[0] // world
assert torch.allclose(g_tp, g_full[rank * size:(rank + 1) * size], atol=2e-4)
# compression on top of the shards: row-parallel layers see N/tp features
names = get_tp_stacr_targets(tp, "all_linear" if os.environ["SCOPE"] == "full" else "all_mlp")
layers = S.apply_stacr(tp, surface="none", target_names=names, min_features=1, rank=4, turbo_after_step=None)
assert any(l.in_features == 1024 // world for l in layers)
tp.zero_grad(); S.set_step(layers, 0)
out2 = tp(input_ids=ids, labels=ids)
# a compressed shard carries its collective inside its own products: the forward is still exact ...
assert all(getattr(l, "tp_context", None) is not None for l in layers)
assert torch.allclose(ref.logits, out2.logits, atol=2e-4), float((ref.logits - out2.logits).abs().max())
out2.loss.backward()
assert all(torch.isfinite(p.grad).all() for p in tp.parameters() if p.grad is not None)
# ... and so is the input gradient, hence every replicated parameter's gradient (only the shards' own dW is approximate)
sync_replicated_grads(tp)
for name, p in replicated_parameters(tp):
    assert torch.allclose(p.grad, full_params[name].grad, atol=2e-4), name
dist.destroy_process_group()
'''


@pytest.mark.parametrize("scope", ["mlp_only", "full"])
def test_two_rank_tensor_parallel_matches_unsharded(tmp_path, scope):
    script = tmp_path / "tp_worker.py"
    script.write_text(_WORKER)
    port = "29621" if scope == "full" else "29622"
    env = {**os.environ, "REPO": REPO, "SCOPE": scope}
    run = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                          "--master-port", port, str(script)], capture_output=True, text=True, env=env, timeout=300)
    assert run.returncode == 0, run.stdout[-1500:] + run.stderr[-3000:]


def test_stacr_target_scopes():
    from stacr_b200.models import build_model
    from stacr_b200.protocols.tp_gpt2 import apply_tensor_parallel_gpt2

    model = build_model("gpt-tiny", n_layer=1)
    apply_tensor_parallel_gpt2(model, 0, 1, None, scope="full")
    assert get_tp_stacr_targets(model, "row_only") == ["transformer.h.0.mlp.c_proj"]
    assert len(get_tp_stacr_targets(model, "all_linear")) == 4
    with pytest.raises(ValueError):
        get_tp_stacr_targets(model, "bogus")
    with pytest.raises(ValueError):
        apply_tensor_parallel_gpt2(build_model("gpt-tiny", n_layer=1), 0, 3, None, scope="full")
