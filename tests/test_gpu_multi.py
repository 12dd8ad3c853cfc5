"""Multi-GPU checks; each test launches its own ranks as child processes on the GPUs that are visible."""

import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _gpus() -> int:
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _launch(module_args, nproc, port, env_extra=None, timeout=420):
    env = {**os.environ, "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port), "NCCL_DEBUG": "WARN", **(env_extra or {})}
    for key in ("RANK", "LOCAL_RANK", "WORLD_SIZE", "LOCAL_WORLD_SIZE", "GROUP_RANK", "ROLE_RANK", "TORCHELASTIC_RUN_ID"):
        env.pop(key, None)          # this file may itself be running under a launcher
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", str(port)] + module_args
    return subprocess.run(cmd, capture_output=True, text=True, env=env, cwd=REPO, timeout=timeout)


@pytest.mark.skipif(_gpus() < 2, reason="needs two GPUs")
def test_peer_memory_collectives_fused_gradient_and_fused_tp_gemm_agree_with_nccl():
    if int(os.environ.get("RANK", "0")) != 0:
        pytest.skip("launched once, from rank 0")
    run = _launch(["-m", "stacr_b200.parallel.selftest"], 2, 29741)
    assert run.returncode == 0, run.stdout[-1500:] + run.stderr[-3000:]
    report = json.loads([l for l in run.stdout.splitlines() if l.startswith("{")][-1])
    assert report["ok"] and report["world"] == 2
    assert report["fused_dw_p2p_max_err"] < 1e-3
    assert report["tp_gemm_allreduce_p2p_rel_err"] < 2e-2


_LEAVER = r'''
import os, sys, time, datetime, torch, torch.distributed as dist
sys.path.insert(0, os.environ["REPO"])
from stacr_b200.parallel.health import Heartbeat, RankFailure
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
dist.init_process_group("nccl", timeout=datetime.timedelta(seconds=20))
hb = Heartbeat(dist.distributed_c10d._get_default_store(), rank, world, timeout=5.0)
x = torch.ones(1 << 20, device="cuda")
dist.all_reduce(x); torch.cuda.synchronize()
outcome = "finished"
try:
    for step in range(6):
        if rank == 1 and step == 3:
            torch.cuda.synchronize()      # nothing of this rank is in flight
            hb.leave()
            outcome = "left"
            break
        time.sleep(0.3)
        hb.check()                         # peers are checked on the host BEFORE the next collective is enqueued
        dist.all_reduce(x); torch.cuda.synchronize()
        hb.beat(step)
except RankFailure as exc:
    outcome = "detected:" + str(exc)[:100]
print(f"RANK{rank} {outcome}", flush=True)
assert float((torch.ones(4, device="cuda") * 2).sum()) == 8.0   # the context is still healthy
os._exit(0)
'''


@pytest.mark.skipif(_gpus() < 2, reason="needs two GPUs")
def test_a_rank_that_leaves_between_steps_is_seen_before_the_next_collective(tmp_path):
    """No collective is left waiting on the GPU: the survivor learns of the departure from the store and stops."""
    if int(os.environ.get("RANK", "0")) != 0:
        pytest.skip("launched once, from rank 0")
    script = tmp_path / "leaver.py"
    script.write_text(_LEAVER)
    run = _launch([str(script)], 2, 29742, env_extra={"REPO": REPO, "NCCL_NVLS_ENABLE": "0"}, timeout=240)
    survivor = next((l for l in run.stdout.splitlines() if l.startswith("RANK0")), "")
    assert survivor.startswith("RANK0 detected:") and "left at step" in survivor, run.stdout[-1500:] + run.stderr[-2500:]
    assert "RANK1 left" in run.stdout


@pytest.mark.skipif(_gpus() < 2, reason="needs two GPUs")
def test_sharded_optimizer_step_replayed_as_a_graph_on_two_gpus():
    """The benchmark's own path at a small shape: reduce-to-owner buckets, 1/W optimizer with multicast weight publication,
    the whole step captured once and replayed; both ranks finish and report one finite number."""
    if int(os.environ.get("RANK", "0")) != 0:
        pytest.skip("launched once, from rank 0")
    run = _launch(["bench.py", "--gpus", "2", "--small", "--steps", "3", "--warmup", "3", "--repeats", "1", "--no-evidence"], 2, 29745)
    assert run.returncode == 0, run.stdout[-1500:] + run.stderr[-3000:]
    line = json.loads([l for l in run.stdout.splitlines() if l.startswith("{")][-1])
    assert line["n_gpus"] == 2 and line["value"] > 0 and line["value"] == line["value"]
    assert line["config"]["cuda_graph"] is True, line["config"].get("cuda_graph_error")
    assert line["config"]["optimizer_sharding"].startswith("ZeRO-1")
    assert line["e2e"]["value"] > 0 and line["gpu_launches"] > 0
