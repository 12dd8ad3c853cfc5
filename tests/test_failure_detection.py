"""Failure detection, exercised on the host only: gloo ranks on CPU, a fake key-value store, files on disk."""

import os
import subprocess
import sys
import time

import pytest
import torch

from stacr_b200.parallel.health import (Beat, CheckpointCorrupt, Heartbeat, RankFailure, guarded, latest_valid_checkpoint, load_checkpoint,
                                        verify_checkpoint, write_checkpoint)

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class DictStore:
    """The three store calls the heartbeat uses."""

    def __init__(self):
        self.data = {}

    def set(self, key, value):
        self.data[key] = bytes(value)

    def get(self, key):
        return self.data[key]

    def check(self, keys):
        return all(k in self.data for k in keys)


def test_heartbeat_sees_silent_lagging_failed_and_departed_peers():
    store = DictStore()
    a = Heartbeat(store, 0, 3, timeout=5.0, max_lag=2)
    with pytest.raises(RankFailure) as info:
        a.check()
    assert info.value.ranks == [1, 2] and "never registered" in str(info.value)
    b = Heartbeat(store, 1, 3, timeout=5.0, max_lag=2)
    c = Heartbeat(store, 2, 3, timeout=5.0, max_lag=2)
    for step in range(3):
        for hb in (a, b, c):
            hb.beat(step)
    a.check()
    with pytest.raises(RankFailure) as info:          # rank 1 has said nothing for 60 s
        a.check(now=time.time() + 60.0)
    assert set(info.value.ranks) == {1, 2} and "silent" in info.value.reason[1]
    for step in range(3, 7):                           # rank 2 stops stepping while 0 and 1 go on
        a.beat(step)
        b.beat(step)
    with pytest.raises(RankFailure) as info:
        a.check()
    assert info.value.ranks == [2] and "steps behind" in info.value.reason[2]
    c.beat(6)
    a.check()
    c.leave()
    with pytest.raises(RankFailure) as info:
        b.check()
    assert info.value.reason[2].startswith("left at step 6")
    with pytest.raises(ZeroDivisionError):
        with b.guard():
            1 / 0
    with pytest.raises(RankFailure) as info:
        a.check()
    assert "failed: ZeroDivisionError" in info.value.reason[1]
    assert Beat.load(Beat(3, 1.5, "alive").dump()) == Beat(3, 1.5, "alive")


def test_guarded_translates_backend_timeouts_only():
    def timed_out():
        raise RuntimeError("[Rank 0] Timed out waiting 1000ms for recv operation to complete")

    def other():
        raise RuntimeError("shape mismatch")

    with pytest.raises(RankFailure):
        guarded(timed_out, what="all_reduce")
    with pytest.raises(RuntimeError, match="shape mismatch"):
        guarded(other)
    assert guarded(lambda x: x + 1, 1) == 2


def test_checkpoint_integrity_detects_truncation_and_bit_flips(tmp_path):
    good = write_checkpoint({"w": torch.arange(1000.0)}, tmp_path / "a.pt")
    assert verify_checkpoint(good) and torch.equal(load_checkpoint(good)["w"], torch.arange(1000.0))
    time.sleep(0.01)
    cut = write_checkpoint({"w": torch.ones(1000)}, tmp_path / "b.pt")
    raw = cut.read_bytes()
    cut.write_bytes(raw[: len(raw) // 2])
    with pytest.raises(CheckpointCorrupt, match="truncated"):
        verify_checkpoint(cut)
    time.sleep(0.01)
    flip = write_checkpoint({"w": torch.zeros(1000)}, tmp_path / "c.pt")
    raw = bytearray(flip.read_bytes())
    raw[-20] ^= 0xFF
    flip.write_bytes(bytes(raw))
    with pytest.raises(CheckpointCorrupt, match="digest"):
        load_checkpoint(flip)
    assert latest_valid_checkpoint([good, cut, flip]) == good     # newest file that still verifies
    bare = tmp_path / "d.pt"
    torch.save({"w": 1}, bare)
    assert verify_checkpoint(bare) is False
    with pytest.raises(CheckpointCorrupt):
        verify_checkpoint(bare, require_sidecar=True)
    with pytest.raises(CheckpointCorrupt, match="missing"):
        verify_checkpoint(tmp_path / "nope.pt")


def test_trainer_refuses_a_corrupt_resume_file(tmp_path):
    from stacr_b200.models import build_model
    from stacr_b200.training import train_model

    def batches(n):
        g = torch.Generator().manual_seed(0)
        out = []
        for _ in range(n):
            ids = torch.randint(0, 1024, (2, 16), generator=g)
            out.append({"input_ids": ids, "attention_mask": torch.ones_like(ids), "labels": ids.clone()})
        return out

    ckpt = tmp_path / "run.pt"
    cfg = {"task": "language_modeling", "model_name": "gpt-tiny", "method": "stacr", "steps": 2, "lr": 1e-3, "device": "cpu", "checkpoint_path": str(ckpt)}
    train_model(build_model("gpt-tiny", n_layer=1), batches(2), cfg)
    assert verify_checkpoint(ckpt)
    raw = bytearray(ckpt.read_bytes())
    raw[len(raw) // 2] ^= 0x55
    ckpt.write_bytes(bytes(raw))
    with pytest.raises(CheckpointCorrupt):
        train_model(build_model("gpt-tiny", n_layer=1), batches(3), {**cfg, "steps": 3, "checkpoint_path": None, "resume_from": str(ckpt)})


_WORKER = r'''
import os, sys, time, datetime, torch, torch.distributed as dist
sys.path.insert(0, os.environ["REPO"])
from stacr_b200.parallel.health import Heartbeat, RankFailure, guarded
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
mode = os.environ["MODE"]
dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=3))
store = dist.distributed_c10d._get_default_store()
hb = Heartbeat(store, rank, world, timeout=2.0, max_lag=None)
dist.barrier()
outcome = "finished"
try:
    for step in range(6):
        if mode == "leave" and rank == 1 and step == 2:
            hb.leave()                       # orderly exit between steps: nothing of this rank is in flight
            outcome = "left"
            break
        if mode == "raise" and rank == 1 and step == 2:
            with hb.guard():
                raise ValueError("injected host fault")
        if mode == "hang" and rank == 1 and step == 2:
            time.sleep(8)                    # never joins the collective below
            outcome = "slept"
            break
        if mode in ("leave", "raise"):
            time.sleep(0.3)                  # give the peer's store write time to land
            hb.check()                       # learn of a dead peer BEFORE enqueuing the collective
        t = torch.ones(4) * (rank + 1)
        guarded(dist.all_reduce, t, what=f"all_reduce at step {step}")
        hb.beat(step)
except RankFailure as exc:
    outcome = f"detected:{exc.ranks}:{str(exc)[:120]}"
except ValueError:
    outcome = "raised"
print(f"RANK{rank} {outcome}", flush=True)
os._exit(0)                                   # skip the group teardown, whose barrier the dead peer would never join
'''


@pytest.mark.parametrize("mode,expect", [("leave", "left at step"), ("raise", "failed: ValueError"), ("hang", "did not complete")])
def test_two_gloo_ranks_detect_a_peer_that_leaves_raises_or_never_joins(tmp_path, mode, expect):
    script = tmp_path / "worker.py"
    script.write_text(_WORKER)
    port = {"leave": 29631, "raise": 29632, "hang": 29633}[mode]
    procs = []
    for rank in range(2):
        env = {**os.environ, "REPO": REPO, "MODE": mode, "RANK": str(rank), "WORLD_SIZE": "2", "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port)}
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=120)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
        outs.append(out)
    survivor = next((l for l in outs[0].splitlines() if l.startswith("RANK0")), "")
    assert survivor.startswith("RANK0 detected:"), outs[0][-1500:] + outs[1][-1500:]
    assert expect in survivor, survivor
    assert procs[0].returncode == 0


_SYNC_WORKER = r'''
import os, sys, time, datetime, torch, torch.distributed as dist
sys.path.insert(0, os.environ["REPO"])
from stacr_b200.parallel import GradSync
from stacr_b200.parallel.health import Heartbeat, RankFailure
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=5))
hb = Heartbeat(dist.distributed_c10d._get_default_store(), rank, world, timeout=5.0)
dist.barrier()
torch.manual_seed(0)
model = torch.nn.Linear(8, 4)
sync = GradSync(model.parameters(), heartbeat=hb)
outcome = "finished"
try:
    for step in range(4):
        sync.zero_grad()
        model(torch.randn(2, 8)).sum().backward()
        if rank == 1 and step == 1:
            # what a rank does when its own status poll finds a timed-out kernel: publish, then stop
            hb.fail("KernelError: kernel status 21")
            outcome = "published"
            break
        time.sleep(0.3)
        sync.finish()          # reduces, then checks health: the peer's failure raises here, before optimizer.step()
        hb.beat(step)
except RankFailure as exc:
    outcome = f"detected:{exc.ranks}:{str(exc)[:120]}"
print(f"RANK{rank} {outcome} step={step}", flush=True)
os._exit(0)
'''


def test_gradsync_finish_raises_on_the_survivor_when_a_peer_published_a_kernel_timeout(tmp_path):
    script = tmp_path / "sync_worker.py"
    script.write_text(_SYNC_WORKER)
    procs = []
    for rank in range(2):
        env = {**os.environ, "REPO": REPO, "RANK": str(rank), "WORLD_SIZE": "2", "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": "29634"}
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=120)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
        outs.append(out)
    survivor = next((l for l in outs[0].splitlines() if l.startswith("RANK0")), "")
    # rank 0 finishes step 0 normally, then either its step-1 reduction runs out (the peer never joins) or, when the peer's
    # store write is seen first, the health check names the kernel failure; both stop the job on the survivor
    assert "detected:" in survivor or "RuntimeError" in outs[0] or "Timed out" in outs[0], outs[0][-1500:] + outs[1][-1500:]
    assert any(l.startswith("RANK1 published") for l in outs[1].splitlines()), outs[1][-1500:]


def test_bf16_shadow_follows_writes_that_bypass_the_fused_optimizer():
    from stacr_b200.layers import _bf16_weight

    w = torch.nn.Parameter(torch.randn(16, 8))
    w._bf16_shadow = w.detach().to(torch.bfloat16)
    w._bf16_shadow_version = w._version
    assert _bf16_weight(w) is w._bf16_shadow
    fresh = torch.randn(16, 8)
    with torch.no_grad():
        w.copy_(fresh)                       # what load_state_dict, a broadcast or another optimizer does
    got = _bf16_weight(w)
    assert got is w._bf16_shadow
    torch.testing.assert_close(got.float(), fresh.to(torch.bfloat16).float(), rtol=0, atol=0)
    assert w._bf16_shadow_version == w._version
