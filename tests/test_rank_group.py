"""Leader + rank-worker processes (plow_b200/serve/rank_group.py) and the lockstep / leader-follower groups
(plow_b200/parallel/group.py), on CPU: workers are real child processes that talk to the leader over the
authenticated local connection; the step groups run as gloo ranks."""
import os
import subprocess
import sys
import time

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _collect(req, timeout=120):
    toks, fin = [], None
    while True:
        ch = req.out.get(timeout=timeout)
        if ch.kind == "token":
            toks.append(ch.token_id)
        elif ch.kind == "done":
            return toks, ch.finish_reason
        else:
            return toks, "error:" + str(ch.error)


def test_rank_workers_serve_requests_and_match_in_process_engine(tiny_assets):
    from plow_b200.parallel.dp import DpRouter
    from plow_b200.runtime.cpu_engine import CpuEngine
    from plow_b200.runtime.scheduler import GenParams, ModelMux
    from plow_b200.serve.rank_group import RankGroup
    from plow_b200.text.tokenizer import ByteTokenizer
    assets = tiny_assets / "assets"
    group = RankGroup(assets, 2, "dp", worker_args=["--backend", "cpu", "--max-slots", "4", "--max-ctx", "256"],
                      env={"PYTHONPATH": ROOT}, startup_timeout_s=180)
    try:
        assert len(group.muxes) == 2
        router = DpRouter(group.muxes)
        prompts = [[5 + i, 9, 11, 200 + i, 17] for i in range(6)]
        reqs = [router.route(None, p).submit(p, GenParams(max_tokens=6, ignore_eos=True)) for p in prompts]
        outs = [_collect(r) for r in reqs]
        assert all(fin == "length" and len(t) == 6 for t, fin in outs), outs
        # the same prompts through an in-process engine give the same greedy tokens
        mux = ModelMux(CpuEngine(assets, max_slots=4, max_ctx=256), ByteTokenizer()).start()
        want = [_collect(mux.submit(p, GenParams(max_tokens=6, ignore_eos=True)))[0] for p in prompts]
        mux.stop()
        assert [t for t, _ in outs] == want
        snap = group.muxes[0].metrics.snapshot()
        assert snap["counters"]["requests_finished"] >= 1
        assert group.muxes[0].load_estimate().get("live") is not None
    finally:
        group.shutdown()
    assert all(p.poll() is not None for p in group.procs)


def test_worker_exit_fails_pending_requests_and_marks_group_dead(tiny_assets):
    from plow_b200.runtime.engine import EngineHealth
    from plow_b200.runtime.scheduler import GenParams
    from plow_b200.serve.rank_group import RankGroup
    group = RankGroup(tiny_assets / "assets", 2, "dp", worker_args=["--backend", "cpu", "--max-slots", "2", "--max-ctx", "4096"],
                      env={"PYTHONPATH": ROOT}, startup_timeout_s=180)
    try:
        req = group.muxes[1].submit([3, 4, 5], GenParams(max_tokens=100000, ignore_eos=True))
        assert req.out.get(timeout=60).kind == "token"   # the request is running (thousands of tokens to go)
        group.procs[1].terminate()                       # the exact child this test started; it leaves between steps of a CPU engine
        toks, fin = _collect(req, timeout=60)
        assert fin.startswith("error")
        t0 = time.monotonic()
        while group.failed is None and time.monotonic() - t0 < 20:
            time.sleep(0.1)
        assert group.failed and "rank 1" in group.failed
        assert all(m.engine.health == EngineHealth.DEAD for m in group.muxes)
        late = group.muxes[0].submit([3, 4], GenParams(max_tokens=2))
        assert _collect(late)[1].startswith("error")     # a failed group stays failed
    finally:
        group.shutdown()


WORKER = r'''
import os, sys, datetime
import torch.distributed as dist
sys.path.insert(0, os.environ["PLOW_ROOT"])
from plow_b200.parallel.group import StepGroup, LeaderGroup, GroupStopped
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=120))      # generous: a cold first import of one rank can take tens of seconds
g = StepGroup(rank, world, timeout_s=120)
# rank 0 decodes 3 rows, rank 1 prefills 40 rows: everyone must run the 40-row prefill step
assert g.agree(rank == 0, 3 if rank == 0 else 40, True, samples=rank + 1) == (False, 40, True, 2)
# rank 1 idle, rank 0 decodes
assert g.agree(True, 5 if rank == 0 else 0, rank == 0) == (True, 5, True, 0)
# nobody has work: no launch
assert g.agree(True, 0, False)[2] is False
lg = LeaderGroup(rank, world, timeout_s=120)
if rank == 0:
    lg.publish({"batch": {"n": 7}, "pages": {2: [1, 2, 3]}})
else:
    st = lg.receive()
    assert st["batch"]["n"] == 7 and st["pages"][2] == [1, 2, 3]
# a stop request reaches every rank as GroupStopped
try:
    g.agree(True, 1, True, stop=(rank == 1))
    raise SystemExit("stop flag ignored")
except GroupStopped:
    pass
if rank == 0:
    lg.stop()
else:
    try:
        lg.receive(); raise SystemExit("follower did not see the stop")
    except GroupStopped:
        pass
print("ok", rank)
'''


def test_step_group_agreement_and_leader_broadcast(tmp_path):
    f = tmp_path / "w.py"
    f.write_text(WORKER)
    env = dict(os.environ, PLOW_ROOT=ROOT)
    import socket
    with socket.socket() as s:                   # a port nobody holds right now (a fixed one can linger from an earlier run)
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                        "--master-port", str(port), str(f)], env=env, capture_output=True, text=True, timeout=400)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert r.stdout.count("ok") == 2
