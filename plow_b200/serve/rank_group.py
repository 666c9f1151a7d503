"""Serving one model over several GPUs: a leader process (HTTP, routing, supervision) and one
``plowrt rank-worker`` process per GPU.

The leader never touches a GPU.  It starts the workers, waits for each to report in over an authenticated
local connection, and talks to them with a small message protocol:

    leader -> worker   ("submit", rid, prompt ids, GenParams)   ("cancel", rid)   ("call", seq, name)   ("stop",)
    worker -> leader   ("hello", rank, info)   ("chunk", rid, Chunk)   ("ret", seq, value)   ("stats", {...})

* expert parallelism (packet sharded with ep > 1): every worker runs its own scheduler over its own requests
  (attention is data-parallel) and the workers step in lockstep (:class:`plow_b200.parallel.group.StepGroup`);
  the leader spreads requests over them with the data-parallel router.
* tensor parallelism (tp > 1): rank 0 runs the scheduler, the other ranks replay its steps
  (:class:`plow_b200.parallel.group.LeaderGroup`); the leader sends every request to rank 0.

Supervision: a worker that exits takes the group down (the leader marks every replica dead, answers pending
requests with an error and stops the remaining workers); a worker whose connection to the leader closes stops
its group and exits.  Between steps each worker posts a heartbeat to the rendezvous store and checks its peers'
(:mod:`plow_b200.parallel.health`), so a rank that is gone is noticed on the host before the next launch.

Reference: crates/plowrt/src/serve/cuda_group.rs:1-8 (leader + rank workers), exec/proc_group.rs:251-339
(barrier that fails instead of hanging, abort flag), main.rs `rank-worker`.
"""
from __future__ import annotations

import os
import queue
import secrets
import subprocess
import sys
import threading
import time
from multiprocessing.connection import Client, Listener

from ..runtime.engine import EngineHealth
from ..runtime.scheduler import Chunk, GenParams, Request


# ------------------------------------------------------------------------------------------------ leader side
class _RemotePool:
    def __init__(self, info):
        self.n_pages = info.get("n_pages", 0)
        self._free = self.n_pages

    def available(self):
        return self._free

    def cached_prefix_len(self, _ids):
        return 0                      # prefix probing stays inside the worker; the router balances by load


class _RemoteEngine:
    def __init__(self, info):
        self.health = EngineHealth.HEALTHY
        self.max_ctx, self.max_slots = info["max_ctx"], info["max_slots"]
        self.pool = _RemotePool(info)
        self.spec = None


class _RemoteMetrics:
    def __init__(self, mux):
        self._mux = mux

    def snapshot(self):
        return self._mux.call("metrics") or {}

    def inc(self, *_a, **_k):
        pass


class _QsizeOnly:
    def __init__(self, mux):
        self._mux = mux

    def qsize(self):
        return 0              # queued requests are part of RemoteMux.live (everything in flight on the worker)


class RemoteMux:
    """Leader-side stand-in for the ModelMux of one rank worker."""

    def __init__(self, conn, rank: int, info: dict):
        self.conn, self.rank = conn, rank
        self.engine = _RemoteEngine(info)
        self.metrics = _RemoteMetrics(self)
        self.ingress = _QsizeOnly(self)
        self.stats: dict = {}
        self.draining = False
        self._reqs: dict[str, Request] = {}
        self._rets: dict[int, "queue.Queue"] = {}
        self._lock = threading.Lock()
        self._n = 0
        self._reader = threading.Thread(target=self._read_loop, daemon=True)
        self._reader.start()

    # -- what serve/app.py and the data-parallel router use
    @property
    def live(self):
        # requests this leader has in flight on the worker: exact and current, unlike the periodic stats message
        return range(len(self._reqs))

    @property
    def waiting(self):
        return range(0)

    def submit(self, prompt, params: GenParams, rid: str | None = None) -> Request:
        with self._lock:
            self._n += 1
            rid = rid or f"r{self.rank}-{self._n}"
            req = Request(rid=rid, prompt=list(prompt), params=params)
            if self.engine.health == EngineHealth.DEAD:
                req.out.put(Chunk("error", error="rank group is down", finish_reason="error"))
                return req
            self._reqs[rid] = req
            try:
                self.conn.send(("submit", rid, list(prompt), params))
            except (OSError, EOFError, BrokenPipeError):
                self._fail_all("lost the rank worker")
        return req

    def call(self, name: str, timeout: float = 10.0):
        with self._lock:
            self._n += 1
            seq = self._n
            q: "queue.Queue" = queue.Queue()
            self._rets[seq] = q
            try:
                self.conn.send(("call", seq, name))
            except (OSError, EOFError, BrokenPipeError):
                self._rets.pop(seq, None)
                return None
        try:
            return q.get(timeout=timeout)
        except queue.Empty:
            return None
        finally:
            self._rets.pop(seq, None)

    def load_estimate(self, window_s: float = 10.0):
        return self.call("load") or {}

    def drain(self, timeout_s: float = 30.0) -> bool:
        self.draining = True
        t0 = time.monotonic()
        while self._reqs and time.monotonic() - t0 < timeout_s:
            time.sleep(0.01)
        return not self._reqs

    def stop(self) -> None:
        try:
            self.conn.send(("stop",))
        except (OSError, EOFError, BrokenPipeError):
            pass

    # -- plumbing
    def _fail_all(self, why: str) -> None:
        self.engine.health = EngineHealth.DEAD
        for req in list(self._reqs.values()):
            req.out.put(Chunk("error", error=why, finish_reason="error"))
        self._reqs.clear()

    def _read_loop(self) -> None:
        while True:
            try:
                msg = self.conn.recv()
            except (EOFError, OSError):
                with self._lock:
                    self._fail_all("rank worker exited")
                return
            kind = msg[0]
            if kind == "chunk":
                _, rid, ch = msg
                req = self._reqs.get(rid)
                if req is not None:
                    req.out.put(ch)
                    if ch.kind in ("done", "error"):
                        self._reqs.pop(rid, None)
            elif kind == "ret":
                q = self._rets.get(msg[1])
                if q is not None:
                    q.put(msg[2])
            elif kind == "stats":
                self.stats = msg[1]
                self.engine.pool._free = msg[1].get("kv_pages_free", self.engine.pool._free)
                if msg[1].get("health") == EngineHealth.DEAD:
                    with self._lock:
                        self._fail_all("rank worker reported a dead engine")


class RankGroup:
    """Starts, supervises and stops the rank workers of one model."""

    def __init__(self, assets, world: int, mode: str, worker_args: list | None = None, startup_timeout_s: float = 600.0,
                 python: str | None = None, env: dict | None = None):
        self.assets, self.world, self.mode = str(assets), world, mode
        self.key = secrets.token_bytes(16)
        self.listener = Listener(("127.0.0.1", 0), authkey=self.key)
        port = self.listener.address[1]
        master_port = _free_port()
        self.procs = []
        base_env = dict(os.environ, PLOW_GROUP_KEY=self.key.hex(), **(env or {}))
        for r in range(world):
            cmd = [python or sys.executable, "-m", "plow_b200.plowrt", "rank-worker", "--assets", self.assets, "--rank", str(r),
                   "--world", str(world), "--mode", mode, "--master-port", str(master_port), "--leader", f"127.0.0.1:{port}"] \
                + list(worker_args or [])
            self.procs.append(subprocess.Popen(cmd, env=base_env))
        self.muxes: list = [None] * world
        self.failed: str | None = None
        deadline = time.monotonic() + startup_timeout_s
        self.listener._listener._socket.settimeout(5.0)
        n_expected = world if mode != "tp" else 1          # tensor parallelism: only rank 0 carries a scheduler
        got = 0
        while got < n_expected:
            if time.monotonic() > deadline or any(p.poll() is not None for p in self.procs):
                self.shutdown()
                raise RuntimeError("rank workers did not come up" + (": a worker exited" if any(p.poll() is not None for p in self.procs) else ""))
            try:
                conn = self.listener.accept()
            except OSError:
                continue
            hello = conn.recv()
            assert hello[0] == "hello"
            self.muxes[hello[1]] = RemoteMux(conn, hello[1], hello[2])
            got += 1
        self.muxes = [m for m in self.muxes if m is not None]
        self._watch = threading.Thread(target=self._supervise, daemon=True)
        self._watch.start()

    def _supervise(self) -> None:
        while self.failed is None:
            for r, p in enumerate(self.procs):
                rc = p.poll()
                if rc is not None:
                    self.failed = f"rank {r} exited with code {rc}"
                    break
            else:
                time.sleep(0.2)
        # a failed group stays failed: every replica is dead, pending requests get an error, the rest is stopped
        for m in self.muxes:
            with m._lock:
                m._fail_all(self.failed or "rank group stopped")
        self.shutdown(kill_after_s=5.0)

    def shutdown(self, kill_after_s: float = 10.0) -> None:
        if self.failed is None:
            self.failed = "shut down"
        for m in self.muxes:
            if m is not None:
                m.stop()
        t0 = time.monotonic()
        for p in self.procs:
            try:
                p.wait(timeout=max(0.1, kill_after_s - (time.monotonic() - t0)))
            except subprocess.TimeoutExpired:
                p.terminate()          # the exact child this object started
        try:
            self.listener.close()
        except OSError:
            pass


def _free_port() -> int:
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


# ------------------------------------------------------------------------------------------------ worker side
class _ConnQueue:
    """`Request.out` of a request that lives in a worker: chunks go straight to the leader."""

    def __init__(self, conn, rid, lock):
        self.conn, self.rid, self.lock = conn, rid, lock

    def put(self, ch) -> None:
        with self.lock:
            try:
                self.conn.send(("chunk", self.rid, ch))
            except (OSError, EOFError, BrokenPipeError):
                pass


def worker_main(args) -> int:
    """Body of ``plowrt rank-worker``."""
    import datetime
    import torch
    import torch.distributed as dist
    from .. import config as cfgmod
    from ..compiler import packet as pk
    from ..parallel.group import GroupStopped, LeaderGroup, StepGroup, follower_loop
    from ..parallel.health import RankFailure, RankHealth
    from ..runtime.scheduler import ModelMux, SchedConfig
    from ..text.tokenizer import load_tokenizer
    from pathlib import Path

    rank, world, mode = args.rank, args.world, args.mode
    cfg = cfgmod.RuntimeConfig.load(cli=dict(max_slots=args.max_slots, max_ctx=args.max_ctx, backend=args.backend))
    cpu = cfg.backend == "cpu" or not torch.cuda.is_available()
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ["MASTER_PORT"] = str(args.master_port)
    if not cpu:
        torch.cuda.set_device(rank % torch.cuda.device_count())
    store = dist.TCPStore("127.0.0.1", args.master_port, world, is_master=(rank == 0), timeout=datetime.timedelta(seconds=120))
    dist.init_process_group("gloo" if cpu else "nccl", store=store, rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=args.group_timeout),
                            **({} if cpu else {"device_id": torch.device("cuda", torch.cuda.current_device())}))
    health = RankHealth(store, rank, world, timeout_s=args.group_timeout)
    name = "model.pkt" if rank == 0 or mode == "dp" else f"model.rank{rank}.pkt"
    path = Path(args.assets) / name
    if not path.exists():
        path = Path(args.assets) / "model.pkt"
    packet = pk.read_packet(path)
    step_group = leader_group = None
    if mode == "tp":
        leader_group = LeaderGroup(rank, world, timeout_s=args.group_timeout)
    elif mode == "ep":
        step_group = StepGroup(rank, world, timeout_s=args.group_timeout)
    # mode "dp": independent replicas, nothing to agree on
    if cpu:
        from ..runtime.cpu_engine import CpuEngine
        if mode != "dp":
            raise SystemExit("rank-worker: the CPU backend runs data-parallel replicas only (--mode dp)")
        eng = CpuEngine(args.assets, max_slots=cfg.max_slots, max_ctx=cfg.max_ctx, n_pages=cfg.n_pages or None, prefix_cache=cfg.prefix_cache)
    else:
        from ..runtime.gpu_engine import CheckpointWeights, GpuEngine
        comm = tp_comm = None
        shards = packet.section_json("weight_shards.json") or {}
        if shards.get("ep", 1) > 1:
            from ..parallel.ep import EpComm
            from ..models.config import ModelSpec
            spec = ModelSpec.from_json(packet.sections["model.json"].decode())
            comm = EpComm(rank, world, spec, max_rows=max(packet.section_json("serve.json")["buckets"]["prefill"]))
        if shards.get("tp", 1) > 1:
            from ..parallel.tp import TpComm
            tp_comm = TpComm(rank, world)
        eng = GpuEngine(packet=packet, weights=CheckpointWeights(Path(args.assets) / "checkpoint", torch.device("cuda", torch.cuda.current_device()),
                                                                 shards.get("tp", 1), rank),
                        max_slots=cfg.max_slots, max_ctx=cfg.max_ctx, n_pages=cfg.n_pages or None, prefix_cache=cfg.prefix_cache,
                        cuda_graphs=cfg.cuda_graphs, rank=rank, comm=comm, tp_comm=tp_comm, step_group=step_group, leader_group=leader_group)
    if mode == "tp" and rank != 0:
        # follower: replay the leader's steps until it stops
        try:
            follower_loop(eng, leader_group)
        finally:
            dist.destroy_process_group()
        return 0

    tok = load_tokenizer(args.assets)
    mux = ModelMux(eng, tok, SchedConfig(token_budget=min(cfg.token_budget, eng.max_rows(False)), objective=cfg.objective,
                                         queue_ttl_s=cfg.queue_ttl_s, ride=cfg.ride, spec_depth=cfg.spec_depth))
    host, port = args.leader.rsplit(":", 1)
    conn = Client((host, int(port)), authkey=bytes.fromhex(os.environ["PLOW_GROUP_KEY"]))
    send_lock = threading.Lock()
    conn.send(("hello", rank, dict(max_ctx=eng.max_ctx, max_slots=eng.max_slots, n_pages=eng.pool.n_pages, rank=rank, world=world)))
    mux.start()
    live: dict = {}

    def stats_loop():
        while not mux._stop.is_set():
            try:
                health.gate()          # heartbeat + peers' heartbeats + abort flag
            except RankFailure as e:
                eng.health = EngineHealth.DEAD
                if step_group or leader_group:
                    (step_group or leader_group).stopped = True
                print(f"rank-worker {rank}: {e}", file=sys.stderr)
            with send_lock:
                try:
                    conn.send(("stats", dict(live=len(mux.live), waiting=len(mux.waiting), queued=mux.ingress.qsize(),
                                             kv_pages_free=eng.pool.available(), health=eng.health)))
                except (OSError, EOFError, BrokenPipeError):
                    return
            time.sleep(0.25)

    threading.Thread(target=stats_loop, daemon=True).start()
    rc = 0
    try:
        while True:
            try:
                msg = conn.recv()
            except (EOFError, OSError):
                break                                   # the leader is gone: stop the group and exit
            if msg[0] == "submit":
                _, rid, prompt, params = msg
                live[rid] = mux.submit(prompt, params, rid=rid, out=_ConnQueue(conn, rid, send_lock))   # chunks go straight to the leader
            elif msg[0] == "cancel":
                r = live.get(msg[1])
                if r is not None:
                    r.cancelled = True
            elif msg[0] == "call":
                _, seq, what = msg
                val = mux.metrics.snapshot() if what == "metrics" else mux.load_estimate() if what == "load" else None
                with send_lock:
                    conn.send(("ret", seq, val))
            elif msg[0] == "stop":
                break
    finally:
        health.abort("worker stopping") if eng.health == EngineHealth.DEAD else None
        mux.stop()
        try:
            dist.destroy_process_group()
        except Exception:
            rc = rc or 0
    return rc
