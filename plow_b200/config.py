"""Runtime configuration and the knob registry.

Every runtime field has a ``PLOW_*`` environment twin; precedence is CLI > environment > default.
Every knob — compile-time ("emit") or runtime — is registered with its layer, domain and
default so ``plowc knob-scope`` / ``plowrt knob-scope`` can list them and the loader can check a
packet's ``build.json`` against the running configuration (reference: crates/plowrt/src/config.rs:1-25,
knob_spec.rs, crates/devgen/src/knob_spec.rs:1335).
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field, fields


@dataclass(frozen=True)
class Knob:
    id: str
    env: str
    layer: str          # emit | runtime
    domain: str         # e.g. "int>=1", "bool", "enum:latency|throughput|auto"
    default: object
    doc: str
    status: str = "stable"


KNOBS = [
    Knob("max_rows", "PLOW_EMIT_MAX_ROWS", "emit", "int>=64", 8192, "largest prefill bucket"),
    Knob("max_seqs", "PLOW_EMIT_MAX_SEQS", "emit", "int>=1", 64, "sequences whose last row a prefill program may sample"),
    Knob("disable_rule", "PLOW_EMIT_DISABLE_RULE", "emit", "list", "", "fusion rules to switch off (comma separated)"),
    Knob("n_cu", "PLOW_EMIT_N_CU", "emit", "int>=1", 148, "compute units the streams are planned for"),
    Knob("host", "PLOW_HOST", "runtime", "str", "127.0.0.1", "bind address"),
    Knob("port", "PLOW_PORT", "runtime", "int", 8000, "bind port"),
    Knob("max_slots", "PLOW_MAX_SLOTS", "runtime", "int>=1", 64, "concurrent sequences"),
    Knob("max_ctx", "PLOW_MAX_CTX", "runtime", "int>=64", 8192, "context bound per sequence"),
    Knob("kv_fraction", "PLOW_KV_FRACTION", "runtime", "float(0,1]", 0.9, "share of free device memory given to KV pages"),
    Knob("n_pages", "PLOW_KV_PAGES", "runtime", "int>=0", 0, "explicit KV page count (0 = derive from kv_fraction)"),
    Knob("prefix_cache", "PLOW_PREFIX_CACHE", "runtime", "bool", True, "share KV pages between prompts with a common prefix"),
    Knob("token_budget", "PLOW_TOKEN_BUDGET", "runtime", "int>=64", 8192, "rows per scheduler tick"),
    Knob("objective", "PLOW_OBJECTIVE", "runtime", "enum:latency|throughput|auto", "auto", "scheduling objective"),
    Knob("tbt_target_ms", "PLOW_TBT_TARGET_MS", "runtime", "float>=0", 0.0, "time-between-tokens budget for prefill sizing"),
    Knob("ride", "PLOW_RIDE", "runtime", "bool", True, "decode rows ride prefill launches (mixed steps)"),
    Knob("spec_depth", "PLOW_SPEC_DEPTH", "runtime", "int>=0", 0, "speculative decoding depth for greedy requests (0 = off)"),
    Knob("spec_drafter", "PLOW_SPEC_DRAFTER", "runtime", "enum:auto|ngram|mtp", "auto",
         "drafter of the speculative steps: the checkpoint's prediction module (assets/mtp, plowc --mtp) or prompt lookup; auto = mtp when compiled"),
    Knob("multi_step", "PLOW_MULTI_STEP", "runtime", "int>=1", 1, "greedy decode steps per engine call (tokens fed back on the device; 1 = off)"),
    Knob("rung_control", "PLOW_RUNG_CONTROL", "runtime", "bool", False, "admission follows the decode-rung controller (widen on backlog / SLO / utilisation, narrow on low load or a faster narrower rung)"),
    Knob("lookahead", "PLOW_LOOKAHEAD", "runtime", "bool", False, "lookahead-1 decode: launch step n+1 (fed on the device) before reading step n's tokens"),
    Knob("device_interp", "PLOW_DEVICE_INTERP", "runtime", "bool", True, "run row-op segments in the persistent on-device interpreter"),
    Knob("pd", "PLOW_PD", "runtime", "bool", False, "prefill/decode disaggregation inside one server (two engines, KV image hand-off)"),
    Knob("queue_ttl_s", "PLOW_QUEUE_TTL_S", "runtime", "float>0", 120.0, "shed queued requests older than this"),
    Knob("dp", "PLOW_DP", "runtime", "int>=1", 1, "data-parallel engine replicas"),
    Knob("api_keys", "PLOW_API_KEYS", "runtime", "list", "", "accepted bearer tokens (empty = open)"),
    Knob("backend", "PLOW_BACKEND", "runtime", "enum:auto|cpu|cuda", "auto", "execution backend"),
    Knob("cuda_graphs", "PLOW_CUDA_GRAPHS", "runtime", "bool", True, "capture decode rungs in CUDA graphs"),
    Knob("trace", "PLOW_TRACE", "runtime", "bool", False, "record a host timeline served at /trace"),
    Knob("step_time", "PLOW_STEP_TIME", "runtime", "bool", False, "CUDA-event time every engine step"),
    Knob("collective_deadline_ms", "PLOW_XR_DEADLINE_MS", "runtime", "int>=1", 1000, "device wait bound for peer flags"),
    Knob("impl", "PLOW_IMPL", "runtime", "enum:fused|nccl", "fused", "collective arm: in-kernel peer memory or NCCL baseline"),
]


def knob_table(layer: str | None = None) -> list:
    return [k.__dict__ for k in KNOBS if layer is None or k.layer == layer]


def _parse(domain: str, raw: str):
    if domain == "bool":
        return raw.lower() in ("1", "true", "yes", "on")
    if domain.startswith("int"):
        return int(raw)
    if domain.startswith("float"):
        return float(raw)
    if domain == "list":
        return [x for x in raw.split(",") if x]
    return raw


def _check(k: Knob, v) -> None:
    d = k.domain
    if d.startswith("enum:") and v not in d[5:].split("|"):
        raise ValueError(f"{k.id}={v!r}: expected one of {d[5:]}")
    if d.startswith("int>=") and int(v) < int(d[5:]):
        raise ValueError(f"{k.id}={v}: must be >= {d[5:]}")
    if d == "float(0,1]" and not (0.0 < float(v) <= 1.0):
        raise ValueError(f"{k.id}={v}: must be in (0, 1]")


@dataclass
class RuntimeConfig:
    values: dict = field(default_factory=dict)

    @staticmethod
    def load(cli: dict | None = None, env: dict | None = None) -> "RuntimeConfig":
        env = os.environ if env is None else env
        cli = cli or {}
        vals = {}
        for k in KNOBS:
            if k.layer != "runtime":
                continue
            if cli.get(k.id) is not None:
                v = cli[k.id]
            elif k.env in env:
                v = _parse(k.domain, env[k.env])
            else:
                v = k.default if k.domain != "list" else []
            _check(k, v)
            vals[k.id] = v
        return RuntimeConfig(vals)

    def replace(self, **kw) -> "RuntimeConfig":
        return RuntimeConfig({**self.values, **kw})

    def __getattr__(self, name):
        try:
            return self.__dict__["values"][name]
        except KeyError:
            raise AttributeError(name)


def check_assets(build: dict, cfg: RuntimeConfig) -> list:
    """Load-time constraint check between a packet's build.json and the runtime knobs."""
    problems = []
    b = build.get("buckets", {})
    if b.get("decode") and cfg.max_slots > max(b["decode"]):
        problems.append(f"max_slots {cfg.max_slots} exceeds the widest decode rung {max(b['decode'])}")
    if b.get("prefill") and cfg.token_budget > max(b["prefill"]):
        problems.append(f"token_budget {cfg.token_budget} exceeds the largest prefill bucket {max(b['prefill'])} (it will be clamped)")
    return problems
