"""Kernel tiers of the CPU interpreter's GEMM (golden / AVX2 / AVX-512 / AMX behind one dispatch): the fp32 tiers agree, the
blocked AVX2 tier is the default where the CPU has it, a whole model gives the same logits on every fp32 tier, and the AMX
tier (bf16 inputs, fp32 accumulation) stays within bf16 distance of them, ragged K / N / row counts included."""
import time

import numpy as np
import pytest

from plow_b200.ops import native
from plow_b200.runtime.cpu_engine import CpuEngine
from plow_b200.runtime.engine import TokenBatch

NAMES = {0: "golden", 1: "avx2", 2: "avx512", 3: "amx"}


def _logits(assets, tier, prompt):
    lib = native.cpu_lib()
    got = lib.plow_cpu_set_tier(tier)
    if got != tier:
        return None, 0.0
    eng = CpuEngine(assets, max_slots=2, max_ctx=512)
    eng.begin_slot(0, prompt)
    eng.reserve(0, len(prompt) + 2)
    t0 = time.perf_counter()
    r = eng.step(TokenBatch(np.asarray(prompt, np.int32), np.arange(len(prompt), dtype=np.int32), np.zeros(len(prompt), np.int32),
                            np.asarray([len(prompt) - 1], np.int32), want_logits=True))
    dt = time.perf_counter() - t0
    eng.close()
    return r.logits[0], dt


def test_gemm_tiers_agree_on_a_whole_model(tiny_assets):
    lib = native.cpu_lib()
    start = lib.plow_cpu_tier()
    assert start in NAMES
    prompt = np.random.default_rng(0).integers(0, 32000, 200).tolist()
    try:
        gold, t_gold = _logits(tiny_assets / "assets", 0, prompt)
        assert gold is not None
        for tier in (1, 2):
            got, dt = _logits(tiny_assets / "assets", tier, prompt)
            if got is None:
                continue                      # this CPU lacks the instruction set: the tier is refused, the old one stays
            rel = float(np.linalg.norm(got - gold) / np.linalg.norm(gold))
            assert rel < 1e-6 and int(got.argmax()) == int(gold.argmax()), (NAMES[tier], rel)
        got, _ = _logits(tiny_assets / "assets", 3, prompt)
        if got is not None:                   # AMX: inputs rounded to bf16
            rel = float(np.linalg.norm(got - gold) / np.linalg.norm(gold))
            assert 1e-5 < rel < 3e-2 and int(got.argmax()) == int(gold.argmax()), rel
        assert lib.plow_cpu_set_tier(7) == lib.plow_cpu_tier()          # out of range: ignored
    finally:
        lib.plow_cpu_set_tier(start)
    # where AVX2 exists it is the default
    if lib.plow_cpu_set_tier(1) == 1:
        lib.plow_cpu_set_tier(start)
        assert start == 1 or __import__("os").environ.get("PLOW_CPU_TIER") not in (None, "auto")


def test_amx_tier_on_ragged_shapes(tmp_path):
    """hidden 528 (K % 32 = 16), intermediate 1400 (K % 32 = 24, per-thread column ranges that are no multiple of 16) and
    a row count that is no multiple of 16: the zero padding of the tile operands leaves the result within bf16 distance."""
    from plow_b200 import plowc
    from plow_b200.models import config, reference
    lib = native.cpu_lib()
    start = lib.plow_cpu_tier()
    if lib.plow_cpu_set_tier(3) != 3:
        lib.plow_cpu_set_tier(start)
        pytest.skip("no AMX on this CPU (or the kernel refused the tile state)")
    cfg = config.tiny_dense_config()
    cfg.update(hidden_size=528, intermediate_size=1400, num_hidden_layers=2)
    reference.write_checkpoint(cfg, tmp_path / "ckpt", seed=1)
    plowc.compile_dir(tmp_path / "ckpt", tmp_path / "assets", arch="cpu", n_cu=8, max_rows=256, decode_rungs=[1, 2], max_seqs=4)
    prompt = np.random.default_rng(1).integers(0, 32000, 77).tolist()
    try:
        gold, _ = _logits(tmp_path / "assets", 0, prompt)
        got, _ = _logits(tmp_path / "assets", 3, prompt)
        rel = float(np.linalg.norm(got - gold) / np.linalg.norm(gold))
        assert np.isfinite(got).all() and rel < 3e-2 and int(got.argmax()) == int(gold.argmax()), rel
        # auto never picks it
        assert start != 3 or __import__("os").environ.get("PLOW_CPU_TIER") == "amx"
    finally:
        lib.plow_cpu_set_tier(start)
