"""Residency manager (LRU eviction inside a memory budget), tuning store and kernel capability registry."""
import pytest


def test_manager_lru_eviction_and_live_protection():
    from plow_b200.serve.manager import ModelManager, ResidencyError
    t = [0.0]
    live = {}
    loaded, unloaded = [], []
    mgr = ModelManager(100, loader=lambda n, p: loaded.append(n) or n, sizer=lambda n, p: {"a": 40, "b": 40, "c": 50, "huge": 500}[n],
                       live_of=lambda e: live.get(e, 0), unloader=lambda e: unloaded.append(e),
                       catalog=dict(a="/a", b="/b", c="/c", huge="/h"), clock=lambda: t[0])
    mgr.acquire("a"); t[0] += 1
    mgr.acquire("b"); t[0] += 1
    mgr.acquire("a"); t[0] += 1                      # touch a: b is now least recently used
    assert mgr.used() == 80 and loaded == ["a", "b"]
    mgr.acquire("c")                                 # needs 50: evicts b only
    assert unloaded == ["b"] and set(mgr.resident) == {"a", "c"} and mgr.evictions == 1
    live["a"] = 2; live["c"] = 1
    with pytest.raises(ResidencyError):
        mgr.acquire("b")                             # nothing idle to evict
    with pytest.raises(ResidencyError):
        mgr.acquire("huge")
    with pytest.raises(ResidencyError):
        mgr.unload("a")
    live.clear()
    mgr.unload("c")
    assert mgr.status()["c"]["state"] == "available" and mgr.status()["a"]["state"] == "resident"
    assert mgr.available() == ["a", "b", "c", "huge"]


def test_packet_bytes_counts_weights_and_kv(tiny_assets):
    from plow_b200.serve.manager import packet_bytes
    small = packet_bytes(tiny_assets / "assets", max_slots=2, max_ctx=128)
    big = packet_bytes(tiny_assets / "assets", max_slots=8, max_ctx=1024)
    assert big > small > 4 * 32000 * 512               # at least the f32 embedding table


def test_tunedb_keeps_fastest(tmp_path):
    from plow_b200.compiler.tunedb import TuneDb, gemm_key
    db = TuneDb(tmp_path, ("nvidia", "sm_100a", "b200"))
    k = gemm_key(64, 7168, 16384, "e4m3")
    assert db.lookup("gemm", k) is None
    assert db.record("gemm", k, dict(bn=64, splits=1), 61.0)
    assert db.record("gemm", k, dict(bn=64, splits=2), 42.6)
    assert not db.record("gemm", k, dict(bn=32, splits=2), 50.0)
    db2 = TuneDb(tmp_path, ("nvidia", "sm_100a", "b200"))
    assert db2.lookup("gemm", k)["config"] == dict(bn=64, splits=2) and db2.keys("gemm") == [k]
    assert (tmp_path / "nvidia" / "sm_100a" / "b200" / "gemm.json").exists()
    with pytest.raises(ValueError):
        db.record("nonsense", k, {}, 1.0)


def test_kernelcaps_select_and_gates():
    from plow_b200.compiler import kernelcaps as kc
    assert kc.select_kernel("attention", "bf16", head_dim=128, group=4).name == "plow_gqa_attention"
    assert kc.select_kernel("attention", "bf16", head_dim=96, group=4) is None
    assert kc.select_kernel("attention", "bf16", head_dim=128, group=3) is None
    assert kc.select_kernel("mla_attention", "e4m3", heads=128, kv_lora=512, qk_rope=64).name == "plow_mla_decode"
    assert kc.select_kernel("mla_attention", "e4m3", heads=64, kv_lora=512, qk_rope=64) is None
    assert kc.select_kernel("linear", "bf16", isa_caps=("mma_sync",)) is None          # no tcgen05: nothing fits
    rep = kc.apply_ptxas_report("""ptxas info    : Compiling entry function '_ZN4plow14gemm_tc_kernelILi64ELb1ELb0ELb1EEEvNS_8GemmArgsE' for 'sm_100a'
ptxas info    : Function properties for _ZN4plow14gemm
    16 bytes stack frame, 40 bytes spill stores, 56 bytes spill loads
ptxas info    : Used 255 registers, used 1 barriers, 1168 bytes smem
ptxas info    : Compiling entry function 'tiny' for 'sm_100a'
    0 bytes stack frame, 0 bytes spill stores, 0 bytes spill loads
ptxas info    : Used 32 registers, used 0 barriers""")
    assert rep["tiny"]["regs"] == 32 and rep["_ZN4plow14gemm_tc_kernelILi64ELb1ELb0ELb1EEEvNS_8GemmArgsE"]["spill"] == 40
    assert kc.resource_gate(rep, max_spill=16) == ["_ZN4plow14gemm_tc_kernelILi64ELb1ELb0ELb1EEEvNS_8GemmArgsE"]

    class Lib:
        plow_gemm = 1
    assert kc.probe(Lib())["plow_gemm"] and not kc.probe(Lib())["plow_gdn"]
