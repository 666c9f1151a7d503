"""Signed asset bundles, the local store with generations and the directory registry."""
import json
import tarfile

import pytest


def test_pack_sign_load_rollback_gc(tiny_assets, tmp_path):
    from plow_b200.dist import store as d
    key = tmp_path / "sign.key"
    pub = d.keygen(key)
    pkg = d.pack(tiny_assets / "assets", tmp_path / "out", "tiny", key_path=key)
    manifest, mbytes, sig = d.read_manifest(pkg)
    assert manifest["name"] == "tiny" and any(e["path"] == "model.pkt" for e in manifest["files"]) and sig["public_key"] == pub
    st = d.Store(tmp_path / "store", trusted_keys=[pub], require_signature=True)
    g1 = st.load(pkg)
    assert (g1 / "model.pkt").exists() and st.active("tiny") == g1
    # a second generation (different manifest: another name of the creation time is enough)
    pkg2 = d.pack(tiny_assets / "assets", tmp_path / "out2", "tiny", key_path=key, with_weights=True)
    g2 = st.load(pkg2)
    assert g2 != g1 and st.active("tiny") == g2 and (g2 / "checkpoint" / "config.json").exists()
    assert [e["active"] for e in st.ls()] .count(True) == 1
    assert st.rollback("tiny") == g1.name and st.active("tiny") == g1
    with pytest.raises(d.DistError):
        st.rm("tiny", g1.name)                       # active
    assert st.gc(keep=2) == []
    st.rm("tiny")
    assert st.ls() == []


def test_tampered_and_untrusted_bundles_are_refused(tiny_assets, tmp_path):
    from plow_b200.dist import store as d
    key = tmp_path / "k"
    pub = d.keygen(key)
    pkg = d.pack(tiny_assets / "assets", tmp_path / "o", "tiny", key_path=key)
    with pytest.raises(d.DistError):
        d.Store(tmp_path / "s1", trusted_keys=["00" * 32]).load(pkg)               # unknown signer
    unsigned = d.pack(tiny_assets / "assets", tmp_path / "o2", "tiny")
    with pytest.raises(d.DistError):
        d.Store(tmp_path / "s2", require_signature=True).load(unsigned)
    # flip one byte of a payload file inside the tar: digest check fails
    bad = tmp_path / "bad.plowpkg"
    with tarfile.open(pkg) as src, tarfile.open(bad, "w") as dst:
        for m in src.getmembers():
            data = src.extractfile(m).read()
            if m.name == "build.json":
                data = data.replace(b"{", b"{ ", 1)
                m.size = len(data)
            import io
            dst.addfile(m, io.BytesIO(data))
    with pytest.raises(d.DistError):
        d.Store(tmp_path / "s3", trusted_keys=[pub]).load(bad)


def test_registry_publish_pull(tiny_assets, tmp_path):
    from plow_b200.dist import store as d
    pkg = d.pack(tiny_assets / "assets", tmp_path / "o", "tiny")
    reg = d.Registry(tmp_path / "registry")
    ent = reg.publish(pkg)
    assert reg.catalog()["tiny"][0]["sha256"] == ent["sha256"]
    got = reg.pull("tiny", tmp_path / "dl")
    assert d.read_manifest(got)[0]["name"] == "tiny"
    with pytest.raises(d.DistError):
        reg.pull("nope", tmp_path / "dl")


def test_unlist_upgrade_and_target(tiny_assets, tmp_path, monkeypatch):
    import time as _time
    from plow_b200.dist import store as d
    reg = d.Registry(tmp_path / "registry")
    st = d.Store(tmp_path / "store")
    clock = [1000]
    monkeypatch.setattr(d.time, "time", lambda: clock[0])
    old = d.pack(tiny_assets / "assets", tmp_path / "o1", "tiny")
    reg.publish(old)
    st.load(old)
    first = st.active("tiny")
    assert st.upgrade("tiny", reg)["upgraded"] is False          # the store already holds the newest build
    clock[0] = 2000
    new = d.pack(tiny_assets / "assets", tmp_path / "o2", "tiny", with_weights=True)
    reg.publish(new)
    dry = st.upgrade("tiny", reg, dry_run=True)
    assert dry["upgraded"] is False and dry["created"] == 2000 and st.active("tiny") == first
    got = st.upgrade("tiny", reg)
    assert got["upgraded"] is True and st.active("tiny") != first and st.active("tiny").name == got["active"]
    # a machine of another architecture finds nothing to move to
    arch = reg.catalog()["tiny"][-1]["arch"]
    assert d.compatible(arch, d.host_target())
    if arch not in (None, "cpu"):
        with pytest.raises(d.DistError):
            st.upgrade("tiny", reg, target=dict(arch="sm_90a"))
    # unlisted: out of the listing, still published and pullable; listed again on request
    assert reg.set_listed("tiny", False) == ["tiny"]
    assert "tiny" not in reg.catalog() and "tiny" in reg.catalog(show_all=True)
    assert d.read_manifest(reg.pull("tiny", tmp_path / "dl2"))[0]["name"] == "tiny"
    assert reg.set_listed("tiny", True) == [] and "tiny" in reg.catalog()
    # unpublish drops the newest entry and its file; the older build is found again
    ent = reg.unpublish("tiny")
    assert ent["created"] == 2000 and not (reg.root / ent["file"]).exists() and len(reg.catalog()["tiny"]) == 1
    reg.unpublish("tiny")
    assert "tiny" not in reg.catalog()
    with pytest.raises(d.DistError):
        reg.unpublish("tiny")
    t = d.host_target()
    assert t["arch"] == "cpu" or t["arch"].startswith("sm_")


def test_cli_target_and_op_audit(tiny_assets, capsys):
    from plow_b200 import plowrt
    assert plowrt.main(["target", "--json"]) == 0
    assert "arch" in json.loads(capsys.readouterr().out)
    assert plowrt.main(["op-audit", "--table", "--format", "json"]) == 0
    rows = json.loads(capsys.readouterr().out)
    assert all(r["cls"] for r in rows) and any(r["op"] == "GEMM" and r["cpu"] for r in rows)
    assert plowrt.main(["op-audit", str(tiny_assets / "assets"), "--format", "json"]) == 0
    out = json.loads(capsys.readouterr().out)
    assert out["cpu"]["ok"] and out["cpu"]["unclassified"] == []
    assert plowrt.main(["op-audit", str(tiny_assets / "assets"), "--program", "1"]) == 0
    assert "[cpu] ok=True" in capsys.readouterr().out


def test_prepare_attaches_a_checkpoint_to_a_weightless_generation(tiny_assets, tmp_path):
    """A bundle packed without weights is loaded, then `prepare` checks the checkpoint against the names the packet binds
    and links it in; a checkpoint that lacks a tensor is refused and nothing is linked; the CPU engine serves from the store."""
    import shutil
    import numpy as np
    from safetensors.torch import load_file, save_file
    from plow_b200.dist import store as d
    from plow_b200.runtime.cpu_engine import CpuEngine
    from plow_b200.runtime.engine import TokenBatch
    st = d.Store(tmp_path / "store")
    st.load(d.pack(tiny_assets / "assets", tmp_path / "o", "tiny"))
    gen = st.active("tiny")
    assert not (gen / "checkpoint").exists()
    bad = tmp_path / "bad"
    shutil.copytree(tiny_assets / "ckpt", bad)
    f = next(bad.glob("*.safetensors"))
    sd = load_file(f)
    dropped = next(k for k in sd if k.endswith("layers.1.self_attn.k_proj.weight"))
    save_file({k: v for k, v in sd.items() if k != dropped}, f)
    idx = bad / "model.safetensors.index.json"
    if idx.exists():
        j = json.loads(idx.read_text())
        j["weight_map"].pop(dropped, None)
        idx.write_text(json.dumps(j))
    with pytest.raises(d.DistError, match="lacks 1 tensor"):
        st.prepare("tiny", bad)
    assert not (gen / "checkpoint").exists()
    got = st.prepare("tiny", tiny_assets / "ckpt")
    assert got["generation"] == gen.name and (gen / "checkpoint").is_symlink()
    eng = CpuEngine(gen, max_slots=2, max_ctx=128)
    eng.begin_slot(0, [1, 2, 3])
    eng.reserve(0, 8)
    r = eng.step(TokenBatch(np.asarray([1, 2, 3], np.int32), np.arange(3, dtype=np.int32), np.zeros(3, np.int32), np.asarray([2], np.int32),
                            want_logits=True))
    eng.close()
    assert np.isfinite(r.logits[0]).all()
