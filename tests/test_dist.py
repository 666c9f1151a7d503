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
    # unlist drops the newest entry and its file; the older build is found again
    ent = reg.unlist("tiny")
    assert ent["created"] == 2000 and not (reg.root / ent["file"]).exists() and len(reg.catalog()["tiny"]) == 1
    reg.unlist("tiny")
    assert "tiny" not in reg.catalog()
    with pytest.raises(d.DistError):
        reg.unlist("tiny")
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
