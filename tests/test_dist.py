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
