"""Asset distribution: signed, content-addressed asset bundles, a local store with generations, and a registry.

A *bundle* is one compiled model (model.pkt, per-rank packets, build.json, weights.json, tokenizer files; the checkpoint
itself is referenced, not copied, unless ``with_weights``): ``pack`` writes ``<name>-<digest12>.plowpkg`` (a tar) with a
``manifest.json`` (sha256 and size per file, packet content hash, target arch) and, when a signing key is given, an
ed25519 signature over the manifest.  The *store* (``$PLOW_HOME/store``) keeps every loaded bundle as a generation
of its model name; ``load`` verifies and activates, ``rollback`` re-activates the previous generation, ``gc`` removes
inactive generations beyond ``keep``.  A *registry* is a directory (local path; the reference speaks R2/S3, this
environment has no network) with ``catalog.json``; ``publish`` / ``pull`` copy bundles to / from it.
Reference: crates/plowrt/src/dist/ (manifests, pull/load/push/sign, local store with generations), docs/DISTRIBUTION.md."""
from __future__ import annotations

import hashlib
import io
import json
import os
import shutil
import tarfile
import time
from pathlib import Path

BUNDLE_FILES = ("model.pkt", "build.json", "weights.json", "tokenizer.json", "tokenizer_config.json", "chat_template.jinja",
                "generation_config.json", "serve.json")


class DistError(RuntimeError):
    pass


def plow_home() -> Path:
    return Path(os.environ.get("PLOW_HOME", Path.home() / ".plow"))


def _sha256(p: Path) -> str:
    h = hashlib.sha256()
    with open(p, "rb") as f:
        for blk in iter(lambda: f.read(1 << 20), b""):
            h.update(blk)
    return h.hexdigest()


def keygen(path) -> str:
    """Write an ed25519 signing key (hex seed) to ``path``; returns the public key (hex)."""
    from nacl.signing import SigningKey
    sk = SigningKey.generate()
    Path(path).write_text(sk.encode().hex())
    os.chmod(path, 0o600)
    return sk.verify_key.encode().hex()


def _sign(manifest_bytes: bytes, key_path) -> dict:
    from nacl.signing import SigningKey
    sk = SigningKey(bytes.fromhex(Path(key_path).read_text().strip()))
    return {"alg": "ed25519", "public_key": sk.verify_key.encode().hex(), "signature": sk.sign(manifest_bytes).signature.hex()}


def _verify(manifest_bytes: bytes, sig: dict, trusted_keys) -> None:
    from nacl.exceptions import BadSignatureError
    from nacl.signing import VerifyKey
    if trusted_keys is not None and sig["public_key"] not in set(trusted_keys):
        raise DistError("bundle is signed by an untrusted key")
    try:
        VerifyKey(bytes.fromhex(sig["public_key"])).verify(manifest_bytes, bytes.fromhex(sig["signature"]))
    except BadSignatureError:
        raise DistError("bundle signature does not verify")


def pack(assets_dir, out_dir, name: str, key_path=None, with_weights: bool = False) -> Path:
    assets = Path(assets_dir)
    files = [p for p in sorted(assets.iterdir()) if p.is_file() and (p.name in BUNDLE_FILES or p.name.startswith("model.rank"))]
    if not any(p.name == "model.pkt" for p in files):
        raise DistError(f"{assets} holds no model.pkt")
    if with_weights and (assets / "checkpoint").exists():
        files += [p for p in sorted((assets / "checkpoint").resolve().iterdir()) if p.is_file()]
    from ..compiler import packet as pk
    pkt = pk.read_packet(assets / "model.pkt")
    build = json.loads((assets / "build.json").read_text()) if (assets / "build.json").exists() else {}
    entries = [dict(path=("checkpoint/" + p.name) if p.parent != assets else p.name, sha256=_sha256(p), bytes=p.stat().st_size) for p in files]
    manifest = dict(schema=1, name=name, created=int(time.time()), packet_hash=pkt.content_hash.hex(), arch=build.get("arch"),
                    gpu=build.get("gpu"), tp=build.get("tp", 1), ep=build.get("ep", 1), with_weights=bool(with_weights), files=entries)
    mbytes = json.dumps(manifest, sort_keys=True, indent=1).encode()
    digest = hashlib.sha256(mbytes).hexdigest()
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    pkg = out / f"{name}-{digest[:12]}.plowpkg"
    with tarfile.open(pkg, "w") as tar:
        def add_bytes(arc, b):
            ti = tarfile.TarInfo(arc)
            ti.size = len(b)
            tar.addfile(ti, io.BytesIO(b))
        add_bytes("manifest.json", mbytes)
        if key_path:
            add_bytes("manifest.sig", json.dumps(_sign(mbytes, key_path)).encode())
        for p, e in zip(files, entries):
            tar.add(p, arcname=e["path"])
    return pkg


def read_manifest(pkg) -> tuple:
    with tarfile.open(pkg) as tar:
        mbytes = tar.extractfile("manifest.json").read()
        sig = json.loads(tar.extractfile("manifest.sig").read()) if "manifest.sig" in tar.getnames() else None
    return json.loads(mbytes), mbytes, sig


class Store:
    def __init__(self, root=None, trusted_keys=None, require_signature: bool = False):
        self.root = Path(root or plow_home() / "store")
        self.trusted_keys, self.require_signature = trusted_keys, require_signature

    def _state_path(self, name):
        return self.root / name / "state.json"

    def _state(self, name) -> dict:
        p = self._state_path(name)
        return json.loads(p.read_text()) if p.exists() else dict(active=None, previous=None, generations=[])

    def _save(self, name, st) -> None:
        p = self._state_path(name)
        p.parent.mkdir(parents=True, exist_ok=True)
        tmp = p.with_suffix(".tmp")
        tmp.write_text(json.dumps(st, indent=1))
        tmp.replace(p)

    def load(self, pkg) -> Path:
        """Verify a bundle, unpack it as a new generation of its model and activate it."""
        manifest, mbytes, sig = read_manifest(pkg)
        if sig is not None:
            _verify(mbytes, sig, self.trusted_keys)
        elif self.require_signature:
            raise DistError("unsigned bundle refused (store requires signatures)")
        name = manifest["name"]
        gen = hashlib.sha256(mbytes).hexdigest()[:12]
        dst = self.root / name / gen
        if not dst.exists():
            tmp = self.root / name / (gen + ".partial")
            if tmp.exists():
                shutil.rmtree(tmp)
            tmp.mkdir(parents=True)
            with tarfile.open(pkg) as tar:
                for e in manifest["files"]:
                    if e["path"].startswith("/") or ".." in Path(e["path"]).parts:
                        raise DistError(f"unsafe path in bundle: {e['path']}")
                    tar.extract(e["path"], tmp, filter="data")
                    if _sha256(tmp / e["path"]) != e["sha256"]:
                        shutil.rmtree(tmp)
                        raise DistError(f"{e['path']}: content does not match the manifest")
            (tmp / "manifest.json").write_bytes(mbytes)
            tmp.rename(dst)
        st = self._state(name)
        if gen not in st["generations"]:
            st["generations"].append(gen)
        if st["active"] != gen:
            st["previous"], st["active"] = st["active"], gen
        self._save(name, st)
        return dst

    def active(self, name) -> Path:
        st = self._state(name)
        if not st["active"]:
            raise DistError(f"model '{name}' is not in the store")
        return self.root / name / st["active"]

    def ls(self) -> list:
        out = []
        for d in sorted(p for p in self.root.iterdir() if p.is_dir()) if self.root.exists() else []:
            st = self._state(d.name)
            for g in st["generations"]:
                m = json.loads((d / g / "manifest.json").read_text())
                out.append(dict(name=d.name, generation=g, active=g == st["active"], created=m["created"], arch=m.get("arch"),
                                bytes=sum(e["bytes"] for e in m["files"])))
        return out

    def rollback(self, name) -> str:
        st = self._state(name)
        if not st["previous"] or st["previous"] not in st["generations"]:
            raise DistError(f"model '{name}' has no previous generation")
        st["active"], st["previous"] = st["previous"], st["active"]
        self._save(name, st)
        return st["active"]

    def rm(self, name, generation=None) -> None:
        st = self._state(name)
        gens = [generation] if generation else list(st["generations"])
        for g in gens:
            if g == st["active"] and generation:
                raise DistError("the active generation cannot be removed; roll back or remove the whole model")
            shutil.rmtree(self.root / name / g, ignore_errors=True)
            st["generations"].remove(g)
        if not st["generations"]:
            shutil.rmtree(self.root / name, ignore_errors=True)
            return
        if st["previous"] not in st["generations"]:
            st["previous"] = None
        self._save(name, st)

    def prepare(self, name, checkpoint) -> dict:
        """Attach a checkpoint to the active generation of a model that was loaded without its weights: every tensor the
        packets bind by name (directly or through a derived-weight recipe) must be in it; then the generation's
        ``checkpoint`` link points there and the engines can serve from the store."""
        from ..compiler import packet as pk
        from ..runtime import weights
        gen = self.active(name)
        src = Path(checkpoint).resolve()
        if not src.exists():
            raise DistError(f"checkpoint {src} does not exist")
        ckpt = weights.open_checkpoint(src)
        missing = sorted({n for f in sorted(gen.glob("model*.pkt")) for n in weights.missing_weights(pk.read_packet(f), ckpt)})
        if missing:
            raise DistError(f"the checkpoint lacks {len(missing)} tensor(s) the packet binds, e.g. {missing[:3]}")
        link = gen / "checkpoint"
        if link.is_symlink() or link.exists():
            if link.is_symlink():
                link.unlink()
            else:
                raise DistError(f"{gen.name} already carries its weights")
        link.symlink_to(src, target_is_directory=src.is_dir())
        return dict(name=name, generation=gen.name, checkpoint=str(src), packets=len(list(gen.glob("model*.pkt"))))

    def upgrade(self, name, registry: "Registry", target: dict | None = None, dry_run: bool = False, scratch=None) -> dict:
        """Move the model's pin to the newest build in the registry that this machine can run."""
        target = target or host_target()
        found = registry.newest_compatible(name, target)
        if found is None:
            raise DistError(f"the registry has no build of '{name}' for {target.get('arch')}")
        idx, ent = found
        st = self._state(name)
        have = None
        if st["active"]:
            m = json.loads((self.root / name / st["active"] / "manifest.json").read_text())
            have = m.get("created")
        if have is not None and ent["created"] <= have:
            return dict(name=name, upgraded=False, active=st["active"], reason="already at the newest compatible build")
        if dry_run:
            return dict(name=name, upgraded=False, would_load=ent["file"], created=ent["created"])
        import tempfile
        with tempfile.TemporaryDirectory(dir=scratch) as d:
            dst = self.load(registry.pull(name, d, idx))
        return dict(name=name, upgraded=True, active=dst.name, created=ent["created"])

    def gc(self, keep: int = 2) -> list:
        removed = []
        for d in [p for p in self.root.iterdir() if p.is_dir()] if self.root.exists() else []:
            st = self._state(d.name)
            protect = {st["active"], st["previous"]}
            extra = [g for g in st["generations"] if g not in protect]
            for g in extra[:max(0, len(st["generations"]) - keep)]:
                shutil.rmtree(d / g, ignore_errors=True)
                st["generations"].remove(g)
                removed.append((d.name, g))
            self._save(d.name, st)
        return removed


def host_target() -> dict:
    """This machine as a registry sees it: the target a published bundle must name to be selected here."""
    try:
        import torch
        if torch.cuda.is_available():
            p = torch.cuda.get_device_properties(0)
            return dict(arch=f"sm_{p.major}{p.minor}{'a' if p.major >= 9 else ''}", gpu=p.name, gpus=torch.cuda.device_count(),
                        memory_gb=round(p.total_memory / 2 ** 30, 1))
    except Exception:
        pass
    import os
    return dict(arch="cpu", gpu=None, gpus=0, memory_gb=0.0, cpu_threads=os.cpu_count())


def compatible(bundle_arch: str | None, target: dict) -> bool:
    """A bundle runs here when it names this machine's architecture. CPU bundles run anywhere, and a host without a GPU
    takes every bundle: the CPU interpreter executes the same packets."""
    return target.get("arch") == "cpu" or bundle_arch in (None, "cpu", target.get("arch"))


class Registry:
    """A directory of bundles with a catalog (stands in for an object-store bucket)."""

    def __init__(self, root):
        self.root = Path(root)

    def _catalog(self) -> dict:
        p = self.root / "catalog.json"
        return json.loads(p.read_text()) if p.exists() else {}

    def publish(self, pkg) -> dict:
        manifest, mbytes, sig = read_manifest(pkg)
        self.root.mkdir(parents=True, exist_ok=True)
        dst = self.root / Path(pkg).name
        shutil.copyfile(pkg, dst)
        cat = self._catalog()
        ent = dict(file=dst.name, sha256=_sha256(dst), created=manifest["created"], arch=manifest.get("arch"), signed=sig is not None)
        cat.setdefault(manifest["name"], []).append(ent)
        (self.root / "catalog.json").write_text(json.dumps(cat, indent=1))
        return ent

    def catalog(self, show_all: bool = False) -> dict:
        """Listed models and their builds; ``show_all`` adds the unlisted ones."""
        cat = self._catalog()
        hidden = set() if show_all else self._unlisted()
        return {k: v for k, v in cat.items() if k not in hidden}

    def _unlisted(self) -> set:
        p = self.root / "unlisted.json"
        return set(json.loads(p.read_text())) if p.exists() else set()

    def set_listed(self, name, listed: bool) -> list:
        """Leave a model out of listings (it stays published and can be pulled) or show it again."""
        if name not in self._catalog():
            raise DistError(f"'{name}' is not in the registry")
        hidden = self._unlisted()
        (hidden.discard if listed else hidden.add)(name)
        (self.root / "unlisted.json").write_text(json.dumps(sorted(hidden)))
        return sorted(hidden)

    def unpublish(self, name, index: int = -1) -> dict:
        """Take one published build out of the catalog (its bundle file goes once nothing else refers to it)."""
        cat = self._catalog()
        if name not in cat or not cat[name]:
            raise DistError(f"'{name}' is not in the registry")
        ent = cat[name].pop(index)
        if not cat[name]:
            del cat[name]
        if not any(e["file"] == ent["file"] for v in cat.values() for e in v):
            (self.root / ent["file"]).unlink(missing_ok=True)
        (self.root / "catalog.json").write_text(json.dumps(cat, indent=1))
        return ent

    def newest_compatible(self, name, target: dict):
        """(index, entry) of the newest build of ``name`` this machine can run, or None."""
        builds = self._catalog().get(name, [])
        for i in range(len(builds) - 1, -1, -1):
            if compatible(builds[i].get("arch"), target):
                return i, builds[i]
        return None

    def pull(self, name, dest_dir, index: int = -1) -> Path:
        cat = self._catalog()
        if name not in cat:
            raise DistError(f"'{name}' is not in the registry")
        ent = cat[name][index]
        dest = Path(dest_dir)
        dest.mkdir(parents=True, exist_ok=True)
        out = dest / ent["file"]
        shutil.copyfile(self.root / ent["file"], out)
        if _sha256(out) != ent["sha256"]:
            out.unlink()
            raise DistError("downloaded bundle does not match the catalog digest")
        return out
