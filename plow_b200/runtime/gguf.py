"""GGUF checkpoints: a reader over a memory map, the block dequantisers the loader needs, a writer, and the adapter that
lets a ``.gguf`` file stand where a safetensors directory does.

* :class:`GgufFile` parses the header (v2 / v3, little endian), every metadata value type, and the tensor catalogue;
  tensor payloads are views into one ``numpy.memmap`` (nothing is copied until a tensor is asked for).
* ``F32``, ``F16``, ``BF16``, ``Q8_0`` (32 values per block: one f16 scale + 32 int8) and ``Q4_0`` (one f16 scale + 16
  bytes of nibbles, value = (nibble - 8) * scale) decode to torch tensors; other quantisations are refused by name.
* :class:`GgufCheckpoint` has the interface of ``runtime.weights.Checkpoint`` and the Hugging Face tensor names: the
  llama.cpp names are mapped (``blk.3.attn_q.weight`` -> ``model.layers.3.self_attn.q_proj.weight`` ...), and the row
  permutation llama.cpp applies to the q / k projections of the llama family (pairs interleaved for its rotary form) is
  undone, so the rest of the system sees the checkpoint it would have seen as safetensors.
* :func:`config_from_gguf` builds the ``config.json`` dictionary from the ``<arch>.*`` metadata keys.
* :func:`write_gguf` writes such a file (used to export and by the tests).

Reference: crates/plowrt/src/asset/gguf.rs (mapped file, catalogue, F16 / F32 / Q8_0 access).
"""
from __future__ import annotations

import struct
from pathlib import Path

import numpy as np
import torch

MAGIC = b"GGUF"
# metadata value types
U8, I8, U16, I16, U32, I32, F32, BOOL, STR, ARR, U64, I64, F64 = range(13)
_SCALAR = {U8: "<B", I8: "<b", U16: "<H", I16: "<h", U32: "<I", I32: "<i", F32: "<f", BOOL: "<?", U64: "<Q", I64: "<q", F64: "<d"}
# tensor types: name -> (id, values per block, bytes per block)
TENSOR_TYPES = {"F32": (0, 1, 4), "F16": (1, 1, 2), "Q4_0": (2, 32, 18), "Q8_0": (8, 32, 34), "BF16": (30, 1, 2)}
_BY_ID = {v[0]: (k, v[1], v[2]) for k, v in TENSOR_TYPES.items()}


class GgufError(ValueError):
    pass


class _Cursor:
    def __init__(self, buf, pos=0):
        self.buf, self.pos = buf, pos

    def take(self, fmt):
        n = struct.calcsize(fmt)
        if self.pos + n > len(self.buf):
            raise GgufError("truncated GGUF header")
        v = struct.unpack_from(fmt, self.buf, self.pos)[0]
        self.pos += n
        return v

    def string(self):
        n = self.take("<Q")
        if self.pos + n > len(self.buf):
            raise GgufError("truncated GGUF string")
        s = bytes(self.buf[self.pos:self.pos + n]).decode("utf-8", errors="replace")
        self.pos += n
        return s

    def value(self, vt):
        if vt in _SCALAR:
            return self.take(_SCALAR[vt])
        if vt == STR:
            return self.string()
        if vt == ARR:
            et, n = self.take("<I"), self.take("<Q")
            if et in _SCALAR and et != BOOL:
                dt = np.dtype(_SCALAR[et])
                nb = dt.itemsize * n
                if self.pos + nb > len(self.buf):
                    raise GgufError("truncated GGUF array")
                a = np.frombuffer(self.buf, dtype=dt, count=n, offset=self.pos).tolist()
                self.pos += nb
                return a
            return [self.value(et) for _ in range(n)]
        raise GgufError(f"unknown GGUF metadata type {vt}")


class GgufTensorInfo:
    def __init__(self, name, shape, ttype, offset):
        self.name, self.shape, self.ttype, self.offset = name, shape, ttype, offset      # shape: outermost first (torch order)
        if ttype not in _BY_ID:
            raise GgufError(f"tensor '{name}': GGUF tensor type {ttype} is not supported (F32, F16, BF16, Q8_0, Q4_0 are)")
        self.type_name, self.block, self.block_bytes = _BY_ID[ttype]
        n = int(np.prod(shape)) if shape else 1
        if shape and shape[-1] % self.block:
            raise GgufError(f"tensor '{name}': row length {shape[-1]} is not a multiple of the {self.type_name} block")
        self.nbytes = n // self.block * self.block_bytes


class GgufFile:
    def __init__(self, path):
        self.path = Path(path)
        self.map = np.memmap(self.path, dtype=np.uint8, mode="r")
        c = _Cursor(self.map)
        if bytes(self.map[:4]) != MAGIC:
            raise GgufError(f"{self.path}: not a GGUF file")
        c.pos = 4
        self.version = c.take("<I")
        if self.version not in (2, 3):
            raise GgufError(f"{self.path}: GGUF version {self.version} is not supported (2 and 3 are)")
        n_tensors, n_kv = c.take("<Q"), c.take("<Q")
        self.metadata: dict = {}
        for _ in range(n_kv):
            k = c.string()
            self.metadata[k] = c.value(c.take("<I"))
        self.tensors: dict[str, GgufTensorInfo] = {}
        for _ in range(n_tensors):
            name = c.string()
            nd = c.take("<I")
            dims = [c.take("<Q") for _ in range(nd)]            # innermost first on disk
            ttype, ofs = c.take("<I"), c.take("<Q")
            self.tensors[name] = GgufTensorInfo(name, tuple(reversed(dims)), ttype, ofs)
        self.alignment = int(self.metadata.get("general.alignment", 32))
        self.data_start = (c.pos + self.alignment - 1) // self.alignment * self.alignment
        for t in self.tensors.values():
            if self.data_start + t.offset + t.nbytes > len(self.map):
                raise GgufError(f"tensor '{t.name}' runs past the end of {self.path}")

    def raw(self, name: str) -> np.ndarray:
        t = self.tensors[name]
        a = self.data_start + t.offset
        return self.map[a:a + t.nbytes]

    def tensor(self, name: str, rows: slice | None = None) -> torch.Tensor:
        """Decoded tensor (f32 for the quantised types and F32, the stored dtype for F16 / BF16); ``rows`` selects a
        range of the outermost axis without decoding the rest."""
        if name not in self.tensors:
            raise KeyError(f"{self.path} has no tensor '{name}'")
        t = self.tensors[name]
        shape = list(t.shape) or [1]
        raw = self.raw(name)
        row_bytes = t.nbytes // shape[0]
        if rows is not None:
            lo, hi, _ = rows.indices(shape[0])
            raw = raw[lo * row_bytes:hi * row_bytes]
            shape[0] = hi - lo
        return _decode(t.type_name, np.ascontiguousarray(raw), shape)


def _decode(type_name: str, raw: np.ndarray, shape) -> torch.Tensor:
    if type_name == "F32":
        return torch.from_numpy(raw.view("<f4").reshape(shape).copy())
    if type_name == "F16":
        return torch.from_numpy(raw.view("<f2").reshape(shape).copy())
    if type_name == "BF16":
        return torch.from_numpy(raw.view("<i2").reshape(shape).copy()).view(torch.bfloat16)
    if type_name == "Q8_0":
        blk = raw.reshape(-1, 34)
        d = blk[:, :2].copy().view("<f2").astype(np.float32)              # [blocks, 1]
        q = blk[:, 2:].view(np.int8).astype(np.float32)                   # [blocks, 32]
        return torch.from_numpy((q * d).reshape(shape))
    if type_name == "Q4_0":
        blk = raw.reshape(-1, 18)
        d = blk[:, :2].copy().view("<f2").astype(np.float32)
        qs = blk[:, 2:]
        q = np.concatenate([qs & 0x0F, qs >> 4], axis=1).astype(np.float32) - 8.0        # low nibbles are values 0..15, high 16..31
        return torch.from_numpy((q * d).reshape(shape))
    raise GgufError(f"no decoder for GGUF tensor type {type_name}")


def _encode(type_name: str, t: torch.Tensor) -> bytes:
    if type_name == "F32":
        return t.float().contiguous().numpy().astype("<f4").tobytes()
    if type_name == "F16":
        return t.to(torch.float16).contiguous().numpy().astype("<f2").tobytes()
    if type_name == "BF16":
        return t.to(torch.bfloat16).contiguous().view(torch.int16).numpy().astype("<i2").tobytes()
    if type_name in ("Q8_0", "Q4_0") and (t.dim() == 0 or t.shape[-1] % 32):
        raise GgufError(f"row length {tuple(t.shape)[-1:] or 1} is not a multiple of the {type_name} block")
    x = t.float().contiguous().numpy().reshape(-1, 32)
    if type_name == "Q8_0":
        d = np.abs(x).max(axis=1, keepdims=True) / 127.0
        q = np.where(d > 0, np.round(x / np.where(d > 0, d, 1.0)), 0.0).astype(np.int8)
        return np.concatenate([d.astype("<f2").view(np.uint8), q.view(np.uint8)], axis=1).tobytes()
    if type_name == "Q4_0":
        idx = np.abs(x).argmax(axis=1)
        mx = x[np.arange(x.shape[0]), idx][:, None]
        d = mx / -8.0
        q = np.clip(np.round(np.where(d != 0, x / np.where(d != 0, d, 1.0), 0.0) + 8.0), 0, 15).astype(np.uint8)
        packed = q[:, :16] | (q[:, 16:] << 4)
        return np.concatenate([d.astype("<f2").view(np.uint8), packed], axis=1).tobytes()
    raise GgufError(f"no encoder for GGUF tensor type {type_name}")


def write_gguf(path, metadata: dict, tensors: dict, types: dict | None = None, alignment: int = 32) -> None:
    """``tensors``: name -> torch tensor; ``types``: name -> "F32" | "F16" | "BF16" | "Q8_0" | "Q4_0" (default F32, or the
    tensor's own 16-bit dtype).  Metadata values: int, float, bool, str, or a list of one of those."""
    types = types or {}

    def s(x: str) -> bytes:
        b = x.encode()
        return struct.pack("<Q", len(b)) + b

    def val(v) -> bytes:
        if isinstance(v, bool):
            return struct.pack("<I?", BOOL, v)
        if isinstance(v, int):
            return struct.pack("<Iq", I64, v) if not 0 <= v < 2 ** 32 else struct.pack("<II", U32, v)
        if isinstance(v, float):
            return struct.pack("<If", F32, v)
        if isinstance(v, str):
            return struct.pack("<I", STR) + s(v)
        if isinstance(v, (list, tuple)):
            if all(isinstance(e, str) for e in v):
                return struct.pack("<IIQ", ARR, STR, len(v)) + b"".join(s(e) for e in v)
            if all(isinstance(e, int) and not isinstance(e, bool) for e in v):
                return struct.pack("<IIQ", ARR, I32, len(v)) + struct.pack(f"<{len(v)}i", *v)
            return struct.pack("<IIQ", ARR, F32, len(v)) + struct.pack(f"<{len(v)}f", *[float(e) for e in v])
        raise GgufError(f"cannot store metadata value {v!r}")
    md = dict(metadata)
    md["general.alignment"] = alignment
    head = MAGIC + struct.pack("<IQQ", 3, len(tensors), len(md))
    for k, v in md.items():
        head += s(k) + val(v)
    blobs, infos, ofs = [], b"", 0
    for name, t in tensors.items():
        tn = types.get(name) or {torch.float16: "F16", torch.bfloat16: "BF16"}.get(t.dtype, "F32")
        b = _encode(tn, t)
        dims = list(reversed(t.shape)) or [1]
        infos += s(name) + struct.pack("<I", len(dims)) + struct.pack(f"<{len(dims)}Q", *dims) + struct.pack("<IQ", TENSOR_TYPES[tn][0], ofs)
        pad = (-len(b)) % alignment
        blobs.append(b + b"\0" * pad)
        ofs += len(b) + pad
    head += infos
    head += b"\0" * ((-len(head)) % alignment)
    with open(path, "wb") as f:
        f.write(head)
        for b in blobs:
            f.write(b)


# ---- names and configuration ------------------------------------------------------------------------------------
_LAYER = {"attn_norm": "input_layernorm", "ffn_norm": "post_attention_layernorm", "attn_q": "self_attn.q_proj",
          "attn_k": "self_attn.k_proj", "attn_v": "self_attn.v_proj", "attn_output": "self_attn.o_proj",
          "attn_q_norm": "self_attn.q_norm", "attn_k_norm": "self_attn.k_norm",
          "ffn_gate": "mlp.gate_proj", "ffn_up": "mlp.up_proj", "ffn_down": "mlp.down_proj"}
_TOP = {"token_embd.weight": "model.embed_tokens.weight", "output_norm.weight": "model.norm.weight", "output.weight": "lm_head.weight"}
_PERMUTED_ARCH = ("llama", "mistral")        # q / k rows are stored pair-interleaved for these architectures


def hf_name(gguf_name: str) -> str | None:
    if gguf_name in _TOP:
        return _TOP[gguf_name]
    p = gguf_name.split(".")
    if len(p) == 4 and p[0] == "blk" and p[2] in _LAYER:
        return f"model.layers.{p[1]}.{_LAYER[p[2]]}.{p[3]}"
    return None


def permute_qk(w: torch.Tensor, n_head: int) -> torch.Tensor:
    """Hugging Face row order -> llama.cpp row order of a q / k projection (per head: the two rotary halves interleaved)."""
    r, c = w.shape
    return w.reshape(n_head, 2, r // n_head // 2, c).transpose(1, 2).reshape(r, c)


def unpermute_qk(w: torch.Tensor, n_head: int) -> torch.Tensor:
    r, c = w.shape
    return w.reshape(n_head, r // n_head // 2, 2, c).transpose(1, 2).reshape(r, c)


def config_from_gguf(g: GgufFile) -> dict:
    md = g.metadata
    arch = md.get("general.architecture")
    if arch not in ("llama", "mistral", "qwen3"):
        raise GgufError(f"GGUF architecture '{arch}' has no mapping to a supported family (llama, mistral, qwen3 have)")

    def key(k, default=None):
        v = md.get(f"{arch}.{k}", default)
        if v is None:
            raise GgufError(f"{g.path}: metadata key {arch}.{k} is missing")
        return v
    n_head = int(key("attention.head_count"))
    hidden = int(key("embedding_length"))
    emb = g.tensors.get("token_embd.weight")
    cfg = dict(model_type=arch, hidden_size=hidden, num_hidden_layers=int(key("block_count")), num_attention_heads=n_head,
               num_key_value_heads=int(key("attention.head_count_kv", n_head)), intermediate_size=int(key("feed_forward_length")),
               head_dim=int(md.get(f"{arch}.attention.key_length", hidden // n_head)),
               rms_norm_eps=float(key("attention.layer_norm_rms_epsilon", 1e-5)), rope_theta=float(key("rope.freq_base", 10000.0)),
               max_position_embeddings=int(key("context_length", 4096)),
               vocab_size=int(md.get(f"{arch}.vocab_size", emb.shape[0] if emb is not None else len(md.get("tokenizer.ggml.tokens", [])))),
               tie_word_embeddings="output.weight" not in g.tensors)
    if "tokenizer.ggml.eos_token_id" in md:
        cfg["eos_token_id"] = int(md["tokenizer.ggml.eos_token_id"])
    if "tokenizer.ggml.bos_token_id" in md:
        cfg["bos_token_id"] = int(md["tokenizer.ggml.bos_token_id"])
    for k, v in md.items():                                   # build-specific keys a checkpoint may carry (dtype of the engine, ...)
        if k.startswith("plow."):
            cfg[k.replace(".", "_", 1)] = v
    return cfg


def find_gguf(path) -> Path | None:
    """The ``.gguf`` file a path stands for: the file itself, or the only one in a directory without safetensors."""
    p = Path(path).resolve()          # an assets directory links its checkpoint: follow the link to the file's own name
    if p.is_file() and p.suffix == ".gguf":
        return p
    if p.is_dir() and not list(p.glob("*.safetensors")):
        files = sorted(p.glob("*.gguf"))
        if len(files) == 1:
            return files[0]
    return None


class GgufCheckpoint:
    """``runtime.weights.Checkpoint`` over a GGUF file, under Hugging Face tensor names."""

    def __init__(self, path):
        self.g = GgufFile(path)
        self.dir = Path(path).parent
        arch = self.g.metadata.get("general.architecture")
        self._permuted = arch in _PERMUTED_ARCH
        self._heads = (int(self.g.metadata.get(f"{arch}.attention.head_count", 0)),
                       int(self.g.metadata.get(f"{arch}.attention.head_count_kv", 0) or self.g.metadata.get(f"{arch}.attention.head_count", 0)))
        self.files = {}
        for name in self.g.tensors:
            h = hf_name(name)
            if h is not None:
                self.files[h] = name

    def names(self):
        return self.files.keys()

    def has(self, name: str) -> bool:
        return name in self.files

    def get(self, name: str) -> torch.Tensor:
        if name not in self.files:
            raise KeyError(f"checkpoint has no tensor '{name}'")
        t = self.g.tensor(self.files[name])
        if self._permuted and t.dim() == 2:
            if name.endswith("self_attn.q_proj.weight"):
                t = unpermute_qk(t, self._heads[0])
            elif name.endswith("self_attn.k_proj.weight"):
                t = unpermute_qk(t, self._heads[1])
        return t

    def get_slice(self, name: str, axis: int, start: int, stop: int) -> torch.Tensor:
        w = self.get(name)            # the q / k permutation mixes rows of a head: slice after undoing it
        return w[start:stop] if axis == 0 else w[:, start:stop]

    def shape(self, name: str) -> tuple:
        return tuple(self.g.tensors[self.files[name]].shape)
