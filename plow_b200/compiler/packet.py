"""Python view of the packet ABI (``csrc/common/plow_packet.h``): writer, reader, validator.

The struct formats below are locked against the C++ header by ``tests/test_packet_abi.py``
(sizeof / opcode values are read back from ``libplow_cpu.so``), the same way the reference
locks its Rust mirror against ``dev_isa.h`` (crates/packet/tests/dev_abi.rs).
"""
from __future__ import annotations

import hashlib
import json
import struct
from dataclasses import dataclass, field
from enum import IntEnum
from pathlib import Path

MAGIC = b"PLOWB200"
VERSION = 3
CTR_STRIDE_U32 = 32
KV_PAGE = 64
T_NONE = 0xFFFF
EXPERT_UNUSED = 0xFFFFFFFF
U64_MAX = 0xFFFFFFFFFFFFFFFF


class Op(IntEnum):
    NOP = 0
    EMBED = 1
    RMSNORM = 2
    ADD_NORM = 3
    GEMM = 4
    ROPE_KV = 5
    ATTN = 6
    ROW_GATHER = 7
    ARGMAX = 8
    SAMPLE = 9
    RESIDUAL = 10
    GLU = 11
    QUANT_ACT = 12
    MLA_KV_WRITE = 20
    MLA_Q_ROPE = 21
    MLA_DECODE = 22
    MLA_PREFILL = 23
    MLA_ABSORB_Q = 24
    MLA_FOLD_V = 25
    DSA_INDEX = 30
    DSA_TOPK = 31
    ROUTER_TOPK = 40
    MOE_ALIGN = 41
    MOE_GATHER = 42
    MOE_GEMM = 43
    MOE_COMBINE = 44
    GDN_CONV = 50
    GDN_GATES = 51
    GDN_STEP = 52
    GDN_CHUNK = 53
    GATED_NORM = 54
    SIGMOID_GATE = 55
    XREDUCE = 60
    XREDUCE_ADD_NORM = 61
    XGATHER = 62
    XREDUCE_SCATTER = 63
    XA2A_DISPATCH = 64
    XA2A_COMBINE = 65
    XARGMAX_FIN = 66
    GEMM_XREDUCE = 67
    XGATHER_GEMM = 68


OP_COUNT = 69

GEMM_DUAL_SILU, GEMM_FP8_BLOCK, GEMM_OUT_F32, GEMM_RESIDUAL, GEMM_QUANT_OUT = 1, 2, 4, 8, 16
GEMM_ACT_GELU_TANH, GEMM_ACT_GELU_ERF = 32, 64          # with DUAL: the gate's activation when it is not SiLU
GEMM_BIAS = 128                                         # t7 holds a bias [N], added before the store
ACT_FLAGS = {"silu": 0, "gelu_tanh": GEMM_ACT_GELU_TANH, "gelu": GEMM_ACT_GELU_ERF}
ATTN_CAUSAL, ATTN_DECODE = 0, 1


class DType(IntEnum):
    F32 = 0
    BF16 = 1
    F16 = 2
    E4M3 = 3
    I32 = 4
    U8 = 5
    I64 = 6


DTYPE_BYTES = {DType.F32: 4, DType.BF16: 2, DType.F16: 2, DType.E4M3: 1, DType.I32: 4, DType.U8: 1, DType.I64: 8}


class TClass(IntEnum):
    WEIGHT = 0
    DERIVED = 1
    GEN = 2
    KV = 3
    STATE = 4
    ACT = 5
    INPUT = 6
    OUTPUT = 7
    PEER = 8


class Role(IntEnum):
    PREFILL = 0
    DECODE = 1
    MIXED = 2


# struct formats (little endian, no implicit padding)
F_INST = "<HH3I8H8I"
F_STREAM = "<IHHIIHHI"
F_WAIT = "<II"
F_TRACE = "<IIIIQQQ"
F_HEADER = "<8sIIIIII7Q32s"
F_TENSOR = "<IHHHHI4qQQ"
F_PROGRAM = "<10I7Q"
F_SECTION = "<IIQQ"

SIZES = {
    "PlowInst": struct.calcsize(F_INST), "PlowStreamEnt": struct.calcsize(F_STREAM),
    "PlowWait": struct.calcsize(F_WAIT), "PlowTraceRec": struct.calcsize(F_TRACE),
    "PlowPktHeader": struct.calcsize(F_HEADER), "PlowTensorEnt": struct.calcsize(F_TENSOR),
    "PlowProgramEnt": struct.calcsize(F_PROGRAM), "PlowSectionEnt": struct.calcsize(F_SECTION),
}


def f2u(x: float) -> int:
    return struct.unpack("<I", struct.pack("<f", float(x)))[0]


def u2f(x: int) -> float:
    return struct.unpack("<f", struct.pack("<I", int(x) & 0xFFFFFFFF))[0]


@dataclass
class Inst:
    op: int
    nslice: int = 1
    f: tuple = (0.0, 0.0, 0.0)
    t: list = field(default_factory=lambda: [T_NONE] * 8)
    i: list = field(default_factory=lambda: [0] * 8)

    def __post_init__(self):
        # always eight operand and eight immediate slots, as in the packed form: an instruction built by the emitter
        # and one read back from a packet file index the same way
        self.t = list(self.t) + [T_NONE] * (8 - len(self.t))
        self.i = list(self.i) + [0] * (8 - len(self.i))

    def pack(self) -> bytes:
        t = list(self.t) + [T_NONE] * (8 - len(self.t))
        i = [int(v) & 0xFFFFFFFF for v in list(self.i) + [0] * (8 - len(self.i))]
        return struct.pack(F_INST, int(self.op), self.nslice, *[f2u(v) for v in self.f], *t, *i)

    @staticmethod
    def unpack(b: bytes) -> "Inst":
        v = struct.unpack(F_INST, b)
        return Inst(op=v[0], nslice=v[1], f=tuple(u2f(x) for x in v[2:5]), t=list(v[5:13]), i=list(v[13:21]))


@dataclass
class StreamEnt:
    inst: int
    slice0: int
    nslice: int
    wait_ofs: int
    succ_ofs: int
    n_wait: int
    n_succ: int
    seg: int = 0

    def pack(self) -> bytes:
        return struct.pack(F_STREAM, self.inst, self.slice0, self.nslice, self.wait_ofs, self.succ_ofs,
                           self.n_wait, self.n_succ, self.seg)

    @staticmethod
    def unpack(b: bytes) -> "StreamEnt":
        return StreamEnt(*struct.unpack(F_STREAM, b))


@dataclass
class TensorEnt:
    name: str
    dtype: int
    tclass: int
    dims: tuple           # -1 stands for the program's row count
    shard_axis: int = 0xFFFFFFFF
    flags: int = 0
    arena_ofs: int = 0
    bytes: int = 0

    def nbytes(self, rows: int) -> int:
        n = DTYPE_BYTES[DType(self.dtype)]
        for d in self.dims:
            n *= rows if d == -1 else d
        return n


@dataclass
class Program:
    role: int
    rows: int
    rank: int
    n_cu: int
    insts: list
    stream: list          # StreamEnt, concatenated per CU
    cu_ofs: list          # n_cu + 1
    waits: list           # (ctr, target)
    succs: list           # ctr ids
    n_ctr: int
    n_seg: int
    actmap: list          # per tensor arena offset or U64_MAX
    arena_bytes: int


@dataclass
class Packet:
    tensors: list
    programs: list
    sections: dict        # name -> bytes
    n_cu: int
    content_hash: bytes = b""

    def tensor_index(self, name: str) -> int:
        for i, t in enumerate(self.tensors):
            if t.name == name:
                return i
        raise KeyError(name)

    def section_json(self, name: str):
        return json.loads(self.sections[name].decode()) if name in self.sections else None

    def find_program(self, role: int, rows: int, rank: int = 0):
        """Smallest program of `role` on `rank` covering `rows`."""
        best = None
        for p in self.programs:
            if p.role == role and p.rank == rank and p.rows >= rows and (best is None or p.rows < best.rows):
                best = p
        return best


class PacketError(ValueError):
    pass


def write_packet(pkt: Packet, path) -> bytes:
    """Serialise and return the content hash."""
    strtab = bytearray()
    str_ofs = {}

    def s(name: str) -> int:
        if name not in str_ofs:
            str_ofs[name] = len(strtab)
            strtab.extend(name.encode() + b"\0")
        return str_ofs[name]

    hdr = SIZES["PlowPktHeader"]
    body = bytearray()

    def put(b: bytes, align: int = 16) -> int:
        pad = (-(hdr + len(body))) % align
        body.extend(b"\0" * pad)
        ofs = hdr + len(body)
        body.extend(b)
        return ofs

    tens_b = bytearray()
    for t in pkt.tensors:
        dims = list(t.dims) + [1] * (4 - len(t.dims))
        tens_b += struct.pack(F_TENSOR, s(t.name), t.dtype, t.tclass, len(t.dims), t.flags, t.shard_axis,
                              *dims, t.arena_ofs, t.bytes)
    tensor_ofs = put(bytes(tens_b))

    prog_ents = []
    for p in pkt.programs:
        inst_ofs = put(b"".join(i.pack() for i in p.insts), 64)
        stream_ofs = put(b"".join(e.pack() for e in p.stream))
        cu_ofs = put(struct.pack(f"<{len(p.cu_ofs)}I", *p.cu_ofs))
        wait_ofs = put(b"".join(struct.pack(F_WAIT, c, tg) for c, tg in p.waits))
        succ_ofs = put(struct.pack(f"<{len(p.succs)}I", *p.succs))
        actmap_ofs = put(struct.pack(f"<{len(p.actmap)}Q", *p.actmap))
        prog_ents.append(struct.pack(F_PROGRAM, p.role, p.rows, p.rank, len(p.insts), len(p.stream),
                                     len(p.waits), len(p.succs), p.n_ctr, p.n_cu, p.n_seg, inst_ofs,
                                     stream_ofs, cu_ofs, wait_ofs, succ_ofs, actmap_ofs, p.arena_bytes))
    program_ofs = put(b"".join(prog_ents))

    sec_ents = []
    for name, blob in pkt.sections.items():
        ofs = put(blob)
        sec_ents.append(struct.pack(F_SECTION, s(name), 4, ofs, len(blob)))
    section_ofs = put(b"".join(sec_ents))
    strtab_ofs = put(bytes(strtab))
    file_bytes = hdr + len(body)
    digest = hashlib.sha256(bytes(body)).digest()
    arena = max([p.arena_bytes for p in pkt.programs] + [0])
    header = struct.pack(F_HEADER, MAGIC, VERSION, hdr, len(pkt.tensors), len(pkt.programs),
                         len(pkt.sections), pkt.n_cu, tensor_ofs, program_ofs, section_ofs, strtab_ofs,
                         len(strtab), file_bytes, arena, digest)
    Path(path).write_bytes(header + bytes(body))
    pkt.content_hash = digest
    return digest


def read_packet(path) -> Packet:
    """Parse and validate (every index / offset is range-checked before use; the reference's
    loader applies the same list, docs/arch/04-packet-abi.md:105-122)."""
    raw = Path(path).read_bytes()
    hs = SIZES["PlowPktHeader"]
    if len(raw) < hs:
        raise PacketError("truncated header")
    (magic, version, header_bytes, n_tensor, n_program, n_section, n_cu, tensor_ofs, program_ofs,
     section_ofs, strtab_ofs, strtab_bytes, file_bytes, _arena, digest) = struct.unpack(F_HEADER, raw[:hs])
    if magic != MAGIC:
        raise PacketError("bad magic")
    if version != VERSION:
        raise PacketError(f"packet version {version}, runtime understands {VERSION}")
    if header_bytes != hs or file_bytes != len(raw):
        raise PacketError("size mismatch")
    if hashlib.sha256(raw[hs:]).digest() != digest:
        raise PacketError("content hash mismatch")

    def span(ofs, n):
        if ofs < hs or ofs + n > len(raw):
            raise PacketError("offset out of range")
        return raw[ofs:ofs + n]

    strtab = span(strtab_ofs, strtab_bytes)

    def name(o):
        if o >= len(strtab):
            raise PacketError("string offset out of range")
        return strtab[o:strtab.index(b"\0", o)].decode()

    tensors = []
    ts = SIZES["PlowTensorEnt"]
    for k in range(n_tensor):
        v = struct.unpack(F_TENSOR, span(tensor_ofs + k * ts, ts))
        rank = v[3]
        if rank > 4:
            raise PacketError("tensor rank > 4")
        tensors.append(TensorEnt(name=name(v[0]), dtype=v[1], tclass=v[2], dims=tuple(v[6:6 + rank]),
                                 shard_axis=v[5], flags=v[4], arena_ofs=v[10], bytes=v[11]))
    programs = []
    ps = SIZES["PlowProgramEnt"]
    for k in range(n_program):
        v = struct.unpack(F_PROGRAM, span(program_ofs + k * ps, ps))
        (role, rows, rank, n_inst, n_stream, n_wait, n_succ, n_ctr, p_cu, n_seg, inst_ofs, stream_ofs,
         cu_ofs, wait_ofs, succ_ofs, actmap_ofs, arena_bytes) = v
        insts = [Inst.unpack(span(inst_ofs + 64 * j, 64)) for j in range(n_inst)]
        stream = [StreamEnt.unpack(span(stream_ofs + 24 * j, 24)) for j in range(n_stream)]
        cu = list(struct.unpack(f"<{p_cu + 1}I", span(cu_ofs, 4 * (p_cu + 1))))
        waits = [struct.unpack(F_WAIT, span(wait_ofs + 8 * j, 8)) for j in range(n_wait)]
        succs = list(struct.unpack(f"<{n_succ}I", span(succ_ofs, 4 * n_succ)))
        actmap = list(struct.unpack(f"<{n_tensor}Q", span(actmap_ofs, 8 * n_tensor)))
        prog = Program(role, rows, rank, p_cu, insts, stream, cu, waits, succs, n_ctr, n_seg, actmap, arena_bytes)
        validate_program(prog, n_tensor)
        programs.append(prog)
    sections = {}
    ss = SIZES["PlowSectionEnt"]
    for k in range(n_section):
        no, kind, ofs, nb = struct.unpack(F_SECTION, span(section_ofs + k * ss, ss))
        sections[name(no)] = span(ofs, nb)
    pkt = Packet(tensors, programs, sections, n_cu, digest)
    check_must_understand(pkt)
    return pkt


def validate_program(p: Program, n_tensor: int) -> None:
    if p.cu_ofs[0] != 0 or p.cu_ofs[-1] != len(p.stream) or any(a > b for a, b in zip(p.cu_ofs, p.cu_ofs[1:])):
        raise PacketError("cu_ofs is not a monotone cover of the stream")
    for ins in p.insts:
        if ins.op >= OP_COUNT:
            raise PacketError(f"unknown opcode {ins.op}")
        for h in ins.t:
            if h != T_NONE and h >= n_tensor:
                raise PacketError("tensor handle out of range")
    covered = [0] * len(p.insts)
    for e in p.stream:
        if e.inst >= len(p.insts):
            raise PacketError("stream entry names a missing instruction")
        if e.slice0 + e.nslice > p.insts[e.inst].nslice:
            raise PacketError("stream entry slice range exceeds the instruction")
        if e.wait_ofs + e.n_wait > len(p.waits) or e.succ_ofs + e.n_succ > len(p.succs):
            raise PacketError("wait/succ range out of bounds")
        covered[e.inst] += e.nslice
    for k, ins in enumerate(p.insts):
        if covered[k] != ins.nslice:
            raise PacketError(f"instruction {k} slices covered {covered[k]} times of {ins.nslice}")
    for c, _ in p.waits:
        if c >= p.n_ctr:
            raise PacketError("wait counter out of range")
    for c in p.succs:
        if c >= p.n_ctr:
            raise PacketError("succ counter out of range")


UNDERSTOOD_SECTIONS = {"abi.json", "serve.json", "live_kv", "recurrent_state", "derived_weights.json",
                       "weight_shards.json", "segment_roles.json", "build.json", "model.json", "moe_ep.json",
                       "decode_objects.json", "spec.json"}


def check_must_understand(pkt: Packet) -> None:
    """abi.json lists sections a loader must understand to run the packet safely (the
    reference's contract: crates/plow-asset/src/abi.rs:27-36)."""
    abi = pkt.section_json("abi.json")
    if not abi:
        return
    for sec in abi.get("must_understand", []):
        if sec not in UNDERSTOOD_SECTIONS:
            raise PacketError(f"packet requires section '{sec}' which this runtime does not understand")
        if sec not in pkt.sections:
            raise PacketError(f"abi.json names section '{sec}' but the packet does not carry it")
