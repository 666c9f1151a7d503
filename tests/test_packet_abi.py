"""ABI lock: the Python view of the packet must agree with the C++ header byte for byte."""
import ctypes as C

import pytest

from plow_b200.compiler import packet as pk
from plow_b200.ops import native


def _lib():
    lib = native.cpu_lib()
    lib.plow_abi_sizeof.restype = C.c_uint64
    lib.plow_abi_sizeof.argtypes = [C.c_char_p]
    lib.plow_abi_constant.restype = C.c_int
    lib.plow_abi_constant.argtypes = [C.c_char_p]
    return lib


def test_struct_sizes():
    lib = _lib()
    for name, size in pk.SIZES.items():
        assert lib.plow_abi_sizeof(name.encode()) == size, name
    assert pk.SIZES["PlowInst"] == 64 and pk.SIZES["PlowStreamEnt"] == 24 and pk.SIZES["PlowWait"] == 8


def test_opcodes_and_constants():
    lib = _lib()
    for op in pk.Op:
        assert lib.plow_abi_constant(f"PLOW_OP_{op.name}".encode()) == int(op), op.name
    assert lib.plow_abi_constant(b"PLOW_OP__COUNT") == pk.OP_COUNT
    assert lib.plow_abi_constant(b"PLOW_PKT_VERSION") == pk.VERSION
    assert lib.plow_abi_constant(b"PLOW_CTR_STRIDE_U32") == pk.CTR_STRIDE_U32
    assert lib.plow_abi_constant(b"PLOW_KV_PAGE") == pk.KV_PAGE
    assert lib.plow_abi_constant(b"PLOW_T_NONE") == pk.T_NONE
    for tc in pk.TClass:
        assert lib.plow_abi_constant(f"PLOW_TC_{tc.name}".encode()) == int(tc)
    for name in ("DUAL_SILU", "FP8_BLOCK", "OUT_F32", "RESIDUAL", "QUANT_OUT"):
        assert lib.plow_abi_constant(f"PLOW_GEMM_{name}".encode()) == getattr(pk, f"GEMM_{name}")


def test_inst_roundtrip():
    i = pk.Inst(op=pk.Op.GEMM, nslice=7, f=(1e-6, 2.5, -1.0), t=[1, 2, 3], i=[4096, 512, 3])
    b = i.pack()
    assert len(b) == 64
    j = pk.Inst.unpack(b)
    assert j.op == pk.Op.GEMM and j.nslice == 7 and j.t[:3] == [1, 2, 3] and j.t[3] == pk.T_NONE
    assert j.i[:3] == [4096, 512, 3] and abs(j.f[0] - 1e-6) < 1e-12


def test_cpp_reader_accepts_and_rejects(tiny_assets, tmp_path):
    lib = native.cpu_lib()
    lib.plow_pkt_open.restype = C.c_void_p
    lib.plow_pkt_open.argtypes = [C.c_char_p, C.c_char_p, C.c_int]
    lib.plow_pkt_close.argtypes = [C.c_void_p]
    err = C.create_string_buffer(256)
    good = tiny_assets / "assets" / "model.pkt"
    h = lib.plow_pkt_open(str(good).encode(), err, 256)
    assert h
    lib.plow_pkt_close(h)
    raw = bytearray(good.read_bytes())
    # corrupt the magic, a table offset, and truncate: every one must be refused with a reason
    for mutate in (lambda b: b.__setitem__(0, 0x58), lambda b: b.__setitem__(slice(32, 40), b"\xff" * 8),
                   lambda b: b.__delitem__(slice(len(b) - 100, len(b)))):
        bad = bytearray(raw)
        mutate(bad)
        f = tmp_path / "bad.pkt"
        f.write_bytes(bytes(bad))
        assert not lib.plow_pkt_open(str(f).encode(), err, 256)
        assert err.value
        with pytest.raises(pk.PacketError):
            pk.read_packet(f)


def test_must_understand(tiny_assets, tmp_path):
    import json
    pkt = pk.read_packet(tiny_assets / "assets" / "model.pkt")
    abi = pkt.section_json("abi.json")
    abi["must_understand"].append("future_section")
    pkt.sections["abi.json"] = json.dumps(abi).encode()
    pk.write_packet(pkt, tmp_path / "x.pkt")
    with pytest.raises(pk.PacketError, match="future_section"):
        pk.read_packet(tmp_path / "x.pkt")
