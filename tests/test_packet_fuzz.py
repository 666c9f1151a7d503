"""Mutated packets against both loaders.  A packet with random bytes of its header and tables overwritten must either be
refused with a reason or accepted as a structurally valid packet: never a crash, in the Python reader or the C++ one.
The C++ loader runs in a child process so that a crash would be seen as one (and which mutation caused it)."""
import subprocess
import sys

import numpy as np

from plow_b200.compiler import packet as pk

CHILD = r'''
import ctypes as C, sys
from plow_b200.ops import native
lib = native.cpu_lib()
lib.plow_pkt_open.restype = C.c_void_p
lib.plow_pkt_open.argtypes = [C.c_char_p, C.c_char_p, C.c_int]
lib.plow_pkt_close.argtypes = [C.c_void_p]
lib.plow_cpu_engine_create.restype = C.c_void_p
lib.plow_cpu_engine_create.argtypes = [C.c_void_p, C.c_int]
lib.plow_cpu_engine_destroy.argtypes = [C.c_void_p]
err = C.create_string_buffer(256)
ok = bad = 0
for path in sys.argv[1:]:
    print("open", path, flush=True)
    h = lib.plow_pkt_open(path.encode(), err, 256)
    if h:
        e = lib.plow_cpu_engine_create(h, 2)          # builds the per-program tables the interpreter indexes
        if e:
            lib.plow_cpu_engine_destroy(e)
        lib.plow_pkt_close(h)
        ok += 1
    else:
        assert err.value, "refused without a reason"
        bad += 1
print("done", ok, bad, flush=True)
'''


def test_mutated_packets_are_refused_or_valid_never_fatal(tiny_assets, tmp_path):
    good = tiny_assets / "assets" / "model.pkt"
    raw = good.read_bytes()
    pkt = pk.read_packet(good)
    tables_end = min(len(raw), 1 << 16)                  # header, tensor table, first program's tables: where indices and offsets live
    rng = np.random.default_rng(0)
    paths, py_refused = [], 0
    for k in range(120):
        b = bytearray(raw)
        if k % 4 == 0:                                   # a whole header field
            at = int(rng.integers(8, 120 - 8))
            b[at:at + 8] = rng.integers(0, 256, 8, dtype=np.uint8).tobytes()
        elif k % 4 == 1:                                 # one byte somewhere in the tables
            b[int(rng.integers(0, tables_end))] = int(rng.integers(0, 256))
        elif k % 4 == 2:                                 # a run of 0xFF (the pattern of a half-written table)
            at = int(rng.integers(120, tables_end - 16))
            b[at:at + 16] = b"\xff" * 16
        else:                                            # truncation
            del b[int(rng.integers(64, len(b))):]
        f = tmp_path / f"m{k}.pkt"
        f.write_bytes(bytes(b))
        paths.append(str(f))
        try:
            got = pk.read_packet(f)
            assert len(got.programs) >= 0
        except pk.PacketError:
            py_refused += 1
    assert py_refused >= 40                              # most mutations of indices, offsets and sizes are caught
    r = subprocess.run([sys.executable, "-c", CHILD] + paths, capture_output=True, text=True, timeout=300,
                       cwd=str(good.parent.parent.parent) if False else None, env=None)
    last = [l for l in r.stdout.splitlines() if l.startswith("open")]
    assert r.returncode == 0, f"the C++ loader died on {last[-1] if last else '?'}: rc={r.returncode} {r.stderr[-400:]}"
    done = r.stdout.strip().splitlines()[-1].split()
    assert done[0] == "done" and int(done[1]) + int(done[2]) == len(paths) and int(done[2]) >= 40
    assert len(pkt.programs) > 0
