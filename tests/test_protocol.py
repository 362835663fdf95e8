"""Wire format of the host transport, checked against the real native code.

(The reference's tests/test_protocol.py:10-91 re-implemented the format in Python and never
called the C++; here Python's ``struct``/``zlib`` are the independent oracle.)
"""
import struct
import zlib

import pytest


def test_crc32_known_value(native):
    assert native._crc32(b"123456789") == 0xCBF43926
    assert native._crc32(b"") == 0


@pytest.mark.parametrize("n", [1, 7, 8, 9, 63, 64, 65, 1000, 65537])
def test_crc32_matches_zlib(native, n):
    import random
    rnd = random.Random(n)
    data = bytes(rnd.randrange(256) for _ in range(n))
    assert native._crc32(data) == zlib.crc32(data) & 0xFFFFFFFF


def test_header_is_24_bytes_little_endian(native):
    assert native.HEADER_BYTES == 24
    ops = native._op_codes()
    raw = native._pack_header(ops["ALLREDUCE"], 7, 0x10002, 3, 4096, 3, 0xDEADBEEF)
    assert len(raw) == 24
    ver, op, flags, seq, tid, chunk, nbytes, crc = struct.unpack("<HBBIIIII", raw)
    assert (ver, op, flags, seq, tid, chunk, nbytes, crc) == (5, 1, 3, 7, 0x10002, 3, 4096, 0xDEADBEEF)


def test_op_codes(native):
    ops = native._op_codes()
    assert ops == {"ALLREDUCE": 1, "BROADCAST": 2, "BARRIER": 3, "ALLGATHER": 4, "REDUCE_SCATTER": 5,
                   "SEND": 6, "RECV": 7, "HANDSHAKE": 10, "HEARTBEAT": 11, "ABORT": 255}


def test_handshake_is_74_bytes(native):
    assert native.HANDSHAKE_BYTES == 74
    raw = native._pack_handshake(3, 8, "node-a")
    assert len(raw) == 74
    ver, rank, ws = struct.unpack_from("<HII", raw, 0)
    assert (ver, rank, ws) == (5, 3, 8)
    assert raw[10:16] == b"node-a" and raw[16:] == b"\0" * 58
