"""Test-side writer of strixw files (formats/strixw.hpp:17-50, formats/strixw.cpp:258-340): header, index and data laid
out exactly as the reference's StrixwWriter lays them out, so that the tests can build weight files of any size.

TEST INFRASTRUCTURE: pinned to the reference by tests/golden/tiny.strixw, which the reference's own writer produced
(oracle/ref_strixw_wrap.cpp) and which this writer must reproduce byte for byte from the same tensors.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass, field
from typing import Dict, List, Sequence, Tuple

import numpy as np

MAGIC = b"STRIXWT\0"
VERSION, HEADER_BYTES, TENSOR_ALIGN, COMPONENT_ALIGN = 4, 128, 4096, 256
Q4, BF16, F32, I64, Q8 = 1, 3, 4, 5, 6
DATA, QCODES, SCALE, MIN = 0, 1, 2, 3
K1, K2, M64 = 0x9E3779B97F4A7C15, 0xD6E8FEB86659FD93, (1 << 64) - 1


def _mix(h: int, w: int) -> int:
    h ^= (w * K1) & M64
    return ((h ^ (h >> 31)) * K2) & M64


def hash64(data: bytes) -> int:
    """strix_hash64 (formats/strixw.cpp:193-244): four multiply-xorshift lanes over 32-byte blocks, seeded by the length."""
    n = len(data)
    h = [n ^ K1, n ^ K2, (~n & M64) ^ K1, (~n & M64) ^ K2]
    full = n // 32 * 32
    if full:
        words = np.frombuffer(data, dtype="<u8", count=full // 8).reshape(-1, 4)
        for lane in range(4):  # a lane's chain is sequential: plain Python integers, one column at a time
            acc = h[lane]
            for w in words[:, lane].tolist():
                acc = _mix(acc, w)
            h[lane] = acc
    tail = data[full:]
    i, lane = 0, 0
    while i + 8 <= len(tail):
        h[lane] = _mix(h[lane], int.from_bytes(tail[i:i + 8], "little"))
        i, lane = i + 8, lane + 1
    if i < len(tail):
        w = int.from_bytes(tail[i:], "little")
        h[0] = _mix(h[0], w ^ ((len(tail) - i) << 56))
    r = _mix(_mix(_mix(h[0], h[1]), h[2]), h[3])
    r ^= r >> 33
    r = (r * K1) & M64
    return r ^ (r >> 29)


@dataclass
class Tensor:
    name: str
    encoding: int
    shape: Sequence[int]
    components: Dict[int, bytes]             # role -> bytes
    group_size: int = 0
    experts: int = 0
    parts: List[Tuple[str, int, int]] = field(default_factory=list)  # (source, row offset, rows)


def quantized(name: str, w, experts: int = 0, parts=()) -> Tensor:
    """A Tensor from an oracle-side QWeight (Q4 or Q8 row-major)."""
    return Tensor(name, Q4 if w.bits == 4 else Q8, (w.N, w.K),
                  {QCODES: np.ascontiguousarray(w.q).tobytes(), SCALE: np.ascontiguousarray(w.scale).tobytes(),
                   MIN: np.ascontiguousarray(w.minv).tobytes()}, w.G, experts, list(parts))


def _align(v: int, a: int) -> int:
    return (v + a - 1) // a * a


def _str16(s: str) -> bytes:
    b = s.encode()
    return struct.pack("<H", len(b)) + b


def write(path, meta: Dict[str, str], tensors: Sequence[Tensor]) -> int:
    """Writes the file; returns its size.  Component order inside a tensor: q, scale, min (or data)."""
    order = {Q4: (QCODES, SCALE, MIN), Q8: (QCODES, SCALE, MIN), BF16: (DATA,), F32: (DATA,), I64: (DATA,)}

    def index(offsets, hashes) -> bytes:
        out = [struct.pack("<I", len(meta))]
        for k in sorted(meta):  # the reference keeps its metadata in a std::map: sorted by key
            v = meta[k].encode()
            out += [_str16(k), struct.pack("<I", len(v)), v]
        out.append(struct.pack("<I", len(tensors)))
        for ti, t in enumerate(tensors):
            out += [_str16(t.name), struct.pack("<BB", t.encoding, len(t.shape))]
            out += [struct.pack("<q", d) for d in t.shape]
            out += [struct.pack("<qq", t.group_size, t.experts), struct.pack("<H", len(t.parts))]
            for src, ro, rows in t.parts:
                out += [_str16(src), struct.pack("<qq", ro, rows)]
            roles = order[t.encoding]
            out.append(struct.pack("<B", len(roles)))
            for ci, role in enumerate(roles):
                out.append(struct.pack("<BQQQ", role, offsets[ti][ci], len(t.components[role]), hashes[ti][ci]))
        return b"".join(out)

    zero = [[0] * 3 for _ in tensors]
    index_bytes = len(index(zero, zero))
    data_offset = _align(HEADER_BYTES + index_bytes, TENSOR_ALIGN)
    cur, offsets, hashes = data_offset, [], []
    for t in tensors:
        cur = _align(cur, TENSOR_ALIGN)
        offs, hs = [], []
        for role in order[t.encoding]:
            cur = _align(cur, COMPONENT_ALIGN)
            offs.append(cur)
            hs.append(hash64(t.components[role]))
            cur += len(t.components[role])
        offsets.append(offs + [0] * (3 - len(offs)))
        hashes.append(hs + [0] * (3 - len(hs)))
    file_bytes = cur
    idx = index(offsets, hashes)
    head = bytearray(HEADER_BYTES)
    head[:8] = MAGIC
    struct.pack_into("<IIQQQQQ", head, 8, VERSION, HEADER_BYTES, HEADER_BYTES, len(idx), data_offset, file_bytes, hash64(idx))
    struct.pack_into("<Q", head, 120, hash64(bytes(head[:120])))
    buf = bytearray(file_bytes)
    buf[:HEADER_BYTES] = head
    buf[HEADER_BYTES:HEADER_BYTES + len(idx)] = idx
    for ti, t in enumerate(tensors):
        for ci, role in enumerate(order[t.encoding]):
            b = t.components[role]
            buf[offsets[ti][ci]:offsets[ti][ci] + len(b)] = b
    with open(path, "wb") as f:
        f.write(buf)
    return file_bytes
