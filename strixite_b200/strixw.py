"""strixw weight files over the C ABI: the reader (formats/strixw.hpp:96-120 StrixwFile) and the device-resident copy with
the quantized views the MoE kernels take (runtime/strixw_loader.hpp:37-75 StrixwDevice)."""
from __future__ import annotations

import ctypes as C
from typing import Optional

import numpy as np

from . import _lib
from .kernels import Error, _check, _stream

ENCODINGS = {1: "q4", 2: "q4-chunk-major", 3: "bf16", 4: "f32", 5: "i64", 6: "q8", 7: "q8-chunk-major", 8: "q6", 9: "q5"}
DATA, QCODES, SCALE, MIN = 0, 1, 2, 3


class StrixwFile:
    def __init__(self, path: str):
        self.handle = C.c_void_p()
        _check(_lib.load().sxb_strixw_open(str(path).encode(), C.byref(self.handle)))

    def close(self):
        if self.handle:
            _lib.load().sxb_strixw_close(self.handle)
            self.handle = C.c_void_p()

    def __len__(self) -> int:
        return int(_lib.load().sxb_strixw_tensor_count(self.handle))

    @staticmethod
    def _info(t: _lib.SxbStrixwTensor) -> dict:
        return dict(name=t.name.decode(), encoding=ENCODINGS.get(t.encoding, "unknown"), shape=[t.shape[i] for i in range(t.ndim)],
                    group_size=t.group_size, experts=t.experts, n_parts=t.n_parts,
                    components=[dict(role=t.component_role[i], offset=t.component_offset[i], bytes=t.component_bytes[i],
                                     hash=t.component_hash[i]) for i in range(t.n_components)])

    def tensor(self, key) -> dict:
        """By index or by name."""
        t = _lib.SxbStrixwTensor()
        if isinstance(key, int):
            _check(_lib.load().sxb_strixw_tensor(self.handle, key, C.byref(t)))
        else:
            _check(_lib.load().sxb_strixw_find(self.handle, key.encode(), C.byref(t)))
        return self._info(t)

    def parts(self, name: str):
        out = []
        for i in range(self.tensor(name)["n_parts"]):
            src, ro, rows = C.c_char_p(), C.c_int64(), C.c_int64()
            _check(_lib.load().sxb_strixw_part(self.handle, name.encode(), i, C.byref(src), C.byref(ro), C.byref(rows)))
            out.append((src.value.decode(), ro.value, rows.value))
        return out

    def meta(self, key: str) -> Optional[str]:
        v = _lib.load().sxb_strixw_meta(self.handle, key.encode())
        return None if v is None else v.decode()

    def data(self, name: str, role: int) -> np.ndarray:
        """A component's bytes in the mapping, as a uint8 array (a copy)."""
        info = self.tensor(name)
        comp = [c for c in info["components"] if c["role"] == role]
        if not comp:
            raise Error(1, f"tensor '{name}' has no component with role {role}")
        p = _lib.load().sxb_strixw_data(self.handle, name.encode(), role)
        return np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_uint8)), shape=(comp[0]["bytes"],)).copy()

    def verify(self, threads: int = 4):
        _check(_lib.load().sxb_strixw_verify(self.handle, threads))

    def load(self, read_threads: int = 8, stream=None) -> float:
        """Makes the data region resident on the current device; returns the seconds it took."""
        _check(_lib.load().sxb_strixw_load(self.handle, read_threads, _stream(stream)))
        return float(_lib.load().sxb_strixw_load_seconds(self.handle))

    def qview(self, name: str, N: int, K: int):
        """(SxbQView, bits) of a Q4 / Q8 row-major tensor on the device."""
        v, bits = _lib.SxbQView(), C.c_int()
        _check(_lib.load().sxb_strixw_qview(self.handle, name.encode(), N, K, C.byref(v), C.byref(bits)))
        return v, bits.value

    def expert_views(self, name: str, E: int):
        """(routed SxbQView, shared SxbQView or None, bits) of a stacked expert tensor."""
        r, s, bits = _lib.SxbQView(), _lib.SxbQView(), C.c_int()
        _check(_lib.load().sxb_strixw_expert_views(self.handle, name.encode(), E, C.byref(r), C.byref(s), C.byref(bits)))
        return r, (s if s.q else None), bits.value

    def device_ptr(self, name: str, role: int) -> int:
        return int(_lib.load().sxb_strixw_device_ptr(self.handle, name.encode(), role) or 0)
