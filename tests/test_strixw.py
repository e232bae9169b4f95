"""The strixw reader against a file the REFERENCE's own writer produced (tests/golden/tiny.strixw, made by
oracle/ref_strixw_wrap.cpp from the reference's formats/strixw.cpp and quantizers), and the test-side writer against the same
bytes.  No GPU needed: the device-resident copy is covered by tests/test_gpu_strixw.py."""
import ctypes as C
import pathlib
import shutil

import numpy as np
import pytest

ROOT = pathlib.Path(__file__).resolve().parent.parent
GOLDEN = ROOT / "tests" / "golden" / "tiny.strixw"
E, d, I = 3, 64, 32


def pattern(n, salt):
    i = (np.arange(n, dtype=np.uint64) + salt).astype(np.uint32)
    h = ((i * np.uint32(2654435761)) >> np.uint32(8)) & np.uint32(0xFFFF)
    return ((h.astype(np.float32) / np.float32(65536.0) - np.float32(0.5)) * np.float32(0.1)).astype(np.float32)


def golden_tensors(oracle):
    from oracle import strixw_file as S
    gu = oracle.quantize(pattern((E + 1) * 2 * I * d, 1).reshape(-1, d), 64, 4)
    dn = oracle.quantize(pattern(E * d * I, 2).reshape(-1, I), 32, 8)
    router = pattern((E + 1) * d, 3)
    norm = (0x3F80 + np.arange(d)).astype(np.uint16)
    return [
        S.quantized("layers.0.mlp.experts_gate_up", gu, E + 1,
                    [("layers.0.mlp.experts.gate_up_proj", 0, E * 2 * I), ("layers.0.mlp.shared_expert.gate_proj.weight", E * 2 * I, I),
                     ("layers.0.mlp.shared_expert.up_proj.weight", E * 2 * I + I, I)]),
        S.quantized("layers.0.mlp.experts_down", dn, E),
        S.Tensor("layers.0.mlp.router", S.F32, (E + 1, d), {S.DATA: router.tobytes()}),
        S.Tensor("norm", S.BF16, (d,), {S.DATA: norm.tobytes()}),
    ], gu, dn, router, norm


def test_reader_accepts_the_reference_written_file(lib, oracle):
    from strixite_b200.strixw import DATA, MIN, QCODES, SCALE, StrixwFile
    f = StrixwFile(GOLDEN)
    assert len(f) == 4 and f.meta("arch") == "qwen4_exp" and f.meta("absent") is None
    f.verify(3)
    _, gu, dn, router, norm = golden_tensors(oracle)
    t = f.tensor("layers.0.mlp.experts_gate_up")
    assert t["encoding"] == "q4" and t["shape"] == [(E + 1) * 2 * I, d] and t["group_size"] == 64 and t["experts"] == E + 1
    assert [c["role"] for c in t["components"]] == [QCODES, SCALE, MIN]
    assert all(c["offset"] % 256 == 0 for c in t["components"]) and t["components"][0]["offset"] % 4096 == 0
    assert f.parts("layers.0.mlp.experts_gate_up")[1] == ("layers.0.mlp.shared_expert.gate_proj.weight", E * 2 * I, I)
    # the bytes are the reference quantizer's, which the oracle's quantizer reproduces
    assert np.array_equal(f.data("layers.0.mlp.experts_gate_up", QCODES), gu.q.reshape(-1))
    assert np.array_equal(f.data("layers.0.mlp.experts_gate_up", SCALE).view(np.uint16), gu.scale.reshape(-1))
    assert np.array_equal(f.data("layers.0.mlp.experts_down", MIN).view(np.uint16), dn.minv.reshape(-1))
    assert np.array_equal(f.data("layers.0.mlp.router", DATA).view(np.float32), router)
    assert np.array_equal(f.data("norm", DATA).view(np.uint16), norm)
    assert f.tensor(2)["name"] == "layers.0.mlp.router" and f.tensor(3)["encoding"] == "bf16"
    # the component hashes in the index are strix_hash64 of the bytes
    for c, role in zip(t["components"], (QCODES, SCALE, MIN)):
        b = f.data("layers.0.mlp.experts_gate_up", role)
        assert lib.sxb_strix_hash64(b.ctypes.data_as(C.c_void_p), b.size) == c["hash"]
    f.close()


def test_hash_matches_the_test_side_restatement(lib):
    from oracle import strixw_file as S
    rng = np.random.default_rng(4)
    for n in (0, 1, 7, 8, 31, 32, 33, 63, 64, 100, 4097):
        b = rng.integers(0, 256, size=n, dtype=np.uint8)
        assert lib.sxb_strix_hash64(b.ctypes.data_as(C.c_void_p), n) == S.hash64(b.tobytes())


def test_test_side_writer_reproduces_the_reference_bytes(oracle, tmp_path):
    from oracle import strixw_file as S
    tensors, *_ = golden_tensors(oracle)
    out = tmp_path / "mine.strixw"
    S.write(out, {"arch": "qwen4_exp", "made_by": "the reference's StrixwWriter"}, tensors)
    assert out.read_bytes() == GOLDEN.read_bytes()


@pytest.mark.parametrize("where,what", [(9, "format version"), (60, "header hash mismatch"), (130, "index hash mismatch"),
                                        (-1, "truncated"), (-2, "hash mismatch in tensor")])
def test_corruption_is_refused(lib, tmp_path, where, what):
    from strixite_b200.kernels import Error
    from strixite_b200.strixw import StrixwFile
    bad = tmp_path / "bad.strixw"
    raw = bytearray(GOLDEN.read_bytes())
    if where == -1:
        raw = raw[:-100]
    elif where == -2:
        raw[-5] ^= 0x40  # inside the last component: the index still validates, the component hash does not
    else:
        raw[where] ^= 0x01
    bad.write_bytes(raw)
    if where == -2:
        f = StrixwFile(bad)
        with pytest.raises(Error, match=what):
            f.verify(2)
        f.close()
    else:
        with pytest.raises(Error, match=what):
            StrixwFile(bad)


def test_views_need_the_device_copy(lib):
    from strixite_b200.kernels import Error
    from strixite_b200.strixw import StrixwFile
    f = StrixwFile(GOLDEN)
    with pytest.raises(Error, match="not loaded onto the device"):
        f.qview("layers.0.mlp.experts_down", E * d, I)
    with pytest.raises(Error, match="no tensor 'nope'"):
        f.tensor("nope")
    f.close()
