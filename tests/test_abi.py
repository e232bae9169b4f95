"""CPU tests of the drop-in boundary: the library loads, exports every symbol the header declares, and refuses bad
arguments before touching the GPU (the reference's STRIX_CHECK preconditions, returned as codes)."""
import ctypes as C
import pathlib
import re
import subprocess

import pytest

ROOT = pathlib.Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "strix_b200.h"


def declared_symbols():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(sxb_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported_and_bound(lib):
    from strixite_b200 import _lib
    names = declared_symbols()
    assert len(names) >= 30
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in strix_b200.h but not exported by the library"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature in strixite_b200/_lib.py"
    assert set(_lib.SIGNATURES) <= set(names)
    assert lib.sxb_version().decode().endswith("sm_100a")


def test_header_compiles_as_c_and_cxx(tmp_path):
    for lang, std in (("c", "-std=c99"), ("c++", "-std=c++17")):
        src = tmp_path / f"t.{ 'c' if lang == 'c' else 'cpp'}"
        src.write_text('#include "strix_b200.h"\nint main(void) { SxbQView v; (void)v; return SXB_OK; }\n')
        subprocess.run(["gcc", "-x", lang, std, "-fsyntax-only", "-Wall", "-Werror", f"-I{ROOT / 'include'}", str(src)], check=True)


def test_shim_compiles(tmp_path):
    """The header-only C++ shim that re-creates strix::kernels:: over the C ABI."""
    src = tmp_path / "t.cpp"
    src.write_text('#include "strix_b200_shim.hpp"\nint main() { return 0; }\n')
    subprocess.run(["g++", "-std=c++20", "-fsyntax-only", "-Wall", f"-I{ROOT / 'include'}", "-I/usr/local/cuda/include",
                    str(src)], check=True)


def test_cxx_host_links_against_the_library(lib, tmp_path):
    """tests/cpp/call_block.cpp - the reference's call block through the C++ shim - compiles and links against
    libstrix_b200.so (it is run, and its output compared, by the GPU tests)."""
    from helpers_cpp import build_call_block
    exe = build_call_block(tmp_path)
    assert exe.exists()


def test_preconditions_fail_before_any_launch(lib):
    from strixite_b200 import kernels as K
    with pytest.raises(K.Error, match="null pointer"):
        K.moe_router(0, 513, 4, 512, 10, None, 1, 0, 0, 0, K.Act.F32, 0, stream=0)
    with pytest.raises(K.Error, match=r"E = 2000 experts, expected 1\.\.1024"):
        K.moe_router(16, 2000, 4, 2000, 10, None, 1, 0, 16, 32, K.Act.F32, 48, stream=0)
    with pytest.raises(K.Error, match="k = 40"):
        K.moe_router(16, 513, 4, 512, 40, None, 1, 0, 16, 32, K.Act.F32, 48, stream=0)
    with pytest.raises(K.Error, match="ld = 100 < E"):
        K.moe_router(16, 100, 4, 512, 10, None, 1, 0, 16, 32, K.Act.F32, 48, stream=0)
    with pytest.raises(K.Error, match=r"M \* A <= 2\^20"):
        K.moe_route_workspace_bytes(1 << 20, 2, 512)
    with pytest.raises(K.Error, match="workspace of 16 bytes, needs"):
        K.moe_group_routes(16, 16, 10, 512, 32, 16, 48, stream=0)
    with pytest.raises(K.Error, match="overlaps"):
        K.swiglu(4096, 4096 + 64, 4, 64, K.Act.BF16, stream=0)
    with pytest.raises(K.Error, match="H = 3 streams"):
        K.moe_shared_add_inject(4096, 1 << 20, 16, 1, 2, 64, 512, 1 << 24, 32, 3, K.Act.BF16, 48, stream=0)
    assert K.moe_route_workspace_bytes(16, 10, 512) == K.route_layout(16, 10, 512)["total"] * 4


def test_weight_view_checks(lib):
    from strixite_b200 import _lib, kernels as K
    def call(q=4096, scale=8192, minv=12288, N=64, K_=256, G=128, x=1 << 20, y=1 << 24, M=4):
        v = _lib.SxbQView(q, scale, minv, N, K_, G)
        rc = lib.sxb_linear_q4(x, C.byref(v), y, M, 1, 1, None)
        return rc, lib.sxb_last_error().decode()
    assert call(G=48) == (1, call(G=48)[1]) and "group size 48 unsupported" in call(G=48)[1]
    assert "must be a positive multiple of group size" in call(K_=200)[1]
    assert "16-byte aligned" in call(q=4100)[1]
    assert "16-byte aligned" in call(x=(1 << 20) + 2)[1]
    assert "overlaps" in call(y=(1 << 20) + 64)[1]
    assert "M (rows of x) = 0" in call(M=0)[1]
    rc, msg = call(q=0)
    assert rc == 1 and "null weight pointer" in msg
    rc = lib.sxb_linear_q4(1 << 20, C.byref(_lib.SxbQView(4096, 8192, 12288, 64, 256, 128)), 1 << 24, 4, 0, 1, None)
    assert rc == 1 and "output dtype BF16 with input F32 unsupported" in lib.sxb_last_error().decode()


def test_report_errors(lib):
    from strixite_b200 import kernels as K
    K.report_router_error([0, 0, 0], "layer 3")
    with pytest.raises(K.Error, match="layer 3: non-finite router logit at token 7, expert 512"):
        K.report_router_error([1, 7, 512], "layer 3")
    with pytest.raises(K.Error, match="expert id -1 at slot 42"):
        K.report_expert_error([1, 0xFFFFFFFF, 42], "L0")


def test_layer_argument_block_matches_the_header(tmp_path):
    """The ctypes mirror of SxbMoeLayerArgs against the C compiler's layout of the header's struct: size and every offset."""
    from strixite_b200 import _lib
    names = [f[0] for f in _lib.SxbMoeLayerArgs._fields_]
    src = tmp_path / "layout.c"
    body = "\n".join(f'    printf("{n} %zu\\n", offsetof(SxbMoeLayerArgs, {n}));' for n in names)
    src.write_text('#include <stdio.h>\n#include <stddef.h>\n#include "strix_b200.h"\nint main(void) {\n'
                   '    printf("sizeof %zu\\n", sizeof(SxbMoeLayerArgs));\n' + body + "\n    return 0;\n}\n")
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-std=c99", f"-I{ROOT / 'include'}", str(src), "-o", str(exe)], check=True)
    out = dict(line.split() for line in subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.splitlines())
    assert int(out["sizeof"]) == C.sizeof(_lib.SxbMoeLayerArgs)
    for n in names:
        assert int(out[n]) == getattr(_lib.SxbMoeLayerArgs, n).offset, n
    for struct, fields in ((_lib.SxbQView, 6), (_lib.SxbMoeSharedAdd, 5)):
        assert len(struct._fields_) == fields


def test_layer_entry_checks_its_argument_block(lib):
    """sxb_moe_layer refuses a bad argument block before anything is enqueued (no GPU needed)."""
    from strixite_b200 import _lib
    assert lib.sxb_moe_layer(None, None) == 1 and "null argument block" in lib.sxb_last_error().decode()
    a = _lib.SxbMoeLayerArgs()
    assert lib.sxb_moe_layer(C.byref(a), None) == 1 and "null weight view" in lib.sxb_last_error().decode()
    gu, dn = _lib.SxbQView(4096, 8192, 12288, 64 * 2 * 128, 256, 128), _lib.SxbQView(4096, 8192, 12288, 64 * 256, 128, 128)
    a.gate_up, a.down, a.gate_up_bits, a.down_bits = C.pointer(gu), C.pointer(dn), 4, 5
    assert lib.sxb_moe_layer(C.byref(a), None) == 1 and "weight bits 4 / 5" in lib.sxb_last_error().decode()
    a.down_bits = 8
    a.M, a.E, a.A, a.E_total, a.e_lo = 4, 64, 4, 32, 0
    assert lib.sxb_moe_layer(C.byref(a), None) == 1 and "experts [0, 64) of 32" in lib.sxb_last_error().decode()
    a.E_total = 64
    assert lib.sxb_moe_layer(C.byref(a), None) == 1 and "null buffer" in lib.sxb_last_error().decode()


def test_hc_wmma_workspace_sizes_and_preconditions(lib):
    """The workspace sizes of the tensor-core hyper-connection mix are host arithmetic: they hold at least what the
    launchers lay out (grouping workspace, restacked weight, F16 operand, per-slot dots / un-chunked weight, F16 h), grow
    with T, and bad shapes are refused with a message, before any launch."""
    from strixite_b200 import kernels as K
    T, H, d, r = 300, 4, 2560, 320
    R, Rp = r + H, 336
    need = K.hc_wmma_workspace_bytes(T, H, d, R, 8, 64)
    parts = K.moe_route_workspace_bytes(T * H, 1, H) + H * Rp * d + 2 * H * Rp * (d // 64) * 2 + T * H * d * 2 + T * H * Rp * 4
    assert parts <= need <= parts + 8 * 256
    assert K.hc_wmma_workspace_bytes(2 * T, H, d, R, 8, 64) > need
    assert K.hc_wmma_workspace_bytes(T, H, d, R, 4, 64) < need
    up = K.hc_mix_up_wmma_workspace_bytes(T, H, d, r, 4, 32)
    Kp = 384
    parts_up = H * d * Kp // 2 + 2 * H * d * (Kp // 32) * 2 + T * Kp * 2
    assert parts_up <= up <= parts_up + 8 * 256
    for bad in ((0, H, d, R, 8, 64), (T, 3, d, R, 8, 64), (T, H, 100, R, 8, 64), (T, H, d, R, 5, 64), (T, H, d, R, 8, 48), (70000, H, d, R, 8, 64)):
        with pytest.raises(K.Error, match="hc_mix_down_wmma_workspace_bytes"):
            K.hc_wmma_workspace_bytes(*bad)
    with pytest.raises(K.Error, match="hc_mix_up_wmma_workspace_bytes"):
        K.hc_mix_up_wmma_workspace_bytes(T, H, d, 48, 8, 32)
    with pytest.raises(K.Error, match="null pointer"):
        K.hc_inject_inv(0, 4096, 8192, 4, 4, 64, 1e-6, 16384, K.Act.BF16, stream=0)
    with pytest.raises(K.Error, match="eps must be finite"):
        K.hc_inject_inv(1 << 20, 4096, 8192, 4, 4, 64, 0.0, 16384, K.Act.BF16, stream=0)
    with pytest.raises(K.Error, match="y overlaps the streams"):
        K.hc_inject_inv(1 << 20, 4096, (1 << 20) + 64, 4, 4, 64, 1e-6, 16384, K.Act.BF16, stream=0)
