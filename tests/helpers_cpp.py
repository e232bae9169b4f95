"""Builds the C++ host program of tests/cpp against the in-tree library."""
import pathlib
import subprocess

ROOT = pathlib.Path(__file__).resolve().parent.parent


def cuda_home() -> pathlib.Path:
    import shutil
    nvcc = shutil.which("nvcc")
    return pathlib.Path(nvcc).resolve().parent.parent if nvcc else pathlib.Path("/usr/local/cuda")


def build_call_block(out_dir: pathlib.Path) -> pathlib.Path:
    from strixite_b200 import _lib
    lib_dir = _lib.LIB_PATH.parent
    cuda = cuda_home()
    exe = pathlib.Path(out_dir) / "call_block"
    subprocess.run(["g++", "-std=c++20", "-Wall", f"-I{ROOT / 'include'}", f"-I{cuda / 'include'}",
                    str(ROOT / "tests" / "cpp" / "call_block.cpp"), "-o", str(exe), f"-L{lib_dir}", "-lstrix_b200",
                    f"-L{cuda / 'lib64'}", "-lcudart", f"-Wl,-rpath,{lib_dir}", f"-Wl,-rpath,{cuda / 'lib64'}"], check=True)
    return exe
