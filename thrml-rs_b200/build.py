"""In-tree build of libthrml_b200.so with nvcc for sm_100a (cross-compiles without a GPU).

Each source is compiled to an object under `_obj/` (in parallel, only when it or a header changed) and the objects are
linked into the shared library beside this file.
"""
import os
import subprocess
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "_obj")
OUT = os.path.join(HERE, "libthrml_b200.so")
SOURCES = ["engine.cu", "lattice.cu", "potts.cu", "comm.cu", "compile_device.cu", "builder.cpp"]
HEADERS = ["tables.h", "ctx.h", "comm.h", "devbuf.h", "dense.cuh", "device_math.cuh", "update_kernels.cuh", "observer_kernels.cuh",
           os.path.join("..", "..", "include", "thrml_b200.h")]
FLAGS = ["-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-Xcompiler", "-fPIC,-fvisibility=default"]


def _newest_header() -> float:
    return max(os.path.getmtime(os.path.join(CSRC, h)) for h in HEADERS)


def _obj_path(src: str) -> str:
    return os.path.join(OBJ, os.path.splitext(src)[0] + ".o")


def _stale_sources(force: bool):
    newest = _newest_header()
    out = []
    for src in SOURCES:
        obj = _obj_path(src)
        if force or not os.path.exists(obj) or os.path.getmtime(obj) < max(newest, os.path.getmtime(os.path.join(CSRC, src))):
            out.append(src)
    return out


def build(force: bool = False, verbose: bool = False) -> str:
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    os.makedirs(OBJ, exist_ok=True)
    todo = _stale_sources(force)
    if not todo and os.path.exists(OUT) and all(os.path.getmtime(OUT) >= os.path.getmtime(_obj_path(s)) for s in SOURCES):
        return OUT

    def compile_one(src):
        cmd = [nvcc] + FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", os.path.join(CSRC, src), "-o", _obj_path(src)]
        subprocess.run(cmd, check=True)

    with ThreadPoolExecutor(max_workers=len(SOURCES)) as pool:
        list(pool.map(compile_one, todo))
    # NCCL is resolved with dlopen when the first communicator call is made, so the library links against libdl only
    subprocess.run([nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", OUT] + [_obj_path(s) for s in SOURCES] + ["-ldl"], check=True)
    return OUT


if __name__ == "__main__":
    import sys
    print(build(force=True, verbose="-v" in sys.argv))
