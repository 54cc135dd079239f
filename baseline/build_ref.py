"""Builds the reference arm's native library, ``baseline/_ref/libsplitrpc_ref.so``.

The original project is a CMake tree whose server needs DPDK, gdrcopy, verbs, ONNX Runtime/TensorRT and an spdlog
submodule that its repository snapshot does not contain, so it cannot be installed as a whole.  What builds offline is
its scatter-gather engine: ``src/transport/g_copy_ng.cu`` and the headers it includes are compiled UNMODIFIED from the
original tree (``--src`` or ``SPLITRPC_REFERENCE_SRC``; default: ``reference/src`` beside this repository) for sm_100a, with two stand-in headers (``spdlog/spdlog.h``:
no-op logging; ``gdrapi.h``: declarations only) and ``ref_harness/ref_driver.cu``, which exports C symbols that call
the original's ``gather_skbs`` / ``scatter_skbs`` / ``sg_on_gpu`` / ``WaitForAppRunComplete``.  The output directory is
git-ignored.  On a machine without the original tree an already built library is used as is.
"""
from __future__ import annotations

import argparse
import hashlib
import shutil
import subprocess
import sys
from pathlib import Path

import os

HERE = Path(__file__).resolve().parent
DEFAULT_SRC = os.environ.get("SPLITRPC_REFERENCE_SRC") or str(HERE.parent.parent / "reference" / "src")
OUT = HERE / "_ref"
LIB = OUT / "libsplitrpc_ref.so"
GENCODE = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _nvcc() -> str:
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found")


def build(src: str = DEFAULT_SRC, force: bool = False) -> Path | None:
    """Returns the library path, or None when it neither exists nor can be built."""
    srcdir = Path(src)
    units = [srcdir / "transport" / "g_copy_ng.cu", HERE / "ref_harness" / "ref_driver.cu"]
    if not units[0].exists():
        return LIB if LIB.exists() else None
    OUT.mkdir(exist_ok=True)
    key = hashlib.sha256(b"".join(u.read_bytes() for u in units)).hexdigest()
    stamp = OUT / "build.stamp"
    if LIB.exists() and stamp.exists() and stamp.read_text() == key and not force:
        return LIB
    inc = [f"-I{srcdir}", f"-I{srcdir / 'utils'}", f"-I{srcdir / 'utils' / 'nv_helpers'}", f"-I{srcdir / 'transport'}",
           f"-I{HERE / 'ref_harness' / 'shims'}"]
    flags = GENCODE + ["-O3", "-std=c++17", "-rdc=true", "-lineinfo", "-w", "-Xcompiler", "-fPIC"]
    objs = []
    for u in units:
        o = OUT / (u.stem + ".o")
        r = subprocess.run([_nvcc(), "-c", str(u), "-o", str(o)] + flags + inc, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"reference build failed for {u}:\n{r.stderr[-4000:]}")
        objs.append(str(o))
    # g_copy_ng.cu has one kernel that calls the device runtime (device-side cudaMemcpyAsync), hence -rdc and cudadevrt
    r = subprocess.run([_nvcc(), "-shared", "-o", str(LIB)] + objs + GENCODE + ["-cudart", "static", "-lcudadevrt"],
                       capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"reference link failed:\n{r.stderr[-4000:]}")
    stamp.write_text(key)
    return LIB


LSTM_LIB = OUT / "libsplitrpc_ref_lstm.so"
LSTM_DIR = OUT / "lstm"  # holds Constant/, copied from the original tree


def build_lstm(src: str = DEFAULT_SRC, force: bool = False) -> Path | None:
    """The original's generated LSTM runtime (``src/apps/nnfusion_lstm/nnfusion_rt.cu``, unmodified) as a library with
    the C entry points of ``ref_harness/ref_lstm_driver.cu``, and a copy of its ``Constant/`` directory beside it.
    Two build-time stand-ins: the shim headers of the copy engine's build, and a force-included header that routes the
    device-side ``cudaDeviceSynchronize`` of its dynamic-parallelism entry point (gone from CUDA 12, never called by
    the harness) to a no-op.  Returns the library path, or None when it neither exists nor can be built."""
    srcdir = Path(src)
    app = srcdir / "apps" / "nnfusion_lstm"
    units = [app / "nnfusion_rt.cu", HERE / "ref_harness" / "ref_lstm_driver.cu"]
    have = LSTM_LIB.exists() and (LSTM_DIR / "Constant").is_dir()
    if not units[0].exists():
        return LSTM_LIB if have else None
    OUT.mkdir(exist_ok=True)
    key = hashlib.sha256(b"".join(u.read_bytes() for u in units)).hexdigest()
    stamp = OUT / "build_lstm.stamp"
    if have and stamp.exists() and stamp.read_text() == key and not force:
        return LSTM_LIB
    shims = HERE / "ref_harness" / "shims"
    inc = [f"-I{srcdir}", f"-I{srcdir / 'utils'}", f"-I{srcdir / 'utils' / 'nv_helpers'}", f"-I{srcdir / 'transport'}", f"-I{app}",
           f"-I{shims}", "-include", str(shims / "cdp_sync_shim.h")]
    flags = GENCODE + ["-O3", "-std=c++17", "-rdc=true", "-lineinfo", "-w", "-Xcompiler", "-fPIC"]
    objs = []
    for u in units:
        o = OUT / (u.stem + ".o")
        r = subprocess.run([_nvcc(), "-c", str(u), "-o", str(o)] + flags + inc, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"reference LSTM build failed for {u}:\n{r.stderr[-4000:]}")
        objs.append(str(o))
    r = subprocess.run([_nvcc(), "-shared", "-o", str(LSTM_LIB)] + objs + GENCODE + ["-cudart", "static", "-lcudadevrt"],
                       capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"reference LSTM link failed:\n{r.stderr[-4000:]}")
    if (LSTM_DIR / "Constant").exists():
        shutil.rmtree(LSTM_DIR / "Constant")
    LSTM_DIR.mkdir(exist_ok=True)
    shutil.copytree(app / "Constant", LSTM_DIR / "Constant")
    stamp.write_text(key)
    return LSTM_LIB


LENET_LIB = OUT / "libsplitrpc_ref_lenet.so"


def build_lenet(src: str = DEFAULT_SRC, force: bool = False) -> Path | None:
    """The original's LeNet (``src/apps/lenet/lenet_vanilla.cu``, unmodified) with the C entry points of
    ``ref_harness/ref_lenet_driver.cu``; same stand-ins as ``build_lstm`` plus a header that maps the NVTX v2 include
    name onto NVTX v3.  Returns the library path, or None when it neither exists nor can be built."""
    srcdir = Path(src)
    app = srcdir / "apps" / "lenet"
    units = [app / "lenet_vanilla.cu", HERE / "ref_harness" / "ref_lenet_driver.cu"]
    if not units[0].exists():
        return LENET_LIB if LENET_LIB.exists() else None
    OUT.mkdir(exist_ok=True)
    key = hashlib.sha256(b"".join(u.read_bytes() for u in units)).hexdigest()
    stamp = OUT / "build_lenet.stamp"
    if LENET_LIB.exists() and stamp.exists() and stamp.read_text() == key and not force:
        return LENET_LIB
    shims = HERE / "ref_harness" / "shims"
    inc = [f"-I{srcdir}", f"-I{srcdir / 'utils'}", f"-I{srcdir / 'utils' / 'nv_helpers'}", f"-I{srcdir / 'transport'}", f"-I{app}",
           f"-I{shims}", "-include", str(shims / "cdp_sync_shim.h")]
    flags = GENCODE + ["-O3", "-std=c++17", "-rdc=true", "-lineinfo", "-w", "-Xcompiler", "-fPIC"]
    objs = []
    for u in units:
        o = OUT / (u.stem + ".o")
        r = subprocess.run([_nvcc(), "-c", str(u), "-o", str(o)] + flags + inc, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"reference LeNet build failed for {u}:\n{r.stderr[-4000:]}")
        objs.append(str(o))
    r = subprocess.run([_nvcc(), "-shared", "-o", str(LENET_LIB)] + objs + GENCODE + ["-cudart", "static", "-lcudadevrt"],
                       capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"reference LeNet link failed:\n{r.stderr[-4000:]}")
    stamp.write_text(key)
    return LENET_LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--src", default=DEFAULT_SRC)
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    p = build(a.src, a.force)
    print(p if p else "unavailable: no original tree and no prebuilt library")
    q = build_lstm(a.src, a.force)
    print(q if q else "LSTM: unavailable: no original tree and no prebuilt library")
    r = build_lenet(a.src, a.force)
    print(r if r else "LeNet: unavailable: no original tree and no prebuilt library")
    sys.exit(0 if p else 1)
