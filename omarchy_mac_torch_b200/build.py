"""In-tree build of the native code.

  libomt_b200.so   C-ABI runtime + sm_100a kernels (csrc/*.cu), built with nvcc directly; no torch dependency.
  _native*.so      the PyTorch PrivateUse1 extension (csrc/ext/*.cpp) that sits on that C ABI.

Both are written next to the sources (omarchy_mac_torch_b200/lib and the package directory) so the built files travel
with the tree. `python -m omarchy_mac_torch_b200.build` builds everything; nvcc cross-compiles without a GPU."""

import concurrent.futures
import hashlib
import json
import os
import pathlib
import shutil
import subprocess
import sys

HERE = pathlib.Path(__file__).resolve().parent
CSRC = HERE / "csrc"
LIB = HERE / "lib"
OBJ = HERE / "build"
NVCC = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xcompiler", "-fvisibility=default"]
NVCC_FLAGS += os.environ.get("OMT_EXTRA_NVCC_FLAGS", "").split()  # e.g. -DOMT_TC_EXPERIMENTS for the timing experiments in conv_tc.cu


def _stamp(src, flags):
    h = hashlib.sha1()
    h.update(" ".join(flags).encode())
    for p in [src] + sorted(CSRC.glob("*.cuh")) + sorted((HERE.parent / "include").glob("*.h")):
        h.update(p.read_bytes())
    return h.hexdigest()


def _compile(src, verbose):
    OBJ.mkdir(exist_ok=True)
    obj = OBJ / (src.stem + ".o")
    flags = ARCH + NVCC_FLAGS
    stamp_file = OBJ / (src.stem + ".stamp")
    stamp = _stamp(src, flags)
    if obj.exists() and stamp_file.exists() and stamp_file.read_text() == stamp:
        return obj
    cmd = [NVCC] + flags + (["-Xptxas", "-v"] if verbose else []) + ["-c", str(src), "-o", str(obj)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
    if verbose:
        print(r.stderr)
    stamp_file.write_text(stamp)
    return obj


def build_lib(verbose=False):
    """Compile csrc/*.cu for sm_100a and link lib/libomt_b200.so. Returns the path."""
    LIB.mkdir(exist_ok=True)
    srcs = sorted(CSRC.glob("*.cu"))
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(lambda s: _compile(s, verbose), srcs))
    out = LIB / "libomt_b200.so"
    newest = max(o.stat().st_mtime for o in objs)
    if not out.exists() or out.stat().st_mtime < newest:
        cmd = [NVCC, "-shared", "-o", str(out)] + [str(o) for o in objs] + ["-lcudart"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return out


def _compile_cpp(src, flags, verbose):
    bdir = OBJ / "ext"
    bdir.mkdir(parents=True, exist_ok=True)
    obj = bdir / (src.stem + ".o")
    stamp_file = bdir / (src.stem + ".stamp")
    h = hashlib.sha1(" ".join(flags).encode())
    for p in [src] + sorted(src.parent.glob("*.h")) + sorted((HERE.parent / "include").glob("*.h")):
        h.update(p.read_bytes())
    stamp = h.hexdigest()
    if obj.exists() and stamp_file.exists() and stamp_file.read_text() == stamp:
        return obj
    cmd = [os.environ.get("CXX", "g++")] + flags + ["-c", str(src), "-o", str(obj)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"g++ failed for {src.name}:\n{r.stdout}\n{r.stderr}")
    if verbose and r.stderr:
        print(r.stderr)
    stamp_file.write_text(stamp)
    return obj


def build_ext(verbose=False):
    """Build the PrivateUse1 torch extension omarchy_mac_torch_b200/_native.so in-tree (g++, linked against the
    installed torch and lib/libomt_b200.so; found at run time through an $ORIGIN rpath)."""
    ext_dir = CSRC / "ext"
    srcs = sorted(ext_dir.glob("*.cpp"))
    if not srcs:
        return None
    import sysconfig

    import torch
    from torch.utils import cpp_extension

    build_lib(verbose)
    incs = [str(HERE.parent / "include"), str(CSRC)] + cpp_extension.include_paths("cuda") + [sysconfig.get_paths()["include"]]
    flags = ["-O2", "-std=c++17", "-fPIC", "-DTORCH_EXTENSION_NAME=_native", "-DTORCH_API_INCLUDE_EXTENSION_H",
             f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}", "-Wno-deprecated-declarations"]
    flags += [f"-I{i}" for i in incs]
    with concurrent.futures.ThreadPoolExecutor(max_workers=8) as ex:
        objs = list(ex.map(lambda s: _compile_cpp(s, flags, verbose), srcs))
    dst = HERE / "_native.so"
    newest = max(max(o.stat().st_mtime for o in objs), (LIB / "libomt_b200.so").stat().st_mtime)
    if not dst.exists() or dst.stat().st_mtime < newest:
        tlib = str(pathlib.Path(torch.__file__).parent / "lib")
        cmd = [os.environ.get("CXX", "g++"), "-shared", "-o", str(dst)] + [str(o) for o in objs] + [
            f"-L{LIB}", "-lomt_b200", f"-L{tlib}", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
            "-L/usr/local/cuda/lib64", "-lcudart", "-Wl,-rpath,$ORIGIN/lib", f"-Wl,-rpath,{tlib}"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    (HERE / "_build_info.json").write_text(json.dumps({"torch": torch.__version__}))
    return dst


def build_all(verbose=False):
    lib = build_lib(verbose)
    ext = build_ext(verbose)
    return lib, ext


if __name__ == "__main__":
    v = "-v" in sys.argv
    print(build_all(v))
