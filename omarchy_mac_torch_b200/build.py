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
        cmd = [NVCC, "-shared", "-o", str(out)] + [str(o) for o in objs] + ["-lcudart", "-Xlinker", "-z,defs"] if False else \
              [NVCC, "-shared", "-o", str(out)] + [str(o) for o in objs] + ["-lcudart"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return out


def build_ext(verbose=False):
    """Build the PrivateUse1 torch extension _native in-tree (ninja via torch.utils.cpp_extension)."""
    ext_dir = CSRC / "ext"
    srcs = sorted(str(p) for p in ext_dir.glob("*.cpp"))
    if not srcs:
        return None
    import torch
    from torch.utils import cpp_extension

    lib = build_lib(verbose)
    bdir = OBJ / "ext"
    bdir.mkdir(parents=True, exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    os.environ.setdefault("MAX_JOBS", "8")
    mod = cpp_extension.load(
        name="_native", sources=srcs, build_directory=str(bdir), verbose=verbose, is_python_module=False,
        extra_include_paths=[str(HERE.parent / "include"), str(CSRC)] + cpp_extension.include_paths("cuda"),
        extra_cflags=["-O2", "-std=c++17", "-DOMT_TORCH_VERSION=\"%s\"" % torch.__version__],
        extra_ldflags=[f"-L{LIB}", "-lomt_b200", "-Wl,-rpath,$ORIGIN/lib", "-L/usr/local/cuda/lib64", "-lcudart",
                       "-lc10_cuda", "-ltorch_cuda"],
        with_cuda=True)
    built = bdir / "_native.so"
    dst = HERE / "_native.so"
    if not dst.exists() or dst.stat().st_mtime < built.stat().st_mtime:
        shutil.copy2(built, dst)
    (HERE / "_build_info.json").write_text(json.dumps({"torch": torch.__version__}))
    return dst


def build_all(verbose=False):
    lib = build_lib(verbose)
    ext = build_ext(verbose)
    return lib, ext


if __name__ == "__main__":
    v = "-v" in sys.argv
    print(build_all(v))
