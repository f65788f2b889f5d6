"""In-tree nvcc build of the package's native libraries (sm_100a).  Each library is a list of translation units
under csrc/; objects are cached under build/obj at the repository root and rebuilt when a source or header is
newer.  `ensure(name)` is what the ctypes bindings call: it compiles only the library that is asked for, so the
first use of a model builds what that model needs and nothing else."""
import os
import subprocess
import sys
import tempfile

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
OBJ_DIR = os.path.join(ROOT, "build", "obj")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17", "-Xcompiler", "-fPIC"]

LIBRARIES = {
    # quantized LLaMA decode / prefill kernels (include/b2l.h)
    "llama": dict(out=os.path.join(PKG, "libb200llama.so"),
                  sources=["api.cu", "q_generic.cu", "elementwise.cu", "attention.cu", "q4_tc.cu", "q4_gemv.cu", "q4_gemv_batch.cu",
                           "q8_gemv.cu", "sampling.cu", "decode_mega.cu", "q4_gemm.cu", "tp_allreduce.cu"]),
    # sequence-mixer kernels: recurrences, local and latent attention, expert routing, f32 residual streams (include/b2l_seq.h)
    "seq": dict(out=os.path.join(PKG, "libb200seq.so"),
                sources=["seq_api.cu", "seq_elementwise.cu", "seq_scan.cu", "seq_attention.cu", "seq_latent.cu", "seq_moe.cu", "seq_streams.cu",
                         "seq_depth.cu", "seq_gru.cu", "seq_convrope.cu"]),
}


def nvcc_path() -> str:
    cand = os.environ.get("NVCC")
    if cand:
        return cand
    for c in ("/usr/local/cuda/bin/nvcc",):
        if os.path.exists(c):
            return c
    return "nvcc"


def _headers():
    inc = os.path.join(ROOT, "include")
    return [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))] + \
           [os.path.join(inc, f) for f in os.listdir(inc)]


def compile_unit(src: str, force: bool = False, obj_dir: str = OBJ_DIR) -> str:
    """csrc/<src> -> <obj_dir>/<name>.o (skipped when newer than the source and every header)."""
    os.makedirs(obj_dir, exist_ok=True)
    obj = os.path.join(obj_dir, os.path.splitext(src)[0] + ".o")
    path = os.path.join(CSRC, src)
    if not force and os.path.exists(obj):
        t = os.path.getmtime(obj)
        if all(os.path.getmtime(d) <= t for d in [path] + _headers()):
            return obj
    cmd = [nvcc_path()] + NVCC_FLAGS + ["-c", path, "-o", obj]
    print("[build]", " ".join(cmd), file=sys.stderr)
    subprocess.run(cmd, check=True, stdout=sys.stderr)
    return obj


def link(objs, out: str) -> None:
    if os.path.exists(out) and all(os.path.getmtime(o) <= os.path.getmtime(out) for o in objs):
        return
    fd, tmp = tempfile.mkstemp(dir=os.path.dirname(out), prefix=".link-", suffix=".so")
    os.close(fd)
    cmd = [nvcc_path(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a"] + list(objs) + ["-o", tmp]
    print("[build]", " ".join(cmd), file=sys.stderr)
    try:
        subprocess.run(cmd, check=True, stdout=sys.stderr)
        os.chmod(tmp, 0o755)
        os.replace(tmp, out)   # another process never sees a half-written library
    finally:
        if os.path.exists(tmp):
            os.unlink(tmp)


def build_library(name: str, force: bool = False) -> str:
    from concurrent.futures import ThreadPoolExecutor

    spec = LIBRARIES[name]
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        objs = list(ex.map(lambda s: compile_unit(s, force), spec["sources"]))
    link(objs, spec["out"])
    return spec["out"]


def is_stale(name: str) -> bool:
    spec = LIBRARIES[name]
    if not os.path.exists(spec["out"]):
        return True
    t = os.path.getmtime(spec["out"])
    return any(os.path.getmtime(p) > t for p in [os.path.join(CSRC, s) for s in spec["sources"]] + _headers())


def ensure(name: str) -> str:
    """Path of the built library, compiling it first when it is missing or older than its sources."""
    if is_stale(name):
        build_library(name)
    return LIBRARIES[name]["out"]
