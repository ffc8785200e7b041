"""Builds libfa_b200.so in-tree with nvcc for sm_100a (cross-compiles without a GPU).

Usage: python -m flash_attention_b200.csrc.build [--force] [--verbose]
The shared library lands next to this file; object files go to csrc/build/.
"""
import concurrent.futures
import hashlib
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
OUT = os.path.join(HERE, "libfa_b200.so")
OBJ_DIR = os.path.join(HERE, "build")

SOURCES = [
    "fa_api.cu",
    "generic_fwd.cu",
    "generic_bwd.cu",
    "combine.cu",
    "kvcache_prep.cu",
    "rotary.cu",
    "sm100/fwd_tc.cu",
    "sm100/bwd_tc.cu",
    "sm100/bwd_dq_tc.cu",
    "sm100/bwd_wide_tc.cu",
    "sm100/decode.cu",
    "sm100/status.cu",
]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo", "--use_fast_math",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
    "-I", os.path.join(ROOT, "include"),
]


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def _deps_hash(src):
    h = hashlib.sha1()
    paths = [os.path.join(HERE, src), os.path.join(ROOT, "include", "fa_b200.h"), os.path.join(HERE, "fa_common.cuh")]
    sm100 = os.path.join(HERE, "sm100")
    if os.path.isdir(sm100):
        paths += sorted(os.path.join(sm100, f) for f in os.listdir(sm100) if f.endswith(".cuh"))
    for p in paths:
        with open(p, "rb") as f:
            h.update(f.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _compile(src, verbose):
    obj = os.path.join(OBJ_DIR, src.replace("/", "_") + ".o")
    stamp = obj + ".sha1"
    want = _deps_hash(src)
    if os.path.exists(obj) and os.path.exists(stamp) and open(stamp).read() == want:
        return obj, ""
    cmd = [_nvcc(), *NVCC_FLAGS, "-c", os.path.join(HERE, src), "-o", obj]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed for %s:\n%s\n%s" % (src, r.stdout, r.stderr))
    with open(stamp, "w") as f:
        f.write(want)
    return obj, r.stderr


def build(force=False, verbose=False):
    os.makedirs(OBJ_DIR, exist_ok=True)
    if force:
        for f in os.listdir(OBJ_DIR):
            os.remove(os.path.join(OBJ_DIR, f))
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(SOURCES))) as ex:
        results = list(ex.map(lambda s: _compile(s, verbose), SOURCES))
    objs = [o for o, _ in results]
    if verbose:
        for _, log in results:
            if log:
                sys.stderr.write(log)
    newest = max(os.path.getmtime(o) for o in objs)
    if force or not os.path.exists(OUT) or os.path.getmtime(OUT) < newest:
        cmd = [_nvcc(), "-shared", "-o", OUT, *objs, "-gencode", "arch=compute_100a,code=sm_100a"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n%s\n%s" % (r.stdout, r.stderr))
    return OUT


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
