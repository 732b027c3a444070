"""Builds libtalos_b200.so in-tree with nvcc for sm_100a (cross-compiles without a GPU).

    python talos-xii_b200/build.py [--force] [--verbose]
"""
import concurrent.futures as cf
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libtalos_b200.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--use_fast_math=false",
         "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall", "-Xptxas", "-v"]
FLAGS = [f for f in FLAGS if f != "--use_fast_math=false"]


def sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith((".cu", ".cpp")))


def _newest_header():
    hdrs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h", ".hpp"))]
    hdrs.append(os.path.join(HERE, "..", "include", "talos_b200.h"))
    return max(os.path.getmtime(h) for h in hdrs)


def _compile(src, force, verbose):
    obj = os.path.join(OBJ, os.path.splitext(src)[0] + ".o")
    path = os.path.join(CSRC, src)
    if not force and os.path.exists(obj) and os.path.getmtime(obj) > max(os.path.getmtime(path), _newest_header()):
        return obj, ""
    cmd = [NVCC] + FLAGS + ["-x", "cu", "-c", path, "-o", obj]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed for %s:\n%s" % (src, r.stdout))
    return obj, r.stdout


def build(force=False, verbose=False):
    os.makedirs(OBJ, exist_ok=True)
    srcs = sources()
    with cf.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        results = list(ex.map(lambda s: _compile(s, force, verbose), srcs))
    objs = [o for o, _ in results]
    if verbose:
        for _, log in results:
            for line in log.splitlines():
                if "registers" in line or "spill" in line or "Compiling entry" in line or "warning" in line:
                    print(line)
    if force or not os.path.exists(LIB) or any(os.path.getmtime(o) > os.path.getmtime(LIB) for o in objs):
        cmd = [NVCC, "-shared", "-o", LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a", "-cudart", "static", "-ldl"]
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n" + r.stdout)
    return LIB


def build_host_tests():
    """Compiles the C++ programs that exercise the host mirror (host/talos.hpp) against the built library."""
    root = os.path.dirname(HERE)
    src_dir = os.path.join(root, "tests", "cpp"); out_dir = os.path.join(src_dir, "bin")
    os.makedirs(out_dir, exist_ok=True)
    hdr_time = max(os.path.getmtime(os.path.join(HERE, "host", h)) for h in os.listdir(os.path.join(HERE, "host")))
    for name in ("test_reference_kats", "host_driver"):
        src = os.path.join(src_dir, name + ".cpp"); out = os.path.join(out_dir, name)
        if os.path.exists(out) and os.path.getmtime(out) > max(os.path.getmtime(src), hdr_time, os.path.getmtime(LIB)):
            continue
        cmd = ["g++", "-std=c++17", "-O2", "-Wall", "-o", out, src, "-L", HERE, "-ltalos_b200", "-Wl,-rpath," + HERE, "-Wl,-rpath,$ORIGIN/../../../talos-xii_b200"]
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if r.returncode != 0:
            raise RuntimeError("g++ failed for %s:\n%s" % (name, r.stdout))
    return out_dir


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
    print(build_host_tests())
