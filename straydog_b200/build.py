"""Compiles the CUDA sources under csrc/ for sm_100a into libstraydog_gpu_b200.so (in-tree).

    python -m straydog_b200.build [--force] [--verbose] [--define NAME ... --out PATH]

nvcc cross-compiles without a GPU. Objects are rebuilt when a source or header is newer.
"""
import concurrent.futures
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "_obj")
LIB = os.path.join(HERE, "libstraydog_gpu_b200.so")
NVCC = os.environ.get("NVCC", "nvcc")
FLAGS = ["-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-Xcompiler", "-fPIC",
         "--expt-relaxed-constexpr", "-Xptxas", "-v"]


def _newest_header() -> float:
    headers = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(HERE, "..", "include", "*.h"))
    return max(os.path.getmtime(h) for h in headers)


def _compile(src: str, force: bool, defines=(), obj_dir: str = OBJ) -> tuple[str, str]:
    obj = os.path.join(obj_dir, os.path.basename(src)[:-3] + ".o")
    if not force and os.path.exists(obj) and os.path.getmtime(obj) >= max(os.path.getmtime(src), _newest_header()):
        return obj, ""
    done = subprocess.run([NVCC, *FLAGS, *[f"-D{name}" for name in defines], "-c", src, "-o", obj], capture_output=True, text=True)
    if done.returncode:
        raise RuntimeError(f"nvcc failed for {src}:\n{done.stdout}\n{done.stderr}")
    return obj, done.stderr


def build(force: bool = False, verbose: bool = False, defines=(), out: str = LIB) -> str:
    """defines + out: a variant build (e.g. --define SDX_TRACE, the kernels' cycle counters) into its own file and object directory."""
    obj_dir = OBJ if out == LIB else out + ".obj"
    os.makedirs(obj_dir, exist_ok=True)
    lib = out
    sources = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
        results = list(pool.map(lambda s: _compile(s, force, defines, obj_dir), sources))
    objects = [obj for obj, _ in results]
    logs = "".join(log for _, log in results)
    if logs:
        with open(os.path.join(obj_dir, "ptxas.log"), "w") as f:
            f.write(logs)
        if verbose:
            print(logs)
    if force or not os.path.exists(lib) or any(os.path.getmtime(o) > os.path.getmtime(lib) for o in objects):
        subprocess.run([NVCC, "-shared", "-o", lib + ".tmp", *objects, "-lcudart"], check=True)
        os.replace(lib + ".tmp", lib)
    return lib


if __name__ == "__main__":
    names = [sys.argv[i + 1] for i, arg in enumerate(sys.argv[:-1]) if arg == "--define"]
    target = sys.argv[sys.argv.index("--out") + 1] if "--out" in sys.argv else LIB
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, defines=names, out=target))
