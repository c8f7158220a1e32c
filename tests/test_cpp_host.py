"""The C++ host mirror (include/straydog_b200.hpp): it compiles and links against the library on any machine; on a B200 the
parity program built from it (tests/cpp/host_parity.cpp) holds the library to F64 restatements through the C++ wrappers."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BUILD = os.path.join(ROOT, "tests", "cpp", "_build")
PROGRAM = os.path.join(BUILD, "host_parity")


def compile_program():
    from straydog_b200 import build
    library_dir = os.path.dirname(build.build())
    os.makedirs(BUILD, exist_ok=True)
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    done = subprocess.run(["g++", "-std=c++17", "-O2", "-Wall", "-I", os.path.join(ROOT, "include"), os.path.join(ROOT, "tests", "cpp", "host_parity.cpp"),
                           "-o", PROGRAM, "-L", library_dir, "-lstraydog_gpu_b200", f"-Wl,-rpath,{library_dir}",
                           f"-Wl,-rpath-link,{cuda}/lib64"], capture_output=True, text=True)
    assert done.returncode == 0, done.stderr
    return PROGRAM


def test_the_seam_header_instantiates_with_the_references_call_shapes():
    # include/qsa_b200.hpp: qsa_attention<P> / qsa_attention_rows<P> with the reference's signatures, over stand-in declarations
    from straydog_b200 import build
    library_dir = os.path.dirname(build.build())
    os.makedirs(BUILD, exist_ok=True)
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    done = subprocess.run(["g++", "-std=c++17", "-O1", "-Wall", "-I", os.path.join(ROOT, "include"), os.path.join(ROOT, "tests", "cpp", "seam_compile.cpp"),
                           "-o", os.path.join(BUILD, "seam_compile"), "-L", library_dir, "-lstraydog_gpu_b200", f"-Wl,-rpath,{library_dir}",
                           f"-Wl,-rpath-link,{cuda}/lib64"], capture_output=True, text=True)
    assert done.returncode == 0, done.stderr


def test_the_cpp_mirror_compiles_and_links():
    assert os.path.exists(compile_program())


@pytest.mark.gpu
def test_parity_through_the_cpp_mirror():
    done = subprocess.run([compile_program()], capture_output=True, text=True, timeout=600)
    assert done.returncode == 0 and done.stdout.strip().startswith("ok"), done.stdout + done.stderr
