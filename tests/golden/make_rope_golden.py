"""Builds the reference's host RoPE code on the CPU and records its outputs.

    python tests/golden/make_rope_golden.py REFERENCE_ROOT

Compiles REFERENCE_ROOT/pulsarlm-core/src/kernels/rope.cpp (unmodified, host-only
C++ over ATen) with rope_driver.cpp against the installed libtorch, runs it and
writes tests/golden/rope_reference.json: for each parameter set the reference's
quadrants-per-position table and its rope_rotate() of a fixed input. The tests
compare the plain implementation (and through it the engine) with that file.
This is the one piece of the reference's model code that builds without a GPU;
the rest of the plain implementation rests on the formulas.
"""

import os
import subprocess
import sys
import tempfile

import torch
from torch.utils import cpp_extension


def main() -> None:
    reference = sys.argv[1]
    here = os.path.dirname(os.path.abspath(__file__))
    core = os.path.join(reference, "pulsarlm-core")
    lib_dir = os.path.join(os.path.dirname(torch.__file__), "lib")
    with tempfile.TemporaryDirectory() as tmp:
        exe = os.path.join(tmp, "rope_driver")
        cmd = ["g++", "-std=c++20", "-O1", os.path.join(here, "rope_driver.cpp"),
               os.path.join(core, "src", "kernels", "rope.cpp"), "-I", os.path.join(core, "inc")]
        for inc in cpp_extension.include_paths():
            cmd += ["-isystem", inc]
        cmd += [f"-D_GLIBCXX_USE_CXX11_ABI={int(torch.compiled_with_cxx11_abi())}", "-L", lib_dir,
                "-ltorch", "-ltorch_cpu", "-lc10", f"-Wl,-rpath,{lib_dir}", "-o", exe]
        subprocess.run(cmd, check=True)
        out = subprocess.run([exe], check=True, stdout=subprocess.PIPE, text=True).stdout
    with open(os.path.join(here, "rope_reference.json"), "w") as f:
        f.write(out)
    print(f"wrote {os.path.join(here, 'rope_reference.json')} ({len(out)} bytes)")


if __name__ == "__main__":
    main()
