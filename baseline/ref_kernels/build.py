"""Builds the reference's kernel library (cosmonomic/pulsarlm, pulsarlm-core/src/kernels) as a
Python extension under baseline/_ref/, from the reference's unmodified sources.

    python baseline/ref_kernels/build.py [--reference /path/to/reference]

The reference's own build (xmake, target "pulsarlm_kernels", pulsarlm-core/xmake.lua:34-48)
compiles src/kernels/*.cu and *.cpp as C++20 against libtorch. This script does the same
for the files the Llama path uses with nvcc and torch's extension builder. One file is
left out: paged_attention.cu (attn_decode_cuda, write_kv_cuda) fails with g++ 13
("'HD' is not captured", paged_attention.cu:613; the reference requires gcc 15).
The whole-model engine (src/engine, C++23) is not built. The result serves two ends:
golden outputs of the reference's kernels for the plain implementation under tests/, and
same-device timings of its prompt attention kernel beside this package's.
"""

from __future__ import annotations

import argparse
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
OUT = os.path.join(ROOT, "baseline", "_ref", "kernels")
NAME = "pulsarlm_ref_kernels"
SOURCES = ["rmsnorm.cu", "rope.cu", "rope.cpp", "moe_routing.cu", "paged_common.cu", "paged_prefill.cu",
           "gumbel_race.cu"]


def load(reference: str | None = None, build: bool = True):
    """The extension module; built first when missing and `build` is set."""
    import torch  # noqa: F401  (the extension links against it)
    from torch.utils import cpp_extension

    reference = reference or os.environ.get("PULSARLM_REFERENCE") or os.path.join(os.path.expanduser("~"), "reference")
    built = os.path.join(OUT, NAME + ".so")
    if os.path.isfile(built):
        import importlib.util

        spec = importlib.util.spec_from_file_location(NAME, built)
        module = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(module)
        return module
    if not build:
        raise FileNotFoundError(f"{built} is not built; run python baseline/ref_kernels/build.py")
    core = os.path.join(reference, "pulsarlm-core")
    if not os.path.isdir(core):
        raise FileNotFoundError(f"no reference checkout at {reference}")
    os.makedirs(OUT, exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    return cpp_extension.load(
        name=NAME,
        sources=[os.path.join(HERE, "binding.cpp")] + [os.path.join(core, "src", "kernels", s) for s in SOURCES],
        extra_include_paths=[os.path.join(core, "inc")],
        extra_cflags=["-O2", "-std=c++20"],
        extra_cuda_cflags=["-O2", "-std=c++20", "--expt-relaxed-constexpr", "--expt-extended-lambda",
                           "-gencode", "arch=compute_100a,code=sm_100a"],
        build_directory=OUT,
        verbose=True,
    )


if __name__ == "__main__":
    p = argparse.ArgumentParser()
    p.add_argument("--reference", default=None)
    args = p.parse_args()
    module = load(args.reference)
    print("built", module.__file__ if hasattr(module, "__file__") else module)
    sys.exit(0)
