"""TEST INFRASTRUCTURE ONLY - compiles the reference's two CUDA extensions for sm_100 from the
sources where they lie (the checkout given on the command line or in QLKA_REFERENCE_DIR), into oracle/_ref/ (git-ignored; binaries only,
no reference source is copied). The reference's setup.py is not used: this is a direct
torch.utils.cpp_extension build of its csrc files with its own flags (-O3 --use_fast_math,
Weighted_*_Sum/setup.py:20-26) and an sm_100 target, which the reference's default arch list
lacks (setup.py:6).

    python oracle/build_ref.py /path/to/reference

`load_ref()` imports the built modules (on the GPU box the sources are absent; only the
prebuilt .so files are used). They serve as a second parity checker for the GPU tests and
as a GPU-side comparison point; the product never imports them.
"""

import importlib.util
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
EXTS = {
    "ref_laplace_ext": ("Weighted_Laplace_Sum/csrc", ["binding.cpp", "laplace_kernels.cu", "sort_utils.cu"]),
    "ref_abs_ext": ("Weighted_Abs_Sum/csrc", ["binding.cpp", "abs_kernels.cu", "sgn_kernels.cu", "sort_utils.cu"]),
}


def build(ref):
    """Compile both extensions from the checkout at `ref`."""
    from torch.utils.cpp_extension import load
    os.environ.setdefault("CXX", "/usr/bin/g++")
    os.environ["TORCH_CUDA_ARCH_LIST"] = "10.0"
    for name, (sub, files) in EXTS.items():
        bdir = os.path.join(OUT, name)
        os.makedirs(bdir, exist_ok=True)
        load(name=name, sources=[os.path.join(ref, sub, f) for f in files], build_directory=bdir,
             extra_cflags=["-O3"], extra_cuda_cflags=["-O3", "--use_fast_math"], is_python_module=True, verbose=False)
        print("built", os.path.join(bdir, name + ".so"))


def load_ref_paths():
    """Paths of the built extensions that exist."""
    paths = [os.path.join(OUT, name, name + ".so") for name in EXTS]
    return [p for p in paths if os.path.exists(p)]


def load_ref():
    """{'laplace': module, 'abs': module} for the extensions found under oracle/_ref, else {}."""
    import torch  # noqa: F401  (the extensions link against libtorch)
    mods = {}
    for key, name in (("laplace", "ref_laplace_ext"), ("abs", "ref_abs_ext")):
        path = os.path.join(OUT, name, name + ".so")
        if os.path.exists(path):
            spec = importlib.util.spec_from_file_location(name, path)
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            mods[key] = mod
    return mods


if __name__ == "__main__":
    where = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("QLKA_REFERENCE_DIR")
    if not where:
        sys.exit("usage: python oracle/build_ref.py /path/to/reference   (or set QLKA_REFERENCE_DIR)")
    build(where)
