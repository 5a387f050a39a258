"""TEST AND BENCHMARK INFRASTRUCTURE ONLY - the reference's own pure-Python caller, unmodified.

`stage(ref)` copies the two files of the reference's `Experiments/kernel_attention` package that the
additive-kernel path needs (`__init__.py` is not taken: it would pull in nothing else, and a generated
empty one keeps `nomic.py` / `vision_transformer.py` and their dependencies out) from a checkout into
the git-ignored folder `baseline/_ref/Experiments/kernel_attention/`. Nothing of it enters the
repository's history; like the compiled extensions of oracle/build_ref.py the folder only travels to the
GPU box, where no checkout exists.

    python oracle/ref_python.py /path/to/reference

`load(stub_extensions)` imports the staged package under the name `ref_kernel_attention` (this repository
has a package called `kernel_attention` of its own):

* stub_extensions=True  - `weighted_abs_sum` / `weighted_laplace_sum`, which the reference's attention.py imports
  at module level (Experiments/kernel_attention/attention.py:11-12), are empty stand-ins for the duration of the
  import. Only the paths that need no extension work: `impl="naive"` and the chunked compiled path
  `_chunked(_normalized_compiled, ...)` (attention.py:38-50), which is the reference's CPU-runnable
  implementation and the CPU arm of the benchmark.
* stub_extensions=False - the two names resolve to whatever is importable, i.e. this repository's drop-in packages
  when their folder is on sys.path: the reference's caller then runs on top of them unchanged (the drop-in test).
"""

import importlib.util
import os
import shutil
import sys
import types

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(os.path.dirname(HERE), "baseline", "_ref", "Experiments", "kernel_attention")
FILES = ("attention.py", "kernels.py")


def staged():
    return all(os.path.exists(os.path.join(DEST, f)) for f in FILES)


def stage(ref):
    src = os.path.join(ref, "Experiments", "kernel_attention")
    os.makedirs(DEST, exist_ok=True)
    for f in FILES:
        shutil.copyfile(os.path.join(src, f), os.path.join(DEST, f))
    with open(os.path.join(DEST, "__init__.py"), "w") as fh:
        fh.write("")
    return DEST


def _use_system_gxx():
    """The compiled chunk function is built by inductor with OpenMP; a toolchain without libgomp.spec cannot
    do that, the distribution's g++ can."""
    if os.path.exists("/usr/bin/g++"):
        os.environ["CXX"] = "/usr/bin/g++"
        try:
            import torch._inductor.config as cfg
            cfg.cpp.cxx = ("/usr/bin/g++",)
        except Exception:
            pass


def load(stub_extensions):
    """The reference's `kernel_attention.attention` module (with `.kernels` beside it), or None if not staged."""
    if not staged():
        return None
    name = "ref_kernel_attention_stubbed" if stub_extensions else "ref_kernel_attention"
    if name + ".attention" in sys.modules:
        return sys.modules[name + ".attention"]
    _use_system_gxx()
    saved = {}
    if stub_extensions:
        for ext in ("weighted_abs_sum", "weighted_laplace_sum"):
            saved[ext] = sys.modules.get(ext)
            stub = types.ModuleType(ext)
            stub.weighted_abs_sum_full = None
            stub.weighted_laplace_sum = None
            sys.modules[ext] = stub
    try:
        pkg_spec = importlib.util.spec_from_file_location(name, os.path.join(DEST, "__init__.py"), submodule_search_locations=[DEST])
        pkg = importlib.util.module_from_spec(pkg_spec)
        sys.modules[name] = pkg
        pkg_spec.loader.exec_module(pkg)
        mods = {}
        for sub in ("kernels", "attention"):
            spec = importlib.util.spec_from_file_location(f"{name}.{sub}", os.path.join(DEST, sub + ".py"))
            mod = importlib.util.module_from_spec(spec)
            sys.modules[f"{name}.{sub}"] = mod
            spec.loader.exec_module(mod)
            setattr(pkg, sub, mod)
            mods[sub] = mod
    finally:
        for ext, old in saved.items():
            if old is None:
                sys.modules.pop(ext, None)
            else:
                sys.modules[ext] = old
    return mods["attention"]


if __name__ == "__main__":
    where = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("QLKA_REFERENCE_DIR")
    if not where:
        sys.exit("usage: python oracle/ref_python.py /path/to/reference   (or set QLKA_REFERENCE_DIR)")
    print(stage(where))
