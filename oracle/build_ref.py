"""Builds the reference's OWN CUDA extensions for sm_100a, from the sources where they lie, into
oracle/_ref/ (test infrastructure; nothing of the product imports this or what it builds).

    python oracle/build_ref.py [path of the reference checkout]        (default: /root/reference)

Two modules are built with torch's extension builder (nvcc + ninja; the reference's setup.py is not
run -- it refuses every architecture but sm80):

  _fused     csrc/fused/fused.cu + csrc/fused/pybind.cpp: the INT8 / FP8 quantisers
             (QuantInt8Kernel fused.cu:64-198, MeanScaleKernel :316-427, TransposePadPermuteKernel :262-313)
  _fused_ieee  the same sources without --use_fast_math (the reference's setup.py:26 turns it on, which
             makes 127/amax an approximate divide; this build shows the algorithm without that flag)
  _qattn     csrc/qattn/qk_int_sv_f16_cuda_sm80.cu with a one-function binding
             (oracle/ref_qattn_binding.cpp): qk_int8_sv_f16_accum_f16_attn, the kernel the reference's
             processors call (its mma.sync / cp.async code compiles for sm_100a as it is)

The built modules are only RUN by tests/golden/make_golden_refcuda.py, on a machine with a GPU, to
produce the committed fixtures tests/golden/refcuda_*.npz against which the CPU oracle is pinned.
"""
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")

NVCC = ["-O3", "-std=c++17", "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__",
        "-diag-suppress=174", "-gencode", "arch=compute_100a,code=sm_100a"]
CXX = ["-O3", "-std=c++17", "-DENABLE_BF16"]


def build(ref: str = "/root/reference", verbose: bool = False):
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    from torch.utils.cpp_extension import load
    csrc = os.path.join(ref, "csrc")
    if not os.path.isdir(csrc):
        raise SystemExit(f"no reference sources under {ref}")
    built = []
    for name, fast in (("_fused", True), ("_fused_ieee", False)):
        d = os.path.join(OUT, name)
        os.makedirs(d, exist_ok=True)
        load(name=name, sources=[os.path.join(csrc, "fused", "pybind.cpp"), os.path.join(csrc, "fused", "fused.cu")],
             extra_cflags=CXX, extra_cuda_cflags=NVCC + (["--use_fast_math"] if fast else []), build_directory=d,
             verbose=verbose, is_python_module=True)
        built.append(os.path.join(d, name + ".so"))
    d = os.path.join(OUT, "_qattn")
    os.makedirs(d, exist_ok=True)
    load(name="_qattn", sources=[os.path.join(HERE, "ref_qattn_binding.cpp"),
                                 os.path.join(csrc, "qattn", "qk_int_sv_f16_cuda_sm80.cu")],
         extra_include_paths=[os.path.join(csrc, "qattn")], extra_cflags=CXX,
         extra_cuda_cflags=NVCC + ["--use_fast_math"], build_directory=d, verbose=verbose, is_python_module=True)
    built.append(os.path.join(d, "_qattn.so"))
    return built


def load_built(name: str):
    """Imports oracle/_ref/<name>/<name>.so (torch must be imported first); None when it was not built."""
    import importlib.machinery
    import importlib.util
    import torch  # noqa: F401  (the extension links against torch's libraries)
    path = os.path.join(OUT, name, name + ".so")
    if not os.path.exists(path):
        return None
    loader = importlib.machinery.ExtensionFileLoader(name, path)
    spec = importlib.util.spec_from_loader(name, loader)
    mod = importlib.util.module_from_spec(spec)
    loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    for p in build(sys.argv[1] if len(sys.argv) > 1 else "/root/reference", verbose=True):
        print("built", p)
