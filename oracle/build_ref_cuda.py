"""Build the reference's OWN CUDA extension for sm_100 as a same-box GPU baseline.

TEST / BENCH INFRASTRUCTURE ONLY (like everything under oracle/): the product never loads it.

    python oracle/build_ref_cuda.py [reference checkout]

Compiles the four translation units that the reference's ``conv_attn/__init__.py:9-26`` JIT-builds
(``bindings.cpp``, ``kernels/fwd_wrapper.cu``, ``kernels/dq_bwd_wrapper.cu``, ``kernels/dkdv_wrapper.cu``)
from where they lie in the reference checkout -- nothing is copied -- with the reference's own flags,
except that the one active ``-gencode`` line (sm_89 there) names sm_100.  The output goes to
``oracle/_ref/`` (git-ignored; it travels to a GPU box with the tree).  The extension exports the pybind
functions ``forward``, ``dq_backward``, ``dkdv_backward`` (``bindings.cpp:43-57``); square filters only,
theta / D / LSE in bf16 -- it is a speed baseline (``bench.py --impl reference-gpu``), not a parity oracle.
"""
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
NAME = "fmta_reference_cuda_sm100"


def reference_root(arg=None):
    if arg:
        return arg
    try:
        with open(os.path.join(HERE, "..", "BASELINE.json")) as f:
            return json.load(f).get("reference_path")
    except Exception:
        return None


def built_path():
    p = os.path.join(OUT, NAME + ".so")
    return p if os.path.exists(p) else None


def build(ref_root=None, verbose=False):
    ref_root = reference_root(ref_root)
    src_dir = os.path.join(ref_root or "", "flash_multi_token_attention", "conv_attn")
    if not ref_root or not os.path.isdir(src_dir):
        return None
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0")      # no GPU is needed to compile
    from torch.utils.cpp_extension import load
    os.makedirs(OUT, exist_ok=True)
    load(name=NAME,
         sources=[os.path.join(src_dir, "bindings.cpp"),
                  os.path.join(src_dir, "kernels", "fwd_wrapper.cu"),
                  os.path.join(src_dir, "kernels", "dq_bwd_wrapper.cu"),
                  os.path.join(src_dir, "kernels", "dkdv_wrapper.cu")],
         extra_cflags=["-O3"],
         extra_cuda_cflags=["-O3", "--use_fast_math", "-gencode=arch=compute_100,code=sm_100"],
         build_directory=OUT, verbose=verbose, is_python_module=False)
    return built_path()


if __name__ == "__main__":
    print(build(sys.argv[1] if len(sys.argv) > 1 else None, verbose=True))
