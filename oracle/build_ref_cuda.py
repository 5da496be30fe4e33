"""Test infrastructure: build the reference's OWN CUDA kernels for sm_100a, as shared libraries under oracle/_ref/.

The reference keeps its kernels as source strings inside Python files and compiles them at run time with nvcc
(minit/cuda/compiler.py:9-25, `-gencode=arch=compute_70,code=compute_70`; `${KEY}` placeholders filled by
minit/compiler/template.py:4-7).  This recipe does the same ahead of time: it cuts the string assigned to
``kernel_template`` out of each file with ``ast`` (nothing of the reference is imported or executed), fills the
placeholders with the values the reference itself passes for fp16, and compiles the text unchanged, for the GPU at hand
instead of Volta.  No reference source is written into the repository: the filled-in text goes to a temporary
directory, only the built libraries stay (oracle/_ref/ is not tracked).

    python oracle/build_ref_cuda.py <root of a checkout of the reference>      (or set MINIT_REFERENCE)

Built: libref_qmm_f16.so (`qmm_ref`, examples/qwen1_5_int8.py:53-216), libref_rms_norm_f16.so (`minit_rms_norm`,
minit/cuda/kernel/cuda/rms_norm.py:11-104), libref_rope_f32.so (`minit_rope`, .../rope.py:11-90; instantiated for
float: with T = __half nvcc 12.9 rejects `real * freq_cos`, half times float, as ambiguous, so the fp16 form of
that kernel cannot be built as it is), libref_softmax_f16.so (`minit_softmax`, .../softmax.py:11-119).  tests/golden/make_cuda_golden.py runs them on a GPU
and stores their outputs as fixtures; only tests and that script load these libraries.
"""
import ast
import os
import shutil
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")

#: (file inside the reference, function that holds `kernel_template`, placeholder values, library name)
UNITS = [
    ("examples/qwen1_5_int8.py", "generate_quantized_matrix_multiply",
     {"DATA_TYPE": "__half", "OUTPUT_DATA_TYPE": "__half", "TILE_NK": "32", "KERNEL_NAME": "qmm_ref"}, "libref_qmm_f16.so"),
    ("minit/cuda/kernel/cuda/rms_norm.py", "generate_rms_norm_kernel",
     {"DATA_TYPE": "__half", "KERNEL_NAME": "minit_rms_norm"}, "libref_rms_norm_f16.so"),
    ("minit/cuda/kernel/cuda/rope.py", "generate_rope_kernel",
     {"DATA_TYPE": "float", "KERNEL_NAME": "minit_rope"}, "libref_rope_f32.so"),
    ("minit/cuda/kernel/cuda/softmax.py", "generate_softmax_kernel",
     {"DATA_TYPE": "__half", "KERNEL_NAME": "minit_softmax"}, "libref_softmax_f16.so"),
]


def kernel_template(path: str, function: str) -> str:
    """The string constant assigned to ``kernel_template`` inside ``function`` of the file at ``path``."""
    tree = ast.parse(open(path).read())
    for node in ast.walk(tree):
        if isinstance(node, ast.FunctionDef) and node.name == function:
            for stmt in ast.walk(node):
                if (isinstance(stmt, ast.Assign) and len(stmt.targets) == 1 and isinstance(stmt.targets[0], ast.Name)
                        and stmt.targets[0].id == "kernel_template" and isinstance(stmt.value, ast.Constant)):
                    return stmt.value.value
    raise RuntimeError(f"{path}: no kernel_template in {function}()")


def fill(source: str, values: dict) -> str:
    for k, v in values.items():                      # the reference's substitution rule: plain replacement of ${KEY}
        source = source.replace("${" + k + "}", v)
    return source


def build(root: str, verbose: bool = False) -> list:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    os.makedirs(OUT, exist_ok=True)
    built = []
    for rel, function, values, lib in UNITS:
        src = os.path.join(root, rel)
        dst = os.path.join(OUT, lib)
        if os.path.exists(dst) and os.path.getmtime(dst) >= max(os.path.getmtime(src), os.path.getmtime(__file__)):
            built.append(dst)
            continue
        text = fill(kernel_template(src, function), values)
        with tempfile.TemporaryDirectory() as tmp:
            with open(os.path.join(tmp, "main.cu"), "w") as f:
                f.write(text)
            cmd = [nvcc, "-shared", "--compiler-options", "-fPIC", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
                   "-w", "main.cu", "-o", dst]
            r = subprocess.run(cmd, cwd=tmp, capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed for the kernel of {rel}:\n{r.stderr[-3000:]}")
        if verbose:
            print("built", dst)
        built.append(dst)
    return built


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("MINIT_REFERENCE")
    if not root or not os.path.isdir(root):
        raise SystemExit("usage: build_ref_cuda.py <path to a checkout of the reference project>  (or set MINIT_REFERENCE)")
    for p in build(root, verbose=True):
        print(p)
