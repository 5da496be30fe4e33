"""Generate tests/golden/dequant_golden.npz by running the REFERENCE's own code on CPU.

Run once, in a container that has the reference checkout (pass its root as argv[1]):

    python tests/golden/make_golden.py /path/to/minit-checkout

What runs from the reference, unmodified:
  * ``minit.quantize.dispatch.dispatch_dequantize`` (through
    ``minit.quantize.tensor.QuantizedTensor.dequantize``), i.e. the formula
    ``(data.cast(T) - (zero.cast(T)+1)) * scale`` with its index/cast/arith
    dispatches;
  * the typed multi-dispatch of ``minit.core.dispatch``.
What this script supplies, because the reference's only backend is CUDA and this
container has no GPU: a torch-CPU ``Tensor`` subclass with dispatch rules for
Index / Cast / Add / Subtract / Multiply whose semantics are those of
the reference CUDA kernels (gather along one axis, C cast, elementwise arithmetic
evaluated in the tensor's own dtype).  ``nvtx`` (a hard import of the reference,
absent here) is replaced by a no-op stub.

  * ``unpack(x, axis)`` of examples/qwen1_5_int8.py:40-50: the function's own source is cut out of the
    example file (importing the whole example would compile its CUDA runtime shims) and executed
    unmodified; its Reinterpret / Expand / AddAxis / Transpose / RemoveAxis / Fold steps run through the
    reference's functional wrappers and dispatch, with torch-CPU rules that restate the view / copy
    semantics of minit/cuda/dispatch.py:210-245, 356-380, 482-490.

The fixture stores inputs (packed GPTQ tensors) and the reference's W bit pattern
(int16 view) for several small cases, and two int32 matrices with the reference's unpack(x, 0) and
unpack(x, 1) of each.  The reference has no 4-bit instantiation of
its unpack(); 4-bit data is unpacked here with the reference's accessor formula
(examples/qwen1_5_int8.py:97-138) before entering the reference dequantize.
"""
import contextlib
import io
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))


def _load_reference(root):
    stub = types.ModuleType("nvtx")

    def annotate(*a, **k):
        def deco(f):
            return f
        return deco
    stub.annotate = annotate
    sys.modules.setdefault("nvtx", stub)
    sys.path.insert(0, root)
    with contextlib.redirect_stdout(io.StringIO()):
        from minit.core.tensor import Tensor
        from minit.core.scalar import ScalarTensor
        from minit.core.dispatch import register_dispatch
        from minit.operator.arith import Add, Subtract, Multiply, Cast
        from minit.operator.index import Index
        from minit.operator.shape import AddAxis, Expand, Fold, Reinterpret, RemoveAxis, Transpose
        import minit.quantize.dispatch  # noqa: F401  registers dispatch_dequantize
        from minit.quantize.tensor import QuantizedTensor

    tdt = {"float16": torch.float16, "bfloat16": torch.bfloat16, "uint8": torch.uint8,
           "int32": torch.int32, "float32": torch.float32}
    names = {v: k for k, v in tdt.items()}

    class CPUTensor(Tensor):
        def __init__(self, t):
            super().__init__()
            self.t = t

        @property
        def shape(self):
            return tuple(CPUTensor(torch.tensor(d, dtype=torch.int32)) for d in self.t.shape)

        @property
        def dtype(self):
            return names[self.t.dtype]

        @property
        def device(self):
            return "cpu"

        def item(self):
            return self.t.item()

    with contextlib.redirect_stdout(io.StringIO()):
        @register_dispatch()
        def _index(op: Index, x: CPUTensor, index: CPUTensor):
            return (CPUTensor(x.t.index_select(op.axis, index.t.long())),)

        @register_dispatch()
        def _cast(op: Cast, x: CPUTensor):
            return (CPUTensor(x.t.to(tdt[op.dtype])),)

        # a python scalar reaches the backend as a ScalarTensor and decays to a filled tensor of
        # the same dtype before the elementwise kernel runs (minit/cuda/dispatch.py:120-129)
        @register_dispatch()
        def _add_scalar(op: Add, x: CPUTensor, y: ScalarTensor):
            assert y.dtype == x.dtype
            return (CPUTensor(x.t + torch.full(x.t.shape, y.value(), dtype=x.t.dtype)),)

        @register_dispatch()
        def _add(op: Add, x: CPUTensor, y: CPUTensor):
            return (CPUTensor(x.t + y.t),)

        @register_dispatch()
        def _sub(op: Subtract, x: CPUTensor, y: CPUTensor):
            return (CPUTensor(x.t - y.t),)

        @register_dispatch()
        def _mul(op: Multiply, x: CPUTensor, y: CPUTensor):
            return (CPUTensor(x.t * y.t),)

        def _dim(v):
            return int(v.item()) if isinstance(v, CPUTensor) else int(v.value())

        @register_dispatch()
        def _reinterpret(op: Reinterpret, x: CPUTensor):
            return (CPUTensor(x.t.contiguous().view(tdt[op.target])),)

        @register_dispatch()
        def _expand(op: Expand, x: CPUTensor, *sizes: Tensor):
            dims = tuple(_dim(v) for v in sizes)
            shape = tuple(x.t.shape)
            return (CPUTensor(x.t.contiguous().reshape(shape[:op.axis] + dims + shape[op.axis + 1:])),)

        @register_dispatch()
        def _add_axis(op: AddAxis, x: CPUTensor):
            return (CPUTensor(x.t.contiguous().unsqueeze(op.axis)),)

        @register_dispatch()
        def _remove_axis(op: RemoveAxis, x: CPUTensor):
            assert x.t.shape[op.axis] == 1
            return (CPUTensor(x.t.contiguous().squeeze(op.axis)),)

        @register_dispatch()
        def _fold(op: Fold, x: CPUTensor):
            shape = tuple(x.t.shape)
            size = 1
            for d in shape[op.start:op.stop]:
                size *= d
            return (CPUTensor(x.t.contiguous().reshape(shape[:op.start] + (size,) + shape[op.stop:])),)

        @register_dispatch()
        def _transpose(op: Transpose, x: CPUTensor):
            return (CPUTensor(x.t.transpose(op.axis_a, op.axis_b).contiguous()),)     # the reference's copy kernel

    # the reference's unpack(), source text taken from the example file as it is
    import ast
    example = os.path.join(root, "examples", "qwen1_5_int8.py")
    src = open(example).read()
    node = next(n for n in ast.parse(src).body if isinstance(n, ast.FunctionDef) and n.name == "unpack")
    ns = {"Tensor": Tensor}
    exec(compile(ast.Module(body=[node], type_ignores=[]), example, "exec"), ns)

    def ref_unpack(x_i32, axis):
        return ns["unpack"](CPUTensor(torch.from_numpy(x_i32)), axis).t.numpy()

    def ref_dequantize(q_u8, g_idx, z_u8, scales):
        qt = QuantizedTensor(CPUTensor(torch.from_numpy(q_u8)), CPUTensor(torch.from_numpy(g_idx)),
                             CPUTensor(torch.from_numpy(z_u8)), CPUTensor(scales))
        return qt.dequantize().t

    return ref_dequantize, ref_unpack


def main():
    if len(sys.argv) < 2 and "MINIT_REFERENCE" not in os.environ:
        raise SystemExit("usage: make_golden.py <path to a checkout of the reference project>  (or set MINIT_REFERENCE)")
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ["MINIT_REFERENCE"]
    ref_dequantize, ref_unpack = _load_reference(root)
    from oracle import qlinear_oracle as O

    cases = {}
    specs = [
        # name, bits, K, N, group, act_order, dtype
        ("int4_f16", 4, 256, 64, 128, False, torch.float16),
        ("int4_f16_act", 4, 256, 64, 128, True, torch.float16),
        ("int4_bf16", 4, 256, 32, 128, False, torch.bfloat16),
        ("int4_f16_g32", 4, 128, 32, 32, True, torch.float16),
        ("int8_f16", 8, 256, 32, 128, False, torch.float16),
        ("int8_f16_act", 8, 256, 32, 128, True, torch.float16),
        ("int8_bf16_act", 8, 128, 32, 64, True, torch.bfloat16),
    ]
    for i, (name, bits, k, n, gs, act, dt) in enumerate(specs):
        c = O.make_gptq_case(k, n, 1, bits=bits, group_size=gs, act_order=act, dtype=dt, seed=100 + i)
        # force the edge values the formula is sensitive to: zero at max (no wrap-around), q at 0 / max
        c["z"][0, :4] = (1 << bits) - 1
        c["q"][0, :4] = 0
        c["q"][1, :4] = (1 << bits) - 1
        c["z"][-1, -4:] = 0
        qweight = O.pack_rows(c["q"], bits)
        qzeros = O.pack_cols(c["z"], bits)
        g_idx = c["g_idx"].numpy()
        w = ref_dequantize(c["q"], g_idx, c["z"], c["scales"])
        cases[f"{name}.bits"] = np.int32(bits)
        cases[f"{name}.qweight"] = qweight
        cases[f"{name}.qzeros"] = qzeros
        cases[f"{name}.g_idx"] = g_idx
        cases[f"{name}.scales_bits"] = c["scales"].view(torch.int16).numpy()
        cases[f"{name}.is_bf16"] = np.int32(dt == torch.bfloat16)
        cases[f"{name}.w_bits"] = w.view(torch.int16).numpy()
    # the per-channel int8 special case in the reference layout (one group, stored zero 127)
    c = O.make_w8_case(64, 32, 1, seed=7)
    qweight, g_idx, qzeros, s = O.w8_perchannel_as_gptq(c["w"].numpy(), c["scales"])
    w = ref_dequantize(O.unpack_rows(qweight, 8), g_idx, O.unpack_cols(qzeros, 8), s)
    cases["w8pc.w_i8"] = c["w"].numpy()
    cases["w8pc.scales_bits"] = c["scales"].view(torch.int16).numpy()
    cases["w8pc.w_bits"] = w.view(torch.int16).numpy()
    # the reference's own unpack() (8-bit, the only width it has) on two packed matrices, both axes
    rng = np.random.default_rng(5)
    for name, shape in (("unpack_a", (8, 12)), ("unpack_b", (32, 16))):
        x = rng.integers(-2**31, 2**31 - 1, size=shape, dtype=np.int64).astype(np.int32)
        x[0, 0], x[0, 1] = np.int32(0x04030201), np.int32(-1)        # byte order and the sign bit at a glance
        cases[f"{name}.x"] = x
        cases[f"{name}.axis0"] = ref_unpack(x, 0)
        cases[f"{name}.axis1"] = ref_unpack(x, 1)
    out = os.path.join(HERE, "dequant_golden.npz")
    np.savez_compressed(out, **cases)
    print("wrote", out, os.path.getsize(out), "bytes;", len(specs) + 1, "dequantize cases, 2 unpack cases")


if __name__ == "__main__":
    main()
