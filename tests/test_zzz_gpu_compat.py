"""Code written against MiniT's Python surface reaching the fused GPTQ kernels: ``F.matrix_multiply(x, QuantizedTensor)``
with the reference's tensor type (``minit.cuda.tensor.CUDATensor`` as provided by ``minit_b200.compat``) and a linear
layer whose ``weight`` property builds the QuantizedTensor the way examples/qwen1_5_int8.py:283-285 does."""
import sys

import numpy as np
import pytest
import torch

from oracle import qlinear_oracle as O
from tests.gpu_util import assert_close, oracle_out

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def minit(lib_built):
    from minit_b200 import compat
    from minit_b200.compat import tensor
    had = "minit" in sys.modules
    assert compat.install() or had
    tensor.set_device(None)                      # the current CUDA device
    return sys.modules["minit"]


@pytest.mark.parametrize("bits", [4, 8])
def test_matrix_multiply_of_device_tensor_and_quantized_tensor(minit, bits):
    import minit.functional as F
    from minit.cuda.tensor import CUDATensor
    from minit.quantize.tensor import QuantizedTensor
    c = O.make_gptq_case(256, 128, 6, bits=bits, act_order=True, seed=21 + bits)
    qt = QuantizedTensor(CUDATensor.from_numpy(c["q"]), CUDATensor.from_numpy(c["g_idx"]),
                         CUDATensor.from_numpy(c["z"]), CUDATensor.from_numpy(c["scales"]))
    x = CUDATensor.from_numpy(c["x"])
    assert x.device == "cuda" and x.as_torch().is_cuda
    out = F.matrix_multiply(x, qt)
    assert isinstance(out, CUDATensor) and out._shape == (6, 128) and out.dtype == "float16"
    ref = oracle_out(c, True)
    assert_close(out.as_torch(), ref, f"compat matrix_multiply bits={bits}")
    folded = F.matrix_multiply(x.expand(0, [2, 3]), qt)                      # leading axes fold and come back
    assert folded._shape == (2, 3, 128) and np.array_equal(folded.numpy().reshape(6, 128), out.numpy())


def test_module_with_a_quantized_weight_property(minit):
    import minit.functional as F
    from minit.core.tensor import Tensor
    from minit.cuda.tensor import CUDATensor
    from minit.module import Module
    from minit.quantize.tensor import QuantizedTensor

    class Linear(Module):
        qweight: Tensor

        def __init__(self, k, n, groups):
            super().__init__()
            self.q = self.register_buffer("q", (k, n), "uint8")
            self.z = self.register_buffer("z", (groups, n), "uint8")
            self.scales = self.register_buffer("scales", (groups, n), "float16")
            self.g_idx = self.register_buffer("g_idx", (k,), "int32")

        @property
        def weight(self):
            return QuantizedTensor(self.q, self.g_idx, self.z, self.scales)

        def forward(self, x):
            return F.matrix_multiply(x, self.weight)

    c = O.make_gptq_case(512, 256, 1, bits=8, seed=33)
    layer = Linear(512, 256, c["scales"].shape[0])
    layer.update_buffer("q", torch.from_numpy(c["q"]))
    layer.update_buffer("z", torch.from_numpy(c["z"]))
    layer.update_buffer("scales", c["scales"])
    layer.update_buffer("g_idx", c["g_idx"])
    assert isinstance(layer.q, CUDATensor) and layer.q.as_torch().is_cuda
    out = layer(CUDATensor.from_numpy(c["x"]))
    assert_close(out.as_torch(), oracle_out(c, False), "module with a QuantizedTensor weight, M=1")
