from .operator import Dequantize  # noqa: F401
from .tensor import QuantizedTensor  # noqa: F401
from .functional import dequantize  # noqa: F401
