"""``minit.functional`` on torch storage (minit/functional/__init__.py:1-9 re-exports the same names).  Every operator
also accepts ``CollectiveTensor`` arguments (``compat.collective``: gathered, computed on whole tensors, broadcast-placed;
``matrix_multiply`` applies the column- / row-parallel rules instead).  The traced control-flow helpers (for_loop /
while_loop / if_block) belong to the reference's graph tracer and are not provided."""
from . import arith, einops, generate, index, linalg, reduce, shape, special
from ..collective import collective_aware as _collective_aware

for _module in (arith, einops, generate, index, linalg, reduce, shape, special):
    for _name in _module.__all__:
        if not (_module is linalg and _name == "matrix_multiply"):          # has placement rules of its own
            setattr(_module, _name, _collective_aware(getattr(_module, _name)))

from .arith import *      # noqa: E402,F401,F403
from .generate import *   # noqa: E402,F401,F403
from .index import *      # noqa: E402,F401,F403
from .linalg import *     # noqa: E402,F401,F403
from .reduce import *     # noqa: E402,F401,F403
from .shape import *      # noqa: E402,F401,F403
from .special import *    # noqa: E402,F401,F403
from .einops import *     # noqa: E402,F401,F403
