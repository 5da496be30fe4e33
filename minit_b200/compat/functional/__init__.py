"""``minit.functional`` on torch storage (minit/functional/__init__.py:1-9 re-exports the same names).  The traced
control-flow helpers (for_loop / while_loop / if_block) belong to the reference's graph tracer and are not provided."""
from . import arith, einops, generate, index, linalg, reduce, shape, special
from .arith import *      # noqa: F401,F403
from .generate import *   # noqa: F401,F403
from .index import *      # noqa: F401,F403
from .linalg import *     # noqa: F401,F403
from .reduce import *     # noqa: F401,F403
from .shape import *      # noqa: F401,F403
from .special import *    # noqa: F401,F403
from .einops import *     # noqa: F401,F403
