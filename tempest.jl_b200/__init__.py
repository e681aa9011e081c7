"""tempest.jl_b200 -- B200 (sm_100a) kernel backend for Tempest.jl's fused-kernel hot path.

The product is `libtempest_b200.so` (hand-written CUDA behind a C ABI, see
include/tempest_b200.h).  This package is the host side used from Python: the
ctypes binding (`lib`), and a mirror of Tempest's `Library` plugin protocol
(`implement`) so that the kernels are driven the way Tempest's cover and
runtime would drive them.

The directory name contains a dot, so it is loaded by path (see
`__graft_entry__.load_package`) under the module name `tempest_jl_b200`.
"""
from . import lib  # noqa: F401
from .lib import TB200Error, load, F32, BF16  # noqa: F401
from . import groups  # noqa: F401
from . import tuning  # noqa: F401
from . import implement  # noqa: F401
from . import mlp  # noqa: F401,E402
from . import dp  # noqa: F401,E402
