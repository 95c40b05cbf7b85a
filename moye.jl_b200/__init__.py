"""moye_b200: the Blackwell (sm_100a) implementation of MoYe.jl's tiled GEMM / TiledCopy hot
path, behind MoYe's own vocabulary (Layout, MoYeArray, @tile / @parallelize, TiledCopy,
TiledMMA, copyto!, gemm!).

The directory is named `moye.jl_b200`, which Python cannot import by name; load it with
`__graft_entry__.load_package()` (or importlib with `submodule_search_locations`) under the
module name `moye_b200`.
"""
from . import _lib
from .layout import *  # noqa: F401,F403
from .array import *  # noqa: F401,F403
from .atom import *  # noqa: F401,F403
from .algorithm import *  # noqa: F401,F403
from .sharding import *  # noqa: F401,F403
from .host_pipeline import *  # noqa: F401,F403
from .printing import *  # noqa: F401,F403
from ._lib import MoyeError

__version__ = "0.1.0"
