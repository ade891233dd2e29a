"""``tileccl``: the reference's package name, served by :mod:`tileccl_b200`.

``import tileccl``, ``tileccl.init(heap_size=...)``, ``tileccl.ops.gemm_allscatter``,
``from tileccl.memory.symmetric_heap import SymmetricHeap`` ... all resolve to the
modules of ``tileccl_b200`` (the same module objects, so state such as the
current context is shared).
"""

import importlib
import pkgutil
import sys

import tileccl_b200 as _impl

_PREFIX = "tileccl_b200"


def _alias_all() -> None:
    names = [_PREFIX]
    for info in pkgutil.walk_packages(_impl.__path__, prefix=_PREFIX + "."):
        # native sources, work files and the build helper are not part of the public tree
        if ".csrc" in info.name or info.name.endswith(("._build", ".__main__")):
            continue
        names.append(info.name)
    for name in names:
        try:
            mod = importlib.import_module(name)
        except Exception:  # an optional sub-module that cannot import must not break `import tileccl`
            continue
        alias = "tileccl" + name[len(_PREFIX):]
        if alias != "tileccl":
            sys.modules.setdefault(alias, mod)


_alias_all()

from tileccl_b200 import *  # noqa: E402,F401,F403
from tileccl_b200 import (  # noqa: E402,F401
    TileCCLContext,
    __version__,
    current_context,
    describe_runtime_support,
    get_rank,
    get_world_size,
    init,
    init_local,
)


def __getattr__(name):
    return getattr(_impl, name)


__all__ = list(_impl.__all__)
