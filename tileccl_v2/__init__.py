"""``tileccl_v2``: the reference's planning package name, served by
:mod:`tileccl_b200.planning` (TileGroup planner, collective specs, transport and
role plans, cost model, signal state, timeline)."""

import importlib
import pkgutil
import sys

import tileccl_b200.planning as _impl

for _info in pkgutil.walk_packages(_impl.__path__, prefix="tileccl_b200.planning."):
    try:
        sys.modules.setdefault("tileccl_v2" + _info.name[len("tileccl_b200.planning"):],
                               importlib.import_module(_info.name))
    except Exception:
        pass

from tileccl_b200.planning import *  # noqa: E402,F401,F403
from tileccl_b200.planning import __version__  # noqa: E402,F401

__all__ = list(_impl.__all__)
