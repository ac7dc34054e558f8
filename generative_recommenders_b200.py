"""Import shim: the package directory is named ``generative-recommenders_b200`` (not a valid
Python identifier), so ``import generative_recommenders_b200`` gives that package from here.

Both names refer to the same module objects (the package and every submodule it has imported), so
module-level state - the prepared-weights cache, the switches of ``hstu_compute`` - exists once
however the package was reached."""

import importlib
import os
import sys

_root = os.path.dirname(os.path.abspath(__file__))
if _root not in sys.path:
    sys.path.insert(0, _root)
_real = "generative-recommenders_b200"
_mod = importlib.import_module(_real)
sys.modules[__name__] = _mod
for _k, _v in list(sys.modules.items()):
    if _k.startswith(_real + "."):
        sys.modules[__name__ + _k[len(_real):]] = _v
