"""Switch a running copy of the reference over to this library, for ``HammerKernel.CUDA``.

``install()`` rebinds the operator entry points of ``generative_recommenders`` - ``hstu_mha`` and
``delta_hstu_mha`` (ops/hstu_attention.py:101-284), ``hstu_compute_uqvk``, ``hstu_compute_output``
and ``hstu_preprocess_and_attention`` (ops/hstu_compute.py:54-335), the jagged concat / split and
the positional embedding op (ops/jagged_tensors.py:55-162, ops/position.py:40-118), ``layer_norm``
(ops/layer_norm.py:50-94) - and the copies of those names that modules which did
``from ... import name`` hold (modules/stu.py imports them that way).  A call with
``kernel=HammerKernel.CUDA`` then runs the sm_100a kernels; any other backend value goes to the
function that was there before, untouched.  ``uninstall()`` puts everything back.

The reference leaves ``HammerKernel.CUDA`` unhandled in ``hstu_mha`` (it falls through to the
PyTorch branch, ops/hstu_attention.py:191-207), so nothing that works today changes meaning.
"""

import functools
import importlib
import inspect
import sys
from typing import Callable, Dict, List, Tuple

_PATCHED: List[Tuple[object, str, object]] = []

# module (relative to the reference package) -> names this library provides with the same signature
_TARGETS: Dict[str, Tuple[str, ...]] = {
    "ops.hstu_attention": ("hstu_mha", "delta_hstu_mha"),
    "ops.hstu_compute": ("hstu_compute_uqvk", "hstu_compute_output", "hstu_preprocess_and_attention"),
    "ops.jagged_tensors": ("concat_2D_jagged", "split_2D_jagged", "hstu_split_l2_embeddings",
                           "hstu_concat_l2_embeddings"),
    "ops.position": ("add_timestamp_positional_embeddings",),
    "ops.layer_norm": ("layer_norm",),
}


def _is_cuda_kernel(value) -> bool:
    return getattr(value, "name", value) == "CUDA"


def _dispatching(ours: Callable, theirs: Callable) -> Callable:
    """``theirs`` unless the call asks for the CUDA backend (by keyword or by position)."""
    try:
        params = list(inspect.signature(theirs).parameters)
    except (TypeError, ValueError):
        params = []
    pos = params.index("kernel") if "kernel" in params else -1

    @functools.wraps(theirs)
    def wrapper(*args, **kwargs):
        kernel = kwargs.get("kernel", args[pos] if 0 <= pos < len(args) else None)
        if _is_cuda_kernel(kernel):
            from .common import HammerKernel

            if "kernel" in kwargs:
                kwargs = dict(kwargs, kernel=HammerKernel.CUDA)
            else:
                args = args[:pos] + (HammerKernel.CUDA,) + args[pos + 1:]
            return ours(*args, **kwargs)
        return theirs(*args, **kwargs)

    wrapper.__b200_hstu_original__ = theirs
    return wrapper


def install(package: str = "generative_recommenders") -> int:
    """Rebind the reference's entry points (see the module docstring); returns how many names were
    rebound.  The reference must be importable; calling it twice is harmless."""
    import generative_recommenders_b200 as G

    if _PATCHED:
        return len(_PATCHED)
    replaced = {}
    for rel, names in _TARGETS.items():
        try:
            mod = importlib.import_module("%s.%s" % (package, rel))
        except ImportError:
            continue
        for name in names:
            theirs = getattr(mod, name, None)
            ours = getattr(G, name, None)
            if theirs is None or ours is None:
                continue
            wrapped = _dispatching(ours, theirs)
            _PATCHED.append((mod, name, theirs))
            setattr(mod, name, wrapped)
            replaced[id(theirs)] = wrapped
    # names imported with ``from ... import name`` elsewhere in the package
    for mname, mod in list(sys.modules.items()):
        if mod is None or not (mname == package or mname.startswith(package + ".")):
            continue
        for attr, val in list(vars(mod).items()):
            w = replaced.get(id(val))
            if w is not None and val is not w:
                _PATCHED.append((mod, attr, val))
                setattr(mod, attr, w)
    return len(_PATCHED)


def uninstall() -> None:
    while _PATCHED:
        mod, name, original = _PATCHED.pop()
        setattr(mod, name, original)
