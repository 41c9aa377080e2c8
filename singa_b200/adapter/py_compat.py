"""Lets apache/singa's UNMODIFIED Python layer import under a current
interpreter: it was written for Python <= 3.9 and numpy < 1.24 and uses two
aliases that have since been removed (``collections.Iterable`` in model.py,
``np.int`` / ``np.float`` / ``np.bool`` in tensor.py).  ``use(variant)`` restores
the aliases, puts the assembled ``singa`` package (see build_singa_wrap.py) at
the front of sys.path and returns the package directory."""
import collections
import collections.abc
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def restore_aliases():
    if not hasattr(collections, "Iterable"):
        collections.Iterable = collections.abc.Iterable
    for name, target in (("int", int), ("float", float), ("bool", bool)):
        if name not in np.__dict__:
            setattr(np, name, target)


def use(variant):
    restore_aliases()
    path = os.path.join(ROOT, "baseline", "_ref", "singa_" + variant)
    if not os.path.isdir(os.path.join(path, "singa")):
        raise ImportError("%s/singa is not built: run python -m singa_b200.adapter.build_singa_wrap %s"
                          % (path, variant))
    if path not in sys.path:
        sys.path.insert(0, path)
    return path
