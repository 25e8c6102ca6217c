"""Drop-in alias: ``import neuzip`` gives the neuzip_b200 implementation under
the reference's module names (``neuzip.nn``, ``neuzip.ops``, ``neuzip.binding``,
``neuzip.utils``)."""
import sys

import neuzip_b200 as _impl
from neuzip_b200 import (Algorithm, Manager, binding, compressed_lomo_hook, lomo_hook, nn, ops,
                         utils)

for _name in ("nn", "ops", "binding", "utils", "backend"):
    sys.modules[__name__ + "." + _name] = getattr(_impl, _name) if hasattr(_impl, _name) \
        else __import__("neuzip_b200." + _name, fromlist=[_name])
sys.modules[__name__ + "._cuda"] = _impl.backend._cuda  # attribute-style stand-in
_cuda = _impl.backend._cuda

__all__ = ["ops", "nn", "Algorithm", "Manager", "lomo_hook", "compressed_lomo_hook"]
