"""``import axonml``: the reference's package name as an alias of ``axonml_b200`` (same objects).

    import axonml
    from axonml import nn, optim
    from axonml.distributed import DistributedDataParallel
"""
import importlib
import sys

import axonml_b200 as _impl

__version__ = _impl.__version__
prelude = _impl.prelude


def __getattr__(name):
    mod = getattr(_impl, name)
    sys.modules.setdefault(f"{__name__}.{name}", mod)
    return mod


for _n in _impl._SUBPACKAGES + tuple(_impl._ALIASES):
    _target = _impl._ALIASES.get(_n, _n)
    try:
        sys.modules[f"{__name__}.{_n}"] = importlib.import_module(f"axonml_b200.{_target}")
    except Exception:        # optional pieces (e.g. CUDA-only imports) stay lazy
        pass
