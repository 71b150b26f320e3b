"""Drop-in modules with the reference's extension names.

``install()`` registers ``atmm_ops`` and ``valora._kernels`` in ``sys.modules``
so that ``from atmm_ops import dispatch_bgmv as dispatch_sgmm`` and
``from valora._kernels import dispatch_bgmv`` - the imports the reference's
engine and kernel tests use - resolve to the sm_100a operators.
"""
import sys
import types

from . import atmm_ops as _atmm
from . import valora_kernels as _kernels


def install(force: bool = False):
    if force or "atmm_ops" not in sys.modules:
        sys.modules["atmm_ops"] = _atmm
    pkg = sys.modules.get("valora")
    if pkg is None:
        pkg = types.ModuleType("valora")
        pkg.__path__ = []
        sys.modules["valora"] = pkg
    if force or "valora._kernels" not in sys.modules:
        sys.modules["valora._kernels"] = _kernels
        setattr(pkg, "_kernels", _kernels)
    return _atmm, _kernels
