"""``import xattn``: the reference's package name for the same public API (xattn/__init__.py:3-45 of
ifm-ai/xattn), served by ``xattn_b200``.  ``xattn.ops`` is ``xattn_b200.ops``."""
import sys

import xattn_b200 as _impl
from xattn_b200 import *  # noqa: F401,F403
from xattn_b200 import ops  # noqa: F401

__all__ = list(getattr(_impl, "__all__", [n for n in vars(_impl) if not n.startswith("_")]))
__version__ = getattr(_impl, "__version__", "0")
sys.modules.setdefault(__name__ + ".ops", ops)
