"""xattn_b200: the xattn attention ops on Blackwell (sm_100a).

Same public functions, tensor layouts and argument meaning as ``xattn`` (xattn/__init__.py:3-45);
``import xattn_b200 as xattn`` is the drop-in.  The kernels live in ``libxattn_b200.so`` (C ABI in
``include/xattn_b200.h``); there is no CPU fallback.
"""
__version__ = "0.1.0"

from .ops import (  # noqa: F401
    causal_flash_attn,
    causal_flash_attn_bwd,
    causal_flash_attn_fwd,
    flash_sca,
    flash_sca_bwd,
    flash_sca_fwd,
    flash_sca_sm90_available,
    flash_swa,
    flash_swa_bwd,
    flash_swa_fwd,
    sliding_chunk_softdelta_attention,
    sliding_chunk_softdelta_attention_bwd,
    sliding_chunk_softdelta_attention_fwd,
    sliding_window_softdelta_attention,
    sliding_window_softdelta_attention_bwd,
    sliding_window_softdelta_attention_fwd,
    softdelta_attention,
    softdelta_attention_bwd,
    softdelta_attention_fwd,
)
from ._native import check_status  # noqa: F401
from .ops._core import clear_plan_cache  # noqa: F401
from .ops import __all__ as _ops_all

__all__ = list(_ops_all) + ["check_status", "clear_plan_cache"]
