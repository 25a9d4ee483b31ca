from .causal_flash_attn import causal_flash_attn, causal_flash_attn_bwd, causal_flash_attn_fwd
from .sliding_chunk_attention import flash_sca, flash_sca_bwd, flash_sca_fwd, flash_sca_sm90_available
from .sliding_window_attention import flash_swa, flash_swa_bwd, flash_swa_fwd
from .softdelta_attention import (
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

__all__ = [
    "flash_sca", "flash_sca_bwd", "flash_sca_fwd", "flash_sca_sm90_available",
    "flash_swa", "flash_swa_bwd", "flash_swa_fwd",
    "causal_flash_attn", "causal_flash_attn_bwd", "causal_flash_attn_fwd",
    "softdelta_attention", "softdelta_attention_bwd", "softdelta_attention_fwd",
    "sliding_window_softdelta_attention", "sliding_window_softdelta_attention_bwd",
    "sliding_window_softdelta_attention_fwd",
    "sliding_chunk_softdelta_attention", "sliding_chunk_softdelta_attention_bwd",
    "sliding_chunk_softdelta_attention_fwd",
]
