"""B200-native attention-with-scores operators: a drop-in for the reference
package's nine entry points (its __init__.py:29-39), backed by hand-written
sm_100a CUDA kernels in libfaws.so.  No Triton, no CPU fallback."""
from .api import (  # noqa: F401
    attention,
    attention_cross_token_qk_sum,
    attention_cross_token_softmax_sum,
    attention_cross_token_softmax_sum_buffered,
    attention_with_col_sum,
    attention_with_col_sum_sequential,
    attention_with_row_sum,
    attention_with_scores,
    attention_with_softmax_col_sum,
    compute_attention_scores,
    device_status,
    last_backend,
    launch_count,
    total_attention,
)

__all__ = [
    "attention",
    "attention_with_scores",
    "attention_with_col_sum",
    "attention_with_col_sum_sequential",
    "attention_with_softmax_col_sum",
    "attention_cross_token_softmax_sum",
    "attention_cross_token_softmax_sum_buffered",
    "attention_with_row_sum",
    "attention_cross_token_qk_sum",
    "total_attention",
    "compute_attention_scores",
]
