"""Import name of the reference package (its README.md:27: ``from flash_attention_with_scores
import attention_with_scores``): the same nine operators (the reference's __init__.py:29-39),
served by the sm_100a kernels of ``flash_attn_with_score_b200``.  Code written against the
reference runs unchanged."""
from flash_attn_with_score_b200 import (  # noqa: F401
    attention,
    attention_cross_token_qk_sum,
    attention_cross_token_softmax_sum,
    attention_cross_token_softmax_sum_buffered,
    attention_with_col_sum,
    attention_with_col_sum_sequential,
    attention_with_row_sum,
    attention_with_scores,
    attention_with_softmax_col_sum,
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
]
