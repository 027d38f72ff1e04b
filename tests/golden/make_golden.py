"""Generate tests/golden/*.npz by running the reference's own PyTorch oracle.

Run once in a container where the reference checkout is present:

    python tests/golden/make_golden.py /path/to/Flash_Attn_with_Score

It imports ``reference_implementations.naive_attention_with_scores`` from the
reference (reference_implementations.py:11-52), feeds it seeded inputs and
stores inputs and outputs.  The fixtures travel with the repository; the
reference does not need to be present when the tests run.
"""
import os
import sys

import numpy as np
import torch

CASES = [
    # name, B, Hq, Hk, M, N, D, dtype, causal, seed
    ("causal_mha_fp32", 1, 2, 2, 64, 64, 16, "float32", True, 0),
    ("causal_gqa_fp16", 2, 4, 2, 48, 48, 32, "float16", True, 1),
    ("noncausal_gqa_bf16", 1, 4, 1, 40, 56, 64, "bfloat16", False, 2),
    ("causal_topleft_m_lt_n_fp16", 1, 2, 1, 32, 48, 64, "float16", True, 3),
    ("causal_mha_fp16_d128", 1, 2, 2, 160, 160, 128, "float16", True, 4),
    ("noncausal_mha_fp16_scale", 1, 2, 2, 33, 47, 32, "float16", False, 5),
]


def main(ref_dir):
    sys.path.insert(0, ref_dir)
    from reference_implementations import naive_attention_with_scores as ref_fn

    here = os.path.dirname(os.path.abspath(__file__))
    for name, B, Hq, Hk, M, N, D, dtype, causal, seed in CASES:
        g = torch.Generator().manual_seed(seed)
        dt = getattr(torch, dtype)
        q = torch.randn(B, Hq, M, D, generator=g).to(dt).float()
        k = torch.randn(B, Hk, N, D, generator=g).to(dt).float()
        v = torch.randn(B, Hk, N, D, generator=g).to(dt).float()
        sm_scale = 0.25 if name.endswith("_scale") else None
        out, scores = ref_fn(q, k, v, causal, sm_scale=sm_scale)
        np.savez_compressed(
            os.path.join(here, name + ".npz"),
            q=q.numpy(), k=k.numpy(), v=v.numpy(),
            out=out.numpy(), scores=scores.numpy(),
            causal=np.array(causal), dtype=np.array(dtype),
            sm_scale=np.array(-1.0 if sm_scale is None else sm_scale),
        )
        print(name, tuple(scores.shape))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    main(sys.argv[1])
