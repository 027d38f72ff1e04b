"""Generate tests/golden/kernels_*.npz by running the reference's own Triton
kernels through Triton's CPU interpreter (TRITON_INTERPRET=1).

    python tests/golden/make_golden_kernels.py /path/to/Flash_Attn_with_Score

The reference's host wrappers query the CUDA device for tile selection only
(flash.py:300-331, attention_with_scores.py:259-263); those queries are
answered here with fixed stand-ins (sm_80, and an SM count of 1 so that `attention` takes its main kernel, not the split-KV decode path of split_kv.py:234-262) so that the unmodified
wrappers and kernels run on CPU tensors.  All nine exported entry points
(__init__.py:29-39) are called on the same seeded inputs and every returned
tensor is stored.  The fixtures travel with the repository.
"""
import contextlib
import importlib.util
import os
import sys
import types

os.environ["TRITON_INTERPRET"] = "1"

import numpy as np
import torch

torch.cuda.device_of = lambda t: 0
torch.cuda.get_device_properties = lambda d=None: types.SimpleNamespace(multi_processor_count=1)
torch.cuda.device = lambda d: contextlib.nullcontext()
torch.cuda.get_device_capability = lambda d=None: (8, 0)

CASES = [
    # name, B, Hq, Hk, M, N, D, dtype, causal, split, seed
    ("kernels_causal_gqa_fp16", 1, 4, 2, 160, 160, 32, "float16", True, 96, 10),
    ("kernels_noncausal_gqa_fp16", 1, 4, 2, 128, 96, 64, "float16", False, 80, 11),
    ("kernels_causal_mha_fp16_ragged", 1, 2, 2, 100, 100, 64, "float16", True, 37, 12),
]


def main(ref_dir):
    spec = importlib.util.spec_from_file_location(
        "faws_reference", os.path.join(ref_dir, "__init__.py"), submodule_search_locations=[ref_dir])
    ref = importlib.util.module_from_spec(spec)
    sys.modules["faws_reference"] = ref
    spec.loader.exec_module(ref)

    here = os.path.dirname(os.path.abspath(__file__))
    for name, B, Hq, Hk, M, N, D, dtype, causal, split, seed in CASES:
        g = torch.Generator().manual_seed(seed)
        dt = getattr(torch, dtype)
        q = torch.randn(B, Hq, M, D, generator=g).to(dt)
        k = torch.randn(B, Hk, N, D, generator=g).to(dt)
        v = torch.randn(B, Hk, N, D, generator=g).to(dt)
        res = {}
        o, L, tot = ref.attention(q, k, v, causal, return_log_normalizer=True,
                                  return_total_attention=True)[:3]
        res["attention_out"], res["attention_L"], res["attention_total"] = o, L, tot
        for fn, key in [
            ("attention_with_scores", "scores"),
            ("attention_with_row_sum", "row_sum"),
            ("attention_with_col_sum", "col_sum"),
            ("attention_with_col_sum_sequential", "col_sum_sequential"),
            ("attention_with_softmax_col_sum", "softmax_col_sum"),
        ]:
            o, aux = getattr(ref, fn)(q, k, v, causal)
            res[key + "_out"], res[key] = o, aux
        for fn, key in [
            ("attention_cross_token_qk_sum", "cross_qk"),
            ("attention_cross_token_softmax_sum", "cross_softmax"),
            ("attention_cross_token_softmax_sum_buffered", "cross_softmax_buffered"),
        ]:
            o, aux = getattr(ref, fn)(q, k, v, split, causal)
            res[key + "_out"], res[key] = o, aux
        arrays = {kk: vv.numpy() for kk, vv in res.items()}  # native dtype (fp16 / fp32)
        np.savez_compressed(
            os.path.join(here, name + ".npz"),
            q=q.numpy(), k=k.numpy(), v=v.numpy(),
            causal=np.array(causal), dtype=np.array(dtype), split=np.array(split), **arrays)
        print(name, {kk: tuple(vv.shape) for kk, vv in arrays.items()})


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    main(sys.argv[1])
