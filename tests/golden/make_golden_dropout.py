"""Generate tests/golden/dropout_*.npz: the reference's Triton kernels with dropout_p > 0, run
through Triton's CPU interpreter (TRITON_INTERPRET=1).

    python tests/golden/make_golden_dropout.py /path/to/Flash_Attn_with_Score

The reference draws (seed, offset) from torch's CUDA generator (dropout.py:5-15), which does not
exist on a CPU box; every operator module's `philox_cuda_seed_offset` is replaced here by a stand-in
that returns the fixed pair stored in the fixture, so the unmodified wrappers and kernels run on CPU
tensors.  Device queries are answered as in make_golden_kernels.py.  A second fixture,
dropout_philox_stream.npz, holds `tl.rand(seed, offsets, n_rounds=6)` itself (Triton's Philox, the
generator the reference kernels call at flash.py:465) for a few seeds and offset ranges.
"""
import contextlib
import importlib.util
import os
import sys
import types

os.environ["TRITON_INTERPRET"] = "1"

import numpy as np
import torch
import triton
import triton.language as tl

torch.cuda.device_of = lambda t: 0
torch.cuda.get_device_properties = lambda d=None: types.SimpleNamespace(multi_processor_count=1)
torch.cuda.device = lambda d: contextlib.nullcontext()
torch.cuda.get_device_capability = lambda d=None: (8, 0)

CASES = [
    # name, B, Hq, Hk, M, N, D, causal, split, data seed, dropout_p, philox seed, philox offset
    ("dropout_causal_gqa_fp16", 2, 4, 2, 96, 96, 32, True, 40, 20, 0.1, 1234567, 0),
    ("dropout_noncausal_mha_fp16_ragged", 1, 2, 2, 70, 100, 64, False, 33, 21, 0.35, (7 << 32) + 99, 4096),
]


@triton.jit
def _rand_kernel(out_ptr, seed, offset, n: tl.constexpr):
    idx = tl.arange(0, n)
    tl.store(out_ptr + idx, tl.rand(seed, offset + idx, n_rounds=6))


def main(ref_dir):
    spec = importlib.util.spec_from_file_location(
        "faws_reference", os.path.join(ref_dir, "__init__.py"), submodule_search_locations=[ref_dir])
    ref = importlib.util.module_from_spec(spec)
    sys.modules["faws_reference"] = ref
    spec.loader.exec_module(ref)
    here = os.path.dirname(os.path.abspath(__file__))

    streams = {}
    for i, (seed, offset) in enumerate([(0, 0), (1234567, 0), ((7 << 32) + 99, 4096), (42, 2**31 - 700)]):
        out = torch.empty(1024, dtype=torch.float32)
        _rand_kernel[(1,)](out, seed, offset, 1024)
        streams[f"seed{i}"] = np.array([seed, offset], dtype=np.int64)
        streams[f"rand{i}"] = out.numpy()
    np.savez_compressed(os.path.join(here, "dropout_philox_stream.npz"), **streams)
    print("philox stream", {k: v[:3] for k, v in streams.items() if k.startswith("rand")})

    for name, B, Hq, Hk, M, N, D, causal, split, dseed, p_drop, pseed, poff in CASES:
        for mod in list(sys.modules.values()):
            if getattr(mod, "__name__", "").startswith("faws_reference") and hasattr(mod, "philox_cuda_seed_offset"):
                mod.philox_cuda_seed_offset = lambda increment, device=None: (pseed, poff)
        g = torch.Generator().manual_seed(dseed)
        q = torch.randn(B, Hq, M, D, generator=g).half()
        k = torch.randn(B, Hk, N, D, generator=g).half()
        v = torch.randn(B, Hk, N, D, generator=g).half()
        res = {}
        o, L, _tot, s_seed, s_off = ref.attention(q, k, v, causal, dropout_p=p_drop, return_log_normalizer=True,
                                            return_seed_offset=True)
        assert (s_seed, s_off) == (pseed, poff)
        res["attention_out"], res["attention_L"] = o, L
        for fn, key in [
            ("attention_with_scores", "scores"),
            ("attention_with_row_sum", "row_sum"),
            ("attention_with_col_sum", "col_sum"),
            ("attention_with_col_sum_sequential", "col_sum_sequential"),
            ("attention_with_softmax_col_sum", "softmax_col_sum"),
        ]:
            o, aux = getattr(ref, fn)(q, k, v, causal, dropout_p=p_drop)
            res[key + "_out"], res[key] = o, aux
        for fn, key in [
            ("attention_cross_token_qk_sum", "cross_qk"),
            ("attention_cross_token_softmax_sum", "cross_softmax"),
            ("attention_cross_token_softmax_sum_buffered", "cross_softmax_buffered"),
        ]:
            o, aux = getattr(ref, fn)(q, k, v, split, causal, dropout_p=p_drop)
            res[key + "_out"], res[key] = o, aux
        arrays = {kk: vv.numpy() for kk, vv in res.items()}
        np.savez_compressed(
            os.path.join(here, name + ".npz"), q=q.numpy(), k=k.numpy(), v=v.numpy(), causal=np.array(causal),
            split=np.array(split), dropout_p=np.array(p_drop, dtype=np.float64),
            philox=np.array([pseed, poff], dtype=np.int64), **arrays)
        print(name, {kk: tuple(vv.shape) for kk, vv in arrays.items()})


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    main(sys.argv[1])
