"""Generates tests/golden/*.npz from the reference's own Python attention.

Run where a checkout of Bruce-Lee-LY/decoding_attention is available (path as the first argument):

    python tests/golden/make_golden.py [/path/to/reference]

It imports ``torch_attn`` from the reference's tests/test_decoding_attn.py:35-57 (the function the
reference's pytest suite uses as its expected value) and evaluates it on seeded inputs from
decoding_attention_b200.synth, once in the input dtype (as the reference's tests do, on the CPU
here) and once on fp32 copies of the same 16-bit inputs.  Inputs are stored as raw 16-bit patterns
so that a fixture is self-contained.  The reference test module imports the reference's CUDA
extension at import time; a stub module takes its place, since only ``torch_attn`` is used.
"""
import importlib.util
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from decoding_attention_b200 import synth  # noqa: E402

# name, dtype, batch, seq_k, head_q, head_k, dim, dim_v, dist, scale
CASES = [
    ("mha_fp16", torch.float16, 2, 96, 4, 4, 128, 128, "uniform", 1.0),
    ("gqa_bf16", torch.bfloat16, 3, 77, 8, 2, 128, 128, "normal", 0.5),
    ("gqa_fp16_d64", torch.float16, 2, 33, 32, 8, 64, 64, "normal", 1.0),
    ("gqa_bf16_d96", torch.bfloat16, 2, 65, 32, 8, 96, 96, "normal", 1.0),
    ("mha_fp16_d256", torch.float16, 1, 40, 4, 4, 256, 256, "normal", 1.0),
    ("mqa_fp16", torch.float16, 2, 100, 32, 1, 128, 128, "uniform", 1.0),
    ("mla_bf16", torch.bfloat16, 2, 48, 16, 1, 576, 512, "normal", 0.3),
    ("mla_fp16_h128", torch.float16, 1, 19, 128, 1, 576, 512, "normal", 0.3),
    ("one_key_fp16", torch.float16, 2, 1, 32, 8, 128, 128, "normal", 1.0),
]


def load_torch_attn(ref_root):
    stub = types.ModuleType("decoding_attn")
    stub.decoding_attn_fwd = None
    sys.modules["decoding_attn"] = stub
    spec = importlib.util.spec_from_file_location("ref_test_decoding_attn",
                                                  os.path.join(ref_root, "tests", "test_decoding_attn.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    del sys.modules["decoding_attn"]
    return mod.torch_attn


def main():
    from oracle import attn_oracle
    ref_root = sys.argv[1] if len(sys.argv) > 1 else attn_oracle.reference_dir()
    if not ref_root:
        sys.exit("usage: make_golden.py <checkout of the reference project>")
    torch_attn = load_torch_attn(ref_root)
    for name, dtype, batch, seq_k, head_q, head_k, dim, dim_v, dist, scale in CASES:
        mla = dim != dim_v
        w = synth.Workload(name, dtype, head_q, head_k, dim, dim_v, [seq_k] * batch, dist=dist, scale=scale,
                           mla=mla, seed=4321)
        q, k, v, cu = w.make("cpu")
        q4 = q.reshape(batch, 1, head_q, dim)
        k4 = k.reshape(batch, seq_k, head_k, dim)
        v4 = None if mla else v.reshape(batch, seq_k, head_k, dim_v)
        kw = dict(dim_v=dim_v) if mla else dict(v=v4)
        o_native = torch_attn(q4, k4, **kw).reshape(batch, head_q, dim_v)
        kw32 = dict(dim_v=dim_v) if mla else dict(v=v4.float())
        o_f32 = torch_attn(q4.float(), k4.float(), **kw32).reshape(batch, head_q, dim_v)
        arrays = dict(
            q=q.view(torch.int16).numpy(), k=k.view(torch.int16).numpy(),
            cu_seq_k=cu.numpy(), o_native=o_native.contiguous().view(torch.int16).numpy(),
            o_f32=o_f32.contiguous().numpy(),
            meta=np.array([batch, seq_k, head_q, head_k, dim, dim_v, int(dtype == torch.bfloat16)], dtype=np.int64))
        if not mla:
            arrays["v"] = v.view(torch.int16).numpy()
        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, **arrays)
        print(name, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
