"""TEST INFRASTRUCTURE ONLY -- ctypes front end of the CPU oracle.

``attn_cpu`` wraps oracle/attn_cpu.cpp (this repository's restatement of the reference's
``Tester<T>::attn_cpu``, csrc/common/tester.h:133-259) and ``ref_attn_cpu`` wraps
oracle/_ref/libref_attn_cpu.so (the reference's own tester.h compiled as it is).  Only tests, the
smoke check and the benchmark's CPU-baseline leg may import this module; the product never does.
Tensors are torch CPU tensors of dtype float16 / bfloat16 (int32 for ``cu_seq_k``).
"""
import ctypes
import os
import subprocess

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None
_REF = None


def reference_dir():
    """A checkout of the reference project: $DA_REFERENCE_DIR, else a folder named "reference" beside this
    repository; None when neither exists."""
    cand = os.environ.get("DA_REFERENCE_DIR") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")
    return cand if os.path.isfile(os.path.join(cand, "csrc", "common", "tester.h")) else None


def build(quiet=True):
    """Compile the oracle (and the reference's CPU path when a reference checkout is present)."""
    ref = reference_dir()
    subprocess.run(["make", "-C", _HERE, "all"] + (["REF=" + ref] if ref else []), check=True,
                   stdout=subprocess.DEVNULL if quiet else None, stderr=subprocess.STDOUT if quiet else None)


def _lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "libattn_oracle.so")
        if not os.path.exists(path):
            build()
        lib = ctypes.CDLL(path)
        lib.oracle_attn_cpu.restype = ctypes.c_int
        lib.oracle_attn_cpu.argtypes = [ctypes.c_void_p] * 7 + [ctypes.c_int64] * 5 + [
            ctypes.c_int, ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_void_p,
            ctypes.c_int64, ctypes.c_int64, ctypes.c_int]
        lib.oracle_num_procs.restype = ctypes.c_int
        for n in ("oracle_half_to_float", "oracle_bf16_to_float"):
            getattr(lib, n).restype = ctypes.c_float
            getattr(lib, n).argtypes = [ctypes.c_uint16]
        for n in ("oracle_float_to_half", "oracle_float_to_bf16"):
            getattr(lib, n).restype = ctypes.c_uint16
            getattr(lib, n).argtypes = [ctypes.c_float]
        _LIB = lib
    return _LIB


def ref_available():
    return os.path.exists(os.path.join(_HERE, "_ref", "libref_attn_cpu.so"))


def _ref():
    global _REF
    if _REF is None:
        lib = ctypes.CDLL(os.path.join(_HERE, "_ref", "libref_attn_cpu.so"))
        lib.ref_attn_cpu.restype = ctypes.c_int
        lib.ref_attn_cpu.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_int64] * 6 + [ctypes.c_int] * 3
        _REF = lib
    return _REF


def num_procs():
    return _lib().oracle_num_procs()


def _chk(t, name):
    assert t.device.type == "cpu" and t.is_contiguous(), f"{name} must be a contiguous CPU tensor"
    return t


def attn_cpu(q, k, v, cu_seq_k, dim_v=None, is_alibi=False, softmax_scale=None, kv_pos_offset=None,
             kv_total_len=None, batch_range=None, threads=0, return_lse=False, return_f32=False):
    """Decode attention on the CPU, the way tester.h:133-259 computes it.

    q [batch, head_q, dim]; k [total_k, head_k, dim]; v [total_k, head_k, dim_v] or None (MLA: V is
    the first ``dim_v`` elements of each K row); cu_seq_k int32 [batch + 1].
    Returns o [batch, head_q, dim_v] in q's dtype (plus fp32 LSE / fp32 o if requested).
    """
    _chk(q, "q"), _chk(k, "k"), _chk(cu_seq_k, "cu_seq_k")
    assert q.dtype in (torch.float16, torch.bfloat16) and k.dtype == q.dtype and cu_seq_k.dtype == torch.int32
    batch = cu_seq_k.numel() - 1
    assert q.shape[0] == batch
    head_q, dim = q.shape[1], q.shape[2]
    head_k = k.shape[1]
    if v is not None:
        _chk(v, "v")
        assert v.dtype == q.dtype
        dim_v = v.shape[2]
    assert dim_v is not None
    o = torch.zeros(batch, head_q, dim_v, dtype=q.dtype)
    o32 = torch.zeros(batch, head_q, dim_v, dtype=torch.float32) if return_f32 else None
    lse = torch.zeros(batch, head_q, dtype=torch.float32) if return_lse else None
    b0, b1 = batch_range if batch_range is not None else (0, batch)
    for t in (kv_pos_offset, kv_total_len):
        assert t is None or (t.dtype == torch.int32 and t.numel() == batch and t.is_contiguous())
    rc = _lib().oracle_attn_cpu(
        q.data_ptr(), k.data_ptr(), v.data_ptr() if v is not None else None, o.data_ptr(),
        o32.data_ptr() if o32 is not None else None, lse.data_ptr() if lse is not None else None,
        cu_seq_k.data_ptr(), batch, head_q, head_k, dim, dim_v, int(is_alibi),
        int(q.dtype == torch.bfloat16), float(softmax_scale) if softmax_scale else 0.0,
        kv_pos_offset.data_ptr() if kv_pos_offset is not None else None,
        kv_total_len.data_ptr() if kv_total_len is not None else None, b0, b1, int(threads))
    if rc != 0:
        raise ValueError(f"oracle_attn_cpu rejected its arguments (code {rc})")
    out = [o]
    if return_lse:
        out.append(lse)
    if return_f32:
        out.append(o32)
    return out[0] if len(out) == 1 else tuple(out)


def ref_attn_cpu(q, k, v, seq_k, dim_v=None, is_alibi=False, threads=1):
    """The reference's own attn_cpu (compiled from its tester.h) on equal-length sequences."""
    _chk(q, "q"), _chk(k, "k")
    batch, head_q, dim = q.shape
    head_k = k.shape[1]
    assert k.shape[0] == batch * seq_k
    if v is not None:
        _chk(v, "v")
        dim_v = v.shape[2]
    o = torch.zeros(batch, head_q, dim_v, dtype=q.dtype)
    rc = _ref().ref_attn_cpu(q.data_ptr(), k.data_ptr(), v.data_ptr() if v is not None else None, o.data_ptr(),
                             batch, seq_k, head_q, head_k, dim, dim_v, int(is_alibi),
                             int(q.dtype == torch.bfloat16), int(threads))
    if rc != 0:
        raise ValueError(f"ref_attn_cpu rejected its arguments (code {rc})")
    return o
