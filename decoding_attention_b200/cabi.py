"""ctypes view of the C ABI in include/decoding_attn_b200.h (libdecoding_attn_b200.so).

This is the binding a non-C++ host would write; the parity tests and the benchmark call the
library through it, with torch only providing the device (or pinned host) memory.  Importing it
fails loudly when the library has not been built: there is no fallback path.
"""
import ctypes
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("DA_LIB_PATH") or os.path.join(_PKG, "libdecoding_attn_b200.so")

DA_OK, DA_ERR_INVALID_ARG, DA_ERR_UNSUPPORTED, DA_ERR_WORKSPACE, DA_ERR_CUDA, DA_ERR_TIMEOUT = range(6)

EXPORTS = ["da_decode_fwd", "da_decode_fwd_host", "da_decode_fwd_static", "da_static_scratch_bytes", "da_decode_workspace_bytes", "da_decode_num_splits", "da_plan_num_splits",
           "da_merge_partials", "da_exchange_merge", "da_exchange_merge_bounded", "da_exchange_buffer_bytes", "da_set_profile_events", "da_selftest_wait_timeout", "da_device_status", "da_status_string", "da_last_error", "da_launch_count"]


class DecodeArgs(ctypes.Structure):
    """Mirror of ``da_decode_args_t``."""
    _fields_ = [
        ("struct_size", ctypes.c_uint32), ("is_bf16", ctypes.c_int32), ("is_alibi", ctypes.c_int32),
        ("num_splits", ctypes.c_int32),
        ("q", ctypes.c_void_p), ("k", ctypes.c_void_p), ("v", ctypes.c_void_p), ("o", ctypes.c_void_p),
        ("cu_seq_k", ctypes.c_void_p),
        ("max_seq_k", ctypes.c_int64), ("batch", ctypes.c_int64), ("head_q", ctypes.c_int64),
        ("head_k", ctypes.c_int64), ("dim", ctypes.c_int64), ("dim_v", ctypes.c_int64),
        ("q_row_stride", ctypes.c_int64), ("k_row_stride", ctypes.c_int64), ("v_row_stride", ctypes.c_int64),
        ("o_row_stride", ctypes.c_int64),
        ("softmax_scale", ctypes.c_float), ("total_k", ctypes.c_uint32),
        ("lse", ctypes.c_void_p), ("o_f32", ctypes.c_void_p),
        ("kv_pos_offset", ctypes.c_void_p), ("kv_total_len", ctypes.c_void_p),
        ("workspace", ctypes.c_void_p), ("workspace_bytes", ctypes.c_size_t),
        ("stream", ctypes.c_void_p),
        ("block_table", ctypes.c_void_p), ("block_table_stride", ctypes.c_int64),
        ("page_size", ctypes.c_int32),
        ("kv_dtype", ctypes.c_int32), ("k_scale", ctypes.c_float), ("v_scale", ctypes.c_float),
    ]


class DecodingAttnError(RuntimeError):
    def __init__(self, status, message):
        super().__init__(f"decoding_attn_b200 status {status}: {message}")
        self.status = status


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: run `python -m decoding_attention_b200.build` "
                              "(there is no CPU or PyTorch fallback)")
        l = ctypes.CDLL(LIB_PATH)
        l.da_decode_fwd.restype = ctypes.c_int
        l.da_decode_fwd.argtypes = [ctypes.POINTER(DecodeArgs)]
        l.da_decode_fwd_host.restype = ctypes.c_int
        l.da_decode_fwd_host.argtypes = [ctypes.POINTER(DecodeArgs)]
        l.da_decode_fwd_static.restype = ctypes.c_int
        l.da_decode_fwd_static.argtypes = [ctypes.POINTER(DecodeArgs)]
        l.da_static_scratch_bytes.restype = ctypes.c_size_t
        l.da_decode_workspace_bytes.restype = ctypes.c_size_t
        l.da_decode_workspace_bytes.argtypes = [ctypes.POINTER(DecodeArgs)]
        l.da_decode_num_splits.restype = ctypes.c_int
        l.da_decode_num_splits.argtypes = [ctypes.POINTER(DecodeArgs)]
        l.da_plan_num_splits.restype = ctypes.c_int
        l.da_plan_num_splits.argtypes = [ctypes.POINTER(DecodeArgs), ctypes.c_int]
        l.da_merge_partials.restype = ctypes.c_int
        l.da_merge_partials.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64,
                                        ctypes.c_int32, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64,
                                        ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                        ctypes.c_int32, ctypes.c_void_p]
        l.da_exchange_merge.restype = ctypes.c_int
        l.da_exchange_merge.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p), ctypes.c_int32, ctypes.c_int32,
                                        ctypes.c_int64, ctypes.c_int32, ctypes.c_uint32, ctypes.c_void_p,
                                        ctypes.c_void_p, ctypes.c_int32, ctypes.c_void_p]
        l.da_exchange_merge_bounded.restype = ctypes.c_int
        l.da_exchange_merge_bounded.argtypes = l.da_exchange_merge.argtypes + [ctypes.c_int64]
        l.da_exchange_buffer_bytes.restype = ctypes.c_size_t
        l.da_exchange_buffer_bytes.argtypes = [ctypes.c_int32, ctypes.c_int64, ctypes.c_int32]
        l.da_set_profile_events.restype = None
        l.da_set_profile_events.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
        l.da_selftest_wait_timeout.restype = ctypes.c_int
        l.da_selftest_wait_timeout.argtypes = [ctypes.c_void_p]
        l.da_device_status.restype = ctypes.c_int
        l.da_status_string.restype = ctypes.c_char_p
        l.da_status_string.argtypes = [ctypes.c_int]
        l.da_last_error.restype = ctypes.c_char_p
        l.da_launch_count.restype = ctypes.c_uint64
        _lib = l
    return _lib


def check(status):
    if status != DA_OK:
        raise DecodingAttnError(status, lib().da_last_error().decode())


def _ptr(t):
    return None if t is None else t.data_ptr()


def make_args(q, k, v, o, cu_seq_k, max_seq_k, dim_v, is_alibi=False, softmax_scale=None, lse=None, o_f32=None,
              kv_pos_offset=None, kv_total_len=None, workspace=None, num_splits=0, stream=0, packed=False,
              block_table=None, page_size=0, k_scale=None, v_scale=None, int4=False):
    """Fill a DecodeArgs from torch tensors (device tensors, or host tensors for the *_host call).

    Paged cache: pass ``block_table`` (int32 [batch, blocks]) and ``page_size``; ``k`` / ``v`` are then the
    page pools, either [num_pages * page_size, head_k, dim] or [num_pages, page_size, head_k, dim].
    Quantised cache (q and o stay fp16 / bf16) with per-tensor ``k_scale`` / ``v_scale`` (default 1): ``k`` / ``v``
    of dtype torch.float8_e4m3fn or torch.int8; or, with ``int4=True``, torch.uint8 tensors [rows, head_k, dim / 2]
    holding two signed 4-bit values per byte (even element in the low nibble)."""
    import torch
    a = DecodeArgs()
    a.struct_size = ctypes.sizeof(DecodeArgs)
    a.is_bf16 = int(q.dtype == torch.bfloat16)
    a.is_alibi = int(bool(is_alibi))
    a.num_splits = int(num_splits)
    a.q, a.k, a.v, a.o, a.cu_seq_k = _ptr(q), _ptr(k), _ptr(v), _ptr(o), _ptr(cu_seq_k)
    a.max_seq_k = int(max_seq_k)
    a.total_k = min(int(k.shape[0]), 0xFFFFFFFF) if block_table is None and k.dim() == 3 else 0  # packed cache: its rows
    a.batch = cu_seq_k.numel() - 1
    if block_table is not None and k.dim() == 4:  # [num_pages, page_size, head_k, dim] -> rows
        k = k.view(-1, k.shape[2], k.shape[3])
        v = v.view(-1, v.shape[2], v.shape[3]) if v is not None else None
    a.head_q, a.dim = q.shape[1], q.shape[2]
    a.head_k = k.shape[1]
    per_byte = 2 if int4 else 1  # elements per stored byte: strides are given in elements
    a.dim_v = int(dim_v)
    if not packed:
        a.q_row_stride, a.k_row_stride = q.stride(0), k.stride(0) * per_byte
        a.v_row_stride = v.stride(0) * per_byte if v is not None else 0
        a.o_row_stride = o.stride(0) if o is not None else 0
    a.softmax_scale = float(softmax_scale) if softmax_scale else 0.0
    a.lse, a.o_f32 = _ptr(lse), _ptr(o_f32)
    a.kv_pos_offset, a.kv_total_len = _ptr(kv_pos_offset), _ptr(kv_total_len)
    if workspace is not None:
        a.workspace = workspace.data_ptr()
        a.workspace_bytes = workspace.numel() * workspace.element_size()
    a.stream = int(stream) if stream else None
    if int4 or k.dtype in (getattr(torch, "float8_e4m3fn", None), torch.int8):
        a.kv_dtype = 3 if int4 else (2 if k.dtype == torch.int8 else 1)
        a.k_scale = float(k_scale) if k_scale else 1.0
        a.v_scale = float(v_scale) if v_scale else 1.0
    if block_table is not None:
        a.block_table = block_table.data_ptr()
        a.block_table_stride = block_table.stride(0)
        a.page_size = int(page_size)
    return a


def decode_fwd(args):
    check(lib().da_decode_fwd(ctypes.byref(args)))


def decode_fwd_host(args):
    check(lib().da_decode_fwd_host(ctypes.byref(args)))


def decode_fwd_static(args):
    check(lib().da_decode_fwd_static(ctypes.byref(args)))


def workspace_bytes(args):
    return lib().da_decode_workspace_bytes(ctypes.byref(args))


def num_splits(args):
    return lib().da_decode_num_splits(ctypes.byref(args))


def plan_num_splits(args, sm_count):
    """Split count the planner picks for a device with `sm_count` SMs; touches no device."""
    return lib().da_plan_num_splits(ctypes.byref(args), int(sm_count))


def device_status():
    return lib().da_device_status()


def launch_count():
    return lib().da_launch_count()


def set_profile_events(start=None, stop=None):
    """torch.cuda.Event objects (already recorded once, so that they exist) or None."""
    lib().da_set_profile_events(start.cuda_event if start is not None else None,
                                stop.cuda_event if stop is not None else None)
