"""ctypes binding of libfa_b200.so (C ABI in include/fa_b200.h).

There is no fallback: if the shared library is missing or a call fails, an exception is raised.
Build it with `python -m flash_attention_b200.csrc.build` (or `__graft_entry__.build()`).
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "csrc", "libfa_b200.so")

FA_DTYPE_FP16 = 0
FA_DTYPE_BF16 = 1

c_i32, c_i64, c_u64, c_f32, c_vp = C.c_int32, C.c_int64, C.c_uint64, C.c_float, C.c_void_p


class FaTensor(C.Structure):
    _fields_ = [("ptr", c_vp), ("stride_b", c_i64), ("stride_s", c_i64), ("stride_h", c_i64)]


class FaFwdArgs(C.Structure):
    _fields_ = [
        ("q", FaTensor), ("k", FaTensor), ("v", FaTensor), ("out", FaTensor),
        ("softmax_lse", c_vp),
        ("lse_seqlen", c_i32),
        ("batch", c_i32), ("seqlen_q", c_i32), ("seqlen_k", c_i32), ("heads", c_i32), ("heads_k", c_i32),
        ("head_dim", c_i32),
        ("dtype", c_i32),
        ("softmax_scale", c_f32),
        ("window_left", c_i32), ("window_right", c_i32),
        ("cu_seqlens_q", c_vp), ("cu_seqlens_k", c_vp),
        ("total_q", c_i32), ("total_k", c_i32),
        ("seqused_k", c_vp),
        ("seqused_k_extra", c_i32),
        ("kv_batch_idx", c_vp),
        ("p_dropout", c_f32),
        ("rng_seed", c_u64), ("rng_offset", c_u64),
        ("s_dmask", c_vp),
        ("sdmask_rows", c_i32), ("sdmask_cols", c_i32),
        ("num_splits", c_i32),
        ("lse_accum", c_vp), ("out_accum", c_vp),
        ("use_mask_shift", c_i32), ("mask_shift", c_i32),
        ("block_table", c_vp), ("block_table_stride", c_i32), ("page_block_size", c_i32),
    ]


class FaBwdArgs(C.Structure):
    _fields_ = [
        ("q", FaTensor), ("k", FaTensor), ("v", FaTensor), ("out", FaTensor), ("dout", FaTensor),
        ("dq", FaTensor), ("dk", FaTensor), ("dv", FaTensor),
        ("softmax_lse", c_vp),
        ("lse_seqlen", c_i32),
        ("softmax_d", c_vp),
        ("d_seqlen", c_i32),
        ("dq_accum", c_vp),
        ("batch", c_i32), ("seqlen_q", c_i32), ("seqlen_k", c_i32), ("heads", c_i32), ("heads_k", c_i32),
        ("head_dim", c_i32),
        ("dtype", c_i32),
        ("softmax_scale", c_f32),
        ("window_left", c_i32), ("window_right", c_i32),
        ("cu_seqlens_q", c_vp), ("cu_seqlens_k", c_vp),
        ("total_q", c_i32), ("total_k", c_i32),
        ("p_dropout", c_f32),
        ("rng_seed", c_u64), ("rng_offset", c_u64),
        ("use_mask_shift", c_i32), ("mask_shift", c_i32),
        ("accumulate_dkv", c_i32),
        ("dk_accum", c_vp), ("dv_accum", c_vp),
        ("parts", c_i32),
        ("deterministic", c_i32),
    ]


class FaKvcacheArgs(C.Structure):
    _fields_ = [
        ("q", FaTensor), ("kcache", FaTensor), ("vcache", FaTensor), ("out", FaTensor),
        ("knew", FaTensor), ("vnew", FaTensor),
        ("softmax_lse", c_vp),
        ("batch", c_i32), ("batch_cache", c_i32), ("seqlen_q", c_i32), ("seqlen_cache", c_i32),
        ("seqlen_new", c_i32), ("heads", c_i32), ("heads_k", c_i32), ("head_dim", c_i32),
        ("dtype", c_i32),
        ("softmax_scale", c_f32),
        ("window_left", c_i32), ("window_right", c_i32),
        ("cache_seqlens", c_vp), ("cache_batch_idx", c_vp),
        ("rotary_cos", c_vp), ("rotary_sin", c_vp),
        ("rotary_dim", c_i32), ("seqlen_ro", c_i32), ("rotary_interleaved", c_i32),
        ("q_rows_share_position", c_i32),
        ("num_splits", c_i32),
        ("lse_accum", c_vp), ("out_accum", c_vp),
        ("q_rotated", c_vp),
        ("block_table", c_vp), ("block_table_stride", c_i32), ("page_block_size", c_i32),
    ]


class FaRotaryArgs(C.Structure):
    _fields_ = [
        ("x", FaTensor), ("out", FaTensor),
        ("cos", c_vp), ("sin", c_vp),
        ("seqlen_offsets", c_vp), ("cu_seqlens", c_vp),
        ("batch", c_i32), ("seqlen", c_i32), ("heads", c_i32), ("head_dim", c_i32),
        ("total", c_i32),
        ("rotary_dim", c_i32), ("seqlen_ro", c_i32),
        ("seqlen_offset", c_i32),
        ("dtype", c_i32),
        ("interleaved", c_i32),
        ("conjugate", c_i32),
    ]


EXPORTS = (
    "fa_fwd", "fa_bwd", "fa_fwd_kvcache", "fa_fwd_num_splits", "fa_kvcache_plan", "fa_bwd_workspace_bytes",
    "fa_combine", "fa_last_error", "fa_build_info", "fa_device_status", "fa_abi_struct_size",
    "fa_fwd_kvcache_noalloc", "fa_noalloc_scratch_bytes", "fa_merge_partial", "fa_rotary",
    "fa_selftest_wait_timeout", "fa_selftest_device_once", "fa_last_path",
)

_lib = None


def lib():
    """Loads (once) and returns the shared library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                "libfa_b200.so not found at %s: build it with `python -m flash_attention_b200.csrc.build`; "
                "there is no CPU or PyTorch fallback" % LIB_PATH
            )
        L = C.CDLL(LIB_PATH)
        L.fa_fwd.argtypes = [C.POINTER(FaFwdArgs), c_vp]
        L.fa_fwd.restype = C.c_int
        L.fa_bwd.argtypes = [C.POINTER(FaBwdArgs), c_vp]
        L.fa_bwd.restype = C.c_int
        L.fa_fwd_kvcache.argtypes = [C.POINTER(FaKvcacheArgs), c_vp]
        L.fa_fwd_kvcache.restype = C.c_int
        L.fa_fwd_kvcache_noalloc.argtypes = [C.POINTER(FaKvcacheArgs), c_vp]
        L.fa_fwd_kvcache_noalloc.restype = C.c_int
        L.fa_noalloc_scratch_bytes.restype = c_i64
        L.fa_fwd_num_splits.argtypes = [c_i32] * 6
        L.fa_fwd_num_splits.restype = C.c_int
        L.fa_kvcache_plan.argtypes = [C.POINTER(FaKvcacheArgs), c_i32, C.POINTER(c_i64), C.POINTER(c_i64)]
        L.fa_kvcache_plan.restype = C.c_int
        L.fa_bwd_workspace_bytes.argtypes = [c_i32] * 6
        L.fa_bwd_workspace_bytes.restype = c_i64
        L.fa_combine.argtypes = [c_vp, c_vp, c_vp, c_vp, c_i32, c_i64, c_i32, c_i64, c_i32, c_vp]
        L.fa_combine.restype = C.c_int
        L.fa_merge_partial.argtypes = [C.POINTER(FaTensor), c_vp, c_i64, c_i64, C.POINTER(FaTensor), c_vp, c_i64, c_i64,
                                       c_i32, c_i32, c_i32, c_i32, c_i32, c_vp]
        L.fa_merge_partial.restype = C.c_int
        L.fa_rotary.argtypes = [C.POINTER(FaRotaryArgs), c_vp]
        L.fa_rotary.restype = C.c_int
        L.fa_last_error.restype = C.c_char_p
        L.fa_build_info.restype = C.c_char_p
        L.fa_last_path.restype = C.c_char_p
        L.fa_device_status.restype = C.c_int
        L.fa_selftest_wait_timeout.argtypes = [c_i64, c_vp]
        L.fa_selftest_wait_timeout.restype = C.c_int
        L.fa_selftest_device_once.argtypes = [C.POINTER(c_i32), c_i32, C.POINTER(c_i32)]
        L.fa_selftest_device_once.restype = C.c_int
        L.fa_abi_struct_size.argtypes = [c_i32]
        L.fa_abi_struct_size.restype = C.c_int
        for which, st in enumerate((FaTensor, FaFwdArgs, FaBwdArgs, FaKvcacheArgs, FaRotaryArgs)):
            if L.fa_abi_struct_size(which) != C.sizeof(st):
                raise ImportError("libfa_b200.so and flash_attention_b200/_lib.py disagree on the layout of %s" % st.__name__)
        _lib = L
    return _lib


def last_error():
    return lib().fa_last_error().decode()


def last_path():
    """Kernels launched by this process's last fa_fwd / fa_bwd / fa_fwd_kvcache call (any thread)."""
    return lib().fa_last_path().decode()


def check(status, what):
    if status != 0:
        raise RuntimeError("%s: %s" % (what, last_error()))


def tensor3(t, varlen=False):
    """FaTensor of a (batch, seq, head, dim) tensor, or of a packed (total, head, dim) one."""
    if t is None:
        return FaTensor(None, 0, 0, 0)
    if varlen:
        return FaTensor(t.data_ptr(), 0, t.stride(0), t.stride(1))
    return FaTensor(t.data_ptr(), t.stride(0), t.stride(1), t.stride(2))


def ptr(t):
    return None if t is None else t.data_ptr()
