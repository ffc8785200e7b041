"""CPU-only checks of the boundary: the shared library loads, exports every symbol that
include/fa_b200.h declares, agrees with the ctypes layout, validates arguments before any launch,
and the drop-in module has the five entry points of the reference's extension."""
import ctypes
import inspect
import os
import re
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from flash_attention_b200.csrc import build as b

    b.build()
    from flash_attention_b200 import _lib

    return _lib.lib()


def test_every_declared_symbol_is_exported(lib):
    header = open(os.path.join(ROOT, "include", "fa_b200.h")).read()
    names = set(re.findall(r"^(?:int|int64_t|const char\*)\s+(fa_\w+)\s*\(", header, flags=re.M))
    from flash_attention_b200 import _lib

    assert names == set(_lib.EXPORTS), names ^ set(_lib.EXPORTS)
    for n in names:
        assert getattr(lib, n) is not None


def test_struct_layouts_match(lib):
    from flash_attention_b200 import _lib

    for which, st in enumerate((_lib.FaTensor, _lib.FaFwdArgs, _lib.FaBwdArgs, _lib.FaKvcacheArgs, _lib.FaRotaryArgs)):
        assert lib.fa_abi_struct_size(which) == ctypes.sizeof(st)
    assert lib.fa_abi_struct_size(99) == -1
    assert b"sm_100a" in lib.fa_build_info()


def test_argument_validation_happens_before_launch(lib):
    from flash_attention_b200 import _lib

    a = _lib.FaFwdArgs()
    a.batch, a.seqlen_q, a.seqlen_k, a.heads, a.heads_k, a.head_dim, a.dtype = 1, 8, 8, 4, 3, 64, 1
    assert lib.fa_fwd(ctypes.byref(a), None) != 0
    assert b"heads" in lib.fa_last_error()
    a.heads_k, a.head_dim = 4, 260
    assert lib.fa_fwd(ctypes.byref(a), None) != 0
    assert b"256" in lib.fa_last_error()
    a.head_dim = 60
    assert lib.fa_fwd(ctypes.byref(a), None) != 0
    assert b"multiple of 8" in lib.fa_last_error()
    a.head_dim = 64
    assert lib.fa_fwd(ctypes.byref(a), None) != 0  # null q pointer
    assert b"null" in lib.fa_last_error()
    k = _lib.FaKvcacheArgs()
    k.batch, k.batch_cache, k.seqlen_q, k.seqlen_cache, k.heads, k.heads_k, k.head_dim, k.dtype = 1, 1, 1, 16, 4, 4, 64, 0
    k.num_splits = 200
    assert lib.fa_kvcache_plan(ctypes.byref(k), 148, None, None) < 0
    assert b"num_splits" in lib.fa_last_error()


def test_rotary_and_merge_validate_before_launch(lib):
    from flash_attention_b200 import _lib

    r = _lib.FaRotaryArgs()
    r.batch, r.seqlen, r.heads, r.head_dim, r.rotary_dim, r.seqlen_ro, r.dtype = 1, 8, 2, 64, 96, 8, 1
    assert lib.fa_rotary(ctypes.byref(r), None) != 0
    assert b"rotary_dim must be <= headdim" in lib.fa_last_error()
    r.rotary_dim, r.seqlen_ro = 32, 4
    assert lib.fa_rotary(ctypes.byref(r), None) != 0
    assert b"seqlen_ro must be >= seqlen" in lib.fa_last_error()
    r.seqlen_ro, r.head_dim = 8, 300
    assert lib.fa_rotary(ctypes.byref(r), None) != 0
    assert b"headdim <= 256" in lib.fa_last_error()
    r.head_dim, r.dtype = 64, 7
    assert lib.fa_rotary(ctypes.byref(r), None) != 0
    assert b"fp16 and bf16" in lib.fa_last_error()
    r.dtype = 0
    assert lib.fa_rotary(ctypes.byref(r), None) != 0  # null x
    assert b"null" in lib.fa_last_error()
    r.seqlen = 0
    assert lib.fa_rotary(ctypes.byref(r), None) == 0  # nothing to do
    t = _lib.FaTensor(None, 0, 0, 0)
    assert lib.fa_merge_partial(ctypes.byref(t), None, 0, 0, ctypes.byref(t), None, 0, 0, 1, 1, 1, 64, 1, None) != 0
    assert b"null" in lib.fa_last_error()


def test_split_heuristic_matches_reference_rules(lib):
    # flash_api.cpp:206-246: no split once 80 % of the SMs are covered; never more splits than key blocks
    assert lib.fa_fwd_num_splits(16, 16, 2048, 2048, 128, 148) == 1
    assert lib.fa_fwd_num_splits(1, 2, 64, 64, 128, 148) == 1
    s = lib.fa_fwd_num_splits(1, 2, 64, 8192, 128, 148)
    assert 1 < s <= 128
    # the dQ workspace covers both layouts: plain rows and whole 128-row blocks of the padded head dim
    assert lib.fa_bwd_workspace_bytes(2, 100, 4, 64, 0, 0) == 2 * 100 * 4 * 64 * 4
    assert lib.fa_bwd_workspace_bytes(2, 100, 4, 64, 150, 1) == 150 * 4 * 64 * 4
    assert lib.fa_bwd_workspace_bytes(16, 2048, 16, 128, 0, 0) == 16 * 2048 * 16 * 128 * 4
    assert lib.fa_noalloc_scratch_bytes() == 24 << 20


def test_dropin_module_has_the_reference_entry_points():
    import flash_attn_2_cuda as ext

    assert os.path.dirname(os.path.abspath(ext.__file__)).startswith(ROOT), "an unrelated flash_attn_2_cuda shadows the shim"
    # positional arities of csrc/flash_attn/flash_api.cpp:248-259, 426-442, 609-625, 813-834, 1038-1055
    want = {"fwd": 11, "varlen_fwd": 16, "bwd": 16, "varlen_bwd": 21, "fwd_kvcache": 16}
    extra = {"bwd": {"deterministic"}, "varlen_bwd": {"deterministic"}, "fwd_kvcache": {"block_table"}}
    for name, n in want.items():
        params = inspect.signature(getattr(ext, name)).parameters.values()
        positional = [p for p in params if p.kind == inspect.Parameter.POSITIONAL_OR_KEYWORD]
        assert len(positional) == n and all(p.default is inspect.Parameter.empty for p in positional), name
        # what goes beyond this version of the reference is keyword-only and optional
        kw_only = {p.name for p in params if p.kind == inspect.Parameter.KEYWORD_ONLY}
        assert kw_only == extra.get(name, set()), name
        assert all(p.default is not inspect.Parameter.empty for p in params if p.kind == inspect.Parameter.KEYWORD_ONLY)


def test_shim_raises_runtime_error_like_torch_check():
    import flash_attn_2_cuda as ext

    q = torch.zeros(1, 4, 2, 16, dtype=torch.float32)
    with pytest.raises(RuntimeError, match="fp16 and bf16"):
        ext.fwd(q, q, q, None, 0.0, 1.0, False, -1, -1, False, None)
    q = q.half()
    with pytest.raises(RuntimeError, match="CUDA"):
        ext.fwd(q, q, q, None, 0.0, 1.0, False, -1, -1, False, None)


def _reference_interface_file():
    """flash_attn/flash_attn_interface.py of an unmodified FlashAttention v2.3.3: from the tree named by
    FLASH_ATTN_REFERENCE_TREE, else from the python-only install under baseline/_ref of this repository."""
    roots = [os.environ.get("FLASH_ATTN_REFERENCE_TREE"), os.path.join(ROOT, "baseline", "_ref")]
    for r in roots:
        if r and os.path.exists(os.path.join(r, "flash_attn", "flash_attn_interface.py")):
            return os.path.join(r, "flash_attn", "flash_attn_interface.py")
    return None


@pytest.mark.skipif(_reference_interface_file() is None, reason="reference tree not present")
def test_unmodified_reference_interface_binds_to_the_shim():
    # the reference's python API file, loaded as is, must find everything it calls in our module
    import importlib.util

    import flash_attn_2_cuda as ext

    spec = importlib.util.spec_from_file_location("ref_iface", _reference_interface_file())
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    assert mod.flash_attn_cuda is ext
    for fn in ("flash_attn_func", "flash_attn_qkvpacked_func", "flash_attn_varlen_func", "flash_attn_with_kvcache"):
        assert callable(getattr(mod, fn))


def test_per_device_setup_runs_once_per_device(lib):
    # the launchers raise a kernel's shared-memory limit once per DEVICE (the attribute is per device):
    # replay the bookkeeping for a process that alternates between GPUs
    devs = [0, 0, 1, 0, 1, 2, 63, 63, 64, 64, -1, -1]
    arr = (ctypes.c_int32 * len(devs))(*devs)
    out = (ctypes.c_int32 * len(devs))()
    assert lib.fa_selftest_device_once(arr, len(devs), out) == 0
    # ordinals outside the 64-entry table are configured on every call rather than never
    assert list(out) == [1, 0, 1, 0, 0, 1, 1, 0, 1, 1, 1, 1]


def test_paged_cache_arguments_are_validated_before_launch(lib):
    """block_table rules of FaKvcacheArgs / FaFwdArgs, checked on the host (fa_kvcache_plan launches nothing)."""
    from flash_attention_b200 import _lib

    a = _lib.FaKvcacheArgs()
    a.batch, a.batch_cache, a.seqlen_q, a.seqlen_cache, a.heads, a.heads_k, a.head_dim, a.dtype = 2, 9, 1, 1024, 8, 2, 128, 1
    table = (ctypes.c_int32 * 8)(*range(8))
    a.block_table = ctypes.cast(table, ctypes.c_void_p)
    a.block_table_stride, a.page_block_size = 4, 256
    assert lib.fa_kvcache_plan(ctypes.byref(a), 148, None, None) >= 1  # 4 pages of 256 rows per sequence
    a.page_block_size = 96
    assert lib.fa_kvcache_plan(ctypes.byref(a), 148, None, None) == -1
    assert b"divisible by 64" in lib.fa_last_error()
    a.page_block_size, a.seqlen_cache = 256, 2048  # more pages than a row of the table holds
    assert lib.fa_kvcache_plan(ctypes.byref(a), 148, None, None) == -1
    assert b"block_table" in lib.fa_last_error()
    a.seqlen_cache = 1000  # not whole pages
    assert lib.fa_kvcache_plan(ctypes.byref(a), 148, None, None) == -1
    a.seqlen_cache = 1024
    idx = (ctypes.c_int32 * 2)(0, 1)
    a.cache_batch_idx = ctypes.cast(idx, ctypes.c_void_p)
    assert lib.fa_kvcache_plan(ctypes.byref(a), 148, None, None) == -1
    assert b"cache_batch_idx" in lib.fa_last_error()
    # a paged pool may hold fewer pages than there are sequences x pages (sharing) or more: batch_cache is not compared
    # with batch
    a.cache_batch_idx = None
    a.batch_cache = 1
    assert lib.fa_kvcache_plan(ctypes.byref(a), 148, None, None) >= 1
    # the plan (split count, workspace sizes) of a paged call is that of the contiguous call of the same capacity
    lb, ob, lb2, ob2 = (ctypes.c_int64(0) for _ in range(4))
    paged = lib.fa_kvcache_plan(ctypes.byref(a), 148, ctypes.byref(lb), ctypes.byref(ob))
    a.block_table, a.block_table_stride, a.page_block_size, a.batch_cache = None, 0, 0, 2
    flat = lib.fa_kvcache_plan(ctypes.byref(a), 148, ctypes.byref(lb2), ctypes.byref(ob2))
    assert paged == flat and lb.value == lb2.value and ob.value == ob2.value

    f = _lib.FaFwdArgs()
    f.batch, f.seqlen_q, f.seqlen_k, f.heads, f.heads_k, f.head_dim, f.dtype = 1, 8, 512, 4, 4, 64, 1
    buf = ctypes.create_string_buffer(4096 + 64)
    base = (ctypes.addressof(buf) + 15) & ~15
    for t in (f.q, f.k, f.v, f.out):
        t.ptr, t.stride_b, t.stride_s, t.stride_h = base, 0, 64, 64
    f.softmax_lse = base
    f.block_table = ctypes.cast(table, ctypes.c_void_p)
    f.block_table_stride, f.page_block_size = 4, 100
    assert lib.fa_fwd(ctypes.byref(f), None) == 1 and b"divisible by 64" in lib.fa_last_error()
    f.page_block_size = 64  # 4 pages x 64 rows < 512 keys
    assert lib.fa_fwd(ctypes.byref(f), None) == 1 and b"cover seqlen_k" in lib.fa_last_error()
    f.block_table_stride = 8
    f.kv_batch_idx = ctypes.cast(idx, ctypes.c_void_p)
    assert lib.fa_fwd(ctypes.byref(f), None) == 1 and b"paged" in lib.fa_last_error()
