"""ctypes binding of libinfer_b200.so (the C ABI declared in include/infer_b200.h).

There is no fallback: if the shared library is missing the import of any op fails with
an ImportError that says how to build it.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

_HERE = Path(__file__).resolve().parent
LIB_PATH = _HERE / "libinfer_b200.so"

OK = 0
ERR_NULL, ERR_ALIGN, ERR_STRIDE, ERR_GEOMETRY, ERR_WORKSPACE, ERR_CUDA, ERR_DTYPE, ERR_DEVICE = range(-1, -9, -1)
ERR_TOO_LARGE = -9
ERR_STATE = -10
KV_BF16, KV_E4M3 = 0, 1

_vp, _i32, _i64, _sz, _f32 = C.c_void_p, C.c_int, C.c_int64, C.c_size_t, C.c_float

# name -> (restype, argtypes); one entry per declaration in include/infer_b200.h
SIGNATURES = {
    "infer_kv_pool_create": (_i32, [C.POINTER(_vp), _vp, _vp, _vp, _vp, _i64, _i32, _i32, _i32, _i32]),
    "infer_kv_pool_destroy": (_i32, [_vp]),
    "infer_kv_append": (_i32, [_vp, _vp, _vp, _i64, _i64, _vp, _i64, _vp, _sz, _vp]),
    "infer_kv_append_workspace_bytes": (_sz, [_vp]),
    "infer_qk_norm_rope_append": (_i32, [_vp, _vp, _i64, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _vp, _f32, _vp, _vp, _i64,
                                         _vp, _i64, _i32, _vp]),
    "infer_decode_step_advance": (_i32, [_vp, _vp, _vp, _vp, _i64, _i32, _i32, _i32, _vp]),
    "infer_paged_decode": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i32, _i32, _f32, _vp, _sz, _vp]),
    "infer_paged_decode_append": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _vp, _vp, _i64, _i32, _i32, _f32, _vp, _sz, _vp]),
    "infer_paged_decode_workspace_bytes": (_sz, [_vp, _i32, _i32]),
    "infer_paged_decode_noalloc": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i32, _i32, _f32, _vp]),
    "infer_paged_prefill": (_i32, [_vp, _vp, _vp, _i64, _vp, _vp, _vp, _i64, _i32, _i32, _i32, _i32, _f32, _vp]),
    "infer_flash_attn_prefill": (_i32, [_vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp]),
    "infer_paged_decode_status": (_i32, [_vp, _vp]),
    "infer_prefill_status": (_i32, [_vp]),
    "infer_block_manager_create": (_i32, [C.POINTER(_vp), _i64, _i32]),
    "infer_block_manager_destroy": (_i32, [_vp]),
    "infer_block_manager_can_allocate": (_i32, [_vp, _i64]),
    "infer_block_manager_allocate": (_i64, [_vp, _i64, _vp, _i64]),
    "infer_block_manager_can_append": (_i32, [_vp, _i64]),
    "infer_block_manager_append": (_i32, [_vp, _i64, _vp, _i64]),
    "infer_block_manager_deallocate": (_i32, [_vp, _i64]),
    "infer_block_manager_block_table": (_i64, [_vp, _i64, _vp, _i64]),
    "infer_block_manager_num_tokens": (_i64, [_vp, _i64]),
    "infer_block_manager_num_free": (_i64, [_vp]),
    "infer_block_manager_free_ids": (_i64, [_vp, _vp, _i64]),
    "infer_block_manager_ref_counts": (_i64, [_vp, _vp, _i64]),
    "infer_block_manager_set_free_order": (_i32, [_vp, _vp, _i64]),
    "infer_block_manager_last_error": (C.c_char_p, [_vp]),
    "infer_strerror": (C.c_char_p, [_i32]),
    "infer_last_cuda_error": (_i32, []),
    "infer_abi_version": (_i32, []),
}

# diagnostic entry points declared in include/infer_b200_selftest.h (used by the test suite only)
_u32 = C.c_uint32
SELFTEST_SIGNATURES = {
    "infer_selftest_paged_decode": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i32, _i32, _f32, _vp, _sz, _vp,
                                           _i32, _u32, _i32]),
    "infer_selftest_paged_prefill": (_i32, [_vp, _vp, _vp, _i64, _vp, _vp, _vp, _i64, _i32, _i32, _i32, _i32, _f32, _vp,
                                            _i32, _u32, _i32]),
    "infer_selftest_flash_attn_prefill": (_i32, [_vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp, _i32]),
}

_lib = None


def load() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m infer_b200.build` "
            "(nvcc, sm_100a).  infer_b200 has no CPU or PyTorch fallback.")
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in {**SIGNATURES, **SELFTEST_SIGNATURES}.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    _lib = lib
    return lib


def check(rc: int, what: str):
    if rc != OK:
        lib = load()
        msg = lib.infer_strerror(rc).decode()
        if rc == ERR_CUDA:
            msg += f" [cudaError {lib.infer_last_cuda_error()}]"
        raise RuntimeError(f"{what}: {msg}")
