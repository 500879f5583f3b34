"""ctypes binding of libftk_sm100.so (declared in include/ftk_api.h).

The library is the only compute path of this package: there is no PyTorch or
CPU fallback.  Importing the package without the built library raises.
"""

from __future__ import annotations

import ctypes as C
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(os.path.dirname(_HERE), "lib", "libftk_sm100.so")

FTK_F16, FTK_BF16 = 0, 1

i64, i32, f32, vp, sz = C.c_int64, C.c_int, C.c_float, C.c_void_p, C.c_size_t

# name -> (restype, argtypes); must list every symbol of include/ftk_api.h
_STRIDES3 = [i64, i64, i64]
SIGNATURES = {
    "ftk_version": (i32, []),
    "ftk_error_string": (C.c_char_p, [i32]),
    "ftk_block_score_workspace": (sz, [i64, i64]),
    "ftk_block_score": (i32, [vp, vp, i32, i64, i64, i64, i64, *_STRIDES3, *_STRIDES3, i64, i64,
                              i32, i32, i32, f32, vp, vp, sz, vp, vp]),
    "ftk_topk_select": (i32, [vp, vp, i64, i32, i32, i32, i32, i32, f32, vp, vp, vp, vp, vp]),
    "ftk_score_topk_workspace": (sz, [i64, i64, i64]),
    "ftk_score_topk": (i32, [vp, vp, i32, i64, i64, i64, i64, *_STRIDES3, *_STRIDES3, i64, i64,
                             i32, i32, i32, f32, i32, f32, vp, vp, vp, vp, sz, vp, vp]),
    "ftk_qblock_merge": (i32, [vp, vp, i64, i64, i32, i32, i32, i32, i32, i32, vp, vp, vp, vp,
                               vp]),
    "ftk_qblock_union": (i32, [vp, i64, i64, i32, i32, i32, i32, i32, i32, vp, vp, vp, vp]),
    "ftk_max_index_plus1": (i32, [vp, i64, vp, vp]),
    "ftk_build_reverse_workspace": (sz, [i64, i32, i32]),
    "ftk_build_reverse": (i32, [vp, vp, i64, i32, i32, i32, vp, vp, vp, vp, sz, vp, vp]),
    "ftk_build_reverse_noalloc_capacity": (sz, []),
    "ftk_build_reverse_noalloc": (i32, [vp, vp, i64, i32, i32, i32, vp, vp, vp, vp, vp]),
    "ftk_sort_by_count_workspace": (sz, [i64, i32]),
    "ftk_sort_by_count": (i32, [vp, i64, i32, vp, vp, vp, sz, vp]),
    "ftk_sparse_fwd_workspace": (sz, [i64, i64, i32, i32]),
    "ftk_sparse_fwd": (i32, [vp, vp, vp, i32, i64, i64, i64, i64, i64, *_STRIDES3, *_STRIDES3,
                             *_STRIDES3, vp, i32, i32, i32, i32, i32, i32, f32, vp, *_STRIDES3,
                             vp, vp, sz, vp, vp]),
    "ftk_sparse_bwd_dq": (i32, [vp, vp, vp, vp, vp, i32, i64, i64, i64, i64, i64, *_STRIDES3,
                                *_STRIDES3, *_STRIDES3, *_STRIDES3, *_STRIDES3, vp, i32, i32,
                                i32, i32, i32, i32, f32, vp, vp, vp, *_STRIDES3, vp, vp]),
    "ftk_sparse_bwd_dkv": (i32, [vp, vp, vp, vp, i32, i64, i64, i64, i64, i64, *_STRIDES3, *_STRIDES3,
                                 *_STRIDES3, *_STRIDES3, vp, vp, vp, i32, i32, i32, i32, i32,
                                 i32, f32, vp, vp, vp, *_STRIDES3, vp, *_STRIDES3, i32, vp, vp]),
}


def _load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with "
            "`python flash-topk-attention_b200/build.py` (needs nvcc, sm_100a). "
            "This package has no fallback path."
        )
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is absent
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


def error_text(code: int) -> str:
    return lib.ftk_error_string(int(code)).decode()


def check(code: int, what: str) -> None:
    """Map a non-zero C-ABI return code to the Python exception the reference
    raises for the same class of problem."""
    if code == 0:
        return
    msg = f"{what}: {error_text(code)} (code {code})"
    if code == -2:
        raise NotImplementedError(msg)
    if code == -1:
        raise ValueError(msg)
    raise RuntimeError(msg)


def dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float16:
        return FTK_F16
    if t.dtype == torch.bfloat16:
        return FTK_BF16
    raise ValueError(f"unsupported dtype {t.dtype}")


def stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


def check_status(status: torch.Tensor, what: str) -> None:
    """Read a launch's device status word (synchronises) and raise on failure."""
    code = int(status.item())
    if code != 0:
        raise RuntimeError(f"{what}: {error_text(code)} (device status {code})")
