"""Loads ``libnuclis_cuda.so`` and declares the C ABI of include/nuclis_cuda.h.

The library is looked for beside this file (built in-tree by
``python -m nuclis_b200.build``). A missing library is an error, never a
fallback.
"""
from __future__ import annotations

import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libnuclis_cuda.so")

u8p = ctypes.POINTER(ctypes.c_uint8)
u32, u64, sz, vp, cint = ctypes.c_uint32, ctypes.c_uint64, ctypes.c_size_t, ctypes.c_void_p, ctypes.c_int


class CBuffer(ctypes.Structure):
    _fields_ = [("id", u32), ("reserved", u32), ("offset", u64), ("len", u64)]


class CMatrix(ctypes.Structure):
    _fields_ = [("encoding", u32), ("layout", u32), ("rows", u64), ("columns", u64), ("bytes", u64)]


class CExpertMatrix(ctypes.Structure):
    _fields_ = [("encoding", u32), ("reserved", u32), ("experts", u64), ("rows", u64), ("columns", u64), ("bytes", u64)]


class CSegment(ctypes.Structure):
    _fields_ = [("weights", CBuffer), ("matrix", CMatrix), ("output", CBuffer)]


class CCombineShape(ctypes.Structure):
    _fields_ = [("columns", u64), ("slots", u64), ("rows", u64), ("experts", u64), ("in_stride", u64), ("out_stride", u64)]


class CNorm(ctypes.Structure):
    _fields_ = [("rows", sz), ("width", sz), ("in_stride", sz), ("out_stride", sz), ("eps", ctypes.c_float)]


BP, MP, EP, SP = ctypes.POINTER(CBuffer), ctypes.POINTER(CMatrix), ctypes.POINTER(CExpertMatrix), ctypes.POINTER(CSegment)

# name -> (restype, argtypes); every function declared in include/nuclis_cuda.h
SIGNATURES = {
    "nu_cuda_create": (vp, [cint, ctypes.c_char_p, sz]),
    "nu_cuda_destroy": (None, [vp]),
    "nu_cuda_last_error": (ctypes.c_char_p, [vp]),
    "nu_cuda_status_name": (ctypes.c_char_p, [cint]),
    "nu_cuda_set_generic_only": (cint, [vp, cint]),
    "nu_cuda_set_chaining": (cint, [vp, cint]),
    "nu_cuda_buffer_create": (cint, [vp, sz, ctypes.POINTER(u32)]),
    "nu_cuda_buffer_upload": (cint, [vp, u32, sz, vp, sz]),
    "nu_cuda_buffer_download": (cint, [vp, u32, sz, vp, sz]),
    "nu_cuda_buffer_wrap": (cint, [vp, vp, sz, ctypes.POINTER(u32)]),
    "nu_cuda_buffer_unwrap": (cint, [vp, vp]),
    "nu_cuda_buffer_release": (cint, [vp, u32]),
    "nu_cuda_buffer_device_ptr": (vp, [vp, u32]),
    "nu_cuda_created_bytes": (u64, [vp]),
    "nu_cuda_matrix_prepare": (cint, [vp, BP, MP, BP, ctypes.POINTER(u32)]),
    "nu_cuda_begin": (cint, [vp]),
    "nu_cuda_commit": (cint, [vp]),
    "nu_cuda_discard": (cint, [vp]),
    "nu_cuda_commit_retain": (cint, [vp, ctypes.POINTER(u32)]),
    "nu_cuda_graph_launch": (cint, [vp, u32, u32, ctypes.POINTER(ctypes.c_float)]),
    "nu_cuda_graph_release": (cint, [vp, u32]),
    "nu_cuda_gpu_seconds": (ctypes.c_double, [vp]),
    "nu_cuda_launch_count": (u64, [vp]),
    "nu_cuda_stream": (vp, [vp]),
    "nu_cuda_profile_enable": (cint, [vp, u32]),
    "nu_cuda_profile_read": (u32, [vp, ctypes.POINTER(ctypes.c_double), u32]),
    "nu_cuda_embed": (cint, [vp, BP, MP, u32, BP, u32]),
    "nu_cuda_matvec": (cint, [vp, BP, MP, BP, BP]),
    "nu_cuda_matvec_rows": (cint, [vp, BP, MP, BP, sz, BP, sz, sz]),
    "nu_cuda_matmul": (cint, [vp, BP, MP, BP, u32, sz, BP, sz, sz]),
    "nu_cuda_matmul_padded": (sz, [sz]),
    "nu_cuda_matvec_add": (cint, [vp, BP, MP, BP, BP, BP]),
    "nu_cuda_matvec_segments": (cint, [vp, SP, sz, BP, u32]),
    "nu_cuda_matvec_segments_normed": (cint, [vp, SP, sz, BP, BP, BP, BP, ctypes.c_float, u32]),
    "nu_cuda_silu_mul": (cint, [vp, BP, BP, sz]),
    "nu_cuda_gelu_mul": (cint, [vp, BP, BP, sz]),
    "nu_cuda_rms_norm": (cint, [vp, BP, BP, BP, ctypes.POINTER(CNorm)]),
    "nu_cuda_add_rms_norm": (cint, [vp, BP, BP, BP, BP, ctypes.POINTER(CNorm)]),
    "nu_cuda_add": (cint, [vp, BP, BP, sz]),
    "nu_cuda_argmax": (cint, [vp, BP, sz, BP]),
    "nu_cuda_route": (cint, [vp, BP, sz, sz, sz, sz, BP, BP]),
    "nu_cuda_expert_lists_words": (sz, [sz, sz]),
    "nu_cuda_expert_lists": (cint, [vp, BP, sz, sz, sz, BP]),
    "nu_cuda_matmul_experts": (cint, [vp, BP, ctypes.POINTER(CExpertMatrix), BP, sz, sz, BP, sz, sz, BP, sz]),
    "nu_cuda_route_local": (cint, [vp, BP, BP, sz, sz, sz, BP, BP]),
    "nu_cuda_matvec_experts": (cint, [vp, BP, EP, BP, sz, BP, sz, sz, BP, sz]),
    "nu_cuda_matvec_experts_gated": (cint, [vp, BP, EP, BP, sz, BP, sz, sz, BP, sz, u32]),
    "nu_cuda_gelu_mul_rows": (cint, [vp, BP, BP, BP, sz, sz, sz, sz, sz]),
    "nu_cuda_combine_experts": (cint, [vp, BP, BP, BP, BP, BP, ctypes.POINTER(CCombineShape)]),
    "nu_cuda_matvec_q4k_static": (cint, [vp, sz, u32, u32, vp, vp, vp, ctypes.c_char_p, sz]),
    "nu_cuda_matvec_q4k_static_plan": (cint, [u32, u32, u32, ctypes.POINTER(u32), ctypes.POINTER(u32)]),
    "nu_cuda_matvec_q4k_static_status": (cint, [vp, ctypes.POINTER(u32)]),
    "nu_cuda_comm_unique_id": (cint, [u8p]),
    "nu_cuda_comm_init": (cint, [vp, u8p, cint, cint]),
    "nu_cuda_allreduce_sum_f32": (cint, [vp, BP, sz]),
    "nu_cuda_allreduce_sum_add_f32": (cint, [vp, BP, BP, sz]),
    "nu_cuda_comm_destroy": (cint, [vp]),
    "nu_cuda_comm_peer_handle": (cint, [vp, u8p]),
    "nu_cuda_comm_attach_peers": (cint, [vp, u8p, cint, cint]),
    "nu_cuda_comm_set_wait_ms": (cint, [vp, u32]),
}

_lib = None


def load() -> ctypes.CDLL:
    """The loaded library; raises if it has not been built."""
    global _lib
    if _lib is None:
        path = os.environ.get("NUCLIS_CUDA_LIB", LIB_PATH)  # another build of the same library, e.g. a tuning variant
        if not os.path.exists(path):
            raise RuntimeError(f"{path} is missing: run `python -m nuclis_b200.build` (there is no CPU fallback)")
        lib = ctypes.CDLL(path)
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = lib
    return _lib
