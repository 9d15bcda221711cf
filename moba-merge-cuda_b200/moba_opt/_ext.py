"""ctypes binding of libmoba_b200.so.  There is no fallback: a missing library is an ImportError at
first use, and a non-zero status from any entry point is raised as RuntimeError."""
import ctypes
from pathlib import Path

_LIB_PATH = Path(__file__).resolve().parent / "libmoba_b200.so"
_lib = None

c_i32, c_i64, c_vp, c_sz = ctypes.c_int32, ctypes.c_int64, ctypes.c_void_p, ctypes.c_size_t


class PrefillDesc(ctypes.Structure):
    """Mirror of moba_prefill_desc in include/moba_b200.h."""
    _fields_ = ([(n, c_i32) for n in ("total_tokens", "num_seqs", "hq", "hkv", "dim", "chunk_size", "remote_k",
                                      "num_chunks", "num_qtiles", "max_tiles_per_seq", "max_chunks_per_seq")]
                + [("flags", c_i32), ("num_self_pairs", c_i32), ("reserved0", c_i32)]
                + [(n, c_i64) for n in ("q_stride_t", "q_stride_h", "k_stride_t", "k_stride_h", "v_stride_t", "v_stride_h")]
                + [(n, c_vp) for n in ("cu_seqlens", "chunk_start", "chunk_seq", "chunk_local", "qtile_chunk",
                                       "qtile_tok0", "qtile_local", "self_pairs", "kv_order")])


def lib():
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            raise ImportError(f"{_LIB_PATH} is missing: build it with `python moba-merge-cuda_b200/build.py` "
                              "(there is no non-CUDA path)")
        L = ctypes.CDLL(str(_LIB_PATH))
        P = ctypes.POINTER(PrefillDesc)
        L.moba_status_string.restype = ctypes.c_char_p
        L.moba_status_string.argtypes = [ctypes.c_int]
        L.moba_abi_sizeof.restype, L.moba_abi_sizeof.argtypes = c_sz, [ctypes.c_int]
        if L.moba_abi_sizeof(0) != ctypes.sizeof(PrefillDesc):
            raise ImportError(f"{_LIB_PATH} was built from another revision of include/moba_b200.h (moba_prefill_desc)")
        L.moba_selftest_umma.argtypes = [ctypes.c_int, c_vp, c_vp, c_vp, ctypes.c_int, ctypes.c_int, c_vp, c_vp]
        L.moba_selftest_wait.argtypes = [ctypes.c_longlong, c_vp, c_vp, c_vp]
        for name in ("moba_prefill_route_state_bytes", "moba_prefill_route_scratch_bytes",
                     "moba_prefill_fwd_scratch_bytes", "moba_prefill_bwd_scratch_bytes"):
            fn = getattr(L, name)
            fn.restype, fn.argtypes = c_sz, [P]
        L.moba_profile_events.argtypes = [ctypes.c_int, c_vp, c_vp]
        L.moba_prefill_route.argtypes = [P, c_vp, c_vp, c_vp, c_vp, c_sz, c_vp]
        L.moba_prefill_route_static.argtypes = [P, c_vp, c_vp, c_vp, c_vp]
        L.moba_prefill_route_static_capacity.restype = c_sz
        L.moba_prefill_route_static_capacity.argtypes = []
        L.moba_prefill_fwd.argtypes = [P, c_vp, c_vp, c_vp, c_vp, c_vp, c_sz, c_vp, c_vp, c_vp, c_vp]
        L.moba_prefill_bwd.argtypes = [P, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_sz, c_vp, c_vp, c_vp, c_vp, c_vp]
        L.moba_merge_scratch_bytes.restype = c_sz
        L.moba_merge_scratch_bytes.argtypes = [ctypes.c_longlong, ctypes.c_int]
        L.moba_merge_forward.argtypes = [c_vp, c_vp, c_vp, c_vp, c_vp, ctypes.c_longlong, ctypes.c_longlong, ctypes.c_int,
                                         ctypes.c_int, ctypes.c_int, c_vp, c_sz, c_vp, c_vp, c_vp, c_vp]
        L.moba_add_rmsnorm.argtypes = [c_vp, c_vp, c_vp, ctypes.c_float, ctypes.c_longlong, ctypes.c_int, c_vp, c_vp, c_vp]
        L.moba_rope_split.argtypes = [c_vp, c_vp, c_vp, ctypes.c_longlong, ctypes.c_int, ctypes.c_int, ctypes.c_int, c_vp, c_vp,
                                      c_vp, c_vp]
        L.moba_silu_mul.argtypes = [c_vp, ctypes.c_longlong, ctypes.c_int, c_vp, c_vp]
        L.moba_decode_step_inputs.argtypes = [c_vp, c_vp, ctypes.c_int, c_vp, c_vp, ctypes.c_float, ctypes.c_int,
                                              ctypes.c_longlong, c_vp, c_vp, c_vp, c_vp]
        L.moba_argmax_workspace_bytes.restype = c_sz
        L.moba_argmax_workspace_bytes.argtypes = []
        L.moba_argmax_bf16.argtypes = [c_vp, ctypes.c_int, c_vp, c_sz, c_vp, c_vp]
        L.moba_decode_linear.argtypes = [c_vp, c_vp, c_vp, c_vp, ctypes.c_float, c_vp, c_vp, c_vp, ctypes.c_int, ctypes.c_int,
                                         ctypes.c_int, c_vp, c_vp]
        _lib = L
    return _lib


class _NoRange:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


_NO_RANGE = _NoRange()


def nvtx(name):
    """An NVTX range around a stage of the host wrapper (routing, forward, backward, a cache call, a decode step) when
    MOBA_NVTX=1 is set in the environment - the counterpart of the reference's record_function stage marks
    (src/moba_opt/diagnostic.py:105-305) for timeline tools; a no-op object otherwise, so the default path pays nothing."""
    global _nvtx_on
    if _nvtx_on is None:
        import os
        _nvtx_on = os.environ.get("MOBA_NVTX", "0") not in ("", "0")
    if not _nvtx_on:
        return _NO_RANGE
    import torch
    return torch.cuda.nvtx.range(name)


_nvtx_on = None


def check(status, what):
    if status != 0:
        raise RuntimeError(f"{what} failed: {lib().moba_status_string(status).decode()} (status {status})")
