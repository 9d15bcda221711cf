"""CPU contract tests: shape/config validation (as tests/test_coverage_contract.py:7-33 of the
reference), the implementation registry, and the C-ABI surface of the built library."""
import ctypes
import re
from pathlib import Path

import pytest

from moba_opt import api
from moba_opt.baseline_adapter import MAINLINE_HEAD_DIMS, MAX_TOPK, validate_config, validate_shapes

ROOT = Path(__file__).resolve().parents[1]


@pytest.mark.parametrize("hq,hkv", [(1, 1), (28, 4), (32, 8), (16, 2), (8, 1), (14, 2)])
def test_grouped_shapes(hq, hkv):
    assert validate_shapes((11, hq, 128), (11, hkv, 128), (11, hkv, 128), True) == hq // hkv


@pytest.mark.parametrize("dim", range(8, 257, 8))
def test_head_dimensions(dim):
    """The prefill kernels go to head_dim 128: anything above is a ValueError from the shape check itself, i.e. before
    any launch (the reference's envelope, up to 256, is what the decode cache accepts)."""
    shapes = ((3, 2, dim),) * 3
    assert validate_shapes(*shapes, head_dims=MAINLINE_HEAD_DIMS) == 1
    if dim <= 128:
        assert validate_shapes(*shapes) == 1
    else:
        with pytest.raises(ValueError, match="head_dim"):
            validate_shapes(*shapes)


@pytest.mark.parametrize("qs,ks,vs", [
    ((0, 2, 64), (0, 2, 64), (0, 2, 64)), ((3, 3, 64), (3, 2, 64), (3, 2, 64)),
    ((3, 2, 7), (3, 2, 7), (3, 2, 7)), ((3, 2, 264), (3, 2, 264), (3, 2, 264)),
    ((3, 2, 64), (4, 2, 64), (4, 2, 64)), ((3, 2, 64), (3, 1, 64), (3, 2, 64)),
])
def test_invalid_shapes(qs, ks, vs):
    with pytest.raises(ValueError):
        validate_shapes(qs, ks, vs, True)


def test_gqa_needs_opt_in():
    with pytest.raises(ValueError):
        validate_shapes((3, 4, 64), (3, 2, 64), (3, 2, 64))


@pytest.mark.parametrize("override", [
    {"chunk_size": 0}, {"chunk_size": True}, {"topk": 0}, {"topk": MAX_TOPK + 1},
    {"topk": 2.5}, {"causal": False}, {"dropout": 0.1},
])
def test_invalid_configs(override):
    with pytest.raises(ValueError):
        validate_config({"chunk_size": 32, "topk": 4, **override})


def test_valid_configs():
    validate_config({"chunk_size": 2048, "topk": 3})
    validate_config({"chunk_size": 4096, "topk": 12, "causal": True, "dropout": 0})


def test_registry():
    assert "opt_gqa_cuda" in api.available_impls()
    assert api.available_impls() == sorted(api.available_impls())
    with pytest.raises(KeyError):
        api.register("opt_gqa_cuda", lambda *a: None)
    with pytest.raises(KeyError):
        api.run_impl("no_such_impl", None, None, None, None, 1, {})


def test_library_exports_every_declared_symbol():
    """The shared library loads without a GPU and exports each function the headers under include/ declare."""
    headers = sorted((ROOT / "include").glob("*.h"))
    assert [h.name for h in headers] == ["moba_b200.h", "moba_b200_debug.h"]
    declared = set()
    for h in headers:
        declared |= set(re.findall(r"\b(moba_[a-z0-9_]+)\s*\(", h.read_text()))
    assert {"moba_prefill_route", "moba_prefill_fwd", "moba_prefill_bwd", "moba_prefill_route_static",
            "moba_profile_events", "moba_selftest_wait"} <= declared
    lib_path = ROOT / "moba-merge-cuda_b200" / "moba_opt" / "libmoba_b200.so"
    if not lib_path.exists():
        import __graft_entry__
        __graft_entry__.build()
    lib = ctypes.CDLL(str(lib_path))
    missing = [name for name in sorted(declared) if not hasattr(lib, name)]
    assert not missing, missing
    lib.moba_status_string.restype = ctypes.c_char_p
    assert lib.moba_status_string(0) == b"ok"


def test_descriptor_mirrors_have_the_library_sizes():
    """The ctypes mirrors of the two descriptor structs are as large as the structs the library was compiled with (the
    loaders refuse a library for which this does not hold); no GPU needed."""
    import ctypes
    from moba_opt import _ext
    from moba_opt.kv_cache import CacheDesc, decode_library
    lib = decode_library()
    assert lib.moba_abi_sizeof(0) == ctypes.sizeof(_ext.PrefillDesc) == 176
    assert lib.moba_abi_sizeof(1) == ctypes.sizeof(CacheDesc) == 80
    assert lib.moba_abi_sizeof(2) == 0


def test_both_16_bit_formats_pass_the_input_check():
    import torch
    from moba_opt import baseline_adapter as ba
    assert ba.SUPPORTED_DTYPES == (torch.bfloat16, torch.float16)      # as src/moba_opt/baseline_adapter.py:13
