"""Shared test helpers: golden-fixture loading and conversions between stored 16-bit patterns, numpy and torch."""
from pathlib import Path

import numpy as np

GOLDEN = Path(__file__).resolve().parent / "golden"

PREFILL_GOLDENS = ["p_gqa_small", "p_mha_tail", "p_mqa_multi", "p_k9", "p_one_chunk", "p_gqa_256", "p_fp16_gqa", "p_fp16_d128"]
DECODE_GOLDENS = ["d_small", "d_d128", "d_mha", "d_fp16"]
ROUTE_GOLDENS = ["r_upstream_gqa", "r_upstream_mqa"]


class HalfBits(np.ndarray):
    """uint16 bit patterns of IEEE half values (plain uint16 arrays in a fixture are bf16 patterns)."""


def load(name):
    """The fixture as a dict; the 16-bit inputs of a fixture whose `dtype` entry says float16 come back as HalfBits,
    so that bits_to_f64 / bits_to_torch decode them in the right format."""
    g = dict(np.load(GOLDEN / f"{name}.npz"))
    if str(g.get("dtype", "bfloat16")) == "float16":
        for key, value in g.items():
            if value.dtype == np.uint16:
                g[key] = value.view(HalfBits)
    return g


def unpack_selected(g, tag):
    """[F,Hq,T] bool selection stored bit-packed as selected_<tag>_packed + selected_shape."""
    shape = g["selected_shape"]
    return np.unpackbits(g[f"selected_{tag}_packed"])[:int(np.prod(shape))].reshape(shape).astype(bool)


def bits_to_f64(bits):
    """uint16 bit patterns (bf16, or half when tagged HalfBits) -> float64 values."""
    if isinstance(bits, HalfBits):
        return np.asarray(bits).view(np.float16).astype(np.float64)
    return (np.asarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32).astype(np.float64)


def bits_to_torch(bits, device="cpu"):
    import torch
    dtype = torch.float16 if isinstance(bits, HalfBits) else torch.bfloat16
    t = torch.from_numpy(np.asarray(bits, dtype=np.uint16).view(np.int16).copy()).view(dtype)
    return t.to(device)


def torch_to_f64(t):
    return t.detach().float().cpu().numpy().astype(np.float64)


def cu_from_lens(lens):
    return np.concatenate(([0], np.cumsum(np.asarray(lens, dtype=np.int64))))


def rel_rms(a, b):
    a, b = np.asarray(a, dtype=np.float64), np.asarray(b, dtype=np.float64)
    return float(np.sqrt(((a - b) ** 2).mean()) / max(np.sqrt((b ** 2).mean()), 1e-30))


def config1_inputs():
    """BASELINE config 1 inputs: seed 0, q, k, v then dO ~ N(0,1), [2048, 8, 64], rounded to bf16."""
    import torch
    rng = torch.Generator().manual_seed(0)
    q, k, v = [torch.randn(2048, 8, 64, generator=rng).bfloat16() for _ in range(3)]
    g = torch.randn(2048, 8, 64, generator=rng).bfloat16()
    return q, k, v, g
