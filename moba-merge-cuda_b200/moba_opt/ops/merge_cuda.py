"""Standalone global-softmax merge, the counterpart of the reference's CUDA merge operator
(src/moba_opt/ops/merge_cuda.py:32-60).  The prefill path does not call it (there the merge is the
epilogue of the forward kernel); it serves callers that hold the self branch and the scattered remote
contributions themselves."""
import ctypes

import torch

from .. import _ext
from ..grouped_attention import _status_word, _stream

MAX_CONTRIBUTIONS = 32  # per row


def merge_forward_cuda(self_out, self_lse, remote_out, remote_lse, mapping, kmax=None, check_capacity=True,
                       deterministic=False):
    """self_out [T,H,D] (bf16, fp16 or fp32, CUDA); self_lse [T,H] fp32; remote_out [M,1,D] or [M,D];
    remote_lse [M] fp32; mapping [M] int32/int64 with the row t*H+h every contribution belongs to.
    Returns (O like self_out, LSE [T,H] fp32).  Contributions are always reduced in ascending index
    order, so `deterministic` only is type-checked.  With check_capacity a row with more than kmax
    contributions or an out-of-range mapping entry raises (one device-to-host read per call)."""
    if not isinstance(deterministic, bool):
        raise ValueError("deterministic must be bool")
    if mapping.dim() != 1 or mapping.dtype not in (torch.int32, torch.int64):
        raise ValueError("mapping must be a 1D int32/int64 tensor")
    if self_out.dim() != 3 or not self_out.is_cuda:
        raise ValueError("self_out must be a CUDA tensor [T,H,D]")
    if self_out.dtype not in (torch.bfloat16, torch.float32, torch.float16):
        raise ValueError("self_out must be bf16, fp16 or fp32")
    T, H, D = self_out.shape
    P, M = T * H, mapping.numel()
    if remote_out.dtype != self_out.dtype or remote_out.device != self_out.device:
        raise ValueError("remote_out must match self_out in dtype and device")
    if remote_out.numel() != M * D or remote_lse.numel() != M or self_lse.numel() != P:
        raise ValueError("shape mismatch between branches, LSEs and mapping")
    mapping = mapping.to(torch.int64).reshape(-1).contiguous()
    if kmax is None:
        kmax = 1
        if M:
            if int(mapping.min().item()) < 0 or int(mapping.max().item()) >= P:
                raise ValueError("mapping entry out of range")
            kmax = max(1, int(torch.bincount(mapping, minlength=P).max().item()))
    kmax = int(kmax)
    if kmax < 1 or kmax > MAX_CONTRIBUTIONS:
        raise ValueError(f"kmax must be in [1, {MAX_CONTRIBUTIONS}]")
    lib = _ext.lib()
    dev = self_out.device
    so, ro = self_out.contiguous(), remote_out.reshape(M, D).contiguous()
    sl = self_lse.to(torch.float32).reshape(P).contiguous()
    rl = remote_lse.to(torch.float32).reshape(M).contiguous()
    out = torch.empty_like(so)
    lse = torch.empty(T, H, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        nbytes = lib.moba_merge_scratch_bytes(P, kmax)
        scratch = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev) if check_capacity else _status_word(dev)
        _ext.check(lib.moba_merge_forward(so.data_ptr(), sl.data_ptr(), ro.data_ptr() if M else None,
                                          rl.data_ptr() if M else None, mapping.data_ptr() if M else None, P, M, D, kmax,
                                          {torch.bfloat16: 0, torch.float32: 1, torch.float16: 2}[so.dtype], scratch.data_ptr(), nbytes, out.data_ptr(),
                                          lse.data_ptr(), status.data_ptr(), _stream(dev)), "moba_merge_forward")
        if check_capacity:
            bits = int(status.item())
            if bits & 2:
                raise ValueError("mapping entry out of range")
            if bits & 4:
                raise RuntimeError(f"a row has more than kmax={kmax} remote contributions")
    return out, lse
