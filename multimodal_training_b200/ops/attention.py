"""Packed variable-length attention on the GPU.

Two backends share one autograd interface:

* ``sm100``: the in-tree tcgen05 flash-attention kernels (``csrc/attention.cu``): non-causal
  head_dim 80 with window / full-image sequence boundaries for the vision encoder and causal
  GQA head_dim 128 for the text decoder (replaces flash-attn's ``flash_attn_varlen_func``
  reached from modeling_qwen2_5_vl.py:431-448,540-557,694-711,1266-1281 in the reference).
* ``lib``: flash-attn 2 from the image, used only by the library baseline (``baseline/``).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import native as nv

BACKEND = "sm100"


def set_backend(name: str) -> None:
    global BACKEND
    if name not in ("sm100", "lib"):
        raise ValueError(name)
    BACKEND = name


@dataclass
class SeqInfo:
    """Sequence boundaries of a packed batch, on the host and (lazily) on the device."""

    host: list[int]                    # cu_seqlens, len = nseq + 1
    device: torch.device
    _cu: torch.Tensor | None = None
    _lo: torch.Tensor | None = None
    _hi: torch.Tensor | None = None

    @classmethod
    def from_list(cls, cu: list[int], device) -> "SeqInfo":
        return cls(host=[int(x) for x in cu], device=torch.device(device))

    @property
    def total(self) -> int:
        return self.host[-1]

    @property
    def max_len(self) -> int:
        return max((b - a for a, b in zip(self.host[:-1], self.host[1:])), default=0)

    @property
    def cu(self) -> torch.Tensor:
        if self._cu is None:
            self._cu = torch.tensor(self.host, dtype=torch.int32).to(self.device, non_blocking=True)
        return self._cu

    def bounds(self) -> tuple[torch.Tensor, torch.Tensor]:
        """Per-token [lo, hi) row range of the token's own sequence (int32, device)."""
        if self._lo is None:
            cu = torch.tensor(self.host, dtype=torch.int64)
            lens = cu[1:] - cu[:-1]
            lo = torch.repeat_interleave(cu[:-1], lens).to(torch.int32)
            hi = torch.repeat_interleave(cu[1:], lens).to(torch.int32)
            self._lo = lo.to(self.device, non_blocking=True)
            self._hi = hi.to(self.device, non_blocking=True)
        return self._lo, self._hi


class _LibAttentionFn(torch.autograd.Function):
    """flash-attn 2 (library) on the fused buffer; used for the baseline arm only."""

    @staticmethod
    def forward(ctx, qkv, n_q, n_kv, dim, info, causal, scale):
        from flash_attn.flash_attn_interface import _flash_attn_varlen_forward

        T = qkv.shape[0]
        q = qkv[:, : n_q * dim].reshape(T, n_q, dim)
        k = qkv[:, n_q * dim: (n_q + n_kv) * dim].reshape(T, n_kv, dim)
        v = qkv[:, (n_q + n_kv) * dim:].reshape(T, n_kv, dim)
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        out, lse, _, rng = _flash_attn_varlen_forward(q, k, v, info.cu, info.cu, info.max_len, info.max_len, 0.0,
                                                      scale, causal)
        ctx.save_for_backward(q, k, v, out, lse, rng)
        ctx.meta = (n_q, n_kv, dim, info, causal, scale)
        return out.reshape(T, n_q * dim)

    @staticmethod
    def backward(ctx, dout):
        from flash_attn.flash_attn_interface import _flash_attn_varlen_backward

        q, k, v, out, lse, rng = ctx.saved_tensors
        n_q, n_kv, dim, info, causal, scale = ctx.meta
        T = q.shape[0]
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        _flash_attn_varlen_backward(dout.reshape(T, n_q, dim).contiguous(), q, k, v, out, lse, dq, dk, dv, info.cu,
                                    info.cu, info.max_len, info.max_len, 0.0, scale, causal, -1, -1, 0.0, None,
                                    False, rng)
        dqkv = torch.cat((dq.reshape(T, -1), dk.reshape(T, -1), dv.reshape(T, -1)), dim=1)
        return dqkv, None, None, None, None, None, None


class _Sm100AttentionFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, n_q, n_kv, dim, info, causal, scale):
        T = qkv.shape[0]
        lo, hi = info.bounds()
        out = torch.empty(T, n_q * dim, device=qkv.device, dtype=qkv.dtype)
        lse = torch.empty(n_q, T, device=qkv.device, dtype=torch.float32)
        nv.call("mmt_attn_fwd", qkv.data_ptr(), out.data_ptr(), lse.data_ptr(), lo.data_ptr(), hi.data_ptr(), T,
                n_q, n_kv, dim, qkv.stride(0), int(causal), scale, nv.stream())
        ctx.save_for_backward(qkv, out, lse)
        ctx.meta = (n_q, n_kv, dim, info, causal, scale)
        return out

    @staticmethod
    def backward(ctx, dout):
        qkv, out, lse = ctx.saved_tensors
        n_q, n_kv, dim, info, causal, scale = ctx.meta
        T = qkv.shape[0]
        lo, hi = info.bounds()
        dout = dout if dout.is_contiguous() else dout.contiguous()
        dqkv = torch.empty_like(qkv)
        delta = torch.empty(n_q, T, device=qkv.device, dtype=torch.float32)
        # GQA with few KV tiles: one dK/dV CTA per q head needs an fp32 partial-sum workspace
        tiles = (T + 127) // 128
        ws = None
        if n_q > n_kv and tiles * n_kv < 2 * _sm_count():
            ws = torch.empty(2 * n_q * T * dim, device=qkv.device, dtype=torch.float32)
        nv.call("mmt_attn_bwd", qkv.data_ptr(), out.data_ptr(), dout.data_ptr(), lse.data_ptr(), delta.data_ptr(),
                dqkv.data_ptr(), lo.data_ptr(), hi.data_ptr(), T, n_q, n_kv, dim, qkv.stride(0), int(causal), scale,
                nv.ptr(ws), nv.stream())
        return dqkv, None, None, None, None, None, None


def flash_attention(qkv: torch.Tensor, n_q: int, n_kv: int, dim: int, info: SeqInfo, causal: bool,
                    scale: float) -> torch.Tensor:
    assert qkv.dim() == 2 and qkv.stride(1) == 1
    if BACKEND == "lib":
        return _LibAttentionFn.apply(qkv, n_q, n_kv, dim, info, causal, scale)
    return _Sm100AttentionFn.apply(qkv, n_q, n_kv, dim, info, causal, scale)


nv.declare("mmt_attn_fwd", nv.c_int, [nv._P, nv._P, nv._P, nv._P, nv._P, nv.c_long, nv.c_int, nv.c_int, nv.c_int,
                                      nv.c_long, nv.c_int, nv.c_float, nv._P])
nv.declare("mmt_attn_bwd", nv.c_int, [nv._P, nv._P, nv._P, nv._P, nv._P, nv._P, nv._P, nv._P, nv.c_long, nv.c_int,
                                      nv.c_int, nv.c_int, nv.c_long, nv.c_int, nv.c_float, nv._P, nv._P])


def _sm_count() -> int:
    return torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
