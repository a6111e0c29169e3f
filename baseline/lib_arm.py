"""Same-box library baseline: the reference's training step restated with library calls only.

Nothing in this file launches a kernel of this repository.  Every GEMM is ``torch.nn.functional.linear``
(cuBLAS), attention is flash-attn 2 (``flash_attn_varlen_func``; PyTorch SDPA when flash-attn is missing or the
tensors are on the CPU), norms / RoPE / SwiGLU / cross-entropy are ATen ops, the optimizer is
``torch.optim.AdamW(fused=True)`` with bf16 states (the reference keeps pure-bf16 optimizer state,
python/ray/trainer.py:775-779), and every collective is an NCCL call placed where the reference places it:

* vision encoder, DeepSpeed-Ulysses sequence parallelism (python/models/qwen2_5_vl/modeling_qwen2_5_vl.py):
  patch embedding on all patches, window-aligned split, 28 local window layers, 4 full-attention layers that pad to
  ``[B, pad_len, heads, d]`` and send q, k, v, cos, sin and the mask through six all-to-alls (:628-640) plus one for
  the attention output (:744-746), a ragged all-gather of the hidden states whose backward is a reduce-scatter
  (:110-189, :1018-1066) and a merger that every rank runs on the whole sequence;
* ZeRO-1 over all vision ranks: gradient reduce-scatter, AdamW on the owned shard, parameter all-gather;
* text decoder with the reference's tensor-parallel plan (python/ray/text.py:1165-1177): replicated activations,
  column-parallel q/k/v/gate/up, row-parallel o/down followed by an all-reduce, vocab-parallel embedding
  (python/tensor_parallel/embedding.py:112-141) and cross-entropy with its three all-reduces
  (python/tensor_parallel/cross_entropy.py:48-236); data-parallel replicas above the tensor-parallel groups
  average their gradients with one all-reduce over a flat buffer;
* the vision -> text handoff is a clone plus ``masked_scatter`` (python/ray/text.py:868-920) and the gradient comes
  back as a clone (:1010-1019);
* every transformer block is activation-checkpointed, as in the reference's published runs.

Where the reference's library stack would issue MORE collectives than this file (DTensor reduces the input
gradient of q, k, v, gate and up separately; this file sums them first and reduces once per half-layer), the
baseline is the faster of the two, never the slower.

Host-side planning (window order, rotary tables, the split of every image over the ranks, sequence packing) is
taken from this repository's pure-Python helpers, computed once per batch shape.
"""
from __future__ import annotations

import math
import os
import sys

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint as torch_checkpoint

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

try:  # library attention; absent or CPU tensors -> SDPA
    from flash_attn import flash_attn_varlen_func as _fa_varlen
except Exception:  # pragma: no cover - depends on the image
    _fa_varlen = None


# --------------------------------------------------------------------------------------------------
# small library-op helpers
# --------------------------------------------------------------------------------------------------
def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return F.rms_norm(x, (x.shape[-1],), w, eps)


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    h = x.shape[-1] // 2
    return torch.cat((-x[..., h:], x[..., :h]), dim=-1)


def varlen_attention(q, k, v, cu: torch.Tensor, cu_host: list[int], causal: bool) -> torch.Tensor:
    """q [T, hq, d], k/v [T, hkv, d] packed sequences -> [T, hq, d]."""
    d = q.shape[-1]
    max_len = max((b - a for a, b in zip(cu_host[:-1], cu_host[1:])), default=0)
    if _fa_varlen is not None and q.is_cuda:
        return _fa_varlen(q, k, v, cu, cu, max_len, max_len, dropout_p=0.0, softmax_scale=1.0 / math.sqrt(d),
                          causal=causal)
    rep = q.shape[1] // k.shape[1]
    outs = []
    for s, e in zip(cu_host[:-1], cu_host[1:]):
        if e == s:
            continue
        qi = q[s:e].transpose(0, 1)
        ki = k[s:e].transpose(0, 1).repeat_interleave(rep, dim=0)
        vi = v[s:e].transpose(0, 1).repeat_interleave(rep, dim=0)
        outs.append(F.scaled_dot_product_attention(qi, ki, vi, is_causal=causal).transpose(0, 1))
    return torch.cat(outs, dim=0) if outs else q.new_zeros(q.shape)


def _a2a_equal(recv: torch.Tensor, send: torch.Tensor, group) -> None:
    """``all_to_all_single`` with equal splits along dim 0 (gloo has none: point-to-point there, CPU tests only)."""
    if send.is_cuda:
        dist.all_to_all_single(recv, send, group=group)
        return
    n, r = dist.get_world_size(group), dist.get_rank(group)
    ranks = dist.get_process_group_ranks(group)
    per = send.shape[0] // n
    recv[r * per:(r + 1) * per].copy_(send[r * per:(r + 1) * per])
    ops = []
    for p in range(n):
        if p != r:
            ops.append(dist.P2POp(dist.isend, send[p * per:(p + 1) * per].contiguous(), ranks[p], group=group))
            ops.append(dist.P2POp(dist.irecv, recv[p * per:(p + 1) * per], ranks[p], group=group))
    for w in dist.batch_isend_irecv(ops):
        w.wait()


def _reduce_scatter(out: torch.Tensor, inp: torch.Tensor, group, mean: bool = False) -> None:
    """``reduce_scatter_tensor`` (sum or mean); gloo has none: all-reduce and slice there (CPU tests only)."""
    n = dist.get_world_size(group)
    if inp.is_cuda:
        dist.reduce_scatter_tensor(out, inp, op=dist.ReduceOp.AVG if mean else dist.ReduceOp.SUM, group=group)
        return
    tmp = inp.clone()
    dist.all_reduce(tmp, group=group)
    r = dist.get_rank(group)
    out.copy_(tmp[r * out.shape[0]:(r + 1) * out.shape[0]])
    if mean:
        out.div_(n)


def _all_reduce_mean(t: torch.Tensor, group) -> None:
    if t.is_cuda:
        dist.all_reduce(t, op=dist.ReduceOp.AVG, group=group)
    else:
        dist.all_reduce(t, group=group)
        t.div_(dist.get_world_size(group))


class _AllToAllSeqHeads(torch.autograd.Function):
    """DeepSpeed's ``_SeqAllToAll`` over ``all_to_all_single``: [B, L, sp*h, d] <-> [B, sp*L, h, d]."""

    @staticmethod
    def forward(ctx, x, group, to_heads: bool):
        ctx.group, ctx.to_heads = group, to_heads
        sp = dist.get_world_size(group)
        B, L, H, D = x.shape
        if to_heads:      # scatter heads, gather sequence
            send = x.reshape(B, L, sp, H // sp, D).permute(2, 0, 1, 3, 4).contiguous()
            recv = torch.empty_like(send)
            _a2a_equal(recv, send, group)
            return recv.permute(1, 0, 2, 3, 4).reshape(B, sp * L, H // sp, D)
        send = x.reshape(B, sp, L // sp, H, D).permute(1, 0, 2, 3, 4).contiguous()      # scatter sequence, gather heads
        recv = torch.empty_like(send)
        _a2a_equal(recv, send, group)
        return recv.permute(1, 2, 0, 3, 4).reshape(B, L // sp, sp * H, D)

    @staticmethod
    def backward(ctx, g):
        return _AllToAllSeqHeads.apply(g.contiguous(), ctx.group, not ctx.to_heads), None, None


class _AllGatherRagged(torch.autograd.Function):
    """Ragged all-gather along dim 0 (pad to the longest rank); backward is a reduce-scatter SUM."""

    @staticmethod
    def forward(ctx, x, lengths, group):
        ctx.lengths, ctx.group = lengths, group
        rank = dist.get_rank(group)
        mx = max(lengths)
        pad = x.new_zeros((mx,) + tuple(x.shape[1:]))
        pad[: lengths[rank]] = x
        out = x.new_empty((len(lengths) * mx,) + tuple(x.shape[1:]))
        dist.all_gather_into_tensor(out, pad, group=group)
        return torch.cat([out[r * mx: r * mx + n] for r, n in enumerate(lengths)], dim=0)

    @staticmethod
    def backward(ctx, g):
        lengths, group = ctx.lengths, ctx.group
        rank = dist.get_rank(group)
        mx = max(lengths)
        pad = g.new_zeros((len(lengths) * mx,) + tuple(g.shape[1:]))
        off = 0
        for r, n in enumerate(lengths):
            pad[r * mx: r * mx + n] = g[off: off + n]
            off += n
        out = g.new_empty((mx,) + tuple(g.shape[1:]))
        _reduce_scatter(out, pad, group)
        return out[: lengths[rank]], None, None


class _CopyToTP(torch.autograd.Function):
    """Identity forward, all-reduce of the gradient (input of a column-parallel layer on replicated activations)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        dist.all_reduce(g, group=ctx.group)
        return g, None


class _ReduceFromTP(torch.autograd.Function):
    """All-reduce forward (output of a row-parallel layer), identity backward."""

    @staticmethod
    def forward(ctx, x, group):
        x = x.contiguous()
        dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


class _VocabParallelCE(torch.autograd.Function):
    """Megatron-style cross-entropy over vocabulary shards: fp32 logits, three all-reduces, softmax kept for
    backward (python/tensor_parallel/cross_entropy.py:48-236)."""

    @staticmethod
    def forward(ctx, logits, labels, vocab_lo, group):
        lf = logits.float()
        mx = lf.max(dim=-1).values
        dist.all_reduce(mx, op=dist.ReduceOp.MAX, group=group)
        lf = lf - mx.unsqueeze(-1)
        V = lf.shape[1]
        local = labels - vocab_lo
        ok = (local >= 0) & (local < V)
        idx = local.clamp(0, V - 1)
        pred = lf.gather(1, idx.unsqueeze(1)).squeeze(1) * ok
        dist.all_reduce(pred, group=group)
        ex = lf.exp_()
        se = ex.sum(dim=-1)
        dist.all_reduce(se, group=group)
        valid = labels >= 0
        n = valid.sum().clamp(min=1)
        loss = ((se.log() - pred) * valid).sum() / n
        ex.div_(se.unsqueeze(-1))
        ctx.save_for_backward(ex, idx, ok, valid, n)
        ctx.dtype = logits.dtype
        return loss

    @staticmethod
    def backward(ctx, g):
        sm, idx, ok, valid, n = ctx.saved_tensors
        grad = sm
        grad.scatter_add_(1, idx.unsqueeze(1), -(ok.to(grad.dtype)).unsqueeze(1))
        grad.mul_((valid.to(grad.dtype) * (g / n)).unsqueeze(1))
        return grad.to(ctx.dtype), None, None, None


def _normal(shape, std, device, dtype, gen):
    return (torch.randn(shape, generator=gen, device=device, dtype=torch.float32) * std).to(dtype)


# --------------------------------------------------------------------------------------------------
# vision encoder (keys follow the reference's module tree: blocks.N.attn.{q,k,v}_proj, mlp.*_proj, merger.*)
# --------------------------------------------------------------------------------------------------
class LibVisionBlock(nn.Module):
    def __init__(self, C, I, device, dtype, gen, std):
        super().__init__()
        self.norm1 = nn.Parameter(torch.ones(C, device=device, dtype=dtype))
        self.norm2 = nn.Parameter(torch.ones(C, device=device, dtype=dtype))
        for n, (o, i) in {"q_proj": (C, C), "k_proj": (C, C), "v_proj": (C, C), "proj": (C, C), "gate_proj": (I, C),
                          "up_proj": (I, C), "down_proj": (C, I)}.items():
            setattr(self, n + "_w", nn.Parameter(_normal((o, i), std, device, dtype, gen)))
            setattr(self, n + "_b", nn.Parameter(torch.zeros(o, device=device, dtype=dtype)))


class LibVision(nn.Module):
    def __init__(self, cfg, sp_group=None, device="cpu", dtype=torch.float32, seed: int = 0):
        super().__init__()
        self.cfg = cfg
        self.group = sp_group
        self.sp = dist.get_world_size(sp_group) if sp_group is not None else 1
        self.rank = dist.get_rank(sp_group) if sp_group is not None else 0
        gen = torch.Generator(device=device).manual_seed(seed + 17)
        C, std = cfg.hidden_size, cfg.initializer_range
        self.patch_embed = nn.Parameter(_normal((C, cfg.patch_dim), std, device, dtype, gen))
        self.blocks = nn.ModuleList([LibVisionBlock(C, cfg.intermediate_size, device, dtype, gen, std)
                                     for _ in range(cfg.depth)])
        M = C * cfg.merge_unit
        self.ln_q = nn.Parameter(torch.ones(C, device=device, dtype=dtype))
        self.fc1_w = nn.Parameter(_normal((M, M), std, device, dtype, gen))
        self.fc1_b = nn.Parameter(torch.zeros(M, device=device, dtype=dtype))
        self.fc2_w = nn.Parameter(_normal((cfg.out_hidden_size, M), std, device, dtype, gen))
        self.fc2_b = nn.Parameter(torch.zeros(cfg.out_hidden_size, device=device, dtype=dtype))
        self.checkpointing = True

    # -------------------------------------------------------------- per-batch host plan -> device tensors
    def prepare(self, grids, device):
        """Everything that depends only on the image grids (cached by the caller per batch shape)."""
        from multimodal_training_b200.parallel.sp import build_vision_plan, compute_geometry
        v = self.cfg
        geom = compute_geometry(grids, sp=self.sp, spatial_merge_size=v.spatial_merge_size, window_size=v.window_size,
                                patch_size=v.patch_size)
        plan = build_vision_plan(None, sp=self.sp, rank=self.rank, head_dim=v.head_dim, geom=geom)
        st = {"plan": plan}
        st["local_index"] = plan.local_patch_index.to(device)
        st["cos"] = plan.local_cos.to(device)
        st["sin"] = plan.local_sin.to(device)
        st["win_cu_host"] = plan.win_cu
        st["win_cu"] = torch.tensor(plan.win_cu, dtype=torch.int32, device=device)
        st["full_cu_host"] = plan.full_cu
        st["full_cu"] = torch.tensor(plan.full_cu, dtype=torch.int32, device=device)
        local_cu = [0]
        for _, n in plan.per_image_local:
            local_cu.append(local_cu[-1] + n)
        st["local_cu_host"] = local_cu
        st["local_cu"] = torch.tensor(local_cu, dtype=torch.int32, device=device)
        # inverse window permutation of the merged tokens (window order -> original order)
        widx = torch.from_numpy(geom.widx)
        st["unpermute"] = torch.argsort(widx).to(device)
        if self.sp > 1:
            B = len(grids)
            # slices[r][b]: every rank's share of every image; pad_len is the reference's global maximum
            lens = [[hi - lo for lo, hi in geom.slices[r]] for r in range(self.sp)]
            pad_len = max(max(row) for row in lens)
            st["pad_len"] = pad_len
            st["my_lens"] = lens[self.rank]
            # rows of the local pack inside the padded [B, pad_len] buffer
            rows = []
            for b, n in enumerate(lens[self.rank]):
                rows.append(torch.arange(n) + b * pad_len)
            st["pad_rows"] = torch.cat(rows).to(device)
            # after the exchange image b holds sp segments of pad_len rows; the valid rows, image by image
            rows = []
            for b in range(B):
                for r in range(self.sp):
                    rows.append(torch.arange(lens[r][b]) + (b * self.sp + r) * pad_len)
            st["gathered_rows"] = torch.cat(rows).to(device)
            st["to_image_major"] = plan.to_image_major.to(device)
            st["rank_tokens"] = plan.rank_tokens
        return st

    # -------------------------------------------------------------- blocks
    def _rope(self, x, cos, sin):
        xf = x.float()
        return (xf * cos.unsqueeze(1) + rotate_half(xf) * sin.unsqueeze(1)).to(x.dtype)

    def _mlp(self, B, x):
        h = rms_norm(x, B.norm2, self.cfg.rms_norm_eps)
        g = F.linear(h, B.gate_proj_w, B.gate_proj_b)
        u = F.linear(h, B.up_proj_w, B.up_proj_b)
        return x + F.linear(F.silu(g) * u, B.down_proj_w, B.down_proj_b)

    def _window_block(self, B, x, st, cu, cu_host):
        nh, d = self.cfg.num_heads, self.cfg.head_dim
        h = rms_norm(x, B.norm1, self.cfg.rms_norm_eps)
        T = h.shape[0]
        q = F.linear(h, B.q_proj_w, B.q_proj_b).view(T, nh, d)
        k = F.linear(h, B.k_proj_w, B.k_proj_b).view(T, nh, d)
        v = F.linear(h, B.v_proj_w, B.v_proj_b).view(T, nh, d)
        q, k = self._rope(q, st["cos"], st["sin"]), self._rope(k, st["cos"], st["sin"])
        a = varlen_attention(q, k, v, cu, cu_host, causal=False).reshape(T, nh * d)
        x = x + F.linear(a, B.proj_w, B.proj_b)
        return self._mlp(B, x)

    def _full_block_sp(self, B, x, st):
        """The reference's ``_forward_sequence_parallel_full``: pad, project, six all-to-alls in, attention over
        whole images with heads/sp heads, one all-to-all out, unpad, project."""
        nh, d, sp = self.cfg.num_heads, self.cfg.head_dim, self.sp
        nimg, pad_len = len(st["my_lens"]), st["pad_len"]
        h = rms_norm(x, B.norm1, self.cfg.rms_norm_eps)
        hp = h.new_zeros(nimg * pad_len, h.shape[1])
        hp.index_copy_(0, st["pad_rows"], h)
        q = F.linear(hp, B.q_proj_w, B.q_proj_b).view(nimg, pad_len, nh, d)
        k = F.linear(hp, B.k_proj_w, B.k_proj_b).view(nimg, pad_len, nh, d)
        v = F.linear(hp, B.v_proj_w, B.v_proj_b).view(nimg, pad_len, nh, d)
        cosp = st["cos"].new_zeros(nimg * pad_len, d)
        sinp = st["sin"].new_zeros(nimg * pad_len, d)
        cosp.index_copy_(0, st["pad_rows"], st["cos"])
        sinp.index_copy_(0, st["pad_rows"], st["sin"])
        mask = h.new_zeros(nimg * pad_len, 1)
        mask.index_fill_(0, st["pad_rows"], 1.0)
        a2a = lambda t: _AllToAllSeqHeads.apply(t, self.group, True)  # noqa: E731
        q, k, v = a2a(q), a2a(k), a2a(v)
        with torch.no_grad():
            cosg = a2a(cosp.view(nimg, pad_len, 1, d).expand(-1, -1, nh, -1).contiguous())
            sing = a2a(sinp.view(nimg, pad_len, 1, d).expand(-1, -1, nh, -1).contiguous())
            a2a(mask.view(nimg, pad_len, 1, 1).expand(-1, -1, nh, -1).contiguous())
        hl = nh // sp
        rows = st["gathered_rows"]
        qg = q.reshape(-1, hl, d).index_select(0, rows)
        kg = k.reshape(-1, hl, d).index_select(0, rows)
        vg = v.reshape(-1, hl, d).index_select(0, rows)
        cg = cosg.reshape(-1, hl, d).index_select(0, rows)
        sg = sing.reshape(-1, hl, d).index_select(0, rows)
        qg = (qg.float() * cg + rotate_half(qg.float()) * sg).to(x.dtype)
        kg = (kg.float() * cg + rotate_half(kg.float()) * sg).to(x.dtype)
        a = varlen_attention(qg, kg, vg, st["full_cu"], st["full_cu_host"], causal=False)
        ap = a.new_zeros(nimg * sp * pad_len, hl, d)
        ap.index_copy_(0, rows, a)
        back = _AllToAllSeqHeads.apply(ap.view(nimg, sp * pad_len, hl, d), self.group, False)
        a_loc = back.reshape(nimg * pad_len, nh * d).index_select(0, st["pad_rows"])
        x = x + F.linear(a_loc, B.proj_w, B.proj_b)
        return self._mlp(B, x)

    def forward(self, pixels_all: torch.Tensor, st: dict) -> torch.Tensor:
        """[n_patches, patch_dim] of ALL images (merge-block order) -> merged tokens of all images in the original
        order, replicated on every rank: [n_patches / 4, out_hidden]."""
        cfg = self.cfg
        x = F.linear(pixels_all, self.patch_embed).index_select(0, st["local_index"])
        for i, B in enumerate(self.blocks):
            full = i in cfg.fullatt_block_indexes
            if full and self.sp > 1:
                fn = lambda t, B=B: self._full_block_sp(B, t, st)  # noqa: E731
            elif full:
                fn = lambda t, B=B: self._window_block(B, t, st, st["local_cu"], st["local_cu_host"])  # noqa: E731
            else:
                fn = lambda t, B=B: self._window_block(B, t, st, st["win_cu"], st["win_cu_host"])  # noqa: E731
            x = torch_checkpoint(fn, x, use_reentrant=False) if (self.checkpointing and x.requires_grad) else fn(x)
        if self.sp > 1:
            x = _AllGatherRagged.apply(x, st["rank_tokens"], self.group)
            x = x.index_select(0, st["to_image_major"])
        h = rms_norm(x, self.ln_q, cfg.rms_norm_eps).view(-1, cfg.hidden_size * cfg.merge_unit)
        h = F.linear(F.gelu(F.linear(h, self.fc1_w, self.fc1_b)), self.fc2_w, self.fc2_b)
        return h.index_select(0, st["unpermute"])

    # -------------------------------------------------------------- state dict (reference key names)
    def reference_state_dict(self) -> dict:
        cfg = self.cfg
        out = {"patch_embed.proj.weight": self.patch_embed.detach().view(
            cfg.hidden_size, cfg.in_channels, cfg.temporal_patch_size, cfg.patch_size, cfg.patch_size)}
        for i, B in enumerate(self.blocks):
            p = f"blocks.{i}."
            out[p + "norm1.weight"], out[p + "norm2.weight"] = B.norm1.detach(), B.norm2.detach()
            for n in ("q_proj", "k_proj", "v_proj", "proj"):
                out[p + f"attn.{n}.weight"] = getattr(B, n + "_w").detach()
                out[p + f"attn.{n}.bias"] = getattr(B, n + "_b").detach()
            for n in ("gate_proj", "up_proj", "down_proj"):
                out[p + f"mlp.{n}.weight"] = getattr(B, n + "_w").detach()
                out[p + f"mlp.{n}.bias"] = getattr(B, n + "_b").detach()
        out["merger.ln_q.weight"] = self.ln_q.detach()
        out["merger.mlp.0.weight"], out["merger.mlp.0.bias"] = self.fc1_w.detach(), self.fc1_b.detach()
        out["merger.mlp.2.weight"], out["merger.mlp.2.bias"] = self.fc2_w.detach(), self.fc2_b.detach()
        return out

    @torch.no_grad()
    def load_reference_state_dict(self, sd: dict) -> None:
        mine = self.reference_state_dict()
        for k, t in mine.items():
            t.copy_(sd[k].reshape(t.shape))


# --------------------------------------------------------------------------------------------------
# text decoder (reference TP plan: replicated activations, all-reduce after o_proj and down_proj)
# --------------------------------------------------------------------------------------------------
class LibTextLayer(nn.Module):
    def __init__(self, cfg, tp, device, dtype, gen):
        super().__init__()
        H, d, std = cfg.hidden_size, cfg.head_dim, cfg.initializer_range
        nq, nkv, I = cfg.num_attention_heads // tp, cfg.num_key_value_heads // tp, cfg.intermediate_size // tp
        P = lambda o, i: nn.Parameter(_normal((o, i), std, device, dtype, gen))  # noqa: E731
        Z = lambda o: nn.Parameter(torch.zeros(o, device=device, dtype=dtype))  # noqa: E731
        self.q_w, self.q_b = P(nq * d, H), Z(nq * d)
        self.k_w, self.k_b = P(nkv * d, H), Z(nkv * d)
        self.v_w, self.v_b = P(nkv * d, H), Z(nkv * d)
        self.o_w = P(H, nq * d)
        self.gate_w, self.up_w, self.down_w = P(I, H), P(I, H), P(H, I)
        self.ln1 = nn.Parameter(torch.ones(H, device=device, dtype=dtype))
        self.ln2 = nn.Parameter(torch.ones(H, device=device, dtype=dtype))


class LibText(nn.Module):
    def __init__(self, cfg, tp_group=None, device="cpu", dtype=torch.float32, seed: int = 0):
        super().__init__()
        self.cfg = cfg
        self.group = tp_group
        self.tp = dist.get_world_size(tp_group) if tp_group is not None else 1
        self.rank = dist.get_rank(tp_group) if tp_group is not None else 0
        gen = torch.Generator(device=device).manual_seed(seed + 1000 * self.rank + 31)
        V = cfg.vocab_size // self.tp
        self.vocab_lo = self.rank * V
        self.embed = nn.Parameter(_normal((V, cfg.hidden_size), cfg.initializer_range, device, dtype, gen))
        self.layers = nn.ModuleList([LibTextLayer(cfg, self.tp, device, dtype, gen)
                                     for _ in range(cfg.num_hidden_layers)])
        self.norm = nn.Parameter(torch.ones(cfg.hidden_size, device=device, dtype=dtype))
        self.lm_head = None if cfg.tie_word_embeddings else nn.Parameter(
            _normal((V, cfg.hidden_size), cfg.initializer_range, device, dtype, gen))
        self.checkpointing = True

    def embed_tokens(self, ids: torch.Tensor) -> torch.Tensor:
        if self.tp == 1:
            return F.embedding(ids, self.embed)
        V = self.embed.shape[0]
        local = ids - self.vocab_lo
        ok = (local >= 0) & (local < V)
        out = F.embedding(local.clamp(0, V - 1), self.embed) * ok.unsqueeze(-1).to(self.embed.dtype)
        return _ReduceFromTP.apply(out, self.group)

    def rope_tables(self, position_ids: torch.Tensor):
        """cos/sin [T, head_dim] from [3, T] position ids (sections doubled, axis i mod 3 per chunk)."""
        cfg = self.cfg
        d = cfg.head_dim
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, d, 2, dtype=torch.float32, device=position_ids.device) / d))
        fr = position_ids.float()[:, :, None] * inv[None, None, :]
        emb = torch.cat((fr, fr), dim=-1)
        chunks = emb.split(list(cfg.mrope_section) * 2, dim=-1)
        sel = torch.cat([c[i % 3] for i, c in enumerate(chunks)], dim=-1)
        return sel.cos(), sel.sin()

    def _layer(self, L, x, cos, sin, cu, cu_host):
        cfg, d = self.cfg, self.cfg.head_dim
        T = x.shape[0]
        tp = self.tp > 1
        h = rms_norm(x, L.ln1, cfg.rms_norm_eps)
        if tp:
            h = _CopyToTP.apply(h, self.group)
        q = F.linear(h, L.q_w, L.q_b).view(T, -1, d)
        k = F.linear(h, L.k_w, L.k_b).view(T, -1, d)
        v = F.linear(h, L.v_w, L.v_b).view(T, -1, d)
        c, s = cos.unsqueeze(1), sin.unsqueeze(1)
        q = q * c + rotate_half(q) * s
        k = k * c + rotate_half(k) * s
        a = varlen_attention(q, k, v, cu, cu_host, causal=True).reshape(T, -1)
        o = F.linear(a, L.o_w)
        x = x + (_ReduceFromTP.apply(o, self.group) if tp else o)
        h = rms_norm(x, L.ln2, cfg.rms_norm_eps)
        if tp:
            h = _CopyToTP.apply(h, self.group)
        m = F.linear(F.silu(F.linear(h, L.gate_w)) * F.linear(h, L.up_w), L.down_w)
        return x + (_ReduceFromTP.apply(m, self.group) if tp else m)

    def forward(self, x, cos, sin, cu, cu_host):
        cos, sin = cos.to(x.dtype), sin.to(x.dtype)
        for L in self.layers:
            fn = lambda t, L=L: self._layer(L, t, cos, sin, cu, cu_host)  # noqa: E731
            x = torch_checkpoint(fn, x, use_reentrant=False) if (self.checkpointing and x.requires_grad) else fn(x)
        return x

    def loss(self, x, shifted_labels):
        h = rms_norm(x, self.norm, self.cfg.rms_norm_eps)
        w = self.embed if self.lm_head is None else self.lm_head
        if self.tp == 1:
            return F.cross_entropy(F.linear(h, w).float(), shifted_labels, ignore_index=-100)
        h = _CopyToTP.apply(h, self.group)
        return _VocabParallelCE.apply(F.linear(h, w), shifted_labels, self.vocab_lo, self.group)

    # -------------------------------------------------------------- state dict (reference key names, FULL tensors in)
    @torch.no_grad()
    def load_reference_state_dict(self, sd: dict) -> None:
        """Take this rank's slices of full (unsharded) tensors under the reference's key names."""
        tp, r = self.tp, self.rank
        rows = lambda t: t.chunk(tp, dim=0)[r]  # noqa: E731
        cols = lambda t: t.chunk(tp, dim=1)[r]  # noqa: E731
        self.embed.copy_(rows(sd["embed_tokens.weight"]))
        for i, L in enumerate(self.layers):
            p = f"layers.{i}."
            for n, w, b in (("q", L.q_w, L.q_b), ("k", L.k_w, L.k_b), ("v", L.v_w, L.v_b)):
                w.copy_(rows(sd[p + f"self_attn.{n}_proj.weight"]))
                b.copy_(rows(sd[p + f"self_attn.{n}_proj.bias"]))
            L.o_w.copy_(cols(sd[p + "self_attn.o_proj.weight"]))
            L.gate_w.copy_(rows(sd[p + "mlp.gate_proj.weight"]))
            L.up_w.copy_(rows(sd[p + "mlp.up_proj.weight"]))
            L.down_w.copy_(cols(sd[p + "mlp.down_proj.weight"]))
            L.ln1.copy_(sd[p + "input_layernorm.weight"])
            L.ln2.copy_(sd[p + "post_attention_layernorm.weight"])
        self.norm.copy_(sd["norm.weight"])
        if self.lm_head is not None:
            self.lm_head.copy_(rows(sd["lm_head.weight"]))


# --------------------------------------------------------------------------------------------------
# one rank of the baseline trainer
# --------------------------------------------------------------------------------------------------
class _FlatZero1:
    """ZeRO-1 with library calls: parameters and gradients are views of flat buffers; reduce-scatter (mean) the
    gradients, fused AdamW on the owned shard, all-gather the parameters."""

    def __init__(self, params, group, lr, betas, eps, weight_decay):
        params = [p for p in params]
        self.group = group
        self.n = dist.get_world_size(group) if group is not None else 1
        self.rank = dist.get_rank(group) if group is not None else 0
        total = sum(p.numel() for p in params)
        self.padded = (total + self.n * 8 - 1) // (self.n * 8) * (self.n * 8)
        dev, dt = params[0].device, params[0].dtype
        self.flat_p = torch.zeros(self.padded, device=dev, dtype=dt)
        self.flat_g = torch.zeros(self.padded, device=dev, dtype=dt)
        off = 0
        for p in params:
            n = p.numel()
            self.flat_p[off:off + n].copy_(p.data.reshape(-1))
            p.data = self.flat_p[off:off + n].view_as(p)
            p.grad = self.flat_g[off:off + n].view_as(p)
            off += n
        self.params = params
        per = self.padded // self.n
        self.shard_p = nn.Parameter(self.flat_p[self.rank * per:(self.rank + 1) * per])
        self.shard_g = self.flat_g[self.rank * per:(self.rank + 1) * per] if self.n == 1 else torch.empty(
            per, device=dev, dtype=dt)
        self.shard_p.grad = self.shard_g
        self.opt = torch.optim.AdamW([self.shard_p], lr=lr, betas=betas, eps=eps, weight_decay=weight_decay,
                                     fused=dev.type == "cuda")

    def zero_grad(self):
        self.flat_g.zero_()

    def step(self):
        if self.n > 1:
            _reduce_scatter(self.shard_g, self.flat_g, self.group, mean=True)
        self.opt.step()
        if self.n > 1:
            dist.all_gather_into_tensor(self.flat_p, self.shard_p.data, group=self.group)


class LibTrainer:
    """One process per GPU: vision rank (sequence parallel over the whole world) + text rank (tp x dp)."""

    def __init__(self, model_cfg, *, tp: int, device, dtype, seed: int = 0, lr: float = 1e-5):
        self.cfg = model_cfg
        self.device = device
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self.tp = tp
        self.tdp = self.world // tp
        self.tdp_rank, self.tp_rank = self.rank // tp, self.rank % tp
        self.world_group = self.tp_group = self.dp_group = None
        if self.world > 1:
            self.world_group = dist.group.WORLD
            for d in range(self.tdp):
                g = dist.new_group(list(range(d * tp, (d + 1) * tp)))
                if d == self.tdp_rank:
                    self.tp_group = g
            for t in range(tp):
                g = dist.new_group([d * tp + t for d in range(self.tdp)])
                if t == self.tp_rank:
                    self.dp_group = g
        self.vision = LibVision(model_cfg.vision, self.world_group, device, dtype, seed)
        self.text = LibText(model_cfg.text, self.tp_group if tp > 1 else None, device, dtype, seed)
        kw = dict(lr=lr, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0)
        self.vopt = _FlatZero1(self.vision.parameters(), self.world_group, **kw)
        if self.tdp > 1:
            # data-parallel replicas: one all-reduce (mean) over a flat gradient buffer, then a local fused AdamW
            self.topt = _FlatZero1(self.text.parameters(), None, **kw)
        else:
            self.topt_plain = torch.optim.AdamW(self.text.parameters(), fused=device.type == "cuda", **kw)
        self._cache = {}
        self.h2d_bytes = 0

    # -------------------------------------------------------------- host batch -> device
    def _prepare(self, samples):
        from multimodal_training_b200.parallel.handoff import pack_text_batch
        cfg = self.cfg
        grids = [g for s in samples for g in s.grid_thw]
        key = (tuple(grids), tuple(int(s.input_ids.numel()) for s in samples))
        st = self._cache.get(key)
        if st is None:
            if len(self._cache) > 8:
                self._cache.clear()
            st = self.vision.prepare(grids, self.device)
            st["merged_per_sample"] = [sum(t * h * w for t, h, w in s.grid_thw) // cfg.vision.merge_unit
                                       for s in samples]
            self._cache[key] = st
        per = len(samples) // self.tdp
        mine = samples[self.tdp_rank * per:(self.tdp_rank + 1) * per]
        tb = pack_text_batch(mine, image_token_id=cfg.image_token_id, vision_start_token_id=cfg.vision_start_token_id,
                             spatial_merge_size=cfg.vision.spatial_merge_size, pad_multiple=8,
                             pad_token_id=cfg.pad_token_id)
        lo = sum(st["merged_per_sample"][: self.tdp_rank * per])
        hi = lo + sum(st["merged_per_sample"][self.tdp_rank * per:(self.tdp_rank + 1) * per])
        return st, tb, (lo, hi)

    def train_step(self, samples) -> torch.Tensor:
        """One optimisation step on the global batch ``samples`` (every rank holds the same list)."""
        dev = self.device
        st, tb, (lo, hi) = self._prepare(samples)
        self.vopt.zero_grad()
        if self.tdp > 1:
            self.topt.zero_grad()
        else:
            self.topt_plain.zero_grad(set_to_none=True)
        # ---- vision forward (every rank loads the whole batch, as the reference's actors do)
        pix = [s.pixel_values for s in samples if s.pixel_values is not None]
        pixels = (pix[0] if len(pix) == 1 else torch.cat(pix, dim=0))
        pixels = pixels.to(dev, non_blocking=True).to(self.vision.patch_embed.dtype)
        ids = tb.input_ids.to(dev, non_blocking=True)
        labels = tb.shifted_labels.to(dev, non_blocking=True)
        pos = tb.position_ids.to(dev, non_blocking=True)
        self.h2d_bytes = pixels.numel() * pixels.element_size() + ids.numel() * 16 + pos.numel() * 8
        vis_out = self.vision(pixels, st)
        # ---- handoff: clone + masked_scatter
        leaf = vis_out[lo:hi].detach().clone().requires_grad_(True)
        emb = self.text.embed_tokens(ids)
        mask = (ids == self.cfg.image_token_id).unsqueeze(-1)
        x = emb.masked_scatter(mask, leaf.to(emb.dtype))
        cos, sin = self.text.rope_tables(pos)
        cu = torch.tensor(tb.cu_seqlens, dtype=torch.int32, device=dev)
        h = self.text(x, cos, sin, cu, tb.cu_seqlens)
        loss = self.text.loss(h, labels)
        # ---- backward: text, gradient clone back, vision
        loss.backward()
        g = torch.zeros_like(vis_out)
        g[lo:hi] = leaf.grad.detach().clone()
        vis_out.backward(g)
        # ---- optimizers
        if self.tdp > 1:
            _all_reduce_mean(self.topt.flat_g, self.dp_group)
            self.topt.step()
        else:
            self.topt_plain.step()
        self.vopt.step()
        return loss.detach()


# --------------------------------------------------------------------------------------------------
# benchmark entry (called by bench.py --impl lib, and by the sm100 arm to time its denominator in the same run)
# --------------------------------------------------------------------------------------------------
def _time_steps(tr, batches, steps: int, warmup: int, world: int):
    """(device ms/step, end-to-end ms/step, losses): CUDA events around ``steps`` steps after ``warmup``; then the
    same steps with every loss copied to pinned host memory and read one step late, on the host clock."""
    import time

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    losses = []
    for s in range(warmup):
        losses.append(float(tr.train_step(batches[s % 2])))
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    last = None
    for s in range(steps):
        last = tr.train_step(batches[s % 2])
    e1.record()
    barrier()
    dev_ms = e0.elapsed_time(e1) / steps
    losses.append(float(last))
    ring = [torch.zeros(1, dtype=torch.float32).pin_memory() for _ in range(4)]
    barrier()
    t0 = time.perf_counter()
    pending = None
    for s in range(steps):
        loss = tr.train_step(batches[s % 2])
        slot = ring[s % len(ring)]
        slot.copy_(loss.float().reshape(1), non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        if pending is not None:
            pending[1].synchronize()
            losses.append(float(pending[0][0]))
        pending = (slot, ev)
    pending[1].synchronize()
    losses.append(float(pending[0][0]))
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / steps
    barrier()
    return dev_ms, e2e_ms, losses


def run(model: str, *, image_size: int, text_tokens: int, global_batch: int, tp: int, steps: int, warmup: int,
        seed: int = 42, also_without_recompute: bool = True) -> dict:
    """Time library-only training steps of the benchmark configuration on the current device(s).

    Returns device ms/step (max over ranks) and end-to-end ms/step with every block activation-checkpointed (the
    reference's setting) and, when it fits in memory, with all activations kept, plus h2d bytes, peak memory and the
    first/last loss.  ``torch.distributed`` must be initialised when WORLD_SIZE > 1."""
    import gc

    from multimodal_training_b200.config.model_configs import get_model_config
    from multimodal_training_b200.data.synthetic import synthetic_global_batch

    cfg = get_model_config(model)
    dev = torch.device("cuda", torch.cuda.current_device())
    world = dist.get_world_size() if dist.is_initialized() else 1
    torch.cuda.reset_peak_memory_stats()
    tr = LibTrainer(cfg, tp=tp, device=dev, dtype=torch.bfloat16, seed=seed)
    batches = [synthetic_global_batch(cfg, i, global_batch, image_size=image_size, text_tokens=text_tokens, seed=seed,
                                      dtype=torch.bfloat16, pin=True) for i in range(2)]

    def reduce_max(*vals):
        t = torch.tensor(list(vals), device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return [float(x) for x in t]

    n_patches = sum(t_ * h * w for s in batches[0] for (t_, h, w) in s.grid_thw)
    dev_ms, e2e_ms, losses = _time_steps(tr, batches, steps, warmup, world)
    dev_ms, e2e_ms, peak = reduce_max(dev_ms, e2e_ms, torch.cuda.max_memory_allocated() / 2 ** 30)
    h2d = torch.tensor([float(tr.h2d_bytes)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(h2d, op=dist.ReduceOp.SUM)
    out = {"ms_per_step": dev_ms, "e2e_ms_per_step": e2e_ms, "peak_mem_gib": peak,
           "h2d_bytes_per_step": float(h2d[0]), "patches_per_step": n_patches,
           "loss_first_last": [losses[0], losses[-1]], "attention": "flash-attn 2" if _fa_varlen is not None else "sdpa",
           "gemm": "torch.nn.functional.linear (cuBLAS)", "collectives": "NCCL, placed as in the reference",
           "activation_checkpointing": "every block (the reference's setting)",
           "optimizer": "torch.optim.AdamW(fused=True), bf16 states, ZeRO-1 for the vision half",
           "without_recompute": None}
    if also_without_recompute:
        # the same steps with every activation kept: decided by all ranks together (an out-of-memory rank would
        # otherwise leave the others waiting in a collective)
        free = (torch.cuda.mem_get_info()[0] + torch.cuda.memory_reserved() - torch.cuda.memory_allocated()) / 2 ** 30
        t, v = cfg.text, cfg.vision
        tok_text = sum(int(s.input_ids.numel()) for s in batches[0]) // max(world // tp, 1)
        tok_vis = n_patches // world
        need = 1.5 * 2 * (tok_text * t.num_hidden_layers * (10 * t.hidden_size + 4 * t.intermediate_size // tp)
                          + tok_vis * v.depth * (10 * v.hidden_size + 4 * v.intermediate_size)
                          + 3 * tok_text * t.vocab_size // tp * 2) / 2 ** 30
        ok = reduce_max(0.0 if free > need else 1.0)[0] == 0.0
        if ok:
            try:
                tr.vision.checkpointing = tr.text.checkpointing = False
                torch.cuda.reset_peak_memory_stats()
                d2, e2, _ = _time_steps(tr, batches, steps, 2, world)
                d2, e2, pk2 = reduce_max(d2, e2, torch.cuda.max_memory_allocated() / 2 ** 30)
                out["without_recompute"] = {"ms_per_step": d2, "e2e_ms_per_step": e2, "peak_mem_gib": pk2}
            except torch.OutOfMemoryError as e:      # single-GPU runs only: nobody waits for this rank
                if world > 1:
                    raise
                out["without_recompute"] = {"error": "out of memory: " + str(e)[:120]}
        else:
            out["without_recompute"] = {"skipped": f"estimated {need:.0f} GiB of activations do not fit {free:.0f} GiB"}
    del tr
    gc.collect()
    torch.cuda.empty_cache()
    return out
