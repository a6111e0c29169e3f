"""Qwen2.5-VL vision encoder with ragged Ulysses sequence parallelism.

Patch embedding (a GEMM: the Conv3d of the reference has kernel = stride), 32 pre-norm blocks with
2-D rotary attention (window attention everywhere except the full-attention layers) and a gated
SiLU MLP, then the 2x2 patch merger.  The math follows the reference's
``Qwen2_5_VisionTransformerPretrainedModel`` (modeling_qwen2_5_vl.py:192-1070).

What differs by design:

* every rank works on its window-aligned slice of every image (``parallel/sp.py``); window layers
  are purely local;
* full-attention layers exchange rows so that each rank attends over whole images with its share
  of the heads.  Rotary embedding is applied BEFORE the exchange, so cos/sin and masks never travel
  (the reference ships both through the all-to-all, modeling_qwen2_5_vl.py:632-640);
* the merger runs on the local slice (cuts are multiples of the 4-token merge unit), so the final
  all-gather of the reference (modeling_qwen2_5_vl.py:1018-1066) does not exist; merged tokens go
  straight to their text rows (``parallel/handoff.py``).
* q|k|v and gate|up are fused projections; the MLP width is zero-padded to a multiple of 8 so that
  activation rows are 16-byte aligned for TMA.  State dicts convert to the reference/HF layout.

``vision.parallelism: tensor`` (the reference's DTensor plan for the encoder, python/ray/vision.py:200-219,687-702)
is the second mode: every rank of the group sees all tokens of its replica's images, holds ``heads / tp`` attention
heads and ``1 / tp`` of the MLP width (column-parallel q|k|v and gate|up, row-parallel proj and down) and the block
outputs are all-reduced; norms, biases of the row-parallel layers, patch embedding and merger are replicated.
Sequence parallelism is the faster layout (28 of 32 layers without communication); this mode exists for parity.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn

from ..config.model_configs import VisionConfig
from ..ops import attention as attn_mod
from ..ops import blocks
from ..ops import functional as F
from ..ops import ulysses_block
from ..ops.attention import SeqInfo
from ..parallel import comm
from ..parallel.sp import VisionPlan
from ..parallel.tp import TPContext, copy_to_tp, reduce_from_tp
from ..utils.checkpointing import bucket_tokens, checkpoint
from ..utils.checkpointing import decide as decide_ckpt


class SPContext:
    """Sequence-parallel group of the vision encoder (None / size 1 = no exchange)."""

    def __init__(self, group=None, size: int = 1, rank: int = 0, fused=None):
        self.group, self.size, self.rank, self.fused = group, size, rank, fused


class VisionEncoder(nn.Module):
    def __init__(self, cfg: VisionConfig, sp: SPContext | None = None, dtype=torch.float32, device="cpu",
                 seed: int = 0, activation_checkpointing: bool = True, tp: TPContext | None = None):
        super().__init__()
        self.cfg = cfg
        self.sp = sp or SPContext()
        self.tp = tp or TPContext.single()
        self.ckpt = activation_checkpointing
        tpn, tpr = self.tp.size, self.tp.rank
        C, I, Ip = cfg.hidden_size, cfg.intermediate_size, cfg.padded_intermediate_size
        if cfg.num_heads % self.sp.size:
            raise ValueError(f"num_heads {cfg.num_heads} is not divisible by sequence_parallel_size {self.sp.size}")
        if tpn > 1:
            if self.sp.size > 1:
                raise ValueError("the vision encoder is either sequence parallel or tensor parallel, not both")
            if cfg.num_heads % tpn:
                raise ValueError(f"num_heads {cfg.num_heads} is not divisible by tensor_parallel_size {tpn}")
            Ip = (I + 8 * tpn - 1) // (8 * tpn) * (8 * tpn)      # every rank's slice of the MLP width 16-byte aligned
        self.Ip, self.Il, self.Cl = Ip, Ip // tpn, C // tpn
        std = cfg.initializer_range
        gen = torch.Generator(device=device)

        def full(shape, idx):
            gen.manual_seed(seed * 1000003 + 7919 + idx)
            return torch.randn(shape, generator=gen, dtype=torch.float32, device=device) * std

        def P(t):
            return nn.Parameter(t.to(device=device, dtype=dtype).contiguous())

        def pad_rows(t, n):
            if t.shape[0] == n:
                return t
            return torch.cat([t, t.new_zeros((n - t.shape[0],) + tuple(t.shape[1:]))], dim=0)

        def pad_cols(t, n):
            if t.shape[1] == n:
                return t
            return torch.cat([t, t.new_zeros(t.shape[0], n - t.shape[1])], dim=1)

        def head_rows(t):                 # [3C, ...] -> this rank's heads of q, of k and of v
            if tpn == 1:
                return t
            Cl = C // tpn
            return torch.cat([t[j * C + tpr * Cl:j * C + (tpr + 1) * Cl] for j in range(3)], 0)

        def my_rows(t):
            n = t.shape[0] // tpn
            return t[tpr * n:(tpr + 1) * n]

        def my_cols(t):
            n = t.shape[1] // tpn
            return t[:, tpr * n:(tpr + 1) * n]

        z = lambda n: torch.zeros(n, device=device)  # noqa: E731
        o = lambda n: torch.ones(n, device=device)   # noqa: E731
        idx = 0
        self.patch_embed_w = P(full((C, cfg.patch_dim), idx))
        idx += 1
        self.blocks = nn.ModuleList()
        for _ in range(cfg.depth):
            B = nn.Module()
            B.norm1_w, B.norm2_w = P(o(C)), P(o(C))
            B.qkv_w, B.qkv_b = P(head_rows(full((3 * C, C), idx))), P(z(3 * C // tpn))
            B.proj_w, B.proj_b = P(my_cols(full((C, C), idx + 1))), P(z(C))
            B.gate_up_w = P(torch.cat([my_rows(pad_rows(full((I, C), idx + 2), Ip)),
                                       my_rows(pad_rows(full((I, C), idx + 3), Ip))], 0))
            B.gate_up_b = P(z(2 * Ip // tpn))
            B.down_w, B.down_b = P(my_cols(pad_cols(full((C, I), idx + 4), Ip))), P(z(C))
            idx += 5
            self.blocks.append(B)
        M = C * cfg.merge_unit
        self.ln_q_w = P(o(C))
        self.merger_fc1_w, self.merger_fc1_b = P(full((M, M), idx)), P(z(M))
        self.merger_fc2_w, self.merger_fc2_b = P(full((cfg.out_hidden_size, M), idx + 1)), P(z(cfg.out_hidden_size))
        if tpn > 1:
            # identical on every tensor-parallel rank (same inputs, all-reduced gradients): counted once in the norm
            sharded = {id(p) for B in self.blocks for p in (B.qkv_w, B.qkv_b, B.proj_w, B.gate_up_w, B.gate_up_b,
                                                            B.down_w)}
            for p in self.parameters():
                if id(p) not in sharded:
                    p.tensor_replicated = True

    # ------------------------------------------------------------------ attention variants
    def _full_attention(self, qkv: torch.Tensor, plan: VisionPlan, full_seq: SeqInfo) -> torch.Tensor:
        """Ulysses: rows x all heads -> all rows x heads/sp, attention per image, and back."""
        cfg, sp = self.cfg, self.sp
        nh, d = cfg.num_heads, cfg.head_dim
        if sp.size == 1:
            return F.attention(qkv, nh, nh, d, full_seq, causal=False)
        if sp.fused is not None and qkv.is_cuda:
            return sp.fused.ulysses_attention(qkv, plan, full_seq, nh, d)
        T = qkv.shape[0]
        hl = nh // sp.size
        # [T, 3, sp, hl, d] -> [sp, T, 3*hl*d]: peer p gets head group p of q, k and v for all my rows
        send = qkv.view(T, 3, sp.size, hl, d).permute(2, 0, 1, 3, 4).reshape(sp.size * T, 3 * hl * d)
        recv = comm.all_to_all_rows(send, [T] * sp.size, plan.rank_tokens, sp.group)
        gathered = F.gather_rows(recv, plan.to_image_major_dev)          # (rank, image) -> (image, rank)
        a = F.attention(gathered, hl, hl, d, full_seq, causal=False)    # [T_all, hl*d]
        a = F.gather_rows(a, plan.to_rank_major_dev)
        back = comm.all_to_all_rows(a, plan.rank_tokens, [T] * sp.size, sp.group)   # [sp*T, hl*d]
        return back.view(sp.size, T, hl * d).permute(1, 0, 2).reshape(T, nh * d)

    def _block(self, x, B, cos, sin, plan, win_seq, full_seq, is_full: bool):
        cfg = self.cfg
        nh, d = cfg.num_heads, cfg.head_dim
        h = F.rmsnorm(x, B.norm1_w, cfg.rms_norm_eps)
        qkv = F.linear(h, B.qkv_w, B.qkv_b)
        qkv = F.rope(qkv, cos, sin, 2 * nh, d)
        if is_full:
            a = self._full_attention(qkv, plan, full_seq)
        else:
            a = F.attention(qkv, nh, nh, d, win_seq, causal=False)
        x = F.linear(a, B.proj_w, B.proj_b, x)
        h = F.rmsnorm(x, B.norm2_w, cfg.rms_norm_eps)
        m = F.swiglu(F.linear(h, B.gate_up_w, B.gate_up_b))
        return F.linear(m, B.down_w, B.down_b, x)

    def _block_tp(self, x, B, cos, sin, seq):
        """Tensor-parallel block on replicated activations: local heads / local MLP columns, two all-reduces."""
        cfg, tp = self.cfg, self.tp
        nh, d = cfg.num_heads // tp.size, cfg.head_dim
        h = copy_to_tp(F.rmsnorm(x, B.norm1_w, cfg.rms_norm_eps), tp)
        qkv = F.linear(h, B.qkv_w, B.qkv_b)
        qkv = F.rope(qkv, cos, sin, 2 * nh, d)
        a = F.attention(qkv, nh, nh, d, seq, causal=False)
        x = x + reduce_from_tp(F.linear(a, B.proj_w), tp) + B.proj_b
        h = copy_to_tp(F.rmsnorm(x, B.norm2_w, cfg.rms_norm_eps), tp)
        m = F.swiglu(F.linear(h, B.gate_up_w, B.gate_up_b))
        return x + reduce_from_tp(F.linear(m, B.down_w), tp) + B.down_b

    def activation_bytes(self, tokens: int) -> int:
        """Bytes of activations that all blocks keep for backward when nothing is recomputed (bf16)."""
        cfg = self.cfg
        per_token = 4 * cfg.hidden_size + 3 * cfg.hidden_size + 3 * cfg.padded_intermediate_size
        return int(tokens) * per_token * 2 * len(self.blocks)

    # ------------------------------------------------------------------ forward
    def forward(self, local_patches: torch.Tensor, plan: VisionPlan) -> torch.Tensor:
        """[T_loc, patch_dim] patches of this rank in local window order -> merged tokens [T_loc/4, out_hidden]."""
        cfg = self.cfg
        dev = local_patches.device
        prepare_plan(plan, dev)
        cos, sin = plan.cos_dev, plan.sin_dev
        win_seq = plan.win_seq
        full_seq = plan.full_seq if self.sp.size > 1 else plan.local_image_seq
        x = F.linear(local_patches, self.patch_embed_w)
        # blocks without communication inside run as one hand-written autograd node each (ops/blocks.py); the
        # Ulysses layers of a sequence-parallel run and the CPU path use the per-op graph.  Whether activations
        # are recomputed in backward is decided per step (True / False / "auto": keep them when they fit)
        peers = self.tp.group if self.tp.size > 1 else self.sp.group
        # the size every peer agrees on: the largest rank's token count (ragged cuts differ per rank), bucketed
        need = self.activation_bytes(bucket_tokens(max(plan.rank_tokens)))
        ckpt = decide_ckpt(self.ckpt, need, x.device, group=peers,
                           key=("vision", id(self))) if torch.is_grad_enabled() else False
        self.ckpt_now = ckpt
        # with memory to spare (twice the estimate still fits the budget) the element-wise intermediates are kept too
        keep_ew = (not ckpt) and x.is_cuda and not decide_ckpt("auto", need * 2, x.device, group=peers,
                                                              key=("vision-ew", id(self)))
        if self.sp.fused is not None:
            self.sp.fused.fc.set_checkpointed("vision", ckpt)
        one_node = (torch.is_grad_enabled() and blocks.usable(x) and attn_mod.BACKEND == "sm100"
                    and self.tp.size == 1)
        spec = blocks.BlockSpec(n_q=cfg.num_heads, n_kv=cfg.num_heads, head_dim=cfg.head_dim,
                                rope_heads=2 * cfg.num_heads, causal=False, eps=cfg.rms_norm_eps,
                                scale=1.0 / math.sqrt(cfg.head_dim))
        for i, B in enumerate(self.blocks):
            is_full = i in cfg.fullatt_block_indexes
            if self.tp.size > 1:
                x = checkpoint(lambda t, B=B, f=is_full: self._block_tp(t, B, cos, sin, full_seq if f else win_seq),
                               (x,), enabled=ckpt)
                continue
            if one_node and (not is_full or self.sp.size == 1):
                x = blocks.local_block(x, spec, cos, sin, full_seq if is_full else win_seq,
                                       (B.norm1_w, B.qkv_w, B.qkv_b, B.proj_w, B.proj_b, B.norm2_w, B.gate_up_w,
                                        B.gate_up_b, B.down_w, B.down_b), recompute=ckpt, keep_elementwise=keep_ew)
                continue
            if one_node and is_full and getattr(self.sp.fused, "one_node", False):
                # full attention across ranks: one node with the Ulysses exchanges inside the GEMMs
                x = ulysses_block.ulysses_block(x, spec, plan, full_seq, self.sp.fused,
                                                (B.norm1_w, B.qkv_w, B.qkv_b, B.proj_w, B.proj_b, B.norm2_w,
                                                 B.gate_up_w, B.gate_up_b, B.down_w, B.down_b), recompute=ckpt)
                continue
            x = checkpoint(lambda t, B=B, f=is_full: self._block(t, B, cos, sin, plan, win_seq, full_seq, f), (x,),
                           enabled=ckpt)
        h = F.rmsnorm(x, self.ln_q_w, cfg.rms_norm_eps)
        h = h.view(-1, cfg.hidden_size * cfg.merge_unit)
        h = F.gelu(F.linear(h, self.merger_fc1_w, self.merger_fc1_b))
        return F.linear(h, self.merger_fc2_w, self.merger_fc2_b)

    # ------------------------------------------------------------------ state dict in the reference/HF key layout
    def reference_state_dict(self, fused_qkv: bool = False) -> dict[str, torch.Tensor]:
        """Keys of the reference's vision model: ``blocks.N.attn.{q_proj,k_proj,v_proj,proj}``
        (modeling_qwen2_5_vl.py:334-338), ``mlp.{gate,up,down}_proj``, ``merger.{ln_q,mlp.0,mlp.2}``,
        ``patch_embed.proj.weight`` [C,3,2,14,14].  ``fused_qkv`` emits HF's ``attn.qkv`` instead of the
        reference's split projections (python/ray/vision.py:322-345)."""
        cfg = self.cfg
        # a tensor-parallel rank emits its shards under the same keys (rows of q/k/v/gate/up, columns of proj/down;
        # the zero padding of the MLP width is cut off, so the shards concatenate to the reference's shapes)
        C, Cl, Il = cfg.hidden_size, self.Cl, self.Il
        I = min(max(cfg.intermediate_size - self.tp.rank * Il, 0), Il)        # valid MLP columns of this rank
        Ip = Il
        out = {"patch_embed.proj.weight": self.patch_embed_w.detach().view(
            C, cfg.in_channels, cfg.temporal_patch_size, cfg.patch_size, cfg.patch_size)}
        for i, B in enumerate(self.blocks):
            p = f"blocks.{i}."
            out[p + "norm1.weight"] = B.norm1_w.detach()
            out[p + "norm2.weight"] = B.norm2_w.detach()
            if fused_qkv and self.tp.size == 1:
                out[p + "attn.qkv.weight"] = B.qkv_w.detach()
                out[p + "attn.qkv.bias"] = B.qkv_b.detach()
            else:
                for j, n in enumerate("qkv"):
                    out[p + f"attn.{n}_proj.weight"] = B.qkv_w.detach()[j * Cl:(j + 1) * Cl]
                    out[p + f"attn.{n}_proj.bias"] = B.qkv_b.detach()[j * Cl:(j + 1) * Cl]
            out[p + "attn.proj.weight"] = B.proj_w.detach()
            out[p + "attn.proj.bias"] = B.proj_b.detach()
            out[p + "mlp.gate_proj.weight"] = B.gate_up_w.detach()[:I]
            out[p + "mlp.up_proj.weight"] = B.gate_up_w.detach()[Ip:Ip + I]
            out[p + "mlp.gate_proj.bias"] = B.gate_up_b.detach()[:I]
            out[p + "mlp.up_proj.bias"] = B.gate_up_b.detach()[Ip:Ip + I]
            out[p + "mlp.down_proj.weight"] = B.down_w.detach()[:, :I]
            out[p + "mlp.down_proj.bias"] = B.down_b.detach()
        out["merger.ln_q.weight"] = self.ln_q_w.detach()
        out["merger.mlp.0.weight"] = self.merger_fc1_w.detach()
        out["merger.mlp.0.bias"] = self.merger_fc1_b.detach()
        out["merger.mlp.2.weight"] = self.merger_fc2_w.detach()
        out["merger.mlp.2.bias"] = self.merger_fc2_b.detach()
        return {k: v.clone() for k, v in out.items()}

    @torch.no_grad()
    def load_reference_state_dict(self, sd: dict[str, torch.Tensor], sharded: bool = False) -> list[str]:
        """Accepts the reference's split ``attn.{q,k,v}_proj`` (also the shorter ``attn.{q,k,v}`` that earlier
        checkpoints of this package used) or HF's fused ``attn.qkv``; prefixes ``visual.`` / ``model.visual.``.
        A tensor-parallel rank takes its slices of full tensors, or with ``sharded`` its own shards as written by
        ``reference_state_dict``."""
        cfg = self.cfg
        C, Cl, Il = cfg.hidden_size, self.Cl, self.Il
        tpn, tpr = self.tp.size, self.tp.rank
        I = min(max(cfg.intermediate_size - tpr * Il, 0), Il)
        Ip = Il
        take = tpn > 1 and not sharded

        def rows(t, width=None):          # this rank's rows of a full column-parallel tensor
            if not take:
                return t
            n = width or t.shape[0] // tpn
            return t[tpr * n:tpr * n + n]

        def cols(t, width=None):
            if not take:
                return t
            n = width or t.shape[1] // tpn
            return t[:, tpr * n:tpr * n + n]

        clean = {}
        for k, v in sd.items():
            for pre in ("model.visual.", "visual."):
                if k.startswith(pre):
                    k = k[len(pre):]
                    break
            clean[k] = v
        used = set()

        def get(k):
            used.add(k)
            return clean[k]

        self.patch_embed_w.copy_(get("patch_embed.proj.weight").reshape(C, -1))
        for i, B in enumerate(self.blocks):
            p = f"blocks.{i}."
            B.norm1_w.copy_(get(p + "norm1.weight"))
            B.norm2_w.copy_(get(p + "norm2.weight"))
            if p + "attn.qkv.weight" in clean:
                w, b = get(p + "attn.qkv.weight"), get(p + "attn.qkv.bias")
                B.qkv_w.copy_(torch.cat([rows(w[j * C:(j + 1) * C]) for j in range(3)], 0) if take else w)
                B.qkv_b.copy_(torch.cat([rows(b[j * C:(j + 1) * C]) for j in range(3)], 0) if take else b)
            else:
                suf = "_proj" if p + "attn.q_proj.weight" in clean else ""
                B.qkv_w.copy_(torch.cat([rows(get(p + f"attn.{n}{suf}.weight")) for n in "qkv"], 0))
                B.qkv_b.copy_(torch.cat([rows(get(p + f"attn.{n}{suf}.bias")) for n in "qkv"], 0))
            B.proj_w.copy_(cols(get(p + "attn.proj.weight")))
            B.proj_b.copy_(get(p + "attn.proj.bias"))
            B.gate_up_w.zero_()
            B.gate_up_b.zero_()
            B.down_w.zero_()
            B.gate_up_w[:I].copy_(rows(get(p + "mlp.gate_proj.weight"), Il))
            B.gate_up_w[Ip:Ip + I].copy_(rows(get(p + "mlp.up_proj.weight"), Il))
            B.gate_up_b[:I].copy_(rows(get(p + "mlp.gate_proj.bias"), Il))
            B.gate_up_b[Ip:Ip + I].copy_(rows(get(p + "mlp.up_proj.bias"), Il))
            B.down_w[:, :I].copy_(cols(get(p + "mlp.down_proj.weight"), Il))
            B.down_b.copy_(get(p + "mlp.down_proj.bias"))
        self.ln_q_w.copy_(get("merger.ln_q.weight"))
        self.merger_fc1_w.copy_(get("merger.mlp.0.weight"))
        self.merger_fc1_b.copy_(get("merger.mlp.0.bias"))
        self.merger_fc2_w.copy_(get("merger.mlp.2.weight"))
        self.merger_fc2_b.copy_(get("merger.mlp.2.bias"))
        return [k for k in clean if k not in used]


def prepare_plan(plan: VisionPlan, device) -> VisionPlan:
    """Attach device tensors and sequence descriptors to a host plan (idempotent)."""
    if getattr(plan, "_prepared", None) == str(device):
        return plan
    plan.cos_dev = plan.local_cos.to(device, non_blocking=True)
    plan.sin_dev = plan.local_sin.to(device, non_blocking=True)
    plan.win_seq = SeqInfo.from_list(plan.win_cu, device)
    plan.full_seq = SeqInfo.from_list(plan.full_cu, device)
    if plan.sp == 1:
        cu = list(plan.full_cu)            # whole images are local: one sequence per temporal patch
    else:
        cu = [0]
        for _, n in plan.per_image_local:
            if n:
                cu.append(cu[-1] + n)
    plan.local_image_seq = SeqInfo.from_list(cu, device)
    if plan.to_image_major is not None:
        plan.to_image_major_dev = plan.to_image_major.to(device, non_blocking=True)
        plan.to_rank_major_dev = plan.to_rank_major.to(device, non_blocking=True)
    plan._prepared = str(device)
    return plan
