"""Qwen2.5-VL text decoder (Qwen2-style: pre-norm, GQA with q/k/v bias, SwiGLU, M-RoPE).

A lean ``nn.Module`` over this package's ops, built directly as its tensor-parallel shard:
fused q|k|v and gate|up projections (column-parallel), o_proj / down_proj (row-parallel),
vocab-parallel embedding and lm_head.  Activations between layers are token shards
(sequence-parallel TP, see ``parallel/tp.py``).  The math follows the reference's
``Qwen2_5_VLTextModel`` (modeling_qwen2_5_vl.py:1098-1527); the state dict converts to and
from the reference/HF key layout (q_proj/k_proj/v_proj, gate_proj/up_proj).
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn

from ..config.model_configs import TextConfig
from ..ops import attention as attn_mod
from ..ops import blocks
from ..ops import functional as F
from ..ops.attention import SeqInfo
from ..parallel import comm
from ..parallel.tp import TPContext, column_parallel_linear, row_parallel_linear, vocab_range
from ..utils.checkpointing import bucket_tokens, checkpoint
from ..utils.checkpointing import decide as decide_ckpt


_MROPE_CACHE: dict = {}


def mrope_cos_sin(position_ids: torch.Tensor, head_dim: int, theta: float, mrope_section: list[int], device=None):
    """cos/sin [T, head_dim] fp32 from 3-axis position ids [3, T].

    The doubled section list picks axis ``i mod 3`` for chunk i of the rotary dims
    (modeling_qwen2_5_vl.py:1123-1133,1185-1187).  With ``device`` the tables are built there from the position ids
    (one small host->device copy instead of two [T, head_dim] fp32 tables) and kept for batches with the same
    positions, which is every step of a fixed-shape run.
    """
    dev = torch.device(device) if device is not None else position_ids.device
    key = None
    if dev.type == "cuda":
        key = (hash(position_ids.cpu().numpy().tobytes()), tuple(position_ids.shape), head_dim, float(theta),
               tuple(mrope_section), str(dev))
        hit = _MROPE_CACHE.get(key)
        if hit is not None:
            return hit
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=dev) / head_dim))
    pos = position_ids.to(dev, non_blocking=True).to(torch.float32)
    freqs = pos[:, :, None] * inv_freq[None, None, :]            # [3, T, d/2]
    emb = torch.cat((freqs, freqs), dim=-1)                      # [3, T, d]
    sections = list(mrope_section) * 2
    chunks = emb.split(sections, dim=-1)
    sel = torch.cat([c[i % 3] for i, c in enumerate(chunks)], dim=-1)  # [T, d]
    out = (sel.cos().contiguous(), sel.sin().contiguous())
    if key is not None:
        if len(_MROPE_CACHE) >= 16:
            _MROPE_CACHE.pop(next(iter(_MROPE_CACHE)))
        _MROPE_CACHE[key] = out
    return out


class TextDecoder(nn.Module):
    def __init__(self, cfg: TextConfig, tp: TPContext | None = None, dtype=torch.float32, device="cpu", seed: int = 0,
                 activation_checkpointing: bool = True):
        super().__init__()
        self.cfg = cfg
        self.tp = tp or TPContext.single()
        self.ckpt = activation_checkpointing
        self.tp_block = True          # one autograd node per tensor-parallel layer on the fused paths (GPU)
        tpn, tpr = self.tp.size, self.tp.rank
        H, I, d = cfg.hidden_size, cfg.intermediate_size, cfg.head_dim
        if cfg.num_key_value_heads % tpn or cfg.num_attention_heads % tpn:
            raise ValueError(f"attention heads ({cfg.num_attention_heads}/{cfg.num_key_value_heads} kv) are not "
                             f"divisible by the tensor-parallel size {tpn}")
        if I % tpn:
            raise ValueError("intermediate_size is not divisible by the tensor-parallel size")
        self.n_q = cfg.num_attention_heads // tpn
        self.n_kv = cfg.num_key_value_heads // tpn
        self.inter = I // tpn
        self.vocab_lo, self.vocab_hi = vocab_range(cfg.vocab_size, tpn, tpr)
        std = cfg.initializer_range
        gen = torch.Generator(device=device)

        def full(shape, idx):
            # generated on the target device (fast for multi-billion-parameter models); every
            # rank draws the full tensor from the same seed and keeps its slice
            gen.manual_seed(seed * 1000003 + idx)
            return torch.randn(shape, generator=gen, dtype=torch.float32, device=device) * std

        def P(t):
            return nn.Parameter(t.to(device=device, dtype=dtype).contiguous())

        def rows(t, n_parts=1):
            """Slice dim 0 for this rank; n_parts>1 slices each of the stacked parts separately."""
            if tpn == 1:
                return t
            parts = t.chunk(n_parts, dim=0) if n_parts > 1 else (t,)
            return torch.cat([p.chunk(tpn, dim=0)[tpr] for p in parts], dim=0)

        hq, hkv = cfg.num_attention_heads * d, cfg.num_key_value_heads * d
        idx = 0
        self.embed_tokens = P(rows(full((cfg.vocab_size, H), idx)))
        idx += 1
        self.layers = nn.ModuleList()
        for _ in range(cfg.num_hidden_layers):
            L = nn.Module()
            wq, wk, wv = full((hq, H), idx), full((hkv, H), idx + 1), full((hkv, H), idx + 2)
            L.qkv_w = P(torch.cat([rows(wq), rows(wk), rows(wv)], dim=0))
            L.qkv_b = P(torch.zeros(L.qkv_w.shape[0], device=device))
            L.o_w = P(full((H, hq), idx + 3).chunk(tpn, dim=1)[tpr])
            L.gate_up_w = P(torch.cat([rows(full((I, H), idx + 4)), rows(full((I, H), idx + 5))], dim=0))
            L.down_w = P(full((H, I), idx + 6).chunk(tpn, dim=1)[tpr])
            L.ln1_w = P(torch.ones(H, device=device))
            L.ln2_w = P(torch.ones(H, device=device))
            L.ln1_w.sequence_parallel = tpn > 1
            L.ln2_w.sequence_parallel = tpn > 1
            idx += 7
            self.layers.append(L)
        self.norm_w = P(torch.ones(H, device=device))
        self.norm_w.sequence_parallel = tpn > 1
        if cfg.tie_word_embeddings:
            self.lm_head = None
        else:
            self.lm_head = P(rows(full((cfg.vocab_size, H), idx)))

    # ------------------------------------------------------------------ forward pieces
    def embed(self, input_ids: torch.Tensor) -> torch.Tensor:
        """Vocab-parallel lookup of all T tokens -> this rank's [T/tp, H] token shard."""
        part = F.embedding(input_ids, self.embed_tokens, self.vocab_lo)
        return comm.reduce_scatter(part, self.tp.group)

    def _layer(self, x, L, cos, sin, seq: SeqInfo):
        d = self.cfg.head_dim
        eps = self.cfg.rms_norm_eps
        qkv = column_parallel_linear(x, L.qkv_w, L.qkv_b, self.tp, norm_w=L.ln1_w, eps=eps, role="qkv")
        qkv = F.rope(qkv, cos, sin, self.n_q + self.n_kv, d)
        a = F.attention(qkv, self.n_q, self.n_kv, d, seq, causal=True)
        x = row_parallel_linear(a, L.o_w, x, self.tp, role="o")
        gu = column_parallel_linear(x, L.gate_up_w, None, self.tp, norm_w=L.ln2_w, eps=eps, role="mlp")
        m = F.swiglu(gu)
        return row_parallel_linear(m, L.down_w, x, self.tp, role="down")

    def activation_bytes(self, shard_tokens: int) -> int:
        """Bytes of activations that all layers of this rank keep for backward when nothing is recomputed (bf16);
        ``shard_tokens`` rows per rank, ``shard_tokens * tp`` gathered rows inside a layer."""
        cfg, tpn = self.cfg, self.tp.size
        T = int(shard_tokens) * tpn
        d = cfg.head_dim
        per_layer = int(shard_tokens) * 4 * cfg.hidden_size \
            + T * ((self.n_q + 2 * self.n_kv) * d + self.n_q * d + 3 * cfg.intermediate_size // tpn + 2 * cfg.hidden_size)
        return per_layer * 2 * len(self.layers)

    def forward(self, x_shard: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, seq: SeqInfo) -> torch.Tensor:
        """[T/tp, H] token shard -> final hidden token shard (before the last norm)."""
        x = x_shard
        # without tensor parallelism a layer has no communication inside and runs as one hand-written autograd
        # node (ops/blocks.py); tensor-parallel layers, the CPU path and un-checkpointed runs use the per-op graph
        need = self.activation_bytes(bucket_tokens(x.shape[0]))       # token shards are equal on all TP ranks
        ckpt = decide_ckpt(self.ckpt, need, x.device, group=self.tp.group,
                           key=("text", id(self))) if torch.is_grad_enabled() else False
        self.ckpt_now = ckpt
        keep_ew = (not ckpt) and x.is_cuda and not decide_ckpt("auto", need * 2, x.device, group=self.tp.group,
                                                              key=("text-ew", id(self)))
        if self.tp.fused is not None:
            self.tp.fused.set_checkpointed("text", ckpt)
        one_node = (self.tp.size == 1 and torch.is_grad_enabled() and blocks.usable(x)
                    and attn_mod.BACKEND == "sm100")
        if one_node:
            d = self.cfg.head_dim
            spec = blocks.BlockSpec(n_q=self.n_q, n_kv=self.n_kv, head_dim=d, rope_heads=self.n_q + self.n_kv,
                                    causal=True, eps=self.cfg.rms_norm_eps, scale=1.0 / math.sqrt(d))
            for L in self.layers:
                x = blocks.local_block(x, spec, cos, sin, seq, (L.ln1_w, L.qkv_w, L.qkv_b, L.o_w, None, L.ln2_w,
                                                                L.gate_up_w, None, L.down_w, None), recompute=ckpt,
                                       keep_elementwise=keep_ew)
            return x
        if (self.tp.size > 1 and self.tp.fused is not None and self.tp_block and torch.is_grad_enabled()
                and blocks.usable(x) and attn_mod.BACKEND == "sm100"):
            # tensor-parallel layers over the fused peer-memory paths: one autograd node per layer as well
            # (ops/tp_blocks.py); the per-op graph below stays for NCCL collectives, the CPU and as the oracle
            from ..ops import tp_blocks
            d = self.cfg.head_dim
            spec = blocks.BlockSpec(n_q=self.n_q, n_kv=self.n_kv, head_dim=d, rope_heads=self.n_q + self.n_kv,
                                    causal=True, eps=self.cfg.rms_norm_eps, scale=1.0 / math.sqrt(d))
            for L in self.layers:
                x = tp_blocks.tp_block(x, spec, cos, sin, seq, self.tp.fused,
                                       (L.ln1_w, L.qkv_w, L.qkv_b, L.o_w, L.ln2_w, L.gate_up_w, L.down_w),
                                       recompute=ckpt)
            return x
        for L in self.layers:
            x = checkpoint(lambda t, L=L: self._layer(t, L, cos, sin, seq), (x,), enabled=ckpt)
        return x

    def loss(self, x_shard: torch.Tensor, shifted_labels: torch.Tensor, chunk_rows: int = 4096,
             label_smoothing: float = 0.0) -> torch.Tensor:
        """Final norm -> all-gather -> lm_head + vocab-parallel CE (mean over rows with label >= 0)."""
        h = F.rmsnorm(x_shard, self.norm_w, self.cfg.rms_norm_eps)
        hg = comm.all_gather(h, self.tp.group)
        w = self.embed_tokens if self.lm_head is None else self.lm_head
        return F.lm_head_cross_entropy(hg, w, shifted_labels, self.vocab_lo, self.tp.group, chunk_rows,
                                       label_smoothing=label_smoothing)

    def logits(self, x_shard: torch.Tensor) -> torch.Tensor:
        """Local vocab-shard logits [T, V/tp] (tests and evaluation)."""
        h = F.rmsnorm(x_shard, self.norm_w, self.cfg.rms_norm_eps)
        hg = comm.all_gather(h, self.tp.group)
        w = self.embed_tokens if self.lm_head is None else self.lm_head
        return F.linear(hg, w)

    # ------------------------------------------------------------------ state dict in the reference/HF key layout
    def reference_state_dict(self) -> dict[str, torch.Tensor]:
        """This rank's shard under the reference's keys (q_proj/k_proj/v_proj, gate_proj/up_proj, ...)."""
        d = self.cfg.head_dim
        out = {"embed_tokens.weight": self.embed_tokens.detach()}
        for i, L in enumerate(self.layers):
            p = f"layers.{i}."
            nq, nkv = self.n_q * d, self.n_kv * d
            out[p + "self_attn.q_proj.weight"] = L.qkv_w.detach()[:nq]
            out[p + "self_attn.k_proj.weight"] = L.qkv_w.detach()[nq:nq + nkv]
            out[p + "self_attn.v_proj.weight"] = L.qkv_w.detach()[nq + nkv:]
            out[p + "self_attn.q_proj.bias"] = L.qkv_b.detach()[:nq]
            out[p + "self_attn.k_proj.bias"] = L.qkv_b.detach()[nq:nq + nkv]
            out[p + "self_attn.v_proj.bias"] = L.qkv_b.detach()[nq + nkv:]
            out[p + "self_attn.o_proj.weight"] = L.o_w.detach()
            out[p + "mlp.gate_proj.weight"] = L.gate_up_w.detach()[: self.inter]
            out[p + "mlp.up_proj.weight"] = L.gate_up_w.detach()[self.inter:]
            out[p + "mlp.down_proj.weight"] = L.down_w.detach()
            out[p + "input_layernorm.weight"] = L.ln1_w.detach()
            out[p + "post_attention_layernorm.weight"] = L.ln2_w.detach()
        out["norm.weight"] = self.norm_w.detach()
        if self.lm_head is not None:
            out["lm_head.weight"] = self.lm_head.detach()
        return {k: v.clone() for k, v in out.items()}

    @torch.no_grad()
    def load_reference_state_dict(self, sd: dict[str, torch.Tensor], sharded: bool = False) -> list[str]:
        """Load full (unsharded, default) or already-sharded weights in the reference key layout.

        Returns the keys that were not consumed.  Prefixes ``model.`` / ``language_model.`` are accepted.
        """
        tpn, tpr = self.tp.size, self.tp.rank
        clean = {}
        for k, v in sd.items():
            for pre in ("model.language_model.", "language_model.model.", "language_model.", "model."):
                if k.startswith(pre):
                    k = k[len(pre):]
                    break
            clean[k] = v
        used = set()

        def get(k):
            used.add(k)
            return clean[k]

        def r(t):
            return t if (sharded or tpn == 1) else t.chunk(tpn, dim=0)[tpr]

        def c(t):
            return t if (sharded or tpn == 1) else t.chunk(tpn, dim=1)[tpr]

        self.embed_tokens.copy_(r(get("embed_tokens.weight")))
        for i, L in enumerate(self.layers):
            p = f"layers.{i}."
            L.qkv_w.copy_(torch.cat([r(get(p + f"self_attn.{n}_proj.weight")) for n in "qkv"], dim=0))
            L.qkv_b.copy_(torch.cat([r(get(p + f"self_attn.{n}_proj.bias")) for n in "qkv"], dim=0))
            L.o_w.copy_(c(get(p + "self_attn.o_proj.weight")))
            L.gate_up_w.copy_(torch.cat([r(get(p + "mlp.gate_proj.weight")), r(get(p + "mlp.up_proj.weight"))], dim=0))
            L.down_w.copy_(c(get(p + "mlp.down_proj.weight")))
            L.ln1_w.copy_(get(p + "input_layernorm.weight"))
            L.ln2_w.copy_(get(p + "post_attention_layernorm.weight"))
        self.norm_w.copy_(get("norm.weight"))
        if self.lm_head is not None:
            key = "lm_head.weight" if "lm_head.weight" in clean else "embed_tokens.weight"
            self.lm_head.copy_(r(get(key)))
        return [k for k in clean if k not in used]
