"""Micro-benchmarks of the fused compute+collective paths against their NCCL + cuBLAS equivalents.

Run with one rank per GPU on one node, e.g.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 4 --master-addr 127.0.0.1 --master-port 29540 \
        -m multimodal_training_b200.utils.fused_bench --paths tp,handoff,ulysses --out fused_bench_n4.jsonl

Paths (all bf16, N(0,1) activations, N(0,0.02) weights):

* ``tp``      tensor-parallel all-gather -> GEMM (rows pushed into every peer's gather buffer, the GEMM's TMA
              producer consuming them per source rank) and GEMM -> reduce-scatter (partial tiles stored from
              the GEMM epilogue into the row owner's staging slot, summed there), hidden 3584 and 5120,
              2k-16k tokens, N = 3 x hidden and the MLP width;
* ``handoff`` vision -> text embedding rows [tokens, 3584] stored straight into the text ranks' buffers;
* ``ulysses`` sequence <-> heads exchange of the vision encoder (hidden 1280, 16 heads, head_dim 80) around the
              QKV projection and the output projection, sequences of 4k-64k patches.

The library arm places NCCL collectives where the reference has them (all-gather / reduce-scatter /
all-to-all) around ``torch.matmul``.  Every number is device time (CUDA events on the launching stream, warm-up
launches first, a 256 MiB write between timed launches so that no operand is served from L2), the MAX over ranks.
Roofline of a fused path = the slower of FLOPs / measured bf16 GEMM peak (``MEASURED_PEAKS.json`` burst figure,
else 1.59 PFLOP/s) and bytes that must cross NVLink / 770 GB/s (measured peer copy, per direction per GPU).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

from ..ops import functional as F
from ..ops import native as nv
from ..parallel.fused import FusedComm
from ..parallel.fused_ulysses import UlyssesFused
from ..parallel.mesh import build_mesh
from ..parallel.sp import build_vision_plan
from .kernel_bench import peaks

LINK_BPS = 770e9


def _timed(fn, iters: int, warmup: int, flush: torch.Tensor | None) -> float:
    """Median device milliseconds of fn over ``iters`` launches, max over ranks.

    The launches are queued behind a short device-side delay, each between its own pair of events, so that the host
    stays ahead of the device: the time between a pair of events is device time of fn alone (what it costs inside a
    training step, where the host also runs ahead), not the host's time to issue fn's second kernel.  Before every
    timed launch the L2 is flushed and a one-element all-reduce on the same stream lines the ranks up."""
    for _ in range(warmup):
        fn()
        dist.barrier()
    torch.cuda.synchronize()
    dist.barrier()
    tick = torch.zeros(1, device="cuda")
    pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
    torch.cuda._sleep(3_000_000)               # ~1.5 ms at 1.9 GHz
    for e0, e1 in pairs:
        if flush is not None:
            flush.zero_()
        dist.all_reduce(tick)
        e0.record()
        fn()
        e1.record()
    torch.cuda.synchronize()
    ts = sorted(e0.elapsed_time(e1) for e0, e1 in pairs)
    t = torch.tensor([ts[len(ts) // 2]], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def _emit(rec: dict, out) -> None:
    nv.raise_on_device_error()
    if dist.get_rank() == 0:
        line = json.dumps(rec)
        print(line, flush=True)
        if out is not None:
            out.write(line + "\n")
            out.flush()


def _roof_ms(flops: float, link_bytes: float) -> float:
    _, fl, _ = peaks()
    return max(flops / fl, link_bytes / LINK_BPS) * 1e3


def bench_tp(fc: FusedComm, args, out) -> None:
    m = fc.mesh
    tp, grp = m.tp, m.tp_group
    dev = fc.device
    shapes = []
    for hidden, inter in ((3584, 18944), (5120, 27648)):
        for tokens in args.tokens:
            shapes.append(("ag_gemm", tokens, hidden, 3 * hidden))       # column-parallel, N = 3 x hidden
            if hidden == 3584:
                shapes.append(("ag_gemm", tokens, hidden, 4608))         # the 7B model's q|k|v width (28 + 2 x 4 heads)
            shapes.append(("ag_gemm", tokens, hidden, 2 * inter))        # gate + up
            shapes.append(("gemm_rs", tokens, hidden, hidden))           # row-parallel o_proj: K = hidden
            shapes.append(("gemm_rs", tokens, hidden, inter))            # down_proj: K = MLP width
    for kind, T, H, W in shapes:
        if T % (tp * 128) or (W // tp) % 8:
            continue
        rows = T // tp
        torch.manual_seed(1 + m.rank)
        if kind == "ag_gemm":
            n_loc = W // tp
            x = torch.randn(rows, H, device=dev, dtype=torch.bfloat16)
            w = torch.randn(n_loc, H, device=dev, dtype=torch.bfloat16) * 0.02
            gathered_lib = torch.empty(T, H, device=dev, dtype=torch.bfloat16)
            y_lib = torch.empty(T, n_loc, device=dev, dtype=torch.bfloat16)

            def fused():          # the all-gather inside the GEMM kernel (chunk flags)
                return fc.ag_gemm(x, None, 0.0, w, role="bench_ag")[0]

            def fused_two_kernels():   # the earlier form: a push kernel in front of the GEMM, one flag per source
                g, _, flags, epoch = fc.push_gather(x, None, 0.0, "bench_ag2")
                return fc.gemm_gathered(g, flags, epoch, rows, w)

            def lib():
                dist.all_gather_into_tensor(gathered_lib, x, group=grp)
                torch.matmul(gathered_lib, w.t(), out=y_lib)

            def gemm_only():
                F.gemm(gathered_lib, w)

            flops = 2.0 * T * n_loc * H
            link = (tp - 1) / tp * T * H * 2
            yf = fused()
            lib()
            err = float((yf.float() - y_lib.float()).abs().max() / (y_lib.float().abs().max() + 1e-9))
        else:
            k_loc = W // tp
            a = torch.randn(T, k_loc, device=dev, dtype=torch.bfloat16)
            w = torch.randn(H, k_loc, device=dev, dtype=torch.bfloat16) * 0.02
            part = torch.empty(T, H, device=dev, dtype=torch.bfloat16)
            y_lib = torch.empty(rows, H, device=dev, dtype=torch.bfloat16)

            def fused():
                return fc.gemm_reduce_scatter(a, w, b_mn=False, residual=None, role=f"bench_rs_{T}_{H}")

            def lib():
                torch.matmul(a, w.t(), out=part)
                dist.reduce_scatter_tensor(y_lib, part, group=grp)

            def gemm_only():
                F.gemm(a, w, out=part)

            flops = 2.0 * T * H * k_loc
            link = (tp - 1) / tp * T * H * 2
            yf = fused()
            lib()
            err = float((yf.float() - y_lib.float()).abs().max() / (y_lib.float().abs().max() + 1e-9))
        flush = torch.empty(256 << 20, device=dev, dtype=torch.uint8)
        t_f = _timed(fused, args.iters, args.warmup, flush)
        t_l = _timed(lib, args.iters, args.warmup, flush)
        t_g = _timed(gemm_only, args.iters, args.warmup, flush)
        roof = _roof_ms(flops, link)
        extra = {}
        if kind == "ag_gemm":
            extra["push_kernel_then_gemm_ms"] = _timed(fused_two_kernels, args.iters, args.warmup, flush)
        _emit({"path": kind, "gpus": tp, "tokens": T, "hidden": H, "width": W, "fused_ms": t_f, "nccl_cublas_ms": t_l,
               **extra,
               "own_gemm_alone_ms": t_g, "speedup_vs_lib": t_l / t_f, "roofline_ms": roof,
               "frac_of_roofline": roof / t_f, "tflops_per_gpu": flops / t_f / 1e9, "link_gbs": link / t_f / 1e6,
               "max_rel_err_vs_lib": err, "peaks": peaks()[2]}, out)
        del flush


def bench_handoff(fc: FusedComm, args, out) -> None:
    m = fc.mesh
    dev = fc.device
    H = 3584
    for tokens in args.handoff_tokens:
        if tokens % m.world:
            continue
        n_loc = tokens // m.world                  # merged tokens produced by this vision rank
        torch.manual_seed(3)
        # every row goes to the text rank that owns its sample: block-cyclic over ranks, rows in arrival order
        dest_rank = (torch.arange(n_loc, device=dev, dtype=torch.int64) * m.world // n_loc).to(torch.int32)
        per = n_loc // m.world
        dest_row = m.rank * per + torch.arange(n_loc, device=dev, dtype=torch.int64) % per      # int64 rows
        src = torch.randn(n_loc, H, device=dev, dtype=torch.bfloat16)
        recv_lib = torch.empty(n_loc, H, device=dev, dtype=torch.bfloat16)
        embeds = torch.zeros(2 * n_loc, H, device=dev, dtype=torch.bfloat16)
        rows = torch.arange(0, 2 * n_loc, 2, device=dev)

        def fused():
            return fc.route(src, dest_rank, dest_row, f"bench_handoff_{tokens}", n_loc, H)

        def lib():
            # what the reference does per step with the same payload: a transport (here NCCL all-to-all instead of
            # its IPC map), a defensive clone, and masked_scatter into the embeddings
            dist.all_to_all_single(recv_lib, src, group=m.world_group)
            c = recv_lib.detach().clone()
            embeds.index_copy_(0, rows, c)

        got = fused()
        dist.all_to_all_single(recv_lib, src, group=m.world_group)
        err = float((got[:n_loc].float() - recv_lib.float()).abs().max())
        flush = torch.empty(256 << 20, device=dev, dtype=torch.uint8)
        t_f = _timed(fused, args.iters, args.warmup, flush)
        t_l = _timed(lib, args.iters, args.warmup, flush)
        link = (m.world - 1) / m.world * n_loc * H * 2
        roof = _roof_ms(0.0, link)
        _emit({"path": "handoff", "gpus": m.world, "tokens": tokens, "hidden": H, "fused_ms": t_f, "nccl_ms": t_l,
               "speedup_vs_lib": t_l / t_f, "roofline_ms": roof, "frac_of_roofline": roof / t_f,
               "link_gbs": link / t_f / 1e6, "max_abs_err_vs_lib": err}, out)
        del flush


def bench_ulysses(fc: FusedComm, args, out) -> None:
    m = fc.mesh
    dev = fc.device
    sp = m.sp
    nh, d, C = 16, 80, 1280
    if nh % sp:
        return
    uf = UlyssesFused(fc)
    hl = nh // sp
    for seq in args.seq:
        side = int(round(seq ** 0.5))
        if side * side != seq or side % 8:
            continue
        plan = build_vision_plan([(1, side, side)], sp=sp, rank=m.sp_rank, head_dim=d)
        T = plan.local_tokens
        torch.manual_seed(5 + m.rank)
        x = torch.randn(T, C, device=dev, dtype=torch.bfloat16)
        w_qkv = torch.randn(3 * C, C, device=dev, dtype=torch.bfloat16) * 0.02
        w_o = torch.randn(C, C, device=dev, dtype=torch.bfloat16) * 0.02
        routes = uf._routes(plan, dev)
        t_all = routes["t_all"]
        attn_out = torch.randn(t_all, hl * d, device=dev, dtype=torch.bfloat16)
        to_img = plan.to_image_major.to(dev)
        to_rank = plan.to_rank_major.to(dev)
        recv = torch.empty(t_all, 3 * hl * d, device=dev, dtype=torch.bfloat16)
        back = torch.empty(sp * T, hl * d, device=dev, dtype=torch.bfloat16)
        splits_in, splits_out = [T] * sp, list(plan.rank_tokens)
        equal = len(set(plan.rank_tokens)) == 1

        def fused_qkv():          # the exchange is the GEMM's epilogue (column scatter to the head owners)
            return uf.gemm_scatter(x, w_qkv, None, 3, routes, f"bench_ul_heads_{seq}")

        def kernel_qkv():         # the earlier form: GEMM, then an exchange kernel over peer memory
            qkv = F.gemm(x, w_qkv)
            return uf._exchange("heads", qkv, 3, hl * d, routes, f"bench_ul_heads_k_{seq}")

        def lib_qkv():
            qkv = torch.matmul(x, w_qkv.t())
            send = qkv.view(T, 3, sp, hl, d).permute(2, 0, 1, 3, 4).reshape(sp * T, 3 * hl * d)
            dist.all_to_all_single(recv, send, output_split_sizes=splits_out, input_split_sizes=splits_in,
                                   group=m.sp_group)
            return recv.index_select(0, to_img)

        def fused_out():          # rows go back without a wait; the GEMM waits per source before that K slice
            a, flags, epoch = uf.to_tokens_nowait(attn_out, hl * d, routes, f"bench_ul_tokens_{seq}")
            return uf.gemm_k_slices(a[:T], w_o, None, None, flags, epoch, hl * d)

        def kernel_out():
            a = uf._exchange("tokens", attn_out, 1, hl * d, routes, f"bench_ul_tokens_k_{seq}")[:T]
            return F.gemm(a, w_o)

        def lib_out():
            a = attn_out.index_select(0, to_rank)
            dist.all_to_all_single(back, a, output_split_sizes=splits_in, input_split_sizes=splits_out,
                                   group=m.sp_group)
            a2 = back.view(sp, T, hl * d).permute(1, 0, 2).reshape(T, nh * d)
            return torch.matmul(a2, w_o.t())

        if not equal:
            continue
        e1 = float((fused_qkv().float() - lib_qkv().float()).abs().max())
        e2 = float((fused_out().float() - lib_out().float()).abs().max())
        flush = torch.empty(256 << 20, device=dev, dtype=torch.uint8)
        for name, ff, kf, lf, flops, link, err in (
                ("ulysses_qkv", fused_qkv, kernel_qkv, lib_qkv, 2.0 * T * 3 * C * C, (sp - 1) / sp * T * 3 * C * 2, e1),
                ("ulysses_out", fused_out, kernel_out, lib_out, 2.0 * T * C * C, (sp - 1) / sp * T * C * 2, e2)):
            t_f = _timed(ff, args.iters, args.warmup, flush)
            t_k = _timed(kf, args.iters, args.warmup, flush)
            t_l = _timed(lf, args.iters, args.warmup, flush)
            roof = _roof_ms(flops, link)
            _emit({"path": name, "gpus": sp, "seq": seq, "rows_per_rank": T, "fused_ms": t_f,
                   "gemm_and_exchange_kernel_ms": t_k, "nccl_cublas_ms": t_l,
                   "speedup_vs_lib": t_l / t_f, "roofline_ms": roof, "frac_of_roofline": roof / t_f,
                   "link_gbs": link / t_f / 1e6, "max_abs_err_vs_lib": err}, out)
        del flush


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--paths", default="tp,handoff,ulysses")
    ap.add_argument("--tokens", type=int, nargs="*", default=[2048, 4096, 8192, 16384])
    ap.add_argument("--handoff-tokens", type=int, nargs="*", default=[1024, 4096, 16384])
    ap.add_argument("--seq", type=int, nargs="*", default=[4096, 16384, 65536])
    ap.add_argument("--iters", type=int, default=7)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--heap-mb", type=int, default=6144)
    ap.add_argument("--out", default=None)
    args = ap.parse_args(argv)
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    world = dist.get_world_size()
    mesh = build_mesh(sp=world, tp=world)
    fc = FusedComm(mesh, torch.device("cuda", local), args.heap_mb << 20)
    out = open(args.out, "a") if (args.out and dist.get_rank() == 0) else None
    paths = args.paths.split(",")
    if "tp" in paths:
        bench_tp(fc, args, out)
    if "handoff" in paths:
        bench_handoff(fc, args, out)
    if "ulysses" in paths:
        bench_ulysses(fc, args, out)
    dist.barrier()
    torch.cuda.synchronize()
    fc.close()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
