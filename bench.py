"""Headline benchmark: Qwen2.5-VL-7B training throughput on N B200 GPUs of one node.

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus 8 --steps 5 --warmup 3

Configuration (weak scaling: one sample per GPU, global batch = N): every sample is one 896x896
image (N(0,1) pixels, 4096 patches -> 1024 merged vision tokens) spliced into 1024 uniform-random
text tokens; random-init weights of the 7B architecture; bf16 compute; full AdamW (fp32 master
weights and moments) with ZeRO-1; activation checkpointing ``auto`` (activations are kept when they fit
in HBM; the same steps are also timed with recomputation forced on and reported in ``config``).  Parallel layout: vision
sequence-parallel over all N GPUs, text tensor-parallel over min(N, 4) GPUs with sequence-parallel
activations, data-parallel above that (N=8: SP=8 + TP=4 x DP=2).

The metric is the reference's: vision patches (before the 2x2 merge) x global batch / step time
(scripts/plot_performance.py:37-44,146-147 in the reference), plus LLM tokens/s in ``config``.
``value`` is device-timed with CUDA events (max over ranks); ``e2e`` times the same step through the
public API (``HybridEngine.train_step``) including, every step, the host->device copies of the
step's inputs from pinned host memory and a device->host read of the loss.

``--impl reference`` reports why the unmodified reference cannot run here.  ``--impl lib`` runs the same-box
library baseline (``baseline/lib_arm.py``): the reference's step restated with cuBLAS GEMMs, flash-attn 2, ATen
element-wise ops, ``torch.optim.AdamW(fused=True)`` and NCCL collectives in the reference's places; no kernel of this
repository runs in that arm.  The default arm times the library baseline first, in the same invocation on the same
GPUs, so that ``vs_baseline`` has a measured denominator (``--no-lib-arm`` skips it).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

REFERENCE_UNAVAILABLE = (
    "pip install of the reference tree fails offline (no setup.py/pyproject.toml) and its public API "
    "(python -m python.train_ray) imports ray, deepspeed (a git fork), hydra and omegaconf, none of which is in "
    "the image or the wheelhouse")


MODEL_NAMES = {"qwen2_5_vl_3b": "Qwen2.5-VL-3B", "qwen2_5_vl_7b": "Qwen2.5-VL-7B", "qwen2_5_vl_32b": "Qwen2.5-VL-32B",
               "qwen2_5_vl_72b": "Qwen2.5-VL-72B"}


def _clock_sampler(path: str):
    q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    try:
        f = open(path, "w")
        return subprocess.Popen(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits", "-lms", "200"],
                                stdout=f, stderr=subprocess.DEVNULL), f
    except Exception:
        return None, None


def _parse_clocks(path: str, n_gpus: int) -> dict:
    sm, mx, reasons, power = [], [], set(), []
    names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
    try:
        for line in open(path):
            p = [x.strip() for x in line.split(",")]
            if len(p) < 9 or not p[0].isdigit() or int(p[0]) >= n_gpus:
                continue
            try:
                sm.append(float(p[1]))
                mx.append(float(p[2]))
                power.append(float(p[3]))
            except ValueError:
                continue
            for name, val in zip(names, p[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
    except OSError:
        pass
    if not sm:
        return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
    busy = [s for s, pw in zip(sm, power) if pw > 300] or sm
    return {"sm_mhz": statistics.median(busy), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
            "samples": len(sm), "power_w_max": max(power)}


def _init_dist(local: int):
    """Process group from the torchrun environment (NCCL), without importing the framework."""
    import torch
    import torch.distributed as dist
    torch.cuda.set_device(local)
    if int(os.environ.get("WORLD_SIZE", "1")) > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))


def _run_lib_arm(args, global_batch: int, tp: int, steps: int, warmup: int) -> dict:
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    import lib_arm
    return lib_arm.run(args.model, image_size=args.image_size, text_tokens=args.text_tokens,
                       global_batch=global_batch, tp=tp, steps=steps, warmup=warmup)


def _native_so_loaded() -> list[str]:
    """Shared libraries from this repository that are mapped into this process right now."""
    found = set()
    root = os.path.realpath(ROOT)
    try:
        for line in open("/proc/self/maps"):
            path = os.path.realpath(line.rsplit(" ", 1)[-1].strip())
            if path.endswith(".so") and path.startswith(root + os.sep):
                found.add(os.path.relpath(path, root))
    except OSError:
        pass
    return sorted(found)


def _lib_best(lib: dict) -> tuple[float, float, str]:
    """(device ms, end-to-end ms, policy) of the faster of the library arm's two activation policies."""
    best = (lib["ms_per_step"], lib["e2e_ms_per_step"], "recompute")
    wo = lib.get("without_recompute") or {}
    if "ms_per_step" in wo and wo["ms_per_step"] < best[0]:
        best = (wo["ms_per_step"], wo["e2e_ms_per_step"], "keep")
    return best


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="sm100", choices=["sm100", "lib", "reference"])
    ap.add_argument("--model", default="qwen2_5_vl_7b")
    ap.add_argument("--image-size", type=int, default=896)
    ap.add_argument("--text-tokens", type=int, default=1024)
    ap.add_argument("--image-sizes", default="", help="comma-separated image sizes drawn per sample, new ones every "
                    "step (ragged run: no two steps have the same shapes; the library arm is skipped)")
    ap.add_argument("--text-token-choices", default="", help="comma-separated text lengths drawn per sample")
    ap.add_argument("--per-gpu-batch", type=int, default=1)
    ap.add_argument("--global-batch", type=int, default=0, help="overrides --per-gpu-batch x N (other configs)")
    ap.add_argument("--tp", type=int, default=0, help="text tensor-parallel size (default min(N, 4))")
    ap.add_argument("--no-fused-comm", action="store_true")
    ap.add_argument("--activation-checkpointing", default="auto", choices=["auto", "on", "off"],
                    help="auto (default): keep activations when they fit in HBM, recompute them otherwise")
    ap.add_argument("--optimizer-states", default="fp32", choices=["fp32", "bf16"],
                    help="fp32 (default): AdamW on fp32 master weights with fp32 moments; bf16: AdamW directly on the "
                         "bf16 parameters with bf16 moments, the precision of the reference's (and the library arm's) "
                         "optimizer")
    ap.add_argument("--symm-heap-mb", type=int, default=0, help="size of the symmetric heap (default: the config's)")
    ap.add_argument("--no-lib-arm", action="store_true",
                    help="do not time the library baseline in front of the sm100 arm (vs_baseline is then null)")
    ap.add_argument("--lib-steps", type=int, default=0, help="timed steps of the library baseline (default min(K, 10))")
    ap.add_argument("--no-idle-gaps", action="store_true",
                    help="skip the traced phase that measures device idle time between kernels")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": REFERENCE_UNAVAILABLE}))
        return 0
    if args.warmup < 3:
        args.warmup = 3

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus != world:
        if world == 1 and args.gpus > 1:
            # relaunch under torchrun so that `python bench.py --gpus N` also works by itself
            port = 29500 + (os.getpid() % 2000)
            cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
                   "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.abspath(__file__)] + sys.argv[1:]
            return subprocess.call(cmd)
        raise SystemExit(f"--gpus {args.gpus} does not match WORLD_SIZE {world}")
    _init_dist(local)

    N = args.gpus
    tp = args.tp or min(N, 4)
    sp = N
    global_batch = args.global_batch or N * args.per_gpu_batch
    if global_batch % (N // tp):
        raise SystemExit(f"global batch {global_batch} is not divisible by the {N // tp} text data-parallel replicas")
    par = f"sp{sp}" + (f"+tp{tp}" if tp > 1 else "") + (f"xdp{N // tp}" if N // tp > 1 else "")
    metric = (f"{MODEL_NAMES.get(args.model, args.model)} train tokens/s (vision patches x global batch / step "
              "time, max over ranks)")
    data = "synthetic (N(0,1) pixels, uniform-random token ids, random-init weights)"
    clock_path = os.path.join("/tmp", f"bench_clocks_{os.getpid()}.csv")

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ------------------------------------------------------------------ library baseline (this arm only, or first)
    lib = None
    if args.impl == "lib" or not (args.no_lib_arm or args.image_sizes or args.text_token_choices):
        lib_steps = args.steps if args.impl == "lib" else (args.lib_steps or min(args.steps, 10))
        sampler, fh = (None, None)
        if rank == 0 and args.impl == "lib":
            sampler, fh = _clock_sampler(clock_path)
        t0 = time.perf_counter()
        try:
            lib = _run_lib_arm(args, global_batch, tp, lib_steps, args.warmup)
            lib["steps"] = lib_steps
        except Exception as e:          # the sm100 arm is still measured; the line says why it has no denominator
            if args.impl == "lib":
                raise
            lib = {"error": f"{type(e).__name__}: {str(e)[:300]}"}
            import gc
            gc.collect()
            torch.cuda.empty_cache()
        lib["wall_s"] = time.perf_counter() - t0
        if sampler is not None:
            sampler.terminate()
            sampler.wait()
            fh.close()
        barrier()
    if args.impl == "lib":
        if rank == 0:
            ms, e2e_ms, policy = _lib_best(lib)
            patches = lib["patches_per_step"]
            out = {"metric": metric, "value": patches / (ms / 1e3), "unit": "tokens/s", "n_gpus": N,
                   "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
                   "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": data, "impl": "lib",
                   "config": {"model": args.model, "global_batch": global_batch,
                              "seq_len": args.text_tokens + patches // global_batch // 4,
                              "image": f"{args.image_size}x{args.image_size}", "parallelism": par,
                              "activation_policy_of_value": policy, "library_arm": lib,
                              "l2": "working set per step far exceeds the 126 MB L2; no explicit flush"},
                   "clocks": _parse_clocks(clock_path, N),
                   "e2e": {"value": patches / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                           "h2d_bytes_per_step": lib["h2d_bytes_per_step"], "d2h_bytes_per_step": 4.0 * N},
                   "gpu_launches": 0,
                   "gpu_launches_note": "library arm: cuBLAS, flash-attn, ATen and NCCL kernels only",
                   "native_so_loaded": _native_so_loaded()}
            print(json.dumps(out))
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return 0

    from multimodal_training_b200.config.loader import load_config
    from multimodal_training_b200.engine import HybridEngine
    from multimodal_training_b200.ops import native as nv

    ov = [
        f"vision.model_name={args.model}", f"text.model_name={args.model}",
        "vision.parallelism=sequence", "text.parallelism=tensor", f"text.tensor_parallel_size={tp}",
        f"training.parallel_size={sp}", "training.dp_size=1",
        f"training.batch_size={global_batch // (N // tp)}",
        "training.learning_rate=1e-5", "training.warmup_ratio=0", "training.warmup_steps=0",
        "training.lr_scheduler_type=constant", "training.num_iterations=1000000",
        f"+data.synthetic.image_size={args.image_size}", f"+data.synthetic.text_tokens={args.text_tokens}",
        f"+data.synthetic.global_batch={global_batch}", "+data.synthetic.repeat=2",
        f"training.fused_comm={'false' if args.no_fused_comm else 'true'}",
    ]
    ragged = bool(args.image_sizes or args.text_token_choices)
    if ragged:
        ov += ["+data.synthetic.repeat=0"]
        if args.image_sizes:
            ov.append(f"+data.synthetic.image_sizes={args.image_sizes}")
        if args.text_token_choices:
            ov.append(f"+data.synthetic.text_token_choices={args.text_token_choices}")
    if args.optimizer_states == "bf16":
        ov.append("training.optimizer_master_weights=false")
    ckpt = {"auto": "auto", "on": "true", "off": "false"}[args.activation_checkpointing]
    ov += [f"vision.activation_checkpointing={ckpt}", f"text.activation_checkpointing={ckpt}"]
    if args.symm_heap_mb:
        ov.append(f"training.symm_heap_mb={args.symm_heap_mb}")
    cfg = load_config(None, ov)
    torch.cuda.reset_peak_memory_stats()
    engine = HybridEngine.from_config(cfg)
    engine.record_optimizer_time = True

    # pre-generate the host batches (pinned) outside every timed region
    for s in range(2):
        engine.vision.step_context(s)
    losses = []
    for s in range(args.warmup):
        losses.append(engine.train_step_async(s).value())
    nv.raise_on_device_error()
    engine.optimizer_ms()

    sampler, fh = (None, None)
    if rank == 0:
        sampler, fh = _clock_sampler(clock_path)

    # ---- device-timed region: K steps between CUDA events, loss read back only at the end
    step0 = args.warmup
    barrier()
    launches0 = nv.launch_count
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    last = None
    h0 = time.perf_counter()
    for s in range(args.steps):
        last = engine.train_step(step0 + s)
    host_enqueue_ms = (time.perf_counter() - h0) * 1e3 / args.steps
    engine.join_streams()          # the timed region ends after the last optimizer update, whichever stream ran it
    e1.record()
    barrier()
    dev_ms = e0.elapsed_time(e1)
    opt_ms = engine.optimizer_ms() / args.steps
    launches = nv.launch_count - launches0
    losses.append(float(last))

    # ---- end-to-end region: same public call, loss read back to the host every step
    step0 += args.steps
    barrier()
    t0 = time.perf_counter()
    # every step: inputs go host -> device from pinned memory inside train_step, the loss goes device -> host into
    # pinned memory; the host reads the loss of step s-1 after it has launched step s
    pending = None
    for s in range(args.steps):
        handle = engine.train_step_async(step0 + s)
        if pending is not None:
            losses.append(pending.value())
        pending = handle
    losses.append(pending.value())
    engine.join_streams()
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    barrier()
    if sampler is not None:
        sampler.terminate()
        sampler.wait()
        fh.close()
    nv.raise_on_device_error()
    engine.optimizer_ms()

    # ---- the same steps with activation recomputation forced on (the reference's setting), for comparison
    policy = {"vision": bool(engine.vision.model.ckpt_now), "text": bool(engine.text.model.ckpt_now)}
    ckpt_on_ms = None
    if args.activation_checkpointing == "auto" and not all(policy.values()):
        saved = (engine.vision.model.ckpt, engine.text.model.ckpt)
        engine.vision.model.ckpt = engine.text.model.ckpt = True
        step0 += args.steps
        for s in range(2):
            engine.train_step(step0 + s)
        barrier()
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        c0.record()
        for s in range(args.steps):
            engine.train_step(step0 + 2 + s)
        engine.join_streams()
        c1.record()
        barrier()
        ckpt_on_ms = c0.elapsed_time(c1) / args.steps
        engine.vision.model.ckpt, engine.text.model.ckpt = saved
        nv.raise_on_device_error()
        engine.optimizer_ms()
        step0 += args.steps + 2
        for s in range(2):              # back to the headline policy before the traced phase
            engine.train_step(step0 + s)
        step0 += 2

    # ---- device time per phase of the step (CUDA events, three extra steps after every timed region)
    phases = None
    try:
        from multimodal_training_b200.utils.tracing import PhaseTimer
        engine.timer = PhaseTimer()
        for s in range(3):
            engine.train_step(step0 + s)
        step0 += 3
        summ = engine.timer.summary()
        engine.timer = None
        names = sorted(summ)
        pt = torch.tensor([summ[k] for k in names], device="cuda", dtype=torch.float64)
        if world > 1:
            dist.all_reduce(pt, op=dist.ReduceOp.MAX)
        phases = {k: float(v) for k, v in zip(names, pt)}
    except Exception as e:
        engine.timer = None
        phases = {"error": f"{type(e).__name__}: {str(e)[:200]}"}
    barrier()

    # ---- device idle time between kernels (host-bound or not), traced, after every timed region
    idle = None
    if not args.no_idle_gaps:
        engine.record_optimizer_time = False
        try:
            if rank == 0:
                from multimodal_training_b200.utils.idle_gaps import measure
                counter = [step0]

                def one_step():
                    engine.train_step(counter[0])
                    counter[0] += 1

                idle = measure(one_step, steps=2, ready=barrier)
            else:
                barrier()
                for s in range(2):
                    engine.train_step(step0 + s)
        except Exception as e:          # a diagnostic: never fails the benchmark
            idle = {"error": f"{type(e).__name__}: {str(e)[:200]}"}
        barrier()

    t = torch.tensor([dev_ms, e2e_s * 1e3, ckpt_on_ms or 0.0, opt_ms], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms, opt_ms = float(t[0]), float(t[1]), float(t[3])
    ckpt_on_ms = float(t[2]) if ckpt_on_ms is not None else None
    h2d = torch.tensor([float(engine.vision.h2d_bytes + engine.text.h2d_bytes)], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(h2d, op=dist.ReduceOp.SUM)
    peak_mem = torch.tensor([torch.cuda.max_memory_allocated() / 2 ** 30], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(peak_mem, op=dist.ReduceOp.MAX)

    if rank == 0:
        ctx = engine.vision.step_context(0)
        patches = ctx.n_vision_patches_global
        llm_tokens = ctx.n_text_tokens_global
        if ragged:
            # shapes differ from step to step: the mean over the steps of the device-timed region
            ctxs = [engine.vision.step_context(args.warmup + s) for s in range(args.steps)]
            patches = sum(c.n_vision_patches_global for c in ctxs) / len(ctxs)
            llm_tokens = sum(c.n_text_tokens_global for c in ctxs) / len(ctxs)
        ms_per_step = dev_ms / args.steps
        value = patches / (ms_per_step / 1e3)
        e2e_value = patches / (e2e_ms / args.steps / 1e3)
        vs_baseline = vs_recompute = e2e_vs = None
        if lib is not None and "ms_per_step" in lib:
            lib_ms, lib_e2e_ms, lib_policy = _lib_best(lib)
            vs_baseline = lib_ms / ms_per_step
            e2e_vs = lib_e2e_ms / (e2e_ms / args.steps)
            vs_recompute = lib["ms_per_step"] / (ckpt_on_ms if ckpt_on_ms else ms_per_step)
        out = {
            "metric": metric,
            "value": value, "unit": "tokens/s", "n_gpus": N, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": vs_baseline,
            "vs_baseline_note": "value / tokens-per-second of the all-library baseline (bench.py --impl lib: cuBLAS, "
                                "flash-attn 2, ATen, torch AdamW, NCCL in the reference's places) timed in this same "
                                "invocation on the same GPUs, each arm with its faster activation policy; the "
                                "unmodified reference does not install here and its published numbers are for "
                                "another model and machine",
            "dtype": "bf16", "data": data,
            "impl": args.impl,
            "baseline": None if lib is None else dict(lib, **{
                "impl": "lib", "vs_baseline_both_recomputing": vs_recompute, "e2e_vs_baseline": e2e_vs}),
            "ms_per_step_excluding_optimizer": ms_per_step - opt_ms,
            "optimizer_ms_per_step": opt_ms,
            "optimizer_note": "device time of the optimizer phase (gradient reduce-scatter, AdamW on fp32 master "
                              "weights and moments, parameter all-gather); one GPU holds all 8.3 G parameters' "
                              "states, N GPUs hold 1/N each, so this part shrinks with N under weak scaling",
            "config": {
                "model": args.model, "global_batch": global_batch, "seq_len": args.text_tokens + patches // global_batch // 4,
                "image": (f"{args.image_size}x{args.image_size}" if not args.image_sizes
                          else f"square, side drawn per sample from {{{args.image_sizes}}}, new shapes every step"),
                "vision_patches_per_sample": patches // global_batch,
                "text_tokens_per_sample": args.text_token_choices or args.text_tokens, "parallelism": par,
                "optimizer": ("AdamW fp32 master+moments, ZeRO-1" if args.optimizer_states == "fp32" else
                              "AdamW on bf16 parameters with bf16 moments (no master copy), ZeRO-1"),
                "activation_checkpointing": {
                    "setting": args.activation_checkpointing,
                    "recompute_in_this_run": policy,
                    "note": "auto keeps the activations of a half of the model when they fit into half of the free "
                            "HBM and recomputes them otherwise; the reference always recomputes (80 GB GPUs)",
                    "ms_per_step_with_recompute_forced_on": ckpt_on_ms,
                    "value_with_recompute_forced_on": (patches / (ckpt_on_ms / 1e3)) if ckpt_on_ms else None},
                "llm_tokens_per_s": llm_tokens / (ms_per_step / 1e3),
                "l2": "working set per step (weights, gradients, optimizer state: >100 GB) far exceeds the 126 MB L2; "
                      "no explicit flush",
                "fused_comm": bool(process_fused()), "peak_mem_gib": float(peak_mem[0]),
                "published_nearest": "15,464 tok/s, Qwen2.5-VL-32B SP+TP on 8xH100 at 4096 patches (different model)",
                "loss_first_last": [losses[0], losses[-1]],
            },
            "clocks": _parse_clocks(clock_path, N),
            "e2e": {"value": e2e_value, "unit": "tokens/s", "ms_per_step": e2e_ms / args.steps,
                    "h2d_bytes_per_step": float(h2d[0]), "d2h_bytes_per_step": 4.0 * N,
                    "timer": "host wall clock between barriers, max over ranks",
                    "loss_read": "copied to pinned host memory every step, read by the host one step later"},
            "host_enqueue_ms_per_step": host_enqueue_ms,
            "host_enqueue_note": "wall time of the loop that enqueues the timed steps; once the host is about a "
                                 "thousand launches ahead it waits for launch-queue slots, so this approaches the "
                                 "device time from below even when the host is not the limit; device_idle is the "
                                 "measurement that separates the two cases",
            "phases_ms": phases,
            "device_idle": idle,
            "gpu_launches": int(launches),
            "gpu_launches_per_step": launches / args.steps,
            "native_so_loaded": _native_so_loaded(),
        }
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


def process_fused():
    from multimodal_training_b200.trainers.trainer import process_state
    return process_state().fused is not None


if __name__ == "__main__":
    sys.exit(main())
