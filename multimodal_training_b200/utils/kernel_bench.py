"""Micro-benchmarks of the sm_100a kernels with roofline fractions.

    python -m multimodal_training_b200.utils.kernel_bench gemm --m 8192 --n 8192 --k 8192
    python -m multimodal_training_b200.utils.kernel_bench attention --tokens 16384 --heads 7 --kv-heads 1 --dim 128 --causal
    python -m multimodal_training_b200.utils.kernel_bench rmsnorm --rows 65536 --cols 3584
    python -m multimodal_training_b200.utils.kernel_bench adamw --elems 268435456
    python -m multimodal_training_b200.utils.kernel_bench gemm_shapes      # the training step's GEMMs beside cuBLAS

Timing: CUDA events on the launching stream, >= 3 warm-up launches, an L2 flush (a 256 MiB write)
between timed launches, median of the timed launches.  Fractions are relative to the measured peaks in
``MEASURED_PEAKS.json`` at the repository root when present (copy bandwidth and cuBLAS bf16 burst
throughput), else to 6.65 TB/s and 1.59 PFLOP/s.  ``--iters 1 --no-flush`` gives a single clean launch
for profilers.
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from ..ops import functional as F
from ..ops import native as nv
from ..ops.attention import SeqInfo


def peaks() -> tuple[float, float, str]:
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))),
                        "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return float(d["hbm_gbs"]) * 1e9, float(d["bf16_tflops"]) * 1e12, "of measured"
    return 6.65e12, 1.59e15, "of fallback"


def timed(fn, iters: int, warmup: int, flush: bool) -> float:
    buf = torch.empty(256 << 20, device="cuda", dtype=torch.uint8) if flush else None
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if buf is not None:
            buf.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2] * 1e-3


def report(name: str, seconds: float, flops: float = 0.0, bytes_: float = 0.0, **extra) -> dict:
    bw, fl, tag = peaks()
    out = {"kernel": name, "ms": seconds * 1e3, **extra}
    if flops:
        out["tflops"] = flops / seconds / 1e12
        out["frac_compute"] = flops / seconds / fl
    if bytes_:
        out["gbs"] = bytes_ / seconds / 1e9
        out["frac_hbm"] = bytes_ / seconds / bw
    out["peaks"] = tag
    print(json.dumps(out))
    return out


# GEMMs of one Qwen2.5-VL-7B training step on one GPU (896 px image + 1024 text tokens): (tokens, out features,
# in features) of every linear layer; each runs as forward, input-gradient and weight-gradient GEMM
STEP_SHAPES = [("text qkv", 2048, 4608, 3584), ("text o_proj", 2048, 3584, 3584), ("text gate|up", 2048, 37888, 3584),
               ("text down", 2048, 3584, 18944), ("lm_head", 2048, 152064, 3584), ("vision qkv", 4096, 3840, 1280),
               ("vision proj", 4096, 1280, 1280), ("vision gate|up", 4096, 6848, 1280),
               ("vision down", 4096, 1280, 3424)]


class _ClockLog:
    """SM clock samples (nvidia-smi, 100 ms) with host timestamps, to attribute a median clock to a timed loop."""

    def __init__(self):
        import subprocess
        import tempfile
        self.path = tempfile.mktemp(suffix=".csv")
        self.f = open(self.path, "w")
        try:
            self.p = subprocess.Popen(["nvidia-smi", "-i", str(torch.cuda.current_device()),
                                       "--query-gpu=timestamp,clocks.sm", "--format=csv,noheader,nounits", "-lms", "100"],
                                      stdout=self.f, stderr=subprocess.DEVNULL)
        except OSError:
            self.p = None

    def close(self):
        if self.p is not None:
            self.p.terminate()
            self.p.wait()
        self.f.close()
        import datetime
        self.samples = []
        for line in open(self.path):
            try:
                ts, mhz = line.rsplit(",", 1)
                t = datetime.datetime.strptime(ts.strip(), "%Y/%m/%d %H:%M:%S.%f").timestamp()
                self.samples.append((t, float(mhz)))
            except ValueError:
                continue

    def median(self, t0: float, t1: float):
        v = sorted(m for t, m in self.samples if t0 + 0.15 <= t <= t1)
        return v[len(v) // 2] if v else None


def sustained(fn, seconds: float) -> tuple[float, float, float]:
    """Back-to-back launches for about ``seconds``: (seconds per launch, host t0, host t1)."""
    import time
    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    fn()
    e1.record()
    torch.cuda.synchronize()
    n = max(3, int(seconds / max(e0.elapsed_time(e1) * 1e-3, 1e-6)))
    t0 = time.time()
    e0.record()
    for _ in range(n):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e-3 / n, t0, time.time()


def gemm_shapes(a) -> int:
    """Every GEMM shape of the 7B step in its three operand layouts: this library's kernel beside cuBLAS
    (``torch.matmul``), burst (L2 flushed, median) and sustained (back to back under the power cap), with the median
    SM clock sampled during each sustained loop."""
    dev = "cuda"
    log = _ClockLog()
    rows = []
    for name, T, O, I in STEP_SHAPES:
        x = torch.randn(T, I, device=dev, dtype=torch.bfloat16)
        w = torch.randn(O, I, device=dev, dtype=torch.bfloat16) * 0.02
        dy = torch.randn(T, O, device=dev, dtype=torch.bfloat16)
        y, dx, dw = torch.empty_like(dy), torch.empty_like(x), torch.empty_like(w)
        cases = [("fwd", lambda: F.gemm(x, w, out=y), lambda: torch.matmul(x, w.t(), out=y)),
                 ("dgrad", lambda: F.gemm(dy, w, b_mn=True, out=dx), lambda: torch.matmul(dy, w, out=dx)),
                 ("wgrad", lambda: F.gemm(dy, x, a_mn=True, b_mn=True, out=dw), lambda: torch.matmul(dy.t(), x, out=dw))]
        for layout, mine, cublas in cases:
            fl = 2.0 * T * O * I
            r = {"gemm": name, "layout": layout, "tokens": T, "out": O, "in": I}
            r["burst_tflops"] = fl / timed(mine, a.iters, a.warmup, True) / 1e12
            r["cublas_burst_tflops"] = fl / timed(cublas, a.iters, a.warmup, True) / 1e12
            ts, t0, t1 = sustained(mine, a.sustain)
            tc, c0, c1 = sustained(cublas, a.sustain)
            r["sustained_tflops"], r["cublas_sustained_tflops"] = fl / ts / 1e12, fl / tc / 1e12
            r["_t"] = (t0, t1, c0, c1)
            rows.append(r)
    log.close()
    tot = {"mine": 0.0, "cublas": 0.0}
    for r in rows:
        t0, t1, c0, c1 = r.pop("_t")
        r["sm_mhz"], r["cublas_sm_mhz"] = log.median(t0, t1), log.median(c0, c1)
        r["burst_vs_cublas"] = r["burst_tflops"] / r["cublas_burst_tflops"]
        r["sustained_vs_cublas"] = r["sustained_tflops"] / r["cublas_sustained_tflops"]
        fl = 2.0 * r["tokens"] * r["out"] * r["in"] * (28 if r["gemm"].startswith("text") else 32 if r["gemm"].startswith("vision") else 1)
        tot["mine"] += fl / r["sustained_tflops"]
        tot["cublas"] += fl / r["cublas_sustained_tflops"]
        print(json.dumps(r))
    print(json.dumps({"step_weighted_sustained_vs_cublas": tot["cublas"] / tot["mine"],
                      "note": "time of all GEMMs of one step (layer counts applied) with cuBLAS / with this kernel"}))
    return 0


def gemm_roles(a) -> int:
    """The GEMM's collective roles on ONE GPU, with local buffers standing in for the peers' (the kernel and its
    instruction stream are the ones that run across GPUs; only the destination addresses are local): what each role
    costs over the plain GEMM of the same shape, and a small case to capture under a profiler.

    * forwarder: rank 0 of 2 computes gathered [2 x rows, K] x [N, K]^T and forwards its own rows to the "peer"
    * scatter:   [rows, K] x [3C, K]^T whose epilogue scatters column blocks to 2 "ranks" at mapped rows
    * k_slices:  [rows, C] x [C, C]^T that waits per K slice (flags already set)"""
    import ctypes

    from ..parallel.fused import GemmCommC
    dev = "cuda"
    rows, K, N = a.m // 2, a.k, a.n
    torch.manual_seed(0)
    gathered = torch.randn(2 * rows, K, device=dev, dtype=torch.bfloat16)
    w = torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.02
    peer = torch.empty_like(gathered)
    flags = torch.ones(8 * 64, device=dev, dtype=torch.int32)
    peer_flags = torch.zeros(8 * 64, device=dev, dtype=torch.int32)
    counter = torch.zeros(64, device=dev, dtype=torch.int32)
    out = torch.empty(2 * rows, N, device=dev, dtype=torch.bfloat16)

    def forwarder():
        c = GemmCommC()
        c.ag_flags, c.ag_epoch, c.ag_rows, c.ag_self, c.rs_rows = flags.data_ptr(), 1, rows, 0, 0
        c.fwd_dst[0], c.fwd_flag[0], c.fwd_peers = peer.data_ptr(), peer_flags.data_ptr(), 1
        c.fwd_counter = counter.data_ptr()
        nv.lib().mmt_gemm_set_comm(ctypes.byref(c))
        F.gemm(gathered, w, out=out)

    def back_to_back(fn, n=40):
        """Seconds per launch with the launches queued back to back (no host gap between them, warm L2)."""
        for _ in range(3):
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e-3 / n

    t_plain = timed(lambda: F.gemm(gathered, w, out=out), a.iters, a.warmup, not a.no_flush)
    t_fwd = timed(forwarder, a.iters, a.warmup, not a.no_flush)
    b_plain, b_fwd = back_to_back(lambda: F.gemm(gathered, w, out=out)), back_to_back(forwarder)
    ok = bool(torch.equal(peer[:rows], gathered[:rows]))
    fl = 2.0 * 2 * rows * N * K
    print(json.dumps({"role": "all-gather forwarder", "shape": [2 * rows, N, K], "plain_ms": t_plain * 1e3,
                      "with_role_ms": t_fwd * 1e3, "tflops_with_role": fl / t_fwd / 1e12, "rows_forwarded_intact": ok,
                      "back_to_back_plain_ms": b_plain * 1e3, "back_to_back_with_role_ms": b_fwd * 1e3}))
    # scatter (vision QKV shapes)
    C, sp, T = 1280, 2, a.tokens
    W = C // sp
    h = torch.randn(T, C, device=dev, dtype=torch.bfloat16)
    wq = torch.randn(3 * C, C, device=dev, dtype=torch.bfloat16) * 0.02
    dst = [torch.empty(2 * T, 3 * W, device=dev, dtype=torch.bfloat16) for _ in range(sp)]
    row_map = torch.arange(T, device=dev, dtype=torch.int32)
    sflags = torch.zeros(8, device=dev, dtype=torch.int32)
    dummy = torch.empty(8, 3 * C, device=dev, dtype=torch.bfloat16)
    qkv = torch.empty(T, 3 * C, device=dev, dtype=torch.bfloat16)

    def scatter():
        c = GemmCommC()
        c.rs_rows, c.rs_self, c.rs_ranks, c.rs_epoch, c.rs_counter = 0, 0, sp, 1, counter.data_ptr()
        for i in range(sp):
            c.rs_base[i], c.rs_flag[i] = dst[i].data_ptr(), sflags.data_ptr()
        c.sc_row, c.sc_part, c.sc_w, c.sc_ld, c.sc_rows_dst = row_map.data_ptr(), C, W, 3 * W, 2 * T
        nv.lib().mmt_gemm_set_comm(ctypes.byref(c))
        F.gemm(h, wq, out=dummy)

    t_plain = timed(lambda: F.gemm(h, wq, out=qkv), a.iters, a.warmup, not a.no_flush)
    t_sc = timed(scatter, a.iters, a.warmup, not a.no_flush)
    b_plain, b_sc = back_to_back(lambda: F.gemm(h, wq, out=qkv)), back_to_back(scatter)
    ref = qkv.view(T, 3, sp, W)
    ok = all(bool(torch.equal(dst[g][:T], ref[:, :, g, :].reshape(T, 3 * W))) for g in range(sp))
    print(json.dumps({"role": "column scatter (Ulysses QKV epilogue)", "shape": [T, 3 * C, C], "plain_ms": t_plain * 1e3,
                      "with_role_ms": t_sc * 1e3, "scattered_equals_plain": ok, "back_to_back_plain_ms": b_plain * 1e3,
                      "back_to_back_with_role_ms": b_sc * 1e3}))
    # K-slice consumer (vision output projection)
    a_tok = torch.randn(T, C, device=dev, dtype=torch.bfloat16)
    wo = torch.randn(C, C, device=dev, dtype=torch.bfloat16) * 0.02
    y = torch.empty(T, C, device=dev, dtype=torch.bfloat16)

    def k_slices():
        c = GemmCommC()
        c.rs_rows = 0
        c.kf_flags, c.kf_epoch, c.kf_w, c.kf_self, c.kf_ranks = flags.data_ptr(), 1, W, a.self_rank % sp, sp
        nv.lib().mmt_gemm_set_comm(ctypes.byref(c))
        F.gemm(a_tok, wo, out=y)

    t_plain = timed(lambda: F.gemm(a_tok, wo, out=y), a.iters, a.warmup, not a.no_flush)
    t_kf = timed(k_slices, a.iters, a.warmup, not a.no_flush)
    b_plain, b_kf = back_to_back(lambda: F.gemm(a_tok, wo, out=y)), back_to_back(k_slices)
    print(json.dumps({"role": "K-slice consumer (Ulysses output projection)", "shape": [T, C, C],
                      "plain_ms": t_plain * 1e3, "with_role_ms": t_kf * 1e3, "back_to_back_plain_ms": b_plain * 1e3,
                      "back_to_back_with_role_ms": b_kf * 1e3}))
    code = nv.get_error()
    if code[0]:
        print(json.dumps({"device_error": code}))
        return 1
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["gemm_shapes", "gemm_roles", "gemm", "attention", "attention_bwd", "rmsnorm", "rmsnorm_bwd", "rope", "swiglu",
                                      "adamw", "ce"])
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--layout", default="kk", choices=["kk", "k_mn", "mn_mn"])
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--seq", type=int, default=0, help="sequence length inside the packed tokens (0 = one sequence)")
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--kv-heads", type=int, default=0)
    ap.add_argument("--dim", type=int, default=80)
    ap.add_argument("--causal", action="store_true")
    ap.add_argument("--rows", type=int, default=65536)
    ap.add_argument("--cols", type=int, default=3584)
    ap.add_argument("--elems", type=int, default=1 << 28)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-flush", action="store_true")
    ap.add_argument("--stream-k", type=int, default=-1, help="GEMM: 1 = stream-K for partial last waves, 0 = off (default)")
    ap.add_argument("--pair", type=int, default=-1, help="GEMM: 1 = 2-CTA kernel, 0 = 1-CTA kernels, -1 = default")
    ap.add_argument("--self-rank", type=int, default=1, help="gemm_roles: rank that the K-slice consumer plays")
    ap.add_argument("--sustain", type=float, default=0.5, help="gemm_shapes: seconds of back-to-back launches per case")
    a = ap.parse_args(argv)
    dev = "cuda"
    nv.lib()
    flush = not a.no_flush
    if a.kernel == "gemm_shapes":
        if a.pair >= 0:
            nv.lib().mmt_gemm_use_pair(a.pair)
        rc = gemm_shapes(a)
        code = nv.get_error()
        if code[0]:
            print(json.dumps({"device_error": code}))
            return 1
        return rc
    if a.kernel == "gemm_roles":
        return gemm_roles(a)
    if a.kernel == "gemm":
        if a.pair >= 0:
            nv.lib().mmt_gemm_use_pair(a.pair)
        if a.stream_k >= 0:
            nv.lib().mmt_gemm_set_stream_k(a.stream_k)
        a_mn, b_mn = a.layout == "mn_mn", a.layout != "kk"
        A = torch.randn((a.k, a.m) if a_mn else (a.m, a.k), device=dev, dtype=torch.bfloat16)
        B = torch.randn((a.k, a.n) if b_mn else (a.n, a.k), device=dev, dtype=torch.bfloat16)
        C = torch.empty(a.m, a.n, device=dev, dtype=torch.bfloat16)
        t = timed(lambda: F.gemm(A, B, a_mn=a_mn, b_mn=b_mn, out=C), a.iters, a.warmup, flush)
        report("gemm_bf16_tcgen05", t, flops=2.0 * a.m * a.n * a.k, bytes_=2.0 * (a.m * a.k + a.n * a.k + a.m * a.n),
               shape=[a.m, a.n, a.k], layout=a.layout)
    elif a.kernel in ("attention", "attention_bwd"):
        nkv = a.kv_heads or a.heads
        seq = a.seq or a.tokens
        cu = list(range(0, a.tokens + 1, seq))
        if cu[-1] != a.tokens:
            cu.append(a.tokens)
        info = SeqInfo.from_list(cu, dev)
        qkv = torch.randn(a.tokens, (a.heads + 2 * nkv) * a.dim, device=dev, dtype=torch.bfloat16,
                          requires_grad=a.kernel == "attention_bwd")
        fl = sum(4.0 * (y - x) ** 2 * a.dim * a.heads * (0.5 if a.causal else 1.0) for x, y in zip(cu, cu[1:]))
        if a.kernel == "attention":
            with torch.no_grad():
                t = timed(lambda: F.attention(qkv, a.heads, nkv, a.dim, info, causal=a.causal), a.iters, a.warmup,
                          flush)
            report("attn_fwd", t, flops=fl, tokens=a.tokens, seq=seq, heads=[a.heads, nkv], dim=a.dim,
                   causal=a.causal)
        else:
            out = F.attention(qkv, a.heads, nkv, a.dim, info, causal=a.causal)
            do = torch.randn_like(out)

            def bwd():
                qkv.grad = None
                out.backward(do, retain_graph=True)

            t = timed(bwd, a.iters, a.warmup, flush)
            report("attn_bwd(delta+dkdv+dq)", t, flops=3.5 * fl, tokens=a.tokens, seq=seq, heads=[a.heads, nkv],
                   dim=a.dim, causal=a.causal, note="3.5x forward flops: the two-kernel backward recomputes S and dP twice")
    elif a.kernel == "rmsnorm":
        x = torch.randn(a.rows, a.cols, device=dev, dtype=torch.bfloat16)
        w = torch.ones(a.cols, device=dev, dtype=torch.bfloat16)
        with torch.no_grad():
            t = timed(lambda: F.rmsnorm(x, w), a.iters, a.warmup, flush)
        report("rmsnorm_fwd", t, bytes_=4.0 * a.rows * a.cols, shape=[a.rows, a.cols])
    elif a.kernel == "rmsnorm_bwd":
        from ..ops import blocks
        x = torch.randn(a.rows, a.cols, device=dev, dtype=torch.bfloat16)
        dy, extra = torch.randn_like(x), torch.randn_like(x)
        w = torch.ones(a.cols, device=dev, dtype=torch.bfloat16)
        _, rstd = blocks._rmsnorm_fwd(x, w, 1e-6)
        t = timed(lambda: blocks._rmsnorm_bwd(dy, x, w, rstd, extra), a.iters, a.warmup, flush)
        report("rmsnorm_bwd(+residual gradient, dw)", t, bytes_=8.0 * a.rows * a.cols, shape=[a.rows, a.cols])
    elif a.kernel == "rope":
        width = a.heads * a.dim
        x = torch.randn(a.rows, width, device=dev, dtype=torch.bfloat16)
        ang = torch.rand(a.rows, a.dim // 2, device=dev) * 6.28
        ang = torch.cat([ang, ang], -1)
        cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
        from ..ops import blocks
        t = timed(lambda: blocks._rope_(x, cos, sin, a.heads, a.dim, False), a.iters, a.warmup, flush)
        report("rope (in place)", t, bytes_=4.0 * a.rows * width + 8.0 * a.rows * a.dim, shape=[a.rows, a.heads, a.dim])
    elif a.kernel == "swiglu":
        gu = torch.randn(a.rows, 2 * a.cols, device=dev, dtype=torch.bfloat16)
        with torch.no_grad():
            t = timed(lambda: F.swiglu(gu), a.iters, a.warmup, flush)
        report("swiglu_fwd", t, bytes_=6.0 * a.rows * a.cols, shape=[a.rows, a.cols])
    elif a.kernel == "adamw":
        n = a.elems // 8 * 8
        p = torch.randn(n, device=dev, dtype=torch.bfloat16)
        g = torch.randn(n, device=dev, dtype=torch.bfloat16)
        master, m, v = p.float(), torch.zeros(n, device=dev), torch.zeros(n, device=dev)
        t = timed(lambda: F.adamw_step(p, g, master, m, v, n_decay=n, lr=1e-4, beta1=0.9, beta2=0.999, eps=1e-8,
                                       weight_decay=0.01, step=1), a.iters, a.warmup, flush)
        report("adamw", t, bytes_=28.0 * n, elems=n)
    elif a.kernel == "ce":
        T, V, H = a.rows, a.cols, a.k
        h = torch.randn(T, H, device=dev, dtype=torch.bfloat16, requires_grad=True)
        w = (torch.randn(V, H, device=dev, dtype=torch.bfloat16) * 0.02).requires_grad_()
        labels = torch.randint(0, V, (T,), device=dev)
        t = timed(lambda: F.lm_head_cross_entropy(h, w, labels), a.iters, a.warmup, flush)
        report("lm_head+ce fwd+bwd", t, flops=6.0 * T * V * H, shape=[T, V, H])
    code = nv.get_error()
    if code[0]:
        print(json.dumps({"device_error": code}))
        return 1
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
