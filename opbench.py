"""Per-operator micro-benchmarks (the method of the reference's
bench/gemm_bench.cc:7-16,102-124 and bench/jax_bench.py: back-to-back launches
cycling through distinct weight buffers so nothing stays in L2; CUDA-event
time; JSON lines).  Also the small cases the ncu summaries under profiles/ come from.

    python opbench.py qmm  --bits 4 --m 1 --n 4096 --k 4096 [--buffers 32] [--reps 5]
    python opbench.py gemm --m 2048 --n 4096 --k 4096 [--act 3] [--bias]
    python opbench.py rows --kind softmax --rows 8192 --n 1024 [--dtype f32]
    python opbench.py sweep          # the benchmark configs 2-4
    python opbench.py umma           # SM cycles per tcgen05.mma by shape
"""
import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
from __graft_entry__ import load_package  # noqa: E402

HBM_NOMINAL = 8000.0
BF16_NOMINAL = 2250.0


def peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    except Exception:
        return 6650.0, 1590.0, "fallback"


def timed(fn, reps, warmup=3, graph=True):
    """Seconds per call of fn.  With graph=True the launches of one call are
    captured into a CUDA graph first, so the figure is device time, not the
    host's launch rate."""
    import torch
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if graph:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn()
        eager, fn = fn, g.replay
        fn()
        torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) * 1e-3 / reps


def bench_qmm(pkg, bits, m, n, k, buffers, reps, group=64, fuse=""):
    import torch
    dev = "cuda"
    ws = []
    for i in range(buffers):
        if bits == 4:
            ws.append({"q4": torch.randint(-2**31, 2**31 - 1, (n, k // 8), dtype=torch.int32, device=dev),
                       "s": torch.full((n, k // 64), 0.008, dtype=torch.bfloat16, device=dev),
                       "b": torch.full((n, k // 64), -0.06, dtype=torch.bfloat16, device=dev)})
        elif bits == 8:
            g = k if group == 0 else group
            ws.append({"q": torch.randint(-127, 128, (n, k), dtype=torch.int8, device=dev),
                       "s": torch.full((n, k // g), 0.001, dtype=torch.bfloat16, device=dev)})
        else:
            ws.append(torch.randn((n, k), device=dev).mul_(0.02).to(torch.bfloat16))
    x = torch.randn((m, 2 * k if fuse == "silu" else k), device=dev).to(torch.bfloat16)
    gain = torch.ones((k,), device=dev, dtype=torch.bfloat16) if fuse == "rms" else None
    res = torch.zeros((m, n), device=dev, dtype=torch.bfloat16) if fuse in ("res", "silu") else None

    def run():
        for w in ws:
            pkg.qwen3.linear(x, w, rms_gain=gain, silu_mul=fuse == "silu", residual=res)
    sec = timed(run, reps) / buffers
    if bits == 4:
        nbytes = n * k * 0.5625
    elif bits == 8:
        nbytes = n * k + 2 * n * (k // (k if group == 0 else group))
    else:
        nbytes = n * k * 2
    nbytes += 2 * m * (k + n)
    hbm, _, kind = peaks()
    gbs = nbytes / sec / 1e9
    plan = pkg.qwen3.qmm_plan(m, n, k, bits, 64 if bits == 4 else (k if group == 0 else group))
    return {"op": "qmm", "bits": bits, "m": m, "n": n, "k": k, "buffers": buffers, "us": sec * 1e6,
            "algorithmic_bytes": nbytes, "gbs": gbs, f"frac_of_{kind}": gbs / hbm, "frac_of_nominal": gbs / HBM_NOMINAL,
            "rows_per_cta": plan[0], "split_k": plan[1]}


def bench_gemm(pkg, m, n, k, act, bias, reps, dtype="bf16", transpose_b=False, buffers=4, route=0):
    import torch
    dt = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}[dtype]
    dev = "cuda"
    As = [torch.randn((m, k), device=dev).to(dt) for _ in range(buffers)]
    Bs = [torch.randn((n, k) if transpose_b else (k, n), device=dev).mul_(0.02).to(dt) for _ in range(buffers)]
    bias_t = torch.randn((n,), device=dev).mul_(0.01).to(dt) if bias else None

    B = pkg.blas
    outs = [torch.empty((m, n), dtype=dt, device=dev) for _ in range(buffers)]
    prms = [B.GemmParams(m, n, k, B.Operand(a, k), B.Operand(b, b.stride(0), transpose=transpose_b), B.Operand(o, n))
            for a, b, o in zip(As, Bs, outs)]
    epi = B.SteelEpilogue(act, bias_t)

    def run():
        for prm in prms:
            B.run_steel_gemm(prm, epi, route=route)
    sec = timed(run, reps) / buffers
    es = 4 if dtype == "f32" else 2
    flops = 2.0 * m * n * k
    nbytes = es * (m * k + k * n + m * n) + (es * n if bias else 0)
    hbm, tf, kind = peaks()
    route = route or B.gemm_route(prms[0], epi)
    return {"op": "gemm", "dtype": dtype, "m": m, "n": n, "k": k, "act": act, "bias": bool(bias), "route": route,
            "us": sec * 1e6, "tflops": flops / sec / 1e12, f"frac_of_{kind}_tensor": flops / sec / 1e12 / tf,
            "frac_of_nominal_tensor": flops / sec / 1e12 / BF16_NOMINAL, "gbs": nbytes / sec / 1e9,
            f"frac_of_{kind}_hbm": nbytes / sec / 1e9 / hbm}


def bench_rows(pkg, kind, rows, n, dtype, reps, buffers=4):
    import torch
    dt = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}[dtype]
    xs = [torch.randn((rows, n), device="cuda").mul_(3.0).to(dt) for _ in range(buffers)]
    ys = [torch.empty_like(x) for x in xs]
    gain = torch.ones((n,), device="cuda").to(dt)
    code = {"rms": 0, "softmax": 1, "log_softmax": 2, "layernorm": 3}[kind]

    def run():
        for x, y in zip(xs, ys):
            pkg.rows.rownorm(code, x, gain=gain if code in (0, 3) else None, eps=1e-6, out=y)
    sec = timed(run, reps) / buffers
    nbytes = 2 * rows * n * xs[0].element_size()
    hbm, _, k = peaks()
    return {"op": "rows", "kind": kind, "rows": rows, "n": n, "dtype": dtype, "us": sec * 1e6,
            "gbs": nbytes / sec / 1e9, f"frac_of_{k}": nbytes / sec / 1e9 / hbm}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("op", choices=["qmm", "gemm", "rows", "sweep", "umma"])
    ap.add_argument("--bits", type=int, default=4)
    ap.add_argument("--group", type=int, default=64, help="int8: 64, or 0 for per-channel")
    ap.add_argument("--m", type=int, default=1)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--buffers", type=int, default=32)
    ap.add_argument("--reps", type=int, default=5)
    ap.add_argument("--act", type=int, default=0)
    ap.add_argument("--bias", action="store_true")
    ap.add_argument("--tb", action="store_true")
    ap.add_argument("--fuse", default="", choices=["", "rms", "silu", "res"],
                    help="qmm: fused RMSNorm prologue / silu(gate)*up prologue + residual / residual epilogue")
    ap.add_argument("--route", type=int, default=0, help="gemm: force a route (1 tcgen05, 2 few-row, 3 SIMT); 0 = the library's choice")
    ap.add_argument("--dtype", default="bf16")
    ap.add_argument("--kind", default="softmax")
    ap.add_argument("--rows", type=int, default=8192)
    a = ap.parse_args()
    pkg = load_package()
    if a.op == "qmm":
        print(json.dumps(bench_qmm(pkg, a.bits, a.m, a.n, a.k, a.buffers, a.reps, a.group, a.fuse)), flush=True)
    elif a.op == "gemm":
        print(json.dumps(bench_gemm(pkg, a.m, a.n, a.k, a.act, a.bias, a.reps, a.dtype, a.tb,
                                    max(4, min(a.buffers, int(512e6 // (a.n * a.k * 2)))), a.route)), flush=True)
    elif a.op == "umma":
        # SM cycles per tcgen05.mma by shape (b200_probe_umma_rate): 256 instructions from one thread
        import torch
        from metal_pjrt_plugin_b200 import _lib
        ctx = pkg.default_context()
        out = torch.zeros(2, dtype=torch.int64, device="cuda")
        for kind, m, n, at, nd in [(0, 128, 16, 1, 1), (0, 128, 16, 1, 8), (0, 128, 16, 0, 8), (0, 128, 64, 1, 1), (0, 128, 256, 1, 1),
                                   (0, 128, 256, 0, 1), (0, 64, 8, 1, 8), (0, 64, 16, 0, 8), (1, 128, 16, 1, 8), (1, 128, 16, 0, 8),
                                   (1, 128, 256, 0, 1), (1, 64, 8, 0, 8)]:
            for _ in range(2):
                _lib.check(pkg.lib().b200_probe_umma_rate(ctx.handle, _lib.current_stream(), kind, m, n, at, nd, 256, out.data_ptr()))
            torch.cuda.synchronize()
            issue, done = (int(v) for v in out.tolist())
            print(json.dumps({"op": "umma", "kind": "f8f6f4" if kind == 0 else "f16", "m": m, "n": n,
                              "a": "tmem" if at else "smem", "accumulators": nd, "cycles_per_mma_issue": issue / 256,
                              "cycles_per_mma_complete": done / 256}), flush=True)
    elif a.op == "rows":
        print(json.dumps(bench_rows(pkg, a.kind, a.rows, a.n, a.dtype, a.reps)), flush=True)
    else:
        shapes = [(4096, 4096), (4096, 1024), (4096, 12288), (12288, 4096)]
        for bits in (4, 8):
            for (k, n) in shapes:
                for m in (1, 8, 32):
                    buffers = max(8, int(512e6 // (n * k * bits / 8)))
                    print(json.dumps(bench_qmm(pkg, bits, m, n, k, min(buffers, 64), 3, 64 if bits == 4 else 0)), flush=True)
        for m in (1, 16, 128, 2048, 8192):
            print(json.dumps(bench_gemm(pkg, m, 4096, 4096, 3, True, 3)), flush=True)
        for kind, rows, n, dt in [("softmax", 8192, 1024, "f32"), ("layernorm", 8192, 1024, "f32"),
                                  ("rms", 8192, 4096, "bf16"), ("softmax", 1024, 2048, "f32"), ("rms", 32, 4096, "bf16")]:
            print(json.dumps(bench_rows(pkg, kind, rows, n, dt, 5)), flush=True)


if __name__ == "__main__":
    main()
