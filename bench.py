"""Benchmark of the FP8 transformer inference path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload cfg5|cfg4]

A step is one greedy decode step of the whole batch (benchmark config 5: 8B-shape decoder,
FP8 linears, batch 128, prompt 2048; config 4: 1.1B shape, batch 64, prompt 512).  The KV
cache is filled by a real prefill before the timed region.  Rank 0 prints ONE JSON line:
tokens/s device-timed over K CUDA-graph replays (`value`), the same through the host-facing
step API with pinned host token buffers (`e2e`), the roofline of the dominant kernel (decode
attention with RoPE and the cache append fused in, plus its merge pass: the step's 32 launch pairs
captured as a graph of their own and timed with CUDA events), the CPU oracle timed on a bounded
sample (`cpu_baseline`), SM clocks sampled during the timed region, and per-kernel figures
(`kernels`): quantize and FP8 GEMM of config 1 and 8192^3 with the cuBLASLt time of the same problems
beside them, the four decode-size GEMMs of a config 5 layer, decode attention of config 3 in both
cache layouts, and the block prefill of config 2.
With N > 1 (torchrun) the model is tensor-parallel over N GPUs: strong scaling; the line then
also carries `parity`, the first block's output on the sharded model against the unsharded one.
`config` is the same in both arms; what only describes how this arm ran sits under `run`.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    "cfg5": dict(name="cfg5: 8B-shape decoder LLM, FP8 linears, greedy decode", layers=32, hidden=4096, q_heads=32,
                 kv_heads=8, head_dim=128, ffn=14336, vocab=128256, theta=500000.0, batch=128, prompt=2048, tied=False,
                 prefill_chunk=8),
    "cfg4": dict(name="cfg4: 1.1B-shape decoder LLM, FP8 linears, greedy decode", layers=22, hidden=2048, q_heads=32,
                 kv_heads=4, head_dim=64, ffn=5632, vocab=32000, theta=10000.0, batch=64, prompt=512, tied=True,
                 prefill_chunk=16),
}


def measured_peaks() -> tuple[float, str]:
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:  # noqa: BLE001
        return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks / throttle reasons every 200 ms while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.rows: list[list[str]] = []
        self.proc = None
        self.gpu = gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "200"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:  # noqa: BLE001
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        sm = sorted(float(r[0]) for r in self.rows if r and r[0].replace(".", "").isdigit())
        mx = [float(r[1]) for r in self.rows if len(r) > 1 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 3 + i and r[3 + i] == "Active" for r in self.rows)]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx[0] if mx else None, "reasons": reasons,
                "samples": len(sm)}


# ---------------------------------------------------------------------------------------
# CPU oracle arm


def oracle_decode_sample(w: dict, seconds_limit: float, steps: int, warmup: int):
    """Times the CPU oracle (the reference's algorithm restated in NumPy) on a bounded sample of
    the decode workload: ONE transformer layer of the workload's shape plus the lm_head, ONE
    sequence, at the workload's context (the prompt length); a full step of one sequence is
    extrapolated as layers * t_layer + t_head."""
    import numpy as np

    from oracle import llm as ollm

    cfg = ollm.LLMConfig(vocab_size=w["vocab"], embed_dim=w["hidden"], q_heads=w["q_heads"], kv_heads=w["kv_heads"],
                         head_dim=w["head_dim"], num_layers=1, mlp_hidden_dim=w["ffn"], rope_theta=w["theta"],
                         rms_eps=1e-5)
    rng = np.random.default_rng(0)
    om = ollm.LLM.build(cfg, rng, use_fp8=True, tie=w["tied"])
    ctx = w["prompt"]
    caches = om.init_cache(ctx + warmup + steps + 1)
    # the cache of the sample sequence: seeded N(0,1) rows stand in for a prefill (untimed either way)
    c0 = caches[0]["self_attn"]
    c0["k"][:ctx] = rng.standard_normal((ctx,) + c0["k"].shape[1:], dtype=np.float32).astype(c0["k"].dtype)
    c0["v"][:ctx] = rng.standard_normal((ctx,) + c0["v"].shape[1:], dtype=np.float32).astype(c0["v"].dtype)
    c0["position"] = np.int32(ctx)
    caches = [caches[0]]
    t_layer, t_head = [], []
    t_start = time.perf_counter()
    tok = np.array([1], np.int32)
    done = 0
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        x = om.embed_tokens(tok)
        x, c = om.blocks[0].forward(x, cache=caches[0])
        caches = [c]
        t1 = time.perf_counter()
        logits = om.get_logits(om.norm(x))
        tok = np.array([ollm.greedy_token(logits[-1])], np.int32)
        t2 = time.perf_counter()
        if i >= warmup:
            t_layer.append(t1 - t0)
            t_head.append(t2 - t1)
            done += 1
        if time.perf_counter() - t_start > seconds_limit and done >= 1:
            break
    tl, th = float(np.median(t_layer)), float(np.median(t_head))
    step_s = w["layers"] * tl + th  # one sequence
    return {"tokens_per_s": 1.0 / step_s, "step_s_one_sequence": step_s, "steps_timed": done,
            "sample": f"NumPy oracle, 1 of {w['layers']} layers + lm_head, 1 of {w['batch']} sequences, context {ctx}; "
                      f"step time extrapolated as {w['layers']}*t_layer+t_head; "
                      f"{done} steps timed; the reference re-quantises every weight on every call and so does this"}


def host_threads() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except Exception:  # noqa: BLE001
        return os.cpu_count() or 1


# ---------------------------------------------------------------------------------------
# per-kernel figures (benchmark configs 1 and 3)


def _time_kernel(fn, iters=20, warm=3, flush=None):
    """Average device time of fn(i).  Before every timed call a 512 MiB buffer is rewritten and then
    read back (two torch kernels): the write evicts the operands from the 126 MB L2, the read
    drains the dirty lines the write left behind (their write-back would otherwise be billed to
    the kernel), and both keep the GPU busy long enough for the host to enqueue the timed launch,
    so the two events bracket device time only."""
    import torch

    for i in range(warm):
        fn(i)
    total = 0.0
    for i in range(iters):
        if flush is not None:
            flush.zero_()
            flush.max()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn(i)
        e1.record()
        e1.synchronize()
        total += e0.elapsed_time(e1)
    return total / iters * 1e-3


def kernel_figures(peak_gbs: float, only: str | None = None) -> dict:
    """cfg1: quantize (HBM) and FP8 GEMM (tensor); cfg3: decode attention (HBM); cfg2: block prefill.  L2 is
    flushed (a 512 MiB buffer is rewritten and read back) between timed launches.  ``only`` keeps the
    groups whose name contains it ("quantize", "gemm", "attn_decode", "block_prefill"): what a profiler run
    of one kernel uses."""
    import numpy as np
    import torch

    from xax_b200 import ops

    dev = "cuda"
    out = {}
    flush = torch.empty(512 << 20, dtype=torch.uint8, device=dev)
    if only is not None:
        if "block_prefill".find(only) >= 0 or only.find("block_prefill") >= 0:
            return {"block_prefill_cfg2": block_prefill_figure(flush)}
        return _kernel_group(only, peak_gbs, flush)
    out.update(_kernel_group("quantize", peak_gbs, flush))
    out.update(_kernel_group("gemm", peak_gbs, flush))
    out.update(_kernel_group("attn_decode", peak_gbs, flush))
    out["block_prefill_cfg2"] = block_prefill_figure(flush)
    return out


def _kernel_group(group: str, peak_gbs: float, flush) -> dict:
    import numpy as np
    import torch

    from xax_b200 import ops

    dev = "cuda"
    out = {}
    if group not in ("quantize", "gemm", "attn_decode", "attn_decode_small", "gemm_8192_1cta"):
        raise SystemExit(f"unknown kernel group {group!r}: quantize, gemm, attn_decode, block_prefill, or the small "
                         "cases for profiler captures attn_decode_small, gemm_8192_1cta")
    g = torch.Generator(device=dev).manual_seed(0)
    if group == "attn_decode_small":
        return _attn_decode_small(g, peak_gbs, flush)
    if group == "gemm_8192_1cta":
        return _gemm_8192_single_cta(g, flush)
    # ---- cfg1: x[2048,2048] bf16 N(0,1) with 0.1 % x20 outliers, W (8192,2048) N(0,0.02^2)
    M, K, N = 2048, 2048, 8192
    x = torch.randn((M, K), generator=g, device=dev)
    x = torch.where(torch.rand((M, K), generator=g, device=dev) < 1e-3, x * 20, x).to(torch.bfloat16)
    w = (torch.randn((N, K), generator=g, device=dev) * 0.02).to(torch.bfloat16)
    bias = (torch.randn((N,), generator=g, device=dev) * 0.01).to(torch.bfloat16)
    scale = torch.tensor(448.0 / 100.0, device=dev)
    hist = torch.zeros(16, device=dev)
    if group == "quantize":
        return _quantize_figures(x, scale, hist, peak_gbs, flush)
    if group == "attn_decode":
        return _attn_decode_figures(g, peak_gbs, flush)
    return _gemm_figures(x, w, bias, scale, hist, g, flush)


def _quantize_figures(x, scale, hist, peak_gbs, flush) -> dict:
    import torch

    from xax_b200 import ops

    out = {}
    M, K = x.shape
    dev = x.device
    g = torch.Generator(device=dev).manual_seed(3)
    t = _time_kernel(lambda i: ops.quantize_delayed(x, scale, hist), flush=flush)
    out["quantize_cfg1"] = {"gbs": M * K * 3 / t / 1e9, "frac_of_hbm_peak": M * K * 3 / t / 1e9 / peak_gbs,
                            "us": t * 1e6, "bytes": M * K * 3}
    xl = torch.randn((8192, 8192), generator=g, device=dev).to(torch.bfloat16)
    t = _time_kernel(lambda i: ops.quantize_delayed(xl, scale, hist), iters=10, flush=flush)
    out["quantize_8192x8192"] = {"gbs": 8192 * 8192 * 3 / t / 1e9, "frac_of_hbm_peak": 8192 * 8192 * 3 / t / 1e9 / peak_gbs,
                                 "us": t * 1e6, "bytes": 8192 * 8192 * 3}
    del xl
    return out


def _gemm_figures(x, w, bias, scale, hist, g, flush) -> dict:
    import torch

    from xax_b200 import ops

    out = {}
    dev = x.device
    M, K = x.shape
    N = w.shape[0]
    xq, _, _, x_inv = ops.quantize_delayed(x, scale, hist)
    wq, _, w_inv, _ = ops.quantize_current(w, N)
    o = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
    t = _time_kernel(lambda i: ops.gemm_fp8(xq, wq, x_inv, w_inv[:1], bias, out=o), flush=flush)
    out["gemm_fp8_cfg1"] = {"tflops": 2.0 * M * N * K / t / 1e12, "us": t * 1e6,
                            "frac_of_4500_nominal": 2.0 * M * N * K / t / 4.5e15}
    # Yardstick on the same box, bench side only (never on the product path): the vendor library's FP8
    # GEMM (cuBLASLt through torch._scaled_mm) on the same operands, per-tensor scales, bias, bf16 out.
    one = torch.ones((), device=dev)
    try:
        t = _time_kernel(lambda i: torch._scaled_mm(xq, wq.t(), scale_a=one, scale_b=one, bias=bias,
                                                    out_dtype=torch.bfloat16), flush=flush)
        out["cublaslt_fp8_cfg1"] = {"tflops": 2.0 * M * N * K / t / 1e12, "us": t * 1e6}
    except Exception as e:  # noqa: BLE001
        out["cublaslt_fp8_cfg1"] = {"error": repr(e)[:200]}
    M2 = N2 = K2 = 8192
    a8 = (torch.randn((M2, K2), generator=g, device=dev)).to(torch.float8_e4m3fn)
    b8 = (torch.randn((N2, K2), generator=g, device=dev)).to(torch.float8_e4m3fn)
    o2 = torch.empty((M2, N2), dtype=torch.bfloat16, device=dev)
    t = _time_kernel(lambda i: ops.gemm_fp8(a8, b8, None, None, None, out=o2), iters=10, flush=flush)
    out["gemm_fp8_8192"] = {"tflops": 2.0 * M2 * N2 * K2 / t / 1e12, "us": t * 1e6,
                            "frac_of_4500_nominal": 2.0 * M2 * N2 * K2 / t / 4.5e15}
    try:
        t = _time_kernel(lambda i: torch._scaled_mm(a8, b8.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16),
                         iters=10, flush=flush)
        out["cublaslt_fp8_8192"] = {"tflops": 2.0 * M2 * N2 * K2 / t / 1e12, "us": t * 1e6}
    except Exception as e:  # noqa: BLE001
        out["cublaslt_fp8_8192"] = {"error": repr(e)[:200]}
    del a8, b8, o2
    out["gemm_fp8_decode_cfg5_layer"] = _decode_gemm_figures(g, flush)
    return out


def _decode_gemm_figures(g, flush) -> dict:
    """The four FP8 GEMMs of one cfg5 layer at decode size (M = 128 token rows): fused q|k|v, out-proj,
    gate|up, down.  Each shape is timed as a CUDA graph of eight launches on eight different weight
    matrices (so the weights stream from HBM, as in the model, and launch gaps are the device's own);
    the figure is weight bytes / time against the measured copy bandwidth."""
    import torch

    from xax_b200 import ops

    peak, _ = measured_peaks()
    M, reps = 128, 8
    shapes = (("qkv", 6144, 4096), ("out", 4096, 4096), ("gate_up", 28672, 4096), ("down", 4096, 14336))
    res, total_us, total_bytes = {}, 0.0, 0
    for name, N, K in shapes:
        a = torch.randn((M, K), generator=g, device="cuda").to(torch.float8_e4m3fn)
        ws = [torch.randn((N, K), generator=g, device="cuda").to(torch.float8_e4m3fn) for _ in range(reps)]
        rm = torch.ones(M, device="cuda")
        cm = torch.ones(1, device="cuda")
        o = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")

        def chain():
            for w_ in ws:
                ops.gemm_fp8(a, w_, rm, cm, None, None, out=o)

        chain()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            chain()
        t = _time_kernel(lambda i: graph.replay(), iters=5, warm=1, flush=flush) / reps
        res[name] = {"us": t * 1e6, "gbs": N * K / t / 1e9, "frac_of_hbm_peak": N * K / t / 1e9 / peak}
        total_us += t * 1e6
        total_bytes += N * K
        del ws
    res["layer"] = {"us": total_us, "gbs": total_bytes / total_us / 1e3, "frac_of_hbm_peak": total_bytes / total_us / 1e3 / peak,
                    "weight_bytes": total_bytes}
    return res


def _attn_decode_figures(g, peak_gbs, flush) -> dict:
    import numpy as np
    import torch

    from xax_b200 import ops

    out = {}
    dev = "cuda"
    # ---- cfg3: B=32, 32q/8kv x 128, lengths U[512, 8192], theta 5e5
    B, Hq, Hkv, D, max_len = 32, 32, 8, 128, 8192
    lens = torch.from_numpy(np.random.default_rng(0).integers(512, 8193, B).astype(np.int32)).to(dev)
    kc = torch.randn((B, max_len, Hkv, D), generator=g, device=dev, dtype=torch.bfloat16)
    vc = torch.randn((B, max_len, Hkv, D), generator=g, device=dev, dtype=torch.bfloat16)
    q = torch.randn((B, Hq, D), generator=g, device=dev, dtype=torch.bfloat16)
    pos = lens - 1
    ws = ops.attn_decode_workspace(B, Hq, D, max_len, dev)
    ao = torch.empty_like(q)
    cos, sin = ops.rope_tables(D, 500000.0, max_len, dev)
    nbytes = int(lens.sum().item()) * (2 * Hkv * D * 2) + 2 * B * Hq * D * 2
    t = _time_kernel(lambda i: ops.attn_decode(q, kc, vc, pos, workspace=ws, out=ao), flush=flush)
    out["attn_decode_cfg3"] = {"gbs": nbytes / t / 1e9, "frac_of_hbm_peak": nbytes / t / 1e9 / peak_gbs, "us": t * 1e6,
                               "bytes": nbytes}
    t = _time_kernel(lambda i: ops.attn_decode(q, kc, vc, pos, workspace=ws, out=ao, k_is_rotated=False, cos=cos,
                                               sin=sin), flush=flush)
    out["attn_decode_cfg3_rope_on_load"] = {"gbs": nbytes / t / 1e9, "frac_of_hbm_peak": nbytes / t / 1e9 / peak_gbs,
                                            "us": t * 1e6}
    return out


def _attn_decode_small(g, peak_gbs, flush) -> dict:
    """Decode attention on a case small enough for a many-pass profiler capture and larger than L2:
    B = 32 sequences of 2053 tokens, 32 query / 8 kv heads x 128 (0.27 GB of K and V)."""
    import torch

    from xax_b200 import ops

    B, Hq, Hkv, D, L = 32, 32, 8, 128, 2053
    max_len = 2304
    kc = torch.randn((B, max_len, Hkv, D), generator=g, device="cuda", dtype=torch.bfloat16)
    vc = torch.randn((B, max_len, Hkv, D), generator=g, device="cuda", dtype=torch.bfloat16)
    q = torch.randn((B, Hq, D), generator=g, device="cuda", dtype=torch.bfloat16)
    pos = torch.full((B,), L - 1, dtype=torch.int32, device="cuda")
    ws = ops.attn_decode_workspace(B, Hq, D, max_len, "cuda")
    ao = torch.empty_like(q)
    nbytes = B * L * (2 * Hkv * D * 2) + 2 * B * Hq * D * 2
    t = _time_kernel(lambda i: ops.attn_decode(q, kc, vc, pos, workspace=ws, out=ao), iters=5, warm=1, flush=flush)
    return {"attn_decode_small": {"gbs": nbytes / t / 1e9, "frac_of_hbm_peak": nbytes / t / 1e9 / peak_gbs,
                                  "us": t * 1e6, "bytes": nbytes}}


def _gemm_8192_single_cta(g, flush) -> dict:
    """FP8 GEMM 8192^3 forced onto the single-CTA kernel with 256-wide tiles (the library itself picks the
    CTA-pair kernel at this size): the case the profiler summary of that kernel was captured on."""
    import torch

    from xax_b200 import _lib, ops

    n = 8192
    a8 = torch.randn((n, n), generator=g, device="cuda").to(torch.float8_e4m3fn)
    b8 = torch.randn((n, n), generator=g, device="cuda").to(torch.float8_e4m3fn)
    o = torch.empty((n, n), dtype=torch.bfloat16, device="cuda")
    lib = _lib.load()
    lib.xaxb_gemm_force_plan(256, 0)
    try:
        t = _time_kernel(lambda i: ops.gemm_fp8(a8, b8, None, None, None, out=o), iters=5, warm=1, flush=flush)
    finally:
        lib.xaxb_gemm_force_plan(0, 0)
    return {"gemm_fp8_8192_single_cta": {"tflops": 2.0 * n ** 3 / t / 1e12, "us": t * 1e6}}


def block_prefill_figure(flush) -> dict:
    """cfg2: one pre-norm block, prefill of 4 sequences x 1024 tokens (hidden 2048, 16 query / 4 kv heads
    x 128, SwiGLU 5632, FP8 linears for QKV / out / MLP), captured in a CUDA graph so the figure is device
    time of the kernel chain.  FLOPs: the seven linears plus causal attention (half of the full square)."""
    import torch

    from xax_b200.arch.attention import TransformerBlock

    B, T, H, Hq, Hkv, D, F = 4, 1024, 2048, 16, 4, 128, 5632
    blk = TransformerBlock.build(H, Hq, F, key=0, num_kv_heads=Hkv, head_dim=D, causal=True,
                                 use_rotary_embeddings=True, rotary_base=10000.0, norm_type="rmsnorm", norm_eps=1e-5,
                                 feedforward_type="swiglu", use_fp8=True, fp8_mlp=True)
    g = torch.Generator(device="cuda").manual_seed(2)
    x = torch.randn((B * T, H), generator=g, device="cuda").to(torch.bfloat16)
    cache = blk.self_attn.init_cache(T, batch=B)
    blk.forward_tokens(x, B, T, cache=cache, advance=False)  # quantises the weights, sizes the allocator
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        blk.forward_tokens(x, B, T, cache=cache, advance=False)
    torch.cuda.current_stream().wait_stream(side)
    with torch.cuda.graph(graph):
        blk.forward_tokens(x, B, T, cache=cache, advance=False)
    t = _time_kernel(lambda i: graph.replay(), iters=10, flush=flush)
    lin = 2.0 * B * T * (H * (Hq + 2 * Hkv) * D + Hq * D * H + 3 * H * F)
    att = 4.0 * B * Hq * T * T * D / 2
    return {"us": t * 1e6, "tflops": (lin + att) / t / 1e12, "linear_gflop": lin / 1e9, "attention_gflop": att / 1e9}


# ---------------------------------------------------------------------------------------


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg5", choices=sorted(WORKLOADS))
    ap.add_argument("--no-kernels", action="store_true", help="skip the per-kernel figures")
    ap.add_argument("--kernels-only", default=None, metavar="GROUP",
                    help="only the per-kernel figures of one group (quantize, gemm, attn_decode, block_prefill, "
                         "'all', or the small profiler cases attn_decode_small / gemm_8192_1cta); prints "
                         "{\"kernels\": ...} -- the command profiler captures of one kernel run")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU oracle timing")
    ap.add_argument("--synthetic-kv", action="store_true", help="fill the KV cache with N(0,1) instead of a prefill")
    args = ap.parse_args()
    w = WORKLOADS[args.workload]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    warmup = max(args.warmup, 3)
    metric, unit = "llm_decode_tokens_per_s", "tokens/s"
    base = {"metric": metric, "unit": unit, "n_gpus": args.gpus, "steps": args.steps, "warmup": warmup,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "fp8_e4m3 (bf16 activations)",
            "data": "synthetic", "config": {"workload": w["name"], "batch": w["batch"], "prompt": w["prompt"],
                                            "layers": w["layers"], "hidden": w["hidden"],
                                            "parallelism": f"tp{args.gpus}",
                                            "l2": "inputs (weights + KV cache) far larger than L2"}}

    if args.kernels_only is not None:
        if rank == 0:
            peak, _ = measured_peaks()
            print(json.dumps({"kernels": kernel_figures(peak, None if args.kernels_only == "all" else args.kernels_only)}),
                  flush=True)
        return
    if args.impl == "reference":
        if rank != 0:
            return
        r = oracle_decode_sample(w, seconds_limit=150.0, steps=args.steps, warmup=1)
        line = dict(base)
        line.update({"impl": "reference", "value": r["tokens_per_s"], "ms_per_step": r["step_s_one_sequence"] * 1e3,
                     "dtype": "bf16/e4m3 emulated in float32 (NumPy)",
                     "cpu_baseline": {"value": r["tokens_per_s"], "unit": unit, "cores": host_threads(),
                                      "kind": "port", "sample": r["sample"]},
                     "e2e": {"value": r["tokens_per_s"], "unit": unit, "h2d_bytes_per_step": 0,
                             "d2h_bytes_per_step": 0},
                     "gpu_launches": 0})
        print(json.dumps(line), flush=True)
        return

    import torch
    import torch.distributed as dist

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    tp = None
    host_group = None
    if world > 1:
        # NCCL carries barriers, the prefill's all-reduces and a few scalars; its NVLink multicast
        # path is not needed and stays off, so that ranks may leave without tearing NCCL down.
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=dev)
        host_group = dist.new_group(backend="gloo")  # host-side barriers: a waiting rank leaves its GPU idle
        from xax_b200.parallel import TensorParallel

        tp = TensorParallel(rank, world, local_amax=os.environ.get("XAXB_TP_AMAX", "global") == "local")
    from xax_b200 import _lib, ops
    from xax_b200.arch.llm import LLM, DecodeState, LLMConfig, tie_embedding_and_head

    run_info: dict = {}

    cfg = LLMConfig(vocab_size=w["vocab"], embed_dim=w["hidden"], q_heads=w["q_heads"], kv_heads=w["kv_heads"],
                    head_dim=w["head_dim"], num_layers=w["layers"], mlp_hidden_dim=w["ffn"], rope_theta=w["theta"],
                    rms_eps=1e-5)
    model = LLM.build(cfg, key=0, use_fp8=True, init_std=0.02, device=dev, tp_rank=rank, tp_size=world)
    if w["tied"]:
        model = tie_embedding_and_head(model)
    if tp is not None:
        tp.prepare_model(model)
        tp.shard_lm_head(model)
        if os.environ.get("XAXB_TP_EXCHANGE", "peer") != "nccl":
            tp.enable_peer_exchange(dev, rows=w["batch"], cols=w["hidden"])
        run_info["tp_exchange"] = "peer-memory kernels" if tp.peer is not None else "nccl"
        run_info["tp_amax"] = ("per-rank slice (deviation from the reference)" if tp.local_amax
                               else "max over ranks (the reference's per-token scale)")
    run_info["launch"] = "programmatic dependent launch" if _lib.load().xaxb_programmatic_launch_enabled() else "stream-ordered"
    B, T0 = w["batch"], w["prompt"]
    K = args.steps
    max_len = (T0 + warmup + K + 8 + 127) // 128 * 128
    st = DecodeState(model, B, max_len, tp=tp)
    gen = torch.Generator(device=dev).manual_seed(1)
    t_prefill = None
    if args.synthetic_kv:
        for c in st.caches:
            c["k"][:, :T0].normal_(generator=gen)
            c["v"][:, :T0].normal_(generator=gen)
        st.positions.fill_(T0)
        st.cur.copy_(torch.randint(0, w["vocab"], (B,), generator=gen, device=dev, dtype=torch.int32))
        st.step()  # builds the weight caches
    else:
        prompt = torch.randint(0, w["vocab"], (B, T0), generator=gen, device=dev, dtype=torch.int32)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        st.prefill(prompt[:w["prefill_chunk"]].contiguous(), w["prefill_chunk"])  # warm: quantises the weights
        st.positions.zero_()
        torch.cuda.synchronize()
        e0.record()
        st.prefill(prompt, w["prefill_chunk"])
        e1.record()
        torch.cuda.synchronize()
        t_prefill = e0.elapsed_time(e1) * 1e-3
    _lib.device_status()
    parity = tp_block_parity(tp, model, cfg, w, dev) if tp is not None else None
    lib = _lib.load()
    lib.xaxb_launch_count(1)
    st.capture()
    launches_per_step = int(lib.xaxb_launch_count(1)) // 2  # capture() runs the step twice (warm-up + capture)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(warmup):
        st.replay()
    sampler = ClockSampler(local_rank)
    barrier()
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(K):
        st.replay()
    e1.record()
    barrier()
    clocks = sampler.stop()
    elapsed = e0.elapsed_time(e1) * 1e-3
    if world > 1:
        tmax = torch.tensor([elapsed], device=dev)
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        elapsed = float(tmax.item())
    _lib.device_status()
    mean_len_timed = T0 + warmup + (K + 1) / 2.0

    # ---- e2e: the same steps through the host-facing API (pinned host tokens in and out)
    tin = torch.empty((B,), dtype=torch.int32).pin_memory()
    tout = torch.empty((B,), dtype=torch.int32).pin_memory()
    tin.copy_(st.cur.cpu())
    st.positions.fill_(T0 + warmup)  # same context range as the device-timed region
    barrier()
    t0 = time.perf_counter()
    for _ in range(K):
        st.step_host(tin, tout)
        tin, tout = tout, tin
    barrier()
    e2e_elapsed = time.perf_counter() - t0
    if world > 1:
        tmax = torch.tensor([e2e_elapsed], device=dev)
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        e2e_elapsed = float(tmax.item())
    _lib.device_status()

    # ---- roofline of the dominant kernel: the decode-attention launches of one step (the fused
    # RoPE + append + attention kernel and its merge pass, one pair per layer, on the model's own caches
    # at the mean context of the timed region) captured in a CUDA graph of their own and timed with CUDA
    # events around its replays, so the figure is device time per launch pair without host launch gaps.
    peak, peak_kind = measured_peaks()
    hkv_local, hq_local, D = w["kv_heads"] // world, w["q_heads"] // world, w["head_dim"]
    st.positions.fill_(int(mean_len_timed) - 1)  # representative length: the mean of the timed region
    gq = torch.Generator(device=dev).manual_seed(11)
    qkv_l = torch.randn((B, (hq_local + 2 * hkv_local) * D), generator=gq, device=dev).to(torch.bfloat16)
    blocks = model.blocks
    tables = [blk.self_attn.rotary_emb.tables(st.max_len, dev) for blk in blocks]

    def attention_of_every_layer():
        for l, blk in enumerate(blocks):
            ops.attn_decode_append(qkv_l, st.caches[l]["k"], st.caches[l]["v"], st.positions, tables[l][0], tables[l][1],
                                   hq_local, want_out=False, cast=True, workspace=st.workspace)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        attention_of_every_layer()
    torch.cuda.current_stream().wait_stream(side)
    agraph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(agraph):
        attention_of_every_layer()
    agraph.replay()
    torch.cuda.synchronize()
    durs = []
    for _ in range(3):
        e_a, e_b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e_a.record()
        agraph.replay()
        e_b.record()
        e_b.synchronize()
        durs.extend([e_a.elapsed_time(e_b) * 1e-3 / len(blocks)] * len(blocks))
    attn_len = int(mean_len_timed) + 0.5
    attn_bytes = B * attn_len * (2 * hkv_local * D * 2) + 2 * B * hq_local * D * 2
    avg = sum(durs) / max(len(durs), 1)
    roofline = {"bound": "hbm", "kernel": "attn_decode_kernel (RoPE + cache append fused in, + its merge pass)", "achieved": attn_bytes / avg / 1e9,
                "peak": peak, "peak_kind": f"of {peak_kind} copy bandwidth", "unit": "GB/s",
                "frac": attn_bytes / avg / 1e9 / peak,
                # DRAM bytes per launch: ncu on a smaller case of the same kernel (B=32, same context, heads)
                # measured dram read+write = 1.0385 x the algorithmic bytes (partial results, and the last
                # chunk fetched in 32-row boxes); traffic is proportional to tokens x kv heads, so the factor
                # carries over
                "traffic": attn_bytes * 1.0385, "bytes_per_launch": attn_bytes,
                "avg_launch_us": avg * 1e6, "launches_timed": len(durs)}
    _lib.device_status()

    if rank != 0:
        # The other ranks have nothing left to compute: they wait on the host (no kernel spins on
        # their GPUs) until rank 0 has printed its line, then leave.
        torch.cuda.synchronize()
        dist.barrier(group=host_group)
        _leave()
    line = dict(base)
    line["run"] = run_info
    if parity is not None:
        line["parity"] = parity
    line.update({"value": B * K / elapsed, "ms_per_step": elapsed / K * 1e3, "clocks": clocks,
                 "e2e": {"value": B * K / e2e_elapsed, "unit": unit, "h2d_bytes_per_step": B * 4,
                         "d2h_bytes_per_step": B * 4, "ms_per_step": e2e_elapsed / K * 1e3},
                 "gpu_launches": launches_per_step * K, "launches_per_step": launches_per_step,
                 "roofline": roofline, "prefill_s": t_prefill,
                 "mean_context_timed": mean_len_timed})
    if not args.no_kernels:
        del st
        torch.cuda.empty_cache()
        try:
            line["kernels"] = kernel_figures(peak)
        except Exception as e:  # noqa: BLE001
            line["kernels"] = {"error": repr(e)}
    if not args.no_cpu:
        r = oracle_decode_sample(w, seconds_limit=20.0, steps=2, warmup=0)
        line["cpu_baseline"] = {"value": r["tokens_per_s"], "unit": unit, "cores": host_threads(), "kind": "port",
                                "sample": r["sample"]}
    else:
        line["cpu_baseline"] = None
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier(group=host_group)
        _leave()


def tp_block_parity(tp, model, cfg, w: dict, dev) -> dict:
    """First transformer block, one decode step of the workload's batch at position 0: the sharded
    block (every rank takes part) against the same block unsharded on rank 0, whose full weights
    are re-drawn from the model's seed (LLM.build draws whole tensors and slices them, in a fixed
    order, so a one-layer build with the same seed holds block 0's full tensors).  Relative
    Frobenius error of the block output, computed on rank 0."""
    from dataclasses import replace

    import torch

    from xax_b200.arch.llm import LLM

    B = w["batch"]
    gen = torch.Generator(device=dev).manual_seed(7)
    toks = torch.randint(0, w["vocab"], (B,), generator=gen, device=dev, dtype=torch.int32)
    x = model.embed_tokens(toks)
    blk = model.blocks[0]
    cache = blk.self_attn.init_cache(128, batch=B, device=dev)
    if tp.peer is not None and tp.peer.exchanges & 1:  # keep the two data buffers alternating in step
        tp.all_reduce_sum(tp.partial_out(B, x.shape[1]).zero_())
    y_tp, _ = tp.block_forward(blk, x, B, 1, cache=cache)
    out = {"what": f"block 0, one decode step, batch {B}: tp{tp.size} vs unsharded, relative Frobenius error"}
    if tp.rank == 0:
        full = LLM.build(replace(cfg, num_layers=1), key=0, use_fp8=True, init_std=0.02, device=dev)
        fb = full.blocks[0]
        y_1, _ = fb.forward_tokens(x, B, 1, cache=fb.self_attn.init_cache(128, batch=B, device=dev))
        out["block0_rel_fro"] = float((y_tp.float() - y_1.float()).norm() / y_1.float().norm())
        del full, fb
        torch.cuda.empty_cache()
    return out


def _leave() -> None:
    """Multi-rank exit.  Tearing down an NCCL process group whose collectives were captured in a
    CUDA graph can block for the whole time limit, so the ranks synchronise, flush and leave without
    it; by then every rank has passed the last host-side barrier with its GPU idle."""
    import torch

    torch.cuda.synchronize()
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
