"""Benchmark of the decode hot path: batch-1 greedy decode of a Llama-3.2-1B-shape model with
Q4_K_M-style weights (Q4_K, attn_v and ffn_down in Q6_K), random-init, synthetic prompt.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = one decode token.  Prints ONE JSON line:
  value      tokens/s with every input resident in HBM (token fed back on the device, CUDA-graph
             replays), timed with CUDA events on the library's stream; whole job = sum over ranks
  e2e        tokens/s through the C-ABI call that takes HOST buffers (token id in, full logits and
             next id out), host<->device copies inside the timed region
  roofline   the dominant kernel (fused gate/up Q4_K GEMV) timed alone over rotating weights
  cpu_baseline  the reference CLI on its own CPU backend, a few tokens, on this box's host cores
At N > 1 every rank runs an independent replica of the same job (the model fits one GPU; the
reference has no multi-device path), so scaling is weak and there is no data-path collective.

--impl reference times the reference's CPU implementation of the same workload (oracle/_ref, built
from the unmodified reference sources; the C restatement if that binary is absent).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from ggnpu_b200.testing import synth as S  # noqa: E402

PROMPT_LEN = 128
WORKLOAD = "llama-3.2-1b-shape Q4_K_M-style (Q4_K; attn_v, ffn_down Q6_K), batch-1 greedy decode after a 128-token prompt, ctx 2048"
METRIC, UNIT = "decode_tokens_per_s_batch1", "tok/s"


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.rows, self.proc = [], None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "20",
                                          "-i", str(index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.th = threading.Thread(target=self._read, daemon=True)
            self.th.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.perf_counter(), [c.strip() for c in line.split(",")]))

    def close(self):
        if self.proc:
            self.proc.terminate()

    def stats(self, t0=None, t1=None):
        """Median SM clock, maximum clock and the throttle reasons seen in [t0, t1] (perf_counter times; None = open end)."""
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        if t1 is not None:
            time.sleep(0.05)                      # let the sample that covers the end of the window arrive
        snap = list(self.rows)
        rows = [r for t, r in snap if (t0 is None or t >= t0) and (t1 is None or t <= t1 + 0.03)] or [r for _, r in snap[-3:]]
        sm, mx, reasons = [], [], set()
        for r in rows:
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
            except Exception:
                continue
            for name, v in zip(["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"], r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def build_synth(device: str):
    return S.build_model(S.LLAMA_1B, device=device)


def prompt_ids(cfg, n=PROMPT_LEN):
    return np.random.default_rng(42).integers(0, cfg.vocab, n).astype(np.int32)


# ---------------------------------------------------------------------------------------------
# CPU side: the reference CLI on its own CPU backend
# ---------------------------------------------------------------------------------------------
def time_reference_cli(synth, n_warm: int, n_timed: int, prompt_len: int = 2, exact: bool = False, budget_s: float = 200.0):
    """Greedy decode with the reference CLI on its CPU backend, one thread (the reference's CPU path is
    single-threaded).  Returns (tok/s, kind, description of the sample).

    exact=False times the stock path, Backend::mul_mat_q of the CPU backend (src/backends/cpu_ref/cpu_ref.cpp:87-117;
    valid for this all-Q4_K / Q6_K workload), with the prompt batched as the CLI does by default; exact=True times the
    diagnostic exact-fp32 matmul (GGNPU_FP32_MATMUL, src/cli/main.cpp:1379-1388) that the parity tests use.  The timed
    tokens are the decode steps after the prompt; the count is cut so that the run stays inside budget_s."""
    from oracle.binding import REF_CLI, Oracle, OracleModel
    cfg = synth.cfg
    ids = prompt_ids(cfg, prompt_len)
    per_tok_guess = 2.6 if exact else 1.4          # seconds per full-model token on one core
    prefill_guess = prompt_len * (per_tok_guess if exact else 0.8)
    total = n_warm + n_timed
    total = max(2, min(total, int(max(budget_s - prefill_guess, 10.0) / per_tok_guess)))
    if os.path.exists(REF_CLI):
        with tempfile.TemporaryDirectory() as td:
            path = os.path.join(td, "model.gguf")
            synth.write(path)
            env = dict(os.environ)
            if exact:
                env.update(GGNPU_FP32_MATMUL="1", GGNPU_NO_PREFILL_BATCH="1")
            cmd = [REF_CLI, "-m", path, "-p", S.prompt_text(ids), "-c", "2048", "--no-cache", "-n", str(total), "--temp", "0", "--quiet"]
            p = subprocess.Popen(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.DEVNULL)
            stamps, buf = [], b""
            while True:
                ch = p.stdout.read(1)
                if not ch:
                    break
                buf += ch
                try:
                    buf.decode("utf-8")
                except UnicodeDecodeError:
                    continue
                stamps.append(time.perf_counter())      # one code point = one generated token
                buf = b""
            p.wait()
        if len(stamps) < total or total < 2:
            raise RuntimeError(f"reference CLI produced {len(stamps)} of {total} tokens")
        first = max(min(n_warm, total - 1), 1)          # token 0's stamp includes model load + prompt
        dt = stamps[total - 1] - stamps[first - 1]
        rate = (total - first) / dt
        kind = "reference"
        what = (f"reference CLI (oracle/_ref, unmodified sources), {'exact fp32 matmul (GGNPU_FP32_MATMUL)' if exact else 'stock cpu_ref::mul_mat_q'}, "
                f"{total - first} timed decode tokens at positions {prompt_len + first}.. after a {prompt_len}-token prompt")
    else:
        o = Oracle()
        om = OracleModel(o, synth)
        om.forward(ids, 0, want_logits=False)
        t0 = time.perf_counter()
        tok, n = int(ids[-1]), max(1, min(n_timed, 4))
        for i in range(n):
            tok = o.argmax_first(om.forward([tok], prompt_len + i))
        rate = n / (time.perf_counter() - t0)
        kind = "port"
        what = f"C restatement of the reference layer loop (exact fp32 matmul), {n} decode tokens after a {prompt_len}-token prompt"
    return rate, kind, what


def run_reference(args):
    """The reference arm: the unmodified reference CLI on the host cores, same model, same 128-token prompt, greedy
    decode from position 128 on (the prompt is prefilled by the CLI's own batched path, outside the timed tokens)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    synth = build_synth(dev)
    rate, kind, what = time_reference_cli(synth, args.warmup, args.steps, prompt_len=args.prompt_len, exact=False, budget_s=240.0)
    out = {"impl": "reference", "metric": METRIC, "value": rate, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
           "warmup": args.warmup, "ms_per_step": 1000.0 / rate, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
           "dtype": "f32", "data": "synthetic", "config": {"workload": WORKLOAD, "prompt_tokens": args.prompt_len, "cpu_matmul": "cpu_ref::mul_mat_q (stock)"},
           "cpu_baseline": {"value": rate, "unit": UNIT, "cores": 1, "kind": kind, "sample": what},
           "e2e": {"value": rate, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(out), flush=True)


# ---------------------------------------------------------------------------------------------
# GPU side
# ---------------------------------------------------------------------------------------------
def run_ours(args):
    global PROMPT_LEN
    PROMPT_LEN = args.prompt_len
    import torch
    import torch.distributed as dist
    from ggnpu_b200.backend import CudaBackend, Model

    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the CUDA path has no CPU fallback (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    cfg = S.LLAMA_1B
    synth = build_synth("cuda")
    b = CudaBackend(local)
    model = Model(b, cfg, synth.tensors)
    ids = prompt_ids(cfg, PROMPT_LEN)
    stream = torch.cuda.ExternalStream(b.stream(), device=torch.device("cuda", local))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # prefill (the metric's second figure): the workload's prompt, and a long prompt that fills the
    # tensor-core GEMM's token tiles; one untimed pass first (it sizes the activation scratch)
    def timed_prefill(tokens):
        model.prefill(tokens, 0, want_logits=False)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record(stream)
        _, nxt = model.prefill(tokens, 0, want_logits=False)
        e1.record(stream)
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e-3, nxt

    long_len = min(args.prefill_long, cfg.ctx)
    prefill_long_s, _ = timed_prefill(prompt_ids(cfg, long_len))
    prefill_s, first = timed_prefill(ids)
    K, W = args.steps, max(args.warmup, 0)
    state = {"tok": int(first), "pos": PROMPT_LEN}

    def generate(n):
        """n device-resident steps; when the 2048-token context is full the position wraps back to
        the end of the prompt (the cache rows there are simply overwritten)."""
        while n > 0:
            room = cfg.ctx - state["pos"]
            if room <= 0:
                state["pos"] = PROMPT_LEN
                continue
            m = min(n, room)
            toks = model.generate(state["tok"], state["pos"], m)
            state["tok"], state["pos"] = int(toks[-1]), state["pos"] + m
            n -= m

    # ---- value: device-resident loop ----
    sampler = ClockSampler(local) if rank == 0 else None      # from before the warm-up to the end of the roofline sweeps
    if W:
        generate(W)
    barrier()
    launches0 = b.launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_start = time.perf_counter()
    ev0.record(stream)
    generate(K)
    ev1.record(stream)
    barrier()
    t_end = time.perf_counter()
    launches = b.launch_count() - launches0
    ms = ev0.elapsed_time(ev1)
    clocks = sampler.stats(t_start, t_end) if sampler else None
    first, pos = state["tok"], state["pos"]
    bytes_step = model.decode_bytes(max(PROMPT_LEN, pos - K // 2))

    # ---- e2e: host buffers through ggb_model_decode ----
    logits = torch.empty(cfg.vocab, dtype=torch.float32, pin_memory=True).numpy()      # page-locked: the library copies straight into it
    tok = first
    for i in range(min(W, 3)):
        pos = pos if pos < cfg.ctx else PROMPT_LEN
        _, tok = model.decode(tok, pos, logits_out=logits)
        pos += 1
    barrier()
    t0 = time.perf_counter()
    for i in range(K):
        pos = pos if pos < cfg.ctx else PROMPT_LEN
        _, tok = model.decode(tok, pos, logits_out=logits)
        pos += 1
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0

    t = torch.tensor([ms, e2e_s * 1000.0], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_max, e2e_ms_max = float(t[0]), float(t[1])

    # ---- roofline of the dominant kernel: the fused gate/up (SwiGLU) Q4_K GEMV, timed alone ----
    roof = gemm_roof = None
    if rank == 0:
        peak, peak_kind = peaks()
        N, Kd = cfg.ffn, cfg.hidden
        copies = []
        for l in range(cfg.n_layer):                         # 16 distinct pairs = 302 MB > 126 MB L2
            g = synth.tensors[f"blk.{l}.ffn_gate.weight"][2]
            u = synth.tensors[f"blk.{l}.ffn_up.weight"][2]
            copies.append((b.upload_weight(S.Q4_K, g, N, Kd), b.upload_weight(S.Q4_K, u, N, Kd)))
        x = torch.randn(1, Kd, device="cuda", dtype=torch.float32)
        gamma = torch.ones(Kd, device="cuda", dtype=torch.float32)
        y = torch.empty(1, N, device="cuda", dtype=torch.float32)
        torch.cuda.synchronize()

        def sweep(timed):
            evs = []
            for wg, wu in copies:
                if timed:
                    a, c = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record(stream)
                b.gemv_swiglu_device(wg, wu, x.data_ptr(), 1, Kd, y.data_ptr(), N, gamma.data_ptr(), 1e-5)
                if timed:
                    c.record(stream)
                    evs.append((a, c))
            b.sync()
            return [a.elapsed_time(c) for a, c in evs]

        for _ in range(3):
            sweep(False)
        times = []
        for _ in range(5):
            times += sweep(True)
        avg_ms = float(np.mean(times))
        # the same launches back to back, one event pair around all of them: consecutive launches overlap under
        # programmatic dependent launch, as they do inside the decode graph
        a0, c0 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record(stream)
        for _ in range(5):
            for wg, wu in copies:
                b.gemv_swiglu_device(wg, wu, x.data_ptr(), 1, Kd, y.data_ptr(), N, gamma.data_ptr(), 1e-5)
        c0.record(stream)
        b.sync()
        b2b_ms = a0.elapsed_time(c0) / (5 * len(copies))
        alg_bytes = 2 * N * (Kd // 256) * 144 + Kd * 4 + Kd * 4 + N * 4
        achieved = alg_bytes / (avg_ms * 1e-3) / 1e9
        roof = {"bound": "hbm", "kernel": "gemv_mma_q4k_kernel (dual gate/up 8192x2048 Q4_K + SwiGLU + RMSNorm prologue, M = 1)", "achieved": achieved, "peak": peak,
                "unit": "GB/s", "frac": achieved / peak, "peak_source": peak_kind,
                # dram__bytes_read.sum + dram__bytes_write.sum of one launch of this kernel on this workload, from the ncu capture
                # summarised in profiles/gemv_mma_q4k_dual_8192x2048_m1.md (1.002 x the algorithmic bytes)
                "traffic": 18969600, "traffic_source": "ncu capture, profiles/gemv_mma_q4k_dual_8192x2048_m1.md",
                "bytes_per_launch": alg_bytes, "avg_launch_us": avg_ms * 1e3, "launches_timed": len(times),
                "timing": "one CUDA-event pair per launch (no overlap between consecutive launches)",
                "back_to_back": {"avg_launch_us": b2b_ms * 1e3, "achieved": alg_bytes / (b2b_ms * 1e-3) / 1e9,
                                 "frac": alg_bytes / (b2b_ms * 1e-3) / 1e9 / peak, "launches_timed": 5 * len(copies),
                                 "timing": "one event pair around all launches"}}
        # ---- tensor roofline of the prefill GEMM: the same gate/up pairs at a 2048-token chunk ----
        Mg = 2048
        xg = torch.randn(Mg, Kd, device="cuda", dtype=torch.float32)
        yg = torch.empty(Mg, N, device="cuda", dtype=torch.float32)
        torch.cuda.synchronize()

        def gemm_sweep(timed):
            evs = []
            for wg, wu in copies:
                if timed:
                    a, c = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record(stream)
                b.gemv_swiglu_device(wg, wu, xg.data_ptr(), Mg, Kd, yg.data_ptr(), N, gamma.data_ptr(), 1e-5)
                if timed:
                    c.record(stream)
                    evs.append((a, c))
            b.sync()
            return [a.elapsed_time(c) for a, c in evs]

        gemm_sweep(False)
        gtimes = []
        for _ in range(3):
            gtimes += gemm_sweep(True)
        g_ms = float(np.mean(gtimes))
        flops = 2.0 * 2 * N * Kd * Mg
        try:
            tpeak = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops"])
            tkind = "measured (cuBLAS bf16 burst; the kernel is timed alone)"
        except Exception:
            tpeak, tkind = 1590.0, "fallback"
        gemm_roof = {"bound": "tensor", "kernel": "gemm_tc_kernel (dual gate/up 8192x2048 Q4_K + SwiGLU, 2048 tokens; includes the fp16 activation preparation kernel)",
                     "achieved": flops / (g_ms * 1e-3) / 1e12, "peak": tpeak, "unit": "TFLOP/s", "frac": flops / (g_ms * 1e-3) / 1e12 / tpeak,
                     "peak_source": tkind, "traffic": 44704768, "traffic_source": "ncu capture (DRAM bytes; the fp32 result mostly stays in L2), profiles/gemm_tc_q4k_dual_8192x2048_m2048.md",
                     "flops_per_launch": flops, "avg_launch_us": g_ms * 1e3, "launches_timed": len(gtimes)}
        for wg, wu in copies:
            b.free_weight(wg); b.free_weight(wu)

    if sampler:
        # the same sampler over everything so far: warm-up, timed loop, end-to-end loop and the two roofline sweeps
        clocks["whole_run"] = sampler.stats(None, None)
        sampler.close()
    if rank == 0:
        peak, peak_kind = peaks()
        value = world * K / (ms_max * 1e-3)
        e2e = world * K / (e2e_ms_max * 1e-3)
        step_gbs = bytes_step / (ms_max / K * 1e-3) / 1e9
        out = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms_max / K,
               "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
               "data": "synthetic", "config": {"workload": WORKLOAD, "weights": "seeded N(0,0.02) random-init, RTN-quantised", "replicas": world,
                                                "l2": "each step streams 773 MB of weights (> 126 MB L2), no flush needed",
                                                "prompt_tokens": PROMPT_LEN, "activations": "f32", "kv_cache": "bf16 paged"},
               "e2e": {"value": e2e, "unit": UNIT, "h2d_bytes_per_step": 8, "d2h_bytes_per_step": cfg.vocab * 4 + 4},
               "gpu_launches": launches, "roofline": roof, "prefill_gemm_roofline": gemm_roof, "clocks": clocks,
               "decode_step": {"algorithmic_bytes": bytes_step, "achieved_gbs": step_gbs, "frac_of_hbm_peak": step_gbs / peak, "peak_source": peak_kind},
               "prefill": {"tokens": PROMPT_LEN, "tok_per_s": PROMPT_LEN / prefill_s, "long_tokens": long_len,
                           "long_tok_per_s": long_len / prefill_long_s,
                           "note": "CUDA events around ggb_model_prefill (host ids in, next token out); projections run on the tcgen05 GEMM"}}
        if world == 1 and not args.no_cpu_baseline:
            try:
                rate, kind, what = time_reference_cli(synth, 1, 8, prompt_len=2, exact=False, budget_s=30.0)
                out["cpu_baseline"] = {"value": rate, "unit": UNIT, "cores": 1, "kind": kind, "sample": what,
                                       "host_cores_available": os.cpu_count()}
                rate_x, _, what_x = time_reference_cli(synth, 1, 4, prompt_len=2, exact=True, budget_s=20.0)
                out["cpu_baseline"]["exact_fp32_path"] = {"value": rate_x, "unit": UNIT, "sample": what_x}
            except Exception as e:  # the GPU numbers stand on their own
                out["cpu_baseline"] = {"value": None, "unit": UNIT, "cores": 1, "kind": "unavailable", "sample": str(e)[:200]}
    model.close()
    extras = {}
    if not args.no_extras:
        if world == 1:
            try:
                extras["config3"] = config3_figures(b, local)
            except Exception as e:
                extras["config3"] = {"unavailable": str(e)[:200]}
            try:
                extras["lfm2"] = lfm2_figures(b, local)
            except Exception as e:
                extras["lfm2"] = {"unavailable": str(e)[:200]}
    b.close()
    if not args.no_extras and world == 1:
        # the 8B-shape model on one GPU: 4096-token prompt, decode at batch 1 and at batch 16
        try:
            extras["config4"] = tp_measure(args, rank, local, world, min(K, 32), W)
        except Exception as e:
            extras["config4"] = {"unavailable": str(e)[:300]}
        # the qwen35moe shape (40 layers): 128-token prompt (one graph replay per token), batch-1 decode
        try:
            c5 = config5_measure(args, rank, local, world, min(K, 64), W)
            extras["config5"] = {k: c5[k] for k in ("value", "unit", "ms_per_step", "steps", "gpu_launches", "ms_per_token_layer", "prefill", "decode_step", "model_build_s")}
            extras["config5"]["workload"] = c5["config"]["workload"]
        except Exception as e:
            extras["config5"] = {"unavailable": str(e)[:300]}
    if not args.no_extras and world > 1:
        # the sharded paths, where the driver can see them: parity of tensor / expert parallel against one GPU, and the
        # tensor-parallel figures of the 8B-shape model over the ranks of this launch (strong scaling)
        try:
            chk = parallel_check(rank, local, world)
            tp = tp_measure(args, rank, local, world, min(K, 32), W)
            if rank == 0:
                extras.update(chk)
                extras["tp"] = tp
        except Exception as e:
            extras["tp"] = {"unavailable": str(e)[:300]}
    if rank == 0:
        out.update(extras)
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_micro(args):
    """Quantised-matmul microbenchmark (weights N x K in several formats, activation rows M): one JSON
    line per case with the kernel's average launch time and algorithmic GB/s.  Weight copies rotate
    through more than 256 MB so every launch reads HBM, not L2.  Used for profiling single kernels:
        python bench.py --micro --types Q4_K --shapes 8192x2048 --ms 1 --dual --reps 3"""
    import torch
    from ggnpu_b200.backend import CudaBackend
    b = CudaBackend(0)
    stream = torch.cuda.ExternalStream(b.stream(), device=torch.device("cuda", 0))
    peak, peak_kind = peaks()
    for tname in args.types.split(","):
        t = S.TYPE_IDS[tname]
        for shp in args.shapes.split(","):
            N, K = (int(v) for v in shp.split("x"))
            g = torch.Generator(device="cuda").manual_seed(7)
            wbytes = N * S.row_bytes(t, K) * (2 if args.dual else 1)
            copies = max(2, min(64, -(-(256 << 20) // wbytes)))
            raw = S.quantize(torch.randn(N, K, generator=g, device="cuda") * 0.02, t).cpu().numpy()
            ws = [b.upload_weight(t, raw, N, K) for _ in range(copies * (2 if args.dual else 1))]   # distinct HBM copies
            for M in (int(v) for v in args.ms.split(",")):
                x = torch.randn(M, K, device="cuda", dtype=torch.float32)
                y = torch.empty(M, N, device="cuda", dtype=torch.float32)
                torch.cuda.synchronize()

                def one(i):
                    if args.dual:
                        b.gemv_swiglu_device(ws[2 * i], ws[2 * i + 1], x.data_ptr(), M, K, y.data_ptr(), N)
                    else:
                        b.gemv_device(ws[i], x.data_ptr(), M, K, y.data_ptr(), N)

                for i in range(copies):
                    one(i)
                b.sync()
                times = []
                for _ in range(args.reps):
                    evs = []
                    for i in range(copies):
                        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        e0.record(stream); one(i); e1.record(stream)
                        evs.append((e0, e1))
                    b.sync()
                    times += [e0.elapsed_time(e1) for e0, e1 in evs]
                # back-to-back launches (no events in between): launch overhead amortised
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                for _ in range(args.reps):
                    for i in range(copies):
                        one(i)
                e1.record(stream)
                b.sync()
                b2b_us = e0.elapsed_time(e1) * 1e3 / (args.reps * copies)
                alg = wbytes + M * K * 4 + M * N * 4
                us = float(np.mean(times)) * 1e3
                print(json.dumps({"micro": "quant_matmul", "type": tname, "N": N, "K": K, "M": M, "dual": bool(args.dual),
                                  "avg_launch_us": us, "back_to_back_us": b2b_us, "alg_bytes": alg, "gbs": alg / us / 1e3,
                                  "gbs_back_to_back": alg / b2b_us / 1e3, "frac_of_hbm_peak": alg / b2b_us / 1e3 / peak,
                                  "tflops_back_to_back": 2.0 * M * N * K * (2 if args.dual else 1) / b2b_us / 1e6,
                                  "peak_source": peak_kind, "copies": copies}), flush=True)
            for w in ws:
                b.free_weight(w)
    b.close()


def run_micro_moe(args):
    """Decode-side MoE FFN microbenchmark at the qwen35moe expert shapes: hidden 2048,
    256 routed experts of FFN 512 (Q4_K gate/up, Q6_K down), top-8 + shared expert.  64 different tokens
    are routed in turn, so successive calls touch different experts of the 0.4 GB expert set (> L2).
        python bench.py --micro-moe"""
    import torch
    from ggnpu_b200.backend import CudaBackend
    b = CudaBackend(0)
    stream = torch.cuda.ExternalStream(b.stream(), device=torch.device("cuda", 0))
    peak, peak_kind = peaks()
    H, eff, nE, k, eff_sh = 2048, 512, args.moe_experts, 8, 512
    g = torch.Generator(device="cuda").manual_seed(7)

    def up(n, kdim, t):
        raw = S.quantize(torch.randn(n, kdim, generator=g, device="cuda") * 0.02, t).cpu().numpy()
        return b.upload_weight(t, raw, n, kdim)

    hg, hu, hd = up(nE * eff, H, S.Q4_K), up(nE * eff, H, S.Q4_K), up(nE * H, eff, S.Q6_K)
    sg, su, sd = up(eff_sh, H, S.Q4_K), up(eff_sh, H, S.Q4_K), up(H, eff_sh, S.Q6_K)
    router = (torch.randn(nE, H, generator=g, device="cuda") * 0.05).contiguous()
    sgi = (torch.randn(H, generator=g, device="cuda") * 0.05).contiguous()
    xs = torch.randn(64, H, generator=g, device="cuda").contiguous()
    y = torch.empty(H, device="cuda")
    torch.cuda.synchronize()

    def one(i):
        x = xs[i % 64]
        b.moe_ffn_device(x=x.data_ptr(), resid=x.data_ptr(), y=y.data_ptr(), router=router.data_ptr(), gate_exps=hg, up_exps=hu,
                         down_exps=hd, sh_gate=sg, sh_up=su, sh_down=sd, sh_gate_inp=sgi.data_ptr(), hidden=H, eff=eff, eff_sh=eff_sh,
                         n_expert=nE, top_k=k, sel_out=None, w_out=None)

    for i in range(64):
        one(i)
    b.sync()
    l0 = b.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n = 64 * args.reps
    e0.record(stream)
    for i in range(n):
        one(i)
    e1.record(stream)
    b.sync()
    us = e0.elapsed_time(e1) * 1e3 / n
    alg = nE * H * 4 + H * 4 + (k + 1) * (2 * eff * (H // 256) * 144 + H * (eff // 256) * 210) + H * 12
    print(json.dumps({"micro": "moe_ffn_decode", "hidden": H, "eff": eff, "n_expert": nE, "top_k": k, "shared_eff": eff_sh,
                      "us_per_token_layer": us, "launches_per_call": (b.launch_count() - l0) / n, "alg_bytes": alg,
                      "gbs": alg / us / 1e3, "frac_of_hbm_peak": alg / us / 1e3 / peak, "peak_source": peak_kind,
                      "reference_equivalent": "9 experts x 3 host-pointer matmuls + sync each (src/cli/main.cpp:3152-3191)"}), flush=True)
    b.close()


def run_micro_deltanet(args):
    """Gated DeltaNet step at the qwen35moe shape (16 key / 32 value heads of 128, conv 4): per layer and token the
    4 MB recurrent state is read and written once.  30 layers' states (60 MB read + 60 MB written per pass) are
    stepped in turn, so the state comes from HBM rather than L2 only partly (126 MB L2).
        python bench.py --micro-deltanet"""
    import torch
    from ggnpu_b200.backend import CudaBackend
    b = CudaBackend(0)
    stream = torch.cuda.ExternalStream(b.stream(), device=torch.device("cuda", 0))
    peak, peak_kind = peaks()
    nK, nV, sk, ck, layers = 16, 32, 128, 4, 30
    cd = 2 * nK * sk + nV * sk
    g = torch.Generator(device="cuda").manual_seed(3)
    rn = lambda *shape: torch.randn(*shape, generator=g, device="cuda")
    conv_w, ssm_a, dt, norm = 0.3 * rn(cd, ck), -torch.exp(0.5 * rn(nV)), rn(nV), 1 + 0.1 * rn(sk)
    cs = [torch.zeros(ck - 1, cd, device="cuda") for _ in range(layers)]
    S = [torch.zeros(nV, sk, sk, device="cuda") for _ in range(layers)]
    mixed, z, ar, br, out = rn(cd), rn(nV * sk), rn(nV), rn(nV), torch.empty(nV * sk, device="cuda")
    torch.cuda.synchronize()

    def one(l):
        b.deltanet_step_device(mixed=mixed.data_ptr(), zgate=z.data_ptr(), araw=ar.data_ptr(), braw=br.data_ptr(), conv_w=conv_w.data_ptr(),
                               ssm_a=ssm_a.data_ptr(), dt_bias=dt.data_ptr(), ssm_norm=norm.data_ptr(), conv_state=cs[l].data_ptr(),
                               rec_state=S[l].data_ptr(), out=out.data_ptr(), n_khead=nK, n_vhead=nV, sk=sk, conv_k=ck, rms_eps=1e-6)

    for l in range(layers):
        one(l)
    b.sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n = layers * args.reps
    e0.record(stream)
    for i in range(n):
        one(i % layers)
    e1.record(stream)
    b.sync()
    us = e0.elapsed_time(e1) * 1e3 / n
    alg = 2 * nV * sk * sk * 4 + 2 * (ck - 1) * cd * 4 + cd * (ck + 2) * 4 + 2 * nV * sk * 4
    print(json.dumps({"micro": "deltanet_step", "n_khead": nK, "n_vhead": nV, "sk": sk, "conv_k": ck, "us_per_token_layer": us,
                      "launches_per_call": 2, "alg_bytes": alg, "gbs": alg / us / 1e3, "frac_of_hbm_peak": alg / us / 1e3 / peak,
                      "peak_source": peak_kind}), flush=True)
    b.close()


def run_micro_allreduce(args):
    """Latency of the tensor-parallel all-reduce at decode message sizes, peer-memory one-shot kernel vs
    NCCL, back to back on the compute stream (run under torchrun, one process per GPU)."""
    import torch
    import torch.distributed as dist
    from ggnpu_b200.backend import CudaBackend
    rank, local, world = int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    b = CudaBackend(local)
    box = [b.tp_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    b.tp_init(box[0], rank, world)
    stream = torch.cuda.ExternalStream(b.stream(), device=torch.device("cuda", local))
    res = {}
    for mode in ("nccl", "one_shot"):
        if mode == "one_shot":
            handles = [None] * world
            dist.all_gather_object(handles, b.tp_ipc_handle())
            b.tp_attach_peers(handles)
        for n in (1024, 4096, 16384):
            t = torch.ones(n, device="cuda")
            for _ in range(20):
                b.tp_all_reduce_device(t.data_ptr(), n)
                t.fill_(1.0)
            b.sync(); dist.barrier(); torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(200):
                b.tp_all_reduce_device(t.data_ptr(), n)
            e1.record(stream)
            b.sync()
            res[f"{mode}_{n * 4}B_us"] = e0.elapsed_time(e1) * 1e3 / 200
    if rank == 0:
        print(json.dumps({"micro": "tp_all_reduce", "ranks": world, **res}), flush=True)
    dist.barrier()
    b.close()
    dist.destroy_process_group()


def join_group(b, rank, world, nccl_only=False):
    """Make backend b one rank of a tensor / expert parallel group over the ranks of this launch."""
    import torch.distributed as dist
    if world <= 1:
        return
    box = [b.tp_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    b.tp_init(box[0], rank, world)
    if not nccl_only:                              # one-shot peer-memory all-reduce for the 16 KB decode messages
        handles = [None] * world
        dist.all_gather_object(handles, b.tp_ipc_handle())
        b.tp_attach_peers(handles)


def tp_measure(args, rank, local, world, steps, warmup):
    """Tensor-parallel decode + prefill of the Llama-3-8B-shape model over all ranks of this launch (strong scaling: the
    model is fixed, each rank holds 1 / N of the heads, FFN rows and vocabulary).  torch.distributed must be up.
    Returns the result dict on rank 0, None elsewhere."""
    import dataclasses
    import torch
    import torch.distributed as dist
    from ggnpu_b200.backend import CudaBackend, Model
    ctx = args.tp_ctx
    cfg = dataclasses.replace(S.LLAMA_8B, ctx=ctx, n_layer=args.tp_layers or S.LLAMA_8B.n_layer)
    b = CudaBackend(local)
    join_group(b, rank, world, args.tp_nccl_only)
    t0 = time.perf_counter()
    synth = S.build_model(cfg, device="cuda")
    nb = max(1, min(16, args.tp_batch))
    model = Model(b, cfg, synth.tensors, n_seq=nb)
    build_s = time.perf_counter() - t0
    del synth
    stream = torch.cuda.ExternalStream(b.stream(), device=torch.device("cuda", local))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    n_prompt = min(args.tp_prompt, ctx - steps - max(warmup, 3) - 1)
    ids = prompt_ids(cfg, n_prompt)
    model.prefill(ids, 0, want_logits=False)                      # untimed pass sizes the scratch
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    _, first = model.prefill(ids, 0, want_logits=False)
    e1.record(stream)
    barrier()
    prefill_ms = e0.elapsed_time(e1)
    K, W = steps, max(warmup, 3)
    toks = model.generate(int(first), n_prompt, W)
    barrier()
    launches0 = b.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    toks = model.generate(int(toks[-1]), n_prompt + W, K)
    e1.record(stream)
    barrier()
    ms = e0.elapsed_time(e1)
    launches = b.launch_count() - launches0
    # the batch leg: nb sequences (every KV stream holds the prompt), one forward per step for all of them
    batch_ms, batch_same = 0.0, None
    if nb > 1:
        single = model.generate(int(first), n_prompt, W)
        for r in range(1, nb):
            model.select_sequence(r)
            model.prefill(ids, 0, want_logits=False)
        model.select_sequence(0)
        firsts, pos = np.full(nb, int(first), np.int32), np.full(nb, n_prompt, np.int32)
        out = model.generate_batch(firsts, pos, W)
        batch_same = bool((out == out[:, :1]).all()) and bool(np.array_equal(out[:, 0], single))
        barrier()
        launches0 = b.launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        model.generate_batch(out[-1], pos + W, K)
        e1.record(stream)
        barrier()
        batch_ms = e0.elapsed_time(e1)
        batch_launches = b.launch_count() - launches0
    t = torch.tensor([ms, prefill_ms, batch_ms], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, prefill_ms, batch_ms = float(t[0]), float(t[1]), float(t[2])
    res = None
    if rank == 0:
        peak, peak_kind = peaks()
        bytes_step = model.decode_bytes(n_prompt + W + K // 2)        # this rank's shard
        res = {"decode_tok_s": K / (ms * 1e-3), "ms_per_step": ms / K, "steps": K, "warmup": W, "prefill_tokens": n_prompt,
               "prefill_tok_s": n_prompt / (prefill_ms * 1e-3), "gpu_launches": launches, "layers": cfg.n_layer, "ctx": ctx,
               "allreduce": "none" if world == 1 else ("NCCL" if args.tp_nccl_only or world < 4 else "one-shot peer-memory kernel (decode), NCCL (prefill)"),
               "algorithmic_bytes_per_rank": bytes_step, "achieved_gbs_per_rank": bytes_step / (ms / K * 1e-3) / 1e9,
               "frac_of_hbm_peak": bytes_step / (ms / K * 1e-3) / 1e9 / peak, "peak_source": peak_kind, "model_build_s": build_s}
        if nb > 1:
            # per step: the weights once, every sequence's KV stream once
            kv_one = model.decode_bytes(n_prompt + W + K // 2) - model.decode_bytes(0)
            bytes_b = model.decode_bytes(0) + nb * kv_one
            res["batch"] = {"sequences": nb, "decode_tok_s": nb * K / (batch_ms * 1e-3), "ms_per_step": batch_ms / K, "gpu_launches": batch_launches,
                            "algorithmic_bytes_per_rank": bytes_b, "frac_of_hbm_peak": bytes_b / (batch_ms / K * 1e-3) / 1e9 / peak,
                            "rows_identical_and_equal_to_single_sequence": batch_same}
    model.close()
    b.close()
    return res


def parallel_check(rank, local, world):
    """Parity of the sharded paths where the driver can see it: a tiny llama (tensor parallel) and a tiny qwen35moe (expert
    parallel) over the ranks of this launch, against the SAME models on one GPU (rank 0, a handle outside the group; that
    path is held to the CPU oracle by the test suite).  Outside every timed region."""
    import torch
    import torch.distributed as dist
    from ggnpu_b200.backend import CudaBackend, Model, Q35Model
    out = {}
    solo = CudaBackend(local) if rank == 0 else None
    grp = CudaBackend(local)
    join_group(grp, rank, world)
    # shapes that split over 2, 4 or 8 ranks (row-parallel K slices must be whole 256-blocks)
    cases = {"tp_check": (S.tiny_config(seed=11, n_head=32, n_kv=8, ffn=2048, vocab=2560), S.build_model, Model),
             "ep_check": (S.tiny_q35_config(seed=5, n_expert=16, top_k=3), S.build_q35_model, Q35Model)}
    for name, (cfg, builder, cls) in cases.items():
        synth = builder(cfg)
        ids = np.random.default_rng(42).integers(0, cfg.vocab, 20).astype(np.int32)
        gm = cls(grp, cfg, synth.tensors)
        logits, first = gm.prefill(ids, 0)
        stream = [int(first)] + [int(t) for t in gm.generate(int(first), len(ids), 8)]
        mine = torch.from_numpy(np.concatenate([logits, np.asarray(stream, np.float32)])).cuda()
        allr = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(allr, mine)
        same = all(torch.equal(allr[0], t) for t in allr[1:])
        gm.close()
        if rank == 0:
            sm = cls(solo, cfg, synth.tensors)
            l1, f1 = sm.prefill(ids, 0)
            s1 = [int(f1)] + [int(t) for t in sm.generate(int(f1), len(ids), 8)]
            sm.close()
            err = float(np.abs(l1 - logits).max())
            out[name] = {"ranks": world, "max_abs_err_vs_one_gpu": err, "logit_range": float(l1.max() - l1.min()),
                         "ranks_identical": bool(same), "greedy_equal": s1 == stream}
    grp.close()
    if solo is not None:
        solo.close()
    return out if rank == 0 else None


def run_tp(args):
    """Tensor-parallel decode + prefill of the Llama-3-8B-shape model over all ranks of this launch (torchrun: one
    process per GPU; a single process is the TP = 1 point).
        python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 bench.py --tp --gpus 8"""
    import torch
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    r = tp_measure(args, rank, local, world, args.steps, args.warmup)
    if rank == 0:
        print(json.dumps({
            "metric": METRIC, "value": r["decode_tok_s"], "unit": UNIT, "n_gpus": world, "steps": r["steps"], "warmup": r["warmup"],
            "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"llama-3-8b-shape Q4_K_M-style ({r['layers']} layers), tensor parallel over {world} GPU(s), batch-1 greedy decode after a {r['prefill_tokens']}-token prompt, ctx {r['ctx']}",
                       "parallelism": f"tp{world}", "collectives": r["allreduce"] + " after attn_output and ffn_down, NCCL all-gather of the logits slices",
                       "l2": "each step streams this rank's weight shard (> 126 MB L2 up to tp8)"},
            "gpu_launches": r["gpu_launches"], "prefill": {"tokens": r["prefill_tokens"], "tok_per_s": r["prefill_tok_s"]},
            "decode_step": {"algorithmic_bytes_per_rank": r["algorithmic_bytes_per_rank"], "achieved_gbs_per_rank": r["achieved_gbs_per_rank"],
                            "frac_of_hbm_peak": r["frac_of_hbm_peak"], "peak_source": r["peak_source"]},
            "batch": r.get("batch"), "model_build_s": r["model_build_s"]}), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def model_figures(b, local, cfg, workload, n_prompt, n_decode=128):
    """Prefill of n_prompt random tokens, then n_decode greedy decode tokens of a random-init model of shape cfg, on one
    GPU, timed with CUDA events on the library's stream.  Returns {"workload", "decode", "prefill"}."""
    import torch
    from ggnpu_b200.backend import Model
    synth = S.build_model(cfg, device="cuda")
    model = Model(b, cfg, synth.tensors)
    del synth
    stream = torch.cuda.ExternalStream(b.stream(), device=torch.device("cuda", local))
    ids = prompt_ids(cfg, n_prompt)
    model.prefill(ids, 0, want_logits=False)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record(stream)
    _, first = model.prefill(ids, 0, want_logits=False)
    e1.record(stream)
    torch.cuda.synchronize()
    prefill_ms = e0.elapsed_time(e1)
    toks = model.generate(int(first), n_prompt, 8)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record(stream)
    toks = model.generate(int(toks[-1]), n_prompt + 8, n_decode)
    e1.record(stream)
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / n_decode
    peak, peak_kind = peaks()
    bytes_step = model.decode_bytes(n_prompt + 8 + n_decode // 2)
    model.close()
    return {"workload": workload,
            "decode": {"tok_per_s": 1000.0 / ms, "ms_per_step": ms, "algorithmic_bytes": bytes_step,
                       "achieved_gbs": bytes_step / (ms * 1e-3) / 1e9, "frac_of_hbm_peak": bytes_step / (ms * 1e-3) / 1e9 / peak, "peak_source": peak_kind},
            "prefill": {"tokens": n_prompt, "tok_per_s": n_prompt / (prefill_ms * 1e-3), "ms": prefill_ms}}


def config3_figures(b, local, n_layer=0):
    """Qwen2.5-1.5B shape, every matrix Q8_0 (28 layers, QKV bias, head_dim 128): prefill of 2048 random tokens, then 128
    greedy decode tokens, on one GPU."""
    import dataclasses
    cfg = dataclasses.replace(S.QWEN25_1P5B, ctx=2048 + 128 + 16, n_layer=n_layer or S.QWEN25_1P5B.n_layer)
    return model_figures(b, local, cfg, "qwen2.5-1.5b shape, all Q8_0, 28 layers, QKV bias: 2048-token prefill then 128 greedy decode tokens", 2048)


def lfm2_figures(b, local):
    """An lfm2 shape of about 1.2 B parameters (16 layers: 10 gated short-convolution, 6 GQA attention with QK-norm; hidden
    2048, FFN 8192, vocab 65536, Q4_K / Q6_K): prefill of 512 random tokens, then 128 greedy decode tokens, on one GPU."""
    import dataclasses
    cfg = dataclasses.replace(S.LFM2_1P2B, ctx=512 + 128 + 16)
    return model_figures(b, local, cfg, "lfm2 shape (~1.2 B: 10 short-convolution + 6 attention layers, hidden 2048, FFN 8192, vocab 65536), "
                         "Q4_K / Q6_K: 512-token prefill then 128 greedy decode tokens", 512)


def run_config5(args):
    """qwen35moe shape (hidden 2048, 256 experts top-8 + shared expert of 512, every 4th layer gated full attention with
    16 / 2 heads of 256, the others Gated DeltaNet with 16 / 32 heads of 128, vocab 248320): prompt of --q35-prompt tokens,
    then --steps greedy decode tokens.  With torchrun the experts are split over the ranks (expert parallel).
    --q35-layers bounds the layer count (40 = the full shape; the per-layer cost does not depend on it)."""
    import torch
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    line = config5_measure(args, rank, local, world, args.steps, args.warmup)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def config5_measure(args, rank, local, world, steps, warmup):
    """The measurement behind run_config5 (torch.distributed already up when world > 1): the JSON line on rank 0, None
    elsewhere."""
    import dataclasses
    import torch
    import torch.distributed as dist
    from ggnpu_b200.backend import CudaBackend, Q35Model
    cfg = dataclasses.replace(S.QWEN35MOE, n_layer=args.q35_layers, ctx=args.q35_prompt + steps + max(warmup, 3) + 8)
    b = CudaBackend(local)
    join_group(b, rank, world)
    t0 = time.perf_counter()
    synth = S.build_q35_model(cfg, device="cuda")
    model = Q35Model(b, cfg, synth.tensors)
    build_s = time.perf_counter() - t0
    del synth
    stream = torch.cuda.ExternalStream(b.stream(), device=torch.device("cuda", local))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    ids = prompt_ids(cfg, args.q35_prompt)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    _, first = model.prefill(ids, 0, want_logits=False)
    e1.record(stream)
    barrier()
    prefill_ms = e0.elapsed_time(e1)
    K, W = steps, max(warmup, 3)
    toks = model.generate(int(first), len(ids), W)
    barrier()
    launches0 = b.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    toks = model.generate(int(toks[-1]), len(ids) + W, K)
    e1.record(stream)
    barrier()
    t = torch.tensor([e0.elapsed_time(e1), prefill_ms], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, prefill_ms = float(t[0]), float(t[1])
    line = None
    if rank == 0:
        peak, peak_kind = peaks()
        bytes_step = model.decode_bytes(len(ids) + W + K // 2)
        line = ({
            "metric": METRIC, "value": K / (ms * 1e-3), "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms / K,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"qwen35moe shape, {cfg.n_layer} of 40 layers, Q4_K (Q6_K attention output and expert down), batch-1 greedy decode after a {len(ids)}-token prompt",
                       "parallelism": f"ep{world}" if world > 1 else "single GPU", "collectives": "all-reduce of the FFN row after every MoE layer (batch-1 form of dispatch / combine)" if world > 1 else "none"},
            "gpu_launches": b.launch_count() - launches0, "ms_per_token_layer": ms / K / cfg.n_layer,
            "prefill": {"tokens": len(ids), "tok_per_s": len(ids) / (prefill_ms * 1e-3), "note": "one graph replay per prompt token (the architecture is a recurrence)"},
            "decode_step": {"algorithmic_bytes_per_rank": bytes_step, "achieved_gbs_per_rank": bytes_step / (ms / K * 1e-3) / 1e9,
                            "frac_of_hbm_peak": bytes_step / (ms / K * 1e-3) / 1e9 / peak, "peak_source": peak_kind},
            "model_build_s": build_s})
    model.close()
    b.close()
    return line


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256, help="timed decode steps (256 = the benchmark configuration's decode length)")
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--prompt-len", type=int, default=128, help="prompt tokens before the timed decode (128 = the benchmark config)")
    ap.add_argument("--prefill-long", type=int, default=2048, help="token count of the long-prompt prefill figure")
    ap.add_argument("--micro-deltanet", action="store_true", help="Gated DeltaNet step microbenchmark (qwen35moe shape)")
    ap.add_argument("--micro-moe", action="store_true", help="MoE FFN decode microbenchmark (qwen35moe expert shapes)")
    ap.add_argument("--moe-experts", type=int, default=256)
    ap.add_argument("--micro-allreduce", action="store_true", help="latency of the tensor-parallel all-reduce (torchrun)")
    ap.add_argument("--tp", action="store_true", help="tensor-parallel benchmark of the 8B-shape model over the ranks of this launch")
    ap.add_argument("--tp-nccl-only", action="store_true", help="keep every all-reduce on NCCL (no peer-memory one-shot kernel)")
    ap.add_argument("--tp-ctx", type=int, default=4352)
    ap.add_argument("--tp-batch", type=int, default=16, help="sequences of the batched decode leg (1 = skip it)")
    ap.add_argument("--tp-prompt", type=int, default=4096)
    ap.add_argument("--tp-layers", type=int, default=0, help="layers to build (0 = all 32)")
    ap.add_argument("--config5", action="store_true", help="qwen35moe-shape decode benchmark (expert parallel under torchrun)")
    ap.add_argument("--config3", action="store_true", help="Qwen2.5-1.5B shape, all Q8_0: 2048-token prefill and 128 decode tokens on one GPU")
    ap.add_argument("--lfm2", action="store_true", help="lfm2 shape (~1.2 B, short-convolution + attention layers): 512-token prefill and 128 decode tokens on one GPU")
    ap.add_argument("--c3-layers", type=int, default=0, help="layers to build for --config3 (0 = all 28; fewer for profiling)")
    ap.add_argument("--q35-layers", type=int, default=40)
    ap.add_argument("--q35-prompt", type=int, default=128)
    ap.add_argument("--no-extras", action="store_true", help="skip the extra figures of the default run (the Qwen2.5-1.5B, Llama-3-8B and qwen35moe shapes on one GPU; tensor / expert parallel figures and checks under torchrun)")
    ap.add_argument("--micro", action="store_true", help="quantised-matmul microbenchmark instead of the decode benchmark")
    ap.add_argument("--types", default="Q4_0,Q8_0,Q4_K,Q6_K,IQ4_XS")
    ap.add_argument("--shapes", default="2048x2048,8192x2048,2048x8192,8960x1536")
    ap.add_argument("--ms", default="1,16")
    ap.add_argument("--dual", action="store_true")
    ap.add_argument("--reps", type=int, default=5)
    args = ap.parse_args()
    if args.tp:
        run_tp(args)
        return
    if args.config3:
        from ggnpu_b200.backend import CudaBackend
        b = CudaBackend(0)
        print(json.dumps({"config3": config3_figures(b, 0, args.c3_layers)}), flush=True)
        b.close()
        return
    if args.lfm2:
        from ggnpu_b200.backend import CudaBackend
        b = CudaBackend(0)
        print(json.dumps({"lfm2": lfm2_figures(b, 0)}), flush=True)
        b.close()
        return
    if args.config5:
        run_config5(args)
        return
    if args.micro_allreduce:
        run_micro_allreduce(args)
        return
    if args.micro_deltanet:
        run_micro_deltanet(args)
        return
    if args.micro_moe:
        run_micro_moe(args)
        return
    if args.micro:
        run_micro(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
