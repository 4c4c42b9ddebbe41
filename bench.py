#!/usr/bin/env python
"""Benchmark of the decode hot path: LLaMA-7B-shape f16, batch 1, greedy decode after a
128-token prompt prefill; tensor-parallel over N GPUs for N > 1.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload 7b|13b|30b|65b|tiny] [--impl reference]

A "step" is one decoded token. Prints ONE JSON line (rank 0).
 * value        tokens/s with the token fed back on the device (inputs resident in HBM),
                device-timed with CUDA events on the library's stream, max over ranks;
 * e2e          the same loop through Transformer.forward with HOST tokens in and HOST logits
                out every step (pinned staging copies inside the timed region), arg-max on the host;
 * roofline     algorithmic bytes per decoded token / time per token against the measured HBM peak;
 * cpu_baseline the CPU oracle (a restatement of the reference's AVX2 path) at the full depth of the
                workload: the real prompt is prefilled, then decode steps are timed on this box's
                host cores (mean without the first token, as src/rllama_main.rs:905-921 does); its
                greedy tokens are compared with the GPU's on the same weights;
 * config.also  (N >= 2, default workload) a second measurement on the 65B shape: 1792-token prompt,
                decode at context ~1800.
With --impl reference only the CPU oracle runs (the reference is Rust and cannot be built here).
"""
import argparse
import hashlib
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

from rllama_b200 import synthetic as S  # noqa: E402

METRIC = "decode_tokens_per_s"
UNIT = "tokens/s"
NOMINAL_HBM_GBS = 8000.0   # the per-GPU figure the target fractions were first stated against
CPU_TIMED_STEPS = 24       # decode steps the CPU oracle is timed on (three groups of eight)


def algorithmic_bytes_per_token(cfg, t_mean, f16=True, head_bytes=4):
    """Bytes one decoded token must read: every per-layer weight once, the f32 vocabulary head,
    the live KV prefix (t_mean positions) plus the appended position, and the norm gains."""
    d, L, F, V = cfg["dim"], cfg["n_layers"], cfg["ffn"], cfg["vocab"]
    bw = 2 if f16 else 4
    weights = L * (4 * d * d + 3 * d * F) * bw + V * d * head_bytes
    kv = L * 2 * t_mean * d * bw + L * 2 * d * bw
    small = (2 * L + 1) * d * 4 + d * 4
    return weights + kv + small


def prefill_flops(cfg, P):
    """2 n (4 d^2 + 3 d F) per layer + causal attention + the last row's head."""
    d, F, L, V = cfg["dim"], cfg["ffn"], cfg["n_layers"], cfg["vocab"]
    return 2.0 * P * L * (4 * d * d + 3 * d * F) + 2.0 * L * P * (P + 1) * d + 2.0 * V * d


def measured_peak_gbs():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS,
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def mark(self):
        """The timed region starts here: samples before it (the warm-up steps, the same load) are used only when the
        region is shorter than the sampling period and caught none."""
        self.first = len(self.lines)

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        timed = self.lines[getattr(self, "first", 0):]
        window = "timed region" if timed else "prefill, warm-up and timed region (the timed region fell between two 100 ms samples)"
        for ln in (timed or self.lines):
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "window": window}


def torch_weights(cfg, device, seed=1234):
    """Yields (kind, layer, tensor) with seeded N(0, 0.02) f16 weights generated on `device`."""
    import torch
    for kind, layer in S.tensor_list(cfg):
        rows, cols = S.tensor_shape(kind, cfg)
        if kind in ("attention_norm", "ffn_norm", "norm"):
            yield kind, layer, torch.ones((rows, cols), dtype=torch.float32, device=device)
            continue
        g = torch.Generator(device=device)
        g.manual_seed(seed * 1000003 + S.TENSOR_KINDS[kind] * 4096 + layer)
        t = torch.empty((rows, cols), dtype=torch.float32, device=device)
        t.normal_(0.0, 0.02, generator=g)
        yield kind, layer, t.half()


def workload_name(cfg):
    return "llama-%s-shape %s batch-1: %d-token prompt prefill then greedy decode (dim %d, %d layers, %d heads, ffn %d, vocab %d)" % (
        cfg["name"], "f16" if cfg["f16"] else "f32", cfg["prompt"], cfg["dim"], cfg["n_layers"], cfg["n_heads"], cfg["ffn"], cfg["vocab"])


def workload_config(cfg, gpus):
    """The keys that name the workload; both arms print exactly these."""
    return {"workload": workload_name(cfg), "model": cfg["name"], "weights": "f16" if cfg["f16"] else "f32",
            "prompt_tokens": cfg["prompt"], "depth": cfg["n_layers"], "gpus": gpus}


# ---- CPU oracle legs --------------------------------------------------------------------------
def new_oracle(cfg, max_seq, threads):
    from oracle import oracle as O
    return O.OracleTransformer(cfg["dim"], cfg["n_layers"], cfg["n_heads"], cfg["ffn"], cfg["vocab"], cfg["norm_eps"], max_seq,
                               cfg["f16"], nthreads=threads)


def time_oracle_decode(orc, cfg, prompt, warm, timed):
    """The reference's own protocol on the CPU oracle at full depth: prefill the whole prompt, then greedy
    single-token steps; `warm` untimed steps, then `timed` steps in three equal groups. Returns (median of
    the group means in ms/token, all tokens produced, description)."""
    c = orc.make_caches()
    t0 = time.perf_counter()
    logits = orc.forward(prompt, 0, c)
    prefill_s = time.perf_counter() - t0
    pos = len(prompt)
    toks = [int(np.argmax(logits))]
    for _ in range(max(1, warm)):  # the first decode step is never timed (src/rllama_main.rs:905-921)
        logits = orc.forward([toks[-1]], pos, c); pos += 1
        toks.append(int(np.argmax(logits)))
    ctx0 = pos
    groups = []
    per = max(1, timed // 3)
    for _ in range(3):
        t0 = time.perf_counter()
        for _ in range(per):
            logits = orc.forward([toks[-1]], pos, c); pos += 1
            toks.append(int(np.argmax(logits)))
        groups.append((time.perf_counter() - t0) * 1e3 / per)
    ms = statistics.median(groups)
    sample = ("%s-shape %s on the CPU oracle at full depth (%d layers + f32 head): %d-token prompt prefilled (%.1f s), %d untimed "
              "then 3 x %d timed greedy decode steps at context %d-%d, median of the three group means (%.1f / %.1f / %.1f ms per token)"
              % (cfg["name"], "f16" if cfg["f16"] else "f32", cfg["n_layers"], len(prompt), prefill_s, max(1, warm), per, ctx0, pos,
                 groups[0], groups[1], groups[2]))
    return ms, toks, sample, {"prefill_s": prefill_s, "context_start": ctx0, "context_end": pos, "group_ms": groups}


def run_reference(args, cfg, rank):
    """--impl reference: the CPU oracle port alone, weights generated on the host."""
    if rank != 0:
        return
    import torch
    from oracle import oracle as O
    threads = O.hw_threads()
    P = cfg["prompt"]
    timed = max(3, min(args.steps, CPU_TIMED_STEPS) // 3 * 3)
    warm = max(1, min(args.warmup, 4))
    orc = new_oracle(cfg, P + warm + timed + 2, threads)
    for kind, layer, t in torch_weights(cfg, torch.device("cpu")):
        orc.set_tensor(kind, layer, t.numpy())
        del t
    prompt = S.synth_tokens(P, cfg["vocab"])
    ms, toks, sample, info = time_oracle_decode(orc, cfg, prompt, warm, timed)
    val = 1e3 / ms
    config = workload_config(cfg, args.gpus)
    config.update({"context_start": info["context_start"], "context_end": info["context_end"], "timed_steps": timed,
                   "note": "the reference is Rust (no toolchain on this box): its CPU restatement is timed, on every host thread"})
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f16" if cfg["f16"] else "f32", "data": "synthetic", "config": config,
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---- GPU legs ---------------------------------------------------------------------------------
class Dist:
    """The few collective helpers the bench needs; no-ops on one rank."""

    def __init__(self, world, device):
        self.world, self.device = world, device

    def barrier(self, cl):
        import torch
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()
        cl.flush()

    def max(self, v):
        if self.world == 1:
            return float(v)
        import torch
        import torch.distributed as dist
        t = torch.tensor([v], device=self.device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def gather(self, array):
        """Every rank's copy of a numpy array (same shape on all ranks)."""
        if self.world == 1:
            return [array]
        import torch
        import torch.distributed as dist
        t = torch.from_numpy(np.ascontiguousarray(array)).to(self.device)
        out = [torch.empty_like(t) for _ in range(self.world)]
        dist.all_gather(out, t)
        return [o.cpu().numpy() for o in out]


def build_model(cfg, max_seq, cl, rank, world, device, oracle=None):
    import torch
    import torch.distributed as dist
    from rllama_b200 import DataSettings, Transformer
    ds = DataSettings(cl=cl)
    if cfg["f16"]:
        ds = ds.force_f16()
    model = Transformer(cfg["dim"], cfg["n_layers"], cfg["n_heads"], cfg["ffn"], cfg["vocab"], max_seq, cfg["norm_eps"], ds,
                        tp_rank=rank, tp_size=world)
    for kind, layer, t in torch_weights(cfg, device):
        model.set_tensor(kind, layer, t)
        if oracle is not None:  # the same values go to the CPU oracle (the checker of the cpu_baseline leg)
            oracle.set_tensor(kind, layer, t.cpu().numpy())
        del t
    model.finalize()
    torch.cuda.empty_cache()
    if world > 1:
        ids = [Transformer.nccl_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        model.nccl_init(ids[0])
        if os.environ.get("RLB_TP_MODE", "push") == "push":
            handles = [None] * world
            dist.all_gather_object(handles, model.peer_export())
            model.peer_import(handles)
            model.set_tp_mode("push")
    return model


def measure(model, cfg, cl, D, local_rank, K, Wm, do_e2e=True):
    """Warm prefill, Wm untimed + K timed device-fed decode steps, then the host-buffer loop."""
    P = cfg["prompt"]
    prompt = S.synth_tokens(P, cfg["vocab"])
    # the first prefill also pays for buffer allocation and module loading: time the second one
    scratch = model.make_caches()
    model.forward_greedy(prompt, 0, scratch)
    scratch.free()
    caches = model.make_caches()
    sampler = ClockSampler(local_rank)   # (started early: nvidia-smi takes a while to deliver its first sample)
    sampler.start()
    D.barrier(cl)
    t0 = time.perf_counter()
    first = model.forward_greedy(prompt, 0, caches)
    cl.flush()
    prefill_ms = D.max((time.perf_counter() - t0) * 1e3)
    warm_tokens, _ = model.decode_greedy(first, P, Wm, caches)
    D.barrier(cl)
    launches0 = cl.kernel_launches()
    sampler.mark()
    tokens, dev_ms = model.decode_greedy(int(warm_tokens[-1]), P + Wm, K, caches)
    D.barrier(cl)
    clocks = sampler.stop()
    launches = cl.kernel_launches() - launches0
    dev_ms = D.max(dev_ms)
    caches.free()
    all_tokens = np.concatenate([[first], warm_tokens, tokens]).astype(np.int32)
    out = {"P": P, "prefill_ms": prefill_ms, "ms_per_token": dev_ms / K, "launches": int(launches), "clocks": clocks,
           "tokens": all_tokens, "kernels_per_step": int(model.get_stat("kernels_per_step"))}

    # every rank must have decoded the same tokens
    gathered = D.gather(all_tokens)
    out["ranks_agree_tokens"] = all(np.array_equal(gathered[0], g) for g in gathered)

    if do_e2e:
        # end-to-end loop through Transformer.forward with host buffers
        c2 = model.make_caches()
        logits = model.forward(prompt, 0, c2)
        tok = int(np.argmax(logits))
        pos = P
        for _ in range(Wm):
            logits = model.forward([tok], pos, c2); tok = int(np.argmax(logits)); pos += 1
        D.barrier(cl)
        t0 = time.perf_counter()
        for _ in range(K):
            logits = model.forward([tok], pos, c2)
            tok = int(np.argmax(logits))
            pos += 1
        D.barrier(cl)
        e2e_ms = D.max((time.perf_counter() - t0) * 1e3)
        out["e2e"] = {"value": 1e3 * K / e2e_ms, "unit": UNIT, "ms_per_token": e2e_ms / K, "h2d_bytes_per_step": 8,
                      "d2h_bytes_per_step": 4 * cfg["vocab"]}
        last_logits = logits
        # untimed replay of the first steps: the gap between the two largest logits behind each greedy token
        def margin(lg):
            top2 = np.partition(lg, -2)[-2:]
            return float(top2[1] - top2[0])
        c2.free()
        c2 = model.make_caches()
        logits = model.forward(prompt, 0, c2)
        margins, pos = [margin(logits)], P
        for _ in range(min(25, Wm + K - 1)):
            tok = int(np.argmax(logits))
            logits = model.forward([tok], pos, c2); pos += 1
            margins.append(margin(logits))
        out["margins"] = margins
        logits = last_logits
        c2.free()
        # the last step's logits, rank against rank (every rank assembles the full vocabulary)
        gl = D.gather(logits)
        out["ranks_logit_max_abs_diff"] = float(max(np.abs(g - gl[0]).max() for g in gl))
    return out


def roofline_of(cfg, m, K, Wm, world):
    t_mean = m["P"] + Wm + (K + 1) / 2.0
    alg = algorithmic_bytes_per_token(cfg, t_mean, cfg["f16"])
    peak, peak_kind = measured_peak_gbs()
    achieved = alg / (m["ms_per_token"] * 1e-3) / 1e9 / world  # per GPU
    return {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "traffic": None,
            "peak_source": peak_kind, "frac_of_nominal_8TBs": achieved / NOMINAL_HBM_GBS, "algorithmic_bytes_per_token": alg,
            "launch": "one decode step (one CUDA-graph launch, %d kernels)" % m["kernels_per_step"]}


def gemm_sweep():
    """Prefill contraction alone: out[n][M] = X[n][K] . W[M][K]^T through the tier-1 op, 20 calls per
    shape bracketed by a flush of the library's stream (wall clock; the calls are back to back)."""
    from rllama_b200 import F16, Cuda
    cl = Cuda(verbose=False, nth_device=0)
    rng = np.random.default_rng(0)
    for n in (128, 512, 1024, 2048):
        for (M, K) in ((12288, 4096), (4096, 4096), (22016, 4096), (4096, 11008), (3072, 8192), (8192, 1024)):
            W = cl.upload(rng.normal(0, 0.02, size=(M, K)).astype(np.float16))
            X = cl.upload(rng.normal(0, 1.0, size=(n, K)).astype(np.float16))
            out = cl.zeros(n, M, F16)
            for _ in range(3):
                out.matrix_mul_inplace_transposed(X, W)
            cl.flush()
            t = time.perf_counter()
            for _ in range(20):
                out.matrix_mul_inplace_transposed(X, W)
            cl.flush()
            dt = (time.perf_counter() - t) / 20
            print(json.dumps({"rows": n, "M": M, "K": K, "us": round(dt * 1e6, 1), "tflops": round(2.0 * n * M * K / dt / 1e12, 1),
                              "weight_gbs": round(M * K * 2 / dt / 1e9, 1)}), flush=True)
            W.free(); X.free(); out.free()


def gemm_trace():
    """Per-CTA timeline of the prefill GEMM (needs the timeline build: ``python -m rllama_b200.build --trace`` and
    ``RLLAMA_B200_LIB=rllama_b200/librllama_b200_trace.so``). One JSON line per shape: medians over the CTAs, us from
    the first CTA's entry; `starved` / `acc_wait` = MMA thread blocked on operand stages / on a busy accumulator."""
    import ctypes
    from rllama_b200 import F16, Cuda, _ffi
    L = _ffi.lib()
    if not hasattr(L, "rlb_debug_gemm_trace"):
        raise SystemExit("this library has no timeline: build it with `python -m rllama_b200.build --trace` and set "
                         "RLLAMA_B200_LIB=rllama_b200/librllama_b200_trace.so")
    L.rlb_debug_gemm_trace.argtypes = [ctypes.c_void_p]
    cl = Cuda(verbose=False, nth_device=0)
    rng = np.random.default_rng(0)
    block = rng.normal(0, 0.02, size=(1024, 22016)).astype(np.float16)
    for (M, K, n) in ((22016, 4096, 128), (4096, 4096, 128), (4096, 11008, 128), (12288, 4096, 128), (22016, 4096, 512),
                      (12288, 4096, 1024), (22016, 4096, 2048), (44032, 8192, 1792)):
        W = cl.upload(np.ascontiguousarray(np.tile(block[:, :K], ((M + 1023) // 1024, 1))[:M]))
        X = cl.upload(rng.normal(0, 1.0, size=(n, K)).astype(np.float16))
        out = cl.zeros(n, M, F16)
        for _ in range(4):
            out.matrix_mul_inplace_transposed(X, W)
        cl.flush()
        buf = np.zeros(256 * 16, dtype=np.uint64)
        if L.rlb_debug_gemm_trace(buf.ctypes.data_as(ctypes.c_void_p)) != 0:
            raise SystemExit("reading the trace failed")
        t = buf.reshape(256, 16).astype(np.int64)
        t = t[t[:, 0] > 0]
        t0 = t[:, 0].min()
        med = lambda v: round(float(np.median(v)) / 1e3, 2)
        print(json.dumps({"M": M, "K": K, "tokens": n, "ctas": int(len(t)), "k_blocks_per_cta": int(np.median(t[:, 10])),
                          "first_stage_us": med(t[:, 3] - t0), "starved_us": med(t[:, 5]), "acc_wait_us": med(t[:, 6]),
                          "last_mma_us": [med(t[:, 4] - t0), round(float((t[:, 4] - t0).max()) / 1e3, 2)],
                          "epilogue_end_us": [med(t[:, 8] - t0), round(float((t[:, 8] - t0).max()) / 1e3, 2)],
                          "epilogue_busy_us": med(t[:, 13]), "ring_full_us": med(t[:, 11])}), flush=True)
        W.free(); X.free(); out.free()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--workload", default="7b")
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--layers", type=int, default=0, help="override depth (debugging; makes the number invalid as a headline)")
    ap.add_argument("--prompt", type=int, default=0, help="override the prompt length (debugging)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-also", action="store_true", help="skip the second (65B-shape) measurement of multi-GPU runs")
    ap.add_argument("--profile-kernels", action="store_true", help="also time each kernel class with events (eager, untimed extra pass)")
    ap.add_argument("--f32", action="store_true", help="keep the weights and caches in f32 (the reference without --f16)")
    ap.add_argument("--gemm-sweep", action="store_true",
                    help="time the prefill GEMM (rlb_matrix_mul_inplace_transposed, f16) over prompt lengths and layer shapes, then exit")
    ap.add_argument("--gemm-trace", action="store_true",
                    help="per-CTA timeline of the prefill GEMM (timeline build of the library, see gemm_trace), then exit")
    args = ap.parse_args()
    if args.gemm_trace:
        return gemm_trace()
    if args.gemm_sweep:
        return gemm_sweep()

    cfg = dict(S.CONFIGS[args.workload]); cfg["name"] = args.workload
    if args.f32:
        cfg["f16"] = False
    if args.layers:
        cfg["n_layers"] = args.layers
    if args.prompt:
        cfg["prompt"] = args.prompt
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit("WORLD_SIZE %d does not match --gpus %d" % (world, args.gpus))

    if args.impl == "reference":
        run_reference(args, cfg, rank)
        return
    args.warmup = max(args.warmup, 3)

    import torch
    import torch.distributed as dist
    from rllama_b200 import Cuda

    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    D = Dist(world, device)

    K, Wm = args.steps, args.warmup
    cl = Cuda(verbose=False, nth_device=local_rank)
    want_cpu = world == 1 and not args.no_cpu_baseline
    oracle = None
    cpu_timed = max(3, min(K, CPU_TIMED_STEPS) // 3 * 3)
    cpu_warm = max(1, min(Wm, 4))
    if want_cpu:
        from oracle import oracle as O
        threads = O.hw_threads()
        oracle = new_oracle(cfg, cfg["prompt"] + cpu_warm + cpu_timed + 2, threads)
    max_seq = max(cfg["max_seq_len"], cfg["prompt"] + Wm + K + 1)
    model = build_model(cfg, max_seq, cl, rank, world, device, oracle)
    m = measure(model, cfg, cl, D, local_rank, K, Wm, do_e2e=not args.no_e2e)

    kernels = None
    if args.profile_kernels:
        # eager pass with events around every kernel class (all ranks run it; rank 0 reports). Under
        # tensor parallelism a class's time includes waiting for the other ranks' partial sums.
        model.set_option("profile", 1)
        c3 = model.make_caches()
        f3 = model.forward_greedy(S.synth_tokens(cfg["prompt"], cfg["vocab"]), 0, c3)
        model.decode_greedy(f3, cfg["prompt"], 16, c3)
        n = model.get_stat("prof_steps")
        kernels = {k: model.get_stat("prof_ms_" + k) / n for k in ("qkv", "attn", "wo", "w13", "w2", "head", "argmax", "comm")}
        model.set_option("profile", 0)
        c3.free()
    model.free()
    torch.cuda.empty_cache()

    # ---- second measurement: the 65B shape under tensor parallelism ---------------------------
    also = None
    if world >= 2 and args.workload == "7b" and not args.no_also and not args.layers and not args.f32:
        big = dict(S.CONFIGS["65b"]); big["name"] = "65b"
        max_seq_b = max(big["max_seq_len"], big["prompt"] + Wm + K + 1)
        model_b = build_model(big, max_seq_b, cl, rank, world, device)
        mb = measure(model_b, big, cl, D, local_rank, K, Wm, do_e2e=False)
        rb = roofline_of(big, mb, K, Wm, world)
        also = {"workload": workload_name(big), "parallelism": "tp%d" % world, "ms_per_token": mb["ms_per_token"],
                "tokens_per_s": 1e3 / mb["ms_per_token"], "context_start": mb["P"] + Wm, "context_end": mb["P"] + Wm + K,
                "frac_of_measured_peak": rb["frac"], "frac_of_nominal_8TBs": rb["frac_of_nominal_8TBs"],
                "algorithmic_bytes_per_token": rb["algorithmic_bytes_per_token"], "prefill_ms": mb["prefill_ms"],
                "prefill_tflops_per_gpu": prefill_flops(big, mb["P"]) / (mb["prefill_ms"] * 1e-3) / 1e12 / world,
                "tokens_sha1": hashlib.sha1(mb["tokens"].tobytes()).hexdigest(), "ranks_agree_tokens": mb["ranks_agree_tokens"],
                "clocks": mb["clocks"]}
        model_b.free()

    if rank == 0:
        roof = roofline_of(cfg, m, K, Wm, world)
        tp = os.path.join(ROOT, "profiles", "decode_step_7b_f16_traffic.txt")
        if os.path.exists(tp) and args.workload == "7b" and cfg["f16"] and world == 1 and not args.layers:
            # dram__bytes_read.sum + dram__bytes_write.sum per decoded token, from the ncu capture
            # summarised beside that file
            for ln in open(tp):
                if ln.startswith("dram_bytes_per_token"):
                    roof["traffic"] = int(ln.split("=")[1])
        config = workload_config(cfg, world)
        config.update({
            "parallelism": "tp%d" % world, "exchange": (os.environ.get("RLB_TP_MODE", "push") if world > 1 else "none"),
            "context_start": m["P"] + Wm, "context_end": m["P"] + Wm + K,
            "l2": "inputs larger than L2 (every step streams all weights)", "prefill_ms": m["prefill_ms"],
            "prefill_tflops_per_gpu": prefill_flops(cfg, m["P"]) / (m["prefill_ms"] * 1e-3) / 1e12 / world,
            # all decoded tokens (first after the prompt, warm-up, timed): same seed and warm-up at every N
            "tokens_sha1": hashlib.sha1(m["tokens"].tobytes()).hexdigest(), "tokens_head": [int(t) for t in m["tokens"][:26]],
            # top-2 logit gap behind each of those tokens: f16 sequences of different N part ways only at a near-tie
            "top2_margin_head": [round(x, 5) for x in m.get("margins", [])[:26]],
            "ranks_agree": {"tokens": m["ranks_agree_tokens"], "last_logits_max_abs_diff": m.get("ranks_logit_max_abs_diff")},
        })
        if also:
            config["also"] = also
        line = {
            "metric": METRIC, "value": 1e3 / m["ms_per_token"], "unit": UNIT, "n_gpus": world, "steps": K, "warmup": Wm,
            "ms_per_step": m["ms_per_token"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f16" if cfg["f16"] else "f32", "data": "synthetic", "config": config, "roofline": roof,
            "e2e": m.get("e2e"), "gpu_launches": m["launches"], "clocks": m["clocks"],
        }
        if kernels:
            line["kernel_ms"] = kernels
        if want_cpu:
            prompt = S.synth_tokens(cfg["prompt"], cfg["vocab"])
            ms, otoks, sample, _ = time_oracle_decode(oracle, cfg, prompt, cpu_warm, cpu_timed)
            line["cpu_baseline"] = {"value": 1e3 / ms, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample}
            # the oracle as checker: its greedy tokens against the GPU's on the same weights and prompt
            n = min(len(otoks), len(m["tokens"]))
            same = 0
            while same < n and int(otoks[same]) == int(m["tokens"][same]):
                same += 1
            config["oracle_check"] = {"tokens_compared": n, "identical_prefix": same,
                                      "note": "greedy tokens of the CPU oracle and the GPU path at full depth, same weights; a "
                                              "difference is possible at a near-tie of two f16 logits and ends the comparison"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
