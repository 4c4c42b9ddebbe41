#!/usr/bin/env python
"""Benchmark of the decode hot path: LLaMA-7B-shape f16, batch 1, greedy decode after a
128-token prefill (BASELINE.json configs[1]); tensor-parallel over N GPUs for N > 1.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload 7b|13b|30b|65b|tiny] [--impl reference]

A "step" is one decoded token. Prints ONE JSON line (rank 0).
 * value        tokens/s with the token fed back on the device (inputs resident in HBM),
                device-timed with CUDA events on the library's stream, max over ranks;
 * e2e          the same loop through Transformer.forward with HOST tokens in and HOST logits
                out every step (pinned staging copies inside the timed region), arg-max on the host;
 * roofline     algorithmic bytes per decoded token / time per token against the measured HBM peak;
 * cpu_baseline the CPU oracle (a restatement of the reference's AVX2 path) timed on this box's
                host cores on a bounded sample.
With --impl reference only the CPU oracle runs (the reference is Rust and cannot be built here).
"""
import argparse
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


def algorithmic_bytes_per_token(cfg, t_mean, f16=True, head_bytes=4):
    """Bytes one decoded token must read: every per-layer weight once, the f32 vocabulary head,
    the live KV prefix (t_mean positions) plus the appended position, and the norm gains."""
    d, L, F, V = cfg["dim"], cfg["n_layers"], cfg["ffn"], cfg["vocab"]
    bw = 2 if f16 else 4
    weights = L * (4 * d * d + 3 * d * F) * bw + V * d * head_bytes
    kv = L * 2 * t_mean * d * bw + L * 2 * d * bw
    small = (2 * L + 1) * d * 4 + d * 4
    return weights + kv + small


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
        for ln in self.lines:
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
                "reasons": sorted(reasons), "samples": len(sm)}


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


def time_oracle(cfg, n_layers_list, steps, prompt_len, threads):
    """Times the CPU oracle's decode step at reduced depths; returns ms/token extrapolated
    linearly in depth to cfg['n_layers'] and the description of the sample."""
    from oracle import oracle as O
    per_depth = {}
    for nl in n_layers_list:
        sub = dict(cfg); sub["n_layers"] = nl
        m = O.OracleTransformer(sub["dim"], nl, sub["n_heads"], sub["ffn"], sub["vocab"], sub["norm_eps"], prompt_len + steps + 2,
                                sub["f16"], nthreads=threads)
        for kind, layer in S.tensor_list(sub):
            m.set_tensor(kind, layer, S.synth_tensor(kind, layer, sub))
        c = m.make_caches()
        toks = S.synth_tokens(prompt_len, sub["vocab"])
        tok = int(toks[0])
        pos = 0
        # fill the cache token by token is too slow for long prompts; a short prefill stands in
        logits = m.forward(toks[: min(prompt_len, 8)], 0, c)
        pos = min(prompt_len, 8)
        tok = int(np.argmax(logits))
        m.forward([tok], pos, c)  # first decode step is not timed (as in src/rllama_main.rs:905-921)
        pos += 1
        t0 = time.perf_counter()
        for _ in range(steps):
            logits = m.forward([tok], pos, c)
            tok = int(np.argmax(logits))
            pos += 1
        per_depth[nl] = (time.perf_counter() - t0) * 1e3 / steps
        del m, c
    (a, ta), (b, tb) = sorted(per_depth.items())[0], sorted(per_depth.items())[-1]
    slope = (tb - ta) / (b - a) if b != a else tb / b
    full = ta + slope * (cfg["n_layers"] - a)
    sample = "%s-shape %s decode step on the CPU oracle, %s of %d layers + f32 head, %d tokens each at context ~%d, " \
             "extrapolated linearly in depth" % (cfg["name"], "f16" if cfg["f16"] else "f32", "/".join(str(k) for k in sorted(per_depth)),
                                                  cfg["n_layers"], steps, pos)
    return full, sample, per_depth


def run_reference(args, cfg, rank):
    if rank != 0:
        return
    from oracle import oracle as O
    threads = O.hw_threads()
    depths = [1, 3] if cfg["n_layers"] >= 3 else [cfg["n_layers"]]
    ms_list = []
    per = None
    for _ in range(max(1, min(args.steps, 3))):
        ms, sample, per = time_oracle(cfg, depths, 3, 16, threads)
        ms_list.append(ms)
    ms = statistics.median(ms_list)
    val = 1e3 / ms
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f16" if cfg["f16"] else "f32", "data": "synthetic",
        "config": {"workload": workload_name(cfg), "note": "reference is Rust (no toolchain here): the CPU oracle port is timed instead"},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_name(cfg):
    return "llama-%s-shape %s batch-1: %d-token prompt prefill then greedy decode (dim %d, %d layers, %d heads, ffn %d, vocab %d)" % (
        cfg["name"], "f16" if cfg["f16"] else "f32", cfg["prompt"], cfg["dim"], cfg["n_layers"], cfg["n_heads"], cfg["ffn"], cfg["vocab"])


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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--workload", default="7b")
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--layers", type=int, default=0, help="override depth (debugging; makes the number invalid as a headline)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--profile-kernels", action="store_true", help="also time each kernel class with events (eager, untimed extra pass)")
    ap.add_argument("--f32", action="store_true", help="keep the weights and caches in f32 (the reference without --f16)")
    ap.add_argument("--gemm-sweep", action="store_true",
                    help="time the prefill GEMM (rlb_matrix_mul_inplace_transposed, f16) over prompt lengths and layer shapes, then exit")
    args = ap.parse_args()
    if args.gemm_sweep:
        return gemm_sweep()

    cfg = dict(S.CONFIGS[args.workload]); cfg["name"] = args.workload
    if args.f32:
        cfg["f16"] = False
    if args.layers:
        cfg["n_layers"] = args.layers
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
    from rllama_b200 import Cuda, DataSettings, Transformer

    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    P, K, Wm = cfg["prompt"], args.steps, args.warmup
    max_seq = max(cfg["max_seq_len"], P + Wm + K + 1)
    cl = Cuda(verbose=False, nth_device=local_rank)
    ds = DataSettings(cl=cl)
    if cfg["f16"]:
        ds = ds.force_f16()
    model = Transformer(cfg["dim"], cfg["n_layers"], cfg["n_heads"], cfg["ffn"], cfg["vocab"], max_seq, cfg["norm_eps"], ds,
                        tp_rank=rank, tp_size=world)
    for kind, layer, t in torch_weights(cfg, device):
        model.set_tensor(kind, layer, t)
        del t
    model.finalize()
    torch.cuda.empty_cache()
    if world > 1:
        ids = [Transformer.nccl_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        model.nccl_init(ids[0])
        tp_mode = os.environ.get("RLB_TP_MODE", "push")
        if tp_mode == "push":
            handles = [None] * world
            dist.all_gather_object(handles, model.peer_export())
            model.peer_import(handles)
            model.set_tp_mode("push")

    prompt = S.synth_tokens(P, cfg["vocab"])

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        cl.flush()

    # ---- device-resident loop ("value") ---------------------------------------------------
    # the first prefill also pays for buffer allocation and module loading: time the second one
    scratch_caches = model.make_caches()
    model.forward_greedy(prompt, 0, scratch_caches)
    scratch_caches.free()
    caches = model.make_caches()
    barrier()
    t0 = time.perf_counter()
    first = model.forward_greedy(prompt, 0, caches)
    cl.flush()
    prefill_ms = (time.perf_counter() - t0) * 1e3
    warm_tokens, _ = model.decode_greedy(first, P, Wm, caches)
    sampler = ClockSampler(local_rank)
    barrier()
    launches0 = cl.kernel_launches()
    sampler.start()
    tokens, dev_ms = model.decode_greedy(int(warm_tokens[-1]), P + Wm, K, caches)
    barrier()
    clocks = sampler.stop()
    launches = cl.kernel_launches() - launches0
    if world > 1:
        t = torch.tensor([dev_ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dev_ms = float(t.item())
    ms_per_token = dev_ms / K
    value = 1e3 / ms_per_token

    # ---- end-to-end loop through Transformer.forward with host buffers ---------------------
    e2e = None
    if not args.no_e2e:
        c2 = model.make_caches()
        logits = model.forward(prompt, 0, c2)
        tok = int(np.argmax(logits))
        pos = P
        for _ in range(Wm):
            logits = model.forward([tok], pos, c2); tok = int(np.argmax(logits)); pos += 1
        barrier()
        t0 = time.perf_counter()
        for _ in range(K):
            logits = model.forward([tok], pos, c2)
            tok = int(np.argmax(logits))
            pos += 1
        barrier()
        e2e_ms = (time.perf_counter() - t0) * 1e3
        if world > 1:
            t = torch.tensor([e2e_ms], device=device, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_ms = float(t.item())
        e2e = {"value": 1e3 * K / e2e_ms, "unit": UNIT, "ms_per_token": e2e_ms / K, "h2d_bytes_per_step": 8,
               "d2h_bytes_per_step": 4 * cfg["vocab"]}
        c2.free()

    kernels = None
    if args.profile_kernels:
        # eager pass with events around every kernel class (all ranks run it; rank 0 reports). Under
        # tensor parallelism a class's time includes waiting for the other ranks' partial sums.
        model.set_option("profile", 1)
        c3 = model.make_caches()
        f3 = model.forward_greedy(prompt, 0, c3)
        model.decode_greedy(f3, P, 16, c3)
        n = model.get_stat("prof_steps")
        kernels = {k: model.get_stat("prof_ms_" + k) / n for k in ("qkv", "attn", "wo", "w13", "w2", "head", "argmax", "comm")}
        model.set_option("profile", 0)
        c3.free()

    if rank == 0:
        # prefill arithmetic: 2 n (4 d^2 + 3 d F) per layer + causal attention + the last row's head
        d_, F_, L_, V_ = cfg["dim"], cfg["ffn"], cfg["n_layers"], cfg["vocab"]
        prefill_flops = 2.0 * P * L_ * (4 * d_ * d_ + 3 * d_ * F_) + 2.0 * L_ * P * (P + 1) * d_ + 2.0 * V_ * d_
        t_mean = P + Wm + (K + 1) / 2.0
        alg = algorithmic_bytes_per_token(cfg, t_mean, cfg["f16"])
        peak, peak_kind = measured_peak_gbs()
        achieved = alg / (ms_per_token * 1e-3) / 1e9 / world  # per GPU
        traffic = None
        tp = os.path.join(ROOT, "profiles", "decode_step_7b_f16_traffic.txt")
        if os.path.exists(tp) and args.workload == "7b" and cfg["f16"] and world == 1 and not args.layers:
            # dram__bytes_read.sum + dram__bytes_write.sum per decoded token, from the ncu capture
            # summarised beside that file
            for ln in open(tp):
                if ln.startswith("dram_bytes_per_token"):
                    traffic = int(ln.split("=")[1])
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": Wm,
            "ms_per_step": ms_per_token, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f16" if cfg["f16"] else "f32", "data": "synthetic",
            "config": {"workload": workload_name(cfg), "parallelism": "tp%d" % world, "exchange": (os.environ.get("RLB_TP_MODE", "push") if world > 1 else "none"), "context_start": P + Wm, "context_end": P + Wm + K,
                       "l2": "inputs larger than L2 (every step streams all weights)", "prefill_ms": prefill_ms,
                       "prefill_tflops_per_gpu": prefill_flops / (prefill_ms * 1e-3) / 1e12 / world,
                       "first_tokens": [int(first)] + [int(t) for t in tokens[:4]]},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": traffic, "peak_source": peak_kind, "algorithmic_bytes_per_token": alg,
                         "launch": "one decode step (one CUDA-graph launch, %d kernels)" % int(model.get_stat("kernels_per_step"))},
            "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks,
        }
        if kernels:
            line["kernel_ms"] = kernels
        if world == 1 and not args.no_cpu_baseline:
            from oracle import oracle as O
            threads = O.hw_threads()
            ms, sample, _ = time_oracle(cfg, [1, 3] if cfg["n_layers"] >= 3 else [cfg["n_layers"]], 3, 16, threads)
            line["cpu_baseline"] = {"value": 1e3 / ms, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
