"""Benchmark of the compressed-KV decode-on-codes attention path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl native|reference]

Workload (N = 1): the Llama-3-8B-shaped decode configuration — 32 layers, 32 query / 8 KV
heads (GQA 4), head_dim 128, K4 asymmetric-NF4 keys with 2 % fp16 outliers, V3 PolarQuant
values, hot window 512, batch 32, uniform context 8192, fp16 K/V, bf16 queries.  A "step"
is one decode step of attention over all layers and sequences.  For N > 1 every rank holds
its own batch of 32 sequences (batch sharding: no collective on the attention path, weak
scaling); launch with ``python -m torch.distributed.run --nproc-per-node N bench.py --gpus N``.

One JSON line is printed by rank 0:
  value     compressed-KV bytes read per second by decode attention, whole job, inputs
            resident in HBM (GB/s); tokens_per_s = sequences advanced per second
  e2e       the same metric through the public API with HOST buffers: every step copies
            the step's q and new K/V token from pinned host memory, appends, decodes and
            copies the attention output back
  roofline  HBM roofline of the attention kernel, timed with CUDA events on its stream
  cpu_baseline  the C restatement of the reference's dequantise-then-attend path timed on
            the host cores on a bounded sample of the same workload

``--impl reference`` times that CPU path alone (the reference is a Python/numpy package
that cannot travel to the GPU box; the multi-threaded C restatement in oracle/ stands in).
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "decode_attn_compressed_kv_GBps"
UNIT = "GB/s"


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=20)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", default="native", choices=["native", "reference"])
    p.add_argument("--model", default="llama-3-8b")
    p.add_argument("--layers", type=int, default=0, help="override the layer count")
    p.add_argument("--batch", type=int, default=32)
    p.add_argument("--ctx", type=int, default=8192)
    p.add_argument("--hot-window", type=int, default=512)
    p.add_argument("--target", default="balanced")
    p.add_argument("--cpu-seconds", type=float, default=12.0)
    p.add_argument("--no-cpu-baseline", action="store_true")
    p.add_argument("--no-e2e", action="store_true")
    p.add_argument("--seed", type=int, default=0)
    return p.parse_args()


# ------------------------------------------------------------------------------------ #
# clocks                                                                                #
# ------------------------------------------------------------------------------------ #

class ClockSampler:
    """Samples nvidia-smi SM clocks and throttle reasons while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self._stop = threading.Event()
        self._t = None

    def _run_nvml(self) -> bool:
        """Reads the same fields through NVML (read-only queries, a few microseconds each, so
        a short timed region still gets many samples).  False if NVML is not usable."""
        try:
            import pynvml as nv

            nv.nvmlInit()
            try:  # the device this process computes on, whatever the visible-device order
                import torch

                h = nv.nvmlDeviceGetHandleByUUID("GPU-" + str(
                    torch.cuda.get_device_properties(torch.cuda.current_device()).uuid))
            except Exception:  # noqa: BLE001
                h = nv.nvmlDeviceGetHandleByIndex(self.index)
            mx = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
            get_reasons = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) \
                or nv.nvmlDeviceGetCurrentClocksThrottleReasons
            nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)
            get_reasons(h)
        except Exception:  # noqa: BLE001
            return False
        bits = ((0x8, 2), (0x40, 3), (0x20, 4), (0x4, 5))  # hw, hw thermal, sw thermal, power cap
        while not self._stop.is_set():
            try:
                r = get_reasons(h)
                row = [str(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)), str(mx),
                       "Not Active", "Not Active", "Not Active", "Not Active"]
                for bit, col in bits:
                    if r & bit:
                        row[col] = "Active"
                self.samples.append(row)
            except Exception:  # noqa: BLE001 - sampling must never break the benchmark
                pass
            self._stop.wait(0.005)
        return True

    def _run(self):
        if self._run_nvml():
            return
        while not self._stop.is_set():
            try:
                out = subprocess.run(
                    ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                     "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5)
                if out.returncode == 0 and out.stdout.strip():
                    self.samples.append([x.strip() for x in out.stdout.strip().split(",")])
            except Exception:  # noqa: BLE001 - sampling must never break the benchmark
                pass
            self._stop.wait(0.02)

    def __enter__(self):
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._t.join(timeout=10)

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            try:
                sm.append(float(s[0]))
                mx.append(float(s[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, s[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": float(np.median(sm)) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


# ------------------------------------------------------------------------------------ #
# CPU path (C restatement of the reference's dequantise-then-attend)                     #
# ------------------------------------------------------------------------------------ #

def cpu_path(args, cfg, seconds: float):
    """Times dequantise-then-attend decode steps of single sequences of the workload on the
    host cores until ``seconds`` have passed.  Returns a dict for the JSON line."""
    from oracle import c_oracle as co
    from oracle import tq_oracle as orc
    from turboquant_pro_b200.synth import make_kv, make_q

    h, hq, d = cfg.n_kv_heads, cfg.n_q_heads, cfg.head_dim
    w, vb = args.hot_window, cfg.value_bits
    n = args.ctx
    f = orc.block_tokens(w)
    nb = orc.n_cold_blocks(n, w)
    pi, pi_t = orc.rotation(d, args.seed)
    cent, bnd = orc.value_tables(d, vb)
    k, v = make_kv(args.seed, h, n, dtype=np.float16)
    k = k.astype(np.float32)
    v = v.astype(np.float32)
    q = make_q(args.seed, hq)
    kout = orc.outlier_count(f, 0.02)
    # encode once (not timed): the cache state the decode step reads
    kb, vbk = [], []
    for b in range(nb):
        xs = np.ascontiguousarray(np.moveaxis(k[b * f:(b + 1) * f], 0, 1))
        vs = np.ascontiguousarray(np.moveaxis(v[b * f:(b + 1) * f], 0, 1))
        kb.append(co.encode_keys(xs, kout))
        vbk.append(co.encode_values(vs, pi_t, bnd))
    hot_k = np.ascontiguousarray(np.moveaxis(k[nb * f:], 0, 1))
    hot_v = np.ascontiguousarray(np.moveaxis(v[nb * f:], 0, 1))
    n_out = sum(b["out_idx"].size for b in kb)
    step_bytes = (h * nb * (f * d * 4 // 8 + f * d * vb // 8 + 4 * f + 8 * d) + 6 * n_out
                  + h * (n - nb * f) * d * 2 * 2 + hq * d * 8)

    def one_step():
        ks = [co.dequant_keys(b["codes"], b["scale"], b["mean"], b["out_idx"], b["out_val"])
              for b in kb] + [hot_k]
        vs = [co.dequant_values(b["codes"], b["norms"], cent, pi) for b in vbk] + [hot_v]
        return co.attention(q, np.concatenate(ks, axis=1), np.concatenate(vs, axis=1))

    one_step()
    t0 = time.perf_counter()
    steps = 0
    while True:
        one_step()
        steps += 1
        el = time.perf_counter() - t0
        if el >= seconds or steps >= 1000:
            break
    per_step = el / steps
    return {
        "value": step_bytes / per_step / 1e9, "unit": UNIT, "cores": co.num_threads(),
        "kind": "port",
        "sample": (f"{steps} decode steps of 1 sequence x 1 layer ({h} KV heads, ctx {n}, "
                   f"{nb} cold blocks + {n - nb * f} hot) through the C restatement of "
                   f"get_keys/get_values + fp32 attention; {per_step * 1e3:.1f} ms per "
                   "sequence-layer step"),
        "ms_per_seq_layer_step": per_step * 1e3,
        "tokens_per_s": 1.0 / (per_step * cfg.n_layers),
    }


def run_reference(args):
    """--impl reference: the CPU path alone, on rank 0."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from turboquant_pro_b200 import AutoConfig

    cfg = AutoConfig.from_pretrained(args.model, target=args.target)
    if args.layers:
        cfg.n_layers = args.layers
    budget = max(5.0, min(60.0, args.cpu_seconds * (args.steps + args.warmup) / 23.0))
    cb = cpu_path(args, cfg, budget)
    line = {
        "impl": "reference", "metric": METRIC, "value": cb["value"], "unit": UNIT,
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": cb["ms_per_seq_layer_step"] * cfg.n_layers * args.batch,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "tokens_per_s": cb["tokens_per_s"],
        "config": workload_config(args, cfg, args.gpus),
        "cpu_baseline": {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": cb["value"], "unit": UNIT, "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(args, cfg, n_gpus):
    return {
        "workload": (f"{args.model} decode attention on compressed KV: {cfg.n_layers} layers, "
                     f"{cfg.n_q_heads}q/{cfg.n_kv_heads}kv heads, head_dim {cfg.head_dim}, "
                     f"K{cfg.key_bits} asym-NF4 + 2% outliers / V{cfg.value_bits}, "
                     f"hot_window {args.hot_window}, batch {args.batch} per GPU, ctx {args.ctx}"),
        "global_batch": args.batch * n_gpus, "ctx": args.ctx, "layers": cfg.n_layers,
        "parallelism": f"batch-shard x{n_gpus} (no collective on the attention path)",
        "l2": "per-step working set (all layers) exceeds L2; no flush needed",
        "kv_dtype": "f16", "q_dtype": "bf16",
    }


# ------------------------------------------------------------------------------------ #
# native arm                                                                            #
# ------------------------------------------------------------------------------------ #

def run_native(args):
    import torch
    import torch.distributed as dist

    from turboquant_pro_b200 import AutoConfig

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py --impl native needs a CUDA device (no CPU fallback)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    cfg = AutoConfig.from_pretrained(args.model, target=args.target)
    if args.layers:
        cfg.n_layers = args.layers
    L, B, H, HQ, D = cfg.n_layers, args.batch, cfg.n_kv_heads, cfg.n_q_heads, cfg.head_dim
    e2e_steps = 0 if args.no_e2e else args.steps + args.warmup
    ctx = cfg.build_context(n_seqs=B, max_tokens_per_seq=args.ctx + e2e_steps + 8,
                            hot_window=args.hot_window, seed=args.seed, kv_dtype="float16",
                            device=local)

    # fill the caches: channel-scaled Gaussians with 2 % x20 key channels, generated on device
    gen = torch.Generator(device=dev)
    gen.manual_seed(args.seed * 1000 + rank)
    n_out_ch = int(round(0.02 * D))
    chunk = 2048
    for layer in range(L):
        sk = torch.exp(0.5 * torch.randn((H, D), generator=gen, device=dev))
        sv = torch.exp(0.5 * torch.randn((H, D), generator=gen, device=dev))
        for hh in range(H):
            idx = torch.randperm(D, generator=gen, device=dev)[:n_out_ch]
            sk[hh, idx] *= 20.0
        for t0 in range(0, args.ctx, chunk):
            t1 = min(args.ctx, t0 + chunk)
            k = (torch.randn((B, t1 - t0, H, D), generator=gen, device=dev) * sk).half()
            v = (torch.randn((B, t1 - t0, H, D), generator=gen, device=dev) * sv).half()
            ctx.append(layer, k, v)
        del k, v
    torch.cuda.synchronize()
    if ctx.status() != 0:
        raise SystemExit("outlier pool overflow while filling the cache")
    q_all = torch.randn((L, B, HQ, D), generator=gen, device=dev).to(torch.bfloat16)
    out_all = torch.empty((L, B, HQ, D), dtype=torch.float32, device=dev)
    step_bytes = sum(ctx.decode_bytes(layer) for layer in range(L))

    def step():
        for layer in range(L):
            ctx.decode(layer, q_all[layer], out=out_all[layer])

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    launches_per_step = L * ctx.last_launches()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clk:
        e0.record()
        for _ in range(args.steps):
            step()
        e1.record()
        barrier()
        # the same K steps once more with an event pair around every kernel launch (on the
        # launching stream, inside the library): the per-kernel times of the roofline.  Kept
        # out of the region above because the events stop the two kernels of a call from
        # overlapping.
        ctx.profile(True)
        for _ in range(args.steps):
            step()
        barrier()
        attn_ms, comb_ms, n_calls = ctx.profile_read()
        ctx.profile(False)
    ms = e0.elapsed_time(e1)
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_max = float(t.item())
    ms_per_step = ms_max / args.steps
    value = world * step_bytes / (ms_per_step * 1e-3) / 1e9

    # ---- end to end through the public API with host buffers -------------------------
    e2e = None
    if not args.no_e2e:
        q_host = torch.randn((L, B, HQ, D)).to(torch.bfloat16).pin_memory()
        k_host = (torch.randn((L, B, 1, H, D))).half().pin_memory()
        v_host = (torch.randn((L, B, 1, H, D))).half().pin_memory()
        out_host = torch.empty((L, B, HQ, D), dtype=torch.float32).pin_memory()

        # Copies run on their own stream so that a layer's inputs arrive while the layer before
        # it is attended and its output leaves while the next one runs; device buffers are
        # double-buffered and handed over with events.
        copy_stream = torch.cuda.Stream(device=dev)
        main_stream = torch.cuda.current_stream(dev)
        qd = [torch.empty((B, HQ, D), dtype=torch.bfloat16, device=dev) for _ in range(2)]
        kd = [torch.empty((B, 1, H, D), dtype=torch.float16, device=dev) for _ in range(2)]
        vd = [torch.empty((B, 1, H, D), dtype=torch.float16, device=dev) for _ in range(2)]
        od = [torch.empty((B, HQ, D), dtype=torch.float32, device=dev) for _ in range(2)]
        ev_in = [torch.cuda.Event() for _ in range(2)]
        ev_done = [torch.cuda.Event() for _ in range(2)]
        ev_out = [torch.cuda.Event() for _ in range(2)]

        def fetch(layer):
            b = layer & 1
            with torch.cuda.stream(copy_stream):
                copy_stream.wait_event(ev_done[b])  # the layer that used these buffers is done
                qd[b].copy_(q_host[layer], non_blocking=True)
                kd[b].copy_(k_host[layer], non_blocking=True)
                vd[b].copy_(v_host[layer], non_blocking=True)
                ev_in[b].record(copy_stream)

        def e2e_step():
            fetch(0)
            for layer in range(L):
                b = layer & 1
                if layer + 1 < L:
                    fetch(layer + 1)
                main_stream.wait_event(ev_in[b])
                main_stream.wait_event(ev_out[b])  # the output buffer has left for the host
                ctx.append(layer, kd[b], vd[b])
                ctx.decode(layer, qd[b], out=od[b])
                ev_done[b].record(main_stream)
                with torch.cuda.stream(copy_stream):
                    copy_stream.wait_event(ev_done[b])
                    out_host[layer].copy_(od[b], non_blocking=True)
                    ev_out[b].record(copy_stream)
            main_stream.wait_stream(copy_stream)

        for _ in range(args.warmup):
            e2e_step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            e2e_step()
        barrier()
        el = time.perf_counter() - t0
        t = torch.tensor([el], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        el = float(t.item())
        e2e_bytes = sum(ctx.decode_bytes(layer) for layer in range(L))
        h2d = q_host.numel() * 2 + k_host.numel() * 2 + v_host.numel() * 2
        e2e = {"value": world * e2e_bytes / (el / args.steps) / 1e9, "unit": UNIT,
               "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(out_host.numel() * 4),
               "ms_per_step": el / args.steps * 1e3,
               "tokens_per_s": world * B / (el / args.steps),
               "path": "per layer: pinned q + new K/V token H2D, KVContext.append, "
                       "KVContext.decode, output D2H; copies on a second stream, "
                       "double-buffered"}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:  # noqa: BLE001
        pass
    peak = float(peaks.get("hbm_gbs", 6650.0))
    layer_bytes = step_bytes / L
    attn_ms_avg = attn_ms / max(n_calls, 1)
    achieved = layer_bytes / (attn_ms_avg * 1e-3) / 1e9 if attn_ms_avg > 0 else None
    roofline = {
        "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
        "frac": achieved / peak if achieved else None,
        "peak_source": "measured (MEASURED_PEAKS.json hbm_gbs)" if peaks else "fallback 6650",
        "frac_of_nominal_8TBps": achieved / 8000.0 if achieved else None,
        "kernel": "decode attention kernel (one launch per layer)",
        "algorithmic_bytes_per_launch": layer_bytes,
        "avg_launch_ms": attn_ms_avg, "combine_avg_launch_ms": comb_ms / max(n_calls, 1),
        "launches_timed": n_calls,
        # dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture of this kernel at the
        # default workload (335.0 MB + 6.8 MB per launch), scaled by the bytes a launch covers
        "traffic": 341.8e6 * layer_bytes / 333578240.0,
        "traffic_source": "ncu capture of the default workload (profiles/), scaled by "
                          "algorithmic bytes",
        "timing": "CUDA events around every launch on the launching stream, in a second pass "
                  "of the same K steps right after the timed region",
    }
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16",
        "data": "synthetic", "tokens_per_s": world * B / (ms_per_step * 1e-3),
        "config": workload_config(args, cfg, world),
        "bytes_per_step_per_gpu": step_bytes,
        "roofline": roofline, "clocks": clk.summary(), "e2e": e2e,
        "gpu_launches": launches_per_step * args.steps,
        "device_bytes": ctx.device_bytes(),
    }
    if world == 1 and not args.no_cpu_baseline:
        cb = cpu_path(args, cfg, args.cpu_seconds)
        line["cpu_baseline"] = {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_native(args)


if __name__ == "__main__":
    main()
