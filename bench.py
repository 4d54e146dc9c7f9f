"""Benchmark of the compressed-KV decode-on-codes attention path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl native|reference]
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...

Headline workload: the Llama-3-8B-shaped decode configuration — 32 layers, 32 query / 8 KV
heads (GQA 4), head_dim 128, K4 asymmetric-NF4 keys with 2 % fp16 outliers, V3 PolarQuant
values, hot window 512, batch 32, uniform context 8192, fp16 K/V, bf16 queries.  A "step" is
one decode step of attention over all layers and sequences.  With N > 1 the same 32 sequences
are divided over the ranks (batch shard, no collective on the attention path: strong scaling).

One JSON line is printed by rank 0:
  value     compressed-KV bytes read per second by decode attention, whole job, inputs
            resident in HBM (GB/s); tokens_per_s = sequences advanced per second
  e2e       the same metric through the public API with HOST buffers: every step copies
            the step's q and new K/V token from pinned host memory, appends, decodes and
            copies the attention output back
  roofline  HBM roofline of the attention kernel, timed with CUDA events on its stream
  cpu_baseline  the reference's own numpy path (get_keys / get_values + float32 attention)
            timed on the host cores on a bounded sample of the same workload
  cfg2, cfg3, cfg4   the other multi-GPU configurations on a stated subset of layers:
            sequence split of one 131072-token sequence with sharded storage and an NCCL
            all-gather of the (m, l, o) states; the Llama-3-70B shape with ragged contexts and
            KV heads sharded over the ranks; append / encode throughput.  Each is preceded by
            a small in-run correctness check and the process exits non-zero on a mismatch.

``--impl reference`` times the reference's numpy path alone (oracle/_ref, the unmodified
package copied there by ``make -C oracle ref``; the C restatement stands in where that copy is
absent, and the line says which).
"""

from __future__ import annotations

import argparse
import hashlib
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

# DRAM traffic of one launch of the attention kernel at the headline workload, from an ncu
# capture (dram__bytes_read.sum + dram__bytes_write.sum); valid for the kernel sources whose
# digest is given, reported as null once they have changed.
TRAFFIC_CAPTURE = {"bytes_per_launch": 334987520 + 5703168, "algorithmic_bytes": 333316096,
                   "sources_sha16": "3d4d4fd70d7baf87"}


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=20)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", default="native", choices=["native", "reference"])
    p.add_argument("--model", default="llama-3-8b")
    p.add_argument("--layers", type=int, default=0, help="override the layer count")
    p.add_argument("--batch", type=int, default=32, help="global batch of the headline workload")
    p.add_argument("--ctx", type=int, default=8192)
    p.add_argument("--hot-window", type=int, default=512)
    p.add_argument("--target", default="balanced")
    p.add_argument("--cpu-seconds", type=float, default=12.0)
    p.add_argument("--cpu-workers", type=int, default=0, help="0: one per host core, at most 16")
    p.add_argument("--no-cpu-baseline", action="store_true")
    p.add_argument("--no-e2e", action="store_true")
    p.add_argument("--extras", default="cfg0,cfg2,cfg3,cfg4",
                   help="comma list of cfg0,cfg2,cfg3,cfg4,weak, or 'none'")
    p.add_argument("--seed", type=int, default=0)
    return p.parse_args()


# ------------------------------------------------------------------------------------ #
# clocks                                                                                #
# ------------------------------------------------------------------------------------ #

class ClockSampler:
    """Samples SM clocks and throttle reasons while the timed region runs (read-only NVML
    queries; nvidia-smi if NVML is not usable)."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self._stop = threading.Event()
        self._t = None

    def _run_nvml(self) -> bool:
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
            except Exception:  # noqa: BLE001
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
# CPU legs: the reference's numpy path, or the C restatement where the copy is absent     #
# ------------------------------------------------------------------------------------ #

def reference_root():
    """Directory that holds the reference's ``turboquant_pro`` package: the copy made by
    ``make -C oracle ref``, else a checkout named by TQ_REF_PATH; None if neither exists."""
    for cand in (os.path.join(ROOT, "oracle", "_ref"), os.environ.get("TQ_REF_PATH", "")):
        if cand and os.path.isdir(os.path.join(cand, "turboquant_pro")):
            return cand
    return None


def step_bytes_one_sequence(h, hq, d, n, w, vb, hot_elem=2, q_elem=2):
    """Algorithmic bytes one decode step of one (sequence, layer) reads, counted like
    tq_decode_bytes: the reference's container sizes for every cold block (with the nominal
    outlier count per channel), the 16-bit hot window, q and the float32 output."""
    f = (w + 1) // 2
    nb = 0 if n <= w else 1 + (n - w - 1) // f
    k_out = max(1, round(f * 0.02))
    blk = f * d * 4 // 8 + f * d * vb // 8 + 4 * f + 8 * d + 6 * k_out * d
    return h * (nb * blk + (n - nb * f) * d * 2 * hot_elem) + hq * d * (q_elem + 4)


def _ref_worker(job):
    """One host process of the reference leg: builds the reference's own cache for one
    sequence of one layer (AutoConfig(...).build_cache, CPU path), fills it token by token
    like the reference's callers do, then repeats dequantise-then-attend decode steps."""
    ref_root, model, target, hq, n, w, seed, seconds, max_steps = job
    sys.path.insert(0, ref_root)
    from turboquant_pro.autoconfig import AutoConfig as RefAutoConfig

    from turboquant_pro_b200.synth import make_kv, make_q

    cfg = RefAutoConfig.from_pretrained(model, target=target)
    cache = cfg.build_cache(hot_window=w, use_gpu=False, seed=seed)
    h, d = cache.n_heads, cache.head_dim
    k, v = make_kv(seed, h, n, dtype=np.float16)
    k = k.astype(np.float32)
    v = v.astype(np.float32)
    t_fill = time.perf_counter()
    for t in range(n):
        cache.append(k[t], v[t])
    t_fill = time.perf_counter() - t_fill
    q = make_q(seed, hq)
    g = hq // h
    scale = np.float32(1.0 / np.sqrt(d))

    def one_step():
        keys = cache.get_keys(0, n)[0]
        vals = cache.get_values(0, n)[0]
        out = np.empty((hq, d), np.float32)
        for i in range(hq):  # query head i reads KV head i // G
            s = (keys[i // g] @ q[i]) * scale
            s -= s.max()
            p = np.exp(s)
            out[i] = (p / p.sum()) @ vals[i // g]
        return out

    one_step()
    t0 = time.perf_counter()
    steps = 0
    while True:
        one_step()
        steps += 1
        el = time.perf_counter() - t0
        if el >= seconds or steps >= max_steps:
            break
    return {"steps": steps, "elapsed": el, "fill_s": t_fill, "n_blocks": len(cache._cold_keys),
            "h": h, "hq": hq, "value_bits": int(cache.value_bits)}


def cpu_reference_leg(args, cfg, seconds: float):
    """The reference's numpy decode path on the host cores: one process per core (numpy is
    single-threaded on this path), each with one sequence of one layer of the workload."""
    ref_root = reference_root()
    if ref_root is None:
        return cpu_port_leg(args, cfg, seconds)
    import multiprocessing as mp

    workers = args.cpu_workers or max(1, min(os.cpu_count() or 1, 16))
    jobs = [(ref_root, args.model, args.target, cfg.n_q_heads, args.ctx, args.hot_window,
             args.seed + i, seconds, 1000) for i in range(workers)]
    ctx = mp.get_context("spawn")
    t0 = time.perf_counter()
    with ctx.Pool(workers) as pool:
        res = pool.map(_ref_worker, jobs)
    wall = time.perf_counter() - t0
    r0 = res[0]
    one = step_bytes_one_sequence(r0["h"], r0["hq"], cfg.head_dim, args.ctx, args.hot_window,
                                  r0["value_bits"])
    rate = sum(r["steps"] / r["elapsed"] for r in res)  # sequence-layer steps per second
    per_step = 1.0 / rate
    import numpy

    return {
        "value": one * rate / 1e9, "unit": UNIT, "cores": workers, "kind": "reference",
        "sample": (f"{sum(r['steps'] for r in res)} decode steps of 1 sequence x 1 layer "
                   f"({r0['h']} KV heads, ctx {args.ctx}, {r0['n_blocks']} cold blocks) through the "
                   f"reference's TurboQuantKVCache.get_keys/get_values + float32 attention, "
                   f"{workers} processes of numpy {numpy.__version__}; "
                   f"{np.mean([r['elapsed'] / r['steps'] for r in res]) * 1e3:.0f} ms per step "
                   f"and process; a full step is {cfg.n_layers} layers x {args.batch} sequences = "
                   f"{cfg.n_layers * args.batch} of these (factor stated, not run); filling one "
                   f"cache token by token took {r0['fill_s']:.1f} s; leg wall time {wall:.0f} s"),
        "ms_per_seq_layer_step": per_step * 1e3,
        "tokens_per_s": 1.0 / (per_step * cfg.n_layers),
    }


def cpu_port_leg(args, cfg, seconds: float):
    """Fallback of the CPU leg: the multi-threaded C restatement of the same path."""
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
    kb, vbk = [], []
    for b in range(nb):  # encode once (not timed): the cache state the decode step reads
        xs = np.ascontiguousarray(np.moveaxis(k[b * f:(b + 1) * f], 0, 1))
        vs = np.ascontiguousarray(np.moveaxis(v[b * f:(b + 1) * f], 0, 1))
        kb.append(co.encode_keys(xs, kout))
        vbk.append(co.encode_values(vs, pi_t, bnd))
    hot_k = np.ascontiguousarray(np.moveaxis(k[nb * f:], 0, 1))
    hot_v = np.ascontiguousarray(np.moveaxis(v[nb * f:], 0, 1))
    one = step_bytes_one_sequence(h, hq, d, n, w, vb)

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
        "value": one / per_step / 1e9, "unit": UNIT, "cores": co.num_threads(), "kind": "port",
        "sample": (f"{steps} decode steps of 1 sequence x 1 layer ({h} KV heads, ctx {n}, "
                   f"{nb} cold blocks + {n - nb * f} hot) through the C restatement of "
                   f"get_keys/get_values + fp32 attention (the reference copy under oracle/_ref "
                   f"is absent); {per_step * 1e3:.1f} ms per sequence-layer step"),
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
    cb = cpu_reference_leg(args, cfg, budget)
    line = {
        "impl": "reference", "metric": METRIC, "value": cb["value"], "unit": UNIT,
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": cb["ms_per_seq_layer_step"] * cfg.n_layers * args.batch,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "tokens_per_s": cb["tokens_per_s"],
        "config": workload_config(args, cfg, args.gpus, args.batch),
        "cpu_baseline": {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": cb["value"], "unit": UNIT, "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "ms_per_step is the measured sequence-layer step time times layers x batch "
                "(the full step is not run on the host)",
    }
    print(json.dumps(line), flush=True)


def workload_config(args, cfg, n_gpus, global_batch):
    return {
        "workload": (f"{args.model} decode attention on compressed KV: {cfg.n_layers} layers, "
                     f"{cfg.n_q_heads}q/{cfg.n_kv_heads}kv heads, head_dim {cfg.head_dim}, "
                     f"K{cfg.key_bits} asym-NF4 + 2% outliers / V{cfg.value_bits}, "
                     f"hot_window {args.hot_window}, batch {global_batch} (whole job), "
                     f"ctx {args.ctx}"),
        "global_batch": global_batch, "ctx": args.ctx, "layers": cfg.n_layers,
        "parallelism": (f"batch-shard x{n_gpus}: the {global_batch} sequences divided over the "
                        "ranks, no collective on the attention path"),
        "l2": "per-step working set (all layers) exceeds L2; no flush needed",
        "kv_dtype": "f16", "q_dtype": "bf16",
    }


# ------------------------------------------------------------------------------------ #
# native arm: helpers                                                                   #
# ------------------------------------------------------------------------------------ #

class Dist:
    """Rank bookkeeping and the few collectives the benchmark needs."""

    def __init__(self):
        import torch

        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        if self.world > 1:
            import torch.distributed as dist

            dist.init_process_group("nccl", device_id=self.dev)

    def barrier(self):
        import torch

        if self.world > 1:
            import torch.distributed as dist

            dist.barrier()
        torch.cuda.synchronize()

    def max_ms(self, ms: float) -> float:
        import torch

        t = torch.tensor([ms], dtype=torch.float64, device=self.dev)
        if self.world > 1:
            import torch.distributed as dist

            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def all_ok(self, ok: bool) -> bool:
        import torch

        t = torch.tensor([1 if ok else 0], dtype=torch.int32, device=self.dev)
        if self.world > 1:
            import torch.distributed as dist

            dist.all_reduce(t, op=dist.ReduceOp.MIN)
        return bool(t.item())

    def finish(self):
        if self.world > 1:
            import torch.distributed as dist

            dist.destroy_process_group()


def timed(dst: Dist, fn, steps: int, warmup: int):
    """W untimed calls, then K calls between two events on the current stream, bracketed by a
    barrier + synchronize on both sides; returns the max over ranks of milliseconds per call."""
    import torch

    for _ in range(max(warmup, 3)):
        fn()
    dst.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    dst.barrier()
    return dst.max_ms(e0.elapsed_time(e1)) / steps


def channel_scales_dev(gen, dev, h, d=128):
    """Per-(head, channel) key and value scales: exp(N(0, 0.5)), round(2 % of D) key channels
    per head times 20."""
    import torch

    sk = torch.exp(0.5 * torch.randn((h, d), generator=gen, device=dev))
    sv = torch.exp(0.5 * torch.randn((h, d), generator=gen, device=dev))
    n_out = int(round(0.02 * d))
    for hh in range(h):
        idx = torch.randperm(d, generator=gen, device=dev)[:n_out]
        sk[hh, idx] *= 20.0
    return sk, sv


def fill_uniform(ctx, dev, seed, n_layers, n_seqs, h, n_tokens, chunk=2048):
    """Fills every layer with ``n_tokens`` tokens per sequence of channel-scaled Gaussians
    generated on the device."""
    import torch

    gen = torch.Generator(device=dev)
    gen.manual_seed(seed)
    for layer in range(n_layers):
        sk, sv = channel_scales_dev(gen, dev, h)
        for t0 in range(0, n_tokens, chunk):
            t1 = min(n_tokens, t0 + chunk)
            k = (torch.randn((n_seqs, t1 - t0, h, 128), generator=gen, device=dev) * sk).half()
            v = (torch.randn((n_seqs, t1 - t0, h, 128), generator=gen, device=dev) * sv).half()
            ctx.append(layer, k, v)
    torch.cuda.synchronize()
    if ctx.status() != 0:
        raise SystemExit("outlier pool overflow while filling the cache")


def peaks():
    try:
        p = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        return float(p["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    except Exception:  # noqa: BLE001
        return 6650.0, "fallback 6650"


def kernel_sources_sha16():
    h = hashlib.sha256()
    for name in ("decode_mma.cu", "common.cuh"):
        with open(os.path.join(ROOT, "turboquant-pro_b200", "csrc", name), "rb") as f:
            h.update(f.read())
    return h.hexdigest()[:16]


def kernel_times(ctx, layers, q_all, out_all, steps):
    """The per-kernel times of the roofline: K more passes over the layers with an event pair
    around every kernel launch (on the launching stream, inside the library).  Kept out of the
    timed region because the events stop the two kernels of a call from overlapping."""
    import torch

    ctx.profile(True)
    for _ in range(steps):
        for layer in layers:
            ctx.decode(layer, q_all[layer], out=out_all[layer])
    torch.cuda.synchronize()
    attn_ms, comb_ms, n_calls = ctx.profile_read()
    ctx.profile(False)
    n = max(n_calls, 1)
    return attn_ms / n, comb_ms / n, n_calls


# ------------------------------------------------------------------------------------ #
# native arm: headline (config 1)                                                       #
# ------------------------------------------------------------------------------------ #

def run_headline(args, dst: Dist, cfg, batch_local, global_batch, scaling):
    import torch

    dev = dst.dev
    L, B, H, HQ, D = cfg.n_layers, batch_local, cfg.n_kv_heads, cfg.n_q_heads, cfg.head_dim
    e2e_steps = 0 if args.no_e2e else args.steps + max(args.warmup, 3)
    ctx = cfg.build_context(n_seqs=B, max_tokens_per_seq=args.ctx + e2e_steps + 8,
                            hot_window=args.hot_window, seed=args.seed, kv_dtype="float16",
                            device=dst.local)
    fill_uniform(ctx, dev, args.seed * 1000 + dst.rank, L, B, H, args.ctx)
    gen = torch.Generator(device=dev)
    gen.manual_seed(args.seed * 1000 + 500 + dst.rank)
    q_all = torch.randn((L, B, HQ, D), generator=gen, device=dev).to(torch.bfloat16)
    out_all = torch.empty((L, B, HQ, D), dtype=torch.float32, device=dev)
    layers = list(range(L))

    def step():
        for layer in layers:
            ctx.decode(layer, q_all[layer], out=out_all[layer])

    step()
    step_bytes = sum(ctx.decode_bytes(layer) for layer in layers)
    launches_per_step = L * ctx.last_launches()
    kernel = ctx.last_kernel()
    with ClockSampler(dst.local) as clk:
        ms_per_step = timed(dst, step, args.steps, args.warmup)
        attn_ms, comb_ms, n_calls = kernel_times(ctx, layers, q_all, out_all, args.steps)
    if ctx.raise_on_timeout() != 0:
        raise SystemExit("status flags set after the timed region")
    value = dst.world * step_bytes / (ms_per_step * 1e-3) / 1e9

    e2e = None
    if not args.no_e2e:
        e2e = run_e2e(args, dst, ctx, L, B, H, HQ, D, global_batch)

    peak, peak_src = peaks()
    layer_bytes = step_bytes / L
    achieved = layer_bytes / (attn_ms * 1e-3) / 1e9 if attn_ms > 0 else None
    sha = kernel_sources_sha16()
    traffic = None
    traffic_src = "no ncu capture of the current kernel sources is recorded in bench.py"
    if TRAFFIC_CAPTURE["sources_sha16"] == sha and TRAFFIC_CAPTURE["bytes_per_launch"]:
        traffic = TRAFFIC_CAPTURE["bytes_per_launch"] * layer_bytes / TRAFFIC_CAPTURE["algorithmic_bytes"]
        traffic_src = ("ncu capture (dram__bytes_read.sum + dram__bytes_write.sum) of this kernel "
                       "at the headline workload, scaled by algorithmic bytes; kernel sources "
                       f"unchanged since (sha {sha})")
    elif TRAFFIC_CAPTURE["sources_sha16"]:
        traffic_src = (f"the recorded capture is of kernel sources {TRAFFIC_CAPTURE['sources_sha16']}, "
                       f"the current ones are {sha}: not reported")
    roofline = {
        "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
        "frac": achieved / peak if achieved else None, "peak_source": peak_src,
        "frac_of_nominal_8TBps": achieved / 8000.0 if achieved else None,
        "kernel": f"decode attention kernel ({kernel}; one launch per layer)",
        "algorithmic_bytes_per_launch": layer_bytes,
        "avg_launch_ms": attn_ms, "combine_avg_launch_ms": comb_ms, "launches_timed": n_calls,
        "traffic": traffic, "traffic_source": traffic_src,
        "timing": "CUDA events around every launch on the launching stream, in a second pass "
                  "of the same K steps right after the timed region",
    }
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": dst.world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": scaling, "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "tokens_per_s": dst.world * B / (ms_per_step * 1e-3),
        "config": workload_config(args, cfg, dst.world, global_batch),
        "bytes_per_step_per_gpu": step_bytes, "kernel": kernel,
        "roofline": roofline, "clocks": clk.summary(), "e2e": e2e,
        "gpu_launches": launches_per_step * args.steps,
        "device_bytes": ctx.device_bytes(),
    }
    del ctx, q_all, out_all
    torch.cuda.empty_cache()
    return line


def run_e2e(args, dst: Dist, ctx, L, B, H, HQ, D, global_batch):
    """The same step through the public API with host buffers.  Every step its inputs (the
    query and the new K/V token of every layer, in pinned host memory) go to the device and
    its outputs come back: one copy per tensor and step on a second stream, double-buffered
    over steps, so that a step's inputs arrive while the step before it is attended and its
    outputs leave while the next one runs.  Per layer the step calls KVContext.append and
    KVContext.decode on views of the device buffers."""
    import torch

    dev = dst.dev
    q_host = torch.randn((L, B, HQ, D)).to(torch.bfloat16).pin_memory()
    k_host = (torch.randn((L, B, 1, H, D))).half().pin_memory()
    v_host = (torch.randn((L, B, 1, H, D))).half().pin_memory()
    out_host = torch.empty((L, B, HQ, D), dtype=torch.float32).pin_memory()
    copy_stream = torch.cuda.Stream(device=dev)
    main_stream = torch.cuda.current_stream(dev)
    qd = [torch.empty((L, B, HQ, D), dtype=torch.bfloat16, device=dev) for _ in range(2)]
    kd = [torch.empty((L, B, 1, H, D), dtype=torch.float16, device=dev) for _ in range(2)]
    vd = [torch.empty((L, B, 1, H, D), dtype=torch.float16, device=dev) for _ in range(2)]
    od = [torch.empty((L, B, HQ, D), dtype=torch.float32, device=dev) for _ in range(2)]
    ev_in = [torch.cuda.Event() for _ in range(2)]    # inputs of buffer b have arrived
    ev_done = [torch.cuda.Event() for _ in range(2)]  # the step that used buffer b is attended
    ev_out = [torch.cuda.Event() for _ in range(2)]   # outputs of buffer b have left
    state = {"step": 0, "fetched": -1}

    def fetch(step):
        b = step & 1
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(ev_done[b])  # the step that read these buffers is done
            qd[b].copy_(q_host, non_blocking=True)
            kd[b].copy_(k_host, non_blocking=True)
            vd[b].copy_(v_host, non_blocking=True)
            ev_in[b].record(copy_stream)
        state["fetched"] = step

    def e2e_step():
        step = state["step"]
        b = step & 1
        if state["fetched"] < step:
            fetch(step)
        main_stream.wait_event(ev_in[b])
        main_stream.wait_event(ev_out[b])  # this buffer's previous outputs have left
        fetch(step + 1)                    # the next step's inputs travel under this step
        for layer in range(L):
            ctx.append(layer, kd[b][layer], vd[b][layer])
            ctx.decode(layer, qd[b][layer], out=od[b][layer])
        ev_done[b].record(main_stream)
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(ev_done[b])
            out_host.copy_(od[b], non_blocking=True)
            ev_out[b].record(copy_stream)
        state["step"] = step + 1

    def drain():
        main_stream.wait_stream(copy_stream)
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        e2e_step()
    drain()
    dst.barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        e2e_step()
    drain()
    dst.barrier()
    el = dst.max_ms((time.perf_counter() - t0) * 1e3) * 1e-3
    e2e_bytes = sum(ctx.decode_bytes(layer) for layer in range(L))
    h2d = q_host.numel() * 2 + k_host.numel() * 2 + v_host.numel() * 2
    return {"value": dst.world * e2e_bytes / (el / args.steps) / 1e9, "unit": UNIT,
            "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(out_host.numel() * 4),
            "ms_per_step": el / args.steps * 1e3,
            "tokens_per_s": dst.world * B / (el / args.steps),
            "path": "per step: pinned q + new K/V token of every layer H2D (one copy per "
                    "tensor), per layer KVContext.append + KVContext.decode, outputs D2H; copies "
                    "on a second stream, double-buffered over steps: every step sends the next "
                    "step's inputs, so the timed region holds K input copies, K steps and K "
                    "output copies; timed by the host clock between device synchronisations"}


# ------------------------------------------------------------------------------------ #
# config 0: the reference's own CPU-runnable case, in full on both sides                #
# ------------------------------------------------------------------------------------ #

def cfg0_inputs(seed, h=32, d=128, n=4096):
    """Post-RoPE float32 K/V: N(0,1) times per-channel scales log-normal(0, 0.5), 2 % of the
    key channels scaled x20; one N(0,1) query per head."""
    rng = np.random.default_rng(seed)
    sk = rng.lognormal(0.0, 0.5, size=(h, d)).astype(np.float32)
    sv = rng.lognormal(0.0, 0.5, size=(h, d)).astype(np.float32)
    hot = rng.random((h, d)) < 0.02
    sk = np.where(hot, sk * 20.0, sk).astype(np.float32)
    k = (rng.standard_normal((n, h, d)).astype(np.float32) * sk)
    v = (rng.standard_normal((n, h, d)).astype(np.float32) * sv)
    q = rng.standard_normal((h, d)).astype(np.float32)
    return k, v, q


def _cfg0_ref_worker(job):
    """The reference itself on configuration 0 (TurboQuantKVCache.robust, CPU path): fills the
    cache token by token, then times fused_decode and dequantise-then-attend."""
    ref_root, seed, reps = job
    sys.path.insert(0, ref_root)
    from turboquant_pro.core import TurboQuantKVCache as RefCache

    k, v, q = cfg0_inputs(seed)
    # (bits=4 beside K4/V4: the reference's fused_decode looks its value codebook up under
    # `bits`, core.py:1191-1192 and kv_fused.py's _rot_matrices)
    cache = RefCache.robust(head_dim=128, n_heads=32, hot_window=512, use_gpu=False, seed=seed,
                            bits=4)
    t0 = time.perf_counter()
    for t in range(k.shape[0]):
        cache.append(k[t], v[t])
    fill_s = time.perf_counter() - t0
    out = np.asarray(cache.fused_decode(q), dtype=np.float32)  # builds the prepared pages
    t0 = time.perf_counter()
    for _ in range(reps):
        out = np.asarray(cache.fused_decode(q), dtype=np.float32)
    fused_ms = (time.perf_counter() - t0) / reps * 1e3
    t0 = time.perf_counter()
    keys = cache.get_keys(0, cache.length)[0]
    vals = cache.get_values(0, cache.length)[0]
    sc = np.einsum("hd,hsd->hs", q, keys) / np.sqrt(np.float32(128.0))
    sc -= sc.max(axis=-1, keepdims=True)
    p = np.exp(sc)
    dq = np.einsum("hs,hsd->hd", p / p.sum(axis=-1, keepdims=True), vals)
    dequant_ms = (time.perf_counter() - t0) * 1e3
    return {"out": out, "dequant_out": dq.astype(np.float32), "fill_s": fill_s,
            "fused_ms": fused_ms, "dequant_ms": dequant_ms, "n_blocks": len(cache._cold_keys),
            "pi": np.asarray(cache._tq._Pi)}


def run_cfg0(args, dst: Dist):
    """Configuration 0 of the baseline (one layer, MHA 32 heads, batch 1, context 4096,
    robust K4/V4, float32 K/V): the drop-in cache on the GPU and, where the reference package
    is at hand, the reference's own CPU path on the very same tensors, both in full, with the
    outputs compared.  Rank 0 only."""
    import torch

    if dst.rank != 0:
        return None
    from turboquant_pro_b200 import TurboQuantKVCache

    seed = args.seed + 40
    k, v, q = cfg0_inputs(seed)
    n, h, d = k.shape
    ref, ref_root = None, reference_root()
    if ref_root is not None:
        try:
            import multiprocessing as mp

            with mp.get_context("spawn").Pool(1) as pool:
                ref = pool.apply(_cfg0_ref_worker, ((ref_root, seed, 5),))
        except Exception as e:  # noqa: BLE001
            ref = {"error": repr(e)[:200]}
    cache = TurboQuantKVCache.robust(head_dim=d, n_heads=h, hot_window=512, seed=seed,
                                     max_tokens=n + 8, device_id=dst.local)
    if ref is not None and "pi" in ref and not np.array_equal(ref["pi"], cache._tq._Pi):
        raise SystemExit("config 0: the rotation matrix differs from the reference's")
    t0 = time.perf_counter()
    for t in range(n):
        cache.append(k[t], v[t])
    torch.cuda.synchronize()
    fill_s = time.perf_counter() - t0
    out = np.asarray(cache.fused_decode(q))
    reps = 50
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(reps):
        out = np.asarray(cache.fused_decode(q))  # numpy in, numpy out: copies included
    facade_ms = (time.perf_counter() - t0) / reps * 1e3
    ctx = cache._ctx
    qd = torch.from_numpy(q)[None].to(ctx.device)
    od = torch.empty((1, h, d), dtype=torch.float32, device=ctx.device)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(5):
        ctx.decode(0, qd, out=od)
    e0.record()
    for _ in range(reps):
        ctx.decode(0, qd, out=od)
    e1.record()
    torch.cuda.synchronize()
    device_ms = e0.elapsed_time(e1) / reps
    res = {
        "workload": "configuration 0: one layer, MHA 32 heads x head_dim 128, batch 1, context "
                    "4096, robust K4 asym-NF4 + 2% outliers / V4, float32 K/V, hot_window 512",
        "gpu_fused_decode_ms_numpy_in_out": facade_ms, "gpu_decode_ms_device": device_ms,
        "gpu_fill_s_token_by_token": fill_s, "kernel": ctx.last_kernel(),
        "n_blocks": ctx.lengths(0, 0)[1] // ctx.block_tokens,
    }
    if ref is None:
        res["reference"] = "the reference package is not on this machine"
    elif "error" in ref:
        res["reference"] = ref["error"]
    else:
        err = float(np.abs(out - ref["out"]).max())
        err_dq = float(np.abs(out - ref["dequant_out"]).max())
        tol = bool(np.allclose(out, ref["dequant_out"], rtol=2e-2, atol=2e-3))
        if not tol:
            raise SystemExit(f"config 0 check failed: output differs from the reference's "
                             f"(max abs err {err_dq:.3e})")
        res.update({
            "reference_fused_decode_ms": ref["fused_ms"],
            "reference_dequantise_then_attend_ms": ref["dequant_ms"],
            "reference_fill_s_token_by_token": ref["fill_s"],
            "reference_n_blocks": ref["n_blocks"],
            "max_abs_err_vs_reference_fused_decode": err,
            "max_abs_err_vs_reference_dequantise_then_attend": err_dq,
            "within_rtol_2e-2_atol_2e-3": tol,
            "what": "the unmodified reference (its numpy path) run in this process's host on "
                    "the same seeded tensors",
        })
    del cache
    torch.cuda.empty_cache()
    return res


# ------------------------------------------------------------------------------------ #
# config 2: one long sequence, sequence split with sharded storage                      #
# ------------------------------------------------------------------------------------ #

def make_token_fn(dev, seed, layer, n_seqs, h, sk, sv, chunk):
    """Tokens [t0, t1) of a layer's sequence, the same on every rank that asks: each chunk of
    ``chunk`` positions has its own generator seed."""
    import torch

    def fn(t0, t1):
        ks, vs = [], []
        c0 = t0 // chunk
        while c0 * chunk < t1:
            gen = torch.Generator(device=dev)
            gen.manual_seed((seed * 1009 + layer) * 100003 + c0)
            k = (torch.randn((n_seqs, chunk, h, 128), generator=gen, device=dev) * sk).half()
            v = (torch.randn((n_seqs, chunk, h, 128), generator=gen, device=dev) * sv).half()
            a, b = max(t0, c0 * chunk) - c0 * chunk, min(t1, (c0 + 1) * chunk) - c0 * chunk
            ks.append(k[:, a:b])
            vs.append(v[:, a:b])
            c0 += 1
        return torch.cat(ks, dim=1).contiguous(), torch.cat(vs, dim=1).contiguous()

    return fn


def build_split_cache(cfg, dst: Dist, args, n_layers, n_tokens, seed):
    """A ShardedSequenceCache of one sequence filled with ``n_tokens`` tokens per layer."""
    import torch

    from turboquant_pro_b200.parallel import ShardedSequenceCache

    cap = ShardedSequenceCache.local_capacity(n_tokens, args.hot_window, dst.rank, dst.world, 8)
    ctx = cfg.build_context(n_seqs=1, max_tokens_per_seq=cap, hot_window=args.hot_window,
                            seed=seed, kv_dtype="float16", n_layers=n_layers, device=dst.local)
    cache = ShardedSequenceCache(ctx)
    gen = torch.Generator(device=dst.dev)
    gen.manual_seed(seed * 77 + 1)
    for layer in range(n_layers):
        sk, sv = channel_scales_dev(gen, dst.dev, cfg.n_kv_heads)  # same draws on every rank
        cache.prefill(layer, n_tokens,
                      make_token_fn(dst.dev, seed, layer, 1, cfg.n_kv_heads, sk, sv, 4096),
                      chunk=16384)
    torch.cuda.synchronize()
    return cache


def check_split(cfg, dst: Dist, args):
    """In-run correctness check of the sequence split: a 9000-token layer decoded through the
    sharded caches + all-gather + merge must equal the same layer held whole on this rank."""
    import torch

    n = 9000
    cache = build_split_cache(cfg, dst, args, 1, n, seed=4242)
    whole = cfg.build_context(n_seqs=1, max_tokens_per_seq=n, hot_window=args.hot_window,
                              seed=4242, kv_dtype="float16", n_layers=1, device=dst.local)
    gen = torch.Generator(device=dst.dev)
    gen.manual_seed(4242 * 77 + 1)
    sk, sv = channel_scales_dev(gen, dst.dev, cfg.n_kv_heads)
    k, v = make_token_fn(dst.dev, 4242, 0, 1, cfg.n_kv_heads, sk, sv, 4096)(0, n)
    whole.append(0, k, v)
    g2 = torch.Generator(device=dst.dev)
    g2.manual_seed(99)
    q = torch.randn((1, cfg.n_q_heads, 128), generator=g2, device=dst.dev).to(torch.bfloat16)
    want = whole.decode(0, q)
    got = cache.decode(0, q)
    torch.cuda.synchronize()
    err = float((got - want).abs().max())
    ok = bool(torch.allclose(got, want, rtol=1e-3, atol=1e-4)) and cache.ctx.status() == 0
    if dst.world == 1:  # one rank: the split is the identity, checked all the same
        ok = ok and err < 1e-4
    return dst.all_ok(ok), err


def run_cfg2(args, dst: Dist):
    import torch

    from turboquant_pro_b200 import AutoConfig

    cfg = AutoConfig.from_pretrained("llama-3-8b", target="balanced")
    ok, err = check_split(cfg, dst, args)
    if not ok:
        raise SystemExit(f"config 2 check failed: sequence split differs from the whole decode "
                         f"(max abs err {err:.3e})")
    n, L = 131072, cfg.n_layers
    cache = build_split_cache(cfg, dst, args, L, n, seed=args.seed + 2)
    ctx = cache.ctx
    dev = dst.dev
    gen = torch.Generator(device=dev)
    gen.manual_seed(args.seed + 2002)
    q_all = torch.randn((L, 1, cfg.n_q_heads, 128), generator=gen, device=dev).to(torch.bfloat16)
    rows = cfg.n_q_heads
    mlo = torch.empty((1, cfg.n_q_heads, 130), dtype=torch.float32, device=dev)
    gathered = torch.empty((dst.world, rows, 130), dtype=torch.float32, device=dev)
    out = torch.empty((L, rows, 128), dtype=torch.float32, device=dev)
    nb_local = [cache.local_blocks(layer) for layer in range(L)]
    last = dst.rank == dst.world - 1
    if dst.world > 1:
        import torch.distributed as dist

    def step():
        for layer in range(L):
            ctx.decode_partial(layer, q_all[layer], 0, nb_local[layer], last, mlo=mlo)
            if dst.world > 1:
                dist.all_gather_into_tensor(gathered.view(-1), mlo.view(-1))
                ctx.lse_combine(gathered, out=out[layer])
            else:
                ctx.lse_combine(mlo.view(1, rows, 130), out=out[layer])

    def run_transport(step_fn):
        # The step is launch-bound once the sequence is spread over several GPUs (a handful of
        # launches per layer against a few tens of microseconds of work), so it is also
        # captured into one CUDA graph, the exchange included, and replayed.
        ms_e = timed(dst, step_fn, args.steps, args.warmup)
        ms_b, graphed_b = ms_e, False
        try:
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                step_fn()
            ok = True
        except Exception:  # noqa: BLE001 - a stack that cannot capture keeps the eager number
            ok = False
            torch.cuda.synchronize()
        if dst.all_ok(ok):
            want = out.clone()
            ms_graph = timed(dst, graph.replay, args.steps, args.warmup)
            same = bool(torch.equal(out, want))
            if dst.all_ok(same) and ms_graph < ms_e:
                ms_b, graphed_b = ms_graph, True
        return ms_e, ms_b, graphed_b

    ms_eager, ms, graphed = run_transport(step)
    transport = "nccl" if dst.world > 1 else "none"
    nccl_numbers = {"ms_per_step": ms, "ms_per_step_eager": ms_eager, "cuda_graph": graphed}
    peer_numbers, xchg_us = None, None
    if dst.world > 1:
        # The same step with the states exchanged and merged by one kernel over peer memory
        # (plain peer stores over NVLink, bounded waits) instead of all-gather + merge kernel.
        from turboquant_pro_b200.parallel import PeerExchange

        ex, ok = None, True
        try:
            ex = PeerExchange(rows, 128, dev)
        except Exception:  # noqa: BLE001 - no peer mapping between these processes
            ok = False
        if dst.all_ok(ok):
            want = out.clone()  # what the all-gather path left

            def step_peer():
                for layer in range(L):
                    ctx.decode_partial(layer, q_all[layer], 0, nb_local[layer], last, mlo=mlo)
                    ex.gather_merge(mlo.view(rows, 130), out=out[layer])

            step_peer()
            torch.cuda.synchronize()
            same = bool(torch.equal(out, want)) and ex.status() == 0
            if not dst.all_ok(same):
                raise SystemExit("config 2 check failed: the peer-memory exchange and the "
                                 "all-gather path give different bits")
            p_eager, p_ms, p_graphed = run_transport(step_peer)
            x_ms = timed(dst, lambda: [ex.gather_merge(mlo.view(rows, 130), out=out[0])
                                       for _ in range(L)], args.steps, args.warmup)
            xchg_us = x_ms * 1e3 / L
            ex.check()
            peer_numbers = {"ms_per_step": p_ms, "ms_per_step_eager": p_eager,
                            "cuda_graph": p_graphed, "exchange_kernel_us": xchg_us,
                            "same_bits_as_all_gather": True}
            if p_ms < ms:
                ms_eager, ms, graphed, transport = p_eager, p_ms, p_graphed, "peer"
            # ... and with the exchange run by the merge kernel of the partial decode itself
            # (one kernel less on the critical path)
            def step_fused():
                for layer in range(L):
                    ctx.decode_exchange(layer, q_all[layer], 0, nb_local[layer], last, ex,
                                        out=out[layer].view(1, rows, 128))

            fused_ok = True
            try:
                step_fused()
                torch.cuda.synchronize()
            except NotImplementedError:
                fused_ok = False
            if dst.all_ok(fused_ok):
                same = bool(torch.equal(out, want)) and ex.status() == 0
                if not dst.all_ok(same):
                    raise SystemExit("config 2 check failed: the merge kernel's own exchange and "
                                     "the all-gather path give different bits")
                f_eager, f_ms, f_graphed = run_transport(step_fused)
                ex.check()
                peer_numbers["fused"] = {"ms_per_step": f_ms, "ms_per_step_eager": f_eager,
                                         "cuda_graph": f_graphed, "same_bits_as_all_gather": True}
                if f_ms < ms:
                    ms_eager, ms, graphed, transport = f_eager, f_ms, f_graphed, "peer-fused"
        if ex is not None:
            ex.close()
    # the collective alone, same sizes, same stream
    ag_us = None
    if dst.world > 1:
        ag_ms = timed(dst, lambda: [dist.all_gather_into_tensor(gathered.view(-1), mlo.view(-1))
                                    for _ in range(L)], args.steps, args.warmup)
        ag_us = ag_ms * 1e3 / L
    # per-rank kernel time of the partial decode (attention + its combine), events per launch
    ctx.profile(True)
    for _ in range(args.steps):
        for layer in range(L):
            ctx.decode_partial(layer, q_all[layer], 0, nb_local[layer], last, mlo=mlo)
    torch.cuda.synchronize()
    attn_ms, comb_ms, n_calls = ctx.profile_read()
    ctx.profile(False)
    attn_ms, comb_ms = attn_ms / max(n_calls, 1), comb_ms / max(n_calls, 1)
    if ctx.raise_on_timeout() != 0:
        raise SystemExit("status flags set after config 2")
    # algorithmic bytes: this rank's blocks (+ window on the last rank) + q + states
    H, D, vb = cfg.n_kv_heads, 128, cfg.value_bits
    blk = 256 * D // 2 + 256 * D * vb // 8 + 4 * 256 + 8 * D + 6 * 5 * D
    rank_bytes = H * (nb_local[0] * blk + (512 * D * 2 * 2 if last else 0)) + rows * D * (2 + 4)
    total_bytes = H * (510 * blk + 512 * D * 2 * 2) + rows * D * (2 + 4)
    peak, _ = peaks()
    rank_gbs = rank_bytes / (attn_ms * 1e-3) / 1e9 if attn_ms > 0 else None
    t = torch.tensor([attn_ms, rank_gbs or 0.0], dtype=torch.float64, device=dev)
    if dst.world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    res = {
        "workload": "llama-3-8b shape, batch 1, ctx 131072 (510 cold blocks + 512 hot), K4/V3, "
                    f"all {L} layers; cold blocks divided over {dst.world} rank(s), each rank "
                    "stores and encodes only its own range, the last rank also the hot window",
        "n_gpus": dst.world, "layers_timed": L, "ms_per_step": ms,
        "ms_per_step_eager": ms_eager, "cuda_graph": graphed,
        "tokens_per_s": 1.0 / (ms * 1e-3),
        "value_GBps": L * total_bytes / (ms * 1e-3) / 1e9,
        "per_layer_us": ms * 1e3 / L,
        "all_gather_us": ag_us, "all_gather_bytes_per_rank": rows * 130 * 4,
        "transport": transport, "nccl": nccl_numbers if dst.world > 1 else None,
        "peer": peer_numbers,
        "rank_attention_kernel_us_max": float(t[0]) * 1e3,
        "rank_combine_kernel_us": comb_ms * 1e3,
        "rank0_blocks": nb_local[0], "rank0_GBps": rank_gbs,
        "rank0_roofline_frac": rank_gbs / peak if rank_gbs else None,
        "kernel": ctx.last_kernel(), "device_bytes_per_rank": ctx.device_bytes(),
        "check": {"split_equals_whole": True, "max_abs_err": err,
                  "what": "9000-token layer, sharded caches + all-gather + merge vs the same "
                          "layer held whole on every rank"},
        "collective": ("none: the kernel that merges the rank's own partials stores its [32][130] "
                       "float32 rows into every rank's region over NVLink, signals per row, waits "
                       "(bounded) and merges in rank order (tq_decode_exchange)"
                       if transport == "peer-fused" else
                       "one exchange kernel per layer: peer stores of [32][130] float32 into every "
                       "rank's region over NVLink, per-row flags, bounded wait, merge in "
                       "rank order (tq_xchg_gather_merge)" if transport == "peer" else
                       "NCCL all_gather_into_tensor of [32][130] float32 per layer, ordered with "
                       "the decode stream, then tq_lse_combine in rank order")
                      if dst.world > 1 else "none",
    }
    del cache, ctx
    torch.cuda.empty_cache()
    return res


# ------------------------------------------------------------------------------------ #
# config 3: Llama-3-70B shape, ragged contexts, KV heads sharded over the ranks          #
# ------------------------------------------------------------------------------------ #

def ragged_lengths(seed, n_seqs, lo=1024, hi=32768):
    rng = np.random.default_rng(seed + 333)
    return [int(x) for x in rng.integers(lo, hi + 1, size=n_seqs)]


def fill_ragged(ctx, dev, seed, n_layers, lens, h_total, h_lo, h_hi, chunk=4096):
    """Fills a head-sharded context (KV heads [h_lo, h_hi) of h_total) with ragged sequences:
    the tokens of all heads are generated, the rank keeps its heads, so every rank sees the
    same model-wide tensors."""
    import torch

    order = sorted(range(len(lens)), key=lambda s: lens[s])
    for layer in range(n_layers):
        gen = torch.Generator(device=dev)
        gen.manual_seed(seed * 7919 + layer)
        sk, sv = channel_scales_dev(gen, dev, h_total)
        for s in order:
            n = lens[s]
            for t0 in range(0, n, chunk):
                t1 = min(n, t0 + chunk)
                k = (torch.randn((1, t1 - t0, h_total, 128), generator=gen, device=dev) * sk).half()
                v = (torch.randn((1, t1 - t0, h_total, 128), generator=gen, device=dev) * sv).half()
                ctx.append(layer, k[:, :, h_lo:h_hi].contiguous(), v[:, :, h_lo:h_hi].contiguous(),
                           seq_begin=s)
    torch.cuda.synchronize()
    if ctx.status() != 0:
        raise SystemExit("outlier pool overflow while filling the cache")


def check_head_shard(cfg, dst: Dist, args, h_lo, h_hi):
    """In-run check of the KV-head shard: this rank's heads of a small ragged layer must equal
    the same heads of the layer held with all heads."""
    import torch

    lens = [700, 1500, 3000]
    H, G = cfg.n_kv_heads, cfg.n_q_heads // cfg.n_kv_heads
    kw = dict(max_tokens_per_seq=3000, hot_window=args.hot_window, seed=5151,
              kv_dtype="float16", n_layers=1, device=dst.local)
    full = cfg.build_context(n_seqs=3, **kw)
    part = cfg.build_context(n_seqs=3, n_kv_heads=h_hi - h_lo, **kw)
    fill_ragged(full, dst.dev, 5151, 1, lens, H, 0, H)
    fill_ragged(part, dst.dev, 5151, 1, lens, H, h_lo, h_hi)
    gen = torch.Generator(device=dst.dev)
    gen.manual_seed(77)
    q = torch.randn((3, cfg.n_q_heads, 128), generator=gen, device=dst.dev).to(torch.bfloat16)
    want = full.decode(0, q)[:, h_lo * G:h_hi * G]
    got = part.decode(0, q[:, h_lo * G:h_hi * G].contiguous())
    torch.cuda.synchronize()
    err = float((got - want).abs().max())
    ok = bool(torch.allclose(got, want, rtol=1e-3, atol=1e-4)) and part.status() == 0
    return dst.all_ok(ok), err


def run_cfg3(args, dst: Dist):
    import torch

    from turboquant_pro_b200 import AutoConfig

    cfg = AutoConfig.from_pretrained("llama-3-70b", target="quality")
    H, HQ = cfg.n_kv_heads, cfg.n_q_heads
    G = HQ // H
    if H % dst.world:
        return {"skipped": f"{H} KV heads do not divide over {dst.world} ranks"}
    hpr = H // dst.world
    h_lo, h_hi = dst.rank * hpr, (dst.rank + 1) * hpr
    ok, err = check_head_shard(cfg, dst, args, h_lo, h_hi)
    if not ok:
        raise SystemExit(f"config 3 check failed: head shard differs from the full context "
                         f"(max abs err {err:.3e})")
    B, L = 64, 8
    lens = ragged_lengths(args.seed, B)
    ctx = cfg.build_context(n_seqs=B, n_kv_heads=hpr, max_tokens_per_seq=32768 + 8,
                            hot_window=args.hot_window, seed=args.seed + 3, kv_dtype="float16",
                            n_layers=L, device=dst.local)
    fill_ragged(ctx, dst.dev, args.seed + 3, L, lens, H, h_lo, h_hi)
    gen = torch.Generator(device=dst.dev)
    gen.manual_seed(args.seed + 3003)
    q_all = torch.randn((L, B, HQ, 128), generator=gen, device=dst.dev).to(torch.bfloat16)
    q_loc = q_all[:, :, h_lo * G:h_hi * G].contiguous()
    out = torch.empty((L, B, hpr * G, 128), dtype=torch.float32, device=dst.dev)

    def step():
        for layer in range(L):
            ctx.decode(layer, q_loc[layer], out=out[layer])

    step()
    launches = ctx.last_launches()
    layer_bytes = ctx.decode_bytes(0)
    ms = timed(dst, step, args.steps, args.warmup)
    attn_ms, comb_ms, n_calls = kernel_times(ctx, list(range(L)), q_loc, out, args.steps)
    if ctx.raise_on_timeout() != 0:
        raise SystemExit("status flags set after config 3")
    peak, _ = peaks()
    gbs = layer_bytes / (attn_ms * 1e-3) / 1e9
    full_layers = cfg.n_layers
    res = {
        "workload": f"llama-3-70b shape ({HQ}q/{H}kv heads, GQA {G}), K4 asym-NF4 + 2% outliers / "
                    f"V4, batch {B}, ragged contexts uniform in [1024, 32768] (seeded; mean "
                    f"{int(np.mean(lens))}), KV heads sharded: {hpr} per rank; {L} of "
                    f"{full_layers} layers held and timed (per-layer work is the same for all)",
        "n_gpus": dst.world, "layers_timed": L, "ms_per_layer": ms / L,
        "value_GBps": dst.world * L * layer_bytes / (ms * 1e-3) / 1e9,
        "tokens_per_s_all_layers": B / (ms / L * full_layers * 1e-3),
        "rank_attention_kernel_ms": attn_ms, "rank_combine_kernel_ms": comb_ms,
        "rank_GBps": gbs, "rank_roofline_frac": gbs / peak,
        "algorithmic_bytes_per_launch_per_rank": layer_bytes,
        "kernel": ctx.last_kernel(), "launches_per_layer": launches,
        "device_bytes_per_rank": ctx.device_bytes(),
        "check": {"head_shard_equals_full": True, "max_abs_err": err,
                  "what": "3 ragged sequences, 1 layer: this rank's heads vs the same heads of "
                          "the all-heads context"},
        "collective": "none (outputs stay head-sharded for the projection that follows)",
    }
    del ctx, q_all, q_loc, out
    torch.cuda.empty_cache()
    return res


# ------------------------------------------------------------------------------------ #
# config 4: append / encode throughput                                                  #
# ------------------------------------------------------------------------------------ #

def check_encode(ctx, k, v, layer, seq, block, vb):
    """A sampled cold block against the C restatement of the reference encoders, bit for bit
    (checker only; not part of anything timed)."""
    from oracle import c_oracle as co
    from oracle import tq_oracle as orc

    f = 256
    xs = np.ascontiguousarray(np.moveaxis(k[block * f:(block + 1) * f].astype(np.float32), 0, 1))
    vs = np.ascontiguousarray(np.moveaxis(v[block * f:(block + 1) * f].astype(np.float32), 0, 1))
    _cent, bnd = orc.value_tables(128, vb)
    kb = co.encode_keys(xs, orc.outlier_count(f, 0.02))
    vbk = co.encode_values(vs, np.ascontiguousarray(ctx.pi.T), bnd)
    blk = ctx.export_block(layer, seq, block)
    return (np.array_equal(blk["key_indices"], orc.pack_key_codes(kb["codes"]))
            and np.array_equal(blk["nf4_scale"][0], kb["scale"])
            and np.array_equal(blk["nf4_mean"][0], kb["mean"])
            and np.array_equal(blk["outlier_idx"], kb["out_idx"])
            and np.array_equal(blk["outlier_val"].view(np.uint16), kb["out_val"].view(np.uint16))
            and np.array_equal(blk["value_indices"], orc.pack_value_codes(vbk["codes"], vb))
            and np.array_equal(blk["value_norms"][0], vbk["norms"]))


def run_cfg4(args, dst: Dist):
    import torch

    from turboquant_pro_b200 import AutoConfig

    cfg = AutoConfig.from_pretrained("llama-3-8b", target="balanced")
    Bg, n_pre, n_dec, L = 8, 16384, 256, 4
    if Bg % dst.world:
        return {"skipped": f"batch {Bg} does not divide over {dst.world} ranks"}
    B = Bg // dst.world
    H, HQ, D = cfg.n_kv_heads, cfg.n_q_heads, 128
    dev = dst.dev
    ctx = cfg.build_context(n_seqs=B, max_tokens_per_seq=n_pre + n_dec + 8,
                            hot_window=args.hot_window, seed=args.seed + 4, kv_dtype="float16",
                            n_layers=L, device=dst.local)
    gen = torch.Generator(device=dev)
    gen.manual_seed(args.seed * 31 + 4 + dst.rank)
    sk, sv = channel_scales_dev(gen, dev, H)
    k_pre = (torch.randn((B, n_pre, H, D), generator=gen, device=dev) * sk).half()
    v_pre = (torch.randn((B, n_pre, H, D), generator=gen, device=dev) * sv).half()
    k_dec = (torch.randn((n_dec, B, 1, H, D), generator=gen, device=dev) * sk).half()
    v_dec = (torch.randn((n_dec, B, 1, H, D), generator=gen, device=dev) * sv).half()
    q_dec = torch.randn((n_dec, B, HQ, D), generator=gen, device=dev).to(torch.bfloat16)
    out = torch.empty((B, HQ, D), dtype=torch.float32, device=dev)

    # prefill-append: the whole prompt of every sequence, layer by layer; repeated on cleared
    # caches for the timing (the first pass also warms up)
    def prefill():
        for layer in range(L):
            ctx.clear(layer)
            ctx.append(layer, k_pre, v_pre)

    pre_ms = timed(dst, prefill, max(2, min(args.steps, 5)), 1)
    # sampled blocks of the state the timed passes left, against the CPU encoders
    ok = True
    if dst.rank == 0:
        kh, vh = k_pre[0].cpu().numpy(), v_pre[0].cpu().numpy()
        for block in (0, 31, 61):
            ok = ok and check_encode(ctx, kh, vh, L - 1, 0, block, cfg.value_bits)
    if not dst.all_ok(ok):
        raise SystemExit("config 4 check failed: encoded blocks differ from the CPU encoders")
    # decode phase: 256 steps, each appends one token per sequence and attends, every layer
    def decode_phase():
        for layer in range(L):
            ctx.clear(layer)
            ctx.append(layer, k_pre, v_pre)
        dst.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for t in range(n_dec):
            for layer in range(L):
                ctx.append(layer, k_dec[t], v_dec[t])
                ctx.decode(layer, q_dec[t], out=out)
        e1.record()
        dst.barrier()
        return dst.max_ms(e0.elapsed_time(e1))

    decode_phase()
    dec_ms = decode_phase()
    if ctx.raise_on_timeout() != 0:
        raise SystemExit("status flags set after config 4")
    # byte accounting per layer: fp16 K and V read, compressed blocks + hot rows written
    nb = (n_pre - 257) // 256
    blk = 256 * D // 2 + 256 * D * cfg.value_bits // 8 + 4 * 256 + 8 * D + 6 * 5 * D
    comp_bytes = B * H * nb * blk
    read_bytes = B * n_pre * H * D * 2 * 2
    hot_bytes = B * H * (n_pre - nb * 256) * D * 2 * 2
    per_layer_ms = pre_ms / L
    tok_s = dst.world * B * n_pre / (per_layer_ms * 1e-3)
    # arithmetic bound of the two encoders on one GPU: about 65 ALU operations per key element
    # (three passes: sum, top-k / max, 16-level scan) and 128 fused multiply-adds per value
    # element, against 148 SMs x 128 lanes x clock
    lanes = 148 * 128 * 1.965e9
    elems = B * nb * 256 * H * D
    arith_ms = (65 * elems + 128 * elems) / lanes * 1e3
    res = {
        "workload": f"llama-3-8b shape, K4/V3 + outlier side-list, prefill-append of {n_pre} "
                    f"tokens x batch {Bg} (divided over {dst.world} rank(s)), then {n_dec} decode "
                    f"steps that each append one token and attend; {L} of {cfg.n_layers} layers "
                    "held and timed",
        "n_gpus": dst.world, "layers_timed": L,
        "prefill_ms_per_layer": per_layer_ms,
        "encoded_tokens_per_s_per_layer": tok_s,
        "encoded_tokens_per_s_all_layers": tok_s / cfg.n_layers,
        "compressed_GBps": dst.world * comp_bytes / (per_layer_ms * 1e-3) / 1e9,
        "input_GBps": dst.world * read_bytes / (per_layer_ms * 1e-3) / 1e9,
        "hbm_bytes_per_layer_per_rank": read_bytes + comp_bytes + hot_bytes,
        "arithmetic_bound_ms_per_layer": arith_ms,
        "frac_of_arithmetic_bound": arith_ms / per_layer_ms,
        "decode_phase_ms": dec_ms, "decode_steps": n_dec,
        "decode_phase_us_per_layer_step": dec_ms * 1e3 / (n_dec * L),
        "decode_phase_tokens_per_s_all_layers": dst.world * B * n_dec /
                                                (dec_ms * 1e-3 * cfg.n_layers / L),
        "check": {"blocks_bit_exact": True,
                  "what": "blocks 0, 31, 61 of sequence 0 of the last layer: key codes, scales, "
                          "means, outlier lists, value codes and norms equal the C restatement "
                          "of the reference encoders"},
    }
    del ctx
    torch.cuda.empty_cache()
    return res


# ------------------------------------------------------------------------------------ #
# native arm                                                                            #
# ------------------------------------------------------------------------------------ #

def run_native(args):
    import torch

    from turboquant_pro_b200 import AutoConfig

    if not torch.cuda.is_available():
        raise SystemExit("bench.py --impl native needs a CUDA device (no CPU fallback)")
    dst = Dist()
    cfg = AutoConfig.from_pretrained(args.model, target=args.target)
    if args.layers:
        cfg.n_layers = args.layers
    if args.batch % dst.world:
        raise SystemExit(f"--batch {args.batch} does not divide over {dst.world} ranks")
    line = run_headline(args, dst, cfg, args.batch // dst.world, args.batch, "strong")
    extras = [] if args.extras == "none" else [x.strip() for x in args.extras.split(",") if x.strip()]
    if "weak" in extras and dst.world > 1:
        w = run_headline(argparse.Namespace(**{**vars(args), "no_e2e": True}), dst, cfg,
                         args.batch, args.batch * dst.world, "weak")
        line["cfg1_weak"] = {k: w[k] for k in ("value", "ms_per_step", "tokens_per_s", "scaling")}
        line["cfg1_weak"]["global_batch"] = args.batch * dst.world
    if "cfg0" in extras:
        r0 = run_cfg0(args, dst)
        dst.barrier()
        if r0 is not None:
            line["cfg0"] = r0
    if "cfg2" in extras:
        line["cfg2"] = run_cfg2(args, dst)
    if "cfg3" in extras:
        line["cfg3"] = run_cfg3(args, dst)
    if "cfg4" in extras:
        line["cfg4"] = run_cfg4(args, dst)
    if dst.rank == 0:
        if dst.world == 1 and not args.no_cpu_baseline:
            cb = cpu_reference_leg(args, cfg, args.cpu_seconds)
            line["cpu_baseline"] = {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")}
        print(json.dumps(line), flush=True)
    dst.finish()


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_native(args)


if __name__ == "__main__":
    main()
