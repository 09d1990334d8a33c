#!/usr/bin/env python
"""Benchmark of the HQMQ hot path on B200: fused decode attention over the compressed KV cache
(headline) and KV-cache encode throughput, on synthetic data of the shapes the baseline names.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2|c3|c4_128k|c1] [--impl reference]

One "step" = one decode-attention call for one new query token per sequence over the whole resident
compressed cache of one layer (the cache is state that lives in HBM, like weights; the step's inputs
are the queries, its result the attention output).  Rank 0 prints one JSON line:
  value / unit   achieved HBM GB/s on the algorithmic compressed bytes, whole job (all ranks);
                 us_per_step and ms_per_step carry the latency side of the same measurement
  e2e            the same through the public Python API with the queries in pinned host memory
                 (H2D inside the timed region) and the output read back (D2H)
  roofline       the dominant kernel (attn_decode_kernel) against the measured HBM peak
  cpu_baseline   the oracle (a torch-CPU restatement of the reference's path) timed on a bounded sample
  encode         encoder throughput (tokens/s, GB/s) on a bounded slice of the same workload
With --gpus N > 1 (launched by torchrun, one rank per GPU) every rank holds its own batch shard of the
same shape (weak scaling by batch; no data-path collective).
"""
import argparse
import ctypes as C
import json
import math
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: B, Hq, Hkv, d, T, S, b_r, C, K-kind, V-kind
    "c1": dict(B=1, Hq=32, Hkv=8, d=128, T=4096, S=24, br=3, C=None, kk="randn", vk="randn", dtype="fp16",
               desc="Mistral-7B-shaped layer, s24_r3, no outliers"),
    "c2": dict(B=16, Hq=32, Hkv=8, d=128, T=32768, S=96, br=4, C=3.0, kk="hot", vk="randn", dtype="bf16",
               desc="Llama-3-8B-shaped GQA decode, s96_r4 + Med3x"),
    "c3": dict(B=32, Hq=28, Hkv=4, d=128, T=8192, S=192, br=6, C=3.0, kk="student", vk="randn", dtype="bf16",
               desc="Qwen2.5-7B-shaped outlier-heavy cache, s192_r6 + Med3x"),
    "c4_128k": dict(B=1, Hq=32, Hkv=8, d=128, T=131072, S=24, br=3, C=3.0, kk="spiky", vk="spiky", dtype="bf16",
                    desc="long-context single sequence, s24_r3 + Med3x"),
    "c5_layer": dict(B=64, Hq=64, Hkv=8, d=64, T=16384, S=96, br=4, C=3.0, kk="onehot", vk="onehot", dtype="bf16",
                     desc="gpt-oss-20b-shaped full-attention layer, s96_r4 + Med3x"),
    "c5_model": dict(B=64, Hq=64, Hkv=8, d=64, T=16384, S=96, br=4, C=3.0, kk="onehot", vk="onehot", dtype="bf16",
                     layers=24, window=128,
                     desc="gpt-oss-20b-shaped attention stack: 24 layers alternating full and 128-token sliding-window "
                          "attention, per step a one-token append-encode and a decode attention in every layer"),
}
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read+write of attn_fast_kernel divided by the algorithmic bytes of the same launch, from the ncu
# capture summarised in profiles/attn_decode_c2.md (batch 4 of the same workload; traffic scales with the tokens)
NCU_TRAFFIC_PER_ALGORITHMIC_BYTE = 1.10
L2_BYTES = 126e6     # B200 L2; a cache within twice this size is timed with a flush before every step


def synth(kind, shape, seed, device, dtype):
    """Seeded synthetic K/V with the value distribution the workload names."""
    B, H, T, d = shape
    g = torch.Generator(device=device).manual_seed(seed)
    gc = torch.Generator().manual_seed(seed)
    x = torch.randn(B, H, T, d, generator=g, device=device, dtype=torch.float32)
    if kind == "hot":
        for h in range(H):
            ch = torch.randperm(d, generator=gc)[:4].to(device)
            x[:, h, :, ch] *= 8.0
    elif kind == "onehot":
        for h in range(H):
            ch = torch.randperm(d, generator=gc)[:1].to(device)
            scale = math.exp(torch.rand(1, generator=gc).item() * math.log(200.0))
            x[:, h, :, ch] *= scale
    elif kind == "student":
        for h in range(H):
            ch = torch.randperm(d, generator=gc)[:2].to(device)
            z = torch.randn(B, T, 2, generator=g, device=device)
            chi = (torch.randn(B, T, 2, generator=g, device=device) ** 2 + torch.randn(B, T, 2, generator=g, device=device) ** 2) / 2
            x[:, h, :, ch] = 100.0 * z / chi.sqrt()
    elif kind == "spiky":
        m = torch.rand(B, H, T, d // 4, generator=g, device=device) < 0.005
        x = (x.view(B, H, T, d // 4, 4) * torch.where(m, 20.0, 1.0).unsqueeze(-1)).view(B, H, T, d)
    return x.to(dtype)


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled every 50 ms while the steps run."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.th = threading.Thread(target=self._read, daemon=True)
            self.th.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm = sorted(float(r[0]) for r in self.rows if r and r[0].replace(".", "").isdigit())
        mx = [float(r[1]) for r in self.rows if len(r) > 1 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 8 for n, v in zip(names, r[4:8]) if v.lower().startswith("active")})
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": reasons}


def hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return float(json.load(open(path))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


# ------------------------------------------------------------------------------------------------------
def cpu_port_run(w, sample_T, reps, threads=None):
    """The oracle (CPU restatement of the reference's path) on a bounded sample: B=1, sample_T tokens of
    the workload's distribution.  Returns seconds per decode step, encode seconds, and the sample's
    algorithmic bytes."""
    from oracle import hqmq_oracle as orc
    # all host threads of this process's CPU set, also under torchrun (which exports OMP_NUM_THREADS=1)
    avail = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    torch.set_num_threads(threads or max(1, avail))
    Hkv, Hq, d, S, br, Cm = w["Hkv"], w["Hq"], w["d"], w["S"], w["br"], w["C"]
    dtype = torch.bfloat16 if w["dtype"] == "bf16" else torch.float16
    K = synth(w["kk"], (1, Hkv, sample_T, d), 1002, "cpu", dtype)
    V = synth(w["vk"], (1, Hkv, sample_T, d), 1003, "cpu", dtype)
    Q = (torch.randn(1, Hq, 1, d, generator=torch.Generator().manual_seed(7)) / math.sqrt(d)).to(dtype)
    raw = orc.secondary_raw(1, Hkv, S, 42)
    jk, jv = orc.joint_codebook(raw[0, :, 0]), orc.joint_codebook(raw[0, :, 1])
    t0 = time.perf_counter()
    ek = orc.encode(K, jk, br, Cm)
    ev = orc.encode(V, jv, br, Cm)
    t_enc = time.perf_counter() - t0
    qmax = (1 << br) - 1
    kw = {}
    if Cm is not None:
        kw = dict(K_flags=ek["flags"], K_orig=K, V_flags=ev["flags"], V_orig=V)
    ts = []
    for _ in range(reps):
        t0 = time.perf_counter()
        orc.fused_attention(Q, ek["idx"], ek["rq"], ek["r_max"], jk, ev["idx"], ev["rq"], ev["r_max"], jv, qmax,
                            causal=False, **kw)
        ts.append(time.perf_counter() - t0)
    n = d // 4
    ib = math.ceil(math.log2(24 * S))
    per_tok = n * (ib + br) / 8 + 2
    nbytes = 2 * Hkv * sample_T * per_tok
    if Cm is not None:
        nbytes += 2 * Hkv * sample_T * n / 8 + 8 * (int(ek["flags"].sum()) + int(ev["flags"].sum()))
    return dict(step_s=sorted(ts)[len(ts) // 2], encode_s=t_enc, bytes=nbytes, tokens=sample_T,
                threads=torch.get_num_threads())


def dense_sdpa_us(B, Hq, Hkv, T, d, dtype, dev, reps=10):
    """Device time of torch's scaled_dot_product_attention (library kernel) for the same decode step over an
    UNcompressed 16-bit cache of the same shape: the number a reader compares the compressed path with.
    Random dense K/V (the values do not change the time); K/V are (B, H_kv, T, d) and the query heads of a
    group are folded into the query length, so the cache is read once per KV head like in the compressed path."""
    import torch.nn.functional as F
    G = Hq // Hkv
    K = torch.randn(B, Hkv, T, d, device=dev, dtype=dtype)
    V = torch.randn(B, Hkv, T, d, device=dev, dtype=dtype)
    Q = torch.randn(B, Hkv, G, d, device=dev, dtype=dtype)
    for _ in range(3):
        F.scaled_dot_product_attention(Q, K, V)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        F.scaled_dot_product_attention(Q, K, V)
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) / reps * 1e3
    return {"us_per_step": us, "bytes": 2 * K.numel() * K.element_size(), "GBps": 2 * K.numel() * K.element_size() / us / 1e3,
            "what": "torch scaled_dot_product_attention over a dense 16-bit cache of the same shape (query heads of a "
                    "KV group as query rows); the cache exceeds L2" if 2 * K.numel() * K.element_size() > 2 * L2_BYTES else
                    "torch scaled_dot_product_attention over a dense 16-bit cache of the same shape; cache within twice L2, not flushed"}


def run_model_sweep(args, w, rank, world, local):
    """Whole-stack decode step (BASELINE config 5): every layer appends one new token per sequence to its
    compressed cache (K and V, own Med3x median per call) and attends over it -- all tokens in even layers, the
    last `window` in odd ones.  With N ranks the KV heads (and their query heads) are split N ways (strong scaling:
    a fixed job), with no data-path collective.  Reports us per step and the compressed bytes the step reads."""
    import hqmq_b200 as hqmq
    from hqmq_b200 import dist as hd
    from hqmq_b200.cache import PackedKVCache
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist_
        dist = dist_
        dist.init_process_group("nccl", device_id=dev)
    B, Hq, Hkv, d, T, S, br, Cm, NL, win = (w[k] for k in ("B", "Hq", "Hkv", "d", "T", "S", "br", "C", "layers", "window"))
    _, hs = hd.kv_head_shard(B, Hkv, world, rank)
    h0, h1 = hs.start, hs.stop
    Hl, G = h1 - h0, Hq // Hkv
    dtype = torch.bfloat16
    full = hqmq.HQMQ(n_layers=NL, n_heads=Hkv, secondary_size=S, radius_bits=br, device=dev, seed=42)
    inner = hqmq.HQMQ(n_layers=NL, n_heads=Hl, secondary_size=S, radius_bits=br, device=dev, seed=42)
    inner.secondary_raw.data = full.secondary_raw.data[:, h0:h1].clone()     # this rank's heads of the same codebooks
    quant = hqmq.with_outlier_extraction(inner, Cm)
    n_steps = max(3, args.warmup) + 2 * args.steps + 8
    cache = PackedKVCache(quant, max_tokens=T + n_steps, sliding_window={l: win for l in range(1, NL, 2)})
    for l in range(NL):
        # a sliding-window layer only ever reads its last `win` tokens: a short prompt gives the same step
        Tl = T if l % 2 == 0 else 2 * win
        k = synth(w["kk"], (B, Hkv, Tl, d), 3000 + l, dev, dtype)[:, h0:h1]
        v = synth(w["vk"], (B, Hkv, Tl, d), 4000 + l, dev, dtype)[:, h0:h1]
        cache.update(k, v, l)
        del k, v
    cache.check()
    new = [(synth(w["kk"], (B, Hkv, 1, d), 5000 + i, dev, dtype)[:, h0:h1].contiguous(),
            synth(w["vk"], (B, Hkv, 1, d), 6000 + i, dev, dtype)[:, h0:h1].contiguous()) for i in range(4)]
    Q = (torch.randn(NL, B, Hl * G, 1, d, generator=torch.Generator().manual_seed(11 + rank)) / math.sqrt(d)).to(dtype).to(dev)
    O = torch.empty_like(Q)
    counter = [0]

    def step():
        i = counter[0] = counter[0] + 1
        for l in range(NL):
            k, v = new[(i + l) % 4]
            cache.update(k, v, l)
            cache.attend(Q[l], l, out=O[l])

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    for _ in range(max(3, args.warmup)):
        step()
    barrier()
    stream = torch.cuda.current_stream()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record(stream)
    for _ in range(args.steps):
        step()
    ev1.record(stream)
    barrier()
    dev_s = ev0.elapsed_time(ev1) * 1e-3
    # e2e: the step's queries come from pinned host memory and its outputs go back, with a sync per step
    Qh, Oh = Q.cpu().pin_memory(), torch.empty(O.shape, dtype=dtype).pin_memory()
    ev2, ev3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev2.record(stream)
    for _ in range(args.steps):
        Q.copy_(Qh, non_blocking=True)
        step()
        Oh.copy_(O, non_blocking=True)
        stream.synchronize()
    ev3.record(stream)
    barrier()
    e2e_s = ev2.elapsed_time(ev3) * 1e-3
    clocks = sampler.stop() if rank == 0 else None
    cache.check()
    read_bytes = 0
    for l in range(NL):
        Kp, Vp = cache._layers[l]
        vis = Kp.T if l % 2 == 0 else win
        for pk in (Kp, Vp):
            read_bytes += pk.algorithmic_bytes(T=vis, n_out=int(pk.n_outliers() * vis / max(pk.T, 1)))
    t = torch.tensor([dev_s, e2e_s], device=dev, dtype=torch.float64)
    tb = torch.tensor([float(read_bytes)], device=dev, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(tb, op=dist.ReduceOp.SUM)
    if rank == 0:
        step_s, e2e_step = float(t[0]) / args.steps, float(t[1]) / args.steps
        peak, peak_kind = hbm_peak()
        gbs = float(tb[0]) / step_s / 1e9
        print(json.dumps({
            "metric": "decode step over the whole attention stack: us per step (append-encode + attention in every layer)",
            "value": step_s * 1e6, "unit": "us", "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup),
            "ms_per_step": step_s * 1e3, "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
            "dtype": "f16 mma / f32 accumulate", "data": "synthetic",
            "config": {"workload": args.workload, "desc": w["desc"], "batch": B, "q_heads": Hq, "kv_heads": Hkv, "d_head": d,
                       "context": T, "layers": NL, "window": win, "S": S, "radius_bits": br, "median_mult": Cm,
                       "sharding": f"KV heads x{world} ({Hl} per GPU)",
                       "l2": "the compressed caches read per step exceed L2 many times over (no flush needed)"},
            "compressed_bytes_read_per_step": float(tb[0]), "achieved_GBps_all_gpus": gbs,
            "e2e": {"value": e2e_step * 1e6, "unit": "us", "h2d_bytes_per_step": Qh.numel() * Qh.element_size(),
                    "d2h_bytes_per_step": Oh.numel() * Oh.element_size()},
            "gpu_launches_note": "per layer and step: 2 append-encode calls of 3 kernels each, attention + merge kernel",
            "gpu_launches": NL * 8 * args.steps,
            "roofline": {"bound": "hbm", "achieved": gbs / world, "peak": peak, "unit": "GB/s", "frac": gbs / world / peak,
                         "peak_kind": f"of {peak_kind}", "traffic": None,
                         "note": "whole step (host-bound appends included), not one kernel"},
            "clocks": clocks}), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def run_reference_arm(args, w, rank, world):
    """--impl reference: the reference's CPU implementation of the path (its torch restatement under
    oracle/, since the Python reference itself does not travel to the GPU box), all host threads, on a
    bounded sample of the same workload."""
    if rank != 0:
        return
    sample_T = min(w["T"], 4096)
    ts = []
    info = None
    for i in range(args.warmup + args.steps):
        info = cpu_port_run(w, sample_T, reps=1)
        if i >= args.warmup:
            ts.append(info["step_s"])
    step = sum(ts) / len(ts)
    gbs = info["bytes"] / step / 1e9
    line = {
        "metric": "decode-attn achieved HBM GB/s on the compressed cache (us/step in us_per_step)", "value": gbs,
        "unit": "GB/s", "impl": "reference", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": step * 1e3, "us_per_step": step * 1e6, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "desc": w["desc"], "sample": f"B=1, T={sample_T} of the workload"},
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": info["threads"], "kind": "port",
                         "sample": f"B=1, H_kv={w['Hkv']}, T={sample_T}: decode_packed + SDPA in fp32 per step"},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "encode": {"tokens_per_s": sample_T / info["encode_s"], "sample_tokens": sample_T},
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=500)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--kv-splits", type=int, default=0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--batch", type=int, default=0, help="override the workload's batch size")
    ap.add_argument("--context", type=int, default=0, help="override the workload's context length")
    ap.add_argument("--no-med3x", action="store_true", help="encode without outlier extraction")
    ap.add_argument("--no-ofrag", action="store_true",
                    help="K cache without fragment records (attention merges K outliers from flags / side buffer)")
    ap.add_argument("--push", action="store_true",
                    help="with --seq-split: exchange the partials by direct stores into the peers' memory (NVLink, "
                         "CUDA-IPC mapped buffers, bounded wait on local flag words) instead of an NCCL all_gather")
    ap.add_argument("--no-dense", action="store_true", help="skip the dense 16-bit SDPA comparison line")
    ap.add_argument("--seq-split", action="store_true",
                    help="with N > 1: split ONE cache by sequence across the ranks (flash-decoding over NVLink: "
                         "partials + all_gather + merge) instead of giving every rank its own batch shard")
    args = ap.parse_args()
    w = dict(WORKLOADS[args.workload])
    if args.batch:
        w["B"] = args.batch
    if args.context:
        w["T"] = args.context
    if args.no_med3x:
        w["C"] = None
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))

    if args.impl == "reference":
        run_reference_arm(args, w, rank, world)
        return
    if "layers" in w:
        run_model_sweep(args, w, rank, world, local)
        return

    import hqmq_b200 as hqmq
    from hqmq_b200 import _lib
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist_
        dist = dist_
        dist.init_process_group("nccl", device_id=dev)

    B, Hq, Hkv, d, T, S, br, Cm = (w[k] for k in ("B", "Hq", "Hkv", "d", "T", "S", "br", "C"))
    seq_mode = args.seq_split and world > 1
    T_full = T
    if seq_mode:
        from hqmq_b200 import dist as hd
        t_lo, t_hi = hd.seq_shard(T, world, rank)
        T = t_hi - t_lo
    dtype = torch.bfloat16 if w["dtype"] == "bf16" else torch.float16
    inner = hqmq.HQMQ(n_layers=1, n_heads=Hkv, secondary_size=S, radius_bits=br, device=dev, seed=42)
    quant = hqmq.with_outlier_extraction(inner, Cm) if Cm is not None else inner

    # ---- build the resident compressed cache (untimed set-up) -------------------------------------------
    caches = []
    enc_times = []
    inner.tables(0, 0, dev), inner.tables(0, 1, dev)     # codebook tables are built once, outside any timing
    for kv in (0, 1):                                    # first launches load the kernels: keep that out of the timing
        quant.encode(synth("randn", (1, Hkv, 64, d), 5, dev, dtype), 0, kv)
    torch.cuda.synchronize()
    for kv, kind, seed in ((0, w["kk"], 1002), (1, w["vk"], 1003)):
        x = synth(kind, (B, Hkv, T, d), seed + 100 * rank, dev, dtype)
        cap = None if Cm is None else max(1024, int(0.2 * T * (d // 4)))
        # the whole tensor is encoded 4 times into fresh caches: the first pass warms the device (first use of
        # a launch configuration costs milliseconds), the median of the other three is reported
        reps = []
        for rep in range(4):
            pk = inner.new_cache(B, T, d, dev, scale_dtype=dtype, with_outliers=Cm is not None, out_dtype=dtype, out_cap=cap,
                                 ofrag=kv == 0 and Cm is not None and not args.no_ofrag)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            quant.encode(x, 0, kv, out=pk)
            e1.record()
            torch.cuda.synchronize()
            reps.append(e0.elapsed_time(e1) * 1e-3)
        enc_times.append(sorted(reps[1:])[1])
        if Cm is not None and int(pk.out_count.max()) > pk.out_cap:
            raise RuntimeError("outlier side buffer too small for this data")
        caches.append(pk)
        del x
    Kp, Vp = caches
    tk, tv = inner.tables(0, 0, dev), inner.tables(0, 1, dev)
    algo_bytes = Kp.algorithmic_bytes() + Vp.algorithmic_bytes()
    enc_in_bytes = 2 * B * Hkv * T * d * 2
    enc_tokens_per_s = B * T / sum(enc_times)
    enc_gbs = (enc_in_bytes + algo_bytes) / sum(enc_times) / 1e9
    outl_frac = [(pk.n_outliers() / (B * Hkv * T * (d // 4))) if Cm is not None else 0.0 for pk in caches]

    # decode-time append: one token per sequence and call into a small cache, through the public encode()
    ap_cache = inner.new_cache(B, 256, d, dev, scale_dtype=dtype, with_outliers=Cm is not None, out_dtype=dtype,
                               ofrag=Cm is not None)
    ap_x = [synth(w["kk"], (B, Hkv, 1, d), 2000 + i, dev, dtype) for i in range(4)]
    quant.encode(synth(w["kk"], (B, Hkv, 64, d), 1999, dev, dtype), 0, 0, out=ap_cache)
    for i in range(16):
        quant.encode(ap_x[i % 4], 0, 0, out=ap_cache)
    torch.cuda.synchronize()
    t_ap = time.perf_counter()
    for i in range(128):
        quant.encode(ap_x[i % 4], 0, 0, out=ap_cache)
    torch.cuda.synchronize()
    append_us = (time.perf_counter() - t_ap) / 128 * 1e6
    del ap_cache, ap_x

    # ---- one decode step through the C ABI, descriptors built once -------------------------------------
    Qh = (torch.randn(B, Hq, 1, d, generator=torch.Generator().manual_seed(7 + rank)) / math.sqrt(d)).to(dtype).pin_memory()
    Oh = torch.empty(B, Hq, 1, d, dtype=dtype).pin_memory()
    Qd = Qh.to(dev)
    Od = torch.empty_like(Qd)
    a = _lib.AttnArgs()
    a.struct_size = C.sizeof(_lib.AttnArgs)
    a.layout = 0
    a.q_dtype = a.o_dtype = _lib.dtype_enum(dtype)
    a.Q, a.O = Qd.data_ptr(), Od.data_ptr()
    a.q_stride = (C.c_int64 * 3)(*Qd.stride()[:3])
    a.o_stride = (C.c_int64 * 3)(*Od.stride()[:3])
    a.B, a.H_q, a.H_kv, a.T_q, a.T_kv, a.d = B, Hq, Hkv, 1, T, d
    a.r_qmax, a.causal, a.window, a.softmax_scale, a.kv_splits = Kp.qmax, 0, 0, 0.0, args.kv_splits
    a.K, a.V = Kp.c_struct(), Vp.c_struct()
    a.table_K, a.table_V = tk["table16"].data_ptr(), tv["table16"].data_ptr()
    L = _lib.lib()
    ws_bytes = L.hqmq_attn_workspace_bytes(C.byref(a))
    if seq_mode:
        part = torch.empty(B, Hq, 1, d + 2, dtype=torch.float32, device=dev)
        allp = torch.empty(world, B, Hq, 1, d + 2, dtype=torch.float32, device=dev)
        a.partials_only, a.partials = 1, part.data_ptr()
        ws_bytes = L.hqmq_attn_workspace_bytes(C.byref(a))
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
    stream = torch.cuda.current_stream()
    px = hd.PushExchange(B * Hq, d, dev) if seq_mode and args.push else None

    def step():
        rc = L.hqmq_attn_decode(C.byref(a), ws.data_ptr(), ws_bytes, stream.cuda_stream)
        if rc:
            raise RuntimeError(L.hqmq_strerror(rc).decode())
        if px is not None:
            px.step(part, Od)
        elif seq_mode:
            dist.all_gather_into_tensor(allp.view(world * B, Hq, 1, d + 2), part)
            rc = L.hqmq_combine_partials(allp.data_ptr(), world, B * Hq, d, 1, _lib.dtype_enum(dtype), Od.data_ptr(),
                                         stream.cuda_stream)
            if rc:
                raise RuntimeError(L.hqmq_strerror(rc).decode())

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    if px is not None:
        # the pushed exchange must reproduce the all_gather exchange bit for bit (same blocks, same merge order)
        step()
        pushed = Od.clone()
        px_keep, px = px, None
        step()
        px = px_keep
        torch.cuda.synchronize()
        px.check()
        if not torch.equal(pushed, Od):
            raise RuntimeError("pushed exchange and all_gather exchange disagree")
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    for _ in range(max(3, args.warmup)):
        step()
    barrier()
    # the timed region: exactly `steps` steps between barriers.  A cache of more than twice the L2 size cannot
    # stay in it; for a smaller one a 256 MiB buffer is rewritten before every timed step (outside the step's
    # own pair of events), so that every step reads its cache from HBM.
    need_flush = algo_bytes <= 2 * L2_BYTES
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if need_flush else None

    def timed(n, one_step):
        """Device seconds of n steps: one event pair around the loop, or one per step when L2 is flushed between."""
        if flush_buf is None:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(n):
                one_step()
            e1.record(stream)
            barrier()
            return e0.elapsed_time(e1) * 1e-3
        pairs = []
        for i in range(n):
            flush_buf.fill_(i & 255)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            one_step()
            e1.record(stream)
            pairs.append((e0, e1))
        barrier()
        return sum(a_.elapsed_time(b_) for a_, b_ in pairs) * 1e-3

    barrier()
    dev_s = timed(args.steps, step)

    # e2e: host queries -> device, attention, output -> host, every step
    def e2e_step():
        Qd.copy_(Qh, non_blocking=True)
        step()
        Oh.copy_(Od, non_blocking=True)
        stream.synchronize()        # the caller consumes the output before the next token

    for _ in range(3):
        e2e_step()
    barrier()
    e2e_s = timed(args.steps, e2e_step)
    # spread of single steps: each of up to 50 steps between its own pair of events (after a flush where one applies)
    def per_step_us(n):
        pairs = []
        for i in range(n):
            if flush_buf is not None:
                flush_buf.fill_(i & 255)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            step()
            e1.record(stream)
            pairs.append((e0, e1))
        barrier()
        return sorted(a_.elapsed_time(b_) * 1e3 for a_, b_ in pairs)
    spread = per_step_us(min(args.steps, 50))
    # sequence split: the same steps without the exchange and the merge, so that their cost can be split out
    local_s = None
    if seq_mode:
        def local_step():
            rc = L.hqmq_attn_decode(C.byref(a), ws.data_ptr(), ws_bytes, stream.cuda_stream)
            if rc:
                raise RuntimeError(L.hqmq_strerror(rc).decode())
        for _ in range(3):
            local_step()
        barrier()
        local_s = timed(args.steps, local_step)
    # a short timed region can fall between two nvidia-smi samples: keep the same step running (untimed)
    # until the sampler has seen the GPU under this load
    t_probe = time.perf_counter()
    while rank == 0 and not seq_mode and len(sampler.rows) < 6 and time.perf_counter() - t_probe < 2.0:
        for _ in range(20):
            step()
        stream.synchronize()
    barrier()
    clocks = sampler.stop() if rank == 0 else None

    if px is not None:
        px.check()
        px.close()
    t = torch.tensor([dev_s, e2e_s, local_s or 0.0], device=dev, dtype=torch.float64)
    tot_bytes = torch.tensor([float(algo_bytes)], device=dev, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(tot_bytes, op=dist.ReduceOp.SUM)
    dev_s, e2e_s, local_s = float(t[0]), float(t[1]), float(t[2])
    total_bytes = float(tot_bytes[0])
    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    step_s = dev_s / args.steps
    gbs = total_bytes / step_s / 1e9
    peak, peak_kind = hbm_peak()
    per_gpu_gbs = algo_bytes / step_s / 1e9
    line = {
        "metric": "decode-attn achieved HBM GB/s on the compressed cache (us/step in us_per_step)",
        "value": gbs, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup),
        "ms_per_step": step_s * 1e3, "us_per_step": step_s * 1e6, "higher_is_better": True, "scaling": "strong" if seq_mode else "weak",
        "vs_baseline": None, "dtype": "f16 mma / f32 accumulate", "data": "synthetic",
        "config": {"workload": args.workload, "desc": w["desc"], "batch_per_gpu": B, "global_batch": B if seq_mode else B * world,
                   "q_heads": Hq, "kv_heads": Hkv, "d_head": d, "context": T, "S": S, "radius_bits": br,
                   "median_mult": Cm, "outlier_fraction_K_V": outl_frac,
                   "k_fragment_records": bool(Kp.with_ofrag),
                   "sharding": (f"sequence x{world} (context {T_full} total, partials pushed into the peers' memory + local merge)" if px is not None
                                else f"sequence x{world} (context {T_full} total, partials all_gather + merge)") if seq_mode else f"batch x{world}",
                   "l2": "compressed cache per GPU exceeds twice the L2 size (inputs larger than L2, no flush needed)"
                   if not need_flush else "cache within twice the L2 size: 256 MiB rewritten before every timed step (L2 flushed)"},
        "us_per_step_median_min_rank0": [spread[len(spread) // 2], spread[0]],
        "compressed_bytes_per_step": total_bytes,
        "fp16_cache_bytes_equiv": 2 * 2 * B * Hkv * T * d * world,
        "e2e": {"value": total_bytes / (e2e_s / args.steps) / 1e9, "unit": "GB/s",
                "us_per_step": e2e_s / args.steps * 1e6,
                "h2d_bytes_per_step": Qh.numel() * Qh.element_size(), "d2h_bytes_per_step": Oh.numel() * Oh.element_size()},
        "gpu_launches": (5 if px is not None else 3 if seq_mode else 2) * args.steps,
        "roofline": {"bound": "hbm", "achieved": per_gpu_gbs, "peak": peak, "unit": "GB/s", "frac": per_gpu_gbs / peak,
                     "peak_kind": f"of {peak_kind}", "frac_of_8TBs_nominal": per_gpu_gbs / 8000.0,
                     "kernel": "attn_fast_kernel (+ combine_kernel, 3 % of the step, inside the same timed region)",
                     "traffic": NCU_TRAFFIC_PER_ALGORITHMIC_BYTE * algo_bytes if args.workload == "c2" else None,
                     "traffic_note": "ncu dram bytes of a batch-4 capture scaled by tokens (profiles/attn_decode_c2.md)"},
        "encode": {"tokens_per_s": enc_tokens_per_s * world, "GBps_per_gpu": enc_gbs, "frac_of_peak": enc_gbs / peak,
                   "tokens": B * T, "seconds_K_V": enc_times, "append_one_token_us_per_call": append_us,
                   "note": "one call per tensor over the whole (B, H_kv, T, d) input, Med3x median per call; median of 3 timed calls after 1 warm-up call"},
        "clocks": clocks,
    }
    if seq_mode:
        line["seq_split"] = {"local_attention_us": local_s / args.steps * 1e6,
                             "exchange_and_merge_us": (dev_s - local_s) / args.steps * 1e6,
                             "exchange": "pushed stores + bounded wait" if args.push else "NCCL all_gather",
                             "note": "max over ranks of each; local = the attention kernel writing its partial block"}
    if not args.no_dense and world == 1:
        try:
            line["dense_sdpa"] = dense_sdpa_us(B, Hq, Hkv, T, d, dtype, dev)
        except Exception as e:      # a comparison line only: never lose the bench line to it
            line["dense_sdpa"] = {"unavailable": f"{type(e).__name__}: {e}"[:200]}
    if not args.no_cpu_baseline:
        sample_T = min(T, 4096)
        info = cpu_port_run(w, sample_T, reps=3)
        line["cpu_baseline"] = {"value": info["bytes"] / info["step_s"] / 1e9, "unit": "GB/s", "cores": info["threads"],
                                "kind": "port", "us_per_step_sample": info["step_s"] * 1e6,
                                "encode_tokens_per_s": sample_T / info["encode_s"],
                                "sample": f"B=1, H_kv={Hkv}, T={sample_T} of the workload; decode_packed + SDPA fp32"}
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
