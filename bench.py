#!/usr/bin/env python
"""Benchmark of the HQMQ hot path on B200: fused decode attention over the compressed KV cache
(headline) and KV-cache encode throughput, on synthetic data of the shapes the baseline names.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2|c3|c4_128k|c4_1m|c1|c5_layer|c5_model]
                    [--impl reference] [--seq-split [--push]] [--weak]

One "step" = one decode-attention call for one new query token per sequence over the whole resident
compressed cache of one layer (the cache is state that lives in HBM, like weights; the step's inputs
are the queries, its result the attention output).  Rank 0 prints one JSON line:
  value / unit   achieved HBM GB/s on the algorithmic compressed bytes, whole job (all ranks), timed on the
                 device around the C-ABI call with every buffer resident; us_per_step carries the latency
  e2e            the same step through the package's public call (hqmq_b200.fused_attention_packed) with the
                 queries in pinned host memory (H2D inside the timed region) and the output read back (D2H)
  parity         one (batch, KV head) column of the timed cache's output against the fp32 oracle, before timing
  roofline       the dominant kernel against the measured HBM peak
  cpu_baseline   the reference's own CPU path timed on a bounded sample (its packages travel under oracle/_ref;
                 without them, the oracle port, and the line says which)
  encode         encoder throughput (tokens/s, GB/s) on the same workload
With --gpus N > 1 (launched by torchrun, one rank per GPU) the FIXED job is split by (KV head, then batch) over
the ranks and the step gathers the outputs with one all_gather inside the timed region (strong scaling); the
line then also carries the long-context sequence split (config 4) at N ranks with both of its exchanges.
--weak gives every rank its own batch shard instead; --seq-split times one sequence-split cache alone.
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
    "c4_1m": dict(B=1, Hq=32, Hkv=8, d=128, T=1048576, S=24, br=3, C=3.0, kk="spiky", vk="spiky", dtype="bf16",
                  desc="long-context single sequence of 1048576 tokens, s24_r3 + Med3x, encoded in calls of 131072 tokens"),
    "c5_layer": dict(B=64, Hq=64, Hkv=8, d=64, T=16384, S=96, br=4, C=3.0, kk="onehot", vk="onehot", dtype="bf16",
                     desc="gpt-oss-20b-shaped full-attention layer, s96_r4 + Med3x"),
    "c5_model": dict(B=64, Hq=64, Hkv=8, d=64, T=16384, S=96, br=4, C=3.0, kk="onehot", vk="onehot", dtype="bf16",
                     layers=24, window=128,
                     desc="gpt-oss-20b-shaped attention stack: 24 layers alternating full and 128-token sliding-window "
                          "attention, per step a one-token append-encode and a decode attention in every layer"),
}
ENC_CALL_TOKENS = 131072     # tokens per encode call (a chunked prefill; keeps a head's norms within torch.quantile's limit)
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read + dram__bytes_write of the attention kernel divided by the algorithmic bytes of the same launch,
# from one ncu capture per workload at a batch that still exceeds L2 (traffic grows in proportion to the tokens):
# c2 at batch 4 (163 MB algorithmic): 174.8 MB read + 4.1 MB written; c4_128k at its own size (124.3 MB): 154.7 + 4.7 MB;
# c5_layer at batch 16 (172.3 MB): 230.3 + 4.8 MB (fragment records and 16-byte-rounded payload slices are the excess).
NCU_TRAFFIC_PER_ALGORITHMIC_BYTE = {
    "c2": (1.097, "batch 4 of the same workload (163 MB, larger than L2), scaled by the tokens of this launch"),
    "c4_128k": (1.282, "the same workload at its full size (124 MB, L2 flushed before the launch)"),
    "c5_layer": (1.364, "batch 16 of the same workload (172 MB, larger than L2), scaled by the tokens of this launch"),
}
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


def host_threads():
    """All host threads of this process's CPU set, also under torchrun (which exports OMP_NUM_THREADS=1)."""
    avail = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    torch.set_num_threads(max(1, avail))
    return torch.get_num_threads()


# ------------------------------------------------------------------------------------------------------
# The CPU legs (the only code of this file that touches oracle/)
# ------------------------------------------------------------------------------------------------------
class CpuSample:
    """A bounded sample of a workload (B=1, sample_T tokens of its distribution) prepared once for the CPU legs:
    inputs, the packed tuple of the reference's decode path, and the time of one encode."""

    def __init__(self, w, sample_T):
        from oracle import hqmq_oracle as orc
        from oracle import make_ref
        self.threads = host_threads()
        Hkv, Hq, d, S, br, Cm = w["Hkv"], w["Hq"], w["d"], w["S"], w["br"], w["C"]
        dtype = torch.bfloat16 if w["dtype"] == "bf16" else torch.float16
        self.w, self.T, self.qmax = w, sample_T, (1 << br) - 1
        K = synth(w["kk"], (1, Hkv, sample_T, d), 1002, "cpu", dtype)
        V = synth(w["vk"], (1, Hkv, sample_T, d), 1003, "cpu", dtype)
        self.Q = (torch.randn(1, Hq, 1, d, generator=torch.Generator().manual_seed(7)) / math.sqrt(d)).to(dtype)
        raw = orc.secondary_raw(1, Hkv, S, 42)
        self.jk, self.jv = orc.joint_codebook(raw[0, :, 0]), orc.joint_codebook(raw[0, :, 1])
        self.kind, self.why_port = "port", None
        ref = None
        if make_ref.available():
            try:
                ref = make_ref.import_reference()
            except Exception as e:                      # noqa: BLE001  (report, then fall back to the port)
                self.why_port = f"oracle/_ref could not be imported: {type(e).__name__}: {e}"[:200]
        else:
            self.why_port = "oracle/_ref is absent (python oracle/make_ref.py was not run where the reference checkout exists)"
        # ---- encode: the reference's fake-quant calls (quantize_K / quantize_V), once, outside any step loop ----
        if ref is not None:
            q = ref.HQMQ(n_layers=1, n_heads=Hkv, secondary_size=S, radius_bits=br, device="cpu")
            if Cm is not None:
                q = ref.with_outlier_extraction(q, C=Cm)
            # T-slices keep the reference's (tokens x chunks x 24 S) similarity tensor within a few GB
            sl = max(64, min(sample_T, int(2e9 / (Hkv * (d // 4) * 24 * S * 4))))
            t0 = time.perf_counter()
            for lo in range(0, sample_T, sl):
                q.quantize_K(K[:, :, lo:lo + sl], 0)
                q.quantize_V(V[:, :, lo:lo + sl], 0)
            self.encode_s = time.perf_counter() - t0
            self.encode_what = (f"reference with_outlier_extraction(HQMQ).quantize_K/V in slices of {sl} tokens "
                                "(each slice takes its own Med3x median)")
            self.kind = "reference"
            self._ref_attn = ref.fused_attention_reference
        # the packed tuple the decode step reads (the reference's fake-quant does not return indices)
        t0 = time.perf_counter()
        ek, ev = orc.encode(K, self.jk, br, Cm), orc.encode(V, self.jv, br, Cm)
        if ref is None:
            self.encode_s = time.perf_counter() - t0
            self.encode_what = "oracle port of the encoder, one call over the sample"
            self._ref_attn = None
        self.ek, self.ev = ek, ev
        self._orc, self.K, self.V = orc, K, V
        n = d // 4
        ib = math.ceil(math.log2(24 * S))
        self.bytes = 2 * Hkv * sample_T * (n * (ib + br) / 8 + 2)
        if Cm is not None:
            self.bytes += 2 * Hkv * sample_T * n / 8 + 8 * (int(ek["flags"].sum()) + int(ev["flags"].sum()))

    def decode_step(self):
        """Seconds of one decode step over the sample: the reference's dequantise-then-SDPA function
        (fused_attention_reference, causal=False) on the packed tuple in fp32, or the port of it."""
        ek, ev = self.ek, self.ev
        t0 = time.perf_counter()
        if self._ref_attn is not None:
            self._ref_attn(self.Q.float(), ek["idx"], ek["rq"], ek["r_max"], self.jk, ev["idx"], ev["rq"], ev["r_max"], self.jv,
                           self.qmax, causal=False)
        else:
            self._orc.fused_attention(self.Q, ek["idx"], ek["rq"], ek["r_max"], self.jk, ev["idx"], ev["rq"], ev["r_max"],
                                      self.jv, self.qmax, causal=False)
        return time.perf_counter() - t0

    def describe(self, step_s):
        d = {"value": self.bytes / step_s / 1e9, "unit": "GB/s", "cores": self.threads, "kind": self.kind,
             "us_per_step_sample": step_s * 1e6, "encode_tokens_per_s": self.T / self.encode_s,
             "encode_what": self.encode_what,
             "sample": f"B=1, H_kv={self.w['Hkv']}, T={self.T} of the workload; decode = dequantise + SDPA in fp32 per step "
                       "(the Med3x merge of the flagged chunks is not part of the reference's decode function)"}
        if self.why_port:
            d["why_port"] = self.why_port
        return d


def oracle_column(Q1, ref_tuple_k, ref_tuple_v, jk, jv, qmax, K1, V1):
    """fp32 oracle output of ONE (batch, KV head) column: Q1 (1, G, 1, d), tuples sliced to (1, 1, T, n)."""
    from oracle import hqmq_oracle as orc
    ki, kr, ks, kf = ref_tuple_k
    vi, vr, vs, vf = ref_tuple_v
    return orc.fused_attention(Q1, ki, kr, ks, jk, vi, vr, vs, jv, qmax, causal=False,
                               K_flags=kf, K_orig=K1, V_flags=vf, V_orig=V1)


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


def triton_reference_us(Qd, Kp, Vp, tk, tv, qmax, reps=5):
    """The incumbent: the reference's own Triton kernel (hqmq.fused_attention, causal=False) on this GPU, on the
    reference's packed tuple of the same cache (int32 indices and radius codes, fp16 scales and joint tables), with
    its default configuration for this device and the best of its decode tuning grid
    (experiments/51_kernel_autotune.py: block_q x block_kv x warps x stages).  Checked against our output first."""
    from oracle import make_ref
    if not make_ref.available():
        return {"unavailable": "oracle/_ref is absent (python oracle/make_ref.py was not run where the reference checkout exists)"}
    ref = make_ref.import_reference()
    ki, kr, ks, _ = Kp.to_reference()
    vi, vr, vs, _ = Vp.to_reference()
    Q16 = Qd.half()
    args = (Q16, ki, kr, ks.half(), tk["joint"].half(), vi, vr, vs.half(), tv["joint"].half())
    out = {"layout": "reference tuple: int32 idx + int32 radius code per chunk, fp16 scale per token",
           "bytes_read_reference_layout": int(2 * (ki.numel() * 8 + ks.numel() * 2))}

    def timed(**cfg):
        for _ in range(2):
            O = ref.fused_attention(*args, r_qmax=qmax, causal=False, **cfg)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            ref.fused_attention(*args, r_qmax=qmax, causal=False, **cfg)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps * 1e3, O

    best = (float("inf"), None)
    try:
        us, _ = timed()
        out["default_config_us"] = us
        best = (us, "device default")
    except Exception as e:                              # noqa: BLE001  (the reference's default for this device may not fit)
        out["default_config_us"] = None
        out["default_config_error"] = f"{type(e).__name__}: {e}"[:200]
    out["outlier_note"] = "the reference kernel has no outlier merge: flagged chunks (radius code 0) read as zeros"
    for bq in (16,):                # (the decode part of the reference's grid that fits this device's shared memory)
        for bk in (32, 64, 128):
            for nw in (4, 8):
                for ns in (1, 2, 3):
                    try:
                        t, _ = timed(block_q=bq, block_kv=bk, num_warps=nw, num_stages=ns)
                    except Exception:                   # noqa: BLE001  (a configuration that does not fit is skipped)
                        continue
                    if t < best[0]:
                        best = (t, f"block_q={bq}, block_kv={bk}, num_warps={nw}, num_stages={ns}")
    if best[1] is None:
        return {"unavailable": "no configuration of the reference kernel's tuning grid ran on this device",
                "default_config_error": out.get("default_config_error")}
    out["best_of_grid_us"], out["best_config"] = best
    return out


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
            "gpu_launches_note": "per layer and step: one append call of 3 kernels for K and V together, attention + merge kernel",
            "gpu_launches": NL * 5 * args.steps,
            "roofline": {"bound": "hbm", "achieved": gbs / world, "peak": peak, "unit": "GB/s", "frac": gbs / world / peak,
                         "peak_kind": f"of {peak_kind}", "traffic": None,
                         "note": "whole step (host-bound appends included), not one kernel"},
            "clocks": clocks}), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def run_reference_arm(args, w, rank, world):
    """--impl reference: the reference's own CPU implementation of the path on the box's host cores (its packages
    under oracle/_ref; the oracle port, with the reason stated, when they are absent), all host threads, on a
    bounded sample of the same workload.  The sample is encoded once; each step is one decode call."""
    if rank != 0:
        return
    sample_T = min(w["T"], 4096)
    cs = CpuSample(w, sample_T)
    ts = []
    for i in range(args.warmup + args.steps):
        t = cs.decode_step()
        if i >= args.warmup:
            ts.append(t)
    step = sum(ts) / len(ts)
    info = cs.describe(step)
    gbs = info["value"]
    line = {
        "metric": "decode-attn achieved HBM GB/s on the compressed cache (us/step in us_per_step)", "value": gbs,
        "unit": "GB/s", "impl": "reference", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": step * 1e3, "us_per_step": step * 1e6, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "desc": w["desc"], "sample": f"B=1, T={sample_T} of the workload",
                   "note": "GB/s on the sample's algorithmic compressed bytes: the per-byte rate is what carries over to "
                           "the full configuration, which does not fit a CPU run of minutes"},
        "cpu_baseline": info,
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "encode": {"tokens_per_s": sample_T / cs.encode_s, "sample_tokens": sample_T, "what": cs.encode_what},
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------------
def build_cache(hqmq, quant, inner, w, x_of, B, T, dev, dtype, no_ofrag, time_it=True):
    """Encode K and V of shape (B, H, T, d) into fresh native caches, in calls of at most ENC_CALL_TOKENS tokens
    (every call takes its own Med3x median, like a chunked prefill).  x_of(kv, t0, t1) returns the tokens [t0, t1)
    of tensor kv.  Returns the caches and the encode seconds per tensor (median of 3 timed passes after a warm-up
    pass when the tensor is encoded in one call; one timed pass otherwise)."""
    Cm, d = w["C"], w["d"]
    caches, enc_times = [], []
    for kv in (0, 1):
        cap = None if Cm is None else max(1024, int(0.2 * T * (d // 4)))
        calls = [(t0, min(T, t0 + ENC_CALL_TOKENS)) for t0 in range(0, T, ENC_CALL_TOKENS)]
        n_pass = 4 if (len(calls) == 1 and time_it) else 1
        x_one = x_of(kv, 0, T) if len(calls) == 1 else None
        reps = []
        if len(calls) > 1 and time_it:
            # one untimed call of the same size into a throw-away cache: allocator, attributes and tables are warm
            # before the single timed pass
            t0w, t1w = calls[0]
            pkw = inner.new_cache(B, t1w - t0w, d, dev, scale_dtype=dtype, with_outliers=Cm is not None, out_dtype=dtype,
                                  out_cap=None if Cm is None else max(1024, int(0.2 * (t1w - t0w) * (d // 4))),
                                  ofrag=kv == 0 and Cm is not None and not no_ofrag)
            quant.encode(x_of(kv, t0w, t1w), 0, kv, out=pkw)
            torch.cuda.synchronize()
            del pkw
        for rep in range(n_pass):
            pk = inner.new_cache(B, T, d, dev, scale_dtype=dtype, with_outliers=Cm is not None, out_dtype=dtype, out_cap=cap,
                                 ofrag=kv == 0 and Cm is not None and not no_ofrag)
            total = 0.0
            for (t0, t1) in calls:
                x = x_one if x_one is not None else x_of(kv, t0, t1)
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                quant.encode(x, 0, kv, out=pk)
                e1.record()
                torch.cuda.synchronize()
                total += e0.elapsed_time(e1) * 1e-3
            reps.append(total)
        enc_times.append(sorted(reps[1:])[len(reps[1:]) // 2] if len(reps) > 1 else reps[0])
        if Cm is not None and int(pk.out_count.max()) > pk.out_cap:
            raise RuntimeError("outlier side buffer too small for this data")
        caches.append(pk)
    return caches, enc_times


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
    ap.add_argument("--no-triton-ref", action="store_true", help="skip timing the reference's Triton kernel")
    ap.add_argument("--no-parity", action="store_true", help="skip the oracle check of one output column")
    ap.add_argument("--weak", action="store_true",
                    help="with N > 1: every rank gets its own batch shard of the workload's shape (no collective)")
    ap.add_argument("--seq-split", action="store_true",
                    help="with N > 1: split ONE cache by sequence across the ranks (flash-decoding over NVLink: "
                         "partials + all_gather + merge) instead of splitting the job by (KV head, batch)")
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
    from hqmq_b200 import dist as hd
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist_
        dist = dist_
        dist.init_process_group("nccl", device_id=dev)

    B, Hq, Hkv, d, T, S, br, Cm = (w[k] for k in ("B", "Hq", "Hkv", "d", "T", "S", "br", "C"))
    G = Hq // Hkv
    dtype = torch.bfloat16 if w["dtype"] == "bf16" else torch.float16
    seq_mode = args.seq_split and world > 1
    strong = world > 1 and not seq_mode and not args.weak
    # ---- this rank's part of the job ------------------------------------------------------------------------
    b_sl, h_sl, t_lo, t_hi = slice(0, B), slice(0, Hkv), 0, T
    med_group = None
    if strong:
        b_sl, h_sl = hd.kv_head_shard(B, Hkv, world, rank)
        if world > Hkv:          # a head's batch is split: its Med3x median is taken over the ranks that share it
            per = world // Hkv
            groups = [dist.new_group(list(range(h * per, (h + 1) * per))) for h in range(Hkv)]
            med_group = groups[rank // per]
    elif seq_mode:
        t_lo, t_hi = hd.seq_shard(T, world, rank)
    Bl, Hl, Tl = b_sl.stop - b_sl.start, h_sl.stop - h_sl.start, t_hi - t_lo
    full = hqmq.HQMQ(n_layers=1, n_heads=Hkv, secondary_size=S, radius_bits=br, device=dev, seed=42)
    inner = full
    if Hl != Hkv:
        inner = hqmq.HQMQ(n_layers=1, n_heads=Hl, secondary_size=S, radius_bits=br, device=dev, seed=42)
        inner.secondary_raw.data = full.secondary_raw.data[:, h_sl].clone()      # this rank's heads of the same codebooks
    quant = hqmq.with_outlier_extraction(inner, Cm) if Cm is not None else inner
    data_seed = 100 * rank if (args.weak and world > 1) else 0    # a fixed job has the same data whatever N is

    def x_of(kv, t0, t1):
        """Tokens [t0, t1) of this rank's part of tensor kv.  A long context is generated call by call (own seed)."""
        kind, seed = (w["kk"], 1002) if kv == 0 else (w["vk"], 1003)
        if T > ENC_CALL_TOKENS:
            x = synth(kind, (B, Hkv, t1 - t0, d), seed + data_seed + 7919 * ((t_lo + t0) // ENC_CALL_TOKENS), dev, dtype)
        else:
            x = synth(kind, (B, Hkv, T, d), seed + data_seed, dev, dtype)[:, :, t_lo + t0:t_lo + t1]
        return x[b_sl, h_sl].contiguous()

    # ---- build the resident compressed cache (untimed set-up) -------------------------------------------
    inner.tables(0, 0, dev), inner.tables(0, 1, dev)     # codebook tables are built once, outside any timing
    for kv in (0, 1):                                    # first launches load the kernels: keep that out of the timing
        quant.encode(synth("randn", (1, Hl, 64, d), 5, dev, dtype), 0, kv)
    torch.cuda.synchronize()
    if med_group is not None:
        # the batch of a head is split over ranks: Med3x medians over all of them (summed histograms), no encode timing
        caches, enc_times = [], [float("nan"), float("nan")]
        for kv in (0, 1):
            pk = inner.new_cache(Bl, Tl, d, dev, scale_dtype=dtype, with_outliers=True, out_dtype=dtype,
                                 out_cap=max(1024, int(0.2 * Tl * (d // 4))), ofrag=kv == 0 and not args.no_ofrag)
            hd.encode_split_batch(quant, x_of(kv, 0, Tl), 0, kv, out=pk, group=med_group)
            caches.append(pk)
    else:
        caches, enc_times = build_cache(hqmq, quant, inner, w, x_of, Bl, Tl, dev, dtype, args.no_ofrag)
    Kp, Vp = caches
    tk, tv = inner.tables(0, 0, dev), inner.tables(0, 1, dev)
    algo_bytes = Kp.algorithmic_bytes() + Vp.algorithmic_bytes()
    enc_in_bytes = 2 * Bl * Hl * Tl * d * 2
    enc_tokens_per_s = Bl * Tl * (Hl / Hkv) / sum(enc_times)      # a token = all KV heads, K and V, one layer
    enc_gbs = (enc_in_bytes + algo_bytes) / sum(enc_times) / 1e9
    outl_frac = [(pk.n_outliers() / (Bl * Hl * Tl * (d // 4))) if Cm is not None else 0.0 for pk in caches]

    # decode-time append: one token per sequence into a small cache, K and V of a layer per call as the cache's
    # update() does it (encode_pair); the figure is per TENSOR, i.e. half the time of a pair call
    ap_cache = [inner.new_cache(Bl, 256, d, dev, scale_dtype=dtype, with_outliers=Cm is not None, out_dtype=dtype,
                                ofrag=Cm is not None and kv == 0) for kv in (0, 1)]
    ap_x = [(synth(w["kk"], (Bl, Hl, 1, d), 2000 + i, dev, dtype), synth(w["vk"], (Bl, Hl, 1, d), 2100 + i, dev, dtype))
            for i in range(4)]
    quant.encode_pair(synth(w["kk"], (Bl, Hl, 64, d), 1999, dev, dtype), synth(w["vk"], (Bl, Hl, 64, d), 1998, dev, dtype),
                      0, ap_cache[0], ap_cache[1])
    for i in range(16):
        quant.encode_pair(ap_x[i % 4][0], ap_x[i % 4][1], 0, ap_cache[0], ap_cache[1])
    torch.cuda.synchronize()
    t_ap = time.perf_counter()
    for i in range(128):
        quant.encode_pair(ap_x[i % 4][0], ap_x[i % 4][1], 0, ap_cache[0], ap_cache[1])
    torch.cuda.synchronize()
    append_us = (time.perf_counter() - t_ap) / 256 * 1e6
    del ap_cache, ap_x

    # ---- one decode step through the C ABI, descriptors built once -------------------------------------
    Q_all = (torch.randn(B, Hq, 1, d, generator=torch.Generator().manual_seed(7 + data_seed)) / math.sqrt(d)).to(dtype)
    Qh = Q_all[b_sl, h_sl.start * G:h_sl.stop * G].contiguous().pin_memory()
    Qd = Qh.to(dev)
    Od = torch.empty_like(Qd)
    Ogath = torch.empty((world,) + tuple(Od.shape), dtype=dtype, device=dev) if strong else None
    Oh = torch.empty(tuple(Ogath.shape) if strong else tuple(Od.shape), dtype=dtype).pin_memory()
    a = _lib.AttnArgs()
    a.struct_size = C.sizeof(_lib.AttnArgs)
    a.layout = 0
    a.q_dtype = a.o_dtype = _lib.dtype_enum(dtype)
    a.Q, a.O = Qd.data_ptr(), Od.data_ptr()
    a.q_stride = (C.c_int64 * 3)(*Qd.stride()[:3])
    a.o_stride = (C.c_int64 * 3)(*Od.stride()[:3])
    a.B, a.H_q, a.H_kv, a.T_q, a.T_kv, a.d = Bl, Hl * G, Hl, 1, Tl, d
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
        if strong:
            dist.all_gather_into_tensor(Ogath, Od)      # the only collective of the partition: the outputs (B*H_q*d values)
        elif px is not None:
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

    # ---- parity of the cache that is about to be timed: one (batch, KV head) column against the fp32 oracle -------
    parity = None
    if rank == 0 and not seq_mode and not args.no_parity:
        O32 = torch.empty(Qd.shape, dtype=torch.float32, device=dev)
        hqmq.fused_attention_packed(Qd, Kp, Vp, tk["table16"], tv["table16"], out=O32)
        col_b, col_h = 0, Hl - 1
        ref_k = tuple(None if t is None else t[col_b:col_b + 1, col_h:col_h + 1].cpu() for t in Kp.to_reference())
        ref_v = tuple(None if t is None else t[col_b:col_b + 1, col_h:col_h + 1].cpu() for t in Vp.to_reference())
        K1 = torch.cat([x_of(0, t0, min(Tl, t0 + ENC_CALL_TOKENS))[col_b:col_b + 1, col_h:col_h + 1].cpu()
                        for t0 in range(0, Tl, ENC_CALL_TOKENS)], dim=2)
        V1 = torch.cat([x_of(1, t0, min(Tl, t0 + ENC_CALL_TOKENS))[col_b:col_b + 1, col_h:col_h + 1].cpu()
                        for t0 in range(0, Tl, ENC_CALL_TOKENS)], dim=2)
        want = oracle_column(Qd[col_b:col_b + 1, col_h * G:(col_h + 1) * G].cpu(), ref_k, ref_v,
                             tk["joint"][col_h:col_h + 1].cpu(), tv["joint"][col_h:col_h + 1].cpu(), Kp.qmax, K1, V1)
        got = O32[col_b:col_b + 1, col_h * G:(col_h + 1) * G].cpu()
        parity = {"max_abs": float((got - want).abs().max()), "rel_l2": float((got - want).norm() / want.norm()),
                  "column": f"batch {col_b}, KV head {h_sl.start + col_h} of this rank: {G} query heads x {d} values, fp32 output",
                  "tolerance": "2e-3 max-abs, 1e-3 relative L2"}
        if not (parity["max_abs"] < 2e-3 and parity["rel_l2"] < 1e-3):
            raise RuntimeError(f"the cache that was about to be timed fails parity with the oracle: {parity}")
        del O32, ref_k, ref_v, K1, V1
        torch.cuda.empty_cache()

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

    # e2e: the call a user of the package makes, host queries -> device, attention, output -> host, every step
    def e2e_step():
        Qd.copy_(Qh, non_blocking=True)
        if seq_mode:
            step()
        else:
            hqmq.fused_attention_packed(Qd, Kp, Vp, tk["table16"], tv["table16"], kv_splits=args.kv_splits or None, out=Od)
            if strong:
                dist.all_gather_into_tensor(Ogath, Od)
        Oh.copy_(Ogath if strong else Od, non_blocking=True)
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
    # the same steps without the exchange (and the merge), so that its cost can be split out
    local_s = None
    if seq_mode or strong:
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
    while rank == 0 and world == 1 and len(sampler.rows) < 6 and time.perf_counter() - t_probe < 2.0:
        for _ in range(20):
            step()
        stream.synchronize()
    barrier()
    clocks = sampler.stop() if rank == 0 else None

    if px is not None:
        px.check()
        px.close()
    t = torch.tensor([dev_s, e2e_s, local_s or 0.0], device=dev, dtype=torch.float64)
    tot = torch.tensor([float(algo_bytes), float(Bl * Tl * Hl) / Hkv / max(sum(enc_times), 1e-12)], device=dev, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(tot, op=dist.ReduceOp.SUM)
    dev_s, e2e_s, local_s = float(t[0]), float(t[1]), float(t[2])
    total_bytes = float(tot[0])
    # the long-context sequence split at N ranks rides along in the line of a split job (collective: every rank takes part)
    c4 = None
    if strong and args.workload == "c2":
        del caches, Kp, Vp, ws
        torch.cuda.empty_cache()
        c4 = seq_split_extra(hqmq, hd, _lib, dist, dev, rank, world, steps=min(args.steps, 100))
    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    step_s = dev_s / args.steps
    gbs = total_bytes / step_s / 1e9
    peak, peak_kind = hbm_peak()
    per_gpu_gbs = algo_bytes / step_s / 1e9
    ring = Tl >= 1024 and Bl * Hl * ((Tl + 15) // 16) >= 148 * 4 * 15     # the library's choice of kernel (csrc/attn.cu)
    kernel = ("attn_ring_kernel (merges its partials itself: one launch per step)" if ring
              else "attn_fast_kernel (+ combine_kernel inside the same timed region)")
    traffic_ratio, traffic_from = (NCU_TRAFFIC_PER_ALGORITHMIC_BYTE.get(args.workload, (None, None))
                                   if (Cm is not None and not args.no_ofrag) else (None, None))
    sharding = (f"sequence x{world} (context {T} total, partials pushed into the peers' memory + local merge)" if px is not None
                else f"sequence x{world} (context {T} total, partials all_gather + merge)" if seq_mode
                else f"fixed job split by (KV head, batch): {Hl} KV heads x {Bl} sequences per GPU, outputs all_gathered" if strong
                else f"batch x{world}")
    line = {
        "metric": "decode-attn achieved HBM GB/s on the compressed cache (us/step in us_per_step)",
        "value": gbs, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup),
        "ms_per_step": step_s * 1e3, "us_per_step": step_s * 1e6, "higher_is_better": True,
        "scaling": "weak" if (args.weak or world == 1) else "strong",
        "vs_baseline": None, "dtype": "f16 mma / f32 accumulate", "data": "synthetic",
        "config": {"workload": args.workload, "desc": w["desc"], "batch_per_gpu": Bl, "global_batch": B * world if args.weak else B,
                   "q_heads": Hq, "kv_heads": Hkv, "d_head": d, "context": T, "S": S, "radius_bits": br,
                   "median_mult": Cm, "outlier_fraction_K_V": outl_frac,
                   "k_fragment_records": bool(caches[0].with_ofrag) if c4 is None else not args.no_ofrag,
                   "sharding": sharding,
                   "l2": "compressed cache per GPU exceeds twice the L2 size (inputs larger than L2, no flush needed)"
                   if not need_flush else "cache within twice the L2 size: 256 MiB rewritten before every timed step (L2 flushed)"},
        "us_per_step_median_min_rank0": [spread[len(spread) // 2], spread[0]],
        "compressed_bytes_per_step": total_bytes,
        "fp16_cache_bytes_equiv": 2 * 2 * B * Hkv * T * d * (world if args.weak else 1),
        "e2e": {"value": total_bytes / (e2e_s / args.steps) / 1e9, "unit": "GB/s",
                "us_per_step": e2e_s / args.steps * 1e6, "through": "hqmq_b200.fused_attention_packed" + (" + all_gather" if strong else ""),
                "h2d_bytes_per_step": Qh.numel() * Qh.element_size(), "d2h_bytes_per_step": Oh.numel() * Oh.element_size()},
        "gpu_launches": (5 if px is not None else 3 if (seq_mode or strong) else 2) * args.steps,
        "parity": parity,
        "roofline": {"bound": "hbm", "achieved": per_gpu_gbs, "peak": peak, "unit": "GB/s", "frac": per_gpu_gbs / peak,
                     "peak_kind": f"of {peak_kind}", "frac_of_8TBs_nominal": per_gpu_gbs / 8000.0, "kernel": kernel,
                     "traffic": traffic_ratio * algo_bytes if traffic_ratio else None,
                     "traffic_note": f"dram read + write bytes of one ncu capture of this kernel at {traffic_from}" if traffic_ratio else
                                     "no ncu capture of this workload"},
        "encode": {"tokens_per_s": float(tot[1]), "GBps_per_gpu": enc_gbs, "frac_of_peak": enc_gbs / peak,
                   "tokens": B * T, "seconds_K_V": enc_times, "append_one_token_us_per_call": append_us,
                   "note": f"calls of at most {ENC_CALL_TOKENS} tokens per tensor over the whole (B, H_kv, T, d) input, Med3x median "
                           "per call; median of 3 timed passes after 1 warm-up pass (one timed pass after one warm-up call when a tensor takes several calls); "
                           "append_one_token_us_per_call: one token per sequence, host wall clock over 128 K + V pair calls "
                           "(encode_pair, what the cache's update() issues) divided by the 256 tensors"},
        "clocks": clocks,
    }
    if seq_mode or strong:
        line["split"] = {"local_attention_us": local_s / args.steps * 1e6,
                         "exchange_us": (dev_s - local_s) / args.steps * 1e6,
                         "exchange": "all_gather of the outputs" if strong else
                                     "pushed stores + bounded wait + merge" if args.push else "NCCL all_gather of the partials + merge",
                         "note": "max over ranks of each; local = the attention kernels alone"}
    if c4 is not None:
        line["c4_seq_split"] = c4
    if not args.no_dense and world == 1:
        try:
            line["dense_sdpa"] = dense_sdpa_us(B, Hq, Hkv, T, d, dtype, dev)
        except Exception as e:      # a comparison line only: never lose the bench line to it
            line["dense_sdpa"] = {"unavailable": f"{type(e).__name__}: {e}"[:200]}
    if not args.no_triton_ref and world == 1 and T <= 131072:
        try:
            line["triton_reference"] = triton_reference_us(Qd, caches[0], caches[1], tk, tv, caches[0].qmax)
        except Exception as e:      # noqa: BLE001
            line["triton_reference"] = {"unavailable": f"{type(e).__name__}: {e}"[:300]}
    if not args.no_cpu_baseline:
        cs = CpuSample(w, min(T, 4096))
        ts = sorted(cs.decode_step() for _ in range(3))
        line["cpu_baseline"] = cs.describe(ts[1])
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def seq_split_extra(hqmq, hd, _lib, dist, dev, rank, world, steps):
    """Config 4 (one sequence of 131072 tokens, s24_r3 + Med3x) split by sequence over the ranks, both exchanges:
    local attention, NCCL all_gather + merge, pushed stores + merge (us per step, max over ranks, L2 flushed)."""
    w = WORKLOADS["c4_128k"]
    B, Hq, Hkv, d, T, S, br, Cm = (w[k] for k in ("B", "Hq", "Hkv", "d", "T", "S", "br", "C"))
    dtype = torch.bfloat16
    t_lo, t_hi = hd.seq_shard(T, world, rank)
    inner = hqmq.HQMQ(n_layers=1, n_heads=Hkv, secondary_size=S, radius_bits=br, device=dev, seed=42)
    quant = hqmq.with_outlier_extraction(inner, Cm)
    caches = []
    for kv, kind, seed in ((0, w["kk"], 1002), (1, w["vk"], 1003)):
        x = synth(kind, (B, Hkv, T, d), seed, dev, dtype)[:, :, t_lo:t_hi].contiguous()
        caches.append(quant.encode(x, 0, kv))
        del x
    Kp, Vp = caches
    tk, tv = inner.tables(0, 0, dev), inner.tables(0, 1, dev)
    Qd = (torch.randn(B, Hq, 1, d, generator=torch.Generator().manual_seed(7)) / math.sqrt(d)).to(dtype).to(dev)
    Od = torch.empty_like(Qd)
    part = torch.empty(B, Hq, 1, d + 2, dtype=torch.float32, device=dev)
    allp = torch.empty(world, B, Hq, 1, d + 2, dtype=torch.float32, device=dev)
    px = hd.PushExchange(B * Hq, d, dev)
    L = _lib.lib()
    stream = torch.cuda.current_stream()
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def local():
        hqmq.fused_attention_packed(Qd, Kp, Vp, tk["table16"], tv["table16"], partials=part)

    def gathered():
        local()
        dist.all_gather_into_tensor(allp.view(world * B, Hq, 1, d + 2), part)
        rc = L.hqmq_combine_partials(allp.data_ptr(), world, B * Hq, d, 1, _lib.dtype_enum(dtype), Od.data_ptr(), stream.cuda_stream)
        if rc:
            raise RuntimeError(L.hqmq_strerror(rc).decode())

    def pushed():
        local()
        px.step(part.view(B * Hq, d + 2), Od.view(B * Hq, d))

    def timed(fn):
        for _ in range(3):
            fn()
        dist.barrier()
        torch.cuda.synchronize()
        pairs = []
        for i in range(steps):
            flush_buf.fill_(i & 255)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            fn()
            e1.record(stream)
            pairs.append((e0, e1))
        dist.barrier()
        torch.cuda.synchronize()
        t = torch.tensor([sum(a.elapsed_time(b) for a, b in pairs) / steps * 1e3], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    gathered()
    want = Od.clone()
    pushed()
    torch.cuda.synchronize()
    px.check()
    same = bool(torch.equal(want, Od))
    out = {"workload": "c4_128k", "context": T, "ranks": world, "local_attention_us": timed(local),
           "all_gather_step_us": timed(gathered), "pushed_step_us": timed(pushed), "pushed_equals_gathered": same,
           "note": "us per step, max over ranks, 256 MiB rewritten before every timed step; exchange + merge = step - local"}
    px.check()
    px.close()
    return out


if __name__ == "__main__":
    main()
