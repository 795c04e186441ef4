#!/usr/bin/env python3
"""Benchmark of the TurboQuant hot path on B200: decode attention over a packed KV cache.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--ctx 16384] [--impl reference] [--no-extra]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

Workload (synthetic stand-in with the shapes of a Llama-3.2-1B decode step): 16 layers, 32 query heads,
8 KV heads, head_dim 64, keys 4 bits / values 2 bits, batch 32, context 16,384 tokens already in the
cache, one new token per sequence per step.  K entries ~ N(0,1) with 4 outlier channels per
(layer, KV head) scaled x20, V entries ~ N(0,1), bf16.  One step = for every layer: quantise and append
the new K/V token, then attend over the whole packed cache (grouped-query heads) -- the fused
decode_step call: one launch per layer.

N > 1: KV heads are sharded over the ranks (8/N per rank, with their 4 query heads each); there is no
collective on the path, total work is fixed ("strong" scaling), value = batch / max-over-ranks step time.

One JSON line is printed by rank 0:
  value     tokens/s with everything resident in HBM: the step is captured once in a CUDA graph
            (16 launches per step) and K replays are timed with CUDA events
  e2e       the same step fed from pinned host buffers: H2D of q/k/v of all layers, the step, D2H of the
            attention output, every step; uploads and downloads run on copy streams over two alternating
            buffer sets, so they overlap the neighbouring steps' kernels
  roofline  HBM roofline of the one kernel of the path (decode_fused_kernel); bytes per launch are the packed
            K/V rows and norms of one layer; its duration is measured with CUDA events in an extra pass
            of the same steps launched eagerly (events cannot be read inside a captured graph), one event
            pair per launch
  cpu_baseline  the upstream project's own OpenMP kernels (compiled in place into oracle/_ref; the CPU port
            under oracle/ where that library is missing) timed on this machine's cores on a sample of the
            same workload
  extra     secondary figures: shorter contexts; the paged Llama-3-8B configuration as a whole (32 layers
            resident, decode step and prefill quantisation timed apart, parity against the CPU port); the
            quantiser; the 4-bit index scan over 10 M rows (QPS, HBM GB/s, and the first queries again with
            the upstream C++ core over all rows)

--impl reference times only that CPU arm, on a bounded sample per step, and prints the same line shape.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "turboquant-kv_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

LAYERS, Q_HEADS, KV_HEADS, HEAD_DIM, BATCH = 16, 32, 8, 64, 32
KEY_BITS, VALUE_BITS = 4, 2
BYTES_PER_TOKEN_HEAD = KEY_BITS * HEAD_DIM // 8 + 4 + VALUE_BITS * HEAD_DIM // 8 + 4   # 56
METRIC, UNIT = "decode_attention_tokens_per_s", "tokens/s"
# DRAM traffic of one decode_fused_kernel launch, cited from an ncu capture of a full-size launch of this
# workload (dram__bytes_read.sum 236.61 MB + dram__bytes_write.sum 6.72 MB against 234.88 MB of algorithmic
# bytes); traffic grows in proportion to the tokens, so other sizes are scaled by the ratio.  It is a
# citation of that capture, not a live measurement: counters cannot be read inside the timed run.
NCU_TRAFFIC_RATIO = (236.61 + 6.72) / 234.88
NCU_TRAFFIC_SOURCE = ("cited from profiles/decode_fused_kernel_c4_ctx16384.md (ncu dram__bytes_read.sum + "
                      "dram__bytes_write.sum of one launch), scaled by the bytes of this launch")


def workload_config(ctx: int, world: int) -> dict:
    return {"workload": f"packed-KV decode attention, K{KEY_BITS}/V{VALUE_BITS}, Llama-3.2-1B shape",
            "layers": LAYERS, "q_heads": Q_HEADS, "kv_heads": KV_HEADS, "head_dim": HEAD_DIM,
            "batch": BATCH, "context": ctx, "new_tokens_per_step": 1,
            "parallelism": f"kv-head sharding x{world}" if world > 1 else "single GPU",
            "l2": "working set per step (packed cache of all layers) exceeds the 126 MB L2; no flush needed"}


def measured_peaks() -> dict:
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "source": "measured"}
    except Exception:
        return {"hbm_gbs": 6650.0, "source": "fallback"}


# ------------------------------------------------------------------------------------------------
# clocks
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples nvidia-smi every 200 ms while the timed region runs."""

    FIELDS = ("uuid,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, uuid: str):
        self.uuid, self.rows, self.proc = uuid, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None
        return self

    def _pump(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 8 and (not self.uuid or self.uuid in parts[0] or parts[0] in self.uuid):
                self.rows.append(parts)

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.25)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()

    def summary(self) -> dict:
        mhz, mx, reasons = [], 0.0, set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for r in self.rows:
            try:
                mhz.append(float(r[1]))
                mx = max(mx, float(r[2]))
            except ValueError:
                continue
            for name, val in zip(names, r[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        mhz.sort()
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(mhz)}


# ------------------------------------------------------------------------------------------------
# CPU arm (the reference arm and the cpu_baseline leg)
# ------------------------------------------------------------------------------------------------
def cpu_sample(ctx: int, sample_seqs: int, steps: int, warmup: int, heads: slice = slice(0, KV_HEADS), threads: int = 0,
               min_seconds: float = 0.0):
    """Dequantise-then-attend on the host for `sample_seqs` sequences x 8 KV heads of ONE layer.

    Returns (tokens_per_s extrapolated to the full step, seconds per sample step, cores, description,
    data) -- data holds the sample's inputs/outputs for the parity check of the GPU arm.  `heads` keeps a
    slice of the KV heads (and their query heads) of the same sample: a rank's share under head sharding.
    With `min_seconds` the timed loop goes on past `steps` until that much host time has been spent."""
    import numpy as np

    from oracle import build as obuild

    obuild.build_oracle()
    from oracle import oracle as orc

    cores = threads or os.cpu_count() or 1
    orc.set_num_threads(cores)
    rng = np.random.default_rng(4000)
    n = sample_seqs * KV_HEADS * ctx
    k = rng.standard_normal((n, HEAD_DIM), dtype=np.float32)
    v = rng.standard_normal((n, HEAD_DIM), dtype=np.float32)
    k[:, rng.permutation(HEAD_DIM)[:4]] *= 20.0
    q = rng.standard_normal((sample_seqs, Q_HEADS, HEAD_DIM), dtype=np.float32)
    rk, rv = orc.make_rotation_matrix(HEAD_DIM, 42), orc.make_rotation_matrix(HEAD_DIM, 43)
    bk, ck = orc.lloyd_max_codebook(KEY_BITS, HEAD_DIM)
    bv, cv = orc.lloyd_max_codebook(VALUE_BITS, HEAD_DIM)
    kp, kn = orc.quantize_mse(k, KEY_BITS, rk, bk)
    vp, vn = orc.quantize_mse(v, VALUE_BITS, rv, bv)
    shape = (sample_seqs, KV_HEADS, ctx)
    kp, vp = kp.reshape(*shape, -1), vp.reshape(*shape, -1)
    kn, vn = kn.reshape(shape), vn.reshape(shape)
    lens = np.full(sample_seqs, ctx, np.int32)
    newk = rng.standard_normal((sample_seqs * KV_HEADS, HEAD_DIM), dtype=np.float32)
    if heads != slice(0, KV_HEADS):
        group = Q_HEADS // KV_HEADS
        kp, kn, vp, vn = (np.ascontiguousarray(a[:, heads]) for a in (kp, kn, vp, vn))
        q = np.ascontiguousarray(q[:, heads.start * group:heads.stop * group])

    # the timed arm: the upstream project's own OpenMP kernels (csrc/cpu/quant_cpu.cpp compiled in place into
    # oracle/_ref) when that library travelled here, else the port
    use_ref = orc.ref_cpu_lib() is not None and not os.environ.get("TQB_BENCH_CPU_PORT")
    if use_ref:
        def one_step():
            orc.ref_cpu_quantize(newk, KEY_BITS, rk, bk)
            orc.ref_cpu_quantize(newk, VALUE_BITS, rv, bv)
            return orc.ref_cpu_decode_attention(q, kp, kn, vp, vn, lens, rk, ck, KEY_BITS, rv, cv, VALUE_BITS, threads=cores)
    else:
        def one_step():
            orc.quantize_mse(newk, KEY_BITS, rk, bk)       # the appended token of this layer
            orc.quantize_mse(newk, VALUE_BITS, rv, bv)
            return orc.decode_attention(q, kp, kn, vp, vn, lens, rk, ck, KEY_BITS, rv, cv, VALUE_BITS)

    out = None
    for _ in range(warmup):
        out = one_step()
    t0 = time.perf_counter()
    done = 0
    while done < steps or (time.perf_counter() - t0 < min_seconds and done < 1000):
        out = one_step()
        done += 1
    dt = (time.perf_counter() - t0) / max(done, 1)
    full_step = dt * LAYERS * BATCH / sample_seqs
    desc = (f"{sample_seqs} of {BATCH} sequences x {KV_HEADS} KV heads of 1 of {LAYERS} layers at context {ctx}, "
            f"scaled by {LAYERS * BATCH // sample_seqs}; {done} timed passes of {dt:.3f} s")
    data = dict(q=q, kp=kp, kn=kn, vp=vp, vn=vn, out=out, kind="reference" if use_ref else "port")
    return BATCH / full_step, dt, cores, desc, data


CPU_NOTE = {
    "reference": "the upstream project's own OpenMP kernels (csrc/cpu/quant_cpu.cpp: rotate_and_quantize_cpu, "
                 "attention_scores_packed_cpu, attention_values_packed_cpu), compiled in place into oracle/_ref and "
                 "driven per (sequence, KV head) as the upstream cache does, units spread over the host threads",
    "port": "CPU port of the upstream dequantise-then-attend path (oracle/tq_oracle.c, OpenMP): the library of the "
            "upstream CPU kernels (oracle/_ref/libtq_ref_cpu.so) is not on this machine",
}


def run_reference(args, rank: int, world: int) -> None:
    if rank != 0:
        return
    value, dt, cores, desc, data = cpu_sample(args.ctx, args.cpu_seqs, args.steps, args.warmup)
    kind = data["kind"]
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * BATCH / value,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "config": workload_config(args.ctx, world),
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": kind, "sample": desc,
                             "sample_step_s": dt},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "note": CPU_NOTE[kind]}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------
def build_cache(torch, ctx: int, kvh: int, device, extra_tokens: int):
    """Packed cache of all layers holding `ctx` tokens, filled through the public append()."""
    from turboquant_kv import QuantizedKVCache, TurboQuantConfig

    cfg = TurboQuantConfig(key_bits=KEY_BITS, value_bits=VALUE_BITS, seed=42)
    cache = QuantizedKVCache(cfg, LAYERS, ctx + extra_tokens, kvh, HEAD_DIM, device=str(device), batch_size=BATCH)
    chunk = 2048
    for layer in range(LAYERS):
        gen = torch.Generator(device=device).manual_seed(4000 + layer)
        scale = torch.ones(kvh, HEAD_DIM, device=device)
        for h in range(kvh):
            scale[h, torch.randperm(HEAD_DIM, generator=gen, device=device)[:4]] = 20.0
        for lo in range(0, ctx, chunk):
            n = min(chunk, ctx - lo)
            k = torch.randn(BATCH, kvh, n, HEAD_DIM, generator=gen, device=device) * scale[None, :, None, :]
            v = torch.randn(BATCH, kvh, n, HEAD_DIM, generator=gen, device=device)
            cache.append(layer, k.bfloat16(), v.bfloat16())
    return cache


def run_gpu(args, rank: int, world: int, local_rank: int) -> None:
    import torch
    import torch.distributed as dist

    from turboquant_kv import _native

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU fallback)"
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    if KV_HEADS % world:
        raise SystemExit(f"--gpus must divide {KV_HEADS} KV heads")
    kvh, qh = KV_HEADS // world, Q_HEADS // world
    ctx, K, W = args.ctx, args.steps, args.warmup
    total_steps = 3 * (K + W) + 12

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    cache = build_cache(torch, ctx, kvh, device, total_steps)
    gen = torch.Generator(device=device).manual_seed(77 + rank)
    q_in = torch.randn(LAYERS, BATCH, qh, HEAD_DIM, generator=gen, device=device).bfloat16()
    k_in = torch.randn(LAYERS, BATCH, kvh, 1, HEAD_DIM, generator=gen, device=device).bfloat16()
    v_in = torch.randn(LAYERS, BATCH, kvh, 1, HEAD_DIM, generator=gen, device=device).bfloat16()
    out = torch.empty(LAYERS, BATCH, qh, HEAD_DIM, device=device, dtype=torch.bfloat16)

    def step_eager(events=None, bufs=None):
        """One decode step: per layer, append the new token and attend (one fused launch per layer).
        With `events`, every launch sits between its own event pair."""
        if bufs is not None:
            for layer in range(LAYERS):
                cache.decode_step(layer, bufs[0][layer], bufs[1][layer], bufs[2][layer], out=bufs[3][layer])
            return
        for layer in range(LAYERS):
            if events is None:
                cache.decode_step(layer, q_in[layer], k_in[layer], v_in[layer], out=out[layer])
                continue
            if layer == 0:
                torch.cuda._sleep(20_000_000)      # ~10 ms: the launches below queue up behind it, so no
                                                   # event pair contains a wait for the host
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
            ev[0].record()
            cache.decode_step(layer, q_in[layer], k_in[layer], v_in[layer], out=out[layer])
            ev[1].record()
            events.append(ev)

    for _ in range(2):            # allocations, attribute settings, first-touch effects
        step_eager()
    torch.cuda.synchronize()
    assert cache.decode_status() == 0, "a bounded device-side wait expired"

    # ---- capture one step; replays keep appending because positions live on the device ----
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream(device=device)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        launches_before = _native.launch_count()
        with torch.cuda.graph(graph, stream=side):
            step_eager()
        launches_per_step = _native.launch_count() - launches_before
    torch.cuda.current_stream().wait_stream(side)
    # the capture advanced the host-side lengths once without running anything: undo that
    cache.seq_lens -= 1

    def replay(n):
        for _ in range(n):
            graph.replay()
        cache.seq_lens += n

    uuid = str(torch.cuda.get_device_properties(device).uuid) if hasattr(torch.cuda.get_device_properties(device), "uuid") else ""

    # ---- value: K replays, device timed ----
    replay(W)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(uuid) as clocks:
        e0.record()
        replay(K)
        e1.record()
        barrier()
    ms_step = max_over_ranks(e0.elapsed_time(e1) / K)

    # ---- e2e: pinned host buffers in, attention output back, every step ----
    # Every step copies its q/k/v from pinned host memory and its output back to pinned host memory.  The
    # copies run on their own streams and two sets of device buffers (with a captured step each) alternate,
    # so the upload of step i+1 and the download of step i-1 overlap the kernels of step i, as a serving
    # loop would arrange it; events keep every buffer's upload -> compute -> download order.
    h_q, h_k, h_v = (t.cpu().pin_memory() for t in (q_in, k_in, v_in))
    h_outs = [torch.empty(out.shape, dtype=out.dtype).pin_memory() for _ in range(2)]
    h2d = sum(t.numel() * t.element_size() for t in (h_q, h_k, h_v))
    d2h = h_outs[0].numel() * h_outs[0].element_size()
    bufs = [(q_in, k_in, v_in, out), tuple(torch.empty_like(t) for t in (q_in, k_in, v_in, out))]
    graph_b = torch.cuda.CUDAGraph()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph_b, stream=side):
            step_eager(bufs=bufs[1])
    torch.cuda.current_stream().wait_stream(side)
    cache.seq_lens -= 1
    graphs = [graph, graph_b]
    main_stream = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(device=device), torch.cuda.Stream(device=device)
    ev_in, ev_comp, ev_out = ([torch.cuda.Event() for _ in range(2)] for _ in range(3))
    e2e_count = [0]

    def step_e2e(n):
        for _ in range(n):
            b = e2e_count[0] & 1
            e2e_count[0] += 1
            q_d, k_d, v_d, o_d = bufs[b]
            with torch.cuda.stream(s_in):
                s_in.wait_event(ev_comp[b])         # the step that last read this input set has finished
                q_d.copy_(h_q, non_blocking=True)
                k_d.copy_(h_k, non_blocking=True)
                v_d.copy_(h_v, non_blocking=True)
                ev_in[b].record(s_in)
            main_stream.wait_event(ev_in[b])
            main_stream.wait_event(ev_out[b])       # this output set has been downloaded
            graphs[b].replay()
            ev_comp[b].record(main_stream)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_comp[b])
                h_outs[b].copy_(o_d, non_blocking=True)
                ev_out[b].record(s_out)
        cache.seq_lens += n
        main_stream.wait_stream(s_in)
        main_stream.wait_stream(s_out)

    step_e2e(W)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    step_e2e(K)
    e1.record()
    barrier()
    ms_e2e = max_over_ranks(e0.elapsed_time(e1) / K)

    # ---- roofline pass: the same steps launched eagerly, one event pair per decode_attention call ----
    events = []
    for _ in range(min(W, 3)):
        step_eager()
    barrier()
    for _ in range(K):
        step_eager(events)
    barrier()
    kernel_ms = sum(ev[0].elapsed_time(ev[1]) for ev in events) / len(events)
    assert cache.decode_status() == 0, "a bounded device-side wait expired"
    seq_now = int(cache.seq_lens[0])
    bytes_per_launch = BATCH * kvh * seq_now * BYTES_PER_TOKEN_HEAD
    peaks = measured_peaks()
    achieved = bytes_per_launch / (kernel_ms * 1e-3) / 1e9
    roofline = {"bound": "hbm", "kernel": "decode_fused_kernel", "achieved": achieved, "peak": peaks["hbm_gbs"],
                "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"], "peak_source": peaks["source"],
                "traffic": bytes_per_launch * NCU_TRAFFIC_RATIO, "traffic_source": NCU_TRAFFIC_SOURCE,
                "bytes_per_launch": bytes_per_launch, "ms_per_launch": kernel_ms,
                "note": "ms_per_launch: one decode_step call = one launch of the fused kernel (append, query "
                        "rotation, streaming attention, merge) between an event pair, launched eagerly behind a "
                        "queue of earlier launches"}

    line = {"metric": METRIC, "value": BATCH / (ms_step * 1e-3), "unit": UNIT, "n_gpus": world, "steps": K,
            "warmup": W, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32 accumulate over fp16 centroid tables (bf16 in/out)", "data": "synthetic",
            "config": workload_config(ctx, world), "roofline": roofline,
            "e2e": {"value": BATCH / (ms_e2e * 1e-3), "unit": UNIT, "ms_per_step": ms_e2e,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": launches_per_step * K, "launches_per_step": launches_per_step,
            "clocks": clocks.summary(),
            "hbm_gbs_whole_step": LAYERS * bytes_per_launch / (ms_step * 1e-3) / 1e9}

    if rank == 0 and world == 1 and not args.no_cpu:
        value, dt, cores, desc, data = cpu_sample(ctx, args.cpu_seqs, 1, 1, min_seconds=10.0)
        line["cpu_baseline"] = {"value": value, "unit": UNIT, "cores": cores, "kind": data["kind"], "sample": desc,
                                "sample_step_s": dt, "note": CPU_NOTE[data["kind"]]}
        line["parity"] = parity_check(torch, data, device)
    elif world > 1 and not args.no_cpu:
        # every rank checks ITS head slice (2 sequences x its KV heads x the full context) against the CPU port
        _, _, _, _, data = cpu_sample(ctx, 2, 1, 0, heads=slice(rank * kvh, (rank + 1) * kvh), threads=max(1, (os.cpu_count() or 1) // world))
        mine = parity_check(torch, data, device)
        t = torch.tensor([mine["max_abs"], -mine["cosine"]], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        line["parity"] = {"max_abs": float(t[0].item()), "cosine": -float(t[1].item()), "tolerance": mine["tolerance"],
                          "against": "CPU port on every rank's own head slice (2 sequences x %d KV heads), worst rank" % kvh}
    if not args.no_extra:
        try:
            line["extra"] = extras(torch, dist, args, rank, world, device)
        except Exception as exc:  # secondary figures must never take the headline down
            line["extra"] = {"error": repr(exc)}
    if rank == 0:
        print(json.dumps(line), flush=True)


def parity_check(torch, data, device) -> dict:
    """GPU fused decode on the CPU sample's packed cache vs the CPU port's output."""
    import numpy as np

    from turboquant_kv import QuantizedKVCache, TurboQuantConfig

    s, h, ctx = data["kn"].shape
    cache = QuantizedKVCache(TurboQuantConfig(key_bits=KEY_BITS, value_bits=VALUE_BITS, seed=42), 1, ctx, h, HEAD_DIM,
                             device=str(device), batch_size=s)
    cache.load_packed(0, *(torch.from_numpy(data[k]) for k in ("kp", "kn", "vp", "vn")))
    got = cache.decode_attention(0, torch.from_numpy(data["q"]).to(device)).float().cpu().numpy()
    ref = data["out"]
    cos = float((got * ref).sum() / np.sqrt((got * got).sum() * (ref * ref).sum()))
    against = ("the upstream CPU kernels (csrc/cpu/quant_cpu.cpp)" if data.get("kind") == "reference" else "CPU port, dequantise-then-attend")
    return {"max_abs": float(np.abs(got - ref).max()), "cosine": cos, "tolerance": "1e-2 max-abs, cosine >= 0.9999",
            "against": against + ", same packed cache"}


# ------------------------------------------------------------------------------------------------
# secondary figures
# ------------------------------------------------------------------------------------------------
def extras(torch, dist, args, rank: int, world: int, device) -> dict:
    from turboquant_kv import _native
    from turboquant_kv.distributed import ShardedTurboQuantIndex, shard_rows

    res = {}
    peaks = measured_peaks()
    kvh, qh = KV_HEADS // world, Q_HEADS // world
    K, W = args.steps, args.warmup

    def sync_max(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- shorter contexts of the same decode workload (graph replay, device resident) ----
    sweep = {}
    for ctx in (1024, 4096):
        if ctx >= args.ctx:
            continue
        cache = build_cache(torch, ctx, kvh, device, K + W + 4)
        gen = torch.Generator(device=device).manual_seed(5)
        q = torch.randn(LAYERS, BATCH, qh, HEAD_DIM, generator=gen, device=device).bfloat16()
        kn = torch.randn(LAYERS, BATCH, kvh, 1, HEAD_DIM, generator=gen, device=device).bfloat16()
        o = torch.empty_like(q)

        def step():
            for layer in range(LAYERS):
                cache.decode_step(layer, q[layer], kn[layer], kn[layer], out=o[layer])

        step()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream(device=device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side), torch.cuda.graph(g, stream=side):
            step()
        torch.cuda.current_stream().wait_stream(side)
        for _ in range(W):
            g.replay()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(K):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        ms = sync_max(e0.elapsed_time(e1) / K)
        nbytes = LAYERS * BATCH * kvh * (ctx + 2 + W + K // 2) * BYTES_PER_TOKEN_HEAD
        sweep[str(ctx)] = {"tokens_per_s": BATCH / (ms * 1e-3), "ms_per_step": ms,
                           "hbm_gbs_per_gpu": nbytes / (ms * 1e-3) / 1e9,
                           "hbm_frac": nbytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"]}
        del cache, g
        torch.cuda.empty_cache()
    res["decode_context_sweep"] = sweep

    # ---- paged decode, Llama-3-8B geometry: all 32 layers resident, prefill quantisation timed apart ----
    try:
        res["paged_decode_llama3_8b"] = paged_model(torch, dist, args, rank, world, device, peaks, sync_max)
    except Exception as exc:
        res["paged_decode_llama3_8b"] = {"error": repr(exc)}
    torch.cuda.empty_cache()

    # ---- multi-token requests (prefill chunks) as the vLLM v1 backend runs them: one pass per query token ----
    if world == 1:
        def timed_prefill(fn):
            for _ in range(3):
                fn()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(5):
                fn()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / 5

        try:
            ms, nbytes, status, finite = prefill_per_token(torch, device, 8, 32, 8, 1024, timed_prefill)
            res["prefill_attention_per_token_passes"] = {
                "requests": 8, "new_tokens_per_request": 1024, "head_dim": 128, "kv_heads": 8, "q_heads": 32,
                "ms_per_layer_call": ms, "prefill_tokens_per_s_per_layer": 8 * 1024 / ms * 1e3,
                "record_bytes_read": nbytes, "hbm_gbs": nbytes / ms / 1e6, "status": status, "finite": finite,
                "note": "no prefill kernel in this build: every query token is a sequence of its own for the paged "
                        "decode kernel (65,536 work items of 5 to 27 us of set-up each, the prefix streamed again "
                        "per token); a kernel sharing one stream per request would read 1/512 of these bytes"}
        except Exception as exc:
            res["prefill_attention_per_token_passes"] = {"error": repr(exc)}
        torch.cuda.empty_cache()

    # ---- quantise: MSE 4-bit round trip (65,536 unit vectors, d = 128) and Prod 3-bit estimator ----
    if rank == 0:
        from turboquant_kv import dequantize_mse, dequantize_prod, quantize_mse, quantize_prod
        from turboquant_kv.reference import _make_qjl_matrix, lloyd_max_codebook, make_rotation_matrix

        # the constants are made once (host-side QR / Lloyd-Max), as the cache and index classes do
        rot = make_rotation_matrix(128, 42).to(device)
        cb4 = tuple(t.to(device) for t in lloyd_max_codebook(4, 128))
        cb2 = tuple(t.to(device) for t in lloyd_max_codebook(2, 128))
        S = _make_qjl_matrix(128, 128, 42, device)

        def timed_ms(fn, reps=10):
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(reps):
                fn()
            b.record()
            torch.cuda.synchronize()
            return a.elapsed_time(b) / reps

        g0 = torch.Generator(device=device).manual_seed(0)
        x = torch.randn(65536, 128, generator=g0, device=device)
        x = x / x.norm(dim=-1, keepdim=True)
        ms_q = timed_ms(lambda: quantize_mse(x, 4, rotation=rot, codebook=cb4))
        pk, nm = quantize_mse(x, 4, rotation=rot, codebook=cb4)
        ms_d = timed_ms(lambda: dequantize_mse(pk, nm, 4, 128, rotation=rot, codebook=cb4))
        xl = torch.randn(1 << 22, 128, generator=g0, device=device)             # 2 GB of rows: beyond the L2
        ms_q4m = timed_ms(lambda: quantize_mse(xl, 4, rotation=rot, codebook=cb4), reps=5)
        del xl
        mse = float(((dequantize_mse(pk, nm, 4, 128, rotation=rot, codebook=cb4) - x) ** 2).sum(-1).mean())
        # Prod: rows with per-coordinate variances log-uniform in [0.1, 10], L2-normalised (shared variance vector)
        g1 = torch.Generator(device=device).manual_seed(1)
        sig = torch.exp(torch.empty(128, device=device).uniform_(math.log(0.1), math.log(10.0), generator=g1)).sqrt()
        db = torch.randn(1_000_000, 128, generator=g1, device=device) * sig
        db = db / db.norm(dim=-1, keepdim=True)
        qs = torch.randn(1024, 128, generator=g1, device=device) * sig
        qs = qs / qs.norm(dim=-1, keepdim=True)
        ms_p = timed_ms(lambda: quantize_prod(db, 3, rotation=rot, codebook=cb2, S_matrix=S), reps=3)
        mp, sg, rn, nr = quantize_prod(db[:100_000], 3, rotation=rot, codebook=cb2, S_matrix=S)
        est = qs @ dequantize_prod(mp, sg, rn, nr, 3, 128, rotation=rot, codebook=cb2, S_matrix=S).t()
        exact = qs @ db[:100_000].t()
        slope = float((est * exact).sum() / (exact * exact).sum())
        # Prod-mode search over the packed rows (1 M x d128, 3 bits): the scan kernel's Algorithm-2 branch
        from turboquant_kv import TurboQuantIndex

        pidx = TurboQuantIndex(dim=128, bit_width=3, mode="prod", seed=42, device=device)
        pidx.add(db)
        pq = qs[:64].contiguous()
        pidx.search(pq[:4], 10)
        ms_ps = timed_ms(lambda: pidx.search(pq, 10), reps=3)
        ps, pi = pidx.search(pq, 10)
        exact_top = (pq @ db.t()).topk(10, dim=-1).indices
        recall = float(torch.tensor([len(set(a.tolist()) & set(b.tolist())) for a, b in zip(pi, exact_top)]).float().mean() / 10)
        del pidx
        res["quantize"] = {
            "mse_4bit_d128_vectors_per_s": 65536 / (ms_q * 1e-3), "mse_4bit_quantize_ms": ms_q,
            "mse_4bit_dequantize_ms": ms_d, "mse_4bit_rotation_tflops": 2 * 128 * 128 * 65536 / (ms_q * 1e-3) / 1e12,
            "mse_4bit_hbm_frac": 65536 * (512 + 68) / (ms_q * 1e-3) / 1e9 / peaks["hbm_gbs"],
            "mse_4bit_4m_rows_ms": ms_q4m, "mse_4bit_4m_rows_vectors_per_s": (1 << 22) / (ms_q4m * 1e-3),
            "mse_4bit_4m_rows_hbm_frac": (1 << 22) * (512 + 68) / (ms_q4m * 1e-3) / 1e9 / peaks["hbm_gbs"],
            "mse_4bit_per_vector_squared_error": mse,
            "prod_3bit_d128_vectors_per_s": 1_000_000 / (ms_p * 1e-3),
            "prod_3bit_estimator_bias": float((est - exact).mean()), "prod_3bit_estimator_slope": slope,
            "prod_3bit_search_1m_rows_64_queries_qps": 64 / (ms_ps * 1e-3), "prod_3bit_search_top10_overlap_with_exact_search": recall,
            "note": "rank 0 only; MSE calls of 512 rows and more run the rotation on tcgen05 (bf16 operand splits, "
                    "float32 accumulation in tensor memory, rows fed by TMA bulk copies), with the codes of the float32 "
                    "FMA kernel; Prod mode and short calls run the float32 FMA kernel"}
        del db, x, est, exact
        torch.cuda.empty_cache()

    # ---- 4-bit index scan, 10M x 128 rows sharded by rows, top-10 ----
    n_total, dim, nq, k = args.scan_rows, 128, args.scan_queries, 10
    lo, hi = shard_rows(n_total, world, rank)
    index = ShardedTurboQuantIndex(dim, bit_width=4, seed=42, id_offset=lo, device=device)
    gam = torch.distributions.Gamma(torch.tensor(0.5, device=device), torch.tensor(1.0 / 40.0, device=device))
    # the database is generated in global chunks of 250,000 rows, chunk c from seed 1000 + c, so that
    # every shard count sees the same 10 M rows (a shard takes the part of each chunk that falls in its range)
    chunk = 250_000
    t_add = 0.0
    for c in range(lo // chunk, (hi + chunk - 1) // chunk):
        torch.manual_seed(1000 + c)
        x = gam.sample((min(chunk, n_total - c * chunk), dim)).clamp_(0, 255).round_()
        x = x[max(lo - c * chunk, 0): hi - c * chunk].contiguous()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        index.add(x)
        b.record()
        torch.cuda.synchronize()
        t_add += a.elapsed_time(b)
        del x
    torch.manual_seed(999)
    queries = gam.sample((nq, dim)).clamp_(0, 255).round_()
    rows_local = hi - lo
    row_bytes = 4 * dim // 8 + 4
    index.search(queries[:8], k)                  # warm-up (workspace, attributes)
    torch.cuda.synchronize()
    # (a) one query per pass: the latency-style figure the upstream project publishes
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = max(K, 5)
    e0.record()
    for i in range(reps):
        index.local.search(queries[i:i + 1], k)
    e1.record()
    torch.cuda.synchronize()
    ms1 = sync_max(e0.elapsed_time(e1) / reps)
    # (b) all queries, merged across shards
    if world > 1:
        dist.barrier()
    launches0 = _native.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    sc, ids = index.search(queries, k)
    e1.record()
    torch.cuda.synchronize()
    msq = sync_max(e0.elapsed_time(e1))
    launches = _native.launch_count() - launches0
    # (c) the same through host buffers
    hq = queries.cpu().pin_memory()
    t0 = time.perf_counter()
    sc_h, ids_h = index.search(hq, k)
    torch.cuda.synchronize()
    ms_host = sync_max((time.perf_counter() - t0) * 1e3)
    per_pass = 8 if nq > 4 else 4        # calls with more than four queries take eight per pass (one fp16 column each)
    passes = math.ceil(nq / per_pass)
    scan_parity = None
    if world == 1 and not args.no_cpu and args.scan_parity_queries > 0:
        scan_parity = scan_reference_check(torch, index.local, queries[:args.scan_parity_queries], sc, ids, k)
    res["index_scan"] = {
        "rows": n_total, "rows_per_gpu": rows_local, "dim": dim, "bits": 4, "k": k, "queries": nq,
        "single_query_pass_ms": ms1, "single_query_hbm_gbs_per_gpu": rows_local * row_bytes / (ms1 * 1e-3) / 1e9,
        "single_query_hbm_frac": rows_local * row_bytes / (ms1 * 1e-3) / 1e9 / peaks["hbm_gbs"],
        "single_query_note": "includes query rotation and merge launches and the host-side call overhead",
        "qps": nq / (msq * 1e-3), "qps_e2e_host_buffers": nq / (ms_host * 1e-3),
        "queries_per_pass": per_pass, "passes": passes,
        "batched_hbm_gbs_per_gpu": passes * rows_local * row_bytes / (msq * 1e-3) / 1e9,
        "add_vectors_per_s_per_gpu": rows_local / (t_add * 1e-3), "gpu_launches": launches,
        "ids_checksum": int(ids.sum().item()) if rank == 0 else None,
        "parity_vs_upstream_core": scan_parity if scan_parity is not None else
        "run at 1 GPU only: the merged ids are the same at every shard count (ids_checksum)",
    }
    return res


def scan_reference_check(torch, index, queries, scores, ids, k: int) -> dict:
    """The first queries of the batch again on the host, over ALL rows, with the upstream project's own C++
    core (turboquant::search_packed, compiled in place into oracle/_ref) on the index's exported rows: id
    identity except for tied scores, and the CPU's queries/s on this machine's cores."""
    import numpy as np

    from oracle import oracle as orc

    if orc.ref_lib() is None:
        return {"unavailable": "oracle/_ref/libtq_ref.so is not built on this machine"}
    nq = queries.shape[0]
    packed = index._packed_codes.cpu().numpy()
    norms = index._norms.cpu().numpy()
    rot = orc.make_rotation_matrix(index.dim, 42)
    _, cent = orc.lloyd_max_codebook(index.bit_width, index.dim)
    cores = os.cpu_count() or 1
    orc.set_num_threads(cores)
    t0 = time.perf_counter()
    r_sc, r_ids = orc.ref_search_packed(queries.cpu().numpy(), packed, norms, rot, cent, index.bit_width, k)
    dt = time.perf_counter() - t0
    g_sc, g_ids = scores[:nq].cpu().numpy(), ids[:nq].cpu().numpy()
    same = g_ids == r_ids
    # a differing id is explained by a tie when the two rows carry the same score at that rank
    tie = (~same) & (g_sc == r_sc)
    rel = np.abs(g_sc - r_sc) / np.maximum(np.abs(r_sc), 1e-30)
    return {"queries": nq, "rows": int(packed.shape[0]), "ids_identical": bool(same.all()),
            "id_mismatches": int((~same).sum()), "tie_explained": int(tie.sum()),
            "unexplained": int(((~same) & ~tie).sum()), "scores_bit_equal": bool((g_sc == r_sc).all()),
            "score_max_rel_diff": float(rel.max()), "cpu_reference_qps": nq / dt, "cpu_reference_seconds": dt,
            "cores": cores, "against": "upstream turboquant::search_packed (csrc/core/turboquant_core.cpp) on the exported rows"}


def paged_model(torch, dist, args, rank: int, world: int, device, peaks, sync_max) -> dict:
    """The paged Llama-3-8B configuration as a whole: 32 layers, 32 query / 8 KV heads (sharded over the ranks),
    head_dim 128, K4/V3, 16-token pages scattered over the pool, batch 64, context 32768.

    prefill   all 64 x 32768 tokens of ONE layer are quantised into the pages through append_slots from bf16
              K/V resident in HBM (timed per call with CUDA events); the other layers receive copies of these
              pages, so every layer holds real records
    decode    one step = for each of the 32 layers: append_slots of the new token of every sequence, then
              paged_decode_attention over the whole context (2 launches per layer, eager)
    parity    the first layer's output for two sequences against dequantise-then-attend on the CPU
    """
    import numpy as np

    from turboquant_kv.vllm_plugin import TurboQuantKVCacheConfig, TurboQuantPagedKVCache

    layers, batch, ctx, dim, bs, kv_heads, q_heads = 32, 64, args.paged_ctx, 128, 16, 8, 32
    kvh, qh = kv_heads // world, q_heads // world
    K, W = max(3, min(args.steps, 10)), 3
    per_seq = ctx // bs + (K + W + bs) // bs + 1           # pages of a sequence, with room for the appended tokens
    pages = batch * per_seq
    cfg = TurboQuantKVCacheConfig(key_bits=4, value_bits=3, block_size=bs, num_gpu_blocks=pages, seed=42)
    pool = TurboQuantPagedKVCache(cfg, num_layers=layers, num_heads=kvh, head_dim=dim, dtype=torch.bfloat16, device=str(device))
    gen = torch.Generator(device=device).manual_seed(11)
    tables = torch.randperm(pages, device=device, generator=gen).to(torch.int32).view(batch, per_seq)

    # ---- prefill quantisation of one layer, in calls of 4 sequences (131,072 tokens) ----
    scale = torch.ones(kvh, dim, device=device)
    for h in range(kvh):
        scale[h, torch.randperm(dim, generator=gen, device=device)[:4]] = 20.0
    group, t_q, keep = 4, 0.0, None
    tok = torch.arange(ctx, device=device)
    for b0 in range(0, batch, group):
        k = (torch.randn(group * ctx, kvh, dim, generator=gen, device=device) * scale).bfloat16()
        v = torch.randn(group * ctx, kvh, dim, generator=gen, device=device).bfloat16()
        slots = torch.cat([tables[b].long()[tok // bs] * bs + tok % bs for b in range(b0, b0 + group)])
        if b0 == 0:
            keep = (k[:2 * ctx].float().cpu().numpy(), v[:2 * ctx].float().cpu().numpy())
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        pool.append_slots(0, k, v, slots)
        e1.record()
        torch.cuda.synchronize()
        t_q += e0.elapsed_time(e1)
        del k, v, slots
    t_q = sync_max(t_q)
    vectors = 2 * batch * ctx * kvh
    q_bytes = batch * ctx * kvh * (2 * dim * 2 + (64 + 4) + (48 + 4))
    for layer in range(1, layers):
        pool._pools[layer].copy_(pool._pools[0])

    # ---- decode steps ----
    q = torch.randn(layers, batch, qh, dim, generator=gen, device=device).bfloat16()
    kn = (torch.randn(layers, batch, kvh, dim, generator=gen, device=device) * scale).bfloat16()
    vn = torch.randn(layers, batch, kvh, dim, generator=gen, device=device).bfloat16()
    out = torch.empty_like(q)
    lens = [torch.full((batch,), ctx + i + 1, dtype=torch.int32, device=device) for i in range(K + W + 1)]
    slot = [tables[:, (ctx + i) // bs].long() * bs + (ctx + i) % bs for i in range(K + W + 1)]

    def step(i):
        for layer in range(layers):
            pool.append_slots(layer, kn[layer], vn[layer], slot[i])
            pool.paged_decode_attention(layer, q[layer], tables, lens[i], max_seq_len=ctx + K + W + 1, out=out[layer])

    from turboquant_kv import _native

    step(0)
    torch.cuda.synchronize()
    first = out[0, :2].float().cpu().numpy()
    for i in range(1, W):
        step(i)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    launches0 = _native.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(W, W + K):
        step(i)
    e1.record()
    torch.cuda.synchronize()
    ms = sync_max(e0.elapsed_time(e1) / K)
    launches = (_native.launch_count() - launches0) // K
    status = pool.kv.status()
    d_bytes = layers * batch * kvh * (ctx + W + K // 2) * (64 + 48 + 8)
    res = {
        "geometry": "32 layers, head_dim 128, K4/V3, 16-token pages (scattered), batch 64, context %d, "
                    "%d KV heads x 4 query heads per GPU" % (ctx, kvh),
        "decode_ms_per_step": ms, "decode_tokens_per_s": batch / (ms * 1e-3), "launches_per_step": launches,
        "decode_hbm_gbs_per_gpu": d_bytes / (ms * 1e-3) / 1e9, "decode_hbm_frac": d_bytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
        "packed_kv_bytes_per_gpu": layers * batch * kvh * ctx * 120, "status": status,
        "prefill_quantize_ms_per_layer": t_q, "prefill_quantize_ms_32_layers": 32 * t_q,
        "prefill_quantize_vectors_per_layer": vectors, "prefill_quantize_vectors_per_s": vectors / (t_q * 1e-3),
        "prefill_quantize_hbm_gbs_per_gpu": q_bytes / (t_q * 1e-3) / 1e9,
        "prefill_quantize_hbm_frac": q_bytes / (t_q * 1e-3) / 1e9 / peaks["hbm_gbs"],
        "note": "every layer resident (one layer quantised from bf16 K/V, timed; the others are copies of its pages); "
                "decode launched eagerly, timed over %d steps with CUDA events, max over ranks" % K}
    # ---- parity of the first layer's first step for two sequences (their KV heads on this rank) ----
    if not args.no_cpu:
        from oracle import build as obuild

        obuild.build_oracle()
        from oracle import oracle as orc

        orc.set_num_threads(max(1, (os.cpu_count() or 1) // world))
        rk, rv = orc.make_rotation_matrix(dim, 42), orc.make_rotation_matrix(dim, 43)
        bk, ck = orc.lloyd_max_codebook(4, dim)
        bv, cv = orc.lloyd_max_codebook(3, dim)
        n = ctx + 1
        kk = np.concatenate([keep[0].reshape(2, ctx, kvh, dim), kn[0, :2].float().cpu().numpy()[:, None]], axis=1)
        vv = np.concatenate([keep[1].reshape(2, ctx, kvh, dim), vn[0, :2].float().cpu().numpy()[:, None]], axis=1)
        kp, knm = orc.quantize_mse(np.ascontiguousarray(kk.transpose(0, 2, 1, 3)).reshape(-1, dim), 4, rk, bk)
        vp, vnm = orc.quantize_mse(np.ascontiguousarray(vv.transpose(0, 2, 1, 3)).reshape(-1, dim), 3, rv, bv)
        ref = orc.decode_attention(q[0, :2].float().cpu().numpy(), kp.reshape(2, kvh, n, -1), knm.reshape(2, kvh, n),
                                   vp.reshape(2, kvh, n, -1), vnm.reshape(2, kvh, n), np.full(2, n, np.int32),
                                   rk, ck, 4, rv, cv, 3)
        cos = float((first * ref).sum() / np.sqrt((first * first).sum() * (ref * ref).sum()))
        worst = [float(np.abs(first - ref).max()), -cos]
        if world > 1:
            t = torch.tensor(worst, device=device, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            worst = [float(t[0].item()), float(t[1].item())]
        res["parity"] = {"max_abs": worst[0], "cosine": -worst[1], "tolerance": "1e-2 max-abs, cosine >= 0.9999",
                         "against": "CPU port, dequantise-then-attend over 2 sequences x %d KV heads x %d tokens of "
                                    "layer 0 (worst rank)" % (kvh, n)}
    del pool
    return res


def paged_layer(torch, device, kvh: int, qh: int, ctx: int, timed, contiguous: bool = False):
    """One layer of paged decode attention in the geometry of the paged Llama-3-8B configuration: head_dim
    128, K4/V3, 16-token pages, batch 64, `kvh` KV heads x 4 query heads.  The pool holds random codes
    (timing only) and every sequence's pages are scattered over the pool by a random permutation.
    Returns (ms per call, algorithmic bytes, status word, output finite)."""
    from turboquant_kv.kvstore import PackedKVStore

    batch, dim, bs = 64, 128, 16
    kv = PackedKVStore(dim, 4, 3, 42, "dense_qr", device)
    pages = batch * (ctx // bs)
    gen = torch.Generator(device=device).manual_seed(1)
    pool = torch.randint(0, 256, (pages * kvh, bs // 16, kv.record_bytes), dtype=torch.uint8, device=device,
                         generator=gen)
    norms = pool.view(pages * kvh, -1)[:, -128:].view(torch.float32)      # the 32 norms of every record
    norms.copy_(torch.rand(norms.shape, device=device, generator=gen) * 8 + 4)
    tables = torch.randperm(pages, device=device, generator=gen).to(torch.int32).view(batch, ctx // bs)
    lens = torch.full((batch,), ctx, dtype=torch.int32, device=device)
    q = torch.randn(batch, qh, dim, device=device, generator=gen).bfloat16()
    o = torch.empty_like(q)
    if contiguous:      # the same records read as one contiguous cache (unit = sequence x head, pitch = ctx)
        ms = timed(lambda: kv.decode_attention(pool.view(batch * kvh, ctx // 16, kv.record_bytes), q, kvh, lens, ctx,
                                               pitch=ctx, out=o))
    else:
        ms = timed(lambda: kv.decode_attention(pool, q, kvh, lens, ctx, block_tables=tables, block_size=bs, out=o))
    nbytes = batch * kvh * ctx * (64 + 48 + 8)
    return ms, nbytes, kv.status(), bool(torch.isfinite(o.float()).all())


def prefill_per_token(torch, device, kvh: int, qh: int, reqs: int, tokens: int, timed):
    """Causal attention of `reqs` requests x `tokens` new tokens over their own packed K/V (head_dim 128, K4/V3,
    16-token pages), run the way the vLLM v1 backend runs multi-token requests: every query token is a sequence of
    its own -- its request's block-table row, its causal prefix as the length -- in one launch of the paged decode
    kernel.  Token t of a request streams t + 1 records' worth of tokens, so the launch reads (tokens + 1) / 2
    times what a kernel sharing one stream per request would.  Random codes (timing only).
    Returns (ms per call, record bytes read, status word, output finite)."""
    from turboquant_kv.kvstore import PackedKVStore

    dim, bs = 128, 16
    kv = PackedKVStore(dim, 4, 3, 42, "dense_qr", device)
    pages = reqs * (tokens // bs)
    gen = torch.Generator(device=device).manual_seed(2)
    pool = torch.randint(0, 256, (pages * kvh, bs // 16, kv.record_bytes), dtype=torch.uint8, device=device,
                         generator=gen)
    norms = pool.view(pages * kvh, -1)[:, -128:].view(torch.float32)
    norms.copy_(torch.rand(norms.shape, device=device, generator=gen) * 8 + 4)
    tables = torch.randperm(pages, device=device, generator=gen).to(torch.int32).view(reqs, tokens // bs)
    req = torch.arange(reqs, device=device).repeat_interleave(tokens)
    tok_lens = (torch.arange(tokens, device=device, dtype=torch.int32) + 1).repeat(reqs).contiguous()
    tok_tables = tables[req].contiguous()
    q = torch.randn(reqs * tokens, qh, dim, device=device, generator=gen).bfloat16()
    o = torch.empty_like(q)
    ms = timed(lambda: kv.decode_attention(pool, q, kvh, tok_lens, tokens, block_tables=tok_tables, block_size=bs, out=o))
    nbytes = reqs * kvh * (tokens * (tokens + 1) // 2) * (64 + 48 + 8)
    return ms, nbytes, kv.status(), bool(torch.isfinite(o.float()).all())


def run_case(args) -> None:
    """Single-kernel cases for profilers: a few eager launches of one hot kernel, timed with CUDA events.

    decode    one layer-call = decode_attention over `--layers` layers of the decode workload
    paged     one layer-call of paged decode attention, Llama-3-8B geometry (head_dim 128, K4/V3, 16-token
              pages, batch 64, context `--ctx`), random codes
    prefill   causal attention of `--prefill-reqs` x `--prefill-tokens` new tokens, one pass of the paged decode
              kernel per query token (the multi-token path of the vLLM v1 backend)
    scan      single-query passes of the 4-bit index scan over `--scan-rows` rows
    quantize  quantize_mse of `--rows` float32 vectors of dim 128 at 4 bits
    """
    import torch

    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    peaks = measured_peaks()
    K, W = args.steps, args.warmup
    out = {"case": args.case}

    def timed(fn):
        for _ in range(W):
            fn()
        torch.cuda.synchronize()
        ev = []
        for _ in range(K):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            ev.append((a, b))
        torch.cuda.synchronize()
        return sum(a.elapsed_time(b) for a, b in ev) / len(ev)

    if args.case == "decode":
        global LAYERS
        LAYERS = args.layers
        cache = build_cache(torch, args.ctx, KV_HEADS, device, 8)
        q = torch.randn(BATCH, Q_HEADS, HEAD_DIM, device=device).bfloat16()
        o = torch.empty_like(q)
        ms = timed(lambda: [cache.decode_attention(l, q, out=o) for l in range(LAYERS)]) / LAYERS
        nbytes = BATCH * KV_HEADS * args.ctx * BYTES_PER_TOKEN_HEAD
        out.update(ms_per_layer_call=ms, bytes=nbytes, gbs=nbytes / ms / 1e6, frac=nbytes / ms / 1e6 / peaks["hbm_gbs"],
                   status=cache.decode_status())
    elif args.case == "paged":
        ms, nbytes, status, finite = paged_layer(torch, device, 8, 32, args.ctx, timed, args.contiguous)
        out.update(contiguous=bool(args.contiguous), ms_per_layer_call=ms, bytes=nbytes, gbs=nbytes / ms / 1e6, frac=nbytes / ms / 1e6 / peaks["hbm_gbs"],
                   status=status, finite=finite)
    elif args.case == "prefill":
        ms, nbytes, status, finite = prefill_per_token(torch, device, 8, 32, args.prefill_reqs, args.prefill_tokens, timed)
        out.update(requests=args.prefill_reqs, tokens=args.prefill_tokens, ms_per_layer_call=ms, bytes=nbytes,
                   gbs=nbytes / ms / 1e6, frac=nbytes / ms / 1e6 / peaks["hbm_gbs"], status=status, finite=finite,
                   prefill_tokens_per_s_per_layer=args.prefill_reqs * args.prefill_tokens / ms * 1e3)
    elif args.case == "scan":
        from turboquant_kv import TurboQuantIndex

        idx = TurboQuantIndex(dim=128, bit_width=4, seed=42, device=device)
        gam = torch.distributions.Gamma(torch.tensor(0.5, device=device), torch.tensor(1.0 / 40.0, device=device))
        for c0 in range(0, args.scan_rows, 1_000_000):
            idx.add(gam.sample((min(1_000_000, args.scan_rows - c0), 128)).clamp_(0, 255).round_())
        qs = gam.sample((max(args.queries_per_call, 1), 128)).clamp_(0, 255).round_()
        ms = timed(lambda: idx.search(qs, 10))
        nbytes = args.scan_rows * 68 * math.ceil(qs.shape[0] / (8 if qs.shape[0] > 4 else 4))
        out.update(ms_per_call=ms, queries=qs.shape[0], bytes=nbytes, gbs=nbytes / ms / 1e6,
                   frac=nbytes / ms / 1e6 / peaks["hbm_gbs"])
    elif args.case == "quantize":
        from turboquant_kv import quantize_mse
        from turboquant_kv.reference import lloyd_max_codebook, make_rotation_matrix

        x = torch.randn(args.rows, 128, device=device)
        rot = make_rotation_matrix(128, 42).to(device)
        cb = tuple(t.to(device) for t in lloyd_max_codebook(4, 128))
        ms = timed(lambda: quantize_mse(x, 4, rotation=rot, codebook=cb))
        nbytes = args.rows * (512 + 68)
        out.update(ms_per_call=ms, rows=args.rows, vectors_per_s=args.rows / ms * 1e3, gbs=nbytes / ms / 1e6,
                   tflops=2 * 128 * 128 * args.rows / ms / 1e9)
    print(json.dumps(out), flush=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", default=None, choices=["decode", "paged", "prefill", "scan", "quantize"],
                    help="run one single-kernel case (for profilers) instead of the benchmark")
    ap.add_argument("--layers", type=int, default=LAYERS, help="--case decode: layers to build")
    ap.add_argument("--rows", type=int, default=65536, help="--case quantize: vectors")
    ap.add_argument("--contiguous", action="store_true",
                    help="--case paged: read the same records as a contiguous cache (no block tables)")
    ap.add_argument("--queries-per-call", type=int, default=1, help="--case scan: queries per search call")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--ctx", type=int, default=16384)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--cpu-seqs", type=int, default=8, help="sequences in the CPU sample")
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--no-extra", action="store_true", help="skip the secondary figures")
    ap.add_argument("--scan-rows", type=int, default=10_000_000)
    ap.add_argument("--scan-queries", type=int, default=10_000)
    ap.add_argument("--scan-parity-queries", type=int, default=32,
                    help="queries searched again with the upstream C++ core over all rows (1 GPU only; 0 = skip)")
    ap.add_argument("--paged-ctx", type=int, default=32768, help="context of the paged 32-layer configuration")
    ap.add_argument("--prefill-reqs", type=int, default=8, help="--case prefill: requests")
    ap.add_argument("--prefill-tokens", type=int, default=1024, help="--case prefill: new tokens per request (multiple of 16)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.case:
        run_case(args)
        return
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if world > 1:
        import torch
        import torch.distributed as dist

        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    try:
        run_gpu(args, rank, world, local_rank)
    finally:
        if world > 1:
            import torch.distributed as dist

            if dist.is_initialized():
                dist.destroy_process_group()


if __name__ == "__main__":
    main()
