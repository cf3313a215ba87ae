#!/usr/bin/env python
"""Benchmark of the LRQK per-layer decode step on B200.

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--layers L] [--rho R]

Workload ("cfg2-layer"): the attention layer of a Llama-3-8B-shaped model at 128K context --
batch 1, 32 query / 8 KV heads, head_dim 128, prompt 131072 tokens, r=32, num_active_tokens=2048,
lite_tokens=64, max_iter=(2,2), bf16 -- with `--layers` independent layer states that a decode
"step" (one token) walks through in order, as a model would.  Metric: microseconds per layer per
decode step (lite-ring write + rank-r projection/update + proxy score + top-k + hit/miss + miss
fetch from pinned host memory + exact attention).  Inputs are seeded synthetic tensors of the
config's distributions; nothing is read from disk.

N > 1 (torchrun, one rank per GPU): KV heads are sharded across ranks (strong scaling), each rank
owns its heads' factors, slot tables, resident rows and host store; the attention kernel stores its
output rows into every rank's exchange buffer over NVLink (`--collective nccl`: an NCCL all-gather
instead), once per layer-step.

`--impl reference` times the CPU restatement of the reference's decode step (oracle/) on the host
cores for the same workload; the default arm also times it on a bounded sample (`cpu_baseline`).
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch

WORKLOADS = {
    # name: bsz, q heads, kv heads, head dim, prompt length, r, k, m, max_iter, tol
    "cfg2-layer": dict(bsz=1, hq=32, hkv=8, d=128, seq=131072, r=32, k=2048, m=64, max_iter=(2, 2), tol=1e-2),
    "cfg1-layer": dict(bsz=4, hq=32, hkv=8, d=128, seq=32768, r=32, k=2048, m=64, max_iter=(2, 2), tol=1e-2),
    "cfg3-layer": dict(bsz=8, hq=28, hkv=4, d=128, seq=65536, r=16, k=1024, m=32, max_iter=(1, 1), tol=1e-2),
    "cfg4-layer": dict(bsz=1, hq=40, hkv=8, d=128, seq=262144, r=64, k=4096, m=128, max_iter=(4, 4), tol=1e-2),
    "cfg0": dict(bsz=1, hq=8, hkv=2, d=128, seq=4096, r=16, k=256, m=16, max_iter=(2, 2), tol=1e-2),
}
# DRAM bytes moved per algorithmic byte of the scoring kernel, from the ncu capture summarised under profiles/
# (dram__bytes_read.sum + dram__bytes_write.sum of one launch = 272.8 MB against 268.6 MB algorithmic); the
# kernel's traffic grows in proportion to the rows it scores, so other sizes are scaled by this ratio.
NCU_TRAFFIC_RATIO = {"score_topk": 1.0156}
FALLBACK_HBM_GBS = 6650.0


# ------------------------------------------------------------------------------------------------
# synthetic inputs
# ------------------------------------------------------------------------------------------------
def make_prompt(seed: int, w: dict, hq: int, hkv: int, device, dtype):
    """K = U W + 0.1 E per KV head (U~N(0,1) [S,32], W~N(0,1/32), E~N(0,1)); V, Q ~ N(0,1)."""
    g = torch.Generator(device=device).manual_seed(seed)
    b, s, d = w["bsz"], w["seq"], w["d"]
    U = torch.randn(b, hkv, s, 32, generator=g, device=device)
    W = torch.randn(b, hkv, 32, d, generator=g, device=device) / math.sqrt(32)
    K = (U @ W + 0.1 * torch.randn(b, hkv, s, d, generator=g, device=device)).to(dtype)
    V = torch.randn(b, hkv, s, d, generator=g, device=device).to(dtype)
    Q = torch.randn(b, hq, s, d, generator=g, device=device).to(dtype)
    return Q, K, V


def make_steps(seed: int, n_tokens: int, layers: int, w: dict, hq: int, hkv: int, rho: float, device, dtype):
    """Per token and layer: q [B,Hq,d], k, v [B,Hkv,d].  q follows q_t = rho q_{t-1} + sqrt(1-rho^2) eps
    per layer (rho = 0: independent N(0,1) queries, the BASELINE configs' distribution)."""
    g = torch.Generator(device=device).manual_seed(seed)
    b, d = w["bsz"], w["d"]
    eps = torch.randn(n_tokens, layers, b, hq, d, generator=g, device=device)
    q = torch.empty_like(eps)
    prev = torch.randn(layers, b, hq, d, generator=g, device=device)
    c = math.sqrt(max(0.0, 1.0 - rho * rho))
    for t in range(n_tokens):
        prev = rho * prev + c * eps[t]
        q[t] = prev
    k = torch.randn(n_tokens, layers, b, hkv, d, generator=g, device=device)
    v = torch.randn(n_tokens, layers, b, hkv, d, generator=g, device=device)
    return q.to(dtype), k.to(dtype), v.to(dtype)


# ------------------------------------------------------------------------------------------------
# clocks
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.gpu_index)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        for ln in self.lines:
            p = [x.strip() for x in ln.split(",")]
            if len(p) < 9:
                continue
            try:
                sm.append(float(p[1])); smax.append(float(p[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), p[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------
def measured_hbm_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


def host_link_peak_gbs(device, world: int = 1, rank: int = 0, sync=None):
    """Pinned host -> device copy bandwidth (256 MiB, best of 5) of this rank: with every rank copying at the
    same moment -- the condition of the timed loop, where the exchange keeps the ranks in step and they all
    fetch at once; this is the roofline's peak -- and with the ranks taking turns.  Returns (together, alone)."""
    n = 256 << 20
    h = torch.empty(n, dtype=torch.uint8, pin_memory=True)
    dv = torch.empty(n, dtype=torch.uint8, device=device)

    def once():
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        dv.copy_(h, non_blocking=True)
        e1.record()
        e1.synchronize()
        return n / (e0.elapsed_time(e1) * 1e-3) / 1e9

    once()
    together = 0.0
    for _ in range(5):
        if sync is not None:
            sync()
        together = max(together, once())
    alone = together
    if world > 1 and sync is not None:
        alone = 0.0
        for r in range(world):
            sync()
            if r == rank:
                alone = max(once() for _ in range(3))
        sync()
    return together, alone


def build_layers(w, layers, hq_local, hkv_local, head_offset, device, dtype, seed, n_tokens):
    """One factory per layer, prefilled through the public API (prompt factorisation, host store,
    first selection, lite ring).  Returns the factories and the mean prefill time per layer."""
    from lrqk_b200 import LightAttentionIndicesFactory
    facs, ms = [], []
    groups = w["hq"] // w["hkv"]
    for li in range(layers):
        Q, K, V = make_prompt(seed + 100 * li + head_offset, w, hq_local, hkv_local, device, dtype)
        fac = LightAttentionIndicesFactory(num_lite_tokens=w["m"], attn_topk=w["k"], num_key_value_groups=groups,
                                           r=w["r"], max_iter=w["max_iter"], tol=w["tol"],
                                           capacity=w["seq"] + n_tokens + 2 * w["m"] + 64, scaling_ratio=1.0,
                                           init_aq_ak_method="randn")
        torch.manual_seed(seed + 7 + li)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fac.prefill(Q, K, V)
        len(fac.KVcpu)      # the prompt's copy into the host store runs on a second stream: count it in
        e1.record()
        e1.synchronize()
        ms.append(e0.elapsed_time(e1))
        facs.append(fac)
        del Q, K, V
    torch.cuda.synchronize()
    return facs, statistics.mean(ms)


def stage_bytes(w, hq, hkv, cand, misses, e=2):
    """Algorithmic bytes per layer-step of each kernel (N = B*Hq heads on this rank)."""
    n = w["bsz"] * hq
    k, m, r, d = w["k"], w["m"], w["r"], w["d"]
    return {
        "lite_append": n * 2 * d * e + w["bsz"] * hkv * 2 * d * e,
        "project": n * (k + m) * (d + r) * e + 2 * n * r * d * e,
        "update": 2 * n * r * d * e,          # the right factors written back (its reads of them are re-reads)
        "score_topk": n * cand * r * e + n * k * 4,
        "slot_diff": 3 * n * k * 4 + n * k,
        "miss_gather": misses * 2 * d * e,
        "flash_decode": n * (k + m) * 2 * d * e + 2 * n * d * e,
        # the fused step's last kernel does both: the missed rows over the host link (its bound; the figure
        # here), the rows that stayed resident out of HBM
        "fetch_attend": misses * 2 * d * e,
    }


def run_ours(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    assert torch.cuda.is_available(), "bench.py needs a CUDA device; there is no CPU fallback"
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    from lrqk_b200 import sharding as _sharding
    numa_cpus = _sharding.bind_host_to_gpu_numa(local_rank)   # the host K|V store is allocated after this
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)
    w = WORKLOADS[args.workload]
    dtype = torch.float32 if args.workload == "cfg0" else torch.bfloat16
    if w["hkv"] % world != 0:
        raise SystemExit(f"{w['hkv']} KV heads do not shard over {world} ranks")
    hkv_l, hq_l = w["hkv"] // world, w["hq"] // world
    n_tokens = args.warmup + 3 * args.steps + 8
    layers = args.layers
    sweep_rhos = [r for r in (0.9, 0.99) if not args.no_rho_sweep and abs(r - args.rho) > 1e-9]
    sweep_warm, sweep_probe = 6, 2
    t_setup = time.time()
    facs, prefill_ms = build_layers(w, layers, hq_l, hkv_l, rank * 1000, device, dtype, args.seed, n_tokens)
    q_all, k_all, v_all = make_steps(args.seed + 1 + rank, n_tokens, layers, w, hq_l, hkv_l, args.rho, device, dtype)
    gathered = torch.empty(world, w["bsz"], hq_l, w["d"], dtype=dtype, device=device) if world > 1 else None
    exchange = None
    if world > 1 and args.collective == "push":
        from lrqk_b200 import sharding
        exchange = sharding.HeadExchange(w["bsz"] * hq_l, w["d"], dtype)
    setup_s = time.time() - t_setup

    def layer(fac, q, k, v):
        """One layer-step; with several ranks, every rank ends up with the rows of all heads."""
        if exchange is not None:
            # ONE call: the attention epilogue stores into every rank's buffer, then the bounded wait for all rows
            out = fac.decode_attend_push(q, k, v, exchange)
        else:
            out = fac.decode_attend(q, k, v)
            if world > 1 and args.collective == "nccl":
                dist.all_gather_into_tensor(gathered, out.squeeze(2))
        return out

    def token(t):
        for li, fac in enumerate(facs):
            layer(fac, q_all[t, li], k_all[t, li], v_all[t, li])

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    tcur = 0
    for _ in range(args.warmup):
        token(tcur); tcur += 1
    # ---- device-resident timing ----
    sampler = ClockSampler(local_rank)
    barrier()
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    t_host = time.perf_counter()
    for _ in range(args.steps):
        token(tcur); tcur += 1
    host_issue_us = (time.perf_counter() - t_host) * 1e6 / (args.steps * layers)   # host time to enqueue one layer-step
    e1.record()
    barrier()
    ms_dev = e0.elapsed_time(e1)
    # ---- end to end: pinned host inputs, host-visible outputs, one sync per token ----
    # a token's q | k | v of all layers sit in ONE page-locked buffer and cross the link as one copy
    nq, nk, nv = q_all[0].numel(), k_all[0].numel(), v_all[0].numel()
    in_pin = torch.cat([q_all[tcur:tcur + args.steps].reshape(args.steps, nq), k_all[tcur:tcur + args.steps].reshape(args.steps, nk),
                        v_all[tcur:tcur + args.steps].reshape(args.steps, nv)], dim=1).cpu().pin_memory()
    out_pin = torch.empty(layers, w["bsz"], hq_l, w["d"], dtype=dtype).pin_memory()
    d_in = torch.empty(nq + nk + nv, dtype=dtype, device=device)
    dq, dk, dv = d_in[:nq].view_as(q_all[0]), d_in[nq:nq + nk].view_as(k_all[0]), d_in[nq + nk:].view_as(v_all[0])
    barrier()
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2.record()
    for i in range(args.steps):
        d_in.copy_(in_pin[i], non_blocking=True)
        for li, fac in enumerate(facs):
            out = layer(fac, dq[li], dk[li], dv[li])
            out_pin[li].copy_(out.squeeze(2), non_blocking=True)
        torch.cuda.current_stream().synchronize()
    e3.record()
    barrier()
    ms_e2e = e2.elapsed_time(e3)
    tcur += args.steps
    h2d = d_in.numel() * d_in.element_size()
    d2h = out_pin.numel() * out_pin.element_size()
    # ---- per-kernel timing: the same step issued stage by stage with events in between ----
    # (the last entry is the kernel the fused step runs instead of the two before it: it fetches the same rows
    # again -- the mask still marks them -- and leaves the same state)
    names = ["lite_append", "project", "update", "score_topk", "slot_diff", "miss_gather", "flash_decode", "fetch_attend"]
    floor_names = names[:7]            # the step's floor: each byte once
    LINK_BOUND = ("miss_gather", "fetch_attend")
    evs, miss_total, cand_seen = [], 0, 0
    miss_acc = torch.zeros((), dtype=torch.int64, device=device)
    for _ in range(args.steps):
        for li, fac in enumerate(facs):
            st = fac.state
            fac._reserve()
            q, k, v = q_all[tcur, li], k_all[tcur, li], v_all[tcur, li]
            slot, position, flush_rows, host_row, cand = fac._step_counters()
            cand_seen = cand
            marks = [torch.cuda.Event(enable_timing=True) for _ in range(9)]
            torch.cuda._sleep(400_000)   # ~0.2 ms of GPU idle spin: the host queues the six launches behind it,
            marks[0].record()            # so the event deltas are device time, not host launch time
            st.lite_append(k, v, slot, position, flush_rows, host_row); marks[1].record()
            st.project(q, k, w["max_iter"][1], position); marks[2].record()     # the fused step's first kernel
            st.update(q, k, w["max_iter"][1], w["tol"], position); marks[3].record()   # (inside its scoring kernel)
            st.score_topk(st.q_hat, cand); marks[4].record()
            st.slot_diff(); marks[5].record()
            st.miss_gather(); marks[6].record()
            st.flash_decode(q); marks[7].record()
            st.fetch_attend(q); marks[8].record()
            miss_acc += st.miss_count.sum()
            evs.append(marks)
        tcur += 1
    torch.cuda.synchronize()
    stage_us = {n: statistics.mean(m[i].elapsed_time(m[i + 1]) for m in evs) * 1e3 for i, n in enumerate(names)}
    misses_per_step = float(miss_acc.item()) / len(evs)
    miss_rate = misses_per_step / (w["bsz"] * hq_l * w["k"])

    # ---- the same timed loop at other query localities: q_t = rho q_(t-1) + sqrt(1 - rho^2) eps.  Independent
    # queries (rho = 0) miss nearly every selected row; a model's consecutive queries are correlated ----
    def floor_us(misses):
        b = stage_bytes(w, hq_l, hkv_l, cand_seen, misses, e=2 if dtype == torch.bfloat16 else 4)
        return sum(b[n] / ((link_peak if n in LINK_BOUND else hbm_peak) * 1e9) for n in floor_names) * 1e6

    hbm_peak, peak_kind = measured_hbm_peak()
    link_peak, link_peak_alone = host_link_peak_gbs(device, world, rank, barrier)
    by_rho = {}
    for rho in sweep_rhos:
        n_sw = sweep_warm + args.steps + sweep_probe
        qs_, ks_, vs_ = make_steps(args.seed + 17 + rank, n_sw, layers, w, hq_l, hkv_l, rho, device, dtype)

        def tok(t):
            for li, fac in enumerate(facs):
                layer(fac, qs_[t, li], ks_[t, li], vs_[t, li])

        for t in range(sweep_warm):
            tok(t)
        barrier()
        r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        r0.record()
        for t in range(sweep_warm, sweep_warm + args.steps):
            tok(t)
        r1.record()
        barrier()
        acc = torch.zeros((), dtype=torch.int64, device=device)
        for t in range(sweep_warm + args.steps, n_sw):
            for li, fac in enumerate(facs):
                layer(fac, qs_[t, li], ks_[t, li], vs_[t, li])
                acc += fac.state.miss_count.sum()
        ms_r = torch.tensor([r0.elapsed_time(r1)], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(ms_r, op=dist.ReduceOp.MAX)
        us_r = float(ms_r[0]) * 1e3 / (args.steps * layers)
        miss_r = float(acc.item()) / (sweep_probe * layers)
        fl = floor_us(miss_r)
        by_rho[str(rho)] = {"us_measured": round(us_r, 2), "us_at_roofline": round(fl, 1), "frac": round(fl / us_r, 4),
                            "miss_rate": round(miss_r / (w["bsz"] * hq_l * w["k"]), 4)}
        del qs_, ks_, vs_
    clocks = sampler.stop()

    # ---- self-check, outside every timed region: one more step per layer state, issued stage by stage and
    # fused from the same starting state; every output must be bit-identical and the diff status clear ----
    from lrqk_b200 import selfcheck
    problems = []
    for li, fac in enumerate(facs):
        bad = selfcheck.compare_factory_step(fac, q_all[tcur, li], k_all[tcur, li], v_all[tcur, li])
        if bad:
            problems.append({"rank": rank, "layer": li, "differs": bad})
    tcur += 1
    if exchange is not None:    # the rows the push delivered against a library all-gather of the same outputs
        out = facs[0].decode_attend_push(q_all[tcur, 0], k_all[tcur, 0], v_all[tcur, 0], exchange)
        rows = exchange.rows().clone()
        ref = torch.empty_like(rows)
        dist.all_gather_into_tensor(ref, out.reshape(-1, w["d"]).contiguous())
        torch.cuda.synchronize()
        if not torch.equal(rows, ref):
            problems.append({"rank": rank, "exchange": "pushed rows differ from all_gather_into_tensor"})
        tcur += 1
    if world > 1:
        everyone = [None] * world
        dist.all_gather_object(everyone, problems)
        problems = [p for ps in everyone for p in ps]

    # kernels one fused layer-step enqueues (the library's own count for the last step's arguments, without the
    # ring flush that every m-th step adds)
    st0 = facs[0].state
    st0._step_args.flush_rows = 0
    launches_per_step = int(st0.lib.lrqk_layer_step_launches(C.byref(st0.c), C.byref(st0._step_args)))

    # max over ranks
    ms_dev_own = ms_dev
    vals = torch.tensor([ms_dev, ms_e2e], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(vals, op=dist.ReduceOp.MAX)
    ms_dev, ms_e2e = vals.tolist()
    us_per_layer = ms_dev * 1e3 / (args.steps * layers)
    us_per_layer_e2e = ms_e2e * 1e3 / (args.steps * layers)

    bytes_ = stage_bytes(w, hq_l, hkv_l, cand_seen, misses_per_step, e=2 if dtype == torch.bfloat16 else 4)
    per_kernel = {}
    for n in names:
        gbs = bytes_[n] / (stage_us[n] * 1e-6) / 1e9 if stage_us[n] > 0 else 0.0
        bound = "host_link" if n in LINK_BOUND else "hbm"
        peak = link_peak if n in LINK_BOUND else hbm_peak
        per_kernel[n] = {"us": round(stage_us[n], 2), "bytes": int(bytes_[n]), "bound": bound,
                         "achieved": round(gbs, 1), "peak": round(peak, 1), "unit": "GB/s", "frac": round(gbs / peak, 4),
                         # DRAM traffic of one launch (ncu) where a capture exists; the miss fetch moves its bytes over
                         # the host link, not out of DRAM, so it has none
                         "traffic": (round(bytes_[n] * NCU_TRAFFIC_RATIO[n]) if n in NCU_TRAFFIC_RATIO else None)}
        if n in LINK_BOUND:
            per_kernel[n]["host_link_bytes"] = int(bytes_[n])
        if n == "fetch_attend":
            per_kernel[n]["hbm_bytes"] = int(bytes_["flash_decode"])  # resident rows read + refilled rows written
    dominant = max(names, key=lambda n: stage_us[n])
    roof = dict(per_kernel[dominant])
    roof.update({"kernel": dominant,
                 "peak_source": ("MEASURED_PEAKS.json hbm_gbs" if peak_kind == "measured" else "fallback 6650 GB/s")
                 if dominant not in LINK_BOUND else "pinned host->device cudaMemcpy measured in this run"})
    hbm_kernel = max((n for n in names if n not in LINK_BOUND), key=lambda n: stage_us[n])
    roof_hbm = dict(per_kernel[hbm_kernel]); roof_hbm["kernel"] = hbm_kernel
    roof_hbm["peak_source"] = "MEASURED_PEAKS.json hbm_gbs" if peak_kind == "measured" else "fallback 6650 GB/s"

    # the stages of a step depend on one another, so the step's roofline is the SUM of the stages'
    # algorithmic bytes over their peaks (HBM for all but the miss fetch, the host link for that)
    step_floor_us = sum(bytes_[n] / ((link_peak if n in LINK_BOUND else hbm_peak) * 1e9) for n in floor_names) * 1e6
    roof_step = {"us_at_roofline": round(step_floor_us, 1), "us_measured": round(us_per_layer, 2),
                 "frac": round(step_floor_us / us_per_layer, 4), "miss_rate": round(miss_rate, 4),
                 "note": "sum over the stages (ring, projection, update, scoring, difference, miss fetch, attention) of algorithmic bytes / measured peak"}
    by_rho[str(args.rho)] = {k2: roof_step[k2] for k2 in ("us_measured", "us_at_roofline", "frac", "miss_rate")}
    # every rank's own figures (the value above is the slowest rank's): unequal host links show up here
    mine = {"rank": rank, "us_per_layer_step": round(ms_dev_own * 1e3 / (args.steps * layers), 2),
            "host_link_peak_gbs": round(link_peak, 1), "host_link_peak_alone_gbs": round(link_peak_alone, 1),
            "host_issue_us_per_layer_step": round(host_issue_us, 1),
            "stage_us": {n: round(stage_us[n], 2) for n in names}}
    per_rank = [mine]
    if world > 1:
        per_rank = [None] * world
        dist.all_gather_object(per_rank, mine)
    line = {
        "metric": "decode_us_per_layer_128k" if args.workload == "cfg2-layer" else f"decode_us_per_layer_{args.workload}",
        "value": round(us_per_layer, 2), "unit": "us/layer/step", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms_dev / args.steps, 4), "higher_is_better": False,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16" if dtype == torch.bfloat16 else "f32",
        "data": "synthetic",
        "config": {"workload": args.workload, **{k2: (list(v2) if isinstance(v2, tuple) else v2) for k2, v2 in w.items()},
                   "layers_cycled": layers, "query_rho": args.rho, "sharding": f"kv-heads/{world}",
                   "host_numa": ("process bound to %d CPUs next to the GPU" % len(numa_cpus)) if numa_cpus else "topology not visible, unbound",
                   "exchange": ("none" if world == 1 else
                                "attention epilogue pushes rows to every rank over NVLink (peer stores + arrival words)"
                                if exchange is not None else
                                "nccl all_gather_into_tensor" if args.collective == "nccl" else "skipped (diagnostic run)"),
                   "l2": "inputs larger than L2: each layer's A_K is %.0f MB and %d layer states are cycled"
                         % (w["bsz"] * hq_l * w["seq"] * w["r"] * 2 / 1e6, layers)},
        "tokens_per_s_8b_equiv": round(1e6 / (us_per_layer * 32), 2),
        "miss_rate": round(miss_rate, 4), "setup_s": round(setup_s, 1), "prefill_ms_per_layer": round(prefill_ms, 2),
        "e2e": {"value": round(us_per_layer_e2e, 2), "unit": "us/layer/step", "h2d_bytes_per_step": int(h2d),
                "d2h_bytes_per_step": int(d2h)},
        "host_issue_us_per_layer_step": round(host_issue_us, 1),
        # per layer-step: projection, update, scoring(+diff), miss fetch, attention (+ exchange wait);
        # plus one ring-flush kernel per layer every m steps
        "gpu_launches": int(args.steps * layers * launches_per_step + layers * (args.steps // w["m"])),
        "roofline": roof, "roofline_hbm": roof_hbm, "roofline_step": roof_step,
        "roofline_step_by_rho": dict(sorted(by_rho.items())), "kernels": per_kernel, "per_rank": per_rank,
        "host_link_peak_gbs": round(link_peak, 1), "clocks": clocks,
        "selfcheck": "ok" if not problems else problems,
    }
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline_from_state(facs[0], w, q_all, k_all, v_all, tcur, n_steps=5)
    if exchange is not None:
        exchange.check_status()
        dist.barrier()
        exchange.close()
    for fac in facs:
        fac.close()
    del facs, q_all, k_all, v_all
    torch.cuda.empty_cache()
    # ---- whole model: tokens/s of the Llama-3-8B architecture at this workload's settings (all 32 layers, the
    # 131072-token prompt, 256 greedy tokens), through the patched forward and DynamicLRQKCache on these ranks ----
    if args.workload == "cfg2-layer" and not args.no_model:
        try:
            m = model_run("llama3-8b", args)
            line["model"] = {"metric": m["metric"], "tokens_per_s": m["value"], "ms_per_token": m["ms_per_step"],
                             "host_issue_ms_per_step": m["host_issue_ms_per_step"], "prefill_s": m["prefill_s"],
                             "prefill_tokens_per_s": m["prefill_tokens_per_s"], "decode_tokens": m["steps"],
                             "us_per_layer_step_including_dense": m["us_per_layer_step_including_dense"],
                             "hit_rate_per_step": m["hit_rate_per_step"], "config": m["config"], "clocks": m["clocks"]}
        except Exception as e:   # the per-layer figures above stand on their own
            line["model"] = {"error": f"{type(e).__name__}: {e}"[:300]}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------------------
# CPU legs (the only code here that may touch oracle/)
# ------------------------------------------------------------------------------------------------
def _use_all_host_threads() -> int:
    """The CPU legs run on every core this process may use (torchrun pins OMP_NUM_THREADS to 1)."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    os.environ["OMP_NUM_THREADS"] = str(n)      # read by the C oracle's OpenMP runtime when it is loaded
    torch.set_num_threads(n)
    return n


def _oracle():
    _use_all_host_threads()
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import lrqk_oracle
    return lrqk_oracle


def oracle_layer_from_tensors(orc, w, A_K, B_Q, B_K, Kres, Vres, table, host, host_len, cur_len, lite_indices, lite_len):
    lay = orc.OracleLayer(w["r"], w["k"], w["m"], w["hq"] // w["hkv"], w["max_iter"], (w["tol"], w["tol"]),
                          capacity=A_K.shape[2], faithful=True)
    lay.A_K, lay.a_len = A_K, cur_len
    lay.B_Q, lay.B_K, lay.Kres, lay.Vres = B_Q, B_K, Kres, Vres
    lay.table = table
    lay.host, lay.host_len = host, host_len
    lay.current_len, lay.lite_indices, lay.lite_len = cur_len, list(lite_indices), lite_len
    return lay


def time_oracle_steps(orc, lay, steps_qkv, warmup: int):
    times = []
    for i, (q, k, v) in enumerate(steps_qkv):
        t0 = time.perf_counter()
        lay.decode(q, k, v, want_attention=True)
        dt = time.perf_counter() - t0
        lay.trace.clear()
        if i >= warmup:
            times.append(dt)
    return times


def cpu_baseline_from_state(fac, w, q_all, k_all, v_all, tcur, n_steps):
    """The oracle's decode step (the reference's op sequence on torch CPU, fp32 arithmetic on the
    bf16-stored state) on layer 0's current state, a few steps, on this box's host cores."""
    orc = _oracle()
    st = fac.state
    lay = oracle_layer_from_tensors(
        orc, w, st.A_K.cpu(), st.B_Q.cpu(), st.B_K.cpu(), st.K_res.cpu(), st.V_res.cpu(),
        st.table.cpu().numpy().copy(), st.host.data.clone(), st.host.current_len, fac.current_len,
        fac.lite_indices, fac.lite_len)
    steps = [(q_all[tcur - 1 - i, 0].cpu().unsqueeze(2), k_all[tcur - 1 - i, 0].cpu().unsqueeze(2),
              v_all[tcur - 1 - i, 0].cpu().unsqueeze(2)) for i in range(n_steps + 2)]
    times = time_oracle_steps(orc, lay, steps, warmup=2)
    return {"value": round(statistics.median(times) * 1e6, 1), "unit": "us/layer/step", "cores": torch.get_num_threads(),
            "kind": "port", "sample": f"{len(times)} decode steps of one layer (after 2 warm-up steps), median",
            "host_cpus": os.cpu_count()}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    orc = _oracle()
    w = WORKLOADS[args.workload]
    dtype = torch.float32 if args.workload == "cfg0" else torch.bfloat16
    groups = w["hq"] // w["hkv"]
    # one layer: the oracle's own prompt factorisation and first selection, then the timed steps
    Q, K, V = make_prompt(args.seed, w, w["hq"], w["hkv"], torch.device("cpu"), dtype)
    n_tokens = args.warmup + args.steps
    lay = orc.OracleLayer(w["r"], w["k"], w["m"], groups, w["max_iter"], (w["tol"], w["tol"]),
                          capacity=w["seq"] + n_tokens + 2 * w["m"] + 64, scaling_ratio=1.0, faithful=True)
    torch.manual_seed(args.seed + 7)
    tp = time.perf_counter()
    lay.prefill(Q, K, V)
    prefill_s = time.perf_counter() - tp
    del Q, K, V
    q_all, k_all, v_all = make_steps(args.seed + 1, n_tokens, 1, w, w["hq"], w["hkv"], args.rho, torch.device("cpu"), dtype)
    steps = [(q_all[t, 0].unsqueeze(2), k_all[t, 0].unsqueeze(2), v_all[t, 0].unsqueeze(2)) for t in range(n_tokens)]
    t0 = time.perf_counter()
    times = time_oracle_steps(orc, lay, steps, warmup=args.warmup)
    us = statistics.mean(times) * 1e6
    cores = torch.get_num_threads()
    line = {
        "impl": "reference",
        "metric": "decode_us_per_layer_128k" if args.workload == "cfg2-layer" else f"decode_us_per_layer_{args.workload}",
        "value": round(us, 1), "unit": "us/layer/step", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(us / 1e3, 3), "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16" if dtype == torch.bfloat16 else "f32", "data": "synthetic",
        "config": {"workload": args.workload, **{k2: (list(v2) if isinstance(v2, tuple) else v2) for k2, v2 in w.items()},
                   "layers_cycled": 1, "query_rho": args.rho},
        "cpu_baseline": {"value": round(us, 1), "unit": "us/layer/step", "cores": cores, "kind": "port",
                         "sample": f"{len(times)} decode steps of one layer on the host cores "
                                   f"(torch CPU ops in the reference's order + C row gather), mean"},
        "e2e": {"value": round(us, 1), "unit": "us/layer/step", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "wall_s": round(time.perf_counter() - t0, 1), "prefill_s_one_layer": round(prefill_s, 1),
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# whole-model run (optional): a random-init decoder stack of a named architecture through the
# patched Hugging Face forward -- prompt pass, then greedy decoding through DynamicLRQKCache
# ------------------------------------------------------------------------------------------------
MODELS = {
    # Llama-3-8B architecture, the settings of the 128K configuration
    "llama3-8b": dict(family="llama", vocab_size=128256, hidden_size=4096, intermediate_size=14336, num_hidden_layers=32,
                      num_attention_heads=32, num_key_value_heads=8, head_dim=128, rope_theta=500000.0,
                      r=32, k=2048, m=64, max_iter=(2, 2), batch=1, prompt=131072, decode=256),
    # Qwen2.5-7B architecture (QKV bias), the settings of the batch-8 64K configuration
    "qwen2.5-7b": dict(family="qwen", vocab_size=152064, hidden_size=3584, intermediate_size=18944, num_hidden_layers=28,
                       num_attention_heads=28, num_key_value_heads=4, rope_theta=1e6,
                       r=16, k=1024, m=32, max_iter=(1, 1), batch=8, prompt=65536, decode=128),
    # Qwen2.5-32B architecture, the settings of the 256K configuration (all 64 layers need several GPUs:
    # the rank-r key factors alone are 1.3 GB per layer per 262144 tokens, beside 65 GB of weights)
    "qwen2.5-32b": dict(family="qwen", vocab_size=152064, hidden_size=5120, intermediate_size=27648, num_hidden_layers=64,
                        num_attention_heads=40, num_key_value_heads=8, rope_theta=1e6,
                        r=64, k=4096, m=128, max_iter=(4, 4), batch=1, prompt=262144, decode=64),
}


def run_model(args):
    """`--model NAME`: the whole-model run alone; prints its own JSON line."""
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    assert torch.cuda.is_available(), "bench.py needs a CUDA device; there is no CPU fallback"
    torch.cuda.set_device(local_rank)
    from lrqk_b200 import sharding as _sharding
    _sharding.bind_host_to_gpu_numa(local_rank)                # the host K|V stores are allocated after this
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    line = model_run(args.model, args)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def model_run(model_name: str, args) -> dict:
    """Prompt pass and greedy decode of a random-init decoder stack of the named architecture through the patched
    forward and DynamicLRQKCache, on this process group (already initialised when there are several ranks)."""
    import transformers
    from lrqk_b200 import DynamicLRQKCache, patch_model
    spec = dict(MODELS[model_name])
    family = spec.pop("family")
    r, k, m, max_iter = spec.pop("r"), spec.pop("k"), spec.pop("m"), spec.pop("max_iter")
    prompt = args.prompt or spec.pop("prompt")
    spec.pop("prompt", None)
    n_decode = args.decode or spec.pop("decode")
    spec.pop("decode", None)
    batch = args.batch or spec.pop("batch")
    spec.pop("batch", None)
    if args.model_layers:
        spec["num_hidden_layers"] = args.model_layers
    cfg_cls = transformers.LlamaConfig if family == "llama" else transformers.Qwen2Config
    cfg = cfg_cls(max_position_embeddings=prompt + n_decode + 64, **spec)
    cfg._attn_implementation = "sdpa"
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    dist = None
    if world > 1:
        import torch.distributed as dist
    torch.manual_seed(args.seed)                               # every rank builds the same weights
    t0 = time.time()
    with torch.device("cuda"):
        model = transformers.AutoModelForCausalLM.from_config(cfg, dtype=torch.bfloat16)
    model.eval()
    patch_model(model)
    build_s = time.time() - t0
    groups = cfg.num_attention_heads // cfg.num_key_value_heads
    ids = torch.randint(0, cfg.vocab_size, (batch, prompt), generator=torch.Generator().manual_seed(args.seed)).cuda()
    cache = DynamicLRQKCache(r=r, num_active_tokens=k, lite_tokens=m, max_iter=max_iter, tol=1e-2,
                             max_sequence_length=prompt + n_decode + 2 * m + 64, num_key_value_groups=groups)
    if world > 1:
        cache.shard_heads()            # this rank keeps 1/world of every layer's (batch x KV head) units

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def step(tok):
        tok = model(input_ids=tok, past_key_values=cache, use_cache=True).logits[:, -1].argmax(-1, keepdim=True)
        if world > 1:
            dist.broadcast(tok, 0)     # the ranks compute the same logits; this keeps them on one token regardless
        return tok

    sampler = ClockSampler(local_rank)
    with torch.no_grad():
        barrier()
        t1 = time.time()
        out = model(input_ids=ids, past_key_values=cache, use_cache=True, logits_to_keep=1)
        barrier()
        prefill_s = time.time() - t1
        tok = out.logits[:, -1].argmax(-1, keepdim=True)
        if world > 1:
            dist.broadcast(tok, 0)
        for _ in range(args.warmup):
            tok = step(tok)
        facs = [cache.lwattn[i] for i in range(cfg.num_hidden_layers)]
        watched = [facs[0], facs[len(facs) // 2], facs[-1]]
        miss_log = torch.zeros((n_decode, len(watched)), dtype=torch.float32, device="cuda")
        barrier()
        sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        h0 = time.perf_counter()
        for t in range(n_decode):
            tok = step(tok)
            for j, f in enumerate(watched):                    # refilled slots of three layers, no host sync
                miss_log[t, j] = f.state.miss_count.sum()
        e1.record()
        host_issue_ms = (time.perf_counter() - h0) * 1e3        # host time to ENQUEUE the steps (no sync inside)
        barrier()
        clocks = sampler.stop()
        if cache.sharding is not None and cache.sharding._exchange is not None:
            cache.sharding._exchange.check_status()
    ms = e0.elapsed_time(e1)
    miss = float(torch.stack([f.state.miss_count.float().mean() for f in cache.lwattn.values()]).mean()) / k
    st0 = facs[0].state
    slots = st0.bsz * st0.q_heads * k                          # selected rows per layer-step on this rank
    hit_per_step = (1.0 - miss_log.mean(dim=1) / slots).cpu()
    row_bytes = 2 * st0.head_dim * 2                            # one K|V row, bf16
    fetched = float(miss_log.mean()) * cfg.num_hidden_layers * n_decode * row_bytes
    if world > 1:
        t = torch.tensor([ms, prefill_s], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)               # the slowest rank's device time counts
        ms, prefill_s = float(t[0]), float(t[1])
    line = {
        "metric": "decode_tokens_per_s", "value": round(batch * n_decode / (ms * 1e-3), 2), "unit": "tokens/s",
        "n_gpus": world, "steps": n_decode, "warmup": args.warmup, "ms_per_step": round(ms / n_decode, 3),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"{model_name} architecture, random init, {cfg.num_hidden_layers} layers, batch {batch}, "
                               f"{prompt}-token uniform-random prompt, greedy decode", "r": r, "k": k, "m": m,
                   "max_iter": list(max_iter), "dense_parts": "transformers modules (library GEMMs, SDPA for the prompt pass)"
                   + (", replicated on every rank" if world > 1 else ""),
                   "parallelism": f"(batch x KV head) units over {world} ranks, attention rows pushed over NVLink"
                   if world > 1 else "single GPU"},
        "us_per_layer_step_including_dense": round(ms * 1e3 / (n_decode * cfg.num_hidden_layers), 1),
        "prefill_s": round(prefill_s, 2), "prefill_tokens_per_s": round(batch * prompt / prefill_s, 1),
        "model_build_s": round(build_s, 1), "last_step_miss_rate": round(miss, 4),
        # close to ms_per_step: the host's launch rate bounds the step (dense parts are ~40 eager launches a layer)
        "host_issue_ms_per_step": round(host_issue_ms / n_decode, 3),
        "hit_rate_per_step": {"first": round(float(hit_per_step[0]), 4), "min": round(float(hit_per_step.min()), 4),
                              "mean": round(float(hit_per_step.mean()), 4), "max": round(float(hit_per_step.max()), 4),
                              "of": "layers 0, L/2, L-1 of rank 0"},
        # bytes the miss fetch moved over this rank's host link, spread over the WHOLE decode time (dense
        # parts included): a floor of the link rate while the fetch kernel runs
        "miss_fetch_host_link_gbs_over_whole_step": round(fetched / (ms * 1e-3) / 1e9, 2),
        "clocks": clocks,
    }
    cache.close()
    del model, cache, out
    torch.cuda.empty_cache()
    return line


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg2-layer", choices=sorted(WORKLOADS))
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--rho", type=float, default=0.0)
    ap.add_argument("--seed", type=int, default=2024)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-rho-sweep", action="store_true", help="skip the extra timed loops at rho = 0.9 and 0.99")
    ap.add_argument("--no-model", action="store_true",
                    help="skip the whole-model tokens/s block (Llama-3-8B architecture) of the default line")
    ap.add_argument("--collective", default="push", choices=["push", "nccl", "none"],
                    help="N > 1: how the attention rows of all heads reach every rank")
    ap.add_argument("--model", default=None, choices=sorted(MODELS),
                    help="run a whole random-init decoder stack instead of the per-layer workload")
    ap.add_argument("--prompt", type=int, default=0, help="--model: prompt length (default: the configuration's)")
    ap.add_argument("--decode", type=int, default=0, help="--model: tokens to decode (default: the configuration's)")
    ap.add_argument("--batch", type=int, default=0, help="--model: sequences (default: the configuration's)")
    ap.add_argument("--model-layers", type=int, default=0, help="--model: fewer decoder layers, for a quick look")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.model is not None:
        return run_model(args)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
