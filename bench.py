#!/usr/bin/env python
"""Benchmark of the Mamba2 SSD forward hot path (chunk cumsum -> per-chunk state ->
inter-chunk state passing) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

One step = one pass of the path over one batch of synthetic input at the Mamba2-2.7B layer
shape (batch 8, seqlen 4096, 80 heads x 64, 1 group, dstate 128, chunk 256, bf16 x/B, fp32
dt / dA_cumsum / final state, bf16 passed states): `_state_path_fwd`, which returns what the
reference's pair of calls `_chunk_cumsum_fwd` + `_fused_chunk_state_state_passing_fwd_concurrent`
returns (bit for bit) from one kernel launch.  The pair of calls is timed beside it ("two_calls").
With N GPUs every rank holds one such shard of heads (heads shard with no communication),
so the job is N x the single-GPU workload: weak scaling.

Prints ONE JSON line (rank 0):
  value     tokens/s over all ranks, inputs resident in HBM, CUDA-event timed, max over ranks
  e2e       the same calls fed from pinned HOST buffers, host->device and device->host copies of
            every step inside the timed region (copies and compute of successive steps overlap
            on three streams)
  roofline  the state kernel (chunk cumsum inside): algorithmic bytes per launch / its mean
            CUDA-event time, against the measured HBM copy bandwidth of this pool (MEASURED_PEAKS.json)
  cpu_baseline  the same chunked math in torch on the host cores, on a bounded sample

Extras on the same line (key "extra", measured after the headline, outside its timed region):
  seq1m        ONE 1 048 576-token sequence sharded along the sequence over the N ranks (strong
               scaling; chunk cumsum + local scan + one NCCL all-gather of slice summaries +
               cross-rank fix-up), with the same step on the whole sequence on one GPU measured in
               the same run, the speed-up, the per-phase split and the clocks
  cfg2_strong  the headline shape with its 80 heads split over the N ranks (80 / N heads each)
  seqpar_check a 32 768-token sequence through the sequence-parallel path over the real process
               group, every rank's slice compared with a single-GPU run of the whole sequence

`--impl reference` times that CPU implementation (the oracle's restatement of the
reference's algorithm; the reference itself is Triton and has no CPU build) on all host
threads and prints the same line shape with "impl": "reference".
"""
import argparse
import json
import os
import statistics
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOAD = dict(name="mamba2-2.7b-layer", batch=8, seqlen=4096, nheads=80, headdim=64, ngroups=1, dstate=128,
                chunk_size=256)
FALLBACK_HBM_GBS = 6650.0
# DRAM bytes the state kernel moved in one ncu capture of a smaller batch (written by
# `bench.py --summarise-ncu`, which names the capture command); traffic grows with the token count
TRAFFIC_FILE = os.path.join(ROOT, "profiles", "fused_state_kernel_traffic.json")


def measured_traffic(tokens):
    """(bytes per launch scaled to `tokens`, description) from the committed ncu summary, or (None, why)."""
    try:
        with open(TRAFFIC_FILE) as f:
            t = json.load(f)
        scale = tokens / float(t["tokens"])
        rd, wr = t["dram_bytes_read"] * scale, t["dram_bytes_write"] * scale
        return rd + wr, {"read": rd, "write": wr, "captured_tokens": t["tokens"], "kernel": t.get("kernel"),
                         "note": "ncu dram__bytes_read.sum / dram__bytes_write.sum of one launch, scaled by tokens; "
                                 "writes still dirty in L2 when the launch ends are not in the write figure"}
    except Exception as e:
        return None, {"note": f"no ncu summary: {e!r}"}


def algorithmic_bytes(w, in_bytes=2, out_bytes=2, with_cumsum=True):
    """x + B + dt/dA traffic + passed states + final state; the fp32 per-chunk states are
    what fusion removes and are not counted."""
    b, l, h, p, g, n, L = (w[k] for k in ("batch", "seqlen", "nheads", "headdim", "ngroups", "dstate", "chunk_size"))
    c = (l + L - 1) // L
    x = b * l * h * p * in_bytes
    B = b * l * g * n * in_bytes
    dtda = 2 * b * h * c * L * 4
    raw_dt = b * l * h * 4
    out = b * c * h * p * n * out_bytes
    fin = b * h * p * n * 4
    fused_only = x + B + dtda + out + fin          # reads dt_out and dA_cumsum
    whole_path = x + B + raw_dt + dtda + out + fin  # reads raw dt, writes dt_out and dA_cumsum (fused re-read not counted)
    return whole_path if with_cumsum else fused_only


_UNIT = {"byte": 1.0, "Kbyte": 1e3, "Mbyte": 1e6, "Gbyte": 1e9, "ns": 1e-3, "us": 1.0, "ms": 1e3, "s": 1e6,
         "usecond": 1.0, "nsecond": 1e-3, "msecond": 1e3, "second": 1e6}


def summarise_ncu(csv_path, tokens, command):
    """Reads `ncu -i <report> --page raw --csv` output, takes the state kernel's launches and writes
    their mean DRAM read / write bytes and duration to TRAFFIC_FILE (which the roofline reads)."""
    import csv
    with open(csv_path, newline="") as f:
        rows = [r for r in csv.reader(f) if r]
    hdr, units, data = rows[0], rows[1], rows[2:]
    col = {h: i for i, h in enumerate(hdr)}

    def get(r, name):
        return float(r[col[name]].replace(",", "")) * _UNIT[units[col[name]]]

    picked = [r for r in data if "fused_state_kernel" in r[col["Kernel Name"]]]
    if not picked:
        raise SystemExit("no fused_state_kernel launch in " + csv_path)
    out = {"kernel": picked[0][col["Kernel Name"]], "launches": len(picked), "tokens": tokens,
           "dram_bytes_read": statistics.mean(get(r, "dram__bytes_read.sum") for r in picked),
           "dram_bytes_write": statistics.mean(get(r, "dram__bytes_write.sum") for r in picked),
           "duration_us_under_ncu": statistics.mean(get(r, "gpu__time_duration.sum") for r in picked),
           "command": command}
    with open(TRAFFIC_FILE, "w") as f:
        json.dump(out, f, indent=1)
        f.write("\n")
    print(json.dumps(out))


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler(threading.Thread):
    """Polls NVML for SM clock and throttle reasons of one GPU while a region runs."""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index = index
        self.samples = []
        self.reasons = set()
        self.max_mhz = None
        self._stop_evt = threading.Event()
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.ok = False

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4): "sw_power_cap",
            getattr(nv, "nvmlClocksThrottleReasonHwPowerBrakeSlowdown", 0x80): "hw_power_brake",
        }
        while not self._stop_evt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if bit and mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.002)

    def stop(self):
        self._stop_evt.set()
        self.join(timeout=2)
        med = statistics.median(self.samples) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


def physical_gpu_index(local):
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local])
        except Exception:
            return local
    return local


def cpu_hot_path(sample_batch, threads, reps):
    """The oracle's cumsum + chunk state + state passing on `threads` host threads.
    Returns (tokens/s, seconds per pass)."""
    from oracle import ssd_oracle as O
    torch.set_num_threads(threads)
    w = dict(WORKLOAD, batch=sample_batch)
    inp = O.make_inputs(w["batch"], w["seqlen"], w["nheads"], w["headdim"], w["ngroups"], w["dstate"],
                        dtype=torch.bfloat16, seed=0)
    times = []
    budget_s = 15.0
    while True:
        t0 = time.perf_counter()
        O.hot_path_fwd(inp["x"], inp["dt"], inp["A"], inp["B"], w["chunk_size"], dt_bias=inp["dt_bias"],
                       dt_softplus=True, out_dtype=torch.bfloat16)
        times.append(time.perf_counter() - t0)
        # first pass warms the allocator; then `reps` timed passes, cut short at ~15 s of work
        if len(times) > reps or (len(times) >= 3 and sum(times) > budget_s):
            break
    t = statistics.median(times[1:])
    return w["batch"] * w["seqlen"] / t, t, len(times) - 1


def run_reference_arm(args, rank, world):
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    sample_batch = WORKLOAD["batch"]
    tok_s, t, n = cpu_hot_path(sample_batch, threads, max(2, min(args.steps, 20)))
    line = {
        "impl": "reference", "metric": "ssd_state_path_tokens_per_s", "value": tok_s, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": t * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": dict(workload=WORKLOAD["name"], **{k: v for k, v in WORKLOAD.items() if k != "name"},
                       parallelism="host threads"),
        "cpu_baseline": {"value": tok_s, "unit": "tokens/s", "cores": threads, "kind": "port",
                         "sample": f"the whole workload per step, {n} timed passes ({t:.2f} s each, median); "
                                   f"torch chunked SSD math, bf16 inputs"},
        "e2e": {"value": tok_s, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def reference_triton_unfused(tree, w, dev):
    """The reference's own Triton kernels on this GPU, the five UNFUSED ones (cumsum, chunk state,
    state passing, chunk bmm, chunk scan; none of them spin-waits), imported from the reference tree at
    `tree`, on the same seeded inputs, each timed by CUDA events (median of 20 after 5 warm-ups, which
    also cover Triton's autotuning), with this library's kernels beside them and the fraction of
    bit-equal outputs.  Returns a dict; {"unavailable": why} if Triton or the tree is missing."""
    try:
        import triton  # noqa: F401
    except Exception as e:
        return {"unavailable": f"triton is not importable: {e!r}"}
    if not os.path.isdir(os.path.join(tree, "kernels")):
        return {"unavailable": f"no kernels/ package under {tree}"}
    sys.path.insert(0, os.path.abspath(tree))
    try:
        import kernels.ssd_bmm as r_bmm
        import kernels.ssd_chunk_scan as r_scan
        import kernels.ssd_chunk_state as r_cs
        import kernels.ssd_state_passing as r_sp
    except Exception as e:
        return {"unavailable": f"the reference's kernels do not import: {e!r}"}
    finally:
        sys.path.pop(0)
    import triton
    from mamba_fused_minimal_b200.kernels.fused_concurrent import _fused_chunk_state_state_passing_fwd_concurrent as fused
    from mamba_fused_minimal_b200.kernels.rand_data import generate_benchmark_data
    from mamba_fused_minimal_b200.kernels.ssd_bmm import _bmm_chunk_fwd as bmm
    from mamba_fused_minimal_b200.kernels.ssd_chunk_scan import _chunk_scan_fwd as scan
    from mamba_fused_minimal_b200.kernels.ssd_chunk_state import _chunk_cumsum_fwd as cumsum, _chunk_state_fwd as cstate
    from mamba_fused_minimal_b200.kernels.ssd_state_passing import _state_passing_fwd as spass
    from mamba_fused_minimal_b200.kernels.state_path import _state_path_fwd as state_path
    b, l, h, p, g, n, L = (w[k] for k in ("batch", "seqlen", "nheads", "headdim", "ngroups", "dstate", "chunk_size"))
    d = generate_benchmark_data(b, l, h, p, g, n, dtype=torch.bfloat16, device=dev, seed=0)
    x, B, C, dt, A, bias, D = d["x"], d["B"], d["C"], d["dt"], d["A"], d["dt_bias"], d["D"].to(torch.bfloat16)

    def med(fn, n_it=20, warm=5):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n_it)]
        for e0, e1 in ev:
            e0.record()
            fn()
            e1.record()
        torch.cuda.synchronize()
        return statistics.median(e0.elapsed_time(e1) for e0, e1 in ev)

    def same(a, r):
        return float((a == r).float().mean().item())

    res = {"triton": triton.__version__, "shape": {k: v for k, v in w.items() if k != "name"},
           "timing": "CUDA events, median of 20 after 5 warm-ups; inputs (365 MB) exceed L2", "ms": {}, "parity": {}}
    ms = res["ms"]
    # cumsum
    ms["ref_chunk_cumsum"] = med(lambda: r_cs._chunk_cumsum_fwd(dt, A, L, dt_bias=bias, dt_softplus=True))
    ms["b200_chunk_cumsum"] = med(lambda: cumsum(dt, A, L, dt_bias=bias, dt_softplus=True))
    r_dA, r_dt = r_cs._chunk_cumsum_fwd(dt, A, L, dt_bias=bias, dt_softplus=True)
    m_dA, m_dt = cumsum(dt, A, L, dt_bias=bias, dt_softplus=True)
    res["parity"]["dA_cumsum_max_abs_diff_over_max"] = float(((m_dA - r_dA).abs().max() / r_dA.abs().max()).item())
    # the state kernels on the REFERENCE's dt / dA_cumsum, so that they see identical inputs
    ms["ref_chunk_state"] = med(lambda: r_cs._chunk_state_fwd(B, x, r_dt, r_dA, states_in_fp32=True))
    r_st = r_cs._chunk_state_fwd(B, x, r_dt, r_dA, states_in_fp32=True)
    ms["ref_state_passing"] = med(lambda: r_sp._state_passing_fwd(r_st.flatten(-2), r_dA[:, :, :, -1], out_dtype=torch.bfloat16))
    r_out, r_fin = r_sp._state_passing_fwd(r_st.flatten(-2), r_dA[:, :, :, -1], out_dtype=torch.bfloat16)
    ms["b200_chunk_state"] = med(lambda: cstate(B, x, r_dt, r_dA))
    m_st = cstate(B, x, r_dt, r_dA)
    ms["b200_state_passing"] = med(lambda: spass(m_st.flatten(-2), r_dA[:, :, :, -1], out_dtype=torch.bfloat16))
    ms["b200_fused_state"] = med(lambda: fused(B, x, r_dt, r_dA, torch.bfloat16))
    ms["b200_state_path_one_call"] = med(lambda: state_path(dt, A, B, x, L, torch.bfloat16, dt_bias=bias, dt_softplus=True))
    m_out, m_fin = fused(B, x, r_dt, r_dA, torch.bfloat16)
    res["parity"]["chunk_states_max_abs_diff_over_max"] = float(((m_st - r_st).abs().max() / r_st.abs().max()).item())
    res["parity"]["passed_states_bit_equal_fraction"] = same(m_out, r_out.view_as(m_out))
    res["parity"]["final_states_bit_equal_fraction"] = same(m_fin, r_fin.view_as(m_fin))
    res["parity"]["final_states_max_abs_diff_over_max"] = float(((m_fin - r_fin.view_as(m_fin)).abs().max() / r_fin.abs().max()).item())
    del r_st, m_st
    # chunk bmm and chunk scan
    ms["ref_bmm_chunk"] = med(lambda: r_bmm._bmm_chunk_fwd(C, B, L, output_dtype=torch.float32))
    ms["b200_bmm_chunk"] = med(lambda: bmm(C, B, L, output_dtype=torch.float32))
    r_cb = r_bmm._bmm_chunk_fwd(C, B, L, output_dtype=torch.float32)
    res["parity"]["cb_bit_equal_fraction"] = same(bmm(C, B, L, output_dtype=torch.float32), r_cb)
    passed = r_out.view_as(m_out)
    ms["ref_chunk_scan"] = med(lambda: r_scan._chunk_scan_fwd(r_cb, x, r_dt, r_dA, C, passed, D=D))
    ms["b200_chunk_scan"] = med(lambda: scan(r_cb, x, r_dt, r_dA, C, passed, D=D))
    r_y, _ = r_scan._chunk_scan_fwd(r_cb, x, r_dt, r_dA, C, passed, D=D)
    m_y, _ = scan(r_cb, x, r_dt, r_dA, C, passed, D=D)
    res["parity"]["out_bit_equal_fraction"] = same(m_y, r_y)
    res["parity"]["out_max_abs_diff_over_max"] = float(((m_y.float() - r_y.float()).abs().max() / r_y.float().abs().max()).item())
    ms["ref_state_path_unfused_total"] = ms["ref_chunk_cumsum"] + ms["ref_chunk_state"] + ms["ref_state_passing"]
    ms["ref_forward_unfused_total"] = ms["ref_state_path_unfused_total"] + ms["ref_bmm_chunk"] + ms["ref_chunk_scan"]
    ms["b200_forward_total"] = ms["b200_state_path_one_call"] + ms["b200_bmm_chunk"] + ms["b200_chunk_scan"]
    res["recorded_earlier"] = {"ref_fused_concurrent_ms": 2.61, "ref_fused_globalbar_ms": 1.89,
                               "note": "the reference's two fused kernels spin without a limit and are not re-run here; "
                                       "these are the figures of a single earlier run on a B200 of this pool"}
    return res


SEQ1M = dict(name="seq-1m", batch=1, seqlen=1048576, nheads=80, headdim=64, ngroups=1, dstate=128, chunk_size=256)


def _sync_barrier(dist):
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()


def _timed_steps(step, K, warmup, dist, dev):
    """K steps bracketed by barrier + synchronize, CUDA events, max over ranks -> ms per step."""
    for _ in range(warmup):
        step()
    _sync_barrier(dist)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(K):
        step()
    e1.record()
    _sync_barrier(dist)
    t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item()) / K


def seq_sharded_case(w, K, warmup, rank, world, dist, dev, sampler_index=None):
    """One long sequence sharded along the sequence over the ranks.  Returns a dict (rank 0: filled)."""
    from mamba_fused_minimal_b200 import parallel as P
    from mamba_fused_minimal_b200._ext import C as _C
    from mamba_fused_minimal_b200.kernels._fused import _fused_chunk_state_state_passing_fwd as fused
    from mamba_fused_minimal_b200.kernels.rand_data import generate_benchmark_data
    from mamba_fused_minimal_b200.kernels.ssd_chunk_state import _chunk_cumsum_fwd as cumsum
    L = w["chunk_size"]
    s0, s1 = P.shard_sequence(w["seqlen"], L, world, rank)
    d = generate_benchmark_data(1, s1 - s0, w["nheads"], w["headdim"], w["ngroups"], w["dstate"],
                                dtype=torch.bfloat16, device=dev, seed=100 + rank)
    x, B, dt, A, bias = d["x"], d["B"], d["dt"], d["A"], d["dt_bias"]

    from mamba_fused_minimal_b200.kernels.state_path import _state_path_fwd as state_path

    def step():
        if dist is None:
            return state_path(dt, A, B, x, L, torch.bfloat16, dt_bias=bias, dt_softplus=True)
        return P.seqpar_state_path_fwd(dt, A, B, x, L, torch.bfloat16, dt_bias=bias, dt_softplus=True)

    sampler = ClockSampler(sampler_index) if sampler_index is not None else None
    if sampler is not None:
        sampler.start()
    ms = _timed_steps(step, K, warmup, dist, dev)
    clocks = sampler.stop() if sampler is not None else None

    # per-phase split on a few extra steps (events between the phases; not part of `ms`)
    phases = None
    if dist is not None:
        names = ["state_kernel_and_segment_fixup", "logP_sum", "all_gather", "cross_rank_fixup"]
        Kp = 5
        acc = [0.0] * len(names)
        for _ in range(Kp):
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(len(names) + 1)]
            buf, Z, logP = P.summary_buffer(1, w["nheads"], w["headdim"], w["dstate"], dev)
            ev[0].record()
            dA, dto, out, _ = state_path(dt, A, B, x, L, torch.bfloat16, dt_bias=bias, dt_softplus=True, final_states=Z)
            ev[1].record()
            dA_last = dA[:, :, :, -1]
            torch.sum(dA_last, dim=-1, out=logP)
            ev[2].record()
            Z_all, logP_all = P.exchange_summaries(buf, (1, w["nheads"], w["headdim"], w["dstate"]))
            ev[3].record()
            if rank > 0:
                _C.seqpar_fixup(Z_all, logP_all, rank, dA_last, out, Z)
            ev[4].record()
            _sync_barrier(dist)
            for i in range(len(names)):
                acc[i] += ev[i].elapsed_time(ev[i + 1]) / Kp
        t = torch.tensor(acc, device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        phases = {n: round(v, 4) for n, v in zip(names, t.tolist())}
        phases["note"] = "ms, max over ranks per phase, events between the phases (5 extra steps)"
    _C.check_status(x)
    del d, x, B, dt
    torch.cuda.empty_cache()
    peak, peak_kind = measured_peak()
    path_bytes = algorithmic_bytes(w, with_cumsum=True)
    gbs = path_bytes / (ms * 1e-3) / 1e9
    return {"workload": w["name"], "seqlen": w["seqlen"], "nheads": w["nheads"], "world": world, "scaling": "strong",
            "ms_per_step": ms, "tokens_per_s": w["seqlen"] / (ms * 1e-3), "steps": K,
            "path_bytes_per_step": path_bytes, "achieved_gbs": gbs, "frac_of_world_x_peak": gbs / (peak * world),
            "peak_kind": peak_kind, "phases": phases, "clocks": clocks}


def head_sharded_case(w, K, warmup, rank, world, dist, dev, sampler_index=None):
    """The headline shape with its heads split over the ranks (strong scaling, no collective on the
    data path: every kernel is independent per head given the group's B)."""
    from mamba_fused_minimal_b200 import parallel as P
    from mamba_fused_minimal_b200.kernels.fused_concurrent import _fused_chunk_state_state_passing_fwd_concurrent as fused
    from mamba_fused_minimal_b200.kernels.rand_data import generate_benchmark_data
    from mamba_fused_minimal_b200.kernels.ssd_chunk_state import _chunk_cumsum_fwd as cumsum
    (h0, h1), (g0, g1) = P.shard_heads(w["nheads"], w["ngroups"], world, rank)
    L = w["chunk_size"]
    d = generate_benchmark_data(w["batch"], w["seqlen"], h1 - h0, w["headdim"], g1 - g0, w["dstate"],
                                dtype=torch.bfloat16, device=dev, seed=200 + rank)
    x, B, dt, A, bias = d["x"], d["B"], d["dt"], d["A"], d["dt_bias"]

    from mamba_fused_minimal_b200.kernels.state_path import _state_path_fwd as state_path

    def step():
        return state_path(dt, A, B, x, L, torch.bfloat16, dt_bias=bias, dt_softplus=True)

    sampler = ClockSampler(sampler_index) if sampler_index is not None else None
    if sampler is not None:
        sampler.start()
    ms = _timed_steps(step, K, warmup, dist, dev)
    clocks = sampler.stop() if sampler is not None else None
    peak, peak_kind = measured_peak()
    # every rank reads the whole B of its group(s): count it once per rank that holds it
    wr = dict(w, nheads=h1 - h0, ngroups=g1 - g0)
    per_rank = algorithmic_bytes(wr, with_cumsum=True)
    gbs = per_rank * world / (ms * 1e-3) / 1e9
    return {"workload": w["name"], "world": world, "scaling": "strong", "heads_per_rank": h1 - h0,
            "ms_per_step": ms, "tokens_per_s": w["batch"] * w["seqlen"] / (ms * 1e-3), "steps": K,
            "achieved_gbs": gbs, "frac_of_world_x_peak": gbs / (peak * world), "peak_kind": peak_kind,
            "clocks": clocks}


def seqpar_check(rank, world, dist, dev):
    """The sequence-parallel path over the real process group against a single-GPU run of the whole
    sequence on every rank (same seeded inputs everywhere).  Errors as max|a-b| / max|b|."""
    from mamba_fused_minimal_b200 import parallel as P
    from mamba_fused_minimal_b200.kernels.fused_concurrent import _fused_chunk_state_state_passing_fwd_concurrent as fused
    from mamba_fused_minimal_b200.kernels.rand_data import generate_benchmark_data
    from mamba_fused_minimal_b200.kernels.ssd_chunk_state import _chunk_cumsum_fwd as cumsum
    b, l, h, L = 1, 32768, 8, 256
    d = generate_benchmark_data(b, l, h, 64, 1, 128, dtype=torch.bfloat16, device=dev, seed=77)
    # decays slow enough for a carried state to reach well into the next rank's slice
    A = d["A"] * 0.002
    dA_f, dt_f = cumsum(d["dt"], A, L, dt_bias=d["dt_bias"], dt_softplus=True)
    out_f, fin_f = fused(d["B"], d["x"], dt_f, dA_f, torch.bfloat16)
    s0, s1 = P.shard_sequence(l, L, world, rank)
    dA, dt = cumsum(d["dt"][:, s0:s1], A, L, dt_bias=d["dt_bias"], dt_softplus=True)
    out, fin = P.seqpar_fused_state_fwd(d["B"][:, s0:s1], d["x"][:, s0:s1], dt, dA, torch.bfloat16)
    torch.cuda.synchronize()
    c0 = s0 // L
    scale = out_f.float().abs().max()
    err_out = ((out.float() - out_f[:, c0:c0 + out.shape[1]].float()).abs().max() / scale).item()
    # the state leaving this slice: the next slice's first passed state, or the final state
    if c0 + out.shape[1] < out_f.shape[1]:
        nxt, tol_kind = out_f[:, c0 + out.shape[1]].float(), 0.0
    else:
        nxt, tol_kind = fin_f, 1.0
    err_fin = ((fin - nxt).abs().max() / nxt.abs().max()).item()
    t = torch.tensor([err_out, err_fin if tol_kind == 1.0 else 0.0, err_fin if tol_kind == 0.0 else 0.0],
                     device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    eo, ef, eb = t.tolist()
    return {"world": world, "seqlen": l, "nheads": h, "max_err_out": eo, "max_err_final": ef,
            "max_err_slice_boundary_state_vs_bf16_neighbour": eb,
            "ok": bool(eo <= 1e-2 and ef <= 1e-3 and eb <= 1e-2),
            "tolerance": "passed states 1e-2 of the tensor's max, final state 1e-3"}


def run_extras(args, rank, world, local, dist, dev):
    """The multi-GPU cases beyond the weak headline; returns the dict for the "extra" key."""
    extra = {}
    K = max(3, min(args.steps, 20))
    idx = physical_gpu_index(local) if rank == 0 else None
    # (the head-sharded case first: the seconds of full load of the long sequence leave the GPU at its
    # power cap for a while, which a 0.1 ms step measured right afterwards would inherit)
    extra["cfg2_strong"] = head_sharded_case(dict(WORKLOAD), 5 * K, 20, rank, world, dist, dev, sampler_index=idx)
    seq = seq_sharded_case(dict(SEQ1M), K, 3, rank, world, dist, dev, sampler_index=idx)
    if world > 1:
        # the same step on the whole sequence on ONE GPU, measured in this run (every rank does it on
        # its own GPU, nothing is exchanged; the maximum over ranks is kept)
        one = seq_sharded_case(dict(SEQ1M), max(3, K // 2), 3, 0, 1, None, dev, sampler_index=idx)
        t = torch.tensor([one["ms_per_step"]], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        seq["world1_ms_per_step"] = float(t.item())
        seq["world1_clocks"] = one["clocks"]
        seq["speedup_over_world1"] = seq["world1_ms_per_step"] / seq["ms_per_step"]
    extra["seq1m"] = seq
    if world > 1:
        extra["seqpar_check"] = seqpar_check(rank, world, dist, dev)
    return extra


def run_forward(args, rank, world, local):
    """`--workload forward`: the reference's whole forward pipeline at the headline shape
    (main.py:93-103 there: chunk bmm, state path, chunk scan), one GPU, per-kernel CUDA events.
    Not the contract's metric: the line for profiling the two chunk GEMM kernels."""
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    from mamba_fused_minimal_b200.kernels.rand_data import generate_benchmark_data
    from mamba_fused_minimal_b200.kernels.ssd_bmm import _bmm_chunk_fwd as bmm
    from mamba_fused_minimal_b200.kernels.ssd_chunk_scan import _bmm_chunk_scan_fwd as bmm_scan, _chunk_scan_fwd as scan
    from mamba_fused_minimal_b200.kernels.state_path import _state_path_fwd as state_path
    w = dict(WORKLOAD)
    if args.batch is not None:
        w["batch"] = args.batch
        w["name"] = f"{WORKLOAD['name']}-batch{args.batch}"
    L = w["chunk_size"]
    d = generate_benchmark_data(w["batch"], w["seqlen"], w["nheads"], w["headdim"], w["ngroups"], w["dstate"],
                                dtype=torch.bfloat16, device=dev, seed=rank)
    x, B, C, dt, A, bias, D = d["x"], d["B"], d["C"], d["dt"], d["A"], d["dt_bias"], d["D"].to(torch.bfloat16)

    def step(ev=None):
        # the forward as `_mamba_chunk_scan_combined_fwd_concurrent` of this library runs it: two launches
        if ev:
            ev[0].record()
        dA, dto, passed, fin = state_path(dt, A, B, x, L, torch.bfloat16, dt_bias=bias, dt_softplus=True)
        if ev:
            ev[1].record()
        y, _ = bmm_scan(C, B, x, dto, dA, passed, D=D)
        if ev:
            ev[2].record()
        return y, fin, dA, dto, passed

    ms = _timed_steps(step, args.steps, args.warmup, None, dev)
    Kp = max(3, min(args.steps, 20))
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(Kp)]
    for e in evs:
        y, fin, dA, dto, passed = step(e)
    torch.cuda.synchronize()
    names = ["state_path_ms", "bmm_chunk_scan_one_kernel_ms"]
    kernels = {n: statistics.median(e[i].elapsed_time(e[i + 1]) for e in evs) for i, n in enumerate(names)}
    # the two separate kernels of the reference's call surface, for comparison
    for e in evs:
        e[0].record()
        cb = bmm(C, B, L, output_dtype=torch.float32)
        e[1].record()
        scan(cb, x, dto, dA, C, passed, D=D)
        e[2].record()
    torch.cuda.synchronize()
    kernels["bmm_chunk_ms"] = statistics.median(e[0].elapsed_time(e[1]) for e in evs)
    kernels["chunk_scan_ms"] = statistics.median(e[1].elapsed_time(e[2]) for e in evs)
    # the same two with the z gate (out_x and out = out_x * z * sigmoid(z))
    z = torch.randn_like(x)
    for e in evs:
        e[0].record()
        bmm_scan(C, B, x, dto, dA, passed, D=D, z=z)
        e[1].record()
        scan(cb, x, dto, dA, C, passed, D=D, z=z)
        e[2].record()
    torch.cuda.synchronize()
    kernels["bmm_chunk_scan_one_kernel_gated_ms"] = statistics.median(e[0].elapsed_time(e[1]) for e in evs)
    kernels["chunk_scan_gated_ms"] = statistics.median(e[1].elapsed_time(e[2]) for e in evs)
    from mamba_fused_minimal_b200._ext import C as _C
    _C.check_status(x)
    if rank == 0:
        print(json.dumps({"metric": "ssd_forward_tokens_per_s", "value": w["batch"] * w["seqlen"] / (ms * 1e-3),
                          "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
                          "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
                          "config": dict(workload=w["name"] + " forward (state path, chunk bmm + chunk scan)",
                                         **{k: v for k, v in w.items() if k != "name"}),
                          "kernels": kernels, "gpu_launches": 2 * args.steps}), flush=True)


def run_seq1m(args, rank, world, local):
    """`--workload seq1m`: the long-context case as the line's own workload."""
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    w = dict(SEQ1M)
    if args.seqlen is not None:
        w["seqlen"] = args.seqlen
        w["name"] = f"seq-{args.seqlen}"
    r = seq_sharded_case(w, args.steps, args.warmup, rank, world, dist, dev,
                         sampler_index=physical_gpu_index(local) if rank == 0 else None)
    if rank == 0:
        peak, peak_kind = measured_peak()
        print(json.dumps({
            "metric": "ssd_state_path_tokens_per_s", "value": r["tokens_per_s"], "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": r["ms_per_step"],
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": dict(workload=w["name"], **{k: v for k, v in w.items() if k != "name"},
                           parallelism=f"sequence sharded over {world} GPU(s); all-gather of slice summaries + fix-up",
                           l2="inputs exceed the 126 MB L2; no explicit flush", path_bytes_per_step=r["path_bytes_per_step"]),
            "roofline": {"bound": "hbm", "achieved": r["achieved_gbs"], "peak": peak * world, "unit": "GB/s",
                         "frac": r["frac_of_world_x_peak"], "traffic": None, "peak_kind": peak_kind,
                         "kernel": "whole step (cumsum + fused + exchange + fix-up), all GPUs"},
            "phases": r["phases"], "e2e": None,
            # per rank: state kernel, segment fix-up, logP sum, and (ranks > 0) the cross-rank fix-up
            "gpu_launches": (2 if world == 1 else 4) * args.steps, "clocks": r["clocks"]}), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--skip-e2e", action="store_true", help="profiling aid: device-resident timing only")
    ap.add_argument("--batch", type=int, default=None,
                    help="profiling aid: override the workload's batch (the bench line then names it)")
    ap.add_argument("--workload", default="mamba2-2.7b-layer", choices=["mamba2-2.7b-layer", "seq1m", "forward"],
                    help="seq1m: the 1 M-token sequence-parallel case; forward: bmm + state path + chunk scan with "
                         "per-kernel times (both extra; the default is the contract's workload)")
    ap.add_argument("--seqlen", type=int, default=None, help="seq1m only: override the sequence length")
    ap.add_argument("--summarise-ncu", default=None, metavar="CSV",
                    help="no benchmark: read `ncu -i REPORT --page raw --csv` output of a capture of this script and "
                         "write profiles/fused_state_kernel_traffic.json (use with --batch as captured)")
    ap.add_argument("--ncu-command", default="", help="with --summarise-ncu: the capture command, kept in the summary")
    ap.add_argument("--reference-tree", default=None, metavar="PATH",
                    help="a checkout of the reference project: also time ITS unfused Triton kernels on this GPU "
                         "(key \"triton_unfused\"; single GPU only)")
    ap.add_argument("--no-extras", action="store_true", help="skip the extra multi-GPU cases (key \"extra\")")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.summarise_ncu is not None:
        batch = args.batch if args.batch is not None else WORKLOAD["batch"]
        summarise_ncu(args.summarise_ncu, batch * WORKLOAD["seqlen"], args.ncu_command)
        return

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return
    if world > 1:
        # the only collectives are a 21 MB all-gather and a few scalars: no in-switch reduction needed,
        # and a rank that dies while bound to a multicast object would disturb its peers
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    if args.workload == "seq1m":
        run_seq1m(args, rank, world, local)
        return
    if args.workload == "forward":
        run_forward(args, rank, world, local)
        return
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    from mamba_fused_minimal_b200.kernels.fused_concurrent import _fused_chunk_state_state_passing_fwd_concurrent as fused
    from mamba_fused_minimal_b200.kernels.rand_data import generate_benchmark_data
    from mamba_fused_minimal_b200.kernels.ssd_chunk_state import _chunk_cumsum_fwd as cumsum
    from mamba_fused_minimal_b200.kernels.state_path import _state_path_fwd as state_path

    w = dict(WORKLOAD)
    if args.batch is not None:
        w["batch"] = args.batch
        w["name"] = f"{WORKLOAD['name']}-batch{args.batch}"
    L = w["chunk_size"]
    # every rank: its own shard of 80 heads (seeded by rank), no data shared between ranks
    d = generate_benchmark_data(w["batch"], w["seqlen"], w["nheads"], w["headdim"], w["ngroups"], w["dstate"],
                                dtype=torch.bfloat16, device=dev, seed=rank)
    x, B, dt, A, bias = d["x"], d["B"], d["dt"], d["A"], d["dt_bias"]

    def step():
        return state_path(dt, A, B, x, L, torch.bfloat16, dt_bias=bias, dt_softplus=True)

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()

    sampler = ClockSampler(physical_gpu_index(local)) if rank == 0 else None
    if sampler is not None:
        sampler.start()

    # ---- device-resident timing -----------------------------------------------------
    # The timed region holds nothing but the K steps (events around each kernel would add host
    # work per step, which shows once eight ranks share the host's cores); the split between the
    # two kernels is measured afterwards on a few extra steps.
    K = args.steps
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    start.record()
    for i in range(K):
        dA, dto, out, fin = state_path(dt, A, B, x, L, torch.bfloat16, dt_bias=bias, dt_softplus=True)
    end.record()
    barrier()
    total_ms = start.elapsed_time(end)
    Kp = max(3, min(K, 50))
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(2)] for _ in range(Kp)]
    for i in range(Kp):
        ev[i][0].record()
        dA, dto, out, fin = state_path(dt, A, B, x, L, torch.bfloat16, dt_bias=bias, dt_softplus=True)
        ev[i][1].record()
    barrier()
    fused_ms = [ev[i][0].elapsed_time(ev[i][1]) for i in range(Kp)]
    # the reference's pair of calls, for comparison: cumsum kernel, then the state kernel fed by it
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(Kp)]
    for i in range(Kp):
        ev[i][0].record()
        dA, dto = cumsum(dt, A, L, dt_bias=bias, dt_softplus=True)
        ev[i][1].record()
        out, fin = fused(B, x, dto, dA, torch.bfloat16)
        ev[i][2].record()
    barrier()
    two_calls = {"cumsum_ms": statistics.median(ev[i][0].elapsed_time(ev[i][1]) for i in range(Kp)),
                 "state_kernel_ms": statistics.median(ev[i][1].elapsed_time(ev[i][2]) for i in range(Kp)),
                 "step_ms": statistics.median(ev[i][0].elapsed_time(ev[i][2]) for i in range(Kp)),
                 "note": "_chunk_cumsum_fwd + _fused_chunk_state_state_passing_fwd_concurrent, events around each call"}
    from mamba_fused_minimal_b200._ext import C as _C
    _C.check_status(x)

    e2e_ms, h2d, d2h, Ke = float('nan'), 0, 0, 0
    if not args.skip_e2e:
        # ---- end to end from pinned host buffers --------------------------------------------
        hx, hB, hdt = (t.cpu().pin_memory() for t in (x, B, dt))
        hA, hbias = A.cpu().pin_memory(), bias.cpu().pin_memory()
        nchunks = (w["seqlen"] + L - 1) // L
        h_out = torch.empty((w["batch"], nchunks, w["nheads"], w["headdim"], w["dstate"]), dtype=torch.bfloat16).pin_memory()
        h_fin = torch.empty((w["batch"], w["nheads"], w["headdim"], w["dstate"]), dtype=torch.float32).pin_memory()
        h_dA = torch.empty((w["batch"], w["nheads"], nchunks, L), dtype=torch.float32).pin_memory()
        h_dt = torch.empty_like(h_dA).pin_memory()
        h2d = sum(t.numel() * t.element_size() for t in (hx, hB, hdt, hA, hbias))
        d2h = sum(t.numel() * t.element_size() for t in (h_out, h_fin, h_dA, h_dt))
        # Three streams (copy in, compute, copy out) and two sets of device input buffers, so
        # that step i+1's inputs cross PCIe while step i computes and step i-1's results go back.
        # Every step still copies all of its inputs in and all of its results out.
        dev_in = [tuple(torch.empty_like(t) for t in (x, B, dt, A, bias)) for _ in range(2)]
        s_in, s_cmp, s_out = (torch.cuda.Stream(device=dev) for _ in range(3))
        in_ready = [torch.cuda.Event() for _ in range(2)]
        in_free = [torch.cuda.Event() for _ in range(2)]
        done = torch.cuda.Event()

        def e2e_step(i):
            slot = i % 2
            dx, dB, ddt, dA_, dbias = dev_in[slot]
            with torch.cuda.stream(s_in):
                if i >= 2:
                    s_in.wait_event(in_free[slot])          # the compute that read this slot is done
                dx.copy_(hx, non_blocking=True)
                dB.copy_(hB, non_blocking=True)
                ddt.copy_(hdt, non_blocking=True)
                dA_.copy_(hA, non_blocking=True)
                dbias.copy_(hbias, non_blocking=True)
                in_ready[slot].record(s_in)
            with torch.cuda.stream(s_cmp):
                s_cmp.wait_event(in_ready[slot])
                a, t_, o, f = state_path(ddt, dA_, dB, dx, L, torch.bfloat16, dt_bias=dbias, dt_softplus=True)
                in_free[slot].record(s_cmp)
                done.record(s_cmp)
            with torch.cuda.stream(s_out):
                s_out.wait_event(done)
                for t in (o, f, a, t_):
                    t.record_stream(s_out)
                h_out.copy_(o, non_blocking=True)
                h_fin.copy_(f, non_blocking=True)
                h_dA.copy_(a, non_blocking=True)
                h_dt.copy_(t_, non_blocking=True)

        Ke = max(3, min(K, 20))
        for i in range(2):
            e2e_step(i)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for st in (s_in, s_cmp, s_out):
            st.wait_event(e0)
        for i in range(Ke):
            e2e_step(i + 2)
        for st in (s_in, s_cmp, s_out):
            torch.cuda.current_stream().wait_stream(st)
        e1.record()
        barrier()
        e2e_ms = e0.elapsed_time(e1) / Ke
    clocks = sampler.stop() if sampler is not None else None
    del out, fin, dA, dto
    torch.cuda.empty_cache()
    extra = None
    if not args.no_extras and args.batch is None:
        extra = run_extras(args, rank, world, local, dist, dev)

    # ---- max over ranks ---------------------------------------------------------------
    stats = torch.tensor([total_ms, e2e_ms, statistics.mean(fused_ms)], device=dev, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    total_ms, e2e_ms, fused_mean_ms = (float(v) for v in stats.tolist())

    if rank == 0:
        tokens_per_rank = w["batch"] * w["seqlen"]
        ms_per_step = total_ms / K
        value = world * tokens_per_rank / (ms_per_step * 1e-3)
        peak, peak_kind = measured_peak()
        fused_bytes = algorithmic_bytes(w, with_cumsum=True)      # the kernel reads raw dt and writes dt_out / dA_cumsum
        achieved = fused_bytes / (fused_mean_ms * 1e-3) / 1e9
        traffic, traffic_detail = measured_traffic(tokens_per_rank)
        line = {
            "metric": "ssd_state_path_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": K, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": dict(workload=w["name"], **{k: v for k, v in w.items() if k != "name"},
                           parallelism=f"heads sharded over {world} GPU(s), no collective; one shard per rank",
                           l2="inputs (365 MB read per step) exceed the 126 MB L2; no explicit flush",
                           path_bytes_per_step=algorithmic_bytes(w, with_cumsum=True)),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": traffic, "traffic_detail": traffic_detail,
                         "peak_kind": peak_kind,
                         "kernel": "fused_state_kernel, chunk cumsum inside (the whole path in one launch)",
                         "bytes_per_launch": fused_bytes,
                         "ms_per_launch": fused_mean_ms, "ms_per_launch_median": statistics.median(fused_ms),
                         "frac_of_8TBs": achieved / 8000.0, "two_calls": two_calls},
            "e2e": {"value": world * tokens_per_rank / (e2e_ms * 1e-3), "unit": "tokens/s",
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms, "steps": Ke,
                    "overlap": "copy-in, compute and copy-out of successive steps on three streams, two input slots"},
            "gpu_launches": K,
            "clocks": clocks,
        }
        if extra is not None:
            line["extra"] = extra
        if args.reference_tree is not None and world == 1:
            line["triton_unfused"] = reference_triton_unfused(args.reference_tree, w, dev)
        if not args.no_cpu_baseline and world == 1:
            threads = os.cpu_count() or 1
            tok_s, t, n = cpu_hot_path(WORKLOAD["batch"], threads, 20)
            line["cpu_baseline"] = {"value": tok_s, "unit": "tokens/s", "cores": threads, "kind": "port",
                                    "sample": f"the whole workload, {n} timed passes ({t:.2f} s each, median); "
                                              "torch chunked SSD math on the host"}
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
