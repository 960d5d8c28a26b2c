#!/usr/bin/env python
"""Benchmark of the chunked delta-rule backward (headline: KDA B=8, T=8192, H=32, K=V=128, BF16).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload cfg2_kda]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

A "step" is one complete backward (saved tensors + dO -> dq, dk, dv, dbeta, dg) of the workload on each rank.
Ranks own disjoint batch slices of a global batch of N x B sequences (weak scaling, no collective on the data
path); NCCL is used only for the barriers and the max-reduce of the elapsed time.  Rank 0 prints ONE JSON line.
Inputs are synthetic (seeded, distributions of the benchmark configuration) and far larger than L2 (126 MB),
so every step reads its inputs from HBM.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "delta-rule bwd tokens/s (KDA T=8192 H=32 K=V=128)"
UNIT = "tokens/s"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="rewy_b200", choices=("rewy_b200", "reference"))
    ap.add_argument("--workload", default="cfg2_kda")
    ap.add_argument("--policy", default="saved", choices=("saved", "recompute"),
                    help="activation policy of the headline value (both are timed and reported)")
    ap.add_argument("--batch", type=int, default=None, help="override the per-rank batch size (smaller captures)")
    ap.add_argument("--seq", type=int, default=None, help="override the sequence length")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    return ap.parse_args()


# ---------------------------------------------------------------------------------------------
# clocks
class ClockSampler:
    """Samples nvidia-smi SM clocks and throttle reasons while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.perf_counter(), line.strip()))

    def stop(self, t0, t1):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        rows = [r for t, r in self.rows if t0 <= t <= t1] or [r for _, r in self.rows[-3:]]
        mhz, mx, reasons = [], None, set()
        for r in rows:
            f = [x.strip() for x in r.split(",")]
            if len(f) < 6:
                continue
            try:
                mhz.append(float(f[0]))
                mx = float(f[1])
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(mhz) if mhz else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(mhz)}


# ---------------------------------------------------------------------------------------------
# CPU arm: the reference's naive chunked PyTorch backward on the host cores
def cpu_sample(steps, warmup, T=2048, H=32, heads_of_workload=32):
    """Times the oracle's port of the reference's naive FP32 chunk path (autograd on CPU) on a bounded sample
    of the workload: B=1, T and H as given; tokens/s are normalised to the workload's head count."""
    import torch
    from oracle import naive_chunk_backward_fp32
    from rewy_b200.synthetic import make_inputs, operator_inputs
    xs = make_inputs("kda", 1, T, H, seed=42, gate_scale=0.1, state=False)
    ins = operator_inputs("kda", xs)
    times = []
    for i in range(warmup + steps):
        _, t_f, t_b = naive_chunk_backward_fp32("kda", ins, xs["do"], None)
        if i >= warmup:
            times.append(t_b)
    t = statistics.mean(times)
    token_heads_per_s = T * H / t
    return dict(value=token_heads_per_s / heads_of_workload, unit=UNIT, cores=torch.get_num_threads(), kind="port",
                sample=f"KDA B=1 T={T} H={H} FP32 autograd backward through the naive chunked forward (oracle port of "
                       f"fla naive_chunk_kda); token-heads/s divided by {heads_of_workload} heads; "
                       f"{steps} timed passes of {t * 1e3:.0f} ms; host has {os.cpu_count()} logical CPUs"), t


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch
    steps, warmup = max(1, min(args.steps, 12)), max(1, min(args.warmup, 2))
    base, t = cpu_sample(steps, warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": t * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "KDA backward B=8 T=8192 H=32 K=V=128 chunk=64 (cfg2); CPU arm: each step is a bounded "
                               "sample (B=1, T=2048, all 32 heads) of it"},
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
def main():
    args = parse()
    if args.impl == "reference":
        return run_reference(args)

    import torch
    import torch.distributed as dist
    from rewy_b200 import _capi, backward as bw
    from rewy_b200.forward import chunk_forward
    from rewy_b200.sharding import shard
    from rewy_b200.synthetic import CONFIGS, make_inputs

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ["NCCL_DEBUG"] = os.environ.get("REWY_NCCL_DEBUG", "WARN")  # keep stdout to the one JSON line
        dist.init_process_group("nccl", device_id=dev)
    _capi.load()

    cfg = dict(CONFIGS[args.workload])
    op = cfg.pop("op")
    if op != "kda":
        raise SystemExit("bench.py measures the KDA headline workload")
    B = args.batch or cfg["B"]
    T = args.seq or cfg["T"]
    H = cfg["H"]
    # weak scaling: rank r owns batches [r*B, (r+1)*B) of a global batch of world*B sequences
    xs = make_inputs(op, world * B, T, H, seed=42, device=dev, gate=cfg["gate"], gate_scale=cfg["gate_scale"],
                     state=cfg["state"], batches=shard(world * B, H, world, rank)[0])
    saved = chunk_forward(op, xs["q"], xs["k"], xs["v"], g=xs["g"], beta=xs["beta"], initial_state=xs["initial_state"],
                          output_final_state=False)
    beta32 = xs["beta"].float()
    torch.cuda.synchronize()

    def call(policy_saved, workspace):
        return bw.kda_backward(
            q=xs["q"], k=xs["k"], v=xs["v"], beta=beta32, Aqk=saved["Aqk"], Akk=saved["Akk"], scale=128 ** -0.5,
            initial_state=xs["initial_state"], do=xs["do"], dht=xs["dht"], g=saved["g_cumsum"],
            disable_recompute=policy_saved, w=saved["w"], u=saved["u"], qg=saved["qg"], kg=saved["kg"],
            v_new=saved["v_new"], h=saved["h"], out_dtype=torch.bfloat16, workspace=workspace)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(policy_saved, steps, warmup, sample_clocks=False):
        fam, pol = _capi.KDA, (_capi.SAVED if policy_saved else _capi.RECOMPUTE)
        ws = torch.empty(_capi.workspace_bytes(fam, pol, B, T, H), dtype=torch.uint8, device=dev)
        for _ in range(warmup):
            call(policy_saved, ws)
        barrier()
        sampler = ClockSampler(local) if sample_clocks else None
        if sampler:
            sampler.start()
            time.sleep(0.3)
        _capi.stage_timing_enable(True)
        launches0 = _capi.launch_count()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        t0 = time.perf_counter()
        ev0.record()
        for _ in range(steps):
            call(policy_saved, ws)
        ev1.record()
        barrier()
        t1 = time.perf_counter()
        ms = ev0.elapsed_time(ev1)
        stage_ms, calls = _capi.stage_timing_read()
        _capi.stage_timing_enable(False)
        launches = _capi.launch_count() - launches0
        clocks = sampler.stop(t0, t1) if sampler else None
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        del ws
        return ms / steps, {k: v / max(calls, 1) for k, v in stage_ms.items()}, launches, clocks

    K, W = args.steps, max(args.warmup, 3)
    head_saved = args.policy == "saved"
    ms_head, stages_head, launches, clocks = timed(head_saved, K, W, sample_clocks=True)
    ms_other, stages_other, _, _ = timed(not head_saved, K, W)
    tokens = world * B * T
    value = tokens / (ms_head * 1e-3)

    # roofline of the dominant kernel of the headline policy
    peaks_file = ROOT / "MEASURED_PEAKS.json"
    if peaks_file.exists():
        peak, peak_src = json.loads(peaks_file.read_text())["hbm_gbs"], "measured (MEASURED_PEAKS.json hbm_gbs)"
    else:
        peak, peak_src = 6650.0, "fallback 6.65 TB/s"
    n_th = B * T * H                      # token-heads one launch processes on one rank
    state_bytes = 2 * 65536 * B * H if cfg["state"] else 0
    alg = {  # algorithmic bytes per token-head of each kernel (inputs read once + outputs written once)
        "prepare": 4 * 256 + 512 + 4 + 128 + 4 * 256,
        "fwd_scan": 3 * 256 + 8 + 512 + 256,
        "bwd_scan": 4 * 256 + 128 + 8 + 512 + 2 * 256,
        "chunk_adjoint": 5 * 256 + 512 + 4 + 128 + 2 * 512 + 2 * 256 + 3 * 256 + 512 + 4,
    }
    # DRAM bytes per token-head from the ncu captures summarised under profiles/ (B=4,T=2048,H=32; per-token-head
    # traffic of these kernels does not depend on B or T), scaled to this launch
    ncu_traffic = {"chunk_adjoint": 4645, "bwd_scan": 2036}
    dom = max(stages_head, key=lambda s: stages_head[s])
    dom_ms = stages_head[dom]
    achieved = alg[dom] * n_th / (dom_ms * 1e-3) / 1e9 if dom_ms > 0 else 0.0
    path_bytes = (4616 if head_saved else 3080) * n_th + state_bytes
    roofline = {
        "bound": "hbm", "kernel": dom, "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
        "traffic": ncu_traffic[dom] * n_th if dom in ncu_traffic else None,
        "traffic_source": "profiles/ (ncu dram__bytes_read+write per token-head on a smaller case, scaled)",
        "peak_source": peak_src, "ms_per_launch": dom_ms,
        "algorithmic_bytes_per_token_head": alg[dom],
        "whole_path": {"algorithmic_bytes_per_token_head": path_bytes / n_th,
                       "achieved": path_bytes / (ms_head * 1e-3) / 1e9, "frac": path_bytes / (ms_head * 1e-3) / 1e9 / peak},
        "stage_ms": stages_head,
    }

    # end to end through the family function with HOST buffers (pinned), copies inside the timed region
    def measure_e2e(pol_saved):
        names_in = ["q", "k", "v", "do"]
        host_in = {n: xs[n] for n in names_in}
        host_in.update(beta=beta32, g=saved["g_cumsum"], Aqk=saved["Aqk"], Akk=saved["Akk"])
        if pol_saved:
            host_in.update({n: saved[n] for n in ("w", "qg", "kg", "v_new", "h")})
        if xs["initial_state"] is not None:
            host_in.update(h0=xs["initial_state"], dht=xs["dht"])
        pinned = {n: torch.empty(t.shape, dtype=t.dtype, pin_memory=True).copy_(t) for n, t in host_in.items()}
        h2d = sum(t.numel() * t.element_size() for t in pinned.values())
        fam, pol = _capi.KDA, (_capi.SAVED if pol_saved else _capi.RECOMPUTE)
        # The path is independent per batch element, so the host-facing call streams it: one batch element per call,
        # two sets of device buffers, and three streams so that the copy in, the backward and the copy out overlap.
        slots = [{n: torch.empty((1,) + tuple(t.shape[1:]), dtype=t.dtype, device=dev) for n, t in host_in.items()}
                 for _ in range(2)]
        ws_slot = [torch.empty(_capi.workspace_bytes(fam, pol, 1, T, H), dtype=torch.uint8, device=dev) for _ in range(2)]
        s_in, s_comp, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
        out_host = None

        def e2e_step():
            nonlocal out_host
            cur = torch.cuda.current_stream()
            for st in (s_in, s_comp, s_out):
                st.wait_stream(cur)
            computed = [None, None]
            keep, nbytes = [], 0
            for ib in range(B):
                slot = ib % 2
                d = slots[slot]
                with torch.cuda.stream(s_in):
                    if computed[slot] is not None:
                        s_in.wait_event(computed[slot])  # the slot's previous batch element has been consumed
                    for n, t in pinned.items():
                        d[n].copy_(t[ib:ib + 1], non_blocking=True)
                    arrived = torch.cuda.Event()
                    arrived.record(s_in)
                with torch.cuda.stream(s_comp):
                    s_comp.wait_event(arrived)
                    r = bw.kda_backward(
                        q=d["q"], k=d["k"], v=d["v"], beta=d["beta"], Aqk=d["Aqk"], Akk=d["Akk"], scale=128 ** -0.5,
                        initial_state=d.get("h0"), do=d["do"], dht=d.get("dht"), g=d["g"], disable_recompute=pol_saved,
                        w=d.get("w"), qg=d.get("qg"), kg=d.get("kg"), v_new=d.get("v_new"), h=d.get("h"),
                        out_dtype=torch.bfloat16, workspace=ws_slot[slot])
                    computed[slot] = torch.cuda.Event()
                    computed[slot].record(s_comp)
                outs = [t for t in r if t is not None]
                if out_host is None:
                    out_host = [torch.empty((B,) + tuple(t.shape[1:]), dtype=t.dtype, pin_memory=True) for t in outs]
                with torch.cuda.stream(s_out):
                    s_out.wait_event(computed[slot])
                    for hb, t in zip(out_host, outs):
                        hb[ib:ib + 1].copy_(t, non_blocking=True)
                        t.record_stream(s_out)
                keep.append(outs)
                nbytes += sum(t.numel() * t.element_size() for t in outs)
            for st in (s_in, s_comp, s_out):
                cur.wait_stream(st)
            return nbytes

        e_steps = max(1, min(K, 3))
        d2h = e2e_step()
        barrier()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for _ in range(e_steps):
            e2e_step()
        ev1.record()
        barrier()
        ms = ev0.elapsed_time(ev1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return {"value": tokens / (ms / e_steps * 1e-3), "unit": UNIT, "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": d2h, "steps": e_steps, "ms_per_step": ms / e_steps,
               "api": "rewy_b200.backward.kda_backward (the function the autograd backward calls), one batch element per "
                      "call, pinned host inputs copied H2D and gradients copied D2H every step on three streams "
                      "(copy in, backward, copy out overlap)"}

    e2e = e2e_other = None
    if not args.no_e2e:
        e2e = measure_e2e(head_saved)
        e2e_other = measure_e2e(not head_saved)
        e2e_other["policy"] = "recompute" if head_saved else "full saving"

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu_baseline, _ = cpu_sample(steps=2, warmup=1)

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms_head, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"KDA backward B={B} per GPU, T={T}, H={H}, K=V=128, chunk=64 ({args.workload})",
                       "policy": "full saving (disable_recompute=True)" if head_saved else "recompute",
                       "global_batch": world * B, "parallelism": f"(batch,head) shards x{world}, no collective",
                       "l2": "inputs (>= 9 GB per step) are far larger than the 126 MB L2; no flush needed",
                       "outputs": "dq,dk,dv BF16; dg,dbeta FP32"},
            "policies": {("saved" if head_saved else "recompute"): {"tokens_per_s": value, "ms_per_step": ms_head,
                                                                     "stage_ms": stages_head},
                         ("recompute" if head_saved else "saved"): {"tokens_per_s": tokens / (ms_other * 1e-3),
                                                                     "ms_per_step": ms_other, "stage_ms": stages_other}},
            "token_heads_per_s": value * H,
            "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e, "e2e_other_policy": e2e_other, "clocks": clocks,
            "gpu_launches": launches,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
