#!/usr/bin/env python
"""Benchmark of the chunked delta-rule backward (headline: KDA B=8, T=8192, H=32, K=V=128, BF16).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload cfg2_kda]
                    [--scaling weak|strong] [--policy saved|recompute]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

A "step" is one complete backward (saved tensors + dO -> every gradient) of the workload on each rank, called through
the whole-family function the autograd backward calls.  Ranks own disjoint (batch, head) shards and there is no
collective on the data path; NCCL carries only the barriers and the max-reduce of the elapsed time.
  --scaling weak    (default) every rank holds the workload's full batch: global batch = N x B
  --scaling strong  the workload's batch is fixed and split by (batch, head): batches first, then heads
Rank 0 prints ONE JSON line.  Inputs are synthetic (seeded, distributions of the benchmark configuration) and far
larger than L2 (126 MB), so every step reads its inputs from HBM.  At N=1 the line also carries the other benchmark
configurations ("families"), the reference's Triton backward on the same GPU ("triton_baseline", timed in a child
process) and the CPU arm ("cpu_baseline").
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

UNIT = "tokens/s"
SCALE = 128 ** -0.5


def metric_name(workload, policy_saved):
    from rewy_b200.synthetic import CONFIGS
    c = CONFIGS[workload]
    fam = {"kda": "KDA", "gdn": "GDN", "gdn2": "GDN2", "delta": "DeltaNet"}[c["op"]]
    pol = ("full-saving policy" if policy_saved else "recompute policy") if c["op"] in ("kda", "gdn2") else "recompute policy"
    return f"delta-rule bwd tokens/s ({fam} T={c['T']} H={c['H']} K=V=128, {pol})"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="rewy_b200", choices=("rewy_b200", "reference"))
    ap.add_argument("--workload", default="cfg2_kda", choices=("cfg1_gdn", "cfg2_kda", "cfg3_delta", "cfg4_gdn2"))
    ap.add_argument("--scaling", default="weak", choices=("weak", "strong"))
    ap.add_argument("--policy", default="saved", choices=("saved", "recompute"),
                    help="activation policy of the headline value (both are timed and reported)")
    ap.add_argument("--batch", type=int, default=None, help="override the workload's batch size (smaller captures)")
    ap.add_argument("--seq", type=int, default=None, help="override the sequence length")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-families", action="store_true")
    ap.add_argument("--no-triton", action="store_true")
    return ap.parse_args()


# ---------------------------------------------------------------------------------------------
# clocks
class ClockSampler:
    """Samples the SM clock and the throttle reasons of one GPU while the timed region runs (read-only NVML queries
    from a thread, every few milliseconds; nvidia-smi in a loop if the NVML binding is missing)."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    REASONS = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40}

    def __init__(self, index, uuid=None):
        self.index, self.uuid, self.rows, self.proc, self.nvml = index, uuid, [], None, None
        self.stop_flag = threading.Event()
        self.max_mhz = None

    def _physical_index(self):
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            ids = [x.strip() for x in vis.split(",") if x.strip()]
            if self.index < len(ids) and ids[self.index].isdigit():
                return int(ids[self.index])
        return self.index

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nvml = pynvml
            if self.uuid:   # the CUDA device's own UUID: immune to CUDA_VISIBLE_DEVICES renumbering
                self.handle = pynvml.nvmlDeviceGetHandleByUUID(self.uuid.encode())
            else:
                self.handle = pynvml.nvmlDeviceGetHandleByIndex(self._physical_index())
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            self.thread = threading.Thread(target=self._poll_nvml, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.nvml = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self._physical_index()}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read_smi, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _poll_nvml(self):
        nv = self.nvml
        while not self.stop_flag.is_set():
            try:
                mhz = float(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM))
                mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle))
            except Exception:
                break
            self.rows.append((time.perf_counter(), mhz, {n for n, bit in self.REASONS.items() if mask & bit}))
            time.sleep(0.004)

    def _read_smi(self):
        for line in self.proc.stdout:
            f = [x.strip() for x in line.split(",")]
            try:
                mhz, self.max_mhz = float(f[0]), float(f[1])
            except (ValueError, IndexError):
                continue
            names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
            self.rows.append((time.perf_counter(), mhz, {n for n, v in zip(names, f[2:6]) if v.lower().startswith("active")}))

    def stop(self, t0, t1):
        """Summary of the samples taken between t0 and t1 (perf_counter); if the region was shorter than one sampling
        period, of the samples closest to it (the warm-up just before runs the same load)."""
        time.sleep(0.03)
        self.stop_flag.set()
        if self.proc is not None:
            self.proc.terminate()
        if self.nvml is None and self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no NVML binding and no nvidia-smi"], "samples": 0}
        inside = [r for r in self.rows if t0 <= r[0] <= t1]
        where = "inside the timed region"
        if not inside:
            inside = sorted(self.rows, key=lambda r: min(abs(r[0] - t0), abs(r[0] - t1)))[:5]
            where = "nearest to the timed region (it was shorter than one sampling period)"
        reasons = set()
        for r in inside:
            reasons |= r[2]
        mhz = [r[1] for r in inside]
        return {"sm_mhz": statistics.median(mhz) if mhz else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(reasons),
                "samples": len(mhz), "sampled": where, "source": "NVML" if self.nvml is not None else "nvidia-smi"}


# ---------------------------------------------------------------------------------------------
# CPU arm: the reference's naive chunked PyTorch backward on the host cores
def cpu_sample(steps, warmup, T=2048, H=32, heads_of_workload=32):
    """Times the oracle's port of the reference's naive FP32 chunk path (autograd on CPU) on a bounded sample
    of the workload: B=1, T and H as given; tokens/s are normalised to the workload's head count."""
    import torch
    from oracle import naive_chunk_backward_fp32
    from rewy_b200.synthetic import make_inputs, operator_inputs
    # every logical CPU of the host, whatever the launcher exported (torch.distributed.run sets OMP_NUM_THREADS=1)
    torch.set_num_threads(os.cpu_count() or 1)
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
                       f"{steps} timed passes of {t * 1e3:.0f} ms; {torch.get_num_threads()} threads on "
                       f"{os.cpu_count()} logical CPUs"), t


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps, warmup = max(1, min(args.steps, 12)), max(1, min(args.warmup, 2))
    base, t = cpu_sample(steps, warmup)
    line = {
        "impl": "reference", "metric": metric_name("cfg2_kda", args.policy == "saved"), "value": base["value"],
        "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": t * 1e3, "higher_is_better": True, "scaling": args.scaling,
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "KDA backward B=8 T=8192 H=32 K=V=128 chunk=64 (cfg2); CPU arm: each step is a bounded "
                               "sample (B=1, T=2048, all 32 heads) of it"},
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
# boundary bytes per token-head: every input of the family function read once, every gradient written once, public
# dtypes (BF16 q,k,v,dO,dq,dk,dv and saved tensors; FP32 gates, beta and their gradients); states amortised over T
def boundary_bytes(op, policy_saved, T, state):
    base = {"kda": (3080, 4616), "gdn2": (4096, 5632), "gdn": (1936, 1936), "delta": (1928, 1928)}[op][1 if policy_saved else 0]
    return base + (3 * 65536 / T if state else 0.0)


class Problem:
    """One rank's shard of a benchmark configuration, resident on the device, with its saved forward tensors."""

    def __init__(self, name, dev, world=1, rank=0, scaling="weak", batch=None, seq=None):
        import torch
        from rewy_b200.forward import chunk_forward
        from rewy_b200.sharding import shard
        from rewy_b200.synthetic import CONFIGS, make_inputs
        cfg = dict(CONFIGS[name])
        self.name, self.op = name, cfg.pop("op")
        B, self.T, self.H = batch or cfg["B"], seq or cfg["T"], cfg["H"]
        self.state = cfg["state"]
        if scaling == "weak":   # rank r owns batches [r*B, (r+1)*B) of a global batch of world*B sequences
            self.global_B = world * B
            batches, heads = shard(world * B, self.H, world, rank)
        else:                   # the configuration's batch is fixed and split by (batch, head)
            self.global_B = B
            batches, heads = shard(B, self.H, world, rank)
        self.B, self.nh = len(batches), len(heads)
        self.shard = f"batches {batches[0]}..{batches[-1]}, heads {heads[0]}..{heads[-1]}"
        xs = make_inputs(self.op, self.global_B, self.T, self.H, seed=42, device=dev, gate=cfg["gate"],
                         gate_scale=cfg["gate_scale"], state=cfg["state"], batches=batches, heads=heads)
        self.xs = xs
        self.sv = chunk_forward(self.op, xs["q"], xs["k"], xs["v"], g=xs.get("g"), beta=xs.get("beta"), b=xs.get("b"),
                                w=xs.get("w"), initial_state=xs.get("initial_state"), output_final_state=False)
        self.sv.pop("o", None)
        self.beta32 = xs["beta"].float() if "beta" in xs else None
        self.dev = dev
        self.policies = (True, False) if self.op in ("kda", "gdn2") else (False,)
        torch.cuda.synchronize()

    @property
    def token_heads(self):
        return self.B * self.T * self.nh

    def family_policy(self, policy_saved):
        from rewy_b200 import _capi
        return _capi.FAMILY_ID[self.op], (_capi.SAVED if policy_saved else _capi.RECOMPUTE)

    def workspace(self, policy_saved):
        import torch
        from rewy_b200 import _capi
        fam, pol = self.family_policy(policy_saved)
        return torch.empty(_capi.workspace_bytes(fam, pol, self.B, self.T, self.nh), dtype=torch.uint8, device=self.dev)

    def call(self, policy_saved, workspace, xs=None, sv=None, beta32=None):
        import torch
        from rewy_b200 import backward as bw
        xs, sv = xs or self.xs, sv or self.sv
        beta32 = self.beta32 if beta32 is None else beta32
        common = dict(q=xs["q"], k=xs["k"], v=xs["v"], scale=SCALE, initial_state=xs.get("initial_state"), do=xs["do"],
                      dht=xs.get("dht"), out_dtype=torch.bfloat16, workspace=workspace)
        keep = (lambda n: sv.get(n)) if policy_saved else (lambda n: None)
        if self.op == "kda":
            return bw.kda_backward(beta=beta32, Aqk=sv["Aqk"], Akk=sv["Akk"], g=sv["g_cumsum"],
                                   disable_recompute=policy_saved, w=keep("w"), u=keep("u"), qg=keep("qg"), kg=keep("kg"),
                                   v_new=keep("v_new"), h=keep("h"), **common)
        if self.op == "gdn2":
            return bw.gdn2_backward(b=xs["b"], w_gate=xs["w"], Aqk=sv["Aqk"], Akk=sv["Akk"], g=sv["g_cumsum"],
                                    disable_recompute=policy_saved, w_wy=keep("w"), u_wy=keep("u"), qg=keep("qg"),
                                    kg=keep("kg"), v_new=keep("v_new"), h=keep("h"), **common)
        if self.op == "gdn":
            return bw.gdn_backward(g=sv["g_cumsum"], beta=beta32, A=sv["Akk"], **common)
        return bw.delta_backward(beta=beta32, A=sv["Akk"], **common)


def main():
    args = parse()
    if args.impl == "reference":
        return run_reference(args)

    import torch
    import torch.distributed as dist
    from rewy_b200 import _capi

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)   # NCCL logs to stderr; stdout stays the one JSON line
    _capi.load()
    try:
        gpu_uuid = "GPU-" + str(torch.cuda.get_device_properties(local).uuid)
    except Exception:
        gpu_uuid = None

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())
        return ms

    def timed(prob, policy_saved, steps, warmup, sample_clocks=False):
        ws = prob.workspace(policy_saved)
        sampler = ClockSampler(local, gpu_uuid) if sample_clocks else None
        if sampler:
            sampler.start()
        for _ in range(warmup):
            prob.call(policy_saved, ws)
        barrier()
        _capi.stage_timing_enable(True)
        launches0 = _capi.launch_count()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        t0 = time.perf_counter()
        ev0.record()
        for _ in range(steps):
            prob.call(policy_saved, ws)
        ev1.record()
        barrier()
        t1 = time.perf_counter()
        ms = ev0.elapsed_time(ev1)
        stage_ms, calls = _capi.stage_timing_read()
        _capi.stage_timing_enable(False)
        launches = _capi.launch_count() - launches0
        clocks = sampler.stop(t0, t1) if sampler else None
        ms = max_over_ranks(ms)
        del ws
        return ms / steps, {k: v / max(calls, 1) for k, v in stage_ms.items()}, launches, clocks

    K, W = args.steps, max(args.warmup, 3)
    prob = Problem(args.workload, dev, world, rank, args.scaling, args.batch, args.seq)
    head_saved = args.policy == "saved" and True in prob.policies
    ms_head, stages_head, launches, clocks = timed(prob, head_saved, K, W, sample_clocks=True)
    policies = {("saved" if head_saved else "recompute"): {"ms_per_step": ms_head, "stage_ms": stages_head}}
    if len(prob.policies) > 1:
        ms_other, stages_other, _, _ = timed(prob, not head_saved, K, W)
        policies["recompute" if head_saved else "saved"] = {"ms_per_step": ms_other, "stage_ms": stages_other}
    tokens = prob.global_B * prob.T
    for p in policies.values():
        p["tokens_per_s"] = tokens / (p["ms_per_step"] * 1e-3)
    value = tokens / (ms_head * 1e-3)

    # roofline of the dominant kernel of the headline policy
    peaks_file = ROOT / "MEASURED_PEAKS.json"
    if peaks_file.exists():
        peak, peak_src = json.loads(peaks_file.read_text())["hbm_gbs"], "measured (MEASURED_PEAKS.json hbm_gbs)"
    else:
        peak, peak_src = 6650.0, "fallback 6.65 TB/s"
    n_th = prob.token_heads               # token-heads one launch processes on this rank
    vec = prob.op in ("kda", "gdn2")
    gate_b = 512 if vec else (4 if prob.op == "gdn" else 0)
    extra_gates = 2 * 256 if prob.op == "gdn2" else 4             # GDN2: b and w gates; others: beta
    alg = {  # algorithmic bytes per token-head of each kernel (its operands read once + its results written once)
        "prepare": 3 * 256 + gate_b + extra_gates + 128 + 4 * 256 + (0 if vec else 128),
        "fwd_scan": 3 * 256 + (8 if vec else 0) + 512 + 256,
        "bwd_scan": 4 * 256 + 128 + (8 if vec else 0) + 512 + 2 * 256,
        "chunk_adjoint": 5 * 256 + gate_b + extra_gates + 128 + 2 * 512 + 2 * 256 + 3 * 256 + gate_b + extra_gates,
    }
    # DRAM bytes per token-head measured with ncu on a smaller case of the same kernels (the per-token-head traffic of
    # these kernels does not depend on B or T); the file is rewritten whenever the captures are refreshed
    traffic_file = ROOT / "profiles" / "traffic.json"
    ncu_traffic = json.loads(traffic_file.read_text()) if traffic_file.exists() else {}
    dom = max(stages_head, key=lambda s: stages_head[s])
    dom_ms = stages_head[dom]
    achieved = alg[dom] * n_th / (dom_ms * 1e-3) / 1e9 if dom_ms > 0 else 0.0
    per_th = boundary_bytes(prob.op, head_saved, prob.T, prob.state)
    path_bytes = per_th * n_th
    t_entry = ncu_traffic.get(f"{prob.op}:{dom}")
    roofline = {
        "bound": "hbm", "kernel": dom, "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
        "traffic": t_entry["dram_bytes_per_token_head"] * n_th if t_entry else None,
        "traffic_source": (f"ncu dram__bytes_read+write per token-head on {t_entry['captured_on']}, scaled by "
                           f"token-heads" if t_entry else None),
        "peak_source": peak_src, "ms_per_launch": dom_ms,
        "algorithmic_bytes_per_token_head": alg[dom],
        "whole_path": {"algorithmic_bytes_per_token_head": per_th,
                       "achieved": path_bytes / (ms_head * 1e-3) / 1e9, "frac": path_bytes / (ms_head * 1e-3) / 1e9 / peak},
        "stage_ms": stages_head,
    }

    # end to end through the family function with HOST buffers (pinned), copies inside the timed region
    def measure_e2e(pol_saved):
        xs, sv = prob.xs, prob.sv
        host_in = {n: xs[n] for n in ("q", "k", "v", "do")}
        host_in.update(beta=prob.beta32, g_cumsum=sv["g_cumsum"], Aqk=sv["Aqk"], Akk=sv["Akk"])
        if pol_saved:
            host_in.update({n: sv[n] for n in ("w", "qg", "kg", "v_new", "h")})
        if xs["initial_state"] is not None:
            host_in.update(initial_state=xs["initial_state"], dht=xs["dht"])
        pinned = {n: torch.empty(t.shape, dtype=t.dtype, pin_memory=True).copy_(t) for n, t in host_in.items()}
        h2d = sum(t.numel() * t.element_size() for t in pinned.values())
        fam, pol = prob.family_policy(pol_saved)
        # The path is independent per batch element, so the host-facing call streams it: one batch element per call,
        # two sets of device buffers, and three streams so that the copy in, the backward and the copy out overlap.
        slots = [{n: torch.empty((1,) + tuple(t.shape[1:]), dtype=t.dtype, device=dev) for n, t in host_in.items()}
                 for _ in range(2)]
        ws_slot = [torch.empty(_capi.workspace_bytes(fam, pol, 1, prob.T, prob.nh), dtype=torch.uint8, device=dev)
                   for _ in range(2)]
        s_in, s_comp, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
        out_host = None

        def e2e_step():
            nonlocal out_host
            cur = torch.cuda.current_stream()
            for st in (s_in, s_comp, s_out):
                st.wait_stream(cur)
            computed = [None, None]
            keep, nbytes = [], 0
            for ib in range(prob.B):
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
                    dx = dict(q=d["q"], k=d["k"], v=d["v"], do=d["do"], initial_state=d.get("initial_state"),
                              dht=d.get("dht"))
                    r = prob.call(pol_saved, ws_slot[slot], xs=dx, sv=d, beta32=d["beta"])
                    computed[slot] = torch.cuda.Event()
                    computed[slot].record(s_comp)
                outs = [t for t in r if t is not None]
                if out_host is None:
                    out_host = [torch.empty((prob.B,) + tuple(t.shape[1:]), dtype=t.dtype, pin_memory=True) for t in outs]
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
        ms = max_over_ranks(ev0.elapsed_time(ev1))
        return {"value": tokens / (ms / e_steps * 1e-3), "unit": UNIT, "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "steps": e_steps, "ms_per_step": ms / e_steps,
                "api": "rewy_b200.backward.kda_backward (the function the autograd backward calls), one batch element per "
                       "call, pinned host inputs copied H2D and gradients copied D2H every step on three streams "
                       "(copy in, backward, copy out overlap)"}

    # the forward that produces the saved set (not part of the metric: the reference's forward is FLA's, unchanged)
    forward = None
    if world == 1:
        from rewy_b200.forward import chunk_forward
        x = prob.xs

        def fwd():
            return chunk_forward(prob.op, x["q"], x["k"], x["v"], g=x.get("g"), beta=x.get("beta"), b=x.get("b"),
                                 w=x.get("w"), initial_state=x.get("initial_state"), output_final_state=False)
        try:
            for _ in range(3):
                fwd()
            f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            f0.record()
            for _ in range(min(K, 10)):
                fwd()
            f1.record()
            torch.cuda.synchronize()
            fms = f0.elapsed_time(f1) / min(K, 10)
            forward = {"ms_per_step": fms, "tokens_per_s": tokens / (fms * 1e-3),
                       "note": "rewy_chunk_fwd incl. the gate cumsum and the allocation of the saved set by torch"}
        except Exception as exc:  # e.g. out of memory beside the resident problem: report, keep the headline
            forward = {"unavailable": f"{type(exc).__name__}: {str(exc)[:200]}"}
        torch.cuda.empty_cache()

    e2e = e2e_other = None
    if not args.no_e2e and prob.op == "kda":
        e2e = measure_e2e(head_saved)
        e2e_other = measure_e2e(not head_saved)
        e2e_other["policy"] = "recompute" if head_saved else "full saving"

    workload_desc = (f"{prob.op.upper()} backward B={prob.global_B} global ({prob.B} x {prob.nh} heads on this rank), "
                     f"T={prob.T}, H={prob.H}, K=V=128, chunk=64 ({args.workload})")
    global_batch, n_heads = prob.global_B, prob.H
    del prob
    torch.cuda.empty_cache()

    # the other benchmark configurations, same public functions, device-resident inputs (N=1 only)
    families = None
    if world == 1 and not args.no_families and args.workload == "cfg2_kda" and args.batch is None and args.seq is None:
        families = {}
        for name in ("cfg1_gdn", "cfg3_delta", "cfg4_gdn2"):
            try:
                fp = Problem(name, dev)
                entry = {"workload": f"{fp.op} B={fp.B} T={fp.T} H={fp.H}", "token_heads": fp.token_heads}
                for pol_saved in fp.policies:
                    ms, st, _, _ = timed(fp, pol_saved, min(K, 10), 3)
                    bb = boundary_bytes(fp.op, pol_saved, fp.T, fp.state)
                    entry["saved" if pol_saved else "recompute"] = {
                        "ms_per_step": ms, "tokens_per_s": fp.B * fp.T / (ms * 1e-3),
                        "token_heads_per_s": fp.token_heads / (ms * 1e-3), "stage_ms": st,
                        "boundary_bytes_per_token_head": bb,
                        "whole_path_frac_of_hbm_peak": bb * fp.token_heads / (ms * 1e-3) / 1e9 / peak}
                families[name] = entry
                del fp
            except Exception as exc:  # e.g. out of memory on a smaller device: report, keep the headline
                families[name] = {"unavailable": f"{type(exc).__name__}: {str(exc)[:200]}"}
            torch.cuda.empty_cache()

    # the reference's Triton backward on this GPU, in a child process (its own CUDA context; a failure there cannot
    # take the headline down).  N=1 only.
    triton_baseline = None
    if rank == 0 and world == 1 and not args.no_triton and args.workload == "cfg2_kda":
        cmd = [sys.executable, str(ROOT / "baseline" / "triton_reference.py"), "--steps", str(min(K, 10)), "--warmup", "3",
               "--policy", "saved" if head_saved else "recompute"]
        if args.batch:
            cmd += ["--batch", str(args.batch)]
        if args.seq:
            cmd += ["--seq", str(args.seq)]
        try:
            r = subprocess.run(cmd, capture_output=True, text=True, timeout=420,
                               env=dict(os.environ, CUDA_VISIBLE_DEVICES=os.environ.get("CUDA_VISIBLE_DEVICES", str(local))))
            lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
            triton_baseline = json.loads(lines[-1]) if lines else {
                "unavailable": f"exit code {r.returncode}: {r.stderr.strip()[-300:]}"}
        except subprocess.TimeoutExpired:
            triton_baseline = {"unavailable": "the child process did not finish within 420 s"}
        ref_arm = (triton_baseline or {}).get("reference_optimized") or {}
        if "ms" in ref_arm:
            triton_baseline["speedup_of_this_library"] = ref_arm["ms"] / ms_head

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu_baseline, _ = cpu_sample(steps=2, warmup=1)

    if rank == 0:
        line = {
            "metric": metric_name(args.workload, head_saved), "value": value, "unit": UNIT, "n_gpus": world, "steps": K,
            "warmup": W, "ms_per_step": ms_head, "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": workload_desc,
                       "policy": "full saving (disable_recompute=True)" if head_saved else "recompute",
                       "global_batch": global_batch,
                       "parallelism": f"(batch,head) shards x{world}, no collective",
                       "l2": "inputs are far larger than the 126 MB L2; no flush needed",
                       "outputs": "dq,dk,dv (and GDN2's db,dw) BF16; dg,dbeta FP32"},
            "policies": policies, "token_heads_per_s": value * n_heads,
            "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e, "e2e_other_policy": e2e_other, "clocks": clocks,
            "gpu_launches": launches, "forward": forward, "families": families, "triton_baseline": triton_baseline,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
