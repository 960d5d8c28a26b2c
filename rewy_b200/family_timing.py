"""Times the backward of every family on the current GPU and prints one JSON line per case.

    python -m rewy_b200.family_timing [--steps 10] [--warmup 3] [--token-heads 2097152]

The headline benchmark (``bench.py``) measures KDA only; this utility runs the other reference shapes
(Gated DeltaNet B=4 T=4096 H=16, DeltaNet B=16 T=2048 H=16, GDN2 T=32768 H=32) through the same public
backward functions, with inputs resident on the device and CUDA events on the current stream.  The
batch of a case is reduced so that it holds at most ``--token-heads`` token-heads (the headline KDA case
holds 2 097 152), which bounds the memory of the torch forward that produces the saved tensors.
"""
from __future__ import annotations

import argparse
import json

import torch

from . import backward as bw
from .forward import chunk_forward
from .synthetic import CONFIGS, make_inputs


def _case(name, steps, warmup, max_token_heads):
    cfg = dict(CONFIGS[name])
    op, B, T, H = cfg.pop("op"), cfg.pop("B"), cfg.pop("T"), cfg.pop("H")
    B = max(1, min(B, max_token_heads // (T * H)))
    dev = torch.device("cuda")
    xs = make_inputs(op, B, T, H, device=dev, **cfg)
    scale = 128 ** -0.5
    sv = chunk_forward(op, xs["q"], xs["k"], xs["v"], g=xs.get("g"), beta=xs.get("beta"), b=xs.get("b"),
                       w=xs.get("w"), initial_state=xs.get("initial_state"))
    h0, do, dht = xs.get("initial_state"), xs["do"], xs.get("dht")

    def call(saved):
        if op == "kda":
            extra = dict(w=sv["w"], u=sv["u"], qg=sv["qg"], kg=sv["kg"], v_new=sv["v_new"], h=sv["h"]) if saved else {}
            return bw.kda_backward(q=xs["q"], k=xs["k"], v=xs["v"], beta=xs["beta"], Aqk=sv["Aqk"], Akk=sv["Akk"],
                                   scale=scale, initial_state=h0, do=do, dht=dht, g=sv["g_cumsum"],
                                   disable_recompute=saved, out_dtype=torch.bfloat16, **extra)
        if op == "gdn2":
            extra = dict(w_wy=sv["w"], u_wy=sv["u"], qg=sv["qg"], kg=sv["kg"], v_new=sv["v_new"], h=sv["h"]) if saved else {}
            return bw.gdn2_backward(q=xs["q"], k=xs["k"], v=xs["v"], b=xs["b"], w_gate=xs["w"], Aqk=sv["Aqk"],
                                    Akk=sv["Akk"], scale=scale, initial_state=h0, do=do, dht=dht, g=sv["g_cumsum"],
                                    disable_recompute=saved, out_dtype=torch.bfloat16, **extra)
        if op == "gdn":
            return bw.gdn_backward(q=xs["q"], k=xs["k"], v=xs["v"], g=sv["g_cumsum"], beta=xs["beta"], A=sv["Akk"],
                                   scale=scale, initial_state=h0, do=do, dht=dht, out_dtype=torch.bfloat16)
        return bw.delta_backward(q=xs["q"], k=xs["k"], v=xs["v"], beta=xs["beta"], A=sv["Akk"], scale=scale,
                                 initial_state=h0, do=do, dht=dht, out_dtype=torch.bfloat16)

    out = {"case": name, "family": op, "B": B, "T": T, "H": H, "token_heads": B * T * H}
    for policy in (("saved", "recompute") if op in ("kda", "gdn2") else ("recompute",)):
        saved = policy == "saved"
        for _ in range(warmup):
            call(saved)
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(steps):
            call(saved)
        t1.record()
        torch.cuda.synchronize()
        ms = t0.elapsed_time(t1) / steps
        out[policy] = {"ms": ms, "tokens_per_s": B * T / (ms * 1e-3), "token_heads_per_s": B * T * H / (ms * 1e-3)}
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--token-heads", type=int, default=2097152)
    ap.add_argument("--cases", default="cfg1_gdn,cfg3_delta,cfg4_gdn2,cfg2_kda")
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("family_timing needs a CUDA device: there is no CPU path")
    for name in args.cases.split(","):
        print(json.dumps(_case(name, args.steps, args.warmup, args.token_heads)), flush=True)
        torch.cuda.empty_cache()


if __name__ == "__main__":
    main()
