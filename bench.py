#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference]

The default run has the layer sizes of the 2B-class MiniCPM configuration (40
layers, width 2304, 36/36 heads of 64, feed-forward 5760, vocabulary 122753,
tied head) with random bfloat16 weights N(0, 0.02), a batch of 8 and a context
of 4096 tokens.  A "step" is one decode step of the whole batch.  It prints ONE
JSON line: ``value`` is decoded tokens per second timed on the device over K
steps (CUDA events), ``e2e`` the same through ``Engine.generate`` with host
token ids in and out every step, ``prefill`` one 2,048-token prompt,
``roofline`` the decode step's bytes (every weight once plus the live cache)
over its time, ``points`` decode at batch 1 and 64.  Peaks come from
MEASURED_PEAKS.json when it exists, else from the stated fallback.

Only one GPU is supported: for N > 1 it says so and exits with 2.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0

# BASELINE.json configs[2]
BENCH_MODEL = dict(hidden_size=2304, num_hidden_layers=40, num_attention_heads=36, num_key_value_heads=36,
                   head_dim=64, intermediate_size=5760, vocab_size=122753, tie_word_embeddings=True,
                   rope_theta=10000.0, rms_norm_eps=1e-5, scale_emb=12.0, scale_depth=1.4, dim_model_base=256,
                   max_position_embeddings=0, model_type="minicpm", architectures=["MiniCPMForCausalLM"])
FULL_LAYERS = 40
# Other layer sizes for looking at the kernels away from the headline configuration (--sizes); the default run and
# its JSON line are the MiniCPM-2B ones above.
OTHER_SIZES = {
    "llama-8b-like": (dict(hidden_size=4096, num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8,
                           head_dim=128, intermediate_size=14336, vocab_size=128256, tie_word_embeddings=False,
                           rope_theta=500000.0, rms_norm_eps=1e-5, max_position_embeddings=0), 32),
}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    hbm, tf, src = FALLBACK_HBM_GBS, FALLBACK_BF16_TFLOPS, "fallback"
    if os.path.exists(path):
        try:
            with open(path) as f:
                j = json.load(f)
            hbm = float(j.get("hbm_gbs", hbm))
            tf = float(j.get("bf16_tflops", tf))
            src = "measured"
        except (OSError, ValueError):
            pass
    return hbm, tf, src


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--layers", type=int, default=FULL_LAYERS, help="fewer layers of the same sizes (stated in config)")
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 and batch 64 decode points")
    ap.add_argument("--sizes", choices=["minicpm-2b"] + sorted(OTHER_SIZES), default="minicpm-2b",
                    help="layer sizes; other than the default only with --only (a short JSON line)")
    ap.add_argument("--only", choices=["all", "decode", "prefill"], default="all",
                    help="run one part only (for profiling small cases); prints a short JSON line")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a C++/CMake program on Apple's MLX and Metal; pip finds nothing to "
                          "install (no setup.py or pyproject.toml) and MLX does not exist for this machine"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.sizes != "minicpm-2b" and args.only == "all":
        print("bench.py: --sizes other than minicpm-2b needs --only decode or --only prefill")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import torch
    import exl3_server_b200 as E
    from exl3_server_b200.engine.decode import DecodeSession
    from exl3_server_b200.engine.model import Model, plan_manifest
    from exl3_server_b200.models.llama import build_plan
    from exl3_server_b200.ops import kernels as K
    from exl3_server_b200.weights.random_init import random_tensors

    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    hbm_gbs, bf16_tf, peak_src = peaks()

    if args.sizes != "minicpm-2b":
        sizes, full = OTHER_SIZES[args.sizes]
        cfg = E.LlamaConfig(**{**sizes, "num_hidden_layers": min(args.layers, full)})
        args.layers = cfg.num_hidden_layers
    else:
        cfg = E.LlamaConfig(**{**BENCH_MODEL, "num_hidden_layers": args.layers})
    # the residual scale belongs to the 40-layer model whatever --layers says
    plan = build_plan(cfg)
    t0 = time.time()
    tensors = dict(random_tensors(plan_manifest(plan), seed=0, std=0.02, norm_std=None, dtype=torch.bfloat16,
                                  device=dev))
    model = Model(plan, tensors, torch.bfloat16, dev)
    del tensors
    B, C, Kst, W = args.batch, args.context, args.steps, args.warmup
    big = 64 if (not args.no_points and args.only == "all") else B
    cache_tokens = (max(big, B) + 1) * ((C + 63) // 64 * 64 + 64)
    engine = E.Engine(model, max_tokens=cache_tokens)
    print(f"[bench] model and cache ready in {time.time() - t0:.1f}s", file=sys.stderr, flush=True)

    g = torch.Generator().manual_seed(1)

    def prompts(n, length):
        return [torch.randint(0, cfg.vocab_size, (length,), generator=g).tolist() for _ in range(n)]

    def prefill(slots, toks, chunk=8192):
        """Real prefill through the step function, in steps of about ``chunk`` tokens."""
        per = max(1, chunk // len(slots))
        n = len(toks[0])
        for a in range(0, n, per):
            engine.step([E.StepEntry(s, t[a:a + per], None) for s, t in zip(slots, toks)])

    def time_decode(batch, ctx, steps, warmup):
        """Device time of ``steps`` decode steps at about ``ctx`` tokens of context."""
        ctx0 = ctx - steps - warmup
        slots = [engine.open() for _ in range(batch)]
        prefill(slots, prompts(batch, ctx0))
        sess = DecodeSession(engine, slots, [1] * batch)
        for _ in range(warmup):
            sess.step()
        torch.cuda.synchronize()
        l0 = K.launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            sess.step()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        launches = sess.launches_per_step * steps if sess.launches_per_step else K.launch_count() - l0
        kv = sum(gr.bytes_per_token(2) for gr in engine.cache.groups) * batch * (ctx0 + warmup + steps / 2.0)
        sess.close()
        for s in slots:
            engine.close(s)
        return ms, launches, kv

    if args.only == "decode":
        ms, launches, _ = time_decode(B, C, Kst, W)
        print(json.dumps({"only": "decode", "sizes": args.sizes, "batch": B, "context": C, "layers": args.layers,
                          "ms_per_step": ms / Kst, "tok_s": B * Kst / (ms / 1e3), "gpu_launches": int(launches)}))
        return 0
    if args.only == "prefill":
        s = engine.open()
        toks = prompts(1, args.prefill_tokens)[0]
        for _ in range(W):
            engine.step([E.StepEntry(s, toks, "last")])
            engine.cache.truncate(s, 0)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(Kst):
            engine.step([E.StepEntry(s, toks, "last")])
            engine.cache.truncate(s, 0)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / Kst
        print(json.dumps({"only": "prefill", "sizes": args.sizes, "tokens": args.prefill_tokens, "layers": args.layers,
                          "ms": ms,
                          "tok_s": args.prefill_tokens / (ms / 1e3)}))
        return 0

    # ---- main: decode at the default batch and context ----------------------
    clocks = ClockSampler()
    clocks.start()
    ms, launches, kv_bytes = time_decode(B, C, Kst, W)
    clk = clocks.stop()
    ms_step = ms / Kst
    value = B * Kst / (ms / 1e3)
    step_bytes = model.weight_bytes() + kv_bytes
    achieved = step_bytes / (ms_step / 1e3) / 1e9

    # ---- end to end through Engine.generate ---------------------------------
    n_new = Kst + W
    e2e_prompts = prompts(B, C - n_new)
    e2e_opt = E.GenerateOptions(max_tokens=n_new, ignore_eos=True, max_batch=B)
    from exl3_server_b200.engine.decode import TRANSFERRED

    def timed_generate(opt):
        before = dict(TRANSFERRED)
        res = engine.generate(e2e_prompts, opt)
        steps = max(r.completion_tokens for r in res) - 1
        rate = sum(r.completion_tokens - 1 for r in res) / max(r.decode_seconds for r in res)
        return rate, (TRANSFERRED["h2d"] - before["h2d"]) / steps, (TRANSFERRED["d2h"] - before["d2h"]) / steps

    engine.generate(e2e_prompts, e2e_opt)               # untimed: records the decode graph this shape needs
    # default user path: greedy, the next step is launched before the host reads the last one's ids
    e2e, h2d, d2h = timed_generate(e2e_opt)
    # the same with the host feeding every step's token ids (what sampling with filters does)
    fed_opt = E.GenerateOptions(max_tokens=n_new, ignore_eos=True, max_batch=B, run_ahead=False)
    e2e_fed, h2d_fed, d2h_fed = timed_generate(fed_opt)

    # ---- prefill of one prompt ------------------------------------------------
    T = args.prefill_tokens
    ptoks = prompts(1, T)[0]
    times = []
    for i in range(3 + 3):
        s = engine.open()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        engine.step([E.StepEntry(s, ptoks, "last")])
        e1.record()
        torch.cuda.synchronize()
        engine.close(s)
        if i >= 3:
            times.append(e0.elapsed_time(e1))
    pf_ms = min(times)
    lin = sum(b.mixer.qkv.weight.numel() + b.mixer.o.weight.numel() + b.feed_forward.gate_up.weight.numel()
              + b.feed_forward.down.weight.numel() for b in model.blocks)
    flops = 2.0 * T * lin + args.layers * 2.0 * cfg.num_attention_heads * cfg.head_dim * T * T \
        + 2.0 * cfg.vocab_size * cfg.hidden_size
    prefill_rec = {"value": T / (pf_ms / 1e3), "tokens": T, "ms": pf_ms,
                   "frac": flops / (pf_ms / 1e3) / (bf16_tf * 1e12), "tflops": flops / (pf_ms / 1e3) / 1e12}

    points = {}
    if not args.no_points:
        for name, b in (("decode_b1", 1), ("decode_b64", 64)):
            st = max(8, Kst // 2)
            m, _, _ = time_decode(b, C, st, 3)
            points[name] = b * st / (m / 1e3)

    out = {
        "metric": "decode tok/s (batch 8, context 4096, 2B-class MiniCPM, bf16)", "value": value, "unit": "tok/s",
        "n_gpus": 1, "steps": Kst, "warmup": W, "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random weights N(0,0.02), uniform random token ids, contexts prefilled by the engine",
        "config": {"model": "MiniCPM-2B layer sizes", "global_batch": B, "seq_len": C, "parallelism": "none",
                   "layers": args.layers, "layers_full": FULL_LAYERS, "hidden": cfg.hidden_size,
                   "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
                   "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size, "tied_head": True,
                   "page_size": 64, "l2": "inputs exceed L2 (weights and cache read per step)",
                   "peaks": peak_src},
        "clocks": clk,
        "e2e": {"value": e2e, "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "host_fed": {"value": e2e_fed, "h2d_bytes_per_step": h2d_fed, "d2h_bytes_per_step": d2h_fed},
                "note": "decode tok/s inside Engine.generate after its prefill (prompts: host lists, one pinned "
                        "H2D copy); greedy ids feed the next step on the GPU and are read by the host every step"},
        "gpu_launches": int(launches),
        "prefill": prefill_rec,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_gbs, "unit": "GB/s",
                     "frac": achieved / hbm_gbs, "bytes_per_step": step_bytes},
        "points": points,
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
