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
over its time, ``points`` decode at batch 1 and 64 and, unless ``--no-points``,
the other measurements the baseline names: the 2B sizes at contexts of 128 and
2,048 tokens, the 8B-class MiniCPM4 sizes (32 query heads on 2 key/value heads
of 128; decode at batch 1, 8, 64 and a 2,048-token prefill) and the 0.5B-class
MiniCPM4 sizes (64 prompts of 16 to 2,048 tokens in one prefill step, then 256
decode steps); ``points_frac`` gives each point's fraction of its roofline
(HBM bytes for decode, bfloat16 flops for prefill).  Every repeat of a point is
printed to stderr as it is measured; a point's value is its best repeat.
Peaks come from MEASURED_PEAKS.json when it exists, else from the stated
fallback.

``--only decode|prefill|unequal`` with ``--sizes NAME`` runs one part at any of
the size tables and prints a short JSON line (for profiling small cases).

Only one GPU is supported: for N > 1 it says so and exits with 2.
"""
from __future__ import annotations

import argparse
import gc
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
HEADLINE = "minicpm-2b"          # BASELINE.json configs[2]


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


def say(msg: str) -> None:
    print(f"[bench] {msg}", file=sys.stderr, flush=True)


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


class Rig:
    """A random-weight model of one of the size tables with a cache, and the timed pieces."""

    def __init__(self, sizes_name: str, layers: int, cache_tokens: int, max_slots: int):
        import torch
        import exl3_server_b200 as E
        from exl3_server_b200.config.presets import SIZES, sizes
        from exl3_server_b200.engine.model import Model, plan_manifest
        from exl3_server_b200.models.llama import build_plan
        from exl3_server_b200.weights.random_init import random_tensors
        self.torch, self.E = torch, E
        self.name = sizes_name
        self.layers_full = SIZES[sizes_name]["num_hidden_layers"]
        self.layers = min(layers, self.layers_full) if layers > 0 else self.layers_full
        # the residual scale belongs to the full model whatever the number of layers run
        self.cfg = E.LlamaConfig(**sizes(sizes_name, num_hidden_layers=self.layers))
        dev = torch.device("cuda:0")
        t0 = time.time()
        plan = build_plan(self.cfg)
        tensors = dict(random_tensors(plan_manifest(plan), seed=0, std=0.02, norm_std=None, dtype=torch.bfloat16,
                                      device=dev))
        self.model = Model(plan, tensors, torch.bfloat16, dev)
        del tensors
        self.engine = E.Engine(self.model, max_tokens=cache_tokens, max_slots=max_slots)
        self.gen = torch.Generator().manual_seed(1)
        say(f"{sizes_name}: {self.layers} of {self.layers_full} layers, cache of {cache_tokens} tokens, ready in "
            f"{time.time() - t0:.1f}s")

    def close(self):
        self.engine = self.model = None
        gc.collect()
        self.torch.cuda.empty_cache()

    def prompts(self, n, length):
        return [self.torch.randint(0, self.cfg.vocab_size, (length,), generator=self.gen).tolist() for _ in range(n)]

    def kv_bytes_per_token(self):
        return sum(g.bytes_per_token(2) for g in self.engine.cache.groups)

    def prefill_flops(self, lengths):
        """Matrix products of every layer for all tokens, causal attention, the head on one row per prompt."""
        c = self.cfg
        lin = sum(b.mixer.qkv.weight.numel() + b.mixer.o.weight.numel() + b.feed_forward.gate_up.weight.numel()
                  + b.feed_forward.down.weight.numel() for b in self.model.blocks)
        att = sum(2.0 * c.num_attention_heads * c.head_dim * n * n for n in lengths) * self.layers
        return 2.0 * sum(lengths) * lin + att + 2.0 * c.vocab_size * c.hidden_size * len(lengths)

    def fill(self, slots, toks, chunk=8192):
        """Real prefill through the step function, in steps of about ``chunk`` tokens."""
        E = self.E
        per = max(1, chunk // len(slots))
        for a in range(0, len(toks[0]), per):
            self.engine.step([E.StepEntry(s, t[a:a + per], None) for s, t in zip(slots, toks)])

    def decode(self, batch, ctx, steps, warmup):
        """Device time of ``steps`` decode steps that end at ``ctx`` tokens of context: (ms, launches, cache bytes
        read per step)."""
        from exl3_server_b200.engine.decode import DecodeSession
        from exl3_server_b200.ops import kernels as K
        torch, eng = self.torch, self.engine
        ctx0 = max(1, ctx - steps - warmup)
        slots = [eng.open() for _ in range(batch)]
        self.fill(slots, self.prompts(batch, ctx0))
        sess = DecodeSession(eng, slots, [1] * batch)
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
        kv = self.kv_bytes_per_token() * batch * (ctx0 + warmup + steps / 2.0)
        sess.close()
        for s in slots:
            eng.close(s)
        return ms, launches, kv

    def decode_point(self, name, batch, ctx, steps, warmup, hbm_gbs, repeats=2):
        """(tokens per second, fraction of the HBM roofline) of the best of ``repeats`` runs; each is printed."""
        best = None
        for r in range(repeats):
            ms, _, kv = self.decode(batch, ctx, steps, warmup)
            rate = batch * steps / (ms / 1e3)
            gbs = (self.model.weight_bytes() + kv) / (ms / steps / 1e3) / 1e9
            say(f"{name} repeat {r}: {ms / steps:.3f} ms/step, {rate:.0f} tok/s, {gbs:.0f} GB/s")
            if best is None or rate > best[0]:
                best = (rate, gbs / hbm_gbs)
        return best

    def prefill(self, tokens, repeats=4, warm=3):
        """Milliseconds of one step with one prompt of ``tokens`` tokens (best repeat; each is printed).  Every
        other timed step starts after a quarter of a second of idling: back to back the steps of the larger sizes
        run into the power cap and each is slower than the one before, after idling the clocks of the smaller
        sizes' short step have to come up again; the burst rate they are compared with was measured on a kernel
        in isolation."""
        torch, E, eng = self.torch, self.E, self.engine
        toks = self.prompts(1, tokens)[0]
        times = []
        for i in range(warm + repeats):
            s = eng.open()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            if i >= warm and (i - warm) % 2 == 1:
                time.sleep(0.25)
            e0.record()
            eng.step([E.StepEntry(s, toks, "last")])
            e1.record()
            torch.cuda.synchronize()
            eng.close(s)
            if i >= warm:
                times.append(e0.elapsed_time(e1))
                say(f"{self.name} prefill of {tokens} tokens, repeat {i - warm}: {times[-1]:.3f} ms")
        return min(times)

    def unequal(self, n_prompts, lo, hi, decode_steps, repeats=2):
        """``n_prompts`` prompts of ``lo`` to ``hi`` tokens (seeded) in ONE prefill step, then ``decode_steps``
        steps of all of them: (prefill tokens, prefill ms, decode ms per step, cache bytes per decode step)."""
        from exl3_server_b200.engine.decode import DecodeSession
        torch, E, eng = self.torch, self.E, self.engine
        lens = torch.randint(lo, hi + 1, (n_prompts,), generator=self.gen).tolist()
        toks = [self.prompts(1, n)[0] for n in lens]
        best_pf, best_dec = None, None
        for r in range(repeats + 1):
            slots = [eng.open() for _ in range(n_prompts)]
            e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
            torch.cuda.synchronize()
            e0.record()
            eng.step([E.StepEntry(s, t, "last") for s, t in zip(slots, toks)])
            e1.record()
            sess = DecodeSession(eng, slots, [1] * n_prompts, max_new=decode_steps + 8)
            for _ in range(3):
                sess.step()
            torch.cuda.synchronize()
            e1b = torch.cuda.Event(enable_timing=True)
            e1b.record()
            for _ in range(decode_steps):
                sess.step()
            e2.record()
            torch.cuda.synchronize()
            pf, dec = e0.elapsed_time(e1), e1b.elapsed_time(e2) / decode_steps
            sess.close()
            for s in slots:
                eng.close(s)
            if r == 0:
                continue                                    # records the graphs and warms the kernels
            say(f"{self.name} unequal batch of {n_prompts} ({sum(lens)} tokens), repeat {r - 1}: prefill {pf:.2f} ms, "
                f"decode {dec:.3f} ms/step")
            best_pf = pf if best_pf is None else min(best_pf, pf)
            best_dec = dec if best_dec is None else min(best_dec, dec)
        kv = self.kv_bytes_per_token() * (sum(lens) + n_prompts * (3 + decode_steps / 2.0))
        return lens, best_pf, best_dec, kv


def main() -> int:
    from exl3_server_b200.config.presets import SIZES
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers of the same sizes (stated in config); 0: all")
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--no-points", action="store_true", help="skip everything but the headline measurements")
    ap.add_argument("--sizes", choices=sorted(SIZES), default=HEADLINE,
                    help="layer sizes; other than the default only with --only (a short JSON line)")
    ap.add_argument("--only", choices=["all", "decode", "prefill", "unequal"], default="all",
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
    if args.sizes != HEADLINE and args.only == "all":
        print(f"bench.py: --sizes other than {HEADLINE} needs --only decode, prefill or unequal")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import torch
    torch.cuda.set_device(0)
    hbm_gbs, bf16_tf, peak_src = peaks()
    B, C, Kst, W = args.batch, args.context, args.steps, args.warmup
    page = 64

    def room(batch, ctx):
        return (batch + 1) * ((ctx + page - 1) // page * page + page)

    # ---- one part only -----------------------------------------------------------------------------------------
    if args.only == "decode":
        rig = Rig(args.sizes, args.layers, room(B, C), B + 1)
        ms, launches, kv = rig.decode(B, C, Kst, W)
        gbs = (rig.model.weight_bytes() + kv) / (ms / Kst / 1e3) / 1e9
        print(json.dumps({"only": "decode", "sizes": args.sizes, "batch": B, "context": C, "layers": rig.layers,
                          "ms_per_step": ms / Kst, "tok_s": B * Kst / (ms / 1e3), "gb_s": gbs,
                          "hbm_frac": gbs / hbm_gbs, "gpu_launches": int(launches)}))
        return 0
    if args.only == "prefill":
        rig = Rig(args.sizes, args.layers, room(1, args.prefill_tokens), 2)
        ms = rig.prefill(args.prefill_tokens, repeats=max(1, Kst // 16))
        tf = rig.prefill_flops([args.prefill_tokens]) / (ms / 1e3) / 1e12
        print(json.dumps({"only": "prefill", "sizes": args.sizes, "tokens": args.prefill_tokens, "layers": rig.layers,
                          "ms": ms, "tok_s": args.prefill_tokens / (ms / 1e3), "tflops": tf, "frac": tf / bf16_tf}))
        return 0
    if args.only == "unequal":
        rig = Rig(args.sizes, args.layers, room(64, 2048 + 256 + 16), 65)
        lens, pf, dec, kv = rig.unequal(64, 16, 2048, 256)
        tf = rig.prefill_flops(lens) / (pf / 1e3) / 1e12
        gbs = (rig.model.weight_bytes() + kv) / (dec / 1e3) / 1e9
        print(json.dumps({"only": "unequal", "sizes": args.sizes, "prompts": 64, "tokens": sum(lens),
                          "layers": rig.layers, "prefill_ms": pf, "prefill_tok_s": sum(lens) / (pf / 1e3),
                          "prefill_tflops": tf, "prefill_frac": tf / bf16_tf, "decode_ms_per_step": dec,
                          "decode_tok_s": 64 / (dec / 1e3), "decode_gb_s": gbs, "decode_hbm_frac": gbs / hbm_gbs}))
        return 0

    # ---- the headline: decode at the default batch and context -----------------------------------------------------
    big = B if args.no_points else max(B, 64)
    rig = Rig(HEADLINE, args.layers, room(big, C), big + 1)
    cfg, engine, model, E = rig.cfg, rig.engine, rig.model, rig.E
    clocks = ClockSampler()
    clocks.start()
    ms, launches, kv_bytes = rig.decode(B, C, Kst, W)
    clk = clocks.stop()
    ms_step = ms / Kst
    value = B * Kst / (ms / 1e3)
    step_bytes = model.weight_bytes() + kv_bytes
    achieved = step_bytes / (ms_step / 1e3) / 1e9

    # ---- end to end through Engine.generate --------------------------------------------------------------------
    n_new = Kst + W
    e2e_prompts = rig.prompts(B, C - n_new)
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

    # ---- prefill of one prompt ---------------------------------------------------------------------------------------
    T = args.prefill_tokens
    pf_ms = rig.prefill(T)
    flops = rig.prefill_flops([T])
    prefill_rec = {"value": T / (pf_ms / 1e3), "tokens": T, "ms": pf_ms,
                   "frac": flops / (pf_ms / 1e3) / (bf16_tf * 1e12), "tflops": flops / (pf_ms / 1e3) / 1e12}

    points, fracs = {}, {}

    def point(name, got):
        points[name], fracs[name] = got

    if not args.no_points:
        st = max(8, Kst // 2)
        point("decode_b1", rig.decode_point("2B b1 ctx %d" % C, 1, C, st, 3, hbm_gbs))
        point("decode_b64", rig.decode_point("2B b64 ctx %d" % C, 64, C, st, 3, hbm_gbs))
        # the other contexts the baseline's table names
        for b, c in ((1, 128), (8, 128), (1, 2048), (8, 2048), (64, 2048)):
            point(f"decode_b{b}_ctx{c}", rig.decode_point(f"2B b{b} ctx {c}", b, c, min(st, c - 16), 3, hbm_gbs))
        # longer contexts: a prompt of 8,192 tokens, and decoding at 16,384 tokens (the cache is then 0.9 of the bytes)
        if big * C >= 8 * 16384 + 8192:
            point("decode_b8_ctx16384", rig.decode_point("2B b8 ctx 16384", 8, 16384, 16, 3, hbm_gbs, repeats=1))
            ms_long = rig.prefill(8192, repeats=2, warm=1)
            point("prefill_8192", (8192 / (ms_long / 1e3),
                                   rig.prefill_flops([8192]) / (ms_long / 1e3) / 1e12 / bf16_tf))
    layers_run, layers_full = rig.layers, rig.layers_full
    del engine, model
    rig.close()

    if not args.no_points:
        # ---- MiniCPM4-8B sizes: 16 query heads per key/value head of 128, untied head ---------------------------
        r8 = Rig("minicpm4-8b", 0, room(64, 2048), 65)
        for b in (1, 8, 64):
            point(f"m4_8b_decode_b{b}_ctx2048", r8.decode_point(f"8B b{b} ctx 2048", b, 2048, 24, 3, hbm_gbs))
        point("m4_8b_decode_b1_ctx128", r8.decode_point("8B b1 ctx 128", 1, 128, 24, 3, hbm_gbs))
        ms8 = r8.prefill(2048)
        tf8 = r8.prefill_flops([2048]) / (ms8 / 1e3) / 1e12
        point("m4_8b_prefill_2048", (2048 / (ms8 / 1e3), tf8 / bf16_tf))
        r8.close()
        # ---- MiniCPM4-0.5B sizes: 64 prompts of 16 to 2,048 tokens in one step, then 256 decode steps ------------
        r05 = Rig("minicpm4-0.5b", 0, room(64, 2048 + 256 + 16), 65)
        lens, pf, dec, kv = r05.unequal(64, 16, 2048, 256)
        point("m4_05b_unequal64_prefill", (sum(lens) / (pf / 1e3),
                                           r05.prefill_flops(lens) / (pf / 1e3) / 1e12 / bf16_tf))
        point("m4_05b_unequal64_decode", (64 / (dec / 1e3),
                                          (r05.model.weight_bytes() + kv) / (dec / 1e3) / 1e9 / hbm_gbs))
        r05.close()

    out = {
        "metric": "decode tok/s (batch 8, context 4096, 2B-class MiniCPM, bf16)", "value": value, "unit": "tok/s",
        "n_gpus": 1, "steps": Kst, "warmup": W, "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random weights N(0,0.02), uniform random token ids, contexts prefilled by the engine",
        "config": {"model": "MiniCPM-2B layer sizes", "global_batch": B, "seq_len": C, "parallelism": "none",
                   "layers": layers_run, "layers_full": layers_full, "hidden": cfg.hidden_size,
                   "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
                   "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size, "tied_head": True,
                   "rope_theta": cfg.rope_theta, "rms_norm_eps": cfg.rms_norm_eps, "page_size": page,
                   "l2": "inputs exceed L2 (weights and cache read per step)", "peaks": peak_src},
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
        "points_frac": fracs,
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
