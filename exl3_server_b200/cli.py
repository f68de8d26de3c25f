"""Command line in the manner of ``exl3-server --model DIR [mode] [options]``
(src/main.cpp:21-70, 98-171).

Flags keep the reference's spelling and meaning where the feature exists here:
``--model``, ``-p/--prompt`` (repeatable), ``--max-tokens``, ``--temp``,
``--top-p``, ``--top-k``, ``--min-p``, ``--repetition-penalty``,
``--presence-penalty``, ``--frequency-penalty``, ``--seed``, ``--ignore-eos``,
``--batch``, ``--quiet``; every value flag takes ``--k v`` and ``--k=v``; an
unknown flag exits with 2.  There is no tokenizer in this library, so a prompt
is a list of token ids (``-p "1,15,27"`` or ``--prompt-file`` with one list per
line) and the output is token ids, one line per request, followed by the
reference's statistics line on standard error (src/cli.cpp:15-19).  The chat,
server and draft flags have no counterpart and are refused as unknown.
"""
from __future__ import annotations

import argparse
import signal
import sys
from typing import List

from .sampling.options import DEFAULT_SEED, SampleOptions


def parse_ids(text: str) -> List[int]:
    parts = [p for p in text.replace(",", " ").split() if p]
    try:
        return [int(p) for p in parts]
    except ValueError:
        raise argparse.ArgumentTypeError(f"a prompt is a list of token ids, got {text!r}")


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(
        prog="exl3-server-b200", allow_abbrev=False,
        description="Llama-family generation on one B200: token ids in, token ids out")
    ap.add_argument("--model", required=True, metavar="DIR", help="folder with config.json and model.safetensors")
    ap.add_argument("-p", "--prompt", action="append", type=parse_ids, default=[], metavar="IDS",
                    help="prompt as token ids, e.g. \"1,15,27\" (repeatable; prompts run as a batch)")
    ap.add_argument("--prompt-file", metavar="FILE", help="one prompt (token ids) per line")
    g = ap.add_argument_group("sampling")
    g.add_argument("--max-tokens", type=int, default=512, metavar="N", help="maximum tokens to generate (default 512)")
    g.add_argument("--temp", type=float, default=0.0, metavar="F", help="temperature, 0 = greedy (default 0)")
    g.add_argument("--top-p", type=float, default=1.0, metavar="F", help="nucleus sampling (default 1.0)")
    g.add_argument("--top-k", type=int, default=0, metavar="N", help="top-k sampling (default 0 = off)")
    g.add_argument("--min-p", type=float, default=0.0, metavar="F", help="min-p sampling (default 0)")
    g.add_argument("--repetition-penalty", type=float, default=1.0, metavar="F", help="(default 1.0)")
    g.add_argument("--presence-penalty", type=float, default=0.0, metavar="F", help="(default 0)")
    g.add_argument("--frequency-penalty", type=float, default=0.0, metavar="F", help="(default 0)")
    g.add_argument("--seed", type=int, default=DEFAULT_SEED, metavar="N", help="RNG seed")
    g.add_argument("--stop-id", action="append", type=int, default=None, metavar="N",
                   help="stop token id, repeatable (default: the model's eos_token_id)")
    g.add_argument("--ignore-eos", action="store_true", help="do not stop on EOS")
    o = ap.add_argument_group("other")
    o.add_argument("--batch", type=int, default=64, metavar="N", help="most prompts that run as one batch (default 64)")
    o.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16", help="(default bfloat16)")
    o.add_argument("--cache-tokens", type=int, default=0, metavar="N",
                   help="tokens the cache holds (default: enough for one batch)")
    o.add_argument("--device", default="cuda:0")
    o.add_argument("--quiet", action="store_true", help="no per-request stats")
    return ap


def print_stats(r, file=sys.stderr) -> None:
    """The reference's line (src/cli.cpp:15-19)."""
    tps = r.completion_tokens / r.decode_seconds if r.decode_seconds > 0 else 0.0
    print(f"[{r.prompt_tokens} prompt + {r.completion_tokens} generated tokens | prefill "
          f"{r.prefill_seconds:.2f}s | {tps:.1f} tok/s | {r.finish_reason}]", file=file)


def main(argv=None) -> int:
    ap = build_parser()
    args = ap.parse_args(argv)                        # unknown option or missing --model: exit code 2
    prompts: List[List[int]] = list(args.prompt)
    if args.prompt_file:
        with open(args.prompt_file) as f:
            prompts += [parse_ids(line) for line in f if line.strip()]
    if not prompts:
        ap.error("no prompt given (-p IDS or --prompt-file FILE)")

    from .engine import Engine, GenerateOptions
    need = sum((len(p) + args.max_tokens + 63) // 64 * 64 for p in prompts[:max(1, args.batch)])
    try:
        engine = Engine.from_folder(args.model, dtype=args.dtype, max_tokens=args.cache_tokens or need,
                                    device=args.device)
    except Exception as e:                            # config, weights or kernel library
        print(f"exl3-server-b200: {e}", file=sys.stderr)
        return 1
    interrupted = {"flag": False}
    signal.signal(signal.SIGINT, lambda *_: interrupted.__setitem__("flag", True))   # src/main.cpp:17-19
    opt = GenerateOptions(
        sample=SampleOptions(temperature=args.temp, top_p=args.top_p, top_k=args.top_k, min_p=args.min_p,
                             repetition_penalty=args.repetition_penalty, presence_penalty=args.presence_penalty,
                             frequency_penalty=args.frequency_penalty, seed=args.seed),
        max_tokens=args.max_tokens, ignore_eos=args.ignore_eos, stop_token_ids=args.stop_id,
        max_batch=args.batch)
    results = engine.generate(prompts, opt, cancelled=lambda: interrupted["flag"])
    for r in results:
        print(",".join(str(t) for t in r.tokens), flush=True)
        if not args.quiet:
            print_stats(r)
    return 0


if __name__ == "__main__":
    sys.exit(main())
