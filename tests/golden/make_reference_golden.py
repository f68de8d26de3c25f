"""Runs the parts of the reference that compile on a machine without Apple's MLX and records what they answer.

Two pieces of muyouming/exl3-server need no MLX: the sampler (``sample_token`` with its generator,
src/model.cpp:656-757, options in src/model.h:191-200) and the safetensors reader (src/safetensors.cpp with
src/fp16.h).  This script compiles both from the reference's own files with ``g++`` (the sampler by cutting its
lines out of src/model.cpp into a scratch file; nothing of the reference is kept in this repository), feeds them
the cases below and writes their answers to ``reference_golden.json`` beside this file.  The tests compare the
library's host sampler and container reader with that file; where the reference and ``g++`` are present they
also run this script again and compare its output with the committed file.

The reference's forward pass (src/model.cpp:514-628) cannot be built here, so the plain implementation under
``tests/`` rests on the formulas; this file anchors only what it says.

    python tests/golden/make_reference_golden.py [--reference DIR] [--out FILE]
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import shutil
import struct
import subprocess
import sys
import tempfile
from typing import Dict, List

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
# where a checkout of muyouming/exl3-server lies: the environment says, else a sibling folder of this repository
DEFAULT_REFERENCE = os.environ.get("EXL3_REFERENCE_DIR") or os.path.normpath(os.path.join(HERE, "..", "..", "..", "reference"))
MASK = (1 << 64) - 1


# -- inputs that depend on nothing but integer arithmetic ----------------------------------------------------

def golden_logits(seed: int, n: int, spread: float = 4.0) -> np.ndarray:
    """n float32 logits, all different: an evenly spaced grid over (-spread, spread) in an order given by a
    64-bit mixing function of (seed, index).  The same numbers on every machine and library version (the
    reference leaves the order of equal logits open, so there are none)."""
    z = (np.arange(1, n + 1, dtype=np.uint64) * np.uint64(0x9E3779B97F4A7C15) + np.uint64(seed & MASK))
    z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    z = z ^ (z >> np.uint64(31))
    order = np.argsort(z, kind="stable")
    grid = ((np.arange(n, dtype=np.float64) + 0.5) / n * 2.0 - 1.0) * spread
    out = np.empty(n, dtype=np.float32)
    out[order] = grid.astype(np.float32)
    return out


# temperature, top_p, top_k, min_p, repetition, presence, frequency, seed, vocabulary, draws, context
SAMPLER_CASES: List[dict] = [
    dict(temperature=0.0, top_p=1.0, top_k=0, min_p=0.0, rep=1.0, pres=0.0, freq=0.0, seed=1, n=300, draws=12, context=[]),
    dict(temperature=0.0, top_p=1.0, top_k=0, min_p=0.0, rep=1.3, pres=0.2, freq=0.1, seed=2, n=300, draws=24, context=[5, 5, 9]),
    dict(temperature=1.0, top_p=1.0, top_k=0, min_p=0.0, rep=1.0, pres=0.0, freq=0.0, seed=3, n=97, draws=40, context=[]),
    dict(temperature=0.7, top_p=0.9, top_k=0, min_p=0.0, rep=1.0, pres=0.0, freq=0.0, seed=4, n=1000, draws=40, context=[]),
    dict(temperature=1.3, top_p=1.0, top_k=40, min_p=0.0, rep=1.0, pres=0.0, freq=0.0, seed=5, n=1000, draws=40, context=[]),
    dict(temperature=0.9, top_p=1.0, top_k=0, min_p=0.05, rep=1.0, pres=0.0, freq=0.0, seed=6, n=1000, draws=40, context=[]),
    dict(temperature=0.8, top_p=0.95, top_k=50, min_p=0.02, rep=1.15, pres=0.3, freq=0.05, seed=7, n=2049, draws=60,
         context=[1, 2, 3, 3, 3, 2000]),
    # more tokens than the 2,048 candidates the reference keeps; top_k above that raises the cap
    dict(temperature=1.5, top_p=1.0, top_k=0, min_p=0.0, rep=1.0, pres=0.0, freq=0.0, seed=8, n=5000, draws=60, context=[]),
    dict(temperature=2.0, top_p=0.999, top_k=3000, min_p=0.0, rep=1.0, pres=0.0, freq=0.0, seed=9, n=5000, draws=60, context=[]),
    dict(temperature=0.5, top_p=0.5, top_k=2, min_p=0.5, rep=2.0, pres=1.0, freq=0.5, seed=0x9E3779B97F4A7C15, n=64,
         draws=40, context=[0, 1, 2, 3, 63, 64, -1]),
]

SAMPLER_DRIVER = r"""
// Reads cases from stdin, prints the tokens the reference's sample_token picks.  Each case: a line of options,
// a line with the context, then one line of logits (as the bits of float32) per draw.  A drawn token joins the
// context and the generator's state carries over, as in a generation loop (src/engine.cpp:341-353).
int main() {
  int ncases = 0;
  if (scanf("%d", &ncases) != 1) return 2;
  for (int c = 0; c < ncases; ++c) {
    exl3::SampleOptions opt;
    unsigned long long seed = 0;
    int n = 0, draws = 0, nctx = 0;
    if (scanf("%f %f %d %f %f %f %f %llu %d %d %d", &opt.temperature, &opt.top_p, &opt.top_k, &opt.min_p,
              &opt.repetition_penalty, &opt.presence_penalty, &opt.frequency_penalty, &seed, &n, &draws, &nctx) != 11)
      return 3;
    std::vector<int> context((size_t)nctx);
    for (int i = 0; i < nctx; ++i) if (scanf("%d", &context[(size_t)i]) != 1) return 4;
    uint64_t state = (uint64_t)seed;
    for (int d = 0; d < draws; ++d) {
      std::vector<float> logits((size_t)n);
      for (int i = 0; i < n; ++i) {
        unsigned bits = 0;
        if (scanf("%x", &bits) != 1) return 5;
        memcpy(&logits[(size_t)i], &bits, 4);
      }
      const int tok = exl3::sample_token(logits, opt, context, state);
      context.push_back(tok);
      printf(d + 1 < draws ? "%d " : "%d\n", tok);
    }
  }
  return 0;
}
"""

SAMPLER_PRELUDE = r"""
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <unordered_map>
#include <vector>
namespace exl3 {
"""

READER_DRIVER = r"""
// Prints what the reference's reader finds in a safetensors file: per tensor its dtype, shape, byte count and
// the first and last 16-bit or 32-bit word of its data; then the error of a typed access with the wrong type.
#include "safetensors.h"
#include <cstdio>
#include <cstring>
int main(int argc, char** argv) {
  exl3::SafetensorsFile f;
  std::string err;
  if (!exl3::SafetensorsFile::load(argv[1], f, err)) { printf("load failed: %s\n", err.c_str()); return 1; }
  for (const auto& kv : f.tensors) {
    const exl3::STTensor& t = kv.second;
    printf("%s %s [", kv.first.c_str(), exl3::dtype_name(t.dtype));
    for (size_t i = 0; i < t.shape.size(); ++i) printf(i ? ",%lld" : "%lld", (long long)t.shape[i]);
    const uint8_t* p = f.data(kv.first, err);
    const int w = (t.dtype == exl3::DT::I32 || t.dtype == exl3::DT::F32) ? 4 : 2;
    unsigned first = 0, last = 0;
    memcpy(&first, p, w);
    memcpy(&last, p + t.nbytes - w, w);
    printf("] %lld %u %u\n", (long long)t.nbytes, first, last);
  }
  std::string e2;
  const uint16_t* wrong = f.f16_data("c.float32", e2);
  printf("wrong-type access: %s\n", wrong == nullptr && !e2.empty() ? "refused" : "allowed");
  return 0;
}
"""


def container_tensors() -> Dict[str, "np.ndarray"]:
    """The tensors of the container case: every element type the reference's reader knows, odd shapes, a scalar
    shape of one element.  Values come from golden_logits, cut to each type."""
    import torch
    a = torch.from_numpy(golden_logits(11, 3 * 5)).reshape(3, 5)
    return {
        "a.bfloat16": a.to(torch.bfloat16),
        "b.float16": torch.from_numpy(golden_logits(12, 7)).to(torch.float16),
        "c.float32": torch.from_numpy(golden_logits(13, 2 * 3 * 4)).reshape(2, 3, 4),
        "d.int32": torch.arange(-3, 8, dtype=torch.int32),
        "e.int16": torch.arange(-2, 4, dtype=torch.int16).reshape(2, 3),
        "f.one": torch.from_numpy(golden_logits(14, 1)).to(torch.bfloat16),
    }


def cut_sampler_source(reference: str) -> str:
    """The options struct and the sampler, cut out of the reference's files by their first and last lines."""
    with open(os.path.join(reference, "src", "model.h")) as f:
        h = f.read()
    a = h.index("struct SampleOptions {")
    b = h.index("};", a) + 2
    with open(os.path.join(reference, "src", "model.cpp")) as f:
        cpp = f.read()
    c = cpp.index("static inline uint64_t splitmix64")
    d = cpp.index("} // namespace exl3", c)
    return SAMPLER_PRELUDE + h[a:b] + "\n" + cpp[c:d] + "\n}  // namespace exl3\n" + SAMPLER_DRIVER


def sampler_input() -> str:
    lines = [str(len(SAMPLER_CASES))]
    for case in SAMPLER_CASES:
        lines.append("%r %r %d %r %r %r %r %d %d %d %d" % (
            case["temperature"], case["top_p"], case["top_k"], case["min_p"], case["rep"], case["pres"], case["freq"],
            case["seed"], case["n"], case["draws"], len(case["context"])))
        lines.append(" ".join(str(t) for t in case["context"]))
        for d in range(case["draws"]):
            logits = golden_logits(case["seed"] * 1000 + d, case["n"])
            if np.unique(logits).size != logits.size:
                raise SystemExit("two equal logits in a case: the reference leaves their order open")
            lines.append(" ".join("%x" % b for b in logits.view(np.uint32)))
    return "\n".join(lines) + "\n"


def make(reference: str) -> dict:
    gxx = shutil.which("g++")
    if gxx is None:
        raise SystemExit("g++ not found")
    out: dict = {"made_from": "muyouming/exl3-server src/model.cpp (sample_token), src/model.h (SampleOptions), "
                              "src/safetensors.cpp, src/fp16.h; compiled with g++ -std=c++20 -O1"}
    with tempfile.TemporaryDirectory() as tmp:
        # the sampler
        src = os.path.join(tmp, "sampler.cpp")
        with open(src, "w") as f:
            f.write(cut_sampler_source(reference))
        exe = os.path.join(tmp, "sampler")
        subprocess.run([gxx, "-std=c++20", "-O1", "-o", exe, src], check=True)
        r = subprocess.run([exe], input=sampler_input(), capture_output=True, text=True, check=True)
        rows = [[int(t) for t in line.split()] for line in r.stdout.strip().splitlines()]
        assert len(rows) == len(SAMPLER_CASES)
        out["sampler"] = [{"case": i, "tokens": " ".join(str(t) for t in row)} for i, row in enumerate(rows)]
        # the container reader, on a file this library's writer wrote
        sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
        from exl3_server_b200.weights import write_safetensors
        path = os.path.join(tmp, "model.safetensors")
        write_safetensors(path, container_tensors().items(), metadata={"format": "pt"})
        with open(path, "rb") as f:
            out["container_sha256"] = hashlib.sha256(f.read()).hexdigest()
        drv = os.path.join(tmp, "reader.cpp")
        with open(drv, "w") as f:
            f.write(READER_DRIVER)
        exe = os.path.join(tmp, "reader")
        inc = ["-I", os.path.join(reference, "src"), "-I", os.path.join(reference, "vendor")]
        subprocess.run([gxx, "-std=c++20", "-O1", *inc, "-o", exe, drv,
                        os.path.join(reference, "src", "safetensors.cpp")], check=True)
        r = subprocess.run([exe, path], capture_output=True, text=True, check=True)
        out["container"] = r.stdout.strip().splitlines()
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=DEFAULT_REFERENCE)
    ap.add_argument("--out", default=os.path.join(HERE, "reference_golden.json"))
    args = ap.parse_args()
    with open(args.out, "w") as f:
        json.dump(make(args.reference), f, indent=1)
        f.write("\n")
    print(f"wrote {args.out}")


if __name__ == "__main__":
    main()
