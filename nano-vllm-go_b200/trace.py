"""Trace replay: feed given token ids through a model step by step and write logits.

Reads one JSON object per line from standard input,

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

runs every step's entries as ONE ragged batch through the runner's step function (prompt
portions beside single decoded tokens; nvllm_run computes tokens [num_cached, len) of every
sequence), writes the logits at the wanted places of a step to <out>/<step>.f32
(little-endian fp32, [wanted, vocab]) and prints "done <step>".  Nothing is sampled.  Cache
blocks come from the engine's block manager and go back to it when a request ends, so a pool
sized for the live requests is used again and again; models with recurrent mixers also get one
of MAX_LIVE state slots per live request from it.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np

from . import config as C
from . import runner as R


MAX_LIVE = 4  # requests that are live at any time


def replay(model_dir: str, dtype: str, out_dir: str, max_tokens: int, lines, echo=print) -> int:
    from harness import go_engine as G

    block = C.KV_BLOCK_SIZE
    # up to MAX_LIVE live requests, each may leave one block partly used
    num_blocks = (max_tokens + block - 1) // block + MAX_LIVE
    prec = C.PREC_BF16 if dtype == "bfloat16" else C.PREC_FP32
    run = R.CudaModelRunner.from_dir(model_dir, precision=prec, num_kv_blocks=num_blocks, sampling=None,
                                     num_state_slots=MAX_LIVE)
    bm = G.BlockManager(num_blocks, block, MAX_LIVE if run.needs_state_slots else 0)
    live, done = {}, {}
    os.makedirs(out_dir, exist_ok=True)
    try:
        for line in lines:
            line = line.strip()
            if not line:
                continue
            step = json.loads(line)
            seqs, cached, rows, row0 = [], [], [], 0
            for e in step.get("entries", []):
                toks = [int(t) for t in e["tokens"]]
                if not toks:
                    continue
                seq = live.get(e["id"])
                if seq is None:
                    seq = live[e["id"]] = G.Sequence(toks, temperature=0.0)
                    done[e["id"]] = 0
                else:
                    for t in toks:
                        seq.append_token(t)
                bm.reserve(seq, len(seq))
                seqs.append(seq)
                cached.append(done[e["id"]])
                rows += [row0 + int(w) for w in e.get("want", [])]
                row0 += len(toks)
                done[e["id"]] = len(seq)
            if seqs:
                run.request_logits(rows)
                # a step of single continuing tokens is a decode step, as the engine issues it
                # (key splits, replayed graph); anything else is a ragged prefill step
                decode = all(len(s) - c == 1 and c > 0 for s, c in zip(seqs, cached))
                run.run_flat([s.token_ids for s in seqs], not decode, num_cached=cached,
                             block_tables=[s.block_table for s in seqs], temperature=[0.0] * len(seqs),
                             state_slots=[s.state_slot for s in seqs] if run.needs_state_slots else None)
                if rows:
                    logits = run.fetch_logits(len(rows))
                    tmp = os.path.join(out_dir, ".%d.tmp" % step["step"])
                    logits.astype("<f4").tofile(tmp)
                    os.replace(tmp, os.path.join(out_dir, "%d.f32" % step["step"]))
            for i in step.get("end", []):
                seq = live.pop(i, None)
                if seq is not None:
                    bm.deallocate(seq)
                    done.pop(i, None)
            echo("done %d" % step["step"])
    finally:
        run.close()
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    ap.add_argument("--out", required=True, help="folder the <step>.f32 files go to")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens the live requests hold at any time")
    a = ap.parse_args(argv)
    return replay(a.model, a.dtype, a.out, a.max_tokens, sys.stdin,
                  echo=lambda s: (sys.stdout.write(s + "\n"), sys.stdout.flush()))
