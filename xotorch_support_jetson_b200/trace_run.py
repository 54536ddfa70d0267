"""Replays a trace of token ids through a model, step by step, and writes the logits that the trace asks for.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Standard input carries one JSON object per line::

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": ["a"]}

``entries``: per request its next tokens and the places among them whose logits are wanted; ``end``: requests that are
finished after the step (their slot -- KV pages, recurrent state -- goes back to the engine).  For a step that wants
something, ``<out>/<step>.f32`` receives little-endian fp32 ``[wanted, vocab]`` in the order of the entries; after every
step the line ``done <step>`` is printed.  Nothing is sampled.

The steps run on the serving path: ``StageRuntime.forward`` on the native engine (slot manager, paged KV, state,
CUDA-graph decode steps), the model class chosen by ``config.json`` like ``B200ShardInferenceEngine.ensure_shard``
does.  A step with more tokens than one native call carries is cut into position chunks, as the engine's chunked
prefill does.  Exit code 3: the model's family has no float32 mode.
"""
import argparse
import json
import os
import sys
from pathlib import Path


def main(argv=None) -> int:
  ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
  ap.add_argument("--model", required=True, help="folder with config.json and *.safetensors")
  ap.add_argument("--dtype", default="bfloat16", choices=("bfloat16", "float32"))
  ap.add_argument("--out", required=True, help="folder for <step>.f32")
  ap.add_argument("--max-tokens", type=int, default=4096, help="most tokens that live requests hold at any time")
  ap.add_argument("--max-requests", type=int, default=8, help="most requests alive at a time")
  ap.add_argument("--chunk", type=int, default=2048, help="most token rows per native call")
  ap.add_argument("--device", type=int, default=int(os.environ.get("XB_DEVICE", "0")))
  a = ap.parse_args(argv)

  from .model_config import is_hybrid, load_model_config
  cfg = load_model_config(Path(a.model) / "config.json")
  if a.dtype == "float32" and not is_hybrid(cfg):
    print("trace_run: this model family runs in bfloat16 only", file=sys.stderr)
    return 3

  from .build import ensure_built
  ensure_built(quiet=True)
  import numpy as np
  import torch
  from .shard import Shard
  from .stage import StageRuntime

  nl = cfg["num_layers"]
  chunk = max(1, min(a.chunk, max(a.max_tokens, 1)))
  kw = dict(device=a.device, max_batch_tokens=chunk, max_seqs=a.max_requests, max_tokens_per_seq=max(a.max_tokens, 8),
            page_tokens=64)
  if is_hybrid(cfg):
    kw.update(dtype=a.dtype, max_logit_rows=chunk)
  st = StageRuntime(Shard(Path(a.model).name or "model", 0, nl - 1, nl), cfg, **kw)
  st.load_dir(Path(a.model))
  os.makedirs(a.out, exist_ok=True)
  stream = torch.cuda.Stream(device=st.device)   # a non-default stream: decode steps replay CUDA graphs
  free = list(range(a.max_requests - 1, -1, -1))
  slot_of, length = {}, {}
  with torch.cuda.stream(stream):
    for line in sys.stdin:
      line = line.strip()
      if not line:
        continue
      step = json.loads(line)
      parts = []
      for en in step.get("entries", []):
        rid, toks, asked = en["id"], [int(t) for t in en["tokens"]], [int(w) for w in en.get("want", [])]
        want = sorted(asked)
        if rid not in slot_of:
          if not free:
            raise RuntimeError(f"more than {a.max_requests} requests alive (--max-requests)")
          slot_of[rid], length[rid] = free.pop(), 0
        slot = slot_of[rid]
        got = []
        for c0 in range(0, len(toks), chunk):
          c1 = min(len(toks), c0 + chunk)
          rows = [w - c0 for w in want if c0 <= w < c1]
          ids = torch.tensor(toks[c0:c1], dtype=torch.int32).to(st.device, non_blocking=False)
          pos = length[rid] + c0
          if not st.hybrid:
            if rows and rows != [c1 - c0 - 1]:
              raise RuntimeError("this model family returns the logits of a portion's last token only")
            out = st.forward([slot], [c1 - c0], [pos], tokens=ids)
            out = out if rows else None
          elif rows == [c1 - c0 - 1]:
            out = st.forward([slot], [c1 - c0], [pos], tokens=ids)          # the serving call: last row of the sequence
          else:
            out = st.forward([slot], [c1 - c0], [pos], tokens=ids, want_rows=rows)
          if out is not None:
            got.append(out)
        length[rid] += len(toks)
        if got:
          rows_sorted = torch.cat(got, dim=0)     # in rising position; back to the order that was asked
          parts.append(rows_sorted[[want.index(w) for w in asked]] if asked != want else rows_sorted)
      if parts:
        logits = torch.cat(parts, dim=0).to(torch.float32).cpu().numpy().astype("<f4")
        tmp = os.path.join(a.out, f".{step['step']}.part")
        with open(tmp, "wb") as f:
          f.write(np.ascontiguousarray(logits).tobytes())
        os.replace(tmp, os.path.join(a.out, f"{step['step']}.f32"))
      else:
        stream.synchronize()
      for rid in step.get("end", []):
        if rid in slot_of:
          st.release_slot(slot_of[rid])
          free.append(slot_of.pop(rid))
          length.pop(rid, None)
      sys.stdout.write(f"done {step['step']}\n")
      sys.stdout.flush()
  st.close()
  return 0


if __name__ == "__main__":
  sys.exit(main())
