"""The Refatar design on the native hybrid engine against the plain restatement in tests/refatar_oracle.py:
small configurations and random weights made here, every mechanism alone, cached decoding, portions, batches,
slot reuse, window / kept-first / page edges, long state, and greedy generation through the serving engine."""
import asyncio

import numpy as np
import pytest
import torch

import refatar_oracle as O

pytestmark = pytest.mark.gpu
TOL = {"float32": 2e-4, "bfloat16": 6e-2}


def delta(heads=4, kv=2, dim=32, vdim=48, conv=3):
  return "delta", {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv}


def pair(heads=4, kv=2, dim=32, vdim=48, window=12, keep=3, scale=None, r_heads=2, r_dim=32, r_vdim=64, ls=0.8, rs=1.3):
  return "parallel", {"left": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale or dim ** -0.5,
                               "mask": {"size": window, "keep_first": keep}},
                      "right": {"heads": r_heads, "dim": r_dim, "vdim": r_vdim}, "left_scale": ls, "right_scale": rs}


def config(layers, width=96, vocab=200, taps=3, side=8, softcap=20.0, eps=1e-5):
  from xotorch_support_jetson_b200.models import _refatar
  return _refatar(width, vocab, [(t, m, ff) for (t, m), ff in layers], taps=taps, side=side, softcap=softcap, eps=eps)


MIXED = config([(delta(), 160), (pair(), 160), (pair(heads=6, kv=6, dim=16, vdim=16, window=5, keep=0, r_heads=3, r_dim=24, r_vdim=40), 0),
                (delta(heads=2, kv=2, dim=64, vdim=40, conv=4), 128)])


def weights(cfg, seed=0):
  from xotorch_support_jetson_b200.synth import random_refatar_state
  return random_refatar_state(cfg, seed=seed)


def stage(cfg, w, dtype="float32", page=8, seqs=4, cap=512, per_seq=1024):
  from xotorch_support_jetson_b200.model_config import hybrid_model_config
  from xotorch_support_jetson_b200.shard import Shard
  from xotorch_support_jetson_b200.stage import StageRuntime
  c = hybrid_model_config(cfg)
  nl = c["num_layers"]
  st = StageRuntime(Shard("refatar-test", 0, nl - 1, nl), c, max_batch_tokens=cap, max_seqs=seqs, max_tokens_per_seq=per_seq,
                    page_tokens=page, dtype=dtype, max_logit_rows=cap)
  st.load_state(w)
  return st


def toks(n, vocab, seed=0):
  g = torch.Generator().manual_seed(seed)
  return torch.randint(0, vocab, (n,), generator=g).tolist()


def run(st, slot, ids, pos, rows=None):
  t = torch.tensor(ids, dtype=torch.int32, device="cuda")
  rows = list(range(len(ids))) if rows is None else rows
  out = st.forward([slot], [len(ids)], [pos], tokens=t, want_rows=rows)
  return None if out is None else out.cpu().double()


def rel(got, ref):
  return float((got - ref).pow(2).mean().sqrt() / ref.pow(2).mean().sqrt())


@pytest.fixture(scope="module")
def lib(built_lib):
  return built_lib


# ----------------------------------------------------------------------------- each mechanism alone, other sizes
ALONE = {
  "delta": config([(delta(), 0)], taps=0, side=0, softcap=0),
  "delta_one_kv_head_odd_dims": config([(delta(heads=3, kv=1, dim=24, vdim=20, conv=2), 0)], width=72, taps=0, side=0, softcap=0),
  "delta_wide_key": config([(delta(heads=2, kv=2, dim=160, vdim=8, conv=5), 0)], taps=0, side=0, softcap=0),
  "attention": config([(pair(rs=0.0), 0)], taps=0, side=0, softcap=0),
  "attention_window_one_no_kept": config([(pair(window=1, keep=0, rs=0.0, heads=2, kv=1, dim=40, vdim=24), 0)], taps=0, side=0, softcap=0),
  "attention_kept_beyond_window": config([(pair(window=3, keep=7, rs=0.0, scale=0.3), 0)], taps=0, side=0, softcap=0),
  "hgrn": config([(pair(ls=0.0), 0)], taps=0, side=0, softcap=0),
  "hgrn_odd": config([(pair(ls=0.0, r_heads=5, r_dim=20, r_vdim=12), 0)], width=50, vocab=77, taps=0, side=0, softcap=0),
  "input_filter": config([(delta(), 64)], taps=5, side=0, softcap=0),
  "input_filter_two_taps": config([(pair(), 64)], taps=2, side=0, softcap=0),
  "feed_forward": config([(delta(), 200)], taps=0, side=0, softcap=0),
  "token_side": config([(delta(), 0), (pair(), 0)], taps=0, side=12, softcap=0),
  "softcap": config([(delta(), 0)], taps=0, side=0, softcap=2.0),
  "mixed": MIXED,
}


@pytest.mark.parametrize("name", sorted(ALONE))
def test_mechanism_against_oracle(lib, name):
  cfg = ALONE[name]
  w = weights(cfg, seed=3)
  ids = toks(70, cfg["vocab"], seed=1)
  ref, layers = O.forward(cfg, w, ids, return_layers=True)
  for dtype in ("float32", "bfloat16"):
    st = stage(cfg, w, dtype)
    taps = [torch.zeros(len(ids), cfg["width"], device="cuda") for _ in cfg["layers"]]
    t = torch.tensor(ids, dtype=torch.int32, device="cuda")
    got = st.forward([1], [len(ids)], [0], tokens=t, want_rows=list(range(len(ids))), taps=taps).cpu().double()
    for i, l in enumerate(layers):
      assert rel(taps[i].cpu().double(), l) < TOL[dtype], (name, dtype, "layer", i)
    assert rel(got, ref) < TOL[dtype], (name, dtype)
    st.close()


# ----------------------------------------------------------------------------- cache and state
@pytest.fixture(scope="module")
def mixed(lib):
  w = weights(MIXED, seed=5)
  st = stage(MIXED, w, "float32")
  yield MIXED, w, st
  st.close()


def test_prefill_equals_token_by_token(mixed):
  cfg, w, st = mixed
  ids = toks(60, cfg["vocab"], seed=2)
  ref = O.forward(cfg, w, ids)
  whole = run(st, 0, ids, 0)
  st.release_slot(0)
  single = torch.cat([run(st, 0, [t], p) for p, t in enumerate(ids)])
  st.release_slot(0)
  assert rel(whole, ref) < TOL["float32"] and rel(single, ref) < TOL["float32"]
  assert rel(single, whole) < 5e-5


@pytest.mark.parametrize("cuts", [[2, 37, 2, 5, 1, 1, 30, 2], [1, 1, 1, 2, 3, 70], [40, 40], [3] * 26 + [2]])
def test_portions(mixed, cuts):
  cfg, w, st = mixed
  ids = toks(sum(cuts), cfg["vocab"], seed=4)
  ref = O.forward(cfg, w, ids)
  out, p = [], 0
  for c in cuts:
    out.append(run(st, 2, ids[p:p + c], p))
    p += c
  st.release_slot(2)
  assert rel(torch.cat(out), ref) < TOL["float32"]


def test_batch_of_unequal_requests_equals_each_alone(mixed):
  cfg, w, st = mixed
  a, b, c = toks(33, cfg["vocab"], 7), toks(9, cfg["vocab"], 8), toks(50, cfg["vocab"], 9)
  ra, rb, rc = (O.forward(cfg, w, x) for x in (a, b, c))
  # step 1: a's first 20 tokens and all of b together; step 2: a's next 13, ONE more token of b's kind of slot (decode row) and c's prompt
  t1 = torch.tensor(a[:20] + b, dtype=torch.int32, device="cuda")
  o1 = st.forward([0, 3], [20, 9], [0, 0], tokens=t1, want_rows=list(range(29))).cpu().double()
  t2 = torch.tensor(a[20:] + c[:1] + b[:0], dtype=torch.int32, device="cuda")
  o2 = st.forward([0, 1], [13, 1], [20, 0], tokens=t2, want_rows=list(range(14))).cpu().double()
  t3 = torch.tensor(c[1:], dtype=torch.int32, device="cuda")
  o3 = st.forward([1], [49], [1], tokens=t3, want_rows=list(range(49))).cpu().double()
  for s in (0, 1, 3):
    st.release_slot(s)
  assert rel(torch.cat([o1[:20], o2[:13]]), ra) < TOL["float32"]
  assert rel(o1[20:], rb) < TOL["float32"]
  assert rel(torch.cat([o2[13:], o3]), rc) < TOL["float32"]
  # decode rows of several requests in one step (the serving call: last row of every sequence), slots in any order
  st.forward([2, 0], [len(a) - 1, len(b) - 1], [0, 0], tokens=torch.tensor(a[:-1] + b[:-1], dtype=torch.int32, device="cuda"), want_rows=[])
  last = st.forward([0, 2], [1, 1], [len(b) - 1, len(a) - 1], tokens=torch.tensor([b[-1], a[-1]], dtype=torch.int32, device="cuda")).cpu().double()
  st.release_slot(0), st.release_slot(2)
  assert rel(last[0:1], rb[-1:]) < TOL["float32"] and rel(last[1:2], ra[-1:]) < TOL["float32"]


def test_slot_and_pages_reused_after_release(mixed):
  cfg, w, st = mixed
  free0 = st.counters()["kv_pages_free"]
  a, b = toks(90, cfg["vocab"], 11), toks(41, cfg["vocab"], 12)
  run(st, 1, a[:50], 0), run(st, 1, a[50:], 50)
  assert st.counters()["kv_pages_free"] < free0
  st.release_slot(1)
  assert st.counters()["kv_pages_free"] == free0
  got = torch.cat([run(st, 1, b[:17], 0), run(st, 1, b[17:], 17)])   # same slot, recycled pages, stale state behind it
  st.release_slot(1)
  assert rel(got, O.forward(cfg, w, b)) < TOL["float32"]


def test_first_tokens_and_single_token_prompt(mixed):
  cfg, w, st = mixed
  for n in (1, 2, 3, 4):
    ids = toks(n, cfg["vocab"], 20 + n)
    assert rel(run(st, 0, ids, 0), O.forward(cfg, w, ids)) < TOL["float32"]
    st.release_slot(0)


def test_long_decoding_and_far_state(mixed):
  """300 decoded tokens behind a 300-token prompt: the recurrent state carries the far past, the window slides over decoded
  tokens and across many 8-token pages."""
  cfg, w, st = mixed
  ids = toks(600, cfg["vocab"], 31)
  ref = O.forward(cfg, w, ids)
  run(st, 3, ids[:300], 0, rows=[])
  got = torch.cat([run(st, 3, [t], 300 + i) for i, t in enumerate(ids[300:])])
  st.release_slot(3)
  assert rel(got, ref[300:]) < TOL["float32"]
  assert float((got - ref[300:]).abs().max()) < 5e-3


# ----------------------------------------------------------------------------- edges made visible
def planted(window, keep, page):
  """One attention layer whose token 1 has a key that every query scores far above all others and a large value: a
  query that sees it (or not) by one position off changes the logits by orders of magnitude more than rounding."""
  cfg = config([(pair(heads=2, kv=1, dim=16, vdim=16, window=window, keep=keep, rs=0.0, ls=1.0, scale=1.0), 0)], width=32, vocab=50,
               taps=0, side=0, softcap=0)
  w = {k: v.float() for k, v in weights(cfg, seed=9).items()}
  w["embed"][1] *= 0.0
  w["embed"][1, 0] = 6.0                       # after the norm: one large channel
  w["l0.mix.left.k"][:, 0] = 0.0
  w["l0.mix.left.k"][0, 0] = 3.0               # key channel 0 reads it
  w["l0.mix.left.q.b"][0::16] = 4.0            # every query head looks for key channel 0
  w["l0.mix.left.v"][:, 0] = 2.0
  return cfg, {k: v.to(torch.bfloat16) for k, v in w.items()}


@pytest.mark.parametrize("window,keep", [(7, 0), (16, 3), (9, 2)])
def test_window_kept_first_and_page_edges(lib, window, keep):
  cfg, w = planted(window, keep, 8)
  st = stage(cfg, w, "float32", page=8)
  n = 70
  for at in sorted({0, keep - 1, keep, keep + 1, 7, 8, 15, 16, 30} - {-1}):
    ids = [(5 + 3 * i) % 48 + 2 for i in range(n)]
    ids[at] = 1                                                             # the planted key
    ref = O.forward(cfg, w, ids)
    seen = [i for i in range(n) if i >= at and (i - at < window or at < keep)]
    edge = [i for i in (at + window - 1, at + window) if i < n]
    assert all((i in seen) == (i - at < window or at < keep) for i in edge)
    whole = run(st, 0, ids, 0)
    st.release_slot(0)
    assert rel(whole, ref) < TOL["float32"], (at, "prompt")
    cut = max(1, at + 1)
    run(st, 0, ids[:cut], 0, rows=[])
    dec = torch.cat([run(st, 0, [t], cut + i) for i, t in enumerate(ids[cut:])])
    st.release_slot(0)
    assert rel(dec, ref[cut:]) < TOL["float32"], (at, "decoded")
    if at >= keep and at + window < n:
      # the oracle itself says the edge is visible: just inside and just outside differ by far more than the tolerance
      inside, outside = ref[at + window - 1], ref[at + window]
      assert float((inside - outside).abs().max()) > 100 * TOL["float32"] * float(ref.abs().max())
  st.close()


def test_far_key_among_hundreds_in_kept_first(lib):
  cfg, w = planted(12, 2, 8)
  st = stage(cfg, w, "float32", page=8)
  ids = [(7 + 5 * i) % 48 + 2 for i in range(400)]
  ids[1] = 1                                    # kept first token, 398 positions behind the last query
  ref = O.forward(cfg, w, ids)
  run(st, 1, ids[:390], 0, rows=[])
  got = torch.cat([run(st, 1, ids[390:395], 390), run(st, 1, [ids[395]], 395), run(st, 1, ids[396:], 396)])
  st.close()
  assert rel(got, ref[390:]) < TOL["float32"]
  ids2 = list(ids)
  ids2[1] = 2
  assert rel(O.forward(cfg, w, ids2)[390:], ref[390:]) > 0.05     # the far key matters


# ----------------------------------------------------------------------------- bf16 serving kernels
def planted64(window, keep, heads=6, kv=2, hd=64):
  """planted() at the head sizes the tensor-core prompt attention takes (key and value heads of 64 or 128), bf16 weights."""
  cfg = config([(pair(heads=heads, kv=kv, dim=hd, vdim=hd, window=window, keep=keep, rs=0.0, ls=1.0, scale=1.0), 0)], width=128, vocab=50,
               taps=0, side=0, softcap=0)
  w = {k: v.float() for k, v in weights(cfg, seed=9).items()}
  w["embed"][1] *= 0.0
  w["embed"][1, 0] = 6.0
  w["l0.mix.left.k"][:, 0] = 0.0
  w["l0.mix.left.k"][0::hd, 0] = 3.0
  w["l0.mix.left.q.b"][0::hd] = 4.0
  w["l0.mix.left.v"][:, 0] = 2.0
  return cfg, {k: v.to(torch.bfloat16) for k, v in w.items()}


@pytest.mark.parametrize("window,keep,heads,kv,hd", [(100, 5, 6, 2, 64), (64, 0, 4, 4, 64), (70, 66, 8, 1, 64), (1, 0, 2, 1, 64),
                                                     (130, 1, 5, 1, 128), (33, 3, 7, 7, 128)])
def test_tensor_core_prompt_attention_edges(lib, window, keep, heads, kv, hd):
  """Prompts long enough for the bf16 projections to come back as matrices run the tcgen05 attention: 64-key tiles are
  visited through the kept-first / window map, so the planted key sits at tile borders, at the window's two edges and
  among the kept first keys, in a whole prompt and in a second portion that starts far from position 0."""
  cfg, w = planted64(window, keep, heads, kv, hd)
  st = stage(cfg, w, "bfloat16", page=16, cap=512)
  n = 400
  for at in sorted({0, keep - 1, keep, 63, 64, 65, 127, 128, 200, 399 - window, 400 - window} - {-1}):
    if at < 0 or at >= n:
      continue
    ids = [(5 + 3 * i) % 48 + 2 for i in range(n)]
    ids[at] = 1
    ref = O.forward(cfg, w, ids)
    before = st.counters()["tc_attention"]
    whole = run(st, 0, ids, 0)
    assert st.counters()["tc_attention"] == before + 1
    st.release_slot(0)
    assert rel(whole, ref) < TOL["bfloat16"], (at, "prompt")
    got = torch.cat([run(st, 0, ids[:207], 0), run(st, 0, ids[207:], 207)])
    st.release_slot(0)
    assert rel(got, ref) < TOL["bfloat16"], (at, "two portions")
    if keep <= at < n - window - 1:
      inside, outside = ref[at + window - 1], ref[at + window]
      assert float((inside - outside).abs().max()) > 5 * TOL["bfloat16"] * float(ref.abs().max())
      assert rel(whole[at + window - 1: at + window + 1], ref[at + window - 1: at + window + 1]) < TOL["bfloat16"]
  st.close()


def test_bf16_prompt_kernels_equal_token_by_token(lib):
  """bf16 serving: a 300-token prompt (tensor-core Linears and attention, tiled filters) against the same tokens one at a
  time (split-K Linears, per-token attention, filters that write their own tails)."""
  cfg = config([(delta(heads=2, kv=1, dim=64, vdim=32, conv=4), 256), (pair(heads=4, kv=2, dim=64, vdim=64, window=90, keep=4, r_heads=2, r_dim=48,
                r_vdim=32), 256)], width=128, taps=4, side=16)
  w = weights(cfg, seed=13)
  ids = toks(300, cfg["vocab"], seed=14)
  ref = O.forward(cfg, w, ids)
  st = stage(cfg, w, "bfloat16", page=64)
  whole = run(st, 0, ids, 0)
  assert st.counters()["tc_attention"] == 1
  st.release_slot(0)
  run(st, 0, ids[:150], 0, rows=[])
  single = torch.cat([run(st, 0, [t], 150 + i) for i, t in enumerate(ids[150:])])
  st.close()
  assert rel(whole, ref) < TOL["bfloat16"] and rel(single, ref[150:]) < TOL["bfloat16"]
  assert rel(single, whole[150:]) < TOL["bfloat16"]


@pytest.mark.parametrize("lanes", ["4", "8", "16"])
def test_recurrence_lanes_per_column(lib, monkeypatch, lanes):
  """The recurrences spread a state column over 4, 8 or 16 lanes depending on the step's shape; every variant, pinned,
  against the oracle: a prompt, portions, and single tokens, key dims that need padding and several chunks per lane."""
  monkeypatch.setenv("XB_HY_LPC", lanes)
  cfg = config([(delta(heads=3, kv=1, dim=24, vdim=20, conv=2), 0), (delta(heads=2, kv=2, dim=160, vdim=40, conv=3), 64),
                (pair(ls=0.3, r_heads=5, r_dim=20, r_vdim=12), 0), (pair(r_heads=2, r_dim=136, r_vdim=70), 64)], width=96, taps=2, side=0)
  w = weights(cfg, seed=21)
  ids = toks(75, cfg["vocab"], seed=22)
  ref = O.forward(cfg, w, ids)
  st = stage(cfg, w, "float32")
  whole = run(st, 0, ids, 0)
  st.release_slot(0)
  parts = torch.cat([run(st, 0, ids[:33], 0), run(st, 0, ids[33:35], 33)] + [run(st, 0, [t], 35 + i) for i, t in enumerate(ids[35:])])
  st.close()
  assert rel(whole, ref) < TOL["float32"] and rel(parts, ref) < TOL["float32"]


# ----------------------------------------------------------------------------- the serving engine
def test_greedy_generation_through_the_engine(lib, tmp_path):
  """B200ShardInferenceEngine (the plugin API the node drives: infer_prompt / sample / infer_tensor, its request table and
  slot scheduler) on the registered refatar-tiny model, checkpoint written and loaded from disk, against greedy decoding of
  the oracle."""
  from safetensors.torch import load_file
  from xotorch_support_jetson_b200.b200_engine import B200ShardInferenceEngine
  from xotorch_support_jetson_b200.models import build_full_shard, model_cards
  from xotorch_support_jetson_b200.synth import LocalShardDownloader
  mid = "refatar-tiny"
  eng = B200ShardInferenceEngine(LocalShardDownloader(root=tmp_path, seed=2), device=0, max_seqs=4, max_tokens_per_seq=256,
                                 max_batch_tokens=16, page_tokens=16, dtype="float32")
  shard = build_full_shard(mid, "B200ShardInferenceEngine")
  cfg = model_cards[mid]["hf_config"]
  prompt = [3 + (11 * i) % 500 for i in range(37)]          # 37 tokens through 16-row native calls: chunked prefill

  async def go():
    out, state = await eng.infer_prompt("g1", shard, "<ids:" + ",".join(map(str, prompt)) + ">")
    ids, logits = [], [out]
    for _ in range(12):
      tok = await eng.sample(out, temp=0.0)
      ids.append(int(tok.item()))
      out, state = await eng.infer_tensor("g1", shard, tok.reshape(1, 1), state)
      logits.append(out)
    eng.end_request("g1")
    return ids, logits

  ids, logits = asyncio.run(go())
  files = sorted((tmp_path / "synthetic--refatar-tiny").glob("*.safetensors"))
  w = {}
  for f in files:
    w.update(load_file(str(f)))
  seq = list(prompt)
  for step, tok in enumerate(ids):
    ref = O.forward(cfg, w, seq)[-1]
    assert rel(torch.from_numpy(logits[step][0]).double(), ref) < TOL["float32"]
    top2 = ref.topk(2).values
    if float(top2[0] - top2[1]) > 1e-3:
      assert tok == int(ref.argmax()), step
    seq.append(tok)


# ----------------------------------------------------------------------------- the command line
def test_trace_runner_replays_steps(lib, tmp_path):
  """bin/trace_run as a user calls it: a model folder (config.json + one safetensors file), steps on standard input -- a
  whole prompt, a prompt in portions with single tokens behind it, a request that ends and whose slot the next one takes --
  and <step>.f32 files with the rows that were asked for, in the order asked, against the oracle."""
  import json
  import subprocess
  import sys
  from pathlib import Path
  from safetensors.torch import save_file
  cfg = config([(pair(heads=6, kv=3, dim=64, vdim=64, window=20, keep=2, r_heads=3, r_dim=24, r_vdim=40), 96), (delta(), 0)], width=64,
               vocab=120, taps=2, side=4, softcap=8.0)
  w = weights(cfg, seed=17)
  model = tmp_path / "model"
  model.mkdir()
  (model / "config.json").write_text(json.dumps(cfg))
  save_file({k: v.contiguous() for k, v in w.items()}, str(model / "model.safetensors"))
  a, b = toks(50, cfg["vocab"], 41), toks(31, cfg["vocab"], 42)
  steps = [
    {"step": 0, "entries": [{"id": "a", "tokens": a, "want": [49, 0, 20]}], "end": ["a"]},
    {"step": 1, "entries": [{"id": "b", "tokens": b[:17], "want": []}], "end": []},
    {"step": 2, "entries": [{"id": "b", "tokens": b[17:19], "want": [0, 1]}], "end": []},
  ] + [{"step": 3 + i, "entries": [{"id": "b", "tokens": [t], "want": [0]}], "end": (["b"] if 19 + i == len(b) - 1 else [])}
       for i, t in enumerate(b[19:])]
  root = Path(__file__).resolve().parent.parent
  ra, rb = O.forward(cfg, w, a), O.forward(cfg, w, b)
  for dtype in ("float32", "bfloat16"):
    out = tmp_path / f"out_{dtype}"
    p = subprocess.run([sys.executable, str(root / "bin" / "trace_run"), "--model", str(model), "--dtype", dtype, "--out", str(out),
                        "--max-tokens", "64"], input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done ")] == [f"done {s['step']}" for s in steps]
    rd = lambda i: torch.from_numpy(np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, cfg["vocab"])).double()  # noqa: E731
    assert rel(rd(0), ra[[49, 0, 20]]) < TOL[dtype]
    assert not (out / "1.f32").exists()
    assert rel(rd(2), rb[17:19]) < TOL[dtype]
    got = torch.cat([rd(3 + i) for i in range(len(b) - 19)])
    assert rel(got, rb[19:]) < TOL[dtype]
