"""The Bibevik design on the native hybrid engine against the plain restatement in tests/bibevik_oracle.py:
small configurations and random weights made here, every mechanism alone and at odd sizes, cached decoding, portions,
batches, slot and page reuse, far keys and page borders made visible, routing whose group limit matters, layers that
share tensors, long state, greedy generation through the serving engine and the trace runner."""
import asyncio
import json

import numpy as np
import pytest
import torch

import bibevik_oracle as O

pytestmark = pytest.mark.gpu
TOL = {"float32": 2e-4, "bfloat16": 6e-2}


def latent(heads=4, dim=24, rot_dim=8, vdim=20, kv_rank=32, base=10000.0, scale=None, dims=None):
  return "latent_attention", {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
                              "scale": scale or (dim + rot_dim) ** -0.5, "rot": {"base": base, "dims": rot_dim if dims is None else dims}}


def gdelta(heads=3, dim=32, rank=8):
  return "general_delta", {"heads": heads, "dim": dim, "rank": rank}


def lightning(heads=3, dim=16, vdim=24, decay=None):
  return "lightning", {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay or [0.5 + 0.49 * h / max(heads - 1, 1) for h in range(heads)]}


def glu(ff=128, limit=1.5):
  return {"kind": "dense", "ff": ff, "limit": limit}


def experts(n=8, top=2, ff=40, groups=4, keep=2, shared=48, scale=1.5, limit=2.0, shared_limit=1.0):
  m = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": n, "top": top, "scale": scale}}
  if groups:
    m["router"]["groups"] = {"count": groups, "keep": keep}
  if shared:
    m["shared"] = {"ff": shared, "limit": shared_limit}
  return m


def config(layers, width=96, vocab=200, eps=1e-5, scale=None):
  """layers: ((type, mixer), mlp) or ((type, mixer), mlp, weights_of)."""
  out = []
  for ent in layers:
    lay = {"type": ent[0][0], "mixer": ent[0][1], "mlp": ent[1]}
    if len(ent) > 2:
      lay["weights_of"] = ent[2]
    out.append(lay)
  return {"architecture": "Bibevik", "width": width, "vocab": vocab, "embedding": {"scale": scale or width ** 0.5}, "norm": {"eps": eps},
          "layers": out}


MIXED = config([(gdelta(), glu()), (latent(), experts()), (lightning(), None), (latent(), experts(), 1),
                (lightning(heads=2, dim=40, vdim=12, decay=[1.0, 0.9]), glu(64, 0.5)), (gdelta(), glu(), 0)])


def weights(cfg, seed=0):
  from xotorch_support_jetson_b200.synth import random_bibevik_state
  return random_bibevik_state(cfg, seed=seed)


def stage(cfg, w, dtype="float32", page=8, seqs=4, cap=512, per_seq=1024):
  from xotorch_support_jetson_b200.model_config import hybrid_model_config
  from xotorch_support_jetson_b200.shard import Shard
  from xotorch_support_jetson_b200.stage import StageRuntime
  c = hybrid_model_config(cfg)
  nl = c["num_layers"]
  st = StageRuntime(Shard("bibevik-test", 0, nl - 1, nl), c, max_batch_tokens=cap, max_seqs=seqs, max_tokens_per_seq=per_seq,
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


def rows_off(got, ref, tol):
  """How many rows differ by more than tol (relative to the reference's overall size)."""
  size = ref.pow(2).mean().sqrt()
  return int(((got - ref).pow(2).mean(dim=-1).sqrt() / size > tol).sum())


def bf16_round(x):
  return x.to(torch.bfloat16).double()


def has_experts(cfg):
  return any(l["mlp"] and l["mlp"]["kind"] == "moe" for l in cfg["layers"])


def logits(cfg, w, ids, rounding=None):
  return O.forward(cfg, w, ids, rounding=rounding)[0]


@pytest.fixture(scope="module")
def lib(built_lib):
  return built_lib


# ----------------------------------------------------------------------------- each mechanism alone, other sizes
ALONE = {
  "latent": config([(latent(), None)]),
  "latent_odd_sizes": config([(latent(heads=3, dim=10, rot_dim=6, vdim=7, kv_rank=21, base=50.0), None)], width=50, vocab=77),
  "latent_one_head_partial_rotation": config([(latent(heads=1, dim=16, rot_dim=12, vdim=16, kv_rank=16, dims=8, scale=0.4), None)]),
  "latent_wide_latent": config([(latent(heads=2, dim=32, rot_dim=16, vdim=24, kv_rank=320), None)]),
  "latent_no_unrotated_gain": config([(latent(heads=2, dim=8, rot_dim=32, vdim=8, kv_rank=8, base=3.0), None)]),
  "gdelta": config([(gdelta(), None)]),
  "gdelta_odd_sizes": config([(gdelta(heads=5, dim=10, rank=3), None)], width=50, vocab=77),
  "gdelta_wide_key_one_head": config([(gdelta(heads=1, dim=160, rank=20), None)]),
  "lightning": config([(lightning(), None)]),
  "lightning_odd_sizes_no_decay": config([(lightning(heads=5, dim=10, vdim=6, decay=[1.0, 0.999, 0.5, 0.01, 0.0]), None)], width=50, vocab=77),
  "lightning_wide_key": config([(lightning(heads=2, dim=136, vdim=70), None)]),
  "glu": config([(lightning(), glu(200, 0.7))]),
  "glu_wide_limit": config([(gdelta(), glu(72, 50.0))], scale=3.0),
  "experts": config([(lightning(), experts())]),
  "experts_no_groups_no_shared_top1": config([(lightning(), experts(n=5, top=1, groups=0, shared=0, scale=0.5))]),
  "experts_every_group_kept": config([(latent(), experts(n=6, top=3, groups=3, keep=3, shared=16))]),
  "experts_groups_of_one": config([(gdelta(), experts(n=6, top=2, groups=6, keep=3, shared=0))]),
  "experts_many": config([(lightning(), experts(n=40, top=6, ff=8, groups=8, keep=3, shared=24))]),
  "shared_tensors": config([(latent(), experts()), (gdelta(), glu()), (latent(), experts(), 0), (gdelta(), glu(), 1), (latent(), experts(), 0)]),
  "shared_from_a_later_layer": config([(lightning(), glu(), 1), (lightning(), glu())]),
  "mixed": MIXED,
}


@pytest.mark.parametrize("name", sorted(ALONE))
def test_mechanism_against_oracle(lib, name):
  cfg = ALONE[name]
  w = weights(cfg, seed=3)
  ids = toks(70, cfg["vocab"], seed=1)
  for dtype in ("float32", "bfloat16"):
    ref, layers = O.forward(cfg, w, ids, rounding=bf16_round if dtype == "bfloat16" else None)
    st = stage(cfg, w, dtype)
    taps = [torch.zeros(len(ids), cfg["width"], device="cuda") for _ in cfg["layers"]]
    t = torch.tensor(ids, dtype=torch.int32, device="cuda")
    got = st.forward([1], [len(ids)], [0], tokens=t, want_rows=list(range(len(ids))), taps=taps).cpu().double()
    st.close()
    if dtype == "bfloat16" and has_experts(cfg):
      # a token whose routing is a near tie may pick another expert once activations are rounded (and every later layer
      # with experts adds its own chances): a few such rows among the 70, the float32 pass above has none
      assert rows_off(got, ref, TOL[dtype]) <= 3, (name, dtype)
      continue
    for i, l in enumerate(layers):
      assert rel(taps[i].cpu().double(), l) < TOL[dtype], (name, dtype, "layer", i)
    assert rel(got, ref) < TOL[dtype], (name, dtype)


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
  ref = logits(cfg, w, ids)
  whole = run(st, 0, ids, 0)
  st.release_slot(0)
  single = torch.cat([run(st, 0, [t], p) for p, t in enumerate(ids)])
  st.release_slot(0)
  assert rel(whole, ref) < TOL["float32"] and rel(single, ref) < TOL["float32"]
  assert rel(single, whole) < 5e-5


@pytest.mark.parametrize("cuts", [[2, 37, 2, 5, 1, 1, 30, 2], [1, 1, 1, 2, 3, 70], [40, 40], [3] * 26 + [2], [17, 16, 2, 15, 31]])
def test_portions(mixed, cuts):
  cfg, w, st = mixed
  ids = toks(sum(cuts), cfg["vocab"], seed=4)
  ref = logits(cfg, w, ids)
  out, p = [], 0
  for c in cuts:
    out.append(run(st, 2, ids[p:p + c], p))
    p += c
  st.release_slot(2)
  assert rel(torch.cat(out), ref) < TOL["float32"]


def test_batch_of_unequal_requests_equals_each_alone(mixed):
  cfg, w, st = mixed
  a, b, c = toks(33, cfg["vocab"], 7), toks(9, cfg["vocab"], 8), toks(50, cfg["vocab"], 9)
  ra, rb, rc = (logits(cfg, w, x) for x in (a, b, c))
  t1 = torch.tensor(a[:20] + b, dtype=torch.int32, device="cuda")
  o1 = st.forward([0, 3], [20, 9], [0, 0], tokens=t1, want_rows=list(range(29))).cpu().double()
  t2 = torch.tensor(a[20:] + c[:1], dtype=torch.int32, device="cuda")
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
  assert rel(got, logits(cfg, w, b)) < TOL["float32"]


def test_first_tokens_and_single_token_prompt(mixed):
  cfg, w, st = mixed
  for n in (1, 2, 3, 4):
    ids = toks(n, cfg["vocab"], 20 + n)
    assert rel(run(st, 0, ids, 0), logits(cfg, w, ids)) < TOL["float32"]
    st.release_slot(0)


def test_long_decoding_and_far_state(mixed):
  """300 decoded tokens behind a 300-token prompt: the recurrent states carry the far past (one lightning head never decays),
  the attention reads every earlier position across many 8-token pages, rotations reach positions near 600."""
  cfg, w, st = mixed
  ids = toks(600, cfg["vocab"], 31)
  ref = logits(cfg, w, ids)
  run(st, 3, ids[:300], 0, rows=[])
  got = torch.cat([run(st, 3, [t], 300 + i) for i, t in enumerate(ids[300:])])
  st.release_slot(3)
  assert rel(got, ref[300:]) < TOL["float32"]
  assert float((got - ref[300:]).abs().max()) < 2e-3 * float(ref.abs().max())


# ----------------------------------------------------------------------------- edges made visible
def planted(rot_base=10000.0, rot_dim=4):
  """One latent-attention layer in which token 1 leaves a latent that every query scores far above all others and that
  carries a large value: a query that misses it (a page border, a lost cache row, the first position) changes the logits by
  orders of magnitude more than rounding does."""
  cfg = config([(latent(heads=2, dim=8, rot_dim=rot_dim, vdim=8, kv_rank=8, scale=1.0, base=rot_base), None)], width=32, vocab=50, scale=1.0)
  w = {k: v.float() for k, v in weights(cfg, seed=9).items()}
  n = 8 + rot_dim
  w["embed"] *= 32 ** 0.5
  w["embed"][:, 0] = 0.0
  w["embed"][:, 1] = 2.0                       # a channel that every token carries: queries are built on it
  w["embed"][1] *= 0.0
  w["embed"][1, 0] = 6.0                       # the planted token: one large channel that no other token has
  w["embed"][1, 1] = 2.0
  w["l0.norm1"] = torch.tensor(1.0)
  w["l0.mix.dkv"][:, 0] = 0.0
  w["l0.mix.dkv"][0, :] = 0.0
  w["l0.mix.dkv"][0, 0] = 3.0                  # latent channel 0 reads it
  w["l0.mix.dkv.norm"][0] = 1.0
  w["l0.mix.uk"][:, 0] = 0.0
  w["l0.mix.uk"][0::8, 0] = 2.0                # every head's first unrotated key entry is the latent's channel 0
  w["l0.mix.q"][0::n, :] = 0.0
  w["l0.mix.q"][0::n, 1] = 4.0                 # every head's first query entry is large and positive for every token
  w["l0.mix.uv"][:, 0] = 2.0
  return cfg, {k: v.to(torch.bfloat16) for k, v in w.items()}


def test_far_key_at_page_borders_and_first_positions(lib):
  cfg, w = planted()
  st = stage(cfg, w, "float32", page=8)
  n = 70
  for at in (0, 1, 7, 8, 9, 15, 16, 31, 32, 40):
    ids = [(5 + 3 * i) % 48 + 2 for i in range(n)]
    ids[at] = 1
    ref = logits(cfg, w, ids)
    ids2 = list(ids)
    ids2[at] = 2
    assert rel(logits(cfg, w, ids2)[at + 1:], ref[at + 1:]) > 0.05          # the planted key matters to every later token
    whole = run(st, 0, ids, 0)
    st.release_slot(0)
    assert rel(whole, ref) < TOL["float32"], (at, "prompt")
    cut = at + 1
    run(st, 0, ids[:cut], 0, rows=[])
    dec = torch.cat([run(st, 0, [t], cut + i) for i, t in enumerate(ids[cut:])])
    st.release_slot(0)
    assert rel(dec, ref[cut:]) < TOL["float32"], (at, "decoded")
  st.close()


def test_far_key_among_hundreds(lib):
  cfg, w = planted()
  st = stage(cfg, w, "float32", page=8)
  ids = [(7 + 5 * i) % 48 + 2 for i in range(400)]
  ids[3] = 1                                    # 396 positions behind the last query
  ref = logits(cfg, w, ids)
  run(st, 1, ids[:390], 0, rows=[])
  got = torch.cat([run(st, 1, ids[390:395], 390), run(st, 1, [ids[395]], 395), run(st, 1, ids[396:], 396)])
  st.close()
  assert rel(got, ref[390:]) < TOL["float32"]
  ids2 = list(ids)
  ids2[3] = 2
  assert rel(logits(cfg, w, ids2)[390:], ref[390:]) > 0.05


def test_rotation_depends_on_distance_only_through_the_rotated_part(lib):
  """Scores come from the rotated parts alone (the unrotated query is zeroed), a low base makes the angles large: prompts,
  portions and single tokens at positions up to 300 agree with the oracle, and the oracle with the positions shifted by one
  (a sequence that starts at another token) does not."""
  cfg = config([(latent(heads=2, dim=8, rot_dim=8, vdim=8, kv_rank=8, scale=2.0, base=7.0), None)], width=32, vocab=50)
  w = {k: v.float() for k, v in weights(cfg, seed=4).items()}
  w["l0.mix.q"].view(2, 16, 32)[:, :8, :] = 0.0
  w["l0.mix.q"] *= 4.0
  w = {k: v.to(torch.bfloat16) for k, v in w.items()}
  ids = toks(300, cfg["vocab"], seed=6)
  ref = logits(cfg, w, ids)
  shifted = logits(cfg, w, ids[:1] + ids)[1:]
  assert rel(shifted[50:], ref[50:]) > 0.02
  st = stage(cfg, w, "float32", page=16)
  got = torch.cat([run(st, 0, ids[:130], 0), run(st, 0, ids[130:132], 130)] + [run(st, 0, [t], 132 + i) for i, t in enumerate(ids[132:])])
  st.close()
  assert rel(got, ref) < TOL["float32"]


def test_state_that_never_decays_and_state_that_is_removed(lib):
  """Lightning with decay 1 keeps a key-value pair of the first token for ever; the general delta rule removes what it wrote
  when the same key comes again.  A planted first token shows in the last logits after 500 tokens (prompt + decoding)."""
  cfg = config([(lightning(heads=2, dim=8, vdim=8, decay=[1.0, 0.5]), None)], width=32, vocab=50)
  w = weights(cfg, seed=8)
  ids = [1] + [(7 + 5 * i) % 48 + 2 for i in range(499)]
  ref = logits(cfg, w, ids)
  assert rel(logits(cfg, w, [2] + ids[1:])[-5:], ref[-5:]) > 1e-3
  st = stage(cfg, w, "float32")
  run(st, 0, ids[:256], 0, rows=[])
  run(st, 0, ids[256:258], 256, rows=[])
  got = torch.cat([run(st, 0, [t], 258 + i) for i, t in enumerate(ids[258:])])
  st.close()
  assert rel(got[-5:], ref[-5:]) < TOL["float32"] and rel(got, ref[258:]) < TOL["float32"]


# ----------------------------------------------------------------------------- bf16 serving kernels
def test_bf16_prompt_kernels_equal_token_by_token(lib):
  """bf16 serving at sizes the tensor-core Linears take: a 300-token prompt (bf16 matrices out of the Linears) against the same
  tokens one at a time (split-K planes) and against the oracle."""
  cfg = config([(gdelta(heads=2, dim=64, rank=16), glu(256, 2.0)), (latent(heads=4, dim=32, rot_dim=32, vdim=64, kv_rank=64), glu(128)),
                (lightning(heads=2, dim=64, vdim=64), glu(256))], width=128)
  w = weights(cfg, seed=13)
  ids = toks(300, cfg["vocab"], seed=14)
  ref = logits(cfg, w, ids, rounding=bf16_round)
  st = stage(cfg, w, "bfloat16", page=64)
  whole = run(st, 0, ids, 0)
  st.release_slot(0)
  run(st, 0, ids[:150], 0, rows=[])
  single = torch.cat([run(st, 0, [t], 150 + i) for i, t in enumerate(ids[150:])])
  st.close()
  assert rel(whole, ref) < TOL["bfloat16"] and rel(single, ref[150:]) < TOL["bfloat16"]
  assert rel(single, whole[150:]) < TOL["bfloat16"]


@pytest.mark.parametrize("form", ["0", "2", "4"])
def test_latent_attention_forms_in_bf16(lib, monkeypatch, form):
  """bf16 serving runs latent attention on the tensor cores, rows = (token, head) pairs over shared 64-key tiles: four warps of
  rows per block for prompts ("4"), one warp per block and every sequence's keys shared out over blocks for steps of few rows
  ("2"); "0" is the per-(token, head) kernel.  Each form pinned: a planted far key at 64-key tile borders in a prompt, in
  portions that start inside a tile, in single tokens, and a batch of three unequal requests whose rows share tiles."""
  monkeypatch.setenv("XB_HY_LAT_MMA", form)
  cfg = config([(latent(heads=3, dim=16, rot_dim=16, vdim=24, kv_rank=48, scale=0.5), None), (latent(heads=5, dim=8, rot_dim=8, vdim=8, kv_rank=160), glu(64))],
               width=64, vocab=50)
  w = {k: v.float() for k, v in weights(cfg, seed=19).items()}
  w["embed"][:, 0] = 0.0
  w["embed"][1] *= 0.2
  w["embed"][1, 0] = 1.5                       # the planted token: a channel no other token has
  w["l0.mix.dkv"][0, :] = 0.0
  w["l0.mix.dkv"][0, 0] = 6.0                  # latent channel 0 of layer 0 reads it
  w["l0.mix.uk"][0::16, 0] += 3.0
  w["l0.mix.uv"][:, 0] += 1.0
  w = {k: v.to(torch.bfloat16) for k, v in w.items()}
  st = stage(cfg, w, "bfloat16", page=16, cap=512)
  n = 200
  for at in (0, 63, 64, 127, 128, 130):
    ids = [(5 + 3 * i) % 48 + 2 for i in range(n)]
    ids[at] = 1
    ref = logits(cfg, w, ids, rounding=bf16_round)
    whole = run(st, 0, ids, 0)
    st.release_slot(0)
    assert rel(whole, ref) < TOL["bfloat16"], (at, "prompt")
    got = torch.cat([run(st, 0, ids[:70], 0), run(st, 0, ids[70:129], 70), run(st, 0, ids[129:131], 129)] +
                    [run(st, 0, [t], 131 + i) for i, t in enumerate(ids[131:150])] + [run(st, 0, ids[150:], 150)])
    st.release_slot(0)
    assert rel(got, ref) < TOL["bfloat16"], (at, "portions")
  ids2 = list(ids)
  ids2[130] = 2
  assert rel(logits(cfg, w, ids2, rounding=bf16_round)[131:], ref[131:]) > 3 * TOL["bfloat16"]     # the planted key shows
  a, b, c = toks(70, 50, 7), toks(3, 50, 8), toks(129, 50, 9)
  ra, rb, rc = (logits(cfg, w, x, rounding=bf16_round) for x in (a, b, c))
  t1 = torch.tensor(a + b + c, dtype=torch.int32, device="cuda")
  o1 = st.forward([0, 3, 1], [70, 3, 129], [0, 0, 0], tokens=t1, want_rows=list(range(202))).cpu().double()
  assert rel(o1[:70], ra) < TOL["bfloat16"] and rel(o1[70:73], rb) < TOL["bfloat16"] and rel(o1[73:], rc) < TOL["bfloat16"]
  nxt = st.forward([3, 0, 1], [1, 1, 1], [3, 70, 129], tokens=torch.tensor([b[0], a[0], c[0]], dtype=torch.int32, device="cuda")).cpu().double()
  for row, seq in zip(nxt, (b + b[:1], a + a[:1], c + c[:1])):
    assert rel(row[None], logits(cfg, w, seq, rounding=bf16_round)[-1:]) < TOL["bfloat16"]
  st.close()


@pytest.mark.parametrize("lanes", ["4", "8", "16"])
def test_recurrence_lanes_per_column(lib, monkeypatch, lanes):
  """The recurrences spread a state column over 4, 8 or 16 lanes depending on the step's shape; every variant, pinned,
  against the oracle: a prompt, portions, and single tokens, key dims that need padding and several chunks per lane."""
  monkeypatch.setenv("XB_HY_LPC", lanes)
  cfg = config([(gdelta(heads=3, dim=24, rank=4), None), (gdelta(heads=2, dim=160, rank=9), glu(64)),
                (lightning(heads=5, dim=20, vdim=12), None), (lightning(heads=2, dim=136, vdim=70), glu(64))])
  w = weights(cfg, seed=21)
  ids = toks(75, cfg["vocab"], seed=22)
  ref = logits(cfg, w, ids)
  st = stage(cfg, w, "float32")
  whole = run(st, 0, ids, 0)
  st.release_slot(0)
  parts = torch.cat([run(st, 0, ids[:33], 0), run(st, 0, ids[33:35], 33)] + [run(st, 0, [t], 35 + i) for i, t in enumerate(ids[35:])])
  st.close()
  assert rel(whole, ref) < TOL["float32"] and rel(parts, ref) < TOL["float32"]


# ----------------------------------------------------------------------------- the serving engine
def test_greedy_generation_through_the_engine(lib, tmp_path):
  """B200ShardInferenceEngine (infer_prompt / sample / infer_tensor, its request table and slot scheduler) on the registered
  bibevik-tiny model, checkpoint written and loaded from disk, against greedy decoding of the oracle."""
  from safetensors.torch import load_file
  from xotorch_support_jetson_b200.b200_engine import B200ShardInferenceEngine
  from xotorch_support_jetson_b200.models import build_full_shard, model_cards
  from xotorch_support_jetson_b200.synth import LocalShardDownloader
  mid = "bibevik-tiny"
  eng = B200ShardInferenceEngine(LocalShardDownloader(root=tmp_path, seed=2), device=0, max_seqs=4, max_tokens_per_seq=256,
                                 max_batch_tokens=16, page_tokens=16, dtype="float32")
  shard = build_full_shard(mid, "B200ShardInferenceEngine")
  cfg = model_cards[mid]["hf_config"]
  prompt = [3 + (11 * i) % 380 for i in range(37)]          # 37 tokens through 16-row native calls: chunked prefill

  async def go():
    out, state = await eng.infer_prompt("g1", shard, "<ids:" + ",".join(map(str, prompt)) + ">")
    ids, lg = [], [out]
    for _ in range(12):
      tok = await eng.sample(out, temp=0.0)
      ids.append(int(tok.item()))
      out, state = await eng.infer_tensor("g1", shard, tok.reshape(1, 1), state)
      lg.append(out)
    eng.end_request("g1")
    return ids, lg

  ids, lg = asyncio.run(go())
  w = {}
  for f in sorted((tmp_path / "synthetic--bibevik-tiny").glob("*.safetensors")):
    w.update(load_file(str(f)))
  seq = list(prompt)
  for step, tok in enumerate(ids):
    ref = logits(cfg, w, seq)[-1]
    assert rel(torch.from_numpy(lg[step][0]).double(), ref) < TOL["float32"]
    top2 = ref.topk(2).values
    if float(top2[0] - top2[1]) > 1e-3:
      assert tok == int(ref.argmax()), step
    seq.append(tok)


# ----------------------------------------------------------------------------- the command line
def test_trace_runner_replays_steps(lib, tmp_path):
  """bin/trace_run on a model folder whose config.json leaves the decay projection's rank to the checkpoint: a whole prompt, a
  prompt in portions with single tokens behind it, a request that ends and whose slot the next one takes."""
  import subprocess
  import sys
  from pathlib import Path
  from safetensors.torch import save_file
  cfg = config([(gdelta(heads=2, dim=24, rank=5), glu(80)), (latent(heads=3, dim=16, rot_dim=8, vdim=12, kv_rank=24), experts(n=4, top=2, groups=2, keep=1)),
                (lightning(heads=2, dim=16, vdim=32), None)], width=64, vocab=120)
  w = weights(cfg, seed=17)
  del cfg["layers"][0]["mixer"]["rank"]
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
  ra, rb = logits(cfg, w, a), logits(cfg, w, b)
  out = tmp_path / "out"
  p = subprocess.run([sys.executable, str(root / "bin" / "trace_run"), "--model", str(model), "--dtype", "float32", "--out", str(out),
                      "--max-tokens", "64"], input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
  assert p.returncode == 0, p.stderr[-2000:]
  assert [l for l in p.stdout.splitlines() if l.startswith("done ")] == [f"done {s['step']}" for s in steps]
  rd = lambda i: torch.from_numpy(np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, cfg["vocab"])).double()  # noqa: E731
  assert rel(rd(0), ra[[49, 0, 20]]) < TOL["float32"]
  assert not (out / "1.f32").exists()
  assert rel(rd(2), rb[17:19]) < TOL["float32"]
  got = torch.cat([rd(3 + i) for i in range(len(b) - 19)])
  assert rel(got, rb[19:]) < TOL["float32"]
