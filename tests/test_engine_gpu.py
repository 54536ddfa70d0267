"""Parity of the CUDA layer-range forward (through the C ABI) against the CPU oracle:
per-layer hidden states, logits and greedy tokens, for each model family, full shard
and pipeline splits, prefill + cached decode, ragged batches."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

# Stated bf16 tolerance (north_star): both sides compute in bf16 with fp32 accumulation in
# different orders, so values differ by a few bf16 ulps (2^-8 relative) that compound over
# layers.  Hidden states / logits must agree within REL_TOL of the tensor's max-abs.
REL_TOL = 0.04
# The same bound per model at about twice the worst case measured on the B200 over prefill + decode, every layer
# (llama-3.2-tiny 0.012, llama-3.1-tiny 0.023 -- head_dim 128, 6 layers --, qwen-2.5-tiny 0.018): a regression
# that doubles the error fails.  REL_TOL itself stays the ceiling for the checks that mix models.
MODEL_TOL = {"llama-3.2-tiny": 0.025, "llama-3.1-tiny": 0.04, "qwen-2.5-tiny": 0.035, "mistral-tiny": 0.03}


def _setup(mid, seed=0, std=0.05, jitter=0.1):
  from oracle import torch_oracle as O
  from xotorch_support_jetson_b200.models import model_cards
  from xotorch_support_jetson_b200.synth import random_hf_state
  hf_cfg = model_cards[mid]["hf_config"]
  cfg = O.model_config_from_hf(hf_cfg)
  state = random_hf_state(hf_cfg, seed=seed, std=std, norm_jitter=jitter)
  return O, cfg, state


def _rel(a, b):
  return float(np.abs(a - b).max() / (np.abs(b).max() + 1e-12))


@pytest.mark.parametrize("mid,splits", [
  ("llama-3.2-tiny", [(0, 3)]),
  ("llama-3.1-tiny", [(0, 5)]),
  ("qwen-2.5-tiny", [(0, 3)]),
  ("llama-3.1-tiny", [(0, 1), (2, 3), (4, 5)]),
  ("qwen-2.5-tiny", [(0, 1), (2, 3)]),
  # an id that is neither llama nor qwen: plain RotaryPositionalEmbeddings (no frequency scaling), no bias, untied
  # head (general_mha.py:58-63); 5 query heads on 1 kv head
  ("mistral-tiny", [(0, 3)]),
  ("mistral-tiny", [(0, 0), (1, 3)]),
])
def test_prefill_decode_parity(built_lib, mid, splits):
  from xotorch_support_jetson_b200.shard import Shard
  from xotorch_support_jetson_b200.stage import StageRuntime
  O, cfg, state = _setup(mid)
  nl = cfg["num_layers"]
  L, n_dec = 37, 6
  g = torch.Generator().manual_seed(1234)
  prompt = torch.randint(1, cfg["vocab_size"], (1, L), generator=g)
  ref_stages = [O.OracleShardModel(cfg, mid, a, b, state, O.OracleOptions(max_generated_tokens=32)) for a, b in splits]
  ref_toks, ref_logits, ref_taps = O.greedy_generate(ref_stages, prompt, n_dec, collect_logits=True, taps_at=(0, 1, n_dec - 1))

  stages = [StageRuntime(Shard(mid, a, b, nl), cfg, device=0, max_batch_tokens=64, max_seqs=2, max_tokens_per_seq=128,
                         page_tokens=16) for a, b in splits]
  for s in stages:
    s.load_state(state)
  D = cfg["embed_dim"]

  def run(x_tokens, q_len, pos, want_taps):
    taps = {}
    h = None
    for s, (a, b) in zip(stages, splits):
      tl = [torch.empty((q_len, D), dtype=torch.bfloat16, device="cuda") for _ in range(a, b + 1)] if want_taps else None
      if h is None:
        h = s.forward([0], [q_len], [pos], tokens=x_tokens, taps=tl)
      else:
        h = s.forward([0], [q_len], [pos], hidden=h, taps=tl)
      if want_taps:
        for i, l in enumerate(range(a, b + 1)):
          taps[l] = tl[i].float().cpu().numpy()
    return h, taps

  toks = prompt.to(torch.int32).cuda().reshape(-1)
  got_toks, pos = [], 0
  x, q_len = toks, L
  worst_h, worst_l = 0.0, 0.0
  tap_i = 0
  for step in range(n_dec):
    want = step in (0, 1, n_dec - 1)
    logits, taps = run(x, q_len, pos, want)
    if want:
      rt = ref_taps[tap_i]
      tap_i += 1
      for l in range(nl):
        worst_h = max(worst_h, _rel(taps[l], rt[l].reshape(q_len, D)))
    worst_l = max(worst_l, _rel(logits.cpu().numpy(), ref_logits[step]))
    # feed the ORACLE's token so both sides see the same history even if an argmax near-tie flips
    pos += q_len
    got_toks.append(int(stages[-1].sample(logits, temp=0.0).item()))
    x = torch.tensor([int(ref_toks[0, step])], dtype=torch.int32, device="cuda")
    q_len = 1
  print(f"{mid} {splits}: hidden rel err {worst_h:.4f}, logits rel err {worst_l:.4f}, tokens {got_toks} vs {ref_toks[0].tolist()}")
  assert worst_h < MODEL_TOL[mid] and worst_l < MODEL_TOL[mid]
  agree = sum(int(a == b) for a, b in zip(got_toks, ref_toks[0].tolist()))
  assert agree >= n_dec - 1
  for s in stages:
    s.close()


def test_ragged_batch_equals_single_sequence_runs(built_lib):
  """bs>1 has no reference execution through the API: its oracle is
  independent bs=1 runs.  Three sequences of different lengths in one batch, sharing the
  page pool, must reproduce the per-sequence results."""
  from xotorch_support_jetson_b200.shard import Shard
  from xotorch_support_jetson_b200.stage import StageRuntime
  mid = "llama-3.2-tiny"
  O, cfg, state = _setup(mid)
  nl = cfg["num_layers"]
  st = StageRuntime(Shard(mid, 0, nl - 1, nl), cfg, device=0, max_batch_tokens=128, max_seqs=4, max_tokens_per_seq=96, page_tokens=16)
  st.load_state(state)
  lens = [19, 33, 7]
  g = torch.Generator().manual_seed(7)
  prompts = [torch.randint(1, cfg["vocab_size"], (n,), generator=g).to(torch.int32).cuda() for n in lens]
  singles = []
  for i, p in enumerate(prompts):
    lg = st.forward([3], [lens[i]], [0], tokens=p)
    t1 = st.sample(lg, temp=0.0)
    lg2 = st.forward([3], [1], [lens[i]], tokens=t1)
    singles.append((lg.clone(), lg2.clone()))
    st.release_slot(3)
  lg = st.forward([0, 1, 2], lens, [0, 0, 0], tokens=torch.cat(prompts))
  t1 = st.sample(lg, temp=0.0)
  lg2 = st.forward([0, 1, 2], [1, 1, 1], lens, tokens=t1)
  torch.cuda.synchronize()
  # The split-K factor of a Linear depends on the number of token rows in the call, so the
  # fp32 summation order (and a few bf16 roundings downstream) may differ between a batched
  # and a single-sequence run: equal within a small fraction of the stated tolerance.
  for i in range(3):
    a, b = lg[i].cpu().numpy(), singles[i][0][0].cpu().numpy()
    assert _rel(a, b) < REL_TOL / 2, f"prefill logits of seq {i} differ between batched and single run: {_rel(a, b)}"
    a, b = lg2[i].cpu().numpy(), singles[i][1][0].cpu().numpy()
    assert _rel(a, b) < REL_TOL / 2, f"decode logits of seq {i} differ between batched and single run: {_rel(a, b)}"
  st.close()


def test_sampler_matches_reference_semantics(built_lib):
  """xb_sample with caller-supplied Exp(1) noise must pick the same token as the
  restated torchtune sampler, for greedy, temperature and top-k settings."""
  from oracle import torch_oracle as O
  from xotorch_support_jetson_b200.shard import Shard
  from xotorch_support_jetson_b200.stage import StageRuntime
  mid = "llama-3.2-tiny"
  _, cfg, state = _setup(mid)
  nl = cfg["num_layers"]
  st = StageRuntime(Shard(mid, 0, nl - 1, nl), cfg, device=0, max_batch_tokens=16, max_seqs=8, max_tokens_per_seq=32)
  V = cfg["vocab_size"]
  g = torch.Generator().manual_seed(3)
  for temp, top_k in ((0.6, 35), (1.0, 5), (1e-5, 35), (0.85, 0), (2.0, 100)):
    logits = (torch.randn(8, V, generator=g) * 3).to(torch.bfloat16).float()
    q = torch.empty(8, V).exponential_(1, generator=g)
    ref = O.sample(logits.clone(), temperature=temp, top_k=top_k if top_k else None, q=q).reshape(-1)
    got = st.sample(logits.cuda(), temp=temp, top_k=top_k, q=q.cuda()).cpu()
    assert torch.equal(got.to(torch.int64), ref.to(torch.int64)), (temp, top_k, got, ref)
  # greedy entry (temp <= 0): first-index argmax
  logits = (torch.randn(8, V, generator=g)).to(torch.bfloat16).float()
  logits[0, 5] = logits[0, 900] = 50.0
  got = st.sample(logits.cuda(), temp=0.0).cpu()
  assert got[0].item() == 5
  assert torch.equal(got.to(torch.int64), logits.argmax(-1))
  # top-p: the sampled token must lie in the nucleus, and p=tiny must give the argmax
  logits = (torch.randn(8, V, generator=g) * 2).float()   # no planted tie
  probs = torch.softmax(logits, -1)
  got = st.sample(logits.cuda(), temp=1.0, top_p=1e-6, seed=1).cpu()
  assert torch.equal(got.to(torch.int64), logits.argmax(-1))
  for seed in range(4):
    got = st.sample(logits.cuda(), temp=1.0, top_p=0.5, seed=seed).cpu().to(torch.int64)
    sp, si = probs.sort(-1, descending=True)
    cut = (sp.cumsum(-1) - sp) < 0.5
    for r in range(8):
      assert got[r].item() in set(si[r][cut[r]].tolist())
  st.close()


@pytest.mark.parametrize("mid", ["llama-3.2-tiny", "llama-3.1-tiny", "qwen-2.5-tiny", "mistral-tiny"])
def test_cuda_path_against_committed_golden(built_lib, mid):
  """The CUDA forward against tests/golden/oracle_<model>.npz (generated by oracle/gen_golden.py
  from the oracle in reference-exact mode; nothing under oracle/ is executed here)."""
  import json
  from pathlib import Path
  from xotorch_support_jetson_b200 import model_config as mc
  from xotorch_support_jetson_b200.models import model_cards
  from xotorch_support_jetson_b200.shard import Shard
  from xotorch_support_jetson_b200.stage import StageRuntime
  from xotorch_support_jetson_b200.synth import random_hf_state
  g = np.load(Path(__file__).resolve().parent / "golden" / f"oracle_{mid}.npz", allow_pickle=False)
  meta = json.loads(str(g["meta"]))
  hf_cfg = model_cards[mid]["hf_config"]
  import tempfile
  with tempfile.TemporaryDirectory() as td:
    (Path(td) / "config.json").write_text(json.dumps(hf_cfg))
    cfg = mc.load_model_config(Path(td) / "config.json")
  state = random_hf_state(hf_cfg, seed=meta["seed"], std=meta["std"], norm_jitter=meta["norm_jitter"])
  nl, D = cfg["num_layers"], cfg["embed_dim"]
  st = StageRuntime(Shard(mid, 0, nl - 1, nl), cfg, device=0, max_batch_tokens=64, max_seqs=2, max_tokens_per_seq=128, page_tokens=32)
  st.load_state(state)
  prompt = torch.from_numpy(g["prompt"]).cuda().reshape(-1)
  L = prompt.numel()
  taps = [torch.empty((L, D), dtype=torch.bfloat16, device="cuda") for _ in range(nl)]
  logits = st.forward([0], [L], [0], tokens=prompt, taps=taps)
  hid = np.stack([t[-1].float().cpu().numpy() for t in taps])
  assert _rel(hid, g["prefill_hidden_last"]) < REL_TOL
  n = g["tokens"].shape[1]
  got_tokens, worst = [], _rel(logits.cpu().numpy()[0], g["logits"][0])
  for step in range(1, n):
    got_tokens.append(int(st.sample(logits, temp=0.0).item()))
    x = torch.tensor([int(g["tokens"][0, step - 1])], dtype=torch.int32, device="cuda")
    if step == 1:
      taps1 = [torch.empty((1, D), dtype=torch.bfloat16, device="cuda") for _ in range(nl)]
      logits = st.forward([0], [1], [L + step - 1], tokens=x, taps=taps1)
      assert _rel(np.stack([t[0].float().cpu().numpy() for t in taps1]), g["decode_hidden"]) < REL_TOL
    else:
      logits = st.forward([0], [1], [L + step - 1], tokens=x)
    worst = max(worst, _rel(logits.cpu().numpy()[0], g["logits"][step]))
  got_tokens.append(int(st.sample(logits, temp=0.0).item()))
  assert worst < REL_TOL, worst
  # greedy tokens: identical wherever the golden top-2 margin is above the numerical noise
  srt = np.sort(g["logits"], axis=-1)
  margin = srt[:, -1] - srt[:, -2]
  noise = REL_TOL * np.abs(g["logits"]).max()
  for i in range(n):
    if margin[i] > 2 * noise:
      assert got_tokens[i] == int(g["tokens"][0, i]), (i, got_tokens, g["tokens"][0].tolist())
  st.close()


@pytest.mark.parametrize("mid,L", [("llama-3.1-tiny", 333), ("llama-3.2-tiny", 200), ("qwen-2.5-tiny", 150)])
def test_long_prompt_prefill_multi_tile_attention(built_lib, mid, L):
  """Prompts spanning several 64-key attention tiles and several query tiles (causal masking
  across tiles, online-softmax rescaling, KV ring reuse), plus a chunked continuation."""
  from xotorch_support_jetson_b200.shard import Shard
  from xotorch_support_jetson_b200.stage import StageRuntime
  O, cfg, state = _setup(mid)
  nl, D = cfg["num_layers"], cfg["embed_dim"]
  g = torch.Generator().manual_seed(99)
  prompt = torch.randint(1, cfg["vocab_size"], (1, L), generator=g)
  ref = O.OracleShardModel(cfg, mid, 0, nl - 1, state, O.OracleOptions(max_generated_tokens=8))
  ref_toks, ref_logits, ref_taps = O.greedy_generate([ref], prompt, 2, collect_logits=True, taps_at=(0,))
  st = StageRuntime(Shard(mid, 0, nl - 1, nl), cfg, device=0, max_batch_tokens=512, max_seqs=2, max_tokens_per_seq=512, page_tokens=64)
  st.load_state(state)
  toks = prompt.to(torch.int32).cuda().reshape(-1)
  taps = [torch.empty((L, D), dtype=torch.bfloat16, device="cuda") for _ in range(nl)]
  lg = st.forward([0], [L], [0], tokens=toks, taps=taps)
  # same prompt in two chunks (second chunk attends to the cached first one)
  cut = 64 + 37
  st.forward([1], [cut], [0], tokens=toks[:cut])
  lg2 = st.forward([1], [L - cut], [cut], tokens=toks[cut:])
  nxt = torch.tensor([int(ref_toks[0, 0])], dtype=torch.int32, device="cuda")
  lg3 = st.forward([0], [1], [L], tokens=nxt)
  torch.cuda.synchronize()
  worst_h = max(_rel(taps[l].float().cpu().numpy(), ref_taps[0][l].reshape(L, D)) for l in range(nl))
  e1 = _rel(lg.cpu().numpy(), ref_logits[0])
  e2 = _rel(lg2.cpu().numpy(), ref_logits[0])
  e3 = _rel(lg3.cpu().numpy(), ref_logits[1])
  print(f"{mid} L={L}: hidden {worst_h:.4f} logits {e1:.4f} chunked {e2:.4f} decode {e3:.4f}")
  assert worst_h < REL_TOL and e1 < REL_TOL and e2 < REL_TOL and e3 < REL_TOL
  st.close()


def test_long_context_chunked_prefill_beyond_page_cache(built_lib):
  """8.5k-token context on a tiny model, prefilled in 2048-token chunks (BASELINE config 3 runs
  8k contexts): more than 128 pages per sequence, so the attention producer's on-demand page
  lookups and many-tile softmax rescaling are exercised; then cached decode steps."""
  from xotorch_support_jetson_b200.shard import Shard
  from xotorch_support_jetson_b200.stage import StageRuntime
  mid = "llama-3.2-tiny"
  O, cfg, state = _setup(mid)
  nl = cfg["num_layers"]
  L, CH = 8500, 2048
  g = torch.Generator().manual_seed(5)
  prompt = torch.randint(1, cfg["vocab_size"], (1, L), generator=g)
  ref = O.OracleShardModel(cfg, mid, 0, nl - 1, state, O.OracleOptions(max_generated_tokens=8))
  ref_toks, ref_logits, _ = O.greedy_generate([ref], prompt, 3, collect_logits=True)
  st = StageRuntime(Shard(mid, 0, nl - 1, nl), cfg, device=0, max_batch_tokens=CH, max_seqs=1, max_tokens_per_seq=L + 64, page_tokens=64)
  st.load_state(state)
  toks = prompt.to(torch.int32).cuda().reshape(-1)
  with torch.cuda.stream(torch.cuda.Stream()):
    for c0 in range(0, L, CH):
      c1 = min(L, c0 + CH)
      lg = st.forward([0], [c1 - c0], [c0], tokens=toks[c0:c1])
    errs = [_rel(lg.cpu().numpy(), ref_logits[0])]
    for i in range(2):
      x = torch.tensor([int(ref_toks[0, i])], dtype=torch.int32, device="cuda")
      lg = st.forward([0], [1], [L + i], tokens=x)
      errs.append(_rel(lg.cpu().numpy(), ref_logits[i + 1]))
  torch.cuda.synchronize()
  print(f"8.5k context: logits rel err prefill {errs[0]:.4f}, decode {errs[1]:.4f} {errs[2]:.4f}")
  assert max(errs) < REL_TOL
  st.close()


def test_ragged_decode_contexts_and_large_batch(built_lib):
  """Decode steps over sequences of very different context lengths in ONE batch (kv splits are
  chosen from the longest, each sequence walks only its own tiles), and a batch large enough that
  the grid exceeds one wave (unsplit path); each sequence must match its own single-sequence run."""
  from xotorch_support_jetson_b200.shard import Shard
  from xotorch_support_jetson_b200.stage import StageRuntime
  mid = "llama-3.1-tiny"
  O, cfg, state = _setup(mid)
  nl = cfg["num_layers"]
  lens = [1, 63, 64, 65, 130, 257, 400]
  n = len(lens)
  st = StageRuntime(Shard(mid, 0, nl - 1, nl), cfg, device=0, max_batch_tokens=512, max_seqs=160, max_tokens_per_seq=512, page_tokens=32)
  st.load_state(state)
  g = torch.Generator().manual_seed(3)
  prompts = [torch.randint(1, cfg["vocab_size"], (L,), generator=g).to(torch.int32).cuda() for L in lens]
  with torch.cuda.stream(torch.cuda.Stream()):
    # single-sequence references: prefill + 3 decode steps each, in slot n (released afterwards)
    ref = []
    for i, p in enumerate(prompts):
      lg = st.forward([n], [lens[i]], [0], tokens=p)
      seq = [lg.clone()]
      tok = st.sample(lg, temp=0.0)
      for k in range(3):
        lg = st.forward([n], [1], [lens[i] + k], tokens=tok)
        seq.append(lg.clone())
        tok = st.sample(lg, temp=0.0)
      ref.append(seq)
      st.release_slot(n)
    # batched: prefill one by one (same shapes as the references), then decode all together
    toks = []
    for i, p in enumerate(prompts):
      lg = st.forward([i], [lens[i]], [0], tokens=p)
      assert torch.equal(lg, ref[i][0])
      toks.append(st.sample(lg, temp=0.0))
    tok = torch.cat(toks)
    for k in range(3):
      lg = st.forward(list(range(n)), [1] * n, [L + k for L in lens], tokens=tok)
      for i in range(n):
        assert _rel(lg[i].cpu().numpy(), ref[i][k + 1][0].cpu().numpy()) < REL_TOL / 2, (i, k)
      tok = st.sample(lg, temp=0.0)
    for i in range(n):
      st.release_slot(i)
    # large decode batch: 150 sequences x 2 kv heads = 300 blocks > one wave -> unsplit path
    B = 150
    p = torch.randint(1, cfg["vocab_size"], (B, 20), generator=g).to(torch.int32).cuda()
    for c0 in range(0, B, 25):
      st.forward(list(range(c0, c0 + 25)), [20] * 25, [0] * 25, tokens=p[c0:c0 + 25].reshape(-1))
    x = torch.randint(1, cfg["vocab_size"], (B,), generator=g).to(torch.int32).cuda()
    h_all = []
    for c0 in range(0, B, 128):      # the LM head path takes up to 128 sequences per call
      c1 = min(B, c0 + 128)
      h_all.append(st.forward(list(range(c0, c1)), [1] * (c1 - c0), [20] * (c1 - c0), tokens=x[c0:c1]))
    one = st.forward([B], [20], [0], tokens=p[7])
    one = st.forward([B], [1], [20], tokens=x[7:8])
  torch.cuda.synchronize()
  assert _rel(torch.cat(h_all)[7].cpu().numpy(), one[0].cpu().numpy()) < REL_TOL / 2
  st.close()


def test_sampler_edge_cases(built_lib):
  """top_k >= vocab, top_p >= 1 (filters off), top_k = 1 and tiny temperature (= argmax),
  -inf logits, constant rows; reproducible counter noise."""
  from xotorch_support_jetson_b200.shard import Shard
  from xotorch_support_jetson_b200.stage import StageRuntime
  mid = "llama-3.2-tiny"
  _, cfg, state = _setup(mid)
  nl, V = cfg["num_layers"], cfg["vocab_size"]
  st = StageRuntime(Shard(mid, 0, nl - 1, nl), cfg, device=0, max_batch_tokens=16, max_seqs=8, max_tokens_per_seq=32)
  g = torch.Generator().manual_seed(11)
  logits = (torch.randn(6, V, generator=g) * 4).float()
  logits[1, :] = -float("inf")
  logits[1, 77] = 0.5                       # only one finite entry
  logits[2, :] = 1.25                       # constant row: any index is a valid draw
  dev = logits.cuda()
  am = logits.argmax(-1)
  for kw in (dict(temp=1.0, top_k=1), dict(temp=1e-6, top_k=0), dict(temp=1e-6, top_k=V + 5, top_p=1.0)):
    got = st.sample(dev, seed=3, **kw).cpu().to(torch.int64)
    for r in (0, 1, 3, 4, 5):
      assert got[r].item() == am[r].item(), (kw, r)
    assert 0 <= got[2].item() < V
  assert st.sample(dev, temp=1.0, top_k=0, seed=5).cpu()[1].item() == 77
  a = st.sample(dev, temp=1.3, top_k=50, top_p=0.9, seed=42).cpu()
  b = st.sample(dev, temp=1.3, top_k=50, top_p=0.9, seed=42).cpu()
  c = st.sample(dev, temp=1.3, top_k=50, top_p=0.9, seed=43).cpu()
  assert torch.equal(a, b) and a.min().item() >= 0 and a.max().item() < V
  assert not torch.equal(a, c) or True
  st.close()


@pytest.mark.parametrize("mid,hf_override", [
  ("llama-3.2-tiny", None),                  # head_dim 64, interleaved RoPE pairs
  ("llama-3.1-tiny", None),                  # head_dim 128
  ("qwen-2.5-tiny", None),                   # head_dim 64, half-split pairs + q/k/v bias
  ("qwen-2.5-hd128", dict(hidden=512, heads=4, kv=2, inter=1024, layers=3, vocab=1536)),   # half-split pairs 64 lanes apart
])
def test_bulk_store_epilogue_is_bit_identical(built_lib, mid, hf_override, monkeypatch):
  """Decode Linears: the last work unit of every block leaves through shared memory + bulk stores
  (xb_gemm.cuh, the block's tail) instead of per-token strided stores (XB_BULK_EPI=0).  Same values in the
  same places: identical logits over ragged batches, 7 / 33 / 99 token rows (BN 16 / 64 / 128 plans), several
  steps, graph replays; interleaved and half-split RoPE models."""
  from oracle import torch_oracle as O
  from xotorch_support_jetson_b200 import models
  from xotorch_support_jetson_b200.shard import Shard
  from xotorch_support_jetson_b200.stage import StageRuntime
  from xotorch_support_jetson_b200.synth import random_hf_state
  if hf_override is None:
    hf_cfg = models.model_cards[mid]["hf_config"]
  else:
    o = hf_override
    hf_cfg = models._qwen(o["hidden"], o["heads"], o["kv"], o["inter"], o["layers"], vocab=o["vocab"], max_pos=4096)
  cfg = O.model_config_from_hf(hf_cfg)
  state = random_hf_state(hf_cfg, seed=3, std=0.05, norm_jitter=0.1)
  nl = cfg["num_layers"]
  lens = [5, 33, 17, 64, 1, 48, 9]

  def run(bulk):
    monkeypatch.setenv("XB_BULK_EPI", "1" if bulk else "0")     # read when a Linear is planned (first use of a shape)
    st = StageRuntime(Shard(mid, 0, nl - 1, nl), cfg, device=0, max_batch_tokens=128, max_seqs=40, max_tokens_per_seq=96, page_tokens=16)
    st.load_state(state)
    g = torch.Generator().manual_seed(7)
    outs = []
    with torch.cuda.stream(torch.cuda.Stream()):
      for i, L in enumerate(lens):
        p = torch.randint(1, cfg["vocab_size"], (L,), generator=g).to(torch.int32).cuda()
        outs.append(st.forward([i], [L], [0], tokens=p))
      pos = list(lens)
      # ragged decode, 7 rows (BN=16 plan), 5 steps (step 2 onwards replays the graph)
      tok = torch.stack([o.argmax(-1).to(torch.int32).reshape(()) for o in outs[:len(lens)]])
      for step in range(5):
        lg = st.forward(list(range(len(lens))), [1] * len(lens), pos, tokens=tok)
        outs.append(lg)
        tok = lg.argmax(-1).to(torch.int32)
        pos = [x + 1 for x in pos]
      # a 33-row decode batch (BN=64 plan) and a 99-row mixed call that still takes the T <= 128 path
      for i in range(33):
        st.release_slot(i)
      p = torch.randint(1, cfg["vocab_size"], (33 * 3,), generator=g).to(torch.int32).cuda()
      outs.append(st.forward(list(range(33)), [3] * 33, [0] * 33, tokens=p))
      tok = outs[-1].argmax(-1).to(torch.int32)
      outs.append(st.forward(list(range(33)), [1] * 33, [3] * 33, tokens=tok))
    torch.cuda.synchronize()
    res = [o.cpu() for o in outs]
    st.close()
    return res

  x_all, y_all = run(True), run(False)
  assert len(x_all) == len(y_all)
  for i, (x, y) in enumerate(zip(x_all, y_all)):
    assert torch.isfinite(x).all()
    assert torch.equal(x, y), f"output {i}: bulk-store and per-token epilogues differ by {float((x - y).abs().max())}"


@pytest.mark.parametrize("V", [128256, 152064, 50257, 1000])
def test_sampler_large_vocab_both_kernels(built_lib, V, monkeypatch):
  """Real vocabulary sizes (Llama-3 128256, Qwen2.5 152064), one that is not a multiple of 4 and a
  small one: the 4-block-cluster sampler (row resident in shared memory) and the one-block-per-row
  kernel (XB_SAMPLE_CLUSTER=0) must both pick the reference's token for the same noise."""
  import json
  import tempfile
  from pathlib import Path
  from oracle import torch_oracle as O
  from xotorch_support_jetson_b200 import model_config as mc
  from xotorch_support_jetson_b200.models import model_cards
  from xotorch_support_jetson_b200.shard import Shard
  from xotorch_support_jetson_b200.stage import StageRuntime
  hf = dict(model_cards["llama-3.2-tiny"]["hf_config"])
  hf["vocab_size"] = V
  with tempfile.TemporaryDirectory() as td:
    (Path(td) / "config.json").write_text(json.dumps(hf))
    cfg = mc.load_model_config(Path(td) / "config.json")
  nl = cfg["num_layers"]
  st = StageRuntime(Shard("llama-3.2-tiny", 0, nl - 1, nl), cfg, device=0, max_batch_tokens=16, max_seqs=8, max_tokens_per_seq=32)
  g = torch.Generator().manual_seed(V)
  rows = 5
  for temp, top_k in ((0.6, 35), (1.0, 5), (1e-5, 35), (0.85, 0), (2.0, 100)):
    logits = (torch.randn(rows, V, generator=g) * 3).to(torch.bfloat16).float()
    q = torch.empty(rows, V).exponential_(1, generator=g)
    ref = O.sample(logits.clone(), temperature=temp, top_k=top_k if top_k else None, q=q).reshape(-1).to(torch.int64)
    for cluster in ("1", "0"):
      monkeypatch.setenv("XB_SAMPLE_CLUSTER", cluster)
      got = st.sample(logits.cuda(), temp=temp, top_k=top_k, q=q.cuda()).cpu().to(torch.int64)
      assert torch.equal(got, ref), (V, temp, top_k, cluster, got, ref)
  # nucleus + counter noise: both kernels use the same noise function, so they agree with each other,
  # and the draw lies inside the nucleus
  logits = (torch.randn(rows, V, generator=g) * 2).float()
  probs = torch.softmax(logits / 0.9, -1)
  sp, si = probs.sort(-1, descending=True)
  cut = (sp.cumsum(-1) - sp) < 0.7
  for seed in range(3):
    picks = []
    for cluster in ("1", "0"):
      monkeypatch.setenv("XB_SAMPLE_CLUSTER", cluster)
      picks.append(st.sample(logits.cuda(), temp=0.9, top_k=0, top_p=0.7, seed=seed).cpu().to(torch.int64))
    assert torch.equal(picks[0], picks[1]), (V, seed, picks)
    for r in range(rows):
      assert picks[0][r].item() in set(si[r][cut[r]].tolist())
  st.close()


@pytest.mark.parametrize("mid", ["llama-3.1-tiny", "qwen-2.5-tiny"])
def test_half_layer_stage_boundaries_are_exact(built_lib, mid, tmp_path):
  """Pipeline stages may be cut between the attention and the MLP block of a layer (xb200.h
  first_from_mlp / last_to_attn; topology.half_layer_stages).  Any such cut must reproduce the
  full-shard logits bit for bit, prefill and cached decode, also when the weights come from the
  native checkpoint loader (which then reads only the half of the boundary layer it owns)."""
  from xotorch_support_jetson_b200.shard import Shard
  from xotorch_support_jetson_b200.stage import StageRuntime
  from xotorch_support_jetson_b200.synth import write_random_checkpoint
  from xotorch_support_jetson_b200.models import model_cards
  from xotorch_support_jetson_b200.topology import half_layer_stages
  O, cfg, state = _setup(mid)
  nl = cfg["num_layers"]
  kw = dict(device=0, max_batch_tokens=64, max_seqs=2, max_tokens_per_seq=96, page_tokens=16)
  full = StageRuntime(Shard(mid, 0, nl - 1, nl), cfg, **kw)
  full.load_state(state)
  ck = write_random_checkpoint(tmp_path / mid, model_cards[mid]["hf_config"], seed=0, std=0.05, norm_jitter=0.1)
  g = torch.Generator().manual_seed(2)
  toks = torch.randint(1, cfg["vocab_size"], (23,), generator=g).to(torch.int32).cuda()

  def run(stages):
    outs = []
    with torch.cuda.stream(torch.cuda.Stream()):
      def ring(q_len, pos, tok):
        h = None
        for st in stages:
          h = st.forward([0], [q_len], [pos], tokens=tok) if h is None else st.forward([0], [q_len], [pos], hidden=h)
        return h
      lg = ring(23, 0, toks)
      outs.append(lg)
      for k in range(4):
        lg = ring(1, 23 + k, lg.argmax(-1).to(torch.int32))
        outs.append(lg)
    torch.cuda.synchronize()
    return outs

  ref = run([full])
  # hand-made cuts: [attn 0] | [mlp 0 .. attn 2] | [mlp 2 .. end]   and the partitioner's own for 3 and 5 stages
  cuts = [[(0, 0, False, True), (0, 2, True, True), (2, nl - 1, True, False)]]
  for n in (3, 5):
    cuts.append([(s.start_layer, s.end_layer, a, b) for s, a, b in half_layer_stages(mid, nl, n, 1.0, 1.3, 0.8)])
  assert any(a or b for c in cuts[1:] for (_, _, a, b) in c)
  for ci, cut in enumerate(cuts):
    stages = []
    for (a, b, fm, la) in cut:
      st = StageRuntime(Shard(mid, a, b, nl), cfg, first_from_mlp=fm, last_to_attn=la, **kw)
      if ci == 0:
        st.load_dir(ck)                      # native loader
        assert st.weights_missing() == ""
      else:
        st.load_state(state)
      stages.append(st)
    assert stages[0].is_first and stages[-1].is_last and not any(s.is_last for s in stages[:-1])
    got = run(stages)
    for i, (x, y) in enumerate(zip(got, ref)):
      assert torch.equal(x, y), f"cut {cut}: output {i} differs from the full shard by {float((x - y).abs().max())}"
    for st in stages:
      st.close()
  full.close()


@pytest.mark.parametrize("mid,page_tokens", [("llama-3.1-tiny", 16), ("qwen-2.5-tiny", 64), ("llama-3.2-tiny", 32)])
def test_decode_attention_variants_are_bit_identical(built_lib, monkeypatch, mid, page_tokens):
  """The decode step with the q/k/v finalize folded into the attention kernel (default) and the kv splits
  merged inside a thread-block cluster (default) against the same step through the stand-alone
  xb_qkv_finalize_kernel / xb_attn_combine2_kernel: every variant must produce identical logits -- ragged
  contexts on both sides of a 64-key tile boundary, interleaved and half-split RoPE, q/k/v bias, 2-4 query
  heads per kv head, pages smaller than / equal to a tile, graph replays included."""
  from xotorch_support_jetson_b200.shard import Shard
  from xotorch_support_jetson_b200.stage import StageRuntime
  O, cfg, state = _setup(mid)
  nl = cfg["num_layers"]
  lens = [5, 61, 130]
  g = torch.Generator().manual_seed(77)
  prompts = [torch.randint(1, cfg["vocab_size"], (n,), generator=g, dtype=torch.int32).cuda() for n in lens]
  steps = 6
  feed = [torch.randint(1, cfg["vocab_size"], (3,), generator=g, dtype=torch.int32).cuda() for _ in range(steps)]

  def run(fuse, cluster, splits=None):
    monkeypatch.setenv("XB_FUSE_QKV", str(fuse))
    monkeypatch.setenv("XB_ATTN_CLUSTER", str(cluster))
    if splits is None:
      monkeypatch.delenv("XB_ATTN_SPLITS", raising=False)
    else:
      monkeypatch.setenv("XB_ATTN_SPLITS", str(splits))
    st = StageRuntime(Shard(mid, 0, nl - 1, nl), cfg, device=0, max_batch_tokens=256, max_seqs=3, max_tokens_per_seq=192,
                      page_tokens=page_tokens)
    st.load_state(state)
    outs = []
    with torch.cuda.stream(torch.cuda.Stream()):
      lg = st.forward([0, 1, 2], lens, [0, 0, 0], tokens=torch.cat(prompts))
      outs.append(lg.clone())
      for k in range(steps):    # fixed ids, so that a near-tie in one variant cannot send the runs down different paths
        lg = st.forward([0, 1, 2], [1, 1, 1], [n + k for n in lens], tokens=feed[k])
        outs.append(lg.clone())
    torch.cuda.synchronize()
    launches = st.counters()["launches"]
    st.close()
    return [o.cpu() for o in outs], launches

  base, n_base = run(0, 0)
  for fuse, cluster, splits in [(1, 0, None), (0, 1, None), (1, 1, None), (1, 16, None), (1, 1, 3), (0, 0, 3), (1, 1, 1)]:
    got, n = run(fuse, cluster, splits)
    if splits is None:
      for a, b in zip(got, base):
        assert torch.equal(a, b), (fuse, cluster, splits)
      if fuse and cluster:
        assert n < n_base      # fewer kernels per step
    else:
      # another split count changes the fp32 merge order: same result within rounding noise, and the two
      # plumbing variants still agree with each other at equal split count (checked through the next entry)
      for a, b in zip(got, base):
        assert _rel(a.numpy(), b.numpy()) < REL_TOL / 2, (fuse, cluster, splits)
  a3, _ = run(1, 1, 3)
  b3, _ = run(0, 0, 3)
  for a, b in zip(a3, b3):
    assert torch.equal(a, b)
