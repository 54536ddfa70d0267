"""Host-side pieces of the Refatar design that need no GPU: the config reader, the registry cards, the checkpoint
shapes, the oracle's own mask, and the trace runner's refusal of float32 for families without it."""
import json

import pytest
import torch

import refatar_oracle as O


def test_config_reader_takes_every_size_from_the_file():
  from xotorch_support_jetson_b200.model_config import hybrid_model_config, is_hybrid, load_model_config  # noqa: F401
  from xotorch_support_jetson_b200.models import model_cards
  raw = model_cards["refatar-tiny"]["hf_config"]
  c = hybrid_model_config(raw)
  assert is_hybrid(c) and c["num_layers"] == len(raw["layers"]) and c["embed_dim"] == raw["width"] and c["vocab_size"] == raw["vocab"]
  assert [l["mixer"] for l in c["layers"]] == [l["type"] for l in raw["layers"]]
  assert c["layers"][2]["ff"] == 0 and c["layers"][0]["ff"] == raw["layers"][0]["mlp"]["ff"]
  assert c["layers"][1]["left"]["window"] == raw["layers"][1]["mixer"]["left"]["mask"]["size"]
  assert c["taps"] == raw["canon"]["taps"] and c["side_dim"] == raw["token_side"]["dim"]
  bare = {k: v for k, v in raw.items() if k not in ("canon", "token_side", "logit_softcap")}
  b = hybrid_model_config(bare)
  assert b["taps"] == 0 and b["side_dim"] == 0 and b["logit_softcap"] == 0.0
  with pytest.raises(ValueError):
    hybrid_model_config(dict(raw, layers=[dict(raw["layers"][0], type="other")]))
  with pytest.raises(ValueError):
    hybrid_model_config(dict(raw, architecture="Else"))


def test_checkpoint_shapes_and_oracle_run_on_the_registered_cards(tmp_path):
  from xotorch_support_jetson_b200.model_config import load_model_config
  from xotorch_support_jetson_b200.models import model_cards
  from xotorch_support_jetson_b200.synth import random_refatar_state, refatar_param_shapes, write_random_checkpoint
  raw = model_cards["refatar-tiny"]["hf_config"]
  w = random_refatar_state(raw, seed=1)
  assert {k: tuple(v.shape) for k, v in w.items()} == refatar_param_shapes(raw)
  assert w["side.embed"].shape[1] == raw["token_side"]["dim"] * len(raw["layers"])
  p = write_random_checkpoint(tmp_path / "m", raw, seed=1)
  assert load_model_config(p / "config.json")["family"] == "hybrid"
  assert json.loads((p / "config.json").read_text())["architecture"] == "Refatar"
  logits = O.forward(raw, w, [1, 2, 3, 4, 5, 6, 7])
  assert logits.shape == (7, raw["vocab"]) and torch.isfinite(logits).all()
  assert float(logits.abs().max()) <= raw["logit_softcap"]
  # causality of the restatement: a later token changes nothing before it
  again = O.forward(raw, w, [1, 2, 3, 4, 9, 6, 7])
  assert torch.equal(again[:4], logits[:4]) and not torch.equal(again[4:], logits[4:])


def test_oracle_window_mask():
  m = O.window_mask(10, 3, 2)
  assert m[9].tolist() == [True, True, False, False, False, False, False, True, True, True]
  assert m[2].tolist() == [True, True, True] + [False] * 7
  assert O.window_mask(4, 1, 0).tolist() == torch.eye(4, dtype=torch.bool).tolist()


def test_trace_runner_refuses_float32_for_a_bfloat16_only_family(tmp_path):
  from xotorch_support_jetson_b200.models import model_cards
  from xotorch_support_jetson_b200.trace_run import main
  (tmp_path / "config.json").write_text(json.dumps(model_cards["llama-3.2-tiny"]["hf_config"]))
  assert main(["--model", str(tmp_path), "--dtype", "float32", "--out", str(tmp_path / "o")]) == 3
