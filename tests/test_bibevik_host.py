"""Bibevik on the CPU: the configuration reader, sizes taken from the checkpoint, tensor names of a synthetic checkpoint, and the
oracle's own routing (no GPU)."""
import json

import pytest
import torch

import bibevik_oracle as O
from xotorch_support_jetson_b200 import model_config as mc
from xotorch_support_jetson_b200.models import model_cards
from xotorch_support_jetson_b200.synth import bibevik_param_shapes, random_bibevik_state, write_random_checkpoint


def test_registered_models_read_into_layer_descriptions():
  for mid in ("bibevik-tiny", "bibevik-1b"):
    raw = model_cards[mid]["hf_config"]
    cfg = mc.hybrid_model_config(raw)
    assert mc.is_hybrid(cfg) and cfg["block"] == "parallel" and cfg["norm_scalar"] and cfg["num_layers"] == model_cards[mid]["layers"]
    assert cfg["embed_scale"] == pytest.approx(raw["width"] ** 0.5)
    kinds = {l["mixer"] for l in cfg["layers"]}
    assert kinds == {"latent", "gdelta", "lightning"}
    for lay, lc in zip(cfg["layers"], raw["layers"]):
      assert lay["weights_of"] == lc.get("weights_of", -1)
      if lc["mlp"] and lc["mlp"]["kind"] == "moe":
        assert lay["ff_kind"] == "moe" and lay["experts"] == lc["mlp"]["router"]["experts"] and lay["groups"] == lc["mlp"]["router"]["groups"]["count"]
      elif lc["mlp"]:
        assert lay["ff_kind"] == "glu_clamp" and lay["ff_limit"] == lc["mlp"]["limit"]
      else:
        assert lay["ff"] == 0


def test_rank_comes_from_the_checkpoint_when_the_config_leaves_it_out(tmp_path):
  raw = json.loads(json.dumps(model_cards["bibevik-tiny"]["hf_config"]))
  write_random_checkpoint(tmp_path, raw, seed=1)
  for lc in raw["layers"]:
    lc["mixer"].pop("rank", None)
  (tmp_path / "config.json").write_text(json.dumps(raw))
  cfg = mc.load_model_config(tmp_path / "config.json")
  assert [l["rank"] for l in cfg["layers"] if l["mixer"] == "gdelta"] == [8, 8]
  shapes = mc.safetensors_shapes(tmp_path)
  assert shapes["l2.mix.w1"] == (8, raw["width"]) and shapes["final.norm"] == ()
  with pytest.raises(ValueError):
    mc.resolve_tensor_sizes(mc.hybrid_model_config(raw), {})


def test_layers_that_share_tensors_have_none_of_their_own():
  raw = model_cards["bibevik-tiny"]["hf_config"]
  names = bibevik_param_shapes(raw)
  assert not any(n.startswith("l3.") for n in names) and "l1.mlp.e7.down" in names and "l1.mlp.shared.up" in names
  w = random_bibevik_state(raw, seed=0)
  logits, stream = O.forward(raw, w, [1, 2, 3, 4, 5])
  assert logits.shape == (5, raw["vocab"]) and stream.shape == (5, 5, raw["width"]) and bool(torch.isfinite(logits).all())


def test_unknown_kinds_are_refused():
  raw = json.loads(json.dumps(model_cards["bibevik-tiny"]["hf_config"]))
  raw["layers"][0]["type"] = "something"
  with pytest.raises(ValueError):
    mc.hybrid_model_config(raw)
  raw = json.loads(json.dumps(model_cards["bibevik-tiny"]["hf_config"]))
  raw["layers"][0]["mixer"]["decay"] = [0.5]
  with pytest.raises(ValueError):
    mc.hybrid_model_config(raw)


def test_group_limit_changes_the_routing():
  """The oracle's own routing: with groups the chosen experts differ from a plain top-k for a good share of tokens, so a
  router that ignores the groups would not pass test_mechanism_against_oracle."""
  g = torch.Generator().manual_seed(5)
  z = torch.randn(500, 8, generator=g, dtype=torch.float64)
  rt = {"experts": 8, "top": 2, "scale": 1.5, "groups": {"count": 4, "keep": 2}}
  with_groups, wt = O.route(z, rt)
  plain, _ = O.route(z, {"experts": 8, "top": 2, "scale": 1.5})
  differ = sum(set(a.tolist()) != set(b.tolist()) for a, b in zip(with_groups, plain))
  assert differ > 50
  assert torch.allclose(wt, torch.sigmoid(z).gather(1, with_groups) * 1.5)
  for row, ch in zip(z, with_groups):     # both chosen experts lie in the two best groups
    gs = torch.sigmoid(row).reshape(4, 2).sum(-1)
    assert {int(c) // 2 for c in ch} <= set(gs.topk(2).indices.tolist())
