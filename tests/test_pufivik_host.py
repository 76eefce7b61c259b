"""CPU checks of the Pufivik configuration reader, the registry entries, the random checkpoints and the oracle."""
import math

import torch

import pufivik_oracle as O
from xotorch_support_jetson_b200.model_config import hybrid_model_config, is_hybrid, load_model_config
from xotorch_support_jetson_b200.models import model_cards
from xotorch_support_jetson_b200.synth import pufivik_param_shapes, random_pufivik_state, write_random_checkpoint


def test_config_reader_maps_every_constant():
  raw = model_cards["pufivik-tiny"]["hf_config"]
  cfg = hybrid_model_config(raw)
  assert is_hybrid(cfg) and cfg["block"] == "sandwich" and cfg["tied_head"] and cfg["norm_plain"] and cfg["ff_unfiltered"]
  assert cfg["norm_groups"] == raw["norm"]["groups"] and cfg["taps"] == raw["canon"]["taps"]
  assert cfg["residual_mult"] == raw["residual_mult"] and cfg["embed_scale"] == raw["embedding"]["scale"]
  a, b = cfg["layers"][0], cfg["layers"][1]
  assert a["mixer"] == "softmax" and a["sink"] and a["talk"] and a["gate"] and a["softcap"] == 0.0
  assert a["rot_pairs"] == "half" and a["rot_scaling"] == "bands" and a["rot_mult"] == 1.0
  sc = raw["layers"][0]["mixer"]["rot"]["scaling"]
  assert (a["rot_factor"], a["rot_orig"], a["rot_p0"], a["rot_p1"]) == (sc["factor"], sc["original"], sc["low"], sc["high"])
  assert a["ff_kind"] == "moe" and a["ff_act"] == "swiglu" and a["route_input"] and a["top"] == 2
  assert not (b["sink"] or b["talk"] or b["gate"]) and b["softcap"] == raw["layers"][1]["mixer"]["softcap"]
  assert b["rot_pairs"] == "interleaved" and b["rot_scaling"] == "ramp" and b["ff"] == 0
  assert abs(b["rot_mult"] - (0.1 * math.log(raw["layers"][1]["mixer"]["rot"]["scaling"]["factor"]) + 1.0)) < 1e-12
  assert cfg["layers"][2]["v_mix"] is False


def test_checkpoint_on_disk_round_trip(tmp_path):
  raw = model_cards["pufivik-tiny"]["hf_config"]
  p = write_random_checkpoint(tmp_path / "m", raw, seed=1)
  cfg = load_model_config(p / "config.json")
  assert cfg["architecture"] == "Pufivik" and cfg["num_layers"] == len(raw["layers"])
  sh = pufivik_param_shapes(raw)
  assert "head" not in sh and "l1.norm2" not in sh and "l1.mix.sink" not in sh and "l2.mix.vmix" not in sh and sh["l0.mix.vmix"] == ()
  w = random_pufivik_state(raw, seed=1)
  assert set(w) == set(sh) and all(tuple(w[k].shape) == tuple(v) for k, v in sh.items())


def test_oracle_pieces():
  torch.manual_seed(0)
  x = torch.randn(3, 12, dtype=torch.float64)
  y = O.group_norm(x, torch.ones(12, dtype=torch.float64), 3, 0.0)
  assert torch.allclose((y.reshape(3, 3, 4) ** 2).mean(-1), torch.ones(3, 3, dtype=torch.float64))
  # a filter whose last tap is 1 doubles the input; the first tap reads taps - 1 steps back
  w = torch.zeros(12, 3, dtype=torch.float64)
  w[:, 0] = 1.0
  f = O.causal_filter(x, w)
  assert torch.allclose(f[2], x[2] + x[0]) and torch.allclose(f[1], x[1])
  # rotation keeps the length of each pair (times the multiplier) and leaves the rest alone, in both layouts
  q = torch.randn(2, 2, 10, dtype=torch.float64)
  for inter in (False, True):
    r = O.rotate(q, [5, 9], [1.0, 0.3, 0.01], 1.2, 6, inter)
    assert torch.allclose(r[..., 6:], q[..., 6:])
    assert torch.allclose((r[..., :6] ** 2).sum(-1), 1.44 * (q[..., :6] ** 2).sum(-1))
  # weights with a sink sum to less than one; the sink's share is exp(sink) over the denominator
  k = torch.randn(4, 1, 5, dtype=torch.float64)
  qq = torch.randn(4, 2, 5, dtype=torch.float64)
  wts = O.attention_weights(qq, k, 0.5, 0.0, torch.tensor([0.0, 2.0], dtype=torch.float64))
  assert abs(float(wts[0, 0, 0]) - 1.0 / (1.0 + math.exp(0.0 - float(k[0, 0] @ qq[0, 0]) * 0.5))) < 1e-12
  assert (wts.sum(-1) < 1.0).all() and float(wts[0, 0, 1:].abs().sum()) == 0.0
  # band frequencies: short waves kept, long ones divided
  fs, m = O.band_frequencies({"base": 10000.0, "dims": 32, "scaling": {"factor": 4.0, "low": 1.0, "high": 8.0, "original": 256}})
  assert m == 1.0 and fs[0] == 1.0 and abs(fs[-1] - 10000.0 ** (-30 / 32) / 4.0) < 1e-18
  fr, m2 = O.ramp_frequencies({"base": 10000.0, "dims": 32, "scaling": {"factor": 16.0, "fast": 32.0, "slow": 1.0, "original": 512}})
  assert abs(m2 - (0.1 * math.log(16.0) + 1.0)) < 1e-15 and fr[0] == 1.0 and abs(fr[-1] - 10000.0 ** (-30 / 32) / 16.0) < 1e-18
