"""CPU checks of the Vusenex configuration reader, the registry entries, the random checkpoints and the oracle."""
import math

import numpy as np
import pytest
import torch

import vusenex_oracle as O
from xotorch_support_jetson_b200.model_config import hybrid_model_config, is_hybrid, load_model_config
from xotorch_support_jetson_b200.models import model_cards
from xotorch_support_jetson_b200.synth import random_vusenex_state, vusenex_param_shapes, write_random_checkpoint


def test_config_reader_maps_every_constant():
  raw = model_cards["vusenex-tiny"]["hf_config"]
  cfg = hybrid_model_config(raw)
  assert is_hybrid(cfg) and cfg["block"] == "branchnorm" and cfg["norm_scalar"] and cfg["gated_residual"]
  assert cfg["pos_rows"] == cfg["max_seq_len"] == raw["max_positions"] and cfg["norm_eps"] == raw["norm"]["eps"]
  assert cfg["bigram"] == raw["embedding"]["bigram"]
  lat, att, bare = cfg["layers"][0], cfg["layers"][1], cfg["layers"][2]
  m0, m1 = raw["layers"][0]["mixer"], raw["layers"][1]["mixer"]
  assert lat["mixer"] == "latent" and lat["rot_dim"] == 0 and lat["rot_dims"] == 0
  assert (lat["heads"], lat["dim"], lat["vdim"], lat["kv_rank"], lat["scale"]) == (m0["heads"], m0["dim"], m0["vdim"], m0["kv_rank"], m0["scale"])
  assert att["mixer"] == "softmax" and att["sink"] == "unit" and att["qkv_bias"] and att["qk_norm"] and att["v_is_k"] and att["dist_bias"]
  assert att["rot_dims"] == 0 and not (att["talk"] or att["gate"] or att["v_mix"]) and att["softcap"] == 0.0
  assert (att["heads"], att["kv_heads"], att["dim"], att["vdim"], att["scale"]) == (m1["heads"], m1["kv_heads"], m1["dim"], m1["dim"], m1["scale"])
  assert (att["qtemp_coef"], att["qtemp_every"]) == (m1["q_temp"]["coef"], m1["q_temp"]["every"])
  r0 = raw["layers"][0]["mlp"]
  assert lat["ff_kind"] == "moe" and lat["ff_act"] == "gelu" and not lat["route_input"] and lat["route_norm"]
  assert lat["route_score"] == "softmax" and lat["group_score"] == "max" and lat["route_scale"] == 1.0
  assert (lat["ff"], lat["experts"], lat["top"], lat["groups"], lat["keep_groups"], lat["shared_ff"]) == \
         (r0["expert"]["ff"], r0["router"]["experts"], r0["router"]["top"], r0["router"]["groups"]["count"], r0["router"]["groups"]["keep"], r0["shared"]["ff"])
  assert att["shared_ff"] == 0 and bare["ff"] == 0 and bare["ff_kind"] == "none"


def test_reader_refuses_values_of_another_size_and_unknown_kinds():
  raw = model_cards["vusenex-tiny"]["hf_config"]
  bad = {**raw, "layers": [{**raw["layers"][1], "mixer": {**raw["layers"][1]["mixer"], "vdim": 8}}]}
  with pytest.raises(ValueError):
    hybrid_model_config(bad)
  with pytest.raises(ValueError):
    hybrid_model_config({**raw, "layers": [{**raw["layers"][0], "type": "convolution"}]})
  with pytest.raises(ValueError):
    hybrid_model_config({**raw, "layers": [{**raw["layers"][0], "mlp": {"kind": "dense", "ff": 8}}]})
  # a model without optional parts: no query temperature, no groups, no shared expert
  lean = {**raw, "layers": [{"type": "attention", "mixer": {"heads": 2, "kv_heads": 2, "dim": 8, "vdim": 8, "scale": 0.3},
                             "mlp": {"kind": "moe", "expert": {"ff": 8}, "router": {"experts": 4, "top": 1}}}]}
  lay = hybrid_model_config(lean)["layers"][0]
  assert lay["qtemp_every"] == 0 and lay["groups"] == 0 and lay["shared_ff"] == 0


def test_checkpoint_on_disk_round_trip(tmp_path):
  raw = model_cards["vusenex-tiny"]["hf_config"]
  p = write_random_checkpoint(tmp_path / "m", raw, seed=1)
  cfg = load_model_config(p / "config.json")
  assert cfg["architecture"] == "Vusenex" and cfg["num_layers"] == len(raw["layers"])
  assert cfg["pos_rows"] == raw["max_positions"]          # taken from the position table's rows
  sh = vusenex_param_shapes(raw)
  assert sh["l0.norm1"] == () and sh["final.norm"] == () and "l2.norm2" not in sh and "l2.rg2" not in sh and "l1.mlp.shared.up" not in sh
  assert sh["bigram"] == (raw["embedding"]["bigram"]["buckets"] + 1, raw["width"]) and sh["pos"] == (raw["max_positions"], raw["width"])
  assert "l1.mix.v" not in sh and "l0.mix.k" not in sh and sh["l1.mix.q.norm"] == (6 * 40,) and sh["l1.mix.k.norm"] == (3 * 40,)
  w = random_vusenex_state(raw, seed=1)
  assert set(w) == set(sh) and all(tuple(w[k].shape) == tuple(v) for k, v in sh.items())
  for mid in ("vusenex-tiny", "vusenex-1b"):
    c = hybrid_model_config(model_cards[mid]["hf_config"])
    assert c["num_layers"] == model_cards[mid]["layers"]


def test_oracle_pieces():
  rng = np.random.default_rng(0)
  y = O.unit(rng.standard_normal((3, 12)), 0.0)
  assert np.allclose((y ** 2).mean(-1), 1.0)
  assert abs(float(O.gelu_erf(np.array([1.0]))[0]) - 0.5 * (1.0 + math.erf(1.0 / math.sqrt(2.0)))) < 1e-15
  # routing: the best expert sits in a group that loses on its best score; weights sum to one over the chosen experts
  z = np.log(np.array([0.30, 0.01, 0.28, 0.27, 0.05, 0.09]))
  got = O.route(z, top=2, groups=3, keep=1)
  assert sorted(got) == [0, 1] and abs(sum(got.values()) - 1.0) < 1e-12 and abs(got[0] / got[1] - 30.0) < 1e-9
  got = O.route(z, top=2, groups=3, keep=2)
  assert sorted(got) == [0, 2] and abs(got[0] / got[2] - 0.30 / 0.28) < 1e-9
  assert sorted(O.route(z, top=3, groups=0, keep=0)) == [0, 2, 3]
  # embedding: the first token takes the table's last row, later ones the hashed row of the pair
  cfg = {"embedding": {"bigram": {"buckets": 7, "mul_prev": 3, "mul_cur": 2}}}
  st = {"embed": torch.zeros(10, 4), "bigram": torch.arange(8.0).reshape(8, 1).repeat(1, 4), "pos": torch.zeros(5, 4)}
  x = O.embed_rows(st, cfg, [4, 9, 1])
  assert x[:, 0].tolist() == [7.0, float((4 * 3 + 9 * 2) % 7), float((9 * 3 + 1 * 2) % 7)]
  # attention: one token sees itself with weight e^s / (1 + e^s); the value is the key as projected, before its norm
  D, dk = 6, 4
  g = torch.Generator().manual_seed(1)
  st = {"p.q": torch.randn(dk, D, generator=g), "p.q.b": torch.randn(dk, generator=g), "p.k": torch.randn(dk, D, generator=g),
        "p.k.b": torch.randn(dk, generator=g), "p.q.norm": torch.ones(dk), "p.k.norm": torch.ones(dk), "p.r1": torch.ones(1),
        "p.r2": torch.ones(1), "p.o": torch.eye(dk)}
  mx = {"heads": 1, "kv_heads": 1, "dim": dk, "scale": 0.7, "q_temp": {"coef": 0.5, "every": 1}}
  xr = rng.standard_normal((1, D))
  out = O.softmax_attention(st, "p.", mx, xr, 0.0)
  q = xr @ st["p.q"].double().numpy().T + st["p.q.b"].double().numpy()
  k = xr @ st["p.k"].double().numpy().T + st["p.k.b"].double().numpy()
  s = float(O.unit(q, 0.0)[0] @ O.unit(k, 0.0)[0]) * 0.7 * (1.0 + 0.5 * math.log(2.0))
  assert np.allclose(out, math.exp(s) / (1.0 + math.exp(s)) * k)
