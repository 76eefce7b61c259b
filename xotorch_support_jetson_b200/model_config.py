"""HF config.json -> the engine's model description.

Same field mapping and the same quirks as the reference's ``load_model_config``
(``xotorch/inference/torch/models/llm_utils.py:30-77``): ``rope_scaling_factor`` is read
from the key ``"rope_factor"`` with default 32, so Llama-3.1 runs with factor 32 like the
reference does.  Family / tied-head detection by model-id
substring follows ``general_mha.py:33-63``.
"""
import json
import math
import os
from pathlib import Path

import torch

HF_PRECISION_STR_TO_DTYPE = {
  "float16": torch.float16, "bfloat16": torch.bfloat16, "float32": torch.float32, "float64": torch.float64,
}


# HF config.json key -> engine key, for the fields that are copied as they are
_DIRECT_FIELDS = (
  ("hidden_size", "embed_dim"), ("num_attention_heads", "num_heads"), ("num_key_value_heads", "num_kv_heads"),
  ("max_position_embeddings", "max_seq_len"), ("intermediate_size", "intermediate_dim"), ("rms_norm_eps", "norm_eps"),
  ("rope_theta", "rope_base"), ("vocab_size", "vocab_size"), ("num_hidden_layers", "num_layers"),
)
# optional HF keys with the defaults the reference applies
_OPTIONAL_FIELDS = (("attention_dropout", "attn_dropout", 0.0), ("attention_bias", "attn_bias", False), ("hidden_act", "hidden_act", "silu"))


HYBRID_ARCHITECTURES = ("Refatar", "Bibevik", "Pufivik", "Vusenex")


def is_hybrid(config: dict) -> bool:
  """True for configs of per-layer-described models (``hybrid_model_config``), which run on the hybrid engine."""
  return config.get("family") == "hybrid"


def hybrid_model_config(raw: dict) -> dict:
  """A Refatar ``config.json`` (``architecture``, ``width``, ``vocab``, ``layers`` [{type, mixer, mlp}], ``norm.eps``,
  optional ``canon.taps``, ``token_side.dim``, ``logit_softcap``) -> the engine's dict.  Every size and constant comes from
  the file; what the file does not mention is switched off.  The keys the Llama-shaped path uses (``embed_dim``,
  ``vocab_size``, ``num_layers``, ``max_seq_len``) are filled so that the serving code above the stage needs no branch.

  Layer kinds: ``delta`` = gated delta rule {heads, kv_heads, dim, vdim, conv}; ``parallel`` = {left: windowed softmax
  attention {heads, kv_heads, dim, vdim, scale, mask{size, keep_first}}, right: HGRN2 {heads, dim, vdim}, left_scale,
  right_scale}; ``mlp`` = {kind: dense, ff} or null."""
  arch = raw.get("architecture")
  if arch not in HYBRID_ARCHITECTURES:
    raise ValueError(f"unknown architecture {arch!r}")
  if arch == "Bibevik":
    return bibevik_model_config(raw)
  if arch == "Pufivik":
    return pufivik_model_config(raw)
  if arch == "Vusenex":
    return vusenex_model_config(raw)
  layers = []
  for i, lc in enumerate(raw["layers"]):
    mx, kind = lc["mixer"], lc["type"]
    if kind == "delta":
      lay = {"mixer": "delta", "heads": int(mx["heads"]), "kv_heads": int(mx["kv_heads"]), "dim": int(mx["dim"]),
             "vdim": int(mx["vdim"]), "taps": int(mx["conv"])}
    elif kind == "parallel":
      le, ri = mx["left"], mx["right"]
      lay = {"mixer": "parallel",
             "left": {"heads": int(le["heads"]), "kv_heads": int(le["kv_heads"]), "dim": int(le["dim"]), "vdim": int(le["vdim"]),
                      "scale": float(le["scale"]), "window": int(le["mask"]["size"]), "keep_first": int(le["mask"]["keep_first"])},
             "right": {"heads": int(ri["heads"]), "dim": int(ri["dim"]), "vdim": int(ri["vdim"])},
             "left_scale": float(mx["left_scale"]), "right_scale": float(mx["right_scale"])}
    else:
      raise ValueError(f"layer {i}: unknown layer type {kind!r}")
    mlp = lc.get("mlp")
    if mlp is not None and mlp.get("kind", "dense") != "dense":
      raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
    lay["ff"] = int(mlp["ff"]) if mlp is not None else 0
    layers.append(lay)
  canon, side = raw.get("canon"), raw.get("token_side")
  return {
    "family": "hybrid", "architecture": arch,
    "embed_dim": int(raw["width"]), "vocab_size": int(raw["vocab"]), "num_layers": len(layers),
    "max_seq_len": int(raw.get("max_seq_len", 1 << 20)), "norm_eps": float(raw["norm"]["eps"]),
    "taps": int(canon["taps"]) if canon else 0, "side_dim": int(side["dim"]) if side else 0,
    "logit_softcap": float(raw.get("logit_softcap") or 0.0), "layers": layers,
    "torch_dtype": HF_PRECISION_STR_TO_DTYPE.get(raw.get("torch_dtype", "bfloat16"), torch.bfloat16),
  }


def _gated_ff(i: int, mlp) -> dict:
  """The feed-forward part of a parallel-block layer: none, a clamped gated one with biases, or experts of that form."""
  if mlp is None:
    return {"ff": 0, "ff_kind": "none"}
  if mlp["kind"] == "dense":
    return {"ff": int(mlp["ff"]), "ff_kind": "glu_clamp", "ff_limit": float(mlp["limit"])}
  if mlp["kind"] == "moe":
    rt, ex, sh = mlp["router"], mlp["expert"], mlp.get("shared")
    gr = rt.get("groups")
    return {"ff": int(ex["ff"]), "ff_kind": "moe", "ff_limit": float(ex["limit"]), "experts": int(rt["experts"]), "top": int(rt["top"]),
            "groups": int(gr["count"]) if gr else 0, "keep_groups": int(gr["keep"]) if gr else 0, "route_scale": float(rt["scale"]),
            "shared_ff": int(sh["ff"]) if sh else 0, "shared_limit": float(sh["limit"]) if sh else 0.0}
  raise ValueError(f"layer {i}: unknown feed-forward kind {mlp['kind']!r}")


def bibevik_model_config(raw: dict) -> dict:
  """A Bibevik ``config.json`` (``width``, ``vocab``, ``embedding.scale``, ``norm.eps``, ``layers`` [{type, mixer, mlp,
  weights_of?}]) -> the engine's dict.  Layers are parallel blocks (one norm of a single number; mixer and feed-forward read
  it and their sum joins the stream).  Mixer kinds: ``latent_attention`` {heads, dim, rot_dim, vdim, kv_rank, scale, rot{base,
  dims}}, ``general_delta`` {heads, dim} (the rank of the decay's first projection comes from the checkpoint's ``w1`` shape,
  see ``StageRuntime``; the config may name it as ``rank``), ``lightning`` {heads, dim, vdim, decay[heads]}.  A layer with
  ``weights_of: j`` uses layer j's tensors."""
  layers = []
  for i, lc in enumerate(raw["layers"]):
    mx, kind = lc["mixer"], lc["type"]
    if kind == "latent_attention":
      rot = mx.get("rot") or {}
      lay = {"mixer": "latent", "heads": int(mx["heads"]), "dim": int(mx["dim"]), "rot_dim": int(mx["rot_dim"]), "vdim": int(mx["vdim"]),
             "kv_rank": int(mx["kv_rank"]), "scale": float(mx["scale"]), "rot_base": float(rot.get("base", 10000.0)),
             "rot_dims": int(rot.get("dims", mx["rot_dim"]))}
    elif kind == "general_delta":
      lay = {"mixer": "gdelta", "heads": int(mx["heads"]), "dim": int(mx["dim"]), "rank": int(mx.get("rank", 0))}
    elif kind == "lightning":
      lay = {"mixer": "lightning", "heads": int(mx["heads"]), "dim": int(mx["dim"]), "vdim": int(mx["vdim"]),
             "decay": [float(v) for v in mx["decay"]]}
      if len(lay["decay"]) != lay["heads"]:
        raise ValueError(f"layer {i}: {len(lay['decay'])} decays for {lay['heads']} heads")
    else:
      raise ValueError(f"layer {i}: unknown layer type {kind!r}")
    lay.update(_gated_ff(i, lc.get("mlp")))
    lay["weights_of"] = int(lc["weights_of"]) if lc.get("weights_of") is not None else -1
    layers.append(lay)
  return {
    "family": "hybrid", "architecture": "Bibevik", "block": "parallel", "norm_scalar": True,
    "embed_scale": float((raw.get("embedding") or {}).get("scale", 1.0)),
    "embed_dim": int(raw["width"]), "vocab_size": int(raw["vocab"]), "num_layers": len(layers),
    "max_seq_len": int(raw.get("max_seq_len", 1 << 20)), "norm_eps": float(raw["norm"]["eps"]),
    "taps": 0, "side_dim": 0, "logit_softcap": 0.0, "layers": layers,
    "torch_dtype": HF_PRECISION_STR_TO_DTYPE.get(raw.get("torch_dtype", "bfloat16"), torch.bfloat16),
  }


def _rotary(i: int, rot, kind: str) -> dict:
  """The rotary part of a Pufivik mixer: how many entries of a head turn, the pair layout and the rescaling of the
  frequencies.  ``attention`` pairs entry i with i + dims/2 and rescales in wavelength bands {factor, low, high, original};
  ``attention_2`` pairs 2i with 2i + 1 and rescales along a ramp over the pair index {factor, original, fast, slow}, with
  cos and sin multiplied by 0.1 ln(factor) + 1."""
  if not rot or not int(rot.get("dims", 0)):
    return {"rot_dims": 0, "rot_pairs": "half", "rot_scaling": "none", "rot_base": 10000.0, "rot_mult": 1.0,
            "rot_factor": 1.0, "rot_orig": 1.0, "rot_p0": 0.0, "rot_p1": 0.0}
  out = {"rot_dims": int(rot["dims"]), "rot_base": float(rot["base"]), "rot_pairs": "half" if kind == "attention" else "interleaved",
         "rot_scaling": "none", "rot_mult": 1.0, "rot_factor": 1.0, "rot_orig": 1.0, "rot_p0": 0.0, "rot_p1": 0.0}
  sc = rot.get("scaling")
  if sc and kind == "attention":
    out.update(rot_scaling="bands", rot_factor=float(sc["factor"]), rot_orig=float(sc["original"]), rot_p0=float(sc["low"]),
               rot_p1=float(sc["high"]))
  elif sc:
    out.update(rot_scaling="ramp", rot_factor=float(sc["factor"]), rot_orig=float(sc["original"]), rot_p0=float(sc["fast"]),
               rot_p1=float(sc["slow"]), rot_mult=0.1 * math.log(float(sc["factor"])) + 1.0)
  return out


def pufivik_model_config(raw: dict) -> dict:
  """A Pufivik ``config.json`` (``width``, ``vocab``, ``embedding.scale``, ``residual_mult``, ``norm`` {eps, groups},
  ``canon.taps``, ``layers`` [{type, mixer, mlp}]) -> the engine's dict.  Layers are sandwich blocks with plain norm weights,
  norms in groups, a residual multiplier, a causal filter in front of the mixer only and a tied head.  Both layer types are
  rotary-position softmax attention {heads, kv_heads, dim, vdim, scale, rot{base, dims, scaling}, v_mix}: ``attention`` adds a
  sink per head, mixed heads and a sigmoid gate per head; ``attention_2`` a soft cap on the scores.  ``mlp``: null or experts
  {expert{ff}, router{experts, top}} of the SiLU-gated form whose routing weight (the sigmoid score, not renormalised)
  multiplies the expert's input."""
  layers = []
  for i, lc in enumerate(raw["layers"]):
    mx, kind = lc["mixer"], lc["type"]
    if kind not in ("attention", "attention_2"):
      raise ValueError(f"layer {i}: unknown layer type {kind!r}")
    first = kind == "attention"
    lay = {"mixer": "softmax", "heads": int(mx["heads"]), "kv_heads": int(mx["kv_heads"]), "dim": int(mx["dim"]), "vdim": int(mx["vdim"]),
           "scale": float(mx["scale"]), "softcap": 0.0 if first else float(mx.get("softcap") or 0.0),
           "sink": first, "talk": first, "gate": first, "v_mix": bool(mx.get("v_mix", False))}
    lay.update(_rotary(i, mx.get("rot"), kind))
    mlp = lc.get("mlp")
    if mlp is None:
      lay.update({"ff": 0, "ff_kind": "none"})
    elif mlp.get("kind", "moe") == "moe":
      lay.update({"ff": int(mlp["expert"]["ff"]), "ff_kind": "moe", "ff_act": "swiglu", "route_input": True, "ff_limit": 0.0,
                  "experts": int(mlp["router"]["experts"]), "top": int(mlp["router"]["top"]), "groups": 0, "keep_groups": 0,
                  "route_scale": 1.0, "shared_ff": 0, "shared_limit": 0.0})
    else:
      raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
    layers.append(lay)
  canon, norm = raw.get("canon"), raw["norm"]
  return {
    "family": "hybrid", "architecture": "Pufivik", "block": "sandwich", "norm_plain": True, "tied_head": True, "ff_unfiltered": True,
    "norm_groups": int(norm.get("groups", 1)), "residual_mult": float(raw.get("residual_mult", 1.0)),
    "embed_scale": float((raw.get("embedding") or {}).get("scale", 1.0)),
    "embed_dim": int(raw["width"]), "vocab_size": int(raw["vocab"]), "num_layers": len(layers),
    "max_seq_len": int(raw.get("max_seq_len", 1 << 20)), "norm_eps": float(norm["eps"]),
    "taps": int(canon["taps"]) if canon else 0, "side_dim": 0, "logit_softcap": 0.0, "layers": layers,
    "torch_dtype": HF_PRECISION_STR_TO_DTYPE.get(raw.get("torch_dtype", "bfloat16"), torch.bfloat16),
  }


def vusenex_model_config(raw: dict) -> dict:
  """A Vusenex ``config.json`` (``width``, ``vocab``, ``max_positions``, ``embedding.bigram`` {buckets, mul_prev, mul_cur},
  ``norm.eps``, ``layers`` [{type, mixer, mlp}]) -> the engine's dict.  Layers are branch-norm blocks: a sublayer reads the
  stream itself, its output is gated by a sigmoid of the stream, RMS-normed with a single number and added.  The embedding is
  the token row plus a hashed row of the (previous, current) token pair plus a learned position row.  Mixer kinds:
  ``attention`` {heads, kv_heads, dim, vdim, scale, q_temp{coef, every}} = grouped-query softmax attention without rotation
  whose values are the projected keys, with q / k biases, whole-projection q / k norms, a query temperature, a logarithmic
  distance penalty per head and one extra unit in the softmax denominator; ``latent_attention`` {heads, dim, vdim, kv_rank,
  scale} = attention over a cached latent without a rotated part.  ``mlp``: null or experts {expert{ff}, router{experts, top,
  groups{count, keep}}, shared{ff}} of the ungated erf-GELU form with softmax scores, groups worth their best score and
  weights renormalised over the chosen experts."""
  layers = []
  for i, lc in enumerate(raw["layers"]):
    mx, kind = lc["mixer"], lc["type"]
    if kind == "attention":
      if int(mx.get("vdim", mx["dim"])) != int(mx["dim"]):
        raise ValueError(f"layer {i}: values are the projected keys, so vdim {mx['vdim']} must equal dim {mx['dim']}")
      qt = mx.get("q_temp") or {}
      lay = {"mixer": "softmax", "heads": int(mx["heads"]), "kv_heads": int(mx["kv_heads"]), "dim": int(mx["dim"]), "vdim": int(mx["dim"]),
             "scale": float(mx["scale"]), "softcap": 0.0, "sink": "unit", "talk": False, "gate": False, "v_mix": False,
             "qkv_bias": True, "qk_norm": True, "v_is_k": True, "dist_bias": True,
             "qtemp_coef": float(qt.get("coef", 0.0)), "qtemp_every": int(qt.get("every", 0))}
      lay.update(_rotary(i, None, kind))
    elif kind == "latent_attention":
      lay = {"mixer": "latent", "heads": int(mx["heads"]), "dim": int(mx["dim"]), "rot_dim": 0, "vdim": int(mx["vdim"]),
             "kv_rank": int(mx["kv_rank"]), "scale": float(mx["scale"]), "rot_base": 10000.0, "rot_dims": 0}
    else:
      raise ValueError(f"layer {i}: unknown layer type {kind!r}")
    mlp = lc.get("mlp")
    if mlp is None:
      lay.update({"ff": 0, "ff_kind": "none"})
    elif mlp.get("kind", "moe") == "moe":
      rt, sh = mlp["router"], mlp.get("shared")
      gr = rt.get("groups")
      lay.update({"ff": int(mlp["expert"]["ff"]), "ff_kind": "moe", "ff_act": "gelu", "route_input": False, "ff_limit": 0.0,
                  "experts": int(rt["experts"]), "top": int(rt["top"]), "groups": int(gr["count"]) if gr else 0,
                  "keep_groups": int(gr["keep"]) if gr else 0, "route_scale": 1.0, "route_score": "softmax", "group_score": "max",
                  "route_norm": True, "shared_ff": int(sh["ff"]) if sh else 0, "shared_limit": 0.0})
    else:
      raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
    lay["weights_of"] = -1
    layers.append(lay)
  bg = (raw.get("embedding") or {}).get("bigram")
  return {
    "family": "hybrid", "architecture": "Vusenex", "block": "branchnorm", "norm_scalar": True, "gated_residual": True,
    "bigram": {"buckets": int(bg["buckets"]), "mul_prev": int(bg["mul_prev"]), "mul_cur": int(bg["mul_cur"])} if bg else None,
    "pos_rows": int(raw["max_positions"]), "embed_scale": 1.0,
    "embed_dim": int(raw["width"]), "vocab_size": int(raw["vocab"]), "num_layers": len(layers),
    "max_seq_len": int(raw["max_positions"]), "norm_eps": float(raw["norm"]["eps"]),
    "taps": 0, "side_dim": 0, "logit_softcap": 0.0, "layers": layers,
    "torch_dtype": HF_PRECISION_STR_TO_DTYPE.get(raw.get("torch_dtype", "bfloat16"), torch.bfloat16),
  }


def safetensors_shapes(folder: Path) -> dict:
  """name -> shape of every tensor in the ``*.safetensors`` files of a folder, from the files' headers alone (8 bytes of
  little-endian length, then that many bytes of JSON)."""
  import struct
  shapes = {}
  for f in sorted(Path(folder).glob("*.safetensors")):
    with open(f, "rb") as fh:
      (n,) = struct.unpack("<Q", fh.read(8))
      header = json.loads(fh.read(n))
    shapes.update({k: tuple(v["shape"]) for k, v in header.items() if k != "__metadata__"})
  return shapes


def resolve_tensor_sizes(cfg: dict, shapes: dict) -> dict:
  """Sizes that a hybrid design leaves to the checkpoint: the rank of a general delta rule's first decay projection is the
  row count of its ``l<i>.mix.w1`` (of the layer that owns the tensors).  ``shapes``: name -> shape."""
  if not is_hybrid(cfg):
    return cfg
  for i, lay in enumerate(cfg["layers"]):
    if lay.get("mixer") == "gdelta" and not lay.get("rank"):
      src = lay["weights_of"] if lay.get("weights_of", -1) >= 0 else i
      name = f"l{src}.mix.w1"
      if name not in shapes:
        raise ValueError(f"layer {i}: neither the configuration nor a tensor {name} gives the rank of the decay projection")
      lay["rank"] = int(shapes[name][0])
  return cfg


def load_model_config(model_config_path: Path) -> dict:
  """Read a ``config.json`` into the flat dict the engine works with: an HF Llama-shaped one, or (key ``architecture``
  naming a hybrid design) a per-layer description; sizes such a design leaves to the checkpoint are taken from the headers of
  the ``*.safetensors`` files beside it."""
  hf = json.loads(Path(model_config_path).read_text())
  if hf.get("architecture") in HYBRID_ARCHITECTURES:
    cfg = hybrid_model_config(hf)
    if any(lay.get("mixer") == "gdelta" and not lay.get("rank") for lay in cfg["layers"]):
      resolve_tensor_sizes(cfg, safetensors_shapes(Path(model_config_path).parent))
    if cfg.get("pos_rows"):   # a learned position table: its own row count bounds the positions
      rows = safetensors_shapes(Path(model_config_path).parent).get("pos")
      if rows:
        cfg["pos_rows"] = cfg["max_seq_len"] = int(rows[0])
    return cfg
  cfg = {ours: hf[theirs] for theirs, ours in _DIRECT_FIELDS}
  cfg.update({ours: hf.get(theirs, default) for theirs, ours, default in _OPTIONAL_FIELDS})
  cfg["head_dim"] = hf.get("head_dim", hf["hidden_size"] // hf["num_attention_heads"])
  cfg["torch_dtype"] = HF_PRECISION_STR_TO_DTYPE.get(hf.get("torch_dtype", "bfloat16"), torch.bfloat16)
  scaling = hf.get("rope_scaling")
  cfg["rope_scaling"] = scaling
  if scaling is not None:
    # reference quirk kept on purpose: the factor is looked up under "rope_factor", a key HF configs
    # do not carry, so Llama-3.x always runs with 32 (llm_utils.py:68-69)
    cfg["rope_scaling_factor"] = scaling.get("rope_factor", 32)
    if os.getenv("TORCH_USE_ORG_SEQ", "False").lower() == "true":
      cfg["max_seq_len"] = scaling["original_max_position_embeddings"]
  return cfg


def model_family(model_id: str) -> str:
  if "llama" in model_id or "Llama" in model_id:
    return "llama"
  if "qwen" in model_id or "Qwen" in model_id:
    return "qwen"
  return "plain"


def uses_tied_head(model_id: str) -> bool:
  fam = model_family(model_id)
  if fam == "llama":
    return "3.2" in model_id
  if fam == "qwen":
    return "0.5B" in model_id or "0.5b" in model_id
  return False


def has_qkv_bias(model_id: str, config: dict) -> bool:
  return True if model_family(model_id) == "qwen" else bool(config.get("attn_bias", False))


def rope_theta(family: str, config: dict) -> torch.Tensor:
  """Per-pair rotation frequencies.  llama: torchtune Llama3ScaledRoPE.apply_scaling with
  its defaults (low_freq_factor 1, high_freq_factor 4, old_context_len 8192) -- the
  reference passes only scale_factor (general_mha.py:35-40)."""
  dim, base = config["head_dim"], config["rope_base"]
  freqs = 1.0 / (base ** (torch.arange(0, dim, 2)[: (dim // 2)].float() / dim))
  if family != "llama":
    return freqs
  scale_factor = config.get("rope_scaling_factor", 8)
  low_freq_factor, high_freq_factor, old_context_len = 1, 4, 8192
  low_freq_wavelen = old_context_len / low_freq_factor
  high_freq_wavelen = old_context_len / high_freq_factor
  new_freqs = []
  for freq in freqs:
    wavelen = 2 * math.pi / freq
    if wavelen < high_freq_wavelen:
      new_freqs.append(freq)
    elif wavelen > low_freq_wavelen:
      new_freqs.append(freq / scale_factor)
    else:
      smooth = (old_context_len / wavelen - low_freq_factor) / (high_freq_factor - low_freq_factor)
      new_freqs.append((1 - smooth) * freq / scale_factor + smooth * freq)
  return torch.tensor(new_freqs, dtype=freqs.dtype)


def rope_table(family: str, config: dict, n_pos: int, bf16_rounded: bool = True) -> torch.Tensor:
  """fp32 ``[n_pos, head_dim/2, 2]`` (cos, sin) table for XB_W_ROPE_TABLE.  With
  ``bf16_rounded`` the values are rounded to bf16 first: the reference's
  ``Module.to(bfloat16)`` also casts the RoPE module's non-persistent cache,
  so this is the reference-exact table."""
  theta = rope_theta(family, config)
  seq_idx = torch.arange(n_pos, dtype=theta.dtype)
  idx_theta = torch.einsum("i, j -> ij", seq_idx, theta).float()
  cache = torch.stack([torch.cos(idx_theta), torch.sin(idx_theta)], dim=-1)
  if bf16_rounded:
    cache = cache.to(torch.bfloat16)
  return cache.float().contiguous()
