"""Offline stand-ins for the reference's download layer.

The reference's ``ShardDownloader.ensure_shard(shard, engine_name) -> Path``
(``xotorch/download/shard_download.py:9-22``) returns a directory holding
``config.json`` + ``*.safetensors`` in HuggingFace naming.  There is no network on the
build or GPU boxes, so ``LocalShardDownloader`` returns such a directory from local
disk and, when asked, fills it with a seeded random-init checkpoint of the registered
architecture (Linear/embedding N(0, std^2) in bf16, RMSNorm scales
1.0 or 1+N(0, std^2), Qwen q/k/v biases N(0, std^2)).
"""
import json
import os
from pathlib import Path
from typing import Dict, Optional

import torch

from .models import model_cards
from .shard import Shard


def hf_param_shapes(cfg: dict) -> Dict[str, tuple]:
  D, H, KV = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"]
  hd = cfg.get("head_dim", D // H)
  I, V, L = cfg["intermediate_size"], cfg["vocab_size"], cfg["num_hidden_layers"]
  bias = cfg.get("model_type") == "qwen2" or cfg.get("attention_bias", False)
  shapes = {"model.embed_tokens.weight": (V, D), "model.norm.weight": (D,)}
  if not cfg.get("tie_word_embeddings", False):
    shapes["lm_head.weight"] = (V, D)
  for l in range(L):
    p = f"model.layers.{l}."
    shapes[p + "self_attn.q_proj.weight"] = (H * hd, D)
    shapes[p + "self_attn.k_proj.weight"] = (KV * hd, D)
    shapes[p + "self_attn.v_proj.weight"] = (KV * hd, D)
    shapes[p + "self_attn.o_proj.weight"] = (D, H * hd)
    if bias:
      shapes[p + "self_attn.q_proj.bias"] = (H * hd,)
      shapes[p + "self_attn.k_proj.bias"] = (KV * hd,)
      shapes[p + "self_attn.v_proj.bias"] = (KV * hd,)
    shapes[p + "mlp.gate_proj.weight"] = (I, D)
    shapes[p + "mlp.up_proj.weight"] = (I, D)
    shapes[p + "mlp.down_proj.weight"] = (D, I)
    shapes[p + "input_layernorm.weight"] = (D,)
    shapes[p + "post_attention_layernorm.weight"] = (D,)
  return shapes


def random_hf_state(cfg: dict, seed: int = 0, std: float = 0.02, norm_jitter: float = 0.0,
                    dtype: torch.dtype = torch.bfloat16, only_layers: Optional[range] = None,
                    peaked_head: float = 0.0, embed_std: Optional[float] = None) -> Dict[str, torch.Tensor]:
  """Seeded random-init state dict in HF naming.  Each tensor draws from its own
  generator (seed, name-hash) so a layer-range subset equals the same rows of the full
  model.  ``peaked_head`` > 0 plants ``lm_head = peaked_head * embed + noise`` so greedy
  decoding has top-2 margins far above one bf16 ulp;
  ``embed_std`` scales the embedding table alone (with a tied head a larger table keeps the
  last token's own embedding visible in the residual stream, which peaks the logits)."""
  out = {}
  names = sorted(hf_param_shapes(cfg).items())
  for idx, (name, shape) in enumerate(names):
    if only_layers is not None and name.startswith("model.layers."):
      l = int(name.split(".")[2])
      if l not in only_layers:
        continue
    g = torch.Generator().manual_seed(seed * 1000003 + idx)
    if name.endswith("layernorm.weight") or name == "model.norm.weight":
      t = torch.ones(shape)
      if norm_jitter:
        t = t + norm_jitter * torch.randn(shape, generator=g)
    elif name == "model.embed_tokens.weight" and embed_std is not None:
      t = embed_std * torch.randn(shape, generator=g)
    else:
      t = std * torch.randn(shape, generator=g)
    out[name] = t.to(dtype)
  if peaked_head and "lm_head.weight" in out:
    out["lm_head.weight"] = (out["lm_head.weight"].float() + peaked_head * out["model.embed_tokens.weight"].float()).to(dtype)
  return out


def refatar_param_shapes(cfg: dict) -> Dict[str, tuple]:
  """Tensor names and shapes of a Refatar checkpoint for its ``config.json`` (Linear weights are [out, in])."""
  D, V, L = cfg["width"], cfg["vocab"], len(cfg["layers"])
  taps = cfg["canon"]["taps"] if cfg.get("canon") else 0
  sd = cfg["token_side"]["dim"] if cfg.get("token_side") else 0
  sh = {"embed": (V, D), "final.norm": (D,), "head": (V, D)}
  if sd:
    sh["side.embed"] = (V, sd * L)
  for i, lc in enumerate(cfg["layers"]):
    p, m = f"l{i}.", lc["mixer"]
    sh[p + "norm1"] = sh[p + "norm1b"] = (D,)
    if taps:
      sh[p + "canon1"] = (D, taps)
    if lc["type"] == "delta":
      H, G, dk, dv, ct = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
      sh.update({p + "mix.q": (G * dk, D), p + "mix.q.conv": (G * dk, ct), p + "mix.k": (G * dk, D), p + "mix.k.conv": (G * dk, ct),
                 p + "mix.v": (H * dv, D), p + "mix.v.conv": (H * dv, ct), p + "mix.b": (H, D), p + "mix.a": (H, D),
                 p + "mix.A_log": (H,), p + "mix.dt_bias": (H,), p + "mix.norm": (dv,), p + "mix.g": (H * dv, D), p + "mix.o": (D, H * dv)})
    else:
      le, ri = m["left"], m["right"]
      H, G, dk, dv = le["heads"], le["kv_heads"], le["dim"], le["vdim"]
      Hr, rk, rv = ri["heads"], ri["dim"], ri["vdim"]
      sh.update({p + "mix.left.q": (H * dk, D), p + "mix.left.q.b": (H * dk,), p + "mix.left.k": (G * dk, D), p + "mix.left.k.b": (G * dk,),
                 p + "mix.left.v": (G * dv, D), p + "mix.left.v.b": (G * dv,), p + "mix.left.g": (H * dv, D), p + "mix.left.o": (D, H * dv),
                 p + "mix.right.q": (Hr * rk, D), p + "mix.right.f": (Hr * rk, D), p + "mix.right.f.b": (Hr * rk,),
                 p + "mix.right.lower": (Hr * rk,), p + "mix.right.v": (Hr * rv, D), p + "mix.right.norm": (rv,),
                 p + "mix.right.o": (D, Hr * rv)})
    if lc.get("mlp"):
      F = lc["mlp"]["ff"]
      sh.update({p + "norm2": (D,), p + "norm2b": (D,), p + "mlp.up": (F, D), p + "mlp.down": (D, F)})
      if taps:
        sh[p + "canon2"] = (D, taps)
    if sd:
      sh.update({p + "side.gate": (sd, D), p + "side.proj": (D, sd), p + "side.norm": (D,)})
  return sh


def random_refatar_state(cfg: dict, seed: int = 0, dtype: torch.dtype = torch.bfloat16, gain: float = 1.0,
                         device: str = "cpu") -> Dict[str, torch.Tensor]:
  """Seeded random Refatar weights: matrices N(0, gain^2 / in), offset-from-one norm weights N(0, 0.1^2), plain norm weights
  1 + N(0, 0.1^2), filters N(0, 0.3^2), forget-gate floors in (0.05, 0.95), decay rates exp(A_log) in (0.5, 4)."""
  out = {}
  for idx, (name, shape) in enumerate(sorted(refatar_param_shapes(cfg).items())):
    g = torch.Generator(device=device).manual_seed(seed * 1000003 + idx)
    rn = lambda: torch.randn(shape, generator=g, device=device)  # noqa: E731
    leaf = name.split(".")[-1]
    if name.endswith("side.norm") or name.endswith("mix.norm") or name.endswith("right.norm"):
      t = 1.0 + 0.1 * rn()
    elif leaf in ("norm1", "norm1b", "norm2", "norm2b") or name == "final.norm":
      t = 0.1 * rn()
    elif leaf in ("canon1", "canon2", "conv"):
      t = 0.3 * rn()
    elif leaf == "lower":
      t = 0.05 + 0.9 * torch.rand(shape, generator=g, device=device)
    elif leaf == "A_log":
      t = torch.log(0.5 + 3.5 * torch.rand(shape, generator=g, device=device))
    elif leaf in ("dt_bias", "b") and len(shape) == 1:
      t = 0.5 * rn()
    elif name in ("embed", "side.embed"):
      t = rn()
    else:
      t = gain * rn() / (shape[-1] ** 0.5)
    out[name] = t.to(dtype)
  return out


def bibevik_param_shapes(cfg: dict, rank: int = 16) -> Dict[str, tuple]:
  """Tensor names and shapes of a Bibevik checkpoint for its ``config.json`` (Linear weights are [out, in]; layers with
  ``weights_of`` have no tensors).  ``rank``: rows of a general delta rule's first decay projection where the mixer's entry
  does not name it (the design leaves that size to the checkpoint)."""
  D, V = cfg["width"], cfg["vocab"]
  sh = {"embed": (V, D), "final.norm": (), "head": (V, D)}
  for i, lc in enumerate(cfg["layers"]):
    if lc.get("weights_of") is not None:
      continue
    p, m = f"l{i}.", lc["mixer"]
    sh[p + "norm1"] = ()
    H, n = m["heads"], m["dim"]
    if lc["type"] == "latent_attention":
      dr, dv, R = m["rot_dim"], m["vdim"], m["kv_rank"]
      sh.update({p + "mix.q": (H * (n + dr), D), p + "mix.dkv": (R + dr, D), p + "mix.dkv.norm": (R,), p + "mix.uk": (H * n, R),
                 p + "mix.uv": (H * dv, R), p + "mix.o": (D, H * dv)})
    elif lc["type"] == "general_delta":
      rk = m.get("rank", rank)
      sh.update({p + "mix." + k: (H * n, D) for k in ("r", "k", "v", "g", "a")})
      sh.update({p + "mix.a.b": (H * n,), p + "mix.w1": (rk, D), p + "mix.w2": (H * n, rk), p + "mix.w0": (H * n,),
                 p + "mix.norm": (H * n,), p + "mix.o": (D, H * n)})
    else:
      dv = m["vdim"]
      sh.update({p + "mix.q": (H * n, D), p + "mix.k": (H * n, D), p + "mix.v": (H * dv, D), p + "mix.g": (H * dv, D),
                 p + "mix.norm": (H * dv,), p + "mix.o": (D, H * dv)})
    mlp = lc.get("mlp")
    if mlp and mlp["kind"] == "dense":
      F = mlp["ff"]
      sh.update({p + "mlp.gate": (F, D), p + "mlp.gate.b": (F,), p + "mlp.up": (F, D), p + "mlp.up.b": (F,),
                 p + "mlp.down": (D, F), p + "mlp.down.b": (D,)})
    elif mlp:
      F = mlp["expert"]["ff"]
      sh[p + "mlp.router"] = (mlp["router"]["experts"], D)
      for e in range(mlp["router"]["experts"]):
        sh.update({f"{p}mlp.e{e}.gate": (F, D), f"{p}mlp.e{e}.up": (F, D), f"{p}mlp.e{e}.down": (D, F)})
      if mlp.get("shared"):
        S = mlp["shared"]["ff"]
        sh.update({p + "mlp.shared.gate": (S, D), p + "mlp.shared.up": (S, D), p + "mlp.shared.down": (D, S)})
  return sh


def random_bibevik_state(cfg: dict, seed: int = 0, dtype: torch.dtype = torch.bfloat16, gain: float = 1.0, device: str = "cpu",
                         rank: int = 16) -> Dict[str, torch.Tensor]:
  """Seeded random Bibevik weights: matrices N(0, gain^2 / in), the stream's one-number norms near 1, vector norm weights
  1 + N(0, 0.1^2), biases and decay offsets N(0, 0.5^2), embedding rows N(0, 1 / width) (the design scales them up again)."""
  out = {}
  for idx, (name, shape) in enumerate(sorted(bibevik_param_shapes(cfg, rank).items())):
    g = torch.Generator(device=device).manual_seed(seed * 1000003 + idx)
    rn = lambda: torch.randn(shape, generator=g, device=device)  # noqa: E731
    leaf = name.split(".")[-1]
    if leaf == "norm1" or name == "final.norm":
      t = 1.0 + 0.2 * rn()
    elif leaf == "norm":
      t = 1.0 + 0.1 * rn()
    elif leaf in ("b", "w0"):
      t = 0.5 * rn()
    elif name == "embed":
      t = rn() / (shape[-1] ** 0.5)
    elif leaf == "router":
      t = 2.0 * gain * rn() / (shape[-1] ** 0.5)
    else:
      t = gain * rn() / (shape[-1] ** 0.5)
    out[name] = t.to(dtype)
  return out


def pufivik_param_shapes(cfg: dict) -> Dict[str, tuple]:
  """name -> shape of every tensor of a Pufivik config.json (the head is the embedding table: no tensor of its own)."""
  D, V = cfg["width"], cfg["vocab"]
  taps = (cfg.get("canon") or {}).get("taps", 0)
  sh = {"embed": (V, D), "final.norm": (D,)}
  for i, lc in enumerate(cfg["layers"]):
    p, m = f"l{i}.", lc["mixer"]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    sh.update({p + "norm1": (D,), p + "norm1b": (D,), p + "mix.q": (H * dk, D), p + "mix.k": (G * dk, D), p + "mix.v": (G * dv, D),
               p + "mix.o": (D, H * dv)})
    if taps:
      sh[p + "canon1"] = (D, taps)
    if m.get("v_mix"):
      sh[p + "mix.vmix"] = ()
    if lc["type"] == "attention":
      sh.update({p + "mix.talk": (H, H), p + "mix.sink": (H,), p + "mix.g": (H, D)})
    mlp = lc.get("mlp")
    if mlp:
      F, E = mlp["expert"]["ff"], mlp["router"]["experts"]
      sh.update({p + "norm2": (D,), p + "norm2b": (D,), p + "mlp.router": (E, D)})
      for e in range(E):
        sh.update({f"{p}mlp.e{e}.gate": (F, D), f"{p}mlp.e{e}.up": (F, D), f"{p}mlp.e{e}.down": (D, F)})
  return sh


def random_pufivik_state(cfg: dict, seed: int = 0, dtype: torch.dtype = torch.bfloat16, gain: float = 1.0,
                         device: str = "cpu") -> Dict[str, torch.Tensor]:
  """Seeded random Pufivik weights: matrices N(0, gain^2 / in), norm weights 1 + N(0, 0.1^2), filters N(0, 0.3^2), sinks
  N(0, 1), head-mixing matrices identity + N(0, 0.3^2), blend factors in (0.2, 0.8), routers spread so that the scores
  differ, embedding rows N(0, 1 / width) (the design scales them up again)."""
  out = {}
  for idx, (name, shape) in enumerate(sorted(pufivik_param_shapes(cfg).items())):
    g = torch.Generator(device=device).manual_seed(seed * 1000003 + idx)
    rn = lambda: torch.randn(shape, generator=g, device=device)  # noqa: E731
    leaf = name.split(".")[-1]
    if leaf.startswith("norm"):
      t = 1.0 + 0.1 * rn()
    elif leaf == "canon1":
      t = 0.3 * rn()
    elif leaf == "sink":
      t = rn()
    elif leaf == "talk":
      t = torch.eye(shape[0], device=device) + 0.3 * rn()
    elif leaf == "vmix":
      t = 0.2 + 0.6 * torch.rand(shape, generator=g, device=device)
    elif leaf == "router":
      t = 2.0 * gain * rn() / (shape[-1] ** 0.5)
    else:
      t = gain * rn() / (shape[-1] ** 0.5)
    out[name] = t.to(dtype)
  return out


def vusenex_param_shapes(cfg: dict) -> Dict[str, tuple]:
  """name -> shape of every tensor of a Vusenex config.json (norms of the stream are single numbers)."""
  D, V = cfg["width"], cfg["vocab"]
  sh = {"embed": (V, D), "pos": (cfg["max_positions"], D), "final.norm": (), "head": (V, D)}
  bg = (cfg.get("embedding") or {}).get("bigram")
  if bg:
    sh["bigram"] = (bg["buckets"] + 1, D)
  for i, lc in enumerate(cfg["layers"]):
    p, m = f"l{i}.", lc["mixer"]
    sh.update({p + "norm1": (), p + "rg1": (D, D), p + "rg1.b": (D,)})
    if lc["type"] == "attention":
      H, G, dk = m["heads"], m["kv_heads"], m["dim"]
      sh.update({p + "mix.q": (H * dk, D), p + "mix.q.b": (H * dk,), p + "mix.k": (G * dk, D), p + "mix.k.b": (G * dk,),
                 p + "mix.q.norm": (H * dk,), p + "mix.k.norm": (G * dk,), p + "mix.r1": (H,), p + "mix.r2": (H,), p + "mix.o": (D, H * dk)})
    else:
      H, dk, dv, R = m["heads"], m["dim"], m["vdim"], m["kv_rank"]
      sh.update({p + "mix.q": (H * dk, D), p + "mix.dkv": (R, D), p + "mix.dkv.norm": (R,), p + "mix.uk": (H * dk, R), p + "mix.uv": (H * dv, R),
                 p + "mix.o": (D, H * dv)})
    mlp = lc.get("mlp")
    if mlp:
      F, E = mlp["expert"]["ff"], mlp["router"]["experts"]
      sh.update({p + "norm2": (), p + "rg2": (D, D), p + "rg2.b": (D,), p + "mlp.router": (E, D)})
      for e in range(E):
        sh.update({f"{p}mlp.e{e}.up": (F, D), f"{p}mlp.e{e}.down": (D, F)})
      if mlp.get("shared"):
        S = mlp["shared"]["ff"]
        sh.update({p + "mlp.shared.up": (S, D), p + "mlp.shared.down": (D, S)})
  return sh


def random_vusenex_state(cfg: dict, seed: int = 0, dtype: torch.dtype = torch.bfloat16, gain: float = 1.0,
                         device: str = "cpu") -> Dict[str, torch.Tensor]:
  """Seeded random Vusenex weights: matrices N(0, gain^2 / in), the stream's norm numbers in (0.5, 1.5), q / k norm weights
  1 + N(0, 0.1^2), biases N(0, 0.3^2), distance penalties r1 in (0.1, 0.9) and r2 in (0.05, 1), routers spread so that the
  scores differ, table rows N(0, 1)."""
  out = {}
  for idx, (name, shape) in enumerate(sorted(vusenex_param_shapes(cfg).items())):
    g = torch.Generator(device=device).manual_seed(seed * 1000003 + idx)
    rn = lambda: torch.randn(shape, generator=g, device=device)  # noqa: E731
    ru = lambda: torch.rand(shape, generator=g, device=device)  # noqa: E731
    leaf = name.split(".")[-1]
    if name in ("embed", "pos", "bigram"):
      t = (0.6 if name == "embed" else 0.4) * rn()
    elif leaf in ("norm1", "norm2") or name == "final.norm":
      t = 0.5 + ru()
    elif leaf == "norm":
      t = 1.0 + 0.1 * rn()
    elif leaf == "b":
      t = 0.3 * rn()
    elif leaf == "r1":
      t = 0.1 + 0.8 * ru()
    elif leaf == "r2":
      t = 0.05 + 0.95 * ru()
    elif leaf == "router":
      t = 2.0 * gain * rn() / (shape[-1] ** 0.5)
    else:
      t = gain * rn() / (shape[-1] ** 0.5)
    out[name] = t.to(dtype)
  return out


def write_random_checkpoint(path: Path, cfg: dict, seed: int = 0, std: float = 0.02,
                            norm_jitter: float = 0.0, shard_bytes: int = 4 << 30,
                            peaked_head: float = 0.0) -> Path:
  from safetensors.torch import save_file
  path = Path(path)
  path.mkdir(parents=True, exist_ok=True)
  with open(path / "config.json", "w") as f:
    json.dump(cfg, f, indent=1)
  if cfg.get("architecture") == "Refatar":
    state = random_refatar_state(cfg, seed=seed)
  elif cfg.get("architecture") == "Bibevik":
    state = random_bibevik_state(cfg, seed=seed)
  elif cfg.get("architecture") == "Pufivik":
    state = random_pufivik_state(cfg, seed=seed)
  elif cfg.get("architecture") == "Vusenex":
    state = random_vusenex_state(cfg, seed=seed)
  else:
    state = random_hf_state(cfg, seed=seed, std=std, norm_jitter=norm_jitter, peaked_head=peaked_head)
  files, cur, cur_bytes = [], {}, 0
  for k, v in state.items():
    nb = v.numel() * v.element_size()
    if cur and cur_bytes + nb > shard_bytes:
      files.append(cur)
      cur, cur_bytes = {}, 0
    cur[k] = v.contiguous()
    cur_bytes += nb
  if cur:
    files.append(cur)
  for i, d in enumerate(files):
    save_file(d, str(path / f"model-{i + 1:05d}-of-{len(files):05d}.safetensors"))
  with open(path / "xb_synth.json", "w") as f:
    json.dump({"seed": seed, "std": std, "norm_jitter": norm_jitter, "peaked_head": peaked_head}, f)
  return path


def xot_home() -> Path:
  return Path(os.environ.get("XOT_HOME", Path.home() / ".cache" / "xotorch"))


class LocalShardDownloader:
  """ShardDownloader (shard_download.py:9-22) that never touches the network.

  ``ensure_shard`` returns ``$XOT_HOME/downloads/<org--repo>/`` (the reference's layout,
  new_shard_download.py:24-49).  With ``synthesize=True`` a missing directory is filled
  with a seeded random-init checkpoint of the registered architecture."""

  def __init__(self, root: Optional[Path] = None, synthesize: bool = True, seed: int = 0,
               std: float = 0.02, norm_jitter: float = 0.0, peaked_head: float = 0.0):
    self.root = Path(root) if root is not None else xot_home() / "downloads"
    self.synthesize, self.seed, self.std, self.norm_jitter = synthesize, seed, std, norm_jitter
    self.peaked_head = peaked_head

  def path_for(self, model_id: str, inference_engine_name: str) -> Path:
    repo = model_cards.get(model_id, {}).get("repo", {}).get(inference_engine_name)
    if repo is None:
      raise ValueError(f"no repo registered for model {model_id!r} and engine {inference_engine_name!r}")
    return self.root / repo.replace("/", "--")

  async def ensure_shard(self, shard: Shard, inference_engine_name: str) -> Path:
    p = self.path_for(shard.model_id, inference_engine_name)
    if not (p / "config.json").exists():
      if not self.synthesize:
        raise FileNotFoundError(f"{p} has no config.json and synthesis is disabled")
      write_random_checkpoint(p, model_cards[shard.model_id]["hf_config"], seed=self.seed, std=self.std,
                              norm_jitter=self.norm_jitter, peaked_head=self.peaked_head)
    return p

  async def get_shard_download_status(self, inference_engine_name: str):
    if False:
      yield


class SyntheticTokenizer:
  """Whitespace-free stand-in for the HF tokenizer the reference resolves
  (``xotorch/inference/tokenizers.py:43-63``): no tokenizer files exist offline.
  ``encode`` hashes the prompt into a seeded id sequence (never id 0, so the
  reference's no-pad ``tril`` branch, sharded_inference_engine.py:178-186, is taken)."""

  def __init__(self, vocab_size: int, eos_token_id: Optional[int] = None):
    self.vocab_size = vocab_size
    self.eos_token_id = eos_token_id if eos_token_id is not None else vocab_size - 1
    self.pad_token_id = None

  def encode(self, text: str, return_tensors: Optional[str] = None):
    import zlib
    if text.startswith("<ids:") and text.endswith(">"):
      ids = [int(t) for t in text[5:-1].split(",") if t]
    else:
      n = max(1, len(text.split()))
      g = torch.Generator().manual_seed(zlib.crc32(text.encode()))
      ids = torch.randint(1, self.vocab_size - 1, (n,), generator=g).tolist()
    if return_tensors == "pt":
      return torch.tensor([ids], dtype=torch.int64)
    return ids

  def decode(self, tokens) -> str:
    return " ".join(f"<{int(t)}>" for t in tokens)

  def apply_chat_template(self, conversation, tokenize=False, add_generation_prompt=True, **kw):
    return "\n".join(str(m.get("content", "")) for m in conversation)
