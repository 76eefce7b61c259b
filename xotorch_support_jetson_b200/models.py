"""Model registry for the configs BASELINE.json names.

Mirrors the reference's ``xotorch/models.py:4-179,231-263`` (``model_cards`` keyed by
model id, repo lookup keyed by *engine class name*) for the five benchmark models, and
adds the public HF ``config.json`` of each so that random-init checkpoints of the right
architecture can be written offline (there is no network here).
"""
from typing import Optional
from .shard import Shard

ENGINE_CLASS_NAME = "B200ShardInferenceEngine"

_LLAMA3_ROPE = {"factor": 32.0, "high_freq_factor": 4.0, "low_freq_factor": 1.0,
                "original_max_position_embeddings": 8192, "rope_type": "llama3"}


def _llama(hidden, heads, kv, inter, layers, head_dim=None, tie=False, factor=32.0, vocab=128256):
  cfg = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_act": "silu",
    "hidden_size": hidden, "intermediate_size": inter, "num_attention_heads": heads,
    "num_key_value_heads": kv, "num_hidden_layers": layers, "vocab_size": vocab,
    "max_position_embeddings": 131072, "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
    "rope_scaling": dict(_LLAMA3_ROPE, factor=factor), "tie_word_embeddings": tie,
    "attention_bias": False, "mlp_bias": False, "torch_dtype": "bfloat16",
  }
  if head_dim is not None:
    cfg["head_dim"] = head_dim
  return cfg


def _qwen(hidden, heads, kv, inter, layers, vocab=152064, tie=False, max_pos=32768):
  return {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "hidden_act": "silu",
    "hidden_size": hidden, "intermediate_size": inter, "num_attention_heads": heads,
    "num_key_value_heads": kv, "num_hidden_layers": layers, "vocab_size": vocab,
    "max_position_embeddings": max_pos, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
    "tie_word_embeddings": tie, "torch_dtype": "bfloat16",
  }


def _mistral(hidden, heads, kv, inter, layers, head_dim, vocab=32768):
  """An id with neither "llama" nor "qwen" in it: the reference then builds plain RotaryPositionalEmbeddings, no
  q/k/v bias, untied head (general_mha.py:58-63) -- its mistral-nemo / nemotron-70b cards take that branch."""
  return {
    "architectures": ["MistralForCausalLM"], "model_type": "mistral", "hidden_act": "silu",
    "hidden_size": hidden, "intermediate_size": inter, "num_attention_heads": heads,
    "num_key_value_heads": kv, "num_hidden_layers": layers, "vocab_size": vocab, "head_dim": head_dim,
    "max_position_embeddings": 131072, "rms_norm_eps": 1e-5, "rope_theta": 1000000.0,
    "tie_word_embeddings": False, "torch_dtype": "bfloat16",
  }


def _refatar(width, vocab, layers, taps=4, side=8, softcap=30.0, eps=1e-5):
  """A Refatar config.json: layers is a list of ("delta", {heads, kv_heads, dim, vdim, conv}, ff) /
  ("parallel", {left, right, left_scale, right_scale}, ff) entries (ff 0 = no feed-forward)."""
  cfg = {"architecture": "Refatar", "width": width, "vocab": vocab, "norm": {"eps": eps},
         "layers": [{"type": t, "mixer": m, "mlp": ({"kind": "dense", "ff": ff} if ff else None)} for t, m, ff in layers]}
  if taps:
    cfg["canon"] = {"taps": taps}
  if side:
    cfg["token_side"] = {"dim": side}
  if softcap:
    cfg["logit_softcap"] = softcap
  return cfg


def _refatar_pair(heads, kv, dim, vdim, window, keep, r_heads, r_dim, r_vdim):
  return {"left": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": dim ** -0.5,
                   "mask": {"size": window, "keep_first": keep}},
          "right": {"heads": r_heads, "dim": r_dim, "vdim": r_vdim}, "left_scale": 1.0, "right_scale": 1.0}


_REFATAR_TINY = _refatar(128, 512, [
  ("delta", {"heads": 4, "kv_heads": 2, "dim": 32, "vdim": 48, "conv": 3}, 256),
  ("parallel", _refatar_pair(4, 2, 32, 48, 24, 3, 2, 32, 64), 256),
  ("parallel", _refatar_pair(8, 8, 16, 16, 9, 0, 4, 16, 32), 0),
  ("delta", {"heads": 2, "kv_heads": 2, "dim": 64, "vdim": 64, "conv": 4}, 192),
], taps=3, side=8)
# 1B-class geometry for throughput runs (random weights): the widths of llama-3.2-1b with alternating mixers
_REFATAR_1B = _refatar(2048, 128256, [
  (("delta", {"heads": 16, "kv_heads": 16, "dim": 128, "vdim": 128, "conv": 4}, 8192) if i % 2 == 0 else
   ("parallel", _refatar_pair(32, 8, 64, 64, 1024, 4, 16, 128, 128), 8192)) for i in range(16)], taps=4, side=32)

def _bibevik(width, vocab, layers, eps=1e-6):
  """A Bibevik config.json: layers is a list of (type, mixer, mlp[, weights_of]) entries."""
  out = []
  for ent in layers:
    lay = {"type": ent[0], "mixer": ent[1], "mlp": ent[2]}
    if len(ent) > 3:
      lay["weights_of"] = ent[3]
    out.append(lay)
  return {"architecture": "Bibevik", "width": width, "vocab": vocab, "embedding": {"scale": width ** 0.5}, "norm": {"eps": eps}, "layers": out}


def _latent(heads, dim, rot_dim, vdim, kv_rank, base=10000.0):
  return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": (dim + rot_dim) ** -0.5,
          "rot": {"base": base, "dims": rot_dim}}


def _glu(ff, limit=7.0):
  return {"kind": "dense", "ff": ff, "limit": limit}


def _experts(n, top, ff, groups, keep, shared_ff, scale=1.0, limit=7.0):
  m = {"kind": "moe", "expert": {"ff": ff, "limit": limit},
       "router": {"experts": n, "top": top, "scale": scale, "groups": {"count": groups, "keep": keep}}}
  if shared_ff:
    m["shared"] = {"ff": shared_ff, "limit": limit}
  return m


def _head_decays(heads):
  return [1.0 - 2.0 ** (-5.0 - 3.0 * h / max(heads - 1, 1)) for h in range(heads)]


_BIBEVIK_TINY = _bibevik(160, 384, [
  ("lightning", {"heads": 4, "dim": 16, "vdim": 24, "decay": [0.5, 0.9, 0.97, 0.995]}, _glu(320, 1.5)),
  ("latent_attention", _latent(5, 24, 16, 40, 48), _experts(8, 2, 48, 4, 2, 64, scale=1.5, limit=2.0)),
  ("general_delta", {"heads": 5, "dim": 32, "rank": 8}, None),
  ("latent_attention", _latent(5, 24, 16, 40, 48), _experts(8, 2, 48, 4, 2, 64, scale=1.5, limit=2.0), 1),
  ("general_delta", {"heads": 5, "dim": 32, "rank": 8}, _glu(256, 1.0)),
])
# 1B-class geometry for throughput runs (random weights): the widths of llama-3.2-1b, mixers in the order delta rule,
# latent attention, lightning, latent attention; dense and expert feed-forwards alternate
_BIBEVIK_1B = _bibevik(2048, 128256, [
  (("general_delta", {"heads": 32, "dim": 64, "rank": 64}, _glu(8192)) if i % 4 == 0 else
   ("lightning", {"heads": 16, "dim": 128, "vdim": 128, "decay": _head_decays(16)}, _glu(8192)) if i % 4 == 2 else
   ("latent_attention", _latent(16, 64, 64, 128, 256, base=500000.0), _experts(16, 4, 384, 4, 2, 2048)))
  for i in range(16)])

def _pufivik(width, vocab, layers, groups=2, taps=3, mult=0.7, scale=8.0, eps=1e-6):
  """A Pufivik config.json: layers is a list of (type, mixer, mlp) entries."""
  return {"architecture": "Pufivik", "width": width, "vocab": vocab, "embedding": {"scale": scale}, "residual_mult": mult,
          "norm": {"eps": eps, "groups": groups}, "canon": {"taps": taps},
          "layers": [{"type": t, "mixer": m, "mlp": f} for t, m, f in layers]}


def _sink_attn(heads, kv, dim, vdim, rot_dims, base=1000000.0, v_mix=True, factor=8.0, low=1.0, high=4.0, original=4096):
  return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": dim ** -0.5, "v_mix": v_mix,
          "rot": {"base": base, "dims": rot_dims, "scaling": {"factor": factor, "low": low, "high": high, "original": original}}}


def _cap_attn(heads, kv, dim, vdim, rot_dims, base=10000.0, v_mix=True, softcap=50.0, factor=4.0, fast=32.0, slow=1.0, original=1024):
  return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": dim ** -0.5, "softcap": softcap, "v_mix": v_mix,
          "rot": {"base": base, "dims": rot_dims, "scaling": {"factor": factor, "fast": fast, "slow": slow, "original": original}}}


def _swiglu_experts(n, top, ff):
  return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": n, "top": top}}


_PUFIVIK_TINY = _pufivik(160, 448, [
  ("attention", _sink_attn(6, 3, 40, 24, 16), _swiglu_experts(6, 2, 48)),
  ("attention_2", _cap_attn(6, 3, 32, 24, 32), None),
  ("attention_2", _cap_attn(4, 1, 24, 36, 8, v_mix=False), _swiglu_experts(8, 1, 32)),
  ("attention", _sink_attn(3, 3, 48, 24, 24), _swiglu_experts(6, 2, 48)),
], groups=4, taps=4)
# 1B-class geometry for throughput runs (random weights): the widths of llama-3.2-1b (32 query / 8 key heads of 64), three
# soft-capped layers to one with sink, mixed heads and head gates; 8 experts of 1024 of which a token uses two
_PUFIVIK_1B = _pufivik(2048, 128256, [
  (("attention", _sink_attn(32, 8, 64, 64, 32), _swiglu_experts(8, 2, 1024)) if i % 4 == 1 else
   ("attention_2", _cap_attn(32, 8, 64, 64, 64), _swiglu_experts(8, 2, 1024))) for i in range(16)], scale=45.0)

def _vusenex(width, vocab, layers, max_pos=4096, buckets=4093, mul_prev=37, mul_cur=11, eps=1e-6):
  """A Vusenex config.json: layers is a list of (type, mixer, mlp) entries."""
  return {"architecture": "Vusenex", "width": width, "vocab": vocab, "max_positions": max_pos,
          "embedding": {"bigram": {"buckets": buckets, "mul_prev": mul_prev, "mul_cur": mul_cur}}, "norm": {"eps": eps},
          "layers": [{"type": t, "mixer": m, "mlp": f} for t, m, f in layers]}


def _kv_attn(heads, kv, dim, coef=0.2, every=64):
  return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "scale": dim ** -0.5, "q_temp": {"coef": coef, "every": every}}


def _plain_latent(heads, dim, vdim, rank):
  return {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": rank, "scale": dim ** -0.5}


def _gelu_experts(n, top, ff, groups, keep, shared_ff):
  m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": n, "top": top, "groups": {"count": groups, "keep": keep}}}
  if shared_ff:
    m["shared"] = {"ff": shared_ff}
  return m


_VUSENEX_TINY = _vusenex(160, 448, [
  ("latent_attention", _plain_latent(5, 24, 40, 48), _gelu_experts(8, 2, 48, 4, 2, 64)),
  ("attention", _kv_attn(6, 3, 40), _gelu_experts(6, 3, 32, 3, 2, 0)),
  ("attention", _kv_attn(4, 1, 24, coef=0.5, every=16), None),
  ("latent_attention", _plain_latent(3, 32, 32, 80), _gelu_experts(8, 2, 48, 4, 2, 64)),
], max_pos=1024, buckets=509)
# 1B-class geometry for throughput runs (random weights): the widths of llama-3.2-1b (32 query / 8 key heads of 64), latent
# layers of 16 heads over a latent of 256, 16 experts of 512 of which a token uses four (the width of four of them plus the
# shared expert = half of Llama's feed-forward)
_VUSENEX_1B = _vusenex(2048, 128256, [
  (("attention", _kv_attn(32, 8, 64, coef=0.25, every=96), _gelu_experts(16, 4, 512, 4, 2, 2048)) if i % 4 in (0, 3) else
   ("latent_attention", _plain_latent(16, 64, 128, 256), _gelu_experts(16, 4, 512, 4, 2, 2048))) for i in range(16)], max_pos=8192, buckets=65521)

# model id -> {layers, repo:{EngineClassName: hf repo}, hf_config}
model_cards = {
  "llama-3.2-1b": {"layers": 16, "repo": {ENGINE_CLASS_NAME: "unsloth/Llama-3.2-1B-Instruct"},
                   "hf_config": _llama(2048, 32, 8, 8192, 16, head_dim=64, tie=True)},
  "llama-3.2-3b": {"layers": 28, "repo": {ENGINE_CLASS_NAME: "unsloth/Llama-3.2-3B-Instruct"},
                   "hf_config": _llama(3072, 24, 8, 8192, 28, head_dim=128, tie=True)},
  "llama-3.1-8b": {"layers": 32, "repo": {ENGINE_CLASS_NAME: "unsloth/Meta-Llama-3.1-8B-Instruct"},
                   "hf_config": _llama(4096, 32, 8, 14336, 32, factor=8.0)},
  "llama-3.1-70b": {"layers": 80, "repo": {ENGINE_CLASS_NAME: "unsloth/Meta-Llama-3.1-70B-Instruct"},
                    "hf_config": _llama(8192, 64, 8, 28672, 80, factor=8.0)},
  "qwen-2.5-7b": {"layers": 28, "repo": {ENGINE_CLASS_NAME: "Qwen/Qwen2.5-7B-Instruct"},
                  "hf_config": _qwen(3584, 28, 4, 18944, 28)},
  # small same-architecture models for parity tests (seconds on the CPU oracle)
  "llama-3.2-tiny": {"layers": 4, "repo": {ENGINE_CLASS_NAME: "synthetic/llama-3.2-tiny"},
                     "hf_config": _llama(256, 8, 2, 512, 4, head_dim=64, tie=True, vocab=1024)},
  "llama-3.1-tiny": {"layers": 6, "repo": {ENGINE_CLASS_NAME: "synthetic/llama-3.1-tiny"},
                     "hf_config": _llama(512, 4, 2, 1024, 6, head_dim=128, factor=8.0, vocab=2048)},
  "qwen-2.5-tiny": {"layers": 4, "repo": {ENGINE_CLASS_NAME: "synthetic/qwen-2.5-tiny"},
                    "hf_config": _qwen(384, 6, 2, 768, 4, vocab=1536, max_pos=4096)},
  "refatar-tiny": {"layers": 4, "repo": {ENGINE_CLASS_NAME: "synthetic/refatar-tiny"}, "hf_config": _REFATAR_TINY},
  "refatar-1b": {"layers": 16, "repo": {ENGINE_CLASS_NAME: "synthetic/refatar-1b"}, "hf_config": _REFATAR_1B},
  "bibevik-tiny": {"layers": 5, "repo": {ENGINE_CLASS_NAME: "synthetic/bibevik-tiny"}, "hf_config": _BIBEVIK_TINY},
  "bibevik-1b": {"layers": 16, "repo": {ENGINE_CLASS_NAME: "synthetic/bibevik-1b"}, "hf_config": _BIBEVIK_1B},
  "pufivik-tiny": {"layers": 4, "repo": {ENGINE_CLASS_NAME: "synthetic/pufivik-tiny"}, "hf_config": _PUFIVIK_TINY},
  "pufivik-1b": {"layers": 16, "repo": {ENGINE_CLASS_NAME: "synthetic/pufivik-1b"}, "hf_config": _PUFIVIK_1B},
  "vusenex-tiny": {"layers": 4, "repo": {ENGINE_CLASS_NAME: "synthetic/vusenex-tiny"}, "hf_config": _VUSENEX_TINY},
  "vusenex-1b": {"layers": 16, "repo": {ENGINE_CLASS_NAME: "synthetic/vusenex-1b"}, "hf_config": _VUSENEX_1B},
  "mistral-tiny": {"layers": 4, "repo": {ENGINE_CLASS_NAME: "synthetic/mistral-tiny"},
                   "hf_config": _mistral(320, 5, 1, 640, 4, head_dim=64, vocab=1280)},
}


def get_repo(model_id: str, inference_engine_classname: str) -> Optional[str]:
  return model_cards.get(model_id, {}).get("repo", {}).get(inference_engine_classname, None)


def build_base_shard(model_id: str, inference_engine_classname: str) -> Optional[Shard]:
  """models.py:237-242 of the reference: Shard(id, 0, 0, n_layers)."""
  repo = get_repo(model_id, inference_engine_classname)
  n_layers = model_cards.get(model_id, {}).get("layers", 0)
  if repo is None or n_layers < 1:
    return None
  return Shard(model_id, 0, 0, n_layers)


def build_full_shard(model_id: str, inference_engine_classname: str) -> Optional[Shard]:
  base = build_base_shard(model_id, inference_engine_classname)
  if base is None:
    return None
  return Shard(base.model_id, 0, base.n_layers - 1, base.n_layers)
