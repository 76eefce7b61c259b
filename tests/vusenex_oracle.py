"""Vusenex restated from its equations: a plain, slow float64 implementation, one function per mechanism.

It shares no code with the engine.  ``state``: name -> torch tensor (any float type; everything is taken to float64),
``cfg``: the design's ``config.json`` as a dict.  Attention is evaluated with dense ``[T, T]`` score matrices.

Notation.  A layer works on the stream ``x`` [T, D] directly (there is no norm in front of a sublayer):

    x <- x + n1 * unit(sigmoid(A1 x + a1) * mixer(x)),      x <- x + n2 * unit(sigmoid(A2 x + a2) * experts(x))

with ``unit(y) = y / sqrt(mean(y^2) + eps)`` over the row and ``n1``, ``n2`` single numbers.
"""
import math

import numpy as np
import torch


def _t(state, name):
  return state[name].detach().to(torch.float64).cpu().numpy()


def unit(y, eps):
  """Rows divided by their root mean square, eps inside the root."""
  return y / np.sqrt(np.mean(y * y, axis=-1, keepdims=True) + eps)


def sigmoid(z):
  return 1.0 / (1.0 + np.exp(-z))


def gelu_erf(z):
  erf = np.vectorize(math.erf)
  return 0.5 * z * (1.0 + erf(z / math.sqrt(2.0)))


def embed_rows(state, cfg, tokens):
  """Token row + hashed row of the (previous, current) pair + learned position row."""
  bg = cfg["embedding"]["bigram"]
  nb, mp, mc = int(bg["buckets"]), int(bg["mul_prev"]), int(bg["mul_cur"])
  E, B, Pm = _t(state, "embed"), _t(state, "bigram"), _t(state, "pos")
  x = np.zeros((len(tokens), E.shape[1]))
  for p, tok in enumerate(tokens):
    row = nb if p == 0 else (int(tokens[p - 1]) * mp + int(tok) * mc) % nb
    x[p] = E[int(tok)] + B[row] + Pm[p]
  return x


def softmax_attention(state, pre, mx, x, eps):
  """Grouped-query attention whose values are the projected keys: both projections normed over their whole width, queries
  scaled by a slowly growing function of the position, a logarithmic distance penalty per head, one extra unit in the
  softmax denominator."""
  T = x.shape[0]
  H, G, dk = int(mx["heads"]), int(mx["kv_heads"]), int(mx["dim"])
  q = x @ _t(state, pre + "q").T + _t(state, pre + "q.b")
  k = x @ _t(state, pre + "k").T + _t(state, pre + "k.b")
  v = k.copy()                                     # values: the keys as projected
  q = unit(q, eps) * _t(state, pre + "q.norm")
  k = unit(k, eps) * _t(state, pre + "k.norm")
  qt = mx.get("q_temp")
  if qt:
    pos = np.arange(T)
    q = q * (1.0 + float(qt["coef"]) * np.log(np.floor((pos + 1) / int(qt["every"])) + 1.0))[:, None]
  r1, r2 = _t(state, pre + "r1"), _t(state, pre + "r2")
  i, j = np.arange(T)[:, None], np.arange(T)[None, :]
  dist = np.maximum(i - j, 0).astype(np.float64)
  out = np.zeros((T, H * dk))
  for h in range(H):
    g = h // (H // G)
    s = (q[:, h * dk:(h + 1) * dk] @ k[:, g * dk:(g + 1) * dk].T) * float(mx["scale"]) - r1[h] * np.log1p(r2[h] * dist)
    s = np.where(j <= i, s, -np.inf)
    mxs = np.maximum(s.max(axis=1, keepdims=True), 0.0)
    e = np.exp(s - mxs)
    w = e / (np.exp(-mxs) + e.sum(axis=1, keepdims=True))
    out[:, h * dk:(h + 1) * dk] = w @ v[:, g * dk:(g + 1) * dk]
  return out @ _t(state, pre + "o").T


def latent_attention(state, pre, mx, x, eps):
  """Keys and values are per-head images of one small normed vector per token; no positions; ordinary softmax."""
  T = x.shape[0]
  H, dk, dv = int(mx["heads"]), int(mx["dim"]), int(mx["vdim"])
  q = x @ _t(state, pre + "q").T
  c = unit(x @ _t(state, pre + "dkv").T, eps) * _t(state, pre + "dkv.norm")
  k = c @ _t(state, pre + "uk").T
  v = c @ _t(state, pre + "uv").T
  i, j = np.arange(T)[:, None], np.arange(T)[None, :]
  out = np.zeros((T, H * dv))
  for h in range(H):
    s = (q[:, h * dk:(h + 1) * dk] @ k[:, h * dk:(h + 1) * dk].T) * float(mx["scale"])
    s = np.where(j <= i, s, -np.inf)
    e = np.exp(s - s.max(axis=1, keepdims=True))
    out[:, h * dv:(h + 1) * dv] = (e / e.sum(axis=1, keepdims=True)) @ v[:, h * dv:(h + 1) * dv]
  return out @ _t(state, pre + "o").T


def route(z, top, groups, keep):
  """Router logits of one token -> {expert: weight}.  Softmax scores; a group is worth its best score and only the best
  ``keep`` groups stay eligible; the ``top`` best eligible experts share weight in proportion to their scores."""
  E = len(z)
  s = np.exp(z - z.max())
  s = s / s.sum()
  ok = np.ones(E, dtype=bool)
  if groups and keep < groups:
    per = E // groups
    gs = [s[g * per:(g + 1) * per].max() for g in range(groups)]
    order = sorted(range(groups), key=lambda g: (-gs[g], g))
    ok[:] = False
    for g in order[:keep]:
      ok[g * per:(g + 1) * per] = True
  cand = sorted([e for e in range(E) if ok[e]], key=lambda e: (-s[e], e))[:top]
  tot = sum(s[e] for e in cand) + 1e-20
  return {e: s[e] / tot for e in cand}


def experts(state, pre, mlp, x):
  rt = mlp["router"]
  E, top = int(rt["experts"]), int(rt["top"])
  gr = rt.get("groups")
  groups, keep = (int(gr["count"]), int(gr["keep"])) if gr else (0, 0)
  Z = x @ _t(state, pre + "router").T
  ups = [_t(state, f"{pre}e{e}.up") for e in range(E)]
  downs = [_t(state, f"{pre}e{e}.down") for e in range(E)]
  y = np.zeros_like(x)
  for t in range(x.shape[0]):
    for e, w in route(Z[t], top, groups, keep).items():
      y[t] += w * (downs[e] @ gelu_erf(ups[e] @ x[t]))
  if mlp.get("shared"):
    y += gelu_erf(x @ _t(state, pre + "shared.up").T) @ _t(state, pre + "shared.down").T
  return y


def forward(state, cfg, tokens, want_layers=False):
  """tokens of ONE sequence from position 0 -> float64 logits [T, vocab] (and the stream after every layer)."""
  eps = float(cfg["norm"]["eps"])
  x = embed_rows(state, cfg, tokens)
  per_layer = []
  for li, lc in enumerate(cfg["layers"]):
    p = f"l{li}."
    fn = {"attention": softmax_attention, "latent_attention": latent_attention}[lc["type"]]
    y = fn(state, p + "mix.", lc["mixer"], x, eps)
    y = y * sigmoid(x @ _t(state, p + "rg1").T + _t(state, p + "rg1.b"))
    x = x + unit(y, eps) * _t(state, p + "norm1").reshape(-1)[0]
    if lc.get("mlp") is not None:
      y = experts(state, p + "mlp.", lc["mlp"], x)
      y = y * sigmoid(x @ _t(state, p + "rg2").T + _t(state, p + "rg2.b"))
      x = x + unit(y, eps) * _t(state, p + "norm2").reshape(-1)[0]
    per_layer.append(x.copy())
  logits = (unit(x, eps) * _t(state, "final.norm").reshape(-1)[0]) @ _t(state, "head").T
  return (logits, per_layer) if want_layers else logits
