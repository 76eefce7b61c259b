"""Plain fp64 restatement of the Pufivik design, one function per mechanism, sharing no code with the engine.

A model is (cfg, W): cfg the config.json dict, W name -> fp64 tensor.  Everything is computed token by token or with
dense T x T score matrices; nothing is cached, so the oracle of a prompt is the oracle of every way of cutting it.
"""
import math

import torch

F64 = torch.float64


def group_norm(x, w, groups, eps):
  """Rows split in `groups` equal consecutive parts; each part over its own sqrt(mean square + eps); then the weight."""
  T, D = x.shape
  parts = x.reshape(T, groups, D // groups)
  parts = parts / torch.sqrt((parts * parts).mean(dim=-1, keepdim=True) + eps)
  return parts.reshape(T, D) * w


def causal_filter(h, w):
  """h_t + sum_j w[:, j] h_(t - taps + 1 + j), zeros before the start.  w: [D, taps]."""
  T, D = h.shape
  taps = w.shape[1]
  out = h.clone()
  for t in range(T):
    for j in range(taps):
      src = t - taps + 1 + j
      if src >= 0:
        out[t] += w[:, j] * h[src]
  return out


def band_frequencies(rot):
  """f_i = base^(-2i/dims); by wavelength l = 2 pi / f: kept below original/high, divided by factor above original/low,
  blended between."""
  dims, base, sc = rot["dims"], rot["base"], rot.get("scaling")
  out = []
  for i in range(dims // 2):
    f = base ** (-2.0 * i / dims)
    if sc:
      l = 2.0 * math.pi / f
      if l < sc["original"] / sc["high"]:
        pass
      elif l > sc["original"] / sc["low"]:
        f = f / sc["factor"]
      else:
        s = (sc["original"] / l - sc["low"]) / (sc["high"] - sc["low"])
        f = (1.0 - s) * f / sc["factor"] + s * f
    out.append(f)
  return out, 1.0


def ramp_frequencies(rot):
  """f_i = base^(-2i/dims) moved towards f_i / factor along a ramp over i; cos and sin get 0.1 ln(factor) + 1."""
  dims, base, sc = rot["dims"], rot["base"], rot.get("scaling")
  fs = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
  if not sc:
    return fs, 1.0
  where = lambda t: dims * math.log(sc["original"] / (2.0 * math.pi * t)) / (2.0 * math.log(base))  # noqa: E731
  lo = max(math.floor(where(sc["fast"])), 0)
  hi = min(math.ceil(where(sc["slow"])), dims - 1)
  out = []
  for i, f in enumerate(fs):
    r = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
    out.append(f / sc["factor"] * r + f * (1.0 - r))
  return out, 0.1 * math.log(sc["factor"]) + 1.0


def rotate(x, pos, freqs, mult, dims, interleaved):
  """x [T, heads, d]; the first `dims` entries of each head turn by pos * f_i, pairs (2i, 2i+1) or (i, i + dims/2)."""
  y = x.clone()
  for t in range(x.shape[0]):
    for i, f in enumerate(freqs):
      a = float(pos[t]) * f
      c, s = math.cos(a) * mult, math.sin(a) * mult
      i0, i1 = (2 * i, 2 * i + 1) if interleaved else (i, i + dims // 2)
      u, v = x[t, :, i0], x[t, :, i1]
      y[t, :, i0] = u * c - v * s
      y[t, :, i1] = v * c + u * s
  return y


def attention_weights(q, k, scale, softcap=0.0, sink=None):
  """q [T, H, d], k [T, G, d] -> causal weights [H, T, T]; optional soft cap on the scores, optional sink in the denominator."""
  T, H, _ = q.shape
  G = k.shape[1]
  w = torch.zeros(H, T, T, dtype=F64)
  for h in range(H):
    g = h // (H // G)
    for i in range(T):
      sc = (k[: i + 1, g] @ q[i, h]) * scale
      if softcap:
        sc = softcap * torch.tanh(sc / softcap)
      mx = sc.max() if sink is None else torch.maximum(sc.max(), sink[h])
      e = torch.exp(sc - mx)
      den = e.sum() + (torch.exp(sink[h] - mx) if sink is not None else 0.0)
      w[h, i, : i + 1] = e / den
  return w


def mix_heads(w, talk):
  """w'_h = sum_g talk[h, g] w_g."""
  return torch.einsum("hg,gij->hij", talk, w)


def apply_weights(w, v):
  """w [H, T, T], v [T, G, dv] -> [T, H * dv]: head h reads the values of key head h // (H / G)."""
  H, T, _ = w.shape
  G = v.shape[1]
  out = torch.zeros(T, H, v.shape[2], dtype=F64)
  for h in range(H):
    out[:, h] = w[h] @ v[:, h // (H // G)]
  return out.reshape(T, -1)


def experts(h, W, p, n_experts, top):
  """Sigmoid scores, the `top` largest; expert e reads score_e * h; SiLU-gated; outputs summed."""
  T = h.shape[0]
  s = torch.sigmoid(h @ W[p + "router"].T)
  y = torch.zeros_like(h)
  for t in range(T):
    order = sorted(range(n_experts), key=lambda e: (-float(s[t, e]), e))[:top]
    for e in order:
      x = s[t, e] * h[t]
      g, u = W[f"{p}e{e}.gate"] @ x, W[f"{p}e{e}.up"] @ x
      y[t] += W[f"{p}e{e}.down"] @ (g * torch.sigmoid(g) * u)
  return y


def mixer(cfg, W, i, h, pos, v_first):
  """One attention layer on its (filtered) input h [T, D].  Returns (output [T, D], v_first)."""
  lc = cfg["layers"][i]
  mx, p = lc["mixer"], f"l{i}.mix."
  T = h.shape[0]
  H, G, dk, dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
  q = (h @ W[p + "q"].T).reshape(T, H, dk)
  k = (h @ W[p + "k"].T).reshape(T, G, dk)
  v = (h @ W[p + "v"].T).reshape(T, G, dv)
  rot = mx.get("rot")
  sinky = lc["type"] == "attention"
  if rot and rot.get("dims"):
    fs, mult = band_frequencies(rot) if sinky else ramp_frequencies(rot)
    q = rotate(q, pos, fs, mult, rot["dims"], not sinky)
    k = rotate(k, pos, fs, mult, rot["dims"], not sinky)
  if mx.get("v_mix"):
    if v_first is None:
      v_first = v
    else:
      lam = W[p + "vmix"]
      v = (1.0 - lam) * v + lam * v_first
  if sinky:
    w = mix_heads(attention_weights(q, k, mx["scale"], 0.0, W[p + "sink"]), W[p + "talk"])
    o = apply_weights(w, v).reshape(T, H, dv) * torch.sigmoid(h @ W[p + "g"].T)[:, :, None]
    o = o.reshape(T, -1)
  else:
    o = apply_weights(attention_weights(q, k, mx["scale"], mx.get("softcap") or 0.0, None), v)
  return o @ W[p + "o"].T, v_first


def forward(cfg, W, tokens, pos0=0, return_layers=False):
  """Logits [T, vocab] of one sequence processed whole."""
  W = {k: v.to(F64) for k, v in W.items()}
  eps, groups, m = cfg["norm"]["eps"], cfg["norm"].get("groups", 1), cfg.get("residual_mult", 1.0)
  taps = (cfg.get("canon") or {}).get("taps", 0)
  T = len(tokens)
  pos = [pos0 + t for t in range(T)]
  x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)] * cfg["embedding"]["scale"]
  v_first, stream = None, []
  for i, lc in enumerate(cfg["layers"]):
    p = f"l{i}."
    h = group_norm(x, W[p + "norm1"], groups, eps)
    if taps:
      h = causal_filter(h, W[p + "canon1"])
    y, v_first = mixer(cfg, W, i, h, pos, v_first)
    x = x + m * group_norm(y, W[p + "norm1b"], groups, eps)
    mlp = lc.get("mlp")
    if mlp:
      h2 = group_norm(x, W[p + "norm2"], groups, eps)
      y = experts(h2, W, p + "mlp.", mlp["router"]["experts"], mlp["router"]["top"])
      x = x + m * group_norm(y, W[p + "norm2b"], groups, eps)
    stream.append(x.clone())
  logits = group_norm(x, W["final.norm"], groups, eps) @ W["embed"].T
  return (logits, stream) if return_layers else logits
