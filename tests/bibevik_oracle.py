"""Slow restatement of the Bibevik design from its equations, one function per mechanism, in float64 on the CPU.

Shares no code with the engine: tests compare the engine's residual stream and logits with these functions on
configurations and random weights that the tests make themselves.  Every function works on one sequence
(``[T, ...]`` tensors, positions 0..T-1); recurrent mixers are plain token loops.

Notation: h is what a layer's sublayers read (the normed stream), W.x means ``x @ W.T`` (weights are [out, in]).
"""
import math

import torch

F64 = torch.float64


def rms(x, eps):
  return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def scalar_norm(x, g, eps):
  """RMS norm whose weight is a single number."""
  return rms(x, eps) * g.to(F64).reshape(())


def lin(W, x, b=None):
  y = x @ W.to(F64).T
  return y if b is None else y + b.to(F64)


def rotate_pairs(x, pos, base, dims):
  """Rotary positions on the first ``dims`` entries of the last axis; entry 2i is paired with 2i+1, angle
  pos * base^(-2i/dims).  x: [T, ..., n], pos: [T]."""
  half = dims // 2
  freq = base ** (-2.0 * torch.arange(half, dtype=F64) / dims)
  ang = pos.to(F64)[:, None] * freq[None, :]
  shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
  cos, sin = torch.cos(ang).reshape(shape), torch.sin(ang).reshape(shape)
  u, v = x[..., 0:dims:2], x[..., 1:dims:2]
  out = x.clone()
  out[..., 0:dims:2] = u * cos - v * sin
  out[..., 1:dims:2] = v * cos + u * sin
  return out


def latent_attention(w, p, mx, h, eps):
  """Softmax attention whose keys and values are up-projections of a small normed latent, plus one rotated key part
  that all heads share.  mx: {heads, dim, rot_dim, vdim, kv_rank, scale, rot{base, dims}}."""
  T = h.shape[0]
  H, dn, dr, dv, R = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"]
  pos = torch.arange(T)
  q = lin(w[p + "q"], h).reshape(T, H, dn + dr)
  q_plain, q_rot = q[..., :dn], rotate_pairs(q[..., dn:], pos, mx["rot"]["base"], mx["rot"]["dims"])
  down = lin(w[p + "dkv"], h)
  c = rms(down[:, :R], eps) * w[p + "dkv.norm"].to(F64)
  k_rot = rotate_pairs(down[:, R:], pos, mx["rot"]["base"], mx["rot"]["dims"])       # [T, dr], one for all heads
  k_plain = lin(w[p + "uk"], c).reshape(T, H, dn)
  v = lin(w[p + "uv"], c).reshape(T, H, dv)
  score = (torch.einsum("thd,shd->hts", q_plain, k_plain) + torch.einsum("thd,sd->hts", q_rot, k_rot)) * mx["scale"]
  mask = torch.ones(T, T, dtype=torch.bool).tril()
  score = score.masked_fill(~mask, -math.inf)
  a = torch.softmax(score, dim=-1)
  o = torch.einsum("hts,shd->thd", a, v).reshape(T, H * dv)
  return lin(w[p + "o"], o)


def general_delta(w, p, mx, h, eps):
  """Delta rule with a decay and a removal rate per key channel:
  S <- diag(d) S - (a*u)(u^T S) + k v^T (both terms on the old S), o = S^T r."""
  T = h.shape[0]
  H, n = mx["heads"], mx["dim"]
  r = lin(w[p + "r"], h).reshape(T, H, n)
  k = lin(w[p + "k"], h).reshape(T, H, n)
  v = lin(w[p + "v"], h).reshape(T, H, n)
  d = torch.exp(-math.exp(-0.5) * torch.sigmoid(lin(w[p + "w2"], torch.tanh(lin(w[p + "w1"], h))) + w[p + "w0"].to(F64))).reshape(T, H, n)
  a = torch.sigmoid(lin(w[p + "a"], h, w[p + "a.b"])).reshape(T, H, n)
  u = k / torch.sqrt((k * k).sum(dim=-1, keepdim=True) + 1e-6)
  S = torch.zeros(H, n, n, dtype=F64)
  o = torch.zeros(T, H, n, dtype=F64)
  for t in range(T):
    uS = torch.einsum("hi,hij->hj", u[t], S)
    S = d[t][:, :, None] * S - (a[t] * u[t])[:, :, None] * uS[:, None, :] + k[t][:, :, None] * v[t][:, None, :]
    o[t] = torch.einsum("hij,hi->hj", S, r[t])
  o = rms(o, eps).reshape(T, H * n) * w[p + "norm"].to(F64) * torch.sigmoid(lin(w[p + "g"], h))
  return lin(w[p + "o"], o)


def lightning(w, p, mx, h, eps):
  """Linear attention with one constant decay per head: S <- decay S + k v^T, o = S^T q, SiLU on q, k and v."""
  T = h.shape[0]
  H, n, dv = mx["heads"], mx["dim"], mx["vdim"]
  silu = torch.nn.functional.silu
  q = silu(lin(w[p + "q"], h)).reshape(T, H, n)
  k = silu(lin(w[p + "k"], h)).reshape(T, H, n)
  v = silu(lin(w[p + "v"], h)).reshape(T, H, dv)
  decay = torch.tensor(mx["decay"], dtype=F64)
  S = torch.zeros(H, n, dv, dtype=F64)
  o = torch.zeros(T, H, dv, dtype=F64)
  for t in range(T):
    S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
    o[t] = torch.einsum("hij,hi->hj", S, q[t])
  o = rms(o.reshape(T, H * dv), eps) * w[p + "norm"].to(F64) * torch.sigmoid(lin(w[p + "g"], h))
  return lin(w[p + "o"], o)


def clamped_glu(w, p, h, limit, bias):
  """down(g * sigmoid(1.702 g) * (u + 1)) with the gate capped above and the up branch clamped on both sides."""
  b = (lambda n: w[p + n + ".b"]) if bias else (lambda n: None)
  g = torch.clamp(lin(w[p + "gate"], h, b("gate")), max=limit)
  u = torch.clamp(lin(w[p + "up"], h, b("up")), min=-limit, max=limit)
  return lin(w[p + "down"], g * torch.sigmoid(1.702 * g) * (u + 1.0), b("down"))


def route(z, rt):
  """Router logits [T, E] -> (chosen experts [T, top], their weights).  Sigmoid scores; experts in neighbouring groups, a
  group is worth the sum of its two best scores, only the best ``keep`` groups stay eligible; weights are the chosen
  scores times ``scale``, not renormalised."""
  E, top = rt["experts"], rt["top"]
  s = torch.sigmoid(z)
  ok = torch.ones_like(s, dtype=torch.bool)
  groups = rt.get("groups")
  if groups:
    per = E // groups["count"]
    gs = s.reshape(-1, groups["count"], per).topk(min(2, per), dim=-1).values.sum(dim=-1)
    best = gs.topk(groups["keep"], dim=-1).indices
    gmask = torch.zeros_like(gs, dtype=torch.bool).scatter_(1, best, True)
    ok = gmask[:, :, None].expand(-1, -1, per).reshape(-1, E)
  chosen = s.masked_fill(~ok, -1.0).topk(top, dim=-1).indices
  return chosen, s.gather(1, chosen) * rt["scale"]


def moe(w, p, mlp, h):
  rt = mlp["router"]
  chosen, weight = route(lin(w[p + "router"], h), rt)
  y = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=F64)
  for t in range(h.shape[0]):
    for e, g in zip(chosen[t].tolist(), weight[t]):
      y[t] += g * clamped_glu(w, f"{p}e{e}.", h[t:t + 1], mlp["expert"]["limit"], False)[0]
  if mlp.get("shared"):
    y = y + clamped_glu(w, p + "shared.", h, mlp["shared"]["limit"], False)
  return y


def feed_forward(w, p, mlp, h):
  if mlp is None:
    return torch.zeros_like(h)
  if mlp["kind"] == "dense":
    return clamped_glu(w, p, h, mlp["limit"], True)
  return moe(w, p, mlp, h)


MIXERS = {"latent_attention": latent_attention, "general_delta": general_delta, "lightning": lightning}


def forward(cfg, w, tokens, rounding=None):
  """tokens [T] -> (logits [T, V], residual stream after every layer [L, T, D]).  ``rounding``: optional function applied to
  what each layer reads (to imitate a bf16 activation)."""
  w = {k: v.to(F64) if v.is_floating_point() else v for k, v in w.items()}
  eps = cfg["norm"]["eps"]
  x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)] * cfg["embedding"]["scale"]
  stream = []
  for i, lc in enumerate(cfg["layers"]):
    src = lc.get("weights_of", i)
    p = f"l{src}."
    h = scalar_norm(x, w[p + "norm1"], eps)
    if rounding is not None:
      h = rounding(h)
    x = x + (MIXERS[lc["type"]](w, p + "mix.", lc["mixer"], h, eps) + feed_forward(w, p + "mlp.", lc.get("mlp"), h))
    stream.append(x)
  logits = lin(w["head"], scalar_norm(x, w["final.norm"], eps))
  return logits, torch.stack(stream)
