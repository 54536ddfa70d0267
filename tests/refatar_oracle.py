"""Plain, slow restatement of the Refatar design for tests: one function per mechanism, torch on the CPU in
float64, whole sequences at once, no cache.  It shares no code with the product path (csrc/xb_hybrid*.cuh);
the state that the product carries between calls does not exist here because every call starts at token 0.

Notation: D = model width, T = tokens of the sequence, weights are [out, in] and applied as W @ x.
"""
import math

import torch

F64 = torch.float64


def rms_unit(x, eps):
  """x scaled to unit root mean square over its last axis (eps inside the root)."""
  return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_offset(x, w, eps):
  """RMS norm whose stored weight is an offset from one."""
  return rms_unit(x, eps) * (1.0 + w)


def norm_plain(x, w, eps):
  return rms_unit(x, eps) * w


def gelu_tanh(z):
  return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
  return z * torch.sigmoid(z)


def causal_taps(h, w):
  """Depthwise causal filter over time.  h [T, C], w [C, taps]; the LAST column weighs the current token,
  column j the token taps-1-j steps back; inputs before the sequence are zero."""
  T, C = h.shape
  taps = w.shape[1]
  out = torch.zeros_like(h)
  for j in range(taps):
    back = taps - 1 - j
    if back < T:
      out[back:] += h[: T - back] * w[:, j]
  return out


def input_filter(h, w):
  """What a sublayer reads: its normed input plus the causal filter of it."""
  return h + causal_taps(h, w)


def window_mask(T, size, keep_first):
  """[T, T] bool: query i sees key j when j <= i and (i - j < size or j < keep_first)."""
  i = torch.arange(T)[:, None]
  j = torch.arange(T)[None, :]
  return (j <= i) & ((i - j < size) | (j < keep_first))


def softmax_window_attention(h, p, c):
  """Grouped-query softmax attention without rotation, window + kept first tokens, sigmoid output gate."""
  T = h.shape[0]
  H, G, dk, dv = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
  q = (h @ p["q"].T + p["q.b"]).view(T, H, dk)
  k = (h @ p["k"].T + p["k.b"]).view(T, G, dk)
  v = (h @ p["v"].T + p["v.b"]).view(T, G, dv)
  mask = window_mask(T, c["mask"]["size"], c["mask"]["keep_first"])
  out = torch.zeros(T, H, dv, dtype=h.dtype)
  for hh in range(H):
    g = hh // (H // G)
    s = (q[:, hh] @ k[:, g].T) * c["scale"]
    s = s.masked_fill(~mask, float("-inf"))
    out[:, hh] = torch.softmax(s, dim=-1) @ v[:, g]
  gate = torch.sigmoid(h @ p["g"].T)
  return (out.reshape(T, H * dv) * gate) @ p["o"].T


def hgrn2(h, p, c, eps):
  """Linear attention whose forget gate also sets the write strength: S <- diag(f) S + (1 - f) v^T, o = S^T q."""
  T = h.shape[0]
  H, dk, dv = c["heads"], c["dim"], c["vdim"]
  q = silu(h @ p["q"].T).view(T, H, dk)
  v = (h @ p["v"].T).view(T, H, dv)
  low = p["lower"]
  f = (low + (1.0 - low) * torch.sigmoid(h @ p["f"].T + p["f.b"])).view(T, H, dk)
  S = torch.zeros(H, dk, dv, dtype=h.dtype)
  o = torch.zeros(T, H, dv, dtype=h.dtype)
  for t in range(T):
    S = f[t][:, :, None] * S + (1.0 - f[t])[:, :, None] * v[t][:, None, :]
    o[t] = torch.einsum("hkv,hk->hv", S, q[t])
  o = norm_plain(o, p["norm"], eps)
  return o.reshape(T, H * dv) @ p["o"].T


def parallel_mixer(h, p, c, eps):
  left = softmax_window_attention(h, {k[5:]: v for k, v in p.items() if k.startswith("left.")}, c["left"])
  right = hgrn2(h, {k[6:]: v for k, v in p.items() if k.startswith("right.")}, c["right"], eps)
  return c["left_scale"] * left + c["right_scale"] * right


def gated_delta(h, p, c, eps):
  """Gated delta rule: S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q (read after the write)."""
  T = h.shape[0]
  H, G, dk, dv = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
  q = silu(causal_taps(h @ p["q"].T, p["q.conv"])).view(T, G, dk)
  k = silu(causal_taps(h @ p["k"].T, p["k.conv"])).view(T, G, dk)
  v = silu(causal_taps(h @ p["v"].T, p["v.conv"])).view(T, H, dv)
  q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
  k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
  beta = torch.sigmoid(h @ p["b"].T)                                                # [T, H]
  decay = torch.exp(-torch.exp(p["A_log"]) * torch.nn.functional.softplus(h @ p["a"].T + p["dt_bias"]))
  rep = H // G
  S = torch.zeros(H, dk, dv, dtype=h.dtype)
  o = torch.zeros(T, H, dv, dtype=h.dtype)
  for t in range(T):
    kt = k[t].repeat_interleave(rep, 0)                                             # head hh uses q/k head hh // rep
    qt = q[t].repeat_interleave(rep, 0)
    S = decay[t][:, None, None] * S
    u = beta[t][:, None] * (v[t] - torch.einsum("hkv,hk->hv", S, kt))
    S = S + kt[:, :, None] * u[:, None, :]
    o[t] = torch.einsum("hkv,hk->hv", S, qt)
  o = norm_plain(o, p["norm"], eps) * silu(h @ p["g"].T).view(T, H, dv)
  return o.reshape(T, H * dv) @ p["o"].T


def dense_ff(h, p):
  return torch.relu(h @ p["up"].T) ** 2 @ p["down"].T


def token_side(x, tokens, layer, p, side_embed, dim, eps):
  e = side_embed[tokens][:, layer * dim:(layer + 1) * dim]
  y = (gelu_tanh(x @ p["gate"].T) * e) @ p["proj"].T
  return x + rms_unit(y, eps) * p["norm"]


def sub(weights, prefix):
  return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def forward(config, weights, tokens, return_layers=False):
  """tokens: list of ids of ONE sequence.  Returns float64 logits [T, vocab] (and the residual stream after each layer)."""
  w = {k: v.to(F64) if v.is_floating_point() else v for k, v in weights.items()}
  eps = config["norm"]["eps"]
  tok = torch.as_tensor(tokens, dtype=torch.long)
  x = w["embed"][tok]
  taps_on = config.get("canon") is not None
  side = config.get("token_side")
  layers = []
  for i, lc in enumerate(config["layers"]):
    L = sub(w, f"l{i}.")
    h = norm_offset(x, L["norm1"], eps)
    if taps_on:
      h = input_filter(h, L["canon1"])
    mix = sub(L, "mix.")
    if lc["type"] == "parallel":
      m = parallel_mixer(h, mix, lc["mixer"], eps)
    elif lc["type"] == "delta":
      m = gated_delta(h, mix, lc["mixer"], eps)
    else:
      raise ValueError(lc["type"])
    x = x + norm_offset(m, L["norm1b"], eps)
    if lc.get("mlp") is not None:
      h = norm_offset(x, L["norm2"], eps)
      if taps_on:
        h = input_filter(h, L["canon2"])
      x = x + norm_offset(dense_ff(h, sub(L, "mlp.")), L["norm2b"], eps)
    if side is not None:
      x = token_side(x, tok, i, sub(L, "side."), w["side.embed"], side["dim"], eps)
    layers.append(x.clone())
  logits = norm_offset(x, w["final.norm"], eps) @ w["head"].T
  cap = config.get("logit_softcap")
  if cap:
    logits = cap * torch.tanh(logits / cap)
  return (logits, layers) if return_layers else logits
