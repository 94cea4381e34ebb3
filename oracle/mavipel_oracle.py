"""Plain, slow restatement of the Mavipel decoder in PyTorch on the CPU: one function per mechanism, whole sequences
at a time, explicit loops over positions where a mechanism is a recurrence or a mask, no cache, no batching.
Test infrastructure only: the product package never imports it and it imports nothing of the product.

Notation: T tokens, D model width, H heads, G key/value heads, dk query/key size per head, dv value size, F
feed-forward width, E experts.  ``w`` maps tensor names to [out, in] matrices (or vectors); ``cfg`` is the dictionary
form of a checkpoint's ``config.json``."""
from __future__ import annotations

import math
from typing import Dict, List

import torch
import torch.nn.functional as F


# ------------------------------------------------------------------------------------------------ norms, activations
def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis"""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def group_norm(x, weight, groups: int, eps: float):
    """the last axis in `groups` equal consecutive parts, each divided by its own root mean square; then the weight"""
    shape = x.shape
    parts = x.reshape(*shape[:-1], groups, shape[-1] // groups)
    return unit_rms(parts, eps).reshape(shape) * weight


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def unit_vector(x, tiny: float = 1e-6):
    """x / sqrt(sum(x^2) + tiny) over the last axis"""
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + tiny)


# ------------------------------------------------------------------------------------------------ short convolution
def causal_conv(x, taps):
    """x [T, C], taps [C, n] (last column weighs the current position, zeros before the start) -> [T, C]"""
    T, C = x.shape
    n = taps.shape[1]
    out = torch.zeros_like(x)
    for t in range(T):
        for j in range(n):
            s = t - (n - 1 - j)
            if s >= 0:
                out[t] += taps[:, j] * x[s]
    return out


# ------------------------------------------------------------------------------------------------ rotation
def rotate_interleaved(x, positions, dims: int, base: float):
    """turns coordinate pairs (2i, 2i + 1), i < dims / 2, of the last axis of x [T, heads, d] by position * base^(-2i/dims)"""
    half = dims // 2
    i = torch.arange(half, dtype=torch.float64)
    ang = positions.to(torch.float64)[:, None] * (base ** (-2.0 * i / dims))[None]
    cos, sin = ang.cos().to(x.dtype)[:, None, :], ang.sin().to(x.dtype)[:, None, :]
    out = x.clone()
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


# ------------------------------------------------------------------------------------------------ mixers
def gated_delta_mixer(h, w: Dict[str, torch.Tensor], m: dict, eps: float):
    """Gated delta rule with a decay per key channel.  h [T, D]; w holds the mixer's tensors by their short names."""
    T = h.shape[0]
    H, dk = m["heads"], m["dim"]
    G, dv = m.get("kv_heads", H), m.get("vdim", dk)
    q = silu(causal_conv(h @ w["q"].T, w["q.conv"])).reshape(T, G, dk)
    k = silu(causal_conv(h @ w["k"].T, w["k.conv"])).reshape(T, G, dk)
    v = silu(causal_conv(h @ w["v"].T, w["v.conv"])).reshape(T, H, dv)
    q = unit_vector(q) * dk ** -0.5
    k = unit_vector(k)
    beta = torch.sigmoid(h @ w["b"].T)                                                  # [T, H]
    rate = torch.exp(w["A_log"])[None, :, None]                                          # [1, H, 1]
    decay = torch.exp(-rate * F.softplus((h @ w["a1"].T) @ w["a2"].T + w["dt_bias"]).reshape(T, H, dk))
    gate = torch.sigmoid((h @ w["g1"].T) @ w["g2"].T).reshape(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for hd in range(H):
        g = hd // (H // G)
        S = torch.zeros(dk, dv, dtype=h.dtype)
        for t in range(T):
            S = decay[t, hd][:, None] * S
            u = beta[t, hd] * (v[t, hd] - S.T @ k[t, g])
            S = S + torch.outer(k[t, g], u)
            out[t, hd] = S.T @ q[t, g]
    out = unit_rms(out, eps) * w["norm"] * gate
    return out.reshape(T, H * dv) @ w["o"].T


def talking_window_attention(h, positions, w, m: dict, eps: float):
    """Softmax attention over a sliding window with capped scores that are mixed across heads before the softmax,
    and a sink per head in the denominator."""
    T = h.shape[0]
    H, dk = m["heads"], m["dim"]
    G, dv = m.get("kv_heads", H), m.get("vdim", dk)
    q = (h @ w["q"].T + w["q.b"]).reshape(T, H, dk)
    k = (h @ w["k"].T + w["k.b"]).reshape(T, G, dk)
    v = (h @ w["v"].T + w["v.b"]).reshape(T, G, dv)
    q = unit_rms(q, eps) * w["q.norm"]
    k = unit_rms(k, eps) * w["k.norm"]
    rot = m.get("rot") or {}
    if rot.get("dims", 0):
        q = rotate_interleaved(q, positions, rot["dims"], rot["base"])
        k = rotate_interleaved(k, positions, rot["dims"], rot["base"])
    size = (m.get("mask") or {}).get("size")
    cap = m.get("softcap")
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for i in range(T):
        lo = 0 if size is None else max(0, i - size + 1)
        s = torch.stack([k[lo:i + 1, hd // (H // G)] @ q[i, hd] for hd in range(H)]) * m["scale"]     # [H, n]
        if cap:
            s = cap * torch.tanh(s / cap)
        s = w["talk"] @ s
        top = torch.maximum(s.max(-1).values, w["sink"])
        e = torch.exp(s - top[:, None])
        p = e / (e.sum(-1) + torch.exp(w["sink"] - top))[:, None]
        for hd in range(H):
            out[i, hd] = p[hd] @ v[lo:i + 1, hd // (H // G)]
    return out.reshape(T, H * dv) @ w["o"].T


def general_delta_mixer(h, w, m: dict, eps: float):
    """Generalised delta rule: a decay per key channel, a removal along the unit key with its own rate per channel,
    then the write; both the decay and the removal read the state the step started from."""
    T = h.shape[0]
    H, dk = m["heads"], m["dim"]
    r = (h @ w["r"].T).reshape(T, H, dk)
    k = (h @ w["k"].T).reshape(T, H, dk)
    v = (h @ w["v"].T).reshape(T, H, dk)
    decay = torch.exp(-math.exp(-0.5) * torch.sigmoid(torch.tanh(h @ w["w1"].T) @ w["w2"].T + w["w0"])).reshape(T, H, dk)
    rate = torch.sigmoid(h @ w["a"].T + w["a.b"]).reshape(T, H, dk)
    u = unit_vector(k)
    out = torch.zeros(T, H, dk, dtype=h.dtype)
    for hd in range(H):
        S = torch.zeros(dk, dk, dtype=h.dtype)
        for t in range(T):
            S = decay[t, hd][:, None] * S - torch.outer(rate[t, hd] * u[t, hd], u[t, hd] @ S) + torch.outer(k[t, hd], v[t, hd])
            out[t, hd] = S.T @ r[t, hd]
    out = unit_rms(out, eps).reshape(T, H * dk) * w["norm"] * torch.sigmoid(h @ w["g"].T)
    return out @ w["o"].T


def sub(w: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: t for k, t in w.items() if k.startswith(prefix)}


def parallel_mixer(h, positions, w, m: dict, eps: float):
    return (m.get("left_scale", 1.0) * talking_window_attention(h, positions, sub(w, "left."), m["left"], eps)
            + m.get("right_scale", 1.0) * general_delta_mixer(h, sub(w, "right."), m["right"], eps))


# ------------------------------------------------------------------------------------------------ feed-forward
def gated_expert(h, w):
    return (silu(h @ w["gate"].T) * (h @ w["up"].T)) @ w["down"].T


def feed_forward(h, w, f: dict):
    if f["kind"] == "dense":
        return gelu_tanh(h @ w["up"].T) @ w["down"].T
    E, top = f["router"]["experts"], f["router"]["top"]
    z = h.float() @ w["router"].float().T + w["router.b"].float()
    val, idx = torch.topk(z, top, dim=-1)
    gates = torch.softmax(val, -1).to(h.dtype)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(idx[t, j])
            out[t] += gates[t, j] * gated_expert(h[t:t + 1], sub(w, f"e{e}."))[0]
    if f.get("shared"):
        out = out + gated_expert(h, sub(w, "shared."))
    return out


# ------------------------------------------------------------------------------------------------ the model
def layer_runs(cfg: dict) -> List[tuple]:
    """(layer, pass or -1, first of its pass) for every layer execution in order"""
    n = len(cfg["layers"])
    lp = cfg.get("loop")
    if not lp:
        return [(i, -1, False) for i in range(n)]
    a, b, times = lp["start"], lp["stop"], lp["times"]
    runs = [(i, -1, False) for i in range(a)]
    for t in range(times):
        runs += [(i, t, i == a) for i in range(a, b)]
    return runs + [(i, -1, False) for i in range(b, n)]


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens, dtype=torch.float64, layers_out: list = None):
    """logits [T, vocab] of one sequence from position 0; every tensor is taken to ``dtype`` first"""
    w = {k: (t.to(dtype) if t.is_floating_point() else t) for k, t in w.items()}
    eps, groups = cfg["norm"]["eps"], cfg["norm"]["groups"]
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(len(tokens))
    x = group_norm(w["embed"][tokens], w["embed.norm"], groups, eps)
    for i, t, first in layer_runs(cfg):
        if first:
            x = x + w["loop.step"][t]
        L, lw = cfg["layers"][i], sub(w, f"l{i}.")
        hn = group_norm(x, lw["norm1"], groups, eps)
        if L["type"] == "channel_delta":
            x = x + gated_delta_mixer(hn, sub(lw, "mix."), L["mixer"], eps)
        elif L["type"] == "parallel":
            x = x + parallel_mixer(hn, positions, sub(lw, "mix."), L["mixer"], eps)
        else:
            raise ValueError(L["type"])
        if L.get("mlp"):
            x = x + feed_forward(group_norm(x, lw["norm2"], groups, eps), sub(lw, "mlp."), L["mlp"])
        if layers_out is not None:
            layers_out.append(x.clone())
    return group_norm(x, w["final.norm"], groups, eps) @ w["head"].T


# ------------------------------------------------------------------------------------------------ random models
def tensor_shapes(cfg: dict) -> Dict[str, tuple]:
    """every tensor of a checkpoint of this configuration, by name.  The inner sizes of the two-matrix projections are
    no configuration keys of a checkpoint (its tensor shapes give them); a test's dictionary carries them as
    ``decay_rank`` / ``gate_rank`` beside the mixer's sizes."""
    D, V = cfg["width"], cfg["vocab"]
    s = {"embed": (V, D), "embed.norm": (D,), "final.norm": (D,), "head": (V, D)}
    if cfg.get("loop"):
        s["loop.step"] = (cfg["loop"]["times"], D)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        s[p + "norm1"] = (D,)
        if L["type"] == "channel_delta":
            H, G, dk, dv, n = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m.get("vdim", m["dim"]), m.get("conv", 1)
            x = p + "mix."
            s.update({x + "q": (G * dk, D), x + "q.conv": (G * dk, n), x + "k": (G * dk, D), x + "k.conv": (G * dk, n),
                      x + "v": (H * dv, D), x + "v.conv": (H * dv, n), x + "b": (H, D), x + "A_log": (H,), x + "norm": (dv,),
                      x + "a1": (m["decay_rank"], D), x + "a2": (H * dk, m["decay_rank"]), x + "dt_bias": (H * dk,),
                      x + "g1": (m["gate_rank"], D), x + "g2": (H * dv, m["gate_rank"]), x + "o": (D, H * dv)})
        else:
            a, r = m["left"], m["right"]
            H, G, dk, dv = a["heads"], a.get("kv_heads", a["heads"]), a["dim"], a.get("vdim", a["dim"])
            x, y, nr = p + "mix.left.", p + "mix.right.", r["heads"] * r["dim"]
            s.update({x + "q": (H * dk, D), x + "q.b": (H * dk,), x + "k": (G * dk, D), x + "k.b": (G * dk,),
                      x + "v": (G * dv, D), x + "v.b": (G * dv,), x + "q.norm": (dk,), x + "k.norm": (dk,),
                      x + "talk": (H, H), x + "sink": (H,), x + "o": (D, H * dv)})
            s.update({y + "r": (nr, D), y + "k": (nr, D), y + "v": (nr, D), y + "g": (nr, D), y + "a": (nr, D),
                      y + "a.b": (nr,), y + "w1": (r["decay_rank"], D), y + "w2": (nr, r["decay_rank"]), y + "w0": (nr,),
                      y + "norm": (nr,), y + "o": (D, nr)})
        f = L.get("mlp")
        if f:
            s[p + "norm2"] = (D,)
            x = p + "mlp."
            if f["kind"] == "dense":
                s.update({x + "up": (f["ff"], D), x + "down": (D, f["ff"])})
            else:
                E, F = f["router"]["experts"], f["expert"]["ff"]
                s.update({x + "router": (E, D), x + "router.b": (E,)})
                for e in range(E):
                    s.update({x + f"e{e}.gate": (F, D), x + f"e{e}.up": (F, D), x + f"e{e}.down": (D, F)})
                if f.get("shared"):
                    Fs = f["shared"]["ff"]
                    s.update({x + "shared.gate": (Fs, D), x + "shared.up": (Fs, D), x + "shared.down": (D, Fs)})
    return s


def random_model(cfg: dict, seed: int, scale: float = 1.0) -> Dict[str, torch.Tensor]:
    """weights whose every mechanism matters in the logits: matrices of unit-variance outputs, norm weights around
    one, a head mix that is far from the identity, sinks, biases and decay parameters of order one"""
    g = torch.Generator().manual_seed(seed)
    w = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.rsplit(".", 1)[-1]
        rnd = lambda: torch.randn(shape, generator=g)
        if leaf in ("norm1", "norm2", "norm"):
            t = 1.0 + 0.3 * rnd()
        elif leaf == "conv":
            t = 0.6 * rnd()
        elif leaf == "talk":
            t = torch.eye(shape[0]) + 0.4 * rnd()
        elif leaf in ("sink", "A_log", "w0"):
            t = rnd()
        elif leaf == "dt_bias":
            t = rnd() - 1.0
        elif leaf == "b" and len(shape) == 1:
            t = 0.5 * rnd()
        elif leaf == "step":
            t = 0.5 * rnd()
        elif leaf == "embed":
            t = rnd()
        else:
            t = rnd() * (scale / math.sqrt(shape[-1]))
        w[name] = t.to(torch.bfloat16)          # what a checkpoint stores
    return w
