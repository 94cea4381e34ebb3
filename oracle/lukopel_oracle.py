"""Plain, slow restatement of the Lukopel decoder in PyTorch on the CPU: one function per mechanism, whole sequences
at a time, explicit masks, no cache, no batching.  Test infrastructure only: the product package never imports it and
it imports nothing of the product.

Notation: T tokens, D model width, S residual streams, H heads, G key/value heads, dk query/key size per head, dv value
size, F feed-forward width.  ``w`` maps tensor names to [out, in] matrices (or vectors); ``cfg`` is the dictionary form
of a checkpoint's ``config.json``."""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


# ------------------------------------------------------------------------------------------------ norms, activations
def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis"""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, weight, eps: float):
    return unit_rms(x, eps) * weight


def relu_squared(z):
    return torch.relu(z) ** 2


# ------------------------------------------------------------------------------------------------ embedding
def embed_tokens(tokens: List[int], table, pos_table, scale: float, first_pos: int = 0):
    """table[token] * scale + pos_table[position]; positions count from first_pos"""
    ids = torch.tensor(tokens, dtype=torch.long)
    p = torch.arange(first_pos, first_pos + len(tokens))
    return table[ids] * scale + pos_table[p]


# ------------------------------------------------------------------------------------------------ residual streams
def streams_read(xs, w_in):
    """xs [S, T, D], w_in [S] -> the sublayer's input before its norm, [T, D]"""
    return torch.einsum("s,std->td", w_in, xs)


def streams_write(xs, y, w_mix, w_out):
    """all streams at once from the old ones: new[t] = sum_s w_mix[s, t] old[s] + w_out[t] y"""
    return torch.einsum("sr,std->rtd", w_mix, xs) + w_out[:, None, None] * y[None]


# ------------------------------------------------------------------------------------------------ masks, biases
def causal_mask(T: int):
    i = torch.arange(T)
    return i[None, :] <= i[:, None]


def same_chunk_mask(T: int, size: int):
    """i sees j <= i of its own chunk; chunks are counted from position 0"""
    i = torch.arange(T)
    return causal_mask(T) & ((i[:, None] // size) == (i[None, :] // size))


def distance_bucket(n: int, rows: int, far: int) -> int:
    """row of the bias table for distance n >= 0: one row per distance below rows / 2, then logarithmic steps that
    reach the last row at distance `far`"""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def distance_bias(T: int, table, far: int):
    """table [rows, H] -> bias [H, T, T] for i >= j (zero elsewhere; masked anyway)"""
    rows, H = table.shape
    out = torch.zeros(H, T, T, dtype=table.dtype)
    for i in range(T):
        for j in range(i + 1):
            out[:, i, j] = table[distance_bucket(i - j, rows, far)]
    return out


def query_temperature(T: int, coef: float, every: int):
    """factor of the queries at positions 0 .. T-1"""
    p = torch.arange(T)
    return 1.0 + coef * torch.log(torch.div(p + 1, every, rounding_mode="floor").to(torch.float64) + 1.0)


def masked_softmax(scores, mask):
    """scores [H, T, T], mask [T, T] (True: visible)"""
    return torch.softmax(scores.masked_fill(~mask[None], float("-inf")), dim=-1)


# ------------------------------------------------------------------------------------------------ mixers
def biased_attention(h, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float):
    """mixer "attention": per-head query/key norm with one weight for all heads, queries scaled by a slowly growing
    function of the position, unit-RMS values, a learned bias per (distance bucket, head) on the scores, causal softmax,
    softmax weights mixed across the heads, a sigmoid gate per head, output projection"""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).reshape(T, H, dk)
    k = (h @ w[p + "k"].T).reshape(T, G, dk)
    v = (h @ w[p + "v"].T).reshape(T, G, dv)
    q = rms_norm(q, w[p + "q.norm"], eps)
    k = rms_norm(k, w[p + "k.norm"], eps)
    q = q * query_temperature(T, m["q_temp"]["coef"], m["q_temp"]["every"]).to(q.dtype)[:, None, None]
    v = unit_rms(v, eps)
    rep = H // G
    kh = k.repeat_interleave(rep, dim=1)                        # head h reads key/value head h // rep
    vh = v.repeat_interleave(rep, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, kh) * m["scale"] + distance_bias(T, w[p + "rel"], m["bias_max"])
    a = masked_softmax(s, causal_mask(T))
    a = torch.einsum("hg,gij->hij", w[p + "talk"], a)           # mixed after the softmax
    o = torch.einsum("hij,jhd->ihd", a, vh)
    gate = torch.sigmoid(h @ w[p + "g"].T)                      # [T, H]
    o = o * gate[:, :, None]
    return o.reshape(T, H * dv) @ w[p + "o"].T


def chunked_attention(h, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float):
    """mixer "attention_2": biased projections, one RMS norm over the whole query (key) projection, a learned factor
    per head on the scores, softmax over the earlier positions of the query's own chunk"""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_norm(h @ w[p + "q"].T + w[p + "q.b"], w[p + "q.norm"], eps).reshape(T, H, dk)
    k = rms_norm(h @ w[p + "k"].T + w[p + "k.b"], w[p + "k.norm"], eps).reshape(T, G, dk)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).reshape(T, G, dv)
    rep = H // G
    kh = k.repeat_interleave(rep, dim=1)
    vh = v.repeat_interleave(rep, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, kh) * m["scale"] * w[p + "temp"][:, None, None]
    a = masked_softmax(s, same_chunk_mask(T, m["mask"]["size"]))
    o = torch.einsum("hij,jhd->ihd", a, vh)
    return o.reshape(T, H * dv) @ w[p + "o"].T + w[p + "o.b"]


def dense_ff(h, w: Dict[str, torch.Tensor], p: str):
    return relu_squared(h @ w[p + "up"].T + w[p + "up.b"]) @ w[p + "down"].T + w[p + "down.b"]


# ------------------------------------------------------------------------------------------------ the decoder
def layer_runs(cfg: dict) -> List[int]:
    n = len(cfg["layers"])
    lp = cfg.get("loop")
    if not lp:
        return list(range(n))
    a, b, times = lp["start"], lp["stop"], lp["times"]
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def forward(tokens: List[int], w: Dict[str, torch.Tensor], cfg: dict, dtype=torch.float64,
            layers_out: Optional[list] = None):
    """logits [T, vocab]; layers_out (a list) receives the sum of the streams after every layer execution"""
    w = {k: v.to(dtype) if v.is_floating_point() else v for k, v in w.items()}
    eps = cfg["norm"]["eps"]
    x0 = embed_tokens(tokens, w["embed"], w["pos"], cfg["embedding"]["scale"])
    hyper = "streams" in cfg
    S = cfg["streams"] if hyper else 1
    xs = x0[None].repeat(S, 1, 1)
    for i in layer_runs(cfg):
        e = cfg["layers"][i]
        p = f"l{i}."
        mixer = biased_attention if e["type"] == "attention" else chunked_attention
        subs = [(1, lambda u: mixer(rms_norm(u, w[p + "norm1"], eps), w, p + "mix.", e["mixer"], eps))]
        if e.get("mlp") is not None:
            subs.append((2, lambda u: dense_ff(rms_norm(u, w[p + "norm2"], eps), w, p + "mlp.")))
        for q, f in subs:
            if hyper:
                hc = f"{p}hc{q}."
                y = f(streams_read(xs, w[hc + "in"]))
                xs = streams_write(xs, y, w[hc + "mix"], w[hc + "out"])
            else:
                xs = xs + f(xs[0])[None]
        if layers_out is not None:
            layers_out.append(xs.sum(0))
    x = xs.sum(0)
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T
