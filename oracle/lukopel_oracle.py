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
    """table [rows, H] -> bias [H, T, T]: entry (i, j) is the row of distance i - j (entries with j > i are masked later)"""
    rows, H = table.shape
    row_of = torch.tensor([distance_bucket(n, rows, far) for n in range(T)])
    i = torch.arange(T)
    dist = (i[:, None] - i[None, :]).clamp(min=0)
    return table[row_of[dist]].permute(2, 0, 1)


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


# ------------------------------------------------------------------------------------------------ test models
def tensor_shapes(cfg: dict, rel_rows=10) -> Dict[str, tuple]:
    """every tensor of a checkpoint with this configuration; rel_rows: rows of the distance-bias tables (one number, or
    one per layer), which no configuration key gives"""
    D, V = cfg["width"], cfg["vocab"]
    hyper = "streams" in cfg
    S = cfg.get("streams", 1)
    s = {"embed": (V, D), "pos": (cfg["max_positions"], D), "final.norm": (D,), "head": (V, D)}
    for i, e in enumerate(cfg["layers"]):
        p, mx, m = f"l{i}.", f"l{i}.mix.", e["mixer"]
        H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        s[p + "norm1"] = (D,)
        s.update({mx + "q": (H * dk, D), mx + "k": (G * dk, D), mx + "v": (G * dv, D), mx + "o": (D, H * dv)})
        if e["type"] == "attention":
            rows = rel_rows[i] if isinstance(rel_rows, (list, tuple)) else rel_rows
            s.update({mx + "q.norm": (dk,), mx + "k.norm": (dk,), mx + "rel": (rows, H), mx + "talk": (H, H),
                      mx + "g": (H, D)})
        else:
            s.update({mx + "q.b": (H * dk,), mx + "k.b": (G * dk,), mx + "v.b": (G * dv,), mx + "o.b": (D,),
                      mx + "q.norm": (H * dk,), mx + "k.norm": (G * dk,), mx + "temp": (H,)})
        subs = [1]
        if e.get("mlp") is not None:
            F = e["mlp"]["ff"]
            s.update({p + "norm2": (D,), p + "mlp.up": (F, D), p + "mlp.up.b": (F,), p + "mlp.down": (D, F),
                      p + "mlp.down.b": (D,)})
            subs.append(2)
        if hyper:
            for q in subs:
                s.update({f"{p}hc{q}.in": (S,), f"{p}hc{q}.out": (S,), f"{p}hc{q}.mix": (S, S)})
    return s


def random_model(cfg: dict, seed: int, scale: float = 1.0, rel_rows=10) -> Dict[str, torch.Tensor]:
    """weights whose every mechanism matters in the logits: matrices of unit-variance outputs, norm weights around one,
    head and stream mixes far from the identity, biases and distance biases of order one"""
    g = torch.Generator().manual_seed(seed)
    w = {}
    for name, shape in tensor_shapes(cfg, rel_rows).items():
        leaf = name.rsplit(".", 1)[-1]
        rnd = lambda: torch.randn(shape, generator=g)
        if leaf in ("norm1", "norm2", "norm"):
            t = 1.0 + 0.3 * rnd()
        elif leaf == "talk":
            t = torch.eye(shape[0]) + 0.4 * rnd()
        elif leaf == "mix":
            t = 0.8 * torch.eye(shape[0]) + 0.3 * rnd()
        elif leaf in ("in", "out"):
            t = 0.6 + 0.4 * rnd()
        elif leaf == "temp":
            t = 1.0 + 0.5 * rnd()
        elif leaf == "rel":
            t = 1.5 * rnd()
        elif leaf == "b":
            t = 0.5 * rnd()
        elif leaf == "pos":
            t = 0.7 * rnd()
        elif leaf == "embed":
            t = rnd()
        else:
            t = rnd() * (scale / math.sqrt(shape[-1]))
        w[name] = t.to(torch.bfloat16)          # what a checkpoint stores
    return w
