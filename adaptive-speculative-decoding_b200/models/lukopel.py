"""Lukopel family: configuration (read from a checkpoint's ``config.json``), tensor names, random initialisation and
the packing of a named state dict into the buffers ``asd_lukopel_set_tensor`` expects (include/asd_b200.h).

A Lukopel model embeds a token as embed[token] * scale + pos[position] and carries ``streams`` residual streams per
token (hyper-connections): a sublayer reads a learned weighted sum of the streams, norms it (RMS norm, plain weight),
and its result returns to every stream through a learned stream-to-stream matrix and a learned write vector; without
``streams`` the ordinary residual sum is used.  A layer names ONE of two attention mixers and an optional feed-forward.
"attention": grouped-query softmax attention with an RMS norm per query / key head (one weight for all heads), queries
scaled by a slowly growing function of the position, unit-RMS values, a learned bias per (distance bucket, head) added
to the scaled scores, a plain causal mask, softmax weights mixed across the heads after the softmax, and a sigmoid gate
per head.  "attention_2": biased projections, one RMS norm over the whole query (key) projection, a learned factor per
head on the scores, and a causal mask cut into chunks counted from position 0.  The feed-forward is a biased two-matrix
layer with a squared relu.  A span of layers may run several times in a row with the same weights; every pass has its own
cache.  The reference project has no model code of its own (its stages are vLLM checkpoints,
src/serving/real_model_pipeline.py:98-108); this family runs behind the same ``Stage`` seam."""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass, field, replace
from typing import Dict, List, Optional, Tuple

import torch

ARCHITECTURE = "Lukopel"
MIXERS = ("attention", "attention_2")


@dataclass(frozen=True)
class LukopelLayer:
    type: str
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    # "attention"
    bias_max: int = 0          # distance from which the last row of the bias table applies
    bias_rows: int = 0         # rows of the bias table: a tensor's shape gives it, not a config key
    temp_coef: float = 0.0
    temp_every: int = 0
    # "attention_2"
    chunk: int = 0
    # feed-forward
    ff_kind: Optional[str] = None
    ff: int = 0

    @property
    def cache_row(self) -> int:
        """cached elements per position (paged)"""
        return self.kv_heads * (self.dim + self.vdim)

    @property
    def far(self) -> int:
        """distance from which the bias no longer changes"""
        return max(self.bias_max, self.bias_rows // 2)


def distance_rows(rows: int, far_at: int, upto: int) -> List[int]:
    """row of a distance-bias table with `rows` rows for every distance 0 .. upto: distances below rows / 2 have a row
    each; from there on the rows are spaced evenly in the logarithm of the distance and the last one is reached at
    distance `far_at`"""
    half = rows // 2
    out = []
    for n in range(upto + 1):
        if n < half:
            out.append(n)
            continue
        step = math.log(n / half) / math.log(far_at / half) * (rows - half)
        out.append(min(rows - 1, half + int(math.floor(step))))
    return out


@dataclass(frozen=True)
class LukopelConfig:
    width: int
    vocab_size: int
    layers: List[LukopelLayer] = field(default_factory=list)
    eps: float = 1e-5
    embed_scale: float = 1.0
    streams: Optional[int] = None                   # None: one stream with the ordinary residual sum
    max_positions: int = 0                          # rows of the learned position table
    loop: Optional[Tuple[int, int, int]] = None     # (start, stop, times): layers start .. stop - 1 run `times` times
    name: str = "lukopel"

    architecture = ARCHITECTURE
    build_components = ("lukopel",)

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    @property
    def hidden_size(self) -> int:
        return self.width

    @property
    def n_streams(self) -> int:
        return self.streams if self.streams is not None else 1

    def runs(self) -> List[Tuple[int, int]]:
        """(layer, pass) of every layer execution in order; pass is -1 outside the repeated span"""
        n = len(self.layers)
        if self.loop is None:
            return [(i, -1) for i in range(n)]
        a, b, times = self.loop
        out = [(i, -1) for i in range(a)]
        for t in range(times):
            out += [(i, t) for i in range(a, b)]
        return out + [(i, -1) for i in range(b, n)]

    @classmethod
    def from_dict(cls, d: dict, name: str = "lukopel") -> "LukopelConfig":
        layers = []
        for i, e in enumerate(d["layers"]):
            t = e.get("type")
            if t not in MIXERS:
                raise ValueError(f"layer {i}: unknown mixer type {t!r} (have {MIXERS})")
            m, f = e["mixer"], e.get("mlp")
            kw = dict(type=t, heads=int(m["heads"]), kv_heads=int(m.get("kv_heads", m["heads"])), dim=int(m["dim"]),
                      vdim=int(m.get("vdim", m["dim"])), scale=float(m["scale"]))
            if t == "attention":
                qt = m.get("q_temp") or {}
                kw.update(bias_max=int(m["bias_max"]), temp_coef=float(qt.get("coef", 0.0)),
                          temp_every=int(qt.get("every", 0)))
            else:
                kw.update(chunk=int((m.get("mask") or {}).get("size") or 0))
            if f is not None:
                kind = f.get("kind", "dense")
                if kind != "dense":
                    raise ValueError(f"layer {i}: unknown feed-forward kind {kind!r}")
                kw.update(ff_kind="dense", ff=int(f["ff"]))
            layers.append(LukopelLayer(**kw))
        lp = d.get("loop")
        loop = None
        if lp:
            loop = (int(lp["start"]), int(lp["stop"]), int(lp["times"]))
            if not (0 <= loop[0] < loop[1] <= len(layers)) or loop[2] < 1:
                raise ValueError(f"loop {lp!r} does not fit {len(layers)} layers")
        return cls(width=int(d["width"]), vocab_size=int(d["vocab"]), layers=layers,
                   eps=float((d.get("norm") or {}).get("eps", 1e-5)),
                   embed_scale=float((d.get("embedding") or {}).get("scale", 1.0)),
                   streams=int(d["streams"]) if d.get("streams") is not None else None,
                   max_positions=int(d.get("max_positions", 0)), loop=loop, name=name)

    def to_dict(self) -> dict:
        """the ``config.json`` form (inverse of ``from_dict``)"""
        out = []
        for l in self.layers:
            m = {"heads": l.heads, "kv_heads": l.kv_heads, "dim": l.dim, "vdim": l.vdim, "scale": l.scale}
            if l.type == "attention":
                m.update(bias_max=l.bias_max, q_temp={"coef": l.temp_coef, "every": l.temp_every})
            else:
                m.update(mask={"size": l.chunk})
            out.append({"type": l.type, "mixer": m, "mlp": {"kind": "dense", "ff": l.ff} if l.ff_kind else None})
        d = {"architecture": ARCHITECTURE, "width": self.width, "vocab": self.vocab_size, "norm": {"eps": self.eps},
             "embedding": {"scale": self.embed_scale}, "max_positions": self.max_positions, "layers": out}
        if self.streams is not None:
            d["streams"] = self.streams
        if self.loop is not None:
            d["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        return d

    def with_shapes(self, shapes: Dict[str, tuple]) -> "LukopelConfig":
        """sizes that only a tensor's shape gives (rows of the distance-bias tables, of the position table)"""
        layers = []
        for i, l in enumerate(self.layers):
            k = f"l{i}.mix.rel"
            if l.type == "attention" and k in shapes:
                l = replace(l, bias_rows=int(shapes[k][0]))
            layers.append(l)
        mp = int(shapes["pos"][0]) if "pos" in shapes else self.max_positions
        return replace(self, layers=layers, max_positions=mp)

    @property
    def params(self) -> int:
        return sum(math.prod(s) for s in tensor_shapes(self).values())

    def streamed_bytes(self, elem: int = 2) -> int:
        """weight bytes one decode step of ONE token reads: every matrix once per execution of its layer, the head"""
        shapes = tensor_shapes(self)
        n = self.vocab_size * self.width
        for i, _ in self.runs():
            n += sum(math.prod(s) for k, s in shapes.items() if k.startswith(f"l{i}.") and len(s) == 2 and ".hc" not in k
                     and not k.endswith((".rel", ".talk")))
        return int(n * elem)

    def kv_bytes_per_token(self, elem: int = 2) -> int:
        return sum(self.layers[i].cache_row for i, _ in self.runs()) * elem


def tensor_shapes(cfg: LukopelConfig) -> Dict[str, tuple]:
    """every tensor of a checkpoint, by name"""
    D, V, S = cfg.width, cfg.vocab_size, cfg.n_streams
    s = {"embed": (V, D), "pos": (cfg.max_positions, D), "final.norm": (D,), "head": (V, D)}
    for i, l in enumerate(cfg.layers):
        p, m = f"l{i}.", f"l{i}.mix."
        nq, nk, nv = l.heads * l.dim, l.kv_heads * l.dim, l.kv_heads * l.vdim
        s[p + "norm1"] = (D,)
        s.update({m + "q": (nq, D), m + "k": (nk, D), m + "v": (nv, D), m + "o": (D, l.heads * l.vdim)})
        if l.type == "attention":
            s.update({m + "q.norm": (l.dim,), m + "k.norm": (l.dim,), m + "rel": (l.bias_rows, l.heads),
                      m + "talk": (l.heads, l.heads), m + "g": (l.heads, D)})
        else:
            s.update({m + "q.b": (nq,), m + "k.b": (nk,), m + "v.b": (nv,), m + "o.b": (D,), m + "q.norm": (nq,),
                      m + "k.norm": (nk,), m + "temp": (l.heads,)})
        subs = [1]
        if l.ff_kind is not None:
            f = p + "mlp."
            s.update({p + "norm2": (D,), f + "up": (l.ff, D), f + "up.b": (l.ff,), f + "down": (D, l.ff),
                      f + "down.b": (D,)})
            subs.append(2)
        if cfg.streams is not None:
            for q in subs:
                s.update({f"{p}hc{q}.in": (S,), f"{p}hc{q}.out": (S,), f"{p}hc{q}.mix": (S, S)})
    return s


def tiny_config(**kw) -> LukopelConfig:
    """a small layer of either kind, unequal sizes, a repeated span, one layer without a feed-forward (tests, smoke runs)"""
    layers = [
        LukopelLayer(type="attention", heads=6, kv_heads=3, dim=20, vdim=12, scale=0.2, bias_max=40, bias_rows=10,
                     temp_coef=0.25, temp_every=7, ff_kind="dense", ff=72),
        LukopelLayer(type="attention_2", heads=4, kv_heads=2, dim=16, vdim=24, scale=0.3, chunk=11, ff_kind="dense", ff=56),
        LukopelLayer(type="attention", heads=2, kv_heads=2, dim=24, vdim=40, scale=0.25, bias_max=18, bias_rows=6,
                     temp_coef=0.5, temp_every=4),
    ]
    base = dict(width=96, vocab_size=120, layers=layers, eps=1e-5, embed_scale=3.0, streams=3, max_positions=160,
                loop=(0, 2, 2), name="tiny")
    base.update(kw)
    return LukopelConfig(**base)


def sized_config(width: int, n_layers: int, heads: int, vocab: int = 32768, dim: int = 128, chunk: int = 1024,
                 ff: Optional[int] = None, streams: Optional[int] = 4, max_positions: int = 8192,
                 loop: Optional[Tuple[int, int, int]] = None, name: str = "lukopel-sized") -> LukopelConfig:
    """layers of a realistic size for throughput measurements (random weights): two chunked layers, then one with the
    distance bias and mixed weights, in turn; dense feed-forwards of width ff (4 x width by default)"""
    ff = ff if ff is not None else 4 * width
    kvh = max(1, heads // 4)
    full = LukopelLayer(type="attention", heads=heads, kv_heads=kvh, dim=dim, vdim=dim, scale=1.0 / math.sqrt(dim),
                        bias_max=2048, bias_rows=32, temp_coef=0.1, temp_every=256, ff_kind="dense", ff=ff)
    chk = LukopelLayer(type="attention_2", heads=heads, kv_heads=kvh, dim=dim, vdim=dim, scale=1.0 / math.sqrt(dim),
                       chunk=chunk, ff_kind="dense", ff=ff)
    return LukopelConfig(width=width, vocab_size=vocab, layers=[(chk, chk, full)[i % 3] for i in range(n_layers)],
                         streams=streams, max_positions=max_positions, loop=loop, name=name)


def random_weights(cfg: LukopelConfig, seed: int, device="cpu", dtype=torch.bfloat16) -> Dict[str, torch.Tensor]:
    """Named state dict with variance-preserving random matrices, norm weights near one, stream matrices near the
    identity (throughput runs and smoke tests; nothing trained)."""
    g = torch.Generator(device=device).manual_seed(seed)
    w = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.rsplit(".", 1)[-1]
        rnd = lambda: torch.randn(shape, generator=g, device=device)
        if leaf in ("norm1", "norm2", "norm"):
            t = 1.0 + 0.1 * rnd()
        elif leaf == "talk" or (leaf == "mix" and ".hc" in name):
            t = torch.eye(shape[0], device=device) + 0.2 * rnd()
        elif leaf == "temp":
            t = 1.0 + 0.2 * rnd()
        elif leaf in ("in", "out"):
            t = 0.7 + 0.3 * rnd()
        elif leaf == "rel":
            t = 0.5 * rnd()
        elif leaf == "b":
            t = 0.3 * rnd()
        elif leaf == "pos":
            t = 0.5 * rnd()
        elif leaf == "embed":
            t = rnd()
        else:
            t = rnd() / math.sqrt(shape[-1])
        w[name] = t.to(dtype)
    return w


def pack(w: Dict[str, torch.Tensor], cfg: LukopelConfig, device, dtype) -> Dict[Tuple[int, str], torch.Tensor]:
    """checkpoint names -> engine buffers keyed (layer or -1, engine tensor name).  The matrices that read the mixer
    input are stacked into one; a distance-bias table becomes one row per distance up to where it stops changing.
    Matrices and the position table take the engine's element type; everything that enters 32-bit arithmetic directly
    (norm weights, biases, per-head factors, the head mix, the distance bias, the streams' weights) stays fp32."""
    want = tensor_shapes(cfg)
    for k, shape in want.items():
        if k not in w:
            raise KeyError(f"checkpoint lacks tensor {k}")
        if tuple(w[k].shape) != tuple(shape):
            raise ValueError(f"tensor {k} has shape {tuple(w[k].shape)}, the configuration says {tuple(shape)}")
    mat = lambda t: t.to(device=device, dtype=dtype).contiguous()
    vec = lambda t: t.to(device=device, dtype=torch.float32).contiguous()
    cat = lambda names: torch.cat([w[n] for n in names], 0)
    out = {(-1, "embed"): mat(w["embed"]), (-1, "pos"): mat(w["pos"]), (-1, "final_norm"): vec(w["final.norm"]),
           (-1, "head"): mat(w["head"])}
    for i, l in enumerate(cfg.layers):
        p, m = f"l{i}.", f"l{i}.mix."
        out[(i, "norm1")] = vec(w[p + "norm1"])
        out[(i, "q_norm")], out[(i, "k_norm")] = vec(w[m + "q.norm"]), vec(w[m + "k.norm"])
        out[(i, "w_o")] = mat(w[m + "o"])
        if l.type == "attention":
            out[(i, "w_in")] = mat(cat([m + "q", m + "k", m + "v", m + "g"]))
            if l.bias_rows < 2 or l.bias_max <= l.bias_rows // 2:
                raise ValueError(f"layer {i}: a distance-bias table of {l.bias_rows} rows cannot reach its last row at "
                                 f"distance {l.bias_max}")
            rows = torch.tensor(distance_rows(l.bias_rows, l.bias_max, l.far), dtype=torch.long)
            out[(i, "dist_bias")] = vec(w[m + "rel"].to(torch.float32)[rows])
            out[(i, "talk")] = vec(w[m + "talk"])
        else:
            out[(i, "w_in")] = mat(cat([m + "q", m + "k", m + "v"]))
            out[(i, "in_bias")] = vec(cat([m + "q.b", m + "k.b", m + "v.b"]))
            out[(i, "head_factor")] = vec(w[m + "temp"])
            out[(i, "o_bias")] = vec(w[m + "o.b"])
        subs = [1]
        if l.ff_kind is not None:
            f = p + "mlp."
            out[(i, "norm2")] = vec(w[p + "norm2"])
            out[(i, "w_up")], out[(i, "up_bias")] = mat(w[f + "up"]), vec(w[f + "up.b"])
            out[(i, "w_down")], out[(i, "down_bias")] = mat(w[f + "down"]), vec(w[f + "down.b"])
            subs.append(2)
        if cfg.streams is not None:
            for q in subs:
                out[(i, f"hc{q}_read")] = vec(w[f"{p}hc{q}.in"])
                out[(i, f"hc{q}_write")] = vec(w[f"{p}hc{q}.out"])
                out[(i, f"hc{q}_mix")] = vec(w[f"{p}hc{q}.mix"])
    return out


def load_config_dir(path: str) -> LukopelConfig:
    with open(os.path.join(path, "config.json")) as f:
        return LukopelConfig.from_dict(json.load(f), name=os.path.basename(os.path.normpath(path)) or "lukopel")
