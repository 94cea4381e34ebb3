"""Mavipel family: configuration (read from a checkpoint's ``config.json``), tensor names, random initialisation and
the packing of a named state dict into the buffers ``asd_mavipel_set_tensor`` expects (include/asd_b200.h).

A Mavipel model is a stack of pre-normed layers, x <- x + mixer(norm(x)) and then x <- x + ff(norm(x)), every norm an
RMS norm over equal consecutive groups of the row with a plain weight; the embedding output passes such a norm too.
A layer names ONE of two mixers.  "channel_delta": the gated delta rule, a recurrence with a [key, value] state per
head that every position decays per key channel, corrects along its unit key and writes into; queries, keys and values
first pass a short causal convolution over time.  "parallel": two mixers side by side on the same input whose scaled
results are summed: grouped-query softmax attention over a sliding window, with normed and partly rotated queries
and keys, tanh-capped scores that are mixed across the heads before the softmax and a learned sink in its
denominator; and the generalised delta rule, whose removal has a rate per key channel of its own.  The feed-forward is
a two-matrix gelu layer, or routed gated experts (gates = softmax over the chosen router logits) plus a shared expert,
or absent.  A span of layers may run several times in a row with the same weights; every pass has its own cache and
state and starts by adding a learned vector.  The reference project has no model code of its own (its stages are vLLM
checkpoints, src/serving/real_model_pipeline.py:98-108); this family runs behind the same ``Stage`` seam."""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass, field, replace
from typing import Dict, List, Optional, Tuple

import torch

ARCHITECTURE = "Mavipel"
MIXERS = ("channel_delta", "parallel")
MIXER_CODE = {m: i for i, m in enumerate(MIXERS)}
FF_KINDS = (None, "dense", "moe")
NO_WINDOW = 1 << 30


@dataclass(frozen=True)
class MavipelLayer:
    type: str
    # channel_delta
    heads: int = 0
    kv_heads: int = 0
    dim: int = 0
    vdim: int = 0
    conv: int = 1
    decay_rank: int = 0      # inner sizes of the two-matrix projections: tensor shapes give them, not config keys
    gate_rank: int = 0
    # parallel, left: window attention
    a_heads: int = 0
    a_kv_heads: int = 0
    a_dim: int = 0
    a_vdim: int = 0
    rot_base: float = 10000.0
    rot_dims: int = 0
    window: int = NO_WINDOW
    scale: float = 1.0
    softcap: float = 0.0     # 0: scores are not capped
    left_scale: float = 1.0
    # parallel, right: generalised delta rule
    r_heads: int = 0
    r_dim: int = 0
    r_decay_rank: int = 0
    right_scale: float = 1.0
    # feed-forward
    ff_kind: Optional[str] = None
    ff: int = 0
    experts: int = 0
    top: int = 0
    expert_ff: int = 0
    shared_ff: int = 0

    @property
    def cache_row(self) -> int:
        """cached elements per position (paged); the recurrent states are per sequence, not per position"""
        return self.a_kv_heads * (self.a_dim + self.a_vdim) if self.type == "parallel" else 0

    @property
    def state_elems(self) -> int:
        return self.heads * self.dim * self.vdim if self.type == "channel_delta" else self.r_heads * self.r_dim * self.r_dim

    @property
    def conv_channels(self) -> int:
        return 2 * self.kv_heads * self.dim + self.heads * self.vdim if self.type == "channel_delta" else 0


@dataclass(frozen=True)
class MavipelConfig:
    width: int
    vocab_size: int
    layers: List[MavipelLayer] = field(default_factory=list)
    eps: float = 1e-5
    norm_groups: int = 1
    loop: Optional[Tuple[int, int, int]] = None     # (start, stop, times): layers start .. stop - 1 run `times` times
    name: str = "mavipel"

    architecture = ARCHITECTURE
    build_components = ("mavipel",)

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    @property
    def hidden_size(self) -> int:
        return self.width

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
    def from_dict(cls, d: dict, name: str = "mavipel") -> "MavipelConfig":
        layers = []
        for i, e in enumerate(d["layers"]):
            t = e.get("type")
            if t not in MIXERS:
                raise ValueError(f"layer {i}: unknown mixer type {t!r} (have {MIXERS})")
            m, f = e["mixer"], e.get("mlp")
            kw = dict(type=t)
            if t == "channel_delta":
                kw.update(heads=int(m["heads"]), kv_heads=int(m.get("kv_heads", m["heads"])), dim=int(m["dim"]),
                          vdim=int(m.get("vdim", m["dim"])), conv=int(m.get("conv", 1)),
                          decay_rank=int(m.get("decay_rank", 0)), gate_rank=int(m.get("gate_rank", 0)))
            else:
                a, r = m["left"], m["right"]
                rot, mask = a.get("rot") or {}, a.get("mask") or {}
                kw.update(a_heads=int(a["heads"]), a_kv_heads=int(a.get("kv_heads", a["heads"])), a_dim=int(a["dim"]),
                          a_vdim=int(a.get("vdim", a["dim"])), rot_base=float(rot.get("base", 10000.0)),
                          rot_dims=int(rot.get("dims", 0)),
                          window=NO_WINDOW if mask.get("size") is None else int(mask["size"]),
                          scale=float(a["scale"]), softcap=float(a.get("softcap") or 0.0),
                          left_scale=float(m.get("left_scale", 1.0)), right_scale=float(m.get("right_scale", 1.0)),
                          r_heads=int(r["heads"]), r_dim=int(r["dim"]), r_decay_rank=int(r.get("decay_rank", 0)))
            if f is not None:
                kind = f.get("kind", "dense")
                if kind == "dense":
                    kw.update(ff_kind="dense", ff=int(f["ff"]))
                elif kind == "moe":
                    kw.update(ff_kind="moe", experts=int(f["router"]["experts"]), top=int(f["router"]["top"]),
                              expert_ff=int(f["expert"]["ff"]), shared_ff=int((f.get("shared") or {}).get("ff", 0)))
                else:
                    raise ValueError(f"layer {i}: unknown feed-forward kind {kind!r}")
            layers.append(MavipelLayer(**kw))
        lp = d.get("loop")
        loop = None
        if lp:
            loop = (int(lp["start"]), int(lp["stop"]), int(lp["times"]))
            if not (0 <= loop[0] < loop[1] <= len(layers)) or loop[2] < 1:
                raise ValueError(f"loop {lp!r} does not fit {len(layers)} layers")
        norm = d.get("norm") or {}
        return cls(width=int(d["width"]), vocab_size=int(d["vocab"]), layers=layers, eps=float(norm.get("eps", 1e-5)),
                   norm_groups=int(norm.get("groups", 1)), loop=loop, name=name)

    def to_dict(self) -> dict:
        """the ``config.json`` form (inverse of ``from_dict``)"""
        out = []
        for l in self.layers:
            if l.type == "channel_delta":
                m = {"heads": l.heads, "kv_heads": l.kv_heads, "dim": l.dim, "vdim": l.vdim, "conv": l.conv}
            else:
                left = {"heads": l.a_heads, "kv_heads": l.a_kv_heads, "dim": l.a_dim, "vdim": l.a_vdim,
                        "rot": {"base": l.rot_base, "dims": l.rot_dims}, "scale": l.scale, "softcap": l.softcap}
                if l.window < NO_WINDOW:
                    left["mask"] = {"size": l.window}
                m = {"left": left, "left_scale": l.left_scale, "right": {"heads": l.r_heads, "dim": l.r_dim},
                     "right_scale": l.right_scale}
            if l.ff_kind == "dense":
                f = {"kind": "dense", "ff": l.ff}
            elif l.ff_kind == "moe":
                f = {"kind": "moe", "router": {"experts": l.experts, "top": l.top}, "expert": {"ff": l.expert_ff}}
                if l.shared_ff:
                    f["shared"] = {"ff": l.shared_ff}
            else:
                f = None
            out.append({"type": l.type, "mixer": m, "mlp": f})
        d = {"architecture": ARCHITECTURE, "width": self.width, "vocab": self.vocab_size,
             "norm": {"eps": self.eps, "groups": self.norm_groups}, "layers": out}
        if self.loop is not None:
            d["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        return d

    def with_shapes(self, shapes: Dict[str, tuple]) -> "MavipelConfig":
        """sizes that only a tensor's shape gives (the inner sizes of the two-matrix decay and gate projections)"""
        layers = []
        for i, l in enumerate(self.layers):
            p = f"l{i}.mix."
            if l.type == "channel_delta":
                if p + "a1" in shapes:
                    l = replace(l, decay_rank=int(shapes[p + "a1"][0]))
                if p + "g1" in shapes:
                    l = replace(l, gate_rank=int(shapes[p + "g1"][0]))
            elif p + "right.w1" in shapes:
                l = replace(l, r_decay_rank=int(shapes[p + "right.w1"][0]))
            layers.append(l)
        return replace(self, layers=layers)

    @property
    def params(self) -> int:
        return sum(math.prod(s) for s in tensor_shapes(self).values())

    def streamed_bytes(self, elem: int = 2) -> int:
        """weight bytes one decode step of ONE token reads: every matrix once per execution of its layer (of the
        experts only the chosen ones), the head"""
        shapes = tensor_shapes(self)
        n = self.vocab_size * self.width
        for i, _ in self.runs():
            l = self.layers[i]
            for k, s in shapes.items():
                if not k.startswith(f"l{i}.") or len(s) != 2:
                    continue
                if ".mlp.e" in k:
                    n += math.prod(s) * l.top / l.experts
                else:
                    n += math.prod(s)
        return int(n * elem)

    def kv_bytes_per_token(self, elem: int = 2) -> int:
        return sum(self.layers[i].cache_row for i, _ in self.runs()) * elem


def tensor_shapes(cfg: MavipelConfig) -> Dict[str, tuple]:
    """every tensor of a checkpoint, by name"""
    D, V = cfg.width, cfg.vocab_size
    s = {"embed": (V, D), "embed.norm": (D,), "final.norm": (D,), "head": (V, D)}
    if cfg.loop is not None:
        s["loop.step"] = (cfg.loop[2], D)
    for i, l in enumerate(cfg.layers):
        p = f"l{i}."
        s[p + "norm1"] = (D,)
        if l.type == "channel_delta":
            m, nk, nv = p + "mix.", l.kv_heads * l.dim, l.heads * l.vdim
            s.update({m + "q": (nk, D), m + "q.conv": (nk, l.conv), m + "k": (nk, D), m + "k.conv": (nk, l.conv),
                      m + "v": (nv, D), m + "v.conv": (nv, l.conv), m + "b": (l.heads, D), m + "A_log": (l.heads,),
                      m + "norm": (l.vdim,), m + "a1": (l.decay_rank, D), m + "a2": (l.heads * l.dim, l.decay_rank),
                      m + "dt_bias": (l.heads * l.dim,), m + "g1": (l.gate_rank, D), m + "g2": (nv, l.gate_rank),
                      m + "o": (D, nv)})
        else:
            a, r = p + "mix.left.", p + "mix.right."
            nq, nk, nv, nr = l.a_heads * l.a_dim, l.a_kv_heads * l.a_dim, l.a_kv_heads * l.a_vdim, l.r_heads * l.r_dim
            s.update({a + "q": (nq, D), a + "q.b": (nq,), a + "k": (nk, D), a + "k.b": (nk,), a + "v": (nv, D),
                      a + "v.b": (nv,), a + "q.norm": (l.a_dim,), a + "k.norm": (l.a_dim,),
                      a + "talk": (l.a_heads, l.a_heads), a + "sink": (l.a_heads,), a + "o": (D, l.a_heads * l.a_vdim)})
            s.update({r + "r": (nr, D), r + "k": (nr, D), r + "v": (nr, D), r + "g": (nr, D), r + "a": (nr, D),
                      r + "a.b": (nr,), r + "w1": (l.r_decay_rank, D), r + "w2": (nr, l.r_decay_rank), r + "w0": (nr,),
                      r + "norm": (nr,), r + "o": (D, nr)})
        f = p + "mlp."
        if l.ff_kind is not None:
            s[p + "norm2"] = (D,)
        if l.ff_kind == "dense":
            s.update({f + "up": (l.ff, D), f + "down": (D, l.ff)})
        elif l.ff_kind == "moe":
            s.update({f + "router": (l.experts, D), f + "router.b": (l.experts,)})
            for e in range(l.experts):
                s.update({f + f"e{e}.gate": (l.expert_ff, D), f + f"e{e}.up": (l.expert_ff, D),
                          f + f"e{e}.down": (D, l.expert_ff)})
            if l.shared_ff:
                s.update({f + "shared.gate": (l.shared_ff, D), f + "shared.up": (l.shared_ff, D),
                          f + "shared.down": (D, l.shared_ff)})
    return s


def tiny_config(**kw) -> MavipelConfig:
    """one small layer of every kind, unequal sizes, a repeated span (tests, smoke runs)"""
    layers = [
        MavipelLayer(type="channel_delta", heads=4, kv_heads=2, dim=24, vdim=16, conv=3, decay_rank=8, gate_rank=12,
                     ff_kind="moe", experts=5, top=2, expert_ff=40, shared_ff=24),
        MavipelLayer(type="parallel", a_heads=6, a_kv_heads=2, a_dim=16, a_vdim=24, rot_base=1000.0, rot_dims=8, window=9,
                     scale=0.3, softcap=12.0, left_scale=0.9, r_heads=3, r_dim=16, r_decay_rank=8, right_scale=1.2,
                     ff_kind="dense", ff=72),
        MavipelLayer(type="channel_delta", heads=2, kv_heads=2, dim=16, vdim=40, conv=4, decay_rank=4, gate_rank=8),
    ]
    base = dict(width=96, vocab_size=120, layers=layers, eps=1e-5, norm_groups=3, loop=(0, 2, 2), name="tiny")
    base.update(kw)
    return MavipelConfig(**base)


def sized_config(width: int, n_layers: int, heads: int, vocab: int = 32768, dim: int = 128, window: int = 1024,
                 ff: Optional[int] = None, experts: int = 0, top: int = 2, loop: Optional[Tuple[int, int, int]] = None,
                 name: str = "mavipel-sized") -> MavipelConfig:
    """layers of a realistic size for throughput measurements (random weights): two gated-delta layers, then a
    parallel one, in turn; dense feed-forwards of width ff (4 x width by default), or `experts` experts of ff / top"""
    ff = ff if ff is not None else 4 * width
    if experts:
        f = dict(ff_kind="moe", experts=experts, top=top, expert_ff=max(64, ff // (top + 1)), shared_ff=max(64, ff // (top + 1)))
    else:
        f = dict(ff_kind="dense", ff=ff)
    cd = MavipelLayer(type="channel_delta", heads=heads, kv_heads=max(1, heads // 2), dim=dim, vdim=dim, conv=4,
                      decay_rank=32, gate_rank=32, **f)
    par = MavipelLayer(type="parallel", a_heads=heads, a_kv_heads=max(1, heads // 4), a_dim=dim, a_vdim=dim, rot_dims=dim // 2,
                       window=window, scale=1.0 / math.sqrt(dim), softcap=30.0, r_heads=max(1, heads // 2), r_dim=dim,
                       r_decay_rank=32, **f)
    return MavipelConfig(width=width, vocab_size=vocab, layers=[(cd, cd, par)[i % 3] for i in range(n_layers)],
                         norm_groups=2, loop=loop, name=name)


def random_weights(cfg: MavipelConfig, seed: int, device="cpu", dtype=torch.bfloat16) -> Dict[str, torch.Tensor]:
    """Named state dict with variance-preserving random matrices, norm weights near one, decay parameters that keep a
    state alive for tens of tokens (throughput runs and smoke tests; nothing trained)."""
    g = torch.Generator(device=device).manual_seed(seed)
    w = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.rsplit(".", 1)[-1]
        rnd = lambda: torch.randn(shape, generator=g, device=device)
        if leaf in ("norm1", "norm2") or name in ("final.norm", "embed.norm") or name.endswith("mix.norm") \
                or name.endswith("right.norm") or name.endswith("q.norm") or name.endswith("k.norm"):
            t = 1.0 + 0.1 * rnd()
        elif leaf == "conv":
            t = 0.5 * rnd()
        elif leaf == "talk":
            t = torch.eye(shape[0], device=device) + 0.2 * rnd()
        elif leaf in ("sink", "A_log"):
            t = 0.5 * rnd()
        elif leaf in ("dt_bias", "w0"):
            t = -2.0 + rnd()
        elif leaf == "b" and len(shape) == 1:
            t = 0.3 * rnd()
        elif leaf == "step":
            t = 0.3 * rnd()
        elif leaf == "embed":
            t = rnd()
        else:
            t = rnd() / math.sqrt(shape[-1])
        w[name] = t.to(dtype)
    return w


def pack(w: Dict[str, torch.Tensor], cfg: MavipelConfig, device, dtype) -> Dict[Tuple[int, str], torch.Tensor]:
    """checkpoint names -> engine buffers keyed (layer or -1, engine tensor name).  Matrices that read the same input
    are stacked into one; the output projections of a parallel layer stand side by side; an expert's gate and up
    matrices are stacked and the experts laid out back to back.  Matrices take the engine's element type, everything
    that enters 32-bit arithmetic directly (norm weights, biases, convolution taps, second matrices of the decay and
    gate projections, head mix, sinks, router) stays fp32."""
    want = tensor_shapes(cfg)
    for k, shape in want.items():
        if k not in w:
            raise KeyError(f"checkpoint lacks tensor {k}")
        if tuple(w[k].shape) != tuple(shape):
            raise ValueError(f"tensor {k} has shape {tuple(w[k].shape)}, the configuration says {tuple(shape)}")
    mat = lambda t: t.to(device=device, dtype=dtype).contiguous()
    vec = lambda t: t.to(device=device, dtype=torch.float32).contiguous()
    cat = lambda names, dim=0: torch.cat([w[n] for n in names], dim)
    out = {(-1, "embed"): mat(w["embed"]), (-1, "embed_norm"): vec(w["embed.norm"]),
           (-1, "final_norm"): vec(w["final.norm"]), (-1, "head"): mat(w["head"])}
    if cfg.loop is not None:
        out[(-1, "loop_step")] = vec(w["loop.step"])
    for i, l in enumerate(cfg.layers):
        p = f"l{i}."
        out[(i, "norm1")] = vec(w[p + "norm1"])
        if l.type == "channel_delta":
            m = p + "mix."
            out[(i, "w_in")] = mat(cat([m + x for x in ("q", "k", "v", "b", "a1", "g1")]))
            out[(i, "conv_w")] = vec(cat([m + x for x in ("q.conv", "k.conv", "v.conv")]))
            out[(i, "a_log")] = vec(w[m + "A_log"])
            out[(i, "w_decay")], out[(i, "b_decay")] = vec(w[m + "a2"]), vec(w[m + "dt_bias"])
            out[(i, "w_gate")] = vec(w[m + "g2"])
            out[(i, "out_norm")] = vec(w[m + "norm"])
            out[(i, "w_o")] = mat(w[m + "o"])
        else:
            a, r = p + "mix.left.", p + "mix.right."
            out[(i, "w_in")] = mat(cat([a + "q", a + "k", a + "v", r + "r", r + "k", r + "v", r + "g", r + "a", r + "w1"]))
            out[(i, "in_bias")] = vec(cat([a + "q.b", a + "k.b", a + "v.b"]))
            out[(i, "q_norm")], out[(i, "k_norm")] = vec(w[a + "q.norm"]), vec(w[a + "k.norm"])
            out[(i, "talk")], out[(i, "sink")] = vec(w[a + "talk"]), vec(w[a + "sink"])
            out[(i, "w_decay")], out[(i, "b_decay")] = vec(w[r + "w2"]), vec(w[r + "w0"])
            out[(i, "rate_bias")] = vec(w[r + "a.b"])
            out[(i, "out_norm")] = vec(w[r + "norm"])
            out[(i, "w_o")] = mat(cat([a + "o", r + "o"], 1))
        f = p + "mlp."
        if l.ff_kind is not None:
            out[(i, "norm2")] = vec(w[p + "norm2"])
        if l.ff_kind == "dense":
            out[(i, "w_up")], out[(i, "w_down")] = mat(w[f + "up"]), mat(w[f + "down"])
        elif l.ff_kind == "moe":
            out[(i, "router")], out[(i, "router_b")] = vec(w[f + "router"]), vec(w[f + "router.b"])
            out[(i, "w_gu")] = mat(torch.stack([cat([f + f"e{e}.gate", f + f"e{e}.up"]) for e in range(l.experts)]))
            out[(i, "w_edown")] = mat(torch.stack([w[f + f"e{e}.down"] for e in range(l.experts)]))
            if l.shared_ff:
                out[(i, "w_sgu")] = mat(cat([f + "shared.gate", f + "shared.up"]))
                out[(i, "w_sdown")] = mat(w[f + "shared.down"])
    return out


def load_config_dir(path: str) -> MavipelConfig:
    with open(os.path.join(path, "config.json")) as f:
        return MavipelConfig.from_dict(json.load(f), name=os.path.basename(os.path.normpath(path)) or "mavipel")
