"""CPU: the Mavipel family's configuration, registry entry, tensor packing and execution order, and the plain
restatement's own mechanisms on inputs made by hand (so that the oracle the GPU tests lean on is itself pinned)."""
import json
import math

import pytest
import torch

from oracle import mavipel_oracle as O

F64 = torch.float64


def with_ranks(cfg):
    """the dictionary form plus the inner sizes that a checkpoint's tensor shapes give"""
    d = cfg.to_dict()
    for e, l in zip(d["layers"], cfg.layers):
        if l.type == "channel_delta":
            e["mixer"].update(decay_rank=l.decay_rank, gate_rank=l.gate_rank)
        else:
            e["mixer"]["right"]["decay_rank"] = l.r_decay_rank
    return d


def test_config_round_trip_and_registry(tmp_path):
    from asd_b200.models import registry
    from asd_b200.models.mavipel import MavipelConfig, tensor_shapes, tiny_config
    cfg = tiny_config()
    d = cfg.to_dict()
    assert d["architecture"] == "Mavipel"
    back = MavipelConfig.from_dict(d, name="tiny").with_shapes(tensor_shapes(cfg))
    assert back == cfg
    fam = registry.family_of_dict(d)
    assert fam.name == "mavipel" and "mavipel" in fam.components and set(fam.dtypes) == {"bfloat16", "float32"}
    assert registry.family_of_config(cfg).name == "mavipel"
    assert O.tensor_shapes(with_ranks(cfg)) == tensor_shapes(cfg)
    # a checkpoint directory: the sizes that only a tensor's shape gives come from the safetensors header
    (tmp_path / "config.json").write_text(json.dumps(d))
    import struct
    shapes = tensor_shapes(cfg)
    header, off = {}, 0
    for k, s in shapes.items():
        n = 2 * math.prod(s)
        header[k] = {"dtype": "BF16", "shape": list(s), "data_offsets": [off, off + n]}
        off += n
    hj = json.dumps(header).encode()
    (tmp_path / "model.safetensors").write_bytes(struct.pack("<Q", len(hj)) + hj + b"\0" * off)
    fam2, cfg2 = registry.read_config(str(tmp_path))
    assert fam2.name == "mavipel" and cfg2.layers == cfg.layers


def test_defaults_of_absent_keys_and_refusals():
    from asd_b200.models.mavipel import NO_WINDOW, MavipelConfig, tiny_config
    d = tiny_config().to_dict()
    left = d["layers"][1]["mixer"]["left"]
    del left["mask"], left["softcap"], left["kv_heads"], left["vdim"], left["rot"]
    del d["layers"][0]["mixer"]["kv_heads"], d["loop"], d["norm"]["groups"]
    d["layers"][2]["mlp"] = None
    cfg = MavipelConfig.from_dict(d)
    l = cfg.layers[1]
    assert l.window == NO_WINDOW and l.softcap == 0.0 and l.a_kv_heads == l.a_heads and l.a_vdim == l.a_dim and l.rot_dims == 0
    assert cfg.layers[0].kv_heads == cfg.layers[0].heads and cfg.loop is None and cfg.norm_groups == 1
    assert cfg.layers[2].ff_kind is None
    for change in (lambda b: b["layers"][0].update(type="convolution"), lambda b: b["layers"][1]["mlp"].update(kind="sparse"),
                   lambda b: b.update(loop={"start": 2, "stop": 5, "times": 2})):
        bad = json.loads(json.dumps(tiny_config().to_dict()))
        change(bad)
        with pytest.raises(ValueError):
            MavipelConfig.from_dict(bad)


def test_execution_order_of_a_repeated_span():
    from asd_b200.models.mavipel import tiny_config
    cfg = tiny_config(loop=(1, 3, 3))
    assert cfg.runs() == [(0, -1), (1, 0), (2, 0), (1, 1), (2, 1), (1, 2), (2, 2)]
    assert tiny_config(loop=None).runs() == [(0, -1), (1, -1), (2, -1)]
    assert [(i, t) for i, t, _ in O.layer_runs(cfg.to_dict())] == cfg.runs()
    assert [first for _, _, first in O.layer_runs(cfg.to_dict())] == [False, True, False, True, False, True, False]
    one = tiny_config(loop=None)
    assert cfg.kv_bytes_per_token() == one.kv_bytes_per_token() + 2 * cfg.layers[1].cache_row * 2


def test_packing_stacks_projections_and_experts():
    from asd_b200.models.mavipel import pack, random_weights, tensor_shapes, tiny_config
    cfg = tiny_config()
    w = random_weights(cfg, seed=1)
    p = pack(w, cfg, "cpu", torch.float32)
    d, a, _ = cfg.layers
    nk = d.kv_heads * d.dim
    assert p[(0, "w_in")].shape == (2 * nk + d.heads * d.vdim + d.heads + d.decay_rank + d.gate_rank, cfg.width)
    assert torch.equal(p[(0, "w_in")][nk:2 * nk], w["l0.mix.k"].float())
    assert torch.equal(p[(0, "conv_w")][2 * nk:], w["l0.mix.v.conv"].float())
    nr, nl = a.r_heads * a.r_dim, a.a_heads * a.a_dim + a.a_kv_heads * (a.a_dim + a.a_vdim)
    assert p[(1, "w_in")].shape == (nl + 5 * nr + a.r_decay_rank, cfg.width)
    assert torch.equal(p[(1, "w_in")][nl + 4 * nr:nl + 5 * nr], w["l1.mix.right.a"].float())
    assert p[(1, "in_bias")].shape == (nl,)
    assert p[(1, "w_o")].shape == (cfg.width, a.a_heads * a.a_vdim + nr)
    assert torch.equal(p[(1, "w_o")][:, a.a_heads * a.a_vdim:], w["l1.mix.right.o"].float())
    assert p[(0, "w_gu")].shape == (d.experts, 2 * d.expert_ff, cfg.width)
    assert torch.equal(p[(0, "w_gu")][3, d.expert_ff:], w["l0.mlp.e3.up"].float())
    assert p[(0, "w_edown")].shape == (d.experts, cfg.width, d.expert_ff) and p[(0, "w_sgu")].shape == (2 * d.shared_ff, cfg.width)
    assert p[(0, "w_decay")].dtype == torch.float32 and p[(-1, "loop_step")].shape == (2, cfg.width)
    assert (1, "w_up") in p and (2, "norm2") not in p and (2, "w_up") not in p            # layer 2 has no feed-forward
    bad = dict(w)
    bad["l1.mix.left.sink"] = torch.zeros(a.a_heads + 1)
    with pytest.raises(ValueError):
        pack(bad, cfg, "cpu", torch.float32)
    del bad["l1.mix.left.sink"]
    with pytest.raises(KeyError):
        pack(bad, cfg, "cpu", torch.float32)
    assert set(tensor_shapes(cfg)) == set(w)


# ------------------------------------------------------------------------------------------------ the oracle itself
def test_oracle_group_norm_by_hand():
    x = torch.tensor([[3.0, 4.0, 1.0, 1.0]], dtype=F64)
    w = torch.tensor([1.0, 2.0, 3.0, 4.0], dtype=F64)
    got = O.group_norm(x, w, 2, 0.0)
    assert torch.allclose(got, torch.tensor([[3 / math.sqrt(12.5), 8 / math.sqrt(12.5), 3.0, 4.0]], dtype=F64))
    assert torch.allclose(O.group_norm(x, w, 1, 0.0), x / math.sqrt(27 / 4) * w)
    assert math.isclose(O.unit_vector(torch.tensor([3.0, 4.0], dtype=F64), 0.0)[1], 0.8)
    assert math.isclose(O.gelu_tanh(torch.tensor(1.0, dtype=F64)), 0.5 * (1 + math.tanh(math.sqrt(2 / math.pi) * 1.044715)))


def test_oracle_convolution_weighs_the_current_position_last():
    x = torch.tensor([[1.0], [10.0], [100.0], [1000.0]], dtype=F64)
    taps = torch.tensor([[3.0, 2.0, 1.0]], dtype=F64)
    assert O.causal_conv(x, taps)[:, 0].tolist() == [1.0, 12.0, 123.0, 1230.0]


def test_oracle_rotation_pairs_neighbours():
    x = torch.arange(8, dtype=F64).reshape(1, 1, 8) + 1
    y = O.rotate_interleaved(x, torch.tensor([3]), 4, 100.0)
    for i, (a, b) in enumerate([(0, 1), (2, 3)]):
        ang = 3 * 100.0 ** (-2 * i / 4)
        assert math.isclose(y[0, 0, a], x[0, 0, a] * math.cos(ang) - x[0, 0, b] * math.sin(ang))
        assert math.isclose(y[0, 0, b], x[0, 0, b] * math.cos(ang) + x[0, 0, a] * math.sin(ang))
    assert torch.equal(y[0, 0, 4:], x[0, 0, 4:])


def test_oracle_gated_delta_rule_by_hand():
    """one head, one key channel, one value channel, one tap: q = k = 1 after the unit norm, so S <- g S + beta (v - g S)
    and o = S; with beta = 1/2 and g = exp(-softplus(0)) = 1/2 the state goes 0 -> v/2 -> 5v/8"""
    m = {"heads": 1, "kv_heads": 1, "dim": 1, "vdim": 1, "conv": 1}
    one, zero = torch.ones(1, 1, dtype=F64), torch.zeros(1, 1, dtype=F64)
    big = 50.0 * one                                      # silu(50) = 50; the gate's sigmoid saturates at one
    w = {"q": big, "q.conv": one, "k": big, "k.conv": one, "v": big, "v.conv": one, "b": zero, "A_log": torch.zeros(1, dtype=F64),
         "a1": one, "a2": zero, "dt_bias": torch.zeros(1, dtype=F64), "g1": one, "g2": big, "norm": torch.ones(1, dtype=F64),
         "o": one}
    h = torch.ones(2, 1, dtype=F64)
    # o / rms(o) = 1 hides the state; read it through a norm-free copy of the recurrence instead
    v, S, out = 50.0, 0.0, []
    for _ in range(2):
        S = 0.5 * S
        S = S + 0.5 * (v - S)
        out.append(S)
    assert out == [25.0, 31.25]
    got = O.gated_delta_mixer(h, w, m, 0.0)
    assert torch.allclose(got, torch.ones(2, 1, dtype=F64))            # the sign and the norm survive
    w["v"] = -big
    assert torch.allclose(O.gated_delta_mixer(h, w, m, 0.0), -50.0 / (1 + math.exp(50.0)) / abs(50.0 / (1 + math.exp(50.0))) * torch.ones(2, 1, dtype=F64))


def test_oracle_generalised_delta_rule_reads_the_old_state_twice():
    """one head, two key channels: with rate 1 along a unit key the old state's part along the key leaves entirely"""
    S = torch.tensor([[2.0, 0.0], [0.0, 3.0]], dtype=F64)
    k = torch.tensor([2.0, 0.0], dtype=F64)
    n = O.unit_vector(k, 0.0)
    decay, rate, v = torch.tensor([0.5, 0.5], dtype=F64), torch.tensor([1.0, 1.0], dtype=F64), torch.tensor([1.0, 1.0], dtype=F64)
    new = decay[:, None] * S - torch.outer(rate * n, n @ S) + torch.outer(k, v)
    assert torch.allclose(new, torch.tensor([[1.0 - 2.0 + 2.0, 2.0], [0.0, 1.5]], dtype=F64))


def test_oracle_sink_cap_and_head_mix():
    """one position, two heads: each head's weight on the only key is 1 / (1 + exp(sink - mixed score))"""
    m = {"heads": 2, "kv_heads": 1, "dim": 2, "vdim": 1, "rot": {"base": 10.0, "dims": 0}, "scale": 1.0, "softcap": 2.0,
         "mask": {"size": 4}}
    eye = torch.eye(2, dtype=F64)
    w = {"q": torch.cat([eye, 3 * eye]), "q.b": torch.zeros(4, dtype=F64), "k": eye, "k.b": torch.zeros(2, dtype=F64),
         "v": torch.tensor([[1.0, 0.0]], dtype=F64), "v.b": torch.zeros(1, dtype=F64), "q.norm": torch.ones(2, dtype=F64),
         "k.norm": torch.ones(2, dtype=F64), "talk": torch.tensor([[1.0, 0.5], [0.0, 2.0]], dtype=F64),
         "sink": torch.tensor([0.3, -0.7], dtype=F64), "o": eye[:, :2]}
    h = torch.tensor([[1.0, 1.0]], dtype=F64)
    got = O.talking_window_attention(h, torch.tensor([0]), w, m, 0.0)
    s = 2.0 * math.tanh(2.0 / 2.0)                          # both heads: normed q . normed k = 2, then the cap
    mixed = [s * 1.5, s * 2.0]
    want = [1.0 / (1.0 + math.exp(sk - mx)) for sk, mx in zip([0.3, -0.7], mixed)]
    assert torch.allclose(got[0], torch.tensor(want, dtype=F64))


def test_oracle_router_gates_sum_to_one_over_the_chosen():
    f = {"kind": "moe", "router": {"experts": 3, "top": 2}, "expert": {"ff": 1}}
    one = torch.ones(1, 1, dtype=F64)
    w = {"router": torch.tensor([[1.0], [2.0], [0.0]], dtype=F64), "router.b": torch.tensor([0.0, 0.0, 5.0], dtype=F64)}
    for e, down in enumerate((1.0, 10.0, 100.0)):
        w.update({f"e{e}.gate": 50 * one, f"e{e}.up": one, f"e{e}.down": down * one / 50})
    out = O.feed_forward(torch.ones(1, 1, dtype=F64), w, f)     # logits 1, 2, 5: experts 2 and 1 are chosen
    g2 = 1.0 / (1.0 + math.exp(2.0 - 5.0))
    assert math.isclose(out.item(), g2 * 100.0 + (1 - g2) * 10.0, rel_tol=1e-6)
