"""CPU: the Lukopel family's configuration, registry entry, tensor packing and execution order, and the plain
restatement's own mechanisms on inputs made by hand (so that the oracle the GPU tests lean on is itself pinned)."""
import json
import math
import struct

import pytest
import torch

from oracle import lukopel_oracle as O

F64 = torch.float64


def test_config_round_trip_and_registry(tmp_path):
    from asd_b200.models import registry
    from asd_b200.models.lukopel import LukopelConfig, tensor_shapes, tiny_config
    cfg = tiny_config()
    d = cfg.to_dict()
    assert d["architecture"] == "Lukopel" and d["streams"] == 3
    back = LukopelConfig.from_dict(d, name="tiny").with_shapes(tensor_shapes(cfg))
    assert back == cfg
    fam = registry.family_of_dict(d)
    assert fam.name == "lukopel" and "lukopel" in fam.components and set(fam.dtypes) == {"bfloat16", "float32"}
    assert registry.family_of_config(cfg).name == "lukopel"
    assert O.tensor_shapes(d, rel_rows=[l.bias_rows for l in cfg.layers]) == tensor_shapes(cfg)
    # a checkpoint directory: the sizes that only a tensor's shape gives come from the safetensors header
    (tmp_path / "config.json").write_text(json.dumps(d))
    shapes = tensor_shapes(cfg)
    header, off = {}, 0
    for k, s in shapes.items():
        n = 2 * math.prod(s)
        header[k] = {"dtype": "BF16", "shape": list(s), "data_offsets": [off, off + n]}
        off += n
    hj = json.dumps(header).encode()
    (tmp_path / "model.safetensors").write_bytes(struct.pack("<Q", len(hj)) + hj + b"\0" * off)
    fam2, cfg2 = registry.read_config(str(tmp_path))
    assert fam2.name == "lukopel" and cfg2.layers == cfg.layers and cfg2.max_positions == cfg.max_positions


def test_defaults_of_absent_keys_and_refusals():
    from asd_b200.models.lukopel import LukopelConfig, tensor_shapes, tiny_config
    d = tiny_config().to_dict()
    del d["streams"], d["loop"]
    d["layers"][1]["mixer"].pop("kv_heads")
    cfg = LukopelConfig.from_dict(d)
    assert cfg.streams is None and cfg.n_streams == 1 and cfg.loop is None
    assert cfg.layers[1].kv_heads == cfg.layers[1].heads
    assert not any(".hc" in k for k in tensor_shapes(cfg))            # the ordinary residual has no stream weights
    assert cfg.layers[2].ff_kind is None and "l2.norm2" not in tensor_shapes(cfg)
    bad = json.loads(json.dumps(d))
    bad["layers"][0]["type"] = "convolution"
    with pytest.raises(ValueError):
        LukopelConfig.from_dict(bad)
    bad = json.loads(json.dumps(d))
    bad["loop"] = {"start": 2, "stop": 2, "times": 2}
    with pytest.raises(ValueError):
        LukopelConfig.from_dict(bad)


def test_execution_order_of_a_repeated_span():
    from asd_b200.models.lukopel import tiny_config
    cfg = tiny_config(loop=(1, 3, 3))
    assert cfg.runs() == [(0, -1), (1, 0), (2, 0), (1, 1), (2, 1), (1, 2), (2, 2)]
    assert [i for i, _ in cfg.runs()] == O.layer_runs(cfg.to_dict())
    assert [i for i, _ in tiny_config(loop=None).runs()] == [0, 1, 2]
    assert cfg.kv_bytes_per_token(2) == 2 * sum(cfg.layers[i].cache_row for i, _ in cfg.runs())


def test_packing_stacks_projections_and_expands_the_distance_bias():
    from asd_b200.models.lukopel import distance_rows, pack, random_weights, tiny_config
    cfg = tiny_config()
    w = random_weights(cfg, seed=1)
    p = pack(w, cfg, "cpu", torch.bfloat16)
    l0, l1 = cfg.layers[0], cfg.layers[1]
    nq, nk, nv = l0.heads * l0.dim, l0.kv_heads * l0.dim, l0.kv_heads * l0.vdim
    assert p[(0, "w_in")].shape == (nq + nk + nv + l0.heads, cfg.width)
    assert torch.equal(p[(0, "w_in")][nq + nk + nv:], w["l0.mix.g"])
    assert p[(1, "w_in")].shape == (l1.heads * l1.dim + l1.kv_heads * (l1.dim + l1.vdim), cfg.width)
    assert p[(1, "in_bias")].dtype == torch.float32 and p[(1, "in_bias")].numel() == p[(1, "w_in")].shape[0]
    assert (1, "dist_bias") not in p and (1, "talk") not in p and (0, "in_bias") not in p and (0, "head_factor") not in p
    tab = p[(0, "dist_bias")]
    assert tab.shape == (l0.far + 1, l0.heads) and tab.dtype == torch.float32
    rows = distance_rows(l0.bias_rows, l0.bias_max, l0.far)
    for n in (0, 1, l0.bias_rows // 2 - 1, l0.bias_rows // 2, l0.bias_max - 1, l0.bias_max):
        assert torch.equal(tab[n], w["l0.mix.rel"][rows[n]].float())
        assert rows[n] == O.distance_bucket(n, l0.bias_rows, l0.bias_max)
    assert rows[l0.bias_max] == l0.bias_rows - 1 and rows == sorted(rows)
    assert p[(0, "hc2_mix")].shape == (3, 3) and (2, "hc2_mix") not in p and (2, "hc1_mix") in p
    assert p[(-1, "pos")].shape == (cfg.max_positions, cfg.width)
    with pytest.raises(KeyError):
        pack({k: v for k, v in w.items() if k != "l1.mix.temp"}, cfg, "cpu", torch.bfloat16)
    w["l0.mix.talk"] = w["l0.mix.talk"][:, :-1]
    with pytest.raises(ValueError):
        pack(w, cfg, "cpu", torch.bfloat16)


@pytest.mark.parametrize("rows,far", [(16, 120), (10, 40), (4, 9), (32, 64), (6, 1000)])
def test_distance_rows_against_their_definition(rows, far):
    """every distance, the slow way: below rows / 2 the distance itself; beyond, the largest step whose lower edge
    half * (far / half)^(step / (rows - half)) is not above the distance"""
    from asd_b200.models.lukopel import distance_rows
    half = rows // 2
    got = distance_rows(rows, far, far + 5)
    for n, r in enumerate(got):
        if n < half:
            assert r == n
            continue
        step = 0
        while step + 1 <= rows - half and half * (far / half) ** ((step + 1) / (rows - half)) <= n * (1 + 1e-12):
            step += 1
        assert r == min(rows - 1, half + step), n
        assert r == O.distance_bucket(n, rows, far)


# ------------------------------------------------------------------------------------------------ the oracle, by hand
def test_oracle_streams_by_hand():
    """two streams holding 1 and 10; y = 100: new[t] = sum_s mix[s, t] old[s] + out[t] y"""
    xs = torch.tensor([1.0, 10.0], dtype=F64).reshape(2, 1, 1)
    assert O.streams_read(xs, torch.tensor([2.0, 0.5], dtype=F64)).item() == 7.0
    mix = torch.tensor([[1.0, 2.0], [3.0, 4.0]], dtype=F64)        # [from, to]
    new = O.streams_write(xs, torch.tensor([[100.0]], dtype=F64), mix, torch.tensor([1.0, -1.0], dtype=F64))
    assert new.flatten().tolist() == [1.0 * 1 + 3.0 * 10 + 100.0, 2.0 * 1 + 4.0 * 10 - 100.0]


def test_oracle_one_stream_with_unit_weights_is_the_residual_sum():
    cfg = {"architecture": "Lukopel", "width": 16, "vocab": 20, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0},
           "max_positions": 12, "layers": [{"type": "attention_2", "mixer": {"heads": 2, "kv_heads": 1, "dim": 4, "vdim": 4,
                                                                              "scale": 0.5, "mask": {"size": 3}},
                                            "mlp": {"kind": "dense", "ff": 8}}]}
    w = O.random_model(cfg, seed=1)
    ids = [3, 1, 4, 1, 5, 9, 2, 6]
    plain = O.forward(ids, w, cfg)
    c1 = dict(cfg, streams=1)
    w1 = dict(w)
    for q in (1, 2):
        w1[f"l0.hc{q}.in"] = torch.ones(1)
        w1[f"l0.hc{q}.out"] = torch.ones(1)
        w1[f"l0.hc{q}.mix"] = torch.ones(1, 1)
    assert torch.allclose(O.forward(ids, w1, c1), plain, rtol=0, atol=1e-12)


def test_oracle_masks_and_query_factor():
    m = O.same_chunk_mask(7, 3)
    assert m.int().tolist() == [[1, 0, 0, 0, 0, 0, 0], [1, 1, 0, 0, 0, 0, 0], [1, 1, 1, 0, 0, 0, 0], [0, 0, 0, 1, 0, 0, 0],
                                [0, 0, 0, 1, 1, 0, 0], [0, 0, 0, 1, 1, 1, 0], [0, 0, 0, 0, 0, 0, 1]]
    assert O.causal_mask(3).int().tolist() == [[1, 0, 0], [1, 1, 0], [1, 1, 1]]
    f = O.query_temperature(9, 0.5, 4)          # floor((p + 1) / 4) = 0 0 0 1 1 1 1 2 2
    want = [1.0] * 3 + [1.0 + 0.5 * math.log(2.0)] * 4 + [1.0 + 0.5 * math.log(3.0)] * 2
    assert torch.allclose(f, torch.tensor(want, dtype=F64))


def test_oracle_weights_are_mixed_after_the_softmax():
    """two positions, two heads, one value channel; the second position's weights are softmax rows, mixed by talk, so
    with talk = [[1, 1], [0, 2]] head 0 applies the SUM of both heads' weights (which adds up to 2, not 1)"""
    m = {"heads": 2, "kv_heads": 1, "dim": 1, "vdim": 1, "scale": 1.0, "bias_max": 4, "q_temp": {"coef": 0.0, "every": 1}}
    one = torch.ones(1, 1, dtype=F64)
    w = {"q": torch.tensor([[1.0], [-1.0]], dtype=F64), "k": one, "v": one, "q.norm": torch.ones(1, dtype=F64),
         "k.norm": torch.ones(1, dtype=F64), "rel": torch.tensor([[0.0, 0.0], [1.0, -2.0]], dtype=F64),
         "talk": torch.tensor([[1.0, 1.0], [0.0, 2.0]], dtype=F64), "g": torch.zeros(2, 1, dtype=F64),
         "o": torch.eye(2, dtype=F64)}
    h = torch.tensor([[1.0], [-1.0]], dtype=F64)
    out = O.biased_attention(h, w, "", m, 0.0)
    # values are unit-RMS: v = +1 at position 0 and -1 at position 1; the gates are sigmoid(0) = 1/2.
    # position 1: q = (-1, +1) after the norm, k = (+1, -1) for positions (0, 1)
    s0 = torch.tensor([-1.0 + 1.0, 1.0 + 0.0])      # head 0: scores of keys 0 (distance 1, bias 1) and 1 (distance 0)
    s1 = torch.tensor([1.0 - 2.0, -1.0 + 0.0])      # head 1
    a0, a1 = torch.softmax(s0, 0), torch.softmax(s1, 0)
    mixed0, mixed1 = a0 + a1, 2 * a1
    want = torch.tensor([(mixed0[0] - mixed0[1]) / 2, (mixed1[0] - mixed1[1]) / 2], dtype=F64)
    assert torch.allclose(out[1], want, atol=1e-12)
    assert torch.allclose(out[0], torch.tensor([1.0, 1.0], dtype=F64), atol=1e-12)       # (1 + 1) / 2 and 2 / 2


def test_oracle_chunked_attention_norms_the_whole_projection():
    """two heads of one channel: the norm divides by the root mean square over BOTH heads, so the heads keep their ratio"""
    m = {"heads": 2, "kv_heads": 2, "dim": 1, "vdim": 1, "scale": 1.0, "mask": {"size": 8}}
    z2 = torch.zeros(2, dtype=F64)
    w = {"q": torch.tensor([[3.0], [4.0]], dtype=F64), "q.b": z2, "k": torch.tensor([[1.0], [1.0]], dtype=F64), "k.b": z2,
         "v": torch.tensor([[1.0], [2.0]], dtype=F64), "v.b": torch.tensor([0.5, 0.0], dtype=F64), "q.norm": torch.ones(2, dtype=F64),
         "k.norm": torch.ones(2, dtype=F64), "temp": torch.ones(2, dtype=F64), "o": torch.eye(2, dtype=F64),
         "o.b": torch.tensor([10.0, 20.0], dtype=F64)}
    h = torch.tensor([[1.0]], dtype=F64)
    q = O.rms_norm(h @ w["q"].T, w["q.norm"], 0.0)
    assert torch.allclose(q, torch.tensor([[3.0, 4.0]], dtype=F64) / math.sqrt(12.5))
    out = O.chunked_attention(h, w, "", m, 0.0)
    assert torch.allclose(out, torch.tensor([[1.5 + 10.0, 2.0 + 20.0]], dtype=F64))     # one key: the biased value itself


def test_oracle_feed_forward_by_hand():
    w = {"up": torch.tensor([[1.0], [-1.0]], dtype=F64), "up.b": torch.tensor([1.0, 0.5], dtype=F64),
         "down": torch.tensor([[1.0, 1.0]], dtype=F64), "down.b": torch.tensor([0.25], dtype=F64)}
    out = O.dense_ff(torch.tensor([[2.0]], dtype=F64), w, "")
    assert out.item() == 3.0 ** 2 + 0.0 + 0.25
