"""GPU: the Lukopel engine against the plain restatement in oracle/lukopel_oracle.py (fp64, whole sequences, no cache).
Every test makes its own small configuration and random weights.  The fp32 engine is held to 2e-4 of the logits'
spread, which a single key missed or double-counted among hundreds, a chunk edge off by one, a wrong bias row, an
unmixed weight, a lost stream or a stale page all exceed; the bf16 engine to what its roundings allow."""
import copy
import json
import os
import struct
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import lukopel_oracle as O  # noqa: E402


# ------------------------------------------------------------------------------------------------ configurations
def dense(ff=48):
    return {"kind": "dense", "ff": ff} if ff else None


def full(heads=6, kv_heads=3, dim=20, vdim=12, scale=0.2, bias_max=40, coef=0.25, every=7, mlp=None):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
                                           "bias_max": bias_max, "q_temp": {"coef": coef, "every": every}}, "mlp": mlp}


def chunked(heads=4, kv_heads=2, dim=16, vdim=24, scale=0.3, size=11, mlp=None):
    return {"type": "attention_2", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
                                             "mask": {"size": size}}, "mlp": mlp}


def config(layers, width=96, vocab=120, eps=1e-5, streams=3, loop=None, embed_scale=3.0, max_positions=800):
    d = {"architecture": "Lukopel", "width": width, "vocab": vocab, "norm": {"eps": eps}, "embedding": {"scale": embed_scale},
         "max_positions": max_positions, "layers": layers}
    if streams is not None:
        d["streams"] = streams
    if loop:
        d["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return d


# both mixers, with and without a feed-forward, a repeated span in the middle
SMALL = config([full(mlp=dense(72)), chunked(mlp=dense(56)), full(heads=2, kv_heads=2, dim=24, vdim=40, bias_max=18, coef=0.5, every=4),
                chunked(heads=2, kv_heads=1, dim=24, vdim=8, size=5, mlp=dense(32))], loop=(1, 3, 2))
# sizes that are multiples of nothing; the span starts at the first layer and runs three times; one key head per query
# head and one for all; two streams; a chunk of one position; a query factor that changes at every position
ODD = config([chunked(heads=3, kv_heads=1, dim=10, vdim=7, size=13, mlp=dense(50)),
              full(heads=5, kv_heads=5, dim=10, vdim=6, bias_max=9, every=1, mlp=dense(9)),
              full(heads=6, kv_heads=1, dim=14, vdim=34, scale=0.5, bias_max=300, coef=0.0, every=1000),
              chunked(heads=1, kv_heads=1, dim=40, vdim=66, size=1, mlp=dense(21))],
             width=72, vocab=101, eps=1e-3, streams=2, loop=(0, 2, 3), embed_scale=0.5)
PLAIN = config([full(mlp=dense(32)), chunked()], streams=None)       # the ordinary residual sum, no repeated span
WHOLE = config([chunked(mlp=dense(40)), full()], streams=1, loop=(0, 2, 1))   # one stream WITH its weights; a span that is all
REL_ROWS = {"small": 10, "odd": [0, 6, 16, 0], "plain": 4, "whole": 12}


def make_engine(cfg_dict, w, dtype=torch.float32, max_tokens=64, max_seq_len=512, page_size=16, num_pages=None,
                max_seqs=4, tc=1):
    from asd_b200.engine import LukopelEngine
    from asd_b200.models.lukopel import LukopelConfig
    cfg = LukopelConfig.from_dict(cfg_dict).with_shapes({k: tuple(v.shape) for k, v in w.items()})
    eng = LukopelEngine(cfg, max_seqs=max_seqs, max_seq_len=max_seq_len, max_tokens=max_tokens, page_size=page_size,
                        dtype=dtype, dynamic_pages=True, num_pages=num_pages)
    eng.load_weights(w)
    eng.set_option("tc_linear", tc)
    return eng


def close(eng):
    """no kernel of the engine gave up a wait"""
    eng.check_device()
    eng.close()


def tokens(n, vocab, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def rel_err(got, want):
    got, want = got.double().cpu(), want.double()
    return ((got - want).norm() / want.norm()).item(), ((got - want).abs().max() / want.std()).item()


def feed(eng, slot, ids, cuts, start=0):
    """feeds ids in portions of the given sizes (the rest in one go), all logits wanted"""
    out, a = [], 0
    sizes = list(cuts)
    while a < len(ids):
        n = sizes.pop(0) if sizes else len(ids) - a
        n = min(n, len(ids) - a)
        eng.reserve(slot, start + a + n)
        out.append(eng.forward_ragged([(slot, start + a, ids[a:a + n], list(range(n)))]))
        a += n
    return torch.cat(out, 0)


def run_whole(cfg_dict, w, ids, **kw):
    eng = make_engine(cfg_dict, w, **kw)
    slot = eng.open_sequence()
    got = feed(eng, slot, ids, [])
    close(eng)
    return got


def oracle(cfg_dict, w, ids, streams=None):
    return O.forward(ids, w, cfg_dict, layers_out=streams)


def silence_mixer(w, i=0):
    for k in (f"l{i}.mix.o", f"l{i}.mix.o.b"):
        if k in w:
            w[k] = torch.zeros_like(w[k])


# ------------------------------------------------------------------------------------------------ whole prompts
@pytest.mark.parametrize("name,cfg_dict", [("small", SMALL), ("odd", ODD), ("plain", PLAIN), ("whole", WHOLE)])
def test_whole_prompt_logits_and_every_layer_execution(name, cfg_dict):
    w = O.random_model(cfg_dict, seed=1, rel_rows=REL_ROWS[name])
    ids = tokens(45, cfg_dict["vocab"], 2)
    streams = []
    ref = oracle(cfg_dict, w, ids, streams)
    eng = make_engine(cfg_dict, w)
    slot = eng.open_sequence()
    eng.reserve(slot, len(ids))
    got, st = eng.forward_ragged([(slot, 0, ids, list(range(len(ids))))], layer_out=True)
    st = torch.cat(st, 1).cpu().double()
    assert st.shape[0] == len(O.layer_runs(cfg_dict)) == len(streams)
    for i in range(st.shape[0]):           # the first execution that differs names the mechanism
        assert (st[i] - streams[i]).abs().max() <= 2e-4 * streams[i].abs().max(), f"streams leaving execution {i}"
    assert rel_err(got, ref)[1] < 2e-4
    close(eng)


# ------------------------------------------------------------------------------------------------ mechanisms alone
def test_embedding_scale_position_vectors_and_final_norm_alone():
    """no layers: logits = head . norm(streams * (embed * scale + pos)); scale and positions change the answer"""
    for streams in (None, 1, 4):
        cfg = config([], width=40, vocab=50, streams=streams, embed_scale=2.5)
        w = O.random_model(cfg, seed=3)
        ids = tokens(20, 50, 4)
        ref = oracle(cfg, w, ids)
        assert rel_err(run_whole(cfg, w, ids), ref)[1] < 1e-4
        # the same tokens later in the sequence: other position vectors
        eng = make_engine(cfg, w)
        slot = eng.open_sequence()
        got = feed(eng, slot, ids + ids, [20])
        assert rel_err(got, oracle(cfg, w, ids + ids))[1] < 1e-4
        assert rel_err(got[20:], ref)[1] > 1e-2
        close(eng)
        c2 = copy.deepcopy(cfg)
        c2["embedding"]["scale"] = 1.0
        assert rel_err(oracle(c2, w, ids).float(), ref)[1] > 1e-2


@pytest.mark.parametrize("streams", [None, 1, 2, 4, 5, 8, 11])
def test_residual_streams_alone(streams):
    """feed-forward sublayers only (the mixers' output projections are zero): reads, stream-to-stream matrices and
    writes; the matrix is indexed [from, to], which its transpose shows"""
    cfg = config([chunked(mlp=dense(40)), chunked(mlp=dense(24)), chunked()], streams=streams, width=64)
    w = O.random_model(cfg, seed=5)
    for i in range(3):
        silence_mixer(w, i)
    ids = tokens(30, 120, 6)
    ref = oracle(cfg, w, ids)
    assert rel_err(run_whole(cfg, w, ids), ref)[1] < 2e-4
    if streams and streams > 1:
        w2 = dict(w)
        w2["l0.hc2.mix"] = w["l0.hc2.mix"].T.contiguous()
        assert rel_err(oracle(cfg, w2, ids).float(), ref)[1] > 1e-2
        w2 = dict(w)
        w2["l1.hc2.in"] = torch.ones_like(w["l1.hc2.in"])
        assert rel_err(oracle(cfg, w2, ids).float(), ref)[1] > 1e-3


def test_squared_relu_feed_forward_alone_with_its_biases():
    cfg = config([chunked(mlp=dense(56))])
    w = O.random_model(cfg, seed=7, scale=2.0)
    silence_mixer(w)
    ids = tokens(33, 120, 8)
    ref = oracle(cfg, w, ids)
    assert rel_err(run_whole(cfg, w, ids), ref)[1] < 2e-4
    for k in ("l0.mlp.up.b", "l0.mlp.down.b"):
        w2 = dict(w)
        w2[k] = torch.zeros_like(w[k])
        assert rel_err(oracle(cfg, w2, ids).float(), ref)[1] > 1e-2, k


def test_biased_attention_alone_every_step_matters():
    cfg = config([full(heads=4, kv_heads=2, dim=16, vdim=12, scale=0.6, bias_max=24, coef=0.8, every=5)])
    w = O.random_model(cfg, seed=9, rel_rows=8)
    ids = tokens(64, 120, 10)
    ref = oracle(cfg, w, ids)
    assert rel_err(run_whole(cfg, w, ids), ref)[1] < 2e-4
    # unmixed weights, a mix before the softmax's normalisation would differ too, no distance bias, shifted rows of
    # it, no gate, no query factor, unnormed values: all far outside
    for k, t in (("l0.mix.talk", torch.eye(4)), ("l0.mix.rel", torch.zeros(8, 4)), ("l0.mix.rel", w["l0.mix.rel"].roll(1, 0)),
                 ("l0.mix.g", torch.zeros(4, 96)), ("l0.mix.talk", w["l0.mix.talk"].T.contiguous())):
        w2 = dict(w)
        w2[k] = t.to(torch.bfloat16)
        assert rel_err(oracle(cfg, w2, ids).float(), ref)[1] > 1e-2, k
    for change in ({"q_temp": {"coef": 0.0, "every": 5}}, {"q_temp": {"coef": 0.8, "every": 6}}, {"bias_max": 23},
                   {"scale": 0.5}):
        c2 = copy.deepcopy(cfg)
        c2["layers"][0]["mixer"].update(change)
        assert rel_err(oracle(c2, w, ids).float(), ref)[1] > 1e-3, change
    for cuts in ([1] * 64, [2] * 32, [33, 3, 1, 1, 2]):
        eng = make_engine(cfg, w)
        slot = eng.open_sequence()
        assert rel_err(feed(eng, slot, ids, cuts), ref)[1] < 2e-4, cuts
        close(eng)


def test_chunked_attention_alone_every_step_matters():
    cfg = config([chunked(heads=4, kv_heads=2, dim=16, vdim=12, scale=0.6, size=9)])
    w = O.random_model(cfg, seed=11)
    ids = tokens(64, 120, 12)
    ref = oracle(cfg, w, ids)
    assert rel_err(run_whole(cfg, w, ids), ref)[1] < 2e-4
    for k in ("l0.mix.q.b", "l0.mix.k.b", "l0.mix.v.b", "l0.mix.o.b"):
        w2 = dict(w)
        w2[k] = torch.zeros_like(w[k])
        assert rel_err(oracle(cfg, w2, ids).float(), ref)[1] > 1e-3, k
    w2 = dict(w)
    w2["l0.mix.temp"] = torch.ones(4, dtype=torch.bfloat16)
    assert rel_err(oracle(cfg, w2, ids).float(), ref)[1] > 1e-2
    w2 = dict(w)       # a norm head by head is not the norm over the whole projection
    w2["l0.mix.q"] = (w["l0.mix.q"].float() * torch.repeat_interleave(torch.tensor([0.2, 1.0, 3.0, 0.5]), 16)[:, None]).to(torch.bfloat16)
    ref2 = oracle(cfg, w2, ids)
    assert rel_err(run_whole(cfg, w2, ids), ref2)[1] < 2e-4
    for size in (8, 10):
        c2 = copy.deepcopy(cfg)
        c2["layers"][0]["mixer"]["mask"]["size"] = size
        assert rel_err(oracle(c2, w, ids).float(), ref)[1] > 1e-2
    for cuts in ([1] * 64, [2] * 32, [8, 1, 1, 9, 17, 2]):
        eng = make_engine(cfg, w)
        slot = eng.open_sequence()
        assert rel_err(feed(eng, slot, ids, cuts), ref)[1] < 2e-4, cuts
        close(eng)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
def test_many_heads_large_heads_and_sizes_that_divide_nothing(dtype):
    """twenty and eighty mixed heads, sixteen key/value heads (an apply CTA then multiplies the values of a part of them),
    value heads of 100, 128, 200 and 256, keys of 136 and of 7, one query head per key head and forty per key head"""
    cfg = config([full(heads=20, kv_heads=4, dim=16, vdim=16, bias_max=30),
                  full(heads=16, kv_heads=16, dim=8, vdim=12, bias_max=12),
                  chunked(heads=2, kv_heads=1, dim=136, vdim=128, size=50, scale=0.05),
                  full(heads=3, kv_heads=1, dim=7, vdim=100, bias_max=64, scale=0.4),
                  chunked(heads=40, kv_heads=1, dim=12, vdim=5, size=23),
                  full(heads=80, kv_heads=10, dim=8, vdim=4, bias_max=20), chunked(heads=2, kv_heads=2, dim=16, vdim=200, size=31),
                  full(heads=2, kv_heads=1, dim=12, vdim=256, bias_max=50)])
    w = O.random_model(cfg, seed=15, rel_rows=[12, 6, 0, 20, 0, 8, 0, 4])
    ids = tokens(80, 120, 16)
    ref = oracle(cfg, w, ids)
    for cuts in ([80], [60] + [1] * 20, [7] * 12):
        eng = make_engine(cfg, w, dtype=dtype, max_tokens=128)
        slot = eng.open_sequence()
        got = feed(eng, slot, ids, cuts)
        assert (rel_err(got, ref)[1] < 2e-4) if dtype == torch.float32 else (rel_err(got, ref)[0] < 5e-2)
        close(eng)


# ------------------------------------------------------------------------------------------------ cache, portions, batches
@pytest.mark.parametrize("name,cfg_dict", [("small", SMALL), ("odd", ODD)])
@pytest.mark.parametrize("page_size", [4, 16])
def test_prefill_then_decode_and_portions(name, cfg_dict, page_size):
    w = O.random_model(cfg_dict, seed=17, rel_rows=REL_ROWS[name])
    ids = tokens(75, cfg_dict["vocab"], 18)
    ref = oracle(cfg_dict, w, ids)
    for cuts in ([75], [1] * 75, [40] + [1] * 35, [2] * 38, [3, 5, 7, 11, 13, 17, 2, 2], [64, 11]):
        eng = make_engine(cfg_dict, w, page_size=page_size)
        slot = eng.open_sequence()
        assert rel_err(feed(eng, slot, ids, cuts), ref)[1] < 2e-4, cuts
        close(eng)


def test_forward_larger_than_the_engine_step_is_cut_inside():
    w = O.random_model(SMALL, seed=19)
    ids = tokens(150, 120, 20)
    assert rel_err(run_whole(SMALL, w, ids, max_tokens=32), oracle(SMALL, w, ids))[1] < 2e-4


def test_batch_of_unequal_requests_equals_each_alone():
    w = O.random_model(SMALL, seed=21)
    reqs = [tokens(n, 120, 22 + n) for n in (37, 1, 64, 9)]
    refs = [oracle(SMALL, w, r) for r in reqs]
    eng = make_engine(SMALL, w, max_tokens=128)
    slots = [eng.open_sequence() for _ in reqs]
    # step 1: a prompt part of every request at once; step 2: what is left, one token for one of them
    first = [20, 1, 50, 8]
    items = []
    for s, r, n in zip(slots, reqs, first):
        eng.reserve(s, len(r))
        items.append((s, 0, r[:n], list(range(n))))
    got1 = eng.forward_ragged(items)
    items = [(s, n, r[n:], list(range(len(r) - n))) for s, r, n in zip(slots, reqs, first) if len(r) > n]
    got2 = eng.forward_ragged(items)
    a = b = 0
    for r, ref, n in zip(reqs, refs, first):
        assert rel_err(got1[a:a + n], ref[:n])[1] < 2e-4
        a += n
        if len(r) > n:
            assert rel_err(got2[b:b + len(r) - n], ref[n:])[1] < 2e-4
            b += len(r) - n
    close(eng)


def test_pages_and_slots_freed_and_used_again():
    """a pool that holds one request at a time: every request lands on the pages and the slot of the one before"""
    w = O.random_model(SMALL, seed=23)
    eng = make_engine(SMALL, w, page_size=8, num_pages=12, max_seqs=2, max_seq_len=96)
    for i, n in enumerate((90, 33, 96, 5, 64)):
        ids = tokens(n, 120, 24 + i)
        slot = eng.open_sequence()
        got = feed(eng, slot, ids, [n // 2, 1, 2])
        assert rel_err(got, oracle(SMALL, w, ids))[1] < 2e-4, i
        eng.close_sequence(slot)
    assert eng.pages.pages_in_use() == 0
    close(eng)


def test_long_decoding_passes_chunk_edges_bias_rows_and_key_shares():
    """300 single-token steps after a short prompt: every chunk edge, every row of the distance bias, the query factor's
    steps, and key ranges long enough to be cut into shares for several CTAs"""
    cfg = config([full(heads=4, kv_heads=2, dim=16, vdim=12, bias_max=200, every=50, mlp=dense(40)),
                  chunked(heads=4, kv_heads=1, dim=16, vdim=20, size=70, mlp=dense(24))], loop=(0, 2, 2))
    w = O.random_model(cfg, seed=25, rel_rows=14)
    ids = tokens(330, 120, 26)
    ref = oracle(cfg, w, ids)
    eng = make_engine(cfg, w, page_size=8)
    slot = eng.open_sequence()
    got = feed(eng, slot, ids, [30] + [1] * 300)
    assert rel_err(got, ref)[1] < 2e-4
    for p in (69, 70, 139, 140, 209, 210, 229, 230, 329):
        assert rel_err(got[p:p + 1], ref[p:p + 1])[1] < 2e-4, p
    close(eng)


# ------------------------------------------------------------------------------------------------ edges, with standout keys
def first_input(cfg, w, tok, layer=0):
    """what the first layer's mixer reads for a token, positions aside (the tests that use it make the position vectors
    small): the normed embedding"""
    x = w["embed"][tok].double() * cfg["embedding"]["scale"]
    return O.rms_norm(x, w[f"l{layer}.norm1"].double(), cfg["norm"]["eps"])


def plant_pair(cfg, w, key_tok, query_tok, boost=60.0):
    """Makes the first layer's queries of ``query_tok`` point, before their norm, along the keys of ``key_tok`` in every
    head: after the norms this one score stands out wherever the key is visible."""
    m = cfg["layers"][0]["mixer"]
    H, G, dk = m["heads"], m["kv_heads"], m["dim"]
    hk, hq = first_input(cfg, w, key_tok), first_input(cfg, w, query_tok)
    k = w["l0.mix.k"].double() @ hk
    if "l0.mix.k.b" in w:
        k = k + w["l0.mix.k.b"].double()
    k = k.reshape(G, dk)
    q = w["l0.mix.q"].double().reshape(H, dk, -1).clone()
    for h in range(H):
        kk = k[h // (H // G)]
        q[h] += boost * torch.outer(kk / kk.norm(), hq) / (hq @ hq)
    w["l0.mix.q"] = q.reshape(H * dk, -1).to(torch.bfloat16)


def quiet_positions(w, factor=0.02):
    w["pos"] = (w["pos"].float() * factor).to(torch.bfloat16)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
@pytest.mark.parametrize("size,page_size", [(9, 16), (16, 16), (33, 4), (150, 16), (64, 8), (129, 8), (1, 8)])
def test_chunk_edges_with_standout_keys(size, page_size, dtype):
    """a key that outweighs everything else is the last position of a chunk, and the query that looks for it either the
    same position's chunk mate or the first position of the next chunk (which must not see it); in a prompt, in
    portions and while decoding"""
    cfg = config([chunked(heads=4, kv_heads=2, dim=48, vdim=16, size=size, scale=0.25)], max_positions=1200)
    w = O.random_model(cfg, seed=33)
    quiet_positions(w)
    w["l0.mix.q.b"] = torch.zeros_like(w["l0.mix.q.b"])
    V = cfg["vocab"]
    nchunks = max(4, 200 // size)
    n = nchunks * size + 3
    ids = [t % (V - 8) for t in tokens(n, V, 34)]
    at_in, at_out = [], []
    # pairs: (key position, query position); the first position of a chunk reaches back to nothing but itself
    c1, c2 = (nchunks // 2) * size, (nchunks - 1) * size
    plan = [(c1 - 1, c1, at_out), (c2 - 1, c2, at_out)]
    if size > 1:
        plan += [(c1, c1 + size - 1, at_in), (c2 - size, c2 - 1, at_in)]
    for i, (a, qpos, where) in enumerate(plan):
        key_tok, query_tok = V - 1 - 2 * i, V - 2 - 2 * i          # every pair has tokens of its own
        plant_pair(cfg, w, key_tok, query_tok)
        ids[a], ids[qpos] = key_tok, query_tok
        where.append(qpos)
    ref = oracle(cfg, w, ids)
    # the oracle itself says that these places see a chunk edge that is off by one
    for dsize in (-1, 1):
        if size + dsize < 1:
            continue
        c3 = copy.deepcopy(cfg)
        c3["layers"][0]["mixer"]["mask"]["size"] = size + dsize
        other = oracle(c3, w, ids)
        assert max(rel_err(other[p:p + 1].float(), ref[p:p + 1])[1] for p in at_in + at_out) > 0.3, dsize
    marked = at_in + at_out
    first_q = min(marked)
    for cuts in ([n], [first_q - 1, 2, 1, 1, 37, 2, 1, 1], [first_q - 3] + [1] * (n - first_q + 3), [2] * (n // 2 + 1)):
        eng = make_engine(cfg, w, max_tokens=512, page_size=page_size, max_seq_len=1280, dtype=dtype)
        slot = eng.open_sequence()
        got = feed(eng, slot, ids, cuts)
        if dtype == torch.float32:
            assert rel_err(got, ref)[1] < 1e-3
        else:
            assert rel_err(got, ref)[0] < 6e-2
        for p in marked:
            assert rel_err(got[p:p + 1], ref[p:p + 1])[1] < (1e-3 if dtype == torch.float32 else 0.3), p
        close(eng)


@pytest.mark.parametrize("bias_max,rows", [(40, 10), (120, 16), (9, 4), (64, 32)])
def test_distance_bias_rows_decide_at_their_edges(bias_max, rows):
    """one head's bias table is a tall step at one row: the query then looks exactly at the distances of that row, so a
    row boundary that is off by one distance shows; checked at every row, in a prompt and while decoding"""
    cfg = config([full(heads=2, kv_heads=1, dim=16, vdim=12, scale=0.05, bias_max=bias_max, coef=0.0, every=3)],
                 max_positions=400)
    n = min(380, 2 * bias_max + 40)
    ids = tokens(n, 120, 36)
    for row in range(rows):
        w = O.random_model(cfg, seed=37, rel_rows=rows)
        rel = torch.zeros(rows, 2)
        rel[row] = torch.tensor([25.0, 20.0])
        w["l0.mix.rel"] = rel.to(torch.bfloat16)
        ref = oracle(cfg, w, ids)
        eng = make_engine(cfg, w, max_tokens=512)
        slot = eng.open_sequence()
        got = feed(eng, slot, ids, [n - 40] + [1] * 40)
        assert rel_err(got, ref)[1] < 5e-4, row
        close(eng)
    # the rows' edges themselves, restated: distances below rows / 2 one by one, the last row from bias_max on
    half = rows // 2
    assert [O.distance_bucket(d, rows, bias_max) for d in range(half)] == list(range(half))
    assert O.distance_bucket(bias_max, rows, bias_max) == rows - 1 and O.distance_bucket(bias_max - 1, rows, bias_max) <= rows - 1


def test_far_key_among_hundreds_and_first_tokens():
    """a plain causal mask sees everything before it; a standout key 600 positions back (the sequence's first token)
    decides the answer, in one prompt, in portions and while decoding"""
    cfg = config([full(heads=4, kv_heads=2, dim=48, vdim=16, scale=0.25, bias_max=100, coef=0.1, every=64)], max_positions=800)
    w = O.random_model(cfg, seed=35, rel_rows=8)
    quiet_positions(w)
    w["l0.mix.rel"] = (w["l0.mix.rel"].float() * 0.2).to(torch.bfloat16)
    ids = [t % 110 for t in tokens(700, 120, 36)]
    plant_pair(cfg, w, 119, 118)
    ids[0], ids[600], ids[655] = 119, 118, 118
    ref = oracle(cfg, w, ids)
    gone = oracle(cfg, w, [5] + ids[1:])
    assert rel_err(gone[600:601].float(), ref[600:601])[1] > 0.3
    for cuts in ([700], [650] + [1] * 50, [37] * 18):
        eng = make_engine(cfg, w, max_tokens=1024, max_seq_len=1024)
        slot = eng.open_sequence()
        got = feed(eng, slot, ids, cuts)
        assert rel_err(got, ref)[1] < 1e-3
        for p in (0, 1, 2, 600, 655):
            assert rel_err(got[p:p + 1], ref[p:p + 1])[1] < 1e-3, p
        close(eng)


def test_single_token_steps_with_key_shares_over_several_ctas():
    """one and three requests that each add a token to 900 cached positions: few CTAs, so the keys are cut into shares
    whose partial results are merged; against the same positions inside one long prompt"""
    cfg = config([full(heads=4, kv_heads=2, dim=32, vdim=24, bias_max=500, every=100),
                  chunked(heads=4, kv_heads=4, dim=16, vdim=72, size=400)], max_positions=1000)
    w = O.random_model(cfg, seed=39, rel_rows=20)
    reqs = [tokens(905, 120, 40 + i) for i in range(3)]
    refs = [oracle(cfg, w, r) for r in reqs]
    for dtype in (torch.float32, torch.bfloat16):
        eng = make_engine(cfg, w, max_tokens=1024, max_seq_len=1024, dtype=dtype, max_seqs=3)
        slots = [eng.open_sequence() for _ in reqs]
        for s, r in zip(slots, reqs):
            eng.reserve(s, 905)
            eng.forward_ragged([(s, 0, r[:900], [])])
        for t in range(900, 905):
            got = eng.forward_ragged([(s, t, [r[t]], [0]) for s, r in zip(slots, reqs)])
            for i, ref in enumerate(refs):
                e = rel_err(got[i:i + 1], ref[t:t + 1])
                assert (e[1] < 2e-4) if dtype == torch.float32 else (e[0] < 5e-2), (t, i)
        close(eng)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
def test_general_and_special_attention_kernels_agree(dtype):
    """prompts of a bf16 engine run on the tensor cores and steps of few tokens keep their scores between two kernels;
    option attn_general sends everything through the general CUDA-core kernels instead: same logits"""
    cfg = config([full(heads=8, kv_heads=2, dim=32, vdim=32, bias_max=70, mlp=dense(64)),
                  chunked(heads=4, kv_heads=4, dim=24, vdim=40, size=37, mlp=dense(64)),
                  full(heads=6, kv_heads=3, dim=20, vdim=12, bias_max=30), chunked(heads=6, kv_heads=2, dim=16, vdim=64, size=100)],
                 max_positions=400)
    w = O.random_model(cfg, seed=47, rel_rows=[12, 0, 8, 0])
    ids = tokens(260, 120, 48)
    ref = oracle(cfg, w, ids)
    outs = []
    for general in (0, 1):
        eng = make_engine(cfg, w, dtype=dtype, max_tokens=256)
        eng.set_option("attn_general", general)
        slot = eng.open_sequence()
        outs.append(feed(eng, slot, ids, [200, 30, 9, 3, 2, 1, 1, 4, 1]))
        close(eng)
    for got in outs:
        assert (rel_err(got, ref)[1] < 2e-4) if dtype == torch.float32 else (rel_err(got, ref)[0] < 5e-2)
    assert rel_err(outs[0], outs[1].double().cpu())[1] < (2e-4 if dtype == torch.float32 else 0.1)


# ------------------------------------------------------------------------------------------------ other sizes
def random_config(seed):
    g = torch.Generator().manual_seed(1000 + seed)
    pick = lambda *xs: xs[int(torch.randint(0, len(xs), (1,), generator=g))]
    layers, rows = [], []
    for _ in range(pick(1, 2, 3, 4)):
        kvh = pick(1, 2, 3)
        heads = kvh * pick(1, 2, 4)
        mlp = dense(pick(0, 8, 33, 64))
        if pick(0, 1):
            layers.append(full(heads=heads, kv_heads=kvh, dim=pick(4, 9, 16, 30, 64), vdim=pick(3, 8, 20, 64), scale=pick(0.1, 0.3),
                               bias_max=pick(5, 17, 64, 200), coef=pick(0.0, 0.3, 1.0), every=pick(1, 3, 16, 64), mlp=mlp))
            rows.append(pick(*[r for r in (2, 4, 6, 10, 16) if r // 2 < layers[-1]["mixer"]["bias_max"]]))
        else:
            layers.append(chunked(heads=heads, kv_heads=kvh, dim=pick(4, 9, 16, 30, 64), vdim=pick(3, 8, 20, 64), scale=pick(0.1, 0.3),
                                  size=pick(1, 2, 7, 16, 50, 1000), mlp=mlp))
            rows.append(0)
    n = len(layers)
    loop = None
    if pick(0, 1):
        a = pick(*range(n))
        loop = (a, pick(*range(a + 1, n + 1)), pick(1, 2, 3))
    cfg = config(layers, width=pick(24, 40, 64, 100), vocab=pick(50, 77, 128), eps=pick(1e-6, 1e-5, 1e-2),
                 streams=pick(None, 1, 2, 3, 4, 6), loop=loop, embed_scale=pick(1.0, 4.0, 0.25))
    return cfg, rows


@pytest.mark.parametrize("seed", list(range(12)))
def test_configurations_drawn_at_random(seed):
    cfg, rows = random_config(seed)
    w = O.random_model(cfg, seed=50 + seed, rel_rows=rows)
    ids = tokens(70, cfg["vocab"], 60 + seed)
    ref = oracle(cfg, w, ids)
    for cuts in ([70], [50] + [1] * 20, [2] * 35, [9, 1, 30, 5]):
        eng = make_engine(cfg, w, page_size=8)
        slot = eng.open_sequence()
        assert rel_err(feed(eng, slot, ids, cuts), ref)[1] < 2e-4, (cfg, cuts)
        close(eng)


@pytest.mark.parametrize("tc", [1, 0], ids=["tcgen05", "cuda-cores"])
@pytest.mark.parametrize("name,cfg_dict", [("small", SMALL), ("odd", ODD)])
def test_bf16_engine_both_linear_paths(name, cfg_dict, tc):
    w = O.random_model(cfg_dict, seed=71, rel_rows=REL_ROWS[name])
    ids = tokens(60, cfg_dict["vocab"], 72)
    ref = oracle(cfg_dict, w, ids)
    for cuts in ([60], [40] + [1] * 20):
        eng = make_engine(cfg_dict, w, dtype=torch.bfloat16, tc=tc)
        slot = eng.open_sequence()
        assert rel_err(feed(eng, slot, ids, cuts), ref)[0] < 5e-2
        close(eng)


def test_bf16_engine_on_sizes_that_fill_tensor_core_tiles():
    cfg = config([full(heads=8, kv_heads=2, dim=64, vdim=64, scale=0.125, bias_max=128, mlp=dense(512)),
                  chunked(heads=8, kv_heads=4, dim=32, vdim=64, scale=0.17, size=128, mlp=dense(512))], width=256, vocab=512,
                 streams=2, max_positions=600)
    w = O.random_model(cfg, seed=73, rel_rows=16)
    ids = tokens(520, 512, 74)
    ref = oracle(cfg, w, ids)
    eng = make_engine(cfg, w, dtype=torch.bfloat16, max_tokens=512, max_seq_len=640)
    slot = eng.open_sequence()
    assert rel_err(feed(eng, slot, ids, [512, 1, 1, 6]), ref)[0] < 5e-2
    close(eng)


# ------------------------------------------------------------------------------------------------ entry points
def test_greedy_generation_through_stage_and_scheduler():
    """Stage.generate (byte tokenizer, ragged prefill, the step loop and the fused sampler at temperature 0) against
    greedy decoding with the oracle"""
    from asd_b200.models.lukopel import LukopelConfig
    from asd_b200.models.stage import Stage
    cfg_dict = copy.deepcopy(SMALL)
    cfg_dict["vocab"] = 256
    w = O.random_model(cfg_dict, seed=41)
    w["head"] = (w["head"].float() * 4).to(torch.bfloat16)          # spread logits: no near ties between arg-maxima
    cfg = LukopelConfig.from_dict(cfg_dict).with_shapes({k: tuple(v.shape) for k, v in w.items()})
    st = Stage("unused", "lukopel-test", config=cfg, weights=w, max_batch=3, max_model_len=128, k=0)
    assert st.get_model_info()["family"] == "lukopel"
    prompts = ["abc", "hello world, this is longer", "z"]
    texts, _, stats = st.generate(prompts, max_tokens=12, temperature=0.0)
    assert stats["decode_steps"] >= 11
    ids = [list(p.encode()) for p in prompts]
    toks = st._generate_ids(ids, 12, 0.0)[0]
    for p, t, new in zip(ids, texts, toks):
        assert st.tokenizer.decode(new) == t and len(new) == 12
        # teacher-forced on the engine's own tokens: each one is the oracle's arg-max, or within bf16 noise of it
        lg = oracle(cfg_dict, w, p + new)
        for j, tok in enumerate(new):
            row = lg[len(p) + j - 1]
            assert row[tok] >= row.max() - 0.02 * row.std(), (j, tok, int(row.argmax()))
        assert sum(int(lg[len(p) + j - 1].argmax()) == tok for j, tok in enumerate(new)) >= 10


def test_speculative_decoding_with_a_lukopel_draft_equals_plain_greedy():
    """a rejected tail is re-fed over cache rows that the draft's guesses already wrote"""
    from asd_b200.engine import LukopelEngine, SpecDecoder
    from asd_b200.models.lukopel import LukopelConfig
    tcfg = copy.deepcopy(SMALL)
    dcfg = config([chunked(heads=2, kv_heads=1, dim=8, vdim=8, size=6), full(heads=2, kv_heads=1, dim=8, vdim=8, bias_max=10)],
                  streams=2)
    wt, wd = O.random_model(tcfg, seed=43), O.random_model(dcfg, seed=44, rel_rows=4)
    wt["head"] = (wt["head"].float() * 4).to(torch.bfloat16)
    prompts = [tokens(9, 120, 45), tokens(15, 120, 46)]

    def run(with_draft):
        kw = dict(max_seqs=2, max_seq_len=96, max_tokens=64, dtype=torch.float32)     # fp32: no near ties
        mk = lambda c, w: LukopelEngine(LukopelConfig.from_dict(c).with_shapes({k: tuple(v.shape) for k, v in w.items()}),
                                        **kw).load_weights(w)
        t = mk(tcfg, wt)
        d = mk(dcfg, wd) if with_draft else None
        return SpecDecoder(t, d, 2, 3, temperature=0.0).generate(prompts, 16)[0].tolist()

    plain = run(False)
    assert run(True) == plain
    lg = oracle(tcfg, wt, prompts[0] + plain[0])
    assert sum(int(lg[len(prompts[0]) + j - 1].argmax()) == t for j, t in enumerate(plain[0])) >= 14


def write_checkpoint(path, cfg_dict, w):
    """config.json + model.safetensors (8-byte little-endian header length, JSON header, raw data)"""
    path.mkdir()
    (path / "config.json").write_text(json.dumps(cfg_dict))
    header, blobs, off = {}, [], 0
    for name, t in w.items():
        raw = t.to(torch.bfloat16).contiguous().view(torch.uint8).numpy().tobytes()
        header[name] = {"dtype": "BF16", "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hj = json.dumps(header).encode()
    with open(path / "model.safetensors", "wb") as f:
        f.write(struct.pack("<Q", len(hj)) + hj + b"".join(blobs))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_command_on_a_checkpoint_directory(tmp_path, dtype):
    """the command-line runner end to end: registry by config.json, safetensors loader (sizes that only tensor shapes
    give), page table with two requests one after the other (the second reuses the first one's slot and pages),
    portions down to one token, wanted rows only"""
    import numpy as np
    w = {k: v.to(torch.bfloat16) for k, v in O.random_model(ODD, seed=51, rel_rows=REL_ROWS["odd"]).items()}
    write_checkpoint(tmp_path / "model", ODD, w)
    a, b = tokens(41, ODD["vocab"], 52), tokens(23, ODD["vocab"], 53)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 29]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[30:32], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": a[32:33], "want": [0]}], "end": []},
             {"step": 3, "entries": [{"id": "a", "tokens": a[33:], "want": [7, 3]}], "end": ["a"]},
             {"step": 4, "entries": [{"id": "b", "tokens": b, "want": [22]}], "end": ["b"]}]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", str(tmp_path / "model"), "--dtype",
                        dtype, "--out", str(out), "--max-tokens", "48"], input="\n".join(json.dumps(x) for x in steps) + "\n",
                       capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.split("\n") if l.startswith("done")] == [f"done {i}" for i in range(5)]
    ra, rb = oracle(ODD, w, a), oracle(ODD, w, b)
    want = {0: ra[[0, 29]], 2: ra[[32]], 3: ra[[40, 36]], 4: rb[[22]]}
    assert not (out / "1.f32").exists()
    for step, ref in want.items():
        got = torch.from_numpy(np.fromfile(out / f"{step}.f32", dtype="<f4").reshape(ref.shape[0], -1).copy())
        if dtype == "float32":
            assert rel_err(got, ref)[1] < 2e-4, step
        else:
            assert rel_err(got, ref)[0] < 5e-2, step
