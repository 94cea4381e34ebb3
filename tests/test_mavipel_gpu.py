"""GPU: the Mavipel engine against the plain restatement in oracle/mavipel_oracle.py (fp64, whole sequences, no cache).
Every test makes its own small configuration and random weights.  The fp32 engine is held to 2e-4 of the logits'
spread, which a single key missed or double-counted among hundreds, a window off by one, a lost state or convolution
input, a left-out sink or a stale page all exceed; the bf16 engine to what its roundings allow."""
import copy
import json
import os
import struct
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import mavipel_oracle as O  # noqa: E402


# ------------------------------------------------------------------------------------------------ configurations
def dense(ff=48):
    return {"kind": "dense", "ff": ff} if ff else None


def moe(experts=5, top=2, ff=40, shared=24):
    f = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared:
        f["shared"] = {"ff": shared}
    return f


def delta(heads=4, kv_heads=2, dim=24, vdim=16, conv=3, decay_rank=8, gate_rank=12, mlp=None):
    return {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv,
                                               "decay_rank": decay_rank, "gate_rank": gate_rank}, "mlp": mlp}


def par(heads=6, kv_heads=2, dim=16, vdim=24, size=9, base=1000.0, rot_dims=8, scale=0.3, softcap=12.0, left_scale=0.9,
        r_heads=3, r_dim=16, r_rank=8, right_scale=1.2, mlp=None, mask=True):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "rot": {"base": base, "dims": rot_dims},
            "scale": scale, "softcap": softcap}
    if mask:
        left["mask"] = {"size": size}
    return {"type": "parallel", "mixer": {"left": left, "left_scale": left_scale, "right_scale": right_scale,
                                          "right": {"heads": r_heads, "dim": r_dim, "decay_rank": r_rank}}, "mlp": mlp}


def config(layers, width=96, vocab=120, eps=1e-5, groups=3, loop=None):
    d = {"architecture": "Mavipel", "width": width, "vocab": vocab, "norm": {"eps": eps, "groups": groups}, "layers": layers}
    if loop:
        d["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return d


# both mixers, every feed-forward kind, a repeated span in the middle
SMALL = config([par(mlp=dense(72)), delta(mlp=moe()), delta(heads=2, kv_heads=2, dim=16, vdim=40, conv=4, decay_rank=4,
                                                            gate_rank=8), par(heads=2, kv_heads=1, dim=24, vdim=8, size=5,
                                                                              rot_dims=24, r_heads=1, r_dim=40, mlp=moe(3, 1, 32, 0))],
               loop=(1, 3, 2))
# sizes that are multiples of nothing; the span starts at the first layer and runs three times; one key head per query
# head and one for all; rotation of nothing and of the whole head; one norm group; a single tap; an uncapped, unmasked layer
ODD = config([delta(heads=3, kv_heads=1, dim=10, vdim=7, conv=1, decay_rank=5, gate_rank=3, mlp=dense(50)),
              par(heads=5, kv_heads=5, dim=10, vdim=6, size=4, rot_dims=10, softcap=0.0, r_heads=2, r_dim=22, r_rank=3,
                  mlp=moe(7, 3, 9, 11)),
              par(heads=6, kv_heads=1, dim=12, vdim=34, rot_dims=0, scale=0.5, r_heads=1, r_dim=6, r_rank=1, mask=False),
              delta(heads=1, kv_heads=1, dim=40, vdim=66, conv=5, decay_rank=3, gate_rank=1, mlp=moe(2, 2, 21, 0))],
             width=72, vocab=101, eps=1e-3, groups=1, loop=(0, 2, 3))
PLAIN = config([delta(mlp=dense(32)), par()], groups=2)       # no repeated span at all
WHOLE = config([par(mlp=moe()), delta()], groups=4, loop=(0, 2, 1))   # a span that is the whole model and runs once


def make_engine(cfg_dict, w, dtype=torch.float32, max_tokens=64, max_seq_len=512, page_size=16, num_pages=None,
                max_seqs=4, ring=1, tc=1):
    from asd_b200.engine import MavipelEngine
    from asd_b200.models.mavipel import MavipelConfig
    cfg = MavipelConfig.from_dict(cfg_dict).with_shapes({k: tuple(v.shape) for k, v in w.items()})
    eng = MavipelEngine(cfg, max_seqs=max_seqs, max_seq_len=max_seq_len, max_tokens=max_tokens, page_size=page_size,
                        dtype=dtype, dynamic_pages=True, num_pages=num_pages, ring=ring)
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
    return O.forward(cfg_dict, w, ids, layers_out=streams)


# ------------------------------------------------------------------------------------------------ whole prompts
@pytest.mark.parametrize("cfg_dict", [SMALL, ODD, PLAIN, WHOLE], ids=["small", "odd", "plain", "whole"])
def test_whole_prompt_logits_and_every_layer_execution(cfg_dict):
    w = O.random_model(cfg_dict, seed=1)
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
        assert (st[i] - streams[i]).abs().max() <= 2e-4 * streams[i].abs().max(), f"stream leaving execution {i}"
    assert rel_err(got, ref)[1] < 2e-4
    close(eng)


# ------------------------------------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("groups", [1, 2, 5])
def test_embedding_norm_groups_and_final_norm_alone(groups):
    """no layers: logits = head . norm(norm(embed)); the number of groups changes the answer"""
    cfg = config([], width=40, vocab=50, groups=groups)
    w = O.random_model(cfg, seed=3)
    w["embed"] = (w["embed"].float() * torch.linspace(0.2, 3.0, 40)).to(torch.bfloat16)    # parts of unequal size
    ids = tokens(20, 50, 4)
    ref = oracle(cfg, w, ids)
    assert rel_err(run_whole(cfg, w, ids), ref)[1] < 1e-4
    other = oracle(config([], width=40, vocab=50, groups=1 if groups > 1 else 2), w, ids)
    assert rel_err(other.float(), ref)[1] > 1e-2


def silence_mixer(cfg, w, i=0):
    for k in list(w):
        if k.startswith(f"l{i}.mix.") and k.rsplit(".", 1)[-1] == "o":
            w[k] = torch.zeros_like(w[k])


def test_gelu_feed_forward_alone():
    cfg = config([delta(mlp=dense(56))])
    w = O.random_model(cfg, seed=5, scale=2.0)
    silence_mixer(cfg, w)
    ids = tokens(33, 120, 6)
    assert rel_err(run_whole(cfg, w, ids), oracle(cfg, w, ids))[1] < 2e-4


@pytest.mark.parametrize("experts,top,ff,shared", [(5, 2, 40, 24), (4, 1, 17, 0), (9, 9, 8, 5), (40, 3, 12, 0), (2, 1, 64, 64)])
def test_routed_experts_alone(experts, top, ff, shared):
    """gates are the softmax over the chosen logits only; the router's bias decides who is chosen"""
    cfg = config([delta(mlp=moe(experts, top, ff, shared))])
    w = O.random_model(cfg, seed=7, scale=2.0)
    silence_mixer(cfg, w)
    w["l0.mlp.router.b"] = torch.linspace(-1.5, 1.5, experts).to(torch.bfloat16)
    ids = tokens(50, 120, 8)
    ref = oracle(cfg, w, ids)
    assert rel_err(run_whole(cfg, w, ids), ref)[1] < 2e-4
    if top < experts:
        w2 = dict(w)
        w2["l0.mlp.router.b"] = torch.zeros(experts, dtype=torch.bfloat16)
        assert rel_err(oracle(cfg, w2, ids).float(), ref)[1] > 1e-2


@pytest.mark.parametrize("entry", [delta(heads=3, kv_heads=3, dim=20, vdim=12, conv=2), delta(heads=4, kv_heads=1, dim=64, vdim=40, conv=4),
                                   delta(heads=2, kv_heads=2, dim=130, vdim=33, conv=1, decay_rank=1, gate_rank=2),
                                   delta(heads=1, kv_heads=1, dim=300, vdim=20, conv=7, decay_rank=2)], ids=["a", "b", "c", "wide"])
def test_gated_delta_rule_alone(entry):
    cfg = config([entry])
    w = O.random_model(cfg, seed=9)
    ids = tokens(70, 120, 10)
    ref = oracle(cfg, w, ids)
    assert rel_err(run_whole(cfg, w, ids, max_tokens=128), ref)[1] < 2e-4
    for cuts in ([1] * 70, [2] * 35, [33, 3, 1, 1, 2]):
        eng = make_engine(cfg, w)
        slot = eng.open_sequence()
        assert rel_err(feed(eng, slot, ids, cuts), ref)[1] < 2e-4, cuts
        close(eng)


def silence(w, side):
    for k in list(w):
        if f".mix.{side}.o" in k:
            w[k] = torch.zeros_like(w[k])


@pytest.mark.parametrize("r_heads,r_dim,rank", [(3, 16, 8), (1, 72, 1), (2, 130, 5), (5, 8, 2)])
def test_generalised_delta_rule_alone(r_heads, r_dim, rank):
    cfg = config([par(r_heads=r_heads, r_dim=r_dim, r_rank=rank)])
    w = O.random_model(cfg, seed=11)
    silence(w, "left")
    ids = tokens(70, 120, 12)
    ref = oracle(cfg, w, ids)
    assert rel_err(run_whole(cfg, w, ids, max_tokens=128), ref)[1] < 2e-4
    for cuts in ([1] * 70, [2] * 35, [40, 1, 1, 5]):
        eng = make_engine(cfg, w)
        slot = eng.open_sequence()
        assert rel_err(feed(eng, slot, ids, cuts), ref)[1] < 2e-4, cuts
        close(eng)


def test_window_attention_alone_sink_cap_and_head_mix():
    cfg = config([par(heads=4, kv_heads=2, dim=16, vdim=12, size=11, softcap=3.0, scale=0.6)])
    w = O.random_model(cfg, seed=13)
    silence(w, "right")
    w["l0.mix.left.sink"] = torch.tensor([3.0, -2.0, 0.5, 6.0]).to(torch.bfloat16)
    ids = tokens(64, 120, 14)
    ref = oracle(cfg, w, ids)
    assert rel_err(run_whole(cfg, w, ids), ref)[1] < 2e-4
    # a left-out sink, an unmixed score, a missing cap, a cap after the mix and unrotated keys are all far outside
    w2 = dict(w)
    w2["l0.mix.left.sink"] = torch.full((4,), -1e4)
    assert rel_err(oracle(cfg, w2, ids).float(), ref)[1] > 1e-2
    w2 = dict(w)
    w2["l0.mix.left.talk"] = torch.eye(4)
    assert rel_err(oracle(cfg, w2, ids).float(), ref)[1] > 1e-2
    for change in ({"softcap": 0.0}, {"rot": {"base": 1e30, "dims": 8}}):
        c2 = copy.deepcopy(cfg)
        c2["layers"][0]["mixer"]["left"].update(change)
        assert rel_err(oracle(c2, w, ids).float(), ref)[1] > 1e-2, change


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
def test_many_heads_and_large_value_heads(dtype):
    """twenty query heads (more than sixteen warps a CTA), value heads of 200, keys of 136"""
    cfg = config([par(heads=20, kv_heads=4, dim=16, vdim=16, size=30, rot_dims=16),
                  par(heads=2, kv_heads=1, dim=136, vdim=200, size=50, rot_dims=64, scale=0.05)])
    w = O.random_model(cfg, seed=15)
    ids = tokens(80, 120, 16)
    ref = oracle(cfg, w, ids)
    for cuts in ([80], [60] + [1] * 20, [7] * 12):
        eng = make_engine(cfg, w, dtype=dtype, max_tokens=128)
        slot = eng.open_sequence()
        got = feed(eng, slot, ids, cuts)
        assert (rel_err(got, ref)[1] < 2e-4) if dtype == torch.float32 else (rel_err(got, ref)[0] < 5e-2)
        close(eng)


def test_pass_vectors_of_a_repeated_span():
    """the same layer three times; each pass adds its own vector first"""
    cfg = config([delta(mlp=dense(32))], loop=(0, 1, 3))
    w = O.random_model(cfg, seed=17)
    ids = tokens(30, 120, 18)
    ref = oracle(cfg, w, ids)
    assert rel_err(run_whole(cfg, w, ids), ref)[1] < 2e-4
    w2 = dict(w)
    w2["loop.step"] = w["loop.step"].flip(0)
    assert rel_err(oracle(cfg, w2, ids).float(), ref)[1] > 1e-2


# ------------------------------------------------------------------------------------------------ cache and state
@pytest.mark.parametrize("cfg_dict", [SMALL, ODD], ids=["small", "odd"])
@pytest.mark.parametrize("page_size", [4, 16])
def test_prefill_then_decode_and_portions(cfg_dict, page_size):
    w = O.random_model(cfg_dict, seed=19)
    ids = tokens(61, cfg_dict["vocab"], 20)
    ref = oracle(cfg_dict, w, ids)
    for cuts in ([1] * 61, [40] + [1] * 21, [2] * 30, [3, 17, 2, 1, 1, 5, 2, 30], [16, 16, 16], [15, 17, 1, 16]):
        eng = make_engine(cfg_dict, w, page_size=page_size)
        slot = eng.open_sequence()
        assert rel_err(feed(eng, slot, ids, cuts), ref)[1] < 2e-4, cuts
        close(eng)


def test_forward_larger_than_the_engine_step_is_cut_inside():
    w = O.random_model(SMALL, seed=21)
    ids = tokens(100, 120, 22)
    assert rel_err(run_whole(SMALL, w, ids, max_tokens=24), oracle(SMALL, w, ids))[1] < 2e-4


def test_batch_of_unequal_requests_equals_each_alone():
    w = O.random_model(SMALL, seed=23)
    seqs = [tokens(n, 120, 20 + n) for n in (31, 5, 1, 18)]
    refs = [oracle(SMALL, w, s) for s in seqs]
    eng = make_engine(SMALL, w, max_tokens=32)
    slots = [eng.open_sequence() for _ in seqs]
    first = [12, 5, 1, 2]
    for sl, s in zip(slots, seqs):
        eng.reserve(sl, len(s))
    a = eng.forward_ragged([(sl, 0, s[:f], list(range(f))) for sl, s, f in zip(slots, seqs, first)])
    b = eng.forward_ragged([(sl, f, s[f:], list(range(len(s) - f))) for sl, s, f in zip(slots, seqs, first) if len(s) > f])
    oa = ob = 0
    for s, f, ref in zip(seqs, first, refs):
        got = a[oa:oa + f]
        oa += f
        if len(s) > f:
            got = torch.cat([got, b[ob:ob + len(s) - f]], 0)
            ob += len(s) - f
        assert rel_err(got, ref)[1] < 2e-4
    close(eng)


def test_pages_slots_and_state_freed_and_used_again():
    """a pool with room for one request at a time: the second request gets the first one's slot, pages, convolution
    inputs and recurrent state with the old contents still in them"""
    w = O.random_model(SMALL, seed=25)
    eng = make_engine(SMALL, w, page_size=4, num_pages=12, max_seqs=1, max_seq_len=48)
    for seed, n in ((30, 44), (31, 47), (32, 9), (33, 48), (34, 1), (35, 2)):
        ids = tokens(n, 120, seed)
        ref = oracle(SMALL, w, ids)
        slot = eng.open_sequence()
        assert slot == 0
        assert rel_err(feed(eng, slot, ids, [7, 1, 1, 13, 2]), ref)[1] < 2e-4
        eng.close_sequence(slot)
        assert eng.pages.pages_in_use() == 0
    from asd_b200._lib import AsdError
    slot = eng.open_sequence()
    with pytest.raises(AsdError):
        eng.reserve(slot, 49)
    close(eng)


def test_refeeding_recent_positions_finds_their_state():
    """rings of states and of convolution inputs: after 30 tokens the last three are taken back and other tokens
    follow, as a verification step does after a rejected tail"""
    w = O.random_model(SMALL, seed=27)
    ids = tokens(30, 120, 28)
    new_tail = tokens(9, 120, 29)
    eng = make_engine(SMALL, w, ring=4)
    slot = eng.open_sequence()
    feed(eng, slot, ids, [11, 1, 6])
    got = feed(eng, slot, new_tail, [4, 1], start=27)
    ref = oracle(SMALL, w, ids[:27] + new_tail)
    assert rel_err(got, ref[27:])[1] < 2e-4
    close(eng)


def test_long_decoding_keeps_the_recurrent_states_and_passes_the_window():
    """slow decays: what the first tokens wrote is still in both states after hundreds of single-token steps"""
    cfg = config([delta(heads=2, kv_heads=1, dim=24, vdim=16), par(size=20)])
    w = O.random_model(cfg, seed=31)
    w["l0.mix.dt_bias"] = torch.full_like(w["l0.mix.dt_bias"], -7.0)
    w["l0.mix.a2"] = w["l0.mix.a2"] * 0.1
    w["l1.mix.right.w0"] = torch.full_like(w["l1.mix.right.w0"], -6.0)
    w["l1.mix.right.a.b"] = torch.full_like(w["l1.mix.right.a.b"], -4.0)
    ids = tokens(260, 120, 32)
    ref = oracle(cfg, w, ids)
    cut = copy.deepcopy(ids)
    cut[0] = (cut[0] + 1) % 120
    assert rel_err(oracle(cfg, w, cut)[-1:].float(), ref[-1:])[1] > 1e-3      # the first token still matters
    eng = make_engine(cfg, w, page_size=8)
    slot = eng.open_sequence()
    assert rel_err(feed(eng, slot, ids, [5] + [1] * 255), ref)[1] < 2e-4
    close(eng)


# ------------------------------------------------------------------------------------------------ edges of the window
def plant_pair(cfg, w, key_tok, query_tok, boost=60.0):
    """Makes the first layer's queries of ``query_tok`` point, before their norm, along the unrotated key coordinates
    of ``key_tok`` in every head: after the norms this one score stands out wherever the key is visible."""
    m, eps, groups = cfg["layers"][0]["mixer"]["left"], cfg["norm"]["eps"], cfg["norm"]["groups"]
    H, G, dk, rd = m["heads"], m["kv_heads"], m["dim"], m["rot"]["dims"]
    f = lambda t: t.double()
    first = lambda tok: O.group_norm(O.group_norm(f(w["embed"][tok]), f(w["embed.norm"]), groups, eps), f(w["l0.norm1"]), groups, eps)
    hk, hq = first(key_tok), first(query_tok)
    k = (f(w["l0.mix.left.k"]) @ hk + f(w["l0.mix.left.k.b"])).reshape(G, dk)
    q = f(w["l0.mix.left.q"]).reshape(H, dk, -1).clone()
    for h in range(H):
        kk = k[h // (H // G), rd:]
        q[h, rd:] += boost * torch.outer(kk / kk.norm(), hq) / (hq @ hq)
    w["l0.mix.left.q"] = q.reshape(H * dk, -1).to(torch.bfloat16)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
@pytest.mark.parametrize("size,page_size", [(9, 16), (16, 16), (33, 4), (150, 16), (129, 8), (32, 32), (1, 8)])
def test_window_edges_with_standout_keys(size, page_size, dtype):
    """a key that outweighs everything else sits exactly size - 1 positions back (the last one visible) for one query
    and exactly size back (the first one hidden) for another; in a prompt, in portions and while decoding"""
    cfg = config([par(heads=4, kv_heads=2, dim=48, vdim=16, size=size, rot_dims=8, scale=0.25, softcap=40.0)])
    w = O.random_model(cfg, seed=33)
    silence(w, "right")
    w["l0.mix.left.talk"] = (torch.eye(4) + 0.1 * torch.randn(4, 4, generator=torch.Generator().manual_seed(1))).to(torch.bfloat16)
    V = cfg["vocab"]
    n = size + 2 * page_size + 70
    ids = [t % (V - 8) for t in tokens(n, V, 34)]
    base = 2 * page_size
    at_in, at_out = [], []
    plan = ((base - 1, base - 1 + size - 1, at_in), (base + 8, base + 8 + size, at_out),
            (base + 21, base + 21 + size - 1, at_in), (base + 30, base + 30 + size, at_out))
    for i, (a, qpos, where) in enumerate(plan):
        key_tok, query_tok = V - 1 - 2 * i, V - 2 - 2 * i          # every pair has tokens of its own
        plant_pair(cfg, w, key_tok, query_tok)
        ids[a], ids[qpos] = key_tok, query_tok
        where.append(qpos)
    ref = oracle(cfg, w, ids)
    # the oracle itself says that these places see an off-by-one of the window
    for dsize, places in ((-1, at_in), (1, at_out)):
        if size + dsize < 1:
            continue
        c2 = copy.deepcopy(cfg)
        c2["layers"][0]["mixer"]["left"]["mask"] = {"size": size + dsize}
        other = oracle(c2, w, ids)
        for p in places:
            assert rel_err(other[p:p + 1].float(), ref[p:p + 1])[1] > 0.3, (dsize, p)
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


def test_far_key_among_hundreds_without_a_mask_and_first_tokens():
    """no mask: attention sees everything before it; a standout key 600 positions back (the sequence's first token)
    decides the answer, in one prompt, in portions and while decoding"""
    cfg = config([par(heads=4, kv_heads=2, dim=48, vdim=16, rot_dims=8, scale=0.25, softcap=40.0, mask=False)])
    w = O.random_model(cfg, seed=35)
    silence(w, "right")
    ids = [t % 110 for t in tokens(700, 120, 36)]
    plant_pair(cfg, w, 119, 118)
    ids[0], ids[600], ids[655] = 119, 118, 118
    ref = oracle(cfg, w, ids)
    gone = oracle(cfg, w, [5] + ids[1:])
    assert rel_err(gone[600:601].float(), ref[600:601])[1] > 0.3
    for cuts in ([700], [650] + [1] * 50, [37] * 18):
        eng = make_engine(cfg, w, max_tokens=1024, max_seq_len=1024)
        slot = eng.open_sequence()
        assert rel_err(feed(eng, slot, ids, cuts), ref)[1] < 1e-3
        close(eng)


def test_both_window_attention_kernels_agree():
    """bf16 cache rows: the tensor-core kernel (weights as two bf16 terms) and the CUDA-core kernel read the same cache
    and the same rounded queries, so they differ by fp32 roundings only; both stay within bf16's reach of the oracle.
    Every value size the tensor-core kernel takes, one and several query heads per key/value head, windows shorter and
    longer than a key tile, prompts, portions that end inside a query tile and single tokens"""
    for heads, kv_heads, dim, vdim, size in ((4, 4, 32, 16, 100), (6, 2, 16, 32, 37), (8, 1, 64, 128, 130), (16, 4, 48, 64, 1000),
                                             (3, 1, 80, 32, 7), (32, 8, 32, 32, 90), (24, 3, 16, 64, 40), (18, 9, 16, 16, 500),
                                             (20, 1, 48, 32, 33)):       # more than 16 heads: two CTAs share a query tile
        cfg = config([par(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, size=size, rot_dims=16, scale=0.3, softcap=15.0)])
        w = O.random_model(cfg, seed=55)
        w["l0.mix.left.sink"] = torch.linspace(-2.0, 4.0, heads).to(torch.bfloat16)
        ids = tokens(330, 120, 56)
        ref = oracle(cfg, w, ids)
        for cuts in ([330], [200, 64, 9, 1, 1, 2, 53], [300] + [1] * 30, [17] * 20):
            got = []
            for mma in (1, 0):
                eng = make_engine(cfg, w, dtype=torch.bfloat16, max_tokens=512, max_seq_len=512, page_size=8)
                eng.set_option("attn_mma", mma)
                slot = eng.open_sequence()
                got.append(feed(eng, slot, ids, cuts))
                close(eng)
                assert rel_err(got[-1], ref)[0] < 5e-2, (heads, kv_heads, cuts, mma)
            assert rel_err(got[0], got[1].cpu())[0] < 2e-3, (heads, kv_heads, cuts)


def test_single_token_steps_with_key_shares_over_several_ctas():
    """a long window and few sequences: single-token steps (and portions of two) cut the key tiles into shares for
    several CTAs and merge them, with the sink entering once, after the merge; two sequences of unequal length"""
    cfg = config([par(heads=4, kv_heads=2, dim=32, vdim=40, size=800, rot_dims=16, scale=0.3)])
    w = O.random_model(cfg, seed=47)
    w["l0.mix.left.sink"] = torch.tensor([4.0, -1.0, 0.0, 2.0]).to(torch.bfloat16)
    a, b = tokens(900, 120, 48), tokens(300, 120, 49)
    ra, rb = oracle(cfg, w, a), oracle(cfg, w, b)
    for dtype in (torch.float32, torch.bfloat16):
        eng = make_engine(cfg, w, dtype=dtype, max_tokens=1024, max_seq_len=1024)
        sa, sb = eng.open_sequence(), eng.open_sequence()
        eng.reserve(sa, 900), eng.reserve(sb, 300)
        eng.forward_ragged([(sa, 0, a[:870], []), (sb, 0, b[:270], [])])
        ga, gb = [], []
        for i in range(15):
            n = 2
            out = eng.forward_ragged([(sa, 870 + n * i, a[870 + n * i:870 + n * (i + 1)], list(range(n))),
                                      (sb, 270 + n * i, b[270 + n * i:270 + n * (i + 1)], list(range(n)))])
            ga.append(out[:n]), gb.append(out[n:])
        for got, ref in ((torch.cat(ga), ra[870:]), (torch.cat(gb), rb[270:])):
            assert (rel_err(got, ref)[1] < 2e-4) if dtype == torch.float32 else (rel_err(got, ref)[0] < 5e-2)
        close(eng)


def random_config(seed):
    """layers in any order and number with sizes drawn at random (multiples of 16 and of nothing), a span anywhere"""
    g = torch.Generator().manual_seed(seed)
    pick = lambda xs: xs[int(torch.randint(0, len(xs), (1,), generator=g))]
    n = pick([2, 3, 4, 5])
    width = pick([48, 64, 80, 120, 128])
    layers = []
    for _ in range(n):
        mlp = pick([None, dense(pick([24, 64, 100])), moe(pick([2, 4, 8, 11]), pick([1, 2]), pick([16, 40, 64]), pick([0, 32, 50]))])
        if pick([True, False]):
            kv = pick([1, 2, 3])
            layers.append(delta(heads=kv * pick([1, 2, 4]), kv_heads=kv, dim=pick([8, 16, 48, 72, 128]), vdim=pick([8, 16, 32, 40, 64]),
                                conv=pick([1, 2, 4, 5]), decay_rank=pick([1, 4, 12]), gate_rank=pick([2, 8, 24]), mlp=mlp))
        else:
            kv = pick([1, 2, 4])
            dim = pick([8, 16, 32, 48, 128])
            layers.append(par(heads=kv * pick([1, 2, 4]), kv_heads=kv, dim=dim, vdim=pick([8, 16, 32, 64, 128, 20]),
                              size=pick([1, 5, 16, 33, 64, 300]), base=pick([100.0, 3e4, 5e5]), rot_dims=pick([dim, dim // 2, 4, 0]),
                              scale=pick([0.09, 0.2]), softcap=pick([0.0, 5.0, 30.0]), left_scale=pick([1.0, 0.7]),
                              r_heads=pick([1, 2, 4]), r_dim=pick([8, 16, 40, 64]), r_rank=pick([1, 6, 16]),
                              right_scale=pick([1.0, 1.4]), mlp=mlp, mask=pick([True, True, True, False])))
    loop = None
    if pick([True, True, False]):
        a = pick(list(range(n)))
        loop = (a, pick(list(range(a + 1, n + 1))), pick([1, 2, 3]))
    return config(layers, width=width, vocab=pick([50, 96, 257]), eps=pick([1e-5, 1e-6]),
                  groups=pick([g_ for g_ in (1, 2, 4, 8) if width % g_ == 0]), loop=loop)


@pytest.mark.parametrize("seed", list(range(12)))
def test_configurations_drawn_at_random(seed):
    """what a checkpoint's config.json may say, drawn at random: whole prompt, prompt then single tokens, portions"""
    cfg = random_config(100 + seed)
    w = O.random_model(cfg, seed=200 + seed)
    ids = tokens(75, cfg["vocab"], 300 + seed)
    ref = oracle(cfg, w, ids)
    for dtype in (torch.float32, torch.bfloat16):
        for cuts in ([75], [50] + [1] * 25, [37, 2, 3, 1, 1, 14, 2]):
            eng = make_engine(cfg, w, dtype=dtype, max_tokens=128, page_size=8)
            slot = eng.open_sequence()
            got = feed(eng, slot, ids, cuts)
            if dtype == torch.float32:
                assert rel_err(got, ref)[1] < 3e-4, (cfg, cuts)
            else:
                assert rel_err(got, ref)[0] < 8e-2, (cfg, cuts)
            close(eng)


# ------------------------------------------------------------------------------------------------ bf16 engine
@pytest.mark.parametrize("tc", [1, 0], ids=["tcgen05", "cuda-cores"])
@pytest.mark.parametrize("cfg_dict", [SMALL, ODD], ids=["small", "odd"])
def test_bf16_engine_both_linear_paths(cfg_dict, tc):
    w = O.random_model(cfg_dict, seed=37)
    ids = tokens(90, cfg_dict["vocab"], 38)
    ref = oracle(cfg_dict, w, ids)
    for cuts in ([90], [50] + [1] * 40, [7] * 13):
        eng = make_engine(cfg_dict, w, dtype=torch.bfloat16, max_tokens=128, tc=tc)
        slot = eng.open_sequence()
        got = feed(eng, slot, ids, cuts).double().cpu()
        # a router choice between two near-equal logits may fall the other way after bf16 roundings and move that
        # position by more than rounding does: the bulk of the positions is held tighter than the whole
        rows = (got - ref).norm(dim=-1) / ref.norm(dim=-1)
        assert rows.median() < 3e-2 and rel_err(got, ref)[0] < 8e-2
        close(eng)


def test_bf16_engine_on_sizes_that_fill_tensor_core_tiles():
    """multiples of 64: every projection and the expert layers take the tcgen05 kernels; 300 tokens take the
    tensor-bound CTA-pair GEMM"""
    cfg = config([delta(heads=4, kv_heads=2, dim=64, vdim=64, conv=4, decay_rank=16, gate_rank=16, mlp=moe(8, 2, 128, 128)),
                  par(heads=4, kv_heads=2, dim=64, vdim=64, size=37, rot_dims=32, scale=0.125, r_heads=2, r_dim=64, r_rank=16,
                      mlp=dense(256))], width=256, vocab=512, groups=2, loop=(0, 2, 2))
    w = O.random_model(cfg, seed=39)
    ids = tokens(300, 512, 40)
    ref = oracle(cfg, w, ids)
    for cuts in ([300], [280] + [1] * 20):
        eng = make_engine(cfg, w, dtype=torch.bfloat16, max_tokens=512)
        slot = eng.open_sequence()
        assert rel_err(feed(eng, slot, ids, cuts), ref)[0] < 5e-2
        close(eng)


# ------------------------------------------------------------------------------------------------ entry points
def test_greedy_generation_through_stage_and_scheduler():
    """Stage.generate (byte tokenizer, ragged prefill, the step loop and the fused sampler at temperature 0) against
    greedy decoding with the oracle"""
    from asd_b200.models.mavipel import MavipelConfig
    from asd_b200.models.stage import Stage
    cfg_dict = copy.deepcopy(SMALL)
    cfg_dict["vocab"] = 256
    w = O.random_model(cfg_dict, seed=41)
    w["head"] = (w["head"].float() * 4).to(torch.bfloat16)          # spread logits: no near ties between arg-maxima
    cfg = MavipelConfig.from_dict(cfg_dict).with_shapes({k: tuple(v.shape) for k, v in w.items()})
    st = Stage("unused", "mavipel-test", config=cfg, weights=w, max_batch=3, max_model_len=128, k=0)
    assert st.get_model_info()["family"] == "mavipel"
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


def test_speculative_decoding_with_a_mavipel_draft_equals_plain_greedy():
    """draft and target both carry recurrent state and convolution inputs; a rejected tail is re-fed from the rings"""
    from asd_b200.engine import MavipelEngine, SpecDecoder
    from asd_b200.models.mavipel import MavipelConfig
    tcfg = copy.deepcopy(SMALL)
    dcfg = config([delta(heads=1, kv_heads=1, dim=16, vdim=8), par(heads=2, kv_heads=1, dim=8, vdim=8, size=6, r_heads=1, r_dim=8)])
    wt, wd = O.random_model(tcfg, seed=43), O.random_model(dcfg, seed=44)
    wt["head"] = (wt["head"].float() * 4).to(torch.bfloat16)
    prompts = [tokens(9, 120, 45), tokens(15, 120, 46)]

    def run(with_draft):
        kw = dict(max_seqs=2, max_seq_len=96, max_tokens=64, dtype=torch.float32, ring=6)     # fp32: no near ties
        mk = lambda c, w: MavipelEngine(MavipelConfig.from_dict(c).with_shapes({k: tuple(v.shape) for k, v in w.items()}),
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
    cfg_dict = copy.deepcopy(cfg_dict)
    for e in cfg_dict["layers"]:          # a checkpoint's tensor shapes give the inner sizes, not its config.json
        for m in (e["mixer"], e["mixer"].get("right", {})):
            m.pop("decay_rank", None)
            m.pop("gate_rank", None)
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
    give), page table with two requests one after the other (the second reuses the first one's slot, pages and state),
    portions down to one token, wanted rows only"""
    import numpy as np
    w = {k: v.to(torch.bfloat16) for k, v in O.random_model(ODD, seed=51).items()}
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
