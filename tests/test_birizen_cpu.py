"""Host-side parts of the Birizen path that need no GPU: config parsing, the order of the layer runs, the registry,
and the oracle's own consistency (a decayed state carried across a cut, attention in the latent space)."""
import math

import pytest
import torch

import birizen_oracle as O
from pg_b200 import registry
from pg_b200.birizen import BirizenConfig
from pg_b200.ragged_engine import RotaryCfg

F64 = torch.float64


def test_config_reads_every_size_and_constant():
    cfg = O.make_config(width=48, vocab=77, eps=3e-4, loop=(1, 3, 4), layers=[
        O.layer(O.lightning(heads=3, dim=6, vdim=10, decay=[0.1, 0.5, 1.0]), None),
        O.layer(O.latent(heads=5, dim=6, rot_dim=8, vdim=4, q_rank=9, kv_rank=7, scale=0.7, base=123.0, scaling=(3.0, 50, 7.0, 0.5)),
                O.experts(n=12, top=3, groups=4, keep=2, ff=20, limit=0.75, shared_ff=28, shared_limit=3.5)),
        O.layer(O.lightning(), O.experts(shared_ff=0))])
    c = BirizenConfig.from_dict(cfg)
    assert (c.vocab, c.width, c.eps) == (77, 48, 3e-4)
    assert (c.loop.start, c.loop.stop, c.loop.times) == (1, 3, 4)
    a = c.layers[0].mixer
    assert (c.layers[0].kind, a.heads, a.dim, a.vdim, a.decay, c.layers[0].mlp) == ("lightning", 3, 6, 10, [0.1, 0.5, 1.0], None)
    b = c.layers[1].mixer
    assert (b.heads, b.dim, b.rot_dim, b.vdim, b.q_rank, b.kv_rank, b.scale) == (5, 6, 8, 4, 9, 7, 0.7)
    assert (b.rot.dims, b.rot.base, b.rot.scaling["factor"], b.rot.scaling["slow"]) == (8, 123.0, 3.0, 0.5)
    m = c.layers[1].mlp
    assert (m.experts, m.top, m.groups, m.keep, m.ff, m.limit, m.shared_ff, m.shared_limit) == (12, 3, 4, 2, 20, 0.75, 28, 3.5)
    assert c.layers[2].mlp.shared_ff == 0
    assert registry.resolve(cfg).__name__ == "BirizenEngine"
    assert "Birizen" in registry.architectures()


def test_layer_runs_follow_the_loop():
    L = [O.layer(O.lightning(), None)] * 5
    runs = lambda **kw: [(r.layer, r.loop_pass) for r in BirizenConfig.from_dict(O.make_config(L, **kw)).runs()]
    assert runs() == [(i, None) for i in range(5)]
    assert runs(loop=(1, 3, 2)) == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (3, None), (4, None)]
    assert runs(loop=(0, 5, 1)) == [(0, 0), (1, None), (2, None), (3, None), (4, None)]
    assert runs(loop=(4, 5, 3)) == [(0, None), (1, None), (2, None), (3, None), (4, 0), (4, 1), (4, 2)]
    for kw in ({}, {"loop": (1, 3, 2)}, {"loop": (0, 5, 1)}, {"loop": (4, 5, 3)}):
        assert runs(**kw) == O.layer_runs(O.make_config(L, **kw))


def test_config_rejects_what_the_design_does_not_have():
    with pytest.raises(ValueError):
        BirizenConfig.from_dict(O.make_config([{"type": "convolution", "mixer": {}, "mlp": None}]))
    with pytest.raises(ValueError):
        BirizenConfig.from_dict(O.make_config([O.layer(O.lightning(heads=3, decay=[0.5, 0.5]), None)]))
    with pytest.raises(ValueError):
        BirizenConfig.from_dict(O.make_config([O.layer(O.lightning(), O.experts(n=6, top=3, groups=3, keep=1))]))   # 2 experts stay, 3 wanted
    with pytest.raises(ValueError):
        BirizenConfig.from_dict(O.make_config([O.layer(O.lightning(), O.experts(n=7, groups=3))]))
    with pytest.raises(ValueError):
        BirizenConfig.from_dict(O.make_config([O.layer(O.lightning(), None)], loop=(0, 2, 2)))
    with pytest.raises(ValueError):
        BirizenConfig.from_dict(O.make_config([O.layer(O.lightning(), {"kind": "dense", "ff": 8})]))


def test_rotary_table_matches_the_oracle():
    for dims, base, sc in [(8, 10000.0, None), (16, 3e5, (3.0, 2048, 24.0, 2.0)), (6, 77.0, (2.5, 100, 8.0, 0.5))]:
        scd = dict(zip(("factor", "original", "fast", "slow"), sc)) if sc else None
        f, mag = RotaryCfg(dims, base, scd).table()
        f2, mag2 = O.rotary_frequencies(dims, base, scd)
        assert torch.allclose(f, f2, rtol=1e-13) and mag == pytest.approx(mag2)
    x = torch.randn(3, 2, 6, dtype=F64)
    f, mag = O.rotary_frequencies(6, 50.0)
    y = O.rotate_neighbours(x, [0, 5, 9], f, mag)
    assert torch.equal(y[0], x[0])                                   # position 0: no turn
    assert torch.allclose(y.pow(2).sum(-1), x.pow(2).sum(-1))        # a turn keeps the length of every pair


def test_oracle_state_carries_across_a_cut():
    g = torch.Generator().manual_seed(1)
    q, k, v = (torch.randn(20, 2, 5, generator=g, dtype=F64) for _ in range(3))
    whole, S = O.decayed_linear_attention(q, k, v, [0.9, 0.3])
    a, Sa = O.decayed_linear_attention(q[:7], k[:7], v[:7], [0.9, 0.3])
    b, Sb = O.decayed_linear_attention(q[7:], k[7:], v[7:], [0.9, 0.3], Sa)
    assert torch.allclose(torch.cat([a, b]), whole) and torch.allclose(Sb, S)
    # the same numbers as decayed causal attention without a softmax: o_i = sum_{j<=i} decay^(i-j) (q_i . k_j) v_j
    i, h = 11, 0
    want = sum(0.9 ** (i - j) * float(q[i, h] @ k[j, h]) * v[j, h] for j in range(i + 1))
    assert torch.allclose(whole[i, h], want)


def test_oracle_attention_in_the_latent_space_is_the_same_attention():
    """Folding the key expansion into the query and applying the value expansion after the weighted sum gives the
    oracle's per-head attention: the identity the served path rests on."""
    g = torch.Generator().manual_seed(2)
    n, H, d, r, e, kr = 9, 3, 4, 2, 5, 6
    q = torch.randn(n, H, d + r, generator=g, dtype=F64)
    c, k_rot = torch.randn(n, kr, generator=g, dtype=F64), torch.randn(n, r, generator=g, dtype=F64)
    uk, uv = torch.randn(H, d, kr, generator=g, dtype=F64), torch.randn(H, e, kr, generator=g, dtype=F64)
    sink = torch.randn(H, generator=g, dtype=F64)
    keys = torch.cat([torch.einsum("hdk,nk->nhd", uk, c), k_rot[:, None, :].expand(n, H, r)], -1)
    vals = torch.einsum("hek,nk->nhe", uv, c)
    direct = O.sink_softmax_attention(q, keys, vals, 0.4, sink)
    q_lat = torch.cat([torch.einsum("nhd,hdk->nhk", q[..., :d], uk), q[..., d:]], -1)
    shared = torch.cat([c, k_rot], -1)[:, None, :].expand(n, H, kr + r)
    lat = O.sink_softmax_attention(q_lat, shared, c[:, None, :].expand(n, H, kr), 0.4, sink)
    assert torch.allclose(torch.einsum("nhk,hek->nhe", lat, uv), direct)


def test_oracle_router_weights_and_groups():
    W = {"router": torch.zeros(4, 3), "correction": torch.tensor([-0.6, -0.9, -0.7, -3.0])}
    idx, w = O.route(torch.zeros(1, 3, dtype=F64), W, "", {"experts": 4, "top": 2, "groups": {"count": 2, "keep": 1}})
    assert idx == [[0, 1]] and torch.allclose(w, torch.tensor([[0.5, 0.5]], dtype=F64))
    idx, _ = O.route(torch.zeros(1, 3, dtype=F64), W, "", {"experts": 4, "top": 2, "groups": {"count": 2, "keep": 2}})
    assert idx == [[0, 2]]
