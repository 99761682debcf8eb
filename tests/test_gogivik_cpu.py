"""Host-side parts of the Gogivik path that need no GPU: config parsing, the registry, the rotary table, and the oracle's
own consistency (what is causal stays causal, the convolutions match torch's, rotated values turned back are an
ordinary weighted sum seen from the query's position)."""
import pytest
import torch

import gogivik_oracle as O
from pg_b200 import registry
from pg_b200.gogivik import GogivikConfig
from pg_b200.ragged_engine import RotaryCfg

F64 = torch.float64


def test_config_reads_every_size_and_constant():
    cfg = O.make_config(width=48, vocab=77, eps=3e-4, taps=3, logit_scale=2.5, layers=[
        O.layer(O.latent(heads=5, dim=6, rot_dim=8, vdim=4, q_rank=9, kv_rank=7, window=11, scale=0.7, base=123.0), 20),
        O.layer(O.attention(heads=6, kv_heads=3, dim=10, vdim=12, chunk=13, rot_dims=4, factor=3.0, scale=0.2, base=77.0), 0),
        O.layer(O.mamba2(heads=4, vdim=6, state=16, groups=2, norm_groups=3, conv=5), 32)])
    c = GogivikConfig.from_dict(cfg)
    assert (c.vocab, c.width, c.eps, c.taps, c.logit_scale) == (77, 48, 3e-4, 3, 2.5)
    a = c.layers[0].mixer
    assert (c.layers[0].kind, a.heads, a.dim, a.rot_dim, a.vdim, a.q_rank, a.kv_rank, a.scale, a.window) == \
        ("latent_attention", 5, 6, 8, 4, 9, 7, 0.7, 11)
    assert (a.rot.dims, a.rot.base, a.rot.scaling, c.layers[0].ff) == (8, 123.0, None, 20)
    b = c.layers[1].mixer
    assert (b.heads, b.kv_heads, b.dim, b.vdim, b.chunk, b.scale, b.rot_base, c.layers[1].ff) == (6, 3, 10, 12, 13, 0.2, 77.0, 0)
    assert (b.rot.dims, b.rot.base, b.rot.scaling) == (4, 77.0, {"factor": 3.0})
    s = c.layers[2].mixer
    assert (s.heads, s.vdim, s.state, s.groups, s.norm_groups, s.taps, s.inner, s.channels) == (4, 6, 16, 2, 3, 5, 24, 24 + 64)
    assert registry.resolve(cfg).__name__ == "GogivikEngine" and "Gogivik" in registry.architectures()


def test_config_rejects_what_the_design_does_not_have():
    mk = lambda layers, **kw: O.make_config(width=16, vocab=9, layers=layers, **kw)
    with pytest.raises(ValueError):
        GogivikConfig.from_dict(mk([{"type": "convolution", "mixer": {}, "mlp": None}]))
    with pytest.raises(ValueError):
        GogivikConfig.from_dict(mk([O.layer(O.attention(heads=3, kv_heads=2, dim=4, vdim=4, chunk=2), 0)]))
    with pytest.raises(ValueError):
        GogivikConfig.from_dict(mk([O.layer(O.attention(heads=2, kv_heads=2, dim=4, vdim=5, chunk=2), 0)]))   # odd values cannot turn
    with pytest.raises(ValueError):
        GogivikConfig.from_dict(mk([O.layer(O.mamba2(heads=3, vdim=4, state=4, groups=2, norm_groups=1, conv=2), 0)]))
    with pytest.raises(ValueError):
        GogivikConfig.from_dict(mk([O.layer(O.mamba2(heads=2, vdim=5, state=4, groups=1, norm_groups=4, conv=2), 0)]))
    with pytest.raises(ValueError):
        GogivikConfig.from_dict(mk([dict(O.attention(heads=2, kv_heads=1, dim=4, vdim=4, chunk=2), mlp={"kind": "moe"})]))
    with pytest.raises(ValueError):
        GogivikConfig.from_dict(mk([O.layer(O.latent(heads=2, dim=4, rot_dim=3, vdim=4, q_rank=4, kv_rank=4, window=3), 0)]))
    with pytest.raises(ValueError):
        GogivikConfig.from_dict(mk([O.layer(O.mamba2(heads=2, vdim=4, state=4, groups=1, norm_groups=1, conv=2), 0)], taps=0))


def test_rotary_table_linear_scaling_matches_the_oracle():
    for dims, base, factor in ((8, 10000.0, None), (48, 20000.0, 2.0), (2, 5.0, 7.5)):
        f, mag = RotaryCfg(dims, base, {"factor": factor} if factor else None).table()
        assert mag == 1.0 and torch.allclose(f, O.frequencies(dims, base, factor or 1.0), rtol=1e-13)


def test_oracle_convolution_is_torch_conv1d_with_left_padding():
    g = torch.Generator().manual_seed(0)
    h, w, b = torch.randn(17, 6, generator=g, dtype=F64), torch.randn(6, 4, generator=g, dtype=F64), torch.randn(6, generator=g, dtype=F64)
    ref = torch.nn.functional.conv1d(torch.nn.functional.pad(h.T[None], (3, 0)), w[:, None, :], b, groups=6)[0].T
    assert torch.allclose(O.causal_conv(h, w, b), ref, atol=1e-12)
    assert torch.allclose(O.input_conv(h, w), h + ref - b, atol=1e-12)


def test_oracle_turned_back_values_depend_on_the_distance_only():
    """Rotating value j by j and the sum by -i is a rotation of every value by j - i: shifting all positions by a
    multiple of the block size changes nothing."""
    g = torch.Generator().manual_seed(1)
    n, e, size = 12, 6, 4
    q, k, v = (torch.randn(n, d, generator=g, dtype=F64) for d in (5, 5, e))
    fv = O.frequencies(e, 50.0)

    def run(shift):
        pos = [shift + t for t in range(n)]
        o = O.masked_softmax_attention(q, k, O.rotate(v, pos, fv, "halves"), 0.5, lambda i, j: O.chunk_visible(i, j, size))
        return O.rotate(o, pos, fv, "halves", sign=-1.0)
    assert torch.allclose(run(0), run(8), atol=1e-9)
    manual = torch.zeros(e, dtype=F64)
    i, js = 6, [4, 5, 6]
    s = torch.stack([(q[i] * k[j]).sum() * 0.5 for j in js])
    p = torch.softmax(s, 0)
    for w_, j in zip(p, js):
        manual += w_ * O.rotate(v[j][None], [j - i], fv, "halves")[0]
    assert torch.allclose(run(0)[i], manual, atol=1e-12)


def test_oracle_is_causal_and_blocks_and_windows_cut_what_they_should():
    cfg = O.make_config(width=24, vocab=30, taps=3, layers=[
        O.layer(O.latent(heads=2, dim=4, rot_dim=2, vdim=4, q_rank=6, kv_rank=6, window=3), 8),
        O.layer(O.attention(heads=2, kv_heads=1, dim=4, vdim=4, chunk=4), 8),
        O.layer(O.mamba2(heads=2, vdim=4, state=4, groups=1, norm_groups=2, conv=2), 0)])
    ck = O.make_checkpoint(cfg, 2)
    toks = torch.randint(0, 30, (20,), generator=torch.Generator().manual_seed(3)).tolist()
    full = O.forward(cfg, ck, toks)
    assert torch.allclose(O.forward(cfg, ck, toks[:9]), full[:9], atol=1e-10)          # later tokens change nothing earlier
    other = list(toks)
    other[19] = (other[19] + 1) % 30
    assert torch.allclose(O.forward(cfg, ck, other)[:19], full[:19], atol=1e-10)
    # without the state-space layer the model forgets: windows, blocks and taps bound how far a token reaches
    # (per layer: 2 taps back twice, plus 2 through the window or up to 3 inside a block: 13 positions in all)
    short = dict(cfg, layers=cfg["layers"][:2])
    ck2 = {k: v for k, v in ck.items() if not k.startswith("l2.")}
    base = O.forward(short, ck2, toks)
    other = list(toks)
    other[0] = (other[0] + 1) % 30
    moved = (O.forward(short, ck2, other) - base).abs().amax(-1)
    assert float(moved[0]) > 1e-6 and float(moved[14:].max()) < 1e-12
