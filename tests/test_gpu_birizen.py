"""Birizen on the GPU against the plain float64 oracle (tests/birizen_oracle.py): every mechanism alone through the
C ABI, then whole models of several shapes through the engine, the latent cache, the state slots and the scheduler."""
import json
import math
import os

import pytest
import torch

import birizen_oracle as O
from test_gpu_ninisun import Paged, _close, _i32, _rows_close, _tokens

pytestmark = pytest.mark.gpu
F64 = torch.float64
PAGE = 64
TOL = {torch.float32: 3e-5, torch.bfloat16: 5e-2}
CT = {torch.float32: 0, torch.bfloat16: 1}


def _lib():
    from pg_b200 import _cabi as cabi
    return cabi, cabi.lib(), cabi.stream()


def _engine(cfg, seed=0, dtype=torch.float32, pool_tokens=1024, **kw):
    from pg_b200.birizen import BirizenEngine
    ck = O.make_checkpoint(cfg, seed)
    return BirizenEngine(cfg, ck, device="cuda:0", dtype=dtype, kv_pool_tokens=pool_tokens, **kw), ck


# ------------------------------------------------------------------ mechanisms alone (C ABI)
@pytest.mark.parametrize("H,dim,vdim", [(2, 8, 12), (3, 32, 32), (1, 20, 7), (2, 64, 96), (5, 128, 40), (1, 130, 16)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_lightning_recurrence_over_segments_and_slots(H, dim, vdim, dtype):
    """Three sequences in one launch (a long portion, a single token, a short portion) that start from given states
    in given slots; an unlisted slot keeps its state; the state after the step is the oracle's."""
    cabi, L, st = _lib()
    g = torch.Generator().manual_seed(7)
    lens, slots = [83, 1, 5], [2, 0, 3]
    T = sum(lens)
    nk, nv = H * dim, H * vdim
    ld = 8 + 2 * nk + nv + 3
    proj = (torch.randn(T, ld, generator=g) * 1.5).to(dtype)
    decay = torch.tensor([0.3 + 0.69 * (h + 1) / H for h in range(H)])
    state0 = torch.randn(4, H, dim, vdim, generator=g)
    state = state0.clone().cuda()
    out = torch.full((T, nv), 3.0, device="cuda")
    segs, row = [], 0
    for n, s in zip(lens, slots):
        segs += [s, row, n]
        row += n
    segs += [1, 0, 0]                                   # an empty segment (padding of a captured launch) touches nothing
    projd, dec = proj.cuda(), decay.cuda()
    rec = torch.empty(L.pg_lightning_record_floats(T, H, dim, vdim), device="cuda")
    cabi.check(L.pg_lightning_prep(rec.data_ptr(), projd.data_ptr(), ld, 8, 8 + nk, 8 + 2 * nk, T, H, dim, vdim, CT[dtype], st))
    cabi.check(L.pg_lightning_attention(out.data_ptr(), state.data_ptr(), rec.data_ptr(), dec.data_ptr(), _i32(segs).data_ptr(),
                                        4, H, dim, vdim, st))
    p64, row = proj.to(F64), 0
    for n, s in zip(lens, slots):
        sl = slice(row, row + n)
        q = O.silu(p64[sl, 8:8 + nk]).view(n, H, dim)
        k = O.silu(p64[sl, 8 + nk:8 + 2 * nk]).view(n, H, dim)
        v = O.silu(p64[sl, 8 + 2 * nk:8 + 2 * nk + nv]).view(n, H, vdim)
        o, S = O.decayed_linear_attention(q, k, v, decay.to(F64), state0[s].to(F64))
        _close(out[sl], o.reshape(n, nv), 2e-5)
        _close(state[s], S, 2e-5)
        row += n
    assert torch.equal(state[1].cpu(), state0[1])


def test_lightning_state_carries_a_first_token_far():
    """decay 1 on one head: what the first token wrote is read undiminished 500 tokens later, in one portion or cut
    into portions and single tokens; decay 0 on another: only the current token is ever seen."""
    cabi, L, st = _lib()
    H, dim, vdim, T = 2, 16, 16, 501
    nk = nv = H * dim
    proj = torch.zeros(T, 2 * nk + nv)
    proj[0, nk:nk + dim] = 4.0                          # head 0: the first token's key and value
    proj[0, 2 * nk:2 * nk + vdim] = 3.0
    proj[0, nk + dim:2 * nk] = 4.0                      # head 1 likewise, but its decay is 0
    proj[0, 2 * nk + vdim:] = 3.0
    proj[T - 1, :nk] = 2.0                              # the last token asks
    decay = torch.tensor([1.0, 0.0]).cuda()
    want_o, _ = O.decayed_linear_attention(O.silu(proj[:, :nk].to(F64)).view(T, H, dim), O.silu(proj[:, nk:2 * nk].to(F64)).view(T, H, dim),
                                           O.silu(proj[:, 2 * nk:].to(F64)).view(T, H, vdim), [1.0, 0.0])
    assert float(want_o[T - 1, 0].abs().min()) > 10 and float(want_o[T - 1, 1].abs().max()) == 0.0
    projd = proj.cuda()
    for cuts in ([T], [1, 2, 61, 64, 300, 2, 1, 69, 1]):
        assert sum(cuts) == T
        state = torch.zeros(1, H, dim, vdim, device="cuda")
        out = torch.zeros(T, nv, device="cuda")
        at = 0
        rec = torch.empty(L.pg_lightning_record_floats(T, H, dim, vdim), device="cuda")
        for n in cuts:
            cabi.check(L.pg_lightning_prep(rec.data_ptr(), projd[at:].data_ptr(), proj.shape[1], 0, nk, 2 * nk, n, H, dim, vdim, 0, st))
            cabi.check(L.pg_lightning_attention(out[at:].data_ptr(), state.data_ptr(), rec.data_ptr(), decay.data_ptr(),
                                                _i32([0, 0, n]).data_ptr(), 1, H, dim, vdim, st))
            at += n
        _close(out, want_o.reshape(T, nv), 1e-5)


@pytest.mark.parametrize("q_rank,kv_rank,rot_dim,scaling", [(12, 14, 4, None), (96, 64, 32, (4.0, 64, 16.0, 1.0)),
                                                            (7, 5, 2, (2.0, 16, 3.0, 0.7)), (40, 24, 0, None)])
def test_latent_norms_rotated_key_and_cache_append(q_rank, kv_rank, rot_dim, scaling):
    cabi, L, st = _lib()
    g = torch.Generator().manual_seed(11)
    T = 6
    positions, slots = [70, 71, 0, 1, 63, 300], [1, 1, 0, 0, 0, 2]
    ldp = (kv_rank + rot_dim + 7) // 8 * 8
    pg = Paged([64, 72, 301], ldp, 1)
    ld = 5 + q_rank + 3 + kv_rank + rot_dim + 2
    dq0, dkv0 = 5, 5 + q_rank + 3
    proj = torch.randn(T, ld, generator=g) * 2
    wq, wkv = torch.randn(q_rank, generator=g), torch.randn(kv_rank, generator=g)
    freq, mag, f64 = None, 1.0, None
    if rot_dim:
        sc = dict(zip(("factor", "original", "fast", "slow"), scaling)) if scaling else None
        f64, mag = O.rotary_frequencies(rot_dim, 777.0, sc)
        from pg_b200.ragged_engine import RotaryCfg
        f_eng, mag_eng = RotaryCfg(rot_dim, 777.0, sc).table()
        assert torch.allclose(f_eng, f64, rtol=1e-12) and abs(mag_eng - mag) < 1e-12
        freq = f_eng.to(torch.float32).cuda()
    cq = torch.empty(T, q_rank, device="cuda")
    dev = [t.cuda() for t in (proj, wq, wkv)]
    cabi.check(L.pg_latent_prep(cq.data_ptr(), dev[0].data_ptr(), ld, dq0, q_rank, dev[1].data_ptr(), dkv0, kv_rank,
                                dev[2].data_ptr(), rot_dim, None if freq is None else freq.data_ptr(), mag, 1e-4,
                                pg.k.data_ptr(), ldp, pg.table.data_ptr(), pg.max_pages, PAGE, _i32(slots).data_ptr(),
                                _i32(positions).data_ptr(), T, cabi.PG_F32, st))
    p64 = proj.to(F64)
    _close(cq, O.rms_norm(p64[:, dq0:dq0 + q_rank], wq, 1e-4), 2e-6)
    want = [O.rms_norm(p64[:, dkv0:dkv0 + kv_rank], wkv, 1e-4)]
    if rot_dim:
        want.append(O.rotate_neighbours(p64[:, dkv0 + kv_rank:dkv0 + kv_rank + rot_dim], positions, f64, mag))
    want.append(torch.zeros(T, ldp - kv_rank - rot_dim, dtype=F64))
    rows = [pg.rows(s, [p])[0] for s, p in zip(slots, positions)]
    _close(pg.k.view(-1, ldp)[rows], torch.cat(want, -1), 2e-6)
    untouched = torch.ones(pg.k.shape[0] * PAGE, dtype=torch.bool)
    untouched[rows] = False
    assert bool((pg.k.view(-1, ldp).cpu()[untouched] == 7.0).all())


def test_rotated_query_columns():
    cabi, L, st = _lib()
    g = torch.Generator().manual_seed(12)
    T, H, dim, rot, kvr = 5, 3, 6, 4, 10
    q = torch.randn(T, H * (dim + rot), generator=g)
    dst = torch.full((T, H * (kvr + rot)), 5.0, device="cuda")
    f64, mag = O.rotary_frequencies(rot, 50.0, {"factor": 3.0, "original": 32, "fast": 4.0, "slow": 1.0})
    positions = [0, 1, 64, 1000, 7]
    fr, qd = f64.to(torch.float32).cuda(), q.cuda()
    cabi.check(L.pg_rotary_cols(dst.data_ptr(), H * (kvr + rot), kvr, kvr + rot, qd.data_ptr(), H * (dim + rot), dim, dim + rot,
                                H, rot, fr.data_ptr(), mag, _i32(positions).data_ptr(), T, cabi.PG_F32, st))
    want = O.rotate_neighbours(q.to(F64).view(T, H, dim + rot)[..., dim:], positions, f64, mag)
    got = dst.view(T, H, kvr + rot)
    _close(got[..., kvr:], want, 3e-6)
    assert bool((got[..., :kvr] == 5.0).all())


@pytest.mark.parametrize("M", [1, 9, 17, 150])         # weight-streaming rows, then tiles
@pytest.mark.parametrize("H,N,K,gated", [(3, 10, 14, True), (4, 96, 64, False), (2, 70, 33, True), (5, 8, 128, True)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_per_head_product_with_gate(M, H, N, K, gated, dtype):
    cabi, L, st = _lib()
    g = torch.Generator().manual_seed(13)
    a_hs, o_hs = K + 3, N + 2
    A = torch.randn(M, H * a_hs + 1, generator=g).to(dtype)
    W = (torch.randn(H, N, K, generator=g) / math.sqrt(K)).to(dtype)
    gate = torch.randn(M, H * N + 4, generator=g).to(dtype)
    out = torch.zeros(M, H * o_hs, dtype=dtype, device="cuda")
    dev = [t.cuda() for t in (A, W, gate)]
    cabi.check(L.pg_head_gemm(out.data_ptr(), H * o_hs, o_hs, dev[0].data_ptr(), A.shape[1], a_hs, dev[1].data_ptr(),
                              dev[2].data_ptr() if gated else None, gate.shape[1], M, H, N, K, CT[dtype], st))
    a64 = A.to(F64)[:, :H * a_hs].view(M, H, a_hs)[..., :K]
    want = torch.einsum("mhk,hnk->mhn", a64, W.to(F64))
    if gated:
        want = want * O.sigmoid(gate.to(F64)[:, :H * N].view(M, H, N))
    _close(out.view(M, H, o_hs)[..., :N], want, 2e-6 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize("M", [64, 150, 300])
@pytest.mark.parametrize("H,N,K,gated", [(3, 16, 24, True), (4, 96, 64, False), (8, 192, 128, False), (5, 128, 192, True),
                                         (2, 40, 72, True)])
def test_per_head_product_on_the_tensor_cores(M, H, N, K, gated):
    """All heads in one launch of the grouped tcgen05 kernel: operand columns and output columns of a head inside the
    token rows (head strides wider than the sizes used), row counts off the 128-row tile, K off the 64-column box."""
    cabi, L, st = _lib()
    dtype = torch.bfloat16
    g = torch.Generator().manual_seed(37)
    a_hs, o_hs = K + 8, N + 16
    A = torch.randn(M, H * a_hs, generator=g).to(dtype)
    W = (torch.randn(H, N, K, generator=g) / math.sqrt(K)).to(dtype)
    gate = torch.randn(M, H * N + 8, generator=g).to(dtype)
    out = torch.zeros(M, H * o_hs, dtype=dtype, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    dev = [t.cuda() for t in (A, W, gate)]
    cabi.check(L.pg_head_gemm_ex(out.data_ptr(), H * o_hs, o_hs, dev[0].data_ptr(), H * a_hs, a_hs, dev[1].data_ptr(),
                                 dev[2].data_ptr() if gated else None, H * N + 8, M, H, N, K, 2, err.data_ptr(), CT[dtype], st))
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    want = torch.einsum("mhk,hnk->mhn", A.to(F64).view(M, H, a_hs)[..., :K], W.to(F64))
    if gated:
        want = want * O.sigmoid(gate.to(F64)[:, :H * N].view(M, H, N))
    _close(out.view(M, H, o_hs)[..., :N], want, 1e-2)
    assert float(out.view(M, H, o_hs)[..., N:].abs().max()) == 0          # nothing beside a head's columns is written


def _latent_attention_case(H, kvr, rot, lens, new, dtype=torch.float32, tower=None, sink_value=None, seed=0):
    """Sequences of lens[s] cached latent rows [c | k_rot] of which the last new[s] are this step's queries, through
    the ragged attention with ONE key/value head whose value is a prefix of its key row; returns (got, want)."""
    cabi, L, st = _lib()
    g = torch.Generator().manual_seed(seed)
    dim, ldp = kvr + rot, (kvr + rot + 7) // 8 * 8
    pg = Paged(lens, ldp, 1, dtype)
    scale = 0.3
    sink = torch.randn(H, generator=g) if sink_value is None else torch.full((H,), float(sink_value))
    qs, want, slots, positions = [], [], [], []
    for s, (n, m) in enumerate(zip(lens, new)):
        q, k = torch.randn(n, H, dim, generator=g), torch.randn(n, 1, dim, generator=g)
        if tower is not None:                     # one key whose score stands far out for the last query
            j = tower(n - 1)
            if 0 <= j < n:
                k[j, 0] = 30.0 * q[n - 1, 0] / scale / dim
                k[j, 0, :kvr] += 6.0
        if dtype != torch.float32:
            q, k = q.to(dtype).float(), k.to(dtype).float()
        pad = torch.zeros(n, ldp - dim)
        pg.fill(s, torch.cat([k[:, 0], pad], -1), torch.zeros(n, 1))
        o = O.sink_softmax_attention(q.to(F64), k.to(F64).expand(n, H, dim), k.to(F64)[..., :kvr].expand(n, H, kvr), scale,
                                     sink.to(F64))
        qs.append(q[n - m:].reshape(m, H * dim))
        want.append(o[n - m:].reshape(m, H * kvr))
        slots += [s] * m
        positions += list(range(n - m, n))
    q_all = torch.cat(qs).to(dtype).cuda()
    T = q_all.shape[0]
    out = torch.zeros(T, H * kvr, dtype=dtype, device="cuda")
    ws = torch.empty(1 << 20, device="cuda")
    sk = sink.cuda()
    cabi.check(L.pg_attention_ragged_sink(out.data_ptr(), H * kvr, q_all.data_ptr(), H * dim, None, 0, 0, pg.k.data_ptr(), ldp,
                                          pg.k.data_ptr(), ldp, pg.table.data_ptr(), pg.max_pages, PAGE, _i32(slots).data_ptr(),
                                          _i32(positions).data_ptr(), T, H, 1, dim, kvr, scale, 0, 0, None, 0, None,
                                          sk.data_ptr(), 1.0, ws.data_ptr(), ws.numel(), CT[dtype], st))
    return out, torch.cat(want)


@pytest.mark.parametrize("H,kvr,rot", [(4, 32, 8), (3, 14, 4), (2, 96, 32), (8, 64, 16), (1, 260, 4), (6, 40, 0), (16, 256, 64),
                                       (4, 512, 64), (12, 128, 32)])
@pytest.mark.parametrize("new", [[1, 1, 1], [40, 3, 150]])     # decoded tokens (key slices), prompt portions
def test_latent_space_attention_with_sink(H, kvr, rot, new):
    got, want = _latent_attention_case(H, kvr, rot, [300, 70, 150], new)
    _rows_close(got, want, 1e-5)


@pytest.mark.parametrize("H,kvr,rot", [(4, 64, 64), (2, 192, 64), (8, 128, 0)])
@pytest.mark.parametrize("tower", [None, 0, 63, 64, 200])
def test_latent_space_attention_on_the_tensor_cores(H, kvr, rot, tower):
    """Prompt portions (query tiles of up to 128 consecutive tokens of one sequence) through the tcgen05 kernel: value
    rows that are a prefix of the key rows of one pool, the sink in the denominator; one far key that stands out."""
    cabi, L, st = _lib()
    dtype, dim, scale = torch.bfloat16, kvr + rot, 0.3
    assert L.pg_attention_ragged_tc_ok(dim, kvr, PAGE, H * dim, H * kvr, 8, CT[dtype])
    g = torch.Generator().manual_seed(29)
    lens, new = [300, 70, 150], [170, 3, 150]
    pg = Paged(lens, dim, 1, dtype)
    sink = torch.randn(H, generator=g)
    qs, want, tiles, row = [], [], [], 0
    for s, (n, m) in enumerate(zip(lens, new)):
        q, k = torch.randn(n, H, dim, generator=g), torch.randn(n, 1, dim, generator=g)
        if tower is not None and tower < n:
            k[tower, 0] = 30.0 * q[n - 1, 0] / scale / dim
        q, k = q.to(dtype).float(), k.to(dtype).float()
        pg.fill(s, k[:, 0], torch.zeros(n, 1))
        o = O.sink_softmax_attention(q.to(F64), k.to(F64).expand(n, H, dim), k.to(F64)[..., :kvr].expand(n, H, kvr), scale,
                                     sink.to(F64))
        qs.append(q[n - m:].reshape(m, H * dim))
        want.append(o[n - m:].reshape(m, H * kvr))
        for t0 in range(0, m, 128):
            tiles += [row + t0, min(128, m - t0), s, n - m + t0]
        row += m
    q_all = torch.cat(qs).to(dtype).cuda()
    T = q_all.shape[0]
    out = torch.zeros(T, H * kvr, dtype=dtype, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    sk = sink.cuda()
    cabi.check(L.pg_attention_ragged_tc_sink(out.data_ptr(), H * kvr, q_all.data_ptr(), H * dim, None, 0, 0, pg.k.data_ptr(), dim,
                                             pg.k.data_ptr(), dim, pg.k.shape[0] * PAGE, pg.table.data_ptr(), pg.max_pages, PAGE,
                                             _i32(tiles).data_ptr(), len(tiles) // 4, T, H, 1, dim, kvr, scale, 0, 0, None, 0,
                                             None, sk.data_ptr(), 1.0, err.data_ptr(), CT[dtype], st))
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    _rows_close(out, torch.cat(want), 2e-2)


@pytest.mark.parametrize("where", [0, 1, 63, 64, 65, 127, 128, 700, 1398, 1399])
@pytest.mark.parametrize("new", [1, 2, 130])
def test_one_far_key_among_many(where, new):
    """A single key at a chosen place (first tokens, both sides of page borders, far back, the token itself) carries
    nearly all the weight of the last query: leaving it out, or reading a neighbour instead, changes the row."""
    got, want = _latent_attention_case(4, 32, 8, [1400], [new], tower=lambda last: where)
    _rows_close(got, want, 1e-5)
    assert float(want[-1].abs().max()) > 2.0


def test_sink_takes_weight_and_counts_once():
    """A large sink leaves almost nothing for the keys; -inf-like sinks give the plain softmax.  With key slices
    (a single decoded token over a long sequence) the sink must join the merged denominator once, not per slice."""
    for n in (5, 2000):
        big, _ = _latent_attention_case(2, 16, 4, [n], [1], sink_value=30.0)
        assert float(big.abs().max()) < 1e-6
        got, want = _latent_attention_case(2, 16, 4, [n], [1], sink_value=2.0)
        _rows_close(got, want, 1e-5)
        none, want0 = _latent_attention_case(2, 16, 4, [n], [1], sink_value=-80.0)
        _rows_close(none, want0, 1e-5)
        assert float((want - want0).abs().max()) > 1e-4


@pytest.mark.parametrize("E,top,groups,keep", [(6, 2, 3, 2), (8, 2, 2, 1), (8, 3, 8, 4), (5, 1, 1, 1), (12, 4, 3, 3),
                                               (64, 6, 8, 3), (4, 4, 2, 2)])
@pytest.mark.parametrize("D", [40, 256])
def test_grouped_sigmoid_router(E, top, groups, keep, D):
    cabi, L, st = _lib()
    g = torch.Generator().manual_seed(17)
    T = 50
    h = torch.randn(T, D + 8, generator=g)
    wr = torch.randn(E, D, generator=g) * 3 / math.sqrt(D)
    corr = torch.randn(E, generator=g) * 0.8 - 1.0      # choice scores on both sides of zero
    idx = torch.zeros(T * top, dtype=torch.int32, device="cuda")
    wts = torch.zeros(T * top, device="cuda")
    dev = [t.cuda() for t in (h, wr, corr)]
    cabi.check(L.pg_moe_route_grouped(idx.data_ptr(), wts.data_ptr(), dev[0].data_ptr(), D + 8, dev[1].data_ptr(),
                                      dev[2].data_ptr(), T, D, E, top, groups, keep, cabi.PG_F32, st))
    W = {"router": wr, "correction": corr}
    want_idx, want_w = O.route(h[:, :D].to(F64), W, "", {"experts": E, "top": top, "groups": {"count": groups, "keep": keep}})
    assert idx.view(T, top).tolist() == want_idx
    _close(wts.view(T, top), want_w, 1e-5)
    assert torch.allclose(wts.view(T, top).sum(-1).cpu(), torch.ones(T), atol=1e-5)


def test_masked_groups_lose_to_negative_choices():
    """All choice scores negative: an expert of a kept group still beats every expert of a dropped group (those count
    as minus infinity, not as zero)."""
    cabi, L, st = _lib()
    E, D = 4, 8
    h = torch.zeros(1, D)
    wr = torch.zeros(E, D)
    corr = torch.tensor([-0.6, -0.9, -0.7, -3.0])         # s = 0.5: choices -0.1, -0.4, -0.2, -2.5; group sums -0.5, -2.7
    idx = torch.zeros(2, dtype=torch.int32, device="cuda")
    wts = torch.zeros(2, device="cuda")
    dev = [t.cuda() for t in (h, wr, corr)]
    cabi.check(L.pg_moe_route_grouped(idx.data_ptr(), wts.data_ptr(), dev[0].data_ptr(), D, dev[1].data_ptr(), dev[2].data_ptr(),
                                      1, D, E, 2, 2, 1, cabi.PG_F32, st))
    assert idx.tolist() == [0, 1]
    assert torch.allclose(wts.cpu(), torch.tensor([0.5, 0.5]))


@pytest.mark.parametrize("dtype,impl", [(torch.float32, 1), (torch.bfloat16, 1), (torch.bfloat16, 2)])
def test_clamped_glu_experts_grouped(dtype, impl):
    """Both expert products with the clamped pairing in the first one's epilogue, through the fp32-FMA kernel and the
    tensor-core kernel, and the same pairing as a kernel of its own; values on both sides of the limits."""
    cabi, L, st = _lib()
    g = torch.Generator().manual_seed(19)
    E, D, ff, limit = 3, 64, 40, 0.9
    counts = [70, 0, 33]
    P = sum(counts)
    a = torch.randn(P, D, generator=g).to(dtype)
    gu = (torch.randn(E, 2 * ff, D, generator=g) * 2.0 / math.sqrt(D)).to(dtype)
    offsets = torch.tensor([0, 70, 70, 103], dtype=torch.int32).cuda()
    out = torch.zeros(P, ff, dtype=dtype, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    ad, gud = a.cuda(), gu.cuda()
    cabi.check(L.pg_moe_gemm_act(out.data_ptr(), ff, ad.data_ptr(), D, None, gud.data_ptr(), offsets.data_ptr(), P, E, ff, D,
                                 cabi.GLU_CLAMPED, limit, impl, err.data_ptr(), CT[dtype], st))
    assert int(err.item()) == 0
    want, row = [], 0
    for e, n in enumerate(counts):
        z = a[row:row + n].to(F64) @ gu[e].to(F64).T
        gg, uu = z[:, :ff].clamp(max=limit), z[:, ff:].clamp(-limit, limit)
        want.append(gg * O.sigmoid(1.702 * gg) * (uu + 1))
        row += n
    want = torch.cat(want)
    assert float((want.abs() > 0).float().mean()) > 0.9
    _close(out, want, 1e-5 if dtype == torch.float32 else 2e-2)
    z = (torch.randn(9, 2 * ff, generator=g) * 2).to(dtype)
    o2 = torch.zeros(9, ff, dtype=dtype, device="cuda")
    zd = z.cuda()
    cabi.check(L.pg_glu_clamped(o2.data_ptr(), zd.data_ptr(), 9, ff, limit, 1.702, CT[dtype], st))
    gg, uu = z.to(F64)[:, :ff].clamp(max=limit), z.to(F64)[:, ff:].clamp(-limit, limit)
    _close(o2, gg * O.sigmoid(1.702 * gg) * (uu + 1), 1e-6 if dtype == torch.float32 else 1e-2)


def test_weighted_expert_sum_as_an_output():
    cabi, L, st = _lib()
    g = torch.Generator().manual_seed(23)
    T, D, top = 7, 20, 3
    y = torch.randn(T * top, D + 4, generator=g)
    sh = torch.randn(T, D, generator=g)
    pos = torch.randperm(T * top, generator=g).to(torch.int32)
    wts = torch.rand(T * top, generator=g)
    out = torch.zeros(T, D + 2, device="cuda")
    dev = [t.cuda() for t in (y, pos, wts, sh)]
    for shared in (True, False):
        cabi.check(L.pg_moe_combine_out(out.data_ptr(), D + 2, dev[0].data_ptr(), D + 4, dev[1].data_ptr(), dev[2].data_ptr(),
                                        dev[3].data_ptr() if shared else None, D, T, D, top, cabi.PG_F32, st))
        want = (wts.view(T, top, 1).to(F64) * y.to(F64)[pos.long(), :D].view(T, top, D)).sum(1)
        _close(out[:, :D], want + (sh.to(F64) if shared else 0), 1e-6)


def test_two_fp32_rows_side_by_side_in_the_model_dtype():
    cabi, L, st = _lib()
    a, b = torch.randn(5, 12).cuda(), torch.randn(5, 12).cuda()
    for dtype in (torch.float32, torch.bfloat16):
        out = torch.zeros(5, 24, dtype=dtype, device="cuda")
        cabi.check(L.pg_concat_cast(out.data_ptr(), a.data_ptr(), b.data_ptr(), 5, 12, CT[dtype], st))
        assert torch.equal(out, torch.cat([a, b], -1).to(dtype))


# ------------------------------------------------------------------ whole models
SC = (4.0, 64, 16.0, 1.0)
CONFIGS = {
    # a looped block of three layers (two passes) after a layer of its own, as many groups kept as there are
    "small": O.make_config(loop=(1, 4, 2), layers=[
        O.layer(O.lightning(), O.experts()), O.layer(O.lightning(heads=3, dim=8, vdim=8), O.experts(groups=2, keep=2)),
        O.layer(O.latent(scaling=SC), O.experts()), O.layer(O.lightning(), None), O.layer(O.latent(heads=2), O.experts(top=1, shared_ff=0))]),
    # no loop, latent attention first, layers without a feed-forward, one expert group
    "no_loop": O.make_config(width=64, vocab=80, eps=1e-3, layers=[
        O.layer(O.latent(heads=4, dim=16, rot_dim=16, vdim=16, q_rank=24, kv_rank=32), None),
        O.layer(O.lightning(heads=4, dim=16, vdim=16), O.experts(n=4, top=2, groups=1, keep=1, ff=24)),
        O.layer(O.latent(heads=1, dim=8, rot_dim=2, vdim=24, q_rank=8, kv_rank=8, scaling=(8.0, 32, 4.0, 2.0)), None)]),
    # the whole model is the loop, three passes; sizes off every vector width; six heads over one latent
    "odd": O.make_config(width=52, vocab=67, loop=(0, 2, 3), layers=[
        O.layer(O.latent(heads=6, dim=5, rot_dim=6, vdim=7, q_rank=9, kv_rank=11), O.experts(n=9, top=3, groups=3, keep=1, ff=7, shared_ff=5)),
        O.layer(O.lightning(heads=5, dim=9, vdim=7, decay=[1.0, 0.0, 0.9, 0.5, 0.999]), O.experts(n=5, top=5, groups=5, keep=5, ff=12))]),
    # head sizes of real models; a loop of one layer, once; the loop at the end
    "wide": O.make_config(width=128, vocab=120, loop=(2, 3, 1), layers=[
        O.layer(O.lightning(heads=2, dim=128, vdim=64), O.experts(n=8, top=2, groups=4, keep=2, ff=64, shared_ff=32)),
        O.layer(O.latent(heads=8, dim=64, rot_dim=32, vdim=64, q_rank=96, kv_rank=128, scale=0.09, scaling=SC), None),
        O.layer(O.lightning(heads=1, dim=64, vdim=128), O.experts(n=16, top=4, groups=4, keep=3, ff=32, shared_ff=64))]),
    # a width at which the 16-bit run crosses the tensor-core GEMM kernels
    "mid": O.make_config(width=384, vocab=600, loop=(0, 2, 2), layers=[
        O.layer(O.lightning(heads=6, dim=32, vdim=64), O.experts(n=8, top=2, groups=2, keep=1, ff=128, shared_ff=128)),
        O.layer(O.latent(heads=4, dim=64, rot_dim=32, vdim=96, q_rank=128, kv_rank=96, scale=0.1, scaling=(2.0, 512, 32.0, 1.0)),
                O.experts(n=8, top=2, groups=2, keep=1, ff=128, shared_ff=128)),
        O.layer(O.lightning(heads=6, dim=32, vdim=64), None)]),
}
NO_ROUTER = {"plain": O.make_config(width=96, vocab=90, loop=(1, 3, 2), layers=[
    O.layer(O.lightning(heads=3, dim=16, vdim=32), None), O.layer(O.latent(heads=4, dim=16, rot_dim=8, vdim=24, q_rank=40, kv_rank=48), None),
    O.layer(O.lightning(heads=2, dim=24, vdim=24), None)]),
    # latent sizes that the tensor-core attention takes (16-bit prompt portions of 48 tokens and more)
    "tensor_core_sizes": O.make_config(width=128, vocab=90, loop=(0, 1, 2), layers=[
        O.layer(O.latent(heads=4, dim=32, rot_dim=64, vdim=32, q_rank=64, kv_rank=64, scale=0.1, scaling=SC), None),
        O.layer(O.lightning(heads=2, dim=32, vdim=32), None)])}
_ORACLE_CACHE = {}


def _cfg(name):
    return CONFIGS.get(name) or NO_ROUTER[name]


def _oracle(name, n, seed=0):
    key = (name, n, seed)
    if key not in _ORACLE_CACHE:
        cfg = _cfg(name)
        ck = O.make_checkpoint(cfg, 0)
        toks = _tokens(n, cfg["vocab"], 100 + seed)
        sink = []
        _ORACLE_CACHE[key] = (toks, O.forward(cfg, ck, toks, sink), sink)
    return _ORACLE_CACHE[key]


def _stray(name, dtype):
    """16-bit runs: a router's close call, decided the other way, changes a token's row and, through the decayed
    state and the attention, later ones; models without a router keep the tight bound."""
    if dtype == torch.float32:
        return 0.0
    return 0.25 if name in CONFIGS else 0.02


def _tol(name, dtype):
    return 0.1 if (dtype == torch.bfloat16 and name in CONFIGS) else TOL[dtype]


@pytest.mark.parametrize("name", list(CONFIGS) + list(NO_ROUTER))
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_whole_prompt_logits_and_every_layer_run(name, dtype):
    n = 150
    toks, want, layers = _oracle(name, n)
    eng, _ = _engine(_cfg(name), dtype=dtype)
    b = eng.new_batcher(slots=2)
    b.admit("a")
    sink = []
    got = b.run_entries([("a", toks, list(range(n)))], layer_sink=sink)
    eng.check_errors(sync=True)
    assert len(sink) == len(layers) == len(O.layer_runs(_cfg(name)))
    for x, ref in zip(sink, layers):
        _rows_close(x, ref, _tol(name, dtype), _stray(name, dtype))
    _rows_close(got, want, _tol(name, dtype) * 2, _stray(name, dtype))
    b.close()


@pytest.mark.parametrize("name", list(CONFIGS) + list(NO_ROUTER))
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_prefill_then_token_by_token_and_portions(name, dtype):
    n = 150
    toks, want, _ = _oracle(name, n)
    eng, _ = _engine(_cfg(name), dtype=dtype, pool_tokens=448)
    b = eng.new_batcher(slots=2)
    b.admit("a")
    rows = [b.run_entries([("a", toks[:100], [99])])]
    rows += [b.run_entries([("a", [t], [0])]) for t in toks[100:]]
    _rows_close(torch.cat(rows), want[99:], _tol(name, dtype) * 2, _stray(name, dtype))
    b.finish("a")
    b.admit("b")          # the slot and the pages of "a" again; portions down to two tokens and single ones
    at, got = 0, []
    for size in [2, 37, 2, 1, 31, 13, 1, 1, 2, 50, 3, 7]:
        got.append(b.run_entries([("b", toks[at:at + size], list(range(size)))]))
        at += size
    assert at == n
    _rows_close(torch.cat(got), want, _tol(name, dtype) * 2, _stray(name, dtype))
    eng.check_errors(sync=True)
    b.close()


@pytest.mark.parametrize("name", ["small", "odd", "wide"])
def test_unequal_requests_in_one_batch_with_slots_and_pages_used_again(name):
    cfg = _cfg(name)
    lens = {"a": 131, "b": 23, "c": 97, "d": 150, "e": 70}
    ref = {k: _oracle(name, n, seed=i) for i, (k, n) in enumerate(lens.items())}
    eng, _ = _engine(cfg, pool_tokens=6 * PAGE)          # a pool that forces pages to be handed on
    b = eng.new_batcher(slots=3)
    fed = {k: 0 for k in lens}
    got = {k: [] for k in lens}
    plan = [
        [("a", 64), ("b", 21), ("c", 2)], [("a", 3), ("b", 1), ("c", 90)], [("a", 1), ("b", 1), ("c", 1)],
        [("a", 60), ("c", 1)], [("c", 1), ("a", 1)], [("c", 2)], [("a", 2), ("d", 65)], [("d", 2), ("e", 64)],
        [("d", 80), ("e", 1)], [("e", 5), ("d", 1)], [("d", 2)]]
    for step in plan:
        entries = []
        for k, n in step:
            if k not in b.slot_of:
                b.admit(k)
            entries.append((k, ref[k][0][fed[k]:fed[k] + n], list(range(n))))
            fed[k] += n
        out = b.run_entries(entries)
        at = 0
        for k, n in step:
            got[k].append(out[at:at + n])
            at += n
        for k, _ in step:
            if fed[k] == lens[k] and k in b.slot_of:
                b.finish(k)
    eng.check_errors(sync=True)
    for k in lens:
        assert fed[k] == lens[k]
        _rows_close(torch.cat(got[k]), ref[k][1], TOL[torch.float32] * 2)
    b.close()
    assert eng.pages_in_use() == 0


def test_long_decoding_through_pages_and_state():
    name, n = "small", 330
    toks, want, _ = _oracle(name, n)
    for dtype in (torch.float32, torch.bfloat16):
        eng, _ = _engine(_cfg(name), dtype=dtype)
        b = eng.new_batcher(slots=1)
        b.admit("a")
        rows = [b.run_entries([("a", toks[:5], list(range(5)))])]
        rows += [b.run_entries([("a", [t], [0])]) for t in toks[5:]]
        _rows_close(torch.cat(rows), want, _tol(name, dtype) * 2, _stray(name, dtype))
        b.close()


def test_every_pass_of_the_loop_keeps_its_own_cache_and_state():
    eng, _ = _engine(_cfg("small"))
    runs = O.layer_runs(_cfg("small"))
    assert len(runs) == 8 and [r for r, _ in runs] == [0, 1, 2, 3, 1, 2, 3, 4]
    assert sorted(eng.c_pools) == [2, 5, 7]                       # runs of the latent layers
    b = eng.new_batcher(slots=2)
    assert sorted(b.kv.state.layers) == [0, 1, 3, 4, 6]           # runs of the lightning layers
    assert b.kv.state.layers[1].shape == (2, 3, 8, 8) and b.kv.state.layers[0].shape == (2, 2, 8, 12)
    b.admit("a")
    b.run_entries([("a", _tokens(70, 61, 1), [])])
    s = b.kv.state.layers
    assert not torch.equal(s[1][0], s[4][0]) and float(s[4][0].abs().max()) > 0 and float(s[1][1].abs().max()) == 0
    assert not torch.equal(eng.c_pools[2], eng.c_pools[5])
    b.finish("a")
    b.admit("again")                                              # the slot is handed on with a zero state
    assert all(float(t[0].abs().max()) == 0 for t in s.values())
    b.close()


def test_greedy_generation_through_the_scheduler():
    name = "small"
    cfg = _cfg(name)
    ck = O.make_checkpoint(cfg, 0)
    eng, _ = _engine(cfg)
    prompts = [_tokens(n, cfg["vocab"], 40 + n) for n in (3, 70, 18)]
    b = eng.new_batcher(slots=2, token_budget=32)
    rids = [b.submit(p, max_new_tokens=6) for p in prompts]
    done = b.run()
    for rid, p in zip(rids, prompts):
        seq = list(p)
        for _ in range(6):                                     # the oracle's own greedy loop
            seq.append(int(O.forward(cfg, ck, seq)[-1].argmax()))
        assert done[rid].tokens == seq[len(p):]
    b.close()
    assert eng.pages_in_use() == 0
    runs = []
    for _ in range(2):
        b = eng.new_batcher(slots=2, token_budget=32, do_sample=True, temperature=0.9, top_p=0.8, seed=5)
        rids = [b.submit(p, max_new_tokens=5) for p in prompts[:2]]
        done = b.run()
        runs.append([done[r].tokens for r in rids])
        b.close()
    assert runs[0] == runs[1] and all(0 <= t < cfg["vocab"] for seq in runs[0] for t in seq)


def test_model_folder_through_the_registry_and_command_line(tmp_path):
    import subprocess
    import sys
    import numpy as np
    from pg_b200.checkpoint import write_safetensors
    from pg_b200.registry import load_engine
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = _cfg("odd")
    ck = O.make_checkpoint(cfg, 3)
    model = tmp_path / "model"
    model.mkdir()
    with open(model / "config.json", "w") as f:
        json.dump(cfg, f)
    write_safetensors(str(model / "model.safetensors"), {k: v.to(torch.bfloat16) for k, v in ck.items()})
    eng = load_engine(str(model), device="cuda:0", dtype=torch.float32, kv_pool_tokens=256)
    assert type(eng).__name__ == "BirizenEngine"
    toks = _tokens(40, cfg["vocab"], 9)
    b = eng.new_batcher(slots=1)
    b.admit(0)
    _rows_close(b.run_entries([(0, toks, [39, 0])]), O.forward(cfg, ck, toks)[[39, 0]], 1e-4)
    b.close()
    more = dict(ck)
    more["l0.mix.extra"] = torch.zeros(3)
    with pytest.warns(UserWarning):
        type(eng)(cfg, more, device="cuda:0", dtype=torch.float32, kv_pool_tokens=64)
    with pytest.raises(ValueError):
        type(eng)(cfg, more, device="cuda:0", dtype=torch.float32, kv_pool_tokens=64, strict=True)
    with pytest.raises(KeyError):
        type(eng)(cfg, {k: v for k, v in ck.items() if k != "l0.mix.sink"}, device="cuda:0", dtype=torch.float32, kv_pool_tokens=64)
    seq = {k: _tokens(n, cfg["vocab"], 60 + n) for k, n in (("a", 22), ("b", 5), ("c", 70))}
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": seq["a"][:20], "want": [19]}, {"id": "b", "tokens": seq["b"], "want": [0, 4]}],
         "end": ["b"]},
        {"step": 1, "entries": [{"id": "a", "tokens": seq["a"][20:21], "want": []}], "end": []},
        {"step": 2, "entries": [{"id": "c", "tokens": seq["c"], "want": [69]}, {"id": "a", "tokens": seq["a"][21:], "want": [0]}],
         "end": ["a", "c"]}]
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", str(model), "--dtype", "float32",
                        "--out", str(out), "--max-tokens", "192"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [ln for ln in r.stdout.splitlines() if ln.startswith("done")] == ["done 0", "done 1", "done 2"]
    ref = {k: O.forward(cfg, ck, v) for k, v in seq.items()}
    got0 = torch.from_numpy(np.fromfile(out / "0.f32", dtype="<f4").reshape(3, cfg["vocab"]))
    _rows_close(got0, torch.stack([ref["a"][19], ref["b"][0], ref["b"][4]]), 1e-4)
    got2 = torch.from_numpy(np.fromfile(out / "2.f32", dtype="<f4").reshape(2, cfg["vocab"]))
    _rows_close(got2, torch.stack([ref["c"][69], ref["a"][21]]), 1e-4)
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "generate"), "--model", str(model), "--dtype", "float32",
                        "--prompt-ids", ",".join(map(str, seq["b"])), "--max-new-tokens", "4", "--max-tokens", "256",
                        "--slots", "2"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [json.loads(ln) for ln in r.stdout.splitlines() if ln.startswith("{")]
    s = list(seq["b"])
    for _ in range(4):
        s.append(int(O.forward(cfg, ck, s)[-1].argmax()))
    assert lines[0] == {"request": 0, "tokens": s[len(seq["b"]):]}
