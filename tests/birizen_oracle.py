"""Plain float64 restatement of the Birizen design: one function per mechanism, whole sequences, no caches, no
batching, no code shared with the served path.  Slow on purpose: loops over tokens and heads where that is clearest.

Shapes: a sequence is [n, ...]; weights are [out, in] and applied as x @ W.T.
"""
import math

import torch

F64 = torch.float64


# ------------------------------------------------------------------ elementary pieces
def sigmoid(z):
    return 1.0 / (1.0 + torch.exp(-z))


def silu(z):
    return z * sigmoid(z)


def rms_norm(x, w, eps):
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w.to(F64)


def lin(x, w):
    return x @ w.to(F64).T


# ------------------------------------------------------------------ rotary positions (pairs of neighbours, YaRN)
def rotary_frequencies(dims, base, scaling=None):
    """(f [dims / 2], magnitude).  scaling = dict(factor, original, fast, slow): pairs that turn fewer than `slow`
    times over `original` positions are slowed by `factor`, those that turn more than `fast` times are kept, a
    linear ramp lies between; cos and sin are multiplied by 0.1 ln(factor) + 1."""
    i = torch.arange(dims // 2, dtype=F64)
    f = float(base) ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, orig = float(scaling["factor"]), float(scaling["original"])

    def pair_with_turns(turns):
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_with_turns(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair_with_turns(float(scaling["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_neighbours(x, positions, f, mag):
    """x [n, ..., 2 * len(f)]: columns (2i, 2i+1) of row t are turned by the angle positions[t] * f[i]."""
    out = torch.empty_like(x)
    for t, p in enumerate(positions):
        ang = float(p) * f
        c, s = torch.cos(ang) * mag, torch.sin(ang) * mag
        u, v = x[t, ..., 0::2], x[t, ..., 1::2]
        out[t, ..., 0::2] = u * c - v * s
        out[t, ..., 1::2] = v * c + u * s
    return out


# ------------------------------------------------------------------ lightning attention
def decayed_linear_attention(q, k, v, decay, state=None):
    """q, k [n, H, d], v [n, H, e], decay [H]: S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t.  Returns (o, S)."""
    n, H, d = q.shape
    e = v.shape[-1]
    S = torch.zeros(H, d, e, dtype=F64) if state is None else state.clone()
    o = torch.zeros(n, H, e, dtype=F64)
    for t in range(n):
        for h in range(H):
            S[h] = float(decay[h]) * S[h] + torch.outer(k[t, h], v[t, h])
            o[t, h] = S[h].T @ q[t, h]
    return o, S


def lightning_mixer(hid, W, p, m, eps):
    n = hid.shape[0]
    H, d, e = m["heads"], m["dim"], m["vdim"]
    q = silu(lin(hid, W[p + "q"])).view(n, H, d)
    k = silu(lin(hid, W[p + "k"])).view(n, H, d)
    v = silu(lin(hid, W[p + "v"])).view(n, H, e)
    o, _ = decayed_linear_attention(q, k, v, m["decay"])
    o = rms_norm(o.reshape(n, H * e), W[p + "norm"], eps) * sigmoid(lin(hid, W[p + "g"]))
    return lin(o, W[p + "o"])


# ------------------------------------------------------------------ latent attention
def sink_softmax_attention(q, k, v, scale, sink):
    """q, k [n, H, d], v [n, H, e], sink [H]: causal softmax whose denominator also holds exp(sink_h)."""
    n, H, _ = q.shape
    o = torch.zeros(n, H, v.shape[-1], dtype=F64)
    for h in range(H):
        for i in range(n):
            s = (k[:i + 1, h] @ q[i, h]) * scale
            m = max(float(s.max()), float(sink[h]))
            w = torch.exp(s - m)
            o[i, h] = (w[:, None] * v[:i + 1, h]).sum(0) / (w.sum() + math.exp(float(sink[h]) - m))
    return o


def latent_mixer(hid, W, p, m, eps, positions=None):
    n = hid.shape[0]
    H, d, r, e, kr = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    positions = list(range(n)) if positions is None else positions
    q = lin(rms_norm(lin(hid, W[p + "dq"]), W[p + "dq.norm"], eps), W[p + "uq"]).view(n, H, d + r)
    down = lin(hid, W[p + "dkv"])
    c = rms_norm(down[:, :kr], W[p + "dkv.norm"], eps)
    k_plain = lin(c, W[p + "uk"]).view(n, H, d)
    v = lin(c, W[p + "uv"]).view(n, H, e)
    q_rot, k_rot = q[..., d:], down[:, kr:]
    if r:
        f, mag = rotary_frequencies(m["rot"]["dims"], m["rot"]["base"], m["rot"].get("scaling"))
        q_rot = rotate_neighbours(q_rot, positions, f, mag)
        k_rot = rotate_neighbours(k_rot, positions, f, mag)
    qq = torch.cat([q[..., :d], q_rot], -1)
    kk = torch.cat([k_plain, k_rot[:, None, :].expand(n, H, r)], -1)
    o = sink_softmax_attention(qq, kk, v, m["scale"], W[p + "sink"].to(F64))
    return lin(o.reshape(n, H * e) * sigmoid(lin(hid, W[p + "g"])), W[p + "o"])


# ------------------------------------------------------------------ mixture of experts
def clamped_glu_expert(hid, W, p, limit):
    g = lin(hid, W[p + "gate"]).clamp(max=limit)
    u = lin(hid, W[p + "up"]).clamp(-limit, limit)
    return lin(g * sigmoid(1.702 * g) * (u + 1.0), W[p + "down"])


def route(hid, W, p, r):
    """Returns (chosen experts [n, top], weights [n, top])."""
    E, top = r["experts"], r["top"]
    s = sigmoid(lin(hid, W[p + "router"]))
    choice = s + W[p + "correction"].to(F64)
    g = r.get("groups")
    idx, wts = [], []
    for t in range(hid.shape[0]):
        c = choice[t].clone()
        if g and g["count"] > 1:
            size = E // g["count"]
            score = [c[a * size:(a + 1) * size].sort(descending=True).values[:2].sum() for a in range(g["count"])]
            best = sorted(range(g["count"]), key=lambda a: (-float(score[a]), a))[:g["keep"]]
            for a in range(g["count"]):
                if a not in best:
                    c[a * size:(a + 1) * size] = -math.inf
        chosen = sorted(range(E), key=lambda e_: (-float(c[e_]), e_))[:top]
        w = s[t, chosen]
        idx.append(chosen)
        wts.append(w / (w.sum() + 1e-20))
    return idx, torch.stack(wts)


def moe(hid, W, p, ml):
    idx, wts = route(hid, W, p, ml["router"])
    out = torch.zeros_like(hid)
    for t in range(hid.shape[0]):
        for j, e in enumerate(idx[t]):
            out[t] += wts[t, j] * clamped_glu_expert(hid[t:t + 1], W, f"{p}e{e}.", ml["expert"]["limit"])[0]
    if ml.get("shared"):
        out = out + clamped_glu_expert(hid, W, p + "shared.", ml["shared"]["limit"])
    return out


# ------------------------------------------------------------------ the model
def layer_runs(cfg):
    """[(layer, number of the pass it opens or None)] in the order of one forward pass."""
    n, lp = len(cfg["layers"]), cfg.get("loop")
    if not lp:
        return [(i, None) for i in range(n)]
    runs = [(i, None) for i in range(lp["start"])]
    for t in range(lp["times"]):
        runs += [(i, t if i == lp["start"] else None) for i in range(lp["start"], lp["stop"])]
    return runs + [(i, None) for i in range(lp["stop"], n)]


def forward(cfg, W, tokens, layer_sink=None):
    """Logits [n, vocab] of a whole sequence; layer_sink receives the residual stream after every layer run."""
    eps = cfg["norm"]["eps"]
    emb = W["embed"].to(F64)
    first = emb[torch.as_tensor(tokens)]
    x = first.clone()
    for li, opens in layer_runs(cfg):
        if opens is not None:
            x = lin(torch.cat([x, first], -1), W["loop.in"]) + W["loop.step"].to(F64)[opens]
        L, p = cfg["layers"][li], f"l{li}."
        hid = rms_norm(x, W[p + "norm1"], eps)
        mix = lightning_mixer if L["type"] == "lightning" else latent_mixer
        x = x + rms_norm(mix(hid, W, p + "mix.", L["mixer"], eps), W[p + "norm1b"], eps)
        if L.get("mlp"):
            hid = rms_norm(x, W[p + "norm2"], eps)
            x = x + rms_norm(moe(hid, W, p + "mlp.", L["mlp"]), W[p + "norm2b"], eps)
        if layer_sink is not None:
            layer_sink.append(x.clone())
    return lin(rms_norm(x, W["final.norm"], eps), emb)


# ------------------------------------------------------------------ small configurations and random checkpoints
def lightning(heads=2, dim=8, vdim=12, decay=None):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim,
                                           "decay": decay or [0.5 + 0.49 * (h + 1) / heads for h in range(heads)]}}


def latent(heads=3, dim=8, rot_dim=4, vdim=10, q_rank=12, kv_rank=14, scale=None, base=300.0, scaling=None):
    rot = {"dims": rot_dim, "base": base}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim,
                                                  "q_rank": q_rank, "kv_rank": kv_rank,
                                                  "scale": scale or (dim + rot_dim) ** -0.5, "rot": rot}}


def experts(n=6, top=2, groups=3, keep=2, ff=10, limit=1.2, shared_ff=14, shared_limit=2.5):
    m = {"kind": "moe", "expert": {"ff": ff, "limit": limit},
         "router": {"experts": n, "top": top, "groups": {"count": groups, "keep": keep}},
         "shared": {"ff": shared_ff, "limit": shared_limit} if shared_ff else None}
    return m


def layer(mixer, mlp):
    return dict(mixer, mlp=mlp)


def make_config(layers, width=40, vocab=61, eps=1e-5, loop=None):
    cfg = {"architecture": "Birizen", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if loop:
        cfg["loop"] = dict(zip(("start", "stop", "times"), loop))
    return cfg


def make_checkpoint(cfg, seed=0, dtype=torch.bfloat16, spread=1.0):
    """Random weights rounded to `dtype` (so a 16-bit engine holds exactly the same numbers), returned as float32."""
    g = torch.Generator().manual_seed(seed)
    D = cfg["width"]

    def mat(rows, cols, gain=1.0):
        return (torch.randn(rows, cols, generator=g) * gain / math.sqrt(cols)).to(dtype).float()

    def vec(n, mean=1.0, dev=0.2):
        return (mean + dev * torch.randn(n, generator=g)).to(dtype).float()

    W = {"embed": (torch.randn(cfg["vocab"], D, generator=g)).to(dtype).float(), "final.norm": vec(D)}
    if cfg.get("loop"):
        W["loop.in"] = mat(D, 2 * D, 1.4)
        W["loop.step"] = vec(cfg["loop"]["times"] * D, 0.0, 0.3).view(cfg["loop"]["times"], D)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        for nm in ("norm1", "norm1b"):
            W[p + nm] = vec(D)
        if L["type"] == "lightning":
            H, d, e = m["heads"], m["dim"], m["vdim"]
            W.update({p + "mix.q": mat(H * d, D, 2.0 * spread), p + "mix.k": mat(H * d, D, 2.0 * spread),
                      p + "mix.v": mat(H * e, D, 2.0), p + "mix.g": mat(H * e, D, 2.0), p + "mix.o": mat(D, H * e),
                      p + "mix.norm": vec(H * e)})
        else:
            H, d, r, e = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
            W.update({p + "mix.dq": mat(m["q_rank"], D), p + "mix.dq.norm": vec(m["q_rank"]),
                      p + "mix.uq": mat(H * (d + r), m["q_rank"], 2.5 * spread),
                      p + "mix.dkv": mat(m["kv_rank"] + r, D, 2.0), p + "mix.dkv.norm": vec(m["kv_rank"]),
                      p + "mix.uk": mat(H * d, m["kv_rank"], 2.5 * spread), p + "mix.uv": mat(H * e, m["kv_rank"], 1.5),
                      p + "mix.sink": vec(H, 0.5, 1.0), p + "mix.g": mat(H * e, D, 2.0), p + "mix.o": mat(D, H * e)})
        ml = L.get("mlp")
        if ml:
            for nm in ("norm2", "norm2b"):
                W[p + nm] = vec(D)
            E, ff = ml["router"]["experts"], ml["expert"]["ff"]
            W[p + "mlp.router"] = mat(E, D, 3.0)
            W[p + "mlp.correction"] = vec(E, 0.0, 0.3)
            for e_ in range(E):
                W.update({f"{p}mlp.e{e_}.gate": mat(ff, D, 2.5), f"{p}mlp.e{e_}.up": mat(ff, D, 2.5),
                          f"{p}mlp.e{e_}.down": mat(D, ff)})
            if ml.get("shared"):
                sf = ml["shared"]["ff"]
                W.update({p + "mlp.shared.gate": mat(sf, D, 2.5), p + "mlp.shared.up": mat(sf, D, 2.5),
                          p + "mlp.shared.down": mat(D, sf)})
    return W
