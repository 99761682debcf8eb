"""Plain float64 restatement of the Gogivik design: one function per mechanism, whole sequences, no caches, no
batching, no code shared with the served path.  Slow on purpose: loops over tokens and heads where that is clearest.

Shapes: a sequence is [n, ...]; weights are [out, in] and applied as x @ W.T.  Positions are 0 .. n-1.
"""
import math

import torch

F64 = torch.float64


# ------------------------------------------------------------------ elementary pieces
def silu(z):
    return z / (1.0 + torch.exp(-z))


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def lin(x, w):
    return x @ w.to(F64).T


def norm_one_plus(x, w, eps):
    """The layer norms store their weight around zero: RMS(x) (1 + w)."""
    return rms(x, eps) * (1.0 + w.to(F64))


# ------------------------------------------------------------------ causal convolutions over time
def causal_conv(h, w, bias=None):
    """h [n, C], w [C, taps]: out_t = sum_j w[:, j] h_(t - taps + 1 + j), zeros before the start (the last column of w
    multiplies the current token)."""
    n, C = h.shape
    taps = w.shape[1]
    w = w.to(F64)
    out = torch.zeros(n, C, dtype=F64)
    for t in range(n):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] += w[:, j] * h[s]
    return out if bias is None else out + bias.to(F64)


def input_conv(h, w):
    """What a sublayer reads: h + conv(h)."""
    return h + causal_conv(h, w)


# ------------------------------------------------------------------ rotary positions
def frequencies(dims, base, factor=1.0):
    i = torch.arange(dims // 2, dtype=F64)
    return float(base) ** (-2.0 * i / dims) / float(factor)


def rotate(x, positions, f, layout, sign=1.0):
    """x [n, ..., >= 2 len(f)]: the first 2 len(f) columns of row t are turned in pairs by sign * positions[t] * f;
    layout "neighbours": (2i, 2i+1); "halves": (i, i + len(f)).  The other columns pass."""
    out = x.clone()
    m = f.shape[0]
    for t, p in enumerate(positions):
        ang = sign * float(p) * f
        c, s = torch.cos(ang), torch.sin(ang)
        if layout == "neighbours":
            u, v = x[t, ..., 0:2 * m:2], x[t, ..., 1:2 * m:2]
            out[t, ..., 0:2 * m:2] = u * c - v * s
            out[t, ..., 1:2 * m:2] = v * c + u * s
        else:
            u, v = x[t, ..., 0:m], x[t, ..., m:2 * m]
            out[t, ..., 0:m] = u * c - v * s
            out[t, ..., m:2 * m] = v * c + u * s
    return out


# ------------------------------------------------------------------ masks
def window_visible(i, j, size):
    return 0 <= i - j < size


def chunk_visible(i, j, size):
    return j <= i and i // size == j // size


def masked_softmax_attention(q, k, v, scale, visible, sink=None):
    """q [n, d], k [n, d], v [n, e] of ONE head; sink: a number whose exp joins the denominator once."""
    n = q.shape[0]
    out = torch.zeros(n, v.shape[1], dtype=F64)
    for i in range(n):
        js = torch.tensor([j for j in range(n) if visible(i, j)], dtype=torch.long)
        s = (k[js] @ q[i]) * scale
        m = s.max() if sink is None else torch.maximum(s.max(), sink)
        e = torch.exp(s - m)
        den = e.sum() + (torch.exp(sink - m) if sink is not None else 0.0)
        out[i] = (e / den) @ v[js]
    return out


# ------------------------------------------------------------------ mixers
def latent_attention_mixer(h, W, p, m, eps):
    n = h.shape[0]
    H, d, r, e, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = list(range(n))
    f = frequencies(m["rot"]["dims"], m["rot"]["base"], ((m["rot"].get("scaling") or {}).get("factor", 1.0)))
    cq = rms(lin(h, W[p + "dq"]), eps) * W[p + "dq.norm"].to(F64)
    q = lin(cq, W[p + "uq"]).view(n, H, d + r)
    a = lin(h, W[p + "dkv"])
    c = rms(a[:, :R], eps) * W[p + "dkv.norm"].to(F64)
    k_rot = rotate(a[:, R:], pos, f, "neighbours")
    k_plain = lin(c, W[p + "uk"]).view(n, H, d)
    v = lin(c, W[p + "uv"]).view(n, H, e)
    size = m["mask"]["size"]
    outs = []
    for hd in range(H):
        qh = torch.cat([q[:, hd, :d], rotate(q[:, hd, d:], pos, f, "neighbours")], -1)
        kh = torch.cat([k_plain[:, hd], k_rot], -1)
        outs.append(masked_softmax_attention(qh, kh, v[:, hd], m["scale"], lambda i, j: window_visible(i, j, size),
                                             sink=W[p + "sink"].to(F64)[hd]))
    return lin(torch.cat(outs, -1), W[p + "o"])


def attention_mixer(h, W, p, m, eps):
    n = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = list(range(n))
    rot = m["rot"]
    f = frequencies(rot["dims"], rot["base"], ((rot.get("scaling") or {}).get("factor", 1.0)))
    fv = frequencies(e, rot["base"])                       # values: all of vdim, never scaled
    q = lin(h, W[p + "q"]).view(n, H, d)
    k = lin(h, W[p + "k"]).view(n, G, d)
    v = lin(h, W[p + "v"]).view(n, G, e)
    q = rotate(rms(q, eps) * W[p + "q.norm"].to(F64), pos, f, "halves")
    k = rotate(rms(k, eps) * W[p + "k.norm"].to(F64), pos, f, "halves")
    v = rotate(rms(v, eps), pos, fv, "halves")
    size = m["mask"]["size"]
    outs = []
    for hd in range(H):
        g = hd // (H // G)
        o = masked_softmax_attention(q[:, hd], k[:, g], v[:, g], m["scale"], lambda i, j: chunk_visible(i, j, size))
        outs.append(rotate(o, pos, fv, "halves", sign=-1.0))
    return lin(torch.cat(outs, -1), W[p + "o"])


def selective_scan(x, B, C, dt, A_log, D, heads_per_group):
    """x [n, H, e], B, C [n, G, N], dt [n, H] (after softplus): S_t = exp(-exp(A_log) dt) S_(t-1) + dt B_t x_t^T,
    y_t = S_t^T C_t + D x_t, S [N, e] per head, zero at the start."""
    n, H, e = x.shape
    N = B.shape[-1]
    y = torch.zeros(n, H, e, dtype=F64)
    for hd in range(H):
        g = hd // heads_per_group
        S = torch.zeros(N, e, dtype=F64)
        for t in range(n):
            S = torch.exp(-torch.exp(A_log[hd]) * dt[t, hd]) * S + dt[t, hd] * torch.outer(B[t, g], x[t, hd])
            y[t, hd] = S.T @ C[t, g] + D[hd] * x[t, hd]
    return y


def mamba2_mixer(h, W, p, m, eps):
    n = h.shape[0]
    H, e, N, G, ng = m["heads"], m["vdim"], m["state"], m["groups"], m["norm_groups"]
    inner = H * e
    u = lin(h, W[p + "in"])
    z, xbc, dt = u[:, :inner], u[:, inner:2 * inner + 2 * G * N], u[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, W[p + "conv"], W[p + "conv.b"]))
    x = xbc[:, :inner].reshape(n, H, e)
    B = xbc[:, inner:inner + G * N].reshape(n, G, N)
    C = xbc[:, inner + G * N:].reshape(n, G, N)
    dt = softplus(dt + W[p + "dt_bias"].to(F64))
    y = selective_scan(x, B, C, dt, W[p + "A_log"].to(F64), W[p + "D"].to(F64), H // G).reshape(n, inner)
    y = y * silu(z)
    y = rms(y.view(n, ng, inner // ng), eps).reshape(n, inner) * W[p + "norm"].to(F64)
    return lin(y, W[p + "o"])


MIXERS = {"latent_attention": latent_attention_mixer, "attention": attention_mixer, "mamba2": mamba2_mixer}


# ------------------------------------------------------------------ feed-forward, the model
def squared_relu_ff(h, W, p):
    return lin(torch.relu(lin(h, W[p + "up"])) ** 2, W[p + "down"])


def forward(cfg, W, tokens, layers_out=None):
    """Logits [n, vocab] (float64) of one sequence; layers_out (a list) receives the residual stream after each layer."""
    eps = cfg["norm"]["eps"]
    taps = cfg["canon"]["taps"]
    x = W["embed"].to(F64)[torch.as_tensor(tokens, dtype=torch.long)]
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        assert W[p + "canon1"].shape[1] == taps
        h = input_conv(norm_one_plus(x, W[p + "norm1"], eps), W[p + "canon1"])
        x = x + MIXERS[L["type"]](h, W, p + "mix.", L["mixer"], eps)
        if L.get("mlp") is not None:
            assert L["mlp"]["kind"] == "dense"
            h = input_conv(norm_one_plus(x, W[p + "norm2"], eps), W[p + "canon2"])
            x = x + squared_relu_ff(h, W, p + "mlp.")
        if layers_out is not None:
            layers_out.append(x.clone())
    return lin(norm_one_plus(x, W["final.norm"], eps), W["head"]) * cfg.get("logit_scale", 1.0)


# ------------------------------------------------------------------ configurations and random checkpoints for tests
def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, window, scale=None, base=10000.0):
    return {"type": "latent_attention", "mixer": {
        "heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
        "scale": scale if scale is not None else 1.0 / math.sqrt(dim + rot_dim), "mask": {"size": window},
        "rot": {"dims": rot_dim, "base": base}}}


def attention(heads, kv_heads, dim, vdim, chunk, rot_dims=None, factor=None, scale=None, base=10000.0):
    rot = {"dims": dim if rot_dims is None else rot_dims, "base": base}
    if factor is not None:
        rot["scaling"] = {"factor": factor}
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
                                           "scale": scale if scale is not None else 1.0 / math.sqrt(dim),
                                           "mask": {"size": chunk}, "rot": rot}}


def mamba2(heads, vdim, state, groups, norm_groups, conv):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups,
                                        "norm_groups": norm_groups, "conv": conv}}


def layer(mixer, ff):
    return dict(mixer, mlp={"kind": "dense", "ff": ff} if ff else None)


def make_config(width, vocab, layers, taps=4, eps=1e-5, logit_scale=1.0):
    return {"architecture": "Gogivik", "vocab": vocab, "width": width, "norm": {"eps": eps}, "canon": {"taps": taps},
            "logit_scale": logit_scale, "layers": layers}


def make_checkpoint(cfg, seed=0, dtype=torch.bfloat16):
    """Random weights rounded to `dtype` (so a 16-bit engine holds exactly the same numbers), returned as float32."""
    g = torch.Generator().manual_seed(seed)
    D, taps = cfg["width"], cfg["canon"]["taps"]

    def mat(rows, cols, gain=1.0):
        return (torch.randn(rows, cols, generator=g) * gain / math.sqrt(cols)).to(dtype).float()

    def vec(n, mean=0.0, dev=0.2):
        return (mean + dev * torch.randn(n, generator=g)).to(dtype).float()

    W = {"embed": torch.randn(cfg["vocab"], D, generator=g).to(dtype).float(), "final.norm": vec(D),
         "head": mat(cfg["vocab"], D, 2.0)}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        W[p + "norm1"] = vec(D)
        W[p + "canon1"] = (torch.randn(D, taps, generator=g) * 0.4).to(dtype).float()
        if L["type"] == "latent_attention":
            H, d, r, e = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
            W.update({p + "mix.dq": mat(m["q_rank"], D), p + "mix.dq.norm": vec(m["q_rank"], 1.0),
                      p + "mix.uq": mat(H * (d + r), m["q_rank"], 2.5),
                      p + "mix.dkv": mat(m["kv_rank"] + r, D, 2.0), p + "mix.dkv.norm": vec(m["kv_rank"], 1.0),
                      p + "mix.uk": mat(H * d, m["kv_rank"], 2.5), p + "mix.uv": mat(H * e, m["kv_rank"], 1.5),
                      p + "mix.sink": vec(H, 0.5, 1.0), p + "mix.o": mat(D, H * e)})
        elif L["type"] == "attention":
            H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            W.update({p + "mix.q": mat(H * d, D, 2.0), p + "mix.k": mat(G * d, D, 2.0), p + "mix.v": mat(G * e, D, 2.0),
                      p + "mix.q.norm": vec(d, 1.5, 0.4), p + "mix.k.norm": vec(d, 1.5, 0.4), p + "mix.o": mat(D, H * e, 2.0)})
        else:
            H, e, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
            ch = H * e + 2 * G * N
            W.update({p + "mix.in": mat(2 * H * e + 2 * G * N + H, D, 2.0),
                      p + "mix.conv": (torch.randn(ch, m["conv"], generator=g) * 0.5).to(dtype).float(),
                      p + "mix.conv.b": vec(ch, 0.0, 0.3), p + "mix.dt_bias": vec(H, -1.0, 1.0),
                      p + "mix.A_log": vec(H, -0.5, 1.0), p + "mix.D": vec(H, 1.0, 0.5), p + "mix.norm": vec(H * e, 1.0),
                      p + "mix.o": mat(D, H * e, 1.5)})
        if L.get("mlp"):
            ff = L["mlp"]["ff"]
            W.update({p + "norm2": vec(D), p + "canon2": (torch.randn(D, taps, generator=g) * 0.4).to(dtype).float(),
                      p + "mlp.up": mat(ff, D, 2.0), p + "mlp.down": mat(D, ff)})
    return W
