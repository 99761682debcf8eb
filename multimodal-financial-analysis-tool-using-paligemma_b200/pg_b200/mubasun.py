"""Mubasun: a decoder-only language model served on ragged token batches.

Design (every size and constant comes from config.json; nothing below is tied to one checkpoint):

  x_0[t]   = embed[token_t] + pos[position_t]                               fp32 residual stream
  layer    : h = GroupRMSNorm(x) * w      (the row is cut into `norm.groups` equal parts, each with its own rms)
             x <- x + (Mixer(h) + FF(h))  (one norm, both sublayers read it)
  mixer    : q = RMS_all(Wq h) * wq, k = RMS_all(Wk h) * wk (norm over the WHOLE projection, before the head split),
             v = Wv h; score_h(i, j) = scale * q_h(i).k_g(j) - 2^(-8 (h+1) / H) * (i - j) for 0 <= i - j < window;
             softmax; o = concat_h(P_h V_g) * sigmoid(Wg h); output Wo o.  A layer with `kv_from: j` has no key /
             value tensors and attends the cache of layer j with its own queries.
  ff dense : Wdown xIELU(Wup h)
  ff moe   : s = softmax(Wrouter h) over experts + identity experts, the `top` largest of s + correction are used
             with weights s * router.scale; expert e: Wdown_e (silu(Wgate_e h) * Wup_e h); an identity expert returns
             h; a shared expert of the same form is added times sigmoid(w_sg . h)
  output   : logits = Whead (GroupRMSNorm(x) * w_final)

The engine owns the repacked weights and the paged key/value pools (one pair per layer that has keys of its own;
layers with `kv_from` alias them) and issues the kernel sequence of one step over a flat token list: every token
carries its page-table row and position, so prompt portions and decoded tokens of different sequences share every
launch, and the logits of a position do not depend on the cut or on its neighbours in the batch.  The cache manager
(`scheduler.SlotKV`), the scheduler (`scheduler.RaggedBatcher`) and sampling are the framework's own.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Dict, List, Mapping, Optional, Sequence

import torch

from . import _cabi as cabi
from ._cabi import ptr
from .ragged_engine import RaggedEngine, StepInputs
from .registry import register


@dataclass
class MixerCfg:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int                     # 0 = every earlier position
    kv_from: Optional[int] = None


@dataclass
class MlpCfg:
    kind: str                       # "dense" | "moe"
    ff: int = 0                     # dense width / expert width
    experts: int = 0
    identity: int = 0
    top: int = 0
    router_scale: float = 1.0
    shared_ff: int = 0              # 0 = no shared expert


@dataclass
class LayerCfg:
    mixer: MixerCfg
    mlp: Optional[MlpCfg]


@dataclass
class MubasunConfig:
    vocab: int
    width: int
    max_positions: int
    eps: float
    groups: int
    layers: List[LayerCfg] = field(default_factory=list)

    @staticmethod
    def from_dict(cfg: Mapping) -> "MubasunConfig":
        norm = cfg.get("norm") or {}
        layers = []
        for i, L in enumerate(cfg["layers"]):
            if L.get("type", "attention") != "attention":
                raise ValueError(f"layer {i}: unknown mixer type {L.get('type')!r}")
            m = L["mixer"]
            heads = int(m["heads"])
            mask = m.get("mask") or {}
            mixer = MixerCfg(heads=heads, kv_heads=int(m.get("kv_heads", heads)), dim=int(m["dim"]),
                             vdim=int(m.get("vdim", m["dim"])), scale=float(m["scale"]),
                             window=int(mask.get("size", 0) or 0),
                             kv_from=None if m.get("kv_from") is None else int(m["kv_from"]))
            if mixer.heads % mixer.kv_heads:
                raise ValueError(f"layer {i}: {mixer.heads} heads over {mixer.kv_heads} key/value heads")
            ml = L.get("mlp")
            if ml is None:
                mlp = None
            elif ml["kind"] == "dense":
                mlp = MlpCfg(kind="dense", ff=int(ml["ff"]))
            elif ml["kind"] == "moe":
                r = ml["router"]
                sh = ml.get("shared")
                mlp = MlpCfg(kind="moe", ff=int(ml["expert"]["ff"]), experts=int(r["experts"]),
                             identity=int(r.get("identity", 0) or 0), top=int(r["top"]),
                             router_scale=float(r.get("scale", 1.0)), shared_ff=int(sh["ff"]) if sh else 0)
            else:
                raise ValueError(f"layer {i}: unknown feed-forward kind {ml['kind']!r}")
            layers.append(LayerCfg(mixer, mlp))
        for i, L in enumerate(layers):
            j = L.mixer.kv_from
            if j is not None:
                if not (0 <= j < i) or layers[j].mixer.kv_from is not None:
                    raise ValueError(f"layer {i}: kv_from {j} must name an earlier layer with keys of its own")
                src = layers[j].mixer
                if (src.kv_heads, src.dim, src.vdim) != (L.mixer.kv_heads, L.mixer.dim, L.mixer.vdim):
                    raise ValueError(f"layer {i}: key/value shape differs from layer {j}")
        return MubasunConfig(vocab=int(cfg["vocab"]), width=int(cfg["width"]),
                             max_positions=int(cfg["max_positions"]), eps=float(norm.get("eps", 1e-6)),
                             groups=int(norm.get("groups", 1)), layers=layers)


def distance_slopes(heads: int) -> torch.Tensor:
    """slope_h = 2^(-8 (h + 1) / H), h = 0 .. H-1."""
    h = torch.arange(1, heads + 1, dtype=torch.float64)
    return torch.pow(torch.tensor(2.0, dtype=torch.float64), -8.0 * h / heads).to(torch.float32)


@register("Mubasun")
class MubasunEngine(RaggedEngine):
    """Weights + paged pools + the launch sequence of one step over a ragged token batch."""

    _ERR_TEXT = {2: "the grouped expert GEMM gave up waiting on its pipeline (its results are invalid)"}

    def __init__(self, config, weights: Mapping[str, torch.Tensor], *, device="cuda", dtype=torch.bfloat16,
                 page_size: int = 64, kv_pool_tokens: int = 65536, gemm_impl: int = 0, moe_impl: int = 0):
        self.cfg = config if isinstance(config, MubasunConfig) else MubasunConfig.from_dict(config)
        self._init_common(device=device, dtype=dtype, page_size=page_size, gemm_impl=gemm_impl)
        self.max_positions = self.cfg.max_positions
        self.moe_impl = int(os.environ.get("PG_MOE_IMPL", moe_impl))
        self._repack(weights)
        for w, lc in zip(self.layers, self.cfg.layers):
            npj = w["proj"].shape[0]
            w["attn_tc"] = bool(cabi.lib().pg_attention_ragged_tc_ok(lc.mixer.dim, lc.mixer.vdim, self.page_size, w["nq"],
                                                                     w["ng"], npj, self.dt)) and w["g_col"] % 8 == 0
        self._attn_tc_any = any(w["attn_tc"] for w in self.layers)
        self._init_runtime(kv_pool_tokens)
        self.k_pools: Dict[int, torch.Tensor] = {}
        self.v_pools: Dict[int, torch.Tensor] = {}
        for i, L in enumerate(self.cfg.layers):
            m = L.mixer
            if m.kv_from is None:
                self.k_pools[i] = torch.zeros((self.num_pages, self.page_size, m.kv_heads * m.dim), dtype=dtype,
                                              device=self.device)
                self.v_pools[i] = torch.zeros((self.num_pages, self.page_size, m.kv_heads * m.vdim), dtype=dtype,
                                              device=self.device)

    # ------------------------------------------------------------------ weights
    def _repack(self, weights: Mapping[str, torch.Tensor]) -> None:
        c = self.cfg
        used = set()

        def W(name, shape=None):
            if name not in weights:
                raise KeyError(f"checkpoint has no tensor {name!r}")
            used.add(name)
            t = weights[name]
            if shape is not None and tuple(t.shape) != tuple(shape):
                raise ValueError(f"tensor {name}: shape {tuple(t.shape)}, the config wants {tuple(shape)}")
            return t.to(device=self.device, dtype=self.dtype).contiguous()

        D = c.width
        if D % c.groups:
            raise ValueError(f"width {D} is not a multiple of norm.groups {c.groups}")
        self.emb, self.pos = W("embed", (c.vocab, D)), W("pos", (c.max_positions, D))
        self.final_norm, self.head = W("final.norm", (D,)), W("head", (c.vocab, D))
        self.layers: List[dict] = []
        for i, L in enumerate(c.layers):
            m, p = L.mixer, f"l{i}."
            nq, nk, nv, ng = m.heads * m.dim, m.kv_heads * m.dim, m.kv_heads * m.vdim, m.heads * m.vdim
            own = m.kv_from is None
            parts = [W(p + "mix.q", (nq, D))]
            if own:
                parts += [W(p + "mix.k", (nk, D)), W(p + "mix.v", (nv, D))]
            parts.append(W(p + "mix.g", (ng, D)))
            w = dict(norm=W(p + "norm1", (D,)), proj=torch.cat(parts, 0).contiguous(), q_norm=W(p + "mix.q.norm", (nq,)),
                     k_norm=W(p + "mix.k.norm", (nk,)) if own else None, o=W(p + "mix.o", (D, ng)),
                     q_col=0, k_col=nq, v_col=nq + nk, g_col=nq + (nk + nv if own else 0), nq=nq, nk=nk if own else 0,
                     nv=nv if own else 0, ng=ng, kv_layer=i if own else m.kv_from,
                     slopes=distance_slopes(m.heads).to(self.device))
            ml = L.mlp
            if ml is not None and ml.kind == "dense":
                w.update(up=W(p + "mlp.up", (ml.ff, D)), down=W(p + "mlp.down", (D, ml.ff)), act=W(p + "mlp.act", (2,)))
            elif ml is not None:
                E, R = ml.experts, ml.experts + ml.identity
                w["gu"] = torch.stack([torch.cat([W(f"{p}mlp.e{e}.gate", (ml.ff, D)), W(f"{p}mlp.e{e}.up", (ml.ff, D))], 0)
                                       for e in range(E)], 0).contiguous()
                w["dn"] = torch.stack([W(f"{p}mlp.e{e}.down", (D, ml.ff)) for e in range(E)], 0).contiguous()
                w["router"] = W(p + "mlp.router", (R, D))
                w["correction"] = W(p + "mlp.correction", (R,)) if (p + "mlp.correction") in weights else None
                if ml.shared_ff:
                    s = p + "mlp.shared."
                    w["s_gu"] = torch.cat([W(s + "gate", (ml.shared_ff, D)), W(s + "up", (ml.shared_ff, D))], 0).contiguous()
                    w["s_dn"] = W(s + "down", (D, ml.shared_ff))
                    w["s_sg"] = W(s + "sg", (1, D)).reshape(D).contiguous()
            self.layers.append(w)
        extra = sorted(set(weights) - used)
        if extra:
            raise ValueError(f"checkpoint holds {len(extra)} tensor(s) the config does not describe: {extra[:5]}")

    # ------------------------------------------------------------------ op wrappers
    def _norm(self, out, x, w, add_a=None, add_b=None, rows_idx=None, rows=None):
        c = self.cfg
        n = x.shape[0] if rows is None else rows
        cabi.check(cabi.lib().pg_group_rmsnorm(
            ptr(out), ptr(x), ptr(add_a), 0 if add_a is None else add_a.stride(0), ptr(add_b),
            0 if add_b is None else add_b.stride(0), ptr(w), ptr(rows_idx), n, c.width, c.groups, c.eps, self.dt,
            cabi.stream()), "group_rmsnorm")

    # ------------------------------------------------------------------ one step
    def _forward_device(self, kv, inp: StepInputs, layer_sink: Optional[list]) -> torch.Tensor:
        c, L, st = self.cfg, cabi.lib(), cabi.stream()
        tm = self._tm
        T, nw = inp.T, inp.nw
        d_ids, d_slot, d_pos, d_want, d_tiles, n_qt = inp.ids, inp.slot, inp.pos, inp.want, inp.tiles, inp.n_tiles
        D = c.width
        x = self._new(T, D, dtype=torch.float32)
        cabi.check(L.pg_embed_pos(ptr(x), ptr(d_ids), ptr(d_pos), ptr(self.emb), ptr(self.pos), T, D, c.vocab,
                                  c.max_positions, 1.0, ptr(self.err_flag), self.dt, st), "embed_pos")
        h = self._new(T, D)
        pend_a = pend_b = None        # sublayer outputs not yet summed into x (the next norm kernel adds them)
        for li, (lc, w) in enumerate(zip(c.layers, self.layers)):
            m = lc.mixer
            with tm("norm"):
                self._norm(h, x, w["norm"], pend_a, pend_b)
            pend_a = pend_b = None
            with tm("proj"):
                proj = self._linear(h, w["proj"])
            q = self._new(T, w["nq"])
            kp, vp = self.k_pools[w["kv_layer"]], self.v_pools[w["kv_layer"]]
            with tm("qknorm_append"):
                cabi.check(L.pg_qknorm_append(ptr(q), ptr(proj), proj.stride(0), w["q_col"], w["nq"], w["k_col"], w["nk"],
                                              w["v_col"], w["nv"], ptr(w["q_norm"]), ptr(w["k_norm"]), c.eps, ptr(kp),
                                              ptr(vp), ptr(kv.page_table), kv.max_pages, self.page_size, ptr(d_slot),
                                              ptr(d_pos), T, self.dt, st), "qknorm_append")
            att = self._new(T, w["ng"])
            gate = proj[:, w["g_col"]:]
            with tm("attention"):
                if n_qt and w["attn_tc"]:
                    cabi.check(L.pg_attention_ragged_tc(ptr(att), att.stride(0), ptr(q), q.stride(0), ptr(gate),
                                                        proj.stride(0), ptr(kp), ptr(vp), self.num_pages * self.page_size,
                                                        ptr(kv.page_table), kv.max_pages, self.page_size, ptr(d_tiles), n_qt,
                                                        T, m.heads, m.kv_heads, m.dim, m.vdim, m.scale, m.window,
                                                        ptr(w["slopes"]), ptr(self.err_flag), self.dt, st),
                               "attention_ragged_tc")
                else:
                    cabi.check(L.pg_attention_ragged(ptr(att), att.stride(0), ptr(q), q.stride(0), ptr(gate),
                                                     proj.stride(0), ptr(kp), ptr(vp), ptr(kv.page_table), kv.max_pages,
                                                     self.page_size, ptr(d_slot), ptr(d_pos), T, m.heads, m.kv_heads, m.dim,
                                                     m.vdim, m.scale, m.window, ptr(w["slopes"]), ptr(self.attn_ws),
                                                     self.attn_ws.numel(), self.dt, st),
                               "attention_ragged")
            with tm("o"):
                pend_a = self._linear(att, w["o"])
            ml = lc.mlp
            if ml is not None and ml.kind == "dense":
                with tm("dense_up"):
                    u = self._linear(h, w["up"])
                with tm("xielu"):
                    cabi.check(L.pg_xielu(ptr(u), ptr(u), ptr(w["act"]), u.numel(), self.dt, st), "xielu")
                with tm("dense_down"):
                    pend_b = self._linear(u, w["down"])
            elif ml is not None:
                self._moe(x, h, ml, w)
            if layer_sink is not None:
                self._norm(None, x, None, pend_a, pend_b)
                pend_a = pend_b = None
                layer_sink.append(x.clone())
        if pend_a is not None or pend_b is not None:
            with tm("norm"):
                self._norm(None, x, None, pend_a, pend_b)
        if nw == 0:
            return torch.empty((0, c.vocab), dtype=torch.float32, device=self.device)
        hf = self._new(nw, D)
        with tm("norm"):
            self._norm(hf, x, self.final_norm, rows_idx=d_want, rows=nw)
        with tm("head"):
            return self._linear(hf, self.head, out_f32=True)

    def _moe(self, x, h, ml: MlpCfg, w: dict) -> None:
        """x += sum over the chosen experts (identity experts return h) + gated shared expert."""
        L, st, tm = cabi.lib(), cabi.stream(), self._tm
        T, D = h.shape
        P, E = T * ml.top, ml.experts
        idx = self._new(P, dtype=torch.int32)
        wts = self._new(P, dtype=torch.float32)
        sg = self._new(T, dtype=torch.float32) if ml.shared_ff else None
        with tm("moe_route"):
            cabi.check(L.pg_moe_route(ptr(idx), ptr(wts), ptr(sg), ptr(h), h.stride(0), ptr(w["router"]),
                                      ptr(w["correction"]), ptr(w.get("s_sg")), T, D, E + ml.identity, ml.top,
                                      ml.router_scale, self.dt, st), "moe_route")
        y, pos = self._moe_experts(h, idx, E, ml.top, ml.ff, w["gu"], w["dn"])
        so = None
        if ml.shared_ff:
            with tm("shared_gate_up"):
                sa = self._linear(h, w["s_gu"], cabi.EPI_SWIGLU)
            with tm("shared_down"):
                so = self._linear(sa, w["s_dn"])
        with tm("moe_combine"):
            cabi.check(L.pg_moe_combine(ptr(x), ptr(y), D, ptr(pos), ptr(wts), ptr(h), h.stride(0), ptr(so),
                                        0 if so is None else so.stride(0), ptr(sg), T, D, ml.top, self.dt, st),
                       "moe_combine")

    def weight_bytes(self) -> int:
        n = sum(t.numel() for t in (self.emb, self.pos, self.final_norm, self.head))
        for w in self.layers:
            n += sum(t.numel() for t in w.values() if isinstance(t, torch.Tensor) and t.dtype == self.dtype)
        return n * torch.tensor([], dtype=self.dtype).element_size()
