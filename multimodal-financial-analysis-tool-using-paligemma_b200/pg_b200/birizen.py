"""Birizen: a decoder-only language model with sandwich norms whose mixers are lightning attention (linear attention
with a constant decay per head) or latent attention (low-rank query and key/value latents, one rotated key part shared
by the heads, a softmax sink and an output gate), a mixture-of-experts feed-forward with a grouped sigmoid router, and
a block of layers that runs several times with the same weights.

Design (every size and every constant that can differ between checkpoints comes from config.json):

  x_0[t]     = embed[token_t]                                                fp32 residual stream; e = x_0 is kept
  schedule   : layers 0 .. start-1 once, layers start .. stop-1 `times` times in a row (same weights, but every pass
               has a cache / state of its own), then stop .. n-1 once.  Right before the first layer of pass t:
               x <- W_in [x ; e] + step[t].  A layer run is one (layer, pass) pair.
  layer      : x <- x + RMS(Mixer(RMS(x) n1)) n1b ;  x <- x + RMS(FF(RMS(x) n2)) n2b   (FF may be absent)
  lightning  : q, k = silu(Wq h), silu(Wk h) (heads x dim), v = silu(Wv h) (heads x vdim);
               S_t = decay_h S_(t-1) + k_t v_t^T,  o_t = S_t^T q_t;  Wo (RMS_all(o) w_norm * sigmoid(Wg h)), the RMS
               over all heads of the token at once; S starts at zero.
  latent     : c_q = RMS(Wdq h) w_dq, q = Wuq c_q, per head [dim plain | rot_dim rotated];
               [a ; r] = Wdkv h: c = RMS(a) w_dkv (kv_rank), k_rot = rotary(r) shared by all heads;
               per head K = Wuk c, V = Wuv c; score(i, j) = scale (q_plain . K_j + rotary(q_rot) . k_rot,j), j <= i;
               softmax whose denominator also holds exp(sink_h); Wo (concat_h(P_h V) * sigmoid(Wg h)).
               Rotary: pairs (2i, 2i+1), angle p * f_i, YaRN-scaled frequencies, cos and sin times 0.1 ln(factor) + 1.
               Only [c | k_rot] is cached; attention runs in the latent space (Wuk folded into the queries, Wuv applied
               to the attended latents), i.e. as attention with ONE key/value head of width kv_rank + rot_dim.
  ff moe     : s = sigmoid(Wrouter h) (fp32); choice = s + correction; experts in `groups.count` equal groups of
               neighbours, group score = sum of its two largest choices, only the `groups.keep` best groups stay;
               the `top` largest choices are used with weights s / (sum of the chosen s + 1e-20);
               expert: g = min(Wgate h, limit), u = clamp(Wup h, -limit, limit), Wdown (g sigmoid(1.702 g) (u + 1));
               a shared expert of the same form (own width and limit) is added for every token.
  output     : logits = embed (RMS(x) n_final)        (the embedding table is the output matrix)

fp32: the residual stream, every norm, positions and angles, attention scores and weights, the router, the decayed
state and its output.  Model dtype (fp32 accumulation): projections and their activations, the latent cache, the
feed-forward.

The engine owns the repacked weights (one fused projection per mixer), one paged latent pool per run of a latent
layer and, through the scheduler's slot table, one fp32 state [slots, heads, dim, vdim] per run of a lightning layer.
The step function, page pool, scheduler and sampling are the framework's (`ragged_engine.RaggedEngine`,
`scheduler.SlotKV` / `SlotState` / `RaggedBatcher`).
"""
from __future__ import annotations

import warnings
from dataclasses import dataclass, field
from typing import Dict, List, Mapping, Optional

import torch

from . import _cabi as cabi
from ._cabi import ptr
from .latent import LatentAttentionMixin, LatentCfg, latent_cfg, pack_latent
from .ragged_engine import RaggedEngine, StepInputs, _stack_rows
from .registry import register

GLU_ALPHA = 1.702                 # the sigmoid's slope in the experts' activation: fixed by the design


@dataclass
class LightningCfg:
    heads: int
    dim: int
    vdim: int
    decay: List[float]


@dataclass
class MoeCfg:
    experts: int
    top: int
    groups: int
    keep: int
    ff: int
    limit: float
    shared_ff: int = 0            # 0 = no shared expert
    shared_limit: float = 0.0


@dataclass
class LayerCfg:
    kind: str                     # "lightning" | "latent_attention"
    mixer: object
    mlp: Optional[MoeCfg]


@dataclass
class LoopCfg:
    start: int
    stop: int
    times: int


@dataclass
class Run:
    layer: int
    loop_pass: Optional[int]      # the number of the pass this run opens (its first layer), else None


@dataclass
class BirizenConfig:
    vocab: int
    width: int
    eps: float
    layers: List[LayerCfg] = field(default_factory=list)
    loop: Optional[LoopCfg] = None

    def runs(self) -> List[Run]:
        """The layer runs of one forward pass, in order."""
        n = len(self.layers)
        if self.loop is None:
            return [Run(i, None) for i in range(n)]
        lp = self.loop
        out = [Run(i, None) for i in range(lp.start)]
        for t in range(lp.times):
            out += [Run(i, t if i == lp.start else None) for i in range(lp.start, lp.stop)]
        return out + [Run(i, None) for i in range(lp.stop, n)]

    @staticmethod
    def from_dict(cfg: Mapping) -> "BirizenConfig":
        layers = []
        for i, L in enumerate(cfg["layers"]):
            m, kind = L["mixer"], L.get("type")
            if kind == "lightning":
                heads = int(m["heads"])
                decay = [float(d) for d in m["decay"]]
                if len(decay) != heads:
                    raise ValueError(f"layer {i}: {len(decay)} decays for {heads} heads")
                mixer = LightningCfg(heads, int(m["dim"]), int(m.get("vdim", m["dim"])), decay)
            elif kind == "latent_attention":
                mixer = latent_cfg(i, m)
            else:
                raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
            ml = L.get("mlp")
            mlp = None
            if ml is not None:
                if ml.get("kind") != "moe":
                    raise ValueError(f"layer {i}: unknown feed-forward kind {ml.get('kind')!r}")
                r, g, sh = ml["router"], (ml["router"].get("groups") or {}), ml.get("shared")
                mlp = MoeCfg(experts=int(r["experts"]), top=int(r["top"]), groups=int(g.get("count", 1)),
                             keep=int(g.get("keep", g.get("count", 1))), ff=int(ml["expert"]["ff"]),
                             limit=float(ml["expert"]["limit"]), shared_ff=int(sh["ff"]) if sh else 0,
                             shared_limit=float(sh["limit"]) if sh else 0.0)
                if mlp.experts % mlp.groups or not (1 <= mlp.keep <= mlp.groups) or \
                        mlp.keep * (mlp.experts // mlp.groups) < mlp.top:
                    raise ValueError(f"layer {i}: top {mlp.top} of {mlp.experts} experts in {mlp.groups} groups, "
                                     f"{mlp.keep} kept")
            layers.append(LayerCfg(kind, mixer, mlp))
        lp = cfg.get("loop")
        loop = None
        if lp:
            loop = LoopCfg(int(lp["start"]), int(lp["stop"]), int(lp["times"]))
            if not (0 <= loop.start < loop.stop <= len(layers)) or loop.times < 1:
                raise ValueError(f"loop over layers {loop.start} .. {loop.stop - 1}, {loop.times} times")
        return BirizenConfig(vocab=int(cfg["vocab"]), width=int(cfg["width"]), eps=float((cfg.get("norm") or {})["eps"]),
                             layers=layers, loop=loop)


@register("Birizen")
class BirizenEngine(LatentAttentionMixin, RaggedEngine):
    """Weights + paged latent pools + recurrent state shapes + the launch sequence of one step over a ragged batch."""

    def __init__(self, config, weights: Mapping[str, torch.Tensor], *, device="cuda", dtype=torch.bfloat16,
                 page_size: int = 64, kv_pool_tokens: int = 65536, gemm_impl: int = 0, strict: bool = False):
        self.cfg = config if isinstance(config, BirizenConfig) else BirizenConfig.from_dict(config)
        self.strict = bool(strict)      # True: tensors the config does not call for raise instead of being reported
        self._init_common(device=device, dtype=dtype, page_size=page_size, gemm_impl=gemm_impl)
        self.runs = self.cfg.runs()
        self.needs_segments = any(self.cfg.layers[r.layer].kind == "lightning" for r in self.runs)
        self._repack(weights)
        for w, lc in zip(self.layers, self.cfg.layers):     # prompt portions of latent layers whose sizes the tensor-core kernel takes
            w["attn_tc"] = lc.kind == "latent_attention" and self._latent_tc_ok(lc.mixer)
        self._attn_tc_any = any(w["attn_tc"] for w in self.layers)
        self._init_runtime(kv_pool_tokens)
        # one latent pool per RUN of a latent layer: a layer that runs twice keeps two caches
        self.c_pools: Dict[int, torch.Tensor] = {}
        for ri, r in enumerate(self.runs):
            if self.cfg.layers[r.layer].kind == "latent_attention":
                self.c_pools[ri] = torch.zeros((self.num_pages, self.page_size, self.layers[r.layer]["ld_pool"]),
                                               dtype=dtype, device=self.device)

    # ------------------------------------------------------------------ weights
    def _repack(self, weights: Mapping[str, torch.Tensor]) -> None:
        c, D = self.cfg, self.cfg.width
        used = set()

        def W(name, shape=None, dtype=None):
            if name not in weights:
                raise KeyError(f"checkpoint has no tensor {name!r}")
            used.add(name)
            t = weights[name]
            if shape is not None and tuple(t.shape) != tuple(shape):
                raise ValueError(f"tensor {name}: shape {tuple(t.shape)}, the config wants {tuple(shape)}")
            return t.to(device=self.device, dtype=dtype or self.dtype).contiguous()

        self.emb, self.final_norm = W("embed", (c.vocab, D)), W("final.norm", (D,))
        self.loop_in = self.loop_step = None
        if c.loop is not None:
            self.loop_in, self.loop_step = W("loop.in", (D, 2 * D)), W("loop.step", (c.loop.times, D))
        self.layers: List[dict] = []
        for i, L in enumerate(c.layers):
            p, m = f"l{i}.", f"l{i}.mix."
            w = dict(norm1=W(p + "norm1", (D,)), norm1b=W(p + "norm1b", (D,)))
            if L.kind == "lightning":
                a = L.mixer
                nk, nv = a.heads * a.dim, a.heads * a.vdim
                w["proj"], w["at"] = _stack_rows([("q", W(m + "q", (nk, D))), ("k", W(m + "k", (nk, D))),
                                                  ("v", W(m + "v", (nv, D))), ("g", W(m + "g", (nv, D)))],
                                                 self.device, self.dtype)
                w.update(onorm=W(m + "norm", (nv,)), o=W(m + "o", (D, nv)),
                         decay=torch.tensor(a.decay, dtype=torch.float32, device=self.device))
            else:
                w.update(pack_latent(W, m, L.mixer, D, self.device, self.dtype, gated=True))
            ml = L.mlp
            if ml is not None:
                f = p + "mlp."
                w.update(norm2=W(p + "norm2", (D,)), norm2b=W(p + "norm2b", (D,)), router=W(f + "router", (ml.experts, D)),
                         correction=W(f + "correction", (ml.experts,)),
                         gu=torch.stack([torch.cat([W(f"{f}e{e}.gate", (ml.ff, D)), W(f"{f}e{e}.up", (ml.ff, D))], 0)
                                         for e in range(ml.experts)], 0).contiguous(),
                         dn=torch.stack([W(f"{f}e{e}.down", (D, ml.ff)) for e in range(ml.experts)], 0).contiguous())
                if ml.shared_ff:
                    s = f + "shared."
                    w["s_gu"] = torch.cat([W(s + "gate", (ml.shared_ff, D)), W(s + "up", (ml.shared_ff, D))], 0).contiguous()
                    w["s_dn"] = W(s + "down", (D, ml.shared_ff))
            self.layers.append(w)
        extra = sorted(set(weights) - used)
        if extra:
            text = f"checkpoint holds {len(extra)} tensor(s) the config does not call for: {extra[:8]}"
            if self.strict:
                raise ValueError(text)
            warnings.warn(text + " (not used)")

    # ------------------------------------------------------------------ recurrent state
    def new_slot_state(self, slots: int):
        from .scheduler import SlotState
        shapes = {}
        for ri, r in enumerate(self.runs):
            L = self.cfg.layers[r.layer]
            if L.kind == "lightning":
                shapes[ri] = (L.mixer.heads, L.mixer.dim, L.mixer.vdim)
        return SlotState(slots, shapes, self.device) if shapes else None

    # ------------------------------------------------------------------ one step
    def _rms(self, out, x, w, add=None, rows_idx=None, rows=None):
        """out = RMS(x) w; `add` (one row of the model dtype) is first added to every row of x."""
        n = x.shape[0] if rows is None else rows
        cabi.check(cabi.lib().pg_group_rmsnorm(ptr(out), ptr(x), ptr(add), 0, None, 0, ptr(w), ptr(rows_idx), n,
                                               self.cfg.width, 1, self.cfg.eps, self.dt, cabi.stream()), "rmsnorm")

    def _post(self, out, x, y, w_post, w_next):
        """x += RMS(y) w_post; out = RMS(x) w_next (when the next sublayer follows at once)."""
        cabi.check(cabi.lib().pg_postnorm_residual(ptr(out) if w_next is not None else None, ptr(x), ptr(y), y.stride(0),
                                                   ptr(w_post), None, ptr(w_next), x.shape[0], self.cfg.width,
                                                   self.cfg.eps, self.dt, cabi.stream()), "postnorm_residual")

    def _lightning(self, kv, inp: StepInputs, ri: int, a: LightningCfg, w: dict, h) -> torch.Tensor:
        L, st, tm, T, at = cabi.lib(), cabi.stream(), self._tm, inp.T, w["at"]
        if kv.state is None or ri not in kv.state.layers:
            raise RuntimeError("this step's slot table carries no recurrent state for the model's lightning layers")
        with tm("proj"):
            proj = self._linear(h, w["proj"])
        nv = a.heads * a.vdim
        o = self._new(T, nv, dtype=torch.float32)
        rec = self._new(int(L.pg_lightning_record_floats(T, a.heads, a.dim, a.vdim)), dtype=torch.float32)
        with tm("lightning_prep"):
            cabi.check(L.pg_lightning_prep(ptr(rec), ptr(proj), proj.stride(0), at["q"], at["k"], at["v"], T, a.heads, a.dim,
                                           a.vdim, self.dt, st), "lightning_prep")
        with tm("lightning"):
            cabi.check(L.pg_lightning_attention(ptr(o), ptr(kv.state.layers[ri]), ptr(rec), ptr(w["decay"]), ptr(inp.segs),
                                                inp.n_segs, a.heads, a.dim, a.vdim, st), "lightning_attention")
        att = self._new(T, nv)
        with tm("headnorm_gate"):       # one RMS over all heads of the token: a single "head" of heads * vdim columns
            cabi.check(L.pg_headnorm_gate(ptr(att), nv, ptr(o), ptr(w["onorm"]), ptr(proj[:, at["g"]:]), proj.stride(0), T, 1,
                                          nv, self.cfg.eps, 1.0, self.dt, st), "headnorm_gate")
        with tm("o"):
            return self._linear(att, w["o"])

    def _moe(self, h, ml: MoeCfg, w: dict) -> torch.Tensor:
        """The feed-forward's output (model dtype): weighted sum of the chosen experts + the shared expert."""
        L, st, tm = cabi.lib(), cabi.stream(), self._tm
        T, D = h.shape
        P = T * ml.top
        idx = self._new(P, dtype=torch.int32)
        wts = self._new(P, dtype=torch.float32)
        with tm("moe_route"):
            cabi.check(L.pg_moe_route_grouped(ptr(idx), ptr(wts), ptr(h), h.stride(0), ptr(w["router"]), ptr(w["correction"]),
                                              T, D, ml.experts, ml.top, ml.groups, ml.keep, self.dt, st), "moe_route_grouped")
        y, pos = self._moe_experts(h, idx, ml.experts, ml.top, ml.ff, w["gu"], w["dn"], cabi.GLU_CLAMPED, ml.limit)
        so = None
        if ml.shared_ff:
            with tm("shared_gate_up"):
                sg = self._linear(h, w["s_gu"])
                sa = self._new(T, ml.shared_ff)
                cabi.check(L.pg_glu_clamped(ptr(sa), ptr(sg), T, ml.shared_ff, ml.shared_limit, GLU_ALPHA, self.dt, st),
                           "glu_clamped")
            with tm("shared_down"):
                so = self._linear(sa, w["s_dn"])
        out = self._new(T, D)
        with tm("moe_combine"):
            cabi.check(L.pg_moe_combine_out(ptr(out), D, ptr(y), D, ptr(pos), ptr(wts), ptr(so),
                                            0 if so is None else so.stride(0), T, D, ml.top, self.dt, st), "moe_combine_out")
        return out

    def _forward_device(self, kv, inp: StepInputs, layer_sink: Optional[list]) -> torch.Tensor:
        c, L, st, tm = self.cfg, cabi.lib(), cabi.stream(), self._tm
        T, nw, D = inp.T, inp.nw, self.cfg.width
        x = self._new(T, D, dtype=torch.float32)
        cabi.check(L.pg_embed_pos(ptr(x), ptr(inp.ids), None, ptr(self.emb), None, T, D, c.vocab, 0, 1.0, ptr(self.err_flag),
                                  self.dt, st), "embed")
        e = x.clone() if c.loop is not None else None      # the embedding output, read again before every pass
        h = self._new(T, D)
        have_h = False                                     # h = RMS(x) norm1 of the coming run is already there
        for ri, run in enumerate(self.runs):
            lc, w = c.layers[run.layer], self.layers[run.layer]
            if run.loop_pass is not None:
                cat = self._new(T, 2 * D)
                with tm("loop_in"):
                    cabi.check(L.pg_concat_cast(ptr(cat), ptr(x), ptr(e), T, D, self.dt, st), "concat_cast")
                    x = self._linear(cat, self.loop_in, out_f32=True)
                with tm("norm"):
                    self._rms(h, x, w["norm1"], add=self.loop_step[run.loop_pass])
            elif not have_h:
                with tm("norm"):
                    self._rms(h, x, w["norm1"])
            if lc.kind == "lightning":
                y = self._lightning(kv, inp, ri, lc.mixer, w, h)
            else:
                y = self._latent(kv, inp, self.c_pools[ri], lc.mixer, w, h)
            nxt = None                                     # the input norm of the coming run, unless a pass opens there
            if ri + 1 < len(self.runs) and self.runs[ri + 1].loop_pass is None:
                nxt = self.layers[self.runs[ri + 1].layer]["norm1"]
            if lc.mlp is not None:
                with tm("post_norm"):
                    self._post(h, x, y, w["norm1b"], w["norm2"])
                y = self._moe(h, lc.mlp, w)
                with tm("post_norm"):
                    self._post(h, x, y, w["norm2b"], nxt)
            else:
                with tm("post_norm"):
                    self._post(h, x, y, w["norm1b"], nxt)
            have_h = nxt is not None
            if layer_sink is not None:
                layer_sink.append(x.clone())
        if nw == 0:
            return torch.empty((0, c.vocab), dtype=torch.float32, device=self.device)
        hf = self._new(nw, D)
        with tm("norm"):
            self._rms(hf, x, self.final_norm, rows_idx=inp.want, rows=nw)
        with tm("head"):
            return self._linear(hf, self.emb, out_f32=True)

    def weight_bytes(self) -> int:
        n = self.emb.numel() + self.final_norm.numel()
        if self.loop_in is not None:
            n += self.loop_in.numel() + self.loop_step.numel()
        for w in self.layers:
            n += sum(t.numel() for t in w.values() if isinstance(t, torch.Tensor) and t.dtype == self.dtype)
        return n * torch.tensor([], dtype=self.dtype).element_size()
