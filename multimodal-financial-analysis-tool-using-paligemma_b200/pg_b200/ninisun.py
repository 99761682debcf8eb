"""Ninisun: a decoder-only language model with sandwich norms, windowed attention with kept first tokens and value
mixing, and a 'parallel' mixer that runs gated sigmoid attention beside a delta-rule recurrence.

Design (every size and every constant that can differ between checkpoints comes from config.json):

  x_0[t]    = embed[token_t]                                                 fp32 residual stream
  layer     : x <- x + ls1 * RMS(Mixer(RMS(x) n1)) n1b ;  x <- x + ls2 * RMS(FF(RMS(x) n2)) n2b   (FF may be absent)
  attention : q, k, v = Wq h, Wk h, Wv h; rotary positions on the first rot.dims columns of every q / k head (pairs
              (2i, 2i+1), angle p * base^(-2i/dims)); from the second layer with v_mix on, v <- (1 - lam) v + lam v_1
              with v_1 the first such layer's values of the same token (the mixed v is cached); key j is visible to
              query i when j <= i and (i - j < mask.size or j < mask.keep_first); softmax(scale q.k) V; Wo.
  parallel  : left  = Wo (sigmoid(wg . h)_n * sum_j sigmoid(scale q_n.k_j + pb_n) v_j) with biased projections, rotary
                      positions with YaRN-scaled frequencies, every j <= i visible, no normalisation over keys;
              right = Wo ((RMS_head(o) * w_norm) * sigmoid(Wg h)), o_t = S_t^T r_t,
                      S_t = diag(w_t) S_(t-1) - (a_t * u_t)(u_t^T S_(t-1)) + k_t v_t^T per head, u = k / |k|,
                      w = exp(-e^(-1/2) sigmoid(W2 tanh(W1 h) + w0)), a = sigmoid(Wa h + ba); S starts at zero;
              result = left_scale * left + right_scale * right.
  ff dense  : Wdown (gelu_tanh(Wgate h) * Wup h)
  output    : logits = embed (RMS(x) n_final)        (the embedding table is the output matrix)

fp32: the residual stream, every norm, positions and angles, attention scores and weights, the decay, the removal
rate, the unit key, the recurrent state and its output.  Model dtype (fp32 accumulation): projections, caches, gates'
pre-activations, the feed-forward.

The engine owns the repacked weights (one fused projection per mixer, one output projection per mixer: the parallel
mixer's two output matrices are stacked along K and the branch scales are applied to their operands), a paged
key/value pool pair per attention (the sigmoid attention included), and, through the scheduler's slot table, one
fp32 state [slots, heads, dim, dim] per recurrent layer.  The step function, cache manager, scheduler and sampling
are the framework's (`ragged_engine.RaggedEngine`, `scheduler.SlotKV` / `SlotState` / `RaggedBatcher`).
"""
from __future__ import annotations

import math
import warnings
from dataclasses import dataclass, field
from typing import Dict, List, Mapping, Optional

import torch

from . import _cabi as cabi
from ._cabi import ptr
from .ragged_engine import RaggedEngine, RotaryCfg, StepInputs, _stack_rows
from .registry import register

DECAY_SCALE = math.exp(-0.5)      # w = exp(-DECAY_SCALE * sigmoid(.)): the design's fixed decay range
KEY_EPS = 1e-6                    # inside the root of the unit key's length


@dataclass
class AttnCfg:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: Optional[RotaryCfg]
    window: int = 0                 # 0 = every earlier position
    keep_first: int = 0
    v_mix: bool = False
    biased: bool = False            # q / k / v projections carry biases
    sigmoid: bool = False           # unnormalised sigmoid weights with a per-head bias and a per-head output gate


@dataclass
class DeltaCfg:
    heads: int
    dim: int


@dataclass
class LayerCfg:
    kind: str                       # "attention" | "parallel"
    attn: AttnCfg                   # the attention mixer, or the parallel mixer's left branch
    delta: Optional[DeltaCfg] = None
    left_scale: float = 1.0
    right_scale: float = 1.0
    ff: int = 0                     # 0 = no feed-forward


def _attn_cfg(i: int, m: Mapping, **kw) -> AttnCfg:
    heads = int(m["heads"])
    mask, rot = m.get("mask") or {}, m.get("rot")
    a = AttnCfg(heads=heads, kv_heads=int(m.get("kv_heads", heads)), dim=int(m["dim"]), vdim=int(m.get("vdim", m["dim"])),
                scale=float(m["scale"]),
                rot=RotaryCfg(int(rot["dims"]), float(rot["base"]), rot.get("scaling")) if rot else None,
                window=int(mask.get("size", 0) or 0), keep_first=int(mask.get("keep_first", 0) or 0),
                v_mix=bool(m.get("v_mix", False)), **kw)
    if a.heads % a.kv_heads:
        raise ValueError(f"layer {i}: {a.heads} heads over {a.kv_heads} key/value heads")
    if a.rot and (a.rot.dims % 2 or a.rot.dims > a.dim):
        raise ValueError(f"layer {i}: {a.rot.dims} rotated columns of {a.dim}")
    return a


@dataclass
class NinisunConfig:
    vocab: int
    width: int
    eps: float
    layers: List[LayerCfg] = field(default_factory=list)

    @staticmethod
    def from_dict(cfg: Mapping) -> "NinisunConfig":
        layers = []
        for i, L in enumerate(cfg["layers"]):
            m, kind = L["mixer"], L.get("type")
            ml = L.get("mlp")
            if ml is not None and ml.get("kind") != "dense":
                raise ValueError(f"layer {i}: unknown feed-forward kind {ml.get('kind')!r}")
            ff = int(ml["ff"]) if ml else 0
            if kind == "attention":
                layers.append(LayerCfg("attention", _attn_cfg(i, m), ff=ff))
            elif kind == "parallel":
                r = m["right"]
                layers.append(LayerCfg("parallel", _attn_cfg(i, m["left"], biased=True, sigmoid=True),
                                       DeltaCfg(int(r["heads"]), int(r["dim"])), float(m.get("left_scale", 1.0)),
                                       float(m.get("right_scale", 1.0)), ff=ff))
            else:
                raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
        mixed = [L.attn for L in layers if L.kind == "attention" and L.attn.v_mix]
        if any((a.kv_heads * a.vdim) != (mixed[0].kv_heads * mixed[0].vdim) for a in mixed):
            raise ValueError("layers that mix values must agree on their value width")
        return NinisunConfig(vocab=int(cfg["vocab"]), width=int(cfg["width"]), eps=float((cfg.get("norm") or {})["eps"]),
                             layers=layers)


@register("Ninisun")
class NinisunEngine(RaggedEngine):
    """Weights + paged pools + recurrent state shapes + the launch sequence of one step over a ragged token batch."""

    def __init__(self, config, weights: Mapping[str, torch.Tensor], *, device="cuda", dtype=torch.bfloat16,
                 page_size: int = 64, kv_pool_tokens: int = 65536, gemm_impl: int = 0, strict: bool = False):
        self.cfg = config if isinstance(config, NinisunConfig) else NinisunConfig.from_dict(config)
        self.strict = bool(strict)      # True: tensors the config does not call for raise instead of being reported
        self._init_common(device=device, dtype=dtype, page_size=page_size, gemm_impl=gemm_impl)
        self.needs_segments = any(L.delta is not None for L in self.cfg.layers)
        self._repack(weights)
        L_ = cabi.lib()
        for w, lc in zip(self.layers, self.cfg.layers):
            a = lc.attn
            w["attn_tc"] = bool(L_.pg_attention_ragged_tc_ok(
                a.dim, a.vdim, self.page_size, a.heads * a.dim, w["att_cols"], w["proj"].shape[0], self.dt))
        self._attn_tc_any = any(w["attn_tc"] for w in self.layers)
        self._init_runtime(kv_pool_tokens)
        self.k_pools: Dict[int, torch.Tensor] = {}
        self.v_pools: Dict[int, torch.Tensor] = {}
        for i, L in enumerate(self.cfg.layers):
            a = L.attn
            self.k_pools[i] = torch.zeros((self.num_pages, self.page_size, a.kv_heads * a.dim), dtype=dtype, device=self.device)
            self.v_pools[i] = torch.zeros((self.num_pages, self.page_size, a.kv_heads * a.vdim), dtype=dtype, device=self.device)

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
        self.layers: List[dict] = []
        first_mix = None
        for i, L in enumerate(c.layers):
            p, a = f"l{i}.", L.attn
            nq, nk, nv, ng = a.heads * a.dim, a.kv_heads * a.dim, a.kv_heads * a.vdim, a.heads * a.vdim
            w = dict(norm1=W(p + "norm1", (D,)), norm1b=W(p + "norm1b", (D,)), ls1=W(p + "ls1", (D,)), nq=nq, ng=ng)
            if a.rot:
                f, mag = a.rot.table()
                w["freq"], w["mag"] = f.to(torch.float32).to(self.device), float(mag)
            else:
                w["freq"], w["mag"] = None, 1.0
            if L.kind == "attention":
                m = p + "mix."
                w["proj"], at = _stack_rows([("q", W(m + "q", (nq, D))), ("k", W(m + "k", (nk, D))), ("v", W(m + "v", (nv, D)))],
                                            self.device, self.dtype)
                w["o"], w["att_cols"] = W(m + "o", (D, ng)), ng
                w["lam"], w["mix_from"] = 0.0, None
                if a.v_mix:
                    if first_mix is None:
                        first_mix = i                 # the first such layer gives its values, its own weight is unused
                        used.add(m + "vmix")
                    else:
                        lam = W(m + "vmix", None, torch.float32)
                        if lam.numel() != 1:
                            raise ValueError(f"tensor {m}vmix: one mixing weight expected, shape {tuple(lam.shape)}")
                        w["lam"], w["mix_from"] = float(lam.reshape(())), first_mix
            else:
                l, r, d = p + "mix.left.", p + "mix.right.", L.delta
                nd = d.heads * d.dim
                lora = int(weights[r + "w1"].shape[0]) if (r + "w1") in weights else 0
                w["proj"], at = _stack_rows(
                    [("q", W(l + "q", (nq, D))), ("k", W(l + "k", (nk, D))), ("v", W(l + "v", (nv, D))),
                     ("g", W(l + "g", (a.heads, D))), ("rr", W(r + "r", (nd, D))), ("rk", W(r + "k", (nd, D))),
                     ("rv", W(r + "v", (nd, D))), ("rg", W(r + "g", (nd, D))), ("ra", W(r + "a", (nd, D))),
                     ("rw1", W(r + "w1", (lora, D)))], self.device, self.dtype)
                w.update(qb=W(l + "q.b", (nq,)), kb=W(l + "k.b", (nk,)), vb=W(l + "v.b", (nv,)),
                         pb=W(l + "pb", (a.heads,), torch.float32), w2=W(r + "w2", (nd, lora)), w0=W(r + "w0", (nd,)),
                         ab=W(r + "a.b", (nd,)), rnorm=W(r + "norm", (nd,)), lora=lora, nd=nd, left_scale=L.left_scale)
                # one output projection over [left | right] operands; each part starts at a multiple of 8 columns
                r_col = (ng + 7) // 8 * 8
                cols = (r_col + nd + 7) // 8 * 8
                o = torch.zeros((D, cols), dtype=self.dtype, device=self.device)
                o[:, :ng] = W(l + "o", (D, ng))
                o[:, r_col:r_col + nd] = W(r + "o", (D, nd))
                w["o"], w["att_cols"], w["r_col"], w["att_pad"] = o.contiguous(), cols, r_col, cols != ng + nd
            w["at"] = at
            if L.ff:
                m = p + "mlp."
                w.update(norm2=W(p + "norm2", (D,)), norm2b=W(p + "norm2b", (D,)), ls2=W(p + "ls2", (D,)),
                         gu=torch.cat([W(m + "gate", (L.ff, D)), W(m + "up", (L.ff, D))], 0).contiguous(),
                         down=W(m + "down", (D, L.ff)))
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
        shapes = {i: (L.delta.heads, L.delta.dim, L.delta.dim) for i, L in enumerate(self.cfg.layers) if L.delta}
        return SlotState(slots, shapes, self.device) if shapes else None

    # ------------------------------------------------------------------ one step
    def _rms(self, out, x, w, rows_idx=None, rows=None):
        n = x.shape[0] if rows is None else rows
        cabi.check(cabi.lib().pg_group_rmsnorm(ptr(out), ptr(x), None, 0, None, 0, ptr(w), ptr(rows_idx), n, self.cfg.width,
                                               1, self.cfg.eps, self.dt, cabi.stream()), "rmsnorm")

    def _post(self, out, x, y, w_post, scale, w_next):
        """x += scale * RMS(y) w_post; out = RMS(x) w_next (when there is a next sublayer in this step)."""
        cabi.check(cabi.lib().pg_postnorm_residual(ptr(out) if w_next is not None else None, ptr(x), ptr(y), y.stride(0),
                                                   ptr(w_post), ptr(scale), ptr(w_next), x.shape[0], self.cfg.width,
                                                   self.cfg.eps, self.dt, cabi.stream()), "postnorm_residual")

    def _attend(self, kv, inp: StepInputs, li: int, a: AttnCfg, w: dict, proj, att, v_first, ld_vf) -> None:
        """Rotary positions + cache append + attention of one attention mixer; the result goes to att[:, :heads*vdim]."""
        L, st, tm, T = cabi.lib(), cabi.stream(), self._tm, inp.T
        at = w["at"]
        q = self._new(T, w["nq"])
        kp, vp = self.k_pools[li], self.v_pools[li]
        with tm("rotary_append"):
            cabi.check(L.pg_rotary_append(ptr(q), ptr(proj), proj.stride(0), at["q"], a.heads, at["k"], a.kv_heads, a.dim,
                                          at["v"], a.vdim, ptr(w.get("qb")), ptr(w.get("kb")), ptr(w.get("vb")),
                                          ptr(w["freq"]), a.rot.dims if a.rot else 0, w["mag"], 1, v_first, ld_vf,
                                          w.get("lam", 0.0), ptr(kp), ptr(vp), ptr(kv.page_table), kv.max_pages,
                                          self.page_size, ptr(inp.slot), ptr(inp.pos), T, self.dt, st), "rotary_append")
        gate = proj[:, at["g"]:] if a.sigmoid else None
        out_scale = w.get("left_scale", 1.0)
        with tm("sigmoid_attention" if a.sigmoid else "attention"):
            if inp.n_tiles and w["attn_tc"]:
                cabi.check(L.pg_attention_ragged_tc_ex(
                    ptr(att), att.stride(0), ptr(q), q.stride(0), ptr(gate), proj.stride(0), 1 if a.sigmoid else 0, ptr(kp),
                    ptr(vp), self.num_pages * self.page_size, ptr(kv.page_table), kv.max_pages, self.page_size,
                    ptr(inp.tiles), inp.n_tiles, T, a.heads, a.kv_heads, a.dim, a.vdim, a.scale, a.window, a.keep_first,
                    None, 1 if a.sigmoid else 0, ptr(w.get("pb")), out_scale, ptr(self.err_flag), self.dt, st),
                    "attention_ragged_tc")
            else:
                cabi.check(L.pg_attention_ragged_ex(
                    ptr(att), att.stride(0), ptr(q), q.stride(0), ptr(gate), proj.stride(0), 1 if a.sigmoid else 0, ptr(kp),
                    ptr(vp), ptr(kv.page_table), kv.max_pages, self.page_size, ptr(inp.slot), ptr(inp.pos), T, a.heads,
                    a.kv_heads, a.dim, a.vdim, a.scale, a.window, a.keep_first, None, 1 if a.sigmoid else 0,
                    ptr(w.get("pb")), out_scale, ptr(self.attn_ws), self.attn_ws.numel(), self.dt, st), "attention_ragged")

    def _recur(self, kv, inp: StepInputs, li: int, lc: LayerCfg, w: dict, proj, att) -> None:
        """The delta-rule branch: decay / removal / unit key, the recurrence from the slots' states, head norm and
        gate; the result (times the branch scale) goes to att[:, r_col:]."""
        L, st, tm, T, d, at = cabi.lib(), cabi.stream(), self._tm, inp.T, lc.delta, w["at"]
        nd = w["nd"]
        if kv.state is None or li not in kv.state.layers:
            raise RuntimeError("this step's slot table carries no recurrent state for the model's recurrent layers")
        rec = self._new(int(L.pg_delta_record_floats(T, d.heads, d.dim)), dtype=torch.float32)
        with tm("delta_prep"):
            cabi.check(L.pg_delta_prep(ptr(rec), ptr(proj), proj.stride(0), at["rr"], at["rk"], at["rv"], at["ra"], at["rw1"],
                                       w["lora"], ptr(w["w2"]), ptr(w["w0"]), ptr(w["ab"]), T, d.heads, d.dim, DECAY_SCALE,
                                       KEY_EPS, self.dt, st), "delta_prep")
        o = self._new(T, nd, dtype=torch.float32)
        with tm("delta_rule"):
            cabi.check(L.pg_delta_rule(ptr(o), ptr(kv.state.layers[li]), ptr(rec), ptr(inp.segs), inp.n_segs, d.heads, d.dim,
                                       st), "delta_rule")
        with tm("headnorm_gate"):
            cabi.check(L.pg_headnorm_gate(ptr(att[:, w["r_col"]:]), att.stride(0), ptr(o), ptr(w["rnorm"]),
                                          ptr(proj[:, at["rg"]:]), proj.stride(0), T, d.heads, d.dim, self.cfg.eps,
                                          lc.right_scale, self.dt, st), "headnorm_gate")

    def _forward_device(self, kv, inp: StepInputs, layer_sink: Optional[list]) -> torch.Tensor:
        c, L, st, tm = self.cfg, cabi.lib(), cabi.stream(), self._tm
        T, nw, D = inp.T, inp.nw, self.cfg.width
        x = self._new(T, D, dtype=torch.float32)
        cabi.check(L.pg_embed_pos(ptr(x), ptr(inp.ids), None, ptr(self.emb), None, T, D, c.vocab, 0, 1.0, ptr(self.err_flag),
                                  self.dt, st), "embed")
        h = self._new(T, D)
        with tm("norm"):
            self._rms(h, x, self.layers[0]["norm1"])
        projs: Dict[int, torch.Tensor] = {}       # fused projections of the layers whose values later layers mix in
        n_layers = len(c.layers)
        for li, (lc, w) in enumerate(zip(c.layers, self.layers)):
            a = lc.attn
            with tm("proj"):
                proj = self._linear(h, w["proj"])
            if lc.kind == "attention":
                if a.v_mix and w["mix_from"] is None:
                    projs[li] = proj
                src = w["mix_from"]
                vf = None if src is None else projs[src][:, self.layers[src]["at"]["v"]:]
                att = self._new(T, w["att_cols"])
                self._attend(kv, inp, li, a, w, proj, att, ptr(vf), 0 if vf is None else vf.stride(0))
            else:
                att = (torch.zeros if w["att_pad"] else torch.empty)((T, w["att_cols"]), dtype=self.dtype, device=self.device)
                self._attend(kv, inp, li, a, w, proj, att, None, 0)
                self._recur(kv, inp, li, lc, w, proj, att)
            with tm("o"):
                y = self._linear(att, w["o"])
            nxt = self.layers[li + 1]["norm1"] if li + 1 < n_layers else None
            if lc.ff:
                with tm("post_norm"):
                    self._post(h, x, y, w["norm1b"], w["ls1"], w["norm2"])
                with tm("gate_up"):
                    act = self._linear(h, w["gu"], cabi.EPI_GEGLU)
                with tm("down"):
                    y = self._linear(act, w["down"])
                with tm("post_norm"):
                    self._post(h, x, y, w["norm2b"], w["ls2"], nxt)
            else:
                with tm("post_norm"):
                    self._post(h, x, y, w["norm1b"], w["ls1"], nxt)
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
        for w in self.layers:
            n += sum(t.numel() for t in w.values() if isinstance(t, torch.Tensor) and t.dtype == self.dtype)
        return n * torch.tensor([], dtype=self.dtype).element_size()
