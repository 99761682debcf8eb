"""Gogivik: a decoder-only language model whose layers mix tokens by latent attention in a sliding window with a
softmax sink, by block-masked attention with per-head query / key norms, normed and rotated values, or by a selective
state-space recurrence; every sublayer reads its input through a short causal convolution over time.

Design (every size and every constant that can differ between checkpoints comes from config.json):

  x_0[t]     = embed[token_t]                                                fp32 residual stream
  layer      : x <- x + Mixer(C1(N1(x))) ;  x <- x + FF(C2(N2(x)))           (FF may be absent)
  N(x)       = x / sqrt(mean(x^2) + eps) * (1 + w)                           the weight is stored around zero
  C(h)_t     = h_t + sum_j k[:, j] h_(t - taps + 1 + j)                      per channel, zeros before the sequence; the
                                                                             last taps - 1 normed rows are sequence state
  latent     : `latent.py` with a window (i - j < mask.size), a sink per head, no gate, rotary pairs (2i, 2i+1).
  attention  : q, k, v = Wq h, Wk h, Wv h (H query heads over G key/value heads); q, k: RMS per head times a weight of
               `dim` entries shared by the heads, then rotary on the first rot.dims columns, pairs (i, i + dims/2),
               frequencies base^(-2i/dims) divided by rot.scaling.factor; v: RMS per head without a weight, then
               rotated over all vdim columns by its own position (pairs (m, m + vdim/2), base^(-2m/vdim), unscaled) and
               cached so; key j is visible to query i when j <= i and floor(i / mask.size) = floor(j / mask.size);
               softmax(scale q.k); each head's sum over the values is turned back by -i; Wo.
  mamba2     : [z | x | B | C | dt] = Win h; x, B, C: causal convolution (taps, bias) + silu; step = softplus(dt + dt_bias);
               per head (groups of heads share B, C): S_t = exp(-exp(A_log) step) S_(t-1) + step B_t x_t^T,
               y_t = S_t^T C_t + D x_t; Wo (RMS in norm_groups parts of (y * silu(z)) * w).  S (fp32) and the
               convolution's last taps - 1 inputs are sequence state.
  ff dense   : Wdown relu(Wup h)^2
  output     : logits = logit_scale * Whead N_final(x)

fp32: the residual stream, every norm, the input convolutions' sums, positions and angles, attention scores and weights,
the turning back of the attention output, the recurrence with its step sizes, decays and state, the gated norm.
Model dtype (fp32 accumulation): projections, caches, the feed-forward.

The engine owns the repacked weights, one paged latent pool per latent layer, one paged key / value pool pair per
attention layer and, through the scheduler's slot table, the per-sequence state: [taps - 1, width] normed rows per
sublayer, [conv - 1, channels] projected inputs and [heads, state, vdim] per state-space layer.  The step function,
page pool, scheduler and sampling are the framework's (`ragged_engine.RaggedEngine`, `scheduler.SlotKV` / `SlotState`
/ `RaggedBatcher`); latent attention is the mixer Birizen uses (`latent.LatentAttentionMixin`), the recurrence runs on
the decayed linear-attention kernel with a decay per token.
"""
from __future__ import annotations

import os
import warnings
from dataclasses import dataclass, field
from typing import Dict, List, Mapping, Optional

import torch

from . import _cabi as cabi
from ._cabi import ptr
from .latent import LatentAttentionMixin, LatentCfg, latent_cfg, pack_latent
from .ragged_engine import RaggedEngine, RotaryCfg, StepInputs, _stack_rows
from .registry import register


@dataclass
class BlockAttnCfg:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: Optional[RotaryCfg]
    rot_base: float                 # the values turn with this base over all of vdim, never scaled
    chunk: int                      # 0 = every earlier position


@dataclass
class SsmCfg:
    heads: int
    vdim: int
    state: int
    groups: int
    norm_groups: int
    taps: int

    @property
    def inner(self) -> int:
        return self.heads * self.vdim

    @property
    def channels(self) -> int:      # what passes the convolution: x, B, C
        return self.inner + 2 * self.groups * self.state


@dataclass
class LayerCfg:
    kind: str                       # "latent_attention" | "attention" | "mamba2"
    mixer: object
    ff: int = 0                     # 0 = no feed-forward


@dataclass
class GogivikConfig:
    vocab: int
    width: int
    eps: float
    taps: int                       # of the input convolutions
    logit_scale: float
    layers: List[LayerCfg] = field(default_factory=list)

    @staticmethod
    def from_dict(cfg: Mapping) -> "GogivikConfig":
        layers = []
        for i, L in enumerate(cfg["layers"]):
            m, kind = L["mixer"], L.get("type")
            ml = L.get("mlp")
            if ml is not None and ml.get("kind") != "dense":
                raise ValueError(f"layer {i}: unknown feed-forward kind {ml.get('kind')!r}")
            ff = int(ml["ff"]) if ml else 0
            mask = m.get("mask") or {}
            if kind == "latent_attention":
                mixer = latent_cfg(i, m, window=int(mask.get("size", 0) or 0))
            elif kind == "attention":
                heads, rot = int(m["heads"]), m.get("rot")
                mixer = BlockAttnCfg(heads=heads, kv_heads=int(m.get("kv_heads", heads)), dim=int(m["dim"]),
                                     vdim=int(m.get("vdim", m["dim"])), scale=float(m["scale"]),
                                     rot=RotaryCfg(int(rot["dims"]), float(rot["base"]), rot.get("scaling")) if rot else None,
                                     rot_base=float(rot["base"]) if rot else 0.0, chunk=int(mask.get("size", 0) or 0))
                if mixer.heads % mixer.kv_heads:
                    raise ValueError(f"layer {i}: {mixer.heads} heads over {mixer.kv_heads} key/value heads")
                if mixer.rot and (mixer.rot.dims % 2 or mixer.rot.dims > mixer.dim or mixer.vdim % 2):
                    raise ValueError(f"layer {i}: {mixer.rot.dims} rotated columns of {mixer.dim}, values of {mixer.vdim}")
            elif kind == "mamba2":
                mixer = SsmCfg(heads=int(m["heads"]), vdim=int(m["vdim"]), state=int(m["state"]), groups=int(m.get("groups", 1)),
                               norm_groups=int(m.get("norm_groups", 1)), taps=int(m["conv"]))
                if mixer.heads % mixer.groups or mixer.inner % mixer.norm_groups or mixer.taps < 1:
                    raise ValueError(f"layer {i}: {mixer.heads} heads in {mixer.groups} groups, norm in {mixer.norm_groups} "
                                     f"parts, {mixer.taps} taps")
            else:
                raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
            layers.append(LayerCfg(kind, mixer, ff))
        taps = int((cfg.get("canon") or {}).get("taps", 1))
        if taps < 1:
            raise ValueError(f"input convolutions of {taps} taps")
        return GogivikConfig(vocab=int(cfg["vocab"]), width=int(cfg["width"]), eps=float((cfg.get("norm") or {})["eps"]),
                             taps=taps, logit_scale=float(cfg.get("logit_scale", 1.0)), layers=layers)


@register("Gogivik")
class GogivikEngine(LatentAttentionMixin, RaggedEngine):
    """Weights + paged pools + per-sequence state shapes + the launch sequence of one step over a ragged token batch."""

    needs_segments = True           # every sublayer's input convolution keeps state per sequence

    def __init__(self, config, weights: Mapping[str, torch.Tensor], *, device="cuda", dtype=torch.bfloat16,
                 page_size: int = 64, kv_pool_tokens: int = 65536, gemm_impl: int = 0, strict: bool = False):
        self.cfg = config if isinstance(config, GogivikConfig) else GogivikConfig.from_dict(config)
        self.strict = bool(strict)      # True: tensors the config does not call for raise instead of being reported
        self._init_common(device=device, dtype=dtype, page_size=page_size, gemm_impl=gemm_impl)
        # residual sum + norm + input convolution as one kernel (0: the three separate kernels, for comparison)
        self.fused_read = os.environ.get("PG_GOGIVIK_FUSED_READ", "1") != "0"
        self._repack(weights)
        L_ = cabi.lib()
        for w, lc in zip(self.layers, self.cfg.layers):
            a = lc.mixer
            if lc.kind == "latent_attention":
                w["attn_tc"] = self._latent_tc_ok(a)
            elif lc.kind == "attention":
                w["attn_tc"] = bool(L_.pg_attention_ragged_tc_ok(a.dim, a.vdim, self.page_size, a.heads * a.dim,
                                                                 a.heads * a.vdim, 8, self.dt))
            else:
                w["attn_tc"] = False
        self._attn_tc_any = any(w["attn_tc"] for w in self.layers)
        self._init_runtime(kv_pool_tokens)
        self.c_pools: Dict[int, torch.Tensor] = {}
        self.k_pools: Dict[int, torch.Tensor] = {}
        self.v_pools: Dict[int, torch.Tensor] = {}
        for i, (lc, w) in enumerate(zip(self.cfg.layers, self.layers)):
            a = lc.mixer
            if lc.kind == "latent_attention":
                self.c_pools[i] = torch.zeros((self.num_pages, self.page_size, w["ld_pool"]), dtype=dtype, device=self.device)
            elif lc.kind == "attention":
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

        f32 = torch.float32
        self.emb, self.final_norm, self.head = W("embed", (c.vocab, D)), W("final.norm", (D,)), W("head", (c.vocab, D))
        self.layers: List[dict] = []
        for i, L in enumerate(c.layers):
            p, m, a = f"l{i}.", f"l{i}.mix.", L.mixer
            w = dict(norm1=W(p + "norm1", (D,)), canon1=W(p + "canon1", (D, c.taps)))
            if L.kind == "latent_attention":
                w.update(pack_latent(W, m, a, D, self.device, self.dtype, gated=False))
            elif L.kind == "attention":
                nq, nk, nv = a.heads * a.dim, a.kv_heads * a.dim, a.kv_heads * a.vdim
                w["proj"], w["at"] = _stack_rows([("q", W(m + "q", (nq, D))), ("k", W(m + "k", (nk, D))),
                                                  ("v", W(m + "v", (nv, D)))], self.device, self.dtype)
                w.update(q_norm=W(m + "q.norm", (a.dim,)), k_norm=W(m + "k.norm", (a.dim,)), o=W(m + "o", (D, a.heads * a.vdim)),
                         freq=None, v_freq=None)
                if a.rot:
                    w["freq"] = a.rot.table()[0].to(f32).to(self.device)
                    w["v_freq"] = RotaryCfg(a.vdim, a.rot_base).table()[0].to(f32).to(self.device)
            else:
                n_in = 2 * a.inner + 2 * a.groups * a.state + a.heads
                w.update(proj=W(m + "in", (n_in, D)), conv=W(m + "conv", (a.channels, a.taps)), conv_b=W(m + "conv.b", (a.channels,)),
                         dt_bias=W(m + "dt_bias", (a.heads,), f32), a_log=W(m + "A_log", (a.heads,), f32),
                         skip=W(m + "D", (a.heads,), f32), gnorm=W(m + "norm", (a.inner,)), o=W(m + "o", (D, a.inner)))
            if L.ff:
                f = p + "mlp."
                w.update(norm2=W(p + "norm2", (D,)), canon2=W(p + "canon2", (D, c.taps)), up=W(f + "up", (L.ff, D)),
                         down=W(f + "down", (D, L.ff)))
            self.layers.append(w)
        extra = sorted(set(weights) - used)
        if extra:
            text = f"checkpoint holds {len(extra)} tensor(s) the config does not call for: {extra[:8]}"
            if self.strict:
                raise ValueError(text)
            warnings.warn(text + " (not used)")

    # ------------------------------------------------------------------ per-sequence state
    def new_slot_state(self, slots: int):
        from .scheduler import SlotState
        c, shapes = self.cfg, {}
        for i, L in enumerate(c.layers):
            if c.taps > 1:
                shapes[("canon1", i)] = (c.taps - 1, c.width)
                if L.ff:
                    shapes[("canon2", i)] = (c.taps - 1, c.width)
            if L.kind == "mamba2":
                a = L.mixer
                shapes[("ssm", i)] = (a.heads, a.state, a.vdim)
                if a.taps > 1:
                    shapes[("conv", i)] = (a.taps - 1, a.channels)
        return SlotState(slots, shapes, self.device)

    # ------------------------------------------------------------------ one step
    def _read(self, kv, inp: StepInputs, key, x, x_alt, y, w_norm, w_conv):
        """What a sublayer reads: x += y (the sublayer output not yet summed in; None: nothing), n = N(x) in fp32,
        h = n + conv(n) over the sequence's positions, the state of the sequence brought up to this step's end.  Returns
        (h, the stream, the spare stream buffer): the fused kernel writes the sum into the spare buffer (a tile re-reads
        rows that its neighbour owns), so the two change places."""
        L, st, tm, c = cabi.lib(), cabi.stream(), self._tm, self.cfg
        T, D = x.shape
        h = self._new(T, D)
        state = kv.state.layers[key] if c.taps > 1 else None
        if self.fused_read and c.taps <= 8:
            with tm("norm_conv"):
                cabi.check(L.pg_norm_time_conv(ptr(h), ptr(x_alt), ptr(x), ptr(y), 0 if y is None else y.stride(0), ptr(w_norm), 1,
                                               c.eps, ptr(w_conv), ptr(state), ptr(inp.slot), ptr(inp.segs), inp.n_segs, T, D,
                                               c.taps, self.dt, st), "norm_time_conv")
            return h, x_alt, x
        n = self._new(T, D, dtype=torch.float32)
        with tm("norm"):
            cabi.check(L.pg_group_rmsnorm_ex(ptr(n), ptr(x), ptr(y), 0 if y is None else y.stride(0), None, 0, ptr(w_norm),
                                             None, T, D, 1, c.eps, 1, 1, self.dt, st), "rmsnorm")
        with tm("input_conv"):
            cabi.check(L.pg_time_conv_residual(ptr(h), ptr(n), ptr(w_conv), ptr(state), ptr(inp.slot), T, D, c.taps,
                                               self.dt, st), "time_conv_residual")
            if state is not None:
                cabi.check(L.pg_time_conv_state(ptr(state), ptr(n), D, 0, 1, ptr(inp.segs), inp.n_segs, D, c.taps, self.dt,
                                                st), "time_conv_state")
        return h, x, x_alt

    def _attention(self, kv, inp: StepInputs, li: int, a: BlockAttnCfg, w: dict, h) -> torch.Tensor:
        L, st, tm, T, at = cabi.lib(), cabi.stream(), self._tm, inp.T, w["at"]
        with tm("proj"):
            proj = self._linear(h, w["proj"])
        q = self._new(T, a.heads * a.dim)
        kp, vp = self.k_pools[li], self.v_pools[li]
        with tm("headnorm_rotary_append"):
            cabi.check(L.pg_headnorm_rotary_append(ptr(q), ptr(proj), proj.stride(0), at["q"], a.heads, at["k"], a.kv_heads,
                                                   a.dim, at["v"], a.vdim, ptr(w["q_norm"]), ptr(w["k_norm"]), self.cfg.eps,
                                                   ptr(w["freq"]), a.rot.dims if a.rot else 0, 0, 1, ptr(w["v_freq"]), 0,
                                                   ptr(kp), ptr(vp), ptr(kv.page_table), kv.max_pages, self.page_size,
                                                   ptr(inp.slot), ptr(inp.pos), T, self.dt, st), "headnorm_rotary_append")
        att = self._new(T, a.heads * a.vdim)
        with tm("attention"):
            if inp.n_tiles and w["attn_tc"]:
                cabi.check(L.pg_attention_ragged_tc_masked(
                    ptr(att), att.stride(0), ptr(q), q.stride(0), None, 0, 0, ptr(kp), 0, ptr(vp), 0,
                    self.num_pages * self.page_size, ptr(kv.page_table), kv.max_pages, self.page_size, ptr(inp.tiles),
                    inp.n_tiles, T, a.heads, a.kv_heads, a.dim, a.vdim, a.scale, 0, 0, a.chunk, None, 0, None, None,
                    ptr(w["v_freq"]), 0, 1.0, ptr(self.err_flag), self.dt, st), "attention_ragged_tc_masked")
            else:
                cabi.check(L.pg_attention_ragged_masked(
                    ptr(att), att.stride(0), ptr(q), q.stride(0), None, 0, 0, ptr(kp), 0, ptr(vp), 0, ptr(kv.page_table),
                    kv.max_pages, self.page_size, ptr(inp.slot), ptr(inp.pos), T, a.heads, a.kv_heads, a.dim, a.vdim,
                    a.scale, 0, 0, a.chunk, None, 0, None, None, ptr(w["v_freq"]), 0, 1.0, ptr(self.attn_ws),
                    self.attn_ws.numel(), self.dt, st), "attention_ragged_masked")
        with tm("o"):
            return self._linear(att, w["o"])

    def _ssm(self, kv, inp: StepInputs, li: int, a: SsmCfg, w: dict, h) -> torch.Tensor:
        L, st, tm, T = cabi.lib(), cabi.stream(), self._tm, inp.T
        with tm("proj"):
            proj = self._linear(h, w["proj"])
        conv_state = kv.state.layers[("conv", li)] if a.taps > 1 else None
        rec = self._new(int(L.pg_ssm_record_floats(T, a.heads, a.vdim, a.state)), dtype=torch.float32)
        with tm("ssm_prep"):
            cabi.check(L.pg_ssm_prep(ptr(rec), ptr(proj), proj.stride(0), a.inner, a.inner + a.channels, ptr(w["conv"]),
                                     ptr(w["conv_b"]), ptr(conv_state), ptr(w["dt_bias"]), ptr(w["a_log"]), ptr(inp.slot), T,
                                     a.heads, a.vdim, a.state, a.groups, a.taps, self.dt, st), "ssm_prep")
            if conv_state is not None:
                cabi.check(L.pg_time_conv_state(ptr(conv_state), ptr(proj), proj.stride(0), a.inner, 0, ptr(inp.segs),
                                                inp.n_segs, a.channels, a.taps, self.dt, st), "time_conv_state")
        y = self._new(T, a.inner, dtype=torch.float32)
        with tm("ssm_scan"):
            cabi.check(L.pg_lightning_attention_ex(ptr(y), ptr(kv.state.layers[("ssm", li)]), ptr(rec), None, ptr(w["skip"]),
                                                   ptr(inp.segs), inp.n_segs, a.heads, a.state, a.vdim, st), "ssm_scan")
        g = self._new(T, a.inner)
        with tm("gate_groupnorm"):
            cabi.check(L.pg_gate_groupnorm(ptr(g), a.inner, ptr(y), ptr(proj), proj.stride(0), ptr(w["gnorm"]), T, a.inner,
                                           a.norm_groups, self.cfg.eps, self.dt, st), "gate_groupnorm")
        with tm("o"):
            return self._linear(g, w["o"])

    def _forward_device(self, kv, inp: StepInputs, layer_sink: Optional[list]) -> torch.Tensor:
        c, L, st, tm = self.cfg, cabi.lib(), cabi.stream(), self._tm
        T, nw, D = inp.T, inp.nw, self.cfg.width
        if kv.state is None:
            raise RuntimeError("this step's slot table carries no per-sequence state for the model's convolutions")
        x, x_alt = self._new(T, D, dtype=torch.float32), self._new(T, D, dtype=torch.float32)
        cabi.check(L.pg_embed_pos(ptr(x), ptr(inp.ids), None, ptr(self.emb), None, T, D, c.vocab, 0, 1.0, ptr(self.err_flag),
                                  self.dt, st), "embed")
        y = None                                            # a sublayer's output that the next norm kernel sums into x
        for li, (lc, w) in enumerate(zip(c.layers, self.layers)):
            h, x, x_alt = self._read(kv, inp, ("canon1", li), x, x_alt, y, w["norm1"], w["canon1"])
            if lc.kind == "latent_attention":
                y = self._latent(kv, inp, self.c_pools[li], lc.mixer, w, h)
            elif lc.kind == "attention":
                y = self._attention(kv, inp, li, lc.mixer, w, h)
            else:
                y = self._ssm(kv, inp, li, lc.mixer, w, h)
            if lc.ff:
                h, x, x_alt = self._read(kv, inp, ("canon2", li), x, x_alt, y, w["norm2"], w["canon2"])
                with tm("up"):
                    u = self._linear(h, w["up"])
                with tm("relu2"):
                    cabi.check(L.pg_relu2(ptr(u), ptr(u), u.numel(), self.dt, st), "relu2")
                with tm("down"):
                    y = self._linear(u, w["down"])
            if layer_sink is not None:
                cabi.check(L.pg_group_rmsnorm_ex(None, ptr(x), ptr(y), y.stride(0), None, 0, None, None, T, D, 1, c.eps, 1, 0,
                                                 self.dt, st), "residual sum")
                y = None
                layer_sink.append(x.clone())
        if y is not None:
            with tm("norm"):
                cabi.check(L.pg_group_rmsnorm_ex(None, ptr(x), ptr(y), y.stride(0), None, 0, None, None, T, D, 1, c.eps, 1, 0,
                                                 self.dt, st), "residual sum")
        if nw == 0:
            return torch.empty((0, c.vocab), dtype=torch.float32, device=self.device)
        hf = self._new(nw, D)
        with tm("norm"):
            cabi.check(L.pg_group_rmsnorm_ex(ptr(hf), ptr(x), None, 0, None, 0, ptr(self.final_norm), ptr(inp.want), nw, D, 1,
                                             c.eps, 1, 0, self.dt, st), "final norm")
        with tm("head"):
            logits = self._linear(hf, self.head, out_f32=True)
            if c.logit_scale != 1.0:
                logits.mul_(c.logit_scale)
        return logits

    def weight_bytes(self) -> int:
        n = self.emb.numel() + self.final_norm.numel() + self.head.numel()
        for w in self.layers:
            n += sum(t.numel() for t in w.values() if isinstance(t, torch.Tensor) and t.dtype == self.dtype)
        return n * torch.tensor([], dtype=self.dtype).element_size()
