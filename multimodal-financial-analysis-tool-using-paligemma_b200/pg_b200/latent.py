"""Latent attention as a mixer that several designs share: low-rank query and key/value latents, one rotated key part
shared by the heads, an optional softmax sink, sliding window and output gate.

    c_q = RMS(Wdq h) w_dq, q = Wuq c_q, per head [dim plain | rot_dim rotated];
    [a ; r] = Wdkv h: c = RMS(a) w_dkv (kv_rank), k_rot = rotary(r) shared by all heads;
    per head K = Wuk c, V = Wuv c; score(i, j) = scale (q_plain . K_j + rotary(q_rot) . k_rot,j) for the visible j
    (j <= i, and i - j < window when there is one); softmax whose denominator also holds exp(sink_h) when the design
    has sinks; Wo (concat_h(P_h V) [* sigmoid(Wg h)]).

Only [c | k_rot] is cached; attention runs in the latent space (Wuk folded into the queries, Wuv applied to the
attended latents), i.e. as attention with ONE key/value head of width kv_rank + rot_dim.

`pack_latent` repacks a layer's tensors (one fused projection [dq; dkv; g], Wuk per head transposed, the rotary table);
`LatentAttentionMixin._latent` is the launch sequence on a ragged token batch.  The engine that mixes it in owns the
latent pool of every layer run and hands it in.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from . import _cabi as cabi
from ._cabi import ptr
from .ragged_engine import RotaryCfg, StepInputs, _stack_rows


@dataclass
class LatentCfg:
    heads: int
    dim: int                      # plain (unrotated) query / key columns per head
    rot_dim: int                  # rotated columns per head (one key part shared by the heads)
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    rot: Optional[RotaryCfg]
    window: int = 0               # 0 = every earlier position


def latent_cfg(i: int, m, window: int = 0) -> LatentCfg:
    """The mixer's sizes from its config entry (layer i, for messages)."""
    rot_dim = int(m["rot_dim"])
    rot = m.get("rot") or {}
    rc = RotaryCfg(int(rot.get("dims", rot_dim)), float(rot["base"]), rot.get("scaling")) if rot_dim else None
    if rc is not None and (rc.dims != rot_dim or rot_dim % 2):
        raise ValueError(f"layer {i}: {rc.dims} rotary columns for a rotated part of {rot_dim}")
    return LatentCfg(int(m["heads"]), int(m["dim"]), rot_dim, int(m["vdim"]), int(m["q_rank"]), int(m["kv_rank"]),
                     float(m["scale"]), rc, int(window))


def pack_latent(W, m: str, a: LatentCfg, D: int, device, dtype, gated: bool, sink: bool = True) -> dict:
    """The repacked tensors of one latent mixer; W(name, shape, dtype=None) fetches a checked tensor, m = its prefix."""
    import torch
    hq, hv = a.heads * (a.dim + a.rot_dim), a.heads * a.vdim
    parts = [("dq", W(m + "dq", (a.q_rank, D))), ("dkv", W(m + "dkv", (a.kv_rank + a.rot_dim, D)))]
    if gated:
        parts.append(("g", W(m + "g", (hv, D))))
    w = {}
    w["proj"], w["at"] = _stack_rows(parts, device, dtype)
    # Wuk per head, transposed: the query of a head is taken into the latent space by [kv_rank, dim]
    uk_t = W(m + "uk", (a.heads * a.dim, a.kv_rank)).view(a.heads, a.dim, a.kv_rank).transpose(1, 2).contiguous()
    w.update(dq_norm=W(m + "dq.norm", (a.q_rank,)), dkv_norm=W(m + "dkv.norm", (a.kv_rank,)),
             uq=W(m + "uq", (hq, a.q_rank)), uk_t=uk_t, uv=W(m + "uv", (hv, a.kv_rank)),
             sink=W(m + "sink", (a.heads,), torch.float32) if sink else None, o=W(m + "o", (D, hv)),
             ld_pool=(a.kv_rank + a.rot_dim + 7) // 8 * 8, gated=gated)
    if a.rot is not None:
        f, mag = a.rot.table()
        w["freq"], w["mag"] = f.to(torch.float32).to(device), float(mag)
    else:
        w["freq"], w["mag"] = None, 1.0
    return w


class LatentAttentionMixin:
    """For engines built on RaggedEngine (uses its `_linear`, `_new`, `_tm`, `cfg.eps`, `err_flag`, `attn_ws`)."""

    head_impl = 0                 # per-head products: 0 = tensor cores where they fit, 1 = fp32 FMA

    def _latent_tc_ok(self, a: LatentCfg) -> bool:
        """Prompt portions of this mixer can run on the tensor-core attention kernel."""
        return bool(cabi.lib().pg_attention_ragged_tc_ok(
            a.kv_rank + a.rot_dim, a.kv_rank, self.page_size, a.heads * (a.kv_rank + a.rot_dim), a.heads * a.kv_rank, 8,
            self.dt))

    def _per_head(self, out, o_hs: int, a, a_hs: int, w, gate, heads: int, N: int, K: int) -> None:
        """out[t, h * o_hs + n] = sum_k a[t, h * a_hs + k] w[h, n, k] (* sigmoid(gate[t, h * N + n])) for every head:
        prompt-sized 16-bit steps as ONE launch of the experts' grouped tensor-core GEMM with the heads as its groups,
        a handful of rows, fp32 and sizes that kernel does not take on the per-head kernels of the latent-attention file."""
        cabi.check(cabi.lib().pg_head_gemm_ex(ptr(out), out.stride(0), o_hs, ptr(a), a.stride(0), a_hs, ptr(w), ptr(gate),
                                              0 if gate is None else gate.stride(0), a.shape[0], heads, N, K, self.head_impl,
                                              ptr(self.err_flag), self.dt, cabi.stream()), "head_gemm")

    def _latent(self, kv, inp: StepInputs, pool, a: LatentCfg, w: dict, h):
        L, st, tm, T, at = cabi.lib(), cabi.stream(), self._tm, inp.T, w["at"]
        ldp = w["ld_pool"]
        with tm("proj"):
            proj = self._linear(h, w["proj"])
        cq = self._new(T, a.q_rank)
        with tm("latent_prep"):
            cabi.check(L.pg_latent_prep(ptr(cq), ptr(proj), proj.stride(0), at["dq"], a.q_rank, ptr(w["dq_norm"]), at["dkv"],
                                        a.kv_rank, ptr(w["dkv_norm"]), a.rot_dim, ptr(w["freq"]), w["mag"], self.cfg.eps,
                                        ptr(pool), ldp, ptr(kv.page_table), kv.max_pages, self.page_size, ptr(inp.slot),
                                        ptr(inp.pos), T, self.dt, st), "latent_prep")
        with tm("q_up"):
            q = self._linear(cq, w["uq"])
        hd, ld_q = a.dim + a.rot_dim, a.kv_rank + a.rot_dim
        qa = self._new(T, a.heads * ld_q)
        with tm("q_absorb"):
            self._per_head(qa, ld_q, q, hd, w["uk_t"], None, a.heads, a.kv_rank, a.dim)
            cabi.check(L.pg_rotary_cols(ptr(qa), qa.stride(0), a.kv_rank, ld_q, ptr(q), q.stride(0), a.dim, hd, a.heads,
                                        a.rot_dim, ptr(w["freq"]), w["mag"], ptr(inp.pos), T, self.dt, st), "rotary_cols")
        ol = self._new(T, a.heads * a.kv_rank)
        with tm("latent_attention"):
            if inp.n_tiles and w["attn_tc"]:
                cabi.check(L.pg_attention_ragged_tc_sink(
                    ptr(ol), ol.stride(0), ptr(qa), qa.stride(0), None, 0, 0, ptr(pool), ldp, ptr(pool), ldp,
                    self.num_pages * self.page_size, ptr(kv.page_table), kv.max_pages, self.page_size, ptr(inp.tiles),
                    inp.n_tiles, T, a.heads, 1, ld_q, a.kv_rank, a.scale, a.window, 0, None, 0, None, ptr(w["sink"]), 1.0,
                    ptr(self.err_flag), self.dt, st), "attention_ragged_tc_sink")
            else:
                cabi.check(L.pg_attention_ragged_sink(
                    ptr(ol), ol.stride(0), ptr(qa), qa.stride(0), None, 0, 0, ptr(pool), ldp, ptr(pool), ldp,
                    ptr(kv.page_table), kv.max_pages, self.page_size, ptr(inp.slot), ptr(inp.pos), T, a.heads, 1, ld_q,
                    a.kv_rank, a.scale, a.window, 0, None, 0, None, ptr(w["sink"]), 1.0, ptr(self.attn_ws),
                    self.attn_ws.numel(), self.dt, st), "attention_ragged_sink")
        att = self._new(T, a.heads * a.vdim)
        with tm("v_up_gate" if w["gated"] else "v_up"):
            self._per_head(att, a.vdim, ol, a.kv_rank, w["uv"], proj[:, at["g"]:] if w["gated"] else None, a.heads, a.vdim,
                           a.kv_rank)
        with tm("o"):
            return self._linear(att, w["o"])
