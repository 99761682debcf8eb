"""Common part of the engines that serve decoder-only models on ragged token batches.

A step is a flat token list: token t carries (id, page-table row of its sequence, position in it), so prompt portions
and single decoded tokens of different sequences share every launch.  This class owns what does not depend on the
design: the page pool, the host -> device packing of a step's inputs, the CUDA-graph replay of small steps, the
projection wrapper over the library's GEMM / GEMV kernels, per-op timing and the serving glue.  A design subclasses it
with its config, its weight repacking (`_repack`), its caches and its launch sequence (`_forward_device`).

Inputs of a step on the device (one int32 buffer, `StepInputs` names its parts):

    ids (int64) | page-table row | position | wanted rows | segments | query tiles

* segments (engines with `needs_segments`: recurrent state per sequence slot): {slot, first token row, tokens} for
  every run of consecutive tokens of one sequence; steps that replay a graph pad the list with empty segments to
  min(tokens, slots) entries so that the captured launch sequence depends on the token count only;
* query tiles (steps of at least `attn_tc_min_tokens` tokens on engines whose attention has a tensor-core kernel):
  {first token row, rows, page-table row, first position} for runs of up to 128 consecutive tokens of one sequence.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from . import _cabi as cabi
from ._cabi import ptr
from .pool import PagePool


@dataclass
class StepInputs:
    T: int
    nw: int
    ids: torch.Tensor            # int64 [T]
    slot: torch.Tensor           # int32 [T]
    pos: torch.Tensor            # int32 [T]
    want: torch.Tensor           # int32 [nw]
    segs: torch.Tensor           # int32 [3 * n_segs]
    n_segs: int
    tiles: torch.Tensor          # int32 [4 * n_tiles]
    n_tiles: int


@dataclass
class RotaryCfg:
    dims: int
    base: float
    scaling: Optional[dict] = None       # YaRN: factor, original, fast, slow; linear: factor alone

    def table(self):
        """(frequencies float64 [dims / 2], magnitude): angle of pair i at position p = p * f_i; with YaRN scaling the
        slow pairs are interpolated (f / factor), the fast ones kept, a linear ramp in between, and cos / sin are
        both multiplied by 0.1 ln(factor) + 1.  A scaling entry that gives a factor alone is linear scaling: every
        frequency is divided by the factor, the magnitude stays 1."""
        i = torch.arange(self.dims // 2, dtype=torch.float64)
        f = torch.pow(torch.tensor(self.base, dtype=torch.float64), -2.0 * i / self.dims)
        mag = 1.0
        sc = self.scaling
        if sc and "original" not in sc:
            f = f / float(sc["factor"])
        elif sc:
            factor, orig = float(sc["factor"]), float(sc["original"])

            def pair_of(turns: float) -> float:     # the pair index that makes `turns` full turns over `orig` positions
                return self.dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(self.base))

            lo = max(math.floor(pair_of(float(sc["fast"]))), 0)
            hi = min(math.ceil(pair_of(float(sc["slow"]))), self.dims - 1)
            ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
            f = f / factor * ramp + f * (1.0 - ramp)
            mag = 0.1 * math.log(factor) + 1.0
        return f, mag



def _stack_rows(parts, device, dtype, align=8):
    """Concatenate [rows_i, K] matrices with every part starting at a multiple of `align` rows (zero rows between),
    so that the columns of the fused projection's output start aligned.  Returns (matrix, {name: first row})."""
    rows, at, n = [], {}, 0
    for name, t in parts:
        at[name] = n
        rows.append(t)
        n += t.shape[0]
        pad = (-n) % align
        if pad:
            rows.append(torch.zeros((pad, t.shape[1]), dtype=dtype, device=device))
            n += pad
    return torch.cat(rows, 0).contiguous(), at



class RaggedEngine(PagePool):
    """Weights + paged pools + the launch sequence of one step over a ragged token batch."""

    ragged = True                    # served by scheduler.RaggedBatcher
    needs_segments = False           # the step needs the per-sequence runs of its tokens (recurrent state)
    max_positions: Optional[int] = None   # longest sequence the design can address (None: no bound of its own)

    def _init_common(self, *, device, dtype, page_size: int, gemm_impl: int = 0) -> None:
        cabi.lib()                   # fail now if the CUDA library is missing
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("pg_b200 runs on CUDA devices only (no CPU fallback)")
        if dtype not in (torch.bfloat16, torch.float32):
            raise RuntimeError(f"unsupported model dtype {dtype} (bfloat16 or float32)")
        self.dtype, self.dt = dtype, cabi.DTYPE_CODE[dtype]
        self.vec = 4 if dtype == torch.float32 else 8
        self.page_size = int(page_size)
        self.gemm_impl = int(os.environ.get("PG_RAGGED_GEMM_IMPL", gemm_impl))
        self.small_m_gemv = os.environ.get("PG_RAGGED_GEMV", "1") != "0"
        # rows up to which a projection streams its weights through the GEMV kernel; from there on the 16-bit path
        # takes the tensor-core GEMMs (the GEMV turns ALU-bound as rows are added), fp32 keeps it to its 8-row limit
        self.gemv_max_rows = cabi.MAX_DECODE_BATCH if dtype == torch.float32 else max(1, cabi.BATCHED_DECODE_MIN - 1)
        # steps of up to this many tokens (decode steps, short portions) replay a CUDA graph captured per token count
        self.graph_max_tokens = int(os.environ.get("PG_RAGGED_GRAPH_TOKENS", "16"))
        # steps of at least this many tokens run the tcgen05 attention kernel (layers whose head sizes it takes)
        self.attn_tc_min_tokens = int(os.environ.get("PG_RAGGED_ATTN_TC_MIN", "48"))
        self._attn_tc_any = False
        # expert GEMMs: 0 = tensor cores where the sizes allow, 1 = the fp32-FMA kernel; pairs from which they are taken
        self.moe_impl = int(os.environ.get("PG_MOE_IMPL", "0"))
        self.moe_tc_min_pairs = int(os.environ.get("PG_MOE_TC_MIN_PAIRS", "1"))
        self._graphs: Dict[tuple, tuple] = {}
        self._op_timing = os.environ.get("PG_OP_TIMING", "0") == "1"
        self._op_events: List[tuple] = []

    def _init_runtime(self, kv_pool_tokens: int) -> None:
        """Page pool, error flag, attention scratch and the GEMM workspace (after the weights are in place)."""
        # +1: the scheduler parks the unused page-table entries on a page of their own
        self._init_pool((int(kv_pool_tokens) + self.page_size - 1) // self.page_size + 1)
        self.err_flag = torch.zeros(1, dtype=torch.int32).pin_memory()
        self._err_np = self.err_flag.numpy()
        self.attn_ws = torch.empty(5 << 19, dtype=torch.float32, device=self.device)   # key-slice partials of decode steps
        if self.dtype != torch.float32:   # scratch of the split-K prompt GEMMs (shared with the other engines)
            from .engine import _WORKSPACES
            key = (self.device.index,)
            if key not in _WORKSPACES:
                _WORKSPACES[key] = torch.empty(int(os.environ.get("PG_WORKSPACE_MB", "80")) << 20, dtype=torch.uint8,
                                               device=self.device)
            ws = _WORKSPACES[key]
            cabi.check(cabi.lib().pg_set_workspace(ptr(ws), ws.numel()), "set_workspace")

    @classmethod
    def from_checkpoint(cls, config, tensors, *, device="cuda", dtype=torch.bfloat16, **kw):
        return cls(config, tensors, device=device, dtype=dtype, **kw)

    # ------------------------------------------------------------------ op wrappers
    def _new(self, *shape, dtype=None):
        return torch.empty(shape, dtype=dtype or self.dtype, device=self.device)

    def _linear(self, a: torch.Tensor, w: torch.Tensor, epi: int = cabi.EPI_NONE, out_f32: bool = False) -> torch.Tensor:
        """out = a w^T (+ the gated pairing of stacked [Wg; Wu] weights), rounded to the model dtype."""
        M, K = a.shape
        N = w.shape[0] // 2 if epi in (cabi.EPI_GEGLU, cabi.EPI_SWIGLU) else w.shape[0]
        out = self._new(M, N, dtype=torch.float32 if out_f32 else None)
        L, st = cabi.lib(), cabi.stream()
        if self.small_m_gemv and M <= self.gemv_max_rows and K % self.vec == 0 and a.is_contiguous():
            # a handful of rows (decode steps): the weight-streaming GEMV kernel of the decode path; the gated pairing
            # and the fp32 copy of the logits (rounded to the model dtype first, as the GEMM epilogue does) follow
            if epi == cabi.EPI_NONE:
                tmp = self._new(M, N) if out_f32 else out
                cabi.check(L.pg_gemv_res(ptr(tmp), ptr(a), ptr(w), None, M, N, K, None, self.dt, st), "gemv")
                if out_f32:
                    out.copy_(tmp)
                return out
            if epi in (cabi.EPI_SWIGLU, cabi.EPI_GEGLU) and not out_f32:
                gu = self._new(M, 2 * N)
                cabi.check(L.pg_gemv_res(ptr(gu), ptr(a), ptr(w), None, M, 2 * N, K, None, self.dt, st), "gemv")
                pair = L.pg_swiglu if epi == cabi.EPI_SWIGLU else L.pg_geglu
                cabi.check(pair(ptr(out), ptr(gu), M, N, self.dt, st), "gated pairing")
                return out
        cabi.check(L.pg_gemm(ptr(out), ptr(a), ptr(w), None, None, M, N, K, a.stride(0), w.stride(0), out.stride(0), 0, 0,
                             epi, 1 if out_f32 else 0, self.gemm_impl, self.dt, st), "gemm")
        return out

    def _moe_experts(self, h: torch.Tensor, idx: torch.Tensor, n_experts: int, top: int, ff: int, w_gu: torch.Tensor,
                     w_dn: torch.Tensor, act: int = cabi.GLU_SILU, limit: float = 0.0):
        """The routed experts' feed-forward of a token batch: the (token, expert) pairs `idx` [T * top] are grouped by
        expert, both expert GEMMs run grouped (w_gu [E, 2 ff, D] with the pairing `act` in its epilogue, w_dn
        [E, D, ff]).  Returns (y [pairs, D] in grouped order, pair_pos [T * top]: the row of every pair in y, -1 for
        an index >= n_experts).  Prompt-sized steps gather the rows into expert order once and run on the tensor
        cores; a handful of pairs read h through the row map in the fp32-FMA kernel."""
        L, st, tm = cabi.lib(), cabi.stream(), self._tm
        T, D = h.shape
        P, E = T * top, n_experts
        offsets = self._new(E + 1, dtype=torch.int32)
        rows, pos = self._new(P, dtype=torch.int32), self._new(P, dtype=torch.int32)
        with tm("moe_sort"):
            cabi.check(L.pg_moe_sort(ptr(offsets), ptr(rows), ptr(pos), ptr(idx), P, top, E, st), "moe_sort")
        act_out, y = self._new(P, ff), self._new(P, D)
        tc = (self.dtype != torch.float32 and self.moe_impl != 1 and P >= self.moe_tc_min_pairs
              and D % 8 == 0 and ff % 8 == 0)
        a, row_map, impl = h, rows, 1
        if tc:
            a, row_map, impl = self._new(P, D), None, 2
            with tm("moe_gather"):
                cabi.check(L.pg_gather_rows(ptr(a), ptr(h), h.stride(0), ptr(rows), ptr(offsets[E:]), P, D, self.dt, st),
                           "gather_rows")
        with tm("moe_gate_up"):
            cabi.check(L.pg_moe_gemm_act(ptr(act_out), ff, ptr(a), a.stride(0), ptr(row_map), ptr(w_gu), ptr(offsets), P, E,
                                         ff, D, act, limit, impl, ptr(self.err_flag), self.dt, st), "moe_gemm gate/up")
        with tm("moe_down"):
            cabi.check(L.pg_moe_gemm_act(ptr(y), D, ptr(act_out), ff, None, ptr(w_dn), ptr(offsets), P, E, D, ff,
                                         cabi.GLU_NONE, 0.0, impl, ptr(self.err_flag), self.dt, st), "moe_gemm down")
        return y, pos

    # ------------------------------------------------------------------ one step
    @staticmethod
    def _runs(slots: np.ndarray, positions: np.ndarray):
        """Starts of the runs of consecutive tokens of one sequence at consecutive positions (and the end)."""
        T = slots.shape[0]
        brk = np.flatnonzero((slots[1:] != slots[:-1]) | (positions[1:] != positions[:-1] + 1)) + 1
        return np.concatenate(([0], brk, [T]))

    @staticmethod
    def _segments(slots: np.ndarray, bounds: np.ndarray) -> List[int]:
        """{slot, first row, tokens} per sequence; a sequence has ONE run of consecutive positions per step."""
        first = slots[bounds[:-1]]
        if np.unique(first).shape[0] != first.shape[0]:
            raise ValueError("the tokens of a sequence must be consecutive rows at consecutive positions of a step")
        return np.stack([first, bounds[:-1], np.diff(bounds)], 1).reshape(-1).tolist()

    @torch.no_grad()
    def forward_tokens(self, kv, ids: Sequence[int], slots: Sequence[int], positions: Sequence[int],
                       want_rows: Sequence[int], layer_sink: Optional[list] = None) -> torch.Tensor:
        """Run the listed tokens (token t: id, page-table row of its sequence, position in it) through the model
        from the cache and state that earlier steps left, append their keys and values, and return the fp32 logits
        [len(want_rows), vocab] of the listed rows.  `kv` is the scheduler's slot table; its pages for the new
        positions must be reserved (SlotKV.ensure).  layer_sink (debugging): receives the residual stream after
        every layer."""
        T, nw = len(ids), len(want_rows)
        if T == 0:
            return torch.empty((0, self.cfg.vocab), dtype=torch.float32, device=self.device)
        slots_np, pos_np = np.asarray(slots, dtype=np.int64), np.asarray(positions, dtype=np.int64)
        if self.max_positions is not None and int(pos_np.max()) >= self.max_positions:
            raise ValueError(f"position {int(pos_np.max())} exceeds max_positions {self.max_positions}")
        bounds = self._runs(slots_np, pos_np)
        segs: List[int] = []
        replay = (T <= self.graph_max_tokens and layer_sink is None and not self._op_timing
                  and not torch.cuda.is_current_stream_capturing())
        if self.needs_segments:
            segs = self._segments(slots_np, bounds)
            if replay:      # a captured launch sequence must depend on the token count only: pad with empty segments
                segs += [0, 0, 0] * (min(T, int(kv.page_table.shape[0])) - len(segs) // 3)
        ns = len(segs) // 3
        # query tiles of the tensor-core attention: runs of <= 128 consecutive tokens of one sequence
        tiles: List[int] = []
        if T >= self.attn_tc_min_tokens and self._attn_tc_any:
            for r0, r1 in zip(bounds[:-1].tolist(), bounds[1:].tolist()):
                for t0 in range(r0, r1, 128):
                    tiles += [t0, min(128, r1 - t0), int(slots_np[t0]), int(pos_np[t0])]
        nt = len(tiles) // 4
        host = torch.empty(4 * T + nw + 3 * ns + 4 * nt, dtype=torch.int32).pin_memory()   # torch caches pinned blocks
        host[:2 * T].view(torch.int64).copy_(torch.from_numpy(np.asarray(ids, dtype=np.int64)))
        host[2 * T:3 * T].copy_(torch.from_numpy(slots_np))
        host[3 * T:4 * T].copy_(torch.from_numpy(pos_np))
        if nw:
            host[4 * T:4 * T + nw].copy_(torch.as_tensor(want_rows, dtype=torch.int32))
        if ns:
            host[4 * T + nw:4 * T + nw + 3 * ns].copy_(torch.as_tensor(segs, dtype=torch.int32))
        if nt:
            host[4 * T + nw + 3 * ns:].copy_(torch.as_tensor(tiles, dtype=torch.int32))
        if replay and nt == 0:
            return self._replay(kv, host, T, nw, ns)
        return self._forward_device(kv, self._inputs(host.to(self.device, non_blocking=True), T, nw, ns), layer_sink)

    @staticmethod
    def _inputs(dev: torch.Tensor, T: int, nw: int, ns: int) -> StepInputs:
        a = 4 * T + nw
        return StepInputs(T=T, nw=nw, ids=dev[:2 * T].view(torch.int64), slot=dev[2 * T:3 * T], pos=dev[3 * T:4 * T],
                          want=dev[4 * T:a], segs=dev[a:a + 3 * ns], n_segs=ns, tiles=dev[a + 3 * ns:],
                          n_tiles=(dev.numel() - a - 3 * ns) // 4)

    def _replay(self, kv, host: torch.Tensor, T: int, nw: int, ns: int) -> torch.Tensor:
        """Small steps are launch-bound (some fifteen launches per layer): the kernel sequence for (T tokens, nw
        wanted rows) over this slot table is captured once; a step copies its ids / slots / positions into the
        graph's static input and replays.  Which kernels run depends on the counts only, never on the values."""
        key = (T, nw, ns, kv.page_table.data_ptr(), kv.max_pages)
        ent = self._graphs.get(key)
        if ent is None:
            static_in = torch.zeros(host.numel(), dtype=torch.int32, device=self.device)
            static_in.copy_(host, non_blocking=True)
            # warm-up outside the capture (module loading, shared-memory attributes) on inputs that touch no sequence:
            # empty segments leave every recurrent state alone, and the cache rows it writes are rewritten by the replay
            warm = static_in.clone()
            if ns:
                warm[4 * T + nw:].zero_()
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                self._forward_device(kv, self._inputs(warm, T, nw, ns), None)
            torch.cuda.current_stream().wait_stream(s)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                out = self._forward_device(kv, self._inputs(static_in, T, nw, ns), None)
            ent = self._graphs[key] = (g, static_in, out)
            if len(self._graphs) > 64:
                self._graphs.pop(next(iter(self._graphs)))
        g, static_in, out = ent
        static_in.copy_(host, non_blocking=True)
        g.replay()
        return out.clone()

    def _forward_device(self, kv, inp: StepInputs, layer_sink: Optional[list]) -> torch.Tensor:
        raise NotImplementedError

    # ------------------------------------------------------------------ per-op timing (diagnostic: PG_OP_TIMING=1)
    def _tm(self, name):
        """CUDA-event bracket around one op when op timing is on (durations inside the real step, with the L2 state
        of the real step); `op_times()` sums them per name.  A no-op otherwise."""
        from .engine import PaliGemmaEngine
        if not self._op_timing:
            return PaliGemmaEngine._NoTimer()
        return PaliGemmaEngine._EvTimer(self._op_events, name)

    def op_times(self, reset: bool = True) -> Dict[str, float]:
        torch.cuda.synchronize()
        out: Dict[str, float] = {}
        for name, e0, e1 in self._op_events:
            out[name] = out.get(name, 0.0) + e0.elapsed_time(e1)
        if reset:
            self._op_events = []
        return out

    # ------------------------------------------------------------------ serving glue
    def new_batcher(self, **kw):
        from .scheduler import RaggedBatcher
        return RaggedBatcher(self, **kw)

    def new_slot_state(self, slots: int):
        """Recurrent state of `slots` sequences (scheduler.SlotState), None for designs without any."""
        return None

    _ERR_TEXT = {2: "a tensor-core kernel gave up waiting on its pipeline (its results are invalid)"}

    def check_errors(self, sync: bool = False) -> None:
        if sync:
            torch.cuda.current_stream(self.device).synchronize()
        if self._err_np[0] != 0:
            code, self._err_np[0] = int(self._err_np[0]), 0
            raise RuntimeError(self._ERR_TEXT.get(code, "a token id lies outside the vocabulary or a position outside "
                                                        "the positions the model has"))
