"""`bench.py --arch mubasun`: prefill and decode throughput of the Mubasun engine at layer sizes that resemble a
real model's (random weights), beside the framework's Gemma decoder (the text half of the PaliGemma engine) at equal
width, depth, query width and feed-forward size, with a per-kernel roofline table for both.
`bench.py --arch ninisun`: the same for the Ninisun engine beside the closest model the framework serves the same
way, a dense Mubasun of equal width, depth, head layout, window and feed-forward width (`run_ninisun`).

`bench.py --arch gogivik`: the Gogivik engine beside the two models that hold its closest kernels: Ninisun (attention in
a mask, dense feed-forward, a recurrence with a gated norm) and Birizen (latent attention with a sink, the decayed
linear-attention scan the state-space layer runs on) (`run_gogivik`).

Timing: CUDA events on the launching stream, >= 3 warm-up steps, an L2-sized scratch write between timed steps.
Roofline of an op = max(algorithmic FLOPs / measured bf16 peak, algorithmic bytes / measured copy bandwidth);
`frac` = that time / measured time (1.0 = on the roofline)."""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List

import torch

from . import _cabi as cabi

SIZES = {
    # width, layers, heads x dim (key) / vdim, kv heads, window, dense ff, experts x ff (top), shared ff, vocab
    "w1024": dict(width=1024, layers=4, heads=8, kv_heads=2, dim=128, vdim=128, window=512, ff=4096, experts=8, top=2,
                  expert_ff=1024, shared_ff=1024, vocab=32000),
    "w2048": dict(width=2048, layers=4, heads=16, kv_heads=4, dim=128, vdim=128, window=1024, ff=8192, experts=16, top=2,
                  expert_ff=2048, shared_ff=2048, vocab=32000),
}
MAX_POS = 4096


def mubasun_config(s: dict) -> dict:
    """Layer order: dense, MoE, MoE reading layer 1's cache, dense ... (every branch of the design is on the path)."""
    layers = []
    for i in range(s["layers"]):
        mixer = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["vdim"],
                 "scale": 1.0 / math.sqrt(s["dim"]), "mask": {"size": s["window"]}}
        if i % 4 == 2:
            mixer["kv_from"] = i - 1
        if i % 2 == 0:
            mlp = {"kind": "dense", "ff": s["ff"]}
        else:
            mlp = {"kind": "moe", "expert": {"ff": s["expert_ff"]}, "shared": {"ff": s["shared_ff"]},
                   "router": {"experts": s["experts"], "identity": 1, "top": s["top"], "scale": 1.0}}
        layers.append({"type": "attention", "mixer": mixer, "mlp": mlp})
    return {"architecture": "Mubasun", "vocab": s["vocab"], "width": s["width"], "max_positions": MAX_POS,
            "norm": {"eps": 1e-6, "groups": 4}, "layers": layers}


def random_mubasun_weights(cfg: dict, device, dtype, seed=0) -> Dict[str, torch.Tensor]:
    g = torch.Generator(device=device).manual_seed(seed)
    D, out = cfg["width"], {}

    def lin(name, o, i, gain=1.0):
        out[name] = (torch.randn(o, i, generator=g, device=device) * (gain / math.sqrt(i))).to(dtype)

    def vec(name, n, mean=1.0, std=0.1):
        out[name] = (mean + std * torch.randn(n, generator=g, device=device)).to(dtype)

    out["embed"] = torch.randn(cfg["vocab"], D, generator=g, device=device).to(dtype)
    out["pos"] = (0.3 * torch.randn(cfg["max_positions"], D, generator=g, device=device)).to(dtype)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        vec(p + "norm1", D)
        lin(p + "mix.q", H * dim, D)
        vec(p + "mix.q.norm", H * dim)
        if "kv_from" not in m:
            lin(p + "mix.k", G * dim, D)
            lin(p + "mix.v", G * vdim, D)
            vec(p + "mix.k.norm", G * dim)
        lin(p + "mix.g", H * vdim, D)
        lin(p + "mix.o", D, H * vdim)
        ml = L["mlp"]
        if ml["kind"] == "dense":
            lin(p + "mlp.up", ml["ff"], D)
            lin(p + "mlp.down", D, ml["ff"])
            out[p + "mlp.act"] = torch.zeros(2, device=device, dtype=dtype)
        else:
            r = ml["router"]
            for e in range(r["experts"]):
                lin(f"{p}mlp.e{e}.gate", ml["expert"]["ff"], D)
                lin(f"{p}mlp.e{e}.up", ml["expert"]["ff"], D)
                lin(f"{p}mlp.e{e}.down", D, ml["expert"]["ff"])
            lin(p + "mlp.router", r["experts"] + r["identity"], D, 2.0)
            vec(p + "mlp.correction", r["experts"] + r["identity"], 0.0, 0.05)
            for n, (o, i) in (("gate", (ml["shared"]["ff"], D)), ("up", (ml["shared"]["ff"], D)), ("down", (D, ml["shared"]["ff"]))):
                lin(p + "mlp.shared." + n, o, i)
            lin(p + "mlp.shared.sg", 1, D)
    vec("final.norm", D)
    lin("head", cfg["vocab"], D)
    return out


def gemma_config(s: dict) -> dict:
    """Gemma decoder of the same width, depth, query width (heads x 256 = Mubasun's heads x 128) and dense
    feed-forward size; the vision half is the smallest that the engine accepts and is never run."""
    hd = 256
    nq = s["heads"] * s["dim"] // hd
    return {"image_token_index": s["vocab"] - 1, "vocab_size": s["vocab"], "projection_dim": s["width"],
            "hidden_size": s["width"], "pad_token_id": 0,
            "vision_config": {"hidden_size": 144, "intermediate_size": 272, "num_hidden_layers": 1, "num_attention_heads": 2,
                              "num_channels": 3, "image_size": 56, "patch_size": 14, "num_image_tokens": 16},
            "text_config": {"vocab_size": s["vocab"], "hidden_size": s["width"], "intermediate_size": s["ff"],
                            "num_hidden_layers": s["layers"], "num_attention_heads": nq,
                            "num_key_value_heads": max(1, s["kv_heads"] * s["dim"] // hd), "head_dim": hd}}


def random_gemma_weights(cfg: dict, device, dtype, seed=0) -> Dict[str, torch.Tensor]:
    from . import synth
    g = torch.Generator(device=device).manual_seed(seed)
    sd = {}
    for key, shape, kind in synth.state_dict_spec(cfg):
        t = torch.randn(shape, generator=g, device=device, dtype=torch.float32) * (0.02 if kind != "ln_w" else 0.1)
        sd[key] = t.to(dtype)
    return sd


class _Timer:
    def __init__(self, flush_mb=256):
        self.scratch = torch.empty(flush_mb << 20, dtype=torch.uint8, device="cuda")

    def run(self, fn, steps, warmup, setup=None):
        """-> list of per-step ms.  `setup` (untimed) runs before every step, then the L2 flush."""
        out = []
        for i in range(warmup + steps):
            if setup:
                setup()
            self.scratch.zero_()                      # larger than L2: the step starts cold
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            if i >= warmup:
                out.append(e0.elapsed_time(e1))
        return out


def _med(xs: List[float]) -> float:
    xs = sorted(xs)
    return xs[len(xs) // 2]


# ------------------------------------------------------------------ algorithmic work per op (one prefill of T tokens)
def mubasun_work(s: dict, cfg: dict, T1: int, seqs: int) -> Dict[str, tuple]:
    """name -> (FLOPs, bytes) summed over the layers that run the op (bf16 operands, fp32 residual stream) for one
    step over `seqs` prompts of T1 tokens."""
    T = T1 * seqs
    D, H, G, dim, vdim, W = s["width"], s["heads"], s["kv_heads"], s["dim"], s["vdim"], s["window"]
    w: Dict[str, List[float]] = {}

    def add(name, flops, nbytes):
        a = w.setdefault(name, [0.0, 0.0])
        a[0] += flops
        a[1] += nbytes

    keys = seqs * sum(min(t + 1, W) for t in range(T1))      # (query, key) pairs per head
    for L in cfg["layers"]:
        own = "kv_from" not in L["mixer"]
        nq, nk, nv, ng = H * dim, G * dim if own else 0, G * vdim if own else 0, H * vdim
        npj = nq + nk + nv + ng
        add("norm", 0, T * D * (4 + 4 + 2 + 2 + 2))
        add("proj", 2 * T * D * npj, 2 * (T * D + npj * D + T * npj))
        add("qknorm_append", 0, 2 * 2 * T * (nq + nk + nv))
        add("attention", 2 * keys * H * (dim + vdim), 2 * T * (nq + 2 * ng) + 2 * T * G * (dim + vdim))
        add("o", 2 * T * ng * D, 2 * (T * ng + ng * D + T * D))
        ml = L["mlp"]
        if ml["kind"] == "dense":
            F = ml["ff"]
            add("dense_up", 2 * T * D * F, 2 * (T * D + D * F + T * F))
            add("xielu", 0, 2 * 2 * T * F)
            add("dense_down", 2 * T * D * F, 2 * (T * F + D * F + T * D))
        else:
            r, F, S = ml["router"], ml["expert"]["ff"], ml["shared"]["ff"]
            E, P = r["experts"], T * r["top"]
            Pe = P * E / (E + r["identity"])           # pairs that reach a real expert, on average
            add("moe_route", 2 * T * D * (E + r["identity"] + 1), 2 * T * D)
            add("moe_sort", 0, 4 * 3 * P)
            add("moe_gather", 0, 2 * 2 * Pe * D)
            add("moe_gate_up", 2 * Pe * D * 2 * F, 2 * (Pe * D + E * 2 * F * D + Pe * F))
            add("moe_down", 2 * Pe * F * D, 2 * (Pe * F + E * F * D + Pe * D))
            add("shared_gate_up", 2 * T * D * 2 * S, 2 * (T * D + 2 * S * D + T * S))
            add("shared_down", 2 * T * S * D, 2 * (T * S + S * D + T * D))
            add("moe_combine", 0, 2 * Pe * D + T * D * (2 + 2 + 8))
    add("head", 2 * seqs * D * s["vocab"], 2 * D * s["vocab"])
    return {k: (v[0], v[1]) for k, v in w.items()}


def gemma_work(s: dict, gcfg: dict, T1: int, seqs: int) -> Dict[str, tuple]:
    t = gcfg["text_config"]
    T = T1 * seqs
    D, F, nq, nkv, hd, Ln = t["hidden_size"], t["intermediate_size"], t["num_attention_heads"], t["num_key_value_heads"], \
        t["head_dim"], t["num_hidden_layers"]
    nqkv = (nq + 2 * nkv) * hd
    return {
        "t_norm": (0, Ln * 2 * T * D * 4),
        "t_qkv": (Ln * 2 * T * D * nqkv, Ln * 2 * (T * D + nqkv * D + T * nqkv)),
        "t_rope_append": (0, Ln * 2 * 2 * T * nqkv),
        "t_attention": (Ln * 2 * T * T1 * nq * 2 * hd, Ln * 2 * (2 * T * nq * hd + 2 * T * nkv * hd)),   # unmasked: T1 keys
        "t_o": (Ln * 2 * T * nq * hd * D, Ln * 2 * (T * nq * hd + nq * hd * D + 2 * T * D)),
        "t_gate_up": (Ln * 2 * T * D * 2 * F, Ln * 2 * (T * D + 2 * F * D + T * F)),
        "t_down": (Ln * 2 * T * F * D, Ln * 2 * (T * F + F * D + 2 * T * D)),
    }


def _roofline(work: Dict[str, tuple], times_ms: Dict[str, float], peaks: dict) -> Dict[str, dict]:
    out = {}
    for name, (flops, nbytes) in work.items():
        if name not in times_ms or times_ms[name] <= 0:
            continue
        ideal = max(flops / (peaks["tc"] * 1e12), nbytes / (peaks["hbm"] * 1e9)) * 1e3
        out[name] = {"ms": round(times_ms[name], 4), "roofline_ms": round(ideal, 4), "frac": round(ideal / times_ms[name], 3),
                     "bound": "tensor" if flops / (peaks["tc"] * 1e12) > nbytes / (peaks["hbm"] * 1e9) else "hbm"}
    return out


# pairs (Mubasun op, the like op of the Gemma decoder)
LIKE = [("norm", "t_norm"), ("proj", "t_qkv"), ("qknorm_append", "t_rope_append"), ("attention", "t_attention"),
        ("o", "t_o"), ("dense_up", "t_gate_up"), ("dense_down", "t_down"), ("moe_gate_up", "t_gate_up"),
        ("moe_down", "t_down"), ("shared_gate_up", "t_gate_up"), ("shared_down", "t_down")]


def _measure_ragged(eng, vocab: int, timer, steps, warmup, peaks, work, decode_bytes, prefill_tokens, prefill_seqs, context,
                    decode_batches) -> dict:
    """Prefill (all prompts in ONE step), per-op rooflines of that step, and decode steps of an engine that is served
    through RaggedBatcher.  work: name -> (FLOPs, bytes) of the prefill step; decode_bytes(B): weight bytes of a step."""
    row = {}
    slots = max(max(decode_batches), prefill_seqs)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, vocab, (prefill_tokens,), generator=g).tolist() for _ in range(prefill_seqs)]
    b = eng.new_batcher(slots=slots + 1, max_seq_tokens=max(prefill_tokens, context) + 256)
    T_all = prefill_tokens * prefill_seqs

    def prefill():                                   # all prompts in ONE step of the engine
        for i in range(prefill_seqs):
            b.admit(("p", i))
        b.run_entries([(("p", i), prompts[i], [prefill_tokens - 1]) for i in range(prefill_seqs)])

    def drop():
        for i in range(prefill_seqs):
            if ("p", i) in b.slot_of:
                b.finish(("p", i))
    ms = timer.run(prefill, steps, warmup, setup=drop)
    drop()
    row["prefill"] = {"tokens": T_all, "sequences": prefill_seqs, "ms": round(_med(ms), 3),
                      "tok_s": round(T_all / _med(ms) * 1e3), "min_ms": round(min(ms), 3), "max_ms": round(max(ms), 3)}
    eng._op_timing = True                                    # one more prefill, bracketed op by op
    for _ in range(2):
        prefill(); drop(); eng.op_times()
    reps = 3
    for _ in range(reps):
        timer.scratch.zero_(); prefill(); drop()
    times = {k: v / reps for k, v in eng.op_times().items()}
    eng._op_timing = False
    row["prefill_ops"] = _roofline(work, times, peaks)
    row["decode"] = {}
    for B in decode_batches:
        for i in range(B):
            b.admit(("d", i))
        ctx = torch.randint(0, vocab, (context,), generator=g).tolist()
        for i in range(B):
            b.run_entries([(("d", i), ctx, [])])
        step_ents = [(("d", i), [7 + i], [0]) for i in range(B)]
        n_dec = min(steps * 4, 200)
        ms = timer.run(lambda: b.run_entries(step_ents), n_dec, warmup + 2)
        row["decode"][f"batch{B}"] = {"context": context, "ms_per_step": round(_med(ms), 4),
                                      "tok_s": round(B / _med(ms) * 1e3), "graph": eng.graph_max_tokens >= B,
                                      "weight_stream_ms": round(decode_bytes(B) / (peaks["hbm"] * 1e9) * 1e3, 4)}
        for i in range(B):
            b.finish(("d", i))
    b.close()
    return row


@torch.no_grad()
def run(sizes, steps: int, warmup: int, peaks: dict, prefill_tokens=2048, prefill_seqs=4, context=1024,
        decode_batches=(1, 8)) -> dict:
    from .engine import PaliGemmaEngine
    from .mubasun import MubasunEngine
    dev, dtype = torch.device("cuda:0"), torch.bfloat16
    timer = _Timer()
    result = {}
    launches0 = cabi.launch_count()
    for name in sizes:
        s = SIZES[name]
        row = {"size": s}
        # ------------------------------------------------ Mubasun
        cfg = mubasun_config(s)
        slots = max(max(decode_batches), prefill_seqs)
        eng = MubasunEngine(cfg, random_mubasun_weights(cfg, dev, dtype), device=dev, dtype=dtype,
                            kv_pool_tokens=(slots + 1) * (max(prefill_tokens, context) + 256))
        row.update(_measure_ragged(eng, s["vocab"], timer, steps, warmup, peaks, mubasun_work(s, cfg, prefill_tokens, prefill_seqs),
                                   lambda B: _decode_bytes(s, cfg, B), prefill_tokens, prefill_seqs, context, decode_batches))
        g = torch.Generator().manual_seed(2)
        T_all = prefill_tokens * prefill_seqs
        reps = 3
        del eng
        torch.cuda.empty_cache()
        # ------------------------------------------------ Gemma decoder at equal size
        gcfg = gemma_config(s)
        geng = PaliGemmaEngine(gcfg, random_gemma_weights(gcfg, dev, dtype), device=dev, dtype=dtype,
                               kv_pool_tokens=(max(max(decode_batches), prefill_seqs) + 1) * (max(prefill_tokens, context) + 512))
        ids = torch.randint(1, s["vocab"] - 2, (prefill_seqs, prefill_tokens), generator=g).to(dev)
        holder = {}

        def g_prefill():
            holder["kv"] = geng.new_kv(prefill_seqs)
            geng.text_forward(ids, None, holder["kv"], logits="last")

        def g_drop():
            if "kv" in holder:
                holder.pop("kv").release()
        ms = timer.run(g_prefill, steps, warmup, setup=g_drop)
        g_drop()
        grow = {"prefill": {"tokens": T_all, "sequences": prefill_seqs, "ms": round(_med(ms), 3),
                            "tok_s": round(T_all / _med(ms) * 1e3)}}
        geng._op_timing = True
        for _ in range(2):
            g_prefill(); g_drop(); geng.op_times()
        for _ in range(reps):
            timer.scratch.zero_(); g_prefill(); g_drop()
        gt = {k: v / reps for k, v in geng.op_times().items()}
        geng._op_timing = False
        grow["prefill_ops"] = _roofline(gemma_work(s, gcfg, prefill_tokens, prefill_seqs), gt, peaks)
        grow["decode"] = {}
        for B in decode_batches:
            kv = geng.new_kv(B)
            kv.reserve(context + 512)
            geng.text_forward(torch.randint(1, s["vocab"] - 2, (B, context), generator=g).to(dev), None, kv, logits="last")
            ds = geng.decode_state(B)
            ds.bind(kv, torch.full((B,), 5, dtype=torch.int64, device=dev), position=context + 1)
            n_dec = min(steps * 4, 200)
            ms = timer.run(lambda: ds.run_steps(kv, 1), n_dec, warmup + 2)
            grow["decode"][f"batch{B}"] = {"context": context, "ms_per_step": round(_med(ms), 4), "tok_s": round(B / _med(ms) * 1e3)}
            kv.release()
        row["gemma_equal_size"] = grow
        # like-for-like: how far each Mubasun op is from its roofline against the like Gemma op
        cmpr = {}
        for a, bname in LIKE:
            if a in row["prefill_ops"] and bname in grow["prefill_ops"]:
                fa, fb = row["prefill_ops"][a]["frac"], grow["prefill_ops"][bname]["frac"]
                cmpr[a] = {"frac": fa, "like": bname, "like_frac": fb, "distance_ratio": round(fb / fa, 2) if fa > 0 else None}
        row["like_for_like"] = cmpr
        result[name] = row
        del geng
        torch.cuda.empty_cache()
    result["gpu_launches"] = int(cabi.launch_count() - launches0)
    return result


def _decode_bytes(s: dict, cfg: dict, B: int) -> float:
    """Weight bytes one decode step of B tokens must stream (experts: at most B * top of them per MoE layer)."""
    D, n = s["width"], 0.0
    for L in cfg["layers"]:
        m = L["mixer"]
        own = "kv_from" not in m
        n += D * (m["heads"] * m["dim"] + (m["kv_heads"] * (m["dim"] + m["vdim"]) if own else 0) + 2 * m["heads"] * m["vdim"])
        ml = L["mlp"]
        if ml["kind"] == "dense":
            n += 2 * D * ml["ff"]
        else:
            r = ml["router"]
            n += min(r["experts"], B * r["top"]) * 3 * D * ml["expert"]["ff"] + 3 * D * ml["shared"]["ff"] + D * (r["experts"] + 2)
    n += D * s["vocab"]
    return 2.0 * n


# ------------------------------------------------------------------ Ninisun beside a dense Mubasun of equal size
NINISUN_SIZES = {
    # attention layers: heads x dim over kv heads, window + kept first tokens, half of every head rotated, value mixing;
    # the parallel layer: the same head layout for the sigmoid attention, r_heads x r_dim recurrent heads, decay rank
    "w1024": dict(width=1024, layers=4, heads=8, kv_heads=2, dim=128, vdim=128, window=512, keep_first=8, ff=4096,
                  r_heads=16, r_dim=64, lora=64, vocab=32000),
    "w2048": dict(width=2048, layers=4, heads=16, kv_heads=4, dim=128, vdim=128, window=1024, keep_first=8, ff=8192,
                  r_heads=32, r_dim=64, lora=64, vocab=32000),
}


def ninisun_config(s: dict) -> dict:
    """attention, attention, parallel, attention, ... (every branch of the design is on the path)."""
    layers = []
    for i in range(s["layers"]):
        mlp = {"kind": "dense", "ff": s["ff"]}
        att = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["vdim"],
               "scale": 1.0 / math.sqrt(s["dim"])}
        if i % 4 == 2:
            left = dict(att, rot={"dims": s["dim"] // 2, "base": 250000.0,
                                  "scaling": {"factor": 8.0, "original": 2048, "fast": 16.0, "slow": 2.0}})
            layers.append({"type": "parallel", "mlp": mlp, "mixer": {
                "left": left, "right": {"heads": s["r_heads"], "dim": s["r_dim"]}, "left_scale": 0.7, "right_scale": 0.6}})
        else:
            layers.append({"type": "attention", "mlp": mlp, "mixer": dict(
                att, rot={"dims": s["dim"] // 2, "base": 10000.0}, v_mix=True,
                mask={"size": s["window"], "keep_first": s["keep_first"]})})
    return {"architecture": "Ninisun", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-6}, "layers": layers}


def random_ninisun_weights(cfg: dict, s: dict, device, dtype, seed=0) -> Dict[str, torch.Tensor]:
    g = torch.Generator(device=device).manual_seed(seed)
    D, out = cfg["width"], {}

    def lin(name, o, i, gain=1.0):
        out[name] = (torch.randn(o, i, generator=g, device=device) * (gain / math.sqrt(i))).to(dtype)

    def vec(name, n, mean=1.0, std=0.1):
        out[name] = (mean + std * torch.randn(n, generator=g, device=device)).to(dtype)

    out["embed"] = torch.randn(cfg["vocab"], D, generator=g, device=device).to(dtype)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        for n in ("norm1", "norm1b", "norm2", "norm2b"):
            vec(p + n, D)
        vec(p + "ls1", D, 0.5), vec(p + "ls2", D, 0.5)
        a = m["left"] if L["type"] == "parallel" else m
        H, G, d, e = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
        q = p + ("mix.left." if L["type"] == "parallel" else "mix.")
        lin(q + "q", H * d, D), lin(q + "k", G * d, D), lin(q + "v", G * e, D), lin(q + "o", D, H * e)
        if L["type"] == "parallel":
            vec(q + "q.b", H * d, 0.0), vec(q + "k.b", G * d, 0.0), vec(q + "v.b", G * e, 0.0), vec(q + "pb", H, -2.0, 0.5)
            lin(q + "g", H, D)
            r, nd = p + "mix.right.", m["right"]["heads"] * m["right"]["dim"]
            for n in ("r", "k", "v", "g", "a"):
                lin(r + n, nd, D)
            vec(r + "a.b", nd, 0.0), lin(r + "w1", s["lora"], D), lin(r + "w2", nd, s["lora"]), vec(r + "w0", nd, 0.0, 1.0)
            vec(r + "norm", nd), lin(r + "o", D, nd)
        else:
            out[p + "mix.vmix"] = torch.tensor(0.4, device=device).to(dtype)
        ff = L["mlp"]["ff"]
        lin(p + "mlp.gate", ff, D), lin(p + "mlp.up", ff, D), lin(p + "mlp.down", D, ff)
    vec("final.norm", D)
    return out


def ninisun_work(s: dict, cfg: dict, T1: int, seqs: int) -> Dict[str, tuple]:
    """name -> (FLOPs, bytes) of one step over `seqs` prompts of T1 tokens (bf16 operands, fp32 residual stream)."""
    T, D, F = T1 * seqs, s["width"], s["ff"]
    H, G, dim, vdim, W, K0 = s["heads"], s["kv_heads"], s["dim"], s["vdim"], s["window"], s["keep_first"]
    nd, lora = s["r_heads"] * s["r_dim"], s["lora"]
    w: Dict[str, List[float]] = {}

    def add(name, flops, nbytes):
        a = w.setdefault(name, [0.0, 0.0])
        a[0] += flops
        a[1] += nbytes

    nq, nk, nv, ng = H * dim, G * dim, G * vdim, H * vdim
    win_keys = seqs * sum(min(t + 1, W + K0) for t in range(T1))
    all_keys = seqs * T1 * (T1 + 1) // 2
    add("norm", 0, T * D * (4 + 2))
    for L in cfg["layers"]:
        par = L["type"] == "parallel"
        npj = nq + nk + nv + ((H + 5 * nd + lora) if par else 0)
        add("proj", 2 * T * D * npj, 2 * (T * D + npj * D + T * npj))
        add("rotary_append", 0, 2 * 2 * T * (nq + nk + nv))
        if par:
            add("sigmoid_attention", 2 * all_keys * H * (dim + vdim), 2 * T * (nq + ng) + 2 * T * G * (dim + vdim))
            add("delta_prep", 2 * T * nd * lora, T * (2 * (4 * nd + lora) + 6 * 4 * nd))     # six fp32 vectors per head out
            add("delta_rule", 10 * T * nd * s["r_dim"], T * nd * (6 * 4 + 4))                # fp32 FMAs, not tensor work
            add("headnorm_gate", 0, T * nd * (4 + 2 + 2))
            add("o", 2 * T * (ng + nd) * D, 2 * (T * (ng + nd) + (ng + nd) * D + T * D))
        else:
            add("attention", 2 * win_keys * H * (dim + vdim), 2 * T * (nq + ng) + 2 * T * G * (dim + vdim))
            add("o", 2 * T * ng * D, 2 * (T * ng + ng * D + T * D))
        add("post_norm", 0, 2 * T * D * (2 + 4 + 4 + 2))
        add("gate_up", 2 * T * D * 2 * F, 2 * (T * D + 2 * D * F + T * F))
        add("down", 2 * T * D * F, 2 * (T * F + D * F + T * D))
    add("head", 2 * seqs * D * s["vocab"], 2 * D * s["vocab"])
    return {k: (v[0], v[1]) for k, v in w.items()}


def _ninisun_decode_bytes(s: dict, cfg: dict) -> float:
    D, n = s["width"], 0.0
    nq, nk, nv, ng, nd = s["heads"] * s["dim"], s["kv_heads"] * s["dim"], s["kv_heads"] * s["vdim"], s["heads"] * s["vdim"], \
        s["r_heads"] * s["r_dim"]
    for L in cfg["layers"]:
        n += D * (nq + nk + nv + ng) + 3 * D * s["ff"]
        if L["type"] == "parallel":
            n += D * (s["heads"] + 6 * nd + s["lora"]) + nd * s["lora"]
    return 2.0 * (n + D * s["vocab"])


def dense_mubasun_config(s: dict) -> dict:
    """The closest model of the framework: Mubasun with dense feed-forwards only, same width, depth, heads, window."""
    layers = [{"type": "attention", "mlp": {"kind": "dense", "ff": s["ff"]},
               "mixer": {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["vdim"],
                         "scale": 1.0 / math.sqrt(s["dim"]), "mask": {"size": s["window"]}}} for _ in range(s["layers"])]
    return {"architecture": "Mubasun", "vocab": s["vocab"], "width": s["width"], "max_positions": MAX_POS,
            "norm": {"eps": 1e-6, "groups": 4}, "layers": layers}


NINISUN_LIKE = [("post_norm", "norm"), ("proj", "proj"), ("rotary_append", "qknorm_append"), ("attention", "attention"),
                ("sigmoid_attention", "attention"), ("o", "o"), ("gate_up", "dense_up"), ("down", "dense_down"),
                ("headnorm_gate", "xielu"), ("delta_prep", "qknorm_append"), ("head", "head")]


@torch.no_grad()
def run_ninisun(sizes, steps: int, warmup: int, peaks: dict, prefill_tokens=2048, prefill_seqs=4, context=1024,
                decode_batches=(1, 8)) -> dict:
    from .mubasun import MubasunEngine
    from .ninisun import NinisunEngine
    dev, dtype = torch.device("cuda:0"), torch.bfloat16
    timer = _Timer()
    result = {}
    launches0 = cabi.launch_count()
    pool = (max(max(decode_batches), prefill_seqs) + 1) * (max(prefill_tokens, context) + 256)
    for name in sizes:
        s = NINISUN_SIZES[name]
        cfg = ninisun_config(s)
        eng = NinisunEngine(cfg, random_ninisun_weights(cfg, s, dev, dtype), device=dev, dtype=dtype, kv_pool_tokens=pool)
        row = {"size": s}
        row.update(_measure_ragged(eng, s["vocab"], timer, steps, warmup, peaks, ninisun_work(s, cfg, prefill_tokens, prefill_seqs),
                                   lambda B: _ninisun_decode_bytes(s, cfg), prefill_tokens, prefill_seqs, context, decode_batches))
        del eng
        torch.cuda.empty_cache()
        ms_ = dict(s, experts=0, top=0, expert_ff=0, shared_ff=0)
        mcfg = dense_mubasun_config(s)
        meng = MubasunEngine(mcfg, random_mubasun_weights(mcfg, dev, dtype), device=dev, dtype=dtype, kv_pool_tokens=pool)
        mrow = _measure_ragged(meng, s["vocab"], timer, steps, warmup, peaks, mubasun_work(ms_, mcfg, prefill_tokens, prefill_seqs),
                               lambda B: _decode_bytes(ms_, mcfg, B), prefill_tokens, prefill_seqs, context, decode_batches)
        row["mubasun_dense_equal_size"] = mrow
        cmpr = {}
        for a, bname in NINISUN_LIKE:
            if a in row["prefill_ops"] and bname in mrow["prefill_ops"]:
                fa, fb = row["prefill_ops"][a]["frac"], mrow["prefill_ops"][bname]["frac"]
                cmpr[a] = {"frac": fa, "like": bname, "like_frac": fb, "distance_ratio": round(fb / fa, 2) if fa > 0 else None}
        row["like_for_like"] = cmpr
        result[name] = row
        del meng
        torch.cuda.empty_cache()
    result["gpu_launches"] = int(cabi.launch_count() - launches0)
    return result


# ------------------------------------------------------------------ Birizen beside the MoE Mubasun and Ninisun of equal size
BIRIZEN_SIZES = {
    # lightning layers: heads x dim / vdim; latent layers: heads x (dim plain + rot_dim rotated) / vdim over latents of
    # q_rank / kv_rank; experts x ff (top, groups kept of groups), shared ff; layers 2..3 run twice
    "w1024": dict(width=1024, layers=4, heads=8, dim=128, vdim=128, rot_dim=64, q_rank=384, kv_rank=192, experts=8, top=2,
                  groups=4, keep=2, expert_ff=1024, shared_ff=1024, loop=(2, 4, 2), vocab=32000),
    "w2048": dict(width=2048, layers=4, heads=16, dim=128, vdim=128, rot_dim=64, q_rank=768, kv_rank=192, experts=16, top=2,
                  groups=4, keep=2, expert_ff=2048, shared_ff=2048, loop=(2, 4, 2), vocab=32000),
}


def birizen_config(s: dict) -> dict:
    """lightning, latent, lightning, latent; the last two layers run `times` times (every branch is on the path)."""
    layers = []
    for i in range(s["layers"]):
        mlp = {"kind": "moe", "expert": {"ff": s["expert_ff"], "limit": 7.0}, "shared": {"ff": s["shared_ff"], "limit": 7.0},
               "router": {"experts": s["experts"], "top": s["top"], "groups": {"count": s["groups"], "keep": s["keep"]}}}
        if i % 2 == 0:
            H = s["heads"]
            mixer = {"heads": H, "dim": s["dim"], "vdim": s["vdim"], "decay": [1.0 - 2.0 ** (-5 - 3 * h / H) for h in range(H)]}
            layers.append({"type": "lightning", "mixer": mixer, "mlp": mlp})
        else:
            mixer = {"heads": s["heads"], "dim": s["dim"], "rot_dim": s["rot_dim"], "vdim": s["vdim"], "q_rank": s["q_rank"],
                     "kv_rank": s["kv_rank"], "scale": 1.0 / math.sqrt(s["dim"] + s["rot_dim"]),
                     "rot": {"dims": s["rot_dim"], "base": 10000.0,
                             "scaling": {"factor": 8.0, "original": 2048, "fast": 32.0, "slow": 1.0}}}
            layers.append({"type": "latent_attention", "mixer": mixer, "mlp": mlp})
    return {"architecture": "Birizen", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-6}, "layers": layers,
            "loop": dict(zip(("start", "stop", "times"), s["loop"]))}


def random_birizen_weights(cfg: dict, device, dtype, seed=0) -> Dict[str, torch.Tensor]:
    g = torch.Generator(device=device).manual_seed(seed)
    D, out = cfg["width"], {}

    def lin(name, o, i, gain=1.0):
        out[name] = (torch.randn(o, i, generator=g, device=device) * (gain / math.sqrt(i))).to(dtype)

    def vec(name, n, mean=1.0, std=0.1):
        out[name] = (mean + std * torch.randn(n, generator=g, device=device)).to(dtype)

    out["embed"] = torch.randn(cfg["vocab"], D, generator=g, device=device).to(dtype)
    lin("loop.in", D, 2 * D)
    out["loop.step"] = (0.1 * torch.randn(cfg["loop"]["times"], D, generator=g, device=device)).to(dtype)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        for n in ("norm1", "norm1b", "norm2", "norm2b"):
            vec(p + n, D)
        H = m["heads"]
        if L["type"] == "lightning":
            lin(p + "mix.q", H * m["dim"], D), lin(p + "mix.k", H * m["dim"], D), lin(p + "mix.v", H * m["vdim"], D)
            lin(p + "mix.g", H * m["vdim"], D), lin(p + "mix.o", D, H * m["vdim"]), vec(p + "mix.norm", H * m["vdim"])
        else:
            lin(p + "mix.dq", m["q_rank"], D), vec(p + "mix.dq.norm", m["q_rank"])
            lin(p + "mix.uq", H * (m["dim"] + m["rot_dim"]), m["q_rank"])
            lin(p + "mix.dkv", m["kv_rank"] + m["rot_dim"], D), vec(p + "mix.dkv.norm", m["kv_rank"])
            lin(p + "mix.uk", H * m["dim"], m["kv_rank"]), lin(p + "mix.uv", H * m["vdim"], m["kv_rank"])
            vec(p + "mix.sink", H, 0.0, 1.0), lin(p + "mix.g", H * m["vdim"], D), lin(p + "mix.o", D, H * m["vdim"])
        ml = L["mlp"]
        for e in range(ml["router"]["experts"]):
            lin(f"{p}mlp.e{e}.gate", ml["expert"]["ff"], D), lin(f"{p}mlp.e{e}.up", ml["expert"]["ff"], D)
            lin(f"{p}mlp.e{e}.down", D, ml["expert"]["ff"])
        lin(p + "mlp.router", ml["router"]["experts"], D, 2.0)
        vec(p + "mlp.correction", ml["router"]["experts"], 0.0, 0.05)
        lin(p + "mlp.shared.gate", ml["shared"]["ff"], D), lin(p + "mlp.shared.up", ml["shared"]["ff"], D)
        lin(p + "mlp.shared.down", D, ml["shared"]["ff"])
    vec("final.norm", D)
    return out


def _birizen_run_layers(s: dict, cfg: dict) -> List[dict]:
    a, b, times = s["loop"]
    order = list(range(a)) + list(range(a, b)) * times + list(range(b, s["layers"]))
    return [cfg["layers"][i] for i in order]


def birizen_work(s: dict, cfg: dict, T1: int, seqs: int) -> Dict[str, tuple]:
    """name -> (FLOPs, bytes) of one step over `seqs` prompts of T1 tokens (bf16 operands, fp32 residual stream and
    recurrent state), summed over the layer runs."""
    T, D = T1 * seqs, s["width"]
    H, dim, vdim, rot, qr, kr = s["heads"], s["dim"], s["vdim"], s["rot_dim"], s["q_rank"], s["kv_rank"]
    E, top, F, S = s["experts"], s["top"], s["expert_ff"], s["shared_ff"]
    w: Dict[str, List[float]] = {}

    def add(name, flops, nbytes):
        a = w.setdefault(name, [0.0, 0.0])
        a[0] += flops
        a[1] += nbytes

    all_keys = seqs * T1 * (T1 + 1) // 2
    add("norm", 0, (1 + s["loop"][2]) * T * D * (4 + 4 + 2))
    add("loop_in", s["loop"][2] * 2 * T * 2 * D * D, s["loop"][2] * (T * D * (8 + 4 + 4) + 2 * 2 * D * D))
    for L in _birizen_run_layers(s, cfg):
        if L["type"] == "lightning":
            nk, nv = H * dim, H * vdim
            npj = 2 * nk + 2 * nv
            add("proj", 2 * T * D * npj, 2 * (T * D + npj * D + T * npj))
            add("lightning_prep", 0, T * (2 * nk + nv) * (2 + 4))                               # fp32 records out
            add("lightning", 4 * T * H * dim * vdim, T * (4 * (2 * nk + nv) + 4 * nv))          # fp32 FMAs, not tensor work
            add("headnorm_gate", 0, T * nv * (4 + 2 + 2))
            add("o", 2 * T * nv * D, 2 * (T * nv + nv * D + T * D))
        else:
            hq, hv, ldq = H * (dim + rot), H * vdim, kr + rot
            npj = qr + kr + rot + hv
            add("proj", 2 * T * D * npj, 2 * (T * D + npj * D + T * npj))
            add("latent_prep", 0, 2 * T * (2 * qr + 2 * (kr + rot)))
            add("q_up", 2 * T * qr * hq, 2 * (T * qr + hq * qr + T * hq))
            add("q_absorb", 2 * T * H * dim * kr, 2 * (T * hq + H * dim * kr + T * H * ldq))
            add("latent_attention", 2 * all_keys * H * (ldq + kr), 2 * T * H * (ldq + kr) + 2 * T * ldq)
            add("v_up_gate", 2 * T * H * kr * vdim, 2 * (T * H * kr + H * vdim * kr + 2 * T * hv))
            add("o", 2 * T * hv * D, 2 * (T * hv + hv * D + T * D))
        P = T * top
        add("post_norm", 0, 2 * T * D * (2 + 4 + 4 + 2))
        add("moe_route", 2 * T * D * E, 2 * T * D)
        add("moe_sort", 0, 4 * 3 * P)
        add("moe_gather", 0, 2 * 2 * P * D)
        add("moe_gate_up", 2 * P * D * 2 * F, 2 * (P * D + E * 2 * F * D + P * F))
        add("moe_down", 2 * P * F * D, 2 * (P * F + E * F * D + P * D))
        add("shared_gate_up", 2 * T * D * 2 * S, 2 * (T * D + 2 * S * D + 2 * T * S + T * S))
        add("shared_down", 2 * T * S * D, 2 * (T * S + S * D + T * D))
        add("moe_combine", 0, 2 * P * D + T * D * (2 + 2))
    add("head", 2 * seqs * D * s["vocab"], 2 * D * s["vocab"])
    return {k: (v[0], v[1]) for k, v in w.items()}


def _birizen_decode_bytes(s: dict, cfg: dict, B: int) -> float:
    """Weight bytes one decode step of B tokens must stream (experts: at most B * top of them per MoE layer run)."""
    D, n = s["width"], 0.0
    H, dim, vdim, rot, qr, kr = s["heads"], s["dim"], s["vdim"], s["rot_dim"], s["q_rank"], s["kv_rank"]
    for L in _birizen_run_layers(s, cfg):
        if L["type"] == "lightning":
            n += D * (2 * H * dim + 3 * H * vdim)
        else:
            n += D * (qr + kr + rot + 2 * H * vdim) + qr * H * (dim + rot) + H * kr * (dim + vdim)
        n += min(s["experts"], B * s["top"]) * 3 * D * s["expert_ff"] + 3 * D * s["shared_ff"] + D * s["experts"]
    n += s["loop"][2] * 2 * D * D + D * s["vocab"]
    return 2.0 * n


# (Birizen op, the like op) against the MoE Mubasun and against Ninisun at equal width
BIRIZEN_LIKE_MUBASUN = [("proj", "proj"), ("loop_in", "o"), ("q_up", "proj"), ("q_absorb", "moe_down"), ("v_up_gate", "moe_down"),
                        ("o", "o"), ("latent_prep", "qknorm_append"), ("latent_attention", "attention"),
                        ("moe_route", "moe_route"), ("moe_gather", "moe_gather"), ("moe_gate_up", "moe_gate_up"),
                        ("moe_down", "moe_down"), ("shared_gate_up", "shared_gate_up"), ("shared_down", "shared_down"),
                        ("moe_combine", "moe_combine"), ("norm", "norm"), ("head", "head")]
BIRIZEN_LIKE_NINISUN = [("lightning", "delta_rule"), ("lightning_prep", "delta_prep"), ("headnorm_gate", "headnorm_gate"), ("post_norm", "post_norm")]


@torch.no_grad()
def run_birizen(sizes, steps: int, warmup: int, peaks: dict, prefill_tokens=2048, prefill_seqs=4, context=1024,
                decode_batches=(1, 8)) -> dict:
    from .birizen import BirizenEngine
    from .mubasun import MubasunEngine
    from .ninisun import NinisunEngine
    dev, dtype = torch.device("cuda:0"), torch.bfloat16
    timer = _Timer()
    result = {}
    launches0 = cabi.launch_count()
    pool = (max(max(decode_batches), prefill_seqs) + 1) * (max(prefill_tokens, context) + 256)
    for name in sizes:
        s = BIRIZEN_SIZES[name]
        cfg = birizen_config(s)
        eng = BirizenEngine(cfg, random_birizen_weights(cfg, dev, dtype), device=dev, dtype=dtype, kv_pool_tokens=pool)
        row = {"size": s}
        row.update(_measure_ragged(eng, s["vocab"], timer, steps, warmup, peaks, birizen_work(s, cfg, prefill_tokens, prefill_seqs),
                                   lambda B: _birizen_decode_bytes(s, cfg, B), prefill_tokens, prefill_seqs, context,
                                   decode_batches))
        del eng
        torch.cuda.empty_cache()
        ms_ = SIZES[name]
        mcfg = mubasun_config(ms_)
        meng = MubasunEngine(mcfg, random_mubasun_weights(mcfg, dev, dtype), device=dev, dtype=dtype, kv_pool_tokens=pool)
        mrow = _measure_ragged(meng, ms_["vocab"], timer, steps, warmup, peaks, mubasun_work(ms_, mcfg, prefill_tokens, prefill_seqs),
                               lambda B: _decode_bytes(ms_, mcfg, B), prefill_tokens, prefill_seqs, context, decode_batches)
        row["mubasun_equal_size"] = mrow
        del meng
        torch.cuda.empty_cache()
        ns_ = NINISUN_SIZES[name]
        ncfg = ninisun_config(ns_)
        neng = NinisunEngine(ncfg, random_ninisun_weights(ncfg, ns_, dev, dtype), device=dev, dtype=dtype, kv_pool_tokens=pool)
        nrow = _measure_ragged(neng, ns_["vocab"], timer, steps, warmup, peaks, ninisun_work(ns_, ncfg, prefill_tokens, prefill_seqs),
                               lambda B: _ninisun_decode_bytes(ns_, ncfg), prefill_tokens, prefill_seqs, context, decode_batches)
        row["ninisun_equal_size"] = nrow
        del neng
        torch.cuda.empty_cache()
        cmpr = {}
        for like, other in ((BIRIZEN_LIKE_MUBASUN, mrow), (BIRIZEN_LIKE_NINISUN, nrow)):
            for a, bname in like:
                if a in row["prefill_ops"] and bname in other["prefill_ops"]:
                    fa, fb = row["prefill_ops"][a]["frac"], other["prefill_ops"][bname]["frac"]
                    cmpr[a] = {"frac": fa, "like": bname, "like_frac": fb, "distance_ratio": round(fb / fa, 2) if fa > 0 else None}
        row["like_for_like"] = cmpr
        result[name] = row
    result["gpu_launches"] = int(cabi.launch_count() - launches0)
    return result


# ---------------------------------------------------------------------------------------------------------------
GOGIVIK_SIZES = {
    # latent layers as Birizen's (window added), attention layers as Ninisun's head layout (blocks instead of a window,
    # per-head norms, rotated values), a state-space layer of inner width 2 x width: ssm_heads x ssm_vdim, state, groups
    "w1024": dict(width=1024, layers=4, heads=8, kv_heads=2, dim=128, vdim=128, rot_dim=64, q_rank=384, kv_rank=192, window=512,
                  chunk=512, ssm_heads=32, ssm_vdim=64, state=128, groups=1, norm_groups=1, conv=4, taps=4, ff=4096, vocab=32000),
    "w2048": dict(width=2048, layers=4, heads=16, kv_heads=4, dim=128, vdim=128, rot_dim=64, q_rank=768, kv_rank=192, window=1024,
                  chunk=1024, ssm_heads=64, ssm_vdim=64, state=128, groups=1, norm_groups=1, conv=4, taps=4, ff=8192, vocab=32000),
}


def gogivik_config(s: dict) -> dict:
    """latent, attention, mamba2, attention, ... (every branch of the design is on the path)."""
    layers = []
    for i in range(s["layers"]):
        if i % 4 == 0:
            L = {"type": "latent_attention", "mixer": {
                "heads": s["heads"], "dim": s["dim"], "rot_dim": s["rot_dim"], "vdim": s["vdim"], "q_rank": s["q_rank"],
                "kv_rank": s["kv_rank"], "scale": 1.0 / math.sqrt(s["dim"] + s["rot_dim"]), "mask": {"size": s["window"]},
                "rot": {"dims": s["rot_dim"], "base": 10000.0}}}
        elif i % 4 == 2:
            L = {"type": "mamba2", "mixer": {"heads": s["ssm_heads"], "vdim": s["ssm_vdim"], "state": s["state"],
                                             "groups": s["groups"], "norm_groups": s["norm_groups"], "conv": s["conv"]}}
        else:
            L = {"type": "attention", "mixer": {
                "heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["vdim"],
                "scale": 1.0 / math.sqrt(s["dim"]), "mask": {"size": s["chunk"]},
                "rot": {"dims": s["dim"], "base": 10000.0, "scaling": {"factor": 2.0}}}}
        L["mlp"] = {"kind": "dense", "ff": s["ff"]}
        layers.append(L)
    return {"architecture": "Gogivik", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-6},
            "canon": {"taps": s["taps"]}, "logit_scale": 1.0, "layers": layers}


def random_gogivik_weights(cfg: dict, device, dtype, seed=0) -> Dict[str, torch.Tensor]:
    g = torch.Generator(device=device).manual_seed(seed)
    D, out, taps = cfg["width"], {}, cfg["canon"]["taps"]

    def lin(name, o, i, gain=1.0):
        out[name] = (torch.randn(o, i, generator=g, device=device) * (gain / math.sqrt(i))).to(dtype)

    def vec(name, n, mean=0.0, std=0.1):
        out[name] = (mean + std * torch.randn(n, generator=g, device=device)).to(dtype)

    out["embed"] = torch.randn(cfg["vocab"], D, generator=g, device=device).to(dtype)
    lin("head", cfg["vocab"], D)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        for n in ("norm1", "norm2"):
            vec(p + n, D)
        for n in ("canon1", "canon2"):
            out[p + n] = (0.2 * torch.randn(D, taps, generator=g, device=device)).to(dtype)
        if L["type"] == "latent_attention":
            H = m["heads"]
            lin(p + "mix.dq", m["q_rank"], D), vec(p + "mix.dq.norm", m["q_rank"], 1.0)
            lin(p + "mix.uq", H * (m["dim"] + m["rot_dim"]), m["q_rank"])
            lin(p + "mix.dkv", m["kv_rank"] + m["rot_dim"], D), vec(p + "mix.dkv.norm", m["kv_rank"], 1.0)
            lin(p + "mix.uk", H * m["dim"], m["kv_rank"]), lin(p + "mix.uv", H * m["vdim"], m["kv_rank"])
            vec(p + "mix.sink", H, 0.0, 1.0), lin(p + "mix.o", D, H * m["vdim"])
        elif L["type"] == "attention":
            H, G = m["heads"], m["kv_heads"]
            lin(p + "mix.q", H * m["dim"], D), lin(p + "mix.k", G * m["dim"], D), lin(p + "mix.v", G * m["vdim"], D)
            vec(p + "mix.q.norm", m["dim"], 1.0), vec(p + "mix.k.norm", m["dim"], 1.0), lin(p + "mix.o", D, H * m["vdim"])
        else:
            inner, ch = m["heads"] * m["vdim"], m["heads"] * m["vdim"] + 2 * m["groups"] * m["state"]
            lin(p + "mix.in", inner + ch + m["heads"], D)
            out[p + "mix.conv"] = (0.3 * torch.randn(ch, m["conv"], generator=g, device=device)).to(dtype)
            vec(p + "mix.conv.b", ch), vec(p + "mix.dt_bias", m["heads"], -1.0, 0.5), vec(p + "mix.A_log", m["heads"], -1.0, 0.5)
            vec(p + "mix.D", m["heads"], 1.0), vec(p + "mix.norm", inner, 1.0), lin(p + "mix.o", D, inner)
        lin(p + "mlp.up", L["mlp"]["ff"], D), lin(p + "mlp.down", D, L["mlp"]["ff"])
    vec("final.norm", D)
    return out


def gogivik_work(s: dict, cfg: dict, T1: int, seqs: int) -> Dict[str, tuple]:
    """name -> (FLOPs, bytes) of one step over `seqs` prompts of T1 tokens (bf16 operands, fp32 residual stream, fp32
    normed rows into the input convolutions, fp32 scan records and state)."""
    T, D, F = T1 * seqs, s["width"], s["ff"]
    w: Dict[str, List[float]] = {}

    def add(name, flops, nbytes):
        a = w.setdefault(name, [0.0, 0.0])
        a[0] += flops
        a[1] += nbytes

    def gemm(name, N, K):
        add(name, 2 * T * N * K, 2 * (T * K + N * K + T * N))

    for L in cfg["layers"]:
        m = L["mixer"]
        add("norm_conv", 0, 2 * T * D * (4 + 2 + 4 + 2))                  # x, y in; x, h out: both sublayers (fused kernel)
        add("norm", 0, 2 * T * D * (4 + 2 + 4 + 4))                       # the separate kernels (PG_GOGIVIK_FUSED_READ=0):
        add("input_conv", 0, 2 * T * D * (4 + 2))                         # x, y in; x, normed fp32 row out | normed row in, h out
        if L["type"] == "latent_attention":
            H, dim, vdim, rot, qr, kr, W = m["heads"], m["dim"], m["vdim"], m["rot_dim"], m["q_rank"], m["kv_rank"], m["mask"]["size"]
            hq, hv, ldq = H * (dim + rot), H * vdim, kr + rot
            keys = seqs * sum(min(i + 1, W) for i in range(T1))
            gemm("proj", qr + kr + rot, D)
            add("latent_prep", 0, 2 * T * (2 * qr + 2 * (kr + rot)))
            gemm("q_up", hq, qr)
            add("q_absorb", 2 * T * H * dim * kr, 2 * (T * hq + H * dim * kr + T * H * ldq))
            add("latent_attention", 2 * keys * H * (ldq + kr), 2 * T * H * (ldq + kr) + 2 * T * ldq)
            add("v_up", 2 * T * H * kr * vdim, 2 * (T * H * kr + H * vdim * kr + T * hv))
            gemm("o", D, hv)
        elif L["type"] == "attention":
            H, G, dim, vdim, C = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["mask"]["size"]
            keys = seqs * sum(i % C + 1 for i in range(T1))
            n = H * dim + G * dim + G * vdim
            gemm("proj", n, D)
            add("headnorm_rotary_append", 0, 2 * 2 * T * n)
            add("attention", 2 * keys * H * (dim + vdim), 2 * T * (H * dim + H * vdim + G * dim + G * vdim))
            gemm("o", D, H * vdim)
        else:
            H, e, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
            inner, ch = H * e, H * e + 2 * G * N
            rec = H * (2 * N + e + 4)
            gemm("proj", inner + ch + H, D)
            add("ssm_prep", 0, T * (2 * (ch + H) + 4 * rec))
            add("ssm_scan", 4 * T * H * N * e, T * 4 * (rec + inner))        # fp32 FMAs, not tensor work
            add("gate_groupnorm", 0, T * inner * (4 + 2 + 2))
            gemm("o", D, inner)
        gemm("up", F, D)
        add("relu2", 0, T * F * (2 + 2))
        gemm("down", D, F)
    add("head", 2 * seqs * D * s["vocab"], 2 * D * s["vocab"])
    return {k: (v[0], v[1]) for k, v in w.items()}


def _gogivik_decode_bytes(s: dict, cfg: dict) -> float:
    """Weight bytes one decode step must stream."""
    D, n = s["width"], 0.0
    for L in cfg["layers"]:
        m = L["mixer"]
        if L["type"] == "latent_attention":
            H = m["heads"]
            n += D * (m["q_rank"] + m["kv_rank"] + m["rot_dim"] + H * m["vdim"]) + m["q_rank"] * H * (m["dim"] + m["rot_dim"]) + \
                H * m["kv_rank"] * (m["dim"] + m["vdim"])
        elif L["type"] == "attention":
            n += D * (2 * m["heads"] * m["dim"] + m["kv_heads"] * (m["dim"] + m["vdim"]))
        else:
            inner = m["heads"] * m["vdim"]
            n += D * (3 * inner + 2 * m["groups"] * m["state"] + m["heads"])
        n += 2 * D * L["mlp"]["ff"]
    return 2.0 * (n + D * s["vocab"])


GOGIVIK_LIKE_NINISUN = [("proj", "proj"), ("o", "o"), ("up", "gate_up"), ("down", "down"), ("attention", "attention"),
                        ("headnorm_rotary_append", "rotary_append"), ("gate_groupnorm", "headnorm_gate"), ("norm", "post_norm"),
                        ("input_conv", "post_norm"), ("norm_conv", "post_norm"), ("relu2", "headnorm_gate"), ("head", "head")]
GOGIVIK_LIKE_BIRIZEN = [("latent_prep", "latent_prep"), ("q_up", "q_up"), ("q_absorb", "q_absorb"),
                        ("latent_attention", "latent_attention"), ("v_up", "v_up_gate"), ("ssm_scan", "lightning"),
                        ("ssm_prep", "lightning_prep")]


@torch.no_grad()
def run_gogivik(sizes, steps: int, warmup: int, peaks: dict, prefill_tokens=2048, prefill_seqs=4, context=1024,
                decode_batches=(1, 8)) -> dict:
    from .birizen import BirizenEngine
    from .gogivik import GogivikEngine
    from .ninisun import NinisunEngine
    dev, dtype = torch.device("cuda:0"), torch.bfloat16
    timer = _Timer()
    result = {}
    launches0 = cabi.launch_count()
    pool = (max(max(decode_batches), prefill_seqs) + 1) * (max(prefill_tokens, context) + 256)
    for name in sizes:
        s = GOGIVIK_SIZES[name]
        cfg = gogivik_config(s)
        eng = GogivikEngine(cfg, random_gogivik_weights(cfg, dev, dtype), device=dev, dtype=dtype, kv_pool_tokens=pool)
        row = {"size": s}
        row.update(_measure_ragged(eng, s["vocab"], timer, steps, warmup, peaks, gogivik_work(s, cfg, prefill_tokens, prefill_seqs),
                                   lambda B: _gogivik_decode_bytes(s, cfg), prefill_tokens, prefill_seqs, context, decode_batches))
        del eng
        torch.cuda.empty_cache()
        ns_ = NINISUN_SIZES[name]
        ncfg = ninisun_config(ns_)
        neng = NinisunEngine(ncfg, random_ninisun_weights(ncfg, ns_, dev, dtype), device=dev, dtype=dtype, kv_pool_tokens=pool)
        nrow = _measure_ragged(neng, ns_["vocab"], timer, steps, warmup, peaks, ninisun_work(ns_, ncfg, prefill_tokens, prefill_seqs),
                               lambda B: _ninisun_decode_bytes(ns_, ncfg), prefill_tokens, prefill_seqs, context, decode_batches)
        row["ninisun_equal_size"] = nrow
        del neng
        torch.cuda.empty_cache()
        bs_ = BIRIZEN_SIZES[name]
        bcfg = birizen_config(bs_)
        beng = BirizenEngine(bcfg, random_birizen_weights(bcfg, dev, dtype), device=dev, dtype=dtype, kv_pool_tokens=pool)
        brow = _measure_ragged(beng, bs_["vocab"], timer, steps, warmup, peaks, birizen_work(bs_, bcfg, prefill_tokens, prefill_seqs),
                               lambda B: _birizen_decode_bytes(bs_, bcfg, B), prefill_tokens, prefill_seqs, context, decode_batches)
        row["birizen_equal_size"] = brow
        del beng
        torch.cuda.empty_cache()
        cmpr = {}
        for like, other in ((GOGIVIK_LIKE_NINISUN, nrow), (GOGIVIK_LIKE_BIRIZEN, brow)):
            for a, bname in like:
                if a in row["prefill_ops"] and bname in other["prefill_ops"]:
                    fa, fb = row["prefill_ops"][a]["frac"], other["prefill_ops"][bname]["frac"]
                    cmpr[a] = {"frac": fa, "like": bname, "like_frac": fb, "distance_ratio": round(fb / fa, 2) if fa > 0 else None}
        row["like_for_like"] = cmpr
        result[name] = row
    result["gpu_launches"] = int(cabi.launch_count() - launches0)
    return result
