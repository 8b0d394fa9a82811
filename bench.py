#!/usr/bin/env python3
"""Decode and prefill throughput of the LFM3 hybrid engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--impl ours|reference]

Default run: the LFM2-1.2B-shaped configuration (16 layers: attention at 2, 5, 8, 10, 12, 14,
short convolution elsewhere; hidden 2048, 32 heads, 8 kv heads, head size 64, feed-forward 5632,
vocabulary 65536), bfloat16 random weights, batch 8, every sequence ending at context 4096.
A step is one decode step of the whole batch.  One JSON line goes to stdout:

  value      decoded tokens per second, timed on the device over K graph-replayed steps that feed
             themselves (the chosen tokens become the next input on the device)
  e2e        the same through the Python entry point (`Engine.generate`): host token ids in, host
             token ids out, every step copying its inputs from pinned memory and reading its
             tokens back
  prefill    one prompt of 2,048 tokens: tokens/s, and the fraction of the bf16 peak
  roofline   the bytes a decode step must read (every weight once, the cache of the live
             sequences) over its time, against the measured copy bandwidth
  points     decode tokens/s at batch 1 and 64, same context; and the scenario of 512-token
             prompts followed by 256 decode steps (context 512 to 768) at batch 1, 8 and 64, each with
             its milliseconds per step and its fraction of the copy bandwidth (p512_*)
  roofline.kernels   the kernels a decode step and the prompt spend most of their time in, each timed
             with CUDA events around its launches (one kernel after the other, outside the timed
             runs) against the bytes or flops it has to move

Weights (1.8 GB) are far larger than L2, so consecutive steps cannot be served from L2.

`--compare zekivik` (or `lenesun`, `kisilix`, `tevilix`) leaves all of that aside and prints a line of its own: prompt and decode times
of that design at a few layer sizes beside the closest LFM3 model at equal sizes, with every kernel entry point's time.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CONFIG_1P2B = {
    "architectures": ["Lfm3ForCausalLM"], "model_type": "lfm3",
    "vocab_size": 65536, "hidden_size": 2048, "num_hidden_layers": 16,
    "layer_types": ["conv", "conv", "attention", "conv", "conv", "attention", "conv", "conv", "attention",
                    "conv", "attention", "conv", "attention", "conv", "attention", "conv"],
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64,
    "intermediate_size": 8192, "block_auto_adjust_ff_dim": True, "block_multiple_of": 256,
    "block_ffn_dim_multiplier": 1.0, "rope_theta": 1000000.0, "conv_L_cache": 3, "norm_eps": 1e-5,
    "tie_embedding": True, "max_position_embeddings": 128000,
}


def _layers(n: int, attention_at: list[int]) -> list[str]:
    return ["attention" if i in attention_at else "conv" for i in range(n)]


# the other shapes the reference's numbers are quoted on; the default run is the 1.2B shape
CONFIG_2P6B = dict(CONFIG_1P2B, num_hidden_layers=30, layer_types=_layers(30, [2, 6, 10, 14, 18, 21, 24, 27]),
                   intermediate_size=7168, block_auto_adjust_ff_dim=False)
CONFIG_8B_A1B = dict(CONFIG_1P2B, num_hidden_layers=24, layer_types=_layers(24, [2, 6, 10, 14, 18, 21]),
                     intermediate_size=7168, block_auto_adjust_ff_dim=False, num_dense_layers=2, num_experts=32,
                     num_experts_per_tok=4, moe_intermediate_size=1792, norm_topk_prob=True, use_expert_bias=True,
                     routed_scaling_factor=1.0)
MODELS = {"1.2b": ("LFM2-1.2B-shaped LFM3 hybrid", CONFIG_1P2B), "2.6b": ("LFM2-2.6B-shaped LFM3 hybrid", CONFIG_2P6B),
          "8b-a1b": ("LFM2-8B-A1B-shaped LFM3 hybrid MoE", CONFIG_8B_A1B)}
CONTEXT = 4096
PREFILL_TOKENS = 2048
P512_PROMPT, P512_STEPS = 512, 256      # the decode scenario the reference's numbers are defined on
E2E_MIN_STEPS = 256                     # the end-to-end run never has fewer decode steps than this
E2E_FIRST_STEPS = 32                    # ... and says separately how the first ones after the prompts went
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks() -> tuple[dict, str]:
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(p) as f:
            raw = json.load(f)
        out = {k: float(raw[k]) for k in ("hbm_gbs", "bf16_tflops") if k in raw}
        out["bf16_tflops_sustained"] = float(raw.get("bf16_tflops_sustained", out.get("bf16_tflops", 0)))
        if "hbm_gbs" in out and "bf16_tflops" in out:
            return out, "measured"
    except (OSError, ValueError, KeyError, TypeError):
        pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0):
        self.rows: list[list[str]] = []
        self.proc = None
        self.index = index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "25", "-i", str(self.index)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def mark(self) -> int:
        return len(self.rows)

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()

    def summary(self, lo: int = 0, hi: int | None = None) -> dict:
        rows = self.rows[lo:hi] or self.rows
        mhz = [float(r[0]) for r in rows if r and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in rows if len(r) > 1 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 3 + i and r[3 + i].lower().startswith("active") for r in rows)]
        return {"sm_mhz": statistics.median(mhz) if mhz else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(rows)}


def model_numbers(eng) -> dict:
    """Bytes and flops of a step, from what the engine's parts say of themselves."""
    c = eng.step_costs()
    return {"weight_bytes": eng.weight_bytes(), "kv_bytes_per_token": c["kv_bytes_per_token"],
            "state_bytes_per_seq": c["state_bytes_per_seq"], "linear_flops_per_token": c["layer_flops_per_row"],
            "head_flops_per_row": c["head_flops_per_row"], "attn_flops_per_qk": c["flops_per_query_key"]}


def decode_step_bytes(eng, nums: dict, batch: int, avg_context: float) -> float:
    """What a decode step has to read: every weight it uses once (of experts the share that `batch`
    rows are expected to choose), the cache of the live sequences, and their fixed-size state (read
    and written)."""
    return (eng.weight_bytes_read(batch) + batch * avg_context * nums["kv_bytes_per_token"]
            + 2 * batch * nums["state_bytes_per_seq"])


def time_prefill(eng, n_tokens: int, warmup: int, reps: int, rng) -> float:
    import torch
    toks = rng.integers(0, eng.vocab_size, size=n_tokens).tolist()
    ms = []
    for i in range(warmup + reps):
        s = eng.new_sequence()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        eng.step([s], [toks], "last")
        b.record()
        torch.cuda.synchronize()
        eng.release(s)
        if i >= warmup:
            ms.append(a.elapsed_time(b))
    return statistics.median(ms)


def fill_context(eng, batch: int, length: int, rng, chunk: int = 8192) -> list[int]:
    """`batch` sequences holding `length` random tokens each."""
    seqs = [eng.new_sequence() for _ in range(batch)]
    per = max(1, chunk // max(1, min(length, chunk)))
    for lo in range(0, batch, per):
        group = seqs[lo:lo + per]
        done = 0
        while done < length:
            n = min(length - done, chunk)
            eng.step(group, [rng.integers(0, eng.vocab_size, size=n).tolist() for _ in group], None)
            done += n
    return seqs


def time_decode(eng, batch: int, context: int, steps: int, warmup: int, rng, clocks=None) -> dict:
    """K self-feeding graph-replayed decode steps of `batch` sequences that end at `context`."""
    import torch
    from lastengine_b200.engine.graph import DecodeGraph
    from lastengine_b200.sampling.params import SamplingParams
    from lastengine_b200.sampling.sampler import Sampler
    from lastengine_b200.ops import kernels
    start_len = context - (steps + warmup + 1)
    seqs = fill_context(eng, batch, start_len, rng)
    total = steps + warmup + 1
    g = DecodeGraph(eng, Sampler(SamplingParams(temperature=0.0), eng.device), batch,
                    table_width=-(-context // eng.cache.page_size), self_feeding=True)
    # room for every step of the run up front, so the page tables stay valid while the graph feeds itself
    eng.cache.reserve({s: total for s in seqs})
    grow = g.stage(seqs, rng.integers(0, eng.vocab_size, size=batch).tolist(), None)
    g.launch()                                      # warm-up run + capture (the step has run once)
    for _ in range(warmup):
        g.launch()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    lo = clocks.mark() if clocks else 0
    a.record()
    for _ in range(steps):
        g.launch()
    b.record()
    torch.cuda.synchronize()
    hi = clocks.mark() if clocks else 0
    ms = a.elapsed_time(b) / steps
    eng.cache.commit({s: total for s in seqs})
    avg_len = start_len + 1 + warmup + steps / 2
    eng.release(seqs)
    return {"ms_per_step": ms, "tok_s": batch * 1e3 / ms, "launches_per_step": g.launches,
            "avg_context": avg_len, "clock_rows": (lo, hi)}


def time_e2e(eng, batch: int, context: int, steps: int, rng) -> dict:
    """The same decode through Engine.generate: host ids in, host ids out, every step.  `value` is
    over all `steps` decode steps of one call; `first_steps_value` over the first E2E_FIRST_STEPS of
    a call of its own (right after the prompts the device runs at its power cap for some tens of
    milliseconds, which a short run shows and a long one averages out)."""
    from lastengine_b200 import SamplingParams
    greedy = SamplingParams(temperature=0.0)
    prompts = [rng.integers(0, eng.vocab_size, size=context - steps - 1).tolist() for _ in range(batch)]
    # short calls first: they capture the decode graphs of this batch size, as a server's first requests would
    eng.generate([p[:64] for p in prompts], greedy, max_new_tokens=4, stop_token_ids=[], max_batch=batch, max_seq_len=context + 1)
    eng.generate(prompts, greedy, max_new_tokens=4, stop_token_ids=[], max_batch=batch, max_seq_len=context + 1)
    first = eng.generate(prompts, greedy, max_new_tokens=E2E_FIRST_STEPS + 1, stop_token_ids=[], max_batch=batch,
                         max_seq_len=context + 1).stats
    res = eng.generate(prompts, greedy, max_new_tokens=steps + 1, stop_token_ids=[], max_batch=batch, max_seq_len=context + 1)
    st = res.stats
    return {"value": st.decode_tok_s, "unit": "tokens/s", "h2d_bytes_per_step": res.backend.h2d_bytes,
            "d2h_bytes_per_step": res.backend.d2h_bytes, "decode_steps": st.decode_steps,
            "first_steps": first.decode_steps, "first_steps_value": first.decode_tok_s,
            "prefill_tok_s": st.prefill_tok_s}


# kernel entry points by what they do, for roofline.kernels
KERNEL_CLASSES = {
    "leb_gemm_bf16_stream": "weight-streaming products", "leb_gemm_bf16_stream_conv": "weight-streaming products",
    "leb_gemm_bf16_stream_grouped": "weight-streaming products", "leb_gemm_bf16_skinny": "weight-streaming products",
    "leb_gemm_bf16_small": "weight-streaming products",
    "leb_attention_decode": "decode attention", "leb_attention_decode_prep": "decode attention",
    "leb_attention_merge": "decode attention",
    "leb_gemm_bf16_tc": "tcgen05 products", "leb_gemm_bf16_tc2": "tcgen05 products", "leb_gemm_bf16_tc_grouped": "tcgen05 products",
    "leb_attention_prefill_tc": "tcgen05 prompt attention", "leb_attention_prefill": "prompt attention",
}


def time_kernels(eng, nums: dict, batch: int, context: int, pk: dict, rng) -> list[dict]:
    """One decode step of `batch` sequences at `context` and one prompt of PREFILL_TOKENS under the
    per-kernel event timer (launched one by one, no graph): for the kernel classes that take most of
    each, the time of their launches against the bytes (decode) or flops (prompt) they have to move."""
    import torch
    from lastengine_b200.ops import kernels
    out = []
    seqs = fill_context(eng, batch, context - 2, rng)
    eng.step(seqs, [[1]] * batch, "last")                      # warm: kernels loaded, scratch sized
    torch.cuda.synchronize()
    with kernels.KernelTimer(head_start_ms=5.0) as t:
        eng.step(seqs, [[2]] * batch, "last")
    eng.release(seqs)
    work = {"weight-streaming products": eng.weight_bytes_read(batch),
            "decode attention": batch * context * nums["kv_bytes_per_token"]}
    out += _classes(t.summary(), work, "GB/s", 1e9, pk["hbm_gbs"], f"decode step, batch {batch}, context {context}")
    toks = rng.integers(0, eng.vocab_size, size=PREFILL_TOKENS).tolist()
    s = eng.new_sequence()
    eng.step([s], [toks], "last")
    eng.release(s)
    s = eng.new_sequence()
    torch.cuda.synchronize()
    with kernels.KernelTimer(head_start_ms=5.0) as t:
        eng.step([s], [toks], "last")
    eng.release(s)
    work = {"tcgen05 products": PREFILL_TOKENS * nums["linear_flops_per_token"],
            "tcgen05 prompt attention": nums["attn_flops_per_qk"] * PREFILL_TOKENS * (PREFILL_TOKENS + 1) // 2}
    out += _classes(t.summary(), work, "TFLOP/s", 1e12, pk["bf16_tflops"], f"prompt of {PREFILL_TOKENS} tokens")
    return out


def _classes(summary: dict, work: dict, unit: str, per: float, peak: float, where: str) -> list[dict]:
    acc: dict[str, list] = {}
    total = sum(ms for _, ms in summary.values())
    for name, (calls, ms) in summary.items():
        e = acc.setdefault(KERNEL_CLASSES.get(name, name), [0, 0.0])
        e[0] += calls
        e[1] += ms
    rows = []
    for cls, (calls, ms) in sorted(acc.items(), key=lambda kv: -kv[1][1])[:3]:
        row = {"where": where, "kernels": cls, "launches": calls, "ms": ms, "share_of_kernel_time": ms / total if total else 0.0}
        if cls in work and ms > 0:
            row.update({"achieved": work[cls] / (ms / 1e3) / per, "unit": unit, "frac": work[cls] / (ms / 1e3) / per / peak})
        rows.append(row)
    return rows


# ---- the Zekivik design beside the LFM3 hybrid at equal layer sizes (--compare zekivik) -------------------
def zekivik_config(width: int, ff: int, heads: int, kv_heads: int, dim: int, vdim: int, ret_heads: int,
                   ret_dim: int, ret_vdim: int, layers: int, vocab: int, loop: bool = True) -> dict:
    """Layers alternate retention and attention, every layer with a feed-forward; the first two run twice
    (`loop`)."""
    att = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": 4, "scale": dim ** -0.5,
           "rot": {"dims": dim, "base": 1000000.0}}
    ret = {"heads": ret_heads, "dim": ret_dim, "vdim": ret_vdim,
           "decay": [1.0 - 2.0 ** (-5 - (i % 8)) for i in range(ret_heads)], "rot": {"dims": ret_dim, "base": 10000.0}}
    ls = [{"type": "retention" if i % 2 == 0 else "attention", "mixer": ret if i % 2 == 0 else att,
           "mlp": {"kind": "dense", "ff": ff}} for i in range(layers)]
    return {"architecture": "Zekivik", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "layers": ls,
            "loop": {"start": 0, "stop": 2, "times": 2 if loop else 1}}


def lfm3_like(width: int, ff: int, heads: int, kv_heads: int, dim: int, runs: int, vocab: int) -> dict:
    """The closest existing design at the same sizes: as many layer runs, short convolution where the
    other has retention, the same attention and feed-forward widths."""
    return {"architectures": ["Lfm3ForCausalLM"], "model_type": "lfm3", "vocab_size": vocab, "hidden_size": width,
            "num_hidden_layers": runs, "layer_types": ["conv" if i % 2 == 0 else "attention" for i in range(runs)],
            "num_attention_heads": heads, "num_key_value_heads": kv_heads, "head_dim": dim, "intermediate_size": ff,
            "block_auto_adjust_ff_dim": False, "rope_theta": 1000000.0, "conv_L_cache": 4, "norm_eps": 1e-5,
            "tie_embedding": False, "max_position_embeddings": 128000}


COMPARE_SIZES = {   # width, ff, heads, kv heads, head size, value head size, retention heads / key size / value size, layers
    "w2048": dict(width=2048, ff=5632, heads=32, kv_heads=8, dim=64, vdim=64, ret_heads=16, ret_dim=128, ret_vdim=128, layers=6),
    "w1024": dict(width=1024, ff=4096, heads=16, kv_heads=4, dim=64, vdim=64, ret_heads=8, ret_dim=64, ret_vdim=128, layers=6),
    "w2048-v32": dict(width=2048, ff=5632, heads=32, kv_heads=8, dim=64, vdim=32, ret_heads=32, ret_dim=32, ret_vdim=64, layers=6),
}

# what a launch of the new design's own kernels has to move, per row of the step (bytes) -- for the roofline of
# the memory-bound ones; the products and the attention kernels are the ones the other design runs too
def _new_kernel_bytes(cfg: dict, rows: int, batch: int) -> dict:
    W = cfg["width"]
    out = {"leb_gated_residual": 0, "leb_gated_act": 0, "leb_stream_add": 0, "leb_causal_conv": 0, "leb_retention": 0}
    runs = []
    lp = cfg["loop"]
    for i, l in enumerate(cfg["layers"]):
        runs += [l] * (lp["times"] if lp["start"] <= i < lp["stop"] else 1)
    for l in runs:
        m = l["mixer"]
        n_sub = 2 if l["mlp"] else 1
        out["leb_gated_residual"] += n_sub * rows * W * 16                     # x read and written, y and z read (float)
        if l["mlp"]:
            out["leb_gated_act"] += rows * l["mlp"]["ff"] * (8 + 2)            # gate and up (float) in, bfloat16 out
        if l["type"] == "attention":
            C = (m["heads"] + m["kv_heads"]) * m["dim"] + m["kv_heads"] * m["vdim"]
            out["leb_causal_conv"] += rows * C * 4 + batch * C * (m["conv"] - 1) * 8
        else:
            H, d, e = m["heads"], m["dim"], m["vdim"]
            out["leb_retention"] += rows * H * (2 * d + 3 * e) * 2 + batch * H * d * e * 8
    out["leb_stream_add"] = lp["times"] * rows * W * 12
    return out


# ---- the Lenesun design beside an LFM3 model of attention layers with experts (--compare lenesun) --------
def lenesun_config(width: int, heads: int, dim: int, rot_dim: int, vdim: int, q_rank: int, kv_rank: int,
                   experts: int, top: int, ff: int, layers: int, vocab: int) -> dict:
    """Latent attention and experts in every layer; the last two layers read the rows the layer before them cached."""
    def mixer(kv_from=None):
        m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
             "scale": (dim + rot_dim) ** -0.5, "rot": {"dims": rot_dim, "base": 10000.0}}
        if kv_from is not None:
            m["kv_from"] = kv_from
        return m
    mlp = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": 7.0}}
    ls = [{"type": "latent_attention", "mixer": mixer(layers - 3 if i >= layers - 2 else None), "mlp": mlp}
          for i in range(layers)]
    return {"architecture": "Lenesun", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "residual_mult": 0.5,
            "embedding": {"scale": 1.0}, "layers": ls}


def lfm3_moe_like(width: int, heads: int, dim: int, experts: int, top: int, ff: int, layers: int, vocab: int) -> dict:
    """The closest existing design at the same sizes: attention in every layer (as many heads of the same
    unrotated size, grouped four to a key/value head) and as many experts of the same width per layer."""
    return {"architectures": ["Lfm3ForCausalLM"], "model_type": "lfm3", "vocab_size": vocab, "hidden_size": width,
            "num_hidden_layers": layers, "layer_types": ["attention"] * layers, "num_attention_heads": heads,
            "num_key_value_heads": max(1, heads // 4), "head_dim": dim, "intermediate_size": ff,
            "block_auto_adjust_ff_dim": False, "rope_theta": 10000.0, "conv_L_cache": 4, "norm_eps": 1e-5,
            "num_experts": experts, "num_experts_per_tok": top, "moe_intermediate_size": ff, "num_dense_layers": 0,
            "tie_embedding": True, "max_position_embeddings": 128000}


LENESUN_SIZES = {
    "w2048": dict(width=2048, heads=16, dim=128, rot_dim=64, vdim=128, q_rank=768, kv_rank=512, experts=32, top=4, ff=1024, layers=6),
    "w1024": dict(width=1024, heads=8, dim=64, rot_dim=32, vdim=64, q_rank=384, kv_rank=256, experts=16, top=2, ff=512, layers=6),
}


def _lenesun_kernel_work(cfg: dict, rows: int, batch: int, context: int) -> dict:
    """What a step's launches of the design's own kernels have to move (bytes) or compute (flops), by entry point."""
    W = cfg["width"]
    out = {"leb_layernorm": rows * W * 6, "leb_scaled_residual": 0, "leb_latent_prep": 0, "leb_latent_q_split": 0,
           "leb_heads_to_rows": 0, "leb_gated_act": 0, "leb_latent_attention": 0}
    attn_flops = 0
    pairs = rows * (rows + 1) // 2 if batch == 1 and rows > 1 else rows * context
    for l in cfg["layers"]:
        m = l["mixer"]
        H, dk = m["heads"], m["kv_rank"] + m["rot_dim"]
        own = "kv_from" not in m
        out["leb_scaled_residual"] += rows * W * 14                       # x read and written, the sum read, the norm written
        out["leb_latent_prep"] += rows * (m["q_rank"] * 4 + (dk * 4 if own else 0))
        out["leb_latent_q_split"] += rows * H * (m["dim"] + m["rot_dim"]) * 4
        out["leb_heads_to_rows"] += rows * H * m["vdim"] * 4
        if l["mlp"]:
            out["leb_gated_act"] += rows * l["mlp"]["router"]["top"] * l["mlp"]["expert"]["ff"] * (8 + 2)
        attn_flops += 2 * H * (dk + m["kv_rank"]) * pairs
        out["leb_latent_attention"] += batch * context * dk * 2 + rows * H * (dk + m["kv_rank"]) * 2
    return {"bytes": out, "attention_flops": attn_flops}


# ---- the Kisilix design beside the Zekivik hybrid at equal layer sizes (--compare kisilix) ---------------
def kisilix_config(width: int, ff: int, heads: int, kv_heads: int, dim: int, vdim: int, ret_heads: int, ret_dim: int,
                   ret_vdim: int, layers: int, vocab: int, window: int, pool: int) -> dict:
    """Recurrent layers (the delta rule and the state-space layer in turn) alternate with windowed attention;
    every layer has the dense feed-forward.  The recurrent layers take the sizes the other design's retention
    has (key size = rows of a head's state), the attention its head sizes."""
    att = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": dim ** -0.5,
           "rot": {"dims": dim, "base": 1000000.0}, "mask": {"size": window, "pool": pool}}
    dlt = {"heads": ret_heads, "kv_heads": ret_heads, "dim": ret_dim, "vdim": ret_vdim, "conv": 4}
    ssm = {"heads": ret_heads, "vdim": ret_vdim, "state": ret_dim, "groups": 1, "norm_groups": 1, "conv": 4}
    ls = []
    for i in range(layers):
        kind, mixer = ("attention", att) if i % 2 else (("channel_delta", dlt) if i % 4 == 0 else ("mamba2", ssm))
        ls.append({"type": kind, "mixer": mixer, "mlp": {"kind": "dense", "ff": ff, "limit": 7.0}})
    return {"architecture": "Kisilix", "vocab": vocab, "width": width, "max_positions": 4096, "norm": {"eps": 1e-5},
            "postln_alpha": 1.0, "layers": ls}


KISILIX_SIZES = {   # as COMPARE_SIZES, and the attention's window and pooled block
    "w2048": dict(COMPARE_SIZES["w2048"], window=1024, pool=64),
    "w1024": dict(COMPARE_SIZES["w1024"], window=512, pool=16),
    "w2048-v32": dict(COMPARE_SIZES["w2048-v32"], window=1024, pool=64),
}


def _seen_keys(i: int, window: int, pool: int) -> int:
    """Positions and pooled blocks that position i sees."""
    return min(i + 1, window) + (max(0, i - window + 1) // pool if pool else 0)


def _kisilix_kernel_work(cfg: dict, rows: int, batch: int, context: int) -> dict:
    """What a step's launches of the design's own kernels have to move (bytes) or compute (flops), by entry point.
    `rows` rows in all, of `batch` sequences that end at `context`."""
    W = cfg["width"]
    by = {"leb_postnorm_residual": 0, "leb_gated_act": 0, "leb_causal_conv": 0, "leb_delta_prep": 0, "leb_ssm_prep": 0,
          "leb_gated_recurrence": 0, "leb_group_norm_gate": 0, "leb_pooled_attn_prep": 0, "leb_attention_pooled": 0}
    fl = {"leb_gated_recurrence": 0, "leb_attention_pooled": 0, "leb_attention_pooled_tc": 0}
    per_seq = rows // batch
    for l in cfg["layers"]:
        m = l["mixer"]
        n_sub = 2 if l["mlp"] else 1
        by["leb_postnorm_residual"] += n_sub * rows * W * (4 + 4 + 4 + 2)            # x and y read (float), x and its bfloat16 copy written
        if l["mlp"]:
            by["leb_gated_act"] += rows * l["mlp"]["ff"] * (8 + 2)
        if l["type"] == "attention":
            nh, nkv, hd, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            by["leb_pooled_attn_prep"] += rows * ((nh + nkv) * hd + nkv * vd) * (4 + 2)
            win, pool = m["mask"]["size"], m["mask"]["pool"]
            seen = sum(_seen_keys(i, win, pool) for i in range(context - per_seq, context))
            fl["leb_attention_pooled"] += 2 * nh * (hd + vd) * seen * batch
            by["leb_attention_pooled"] += batch * _seen_keys(context - 1, win, pool) * nkv * (hd + vd) * 2 + rows * nh * (hd + vd) * 2
            fl["leb_attention_pooled_tc"] = fl["leb_attention_pooled"]      # prompts at the tensor-core kernel's sizes
        else:
            delta = l["type"] == "channel_delta"
            H, e = m["heads"], m["vdim"]
            d = m["dim"] if delta else m["state"]
            kq = 2 * (m["kv_heads"] if delta else m["groups"]) * d
            C = kq + H * e
            by["leb_causal_conv"] += rows * C * 8 + batch * C * (m["conv"] - 1) * 8
            if delta:
                by["leb_delta_prep"] += rows * (2 * C + 2 * H * d + 2 * H) * 4
            else:
                by["leb_ssm_prep"] += rows * (2 * C + 3 * H) * 4
            by["leb_gated_recurrence"] += rows * (kq + 2 * H * e + (H * d if delta else H) + H) * 4 + batch * H * d * e * 8
            fl["leb_gated_recurrence"] += rows * H * d * e * (8 if delta else 6)
            by["leb_group_norm_gate"] += rows * H * e * (4 + 4 + 2)
    return {"bytes": by, "flops": fl}


# ---- the Tevilix design beside the Kisilix design at equal layer sizes (--compare tevilix) ----------------
def tevilix_config(width: int, ff: int, heads: int, kv_heads: int, dim: int, vdim: int, ret_heads: int, ret_dim: int,
                   ret_vdim: int, layers: int, vocab: int, window: int, pool: int = 0) -> dict:
    """Side-by-side layers (windowed attention with mixed heads beside the minimal recurrent unit, as wide as the
    model) alternate with the matrix memory with exponential gates; every layer has the dense feed-forward.  The
    attention takes the other design's head sizes and window, the matrix memory its recurrent layers' sizes."""
    att = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": dim ** -0.5,
           "rot": {"dims": dim, "base": 1000000.0, "scaling": {"factor": 4.0}}, "mask": {"size": window}}
    par = {"left": att, "left_scale": 0.75, "right": {"width": width}, "right_scale": 1.25}
    mem = {"heads": ret_heads, "dim": ret_dim, "vdim": ret_vdim, "gate_cap": 10.0}
    ls = [{"type": "mlstm" if i % 2 else "parallel", "mixer": mem if i % 2 else par, "mlp": {"kind": "dense", "ff": ff}}
          for i in range(layers)]
    return {"architecture": "Tevilix", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0},
            "layers": ls}


def _tevilix_kernel_work(cfg: dict, rows: int, batch: int, context: int) -> dict:
    """What a step's launches of the design's own kernels have to move (bytes) or compute (flops), by entry point."""
    W = cfg["width"]
    by = {"leb_layernorm_pair": 0, "leb_activation": 0, "leb_weighted_pair_sum": 0, "leb_pooled_attn_prep": 0,
          "leb_attention_mixed": 0, "leb_min_gru": 0, "leb_exp_gates": 0, "leb_gated_recurrence": 0, "leb_exp_gates_finish": 0}
    fl = {"leb_attention_mixed": 0, "leb_gated_recurrence": 0}
    per_seq = rows // batch
    for l in cfg["layers"]:
        m = l["mixer"]
        by["leb_layernorm_pair"] += rows * W * (4 + 4 + 4 + 2 + 2)                    # x and y read, x written, two norms written
        if l["mlp"]:
            by["leb_activation"] += rows * l["mlp"]["ff"] * (4 + 2)
        if l["type"] == "parallel":
            a = m["left"]
            nh, nkv, hd, vd, win = a["heads"], a["kv_heads"], a["dim"], a["vdim"], a["mask"]["size"]
            by["leb_weighted_pair_sum"] += rows * W * 12
            by["leb_pooled_attn_prep"] += rows * ((nh + nkv) * hd + nkv * vd) * (4 + 2)
            seen = sum(min(i + 1, win) for i in range(context - per_seq, context))
            fl["leb_attention_mixed"] += 2 * nh * (hd + vd + nh) * seen * batch
            by["leb_attention_mixed"] += batch * min(context, win) * nkv * (hd + vd) * 2 + rows * nh * (hd + 3 * vd) * 2
            by["leb_min_gru"] += rows * m["right"]["width"] * (12 + 2) + batch * m["right"]["width"] * 8
        else:
            H, d, e = m["heads"], m["dim"], m["vdim"]
            by["leb_exp_gates"] += rows * H * 5 * 4
            by["leb_gated_recurrence"] += rows * (2 * H * d + 2 * H * e + 2 * H) * 4 + batch * H * d * (e + 1) * 8
            fl["leb_gated_recurrence"] += rows * H * d * (e + 1) * 6
            by["leb_exp_gates_finish"] += rows * H * e * (4 + 4 + 2)
    return {"bytes": by, "flops": fl}


def compare_designs(which: str, steps: int, warmup: int) -> int:
    import numpy as np
    import torch
    from lastengine_b200 import Engine
    from lastengine_b200.ops import kernels
    pk, pk_src = peaks()
    rng = np.random.default_rng(0)
    results = {}
    other = "zekivik" if which == "kisilix" else ("kisilix" if which == "tevilix" else "lfm3")
    for size_name, sz in {"zekivik": COMPARE_SIZES, "lenesun": LENESUN_SIZES, "kisilix": KISILIX_SIZES,
                          "tevilix": KISILIX_SIZES}[which].items():
        if which == "tevilix":
            zc = tevilix_config(vocab=32768, **sz)
            lc = kisilix_config(vocab=32768, **sz)
        elif which == "kisilix":
            zc = kisilix_config(vocab=32768, **sz)
            lc = zekivik_config(vocab=32768, loop=False, **{k: v for k, v in sz.items() if k not in ("window", "pool")})
        elif which == "zekivik":
            zc = zekivik_config(vocab=32768, **sz)
            runs = sz["layers"] + 2
            lc = lfm3_like(sz["width"], sz["ff"], sz["heads"], sz["kv_heads"], sz["dim"], runs, 32768)
        else:
            zc = lenesun_config(vocab=32768, **sz)
            lc = lfm3_moe_like(sz["width"], sz["heads"], sz["dim"], sz["experts"], sz["top"], sz["ff"], sz["layers"], 32768)
        row = {}
        for label, cfg in ((which, zc), (other, lc)):
            eng = Engine.from_config(cfg, seed=0, dtype="bfloat16", max_tokens=8 * 2304 + 4096, max_seqs=16)
            nums = model_numbers(eng)
            r = {"weights_gb": round(nums["weight_bytes"] / 1e9, 3)}
            print(f"[bench] {size_name} {label}: {r['weights_gb']} GB of weights", file=sys.stderr, flush=True)
            pre_ms = time_prefill(eng, PREFILL_TOKENS, 3, 5, rng)
            print(f"[bench] {size_name} {label}: prompt of {PREFILL_TOKENS} tokens {pre_ms:.3f} ms", file=sys.stderr, flush=True)
            if label == "tevilix":      # a position sees its window
                attn_flops = _tevilix_kernel_work(cfg, PREFILL_TOKENS, 1, PREFILL_TOKENS)["flops"]["leb_attention_mixed"]
                kv_seen = [sum(min(2048, l["mixer"]["left"]["mask"]["size"]) * l["mixer"]["left"]["kv_heads"]
                               * (l["mixer"]["left"]["dim"] + l["mixer"]["left"]["vdim"]) * 2
                               for l in cfg["layers"] if l["type"] == "parallel")]
            elif label == "kisilix":      # a position sees its window and the pooled blocks behind it, not every earlier one
                attn_flops = _kisilix_kernel_work(cfg, PREFILL_TOKENS, 1, PREFILL_TOKENS)["flops"]["leb_attention_pooled"]
                kv_seen = [sum(_seen_keys(2047, l["mixer"]["mask"]["size"], l["mixer"]["mask"]["pool"]) * l["mixer"]["kv_heads"]
                               * (l["mixer"]["dim"] + l["mixer"]["vdim"]) * 2 for l in cfg["layers"] if l["type"] == "attention")]
            else:
                attn_flops = nums["attn_flops_per_qk"] * PREFILL_TOKENS * (PREFILL_TOKENS + 1) // 2
                kv_seen = None
            flops = PREFILL_TOKENS * nums["linear_flops_per_token"] + nums["head_flops_per_row"] + attn_flops
            r["prefill_2048_ms"] = pre_ms
            r["prefill_tok_s"] = PREFILL_TOKENS / (pre_ms / 1e3)
            r["prefill_frac_of_bf16_peak"] = flops / (pre_ms / 1e3) / (pk["bf16_tflops"] * 1e12)
            for b in (1, 8):
                d = time_decode(eng, b, 2048, steps, warmup, rng)
                r[f"decode_b{b}_ms"] = d["ms_per_step"]
                r[f"decode_b{b}_tok_s"] = d["tok_s"]
                r[f"decode_b{b}_launches"] = d["launches_per_step"]
                step_bytes = decode_step_bytes(eng, nums, b, d["avg_context"]) if kv_seen is None else \
                    eng.weight_bytes_read(b) + b * kv_seen[0] + 2 * b * nums["state_bytes_per_seq"]
                r[f"decode_b{b}_frac_of_hbm"] = step_bytes / (d["ms_per_step"] / 1e3) / 1e9 / pk["hbm_gbs"]
                print(f"[bench] {size_name} {label}: decode b{b} {d['ms_per_step']:.4f} ms/step", file=sys.stderr, flush=True)
            # every entry point of a prompt and of a decode step, one after the other under the event timer
            toks = rng.integers(0, eng.vocab_size, size=PREFILL_TOKENS).tolist()
            s = eng.new_sequence()
            eng.step([s], [toks], "last")
            eng.release(s)
            s = eng.new_sequence()
            torch.cuda.synchronize()
            with kernels.KernelTimer(head_start_ms=5.0) as t:
                eng.step([s], [toks], "last")
            eng.release(s)
            pre_k = t.summary()
            seqs = fill_context(eng, 8, 2046, rng)
            eng.step(seqs, [[1]] * 8, "last")
            torch.cuda.synchronize()
            with kernels.KernelTimer(head_start_ms=5.0) as t:
                eng.step(seqs, [[2]] * 8, "last")
            eng.release(seqs)
            dec_k = t.summary()
            by, fl = {}, {}
            if label == "tevilix":
                wp, wd = _tevilix_kernel_work(cfg, PREFILL_TOKENS, 1, PREFILL_TOKENS), _tevilix_kernel_work(cfg, 8, 8, 2048)
                by = {"prefill": wp["bytes"], "decode_b8": wd["bytes"]}
                fl = {"prefill": dict(wp["flops"], leb_attention_mixed_mma=wp["flops"]["leb_attention_mixed"])}
            elif label == "kisilix":
                wp, wd = _kisilix_kernel_work(cfg, PREFILL_TOKENS, 1, PREFILL_TOKENS), _kisilix_kernel_work(cfg, 8, 8, 2048)
                by = {"prefill": wp["bytes"], "decode_b8": wd["bytes"]}
                fl = {"prefill": wp["flops"]}
            elif label == "zekivik":
                by = {"prefill": _new_kernel_bytes(cfg, PREFILL_TOKENS, 1), "decode_b8": _new_kernel_bytes(cfg, 8, 8)}
                if which == "kisilix":     # the like kernels of the other side: retention's flops, attention's flops and cache bytes
                    ret = sum(6 * l["mixer"]["heads"] * l["mixer"]["dim"] * l["mixer"]["vdim"] for l in cfg["layers"] if l["type"] == "retention")
                    att = nums["attn_flops_per_qk"] * PREFILL_TOKENS * (PREFILL_TOKENS + 1) // 2
                    fl = {"prefill": {"leb_retention": ret * PREFILL_TOKENS, "leb_attention_prefill_tc": att,
                                      "leb_attention_prefill": att, "leb_attention_general": att}}
                    for name in ("leb_attention_decode", "leb_attention_decode_prep", "leb_attention_general"):
                        by["decode_b8"][name] = 8 * 2048 * nums["kv_bytes_per_token"]
            elif label == "lenesun":
                wp, wd = _lenesun_kernel_work(zc, PREFILL_TOKENS, 1, PREFILL_TOKENS), _lenesun_kernel_work(zc, 8, 8, 2048)
                by = {"prefill": {k: v for k, v in wp["bytes"].items() if k != "leb_latent_attention"}, "decode_b8": wd["bytes"]}
                fl = {"prefill": {"leb_latent_attention": wp["attention_flops"]}}
            else:     # the other design's attention, for the comparison: flops of a prompt, cache bytes of a decode step
                att = nums["attn_flops_per_qk"] * PREFILL_TOKENS * (PREFILL_TOKENS + 1) // 2
                fl = {"prefill": {"leb_attention_prefill_tc": att, "leb_attention_prefill": att}}
                by = {"decode_b8": {"leb_attention_decode": 8 * 2048 * nums["kv_bytes_per_token"],
                                    "leb_attention_decode_prep": 8 * 2048 * nums["kv_bytes_per_token"]}}
            for where, summ in (("prefill", pre_k), ("decode_b8", dec_k)):
                ks = {}
                for name, (calls, ms) in summ.items():
                    e = {"launches": calls, "ms": round(ms, 4)}
                    nb = by.get(where, {}).get(name)
                    if nb and ms > 0:
                        e["gb_s"] = round(nb / (ms / 1e3) / 1e9, 1)
                        e["frac_of_hbm"] = round(nb / (ms / 1e3) / 1e9 / pk["hbm_gbs"], 3)
                    nf = fl.get(where, {}).get(name)
                    if nf and ms > 0:
                        e["tflops"] = round(nf / (ms / 1e3) / 1e12, 1)
                        e["frac_of_bf16_peak"] = round(nf / (ms / 1e3) / 1e12 / pk["bf16_tflops"], 3)
                    ks[name] = e
                r[f"kernels_{where}"] = ks
            row[label] = r
            del eng
            torch.cuda.empty_cache()
        results[size_name] = {"sizes": sz, **row}
    against = {"zekivik": "lfm3 hybrid at equal layer sizes", "kisilix": "zekivik hybrid at equal layer sizes",
               "tevilix": "kisilix at equal layer sizes",
               "lenesun": "lfm3 with attention and experts in every layer at equal layer sizes"}[which]
    print(json.dumps({"compare": which, "against": against, "dtype": "bf16",
                      "data": "synthetic (random weights, uniform random token ids)", "peaks": pk_src,
                      "prefill_tokens": PREFILL_TOKENS, "decode_context": 2048, "steps": steps, "warmup": warmup,
                      "sizes": results}))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=CONTEXT)
    ap.add_argument("--layers", type=int, default=0, help="run fewer layers than the configuration has (reported)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="1.2b", choices=sorted(MODELS), help="shape to run (default: the 1.2B shape the headline is quoted on)")
    ap.add_argument("--skip-points", action="store_true")
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--no-per-kernel", action="store_true", help="leave out roofline.kernels (the per-kernel event timing)")
    ap.add_argument("--only-prefill", action="store_true", help="time the prompt step only (for profiling)")
    ap.add_argument("--only-decode", action="store_true", help="skip the prompt timing (for profiling)")
    ap.add_argument("--unequal", type=int, default=0, metavar="N",
                    help="instead of the default run: N requests with prompts of U[64, 2048] tokens generate "
                         "--steps tokens each in one batch through the Python entry point (prints its own JSON line)")
    ap.add_argument("--compare", default="", choices=["", "zekivik", "lenesun", "kisilix", "tevilix"],
                    help="instead of the default run: prefill and decode of that design at a few layer sizes beside "
                         "the closest other design at equal sizes, with every kernel's time (prints its own JSON line)")
    args = ap.parse_args()

    if args.compare:
        return compare_designs(args.compare, min(args.steps, 128), max(args.warmup, 3))
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a Rust crate (cargo, NVRTC); no Rust toolchain here, pip cannot install it "
                          "('neither setup.py nor pyproject.toml'), and its GPU path reads only quantized GGUF files"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import numpy as np
    import torch
    from lastengine_b200 import Engine
    from lastengine_b200.ops import kernels

    model_name, base_cfg = MODELS[args.model]
    cfg = dict(base_cfg)
    full_layers = cfg["num_hidden_layers"]
    if args.layers and args.layers < full_layers:
        cfg["num_hidden_layers"] = args.layers
        cfg["layer_types"] = cfg["layer_types"][:args.layers]
    pk, pk_src = peaks()
    rng = np.random.default_rng(0)
    max_b = max(args.batch, 1 if args.skip_points else 64)
    t0 = time.time()
    eng = Engine.from_config(cfg, seed=0, dtype="bfloat16", max_tokens=max_b * (args.context + 64) + 4096,
                             max_seqs=max_b + 8)
    nums = model_numbers(eng)
    from lastengine_b200.config import Lfm3Config
    tc = Lfm3Config.from_dict(cfg)
    print(f"[bench] model ready in {time.time() - t0:.1f}s: {nums['weight_bytes'] / 1e9:.3f} GB of weights", file=sys.stderr)

    if args.unequal > 0:
        # a batch of prompts of unequal lengths through Engine.generate: prompt tokens / time to the first
        # tokens, decoded tokens / the time after (the reference's definitions, src/server/mod.rs:270-286)
        from lastengine_b200 import SamplingParams
        lens = rng.integers(64, 2049, size=args.unequal)
        prompts = [rng.integers(0, eng.vocab_size, size=int(n)).tolist() for n in lens]
        greedy = SamplingParams(temperature=0.0)
        eng.generate([p[:32] for p in prompts], greedy, max_new_tokens=4, stop_token_ids=[], max_batch=args.unequal,
                     max_seq_len=2048 + args.steps + 1)     # captures the graph of this batch size
        res = eng.generate(prompts, greedy, max_new_tokens=args.steps, stop_token_ids=[], max_batch=args.unequal,
                           max_seq_len=2048 + args.steps + 1)
        st = res.stats
        print(json.dumps({"scenario": f"{args.unequal} prompts of U[64, 2048] tokens, {args.steps} tokens each, one batch",
                          "model": model_name, "prompt_tokens": int(lens.sum()), "prefill_tok_s": st.prefill_tok_s,
                          "decode_tok_s": st.decode_tok_s, "decode_steps": st.decode_steps, "batches": st.batches}))
        return 0

    clocks = ClockSampler()
    clocks.start()
    # ---- prefill ---------------------------------------------------------------------------
    pre_ms = time_prefill(eng, PREFILL_TOKENS, 0 if args.only_decode else 3, 1 if args.only_decode else 5, rng)
    pre_flops = (PREFILL_TOKENS * nums["linear_flops_per_token"] + nums["head_flops_per_row"]
                 + nums["attn_flops_per_qk"] * PREFILL_TOKENS * (PREFILL_TOKENS + 1) // 2)
    prefill = {"value": PREFILL_TOKENS / (pre_ms / 1e3), "tokens": PREFILL_TOKENS, "ms": pre_ms,
               "frac": pre_flops / (pre_ms / 1e3) / (pk["bf16_tflops"] * 1e12), "unit": "tokens/s",
               "tflops": pre_flops / (pre_ms / 1e3) / 1e12}
    print(f"[bench] prefill {PREFILL_TOKENS} tokens: {pre_ms:.3f} ms", file=sys.stderr)
    if args.only_prefill:
        clocks.stop()
        print(json.dumps({"prefill": prefill}))
        return 0
    # ---- decode ----------------------------------------------------------------------------
    launches0 = kernels.launch_count()
    main_run = time_decode(eng, args.batch, args.context, args.steps, args.warmup, rng, clocks)
    launches = main_run["launches_per_step"] * args.steps
    step_bytes = decode_step_bytes(eng, nums, args.batch, main_run["avg_context"])
    achieved = step_bytes / (main_run["ms_per_step"] / 1e3) / 1e9
    clk = clocks.summary(*main_run["clock_rows"])
    print(f"[bench] decode b{args.batch}: {main_run['ms_per_step']:.4f} ms/step", file=sys.stderr)
    points = {}
    if not args.skip_points:
        for b in (1, 64):
            r = time_decode(eng, b, args.context, args.steps, args.warmup, rng)
            points[f"decode_b{b}"] = r["tok_s"]
            points[f"decode_b{b}_ms"] = r["ms_per_step"]
            points[f"decode_b{b}_frac"] = decode_step_bytes(eng, nums, b, r["avg_context"]) / (r["ms_per_step"] / 1e3) / 1e9 / pk["hbm_gbs"]
            print(f"[bench] decode b{b}: {r['ms_per_step']:.4f} ms/step", file=sys.stderr)
        # the scenario the reference's numbers are defined on: prompts of 512 tokens, then 256 decode steps
        for b in (1, 8, 64):
            r = time_decode(eng, b, P512_PROMPT + P512_STEPS + args.warmup + 1, P512_STEPS, args.warmup, rng)
            nbytes = decode_step_bytes(eng, nums, b, r["avg_context"])
            points[f"p512_decode_b{b}"] = r["tok_s"]
            points[f"p512_decode_b{b}_ms"] = r["ms_per_step"]
            points[f"p512_decode_b{b}_gb"] = nbytes / 1e9
            points[f"p512_decode_b{b}_frac"] = nbytes / (r["ms_per_step"] / 1e3) / 1e9 / pk["hbm_gbs"]
            print(f"[bench] 512-token prompts, {P512_STEPS} steps, b{b}: {r['ms_per_step']:.4f} ms/step", file=sys.stderr)
    e2e = None
    if not args.skip_e2e:
        e2e = time_e2e(eng, args.batch, args.context, max(args.steps, E2E_MIN_STEPS), rng)
        print(f"[bench] e2e b{args.batch}: {e2e['value']:.1f} tok/s over {e2e['decode_steps']} steps "
              f"({e2e['first_steps_value']:.1f} over the first {E2E_FIRST_STEPS})", file=sys.stderr)
    per_kernel = None
    if not args.no_per_kernel:
        per_kernel = time_kernels(eng, nums, args.batch, args.context, pk, rng)
    clocks.stop()

    line = {
        "metric": f"decode tokens/s, batch {args.batch} ({model_name}, bf16, context {args.context})",
        "value": main_run["tok_s"], "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": main_run["ms_per_step"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (random weights N(0,0.02), uniform random token ids)",
        "config": {"model": model_name, "global_batch": args.batch, "seq_len": args.context,
                   "parallelism": "single GPU", "layers": cfg["num_hidden_layers"], "layers_in_config": full_layers,
                   "attention_layers": sum(t != "conv" for t in cfg["layer_types"]), "hidden_size": tc.hidden_size,
                   "heads": tc.num_attention_heads, "kv_heads": tc.num_key_value_heads, "head_dim": tc.head_dim,
                   "ffn": tc.ffn_dim, "vocab": tc.vocab_size, "conv_L_cache": tc.conv_L_cache,
                   "prefill_tokens": PREFILL_TOKENS, "weights_gb": round(nums["weight_bytes"] / 1e9, 3),
                   "cache_defeat": f"inputs larger than L2 ({step_bytes / 1e9:.1f} GB read per step)",
                   "peaks": pk_src},
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"], "of": pk_src, "bytes_per_step": step_bytes,
                     **({"kernels": per_kernel} if per_kernel else {})},
        "points": points,
        "gpu_launches": launches,
        "clocks": clk,
    }
    if e2e is not None:
        line["e2e"] = e2e
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
