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
                    help="instead of the contract's run: N requests with prompts of U[64, 2048] tokens generate "
                         "--steps tokens each in one batch through the Python entry point (prints its own JSON line)")
    args = ap.parse_args()

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
