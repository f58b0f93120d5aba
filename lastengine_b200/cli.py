"""Command line, in the reference's manner: `lastengine <command>`.

The reference's commands (src/cli.rs:11-36) that belong to the engine are kept with their names
and meanings; prompts are token ids here (comma or space separated), since tokenizer and chat
template are outside this library:

  gpu PATH PROMPT [TOP]        GPU forward: top-N next-token logprobs, then a 32-token greedy decode
  tf-dump PATH PROMPT [N]      greedy-decode N tokens; JSON {prompt_ids, gen_ids, top} with the five
                               best (id, logprob) per step, for teacher-forced comparison elsewhere
  inspect PATH                 the model folder's configuration and tensors
  probe [--json]               hardware facts as JSON
and, where the reference takes requests over HTTP with sampling fields (src/server/mod.rs:106-110):
  generate --model DIR ...     generation with the same sampling names: --temperature --top-p --top-k
                               --min-p --presence-penalty --repeat-penalty --seed, --ctx as in `serve`
  init --config JSON --seed S --out DIR    write a model folder with random weights
  replay ...                   the trace replay program (same as bin/trace_run)
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys


def parse_ids(text: str) -> list[int]:
    parts = text.replace(",", " ").split()
    if not parts:
        raise SystemExit("lastengine: the prompt is empty (give token ids, e.g. \"1,5,17\")")
    try:
        return [int(p) for p in parts]
    except ValueError:
        raise SystemExit(f"lastengine: prompts are token ids here, got '{text}'") from None


def _engine(path: str, dtype: str, ctx: int, n_seqs: int = 1):
    from . import Engine
    page = 64
    per = -(-(ctx + 1) // page) * page
    return Engine.from_pretrained(path, dtype=dtype, max_tokens=per * n_seqs, max_seqs=max(n_seqs, 1))


def _logprobs(logits):
    import torch
    row = logits.float()
    return row - torch.logsumexp(row, dim=-1, keepdim=True)


def cmd_gpu(a) -> int:
    import torch
    from . import SamplingParams
    ids = parse_ids(a.prompt)
    eng = _engine(a.path, a.dtype, a.ctx)
    s = eng.new_sequence()
    lp = _logprobs(eng.step([s], [ids], "last", check=True))[0]
    eng.release(s)
    top = torch.topk(lp, min(a.top, lp.numel()))
    for i, v in zip(top.indices.tolist(), top.values.tolist()):
        print(f"{i} logprob {v:.4f}")
    res = eng.generate([ids], SamplingParams(temperature=0.0), max_new_tokens=32, stop_token_ids=[],
                       max_seq_len=a.ctx)
    print("greedy:", " ".join(str(t) for t in res.tokens[0]))
    st = res.stats
    print(f"prefill {st.prefill_tok_s:.1f} tok/s, decode {st.decode_tok_s:.1f} tok/s", file=sys.stderr)
    return 0


def cmd_tf_dump(a) -> int:
    import torch
    ids = parse_ids(a.prompt)
    eng = _engine(a.path, a.dtype, a.ctx)
    s = eng.new_sequence()
    logits = eng.step([s], [ids], "last", check=True)
    gen, top = [], []
    for _ in range(a.n):
        lp = _logprobs(logits)[0]
        t5 = torch.topk(lp, min(5, lp.numel()))
        top.append([[int(i), float(v)] for i, v in zip(t5.indices.tolist(), t5.values.tolist())])
        nxt = int(t5.indices[0])
        gen.append(nxt)
        logits = eng.step([s], [[nxt]], "last", check=True)
    eng.release(s)
    print(json.dumps({"prompt_ids": ids, "gen_ids": gen, "top": top}))
    return 0


def cmd_dense_cmp(a) -> int:
    """The reference's dense-cmp (src/main.rs:138-158) compares its CPU forward with its GPU forward
    token by token; here the true 32-bit path stands where the CPU stood and the bfloat16 path is
    the one under test.  Both follow the 32-bit path's greedy tokens."""
    import time
    import torch
    ids = parse_ids(a.prompt)
    exact = _engine(a.path, "float32", a.ctx)
    fast = _engine(a.path, "bfloat16", a.ctx)
    se, sf = exact.new_sequence(), fast.new_sequence()
    le = _logprobs(exact.step([se], [ids], "last", check=True))[0].clone()
    t0 = time.perf_counter()
    lf = _logprobs(fast.step([sf], [ids], "last", check=True))[0].clone()
    torch.cuda.synchronize()
    print(f"bfloat16 prefill {len(ids)} tok in {time.perf_counter() - t0:.3f}s")
    agree, shown, maxd, sumd = 0, 0, 0.0, 0.0
    for k in range(a.n):
        ta, tb = int(torch.argmax(le)), int(torch.argmax(lf))
        d = abs(float(le[ta]) - float(lf[ta]))
        maxd, sumd = max(maxd, d), sumd + d
        if ta == tb:
            agree += 1
        elif shown < 8:
            shown += 1
            print(f"step {k}: float32 {ta} lp {float(le[ta]):.3f} (bfloat16 lp {float(lf[ta]):.3f}) vs bfloat16 {tb} "
                  f"lp {float(lf[tb]):.3f} (float32 lp {float(le[tb]):.3f})")
        le = _logprobs(exact.step([se], [[ta]], "last", check=True))[0].clone()
        lf = _logprobs(fast.step([sf], [[ta]], "last", check=True))[0].clone()
    print(f"{agree}/{a.n} argmax agree, mean |dlogprob| {sumd / max(a.n, 1):.4f}, max {maxd:.4f}")
    return 0


def cmd_inspect(a) -> int:
    from .config.base import architecture_name, read_config_json
    from .registry import plan_from_config
    from .weights.safetensors_io import open_checkpoint
    raw = read_config_json(a.path)
    plan = plan_from_config(raw)
    print(f"architecture {architecture_name(raw)}: {len(plan.layers)} layers, hidden {plan.hidden_size}, "
          f"vocab {plan.vocab_size}")
    for i, l in enumerate(plan.layers):
        print(f"  layer {i}: {l.mixer.kind} + {l.ffn.kind}")
    ck = open_checkpoint(a.path)
    by: dict[tuple[str, str], list[int]] = {}
    total = 0
    for name, (f, k) in ck.items():
        base = ".".join(p for p in name.split(".") if not p.isdigit())
        n = math.prod(f.shape(k))
        e = by.setdefault((str(f.dtype(k)).replace("torch.", ""), base), [0, 0])
        e[0] += 1
        e[1] += n
        total += n
    for (dt, base), (cnt, n) in sorted(by.items()):
        print(f"  {dt:9s} x{cnt:<4d} {base} ({n} elems)")
    print(f"{len(ck)} tensors, {total} parameters")
    return 0


def cmd_probe(a) -> int:
    import torch
    out = {"cuda": torch.cuda.is_available(), "gpus": []}
    if out["cuda"]:
        for i in range(torch.cuda.device_count()):
            p = torch.cuda.get_device_properties(i)
            free, tot = torch.cuda.mem_get_info(i)
            out["gpus"].append({"index": i, "name": p.name, "compute_capability": f"{p.major}.{p.minor}",
                                "sm_count": p.multi_processor_count, "memory_total_mib": tot // (1 << 20),
                                "memory_free_mib": free // (1 << 20)})
    print(json.dumps(out))
    return 0


def cmd_generate(a) -> int:
    from . import Engine, SamplingParams
    prompts = [parse_ids(p) for p in a.prompt_ids]
    need = sum(-(-(len(p) + a.max_new_tokens) // 64) * 64 for p in prompts)
    kw = dict(dtype=a.dtype, max_tokens=max(need, 64), max_seqs=len(prompts))
    if a.model:
        eng = Engine.from_pretrained(a.model, **kw)
    elif a.config:
        eng = Engine.from_config(a.config, seed=a.random_seed, **kw)
    else:
        raise SystemExit("lastengine generate: give --model DIR, or --config JSON with --random-seed")
    sp = SamplingParams(temperature=a.temperature, top_p=a.top_p, top_k=a.top_k, min_p=a.min_p,
                        presence_penalty=a.presence_penalty, repeat_penalty=a.repeat_penalty, seed=a.seed)
    res = eng.generate(prompts, sp, max_new_tokens=a.max_new_tokens,
                       stop_token_ids=a.stop_token_id if a.stop_token_id is not None else None,
                       max_seq_len=a.ctx)
    for toks, reason in zip(res.tokens, res.finish_reasons):
        print(json.dumps({"tokens": toks, "finish_reason": reason}))
    st = res.stats
    print(f"prefill {st.prefill_tokens} tok {st.prefill_tok_s:.1f} tok/s; decode {st.decode_tokens} tok "
          f"{st.decode_tok_s:.1f} tok/s", file=sys.stderr)
    return 0


def cmd_init(a) -> int:
    from .config.base import read_config_json
    from .weights import write_model_dir
    cfg = read_config_json(a.config)
    write_model_dir(cfg, a.out, seed=a.seed, dtype=a.dtype, norm_init=a.norm_init)
    print(f"wrote {os.path.join(a.out, 'config.json')} and model.safetensors (seed {a.seed}, {a.dtype})")
    return 0


def cmd_replay(a) -> int:
    exe = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bin", "trace_run")
    os.execv(sys.executable, [sys.executable, exe, "--model", a.model, "--dtype", a.dtype, "--out", a.out,
                              "--max-tokens", str(a.max_tokens)])
    return 0


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="lastengine", description="LFM3 hybrid engine for B200 (token ids in, token ids out)")
    sub = ap.add_subparsers(dest="cmd", required=True)

    def common(p, dtype_default="bfloat16"):
        p.add_argument("--dtype", default=dtype_default, choices=["bfloat16", "float32"])
        p.add_argument("--ctx", type=int, default=4096, help="context length (tokens per sequence)")

    p = sub.add_parser("gpu", help="top-N next-token logprobs + a 32-token greedy decode")
    p.add_argument("path")
    p.add_argument("prompt")
    p.add_argument("top", nargs="?", type=int, default=5)
    common(p)
    p.set_defaults(fn=cmd_gpu)

    p = sub.add_parser("tf-dump", help="greedy-decode N tokens, print JSON {prompt_ids, gen_ids, top}")
    p.add_argument("path")
    p.add_argument("prompt")
    p.add_argument("n", nargs="?", type=int, default=100)
    common(p)
    p.set_defaults(fn=cmd_tf_dump)

    p = sub.add_parser("dense-cmp", help="bfloat16 path against the true 32-bit path, greedy step by step")
    p.add_argument("path")
    p.add_argument("prompt")
    p.add_argument("n", nargs="?", type=int, default=32)
    p.add_argument("--ctx", type=int, default=4096)
    p.set_defaults(fn=cmd_dense_cmp)

    p = sub.add_parser("inspect", help="print the model folder's configuration and tensors")
    p.add_argument("path")
    p.set_defaults(fn=cmd_inspect)

    p = sub.add_parser("probe", help="print hardware facts as JSON")
    p.add_argument("--json", action="store_true", help="accepted for launchers; output is always JSON")
    p.set_defaults(fn=cmd_probe)

    p = sub.add_parser("generate", help="generate from prompts of token ids")
    p.add_argument("--model", help="folder with config.json and model.safetensors")
    p.add_argument("--config", help="a config.json to build random weights from (with --random-seed)")
    p.add_argument("--random-seed", type=int, default=0)
    p.add_argument("--prompt-ids", action="append", required=True, help="token ids; repeat for a batch")
    p.add_argument("--max-new-tokens", type=int, default=32)
    p.add_argument("--temperature", type=float, default=0.7)
    p.add_argument("--top-p", type=float, default=0.95)
    p.add_argument("--top-k", type=int, default=40)
    p.add_argument("--min-p", type=float, default=0.0)
    p.add_argument("--presence-penalty", type=float, default=0.0)
    p.add_argument("--repeat-penalty", type=float, default=1.0)
    p.add_argument("--seed", type=int, default=None)
    p.add_argument("--stop-token-id", type=int, action="append", default=None,
                   help="ends a request (not emitted); default: the model's eos_token_id")
    common(p)
    p.set_defaults(fn=cmd_generate)

    p = sub.add_parser("init", help="write a model folder with random weights")
    p.add_argument("--config", required=True)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--out", required=True)
    p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    p.add_argument("--norm-init", default="ones", choices=["ones", "random"])
    p.set_defaults(fn=cmd_init)

    p = sub.add_parser("replay", help="feed given token ids step by step and write logits (bin/trace_run)")
    p.add_argument("--model", required=True)
    p.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    p.add_argument("--out", required=True)
    p.add_argument("--max-tokens", type=int, required=True)
    p.set_defaults(fn=cmd_replay)
    return ap


def main(argv=None) -> int:
    a = build_parser().parse_args(argv)
    from .config.base import ConfigError
    from .registry import RegistryError
    from .weights.safetensors_io import WeightsError
    try:
        return a.fn(a)
    except (ConfigError, RegistryError, WeightsError) as e:
        print(f"lastengine: {e}", file=sys.stderr)
        return 1


if __name__ == "__main__":
    sys.exit(main())
