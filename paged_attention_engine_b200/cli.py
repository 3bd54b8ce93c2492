"""Command line of the engine.

    python -m paged_attention_engine_b200 generate --model DIR --prompt-ids 1,2,3 --max-new-tokens 16
    python -m paged_attention_engine_b200 random-model --config config.json --seed 0 --out DIR
    python -m paged_attention_engine_b200 stream --model DIR --stream mixed --seed 0 -C 64 --out run.json

The reference has no command line for generation; its command lines drive measurement runs
(`python -m bench.run --stream {mixed,control} --seed S -C N --model M --out FILE --smoke`,
bench/run.py:846-885; `python -m bench.workload`, bench/workload.py:438-455). `stream` keeps
those option names and meanings for a seeded synthetic request stream run through the
scheduler: `--stream control` is 256 requests of 512 prompt + 512 decoded tokens
(bench/workload.py:256-272), `--stream mixed` a ragged one (prompts 16-2048, decodes 8-1024);
`-C` is the most requests that run at a time (`max_num_seqs`); `--smoke` makes a small
structural run. Engine options carry the names of the reference's constructor arguments
(`num_blocks`, `block_size`, `max_num_seqs`, `max_num_batched_tokens`).
"""

from __future__ import annotations

import argparse
import json
import random
import sys
import time
from pathlib import Path


def _engine_options(parser: argparse.ArgumentParser) -> None:
    source = parser.add_mutually_exclusive_group(required=True)
    source.add_argument("--model", help="folder with config.json and model.safetensors")
    source.add_argument("--random", metavar="CONFIG", help="a config.json: the model gets random weights (see --weights-seed)")
    parser.add_argument("--weights-seed", type=int, default=0, help="seed of the random weights of --random")
    parser.add_argument("--dtype", choices=("bfloat16", "float32"), default="bfloat16")
    parser.add_argument("--num-blocks", type=int, default=None, help="pages of the cache pool (reference: 3584, the default)")
    parser.add_argument("--kv-gb", type=float, default=None,
                        help="size the cache pool by bytes instead: as many pages as this many GB (1e9 bytes) pay for")
    parser.add_argument("--block-size", type=int, default=16, help="tokens per page (reference: 16)")
    parser.add_argument("--max-num-seqs", type=int, default=64)
    parser.add_argument("--max-num-batched-tokens", type=int, default=8192)
    parser.add_argument("--admission-margin-blocks", type=int, default=1)


def _llm(args, max_num_seqs=None):
    from .engine.api import LLM

    options = dict(
        dtype=args.dtype, num_blocks=args.num_blocks, block_size=args.block_size,
        kv_bytes=int(args.kv_gb * 1e9) if args.kv_gb is not None else None,
        max_num_seqs=max_num_seqs or args.max_num_seqs, max_num_batched_tokens=args.max_num_batched_tokens,
        admission_margin_blocks=args.admission_margin_blocks,
    )
    if args.random:
        # the same weights as `random-model --seed` writes for this configuration
        return LLM.from_random(json.loads(Path(args.random).read_text()), seed=args.weights_seed, as_written=True, **options)
    return LLM.from_pretrained(args.model, **options)


def cmd_generate(args) -> int:
    from .engine.scheduler import Request

    prompts: list[list[int]] = []
    for text in args.prompt_ids or []:
        prompts.append([int(t) for t in text.replace(",", " ").split()])
    if args.prompts_file:
        for line in Path(args.prompts_file).read_text().splitlines():
            if line.strip():
                prompts.append([int(t) for t in line.replace(",", " ").split()])
    if not prompts:
        print("generate: give --prompt-ids or --prompts-file (token ids; this engine has no tokenizer)", file=sys.stderr)
        return 2
    llm = _llm(args)
    for i, prompt in enumerate(prompts):
        ok = llm.add_request(Request(f"prompt-{i}", tuple(prompt), args.max_new_tokens, args.temperature, args.seed))
        if not ok:
            print(f"prompt-{i}: rejected, {len(prompt)} + {args.max_new_tokens} tokens cannot fit the pool", file=sys.stderr)
    out = llm.run_to_completion()
    for i in range(len(prompts)):
        rid = f"prompt-{i}"
        if rid in out:
            print(json.dumps({"request_id": rid, "token_ids": list(out[rid])}))
    return 0


def cmd_random_model(args) -> int:
    import torch

    from .weights import write_random_model

    raw = json.loads(Path(args.config).read_text())
    dtype = torch.bfloat16 if args.dtype == "bfloat16" else torch.float32
    folder = write_random_model(args.out, raw, args.seed, dtype)
    print(folder)
    return 0


def synthetic_stream(kind: str, seed: int, count: int, vocab: int, smoke: bool):
    """(prompt length, decode length) pairs and token ids from one seeded generator."""
    rng = random.Random(f"{kind}-{seed}")
    lengths = []
    for _ in range(count):
        if kind == "control":
            lengths.append((512, 512))
        else:
            lengths.append((rng.randint(16, 2048), rng.randint(8, 1024)))
    if smoke:
        lengths = [(max(1, p // 32), max(1, d // 32)) for p, d in lengths[: min(count, 16)]]
    return [([rng.randrange(vocab) for _ in range(p)], d) for p, d in lengths]


def cmd_stream(args) -> int:
    from .engine.scheduler import EventKind, Request

    results = []
    for concurrency in args.concurrency or [64]:
        llm = _llm(args, max_num_seqs=concurrency)
        stream = synthetic_stream(args.stream, int(args.seed), args.requests, llm.engine.vocab_size, args.smoke)
        accepted = 0
        for i, (prompt, decode) in enumerate(stream):
            accepted += bool(llm.add_request(Request(f"req-{i}", tuple(prompt), decode)))
        started = time.perf_counter()
        out = llm.run_to_completion()
        elapsed = time.perf_counter() - started
        generated = sum(len(v) for v in out.values())
        results.append({
            "stream": args.stream, "seed": args.seed, "concurrency": concurrency, "requests": len(stream),
            "accepted": accepted, "generated_tokens": generated, "seconds": round(elapsed, 4),
            "tokens_per_second": round(generated / elapsed, 2) if elapsed > 0 else None,
            "steps": llm.scheduler._step, "preemptions": len(llm.scheduler.events_of(EventKind.PREEMPT)),
            "smoke": bool(args.smoke),
        })
        print(json.dumps(results[-1]))
    if args.out:
        Path(args.out).parent.mkdir(parents=True, exist_ok=True)
        Path(args.out).write_text(json.dumps(results, indent=2) + "\n")
    return 0


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(prog="paged_attention_engine_b200")
    sub = parser.add_subparsers(dest="command", required=True)

    gen = sub.add_parser("generate", help="generate tokens for prompts given as token ids")
    _engine_options(gen)
    gen.add_argument("--prompt-ids", action="append", help="token ids, comma or space separated; repeatable")
    gen.add_argument("--prompts-file", help="one prompt of token ids per line")
    gen.add_argument("--max-new-tokens", type=int, default=16)
    gen.add_argument("--temperature", type=float, default=0.0, help="0 is greedy")
    gen.add_argument("--seed", type=int, default=0)
    gen.set_defaults(run=cmd_generate)

    rnd = sub.add_parser("random-model", help="write config.json and model.safetensors with random weights")
    rnd.add_argument("--config", required=True, help="a config.json of a registered architecture")
    rnd.add_argument("--seed", type=int, default=0)
    rnd.add_argument("--dtype", choices=("bfloat16", "float32"), default="bfloat16")
    rnd.add_argument("--out", required=True)
    rnd.set_defaults(run=cmd_random_model)

    stream = sub.add_parser("stream", help="run a seeded synthetic request stream through the scheduler")
    _engine_options(stream)
    stream.add_argument("--stream", choices=("mixed", "control"), default="control")
    stream.add_argument("--seed", default="0")
    stream.add_argument("-C", "--concurrency", type=int, action="append", default=None, help="sweep level; repeatable")
    stream.add_argument("--requests", type=int, default=256)
    stream.add_argument("--out", default=None)
    stream.add_argument("--smoke", action="store_true", help="a small structural run, no timing claim")
    stream.set_defaults(run=cmd_stream)

    args = parser.parse_args(argv)
    return args.run(args)


if __name__ == "__main__":
    raise SystemExit(main())
