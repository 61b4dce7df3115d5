"""The command line, a dispatcher in LockStep's manner: ``lockstep <command> [args]``
(LockStep: lockstep:32-95, docs/kickoff/04-cli-and-report-spec.md:24-33).

  run           run a workload of requests under a named policy and print the tokens
  replay        feed given tokens step by step and write logits (bin/trace_run)
  bench         the throughput line of bench.py
  random-model  write a model folder (config.json, model.safetensors) from a
                configuration and a seed

Request and scheduler options carry LockStep's names and meanings: ``--seed``,
``--max-new-tokens``, ``--temperature``, ``--top-p`` (engine/sched/scheduler.py:19-28),
``--num-blocks``, ``--block-size``, ``--enable-prefix-cache``, ``--eos-token-ids``
(engine/sched/scheduler.py:51-60), policies ``default`` and ``fixed-chunk:N``
(engine/sched/policy.py).  Token ids go in and come out; the engine never tokenizes.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

COMMANDS = {
    "run": "run a workload under a named policy",
    "replay": "re-execute given tokens step by step and write logits",
    "bench": "produce the throughput line",
    "random-model": "write a random-weights model folder",
}


def _policy(name: str, max_running: int):
    from .engine import DefaultPolicy, FixedChunkPolicy

    if name == "default":
        return DefaultPolicy(max_running=max_running)
    if name.startswith("fixed-chunk:"):
        return FixedChunkPolicy(int(name.split(":", 1)[1]), max_running=max_running)
    raise SystemExit(f"unknown policy {name!r}; use default or fixed-chunk:N")


def cmd_run(argv) -> int:
    p = argparse.ArgumentParser(prog="lockstep run", description=COMMANDS["run"])
    p.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    p.add_argument("--workload", help="JSON file: a list of requests {uid, prompt, seed, max_new_tokens, "
                                      "temperature, top_p}")
    p.add_argument("--prompt-ids", action="append", default=[],
                   help="comma-separated token ids of one prompt (may be repeated)")
    p.add_argument("--prompt-len", type=int, action="append", default=[],
                   help="a seeded random prompt of this many tokens (may be repeated)")
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--max-new-tokens", type=int, default=8)
    p.add_argument("--temperature", type=float, default=0.0)
    p.add_argument("--top-p", type=float, default=1.0)
    p.add_argument("--policy", default="default")
    p.add_argument("--num-blocks", type=int, default=4096, help="pages in the cache pool")
    p.add_argument("--block-size", type=int, default=16, help="tokens per page")
    p.add_argument("--max-running", type=int, default=32)
    p.add_argument("--max-step-tokens", type=int, default=2048, help="token budget of a step")
    p.add_argument("--max-len", type=int, default=None, help="longest sequence (default: the model's)")
    p.add_argument("--enable-prefix-cache", action="store_true")
    p.add_argument("--eos-token-ids", default="", help="comma-separated ids that end a request")
    p.add_argument("--device", default="cuda:0")
    a = p.parse_args(argv)

    import random

    from .engine import Engine, Request

    eos = {int(t) for t in a.eos_token_ids.split(",") if t.strip()}
    engine = Engine(a.model, dtype=a.dtype, device=a.device, num_pages=a.num_blocks,
                    page_size=a.block_size, max_running=a.max_running,
                    max_step_tokens=a.max_step_tokens, max_seq_len=a.max_len,
                    enable_prefix_cache=a.enable_prefix_cache, eos_token_ids=eos,
                    policy=_policy(a.policy, a.max_running))
    requests = []
    if a.workload:
        for i, r in enumerate(json.loads(Path(a.workload).read_text())):
            requests.append(Request(uid=str(r.get("uid", f"r{i:02d}")), prompt=[int(t) for t in r["prompt"]],
                                    seed=int(r.get("seed", a.seed)),
                                    max_new_tokens=int(r.get("max_new_tokens", a.max_new_tokens)),
                                    temperature=float(r.get("temperature", a.temperature)),
                                    top_p=float(r.get("top_p", a.top_p))))
    for ids in a.prompt_ids:
        requests.append(Request(uid=f"r{len(requests):02d}", prompt=[int(t) for t in ids.split(",")],
                                seed=a.seed, max_new_tokens=a.max_new_tokens,
                                temperature=a.temperature, top_p=a.top_p))
    vocab = engine.runner.spec.vocab_size
    for n in a.prompt_len:
        rng = random.Random(a.seed * 1000003 + len(requests))
        requests.append(Request(uid=f"r{len(requests):02d}", prompt=[rng.randrange(vocab) for _ in range(n)],
                                seed=a.seed, max_new_tokens=a.max_new_tokens,
                                temperature=a.temperature, top_p=a.top_p))
    if not requests:
        raise SystemExit("no requests: give --workload, --prompt-ids or --prompt-len")
    out = engine.generate(requests)
    for r in requests:
        print(json.dumps({"uid": r.uid, "prompt_tokens": len(r.prompt), "generated": out[r.uid]}))
    s = engine.scheduler.stats
    print(f"{len(requests)} requests, {s['steps']} steps, {s['tokens_run']} tokens run, "
          f"{s['preemptions']} preemptions, {s['evictions']} evictions", file=sys.stderr)
    return 0


def cmd_random_model(argv) -> int:
    p = argparse.ArgumentParser(prog="lockstep random-model", description=COMMANDS["random-model"])
    p.add_argument("--config", required=True, help="a config.json to take the sizes from")
    p.add_argument("--out", required=True)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    p.add_argument("--init-std", type=float, default=0.02)
    p.add_argument("--gain-std", type=float, default=0.02)
    a = p.parse_args(argv)
    from .weights import write_random_model

    folder = write_random_model(a.out, json.loads(Path(a.config).read_text()), seed=a.seed, dtype=a.dtype,
                                init_std=a.init_std, gain_std=a.gain_std)
    print(folder)
    return 0


def usage() -> int:
    print("lockstep <command> [args]\n")
    width = max(len(c) for c in COMMANDS)
    for name, what in COMMANDS.items():
        print(f"  {name:<{width}}  {what}")
    return 0


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv or argv[0] in ("-h", "--help", "help"):
        return usage()
    command, rest = argv[0], argv[1:]
    if command == "run":
        return cmd_run(rest)
    if command == "replay":
        from .engine.replay import main as replay_main

        return replay_main(rest)
    if command == "random-model":
        return cmd_random_model(rest)
    if command == "bench":
        import runpy

        sys.argv = ["bench.py", *rest]
        try:
            runpy.run_path(str(Path(__file__).resolve().parent.parent / "bench.py"), run_name="__main__")
        except SystemExit as e:
            return int(e.code or 0)
        return 0
    print(f"unknown command {command!r}. Try --help.")
    return 2


if __name__ == "__main__":
    raise SystemExit(main())
