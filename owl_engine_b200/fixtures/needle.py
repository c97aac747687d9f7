"""Needle-in-a-haystack and context-ladder evaluation against a live server.

``needle``: a fact (``The pass phrase for <key> is <value>.``) is planted at a relative depth inside filler
text of a target length; the model is asked for the value; a grid of (context length x depth) gives the
retrieval map. ``ladder``: time to first token and decode rate at a ladder of context lengths, each prompt
made of fresh random words (no prefix reuse between rungs). Both use only the HTTP client.

``python -m owl_engine_b200.fixtures.needle --url http://127.0.0.1:8135 needle --lengths 2000 8000 --depths 0.1 0.5 0.9``
``python -m owl_engine_b200.fixtures.needle --url ... ladder --lengths 1000 4000 16000``

Reference counterpart: ``tools/fixture`` (needle eval, quality eval, ctx ladder).
"""
from __future__ import annotations

import argparse
import json
import random

from ..cli.client import Client
from ..cli.workload import WORDS


def filler(n_words: int, rng: random.Random) -> list[str]:
    return [rng.choice(WORDS) for _ in range(n_words)]


def needle_prompt(n_words: int, depth: float, rng: random.Random) -> tuple[str, str]:
    key, value = f"{rng.choice(WORDS)}-{rng.randrange(100, 999)}", f"{rng.choice(WORDS)}-{rng.randrange(1000, 9999)}"
    words = filler(n_words, rng)
    words.insert(int(len(words) * depth), f"The pass phrase for {key} is {value}.")
    return " ".join(words) + f"\n\nWhat is the pass phrase for {key}? Answer with the phrase only.", value


def run_needle(client: Client, lengths: list[int], depths: list[float], trials: int = 1, seed: int = 0) -> list[dict]:
    rng, rows = random.Random(seed), []
    for n in lengths:
        for d in depths:
            hits = 0
            for _ in range(trials):
                prompt, value = needle_prompt(n, d, rng)
                r = client.chat([{"role": "user", "content": prompt}], max_tokens=24, temperature=0)
                hits += int(r.error is None and value in r.content)
            rows.append({"words": n, "depth": d, "hit_rate": hits / trials})
    return rows


def run_ladder(client: Client, lengths: list[int], new_tokens: int = 64, seed: int = 0) -> list[dict]:
    rng, rows = random.Random(seed), []
    for n in lengths:
        prompt = " ".join(filler(n, rng)) + "\nContinue."
        r = client.chat([{"role": "user", "content": prompt}], max_tokens=new_tokens, ignore_eos=True, temperature=0)
        done = r.usage.get("completion_tokens", 0)
        dec = (done - 1) / max(1e-9, (r.total_ms - r.ttft_ms) / 1e3) if done > 1 else 0.0
        rows.append({"words": n, "prompt_tokens": r.usage.get("prompt_tokens"), "ttft_ms": round(r.ttft_ms, 1),
                     "decode_tok_s": round(dec, 1), "p50_gap_ms": round(sorted(r.gaps_ms)[len(r.gaps_ms) // 2], 2) if r.gaps_ms else None,
                     "error": r.error})
    return rows


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="owl-b200-eval")
    ap.add_argument("--url", default="http://127.0.0.1:8135")
    sub = ap.add_subparsers(dest="cmd", required=True)
    n = sub.add_parser("needle")
    n.add_argument("--lengths", type=int, nargs="+", default=[1000, 4000])
    n.add_argument("--depths", type=float, nargs="+", default=[0.1, 0.5, 0.9])
    n.add_argument("--trials", type=int, default=1)
    l = sub.add_parser("ladder")
    l.add_argument("--lengths", type=int, nargs="+", default=[500, 2000, 8000])
    l.add_argument("--new-tokens", type=int, default=64)
    a = ap.parse_args(argv)
    c = Client(a.url)
    rows = run_needle(c, a.lengths, a.depths, a.trials) if a.cmd == "needle" else run_ladder(c, a.lengths, a.new_tokens)
    for r in rows:
        print(json.dumps(r))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
