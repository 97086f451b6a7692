"""Ways of cutting the same requests into steps for trace replay.

Every function returns a list of step records in the format of ``bin/trace_run`` and asks for
the logits at every position, so that each can be compared with the plain implementation's
whole-sequence logits.  ``collect`` maps what a replay returned back to (request, position).
"""

from __future__ import annotations

import random


def whole(requests: dict[str, list[int]]) -> list[dict]:
    """Each request alone, in one step."""
    return [
        {"step": i, "entries": [{"id": name, "tokens": toks, "want": list(range(len(toks)))}], "end": [name]}
        for i, (name, toks) in enumerate(requests.items())
    ]


def tail_one_by_one(requests: dict[str, list[int]], tail: int = 32) -> list[dict]:
    """Most of the request in one step, then its last ``tail`` tokens one by one."""
    steps, number = [], 0
    for name, toks in requests.items():
        head = max(len(toks) - tail, 1)
        steps.append({"step": number, "entries": [{"id": name, "tokens": toks[:head], "want": list(range(head))}], "end": []})
        number += 1
        for i in range(head, len(toks)):
            last = i == len(toks) - 1
            steps.append({"step": number, "entries": [{"id": name, "tokens": [toks[i]], "want": [0]}], "end": [name] if last else []})
            number += 1
        if head == len(toks):
            steps[-1]["end"] = [name]
    return steps


def changing_portions(requests: dict[str, list[int]], seed: int = 0) -> list[dict]:
    """Each request alone, in portions of changing size, down to two tokens."""
    rng = random.Random(seed)
    sizes = [2, 7, 3, 16, 2, 5, 33, 2, 17, 8, 64, 3]
    steps, number = [], 0
    for name, toks in requests.items():
        done = 0
        while done < len(toks):
            size = sizes[rng.randrange(len(sizes))]
            if len(toks) - done - size == 1:  # never leave a single token for a "portion"
                size += 1
            chunk = toks[done : done + size]
            done += len(chunk)
            steps.append({
                "step": number,
                "entries": [{"id": name, "tokens": chunk, "want": list(range(len(chunk)))}],
                "end": [name] if done >= len(toks) else [],
            })
            number += 1
    return steps


def mixed(requests: dict[str, list[int]], prompt_fraction: float = 0.6, max_live: int = 4, seed: int = 1) -> list[dict]:
    """Up to ``max_live`` requests at a time: portions of some beside single decoded tokens of
    others; requests sometimes sit a step out; as soon as one ends the next one starts, so
    that its pages are handed out again."""
    rng = random.Random(seed)
    waiting = list(requests.items())
    live: dict[str, dict] = {}
    steps, number = [], 0
    while waiting or live:
        while waiting and len(live) < max_live:
            name, toks = waiting.pop(0)
            live[name] = {"toks": toks, "done": 0, "prompt": max(2, int(len(toks) * prompt_fraction))}
        entries, ended = [], []
        for name, st in list(live.items()):
            if len(live) > 1 and rng.random() < 0.2:
                continue  # left out of this step, goes on later
            left_in_prompt = st["prompt"] - st["done"]
            if left_in_prompt > 0:
                size = min(left_in_prompt, rng.choice([2, 3, 5, 8, 13, 24, 40]))
                if left_in_prompt - size == 1:
                    size += 1
            else:
                size = 1
            chunk = st["toks"][st["done"] : st["done"] + size]
            st["done"] += len(chunk)
            entries.append({"id": name, "tokens": chunk, "want": list(range(len(chunk)))})
            if st["done"] >= len(st["toks"]):
                ended.append(name)
                del live[name]
        if entries:
            steps.append({"step": number, "entries": entries, "end": ended})
            number += 1
    return steps


def collect(steps: list[dict], outputs: dict[int, "object"]) -> dict[str, dict[int, "object"]]:
    """``outputs[step]`` is ``[wanted, vocab]``; returns ``{request: {position: logits row}}``."""
    held: dict[str, int] = {}
    result: dict[str, dict[int, object]] = {}
    for record in steps:
        rows = outputs.get(record["step"])
        cursor = 0
        for item in record["entries"]:
            start = held.get(item["id"], 0)
            for place in item.get("want", []):
                result.setdefault(item["id"], {})[start + place] = rows[cursor]
                cursor += 1
            held[item["id"]] = start + len(item["tokens"])
        for name in record.get("end", []):
            held.pop(name, None)
    return result


def peak_live_tokens(steps: list[dict], round_to: int = 64) -> int:
    """The most tokens that live requests hold at any time, each rounded up to ``round_to``."""
    held: dict[str, int] = {}
    peak = 0
    for record in steps:
        for item in record["entries"]:
            held[item["id"]] = held.get(item["id"], 0) + len(item["tokens"])
        peak = max(peak, sum(-(-n // round_to) * round_to for n in held.values()))
        for name in record.get("end", []):
            held.pop(name, None)
    return peak
