"""Ways of cutting the same requests into steps.  A trace is a list of steps
``{"step": i, "entries": [{"id", "tokens", "want"}], "end": [ids]}``, the format bin/trace_run reads."""
import random


def whole(requests):
    """Each request alone and whole, every position wanted."""
    steps = []
    for rid, toks in requests.items():
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": list(toks), "want": list(range(len(toks)))}],
                      "end": [rid]})
    return steps


def tail_decode(requests, tail=32):
    """Most of a request in one step, its last ``tail`` tokens one by one."""
    steps = []
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": list(toks[:head]), "want": list(range(head))}],
                      "end": []})
        for i in range(head, len(toks)):
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": [toks[i]], "want": [0]}], "end": []})
        steps[-1]["end"] = [rid]
    return steps


def chunks(requests, sizes=(5, 2, 11, 3, 2, 7, 16, 1, 4, 2, 9, 13)):
    """Portions of changing size, down to two tokens (and a single one now and then)."""
    steps = []
    k = 0
    for rid, toks in requests.items():
        i = 0
        while i < len(toks):
            c = min(sizes[k % len(sizes)], len(toks) - i)
            k += 1
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": list(toks[i:i + c]), "want": list(range(c))}],
                          "end": []})
            i += c
        steps[-1]["end"] = [rid]
    return steps


def mixed(requests, seed=0, max_live=4, decode_tail=8):
    """Up to ``max_live`` requests at a time: portions of some beside single tokens of others; a request may
    sit a step out.  Requests start as others end, so a small pool hands the same pages out again."""
    rng = random.Random(seed)
    pending = list(requests.items())
    live = {}          # rid -> progress
    steps = []
    while pending or live:
        while pending and len(live) < max_live:
            rid, toks = pending.pop(0)
            live[rid] = 0
        entries, ended = [], []
        for rid in list(live):
            toks = requests[rid]
            done = live[rid]
            if len(live) > 1 and rng.random() < 0.2:
                continue                                   # sits this step out
            left = len(toks) - done
            if left <= decode_tail:
                c = 1
            else:
                c = min(rng.choice([2, 2, 3, 5, 8, 13, 17]), left - decode_tail)
            entries.append({"id": rid, "tokens": list(toks[done:done + c]), "want": list(range(c))})
            live[rid] = done + c
            if live[rid] == len(toks):
                ended.append(rid)
        if not entries:
            continue
        rng.shuffle(entries)
        steps.append({"step": len(steps), "entries": entries, "end": ended})
        for rid in ended:
            del live[rid]
    return steps


def decode_heavy(requests, seed=0, max_live=12, tail=(8, 24), sit_out=0.1, portion=64):
    """Many decoding requests at a time, as a scheduler runs them: every step feeds one token of each decoding
    request (a request sits a step out now and then) and, while someone is still in his prompt, one portion of that
    prompt beside them.  Once all are admitted the steps are decode-only with up to ``max_live`` rows, and as requests
    end without successors the number of rows falls through every batch size down to one.  Logits are wanted at the
    last prompt token and at every decoded token.  ``tail``: how many of its last tokens a request decodes."""
    rng = random.Random(seed)
    pending = list(requests.items())
    live, tails = {}, {}
    steps = []
    while pending or live:
        while pending and len(live) < max_live:
            rid, toks = pending.pop(0)
            live[rid] = 0
            tails[rid] = min(len(toks) - 1, rng.randint(*tail))
        entries, ended = [], []
        in_prompt = next((rid for rid in live if live[rid] < len(requests[rid]) - tails[rid]), None)
        for rid in list(live):
            toks, done = requests[rid], live[rid]
            head = len(toks) - tails[rid]
            if done < head:
                if rid != in_prompt:
                    continue
                c = min(portion, head - done)
                entries.append({"id": rid, "tokens": list(toks[done:done + c]), "want": [c - 1] if done + c == head else []})
            else:
                if len(live) > 1 and rng.random() < sit_out:
                    continue
                c = 1
                entries.append({"id": rid, "tokens": [toks[done]], "want": [0]})
            live[rid] = done + c
            if live[rid] == len(toks):
                ended.append(rid)
        if not entries:
            continue
        entries.sort(key=lambda e: len(e["tokens"]) != 1)          # decoding requests first, as the engine batches
        steps.append({"step": len(steps), "entries": entries, "end": ended})
        for rid in ended:
            del live[rid]
    return steps


def max_live_tokens(steps, round_to=64):
    """The most tokens live requests hold at any time, each request's count rounded up to ``round_to``."""
    held, best = {}, 0
    for st in steps:
        for e in st["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        best = max(best, sum(-(-n // round_to) * round_to for n in held.values()))
        for rid in st["end"]:
            held.pop(rid, None)
    return best
