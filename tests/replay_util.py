"""Run a trace through the engine's step function in-process and collect logits per (request, position)."""
import torch

from zedinfer_b200.engine.core import EngineCore, StepEntry


def run_trace(core: EngineCore, steps):
    got = {}
    progress = {}
    for st in steps:
        entries = [StepEntry(e["id"], e["tokens"], e["want"]) for e in st["entries"]]
        logits = core.step(entries)
        row = 0
        for e in st["entries"]:
            base = progress.get(e["id"], 0)
            for j in e["want"]:
                got[(e["id"], base + j)] = logits[row].float().cpu()
                row += 1
            progress[e["id"]] = base + len(e["tokens"])
        for rid in st["end"]:
            core.end(rid)
            progress.pop(rid, None)
    core.cache.check()
    return got


def compare(got, expected, requests):
    """Largest absolute difference over all positions, and the first position where it is worst."""
    worst, where = 0.0, None
    for rid, toks in requests.items():
        for p in range(len(toks)):
            d = float((got[(rid, p)] - expected[rid][p]).abs().max())
            if d > worst:
                worst, where = d, (rid, p)
    return worst, where


def first_bad(got, expected, requests, tol):
    for rid, toks in requests.items():
        for p in range(len(toks)):
            d = float((got[(rid, p)] - expected[rid][p]).abs().max())
            if not d <= tol:
                return rid, p, d
    return None


def first_bad_wanted(got, expected, tol):
    """As :func:`first_bad`, over the positions that were asked for (``got``'s keys) instead of every position."""
    for (rid, p), row in sorted(got.items(), key=lambda kv: (str(kv[0][0]), kv[0][1])):
        d = float((row - expected[rid][p]).abs().max())
        if not d <= tol:
            return rid, p, d
    return None
