"""The packed int32 descriptor of a step, built on the host with numpy alone (no device in here, so the layout is
tested without a GPU).

One array holds everything a step's kernels index by: ``ids | positions (one run per axis) | token -> segment | wanted rows | state slots
| attention tiles | block tables of every cache group``.  It goes to the device in a single copy, and a captured step
keeps it in a static buffer, so its length and every offset must depend on the step's *counts* alone
(:func:`step_signature`), never on which requests or how many of the single tokens are real.

Single-token entries at the head of a step that also holds longer ones (decoding requests beside a prompt portion) are
left to the decode attention kernel; the padding tokens of a captured step stand right behind them, so that their
number is a count too.  Attention tiles cover the rest.  Padding tokens want their logits as well (rows nobody reads, at
the end of the wanted rows), for the same reason.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Sequence, Tuple

import numpy as np


def step_padding(lens: Sequence[int]) -> int:
    """Single-token segments beside longer ones are padded to a power of two, so that fewer different counts occur;
    a step of single tokens only (pure decode) and a step without any are not padded here."""
    singles = sum(1 for k in lens if k == 1)
    if singles == 0 or singles == len(lens):
        return 0
    bucket = 1
    while bucket < singles:
        bucket *= 2
    return bucket - singles


def step_signature(lens: Sequence[int], n_wants: int, pad: int, tile_rows: int) -> tuple:
    """The counts that every launch of the step depends on: tokens, segments, the single tokens at its head (padding
    included) that the decode attention kernel takes, attention tiles of the rest, wanted rows, pure decode or not."""
    lead = 0
    if any(k != 1 for k in lens):
        while lens[lead] == 1:
            lead += 1
        tiles = sum(-(-k // tile_rows) for k in lens[lead:])
        lead += pad
    else:
        tiles = len(lens) + pad
    return (sum(lens) + pad, len(lens) + pad, lead, tiles, n_wants + pad, lead == 0 and all(k == 1 for k in lens))


@dataclass
class StepLayout:
    n_tok: int
    n_seg: int
    n_want: int            # padding rows included
    n_real_want: int
    n_tiles: int
    lead: int              # single tokens at the head (padding included) that go to the decode attention kernel
    off_ids: int
    off_pos: int
    off_seg: int
    off_want: int
    off_slots: int
    off_tiles: int
    off_tab: int
    total: int
    width: int
    n_groups: int
    pos_width: int = 1
    max_kv: int = 1
    seg_start: List[int] = field(default_factory=list)
    seg_len: List[int] = field(default_factory=list)
    seg_pos0: List[int] = field(default_factory=list)
    slots: List[int] = field(default_factory=list)


def pack_step(names: Sequence, tokens: Sequence[Sequence[int]], wants: Sequence[Sequence[int]], lengths: Sequence[int],
              slots: Sequence[int], tables: Sequence[Sequence[Sequence[int]]], n_groups: int, width: int, vocab: int,
              scratch_pages: Sequence[int], tile_rows: int, pad_segments: int = 0, pos_width: int = 1
              ) -> Tuple[np.ndarray, StepLayout]:
    """``names[i]``: the request of entry i (for messages); ``tokens[i]`` its new tokens; ``wants[i]`` the places
    among them whose logits are wanted; ``lengths[i]`` the tokens it has in the cache; ``slots[i]`` its state slot;
    ``tables[i][g]`` its page numbers in cache group g.  ``pos_width``: position numbers per token (the model's
    ``position_width``); they lie axis by axis, ``pos_width`` runs of one number per token, and every axis of a token
    holds its index in the request.  Returns the descriptor and where everything lies in it."""
    lens = [len(t) for t in tokens]
    n_seg = len(tokens) + pad_segments
    n_tok = sum(lens) + pad_segments
    n_real_want = sum(len(w) for w in wants)
    n_want = n_real_want + pad_segments
    lead_real = lead = 0
    if any(k != 1 for k in lens):
        while lens[lead_real] == 1:
            lead_real += 1
        lead = lead_real + pad_segments
    if lead:
        n_tiles = sum(-(-k // tile_rows) for k in lens[lead_real:])
    else:
        n_tiles = sum(-(-k // tile_rows) for k in lens) + pad_segments
    off_ids, off_pos, off_seg = 0, n_tok, (1 + pos_width) * n_tok
    off_want = off_seg + n_tok
    off_slots = off_want + n_want
    off_tiles = off_slots + n_seg
    off_tab = off_tiles + 3 * n_tiles
    total = off_tab + n_groups * n_seg * width
    lay = StepLayout(n_tok, n_seg, n_want, n_real_want, n_tiles, lead, off_ids, off_pos, off_seg, off_want, off_slots,
                     off_tiles, off_tab, total, width, n_groups, pos_width)
    host = np.zeros(total, dtype=np.int32)
    t = w = s = tile = 0
    pad_rows: List[int] = []

    def pad_tokens():                      # padding: one token each at position 0 of the scratch page
        nonlocal t, s, tile
        for _ in range(pad_segments):
            pad_rows.append(t)
            host[off_seg + t] = s
            host[off_slots + s] = -1
            for g in range(n_groups):
                host[off_tab + (g * n_seg + s) * width] = scratch_pages[g]
            if not lead:
                host[off_tiles + 3 * tile: off_tiles + 3 * tile + 3] = (t, 1, s)
                tile += 1
            lay.seg_start.append(t), lay.seg_len.append(1), lay.seg_pos0.append(0), lay.slots.append(-1)
            t, s = t + 1, s + 1

    for i, toks_i in enumerate(tokens):
        if lead and i == lead_real:
            pad_tokens()
        toks = np.asarray(toks_i, dtype=np.int64)
        k = toks.size
        if k and (toks.min() < 0 or toks.max() >= vocab):
            raise ValueError(f"request {names[i]!r}: token id outside [0, {vocab})")
        host[off_ids + t: off_ids + t + k] = toks
        for axis in range(pos_width):
            host[off_pos + axis * n_tok + t: off_pos + axis * n_tok + t + k] = np.arange(lengths[i], lengths[i] + k, dtype=np.int32)
        host[off_seg + t: off_seg + t + k] = s
        for j in wants[i]:
            if not 0 <= j < k:
                raise ValueError(f"request {names[i]!r}: wanted place {j} is outside its {k} tokens")
            host[off_want + w] = t + j
            w += 1
        host[off_slots + s] = slots[i]
        for g in range(n_groups):
            tab = np.asarray(tables[i][g], dtype=np.int32)
            base = off_tab + (g * n_seg + s) * width
            # a page that a window has passed and given back (-1) is shown to the kernels as the scratch page:
            # its keys are masked anyway, and no kernel ever forms an address or a TMA coordinate from -1
            host[base: base + tab.size] = np.where(tab < 0, scratch_pages[g], tab)
        if not (lead and i < lead_real):
            for q0 in range(0, k, tile_rows):
                host[off_tiles + 3 * tile: off_tiles + 3 * tile + 3] = (t + q0, min(tile_rows, k - q0), s)
                tile += 1
        lay.seg_start.append(t), lay.seg_len.append(k), lay.seg_pos0.append(lengths[i]), lay.slots.append(slots[i])
        lay.max_kv = max(lay.max_kv, lengths[i] + k)
        t += k
        s += 1
    if not lead:
        pad_tokens()
    host[off_want + w: off_want + w + len(pad_rows)] = pad_rows
    return host, lay
