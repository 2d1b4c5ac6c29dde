"""The packed descriptor of a step (zedinfer_b200/engine/descriptor.py), on the host: every token once, at its place;
single tokens at the head and the padding behind them; tiles over the rest; wanted rows with the padding's last; and
a layout that depends on the step's counts alone."""
import random

import numpy as np
import pytest

from zedinfer_b200.engine.descriptor import pack_step, step_padding, step_signature

TILE = 128
SCRATCH = [999, 777]          # the scratch page of each group: pools of different sizes


def make(lens, cached=None, wants=None, n_groups=2, width=48, pad=None, vocab=5000, seed=0):
    rng = random.Random(seed)
    cached = cached or [rng.randrange(0, 40) for _ in lens]
    tokens = [[rng.randrange(vocab) for _ in range(k)] for k in lens]
    wants = wants if wants is not None else [[k - 1] for k in lens]
    tables = [[[100 * (i + 1) + 10 * g + b for b in range((cached[i] + lens[i] + 15) // 16)] for g in range(n_groups)]
              for i in range(len(lens))]
    slots = list(range(len(lens)))
    pad = step_padding(lens) if pad is None else pad
    host, lay = pack_step([f"r{i}" for i in range(len(lens))], tokens, wants, cached, slots, tables, n_groups, width, vocab,
                          SCRATCH, TILE, pad)
    return host, lay, tokens, cached, wants, tables, pad


def check(host, lay, tokens, cached, wants, tables, pad):
    lens = [len(t) for t in tokens]
    assert host.dtype == np.int32 and host.size == lay.total
    ids = host[lay.off_ids: lay.off_ids + lay.n_tok]
    pos = host[lay.off_pos: lay.off_pos + lay.n_tok]
    seg = host[lay.off_seg: lay.off_seg + lay.n_tok]
    assert lay.n_tok == sum(lens) + pad and lay.n_seg == len(lens) + pad
    mixed = any(k != 1 for k in lens)
    lead_real = 0
    if mixed:
        while lens[lead_real] == 1:
            lead_real += 1
    assert lay.lead == (lead_real + pad if mixed else 0)
    # where each entry's tokens lie: the padding stands behind the leading single tokens of a mixed step, else last
    row, s, first_row, first_seg = 0, 0, [], []
    for i, k in enumerate(lens):
        if mixed and i == lead_real:
            row, s = row + pad, s + pad
        first_row.append(row), first_seg.append(s)
        row, s = row + k, s + 1
    for i, k in enumerate(lens):
        r0 = first_row[i]
        assert list(ids[r0: r0 + k]) == tokens[i]
        assert list(pos[r0: r0 + k]) == list(range(cached[i], cached[i] + k))
        assert set(seg[r0: r0 + k]) == {first_seg[i]}
        assert host[lay.off_slots + first_seg[i]] == i
        for g in range(lay.n_groups):
            base = lay.off_tab + (g * lay.n_seg + first_seg[i]) * lay.width
            assert list(host[base: base + len(tables[i][g])]) == tables[i][g]
    pad_rows = list(range(lead_real, lead_real + pad)) if mixed else list(range(lay.n_tok - pad, lay.n_tok))
    for r in pad_rows:
        assert pos[r] == 0 and host[lay.off_slots + seg[r]] == -1
        for g in range(lay.n_groups):
            assert host[lay.off_tab + (g * lay.n_seg + seg[r]) * lay.width] == SCRATCH[g]
    assert sorted(seg[r] for r in pad_rows) == sorted(set(range(lay.n_seg)) - set(first_seg))
    # wanted rows: the real ones in the order of the entries, the padding's behind them
    want = list(host[lay.off_want: lay.off_want + lay.n_want])
    real = [first_row[i] + j for i in range(len(lens)) for j in wants[i]]
    assert want == real + pad_rows and lay.n_real_want == len(real)
    # tiles: every token that is not a leading single (or its padding) once, a tile inside one segment, at most TILE rows
    tiles = host[lay.off_tiles: lay.off_tiles + 3 * lay.n_tiles].reshape(-1, 3)
    covered = []
    for r0, n, sg in tiles:
        assert 1 <= n <= TILE and set(seg[r0: r0 + n]) == {sg}
        assert list(pos[r0: r0 + n]) == list(range(pos[r0], pos[r0] + n))
        covered += list(range(r0, r0 + n))
    assert sorted(covered) == list(range(lay.lead, lay.n_tok)) and len(covered) == len(set(covered))
    assert lay.max_kv == max(c + k for c, k in zip(cached, lens))
    assert lay.seg_len == [len(np.where(seg == s)[0]) for s in range(lay.n_seg)]


@pytest.mark.parametrize("lens", [[1, 1, 1, 300], [1, 200, 1, 57], [64], [1, 1, 1, 1, 1], [5, 2, 11], [1, 1, 130, 2, 1],
                                  [1] * 33 + [512], [2, 1], [129, 128, 127]])
def test_every_token_tile_and_wanted_row_is_where_it_belongs(lens):
    check(*make(lens))
    check(*make(lens, wants=[[] for _ in lens]))
    check(*make(lens, wants=[list(range(k)) for k in lens], n_groups=1, width=40, seed=3))


def test_random_steps():
    rng = random.Random(9)
    for trial in range(200):
        n = rng.randrange(1, 9)
        lens = [rng.choice([1, 1, 1, 2, 3, 17, 128, 129, 260]) for _ in range(n)]
        wants = [sorted(rng.sample(range(k), rng.randrange(0, min(k, 3) + 1))) for k in lens]
        check(*make(lens, wants=wants, seed=trial))


def test_the_layout_depends_on_counts_alone():
    """Five to eight decoding requests beside a portion of 512 are one shape: same signature, same length, same
    offsets, whichever of the single tokens are padding."""
    seen = set()
    for singles in (5, 6, 7, 8):
        lens = [1] * singles + [512]
        wants = [[0]] * singles + [[511]]
        host, lay, *_ = make(lens, wants=wants)
        sig = step_signature(lens, sum(len(w) for w in wants), step_padding(lens), TILE)
        seen.add((sig, lay.total, lay.lead, lay.n_want, lay.n_tiles, lay.off_want, lay.off_slots, lay.off_tiles, lay.off_tab))
        assert lay.lead == 8 and lay.n_want == 9 and lay.n_tiles == 4
    assert len(seen) == 1
    # a portion cut into two segments, or without a wanted row, is another shape
    a = step_signature([1] * 8 + [512], 9, 0, TILE)
    assert a != step_signature([1] * 8 + [200, 312], 10, 0, TILE) and a != step_signature([1] * 8 + [512], 8, 0, TILE)
    assert step_signature([1] * 4, 4, 0, TILE)[-1] and not a[-1]


def test_padding_rule():
    assert step_padding([1, 1, 1, 40]) == 1 and step_padding([1, 40]) == 0 and step_padding([40, 1, 1, 1, 1, 1]) == 3
    assert step_padding([1, 1, 1]) == 0 and step_padding([40, 30]) == 0            # pure decode / no single token


def test_bad_input_is_refused():
    with pytest.raises(ValueError, match="token id outside"):
        pack_step(["a"], [[5, 7000]], [[1]], [0], [0], [[[1]]], 1, 4, 5000, SCRATCH, TILE)
    with pytest.raises(ValueError, match="wanted place"):
        pack_step(["a"], [[5, 6]], [[2]], [0], [0], [[[1]]], 1, 4, 5000, SCRATCH, TILE)


def test_pages_given_back_behind_a_window_are_shown_as_the_scratch_page():
    """A block-table entry of -1 (the window has passed the page and the pool has it back) never reaches a kernel:
    the descriptor shows the scratch page there, so no address or TMA coordinate is formed from -1."""
    tokens = [[5, 6, 7], [9]]
    tables = [[[-1, -1, 40, 41], [3, 4, 5, 6]], [[-1, 8], [7, 8]]]      # group 0 has a window, group 1 has none
    host, lay = pack_step(["a", "b"], tokens, [[2], [0]], [50, 20], [-1, -1], tables, 2, 6, 100, SCRATCH, TILE, 0)
    tab = host[lay.off_tab:].reshape(2, lay.n_seg, lay.width)
    assert tab[0, 0].tolist() == [999, 999, 40, 41, 0, 0] and tab[1, 0].tolist() == [3, 4, 5, 6, 0, 0]
    assert tab[0, 1].tolist() == [999, 8, 0, 0, 0, 0] and tab[1, 1].tolist() == [7, 8, 0, 0, 0, 0]
    assert (host[lay.off_tab:] >= 0).all()
