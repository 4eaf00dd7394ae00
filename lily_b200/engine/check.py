"""Checks of what a step hands to the kernels, for debugging: ``LILY_B200_CHECK_STEPS=1``.

The kernels index the paged cache through the step's block tables, positions and slots and trust them:
a page id beyond the pool, a table row that does not cover a position, or a page that two live
requests both hold would read or write somebody else's keys, or memory outside the cache, without
any error (the device-side memory checker is not available where this engine is developed).  With the
switch on, the step function verifies, on the host and before anything is launched, that

* every request of the step is open, and its cached length is what the cache manager believes;
* it stays within the context length;
* in every cache group its block table covers every position the step writes and every position the
  step may read (all of them, or the window's), with page ids inside the pool and never page 0;
* no page is held by two live requests of a group;
* the wanted rows lie inside the step's tokens, and token ids inside the vocabulary;
* a captured decode batch's padded rows name slot 0 and page 0, which belong to no request.

It costs a pass over the live block tables each step, so it is off unless asked for; the tests switch it on.
"""

from __future__ import annotations

import os
from typing import List, Sequence

ENABLED = os.environ.get("LILY_B200_CHECK_STEPS", "") not in ("", "0")


class StepCheckError(AssertionError):
    pass


def _fail(msg: str) -> None:
    raise StepCheckError("step check: " + msg)


def check_tables(cache, slots_and_lengths: Sequence[tuple]) -> None:
    """``slots_and_lengths``: (slot, positions cached before the step, positions after it)."""
    for g, group in enumerate(cache.groups):
        tables, window, page = group.tables, group.tables.window, cache.page_size
        for slot, before, after in slots_and_lengths:
            if slot not in tables.tables:
                _fail(f"slot {slot} has no block table in cache group {g}")
            pages = tables.tables[slot].pages
            if len(pages) * page < after:
                _fail(f"slot {slot}, group {g}: {len(pages)} pages of {page} do not cover {after} positions")
            # the oldest position any query of this step may look at
            first_read = 0 if window is None else max(0, before + 1 - window)
            for i in range(first_read // page, -(-after // page)):
                if not (1 <= pages[i] <= cache.num_pages):
                    _fail(f"slot {slot}, group {g}: page id {pages[i]} at table entry {i}, whose positions {i * page} to "
                          f"{(i + 1) * page - 1} this step reads or writes (the pool has pages 1 to {cache.num_pages})")
        owner = {}
        for slot, table in tables.tables.items():
            for p in table.pages:
                if p == 0:
                    continue
                if p in owner and owner[p] != slot:
                    _fail(f"group {g}: page {p} is held by slots {owner[p]} and {slot}")
                owner[p] = slot


def check_entries(runner, entries) -> None:
    """Before a step: the requests, their lengths and their tables (after the tables have grown)."""
    triples = []
    for e in entries:
        if e.slot not in runner.seq_lens or not (1 <= e.slot <= runner.max_requests):
            _fail(f"request slot {e.slot} is not open")
        before = runner.seq_lens[e.slot]
        after = before + len(e.tokens)
        if after > runner.context_len:
            _fail(f"slot {e.slot} would hold {after} positions, the context length is {runner.context_len}")
        if runner.cache.lengths.get(e.slot, -1) < after:
            _fail(f"slot {e.slot}: the cache manager holds pages for {runner.cache.lengths.get(e.slot)} positions, the step needs {after}")
        triples.append((e.slot, before, after))
    check_tables(runner.cache, triples)


def check_batch(runner, batch) -> None:
    """A packed batch against its own host fields."""
    n = batch.num_tokens
    if sum(batch.h_new_lens) != n or len(batch.h_new_lens) != batch.num_requests:
        _fail("token counts of the batch do not add up")
    rows = batch.logit_rows.tolist()
    if any(not (0 <= r < n) for r in rows):
        _fail(f"a wanted row lies outside the {n} tokens of the step")
    ids = batch.token_ids.tolist()
    vocab = runner.spec.vocab_size
    for t in ids:
        if t >= vocab or (t < 0 and not (1 <= -t - 1 <= runner.max_requests)):
            _fail(f"token id {t} is neither in the vocabulary of {vocab} nor the mark of a request slot")
    if any(ln == 1 for ln in batch.h_new_lens[batch.num_decode:]) or any(ln != 1 for ln in batch.h_new_lens[:batch.num_decode]):
        _fail("one-token requests must come first")


def check_graph_fill(runner, graph, live: int) -> None:
    """The padded rows of a captured decode batch name slot 0 and page 0."""
    if any(int(s) != 0 for s in graph._slots[live:]):
        _fail("a padded row of a captured batch names a request slot")
    for view in graph._tables:
        if view[live:].any():
            _fail("a padded row of a captured batch names a page")
    for r in range(live):
        if int(graph._seq[r]) != int(graph._positions[r]) + 1 or int(graph._prefix[r]) != int(graph._positions[r]):
            _fail(f"row {r} of a captured batch: position {int(graph._positions[r])}, prefix {int(graph._prefix[r])}, length {int(graph._seq[r])}")
        slot = int(graph._slots[r])
        for view, group in zip(graph._tables, range(len(runner.cache.groups))):
            pages: List[int] = runner.cache.block_table(group, slot)
            if view[r, :len(pages)].tolist() != list(pages) or view[r, len(pages):].any():
                _fail(f"row {r} of a captured batch does not hold the block table of slot {slot} in group {group}")
