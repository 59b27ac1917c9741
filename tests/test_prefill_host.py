"""Host-side prefill set-up (CPU): the vectorised row arrays and the query-tile list equal the plain
per-row statement of the same thing."""
import random

import numpy as np
import torch


def test_prefill_rows_equal_per_row_loop():
    from libtbvcoll_b200.engine.engine import prefill_rows
    from libtbvcoll_b200.engine.kv_cache import BlockManager
    rng = random.Random(1)
    for _ in range(40):
        B = rng.randint(1, 5)
        prompts = [[rng.randint(0, 999) for _ in range(rng.randint(1, 90))] for _ in range(B)]
        bm = BlockManager(200, 16, 8, 16, "cpu")
        for b, p in enumerate(prompts):
            bm.reserve(b, len(p) + 4)
        total, seq, pos, ids, slots, is_last = prefill_rows(prompts, bm.tables_host.numpy(), bm.block_size)
        rows = [(b, i, t) for b, p in enumerate(prompts) for i, t in enumerate(p)]
        assert total == len(rows)
        assert seq.tolist() == [r[0] for r in rows] and pos.tolist() == [r[1] for r in rows] and ids.tolist() == [r[2] for r in rows]
        assert slots.tolist() == [bm.slot(b, i) for b, i, _ in rows]
        assert is_last.tolist() == [i == len(prompts[b]) - 1 for b, i, _ in rows]
        assert len(set(slots.tolist())) == total and int(slots.min()) >= bm.block_size      # distinct, never in reserved block 0


def test_prefill_tiles_equal_greedy_segmentation():
    from libtbvcoll_b200 import ops

    def greedy(seqs, group):
        qt = max(1, 64 // group)
        tiles, i, n = [], 0, len(seqs)
        while i < n:
            j = i
            while j < n and j - i < qt and seqs[j] == seqs[i]:
                j += 1
            tiles.append((i, j - i))
            i = j
        return tiles
    rng = random.Random(2)
    for _ in range(100):
        lens = [rng.randint(1, 70) for _ in range(rng.randint(1, 6))]
        seq = np.repeat(np.arange(len(lens)), lens)
        c0 = rng.randint(0, len(seq) - 1)
        c1 = rng.randint(c0 + 1, len(seq))
        chunk = torch.from_numpy(seq[c0:c1].astype(np.int32))
        for g in (1, 4, 8, 64):
            got = ops.prefill_tiles(chunk, g)
            assert got.dtype is torch.int32 and got.tolist() == [list(t) for t in greedy(chunk.tolist(), g)]
    assert ops.prefill_tiles(torch.zeros(0, dtype=torch.int32), 4).shape == (0, 2)
