"""Block allocator of the paged KV cache (CPU)."""
import pytest
import torch


def test_reserve_release_and_block_zero_is_never_handed_out():
    from libtbvcoll_b200.engine.kv_cache import BlockManager
    bm = BlockManager(num_blocks=10, block_size=16, max_batch=4, max_blocks_per_seq=4, device="cpu")
    bm.reserve(0, 33)                                   # 3 blocks
    bm.reserve(1, 16)                                   # 1 block
    assert len(bm.owned[0]) == 3 and len(bm.owned[1]) == 1
    used = bm.owned[0] + bm.owned[1]
    assert 0 not in used and len(set(used)) == 4
    bm.reserve(0, 40)                                   # already covered: nothing new
    assert len(bm.owned[0]) == 3
    assert bm.slot(0, 17) == bm.owned[0][1] * 16 + 1
    bm.sync_to_device()
    assert torch.equal(bm.tables, bm.tables_host)
    with pytest.raises(ValueError):
        bm.reserve(2, 16 * 4 + 1)                       # longer than max_blocks_per_seq
    bm.reserve(2, 64)
    with pytest.raises(RuntimeError):
        bm.reserve(3, 32)                               # 9 usable blocks: 3 + 1 + 4 taken, 1 left, 2 wanted
    bm.release(0)
    assert bm.tables_host[0].abs().sum().item() == 0 and not bm.owned[0]
    bm.reserve(3, 32)                                   # the freed blocks are reusable
    bm.release_all()
    assert sorted(bm.free) == list(range(1, 10))
