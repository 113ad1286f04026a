"""Device pool of the GPU provider, exercised on the CPU device (reuse within a size factor, pool cap, byte limit,
statistics, registry of handed-out blocks); reference behaviour: crates/ronn-providers/src/gpu/allocator.rs:144-370."""
import threading

import pytest
import torch

from ronn_b200.api.errors import ProviderError
from ronn_b200.core.types import DataType
from ronn_b200.providers.device_pool import DevicePool


def test_blocks_are_reused_within_the_size_factor_and_counted():
    pool = DevicePool("cpu")
    a = pool.acquire(1000)
    assert a.numel() == 1024 and a.dtype == torch.uint8                 # rounded to the 512-byte granularity
    pool.release(a)
    b = pool.acquire(600)                                               # 1024 <= 2 x 1024(rounded 600 -> 1024)
    assert b.data_ptr() == a.data_ptr()
    pool.release(b)
    c = pool.acquire(100)                                               # 512 needed: 1024 is within the factor of two
    assert c.data_ptr() == a.data_ptr()
    pool.release(c)
    d = pool.acquire(200)
    e = pool.acquire(200)                                               # pool is empty now: a miss
    st = pool.stats()
    assert (st.hits, st.misses) == (3, 2) and st.live_buffers == 2 and st.hit_rate == pytest.approx(0.6)
    pool.release(d)
    pool.release(e)
    big = pool.acquire(1 << 20)                                         # far more than twice any pooled block: a miss
    assert big.numel() == 1 << 20 and pool.stats().misses == 3
    pool.release(big)
    assert pool.stats().allocated_bytes == 0 and pool.stats().pooled_buffers == 3


def test_small_request_does_not_take_a_much_larger_block():
    pool = DevicePool("cpu")
    big = pool.acquire(1 << 16)
    pool.release(big)
    small = pool.acquire(512)
    assert small.data_ptr() != big.data_ptr() and pool.stats().pooled_buffers == 1


def test_limit_drops_pooled_blocks_before_it_refuses():
    pool = DevicePool("cpu", limit_bytes=4096)
    a = pool.acquire(2048)
    pool.release(a)                                                     # 2048 pooled
    b = pool.acquire(3072 + 512)                                        # needs the pooled block gone
    assert pool.stats().pooled_buffers == 0 and b.numel() == 3584
    with pytest.raises(ProviderError, match="limit"):
        pool.acquire(1024)
    info = pool.get_memory_info()
    assert info.total_bytes == 4096 and info.allocated_bytes == 3584 and info.peak_bytes >= 3584
    pool.release(b)


def test_pool_cap_zero_size_and_foreign_buffers():
    pool = DevicePool("cpu", max_pool_bytes=1024)
    a, b = pool.acquire(1024), pool.acquire(1024)
    pool.release(a)
    pool.release(b)                                                     # the second one does not fit the pool
    assert pool.stats().pooled_bytes == 1024
    with pytest.raises(ProviderError):
        pool.acquire(0)
    with pytest.raises(ProviderError):
        pool.release(torch.empty(16, dtype=torch.uint8))
    with pytest.raises(ProviderError):
        pool.release(a)                                                 # released twice
    assert pool.clear_pools() == (1, 1024)
    with pytest.raises(ProviderError):
        DevicePool("cpu", granularity=300)


def test_typed_tensors_and_the_allocator_interface():
    pool = DevicePool("cpu")
    t = pool.tensor((3, 5), torch.bfloat16)
    assert t.shape == (3, 5) and t.dtype == torch.bfloat16
    t.fill_(1.5)
    pool.release(t)
    e = pool.tensor((0, 4), torch.float32)
    assert e.numel() == 0
    pool.release(e)
    buf = pool.allocate([4, 4], DataType.F32)
    assert buf.size >= 64 and pool.stats().live_buffers == 1
    pool.deallocate(buf)
    assert pool.stats().live_buffers == 0 and pool.stats().deallocation_count == 2


def test_concurrent_use_keeps_the_books_straight():
    pool = DevicePool("cpu", max_pool_bytes=1 << 20)
    errors = []

    def work(seed):
        g = torch.Generator().manual_seed(seed)
        try:
            for _ in range(200):
                n = int(torch.randint(1, 5000, (1,), generator=g))
                blk = pool.acquire(n)
                blk[:1] = 1
                pool.release(blk)
        except Exception as ex:                                         # pragma: no cover
            errors.append(ex)
    threads = [threading.Thread(target=work, args=(i,)) for i in range(8)]
    [t.start() for t in threads]
    [t.join() for t in threads]
    st = pool.stats()
    assert not errors and st.live_buffers == 0 and st.allocated_bytes == 0
    assert st.allocation_count == st.deallocation_count == 1600 and st.hits + st.misses == 1600


def test_random_sequences_keep_the_invariants():
    """Property test: under any interleaving of acquire / release the books balance, the limit holds, blocks handed out
    never alias, and a pooled block is reused only within the size factor."""
    from hypothesis import given, settings, strategies as st

    @settings(max_examples=60, deadline=None)
    @given(st.lists(st.tuples(st.booleans(), st.integers(min_value=1, max_value=20000)), min_size=1, max_size=60))
    def run(ops):
        limit = 64 * 1024
        pool = DevicePool("cpu", limit_bytes=limit, max_pool_bytes=16 * 1024)
        live = []
        for is_alloc, n in ops:
            if is_alloc or not live:
                try:
                    blk = pool.acquire(n)
                except ProviderError:
                    assert sum(b.numel() for b in live) + pool._round(n) > limit      # refused only when it cannot fit
                    continue
                assert blk.numel() >= n and blk.numel() <= 2 * pool._round(n)
                assert all(blk.data_ptr() != b.data_ptr() for b in live)
                live.append(blk)
            else:
                pool.release(live.pop(n % len(live)))
            s = pool.stats()
            assert s.live_buffers == len(live) and s.allocated_bytes == sum(b.numel() for b in live)
            assert s.allocated_bytes + s.pooled_bytes <= limit and s.pooled_bytes <= 16 * 1024
            assert s.peak_bytes >= s.allocated_bytes
        for b in live:
            pool.release(b)
        assert pool.stats().allocated_bytes == 0
    run()
