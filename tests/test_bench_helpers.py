"""Host-side pieces of bench.py that the multi-GPU parity record rests on: rows drawn from the GLOBAL token index
are the same however the batch is sharded, and the bit-pattern checksum of a sharded tensor, summed over the
shards, equals the checksum of the whole."""
import importlib.util
import os

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
spec = importlib.util.spec_from_file_location("bench", os.path.join(ROOT, "bench.py"))
bench = importlib.util.module_from_spec(spec)
spec.loader.exec_module(bench)

from omega_ai_b200.ep_layout import shard_tokens  # noqa: E402


def test_rows_do_not_depend_on_the_sharding():
    dev, d, T = torch.device("cpu"), 64, 5000   # spans three seed blocks of 2048 tokens, the last one partial
    whole = bench.global_rows(torch, dev, 0, T, d, torch.bfloat16, bench.SEED)
    for world in (2, 4, 8):
        parts = [bench.global_rows(torch, dev, *shard_tokens(T, world, r), d, torch.bfloat16, bench.SEED)
                 for r in range(world)]
        assert torch.equal(torch.cat(parts), whole)
    assert not torch.equal(whole[:2048], bench.global_rows(torch, dev, 0, 2048, d, torch.bfloat16, bench.SEED + 1))


def test_checksum_adds_up_over_shards_and_sees_single_bit_changes():
    dev, d, T = torch.device("cpu"), 32, 777
    y = torch.randn(T, d, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16)
    whole = bench.bits_checksum(torch, y, 0)
    for world in (2, 4, 8):
        total = 0
        for r in range(world):
            lo, hi = shard_tokens(T, world, r)
            total += bench.bits_checksum(torch, y[lo:hi], lo * d) if hi > lo else 0
        assert total == whole
    z = y.clone()
    z.view(torch.int16)[123, 7] ^= 1   # one bit of one element
    assert bench.bits_checksum(torch, z, 0) != whole
    # a swap of two rows changes it too (the weights depend on the global position)
    w = y.clone()
    w[[3, 4]] = w[[4, 3]]
    assert bench.bits_checksum(torch, w, 0) != whole
    idx = torch.randint(0, 8, (T, 2), generator=torch.Generator().manual_seed(2), dtype=torch.int64)
    assert bench.bits_checksum(torch, idx, 0) == bench.bits_checksum(torch, idx[:400], 0) + bench.bits_checksum(torch, idx[400:], 800)
