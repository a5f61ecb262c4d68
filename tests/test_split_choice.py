"""How many ways the attention part splits the keys: the estimates are plain
arithmetic over the device's size, checked here against a described device (148 SMs,
the thread-block clusters a B200 was measured to hold) without one."""

import pytest
import torch

DEVICE = torch.device("cpu")  # a key into the part's tables, nothing runs on it
CLUSTERS = {2: 148, 3: 93, 4: 71, 5: 56, 6: 45, 7: 37, 8: 33, 9: 30, 10: 26, 11: 21, 12: 21, 13: 17, 14: 14, 15: 14,
            16: 14}


@pytest.fixture()
def part(monkeypatch):
    from pulsarlm_b200.parts import attention

    monkeypatch.setitem(attention._SM_COUNT, DEVICE, 148)
    for group in (1, 4):
        for splits, room in CLUSTERS.items():
            monkeypatch.setitem(attention._CLUSTER_ROOM, (DEVICE, 128, group, splits), room)
    monkeypatch.setattr(attention, "_DECODE_SPLITS", {})
    return attention


def test_decode_splits_fill_the_device_without_a_sparse_last_round(part):
    pick = lambda n, context, group=4: part.decode_splits(n, context, DEVICE, 128, group)  # noqa: E731
    assert pick(64, 2048) == 4            # batch 8 x 8 kv heads: 256 CTAs in one round
    assert pick(8, 2048) == 16            # batch 1: the largest cluster
    assert pick(8, 32768) > 16            # batch 1, long history: through scratch memory
    assert pick(128, 2048) == 2           # 128 CTAs alone stream at 36 GB/s each
    assert pick(192, 2048) == 1 and pick(256, 2048) == 1 and pick(512, 2048) == 1
    assert pick(320, 4096, group=1) > 1   # 320 CTAs unsplit leave a second round of 24 long ones
    for n in (1, 3, 8, 40, 64, 100, 320, 1000):
        for context in (1, 16, 200, 2048, 100000):
            splits = pick(n, context)
            assert splits >= 1
            # no split shorter than eight 16-key tiles
            assert splits == 1 or context // splits >= 8 * 16 - 16
            # more than sixteen only when few CTAs would otherwise run
            assert splits <= 16 or n * 32 <= 2 * 148 * 2


def test_prefill_splits_only_for_few_tiles_over_many_keys(part):
    pick = lambda ctas, keys, tokens: part.prefill_splits(ctas, keys, tokens, 32, 128, DEVICE)  # noqa: E731
    assert pick(32, 256, 256) == 1                 # a short prompt: nothing to split
    assert pick(32, 8192 + 256, 256) == 4          # 256 tokens after 8,192: 128 CTAs
    assert pick(64, 8192 + 512, 512) == 2
    assert pick(16, 32768 + 128, 128) == 9         # 144 CTAs
    assert pick(128, 32768 + 1024, 1024) == 1      # 128 CTAs already: a second round would cost more
    assert pick(256, 32768 + 2048, 2048) == 1
    for ctas in (1, 16, 40, 80, 147, 148, 500):
        for keys in (1, 300, 2048, 40000):
            splits = pick(ctas, keys, 128)
            assert 1 <= splits <= 16
            assert splits == 1 or keys // splits >= 256


def test_work_items_cover_every_tile_once_and_leave_even_batches_whole():
    import random

    from pulsarlm_b200.parts.attention import decode_work_items

    rng = random.Random(4)
    for trial in range(200):
        n = rng.choice([1, 2, 7, 64, 130])
        lengths = [rng.choice([1, 16, 17, rng.randrange(1, 9000)]) for _ in range(n)]
        window = rng.choice([None, None, 40, 1000])
        target = rng.choice([1, 5, 74, 300, 1200])
        pad = rng.choice([None, target + n])
        items, slots = decode_work_items(lengths, window, target, pad, min_tiles=8)
        assert items.dtype.name == "int32" and items.shape[1] == 4 and slots.shape == (n,)
        assert pad is None or items.shape[0] == pad
        real = [tuple(int(v) for v in r) for r in items if r[2] > 0]
        assert len(real) <= target + n
        assert [r[2] for r in real] == sorted((r[2] for r in real), reverse=True)   # longest first
        assert pad is None or len(real) == pad or items[-1, 0] == len(real)   # the padding says how many are real
        used_slots = set()
        for t, c in enumerate(lengths):
            first = (max(0, c - window) if window else 0) // 16
            mine = sorted(r for r in real if r[0] == t)
            assert mine[0][1] == first and mine[-1][1] + mine[-1][2] == -(-c // 16)
            assert all(a[1] + a[2] == b[1] for a, b in zip(mine, mine[1:]))
            splits = {r[3] >> 12 for r in mine}
            assert splits == {len(mine)} and sorted(r[3] & 4095 for r in mine) == list(range(len(mine)))
            if len(mine) > 1:
                assert all(r[2] >= 4 for r in mine)       # no sliver: at least half the smallest item
                for s in range(len(mine)):
                    assert slots[t] + s not in used_slots and slots[t] + s < items.shape[0]
                    used_slots.add(int(slots[t]) + s)
    # requests of about one length are left whole, whatever the target
    items, _ = decode_work_items([2000, 2100, 1900, 2050], None, 1000)
    assert int((items[:, 2] > 0).sum()) == 4
    # one long request among short ones is cut into about `target` items
    items, _ = decode_work_items([100000] + [500] * 31, None, 148)
    assert 100 <= int((items[:, 2] > 0).sum()) <= 148 + 32


def test_unequal_lengths_are_told_from_equal_ones(part):
    assert not part._uneven([2048] * 24) and not part._uneven([7])
    assert not part._uneven([2000, 2100, 2200, 2500])            # the longest within 1.3 of the mean
    assert part._uneven([300, 900, 2400, 4500]) and part._uneven([100] * 23 + [4000])


def test_small_batches_take_clusters_that_find_room_inside_a_step(part):
    pick = lambda n, context: part.decode_splits(n, context, DEVICE, 128, 4)  # noqa: E731
    # (two, three and four requests of 8 kv heads: not the 13, 10 and 8 shares the occupancy query alone allows)
    assert [pick(16, 2048), pick(24, 2048), pick(32, 2048)] == [10, 8, 6]
    assert pick(8, 2048) == 16 and pick(128, 2048) == 2
