"""The kernel's work plan, checked on a CPU through `b200_attn_plan` (no launch, no GPU).

`b200_attn_plan` runs the very functions every CTA of the kernel runs at set-up. For each problem the union of all
CTAs' items must cover every (batch, head, query tile, key tile) exactly once; in key-split mode every item that is
cut has exactly one owner (the part with key tile 0, its CTA's last item), whose `later_parts` following CTAs each
hold one later part as their FIRST item (so a CTA has at most two parts to account for: the kernel keeps one
workspace slot for its first and one for its last item), and two-tile items always come before one-tile items in a
CTA's list.
"""

from __future__ import annotations

import ctypes

import pytest

from fastforks_b200 import _lib

SMS = 148
WHOLE, PARTIAL, OWNER = 0, 1, 2


@pytest.fixture(scope="module")
def lib() -> ctypes.CDLL:
    if _lib.needs_build():
        _lib.build()
    _lib.library.cache_clear()
    return _lib.library()


def args_for(b: int, h: int, n: int, nk: int | None = None, *, workspace: bool = True) -> _lib.B200AttnArgs:
    nk = n if nk is None else nk
    a = _lib.B200AttnArgs()
    a.struct_size = ctypes.sizeof(_lib.B200AttnArgs)
    a.dtype = _lib.F16
    a.q = a.k = a.v = a.o = 0x10000
    for s, tokens in ((a.q_stride, n), (a.k_stride, nk), (a.v_stride, nk), (a.o_stride, n)):
        s[:] = (tokens * h * 64, h * 64, 64)
    a.batch, a.heads, a.q_tokens, a.kv_tokens, a.head_dim = b, h, n, nk, 64
    a.scale = 0.125
    if workspace:
        a.workspace, a.workspace_bytes = 0x100000, 1 << 26
    return a


def plan(lib: ctypes.CDLL, a: _lib.B200AttnArgs, sms: int = SMS) -> tuple[int, list[list[tuple[int, ...]]], list[int]]:
    """(grid, items per CTA, later_parts per CTA)."""
    grid, n_items, later = ctypes.c_int32(), ctypes.c_int32(), ctypes.c_int32()
    assert lib.b200_attn_plan(ctypes.byref(a), sms, 0, ctypes.byref(grid), None, 0, ctypes.byref(n_items), ctypes.byref(later)) == 0, _lib.last_error()
    ctas, laters = [], []
    for cta in range(grid.value):
        assert lib.b200_attn_plan(ctypes.byref(a), sms, cta, ctypes.byref(grid), None, 0, ctypes.byref(n_items), ctypes.byref(later)) == 0
        buf = (ctypes.c_int32 * (7 * max(1, n_items.value)))()
        assert lib.b200_attn_plan(ctypes.byref(a), sms, cta, ctypes.byref(grid), buf, n_items.value, ctypes.byref(n_items), ctypes.byref(later)) == 0
        ctas.append([tuple(buf[7 * i : 7 * i + 7]) for i in range(n_items.value)])
        laters.append(later.value)
    return grid.value, ctas, laters


SHAPES = [
    (8, 6, 1370, None), (4, 16, 1370, None), (32, 24, 1370, None), (1, 12, 4096, None), (1, 6, 1370, None),
    (2, 16, 1370, None), (1, 1, 1370, None), (1, 1, 4096, None), (3, 7, 900, None), (5, 31, 640, None),
    (1, 2, 129, 4000), (1, 1, 128, 20000), (2, 3, 385, 385), (256, 12, 197, None), (25, 12, 196, None),
    (1, 12, 197, None), (1, 1, 1, 1), (2, 3, 300, 77), (1, 3, 257, 1025),
]  # fmt: skip


@pytest.mark.parametrize("workspace", [True, False])
@pytest.mark.parametrize(("b", "h", "n", "nk"), SHAPES)
def test_every_tile_pair_is_covered_exactly_once(lib: ctypes.CDLL, b: int, h: int, n: int, nk: int | None, workspace: bool) -> None:
    nk = n if nk is None else nk
    q_tiles, kv_tiles = -(-n // 128), -(-nk // 128)
    grid, ctas, laters = plan(lib, args_for(b, h, n, nk, workspace=workspace))
    assert 1 <= grid <= SMS
    seen: dict[tuple[int, int, int, int], int] = {}
    for cta, items in enumerate(ctas):
        assert items, f"CTA {cta} has no work"
        tiles_per_item = [it[3] for it in items]
        assert tiles_per_item == sorted(tiles_per_item, reverse=True), "two-tile items must come first"
        for i, (bi, hi, row0, n_tiles, ja, jb, kind) in enumerate(items):
            assert 0 <= bi < b and 0 <= hi < h and row0 % 128 == 0 and n_tiles in (1, 2)
            assert 0 <= ja < jb <= kv_tiles
            assert row0 // 128 + n_tiles <= q_tiles
            assert kind == (PARTIAL if ja > 0 else OWNER if jb < kv_tiles else WHOLE)
            if kind == PARTIAL:
                assert i == 0, "a part that goes to the workspace must be its CTA's first item"
            if kind == OWNER:
                assert i == len(items) - 1 and laters[cta] >= 1
            for t in range(n_tiles):
                for j in range(ja, jb):
                    key = (bi, hi, row0 // 128 + t, j)
                    seen[key] = seen.get(key, 0) + 1
        if items[-1][6] != OWNER:
            assert laters[cta] == 0
    assert len(seen) == b * h * q_tiles * kv_tiles
    assert set(seen.values()) == {1}
    if not workspace or kv_tiles < 3:
        assert all(it[6] == WHOLE for items in ctas for it in items)


@pytest.mark.parametrize(("b", "h", "n", "nk"), [s for s in SHAPES if -(-(s[3] or s[2]) // 128) >= 3])
def test_owner_and_its_later_parts_line_up(lib: ctypes.CDLL, b: int, h: int, n: int, nk: int | None) -> None:
    """The `later_parts` CTAs after an owner hold, as their first items, the rest of the owner's item: same head and
    query rows, key ranges that continue where the previous part stopped and end at the last key tile."""
    nk = n if nk is None else nk
    kv_tiles = -(-nk // 128)
    _, ctas, laters = plan(lib, args_for(b, h, n, nk))
    for cta, items in enumerate(ctas):
        if items[-1][6] != OWNER:
            continue
        head = items[-1]
        at = head[5]
        for part in range(1, laters[cta] + 1):
            nxt = ctas[cta + part][0]
            assert nxt[:4] == head[:4] and nxt[6] == PARTIAL and nxt[4] == at
            at = nxt[5]
        assert at == kv_tiles
        if cta + laters[cta] + 1 < len(ctas):
            after = ctas[cta + laters[cta] + 1][0]
            assert after[:4] != head[:4] or after[4] == 0


def test_key_split_is_taken_where_it_levels_and_left_where_it_does_not(lib: ctypes.CDLL) -> None:
    """[1,12,4096,64] is 192 two-tile items on 148 SMs and [2,16,1370,64] 352 query tiles: dealt whole, the longest
    list is far above the mean; split along the keys every CTA's cost is within two steps of the mean.
    [8,6,1370,64] and [32,24,1370,64] level well enough whole: they stay dealt (a split launch has costs of its own)."""

    def cost(items: list[tuple[int, ...]]) -> float:
        return sum((it[5] - it[4]) * (1.0 if it[3] == 2 else 0.78) for it in items)

    for b, h, n in ((1, 12, 4096), (2, 16, 1370)):
        _, split, _ = plan(lib, args_for(b, h, n))
        _, whole, _ = plan(lib, args_for(b, h, n, workspace=False))
        costs = [cost(items) for items in split]
        assert any(it[6] != WHOLE for items in split for it in items), (b, h, n)
        assert max(costs) - min(costs) <= 2.0
        assert max(costs) < 0.9 * max(cost(items) for items in whole), (b, h, n)
    for b, h, n in ((8, 6, 1370), (32, 24, 1370), (256, 12, 197), (2, 6, 1370), (4, 16, 1370)):
        _, ctas, _ = plan(lib, args_for(b, h, n))
        assert all(it[6] == WHOLE for items in ctas for it in items), (b, h, n)


def test_one_long_item_is_spread_over_many_ctas(lib: ctypes.CDLL) -> None:
    """One head, 129 queries, 20000 keys: one item of 157 key tiles. Whole, it runs on one SM; split, in runs of at
    least eight steps on about twenty."""
    grid, ctas, laters = plan(lib, args_for(1, 1, 129, 20000))
    assert 15 <= grid <= 25
    assert all(len(items) == 1 and items[0][5] - items[0][4] >= 7 for items in ctas)
    assert laters[0] == grid - 1


def test_small_workspace_is_ignored_not_used(lib: ctypes.CDLL) -> None:
    a = args_for(8, 6, 1370)
    a.workspace_bytes = 4096
    _, ctas, _ = plan(lib, a)
    assert all(it[6] == WHOLE for items in ctas for it in items)


@pytest.mark.parametrize(("b", "h", "n"), [(8, 16, 1370), (8, 192, 49), (3, 5, 700), (2, 16, 1370)])
def test_a_bias_shared_by_the_batch_numbers_the_items_batch_fastest(lib: ctypes.CDLL, b: int, h: int, n: int) -> None:
    """With a 16-bit tile-layout bias whose batch stride is 0 the (batch, head) pairs are numbered batch-fastest, so
    the CTAs that read one head's bias run side by side; the coverage is the same, and CTA 0 begins with head 0 of
    image 0 followed (dealt round robin over the grid) by head 0 of other images, not by head 1 of image 0."""
    a = args_for(b, h, n)
    row = (n + 7) // 8 * 8
    a.bias, a.bias_dtype = 0x200000, _lib.F16
    a.bias_stride[:] = (0, n * row, row)
    q_tiles, kv_tiles = -(-n // 128), -(-n // 128)
    grid, ctas, _ = plan(lib, a)
    seen: dict[tuple[int, int, int, int], int] = {}
    for items in ctas:
        for bi, hi, row0, n_tiles, ja, jb, _kind in items:
            for t in range(n_tiles):
                for j in range(ja, jb):
                    key = (bi, hi, row0 // 128 + t, j)
                    seen[key] = seen.get(key, 0) + 1
    assert len(seen) == b * h * q_tiles * kv_tiles and set(seen.values()) == {1}
    first_items = [items[0] for items in ctas]
    per_head = q_tiles // 2 or 1  # items of one (batch, head) at the front of the lists: its two-tile items (a lone tile if it has none)
    if grid > per_head * b and all(it[6] == WHOLE for items in ctas for it in items):  # dealt plans: one item per CTA at the front
        heads_at_the_front = {it[1] for it in first_items[: per_head * b]}
        assert heads_at_the_front == {0}, "the first CTAs should all work on head 0 (every image of it)"
    # without the bias the same problem is numbered head-fastest
    _, plain, _ = plan(lib, args_for(b, h, n))
    if grid > per_head * h and all(it[6] == WHOLE for items in plain for it in items):
        assert {items[0][0] for items in plain[: per_head * h]} == {0}


@pytest.mark.parametrize(("b", "h", "n", "kb", "extra"), [(25, 12, 196, 2, 8), (13, 12, 197, 1, 16), (4, 16, 1370, 2, 112)])
def test_a_thin_last_round_of_two_tile_items_is_taken_apart(lib: ctypes.CDLL, b: int, h: int, n: int, kb: int, extra: int) -> None:
    """300 two-tile items on 148 CTAs: instead of 4 CTAs running a third item while 144 wait, every CTA takes two and
    the 4 left over are worked on as 8 one-tile items by 8 CTAs. Likewise 156 items (8 over) and, with the one-tile
    items a head of 11 query tiles has anyway, [4,16,1370,64] (24 over: 48 + 64 one-tile items on 112 CTAs).
    Coverage is checked by test_every_tile_pair_is_covered_exactly_once; here the shape of the lists."""
    _, ctas, _ = plan(lib, args_for(b, h, n))
    assert all(it[6] == WHOLE for items in ctas for it in items)
    assert {sum(1 for it in items if it[3] == 2) for items in ctas} == {kb}
    singles = [sum(1 for it in items if it[3] == 1) for items in ctas]
    assert set(singles) <= {0, 1} and sum(singles) == extra
    # with eight times the items the lists are long and the last round is left as it is
    _, ctas, _ = plan(lib, args_for(8 * b, h, n) if n < 1000 else args_for(b, h, n, workspace=False))
    assert all(it[6] == WHOLE for items in ctas for it in items)
