"""Tiered paging HBM <-> pinned host: bit-exact round trips of whole pages (all layers, K and V)."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
from breccia_b200 import _lib, synth
from breccia_b200.qsa import DecodeBatch, KvPool
from helpers import fill_pool_from_host

pytestmark = pytest.mark.gpu
U32P = C.POINTER(C.c_uint32)


def arr(a):
    a = np.ascontiguousarray(a, np.uint32)
    return a, a.ctypes.data_as(U32P)


def test_demote_promote_round_trip_is_bit_exact_and_pages_move_between_tiers(cuda_device):
    n_layers, n_pages = 3, 40
    pool = KvPool(0, n_layers, 2, 256, n_pages)
    L = _lib.load()
    mine, mp = arr(np.zeros(30))
    assert L.brc_pages_alloc(pool.handle, 30, mp) == 0
    before = []
    for layer in range(n_layers):
        fill_pool_from_host(pool, layer, 900 + 2 * layer)
        before.append((pool.read(0, layer).copy(), pool.read(1, layer).copy()))
    tier = C.c_void_p()
    assert L.brc_tier_create(pool.handle, 16, C.byref(tier)) == 0
    # LRU: touch everything, then re-touch a few; the least recently used come out first
    assert L.brc_tier_touch(tier, mp, 30) == 0
    hot, hp = arr(mine[:20])
    assert L.brc_tier_touch(tier, hp, 20) == 0
    vict, vp = arr(np.zeros(10))
    nv = C.c_uint32()
    assert L.brc_tier_lru(tier, 10, vp, C.byref(nv)) == 0 and nv.value == 10
    assert sorted(vict.tolist()) == sorted(mine[20:].tolist())
    slots, sp = arr(np.zeros(10))
    assert L.brc_tier_demote(tier, vp, 10, sp, None) == 0
    assert pool.free_count() == n_pages - 30 + 10
    assert L.brc_tier_sync(tier) == 0
    # scribble over the freed HBM pages: the host copy must be independent of them
    pool.poison_nan()
    for layer in range(n_layers):
        pool.write(0, layer, before[layer][0])
        pool.write(1, layer, before[layer][1])
        junk = np.full((2, 16, 256), 0xABCD, np.uint16)
        for pg in vict:
            pool.write(0, layer, junk, byte_offset=int(pg) * pool.half_page_bytes)
            pool.write(1, layer, junk, byte_offset=int(pg) * pool.half_page_bytes)
    back, bp = arr(np.zeros(10))
    assert L.brc_tier_promote(tier, sp, 10, bp) == 0
    assert L.brc_tier_fence(tier, None) == 0
    torch.cuda.synchronize()
    for layer in range(n_layers):
        k, v = pool.read(0, layer), pool.read(1, layer)
        for old, new in zip(vict, back):
            assert np.array_equal(k[new], before[layer][0][old]), f"K layer {layer} page {old}->{new}"
            assert np.array_equal(v[new], before[layer][1][old])
    st = [C.c_uint64() for _ in range(4)]
    fs = C.c_uint32()
    assert L.brc_tier_stats(tier, *(C.byref(x) for x in st), C.byref(fs)) == 0
    slot_bytes = 2 * n_layers * pool.half_page_bytes
    assert [x.value for x in st] == [10, 10, 10 * slot_bytes, 10 * slot_bytes] and fs.value == 16
    # refusals: a shared page cannot leave HBM, an empty slot cannot be promoted, the tier can fill up
    pool.retain(mine[:1])
    one, op = arr(mine[:1])
    assert L.brc_tier_demote(tier, op, 1, sp, None) == _lib.ERR_INVALID and b"holders" in L.brc_last_error()
    pool.release_pages(mine[:1])
    assert L.brc_tier_promote(tier, sp, 1, bp) == _lib.ERR_NOT_RESIDENT
    many, manyp = arr(mine[:17])
    big, bigp = arr(np.zeros(17))
    assert L.brc_tier_demote(tier, manyp, 17, bigp, None) == _lib.ERR_CAPACITY
    L.brc_tier_destroy(tier)
    pool.release()


def test_attention_over_promoted_pages_equals_attention_before_demotion(cuda_device):
    """Decode, demote half of a sequence's pages, promote them to other page ids, patch the block
    table, decode again: identical output (the cache content did not change, only its placement)."""
    n_head, n_kv, hd = 16, 2, 256
    lens = np.array([1000])
    n_seq_pages = 63
    pool = KvPool(0, 2, n_kv, hd, 100)
    L = _lib.load()
    table, tp = arr(np.zeros(n_seq_pages))
    assert L.brc_pages_alloc(pool.handle, n_seq_pages, tp) == 0
    for layer in range(2):
        fill_pool_from_host(pool, layer, 950 + 2 * layer)
    q = torch.from_numpy(synth.normal(960, n_head * hd)).cuda().half().view(1, n_head, hd)
    out0 = torch.empty((1, n_head, hd), device="cuda")
    DecodeBatch(pool, n_head, table[None, :], lens).attend(1, q, out0)
    tier = C.c_void_p()
    assert L.brc_tier_create(pool.handle, 40, C.byref(tier)) == 0
    cold, cp = arr(table[::2].copy())
    slots, sp = arr(np.zeros(cold.size))
    assert L.brc_tier_demote(tier, cp, cold.size, sp, C.c_void_p(torch.cuda.current_stream().cuda_stream)) == 0
    filler, fp = arr(np.zeros(5))
    assert L.brc_pages_alloc(pool.handle, 5, fp) == 0      # so the promoted pages land elsewhere
    new, npp = arr(np.zeros(cold.size))
    assert L.brc_tier_promote(tier, sp, cold.size, npp) == 0
    assert L.brc_tier_fence(tier, C.c_void_p(torch.cuda.current_stream().cuda_stream)) == 0
    table2 = table.copy()
    table2[::2] = new
    assert not np.array_equal(table2, table)
    out1 = torch.empty((1, n_head, hd), device="cuda")
    DecodeBatch(pool, n_head, table2[None, :], lens).attend(1, q, out1)
    pool.check()
    assert np.array_equal(out0.cpu().numpy(), out1.cpu().numpy())
    L.brc_tier_destroy(tier)
    pool.release()


def test_back_to_back_batches_in_both_directions_keep_every_byte(cuda_device):
    """Demotions and promotions issued back to back with no host-side wait in between: batches larger
    than one staging pass (256 pages), slots reused as the cursor comes round, pages freed by a demotion
    refilled at once by a promotion, promoted pages demoted again straight away.  Whatever the two copy
    streams overlap, every page must come back with its bytes."""
    n_layers, n_pages, n_move = 2, 700, 300
    pool = KvPool(0, n_layers, 2, 256, n_pages)
    L = _lib.load()
    ids, ip = arr(np.zeros(600))
    assert L.brc_pages_alloc(pool.handle, 600, ip) == 0
    want = []
    for layer in range(n_layers):
        fill_pool_from_host(pool, layer, 950 + layer)
        want.append((pool.read(0, layer).copy(), pool.read(1, layer).copy()))
    tier = C.c_void_p()
    assert L.brc_tier_create(pool.handle, 640, C.byref(tier)) == 0   # 640 slots: the cursor wraps in the third pass
    where = {int(p): int(p) for p in ids}          # original page -> where its bytes are now (HBM page id)
    group_a, group_b = [int(p) for p in ids[:n_move]], [int(p) for p in ids[n_move:2 * n_move]]
    slots_a = None
    for rnd in range(4):
        # A goes out (or comes back) while B does the opposite, without waiting for anything
        if slots_a is None:
            pages, pp = arr([where[p] for p in group_a])
            slots_a, sp = arr(np.zeros(n_move))
            assert L.brc_tier_demote(tier, pp, n_move, sp, None) == 0
            pages_b, pbp = arr([where[p] for p in group_b])
            slots_b, sbp = arr(np.zeros(n_move))
            assert L.brc_tier_demote(tier, pbp, n_move, sbp, None) == 0
            back, bp = arr(np.zeros(n_move))
            assert L.brc_tier_promote(tier, sbp, n_move, bp) == 0       # B straight back in
            for p, new in zip(group_b, back):
                where[p] = int(new)
        else:
            back, bp = arr(np.zeros(n_move))
            _, sp = arr(slots_a)
            assert L.brc_tier_promote(tier, sp, n_move, bp) == 0         # A comes back ...
            for p, new in zip(group_a, back):
                where[p] = int(new)
            pages, pp = arr([where[p] for p in group_a])
            slots_a, sp = arr(np.zeros(n_move))
            assert L.brc_tier_demote(tier, pp, n_move, sp, None) == 0    # ... and leaves again at once
    back, bp = arr(np.zeros(n_move))
    _, sp = arr(slots_a)
    assert L.brc_tier_promote(tier, sp, n_move, bp) == 0
    for p, new in zip(group_a, back):
        where[p] = int(new)
    assert L.brc_tier_sync(tier) == 0
    for layer in range(n_layers):
        k, v = pool.read(0, layer), pool.read(1, layer)
        for p in group_a + group_b:
            assert np.array_equal(k[where[p]], want[layer][0][p]), f"K layer {layer} page {p}"
            assert np.array_equal(v[where[p]], want[layer][1][p]), f"V layer {layer} page {p}"
    L.brc_tier_destroy(tier)
    pool.release()


def test_pages_held_by_a_radix_tree_stay_in_hbm_and_a_bad_batch_queues_nothing(cuda_device):
    """A page whose only holder is the radix tree has one reference, like a page held by one caller: the
    tier must neither offer it for demotion nor accept it (the tree's node would go on naming a freed
    page).  And a batch that names a page twice is refused before any copy is queued: no slot is taken."""
    pool = KvPool(0, 1, 2, 256, 24)
    L = _lib.load()
    mine, mp = arr(np.zeros(8))
    assert L.brc_pages_alloc(pool.handle, 8, mp) == 0
    radix, tier = C.c_void_p(), C.c_void_p()
    assert L.brc_radix_create(pool.handle, C.byref(radix)) == 0
    assert L.brc_tier_create(pool.handle, 8, C.byref(tier)) == 0
    tokens, tp = arr(np.arange(4 * 16) + 11)
    new = C.c_uint32()
    assert L.brc_radix_insert(radix, tp, tokens.size, mp, 4, C.byref(new)) == 0 and new.value == 4
    pool.release_pages(mine[:4])                       # pages 0..3: the tree is their only holder now
    assert all(pool.refcount(int(p)) == 1 for p in mine)
    assert L.brc_tier_touch(tier, mp, 8) == 0
    out, op = arr(np.zeros(8))
    n = C.c_uint32()
    assert L.brc_tier_lru(tier, 8, op, C.byref(n)) == 0
    assert sorted(out[:n.value].tolist()) == sorted(mine[4:].tolist())     # only the caller's own four
    slots, sp = arr(np.zeros(8))
    tree_page, tpp = arr(mine[:1])
    assert L.brc_tier_demote(tier, tpp, 1, sp, None) == _lib.ERR_INVALID and b"radix tree" in L.brc_last_error()
    twice, twp = arr([mine[4], mine[5], mine[4]])
    assert L.brc_tier_demote(tier, twp, 3, sp, None) == _lib.ERR_INVALID and b"twice" in L.brc_last_error()
    st = [C.c_uint64() for _ in range(4)]
    fs = C.c_uint32()
    assert L.brc_tier_stats(tier, *(C.byref(x) for x in st), C.byref(fs)) == 0
    assert fs.value == 8 and st[0].value == 0           # nothing queued, no slot taken
    # the tree's pages still match, and once evicted from the tree they are ordinary pages again
    got, gp = arr(np.zeros(8))
    assert L.brc_radix_match(radix, tp, tokens.size, gp, 8, C.byref(n)) == 0 and n.value == 4
    assert L.brc_radix_release(radix, gp, 4) == 0
    ev = C.c_uint32()
    assert L.brc_radix_evict(radix, 4, C.byref(ev)) == 0 and ev.value == 4
    assert pool.free_count() == 24 - 4
    L.brc_tier_destroy(tier)
    L.brc_radix_destroy(radix)
    pool.release()


def test_pages_spilled_to_a_file_come_back_bit_exact_in_another_store_handle(cuda_device, tmp_path):
    """HBM -> host slot -> file record, the store closed and opened again (as another process would), the records
    found by their tags, -> host slot -> HBM: every byte of every layer as it was.  A store written for another
    page geometry is refused."""
    n_layers, n_pages = 2, 30
    pool = KvPool(0, n_layers, 2, 256, n_pages)
    L = _lib.load()
    mine, mp = arr(np.zeros(12))
    assert L.brc_pages_alloc(pool.handle, 12, mp) == 0
    before = []
    for layer in range(n_layers):
        fill_pool_from_host(pool, layer, 950 + 2 * layer)
        before.append((pool.read(0, layer).copy(), pool.read(1, layer).copy()))
    tier, cold = C.c_void_p(), C.c_void_p()
    assert L.brc_tier_create(pool.handle, 8, C.byref(tier)) == 0
    path = str(tmp_path / "prefix.brccold").encode()
    assert L.brc_cold_open(tier, path, 16, 1, C.byref(cold)) == 0
    vict, vp = arr(mine[2:10])
    slots, sp = arr(np.zeros(8))
    assert L.brc_tier_demote(tier, vp, 8, sp, None) == 0
    tags = np.ascontiguousarray([0xABCD0000 + int(p) * 7919 for p in vict], np.uint64)
    recs, rp = arr(np.zeros(8))
    assert L.brc_cold_spill(cold, sp, tags.ctypes.data_as(C.POINTER(C.c_uint64)), 8, rp) == 0
    st = [C.c_uint64() for _ in range(4)]
    fs = C.c_uint32()
    assert L.brc_tier_stats(tier, *(C.byref(x) for x in st), C.byref(fs)) == 0 and fs.value == 8      # the host slots are free again
    used, total = C.c_uint32(), C.c_uint32()
    assert L.brc_cold_stats(cold, C.byref(used), C.byref(total), None, None) == 0 and (used.value, total.value) == (8, 16)
    assert L.brc_cold_spill(cold, sp, None, 1, rp) == _lib.ERR_NOT_RESIDENT                             # that slot holds nothing now
    assert L.brc_cold_close(cold) == 0
    pool.poison_nan()                                                                                   # HBM forgets everything
    # ---- later: open the same file, find the pages by tag, bring them back
    assert L.brc_cold_open(tier, path, 0, 0, C.byref(cold)) == 0
    found = np.zeros(8, np.uint32)
    one = C.c_uint32()
    for i, tag in enumerate(tags):
        assert L.brc_cold_find(cold, int(tag), C.byref(one)) == 0
        found[i] = one.value
    assert L.brc_cold_find(cold, 12345, C.byref(one)) == _lib.ERR_NOT_RESIDENT
    f, fp = arr(found)
    hs, hp = arr(np.zeros(8))
    assert L.brc_cold_fetch(cold, fp, 8, 1, hp) == 0
    back, bp = arr(np.zeros(8))
    assert L.brc_tier_promote(tier, hp, 8, bp) == 0
    assert L.brc_tier_fence(tier, None) == 0
    torch.cuda.synchronize()
    for layer in range(n_layers):
        k, v = pool.read(0, layer), pool.read(1, layer)
        for old, new in zip(vict, back):
            assert np.array_equal(k[new], before[layer][0][old]) and np.array_equal(v[new], before[layer][1][old]), f"layer {layer} page {old}->{new}"
    assert L.brc_cold_close(cold) == 0
    # ---- a pool of another geometry must not read these records as its own
    other = KvPool(0, 3, 2, 256, 8)
    tier2 = C.c_void_p()
    assert L.brc_tier_create(other.handle, 2, C.byref(tier2)) == 0
    assert L.brc_cold_open(tier2, path, 0, 0, C.byref(cold)) == _lib.ERR_INVALID and b"layers" in L.brc_last_error()
    L.brc_tier_destroy(tier2)
    other.release()
    L.brc_tier_destroy(tier)
    pool.release()


def test_q8_0_v_pool_pages_move_between_the_tiers_and_a_file_byte_for_byte(cuda_device, tmp_path):
    """A pool whose V pages are q8_0 blocks: a host slot holds 16 KiB of K and 9 KiB of V per layer; demote ->
    spill to a file -> fetch -> promote brings back every byte of both, and decode attention over the promoted
    pages equals attention before the demotion bit for bit."""
    n_layers, n_pages, n_kv, hd = 2, 40, 2, 256
    pool = KvPool(0, n_layers, n_kv, hd, n_pages, v_q8=True)
    L = _lib.load()
    mine, mp = arr(np.zeros(20))
    assert L.brc_pages_alloc(pool.handle, 20, mp) == 0
    rng = np.random.default_rng(77)
    before = []
    for layer in range(n_layers):
        k = oracle.f32_to_f16_bits_np(synth.normal(960 + layer, n_pages * n_kv * 16 * hd, 0.5))
        rows = n_pages * n_kv * 16
        v = np.zeros((rows, hd // 32, 36), np.uint8)          # [row][block]: f32 scale then 32 quanta
        v[:, :, :4] = rng.uniform(0.001, 0.05, (rows, hd // 32)).astype(np.float32).view(np.uint8).reshape(rows, hd // 32, 4)
        v[:, :, 4:] = rng.integers(-127, 128, (rows, hd // 32, 32), dtype=np.int8).view(np.uint8)
        pool.write(0, layer, k)
        pool.write(1, layer, v)
        before.append((pool.read(0, layer).copy(), pool.read(1, layer).copy()))
    v_page = n_kv * 16 * (hd // 32 * 36)                      # bytes of the V half of a page
    # attention over a sequence that lives in pages mine[4:12], before anything moves
    lens = np.array([8 * 16 - 5])
    tables = mine[4:12][None, :].astype(np.uint32)
    q = torch.randn((1, 16, hd), device="cuda").half()
    out0 = torch.full((1, 16, hd), float("nan"), device="cuda")
    DecodeBatch(pool, 16, tables, lens).attend(1, q, out0)
    pool.check()
    tier, cold = C.c_void_p(), C.c_void_p()
    assert L.brc_tier_create(pool.handle, 8, C.byref(tier)) == 0
    assert L.brc_cold_open(tier, str(tmp_path / "q8.brccold").encode(), 8, 1, C.byref(cold)) == 0
    vict, vp = arr(mine[4:12])
    slots, sp = arr(np.zeros(8))
    assert L.brc_tier_demote(tier, vp, 8, sp, None) == 0
    st = [C.c_uint64() for _ in range(4)]
    fs = C.c_uint32()
    assert L.brc_tier_stats(tier, *(C.byref(x) for x in st), C.byref(fs)) == 0
    slot_bytes = n_layers * (pool.half_page_bytes + v_page)
    assert st[2].value == 8 * slot_bytes and v_page * 16 == pool.half_page_bytes * 9
    recs, rp = arr(np.zeros(8))
    assert L.brc_cold_spill(cold, sp, None, 8, rp) == 0
    pool.poison_nan()
    for layer in range(n_layers):                             # the pages that stayed keep their bytes
        pool.write(0, layer, before[layer][0])
        pool.write(1, layer, before[layer][1])
        for pg in vict:
            pool.write(0, layer, np.full(pool.half_page_bytes // 2, 0xABCD, np.uint16), byte_offset=int(pg) * pool.half_page_bytes)
            pool.write(1, layer, np.full(v_page, 0xEE, np.uint8), byte_offset=int(pg) * v_page)
    hs, hp = arr(np.zeros(8))
    assert L.brc_cold_fetch(cold, rp, 8, 0, hp) == 0
    back, bp = arr(np.zeros(8))
    assert L.brc_tier_promote(tier, hp, 8, bp) == 0
    assert L.brc_tier_fence(tier, None) == 0
    torch.cuda.synchronize()
    rows_per_page = n_kv * 16
    for layer in range(n_layers):
        k, v = pool.read(0, layer), pool.read(1, layer)
        for old, new in zip(vict, back):
            assert np.array_equal(k[new], before[layer][0][old]), f"K layer {layer} page {old}->{new}"
            assert np.array_equal(v[new * rows_per_page:(new + 1) * rows_per_page], before[layer][1][old * rows_per_page:(old + 1) * rows_per_page])
    out1 = torch.full_like(out0, float("nan"))
    DecodeBatch(pool, 16, back[None, :].astype(np.uint32), lens).attend(1, q, out1)
    pool.check()
    assert torch.equal(out0, out1)
    assert L.brc_cold_close(cold) == 0
    L.brc_tier_destroy(tier)
    pool.release()


def test_a_prompt_prefix_persisted_to_a_file_is_found_again_by_its_tokens(cuda_device, tmp_path):
    """The disk-persisted prefix cache end to end: a first "process" fills the pages of a 5-page prompt prefix,
    demotes them and spills them to a cold store under brc_radix_prefix_tags; a second one (fresh pool, tier, tree
    and store handle) computes the tags of ITS prompt (the same first four pages, then different tokens), finds
    four records, fetches and promotes them, adopts them into its prefix tree - and attention over the restored
    prefix equals attention over the original pages bit for bit."""
    n_layers, n_kv, hd = 2, 2, 256
    L = _lib.load()
    path = str(tmp_path / "prefix.brccold").encode()
    prompt_a = (np.arange(5 * 16) * 7 + 3).astype(np.uint32)
    prompt_b = prompt_a.copy()
    prompt_b[4 * 16 + 5] += 1                                    # the fifth page differs
    q = torch.randn((1, 16, hd), generator=torch.Generator().manual_seed(5)).cuda().half()

    def tags_of(prompt):
        tags = np.zeros(8, np.uint64)
        n = C.c_uint32()
        assert L.brc_radix_prefix_tags(prompt.ctypes.data_as(C.POINTER(C.c_uint32)), prompt.size, 16, tags.ctypes.data_as(C.POINTER(C.c_uint64)),
                                       8, C.byref(n)) == 0
        return tags[:n.value]

    ta, tb = tags_of(prompt_a), tags_of(prompt_b)
    assert ta.size == 5 and np.array_equal(ta[:4], tb[:4]) and ta[4] != tb[4] and (ta != 0).all() and len(set(ta.tolist())) == 5
    assert np.array_equal(tags_of(prompt_a[:40]), ta[:2])        # a partial page has no tag

    # ---- first process: compute (here: fill) the prefix, attend, persist
    pool = KvPool(0, n_layers, n_kv, hd, 16)
    pages, pp = arr(np.zeros(5))
    assert L.brc_pages_alloc(pool.handle, 5, pp) == 0
    for layer in range(n_layers):
        fill_pool_from_host(pool, layer, 700 + layer)
    out_a = torch.full((1, 16, hd), float("nan"), device="cuda")
    DecodeBatch(pool, 16, pages[None, :4].astype(np.uint32), np.array([64])).attend(1, q, out_a)
    pool.check()
    tier, cold = C.c_void_p(), C.c_void_p()
    assert L.brc_tier_create(pool.handle, 8, C.byref(tier)) == 0
    assert L.brc_cold_open(tier, path, 8, 1, C.byref(cold)) == 0
    slots, sp = arr(np.zeros(5))
    assert L.brc_tier_demote(tier, pp, 5, sp, None) == 0
    recs, rp = arr(np.zeros(5))
    assert L.brc_cold_spill(cold, sp, ta.ctypes.data_as(C.POINTER(C.c_uint64)), 5, rp) == 0
    assert L.brc_cold_close(cold) == 0
    L.brc_tier_destroy(tier)
    pool.release()

    # ---- second process: another pool (other page ids), the store found on disk
    pool = KvPool(0, n_layers, n_kv, hd, 24)
    pool.poison_nan()
    taken = pool.alloc(7)                                         # so that the restored pages get other ids
    tier, cold, radix = C.c_void_p(), C.c_void_p(), C.c_void_p()
    assert L.brc_tier_create(pool.handle, 8, C.byref(tier)) == 0
    assert L.brc_cold_open(tier, path, 0, 0, C.byref(cold)) == 0
    assert L.brc_radix_create(pool.handle, C.byref(radix)) == 0
    found = []
    one = C.c_uint32()
    for tag in tb:                                                # the longest run of prefix pages the store holds
        if L.brc_cold_find(cold, int(tag), C.byref(one)) != 0:
            break
        found.append(one.value)
    assert len(found) == 4
    f, fp = arr(found)
    hs, hp = arr(np.zeros(4))
    assert L.brc_cold_fetch(cold, fp, 4, 1, hp) == 0
    back, bp = arr(np.zeros(4))
    assert L.brc_tier_promote(tier, hp, 4, bp) == 0
    assert L.brc_tier_fence(tier, None) == 0
    new = C.c_uint32()
    assert L.brc_radix_insert(radix, prompt_b.ctypes.data_as(C.POINTER(C.c_uint32)), 64, bp, 4, C.byref(new)) == 0 and new.value == 4
    got, gp = arr(np.zeros(8))
    n = C.c_uint32()
    assert L.brc_radix_match(radix, prompt_b.ctypes.data_as(C.POINTER(C.c_uint32)), prompt_b.size, gp, 8, C.byref(n)) == 0 and n.value == 4
    assert got[:4].tolist() == back.tolist() and not set(back.tolist()) & set(taken.tolist())
    out_b = torch.full((1, 16, hd), float("nan"), device="cuda")
    DecodeBatch(pool, 16, got[None, :4].astype(np.uint32), np.array([64])).attend(1, q, out_b)
    pool.check()
    assert torch.equal(out_a, out_b)
    assert L.brc_radix_release(radix, gp, 4) == 0
    assert L.brc_cold_close(cold) == 0
    L.brc_radix_destroy(radix)
    L.brc_tier_destroy(tier)
    pool.release()
