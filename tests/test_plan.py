"""Planner (metadata stage) invariants, checked on the host through dsa_v32_plan_host: every slot of
every (query row, head block) is covered exactly once, split units own distinct partial slots that
the reduce tables list, and the work is balanced across the CTA pairs."""
import ctypes as C
import struct

import numpy as np
import pytest

from opfoundry_b200 import api

HDR = struct.Struct("<I" + "i" * 11 + "q" * 8)
TILE = 32


def parse(blob):
    f = HDR.unpack_from(blob, 0)
    h = dict(zip(["magic", "total_q", "H", "topk", "s_q", "num_lists", "num_works", "num_partials", "num_reduce_rows",
                  "num_head_blocks", "status", "_pad", "off_list_indptr", "off_works", "off_reduce_indptr",
                  "off_reduce_slots", "off_reduce_dst", "off_o_accum", "off_lse_accum", "total_bytes"], f))
    indptr = np.frombuffer(blob, np.int32, h["num_lists"] + 1, h["off_list_indptr"])
    works = np.frombuffer(blob, np.int32, h["num_works"] * 8, h["off_works"]).reshape(-1, 8)
    r_indptr = np.frombuffer(blob, np.int32, h["num_reduce_rows"] + 1, h["off_reduce_indptr"])
    r_slots = np.frombuffer(blob, np.int32, int(r_indptr[-1]), h["off_reduce_slots"])
    r_dst = np.frombuffer(blob, np.int32, h["num_reduce_rows"] * 2, h["off_reduce_dst"]).reshape(-1, 2)
    return h, indptr, works, r_indptr, r_slots, r_dst


def check_plan(total_q, H, topk, s_q=1, num_sms=148, hint=None, auto_split=False):
    built = pytest.importorskip("opfoundry_b200.build")
    built.build()
    blob = api.plan_host(total_q, H, topk, s_q, num_sms=num_sms, valid_len_hint=hint, auto_split=auto_split)
    h, indptr, works, r_indptr, r_slots, r_dst = parse(blob)
    assert h["magic"] == 0x44534133 and h["num_lists"] == num_sms // 2
    assert indptr[0] == 0 and indptr[-1] == h["num_works"] and np.all(np.diff(indptr) >= 0)
    n_hb = (H + 127) // 128
    cover = {}
    for w in works:
        q, slot, kb, ke, hb, rr = (int(x) for x in w[:6])
        assert 0 <= q < total_q and 0 <= hb < n_hb and 0 <= kb < ke <= topk
        assert kb % TILE == 0
        cover.setdefault((q, hb), []).append((kb, ke, slot, rr))
    assert len(cover) == total_q * n_hb
    seen_slots = set()
    for (q, hb), pieces in cover.items():
        pieces.sort()
        want_len = topk if hint is None else max(1, min(topk, int(hint[q])))
        assert pieces[0][0] == 0 and pieces[-1][1] == want_len
        for a, b in zip(pieces, pieces[1:]):
            assert a[1] == b[0]
        if len(pieces) == 1:
            assert pieces[0][2] == -1 and pieces[0][3] == -1
        else:
            rr = pieces[0][3]
            assert all(p[3] == rr for p in pieces) and tuple(r_dst[rr]) == (q, hb)
            slots = [p[2] for p in pieces]
            assert all(s >= 0 for s in slots) and not (set(slots) & seen_slots)
            seen_slots |= set(slots)
            assert sorted(r_slots[r_indptr[rr]:r_indptr[rr + 1]].tolist()) == sorted(slots)
    assert len(seen_slots) == h["num_partials"]
    assert h["total_bytes"] >= h["off_lse_accum"] + h["num_partials"] * 128 * 4
    # balance: cost of a list in tile steps
    cost = [sum((int(w[3]) - int(w[2]) + TILE - 1) // TILE for w in works[indptr[i]:indptr[i + 1]])
            for i in range(h["num_lists"])]
    return h, cost


def test_decode_config2_shape():
    # 64 units on 74 lists: whole units (one list each, ten lists idle) are within the merge cost of the
    # balanced plan, so the planner does not split at all - no partial results, no merge
    h, cost = check_plan(64, 128, 2048)
    used = [c for c in cost if c > 0]
    assert h["num_partials"] == 0 and len(used) == 64 and max(used) == min(used)


def test_decode_split_when_it_pays():
    # 16 units on 74 lists: whole units would leave 58 lists idle, so they are cut and merged
    h, cost = check_plan(16, 128, 2048)
    assert h["num_partials"] > 16
    assert max(cost) <= 1.25 * (sum(cost) / len(cost)) + 8
    assert min(cost) > 0


def test_decode_small_batches_and_heads():
    for (tq, H, topk, sq) in [(1, 16, 2048, 1), (2, 16, 2048, 1), (4, 128, 100, 1), (256, 128, 2048, 2), (3, 200, 65, 1),
                              (7, 128, 1, 1), (148, 128, 33, 1), (1, 128, 31, 1)]:
        check_plan(tq, H, topk, sq)


def test_prefill_with_valid_len_hint():
    T, topk = 600, 256
    hint = np.minimum(np.arange(T) + 1, topk).astype(np.int32)
    h, cost = check_plan(T, 128, topk, s_q=T, hint=hint)
    assert max(cost) <= 1.3 * (sum(cost) / len(cost)) + 8


def test_other_sm_counts():
    for sms in (2, 8, 132, 160):
        check_plan(16, 128, 512, num_sms=sms)


def test_bad_shapes_rejected():
    for args in [(0, 128, 64, 1), (4, 0, 64, 1), (4, 128, 0, 1), (5, 128, 64, 2)]:
        with pytest.raises(api.DsaError) as e:
            api.plan_host(*args)
        assert e.value.status == -2


def _used_lists(blob):
    h, indptr, *_ = parse(blob)
    return int((np.diff(indptr) > 0).sum())


def test_varlen_and_auto_split_cover_exactly():
    """Scheduler parity with the reference's metadata kernel in the sense that matters (integer-exact
    coverage, not identical cuts): variable per-sequence lengths as its --varlen harness draws them
    (common/host.cc:239-261: uniform in [min(5, s), s]) and its auto_split option
    (common/get_mla_metadata.hpp:8-13) both leave every slot covered exactly once."""
    rng = np.random.RandomState(1234)
    for (B, s_q, topk, s) in [(3, 1, 2048, 4096), (16, 2, 2048, 1500), (64, 1, 512, 300), (5, 2, 96, 40)]:
        lens = rng.randint(min(5, s), s + 1, size=B)
        hint = np.repeat(np.minimum(lens, topk), s_q).astype(np.int32)
        check_plan(B * s_q, 128, topk, s_q, hint=hint)
        check_plan(B * s_q, 128, topk, s_q, hint=hint, auto_split=True)
        check_plan(B * s_q, 16, topk, s_q, num_sms=20, hint=hint, auto_split=True)


def test_auto_split_limits_the_lists_of_a_small_problem():
    """effective lists = min(lists, round(1.2 * sqrt(cost * lists))), cost in tile steps + per-unit overhead."""
    # 2 queries of 8 tiles each: cost = 16 + 2 * 6 = 28 steps, 74 lists -> round(1.2 * sqrt(28 * 74)) = 55 > 16 / 4 = 4 pieces
    assert _used_lists(api.plan_host(2, 128, 256, 1, auto_split=True)) <= 4
    # one query of 64 tiles: without the option it is cut into 16 pieces; with it into at most round(1.2 * sqrt(70 * 4)) = 20 -> unchanged,
    # and on a 4-list device round(1.2 * sqrt(70 * 2)) = 14 -> at most 2
    a = _used_lists(api.plan_host(1, 128, 2048, 1, num_sms=148))
    b = _used_lists(api.plan_host(1, 128, 2048, 1, num_sms=148, auto_split=True))
    assert b <= a
    # a tiny problem on many lists: one tile step of work -> one list
    assert _used_lists(api.plan_host(1, 16, 32, 1, auto_split=True)) == 1
    import math
    for (q, topk) in [(1, 64), (2, 128), (4, 2048)]:
        tiles = q * ((topk + 31) // 32)
        eff = max(1, min(74, int(round(1.2 * math.sqrt((tiles + q * 6) * 74)))))
        assert _used_lists(api.plan_host(q, 128, topk, 1, auto_split=True)) <= eff


def test_mtp_rows_that_share_a_list_are_planned_as_one_stacked_item():
    """With s_q * H <= 128 the query rows of a sequence flagged as sharing one index list become one
    work item (stacked_rows = s_q, gathered once); other sequences keep one item per row; every slot
    of every query row is still covered exactly once."""
    B, s_q, H, topk = 12, 2, 64, 512
    shared = [b % 3 != 0 for b in range(B)]
    for num_sms in (148, 8):
        blob = api.plan_host(B * s_q, H, topk, s_q, num_sms=num_sms, mtp_shared=shared)
        h, indptr, works, r_indptr, r_slots, r_dst = parse(blob)
        cover = {}
        for w in works:
            q, slot, kb, ke, hb, rr, stacked = (int(x) for x in w[:7])
            rows = stacked if stacked > 1 else 1
            assert (stacked == s_q) == shared[q // s_q] and hb == 0
            if stacked > 1:
                assert q % s_q == 0
            for t in range(rows):
                cover.setdefault(q + t, []).append((kb, ke))
            if rr >= 0:
                assert int(r_dst[rr][0]) == q and int(r_dst[rr][1]) == (-stacked if stacked > 1 else 0)
        assert sorted(cover) == list(range(B * s_q))
        for q, pieces in cover.items():
            pieces.sort()
            assert pieces[0][0] == 0 and pieces[-1][1] == topk and all(a[1] == b[0] for a, b in zip(pieces, pieces[1:]))
    # stacking needs s_q * H <= 128: at H = 128 the flags change nothing
    a = api.plan_host(B * s_q, 128, topk, s_q, mtp_shared=shared)
    b = api.plan_host(B * s_q, 128, topk, s_q)
    assert a == b
