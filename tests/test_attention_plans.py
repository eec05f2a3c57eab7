"""CPU tests of the attention kernels' work distribution (prefill first, decode at the end). vkc_attn_prefill_plan,
vkc_attn_prefill_items and vkc_attn_decode_items run, on the host, the arithmetic the launchers and the kernels use to decide
which CTA computes which key tiles of which query tiles. The tests walk every CTA of a plan and check that the items cover
every (batch, head, query tile, key tile) exactly once, that partial results land where the merge kernels look for them, and
that every CTA's list ends with its `last` mark."""
import random

import pytest

from vknn_b200 import capi

SMS = 148  # B200


def tile_steps(Sq, Skv, causal, first):
    """Key tiles of 128 keys that the 128-row query tile starting at row `first` needs (a restatement for the check: rows
    past Sq need nothing; with a causal mask row i sees keys j <= i + (Skv - Sq))."""
    if first >= Sq:
        return 0
    kend = Skv
    if causal:
        last = min(first + 127, Sq - 1)
        kend = max(0, min(kend, last + (Skv - Sq) + 1))
    return (kend + 127) // 128


def walk(sm, B, Hq, Sq, Skv, D, causal, has_kv_len=False):
    plan = capi.attn_prefill_plan(sm, B, Hq, Sq, Skv, D, causal, has_kv_len)
    items = [capi.attn_prefill_items(sm, B, Hq, Sq, Skv, D, c, causal, has_kv_len) for c in range(plan["ctas"])]
    return plan, items


def check(sm, B, Hq, Sq, Skv, D, causal, has_kv_len=False):
    plan, per_cta = walk(sm, B, Hq, Sq, Skv, D, causal, has_kv_len)
    qt = plan["query_tiles"]
    nq = (Sq + qt * 128 - 1) // (qt * 128)
    where = "sm=%d B=%d Hq=%d Sq=%d Skv=%d D=%d causal=%d plan=%s" % (sm, B, Hq, Sq, Skv, D, causal, plan)
    assert qt in (1, 2) and (qt == 2 or D == 64), where
    if plan["form"] == 0:
        assert plan["ctas"] == nq * Hq * B, where
    else:
        assert not has_kv_len, where
        assert plan["ctas"] <= sm * (2 if qt == 1 else 1), where  # every persistent CTA is resident at once
    # 1. every key tile of every query tile exactly once
    seen = {}
    slots_used = set()
    for c, items in enumerate(per_cta):
        assert plan["form"] == 0 or items or plan["rounds"] == 0, where
        for i, it in enumerate(items):
            assert it["last"] == (1 if i == len(items) - 1 else 0), (where, c, i, it)
            assert 0 <= it["b"] < B and 0 <= it["h"] < Hq and 0 <= it["qg"] < nq, (where, it)
            assert it["slot"] in (-1, 0, 1), (where, it)
            if it["slot"] >= 0:
                assert (c, it["slot"]) not in slots_used, (where, c, it)  # one partial per slot of a CTA
                slots_used.add((c, it["slot"]))
            for t in range(qt):
                key = (it["b"], it["h"], it["qg"] * qt + t)
                n = it["n_t0"] if t == 0 else it["n_t1"]
                cover = seen.setdefault(key, [])
                cover.append((it["j0"], it["j0"] + n, c, it["slot"]))
    for b in range(B):
        for h in range(Hq):
            for tile in range(nq * qt):
                need = tile_steps(Sq, Skv, causal, tile * 128)
                got = sorted(r for r in seen.get((b, h, tile), []) if r[1] > r[0])
                pos = 0
                for lo, hi, _, _ in got:
                    assert lo == pos, (where, (b, h, tile), got)
                    pos = hi
                assert pos == need, (where, (b, h, tile), got, need)
    if plan["form"] == 0:
        assert all(len(items) == 1 and items[0]["slot"] == -1 for items in per_cta), where
        return plan
    # 2. the pieces of a cut unit are where the merge kernel reads them: the unit occupies steps [s0, s1] of the line of
    # left-over blocks, CTA cc owns [cc * quota, (cc + 1) * quota), and holds the partial in slot 0 unless the unit begins
    # inside its stretch (slot 1); a unit inside one CTA's stretch is written whole (slot -1)
    pairing = bool(causal)
    nb = nq // 2 if pairing else nq
    quota, ustride = plan["quota"], plan["pieces"] * plan["quota"]
    by_unit = {}
    for c, items in enumerate(per_cta):
        for it in items:
            by_unit.setdefault((it["b"], it["h"], it["qg"]), []).append((c, it))
    for br in range(plan["left"]):
        blk = plan["rounds"] * plan["ctas"] + br
        bh, k2 = divmod(blk, nb)
        b, h = divmod(bh, Hq)
        units = [(k2, plan["steps"], 0)]
        if pairing:
            n_hi = max(tile_steps(Sq, Skv, True, ((nq - 1 - k2) * qt + t) * 128) for t in range(qt))
            units = [(nq - 1 - k2, n_hi, 0), (k2, plan["steps"] - n_hi, n_hi)]
        for qg, nu, uoff in units:
            if nu <= 0:
                continue
            s0 = br * ustride + uoff
            s1 = s0 + nu - 1
            ca, cb = s0 // quota, s1 // quota
            holders = sorted((c, it["slot"], it["j0"]) for c, it in by_unit[(b, h, qg)])
            if ca == cb:
                assert [(c, s) for c, s, _ in holders] == [(ca, -1)], (where, (b, h, qg), holders)
            else:
                want = [(cc, 0 if s0 < cc * quota else 1) for cc in range(ca, cb + 1)]
                assert [(c, s) for c, s, _ in holders] == want, (where, (b, h, qg), holders, want)
                assert [j for _, _, j in holders] == sorted(j for _, _, j in holders), where
    # whole blocks of the round-robin part never leave partials unless a causal pair is split at the pair's seam (it is not)
    for c, items in enumerate(per_cta):
        n_whole = sum(1 for it in items if it["slot"] == -1)
        assert n_whole >= plan["rounds"] * (2 if pairing else 1), (where, c)
    return plan


def test_forms_on_the_bench_shapes():
    # (B, Hq, Sq, Skv, D, causal) -> form, query tiles per CTA, CTAs
    assert check(SMS, 8, 32, 2048, 2048, 128, False)["form"] == 1  # 2048 units on 148 SMs: 13 rounds and a cut remainder
    p = check(SMS, 1, 12, 197, 197, 64, False)                     # a ViT-B layer: 24 one-tile units
    assert p["query_tiles"] == 1
    p = check(SMS, 32, 12, 197, 197, 64, False)                    # batch 32: 384 two-tile units, two rounds and 88 more
    assert (p["form"], p["query_tiles"], p["rounds"], p["left"], p["pieces"]) == (1, 2, 2, 88, 1)
    p = check(SMS, 1, 16, 2738, 2738, 64, False)                   # 176 units: one round, the other 28 cut five ways
    assert (p["form"], p["rounds"], p["left"], p["pieces"], p["quota"]) == (1, 1, 28, 5, 5)
    p = check(SMS, 1, 32, 8192, 8192, 128, True)
    assert p["form"] == 1 and p["rounds"] >= 2                     # causal pairs, several rounds deep
    p = check(SMS, 1, 32, 1024, 1024, 128, True)
    assert p["form"] == 0                                          # too few pairs to fill the SMs twice
    p = check(SMS, 4, 8, 512, 512, 128, False, has_kv_len=True)
    assert p["form"] == 0                                          # per-sequence lengths: one CTA per unit


@pytest.mark.parametrize("causal", [False, True])
def test_every_key_tile_once_random_shapes(causal):
    rng = random.Random(20 + causal)
    for _ in range(120):
        D = rng.choice((64, 128))
        B, Hq = rng.randint(1, 6), rng.choice((1, 2, 3, 5, 8, 12, 16, 20, 37))
        Sq = rng.choice((1, 64, 128, 197, 256, 300, 512, 777, 1024, 1536, 2048, 2738, 4096))
        Skv = Sq if causal and rng.random() < 0.8 else rng.choice((1, 100, 128, 197, 512, 1000, 2048, 4096, 5000))
        if causal and Skv < Sq:
            Skv = Sq
        check(SMS, B, Hq, Sq, Skv, D, causal)


def test_other_sm_counts_and_many_rounds():
    for sm in (1, 2, 7, 16, 132):
        check(sm, 2, 12, 1024, 1024, 64, False)
        check(sm, 2, 6, 2048, 2048, 128, True)
    check(SMS, 16, 64, 512, 512, 128, False)
    check(SMS, 5, 64, 512, 512, 128, True)
    check(SMS, 3, 40, 2048, 2048, 64, True)
    check(SMS, 7, 16, 1536, 1536, 128, True)


def test_causal_pairs_of_query_groups():
    """Shapes deep enough for the persistent causal form: blocks are pairs of query groups (nq-1-k, k)."""
    rng, paired = random.Random(7), 0
    for _ in range(40):
        S = 256 * rng.choice((2, 3, 4, 6, 8, 12, 16, 32))
        nq = S // 256
        bh = max(1, (rng.randint(2, 9) * SMS + rng.randint(0, SMS)) // (nq // 2))
        Hq = rng.choice((1, 2, 4, 8, 16, 32))
        B = max(1, bh // Hq)
        if B * Hq * nq * (S // 128) > 3_000_000:
            continue
        p = check(SMS, B, Hq, S, S, 128, True)
        paired += p["form"]
        if p["form"] == 1:
            assert p["steps"] == S // 128 + 2 and p["rounds"] >= 2, p  # a pair of groups: (S/128) + 2 key tiles, whatever k
    assert paired >= 10


def test_bad_arguments_are_refused():
    lib = capi.load_library()
    import ctypes as C
    out = (C.c_int32 * 8)()
    assert lib.vkc_attn_prefill_plan(0, 1, 1, 128, 128, 64, 0, 0, out) == -1
    assert lib.vkc_attn_prefill_plan(148, 1, 1, 128, 128, 96, 0, 0, out) == -1
    assert lib.vkc_attn_prefill_plan(148, 1, 1, 128, 128, 64, 0, 0, None) == -1
    assert lib.vkc_attn_prefill_items(148, 1, 1, 128, 128, 64, 0, 0, 5, out, 1) == -1  # the plan has one CTA
    assert lib.vkc_attn_prefill_items(148, 1, 1, 128, 128, 64, 0, 0, 0, None, 0) == 1  # count only


# ---- decode: equal runs of key tiles over the CTAs -------------------------------------------------------------------
def check_decode(B, Hq, Hkv, Lmax, lens):
    plan, per_cta = capi.attn_decode_items(SMS, B, Hq, Hkv, Lmax, 128, lens)
    where = "B=%d Hq=%d Hkv=%d Lmax=%d plan=%s" % (B, Hq, Hkv, Lmax, plan)
    assert 1 <= plan["grid"] <= SMS and len(per_cta) == plan["grid"], where
    eff = [min(max(l, 0), Lmax) for l in (lens if lens is not None else [Lmax] * B)]
    total_tiles = sum((l + 127) // 128 for l in eff) * Hkv
    quota = max(plan["min_tiles"], (total_tiles + plan["grid"] - 1) // plan["grid"])
    pieces = {}
    for c, items in enumerate(per_cta):
        tiles = 0
        for it in items:
            assert 0 <= it["b"] < B and 0 <= it["hk"] < Hkv and it["start"] % 128 == 0 and it["start"] < it["end"] <= eff[it["b"]], (where, c, it)
            assert 0 <= 2 * it["pair"] + 1 < plan["slots"], (where, c, it)  # the partials stay inside the workspace
            tiles += (it["end"] - it["start"] + 127) // 128
            pieces.setdefault((it["b"], it["hk"]), []).append(it)
        assert tiles <= quota, (where, c)  # equal runs: no CTA streams more than its share
    for b in range(B):
        for hk in range(Hkv):
            got = sorted(pieces.get((b, hk), []), key=lambda it: it["start"])
            if eff[b] == 0:
                assert not got, where  # an empty sequence has no item (the merge kernel writes its NaN rows)
                continue
            pos = 0
            for i, it in enumerate(got):
                assert it["start"] == pos and it["pair"] == i, (where, (b, hk), got)  # contiguous keys, slot pairs 0, 1, 2, ...
                assert it["last"] == (1 if i == len(got) - 1 else 0), (where, (b, hk), got)
                pos = it["end"]
            assert pos == eff[b], (where, (b, hk), got)
    return plan


def test_decode_every_key_once_and_slots_in_bounds():
    rng = random.Random(3)
    plan = check_decode(32, 32, 8, 8192, [rng.randint(1024, 8192) for _ in range(32)])  # the bench's decode configuration
    assert plan["grid"] == SMS
    check_decode(32, 32, 8, 8192, None)
    for _ in range(150):
        Hkv = rng.choice((1, 2, 4, 8))
        Hq = Hkv * rng.choice((1, 2, 4, 8, 16))
        B = rng.choice((1, 2, 3, 8, 17, 32, 64, 200))
        Lmax = rng.choice((1, 100, 128, 129, 1000, 4096, 8192, 20000, 65536))
        kind = rng.random()
        if kind < 0.15:
            lens = None
        elif kind < 0.3:
            lens = [rng.choice((0, 1, Lmax, Lmax + 5, -3)) for _ in range(B)]  # empty, over-long and negative lengths are clamped
        elif kind < 0.45:
            lens = [Lmax if i == 0 else rng.randint(0, 3) for i in range(B)]   # one long sequence among nearly empty ones
        else:
            lens = [rng.randint(0, Lmax) for _ in range(B)]
        check_decode(B, Hq, Hkv, Lmax, lens)


def test_decode_items_refuses_what_the_kernel_does_not_take():
    with pytest.raises(capi.VkcError):
        capi.attn_decode_items(SMS, 4, 8, 8, 1024, 64)      # head size 64: the SIMT form's
    with pytest.raises(capi.VkcError):
        capi.attn_decode_items(SMS, 4, 64, 2, 1024, 128)    # 32 query heads per kv head
    with pytest.raises(capi.VkcError):
        capi.attn_decode_items(SMS, 4, 8, 3, 1024, 128)     # Hq not a multiple of Hkv
