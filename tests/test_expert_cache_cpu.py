"""Expert-bundle cache bookkeeping against the reference's own unit tests
(crates/rnb-memory/src/sparse_expert_cache.rs `mod tests`, :531-993, and byte_lru.rs), restated
through the C ABI.  Host accounting only: no GPU."""
import ctypes as C

import pytest


@pytest.fixture(scope="module")
def ec():
    from runnburn_b200 import build
    build.build_library()
    from runnburn_b200 import expert_cache
    expert_cache._L()
    return expert_cache


U64_MAX = (1 << 64) - 1


def test_classifies_and_records_one_bundle_outcome_per_lookup(ec):
    assert ec.evaluate_bundle(1, 1, 1, (True, True, True))["residency"] == "full"
    assert ec.evaluate_bundle(1, 1, 1, (False, False, False))["residency"] == "miss"
    for roles in [(True, False, False), (False, True, False), (False, False, True), (True, True, False), (True, False, True), (False, True, True)]:
        assert ec.evaluate_bundle(1, 1, 1, roles)["residency"] == "partial"
    s = ec.BundleStats()
    L = ec._L()
    L.rnb_b200_expert_stats_record_lookup(C.byref(s), 1, 1, 1)
    L.rnb_b200_expert_stats_record_lookup(C.byref(s), 1, 0, 1)
    L.rnb_b200_expert_stats_record_lookup(C.byref(s), 0, 0, 0)
    d = s.as_dict()
    assert (d["bundle_lookups"], d["bundle_hits"], d["bundle_partial_hits"], d["bundle_misses"]) == (3, 1, 1, 1)


def test_bundle_stats_delta_saturates_every_field(ec):
    before = ec.BundleStats(1, 2, 3, 4, 5, 6, 8, 9, 10, 11)
    after = ec.BundleStats(11, 1, 13, 2, 15, 3, 4, 19, 5, 21)
    out = ec.BundleStats()
    ec._L().rnb_b200_expert_stats_delta(C.byref(after), C.byref(before), C.byref(out))
    assert list(out.as_dict().values()) == [10, 0, 10, 0, 10, 0, 0, 10, 0, 10]


def test_observation_receipt_accumulates_and_clears_without_reopening(ec):
    L = ec._L()
    r = ec.BundleReceipt()
    assert r.consumed == 0 and all(v == 0 for v in r.pending_stats.as_dict().values())
    a = ec.BundleStats(bundle_lookups=1, bundle_partial_hits=1, h2d_bytes=U64_MAX)
    b = ec.BundleStats(bundle_lookups=2, bundle_admissions=1, h2d_bytes=1)
    L.rnb_b200_expert_receipt_record(C.byref(r), C.byref(a))
    L.rnb_b200_expert_receipt_record(C.byref(r), C.byref(b))
    L.rnb_b200_expert_receipt_mark_consumed(C.byref(r))
    d = r.pending_stats.as_dict()
    assert r.consumed == 1 and d["bundle_lookups"] == 3 and d["bundle_partial_hits"] == 1 and d["bundle_admissions"] == 1 and d["h2d_bytes"] == U64_MAX
    L.rnb_b200_expert_receipt_clear_stats(C.byref(r))
    assert r.consumed == 1 and all(v == 0 for v in r.pending_stats.as_dict().values())


def test_cold_seen_once_and_reused_follow_current_transfer_break_even(ec):
    h = ec.ReuseHistory(4)
    cold = ec.evaluate_bundle(20, 30, 50, predicted_future_reuses=h.observe(3, 7))
    assert (cold["predicted_future_reuses"], cold["predicted_saved_bytes"], cold["net_saved_bytes"], cold["admit"]) == (0, 100, 0, False)
    once = ec.evaluate_bundle(20, 30, 50, predicted_future_reuses=h.observe(3, 7))
    assert (once["predicted_future_reuses"], once["predicted_saved_bytes"], once["net_saved_bytes"], once["admit"]) == (1, 200, 100, True)
    again = ec.evaluate_bundle(20, 30, 50, predicted_future_reuses=h.observe(3, 7))
    assert (again["predicted_future_reuses"], again["predicted_saved_bytes"], again["net_saved_bytes"], again["admit"]) == (2, 300, 200, True)


def test_no_current_upload_requires_more_than_one_future_reuse(ec):
    first = ec.evaluate_bundle(20, 30, 50, predicted_future_reuses=1, replaces_temp_upload=False)
    assert (first["predicted_saved_bytes"], first["net_saved_bytes"], first["admit"]) == (100, 0, False)
    second = ec.evaluate_bundle(20, 30, 50, predicted_future_reuses=2, replaces_temp_upload=False)
    assert (second["predicted_saved_bytes"], second["net_saved_bytes"], second["admit"]) == (200, 100, True)


def test_eviction_reload_cost_uses_strict_break_even(ec):
    below = ec.evaluate_bundle(25, 25, 50, predicted_future_reuses=3, eviction_reload_bytes=299)
    assert (below["predicted_saved_bytes"], below["net_saved_bytes"], below["admit"]) == (400, 1, True)
    exact = ec.evaluate_bundle(25, 25, 50, predicted_future_reuses=3, eviction_reload_bytes=300)
    assert (exact["predicted_saved_bytes"], exact["net_saved_bytes"], exact["admit"]) == (400, 0, False)
    above = ec.evaluate_bundle(25, 25, 50, predicted_future_reuses=3, eviction_reload_bytes=301)
    assert (above["net_saved_bytes"], above["admit"]) == (-1, False)


def test_partial_bundle_charges_and_saves_only_missing_roles(ec):
    res = (True, False, True)
    cold = ec.evaluate_bundle(10, 20, 30, res)
    assert (cold["residency"], cold["missing_admission_bytes"], cold["predicted_saved_bytes"], cold["net_saved_bytes"], cold["admit"]) == ("partial", 20, 20, 0, False)
    first = ec.evaluate_bundle(10, 20, 30, res, predicted_future_reuses=1)
    assert (first["predicted_saved_bytes"], first["net_saved_bytes"], first["admit"]) == (40, 20, True)
    exact = ec.evaluate_bundle(10, 20, 30, res, predicted_future_reuses=1, eviction_reload_bytes=20)
    assert (exact["predicted_saved_bytes"], exact["net_saved_bytes"], exact["admit"]) == (40, 0, False)


def test_already_full_bundle_is_profitable_without_admission(ec):
    d = ec.evaluate_bundle(10, 20, 30, (True, True, True), predicted_future_reuses=U64_MAX, eviction_reload_bytes=500, replaces_temp_upload=False)
    assert (d["residency"], d["missing_admission_bytes"], d["predicted_saved_bytes"], d["profitable"], d["admit"]) == ("full", 0, 0, True, False)


def test_admission_cost_uses_wide_and_saturating_arithmetic(ec):
    d = ec.evaluate_bundle(U64_MAX, U64_MAX, U64_MAX, predicted_future_reuses=U64_MAX, eviction_reload_bytes=U64_MAX)
    assert d["missing_admission_bytes"] == U64_MAX and d["predicted_future_reuses"] == U64_MAX
    assert d["predicted_saved_bytes"] == U64_MAX * (U64_MAX + 1)
    assert d["net_saved_bytes"] == (1 << 127) - 1 and d["admit"]


def test_zero_capacity_history_never_retains_or_predicts_reuse(ec):
    h = ec.ReuseHistory(0)
    assert h.observe(7, 8) == 0 and h.observe(7, 8) == 0
    i = h.info()
    assert i["capacity"] == 0 and i["len"] == 0 and i["epoch"] == 2 and not h.contains(7, 8)


def test_resizing_history_preserves_hot_entries_and_reapplies_capacity_decay(ec):
    h = ec.ReuseHistory(3, 100)
    h.observe(0, 1)
    h.observe(0, 1)
    h.observe(0, 2)
    h.observe(0, 3)
    h.set_capacity(2)
    assert h.info()["capacity"] == 2 and h.info()["decay_interval"] == 2
    assert h.contains(0, 1) and not h.contains(0, 2) and h.contains(0, 3)
    h.set_capacity(1)
    assert h.contains(0, 1) and not h.contains(0, 3)
    h.set_capacity(4)
    assert h.observe(0, 1) == 2 and h.info()["capacity"] == 4 and h.info()["decay_interval"] == 4
    h.set_capacity(0)
    assert h.info()["len"] == 0 and h.info()["decay_interval"] == 1


def test_history_eviction_uses_frequency_then_recency(ec):
    r = ec.ReuseHistory(2, 100)
    for e in (1, 2, 3):
        r.observe(0, e)
    assert not r.contains(0, 1) and r.contains(0, 2) and r.contains(0, 3)
    f = ec.ReuseHistory(2, 100)
    for e in (1, 1, 2, 3):
        f.observe(0, e)
    assert f.contains(0, 1) and not f.contains(0, 2) and f.contains(0, 3)


def test_history_key_tie_break_is_deterministic_at_saturated_epoch(ec):
    first = ec.ReuseHistory(1, 100)
    first.set_epoch_for_test(U64_MAX)
    first.observe(0, 1)
    first.observe(0, 2)
    second = ec.ReuseHistory(1, 100)
    second.set_epoch_for_test(U64_MAX)
    second.observe(0, 2)
    second.observe(0, 1)
    assert not first.contains(0, 1) and first.contains(0, 2)
    assert not second.contains(0, 1) and second.contains(0, 2)


def test_frequency_halves_per_decay_interval_of_unobserved_epochs(ec):
    """effective_frequency (:381-392): epochs spent unobserved, minus the lookup itself, divided by the interval."""
    h = ec.ReuseHistory(8, 2)
    for _ in range(4):
        h.observe(1, 1)                      # frequency 4
    h.observe(1, 2)                          # one unobserved epoch: still 4 ...
    assert h.observe(1, 1) == 4              # ... (epoch - last_seen - 1) = 1 < interval
    for e in (2, 3, 4):
        h.observe(1, e)                      # three unobserved epochs -> one halving at the next look
    assert h.observe(1, 1) == (5 >> 1)


def test_byte_budget_lru(ec):
    b = ec.CacheBudget(20)
    assert b.touch(0, 1, 10) == [] and b.touch(0, 2, 10) == [] and b.touch(0, 1, 10) == []
    assert b.touch(1, 3, 10) == [(0, 2)] and b.resident_bytes() == 20
    z = ec.CacheBudget(0)
    assert z.touch(4, 7, 42) == [(4, 7)] and z.resident_bytes() == 0
    p = ec.CacheBudget(10)                   # byte_lru.rs tests: size updates and removals are accounted
    p.touch(0, 1, 4), p.touch(0, 2, 4), p.touch(0, 1, 4)
    assert p.touch(0, 3, 5) == [(0, 2)] and p.resident_bytes() == 9
    q = ec.CacheBudget(10)
    q.touch(0, 1, 8)
    q.touch(0, 1, 3)
    assert q.resident_bytes() == 3 and q.remove(0, 1) and not q.remove(0, 1) and q.resident_bytes() == 0


def test_moe_layer_cache_limit_rule(ec):
    """qwen35_moe_layer_cache_limit (moe_cache.rs:18-29): the smallest of what was asked for, the
    model's expert bytes, free memory minus headroom (saturating), and the device residency limit."""
    GiB = 1 << 30
    assert ec.moe_layer_cache_limit(60 * GiB, 170 * GiB, 178 * GiB, 60 * GiB, 2 * GiB) == 60 * GiB
    assert ec.moe_layer_cache_limit(60 * GiB, 20 * GiB, 178 * GiB, 60 * GiB, 2 * GiB) == 18 * GiB
    assert ec.moe_layer_cache_limit(60 * GiB, 170 * GiB, 16 * GiB, 60 * GiB, 2 * GiB) == 16 * GiB
    assert ec.moe_layer_cache_limit(60 * GiB, 170 * GiB, 178 * GiB, 8 * GiB, 2 * GiB) == 8 * GiB
    assert ec.moe_layer_cache_limit(60 * GiB, 1 * GiB, 178 * GiB, 60 * GiB, 2 * GiB) == 0
    assert ec.moe_transient_reserve_bytes(2 * GiB, 60 * GiB, 60 * GiB, GiB // 2) == GiB // 2
    assert ec.moe_transient_reserve_bytes(2 * GiB, 60 * GiB, 59 * GiB, GiB // 2) == 2 * GiB
    assert ec.moe_transient_reserve_bytes(2 * GiB, 0, 0, GiB // 2) == 2 * GiB
