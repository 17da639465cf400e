"""Expert-bundle cache bookkeeping over the C ABI: the host-side accounting of
crates/rnb-memory/src/sparse_expert_cache.rs (reuse history, byte-budgeted LRU, admission cost,
statistics, observation receipt).  No device calls."""
from __future__ import annotations

import ctypes as C

from ._lib import check, load

U64 = C.c_uint64


class HistoryInfo(C.Structure):
    _fields_ = [(n, U64) for n in ("capacity", "decay_interval", "epoch", "len")]


class BundleCandidate(C.Structure):
    _fields_ = [("gate_bytes", U64), ("up_bytes", U64), ("down_bytes", U64), ("gate_resident", C.c_uint32), ("up_resident", C.c_uint32),
                ("down_resident", C.c_uint32), ("replaces_temp_upload", C.c_uint32), ("predicted_future_reuses", U64), ("eviction_reload_bytes", U64)]


class BundleDecision(C.Structure):
    _fields_ = [("admit", C.c_uint32), ("profitable", C.c_uint32), ("residency", C.c_uint32), ("reserved", C.c_uint32),
                ("missing_admission_bytes", U64), ("eviction_reload_bytes", U64), ("predicted_future_reuses", U64),
                ("predicted_saved_lo", U64), ("predicted_saved_hi", U64), ("net_saved_lo", U64), ("net_saved_hi", C.c_int64)]


STATS_FIELDS = ("bundle_lookups", "bundle_hits", "bundle_partial_hits", "bundle_misses", "bundle_admissions", "bundle_evictions",
                "admitted_bytes", "evicted_bytes", "h2d_bytes", "temp_h2d_bytes")


class BundleStats(C.Structure):
    _fields_ = [(n, U64) for n in STATS_FIELDS]

    def as_dict(self) -> dict:
        return {n: int(getattr(self, n)) for n in STATS_FIELDS}


class BundleReceipt(C.Structure):
    _fields_ = [("consumed", C.c_uint32), ("reserved", C.c_uint32), ("pending_stats", BundleStats)]


def _L():
    L = load()
    if not getattr(L, "_expert_cache_sigs", False):
        vp = C.c_void_p
        L.rnb_b200_expert_history_create.argtypes = [C.c_size_t, U64, vp]
        L.rnb_b200_expert_history_destroy.argtypes = [vp]
        L.rnb_b200_expert_history_destroy.restype = None
        L.rnb_b200_expert_history_observe.argtypes = [vp, C.c_uint32, C.c_uint32]
        L.rnb_b200_expert_history_observe.restype = U64
        L.rnb_b200_expert_history_set_capacity.argtypes = [vp, C.c_size_t]
        L.rnb_b200_expert_history_set_capacity.restype = None
        L.rnb_b200_expert_history_contains.argtypes = [vp, C.c_uint32, C.c_uint32]
        L.rnb_b200_expert_history_get_info.argtypes = [vp, vp]
        L.rnb_b200_expert_history_get_info.restype = None
        L.rnb_b200_expert_history_set_epoch_for_test.argtypes = [vp, U64]
        L.rnb_b200_expert_history_set_epoch_for_test.restype = None
        L.rnb_b200_expert_budget_create.argtypes = [U64, vp]
        L.rnb_b200_expert_budget_destroy.argtypes = [vp]
        L.rnb_b200_expert_budget_destroy.restype = None
        L.rnb_b200_expert_budget_touch.argtypes = [vp, C.c_uint32, C.c_uint32, U64, vp, C.c_size_t, vp]
        L.rnb_b200_expert_budget_remove.argtypes = [vp, C.c_uint32, C.c_uint32]
        L.rnb_b200_expert_budget_resident_bytes.argtypes = [vp]
        L.rnb_b200_expert_budget_resident_bytes.restype = U64
        L.rnb_b200_evaluate_expert_bundle.argtypes = [vp, vp]
        L.rnb_b200_expert_stats_record_lookup.argtypes = [vp, C.c_int, C.c_int, C.c_int]
        L.rnb_b200_expert_stats_record_lookup.restype = None
        for n in ("rnb_b200_expert_stats_delta",):
            getattr(L, n).argtypes = [vp, vp, vp]
            getattr(L, n).restype = None
        for n in ("rnb_b200_expert_stats_add", "rnb_b200_expert_receipt_record"):
            getattr(L, n).argtypes = [vp, vp]
            getattr(L, n).restype = None
        for n in ("rnb_b200_expert_receipt_mark_consumed", "rnb_b200_expert_receipt_clear_stats"):
            getattr(L, n).argtypes = [vp]
            getattr(L, n).restype = None
        L.rnb_b200_qwen35_moe_layer_cache_limit.argtypes = [U64] * 5
        L.rnb_b200_qwen35_moe_layer_cache_limit.restype = U64
        L.rnb_b200_qwen35_moe_transient_reserve_bytes.argtypes = [U64] * 4
        L.rnb_b200_qwen35_moe_transient_reserve_bytes.restype = U64
        L._expert_cache_sigs = True
    return L


class ReuseHistory:
    """ExpertBundleReuseHistory: `decay_interval=None` takes the capacity-proportional default."""

    def __init__(self, capacity: int, decay_interval: int | None = None):
        self._h = C.c_void_p()
        check(_L().rnb_b200_expert_history_create(capacity, decay_interval or 0, C.byref(self._h)))

    def __del__(self):
        if getattr(self, "_h", None):
            _L().rnb_b200_expert_history_destroy(self._h)
            self._h = None

    def observe(self, layer: int, expert: int) -> int:
        return int(_L().rnb_b200_expert_history_observe(self._h, layer, expert))

    def set_capacity(self, capacity: int) -> None:
        _L().rnb_b200_expert_history_set_capacity(self._h, capacity)

    def contains(self, layer: int, expert: int) -> bool:
        return bool(_L().rnb_b200_expert_history_contains(self._h, layer, expert))

    def info(self) -> dict:
        i = HistoryInfo()
        _L().rnb_b200_expert_history_get_info(self._h, C.byref(i))
        return {n: int(getattr(i, n)) for n, _ in i._fields_}

    def set_epoch_for_test(self, epoch: int) -> None:
        _L().rnb_b200_expert_history_set_epoch_for_test(self._h, epoch)


class CacheBudget:
    """SparseExpertCacheBudget: byte-budgeted LRU accounting; touch() returns the (layer, expert) keys to reclaim."""

    def __init__(self, max_bytes: int):
        self._h = C.c_void_p()
        check(_L().rnb_b200_expert_budget_create(max_bytes, C.byref(self._h)))

    def __del__(self):
        if getattr(self, "_h", None):
            _L().rnb_b200_expert_budget_destroy(self._h)
            self._h = None

    def touch(self, layer: int, expert: int, nbytes: int) -> list:
        buf = (U64 * 64)()
        n = C.c_size_t()
        check(_L().rnb_b200_expert_budget_touch(self._h, layer, expert, nbytes, buf, 64, C.byref(n)))
        return [(int(v) >> 32, int(v) & 0xFFFFFFFF) for v in list(buf)[:min(n.value, 64)]]

    def remove(self, layer: int, expert: int) -> bool:
        return bool(_L().rnb_b200_expert_budget_remove(self._h, layer, expert))

    def resident_bytes(self) -> int:
        return int(_L().rnb_b200_expert_budget_resident_bytes(self._h))


def evaluate_bundle(gate_bytes, up_bytes, down_bytes, resident=(False, False, False), predicted_future_reuses=0,
                    eviction_reload_bytes=0, replaces_temp_upload=True) -> dict:
    c = BundleCandidate(gate_bytes, up_bytes, down_bytes, int(resident[0]), int(resident[1]), int(resident[2]), int(replaces_temp_upload),
                        predicted_future_reuses, eviction_reload_bytes)
    d = BundleDecision()
    check(_L().rnb_b200_evaluate_expert_bundle(C.byref(c), C.byref(d)))
    net = (int(d.net_saved_hi) << 64) | int(d.net_saved_lo)
    return dict(admit=bool(d.admit), profitable=bool(d.profitable), residency=("full", "partial", "miss")[d.residency],
                missing_admission_bytes=int(d.missing_admission_bytes), eviction_reload_bytes=int(d.eviction_reload_bytes),
                predicted_future_reuses=int(d.predicted_future_reuses),
                predicted_saved_bytes=(int(d.predicted_saved_hi) << 64) | int(d.predicted_saved_lo), net_saved_bytes=net)


def moe_layer_cache_limit(model_moe_bytes, free_bytes, device_resident_limit_bytes, requested_bytes, runtime_headroom_bytes) -> int:
    return int(_L().rnb_b200_qwen35_moe_layer_cache_limit(model_moe_bytes, free_bytes, device_resident_limit_bytes, requested_bytes, runtime_headroom_bytes))


def moe_transient_reserve_bytes(dynamic_reserve_bytes, model_moe_bytes, resident_moe_bytes, min_layer_bytes) -> int:
    return int(_L().rnb_b200_qwen35_moe_transient_reserve_bytes(dynamic_reserve_bytes, model_moe_bytes, resident_moe_bytes, min_layer_bytes))
