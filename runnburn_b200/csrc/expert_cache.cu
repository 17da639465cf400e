// Expert-bundle cache bookkeeping: pure host accounting, no device calls.
//
// Mirrors crates/rnb-memory/src/sparse_expert_cache.rs of the reference - the admission cost
// model (:221-270), ExpertBundleReuseHistory (:272-393: per (layer, expert) frequency that halves
// once per decay interval of unobserved epochs, victim = minimum of (effective frequency,
// last-seen epoch, key)), ExpertBundleCacheStats and the observation receipt (:395-500), and
// SparseExpertCacheBudget over crates/rnb-memory/src/byte_lru.rs:17-116 - and the layer-cache
// limit rule of crates/rnb-backend/cuda/src/runtime/state/moe_cache.rs:6-29.
#include <map>
#include <queue>
#include <vector>

#include "state.hpp"

using namespace rnb;

namespace {

using Key = std::pair<uint32_t, uint32_t>;   // (layer, expert): ordered like SparseExpertCacheKey

inline uint64_t sat_add(uint64_t a, uint64_t b) { return a > UINT64_MAX - b ? UINT64_MAX : a + b; }
inline uint64_t sat_sub(uint64_t a, uint64_t b) { return a > b ? a - b : 0; }

}  // namespace

struct rnb_b200_expert_history {
    struct Entry {
        uint64_t frequency, last_seen_epoch;
    };
    size_t capacity = 0;
    uint64_t decay_interval = 1, epoch = 0;
    std::map<Key, Entry> entries;

    static uint64_t capacity_decay_interval(size_t cap) { return cap > 0 ? (uint64_t)cap : 1; }
    uint64_t effective_frequency(const Entry &e) const {
        const uint64_t unobserved = sat_sub(sat_sub(epoch, e.last_seen_epoch), 1);
        const uint64_t periods = unobserved / decay_interval;
        return periods >= 64 ? 0 : e.frequency >> periods;
    }
    void evict_lowest_priority() {
        auto victim = entries.end();
        uint64_t vf = 0, vs = 0;
        for (auto it = entries.begin(); it != entries.end(); ++it) {   // key order: the first minimum has the lowest key
            const uint64_t f = effective_frequency(it->second), s = it->second.last_seen_epoch;
            if (victim == entries.end() || f < vf || (f == vf && s < vs)) {
                victim = it;
                vf = f;
                vs = s;
            }
        }
        if (victim != entries.end()) entries.erase(victim);
    }
    uint64_t observe(Key key) {
        epoch = sat_add(epoch, 1);
        if (capacity == 0) return 0;
        uint64_t prior = 0;
        auto it = entries.find(key);
        if (it != entries.end()) prior = effective_frequency(it->second);
        entries[key] = Entry{sat_add(prior, 1), epoch};
        if (entries.size() > capacity) evict_lowest_priority();
        return prior;
    }
    void set_capacity(size_t cap) {
        while (entries.size() > cap) evict_lowest_priority();
        capacity = cap;
        decay_interval = capacity_decay_interval(cap);
    }
};

struct rnb_b200_expert_budget {
    struct Entry {
        uint64_t bytes, last_touch;
    };
    uint64_t max_bytes = 0, resident_bytes = 0, clock = 0;
    std::map<Key, Entry> entries;
    typedef std::pair<uint64_t, Key> Aged;
    std::priority_queue<Aged, std::vector<Aged>, std::greater<Aged>> oldest;

    bool pop_oldest(Key *out) {
        while (!oldest.empty()) {
            const Aged a = oldest.top();
            oldest.pop();
            auto it = entries.find(a.second);
            if (it == entries.end() || it->second.last_touch != a.first) continue;   // stale heap record
            resident_bytes = sat_sub(resident_bytes, it->second.bytes);
            entries.erase(it);
            *out = a.second;
            return true;
        }
        return false;
    }
    void touch(Key key, uint64_t bytes, std::vector<Key> &evicted) {
        clock += 1;
        auto it = entries.find(key);
        if (it != entries.end()) {
            resident_bytes = sat_add(sat_sub(resident_bytes, it->second.bytes), bytes);
            it->second = Entry{bytes, clock};
        } else {
            resident_bytes = sat_add(resident_bytes, bytes);
            entries[key] = Entry{bytes, clock};
        }
        oldest.push(Aged(clock, key));
        while (resident_bytes > max_bytes) {
            Key k;
            if (!pop_oldest(&k)) break;
            evicted.push_back(k);
        }
    }
};

extern "C" {

// ---- reuse history ------------------------------------------------------------------------------
int rnb_b200_expert_history_create(size_t capacity, uint64_t decay_interval, rnb_b200_expert_history **out) {
    if (!out) return fail(RNB_B200_VALIDATION_FAILED, "null pointer argument");
    rnb_b200_expert_history *h = new rnb_b200_expert_history();
    h->capacity = capacity;
    const uint64_t d = decay_interval ? decay_interval : rnb_b200_expert_history::capacity_decay_interval(capacity);
    h->decay_interval = d < 1 ? 1 : d;
    *out = h;
    return RNB_B200_OK;
}
void rnb_b200_expert_history_destroy(rnb_b200_expert_history *h) { delete h; }
uint64_t rnb_b200_expert_history_observe(rnb_b200_expert_history *h, uint32_t layer, uint32_t expert) {
    return h ? h->observe(Key(layer, expert)) : 0;
}
void rnb_b200_expert_history_set_capacity(rnb_b200_expert_history *h, size_t capacity) {
    if (h) h->set_capacity(capacity);
}
int rnb_b200_expert_history_contains(const rnb_b200_expert_history *h, uint32_t layer, uint32_t expert) {
    return h && h->entries.count(Key(layer, expert)) ? 1 : 0;
}
void rnb_b200_expert_history_get_info(const rnb_b200_expert_history *h, rnb_b200_expert_history_info *out) {
    if (!h || !out) return;
    out->capacity = h->capacity;
    out->decay_interval = h->decay_interval;
    out->epoch = h->epoch;
    out->len = h->entries.size();
}
void rnb_b200_expert_history_set_epoch_for_test(rnb_b200_expert_history *h, uint64_t epoch) {
    if (h) h->epoch = epoch;
}

// ---- byte-budgeted LRU of file-backed experts -------------------------------------------------------
int rnb_b200_expert_budget_create(uint64_t max_bytes, rnb_b200_expert_budget **out) {
    if (!out) return fail(RNB_B200_VALIDATION_FAILED, "null pointer argument");
    rnb_b200_expert_budget *b = new rnb_b200_expert_budget();
    b->max_bytes = max_bytes;
    *out = b;
    return RNB_B200_OK;
}
void rnb_b200_expert_budget_destroy(rnb_b200_expert_budget *b) { delete b; }
// Touches (layer, expert) with its byte size; the keys that must be reclaimed come back as
// (layer << 32) | expert, oldest first.  *n_evicted is the full count even when cap is smaller.
int rnb_b200_expert_budget_touch(rnb_b200_expert_budget *b, uint32_t layer, uint32_t expert, uint64_t bytes, uint64_t *evicted, size_t cap,
                                 size_t *n_evicted) {
    if (!b) return fail(RNB_B200_VALIDATION_FAILED, "null pointer argument");
    std::vector<Key> ev;
    b->touch(Key(layer, expert), bytes, ev);
    for (size_t i = 0; i < ev.size() && i < cap && evicted; i++) evicted[i] = ((uint64_t)ev[i].first << 32) | ev[i].second;
    if (n_evicted) *n_evicted = ev.size();
    return RNB_B200_OK;
}
int rnb_b200_expert_budget_remove(rnb_b200_expert_budget *b, uint32_t layer, uint32_t expert) {
    if (!b) return 0;
    auto it = b->entries.find(Key(layer, expert));
    if (it == b->entries.end()) return 0;
    b->resident_bytes = sat_sub(b->resident_bytes, it->second.bytes);
    b->entries.erase(it);
    return 1;
}
uint64_t rnb_b200_expert_budget_resident_bytes(const rnb_b200_expert_budget *b) { return b ? b->resident_bytes : 0; }

// ---- admission cost ------------------------------------------------------------------------------
int rnb_b200_evaluate_expert_bundle(const rnb_b200_bundle_candidate *c, rnb_b200_bundle_decision *out) {
    if (!c || !out) return fail(RNB_B200_VALIDATION_FAILED, "null pointer argument");
    const bool full = c->gate_resident && c->up_resident && c->down_resident;
    const uint64_t missing = sat_add(sat_add(c->gate_resident ? 0 : c->gate_bytes, c->up_resident ? 0 : c->up_bytes), c->down_resident ? 0 : c->down_bytes);
    const unsigned __int128 saved = (unsigned __int128)missing * ((unsigned __int128)c->predicted_future_reuses + (c->replaces_temp_upload ? 1 : 0));
    const unsigned __int128 cost = (unsigned __int128)missing + (unsigned __int128)c->eviction_reload_bytes;
    const unsigned __int128 i128_max = ((unsigned __int128)1 << 127) - 1;
    __int128 net;
    if (saved >= cost) {
        const unsigned __int128 d = saved - cost;
        net = (__int128)(d > i128_max ? i128_max : d);
    } else {
        const unsigned __int128 d = cost - saved;
        net = d > i128_max ? -(__int128)i128_max - 1 : -(__int128)d;
    }
    const bool profitable = full || saved > cost;
    memset(out, 0, sizeof(*out));
    out->admit = (!full && profitable) ? 1 : 0;
    out->profitable = profitable ? 1 : 0;
    out->residency = full ? 0 : ((c->gate_resident || c->up_resident || c->down_resident) ? 1 : 2);
    out->missing_admission_bytes = missing;
    out->eviction_reload_bytes = c->eviction_reload_bytes;
    out->predicted_future_reuses = c->predicted_future_reuses;
    out->predicted_saved_lo = (uint64_t)saved;
    out->predicted_saved_hi = (uint64_t)(saved >> 64);
    out->net_saved_lo = (uint64_t)(unsigned __int128)net;
    out->net_saved_hi = (int64_t)(net >> 64);
    return RNB_B200_OK;
}

// ---- statistics and the per-token observation receipt ----------------------------------------------
void rnb_b200_expert_stats_record_lookup(rnb_b200_expert_bundle_stats *s, int gate_resident, int up_resident, int down_resident) {
    if (!s) return;
    s->bundle_lookups = sat_add(s->bundle_lookups, 1);
    if (gate_resident && up_resident && down_resident) s->bundle_hits = sat_add(s->bundle_hits, 1);
    else if (!gate_resident && !up_resident && !down_resident) s->bundle_misses = sat_add(s->bundle_misses, 1);
    else s->bundle_partial_hits = sat_add(s->bundle_partial_hits, 1);
}
void rnb_b200_expert_stats_delta(const rnb_b200_expert_bundle_stats *after, const rnb_b200_expert_bundle_stats *before, rnb_b200_expert_bundle_stats *out) {
    if (!after || !before || !out) return;
    const uint64_t *a = reinterpret_cast<const uint64_t *>(after), *b = reinterpret_cast<const uint64_t *>(before);
    uint64_t *o = reinterpret_cast<uint64_t *>(out);
    for (size_t i = 0; i < sizeof(*out) / 8; i++) o[i] = sat_sub(a[i], b[i]);
}
void rnb_b200_expert_stats_add(rnb_b200_expert_bundle_stats *acc, const rnb_b200_expert_bundle_stats *delta) {
    if (!acc || !delta) return;
    uint64_t *a = reinterpret_cast<uint64_t *>(acc);
    const uint64_t *d = reinterpret_cast<const uint64_t *>(delta);
    for (size_t i = 0; i < sizeof(*acc) / 8; i++) a[i] = sat_add(a[i], d[i]);
}
void rnb_b200_expert_receipt_record(rnb_b200_expert_bundle_receipt *r, const rnb_b200_expert_bundle_stats *stats) {
    if (r && stats) rnb_b200_expert_stats_add(&r->pending_stats, stats);
}
void rnb_b200_expert_receipt_mark_consumed(rnb_b200_expert_bundle_receipt *r) {
    if (r) r->consumed = 1;
}
void rnb_b200_expert_receipt_clear_stats(rnb_b200_expert_bundle_receipt *r) {
    if (r) memset(&r->pending_stats, 0, sizeof(r->pending_stats));
}

// ---- layer-cache limit rule ------------------------------------------------------------------------
uint64_t rnb_b200_qwen35_moe_layer_cache_limit(uint64_t model_moe_bytes, uint64_t free_bytes, uint64_t device_resident_limit_bytes, uint64_t requested_bytes,
                                               uint64_t runtime_headroom_bytes) {
    return std::min(std::min(requested_bytes, model_moe_bytes), std::min(sat_sub(free_bytes, runtime_headroom_bytes), device_resident_limit_bytes));
}
uint64_t rnb_b200_qwen35_moe_transient_reserve_bytes(uint64_t dynamic_reserve_bytes, uint64_t model_moe_bytes, uint64_t resident_moe_bytes, uint64_t min_layer_bytes) {
    if (model_moe_bytes > 0 && resident_moe_bytes >= model_moe_bytes && min_layer_bytes > 0) return std::min(dynamic_reserve_bytes, min_layer_bytes);
    return dynamic_reserve_bytes;
}

}  // extern "C"
