// Slot policy of the partially resident expert store: a per-layer LRU over the
// layer's device slots with a plan / commit hand-over (host code only).
//
// Behaviour follows the reference's k3_expert_cache.c call for call - which
// accesses hit, which misses are admitted and into which slot, what is evicted,
// the telemetry, the error texts (k3_expert_cache.c:118-281, 311-421) - so that a
// trace recorded by the reference replays to the same hit masks.  The state is
// kept differently: one ordered vector of (expert, slot) per layer, oldest first,
// and a staged copy that plan() fills and commit() swaps in.
#include "k3_moe_store.h"

#include <algorithm>
#include <cstdio>
#include <new>
#include <vector>

namespace {

constexpr uint16_t kNoSlot = UINT16_MAX;

struct Resident {
    uint16_t expert;
    uint16_t slot;
};

struct LayerState {
    std::vector<Resident> live;      // oldest ... newest
    std::vector<Resident> staged;    // outcome of the pending plan
    bool pending = false;
    uint16_t accesses = 0, hits = 0, admissions = 0, evictions = 0;
};

void say(char *error, size_t error_size, const char *message) {
    if (error && error_size) snprintf(error, error_size, "%s", message);
}

void clear_message(char *error, size_t error_size) {
    if (error && error_size) error[0] = '\0';
}

int position_of(const std::vector<Resident> &list, uint16_t expert) {
    for (size_t i = 0; i < list.size(); i++) {
        if (list[i].expert == expert) return (int)i;
    }
    return -1;
}

}  // namespace

struct k3_moe_slot_cache {
    uint16_t layer_count = 0;
    uint16_t capacity = 0;
    std::vector<LayerState> layers;
    k3_moe_slot_stats stats{};

    uint32_t global_slot(uint16_t layer, uint16_t slot) const { return (uint32_t)layer * capacity + slot; }
    bool any_pending() const {
        return std::any_of(layers.begin(), layers.end(), [](const LayerState &l) { return l.pending; });
    }
};

extern "C" {

bool k3_moe_slot_cache_create(k3_moe_slot_cache **out, uint16_t layer_count, uint16_t slots_per_layer,
                              char *error, size_t error_size) {
    clear_message(error, error_size);
    if (out) *out = nullptr;
    if (!out || layer_count == 0 || slots_per_layer == 0) {
        say(error, error_size, "invalid expert-cache dimensions");
        return false;
    }
    k3_moe_slot_cache *cache = new (std::nothrow) k3_moe_slot_cache;
    if (!cache) {
        say(error, error_size, "expert-cache allocation failed");
        return false;
    }
    try {
        cache->layer_count = layer_count;
        cache->capacity = slots_per_layer;
        cache->layers.resize(layer_count);
        for (LayerState &l : cache->layers) {
            l.live.reserve(slots_per_layer);
            l.staged.reserve((size_t)slots_per_layer + 1u);
        }
    } catch (const std::bad_alloc &) {
        delete cache;
        say(error, error_size, "expert-cache table allocation failed");
        return false;
    }
    *out = cache;
    return true;
}

void k3_moe_slot_cache_destroy(k3_moe_slot_cache *cache) { delete cache; }

bool k3_moe_slot_cache_plan(k3_moe_slot_cache *cache, uint16_t layer, const uint16_t *expert_ids,
                            uint16_t expert_count, k3_moe_slot_access *accesses, char *error,
                            size_t error_size) {
    clear_message(error, error_size);
    if (!cache || layer >= cache->layer_count || !expert_ids || expert_count == 0 || !accesses) {
        say(error, error_size, "invalid expert-cache plan arguments");
        return false;
    }
    LayerState &state = cache->layers[layer];
    if (state.pending) {
        say(error, error_size, "expert-cache layer already has a pending plan");
        return false;
    }
    for (uint16_t i = 1; i < expert_count; i++) {
        if (std::find(expert_ids, expert_ids + i, expert_ids[i]) != expert_ids + i) {
            say(error, error_size, "expert-cache batch contains duplicate IDs");
            return false;
        }
    }
    const std::vector<Resident> &live = state.live;
    std::vector<Resident> &next = state.staged;
    next = live;

    // touch the batch in rank order on the staged copy: a resident expert moves to
    // the newest end with its slot, a new one pushes the oldest out when full
    uint16_t hits = 0;
    for (uint16_t rank = 0; rank < expert_count; rank++) {
        k3_moe_slot_access &access = accesses[rank];
        access = k3_moe_slot_access{false, false, K3_MOE_SLOT_NONE, K3_MOE_SLOT_NONE};
        const int at_live = position_of(live, expert_ids[rank]);
        if (at_live >= 0) {
            access.hit = true;
            access.source_slot = cache->global_slot(layer, live[(size_t)at_live].slot);
            hits++;
        }
        Resident touched{expert_ids[rank], kNoSlot};
        const int at_next = position_of(next, expert_ids[rank]);
        if (at_next >= 0) {
            touched.slot = next[(size_t)at_next].slot;
            next.erase(next.begin() + at_next);
        } else if (next.size() == cache->capacity) {
            next.erase(next.begin());
        }
        next.push_back(touched);
    }

    // slots: kept ones first; an expert that fell out and came back inside the batch
    // returns to its old slot if nobody took it (its bytes are still there); the rest
    // take the lowest free slot, oldest entry first
    std::vector<bool> used(cache->capacity, false);
    for (const Resident &r : next) {
        if (r.slot != kNoSlot) used[r.slot] = true;
    }
    for (Resident &r : next) {
        if (r.slot != kNoSlot) continue;
        const int old = position_of(live, r.expert);
        if (old >= 0 && !used[live[(size_t)old].slot]) {
            r.slot = live[(size_t)old].slot;
            used[r.slot] = true;
        }
    }
    for (Resident &r : next) {
        if (r.slot != kNoSlot) continue;
        const auto free_slot = std::find(used.begin(), used.end(), false);
        if (free_slot == used.end()) {
            say(error, error_size, "expert-cache plan has no free slot");
            return false;
        }
        r.slot = (uint16_t)(free_slot - used.begin());
        *free_slot = true;
    }

    uint16_t admissions = 0;
    for (uint16_t rank = 0; rank < expert_count; rank++) {
        if (accesses[rank].hit) continue;
        const int at = position_of(next, expert_ids[rank]);
        if (at >= 0) {
            accesses[rank].admit = true;
            accesses[rank].destination_slot = cache->global_slot(layer, next[(size_t)at].slot);
            admissions++;
        }
    }
    uint16_t evictions = 0;
    for (const Resident &r : live) {
        if (position_of(next, r.expert) < 0) evictions++;
    }
    state.pending = true;
    state.accesses = expert_count;
    state.hits = hits;
    state.admissions = admissions;
    state.evictions = evictions;
    return true;
}

bool k3_moe_slot_cache_commit(k3_moe_slot_cache *cache, uint16_t layer, char *error, size_t error_size) {
    clear_message(error, error_size);
    if (!cache || layer >= cache->layer_count || !cache->layers[layer].pending) {
        say(error, error_size, "expert-cache layer has no pending plan");
        return false;
    }
    LayerState &state = cache->layers[layer];
    state.live.swap(state.staged);
    cache->stats.batches++;
    cache->stats.accesses += state.accesses;
    cache->stats.hits += state.hits;
    cache->stats.misses += (uint64_t)state.accesses - state.hits;
    cache->stats.admissions += state.admissions;
    cache->stats.evictions += state.evictions;
    state.pending = false;
    state.accesses = state.hits = state.admissions = state.evictions = 0;
    return true;
}

void k3_moe_slot_cache_abort(k3_moe_slot_cache *cache, uint16_t layer) {
    if (!cache || layer >= cache->layer_count) return;
    LayerState &state = cache->layers[layer];
    state.pending = false;
    state.accesses = state.hits = state.admissions = state.evictions = 0;
}

uint32_t k3_moe_slot_cache_slot_count(const k3_moe_slot_cache *cache) {
    return cache ? (uint32_t)cache->layer_count * cache->capacity : 0u;
}

uint64_t k3_moe_slot_cache_storage_bytes(const k3_moe_slot_cache *cache, uint64_t bytes_per_expert) {
    const uint64_t slots = k3_moe_slot_cache_slot_count(cache);
    if (!cache || (bytes_per_expert != 0 && slots > UINT64_MAX / bytes_per_expert)) return UINT64_MAX;
    return slots * bytes_per_expert;
}

void k3_moe_slot_cache_get_stats(const k3_moe_slot_cache *cache, k3_moe_slot_stats *stats) {
    if (!stats) return;
    *stats = cache ? cache->stats : k3_moe_slot_stats{};
}

bool k3_moe_slot_cache_snapshot_layer(const k3_moe_slot_cache *cache, uint16_t layer, uint16_t *expert_ids,
                                      uint16_t expert_capacity, uint16_t *expert_count, char *error,
                                      size_t error_size) {
    clear_message(error, error_size);
    if (expert_count) *expert_count = 0u;
    if (!cache || layer >= cache->layer_count || !expert_ids || !expert_count ||
        cache->layers[layer].pending || expert_capacity < cache->layers[layer].live.size()) {
        say(error, error_size, "invalid expert-cache snapshot request");
        return false;
    }
    const std::vector<Resident> &live = cache->layers[layer].live;
    for (size_t i = 0; i < live.size(); i++) expert_ids[i] = live[i].expert;
    *expert_count = (uint16_t)live.size();
    return true;
}

bool k3_moe_slot_cache_reset(k3_moe_slot_cache *cache, char *error, size_t error_size) {
    clear_message(error, error_size);
    if (!cache) {
        say(error, error_size, "invalid expert-cache reset");
        return false;
    }
    if (cache->any_pending()) {
        say(error, error_size, "cannot reset expert cache with a pending plan");
        return false;
    }
    for (LayerState &l : cache->layers) {
        l.live.clear();
        l.staged.clear();
    }
    cache->stats = k3_moe_slot_stats{};
    return true;
}

bool k3_moe_slot_cache_invalidate_slots(k3_moe_slot_cache *cache, uint32_t first_slot, uint32_t slot_count,
                                        char *error, size_t error_size) {
    clear_message(error, error_size);
    const uint32_t total = k3_moe_slot_cache_slot_count(cache);
    if (!cache || slot_count == 0u || first_slot > total || slot_count > total - first_slot) {
        say(error, error_size, "invalid expert-cache invalidation range");
        return false;
    }
    if (cache->any_pending()) {
        say(error, error_size, "cannot invalidate expert cache with a pending plan");
        return false;
    }
    const uint32_t end_slot = first_slot + slot_count;
    for (uint16_t layer = 0; layer < cache->layer_count; layer++) {
        std::vector<Resident> &live = cache->layers[layer].live;
        const size_t before = live.size();
        live.erase(std::remove_if(live.begin(), live.end(),
                                  [&](const Resident &r) {
                                      const uint32_t g = cache->global_slot(layer, r.slot);
                                      return g >= first_slot && g < end_slot;
                                  }),
                   live.end());
        cache->stats.evictions += before - live.size();
    }
    return true;
}

bool k3_moe_slot_cache_replay_line(k3_moe_slot_cache *cache, uint16_t layer, const uint16_t *expert_ids,
                                   uint16_t expert_count, uint32_t *hit_mask, uint32_t *admissions,
                                   char *error, size_t error_size) {
    if (hit_mask) *hit_mask = 0u;
    if (admissions) *admissions = 0u;
    if (expert_count > 32u) {
        say(error, error_size, "a trace line holds at most 32 experts");
        return false;
    }
    k3_moe_slot_access accesses[32];
    if (!k3_moe_slot_cache_plan(cache, layer, expert_ids, expert_count, accesses, error, error_size)) return false;
    uint32_t mask = 0u, admitted = 0u;
    for (uint16_t rank = 0; rank < expert_count; rank++) {
        if (accesses[rank].hit) mask |= 1u << rank;
        if (accesses[rank].admit) admitted++;
    }
    if (!k3_moe_slot_cache_commit(cache, layer, error, error_size)) return false;
    if (hit_mask) *hit_mask = mask;
    if (admissions) *admissions = admitted;
    return true;
}

}  // extern "C"
