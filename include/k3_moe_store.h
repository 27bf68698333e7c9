/* Expert slot policy of the partially resident mode: which experts of a layer
 * occupy the layer's device slots, as a token-batch LRU with a two-phase
 * plan / commit contract.
 *
 * These entry points replace the reference's k3_expert_cache_* functions
 * (k3_expert_cache.h:38-110) one for one: same argument meaning, same results
 * and slot numbers for the same call sequence, same error texts.  Storage stays
 * caller-owned - a slot number returned here is the `slot` argument of
 * k3_moe_store_admit (k3_moe_layer.h) and the expert id the expert kernels see
 * when a layer descriptor points at the slot table.
 *
 * Contract (k3_expert_cache.h:44-53): plan() does not change the live state.
 * Hits may be read from source_slot until commit(); a miss that the LRU keeps
 * has admit = true and must be copied into destination_slot after the readers
 * of the current state have finished; exactly one plan may be pending per
 * layer; abort() drops it.
 */
#ifndef K3_MOE_STORE_H
#define K3_MOE_STORE_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define K3_MOE_SLOT_NONE UINT32_MAX

typedef struct k3_moe_slot_cache k3_moe_slot_cache;

/* Field for field k3_expert_cache_access (k3_expert_cache.h:16-21). */
typedef struct {
    bool hit;
    bool admit;
    uint32_t source_slot;        /* global slot = layer * slots_per_layer + slot */
    uint32_t destination_slot;
} k3_moe_slot_access;

/* Field for field k3_expert_cache_stats (k3_expert_cache.h:23-30). */
typedef struct {
    uint64_t batches;
    uint64_t accesses;
    uint64_t hits;
    uint64_t misses;
    uint64_t admissions;
    uint64_t evictions;
} k3_moe_slot_stats;

/* k3_expert_cache_create (k3_expert_cache.h:38-42) */
bool k3_moe_slot_cache_create(k3_moe_slot_cache **out, uint16_t layer_count,
                              uint16_t slots_per_layer, char *error,
                              size_t error_size);

/* k3_expert_cache_plan (k3_expert_cache.h:54-60): ids must be distinct */
bool k3_moe_slot_cache_plan(k3_moe_slot_cache *cache, uint16_t layer,
                            const uint16_t *expert_ids, uint16_t expert_count,
                            k3_moe_slot_access *accesses, char *error,
                            size_t error_size);

/* k3_expert_cache_commit / _abort (k3_expert_cache.h:62-67) */
bool k3_moe_slot_cache_commit(k3_moe_slot_cache *cache, uint16_t layer,
                              char *error, size_t error_size);
void k3_moe_slot_cache_abort(k3_moe_slot_cache *cache, uint16_t layer);

/* k3_expert_cache_slot_count / _storage_bytes / _get_stats (:69-73) */
uint32_t k3_moe_slot_cache_slot_count(const k3_moe_slot_cache *cache);
uint64_t k3_moe_slot_cache_storage_bytes(const k3_moe_slot_cache *cache,
                                         uint64_t bytes_per_expert);
void k3_moe_slot_cache_get_stats(const k3_moe_slot_cache *cache,
                                 k3_moe_slot_stats *stats);

/* k3_expert_cache_snapshot_layer (:78-85): expert ids oldest to newest */
bool k3_moe_slot_cache_snapshot_layer(const k3_moe_slot_cache *cache,
                                      uint16_t layer, uint16_t *expert_ids,
                                      uint16_t expert_capacity,
                                      uint16_t *expert_count, char *error,
                                      size_t error_size);

/* k3_expert_cache_reset (:92-94) and _invalidate_slots (:101-106) */
bool k3_moe_slot_cache_reset(k3_moe_slot_cache *cache, char *error,
                             size_t error_size);
bool k3_moe_slot_cache_invalidate_slots(k3_moe_slot_cache *cache,
                                        uint32_t first_slot,
                                        uint32_t slot_count, char *error,
                                        size_t error_size);

void k3_moe_slot_cache_destroy(k3_moe_slot_cache *cache);

/* One line of the reference's decode-routes trace
 * (`capture,step,position,layer,observed_hit_mask,expert_0..expert_15`,
 * docs/observability.md:57-70, written at k3_engine.cu:1622-1644) replayed
 * through the cache: plan + commit of the line's experts on `layer`, returning
 * the hit mask the reference would have logged (bit r = expert_r was resident).
 * Returns false with a message when the plan fails. */
bool k3_moe_slot_cache_replay_line(k3_moe_slot_cache *cache, uint16_t layer,
                                   const uint16_t *expert_ids,
                                   uint16_t expert_count, uint32_t *hit_mask,
                                   uint32_t *admissions, char *error,
                                   size_t error_size);

#ifdef __cplusplus
}
#endif

#endif
