// Host-side routing metadata: token-major pair list and the grouped/tiled
// schedule. Replaces PrefillRouter.makeTokenExpertPairs
// (Kernels/Prefill/MoE/PrefillRouter.swift:91-111) and
// PrefillMoEGrouping.groupTokenExpertPairs (Kernels/Prefill/MoE/PrefillMoEGrouping.swift:91-193).
//
// The order required is (expert sort key, expert, token, rank). Because a valid
// pair list holds every (token, rank) exactly once, the pairs are first placed
// at slot token*topK + rank (which is also the duplicate check), and a stable
// counting sort over that token-major sequence, keyed by the expert's position
// in the (sort key, expert) order, yields the result in O(pairs + experts log experts).
#include <algorithm>
#include <cstdint>
#include <numeric>
#include <vector>

#include "turbofieldfare_cuda.h"

namespace tf {
void set_global_error(const char* fmt, ...);
}

extern "C" {

tf_status tf_make_token_expert_pairs(const uint32_t* host_indices, const uint16_t* host_weights_f16,
                                     uint32_t query_count, uint32_t top_k, tf_pair* host_pairs_out) {
    if ((query_count && top_k) && (!host_indices || !host_weights_f16 || !host_pairs_out)) {
        tf::set_global_error("tf_make_token_expert_pairs: NULL array");
        return TF_ERR_INVALID_ARGUMENT;
    }
    for (uint32_t t = 0; t < query_count; ++t)
        for (uint32_t r = 0; r < top_k; ++r) {
            const size_t i = (size_t)t * top_k + r;
            host_pairs_out[i] = tf_pair{t, host_indices[i], r, (uint32_t)host_weights_f16[i]};
        }
    return TF_OK;
}

tf_status tf_group_pairs(const tf_pair* host_pairs, uint32_t pair_count, int32_t query_count, int32_t top_k,
                         int32_t num_experts, int32_t tile_expert_count,
                         const uint64_t* host_expert_sort_keys, uint32_t sort_key_count,
                         tf_pair* sorted_out, uint32_t* per_expert_offsets, uint32_t* per_expert_counts,
                         tf_group* groups_out, uint32_t* group_count_out,
                         tf_tile* tiles_out, uint32_t* tile_count_out) {
    // Validation order follows PrefillMoEGrouping.swift:99-145.
    if (query_count < 0) { tf::set_global_error("queryCount must be non-negative, got %d", query_count); return TF_ERR_GROUPING_INVALID_QUERY_COUNT; }
    if (top_k <= 0) { tf::set_global_error("topK must be positive, got %d", top_k); return TF_ERR_GROUPING_INVALID_TOP_K; }
    if (num_experts <= 0) { tf::set_global_error("numExperts must be positive, got %d", num_experts); return TF_ERR_GROUPING_INVALID_NUM_EXPERTS; }
    if (tile_expert_count < 1 || tile_expert_count > TF_MAX_TILE_EXPERTS) {
        tf::set_global_error("tileExpertCount must be in 1...16, got %d", tile_expert_count);
        return TF_ERR_GROUPING_INVALID_TILE_EXPERT_COUNT;
    }
    if (host_expert_sort_keys && sort_key_count != (uint32_t)num_experts) {
        tf::set_global_error("expected %d expert sort keys, got %u", num_experts, sort_key_count);
        return TF_ERR_GROUPING_SORT_KEY_COUNT_MISMATCH;
    }
    const uint64_t expected = (uint64_t)query_count * (uint64_t)top_k;
    if ((uint64_t)pair_count != expected) {
        tf::set_global_error("expected %llu route pairs, got %u", (unsigned long long)expected, pair_count);
        return TF_ERR_GROUPING_PAIR_COUNT_MISMATCH;
    }
    if (!group_count_out || !tile_count_out || !per_expert_offsets || !per_expert_counts ||
        (pair_count && (!host_pairs || !sorted_out || !groups_out || !tiles_out))) {
        tf::set_global_error("tf_group_pairs: NULL array");
        return TF_ERR_INVALID_ARGUMENT;
    }

    std::vector<int64_t> slot_of(pair_count, -1);   // token-major slot -> input position
    for (uint32_t i = 0; i < pair_count; ++i) {
        const tf_pair& p = host_pairs[i];
        if (p.token >= (uint32_t)query_count) { tf::set_global_error("route token %u is out of range", p.token); return TF_ERR_GROUPING_TOKEN_OUT_OF_RANGE; }
        if (p.rank >= (uint32_t)top_k) { tf::set_global_error("route rank %u is out of range", p.rank); return TF_ERR_GROUPING_RANK_OUT_OF_RANGE; }
        if (p.expert >= (uint32_t)num_experts) { tf::set_global_error("route expert %u is out of range", p.expert); return TF_ERR_GROUPING_EXPERT_OUT_OF_RANGE; }
        const size_t slot = (size_t)p.token * (size_t)top_k + p.rank;
        if (slot_of[slot] >= 0) {
            tf::set_global_error("duplicate route pair for token %u, rank %u", p.token, p.rank);
            return TF_ERR_GROUPING_DUPLICATE_TOKEN_RANK;
        }
        slot_of[slot] = i;
    }

    // Experts in (sort key, expert id) order.
    std::vector<uint32_t> expert_order(num_experts);
    std::iota(expert_order.begin(), expert_order.end(), 0u);
    if (host_expert_sort_keys)
        std::stable_sort(expert_order.begin(), expert_order.end(), [&](uint32_t a, uint32_t b) {
            return host_expert_sort_keys[a] < host_expert_sort_keys[b];
        });

    std::vector<uint32_t> counts(num_experts, 0);
    for (uint32_t i = 0; i < pair_count; ++i) counts[host_pairs[i].expert]++;
    std::vector<uint32_t> cursor(num_experts, 0);
    uint32_t running = 0, ng = 0;
    for (int32_t e = 0; e < num_experts; ++e) { per_expert_offsets[e] = UINT32_MAX; per_expert_counts[e] = 0; }
    for (uint32_t pos = 0; pos < (uint32_t)num_experts; ++pos) {
        const uint32_t e = expert_order[pos];
        if (counts[e] == 0) continue;
        cursor[e] = running;
        per_expert_offsets[e] = running;
        per_expert_counts[e] = counts[e];
        groups_out[ng++] = tf_group{e, running, counts[e]};
        running += counts[e];
    }
    for (uint32_t slot = 0; slot < pair_count; ++slot) {          // token-major walk keeps (token, rank) order
        const tf_pair& p = host_pairs[slot_of[slot]];
        sorted_out[cursor[p.expert]++] = p;
    }

    uint32_t nt = 0;
    for (uint32_t gs = 0; gs < ng; gs += (uint32_t)tile_expert_count) {
        const uint32_t ge = std::min(ng, gs + (uint32_t)tile_expert_count);
        const tf_group& first = groups_out[gs];
        const tf_group& last = groups_out[ge - 1];
        tiles_out[nt++] = tf_tile{gs, ge - gs, first.pair_start, last.pair_start + last.pair_count - first.pair_start};
    }
    *group_count_out = ng;
    *tile_count_out = nt;
    return TF_OK;
}

}  // extern "C"
