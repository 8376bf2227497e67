// Kernel-side description of one decode launch (device copy of plx_decode_problem + pointers).
#pragma once
#include <stdint.h>

#include "../../include/plx_abi.h"

namespace plx {

// One step of the peer-memory exchange of a KV-sharded decode (see decode_exchange_merge_kernel).
struct ExchangeArgs {
    float *inbox[PLX_EXCHANGE_MAX_RANKS];   // every rank's inbox as mapped into this process, own included
    int world, rank, n_records;
    int *status;         // caller-owned device word (may be null): bit r is set when rank r never delivered
    uint32_t wait_ms;    // bound of the wait for the other ranks' records
    int *err_word, *err_mirror;   // error words of this device (see sm100::ErrSink), used by the fused sweep + exchange
};

struct DecodeArgs {
    const void *q, *r, *k, *v;
    void *out;         // (batch, heads_q, D) or nullptr
    float *part_out;   // nullptr, or one partial-state record per (batch, head) instead of `out`
    const int32_t *seqused, *cache_start;
    float *ws_parts;   // (batch * heads_q, n_splits) partial records
    int *ws_counters;  // (batch * heads_q) arrival counters, zero between launches
    float *ws_gparts;  // (batch * heads_q, n_groups) records of the first merge level (n_groups > 0)
    int *ws_gcounters; // (batch * heads_q, n_groups) arrival counters of the groups
    int n_groups;      // 0: single-level merge
    int batch, heads_q, heads_kv, n_rep, cache_len, window, n_splits, kv_offset, total_len;
    float c2;  // qk_scale * log2(e)
    int64_t kv_sb, kv_st, kv_sh;   // paged: kv_sb is the stride between pages
    // paged cache (page_table != nullptr): key j of batch row b lives in page
    // page_table[b * pages_per_seq + (j >> page_shift)] at row j & page_mask
    const int32_t *page_table;
    int page_shift, page_mask, pages_per_seq;
    // Fused sweep + exchange (xch.world >= 1): the warp that holds the merged state of a (batch, head) does
    // not write a partial record but pushes it to every rank's inbox, waits for the peers' and merges.
    ExchangeArgs xch;
};

}  // namespace plx
