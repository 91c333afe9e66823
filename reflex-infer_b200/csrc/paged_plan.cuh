// Layout of the caller-provided paged-attention workspace, shared by the plan kernel,
// the two partial kernels (scalar and TMA/MMA) and the combine kernel.
//
// The work is the stream of 64-key tiles of every (request, kv_head) pair laid end to
// end. It is cut into `parts` equal runs of tiles (one per CTA of the persistent decode
// kernel), and every piece of a pair that falls into one run is an item. A pair that is
// cut by run boundaries has several items; their partials are merged by the combine.
//
//   header          : 64 int32 (see Hdr*)
//   pair_item_begin : int32[B*Hkv+1]      first item of each (request, kv_head) pair
//   pair_counter    : int32[B*Hkv]        finished items of each pair (decode kernel's in-kernel merge;
//                                         zeroed by the plan, put back to zero by the last item of a pair)
//   part_first      : int32[max_parts+1]  first item of each run
//   items           : int4[max_items]     (request, kv_head, key_begin, key_end)
//   unit_order      : int2[max_units]     chunked prefill: (item, pair of query tiles) of every CTA, the longest first
//   item_prow       : int32[max_items+1]  first partial row of each item
//   m, l            : float[cap_rows] each   running max (scaled, natural-log domain), sum
//   acc             : float[cap_rows][D]     un-normalised sum of p*V
//
// Items are ordered by position in the tile stream, so the items of one pair are
// consecutive. An item owns n_b*G partial rows (n_b query rows of the request times the G
// query heads that share the kv head), row (qi*G + g) at item_prow[item] + qi*G + g.
#pragma once

#include "common.cuh"

namespace rfx {

enum : int {
    HdrNumItems = 0,
    HdrTilesPerPart = 1,
    HdrNumParts = 2,
    HdrStatus = 3,
    HdrTotalRows = 4,
    HdrOneRowRequests = 5,  // 1: some request has a single query row (and keys)
    HdrNumUnits = 6,        // entries of unit_order
    HdrWords = 64
};

constexpr int kStatusWaitExpired = 1;
constexpr int kStatusBadPage = 2;
constexpr int kStatusCapacity = 4;   // the device-side row counts exceed what the host sized the workspace for
constexpr int kPlanTile = 64;  // keys per tile of the stream

struct PlanLayout {
    size_t off_pair_begin, off_pair_counter, off_part_first, off_items, off_unit_order, off_item_prow, off_m, off_l, off_acc, total;
    int64_t max_parts, max_items, cap_rows, max_units;
};

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Capacity rule: every pair contributes one item plus one more per run boundary inside it,
// and there are at most max_parts - 1 boundaries.
inline PlanLayout plan_layout(int64_t B, int64_t Hkv, int64_t G, int64_t n_q, int64_t max_q_len,
                              int64_t D, int sms) {
    PlanLayout L;
    L.max_parts = 8ll * sms;
    L.max_items = Hkv * B + L.max_parts;
    L.cap_rows = G * (Hkv * n_q + L.max_parts * (max_q_len < 1 ? 1 : max_q_len));
    size_t o = HdrWords * sizeof(int32_t);
    L.off_pair_begin = o; o = align_up(o + (size_t)(B * Hkv + 1) * 4, 256);
    L.off_pair_counter = o; o = align_up(o + (size_t)(B * Hkv) * 4, 256);
    L.off_part_first = o; o = align_up(o + (size_t)(L.max_parts + 1) * 4, 256);
    L.off_items = o;      o = align_up(o + (size_t)L.max_items * 16, 256);
    // an item of a request with n rows has ceil(n / 2T) units, 2T * G > 128; the items' rows sum to <= cap_rows / G
    L.max_units = L.cap_rows / 128 + L.max_items;
    L.off_unit_order = o; o = align_up(o + (size_t)L.max_units * 8, 256);
    L.off_item_prow = o;  o = align_up(o + (size_t)(L.max_items + 1) * 4, 256);
    L.off_m = o;          o = align_up(o + (size_t)L.cap_rows * 4, 256);
    L.off_l = o;          o = align_up(o + (size_t)L.cap_rows * 4, 256);
    L.off_acc = o;        o = align_up(o + (size_t)L.cap_rows * (size_t)D * 4, 256);
    L.total = o;
    return L;
}

struct PlanPtrs {
    int32_t* hdr;
    int32_t* pair_item_begin;
    int32_t* pair_counter;
    int32_t* part_first;
    int4* items;
    int2* unit_order;
    int32_t* item_prow;
    float* m;
    float* l;
    float* acc;
};

inline PlanPtrs plan_ptrs(void* ws, const PlanLayout& L) {
    char* p = (char*)ws;
    PlanPtrs r;
    r.hdr = (int32_t*)p;
    r.pair_item_begin = (int32_t*)(p + L.off_pair_begin);
    r.pair_counter = (int32_t*)(p + L.off_pair_counter);
    r.part_first = (int32_t*)(p + L.off_part_first);
    r.items = (int4*)(p + L.off_items);
    r.unit_order = (int2*)(p + L.off_unit_order);
    r.item_prow = (int32_t*)(p + L.off_item_prow);
    r.m = (float*)(p + L.off_m);
    r.l = (float*)(p + L.off_l);
    r.acc = (float*)(p + L.off_acc);
    return r;
}

// What finishing a (request, kv head) pair costs a CTA of the decode kernel, in 64-key tiles of
// streaming time (see plan_kernel).
#ifndef RFX_DECODE_ITEM_COST
#define RFX_DECODE_ITEM_COST 4
#endif
constexpr int kDecodeItemCost = RFX_DECODE_ITEM_COST;

// Host launchers implemented in their own files. `parts_hint` is the number of runs the
// partial kernel wants (its CTA count).
// `unit_rows` > 0 (chunked prefill): also list the kernel's units of work -- (item, pair of query tiles of
// unit_rows rows) -- by falling length; `skip_one_row`: without the requests of one query row.
int launch_plan(const RfxPagedAttentionArgs* a, const PlanLayout& L, const PlanPtrs& P, int parts_hint, int item_cost = 0,
                int unit_rows = 0, bool skip_one_row = false);
int launch_paged_generic(const RfxPagedAttentionArgs* a, const PlanLayout& L, const PlanPtrs& P);
// `gather` != nullptr: rows go to every rank's full output (see RfxHeadGatherArgs).
int launch_paged_combine(const RfxPagedAttentionArgs* a, const PlanLayout& L, const PlanPtrs& P,
                         const RfxHeadGatherArgs* gather = nullptr);
bool decode_mma_supported(const RfxPagedAttentionArgs* a);
bool decode_mma_shape_ok(const RfxPagedAttentionArgs* a);  // ... whatever the number of query rows per request
// `single_row_requests_only`: a mixed batch (q_start given); requests with more than one query
// row are left to the tcgen05 kernel. `merge_in_kernel`: the kernel writes `out` itself (whole pairs
// directly, cut pairs merged by their last item) and no combine kernel is needed.
int launch_decode_mma(const RfxPagedAttentionArgs* a, const PlanLayout& L, const PlanPtrs& P,
                      bool single_row_requests_only = false, bool merge_in_kernel = false);
int decode_mma_ctas(const RfxPagedAttentionArgs* a);
// tcgen05 kernel for ragged query chunks (prefill_tc.cu).
bool prefill_paged_supported(const RfxPagedAttentionArgs* a);
bool prefill_paged_split(const RfxPagedAttentionArgs* a);  // split-K over the plan's items?
int prefill_paged_parts(const RfxPagedAttentionArgs* a);
int prefill_paged_unit_rows(const RfxPagedAttentionArgs* a);  // query rows of a request that one CTA takes
// `split` = nullptr: whole rows per CTA, output written directly; else partials for the combine.
int launch_prefill_paged(const RfxPagedAttentionArgs* a, int32_t* status_word, const PlanLayout* L,
                         const PlanPtrs* split, bool skip_single_row_requests = false);
// Mixed batches: decode rows on the TMA/MMA decode kernel, longer chunks on the tcgen05 kernel.
bool prefill_paged_mixed(const RfxPagedAttentionArgs* a);

}  // namespace rfx
