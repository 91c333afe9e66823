// Layout of the caller-provided paged-attention workspace, shared by the plan kernel,
// the two partial kernels (scalar and TMA/MMA) and the combine kernel.
//
//   header        : 64 int32 (see Hdr*)
//   split_base    : int32[B+1]   prefix sum of splits per request
//   prow_base     : int32[B+1]   first partial row of each request
//   items         : int4[max_items]   (request, kv_head, key_begin, key_end)
//   item_prow     : int32[max_items+1] first partial row of each item
//   m, l          : float[cap_rows] each   running max (scaled, natural log domain), sum
//   acc           : float[cap_rows][D]     un-normalised sum of p*V
//
// Items are ordered request-major, then kv head, then split, so the splits of one
// (request, kv_head) are consecutive: item = Hkv*split_base[b] + hkv*nsplit_b + s. An item
// owns n_b*G partial rows (n_b query rows of the request times the G query heads that
// share the kv head), row (qi*G + g) at item_prow[item] + qi*G + g.
#pragma once

#include "common.cuh"

namespace rfx {

enum : int {
    HdrNumItems = 0,
    HdrChunk = 1,
    HdrWorkCounter = 2,
    HdrStatus = 3,
    HdrTotalRows = 4,
    HdrWords = 64
};

constexpr int kStatusWaitExpired = 1;
constexpr int kStatusBadPage = 2;

struct PlanLayout {
    size_t off_split_base, off_prow_base, off_items, off_item_prow, off_m, off_l, off_acc, total;
    int64_t max_items, cap_rows;
};

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Capacity rule: one item per (request, kv_head) always fits, plus 16 extra splits per SM.
inline PlanLayout plan_layout(int64_t B, int64_t Hkv, int64_t G, int64_t n_q, int64_t max_q_len,
                              int64_t D, int sms) {
    PlanLayout L;
    L.max_items = Hkv * B + 16ll * sms;
    L.cap_rows = G * (Hkv * n_q + 16ll * sms * (max_q_len < 1 ? 1 : max_q_len));
    size_t o = HdrWords * sizeof(int32_t);
    L.off_split_base = o; o = align_up(o + (size_t)(B + 1) * 4, 256);
    L.off_prow_base = o;  o = align_up(o + (size_t)(B + 1) * 4, 256);
    L.off_items = o;      o = align_up(o + (size_t)L.max_items * 16, 256);
    L.off_item_prow = o;  o = align_up(o + (size_t)(L.max_items + 1) * 4, 256);
    L.off_m = o;          o = align_up(o + (size_t)L.cap_rows * 4, 256);
    L.off_l = o;          o = align_up(o + (size_t)L.cap_rows * 4, 256);
    L.off_acc = o;        o = align_up(o + (size_t)L.cap_rows * (size_t)D * 4, 256);
    L.total = o;
    return L;
}

struct PlanPtrs {
    int32_t* hdr;
    int32_t* split_base;
    int32_t* prow_base;
    int4* items;
    int32_t* item_prow;
    float* m;
    float* l;
    float* acc;
};

inline PlanPtrs plan_ptrs(void* ws, const PlanLayout& L) {
    char* p = (char*)ws;
    PlanPtrs r;
    r.hdr = (int32_t*)p;
    r.split_base = (int32_t*)(p + L.off_split_base);
    r.prow_base = (int32_t*)(p + L.off_prow_base);
    r.items = (int4*)(p + L.off_items);
    r.item_prow = (int32_t*)(p + L.off_item_prow);
    r.m = (float*)(p + L.off_m);
    r.l = (float*)(p + L.off_l);
    r.acc = (float*)(p + L.off_acc);
    return r;
}

// Host launchers implemented in their own files.
int launch_plan(const RfxPagedAttentionArgs* a, const PlanLayout& L, const PlanPtrs& P, int ctas_hint);
int launch_paged_generic(const RfxPagedAttentionArgs* a, const PlanLayout& L, const PlanPtrs& P);
int launch_paged_combine(const RfxPagedAttentionArgs* a, const PlanLayout& L, const PlanPtrs& P);
// Returns RFX_NOT_IMPLEMENTED when the shape is outside what the TMA/MMA kernel covers.
bool decode_mma_supported(const RfxPagedAttentionArgs* a);
int launch_decode_mma(const RfxPagedAttentionArgs* a, const PlanLayout& L, const PlanPtrs& P);
int decode_mma_ctas(const RfxPagedAttentionArgs* a);

}  // namespace rfx
