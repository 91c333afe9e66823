// Split-K planning for paged attention, entirely on the device so a step needs no
// device->host read of the context lengths. One CTA lays the 64-key tiles of every
// (request, kv_head) pair end to end, cuts that stream into equal runs (one per CTA of the
// persistent partial kernel, so every CTA streams the same number of bytes whatever the mix
// of request lengths), and writes the items -- the pieces of pairs inside one run.
#include "paged_plan.cuh"
#include "ptx.cuh"

namespace rfx {

constexpr int kPlanMaxThreads = 1024;  // one request per thread up to here; small batches take a warp or four

// Exclusive scan of two values per thread across the CTA of THREADS threads.
template <int THREADS>
__device__ inline void block_exscan2(long long& a, long long& b, long long (*red)[2], long long& tot_a,
                                     long long& tot_b) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    long long ia = a, ib = b;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const long long ta = __shfl_up_sync(0xffffffffu, ia, o);
        const long long tb = __shfl_up_sync(0xffffffffu, ib, o);
        if (lane >= o) { ia += ta; ib += tb; }
    }
    __syncthreads();
    if (lane == 31) { red[warp][0] = ia; red[warp][1] = ib; }
    __syncthreads();
    long long ba = 0, bb = 0;
    tot_a = 0; tot_b = 0;
#pragma unroll
    for (int i = 0; i < THREADS / 32; ++i) {
        if (i < warp) { ba += red[i][0]; bb += red[i][1]; }
        tot_a += red[i][0]; tot_b += red[i][1];
    }
    a = ba + ia - a;
    b = bb + ib - b;
}

// Length classes of the chunked-prefill kernel's units of work: eighths of the longest a unit can be
// (K/V steps of 128 keys in a run of `q` 64-key tiles, a unit with two live query tiles counted an
// eighth longer). Class 0 holds the longest.
constexpr int kUnitClasses = 8;
// 32-bit compares only: one warp runs this, every instruction at its full latency, and a 64-bit division
// per unit made the plan three times as long.
__device__ inline int unit_class(int cost, const int (&thr)[kUnitClasses - 1]) {
    int k = 0;
#pragma unroll
    for (int i = 0; i < kUnitClasses - 1; ++i) k += cost >= thr[i] ? 1 : 0;
    return kUnitClasses - 1 - k;
}

template <int kPlanThreads>
__global__ void __launch_bounds__(kPlanThreads)
plan_kernel(const int32_t* __restrict__ ctx_lens, const int32_t* __restrict__ q_start, int B, int Hkv,
            int G, long long max_parts, long long target_chunk, int parts_hint, long long item_cost, long long max_items,
            long long cap_rows, long long max_q_len, long long n_q, int32_t* hdr,
            int32_t* pair_item_begin, int32_t* pair_counter, int32_t* part_first, int4* items, int32_t* item_prow,
            int2* unit_order, long long max_units, int unit_rows, int skip_one_row) {
    __shared__ long long red[kPlanThreads / 32][2];
    ptx::pdl_trigger();  // the partial kernel may set itself up while the plan is computed
    const int tid = threadIdx.x;
    for (long long i = tid; i < (long long)B * Hkv; i += kPlanThreads) pair_counter[i] = 0;
    const int per = (B + kPlanThreads - 1) / kPlanThreads;  // requests per thread, contiguous
    const int b0 = min(B, tid * per), b1 = min(B, b0 + per);

    // With one request per thread (B <= 1024) its length and row count live in registers, so
    // the three passes below cost one global round trip, not three.
    const bool single = per == 1 && b0 < b1;
    const int ctx_reg = single ? max(0, ctx_lens[b0]) : 0;
    const int nq_reg = single ? (q_start ? max(0, q_start[b0 + 1] - q_start[b0]) : 1) : 0;
    auto ctx_of = [&](int b) { return single ? ctx_reg : max(0, ctx_lens[b]); };
    auto nq_of = [&](int b) -> long long { return single ? nq_reg : (q_start ? max(0, q_start[b + 1] - q_start[b]) : 1); };

    // tiles and non-empty requests before each request (per kv head), and in total
    long long tile_pre = 0, ne_pre = 0, tiles_all, ne_all;
    for (int b = b0; b < b1; ++b) {
        tile_pre += (ctx_of(b) + kPlanTile - 1) / kPlanTile;
        ne_pre += ctx_of(b) > 0 ? 1 : 0;
    }
    block_exscan2<kPlanThreads>(tile_pre, ne_pre, red, tiles_all, ne_all);
    const long long T_tiles = tiles_all * Hkv;
    // The stream that is cut into equal runs holds, between two consecutive pairs, `item_cost` units that
    // stand for no tile: finishing a pair (merging the warps' partials, writing rows or a partial and
    // counting it) costs a CTA about as much as streaming that many tiles, and a run that holds several
    // pairs would otherwise end later than the others. Only when runs are long against that cost.
    long long c = item_cost;
    {
        long long parts0 = parts_hint < 1 ? 1 : parts_hint;
        if (target_chunk > 0 || T_tiles < 4 * c * parts0) c = 0;
    }
    const long long T = T_tiles > 0 ? T_tiles + c * (ne_all * Hkv - 1) : 0;

    // tiles per run
    long long parts = parts_hint;
    if (target_chunk > 0) parts = (T + (target_chunk + kPlanTile - 1) / kPlanTile - 1) /
                                  ((target_chunk + kPlanTile - 1) / kPlanTile);
    if (parts > max_parts) parts = max_parts;
    if (parts < 1) parts = 1;
    const long long q = T > 0 ? (T + parts - 1) / parts : 1;
    const long long n_parts = T > 0 ? (T + q - 1) / q : 0;
    // Positions in the stream are divided by the run length twice per (request, kv head) and pass. One or
    // two warps run this kernel, every instruction at its full latency, and a 64-bit division is some 150
    // of them: with the stream shorter than 2^31 tiles (it always is) the 32-bit one is taken.
    const bool small_stream = T < (1ll << 31);
    auto run_of = [&](long long pos) -> long long {
        return small_stream ? (long long)((unsigned)pos / (unsigned)q) : pos / q;
    };

    const bool list_units = unit_order != nullptr && unit_rows > 0;
    int ucnt[kUnitClasses];  // this thread's units per class (kept in registers: constant indices only)
#pragma unroll
    for (int k = 0; k < kUnitClasses; ++k) ucnt[k] = 0;
    int uthr[kUnitClasses - 1];  // a unit's cost is its steps times 9 (two live query tiles) or 8 (one)
    {
        const int cmax = (int)min((long long)(1 << 24), ((q + 1) / 2 + 1)) * 9;
#pragma unroll
        for (int k = 0; k < kUnitClasses - 1; ++k) uthr[k] = (cmax * (k + 1) + kUnitClasses - 1) / kUnitClasses;
    }
    // units of an item of a request with nq rows: all but possibly the last have two live tiles
    auto units_of = [&](int nq, int& n_two, int& n_one) {
        const int n_u = (nq + unit_rows - 1) / unit_rows;
        n_one = (nq - (n_u - 1) * unit_rows <= unit_rows / 2) ? 1 : 0;
        n_two = n_u - n_one;
    };
    // items and partial rows before each request
    long long item_pre = 0, row_pre = 0, n_items, n_rows;
    {
        long long pre = tile_pre, ne = ne_pre;
        for (int b = b0; b < b1; ++b) {
            const long long tb = (ctx_of(b) + kPlanTile - 1) / kPlanTile;
            const long long nq = nq_of(b);
            if (tb > 0) {
                for (int h = 0; h < Hkv; ++h) {
                    const long long off = pre * Hkv + h * tb + c * (ne * Hkv + h);
                    const long long p0 = run_of(off), p1 = run_of(off + tb - 1);
                    const long long ni = p1 - p0 + 1;
                    item_pre += ni;
                    row_pre += ni * nq * G;
                    if (list_units && !(skip_one_row && nq == 1)) {
                        int n_two, n_one;
                        units_of((int)nq, n_two, n_one);
                        const int ctx = ctx_of(b);
                        for (long long p = p0; p <= p1; ++p) {
                            const long long s = max(off, p * q), e = min(off + tb, (p + 1) * q);
                            const int kb = (int)((s - off) * kPlanTile), ke = min(ctx, (int)((e - off) * kPlanTile));
                            const int steps = (ke - kb + 127) / 128;
                            const int c2 = unit_class(steps * 9, uthr), c1 = unit_class(steps * 8, uthr);
#pragma unroll
                            for (int k = 0; k < kUnitClasses; ++k) ucnt[k] += (c2 == k ? n_two : 0) + (c1 == k ? n_one : 0);
                        }
                    }
                }
                ++ne;
            }
            pre += tb;
        }
    }
    block_exscan2<kPlanThreads>(item_pre, row_pre, red, n_items, n_rows);
    // places in the unit list: the classes one after the other, inside a class the threads in order (no
    // atomics: most units of a batch fall into one class)
    long long upos[kUnitClasses], n_units = 0;
    if (list_units) {
        long long utot[kUnitClasses];
#pragma unroll
        for (int k = 0; k < kUnitClasses; k += 2) {
            upos[k] = ucnt[k]; upos[k + 1] = ucnt[k + 1];
            block_exscan2<kPlanThreads>(upos[k], upos[k + 1], red, utot[k], utot[k + 1]);
        }
#pragma unroll
        for (int k = 0; k < kUnitClasses; ++k) { upos[k] += n_units; n_units += utot[k]; }
    }
    const bool units_over = n_units > max_units;  // not by the capacity rule; then the kernel finds no unit and the status says so

    // The workspace was sized on the host from max_q_len and n_q; the row counts used here come
    // from q_start on the device. If they do not agree (a request with more rows than max_q_len,
    // q_start[B] - q_start[0] != n_q, more partial rows or items than the workspace holds), nothing
    // may be written past the capacity: the plan is left empty -- no items, no runs, every pair
    // without splits, so the partial kernels do nothing and the combine writes zeros -- and
    // kStatusCapacity is raised in the status word.
    int over = 0, one_row = 0;  // one_row: a request with a single query row and keys (the decode kernel's in a mixed batch)
    for (int b = b0; b < b1; ++b) {
        over |= nq_of(b) > max_q_len ? 1 : 0;
        one_row |= (nq_of(b) == 1 && ctx_of(b) > 0) ? 1 : 0;
    }
    const int any_one_row = __syncthreads_or(one_row);
    if (tid == 0 && q_start) over |= ((long long)q_start[B] - q_start[0] != n_q) ? 1 : 0;
    over |= (n_items > max_items || n_rows > cap_rows) ? 1 : 0;
    if (__syncthreads_or(over)) {
        for (long long i = tid; i <= (long long)B * Hkv; i += kPlanThreads) pair_item_begin[i] = 0;
        if (tid == 0) {
            part_first[0] = 0;
            item_prow[0] = 0;
            hdr[HdrNumItems] = 0;
            hdr[HdrTilesPerPart] = 1;
            hdr[HdrNumParts] = 0;
            hdr[HdrStatus] = kStatusCapacity;
            hdr[HdrTotalRows] = 0;
            hdr[HdrOneRowRequests] = 0;
            hdr[HdrNumUnits] = 0;
        }
        ptx::pdl_wait();
        return;
    }

    long long pre = tile_pre, ne = ne_pre, it = item_pre, rw = row_pre;
    for (int b = b0; b < b1; ++b) {
        const int ctx = ctx_of(b);
        const long long tb = (ctx + kPlanTile - 1) / kPlanTile;
        const long long nq = nq_of(b);
        for (int h = 0; h < Hkv; ++h) {
            pair_item_begin[(long long)b * Hkv + h] = (int)it;
            if (tb == 0) continue;
            const long long off = pre * Hkv + h * tb + c * (ne * Hkv + h);
            const long long p0 = run_of(off), p1 = run_of(off + tb - 1);
            for (long long p = p0; p <= p1; ++p) {
                const long long s = max(off, p * q), e = min(off + tb, (p + 1) * q);
                items[it] = make_int4(b, h, (int)((s - off) * kPlanTile), min(ctx, (int)((e - off) * kPlanTile)));
                item_prow[it] = (int)rw;
                // the first item of run p: it starts the run, or it starts its pair and the pair before it
                // (whose last tile sits at off - c - 1) ended in an earlier run
                if (s == p * q || (s == off && off - c <= p * q)) part_first[p] = (int)it;
                if (list_units && !units_over && !(skip_one_row && nq == 1)) {
                    const int kb = (int)((s - off) * kPlanTile), ke = min(ctx, (int)((e - off) * kPlanTile));
                    const int steps = (ke - kb + 127) / 128;
                    int n_two, n_one;
                    units_of((int)nq, n_two, n_one);
                    const int c2 = unit_class(steps * 9, uthr), c1 = unit_class(steps * 8, uthr);
                    for (int u = 0; u < n_two + n_one; ++u) {
                        const int cls = u < n_two ? c2 : c1;
                        long long at = 0;
#pragma unroll
                        for (int k = 0; k < kUnitClasses; ++k)
                            if (cls == k) at = upos[k]++;
                        unit_order[at] = make_int2((int)it, u);
                    }
                }
                ++it;
                rw += nq * G;
            }
        }
        if (tb > 0) ++ne;
        pre += tb;
    }
    if (tid == 0) {
        pair_item_begin[(long long)B * Hkv] = (int)n_items;
        part_first[n_parts] = (int)n_items;
        item_prow[n_items] = (int)n_rows;
        hdr[HdrNumItems] = (int)n_items;
        hdr[HdrTilesPerPart] = (int)q;
        hdr[HdrNumParts] = (int)n_parts;
        hdr[HdrStatus] = units_over ? kStatusCapacity : 0;
        hdr[HdrNumUnits] = (list_units && !units_over) ? (int)n_units : 0;
        hdr[HdrTotalRows] = (int)n_rows;
        hdr[HdrOneRowRequests] = any_one_row ? 1 : 0;
    }
    // The plan reads nothing its predecessor wrote, but its successor (the partial kernel) does
    // (the pool pages just appended): do not complete before the predecessor has.
    ptx::pdl_wait();
}

int launch_plan(const RfxPagedAttentionArgs* a, const PlanLayout& L, const PlanPtrs& P, int parts_hint, int item_cost,
                int unit_rows, bool skip_one_row) {
    const int G = (int)(a->num_q_heads / a->num_kv_heads);
    // a small batch gets a small CTA: the scans and barriers of 32 warps cost a one-CTA kernel microseconds
    cudaError_t e;
#define RFX_PLAN_LAUNCH(THREADS)                                                                                     \
    e = launch_pdl(plan_kernel<THREADS>, dim3(1), dim3(THREADS), 0, as_stream(a->stream), a->context_lens, a->q_start, \
                   (int)a->batch, (int)a->num_kv_heads, G, (long long)L.max_parts, (long long)a->target_chunk,        \
                   parts_hint, (long long)item_cost, (long long)L.max_items, (long long)L.cap_rows,                   \
                   (long long)(a->max_q_len < 1 ? 1 : a->max_q_len), (long long)a->n_q, P.hdr, P.pair_item_begin,     \
                   P.pair_counter, P.part_first, P.items, P.item_prow, unit_rows > 0 ? P.unit_order : (int2*)nullptr,     \
                   (long long)L.max_units, unit_rows, skip_one_row ? 1 : 0)
    if (a->batch <= 32) RFX_PLAN_LAUNCH(32);
    else if (a->batch <= 128) RFX_PLAN_LAUNCH(128);
    else RFX_PLAN_LAUNCH(kPlanMaxThreads);
#undef RFX_PLAN_LAUNCH
    if (e != cudaSuccess) return fail(RFX_CUDA_ERROR, "rfx_paged_attention_plan: %s", cudaGetErrorString(e));
    return check_launch("rfx_paged_attention_plan");
}

}  // namespace rfx
