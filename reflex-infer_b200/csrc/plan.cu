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

// Length classes of the chunked-prefill kernel's units of work (K/V steps of 128 keys, a unit with two
// live query tiles counted an eighth longer).
constexpr int kUnitBuckets = 64;
__device__ inline int unit_bucket(int kb, int ke, bool two_tiles) {
    const int steps = (ke - kb + 127) / 128;
    const int c = two_tiles ? steps + (steps + 7) / 8 : steps;
    return kUnitBuckets - 1 - min(kUnitBuckets - 1, c);  // 0 = the longest
}

template <int kPlanThreads>
__global__ void __launch_bounds__(kPlanThreads)
plan_kernel(const int32_t* __restrict__ ctx_lens, const int32_t* __restrict__ q_start, int B, int Hkv,
            int G, long long max_parts, long long target_chunk, int parts_hint, long long item_cost, long long max_items,
            long long cap_rows, long long max_q_len, long long n_q, int32_t* hdr,
            int32_t* pair_item_begin, int32_t* pair_counter, int32_t* part_first, int4* items, int32_t* item_prow,
            int2* unit_order, long long max_units, int unit_rows, int skip_one_row) {
    __shared__ long long red[kPlanThreads / 32][2];
    __shared__ int unit_hist[kUnitBuckets];  // units per length class, the longest class first; then the class's cursor
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
                    const long long ni = (off + tb - 1) / q - off / q + 1;
                    item_pre += ni;
                    row_pre += ni * nq * G;
                }
                ++ne;
            }
            pre += tb;
        }
    }
    block_exscan2<kPlanThreads>(item_pre, row_pre, red, n_items, n_rows);

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

    const bool list_units = unit_order != nullptr && unit_rows > 0;
    if (list_units) {
        for (int i = tid; i < kUnitBuckets; i += kPlanThreads) unit_hist[i] = 0;
        __syncthreads();
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
            const long long p0 = off / q, p1 = (off + tb - 1) / q;
            for (long long p = p0; p <= p1; ++p) {
                const long long s = max(off, p * q), e = min(off + tb, (p + 1) * q);
                items[it] = make_int4(b, h, (int)((s - off) * kPlanTile), min(ctx, (int)((e - off) * kPlanTile)));
                item_prow[it] = (int)rw;
                // the first item of run p: it starts the run, or it starts its pair and the pair before it
                // (whose last tile sits at off - c - 1) ended in an earlier run
                if (s == p * q || (s == off && off - c <= p * q)) part_first[p] = (int)it;
                if (list_units && !(skip_one_row && nq == 1)) {
                    const int kb = (int)((s - off) * kPlanTile), ke = min(ctx, (int)((e - off) * kPlanTile));
                    for (long long u = 0; u * unit_rows < nq; ++u)
                        atomicAdd(&unit_hist[unit_bucket(kb, ke, u * unit_rows + unit_rows / 2 < nq)], 1);
                }
                ++it;
                rw += nq * G;
            }
        }
        if (tb > 0) ++ne;
        pre += tb;
    }
    bool units_over = false;
    if (list_units) {
        // classes to cursors (one thread: 64 additions), then every unit takes the next place of its class
        __shared__ int n_units_s;
        __syncthreads();
        if (tid == 0) {
            int run = 0;
            for (int i = 0; i < kUnitBuckets; ++i) { const int n = unit_hist[i]; unit_hist[i] = run; run += n; }
            n_units_s = run;
        }
        __syncthreads();
        const bool fits = n_units_s <= max_units;  // by the capacity rule; if not, the kernel finds no unit and the status says so
        long long pre2 = tile_pre, ne2 = ne_pre, it2 = item_pre;
        for (int b = b0; b < b1 && fits; ++b) {
            const int ctx = ctx_of(b);
            const long long tb = (ctx + kPlanTile - 1) / kPlanTile;
            const long long nq = nq_of(b);
            for (int h = 0; h < Hkv && tb > 0; ++h) {
                const long long off = pre2 * Hkv + h * tb + c * (ne2 * Hkv + h);
                const long long p0 = off / q, p1 = (off + tb - 1) / q;
                for (long long p = p0; p <= p1; ++p, ++it2) {
                    if (skip_one_row && nq == 1) continue;
                    const long long s = max(off, p * q), e = min(off + tb, (p + 1) * q);
                    const int kb = (int)((s - off) * kPlanTile), ke = min(ctx, (int)((e - off) * kPlanTile));
                    for (long long u = 0; u * unit_rows < nq; ++u) {
                        const int at = atomicAdd(&unit_hist[unit_bucket(kb, ke, u * unit_rows + unit_rows / 2 < nq)], 1);
                        unit_order[at] = make_int2((int)it2, (int)u);
                    }
                }
            }
            if (tb > 0) ++ne2;
            pre2 += tb;
        }
        units_over = !fits;
        if (tid == 0) hdr[HdrNumUnits] = fits ? n_units_s : 0;
    }
    if (tid == 0) {
        pair_item_begin[(long long)B * Hkv] = (int)n_items;
        part_first[n_parts] = (int)n_items;
        item_prow[n_items] = (int)n_rows;
        hdr[HdrNumItems] = (int)n_items;
        hdr[HdrTilesPerPart] = (int)q;
        hdr[HdrNumParts] = (int)n_parts;
        hdr[HdrStatus] = units_over ? kStatusCapacity : 0;
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
