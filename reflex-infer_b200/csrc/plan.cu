// Split-K planning for paged attention, entirely on the device so a step needs no
// device->host read of the context lengths: one CTA sums the lengths, picks the keys per
// split, prefix-sums the splits and writes the (request, kv_head, key range) item list
// that the persistent partial kernels pull from with an atomic work counter.
#include "paged_plan.cuh"

namespace rfx {

constexpr int kPlanThreads = 1024;

__device__ inline long long block_sum_ll(long long v, long long* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    long long r = 0;
    for (int i = 0; i < kPlanThreads / 32; ++i) r += red[i];
    return r;
}

// Exclusive scan of one value per thread across the CTA; returns the prefix, *total gets the sum.
__device__ inline long long block_exscan_ll(long long v, long long* red, long long* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    long long inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        long long t = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += t;
    }
    __syncthreads();
    if (lane == 31) red[warp] = inc;
    __syncthreads();
    long long base = 0, all = 0;
    for (int i = 0; i < kPlanThreads / 32; ++i) {
        if (i < warp) base += red[i];
        all += red[i];
    }
    *total = all;
    return base + inc - v;
}

__global__ void __launch_bounds__(kPlanThreads)
plan_kernel(const int32_t* __restrict__ ctx_lens, const int32_t* __restrict__ q_start, int B, int Hkv,
            int G, long long max_items, long long cap_rows, long long target_chunk, int ctas,
            int32_t* hdr, int32_t* split_base, int32_t* prow_base, int4* items, int32_t* item_prow) {
    __shared__ long long red[kPlanThreads / 32];
    __shared__ long long s_chunk;
    const int tid = threadIdx.x;
    const int per = (B + kPlanThreads - 1) / kPlanThreads;  // requests per thread, contiguous
    const int b0 = min(B, tid * per), b1 = min(B, b0 + per);

    long long my_tokens = 0;
    for (int b = b0; b < b1; ++b) my_tokens += max(0, ctx_lens[b]);
    const long long total_tokens = block_sum_ll(my_tokens, red);

    long long chunk;
    if (target_chunk > 0) {
        chunk = (target_chunk + 63) / 64 * 64;
    } else {
        // Keys per CTA, then the split length that balances per-item overhead (~48 keys'
        // worth of time) against the tail left by the last item: sqrt(2*48*per_cta).
        const double per_cta = (double)total_tokens * Hkv / (double)max(1, ctas);
        chunk = (long long)(sqrt(96.0 * per_cta) / 64.0 + 0.5) * 64;
        if (chunk < 128) chunk = 128;
    }
    // Grow the split length until items and partial rows fit the workspace.
    for (int it = 0; it < 40; ++it) {
        long long my_items = 0, my_rows = 0;
        for (int b = b0; b < b1; ++b) {
            const long long c = max(0, ctx_lens[b]);
            const long long ns = c > 0 ? (c + chunk - 1) / chunk : 1;
            const long long nq = q_start ? max(0, q_start[b + 1] - q_start[b]) : 1;
            my_items += ns;
            my_rows += ns * nq;
        }
        const long long n_items = block_sum_ll(my_items, red) * Hkv;
        const long long n_rows = block_sum_ll(my_rows, red) * Hkv * G;
        if (n_items <= max_items && n_rows <= cap_rows) break;
        chunk *= 2;
    }
    if (tid == 0) s_chunk = chunk;
    __syncthreads();
    chunk = s_chunk;

    long long my_splits = 0, my_rows = 0;
    for (int b = b0; b < b1; ++b) {
        const long long c = max(0, ctx_lens[b]);
        const long long ns = c > 0 ? (c + chunk - 1) / chunk : 1;
        const long long nq = q_start ? max(0, q_start[b + 1] - q_start[b]) : 1;
        my_splits += ns;
        my_rows += ns * nq * Hkv * G;
    }
    long long tot_splits, tot_rows;
    long long sp = block_exscan_ll(my_splits, red, &tot_splits);
    long long rw = block_exscan_ll(my_rows, red, &tot_rows);

    for (int b = b0; b < b1; ++b) {
        const int c = max(0, ctx_lens[b]);
        const int ns = c > 0 ? (int)((c + chunk - 1) / chunk) : 1;
        const int nq = q_start ? max(0, q_start[b + 1] - q_start[b]) : 1;
        split_base[b] = (int)sp;
        prow_base[b] = (int)rw;
        int len = (c + ns - 1) / ns;
        len = (len + 63) / 64 * 64;
        for (int h = 0; h < Hkv; ++h) {
            for (int s = 0; s < ns; ++s) {
                const long long item = (long long)Hkv * sp + (long long)h * ns + s;
                const int kb = min(c, s * len), ke = min(c, (s + 1) * len);
                items[item] = make_int4(b, h, kb, ke);
                item_prow[item] = (int)(rw + ((long long)h * ns + s) * nq * G);
            }
        }
        sp += ns;
        rw += (long long)ns * nq * Hkv * G;
    }
    if (tid == 0) {
        split_base[B] = (int)tot_splits;
        prow_base[B] = (int)tot_rows;
        item_prow[tot_splits * Hkv] = (int)tot_rows;
        hdr[HdrNumItems] = (int)(tot_splits * Hkv);
        hdr[HdrChunk] = (int)chunk;
        hdr[HdrWorkCounter] = 0;
        hdr[HdrStatus] = 0;
        hdr[HdrTotalRows] = (int)tot_rows;
    }
}

int launch_plan(const RfxPagedAttentionArgs* a, const PlanLayout& L, const PlanPtrs& P, int ctas_hint) {
    const int G = (int)(a->num_q_heads / a->num_kv_heads);
    plan_kernel<<<1, kPlanThreads, 0, as_stream(a->stream)>>>(
        a->context_lens, a->q_start, (int)a->batch, (int)a->num_kv_heads, G, L.max_items, L.cap_rows,
        a->target_chunk, ctas_hint, P.hdr, P.split_base, P.prow_base, P.items, P.item_prow);
    return check_launch("rfx_paged_attention_plan");
}

}  // namespace rfx
