// Split-K combine: merges the un-normalised (m, l, acc) partials of one attention row
// with the running-max recurrence of kernels/softmax/triton_softmax.py:84-89 (with an
// accumulator: triton_fused_attention.py:205-227), written as max-then-weighted-sum so
// the result does not depend on the order of the splits:
//   M = max_s m_s ; out = sum_s acc_s*exp(m_s - M) / sum_s l_s*exp(m_s - M).
// One warp per output row, lanes across head_dim. Traffic: (D+2)*4 bytes per partial
// row read, D*e bytes per output row written.
#include "paged_plan.cuh"
#include "ptx.cuh"

namespace rfx {

constexpr int kCombineWarps = 4;

// Where a combined row goes: put(d, v, n) takes n (1..4) consecutive dims starting at d.
template <typename T>
struct LocalRow {
    T* row;
    __device__ inline void put(int d, const float4& v, int n) const {
        row[d] = Num<T>::from_f(v.x);
        if (n > 1) row[d + 1] = Num<T>::from_f(v.y);
        if (n > 2) row[d + 2] = Num<T>::from_f(v.z);
        if (n > 3) row[d + 3] = Num<T>::from_f(v.w);
    }
};

// Device-side form of RfxHeadGatherArgs.
struct HeadGatherDev {
    void* out[RFX_MAX_PEERS];
    uint32_t* flags[RFX_MAX_PEERS];
    uint32_t* counter;
    int32_t* status;
    long long spin_limit;
    uint32_t epoch;
    int world, rank, wait;
    uint32_t* epoch_word;   // replayable form: the epoch lives on the device (see RfxHeadGatherArgs)
    long long out_alt_offset;
};

// The same row slice stored into every rank's full output (plain stores through peer mappings).
template <typename T>
struct PeerRows {
    const HeadGatherDev* hg;
    int64_t elem;  // offset of the row slice inside a full output
    long long buf_off;  // bytes: which of the two output buffers this step writes (replayable form)
    __device__ inline void put(int d, const float4& v, int n) const {
        T t[4] = {Num<T>::from_f(v.x), Num<T>::from_f(v.y), Num<T>::from_f(v.z), Num<T>::from_f(v.w)};
        for (int p = 0; p < hg->world; ++p) {
            T* row = reinterpret_cast<T*>(reinterpret_cast<char*>(hg->out[p]) + buf_off) + elem;
            if (n == 4 && sizeof(T) == 2) {
                *reinterpret_cast<uint2*>(row + d) = *reinterpret_cast<const uint2*>(t);  // d % 4 == 0
            } else {
                for (int i = 0; i < n; ++i) row[d + i] = t[i];
            }
        }
    }
};

// `prow_of(s)` gives the partial row of split s. Lanes first fetch the splits' rows and
// statistics side by side (one round trip for up to 32 splits), then walk the splits with
// every lane owning four consecutive dims, the loads of successive splits independent.
template <typename T, typename PartialRow, typename Sink>
__device__ inline void combine_row(int ns, PartialRow prow_of, const float* __restrict__ pm,
                                   const float* __restrict__ pl, const float* __restrict__ pacc, int D,
                                   const Sink& sink) {
    const int lane = threadIdx.x & 31;
    if (ns <= 4 && (D & 3) == 0 && D <= 128) {
        // Few splits (the usual case): issue every load at once -- statistics and the lane's
        // four dims of each split -- so the row costs one memory round trip.
        const int d = lane * 4;
        float m[4], l[4];
        float4 a[4];
#pragma unroll
        for (int s = 0; s < 4; ++s) {
            m[s] = -INFINITY; l[s] = 0.f; a[s] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (s < ns) {
                const long long pr = prow_of(s);
                m[s] = pm[pr];
                l[s] = pl[pr];
                if (d < D) a[s] = *reinterpret_cast<const float4*>(pacc + pr * D + d);
            }
        }
        const float M = fmaxf(fmaxf(m[0], m[1]), fmaxf(m[2], m[3]));
        float L = 0.f;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int s = 0; s < 4; ++s) {
            const float w = (m[s] == -INFINITY) ? 0.f : expf(m[s] - M);
            L = fmaf(l[s], w, L);
            acc.x = fmaf(w, a[s].x, acc.x); acc.y = fmaf(w, a[s].y, acc.y);
            acc.z = fmaf(w, a[s].z, acc.z); acc.w = fmaf(w, a[s].w, acc.w);
        }
        const float inv = L > 0.f ? 1.f / L : 0.f;
        if (d < D) sink.put(d, make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv), 4);
        return;
    }
    float M = -INFINITY;
    for (int s0 = 0; s0 < ns; s0 += 32) {
        const int s = s0 + lane;
        if (s < ns) M = fmaxf(M, pm[prow_of(s)]);
    }
    M = warp_max(M);
    float L = 0.f;
    float4 acc[2] = {make_float4(0.f, 0.f, 0.f, 0.f), make_float4(0.f, 0.f, 0.f, 0.f)};
    const bool vec = (D & 3) == 0;
    if (M > -INFINITY) {
        for (int s0 = 0; s0 < ns; s0 += 32) {
            const int s = s0 + lane;
            long long pr = 0;
            float w = 0.f;
            if (s < ns) {
                pr = prow_of(s);
                const float m = pm[pr];
                w = (m == -INFINITY) ? 0.f : expf(m - M);
                L += pl[pr] * w;
            }
            const int cnt = min(32, ns - s0);
#pragma unroll 4
            for (int j = 0; j < cnt; ++j) {
                const float wj = __shfl_sync(0xffffffffu, w, j);
                const long long pj = __shfl_sync(0xffffffffu, pr, j);
                const float* ar = pacc + pj * D;
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    const int d = r * 128 + lane * 4;
                    if (d >= D) continue;
                    if (vec) {
                        const float4 v = *reinterpret_cast<const float4*>(ar + d);
                        acc[r].x = fmaf(wj, v.x, acc[r].x); acc[r].y = fmaf(wj, v.y, acc[r].y);
                        acc[r].z = fmaf(wj, v.z, acc[r].z); acc[r].w = fmaf(wj, v.w, acc[r].w);
                    } else {
                        acc[r].x = fmaf(wj, ar[d], acc[r].x);
                        if (d + 1 < D) acc[r].y = fmaf(wj, ar[d + 1], acc[r].y);
                        if (d + 2 < D) acc[r].z = fmaf(wj, ar[d + 2], acc[r].z);
                        if (d + 3 < D) acc[r].w = fmaf(wj, ar[d + 3], acc[r].w);
                    }
                }
            }
        }
    }
    L = warp_sum(L);
    const float inv = L > 0.f ? 1.f / L : 0.f;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int d = r * 128 + lane * 4;
        if (d >= D) continue;
        sink.put(d, make_float4(acc[r].x * inv, acc[r].y * inv, acc[r].z * inv, acc[r].w * inv), min(4, D - d));
    }
}

// Output rows = n_q * Hq, row = (query row r, head h). GATHER: rows go to every rank's full
// output instead of `out`, and the last CTA to finish publishes the epoch (see RfxHeadGatherArgs).
template <typename T, bool GATHER>
__global__ void __launch_bounds__(kCombineWarps * 32)
paged_combine_kernel(T* __restrict__ out, const __grid_constant__ HeadGatherDev hg,
                     const int32_t* __restrict__ q_start, int B, int64_t n_q, int Hq,
                     int Hkv, int D, int rows_follow_items, const int32_t* __restrict__ pair_item_begin,
                     const int32_t* __restrict__ item_prow, const float* __restrict__ pm,
                     const float* __restrict__ pl, const float* __restrict__ pacc) {
    ptx::pdl_wait();  // partials come from the kernel just before this one
    // The step's epoch: a launch argument, or (replayable form) the device word + 1 -- no CTA of this
    // launch changes the word before every CTA has finished, so all read the same value.
    uint32_t epoch = hg.epoch;
    long long buf_off = 0;
    if (GATHER && hg.epoch_word) {
        epoch = *reinterpret_cast<volatile uint32_t*>(hg.epoch_word) + 1u;
        buf_off = (long long)(epoch & 1u) * hg.out_alt_offset;
    }
    const int warp = threadIdx.x >> 5;
    const int G = Hq / Hkv;
    // A warp takes the G rows of one (query row, kv head) after one another: they belong to the same
    // request and pair and share its items, so the look-ups that come before a row's partials (request,
    // pair, items: dependent round trips, most of this kernel's time when each row did its own) are made
    // once per group.
    const int64_t groups = n_q * Hkv;
    for (int64_t grp = (int64_t)blockIdx.x * kCombineWarps + warp; grp < groups;
         grp += (int64_t)gridDim.x * kCombineWarps) {
        const int hkv = (int)(grp % Hkv);
        const int64_t r = grp / Hkv;
        int b, qi;
        if (q_start) {
            // The last b with q_start[b] <= r, 32 probes at a time: every probe of a binary search is a
            // dependent round trip (ten of them for a thousand requests).
            int lo = 0, span = B;  // the answer is in [lo, lo + span)
            while (span > 1) {
                const int step = (span + 31) >> 5;
                const int idx = lo + (int)(threadIdx.x & 31) * step;
                const bool le = idx < lo + span && (int64_t)q_start[idx] <= r;  // true for lane 0
                const unsigned m = __ballot_sync(0xffffffffu, le);
                const int k = 31 - __clz((int)(m | 1u));
                lo += k * step;
                span = min(step, span - k * step);
            }
            b = lo;
            qi = (int)(r - q_start[b]);
        } else {
            b = (int)r;
            qi = 0;
        }
        const long long pair = (long long)b * Hkv + hkv;
        const int item0 = pair_item_begin[pair];
        const int ns = pair_item_begin[pair + 1] - item0;
        for (int g = 0; g < G; ++g) {
            const int h = hkv * G + g;
            const int64_t orow = r * Hq + h;
            const int within = qi * G + g;
            auto run = [&](const auto& sink) {
                if (rows_follow_items)  // one query row per request: item i owns partial rows [i*G, i*G + G)
                    combine_row<T>(ns, [&](int s) { return (long long)(item0 + s) * G + g; }, pm, pl, pacc, D, sink);
                else
                    combine_row<T>(ns, [&](int s) { return (long long)item_prow[item0 + s] + within; }, pm, pl, pacc, D,
                                   sink);
            };
            if (GATHER)
                run(PeerRows<T>{&hg, (r * ((int64_t)hg.world * Hq) + (int64_t)hg.rank * Hq + h) * D, buf_off});
            else
                run(LocalRow<T>{out + orow * D});
        }
    }
    if (GATHER) {
        // Every thread's stores are visible system-wide before its CTA is counted.
        __threadfence_system();
        __syncthreads();
        if (threadIdx.x == 0) {
            const unsigned prev = atomicAdd(hg.counter, 1u);
            if (prev == gridDim.x - 1) {  // all CTAs of this rank have stored their rows
                __threadfence();
                *hg.counter = 0;  // for the next launch on this stream
                __threadfence_system();
                for (int p = 0; p < hg.world; ++p)
                    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(hg.flags[p] + hg.rank), "r"(epoch) : "memory");
                if (hg.epoch_word) *reinterpret_cast<volatile uint32_t*>(hg.epoch_word) = epoch;
                if (hg.wait) {
                    bool expired = false;
                    for (int q = 0; q < hg.world && !expired; ++q) {
                        const uint32_t* f = hg.flags[hg.rank] + q;
                        long long polls = 0;
                        for (;;) {
                            uint32_t v;
                            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
                            if ((int32_t)(v - epoch) >= 0) break;
                            if (++polls > hg.spin_limit) { expired = true; break; }
                            __nanosleep(100);
                        }
                    }
                    if (expired && hg.status) atomicOr(hg.status, kStatusWaitExpired);
                }
            }
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(kCombineWarps * 32)
splitk_combine_kernel(T* __restrict__ out, const int32_t* __restrict__ split_begin, int64_t rows, int D,
                      const float* __restrict__ pm, const float* __restrict__ pl,
                      const float* __restrict__ pacc) {
    const int warp = threadIdx.x >> 5;
    for (int64_t r = (int64_t)blockIdx.x * kCombineWarps + warp; r < rows;
         r += (int64_t)gridDim.x * kCombineWarps) {
        const int s0 = split_begin[r], ns = split_begin[r + 1] - s0;
        combine_row<T>(ns, [&](int s) { return (long long)(s0 + s); }, pm, pl, pacc, D, LocalRow<T>{out + r * D});
    }
}

int launch_paged_combine(const RfxPagedAttentionArgs* a, const PlanLayout& L, const PlanPtrs& P,
                         const RfxHeadGatherArgs* g) {
    const int64_t groups = a->n_q * a->num_kv_heads;  // a warp per (query row, kv head)
    int64_t blocks = ceil_div<int64_t>(groups, kCombineWarps);
    const int64_t cap = (int64_t)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    HeadGatherDev hg = {};
    if (g) {
        const char* name = "rfx_paged_attention_combine_gather";
        RFX_REQUIRE(g->world >= 1 && g->world <= RFX_MAX_PEERS && g->rank >= 0 && g->rank < g->world,
                    "%s: rank %d of %d (at most %d ranks)", name, g->rank, g->world, RFX_MAX_PEERS);
        RFX_REQUIRE((g->epoch > 0 || g->epoch_word) && g->arrival_counter,
                    "%s: epoch must be > 0 (or epoch_word given) and arrival_counter set", name);
        for (int p = 0; p < g->world; ++p) {
            RFX_REQUIRE(g->peer_out[p] && g->peer_flags[p], "%s: null pointer for rank %d", name, p);
            RFX_REQUIRE(((uintptr_t)g->peer_out[p] % 16) == 0 && ((uintptr_t)g->peer_flags[p] % 4) == 0,
                        "%s: misaligned buffer for rank %d", name, p);
            hg.out[p] = g->peer_out[p];
            hg.flags[p] = g->peer_flags[p];
        }
        hg.counter = g->arrival_counter;
        hg.status = P.hdr + HdrStatus;
        hg.spin_limit = g->spin_limit > 0 ? g->spin_limit : 10000000ll;
        hg.epoch = g->epoch;
        hg.epoch_word = g->epoch_word;
        hg.out_alt_offset = g->out_alt_offset;
        hg.world = g->world; hg.rank = g->rank; hg.wait = g->wait ? 1 : 0;
    }
    RFX_DISPATCH_DTYPE(a->dtype, T, {
        auto kern = g ? paged_combine_kernel<T, true> : paged_combine_kernel<T, false>;
        cudaError_t le = launch_pdl(kern, dim3((int)blocks), dim3(kCombineWarps * 32), 0,
                                    as_stream(a->stream), (T*)a->out, hg, a->q_start, (int)a->batch, (int64_t)a->n_q,
                                    (int)a->num_q_heads, (int)a->num_kv_heads, (int)a->head_dim,
                                    a->q_start == nullptr ? 1 : 0, (const int32_t*)P.pair_item_begin,
                                    (const int32_t*)P.item_prow, (const float*)P.m, (const float*)P.l,
                                    (const float*)P.acc);
        if (le != cudaSuccess) return fail(RFX_CUDA_ERROR, "combine launch: %s", cudaGetErrorString(le));
    });
    return check_launch("rfx_paged_attention (combine)");
}

}  // namespace rfx

extern "C" int rfx_splitk_combine(const RfxCombineArgs* a) {
    using namespace rfx;
    const char* name = "rfx_splitk_combine";
    if (!a) return fail(RFX_INVALID_ARGUMENT, "%s: null args", name);
    RFX_REQUIRE(dtype_ok(a->dtype), "%s: unknown dtype %d", name, a->dtype);
    RFX_REQUIRE(a->rows >= 0 && a->head_dim > 0 && a->head_dim <= 256, "%s: bad sizes", name);
    if (a->rows == 0) return RFX_SUCCESS;
    RFX_REQUIRE(a->acc && a->m && a->l && a->split_begin && a->out, "%s: null pointer", name);
    RFX_REQUIRE(((uintptr_t)a->acc % 16) == 0, "%s: acc must be 16-byte aligned", name);
    int st = check_device();
    if (st != RFX_SUCCESS) return st;
    int64_t blocks = ceil_div<int64_t>(a->rows, kCombineWarps);
    const int64_t cap = (int64_t)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    RFX_DISPATCH_DTYPE(a->dtype, T, {
        splitk_combine_kernel<T><<<(int)blocks, kCombineWarps * 32, 0, as_stream(a->stream)>>>(
            (T*)a->out, a->split_begin, a->rows, (int)a->head_dim, a->m, a->l, a->acc);
    });
    return check_launch(name);
}
