// Scalar attention kernels: one warp per (query row, head[, key split]). They cover every
// dtype, head_dim <= 256, masks and strides the specialised kernels do not, and serve as
// the in-library cross-check of the TMA/MMA decode kernel. fp32 accumulation throughout.
//
// Per 32 keys a warp (1) gives each lane one key and lets it run the whole q.k dot
// product from 16-byte loads, (2) does the online-softmax update with shuffles, (3) walks
// the 32 keys again with the lanes spread over head_dim so V rows are read coalesced.
#include "paged_plan.cuh"

namespace rfx {

constexpr int kGenWarps = 4;
constexpr int kMaxD = 256;

template <typename T>
__device__ inline float dot_row(const float* __restrict__ qs, const T* __restrict__ krow, int D, bool vec_ok) {
    float s = 0.f;
    if (vec_ok) {
        constexpr int V = 16 / sizeof(T);
        struct alignas(16) P { T v[V]; };
        for (int d = 0; d < D; d += V) {
            const P kv = *reinterpret_cast<const P*>(krow + d);
#pragma unroll
            for (int j = 0; j < V; ++j) s = fmaf(qs[d + j], Num<T>::to_f(kv.v[j]), s);
        }
    } else {
        for (int d = 0; d < D; ++d) s = fmaf(qs[d], Num<T>::to_f(krow[d]), s);
    }
    return s;
}

// State of one attention row held by a warp: m, l replicated; acc[k] is dim lane + 32k.
struct RowState {
    float m, l;
    float acc[kMaxD / 32];
};

// Processes keys [j0, j1) (all visible) for one row. row_off(j) gives the element offset
// of key j's row in the K and V arrays (or -1 when the key has no storage); bias(j) the
// additive mask. int8 pools (T = int8_t) pass their per-row scales: score and probability
// of key row r are multiplied by kscale[r] and vscale[r], r = element offset / D.
template <typename T, typename RowOff, typename Bias>
__device__ inline void attend_keys(RowState& st, const float* qs, const T* __restrict__ kbase,
                                   const T* __restrict__ vbase, int D, float scale, int j0, int j1,
                                   bool vec_ok, RowOff row_off, Bias bias,
                                   const float* __restrict__ kscale = nullptr,
                                   const float* __restrict__ vscale = nullptr) {
    const int lane = threadIdx.x & 31;
    for (int jc = j0; jc < j1; jc += 32) {
        const int j = jc + lane;
        long long off = -1;
        float s = -INFINITY;
        if (j < j1) {
            off = row_off(j);
            if (off >= 0) {
                s = dot_row<T>(qs, kbase + off, D, vec_ok);
                if (kscale) s *= kscale[off / D];
                s = s * scale + bias(j);
            }
        }
        const float cm = warp_max(s);
        if (cm == -INFINITY) continue;  // nothing visible in this chunk
        const float m_new = fmaxf(st.m, cm);
        const float alpha = expf(st.m - m_new);  // exp(-inf) = 0 on the first chunk
        const float p = (s == -INFINITY) ? 0.f : expf(s - m_new);
        st.l = st.l * alpha + warp_sum(p);
        st.m = m_new;
#pragma unroll
        for (int k = 0; k < kMaxD / 32; ++k) st.acc[k] *= alpha;
        const int cnt = min(32, j1 - jc);
        for (int jj = 0; jj < cnt; ++jj) {
            float pj = __shfl_sync(0xffffffffu, p, jj);
            const long long oj = __shfl_sync(0xffffffffu, off, jj);
            if (pj == 0.f || oj < 0) continue;
            if (vscale) pj *= vscale[oj / D];
            const T* vr = vbase + oj;
#pragma unroll
            for (int k = 0; k < kMaxD / 32; ++k) {
                const int d = lane + 32 * k;
                if (d < D) st.acc[k] = fmaf(pj, Num<T>::to_f(vr[d]), st.acc[k]);
            }
        }
    }
}

__device__ inline void state_init(RowState& st) {
    st.m = -INFINITY;
    st.l = 0.f;
#pragma unroll
    for (int k = 0; k < kMaxD / 32; ++k) st.acc[k] = 0.f;
}

// ---- dense fused_attention ------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kGenWarps * 32)
dense_attention_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                       T* __restrict__ out, const T* __restrict__ mask, int64_t B, int H, int Hkv,
                       int Sq, int Sk, int D, float scale, int causal, int vec_ok) {
    __shared__ float qsm[kGenWarps][kMaxD];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t rows = B * H * Sq;
    const int G = H / Hkv;
    for (int64_t r = (int64_t)blockIdx.x * kGenWarps + warp; r < rows; r += (int64_t)gridDim.x * kGenWarps) {
        const int i = (int)(r % Sq);
        const int64_t bh = r / Sq;
        const int h = (int)(bh % H);
        const int64_t b = bh / H;
        const int hkv = h / G;
        const T* qr = q + r * D;
        __syncwarp();
        for (int d = lane; d < D; d += 32) qsm[warp][d] = Num<T>::to_f(qr[d]);
        __syncwarp();
        const T* kb = k + (b * Hkv + hkv) * (int64_t)Sk * D;
        const T* vb = v + (b * Hkv + hkv) * (int64_t)Sk * D;
        const T* mrow = mask ? mask + r * (int64_t)Sk : nullptr;
        const int j1 = causal ? min(Sk, i + 1) : Sk;  // top-left aligned
        RowState st;
        state_init(st);
        attend_keys<T>(st, qsm[warp], kb, vb, D, scale, 0, j1, vec_ok != 0,
                       [&](int j) { return (long long)j * D; },
                       [&](int j) { return mrow ? Num<T>::to_f(mrow[j]) : 0.f; });
        const float inv = st.l > 0.f ? 1.f / st.l : 0.f;
        T* orow = out + r * D;
#pragma unroll
        for (int kk = 0; kk < kMaxD / 32; ++kk) {
            const int d = lane + 32 * kk;
            if (d < D) orow[d] = Num<T>::from_f(st.acc[kk] * inv);
        }
    }
}

// ---- paged items (split-K partials) ----------------------------------------------
// One warp per partial row (item, query row, head in group). Rows are enumerated through
// item_prow, found by binary search.
template <typename T, typename KT>
__global__ void __launch_bounds__(kGenWarps * 32)
paged_partial_generic_kernel(const T* __restrict__ q, const KT* __restrict__ kc, const KT* __restrict__ vc,
                             const float* __restrict__ kscale, const float* __restrict__ vscale,
                             const int64_t* __restrict__ block_table, const int32_t* __restrict__ ctx_lens,
                             const int32_t* __restrict__ q_start, const T* __restrict__ rcos,
                             const T* __restrict__ rsin, const int32_t* __restrict__ rpos,
                             int Hq, int Hkv, int D, int64_t num_blocks, int block_size, int64_t max_blocks,
                             int64_t bt_sb, int64_t table_rows, float scale, int causal, int rope_inter,
                             int vec_ok, int32_t* hdr, const int4* __restrict__ items,
                             const int32_t* __restrict__ item_prow, float* __restrict__ pm,
                             float* __restrict__ pl, float* __restrict__ pacc) {
    __shared__ float qsm[kGenWarps][kMaxD];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_items = hdr[HdrNumItems];
    const int total_rows = hdr[HdrTotalRows];
    const int G = Hq / Hkv;
    for (int64_t pr = (int64_t)blockIdx.x * kGenWarps + warp; pr < total_rows;
         pr += (int64_t)gridDim.x * kGenWarps) {
        int lo = 0, hi = n_items;  // last item with item_prow[item] <= pr
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (item_prow[mid] <= pr) lo = mid; else hi = mid;
        }
        const int4 it = items[lo];
        const int b = it.x, hkv = it.y, kb = it.z, ke = it.w;
        const int local = (int)(pr - item_prow[lo]);
        const int qi = local / G, g = local % G;
        const int h = hkv * G + g;
        const int qrow0 = q_start ? q_start[b] : b;
        const int nq = q_start ? q_start[b + 1] - q_start[b] : 1;
        const int64_t qrow = qrow0 + qi;
        const T* qr = q + (qrow * Hq + h) * D;
        __syncwarp();
        if (rcos) {
            // RoPE fused into the Q load, same per-op rounding as the standalone op.
            const int64_t pos = rpos[qrow];
            const bool ok = pos >= 0 && pos < table_rows;
            const T* cr = rcos + (ok ? pos : 0) * D;
            const T* sr = rsin + (ok ? pos : 0) * D;
            const int half = D >> 1;
            for (int p = lane; p < half; p += 32) {
                const int d1 = rope_inter ? 2 * p : p, d2 = rope_inter ? 2 * p + 1 : p + half;
                T y1, y2;
                if (ok) rope_pair<T>(qr[d1], qr[d2], cr[d1], sr[d1], y1, y2);
                else { y1 = qr[d1]; y2 = qr[d2]; }
                qsm[warp][d1] = Num<T>::to_f(y1);
                qsm[warp][d2] = Num<T>::to_f(y2);
            }
        } else {
            for (int d = lane; d < D; d += 32) qsm[warp][d] = Num<T>::to_f(qr[d]);
        }
        __syncwarp();
        const int ctx = max(0, ctx_lens[b]);
        int vis = ctx;  // keys [0, vis) are visible to this row (bottom-right causal)
        if (causal) vis = min(ctx, ctx - nq + qi + 1);
        const int j1 = min(ke, vis);
        RowState st;
        state_init(st);
        bool bad_page = false;
        if (kb < j1) {
            attend_keys<KT>(st, qsm[warp], kc, vc, D, scale, kb, j1, vec_ok != 0,
                           [&](int j) -> long long {
                               const int64_t lb = j / block_size;
                               if (lb >= max_blocks) { bad_page = true; return -1; }
                               const int64_t page = block_table[b * bt_sb + lb];
                               if (page < 0 || page >= num_blocks) { bad_page = true; return -1; }
                               return ((page * Hkv + hkv) * block_size + (j - lb * block_size)) * (long long)D;
                           },
                           [&](int) { return 0.f; }, kscale, vscale);
        }
        if (bad_page) atomicOr(hdr + HdrStatus, kStatusBadPage);
        if (lane == 0) { pm[pr] = st.m; pl[pr] = st.l; }
        float* ar = pacc + pr * (int64_t)D;
#pragma unroll
        for (int kk = 0; kk < kMaxD / 32; ++kk) {
            const int d = lane + 32 * kk;
            if (d < D) ar[d] = st.acc[kk];
        }
    }
}

int launch_paged_generic(const RfxPagedAttentionArgs* a, const PlanLayout& L, const PlanPtrs& P) {
    const size_t e = a->kv_int8 ? 1 : dtype_size(a->dtype);
    const int D = (int)a->head_dim;
    const int vec_ok = ((D * e) % 16 == 0 && ((uintptr_t)a->k_cache % 16) == 0 && ((uintptr_t)a->v_cache % 16) == 0) ? 1 : 0;
    int64_t blocks = ceil_div<int64_t>(L.cap_rows, kGenWarps);
    const int64_t cap = (int64_t)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    if (a->kv_int8) {
        RFX_DISPATCH_DTYPE(a->dtype, T, {
            paged_partial_generic_kernel<T, int8_t><<<(int)blocks, kGenWarps * 32, 0, as_stream(a->stream)>>>(
                (const T*)a->q, (const int8_t*)a->k_cache, (const int8_t*)a->v_cache, a->k_scales, a->v_scales,
                a->block_table, a->context_lens,
                a->q_start, (const T*)a->rope_cos, (const T*)a->rope_sin, a->rope_positions,
                (int)a->num_q_heads, (int)a->num_kv_heads, D, a->num_blocks, (int)a->block_size, a->max_blocks,
                a->bt_stride_b, a->table_rows, a->sm_scale, a->is_causal, a->rope_interleaved, vec_ok, P.hdr,
                P.items, P.item_prow, P.m, P.l, P.acc);
        });
        return check_launch("rfx_paged_attention (scalar partial kernel, int8 pool)");
    }
    RFX_DISPATCH_DTYPE(a->dtype, T, {
        paged_partial_generic_kernel<T, T><<<(int)blocks, kGenWarps * 32, 0, as_stream(a->stream)>>>(
            (const T*)a->q, (const T*)a->k_cache, (const T*)a->v_cache, nullptr, nullptr, a->block_table, a->context_lens,
            a->q_start, (const T*)a->rope_cos, (const T*)a->rope_sin, a->rope_positions,
            (int)a->num_q_heads, (int)a->num_kv_heads, D, a->num_blocks, (int)a->block_size, a->max_blocks,
            a->bt_stride_b, a->table_rows, a->sm_scale, a->is_causal, a->rope_interleaved, vec_ok, P.hdr,
            P.items, P.item_prow, P.m, P.l, P.acc);
    });
    return check_launch("rfx_paged_attention (scalar partial kernel)");
}

}  // namespace rfx

extern "C" size_t rfx_fused_attention_workspace_bytes(const RfxAttentionArgs*) { return 0; }

namespace rfx {
// Implemented in prefill_mma.cu: tensor-core path for bf16/fp16 dense attention. Returns
// RFX_NOT_IMPLEMENTED when the shape is outside its coverage.
int launch_dense_tensor(const RfxAttentionArgs* a);
bool dense_tensor_ok(const RfxAttentionArgs* a);
}

extern "C" int rfx_fused_attention_kernel_kind(const RfxAttentionArgs* a) {
    if (!a || a->num_kv_heads <= 0 || a->num_q_heads <= 0) return -1;
    return rfx::dense_tensor_ok(a) ? 1 : 0;
}

extern "C" int rfx_fused_attention(const RfxAttentionArgs* a) {
    using namespace rfx;
    const char* name = "rfx_fused_attention";
    if (!a) return fail(RFX_INVALID_ARGUMENT, "%s: null args", name);
    RFX_REQUIRE(dtype_ok(a->dtype), "%s: unknown dtype %d", name, a->dtype);
    RFX_REQUIRE(a->batch >= 0 && a->num_q_heads > 0 && a->num_kv_heads > 0 && a->seq_q >= 0 &&
                    a->seq_k >= 0 && a->head_dim > 0,
                "%s: bad sizes", name);
    RFX_REQUIRE(a->num_q_heads % a->num_kv_heads == 0,
                "GQA requires num_heads_q (%lld) divisible by num_heads_kv (%lld)",
                (long long)a->num_q_heads, (long long)a->num_kv_heads);
    RFX_REQUIRE(a->head_dim <= kMaxD, "%s: head_dim %lld > %d", name, (long long)a->head_dim, kMaxD);
    RFX_REQUIRE(a->seq_k < (1ll << 31) && a->seq_q < (1ll << 31), "%s: sequence too long", name);
    if (a->batch * a->seq_q == 0) return RFX_SUCCESS;
    RFX_REQUIRE(a->q && a->out && (a->seq_k == 0 || (a->k && a->v)), "%s: null pointer", name);
    int st = check_device();
    if (st != RFX_SUCCESS) return st;

    st = launch_dense_tensor(a);
    if (st != RFX_NOT_IMPLEMENTED) return st;

    const size_t e = dtype_size(a->dtype);
    const int D = (int)a->head_dim;
    const int vec_ok = ((D * e) % 16 == 0 && ((uintptr_t)a->k % 16) == 0 && ((uintptr_t)a->v % 16) == 0) ? 1 : 0;
    const int64_t rows = a->batch * a->num_q_heads * a->seq_q;
    int64_t blocks = ceil_div<int64_t>(rows, kGenWarps);
    const int64_t cap = (int64_t)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    RFX_DISPATCH_DTYPE(a->dtype, T, {
        dense_attention_kernel<T><<<(int)blocks, kGenWarps * 32, 0, as_stream(a->stream)>>>(
            (const T*)a->q, (const T*)a->k, (const T*)a->v, (T*)a->out, (const T*)a->attn_mask, a->batch,
            (int)a->num_q_heads, (int)a->num_kv_heads, (int)a->seq_q, (int)a->seq_k, D, a->sm_scale,
            a->is_causal, vec_ok);
    });
    return check_launch(name);
}
