// Entry points of paged attention: argument checks, workspace layout, and the three
// launches of a step (plan, split-K partials, combine).
#include <atomic>

#include "paged_plan.cuh"

namespace rfx {

static int validate(const RfxPagedAttentionArgs* a, const char* name) {
    if (!a) return fail(RFX_INVALID_ARGUMENT, "%s: null args", name);
    RFX_REQUIRE(dtype_ok(a->dtype), "%s: unknown dtype %d", name, a->dtype);
    RFX_REQUIRE(a->batch >= 0 && a->n_q >= 0 && a->num_q_heads > 0 && a->num_kv_heads > 0 && a->head_dim > 0 &&
                    a->num_blocks > 0 && a->block_size > 0 && a->max_blocks >= 0,
                "%s: bad sizes", name);
    RFX_REQUIRE(a->num_q_heads % a->num_kv_heads == 0,
                "GQA requires num_heads_q (%lld) divisible by num_heads_kv (%lld)", (long long)a->num_q_heads,
                (long long)a->num_kv_heads);
    RFX_REQUIRE(a->head_dim <= 256, "%s: head_dim %lld > 256", name, (long long)a->head_dim);
    RFX_REQUIRE(a->q_start != nullptr || a->n_q == a->batch,
                "%s: without q_start there is one query row per request (n_q=%lld, batch=%lld)", name,
                (long long)a->n_q, (long long)a->batch);
    RFX_REQUIRE(a->batch < (1ll << 24) && a->n_q < (1ll << 31), "%s: batch too large", name);
    RFX_REQUIRE((a->rope_cos == nullptr) == (a->rope_sin == nullptr), "%s: rope_cos and rope_sin go together", name);
    RFX_REQUIRE(a->rope_cos == nullptr || (a->rope_positions != nullptr && a->head_dim % 2 == 0),
                "%s: fused RoPE needs rope_positions and an even head_dim", name);
    RFX_REQUIRE(!a->kv_int8 || (a->k_scales && a->v_scales), "%s: an int8 pool needs k_scales and v_scales", name);
    return RFX_SUCCESS;
}

static PlanLayout layout_of(const RfxPagedAttentionArgs* a) {
    const int64_t G = a->num_q_heads / a->num_kv_heads;
    return plan_layout(a->batch, a->num_kv_heads, G, a->n_q, a->max_q_len, a->head_dim, sm_count());
}

}  // namespace rfx

extern "C" size_t rfx_paged_attention_workspace_bytes(const RfxPagedAttentionArgs* a) {
    using namespace rfx;
    if (validate(a, "rfx_paged_attention_workspace_bytes") != RFX_SUCCESS) return 0;
    return layout_of(a).total;
}

extern "C" int rfx_paged_attention_plan(const RfxPagedAttentionArgs* a) {
    using namespace rfx;
    const char* name = "rfx_paged_attention_plan";
    int st = validate(a, name);
    if (st != RFX_SUCCESS) return st;
    if (a->batch == 0) return RFX_SUCCESS;
    RFX_REQUIRE(a->context_lens && a->workspace, "%s: null pointer", name);
    st = check_device();
    if (st != RFX_SUCCESS) return st;
    const PlanLayout L = layout_of(a);
    if (a->workspace_bytes < L.total)
        return fail(RFX_WORKSPACE_TOO_SMALL, "%s: workspace %zu B < %zu B", name, a->workspace_bytes, L.total);
    RFX_REQUIRE(((uintptr_t)a->workspace % 256) == 0, "%s: workspace must be 256-byte aligned", name);
    const PlanPtrs P = plan_ptrs(a->workspace, L);
    int ctas = decode_mma_supported(a) ? decode_mma_ctas(a) : sm_count() * 4;
    int item_cost = decode_mma_supported(a) ? kDecodeItemCost : 0;
    if (prefill_paged_supported(a)) {
        if (!prefill_paged_split(a)) return RFX_SUCCESS;  // that kernel needs no plan
        ctas = prefill_paged_parts(a);
        return launch_plan(a, L, P, ctas, 0, prefill_paged_unit_rows(a), prefill_paged_mixed(a));
    }
    return launch_plan(a, L, P, ctas, item_cost);
}

namespace rfx {
enum : int { kStagePlan = 1, kStagePartials = 2, kStageCombine = 4 };

static int run_stages(const RfxPagedAttentionArgs* a, const char* name, int stages,
                      const RfxHeadGatherArgs* gather = nullptr) {
    int st = validate(a, name);
    if (st != RFX_SUCCESS) return st;
    if (a->batch == 0 || a->n_q == 0) return RFX_SUCCESS;
    RFX_REQUIRE(a->q && (a->out || gather) && a->k_cache && a->v_cache && a->block_table && a->context_lens &&
                    a->workspace,
                "%s: null pointer", name);
    st = check_device();
    if (st != RFX_SUCCESS) return st;
    const PlanLayout L = layout_of(a);
    if (a->workspace_bytes < L.total)
        return fail(RFX_WORKSPACE_TOO_SMALL, "%s: workspace %zu B < %zu B", name, a->workspace_bytes, L.total);
    RFX_REQUIRE(((uintptr_t)a->workspace % 256) == 0, "%s: workspace must be 256-byte aligned", name);
    const PlanPtrs P = plan_ptrs(a->workspace, L);
    if (prefill_paged_supported(a)) {
        // Query chunks on the tcgen05 kernel.
        if (!prefill_paged_split(a)) {
            // whole rows per CTA: no plan and no combine
            if (gather) return fail(RFX_NOT_IMPLEMENTED, "%s: the head gather rides on the combine kernel", name);
            if (!(stages & kStagePartials)) return RFX_SUCCESS;
            cudaError_t e = cudaMemsetAsync(P.hdr + HdrStatus, 0, sizeof(int32_t), as_stream(a->stream));
            if (e != cudaSuccess) return fail(RFX_CUDA_ERROR, "%s: cudaMemsetAsync: %s", name, cudaGetErrorString(e));
            return launch_prefill_paged(a, P.hdr + HdrStatus, &L, nullptr);
        }
        if (stages & kStagePlan) {
            st = launch_plan(a, L, P, prefill_paged_parts(a), 0, prefill_paged_unit_rows(a), prefill_paged_mixed(a));
            if (st != RFX_SUCCESS) return st;
        }
        if (stages & kStagePartials) {
            const bool mixed = prefill_paged_mixed(a);
            if (mixed) {
                st = launch_decode_mma(a, L, P, true);
                if (st != RFX_SUCCESS) return st;
            }
            st = launch_prefill_paged(a, P.hdr + HdrStatus, &L, &P, mixed);
            if (st != RFX_SUCCESS) return st;
        }
        if (stages & kStageCombine) return launch_paged_combine(a, L, P, gather);
        return RFX_SUCCESS;
    }
    const bool mma = decode_mma_supported(a);
    if (stages & kStagePlan) {
        st = launch_plan(a, L, P, mma ? decode_mma_ctas(a) : sm_count() * 4, mma ? kDecodeItemCost : 0);
        if (st != RFX_SUCCESS) return st;
    }
    // One call for the whole step and no gather: the decode kernel merges the split pairs itself and
    // writes `out`; the combine kernel is for the staged calls, the gather and the scalar kernel.
    const bool merge_in_kernel = mma && !gather && (stages & kStagePartials) && (stages & kStageCombine);
    if (stages & kStagePartials) {
        st = mma ? launch_decode_mma(a, L, P, false, merge_in_kernel) : launch_paged_generic(a, L, P);
        if (st != RFX_SUCCESS) return st;
    }
    if ((stages & kStageCombine) && !merge_in_kernel) return launch_paged_combine(a, L, P, gather);
    return RFX_SUCCESS;
}
}  // namespace rfx

extern "C" int rfx_paged_attention(const RfxPagedAttentionArgs* a) {
    using namespace rfx;
    const int plan = (a && a->reuse_plan) ? 0 : kStagePlan;
    return run_stages(a, "rfx_paged_attention", plan | kStagePartials | kStageCombine);
}

extern "C" int rfx_paged_attention_partials(const RfxPagedAttentionArgs* a) {
    return rfx::run_stages(a, "rfx_paged_attention_partials", rfx::kStagePartials);
}

extern "C" int rfx_paged_attention_partials_final(const RfxPagedAttentionArgs* a) {
    using namespace rfx;
    if (validate(a, "rfx_paged_attention_partials_final") != RFX_SUCCESS) return RFX_INVALID_ARGUMENT;
    if (prefill_paged_supported(a) || !decode_mma_supported(a))
        return fail(RFX_NOT_IMPLEMENTED, "rfx_paged_attention_partials_final: only the decode kernel finishes its own rows");
    return run_stages(a, "rfx_paged_attention_partials_final", kStagePartials | kStageCombine);
}

extern "C" int rfx_paged_attention_kernel_kind(const RfxPagedAttentionArgs* a) {
    if (rfx::validate(a, "rfx_paged_attention_kernel_kind") != RFX_SUCCESS) return -1;
    if (rfx::prefill_paged_supported(a)) return rfx::prefill_paged_mixed(a) ? 3 : 2;
    return rfx::decode_mma_supported(a) ? 1 : 0;
}

extern "C" int rfx_paged_attention_combine(const RfxPagedAttentionArgs* a) {
    return rfx::run_stages(a, "rfx_paged_attention_combine", rfx::kStageCombine);
}

extern "C" int rfx_paged_attention_combine_gather(const RfxPagedAttentionArgs* a, const RfxHeadGatherArgs* g) {
    if (!g) return rfx::fail(RFX_INVALID_ARGUMENT, "rfx_paged_attention_combine_gather: null gather args");
    return rfx::run_stages(a, "rfx_paged_attention_combine_gather", rfx::kStageCombine, g);
}

extern "C" int rfx_paged_attention_gather(const RfxPagedAttentionArgs* a, const RfxHeadGatherArgs* g) {
    using namespace rfx;
    if (!g) return fail(RFX_INVALID_ARGUMENT, "rfx_paged_attention_gather: null gather args");
    const int plan = (a && a->reuse_plan) ? 0 : kStagePlan;
    return run_stages(a, "rfx_paged_attention_gather", plan | kStagePartials | kStageCombine, g);
}

// ---- paged attention without a caller workspace ----------------------------------------
// Scratch for rfx_paged_attention_static: one fixed array in device memory, part of the
// library image. Every GPU that loads the library holds these bytes until the process exits.
namespace rfx {
constexpr size_t kStaticScratchBytes = 8u << 20;  // 8 MiB
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];
// Device address of the array per device ordinal, resolved on the first call on that device. Two
// host threads may both resolve it; they store the same value.
static std::atomic<void*> g_static_scratch_ptr[64];

// In host code the array's name is only a handle; a kernel needs its device address.
static int static_scratch(const char* name, void** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(RFX_CUDA_ERROR, "%s: cudaGetDevice: %s", name, cudaGetErrorString(e));
    if (dev < 0 || dev >= 64) return fail(RFX_UNSUPPORTED_DEVICE, "%s: device ordinal %d out of range", name, dev);
    void* p = g_static_scratch_ptr[dev].load(std::memory_order_acquire);
    if (!p) {
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess || !p)
            return fail(RFX_CUDA_ERROR, "%s: cudaGetSymbolAddress: %s", name, cudaGetErrorString(e));
        g_static_scratch_ptr[dev].store(p, std::memory_order_release);
    }
    *out = p;
    return RFX_SUCCESS;
}
}  // namespace rfx

extern "C" size_t rfx_paged_attention_static_capacity(void) { return rfx::kStaticScratchBytes; }

extern "C" int rfx_paged_attention_static(const RfxPagedAttentionArgs* a) {
    using namespace rfx;
    const char* name = "rfx_paged_attention_static";
    int st = validate(a, name);
    if (st != RFX_SUCCESS) return st;
    st = check_device();
    if (st != RFX_SUCCESS) return st;
    const PlanLayout L = layout_of(a);
    if (L.total > kStaticScratchBytes)
        return fail(RFX_WORKSPACE_TOO_SMALL,
                    "%s: this problem needs %zu B of scratch, the built-in array holds %zu B; use "
                    "rfx_paged_attention with a caller workspace",
                    name, L.total, kStaticScratchBytes);
    void* scratch = nullptr;
    st = static_scratch(name, &scratch);
    if (st != RFX_SUCCESS) return st;
    RfxPagedAttentionArgs b = *a;
    b.workspace = scratch;
    b.workspace_bytes = kStaticScratchBytes;
    b.reuse_plan = 0;  // the array is shared by every caller: always plan afresh
    return run_stages(&b, name, kStagePlan | kStagePartials | kStageCombine);
}

extern "C" int rfx_paged_attention_status(const void* workspace, rfx_stream stream, int* status_word_host) {
    using namespace rfx;
    if (!status_word_host) return fail(RFX_INVALID_ARGUMENT, "rfx_paged_attention_status: null pointer");
    if (!workspace) {  // the built-in array of rfx_paged_attention_static on the current device
        void* p = nullptr;
        int st = static_scratch("rfx_paged_attention_status", &p);
        if (st != RFX_SUCCESS) return st;
        workspace = p;
    }
    int32_t w = 0;
    cudaError_t e = cudaMemcpyAsync(&w, (const int32_t*)workspace + HdrStatus, sizeof(w), cudaMemcpyDeviceToHost,
                                    as_stream(stream));
    if (e == cudaSuccess) e = cudaStreamSynchronize(as_stream(stream));
    if (e != cudaSuccess) return fail(RFX_CUDA_ERROR, "rfx_paged_attention_status: %s", cudaGetErrorString(e));
    *status_word_host = w;
    if (w & kStatusWaitExpired) return fail(RFX_TIMEOUT, "a bounded device-side wait expired (status word %d)", w);
    return RFX_SUCCESS;
}
