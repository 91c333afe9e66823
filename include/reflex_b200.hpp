// reflex_b200.hpp -- header-only C++ face of libreflex_b200.so in the style of the reference's
// C++ API (include/reflex/infer.h): an `enum class Status` with the reference's six codes first
// (infer.h:16-23), plain argument structs with defaulted fields, `StreamHandle` (infer.h:92),
// and free functions taking `const Args&`. It adds the paged decode entry the reference's
// `KernelSupport::paged_decode_attention` flag (infer.h:81-90) reserves but does not implement.
// Everything forwards to the C ABI in reflex_b200.h; nothing here allocates.
#ifndef REFLEX_B200_HPP_
#define REFLEX_B200_HPP_

#include <cstddef>
#include <cstdint>

#include "reflex_b200.h"

namespace reflex::b200 {

enum class Status : std::uint8_t {
    Success = RFX_SUCCESS,
    UnsupportedDevice = RFX_UNSUPPORTED_DEVICE,
    UnsupportedModel = RFX_UNSUPPORTED_MODEL,
    UnsupportedQuantFormat = RFX_UNSUPPORTED_QUANT_FORMAT,
    InvalidArgument = RFX_INVALID_ARGUMENT,
    NotImplemented = RFX_NOT_IMPLEMENTED,
    CudaError = RFX_CUDA_ERROR,
    Timeout = RFX_TIMEOUT,
    WorkspaceTooSmall = RFX_WORKSPACE_TOO_SMALL,
};

using StreamHandle = void*;

enum class DType : int { F32 = RFX_F32, BF16 = RFX_BF16, F16 = RFX_F16 };

// What this library provides of the reference's KernelSupport list (infer.h:81-90).
struct KernelSupport {
    bool decode_attention = true;
    bool paged_decode_attention = true;
    bool rope = true;
    bool kv_convert = true;   // int8 KV with per-position scales: written by rfx_rope_append, read by paged decode
};
inline KernelSupport kernel_support() { return {}; }

// Paged GQA decode: one new query row per request against K/V pages
// [num_blocks, n_kv_heads, block_size, head_dim]. Field names follow AttentionDecodeArgs
// (infer.h:189-203); the page-table fields follow kernels/kv_cache/triton_kv_paged.py:9-15.
struct PagedAttentionDecodeArgs {
    void* output = nullptr;             // [batch, n_heads, head_dim]
    const void* q = nullptr;            // [batch, n_heads, head_dim]
    const void* k_cache = nullptr;
    const void* v_cache = nullptr;
    const std::int64_t* block_table = nullptr;  // [batch, max_blocks]
    const std::int32_t* context_lens = nullptr; // [batch]
    int batch = 0;
    int n_heads = 0;
    int n_kv_heads = 0;
    int head_dim = 0;
    std::int64_t num_blocks = 0;
    int block_size = 0;
    int max_blocks = 0;
    float scale = 1.0f;
    DType dtype = DType::BF16;
    // optional RoPE fused into the Q load: tables [table_rows, head_dim] in `dtype`, positions [batch]
    const void* rope_cos = nullptr;
    const void* rope_sin = nullptr;
    const std::int32_t* rope_positions = nullptr;
    std::int64_t table_rows = 0;
    bool rope_interleaved = false;
    void* workspace = nullptr;          // paged_decode_workspace_bytes(args) bytes, 256-byte aligned
    std::size_t workspace_bytes = 0;
    StreamHandle stream = nullptr;
    // int8 pool, as AttentionDecodeArgs::kv_int8 / k_scales / v_scales (infer.h:199-201): caches int8,
    // one fp32 scale per (page, kv head, position), scales [num_blocks, n_kv_heads, block_size]
    bool kv_int8 = false;
    const float* k_scales = nullptr;
    const float* v_scales = nullptr;
};

namespace detail {
inline RfxPagedAttentionArgs to_c(const PagedAttentionDecodeArgs& a) {
    RfxPagedAttentionArgs c = {};
    c.q = a.q; c.out = a.output; c.k_cache = a.k_cache; c.v_cache = a.v_cache;
    c.block_table = a.block_table; c.context_lens = a.context_lens;
    c.rope_cos = a.rope_cos; c.rope_sin = a.rope_sin; c.rope_positions = a.rope_positions;
    c.n_q = a.batch; c.batch = a.batch; c.num_q_heads = a.n_heads; c.num_kv_heads = a.n_kv_heads;
    c.head_dim = a.head_dim; c.num_blocks = a.num_blocks; c.block_size = a.block_size;
    c.max_blocks = a.max_blocks; c.bt_stride_b = a.max_blocks; c.table_rows = a.table_rows;
    c.max_q_len = 1; c.sm_scale = a.scale; c.is_causal = 1; c.rope_interleaved = a.rope_interleaved ? 1 : 0;
    c.dtype = static_cast<int>(a.dtype);
    c.workspace = a.workspace; c.workspace_bytes = a.workspace_bytes; c.stream = a.stream;
    c.kv_int8 = a.kv_int8 ? 1 : 0; c.k_scales = a.k_scales; c.v_scales = a.v_scales;
    return c;
}
}  // namespace detail

inline std::size_t paged_decode_workspace_bytes(const PagedAttentionDecodeArgs& a) {
    const RfxPagedAttentionArgs c = detail::to_c(a);
    return rfx_paged_attention_workspace_bytes(&c);
}

inline Status paged_flash_attention_decode(const PagedAttentionDecodeArgs& a) {
    const RfxPagedAttentionArgs c = detail::to_c(a);
    return static_cast<Status>(rfx_paged_attention(&c));
}

inline const char* last_error() { return rfx_last_error(); }

}  // namespace reflex::b200

#endif  // REFLEX_B200_HPP_
