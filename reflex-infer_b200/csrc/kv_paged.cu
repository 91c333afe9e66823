// Paged KV pool movement: append / scatter (write rows by flat slot) and lookup (gather
// pages into dense tensors with a zero tail). Pure byte movement, so one template over
// the vector width; 16-byte accesses whenever pointers and strides allow it.
//
// Algorithmic bytes: append 2*N*H*D*e read + the same written (+8 B per slot);
// lookup 2*B*H*ctx*D*e read + 2*B*H*max_ctx*D*e written.
#include "common.cuh"

namespace rfx {

// One thread moves one VEC-typed piece of one (token, head) row, for K and for V.
template <typename VEC>
__global__ void __launch_bounds__(256)
kv_append_kernel(const VEC* __restrict__ k_in, const VEC* __restrict__ v_in,
                 VEC* __restrict__ k_cache, VEC* __restrict__ v_cache,
                 const int64_t* __restrict__ slots,
                 int64_t n_tokens, int heads, int vec_per_row, int64_t num_slots, int block_size,
                 int64_t in_sn, int64_t in_sh,              // strides in VEC units
                 int64_t c_sblk, int64_t c_sh, int64_t c_spos) {
    const int64_t total = n_tokens * heads * vec_per_row;
    // a 64-bit division costs about a hundred instructions, several per piece more than the copy
    // itself: below 2^31 pieces (and slots) the indices are taken apart in 32 bits
    const bool small = total < (1ll << 31) && num_slots < (1ll << 31);
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        int c, h;
        int64_t n;
        if (small) {
            uint32_t r = (uint32_t)i;
            c = (int)(r % (uint32_t)vec_per_row);
            r /= (uint32_t)vec_per_row;
            h = (int)(r % (uint32_t)heads);
            n = (int64_t)(r / (uint32_t)heads);
        } else {
            c = (int)(i % vec_per_row);
            const int64_t row = i / vec_per_row;
            h = (int)(row % heads);
            n = row / heads;
        }
        const int64_t slot = slots[n];
        if (slot < 0 || slot >= num_slots) continue;
        const int64_t page = small ? (int64_t)((uint32_t)slot / (uint32_t)block_size) : slot / block_size;
        const int pos = (int)(slot - page * block_size);
        const int64_t src = n * in_sn + h * in_sh + c;
        const int64_t dst = page * c_sblk + h * c_sh + pos * c_spos + c;
        k_cache[dst] = k_in[src];
        v_cache[dst] = v_in[src];
    }
}

// One thread writes one VEC piece of out[b, h, t, :] for K and V; t >= ctx_len -> zeros.
template <typename VEC>
__global__ void __launch_bounds__(256)
kv_lookup_kernel(const VEC* __restrict__ k_cache, const VEC* __restrict__ v_cache,
                 VEC* __restrict__ k_out, VEC* __restrict__ v_out,
                 const int64_t* __restrict__ block_table, const int32_t* __restrict__ ctx_lens,
                 int64_t batch, int heads, int64_t max_ctx, int vec_per_row,
                 int64_t num_blocks, int block_size, int64_t max_blocks, int64_t bt_sb,
                 int64_t c_sblk, int64_t c_sh, int64_t c_spos) {
    const int64_t total = batch * heads * max_ctx * vec_per_row;
    const bool small = total < (1ll << 31);  // then the index is taken apart in 32 bits (see kv_append_kernel)
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        int c, h;
        int64_t t, b, j;
        if (small) {
            uint32_t r = (uint32_t)i;
            c = (int)(r % (uint32_t)vec_per_row);
            r /= (uint32_t)vec_per_row;
            const uint32_t t32 = r % (uint32_t)max_ctx;
            r /= (uint32_t)max_ctx;
            h = (int)(r % (uint32_t)heads);
            b = (int64_t)(r / (uint32_t)heads);
            t = (int64_t)t32;
            j = (int64_t)(t32 / (uint32_t)block_size);
        } else {
            c = (int)(i % vec_per_row);
            int64_t r = i / vec_per_row;
            t = r % max_ctx;
            r /= max_ctx;
            h = (int)(r % heads);
            b = r / heads;
            j = t / block_size;
        }
        VEC kv, vv;
        memset(&kv, 0, sizeof(VEC));
        memset(&vv, 0, sizeof(VEC));
        if (t < (int64_t)ctx_lens[b] && j < max_blocks) {
            const int64_t page = block_table[b * bt_sb + j];
            if (page >= 0 && page < num_blocks) {
                const int pos = (int)(t - j * block_size);
                const int64_t src = page * c_sblk + h * c_sh + pos * c_spos + c;
                kv = k_cache[src];
                vv = v_cache[src];
            }
        }
        k_out[i] = kv;
        v_out[i] = vv;
    }
}

static inline bool aligned_to(const void* p, size_t a) { return ((uintptr_t)p % a) == 0; }

static int grid_for(int64_t total_threads) {
    int64_t blocks = ceil_div<int64_t>(total_threads, 256);
    const int64_t cap = (int64_t)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (int)blocks;
}

static int append_impl(const RfxKvAppendArgs* a, const char* name) {
    if (!a) return fail(RFX_INVALID_ARGUMENT, "%s: null args", name);
    RFX_REQUIRE(dtype_ok(a->dtype), "%s: unknown dtype %d", name, a->dtype);
    RFX_REQUIRE(a->n_tokens >= 0 && a->num_kv_heads > 0 && a->head_dim > 0 && a->num_blocks > 0 &&
                    a->block_size > 0,
                "%s: bad sizes N=%lld H=%lld D=%lld blocks=%lld bs=%lld", name, (long long)a->n_tokens,
                (long long)a->num_kv_heads, (long long)a->head_dim, (long long)a->num_blocks,
                (long long)a->block_size);
    if (a->n_tokens == 0) return RFX_SUCCESS;
    RFX_REQUIRE(a->k_in && a->v_in && a->k_cache && a->v_cache && a->slot_mapping, "%s: null pointer", name);
    int st = check_device();
    if (st != RFX_SUCCESS) return st;

    const size_t e = dtype_size(a->dtype);
    const size_t row_bytes = (size_t)a->head_dim * e;
    // Widest vector that divides the row and every stride and base address.
    size_t vec = 16;
    auto fits = [&](size_t v) {
        if (row_bytes % v) return false;
        const int64_t strides[] = {a->in_stride_n, a->in_stride_h, a->cache_stride_blk,
                                   a->cache_stride_h, a->cache_stride_pos};
        for (int64_t s : strides)
            if (((size_t)s * e) % v) return false;
        return aligned_to(a->k_in, v) && aligned_to(a->v_in, v) && aligned_to(a->k_cache, v) &&
               aligned_to(a->v_cache, v);
    };
    while (vec > e && !fits(vec)) vec /= 2;
    const int vpr = (int)(row_bytes / vec);
    const int64_t per = (int64_t)(vec / e);  // elements per vector
    const int64_t total = a->n_tokens * a->num_kv_heads * vpr;
    const int grid = grid_for(total);
    cudaStream_t s = as_stream(a->stream);
    const int64_t num_slots = a->num_blocks * a->block_size;

#define LAUNCH_APPEND(VEC)                                                                         \
    kv_append_kernel<VEC><<<grid, 256, 0, s>>>(                                                    \
        (const VEC*)a->k_in, (const VEC*)a->v_in, (VEC*)a->k_cache, (VEC*)a->v_cache,              \
        a->slot_mapping, a->n_tokens, (int)a->num_kv_heads, vpr, num_slots, (int)a->block_size,    \
        a->in_stride_n / per, a->in_stride_h / per, a->cache_stride_blk / per,                     \
        a->cache_stride_h / per, a->cache_stride_pos / per)
    switch (vec) {
        case 16: LAUNCH_APPEND(uint4); break;
        case 8: LAUNCH_APPEND(uint2); break;
        case 4: LAUNCH_APPEND(uint32_t); break;
        default: LAUNCH_APPEND(uint16_t); break;
    }
#undef LAUNCH_APPEND
    return check_launch(name);
}

}  // namespace rfx

extern "C" int rfx_kv_paged_append(const RfxKvAppendArgs* a) {
    return rfx::append_impl(a, "rfx_kv_paged_append");
}

extern "C" int rfx_kv_paged_scatter(const RfxKvAppendArgs* a) {
    return rfx::append_impl(a, "rfx_kv_paged_scatter");
}

extern "C" int rfx_kv_paged_lookup(const RfxKvLookupArgs* a) {
    using namespace rfx;
    const char* name = "rfx_kv_paged_lookup";
    if (!a) return fail(RFX_INVALID_ARGUMENT, "%s: null args", name);
    RFX_REQUIRE(dtype_ok(a->dtype), "%s: unknown dtype %d", name, a->dtype);
    RFX_REQUIRE(a->batch >= 0 && a->num_kv_heads > 0 && a->head_dim > 0 && a->num_blocks > 0 &&
                    a->block_size > 0 && a->max_ctx >= 0 && a->max_blocks >= 0,
                "%s: bad sizes", name);
    if (a->batch == 0 || a->max_ctx == 0) return RFX_SUCCESS;
    RFX_REQUIRE(a->k_cache && a->v_cache && a->k_out && a->v_out && a->block_table && a->context_lens,
                "%s: null pointer", name);
    int st = check_device();
    if (st != RFX_SUCCESS) return st;

    const size_t e = dtype_size(a->dtype);
    const size_t row_bytes = (size_t)a->head_dim * e;
    size_t vec = 16;
    auto fits = [&](size_t v) {
        if (row_bytes % v) return false;
        const int64_t strides[] = {a->cache_stride_blk, a->cache_stride_h, a->cache_stride_pos};
        for (int64_t s : strides)
            if (((size_t)s * e) % v) return false;
        return aligned_to(a->k_cache, v) && aligned_to(a->v_cache, v) && aligned_to(a->k_out, v) &&
               aligned_to(a->v_out, v);
    };
    while (vec > e && !fits(vec)) vec /= 2;
    const int vpr = (int)(row_bytes / vec);
    const int64_t per = (int64_t)(vec / e);
    const int64_t total = a->batch * a->num_kv_heads * a->max_ctx * vpr;
    const int grid = grid_for(total);
    cudaStream_t s = as_stream(a->stream);

#define LAUNCH_LOOKUP(VEC)                                                                        \
    kv_lookup_kernel<VEC><<<grid, 256, 0, s>>>(                                                   \
        (const VEC*)a->k_cache, (const VEC*)a->v_cache, (VEC*)a->k_out, (VEC*)a->v_out,           \
        a->block_table, a->context_lens, a->batch, (int)a->num_kv_heads, a->max_ctx, vpr,         \
        a->num_blocks, (int)a->block_size, a->max_blocks, a->bt_stride_b,                         \
        a->cache_stride_blk / per, a->cache_stride_h / per, a->cache_stride_pos / per)
    switch (vec) {
        case 16: LAUNCH_LOOKUP(uint4); break;
        case 8: LAUNCH_LOOKUP(uint2); break;
        case 4: LAUNCH_LOOKUP(uint32_t); break;
        default: LAUNCH_LOOKUP(uint16_t); break;
    }
#undef LAUNCH_LOOKUP
    return check_launch(name);
}
