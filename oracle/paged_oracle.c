/* CPU oracle in plain C for the integer / byte part of reflex-infer's paged-KV path and
 * an independent scalar statement of its floating-point ops. TEST INFRASTRUCTURE ONLY:
 * built by oracle/Makefile into oracle/_build/libpaged_oracle.so and loaded by the tests;
 * the product never links or calls it.
 *
 * Pinned against vectors generated from the reference's torch path
 * (tests/golden/make_golden.py) in tests/test_oracle_golden.py.
 *
 * Elements are handled as opaque `esize`-byte items for the copy ops. 16-bit floating
 * values are bf16 bit patterns (uint16_t) converted through float with round-to-nearest-
 * even, the conversion torch applies after every eager op.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* cache[slot / bs, h, slot % bs, :] = in[n, h, :]; follows torch_reference_kv_paged_append,
 * kernels/kv_cache/triton_kv_paged.py:279-292, including Python floor-division/modulo for
 * negative slots (they wrap from the end of the pool). Returns -1 on an out-of-range slot,
 * where torch raises IndexError. */
int oracle_kv_append(const uint8_t* k_in, const uint8_t* v_in, uint8_t* k_cache, uint8_t* v_cache,
                     const int64_t* slots, int64_t n, int64_t heads, int64_t dim, int64_t num_blocks,
                     int64_t bs, int64_t esize) {
    const int64_t row = dim * esize;
    for (int64_t i = 0; i < n; ++i) {
        int64_t slot = slots[i];
        int64_t page = slot / bs, pos = slot % bs;
        if (pos < 0) { pos += bs; page -= 1; }   /* floor semantics */
        if (page < 0) page += num_blocks;        /* negative index wraps once */
        if (page < 0 || page >= num_blocks) return -1;
        for (int64_t h = 0; h < heads; ++h) {
            const int64_t dst = ((page * heads + h) * bs + pos) * row;
            const int64_t src = (i * heads + h) * row;
            memcpy(k_cache + dst, k_in + src, (size_t)row);
            memcpy(v_cache + dst, v_in + src, (size_t)row);
        }
    }
    return 0;
}

/* out[b, h, t, :] = cache[block_table[b, t / bs], h, t % bs, :] for t < ctx[b], else zero;
 * follows torch_reference_kv_paged_lookup, kernels/kv_cache/triton_kv_paged.py:295-317. */
int oracle_kv_lookup(const uint8_t* k_cache, const uint8_t* v_cache, uint8_t* k_out, uint8_t* v_out,
                     const int64_t* block_table, const int32_t* ctx, int64_t batch, int64_t heads,
                     int64_t dim, int64_t num_blocks, int64_t bs, int64_t max_ctx, int64_t max_blocks,
                     int64_t esize) {
    const int64_t row = dim * esize;
    memset(k_out, 0, (size_t)(batch * heads * max_ctx * row));
    memset(v_out, 0, (size_t)(batch * heads * max_ctx * row));
    for (int64_t b = 0; b < batch; ++b) {
        for (int64_t t = 0; t < ctx[b]; ++t) {
            if (t >= max_ctx || t / bs >= max_blocks) return -1;
            const int64_t page = block_table[b * max_blocks + t / bs];
            if (page < 0 || page >= num_blocks) return -1;
            for (int64_t h = 0; h < heads; ++h) {
                const int64_t src = ((page * heads + h) * bs + t % bs) * row;
                const int64_t dst = ((b * heads + h) * max_ctx + t) * row;
                memcpy(k_out + dst, k_cache + src, (size_t)row);
                memcpy(v_out + dst, v_cache + src, (size_t)row);
            }
        }
    }
    return 0;
}

static float bf16_to_f(uint16_t v) {
    uint32_t u = (uint32_t)v << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

static uint16_t f_to_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40); /* NaN */
    u += 0x7fffu + ((u >> 16) & 1u); /* round to nearest even */
    return (uint16_t)(u >> 16);
}

/* Half-rotated or interleaved RoPE on bf16 rows with bf16 tables, every product and sum
 * rounded to bf16: the eager sequence of torch_reference_rope,
 * kernels/rope/triton_rope.py:216-240. x, y: [rows, dim]; table row for x row r is pos[r]. */
void oracle_rope_bf16(const uint16_t* x, uint16_t* y, const uint16_t* cos_t, const uint16_t* sin_t,
                      const int32_t* pos, int64_t rows, int64_t dim, int interleaved) {
    const int64_t half = dim / 2;
    for (int64_t r = 0; r < rows; ++r) {
        const uint16_t* xr = x + r * dim;
        uint16_t* yr = y + r * dim;
        const uint16_t* c = cos_t + (int64_t)pos[r] * dim;
        const uint16_t* s = sin_t + (int64_t)pos[r] * dim;
        for (int64_t i = 0; i < half; ++i) {
            const int64_t d1 = interleaved ? 2 * i : i, d2 = interleaved ? 2 * i + 1 : i + half;
            const float x1 = bf16_to_f(xr[d1]), x2 = bf16_to_f(xr[d2]);
            const float cc = bf16_to_f(c[d1]), ss = bf16_to_f(s[d1]);
            volatile float p1 = bf16_to_f(f_to_bf16(x1 * cc));
            volatile float p2 = bf16_to_f(f_to_bf16(x2 * ss));
            volatile float p3 = bf16_to_f(f_to_bf16(x1 * ss));
            volatile float p4 = bf16_to_f(f_to_bf16(x2 * cc));
            yr[d1] = f_to_bf16(p1 - p2);
            yr[d2] = f_to_bf16(p3 + p4);
        }
    }
}

/* One attention row in double: out[d] = sum_j softmax_j(scale * q.k_j) v_j[d] over n keys
 * given as row pointers into float arrays; the naive softmax(QK^T/sqrt(d))V. */
void oracle_attention_row_f64(const float* q, const float* k, const float* v, int64_t n, int64_t dim,
                              double scale, double* out) {
    double* s = (double*)malloc(sizeof(double) * (size_t)(n > 0 ? n : 1));
    double m = -INFINITY;
    for (int64_t j = 0; j < n; ++j) {
        double acc = 0.0;
        for (int64_t d = 0; d < dim; ++d) acc += (double)q[d] * (double)k[j * dim + d];
        s[j] = acc * scale;
        if (s[j] > m) m = s[j];
    }
    double l = 0.0;
    for (int64_t d = 0; d < dim; ++d) out[d] = 0.0;
    for (int64_t j = 0; j < n; ++j) {
        const double p = exp(s[j] - m);
        l += p;
        for (int64_t d = 0; d < dim; ++d) out[d] += p * (double)v[j * dim + d];
    }
    if (l > 0.0)
        for (int64_t d = 0; d < dim; ++d) out[d] /= l;
    free(s);
}
