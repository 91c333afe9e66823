// RoPE: table builder, standalone apply (both pair conventions, any strides, in or out
// of place) and the fused RoPE + paged append. All arithmetic goes through
// rope_pair<T>() so the result carries torch's per-op rounding and the KV pool ends up
// bit-identical to the reference's apply_rope -> kv_paged_append composition.
//
// Algorithmic bytes: apply 2*numel*e (+ tables); rope_append reads N*(H_q+2*H_kv)*D*e
// and writes the same.
#include "common.cuh"

namespace rfx {

template <typename T, int V> struct alignas(sizeof(T) * V) Pack { T v[V]; };

// Rotate one piece of one row. Half-rotated (INTER=false): piece p covers elements
// [p*V, p*V+V) of the first half and their partners half further on; both table factors
// come from the first half of the table row (triton_rope.py:226-227). Interleaved:
// piece p covers [p*V, p*V+V), pairs (2i, 2i+1), factors from the even entries (:218-219).
// 16-bit rows, two elements per instruction: same values as rope_pair (see Pair16). The kernels
// were bound by their instruction count (widen, multiply, round, widen again: ~14 per element).
template <typename T, int V, bool INTER>
__device__ inline void rope_piece_packed(const T* x, T* y, const T* __restrict__ cosr,
                                         const T* __restrict__ sinr, int D, int p) {
    using P = Pack<T, V>;
    using A = Pair16<T>;
    using W = typename A::P;
    const int o = p * V;
    if (INTER) {
        P xv = *reinterpret_cast<const P*>(x + o);
        P cv = *reinterpret_cast<const P*>(cosr + o);
        P sv = *reinterpret_cast<const P*>(sinr + o);
        P out;
        const W* xw = reinterpret_cast<const W*>(&xv);
        const W* cw = reinterpret_cast<const W*>(&cv);
        const W* sw = reinterpret_cast<const W*>(&sv);
        W* ow = reinterpret_cast<W*>(&out);
#pragma unroll
        for (int j = 0; j < V / 2; ++j) {
            // pair (x0, x1), factors from the even entry: y0 = x0 c - x1 s, y1 = x0 s + x1 c
            const float2 pc = A::widen(A::mul(xw[j], A::both_low(cw[j])));
            const float2 ps = A::widen(A::mul(xw[j], A::both_low(sw[j])));
            ow[j] = A::round(__fsub_rn(pc.x, ps.y), __fadd_rn(ps.x, pc.y));
        }
        *reinterpret_cast<P*>(y + o) = out;
    } else {
        const int half = D >> 1;
        P x1 = *reinterpret_cast<const P*>(x + o);
        P x2 = *reinterpret_cast<const P*>(x + half + o);
        P cv = *reinterpret_cast<const P*>(cosr + o);
        P sv = *reinterpret_cast<const P*>(sinr + o);
        P y1, y2;
        const W* x1w = reinterpret_cast<const W*>(&x1);
        const W* x2w = reinterpret_cast<const W*>(&x2);
        const W* cw = reinterpret_cast<const W*>(&cv);
        const W* sw = reinterpret_cast<const W*>(&sv);
        W* y1w = reinterpret_cast<W*>(&y1);
        W* y2w = reinterpret_cast<W*>(&y2);
#pragma unroll
        for (int j = 0; j < V / 2; ++j) {
            const float2 a = A::widen(A::mul(x1w[j], cw[j])), bb = A::widen(A::mul(x2w[j], sw[j]));
            const float2 c = A::widen(A::mul(x1w[j], sw[j])), d = A::widen(A::mul(x2w[j], cw[j]));
            y1w[j] = A::round(__fsub_rn(a.x, bb.x), __fsub_rn(a.y, bb.y));
            y2w[j] = A::round(__fadd_rn(c.x, d.x), __fadd_rn(c.y, d.y));
        }
        *reinterpret_cast<P*>(y + o) = y1;
        *reinterpret_cast<P*>(y + half + o) = y2;
    }
}

template <typename T, int V, bool INTER>
__device__ inline void rope_piece(const T* x, T* y, const T* __restrict__ cosr,
                                  const T* __restrict__ sinr, int D, int p) {
    using P = Pack<T, V>;
    if constexpr (sizeof(T) == 2 && V >= 2) {
        rope_piece_packed<T, V, INTER>(x, y, cosr, sinr, D, p);
        return;
    }
    if (INTER) {
        const int o = p * V;
        P xv = *reinterpret_cast<const P*>(x + o);
        P cv = *reinterpret_cast<const P*>(cosr + o);
        P sv = *reinterpret_cast<const P*>(sinr + o);
        P out;
#pragma unroll
        for (int j = 0; j < V; j += 2)
            rope_pair<T>(xv.v[j], xv.v[j + 1], cv.v[j], sv.v[j], out.v[j], out.v[j + 1]);
        *reinterpret_cast<P*>(y + o) = out;
    } else {
        const int half = D >> 1;
        const int o = p * V;
        P x1 = *reinterpret_cast<const P*>(x + o);
        P x2 = *reinterpret_cast<const P*>(x + half + o);
        P cv = *reinterpret_cast<const P*>(cosr + o);
        P sv = *reinterpret_cast<const P*>(sinr + o);
        P y1, y2;
#pragma unroll
        for (int j = 0; j < V; ++j) rope_pair<T>(x1.v[j], x2.v[j], cv.v[j], sv.v[j], y1.v[j], y2.v[j]);
        *reinterpret_cast<P*>(y + o) = y1;
        *reinterpret_cast<P*>(y + half + o) = y2;
    }
}

template <typename T, int V, bool INTER>
__device__ inline void copy_piece(const T* __restrict__ x, T* y, int D, int p) {
    using P = Pack<T, V>;
    const int o = p * V;
    if (INTER) {
        *reinterpret_cast<P*>(y + o) = *reinterpret_cast<const P*>(x + o);
    } else {
        const int half = D >> 1;
        *reinterpret_cast<P*>(y + o) = *reinterpret_cast<const P*>(x + o);
        *reinterpret_cast<P*>(y + half + o) = *reinterpret_cast<const P*>(x + half + o);
    }
}

template <typename T, int V, bool INTER>
__global__ void __launch_bounds__(256)
rope_apply_kernel(const T* x, T* y, const T* __restrict__ cosb, const T* __restrict__ sinb,
                  int64_t B, int64_t S, int H, int D, int pieces,
                  int64_t xsb, int64_t xss, int64_t xsh, int64_t ysb, int64_t yss, int64_t ysh,
                  int64_t tss) {
    const int64_t total = B * S * H * pieces;
    // 64-bit divisions cost a few hundred instructions per piece, more than the rotation itself:
    // below 2^31 pieces the index is taken apart in 32 bits
    const bool small = total < (1ll << 31);
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        int p, h;
        int64_t s, b;
        if (small) {
            uint32_t r = (uint32_t)i;
            p = (int)(r % (uint32_t)pieces);
            r /= (uint32_t)pieces;
            h = (int)(r % (uint32_t)H);
            r /= (uint32_t)H;
            s = (int64_t)(r % (uint32_t)S);
            b = (int64_t)(r / (uint32_t)S);
        } else {
            p = (int)(i % pieces);
            int64_t r = i / pieces;
            h = (int)(r % H);
            r /= H;
            s = r % S;
            b = r / S;
        }
        rope_piece<T, V, INTER>(x + b * xsb + s * xss + h * xsh, y + b * ysb + s * yss + h * ysh,
                                cosb + s * tss, sinb + s * tss, D, p);
    }
}

// Rows of token n: [0, Hkv) K rotate -> pool, [Hkv, 2Hkv) V copy -> pool, then Hq Q rows.
template <typename T, int V, bool INTER>
__global__ void __launch_bounds__(256)
rope_append_kernel(const T* __restrict__ k_in, const T* __restrict__ v_in, const T* q_in,
                   T* q_out, T* __restrict__ k_cache, T* __restrict__ v_cache,
                   const int64_t* __restrict__ slots, const int32_t* __restrict__ positions,
                   const T* __restrict__ cosb, const T* __restrict__ sinb,
                   int64_t N, int Hq, int Hkv, int D, int pieces, int64_t num_slots, int block_size,
                   int64_t table_rows, int64_t c_sblk, int64_t c_sh, int64_t c_spos) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // the split-K plan may start alongside
    const int rows_per_tok = 2 * Hkv + Hq;
    const int64_t total = N * rows_per_tok * pieces;
    const bool small = total < (1ll << 31);  // then the index is taken apart in 32 bits (see rope_apply_kernel)
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        int p, row;
        int64_t n;
        if (small) {
            uint32_t r = (uint32_t)i;
            p = (int)(r % (uint32_t)pieces);
            r /= (uint32_t)pieces;
            row = (int)(r % (uint32_t)rows_per_tok);
            n = (int64_t)(r / (uint32_t)rows_per_tok);
        } else {
            p = (int)(i % pieces);
            const int64_t r = i / pieces;
            row = (int)(r % rows_per_tok);
            n = r / rows_per_tok;
        }
        int64_t pos = positions[n];
        if (pos < 0 || pos >= table_rows) continue;  // no table row: leave the token untouched
        const T* cr = cosb + pos * D;
        const T* sr = sinb + pos * D;
        if (row < 2 * Hkv) {
            const int64_t slot = slots[n];
            if (slot < 0 || slot >= num_slots) continue;
            const int64_t page = slot / block_size;
            const int at = (int)(slot - page * block_size);
            if (row < Hkv) {
                const int h = row;
                rope_piece<T, V, INTER>(k_in + (n * Hkv + h) * D,
                                        k_cache + page * c_sblk + h * c_sh + at * c_spos, cr, sr, D, p);
            } else {
                const int h = row - Hkv;
                copy_piece<T, V, INTER>(v_in + (n * Hkv + h) * D,
                                        v_cache + page * c_sblk + h * c_sh + at * c_spos, D, p);
            }
        } else {
            const int h = row - 2 * Hkv;
            rope_piece<T, V, INTER>(q_in + (n * Hq + h) * D, q_out + (n * Hq + h) * D, cr, sr, D, p);
        }
    }
}

// Fused RoPE + append into an int8 pool: one warp per row of a token -- [0, Hkv) K rotate and
// quantise, [Hkv, 2Hkv) V quantise, then Hq Q rows rotated in T. The rotation carries the same per-op
// rounding as above, so the values that are quantised are the rows the 16-bit pool would hold.
// Quantiser (fp32): scale = max|x| / 127 (1 for an all-zero row), q = rint(x / scale).
template <typename T, bool INTER>
__global__ void __launch_bounds__(256)
rope_append_q8_kernel(const T* __restrict__ k_in, const T* __restrict__ v_in, const T* q_in, T* q_out,
                      int8_t* __restrict__ k_cache, int8_t* __restrict__ v_cache, float* __restrict__ k_scales,
                      float* __restrict__ v_scales, const int64_t* __restrict__ slots,
                      const int32_t* __restrict__ positions, const T* __restrict__ cosb,
                      const T* __restrict__ sinb, int64_t N, int Hq, int Hkv, int D, int64_t num_slots,
                      int block_size, int64_t table_rows) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // the split-K plan may start alongside
    constexpr int kMaxPairs = 4;  // head_dim <= 256: at most 4 pairs per lane
    const int lane = threadIdx.x & 31;
    const int rows_per_tok = 2 * Hkv + Hq;
    const int64_t total = N * rows_per_tok;
    const int half = D >> 1;
    for (int64_t w = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5; w < total;
         w += ((int64_t)gridDim.x * blockDim.x) >> 5) {
        const int row = (int)(w % rows_per_tok);
        const int64_t n = w / rows_per_tok;
        const int64_t pos = positions[n];
        if (pos < 0 || pos >= table_rows) continue;  // no table row: leave the token untouched
        const bool is_v = row >= Hkv && row < 2 * Hkv;
        const bool is_q = row >= 2 * Hkv;
        const int h = is_q ? row - 2 * Hkv : (is_v ? row - Hkv : row);
        const T* x = is_q ? q_in + (n * Hq + h) * D : (is_v ? v_in : k_in) + (n * Hkv + h) * D;
        // element pairs (d1, d2) of this lane, rotated unless this is a V row
        float y1[kMaxPairs], y2[kMaxPairs];
        T t1[kMaxPairs], t2[kMaxPairs];
        float amax = 0.f;
#pragma unroll
        for (int k = 0; k < kMaxPairs; ++k) {
            const int p = lane + 32 * k;
            y1[k] = y2[k] = 0.f;
            if (p >= half) continue;
            const int d1 = INTER ? 2 * p : p, d2 = INTER ? 2 * p + 1 : p + half;
            T a = x[d1], b = x[d2];
            if (!is_v) {
                const T* cr = cosb + pos * D;
                const T* sr = sinb + pos * D;
                T r1, r2;
                rope_pair<T>(a, b, cr[d1], sr[d1], r1, r2);
                a = r1; b = r2;
            }
            t1[k] = a; t2[k] = b;
            y1[k] = Num<T>::to_f(a); y2[k] = Num<T>::to_f(b);
            amax = fmaxf(amax, fmaxf(fabsf(y1[k]), fabsf(y2[k])));
        }
        if (is_q) {
            T* y = q_out + (n * Hq + h) * D;
#pragma unroll
            for (int k = 0; k < kMaxPairs; ++k) {
                const int p = lane + 32 * k;
                if (p >= half) continue;
                y[INTER ? 2 * p : p] = t1[k];
                y[INTER ? 2 * p + 1 : p + half] = t2[k];
            }
            continue;
        }
        const int64_t slot = slots[n];
        if (slot < 0 || slot >= num_slots) continue;
        const int64_t page = slot / block_size;
        const int at = (int)(slot - page * block_size);
        amax = warp_max(amax);
        const float scale = amax > 0.f ? __fdiv_rn(amax, 127.f) : 1.f;
        const int64_t r = (page * Hkv + h) * block_size + at;
        int8_t* dst = (is_v ? v_cache : k_cache) + r * D;
        if (lane == 0) (is_v ? v_scales : k_scales)[r] = scale;
#pragma unroll
        for (int k = 0; k < kMaxPairs; ++k) {
            const int p = lane + 32 * k;
            if (p >= half) continue;
            const float q1 = fminf(127.f, fmaxf(-127.f, rintf(__fdiv_rn(y1[k], scale))));
            const float q2 = fminf(127.f, fmaxf(-127.f, rintf(__fdiv_rn(y2[k], scale))));
            dst[INTER ? 2 * p : p] = (int8_t)q1;
            dst[INTER ? 2 * p + 1 : p + half] = (int8_t)q2;
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
rope_table_kernel(T* __restrict__ cosb, T* __restrict__ sinb, const float* __restrict__ inv_freq,
                  int64_t S, int D, double base, int interleaved) {
    const int half = D >> 1;
    const int64_t total = S * half;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int j = (int)(i % half);
        const int64_t s = i / half;
        float theta;
        if (inv_freq) {
            theta = inv_freq[j];
        } else {
            const float e = __fdiv_rn((float)j, (float)half);
            theta = __fdiv_rn(1.0f, (float)pow(base, (double)e));
        }
        const float ang = __fmul_rn((float)s, theta);
        const float c = (float)cos((double)ang);
        const float sn = (float)sin((double)ang);
        const T ct = Num<T>::from_f(c), st = Num<T>::from_f(sn);
        T* cr = cosb + s * D;
        T* sr = sinb + s * D;
        if (interleaved) {
            cr[2 * j] = ct; cr[2 * j + 1] = ct;
            sr[2 * j] = st; sr[2 * j + 1] = st;
        } else {
            cr[j] = ct; cr[j + half] = ct;
            sr[j] = st; sr[j + half] = st;
        }
    }
}

static int grid_for(int64_t total_threads) {
    int64_t blocks = ceil_div<int64_t>(total_threads, 256);
    const int64_t cap = (int64_t)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (int)blocks;
}

// Largest V in {8,4,2,1} (>=2 when interleaved) such that V*e divides `unit` elements*e
// and every listed byte quantity.
static int pick_v(int unit_elems, size_t e, bool inter, const size_t* quantities, int nq) {
    for (int v = 8; v >= 1; v >>= 1) {
        if (v * e > 16) continue;
        if (inter && v < 2) break;
        if (unit_elems % v) continue;
        bool ok = true;
        for (int i = 0; i < nq; ++i)
            if (quantities[i] % (v * e)) ok = false;
        if (ok) return v;
    }
    return inter ? 0 : 1;
}

}  // namespace rfx

extern "C" int rfx_rope_apply(const RfxRopeArgs* a) {
    using namespace rfx;
    const char* name = "rfx_rope_apply";
    if (!a) return fail(RFX_INVALID_ARGUMENT, "%s: null args", name);
    RFX_REQUIRE(dtype_ok(a->dtype), "%s: unknown dtype %d", name, a->dtype);
    RFX_REQUIRE(a->head_dim > 0 && a->head_dim % 2 == 0, "head_dim must be even for RoPE");
    RFX_REQUIRE(a->batch >= 0 && a->seq >= 0 && a->heads >= 0, "%s: bad sizes", name);
    if (a->batch * a->seq * a->heads == 0) return RFX_SUCCESS;
    RFX_REQUIRE(a->x && a->y && a->cos && a->sin, "%s: null pointer", name);
    int st = check_device();
    if (st != RFX_SUCCESS) return st;
    const size_t e = dtype_size(a->dtype);
    const int D = (int)a->head_dim;
    const bool inter = a->interleaved != 0;
    const size_t q[] = {(size_t)a->x,
                        (size_t)a->y,
                        (size_t)a->cos,
                        (size_t)a->sin,
                        (size_t)a->x_stride_b * e,
                        (size_t)a->x_stride_s * e,
                        (size_t)a->x_stride_h * e,
                        (size_t)a->y_stride_b * e,
                        (size_t)a->y_stride_s * e,
                        (size_t)a->y_stride_h * e,
                        (size_t)a->table_stride_s * e,
                        (size_t)(D / 2) * e * (inter ? 2 : 1)};
    const int V = pick_v(inter ? D : D / 2, e, inter, q, (int)(sizeof(q) / sizeof(q[0])));
    RFX_REQUIRE(V > 0, "%s: interleaved RoPE needs 2-element alignment of x, y and the tables", name);
    const int pieces = (inter ? D : D / 2) / V;
    const int64_t total = a->batch * a->seq * a->heads * pieces;
    const int grid = grid_for(total);
    cudaStream_t s = as_stream(a->stream);

#define RFX_ROPE_LAUNCH(T, VV, II)                                                               \
    rope_apply_kernel<T, VV, II><<<grid, 256, 0, s>>>(                                           \
        (const T*)a->x, (T*)a->y, (const T*)a->cos, (const T*)a->sin, a->batch, a->seq,          \
        (int)a->heads, D, pieces, a->x_stride_b, a->x_stride_s, a->x_stride_h, a->y_stride_b,    \
        a->y_stride_s, a->y_stride_h, a->table_stride_s)
#define RFX_ROPE_V(T, II)                                            \
    switch (V) {                                                     \
        case 8: if (sizeof(T) == 2) { RFX_ROPE_LAUNCH(T, (sizeof(T) == 2 ? 8 : 4), II); break; } \
        case 4: RFX_ROPE_LAUNCH(T, 4, II); break;                    \
        case 2: RFX_ROPE_LAUNCH(T, 2, II); break;                    \
        default: RFX_ROPE_LAUNCH(T, (II ? 2 : 1), II); break;        \
    }
    RFX_DISPATCH_DTYPE(a->dtype, T, {
        if (inter) { RFX_ROPE_V(T, true) } else { RFX_ROPE_V(T, false) }
    });
#undef RFX_ROPE_V
#undef RFX_ROPE_LAUNCH
    return check_launch(name);
}

extern "C" int rfx_rope_build_tables(const RfxRopeTableArgs* a) {
    using namespace rfx;
    const char* name = "rfx_rope_build_tables";
    if (!a) return fail(RFX_INVALID_ARGUMENT, "%s: null args", name);
    RFX_REQUIRE(dtype_ok(a->dtype), "%s: unknown dtype %d", name, a->dtype);
    RFX_REQUIRE(a->head_dim > 0 && a->head_dim % 2 == 0, "head_dim must be even for RoPE");
    RFX_REQUIRE(a->seq_len >= 0, "%s: negative seq_len", name);
    RFX_REQUIRE(a->inv_freq || a->base > 0.0, "%s: base must be positive", name);
    if (a->seq_len == 0) return RFX_SUCCESS;
    RFX_REQUIRE(a->cos && a->sin, "%s: null pointer", name);
    int st = check_device();
    if (st != RFX_SUCCESS) return st;
    const int64_t total = a->seq_len * (a->head_dim / 2);
    const int grid = grid_for(total);
    cudaStream_t s = as_stream(a->stream);
    RFX_DISPATCH_DTYPE(a->dtype, T, {
        rope_table_kernel<T><<<grid, 256, 0, s>>>((T*)a->cos, (T*)a->sin, a->inv_freq, a->seq_len,
                                                 (int)a->head_dim, a->base, a->interleaved);
    });
    return check_launch(name);
}

extern "C" int rfx_rope_append(const RfxRopeAppendArgs* a) {
    using namespace rfx;
    const char* name = "rfx_rope_append";
    if (!a) return fail(RFX_INVALID_ARGUMENT, "%s: null args", name);
    RFX_REQUIRE(dtype_ok(a->dtype), "%s: unknown dtype %d", name, a->dtype);
    RFX_REQUIRE(a->head_dim > 0 && a->head_dim % 2 == 0, "head_dim must be even for RoPE");
    RFX_REQUIRE(a->n_tokens >= 0 && a->num_kv_heads > 0 && a->num_blocks > 0 && a->block_size > 0 &&
                    a->table_rows >= 0 && a->num_q_heads >= 0,
                "%s: bad sizes", name);
    if (a->n_tokens == 0) return RFX_SUCCESS;
    RFX_REQUIRE(a->k_in && a->v_in && a->k_cache && a->v_cache && a->slot_mapping && a->positions &&
                    a->cos && a->sin,
                "%s: null pointer", name);
    const bool has_q = a->q_in != nullptr;
    RFX_REQUIRE(!has_q || (a->q_out && a->num_q_heads > 0), "%s: q_in given without q_out / num_q_heads", name);
    int st = check_device();
    if (st != RFX_SUCCESS) return st;
    const size_t e = dtype_size(a->dtype);
    const int D = (int)a->head_dim;
    const bool inter = a->interleaved != 0;
    if (a->kv_int8) {
        RFX_REQUIRE(a->k_scales && a->v_scales, "%s: an int8 pool needs k_scales and v_scales", name);
        RFX_REQUIRE(D <= 256, "%s: head_dim %d > 256", name, D);
        const int Hq8 = has_q ? (int)a->num_q_heads : 0;
        const int64_t warps = a->n_tokens * (2 * a->num_kv_heads + Hq8);
        const int grid8 = grid_for(warps * 32);
        cudaStream_t s8 = as_stream(a->stream);
#define RFX_RA8(T, II)                                                                                        \
    rope_append_q8_kernel<T, II><<<grid8, 256, 0, s8>>>(                                                      \
        (const T*)a->k_in, (const T*)a->v_in, (const T*)a->q_in, (T*)a->q_out, (int8_t*)a->k_cache,           \
        (int8_t*)a->v_cache, a->k_scales, a->v_scales, a->slot_mapping, a->positions, (const T*)a->cos,       \
        (const T*)a->sin, a->n_tokens, Hq8, (int)a->num_kv_heads, D, a->num_blocks * a->block_size,           \
        (int)a->block_size, a->table_rows)
        RFX_DISPATCH_DTYPE(a->dtype, T, {
            if (inter) RFX_RA8(T, true); else RFX_RA8(T, false);
        });
#undef RFX_RA8
        return check_launch(name);
    }
    const size_t q[] = {(size_t)a->k_in,
                        (size_t)a->v_in,
                        (size_t)a->q_in,
                        (size_t)a->q_out,
                        (size_t)a->k_cache,
                        (size_t)a->v_cache,
                        (size_t)a->cos,
                        (size_t)a->sin,
                        (size_t)D * e,
                        (size_t)a->cache_stride_blk * e,
                        (size_t)a->cache_stride_h * e,
                        (size_t)a->cache_stride_pos * e,
                        (size_t)(D / 2) * e * (inter ? 2 : 1)};
    const int V = pick_v(inter ? D : D / 2, e, inter, q, (int)(sizeof(q) / sizeof(q[0])));
    RFX_REQUIRE(V > 0, "%s: interleaved RoPE needs 2-element alignment", name);
    const int pieces = (inter ? D : D / 2) / V;
    const int Hq = has_q ? (int)a->num_q_heads : 0;
    const int64_t total = a->n_tokens * (2 * a->num_kv_heads + Hq) * pieces;
    const int grid = grid_for(total);
    cudaStream_t s = as_stream(a->stream);
    const int64_t num_slots = a->num_blocks * a->block_size;

#define RFX_RA_LAUNCH(T, VV, II)                                                                   \
    rope_append_kernel<T, VV, II><<<grid, 256, 0, s>>>(                                            \
        (const T*)a->k_in, (const T*)a->v_in, (const T*)a->q_in, (T*)a->q_out, (T*)a->k_cache,     \
        (T*)a->v_cache, a->slot_mapping, a->positions, (const T*)a->cos, (const T*)a->sin,         \
        a->n_tokens, Hq, (int)a->num_kv_heads, D, pieces, num_slots, (int)a->block_size,           \
        a->table_rows, a->cache_stride_blk, a->cache_stride_h, a->cache_stride_pos)
#define RFX_RA_V(T, II)                                              \
    switch (V) {                                                     \
        case 8: if (sizeof(T) == 2) { RFX_RA_LAUNCH(T, (sizeof(T) == 2 ? 8 : 4), II); break; } \
        case 4: RFX_RA_LAUNCH(T, 4, II); break;                      \
        case 2: RFX_RA_LAUNCH(T, 2, II); break;                      \
        default: RFX_RA_LAUNCH(T, (II ? 2 : 1), II); break;          \
    }
    RFX_DISPATCH_DTYPE(a->dtype, T, {
        if (inter) { RFX_RA_V(T, true) } else { RFX_RA_V(T, false) }
    });
#undef RFX_RA_V
#undef RFX_RA_LAUNCH
    return check_launch(name);
}
