// Row softmax / log-softmax (the public online_softmax op). Bandwidth-bound: 2*numel*e
// bytes (benchmark/bench_softmax.py:34), every element read once and written once.
//   * rows whose 16-byte vectors divide evenly (and up to 16 K elements): the row lives in
//     registers -- fp32 rows as they are, 16-bit rows in their own type, widened in each pass --
//     1/2/4/8 vectors per thread (templated, so short rows keep their occupancy); a warp per row
//     with shuffles only (eight rows per CTA) or a CTA of 128 or 256 threads per row with two block
//     reductions; vector stores;
//   * other rows below 64 KB: one CTA per row, the row staged in shared memory in its own type; loads
//     and stores are 16-byte vectors over the aligned body of the row with scalar head and tail, so
//     odd lengths and unaligned rows still move full sectors;
//   * longer rows (the vocabulary-sized ones): two passes over global memory with a running
//     (maximum, sum) per thread, the second pass served by L2.
#include <type_traits>

#include "common.cuh"
#include "ptx.cuh"

namespace rfx {

constexpr int kVecThreads = 256;
constexpr int kVecItems = 8;                  // vectors per thread in the register kernel

__device__ inline float block_reduce(float v, bool is_max, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = is_max ? warp_max(v) : warp_sum(v);
    __syncthreads();  // red[] may still be read from a previous reduction
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float r = is_max ? -INFINITY : 0.f;
    for (int i = 0; i < nw; ++i) r = is_max ? fmaxf(r, red[i]) : r + red[i];
    return r;
}

// Over the TPR threads that share a row: a warp (shuffles only) or the whole CTA of TPR threads.
template <int TPR>
__device__ inline float row_reduce(float v, bool is_max, float* red) {
    if (TPR == 32) return is_max ? warp_max(v) : warp_sum(v);
    if (TPR == kVecThreads) return block_reduce(v, is_max, red);
    constexpr int WPR = TPR / 32;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, first = (warp / WPR) * WPR;
    v = is_max ? warp_max(v) : warp_sum(v);
    __syncthreads();  // red[] may still be read from a previous reduction
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float r = is_max ? -INFINITY : 0.f;
#pragma unroll
    for (int i = 0; i < WPR; ++i) r = is_max ? fmaxf(r, red[first + i]) : r + red[first + i];
    return r;
}

template <typename T> struct alignas(16) Vec16 { T v[16 / sizeof(T)]; };

// 2^x by the hardware approximation (2 ulp, results below the normal range flush to zero): the
// library exp2f spends four more instructions per element on that range, and the register
// kernels are bound by their instruction count.
__device__ __forceinline__ float ex2_fast(float x) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}

// Two results rounded to T and stored side by side: one packed conversion for the 16-bit types.
template <typename T> __device__ __forceinline__ void put2(T* dst, float a, float b) {
    dst[0] = Num<T>::from_f(a);
    dst[1] = Num<T>::from_f(b);
}
template <> __device__ __forceinline__ void put2<__nv_bfloat16>(__nv_bfloat16* dst, float a, float b) {
    *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(a, b);
}
template <> __device__ __forceinline__ void put2<__half>(__half* dst, float a, float b) {
    *reinterpret_cast<__half2*>(dst) = __floats2half2_rn(a, b);
}

// Two 16-bit values in one 32-bit word: widened to fp32 (bf16 by moving bits, fp16 by the packed
// conversion) and compared two at a time (the maximum of two 16-bit values is one of them, so the
// packed maximum is exact and, like fmaxf, returns the other operand when one is NaN).
template <typename T> __device__ __forceinline__ float2 widen2(uint32_t w);
template <> __device__ __forceinline__ float2 widen2<__nv_bfloat16>(uint32_t w) {
    return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}
template <> __device__ __forceinline__ float2 widen2<__half>(uint32_t w) {
    return __half22float2(*reinterpret_cast<const __half2*>(&w));
}
template <typename T> __device__ __forceinline__ uint32_t max2_16(uint32_t a, uint32_t b);
template <> __device__ __forceinline__ uint32_t max2_16<__nv_bfloat16>(uint32_t a, uint32_t b) {
    const __nv_bfloat162 r = __hmax2(*reinterpret_cast<const __nv_bfloat162*>(&a), *reinterpret_cast<const __nv_bfloat162*>(&b));
    return *reinterpret_cast<const uint32_t*>(&r);
}
template <> __device__ __forceinline__ uint32_t max2_16<__half>(uint32_t a, uint32_t b) {
    const __half2 r = __hmax2(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b));
    return *reinterpret_cast<const uint32_t*>(&r);
}
template <typename T> __device__ __forceinline__ uint32_t pack2_16(float2 v);
template <> __device__ __forceinline__ uint32_t pack2_16<__nv_bfloat16>(float2 v) {
    const __nv_bfloat162 r = __floats2bfloat162_rn(v.x, v.y);
    return *reinterpret_cast<const uint32_t*>(&r);
}
template <> __device__ __forceinline__ uint32_t pack2_16<__half>(float2 v) {
    const __half2 r = __floats2half2_rn(v.x, v.y);
    return *reinterpret_cast<const uint32_t*>(&r);
}

// Register kernel: n % V == 0, rows 16-byte aligned, n <= TPR * kVecItems * V. TPR threads
// share a row: a whole CTA (two block reductions) or one warp (shuffles only, eight rows
// per CTA). exp through ex2 of the pre-scaled difference, one reciprocal per row.
// ITEMS = vectors per thread (1, 2, 4 or 8): the row is held in ITEMS * V registers, so short rows
// do not pay the register footprint (and the occupancy) of the longest one.
template <typename T, int TPR, int ITEMS>
__device__ __forceinline__ void
softmax_rows_reg_body(const T* __restrict__ x, T* __restrict__ y, int64_t rows, int n, int causal, int is_log) {
    constexpr int V = 16 / sizeof(T);
    constexpr int RPC = TPR == 32 ? kVecThreads / 32 : 1;  // rows per CTA: eight warps with a row each, or one row
    constexpr float kLog2e = 1.4426950408889634f;
    __shared__ float red[32];
    const int nvec = n / V;
    const int tr = threadIdx.x % TPR;
    const int sub = threadIdx.x / TPR;
    const int64_t row_groups = (rows + RPC - 1) / RPC;
    // Long fp32 rows on a whole CTA (PIPE): only two or three such CTAs fit an SM and their
    // block-wide reductions leave the memory system idle, so the grid is one wave of resident CTAs,
    // every CTA walks several rows, and the raw vectors of its next row are requested before the
    // current row's reductions and stores (fp32 8192 x 8192: 152 -> 91 us, 4096 x 4096: 39 -> 29 us).
    // Measured slower with it, and so left as they were: 16-bit rows (twice the arithmetic per
    // byte; 8192 x 8192 bf16 72 -> 90 us), short rows, and a warp per row.
    constexpr bool PIPE = TPR == kVecThreads && sizeof(T) == 4 && ITEMS >= 4;
    Vec16<T> nxt[PIPE ? ITEMS : 1];
    auto fetch = [&](int64_t grp) {
        const int64_t row = grp * RPC + sub;
        if (grp >= row_groups || row >= rows) return;
        const Vec16<T>* xr = reinterpret_cast<const Vec16<T>*>(x + row * (int64_t)n);
        const int valid = causal ? (int)(row % n) + 1 : n;
        if constexpr (PIPE) {
#pragma unroll
            for (int it = 0; it < ITEMS; ++it) {
                const int vi = it * TPR + tr;
                if (vi < nvec && vi * V < valid) nxt[it] = xr[vi];  // wholly masked vectors (causal) are not read
            }
        }
    };
    if (PIPE) fetch(blockIdx.x);
    for (int64_t grp = blockIdx.x; grp < row_groups; grp += gridDim.x) {
        const int64_t row = grp * RPC + sub;
        const bool live = row < rows;
        const Vec16<T>* xr = reinterpret_cast<const Vec16<T>*>(x + row * (int64_t)n);
        Vec16<T>* yr = reinterpret_cast<Vec16<T>*>(y + row * (int64_t)n);
        const int valid = causal ? (int)(row % n) + 1 : n;  // columns [0, valid) take part
        if constexpr (sizeof(T) == 2) {
            // 16-bit rows stay in registers in their own type (four registers per 16-byte vector, as for
            // fp32 rows) and are widened in each of the three passes: what bounds these rows is the bytes a
            // thread has in flight, and as fp32 copies they took twice the registers per byte of an fp32 row.
            // The exponentials are evaluated twice (sum, output). Two elements per instruction wherever the
            // arithmetic allows it (packed maximum on the raw words, packed fp32 multiply-add / add / multiply).
            constexpr int W = V / 2;  // 32-bit words per vector
            constexpr uint32_t kNegInf2 = std::is_same<T, __nv_bfloat16>::value ? 0xff80ff80u : 0xfc00fc00u;
            constexpr uint32_t kNegInfLo = kNegInf2 & 0xffffu, kNegInfHi = kNegInf2 & 0xffff0000u;
            uint32_t raw[ITEMS][W];
            uint32_t m2 = kNegInf2;
#pragma unroll
            for (int it = 0; it < ITEMS; ++it) {
                const int vi = it * TPR + tr;
#pragma unroll
                for (int k = 0; k < W; ++k) raw[it][k] = kNegInf2;  // masked columns and vectors past the row
                if (live && vi < nvec && vi * V < valid) {
                    const Vec16<T> p = xr[vi];
                    const uint32_t* w = reinterpret_cast<const uint32_t*>(&p);
#pragma unroll
                    for (int k = 0; k < W; ++k) raw[it][k] = w[k];
                    if (vi * V + V > valid) {  // the vector the causal boundary cuts
#pragma unroll
                        for (int k = 0; k < W; ++k) {
                            if (vi * V + 2 * k >= valid) raw[it][k] = (raw[it][k] & 0xffff0000u) | kNegInfLo;
                            if (vi * V + 2 * k + 1 >= valid) raw[it][k] = (raw[it][k] & 0xffffu) | kNegInfHi;
                        }
                    }
#pragma unroll
                    for (int k = 0; k < W; ++k) m2 = max2_16<T>(m2, raw[it][k]);
                }
            }
            // The compiler must not keep the widened values from one pass to the next (it would: widening is
            // pure), or the row is back to eight registers per vector.
            auto forget = [&]() {
#pragma unroll
                for (int it = 0; it < ITEMS; ++it)
#pragma unroll
                    for (int k = 0; k < W; ++k) asm volatile("" : "+r"(raw[it][k]));
            };
            const float2 mm = widen2<T>(m2);
            float m = fmaxf(mm.x, mm.y);
            m = row_reduce<TPR>(m, true, red);
            forget();
            const float mb = m * kLog2e;
            const float2 k2 = make_float2(kLog2e, kLog2e), nmb2 = make_float2(-mb, -mb);
            float2 l2 = make_float2(0.f, 0.f);
#pragma unroll
            for (int it = 0; it < ITEMS; ++it) {
#pragma unroll
                for (int k = 0; k < W; ++k) {
                    const float2 t = __ffma2_rn(widen2<T>(raw[it][k]), k2, nmb2);
                    const float2 ex = make_float2(ex2_fast(t.x), ex2_fast(t.y));  // 0 for masked columns
                    l2 = __fadd2_rn(l2, ex);
                    // The exponentials take the place of the inputs, rounded to the row's type (the sum is
                    // taken before the rounding): one exponential per element instead of two -- the XU pipe
                    // was more than half busy -- at the price of a second rounding of the result, which stays
                    // within one unit of the 16-bit type.
                    if (!is_log) raw[it][k] = pack2_16<T>(ex);
                }
            }
            float l = l2.x + l2.y;
            l = row_reduce<TPR>(l, false, red);
            forget();
            const float logl = logf(l);
            const float inv = 1.0f / l;
            const float2 inv2 = make_float2(inv, inv), nm2 = make_float2(-m, -m), nlogl2 = make_float2(-logl, -logl);
#pragma unroll
            for (int it = 0; it < ITEMS; ++it) {
                const int vi = it * TPR + tr;
                if (live && vi < nvec) {
                    Vec16<T> o;
                    uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
                    for (int k = 0; k < W; ++k) {
                        const float2 f = widen2<T>(raw[it][k]);
                        ow[k] = pack2_16<T>(is_log ? __fadd2_rn(__fadd2_rn(f, nm2), nlogl2) : __fmul2_rn(f, inv2));
                    }
                    yr[vi] = o;
                }
            }
            continue;
        }
        float f[ITEMS][V];
        float m = -INFINITY;
#pragma unroll
        for (int it = 0; it < ITEMS; ++it) {
            const int vi = it * TPR + tr;
            if (live && vi < nvec) {
                if (vi * V < valid) {
                    const Vec16<T> p = PIPE ? nxt[PIPE ? it : 0] : xr[vi];
                    if (vi * V + V <= valid) {  // the usual case: no column of this vector is masked
#pragma unroll
                        for (int j = 0; j < V; ++j) {
                            f[it][j] = Num<T>::to_f(p.v[j]);
                            m = fmaxf(m, f[it][j]);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < V; ++j) {
                            float v = Num<T>::to_f(p.v[j]);
                            if (vi * V + j >= valid) v = -INFINITY;
                            f[it][j] = v;
                            m = fmaxf(m, v);
                        }
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < V; ++j) f[it][j] = -INFINITY;
                }
            }
        }
        if (PIPE) fetch(grp + gridDim.x);
        m = row_reduce<TPR>(m, true, red);
        const float mb = m * kLog2e;
        float l = 0.f;
#pragma unroll
        for (int it = 0; it < ITEMS; ++it) {
            const int vi = it * TPR + tr;
            if (live && vi < nvec) {
                if (is_log) {
#pragma unroll
                    for (int j = 0; j < V; ++j) l += ex2_fast(fmaf(f[it][j], kLog2e, -mb));  // 0 for masked columns
                } else {
#pragma unroll
                    for (int j = 0; j < V; ++j) {
                        f[it][j] = ex2_fast(fmaf(f[it][j], kLog2e, -mb));
                        l += f[it][j];
                    }
                }
            }
        }
        l = row_reduce<TPR>(l, false, red);
        const float logl = logf(l);
        const float inv = 1.0f / l;
#pragma unroll
        for (int it = 0; it < ITEMS; ++it) {
            const int vi = it * TPR + tr;
            if (live && vi < nvec) {
                Vec16<T> o;
                if (is_log) {
#pragma unroll
                    for (int j = 0; j < V; j += 2) put2<T>(&o.v[j], (f[it][j] - m) - logl, (f[it][j + 1] - m) - logl);
                } else {
#pragma unroll
                    for (int j = 0; j < V; j += 2) put2<T>(&o.v[j], f[it][j] * inv, f[it][j + 1] * inv);
                }
                yr[vi] = o;
            }
        }
    }
}

// The softmax kernels are launched with programmatic stream serialisation: the kernel behind one of them
// may be scheduled as soon as all its CTAs have started, so that a CTA slot is taken again the moment
// it is freed, and reads nothing before everything ahead of it in the stream has completed. A short call
// between two others no longer pays its launch latency on top of its memory time.
__device__ __forceinline__ void pdl_prologue() {
    ptx::pdl_trigger();
    ptx::pdl_wait();
}

// MINB = resident CTAs per SM asked of the compiler. Rows of one or two fp32 vectors per thread are
// bound by the warps in flight (ncu: 40 of 64 warps at 48 registers): eight CTAs per SM, which fits them
// into 32 registers without spills (4096 x 4096 bf16 24.6 -> 22.5 us); longer fp32 rows keep the plain
// bound (a hint made them slower). 16-bit rows are held raw, four registers per vector, and take the
// bound that leaves room for just that: unbounded, the compiler spreads the widened values of a whole
// pass over 120-240 registers and the occupancy is gone.
template <typename T, int TPR, int ITEMS, int MINB>
__global__ void __launch_bounds__(kVecThreads, MINB)
softmax_rows_reg_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t rows, int n, int causal, int is_log) {
    pdl_prologue();
    softmax_rows_reg_body<T, TPR, ITEMS>(x, y, rows, n, causal, is_log);
}

// Writes elements [0, count) of a row from `val(index)`: scalar head up to the first 16-byte boundary,
// vector body, scalar tail.
template <typename T, typename F>
__device__ inline void for_each_store(T* row, int count, F val) {
    constexpr int V = 16 / sizeof(T);
    const int mis = (int)(((uintptr_t)row % 16) / sizeof(T));
    const int head = min(count, mis ? V - mis : 0);
    for (int i = threadIdx.x; i < head; i += blockDim.x) row[i] = Num<T>::from_f(val(i));
    const int nbody = (count - head) / V;
    Vec16<T>* body = reinterpret_cast<Vec16<T>*>(row + head);
    for (int vi = threadIdx.x; vi < nbody; vi += blockDim.x) {
        Vec16<T> o;
#pragma unroll
        for (int j = 0; j < V; ++j) o.v[j] = Num<T>::from_f(val(head + vi * V + j));
        body[vi] = o;
    }
    for (int i = head + nbody * V + threadIdx.x; i < count; i += blockDim.x) row[i] = Num<T>::from_f(val(i));
}

// Rows below 64 KB that the register kernels do not take (odd lengths, unaligned rows): the row is kept
// in shared memory in its own type, read from global memory once and written once.
template <typename T>
__global__ void softmax_rows_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t rows, int n,
                                    int causal, int is_log) {
    pdl_prologue();
    extern __shared__ __align__(16) unsigned char srow_raw[];
    T* srow = reinterpret_cast<T*>(srow_raw);
    __shared__ float red[32];
    constexpr float kLog2e = 1.4426950408889634f;
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const T* xr = x + row * (int64_t)n;
        T* yr = y + row * (int64_t)n;
        const int valid = causal ? (int)(row % n) + 1 : n;  // columns [0, valid) take part
        float m = -INFINITY;
        {
            // raw copy with 16-byte vectors over the aligned body of the row
            constexpr int V = 16 / sizeof(T);
            const int mis = (int)(((uintptr_t)xr % 16) / sizeof(T));
            const int head = min(valid, mis ? V - mis : 0);
            // the staged row keeps the global row's misalignment so that vector k of the body lands
            // on a 16-byte boundary of shared memory too
            T* sr = srow + mis;
            for (int i = threadIdx.x; i < head; i += blockDim.x) { const T v = xr[i]; sr[i] = v; m = fmaxf(m, Num<T>::to_f(v)); }
            const int nbody = (valid - head) / V;
            struct alignas(16) Vec { T v[V]; };
            const Vec* gb = reinterpret_cast<const Vec*>(xr + head);
            Vec* sb = reinterpret_cast<Vec*>(sr + head);
            [[maybe_unused]] uint32_t m2 = std::is_same<T, __nv_bfloat16>::value ? 0xff80ff80u : 0xfc00fc00u;  // (-inf, -inf)
#pragma unroll 8
            for (int vi = threadIdx.x; vi < nbody; vi += blockDim.x) {
                const Vec p = gb[vi];
                sb[vi] = p;
                if constexpr (sizeof(T) == 2) {
                    const uint32_t* w = reinterpret_cast<const uint32_t*>(&p);
#pragma unroll
                    for (int k = 0; k < V / 2; ++k) m2 = max2_16<T>(m2, w[k]);
                } else {
#pragma unroll
                    for (int j = 0; j < V; ++j) m = fmaxf(m, Num<T>::to_f(p.v[j]));
                }
            }
            if constexpr (sizeof(T) == 2) {
                const float2 mm = widen2<T>(m2);
                m = fmaxf(m, fmaxf(mm.x, mm.y));
            }
            for (int i = head + nbody * V + threadIdx.x; i < valid; i += blockDim.x) { const T v = xr[i]; sr[i] = v; m = fmaxf(m, Num<T>::to_f(v)); }
            m = block_reduce(m, true, red);  // also orders the smem writes before the reads below
            const float mb = m * kLog2e;
            // The two passes over the staged row read it as 16-byte vectors too: with one element per
            // load the kernel was bound by its instruction count, not by memory.
            // For 16-bit rows of the plain softmax the exponentials replace the staged inputs, rounded to the
            // row's type (the sum is taken before the rounding): one exponential per element instead of two
            // (at two, the XU pipe needs 3.3 us for a 50 257-element row, which did not overlap the 4.6 us
            // of memory time) at the price of a second rounding of the result, within one unit of the type.
            constexpr bool kKeep = sizeof(T) == 2;
            float l = 0.f;
            const int tail0 = head + nbody * V;
            auto one = [&](int i) {
                const float ex = ex2_fast(fmaf(Num<T>::to_f(sr[i]), kLog2e, -mb));
                l += ex;
                if (kKeep && !is_log) sr[i] = Num<T>::from_f(ex);
            };
            for (int i = threadIdx.x; i < head; i += blockDim.x) one(i);
            [[maybe_unused]] const float2 k2 = make_float2(kLog2e, kLog2e), nmb2 = make_float2(-mb, -mb);
            [[maybe_unused]] float2 l2 = make_float2(0.f, 0.f);
            for (int vi = threadIdx.x; vi < nbody; vi += blockDim.x) {
                Vec p = sb[vi];
                if constexpr (sizeof(T) == 2) {
                    uint32_t* w = reinterpret_cast<uint32_t*>(&p);
#pragma unroll
                    for (int k = 0; k < V / 2; ++k) {
                        const float2 t = __ffma2_rn(widen2<T>(w[k]), k2, nmb2);
                        const float2 ex = make_float2(ex2_fast(t.x), ex2_fast(t.y));
                        l2 = __fadd2_rn(l2, ex);
                        w[k] = pack2_16<T>(ex);
                    }
                    if (!is_log) sb[vi] = p;
                } else {
#pragma unroll
                    for (int j = 0; j < V; ++j) l += ex2_fast(fmaf(Num<T>::to_f(p.v[j]), kLog2e, -mb));
                }
            }
            if constexpr (sizeof(T) == 2) l += l2.x + l2.y;
            for (int i = tail0 + threadIdx.x; i < valid; i += blockDim.x) one(i);
            l = block_reduce(l, false, red);
            const float logl = logf(l), inv = 1.0f / l;
            auto out_of = [&](int i, float v) -> float {  // v: the staged value (16-bit rows, plain softmax: its exponential)
                if (i >= valid) return is_log ? -INFINITY : 0.f;
                return is_log ? (v - m) - logl : (kKeep ? v : ex2_fast(fmaf(v, kLog2e, -mb))) * inv;
            };
            if ((int)(((uintptr_t)yr % 16) / sizeof(T)) == mis) {
                // output row aligned like the input row: vector k of the staged body is vector k of the output
                const int head_y = min(n, mis ? V - mis : 0);
                const int nbody_y = (n - head_y) / V;
                for (int i = threadIdx.x; i < head_y; i += blockDim.x) yr[i] = Num<T>::from_f(out_of(i, Num<T>::to_f(sr[i])));
                Vec* yb = reinterpret_cast<Vec*>(yr + head_y);
                const Vec* sby = reinterpret_cast<const Vec*>(sr + head_y);
                for (int vi = threadIdx.x; vi < nbody_y; vi += blockDim.x) {
                    const Vec p = sby[vi];  // columns past `valid` were never staged: whatever is read there is not used
                    Vec o;
                    const int c0 = head_y + vi * V;
                    if (c0 + V <= valid && !is_log) {  // the usual case, two results per conversion
                        if constexpr (sizeof(T) == 2) {
                            const uint32_t* w = reinterpret_cast<const uint32_t*>(&p);
                            uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
                            const float2 inv2 = make_float2(inv, inv);
#pragma unroll
                            for (int k = 0; k < V / 2; ++k) ow[k] = pack2_16<T>(__fmul2_rn(widen2<T>(w[k]), inv2));
                        } else {
#pragma unroll
                            for (int j = 0; j < V; j += 2)
                                put2<T>(&o.v[j], ex2_fast(fmaf(Num<T>::to_f(p.v[j]), kLog2e, -mb)) * inv,
                                        ex2_fast(fmaf(Num<T>::to_f(p.v[j + 1]), kLog2e, -mb)) * inv);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < V; ++j) o.v[j] = Num<T>::from_f(out_of(c0 + j, Num<T>::to_f(p.v[j])));
                    }
                    yb[vi] = o;
                }
                for (int i = head_y + nbody_y * V + threadIdx.x; i < n; i += blockDim.x)
                    yr[i] = Num<T>::from_f(out_of(i, Num<T>::to_f(sr[i])));
            } else {
                for_each_store<T>(yr, n, [&](int i) -> float { return out_of(i, i < valid ? Num<T>::to_f(sr[i]) : 0.f); });
            }
        }
        __syncthreads();  // srow is reused by the next row
    }
}

// Long rows (64 KB and more: the vocabulary-sized ones): two passes over global memory, no row staged.
// Pass one streams the row and keeps a running (maximum, sum of exponentials) per thread, rescaling
// the sum when a vector brings a larger maximum; the threads' pairs are merged once. Pass two reads
// the row again -- it is still in L2, a CTA re-reads what it has just read -- and writes the result,
// so DRAM sees the row once in and once out. A staged row of 100 KB lets only two rows share an SM,
// and their loads, reductions and stores take turns. Here a thread walks its vectors through a ring of
// eight 16-byte slots of its own in shared memory, filled by cp.async: eight vectors per thread are on
// their way at all times (a slot is refilled as soon as its vector has been used) and no thread ever
// reads another's slot, so there is no barrier in the loop.
constexpr int kTwoPassThreads = 256;
constexpr int kTwoPassDepth = 8;

template <typename VecT, typename F>
__device__ __forceinline__ void stream_vectors(const VecT* gb, int nvec, unsigned char* ring, F fn) {
    constexpr int D = kTwoPassDepth;
    constexpr uint32_t kSlot = kTwoPassThreads * 16;  // bytes between a thread's consecutive slots
    VecT* mine = reinterpret_cast<VecT*>(ring) + threadIdx.x;
    const uint32_t base = (uint32_t)__cvta_generic_to_shared(mine);
#pragma unroll
    for (int d = 0; d < D; ++d) {
        const int vi = threadIdx.x + d * kTwoPassThreads;
        if (vi < nvec) asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(base + d * kSlot), "l"(gb + vi) : "memory");
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    int slot = 0;
    for (int vi = threadIdx.x; vi < nvec; vi += kTwoPassThreads) {
        asm volatile("cp.async.wait_group %0;" ::"n"(D - 1) : "memory");  // this thread's oldest copy has landed
        const VecT p = mine[slot * kTwoPassThreads];
        fn(vi, p);  // p is in registers before the slot is refilled
        const int nx = vi + D * kTwoPassThreads;
        if (nx < nvec) asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(base + slot * kSlot), "l"(gb + nx) : "memory");
        asm volatile("cp.async.commit_group;" ::: "memory");
        slot = slot + 1 == D ? 0 : slot + 1;
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
}

template <typename T>
__global__ void __launch_bounds__(kTwoPassThreads)
softmax_rows_twopass_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t rows, int n, int causal, int is_log) {
    pdl_prologue();
    __shared__ float red[32];
    extern __shared__ __align__(16) unsigned char ring[];  // kTwoPassThreads * kTwoPassDepth * 16 bytes (+ padding, see the launch)
    constexpr float kLog2e = 1.4426950408889634f;
    constexpr int V = 16 / sizeof(T);
    struct alignas(16) Vec { T v[V]; };
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const T* xr = x + row * (int64_t)n;
        T* yr = y + row * (int64_t)n;
        const int valid = causal ? (int)(row % n) + 1 : n;  // columns [0, valid) take part
        const int mis = (int)(((uintptr_t)xr % 16) / sizeof(T));
        const int head = min(valid, mis ? V - mis : 0);
        const int nbody = (valid - head) / V;  // whole vectors of the aligned body, all inside `valid`
        const int tail0 = head + nbody * V;
        const Vec* gb = reinterpret_cast<const Vec*>(xr + head);
        // ---- pass one: running maximum (natural units) and sum of 2^((x - m) log2 e)
        float m = -INFINITY, l = 0.f;
        auto take = [&](float vmax, auto&& add) {
            if (vmax > m) {
                l *= ex2_fast((m - vmax) * kLog2e);  // 0 * 0 at the start
                m = vmax;
            }
            if (m > -INFINITY) add(m * kLog2e);
        };
        auto one = [&](int i) {
            const float v = Num<T>::to_f(xr[i]);
            take(v, [&](float mb) { l += ex2_fast(fmaf(v, kLog2e, -mb)); });
        };
        for (int i = threadIdx.x; i < head; i += blockDim.x) one(i);
        stream_vectors(gb, nbody, ring, [&](int, const Vec& p) {
            if constexpr (sizeof(T) == 2) {
                const uint32_t* w = reinterpret_cast<const uint32_t*>(&p);
                const uint32_t m2 = max2_16<T>(max2_16<T>(w[0], w[1]), max2_16<T>(w[2], w[3]));
                const float2 mm = widen2<T>(m2);
                take(fmaxf(mm.x, mm.y), [&](float mb) {
                    const float2 k2 = make_float2(kLog2e, kLog2e), nmb2 = make_float2(-mb, -mb);
                    float2 acc = make_float2(0.f, 0.f);
#pragma unroll
                    for (int k = 0; k < V / 2; ++k) {
                        const float2 t = __ffma2_rn(widen2<T>(w[k]), k2, nmb2);
                        acc = __fadd2_rn(acc, make_float2(ex2_fast(t.x), ex2_fast(t.y)));
                    }
                    l += acc.x + acc.y;
                });
            } else {
                float f[V];
                float vm = -INFINITY;
#pragma unroll
                for (int j = 0; j < V; ++j) { f[j] = Num<T>::to_f(p.v[j]); vm = fmaxf(vm, f[j]); }
                take(vm, [&](float mb) {
#pragma unroll
                    for (int j = 0; j < V; ++j) l += ex2_fast(fmaf(f[j], kLog2e, -mb));
                });
            }
        });
        for (int i = tail0 + threadIdx.x; i < valid; i += blockDim.x) one(i);
        const float M = block_reduce(m, true, red);
        l = (m > -INFINITY) ? l * ex2_fast((m - M) * kLog2e) : 0.f;
        l = block_reduce(l, false, red);
        const float mb = M * kLog2e, logl = logf(l), inv = 1.0f / l;
        auto out_of = [&](int i, float v) -> float {
            if (i >= valid) return is_log ? -INFINITY : 0.f;
            return is_log ? (v - M) - logl : ex2_fast(fmaf(v, kLog2e, -mb)) * inv;
        };
        // ---- pass two
        if ((int)(((uintptr_t)yr % 16) / sizeof(T)) == mis) {
            // the output row is aligned like the input row: vector k of one body is vector k of the other
            const int head_y = min(n, mis ? V - mis : 0);
            const int nbody_y = (n - head_y) / V;
            for (int i = threadIdx.x; i < head_y; i += blockDim.x) yr[i] = Num<T>::from_f(out_of(i, i < valid ? Num<T>::to_f(xr[i]) : 0.f));
            Vec* yb = reinterpret_cast<Vec*>(yr + head_y);
            const float2 k2 = make_float2(kLog2e, kLog2e), nmb2 = make_float2(-mb, -mb), inv2 = make_float2(inv, inv);
            const int nfull = head_y == head ? nbody : 0;  // (they differ only when `valid` ends inside the head)
            stream_vectors(gb, nfull, ring, [&](int vi, const Vec& p) {
                Vec o;
                if constexpr (sizeof(T) == 2) {
                    if (!is_log) {
                        const uint32_t* w = reinterpret_cast<const uint32_t*>(&p);
                        uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
                        for (int k = 0; k < V / 2; ++k) {
                            const float2 t = __ffma2_rn(widen2<T>(w[k]), k2, nmb2);
                            ow[k] = pack2_16<T>(__fmul2_rn(make_float2(ex2_fast(t.x), ex2_fast(t.y)), inv2));
                        }
                        yb[vi] = o;
                        return;
                    }
                }
#pragma unroll
                for (int j = 0; j < V; ++j) o.v[j] = Num<T>::from_f(out_of(head + vi * V + j, Num<T>::to_f(p.v[j])));
                yb[vi] = o;
            });
            // the vector the causal boundary cuts and those past it (their input is not read), then the tail
            for (int vi = nfull + threadIdx.x; vi < nbody_y; vi += blockDim.x) {
                const int c0 = head_y + vi * V;
                Vec o;
#pragma unroll
                for (int j = 0; j < V; ++j) o.v[j] = Num<T>::from_f(out_of(c0 + j, c0 + j < valid ? Num<T>::to_f(xr[c0 + j]) : 0.f));
                yb[vi] = o;
            }
            for (int i = head_y + nbody_y * V + threadIdx.x; i < n; i += blockDim.x)
                yr[i] = Num<T>::from_f(out_of(i, i < valid ? Num<T>::to_f(xr[i]) : 0.f));
        } else {
            for_each_store<T>(yr, n, [&](int i) -> float { return out_of(i, i < valid ? Num<T>::to_f(xr[i]) : 0.f); });
        }
    }
}

// One instantiation of the register kernel. The grid is one wave of resident CTAs (what the occupancy
// query says fits) for long fp32 rows, each CTA walking several rows; the usual cap otherwise.
template <typename T, int TPR, int ITEMS>
static void launch_softmax_reg(const RfxSoftmaxArgs* a, int64_t groups, int64_t cap, cudaStream_t s) {
    constexpr int kMinB = sizeof(T) == 2 ? (ITEMS <= 4 ? 8 : ITEMS <= 8 ? 4 : 2) : (ITEMS <= 2 ? 8 : 0);
    auto kern = softmax_rows_reg_kernel<T, TPR, ITEMS, kMinB>;
    static PerDeviceOnce occ;  // resident CTAs per SM of this instantiation, by device
    int dev = 0;
    cudaGetDevice(&dev);
    int per_sm = occ.value(dev);
    if (!per_sm) {
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, TPR == 32 ? kVecThreads : TPR, 0) != cudaSuccess || per_sm < 1)
            per_sm = 1;
        occ.mark(dev, per_sm);
    }
    const int64_t wave = (TPR == 32 || sizeof(T) != 4 || ITEMS < 4) ? cap : (int64_t)sm_count() * (per_sm > 0 ? per_sm : 1);
    const int64_t g2 = groups < wave ? groups : wave;
    launch_pdl(kern, dim3((unsigned)g2), dim3(TPR == 32 ? kVecThreads : TPR), 0, s, (const T*)a->x, (T*)a->y, a->rows, (int)a->n,
               (int)a->is_causal, (int)a->log);
}

template <typename T, int TPR>
static void launch_softmax_reg_items(const RfxSoftmaxArgs* a, int need, int64_t groups, int64_t cap, cudaStream_t s) {
    if (need <= 1) launch_softmax_reg<T, TPR, 1>(a, groups, cap, s);
    else if (need <= 2) launch_softmax_reg<T, TPR, 2>(a, groups, cap, s);
    else if (need <= 4) launch_softmax_reg<T, TPR, 4>(a, groups, cap, s);
    else launch_softmax_reg<T, TPR, 8>(a, groups, cap, s);
}

// 128 threads per row, four vectors each: 16-bit rows only.
template <typename T>
static void launch_softmax_reg_part(const RfxSoftmaxArgs* a, int64_t groups, int64_t cap, cudaStream_t s) {
    if constexpr (sizeof(T) == 2) launch_softmax_reg<T, 128, 4>(a, groups, cap, s);
}

}  // namespace rfx

extern "C" int rfx_online_softmax(const RfxSoftmaxArgs* a) {
    using namespace rfx;
    const char* name = "rfx_online_softmax";
    if (!a) return fail(RFX_INVALID_ARGUMENT, "%s: null args", name);
    RFX_REQUIRE(dtype_ok(a->dtype), "%s: unknown dtype %d", name, a->dtype);
    RFX_REQUIRE(a->rows >= 0 && a->n >= 0 && a->n < (1ll << 31), "%s: bad sizes", name);
    if (a->is_causal)
        RFX_REQUIRE(a->n > 0 && a->rows % a->n == 0,
                    "causal mode requires square input (last two dims equal); rows=%lld n=%lld",
                    (long long)a->rows, (long long)a->n);
    if (a->rows == 0 || a->n == 0) return RFX_SUCCESS;
    RFX_REQUIRE(a->x && a->y, "%s: null pointer", name);
    int st = check_device();
    if (st != RFX_SUCCESS) return st;

    const int n = (int)a->n;
    const size_t e = dtype_size(a->dtype);
    const int V = (int)(16 / e);
    cudaStream_t s = as_stream(a->stream);
    int64_t grid = a->rows;
    const int64_t cap = (int64_t)sm_count() * 32;
    if (grid > cap) grid = cap;

    const bool reg_ok = n % V == 0 && n <= kVecThreads * kVecItems * V && ((uintptr_t)a->x % 16) == 0 &&
                        ((uintptr_t)a->y % 16) == 0;
    if (reg_ok) {
        // Threads per row: a warp (eight rows per CTA of 256 threads) up to eight vectors per lane, else a
        // CTA per row. What bounds these rows is the bytes in flight per SM = resident rows x row bytes, so
        // a 16-bit row of up to 4096 elements takes a CTA of 128 threads (sixteen of them per SM; 4096 x 4096
        // bf16 with 256 threads: 0.65 of the copy rate). Several rows in one CTA that reduce together, or a
        // warp per row with sixteen vectors per lane, were measured slower (0.56 / 0.40).
        const int nvec = n / V;
        int tpr = kVecThreads;
        if (nvec <= 32 * kVecItems) tpr = 32;
        else if (e == 2 && nvec <= 128 * 4) tpr = 128;
        const int rpc = tpr == 32 ? kVecThreads / 32 : 1;
        const int64_t groups = (a->rows + rpc - 1) / rpc;
        const int need = (nvec + tpr - 1) / tpr;  // vectors per thread
        RFX_DISPATCH_DTYPE(a->dtype, T, {
            if (tpr == 32) launch_softmax_reg_items<T, 32>(a, need, groups, cap, s);
            else if (tpr == kVecThreads) launch_softmax_reg_items<T, kVecThreads>(a, need, groups, cap, s);
            else launch_softmax_reg_part<T>(a, groups, 2 * cap, s);
        });
        return check_launch(name);
    }
    const size_t smem_need = (size_t)n * e + 32;  // the row in its own type + room for its misalignment
    if ((size_t)n * e >= 64 * 1024) {
        // in place is fine: pass one has read the whole row before pass two writes any of it, and in pass two
        // a vector is read by the thread that then overwrites it
        const int64_t g = a->rows < cap ? a->rows : cap;
        // CTAs per SM. Pass two finds the row in L2 only while the rows between their two passes fit there
        // with room to spare: at six CTAs per SM 8 x 1024 x 50 257 fp16 has 90 MB of rows under way and
        // runs at 0.69 of the copy rate, at four 0.76, at three (44 MB) 0.82, at two 0.71 (too few bytes in
        // flight). A batch that fits into one wave of at most six CTAs per SM takes that wave. The dynamic
        // shared memory beyond the ring is padding that sets the number.
        const size_t row_bytes = (size_t)n * e;
        const int sms = sm_count();
        int64_t k = (int64_t)((45ull << 20) / ((size_t)sms * row_bytes));
        k = k < 2 ? 2 : k > 6 ? 6 : k;
        const int64_t k_wave = (a->rows + sms - 1) / sms;
        if (k_wave > k && k_wave <= 6 && (size_t)a->rows * row_bytes <= (64ull << 20)) k = k_wave;
        const int ring = kTwoPassThreads * kTwoPassDepth * 16;
        int dyn = (int)(233472 / k) - 1024 - 256;  // shared memory of an SM / k, less the per-CTA reserve and the static part
        if (dyn < ring) dyn = ring;
        RFX_DISPATCH_DTYPE(a->dtype, T, {
            auto kern = softmax_rows_twopass_kernel<T>;
            cudaError_t ce = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, dyn);
            if (ce != cudaSuccess) return fail(RFX_CUDA_ERROR, "%s: smem opt-in: %s", name, cudaGetErrorString(ce));
            launch_pdl(kern, dim3((unsigned)g), dim3(kTwoPassThreads), (size_t)dyn, s, (const T*)a->x, (T*)a->y, a->rows, n,
                       (int)a->is_causal, (int)a->log);
        });
        return check_launch(name);
    }
    const int threads = n <= 512 ? 64 : n <= 4096 ? 128 : n <= 16384 ? 256 : 1024;
    RFX_DISPATCH_DTYPE(a->dtype, T, {
        auto kern = softmax_rows_kernel<T>;
        if (smem_need > 48 * 1024) {
            cudaError_t ce = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_need);
            if (ce != cudaSuccess) return fail(RFX_CUDA_ERROR, "%s: smem opt-in: %s", name, cudaGetErrorString(ce));
        }
        launch_pdl(kern, dim3((unsigned)grid), dim3(threads), smem_need, s, (const T*)a->x, (T*)a->y, a->rows, n,
                   (int)a->is_causal, (int)a->log);
    });
    return check_launch(name);
}
