// Fused linear + LayerNorm / RMSNorm (kernels/fused_linear_norm/__init__.py:27-73, semantics of
// torch_reference_fused_linear_norm, kernels/fused_linear_norm/triton_kernel.py:204-233).
//
// Two launches:
//   1. y = x @ W^T + bias, rounded to the activation dtype, written to `out`; the epilogue also
//      adds each row's sum and sum of squares of the ROUNDED values to the workspace (the norm
//      of the reference sees the rounded y). 16-bit inputs run on the tensor cores:
//      persistent CTAs over 128x256 output tiles, a TMA producer warp filling a four-stage ring of
//      [128x64] x-tiles and [256x64] W-tiles (128-byte swizzle, both K-major), one thread issuing
//      tcgen05.mma 128x256x16 into one of two 256-column accumulators in tensor memory, four
//      epilogue warps reading the other one's rows with tcgen05.ld under the next tile's main loop. Tensor-pipe bound: 2*M*N*K FLOPs.
//      fp32 and sizes the tensor maps cannot express take a plain shared-memory GEMM.
//   2. the norm over `out` in place, one warp per row: bandwidth-bound, 2*M*N*e bytes (the rows
//      are still in L2 for the reference's sizes).
#include "common.cuh"
#include "ptx.cuh"

#include <type_traits>

namespace rfx {

constexpr int kLnTileM = 128, kLnTileN = 256, kLnTileK = 64, kLnStages = 4;
constexpr int kLnABytes = kLnTileM * kLnTileK * 2;  // 16 KiB
constexpr int kLnBBytes = kLnTileN * kLnTileK * 2;  // 32 KiB
constexpr int kLnThreads = 192;                     // producer, issuer, four epilogue warps
// Row statistics are spread over 16 slots per row (producer CTA index mod 16), so that the
// atomics of the many CTAs of a narrow-M problem do not all hit one address.
constexpr int kLnStatSlots = 16;
constexpr size_t kLnSmem = (size_t)kLnStages * (kLnABytes + kLnBBytes) + 256 + 1024;  // ring, barriers, alignment slack

struct LnGemmParams {
    const void* bias;
    void* out;
    float* stats;      // [M][16 slots][2]: sum, sum of squares of the rounded y
    int32_t* status;   // bit 0: a bounded wait expired
    int M, N, K;
};

template <typename T>
__global__ void __launch_bounds__(kLnThreads, 1)
linear_stats_tc_kernel(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap wmap,
                       const LnGemmParams P) {
    constexpr bool BF = std::is_same<T, __nv_bfloat16>::value;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (ptx::smem_u32(smem_raw) & 1023u)) & 1023u);
    unsigned char* sA = smem;
    unsigned char* sB = smem + (size_t)kLnStages * kLnABytes;
    // barriers: full[4], empty[4] (smem ring), acc_full[2], acc_empty[2] (the two accumulators)
    uint64_t* bars = reinterpret_cast<uint64_t*>(sB + (size_t)kLnStages * kLnBBytes);
    uint32_t* misc = reinterpret_cast<uint32_t*>(bars + 2 * kLnStages + 4);
    uint64_t* full = bars;
    uint64_t* empty = bars + kLnStages;
    uint64_t* acc_full = bars + 2 * kLnStages;
    uint64_t* acc_empty = acc_full + 2;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nk = (P.K + kLnTileK - 1) / kLnTileK;
    // Persistent: CTA c takes tiles c, c + gridDim.x, ... (N-tile index fastest, so the CTAs of a
    // wave share x rows); two accumulators in tensor memory, so the epilogue of one tile runs
    // under the main loop of the next.
    const int tiles_n = (P.N + kLnTileN - 1) / kLnTileN;
    const int n_tiles = tiles_n * ((P.M + kLnTileM - 1) / kLnTileM);

    if (threadIdx.x == 0) {
        for (int i = 0; i < 2 * kLnStages + 2; ++i) ptx::mbar_init(&bars[i], 1);
        ptx::mbar_init(&acc_empty[0], 128);  // the four epilogue warps
        ptx::mbar_init(&acc_empty[1], 128);
        ptx::fence_barrier_init();
    }
    if (warp == 1) ptx::tmem_alloc(&misc[0], 2 * kLnTileN);
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem = misc[0];

    if (warp == 0) {
        // ---- TMA producer: rows past M / N and columns past K arrive as zeros
        if (lane == 0) {
            ptx::prefetch_tensormap(&xmap);
            ptx::prefetch_tensormap(&wmap);
            int g = 0;  // K steps so far: step g uses stage g % 4, use g / 4 of that stage
            for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
                const int n0 = (tile % tiles_n) * kLnTileN, m0 = (tile / tiles_n) * kLnTileM;
                for (int ks = 0; ks < nk; ++ks, ++g) {
                    const int st = g % kLnStages;
                    if (!ptx::mbar_wait_bounded(&empty[st], (uint32_t)(((g / kLnStages) & 1) ^ 1))) {
                        atomicOr(P.status, 1);
                        tile = n_tiles;
                        break;
                    }
                    ptx::mbar_arrive_expect_tx(&full[st], (uint32_t)(kLnABytes + kLnBBytes));
                    ptx::tma_load_2d(sA + (size_t)st * kLnABytes, &xmap, &full[st], ks * kLnTileK, m0);
                    ptx::tma_load_2d(sB + (size_t)st * kLnBBytes, &wmap, &full[st], ks * kLnTileK, n0);
                }
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer
        constexpr uint32_t idesc = ptx::umma_idesc_f16(kLnTileM, kLnTileN, BF ? 1 : 0, 0, 0);  // x, W both K-major
        if (lane == 0) {
            int g = 0, t = 0;  // t: tiles so far; tile t accumulates into buffer t & 1, use t / 2 of it
            bool ok = true;
            for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++t) {
                const int buf = t & 1;
                // the epilogue has drained this buffer's previous tile
                ok = ptx::mbar_wait_bounded(&acc_empty[buf], (uint32_t)(((t >> 1) & 1) ^ 1));
                if (!ok) { atomicOr(P.status, 1); break; }
                ptx::tc_fence_after_sync();
                for (int ks = 0; ks < nk; ++ks, ++g) {
                    const int st = g % kLnStages;
                    ok = ptx::mbar_wait_bounded(&full[st], (uint32_t)((g / kLnStages) & 1));
                    if (!ok) { atomicOr(P.status, 1); break; }
                    ptx::tc_fence_after_sync();
                    const uint32_t a_addr = ptx::smem_u32(sA + (size_t)st * kLnABytes);
                    const uint32_t b_addr = ptx::smem_u32(sB + (size_t)st * kLnBBytes);
#pragma unroll
                    for (int k = 0; k < kLnTileK / 16; ++k)
                        ptx::umma_ss(tmem + buf * kLnTileN, ptx::umma_desc_sw128(a_addr + k * 32, 16, 1024),
                                     ptx::umma_desc_sw128(b_addr + k * 32, 16, 1024), idesc, (ks > 0 || k > 0) ? 1u : 0u);
                    ptx::umma_commit(&empty[st]);
                }
                ptx::umma_commit(&acc_full[buf]);  // also after a failed wait: the epilogue must not hang
            }
        }
        __syncwarp();
    } else {
        // ---- epilogue: thread = accumulator row (a warp reaches the TMEM lanes of its quadrant)
        const int quad = warp & 3;
        const T* bias = reinterpret_cast<const T*>(P.bias);
        int t = 0;
        for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++t) {
            const int buf = t & 1;
            const int n0 = (tile % tiles_n) * kLnTileN, m0 = (tile / tiles_n) * kLnTileM;
            const int row = m0 + quad * 32 + lane;
            const bool live = row < P.M;
            const bool ok = __all_sync(0xffffffffu, ptx::mbar_wait_bounded(&acc_full[buf], (uint32_t)((t >> 1) & 1)) ? 1 : 0) != 0;
            ptx::tc_fence_after_sync();
            if (!ok) {
                if (lane == 0) atomicOr(P.status, 1);
                break;
            }
            float sum = 0.f, sumsq = 0.f;
            T* orow = reinterpret_cast<T*>(P.out) + (int64_t)row * P.N;
            if (nk > 0) {
#pragma unroll 1
                for (int c = 0; c < kLnTileN / 32; ++c) {
                    const int col0 = n0 + c * 32;
                    if (col0 >= P.N) break;  // uniform
                    uint32_t w[32];
                    ptx::tmem_ld32(tmem + ((uint32_t)(quad * 32) << 16) + buf * kLnTileN + c * 32, w);
                    ptx::tmem_wait_ld();
                    uint32_t pk[16];
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        float a = __uint_as_float(w[i]), b2 = __uint_as_float(w[i + 1]);
                        if (bias) {
                            if (col0 + i < P.N) a += Num<T>::to_f(bias[col0 + i]);
                            if (col0 + i + 1 < P.N) b2 += Num<T>::to_f(bias[col0 + i + 1]);
                        }
                        const T ra = Num<T>::from_f(a), rb = Num<T>::from_f(b2);
                        const float fa = Num<T>::to_f(ra), fb = Num<T>::to_f(rb);
                        if (col0 + i < P.N) { sum += fa; sumsq = fmaf(fa, fa, sumsq); }
                        if (col0 + i + 1 < P.N) { sum += fb; sumsq = fmaf(fb, fb, sumsq); }
                        pk[i >> 1] = (uint32_t)(*reinterpret_cast<const uint16_t*>(&ra)) |
                                     ((uint32_t)(*reinterpret_cast<const uint16_t*>(&rb)) << 16);
                    }
                    if (live) {
                        if (col0 + 32 <= P.N) {
                            uint4* dst = reinterpret_cast<uint4*>(orow + col0);  // N % 8 == 0: 16-byte aligned
#pragma unroll
                            for (int i = 0; i < 4; ++i) dst[i] = make_uint4(pk[4 * i], pk[4 * i + 1], pk[4 * i + 2], pk[4 * i + 3]);
                        } else {
                            for (int i = 0; i < 32 && col0 + i < P.N; ++i)
                                reinterpret_cast<uint16_t*>(orow)[col0 + i] = (uint16_t)(pk[i >> 1] >> ((i & 1) * 16));
                        }
                    }
                }
            }
            // the accumulator is in registers / stored: the issuer may reuse the buffer
            ptx::tc_fence_before_sync();
            ptx::mbar_arrive(&acc_empty[buf]);
            if (live && nk > 0) {
                float* st = P.stats + ((int64_t)row * kLnStatSlots + ((tile % tiles_n) % kLnStatSlots)) * 2;
                atomicAdd(st, sum);
                atomicAdd(st + 1, sumsq);
            }
        }
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem, 2 * kLnTileN);
    }
}

// Plain GEMM for everything else: 32x32 tiles through shared memory, fp32 accumulate.
template <typename T>
__global__ void __launch_bounds__(1024)
linear_stats_generic_kernel(const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ bias,
                            T* __restrict__ out, float* __restrict__ stats, int M, int N, int K) {
    __shared__ float sx[32][33], sw[32][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int row = blockIdx.y * 32 + ty, col = blockIdx.x * 32 + tx;
    float acc = 0.f;
    for (int k0 = 0; k0 < K; k0 += 32) {
        const int kx = k0 + tx;
        sx[ty][tx] = (row < M && kx < K) ? Num<T>::to_f(x[(int64_t)row * K + kx]) : 0.f;
        const int wr = blockIdx.x * 32 + ty;
        sw[ty][tx] = (wr < N && kx < K) ? Num<T>::to_f(w[(int64_t)wr * K + kx]) : 0.f;
        __syncthreads();
#pragma unroll
        for (int k = 0; k < 32; ++k) acc = fmaf(sx[ty][k], sw[tx][k], acc);
        __syncthreads();
    }
    float v = 0.f;
    if (row < M && col < N) {
        if (bias) acc += Num<T>::to_f(bias[col]);
        const T r = Num<T>::from_f(acc);
        out[(int64_t)row * N + col] = r;
        v = Num<T>::to_f(r);
    }
    const float s = warp_sum(v), q = warp_sum(v * v);
    if (tx == 0 && row < M) {
        float* st = stats + ((int64_t)row * kLnStatSlots + (blockIdx.x % kLnStatSlots)) * 2;
        atomicAdd(st, s);
        atomicAdd(st + 1, q);
    }
}

// Up to eight rows of x (decode): the weight matrix is streamed once at HBM speed, one warp per
// output column, 16-byte loads along K, fp32 accumulate. 2*N*K*e bytes of weights dominate.
constexpr int kLnSmallM = 8;
template <typename T>
__global__ void __launch_bounds__(256, 4)
linear_stats_small_m_kernel(const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ bias,
                            T* __restrict__ out, float* __restrict__ stats, int M, int N, int K) {
    constexpr int V = 16 / sizeof(T);
    struct alignas(16) Vec { T v[V]; };
    __shared__ float part[8][kLnSmallM];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * 8 + warp;
    float acc[kLnSmallM];
#pragma unroll
    for (int m = 0; m < kLnSmallM; ++m) acc[m] = 0.f;
    if (n < N) {
        const Vec* wr = reinterpret_cast<const Vec*>(w + (int64_t)n * K);
        const int nv = K / V;
        // four 16-byte weight loads in flight per lane (2 KB of the row per warp), then the math;
        // registers are kept to 64 so that four CTAs fit an SM
        for (int kv0 = 0; kv0 < nv; kv0 += 4 * 32) {
            Vec wv[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int kv = kv0 + u * 32 + lane;
                if (kv < nv) wv[u] = wr[kv];
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int kv = kv0 + u * 32 + lane;
                if (kv < nv) {
#pragma unroll
                    for (int m = 0; m < kLnSmallM; ++m) {
                        if (m < M) {
                            const Vec xv = reinterpret_cast<const Vec*>(x + (int64_t)m * K)[kv];
#pragma unroll
                            for (int j = 0; j < V; ++j)
                                acc[m] = fmaf(Num<T>::to_f(xv.v[j]), Num<T>::to_f(wv[u].v[j]), acc[m]);
                        }
                    }
                }
            }
        }
    }
#pragma unroll
    for (int m = 0; m < kLnSmallM; ++m) {
        float v = warp_sum(acc[m]);
        float y = 0.f;
        if (n < N && m < M) {
            if (bias) v += Num<T>::to_f(bias[n]);
            const T r = Num<T>::from_f(v);
            if (lane == 0) out[(int64_t)m * N + n] = r;
            y = Num<T>::to_f(r);
        }
        if (lane == 0) part[warp][m] = y;
    }
    __syncthreads();
    if (threadIdx.x < M) {
        float s1 = 0.f, s2 = 0.f;
#pragma unroll
        for (int wv = 0; wv < 8; ++wv) { const float y = part[wv][threadIdx.x]; s1 += y; s2 = fmaf(y, y, s2); }
        float* st = stats + ((int64_t)threadIdx.x * kLnStatSlots + (blockIdx.x % kLnStatSlots)) * 2;
        atomicAdd(st, s1);
        atomicAdd(st + 1, s2);
    }
}

// The norm over y (in `out`), one warp per row, following the reference's rounding:
//   RMS:   o = round(y * rsqrt(mean(y^2) + eps)); o = round(o * gamma)
//   Layer: o = round((y - mean) * rstd * gamma + beta)
template <typename T>
__global__ void __launch_bounds__(256)
norm_rows_kernel(T* __restrict__ out, const float* __restrict__ stats, const T* __restrict__ gamma,
                 const T* __restrict__ beta, int64_t M, int N, float eps, int rms) {
    constexpr int V = 16 / sizeof(T);
    for (int64_t row = blockIdx.x; row < M; row += gridDim.x) {  // one CTA per row
        float s = 0.f, q = 0.f;
#pragma unroll
        for (int i = 0; i < kLnStatSlots; ++i) {
            s += stats[(row * kLnStatSlots + i) * 2];
            q += stats[(row * kLnStatSlots + i) * 2 + 1];
        }
        const float mean = rms ? 0.f : s / (float)N;
        const float var = rms ? q / (float)N : fmaxf(q / (float)N - mean * mean, 0.f);
        const float rstd = rsqrtf(var + eps);
        T* r = out + row * (int64_t)N;
        auto one = [&](T y, int c) -> T {
            const float yf = Num<T>::to_f(y);
            if (rms) {
                const T o = Num<T>::from_f(yf * rstd);
                return gamma ? mul_r<T>(o, gamma[c]) : o;
            }
            float o = (yf - mean) * rstd;
            if (gamma) o *= Num<T>::to_f(gamma[c]);
            if (beta) o += Num<T>::to_f(beta[c]);
            return Num<T>::from_f(o);
        };
        if (N % V == 0 && ((uintptr_t)r % 16) == 0) {
            struct alignas(16) Vec { T v[V]; };
            Vec* rv = reinterpret_cast<Vec*>(r);
            for (int i = threadIdx.x; i < N / V; i += blockDim.x) {
                Vec p = rv[i];
#pragma unroll
                for (int j = 0; j < V; ++j) p.v[j] = one(p.v[j], i * V + j);
                rv[i] = p;
            }
        } else {
            for (int c = threadIdx.x; c < N; c += blockDim.x) r[c] = one(r[c], c);
        }
    }
}

template <typename T>
static int launch_ln_tc(const CUtensorMap& xm, const CUtensorMap& wm, const LnGemmParams& P, dim3 grid, cudaStream_t s) {
    auto kern = linear_stats_tc_kernel<T>;
    static PerDeviceOnce attr_set;  // per instantiation
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr_set.done(dev)) {
        cudaError_t ce = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kLnSmem);
        if (ce != cudaSuccess) return fail(RFX_CUDA_ERROR, "linear GEMM smem opt-in: %s", cudaGetErrorString(ce));
        attr_set.mark(dev);
    }
    kern<<<grid, kLnThreads, kLnSmem, s>>>(xm, wm, P);
    return check_launch("rfx_fused_linear_norm (GEMM)");
}

static int validate_ln(const RfxLinearNormArgs* a, const char* name) {
    if (!a) return fail(RFX_INVALID_ARGUMENT, "%s: null args", name);
    RFX_REQUIRE(dtype_ok(a->dtype), "%s: unknown dtype %d", name, a->dtype);
    RFX_REQUIRE(a->M >= 0 && a->K > 0 && a->N > 0 && a->M < (1ll << 31) && a->N < (1ll << 31) && a->K < (1ll << 31),
                "%s: bad sizes", name);
    RFX_REQUIRE(a->norm_type == 0 || a->norm_type == 1, "%s: norm_type must be 0 (layer) or 1 (rms)", name);
    RFX_REQUIRE(a->norm_type == 0 || a->beta == nullptr, "%s: RMSNorm takes no beta", name);
    return RFX_SUCCESS;
}

static bool ln_tensor_ok(const RfxLinearNormArgs* a) {
    if (a->force_generic || (debug_flags() & kDbgNoTensorCore)) return false;
    if (a->dtype != RFX_BF16 && a->dtype != RFX_F16) return false;
    if (a->K % 8 || a->N % 8) return false;  // 16-byte row pitch for the tensor maps and the vector stores
    if (((uintptr_t)a->x % 16) || ((uintptr_t)a->weight % 16) || ((uintptr_t)a->out % 16)) return false;
    return true;
}

static bool ln_small_m_ok(const RfxLinearNormArgs* a) {
    if (a->force_generic || a->dtype == RFX_F32 || a->M > kLnSmallM) return false;
    if (a->K % 8 || ((uintptr_t)a->x % 16) || ((uintptr_t)a->weight % 16)) return false;
    return true;
}

static size_t ln_ws_bytes(const RfxLinearNormArgs* a) {
    return round_up<size_t>((size_t)a->M * kLnStatSlots * 8 + 256, 256);
}

}  // namespace rfx

extern "C" size_t rfx_fused_linear_norm_workspace_bytes(const RfxLinearNormArgs* a) {
    if (rfx::validate_ln(a, "rfx_fused_linear_norm_workspace_bytes") != RFX_SUCCESS) return 0;
    return rfx::ln_ws_bytes(a);
}

extern "C" int rfx_fused_linear_norm_kernel_kind(const RfxLinearNormArgs* a) {
    if (rfx::validate_ln(a, "rfx_fused_linear_norm_kernel_kind") != RFX_SUCCESS) return -1;
    if (rfx::ln_small_m_ok(a)) return 2;
    return rfx::ln_tensor_ok(a) ? 1 : 0;
}

extern "C" int rfx_fused_linear_norm(const RfxLinearNormArgs* a) {
    using namespace rfx;
    const char* name = "rfx_fused_linear_norm";
    int st = validate_ln(a, name);
    if (st != RFX_SUCCESS) return st;
    if (a->M == 0) return RFX_SUCCESS;
    RFX_REQUIRE(a->x && a->weight && a->out && a->workspace, "%s: null pointer", name);
    st = check_device();
    if (st != RFX_SUCCESS) return st;
    if (a->workspace_bytes < ln_ws_bytes(a))
        return fail(RFX_WORKSPACE_TOO_SMALL, "%s: workspace %zu B < %zu B", name, a->workspace_bytes, ln_ws_bytes(a));
    RFX_REQUIRE(((uintptr_t)a->workspace % 256) == 0, "%s: workspace must be 256-byte aligned", name);
    cudaStream_t s = as_stream(a->stream);
    // [0, 256): status word; then the row statistics
    int32_t* status = (int32_t*)a->workspace;
    float* stats = (float*)((char*)a->workspace + 256);
    cudaError_t e = cudaMemsetAsync(a->workspace, 0, ln_ws_bytes(a), s);
    if (e != cudaSuccess) return fail(RFX_CUDA_ERROR, "%s: cudaMemsetAsync: %s", name, cudaGetErrorString(e));

    const int M = (int)a->M, N = (int)a->N, K = (int)a->K;
    bool done = false;
    if (ln_small_m_ok(a)) {
        RFX_DISPATCH_DTYPE(a->dtype, T, {
            linear_stats_small_m_kernel<T><<<(unsigned)ceil_div(N, 8), 256, 0, s>>>(
                (const T*)a->x, (const T*)a->weight, (const T*)a->bias, (T*)a->out, stats, M, N, K);
        });
        st = check_launch(name);
        if (st != RFX_SUCCESS) return st;
        done = true;
    }
    if (!done && ln_tensor_ok(a)) {
        CUtensorMap xm, wm;
        const uint64_t xd[2] = {(uint64_t)K, (uint64_t)M}, wd[2] = {(uint64_t)K, (uint64_t)N};
        const uint64_t str[1] = {(uint64_t)K * 2};
        const uint32_t xb[2] = {kLnTileK, kLnTileM}, wb[2] = {kLnTileK, kLnTileN};
        if (!encode_tiled_16bit(&xm, a->x, 2, xd, str, xb) && !encode_tiled_16bit(&wm, a->weight, 2, wd, str, wb)) {
            LnGemmParams P;
            P.bias = a->bias; P.out = a->out; P.stats = stats; P.status = status;
            P.M = M; P.N = N; P.K = K;
            const int tiles = ceil_div(N, kLnTileN) * ceil_div(M, kLnTileM);
            const dim3 grid((unsigned)(tiles < sm_count() ? tiles : sm_count()));
            st = a->dtype == RFX_BF16 ? launch_ln_tc<__nv_bfloat16>(xm, wm, P, grid, s)
                                      : launch_ln_tc<__half>(xm, wm, P, grid, s);
            if (st != RFX_SUCCESS) return st;
            done = true;
        }
    }
    if (!done) {
        const dim3 grid((unsigned)ceil_div(N, 32), (unsigned)ceil_div(M, 32));
        RFX_DISPATCH_DTYPE(a->dtype, T, {
            linear_stats_generic_kernel<T><<<grid, 1024, 0, s>>>((const T*)a->x, (const T*)a->weight, (const T*)a->bias,
                                                                (T*)a->out, stats, M, N, K);
        });
        st = check_launch(name);
        if (st != RFX_SUCCESS) return st;
    }
    int64_t blocks = a->M;
    const int64_t cap = (int64_t)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    RFX_DISPATCH_DTYPE(a->dtype, T, {
        norm_rows_kernel<T><<<(int)blocks, 256, 0, s>>>((T*)a->out, stats, (const T*)a->gamma, (const T*)a->beta, a->M, N,
                                                       a->eps, a->norm_type);
    });
    return check_launch(name);
}
