// Row softmax / log-softmax (the public online_softmax op). One CTA per row; the row is
// read from HBM once into shared memory as fp32 (rows up to 50k elements fit the 227 KB
// of an sm_100 CTA), reduced with warp shuffles, and written once: 2*numel*e bytes of
// traffic, which is the reference's own byte accounting (benchmark/bench_softmax.py:34).
// Rows too long for shared memory take three passes over global memory instead.
#include "common.cuh"

namespace rfx {

constexpr int kSoftmaxMaxSmemFloats = 51200;  // 200 KiB

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

template <typename T, bool STAGED>
__global__ void softmax_rows_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t rows, int n,
                                    int causal, int is_log) {
    extern __shared__ float srow[];
    __shared__ float red[32];
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const T* xr = x + row * (int64_t)n;
        T* yr = y + row * (int64_t)n;
        const int valid = causal ? (int)(row % n) + 1 : n;  // columns [0, valid) take part
        float m = -INFINITY;
        for (int i = threadIdx.x; i < valid; i += blockDim.x) {
            const float v = Num<T>::to_f(xr[i]);
            if (STAGED) srow[i] = v;
            m = fmaxf(m, v);
        }
        m = block_reduce(m, true, red);
        float l = 0.f;
        for (int i = threadIdx.x; i < valid; i += blockDim.x) {
            const float v = STAGED ? srow[i] : Num<T>::to_f(xr[i]);
            const float e = expf(v - m);
            if (STAGED && !is_log) srow[i] = e;
            l += e;
        }
        l = block_reduce(l, false, red);
        const float logl = logf(l);
        for (int i = threadIdx.x; i < n; i += blockDim.x) {
            float o;
            if (i >= valid) {
                o = is_log ? -INFINITY : 0.f;
            } else if (is_log) {
                const float v = STAGED ? srow[i] : Num<T>::to_f(xr[i]);
                o = (v - m) - logl;
            } else {
                const float e = STAGED ? srow[i] : expf(Num<T>::to_f(xr[i]) - m);
                o = e / l;
            }
            yr[i] = Num<T>::from_f(o);
        }
        __syncthreads();  // srow is reused by the next row
    }
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
    int threads = n <= 512 ? 64 : n <= 4096 ? 128 : n <= 16384 ? 256 : 512;
    const bool staged = n <= kSoftmaxMaxSmemFloats;
    const size_t smem = staged ? (size_t)n * sizeof(float) : 0;
    int64_t grid = a->rows;
    const int64_t cap = (int64_t)sm_count() * 32;
    if (grid > cap) grid = cap;
    cudaStream_t s = as_stream(a->stream);
    RFX_DISPATCH_DTYPE(a->dtype, T, {
        if (staged) {
            auto kern = softmax_rows_kernel<T, true>;
            if (smem > 48 * 1024) {
                cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
                if (e != cudaSuccess) return fail(RFX_CUDA_ERROR, "%s: smem opt-in: %s", name, cudaGetErrorString(e));
            }
            kern<<<(int)grid, threads, smem, s>>>((const T*)a->x, (T*)a->y, a->rows, n, a->is_causal, a->log);
        } else {
            softmax_rows_kernel<T, false><<<(int)grid, threads, 0, s>>>((const T*)a->x, (T*)a->y, a->rows, n,
                                                                      a->is_causal, a->log);
        }
    });
    return check_launch(name);
}
