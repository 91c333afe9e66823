// Status plumbing and device checks shared by every entry point of libreflex_b200.
#include <stdarg.h>
#include <stdlib.h>
#include <string.h>

#include <mutex>

#include "common.cuh"

namespace rfx {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int fail(int status, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return status;
}

struct DevInfo {
    int known = 0;  // 0 unknown, 1 ok, 2 unsupported, 3 error
    int sms = 0;
    int major = 0, minor = 0;
};
static DevInfo g_dev[64];
static std::mutex g_dev_mutex;

static int probe(int dev) {
    std::lock_guard<std::mutex> lock(g_dev_mutex);
    DevInfo& d = g_dev[dev];
    if (d.known) return d.known;
    cudaDeviceProp p;
    cudaError_t e = cudaGetDeviceProperties(&p, dev);
    if (e != cudaSuccess) {
        set_error("cudaGetDeviceProperties: %s", cudaGetErrorString(e));
        return 3;
    }
    d.sms = p.multiProcessorCount;
    d.major = p.major;
    d.minor = p.minor;
    d.known = (p.major == 10) ? 1 : 2;
    return d.known;
}

int check_device() {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(RFX_CUDA_ERROR, "cudaGetDevice: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= 64) return fail(RFX_UNSUPPORTED_DEVICE, "device ordinal %d out of range", dev);
    int k = probe(dev);
    if (k == 1) return RFX_SUCCESS;
    if (k == 2)
        return fail(RFX_UNSUPPORTED_DEVICE,
                    "device %d is sm_%d%d; this library is built for sm_100a (B200) only",
                    dev, g_dev[dev].major, g_dev[dev].minor);
    return RFX_CUDA_ERROR;
}

int sm_count() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (probe(dev) == 3) return 148;
    return g_dev[dev].sms > 0 ? g_dev[dev].sms : 148;
}

static uint32_t parse_debug_words(const char* csv) {
    uint32_t f = 0;
    if (!csv) return 0;
    const char* p = csv;
    while (*p) {
        const char* e = strchr(p, ',');
        const size_t n = e ? (size_t)(e - p) : strlen(p);
        auto is = [&](const char* w) { return strlen(w) == n && strncmp(p, w, n) == 0; };
        if (is("no_tc")) f |= kDbgNoTensorCore;
        else if (is("prefill_nosplit")) f |= kDbgPrefillNoSplit;
        else if (is("mixed=1")) f |= kDbgMixedOn;
        else if (is("mixed=0")) f |= kDbgMixedOff;
        else if (is("tma2d")) f |= kDbgTma2d;
        p += n + (e ? 1 : 0);
    }
    return f;
}

static std::atomic<uint32_t> g_debug_flags{0};
static std::atomic<int> g_debug_set{0};  // 1: rfx_debug_set_flags has spoken
static std::once_flag g_debug_env_once;

uint32_t debug_flags() {
    if (g_debug_set.load(std::memory_order_acquire)) return g_debug_flags.load(std::memory_order_acquire);
    static uint32_t from_env = 0;
    std::call_once(g_debug_env_once, [] { from_env = parse_debug_words(getenv("REFLEX_B200_DEBUG")); });
    return from_env;
}

int check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(RFX_CUDA_ERROR, "%s: %s", what, cudaGetErrorString(e));
    return RFX_SUCCESS;
}

}  // namespace rfx

extern "C" {

int rfx_abi_version(void) { return RFX_ABI_VERSION; }

const char* rfx_last_error(void) { return rfx::g_err; }

int rfx_debug_set_flags(const char* words) {
    using namespace rfx;
    if (!words) {  // back to what the environment said
        g_debug_set.store(0, std::memory_order_release);
        return RFX_SUCCESS;
    }
    g_debug_flags.store(parse_debug_words(words), std::memory_order_release);
    g_debug_set.store(1, std::memory_order_release);
    return RFX_SUCCESS;
}

size_t rfx_args_size(int which) {
    switch (which) {
        case 0: return sizeof(RfxKvAppendArgs);
        case 1: return sizeof(RfxKvLookupArgs);
        case 2: return sizeof(RfxRopeArgs);
        case 3: return sizeof(RfxRopeTableArgs);
        case 4: return sizeof(RfxRopeAppendArgs);
        case 5: return sizeof(RfxSoftmaxArgs);
        case 6: return sizeof(RfxAttentionArgs);
        case 7: return sizeof(RfxPagedAttentionArgs);
        case 8: return sizeof(RfxCombineArgs);
        case 9: return sizeof(RfxHeadGatherArgs);
        case 10: return sizeof(RfxPeerHandle);
        case 11: return sizeof(RfxLinearNormArgs);
        default: return 0;
    }
}

const char* rfx_status_string(int s) {
    switch (s) {
        case RFX_SUCCESS: return "Success";
        case RFX_UNSUPPORTED_DEVICE: return "UnsupportedDevice";
        case RFX_UNSUPPORTED_MODEL: return "UnsupportedModel";
        case RFX_UNSUPPORTED_QUANT_FORMAT: return "UnsupportedQuantFormat";
        case RFX_INVALID_ARGUMENT: return "InvalidArgument";
        case RFX_NOT_IMPLEMENTED: return "NotImplemented";
        case RFX_CUDA_ERROR: return "CudaError";
        case RFX_TIMEOUT: return "Timeout";
        case RFX_WORKSPACE_TOO_SMALL: return "WorkspaceTooSmall";
        default: return "Unknown";
    }
}

}  // extern "C"
