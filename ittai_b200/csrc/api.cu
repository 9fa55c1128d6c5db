// Library-level entry points: version, per-thread error text, device check, status decoding.
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "common.cuh"

namespace ittai {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int cuda_fail(cudaError_t e, const char* what) {
    set_error("%s: %s (%s)", what, cudaGetErrorString(e), cudaGetErrorName(e));
    return ITTAI_E_CUDA;
}

}  // namespace ittai

extern "C" int ittai_version(void) { return ITTAI_ABI_VERSION; }

extern "C" const char* ittai_last_error(void) { return ittai::g_err; }

extern "C" int ittai_device_check(int device, int* n_sms) {
    cudaDeviceProp prop;
    cudaError_t e = cudaGetDeviceProperties(&prop, device);
    if (e != cudaSuccess) return ittai::cuda_fail(e, "cudaGetDeviceProperties");
    if (prop.major != 10) {
        ittai::set_error("device %d is sm_%d%d; this library is built for sm_100a only", device, prop.major, prop.minor);
        return ITTAI_E_DEVICE;
    }
    if (!prop.cooperativeLaunch) {
        ittai::set_error("device %d cannot launch cooperative grids", device);
        return ITTAI_E_DEVICE;
    }
    if (n_sms) *n_sms = prop.multiProcessorCount;
    return ITTAI_OK;
}

extern "C" int ittai_decode_status(const uint32_t* st, char* msg, size_t n) {
    if (!st) { ittai::set_error("null status"); return ITTAI_E_ARG; }
    const char* what = "ok";
    switch (st[0]) {
        case ITTAI_ST_OK: what = "ok"; break;
        case ITTAI_ST_BARRIER_TIMEOUT: what = "grid barrier wait ran out (a=tag b=cta c=arrivals seen d=arrivals expected)"; break;
        case ITTAI_ST_FLAG_TIMEOUT: what = "flag wait ran out (a=what was awaited b=cta c=tag seen d=tag expected)"; break;
        case ITTAI_ST_STREAM_TIMEOUT: what = "weight-stream copy did not land (a=entry b=cta c=slot d=parity)"; break;
        case ITTAI_ST_GEMM_TIMEOUT: what = "tensor-core GEMM pipeline wait ran out (a=cta b=k-blocks)"; break;
        case ITTAI_ST_BAD_TOKEN: what = "token id or cache position out of range (a=id b=step c=position d=sequence)"; break;
        default: what = "unknown status code"; break;
    }
    if (msg && n) snprintf(msg, n, "status %u: %s; a=%u b=%u c=%u d=%u", st[0], what, st[1], st[2], st[3], st[4]);
    if (st[0] != ITTAI_ST_OK) {
        ittai::set_error("device status %u: %s; a=%u b=%u c=%u d=%u", st[0], what, st[1], st[2], st[3], st[4]);
        return ITTAI_E_STATUS;
    }
    return ITTAI_OK;
}

static_assert(sizeof(IttaiQwen3Decode) == 40 + 22 * sizeof(void*), "IttaiQwen3Decode layout differs from the ctypes mirror");
