// cwrnnt_costs_static: the costs-only forward for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc at all: a plug-in inside a serving process whose framework has
// already claimed the whole GPU for its own memory pool and hands the plug-in nothing but input and output buffers;
// a foreign-language binding (cgo, JNI, a C host) that has no device allocator of its own to size a workspace with;
// a latency-critical scoring loop in which an allocation - an implicit device-wide synchronisation - is not
// acceptable. For them the scratch that cwrnnt_forward takes from the caller (offsets, order, the gathered
// log-probabilities, the backward variables) lives here, in one file-scope device array of fixed capacity that every
// GPU loading the library holds until the process exits.
//
// In host code the array's name is only a stand-in for the symbol, not a device address, so the address is taken
// once per device with cudaGetSymbolAddress (that device current) and that pointer is what the kernels receive.
#include <cstdio>
#include <mutex>

#include "cwrnnt_kernels.h"

namespace {

using namespace cwrnnt;

// capacity of the shared scratch: the carve for the largest accepted problem plus slack for section alignment
constexpr long long kStaticBytes =
    40LL * CWRNNT_STATIC_MAX_ROWS + 28LL * CWRNNT_STATIC_MAX_SEQUENCES + 16 * 256;

static __device__ __align__(256) unsigned char g_static_scratch[kStaticBytes];

// Device code may name the array directly. The header (4 status words + the completion ticket) is the only part
// that must start from zero on every call; everything else is fully rewritten before it is read.
__global__ void static_header_clear_kernel()
{
    if (threadIdx.x < 16) reinterpret_cast<int *>(g_static_scratch)[threadIdx.x] = 0;
}

constexpr int kMaxDevices = 64;
std::mutex g_setup_lock;
void *g_scratch_addr[kMaxDevices] = {};  // device address of g_static_scratch on each device, filled on first use

}  // namespace

extern "C" int cwrnnt_costs_static(const cwrnnt_problem *p, const void *x, const int32_t *lx, const int32_t *ly,
                                   const int32_t *y, void *costs, void *loss, cwrnnt_stream_t stream)
{
    cwrnnt_problem q;
    if (!p) return CWRNNT_ERR_ARGUMENT;
    q = *p;
    q.flags |= CWRNNT_COSTS_ONLY;
    if (cwrnnt_workspace_bytes(&q) < 0) return (q.max_u + 1 > CWRNNT_MAX_COLUMNS) ? CWRNNT_ERR_UNSUPPORTED
                                                                                 : CWRNNT_ERR_ARGUMENT;
    if (!lx || !ly || !costs || (q.n_rows > 0 && !x) || (q.max_u > 0 && !y)) return CWRNNT_ERR_ARGUMENT;
    if (q.n_rows > CWRNNT_STATIC_MAX_ROWS || q.B > CWRNNT_STATIC_MAX_SEQUENCES ||
        carve_workspace(q.n_rows, q.B, nullptr, nullptr) > kStaticBytes) {
        char msg[160];
        std::snprintf(msg, sizeof msg, "cwrnnt_costs_static accepts at most %d rows and %d sequences, got %lld and %d",
                      CWRNNT_STATIC_MAX_ROWS, CWRNNT_STATIC_MAX_SEQUENCES, static_cast<long long>(q.n_rows), q.B);
        set_last_error(msg);
        return CWRNNT_ERR_CAPACITY;
    }
    if (q.B == 0) return CWRNNT_OK;

    // one-time set-up per device: resolve the device address of the scratch symbol
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        set_last_error("cwrnnt_costs_static: cannot identify the current device");
        return CWRNNT_ERR_LAUNCH;
    }
    void *base = nullptr;
    {
        std::lock_guard<std::mutex> hold(g_setup_lock);
        if (!g_scratch_addr[dev]) {
            void *ptr = nullptr;
            e = cudaGetSymbolAddress(&ptr, g_static_scratch);
            if (e != cudaSuccess || !ptr) {
                char msg[160];
                std::snprintf(msg, sizeof msg, "cudaGetSymbolAddress(static scratch): %s", cudaGetErrorString(e));
                set_last_error(msg);
                return CWRNNT_ERR_LAUNCH;
            }
            g_scratch_addr[dev] = ptr;
        }
        base = g_scratch_addr[dev];
    }

    Workspace w{};
    carve_workspace(q.n_rows, q.B, base, &w);
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    static_header_clear_kernel<<<1, 32, 0, s>>>();
    const char *what = "static header clear";
    e = cudaGetLastError();
    if (e == cudaSuccess) what = "prep", e = launch_prep(q, lx, ly, w, costs, s, GroupPlan{1, 1}, loss);
    if (e == cudaSuccess) what = "gather", e = launch_gather(q, x, lx, ly, y, w, s);
    if (e == cudaSuccess) what = "wavefront", e = launch_wavefront(q, lx, ly, w, costs, loss, nullptr, s);
    if (e != cudaSuccess) {
        char msg[160];
        std::snprintf(msg, sizeof msg, "cwrnnt_costs_static %s: %s", what, cudaGetErrorString(e));
        set_last_error(msg);
        return CWRNNT_ERR_LAUNCH;
    }
    return CWRNNT_OK;
}

// The status words of the last cwrnnt_costs_static on the current device (the scratch is private to the library, so
// cwrnnt_read_status cannot reach them). Copies 16 bytes to HOST memory `out` and waits for the stream; allocates
// nothing. Before the first cwrnnt_costs_static on this device there is nothing to report: all-clear words come back.
extern "C" int cwrnnt_static_status(int32_t out[4], cwrnnt_stream_t stream)
{
    if (!out) return CWRNNT_ERR_ARGUMENT;
    out[0] = 0, out[1] = -1, out[2] = 0, out[3] = 0;
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        set_last_error("cwrnnt_static_status: cannot identify the current device");
        return CWRNNT_ERR_LAUNCH;
    }
    void *base = nullptr;
    {
        std::lock_guard<std::mutex> hold(g_setup_lock);
        base = g_scratch_addr[dev];
    }
    if (!base) return CWRNNT_OK;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    e = cudaMemcpyAsync(out, base, 4 * sizeof(int32_t), cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) {
        char msg[160];
        std::snprintf(msg, sizeof msg, "cwrnnt_static_status: %s", cudaGetErrorString(e));
        set_last_error(msg);
        return CWRNNT_ERR_LAUNCH;
    }
    return CWRNNT_OK;
}
