// escha_coded_gemv_static: the tensor-core coded GEMV for callers that cannot
// hand the library a workspace because they cannot allocate device memory
// themselves.
//
// Who that is: a plugin running inside a host runtime that owns every byte of
// device memory (an inference server with a pre-sized arena, an embedded
// runtime with a fixed memory map), a callback invoked from a context where the
// host allocator must not be re-entered, or a decode loop that cannot afford
// cudaMalloc's implicit device-wide synchronisation.  Such a caller still owns
// its inputs and outputs, but has nowhere to get the split-K scratch from.
//
// Here the scratch lives in a file-scope device array that is part of the
// library image: every GPU that loads the library carries it until the process
// exits (8.06 MiB).  Nothing in this file calls cudaMalloc, cudaFree or any
// allocating routine.
//
// Consequences the caller must know:
//  * The array is shared by every call on a device and keeps the previous
//    call's contents.  Two calls that may overlap on the GPU (different streams
//    with no ordering between them) race on it; serialise them.
//  * The first call on each device performs a one-time set-up (it resolves the
//    array's device address and clears its counter region).  Make that first
//    call outside any stream capture.
//  * Problem sizes are bounded by the array; larger ones are refused with
//    ESCHA_EINVAL and a message, never truncated.
#include <cstdio>

#include "../../include/escha_b200.h"
#include "kernels.h"

namespace {

constexpr size_t kStaticCounterBytes = 64 * 1024;        // 16384 (job, output block) counters
constexpr size_t kStaticPartialBytes = 8 * 1024 * 1024;  // split-K partial sums
constexpr size_t kStaticBytes = kStaticCounterBytes + kStaticPartialBytes;

// The scratch itself.  In host code this name is only a stand-in for the
// symbol, not a device address: it must be resolved with cudaGetSymbolAddress
// before a kernel can be given a pointer to it.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticBytes];

struct DeviceSlot {
    void* base = nullptr;  // resolved device address of g_static_scratch on this device
};
DeviceSlot g_slots[64];
std::mutex g_slots_mu;   // the one-time set-up below may be reached from several host threads

}  // namespace

extern "C" int escha_coded_gemv_static(const void* xh, const void* code, const float* rout, int M,
                                       int IC, int OC, int K, int splits, float rs, void* out,
                                       void* stream) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64) {
        escha::set_last_error("escha_coded_gemv_static: cannot identify the current device");
        return ESCHA_ECUDA;
    }
    // size limits first: nothing below may exceed the static array
    if (M < 1 || M > 16) {
        escha::set_last_error("escha_coded_gemv_static: M must be in [1, 16] (the static scratch "
                             "holds one row group)");
        return ESCHA_EINVAL;
    }
    if (IC < 128 || OC < 128 || IC % 128 || OC % 128) {
        escha::set_last_error("escha_coded_gemv_static: dimensions must be positive multiples of 128");
        return ESCHA_EINVAL;
    }
    if (splits <= 0) splits = escha_coded_gemv_splits(IC, OC, 1, 0);
    const int rows_per_job = M <= 8 ? 8 : 16;
    const size_t ocb = static_cast<size_t>(OC / 128);
    const size_t need = splits > 1 ? static_cast<size_t>(splits) * ocb * rows_per_job * 128u * sizeof(float) : 0;
    if (need > kStaticPartialBytes || ocb * sizeof(int32_t) > kStaticCounterBytes) {
        char msg[256];
        snprintf(msg, sizeof(msg),
                 "escha_coded_gemv_static: %d splits x %zu output blocks x %d rows need %zu bytes of "
                 "scratch; the static array holds %zu (use escha_coded_gemv with a caller workspace)",
                 splits, ocb, rows_per_job, need, kStaticPartialBytes);
        escha::set_last_error(msg);
        return ESCHA_EINVAL;
    }
    DeviceSlot& slot = g_slots[dev];
    std::unique_lock<std::mutex> setup_lock(g_slots_mu);
    if (slot.base == nullptr) {
        // one-time set-up for this device, with this device current
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_static_scratch);
        if (e != cudaSuccess || ptr == nullptr) {
            escha::set_last_error("escha_coded_gemv_static: cudaGetSymbolAddress failed for the static scratch");
            return ESCHA_ECUDA;
        }
        // counters must start at zero; kernels leave them zero afterwards
        e = cudaMemsetAsync(ptr, 0, kStaticCounterBytes, static_cast<cudaStream_t>(stream));
        if (e != cudaSuccess) {
            escha::set_last_error("escha_coded_gemv_static: clearing the counter region failed");
            return ESCHA_ECUDA;
        }
        slot.base = ptr;
    }
    setup_lock.unlock();
    return escha::coded_gemv_with_scratch(xh, code, rout, M, IC, OC, K, splits, rs,
                                         static_cast<int32_t*>(slot.base),
                                         reinterpret_cast<float*>(static_cast<unsigned char*>(slot.base) +
                                                                  kStaticCounterBytes),
                                         out, stream);
}
