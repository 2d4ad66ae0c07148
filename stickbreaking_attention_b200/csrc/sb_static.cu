// sbattn_fwd_static: a forward pass for callers that cannot allocate device memory.
//
// The ordinary forward needs a workspace from its caller (the table of work items built on the device, plus the
// carries when a backward follows).  Some hosts cannot provide one: a serving runtime that has handed all device
// memory to its own pool and forbids further cudaMalloc calls, a plugin loaded into a process whose allocator it may
// not touch, code running inside a region where allocation is not permitted.  For those, this entry point keeps the
// workspace of a gradient-free forward in a fixed array that is part of the library image.
#include <mutex>

#include "sb_common.cuh"

namespace {

constexpr size_t kStaticScratchBytes = 1u << 20;  // 1 MiB per GPU that loads the library, held until the process exits

// In host code this name is only a handle for the symbol, not a device address: the address is looked up once
// per device below and that pointer is what the kernels receive.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
void* g_scratch_ptr[kMaxDevices] = {nullptr};
std::mutex g_scratch_mutex;

// device address of the scratch array on the current device (0 on failure)
void* scratch_for_current_device(int* err) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        *err = SBATTN_ECUDA;
        return nullptr;
    }
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (!g_scratch_ptr[dev]) {
        void* ptr = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
        if (e != cudaSuccess || !ptr) {
            *err = SBATTN_ECUDA;
            return nullptr;
        }
        g_scratch_ptr[dev] = ptr;
    }
    return g_scratch_ptr[dev];
}

}  // namespace

extern "C" size_t sbattn_static_scratch_bytes(void) { return kStaticScratchBytes; }

extern "C" int sbattn_fwd_static(const SbParams* p) {
    if (!p) return SBATTN_ENULL;
    SbParams q = *p;
    q.save_carries = 0;  // no backward can follow: the carries would not fit a fixed array
    size_t need = 0;
    const int rc = sbattn_workspace_bytes(&q, &need, nullptr);
    if (rc != SBATTN_OK) return rc;
    if (need > kStaticScratchBytes) return SBATTN_ECAPACITY;
    int err = SBATTN_OK;
    void* scratch = scratch_for_current_device(&err);
    if (!scratch) return err;
    q.fwd_workspace = scratch;
    q.fwd_workspace_bytes = kStaticScratchBytes;
    return sbattn_fwd(&q);
}
