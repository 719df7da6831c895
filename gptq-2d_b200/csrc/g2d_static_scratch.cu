// g2d_sweep_fused_static: the fused sweep for callers that cannot hand over a workspace.
//
// Some hosts of this library own no device allocator of their own: a plugin loaded into an application that
// reserves all device memory at start-up and gives its plugins none, or code on a latency-critical path where a
// cudaMalloc (which synchronises the whole device) is not acceptable once the service is running.  For them the
// two scratch planes of the sweep (the down-feedback buffer C and the error buffer E) live in the fixed array
// below instead of in a caller-provided workspace.  The price: every device that loads the library carries the
// array until the process exits, problems beyond G2D_STATIC_SCRATCH_BYTES are refused, and all calls on a device
// share the one array.
#include <mutex>

#include "g2d_common.cuh"

namespace {

// Scratch shared by every call on a device.  It keeps whatever the last call left in it; the sweep clears the
// C plane itself before use and writes every E entry before reading it, so stale contents are harmless.
static __device__ __align__(256) unsigned char g2d_static_scratch[G2D_STATIC_SCRATCH_BYTES];

// In host code `g2d_static_scratch` is only a handle for the runtime, not a device address: the address each
// device gave the array is looked up once per device and kept here.
std::mutex g_setup_mutex;
void *g_scratch_address[64] = {};
bool g_scratch_ready[64] = {};

int scratch_of_current_device(void **address) {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return G2D_ERR_CUDA;
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (!g_scratch_ready[device]) {
        void *found = nullptr;
        if (cudaGetSymbolAddress(&found, g2d_static_scratch) != cudaSuccess || found == nullptr) return G2D_ERR_CUDA;
        g_scratch_address[device] = found;
        g_scratch_ready[device] = true;
    }
    *address = g_scratch_address[device];
    return G2D_OK;
}

}  // namespace

extern "C" int g2d_sweep_fused_static(const g2d_sweep_desc *desc, void *stream) {
    if (!desc) return G2D_ERR_BAD_ARGUMENT;
    g2d_sweep_desc local = *desc;
    local.workspace = nullptr;
    local.workspace_bytes = 0;
    local.reserved = 1;  // the tile schedule: its scratch is the two planes this array is sized for
    size_t need = 0;
    const int status = g2d_sweep_workspace_bytes(&local, &need);
    if (status != G2D_OK) return status;
    if (need > (size_t)G2D_STATIC_SCRATCH_BYTES) return G2D_ERR_TOO_LARGE;  // "size exceeds a fixed maximum"
    void *scratch = nullptr;
    const int found = scratch_of_current_device(&scratch);
    if (found != G2D_OK) return found;
    local.workspace = scratch;
    local.workspace_bytes = (size_t)G2D_STATIC_SCRATCH_BYTES;
    return g2d_sweep_fused(&local, stream);
}
