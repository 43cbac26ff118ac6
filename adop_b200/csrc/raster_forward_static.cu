// adop_raster_forward_static: the forward pass for callers that cannot provide a workspace.
//
// adop_raster_forward needs a scratch buffer that the caller allocates with cudaMalloc (or a framework allocator).
// Some hosts of this library cannot do that: code that runs inside a region where the allocator is off limits (a
// render callback that must not touch the CUDA memory pool, a plugin whose host application owns all device memory
// and hands out only input and output buffers), or a process whose memory budget was fixed up front. For them the
// scratch lives here, in a file-scope device array that exists on every GPU that loads the library, from the moment
// the module is loaded until the process exits.
//
// The array's name is a device symbol. In host code it is only a stand-in: the address that kernels can use comes from
// cudaGetSymbolAddress, asked once per device with that device current, and is then passed on like any other pointer.
#include <mutex>

#include "common.cuh"

namespace adop {

// 32 MiB: enough for a 4-layer pyramid of up to about 780 000 layer-0 pixels with 4 descriptor channels (32 bytes of
// scratch per pyramid pixel), e.g. 1024 x 576; less with more channels. See adop_raster_static_scratch_bytes().
constexpr size_t kStaticScratchBytes = size_t(32) << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
static std::mutex g_static_mutex;
static void* g_static_ptr[kMaxDevices] = {nullptr};

// Device address of the array on the current device; resolved on the first call per device.
static adop_status static_scratch_address(void** out)
{
    int dev = -1;
    ADOP_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return ADOP_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> lock(g_static_mutex);
    if (!g_static_ptr[dev])
    {
        void* p = nullptr;
        ADOP_CUDA_TRY(cudaGetSymbolAddress(&p, g_static_scratch));
        if (!p) return ADOP_ERR_CUDA;
        g_static_ptr[dev] = p;
    }
    *out = g_static_ptr[dev];
    return ADOP_OK;
}

}  // namespace adop

using namespace adop;

extern "C" size_t adop_raster_static_scratch_bytes(void) { return kStaticScratchBytes; }

extern "C" adop_status adop_raster_forward_static(const adop_scene* scene, const adop_view* views, int32_t num_views,
                                                  const adop_render_params* params, int32_t num_layers,
                                                  adop_forward_io* io, void* stream)
{
    if (!scene || !views || !io || num_views <= 0) return ADOP_ERR_INVALID_ARGUMENT;
    const size_t need = adop_raster_workspace_bytes(views[0].w, views[0].h, num_layers, scene->channels);
    if (need == 0) return ADOP_ERR_INVALID_ARGUMENT;
    if (need > kStaticScratchBytes)
    {
        snprintf(last_error_buffer(), 512,
                 "adop_raster_forward_static: a %d x %d view with %d layers and %d channels needs %zu bytes of scratch, "
                 "the built-in array holds %zu; use adop_raster_forward with a caller-owned workspace",
                 views[0].w, views[0].h, num_layers, scene->channels, need, kStaticScratchBytes);
        return ADOP_ERR_SIZE_LIMIT;
    }
    void* scratch = nullptr;
    adop_status st = static_scratch_address(&scratch);
    if (st != ADOP_OK) return st;
    // Same pass as adop_raster_forward, pointed at the built-in array. That function clears the part of the scratch it
    // is about to use before the first kernel reads it, so whatever the previous call left behind does not matter.
    adop_forward_io local = *io;
    local.workspace = scratch;
    local.workspace_bytes = kStaticScratchBytes;
    return adop_raster_forward(scene, views, num_views, params, num_layers, &local, stream);
}
