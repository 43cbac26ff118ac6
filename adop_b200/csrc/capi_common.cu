// Status strings, defaults, argument validation: the parts of the C ABI that launch nothing.
#include <string.h>

#include "common.cuh"

namespace adop {

char* last_error_buffer()
{
    static thread_local char buf[512] = {0};
    return buf;
}

adop_status record_cuda_error(cudaError_t e, const char* what)
{
    snprintf(last_error_buffer(), 512, "%s: %s (%s)", what, cudaGetErrorName(e), cudaGetErrorString(e));
    return ADOP_ERR_CUDA;
}

int sm_count()
{
    static thread_local int cached_dev = -1;
    static thread_local int cached = 148;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (dev != cached_dev)
    {
        int v = 0;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && v > 0) cached = v;
        cached_dev = dev;
    }
    return cached;
}

// the SAIGA_ASSERTs of PointRenderer.cu:902-1162 become argument checks with a status
adop_status validate_common(const adop_scene* s, const adop_view* views, int B, const adop_render_params* rp, int L)
{
    if (!s || !views || !rp) return ADOP_ERR_INVALID_ARGUMENT;
    if (B <= 0 || L <= 0 || L > ADOP_MAX_LAYERS) return ADOP_ERR_INVALID_ARGUMENT;
    if (s->num_points < 0 || s->channels <= 0 || s->channels > ADOP_MAX_CHANNELS) return ADOP_ERR_INVALID_ARGUMENT;
    if (s->num_texels <= 0 || s->num_images <= 0 || s->num_cameras <= 0) return ADOP_ERR_INVALID_ARGUMENT;
    if (!s->position || !s->texture || !s->background || !s->poses || !s->intrinsics) return ADOP_ERR_INVALID_ARGUMENT;
    if (!s->index && s->num_texels < s->num_points) return ADOP_ERR_INVALID_ARGUMENT;
    if (rp->composite_environment_map && s->env_map && (s->env_h <= 0 || s->env_w <= 0)) return ADOP_ERR_INVALID_ARGUMENT;
    const int w = views[0].w, h = views[0].h;
    if (w <= 0 || h <= 0) return ADOP_ERR_INVALID_ARGUMENT;
    if ((w >> (L - 1)) <= 0 || (h >> (L - 1)) <= 0) return ADOP_ERR_INVALID_ARGUMENT;
    // pyramid pixel count must fit the 32-bit record index
    unsigned long long total = 0;
    for (int l = 0, ww = w, hh = h; l < L; ++l, ww /= 2, hh /= 2) total += (unsigned long long)ww * hh;
    if (total >= (1ull << 31)) return ADOP_ERR_SIZE_LIMIT;
    for (int b = 0; b < B; ++b)
    {
        const adop_view& v = views[b];
        if (v.w != w || v.h != h) return ADOP_ERR_INVALID_ARGUMENT;  // one size per batch, PointRenderer.cu:954-956
        if (v.image_index < 0 || v.image_index >= s->num_images) return ADOP_ERR_INVALID_ARGUMENT;
        if (v.camera_index < 0 || v.camera_index >= s->num_cameras) return ADOP_ERR_INVALID_ARGUMENT;
        if (v.camera_model == ADOP_CAMERA_PINHOLE_DISTORTION)
        {
            if (s->intrinsics_cols < 13) return ADOP_ERR_INVALID_ARGUMENT;
        }
        else if (v.camera_model == ADOP_CAMERA_OCAM)
        {
            if (s->intrinsics_cols < 6 || s->intrinsics_cols > 5 + ADOP_MAX_OCAM_POLY) return ADOP_ERR_INVALID_ARGUMENT;
        }
        else
            return ADOP_ERR_INVALID_ARGUMENT;
    }
    return ADOP_OK;
}

}  // namespace adop

extern "C" const char* adop_status_string(adop_status s)
{
    switch (s)
    {
        case ADOP_OK: return "ok";
        case ADOP_ERR_INVALID_ARGUMENT: return "invalid argument";
        case ADOP_ERR_UNSUPPORTED: return "unsupported configuration";
        case ADOP_ERR_CUDA: return "CUDA error";
        case ADOP_ERR_WORKSPACE_TOO_SMALL: return "workspace too small";
        case ADOP_ERR_SIZE_LIMIT: return "size beyond the supported maximum";
    }
    return "unknown status";
}

extern "C" const char* adop_last_error(void) { return adop::last_error_buffer(); }

extern "C" void adop_render_params_default(adop_render_params* p)
{
    if (!p) return;
    memset(p, 0, sizeof(*p));
    p->test_backward_mode = 0;
    p->check_normal = 1;
    p->dropout = 0.25f;
    p->dropout_seed = 0;
    p->depth_accept = 0.01f;
    p->ghost_gradients = 0;
    p->drop_out_radius_threshold = 0.6f;
    p->drop_out_points_by_radius = 1;
    p->distortion_gradient_factor = 0.005f;
    p->K_gradient_factor = 0.5f;
    p->dist_cutoff = 2.f;
    p->output_background_mask = 0;
    p->output_background_mask_value = 0.f;
    p->composite_environment_map = 0;
}
