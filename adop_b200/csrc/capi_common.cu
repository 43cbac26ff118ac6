// Status strings, defaults, argument validation: the parts of the C ABI that launch nothing.
#include <string.h>

#include <map>
#include <string>
#include <vector>

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

namespace {
struct ProfileMark { const char* name; cudaEvent_t begin, end; };
struct ProfileState
{
    bool on = false;
    std::vector<ProfileMark> marks;
    std::vector<cudaEvent_t> pool;
};
ProfileState& profile_state()
{
    static thread_local ProfileState st;
    return st;
}
cudaEvent_t profile_event(ProfileState& ps)
{
    if (!ps.pool.empty()) { cudaEvent_t e = ps.pool.back(); ps.pool.pop_back(); return e; }
    cudaEvent_t e = nullptr;
    cudaEventCreate(&e);
    return e;
}
}  // namespace

bool profile_on() { return profile_state().on; }

void profile_mark(const char* name, cudaStream_t st, bool begin)
{
    ProfileState& ps = profile_state();
    if (begin)
    {
        ProfileMark m{name, profile_event(ps), nullptr};
        if (m.begin) cudaEventRecord(m.begin, st);
        ps.marks.push_back(m);
    }
    else if (!ps.marks.empty())
    {
        ProfileMark& m = ps.marks.back();
        m.end = profile_event(ps);
        if (m.end) cudaEventRecord(m.end, st);
    }
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
    if (s->num_points > 0x7F000000) return ADOP_ERR_SIZE_LIMIT;  // grid-stride loops index points with 32-bit ints
    if (s->num_points < 0 || s->channels <= 0 || s->channels > ADOP_MAX_CHANNELS) return ADOP_ERR_INVALID_ARGUMENT;
    if (s->num_texels <= 0 || s->num_images <= 0 || s->num_cameras <= 0) return ADOP_ERR_INVALID_ARGUMENT;
    // an empty cloud (no points, no position tensor) is a valid scene: every pixel takes the background
    if ((!s->position && s->num_points > 0) || !s->texture || !s->background || !s->poses || !s->intrinsics) return ADOP_ERR_INVALID_ARGUMENT;
    if (!s->index && s->num_texels < s->num_points) return ADOP_ERR_INVALID_ARGUMENT;
    if (s->outlier_position)
    {
        // the second cloud shares the main cloud's drop-out decisions (point i with point i), PointRenderer.cu:1437-1440
        if (s->num_outliers < 0 || s->num_outliers > s->num_points) return ADOP_ERR_INVALID_ARGUMENT;
        if (reinterpret_cast<uintptr_t>(s->outlier_position) & 15) return ADOP_ERR_INVALID_ARGUMENT;
        if (!s->outlier_index && s->num_texels < s->num_outliers) return ADOP_ERR_INVALID_ARGUMENT;
    }
    if (rp->composite_environment_map && s->env_map && (s->env_h <= 0 || s->env_w <= 0)) return ADOP_ERR_INVALID_ARGUMENT;
    const int w = views[0].w, h = views[0].h;
    if (w <= 0 || h <= 0) return ADOP_ERR_INVALID_ARGUMENT;
    if (w > 32767 || h > 32767) return ADOP_ERR_SIZE_LIMIT;  // the tile tables and region offsets of the backward pass are 16-bit pixel coordinates
    if ((w >> (L - 1)) <= 0 || (h >> (L - 1)) <= 0) return ADOP_ERR_INVALID_ARGUMENT;
    // pixel indices are 32-bit: a view's pyramid, and the layer-0 planes of a group of four views, must stay below 2^32
    unsigned long long total = 0;
    for (int l = 0, ww = w, hh = h; l < L; ++l, ww /= 2, hh /= 2) total += (unsigned long long)ww * hh;
    if (total >= (1ull << 30)) return ADOP_ERR_SIZE_LIMIT;
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

extern "C" adop_status adop_profile_enable(int32_t on)
{
    adop::profile_state().on = on != 0;
    return ADOP_OK;
}

extern "C" int32_t adop_profile_collect(adop_kernel_time* out, int32_t max_entries)
{
    auto& ps = adop::profile_state();
    std::map<std::string, std::pair<int, float>> acc;
    std::vector<std::string> order;
    bool failed = false;
    for (auto& m : ps.marks)
    {
        float ms = 0.f;
        if (m.begin && m.end && cudaEventSynchronize(m.end) == cudaSuccess && cudaEventElapsedTime(&ms, m.begin, m.end) == cudaSuccess)
        {
            auto it = acc.find(m.name);
            if (it == acc.end()) { acc[m.name] = {1, ms}; order.push_back(m.name); }
            else { it->second.first += 1; it->second.second += ms; }
        }
        else
            failed = true;
        if (m.begin) ps.pool.push_back(m.begin);
        if (m.end) ps.pool.push_back(m.end);
    }
    ps.marks.clear();
    if (failed) return -1;
    int n = 0;
    for (auto& name : order)
    {
        if (out && n < max_entries)
        {
            memset(&out[n], 0, sizeof(out[n]));
            strncpy(out[n].name, name.c_str(), sizeof(out[n].name) - 1);
            out[n].launches = acc[name].first;
            out[n].total_ms = acc[name].second;
        }
        ++n;
    }
    return n;
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
