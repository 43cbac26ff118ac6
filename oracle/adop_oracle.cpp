// adop_oracle.cpp — TEST INFRASTRUCTURE, not part of the product.
//
// A scalar CPU restatement of the semantics of the reference's CUDA rasterizer (darglein/ADOP,
// src/lib/rendering/PointRenderer.cu and PointRendererHelper.h, EnvironmentMap.cu, NeuralCamera.cpp). It is
// the checker the GPU kernels are compared with and the program timed as the CPU baseline. Nothing in the
// shipped library calls it.
//
// PARITY UNPINNED: the reference has no tests or golden vectors and its own CUDA code cannot be compiled
// without the saiga library, which is not part of the reference tree. The camera arithmetic therefore
// comes from include/adop/adop_math.h (restated from the call-site contracts), and is pinned only by
// independent checks (finite differences, float64 re-derivations, torch CPU grid_sample) in tests/.
//
// Same structs as the C ABI (include/adop/adop_raster.h), but every pointer is a HOST pointer.
// `threads` > 1 runs the point loops with OpenMP and atomic min/add (the CPU baseline's parallel form);
// threads == 1 is the deterministic scalar checker.
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <vector>

#include "adop/adop_math.h"
#include "adop/adop_raster.h"

#ifdef _OPENMP
#include <omp.h>
#endif

using namespace adop;

namespace {

struct LayerDims { int w, h; };

void layer_dims(int w, int h, int L, LayerDims* d)
{
    for (int l = 0; l < L; ++l) { d[l].w = w; d[l].h = h; w /= 2; h /= 2; }  // PointRenderer.cu:1015-1016
}

inline void atomic_min_float_as_int(float* addr, float z)
{
    int zi = float_as_int_bits(z);
    int* ai = reinterpret_cast<int*>(addr);
    int old = __atomic_load_n(ai, __ATOMIC_RELAXED);
    while (zi < old && !__atomic_compare_exchange_n(ai, &old, zi, true, __ATOMIC_RELAXED, __ATOMIC_RELAXED)) {}
}
inline void atomic_add_float(float* addr, float v)
{
    uint32_t* ai = reinterpret_cast<uint32_t*>(addr);
    uint32_t old = __atomic_load_n(ai, __ATOMIC_RELAXED);
    for (;;)
    {
        float f; memcpy(&f, &old, 4);
        f += v;
        uint32_t nw; memcpy(&nw, &f, 4);
        if (__atomic_compare_exchange_n(ai, &old, nw, true, __ATOMIC_RELAXED, __ATOMIC_RELAXED)) break;
    }
}
inline void atomic_add_double(double* addr, double v)
{
    uint64_t* ai = reinterpret_cast<uint64_t*>(addr);
    uint64_t old = __atomic_load_n(ai, __ATOMIC_RELAXED);
    for (;;)
    {
        double f; memcpy(&f, &old, 8);
        f += v;
        uint64_t nw; memcpy(&nw, &f, 8);
        if (__atomic_compare_exchange_n(ai, &old, nw, true, __ATOMIC_RELAXED, __ATOMIC_RELAXED)) break;
    }
}

struct PointFetch { V3 p; V3 n; float r; bool has_normal; };

// DevicePointCloud::GetPoint, NeuralPointCloudCuda.h:82-103
inline PointFetch fetch_point(const adop_scene* s, int i)
{
    PointFetch f;
    const float* q = s->position + (size_t)i * 4;
    f.p.x = q[0]; f.p.y = q[1]; f.p.z = q[2]; f.r = q[3];
    f.has_normal = s->normal != nullptr;
    if (f.has_normal) f.n = unpack_normal_10bit(s->normal[i]);
    else { f.n.x = f.n.y = f.n.z = 0.f; }
    return f;
}
inline int fetch_index(const adop_scene* s, int i) { return s->index ? s->index[i] : i; }

// The main cloud, or the optional second one (the outlier cloud of PointRenderer.cu:1402-1441), as a scene of its own
// that shares every other tensor: the forward loops below run over both.
inline adop_scene cloud_of(const adop_scene* s, int which)
{
    adop_scene c = *s;
    if (which == 1)
    {
        c.position = s->outlier_position;
        c.normal = s->outlier_normal;
        c.index = s->outlier_index;
        c.num_points = s->outlier_position ? s->num_outliers : 0;
    }
    return c;
}

inline bool is_dropped(const adop_render_params* rp, const uint8_t* mask, int N, int b, int i)
{
    if (mask) return mask[(size_t)b * N + i] == 1;
    return dropout_decision(rp->dropout, rp->dropout_seed, (uint32_t)b, (uint32_t)i);
}

ViewCam view_cam(const adop_scene* s, const adop_view* v)
{
    return load_view_cam(s->poses, s->intrinsics, s->intrinsics_cols, v->image_index, v->camera_index,
                         v->camera_model, v->crop, v->w);
}

bool check_common(const adop_scene* s, const adop_view* views, int B, int L)
{
    if (!s || !views || B <= 0 || L <= 0 || L > ADOP_MAX_LAYERS) return false;
    if (s->channels <= 0 || s->channels > ADOP_MAX_CHANNELS) return false;
    for (int b = 0; b < B; ++b)
    {
        if (views[b].w != views[0].w || views[b].h != views[0].h) return false;
        if (views[b].image_index < 0 || views[b].image_index >= s->num_images) return false;
        if (views[b].camera_index < 0 || views[b].camera_index >= s->num_cameras) return false;
    }
    return true;
}

}  // namespace

extern "C" {

// ---- forward: PointRenderer.cu:1389-1531 --------------------------------------------------------------
int adop_oracle_forward(const adop_scene* s, const adop_view* views, int B, const adop_render_params* rp, int L,
                        adop_forward_io* io, int threads)
{
    if (!check_common(s, views, B, L) || !rp || !io) return ADOP_ERR_INVALID_ARGUMENT;
    const int N = s->num_points, C = s->channels, T = s->num_texels;
    LayerDims dims[ADOP_MAX_LAYERS];
    layer_dims(views[0].w, views[0].h, L, dims);
#ifdef _OPENMP
    if (threads > 0) omp_set_num_threads(threads);
#else
    (void)threads;
#endif
    const bool par = threads != 1;

    // InitializeData, PointRenderer.cu:1039-1059
    for (int l = 0; l < L; ++l)
    {
        size_t px = (size_t)dims[l].w * dims[l].h;
        for (size_t k = 0; k < (size_t)B * px; ++k) { io->layers[l].depth[k] = kDepthInit; io->layers[l].weight[k] = 0.f; }
        memset(io->layers[l].color, 0, sizeof(float) * (size_t)B * C * px);
    }
    // the packed depth|index word of PointRendererHelper.h:21-34 (dead in the reference's live path), single-threaded
    if (io->packed_depth[0])
    {
        uint32_t init_bits;
        memcpy(&init_bits, &kDepthInit, 4);
        for (int l = 0; l < L; ++l)
        {
            if (!io->packed_depth[l]) return ADOP_ERR_INVALID_ARGUMENT;
            size_t px = (size_t)dims[l].w * dims[l].h;
            for (size_t k = 0; k < (size_t)B * px; ++k) io->packed_depth[l][k] = ((uint64_t)init_bits << 32) | 0xFFFFFFFFull;
        }
        for (int b = 0; b < B; ++b)
        {
            ViewCam cam = view_cam(s, &views[b]);
            for (int i = 0; i < N; ++i)
            {
                PointFetch f = fetch_point(s, i);
                RasterPoint q;
                if (!project_for_raster(cam, f.p, f.r, f.n, f.has_normal, rp->check_normal != 0, rp->dist_cutoff, &q)) continue;
                float x = q.x, y = q.y, rad = q.radius_px;
                uint32_t zb;
                memcpy(&zb, &q.z, 4);
                const uint64_t word = ((uint64_t)zb << 32) | (uint32_t)i;
                for (int l = 0; l < L; ++l, rad *= 0.5f, x *= 0.5f, y *= 0.5f)
                {
                    if (rp->drop_out_points_by_radius && rad < rp->drop_out_radius_threshold) break;
                    int px = round_half_even(x), py = round_half_even(y);
                    if (px < 0 || py < 0 || px >= dims[l].w || py >= dims[l].h) continue;
                    uint64_t* d = io->packed_depth[l] + ((size_t)b * dims[l].h + py) * dims[l].w + px;
                    if (word < *d) *d = word;
                }
            }
        }
    }

    for (int b = 0; b < B; ++b)
    {
        ViewCam cam = view_cam(s, &views[b]);
        // DepthPrepassMulti, PointRenderer.cu:203-301 (drop-out is ignored here: dropped points still occlude);
        // main cloud, then the outlier cloud (:1417-1425)
        for (int which = 0; which < 2; ++which)
        {
        const adop_scene cloud = cloud_of(s, which);
        const adop_scene* s = &cloud;
        const int N = cloud.num_points;
#pragma omp parallel for schedule(static) if (par)
        for (int i = 0; i < N; ++i)
        {
            PointFetch f = fetch_point(s, i);
            RasterPoint q;
            if (!project_for_raster(cam, f.p, f.r, f.n, f.has_normal, rp->check_normal != 0, rp->dist_cutoff, &q)) continue;
            float x = q.x, y = q.y, rad = q.radius_px;
            for (int l = 0; l < L; ++l, rad *= 0.5f, x *= 0.5f, y *= 0.5f)
            {
                if (rp->drop_out_points_by_radius && rad < rp->drop_out_radius_threshold) break;
                int px = round_half_even(x), py = round_half_even(y);
                if (px < 0 || py < 0 || px >= dims[l].w || py >= dims[l].h) continue;
                float* d = io->layers[l].depth + ((size_t)b * dims[l].h + py) * dims[l].w + px;
                if (par) atomic_min_float_as_int(d, q.z);
                else if (q.z < *d) *d = q.z;
            }
        }
        }
        // RenderForwardMulti, PointRenderer.cu:303-393; main cloud, then the outlier cloud (:1433-1441), whose point i
        // takes the drop-out decision of main point i (both index the same [B,N] tensor)
        for (int which = 0; which < 2; ++which)
        {
        const adop_scene cloud = cloud_of(s, which);
        const int N_main = N;
        const adop_scene* s = &cloud;
        const int N = cloud.num_points;
#pragma omp parallel for schedule(static) if (par)
        for (int i = 0; i < N; ++i)
        {
            if (is_dropped(rp, io->dropout_mask, N_main, b, i)) continue;
            PointFetch f = fetch_point(s, i);
            RasterPoint q;
            if (!project_for_raster(cam, f.p, f.r, f.n, f.has_normal, rp->check_normal != 0, rp->dist_cutoff, &q)) continue;
            int ti = fetch_index(s, i);
            float x = q.x, y = q.y, rad = q.radius_px;
            for (int l = 0; l < L; ++l, rad *= 0.5f, x *= 0.5f, y *= 0.5f)
            {
                if (rp->drop_out_points_by_radius && rad < rp->drop_out_radius_threshold) break;
                int px = round_half_even(x), py = round_half_even(y);
                if (px < 0 || py < 0 || px >= dims[l].w || py >= dims[l].h) continue;
                size_t plane = (size_t)dims[l].w * dims[l].h;
                size_t pix = (size_t)py * dims[l].w + px;
                float image_depth = io->layers[l].depth[(size_t)b * plane + pix];
                if (q.z > image_depth * (rp->depth_accept + 1.0f)) continue;
                for (int c = 0; c < C; ++c)
                {
                    float t = s->texture[(size_t)c * T + ti];
                    float* dst = io->layers[l].color + ((size_t)b * C + c) * plane + pix;
                    if (par) atomic_add_float(dst, t); else *dst += t;
                }
                float* wdst = io->layers[l].weight + (size_t)b * plane + pix;
                if (par) atomic_add_float(wdst, 1.f); else *wdst += 1.f;
            }
        }
        }
        // CombineAndFill + CreateMask (+ environment-map composite), PointRenderer.cu:726-754, 828-847,
        // EnvironmentMap.cu:62-156, RenderModule.cpp:106-127
        for (int l = 0; l < L; ++l)
        {
            const int w = dims[l].w, h = dims[l].h;
            const size_t plane = (size_t)w * h;
            Intr5 crop_l = scale_intr(cam.crop, ldexpf(1.0f, -l));
            const bool env = rp->composite_environment_map && s->env_map;
#pragma omp parallel for schedule(static) if (par)
            for (int y = 0; y < h; ++y)
                for (int x = 0; x < w; ++x)
                {
                    size_t pix = (size_t)y * w + x;
                    float cou = io->layers[l].weight[(size_t)b * plane + pix];
                    float m = cou == 0.f ? rp->output_background_mask_value : 1.f;
                    if (io->layers[l].mask) io->layers[l].mask[(size_t)b * plane + pix] = m;
                    BilinearTap tp{};
                    if (env && cou == 0.f)
                    {
                        V2 uv = env_uv_for_pixel(x, y, cam.V, cam.K, cam.dist, crop_l);
                        tp = bilinear_taps(uv, s->env_w, s->env_h);
                    }
                    for (int c = 0; c < C; ++c)
                    {
                        float* o = io->layers[l].color + ((size_t)b * C + c) * plane + pix;
                        if (cou == 0.f)
                        {
                            float v = s->background[c];
                            if (env)
                            {
                                const float* e = s->env_map + (size_t)c * s->env_h * s->env_w;
                                float e00 = e[(size_t)tp.y0 * s->env_w + tp.x0], e01 = e[(size_t)tp.y0 * s->env_w + tp.x1];
                                float e10 = e[(size_t)tp.y1 * s->env_w + tp.x0], e11 = e[(size_t)tp.y1 * s->env_w + tp.x1];
                                float top = e00 + (e01 - e00) * tp.wx;
                                float bot = e10 + (e11 - e10) * tp.wx;
                                float ev = top + (bot - top) * tp.wy;
                                v = v + (1.0f - m) * ev;
                            }
                            *o = v;
                        }
                        else
                        {
                            *o = *o / cou;
                        }
                    }
                }
        }
    }
    return ADOP_OK;
}

// ---- backward: PointRenderer.cu:1549-1644 -------------------------------------------------------------
int adop_oracle_backward(const adop_scene* s, const adop_view* views, int B, const adop_render_params* rp, int L,
                         adop_backward_io* io, int threads)
{
    if (!check_common(s, views, B, L) || !rp || !io) return ADOP_ERR_INVALID_ARGUMENT;
    const int N = s->num_points, C = s->channels, T = s->num_texels;
    LayerDims dims[ADOP_MAX_LAYERS];
    layer_dims(views[0].w, views[0].h, L, dims);
#ifdef _OPENMP
    if (threads > 0) omp_set_num_threads(threads);
#else
    (void)threads;
#endif
    const bool par = threads != 1;
    std::vector<double> intr_sum(io->grad_intrinsics ? (size_t)s->num_cameras * s->intrinsics_cols : 0, 0.0);
    const int cols = s->intrinsics_cols;

    if (!io->accumulate)
    {
        if (io->grad_texture) memset(io->grad_texture, 0, sizeof(float) * (size_t)C * T);
        if (io->grad_background) memset(io->grad_background, 0, sizeof(float) * C);
        if (io->grad_points) memset(io->grad_points, 0, sizeof(float) * (size_t)N * 4);
        if (io->grad_pose) memset(io->grad_pose, 0, sizeof(double) * (size_t)s->num_images * 6);
        if (io->count_pose) memset(io->count_pose, 0, sizeof(float) * s->num_images);
        if (io->grad_intrinsics) memset(io->grad_intrinsics, 0, sizeof(float) * (size_t)s->num_cameras * cols);
        if (io->count_intrinsics) memset(io->count_intrinsics, 0, sizeof(float) * s->num_cameras);
        if (io->grad_env_map) memset(io->grad_env_map, 0, sizeof(float) * (size_t)C * s->env_h * s->env_w);
    }
    if ((io->grad_pose && !io->count_pose) || (io->grad_intrinsics && !io->count_intrinsics))
        return ADOP_ERR_INVALID_ARGUMENT;

    for (int b = 0; b < B; ++b)
    {
        ViewCam cam = view_cam(s, &views[b]);
        const adop_view& vw = views[b];

        // CombineAndFillBackward, PointRenderer.cu:851-900 (+ the gradient of the environment-map composite)
        for (int l = 0; l < L; ++l)
        {
            const int w = dims[l].w, h = dims[l].h;
            const size_t plane = (size_t)w * h;
            Intr5 crop_l = scale_intr(cam.crop, ldexpf(1.0f, -l));
            const bool env = rp->composite_environment_map && s->env_map && io->grad_env_map;
            std::vector<double> bg_rows((size_t)h * C, 0.0);  // per-row partial sums keep the scalar order fixed
#pragma omp parallel for schedule(static) if (par)
            for (int y = 0; y < h; ++y)
                for (int x = 0; x < w; ++x)
                {
                    size_t pix = (size_t)y * w + x;
                    if (io->layers[l].weight[(size_t)b * plane + pix] != 0.f) continue;
                    BilinearTap tp{};
                    if (env)
                    {
                        V2 uv = env_uv_for_pixel(x, y, cam.V, cam.K, cam.dist, crop_l);
                        tp = bilinear_taps(uv, s->env_w, s->env_h);
                    }
                    for (int c = 0; c < C; ++c)
                    {
                        float g = io->grad_color[l][((size_t)b * C + c) * plane + pix];
                        bg_rows[(size_t)y * C + c] += g;
                        if (env)
                        {
                            float ge = (1.0f - rp->output_background_mask_value) * g;
                            float* e = io->grad_env_map + (size_t)c * s->env_h * s->env_w;
                            float v00 = ge * (1.0f - tp.wx) * (1.0f - tp.wy), v01 = ge * tp.wx * (1.0f - tp.wy);
                            float v10 = ge * (1.0f - tp.wx) * tp.wy, v11 = ge * tp.wx * tp.wy;
                            if (par)
                            {
                                atomic_add_float(e + (size_t)tp.y0 * s->env_w + tp.x0, v00);
                                atomic_add_float(e + (size_t)tp.y0 * s->env_w + tp.x1, v01);
                                atomic_add_float(e + (size_t)tp.y1 * s->env_w + tp.x0, v10);
                                atomic_add_float(e + (size_t)tp.y1 * s->env_w + tp.x1, v11);
                            }
                            else
                            {
                                e[(size_t)tp.y0 * s->env_w + tp.x0] += v00;
                                e[(size_t)tp.y0 * s->env_w + tp.x1] += v01;
                                e[(size_t)tp.y1 * s->env_w + tp.x0] += v10;
                                e[(size_t)tp.y1 * s->env_w + tp.x1] += v11;
                            }
                        }
                    }
                }
            if (io->grad_background)
                for (int c = 0; c < C; ++c)
                {
                    double acc = 0.0;
                    for (int y = 0; y < h; ++y) acc += bg_rows[(size_t)y * C + c];
                    io->grad_background[c] += (float)acc;
                }
        }

        // RenderBackward, PointRenderer.cu:396-724
#pragma omp parallel for schedule(static) if (par)
        for (int i = 0; i < N; ++i)
        {
            bool drop_out = is_dropped(rp, io->dropout_mask, N, b, i);
            PointFetch f = fetch_point(s, i);
            RasterPoint q;
            if (!project_for_raster(cam, f.p, f.r, f.n, f.has_normal, rp->check_normal != 0, rp->dist_cutoff, &q)) continue;
            int ti = fetch_index(s, i);
            float x = q.x, y = q.y, rad = q.radius_px, scale = 1.f;
            for (int l = 0; l < L; ++l, scale *= 0.5f, rad *= 0.5f, x *= 0.5f, y *= 0.5f)
            {
                if (rp->drop_out_points_by_radius && rad < rp->drop_out_radius_threshold) continue;  // :451-454
                int px = round_half_even(x), py = round_half_even(y);
                const int w = dims[l].w, h = dims[l].h;
                if (px < 0 || py < 0 || px >= w || py >= h) continue;
                const size_t plane = (size_t)w * h;
                const float* D = io->layers[l].depth + (size_t)b * plane;
                const float* W = io->layers[l].weight + (size_t)b * plane;
                const float* I = io->layers[l].color + (size_t)b * C * plane;
                const float* G = io->grad_color[l] + (size_t)b * C * plane;
                size_t pix = (size_t)py * w + px;
                if (q.z > D[pix] * (rp->depth_accept + 1.0f)) break;  // :462
                float wgt = W[pix];
                if (!drop_out)
                {
                    if (wgt == 0.f) continue;  // :473
                    float iw = 1.f / wgt;
                    if (io->grad_texture)
                        for (int c = 0; c < C; ++c)
                        {
                            float g = iw * G[(size_t)c * plane + pix];
                            float* dst = io->grad_texture + (size_t)c * T + ti;
                            if (par) atomic_add_float(dst, g); else *dst += g;
                        }
                }
                bool point_grad = (rp->ghost_gradients && drop_out) || (!rp->ghost_gradients && !drop_out);  // :487-488
                int edge = px < py ? px : py;  // distanceFromEdge(y,x) > 2, :489
                if (w - 1 - px < edge) edge = w - 1 - px;
                if (h - 1 - py < edge) edge = h - 1 - py;
                if (!(point_grad && edge > 2)) continue;
                if (!io->grad_points && !io->grad_pose && !io->grad_intrinsics) continue;

                const int nx[4] = {px - 1, px + 1, px, px};
                const int ny[4] = {py, py, py - 1, py + 1};
                float dR[4] = {0.f, 0.f, 0.f, 0.f};
                float dRx = 0.f, dRy = 0.f;
                for (int c = 0; c < C; ++c)
                {
                    float T_p = s->texture[(size_t)c * T + ti];
                    for (int k = 0; k < 4; ++k)
                    {
                        size_t np = (size_t)ny[k] * w + nx[k];
                        float W_x = W[np];
                        // the saved forward image is the normalised, background-filled, pre-composite one
                        float I_x = W_x > 0.f ? I[(size_t)c * plane + np] : s->background[c];
                        float G_x = G[(size_t)c * plane + np];
                        float dI;
                        if (rp->test_backward_mode == 4)  // :543-566
                        {
                            float D_x = D[np];
                            if (W_x == 0.f || q.z * (rp->depth_accept + 1.0f) < D_x) dI = T_p - I_x;
                            else if (q.z > D_x * (rp->depth_accept + 1.0f)) dI = 0.f;
                            else dI = (W_x / (W_x + 1.f) * I_x + 1.f / (W_x + 1.f) * T_p - I_x);
                        }
                        else
                            dI = T_p - I_x;
                        dR[k] = dI * G_x;
                    }
                    dRx += 0.5f * (-dR[0] + dR[1]);  // :601-608
                    dRy += 0.5f * (-dR[2] + dR[3]);
                }
                V2 g; g.x = dRx / (float)C; g.y = dRy / (float)C;  // :611
                Intr5 crop_l = scale_intr(cam.crop, scale);        // :616

                float g_point[3], g_pose[6];
                if (vw.camera_model == ADOP_CAMERA_PINHOLE_DISTORTION)
                {
                    GradPinhole o;
                    if (!project_pinhole_backward(f.p, f.n, f.has_normal, g, cam.V, cam.K, crop_l, cam.dist,
                                                  rp->check_normal != 0, rp->dist_cutoff, &o))
                        continue;
                    memcpy(g_point, o.g_point, sizeof(g_point));
                    memcpy(g_pose, o.g_pose, sizeof(g_pose));
                    if (io->grad_intrinsics)  // :645-682
                    {
                        double* gi = intr_sum.data() + (size_t)vw.camera_index * cols;
                        float kf = rp->K_gradient_factor;
                        o.g_k[4] = 0.f;
                        float df = rp->distortion_gradient_factor;
                        o.g_dis[2] *= 0.25f;
                        o.g_dis[3] *= 0.1f; o.g_dis[4] *= 0.1f; o.g_dis[5] *= 0.1f;
                        o.g_dis[6] *= 0.1f; o.g_dis[7] *= 0.1f;
                        for (int k = 0; k < 5; ++k) { if (par) atomic_add_double(gi + k, (double)(kf * o.g_k[k])); else gi[k] += (double)(kf * o.g_k[k]); }
                        for (int k = 0; k < 8; ++k) { if (par) atomic_add_double(gi + 5 + k, (double)(df * o.g_dis[k])); else gi[5 + k] += (double)(df * o.g_dis[k]); }
                        float* ci = io->count_intrinsics + vw.camera_index;
                        if (par) atomic_add_float(ci, 1.f / 1024.f); else *ci += 1.f / 1024.f;
                    }
                }
                else
                {
                    GradOcam o;
                    if (!project_ocam_backward(f.p, f.n, f.has_normal, g, cam.V, crop_l, cam.ocam, rp->check_normal != 0,
                                               rp->dist_cutoff, &o))
                        continue;
                    memcpy(g_point, o.g_point, sizeof(g_point));
                    memcpy(g_pose, o.g_pose, sizeof(g_pose));
                    if (io->grad_intrinsics)  // :711-719
                    {
                        double* gi = intr_sum.data() + (size_t)vw.camera_index * cols;
                        for (int k = 0; k < 5; ++k) { if (par) atomic_add_double(gi + k, (double)o.g_affine[k]); else gi[k] += (double)o.g_affine[k]; }
                        float* ci = io->count_intrinsics + vw.camera_index;
                        if (par) atomic_add_float(ci, 1.f); else *ci += 1.f;
                    }
                }
                if (io->grad_points)  // :626-633
                {
                    float* gp = io->grad_points + (size_t)i * 4;
                    for (int k = 0; k < 3; ++k) { if (par) atomic_add_float(gp + k, g_point[k]); else gp[k] += g_point[k]; }
                    if (par) atomic_add_float(gp + 3, 1.f); else gp[3] += 1.f;
                }
                if (io->grad_pose)  // :635-643
                {
                    double* gp = io->grad_pose + (size_t)vw.image_index * 6;
                    for (int k = 0; k < 6; ++k) { if (par) atomic_add_double(gp + k, (double)g_pose[k]); else gp[k] += (double)g_pose[k]; }
                    float* cp = io->count_pose + vw.image_index;
                    if (par) atomic_add_float(cp, 1.f); else *cp += 1.f;
                }
            }
        }
    }

    // the per-camera sums run over millions of cancelling terms: they are formed in double here (the reference adds float
    // atomics in an order of its own, PointRenderer.cu:645-682), so that this checker is the better-conditioned side
    if (io->grad_intrinsics)
        for (size_t k = 0; k < intr_sum.size(); ++k) io->grad_intrinsics[k] = (float)((double)io->grad_intrinsics[k] + intr_sum[k]);

    if (io->normalize)  // NormalizeGradient, PointRenderer.cu:1534-1547, 1609-1637
    {
        if (io->grad_pose)
            for (int i = 0; i < s->num_images; ++i)
            {
                float c = io->count_pose[i];
                if (c > 0) for (int k = 0; k < 6; ++k) io->grad_pose[(size_t)i * 6 + k] /= (double)c;
            }
        if (io->grad_points)
#pragma omp parallel for schedule(static) if (par)
            for (int i = 0; i < N; ++i)
            {
                float* gp = io->grad_points + (size_t)i * 4;
                float c = gp[3];
                if (c > 0) { gp[0] /= c; gp[1] /= c; gp[2] /= c; }
                gp[3] = 0.f;
            }
        if (io->grad_intrinsics)
            for (int i = 0; i < s->num_cameras; ++i)
            {
                float c = io->count_intrinsics[i];
                if (c > 0) for (int k = 0; k < cols; ++k) io->grad_intrinsics[(size_t)i * cols + k] /= c;
            }
    }
    return ADOP_OK;
}

// ---- ApplyTangent, PointRenderer.cu:1646-1657 ---------------------------------------------------------
int adop_oracle_apply_tangent(double* tangent, double* pose, int n)
{
    for (int i = 0; i < n; ++i)
    {
        se3_exp_left_multiply(tangent + (size_t)i * 6, pose + (size_t)i * 8);
        for (int k = 0; k < 6; ++k) tangent[(size_t)i * 6 + k] = 0.0;
    }
    return ADOP_OK;
}

// ---- tonemapper: NeuralCamera.cpp:258-335 with :22-42 and :87-135 ----------------------------------------
namespace {
struct TonePixel { float y; float scale; float r2; float vig; };
}

int adop_oracle_tonemap_forward(const adop_tonemap_params* p, const float* x, float* out)
{
    const int B = p->batch, H = p->height, W = p->width, K = p->response_bins;
    const size_t plane = (size_t)H * W;
    const float aspect = (float)p->vignette_image_w / (float)p->vignette_image_h;
    for (int b = 0; b < B; ++b)
    {
        int fi = p->frame_index ? p->frame_index[b] : 0;
        float ef = p->exposure ? 1.0f / exp2f(p->exposure[fi]) : 1.0f;
        for (int c = 0; c < 3; ++c)
        {
            float wb = p->white_balance ? p->white_balance[(size_t)fi * 3 + c] : 1.0f;
            for (int yy = 0; yy < H; ++yy)
                for (int xx = 0; xx < W; ++xx)
                {
                    size_t pix = (size_t)yy * W + xx;
                    float v = x[((size_t)b * 3 + c) * plane + pix] * ef;
                    v = wb * v;
                    if (p->vignette)
                    {
                        float u0, v0;
                        if (p->uv) { u0 = p->uv[((size_t)b * 2 + 0) * plane + pix]; v0 = p->uv[((size_t)b * 2 + 1) * plane + pix]; }
                        else { u0 = 2.0f * ((float)xx / (float)(W - 1)) - 1.0f; v0 = 2.0f * ((float)yy / (float)(H - 1)) - 1.0f; }
                        float du = (u0 - p->vignette[3]) * aspect, dv = v0 - p->vignette[4];
                        float r2 = du * du + dv * dv, r4 = r2 * r2, r6 = r4 * r2;
                        float fac = 1.f + p->vignette[0] * r2 + p->vignette[1] * r4 + p->vignette[2] * r6;
                        v = fac * v;
                    }
                    float o;
                    if (p->response)
                    {
                        float leak_add = 0.f;
                        if (p->leak > 0.f)
                        {
                            if (v < 0.f) leak_add = v * p->leak;
                            if (v > 1.f) leak_add = -p->leak / sqrtf(fabsf(v) + 1e-4f) + p->leak;
                        }
                        float t = fminf(fmaxf(v, 0.f), 1.f) * (float)(K - 1);
                        int i0 = (int)floorf(t);
                        int i1 = i0 + 1 < K ? i0 + 1 : K - 1;
                        float fr = t - (float)i0;
                        const float* lut = p->response + (size_t)c * K;
                        o = lut[i0] * (1.0f - fr) + lut[i1] * fr + leak_add;
                    }
                    else
                        o = fminf(fmaxf(v, 0.f), 1.f);
                    out[((size_t)b * 3 + c) * plane + pix] = o;
                }
        }
    }
    return ADOP_OK;
}

// gradients of the above, accumulated in double and written as float
int adop_oracle_tonemap_backward(const adop_tonemap_params* p, const float* x, const float* grad_out,
                                 adop_tonemap_grads* g)
{
    const int B = p->batch, H = p->height, W = p->width, K = p->response_bins;
    const size_t plane = (size_t)H * W;
    const float aspect = (float)p->vignette_image_w / (float)p->vignette_image_h;
    const int nf = g->num_frames;
    std::vector<double> gE(nf, 0.0), gWB((size_t)nf * 3, 0.0), gV(5, 0.0), gR((size_t)3 * (K > 0 ? K : 1), 0.0);
    const float ln2 = 0.69314718056f;
    for (int b = 0; b < B; ++b)
    {
        int fi = p->frame_index ? p->frame_index[b] : 0;
        float ef = p->exposure ? 1.0f / exp2f(p->exposure[fi]) : 1.0f;
        for (int c = 0; c < 3; ++c)
        {
            float wb = p->white_balance ? p->white_balance[(size_t)fi * 3 + c] : 1.0f;
            for (int yy = 0; yy < H; ++yy)
                for (int xx = 0; xx < W; ++xx)
                {
                    size_t pix = (size_t)yy * W + xx;
                    float xin = x[((size_t)b * 3 + c) * plane + pix];
                    float go = grad_out[((size_t)b * 3 + c) * plane + pix];
                    float fac = 1.f, du = 0.f, dv = 0.f, r2 = 0.f, r4 = 0.f, r6 = 0.f;
                    if (p->vignette)
                    {
                        float u0, v0;
                        if (p->uv) { u0 = p->uv[((size_t)b * 2 + 0) * plane + pix]; v0 = p->uv[((size_t)b * 2 + 1) * plane + pix]; }
                        else { u0 = 2.0f * ((float)xx / (float)(W - 1)) - 1.0f; v0 = 2.0f * ((float)yy / (float)(H - 1)) - 1.0f; }
                        du = (u0 - p->vignette[3]) * aspect; dv = v0 - p->vignette[4];
                        r2 = du * du + dv * dv; r4 = r2 * r2; r6 = r4 * r2;
                        fac = 1.f + p->vignette[0] * r2 + p->vignette[1] * r4 + p->vignette[2] * r6;
                    }
                    float pre = wb * (xin * ef);  // value before the vignette
                    float v = fac * pre;
                    // d out / d v
                    float dv_out;
                    if (p->response)
                    {
                        const float* lut = p->response + (size_t)c * K;
                        float dleak = 0.f;
                        if (p->leak > 0.f)
                        {
                            if (v < 0.f) dleak = p->leak;
                            if (v > 1.f) { float a = fabsf(v) + 1e-4f; dleak = 0.5f * p->leak / (a * sqrtf(a)); }
                        }
                        float vc = fminf(fmaxf(v, 0.f), 1.f);
                        float t = vc * (float)(K - 1);
                        int i0 = (int)floorf(t);
                        int i1 = i0 + 1 < K ? i0 + 1 : K - 1;
                        float fr = t - (float)i0;
                        gR[(size_t)c * K + i0] += (double)go * (1.0f - fr);
                        gR[(size_t)c * K + i1] += (double)go * fr;
                        float inside = (v > 0.f && v < 1.f) ? 1.f : 0.f;  // gradient of the clamp
                        dv_out = inside * (lut[i1] - lut[i0]) * (float)(K - 1) + dleak;
                    }
                    else
                        dv_out = (v > 0.f && v < 1.f) ? 1.f : 0.f;
                    float gv = go * dv_out;
                    if (p->vignette)
                    {
                        float gfac = gv * pre;
                        gV[0] += (double)gfac * r2; gV[1] += (double)gfac * r4; gV[2] += (double)gfac * r6;
                        float gr2 = gfac * (p->vignette[0] + 2.f * p->vignette[1] * r2 + 3.f * p->vignette[2] * r4);
                        gV[3] += (double)(gr2 * 2.f * du * (-aspect));
                        gV[4] += (double)(gr2 * 2.f * dv * (-1.f));
                    }
                    float gpre = gv * fac;
                    if (p->white_balance) gWB[(size_t)fi * 3 + c] += (double)gpre * (xin * ef);
                    float gxe = gpre * wb;  // gradient w.r.t. x*ef
                    if (p->exposure) gE[fi] += (double)gxe * xin * ef * (-ln2);
                    if (g->grad_x) g->grad_x[((size_t)b * 3 + c) * plane + pix] = gxe * ef;
                }
        }
    }
    auto put = [&](float* dst, const std::vector<double>& src, size_t n)
    {
        if (!dst) return;
        for (size_t i = 0; i < n; ++i) dst[i] = (g->accumulate ? dst[i] : 0.f) + (float)src[i];
    };
    put(g->grad_exposure, gE, (size_t)nf);
    put(g->grad_white_balance, gWB, (size_t)nf * 3);
    put(g->grad_vignette, gV, 5);
    put(g->grad_response, gR, (size_t)3 * K);
    return ADOP_OK;
}

// ---- probes for the unit tests of the shared arithmetic -----------------------------------------------
float adop_oracle_atan(float t) { return atan_f(t); }
float adop_oracle_atan2(float y, float x) { return atan2_f(y, x); }
float adop_oracle_acos(float c) { return acos_f(c); }
int adop_oracle_round(float x) { return round_half_even(x); }
uint32_t adop_oracle_hash(uint32_t seed, uint32_t view, uint32_t point) { return hash_u32(seed, view, point); }
int adop_oracle_dropout(float p, uint32_t seed, uint32_t view, uint32_t point) { return dropout_decision(p, seed, view, point) ? 1 : 0; }
int32_t adop_oracle_pack_normal(float x, float y, float z) { return pack_normal_10bit(x, y, z); }
void adop_oracle_unpack_normal(int32_t e, float* out3) { V3 n = unpack_normal_10bit(e); out3[0] = n.x; out3[1] = n.y; out3[2] = n.z; }

// project n points into one view: out [n,4] = x, y (cropped layer-0 image position), z, radius_px; z = 0 if rejected
void adop_oracle_project(const adop_scene* s, const adop_view* v, const adop_render_params* rp, float* out)
{
    ViewCam cam = view_cam(s, v);
    for (int i = 0; i < s->num_points; ++i)
    {
        PointFetch f = fetch_point(s, i);
        RasterPoint q;
        bool ok = project_for_raster(cam, f.p, f.r, f.n, f.has_normal, rp->check_normal != 0, rp->dist_cutoff, &q);
        out[(size_t)i * 4 + 0] = ok ? q.x : 0.f; out[(size_t)i * 4 + 1] = ok ? q.y : 0.f;
        out[(size_t)i * 4 + 2] = ok ? q.z : 0.f; out[(size_t)i * 4 + 3] = ok ? q.radius_px : 0.f;
    }
}

// the five-vector form of the projection (project_for_raster_hot) on every point: out[i] = x, y, z, accepted (1 / 0);
// returns 0 when the view's camera does not allow that form
int adop_oracle_project_hot(const adop_scene* s, const adop_view* v, const adop_render_params* rp, float* out)
{
    ViewCam cam = view_cam(s, v);
    if (cam.hot[19] == 0.f) return 0;
    V4 h[5];
    for (int k = 0; k < 5; ++k) { h[k].x = cam.hot[4 * k]; h[k].y = cam.hot[4 * k + 1]; h[k].z = cam.hot[4 * k + 2]; h[k].w = cam.hot[4 * k + 3]; }
    for (int i = 0; i < s->num_points; ++i)
    {
        PointFetch f = fetch_point(s, i);
        RasterPoint q;
        bool ok = project_for_raster_hot(h[0], h[1], h[2], h[3], h[4], f.p, rp->dist_cutoff, &q);
        out[(size_t)i * 4 + 0] = ok ? q.x : 0.f; out[(size_t)i * 4 + 1] = ok ? q.y : 0.f;
        out[(size_t)i * 4 + 2] = ok ? q.z : 0.f; out[(size_t)i * 4 + 3] = ok ? 1.f : 0.f;
    }
    return 1;
}

// gradient chain of one point for an image-space gradient g (layer 0): out = g_point[3], g_pose[6], then
// g_k[5] + g_dis[8] (pinhole) or g_affine[5] (OCam); returns 0 if the chain rejects the point
int adop_oracle_project_backward(const adop_scene* s, const adop_view* v, const adop_render_params* rp, int point,
                                 float gx, float gy, float* out)
{
    ViewCam cam = view_cam(s, v);
    PointFetch f = fetch_point(s, point);
    V2 g; g.x = gx; g.y = gy;
    if (v->camera_model == ADOP_CAMERA_PINHOLE_DISTORTION)
    {
        GradPinhole o;
        if (!project_pinhole_backward(f.p, f.n, f.has_normal, g, cam.V, cam.K, cam.crop, cam.dist, rp->check_normal != 0,
                                      rp->dist_cutoff, &o))
            return 0;
        memcpy(out, o.g_point, 12); memcpy(out + 3, o.g_pose, 24); memcpy(out + 9, o.g_k, 20); memcpy(out + 14, o.g_dis, 32);
    }
    else
    {
        GradOcam o;
        if (!project_ocam_backward(f.p, f.n, f.has_normal, g, cam.V, cam.crop, cam.ocam, rp->check_normal != 0,
                                   rp->dist_cutoff, &o))
            return 0;
        memcpy(out, o.g_point, 12); memcpy(out + 3, o.g_pose, 24); memcpy(out + 9, o.g_affine, 20);
    }
    return 1;
}

// environment-map sampling position of every pixel of layer l of one view: out [h_l, w_l, 2] in [-1,1]
void adop_oracle_env_uv(const adop_scene* s, const adop_view* v, int layer, float* out)
{
    ViewCam cam = view_cam(s, v);
    int w = v->w, h = v->h;
    for (int l = 0; l < layer; ++l) { w /= 2; h /= 2; }
    Intr5 crop_l = scale_intr(cam.crop, ldexpf(1.0f, -layer));
    for (int y = 0; y < h; ++y)
        for (int x = 0; x < w; ++x)
        {
            V2 uv = env_uv_for_pixel(x, y, cam.V, cam.K, cam.dist, crop_l);
            out[((size_t)y * w + x) * 2 + 0] = uv.x; out[((size_t)y * w + x) * 2 + 1] = uv.y;
        }
}

int adop_oracle_max_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

}  // extern "C"
