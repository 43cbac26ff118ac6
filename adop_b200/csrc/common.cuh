// Shared device/host helpers of the rasterizer kernels (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "adop/adop_math.h"
#include "adop/adop_raster.h"

namespace adop {

constexpr int kBlock = 256;  // threads per block of the point kernels (one point per thread and iteration)

// thread-local text of the last CUDA error, returned by adop_last_error()
char* last_error_buffer();
adop_status record_cuda_error(cudaError_t e, const char* what);

#define ADOP_CUDA_TRY(expr)                                                     \
    do {                                                                        \
        cudaError_t _e = (expr);                                                \
        if (_e != cudaSuccess) return ::adop::record_cuda_error(_e, #expr);     \
    } while (0)

// Optional per-kernel timing (adop_profile_enable): records an event before and after the launch expression.
bool profile_on();
void profile_mark(const char* name, cudaStream_t st, bool begin);
#define ADOP_LAUNCH(name, st, launch_expr)                          \
    do {                                                            \
        if (::adop::profile_on()) ::adop::profile_mark(name, st, true);  \
        launch_expr;                                                \
        if (::adop::profile_on()) ::adop::profile_mark(name, st, false); \
    } while (0)

// Everything a kernel needs to know about the pyramid of ONE view: sizes and the view's slice of every
// per-layer tensor (pointers already advanced to batch entry b).
struct LayerTable
{
    int L;
    int w[kMaxLayers], h[kMaxLayers];
    unsigned rec_off[kMaxLayers + 1];  // first accumulator record (= pixel) of each layer; [L] = total
    float* depth[kMaxLayers];
    float* weight[kMaxLayers];
    float* color[kMaxLayers];   // [C,h,w] of this view
    float* mask[kMaxLayers];    // may be null
    const float* grad[kMaxLayers];  // upstream gradient [C,h,w] of this view (backward only)
};

struct PointStreams
{
    const float4* position;
    const int32_t* normal;  // may be null
    const int32_t* index;   // may be null (identity)
    int n;
};

// the handful of RenderParams fields the kernels read (Settings.h:16-52)
struct KernelParams
{
    float depth_accept_plus_one;  // formed once in float like PointRenderer.cu:380
    float dropout;
    uint32_t dropout_seed;
    float drop_out_radius_threshold;
    float dist_cutoff;
    float K_gradient_factor, distortion_gradient_factor;
    float mask_background_value;
    int drop_out_points_by_radius;
    int check_normal;
    int ghost_gradients;
    int test_backward_mode;
    int batch_slot;               // b: index of the view inside the batch (drop-out stream id)
    const uint8_t* dropout_mask;  // already advanced to view b, or null
};

inline KernelParams make_kernel_params(const adop_render_params* rp, const uint8_t* dropout_mask, int n_points, int b)
{
    KernelParams k;
    k.depth_accept_plus_one = rp->depth_accept + 1.0f;
    k.dropout = rp->dropout;
    k.dropout_seed = rp->dropout_seed;
    k.drop_out_radius_threshold = rp->drop_out_radius_threshold;
    k.dist_cutoff = rp->dist_cutoff;
    k.K_gradient_factor = rp->K_gradient_factor;
    k.distortion_gradient_factor = rp->distortion_gradient_factor;
    k.mask_background_value = rp->output_background_mask_value;
    k.drop_out_points_by_radius = rp->drop_out_points_by_radius;
    k.check_normal = rp->check_normal;
    k.ghost_gradients = rp->ghost_gradients;
    k.test_backward_mode = rp->test_backward_mode;
    k.batch_slot = b;
    k.dropout_mask = dropout_mask ? dropout_mask + (size_t)b * n_points : nullptr;
    return k;
}

// floats per accumulator record: C colour sums, the weight, padded to whole 16-byte vectors so that one
// splat is one or two vector atomics into a single 32-byte sector (for C <= 7)
__host__ __device__ inline int record_floats(int C) { return ((C + 1) + 3) & ~3; }

inline void fill_layer_dims(int w, int h, int L, LayerTable* lt)
{
    lt->L = L;
    unsigned off = 0;
    for (int l = 0; l < kMaxLayers; ++l)
    {
        if (l < L)
        {
            lt->w[l] = w; lt->h[l] = h;
            lt->rec_off[l] = off;
            off += (unsigned)w * (unsigned)h;
            w /= 2; h /= 2;  // PointRenderer.cu:1015-1016
        }
        else
        {
            lt->w[l] = 0; lt->h[l] = 0; lt->rec_off[l] = off;
        }
        lt->depth[l] = lt->weight[l] = lt->color[l] = lt->mask[l] = nullptr;
        lt->grad[l] = nullptr;
    }
    lt->rec_off[kMaxLayers] = off;
    for (int l = L; l <= kMaxLayers; ++l) lt->rec_off[l] = off;
}

// One view's camera is gathered from rows of the pose / intrinsics tensors (device memory: they are trainable
// parameters) plus the ReducedImageInfo fields of the view. A small kernel does that for a chunk of views and leaves the
// ViewCam records at the head of the workspace; the point kernels read their view's record through a pointer. (Measured
// on the depth prepass: camera as a by-value kernel argument 72 us, through this pointer 82 us, in shared memory 90 us, in
// an indexed __constant__ array 100 us; by-value needs the numbers on the host, which would cost a device-to-host sync.)
constexpr int kCamChunk = 64;                      // views per chunk
constexpr size_t kCamRegionBytes = 32768;          // head of the workspace, >= kCamChunk * sizeof(ViewCam)
struct CamChunkSource
{
    const double* poses;
    const float* intrinsics;
    int intrinsics_cols;
    int n;
    struct View { int image_index, camera_index, camera_model, w0; float crop[5]; } v[kCamChunk];
};
static_assert(sizeof(ViewCam) * kCamChunk <= kCamRegionBytes, "camera region too small");
inline void fill_cam_chunk(CamChunkSource* c, const adop_scene* s, const adop_view* views, int n)
{
    c->poses = s->poses; c->intrinsics = s->intrinsics; c->intrinsics_cols = s->intrinsics_cols; c->n = n;
    for (int k = 0; k < n; ++k)
    {
        c->v[k].image_index = views[k].image_index; c->v[k].camera_index = views[k].camera_index;
        c->v[k].camera_model = views[k].camera_model; c->v[k].w0 = views[k].w;
        for (int i = 0; i < 5; ++i) c->v[k].crop[i] = views[k].crop[i];
    }
}

// Splat list of one view: every (point, layer) pair that the backward pass has to visit - the point passed the fuzzy
// depth test on that layer and on every finer layer it landed in (the backward pass stops at the first failure,
// PointRenderer.cu:462). Written by the blend kernel, consumed by the backward kernel; it takes the role of the
// reference's saved [B,N] drop-out tensor as the per-view state carried from forward to backward (:1524).
// Layout per view, in int32:
//   [0, kVisibleSegments)            number of entries of each segment (one segment per block of the blend launch)
//   [kVisibleSegments + 0 / + 1]     segments in use / entries per segment (`seg_cap`), written by the blend kernel
//   [kVisibleSegments + 2]           overflow flag: a segment ran out of room, the list is incomplete and not used
//   [kVisibleHeaderInts, ...)        segments of `seg_cap` entries each, unordered; an entry is four ints:
//                                    point id | layer << 28, the pixel index inside that layer, and two floats that the
//                                    backward pass fills with the splat's image-space gradient (its first kernel gathers
//                                    pixel data with few registers, its second chains the gradient through the projection)
// A segment holds as many entries as its block has points. A view typically has 0.2-0.3 splats per point, but they come
// in clumps (whole chunks of neighbouring points on a front surface are accepted on every layer), so single blocks see
// several times the average.
constexpr unsigned kSplatPointMask = 0x0FFFFFFFu;
constexpr int kSplatLayerShift = 28;
constexpr int kSplatMaxPoints = 1 << 28;  // larger clouds are rendered without a list
constexpr int kVisibleSegments = 2048;
constexpr int kVisibleHeaderInts = kVisibleSegments + 8;
inline size_t visible_list_ints(int num_points) { return (size_t)kVisibleHeaderInts + 4 * ((size_t)num_points + (size_t)kVisibleSegments * kBlock); }
struct VisibleList
{
    int* header;   // null = no list
    int4* entries;
    int segments;  // blocks of the blend launch
    int seg_cap;   // entries per segment
};
inline VisibleList make_visible_list(int32_t* base, int num_points, int view, int segments)
{
    VisibleList v;
    if (!base) { v.header = nullptr; v.entries = nullptr; v.segments = 0; v.seg_cap = 0; return v; }
    int* p = base + (size_t)view * visible_list_ints(num_points);
    v.header = p;
    v.entries = reinterpret_cast<int4*>(p + kVisibleHeaderInts);  // 16-byte aligned: header and per-view size are multiples of 4 ints
    v.segments = segments;
    long long iters = ((long long)(num_points + kBlock - 1) / kBlock + segments - 1) / segments;
    v.seg_cap = (int)(iters * kBlock);
    return v;
}

adop_status validate_common(const adop_scene* s, const adop_view* views, int B, const adop_render_params* rp, int L);
int sm_count();

#if defined(__CUDACC__)
// Grid of a persistent grid-stride kernel: exactly the blocks that are resident at once (occupancy x SMs),
// so there is no partial second wave, capped by the work available.
template <class Kernel>
inline int resident_grid(Kernel kernel, long long work_items)
{
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kBlock, 0) != cudaSuccess || per_sm < 1) per_sm = 1;
    long long need = (work_items + kBlock - 1) / kBlock;
    long long g = (long long)per_sm * sm_count();
    if (g > need) g = need;
    return g < 1 ? 1 : (int)g;
}

// Projection of the PLAIN kernels (no normal test, no radius rule): the five-vector camera record when the view's
// camera allows it (pinhole, k1 and k2 only), else the general function. Same results either way.
__device__ __forceinline__ bool project_plain(const ViewCam& cam, V3 p, float dist_cutoff, RasterPoint* q)
{
    const float4* hot = reinterpret_cast<const float4*>(cam.hot);
    const float4 h4 = __ldg(hot + 4);
    if (h4.w != 0.f)
    {
        const float4 h0 = __ldg(hot), h1 = __ldg(hot + 1), h2 = __ldg(hot + 2), h3 = __ldg(hot + 3);
        return project_for_raster_hot(V4{h0.x, h0.y, h0.z, h0.w}, V4{h1.x, h1.y, h1.z, h1.w}, V4{h2.x, h2.y, h2.z, h2.w},
                                      V4{h3.x, h3.y, h3.z, h3.w}, V4{h4.x, h4.y, h4.z, h4.w}, p, dist_cutoff, q);
    }
    V3 n;
    n.x = n.y = n.z = 0.f;
    return project_for_raster(cam, p, 0.f, n, false, false, dist_cutoff, q, false);
}

// layer that holds pyramid pixel (= accumulator record) r of a view
__device__ __forceinline__ int layer_of_record(const LayerTable& lt, unsigned r)
{
    int l = 0;
#pragma unroll
    for (int k = 1; k < kMaxLayers; ++k)
        if (k < lt.L && r >= lt.rec_off[k]) l = k;
    return l;
}

struct FetchedPoint { V3 p; V3 n; float r; bool has_normal; };

// DevicePointCloud::GetPoint (NeuralPointCloudCuda.h:82-103): one 128-bit load of xyz + radius
__device__ __forceinline__ FetchedPoint fetch_point(const PointStreams& s, int i, float4 q)
{
    FetchedPoint f;
    f.p.x = q.x; f.p.y = q.y; f.p.z = q.z; f.r = q.w;
    f.has_normal = s.normal != nullptr;
    if (f.has_normal) f.n = unpack_normal_10bit(__ldg(s.normal + i));
    else { f.n.x = 0.f; f.n.y = 0.f; f.n.z = 0.f; }
    return f;
}
__device__ __forceinline__ FetchedPoint fetch_point(const PointStreams& s, int i) { return fetch_point(s, i, __ldg(s.position + i)); }
static __global__ void k_build_cams(CamChunkSource src, ViewCam* __restrict__ out)
{
    const int k = blockIdx.x * blockDim.x + threadIdx.x;
    if (k >= src.n) return;
    out[k] = load_view_cam(src.poses, src.intrinsics, src.intrinsics_cols, src.v[k].image_index, src.v[k].camera_index,
                           src.v[k].camera_model, src.v[k].crop, src.v[k].w0);
}
// A point's descriptor: from the interleaved [T,C] copy when the caller provides one (one or two 16-byte loads), else
// from the C planes of the [C,T] tensor.
template <int C>
__device__ __forceinline__ void load_descriptor(const float* __restrict__ planar, const float* __restrict__ interleaved,
                                                int num_texels, int ti, float* t)
{
    if (interleaved)
    {
        const float* src = interleaved + (size_t)ti * C;
        if (C % 4 == 0)
        {
#pragma unroll
            for (int k = 0; k < C / 4; ++k)
            {
                float4 a = __ldg(reinterpret_cast<const float4*>(src) + k);
                t[4 * k] = a.x; t[4 * k + 1] = a.y; t[4 * k + 2] = a.z; t[4 * k + 3] = a.w;
            }
        }
        else
        {
#pragma unroll
            for (int c = 0; c < C; ++c) t[c] = __ldg(src + c);
        }
    }
    else
    {
#pragma unroll
        for (int c = 0; c < C; ++c) t[c] = __ldg(planar + (size_t)c * num_texels + ti);
    }
}
// Add a descriptor gradient: one vector atomic per 4 channels into the interleaved scratch, else C scalar atomics
// into the planes.
template <int C>
__device__ __forceinline__ void add_descriptor_gradient(float* __restrict__ planar, float* __restrict__ interleaved,
                                                        int num_texels, int ti, const float* g)
{
    if (interleaved)
    {
        float* dst = interleaved + (size_t)ti * C;
        if (C % 4 == 0)
        {
#pragma unroll
            for (int k = 0; k < C / 4; ++k)
                atomicAdd(reinterpret_cast<float4*>(dst) + k, make_float4(g[4 * k], g[4 * k + 1], g[4 * k + 2], g[4 * k + 3]));
        }
        else
        {
#pragma unroll
            for (int c = 0; c < C; ++c) atomicAdd(dst + c, g[c]);
        }
    }
    else
    {
#pragma unroll
        for (int c = 0; c < C; ++c) atomicAdd(planar + (size_t)c * num_texels + ti, g[c]);
    }
}
__device__ __forceinline__ bool point_dropped(const KernelParams& kp, int i)
{
    if (kp.dropout_mask) return kp.dropout_mask[i] == 1;
    return dropout_decision(kp.dropout, kp.dropout_seed, (uint32_t)kp.batch_slot, (uint32_t)i);
}
__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
#endif

}  // namespace adop
