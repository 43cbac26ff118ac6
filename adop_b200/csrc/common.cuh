// Shared device/host helpers of the rasterizer kernels (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

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

// Which chunk of kBlock consecutive points a block works on in its k-th round. The cloud is Morton-sorted, so a plain
// grid-stride loop has all resident blocks inside one small region of space at any time, and their atomics (depth
// minima, accumulator sums, tile counters) pile up on a few image tiles and L2 slices. Here the cloud is cut into G
// superblocks of `rounds` chunks; in round k block b takes chunk k of superblock (b + k * spread) mod G (spread coprime
// to G): at any time the blocks are spread over the whole cloud, and over its rounds a block samples superblocks from
// all over the cloud, so that blocks carry similar loads.
struct ChunkSchedule
{
    int rounds;   // K = ceil(chunks / G)
    int spread;   // S
    int chunks;   // ceil(n / kBlock)
};
inline ChunkSchedule make_chunk_schedule(int n_points, int grid)
{
    ChunkSchedule c;
    c.chunks = (n_points + kBlock - 1) / kBlock;
    if (grid < 1) grid = 1;
    c.rounds = (c.chunks + grid - 1) / grid;
    int s = grid / 29 + 1;
    auto gcd = [](int a, int b) { while (b) { int t = a % b; a = b; b = t; } return a; };
    while (gcd(s, grid) != 1) ++s;
    c.spread = s;
    return c;
}

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

// Visible list of one view: the points that passed the fuzzy depth test on their finest layer, each with the float image
// position the forward pass computed for it and two layer masks, grouped by screen tile. It takes the role of the
// reference's saved [B,N] drop-out tensor as the per-view state carried from forward to backward (PointRenderer.cu:1524).
// An entry is four 32-bit words:
//   point id | dropped << 31        (dropped: the drop-out decision of this view; such points are listed in ghost mode only)
//   forward mask | backward mask << 8
//                                   forward mask: layers on which the point is blended (it landed there and passed the
//                                   depth test; the forward pass goes on after a failure, :380); backward mask: the layers
//                                   the backward pass visits (it stops at the first failure, :462); never 0 in the list
//   x, y                            image position at full resolution as float bits; layer l's pixel is
//                                   rne(x * 0.5^l), rne(y * 0.5^l), the same arithmetic as in the forward pass
// Entries are grouped by screen tile (kTileW x kTileH pixels of layer 0; a point's pixels on the coarser layers lie in the
// corresponding quarter-size regions, give or take a pixel of rounding): every tile owns a bucket of `cap` slots, the
// blend kernel appends to it behind a per-tile cursor (a run of lanes with the same tile takes consecutive slots behind
// one atomic). A bucket holds max(2048, 2 N / tiles) entries: four visible points per pixel of the tile, or twice the
// tile's share of the whole cloud. A view that needs more marks its list unusable and the backward pass walks all points.
// The backward pass overwrites each entry with the work item of its chain kernel, so a list serves one backward call
// with geometry gradients; it is then marked consumed and a further call walks all points.
// Layout of the list per view, in int32:
//   [0, kVisibleHeaderInts)         control words (kListUnusable, kListConsumed, kListGo below), the rest is reserved
//   [.., + T)                       entries in each tile's bucket (fill cursors; may exceed cap when the list overflowed)
//   entries                         T buckets of cap entries, 4 ints each
constexpr int kVisibleSegments = 2048;    // most blocks the depth prepass writes candidate segments with
constexpr int kVisibleHeaderInts = kVisibleSegments + 8;
// granularity of the optional "a gradient was added here" flags of the backward pass (ADOP_TOUCHED_CHUNK in the header)
constexpr int kTouchedShift = 8, kTouchedChunk = 1 << kTouchedShift;
constexpr int kTileW = 32, kTileH = 16;   // screen tile, in layer-0 pixels (shifts 5 and 4 below)
constexpr int kTileShiftX = 5, kTileShiftY = 4;
constexpr unsigned kEntryDropped = 0x80000000u;

struct TileTable
{
    int n_tiles;
    int tiles_x, tiles_y;
    int w0, h0;
    int cap;      // entries per bucket
};
inline TileTable make_tile_table(int w, int h, int num_points)
{
    TileTable t;
    t.w0 = w; t.h0 = h;
    t.tiles_x = (w + kTileW - 1) / kTileW;
    t.tiles_y = (h + kTileH - 1) / kTileH;
    t.n_tiles = t.tiles_x * t.tiles_y;
    long long cap = 2ll * num_points / t.n_tiles;
    if (cap < 2048) cap = 2048;
    if (cap > num_points) cap = num_points;  // a bucket never needs more room than the cloud has points
    if (cap < 4) cap = 4;
    t.cap = (int)((cap + 3) & ~3ll);
    return t;
}
inline size_t tile_table_ints(int n_tiles) { return ((size_t)n_tiles + 3) & ~(size_t)3; }
inline size_t entry_capacity(int num_points) { return (size_t)num_points + (size_t)kVisibleSegments * kBlock; }
inline size_t visible_list_ints(int num_points, int w, int h)
{
    const TileTable t = make_tile_table(w, h, num_points);
    return (size_t)kVisibleHeaderInts + tile_table_ints(t.n_tiles) + 4 * (size_t)t.n_tiles * t.cap;
}
struct VisibleList
{
    int* header;     // null = no list
    int* tile_cur;   // [n_tiles] entries in each bucket
    int4* entries;   // bucket t: entries + t * cap
};
inline VisibleList make_visible_list(int32_t* base, int num_points, int w, int h, int view)
{
    VisibleList v;
    memset(&v, 0, sizeof(v));
    if (!base) return v;
    const int n_tiles = make_tile_table(w, h, num_points).n_tiles;
    int* p = base + (size_t)view * visible_list_ints(num_points, w, h);
    v.header = p;
    v.tile_cur = p + kVisibleHeaderInts;
    // 16-byte aligned: header, tile table and per-view size are multiples of 4 ints
    v.entries = reinterpret_cast<int4*>(p + kVisibleHeaderInts + tile_table_ints(n_tiles));
    return v;
}
// ints at the head of a view's list that the forward pass clears before the blend kernel appends
inline size_t visible_list_clear_ints(int w, int h, int num_points) { return (size_t)kVisibleHeaderInts + make_tile_table(w, h, num_points).n_tiles; }
#if defined(__CUDACC__)
// screen tile of an image position (clamped into the image: positions just outside layer 0 can still land in a coarser layer)
__device__ __forceinline__ int tile_of_position(const TileTable& tt, float x, float y)
{
    const int px = min(max(round_half_even_bounded(x), 0), tt.w0 - 1), py = min(max(round_half_even_bounded(y), 0), tt.h0 - 1);
    return (py >> kTileShiftY) * tt.tiles_x + (px >> kTileShiftX);
}
// Header words of the list that steer the backward pass on the device (no host round trip):
//   [kVisibleSegments + 2]  set by the forward pass: the list is not usable (a bucket overflowed)
//   [kVisibleSegments + 3]  set by the last kernel of a backward pass that turned the entries into work items: consumed
//   [kVisibleSegments + 4]  written by the first kernel of every backward pass (the tile kernel): 1 = this pass runs on the
//                           list, 0 = the all-points kernels behind it do the work. The later kernels of the pass read
//                           this word only, so nothing races with the mark in [+3].
constexpr int kListUnusable = kVisibleSegments + 2, kListConsumed = kVisibleSegments + 3, kListGo = kVisibleSegments + 4;
#endif

// Large region of a full workspace (behind the camera records and pixel records).
// Forward: candidate streams - the depth prepass leaves, per view of its group of up to four, the points that landed inside
// the image as (x, y, depth, point id) records, one segment per block, so that the blend kernel neither reads the
// positions again nor projects a second time.
constexpr int kCandViews = 4;
struct LargeRegion
{
    size_t cand_rec, cand_count, total;  // byte offsets from the region's start (forward)
};
inline LargeRegion large_region_layout(int num_points, int num_views)
{
    const int v = num_views < kCandViews ? (num_views < 1 ? 1 : num_views) : kCandViews;
    const size_t cap = entry_capacity(num_points);
    LargeRegion r;
    r.cand_rec = 0;
    r.cand_count = r.cand_rec + (size_t)v * cap * 16;
    r.total = r.cand_count + (size_t)v * kVisibleSegments * sizeof(int) + 256;
    return r;
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
// chunk of round k of this block, or -1 when the round has none (the last superblocks can be short)
__device__ __forceinline__ int scheduled_chunk(const ChunkSchedule& cs, int k)
{
    const int sb = (int)((blockIdx.x + (unsigned)k * (unsigned)cs.spread) % gridDim.x);
    const int chunk = sb * cs.rounds + k;
    return chunk < cs.chunks ? chunk : -1;
}
__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
#endif

}  // namespace adop
