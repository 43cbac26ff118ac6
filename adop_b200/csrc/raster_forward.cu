// Forward pass of the one-pixel point rasterizer for sm_100a: depth prepass, fuzzy-depth blend, resolve.
// Stands in for BlendPointCloudForward and its kernels (darglein/ADOP src/lib/rendering/PointRenderer.cu:
// DepthPrepassMulti :203-301, RenderForwardMulti :303-393, CombineAndFill :726-754, CreateMask :828-847)
// plus the environment-map composite of RenderModule.cpp:106-127 / EnvironmentMap.cu:62-156.
//
// Layout choices (none of these kernels is a dense contraction, so no tensor cores):
//  * points stream as one 128-bit load per thread; normals / indices are separate 4-byte streams;
//  * descriptor sums go to a pixel-interleaved accumulator record (C sums, padded to 16-byte vectors; the splat count
//    goes straight into the weight image when C is a multiple of four) so that one splat is one vector atomic per four
//    channels plus one scalar atomic, instead of C+1 atomics into C+1 planes;
//  * the resolve kernel turns records into the NCHW tensors of the operator's interface in a single pass
//    (normalise, background, environment map, mask, weight plane) and clears the records it read, so one accumulator
//    (44 MB at 1080p with four channels) is reused by every view of the batch. It does not stay in L2 while a 10 M point
//    cloud streams through: the blend kernel's L2 hit rate is about 40 %;
//  * the blend kernel also lists, per 32 x 16 screen tile, the points the backward pass will visit, and the depth prepass can
//    hand the blend kernel the projected in-image points (candidate streams) when the workspace has room for them.
#include <cooperative_groups.h>

#include <cstring>

#include "common.cuh"

namespace adop {

// ------------------------------------------------------------------------------------------------------
__global__ void k_fill(float* __restrict__ dst, size_t n, float v)
{
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    size_t n4 = n / 4;
    float4 v4 = make_float4(v, v, v, v);
    for (size_t k = i; k < n4; k += stride) reinterpret_cast<float4*>(dst)[k] = v4;
    for (size_t k = n4 * 4 + i; k < n; k += stride) dst[k] = v;
}

// [C,T] planes <-> [T,C] interleaved descriptors (one texel per thread; plane accesses are coalesced, interleaved
// accesses are contiguous vectors)
template <int C4>  // C4 = C / 4 when C is a multiple of 4 (vector stores), 0 = any C (scalar)
__global__ void k_texture_interleave(const float* __restrict__ in, float* __restrict__ out, int C, int T)
{
    for (int t = blockIdx.x * blockDim.x + threadIdx.x; t < T; t += gridDim.x * blockDim.x)
    {
        if (C4 > 0)
        {
#pragma unroll
            for (int k = 0; k < C4; ++k)
            {
                float4 v;
                v.x = __ldcs(in + (size_t)(4 * k + 0) * T + t); v.y = __ldcs(in + (size_t)(4 * k + 1) * T + t);
                v.z = __ldcs(in + (size_t)(4 * k + 2) * T + t); v.w = __ldcs(in + (size_t)(4 * k + 3) * T + t);
                reinterpret_cast<float4*>(out + (size_t)t * (4 * C4))[k] = v;
            }
        }
        else
            for (int c = 0; c < C; ++c) out[(size_t)t * C + c] = __ldcs(in + (size_t)c * T + t);
    }
}
template <int C4>
__global__ void k_texture_deinterleave(const float* __restrict__ in, float* __restrict__ out, int C, int T, int accumulate)
{
    for (int t = blockIdx.x * blockDim.x + threadIdx.x; t < T; t += gridDim.x * blockDim.x)
    {
        if (C4 > 0)
        {
#pragma unroll
            for (int k = 0; k < C4; ++k)
            {
                const float4 v = __ldcs(reinterpret_cast<const float4*>(in + (size_t)t * (4 * C4)) + k);
                const float vv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int j = 0; j < 4; ++j)
                {
                    float* dst = out + (size_t)(4 * k + j) * T + t;
                    *dst = accumulate ? *dst + vv[j] : vv[j];
                }
            }
        }
        else
            for (int c = 0; c < C; ++c)
            {
                float v = __ldcs(in + (size_t)t * C + c);
                float* dst = out + (size_t)c * T + t;
                *dst = accumulate ? *dst + v : v;
            }
    }
}

// ------------------------------------------------------------------------------------------------------
// K1: depth prepass. One thread per point and iteration; per layer an atomicMin on the float's bit pattern (valid
// because z > 0). On the coarser layers, where hundreds of points share a pixel, an early-z read first drops the points
// that cannot win (PointRenderer.cu:275-279; a stale value only costs an extra atomic). On the finest layer the read costs
// more than the atomics it saves, so it is skipped there. Warp-level aggregation of equal pixels (__match_any_sync) was
// measured 3-6x slower than plain atomics on this workload and is not used.
// PLAIN: neither the normal test nor the radius drop-out rule is in use, so their code (and registers) are compiled out.
// V consecutive views of the batch per launch (camera records and depth planes of a batch are consecutive): the point
// is loaded once and projected V times. Measured on the 4-layer prepass: 120 / 101 / 93 us per view for V = 1 / 2 / 4,
// 149 us for V = 8 (too many depth pyramids in flight), so groups of four are used.
// CAND: every point that lands inside the image of view v is also appended, as (x, y, depth, point id), to this block's
// segment of view v's candidate stream (warp vote + one shared-memory atomic per warp and view; a segment has room for
// every point of the block, so it cannot overflow). The blend kernel then reads those records instead of the positions
// and does not project again: it sees the same float x, y, depth, hence takes the same decisions bit for bit.
struct CandOut
{
    float4* rec;          // view v: rec + v * view_stride
    int* count;           // view v: count + v * kVisibleSegments, one entry per block
    size_t view_stride;   // records per view
    int seg_cap;          // records per block segment
};
template <int L, bool PLAIN, int V, bool CAND>
__global__ void __launch_bounds__(kBlock, 8) k_depth_prepass(PointStreams pts, ChunkSchedule sched, const ViewCam* __restrict__ camp, KernelParams kp,
                                                           LayerTable lt, CandOut co)
{
    static_assert(!CAND || PLAIN, "candidate records carry no drop-out radius");
    const bool use_normal = PLAIN ? false : kp.check_normal != 0;
    const bool use_radius = PLAIN ? false : kp.drop_out_points_by_radius != 0;
    __shared__ int s_cnt[V];
    const int lane = threadIdx.x & 31;
    if (CAND)
    {
        if (threadIdx.x < V) s_cnt[threadIdx.x] = 0;
        __syncthreads();
    }
    // warp-uniform trip count (the candidate append votes across the warp)
    for (int k = 0; k < sched.rounds; ++k)
    {
        const int chunk = scheduled_chunk(sched, k);
        if (chunk < 0) continue;  // block-uniform
        const int i = chunk * kBlock + threadIdx.x;
        const bool valid = i < pts.n;
        FetchedPoint f;
        f.p.x = f.p.y = f.p.z = f.r = 0.f; f.has_normal = false; f.n.x = f.n.y = f.n.z = 0.f;
        if (valid)
        {
            if (PLAIN) { float4 c = __ldg(pts.position + i); f.p.x = c.x; f.p.y = c.y; f.p.z = c.z; f.r = c.w; }
            else f = fetch_point(pts, i);
        }
#pragma unroll
        for (int v = 0; v < V; ++v)
        {
            RasterPoint q;
            q.x = q.y = q.z = q.radius_px = 0.f;
            bool in_image = false;
            if (valid && (PLAIN ? project_plain(camp[v], f.p, kp.dist_cutoff, &q)
                                : project_for_raster(camp[v], f.p, f.r, f.n, f.has_normal, use_normal, kp.dist_cutoff, &q, use_radius)))
            {
                float x = q.x, y = q.y, rad = q.radius_px;
                const int zi = __float_as_int(q.z);
#pragma unroll
                for (int l = 0; l < L; ++l, rad *= 0.5f, x *= 0.5f, y *= 0.5f)
                {
                    if (use_radius && rad < kp.drop_out_radius_threshold) break;
                    int px = round_half_even_bounded(x), py = round_half_even_bounded(y);
                    if ((unsigned)px >= (unsigned)lt.w[l] || (unsigned)py >= (unsigned)lt.h[l]) continue;
                    in_image = true;
                    // depth plane of view v of the group: the planes of a batch follow each other
                    // (32-bit index: a group's planes of one layer hold fewer than 2^31 pixels, checked by the entry point)
                    int* dst = reinterpret_cast<int*>(lt.depth[l]) + ((unsigned)(v * lt.h[l] + py) * (unsigned)lt.w[l] + (unsigned)px);
                    // early z: the plane is being updated by other blocks' atomicMin while it is read, so the read goes through L2
                    // (__ldcg), not the non-coherent path. A value that is older than the latest minimum can only be
                    // LARGER than the true one (depths only decrease), so it never drops a point that should win; at worst
                    // it lets through an atomic that changes nothing.
                    if (l == 0 || zi < __ldcg(dst)) atomicMin(dst, zi);
                }
            }
            if (CAND)
            {
                const unsigned vote = __ballot_sync(0xffffffffu, in_image);
                if (vote)
                {
                    int wbase = 0;
                    if (lane == 0) wbase = atomicAdd(&s_cnt[v], __popc(vote));
                    wbase = __shfl_sync(0xffffffffu, wbase, 0);
                    if (in_image)
                        co.rec[(size_t)v * co.view_stride + (size_t)blockIdx.x * co.seg_cap + wbase + __popc(vote & ((1u << lane) - 1u))] =
                            make_float4(q.x, q.y, q.z, __int_as_float(i));
                }
            }
        }
    }
    if (CAND)
    {
        __syncthreads();
        if (threadIdx.x < V) co.count[threadIdx.x * kVisibleSegments + blockIdx.x] = s_cnt[threadIdx.x];
    }
}

// K1b (optional by-product): the packed depth|index word per pixel (PackIndex / ExtractIndex,
// PointRendererHelper.h:21-34): one 64-bit atomicMin of (depth bits << 32 | point index) per layer the point lands in.
// The winner of a pixel is the nearest point, the lowest index among equal depths, whatever order the points come in.
struct PackedPlanes
{
    unsigned long long* plane[kMaxLayers];
};
__global__ void __launch_bounds__(kBlock) k_fill_u64(unsigned long long* __restrict__ dst, size_t n, unsigned long long v)
{
    for (size_t k = (size_t)blockIdx.x * blockDim.x + threadIdx.x; k < n; k += (size_t)gridDim.x * blockDim.x) dst[k] = v;
}
__global__ void __launch_bounds__(kBlock) k_depth_prepass_packed(PointStreams pts, const ViewCam* __restrict__ camp, KernelParams kp,
                                                                  LayerTable lt, PackedPlanes out)
{
    const ViewCam& cam = *camp;
    const bool use_normal = kp.check_normal != 0;
    const bool use_radius = kp.drop_out_points_by_radius != 0;
    const int stride = gridDim.x * blockDim.x;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < pts.n; i += stride)
    {
        FetchedPoint f = fetch_point(pts, i);
        RasterPoint q;
        if (!project_for_raster(cam, f.p, f.r, f.n, f.has_normal, use_normal, kp.dist_cutoff, &q, use_radius)) continue;
        float x = q.x, y = q.y, rad = q.radius_px;
        const unsigned long long word = ((unsigned long long)__float_as_uint(q.z) << 32) | (unsigned)i;
        for (int l = 0; l < lt.L; ++l, rad *= 0.5f, x *= 0.5f, y *= 0.5f)
        {
            if (use_radius && rad < kp.drop_out_radius_threshold) break;
            int px = round_half_even_bounded(x), py = round_half_even_bounded(y);
            if ((unsigned)px >= (unsigned)lt.w[l] || (unsigned)py >= (unsigned)lt.h[l]) continue;
            unsigned long long* dst = out.plane[l] + ((unsigned)py * (unsigned)lt.w[l] + (unsigned)px);
            if (word < __ldcg(dst)) atomicMin(dst, word);  // coherent read of a plane under update, see k_depth_prepass
        }
    }
}

// ------------------------------------------------------------------------------------------------------
// K2: fuzzy-depth blend into the interleaved accumulator.
// Accumulator layout. C % 4 == 0: the colour sums of a pixel are C/4 float4 (nothing padded) and the splat count goes
// straight into the layer's weight image, which is an output anyway (PointRenderer.cu:1006), so the resolve kernel
// neither writes the count nor clears a padded fifth value per pixel. Otherwise colours and count share one padded record.
template <int C>
struct AccumLayout
{
    static constexpr bool kSplit = C % 4 == 0;
    static constexpr int kFloats = kSplit ? C : ((C + 1) + 3) & ~3;
};
template <int C>
__device__ __forceinline__ void splat_record(float* rec, float* weight, const float* t)
{
    constexpr int full = C / 4;
    constexpr int rem = C % 4;
#pragma unroll
    for (int v = 0; v < full; ++v)
        atomicAdd(reinterpret_cast<float4*>(rec) + v, make_float4(t[4 * v], t[4 * v + 1], t[4 * v + 2], t[4 * v + 3]));
    if (rem == 0)
    {
        atomicAdd(weight, 1.0f);
    }
    else
    {
        float a[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int k = 0; k < rem; ++k) a[k] = t[4 * full + k];
        a[rem] = 1.0f;
        atomicAdd(reinterpret_cast<float4*>(rec) + full, make_float4(a[0], a[1], a[2], a[3]));
    }
}

// One kernel tests every candidate (or, without candidate streams, every point of the cloud) against the depth buffers
// and blends the accepted ones. Only about a third of the lanes of a warp that has accepted points at all have one (11 of
// 32 on the 1080p benchmark scene), so the work on accepted points - descriptor load, atomics, the list entry - is not
// done where the point is tested: a warp parks its accepted points (index, layer masks, image position) in a queue of its
// own in shared memory and finishes them 32 at a time with every lane busy.
// EMIT: the points the backward pass will visit are also written to the visible list, straight into the bucket of their
// screen tile (a run of lanes with the same tile takes consecutive slots behind one atomic). In ghost-gradient mode
// dropped points are tested too (they blend nothing but the backward pass needs them, PointRenderer.cu:487-488).
// CAND: block b reads the candidate segment that block b of the depth prepass wrote, (x, y, depth, point id) records,
// instead of the positions, and does not project.
struct CandIn
{
    const float4* rec;   // this view's records
    const int* count;    // this view's per-block counts
    int seg_cap;
};
template <int L, int C, bool PLAIN, bool CAND, bool EMIT>
__global__ void __launch_bounds__(kBlock, 8) k_blend(PointStreams pts, ChunkSchedule sched, CandIn cs, const float* __restrict__ texture,
                                                   const float* __restrict__ texture_interleaved, int num_texels,
                                                   const ViewCam* __restrict__ camp, KernelParams kp, LayerTable lt, TileTable tt,
                                                   float* __restrict__ accum, VisibleList vl, unsigned char* __restrict__ touched_points,
                                                   unsigned char* __restrict__ touched_texels)
{
    static_assert(!CAND || PLAIN, "candidate records carry no drop-out radius");
    const ViewCam& cam = *camp;
    const bool use_normal = PLAIN ? false : kp.check_normal != 0;
    const bool use_radius = PLAIN ? false : kp.drop_out_points_by_radius != 0;
    constexpr int RS = AccumLayout<C>::kFloats;
    const int lane = threadIdx.x & 31;
    // parked record: point id | dropped, forward mask | backward mask << 8, x, y
    __shared__ int4 s_park[kBlock / 32][64];
    int4* park = s_park[threadIdx.x >> 5];
    int n_parked = 0;  // the same in every lane of the warp

    // masks of a projected point: forward mask (layers to blend: landed and passed the depth test) | backward mask << 8
    // (the layers the backward pass will visit: it skips layers the point does not land in and stops at the first depth
    // failure, PointRenderer.cu:451-462)
    auto test_layers = [&](float x, float y, float z, float rad) -> unsigned
    {
        int lin[L];
        bool in[L];
        bool live = true;
#pragma unroll
        for (int l = 0; l < L; ++l, rad *= 0.5f, x *= 0.5f, y *= 0.5f)
        {
            if (use_radius && rad < kp.drop_out_radius_threshold) live = false;  // break, :368-371
            int px = round_half_even_bounded(x), py = round_half_even_bounded(y);
            in[l] = live && (unsigned)px < (unsigned)lt.w[l] && (unsigned)py < (unsigned)lt.h[l];
            lin[l] = py * lt.w[l] + px;
        }
        unsigned pass = 0;  // the depth reads of all layers go out together
#pragma unroll
        for (int l = 0; l < L; ++l)
        {
            float image_depth = in[l] ? __ldg(lt.depth[l] + lin[l]) : 0.f;
            if (in[l] && !(z > image_depth * kp.depth_accept_plus_one)) pass |= 1u << l;
        }
        if (!EMIT) return pass;
        unsigned bmask = 0;
#pragma unroll
        for (int l = 0; l < L; ++l)
        {
            if (!in[l]) continue;
            if (!(pass & (1u << l))) break;
            bmask |= 1u << l;
        }
        return pass | (bmask << 8);
    };
    // one candidate / point -> parked record (y = 0: nothing to do)
    auto make_entry = [&](int i, float4 cur) -> int4
    {
        const bool dropped = point_dropped(kp, i);
        if (dropped && !(EMIT && kp.ghost_gradients)) return make_int4(0, 0, 0, 0);
        float x, y;
        unsigned masks;
        if (CAND)
        {
            x = cur.x; y = cur.y;
            masks = test_layers(cur.x, cur.y, cur.z, 0.f);
        }
        else
        {
            FetchedPoint f;
            if (PLAIN) { f.p.x = cur.x; f.p.y = cur.y; f.p.z = cur.z; f.r = cur.w; f.has_normal = false; f.n.x = f.n.y = f.n.z = 0.f; }
            else f = fetch_point(pts, i, cur);
            RasterPoint q;
            if (PLAIN ? !project_plain(cam, f.p, kp.dist_cutoff, &q)
                      : !project_for_raster(cam, f.p, f.r, f.n, f.has_normal, use_normal, kp.dist_cutoff, &q, use_radius)) return make_int4(0, 0, 0, 0);
            x = q.x; y = q.y;
            masks = test_layers(q.x, q.y, q.z, q.radius_px);
        }
        if (dropped) masks &= 0xff00u;  // a dropped point blends nothing
        return make_int4((int)((unsigned)i | (dropped ? kEntryDropped : 0u)), (int)masks, __float_as_int(x), __float_as_int(y));
    };
    // All 32 lanes together: blend the accepted point of every valid lane and write its list entry.
    auto finish = [&](bool valid, int4 e)
    {
        const unsigned code = valid ? ((unsigned)e.y & 0xffu) : 0u;
        if (code)
        {
            const int i = (int)((unsigned)e.x & ~kEntryDropped);
            float t[C];
            const int ti = pts.index ? __ldg(pts.index + i) : i;
            load_descriptor<C>(texture, texture_interleaved, num_texels, ti, t);
            float x = __int_as_float(e.z), y = __int_as_float(e.w);
#pragma unroll
            for (int l = 0; l < L; ++l, x *= 0.5f, y *= 0.5f)
                if (code & (1u << l))
                {
                    const int lin = round_half_even_bounded(y) * lt.w[l] + round_half_even_bounded(x);
                    splat_record<C>(accum + ((size_t)lt.rec_off[l] + lin) * RS, lt.weight[l] + lin, t);
                }
        }
        if (EMIT)
        {
            const bool keep = valid && ((unsigned)e.y >> 8) != 0;
            if (__ballot_sync(0xffffffffu, keep))
            {
                // the lanes of one tile take consecutive slots behind one atomic (32 Morton neighbours spread over a few
                // tiles: grouping all lanes of a tile, not only adjacent ones, sends a third of the atomics)
                const int tile = keep ? tile_of_position(tt, __int_as_float(e.z), __int_as_float(e.w)) : -1;
                const unsigned same = __match_any_sync(0xffffffffu, tile);
                const int leader = __ffs(same) - 1;
                int slot = 0;
                if (keep && leader == lane) slot = atomicAdd(vl.tile_cur + tile, __popc(same));
                slot = __shfl_sync(0xffffffffu, slot, leader) + __popc(same & ((1u << lane) - 1u));
                if (keep)
                {
                    if (slot < tt.cap) vl.entries[(size_t)tile * tt.cap + slot] = e;
                    else vl.header[kListUnusable] = 1;  // the bucket is full: the backward pass walks all points instead
                }
            }
        }
    };
    // chunk >= 0: all 32 points belong to that chunk of kBlock consecutive points; -1: they are candidates from anywhere
    auto park_and_finish = [&](int4 e, int chunk)
    {
        const bool keep = e.y != 0;
        const unsigned vote = __ballot_sync(0xffffffffu, keep);
        if (vote)
        {
            // the backward pass can add gradients only where a point was kept: one mark per warp and chunk
            if (touched_points)
            {
                if (chunk >= 0)
                {
                    if (lane == 0) { touched_points[chunk] = 1; touched_texels[chunk] = 1; }
                }
                else if (keep)
                {
                    const int c = (int)(((unsigned)e.x & ~kEntryDropped) >> kTouchedShift);
                    if (touched_points[c] == 0) { touched_points[c] = 1; touched_texels[c] = 1; }
                }
            }
            if (keep) park[n_parked + __popc(vote & ((1u << lane) - 1u))] = e;
            n_parked += __popc(vote);
            __syncwarp();
            if (n_parked >= 32)
            {
                n_parked -= 32;
                finish(true, park[n_parked + lane]);
            }
            __syncwarp();
        }
    };
    // warp-uniform trip counts: parking and finishing use full-warp votes and shuffles
    if (CAND)
    {
        const int cnt = __ldg(cs.count + blockIdx.x);
        const float4* rec = cs.rec + (size_t)blockIdx.x * cs.seg_cap;
        for (int k0 = 0; k0 < cnt; k0 += kBlock)
        {
            const int k = k0 + threadIdx.x;
            int4 e = make_int4(0, 0, 0, 0);
            if (k < cnt)
            {
                const float4 c = __ldcs(rec + k);
                e = make_entry(__float_as_int(c.w), c);
            }
            park_and_finish(e, -1);
        }
    }
    else
    {
        for (int k = 0; k < sched.rounds; ++k)
        {
            const int chunk = scheduled_chunk(sched, k);
            if (chunk < 0) continue;  // block-uniform
            const int i = chunk * kBlock + threadIdx.x;
            int4 e = make_int4(0, 0, 0, 0);
            if (i < pts.n) e = make_entry(i, __ldg(pts.position + i));
            park_and_finish(e, chunk);
        }
    }
    if (n_parked > 0) finish(lane < n_parked, lane < n_parked ? park[lane] : make_int4(0, 0, 0, 0));
}

// ------------------------------------------------------------------------------------------------------
// K3: resolve. One thread per pyramid pixel of the view (all layers in one launch).
// Uncovered pixels that take the environment map need a ray through the inverse camera model and a spherical lookup,
// a few hundred instructions, and they are scattered (single-pixel holes between splats), so that almost every warp
// would run that code for a handful of lanes. Instead each warp parks its holes in a small queue of its own and works
// them off 32 at a time with all lanes busy (measured on the 1080p pyramid with 15 % holes: 55 -> 28 us without the
// environment map, which is what the parked version aims at).
template <int C>
__device__ __forceinline__ void resolve_environment_pixel(const LayerTable& lt, const ViewCam& cam, const KernelParams& kp, unsigned r,
                                                          const float* __restrict__ background, const float* __restrict__ env,
                                                          int env_h, int env_w)
{
    const int l = layer_of_record(lt, r);
    const unsigned pix = r - lt.rec_off[l];
    const int w = lt.w[l];
    const size_t plane = (size_t)w * lt.h[l];
    const int gy = pix / w, gx = pix - gy * w;
    Intr5 crop_l = scale_intr(cam.crop, __int_as_float((127 - l) << 23));  // 0.5^l
    V2 uv = env_uv_for_pixel(gx, gy, cam.V, cam.K, cam.dist, crop_l);
    BilinearTap tp = bilinear_taps(uv, env_w, env_h);
    const float one_minus_m = 1.0f - kp.mask_background_value;
    float* color = lt.color[l] + pix;
#pragma unroll
    for (int c = 0; c < C; ++c)
    {
        const float* e = env + (size_t)c * env_h * env_w;
        float e00 = __ldg(e + (size_t)tp.y0 * env_w + tp.x0), e01 = __ldg(e + (size_t)tp.y0 * env_w + tp.x1);
        float e10 = __ldg(e + (size_t)tp.y1 * env_w + tp.x0), e11 = __ldg(e + (size_t)tp.y1 * env_w + tp.x1);
        float top = e00 + (e01 - e00) * tp.wx;
        float bot = e10 + (e11 - e10) * tp.wx;
        float ev = top + (bot - top) * tp.wy;
        color[c * plane] = __ldg(background + c) + one_minus_m * ev;
    }
}

template <int C>
__global__ void __launch_bounds__(kBlock, 6) k_resolve(LayerTable lt, const ViewCam* __restrict__ camp, KernelParams kp, float* __restrict__ accum,
                                                     const float* __restrict__ background, const float* __restrict__ env,
                                                     int env_h, int env_w)
{
    const ViewCam& cam = *camp;
    constexpr int RS = AccumLayout<C>::kFloats;
    constexpr bool kSplit = AccumLayout<C>::kSplit;
    __shared__ unsigned s_parked[kBlock / 32][64];
    unsigned* parked = s_parked[threadIdx.x >> 5];
    const int lane = threadIdx.x & 31;
    int n_parked = 0;  // the same in every lane of the warp
    const unsigned total = lt.rec_off[kMaxLayers];
    const unsigned stride = gridDim.x * blockDim.x;
    // warp-uniform trip count: the parking uses full-warp votes
    for (unsigned base = blockIdx.x * blockDim.x; base < total; base += stride)
    {
        const unsigned r = base + threadIdx.x;
        bool hole = false;
        if (r < total)
        {
            const int l = layer_of_record(lt, r);
            const unsigned pix = r - lt.rec_off[l];
            const size_t plane = (size_t)lt.w[l] * lt.h[l];
            float4* rec = reinterpret_cast<float4*>(accum + (size_t)r * RS);
            // split layout: the blend kernel counted into the weight image itself (requested together with the record:
            // a dependent second load costs more than the bytes it could save)
            const float cou_split = kSplit ? __ldcg(lt.weight[l] + pix) : 0.f;
            float v[RS];
#pragma unroll
            for (int k = 0; k < RS / 4; ++k)
            {
                float4 a = __ldcg(rec + k);
                v[4 * k] = a.x; v[4 * k + 1] = a.y; v[4 * k + 2] = a.z; v[4 * k + 3] = a.w;
            }
            const float cou = kSplit ? cou_split : v[C < RS ? C : 0];
            float* color = lt.color[l] + pix;
            if (!kSplit) lt.weight[l][pix] = cou;
            if (lt.mask[l]) lt.mask[l][pix] = cou == 0.f ? kp.mask_background_value : 1.f;
            if (cou == 0.f)
            {
                hole = env != nullptr;
                if (!hole)
                {
#pragma unroll
                    for (int c = 0; c < C; ++c) color[c * plane] = __ldg(background + c);
                }
            }
            else
            {
                // one division per pixel instead of one per channel: sum * (1 / count) is within an ulp of sum / count, far
                // inside what the order of the atomic sums already leaves open; a single splat (count 1) stays exact
                const float inv = reciprocal(cou);
#pragma unroll
                for (int c = 0; c < C; ++c) color[c * plane] = v[c] * inv;
                // leave the record clean for the next view
#pragma unroll
                for (int k = 0; k < RS / 4; ++k) rec[k] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
        const unsigned vote = __ballot_sync(0xffffffffu, hole);
        if (vote)
        {
            if (hole) parked[n_parked + __popc(vote & ((1u << lane) - 1u))] = r;
            n_parked += __popc(vote);
            __syncwarp();
            if (n_parked >= 32)
            {
                n_parked -= 32;
                resolve_environment_pixel<C>(lt, cam, kp, parked[n_parked + lane], background, env, env_h, env_w);
            }
            __syncwarp();
        }
    }
    if (lane < n_parked) resolve_environment_pixel<C>(lt, cam, kp, parked[lane], background, env, env_h, env_w);
}

// ------------------------------------------------------------------------------------------------------
// What one forward call decided once for all its views.
struct ForwardPlan
{
    float* accum;
    bool env;
    int32_t* list_base;   // null = no visible list
    int w, h;             // layer-0 size (geometry of the visible list)
    int num_views;
    char* large;          // large region of a full workspace (candidate streams), null = small workspace
    LargeRegion lr;
    size_t cand_view_stride;  // records per candidate stream
    TileTable tiles;
    PointStreams outliers;  // the optional second cloud (n = 0: none): forward only, never listed
    unsigned char* touched_points;  // optional flags per chunk of kTouchedChunk points / texels (null: none)
    unsigned char* touched_texels;
};

template <int L, int C, bool PLAIN>
static adop_status launch_view_forward_impl(const PointStreams& pts, const adop_scene* s, const ViewCam* cam, const KernelParams& kp,
                                            const LayerTable& lt, const ForwardPlan& plan, cudaStream_t st, int view, int depth_views)
{
    constexpr bool kCand = PLAIN;  // candidate streams exist when neither the normal test nor the radius rule is in use
    static const int g_depth = resident_grid(k_depth_prepass<L, PLAIN, 4, false>, 1ll << 40);
    static const int g_depth_cand = resident_grid(k_depth_prepass<L, PLAIN, 4, kCand>, 1ll << 40);
    static const int g_blend = resident_grid(k_blend<L, C, PLAIN, false, false>, 1ll << 40);
    static const int g_blend_emit = resident_grid(k_blend<L, C, PLAIN, false, true>, 1ll << 40);
    static const int g_blend_cand = resident_grid(k_blend<L, C, PLAIN, kCand, false>, 1ll << 40);
    static const int g_blend_cand_emit = resident_grid(k_blend<L, C, PLAIN, kCand, true>, 1ll << 40);
    static const int g_resolve = resident_grid(k_resolve<C>, 1ll << 40);
    const int need = (pts.n + kBlock - 1) / kBlock;
    const bool cand = kCand && plan.large != nullptr;
    const bool emit = plan.list_base != nullptr;
    // With candidate streams the depth prepass and the blend kernel run on the same grid (block b of the blend kernel reads
    // what block b of the prepass wrote).
    int grid_blend = cand ? (emit ? g_blend_cand_emit : g_blend_cand) : (emit ? g_blend_emit : g_blend);
    if (cand)
    {
        if (grid_blend > g_depth_cand) grid_blend = g_depth_cand;
        if (grid_blend > kVisibleSegments) grid_blend = kVisibleSegments;
    }
    if (grid_blend > need) grid_blend = need < 1 ? 1 : need;
    const int seg_cap = (int)((((long long)need + grid_blend - 1) / grid_blend) * kBlock);
    CandOut co;
    co.rec = cand ? reinterpret_cast<float4*>(plan.large + plan.lr.cand_rec) : nullptr;
    co.count = cand ? reinterpret_cast<int*>(plan.large + plan.lr.cand_count) : nullptr;
    co.view_stride = plan.cand_view_stride;
    co.seg_cap = seg_cap;
    // the depth prepass of this view was done by the launch of its group's first view, unless this is that view
    if (depth_views > 0)
    {
        const int grid_depth = cand ? grid_blend : (need < g_depth ? (need < 1 ? 1 : need) : g_depth);
#define ADOP_PREPASS(VV)                                                                                                         \
    if (cand) ADOP_LAUNCH("k_depth_prepass", st, (k_depth_prepass<L, PLAIN, VV, kCand><<<grid_depth, kBlock, 0, st>>>(pts, make_chunk_schedule(pts.n, grid_depth), cam, kp, lt, co))); \
    else ADOP_LAUNCH("k_depth_prepass", st, (k_depth_prepass<L, PLAIN, VV, false><<<grid_depth, kBlock, 0, st>>>(pts, make_chunk_schedule(pts.n, grid_depth), cam, kp, lt, co)));
        switch (depth_views)
        {
            case 1: ADOP_PREPASS(1) break;
            case 2: ADOP_PREPASS(2) break;
            case 3: ADOP_PREPASS(3) break;
            default: ADOP_PREPASS(4) break;
        }
#undef ADOP_PREPASS
        // the second cloud goes into the same depth planes (PointRenderer.cu:1421-1424); never through candidate streams
        if (plan.outliers.n > 0)
        {
            const PointStreams& op = plan.outliers;
            const int oneed = (op.n + kBlock - 1) / kBlock;
            const int og = oneed < g_depth ? oneed : g_depth;
            CandOut none;
            none.rec = nullptr; none.count = nullptr; none.view_stride = 0; none.seg_cap = 0;
#define ADOP_PREPASS_OUT(VV) ADOP_LAUNCH("k_depth_prepass", st, (k_depth_prepass<L, PLAIN, VV, false><<<og, kBlock, 0, st>>>(op, make_chunk_schedule(op.n, og), cam, kp, lt, none)))
            switch (depth_views)
            {
                case 1: ADOP_PREPASS_OUT(1); break;
                case 2: ADOP_PREPASS_OUT(2); break;
                case 3: ADOP_PREPASS_OUT(3); break;
                default: ADOP_PREPASS_OUT(4); break;
            }
#undef ADOP_PREPASS_OUT
        }
    }
    VisibleList vl = make_visible_list(plan.list_base, pts.n, plan.w, plan.h, view);
    if (vl.header) ADOP_CUDA_TRY(cudaMemsetAsync(vl.header, 0, sizeof(int) * visible_list_clear_ints(plan.w, plan.h, pts.n), st));
    CandIn ci;
    ci.rec = cand ? co.rec + (size_t)(view % kCandViews) * plan.cand_view_stride : nullptr;
    ci.count = cand ? co.count + (view % kCandViews) * kVisibleSegments : nullptr;
    ci.seg_cap = seg_cap;
#define ADOP_BLEND(CAND_, EMIT_)                                                                                                 \
    ADOP_LAUNCH("k_blend", st, (k_blend<L, C, PLAIN, CAND_, EMIT_><<<grid_blend, kBlock, 0, st>>>(                               \
                                   pts, make_chunk_schedule(pts.n, grid_blend), ci, s->texture, s->texture_interleaved, s->num_texels, cam, kp, lt, plan.tiles, plan.accum, vl, emit ? plan.touched_points : nullptr, emit ? plan.touched_texels : nullptr)))
    if (cand)
    {
        if (emit) ADOP_BLEND(kCand, true); else ADOP_BLEND(kCand, false);
    }
    else
    {
        if (emit) ADOP_BLEND(false, true); else ADOP_BLEND(false, false);
    }
    // the second cloud is blended into the same accumulator (PointRenderer.cu:1437-1440), from its positions, without a list
    if (plan.outliers.n > 0)
    {
        const PointStreams& op = plan.outliers;
        const int oneed = (op.n + kBlock - 1) / kBlock;
        const int og = oneed < g_blend ? oneed : g_blend;
        CandIn no_cand;
        no_cand.rec = nullptr; no_cand.count = nullptr; no_cand.seg_cap = 0;
        VisibleList no_list = make_visible_list(nullptr, op.n, plan.w, plan.h, view);
        ADOP_LAUNCH("k_blend", st, (k_blend<L, C, PLAIN, false, false><<<og, kBlock, 0, st>>>(
                                       op, make_chunk_schedule(op.n, og), no_cand, s->texture, s->texture_interleaved, s->num_texels, cam, kp, lt,
                                       plan.tiles, plan.accum, no_list, nullptr, nullptr)));
    }
#undef ADOP_BLEND
    unsigned total = lt.rec_off[kMaxLayers];
    int grid_px = (int)((total + kBlock - 1) / kBlock);
    if (grid_px > g_resolve) grid_px = g_resolve;
    ADOP_LAUNCH("k_resolve", st, (k_resolve<C><<<grid_px, kBlock, 0, st>>>(lt, cam, kp, plan.accum, s->background,
                                                                          plan.env ? s->env_map : nullptr, s->env_h, s->env_w)));
    ADOP_CUDA_TRY(cudaGetLastError());
    return ADOP_OK;
}

template <int L, int C>
static adop_status launch_view_forward(const PointStreams& pts, const adop_scene* s, const ViewCam* cam, const KernelParams& kp,
                                       const LayerTable& lt, const ForwardPlan& plan, cudaStream_t st, int view, int depth_views)
{
    // the common case - no normal test (or no normals) and no radius drop-out - gets kernels without that code
    const bool plain = !(kp.check_normal && (pts.normal || plan.outliers.normal)) && !kp.drop_out_points_by_radius;
    return plain ? launch_view_forward_impl<L, C, true>(pts, s, cam, kp, lt, plan, st, view, depth_views)
                 : launch_view_forward_impl<L, C, false>(pts, s, cam, kp, lt, plan, st, view, depth_views);
}

template <int C>
static adop_status dispatch_layers_forward(int L, const PointStreams& pts, const adop_scene* s, const ViewCam* cam,
                                           const KernelParams& kp, const LayerTable& lt, const ForwardPlan& plan,
                                           cudaStream_t st, int view, int depth_views)
{
    switch (L)
    {
        case 1: return launch_view_forward<1, C>(pts, s, cam, kp, lt, plan, st, view, depth_views);
        case 2: return launch_view_forward<2, C>(pts, s, cam, kp, lt, plan, st, view, depth_views);
        case 3: return launch_view_forward<3, C>(pts, s, cam, kp, lt, plan, st, view, depth_views);
        case 4: return launch_view_forward<4, C>(pts, s, cam, kp, lt, plan, st, view, depth_views);
        case 5: return launch_view_forward<5, C>(pts, s, cam, kp, lt, plan, st, view, depth_views);
        case 6: return launch_view_forward<6, C>(pts, s, cam, kp, lt, plan, st, view, depth_views);
        case 7: return launch_view_forward<7, C>(pts, s, cam, kp, lt, plan, st, view, depth_views);
        case 8: return launch_view_forward<8, C>(pts, s, cam, kp, lt, plan, st, view, depth_views);
    }
    return ADOP_ERR_INVALID_ARGUMENT;
}

}  // namespace adop

using namespace adop;

extern "C" size_t adop_raster_workspace_bytes(int32_t w, int32_t h, int32_t layers, int32_t channels)
{
    if (w <= 0 || h <= 0 || layers <= 0 || layers > ADOP_MAX_LAYERS || channels <= 0) return 0;
    LayerTable lt;
    fill_layer_dims(w, h, layers, &lt);
    // forward: accumulator records (C sums + weight); backward: interleaved [image | gradient] records
    int fwd = record_floats(channels), bwd = (2 * channels + 3) & ~3;
    size_t bytes = (size_t)lt.rec_off[kMaxLayers] * (fwd > bwd ? fwd : bwd) * sizeof(float);
    return kCamRegionBytes + bytes + 256;  // per-view camera records, then the pixel records
}

// The small workspace rounded up to 256 bytes = where the large region of a full workspace starts.
static size_t workspace_large_offset(int32_t w, int32_t h, int32_t layers, int32_t channels)
{
    return (adop_raster_workspace_bytes(w, h, layers, channels) + 255) & ~(size_t)255;
}

extern "C" size_t adop_raster_workspace_bytes_full(int32_t num_points, int32_t num_views, int32_t w, int32_t h, int32_t layers,
                                                   int32_t channels)
{
    const size_t small = adop_raster_workspace_bytes(w, h, layers, channels);
    if (small == 0 || num_points < 0 || num_views <= 0) return 0;
    // candidate streams of a group of views
    return workspace_large_offset(w, h, layers, channels) + large_region_layout(num_points, num_views).total;
}

extern "C" adop_status adop_texture_interleave(const float* texture, float* out, int32_t channels, int32_t num_texels, void* stream)
{
    if (!texture || !out || channels <= 0 || num_texels <= 0) return ADOP_ERR_INVALID_ARGUMENT;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int grid = (num_texels + kBlock - 1) / kBlock;
    if (grid > sm_count() * 16) grid = sm_count() * 16;
    switch (channels)
    {
        case 4: ADOP_LAUNCH("k_texture_interleave", st, (k_texture_interleave<1><<<grid, kBlock, 0, st>>>(texture, out, channels, num_texels))); break;
        case 8: ADOP_LAUNCH("k_texture_interleave", st, (k_texture_interleave<2><<<grid, kBlock, 0, st>>>(texture, out, channels, num_texels))); break;
        case 16: ADOP_LAUNCH("k_texture_interleave", st, (k_texture_interleave<4><<<grid, kBlock, 0, st>>>(texture, out, channels, num_texels))); break;
        default: ADOP_LAUNCH("k_texture_interleave", st, (k_texture_interleave<0><<<grid, kBlock, 0, st>>>(texture, out, channels, num_texels))); break;
    }
    ADOP_CUDA_TRY(cudaGetLastError());
    return ADOP_OK;
}

extern "C" adop_status adop_texture_deinterleave(const float* in, float* out, int32_t channels, int32_t num_texels,
                                                 int32_t accumulate, void* stream)
{
    if (!in || !out || channels <= 0 || num_texels <= 0) return ADOP_ERR_INVALID_ARGUMENT;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int grid = (num_texels + kBlock - 1) / kBlock;
    if (grid > sm_count() * 16) grid = sm_count() * 16;
    switch (channels)
    {
        case 4: ADOP_LAUNCH("k_texture_deinterleave", st, (k_texture_deinterleave<1><<<grid, kBlock, 0, st>>>(in, out, channels, num_texels, accumulate))); break;
        case 8: ADOP_LAUNCH("k_texture_deinterleave", st, (k_texture_deinterleave<2><<<grid, kBlock, 0, st>>>(in, out, channels, num_texels, accumulate))); break;
        case 16: ADOP_LAUNCH("k_texture_deinterleave", st, (k_texture_deinterleave<4><<<grid, kBlock, 0, st>>>(in, out, channels, num_texels, accumulate))); break;
        default: ADOP_LAUNCH("k_texture_deinterleave", st, (k_texture_deinterleave<0><<<grid, kBlock, 0, st>>>(in, out, channels, num_texels, accumulate))); break;
    }
    ADOP_CUDA_TRY(cudaGetLastError());
    return ADOP_OK;
}

extern "C" size_t adop_raster_visible_list_ints(int32_t num_points, int32_t w, int32_t h, int32_t layers)
{
    if (num_points < 0 || w <= 0 || h <= 0 || layers <= 0 || layers > ADOP_MAX_LAYERS) return 0;
    return visible_list_ints(num_points, w, h);
}

extern "C" adop_status adop_raster_forward(const adop_scene* s, const adop_view* views, int32_t B,
                                           const adop_render_params* rp, int32_t L, adop_forward_io* io, void* stream)
{
    adop_status vs = validate_common(s, views, B, rp, L);
    if (vs != ADOP_OK) return vs;
    if (!io || !io->workspace) return ADOP_ERR_INVALID_ARGUMENT;
    const int C = s->channels, N = s->num_points;
    const int w0 = views[0].w, h0 = views[0].h;
    if (io->workspace_bytes < adop_raster_workspace_bytes(w0, h0, L, C)) return ADOP_ERR_WORKSPACE_TOO_SMALL;
    if ((reinterpret_cast<uintptr_t>(io->workspace) & 15) || (reinterpret_cast<uintptr_t>(s->position) & 15))
        return ADOP_ERR_INVALID_ARGUMENT;
    const bool env = rp->composite_environment_map && s->env_map;
    for (int l = 0; l < L; ++l)
    {
        if (!io->layers[l].color || !io->layers[l].depth || !io->layers[l].weight) return ADOP_ERR_INVALID_ARGUMENT;
        if (rp->output_background_mask && !io->layers[l].mask) return ADOP_ERR_INVALID_ARGUMENT;
    }
    if (env)
        for (int b = 0; b < B; ++b)
            if (views[b].camera_model != ADOP_CAMERA_PINHOLE_DISTORTION) return ADOP_ERR_UNSUPPORTED;  // EnvironmentMap.cu:129

    cudaStream_t st = static_cast<cudaStream_t>(stream);
    LayerTable base;
    fill_layer_dims(w0, h0, L, &base);
    ViewCam* cams = static_cast<ViewCam*>(io->workspace);
    float* accum = reinterpret_cast<float*>(static_cast<char*>(io->workspace) + kCamRegionBytes);
    const bool split = C % 4 == 0;  // AccumLayout: colour sums only, the counts go into the weight images
    const size_t accum_bytes = (size_t)base.rec_off[kMaxLayers] * (split ? C : record_floats(C)) * sizeof(float);
    ADOP_CUDA_TRY(cudaMemsetAsync(accum, 0, accum_bytes, st));
    if (split)
        for (int l = 0; l < L; ++l)
            ADOP_CUDA_TRY(cudaMemsetAsync(io->layers[l].weight, 0, sizeof(float) * (size_t)B * base.w[l] * base.h[l], st));
    const int sms = sm_count();
    // depth.fill_(100000), PointRenderer.cu:1045 (weights and colours are written by the resolve kernel)
    for (int l = 0; l < L; ++l)
    {
        size_t n = (size_t)B * base.w[l] * base.h[l];
        if (n == 0) continue;
        int grid = (int)((n / 4 + kBlock - 1) / kBlock) + 1;
        if (grid > sms * 16) grid = sms * 16;
        ADOP_LAUNCH("k_fill", st, (k_fill<<<grid, kBlock, 0, st>>>(io->layers[l].depth, n, kDepthInit)));
    }
    // optional packed depth|index planes: all layers or none
    const bool packed = io->packed_depth[0] != nullptr;
    for (int l = 0; l < L; ++l)
        if ((io->packed_depth[l] != nullptr) != packed || (reinterpret_cast<uintptr_t>(io->packed_depth[l]) & 7))
            return ADOP_ERR_INVALID_ARGUMENT;
    if (packed)
    {
        unsigned init_bits;
        const float init_depth = kDepthInit;
        memcpy(&init_bits, &init_depth, sizeof(init_bits));
        const unsigned long long empty = ((unsigned long long)init_bits << 32) | 0xFFFFFFFFull;
        for (int l = 0; l < L; ++l)
        {
            size_t n = (size_t)B * base.w[l] * base.h[l];
            if (n == 0) continue;
            int grid = (int)((n + kBlock - 1) / kBlock);
            if (grid > sms * 16) grid = sms * 16;
            ADOP_LAUNCH("k_fill", st, (k_fill_u64<<<grid, kBlock, 0, st>>>(reinterpret_cast<unsigned long long*>(io->packed_depth[l]), n, empty)));
        }
    }
    ADOP_CUDA_TRY(cudaGetLastError());

    PointStreams pts;
    pts.position = reinterpret_cast<const float4*>(s->position);
    pts.normal = s->normal;
    pts.index = s->index;
    pts.n = N;
    ForwardPlan plan;
    plan.accum = accum;
    plan.env = env;
    plan.list_base = io->visible_list;
    plan.w = w0; plan.h = h0;
    plan.num_views = B;
    plan.tiles = make_tile_table(w0, h0, N);
    // flags "the backward pass of these views can touch this chunk": zeroed here, set by the blend kernel where it lists a
    // point; descriptor columns follow the point numbers only without an index array, else every texel chunk counts as touched
    static_assert(kTouchedChunk == kBlock, "the blend kernel marks one flag per chunk of kBlock points");
    if ((io->touched_points != nullptr) != (io->touched_texels != nullptr) || (io->touched_points && !io->visible_list))
        return ADOP_ERR_INVALID_ARGUMENT;
    plan.touched_points = io->touched_points;
    plan.touched_texels = io->touched_texels;
    if (io->touched_points)
    {
        const size_t t_chunks = ((size_t)s->num_texels + kTouchedChunk - 1) / kTouchedChunk;
        ADOP_CUDA_TRY(cudaMemsetAsync(io->touched_points, 0, ((size_t)N + kTouchedChunk - 1) / kTouchedChunk, st));
        ADOP_CUDA_TRY(cudaMemsetAsync(io->touched_texels, s->index ? 1 : 0, t_chunks, st));
        if (s->index) plan.touched_texels = io->touched_points;  // the kernel's second store then repeats the first
    }
    plan.outliers.position = reinterpret_cast<const float4*>(s->outlier_position);
    plan.outliers.normal = s->outlier_normal;
    plan.outliers.index = s->outlier_index;
    plan.outliers.n = s->outlier_position ? s->num_outliers : 0;
    plan.large = nullptr;
    plan.lr = large_region_layout(N, B);
    plan.cand_view_stride = entry_capacity(N);
    // A workspace of adop_raster_workspace_bytes_full has a large region behind the pixel records: candidate streams from
    // the depth prepass to the accept kernel, and the accept kernel's entry segments.
    if (io->workspace_bytes >= adop_raster_workspace_bytes_full(N, B, w0, h0, L, C))
        plan.large = static_cast<char*>(io->workspace) + workspace_large_offset(w0, h0, L, C);
    // the pose and intrinsics tensors live on the device; the per-view cameras are gathered there, a chunk at a time
    for (int b = 0; b < B; ++b)
    {
        if (b % kCamChunk == 0)
        {
            CamChunkSource src;
            fill_cam_chunk(&src, s, views + b, B - b < kCamChunk ? B - b : kCamChunk);
            ADOP_LAUNCH("k_build_cams", st, (k_build_cams<<<1, kCamChunk, 0, st>>>(src, cams)));
        }
        LayerTable lt = base;
        for (int l = 0; l < L; ++l)
        {
            size_t plane = (size_t)base.w[l] * base.h[l];
            lt.depth[l] = io->layers[l].depth + (size_t)b * plane;
            lt.weight[l] = io->layers[l].weight + (size_t)b * plane;
            lt.color[l] = io->layers[l].color + (size_t)b * C * plane;
            lt.mask[l] = (rp->output_background_mask && io->layers[l].mask) ? io->layers[l].mask + (size_t)b * plane : nullptr;
        }
        KernelParams kp = make_kernel_params(rp, io->dropout_mask, N, b);
        const ViewCam* cam = cams + (b % kCamChunk);
        if (packed)
        {
            PackedPlanes pp;
            for (int l = 0; l < kMaxLayers; ++l)
                pp.plane[l] = l < L ? reinterpret_cast<unsigned long long*>(io->packed_depth[l]) + (size_t)b * base.w[l] * base.h[l] : nullptr;
            static const int g_packed = resident_grid(k_depth_prepass_packed, 1ll << 40);
            const int need = (N + kBlock - 1) / kBlock;
            ADOP_LAUNCH("k_depth_prepass_packed", st, (k_depth_prepass_packed<<<need < g_packed ? (need < 1 ? 1 : need) : g_packed, kBlock, 0, st>>>(
                                                          pts, cam, kp, lt, pp)));
        }
        // depth prepass in groups of four consecutive views (a group never straddles a camera chunk: 64 = 16 x 4)
        const int depth_views = (b % 4 == 0) ? (B - b < 4 ? B - b : 4) : 0;
        adop_status r;
        switch (C)
        {
            case 3: r = dispatch_layers_forward<3>(L, pts, s, cam, kp, lt, plan, st, b, depth_views); break;
            case 4: r = dispatch_layers_forward<4>(L, pts, s, cam, kp, lt, plan, st, b, depth_views); break;
            case 8: r = dispatch_layers_forward<8>(L, pts, s, cam, kp, lt, plan, st, b, depth_views); break;
            case 16: r = dispatch_layers_forward<16>(L, pts, s, cam, kp, lt, plan, st, b, depth_views); break;
            default:
                snprintf(last_error_buffer(), 512, "%d descriptor channels: the kernels are built for 3, 4, 8 and 16", C);
                return ADOP_ERR_UNSUPPORTED;
        }
        if (r != ADOP_OK) return r;
    }
    return ADOP_OK;
}
