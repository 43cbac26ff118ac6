// Forward pass of the one-pixel point rasterizer for sm_100a: depth prepass, fuzzy-depth blend, resolve.
// Stands in for BlendPointCloudForward and its kernels (darglein/ADOP src/lib/rendering/PointRenderer.cu:
// DepthPrepassMulti :203-301, RenderForwardMulti :303-393, CombineAndFill :726-754, CreateMask :828-847)
// plus the environment-map composite of RenderModule.cpp:106-127 / EnvironmentMap.cu:62-156.
//
// Layout choices (none of these kernels is a dense contraction, so no tensor cores):
//  * points stream as one 128-bit load per thread; normals / indices are separate 4-byte streams;
//  * descriptor sums go to a pixel-interleaved accumulator record (C sums + weight, padded to 16-byte
//    vectors) so that one splat is one vector atomic plus one scalar atomic into the same 32-byte sector,
//    instead of C+1 atomics into C+1 planes;
//  * the resolve kernel turns records into the NCHW tensors of the operator's interface in a single pass
//    (normalise, background, environment map, mask, weight plane) and clears the records it read, so the
//    one accumulator, small enough to stay in the 126 MB L2, is reused by every view of the batch.
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
template <int L, bool PLAIN, int V>
__global__ void __launch_bounds__(kBlock, 8) k_depth_prepass(PointStreams pts, const ViewCam* __restrict__ camp, KernelParams kp, LayerTable lt)
{
    const bool use_normal = PLAIN ? false : kp.check_normal != 0;
    const bool use_radius = PLAIN ? false : kp.drop_out_points_by_radius != 0;
    const int stride = gridDim.x * blockDim.x;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < pts.n; i += stride)
    {
        FetchedPoint f;
        if (PLAIN) { float4 c = __ldg(pts.position + i); f.p.x = c.x; f.p.y = c.y; f.p.z = c.z; f.r = c.w; f.has_normal = false; f.n.x = f.n.y = f.n.z = 0.f; }
        else f = fetch_point(pts, i);
#pragma unroll
        for (int v = 0; v < V; ++v)
        {
            RasterPoint q;
            if (PLAIN ? !project_plain(camp[v], f.p, kp.dist_cutoff, &q)
                      : !project_for_raster(camp[v], f.p, f.r, f.n, f.has_normal, use_normal, kp.dist_cutoff, &q, use_radius)) continue;
            float x = q.x, y = q.y, rad = q.radius_px;
            const int zi = __float_as_int(q.z);
#pragma unroll
            for (int l = 0; l < L; ++l, rad *= 0.5f, x *= 0.5f, y *= 0.5f)
            {
                if (use_radius && rad < kp.drop_out_radius_threshold) break;
                int px = round_half_even_bounded(x), py = round_half_even_bounded(y);
                if ((unsigned)px >= (unsigned)lt.w[l] || (unsigned)py >= (unsigned)lt.h[l]) continue;
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

// With EMIT the kernel also appends the (point, layer) splats that the backward pass will visit to this block's segment
// of the view's splat list (shared-memory counter, no global atomics); in ghost-gradient mode dropped points are tested
// too (they blend nothing but the backward pass needs them, PointRenderer.cu:487-488).
template <int L, int C, bool EMIT, bool PLAIN>
__global__ void __launch_bounds__(kBlock, 8) k_blend(PointStreams pts, const float* __restrict__ texture,
                                                   const float* __restrict__ texture_interleaved, int num_texels,
                                                   const ViewCam* __restrict__ camp, KernelParams kp, LayerTable lt,
                                                   float* __restrict__ accum, VisibleList vl)
{
    const ViewCam& cam = *camp;
    const bool use_normal = PLAIN ? false : kp.check_normal != 0;
    const bool use_radius = PLAIN ? false : kp.drop_out_points_by_radius != 0;
    __shared__ int s_count;
    if (EMIT)
    {
        if (threadIdx.x == 0) s_count = 0;
        __syncthreads();
    }
    constexpr int RS = AccumLayout<C>::kFloats;
    const int stride = gridDim.x * blockDim.x;
    int4* seg = EMIT ? vl.entries + (size_t)blockIdx.x * vl.seg_cap : nullptr;
    const int lane = threadIdx.x & 31;
    // Only about a third of the lanes of a warp that has accepted points at all have one (11 of 32 on the 1080p
    // benchmark scene), so the work on accepted points - descriptor load, atomics, the list entries - is not done where the
    // point is tested: a warp parks its accepted points (index, layer mask, pixel per layer) in a queue of its own in
    // shared memory and finishes them 32 at a time with every lane busy.
    constexpr int PW = L + 2;
    __shared__ int s_park[kBlock / 32][64 * PW];
    int* park = s_park[threadIdx.x >> 5];
    int n_parked = 0;  // the same in every lane of the warp

    // Tests one point against the depth buffers: 0 = nothing to do, else the mask of accepted layers, bit 31 = the point
    // is dropped in this view (it blends nothing but the backward pass visits it in ghost-gradient mode).
    auto test_point = [&](int i, float4 cur, int* pix) -> unsigned
    {
        const bool dropped = point_dropped(kp, i);
        if (dropped && !(EMIT && kp.ghost_gradients)) return 0u;
        FetchedPoint f;
        if (PLAIN) { f.p.x = cur.x; f.p.y = cur.y; f.p.z = cur.z; f.r = cur.w; f.has_normal = false; f.n.x = f.n.y = f.n.z = 0.f; }
        else f = fetch_point(pts, i, cur);
        RasterPoint q;
        if (PLAIN ? !project_plain(cam, f.p, kp.dist_cutoff, &q)
                  : !project_for_raster(cam, f.p, f.r, f.n, f.has_normal, use_normal, kp.dist_cutoff, &q, use_radius)) return 0u;
        float x = q.x, y = q.y, rad = q.radius_px;
        // pixel index inside the layer (a pyramid has fewer than 2^31 pixels), -1 = not in this layer; the depth reads
        // of all layers go out together
        bool live = true;
#pragma unroll
        for (int l = 0; l < L; ++l, rad *= 0.5f, x *= 0.5f, y *= 0.5f)
        {
            if (use_radius && rad < kp.drop_out_radius_threshold) live = false;  // break, :368-371
            int px = round_half_even_bounded(x), py = round_half_even_bounded(y);
            bool in = live && (unsigned)px < (unsigned)lt.w[l] && (unsigned)py < (unsigned)lt.h[l];
            pix[l] = in ? py * lt.w[l] + px : -1;
        }
        unsigned pass = 0;
#pragma unroll
        for (int l = 0; l < L; ++l)
        {
            float image_depth = pix[l] >= 0 ? __ldg(lt.depth[l] + pix[l]) : 0.f;
            if (pix[l] >= 0 && !(q.z > image_depth * kp.depth_accept_plus_one)) pass |= 1u << l;
        }
        if (pass == 0) return 0u;
        return pass | (dropped ? 0x80000000u : 0u);
    };

    // All 32 lanes together: blend the accepted point of every valid lane and append its splats to the list.
    auto finish = [&](bool valid, const int* e)
    {
        unsigned bmask = 0;
        int i = 0;
        int pix[L];
#pragma unroll
        for (int l = 0; l < L; ++l) pix[l] = -1;
        if (valid)
        {
            i = e[0];
            const unsigned code = (unsigned)e[1];
#pragma unroll
            for (int l = 0; l < L; ++l) pix[l] = e[2 + l];
            if (!(code >> 31))
            {
                float t[C];
                const int ti = pts.index ? __ldg(pts.index + i) : i;
                load_descriptor<C>(texture, texture_interleaved, num_texels, ti, t);
#pragma unroll
                for (int l = 0; l < L; ++l)
                    if (code & (1u << l)) splat_record<C>(accum + ((size_t)lt.rec_off[l] + pix[l]) * RS, lt.weight[l] + pix[l], t);
            }
            // the layers the backward pass will visit: it skips layers the point does not land in and stops at the
            // first depth failure (PointRenderer.cu:451-462)
#pragma unroll
            for (int l = 0; l < L; ++l)
            {
                if (pix[l] < 0) continue;
                if (!(code & (1u << l))) break;
                bmask |= 1u << l;
            }
        }
        if (EMIT)
        {
            const int cnt = __popc(bmask);
            int incl = cnt;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1)
            {
                int v = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += v;
            }
            const int total = __shfl_sync(0xffffffffu, incl, 31);
            if (total > 0)
            {
                // one shared-memory atomic per warp reserves room in this block's segment of the splat list
                int wbase = 0;
                if (lane == 0) wbase = atomicAdd(&s_count, total);
                wbase = __shfl_sync(0xffffffffu, wbase, 0);
                int at = wbase + incl - cnt;
                if (wbase + total <= vl.seg_cap)
                {
#pragma unroll
                    for (int l = 0; l < L; ++l)
                        if (bmask & (1u << l)) seg[at++] = make_int4(i | (l << kSplatLayerShift), pix[l], 0, 0);
                }
                else if (lane == 0)
                    vl.header[kVisibleSegments + 2] = 1;  // out of room: the backward pass falls back to walking all points
            }
        }
    };

    // warp-uniform trip count: parking and finishing use full-warp votes and shuffles
    for (int base = blockIdx.x * blockDim.x; base < pts.n; base += stride)
    {
        const int i = base + threadIdx.x;
        unsigned code = 0;
        int pix[L];
        if (i < pts.n) code = test_point(i, __ldg(pts.position + i), pix);
        const unsigned vote = __ballot_sync(0xffffffffu, code != 0);
        if (vote)
        {
            if (code)
            {
                int* e = park + (n_parked + __popc(vote & ((1u << lane) - 1u))) * PW;
                e[0] = i;
                e[1] = (int)code;
#pragma unroll
                for (int l = 0; l < L; ++l) e[2 + l] = pix[l];
            }
            n_parked += __popc(vote);
            __syncwarp();
            if (n_parked >= 32)
            {
                n_parked -= 32;
                finish(true, park + (n_parked + lane) * PW);
            }
            __syncwarp();
        }
    }
    if (n_parked > 0) finish(lane < n_parked, park + lane * PW);
    if (EMIT)
    {
        __syncthreads();
        if (threadIdx.x == 0)
        {
            vl.header[blockIdx.x] = s_count < vl.seg_cap ? s_count : vl.seg_cap;
            if (blockIdx.x == 0) { vl.header[kVisibleSegments] = vl.segments; vl.header[kVisibleSegments + 1] = vl.seg_cap; }
        }
    }
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
__global__ void __launch_bounds__(kBlock) k_resolve(LayerTable lt, const ViewCam* __restrict__ camp, KernelParams kp, float* __restrict__ accum,
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
#pragma unroll
                for (int c = 0; c < C; ++c) color[c * plane] = v[c] / cou;
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
template <int L, int C, bool PLAIN>
static adop_status launch_view_forward_impl(const PointStreams& pts, const adop_scene* s, const ViewCam* cam, const KernelParams& kp,
                                            const LayerTable& lt, float* accum, bool env, cudaStream_t st, int32_t* list_base, int view,
                                            int depth_views)
{
    static const int g_depth = resident_grid(k_depth_prepass<L, PLAIN, 4>, 1ll << 40);
    static const int g_blend_plain = resident_grid(k_blend<L, C, false, PLAIN>, 1ll << 40);
    static const int g_blend_emit = resident_grid(k_blend<L, C, true, PLAIN>, 1ll << 40);
    static const int g_resolve = resident_grid(k_resolve<C>, 1ll << 40);
    const int g_blend = list_base ? (g_blend_emit < kVisibleSegments ? g_blend_emit : kVisibleSegments) : g_blend_plain;
    const int need = (pts.n + kBlock - 1) / kBlock;
    // the depth prepass of this view was done by the launch of its group's first view, unless this is that view
    const int grid_depth = need < g_depth ? (need < 1 ? 1 : need) : g_depth;
    switch (depth_views)
    {
        case 1: ADOP_LAUNCH("k_depth_prepass", st, (k_depth_prepass<L, PLAIN, 1><<<grid_depth, kBlock, 0, st>>>(pts, cam, kp, lt))); break;
        case 2: ADOP_LAUNCH("k_depth_prepass", st, (k_depth_prepass<L, PLAIN, 2><<<grid_depth, kBlock, 0, st>>>(pts, cam, kp, lt))); break;
        case 3: ADOP_LAUNCH("k_depth_prepass", st, (k_depth_prepass<L, PLAIN, 3><<<grid_depth, kBlock, 0, st>>>(pts, cam, kp, lt))); break;
        case 4: ADOP_LAUNCH("k_depth_prepass", st, (k_depth_prepass<L, PLAIN, 4><<<grid_depth, kBlock, 0, st>>>(pts, cam, kp, lt))); break;
        default: break;
    }
    int grid_blend = need < g_blend ? (need < 1 ? 1 : need) : g_blend;
    if (list_base)
    {
        // a block's list segment holds as many entries as the block has points; visible splats come in clumps (a chunk of
        // neighbouring points on a front surface is accepted on every layer), so every block should average over at
        // least 16 chunks from all over the cloud
        int cap = need / 16;
        if (cap < 1) cap = 1;
        if (grid_blend > cap) grid_blend = cap;
    }
    VisibleList vl = make_visible_list(list_base, pts.n, view, grid_blend);
    if (list_base && pts.n >= kSplatMaxPoints)
    {
        // too many points for the 28-bit ids of the list: mark it unusable and blend without recording
        ADOP_CUDA_TRY(cudaMemsetAsync(vl.header, 0, sizeof(int) * kVisibleHeaderInts, st));
        ADOP_CUDA_TRY(cudaMemsetAsync(vl.header + kVisibleSegments + 2, 1, sizeof(int), st));
        ADOP_LAUNCH("k_blend", st, (k_blend<L, C, false, PLAIN><<<grid_blend, kBlock, 0, st>>>(pts, s->texture, s->texture_interleaved, s->num_texels, cam, kp, lt, accum, vl)));
    }
    else if (list_base)
    {
        ADOP_CUDA_TRY(cudaMemsetAsync(vl.header, 0, sizeof(int) * kVisibleHeaderInts, st));
        ADOP_LAUNCH("k_blend", st, (k_blend<L, C, true, PLAIN><<<grid_blend, kBlock, 0, st>>>(pts, s->texture, s->texture_interleaved, s->num_texels, cam, kp, lt, accum, vl)));
    }
    else
        ADOP_LAUNCH("k_blend", st, (k_blend<L, C, false, PLAIN><<<grid_blend, kBlock, 0, st>>>(pts, s->texture, s->texture_interleaved, s->num_texels, cam, kp, lt, accum, vl)));
    unsigned total = lt.rec_off[kMaxLayers];
    int grid_px = (int)((total + kBlock - 1) / kBlock);
    if (grid_px > g_resolve) grid_px = g_resolve;
    ADOP_LAUNCH("k_resolve", st, (k_resolve<C><<<grid_px, kBlock, 0, st>>>(lt, cam, kp, accum, s->background,
                                                                          env ? s->env_map : nullptr, s->env_h, s->env_w)));
    ADOP_CUDA_TRY(cudaGetLastError());
    return ADOP_OK;
}

template <int L, int C>
static adop_status launch_view_forward(const PointStreams& pts, const adop_scene* s, const ViewCam* cam, const KernelParams& kp,
                                       const LayerTable& lt, float* accum, bool env, cudaStream_t st, int32_t* list_base, int view,
                                       int depth_views)
{
    // the common case - no normal test (or no normals) and no radius drop-out - gets kernels without that code
    const bool plain = !(kp.check_normal && pts.normal) && !kp.drop_out_points_by_radius;
    return plain ? launch_view_forward_impl<L, C, true>(pts, s, cam, kp, lt, accum, env, st, list_base, view, depth_views)
                 : launch_view_forward_impl<L, C, false>(pts, s, cam, kp, lt, accum, env, st, list_base, view, depth_views);
}

template <int C>
static adop_status dispatch_layers_forward(int L, const PointStreams& pts, const adop_scene* s, const ViewCam* cam,
                                           const KernelParams& kp, const LayerTable& lt, float* accum, bool env,
                                           cudaStream_t st, int32_t* list_base, int view, int depth_views)
{
    switch (L)
    {
        case 1: return launch_view_forward<1, C>(pts, s, cam, kp, lt, accum, env, st, list_base, view, depth_views);
        case 2: return launch_view_forward<2, C>(pts, s, cam, kp, lt, accum, env, st, list_base, view, depth_views);
        case 3: return launch_view_forward<3, C>(pts, s, cam, kp, lt, accum, env, st, list_base, view, depth_views);
        case 4: return launch_view_forward<4, C>(pts, s, cam, kp, lt, accum, env, st, list_base, view, depth_views);
        case 5: return launch_view_forward<5, C>(pts, s, cam, kp, lt, accum, env, st, list_base, view, depth_views);
        case 6: return launch_view_forward<6, C>(pts, s, cam, kp, lt, accum, env, st, list_base, view, depth_views);
        case 7: return launch_view_forward<7, C>(pts, s, cam, kp, lt, accum, env, st, list_base, view, depth_views);
        case 8: return launch_view_forward<8, C>(pts, s, cam, kp, lt, accum, env, st, list_base, view, depth_views);
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

extern "C" size_t adop_raster_visible_list_ints(int32_t num_points)
{
    return num_points < 0 ? 0 : visible_list_ints(num_points);
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
            case 3: r = dispatch_layers_forward<3>(L, pts, s, cam, kp, lt, accum, env, st, io->visible_list, b, depth_views); break;
            case 4: r = dispatch_layers_forward<4>(L, pts, s, cam, kp, lt, accum, env, st, io->visible_list, b, depth_views); break;
            case 8: r = dispatch_layers_forward<8>(L, pts, s, cam, kp, lt, accum, env, st, io->visible_list, b, depth_views); break;
            case 16: r = dispatch_layers_forward<16>(L, pts, s, cam, kp, lt, accum, env, st, io->visible_list, b, depth_views); break;
            default: return ADOP_ERR_UNSUPPORTED;
        }
        if (r != ADOP_OK) return r;
    }
    return ADOP_OK;
}
