// Backward pass of the one-pixel point rasterizer for sm_100a.
// Stands in for BlendPointCloudBackward and its kernels (darglein/ADOP src/lib/rendering/PointRenderer.cu:
// CombineAndFillBackward :851-900, RenderBackward :396-724, NormalizeGradient :1534-1547) and the gradient
// of the environment-map composite (RenderModule.cpp:121-125, grid_sample backward).
//
// Differences in how the same sums are formed (results agree within float-ordering tolerance):
//  * the forward pass lists, per 32 x 16 screen tile, the points that were accepted on some layer; the backward pass runs
//    one block per tile over that list, with the tile's region of every layer (weight, forward image, upstream gradient)
//    staged in shared memory, instead of one thread per point of the cloud reading scattered pixels (kernels with the
//    reference's structure stay behind it for calls without a usable list);
//  * a point's descriptor gradient is summed over its layers and leaves as one vector atomic; its image-space ghost
//    gradient is summed over its layers too (scaled by 0.5^layer), so the projection chain runs once per visible point;
//  * the point gradient and its counter leave as ONE 16-byte vector atomic (x, y, z, count);
//  * pose and intrinsics gradients, which the reference adds with 7 + 14 same-address atomics per splat,
//    are reduced warp -> block in shared memory and leave as one atomic per component and block;
//  * the all-points kernels read the ghost stencil from one interleaved record per pixel [I_0..I_C-1, G_0..G_C-1] that a
//    preparation pass builds (a neighbour then costs one or two 32-byte sectors instead of 2C).
#include "common.cuh"

namespace adop {

// ------------------------------------------------------------------------------------------------------
// K4: preparation pass over the pyramid pixels of one view (all-points path only; returns at once behind a usable list).
//  * writes the interleaved record [I_0..I_C-1 | G_0..G_C-1] (I = the forward image before the environment-map
//    composite: the background colour where nothing was blended, PointRenderer.cu:1523);
//  * sums the gradient of the background colour over uncovered pixels (CombineAndFillBackward, :851-900);
//  * with the fused composite, scatters the environment-map gradient (bilinear, 4 taps).
__host__ __device__ inline int backward_record_floats(int C) { return (2 * C + 3) & ~3; }

// The environment-map gradient of an uncovered pixel (bilinear scatter, 4 taps): as in the forward resolve kernel the
// uncovered pixels are scattered single-pixel holes, so each warp parks them and works them off 32 at a time.
template <int C>
__device__ __forceinline__ void scatter_environment_gradient(const LayerTable& lt, const ViewCam& cam, const KernelParams& kp, unsigned r,
                                                             float* __restrict__ grad_env, int env_h, int env_w, bool interleaved)
{
    const int l = layer_of_record(lt, r);
    const unsigned pix = r - lt.rec_off[l];
    const int w = lt.w[l];
    const size_t plane = (size_t)w * lt.h[l];
    const int gy = pix / w, gx = pix - gy * w;
    float gup[C];
#pragma unroll
    for (int c = 0; c < C; ++c) gup[c] = __ldg(lt.grad[l] + c * plane + pix);
    Intr5 crop_l = scale_intr(cam.crop, __int_as_float((127 - l) << 23));
    V2 uv = env_uv_for_pixel(gx, gy, cam.V, cam.K, cam.dist, crop_l);
    BilinearTap tp = bilinear_taps(uv, env_w, env_h);
    const float om = 1.0f - kp.mask_background_value;
    const float w00 = (1.0f - tp.wx) * (1.0f - tp.wy), w01 = tp.wx * (1.0f - tp.wy);
    const float w10 = (1.0f - tp.wx) * tp.wy, w11 = tp.wx * tp.wy;
    if (interleaved && C % 4 == 0)
    {
        // [eh,ew,C] scratch: one vector atomic per tap and four channels instead of one per channel
        float4* e = reinterpret_cast<float4*>(grad_env);
        const size_t t00 = ((size_t)tp.y0 * env_w + tp.x0) * (C / 4), t01 = ((size_t)tp.y0 * env_w + tp.x1) * (C / 4);
        const size_t t10 = ((size_t)tp.y1 * env_w + tp.x0) * (C / 4), t11 = ((size_t)tp.y1 * env_w + tp.x1) * (C / 4);
#pragma unroll
        for (int k = 0; k < C / 4; ++k)
        {
            const float a = om * gup[4 * k], b = om * gup[4 * k + 1], c2 = om * gup[4 * k + 2], d = om * gup[4 * k + 3];
            atomicAdd(e + t00 + k, make_float4(a * w00, b * w00, c2 * w00, d * w00));
            atomicAdd(e + t01 + k, make_float4(a * w01, b * w01, c2 * w01, d * w01));
            atomicAdd(e + t10 + k, make_float4(a * w10, b * w10, c2 * w10, d * w10));
            atomicAdd(e + t11 + k, make_float4(a * w11, b * w11, c2 * w11, d * w11));
        }
        return;
    }
#pragma unroll
    for (int c = 0; c < C; ++c)
    {
        float* e = grad_env + (size_t)c * env_h * env_w;
        float ge = om * gup[c];
        atomicAdd(e + (size_t)tp.y0 * env_w + tp.x0, ge * w00);
        atomicAdd(e + (size_t)tp.y0 * env_w + tp.x1, ge * w01);
        atomicAdd(e + (size_t)tp.y1 * env_w + tp.x0, ge * w10);
        atomicAdd(e + (size_t)tp.y1 * env_w + tp.x1, ge * w11);
    }
}

template <int C>
__global__ void __launch_bounds__(kBlock) k_prepare_backward(LayerTable lt, const ViewCam* __restrict__ camp, KernelParams kp,
                                                              const float* __restrict__ background, float* __restrict__ records,
                                                              float* __restrict__ grad_background,
                                                              float* __restrict__ grad_env, int env_h, int env_w, bool env_interleaved,
                                                              const int* __restrict__ skip_if_nonzero)
{
    constexpr int RB = (2 * C + 3) & ~3;
    if (skip_if_nonzero && __ldg(skip_if_nonzero) != 0) return;  // this pass runs on the visible list: nothing to prepare
    const ViewCam& cam = *camp;
    __shared__ float s_bg[C];
    __shared__ unsigned s_parked[kBlock / 32][64];
    unsigned* parked = s_parked[threadIdx.x >> 5];
    const int lane = threadIdx.x & 31;
    int n_parked = 0;  // the same in every lane of the warp
    if (threadIdx.x < C) s_bg[threadIdx.x] = 0.f;
    __syncthreads();
    const unsigned total = lt.rec_off[kMaxLayers];
    const unsigned stride = gridDim.x * blockDim.x;
    float g[C], bgc[C];
#pragma unroll
    for (int c = 0; c < C; ++c) { g[c] = 0.f; bgc[c] = __ldg(background + c); }
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
            // every load of the pixel is requested before the coverage is known
            const float wgt = __ldg(lt.weight[l] + pix);
            float rec[RB];
#pragma unroll
            for (int c = 0; c < C; ++c)
            {
                rec[C + c] = __ldcs(lt.grad[l] + c * plane + pix);
                rec[c] = __ldg(lt.color[l] + c * plane + pix);
            }
            const bool covered = wgt != 0.f;
            if (!covered)
            {
                // the image before the environment map was added (PointRenderer.cu:1523)
#pragma unroll
                for (int c = 0; c < C; ++c) rec[c] = bgc[c];
            }
#pragma unroll
            for (int k = 2 * C; k < RB; ++k) rec[k] = 0.f;
            float4* dst = reinterpret_cast<float4*>(records + (size_t)r * RB);
#pragma unroll
            for (int k = 0; k < RB / 4; ++k) dst[k] = make_float4(rec[4 * k], rec[4 * k + 1], rec[4 * k + 2], rec[4 * k + 3]);
            if (!covered)
            {
#pragma unroll
                for (int c = 0; c < C; ++c) g[c] += rec[C + c];
                hole = grad_env != nullptr;
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
                scatter_environment_gradient<C>(lt, cam, kp, parked[n_parked + lane], grad_env, env_h, env_w, env_interleaved);
            }
            __syncwarp();
        }
    }
    if (lane < n_parked) scatter_environment_gradient<C>(lt, cam, kp, parked[lane], grad_env, env_h, env_w, env_interleaved);
    if (grad_background)
    {
#pragma unroll
        for (int c = 0; c < C; ++c)
        {
            float v = warp_sum(g[c]);
            if ((threadIdx.x & 31) == 0 && v != 0.f) atomicAdd(&s_bg[c], v);
        }
        __syncthreads();
        if (threadIdx.x < C && s_bg[threadIdx.x] != 0.f) atomicAdd(grad_background + threadIdx.x, s_bg[threadIdx.x]);
    }
}

// ------------------------------------------------------------------------------------------------------
// K5: gradients of the splats.
struct BackwardTargets
{
    const float* texture;
    const float* texture_interleaved;  // optional [T,C]
    int num_texels;
    const float* background;
    float* grad_texture;
    float* grad_texture_interleaved;   // optional [T,C]; when set the descriptor gradient goes there
    float4* grad_points;
    double* grad_pose;        // row of this view's image, 6 doubles
    float* count_pose;        // element of this view's image
    float* grad_intrinsics;   // row of this view's camera
    float* count_intrinsics;  // element of this view's camera
    const float* records;     // interleaved [I | G] per pyramid pixel, written by k_prepare_backward
};

template <int C>
__device__ __forceinline__ void load_record(const float* records, size_t r, float* out)
{
    constexpr int RB = (2 * C + 3) & ~3;
    const float4* src = reinterpret_cast<const float4*>(records + r * RB);
#pragma unroll
    for (int k = 0; k < RB / 4; ++k)
    {
        float4 a = __ldg(src + k);
        out[4 * k] = a.x; out[4 * k + 1] = a.y; out[4 * k + 2] = a.z; out[4 * k + 3] = a.w;
    }
}

// per-thread partial sums of the view's pose / intrinsics gradient
template <int MODEL>
struct GeoAccum
{
    static constexpr int NI = MODEL == kPinholeDistortion ? 13 : 5;
    float pose[6];
    float intr[NI];
    float cnt;
    __device__ __forceinline__ void clear()
    {
#pragma unroll
        for (int k = 0; k < 6; ++k) pose[k] = 0.f;
#pragma unroll
        for (int k = 0; k < NI; ++k) intr[k] = 0.f;
        cnt = 0.f;
    }
};

// The ghost-geometry image gradient of one splat (PointRenderer.cu:522-611): central differences over the four
// neighbours of (T_p - I_x) * G_x, averaged over the channels. rn[k] = record of neighbour k (left, right, up, down).
template <int C>
__device__ __forceinline__ V2 stencil_gradient(const KernelParams& kp, const float* T_p, const float (*rn)[(2 * C + 3) & ~3],
                                               float z, const float* __restrict__ W, const float* __restrict__ D, const size_t* nb)
{
    float dR[4];
#pragma unroll
    for (int k = 0; k < 4; ++k)
    {
        float acc = 0.f;
        if (kp.test_backward_mode == 4)  // PointRenderer.cu:543-566
        {
            const float W_x = __ldg(W + nb[k]), D_x = __ldg(D + nb[k]);
#pragma unroll
            for (int c = 0; c < C; ++c)
            {
                float dI;
                if (W_x == 0.f || z * kp.depth_accept_plus_one < D_x) dI = T_p[c] - rn[k][c];
                else if (z > D_x * kp.depth_accept_plus_one) dI = 0.f;
                else dI = (W_x / (W_x + 1.f) * rn[k][c] + 1.f / (W_x + 1.f) * T_p[c] - rn[k][c]);
                acc += dI * rn[k][C + c];
            }
        }
        else
        {
#pragma unroll
            for (int c = 0; c < C; ++c) acc += (T_p[c] - rn[k][c]) * rn[k][C + c];
        }
        dR[k] = acc;
    }
    V2 g;
    g.x = 0.5f * (-dR[0] + dR[1]) / (float)C;
    g.y = 0.5f * (-dR[2] + dR[3]) / (float)C;
    return g;
}

// Chain the image gradient through the projection (PointRenderer.cu:613-720) and add to the partial sums.
// Returns false when the chain rejects the point; gp = (x, y, z, count) partial sum of the point gradient.
template <int MODEL>
__device__ __forceinline__ bool chain_gradient(const ViewCam& cam, const KernelParams& kp, const FetchedPoint& f, V2 g,
                                               float scale, float* gp, GeoAccum<MODEL>& acc)
{
    Intr5 crop_l = scale_intr(cam.crop, scale);
    if (MODEL == kPinholeDistortion)
    {
        GradPinhole o;
        if (!project_pinhole_backward(f.p, f.n, f.has_normal, g, cam.V, cam.K, crop_l, cam.dist, kp.check_normal != 0,
                                      kp.dist_cutoff, &o))
            return false;
        gp[0] += o.g_point[0]; gp[1] += o.g_point[1]; gp[2] += o.g_point[2]; gp[3] += 1.f;
#pragma unroll
        for (int k = 0; k < 6; ++k) acc.pose[k] += o.g_pose[k];
        // damping of PointRenderer.cu:647-678 (skew gets no gradient)
        const float kf = kp.K_gradient_factor, df = kp.distortion_gradient_factor;
        acc.intr[0] += kf * o.g_k[0]; acc.intr[1] += kf * o.g_k[1]; acc.intr[2] += kf * o.g_k[2]; acc.intr[3] += kf * o.g_k[3];
        acc.intr[5] += df * o.g_dis[0]; acc.intr[6] += df * o.g_dis[1];
        acc.intr[7] += df * (o.g_dis[2] * 0.25f);
        acc.intr[8] += df * (o.g_dis[3] * 0.1f); acc.intr[9] += df * (o.g_dis[4] * 0.1f); acc.intr[10] += df * (o.g_dis[5] * 0.1f);
        acc.intr[11] += df * (o.g_dis[6] * 0.1f); acc.intr[12] += df * (o.g_dis[7] * 0.1f);
    }
    else
    {
        GradOcam o;
        if (!project_ocam_backward(f.p, f.n, f.has_normal, g, cam.V, crop_l, cam.ocam, kp.check_normal != 0, kp.dist_cutoff, &o))
            return false;
        gp[0] += o.g_point[0]; gp[1] += o.g_point[1]; gp[2] += o.g_point[2]; gp[3] += 1.f;
#pragma unroll
        for (int k = 0; k < 6; ++k) acc.pose[k] += o.g_pose[k];
#pragma unroll
        for (int k = 0; k < 5; ++k) acc.intr[k] += o.g_affine[k];
    }
    acc.cnt += 1.f;
    return true;
}

// Block reduction of the per-view pose / intrinsics sums: warp shuffle, shared memory (double for the pose, which the
// reference accumulates in double, :1113), then one global atomic per component and block.
template <int MODEL>
struct GeoShared
{
    double pose[6];
    float intr[GeoAccum<MODEL>::NI];
    float cnt;
    int any;
};
template <int MODEL>
__device__ __forceinline__ void geo_shared_init(GeoShared<MODEL>* s)
{
    if (threadIdx.x < 6) s->pose[threadIdx.x] = 0.0;
    if (threadIdx.x < GeoAccum<MODEL>::NI) s->intr[threadIdx.x] = 0.f;
    if (threadIdx.x == 0) { s->cnt = 0.f; s->any = 0; }
}
// every thread of the block must call this
template <int MODEL>
__device__ __forceinline__ void geo_block_reduce(GeoShared<MODEL>* s, const GeoAccum<MODEL>& acc, const BackwardTargets& bt)
{
    constexpr int NI = GeoAccum<MODEL>::NI;
    if (!(bt.grad_pose || bt.grad_intrinsics)) return;
    const unsigned any = __ballot_sync(0xffffffffu, acc.cnt > 0.f);
    if (any)
    {
        const bool lane0 = (threadIdx.x & 31) == 0;
        if (bt.grad_pose)
        {
#pragma unroll
            for (int k = 0; k < 6; ++k)
            {
                float v = warp_sum(acc.pose[k]);
                if (lane0) atomicAdd(&s->pose[k], (double)v);
            }
        }
        if (bt.grad_intrinsics)
        {
#pragma unroll
            for (int k = 0; k < NI; ++k)
            {
                float v = warp_sum(acc.intr[k]);
                if (lane0) atomicAdd(&s->intr[k], v);
            }
        }
        float c = warp_sum(acc.cnt);
        if (lane0) { atomicAdd(&s->cnt, c); s->any = 1; }
    }
    __syncthreads();
    if (!s->any) return;
    if (bt.grad_pose)
    {
        if (threadIdx.x < 6) atomicAdd(bt.grad_pose + threadIdx.x, s->pose[threadIdx.x]);
        if (threadIdx.x == 6) atomicAdd(bt.count_pose, s->cnt);
    }
    if (bt.grad_intrinsics)
    {
        if (threadIdx.x >= 32 && threadIdx.x < 32 + NI) atomicAdd(bt.grad_intrinsics + (threadIdx.x - 32), s->intr[threadIdx.x - 32]);
        // the reference counts 1/1024 per pinhole contribution and 1 per OCam contribution (:680-681, :718)
        if (threadIdx.x == 64) atomicAdd(bt.count_intrinsics, MODEL == kPinholeDistortion ? s->cnt * (1.f / 1024.f) : s->cnt);
    }
}

// K5 (all points): the reference's structure, one thread per point walking its layers (RenderBackward, :396-724). Used
// when the forward pass recorded no visible list (or a tile's bucket overflowed, or the list was used before).
template <int C, int MODEL>
__global__ void __launch_bounds__(kBlock) k_splat_backward_all(PointStreams pts, const ViewCam* __restrict__ camp, KernelParams kp, LayerTable lt,
                                                                BackwardTargets bt, int* __restrict__ list_header, int mark_consumed)
{
    constexpr int RB = (2 * C + 3) & ~3;
    // Behind a visible list (last kernel of the pass): if the pass ran on the list there is nothing left to do but to mark
    // the list consumed when its entries were turned into work items.
    if (list_header && __ldg(list_header + kListGo) != 0)
    {
        if (mark_consumed && blockIdx.x == 0 && threadIdx.x == 0) list_header[kListConsumed] = 1;
        return;
    }
    const ViewCam& cam = *camp;
    __shared__ GeoShared<MODEL> s_geo;
    geo_shared_init(&s_geo);
    __syncthreads();
    const bool want_geo = bt.grad_points || bt.grad_pose || bt.grad_intrinsics;
    GeoAccum<MODEL> acc;
    acc.clear();
    const int stride = gridDim.x * blockDim.x;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < pts.n; i += stride)
    {
        const bool drop_out = point_dropped(kp, i);
        FetchedPoint f = fetch_point(pts, i);
        RasterPoint q;
        if (!project_for_raster(cam, f.p, f.r, f.n, f.has_normal, kp.check_normal != 0, kp.dist_cutoff, &q,
                                kp.drop_out_points_by_radius != 0)) continue;
        float x = q.x, y = q.y, rad = q.radius_px, scale = 1.f;
        const bool point_grad = want_geo && ((kp.ghost_gradients && drop_out) || (!kp.ghost_gradients && !drop_out));
        int ti = -1;
        float T_p[C], dg[C];
        bool have_t = false, have_dg = false;
        float gp[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int c = 0; c < C; ++c) dg[c] = 0.f;
#pragma unroll 1
        for (int l = 0; l < lt.L; ++l, scale *= 0.5f, rad *= 0.5f, x *= 0.5f, y *= 0.5f)
        {
            if (kp.drop_out_points_by_radius && rad < kp.drop_out_radius_threshold) continue;
            const int px = round_half_even_bounded(x), py = round_half_even_bounded(y);
            const int w = lt.w[l], h = lt.h[l];
            if ((unsigned)px >= (unsigned)w || (unsigned)py >= (unsigned)h) continue;
            const size_t pix = (size_t)py * w + px;
            const float* __restrict__ D = lt.depth[l];
            const float* __restrict__ W = lt.weight[l];
            if (q.z > __ldg(D + pix) * kp.depth_accept_plus_one) break;
            const float wgt = __ldg(W + pix);
            const size_t rbase = (size_t)lt.rec_off[l] + pix;
            if (!drop_out)
            {
                if (wgt == 0.f) continue;
                if (bt.grad_texture)
                {
                    float rc[RB];
                    load_record<C>(bt.records, rbase, rc);
                    const float iw = 1.f / wgt;
#pragma unroll
                    for (int c = 0; c < C; ++c) dg[c] += iw * rc[C + c];
                    have_dg = true;
                }
            }
            const int edge = min(min(px, py), min(w - 1 - px, h - 1 - py));
            if (!(point_grad && edge > 2)) continue;
            if (!have_t)
            {
                ti = pts.index ? __ldg(pts.index + i) : i;
                load_descriptor<C>(bt.texture, bt.texture_interleaved, bt.num_texels, ti, T_p);
                have_t = true;
            }
            const size_t nb[4] = {pix - 1, pix + 1, pix - (size_t)w, pix + (size_t)w};
            float rn[4][RB];
#pragma unroll
            for (int k = 0; k < 4; ++k) load_record<C>(bt.records, (size_t)lt.rec_off[l] + nb[k], rn[k]);
            V2 g = stencil_gradient<C>(kp, T_p, rn, q.z, W, D, nb);
            chain_gradient<MODEL>(cam, kp, f, g, scale, gp, acc);
        }
        if (have_dg)
        {
            if (ti < 0) ti = pts.index ? __ldg(pts.index + i) : i;
            add_descriptor_gradient<C>(bt.grad_texture, bt.grad_texture_interleaved, bt.num_texels, ti, dg);
        }
        if (gp[3] > 0.f && bt.grad_points) atomicAdd(bt.grad_points + i, make_float4(gp[0], gp[1], gp[2], gp[3]));
    }
    geo_block_reduce<MODEL>(&s_geo, acc, bt);
}

// ------------------------------------------------------------------------------------------------------
// K5 (visible list): the backward pass over the points that the forward pass listed, grouped by screen tile.
//   k_backward_tiles  one block per screen tile at a time. The tile's region of every layer - weight, forward image and
//                   upstream gradient, with a one-pixel halo (plus one pixel for the rounding of the halved coordinates
//                   on the coarser layers) - is copied from the NCHW planes into shared memory with asynchronous
//                   16-byte copies of whole rows; every listed point of the tile then takes its pixel and its four
//                   stencil neighbours, layer by layer, from there (a point whose pixel falls outside the staged region
//                   reads the planes directly). Per point: ONE descriptor-gradient atomic (summed over its layers) and
//                   ONE work item for the chain kernel: the point's image-space ghost gradient summed over its layers,
//                   each scaled by 0.5^layer (the projection chain is linear in that gradient, and a layer's crop
//                   transform is the full-resolution one times 0.5^layer, PointRenderer.cu:616).
//   k_chain_and_holes  one launch whose blocks split 3 : 1 between two independent parts: per work item, the summed
//                   image-space gradient chained through the projection to the point, pose and intrinsics gradients
//                   (block-reduced); and the background-colour and environment-map gradient of the uncovered pixels.
// Nothing here waits on another block. These kernels are bound by memory latency, not by bandwidth or arithmetic: each
// keeps several independent loads per thread in flight and as many blocks resident as registers and shared memory allow.
constexpr int kTileThreads = 256;
constexpr int kTilePass = 2 * kTileThreads;  // points of a tile that are staged and sorted in shared memory at a time
constexpr int kSortBins = kMaxLayers * kTileH;  // sort key of a point: (layers it visits, image row)
// staged region of layer l: rows [ (y0 >> l) - 1, + rows ), columns [ start, + pitch ), start = x0 - 4 on layer 0 and
// ((x0 >> l) - 1) & ~3 on the others (a multiple of four, so that rows can be copied as aligned 16-byte pieces)
__host__ __device__ constexpr int region_pitch(int l) { return l == 0 ? kTileW + 8 : (l == 1 ? 24 : (l == 2 ? 16 : 12)); }
__host__ __device__ constexpr int region_rows(int l) { return l == 0 ? kTileH + 2 : (l == 1 ? 11 : (l == 2 ? 7 : (l == 3 ? 5 : 4))); }
__host__ __device__ constexpr int region_offset(int l)
{
    int n = 0;
    for (int k = 0; k < l; ++k) n += region_pitch(k) * region_rows(k);
    return n;
}
// floats per plane: the regions of the first four layers, or of all eight (two kernel variants, so that every offset
// into the staged planes is a compile-time constant)
template <bool DEEP>
struct PlaneStride { static constexpr int value = DEEP ? region_offset(kMaxLayers) : region_offset(4); };
inline size_t tile_smem_bytes(int C, int L)
{
    const int stride = L > 4 ? region_offset(kMaxLayers) : region_offset(4);
    return sizeof(float) * (size_t)stride * (2 * C + 1) + sizeof(int4) * kTilePass + sizeof(unsigned short) * kTilePass;
}

__device__ __forceinline__ void async_copy_16(void* smem, const void* gmem)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void async_copy_4(void* smem, const void* gmem)
{
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((unsigned)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void async_copy_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// Copies layer LAYER's region of the 2C + 1 planes into shared memory (asynchronously; the caller waits).
template <int C, int LAYER, int STRIDE>
__device__ __forceinline__ void stage_region(const LayerTable& lt, float* s_tile, int x0, int y0)
{
    constexpr int pitch = region_pitch(LAYER), rows = region_rows(LAYER);
    const int w = lt.w[LAYER], h = lt.h[LAYER];
    const size_t plane = (size_t)w * h;
    const int sx = LAYER == 0 ? x0 - 4 : (((x0 >> LAYER) - 1) & ~3), sy = (y0 >> LAYER) - 1;
    float* dst = s_tile + region_offset(LAYER);
    const bool vec = (w & 3) == 0 && ((reinterpret_cast<uintptr_t>(lt.weight[LAYER]) | reinterpret_cast<uintptr_t>(lt.color[LAYER]) |
                                       reinterpret_cast<uintptr_t>(lt.grad[LAYER])) & 15) == 0;
    if (vec)
    {
        constexpr int p4 = pitch / 4, per_plane = rows * p4;
        for (int q = threadIdx.x; q < per_plane * (2 * C + 1); q += kTileThreads)
        {
            const int p = q / per_plane, r = q - p * per_plane;
            const int row = r / p4, c4 = r - row * p4;
            const int gy = sy + row, gx = sx + 4 * c4;
            if ((unsigned)gy < (unsigned)h && (unsigned)gx < (unsigned)w)
            {
                const float* src = p == 0 ? lt.weight[LAYER] : (p <= C ? lt.color[LAYER] + (size_t)(p - 1) * plane : lt.grad[LAYER] + (size_t)(p - 1 - C) * plane);
                async_copy_16(dst + p * STRIDE + row * pitch + 4 * c4, src + (size_t)gy * w + gx);
            }
        }
    }
    else
    {
        constexpr int per_plane = rows * pitch;
        for (int q = threadIdx.x; q < per_plane * (2 * C + 1); q += kTileThreads)
        {
            const int p = q / per_plane, r = q - p * per_plane;
            const int row = r / pitch, col = r - row * pitch;
            const int gy = sy + row, gx = sx + col;
            if ((unsigned)gy < (unsigned)h && (unsigned)gx < (unsigned)w)
            {
                const float* src = p == 0 ? lt.weight[LAYER] : (p <= C ? lt.color[LAYER] + (size_t)(p - 1) * plane : lt.grad[LAYER] + (size_t)(p - 1 - C) * plane);
                async_copy_4(dst + p * STRIDE + row * pitch + col, src + (size_t)gy * w + gx);
            }
        }
    }
}
template <int C, int LAYER, int STRIDE, int LMAX>
__device__ __forceinline__ void stage_regions(const LayerTable& lt, float* s_tile, int x0, int y0)
{
    if (LAYER < lt.L) stage_region<C, LAYER, STRIDE>(lt, s_tile, x0, y0);
    if constexpr (LAYER + 1 < LMAX) stage_regions<C, LAYER + 1, STRIDE, LMAX>(lt, s_tile, x0, y0);
}

// One (point, layer) visit of the backward pass: descriptor gradient and ghost-geometry image gradient of the point's pixel
// on a layer. at(p, dx, dy) reads a value of plane p (0 = weight, 1.. = image, 1 + C.. = upstream gradient) at an offset
// from the pixel; with p, dx, dy constants after unrolling the staged form is one shared-memory load with an immediate
// offset each.
template <int C, class PIX>
__device__ __forceinline__ void visit_layer(PIX at, bool drop_out, bool want_dg, bool stencil, const float* T_p, const float* bgc, float scale,
                                            float* dg, bool* have_dg, float* gx, float* gy, float* cnt)
{
    const float wgt = at(0, 0, 0);
    if (!drop_out)
    {
        if (wgt == 0.f) return;  // :473
        if (want_dg)
        {
            const float iw = reciprocal(wgt);
#pragma unroll
            for (int c = 0; c < C; ++c) dg[c] += iw * at(1 + C + c, 0, 0);
            *have_dg = true;
        }
    }
    if (!stencil) return;
    // ghost-geometry gradient (PointRenderer.cu:522-611): central differences of (T_p - I_x) * G_x over the four neighbours,
    // averaged over the channels; I = the image before the environment-map composite (:1523)
    float dR[4];
#pragma unroll
    for (int k = 0; k < 4; ++k)
    {
        const int dx = k == 0 ? -1 : (k == 1 ? 1 : 0), dy = k == 2 ? -1 : (k == 3 ? 1 : 0);
        const bool covered = at(0, dx, dy) != 0.f;
        float acc = 0.f;
#pragma unroll
        for (int c = 0; c < C; ++c)
        {
            const float I = covered ? at(1 + c, dx, dy) : bgc[c];
            acc += (T_p[c] - I) * at(1 + C + c, dx, dy);
        }
        dR[k] = acc;
    }
    *gx += (0.5f * (-dR[0] + dR[1]) / (float)C) * scale;
    *gy += (0.5f * (-dR[2] + dR[3]) / (float)C) * scale;
    *cnt += 1.f;
}

// per-point state of the tile kernel while it walks the point's layers
template <int C>
struct PointVisit
{
    float T_p[C], dg[C], bgc[C];
    bool drop_out, point_grad, want_dg, have_dg;
    float gx, gy, cnt;
    unsigned bmask;
};
// the visit of layer LAYER (and, recursively, of the coarser ones); x, y = the position on this layer, scale = 0.5^LAYER
template <int C, int LAYER, int STRIDE, int LMAX>
__device__ __forceinline__ void visit_layers(const LayerTable& lt, const float* s_tile, int x0, int y0, float x, float y, float scale, PointVisit<C>& pv)
{
    if (LAYER < lt.L && (pv.bmask >> LAYER) != 0)  // no coarser layer to visit either: stop
    {
        if (pv.bmask & (1u << LAYER))
        {
            constexpr int pitch = region_pitch(LAYER), rows = region_rows(LAYER);
            const int px = round_half_even_bounded(x), py = round_half_even_bounded(y);
            const int w = lt.w[LAYER], h = lt.h[LAYER];
            const int sx = LAYER == 0 ? x0 - 4 : (((x0 >> LAYER) - 1) & ~3), sy = (y0 >> LAYER) - 1;
            const int cx = px - sx, cy = py - sy;
            const int edge = min(min(px, py), min(w - 1 - px, h - 1 - py));
            const bool stencil = pv.point_grad && edge > 2;
            // the pixel and its four neighbours lie in the staged region (else, rarely: read the planes)
            if (cx >= 1 && cx <= pitch - 2 && cy >= 1 && cy <= rows - 2)
            {
                const float* sp = s_tile + region_offset(LAYER) + cy * pitch + cx;
                visit_layer<C>([&](int p, int dx, int dy) { return sp[p * STRIDE + dy * pitch + dx]; },
                               pv.drop_out, pv.want_dg, stencil, pv.T_p, pv.bgc, scale, pv.dg, &pv.have_dg, &pv.gx, &pv.gy, &pv.cnt);
            }
            else
            {
                const size_t plane = (size_t)w * h;
                const size_t pix = (size_t)py * w + px;
                const float* W = lt.weight[LAYER];
                const float* I = lt.color[LAYER];
                const float* G = lt.grad[LAYER];
                visit_layer<C>([&](int p, int dx, int dy) {
                                   const size_t a = pix + dy * w + dx;
                                   return p == 0 ? __ldg(W + a) : (p <= C ? __ldg(I + (size_t)(p - 1) * plane + a) : __ldg(G + (size_t)(p - 1 - C) * plane + a));
                               },
                               pv.drop_out, pv.want_dg, stencil, pv.T_p, pv.bgc, scale, pv.dg, &pv.have_dg, &pv.gx, &pv.gy, &pv.cnt);
            }
        }
        if constexpr (LAYER + 1 < LMAX) visit_layers<C, LAYER + 1, STRIDE, LMAX>(lt, s_tile, x0, y0, x * 0.5f, y * 0.5f, scale * 0.5f, pv);
    }
}

template <int C, bool DEEP>
__global__ void __launch_bounds__(kTileThreads, C <= 4 ? (DEEP ? 3 : 4) : (C <= 8 ? 2 : 1))
    k_backward_tiles(PointStreams pts, KernelParams kp, LayerTable lt, TileTable tt, BackwardTargets bt, VisibleList vl, int want_geo)
{
    // first kernel of the pass: decides whether the pass runs on the list and leaves the decision for the kernels behind it
    const bool go = (__ldg(vl.header + kListUnusable) | __ldg(vl.header + kListConsumed)) == 0;
    if (blockIdx.x == 0 && threadIdx.x == 0) vl.header[kListGo] = go ? 1 : 0;
    if (!go) return;  // the all-points kernels take over
    constexpr int STRIDE = PlaneStride<DEEP>::value;
    constexpr int LMAX = DEEP ? kMaxLayers : 4;
    extern __shared__ __align__(16) float s_tile[];
    __shared__ int s_hist[kSortBins];
    // plane p of layer l: s_tile[p * STRIDE + region_offset(l) + row * pitch + col]
    int4* sE = reinterpret_cast<int4*>(s_tile + (size_t)STRIDE * (2 * C + 1));
    unsigned short* sOrder = reinterpret_cast<unsigned short*>(sE + kTilePass);
    PointVisit<C> pv;
#pragma unroll
    for (int c = 0; c < C; ++c) pv.bgc[c] = __ldg(bt.background + c);
    // The entry count of the next tile is fetched while this one is worked on.
    int tile = (int)blockIdx.x;
    int n_pts = tile < tt.n_tiles ? min(__ldg(vl.tile_cur + tile), tt.cap) : 0;
    for (; tile < tt.n_tiles; tile += (int)gridDim.x)
    {
        const int next = tile + (int)gridDim.x;
        const int next_n = next < tt.n_tiles ? min(__ldg(vl.tile_cur + next), tt.cap) : 0;
        const int ty = tile / tt.tiles_x, tx = tile - ty * tt.tiles_x;
        const int x0 = tx << kTileShiftX, y0 = ty << kTileShiftY;
        int4* ent = vl.entries + (size_t)tile * tt.cap;
        for (int pass0 = 0; pass0 < n_pts; pass0 += kTilePass)  // block-uniform
        {
            const int n_pass = min(n_pts - pass0, kTilePass);
            __syncthreads();  // the previous readers of the staged data are done
            if (pass0 == 0) stage_regions<C, 0, STRIDE, LMAX>(lt, s_tile, x0, y0);
            for (int q = threadIdx.x; q < n_pass; q += kTileThreads) async_copy_16(sE + q, ent + pass0 + q);
            if (threadIdx.x < kSortBins) s_hist[threadIdx.x] = 0;
            async_copy_wait_all();
            __syncthreads();
            // ---- order the points: by their coarsest layer, most layers first (the warps then walk the same layers in all
            // lanes), and within that by image row (the lanes of a warp then read mostly one row of the staged planes, in
            // different columns: few shared-memory bank conflicts)
            int key[kTilePass / kTileThreads], rank[kTilePass / kTileThreads];
#pragma unroll
            for (int j = 0; j < kTilePass / kTileThreads; ++j)
            {
                const int q = j * kTileThreads + threadIdx.x;
                key[j] = -1;
                if (q < n_pass)
                {
                    const int4 e = sE[q];
                    const unsigned bmask = ((unsigned)e.y >> 8) & 0xffu;
                    const int cls = 32 - __clz(bmask);  // 1 .. kMaxLayers (the backward mask of a listed point is not 0)
                    const int row = min(max(round_half_even_bounded(__int_as_float(e.w)) - y0, 0), kTileH - 1);
                    key[j] = (kMaxLayers - cls) * kTileH + row;
                    rank[j] = atomicAdd(&s_hist[key[j]], 1);
                }
            }
            __syncthreads();
            if (threadIdx.x < 32)
            {
                // exclusive prefix sums of the kSortBins counts: four bins per lane
                constexpr int per = kSortBins / 32;
                int v[per], sum = 0;
#pragma unroll
                for (int k = 0; k < per; ++k) { v[k] = s_hist[threadIdx.x * per + k]; sum += v[k]; }
                int incl = sum;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1)
                {
                    int t = __shfl_up_sync(0xffffffffu, incl, o);
                    if ((int)threadIdx.x >= o) incl += t;
                }
                int run = incl - sum;
#pragma unroll
                for (int k = 0; k < per; ++k) { s_hist[threadIdx.x * per + k] = run; run += v[k]; }
            }
            __syncthreads();
#pragma unroll
            for (int j = 0; j < kTilePass / kTileThreads; ++j)
                if (key[j] >= 0) sOrder[s_hist[key[j]] + rank[j]] = (unsigned short)(j * kTileThreads + threadIdx.x);
            __syncthreads();
            // ---- the points
            for (int sidx = threadIdx.x; sidx < n_pass; sidx += kTileThreads)
            {
                const int4 e = sE[sOrder[sidx]];
                pv.bmask = ((unsigned)e.y >> 8) & 0xffu;
                const int i = (int)((unsigned)e.x & ~kEntryDropped);
                pv.drop_out = ((unsigned)e.x & kEntryDropped) != 0;
                pv.point_grad = want_geo && ((kp.ghost_gradients && pv.drop_out) || (!kp.ghost_gradients && !pv.drop_out));
                pv.want_dg = !pv.drop_out && bt.grad_texture != nullptr;
                const int ti = pts.index ? __ldg(pts.index + i) : i;
                if (pv.point_grad) load_descriptor<C>(bt.texture, bt.texture_interleaved, bt.num_texels, ti, pv.T_p);
                else
                {
#pragma unroll
                    for (int c = 0; c < C; ++c) pv.T_p[c] = 0.f;
                }
#pragma unroll
                for (int c = 0; c < C; ++c) pv.dg[c] = 0.f;
                pv.have_dg = false;
                pv.gx = pv.gy = pv.cnt = 0.f;
                visit_layers<C, 0, STRIDE, LMAX>(lt, s_tile, x0, y0, __int_as_float(e.z), __int_as_float(e.w), 1.f, pv);
                if (pv.have_dg) add_descriptor_gradient<C>(bt.grad_texture, bt.grad_texture_interleaved, bt.num_texels, ti, pv.dg);
                // the entry becomes the chain kernel's work item (every entry of this pass has been read into shared memory)
                if (want_geo)
                    reinterpret_cast<float4*>(ent)[pass0 + sidx] = pv.cnt > 0.f ? make_float4(__int_as_float(i), pv.gx, pv.gy, pv.cnt) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
        n_pts = next_n;
    }
}

// Background-colour gradient (CombineAndFillBackward, PointRenderer.cu:851-900) and environment-map gradient (the
// composite's backward, RenderModule.cpp:121-125, grid_sample backward) of the uncovered pixels of one view: one thread
// per four pyramid pixels reads the weights; the holes, scattered single pixels, are parked per warp and worked off 32
// at a time (gradient of each channel; for the environment map the ray through the inverse camera model and the bilinear
// scatter).
struct HoleArgs
{
    float* grad_background;
    float* grad_env;
    int env_h, env_w;
    bool env_interleaved;
};
// part of k_chain_and_holes: `block` of `blocks` thread blocks
template <int C>
__device__ __forceinline__ void hole_gradients_part(const LayerTable& lt, const ViewCam* __restrict__ camp, const KernelParams& kp, const HoleArgs& ha,
                                                    int block, int blocks)
{
    float* __restrict__ grad_background = ha.grad_background;
    float* __restrict__ grad_env = ha.grad_env;
    const int env_h = ha.env_h, env_w = ha.env_w;
    const bool env_interleaved = ha.env_interleaved;
    const ViewCam& cam = *camp;
    __shared__ float s_bg[C];
    __shared__ unsigned s_parked[kBlock / 32][160];
    unsigned* parked = s_parked[threadIdx.x >> 5];
    const int lane = threadIdx.x & 31;
    int n_parked = 0;  // the same in every lane of the warp
    if (threadIdx.x < C) s_bg[threadIdx.x] = 0.f;
    __syncthreads();
    float g[C];
#pragma unroll
    for (int c = 0; c < C; ++c) g[c] = 0.f;
    auto work_off = [&](unsigned r)
    {
        const int l = layer_of_record(lt, r);
        const unsigned pix = r - lt.rec_off[l];
        const size_t plane = (size_t)lt.w[l] * lt.h[l];
        if (grad_background)
        {
#pragma unroll
            for (int c = 0; c < C; ++c) g[c] += __ldg(lt.grad[l] + c * plane + pix);
        }
        if (grad_env) scatter_environment_gradient<C>(lt, cam, kp, r, grad_env, env_h, env_w, env_interleaved);
    };
    const unsigned total = lt.rec_off[kMaxLayers];
    const unsigned groups = (total + 3) / 4;
    const unsigned stride = (unsigned)blocks * blockDim.x;
    for (unsigned base = (unsigned)block * blockDim.x; base < groups; base += stride)  // warp-uniform trip count
    {
        // four consecutive pyramid pixels per thread (they may straddle a layer boundary: the weights are read one by one)
        const unsigned r0 = (base + threadIdx.x) * 4;
        bool hole[4];
#pragma unroll
        for (int k = 0; k < 4; ++k)
        {
            hole[k] = false;
            const unsigned r = r0 + k;
            if (r < total)
            {
                const int l = layer_of_record(lt, r);
                hole[k] = __ldg(lt.weight[l] + (r - lt.rec_off[l])) == 0.f;
            }
        }
#pragma unroll
        for (int k = 0; k < 4; ++k)
        {
            const unsigned vote = __ballot_sync(0xffffffffu, hole[k]);
            if (hole[k]) parked[n_parked + __popc(vote & ((1u << lane) - 1u))] = r0 + k;
            n_parked += __popc(vote);
        }
        __syncwarp();
        while (n_parked >= 32)
        {
            n_parked -= 32;
            work_off(parked[n_parked + lane]);
        }
        __syncwarp();
    }
    if (lane < n_parked) work_off(parked[lane]);
    if (grad_background)
    {
#pragma unroll
        for (int c = 0; c < C; ++c)
        {
            float v = warp_sum(g[c]);
            if (lane == 0 && v != 0.f) atomicAdd(&s_bg[c], v);
        }
        __syncthreads();
        if (threadIdx.x < C && s_bg[threadIdx.x] != 0.f) atomicAdd(grad_background + threadIdx.x, s_bg[threadIdx.x]);
    }
}

// ---- per-point chain ---------------------------------------------------------------------------------------------------
// A visible point with its summed image-space gradient, as parked in shared memory by k_point_chain.
struct ChainItem
{
    int id;
    float gx, gy, count;
    float px, py, pz;
    int normal;
};

// Pinhole chain in a short form (same mathematics as project_pinhole_backward, PointRendererHelper.h:109-170, summed
// straight into the per-thread partial sums). With q = x g1x + y g1y (m = (x, y) the normalised point, g1 the gradient
// behind K) the sixteen entries of the distortion Jacobian and the four of J_m collapse:
//   d/dk1..k3 = {r2, r4, r6} q / den,  d/dk4..k6 = -rad {r2, r4, r6} q / den,  d/dp1 = 2xy g1x + (r2 + 2y2) g1y,  d/dp2 = (r2 + 2x2) g1x + 2xy g1y,
//   gm = rad g1 + 2 m drad q + tangential terms,   drad = (dnum - rad dden) / den.
// The partial sums are undamped; the damping factors of PointRenderer.cu:647-678 are applied once per block.
struct PinholeSums
{
    float pose[6];
    float k[4];
    float d[8];
    float cnt;
};
__device__ __forceinline__ void chain_pinhole_fast(const ViewCam& cam, bool check_normal, const ChainItem& it, float4* __restrict__ grad_points,
                                                   PinholeSums& a)
{
    const Rigid32& V = cam.V;
    V3 view;
    view.x = fmaf(V.r[0], it.px, fmaf(V.r[1], it.py, fmaf(V.r[2], it.pz, V.t[0])));
    view.y = fmaf(V.r[3], it.px, fmaf(V.r[4], it.py, fmaf(V.r[5], it.pz, V.t[1])));
    view.z = fmaf(V.r[6], it.px, fmaf(V.r[7], it.py, fmaf(V.r[8], it.pz, V.t[2])));
    if (!(view.z > 0.f)) return;
    if (check_normal)
    {
        V3 vn = rotate(V, unpack_normal_10bit(it.normal));
        if (fmaf(view.z, vn.z, fmaf(view.y, vn.y, view.x * vn.x)) > 0.f) return;
    }
    const float iz = reciprocal(view.z);
    const float x = view.x * iz, y = view.y * iz;
    const float x2 = x * x, y2 = y * y, r2 = x2 + y2, r4 = r2 * r2, r6 = r4 * r2, xy2 = 2.f * x * y;
    const Dist8& d = cam.dist;
    const float num = fmaf(fmaf(fmaf(d.k3, r2, d.k2), r2, d.k1), r2, 1.0f);
    const float den = fmaf(fmaf(fmaf(d.k6, r2, d.k5), r2, d.k4), r2, 1.0f);
    const float iden = reciprocal(den);
    const float rad = num * iden;
    const float dnum = fmaf(fmaf(3.f * d.k3, r2, 2.f * d.k2), r2, d.k1);
    const float dden = fmaf(fmaf(3.f * d.k6, r2, 2.f * d.k5), r2, d.k4);
    const float drad = fmaf(-rad, dden, dnum) * iden;
    const float dpx = fmaf(x, rad, fmaf(d.p1, xy2, d.p2 * fmaf(2.f, x2, r2)));
    const float dpy = fmaf(y, rad, fmaf(d.p2, xy2, d.p1 * fmaf(2.f, y2, r2)));
    // crop^T, K
    const float g2x = cam.crop.fx * it.gx;
    const float g2y = fmaf(cam.crop.s, it.gx, cam.crop.fy * it.gy);
    a.k[0] = fmaf(dpx, g2x, a.k[0]); a.k[1] = fmaf(dpy, g2y, a.k[1]); a.k[2] += g2x; a.k[3] += g2y;
    const float g1x = cam.K.fx * g2x;
    const float g1y = fmaf(cam.K.s, g2x, cam.K.fy * g2y);
    const float q = fmaf(x, g1x, y * g1y);
    const float qd = q * iden, qr = -rad * qd;
    a.d[0] = fmaf(r2, qd, a.d[0]); a.d[1] = fmaf(r4, qd, a.d[1]); a.d[2] = fmaf(r6, qd, a.d[2]);
    a.d[3] = fmaf(r2, qr, a.d[3]); a.d[4] = fmaf(r4, qr, a.d[4]); a.d[5] = fmaf(r6, qr, a.d[5]);
    const float ry = fmaf(2.f, y2, r2), rx = fmaf(2.f, x2, r2);
    a.d[6] += fmaf(xy2, g1x, ry * g1y);
    a.d[7] += fmaf(rx, g1x, xy2 * g1y);
    // J_m^T g1
    const float wq = 2.f * drad * q;
    const float j01 = 2.f * fmaf(d.p1, x, d.p2 * y);  // the off-diagonal tangential term
    const float gmx = fmaf(rad + fmaf(2.f * d.p1, y, 6.f * d.p2 * x), g1x, fmaf(j01, g1y, x * wq));
    const float gmy = fmaf(rad + fmaf(6.f * d.p1, y, 2.f * d.p2 * x), g1y, fmaf(j01, g1x, y * wq));
    // divide by z, rigid transform
    V3 gv;
    gv.x = iz * gmx;
    gv.y = iz * gmy;
    gv.z = -fmaf(x, gv.x, y * gv.y);
    const V3 gp = rotate_inv(V, gv);
    a.pose[0] += gv.x; a.pose[1] += gv.y; a.pose[2] += gv.z;
    a.pose[3] += fmaf(view.y, gv.z, -view.z * gv.y);
    a.pose[4] += fmaf(view.z, gv.x, -view.x * gv.z);
    a.pose[5] += fmaf(view.x, gv.y, -view.y * gv.x);
    a.cnt += it.count;
    if (grad_points) atomicAdd(grad_points + it.id, make_float4(gp.x, gp.y, gp.z, it.count));
}

// General form (used for the omnidirectional model): chain of one point's summed image-space gradient (already scaled
// to full resolution) with `count` contributions, through the Jacobian functions of the arithmetic header.
template <int MODEL>
__device__ __forceinline__ bool chain_gradient_sum(const ViewCam& cam, const KernelParams& kp, const FetchedPoint& f, V2 g, float count,
                                                   float* gp, GeoAccum<MODEL>& acc)
{
    static_assert(MODEL == kOcam, "the pinhole model takes chain_pinhole_fast");
    GradOcam o;
    if (!project_ocam_backward(f.p, f.n, f.has_normal, g, cam.V, cam.crop, cam.ocam, kp.check_normal != 0, kp.dist_cutoff, &o))
        return false;
    gp[0] = o.g_point[0]; gp[1] = o.g_point[1]; gp[2] = o.g_point[2]; gp[3] = count;
#pragma unroll
    for (int k = 0; k < 6; ++k) acc.pose[k] += o.g_pose[k];
#pragma unroll
    for (int k = 0; k < 5; ++k) acc.intr[k] += o.g_affine[k];
    acc.cnt += count;
    return true;
}

// part of k_chain_and_holes: `block` of `blocks` thread blocks
template <int MODEL>
__device__ __forceinline__ void point_chain_part(const PointStreams& pts, const ViewCam* __restrict__ camp, const KernelParams& kp, const BackwardTargets& bt,
                                                 const VisibleList& vl, const TileTable& tt, int block, int blocks)
{
    __shared__ ViewCam s_cam;
    __shared__ GeoShared<MODEL> s_geo;
    // points with a gradient are parked per warp, with their position, and chained 32 at a time with every lane busy
    __shared__ ChainItem s_park[kBlock / 32][96];
    ChainItem* park = s_park[threadIdx.x >> 5];
    const int lane = threadIdx.x & 31;
    int n_parked = 0;
    for (int k = threadIdx.x; k < (int)(sizeof(ViewCam) / 4); k += kBlock) reinterpret_cast<int*>(&s_cam)[k] = __ldg(reinterpret_cast<const int*>(camp) + k);
    geo_shared_init(&s_geo);
    __syncthreads();
    const ViewCam& cam = s_cam;
    const bool check_normal = kp.check_normal != 0 && pts.normal != nullptr;
    GeoAccum<MODEL> acc;
    acc.clear();
    PinholeSums ps;
#pragma unroll
    for (int k = 0; k < 6; ++k) ps.pose[k] = 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) ps.k[k] = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) ps.d[k] = 0.f;
    ps.cnt = 0.f;
    auto chain_one = [&](const ChainItem& it)
    {
        if (MODEL == kPinholeDistortion)
            chain_pinhole_fast(cam, check_normal, it, bt.grad_points, ps);
        else
        {
            FetchedPoint f;
            f.p.x = it.px; f.p.y = it.py; f.p.z = it.pz; f.r = 0.f;
            f.has_normal = pts.normal != nullptr;
            f.n = unpack_normal_10bit(it.normal);
            V2 g; g.x = it.gx; g.y = it.gy;
            float gp[4];
            if (chain_gradient_sum<kOcam>(cam, kp, f, g, it.count, gp, reinterpret_cast<GeoAccum<kOcam>&>(acc)) && bt.grad_points)
                atomicAdd(bt.grad_points + it.id, make_float4(gp[0], gp[1], gp[2], gp[3]));
        }
    };
    constexpr int U = 2;  // items per thread and round: their dependent loads (item -> position) are in flight together
    for (int tile = block; tile < tt.n_tiles; tile += blocks)
    {
        const int total = min(__ldg(vl.tile_cur + tile), tt.cap);
        const float4* work = reinterpret_cast<const float4*>(vl.entries + (size_t)tile * tt.cap);  // the tile kernel's work items
        for (int k0 = 0; k0 < total; k0 += kBlock * U)  // warp-uniform trip count
        {
            float4 v[U], p[U];
            int nrm[U];
#pragma unroll
            for (int j = 0; j < U; ++j)
            {
                const int k = k0 + j * kBlock + threadIdx.x;
                v[j] = k < total ? __ldcs(work + k) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int j = 0; j < U; ++j)
            {
                p[j] = make_float4(0.f, 0.f, 0.f, 0.f); nrm[j] = 0;
                if (v[j].w > 0.f)
                {
                    const int id = __float_as_int(v[j].x);
                    p[j] = __ldg(pts.position + id);
                    if (pts.normal) nrm[j] = __ldg(pts.normal + id);
                }
            }
#pragma unroll
            for (int j = 0; j < U; ++j)
            {
                const bool has = v[j].w > 0.f;
                const unsigned vote = __ballot_sync(0xffffffffu, has);
                if (has)
                {
                    ChainItem& it = park[n_parked + __popc(vote & ((1u << lane) - 1u))];
                    it.id = __float_as_int(v[j].x); it.gx = v[j].y; it.gy = v[j].z; it.count = v[j].w;
                    it.px = p[j].x; it.py = p[j].y; it.pz = p[j].z; it.normal = nrm[j];
                }
                n_parked += __popc(vote);
            }
            __syncwarp();
            while (n_parked >= 32)
            {
                n_parked -= 32;
                chain_one(park[n_parked + lane]);
            }
            __syncwarp();
        }
    }
    if (lane < n_parked) chain_one(park[lane]);
    if (MODEL == kPinholeDistortion)
    {
        // into the common form, with the damping of PointRenderer.cu:647-678 (skew gets no gradient)
        const float kf = kp.K_gradient_factor, df = kp.distortion_gradient_factor;
#pragma unroll
        for (int k = 0; k < 6; ++k) acc.pose[k] = ps.pose[k];
        acc.intr[0] = kf * ps.k[0]; acc.intr[1] = kf * ps.k[1]; acc.intr[2] = kf * ps.k[2]; acc.intr[3] = kf * ps.k[3];
        acc.intr[5] = df * ps.d[0]; acc.intr[6] = df * ps.d[1]; acc.intr[7] = df * (ps.d[2] * 0.25f);
        acc.intr[8] = df * (ps.d[3] * 0.1f); acc.intr[9] = df * (ps.d[4] * 0.1f); acc.intr[10] = df * (ps.d[5] * 0.1f);
        acc.intr[11] = df * (ps.d[6] * 0.1f); acc.intr[12] = df * (ps.d[7] * 0.1f);
        acc.cnt = ps.cnt;
    }
    geo_block_reduce<MODEL>(&s_geo, acc, bt);
}

// The chain kernel and the hole kernel of one view in one launch: they are independent, the first waits on memory most of
// the time and the second on arithmetic, so side by side they take little more than the longer of the two.
// Blocks [0, chain_blocks) chain the tile kernel's work items, the others walk the uncovered pixels.
template <int C, int MODEL>
__global__ void __launch_bounds__(kBlock, MODEL == kPinholeDistortion ? 4 : 3)
    k_chain_and_holes(PointStreams pts, const ViewCam* __restrict__ camp, KernelParams kp, LayerTable lt, BackwardTargets bt, VisibleList vl, TileTable tt,
                      HoleArgs ha, int chain_blocks)
{
    if (__ldg(vl.header + kListGo) == 0) return;  // the all-points kernels do this work
    if ((int)blockIdx.x < chain_blocks) point_chain_part<MODEL>(pts, camp, kp, bt, vl, tt, (int)blockIdx.x, chain_blocks);
    else hole_gradients_part<C>(lt, camp, kp, ha, (int)blockIdx.x - chain_blocks, (int)gridDim.x - chain_blocks);
}

// ------------------------------------------------------------------------------------------------------
// NormalizeGradient, PointRenderer.cu:1534-1547
__global__ void k_normalize_points(float4* g, int n)
{
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float4 v = g[i];
    if (v.w > 0.f) { v.x = v.x / v.w; v.y = v.y / v.w; v.z = v.z / v.w; }
    v.w = 0.f;
    g[i] = v;
}
__global__ void k_normalize_pose(double* g, const float* cnt, int n)
{
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n * 6) return;
    float c = cnt[i / 6];
    if (c > 0.f) g[i] = g[i] / (double)c;
}
__global__ void k_normalize_intrinsics(float* g, const float* cnt, int n, int cols)
{
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n * cols) return;
    float c = cnt[i / cols];
    if (c > 0.f) g[i] = g[i] / c;
}

// ------------------------------------------------------------------------------------------------------
template <int C>
static adop_status launch_view_backward(const PointStreams& pts, const ViewCam* cam, const KernelParams& kp, const LayerTable& lt,
                                        const TileTable& tt, const BackwardTargets& bt, float* grad_background, float* grad_env, int env_h,
                                        int env_w, bool env_interleaved, cudaStream_t st, const VisibleList& vl, int model)
{
    const int need = (pts.n + kBlock - 1) / kBlock;
    // With a visible list the tile kernels run; the all-points kernels are launched behind them and return at once unless
    // the list turns out not to be usable (decided on the device by the first kernel, no host round trip). The debug
    // stencil rule (test_backward_mode 4) needs the point's depth next to its neighbours' and always takes the all-points
    // kernels.
    const bool use_list = vl.header && kp.test_backward_mode != 4;
    int* go = use_list ? vl.header + kListGo : nullptr;
    const int want_geo = (bt.grad_points || bt.grad_pose || bt.grad_intrinsics) ? 1 : 0;
    if (use_list)
    {
        const size_t smem = tile_smem_bytes(C, lt.L);
        const bool deep = lt.L > 4;
        static size_t smem_set[2] = {0, 0};
        if (smem > smem_set[deep])
        {
            if (deep) ADOP_CUDA_TRY(cudaFuncSetAttribute(k_backward_tiles<C, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            else ADOP_CUDA_TRY(cudaFuncSetAttribute(k_backward_tiles<C, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            smem_set[deep] = smem;
        }
        int per_sm = 0;
        cudaError_t oe = deep ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k_backward_tiles<C, true>, kTileThreads, smem)
                              : cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k_backward_tiles<C, false>, kTileThreads, smem);
        if (oe != cudaSuccess || per_sm < 1) per_sm = 1;
        const int g_tiles = per_sm * sm_count();
        const int grid_tiles = tt.n_tiles < g_tiles ? (tt.n_tiles < 1 ? 1 : tt.n_tiles) : g_tiles;
        if (deep) ADOP_LAUNCH("k_backward_tiles", st, (k_backward_tiles<C, true><<<grid_tiles, kTileThreads, smem, st>>>(pts, kp, lt, tt, bt, vl, want_geo)));
        else ADOP_LAUNCH("k_backward_tiles", st, (k_backward_tiles<C, false><<<grid_tiles, kTileThreads, smem, st>>>(pts, kp, lt, tt, bt, vl, want_geo)));
        if (grad_env || grad_background || want_geo)
        {
            HoleArgs ha;
            ha.grad_background = grad_background; ha.grad_env = grad_env; ha.env_h = env_h; ha.env_w = env_w; ha.env_interleaved = env_interleaved;
            const unsigned groups = (lt.rec_off[kMaxLayers] + 3) / 4;
            const int hole_need = (grad_env || grad_background) ? (int)((groups + kBlock - 1) / kBlock) : 0;
            if (model == kPinholeDistortion)
            {
                static const int g = resident_grid(k_chain_and_holes<C, kPinholeDistortion>, 1ll << 40);
                // the chain blocks get five eighths of the resident blocks when both parts have work (measured: between a half
                // and three quarters the kernel's time is flat, beyond it rises quickly)
                int chain_blocks = want_geo ? (hole_need ? g * 5 / 8 : g) : 0;
                if (chain_blocks > tt.n_tiles) chain_blocks = tt.n_tiles;
                int hole_blocks = g - chain_blocks < hole_need ? g - chain_blocks : hole_need;
                if (hole_need && hole_blocks < 1) hole_blocks = 1;
                ADOP_LAUNCH("k_chain_and_holes", st, (k_chain_and_holes<C, kPinholeDistortion><<<chain_blocks + hole_blocks, kBlock, 0, st>>>(
                                                         pts, cam, kp, lt, bt, vl, tt, ha, chain_blocks)));
            }
            else
            {
                static const int g = resident_grid(k_chain_and_holes<C, kOcam>, 1ll << 40);
                int chain_blocks = want_geo ? (hole_need ? g * 5 / 8 : g) : 0;
                if (chain_blocks > tt.n_tiles) chain_blocks = tt.n_tiles;
                int hole_blocks = g - chain_blocks < hole_need ? g - chain_blocks : hole_need;
                if (hole_need && hole_blocks < 1) hole_blocks = 1;
                ADOP_LAUNCH("k_chain_and_holes", st, (k_chain_and_holes<C, kOcam><<<chain_blocks + hole_blocks, kBlock, 0, st>>>(
                                                         pts, cam, kp, lt, bt, vl, tt, ha, chain_blocks)));
            }
        }
    }
    // Behind a visible list these two launches are almost always no-ops that only read the list's control word, so they
    // get one block per SM (an empty launch costs by its block count); without a list they are the backward pass and fill
    // the GPU.
    const int fallback_cap = use_list ? sm_count() : (1 << 30);
    {
        static const int cap = resident_grid(k_prepare_backward<C>, 1ll << 40);
        unsigned total = lt.rec_off[kMaxLayers];
        int grid_px = (int)((total + kBlock - 1) / kBlock);
        if (grid_px > cap) grid_px = cap;
        if (grid_px > fallback_cap) grid_px = fallback_cap;
        ADOP_LAUNCH("k_prepare_backward", st, (k_prepare_backward<C><<<grid_px, kBlock, 0, st>>>(
                                                  lt, cam, kp, bt.background, const_cast<float*>(bt.records), grad_background,
                                                  grad_env, env_h, env_w, env_interleaved, go)));
    }
    int* header = use_list ? vl.header : nullptr;
    if (model == kPinholeDistortion)
    {
        static const int g = resident_grid(k_splat_backward_all<C, kPinholeDistortion>, 1ll << 40);
        int grid = need < g ? (need < 1 ? 1 : need) : g;
        if (grid > fallback_cap) grid = fallback_cap;
        ADOP_LAUNCH("k_splat_backward_all", st, (k_splat_backward_all<C, kPinholeDistortion><<<grid, kBlock, 0, st>>>(pts, cam, kp, lt, bt, header, want_geo)));
    }
    else
    {
        static const int g = resident_grid(k_splat_backward_all<C, kOcam>, 1ll << 40);
        int grid = need < g ? (need < 1 ? 1 : need) : g;
        if (grid > fallback_cap) grid = fallback_cap;
        ADOP_LAUNCH("k_splat_backward_all", st, (k_splat_backward_all<C, kOcam><<<grid, kBlock, 0, st>>>(pts, cam, kp, lt, bt, header, want_geo)));
    }
    ADOP_CUDA_TRY(cudaGetLastError());
    return ADOP_OK;
}

}  // namespace adop

using namespace adop;

extern "C" adop_status adop_raster_normalize_gradients(float* grad_points, int32_t num_points, double* grad_pose,
                                                       const float* count_pose, int32_t num_images, float* grad_intrinsics,
                                                       const float* count_intrinsics, int32_t num_cameras,
                                                       int32_t intrinsics_cols, void* stream)
{
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (grad_pose)
    {
        if (!count_pose || num_images <= 0) return ADOP_ERR_INVALID_ARGUMENT;
        int n = num_images * 6;
        ADOP_LAUNCH("k_normalize", st, (k_normalize_pose<<<(n + 127) / 128, 128, 0, st>>>(grad_pose, count_pose, num_images)));
    }
    if (grad_points && num_points > 0)
        ADOP_LAUNCH("k_normalize", st, (k_normalize_points<<<(num_points + 255) / 256, 256, 0, st>>>(reinterpret_cast<float4*>(grad_points), num_points)));
    if (grad_intrinsics)
    {
        if (!count_intrinsics || num_cameras <= 0 || intrinsics_cols <= 0) return ADOP_ERR_INVALID_ARGUMENT;
        int n = num_cameras * intrinsics_cols;
        ADOP_LAUNCH("k_normalize", st, (k_normalize_intrinsics<<<(n + 127) / 128, 128, 0, st>>>(grad_intrinsics, count_intrinsics, num_cameras, intrinsics_cols)));
    }
    ADOP_CUDA_TRY(cudaGetLastError());
    return ADOP_OK;
}

extern "C" adop_status adop_raster_backward(const adop_scene* s, const adop_view* views, int32_t B,
                                            const adop_render_params* rp, int32_t L, adop_backward_io* io, void* stream)
{
    adop_status vs = validate_common(s, views, B, rp, L);
    if (vs != ADOP_OK) return vs;
    if (!io) return ADOP_ERR_INVALID_ARGUMENT;
    const int C = s->channels, N = s->num_points, T = s->num_texels, cols = s->intrinsics_cols;
    for (int l = 0; l < L; ++l)
        if (!io->layers[l].color || !io->layers[l].depth || !io->layers[l].weight || !io->grad_color[l])
            return ADOP_ERR_INVALID_ARGUMENT;
    if ((io->grad_pose && !io->count_pose) || (io->grad_intrinsics && !io->count_intrinsics)) return ADOP_ERR_INVALID_ARGUMENT;
    if (reinterpret_cast<uintptr_t>(io->grad_points) & 15) return ADOP_ERR_INVALID_ARGUMENT;
    if (!io->workspace || (reinterpret_cast<uintptr_t>(io->workspace) & 15)) return ADOP_ERR_INVALID_ARGUMENT;
    if (io->workspace_bytes < adop_raster_workspace_bytes(views[0].w, views[0].h, L, C)) return ADOP_ERR_WORKSPACE_TOO_SMALL;
    const bool env = rp->composite_environment_map && s->env_map && io->grad_env_map;
    if (env)
        for (int b = 0; b < B; ++b)
            if (views[b].camera_model != ADOP_CAMERA_PINHOLE_DISTORTION) return ADOP_ERR_UNSUPPORTED;

    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (!io->accumulate)
    {
        if (io->grad_texture && !io->grad_texture_interleaved)
            ADOP_CUDA_TRY(cudaMemsetAsync(io->grad_texture, 0, sizeof(float) * (size_t)C * T, st));
        if (io->grad_background) ADOP_CUDA_TRY(cudaMemsetAsync(io->grad_background, 0, sizeof(float) * C, st));
        if (io->grad_points) ADOP_CUDA_TRY(cudaMemsetAsync(io->grad_points, 0, sizeof(float) * (size_t)N * 4, st));
        if (io->grad_pose) ADOP_CUDA_TRY(cudaMemsetAsync(io->grad_pose, 0, sizeof(double) * (size_t)s->num_images * 6, st));
        if (io->count_pose) ADOP_CUDA_TRY(cudaMemsetAsync(io->count_pose, 0, sizeof(float) * s->num_images, st));
        if (io->grad_intrinsics) ADOP_CUDA_TRY(cudaMemsetAsync(io->grad_intrinsics, 0, sizeof(float) * (size_t)s->num_cameras * cols, st));
        if (io->count_intrinsics) ADOP_CUDA_TRY(cudaMemsetAsync(io->count_intrinsics, 0, sizeof(float) * s->num_cameras, st));
        if (io->grad_env_map && s->env_h > 0 && s->env_w > 0)
            ADOP_CUDA_TRY(cudaMemsetAsync(io->grad_env_map, 0, sizeof(float) * (size_t)C * s->env_h * s->env_w, st));
    }

    // environment-map gradient: summed in an [eh,ew,C] scratch with vector atomics when the caller gave one
    const bool env_inter = env && io->grad_env_map_interleaved && C % 4 == 0 &&
                           (reinterpret_cast<uintptr_t>(io->grad_env_map_interleaved) & 15) == 0;
    if (env_inter)
        ADOP_CUDA_TRY(cudaMemsetAsync(io->grad_env_map_interleaved, 0, sizeof(float) * (size_t)C * s->env_h * s->env_w, st));
    // descriptor gradients stay in the [T,C] buffer when there is no [C,T] tensor to move them into
    const bool interleaved_only = !io->grad_texture && io->grad_texture_interleaved;
    if (io->grad_texture_interleaved && (io->grad_texture || !io->accumulate))
        ADOP_CUDA_TRY(cudaMemsetAsync(io->grad_texture_interleaved, 0, sizeof(float) * (size_t)C * T, st));
    LayerTable base;
    fill_layer_dims(views[0].w, views[0].h, L, &base);
    const TileTable tiles = make_tile_table(views[0].w, views[0].h, N);
    ViewCam* cams = static_cast<ViewCam*>(io->workspace);
    PointStreams pts;
    pts.position = reinterpret_cast<const float4*>(s->position);
    pts.normal = s->normal;
    pts.index = s->index;
    pts.n = N;
    for (int b = 0; b < B; ++b)
    {
        LayerTable lt = base;
        for (int l = 0; l < L; ++l)
        {
            size_t plane = (size_t)base.w[l] * base.h[l];
            lt.depth[l] = io->layers[l].depth + (size_t)b * plane;
            lt.weight[l] = io->layers[l].weight + (size_t)b * plane;
            lt.color[l] = io->layers[l].color + (size_t)b * C * plane;
            lt.grad[l] = io->grad_color[l] + (size_t)b * C * plane;
        }
        KernelParams kp = make_kernel_params(rp, io->dropout_mask, N, b);
        if (b % kCamChunk == 0)
        {
            CamChunkSource src;
            fill_cam_chunk(&src, s, views + b, B - b < kCamChunk ? B - b : kCamChunk);
            ADOP_LAUNCH("k_build_cams", st, (k_build_cams<<<1, kCamChunk, 0, st>>>(src, cams)));
        }
        const ViewCam* cam = cams + (b % kCamChunk);
        BackwardTargets bt;
        bt.texture = s->texture;
        bt.texture_interleaved = s->texture_interleaved;
        bt.grad_texture_interleaved = io->grad_texture_interleaved;
        bt.num_texels = T;
        bt.background = s->background;
        // the kernels take a non-null grad_texture as "descriptor gradients wanted" and write the [T,C] buffer if there is one
        bt.grad_texture = interleaved_only ? io->grad_texture_interleaved : io->grad_texture;
        bt.grad_points = reinterpret_cast<float4*>(io->grad_points);
        bt.grad_pose = io->grad_pose ? io->grad_pose + (size_t)views[b].image_index * 6 : nullptr;
        bt.count_pose = io->grad_pose ? io->count_pose + views[b].image_index : nullptr;
        bt.grad_intrinsics = io->grad_intrinsics ? io->grad_intrinsics + (size_t)views[b].camera_index * cols : nullptr;
        bt.count_intrinsics = io->grad_intrinsics ? io->count_intrinsics + views[b].camera_index : nullptr;
        bt.records = reinterpret_cast<const float*>(static_cast<const char*>(io->workspace) + kCamRegionBytes);
        float* ge = env ? (env_inter ? io->grad_env_map_interleaved : io->grad_env_map) : nullptr;
        // the list's layout (tiles, bucket size) follows from the view size and the point count, as in the forward pass
        VisibleList vl = make_visible_list(const_cast<int32_t*>(io->visible_list), N, views[0].w, views[0].h, b);
        adop_status r;
        switch (C)
        {
            case 3: r = launch_view_backward<3>(pts, cam, kp, lt, tiles, bt, io->grad_background, ge, s->env_h, s->env_w, env_inter, st, vl, views[b].camera_model); break;
            case 4: r = launch_view_backward<4>(pts, cam, kp, lt, tiles, bt, io->grad_background, ge, s->env_h, s->env_w, env_inter, st, vl, views[b].camera_model); break;
            case 8: r = launch_view_backward<8>(pts, cam, kp, lt, tiles, bt, io->grad_background, ge, s->env_h, s->env_w, env_inter, st, vl, views[b].camera_model); break;
            case 16: r = launch_view_backward<16>(pts, cam, kp, lt, tiles, bt, io->grad_background, ge, s->env_h, s->env_w, env_inter, st, vl, views[b].camera_model); break;
            default:
                snprintf(last_error_buffer(), 512, "%d descriptor channels: the kernels are built for 3, 4, 8 and 16", C);
                return ADOP_ERR_UNSUPPORTED;
        }
        if (r != ADOP_OK) return r;
    }
    if (io->grad_texture && io->grad_texture_interleaved)
    {
        adop_status ds = adop_texture_deinterleave(io->grad_texture_interleaved, io->grad_texture, C, T, io->accumulate ? 1 : 0, stream);
        if (ds != ADOP_OK) return ds;
    }
    if (env_inter)
    {
        // [eh,ew,C] -> [C,eh,ew]; the tensor was zeroed above unless the caller accumulates
        adop_status ds = adop_texture_deinterleave(io->grad_env_map_interleaved, io->grad_env_map, C, s->env_h * s->env_w, 1, stream);
        if (ds != ADOP_OK) return ds;
    }
    if (io->normalize)
        return adop_raster_normalize_gradients(io->grad_points, N, io->grad_pose, io->count_pose, s->num_images,
                                               io->grad_intrinsics, io->count_intrinsics, s->num_cameras, cols, stream);
    return ADOP_OK;
}
