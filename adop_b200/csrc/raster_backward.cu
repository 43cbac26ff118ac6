// Backward pass of the one-pixel point rasterizer for sm_100a.
// Stands in for BlendPointCloudBackward and its kernels (darglein/ADOP src/lib/rendering/PointRenderer.cu:
// CombineAndFillBackward :851-900, RenderBackward :396-724, NormalizeGradient :1534-1547) and the gradient
// of the environment-map composite (RenderModule.cpp:121-125, grid_sample backward).
//
// Differences in how the same sums are formed (results agree within float-ordering tolerance):
//  * the forward pass records which (point, layer) splats the backward pass will visit; the backward kernel then runs
//    one thread per recorded splat in dense warps instead of one thread per point of the cloud (a fallback kernel
//    with the reference's structure handles calls without such a list);
//  * the point gradient and its counter leave as ONE 16-byte vector atomic (x, y, z, count);
//  * pose and intrinsics gradients, which the reference adds with 7 + 14 same-address atomics per splat,
//    are reduced warp -> block in shared memory and leave as one atomic per component and block;
//  * the ghost-gradient stencil reads, per neighbour pixel, C values of the forward image and C of the upstream
//    gradient. From NCHW planes that is 2C scattered 4-byte reads in 2C different sectors; a preparation pass
//    (fused with the background / environment-map gradient) first interleaves both into one record per pixel
//    [I_0..I_C-1, G_0..G_C-1], so a neighbour costs one or two 32-byte sectors.
#include "common.cuh"

namespace adop {

// ------------------------------------------------------------------------------------------------------
// K4: preparation pass over the pyramid pixels of one view.
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
                                                              float* __restrict__ grad_env, int env_h, int env_w, bool env_interleaved)
{
    constexpr int RB = (2 * C + 3) & ~3;
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
// when the forward pass recorded no splat list (or the list overflowed).
template <int C, int MODEL>
__global__ void __launch_bounds__(kBlock) k_splat_backward_all(PointStreams pts, const ViewCam* __restrict__ camp, KernelParams kp, LayerTable lt,
                                                                BackwardTargets bt, const int* __restrict__ run_if_nonzero)
{
    constexpr int RB = (2 * C + 3) & ~3;
    if (run_if_nonzero && __ldg(run_if_nonzero) == 0) return;
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

// Inclusive prefix sums of the splat list's segment counts, in shared memory (every thread of the block takes part).
__device__ __forceinline__ int scan_segments(const int* __restrict__ header, int* s_prefix, int* s_warp)
{
    constexpr int PER = kVisibleSegments / kBlock;
    int local[PER];
    int sum = 0;
#pragma unroll
    for (int j = 0; j < PER; ++j) { sum += __ldg(header + threadIdx.x * PER + j); local[j] = sum; }
    int incl = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1)
    {
        int v = __shfl_up_sync(0xffffffffu, incl, o);
        if ((threadIdx.x & 31) >= o) incl += v;
    }
    if ((threadIdx.x & 31) == 31) s_warp[threadIdx.x >> 5] = incl;
    __syncthreads();
    int woff = 0;
    for (int k = 0; k < (int)(threadIdx.x >> 5); ++k) woff += s_warp[k];
    const int excl = woff + incl - sum;
#pragma unroll
    for (int j = 0; j < PER; ++j) s_prefix[threadIdx.x * PER + j] = excl + local[j];
    __syncthreads();
    return s_prefix[kVisibleSegments - 1];
}

// K5 (splat list): the backward pass over the (point, layer) splats that the blend kernel recorded, in dense warps, with
// no layer loop and no depth test (the forward pass already applied it, including the stop at a point's first failure).
// Two kernels, because one needs memory-level parallelism and the other registers:
//   k_splat_gather: per splat, the pixel's weight and record, the four neighbour records and the point's descriptor are
//                   requested at once (the pixel index comes with the list entry, nothing waits for a projection); it
//                   adds the descriptor gradient and stores the splat's image-space gradient in the entry. ~40 registers.
//   k_splat_chain:  per splat, re-projects the point with Jacobians and chains the stored gradient to the point, pose
//                   and intrinsics gradients. ~100 registers, almost no memory traffic.
__device__ __forceinline__ int4 list_entry(const VisibleList& vl, const int* s_prefix, int n_segments, int seg_cap, int t, size_t* where)
{
    int lo = 0, hi = n_segments - 1;
    while (lo < hi)
    {
        int mid = (lo + hi) >> 1;
        if (s_prefix[mid] > t) hi = mid; else lo = mid + 1;
    }
    const int before = lo ? s_prefix[lo - 1] : 0;
    *where = (size_t)lo * seg_cap + (t - before);
    return __ldg(vl.entries + *where);
}
constexpr int kNoStencil = 0x7fc00000;  // quiet NaN in the gradient slot: the splat has no ghost gradient

// (resident blocks per SM by channel count: the four neighbour records of the stencil are 8C floats that want registers)
template <int C>
__global__ void __launch_bounds__(kBlock, C <= 4 ? 4 : (C <= 8 ? 2 : 1)) k_splat_gather(PointStreams pts, KernelParams kp, LayerTable lt, BackwardTargets bt,
                                                            VisibleList vl, int want_geo)
{
    constexpr int RB = (2 * C + 3) & ~3;
    if (__ldg(vl.header + kVisibleSegments + 2) != 0) return;  // the list overflowed: k_splat_backward_all takes over
    __shared__ int s_prefix[kVisibleSegments];
    __shared__ int s_warp[kBlock / 32];
    const int work = scan_segments(vl.header, s_prefix, s_warp);
    const int n_segments = __ldg(vl.header + kVisibleSegments);
    const int seg_cap = __ldg(vl.header + kVisibleSegments + 1);
    const int stride = gridDim.x * blockDim.x;
    for (int t = blockIdx.x * blockDim.x + threadIdx.x; t < work; t += stride)
    {
        size_t where;
        const int4 e = list_entry(vl, s_prefix, n_segments, seg_cap, t, &where);
        const int i = (int)((unsigned)e.x & kSplatPointMask);
        const int l = (int)((unsigned)e.x >> kSplatLayerShift);
        const bool drop_out = point_dropped(kp, i);
        const bool point_grad = want_geo && ((kp.ghost_gradients && drop_out) || (!kp.ghost_gradients && !drop_out));
        const int w = lt.w[l], h = lt.h[l];
        const size_t pix = (size_t)e.y;
        const int py = e.y / w, px = e.y - py * w;
        const size_t rbase = (size_t)lt.rec_off[l] + pix;
        const int edge = min(min(px, py), min(w - 1 - px, h - 1 - py));
        const bool stencil = point_grad && edge > 2;
        const int ti = pts.index ? __ldg(pts.index + i) : i;
        const float wgt = __ldg(lt.weight[l] + pix);
        const bool want_dg = !drop_out && bt.grad_texture && wgt != 0.f;
        float2 g = make_float2(0.f, __int_as_float(kNoStencil));
        if (drop_out || wgt != 0.f)  // :473
        {
            if (want_dg)
            {
                float rc[RB], dg[C];
                load_record<C>(bt.records, rbase, rc);
                const float iw = 1.f / wgt;
#pragma unroll
                for (int c = 0; c < C; ++c) dg[c] = iw * rc[C + c];
                add_descriptor_gradient<C>(bt.grad_texture, bt.grad_texture_interleaved, bt.num_texels, ti, dg);
            }
            if (stencil)
            {
                const size_t nb[4] = {pix - 1, pix + 1, pix - (size_t)w, pix + (size_t)w};
                float rn[4][RB], T_p[C];
#pragma unroll
                for (int k = 0; k < 4; ++k) load_record<C>(bt.records, (size_t)lt.rec_off[l] + nb[k], rn[k]);
                load_descriptor<C>(bt.texture, bt.texture_interleaved, bt.num_texels, ti, T_p);
                V2 gg = stencil_gradient<C>(kp, T_p, rn, 0.f, lt.weight[l], lt.depth[l], nb);
                g = make_float2(gg.x, gg.y);
            }
        }
        // only the gradient half of the entry is written (the chain kernel reads the whole entry)
        reinterpret_cast<float2*>(vl.entries + where)[1] = g;
    }
}

template <int MODEL>
__global__ void __launch_bounds__(kBlock, 4) k_splat_chain(PointStreams pts, const ViewCam* __restrict__ camp, KernelParams kp,
                                                         LayerTable lt, BackwardTargets bt, VisibleList vl)
{
    if (__ldg(vl.header + kVisibleSegments + 2) != 0) return;
    const ViewCam& cam = *camp;
    __shared__ GeoShared<MODEL> s_geo;
    __shared__ int s_prefix[kVisibleSegments];
    __shared__ int s_warp[kBlock / 32];
    geo_shared_init(&s_geo);
    const int work = scan_segments(vl.header, s_prefix, s_warp);
    const int n_segments = __ldg(vl.header + kVisibleSegments);
    const int seg_cap = __ldg(vl.header + kVisibleSegments + 1);
    GeoAccum<MODEL> acc;
    acc.clear();
    const int stride = gridDim.x * blockDim.x;
    for (int t = blockIdx.x * blockDim.x + threadIdx.x; t < work; t += stride)
    {
        size_t where;
        const int4 e = list_entry(vl, s_prefix, n_segments, seg_cap, t, &where);
        if (e.w == kNoStencil) continue;
        const int i = (int)((unsigned)e.x & kSplatPointMask);
        const int l = (int)((unsigned)e.x >> kSplatLayerShift);
        FetchedPoint f = fetch_point(pts, i);
        V2 g; g.x = __int_as_float(e.z); g.y = __int_as_float(e.w);
        const float scale = __int_as_float((127 - l) << 23);  // 0.5^l, the same value l halvings give
        float gp[4] = {0.f, 0.f, 0.f, 0.f};
        if (chain_gradient<MODEL>(cam, kp, f, g, scale, gp, acc) && bt.grad_points)
            atomicAdd(bt.grad_points + i, make_float4(gp[0], gp[1], gp[2], gp[3]));
    }
    geo_block_reduce<MODEL>(&s_geo, acc, bt);
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
                                        const BackwardTargets& bt, float* grad_background, float* grad_env, int env_h, int env_w, bool env_interleaved,
                                        cudaStream_t st, const VisibleList& vl, int model)
{
    const int need = (pts.n + kBlock - 1) / kBlock;
    {
        static const int cap = resident_grid(k_prepare_backward<C>, 1ll << 40);
        unsigned total = lt.rec_off[kMaxLayers];
        int grid_px = (int)((total + kBlock - 1) / kBlock);
        if (grid_px > cap) grid_px = cap;
        ADOP_LAUNCH("k_prepare_backward", st, (k_prepare_backward<C><<<grid_px, kBlock, 0, st>>>(
                                                  lt, cam, kp, bt.background, const_cast<float*>(bt.records), grad_background,
                                                  grad_env, env_h, env_w, env_interleaved)));
    }
    // With a splat list the two dense kernels run; the all-points kernel is launched behind them and returns at once
    // unless the list's overflow flag is set (decided on the device, no host round trip). The debug stencil rule
    // (test_backward_mode 4) needs the point's depth next to its neighbours' and always takes the all-points kernel.
    const bool use_list = vl.header && kp.test_backward_mode != 4;
    const int* flag = use_list ? vl.header + kVisibleSegments + 2 : nullptr;
    const int want_geo = (bt.grad_points || bt.grad_pose || bt.grad_intrinsics) ? 1 : 0;
    if (use_list)
    {
        static const int gg = resident_grid(k_splat_gather<C>, 1ll << 40);
        ADOP_LAUNCH("k_splat_gather", st, (k_splat_gather<C><<<gg, kBlock, 0, st>>>(pts, kp, lt, bt, vl, want_geo)));
        if (want_geo)
        {
            if (model == kPinholeDistortion)
            {
                static const int g = resident_grid(k_splat_chain<kPinholeDistortion>, 1ll << 40);
                ADOP_LAUNCH("k_splat_chain", st, (k_splat_chain<kPinholeDistortion><<<g, kBlock, 0, st>>>(pts, cam, kp, lt, bt, vl)));
            }
            else
            {
                static const int g = resident_grid(k_splat_chain<kOcam>, 1ll << 40);
                ADOP_LAUNCH("k_splat_chain", st, (k_splat_chain<kOcam><<<g, kBlock, 0, st>>>(pts, cam, kp, lt, bt, vl)));
            }
        }
    }
    // Behind a splat list this launch is almost always a no-op that only reads the overflow flag, so it gets one block
    // per SM (an empty launch costs by its block count); without a list it is the backward pass and fills the GPU.
    const int fallback_cap = use_list ? sm_count() : (1 << 30);
    if (model == kPinholeDistortion)
    {
        static const int g = resident_grid(k_splat_backward_all<C, kPinholeDistortion>, 1ll << 40);
        int grid = need < g ? (need < 1 ? 1 : need) : g;
        if (grid > fallback_cap) grid = fallback_cap;
        ADOP_LAUNCH("k_splat_backward_all", st, (k_splat_backward_all<C, kPinholeDistortion><<<grid, kBlock, 0, st>>>(pts, cam, kp, lt, bt, flag)));
    }
    else
    {
        static const int g = resident_grid(k_splat_backward_all<C, kOcam>, 1ll << 40);
        int grid = need < g ? (need < 1 ? 1 : need) : g;
        if (grid > fallback_cap) grid = fallback_cap;
        ADOP_LAUNCH("k_splat_backward_all", st, (k_splat_backward_all<C, kOcam><<<grid, kBlock, 0, st>>>(pts, cam, kp, lt, bt, flag)));
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
        // the list's geometry (segments in use, entries per segment) sits in its header, written by the forward pass
        VisibleList vl = make_visible_list(const_cast<int32_t*>(io->visible_list), N, b, 1);
        adop_status r;
        switch (C)
        {
            case 3: r = launch_view_backward<3>(pts, cam, kp, lt, bt, io->grad_background, ge, s->env_h, s->env_w, env_inter, st, vl, views[b].camera_model); break;
            case 4: r = launch_view_backward<4>(pts, cam, kp, lt, bt, io->grad_background, ge, s->env_h, s->env_w, env_inter, st, vl, views[b].camera_model); break;
            case 8: r = launch_view_backward<8>(pts, cam, kp, lt, bt, io->grad_background, ge, s->env_h, s->env_w, env_inter, st, vl, views[b].camera_model); break;
            case 16: r = launch_view_backward<16>(pts, cam, kp, lt, bt, io->grad_background, ge, s->env_h, s->env_w, env_inter, st, vl, views[b].camera_model); break;
            default: return ADOP_ERR_UNSUPPORTED;
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
