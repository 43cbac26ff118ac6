// Pose update and the fused photometric tonemapper for sm_100a.
//  * adop_apply_tangent      <- ApplyTangent / ApplyTangentToPose (darglein/ADOP src/lib/rendering/PointRenderer.cu:1646-1665)
//  * adop_tonemap_forward/backward <- NeuralCameraImpl::forward (src/lib/models/NeuralCamera.cpp:258-335) with
//    VignetteNetImpl::forward (:22-42) and CameraResponseNetImpl::forward (:87-135). The reference runs about
//    fifteen elementwise / grid_sample kernels, each a full image read and write; here one kernel reads x once
//    and writes the result once (forward), or reads x and the upstream gradient and writes grad_x (backward),
//    with the parameter gradients reduced in shared memory per block.
#include "common.cuh"

namespace adop {

constexpr int kMaxResponseBins = 1024;

__global__ void k_apply_tangent(double* tangent, double* pose, int n)
{
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    se3_exp_left_multiply(tangent + (size_t)i * 6, pose + (size_t)i * 8);
#pragma unroll
    for (int k = 0; k < 6; ++k) tangent[(size_t)i * 6 + k] = 0.0;
}

struct ToneArgs
{
    int B, H, W, K;
    float aspect, leak;
    const int* frame_index;
    const float* exposure;
    const float* white_balance;
    const float* vignette;
    const float* uv;
    const float* response;
};

// VEC pixels per thread: 4 (128-bit loads and stores of every plane) when the plane size is a multiple of 4, else 1.
template <int VEC>
__device__ __forceinline__ void load_vec(const float* __restrict__ p, float* v)
{
    if (VEC == 4) { float4 a = __ldcs(reinterpret_cast<const float4*>(p)); v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; }
    else v[0] = __ldcs(p);
}
template <int VEC>
__device__ __forceinline__ void store_vec(float* __restrict__ p, const float* v)
{
    if (VEC == 4) __stcs(reinterpret_cast<float4*>(p), make_float4(v[0], v[1], v[2], v[3]));
    else __stcs(p, v[0]);
}
// vignette geometry of VEC consecutive pixels starting at pix; vg = the five vignette parameters (polynomial, centre).
// Default coordinates: u = 2 x / (W - 1) - 1 as x times a precomputed step (32-bit pixel arithmetic: the entry points
// reject planes of 2^31 pixels or more).
template <int VEC>
__device__ __forceinline__ void tone_geometry(const ToneArgs& a, const float* vg, int b, size_t pix, size_t plane, float* du, float* dv, float* r2,
                                              float* fac)
{
    float u0[VEC], v0[VEC];
    if (a.uv)
    {
        load_vec<VEC>(a.uv + ((size_t)b * 2 + 0) * plane + pix, u0);
        load_vec<VEC>(a.uv + ((size_t)b * 2 + 1) * plane + pix, v0);
    }
    else
    {
        const float step_u = 2.0f / (float)(a.W - 1), step_v = 2.0f / (float)(a.H - 1);
        unsigned yy = (unsigned)pix / (unsigned)a.W, xx = (unsigned)pix - yy * (unsigned)a.W;
#pragma unroll
        for (int k = 0; k < VEC; ++k)
        {
            u0[k] = fmaf((float)xx, step_u, -1.0f);
            v0[k] = fmaf((float)yy, step_v, -1.0f);
            if (++xx == (unsigned)a.W) { xx = 0; ++yy; }
        }
    }
#pragma unroll
    for (int k = 0; k < VEC; ++k)
    {
        du[k] = (u0[k] - vg[3]) * a.aspect; dv[k] = v0[k] - vg[4];
        r2[k] = fmaf(du[k], du[k], dv[k] * dv[k]);
        fac[k] = fmaf(fmaf(fmaf(vg[2], r2[k], vg[1]), r2[k], vg[0]), r2[k], 1.0f);
    }
}

// grid: (blocks per image, B); a block walks over many chunks of 256 x VEC pixels, so the curve is staged once per block
template <int VEC>
__global__ void __launch_bounds__(256) k_tonemap_forward(ToneArgs a, const float* __restrict__ x, float* __restrict__ out)
{
    extern __shared__ float s_lut[];  // [3,K]
    const int K = a.K;
    for (int k = threadIdx.x; k < 3 * K; k += blockDim.x) s_lut[k] = a.response[k];
    __syncthreads();
    const int b = blockIdx.y;
    const size_t plane = (size_t)a.H * a.W;
    const int fi = a.frame_index ? a.frame_index[b] : 0;
    const float ef = a.exposure ? 1.0f / exp2f(a.exposure[fi]) : 1.0f;
    const float Km1 = (float)(K - 1);
    float wb[3];
#pragma unroll
    for (int c = 0; c < 3; ++c) wb[c] = a.white_balance ? a.white_balance[(size_t)fi * 3 + c] : 1.0f;
    float vg[5] = {0.f, 0.f, 0.f, 0.f, 0.f};
    if (a.vignette)
#pragma unroll
        for (int k = 0; k < 5; ++k) vg[k] = a.vignette[k];
    const float* xb = x + (size_t)b * 3 * plane;
    float* ob = out + (size_t)b * 3 * plane;
    const size_t per_chunk = (size_t)blockDim.x * VEC;
    for (size_t pix = (size_t)blockIdx.x * per_chunk + (size_t)threadIdx.x * VEC; pix < plane; pix += (size_t)gridDim.x * per_chunk)
    {
        float xin[3][VEC];
#pragma unroll
        for (int c = 0; c < 3; ++c) load_vec<VEC>(xb + c * plane + pix, xin[c]);
        float du[VEC], dv[VEC], r2[VEC], fac[VEC];
#pragma unroll
        for (int k = 0; k < VEC; ++k) fac[k] = 1.f;
        if (a.vignette) tone_geometry<VEC>(a, vg, b, pix, plane, du, dv, r2, fac);
#pragma unroll
        for (int c = 0; c < 3; ++c)
        {
            float o[VEC];
#pragma unroll
            for (int k = 0; k < VEC; ++k)
            {
                float v = xin[c][k] * ef;
                v = wb[c] * v;
                v = fac[k] * v;
                if (a.response)
                {
                    float leak_add = 0.f;
                    if (a.leak > 0.f)
                    {
                        if (v < 0.f) leak_add = v * a.leak;
                        // reciprocal square root of the hardware (2 ulp): the soft knee above 1 needs no correctly rounded division
                        if (v > 1.f) leak_add = fmaf(-a.leak, rsqrtf(fabsf(v) + 1e-4f), a.leak);
                    }
                    const float t = fminf(fmaxf(v, 0.f), 1.f) * Km1;
                    const int i0 = (int)t;  // t >= 0: truncation is the floor
                    const int i1 = i0 + 1 < K ? i0 + 1 : K - 1;
                    const float fr = t - (float)i0;
                    o[k] = s_lut[c * K + i0] * (1.0f - fr) + s_lut[c * K + i1] * fr + leak_add;
                }
                else
                    o[k] = fminf(fmaxf(v, 0.f), 1.f);
            }
            store_vec<VEC>(ob + c * plane + pix, o);
        }
    }
}

struct ToneGradPtrs
{
    float* grad_x;
    float* grad_exposure;
    float* grad_white_balance;
    float* grad_vignette;
    float* grad_response;
};

// The response-curve gradient is a histogram-like scatter: two bins per pixel and channel. Shared-memory atomicAdd on
// float is a compare-and-swap loop and cost more than the rest of the kernel together; the integer one is a single
// instruction. So the terms are summed in scaled fixed point, and every WARP keeps a histogram pair of its own, so that no
// step of the pixel loop needs a block-wide barrier:
//   1. a warp takes 32 x VEC consecutive pixels at a time, finds M = max |upstream gradient| among them (one
//      warp-wide reduction) and works with scale = 2^(18 - e), e = the exponent of the largest M since its last flush:
//      every term |g * weight * scale| < 2^19;
//   2. terms are rounded to nearest and added with integer atomics to the warp's integer histogram;
//   3. a flush converts the warp's integer bins back (exactly: a power-of-two factor) into the warp's float histogram. It
//      happens when a larger exponent turns up, and after kFlushEvery rounds (a bin takes at most 32 x VEC terms per round,
//      so 2^19 x 128 x 16 < 2^31 never overflows);
//   4. at the end the block adds its warps' float histograms up and sends one atomic per touched bin to global memory.
// A term is off by at most 2^-19 of the largest gradient among the at most kFlushEvery x 32 x VEC neighbouring pixels
// that share a scale, unbiased; rounds whose M is not finite or is below 2^-100 take float atomics on the warp's float
// histogram instead, so NaN / Inf gradients still show up in the result.
constexpr int kFlushEvery = 16;
template <int VEC>
__global__ void __launch_bounds__(256, 3) k_tonemap_backward(ToneArgs a, const float* __restrict__ x, const float* __restrict__ grad_out,
                                                           ToneGradPtrs g)
{
    extern __shared__ float smem[];  // lut [3,K], slopes [3,K], per warp: float histogram [3,K], integer histogram [3,K]
    const int K = a.K, K3 = 3 * a.K;
    const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* s_lut = smem;
    float* s_slope = smem + K3;
    float* s_acc_all = smem + 2 * K3;
    float* s_acc = s_acc_all + warp * K3;
    int* s_int = reinterpret_cast<int*>(s_acc_all + warps * K3) + warp * K3;
    __shared__ float s_small[9];  // exposure, wb[3], vignette[5]
    const bool want_resp = g.grad_response && a.response;
    const float Km1 = (float)(K - 1);
    for (int k = threadIdx.x; k < K3; k += blockDim.x) s_lut[k] = a.response[k];
    if (threadIdx.x < 9) s_small[threadIdx.x] = 0.f;
    __syncthreads();
    // slope of the curve in bin i (0 in the last one, where both taps are the same entry)
    for (int k = threadIdx.x; k < K3; k += blockDim.x)
    {
        const int i = k % K;
        s_slope[k] = i + 1 < K ? (s_lut[k + 1] - s_lut[k]) * Km1 : 0.f;
    }
    if (want_resp)
        for (int k = lane; k < K3; k += 32) { s_acc[k] = 0.f; s_int[k] = 0; }
    __syncthreads();
    const int b = blockIdx.y;
    const size_t plane = (size_t)a.H * a.W;
    const int fi = a.frame_index ? a.frame_index[b] : 0;
    const float ef = a.exposure ? 1.0f / exp2f(a.exposure[fi]) : 1.0f;
    float wb[3], wbef[3];
#pragma unroll
    for (int c = 0; c < 3; ++c) { wb[c] = a.white_balance ? a.white_balance[(size_t)fi * 3 + c] : 1.0f; wbef[c] = wb[c] * ef; }
    float vg[5] = {0.f, 0.f, 0.f, 0.f, 0.f};
    if (a.vignette)
#pragma unroll
        for (int k = 0; k < 5; ++k) vg[k] = a.vignette[k];
    const float* xb = x + (size_t)b * 3 * plane;
    const float* gob = grad_out + (size_t)b * 3 * plane;
    float* gxb = g.grad_x ? g.grad_x + (size_t)b * 3 * plane : nullptr;
    float gPre = 0.f, gWB[3] = {0.f, 0.f, 0.f}, gV[5] = {0.f, 0.f, 0.f, 0.f, 0.f};
    // a warp walks over many rounds of its image, so the parameter gradients leave it once; the trip count is the same
    // for all lanes of a warp (the loop holds warp-wide votes)
    const size_t per_round = (size_t)32 * VEC;
    const size_t rounds = (plane + per_round - 1) / per_round;
    int e_cur = 0, since = 0;  // exponent of the warp's current scale, rounds since its last flush (warp-uniform)
    auto flush = [&]() {
        __syncwarp();
        const float inv = __int_as_float((127 - 18 + e_cur) << 23);  // 1 / scale, exact
        for (int k = lane; k < K3; k += 32)
        {
            const int q = s_int[k];
            if (q != 0) { s_acc[k] += (float)q * inv; s_int[k] = 0; }
        }
        __syncwarp();
        since = 0;
    };
    for (size_t round = (size_t)blockIdx.x * warps + warp; round < rounds; round += (size_t)gridDim.x * warps)
    {
        const size_t pix = round * per_round + (size_t)lane * VEC;
        const bool live = pix < plane;
        // all six loads of the round are requested before anything waits
        float go[3][VEC], xall[3][VEC];
#pragma unroll
        for (int c = 0; c < 3; ++c)
        {
#pragma unroll
            for (int k = 0; k < VEC; ++k) { go[c][k] = 0.f; xall[c][k] = 0.f; }
            if (live)
            {
                load_vec<VEC>(gob + c * plane + pix, go[c]);
                load_vec<VEC>(xb + c * plane + pix, xall[c]);
            }
        }
        float du[VEC], dv[VEC], r2[VEC], fac[VEC];
#pragma unroll
        for (int k = 0; k < VEC; ++k) { fac[k] = 1.f; du[k] = dv[k] = r2[k] = 0.f; }
        if (a.vignette && live) tone_geometry<VEC>(a, vg, b, pix, plane, du, dv, r2, fac);
        float scale = 0.f;  // 0: this round adds to the float histogram directly
        if (want_resp)
        {
            // the bit patterns of non-negative floats order like the floats, with the NaNs above infinity: an integer
            // maximum keeps a NaN anywhere in the round visible (fmaxf would drop it)
            unsigned mi = 0u;
#pragma unroll
            for (int c = 0; c < 3; ++c)
#pragma unroll
                for (int k = 0; k < VEC; ++k) mi = max(mi, __float_as_uint(go[c][k]) & 0x7fffffffu);
            const float M = __uint_as_float(__reduce_max_sync(0xffffffffu, mi));
            const int e = (int)((__float_as_uint(M) >> 23) & 0xffu) - 127;
            if (M <= 3.0e38f && e >= -100)
            {
                if (since > 0 && (e > e_cur || since >= kFlushEvery)) flush();
                if (since == 0) e_cur = e;
                scale = __int_as_float((127 + 18 - e_cur) << 23);
                ++since;
            }
        }
        if (live)
        {
            float gsum[VEC];  // sum over the channels of (gradient behind the vignette factor) x (value before it)
#pragma unroll
            for (int k = 0; k < VEC; ++k) gsum[k] = 0.f;
#pragma unroll
            for (int c = 0; c < 3; ++c)
            {
                float gx[VEC];
                const float* xin = xall[c];
                // neighbouring pixels mostly fall into the same pair of bins: their two weights are added up in
                // registers and reach shared memory once per run
                int run_i0 = -1;
                float run_w0 = 0.f, run_w1 = 0.f;
                auto put = [&]() {
                    const int i1 = run_i0 + 1 < K ? run_i0 + 1 : K - 1;
                    if (scale != 0.f)
                    {
                        atomicAdd(&s_int[c * K + run_i0], __float2int_rn(run_w0 * scale));
                        atomicAdd(&s_int[c * K + i1], __float2int_rn(run_w1 * scale));
                    }
                    else
                    {
                        atomicAdd(&s_acc[c * K + run_i0], run_w0);
                        atomicAdd(&s_acc[c * K + i1], run_w1);
                    }
                };
#pragma unroll
                for (int k = 0; k < VEC; ++k)
                {
                    const float xe = xin[k] * ef;
                    const float pre = wb[c] * xe;
                    const float v = fac[k] * pre;
                    const bool inside = v > 0.f && v < 1.f;
                    float dv_out;
                    if (a.response)
                    {
                        float dleak = 0.f;
                        if (a.leak > 0.f)
                        {
                            if (v < 0.f) dleak = a.leak;
                            if (v > 1.f) { const float r = rsqrtf(fabsf(v) + 1e-4f); dleak = 0.5f * a.leak * (r * r * r); }
                        }
                        const float t = fminf(fmaxf(v, 0.f), 1.f) * Km1;
                        const int i0 = (int)t;  // t >= 0: truncation is the floor
                        const float fr = t - (float)i0;
                        if (want_resp)
                        {
                            if (i0 != run_i0)
                            {
                                if (run_i0 >= 0) put();
                                run_i0 = i0; run_w0 = 0.f; run_w1 = 0.f;
                            }
                            run_w0 = fmaf(go[c][k], 1.0f - fr, run_w0);
                            run_w1 = fmaf(go[c][k], fr, run_w1);
                        }
                        dv_out = (inside ? s_slope[c * K + i0] : 0.f) + dleak;
                    }
                    else
                        dv_out = inside ? 1.f : 0.f;
                    const float gv = go[c][k] * dv_out;
                    gsum[k] = fmaf(gv, pre, gsum[k]);
                    const float gpre = gv * fac[k];
                    gWB[c] = fmaf(gpre, xe, gWB[c]);
                    gPre = fmaf(gpre, pre, gPre);
                    gx[k] = gpre * wbef[c];
                }
                if (run_i0 >= 0) put();
                if (gxb) store_vec<VEC>(gxb + c * plane + pix, gx);
            }
            if (a.vignette)
            {
#pragma unroll
                for (int k = 0; k < VEC; ++k)
                {
                    const float r4 = r2[k] * r2[k];
                    gV[0] = fmaf(gsum[k], r2[k], gV[0]); gV[1] = fmaf(gsum[k], r4, gV[1]); gV[2] = fmaf(gsum[k], r4 * r2[k], gV[2]);
                    const float gr2 = gsum[k] * fmaf(3.f * vg[2], r4, fmaf(2.f * vg[1], r2[k], vg[0]));
                    gV[3] = fmaf(gr2, -2.f * a.aspect * du[k], gV[3]);
                    gV[4] = fmaf(gr2, -2.f * dv[k], gV[4]);
                }
            }
        }
    }
    if (want_resp && since > 0) flush();
    const bool lane0 = lane == 0;
    float r;
    // exposure: x * 2^-e, so d/de = -ln 2 times the sum of (gradient at the exposed value) x (exposed value)
    r = warp_sum(gPre); if (lane0) atomicAdd(&s_small[0], r * -0.69314718056f);
#pragma unroll
    for (int c = 0; c < 3; ++c) { r = warp_sum(gWB[c]); if (lane0) atomicAdd(&s_small[1 + c], r); }
#pragma unroll
    for (int k = 0; k < 5; ++k) { r = warp_sum(gV[k]); if (lane0) atomicAdd(&s_small[4 + k], r); }
    __syncthreads();
    if (threadIdx.x == 0 && g.grad_exposure && a.exposure) atomicAdd(g.grad_exposure + fi, s_small[0]);
    if (threadIdx.x >= 1 && threadIdx.x < 4 && g.grad_white_balance && a.white_balance)
        atomicAdd(g.grad_white_balance + (size_t)fi * 3 + (threadIdx.x - 1), s_small[threadIdx.x]);
    if (threadIdx.x >= 4 && threadIdx.x < 9 && g.grad_vignette && a.vignette)
        atomicAdd(g.grad_vignette + (threadIdx.x - 4), s_small[threadIdx.x]);
    if (want_resp)
        for (int k = threadIdx.x; k < K3; k += blockDim.x)
        {
            float sum = 0.f;
            for (int w = 0; w < warps; ++w) sum += s_acc_all[w * K3 + k];
            if (sum != 0.f) atomicAdd(g.grad_response + k, sum);
        }
}

static adop_status make_tone_args(const adop_tonemap_params* p, ToneArgs* a)
{
    if (!p || p->batch <= 0 || p->height <= 0 || p->width <= 0) return ADOP_ERR_INVALID_ARGUMENT;
    if (p->response && (p->response_bins < 2)) return ADOP_ERR_INVALID_ARGUMENT;
    if (p->response && p->response_bins > kMaxResponseBins) return ADOP_ERR_SIZE_LIMIT;
    if (p->vignette && (p->vignette_image_w <= 0 || p->vignette_image_h <= 0)) return ADOP_ERR_INVALID_ARGUMENT;
    if (p->batch > 65535 || (size_t)p->height * (size_t)p->width >= ((size_t)1 << 31)) return ADOP_ERR_SIZE_LIMIT;
    a->B = p->batch; a->H = p->height; a->W = p->width;
    a->K = p->response ? p->response_bins : 0;
    a->aspect = p->vignette ? (float)p->vignette_image_w / (float)p->vignette_image_h : 1.f;
    a->leak = p->leak;
    a->frame_index = p->frame_index; a->exposure = p->exposure; a->white_balance = p->white_balance;
    a->vignette = p->vignette; a->uv = p->uv; a->response = p->response;
    return ADOP_OK;
}

}  // namespace adop

using namespace adop;

extern "C" adop_status adop_apply_tangent(double* tangent, double* pose, int32_t n, void* stream)
{
    if (!tangent || !pose || n < 0) return ADOP_ERR_INVALID_ARGUMENT;
    if (n == 0) return ADOP_OK;
    k_apply_tangent<<<(n + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(tangent, pose, n);
    ADOP_CUDA_TRY(cudaGetLastError());
    return ADOP_OK;
}

extern "C" adop_status adop_tonemap_forward(const adop_tonemap_params* p, const float* x, float* out, void* stream)
{
    ToneArgs a;
    adop_status s = make_tone_args(p, &a);
    if (s != ADOP_OK) return s;
    if (!x || !out) return ADOP_ERR_INVALID_ARGUMENT;
    size_t plane = (size_t)a.H * a.W;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool vec = plane % 4 == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(a.uv)) & 15) == 0;
    // as many blocks as stay resident at once, shared out over the images
    const size_t chunks = vec ? (plane / 4 + 255) / 256 : (plane + 255) / 256;
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k_tonemap_forward<4>, 256, sizeof(float) * 3 * a.K) != cudaSuccess || per_sm < 1)
        per_sm = 1;
    const size_t per_image = (size_t)((sm_count() * per_sm + a.B - 1) / a.B);
    dim3 grid((unsigned)(chunks < per_image ? chunks : per_image), (unsigned)a.B);
    if (vec) ADOP_LAUNCH("k_tonemap_forward", st, (k_tonemap_forward<4><<<grid, 256, sizeof(float) * 3 * a.K, st>>>(a, x, out)));
    else ADOP_LAUNCH("k_tonemap_forward", st, (k_tonemap_forward<1><<<grid, 256, sizeof(float) * 3 * a.K, st>>>(a, x, out)));
    ADOP_CUDA_TRY(cudaGetLastError());
    return ADOP_OK;
}

extern "C" adop_status adop_tonemap_backward(const adop_tonemap_params* p, const float* x, const float* grad_out,
                                             adop_tonemap_grads* g, void* stream)
{
    ToneArgs a;
    adop_status s = make_tone_args(p, &a);
    if (s != ADOP_OK) return s;
    if (!x || !grad_out || !g) return ADOP_ERR_INVALID_ARGUMENT;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (!g->accumulate)
    {
        if (g->num_frames <= 0 && (g->grad_exposure || g->grad_white_balance)) return ADOP_ERR_INVALID_ARGUMENT;
        if (g->grad_exposure) ADOP_CUDA_TRY(cudaMemsetAsync(g->grad_exposure, 0, sizeof(float) * g->num_frames, st));
        if (g->grad_white_balance) ADOP_CUDA_TRY(cudaMemsetAsync(g->grad_white_balance, 0, sizeof(float) * 3 * g->num_frames, st));
        if (g->grad_vignette) ADOP_CUDA_TRY(cudaMemsetAsync(g->grad_vignette, 0, sizeof(float) * 5, st));
        if (g->grad_response && a.K > 0) ADOP_CUDA_TRY(cudaMemsetAsync(g->grad_response, 0, sizeof(float) * 3 * a.K, st));
    }
    ToneGradPtrs gp;
    gp.grad_x = g->grad_x; gp.grad_exposure = g->grad_exposure; gp.grad_white_balance = g->grad_white_balance;
    gp.grad_vignette = g->grad_vignette; gp.grad_response = g->grad_response;
    size_t plane = (size_t)a.H * a.W;
    // fewer warps per block when the curve has many bins: every warp keeps two histograms of its own
    const int threads = a.K <= 256 ? 256 : (a.K <= 512 ? 128 : 64);
    // lut + slopes, and per warp a float and an integer histogram
    const size_t smem_bytes = sizeof(float) * 3 * a.K * (2 + 2 * (threads / 32));
    if (smem_bytes > 40 * 1024)
    {
        ADOP_CUDA_TRY(cudaFuncSetAttribute(k_tonemap_backward<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes));
        ADOP_CUDA_TRY(cudaFuncSetAttribute(k_tonemap_backward<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes));
    }
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k_tonemap_backward<4>, threads, smem_bytes) != cudaSuccess || per_sm < 1)
        per_sm = 1;
    // about as many blocks as stay resident at once, shared out over the images
    const size_t per_image = (size_t)((sm_count() * per_sm + a.B - 1) / a.B);
    const bool vec = plane % 4 == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(grad_out) |
                                         reinterpret_cast<uintptr_t>(g->grad_x) | reinterpret_cast<uintptr_t>(a.uv)) & 15) == 0;
    const size_t rounds = vec ? (plane / 4 + 31) / 32 : (plane + 31) / 32;
    const size_t blocks_needed = (rounds + threads / 32 - 1) / (threads / 32);
    dim3 grid((unsigned)(blocks_needed < per_image ? blocks_needed : per_image), (unsigned)a.B);
    if (vec) ADOP_LAUNCH("k_tonemap_backward", st, (k_tonemap_backward<4><<<grid, threads, smem_bytes, st>>>(a, x, grad_out, gp)));
    else ADOP_LAUNCH("k_tonemap_backward", st, (k_tonemap_backward<1><<<grid, threads, smem_bytes, st>>>(a, x, grad_out, gp)));
    ADOP_CUDA_TRY(cudaGetLastError());
    return ADOP_OK;
}
