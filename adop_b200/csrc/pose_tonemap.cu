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

__device__ __forceinline__ void tone_uv(const ToneArgs& a, int b, int xx, int yy, size_t pix, size_t plane, float* u0, float* v0)
{
    if (a.uv)
    {
        *u0 = __ldg(a.uv + ((size_t)b * 2 + 0) * plane + pix);
        *v0 = __ldg(a.uv + ((size_t)b * 2 + 1) * plane + pix);
    }
    else
    {
        *u0 = 2.0f * ((float)xx / (float)(a.W - 1)) - 1.0f;
        *v0 = 2.0f * ((float)yy / (float)(a.H - 1)) - 1.0f;
    }
}

// grid: (ceil(H*W / block), B)
__global__ void __launch_bounds__(256) k_tonemap_forward(ToneArgs a, const float* __restrict__ x, float* __restrict__ out)
{
    extern __shared__ float s_lut[];  // [3,K]
    for (int k = threadIdx.x; k < 3 * a.K; k += blockDim.x) s_lut[k] = a.response[k];
    __syncthreads();
    const int b = blockIdx.y;
    const size_t plane = (size_t)a.H * a.W;
    const size_t pix = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (pix >= plane) return;
    const int fi = a.frame_index ? a.frame_index[b] : 0;
    const float ef = a.exposure ? 1.0f / exp2f(a.exposure[fi]) : 1.0f;
    float fac = 1.f;
    if (a.vignette)
    {
        int yy = (int)(pix / a.W), xx = (int)(pix - (size_t)yy * a.W);
        float u0, v0;
        tone_uv(a, b, xx, yy, pix, plane, &u0, &v0);
        float du = (u0 - a.vignette[3]) * a.aspect, dv = v0 - a.vignette[4];
        float r2 = du * du + dv * dv, r4 = r2 * r2, r6 = r4 * r2;
        fac = 1.f + a.vignette[0] * r2 + a.vignette[1] * r4 + a.vignette[2] * r6;
    }
#pragma unroll
    for (int c = 0; c < 3; ++c)
    {
        const float wb = a.white_balance ? a.white_balance[(size_t)fi * 3 + c] : 1.0f;
        float v = __ldcs(x + ((size_t)b * 3 + c) * plane + pix) * ef;
        v = wb * v;
        v = fac * v;
        float o;
        if (a.response)
        {
            float leak_add = 0.f;
            if (a.leak > 0.f)
            {
                if (v < 0.f) leak_add = v * a.leak;
                if (v > 1.f) leak_add = -a.leak / sqrtf(fabsf(v) + 1e-4f) + a.leak;
            }
            float t = fminf(fmaxf(v, 0.f), 1.f) * (float)(a.K - 1);
            int i0 = (int)floorf(t);
            int i1 = i0 + 1 < a.K ? i0 + 1 : a.K - 1;
            float fr = t - (float)i0;
            o = s_lut[c * a.K + i0] * (1.0f - fr) + s_lut[c * a.K + i1] * fr + leak_add;
        }
        else
            o = fminf(fmaxf(v, 0.f), 1.f);
        __stcs(out + ((size_t)b * 3 + c) * plane + pix, o);
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

__global__ void __launch_bounds__(256) k_tonemap_backward(ToneArgs a, const float* __restrict__ x, const float* __restrict__ grad_out,
                                                           ToneGradPtrs g)
{
    extern __shared__ float smem[];  // lut [3,K], then response gradient [3,K]
    float* s_lut = smem;
    float* s_gr = smem + 3 * a.K;
    __shared__ float s_small[9];  // exposure, wb[3], vignette[5]
    for (int k = threadIdx.x; k < 3 * a.K; k += blockDim.x) { s_lut[k] = a.response[k]; s_gr[k] = 0.f; }
    if (threadIdx.x < 9) s_small[threadIdx.x] = 0.f;
    __syncthreads();
    const int b = blockIdx.y;
    const size_t plane = (size_t)a.H * a.W;
    const size_t pix = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const bool live = pix < plane;
    const int fi = a.frame_index ? a.frame_index[b] : 0;
    const float ef = a.exposure ? 1.0f / exp2f(a.exposure[fi]) : 1.0f;
    const float ln2 = 0.69314718056f;
    float gE = 0.f, gWB[3] = {0.f, 0.f, 0.f}, gV[5] = {0.f, 0.f, 0.f, 0.f, 0.f};
    if (live)
    {
        float fac = 1.f, du = 0.f, dv = 0.f, r2 = 0.f, r4 = 0.f, r6 = 0.f;
        if (a.vignette)
        {
            int yy = (int)(pix / a.W), xx = (int)(pix - (size_t)yy * a.W);
            float u0, v0;
            tone_uv(a, b, xx, yy, pix, plane, &u0, &v0);
            du = (u0 - a.vignette[3]) * a.aspect; dv = v0 - a.vignette[4];
            r2 = du * du + dv * dv; r4 = r2 * r2; r6 = r4 * r2;
            fac = 1.f + a.vignette[0] * r2 + a.vignette[1] * r4 + a.vignette[2] * r6;
        }
#pragma unroll
        for (int c = 0; c < 3; ++c)
        {
            const float wb = a.white_balance ? a.white_balance[(size_t)fi * 3 + c] : 1.0f;
            const float xin = __ldcs(x + ((size_t)b * 3 + c) * plane + pix);
            const float go = __ldcs(grad_out + ((size_t)b * 3 + c) * plane + pix);
            const float pre = wb * (xin * ef);
            const float v = fac * pre;
            float dv_out;
            if (a.response)
            {
                float dleak = 0.f;
                if (a.leak > 0.f)
                {
                    if (v < 0.f) dleak = a.leak;
                    if (v > 1.f) { float q = fabsf(v) + 1e-4f; dleak = 0.5f * a.leak / (q * sqrtf(q)); }
                }
                float t = fminf(fmaxf(v, 0.f), 1.f) * (float)(a.K - 1);
                int i0 = (int)floorf(t);
                int i1 = i0 + 1 < a.K ? i0 + 1 : a.K - 1;
                float fr = t - (float)i0;
                if (g.grad_response)
                {
                    atomicAdd(&s_gr[c * a.K + i0], go * (1.0f - fr));
                    atomicAdd(&s_gr[c * a.K + i1], go * fr);
                }
                float inside = (v > 0.f && v < 1.f) ? 1.f : 0.f;
                dv_out = inside * (s_lut[c * a.K + i1] - s_lut[c * a.K + i0]) * (float)(a.K - 1) + dleak;
            }
            else
                dv_out = (v > 0.f && v < 1.f) ? 1.f : 0.f;
            const float gv = go * dv_out;
            if (a.vignette)
            {
                float gfac = gv * pre;
                gV[0] += gfac * r2; gV[1] += gfac * r4; gV[2] += gfac * r6;
                float gr2 = gfac * (a.vignette[0] + 2.f * a.vignette[1] * r2 + 3.f * a.vignette[2] * r4);
                gV[3] += gr2 * 2.f * du * (-a.aspect);
                gV[4] += gr2 * 2.f * dv * (-1.f);
            }
            const float gpre = gv * fac;
            gWB[c] = gpre * (xin * ef);
            const float gxe = gpre * wb;
            gE += gxe * xin * ef * (-ln2);
            if (g.grad_x) __stcs(g.grad_x + ((size_t)b * 3 + c) * plane + pix, gxe * ef);
        }
    }
    const bool lane0 = (threadIdx.x & 31) == 0;
    float r;
    r = warp_sum(gE); if (lane0) atomicAdd(&s_small[0], r);
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
    if (g.grad_response && a.response)
        for (int k = threadIdx.x; k < 3 * a.K; k += blockDim.x)
            if (s_gr[k] != 0.f) atomicAdd(g.grad_response + k, s_gr[k]);
}

static adop_status make_tone_args(const adop_tonemap_params* p, ToneArgs* a)
{
    if (!p || p->batch <= 0 || p->height <= 0 || p->width <= 0) return ADOP_ERR_INVALID_ARGUMENT;
    if (p->response && (p->response_bins < 2)) return ADOP_ERR_INVALID_ARGUMENT;
    if (p->response && p->response_bins > kMaxResponseBins) return ADOP_ERR_SIZE_LIMIT;
    if (p->vignette && (p->vignette_image_w <= 0 || p->vignette_image_h <= 0)) return ADOP_ERR_INVALID_ARGUMENT;
    if (p->batch > 65535) return ADOP_ERR_SIZE_LIMIT;
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
    dim3 grid((unsigned)((plane + 255) / 256), (unsigned)a.B);
    k_tonemap_forward<<<grid, 256, sizeof(float) * 3 * a.K, static_cast<cudaStream_t>(stream)>>>(a, x, out);
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
    dim3 grid((unsigned)((plane + 255) / 256), (unsigned)a.B);
    k_tonemap_backward<<<grid, 256, sizeof(float) * 6 * a.K, st>>>(a, x, grad_out, gp);
    ADOP_CUDA_TRY(cudaGetLastError());
    return ADOP_OK;
}
