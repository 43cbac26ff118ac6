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
// vignette geometry of VEC consecutive pixels starting at pix
template <int VEC>
__device__ __forceinline__ void tone_geometry(const ToneArgs& a, int b, size_t pix, size_t plane, float* du, float* dv, float* r2, float* fac)
{
    float u0[VEC], v0[VEC];
    if (a.uv)
    {
        load_vec<VEC>(a.uv + ((size_t)b * 2 + 0) * plane + pix, u0);
        load_vec<VEC>(a.uv + ((size_t)b * 2 + 1) * plane + pix, v0);
    }
    else
    {
        int yy = (int)(pix / a.W), xx = (int)(pix - (size_t)yy * a.W);
#pragma unroll
        for (int k = 0; k < VEC; ++k)
        {
            u0[k] = 2.0f * ((float)xx / (float)(a.W - 1)) - 1.0f;
            v0[k] = 2.0f * ((float)yy / (float)(a.H - 1)) - 1.0f;
            if (++xx == a.W) { xx = 0; ++yy; }
        }
    }
#pragma unroll
    for (int k = 0; k < VEC; ++k)
    {
        du[k] = (u0[k] - a.vignette[3]) * a.aspect; dv[k] = v0[k] - a.vignette[4];
        r2[k] = du[k] * du[k] + dv[k] * dv[k];
        float r4 = r2[k] * r2[k], r6 = r4 * r2[k];
        fac[k] = 1.f + a.vignette[0] * r2[k] + a.vignette[1] * r4 + a.vignette[2] * r6;
    }
}

// grid: (ceil(H*W / (block * VEC)), B)
template <int VEC>
__global__ void __launch_bounds__(256) k_tonemap_forward(ToneArgs a, const float* __restrict__ x, float* __restrict__ out)
{
    extern __shared__ float s_lut[];  // [3,K]
    for (int k = threadIdx.x; k < 3 * a.K; k += blockDim.x) s_lut[k] = a.response[k];
    __syncthreads();
    const int b = blockIdx.y;
    const size_t plane = (size_t)a.H * a.W;
    const size_t pix = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * VEC;
    if (pix >= plane) return;
    const int fi = a.frame_index ? a.frame_index[b] : 0;
    const float ef = a.exposure ? 1.0f / exp2f(a.exposure[fi]) : 1.0f;
    float du[VEC], dv[VEC], r2[VEC], fac[VEC];
#pragma unroll
    for (int k = 0; k < VEC; ++k) fac[k] = 1.f;
    if (a.vignette) tone_geometry<VEC>(a, b, pix, plane, du, dv, r2, fac);
#pragma unroll
    for (int c = 0; c < 3; ++c)
    {
        const float wb = a.white_balance ? a.white_balance[(size_t)fi * 3 + c] : 1.0f;
        float xin[VEC], o[VEC];
        load_vec<VEC>(x + ((size_t)b * 3 + c) * plane + pix, xin);
#pragma unroll
        for (int k = 0; k < VEC; ++k)
        {
            float v = xin[k] * ef;
            v = wb * v;
            v = fac[k] * v;
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
                o[k] = s_lut[c * a.K + i0] * (1.0f - fr) + s_lut[c * a.K + i1] * fr + leak_add;
            }
            else
                o[k] = fminf(fmaxf(v, 0.f), 1.f);
        }
        store_vec<VEC>(out + ((size_t)b * 3 + c) * plane + pix, o);
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
// float is a compare-and-swap loop and cost more than the rest of the kernel together (185 us of 320 us per 4K image);
// the integer one is a single instruction (22 us). So each chunk of 256 x VEC pixels is summed in block-scaled fixed point:
//   1. the block finds M = max |upstream gradient| of the chunk and takes scale = 2^(18 - exponent(M)), an exact power
//      of two, so that every term |g * weight * scale| < 2^19 and a bin can take all 2 x 256 x VEC terms of a chunk in 32 bits;
//   2. terms are rounded to nearest and added with integer atomics into one of two integer histograms (ping-pong);
//   3. after the chunk every thread converts the bins it owns back (exactly: a power-of-two factor) and adds them to the
//      block's float histogram, which goes to global memory once at the end.
// A term is off by at most 2^-19 of the chunk's largest gradient, unbiased; chunks whose M is not finite or is below
// 2^-100 take the float atomics instead, so NaN / Inf gradients still show up in the result.
template <int VEC>
__global__ void __launch_bounds__(256, 3) k_tonemap_backward(ToneArgs a, const float* __restrict__ x, const float* __restrict__ grad_out,
                                                           ToneGradPtrs g)
{
    extern __shared__ float smem[];  // lut [3,K], float histogram [3,K], two integer histograms [3,K]
    const int K3 = 3 * a.K;
    float* s_lut = smem;
    float* s_acc = smem + K3;
    int* s_int = reinterpret_cast<int*>(smem + 2 * K3);
    __shared__ float s_small[9];  // exposure, wb[3], vignette[5]
    __shared__ float s_max[2][8];
    const bool want_resp = g.grad_response && a.response;
    for (int k = threadIdx.x; k < K3; k += blockDim.x) s_lut[k] = a.response[k];
    if (want_resp)
        for (int k = threadIdx.x; k < K3; k += blockDim.x) { s_acc[k] = 0.f; s_int[k] = 0; s_int[K3 + k] = 0; }
    if (threadIdx.x < 9) s_small[threadIdx.x] = 0.f;
    __syncthreads();
    const int b = blockIdx.y;
    const size_t plane = (size_t)a.H * a.W;
    const int fi = a.frame_index ? a.frame_index[b] : 0;
    const float ef = a.exposure ? 1.0f / exp2f(a.exposure[fi]) : 1.0f;
    const float ln2 = 0.69314718056f;
    float gE = 0.f, gWB[3] = {0.f, 0.f, 0.f}, gV[5] = {0.f, 0.f, 0.f, 0.f, 0.f};
    // a block walks over many pixel chunks of its image, so the parameter gradients leave it once, not once per chunk;
    // every thread of the block makes the same number of rounds (the loop holds block-wide barriers)
    const size_t per_chunk = (size_t)blockDim.x * VEC;
    const size_t chunks = (plane + per_chunk - 1) / per_chunk;
    int parity = 0;
    for (size_t chunk = blockIdx.x; chunk < chunks; chunk += gridDim.x, parity ^= 1)
    {
        const size_t pix = chunk * per_chunk + (size_t)threadIdx.x * VEC;
        const bool live = pix < plane;
        // all six loads of the chunk are requested before anything waits (the block-wide maximum needs a barrier)
        float go[3][VEC], xall[3][VEC];
#pragma unroll
        for (int c = 0; c < 3; ++c)
        {
#pragma unroll
            for (int k = 0; k < VEC; ++k) { go[c][k] = 0.f; xall[c][k] = 0.f; }
            if (live)
            {
                load_vec<VEC>(grad_out + ((size_t)b * 3 + c) * plane + pix, go[c]);
                load_vec<VEC>(x + ((size_t)b * 3 + c) * plane + pix, xall[c]);
            }
        }
        float scale = 0.f;  // 0: this chunk adds to the float histogram directly
        int* my_int = s_int + parity * K3;
        if (want_resp)
        {
            float m = 0.f;
            bool odd = false;  // a NaN anywhere: fmaxf would drop it
#pragma unroll
            for (int c = 0; c < 3; ++c)
#pragma unroll
                for (int k = 0; k < VEC; ++k) { m = fmaxf(m, fabsf(go[c][k])); odd = odd || !(fabsf(go[c][k]) <= 3.0e38f); }
            if (odd) m = __int_as_float(0x7f800000);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
            if ((threadIdx.x & 31) == 0) s_max[parity][threadIdx.x >> 5] = m;
            __syncthreads();
            float M = 0.f;
#pragma unroll
            for (int k = 0; k < 8; ++k) M = fmaxf(M, s_max[parity][k]);
            const int e = (int)((__float_as_uint(M) >> 23) & 0xffu) - 127;
            if (M <= 3.0e38f && e >= -100) scale = __int_as_float((127 + 18 - e) << 23);
        }
        if (live)
        {
            float du[VEC], dv[VEC], r2[VEC], fac[VEC];
#pragma unroll
            for (int k = 0; k < VEC; ++k) { fac[k] = 1.f; du[k] = dv[k] = r2[k] = 0.f; }
            if (a.vignette) tone_geometry<VEC>(a, b, pix, plane, du, dv, r2, fac);
#pragma unroll
            for (int c = 0; c < 3; ++c)
            {
                const float wb = a.white_balance ? a.white_balance[(size_t)fi * 3 + c] : 1.0f;
                float gx[VEC];
                const float* xin = xall[c];
                // neighbouring pixels mostly fall into the same pair of bins: their two weights are added up in
                // registers and reach shared memory once per run
                int run_i0 = -1, run_i1 = 0;
                float run_w0 = 0.f, run_w1 = 0.f;
                auto flush = [&]() {
                    if (scale != 0.f)
                    {
                        atomicAdd(&my_int[c * a.K + run_i0], __float2int_rn(run_w0 * scale));
                        atomicAdd(&my_int[c * a.K + run_i1], __float2int_rn(run_w1 * scale));
                    }
                    else
                    {
                        atomicAdd(&s_acc[c * a.K + run_i0], run_w0);
                        atomicAdd(&s_acc[c * a.K + run_i1], run_w1);
                    }
                };
#pragma unroll
                for (int k = 0; k < VEC; ++k)
                {
                    const float pre = wb * (xin[k] * ef);
                    const float v = fac[k] * pre;
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
                        if (want_resp)
                        {
                            if (i0 != run_i0)
                            {
                                if (run_i0 >= 0) flush();
                                run_i0 = i0; run_i1 = i1; run_w0 = 0.f; run_w1 = 0.f;
                            }
                            run_w0 += go[c][k] * (1.0f - fr);
                            run_w1 += go[c][k] * fr;
                        }
                        float inside = (v > 0.f && v < 1.f) ? 1.f : 0.f;
                        dv_out = inside * (s_lut[c * a.K + i1] - s_lut[c * a.K + i0]) * (float)(a.K - 1) + dleak;
                    }
                    else
                        dv_out = (v > 0.f && v < 1.f) ? 1.f : 0.f;
                    const float gv = go[c][k] * dv_out;
                    if (a.vignette)
                    {
                        float gfac = gv * pre;
                        float r4 = r2[k] * r2[k];
                        gV[0] += gfac * r2[k]; gV[1] += gfac * r4; gV[2] += gfac * (r4 * r2[k]);
                        float gr2 = gfac * (a.vignette[0] + 2.f * a.vignette[1] * r2[k] + 3.f * a.vignette[2] * r4);
                        gV[3] += gr2 * 2.f * du[k] * (-a.aspect);
                        gV[4] += gr2 * 2.f * dv[k] * (-1.f);
                    }
                    const float gpre = gv * fac[k];
                    gWB[c] += gpre * (xin[k] * ef);
                    const float gxe = gpre * wb;
                    gE += gxe * xin[k] * ef * (-ln2);
                    gx[k] = gxe * ef;
                }
                if (run_i0 >= 0) flush();
                if (g.grad_x) store_vec<VEC>(g.grad_x + ((size_t)b * 3 + c) * plane + pix, gx);
            }
        }
        if (want_resp)
        {
            __syncthreads();  // the chunk's integer terms are all in
            if (scale != 0.f)
            {
                const float inv = __int_as_float((254 - (int)(__float_as_uint(scale) >> 23)) << 23);  // 1 / scale, exact
                for (int k = threadIdx.x; k < K3; k += blockDim.x)
                {
                    const int q = my_int[k];
                    if (q != 0) { s_acc[k] += (float)q * inv; my_int[k] = 0; }
                }
            }
            // the other integer histogram takes the next chunk; this one is touched again only after that chunk's barrier
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
    if (want_resp)
        for (int k = threadIdx.x; k < K3; k += blockDim.x)
        {
            const float sum = s_acc[k];
            if (sum != 0.f) atomicAdd(g.grad_response + k, sum);
        }
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
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool vec = plane % 4 == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(a.uv)) & 15) == 0;
    if (vec)
    {
        dim3 grid((unsigned)((plane / 4 + 255) / 256), (unsigned)a.B);
        ADOP_LAUNCH("k_tonemap_forward", st, (k_tonemap_forward<4><<<grid, 256, sizeof(float) * 3 * a.K, st>>>(a, x, out)));
    }
    else
    {
        dim3 grid((unsigned)((plane + 255) / 256), (unsigned)a.B);
        ADOP_LAUNCH("k_tonemap_forward", st, (k_tonemap_forward<1><<<grid, 256, sizeof(float) * 3 * a.K, st>>>(a, x, out)));
    }
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
    // lut + float histogram + two integer histograms
    const size_t smem_bytes = sizeof(float) * 3 * a.K * 4;
    if (smem_bytes > 40 * 1024)
    {
        // beyond the default 48 KB with the static part: ask for it (1024 bins need 48 KB + 100 bytes)
        ADOP_CUDA_TRY(cudaFuncSetAttribute(k_tonemap_backward<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes));
        ADOP_CUDA_TRY(cudaFuncSetAttribute(k_tonemap_backward<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes));
    }
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k_tonemap_backward<4>, 256, smem_bytes) != cudaSuccess || per_sm < 1)
        per_sm = 1;
    // about as many blocks as stay resident at once, shared out over the images
    const size_t per_image = (size_t)((sm_count() * per_sm + a.B - 1) / a.B);
    const bool vec = plane % 4 == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(grad_out) |
                                         reinterpret_cast<uintptr_t>(g->grad_x) | reinterpret_cast<uintptr_t>(a.uv)) & 15) == 0;
    if (vec)
    {
        size_t chunks = (plane / 4 + 255) / 256;
        dim3 grid((unsigned)(chunks < per_image ? chunks : per_image), (unsigned)a.B);
        ADOP_LAUNCH("k_tonemap_backward", st, (k_tonemap_backward<4><<<grid, 256, smem_bytes, st>>>(a, x, grad_out, gp)));
    }
    else
    {
        size_t chunks = (plane + 255) / 256;
        dim3 grid((unsigned)(chunks < per_image ? chunks : per_image), (unsigned)a.B);
        ADOP_LAUNCH("k_tonemap_backward", st, (k_tonemap_backward<1><<<grid, 256, smem_bytes, st>>>(a, x, grad_out, gp)));
    }
    ADOP_CUDA_TRY(cudaGetLastError());
    return ADOP_OK;
}
