// Optimiser step on the shard a rank owns + all-gather of the updated parameters, as ONE kernel over peer memory.
// Follows adop_peer_reduce_gradients in a view-sharded training step: that kernel leaves every rank with the final
// gradients of its texels and points; this one applies the reference's optimisers to exactly those elements - Adam for
// the descriptors (torch::optim::Adam with default betas, NeuralScene.cpp:76-107), plain SGD for the point positions
// (NeuralScene.cpp:204-240) - and writes each new value into EVERY rank's replica of the parameter tensors with plain
// peer stores over NVLink. The Adam moments exist only for the owned shard (1 / world of the optimiser state per GPU).
// The reference trains on one GPU and has nothing of this.
//
// The kernel never waits for another GPU: the caller orders it after everyone's last read of the parameters (the
// backward pass) and before anyone's next read (a stream-ordered collective on either side), so there is no spin loop.
#include "common.cuh"

namespace adop
{

constexpr int kMaxUpdatePeers = 8;

struct ReplicaBlocks
{
    char* base[kMaxUpdatePeers];
    int world;
};

struct UpdateWork
{
    int t_lo, t_n;  // owned texels
    int p_lo, p_n;  // owned points
    int T, C;
    size_t off_texture, off_points;
    // Adam, in the operation order of torch::optim::Adam::step: step_size = lr / (1 - beta1^t), sqrt_bias2 = sqrt(1 - beta2^t)
    float beta1, one_minus_beta1, beta2, one_minus_beta2, eps, neg_step_size, sqrt_bias2;
    float neg_lr_points;
};

__device__ __forceinline__ float adam_element(const UpdateWork& w, float p, float g, float* m, float* v)
{
    const float mm = *m * w.beta1 + g * w.one_minus_beta1;         // exp_avg.mul_(beta1).add_(grad, 1 - beta1)
    const float vv = *v * w.beta2 + (g * g) * w.one_minus_beta2;   // exp_avg_sq.mul_(beta2).addcmul_(grad, grad, 1 - beta2)
    *m = mm; *v = vv;
    const float denom = sqrtf(vv) / w.sqrt_bias2 + w.eps;          // (exp_avg_sq.sqrt() / sqrt(bias_correction2)).add_(eps)
    return p + w.neg_step_size * (mm / denom);                     // param.addcdiv_(exp_avg, denom, -step_size)
}

// VEC = 4: four consecutive texels of a channel plane per item (every rank's share starts and ends on a multiple of four)
template <int VEC>
__global__ void __launch_bounds__(kBlock) k_peer_update(ReplicaBlocks rb, int rank, UpdateWork w, const float* __restrict__ grad_texture,
                                                        float* __restrict__ adam_m, float* __restrict__ adam_v,
                                                        const float* __restrict__ grad_points)
{
    const long long stride = (long long)gridDim.x * blockDim.x;
    const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    // descriptors: planes [C, t_n] of gradient and moments, parameter planes [C, T] in every replica
    if (grad_texture && w.t_n > 0)
    {
        const int per_plane = (w.t_n + VEC - 1) / VEC;
        const long long items = (long long)w.C * per_plane;
        const float* own = reinterpret_cast<const float*>(rb.base[rank] + w.off_texture);
        for (long long it = tid; it < items; it += stride)
        {
            const int c = (int)(it / per_plane), k = (int)(it - (long long)c * per_plane) * VEC;
            const size_t s = (size_t)c * w.t_n + k;           // in the shard's planes
            const size_t d = (size_t)c * w.T + w.t_lo + k;    // in the parameter planes
            if (VEC == 4)
            {
                const float4 g = __ldcs(reinterpret_cast<const float4*>(grad_texture + s));
                float4 m = *reinterpret_cast<const float4*>(adam_m + s), v = *reinterpret_cast<const float4*>(adam_v + s);
                const float4 p = *reinterpret_cast<const float4*>(own + d);
                float4 q;
                q.x = adam_element(w, p.x, g.x, &m.x, &v.x); q.y = adam_element(w, p.y, g.y, &m.y, &v.y);
                q.z = adam_element(w, p.z, g.z, &m.z, &v.z); q.w = adam_element(w, p.w, g.w, &m.w, &v.w);
                *reinterpret_cast<float4*>(adam_m + s) = m;
                *reinterpret_cast<float4*>(adam_v + s) = v;
                for (int r = 0; r < rb.world; ++r) *reinterpret_cast<float4*>(reinterpret_cast<float*>(rb.base[r] + w.off_texture) + d) = q;
            }
            else
            {
                float m = adam_m[s], v = adam_v[s];
                const float q = adam_element(w, own[d], __ldcs(grad_texture + s), &m, &v);
                adam_m[s] = m; adam_v[s] = v;
                for (int r = 0; r < rb.world; ++r) reinterpret_cast<float*>(rb.base[r] + w.off_texture)[d] = q;
            }
        }
    }
    // points: p.xyz += -lr * g.xyz (torch::optim::SGD without momentum), the drop-out radius in w stays
    if (grad_points && w.p_n > 0)
    {
        const float4* own = reinterpret_cast<const float4*>(rb.base[rank] + w.off_points);
        for (long long it = tid; it < w.p_n; it += stride)
        {
            const float4 g = __ldcs(reinterpret_cast<const float4*>(grad_points) + it);
            float4 p = own[w.p_lo + it];
            p.x = p.x + w.neg_lr_points * g.x; p.y = p.y + w.neg_lr_points * g.y; p.z = p.z + w.neg_lr_points * g.z;
            for (int r = 0; r < rb.world; ++r) reinterpret_cast<float4*>(rb.base[r] + w.off_points)[w.p_lo + it] = p;
        }
    }
}

}  // namespace adop

using namespace adop;

extern "C" adop_status adop_peer_param_layout_fill(adop_peer_param_layout* l)
{
    if (!l || l->channels <= 0 || l->num_texels <= 0 || l->num_points < 0) return ADOP_ERR_INVALID_ARGUMENT;
    size_t off = 0;
    l->off_texture = off;
    off += ((size_t)l->channels * l->num_texels * sizeof(float) + 255) & ~(size_t)255;
    l->off_points = off;
    off += ((size_t)l->num_points * 4 * sizeof(float) + 255) & ~(size_t)255;
    l->total_bytes = off;
    return ADOP_OK;
}

extern "C" adop_status adop_peer_apply_update(void* const* param_blocks, int32_t world, int32_t rank, const adop_peer_param_layout* layout,
                                              const adop_peer_update* u, void* stream)
{
    if (!param_blocks || !layout || !u || world < 1 || world > kMaxUpdatePeers || rank < 0 || rank >= world) return ADOP_ERR_INVALID_ARGUMENT;
    adop_peer_param_layout check = *layout;
    if (adop_peer_param_layout_fill(&check) != ADOP_OK || check.total_bytes != layout->total_bytes || check.off_points != layout->off_points)
        return ADOP_ERR_INVALID_ARGUMENT;
    ReplicaBlocks rb;
    rb.world = world;
    for (int r = 0; r < kMaxUpdatePeers; ++r)
    {
        rb.base[r] = r < world ? static_cast<char*>(param_blocks[r]) : nullptr;
        if (r < world && (!param_blocks[r] || (reinterpret_cast<uintptr_t>(param_blocks[r]) & 15))) return ADOP_ERR_INVALID_ARGUMENT;
    }
    UpdateWork w;
    memset(&w, 0, sizeof(w));
    w.T = layout->num_texels; w.C = layout->channels;
    w.off_texture = layout->off_texture; w.off_points = layout->off_points;
    int lo, hi;
    const bool tex = u->grad_texture_shard != nullptr;
    if (tex)
    {
        if (!u->adam_m || !u->adam_v || u->step < 1 || !(u->beta1 >= 0.f && u->beta1 < 1.f) || !(u->beta2 >= 0.f && u->beta2 < 1.f))
            return ADOP_ERR_INVALID_ARGUMENT;
        adop_peer_shard_range(layout->num_texels, world, rank, &lo, &hi);
        w.t_lo = lo; w.t_n = hi - lo;
        // the scalars as torch forms them: in double, then rounded once
        const double bias1 = 1.0 - pow((double)u->beta1, (double)u->step), bias2 = 1.0 - pow((double)u->beta2, (double)u->step);
        w.beta1 = u->beta1; w.one_minus_beta1 = (float)(1.0 - (double)u->beta1);
        w.beta2 = u->beta2; w.one_minus_beta2 = (float)(1.0 - (double)u->beta2);
        w.eps = u->eps;
        w.neg_step_size = (float)(-(double)u->lr_texture / bias1);
        w.sqrt_bias2 = (float)sqrt(bias2);
    }
    const bool pts = u->grad_points_shard != nullptr && layout->num_points > 0;
    if (pts)
    {
        if (reinterpret_cast<uintptr_t>(u->grad_points_shard) & 15) return ADOP_ERR_INVALID_ARGUMENT;
        adop_peer_shard_range(layout->num_points, world, rank, &lo, &hi);
        w.p_lo = lo; w.p_n = hi - lo;
        w.neg_lr_points = -u->lr_points;
    }
    if (w.t_n == 0 && w.p_n == 0) return ADOP_OK;
    // four texels per item when every address involved is a multiple of 16 bytes
    const bool vec = tex && w.t_n % 4 == 0 && w.t_lo % 4 == 0 && w.T % 4 == 0 &&
                     ((reinterpret_cast<uintptr_t>(u->grad_texture_shard) | reinterpret_cast<uintptr_t>(u->adam_m) |
                       reinterpret_cast<uintptr_t>(u->adam_v)) & 15) == 0;
    const long long tex_items = tex ? (long long)w.C * (vec ? w.t_n / 4 : w.t_n) : 0;
    const long long items = tex_items > w.p_n ? tex_items : w.p_n;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    long long need = (items + kBlock - 1) / kBlock;
    if (need < 1) need = 1;
    const float* gt = tex ? u->grad_texture_shard : nullptr;
    const float* gp = pts ? u->grad_points_shard : nullptr;
    if (vec)
    {
        static const int g = resident_grid(k_peer_update<4>, 1ll << 40);
        ADOP_LAUNCH("k_peer_update", st, (k_peer_update<4><<<(int)(need < g ? need : g), kBlock, 0, st>>>(rb, rank, w, gt, u->adam_m, u->adam_v, gp)));
    }
    else
    {
        static const int g = resident_grid(k_peer_update<1>, 1ll << 40);
        ADOP_LAUNCH("k_peer_update", st, (k_peer_update<1><<<(int)(need < g ? need : g), kBlock, 0, st>>>(rb, rank, w, gt, u->adam_m, u->adam_v, gp)));
    }
    ADOP_CUDA_TRY(cudaGetLastError());
    return ADOP_OK;
}
