// Gradient exchange between the GPUs of one node over peer memory: reduce-scatter of the descriptor and point
// gradients, all-reduce of the small ones, the move of the descriptor gradients into the reference's [C,T] layout
// and NormalizeGradient (PointRenderer.cu:1609-1637), as ONE kernel that reads every rank's gradient block with plain
// peer loads over NVLink. The reference is single-GPU and has nothing of this.
//
// With touched flags in the blocks (set by the forward pass where it listed points for the backward pass) a small kernel
// first gathers, per chunk of the owned ranges, which ranks have anything there, and the reduce kernel reads a peer's
// descriptor and point gradients only in those chunks: zeros do not cross NVLink.
//
// The kernels never wait for another GPU: the caller orders them between two stream-ordered collectives of its
// communication library, so there is no spin loop here that could hang.
#include <cstdio>
#include <cstring>

#include "common.cuh"

namespace adop
{

constexpr int kMaxPeers = 8;

struct PeerBlocks
{
    const char* base[kMaxPeers];
    int world;
};

// work items of the one kernel, in this order: owned texels, owned points, then the small tensors element by element
struct PeerWork
{
    int t_lo, t_n;  // owned texels
    int p_lo, p_n;  // owned points
    int n_pose, n_count_pose, n_intr, n_count_intr, n_bg;  // elements
    long long n_env;
};

// A load that may cross NVLink: never served from this SM's L1, which is not coherent with what another GPU wrote.
__device__ __forceinline__ float4 peer_load4(const float4* p) { return __ldcv(p); }
__device__ __forceinline__ float peer_load(const float* p) { return __ldcv(p); }
__device__ __forceinline__ double peer_load(const double* p) { return __ldcv(p); }

// With touched flags in the blocks: which ranks added anything to each chunk of the texels and points this rank owns.
// One byte per chunk (bit r = rank r), written to this rank's own block ahead of the reduce kernel, so that the reduce
// kernel decides with a local load which peers it has to read a vector from. A rank's view arc sees one side of the scene:
// about half of the chunks of a Morton-sorted cloud get no gradient from it, and their zeros need not cross NVLink.
__global__ void __launch_bounds__(kBlock) k_peer_gather_touched(PeerBlocks pb, int rank, adop_peer_layout lay, PeerWork w)
{
    unsigned char* dst = reinterpret_cast<unsigned char*>(const_cast<char*>(pb.base[rank]) + lay.off_gathered);
    const int t_chunks = (lay.num_texels + kTouchedChunk - 1) / kTouchedChunk;
    const int tc_lo = w.t_lo >> kTouchedShift, tc_hi = w.t_n > 0 ? ((w.t_lo + w.t_n - 1) >> kTouchedShift) + 1 : tc_lo;
    const int pc_lo = w.p_lo >> kTouchedShift, pc_hi = w.p_n > 0 ? ((w.p_lo + w.p_n - 1) >> kTouchedShift) + 1 : pc_lo;
    const int n_t = tc_hi - tc_lo, n_p = pc_hi - pc_lo;
    for (int k = blockIdx.x * blockDim.x + threadIdx.x; k < n_t + n_p; k += gridDim.x * blockDim.x)
    {
        const bool tex = k < n_t;
        const int c = tex ? tc_lo + k : pc_lo + (k - n_t);
        const size_t off = tex ? lay.off_touched_texels : lay.off_touched_points;
        unsigned mask = 0;
        for (int r = 0; r < pb.world; ++r)
            if (__ldcv(reinterpret_cast<const unsigned char*>(pb.base[r] + off) + c) != 0) mask |= 1u << r;
        dst[tex ? c : t_chunks + c] = (unsigned char)mask;
    }
}

// MAXR = upper bound of the rank count (2, 4 or 8), U = texels or points a thread has in flight at once: U * MAXR = 8
// independent 16-byte loads per thread keep enough bytes in flight to fill NVLink whatever the rank count.
template <int C, int MAXR, int U>
__global__ void __launch_bounds__(kBlock) k_peer_reduce(PeerBlocks pb, int rank, adop_peer_layout lay, PeerWork w, adop_peer_reduce_out out)
{
    const long long stride = (long long)gridDim.x * blockDim.x;
    const long long first = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    // which ranks to read a texel's / point's vector from: all of them, or those that flagged its chunk (k_peer_gather_touched)
    const unsigned char* gathered = lay.touched ? reinterpret_cast<const unsigned char*>(pb.base[rank] + lay.off_gathered) : nullptr;
    const unsigned char* gathered_points = gathered ? gathered + (lay.num_texels + kTouchedChunk - 1) / kTouchedChunk : nullptr;
    // ---- owned texels: C floats from each rank, summed in rank order, written to the channel planes of the shard ----
    if (C % 4 == 0)
    {
        constexpr int Q = C / 4 > 0 ? C / 4 : 1;
        for (long long item = first; item < w.t_n; item += stride * U)
        {
            float4 v[U][MAXR][Q];
#pragma unroll
            for (int u = 0; u < U; ++u)
            {
                const long long it = item + u * stride;
                if (it < w.t_n)
                {
                    const unsigned mask = gathered ? gathered[(w.t_lo + it) >> kTouchedShift] : 0xffu;
#pragma unroll
                    for (int r = 0; r < MAXR; ++r)
                        if (r < pb.world)
                        {
                            const float4* src = reinterpret_cast<const float4*>(pb.base[r] + lay.off_texture) + (size_t)(w.t_lo + it) * Q;
#pragma unroll
                            for (int k = 0; k < Q; ++k) v[u][r][k] = (mask >> r) & 1u ? peer_load4(src + k) : make_float4(0.f, 0.f, 0.f, 0.f);
                        }
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u)
            {
                const long long it = item + u * stride;
                if (it < w.t_n)
                {
                    float acc[C];
#pragma unroll
                    for (int c = 0; c < C; ++c) acc[c] = 0.f;
#pragma unroll
                    for (int r = 0; r < MAXR; ++r)
                        if (r < pb.world)
                        {
#pragma unroll
                            for (int k = 0; k < Q; ++k)
                            {
                                acc[4 * k] += v[u][r][k].x; acc[4 * k + 1] += v[u][r][k].y;
                                acc[4 * k + 2] += v[u][r][k].z; acc[4 * k + 3] += v[u][r][k].w;
                            }
                        }
#pragma unroll
                    for (int c = 0; c < C; ++c) out.grad_texture_shard[(size_t)c * w.t_n + it] = acc[c];
                }
            }
        }
    }
    else
    {
        for (long long item = first; item < w.t_n; item += stride)
        {
            float acc[C];
#pragma unroll
            for (int c = 0; c < C; ++c) acc[c] = 0.f;
            const unsigned mask = gathered ? gathered[(w.t_lo + item) >> kTouchedShift] : 0xffu;
            for (int r = 0; r < pb.world; ++r)
            {
                if (!((mask >> r) & 1u)) continue;
                const float* src = reinterpret_cast<const float*>(pb.base[r] + lay.off_texture) + (size_t)(w.t_lo + item) * C;
#pragma unroll
                for (int c = 0; c < C; ++c) acc[c] += peer_load(src + c);
            }
#pragma unroll
            for (int c = 0; c < C; ++c) out.grad_texture_shard[(size_t)c * w.t_n + item] = acc[c];
        }
    }
    // ---- owned points: sums and NormalizeGradient (PointRenderer.cu:1620-1627) ----
    for (long long item = first; item < w.p_n; item += stride * U)
    {
        float4 v[U][MAXR];
#pragma unroll
        for (int u = 0; u < U; ++u)
        {
            const long long it = item + u * stride;
            if (it < w.p_n)
            {
                const unsigned mask = gathered_points ? gathered_points[(w.p_lo + it) >> kTouchedShift] : 0xffu;
#pragma unroll
                for (int r = 0; r < MAXR; ++r)
                    if (r < pb.world)
                        v[u][r] = (mask >> r) & 1u ? peer_load4(reinterpret_cast<const float4*>(pb.base[r] + lay.off_points) + (size_t)w.p_lo + (size_t)it)
                                                   : make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u)
        {
            const long long it = item + u * stride;
            if (it < w.p_n)
            {
                float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int r = 0; r < MAXR; ++r)
                    if (r < pb.world) { a.x += v[u][r].x; a.y += v[u][r].y; a.z += v[u][r].z; a.w += v[u][r].w; }
                if (out.normalize)
                {
                    if (a.w > 0.f) { a.x = a.x / a.w; a.y = a.y / a.w; a.z = a.z / a.w; }
                    a.w = 0.f;
                }
                reinterpret_cast<float4*>(out.grad_points_shard)[it] = a;
            }
        }
    }
    // ---- the small tensors, element by element: every rank sums all of them ----
    const long long n_small = (long long)w.n_pose + w.n_count_pose + w.n_intr + w.n_count_intr + w.n_bg;
    for (long long item = first; item < n_small; item += stride)
    {
        long long e = item;
        if (e < w.n_pose)
        {
            double a = 0.0;
            float cnt = 0.f;
            for (int r = 0; r < pb.world; ++r)
            {
                a += peer_load(reinterpret_cast<const double*>(pb.base[r] + lay.off_pose) + e);
                cnt += peer_load(reinterpret_cast<const float*>(pb.base[r] + lay.off_count_pose) + e / 6);
            }
            if (out.normalize && cnt > 0.f) a = a / (double)cnt;  // PointRenderer.cu:1609-1613
            out.grad_pose[e] = a;
            continue;
        }
        e -= w.n_pose;
        if (e < w.n_count_pose)
        {
            float a = 0.f;
            for (int r = 0; r < pb.world; ++r) a += peer_load(reinterpret_cast<const float*>(pb.base[r] + lay.off_count_pose) + e);
            out.count_pose[e] = a;
            continue;
        }
        e -= w.n_count_pose;
        if (e < w.n_intr)
        {
            float a = 0.f, cnt = 0.f;
            for (int r = 0; r < pb.world; ++r)
            {
                a += peer_load(reinterpret_cast<const float*>(pb.base[r] + lay.off_intrinsics) + e);
                cnt += peer_load(reinterpret_cast<const float*>(pb.base[r] + lay.off_count_intrinsics) + e / lay.intrinsics_cols);
            }
            if (out.normalize && cnt > 0.f) a = a / cnt;  // PointRenderer.cu:1629-1636
            out.grad_intrinsics[e] = a;
            continue;
        }
        e -= w.n_intr;
        if (e < w.n_count_intr)
        {
            float a = 0.f;
            for (int r = 0; r < pb.world; ++r) a += peer_load(reinterpret_cast<const float*>(pb.base[r] + lay.off_count_intrinsics) + e);
            out.count_intrinsics[e] = a;
            continue;
        }
        e -= w.n_count_intr;
        {
            float a = 0.f;
            for (int r = 0; r < pb.world; ++r) a += peer_load(reinterpret_cast<const float*>(pb.base[r] + lay.off_background) + e);
            out.grad_background[e] = a;
        }
    }
    // ---- the environment-map gradient, four floats at a time (every rank sums all of it) ----
    const long long env4 = (reinterpret_cast<uintptr_t>(out.grad_env_map) & 15) == 0 ? w.n_env / 4 : 0;
    for (long long item = first; item < env4; item += stride * U)
    {
        float4 v[U][MAXR];
#pragma unroll
        for (int u = 0; u < U; ++u)
        {
            const long long it = item + u * stride;
            if (it < env4)
            {
#pragma unroll
                for (int r = 0; r < MAXR; ++r)
                    if (r < pb.world) v[u][r] = peer_load4(reinterpret_cast<const float4*>(pb.base[r] + lay.off_env_map) + it);
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u)
        {
            const long long it = item + u * stride;
            if (it < env4)
            {
                float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int r = 0; r < MAXR; ++r)
                    if (r < pb.world) { a.x += v[u][r].x; a.y += v[u][r].y; a.z += v[u][r].z; a.w += v[u][r].w; }
                reinterpret_cast<float4*>(out.grad_env_map)[it] = a;
            }
        }
    }
    for (long long e = env4 * 4 + first; e < w.n_env; e += stride)
    {
        float a = 0.f;
        for (int r = 0; r < pb.world; ++r) a += peer_load(reinterpret_cast<const float*>(pb.base[r] + lay.off_env_map) + e);
        out.grad_env_map[e] = a;
    }
}

static size_t align_up(size_t v) { return (v + 255) & ~(size_t)255; }

}  // namespace adop

using namespace adop;

static_assert(sizeof(adop_peer_handle) >= sizeof(cudaIpcMemHandle_t), "handle too small");

extern "C" adop_status adop_peer_alloc(size_t bytes, void** ptr, adop_peer_handle* handle)
{
    if (!ptr || !handle || bytes == 0) return ADOP_ERR_INVALID_ARGUMENT;
    void* p = nullptr;
    ADOP_CUDA_TRY(cudaMalloc(&p, bytes));
    cudaError_t e = cudaMemset(p, 0, bytes);
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess)
    {
        cudaFree(p);
        return record_cuda_error(e, "adop_peer_alloc");
    }
    memset(handle->bytes, 0, sizeof(handle->bytes));
    memcpy(handle->bytes, &h, sizeof(h));
    *ptr = p;
    return ADOP_OK;
}

extern "C" adop_status adop_peer_free(void* ptr)
{
    if (!ptr) return ADOP_OK;
    ADOP_CUDA_TRY(cudaFree(ptr));
    return ADOP_OK;
}

extern "C" adop_status adop_peer_open(const adop_peer_handle* handle, void** ptr)
{
    if (!handle || !ptr) return ADOP_ERR_INVALID_ARGUMENT;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle->bytes, sizeof(h));
    void* p = nullptr;
    ADOP_CUDA_TRY(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    *ptr = p;
    return ADOP_OK;
}

extern "C" adop_status adop_peer_close(void* ptr)
{
    if (!ptr) return ADOP_OK;
    ADOP_CUDA_TRY(cudaIpcCloseMemHandle(ptr));
    return ADOP_OK;
}

extern "C" adop_status adop_peer_layout_fill(adop_peer_layout* l)
{
    if (!l) return ADOP_ERR_INVALID_ARGUMENT;
    if (l->channels <= 0 || l->num_texels < 0 || l->num_points < 0 || l->num_images < 0 || l->num_cameras < 0 ||
        l->env_h < 0 || l->env_w < 0 || (l->num_cameras > 0 && l->intrinsics_cols <= 0))
        return ADOP_ERR_INVALID_ARGUMENT;
    size_t at = 0;
    auto take = [&](size_t bytes) { size_t o = at; at = align_up(at + bytes); return o; };
    l->off_texture = take(sizeof(float) * (size_t)l->num_texels * l->channels);
    l->off_points = take(sizeof(float) * 4 * (size_t)l->num_points);
    l->off_pose = take(sizeof(double) * 6 * (size_t)l->num_images);
    l->off_count_pose = take(sizeof(float) * (size_t)l->num_images);
    l->off_intrinsics = take(sizeof(float) * (size_t)l->num_cameras * (l->num_cameras ? l->intrinsics_cols : 0));
    l->off_count_intrinsics = take(sizeof(float) * (size_t)l->num_cameras);
    l->off_background = take(l->background ? sizeof(float) * l->channels : 0);
    l->off_env_map = take(sizeof(float) * (size_t)l->channels * l->env_h * l->env_w);
    const size_t t_chunks = l->touched ? ((size_t)l->num_texels + kTouchedChunk - 1) / kTouchedChunk : 0;
    const size_t p_chunks = l->touched ? ((size_t)l->num_points + kTouchedChunk - 1) / kTouchedChunk : 0;
    l->off_touched_texels = take(t_chunks);
    l->off_touched_points = take(p_chunks);
    l->off_gathered = take(t_chunks + p_chunks);
    l->total_bytes = at ? at : 256;
    return ADOP_OK;
}

extern "C" void adop_peer_shard_range(int32_t count, int32_t world, int32_t rank, int32_t* lo, int32_t* hi)
{
    if (world < 1) world = 1;
    long long per = ((long long)count + world - 1) / world;
    long long a = per * rank, b = per * (rank + 1);
    if (a > count) a = count;
    if (b > count) b = count;
    if (a < 0) a = 0;
    if (b < a) b = a;
    if (lo) *lo = (int32_t)a;
    if (hi) *hi = (int32_t)b;
}

extern "C" adop_status adop_peer_reduce_gradients(const void* const* blocks, int32_t world, int32_t rank,
                                                  const adop_peer_layout* layout, const adop_peer_reduce_out* out, void* stream)
{
    if (!blocks || !layout || !out || world < 1 || world > kMaxPeers || rank < 0 || rank >= world) return ADOP_ERR_INVALID_ARGUMENT;
    adop_peer_layout check = *layout;
    if (adop_peer_layout_fill(&check) != ADOP_OK || check.total_bytes != layout->total_bytes || check.off_env_map != layout->off_env_map)
        return ADOP_ERR_INVALID_ARGUMENT;
    PeerBlocks pb;
    pb.world = world;
    for (int r = 0; r < kMaxPeers; ++r)
    {
        pb.base[r] = r < world ? static_cast<const char*>(blocks[r]) : nullptr;
        if (r < world && (!blocks[r] || (reinterpret_cast<uintptr_t>(blocks[r]) & 15))) return ADOP_ERR_INVALID_ARGUMENT;
    }
    if ((reinterpret_cast<uintptr_t>(out->grad_points_shard) & 15)) return ADOP_ERR_INVALID_ARGUMENT;
    PeerWork w;
    memset(&w, 0, sizeof(w));
    int lo, hi;
    if (out->grad_texture_shard && layout->num_texels > 0)
    {
        adop_peer_shard_range(layout->num_texels, world, rank, &lo, &hi);
        w.t_lo = lo; w.t_n = hi - lo;
    }
    if (out->grad_points_shard && layout->num_points > 0)
    {
        adop_peer_shard_range(layout->num_points, world, rank, &lo, &hi);
        w.p_lo = lo; w.p_n = hi - lo;
    }
    if (layout->num_images > 0)
    {
        if (out->grad_pose) w.n_pose = layout->num_images * 6;
        if (out->count_pose) w.n_count_pose = layout->num_images;
    }
    if (layout->num_cameras > 0)
    {
        if (out->grad_intrinsics) w.n_intr = layout->num_cameras * layout->intrinsics_cols;
        if (out->count_intrinsics) w.n_count_intr = layout->num_cameras;
    }
    if (layout->background && out->grad_background) w.n_bg = layout->channels;
    if (out->grad_env_map) w.n_env = (long long)layout->channels * layout->env_h * layout->env_w;
    const long long total = (long long)w.t_n + w.p_n + w.n_pose + w.n_count_pose + w.n_intr + w.n_count_intr + w.n_bg + w.n_env;
    if (total == 0) return ADOP_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int C = layout->channels;
    if (layout->touched && (w.t_n > 0 || w.p_n > 0))
    {
        const int chunks = (w.t_n + w.p_n) / kTouchedChunk + 4;
        const int grid = (chunks + kBlock - 1) / kBlock;
        ADOP_LAUNCH("k_peer_gather_touched", st, (k_peer_gather_touched<<<grid, kBlock, 0, st>>>(pb, rank, *layout, w)));
    }
#define ADOP_PEER_LAUNCH(CC, MAXR)                                                                                      \
    {                                                                                                                   \
        constexpr int Q = CC % 4 == 0 ? CC / 4 : 1;                                                                     \
        constexpr int U = 8 / (MAXR * Q) > 0 ? 8 / (MAXR * Q) : 1;                                                      \
        static const int per_sm_grid = resident_grid(k_peer_reduce<CC, MAXR, U>, 1ll << 40);                            \
        int grid = need < per_sm_grid ? (int)need : per_sm_grid;                                                        \
        ADOP_LAUNCH("k_peer_reduce", st, (k_peer_reduce<CC, MAXR, U><<<grid, kBlock, 0, st>>>(pb, rank, *layout, w, *out)));  \
    }
#define ADOP_PEER_CASE(CC)                                                                                              \
    case CC:                                                                                                            \
        if (world <= 2) ADOP_PEER_LAUNCH(CC, 2)                                                                         \
        else if (world <= 4) ADOP_PEER_LAUNCH(CC, 4)                                                                    \
        else ADOP_PEER_LAUNCH(CC, 8)                                                                                    \
        break;
    // the largest of the three parts decides the grid (each thread strides through all three)
    long long largest = w.t_n > w.p_n ? w.t_n : w.p_n;
    const long long n_small = (long long)w.n_pose + w.n_count_pose + w.n_intr + w.n_count_intr + w.n_bg;
    if (n_small > largest) largest = n_small;
    // the environment map goes four floats at a time when its size allows, else float by float: count what the kernel
    // will loop over, and never launch an empty grid (a tail of one to three floats is work too)
    const bool env_vec = (reinterpret_cast<uintptr_t>(out->grad_env_map) & 15) == 0;
    const long long n_env_items = env_vec ? (w.n_env / 4 > w.n_env % 4 ? w.n_env / 4 : w.n_env % 4) : w.n_env;
    if (n_env_items > largest) largest = n_env_items;
    long long need = (largest + kBlock - 1) / kBlock;
    if (need < 1) need = 1;
    switch (C)
    {
        ADOP_PEER_CASE(3)
        ADOP_PEER_CASE(4)
        ADOP_PEER_CASE(8)
        ADOP_PEER_CASE(16)
        default: return ADOP_ERR_UNSUPPORTED;
    }
#undef ADOP_PEER_LAUNCH
#undef ADOP_PEER_CASE
    ADOP_CUDA_TRY(cudaGetLastError());
    return ADOP_OK;
}
