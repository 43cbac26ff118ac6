// Point-cloud preprocessing on the GPU: the Morton-64 reorder that the rasterizer's memory behaviour depends on
// (the reference calls point_cloud.ReorderMorton64() once per scene, src/lib/data/SceneData.cpp:100; the function itself
// lives in saiga and is not in the reference tree, so the key below is this library's own definition, the same as the
// numpy statement in adop_b200/synth.py: 21 bits per axis over the bounding box, x in the lowest interleaved bit).
//
//   k_bbox_partial / k_bbox_final   exact min / max of the positions (two deterministic stages)
//   k_morton_keys                   float32 quantisation (no contraction: the same bits as numpy), bit interleave
//   eight radix passes              least-significant digit first, 8 bits per pass, stable:
//       k_radix_histogram           per-block digit counts of its tile (native integer shared-memory atomics)
//       k_radix_scan                exclusive scan of each digit's per-block counts (one block per digit) + digit totals
//       k_radix_scatter             rank inside the tile by warp match + per-warp digit counters, keys and point indices
//                                   move to their sorted place
//   k_permute_rows                  dst[i] = src[order[i]] for rows of 4..64 bytes (positions, normals, indices, planes)
//
// Integer / byte work bound by HBM: per pass a key is read twice and written once with its index (32 bytes), 8 passes.
#include <cstdint>
#include <cstring>

#include "common.cuh"

namespace adop
{

constexpr int kRadixBits = 8;
constexpr int kRadixBins = 1 << kRadixBits;
constexpr int kRadixItems = 8;                        // keys per thread and tile
constexpr int kRadixTile = kBlock * kRadixItems;      // 2048 keys per block
constexpr int kRadixPasses = 8;                       // 63-bit keys
constexpr int kBboxBlocks = 1024;
static_assert(kBlock == kRadixBins, "one thread per digit");

struct MortonWorkspace
{
    unsigned long long* keys[2];
    int* index[2];
    unsigned* hist;  // [kRadixBins][blocks]
    float* bbox;     // [kBboxBlocks][6] partials, then [6] final at the end
    unsigned* totals;  // [kRadixBins] keys per digit of the current pass
    int blocks;
};

static size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

static size_t morton_layout(int n, char* base, MortonWorkspace* w)
{
    const int blocks = (n + kRadixTile - 1) / kRadixTile;
    size_t at = 0;
    auto take = [&](size_t bytes) { size_t o = at; at = align256(at + bytes); return o; };
    size_t k0 = take(sizeof(unsigned long long) * (size_t)n), k1 = take(sizeof(unsigned long long) * (size_t)n);
    size_t i0 = take(sizeof(int) * (size_t)n), i1 = take(sizeof(int) * (size_t)n);
    size_t h = take(sizeof(unsigned) * (size_t)kRadixBins * (blocks > 0 ? blocks : 1));
    size_t b = take(sizeof(float) * 6 * (kBboxBlocks + 1));
    size_t t = take(sizeof(unsigned) * kRadixBins);
    if (w)
    {
        w->keys[0] = reinterpret_cast<unsigned long long*>(base + k0);
        w->keys[1] = reinterpret_cast<unsigned long long*>(base + k1);
        w->index[0] = reinterpret_cast<int*>(base + i0);
        w->index[1] = reinterpret_cast<int*>(base + i1);
        w->hist = reinterpret_cast<unsigned*>(base + h);
        w->bbox = reinterpret_cast<float*>(base + b);
        w->totals = reinterpret_cast<unsigned*>(base + t);
        w->blocks = blocks;
    }
    return at;
}

// ---- bounding box -------------------------------------------------------------------------------------------------
__device__ __forceinline__ void block_minmax(float* lo, float* hi, float* out6)
{
    __shared__ float s[kBlock / 32][6];
#pragma unroll
    for (int k = 0; k < 3; ++k)
    {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
        {
            lo[k] = fminf(lo[k], __shfl_xor_sync(0xffffffffu, lo[k], o));
            hi[k] = fmaxf(hi[k], __shfl_xor_sync(0xffffffffu, hi[k], o));
        }
    }
    if ((threadIdx.x & 31) == 0)
    {
#pragma unroll
        for (int k = 0; k < 3; ++k) { s[threadIdx.x >> 5][k] = lo[k]; s[threadIdx.x >> 5][3 + k] = hi[k]; }
    }
    __syncthreads();
    if (threadIdx.x < 6)
    {
        float v = s[0][threadIdx.x];
        for (int wv = 1; wv < kBlock / 32; ++wv) v = threadIdx.x < 3 ? fminf(v, s[wv][threadIdx.x]) : fmaxf(v, s[wv][threadIdx.x]);
        out6[threadIdx.x] = v;
    }
}

__global__ void __launch_bounds__(kBlock) k_bbox_partial(const float4* __restrict__ pos, int n, float* __restrict__ partial)
{
    const float inf = __int_as_float(0x7f800000);
    float lo[3] = {inf, inf, inf}, hi[3] = {-inf, -inf, -inf};
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
    {
        const float4 p = __ldg(pos + i);
        lo[0] = fminf(lo[0], p.x); lo[1] = fminf(lo[1], p.y); lo[2] = fminf(lo[2], p.z);
        hi[0] = fmaxf(hi[0], p.x); hi[1] = fmaxf(hi[1], p.y); hi[2] = fmaxf(hi[2], p.z);
    }
    block_minmax(lo, hi, partial + 6 * blockIdx.x);
}

__global__ void __launch_bounds__(kBlock) k_bbox_final(const float* __restrict__ partial, int count, float* __restrict__ out6)
{
    const float inf = __int_as_float(0x7f800000);
    float lo[3] = {inf, inf, inf}, hi[3] = {-inf, -inf, -inf};
    for (int b = threadIdx.x; b < count; b += blockDim.x)
    {
#pragma unroll
        for (int k = 0; k < 3; ++k) { lo[k] = fminf(lo[k], partial[6 * b + k]); hi[k] = fmaxf(hi[k], partial[6 * b + 3 + k]); }
    }
    block_minmax(lo, hi, out6);
}

// ---- keys ----------------------------------------------------------------------------------------------------------
__device__ __forceinline__ unsigned long long spread21(unsigned long long v)
{
    v &= 0x1FFFFFull;
    v = (v | (v << 32)) & 0x1F00000000FFFFull;
    v = (v | (v << 16)) & 0x1F0000FF0000FFull;
    v = (v | (v << 8)) & 0x100F00F00F00F00Full;
    v = (v | (v << 4)) & 0x10C30C30C30C30C3ull;
    v = (v | (v << 2)) & 0x1249249249249249ull;
    return v;
}

// q = min(trunc((p - lo) / span * 2097151), 2097151) in float32, one rounding per operation (this file is compiled
// without contraction), span = max(hi - lo, 1e-12)
__device__ __forceinline__ unsigned long long quantise21(float p, float lo, float hi)
{
    const float span = fmaxf(hi - lo, 1e-12f);
    const float t = ((p - lo) / span) * 2097151.0f;
    unsigned long long q = t > 0.f ? (unsigned long long)t : 0ull;  // NaN and negatives -> 0
    return q < 2097151ull ? q : 2097151ull;
}

__global__ void __launch_bounds__(kBlock) k_morton_keys(const float4* __restrict__ pos, int n, const float* __restrict__ bbox,
                                                         unsigned long long* __restrict__ keys, int* __restrict__ index)
{
    const float lx = bbox[0], ly = bbox[1], lz = bbox[2], hx = bbox[3], hy = bbox[4], hz = bbox[5];
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
    {
        const float4 p = __ldg(pos + i);
        keys[i] = spread21(quantise21(p.x, lx, hx)) | (spread21(quantise21(p.y, ly, hy)) << 1) | (spread21(quantise21(p.z, lz, hz)) << 2);
        index[i] = i;
    }
}

// ---- radix sort ----------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kBlock) k_radix_histogram(const unsigned long long* __restrict__ keys, int n, int shift,
                                                             unsigned* __restrict__ hist, int blocks)
{
    __shared__ unsigned s_hist[kRadixBins];
    s_hist[threadIdx.x] = 0;  // kBlock == kRadixBins
    __syncthreads();
    const int base = blockIdx.x * kRadixTile;
#pragma unroll
    for (int j = 0; j < kRadixItems; ++j)
    {
        const int i = base + j * kBlock + threadIdx.x;
        if (i < n) atomicAdd(&s_hist[(unsigned)(__ldg(keys + i) >> shift) & (kRadixBins - 1)], 1u);
    }
    __syncthreads();
    hist[(size_t)threadIdx.x * blocks + blockIdx.x] = s_hist[threadIdx.x];
}

// One block per digit: exclusive scan of that digit's per-block counts in place, and the digit's total. (A first version
// with a single block walking the whole [digit][block] array took 0.87 ms per pass for 10 M keys, 80 % of the sort.)
__global__ void __launch_bounds__(kBlock) k_radix_scan(unsigned* __restrict__ data, int blocks, unsigned* __restrict__ totals)
{
    constexpr int PER = 8;
    __shared__ unsigned s_warp[kBlock / 32];
    __shared__ unsigned s_carry;
    unsigned* row = data + (size_t)blockIdx.x * blocks;
    if (threadIdx.x == 0) s_carry = 0;
    __syncthreads();
    for (int base = 0; base < blocks; base += kBlock * PER)
    {
        unsigned v[PER];
        unsigned sum = 0;
        const int first = base + threadIdx.x * PER;
#pragma unroll
        for (int k = 0; k < PER; ++k) { v[k] = first + k < blocks ? row[first + k] : 0u; sum += v[k]; }
        unsigned incl = sum;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1)
        {
            unsigned t = __shfl_up_sync(0xffffffffu, incl, o);
            if ((threadIdx.x & 31) >= o) incl += t;
        }
        if ((threadIdx.x & 31) == 31) s_warp[threadIdx.x >> 5] = incl;
        __syncthreads();
        unsigned before = s_carry;
        for (int w = 0; w < (int)(threadIdx.x >> 5); ++w) before += s_warp[w];
        unsigned run = before + incl - sum;
#pragma unroll
        for (int k = 0; k < PER; ++k)
        {
            if (first + k < blocks) row[first + k] = run;
            run += v[k];
        }
        __syncthreads();
        if (threadIdx.x == kBlock - 1) s_carry = run;
        __syncthreads();
    }
    if (threadIdx.x == 0) totals[blockIdx.x] = s_carry;
}

// Stable scatter of one tile (2048 keys) per block. Warp w owns keys [256 w, 256 w + 256) of the tile and keeps them in
// registers (8 rounds of 32 consecutive keys). Three block-wide barriers per tile:
//   1. every warp counts its digits (match.any per round, the lowest lane of each group adds the group size);
//   2. thread d turns the per-warp counts of digit d into places inside the tile sorted by digit (tile prefix of the
//      digit + warps before), and remembers where the tile's run of digit d starts in the output;
//   3. every warp walks its rounds again (with the groups it found in step 1): place = its digit's place + keys of that
//      digit in earlier rounds + rank in the round (per-warp running counts in the same shared array, __syncwarp only); keys and indices go to that place of
//      a shared-memory copy of the tile;
//   4. the tile leaves in sorted order: neighbouring threads write neighbouring addresses of a digit's run (8 keys per
//      digit and tile on average), instead of every lane writing a sector of its own.
// (Versions without the staged copy: 0.18-0.19 ms per pass for 10 M keys, stores 25 % efficient.)
__global__ void __launch_bounds__(kBlock) k_radix_scatter(const unsigned long long* __restrict__ keys_in, const int* __restrict__ index_in,
                                                           int n, int shift, const unsigned* __restrict__ offsets, int blocks,
                                                           const unsigned* __restrict__ totals,
                                                           unsigned long long* __restrict__ keys_out, int* __restrict__ index_out)
{
    __shared__ unsigned s_count[kBlock / 32][kRadixBins];
    __shared__ unsigned s_tot[kBlock / 32];
    __shared__ unsigned s_tile_prefix[kRadixBins];   // keys of the tile with a smaller digit
    __shared__ unsigned s_out_base[kRadixBins];      // where the tile's run of the digit starts in the output
    __shared__ unsigned long long s_key[kRadixTile];
    __shared__ int s_idx[kRadixTile];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // digit base: keys with smaller digits (exclusive scan of the 256 digit totals, done by every block for itself) + keys
    // with this digit in earlier blocks
    {
        const unsigned t = totals[threadIdx.x];
        unsigned incl = t;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1)
        {
            unsigned u = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += u;
        }
        if (lane == 31) s_tot[warp] = incl;
#pragma unroll
        for (int w = 0; w < kBlock / 32; ++w) s_count[w][threadIdx.x] = 0;
        __syncthreads();
        unsigned before = 0;
        for (int w = 0; w < warp; ++w) before += s_tot[w];
        s_out_base[threadIdx.x] = before + incl - t + offsets[(size_t)threadIdx.x * blocks + blockIdx.x];
    }
    const int tile_base = blockIdx.x * kRadixTile;
    const int first = tile_base + warp * (kRadixItems * 32) + lane;
    unsigned long long key[kRadixItems];
    int idx[kRadixItems];
    unsigned digit[kRadixItems];
#pragma unroll
    for (int j = 0; j < kRadixItems; ++j)
    {
        const int i = first + j * 32;
        const bool live = i < n;
        key[j] = live ? __ldg(keys_in + i) : 0ull;
        idx[j] = live ? __ldg(index_in + i) : 0;
        // dead lanes get a digit value no live key can have, so they form their own group
        digit[j] = live ? (unsigned)(key[j] >> shift) & (kRadixBins - 1) : kRadixBins;
    }
    unsigned* cnt = s_count[warp];
    unsigned peers_of[kRadixItems];  // lanes of the round with the same digit: found once, used by both walks (match.any is slow)
#pragma unroll
    for (int j = 0; j < kRadixItems; ++j)
    {
        const unsigned peers = __match_any_sync(0xffffffffu, digit[j]);
        peers_of[j] = peers;
        if (digit[j] < kRadixBins && (peers & ((1u << lane) - 1u)) == 0) cnt[digit[j]] += __popc(peers);
        __syncwarp();
    }
    __syncthreads();
    {
        // thread d: the tile's count of digit d, its exclusive prefix over the digits, then per-warp places inside the tile
        const unsigned d = threadIdx.x;
        unsigned mine = 0;
#pragma unroll
        for (int w = 0; w < kBlock / 32; ++w) mine += s_count[w][d];
        unsigned incl = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1)
        {
            unsigned u = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += u;
        }
        __syncthreads();  // s_tot is reused: its readers above are done
        if (lane == 31) s_tot[warp] = incl;
        __syncthreads();
        unsigned before = 0;
        for (int w = 0; w < warp; ++w) before += s_tot[w];
        unsigned run = before + incl - mine;
        s_tile_prefix[d] = run;
#pragma unroll
        for (int w = 0; w < kBlock / 32; ++w)
        {
            const unsigned c = s_count[w][d];
            s_count[w][d] = run;
            run += c;
        }
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < kRadixItems; ++j)
    {
        const unsigned peers = peers_of[j];
        const unsigned rank = __popc(peers & ((1u << lane) - 1u));
        unsigned at = 0;
        if (digit[j] < kRadixBins) at = cnt[digit[j]] + rank;
        __syncwarp();
        if (digit[j] < kRadixBins && rank == 0) cnt[digit[j]] += __popc(peers);  // the next rounds of this warp start behind this group
        __syncwarp();
        if (digit[j] < kRadixBins)
        {
            s_key[at] = key[j];
            s_idx[at] = idx[j];
        }
    }
    __syncthreads();
    const int live_keys = min(kRadixTile, n - tile_base);
    for (int e = threadIdx.x; e < live_keys; e += kBlock)
    {
        const unsigned long long k = s_key[e];
        const unsigned d = (unsigned)(k >> shift) & (kRadixBins - 1);
        const unsigned at = s_out_base[d] + ((unsigned)e - s_tile_prefix[d]);
        keys_out[at] = k;
        index_out[at] = s_idx[e];
    }
}

// ---- apply a permutation to rows -----------------------------------------------------------------------------------
template <int WORDS>
__global__ void __launch_bounds__(kBlock) k_permute_rows(const uint32_t* __restrict__ src, uint32_t* __restrict__ dst,
                                                          const int* __restrict__ order, int n)
{
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
    {
        const size_t from = (size_t)__ldg(order + i) * WORDS, to = (size_t)i * WORDS;
        if (WORDS % 4 == 0)
        {
#pragma unroll
            for (int k = 0; k < WORDS / 4; ++k)
                reinterpret_cast<uint4*>(dst + to)[k] = __ldg(reinterpret_cast<const uint4*>(src + from) + k);
        }
        else
        {
#pragma unroll
            for (int k = 0; k < WORDS; ++k) dst[to + k] = __ldg(src + from + k);
        }
    }
}

// ---- ComputeRadius(n), SceneData.cpp:441-484: distance to the n-th nearest other point, exact -----------------------
// (the reference builds a saiga KD-tree on the host; here: a uniform grid over the bounding box, points sorted by cell
// with the radix sort above, and per point a search over growing cubes of cells that stops as soon as the (n+1)-th
// smallest squared distance found - the point itself included, as in the reference - cannot be beaten from outside
// the cube). Distances are float32: ((dx*dx + dy*dy) + dz*dz), no contraction; the result is the square root of the
// (n+1)-th smallest such value, which does not depend on the order in which the candidates are seen.
constexpr int kGridMax = 256;   // cells per axis at most: 2^24 cells, three radix passes
constexpr int kKnnMax = 16;

struct GridParams
{
    float lo[3];
    float cell;      // edge length of a cell
    float inv_cell;
    int dim[3];
    int status;      // set by k_knn_distance when a query gave up (see kKnnVisitLimit)
};
// Most points one query of k_knn_distance looks at before it gives up. The grid is sized for a few points per cell, and a
// query of an ordinary cloud looks at tens to a few hundred; a cloud with millions of coincident points, or with all its
// points in a corner of a bounding box that one far outlier stretched, puts them into one cell, and every query would
// walk them all: hours of one kernel. A query that reaches the limit writes the bound it has, raises the status word,
// and every query that starts afterwards returns at once; the entry point then reports ADOP_ERR_SIZE_LIMIT.
constexpr int kKnnVisitLimit = 1 << 16;

__global__ void k_grid_params(const float* __restrict__ bbox, int n, float per_cell, GridParams* __restrict__ out)
{
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    GridParams g;
    float ext[3], longest = 0.f, volume = 1.f;
    for (int k = 0; k < 3; ++k)
    {
        g.lo[k] = bbox[k];
        ext[k] = fmaxf(bbox[3 + k] - bbox[k], 1e-12f);
        longest = fmaxf(longest, ext[k]);
    }
    for (int k = 0; k < 3; ++k) volume *= fmaxf(ext[k], longest * 1e-3f);  // flat clouds: do not let one thin axis shrink the cells
    float cell = cbrtf(volume * per_cell / (float)n);
    cell = fmaxf(cell, longest / (float)kGridMax * 1.0001f);
    g.cell = cell;
    g.inv_cell = 1.0f / cell;
    for (int k = 0; k < 3; ++k)
    {
        int d = (int)(ext[k] * g.inv_cell) + 1;
        g.dim[k] = d < 1 ? 1 : (d > kGridMax ? kGridMax : d);
    }
    g.status = 0;
    *out = g;
}

__device__ __forceinline__ int cell_coord(float p, float lo, float inv_cell, int dim)
{
    int c = (int)((p - lo) * inv_cell);
    return c < 0 ? 0 : (c >= dim ? dim - 1 : c);
}

__global__ void __launch_bounds__(kBlock) k_cell_keys(const float4* __restrict__ pos, int n, const GridParams* __restrict__ gp,
                                                       unsigned long long* __restrict__ keys, int* __restrict__ index)
{
    const GridParams g = *gp;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
    {
        const float4 p = __ldg(pos + i);
        const int cx = cell_coord(p.x, g.lo[0], g.inv_cell, g.dim[0]);
        const int cy = cell_coord(p.y, g.lo[1], g.inv_cell, g.dim[1]);
        const int cz = cell_coord(p.z, g.lo[2], g.inv_cell, g.dim[2]);
        keys[i] = (unsigned long long)((cz * g.dim[1] + cy) * g.dim[0] + cx);
        index[i] = i;
    }
}

__global__ void __launch_bounds__(kBlock) k_cell_bounds(const unsigned long long* __restrict__ sorted_keys, int n, int* __restrict__ start,
                                                         int* __restrict__ end)
{
    for (int j = blockIdx.x * blockDim.x + threadIdx.x; j < n; j += gridDim.x * blockDim.x)
    {
        const unsigned long long c = sorted_keys[j];
        if (j == 0 || sorted_keys[j - 1] != c) start[c] = j;
        if (j == n - 1 || sorted_keys[j + 1] != c) end[c] = j + 1;
    }
}

// KT > 0: k known at compile time (the list of the k+1 smallest stays in registers); KT = 0: any k up to kKnnMax
template <int KT>
__global__ void __launch_bounds__(kBlock) k_knn_distance(const float4* __restrict__ sorted_pos, const int* __restrict__ order, int n,
                                                          const GridParams* __restrict__ gp, const int* __restrict__ start,
                                                          const int* __restrict__ end, int k_runtime, float* __restrict__ out)
{
    constexpr int KCAP = KT > 0 ? KT : kKnnMax;
    const int k = KT > 0 ? KT : k_runtime;
    const GridParams g = *gp;
    const float inf = __int_as_float(0x7f800000);
    volatile int* status = const_cast<volatile int*>(&gp->status);
    for (int j = blockIdx.x * blockDim.x + threadIdx.x; j < n; j += gridDim.x * blockDim.x)
    {
        if (*status != 0) { out[__ldg(order + j)] = inf; continue; }  // another query gave up: drain
        int visited = 0;
        const float4 p = __ldg(sorted_pos + j);
        const int cx = cell_coord(p.x, g.lo[0], g.inv_cell, g.dim[0]);
        const int cy = cell_coord(p.y, g.lo[1], g.inv_cell, g.dim[1]);
        const int cz = cell_coord(p.z, g.lo[2], g.inv_cell, g.dim[2]);
        float best[KCAP + 1];
        float kth = inf;
        for (int r = 1;; ++r)
        {
#pragma unroll
            for (int q = 0; q <= KCAP; ++q) best[q] = inf;
            const int x0 = max(cx - r, 0), x1 = min(cx + r, g.dim[0] - 1);
            const int y0 = max(cy - r, 0), y1 = min(cy + r, g.dim[1] - 1);
            const int z0 = max(cz - r, 0), z1 = min(cz + r, g.dim[2] - 1);
            for (int z = z0; z <= z1; ++z)
                for (int y = y0; y <= y1; ++y)
                {
                    // the cells of a row are consecutive keys, and so are their points in the sorted array
                    const int row = (z * g.dim[1] + y) * g.dim[0];
                    int a = -1, b = -1;
                    for (int x = x0; x <= x1; ++x)
                    {
                        const int e = __ldg(end + row + x);
                        if (e == 0) continue;  // empty cell
                        if (a < 0) a = __ldg(start + row + x);
                        b = e;
                    }
                    visited += b - a;
                    if (visited > kKnnVisitLimit) { *status = 1; b = a; }  // give up: the rows left are skipped as well
                    for (int m = a; m < b; ++m)
                    {
                        const float4 o = __ldg(sorted_pos + m);
                        const float dx = p.x - o.x, dy = p.y - o.y, dz = p.z - o.z;
                        const float d2 = (dx * dx + dy * dy) + dz * dz;
                        if (d2 < best[k])
                        {
                            // insertion into the ascending list of the k+1 smallest
                            float carry = d2;
#pragma unroll
                            for (int q = 0; q <= KCAP; ++q)
                                if (q <= k && carry < best[q]) { const float t = best[q]; best[q] = carry; carry = t; }
                        }
                    }
                }
            kth = best[k];
            if (visited > kKnnVisitLimit) break;
            const bool whole = x0 == 0 && y0 == 0 && z0 == 0 && x1 == g.dim[0] - 1 && y1 == g.dim[1] - 1 && z1 == g.dim[2] - 1;
            if (whole) break;
            // nothing outside the cube is nearer than the nearest face that is not a face of the grid itself
            float reach = inf;
            if (x0 > 0) reach = fminf(reach, p.x - (g.lo[0] + (float)x0 * g.cell));
            if (y0 > 0) reach = fminf(reach, p.y - (g.lo[1] + (float)y0 * g.cell));
            if (z0 > 0) reach = fminf(reach, p.z - (g.lo[2] + (float)z0 * g.cell));
            if (x1 < g.dim[0] - 1) reach = fminf(reach, (g.lo[0] + (float)(x1 + 1) * g.cell) - p.x);
            if (y1 < g.dim[1] - 1) reach = fminf(reach, (g.lo[1] + (float)(y1 + 1) * g.cell) - p.y);
            if (z1 < g.dim[2] - 1) reach = fminf(reach, (g.lo[2] + (float)(z1 + 1) * g.cell) - p.z);
            reach -= 1.0e-4f * g.cell;  // cell faces are rounded numbers (up to 256 cells times one float32 rounding each)
            if (reach > 0.f && kth <= reach * reach) break;
        }
        out[__ldg(order + j)] = sqrtf(kth);
    }
}

// data(3) = data(0) * sqrt(1 / u), u uniform in (0, 1] (SceneData.cpp:476-482; the reference draws u from its global
// random generator, here it is the counter hash of (seed, 1, point))
__global__ void __launch_bounds__(kBlock) k_radius_sample(const float* __restrict__ distance, int n, unsigned seed, float* __restrict__ radius)
{
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
    {
        const float u = (float)((hash_u32(seed, 1u, (unsigned)i) >> 8) + 1u) * (1.0f / 16777216.0f);
        radius[i] = distance[i] * sqrtf(1.0f / u);
    }
}

// ---- RandomBlockShuffle(256) and SortBlocksByRadius(256), SceneData.cpp:101-103, 671-684 -----------------------------
// Blocks of `block` consecutive points are put into a seeded pseudo-random order (key = hash_u32(seed, 0, block number),
// ties by block number); points past the last full block stay where they are.
__global__ void __launch_bounds__(kBlock) k_block_keys(int blocks, unsigned seed, unsigned long long* __restrict__ keys, int* __restrict__ index)
{
    for (int b = blockIdx.x * blockDim.x + threadIdx.x; b < blocks; b += gridDim.x * blockDim.x)
    {
        keys[b] = ((unsigned long long)hash_u32(seed, 0u, (unsigned)b) << 32) | (unsigned)b;
        index[b] = b;
    }
}
__global__ void __launch_bounds__(kBlock) k_expand_block_order(const int* __restrict__ block_order, int blocks, int block, int n,
                                                                int* __restrict__ order)
{
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
    {
        const int b = i / block;
        order[i] = b < blocks ? __ldg(block_order + b) * block + (i - b * block) : i;
    }
}

// Inside every full block of 256 points: ascending drop-out radius (position.w), equal radii by index. One thread block
// per point block, bitonic network in shared memory on (orderable radius bits << 32 | index in block): keys are unique.
__global__ void __launch_bounds__(kBlock) k_sort_blocks_by_radius(const float4* __restrict__ pos, int n, int* __restrict__ order)
{
    __shared__ unsigned long long s_key[kBlock];
    const int base = blockIdx.x * kBlock;
    if (base + kBlock > n)
    {
        // the incomplete last block is left alone (SceneData.cpp:673)
        if (base + (int)threadIdx.x < n) order[base + threadIdx.x] = base + threadIdx.x;
        return;
    }
    unsigned bits = __float_as_uint(__ldg(pos + base + threadIdx.x).w);
    bits = (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);  // total order of the floats as unsigned integers
    s_key[threadIdx.x] = ((unsigned long long)bits << 32) | threadIdx.x;
    __syncthreads();
    for (int k = 2; k <= kBlock; k <<= 1)
        for (int j = k >> 1; j > 0; j >>= 1)
        {
            const int partner = threadIdx.x ^ j;
            if (partner > (int)threadIdx.x)
            {
                const unsigned long long a = s_key[threadIdx.x], b = s_key[partner];
                const bool up = (threadIdx.x & k) == 0;
                if ((a > b) == up) { s_key[threadIdx.x] = b; s_key[partner] = a; }
            }
            __syncthreads();
        }
    order[base + threadIdx.x] = base + (int)(s_key[threadIdx.x] & 0xFFFFFFFFu);
}

// keys[0] / index[0] of the workspace -> the sorted indices in `order` (stable); `passes` digits of 8 bits are sorted
static void radix_sort_passes(const MortonWorkspace& w, int n, int passes, int* order, cudaStream_t st)
{
    int cur = 0;
    for (int pass = 0; pass < passes; ++pass)
    {
        const int shift = pass * kRadixBits;
        // the last pass writes the indices straight into the caller's array
        int* index_out = pass == passes - 1 ? order : w.index[cur ^ 1];
        ADOP_LAUNCH("k_radix_histogram", st, (k_radix_histogram<<<w.blocks, kBlock, 0, st>>>(w.keys[cur], n, shift, w.hist, w.blocks)));
        ADOP_LAUNCH("k_radix_scan", st, (k_radix_scan<<<kRadixBins, kBlock, 0, st>>>(w.hist, w.blocks, w.totals)));
        ADOP_LAUNCH("k_radix_scatter", st, (k_radix_scatter<<<w.blocks, kBlock, 0, st>>>(w.keys[cur], w.index[cur], n, shift, w.hist, w.blocks,
                                                                                        w.totals, w.keys[cur ^ 1], index_out)));
        cur ^= 1;
    }
}

}  // namespace adop

using namespace adop;

extern "C" size_t adop_points_morton_workspace_bytes(int32_t num_points)
{
    if (num_points <= 0) return 0;
    return morton_layout(num_points, nullptr, nullptr);
}

extern "C" adop_status adop_points_morton_order(const float* position, int32_t num_points, int32_t* order, void* workspace,
                                                size_t workspace_bytes, void* stream)
{
    if (!position || !order || !workspace || num_points <= 0) return ADOP_ERR_INVALID_ARGUMENT;
    if ((reinterpret_cast<uintptr_t>(position) & 15) || (reinterpret_cast<uintptr_t>(workspace) & 255)) return ADOP_ERR_INVALID_ARGUMENT;
    if (num_points > 0x7F000000) return ADOP_ERR_SIZE_LIMIT;
    MortonWorkspace w;
    if (workspace_bytes < morton_layout(num_points, static_cast<char*>(workspace), &w)) return ADOP_ERR_WORKSPACE_TOO_SMALL;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int n = num_points;
    const float4* pos = reinterpret_cast<const float4*>(position);
    int bbox_blocks = (n + kBlock - 1) / kBlock;
    if (bbox_blocks > kBboxBlocks) bbox_blocks = kBboxBlocks;
    float* bbox_final = w.bbox + 6 * kBboxBlocks;
    ADOP_LAUNCH("k_bbox", st, (k_bbox_partial<<<bbox_blocks, kBlock, 0, st>>>(pos, n, w.bbox)));
    ADOP_LAUNCH("k_bbox", st, (k_bbox_final<<<1, kBlock, 0, st>>>(w.bbox, bbox_blocks, bbox_final)));
    int grid = (n + kBlock - 1) / kBlock;
    if (grid > sm_count() * 8) grid = sm_count() * 8;
    ADOP_LAUNCH("k_morton_keys", st, (k_morton_keys<<<grid, kBlock, 0, st>>>(pos, n, bbox_final, w.keys[0], w.index[0])));
    radix_sort_passes(w, n, kRadixPasses, order, st);
    ADOP_CUDA_TRY(cudaGetLastError());
    return ADOP_OK;
}

extern "C" adop_status adop_points_permute(const void* src, void* dst, const int32_t* order, int32_t num_rows, int32_t row_bytes,
                                           void* stream)
{
    if (!src || !dst || !order || num_rows <= 0 || src == dst) return ADOP_ERR_INVALID_ARGUMENT;
    if (row_bytes <= 0 || row_bytes % 4 != 0) return ADOP_ERR_INVALID_ARGUMENT;
    const bool wide = row_bytes % 16 == 0;
    if (wide && ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15)) return ADOP_ERR_INVALID_ARGUMENT;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int grid = (num_rows + kBlock - 1) / kBlock;
    if (grid > sm_count() * 16) grid = sm_count() * 16;
    const uint32_t* s = static_cast<const uint32_t*>(src);
    uint32_t* d = static_cast<uint32_t*>(dst);
    switch (row_bytes / 4)
    {
        case 1: ADOP_LAUNCH("k_permute_rows", st, (k_permute_rows<1><<<grid, kBlock, 0, st>>>(s, d, order, num_rows))); break;
        case 2: ADOP_LAUNCH("k_permute_rows", st, (k_permute_rows<2><<<grid, kBlock, 0, st>>>(s, d, order, num_rows))); break;
        case 3: ADOP_LAUNCH("k_permute_rows", st, (k_permute_rows<3><<<grid, kBlock, 0, st>>>(s, d, order, num_rows))); break;
        case 4: ADOP_LAUNCH("k_permute_rows", st, (k_permute_rows<4><<<grid, kBlock, 0, st>>>(s, d, order, num_rows))); break;
        case 8: ADOP_LAUNCH("k_permute_rows", st, (k_permute_rows<8><<<grid, kBlock, 0, st>>>(s, d, order, num_rows))); break;
        case 16: ADOP_LAUNCH("k_permute_rows", st, (k_permute_rows<16><<<grid, kBlock, 0, st>>>(s, d, order, num_rows))); break;
        default: return ADOP_ERR_UNSUPPORTED;
    }
    ADOP_CUDA_TRY(cudaGetLastError());
    return ADOP_OK;
}

extern "C" adop_status adop_points_block_shuffle_order(int32_t num_points, int32_t block, uint32_t seed, int32_t* order, void* workspace,
                                                       size_t workspace_bytes, void* stream)
{
    if (!order || !workspace || num_points <= 0 || block <= 0) return ADOP_ERR_INVALID_ARGUMENT;
    if (reinterpret_cast<uintptr_t>(workspace) & 255) return ADOP_ERR_INVALID_ARGUMENT;
    if (num_points > 0x7F000000) return ADOP_ERR_SIZE_LIMIT;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int blocks = num_points / block;
    int grid = (num_points + kBlock - 1) / kBlock;
    if (grid > sm_count() * 16) grid = sm_count() * 16;
    if (blocks < 2)
    {
        ADOP_LAUNCH("k_expand_block_order", st, (k_expand_block_order<<<grid, kBlock, 0, st>>>(nullptr, 0, block, num_points, order)));
        ADOP_CUDA_TRY(cudaGetLastError());
        return ADOP_OK;
    }
    // the workspace of a Morton reorder of the same cloud is always large enough (one key per block of points here)
    MortonWorkspace w;
    if (workspace_bytes < morton_layout(blocks, static_cast<char*>(workspace), &w) + align256(sizeof(int) * (size_t)blocks))
        return ADOP_ERR_WORKSPACE_TOO_SMALL;
    int* block_order = reinterpret_cast<int*>(static_cast<char*>(workspace) + morton_layout(blocks, nullptr, nullptr));
    int gb = (blocks + kBlock - 1) / kBlock;
    ADOP_LAUNCH("k_block_keys", st, (k_block_keys<<<gb, kBlock, 0, st>>>(blocks, seed, w.keys[0], w.index[0])));
    radix_sort_passes(w, blocks, kRadixPasses, block_order, st);
    ADOP_LAUNCH("k_expand_block_order", st, (k_expand_block_order<<<grid, kBlock, 0, st>>>(block_order, blocks, block, num_points, order)));
    ADOP_CUDA_TRY(cudaGetLastError());
    return ADOP_OK;
}

extern "C" adop_status adop_points_sort_blocks_by_radius_order(const float* position, int32_t num_points, int32_t* order, void* stream)
{
    if (!position || !order || num_points <= 0 || (reinterpret_cast<uintptr_t>(position) & 15)) return ADOP_ERR_INVALID_ARGUMENT;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int grid = (num_points + kBlock - 1) / kBlock;
    ADOP_LAUNCH("k_sort_blocks_by_radius", st, (k_sort_blocks_by_radius<<<grid, kBlock, 0, st>>>(reinterpret_cast<const float4*>(position),
                                                                                                num_points, order)));
    ADOP_CUDA_TRY(cudaGetLastError());
    return ADOP_OK;
}

static size_t knn_extra_layout(int n, char* base, GridParams** gp, float4** sorted_pos, int** start, int** end, int** order, float** dist)
{
    size_t at = 0;
    auto take = [&](size_t bytes) { size_t o = at; at = align256(at + bytes); return o; };
    const size_t cells = (size_t)kGridMax * kGridMax * kGridMax;
    size_t a = take(sizeof(GridParams)), b = take(sizeof(float4) * (size_t)n), c = take(sizeof(int) * cells), d = take(sizeof(int) * cells);
    size_t e = take(sizeof(int) * (size_t)n), f = take(sizeof(float) * (size_t)n);
    if (base)
    {
        *gp = reinterpret_cast<GridParams*>(base + a);
        *sorted_pos = reinterpret_cast<float4*>(base + b);
        *start = reinterpret_cast<int*>(base + c);
        *end = reinterpret_cast<int*>(base + d);
        *order = reinterpret_cast<int*>(base + e);
        *dist = reinterpret_cast<float*>(base + f);
    }
    return at;
}

extern "C" size_t adop_points_knn_workspace_bytes(int32_t num_points)
{
    if (num_points <= 0) return 0;
    return morton_layout(num_points, nullptr, nullptr) + knn_extra_layout(num_points, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr);
}

extern "C" adop_status adop_points_knn_distance(const float* position, int32_t num_points, int32_t k, float* distance, void* workspace,
                                                size_t workspace_bytes, void* stream)
{
    if (!position || !distance || !workspace || num_points <= 0 || k < 1 || k > kKnnMax) return ADOP_ERR_INVALID_ARGUMENT;
    if ((reinterpret_cast<uintptr_t>(position) & 15) || (reinterpret_cast<uintptr_t>(workspace) & 255)) return ADOP_ERR_INVALID_ARGUMENT;
    if (num_points > 0x7F000000) return ADOP_ERR_SIZE_LIMIT;
    if (workspace_bytes < adop_points_knn_workspace_bytes(num_points)) return ADOP_ERR_WORKSPACE_TOO_SMALL;
    MortonWorkspace w;
    const size_t first = morton_layout(num_points, static_cast<char*>(workspace), &w);
    GridParams* gp; float4* sorted_pos; int *start, *end, *order; float* dist_unused;
    knn_extra_layout(num_points, static_cast<char*>(workspace) + first, &gp, &sorted_pos, &start, &end, &order, &dist_unused);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int n = num_points;
    const float4* pos = reinterpret_cast<const float4*>(position);
    int bbox_blocks = (n + kBlock - 1) / kBlock;
    if (bbox_blocks > kBboxBlocks) bbox_blocks = kBboxBlocks;
    float* bbox_final = w.bbox + 6 * kBboxBlocks;
    ADOP_LAUNCH("k_bbox", st, (k_bbox_partial<<<bbox_blocks, kBlock, 0, st>>>(pos, n, w.bbox)));
    ADOP_LAUNCH("k_bbox", st, (k_bbox_final<<<1, kBlock, 0, st>>>(w.bbox, bbox_blocks, bbox_final)));
    ADOP_LAUNCH("k_grid_params", st, (k_grid_params<<<1, 32, 0, st>>>(bbox_final, n, 2.0f, gp)));
    int grid = (n + kBlock - 1) / kBlock;
    if (grid > sm_count() * 8) grid = sm_count() * 8;
    ADOP_LAUNCH("k_cell_keys", st, (k_cell_keys<<<grid, kBlock, 0, st>>>(pos, n, gp, w.keys[0], w.index[0])));
    radix_sort_passes(w, n, 3, order, st);  // 2^24 cells: three digits; the sorted keys end up in keys[1]
    ADOP_LAUNCH("k_permute_rows", st, (k_permute_rows<4><<<grid, kBlock, 0, st>>>(reinterpret_cast<const uint32_t*>(position),
                                                                                 reinterpret_cast<uint32_t*>(sorted_pos), order, n)));
    const size_t cells = (size_t)kGridMax * kGridMax * kGridMax;
    ADOP_CUDA_TRY(cudaMemsetAsync(end, 0, sizeof(int) * cells, st));  // end == 0 marks an empty cell; start is read only where end != 0
    ADOP_LAUNCH("k_cell_bounds", st, (k_cell_bounds<<<grid, kBlock, 0, st>>>(w.keys[1], n, start, end)));
    if (k == 4)  // ComputeRadius' default
        ADOP_LAUNCH("k_knn_distance", st, (k_knn_distance<4><<<grid, kBlock, 0, st>>>(sorted_pos, order, n, gp, start, end, k, distance)));
    else
        ADOP_LAUNCH("k_knn_distance", st, (k_knn_distance<0><<<grid, kBlock, 0, st>>>(sorted_pos, order, n, gp, start, end, k, distance)));
    ADOP_CUDA_TRY(cudaGetLastError());
    // Scene preprocessing runs once: this call waits for its kernels and reports a cloud that it could not handle.
    int status = 0;
    ADOP_CUDA_TRY(cudaMemcpyAsync(&status, &gp->status, sizeof(int), cudaMemcpyDeviceToHost, st));
    ADOP_CUDA_TRY(cudaStreamSynchronize(st));
    if (status != 0)
    {
        snprintf(last_error_buffer(), 512,
                 "adop_points_knn_distance: a query met more than %d points in the cells around it (coincident points, or a "
                 "bounding box stretched by far outliers): distances are incomplete; remove duplicates / outliers first",
                 kKnnVisitLimit);
        return ADOP_ERR_SIZE_LIMIT;
    }
    return ADOP_OK;
}

extern "C" adop_status adop_points_radius_sample(const float* distance, int32_t num_points, uint32_t seed, float* radius, void* stream)
{
    if (!distance || !radius || num_points <= 0) return ADOP_ERR_INVALID_ARGUMENT;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int grid = (num_points + kBlock - 1) / kBlock;
    if (grid > sm_count() * 16) grid = sm_count() * 16;
    ADOP_LAUNCH("k_radius_sample", st, (k_radius_sample<<<grid, kBlock, 0, st>>>(distance, num_points, seed, radius)));
    ADOP_CUDA_TRY(cudaGetLastError());
    return ADOP_OK;
}
