/* adop_raster.h — C ABI of the B200 one-pixel point rasterizer (libadop_raster.so).
 *
 * Plain pointers and sizes only. Unless a function says "host", every pointer inside the structs is a
 * DEVICE pointer owned by the caller; the library allocates nothing and writes results in place.
 * Each entry point names the reference interface (darglein/ADOP, path:line) that it stands in for.
 * All functions return an adop_status; none aborts, traps or throws.
 */
#ifndef ADOP_RASTER_H
#define ADOP_RASTER_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ADOP_MAX_LAYERS 8
#define ADOP_MAX_CHANNELS 32 /* bound of the argument checks; the kernels are built for 3, 4, 8 and 16 channels and the
                                entry points return ADOP_ERR_UNSUPPORTED (with a message) for other counts */
#define ADOP_MAX_OCAM_POLY 16
#define ADOP_TOUCHED_CHUNK 256

typedef enum adop_status
{
    ADOP_OK                      = 0,
    ADOP_ERR_INVALID_ARGUMENT    = 1,
    ADOP_ERR_UNSUPPORTED         = 2,
    ADOP_ERR_CUDA                = 3,
    ADOP_ERR_WORKSPACE_TOO_SMALL = 4,
    ADOP_ERR_SIZE_LIMIT          = 5
} adop_status;

/* camera models: CameraModel in src/lib/data/SceneData.h:27-31 */
#define ADOP_CAMERA_PINHOLE_DISTORTION 0
#define ADOP_CAMERA_OCAM 1

/* One image of the batch: ReducedImageInfo, src/lib/data/SceneData.h:37-47.
 * crop = the 5 coefficients fx fy cx cy s of crop_transform. */
typedef struct adop_view
{
    int32_t w, h;
    int32_t image_index;
    int32_t camera_index;
    int32_t camera_model;
    float crop[5];
} adop_view;

/* The compute-relevant fields of RenderParams, src/lib/data/Settings.h:16-52 (same names, same defaults
 * through adop_render_params_default). Added: dropout_seed (the reference draws a [B,N] Bernoulli tensor,
 * PointRenderer.cu:1081-1088; here the decision is a hash of (seed, batch slot, point)). */
typedef struct adop_render_params
{
    int32_t test_backward_mode;
    int32_t check_normal;
    float dropout;
    uint32_t dropout_seed;
    float depth_accept;
    int32_t ghost_gradients;
    float drop_out_radius_threshold;
    int32_t drop_out_points_by_radius;
    float distortion_gradient_factor;
    float K_gradient_factor;
    float dist_cutoff;
    int32_t output_background_mask;
    float output_background_mask_value;
    /* fused extras, off by default so that the plain operator stays a drop-in */
    int32_t composite_environment_map; /* out = img + (1 - mask) * env, RenderModule.cpp:106-127 */
} adop_render_params;

/* The tensors the operator reads from the scene modules (PointRenderer.cu:1146-1155, RenderInfo.cpp:25-30):
 *   position   [N,4] f32  xyz + drop-out radius            (NeuralPointCloudCuda.h:34)
 *   normal     [N]   i32  10-bit packed, may be NULL       (NeuralPointCloudCuda.h:36)
 *   index      [N]   i32  descriptor column, NULL=identity (NeuralPointCloudCuda.h:41)
 *   texture    [C,T] f32  descriptors, C = 3, 4, 8 or 16   (NeuralTexture.h:62)
 *   background [C]   f32                                    (NeuralTexture.h:65)
 *   poses      [I,8] f64  world->camera, quaternion xyzw + translation + pad (NeuralStructure.cpp:13-27)
 *   intrinsics [K,cols] f32: pinhole cols=13 (fx fy cx cy s k1..k6 p1 p2), OCam cols=5+m (c d e cx cy a0..)
 *   env_map    [C,eh,ew] f32, may be NULL                  (EnvironmentMap.h:28) */
typedef struct adop_scene
{
    int32_t num_points;
    int32_t num_texels;
    int32_t channels;
    int32_t num_images;
    int32_t num_cameras;
    int32_t intrinsics_cols;
    int32_t env_h, env_w;
    const float* position;
    const int32_t* normal;
    const int32_t* index;
    const float* texture;
    const float* background;
    const double* poses;
    const float* intrinsics;
    const float* env_map;
    /* optional [T,C] copy of `texture` (adop_texture_interleave). The kernels then fetch a point's descriptor as one
     * contiguous vector instead of C values from C planes. The caller refreshes it whenever `texture` changes. */
    const float* texture_interleaved;
    /* optional second cloud, rendered into the same depth and colour buffers before they are resolved (the reference's
     * outlier cloud, PointRenderer.cu:1402-1441: random points around the scene whose descriptors the training drives
     * towards the background). Same tensor layouts as the main cloud; its descriptor columns index the same `texture`.
     * As in the reference it takes part in the forward pass only - the backward pass walks the main cloud - and a point
     * i of it shares the drop-out decision of main point i, so num_outliers <= num_points. NULL / 0 = none. */
    const float* outlier_position;   /* [M,4] */
    const int32_t* outlier_normal;   /* [M], may be NULL */
    const int32_t* outlier_index;    /* [M], NULL = identity */
    int32_t num_outliers;
    int32_t reserved_;
} adop_scene;

/* Per pyramid layer l (size w>>l, h>>l by integer halving, PointRenderer.cu:1015-1016), batch-major:
 *   color  [B,C,h_l,w_l]  output image (PointRenderer.cu:1057)
 *   depth  [B,1,h_l,w_l]  closest depth, 100000 where empty (PointRenderer.cu:1004,1045)
 *   weight [B,1,h_l,w_l]  number of blended points (PointRenderer.cu:1006)
 *   mask   [B,1,h_l,w_l]  1 where covered else output_background_mask_value; NULL unless requested */
typedef struct adop_layer_buffers
{
    float* color;
    float* depth;
    float* weight;
    float* mask;
} adop_layer_buffers;

typedef struct adop_forward_io
{
    adop_layer_buffers layers[ADOP_MAX_LAYERS];
    const uint8_t* dropout_mask; /* optional [B,N]: 1 = dropped; NULL = hash of dropout_seed */
    void* workspace;
    size_t workspace_bytes;
    /* optional, [B, adop_raster_visible_list_ints(N, w, h, layers)] i32: per view, the forward pass lists the points that were
     * accepted on at least one layer, grouped by 32 x 16 screen tile (one bucket of max(2048, 2N / tiles) entries of 16 bytes
     * per tile), so that the backward pass runs per tile over those points, with the tile's pixels in shared memory, instead
     * of over the whole cloud. It takes the place of the [B,N] drop-out tensor the reference saves for backward
     * (PointRenderer.cu:1524). A view with more visible points in one tile than its bucket holds marks its list unusable and
     * the backward pass of that view walks all points (decided on the device). The backward pass overwrites the entries:
     * a list serves one backward call, a second one walks all points. NULL = not recorded. */
    int32_t* visible_list;
    /* optional, per layer [B,1,h_l,w_l] u64 (all of the first num_layers entries or none): for every pixel the minimum
     * over the points landing there of (bits of the depth << 32 | point index), the packed depth|index word of
     * PackIndex / ExtractIndex (PointRendererHelper.h:21-34), which the reference's live path no longer uses. Its
     * high word is bit-identical to `depth`; its low word names the nearest point (the lowest index among ties), which
     * the 32-bit depth buffer cannot tell and which does not depend on the order the GPU visits the points in.
     * Empty pixels hold (bits of 100000.0f << 32 | 0xFFFFFFFF). One extra pass over the points per view. */
    uint64_t* packed_depth[ADOP_MAX_LAYERS];
    /* optional, [ceil(N / ADOP_TOUCHED_CHUNK)] and [ceil(T / ADOP_TOUCHED_CHUNK)] bytes (both or none; needs visible_list):
     * zeroed, then set to 1 for every chunk of ADOP_TOUCHED_CHUNK consecutive points in which a view of this call listed a
     * point for the backward pass, i.e. the only chunks in which the backward pass of these views can add a point or
     * descriptor gradient. The texel flags are the same flags when the scene has no index array (descriptor column =
     * point number) and all 1 otherwise. adop_peer_reduce_gradients uses them to skip what a rank did not touch. */
    uint8_t* touched_points;
    uint8_t* touched_texels;
} adop_forward_io;

/* Gradients (outputs) follow the reference's order {texture, background, points, pose tangents, intrinsics}
 * (PointRenderer.cu:1641-1643). NULL = not requested.
 *   grad_texture    [C,T] f32
 *   grad_background [C]   f32
 *   grad_points     [N,4] f32  xyz = gradient, w = number of contributions until normalised, then 0
 *   grad_pose       [I,6] f64, count_pose [I] f32
 *   grad_intrinsics [K,cols] f32, count_intrinsics [K] f32
 *   grad_env_map    [C,eh,ew] f32 (only with composite_environment_map)
 * accumulate = 0: the library zeroes the gradient buffers first (the reference allocates zeros,
 * PointRenderer.cu:924-948). normalize = 1: divide by the counts as PointRenderer.cu:1609-1637 does;
 * 0 leaves sums and counts so that several ranks can add them up first (adop_raster_normalize_gradients). */
typedef struct adop_backward_io
{
    adop_layer_buffers layers[ADOP_MAX_LAYERS]; /* saved forward results (color, depth, weight) */
    const float* grad_color[ADOP_MAX_LAYERS];   /* upstream gradient, [B,C,h_l,w_l] */
    const uint8_t* dropout_mask;
    float* grad_texture;
    float* grad_background;
    float* grad_points;
    double* grad_pose;
    float* count_pose;
    float* grad_intrinsics;
    float* count_intrinsics;
    float* grad_env_map;
    int32_t accumulate;
    int32_t normalize;
    void* workspace;
    size_t workspace_bytes;
    /* optional: the list the forward call of the same views, scene and parameters filled (see adop_forward_io).
     * The backward pass groups its entries by screen tile inside the same buffer (so it is not const) and leaves what
     * the forward pass wrote untouched: a list can serve several backward calls.
     * NULL = the backward pass walks all points again, as the reference does. */
    int32_t* visible_list;
    /* optional [T,C] scratch: descriptor gradients are then summed there with one vector atomic per visible point and moved
     * into grad_texture [C,T] at the end of the call. Contents on entry are ignored.
     * With grad_texture == NULL the descriptor gradients STAY here, in [T,C] layout (zeroed first unless accumulate):
     * the form adop_peer_reduce_gradients reads from every GPU. */
    float* grad_texture_interleaved;
    /* optional [env_h,env_w,C] scratch (C a multiple of 4): the environment-map gradient is summed there with one
     * vector atomic per bilinear tap and added to grad_env_map [C,env_h,env_w] at the end of the call. */
    float* grad_env_map_interleaved;
} adop_backward_io;

const char* adop_status_string(adop_status s);
/* text of the last CUDA error seen by this thread's calls ("" if none) */
const char* adop_last_error(void);

/* RenderParams defaults, Settings.h:22-52 */
void adop_render_params_default(adop_render_params* p);

/* Bytes of scratch that forward/backward need for views of w x h with `layers` layers and `channels`
 * descriptor channels. Replaces the size-keyed PointRendererCache (PointRenderer.h:96-157). */
size_t adop_raster_workspace_bytes(int32_t w, int32_t h, int32_t layers, int32_t channels);
/* The same plus 16 bytes per point and view of a group of up to four views (about 64 N bytes): with a workspace of at
 * least this size the depth prepass also hands the projected in-image points of each view to the blend kernel, which then
 * neither reads the cloud again nor projects a second time. Same results either way. Whether it pays depends on the view:
 * measured, the forward pass of a 100 M point cloud through the omnidirectional model gets a third faster (expensive
 * projection, a small part of the cloud in the image), while on 1080p pinhole training views with 70 % of a 10 M point cloud
 * in the image the extra stream costs the prepass more than it saves the blend kernel. The host layers of this library
 * ask for it when a batch has omnidirectional views. */
size_t adop_raster_workspace_bytes_full(int32_t num_points, int32_t num_views, int32_t w, int32_t h, int32_t layers,
                                        int32_t channels);

/* [C,T] -> [T,C] (and back, optionally adding to `out`): the descriptor tensor keeps the reference's planar layout
 * at the boundary (NeuralTexture.h:62); these build the interleaved working copy the kernels prefer. */
adop_status adop_texture_interleave(const float* texture, float* out, int32_t channels, int32_t num_texels, void* stream);
adop_status adop_texture_deinterleave(const float* in, float* out, int32_t channels, int32_t num_texels,
                                      int32_t accumulate, void* stream);

/* int32 elements per view of adop_forward_io.visible_list for a cloud of num_points points rendered into views of
 * w x h with `layers` layers (the list keeps a small table per screen tile besides 16 bytes per point). */
size_t adop_raster_visible_list_ints(int32_t num_points, int32_t w, int32_t h, int32_t layers);

/* BlendPointCloudForward, src/lib/rendering/PointRenderer.cu:1389-1531: depth prepass, fuzzy-depth blend,
 * combine-and-fill, mask, and (optionally) the environment-map composite of RenderModule.cpp:106-127.
 * `views` is a HOST array of B entries. stream is a cudaStream_t (NULL = default stream). */
adop_status adop_raster_forward(const adop_scene* scene, const adop_view* views, int32_t num_views,
                                const adop_render_params* params, int32_t num_layers, adop_forward_io* io,
                                void* stream);

/* The forward pass without a caller-owned workspace. No counterpart in the reference (which allocates through
 * libtorch whenever it likes): this entry point exists for hosts that may not allocate device memory at the time
 * they render - a callback running while the allocator is locked, a plugin that only ever receives input and
 * output buffers from its host application, a process with a memory budget fixed at start-up. io->workspace and
 * io->workspace_bytes are ignored; the scratch is a built-in device array of adop_raster_static_scratch_bytes()
 * bytes (32 MiB) that every GPU which loads this library keeps until the process exits. Inputs and outputs are
 * still the caller's.
 *   - Limit: adop_raster_workspace_bytes(w, h, layers, channels) must not exceed that size (e.g. 1024 x 576 with
 *     4 layers and 4 channels fits); larger views return ADOP_ERR_SIZE_LIMIT and adop_last_error() names both sizes.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that device
 *     current). Make that first call outside any stream capture. With CUDA's lazy module loading that first call is
 *     also the one that loads this library's device code and the array itself onto the GPU, so it can need (and fail
 *     for lack of) device memory: make it at start-up, while memory is still available.
 *   - The function itself calls no cudaMalloc / cudaFree and no allocating library routine.
 *   - All calls on a device share the one array. Each call clears what it needs before use, so earlier contents do
 *     not leak into results, but two calls whose kernels overlap on the GPU (different streams, different threads)
 *     race on it: run them one after the other. */
size_t adop_raster_static_scratch_bytes(void);
adop_status adop_raster_forward_static(const adop_scene* scene, const adop_view* views, int32_t num_views,
                                       const adop_render_params* params, int32_t num_layers, adop_forward_io* io,
                                       void* stream);

/* BlendPointCloudBackward, src/lib/rendering/PointRenderer.cu:1549-1644. */
adop_status adop_raster_backward(const adop_scene* scene, const adop_view* views, int32_t num_views,
                                 const adop_render_params* params, int32_t num_layers, adop_backward_io* io,
                                 void* stream);

/* NormalizeGradient calls of PointRenderer.cu:1609-1637, as a separate step for callers that sum the
 * un-normalised gradients of several GPUs first. NULL pointers are skipped. */
adop_status adop_raster_normalize_gradients(float* grad_points, int32_t num_points, double* grad_pose,
                                            const float* count_pose, int32_t num_images, float* grad_intrinsics,
                                            const float* count_intrinsics, int32_t num_cameras,
                                            int32_t intrinsics_cols, void* stream);

/* ---- Gradient exchange between the GPUs of one node, over peer memory -------------------------------------------
 * The reference renders on one GPU and has no counterpart to this section. Views are independent given the scene, so
 * every GPU renders its own views of the replicated scene and the un-normalised gradient sums are added up afterwards.
 * Each rank keeps ALL its gradient outputs of adop_raster_backward in one device block laid out by adop_peer_layout
 * (the same on every rank), exported to the other processes as a CUDA IPC handle. adop_peer_reduce_gradients is one
 * kernel that reads the blocks of all ranks with plain peer loads and, in that one pass,
 *   - sums the descriptor gradients of the texels this rank owns, and writes them in the reference's [C,.] layout,
 *   - sums the point gradients of the points this rank owns and divides by the summed counts (PointRenderer.cu:1620-1627),
 *   - sums pose, intrinsics, background and environment-map gradients in full (every rank gets all of them) and
 *     divides pose and intrinsics by their summed counts (PointRenderer.cu:1609-1637).
 * It is reduce-scatter + all-reduce + de-interleave + NormalizeGradient in one pass over the data; sums run over the
 * ranks in rank order, so every rank computes the same bits. The kernel does not wait for other GPUs: the caller
 * orders it after every rank's backward pass and before anyone's next write to its block (a stream-ordered
 * collective of the caller's communication library on either side, e.g. a one-element all-reduce). */
typedef struct adop_peer_handle
{
    unsigned char bytes[64]; /* a cudaIpcMemHandle_t */
} adop_peer_handle;

/* cudaMalloc of `bytes` (zero-filled) on the current device, plus its handle for the other processes. */
adop_status adop_peer_alloc(size_t bytes, void** ptr, adop_peer_handle* handle);
adop_status adop_peer_free(void* ptr);
/* Map another process's block into this process (peer access between the two GPUs is switched on as needed). */
adop_status adop_peer_open(const adop_peer_handle* handle, void** ptr);
adop_status adop_peer_close(void* ptr);

/* Byte offsets of the gradient tensors inside a rank's block; a count of 0 leaves that tensor out. */
typedef struct adop_peer_layout
{
    int32_t channels;        /* C */
    int32_t num_texels;      /* T: descriptor gradients [T,C] f32 (adop_backward_io.grad_texture_interleaved) */
    int32_t num_points;      /* N: point gradients [N,4] f32, count in .w */
    int32_t num_images;      /* pose gradients [images,6] f64 + counts [images] f32 */
    int32_t num_cameras;     /* intrinsics gradients [cameras, intrinsics_cols] f32 + counts [cameras] f32 */
    int32_t intrinsics_cols;
    int32_t env_h, env_w;    /* environment-map gradient [C,env_h,env_w] f32 */
    int32_t background;      /* 1: background gradient [C] f32 */
    int32_t touched;         /* 1: the block also holds adop_forward_io's touched_points / touched_texels flags of the step, and
                                the reduce kernel reads a peer's descriptor / point gradients only where that peer set them */
    size_t off_texture, off_points, off_pose, off_count_pose, off_intrinsics, off_count_intrinsics, off_background,
        off_env_map;
    size_t off_touched_texels, off_touched_points; /* one byte per ADOP_TOUCHED_CHUNK texels / points */
    size_t off_gathered;     /* scratch of the reduce call: which ranks touched each chunk of the owned ranges */
    size_t total_bytes;
} adop_peer_layout;
/* Fills the offsets (256-byte aligned) and total_bytes from the counts. */
adop_status adop_peer_layout_fill(adop_peer_layout* layout);
/* Rank `rank` of `world` owns elements [*lo, *hi) of `count`: equal shares of ceil(count / world), the last ones shorter. */
void adop_peer_shard_range(int32_t count, int32_t world, int32_t rank, int32_t* lo, int32_t* hi);

typedef struct adop_peer_reduce_out
{
    float* grad_texture_shard;   /* [C, t_hi - t_lo] f32: the owned texels, channel planes as in grad_texture */
    float* grad_points_shard;    /* [n_hi - n_lo, 4] f32: the owned points, xyz divided by the count, w = 0 */
    double* grad_pose;           /* [images,6], divided by the counts */
    float* count_pose;           /* [images], summed */
    float* grad_intrinsics;      /* [cameras, cols], divided by the counts */
    float* count_intrinsics;     /* [cameras], summed */
    float* grad_background;      /* [C] */
    float* grad_env_map;         /* [C,env_h,env_w] */
    int32_t normalize;           /* 0: leave sums (points keep their count in w) */
} adop_peer_reduce_out;
/* blocks[r] = rank r's block as mapped in THIS process (own block: the pointer adop_peer_alloc gave), 1 <= world <= 8.
 * Outputs whose tensor the layout leaves out, or that are NULL, are skipped. Outputs must not lie inside a block. */
adop_status adop_peer_reduce_gradients(const void* const* blocks, int32_t world, int32_t rank,
                                       const adop_peer_layout* layout, const adop_peer_reduce_out* out, void* stream);

/* ---- Optimiser step + parameter all-gather over peer memory ------------------------------------------------------
 * The step after adop_peer_reduce_gradients in a view-sharded training step (the reference trains on one GPU: its
 * optimisers are torch::optim::Adam for the descriptors, NeuralScene.cpp:76-107, and torch::optim::SGD for the point
 * positions, NeuralScene.cpp:204-240, stepped at NeuralScene.cpp:384-411, adop_train.cpp:530-532). Every rank keeps its replica of the two large
 * trainable tensors in one device block of its own, laid out by adop_peer_param_layout: descriptors [C,T], then points
 * [N,4]; the other ranks map it like the gradient blocks. adop_peer_apply_update is one kernel that applies the
 * optimiser to the texels and points this rank owns (the ranges of adop_peer_shard_range, i.e. exactly the gradient shards
 * the reduce kernel produced) and writes every new value into ALL replicas with plain peer stores: optimiser step and
 * all-gather in one pass, with the Adam moments kept for the owned shard only. Same arithmetic, in the same order of
 * operations, as torch::optim::Adam::step (no weight decay, no amsgrad) and SGD without momentum. The kernel does not
 * wait for other GPUs: the caller orders it after every rank's last read of the parameters and before anyone's next one. */
typedef struct adop_peer_param_layout
{
    int32_t channels;    /* C */
    int32_t num_texels;  /* T: descriptors [C,T] f32 */
    int32_t num_points;  /* N: positions [N,4] f32 (0: not part of the block) */
    int32_t reserved;
    size_t off_texture, off_points;
    size_t total_bytes;
} adop_peer_param_layout;
adop_status adop_peer_param_layout_fill(adop_peer_param_layout* layout);

typedef struct adop_peer_update
{
    const float* grad_texture_shard; /* [C, t_hi - t_lo]: adop_peer_reduce_out.grad_texture_shard; NULL = descriptors stay */
    float* adam_m;                   /* [C, t_hi - t_lo] first moments of the owned texels (zero before the first step) */
    float* adam_v;                   /* [C, t_hi - t_lo] second moments */
    const float* grad_points_shard;  /* [n_hi - n_lo, 4]: adop_peer_reduce_out.grad_points_shard; NULL = points stay */
    float lr_texture, beta1, beta2, eps; /* Adam (torch defaults: 0.9, 0.999, 1e-8) */
    int32_t step;                    /* 1 for the first step */
    float lr_points;                 /* SGD */
} adop_peer_update;
/* param_blocks[r] = rank r's parameter block as mapped in THIS process, 1 <= world <= 8. */
adop_status adop_peer_apply_update(void* const* param_blocks, int32_t world, int32_t rank, const adop_peer_param_layout* layout,
                                   const adop_peer_update* update, void* stream);

/* ---- Point-cloud preprocessing on the GPU ----------------------------------------------------------------------
 * point_cloud.ReorderMorton64(), called once per scene at src/lib/data/SceneData.cpp:100 (the function itself is saiga
 * code that is not in the reference tree; the key is this library's definition: each coordinate quantised in float32
 * to 21 bits over the cloud's bounding box, q = min(trunc((p - lo) / max(hi - lo, 1e-12) * 2097151), 2097151), bits
 * interleaved with x lowest). The rasterizer's memory behaviour depends on this order.
 *   position [N,4] f32 (device), order [N] i32 (device, out): order[i] = index of the point that comes i-th; points
 *   with equal keys keep their original order (stable), so the result does not depend on the GPU's scheduling.
 *   workspace: adop_points_morton_workspace_bytes(N) bytes, 256-byte aligned, contents irrelevant. */
size_t adop_points_morton_workspace_bytes(int32_t num_points);
adop_status adop_points_morton_order(const float* position, int32_t num_points, int32_t* order, void* workspace,
                                     size_t workspace_bytes, void* stream);
/* point_cloud.RandomBlockShuffle(256), SceneData.cpp:101 (saiga function; here: blocks of `block` consecutive points
 * in ascending order of hash(seed, block number), the counter hash of the drop-out decision, ties by block number; the
 * points behind the last full block keep their place). order [N] i32 as above. The workspace of a Morton reorder of
 * the same cloud is large enough. */
adop_status adop_points_block_shuffle_order(int32_t num_points, int32_t block, uint32_t seed, int32_t* order, void* workspace,
                                            size_t workspace_bytes, void* stream);
/* SceneData::SortBlocksByRadius(256), SceneData.cpp:671-684: inside every full block of 256 points ascending drop-out
 * radius (position.w); equal radii by index (the reference's std::sort leaves their order open). */
adop_status adop_points_sort_blocks_by_radius_order(const float* position, int32_t num_points, int32_t* order, void* stream);
/* SceneData::ComputeRadius(n), SceneData.cpp:441-484. distance [N] f32 (out): for every point the distance to its
 * k-th nearest OTHER point (the reference asks its KD-tree for k+1 neighbours, the point itself included, and takes the
 * last), exact: the square root of the (k+1)-th smallest float32 value ((dx*dx + dy*dy) + dz*dz) over all points.
 * 1 <= k <= 16 (the reference's default is 4); fewer than k+1 points in the cloud give +inf.
 * The call waits for its kernels (scene preprocessing runs once). A cloud whose points pile up in single cells of the
 * search grid (millions of coincident points; a bounding box stretched by a far outlier) would cost a full scan per
 * query: a query gives up after 65536 visited points, the call returns ADOP_ERR_SIZE_LIMIT and `distance` is incomplete.
 * adop_points_radius_sample then forms the drop-out radius data(3) = distance * sqrt(1 / u) (SceneData.cpp:476-482) with
 * u in (0,1] from the counter hash of (seed, 1, point) instead of the reference's global random generator; the caller
 * stores it in position.w. */
size_t adop_points_knn_workspace_bytes(int32_t num_points);
adop_status adop_points_knn_distance(const float* position, int32_t num_points, int32_t k, float* distance, void* workspace,
                                     size_t workspace_bytes, void* stream);
adop_status adop_points_radius_sample(const float* distance, int32_t num_points, uint32_t seed, float* radius, void* stream);
/* dst row i = src row order[i], rows of row_bytes bytes (4, 8, 12, 16, 32 or 64): positions [N,4], normals, indices,
 * gradient rows, or one descriptor plane at a time. src and dst must not overlap. */
adop_status adop_points_permute(const void* src, void* dst, const int32_t* order, int32_t num_rows, int32_t row_bytes,
                                void* stream);

/* ApplyTangentToPose, src/lib/rendering/PointRenderer.cu:1646-1665: pose <- exp(tangent) * pose, tangent <- 0.
 * tangent [n,6] f64, pose [n,8] f64. */
adop_status adop_apply_tangent(double* tangent, double* pose, int32_t n, void* stream);

/* Photometric tonemapper, NeuralCameraImpl::forward, src/lib/models/NeuralCamera.cpp:258-335, with
 * VignetteNetImpl::forward (:22-42) and CameraResponseNetImpl::forward (:87-135) fused into one pass.
 *   x, out        [B,3,H,W] f32
 *   frame_index   [B] i32  row of exposure / white_balance per image
 *   exposure      [n] f32 or NULL          (exposures_values [n,1,1,1])
 *   white_balance [n,3] f32 or NULL        (white_balance_values [n,3,1,1])
 *   vignette      3 polynomial coefficients then the centre (2), f32[5], or NULL
 *   uv            [B,2,H,W] f32 or NULL = 2*(col/(W-1), row/(H-1))-1 (Dataset.cpp:12-34)
 *   response      [3,K] f32 or NULL (then clamp to [0,1])
 *   leak          leaky-clamp slope used while training (0 = hard clamp) */
typedef struct adop_tonemap_params
{
    int32_t batch, height, width;
    int32_t response_bins;
    int32_t vignette_image_w, vignette_image_h; /* aspect = w / h of VignetteNet's image_size */
    float leak;
    const int32_t* frame_index;
    const float* exposure;
    const float* white_balance;
    const float* vignette;
    const float* uv;
    const float* response;
} adop_tonemap_params;

typedef struct adop_tonemap_grads
{
    float* grad_x;             /* [B,3,H,W] */
    float* grad_exposure;      /* [n] */
    float* grad_white_balance; /* [n,3] */
    float* grad_vignette;      /* [5] */
    float* grad_response;      /* [3,K] */
    int32_t num_frames;        /* n, for zeroing */
    int32_t accumulate;
} adop_tonemap_grads;

/* Per-kernel device timing, the role of the CudaTimerSystem scopes threaded through the reference
 * (NeuralRenderInfo::timer_system, src/lib/rendering/PointRenderer.h:32; scopes at PointRenderer.cu:1414-1447,
 * 1594-1610). While enabled, every kernel launch of this library is bracketed by CUDA events on its stream.
 * adop_profile_collect synchronises those events, adds the times up per kernel name, writes up to max_entries
 * records, forgets what it collected and returns the number of distinct kernels (or -1 on a CUDA error).
 * Per host thread; off by default. */
typedef struct adop_kernel_time
{
    char name[48];
    int32_t launches;
    float total_ms;
} adop_kernel_time;
adop_status adop_profile_enable(int32_t on);
int32_t adop_profile_collect(adop_kernel_time* out, int32_t max_entries);

adop_status adop_tonemap_forward(const adop_tonemap_params* p, const float* x, float* out, void* stream);
adop_status adop_tonemap_backward(const adop_tonemap_params* p, const float* x, const float* grad_out,
                                  adop_tonemap_grads* g, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* ADOP_RASTER_H */
