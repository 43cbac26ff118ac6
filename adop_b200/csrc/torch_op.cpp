// libTorch operator over the C ABI: the reference-facing host side of the rasterizer, in the reference's language.
//
// Mirrors darglein/ADOP's operator surface for this path:
//   torch::autograd::PointRender (src/lib/rendering/PointRenderer.h:37-47, RenderInfo.cpp:34-58)  -> adop::PointRender
//   NeuralRenderInfo             (PointRenderer.h:25-34), registered as a custom class (RenderInfo.cpp:11-15) -> adop::RenderInfo
//   BlendPointCloud              (PointRenderer.h:52, RenderInfo.cpp:19-31)                        -> adop::blend_point_cloud
//   ApplyTangentToPose           (PointRenderer.h:63)                                              -> adop::apply_tangent_to_pose
//   NeuralCameraImpl::forward    (src/lib/models/NeuralCamera.h:128-129)                          -> adop::tonemap (adop::Tonemap)
// Same differentiable inputs in the same order (texture [C,N], background [C], points [N,4], pose tangents [I,6] f64,
// intrinsics [K,cols]), same outputs (L colour tensors, then L masks when requested), gradients in the same order.
// The reference's NeuralRenderInfo points at a NeuralScene (which needs the whole saiga library); RenderInfo carries the
// non-differentiable tensors the operator reads from it directly. All computation happens in libadop_raster.so.
#include <torch/custom_class.h>
#include <torch/library.h>
#include <torch/torch.h>

#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>

#include "adop/adop_raster.h"

namespace adop {

using torch::Tensor;
using torch::autograd::AutogradContext;
using torch::autograd::Variable;
using torch::autograd::variable_list;

struct RenderInfo : torch::CustomClassHolder
{
    // scene tensors that take no gradient (PointRenderer.cu:1146-1155, RenderModule.cpp:106-110)
    Tensor poses;    // [I,8] f64, world -> camera
    c10::optional<Tensor> normal, index, env_map;
    // optional second cloud of the forward pass (scene.outlier_point_cloud_cuda, PointRenderer.cu:1402-1441)
    c10::optional<Tensor> outlier_position, outlier_normal, outlier_index;
    // the batch: ReducedImageInfo per image (SceneData.h:37-47)
    std::vector<adop_view> images;
    adop_render_params params;
    int64_t num_layers = 1;
    // reusable buffers (the role of PointRendererCache, PointRenderer.h:96-157)
    Tensor workspace, texture_interleaved, grad_texture_interleaved;

    RenderInfo() { adop_render_params_default(&params); }

    void set_scene(Tensor poses_, c10::optional<Tensor> normal_, c10::optional<Tensor> index_, c10::optional<Tensor> env_map_)
    {
        TORCH_CHECK(poses_.dim() == 2 && poses_.size(1) == 8 && poses_.scalar_type() == torch::kFloat64, "poses must be [I,8] float64");
        poses = poses_.contiguous();
        normal = normal_; index = index_; env_map = env_map_;
    }
    // render_outliers = true: positions [M,4] f32, packed normals [M] i32 or none, descriptor columns [M] i32 or none
    void set_outlier_cloud(c10::optional<Tensor> position_, c10::optional<Tensor> normal_, c10::optional<Tensor> index_)
    {
        if (position_)
            TORCH_CHECK(position_->is_cuda() && position_->is_contiguous() && position_->dim() == 2 && position_->size(1) == 4 &&
                            position_->scalar_type() == torch::kFloat32,
                        "outlier positions must be a contiguous CUDA [M,4] float32 tensor");
        outlier_position = position_; outlier_normal = normal_; outlier_index = index_;
    }
    // views: [B,5] int64 on the CPU (w, h, image_index, camera_index, camera_model); crops: [B,5] float32 on the CPU
    void set_views(Tensor views, Tensor crops)
    {
        TORCH_CHECK(views.dim() == 2 && views.size(1) == 5 && crops.sizes() == views.sizes(), "views and crops must be [B,5]");
        auto v = views.to(torch::kCPU, torch::kInt64).contiguous();
        auto c = crops.to(torch::kCPU, torch::kFloat32).contiguous();
        images.resize(v.size(0));
        for (int64_t b = 0; b < v.size(0); ++b)
        {
            const int64_t* r = v.data_ptr<int64_t>() + b * 5;
            images[b].w = (int32_t)r[0]; images[b].h = (int32_t)r[1];
            images[b].image_index = (int32_t)r[2]; images[b].camera_index = (int32_t)r[3]; images[b].camera_model = (int32_t)r[4];
            for (int k = 0; k < 5; ++k) images[b].crop[k] = c.data_ptr<float>()[b * 5 + k];
        }
    }
    // RenderParams by name (Settings.h:16-52)
    void set_param(std::string name, double value)
    {
#define ADOP_PARAM_I(field) if (name == #field) { params.field = (int32_t)value; return; }
#define ADOP_PARAM_F(field) if (name == #field) { params.field = (float)value; return; }
        ADOP_PARAM_I(test_backward_mode) ADOP_PARAM_I(check_normal) ADOP_PARAM_F(dropout)
        if (name == "dropout_seed") { params.dropout_seed = (uint32_t)value; return; }
        ADOP_PARAM_F(depth_accept) ADOP_PARAM_I(ghost_gradients) ADOP_PARAM_F(drop_out_radius_threshold)
        ADOP_PARAM_I(drop_out_points_by_radius) ADOP_PARAM_F(distortion_gradient_factor) ADOP_PARAM_F(K_gradient_factor)
        ADOP_PARAM_F(dist_cutoff) ADOP_PARAM_I(output_background_mask) ADOP_PARAM_F(output_background_mask_value)
        ADOP_PARAM_I(composite_environment_map)
#undef ADOP_PARAM_I
#undef ADOP_PARAM_F
        TORCH_CHECK(false, "unknown render parameter ", name);
    }
    void set_num_layers(int64_t n) { num_layers = n; }
};

static void check_status(adop_status st, const char* what)
{
    TORCH_CHECK(st == ADOP_OK, what, ": ", adop_status_string(st), " ", adop_last_error());
}

static adop_scene make_scene(RenderInfo& info, const Tensor& texture, const Tensor& background, const Tensor& points,
                             const Tensor& intrinsics)
{
    TORCH_CHECK(texture.is_cuda() && points.is_cuda() && background.is_cuda() && intrinsics.is_cuda() && info.poses.is_cuda(),
                "the rasterizer takes CUDA tensors only");
    TORCH_CHECK(texture.is_contiguous() && points.is_contiguous() && background.is_contiguous() && intrinsics.is_contiguous(),
                "tensors must be contiguous");
    TORCH_CHECK(texture.scalar_type() == torch::kFloat32 && points.scalar_type() == torch::kFloat32, "texture and points are float32");
    adop_scene sc{};
    sc.num_points = (int32_t)points.size(0);
    sc.num_texels = (int32_t)texture.size(1);
    sc.channels = (int32_t)texture.size(0);
    sc.num_images = (int32_t)info.poses.size(0);
    sc.num_cameras = (int32_t)intrinsics.size(0);
    sc.intrinsics_cols = (int32_t)intrinsics.size(1);
    sc.position = points.data_ptr<float>();
    sc.normal = info.normal ? info.normal->data_ptr<int32_t>() : nullptr;
    sc.index = info.index ? info.index->data_ptr<int32_t>() : nullptr;
    sc.texture = texture.data_ptr<float>();
    sc.background = background.data_ptr<float>();
    sc.poses = info.poses.data_ptr<double>();
    sc.intrinsics = intrinsics.data_ptr<float>();
    if (info.outlier_position)
    {
        sc.outlier_position = info.outlier_position->data_ptr<float>();
        sc.num_outliers = (int32_t)info.outlier_position->size(0);
        sc.outlier_normal = info.outlier_normal ? info.outlier_normal->data_ptr<int32_t>() : nullptr;
        sc.outlier_index = info.outlier_index ? info.outlier_index->data_ptr<int32_t>() : nullptr;
    }
    if (info.env_map)
    {
        Tensor e = *info.env_map;
        TORCH_CHECK(e.dim() == 3 || (e.dim() == 4 && e.size(0) == 1), "env_map must be [C,h,w] or [1,C,h,w]");
        sc.env_map = e.data_ptr<float>();
        sc.env_h = (int32_t)e.size(e.dim() - 2);
        sc.env_w = (int32_t)e.size(e.dim() - 1);
    }
    return sc;
}

// Returns the size the library is told (it picks its kernels by it), which may be less than what an earlier call left behind.
static size_t ensure_workspace(RenderInfo& info, const std::vector<adop_view>& views, int64_t num_layers, const adop_scene& sc,
                               const torch::TensorOptions& opt, bool forward)
{
    // Candidate streams (adop_raster_workspace_bytes_full) pay for views of the omnidirectional model, whose projection is
    // expensive and whose image holds a small part of the cloud; on pinhole training views they measured slower.
    bool ocam = false;
    for (const adop_view& v : views) ocam = ocam || v.camera_model == ADOP_CAMERA_OCAM;
    const size_t need = (forward && ocam)
                            ? adop_raster_workspace_bytes_full(sc.num_points, (int32_t)views.size(), views[0].w, views[0].h, (int32_t)num_layers,
                                                               sc.channels)
                            : adop_raster_workspace_bytes(views[0].w, views[0].h, (int32_t)num_layers, sc.channels);
    TORCH_CHECK(need > 0, "invalid view size / layer count");
    if (!info.workspace.defined() || (size_t)info.workspace.numel() < need)
        info.workspace = torch::empty({(int64_t)need}, opt.dtype(torch::kUInt8));
    if (!info.texture_interleaved.defined() || info.texture_interleaved.size(0) != sc.num_texels || info.texture_interleaved.size(1) != sc.channels)
    {
        info.texture_interleaved = torch::empty({sc.num_texels, sc.channels}, opt);
        info.grad_texture_interleaved = torch::empty({sc.num_texels, sc.channels}, opt);
    }
    return need;
}

// What a forward call used and its backward call must use again, whatever happens to the RenderInfo in between (a second
// forward with other views or another drop-out seed, gradient accumulation, an evaluation render): the reference keeps its
// per-call state in the autograd context as well (the saved drop-out tensor, PointRenderer.cu:1524).
// "no tensor" as an argument of an autograd function: an empty one (an undefined tensor has no device to dispatch on)
static Tensor none_like(const Tensor& x) { return torch::empty({0}, x.options()); }
static bool has(const Tensor& t) { return t.defined() && t.numel() > 0; }
static Tensor blob_of(const void* data, size_t bytes)
{
    Tensor t = torch::empty({(int64_t)bytes}, torch::TensorOptions().dtype(torch::kUInt8).device(torch::kCPU));
    memcpy(t.data_ptr(), data, bytes);
    return t;
}

struct PointRender : public torch::autograd::Function<PointRender>
{
    // returns a tensor for every layer, then (if requested) a mask for every layer.
    // env_map: an undefined tensor takes the RenderInfo's environment map (no gradient for it); a defined one is the
    // differentiable texture of EnvironmentMapImpl (RenderModule.cpp:106-127, EnvironmentMap.cu:107-156) and gets one.
    static variable_list forward(AutogradContext* ctx, Variable texture, Variable background_color, Variable points,
                                 Variable pose_tangents, Variable intrinsics, Variable env_map, torch::IValue info_value)
    {
        auto info = info_value.toCustomClass<RenderInfo>();
        TORCH_CHECK(!info->images.empty(), "RenderInfo has no views");
        c10::cuda::CUDAGuard guard(texture.device());
        cudaStream_t stream = c10::cuda::getCurrentCUDAStream().stream();
        adop_scene sc = make_scene(*info, texture, background_color, points, intrinsics);
        if (has(env_map))
        {
            TORCH_CHECK(env_map.is_cuda() && env_map.is_contiguous() && env_map.scalar_type() == torch::kFloat32, "env_map: contiguous float32 CUDA tensor");
            TORCH_CHECK(env_map.dim() == 3 || (env_map.dim() == 4 && env_map.size(0) == 1), "env_map must be [C,h,w] or [1,C,h,w]");
            TORCH_CHECK(env_map.size(env_map.dim() - 3) == sc.channels, "env_map must have as many channels as the descriptors");
            sc.env_map = env_map.data_ptr<float>();
            sc.env_h = (int32_t)env_map.size(env_map.dim() - 2);
            sc.env_w = (int32_t)env_map.size(env_map.dim() - 1);
        }
        const int B = (int)info->images.size(), L = (int)info->num_layers, C = sc.channels;
        auto opt = texture.options();
        const size_t workspace_bytes = ensure_workspace(*info, info->images, info->num_layers, sc, opt, true);
        check_status(adop_texture_interleave(sc.texture, info->texture_interleaved.data_ptr<float>(), C, sc.num_texels, stream),
                     "adop_texture_interleave");
        sc.texture_interleaved = info->texture_interleaved.data_ptr<float>();
        variable_list color(L), depth(L), weight(L), mask;
        adop_forward_io io{};
        int w = info->images[0].w, h = info->images[0].h;
        for (int l = 0; l < L; ++l, w /= 2, h /= 2)
        {
            color[l] = torch::empty({B, C, h, w}, opt);
            depth[l] = torch::empty({B, 1, h, w}, opt);
            weight[l] = torch::empty({B, 1, h, w}, opt);
            io.layers[l].color = color[l].data_ptr<float>();
            io.layers[l].depth = depth[l].data_ptr<float>();
            io.layers[l].weight = weight[l].data_ptr<float>();
            if (info->params.output_background_mask)
            {
                mask.push_back(torch::empty({B, 1, h, w}, opt));
                io.layers[l].mask = mask.back().data_ptr<float>();
            }
        }
        Tensor visible = torch::empty({B, (int64_t)adop_raster_visible_list_ints(sc.num_points, info->images[0].w, info->images[0].h, L)}, opt.dtype(torch::kInt32));
        io.visible_list = visible.data_ptr<int32_t>();
        io.workspace = info->workspace.data_ptr();
        io.workspace_bytes = workspace_bytes;
        check_status(adop_raster_forward(&sc, info->images.data(), B, &info->params, L, &io, stream), "adop_raster_forward");

        // saved for backward: depth, weight per layer, then the colours (PointRenderer.cu:1514-1527); the visible list
        // takes the place of the drop-out tensor
        variable_list save;
        for (int l = 0; l < L; ++l) { save.push_back(depth[l]); save.push_back(weight[l]); }
        save.insert(save.end(), color.begin(), color.end());
        save.push_back(visible);
        save.push_back(texture); save.push_back(background_color); save.push_back(points); save.push_back(intrinsics);
        save.push_back(has(env_map) ? env_map : (info->env_map ? *info->env_map : none_like(texture)));
        save.push_back(info->poses);
        ctx->save_for_backward(save);
        ctx->saved_data["render_info"] = info_value;  // for its reusable buffers only
        ctx->saved_data["params"] = blob_of(&info->params, sizeof(adop_render_params));
        ctx->saved_data["views"] = blob_of(info->images.data(), sizeof(adop_view) * info->images.size());
        ctx->saved_data["num_layers"] = (int64_t)L;
        ctx->saved_data["has_normal"] = info->normal.has_value();
        ctx->saved_data["has_index"] = info->index.has_value();
        if (info->normal) ctx->saved_data["normal"] = *info->normal;
        if (info->index) ctx->saved_data["index"] = *info->index;
        ctx->saved_data["need_points"] = points.requires_grad();
        ctx->saved_data["need_pose"] = pose_tangents.requires_grad();
        ctx->saved_data["need_intrinsics"] = intrinsics.requires_grad();
        ctx->saved_data["need_env"] = has(env_map) && env_map.requires_grad() && info->params.composite_environment_map != 0;
        ctx->saved_data["num_tangents"] = pose_tangents.size(0);
        variable_list out = color;
        out.insert(out.end(), mask.begin(), mask.end());
        if (!mask.empty()) ctx->mark_non_differentiable(mask);
        return out;
    }

    static variable_list backward(AutogradContext* ctx, variable_list grad_output)
    {
        auto info = ctx->saved_data["render_info"].toCustomClass<RenderInfo>();
        // the call's own copies of everything that can change on the RenderInfo between forward and backward
        Tensor params_blob = ctx->saved_data["params"].toTensor(), views_blob = ctx->saved_data["views"].toTensor();
        adop_render_params params;
        memcpy(&params, params_blob.data_ptr(), sizeof(params));
        std::vector<adop_view> views((size_t)views_blob.numel() / sizeof(adop_view));
        memcpy(views.data(), views_blob.data_ptr(), sizeof(adop_view) * views.size());
        const int B = (int)views.size(), L = (int)ctx->saved_data["num_layers"].toInt();
        auto saved = ctx->get_saved_variables();
        TORCH_CHECK((int)saved.size() == 3 * L + 7, "unexpected number of saved tensors");
        Tensor texture = saved[3 * L + 1], background = saved[3 * L + 2], points = saved[3 * L + 3], intrinsics = saved[3 * L + 4];
        Tensor env_map = saved[3 * L + 5], poses = saved[3 * L + 6];
        c10::cuda::CUDAGuard guard(texture.device());
        cudaStream_t stream = c10::cuda::getCurrentCUDAStream().stream();
        RenderInfo call;  // the scene as the forward call saw it
        call.poses = poses;
        if (ctx->saved_data["has_normal"].toBool()) call.normal = ctx->saved_data["normal"].toTensor();
        if (ctx->saved_data["has_index"].toBool()) call.index = ctx->saved_data["index"].toTensor();
        if (has(env_map)) call.env_map = env_map;
        adop_scene sc = make_scene(call, texture, background, points, intrinsics);
        // the shared [T,C] working copy may belong to a later forward call by now: rebuild it from this call's descriptors
        const size_t workspace_bytes = ensure_workspace(*info, views, L, sc, texture.options(), false);
        check_status(adop_texture_interleave(sc.texture, info->texture_interleaved.data_ptr<float>(), sc.channels, sc.num_texels, stream),
                     "adop_texture_interleave");
        sc.texture_interleaved = info->texture_interleaved.data_ptr<float>();
        adop_backward_io io{};
        std::vector<Tensor> grads(L);
        for (int l = 0; l < L; ++l)
        {
            io.layers[l].depth = saved[2 * l].data_ptr<float>();
            io.layers[l].weight = saved[2 * l + 1].data_ptr<float>();
            io.layers[l].color = saved[2 * L + l].data_ptr<float>();
            // only the first L gradients are image gradients; those of the masks carry nothing (PointRenderer.cu:1568-1571)
            TORCH_CHECK(grad_output[l].defined(), "missing image gradient for layer ", l);
            TORCH_CHECK(grad_output[l].scalar_type() == torch::kFloat32, "image gradients must be float32");  // :1553-1556
            grads[l] = grad_output[l].contiguous();
            io.grad_color[l] = grads[l].data_ptr<float>();
        }
        Tensor visible = saved[3 * L];
        io.visible_list = visible.data_ptr<int32_t>();
        Tensor g_texture = torch::empty_like(texture), g_background = torch::empty_like(background);
        Tensor g_points, g_pose, c_pose, g_intr, c_intr, g_env, g_env_scratch;
        io.grad_texture = g_texture.data_ptr<float>();
        io.grad_texture_interleaved = info->grad_texture_interleaved.data_ptr<float>();
        io.grad_background = g_background.data_ptr<float>();
        if (ctx->saved_data["need_points"].toBool())
        {
            g_points = torch::empty_like(points);
            io.grad_points = g_points.data_ptr<float>();
        }
        if (ctx->saved_data["need_pose"].toBool())
        {
            g_pose = torch::empty({ctx->saved_data["num_tangents"].toInt(), 6}, texture.options().dtype(torch::kFloat64));
            c_pose = torch::empty({g_pose.size(0)}, texture.options());
            TORCH_CHECK(g_pose.size(0) == poses.size(0), "one pose tangent per pose");
            io.grad_pose = g_pose.data_ptr<double>();
            io.count_pose = c_pose.data_ptr<float>();
        }
        if (ctx->saved_data["need_intrinsics"].toBool())
        {
            g_intr = torch::empty_like(intrinsics);
            c_intr = torch::empty({intrinsics.size(0)}, texture.options());
            io.grad_intrinsics = g_intr.data_ptr<float>();
            io.count_intrinsics = c_intr.data_ptr<float>();
        }
        if (ctx->saved_data["need_env"].toBool())
        {
            g_env = torch::empty_like(env_map);
            io.grad_env_map = g_env.data_ptr<float>();
            if (sc.channels % 4 == 0)
            {
                g_env_scratch = torch::empty_like(env_map);
                io.grad_env_map_interleaved = g_env_scratch.data_ptr<float>();
            }
        }
        io.accumulate = 0;
        io.normalize = 1;
        io.workspace = info->workspace.data_ptr();
        io.workspace_bytes = workspace_bytes;
        check_status(adop_raster_backward(&sc, views.data(), B, &params, L, &io, stream), "adop_raster_backward");
        // {texture, background, points, pose tangents, intrinsics}, the environment map, and nothing for the info object
        // (PointRenderer.cu:1641-1643, RenderInfo.cpp:56)
        return {g_texture, g_background, g_points, g_pose, g_intr, g_env, Variable()};
    }
};

// BlendPointCloud (RenderInfo.cpp:19-31)
static std::vector<Tensor> blend_point_cloud(Tensor texture, Tensor background_color, Tensor points, Tensor pose_tangents,
                                             Tensor intrinsics, c10::intrusive_ptr<RenderInfo> info)
{
    return PointRender::apply(texture, background_color, points, pose_tangents, intrinsics, none_like(texture), torch::IValue(info));
}
// The same with the environment map as a differentiable input: with composite_environment_map set, the composite
// out = img + (1 - mask) * grid_sample(env_map, uv) of RenderModule.cpp:106-127 is part of the operator, and the gradient
// of the texture of EnvironmentMapImpl (EnvironmentMap.cu:107-156) comes back through it.
static std::vector<Tensor> blend_point_cloud_environment(Tensor texture, Tensor background_color, Tensor points, Tensor pose_tangents,
                                                         Tensor intrinsics, Tensor env_map, c10::intrusive_ptr<RenderInfo> info)
{
    return PointRender::apply(texture, background_color, points, pose_tangents, intrinsics, env_map, torch::IValue(info));
}

// ApplyTangentToPose (PointRenderer.cu:1659-1665)
static void apply_tangent_to_pose(Tensor tangent, Tensor pose)
{
    TORCH_CHECK(tangent.is_contiguous() && pose.is_contiguous(), "tangent and pose must be contiguous");  // SAIGA_ASSERT, :1661
    TORCH_CHECK(tangent.scalar_type() == torch::kFloat64 && pose.scalar_type() == torch::kFloat64, "tangent and pose are float64");
    TORCH_CHECK(tangent.is_cuda() && pose.is_cuda(), "CUDA tensors only");
    c10::cuda::CUDAGuard guard(tangent.device());
    check_status(adop_apply_tangent(tangent.data_ptr<double>(), pose.data_ptr<double>(), (int32_t)tangent.size(0),
                                    c10::cuda::getCurrentCUDAStream().stream()),
                 "adop_apply_tangent");
}

// NeuralCameraImpl::forward (src/lib/models/NeuralCamera.h:128-129, NeuralCamera.cpp:258-335) as one autograd function over
// the fused kernels: exposure, white balance, vignette (VignetteNetImpl::forward, :22-42) and camera response
// (CameraResponseNetImpl::forward, :87-135). Parameter tensors in the reference's shapes (NeuralCamera.h:45-46,114,135-139):
//   exposures_values [n,1,1,1], white_balance_values [n,3,1,1], vignette_params [3], vignette_center [1,2,1,1],
//   response [1,3,1,K]; an undefined tensor switches the stage off (enable_exposure / enable_white_balance /
//   enable_vignette / no camera_response: clamp to [0,1]). frame_index [B] int32 selects the rows; uv [B,2,H,W] or undefined.
struct Tonemap : public torch::autograd::Function<Tonemap>
{
    static adop_tonemap_params make_params(const Tensor& x, const Tensor& frame_index, const Tensor& uv, const Tensor& exposure,
                                           const Tensor& wb, const Tensor& vignette5, const Tensor& response, int64_t image_w,
                                           int64_t image_h, double leak)
    {
        TORCH_CHECK(x.is_cuda() && x.is_contiguous() && x.scalar_type() == torch::kFloat32 && x.dim() == 4, "x: contiguous float32 CUDA [B,3,H,W]");
        TORCH_CHECK(x.size(1) == 3, "the tonemapper works on RGB images");  // SAIGA_ASSERT(x.size(1) == 3), NeuralCamera.cpp:263
        adop_tonemap_params p{};
        p.batch = (int32_t)x.size(0); p.height = (int32_t)x.size(2); p.width = (int32_t)x.size(3);
        p.vignette_image_w = (int32_t)image_w; p.vignette_image_h = (int32_t)image_h;
        p.leak = (float)leak;
        if (has(frame_index))
        {
            TORCH_CHECK(frame_index.is_cuda() && frame_index.scalar_type() == torch::kInt32 && frame_index.numel() == x.size(0), "frame_index: int32 CUDA [B]");
            p.frame_index = frame_index.data_ptr<int32_t>();
        }
        if (has(exposure)) p.exposure = exposure.data_ptr<float>();
        if (has(wb)) p.white_balance = wb.data_ptr<float>();
        if (has(vignette5)) p.vignette = vignette5.data_ptr<float>();
        if (has(uv))
        {
            TORCH_CHECK(uv.is_cuda() && uv.is_contiguous() && uv.scalar_type() == torch::kFloat32 && uv.numel() == x.size(0) * 2 * x.size(2) * x.size(3), "uv: contiguous float32 CUDA [B,2,H,W]");
            p.uv = uv.data_ptr<float>();
        }
        if (has(response))
        {
            p.response = response.data_ptr<float>();
            p.response_bins = (int32_t)response.size(response.dim() - 1);
        }
        return p;
    }
    static Variable forward(AutogradContext* ctx, Variable x, Variable exposures_values, Variable white_balance_values, Variable vignette_params,
                            Variable vignette_center, Variable response, Tensor frame_index, Tensor uv, int64_t image_w, int64_t image_h, double leak)
    {
        c10::cuda::CUDAGuard guard(x.device());
        cudaStream_t stream = c10::cuda::getCurrentCUDAStream().stream();
        Tensor xc = x.contiguous();
        Tensor e = exposures_values.contiguous(), wb = white_balance_values.contiguous(), r = response.contiguous();
        Tensor vig = none_like(xc);
        if (has(vignette_params))
        {
            Tensor c = has(vignette_center) ? vignette_center.reshape({2}) : torch::zeros({2}, vignette_params.options());
            vig = torch::cat({vignette_params.reshape({3}), c}).contiguous();
        }
        if (has(wb)) TORCH_CHECK(wb.numel() % 3 == 0, "white_balance_values must be [n,3,1,1]");
        if (has(r)) TORCH_CHECK(r.numel() == 3 * r.size(r.dim() - 1), "response must be [1,3,1,K]");
        adop_tonemap_params p = make_params(xc, frame_index, uv, e, wb, vig, r, image_w, image_h, leak);
        Tensor out = torch::empty_like(xc);
        check_status(adop_tonemap_forward(&p, xc.data_ptr<float>(), out.data_ptr<float>(), stream), "adop_tonemap_forward");
        ctx->save_for_backward({xc, e, wb, vig, r, frame_index, uv});
        ctx->saved_data["image_w"] = image_w; ctx->saved_data["image_h"] = image_h; ctx->saved_data["leak"] = leak;
        ctx->saved_data["has_center"] = has(vignette_center);
        return out;
    }
    static variable_list backward(AutogradContext* ctx, variable_list grad_output)
    {
        auto saved = ctx->get_saved_variables();
        Tensor x = saved[0], e = saved[1], wb = saved[2], vig = saved[3], r = saved[4], frame_index = saved[5], uv = saved[6];
        c10::cuda::CUDAGuard guard(x.device());
        cudaStream_t stream = c10::cuda::getCurrentCUDAStream().stream();
        adop_tonemap_params p = make_params(x, frame_index, uv, e, wb, vig, r, ctx->saved_data["image_w"].toInt(), ctx->saved_data["image_h"].toInt(),
                                            ctx->saved_data["leak"].toDouble());
        Tensor go = grad_output[0].contiguous();
        TORCH_CHECK(go.scalar_type() == torch::kFloat32, "the image gradient must be float32");
        adop_tonemap_grads g{};
        Tensor gx = torch::empty_like(x), ge, gwb, gvig, gr;
        g.grad_x = gx.data_ptr<float>();
        if (has(e)) { ge = torch::empty_like(e); g.grad_exposure = ge.data_ptr<float>(); }
        if (has(wb)) { gwb = torch::empty_like(wb); g.grad_white_balance = gwb.data_ptr<float>(); }
        if (has(vig)) { gvig = torch::empty_like(vig); g.grad_vignette = gvig.data_ptr<float>(); }
        if (has(r)) { gr = torch::empty_like(r); g.grad_response = gr.data_ptr<float>(); }
        g.num_frames = has(e) ? (int32_t)e.numel() : (has(wb) ? (int32_t)(wb.numel() / 3) : 0);
        g.accumulate = 0;
        check_status(adop_tonemap_backward(&p, x.data_ptr<float>(), go.data_ptr<float>(), &g, stream), "adop_tonemap_backward");
        Tensor g_params, g_center;
        if (has(gvig))
        {
            g_params = gvig.slice(0, 0, 3).clone();
            if (ctx->saved_data["has_center"].toBool()) g_center = gvig.slice(0, 3, 5).reshape({1, 2, 1, 1}).clone();
        }
        return {gx, ge, gwb, g_params, g_center, gr, Variable(), Variable(), Variable(), Variable(), Variable()};
    }
};

static Tensor tonemap(Tensor x, c10::optional<Tensor> frame_index, c10::optional<Tensor> uv, c10::optional<Tensor> exposures_values,
                      c10::optional<Tensor> white_balance_values, c10::optional<Tensor> vignette_params, c10::optional<Tensor> vignette_center,
                      c10::optional<Tensor> response, int64_t image_w, int64_t image_h, double leak)
{
    auto t = [&](const c10::optional<Tensor>& o) { return o ? *o : none_like(x); };
    auto ti = [&](const c10::optional<Tensor>& o) { return o ? *o : torch::empty({0}, x.options().dtype(torch::kInt32)); };
    return Tonemap::apply(x, t(exposures_values), t(white_balance_values), t(vignette_params), t(vignette_center), t(response), ti(frame_index), t(uv),
                          image_w, image_h, leak);
}

}  // namespace adop

TORCH_LIBRARY(adop, m)
{
    m.class_<adop::RenderInfo>("RenderInfo")
        .def(torch::init<>())
        .def("set_scene", &adop::RenderInfo::set_scene)
        .def("set_outlier_cloud", &adop::RenderInfo::set_outlier_cloud)
        .def("set_views", &adop::RenderInfo::set_views)
        .def("set_param", &adop::RenderInfo::set_param)
        .def("set_num_layers", &adop::RenderInfo::set_num_layers);
    m.def("blend_point_cloud", &adop::blend_point_cloud);
    m.def("blend_point_cloud_environment", &adop::blend_point_cloud_environment);
    m.def("apply_tangent_to_pose", &adop::apply_tangent_to_pose);
    m.def("tonemap", &adop::tonemap);
}
