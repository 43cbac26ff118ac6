// libTorch operator over the C ABI: the reference-facing host side of the rasterizer, in the reference's language.
//
// Mirrors darglein/ADOP's operator surface for this path:
//   torch::autograd::PointRender (src/lib/rendering/PointRenderer.h:37-47, RenderInfo.cpp:34-58)  -> adop::PointRender
//   NeuralRenderInfo             (PointRenderer.h:25-34), registered as a custom class (RenderInfo.cpp:11-15) -> adop::RenderInfo
//   BlendPointCloud              (PointRenderer.h:52, RenderInfo.cpp:19-31)                        -> adop::blend_point_cloud
//   ApplyTangentToPose           (PointRenderer.h:63)                                              -> adop::apply_tangent_to_pose
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

static void ensure_workspace(RenderInfo& info, const adop_scene& sc, const torch::TensorOptions& opt)
{
    const size_t need = adop_raster_workspace_bytes_full(sc.num_points, (int32_t)info.images.size(), info.images[0].w, info.images[0].h,
                                                         (int32_t)info.num_layers, sc.channels);
    TORCH_CHECK(need > 0, "invalid view size / layer count");
    if (!info.workspace.defined() || (size_t)info.workspace.numel() < need)
        info.workspace = torch::empty({(int64_t)need}, opt.dtype(torch::kUInt8));
    if (!info.texture_interleaved.defined() || info.texture_interleaved.size(0) != sc.num_texels || info.texture_interleaved.size(1) != sc.channels)
    {
        info.texture_interleaved = torch::empty({sc.num_texels, sc.channels}, opt);
        info.grad_texture_interleaved = torch::empty({sc.num_texels, sc.channels}, opt);
    }
}

struct PointRender : public torch::autograd::Function<PointRender>
{
    // returns a tensor for every layer, then (if requested) a mask for every layer
    static variable_list forward(AutogradContext* ctx, Variable texture, Variable background_color, Variable points,
                                 Variable pose_tangents, Variable intrinsics, torch::IValue info_value)
    {
        auto info = info_value.toCustomClass<RenderInfo>();
        TORCH_CHECK(!info->images.empty(), "RenderInfo has no views");
        c10::cuda::CUDAGuard guard(texture.device());
        cudaStream_t stream = c10::cuda::getCurrentCUDAStream().stream();
        adop_scene sc = make_scene(*info, texture, background_color, points, intrinsics);
        const int B = (int)info->images.size(), L = (int)info->num_layers, C = sc.channels;
        auto opt = texture.options();
        ensure_workspace(*info, sc, opt);
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
        io.workspace_bytes = (size_t)info->workspace.numel();
        check_status(adop_raster_forward(&sc, info->images.data(), B, &info->params, L, &io, stream), "adop_raster_forward");

        // saved for backward: depth, weight per layer, then the colours (PointRenderer.cu:1514-1527); the splat list
        // takes the place of the drop-out tensor
        variable_list save;
        for (int l = 0; l < L; ++l) { save.push_back(depth[l]); save.push_back(weight[l]); }
        save.insert(save.end(), color.begin(), color.end());
        save.push_back(visible);
        save.push_back(texture); save.push_back(background_color); save.push_back(points); save.push_back(intrinsics);
        ctx->save_for_backward(save);
        ctx->saved_data["render_info"] = info_value;
        ctx->saved_data["need_points"] = points.requires_grad();
        ctx->saved_data["need_pose"] = pose_tangents.requires_grad();
        ctx->saved_data["need_intrinsics"] = intrinsics.requires_grad();
        ctx->saved_data["num_tangents"] = pose_tangents.size(0);
        variable_list out = color;
        out.insert(out.end(), mask.begin(), mask.end());
        if (!mask.empty()) ctx->mark_non_differentiable(mask);
        return out;
    }

    static variable_list backward(AutogradContext* ctx, variable_list grad_output)
    {
        auto info = ctx->saved_data["render_info"].toCustomClass<RenderInfo>();
        const int B = (int)info->images.size(), L = (int)info->num_layers;
        auto saved = ctx->get_saved_variables();
        TORCH_CHECK((int)saved.size() == 3 * L + 5, "unexpected number of saved tensors");
        Tensor texture = saved[3 * L + 1], background = saved[3 * L + 2], points = saved[3 * L + 3], intrinsics = saved[3 * L + 4];
        c10::cuda::CUDAGuard guard(texture.device());
        cudaStream_t stream = c10::cuda::getCurrentCUDAStream().stream();
        adop_scene sc = make_scene(*info, texture, background, points, intrinsics);
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
        Tensor g_points, g_pose, c_pose, g_intr, c_intr;
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
            TORCH_CHECK(g_pose.size(0) == info->poses.size(0), "one pose tangent per pose");
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
        io.accumulate = 0;
        io.normalize = 1;
        io.workspace = info->workspace.data_ptr();
        io.workspace_bytes = (size_t)info->workspace.numel();
        check_status(adop_raster_backward(&sc, info->images.data(), B, &info->params, L, &io, stream), "adop_raster_backward");
        // {texture, background, points, pose tangents, intrinsics} and nothing for the info object
        // (PointRenderer.cu:1641-1643, RenderInfo.cpp:56)
        return {g_texture, g_background, g_points, g_pose, g_intr, Variable()};
    }
};

// BlendPointCloud (RenderInfo.cpp:19-31)
static std::vector<Tensor> blend_point_cloud(Tensor texture, Tensor background_color, Tensor points, Tensor pose_tangents,
                                             Tensor intrinsics, c10::intrusive_ptr<RenderInfo> info)
{
    return PointRender::apply(texture, background_color, points, pose_tangents, intrinsics, torch::IValue(info));
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

}  // namespace adop

TORCH_LIBRARY(adop, m)
{
    m.class_<adop::RenderInfo>("RenderInfo")
        .def(torch::init<>())
        .def("set_scene", &adop::RenderInfo::set_scene)
        .def("set_views", &adop::RenderInfo::set_views)
        .def("set_param", &adop::RenderInfo::set_param)
        .def("set_num_layers", &adop::RenderInfo::set_num_layers);
    m.def("blend_point_cloud", &adop::blend_point_cloud);
    m.def("apply_tangent_to_pose", &adop::apply_tangent_to_pose);
}
