"""The libTorch autograd operator (adop_b200/libadop_torch.so, C++) against the CPU checker: the reference's call shape
`BlendPointCloud(info)` -> `PointRender::apply(texture, background, points, pose_tangents, intrinsics, info)`
(RenderInfo.cpp:19-58), driven through torch autograd."""
import numpy as np
import pytest
import torch

from adop_b200 import build, synth

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def op():
    torch.ops.load_library(build.TORCH_OP_LIB)
    return torch.ops.adop


def _info(cfg, dev):
    a = cfg["arrays"]
    info = torch.classes.adop.RenderInfo()
    t = lambda v: torch.from_numpy(v).to(dev) if v is not None else None
    info.set_scene(t(a["poses"]), t(a["normal"]), t(a["index"]), t(a["env_map"]))
    if a.get("outlier_position") is not None:
        info.set_outlier_cloud(t(a["outlier_position"]), t(a.get("outlier_normal")), t(a.get("outlier_index")))
    v = cfg["views"]
    views = torch.tensor([[x["w"], x["h"], x["image_index"], x["camera_index"], x.get("camera_model", 0)] for x in v])
    crops = torch.tensor([list(x.get("crop", (1.0, 1.0, 0.0, 0.0, 0.0))) for x in v], dtype=torch.float32)
    info.set_views(views, crops)
    info.set_num_layers(cfg["num_layers"])
    p = cfg["params"]
    for name, _ in type(p)._fields_:
        info.set_param(name, float(getattr(p, name)))
    return info


def _close(a, b, name, rtol=1e-4):
    a = a.detach().cpu().numpy()
    scale = max(float(np.abs(b).max()), 1e-12)
    assert float(np.abs(a.astype(np.float64) - b).max()) <= rtol * scale, name


@pytest.mark.parametrize("name,kw", [("c2", dict(n_points=300_000, n_views=2, size=(320, 180))),
                                      ("c3", dict(n_points=300_000, size=(320, 180)))])
def test_point_render_autograd_matches_checker(oracle, cuda_lib, op, name, kw):
    cfg = synth.make_config(name, **kw)
    a, L = cfg["arrays"], cfg["num_layers"]
    dev = torch.device("cuda:0")
    grads_up = synth.upstream_gradients(cfg["meta"], batch=len(cfg["views"]))
    ref = oracle.forward(a, cfg["views"], cfg["params"], L)
    ref_b = oracle.backward(a, cfg["views"], cfg["params"], L, ref, grads_up)
    texture = torch.from_numpy(a["texture"]).to(dev).requires_grad_(True)
    background = torch.from_numpy(a["background"]).to(dev).requires_grad_(True)
    points = torch.from_numpy(a["position"]).to(dev).requires_grad_(True)
    tangents = torch.zeros((a["poses"].shape[0], 6), dtype=torch.float64, device=dev, requires_grad=True)
    intrinsics = torch.from_numpy(a["intrinsics"]).to(dev).requires_grad_(True)
    info = _info(cfg, dev)
    out = op.blend_point_cloud(texture, background, points, tangents, intrinsics, info)
    n_masks = L if cfg["params"].output_background_mask else 0
    assert len(out) == L + n_masks
    for l in range(L):
        _close(out[l], ref["colors"][l], f"colour {l}")
        if n_masks:
            assert np.array_equal(out[L + l].cpu().numpy(), ref["masks"][l]) and not out[L + l].requires_grad
    loss = sum((o * torch.from_numpy(g).to(dev)).sum() for o, g in zip(out[:L], grads_up))
    loss.backward()
    _close(texture.grad, ref_b["texture"], "grad texture")
    _close(background.grad, ref_b["background"], "grad background")
    _close(points.grad, ref_b["points"], "grad points")
    _close(tangents.grad, ref_b["pose"], "grad pose")
    _close(intrinsics.grad, ref_b["intrinsics"], "grad intrinsics")


def test_only_requested_gradients_are_returned(cuda_lib, op):
    cfg = synth.make_config("c1", n_points=20_000, size=(64, 64))
    a = cfg["arrays"]
    dev = torch.device("cuda:0")
    texture = torch.from_numpy(a["texture"]).to(dev).requires_grad_(True)
    background = torch.from_numpy(a["background"]).to(dev)
    points = torch.from_numpy(a["position"]).to(dev)
    tangents = torch.zeros((1, 6), dtype=torch.float64, device=dev)
    intrinsics = torch.from_numpy(a["intrinsics"]).to(dev)
    out = op.blend_point_cloud(texture, background, points, tangents, intrinsics, _info(cfg, dev))
    sum(o.sum() for o in out).backward()
    assert texture.grad is not None and points.grad is None and tangents.grad is None


def test_apply_tangent_to_pose_op(oracle, cuda_lib, op):
    rng = np.random.default_rng(0)
    poses = np.stack([synth.look_at_pose(rng.normal(size=3) * 3 + 0.2, rng.normal(size=3)) for _ in range(10)])
    tang = rng.normal(size=(10, 6)) * 0.1
    t_ref, p_ref = tang.copy(), poses.copy()
    oracle.apply_tangent(t_ref, p_ref)
    t, p = torch.from_numpy(tang).cuda(), torch.from_numpy(poses).cuda()
    op.apply_tangent_to_pose(t, p)
    assert float(t.abs().max()) == 0 and np.abs(p.cpu().numpy() - p_ref).max() < 1e-12
    with pytest.raises(RuntimeError):
        op.apply_tangent_to_pose(t.float(), p)


def _inputs(a, dev, env=False):
    t = dict(texture=torch.from_numpy(a["texture"]).to(dev).requires_grad_(True),
             background=torch.from_numpy(a["background"]).to(dev).requires_grad_(True),
             points=torch.from_numpy(a["position"]).to(dev).requires_grad_(True),
             tangents=torch.zeros((a["poses"].shape[0], 6), dtype=torch.float64, device=dev, requires_grad=True),
             intrinsics=torch.from_numpy(a["intrinsics"]).to(dev).requires_grad_(True))
    if env:
        t["env_map"] = torch.from_numpy(a["env_map"]).to(dev).requires_grad_(True)
    return t


def test_environment_map_gets_its_gradient_through_the_operator(oracle, cuda_lib, op):
    """composite_environment_map = 1 with the environment map as a differentiable input (the texture of the reference's
    EnvironmentMapImpl, RenderModule.cpp:106-127): images and all gradients, the environment map's included, against the
    checker."""
    cfg = synth.make_config("c2", n_points=200_000, n_views=2, size=(256, 144))
    a, L = cfg["arrays"], cfg["num_layers"]
    dev = torch.device("cuda:0")
    grads_up = synth.upstream_gradients(cfg["meta"], batch=len(cfg["views"]))
    ref = oracle.forward(a, cfg["views"], cfg["params"], L)
    ref_b = oracle.backward(a, cfg["views"], cfg["params"], L, ref, grads_up, want_env=True)
    t = _inputs(a, dev, env=True)
    out = op.blend_point_cloud_environment(t["texture"], t["background"], t["points"], t["tangents"], t["intrinsics"], t["env_map"], _info(cfg, dev))
    for l in range(L):
        _close(out[l], ref["colors"][l], f"colour {l}")
    sum((o * torch.from_numpy(g).to(dev)).sum() for o, g in zip(out[:L], grads_up)).backward()
    assert float(np.abs(ref_b["env_map"]).max()) > 0
    _close(t["env_map"].grad, ref_b["env_map"], "grad env_map")
    _close(t["texture"].grad, ref_b["texture"], "grad texture")
    _close(t["tangents"].grad, ref_b["pose"], "grad pose")


def test_backward_uses_what_its_own_forward_used(cuda_lib, op):
    """Forward A, then the RenderInfo gets another drop-out seed and other views and forward B runs on it; backward of A
    must equal the backward of A run alone (the per-call state lives in the autograd context, as the reference's saved
    drop-out tensor does, PointRenderer.cu:1524)."""
    cfg = synth.make_config("c2", n_points=120_000, n_views=4, size=(192, 108))
    cfg["params"].dropout = 0.3
    cfg["params"].dropout_seed = 11
    a, L = cfg["arrays"], cfg["num_layers"]
    dev = torch.device("cuda:0")
    views_a, views_b = cfg["views"][:2], cfg["views"][2:]
    g = torch.Generator(device=dev)
    g.manual_seed(3)

    def run(interfere):
        t = _inputs(a, dev)
        info = _info(dict(cfg, views=views_a), dev)
        out = op.blend_point_cloud(t["texture"], t["background"], t["points"], t["tangents"], t["intrinsics"], info)
        if interfere:
            info.set_param("dropout_seed", 99.0)
            v = torch.tensor([[x["w"], x["h"], x["image_index"], x["camera_index"], 0] for x in views_b])
            info.set_views(v, torch.tensor([[1.0, 1.0, 0.0, 0.0, 0.0]] * len(views_b)))
            other = torch.from_numpy(a["texture"]).to(dev) * 0.5
            op.blend_point_cloud(other, t["background"].detach(), t["points"].detach(), t["tangents"].detach(), t["intrinsics"].detach(), info)
        torch.manual_seed(0)
        ups = [torch.randn(o.shape, device=dev, generator=torch.Generator(device=dev).manual_seed(5 + i)) for i, o in enumerate(out[:L])]
        sum((o * u).sum() for o, u in zip(out[:L], ups)).backward()
        return {k: v.grad.clone() for k, v in t.items()}

    alone, disturbed = run(False), run(True)
    for k in alone:
        scale = max(float(alone[k].abs().max()), 1e-12)
        assert float((alone[k] - disturbed[k]).abs().max()) <= 1e-4 * scale, k
    assert float(alone["points"].abs().max()) > 0


def test_tonemap_operator_through_autograd(cuda_lib, op):
    """adop::tonemap with the reference's parameter shapes against the reference's sequence of libtorch operations
    (NeuralCamera.cpp:22-42, 87-135, 258-335) re-typed in torch, values and every parameter gradient."""
    from tests.test_oracle_cpu import _torch_tonemap
    dev = torch.device("cuda:0")
    rng = np.random.default_rng(2)
    B, H, W, K, n, leak = 3, 40, 56, 25, 6, 0.01
    x = torch.from_numpy(rng.uniform(-0.2, 2.5, (B, 3, H, W)).astype(np.float32)).to(dev)
    fi = torch.tensor([4, 0, 2], dtype=torch.int32, device=dev)
    ys, xs = np.meshgrid(np.arange(H), np.arange(W), indexing="ij")
    uv = np.stack([2 * xs / (W - 1) - 1, 2 * ys / (H - 1) - 1])[None].repeat(B, 0).astype(np.float32)
    uv = torch.from_numpy(uv + rng.normal(0, 0.01, uv.shape).astype(np.float32)).to(dev)
    vals = dict(exposure=rng.uniform(-1, 1, (n, 1, 1, 1)), wb=rng.normal(1, 0.05, (n, 3, 1, 1)), vig=np.array([0.1, -0.05, 0.01]),
                center=np.array([0.02, -0.03]).reshape(1, 2, 1, 1), response=np.sort(rng.uniform(0, 1, (1, 3, 1, K)), axis=3))

    def params():
        return {k: torch.from_numpy(v.astype(np.float32)).to(dev).requires_grad_(True) for k, v in vals.items()}

    go = torch.from_numpy(rng.normal(size=(B, 3, H, W)).astype(np.float32)).to(dev)
    p, xa = params(), x.clone().requires_grad_(True)
    out = op.tonemap(xa, fi, uv, p["exposure"], p["wb"], p["vig"], p["center"], p["response"], W, H, leak)
    out.backward(go)
    q, xb = params(), x.clone().requires_grad_(True)
    vig5 = torch.cat([q["vig"], q["center"].reshape(2)])
    want = _torch_tonemap(xb, fi, q["exposure"].reshape(n), q["wb"].reshape(n, 3), vig5, uv, q["response"].reshape(3, K), leak, (W, H))
    want.backward(go)
    assert torch.allclose(out, want, rtol=1e-5, atol=2e-6)
    assert torch.allclose(xa.grad, xb.grad, rtol=1e-4, atol=1e-5)
    for k in vals:
        scale = max(float(q[k].grad.abs().max()), 1e-12)
        assert p[k].grad.shape == q[k].grad.shape
        assert float((p[k].grad - q[k].grad).abs().max()) <= 1e-4 * scale, k
    # stages switched off: exposure only, no response -> clamp
    out2 = op.tonemap(x, fi, None, p["exposure"].detach(), None, None, None, None, W, H, 0.0)
    want2 = torch.clamp(x * (1.0 / torch.exp2(p["exposure"].detach().reshape(n)[fi.long()])).view(-1, 1, 1, 1), 0, 1)
    assert torch.allclose(out2, want2, rtol=1e-5, atol=1e-6)


def test_outlier_cloud_through_the_operator(oracle, cuda_lib, op):
    """RenderInfo.set_outlier_cloud: the second cloud of the forward pass (the reference's render_outliers,
    PointRenderer.cu:1402-1441). Images and gradients against the checker; the outliers occlude and count, and get no
    gradient of their own."""
    cfg = synth.make_config("c2", n_points=200_000, n_views=2, size=(320, 180))
    a, L = cfg["arrays"], cfg["num_layers"]
    a.update(synth.outlier_cloud(a, 20_000, seed=3, distance=-0.5))
    dev = torch.device("cuda:0")
    grads_up = synth.upstream_gradients(cfg["meta"], batch=len(cfg["views"]))
    ref = oracle.forward(a, cfg["views"], cfg["params"], L)
    plain = oracle.forward({k: v for k, v in a.items() if not k.startswith("outlier")}, cfg["views"], cfg["params"], L)
    assert (ref["weights"][0] != plain["weights"][0]).sum() > 500
    ref_b = oracle.backward(a, cfg["views"], cfg["params"], L, ref, grads_up)
    texture = torch.from_numpy(a["texture"]).to(dev).requires_grad_(True)
    background = torch.from_numpy(a["background"]).to(dev).requires_grad_(True)
    points = torch.from_numpy(a["position"]).to(dev).requires_grad_(True)
    tangents = torch.zeros((a["poses"].shape[0], 6), dtype=torch.float64, device=dev, requires_grad=True)
    intrinsics = torch.from_numpy(a["intrinsics"]).to(dev).requires_grad_(True)
    out = op.blend_point_cloud(texture, background, points, tangents, intrinsics, _info(cfg, dev))
    for l in range(L):
        _close(out[l], ref["colors"][l], f"colour {l}")
    sum((o * torch.from_numpy(g).to(dev)).sum() for o, g in zip(out[:L], grads_up)).backward()
    _close(texture.grad, ref_b["texture"], "grad texture")
    _close(points.grad, ref_b["points"], "grad points")
    _close(tangents.grad, ref_b["pose"], "grad pose")
    _close(intrinsics.grad, ref_b["intrinsics"], "grad intrinsics")
