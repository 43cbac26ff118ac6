"""GPU parity of the fused tonemapper and of the pose update against the CPU checker, through the C ABI."""
import numpy as np
import pytest
import torch

from adop_b200.raster import Tonemapper, apply_tangent_to_pose
from adop_b200 import synth

pytestmark = pytest.mark.gpu


def _case(seed, B=3, H=37, W=53, K=25, n=6, with_uv=True):
    rng = np.random.default_rng(seed)
    x = rng.uniform(-0.3, 2.5, (B, 3, H, W)).astype(np.float32)
    fi = rng.integers(0, n, B).astype(np.int32)
    exposure = rng.uniform(-2, 2, n).astype(np.float32)
    wb = rng.normal(1, 0.05, (n, 3)).astype(np.float32)
    wb[:, 1] = 1.0
    vig = np.array([0.1, -0.05, 0.01, 0.02, -0.03], np.float32)
    uv = None
    if with_uv:
        ys, xs = np.meshgrid(np.arange(H), np.arange(W), indexing="ij")
        uv = np.stack([2 * xs / (W - 1) - 1, 2 * ys / (H - 1) - 1])[None].repeat(B, 0).astype(np.float32)
        uv += rng.normal(0, 0.02, uv.shape).astype(np.float32)
    response = np.sort(rng.uniform(0, 1, (3, K)), axis=1).astype(np.float32)
    go = rng.normal(size=x.shape).astype(np.float32)
    return dict(x=x, frame_index=fi, exposure=exposure, white_balance=wb, vignette=vig, uv=uv, response=response), go


def _close(a, b, rtol=1e-4, name=""):
    a = a.detach().cpu().numpy()
    scale = max(float(np.abs(b).max()), 1e-12)
    err = float(np.abs(a.astype(np.float64) - b).max())
    assert err <= rtol * scale, f"{name}: {err:.3e} vs scale {scale:.3e}"


@pytest.mark.parametrize("leak", [0.0, 0.01])
@pytest.mark.parametrize("with_uv", [True, False])
def test_tonemapper_forward_backward(oracle, cuda_lib, leak, with_uv):
    c, go = _case(0, with_uv=with_uv)
    H, W = c["x"].shape[2:]
    kw = dict(image_size=(W, H), frame_index=c["frame_index"], exposure=c["exposure"], white_balance=c["white_balance"],
              vignette=c["vignette"], uv=c["uv"], response=c["response"], leak=leak)
    ref = oracle.tonemap_forward(c["x"], **kw)
    ref_g = oracle.tonemap_backward(c["x"], go, **kw)
    d = {k: (torch.from_numpy(v).cuda() if v is not None else None) for k, v in c.items()}
    tm = Tonemapper((W, H), exposure=d["exposure"], white_balance=d["white_balance"], vignette=d["vignette"],
                    response=d["response"], leak=leak)
    out = tm.forward(d["x"], d["frame_index"], d["uv"])
    _close(out, ref, rtol=1e-5, name="tonemapped image")
    g = tm.backward(d["x"], torch.from_numpy(go).cuda(), d["frame_index"], d["uv"])
    for k in ("x", "exposure", "white_balance", "vignette", "response"):
        _close(g[k], ref_g[k], name="grad " + k)


def test_tonemapper_without_response_is_a_clamp(oracle, cuda_lib):
    c, go = _case(1, K=2)
    x = torch.from_numpy(c["x"]).cuda()
    tm = Tonemapper((53, 37))
    out = tm.forward(x)
    assert torch.equal(out, x.clamp(0, 1))
    g = tm.backward(x, torch.from_numpy(go).cuda())
    want = torch.from_numpy(go).cuda() * ((x > 0) & (x < 1))
    assert torch.allclose(g["x"], want)


def test_tonemapper_256_bin_response_hd_image(oracle, cuda_lib):
    """The HDR-4K configuration's tonemapper parameters (256-entry response) on a smaller image."""
    c, go = _case(2, B=2, H=135, W=240, K=256, n=4)
    kw = dict(image_size=(240, 135), frame_index=c["frame_index"], exposure=c["exposure"], white_balance=c["white_balance"],
              vignette=c["vignette"], uv=None, response=c["response"], leak=0.0)
    ref = oracle.tonemap_forward(c["x"], **kw)
    ref_g = oracle.tonemap_backward(c["x"], go, **kw)
    d = {k: (torch.from_numpy(v).cuda() if v is not None else None) for k, v in c.items()}
    tm = Tonemapper((240, 135), exposure=d["exposure"], white_balance=d["white_balance"], vignette=d["vignette"],
                    response=d["response"])
    _close(tm.forward(d["x"], d["frame_index"]), ref, rtol=1e-5)
    g = tm.backward(d["x"], torch.from_numpy(go).cuda(), d["frame_index"])
    for k in ("x", "exposure", "white_balance", "vignette", "response"):
        _close(g[k], ref_g[k], name="grad " + k)


def test_apply_tangent_to_pose(oracle, cuda_lib):
    rng = np.random.default_rng(3)
    n = 300
    poses = np.stack([synth.look_at_pose(rng.normal(size=3) * 3 + 0.1, rng.normal(size=3)) for _ in range(n)])
    tangents = rng.normal(size=(n, 6)) * 0.1
    tangents[0] = 0
    t_ref, p_ref = tangents.copy(), poses.copy()
    oracle.apply_tangent(t_ref, p_ref)
    t, p = torch.from_numpy(tangents).cuda(), torch.from_numpy(poses).cuda()
    apply_tangent_to_pose(t, p)
    assert float(t.abs().max()) == 0.0
    assert np.abs(p.cpu().numpy() - p_ref).max() < 1e-12
    with pytest.raises(TypeError):
        apply_tangent_to_pose(t.float(), p)


@pytest.mark.parametrize("K", [300, 512, 1024])
def test_tonemapper_long_response_curves(oracle, cuda_lib, K):
    """Curves with more than 256 bins: the backward kernel runs with fewer warps per block (every warp keeps two histograms
    of its own in shared memory), up to the 1024 bins the entry point accepts."""
    c, go = _case(3, B=2, H=48, W=64, K=K, n=3, with_uv=False)
    kw = dict(image_size=(64, 48), frame_index=c["frame_index"], exposure=c["exposure"], white_balance=c["white_balance"],
              vignette=c["vignette"], uv=None, response=c["response"], leak=0.01)
    ref = oracle.tonemap_forward(c["x"], **kw)
    ref_g = oracle.tonemap_backward(c["x"], go, **kw)
    d = {k: (torch.from_numpy(v).cuda() if v is not None else None) for k, v in c.items()}
    tm = Tonemapper((64, 48), exposure=d["exposure"], white_balance=d["white_balance"], vignette=d["vignette"],
                    response=d["response"], leak=0.01)
    _close(tm.forward(d["x"], d["frame_index"]), ref, rtol=1e-5)
    g = tm.backward(d["x"], torch.from_numpy(go).cuda(), d["frame_index"])
    for k in ("x", "exposure", "white_balance", "vignette", "response"):
        _close(g[k], ref_g[k], name="grad " + k)


def test_tonemapper_gradient_that_is_not_finite_shows_up(cuda_lib):
    """The response-curve histogram is summed in scaled fixed point; rounds whose upstream gradient holds an infinity or a NaN
    take float atomics instead, so the non-finite value reaches the curve's gradient (and only the bins that pixel touches),
    and huge and tiny finite gradients next to each other keep their sums."""
    c, go = _case(4, B=1, H=64, W=64, K=256, n=1, with_uv=False)
    d = {k: (torch.from_numpy(v).cuda() if v is not None else None) for k, v in c.items()}
    tm = Tonemapper((64, 64), exposure=d["exposure"], white_balance=d["white_balance"], vignette=d["vignette"],
                    response=d["response"])
    g0 = torch.from_numpy(go).cuda()
    clean = tm.backward(d["x"], g0, d["frame_index"])["response"]
    assert bool(torch.isfinite(clean).all())
    g1 = g0.clone()
    g1[0, 1, 10, 7] = float("inf")
    bad = tm.backward(d["x"], g1, d["frame_index"])["response"]
    assert not bool(torch.isfinite(bad[1]).all())                      # the green curve got the infinity
    assert int((~torch.isfinite(bad)).sum()) <= 2                      # in the two bins of that pixel only
    ok = torch.isfinite(bad)
    assert torch.allclose(bad[ok], clean[ok], rtol=1e-4, atol=1e-4 * float(clean.abs().max()))
    # a wide dynamic range inside one image: rows of gradients scaled by 1e+12 and 1e-12
    g2 = g0.clone()
    g2[:, :, :8] *= 1e12
    g2[:, :, 8:16] *= 1e-12
    wide = tm.backward(d["x"], g2, d["frame_index"])["response"]
    assert bool(torch.isfinite(wide).all())
    gl, gh = g0.clone(), g0.clone()
    gl[:, :, :16] = 0
    gh[:, :, 16:] = 0
    gh[:, :, 8:16] = 0
    part = tm.backward(d["x"], gl, d["frame_index"])["response"] + 1e12 * tm.backward(d["x"], gh, d["frame_index"])["response"]
    assert torch.allclose(wide, part, rtol=2e-4, atol=2e-4 * float(part.abs().max()))
