"""Run one of the benchmark configurations end to end on one GPU and print its timings as one JSON line.

    python -m adop_b200.run_config c1|c2|c3|c4|c5|reorder|tonemap [--points N] [--views V] [--reps R]

bench.py measures the headline configuration (c2) under the driver's contract; this runner covers the others:
c1 (small cloud, 512x512), c3 (100 M points, omnidirectional camera, forward only, ms per frame), c4 (30 M points, 8 views),
c5 (50 M points, 4K, 6 layers, 8 channels, plus the fused tonemapper forward + backward on the 4K frames).
Times are CUDA-event times of whole calls after warm-up; per-kernel times come from the library's own event brackets.
"""
import argparse
import json
import statistics
import sys

import torch

from . import capi, synth
from .raster import PointRasterizer, Scene, Tonemapper


def timed(fn, reps):
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(reps + 1)]
    ev[0].record()
    for i in range(reps):
        fn()
        ev[i + 1].record()
    torch.cuda.synchronize()
    return [ev[i].elapsed_time(ev[i + 1]) for i in range(reps)]


def reorder(dev, args):
    """Morton reorder of a c2-shaped cloud (default 10 M points): GPU time per kernel, keys/s, fraction of the HBM
    roofline (32 bytes per key and pass: the key read for the histogram, key + index read and written by the scatter;
    8 passes; 28 bytes per key to form the keys), and the numpy statement of the same sort timed beside it."""
    import time
    import numpy as np
    from . import preprocess
    n = args.points or 10_000_000
    rng = np.random.default_rng(0)
    xyz = rng.normal(0, 1.5, (n, 3)).astype(np.float32)
    pos = torch.from_numpy(np.concatenate([xyz, np.ones((n, 1), np.float32)], axis=1)).to(dev)
    order = preprocess.morton_order(pos)
    torch.cuda.synchronize()
    t = statistics.median(timed(lambda: preprocess.morton_order(pos), args.reps))
    capi.profile_enable(True)
    preprocess.morton_order(pos)
    torch.cuda.synchronize()
    kernel_ms = {k: round(v[1], 4) for k, v in capi.profile_collect().items()}
    capi.profile_enable(False)
    t_perm = statistics.median(timed(lambda: preprocess.permute_rows(pos, order), args.reps))
    n_cpu = min(n, 2_000_000)
    t0 = time.perf_counter()
    want = synth.morton_order(xyz[:n_cpu])
    t_cpu = time.perf_counter() - t0
    same = bool(np.array_equal(preprocess.morton_order(pos[:n_cpu].contiguous()).cpu().numpy().astype(np.int64), want))
    # the other preprocessing steps on a cloud shaped like the benchmark scene (points on surfaces)
    surf = torch.from_numpy(synth.make_config("c2", n_points=n, n_views=1, size=(64, 36))["arrays"]["position"]).to(dev)
    preprocess.knn_distance(surf, k=4)
    torch.cuda.synchronize()
    t_knn = statistics.median(timed(lambda: preprocess.knn_distance(surf, k=4), max(2, args.reps // 2)))
    t_shuffle = statistics.median(timed(lambda: preprocess.block_shuffle_order(n, dev), args.reps))
    t_radius = statistics.median(timed(lambda: preprocess.sort_blocks_by_radius_order(surf), args.reps))
    algo_bytes = n * (8 * 32 + 28)
    peak = 6542.7
    out = {"config": "reorder", "n_points": n, "morton_order_ms": t, "gkeys_per_s": n / (t * 1e-3) / 1e9,
           "algorithmic_bytes": algo_bytes, "achieved_gbs": algo_bytes / (t * 1e-3) / 1e9,
           "roofline_frac_of_measured_6542.7": algo_bytes / (t * 1e-3) / 1e9 / peak, "kernel_ms": kernel_ms,
           "knn4_distance_ms": t_knn, "knn_mpts_per_s": n / (t_knn * 1e-3) / 1e6, "block_shuffle_order_ms": t_shuffle,
           "sort_blocks_by_radius_ms": t_radius,
           "permute_positions_ms": t_perm, "permute_gbs": n * 36 / (t_perm * 1e-3) / 1e9,
           "cpu_numpy": {"points": n_cpu, "seconds": t_cpu, "gkeys_per_s": n_cpu / t_cpu / 1e9, "cores": 1,
                         "same_permutation_as_gpu": same}}
    print(json.dumps(out), flush=True)
    return 0


def tonemap(dev, args):
    """The fused tonemapper on one 4K frame of uniformly random values (the worst case for the response-curve histogram of
    the backward pass) and on a smooth frame: time per image and fraction of the HBM roofline (24 bytes per pixel forward,
    36 backward), with and without the response-curve gradient."""
    w, h = 3840, 2160
    g = torch.Generator(device=dev)
    g.manual_seed(0)
    exposure = torch.rand(1, device=dev, generator=g) * 4 - 2
    wb = (1 + 0.05 * torch.randn((1, 3), device=dev, generator=g)).contiguous()
    vig = torch.tensor([0.1, -0.05, 0.01, 0.0, 0.0], device=dev)
    response = (torch.linspace(0, 1, 256, device=dev) ** (1 / 2.2)).repeat(3, 1).contiguous()
    fi = torch.zeros(1, device=dev, dtype=torch.int32)
    peak = 6542.7
    out = {"config": "tonemap", "image": [w, h], "response_bins": 256}
    yy, xx = torch.meshgrid(torch.linspace(0, 1, h, device=dev), torch.linspace(0, 1, w, device=dev), indexing="ij")
    smooth = torch.stack([0.5 + 0.4 * torch.sin(6 * xx + 3 * yy), 0.5 + 0.4 * torch.cos(5 * yy), xx * yy]).unsqueeze(0)
    frames = {"random": torch.rand((1, 3, h, w), device=dev, generator=g),
              "smooth": (smooth + 0.01 * torch.rand((1, 3, h, w), device=dev, generator=g)).contiguous()}
    go = torch.randn((1, 3, h, w), device=dev, generator=g)
    for name, x in frames.items():
        for label, resp in (("", response), ("_no_response_gradient", None)):
            tm = Tonemapper((w, h), exposure=exposure, white_balance=wb, vignette=vig, response=response, leak=0.01)
            if resp is None:
                # same forward arithmetic, no histogram in the backward pass: the curve is not a trainable tensor here
                bw = lambda: tm.backward(x, go, fi, want_response=False)
            else:
                bw = lambda: tm.backward(x, go, fi)
            for _ in range(3):
                bw()
            t_b = statistics.median(timed(bw, args.reps))
            out[f"{name}{label}_bwd_us"] = t_b * 1e3
            out[f"{name}{label}_bwd_frac"] = 36 * w * h / (t_b * 1e-3) / 1e9 / peak
        t_f = statistics.median(timed(lambda: tm.forward(x, fi), args.reps))
        out[f"{name}_fwd_us"] = t_f * 1e3
        out[f"{name}_fwd_frac"] = 24 * w * h / (t_f * 1e-3) / 1e9 / peak
    print(json.dumps(out), flush=True)
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("config", choices=["c1", "c2", "c3", "c4", "c5", "reorder", "tonemap"])
    ap.add_argument("--points", type=int, default=None)
    ap.add_argument("--views", type=int, default=None)
    ap.add_argument("--reps", type=int, default=5)
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("needs a CUDA device")
    dev = torch.device("cuda:0")
    if args.config == "reorder":
        return reorder(dev, args)
    if args.config == "tonemap":
        return tonemap(dev, args)
    cfg = synth.make_config(args.config, n_points=args.points, n_views=args.views)
    meta, params, L = cfg["meta"], cfg["params"], cfg["num_layers"]
    forward_only = args.config == "c3"
    scene = Scene(**{k: (torch.from_numpy(v).to(dev) if v is not None else None) for k, v in cfg["arrays"].items()})
    ras = PointRasterizer(dev)
    fwd = ras.forward(scene, cfg["views"], params, L, record_visible=not forward_only)
    out = {"config": args.config, **{k: meta[k] for k in ("n_points", "n_views", "w", "h", "layers", "channels")}}
    out["coverage_layer0"] = float((fwd.weights[0] > 0).float().mean())
    out["accepted_layer0_per_view"] = float(fwd.weights[0].sum()) / meta["n_views"]
    # a viewer renders frame after frame with unchanged descriptors: their working copy is not rebuilt per frame
    t_f = timed(lambda: ras.forward(scene, cfg["views"], params, L, out=fwd, record_visible=not forward_only,
                                    refresh_descriptors=not forward_only), args.reps)
    out["fwd_ms"] = statistics.median(t_f)
    out["fwd_ms_per_view"] = out["fwd_ms"] / meta["n_views"]
    total = out["fwd_ms"]
    if not forward_only:
        grads = [torch.randn_like(c) for c in fwd.colors]
        has_env = scene.env_map is not None and params.composite_environment_map
        bwd = ras.backward(scene, params, fwd, grads, want_env=has_env)
        out["visible_list_unusable"] = bool(fwd.list_unusable().any())

        def both():
            ras.forward(scene, cfg["views"], params, L, out=fwd)
            ras.backward(scene, params, fwd, grads, want_env=has_env, out=bwd)

        t_fb = timed(both, args.reps)
        total = statistics.median(t_fb)
        out["fwd_bwd_ms"] = total
        if args.config == "c1":
            # launch-bound at this size: the same step captured once into a CUDA graph and replayed
            side = torch.cuda.Stream()
            with torch.cuda.stream(side):
                both()
                side.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    both()
            torch.cuda.synchronize()
            out["fwd_bwd_ms_cuda_graph"] = statistics.median(timed(graph.replay, max(args.reps, 20)))
        out["bwd_ms_per_view"] = (total - out["fwd_ms"]) / meta["n_views"]
    out["gpts_per_s"] = meta["n_points"] * meta["n_views"] / (total * 1e-3) / 1e9
    capi.profile_enable(True)
    ras.forward(scene, cfg["views"], params, L, out=fwd, record_visible=not forward_only, refresh_descriptors=not forward_only)
    if not forward_only:
        ras.backward(scene, params, fwd, grads, want_env=has_env, out=bwd)
    torch.cuda.synchronize()
    out["kernel_ms"] = {k: round(v[1], 4) for k, v in capi.profile_collect().items()}
    capi.profile_enable(False)
    if args.config == "c5":
        # the fused tonemapper on the 4K frames: per-image exposure ~ U[-2,2] EV, white balance ~ N(1,0.05) with green fixed,
        # vignette polynomial (0.1,-0.05,0.01), monotone 256-entry response (gamma 1/2.2 curve)
        B, w, h = meta["n_views"], meta["w"], meta["h"]
        g = torch.Generator(device=dev)
        g.manual_seed(0)
        exposure = (torch.rand(B, device=dev, generator=g) * 4 - 2)
        wb = 1 + 0.05 * torch.randn((B, 3), device=dev, generator=g)
        wb[:, 1] = 1.0
        vig = torch.tensor([0.1, -0.05, 0.01, 0.0, 0.0], device=dev)
        response = (torch.linspace(0, 1, 256, device=dev) ** (1 / 2.2)).repeat(3, 1).contiguous()
        tm = Tonemapper((w, h), exposure=exposure, white_balance=wb.contiguous(), vignette=vig, response=response, leak=0.01)
        x = fwd.colors[0][:, :3].contiguous()
        fi = torch.arange(B, device=dev, dtype=torch.int32)
        go = torch.randn_like(x)
        tm.forward(x, fi)
        tm.backward(x, go, fi)
        out["tonemap_fwd_ms_per_image"] = statistics.median(timed(lambda: tm.forward(x, fi), args.reps)) / B
        out["tonemap_bwd_ms_per_image"] = statistics.median(timed(lambda: tm.backward(x, go, fi), args.reps)) / B
        px = w * h
        out["tonemap_fwd_gbs"] = 24 * px / (out["tonemap_fwd_ms_per_image"] * 1e-3) / 1e9
        out["tonemap_bwd_gbs"] = 36 * px / (out["tonemap_bwd_ms_per_image"] * 1e-3) / 1e9
    print(json.dumps(out), flush=True)


if __name__ == "__main__":
    sys.exit(main())
