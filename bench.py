"""Benchmark of the point-rasterizer hot path: forward + backward of the training-scene workload.

    python bench.py --gpus 1 --steps 20 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P bench.py --gpus N ...
    python bench.py --impl reference ...      # the CPU restatement of the reference kernels on the host cores

A step = one forward + backward of the rasterizer over one batch of views of the synthetic training scene
(10 M points on 64 random spheres / plane patches, 16 views per GPU at 1920x1080 on a radius-4 orbit, pinhole with
k1=-0.1 k2=0.02, 4-layer pyramid, 4 descriptor channels, 1024x512 environment map, pose / intrinsics / point gradients
on). Metric: points rasterized per second forward+backward = points x views / time, in Gpts/s, summed over all GPUs.
Multi-GPU: views are sharded over ranks (weak scaling: 16 views per GPU), the scene is replicated, and the descriptor
and point gradients are reduce-scattered with NCCL before normalisation.
Prints ONE JSON line on rank 0.
"""
import argparse
import datetime
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "points rasterized/sec fwd+bwd at 1080p"
UNIT = "Gpts/s"
WORKLOAD = "c2: 10M points x 16 views/GPU, 1920x1080, L=4, C=4, pinhole k1=-0.1 k2=0.02, env 1024x512, fwd+bwd with pose grads"


# DRAM bytes (read + write) per launch of the kernels that can dominate, from ncu captures of a four-view run of this
# workload (profiles/point_kernels_c2_ncu.md); one launch there = one launch here. Valid for the default workload only.
NCU_TRAFFIC_BYTES = {"k_depth_prepass": 220.0e6, "k_blend": 421.2e6, "k_resolve": 106.6e6, "k_backward_tiles": 313.9e6,
                     "k_chain_and_holes": 222.1e6}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--points", type=int, default=10_000_000)
    ap.add_argument("--views", type=int, default=16, help="views per GPU")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-c4", action="store_true", help="N > 1: skip the 30 M point record")
    ap.add_argument("--no-extras", action="store_true", help="N = 1: skip the tonemapper / Morton reorder record")
    ap.add_argument("--candidates", action="store_true",
                    help="size the scratch with room for candidate streams (the depth prepass then hands projected points to "
                         "the blend kernel; measured slightly slower overall than projecting twice)")
    ap.add_argument("--no-touched", action="store_true",
                    help="N > 1: the exchange kernel reads every rank's whole gradient block instead of only the chunks a rank flagged")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                    help="N > 1: gradient exchange by the peer-memory kernel (default) or by NCCL reduce-scatter / all-reduce")
    return ap.parse_args()


class ClockSampler:
    """nvidia-smi samples of SM clock and throttle reasons while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap,timestamp")

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu_index), f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def wait_ready(self, timeout=8.0):
        """nvidia-smi can take a few hundred ms to print its first sample, longer than a short timed region: wait for it."""
        t_end = time.time() + timeout
        while self.proc is not None and not self.lines and time.time() < t_end and self.proc.poll() is None:
            time.sleep(0.01)

    def stop(self, window=None):
        """window = (start, end) datetimes of the timed region: only samples taken inside it count. The sampler runs from
        before the warm-up (nvidia-smi needs a moment to start), so the samples outside the window are under load too;
        they are used only if the region was too short to catch one."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        rows = []
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 8:
                continue
            try:
                when = datetime.datetime.strptime(parts[7], "%Y/%m/%d %H:%M:%S.%f")
                rows.append((when, float(parts[0]), float(parts[1]), [n for n, v in zip(names, parts[3:7]) if v.lower().startswith("active")]))
            except ValueError:
                continue
        inside = [r for r in rows if window and window[0] <= r[0] <= window[1]]
        used = inside if inside else rows
        sm = [r[1] for r in used]
        reasons = sorted({n for r in used for n in r[3]})
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": used[-1][2] if used else None, "reasons": reasons,
                "samples": len(sm), "window": "timed region" if inside else "warm-up and timed region"}


def bind_to_gpu_numa_node(gpu_index):
    """Pin this process to the CPU cores that `nvidia-smi topo -m` lists as the GPU's CPU affinity, BEFORE it allocates its
    pinned host buffers (they are then placed on that socket's memory): with several ranks per node every rank otherwise
    pulls its host->device copies through whatever socket it happened to start on. Read-only query; returns the core list
    (or None when the table cannot be read)."""
    try:
        out = subprocess.run(["nvidia-smi", "topo", "-m"], capture_output=True, text=True, timeout=20).stdout
    except (OSError, subprocess.SubprocessError):
        return None
    header = None
    for ln in out.splitlines():
        cols = [c.strip() for c in ln.split("\t") if c.strip()]
        if not cols:
            continue
        if "CPU Affinity" in ln and header is None:
            header = cols
            continue
        if header and cols[0] == f"GPU{gpu_index}":
            # the header has no cell above the row labels: data column k sits under header[k - 1]
            try:
                spec = cols[header.index("CPU Affinity") + 1]
            except (ValueError, IndexError):
                return None
            cores = set()
            for part in spec.split(","):
                part = part.strip()
                if not part or not part[0].isdigit():
                    return None
                a, _, b = part.partition("-")
                cores.update(range(int(a), int(b or a) + 1))
            allowed = cores & os.sched_getaffinity(0)
            if not allowed:
                return None
            os.sched_setaffinity(0, allowed)
            return sorted(allowed)
    return None


def algorithmic_bytes(N, C, P, U_views, normals=False, point_grads=True, env_hw=None):
    """Bytes that one step has to move at the least. Per view: forward N*2*(16+n) + U*(4+4C) + P*(4C+8), backward
    N*(16+n) + U*(4+4C) + P*(8C+8); per step + 4CN for the descriptor gradient, + 20N with point gradients, + the
    environment map read once forward and its gradient written once backward."""
    n = 4 if normals else 0
    fwd = sum(N * 2 * (16 + n) + U * (4 + 4 * C) + P * (4 * C + 8) for U in U_views)
    bwd = sum(N * (16 + n) + U * (4 + 4 * C) + P * (8 * C + 8) for U in U_views)
    step = 4 * C * N + (20 * N if point_grads else 0)
    if env_hw:
        step += 2 * 4 * C * env_hw[0] * env_hw[1]
    per_view_bwd = [N * (16 + n) + U * (4 + 4 * C) + P * (8 * C + 8) for U in U_views]
    return fwd, bwd, step, per_view_bwd


def cpu_one_view(ora, cfg, arrays, grads_one_view, cores, max_seconds, max_reps):
    """Times the CPU restatement on ONE FULL view of the workload (all points, full image pyramid, forward + backward
    with every gradient); returns (Gpts/s, repetitions, seconds per repetition list)."""
    one_view = [cfg["views"][0]]
    times = []
    while sum(times) < max_seconds and len(times) < max_reps:
        t0 = time.perf_counter()
        f = ora.forward(arrays, one_view, cfg["params"], cfg["num_layers"], threads=cores)
        ora.backward(arrays, one_view, cfg["params"], cfg["num_layers"], f, grads_one_view, want_env=True, threads=cores)
        times.append(time.perf_counter() - t0)
    n = arrays["position"].shape[0]
    return n * len(times) / sum(times) / 1e9, times


def cpu_reference_arm(args, rank, world):
    """--impl reference: the reference has no CPU rasterizer and its CUDA code cannot be built without the saiga library,
    so this arm times the CPU restatement of the reference kernels (oracle/) with all host threads. A step = one full
    view of the workload (all points, the full 1080p pyramid, forward + backward): the metric, points x views / time,
    does not depend on how many views a step holds."""
    if rank != 0:
        return
    from adop_b200 import synth
    from tests.oracle_lib import Oracle
    ora = Oracle()
    cores = os.cpu_count() or ora.lib.adop_oracle_max_threads()  # torchrun sets OMP_NUM_THREADS=1; ask for all cores anyway
    cfg = synth.make_config("c2", n_points=args.points, n_views=1)
    arrays = cfg["arrays"]
    n = arrays["position"].shape[0]
    grads = synth.upstream_gradients(cfg["meta"], batch=1)
    times = []
    for it in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        fwd = ora.forward(arrays, cfg["views"], cfg["params"], cfg["num_layers"], threads=cores)
        ora.backward(arrays, cfg["views"], cfg["params"], cfg["num_layers"], fwd, grads, want_env=True, threads=cores)
        dt = time.perf_counter() - t0
        if it >= args.warmup:
            times.append(dt)
    total = sum(times)
    value = n * len(times) / total / 1e9
    sample = f"1 full view per step: all {n} points, full 1080p pyramid, fwd+bwd with pose, intrinsics, point, descriptor and environment-map gradients"
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": 1e3 * total / len(times), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "points": n, "views_per_step": 1,
                       "note": "CPU restatement of the reference kernels; the reference's own CUDA renderer needs the saiga "
                               "library, which is not in its tree. One view of the workload per step instead of 16: points x "
                               "views / time is the same quantity"},
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def exchange_check(peer, dist, torch):
    """Largest relative difference (|a - b| / max|b| per tensor) between what the peer-memory kernel just produced and the
    same sums formed by NCCL all-reduces of the raw gradient blocks, on this rank's shards. Outside any timed region."""
    res = peer.reduce()  # the blocks still hold this step's raw sums
    raw = peer.backward_outputs()
    worst = 0.0

    def rel(a, b):
        scale = float(b.abs().max())
        return float((a.double() - b.double()).abs().max()) / scale if scale > 0 else 0.0

    tex = raw["texture_interleaved"].clone()
    dist.all_reduce(tex)
    t_lo, t_hi = res["texel_range"]
    worst = max(worst, rel(res["texture_shard"], tex[t_lo:t_hi].t()))
    del tex
    pts = raw["points"].clone()
    dist.all_reduce(pts)
    p_lo, p_hi = res["point_range"]
    mine = pts[p_lo:p_hi]
    want = mine.clone()
    nz = mine[:, 3] > 0
    want[nz, :3] = mine[nz, :3] / mine[nz, 3:4]
    want[:, 3] = 0
    worst = max(worst, rel(res["points_shard"], want))
    del pts
    pose, cnt = raw["pose"].clone(), raw["count_pose"].clone()
    dist.all_reduce(pose)
    dist.all_reduce(cnt)
    pose = torch.where(cnt[:, None] > 0, pose / cnt[:, None].double().clamp(min=1), pose)
    worst = max(worst, rel(res["pose"], pose))
    t = torch.tensor([worst], device=pose.device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def measure_parameter_update(peer, scene, dev, dist, torch, adist, capi):
    """The step that follows the exchange in a training step, outside any timed region: Adam on the owned descriptor shard,
    SGD on the owned point shard, every new value written to all ranks' replicas (adop_peer_apply_update, one kernel
    between two stream-ordered barriers). Returns the time of a whole step call and of the kernel alone (max over ranks),
    and the largest difference between this rank's replica and rank 0's afterwards (must be 0)."""
    import statistics
    res = peer.reduce()
    C_, T = scene.texture.shape
    pp = adist.PeerParameters(adist.peer_param_layout(C_, T, scene.position.shape[0]), dev)
    pp.texture.copy_(scene.texture)
    pp.points.copy_(scene.position)
    for _ in range(2):
        pp.step(res, lr_texture=0.08, lr_points=0.005)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(6)]
    capi.profile_collect()
    capi.profile_enable(True)
    ev[0].record()
    for i in range(5):
        pp.step(res, lr_texture=0.08, lr_points=0.005)
        ev[i + 1].record()
    torch.cuda.synchronize()
    kt = capi.profile_collect()
    capi.profile_enable(False)
    t = torch.tensor([statistics.median(ev[i].elapsed_time(ev[i + 1]) for i in range(5)),
                      kt["k_peer_update"][1] / max(kt["k_peer_update"][0], 1) if "k_peer_update" in kt else 0.0], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    same = pp.texture.clone()
    dist.broadcast(same, src=0)
    diff = torch.tensor([float((same - pp.texture).abs().max())], device=dev)
    dist.all_reduce(diff, op=dist.ReduceOp.MAX)
    world = dist.get_world_size()
    own_bytes = (C_ * T * 4 * 4 + scene.position.shape[0] * 16 * 2) // world   # gradient, two moments, parameter; point gradient, point
    pushed = (C_ * T * 4 + scene.position.shape[0] * 16) // world * (world - 1)    # to the other replicas over NVLink
    pp.close()
    return {"what": "Adam on the owned descriptor shard + SGD on the owned points, new values written to every rank's replica: "
                    "one kernel between two stream-ordered barriers", "step_ms": float(t[0]), "kernel_ms": float(t[1]),
            "local_bytes_per_rank": own_bytes, "nvlink_bytes_per_rank": pushed, "replica_difference": float(diff.item())}


def measure_c4(rank, world, dev, steps, exchange, touched=True):
    """The multi-GPU configuration (30 M points, 8 views per GPU, 1080p): forward + backward + gradient exchange, timed
    like the headline (barrier, CUDA events, maximum over ranks). Returns the record for the bench line."""
    import torch
    import torch.distributed as dist
    from adop_b200 import capi, synth
    from adop_b200 import dist as adist
    from adop_b200.raster import PointRasterizer, Scene
    V, n_points = 8, 30_000_000
    cfg = synth.make_config("c4", n_points=n_points, n_views=V * world)
    arrays, params, L = cfg["arrays"], cfg["params"], cfg["num_layers"]
    views = capi.make_views([cfg["views"][i] for i in adist.shard_views(list(range(V * world)), rank, world)])
    C = cfg["meta"]["channels"]
    scene = Scene(**{k: (torch.from_numpy(v).to(dev) if v is not None else None) for k, v in arrays.items()})
    ras = PointRasterizer(dev)
    gen = torch.Generator(device=dev)
    gen.manual_seed(4321 + rank)
    grads = [torch.randn((V, C, hh, ww), device=dev, generator=gen) for ww, hh in capi.layer_sizes(cfg["meta"]["w"], cfg["meta"]["h"], L)]
    fwd = ras.forward(scene, views, params, L)
    bwd = ras.backward(scene, params, fwd, grads, want_env=True, normalize=False)
    peer = None
    if exchange == "peer":
        try:
            layout = adist.peer_layout(C, bwd["texture"].shape[1], n_points, num_images=bwd["pose"].shape[0],
                                       num_cameras=bwd["intrinsics"].shape[0], intrinsics_cols=bwd["intrinsics"].shape[1],
                                       env_hw=tuple(arrays["env_map"].shape[1:]), touched=touched)
            peer = adist.PeerGradientExchange(layout, dev)
            bwd = peer.backward_outputs()
        except capi.AdopError:
            peer = None
    touched_flags = peer.touched_flags() if peer is not None else None

    def step():
        ras.forward(scene, views, params, L, out=fwd, touched=touched_flags)
        if peer is not None:
            peer.release()  # the barrier deferred by the last reduce: everyone has read this rank's block
        ras.backward(scene, params, fwd, grads, want_env=True, normalize=False, out=bwd)
        if peer is not None:
            peer.reduce(defer_release=True)
        else:
            adist.exchange_gradients(bwd)

    for _ in range(3):
        step()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    dist.barrier()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1)], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item()) / steps
    capi.profile_enable(True)
    step()
    torch.cuda.synchronize()
    kt = capi.profile_collect()
    capi.profile_enable(False)
    check = exchange_check(peer, dist, torch) if peer is not None else None
    if peer is not None:
        peer.close()
    return {"workload": "c4: 30M points x 8 views/GPU, 1920x1080, L=4, C=4", "points": n_points, "views_per_gpu": V,
            "value": n_points * V * world / (ms * 1e-3) / 1e9, "unit": UNIT, "ms_per_step": ms,
            "exchange_ms": kt["k_peer_reduce"][1] if "k_peer_reduce" in kt else None,
            "exchange": "peer-memory kernel" if peer is not None else "NCCL", "exchange_check": check}


def single_gpu_extras(dev):
    """Two kernels outside the headline that have a roofline of their own: the tonemapper's backward pass on a 4K frame
    (36 bytes per pixel) and the Morton reorder of a 10 M point cloud (8 radix passes)."""
    import statistics
    import numpy as np
    import torch
    from adop_b200 import preprocess
    from adop_b200.raster import Tonemapper
    from adop_b200.run_config import timed
    w, h = 3840, 2160
    g = torch.Generator(device=dev)
    g.manual_seed(0)
    exposure = torch.rand(1, device=dev, generator=g) * 4 - 2
    wb = (1 + 0.05 * torch.randn((1, 3), device=dev, generator=g)).contiguous()
    vig = torch.tensor([0.1, -0.05, 0.01, 0.0, 0.0], device=dev)
    response = (torch.linspace(0, 1, 256, device=dev) ** (1 / 2.2)).repeat(3, 1).contiguous()
    tm = Tonemapper((w, h), exposure=exposure, white_balance=wb, vignette=vig, response=response, leak=0.01)
    x = torch.rand((1, 3, h, w), device=dev, generator=g)
    go = torch.randn((1, 3, h, w), device=dev, generator=g)
    fi = torch.zeros(1, device=dev, dtype=torch.int32)
    for _ in range(3):
        tm.backward(x, go, fi)
    t_b = statistics.median(timed(lambda: tm.backward(x, go, fi), 10))
    t_f = statistics.median(timed(lambda: tm.forward(x, fi), 10))
    n = 10_000_000
    rng = np.random.default_rng(0)
    pos = torch.from_numpy(np.concatenate([rng.normal(0, 1.5, (n, 3)).astype(np.float32), np.ones((n, 1), np.float32)], axis=1)).to(dev)
    for _ in range(2):
        preprocess.morton_order(pos)
    t_r = statistics.median(timed(lambda: preprocess.morton_order(pos), 5))
    return {"tonemap_4k_backward_gbs": 36 * w * h / (t_b * 1e-3) / 1e9, "tonemap_4k_forward_gbs": 24 * w * h / (t_f * 1e-3) / 1e9,
            "morton_reorder_10m_gkeys_per_s": n / (t_r * 1e-3) / 1e9, "morton_reorder_10m_ms": t_r}


def main():
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        cpu_reference_arm(args, rank, world)
        return

    import numpy as np
    import torch
    import torch.distributed as dist
    from adop_b200 import capi, synth
    from adop_b200 import dist as adist
    from adop_b200.raster import PointRasterizer, Scene

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path in the product)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    numa_cores = bind_to_gpu_numa_node(local_rank) if world > 1 else None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    capi.load_library()

    # ---- workload: the scene is replicated, every rank gets its own views on the orbit -------------------------------
    V = args.views
    cfg = synth.make_config("c2", n_points=args.points, n_views=V * world)
    arrays, params, L = cfg["arrays"], cfg["params"], cfg["num_layers"]
    my_ids = adist.shard_views(list(range(V * world)), rank, world)
    views = capi.make_views([cfg["views"][i] for i in my_ids])
    N, C = cfg["meta"]["n_points"], cfg["meta"]["channels"]
    w, h = cfg["meta"]["w"], cfg["meta"]["h"]
    P = sum(a * b for a, b in capi.layer_sizes(w, h, L))
    scene = Scene(**{k: (torch.from_numpy(v).to(dev) if v is not None else None) for k, v in arrays.items()})
    ras = PointRasterizer(dev, full_workspace=True if args.candidates else None)
    gen = torch.Generator(device=dev)
    gen.manual_seed(1234 + rank)
    grads_dev = [torch.randn((V, C, hh, ww), device=dev, generator=gen) for ww, hh in capi.layer_sizes(w, h, L)]
    grads_host = [g.cpu().pin_memory() for g in grads_dev]
    normalize_local = world == 1

    fwd = ras.forward(scene, views, params, L)
    bwd = ras.backward(scene, params, fwd, grads_dev, want_env=True, normalize=normalize_local)
    torch.cuda.synchronize()
    # N > 1: all gradient outputs live in one block per rank that the other ranks map; one kernel reads every block
    # over NVLink and writes the owned, summed, normalised gradients. NCCL reduce-scatter / all-reduce is the fallback.
    peer = None
    if world > 1 and args.exchange == "peer":
        try:
            layout = adist.peer_layout(C, bwd["texture"].shape[1], N, num_images=bwd["pose"].shape[0],
                                       num_cameras=bwd["intrinsics"].shape[0], intrinsics_cols=bwd["intrinsics"].shape[1],
                                       env_hw=tuple(arrays["env_map"].shape[1:]), touched=not args.no_touched)
            peer = adist.PeerGradientExchange(layout, dev)
            bwd = peer.backward_outputs()
        except capi.AdopError as e:
            if rank == 0:
                print(f"bench: {e}; using the NCCL exchange", file=sys.stderr, flush=True)
    touched_flags = peer.touched_flags() if peer is not None else None
    final = {}  # the step's final small gradients (what the end-to-end loop reads back)

    def exchange():
        if peer is not None:
            final.update(peer.reduce(defer_release=True))
        elif world > 1:
            ex = adist.exchange_gradients(bwd)
            # normalise the owned shard of the point gradients (sum / count), PointRenderer.cu:1620-1627
            if adist.points_shard_is_aligned(N, world):
                shard = ex["points_shard"]
                ras.normalize_gradients({"points": shard.view(-1, 4), "pose": None, "intrinsics": None})
            ras.normalize_gradients({"points": None, "pose": ex["pose"], "count_pose": ex["count_pose"],
                                     "intrinsics": ex["intrinsics"], "count_intrinsics": ex["count_intrinsics"]})
            final.update(ex)
        else:
            final.update(bwd)

    def step():
        ras.forward(scene, views, params, L, out=fwd, touched=touched_flags)
        if peer is not None:
            peer.release()  # the barrier deferred by the last reduce: everyone has read this rank's block
        ras.backward(scene, params, fwd, grads_dev, want_env=True, normalize=normalize_local, out=bwd)
        exchange()

    # per step: interleave, depth fills, camera records (forward and backward), one depth prepass per group of four views,
    # (blend, resolve) and (prepare, gather, chain, all-points fallback) per view, then either de-interleave + three
    # normalisations or the one peer-reduce kernel (NCCL's own kernels are not counted)
    kernels_per_step = 1 + L + 2 + (V + 3) // 4 + 2 * V + 4 * V + (2 if peer is not None else 2 + 3)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-timed region (inputs resident in HBM) ---------------------------------------------------------------
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        sampler.wait_ready()
    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    wall0 = datetime.datetime.now()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    wall1 = datetime.datetime.now()
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop((wall0, wall1)) if rank == 0 else None
    t = torch.tensor([ms], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total = float(t.item())
    value = N * V * world * args.steps / (ms_total * 1e-3) / 1e9

    # ---- end-to-end through the public API with host buffers ---------------------------------------------------------
    # per step: host->device copy of the step's upstream gradient pyramid from pinned memory (it overlaps the forward
    # pass on a copy stream), forward, backward, device->host read of the pose / intrinsics / background gradients.
    # The copies are double-buffered: step k+1's gradients travel while step k computes, so every step still pays for its own
    # 705 MB over PCIe inside the timed region, but behind the kernels where it fits.
    copy_stream = torch.cuda.Stream(device=dev)
    staged = [[torch.empty_like(g) for g in grads_dev] for _ in range(2)]
    copied = [torch.cuda.Event(), torch.cuda.Event()]
    consumed = [torch.cuda.Event(), torch.cuda.Event()]
    small_host = {k: torch.empty_like(bwd[k], device="cpu").pin_memory() for k in ("pose", "intrinsics", "background")}
    h2d_bytes = sum(g.numel() * 4 for g in grads_host) + len(views) * 40
    d2h_bytes = sum(v.numel() * v.element_size() for v in small_host.values())
    main_stream = torch.cuda.current_stream(dev)

    def start_copy(slot):
        copy_stream.wait_event(consumed[slot])  # the backward pass that last read this buffer is done
        with torch.cuda.stream(copy_stream):
            for s_, hsrc in zip(staged[slot], grads_host):
                s_.copy_(hsrc, non_blocking=True)
            copied[slot].record(copy_stream)

    def run_e2e(n_steps):
        for ev in consumed:
            ev.record(main_stream)
        start_copy(0)
        for k in range(n_steps):
            slot = k & 1
            if k + 1 < n_steps:
                start_copy(slot ^ 1)
            ras.forward(scene, views, params, L, out=fwd, touched=touched_flags)
            main_stream.wait_event(copied[slot])
            if peer is not None:
                peer.release()
            ras.backward(scene, params, fwd, staged[slot], want_env=True, normalize=normalize_local, out=bwd)
            consumed[slot].record(main_stream)
            exchange()
            for kk, hdst in small_host.items():
                hdst.copy_(final[kk], non_blocking=True)
        main_stream.synchronize()

    # the host limit of the end-to-end figure, measured: all ranks copy their step's pinned gradients to the device at the
    # same time, nothing else running (GB/s per rank, slowest rank)
    barrier()
    hc0, hc1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    hc0.record()
    for _ in range(3):
        for s_, hsrc in zip(staged[0], grads_host):
            s_.copy_(hsrc, non_blocking=True)
    hc1.record()
    torch.cuda.synchronize()
    t_copy = torch.tensor([hc0.elapsed_time(hc1) / 3], device=dev)
    if world > 1:
        dist.all_reduce(t_copy, op=dist.ReduceOp.MAX)
    h2d_gbs_per_rank = sum(g.numel() * 4 for g in grads_host) / (float(t_copy.item()) * 1e-3) / 1e9

    run_e2e(3)
    barrier()
    e0.record()
    run_e2e(args.steps)
    e1.record()
    barrier()
    ms_e2e = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if world > 1:
        dist.all_reduce(ms_e2e, op=dist.ReduceOp.MAX)
    e2e_value = N * V * world * args.steps / (float(ms_e2e.item()) * 1e-3) / 1e9

    # ---- per-kernel times (CUDA events around every launch, on the launching stream) and the roofline -----------------
    capi.profile_enable(True)
    for _ in range(max(1, min(args.steps, 5))):
        ras.forward(scene, views, params, L, out=fwd, touched=touched_flags)
        if peer is not None:
            peer.release()
        ras.backward(scene, params, fwd, grads_dev, want_env=True, normalize=normalize_local, out=bwd)
        if peer is not None:
            peer.reduce(defer_release=True)
    torch.cuda.synchronize()
    ktimes = capi.profile_collect()
    capi.profile_enable(False)
    ras.forward(scene, views, params, L, out=fwd, touched=touched_flags)
    torch.cuda.synchronize()
    # U_v: points of the view with at least one accepted layer. The forward pass records (point, layer) splats; the
    # points accepted on the finest layer are a lower bound of U_v, the splat count an upper bound; the lower bound is used.
    U_views = [float(fwd.weights[0][b].sum().item()) for b in range(V)]
    fwd_b, bwd_b, step_b, per_view_bwd = algorithmic_bytes(N, C, P, U_views, env_hw=arrays["env_map"].shape[1:])
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except (OSError, ValueError):
        pass
    peak = float(peaks.get("hbm_gbs", 6650.0))
    peak_kind = "measured (MEASURED_PEAKS.json hbm_gbs)" if "hbm_gbs" in peaks else "fallback 6650 GB/s"
    dom = max(ktimes.items(), key=lambda kv: kv[1][1])
    dom_name, (dom_launches, dom_ms) = dom
    # Algorithmic bytes of one launch (= one view, four for the depth prepass) of each kernel that can dominate, two ways:
    #  "survey": the kernel's share of the per-view formula above (forward N*2*16 + U(4+4C) + P(4C+8), backward
    #            N*16 + U(4+4C) + P(8C+8)); the backward formula assumes that every position is read again, which this
    #            backward pass does not do, so the tile kernel is charged the backward formula without its N*16 term;
    #  "own":    what this kernel has to move at the least in this design (adds the depth planes the blend kernel reads, the
    #            visible-list entry it writes or reads, 16 bytes per visible point, and the read-modify-write of the gradient
    #            rows the backward kernels add into).
    U_mean = sum(U_views) / V
    survey_bytes = {"k_depth_prepass": N * 16 + 4 * 4 * P,  # one launch covers four views: the points once, four depth pyramids
                    "k_blend": N * 16 + U_mean * (4 + 4 * C),
                    "k_resolve": P * (4 * C + 8),
                    "k_backward_tiles": U_mean * (4 + 4 * C) + P * (8 * C + 8),
                    "k_chain_and_holes": U_mean * (16 + 16) + 4 * P}
    own_bytes = {"k_depth_prepass": N * 16 + 4 * 4 * P,
                 "k_blend": N * 16 + 4 * P + U_mean * (4 * C + 16),
                 "k_resolve": P * (4 * C + 8),
                 "k_backward_tiles": P * (8 * C + 4) + U_mean * (16 + 4 * C + 2 * 4 * C + 16),
                 "k_chain_and_holes": U_mean * (16 + 16 + 2 * 16) + 4 * P}
    dom_survey = survey_bytes.get(dom_name, sum(per_view_bwd) / V)
    dom_own = own_bytes.get(dom_name, dom_survey)
    dom_s = dom_ms / dom_launches * 1e-3
    step_ms = ms_total / args.steps
    step_achieved = (fwd_b + bwd_b + step_b) / (step_ms * 1e-3) / 1e9
    roofline = {"bound": "hbm", "kernel": dom_name, "achieved": dom_own / dom_s / 1e9, "peak": peak, "unit": "GB/s",
                "frac": dom_own / dom_s / 1e9 / peak,
                "frac_survey_bytes": dom_survey / dom_s / 1e9 / peak,
                "traffic": NCU_TRAFFIC_BYTES.get(dom_name) if (args.points == 10_000_000 and w == 1920) else None,
                "peak_kind": peak_kind,
                "algorithmic_bytes_per_launch": dom_own, "algorithmic_bytes_per_launch_survey": dom_survey,
                "avg_launch_ms": dom_ms / dom_launches,
                "step": {"algorithmic_bytes": fwd_b + bwd_b + step_b, "achieved": step_achieved, "frac": step_achieved / peak},
                "kernel_ms_per_step": {k: v[1] / max(1, min(args.steps, 5)) for k, v in ktimes.items()}}

    # ---- CPU baseline (rank 0, N = 1): the CPU restatement on a bounded sample ------------------------------------------
    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        from tests.oracle_lib import Oracle
        ora = Oracle()
        cores = os.cpu_count() or ora.lib.adop_oracle_max_threads()
        g1 = [g[:1].contiguous().numpy() for g in grads_host]
        cpu_value, cpu_times = cpu_one_view(ora, cfg, arrays, g1, cores, max_seconds=12.0, max_reps=6)
        cpu_baseline = {"value": cpu_value, "unit": UNIT, "cores": cores, "kind": "port",
                        "sample": f"{len(cpu_times)} x (1 full view: all {N} points, full 1080p pyramid, fwd+bwd with all gradients)"}

    # ---- records outside the headline: the exchange check and the 30 M point configuration (N > 1), two more kernels (N = 1)
    check = exchange_check(peer, dist, torch) if peer is not None else None
    update = measure_parameter_update(peer, scene, dev, dist, torch, adist, capi) if peer is not None else None
    c4 = None
    extras = None
    if world > 1 and not args.no_c4:
        if peer is not None:
            peer.close()
            peer = None
        final.clear()
        del fwd, bwd, scene, grads_dev, staged
        ras = None
        torch.cuda.empty_cache()
        c4 = measure_c4(rank, world, dev, max(3, min(args.steps, 10)), args.exchange, not args.no_touched)
    elif world == 1 and not args.no_extras:
        extras = single_gpu_extras(dev)
    parallelism_peer = check is not None
    if rank == 0:
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
                "ms_per_step": step_ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
                "data": "synthetic",
                "config": {"workload": WORKLOAD, "points": N, "views_per_gpu": V, "image": [w, h], "layers": L, "channels": C,
                           "l2": "inputs exceed L2: 160 MB of points and ~100 MB of image state per view stream per pass",
                           "parallelism": ("single GPU" if world == 1 else
                                           f"view-sharded x{world}, gradients exchanged by one peer-memory kernel over NVLink "
                                           "(reduce-scatter + all-reduce + normalise)" if parallelism_peer else
                                           f"view-sharded x{world}, gradients reduce-scattered by NCCL"),
                           "point_order": "Morton-sorted once (untimed), as the reference's scene preprocessing does",
                           "host_binding": (f"rank 0 pinned to {len(numa_cores)} cores of its GPU's NUMA node" if numa_cores else "none"),
                           "h2d_copy_gbs_per_rank": round(h2d_gbs_per_rank, 1),  # all ranks copying at once, nothing else running
                           "e2e": "per step 705 MB host->device (the upstream gradient pyramid, pinned, double-buffered behind the kernels); "
                                  "device->host only the pose, intrinsics and background gradients (836 B): the descriptor and point "
                                  "gradients (320 MB) and the image pyramid stay on the device, where the optimiser and the U-Net use them"},
                "fwd_ms_per_view": ktimes_ms(ktimes, ("k_texture_interleave", "k_fill", "k_build_cams", "k_depth_prepass", "k_blend", "k_accept",
                                                      "k_bin_offsets", "k_bin_scatter", "k_splat", "k_resolve"), V, args),
                "bwd_ms_per_view": ktimes_ms(ktimes, ("k_prepare_backward", "k_backward_tiles", "k_chain_and_holes", "k_splat_backward_all",
                                                      "k_texture_deinterleave", "k_normalize", "k_peer_reduce"), V, args),
                "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": d2h_bytes},
                "gpu_launches": kernels_per_step * args.steps,
                "clocks": clocks, "roofline": roofline, "cpu_baseline": cpu_baseline}
        if world > 1:
            line["exchange_check"] = check  # peer-memory kernel against NCCL all-reduces of the same gradients: largest relative difference
            line["c4"] = c4
            line["parameter_update"] = update  # optimiser step + all-gather of the updated parameters (outside the timed region)
        if extras is not None:
            line["extra"] = extras
        print(json.dumps(line), flush=True)
    if peer is not None:
        peer.close()
    if world > 1:
        dist.destroy_process_group()


def ktimes_ms(ktimes, names, V, args):
    reps = max(1, min(args.steps, 5))
    return sum(ktimes[k][1] for k in names if k in ktimes) / reps / V


if __name__ == "__main__":
    main()
