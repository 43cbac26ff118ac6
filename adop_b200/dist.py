"""View-sharded multi-GPU step: every rank renders its own views of the replicated scene; the only exchange is
in the backward pass. The reference is single-GPU (no collective anywhere in its tree); this is the layout that the
path shards into naturally, since views are independent given the scene parameters.

  * descriptor gradients [C,T] and point gradients [N,4] (x, y, z sums and the contribution count in w) are
    reduce-scattered as un-normalised sums, so each rank ends up owning 1/world of the elements;
  * pose, intrinsics, background and environment-map gradients are small and all-reduced (with their counts);
  * normalisation (sum / count, PointRenderer.cu:1609-1637) happens AFTER the reduction, on the owned shard.

The collectives are torch.distributed calls (NCCL over NVLink on GPUs, gloo in the CPU tests); tensors stay on the
device they are on.
"""
import torch
import torch.distributed as dist


def shard_views(views, rank, world):
    """Contiguous split of a list of views over ranks (the remainder goes to the first ranks)."""
    n = len(views)
    base, rem = divmod(n, world)
    start = rank * base + min(rank, rem)
    return views[start:start + base + (1 if rank < rem else 0)]


def shard_range(numel, rank, world):
    """Element range [lo, hi) of the flattened, padded tensor that `rank` owns after the reduce-scatter."""
    per = (numel + world - 1) // world
    return rank * per, min(numel, (rank + 1) * per)


def _reduce_scatter_flat(t, group):
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    flat = t.reshape(-1)
    per = (flat.numel() + world - 1) // world
    if per * world != flat.numel():
        padded = flat.new_zeros(per * world)
        padded[:flat.numel()] = flat
        flat = padded
    out = flat.new_empty(per)
    if dist.get_backend(group) == "nccl":
        dist.reduce_scatter_tensor(out, flat, op=dist.ReduceOp.SUM, group=group)
    else:
        # gloo (CPU tests of the host logic) has no reduce-scatter: all-reduce and keep the own slice
        tmp = flat.clone()
        dist.all_reduce(tmp, op=dist.ReduceOp.SUM, group=group)
        out.copy_(tmp[rank * per:(rank + 1) * per])
    lo, hi = shard_range(t.numel(), rank, world)
    return out[:hi - lo]


def exchange_gradients(grads, group=None):
    """grads: the dict of PointRasterizer.backward(..., normalize=False) of this rank's views.

    Returns a dict with
      texture_shard, points_shard : 1-D slices of the summed [C,T] / [N,4] tensors that this rank owns
                                    (element ranges from shard_range); points still carry the count in every 4th slot
      pose, count_pose, intrinsics, count_intrinsics, background, env_map : summed over ranks (in place)."""
    out = {}
    out["texture_shard"] = _reduce_scatter_flat(grads["texture"], group)
    if grads.get("points") is not None:
        out["points_shard"] = _reduce_scatter_flat(grads["points"], group)
    for k in ("pose", "count_pose", "intrinsics", "count_intrinsics", "background", "env_map"):
        t = grads.get(k)
        if t is not None:
            dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
            out[k] = t
    return out


def points_shard_is_aligned(num_points, world):
    """True when every rank's share of the flattened [N,4] tensor starts on a point boundary."""
    per = (num_points * 4 + world - 1) // world
    return per % 4 == 0
