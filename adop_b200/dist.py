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


class ShardedParameterUpdate:
    """The optimiser step of the NCCL path (what PeerParameters.step does in one kernel over peer memory, here as library
    collectives; also what runs under gloo in the CPU tests): every rank applies the reference's optimisers to the shard
    of the flattened tensors it owns after exchange_gradients - torch Adam for the descriptors, SGD for the point positions
    (NeuralScene.cpp:76-107, 204-240) - and the updated shards are all-gathered into every rank's replica. Adam moments
    exist for the owned shard only.

        upd = ShardedParameterUpdate(texture, points)     # this rank's replicas, updated in place
        ex = exchange_gradients(backward_outputs)
        upd.step(ex, lr_texture=0.08, lr_points=0.005)"""

    def __init__(self, texture, points=None, group=None, betas=(0.9, 0.999), eps=1e-8):
        self.texture, self.points, self.group = texture, points, group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        lo, hi = shard_range(texture.numel(), self.rank, self.world)
        self._tex_shard = texture.detach().reshape(-1)[lo:hi].clone().requires_grad_(True)
        self._adam = torch.optim.Adam([self._tex_shard], lr=1.0, betas=betas, eps=eps)
        if points is not None and not points_shard_is_aligned(points.shape[0], self.world):
            raise ValueError("the point shards of this rank count do not start on point boundaries")

    def _all_gather_into(self, full, shard):
        flat = full.reshape(-1)
        per = (flat.numel() + self.world - 1) // self.world
        mine = flat.new_zeros(per)
        mine[:shard.numel()] = shard
        parts = [torch.empty_like(mine) for _ in range(self.world)]
        dist.all_gather(parts, mine, group=self.group)
        flat.copy_(torch.cat(parts)[:flat.numel()])

    def step(self, exchanged, lr_texture, lr_points=0.0):
        for g in self._adam.param_groups:
            g["lr"] = lr_texture
        self._tex_shard.grad = exchanged["texture_shard"].reshape(-1).to(self._tex_shard.dtype)
        self._adam.step()
        with torch.no_grad():
            self._all_gather_into(self.texture, self._tex_shard.detach())
            if self.points is not None and lr_points != 0.0 and exchanged.get("points_shard") is not None:
                g = exchanged["points_shard"].reshape(-1, 4)   # sums of x, y, z and the contribution count
                lo, hi = shard_range(self.points.numel(), self.rank, self.world)
                p = self.points.reshape(-1)[lo:hi].reshape(-1, 4).clone()
                cnt = g[:, 3:4]
                p[:, :3] -= lr_points * torch.where(cnt > 0, g[:, :3] / cnt.clamp(min=1e-30), g[:, :3])  # NormalizeGradient, then SGD
                self._all_gather_into(self.points, p.reshape(-1))


def points_shard_is_aligned(num_points, world):
    """True when every rank's share of the flattened [N,4] tensor starts on a point boundary."""
    per = (num_points * 4 + world - 1) // world
    return per % 4 == 0


# ----------------------------------------------------------------------------------------------------------------------
# The same exchange as one kernel over peer memory (adop_peer_reduce_gradients): every rank keeps its gradient outputs in
# one device block that the other ranks map through a CUDA IPC handle; after a stream-ordered barrier each rank reads
# its share of every block over NVLink and writes final gradients (summed, normalised, descriptor gradients in [C,.]).
# ----------------------------------------------------------------------------------------------------------------------
class _DeviceSpan:
    """A span of device memory for torch.as_tensor (CUDA array interface)."""

    def __init__(self, ptr, shape, typestr, owner):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (ptr, False), "version": 2}
        self._owner = owner


def peer_layout(channels, num_texels, num_points=0, num_images=0, num_cameras=0, intrinsics_cols=0, env_hw=(0, 0),
                background=True, touched=False):
    """adop_peer_layout for these tensor sizes (0 = tensor not exchanged); the same call on every rank.
    touched: the blocks also carry the forward pass's flags "the backward pass of this rank's views can add a gradient in
    this chunk of 256 points / texels", and the reduce kernel reads a peer's descriptor / point gradients only where that
    peer set them (PeerGradientExchange.touched_flags() are the tensors to hand to PointRasterizer.forward)."""
    from . import capi
    import ctypes as C
    lay = capi.AdopPeerLayout()
    lay.channels, lay.num_texels, lay.num_points = channels, num_texels, num_points
    lay.num_images, lay.num_cameras, lay.intrinsics_cols = num_images, num_cameras, intrinsics_cols
    lay.env_h, lay.env_w = env_hw
    lay.background = 1 if background else 0
    lay.touched = 1 if touched else 0
    capi.check(capi.load_library().adop_peer_layout_fill(C.byref(lay)), "adop_peer_layout_fill")
    return lay


def peer_shard_range(count, rank, world):
    """[lo, hi) of `count` texels or points that `rank` owns in the peer exchange (whole texels / points per rank)."""
    per = (count + world - 1) // world
    return min(count, rank * per), min(count, (rank + 1) * per)


class _MappedBlocks:
    """One device block per rank of `group` (all on one node): this rank's own allocation plus the other ranks' blocks
    mapped through CUDA IPC handles. Every rank runs the same collectives whether or not its own CUDA calls succeed, so a
    failure on one rank (no peer access between two GPUs, IPC not permitted) ends in an exception on all of them, not in
    a hang."""

    def __init__(self, total_bytes, device, group):
        from . import capi
        import ctypes as C
        self.capi, self.C = capi, C
        self.lib = capi.load_library()
        self.device, self.group = torch.device(device), group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if self.world > 8:
            raise ValueError("the peer exchange covers the GPUs of one node (at most 8 ranks)")
        self.own = C.c_void_p()
        self._opened = []
        handle = capi.AdopPeerHandle()
        problem = None
        with torch.cuda.device(self.device):
            try:
                capi.check(self.lib.adop_peer_alloc(total_bytes, C.byref(self.own), C.byref(handle)), "adop_peer_alloc")
            except capi.AdopError as e:
                problem = e
                self.own = C.c_void_p()
            mine = torch.tensor(list(bytes(handle.bytes)), dtype=torch.uint8, device=self.device)
            everyone = [torch.empty_like(mine) for _ in range(self.world)]
            dist.all_gather(everyone, mine, group=group)
            self.blocks = (C.c_void_p * self.world)()
            for r in range(self.world):
                if problem is not None:
                    break
                if r == self.rank:
                    self.blocks[r] = self.own.value
                    continue
                h = capi.AdopPeerHandle()
                C.memmove(h.bytes, bytes(everyone[r].cpu().tolist()), 64)
                ptr = C.c_void_p()
                try:
                    capi.check(self.lib.adop_peer_open(C.byref(h), C.byref(ptr)), "adop_peer_open")
                except capi.AdopError as e:
                    problem = e
                    break
                self._opened.append(ptr)
                self.blocks[r] = ptr.value
            self.flag = torch.zeros(1, device=self.device)
            ok = torch.tensor([0.0 if problem is not None else 1.0], device=self.device)
            # also: nobody may free its block before every rank has mapped it
            dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
            if float(ok.item()) == 0.0:
                for ptr in self._opened:
                    self.lib.adop_peer_close(ptr)
                self._opened = []
                dist.all_reduce(self.flag, group=group)
                torch.cuda.synchronize(self.device)
                if self.own.value:
                    self.lib.adop_peer_free(self.own)
                self.own = None
                raise capi.AdopError(f"peer-memory exchange unavailable: {problem if problem is not None else 'another rank failed'}")

    def span(self, offset, shape, typestr, dtype, owner):
        """Tensor view of a part of this rank's own block."""
        n = 1
        for d in shape:
            n *= d
        if n == 0:
            return None
        t = torch.as_tensor(_DeviceSpan(self.own.value + offset, shape, typestr, owner), device=self.device)
        assert t.dtype == dtype and t.data_ptr() == self.own.value + offset
        return t

    def barrier(self):
        """Stream-ordered: everything the ranks launched before it is complete once it has run on every rank's stream."""
        dist.all_reduce(self.flag, group=self.group)

    def close(self):
        if self.own is None:
            return
        with torch.cuda.device(self.device):
            torch.cuda.synchronize(self.device)
            dist.all_reduce(self.flag, group=self.group)
            torch.cuda.synchronize(self.device)
            for ptr in self._opened:
                self.lib.adop_peer_close(ptr)
            self._opened = []
            # the other ranks have closed their mappings of this block only after the next collective
            dist.all_reduce(self.flag, group=self.group)
            torch.cuda.synchronize(self.device)
            self.lib.adop_peer_free(self.own)
            self.own = None


class PeerGradientExchange:
    """Gradient block of this rank + the mapped blocks of the other ranks of `group` (all on one node).

        ex = PeerGradientExchange(layout, device, group)
        grads = ex.backward_outputs()            # pass as `out=` to PointRasterizer.backward(..., normalize=False)
        ...backward...
        result = ex.reduce()                      # dict of final gradients (owned shards + small tensors)

    The barrier on either side of the kernel is a one-element all-reduce of the group's backend, in stream order."""

    def __init__(self, layout, device, group=None):
        self._mapped = _MappedBlocks(layout.total_bytes, device, group)
        m = self._mapped
        self.capi, self.C, self.lib = m.capi, m.C, m.lib
        self.layout, self.device, self.group = layout, m.device, group
        self.world, self.rank, self.blocks = m.world, m.rank, m.blocks
        self._own, self._flag = m.own, m.flag
        self._outputs = self._make_outputs()
        self._results = self._make_results()

    def _span(self, offset, shape, typestr, dtype):
        return self._mapped.span(offset, shape, typestr, dtype, self)

    def _make_outputs(self):
        lay = self.layout
        f32, f64 = torch.float32, torch.float64
        o = {"texture": None}
        o["texture_interleaved"] = self._span(lay.off_texture, (lay.num_texels, lay.channels), "<f4", f32)
        o["points"] = self._span(lay.off_points, (lay.num_points, 4), "<f4", f32)
        o["pose"] = self._span(lay.off_pose, (lay.num_images, 6), "<f8", f64)
        o["count_pose"] = self._span(lay.off_count_pose, (lay.num_images,), "<f4", f32)
        o["intrinsics"] = self._span(lay.off_intrinsics, (lay.num_cameras, lay.intrinsics_cols), "<f4", f32)
        o["count_intrinsics"] = self._span(lay.off_count_intrinsics, (lay.num_cameras,), "<f4", f32)
        o["background"] = self._span(lay.off_background, (lay.channels if lay.background else 0,), "<f4", f32)
        o["env_map"] = self._span(lay.off_env_map, (lay.channels, lay.env_h, lay.env_w), "<f4", f32)
        self._touched = None
        if lay.touched:
            chunk = 256
            self._touched = (self._span(lay.off_touched_points, ((lay.num_points + chunk - 1) // chunk,), "|u1", torch.uint8),
                             self._span(lay.off_touched_texels, ((lay.num_texels + chunk - 1) // chunk,), "|u1", torch.uint8))
        return o

    def _make_results(self):
        lay, dev = self.layout, self.device
        t_lo, t_hi = peer_shard_range(lay.num_texels, self.rank, self.world)
        p_lo, p_hi = peer_shard_range(lay.num_points, self.rank, self.world)
        r = {"texel_range": (t_lo, t_hi), "point_range": (p_lo, p_hi)}
        r["texture_shard"] = torch.empty((lay.channels, t_hi - t_lo), device=dev) if t_hi > t_lo else None
        r["points_shard"] = torch.empty((p_hi - p_lo, 4), device=dev) if p_hi > p_lo else None
        has_pose, has_intr = lay.num_images > 0, lay.num_cameras > 0
        r["pose"] = torch.empty((lay.num_images, 6), dtype=torch.float64, device=dev) if has_pose else None
        r["count_pose"] = torch.empty((lay.num_images,), device=dev) if has_pose else None
        r["intrinsics"] = torch.empty((lay.num_cameras, lay.intrinsics_cols), device=dev) if has_intr else None
        r["count_intrinsics"] = torch.empty((lay.num_cameras,), device=dev) if has_intr else None
        r["background"] = torch.empty((lay.channels,), device=dev) if lay.background else None
        r["env_map"] = torch.empty((lay.channels, lay.env_h, lay.env_w), device=dev) if lay.env_h * lay.env_w > 0 else None
        return r

    def touched_flags(self):
        """(points, texels) byte flags inside this rank's block, or None when the layout has none: pass them as `touched=` to
        the step's PointRasterizer.forward call, which marks the chunks its views can give gradients to; reduce() on every
        rank then reads this rank's descriptor and point gradients only there."""
        return self._touched

    def backward_outputs(self):
        """The `out=` dict for PointRasterizer.backward: tensors inside this rank's block (texture stays [T,C])."""
        return self._outputs

    def release(self):
        """The barrier that reduce(defer_release=True) left out: call it before this rank writes its block again (before the
        next backward pass). By then the other ranks finished reading long ago, so it costs no waiting."""
        if getattr(self, "_pending_release", False):
            with torch.cuda.device(self.device):
                dist.all_reduce(self._flag, group=self.group)
            self._pending_release = False

    def reduce(self, normalize=True, defer_release=False):
        """defer_release: leave out the barrier behind the kernel ("every rank has read my block"); the caller then calls
        release() before its next backward pass, typically after the next forward pass, where the barrier finds every rank
        long done instead of making all of them wait for the slowest reader right away."""
        C, capi = self.C, self.capi
        self.release()
        res = self._results
        o = capi.AdopPeerReduceOut()

        def p(name):
            t = res.get(name)
            return t.data_ptr() if t is not None else None

        o.grad_texture_shard, o.grad_points_shard = p("texture_shard"), p("points_shard")
        o.grad_pose, o.count_pose = p("pose"), p("count_pose")
        o.grad_intrinsics, o.count_intrinsics = p("intrinsics"), p("count_intrinsics")
        o.grad_background, o.grad_env_map = p("background"), p("env_map")
        o.normalize = 1 if normalize else 0
        with torch.cuda.device(self.device):
            # every rank's backward pass is complete once this collective has run on every rank's stream ...
            dist.all_reduce(self._flag, group=self.group)
            stream = torch.cuda.current_stream(self.device).cuda_stream
            capi.check(self.lib.adop_peer_reduce_gradients(self.blocks, self.world, self.rank, C.byref(self.layout),
                                                           C.byref(o), C.c_void_p(stream)), "adop_peer_reduce_gradients")
            # ... and nobody overwrites its block (the next backward pass) before every rank has read it
            if defer_release:
                self._pending_release = True
            else:
                dist.all_reduce(self._flag, group=self.group)
        return res

    def close(self):
        if self._own is None:
            return
        self.release()
        self._outputs = self._results = None
        self._mapped.close()
        self._own = None


def peer_param_layout(channels, num_texels, num_points=0):
    """adop_peer_param_layout for these tensor sizes; the same call on every rank."""
    from . import capi
    import ctypes as C
    lay = capi.AdopPeerParamLayout()
    lay.channels, lay.num_texels, lay.num_points = channels, num_texels, num_points
    capi.check(capi.load_library().adop_peer_param_layout_fill(C.byref(lay)), "adop_peer_param_layout_fill")
    return lay


class PeerParameters:
    """This rank's replica of the two large trainable tensors - descriptors [C,T] and point positions [N,4] - inside a
    block that the other ranks map, and the optimiser state of the elements this rank owns.

        params = PeerParameters(layout, device, group)
        params.texture.copy_(...); params.points.copy_(...)      # same initial values on every rank
        scene = Scene(position=params.points, texture=params.texture, ...)
        ... forward, backward, result = exchange.reduce() ...
        params.step(result, lr_texture=0.08, lr_points=0.005)     # Adam / SGD on the owned shard, written to all replicas

    `step` is one kernel (adop_peer_apply_update) between two stream-ordered barriers: optimiser step and all-gather of
    the updated parameters in one pass, Adam moments for 1 / world of the texels per rank. It follows the reference's
    optimisers (torch Adam for the descriptors, SGD for the points: NeuralScene.cpp:76-107, 204-240)."""

    def __init__(self, layout, device, group=None, beta1=0.9, beta2=0.999, eps=1e-8):
        self._mapped = _MappedBlocks(layout.total_bytes, device, group)
        m = self._mapped
        self.layout, self.device, self.group = layout, m.device, group
        self.world, self.rank = m.world, m.rank
        self.texture = m.span(layout.off_texture, (layout.channels, layout.num_texels), "<f4", torch.float32, self)
        self.points = m.span(layout.off_points, (layout.num_points, 4), "<f4", torch.float32, self)
        t_lo, t_hi = peer_shard_range(layout.num_texels, self.rank, self.world)
        self.texel_range = (t_lo, t_hi)
        self.point_range = peer_shard_range(layout.num_points, self.rank, self.world)
        self.adam_m = torch.zeros((layout.channels, t_hi - t_lo), device=self.device)
        self.adam_v = torch.zeros_like(self.adam_m)
        self.beta1, self.beta2, self.eps = beta1, beta2, eps
        self.steps = 0

    def step(self, reduced, lr_texture, lr_points=0.0):
        """reduced: the dict PeerGradientExchange.reduce() returned (its texture_shard / points_shard are read)."""
        m = self._mapped
        C, capi = m.C, m.capi
        self.steps += 1
        u = capi.AdopPeerUpdate()
        gt, gp = reduced.get("texture_shard"), reduced.get("points_shard")
        u.grad_texture_shard = gt.data_ptr() if gt is not None else None
        u.adam_m, u.adam_v = self.adam_m.data_ptr(), self.adam_v.data_ptr()
        u.grad_points_shard = gp.data_ptr() if (gp is not None and lr_points != 0.0) else None
        u.lr_texture, u.beta1, u.beta2, u.eps = lr_texture, self.beta1, self.beta2, self.eps
        u.step, u.lr_points = self.steps, lr_points
        with torch.cuda.device(self.device):
            # nobody still reads the parameters (every rank's backward pass is behind this collective) ...
            m.barrier()
            stream = torch.cuda.current_stream(self.device).cuda_stream
            capi.check(m.lib.adop_peer_apply_update(m.blocks, self.world, self.rank, C.byref(self.layout), C.byref(u),
                                                    C.c_void_p(stream)), "adop_peer_apply_update")
            # ... and nobody reads them again (the next forward pass) before every rank's writes have landed
            m.barrier()

    def close(self):
        self.texture = self.points = None
        self._mapped.close()
