"""The scene's optimiser step for a view-sharded training job: NeuralScene's optimisers (NeuralScene.cpp:72-246) and
NeuralScene::OptimizerStep (NeuralScene.cpp:384-411), with the two large tensors sharded over the ranks.

In the reference one process owns everything: `texture_optimizer` (Adam: descriptors, background colour, environment map)
and `structure_optimizer` (SGD: point positions, pose tangents, pinhole intrinsics; stepped only after
`lock_structure_params_epochs`, followed by `poses->ApplyTangent()`). Here every rank renders its own views, the gradients
are exchanged (dist.PeerGradientExchange), and then

  * descriptors (Adam) and point positions (SGD) are updated by the rank that owns the element and written to every rank's
    replica in the same kernel (dist.PeerParameters.step: optimiser step + all-gather, Adam moments for 1 / world of the
    texels per rank);
  * background colour and environment map (Adam), pose tangents and intrinsics (SGD) are small: every rank steps its own
    replica with torch's optimisers on the all-reduced gradients the exchange returned, which are the same bits on every
    rank, so the replicas stay identical without another collective;
  * the pose update pose <- exp(tangent) * pose, tangent <- 0 (PoseModuleImpl::ApplyTangent, NeuralStructure.cpp:41-44) runs
    on every rank after the SGD step, as in the reference.

torch is used for the small tensors' optimisers and for device memory; the large tensors never pass through it.
"""
import torch

from .raster import apply_tangent_to_pose


class SceneLearningRates:
    """OptimizerParams of the reference (Settings.h:171-178) and TrainParams::lock_structure_params_epochs (Settings.h:340),
    same names and defaults."""

    def __init__(self, lr_texture=0.08, lr_background_color=0.004, lr_environment_map=0.02, lr_points=0.005, lr_poses=0.01,
                 lr_intrinsics=1.0, fix_points=False, fix_poses=False, fix_intrinsics=False, lock_structure_params_epochs=25):
        self.lr_texture, self.lr_background_color, self.lr_environment_map = lr_texture, lr_background_color, lr_environment_map
        self.lr_points, self.lr_poses, self.lr_intrinsics = lr_points, lr_poses, lr_intrinsics
        self.fix_points, self.fix_poses, self.fix_intrinsics = fix_points, fix_poses, fix_intrinsics
        self.lock_structure_params_epochs = lock_structure_params_epochs


class ViewShardedSceneOptimizer:
    """parameters: dist.PeerParameters (descriptors [C,T] and points [N,4] of this rank's replica);
    background [C], env_map [C,eh,ew] or None, pose_tangents [I,6] f64, poses [I,8] f64, intrinsics [K,cols]: this rank's
    replicas of the small tensors (updated in place).

        opt = ViewShardedSceneOptimizer(parameters, background, env_map, tangents, poses, intrinsics, SceneLearningRates())
        ... forward, backward into exchange.backward_outputs() ...
        opt.step(exchange.reduce(), epoch_id)"""

    def __init__(self, parameters, background, env_map, pose_tangents, poses, intrinsics, rates=None):
        self.parameters, self.rates = parameters, rates or SceneLearningRates()
        self.background, self.env_map = background, env_map
        self.pose_tangents, self.poses, self.intrinsics = pose_tangents, poses, intrinsics
        r = self.rates
        groups = [{"params": [background], "lr": r.lr_background_color}]
        if env_map is not None:
            groups.append({"params": [env_map], "lr": r.lr_environment_map})
        for g in groups:
            for p in g["params"]:
                p.requires_grad_(True)
        self._adam = torch.optim.Adam(groups, lr=1.0)   # NeuralScene.cpp:76-107 (descriptors: in the peer kernel)
        structure = []
        if not r.fix_poses:
            structure.append({"params": [pose_tangents.requires_grad_(True)], "lr": r.lr_poses})
        if not r.fix_intrinsics:
            structure.append({"params": [intrinsics.requires_grad_(True)], "lr": r.lr_intrinsics})
        self._sgd = torch.optim.SGD(structure, lr=1e-10) if structure else None   # NeuralScene.cpp:204-240

    def step(self, reduced, epoch_id=1):
        """reduced: what PeerGradientExchange.reduce() returned for this step (normalised gradients). NeuralScene::OptimizerStep."""
        r = self.rates
        structure = epoch_id > r.lock_structure_params_epochs
        # the large tensors: Adam on the owned texels, SGD on the owned points, every new value to every replica
        self.parameters.step(reduced, lr_texture=r.lr_texture,
                             lr_points=(r.lr_points if (structure and not r.fix_points) else 0.0))
        self.background.grad = reduced["background"].to(self.background.dtype)
        if self.env_map is not None and reduced.get("env_map") is not None:
            self.env_map.grad = reduced["env_map"].reshape(self.env_map.shape)
        self._adam.step()
        self._adam.zero_grad(set_to_none=True)
        if structure and self._sgd is not None:
            if not r.fix_poses:
                self.pose_tangents.grad = reduced["pose"].reshape(self.pose_tangents.shape)
            if not r.fix_intrinsics:
                self.intrinsics.grad = reduced["intrinsics"].reshape(self.intrinsics.shape)
            self._sgd.step()
            self._sgd.zero_grad(set_to_none=True)
            if not r.fix_poses:
                with torch.no_grad():
                    apply_tangent_to_pose(self.pose_tangents.detach(), self.poses)   # and the tangents are zero again
